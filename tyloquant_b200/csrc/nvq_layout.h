// Device layout of NVQ3 (D4 lattice) weights and its host-side packer.
//
// As for NINT, rows are taken 16 at a time (a row-block) and groups of 24 weights 8 at a time
// (a chunk).  A group is six 4-wide lattice vectors; two neighbouring groups (a group pair p)
// are twelve vectors = three mma.m16n8k16 steps in which every lane of a quad supplies one
// whole vector (its two bf16x2 operand registers) per row:
//
//   lane = 4*q + c, rows q (lo) and q+8 (hi);   step u of pair p, lane c supplies
//     u = 0: group 2p,   vector c
//     u = 1: group 2p,   vector 4+c   (c < 2)      group 2p+1, vector c-2   (c >= 2)
//     u = 2: group 2p+1, vector 2+c
//
// Per lane and chunk that is 24 fields, t = (p*2 + r)*3 + u, each FB = index_bits + 4 wide:
// the codebook index and the four sign bits of the vector (the format stores seven sign bits per
// eight weights and derives the eighth as their parity; the packer materialises it, which costs
// one bit per eight weights and saves the kernels a popcount per block).  The fields form a dense
// LSB-first bitstream of WC = ceil(24*FB/32) words per lane, stored [word][lane].
//
// Scales: per quad 8 pairs of 4 bits, pair g = (sub[lo][g], sub[hi][g]) (the integer sub-scale,
// or the joint scale/codebook state of NVQ-JSC), PairUnit<4> -> 2 words, stored [word][quad].
// One (row-block, chunk) item is one contiguous record [WC*32][2*8] words; records are ordered
// [row-block][chunk].  Anchors: one word per row holding the f16 anchor in its low half.
// Tables: the codebook banks as bf16x2 pairs (entry e of bank b at cb[b*entries + e] =
// {(m0,m1),(m2,m3)}), the 16 float scales of NVQ-JSC and its state->bank map (2 bits per state).
#pragma once
#include <cstdint>
#include <vector>

namespace mfqb {

struct alignas(8) NvqPair { uint32_t x, y; };

struct NvqDev {
    const uint32_t* items;
    const uint32_t* anchors;
    const NvqPair* cb;     // {(m0,m1),(m2,m3)} as two bf16x2 words
    int n, k, ng, nrb, nchunks;
    int index_bits, fb, wc, rec_words;
    int entries, banks, jsc;
    uint32_t bankmap;      // 2 bits per state
    float lut[16];         // JSC scale per state (float value of the f16 table)
};

constexpr int kNvqGroup = 24;
constexpr int kNvqChunkGroups = 8;

// (group in chunk, vector in group) of step u of pair p for lane-in-quad c
inline
#if defined(__CUDACC__)
__host__ __device__
#endif
void nvq_slot(int p, int u, int c, int& g, int& v) {
    if (u == 0) { g = 2 * p; v = c; }
    else if (u == 2) { g = 2 * p + 1; v = 2 + c; }
    else if (c < 2) { g = 2 * p; v = 4 + c; }
    else { g = 2 * p + 1; v = c - 2; }
}

struct HostNvq;
struct NvqPacked {
    std::vector<uint32_t> items, anchors;
    std::vector<uint32_t> cb;   // 2 words per entry
    NvqDev d{};
};
NvqPacked pack_nvq_device(const HostNvq& t);

}  // namespace mfqb
