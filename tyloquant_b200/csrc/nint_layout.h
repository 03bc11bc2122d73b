// Device layout of NINT weights ("lane streams") and its host-side packer.
//
// Rows are taken 16 at a time (a row-block: the M of one mma.m16n8k16), groups 8 at a
// time (a chunk).  For one (row-block, chunk) every lane of a warp owns a private stream of
// code pairs, already in tensor-core fragment order:
//
//   lane = 4*q + c     q = 0..7  -> rows  q (lo) and q+8 (hi) of the row-block
//                      c = 0..3  -> codes [c*PER, c*PER+PER) of each (padded) group
//   pair t = (g*2 + r)*(PER/2) + j   g = group in chunk, r = lo/hi row, j = pair in lane
//          = codes (c*PER + 2j, c*PER + 2j + 1) of row r, group g   (0 beyond the group)
//
// PER = groupsize/4 rounded up to an even number.  The pairs of a lane are packed with
// PairUnit<bits>; word w of the 32 lanes is stored contiguously ([w][lane]) so one warp load
// instruction reads 128 consecutive bytes.
//
// Scales: per (row-block, chunk, quad q) 16 pairs of width SW (the stored sub-scale width,
// >= the tensor's sub_bits), packed with PairUnit<SW>:
//   pair g      (g = 0..7)        = (sub_scale[lo][g], sub_scale[hi][g])
//   pair 8+4r+j (r = 0..1, j<4)   = (sub_min[r][2j],   sub_min[r][2j+1])
// stored as [word][quad].
//
// One (row-block, chunk) item is one contiguous record of rec_words 32-bit words,
//   [wc x 32 code words][swc x 8 scale words],   a multiple of 32 bytes,
// records ordered [row-block][chunk]; a kernel moves a record with a few 16-byte async copies.
// Anchors: one 32-bit word per row: f16 neuron_scale | f16 neuron_min << 16.
#pragma once
#include <cstdint>
#include <vector>

namespace mfqb {

struct NintDev {
    const uint32_t* items;    // [nrb * nchunks][rec_words]
    const uint32_t* anchors;
    int n, k, ng;        // rows, columns, groups per row
    int nrb, nchunks;    // row-blocks of 16, chunks of 8 groups
    int bits, gs, sub_bits;
    int per;             // codes per lane per row per group (even)
    int sw;              // stored scale width
    int wc;              // code words per lane per chunk
    int swc;             // scale words per quad per chunk
    int rec_words;       // wc * 32 + swc * 8
};

constexpr int kChunkGroups = 8;

inline int nint_per(int gs) { return ((gs + 3) / 4 + 1) & ~1; }

// Stored scale width for a tensor: the narrowest width the kernels are built for.
inline int nint_stored_sub_width(int bits, int sub_bits) {
    const int canon = bits <= 3 ? 5 : (bits == 4 ? 6 : 7);
    return sub_bits <= canon ? canon : 8;
}

struct HostNint;
struct NintPacked {
    std::vector<uint32_t> items, anchors;
    NintDev d{};   // pointers unset; geometry filled
};
NintPacked pack_nint_device(const HostNint& t);
uint64_t selfcheck_nint_layout(const HostNint& t);

}  // namespace mfqb
