// Byte-lane device layout of NINT weights: codes stored so that a shift + mask yields a
// register of four 8-bit codes -- an A operand of the int8 tensor-core instruction
// mma.m16n8k32 -- and its host-side packer.
//
// Rows are taken 16 at a time (a row-block: the M of the mma), groups 8 at a time (a chunk),
// slots of a group 8 at a time (an octet; T = ceil(groupsize / 8) octets per group).  For one
// (row-block, chunk) *item* the warp issues the mma steps (f, t), f = 0..1, t = 0..T-1; the
// 32 k-slots of step (f, t) are octet t of the four groups 4f .. 4f+3:
//
//   k = 8*o + i      o = 0..3 -> group 4f + o,   i = 0..7 -> slot 8t + i of that group.
//
// With the fragment layout of the instruction, lane = 4*q + c holds in step (f, t)
//
//   a0: row q,   group 4f +     (c>>1), slots 8t + 4(c&1) + {0,1,2,3}      (one byte each)
//   a1: row q+8, same group and slots
//   a2: row q,   group 4f + 2 + (c>>1), same slots
//   a3: row q+8, same
//
// so every lane owns a private stream of 8T registers, register ((f*T + t)*4 + a), packed with
// ByteUnit<bits> (no wasted bits for any code width).  Word w of the 32 lanes is stored
// contiguously ([w][lane]): one warp load instruction reads 128 consecutive bytes.  Codes of
// slots past the group size (a group size that is not a multiple of 8 is padded), of groups past
// the row's last group and of rows past the last row are zero.
//
// Scales: two words per lane, one byte per field.  The accumulator fragment gives lane (q, c)
// the sums of rows q, q+8 for the chunk's groups 2c, 2c+1, so it stores exactly those:
//
//   word 0: sub_scale[q][2c], sub_scale[q][2c+1], sub_scale[q+8][2c], sub_scale[q+8][2c+1]
//   word 1: sub_min, same order.
//
// One item is one contiguous record of rec_words = (wc + 2) * 32 words,
//   [wc x 32 code words][2 x 32 scale words],   a multiple of 128 bytes,
// records ordered [row-block][chunk]; a kernel moves a record with a few 16-byte async copies.
// Anchors: one 32-bit word per row: f16 neuron_scale | f16 neuron_min << 16.
#pragma once
#include <cstdint>
#include <vector>

namespace mfqb {

struct NintDevB {
    const uint32_t* items;    // [nrb * nchunks][rec_words]
    const uint32_t* anchors;  // [nrb * 16]
    int n, k, ng;        // rows, columns, groups per row
    int nrb, nchunks;    // row-blocks of 16, chunks of 8 groups
    int bits, gs, sub_bits;
    int t8;              // octets per group
    int wc;              // code words per lane per item
    int rec_words;       // (wc + scale words) * 32
    // Lattice (NVQ) weights only: the signed codebook table and the joint scale/codebook states.
    const uint32_t* table;   // [banks][entries][16 sign patterns] of four int8 each
    int table_words;
    int index_bits, entries, banks, jsc;
    float lut[16];           // scale of each state (JSC); plain NVQ uses the sub-scale itself
    uint32_t bankmap;        // 2 bits per state: codebook bank
};

constexpr int kChunkGroupsB = 8;

// Register index of a lane's stream and the coordinates it covers.
struct NintRegCoord {
    int row;     // 0..15 inside the row-block
    int group;   // 0..7 inside the chunk
    int slot;    // first of four consecutive slots
};
inline NintRegCoord nint_reg_coord(int t8, int lane, int reg) {
    const int q = lane >> 2, c = lane & 3, a = reg & 3, ft = reg >> 2, f = ft / t8, t = ft % t8;
    return NintRegCoord{q + 8 * (a & 1), 4 * f + 2 * (a >> 1) + (c >> 1), 8 * t + 4 * (c & 1)};
}

// The (code width, octets per group) pairs of the runtime catalog.
constexpr bool nint_bl_in_catalog(int bits, int t8) {
    return bits == 2 ? t8 == 2
         : bits == 3 ? t8 == 3
         : bits == 4 ? (t8 == 2 || t8 == 3 || t8 == 4 || t8 == 6)
         : bits == 6 ? (t8 == 3 || t8 == 4 || t8 == 5 || t8 == 6 || t8 == 8)
         : (bits == 5 || bits == 8) ? (t8 == 2 || t8 == 3 || t8 == 4 || t8 == 6 || t8 == 8)
         : false;
}

struct HostNint;
struct NintPackedB {
    std::vector<uint32_t> items, anchors;
    NintDevB d{};   // pointers unset; geometry filled
};
NintPackedB pack_nint_bytes(const HostNint& t);
uint64_t selfcheck_nint_bytes(const HostNint& t);

}  // namespace mfqb
