// Byte-lane device layout of NVQ3 (D4 lattice) weights and its host-side packer.
//
// A lattice vector is four weights: exactly one A register of the int8 tensor-core instruction.
// The item / step / lane structure is that of the NINT byte-lane layout with T = 3 octets per
// 24-weight group (nint_blayout.h): register ((f*3 + t)*4 + a) of lane 4q + c is vector
// 2t + (c&1) of group 4f + 2(a>>1) + (c>>1) of row q + 8(a&1).  Instead of codes the lane stream
// holds one field per register,
//
//   field = sign nibble | index << 4            (FB = index_bits + 4 bits),
//
// 24 fields as a dense LSB-first bitstream of WC = ceil(24*FB/32) words, stored [word][lane].
// The sign nibble holds the four sign bits of the vector (the format stores seven sign bits per
// eight weights and derives the eighth as their parity; the packer materialises it).  A kernel
// turns a field into its register with one shared-memory load from the *signed table*
//
//   table[bank][index][nibble] = the four int8 codebook entries with the signs applied,
//
// built at load time (16 KB for a 256-entry codebook).
//
// Scales: one word per lane, one byte per (row, group) the lane's accumulators own, in the NINT
// order (row q, group 2c), (q, 2c+1), (q+8, 2c), (q+8, 2c+1): low nibble = the integer sub-scale
// or the joint scale/codebook state of NVQ-JSC.  The high nibbles together carry, two bits each,
// the codebook bank of the eight (row, group) pairs the lane's *registers* belong to, pair
// f*4 + a at bits 8*(i>>1) + 4 + 2*(i&1), i = f*4 + a.
// One item is one record [WC x 32][1 x 32] words; anchors: f16 anchor in the low half of a word
// per row (the high half, the NINT neuron minimum, is zero).
#pragma once
#include "nint_blayout.h"

namespace mfqb {

struct HostNvq;
struct NvqPackedB {
    std::vector<uint32_t> items, anchors, table;
    NintDevB d{};   // pointers unset; geometry filled
};
NvqPackedB pack_nvq_bytes(const HostNvq& t);
uint64_t selfcheck_nvq_bytes(const HostNvq& t);

// Four sign bits of vector `vec` of a row (bit e set: weight 4*vec + e is negative).
uint32_t nvq_sign_nibble(const HostNvq& t, int64_t row, int64_t vec);

}  // namespace mfqb
