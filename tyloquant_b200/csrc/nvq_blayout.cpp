// Host-side packer: HostNvq -> byte-lane NVQ device layout (see nvq_blayout.h), and its read-back check.
#include "nvq_blayout.h"

#include "common.h"

namespace mfqb {

// Weight k = 4*vec + e takes bit (k % 8) of its block's 7-bit mask, the eighth weight of a block
// the parity of the seven (mfq/quantize/nvq_quant.py:591-611).
uint32_t nvq_sign_nibble(const HostNvq& t, int64_t row, int64_t vec) {
    const int64_t block = vec / 2;
    if (block >= t.nsign) return 0u;
    const uint32_t m = t.signs[row * t.nsign + block] & 0x7Fu;
    const uint32_t full = m | ((uint32_t)(__builtin_popcount(m) & 1) << 7);
    return (full >> ((vec & 1) * 4)) & 0xFu;
}

static void put_bits(std::vector<uint32_t>& w, int pos, int nbits, uint32_t v) {
    const int wi = pos >> 5, sh = pos & 31;
    w[wi] |= v << sh;
    if (sh + nbits > 32) w[wi + 1] |= v >> (32 - sh);
}
static uint32_t get_bits(const uint32_t* w, int pos, int nbits) {
    const int wi = pos >> 5, sh = pos & 31;
    uint64_t v = w[wi];
    if (sh + nbits > 32) v |= (uint64_t)w[wi + 1] << 32;
    return (uint32_t)(v >> sh) & ((1u << nbits) - 1u);
}

NvqPackedB pack_nvq_bytes(const HostNvq& t) {
    if (t.gs != 24 || t.vec != 4) fail(MFQB_ERR_UNSUPPORTED, "NVQ runtime layout needs 24-weight groups of 4-wide vectors");
    NvqPackedB p;
    NintDevB& d = p.d;
    d.n = (int)t.n;
    d.k = (int)t.k;
    d.ng = (int)t.ng;
    d.bits = 0;
    d.gs = 24;
    d.sub_bits = t.sub_bits;
    d.t8 = 3;
    d.nrb = (d.n + 15) / 16;
    d.nchunks = (d.ng + kChunkGroupsB - 1) / kChunkGroupsB;
    const int fb = t.index_bits + 4;
    d.wc = (24 * fb + 31) / 32;
    d.rec_words = (d.wc + 1) * 32;
    d.index_bits = t.index_bits;
    d.entries = t.entries;
    d.banks = t.banks;
    d.jsc = t.jsc ? 1 : 0;
    d.bankmap = 0;
    for (int s = 0; s < 16; ++s) {
        d.lut[s] = t.jsc ? f16_to_f32(t.lut_h[s]) : (float)s;
        d.bankmap |= (uint32_t)(t.jsc ? t.bank_for_state[s] : 0) << (2 * s);
    }
    // signed table: entry (bank, index, nibble) = the four int8 codes, negated where the nibble says so
    p.table.resize((size_t)t.banks * t.entries * 16);
    for (size_t e = 0; e < (size_t)t.banks * t.entries; ++e)
        for (uint32_t sg = 0; sg < 16; ++sg) {
            uint32_t v = 0;
            for (int j = 0; j < 4; ++j) {
                const int code = t.codebooks[e * 4 + j];
                v |= (uint32_t)(uint8_t)(int8_t)(((sg >> j) & 1u) ? -code : code) << (8 * j);
            }
            p.table[e * 16 + sg] = v;
        }
    d.table_words = (int)p.table.size();
    p.items.assign((size_t)d.nrb * d.nchunks * d.rec_words, 0u);
    p.anchors.assign((size_t)d.nrb * 16, 0u);
    for (int64_t r = 0; r < t.n; ++r) p.anchors[r] = t.anchors[r];

    auto state_of = [&](int64_t row, int64_t grp) -> uint32_t { return (row < t.n && grp < t.ng) ? t.sub[row * t.ng + grp] : 0u; };
    std::vector<uint32_t> lane_words(d.wc + 1);
    for (int rb = 0; rb < d.nrb; ++rb)
        for (int ch = 0; ch < d.nchunks; ++ch) {
            uint32_t* rec = &p.items[((size_t)rb * d.nchunks + ch) * d.rec_words];
            for (int lane = 0; lane < 32; ++lane) {
                const int q = lane >> 2, c = lane & 3;
                std::fill(lane_words.begin(), lane_words.end(), 0u);
                uint32_t sword = 0;
                for (int reg = 0; reg < 24; ++reg) {
                    const NintRegCoord rc = nint_reg_coord(3, lane, reg);
                    const int64_t row = (int64_t)rb * 16 + rc.row, grp = (int64_t)ch * kChunkGroupsB + rc.group;
                    const int64_t vec = grp * 6 + rc.slot / 4;
                    if (row >= t.n || grp >= t.ng || vec >= t.nvec) continue;
                    const uint32_t field = nvq_sign_nibble(t, row, vec) | ((uint32_t)t.idx[row * t.nvec + vec] << 4);
                    put_bits(lane_words, reg * fb, fb, field);
                    if ((reg % 12) < 4) {   // step t = 0 of family f: record the bank of pair f*4 + a
                        const int i = (reg / 12) * 4 + (reg & 3);
                        const uint32_t bank = (d.bankmap >> (2 * state_of(row, grp))) & 3u;
                        sword |= bank << (8 * (i >> 1) + 4 + 2 * (i & 1));
                    }
                }
                for (int i = 0; i < 4; ++i)
                    sword |= (state_of((int64_t)rb * 16 + q + 8 * (i >> 1), (int64_t)ch * kChunkGroupsB + 2 * c + (i & 1)) & 15u) << (8 * i);
                for (int w = 0; w < d.wc; ++w) rec[w * 32 + lane] = lane_words[w];
                rec[d.wc * 32 + lane] = sword;
            }
        }
    return p;
}

uint64_t selfcheck_nvq_bytes(const HostNvq& t) {
    NvqPackedB p = pack_nvq_bytes(t);
    const NintDevB& d = p.d;
    const int fb = d.index_bits + 4;
    uint64_t bad = 0, seen = 0;
    std::vector<uint32_t> lane_words(d.wc + 1, 0u);
    for (int64_t row = 0; row < t.n; ++row)
        if ((p.anchors[row] & 0xFFFFu) != t.anchors[row] || (p.anchors[row] >> 16) != 0) ++bad;
    for (int rb = 0; rb < d.nrb; ++rb)
        for (int ch = 0; ch < d.nchunks; ++ch) {
            const uint32_t* rec = &p.items[((size_t)rb * d.nchunks + ch) * d.rec_words];
            for (int lane = 0; lane < 32; ++lane) {
                const int q = lane >> 2, c = lane & 3;
                for (int w = 0; w < d.wc; ++w) lane_words[w] = rec[w * 32 + lane];
                const uint32_t sword = rec[d.wc * 32 + lane];
                for (int reg = 0; reg < 24; ++reg) {
                    const NintRegCoord rc = nint_reg_coord(3, lane, reg);
                    const int64_t row = (int64_t)rb * 16 + rc.row, grp = (int64_t)ch * kChunkGroupsB + rc.group;
                    const int64_t vec = grp * 6 + rc.slot / 4;
                    if (row >= t.n || grp >= t.ng || vec >= t.nvec) continue;
                    ++seen;
                    const uint32_t f = get_bits(lane_words.data(), reg * fb, fb);
                    if ((f >> 4) != t.idx[row * t.nvec + vec] || (f & 15u) != nvq_sign_nibble(t, row, vec)) ++bad;
                    const int i = (reg / 12) * 4 + (reg & 3);
                    const uint32_t bank = (sword >> (8 * (i >> 1) + 4 + 2 * (i & 1))) & 3u;
                    if (bank != ((d.bankmap >> (2 * t.sub[row * t.ng + grp])) & 3u)) ++bad;
                    // the table entry decodes to the signed codebook vector
                    const uint32_t v = p.table[((size_t)bank * d.entries + (f >> 4)) * 16 + (f & 15u)];
                    for (int j = 0; j < 4; ++j) {
                        const int code = t.codebooks[((size_t)bank * t.entries + (f >> 4)) * 4 + j];
                        if ((int)(int8_t)(v >> (8 * j)) != (((f >> j) & 1u) ? -code : code)) ++bad;
                    }
                }
                for (int i = 0; i < 4; ++i) {
                    const int64_t row = (int64_t)rb * 16 + q + 8 * (i >> 1), grp = (int64_t)ch * kChunkGroupsB + 2 * c + (i & 1);
                    const uint32_t want = (row < t.n && grp < t.ng) ? t.sub[row * t.ng + grp] : 0u;
                    if (((sword >> (8 * i)) & 15u) != want) ++bad;
                }
            }
        }
    if (seen != (uint64_t)t.n * t.nvec) ++bad;   // every vector of the tensor is stored exactly once
    return bad;
}

}  // namespace mfqb
