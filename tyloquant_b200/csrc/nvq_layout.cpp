// Host-side packer: HostNvq -> NVQ device layout (see nvq_layout.h), and its read-back check.
#include "common.h"
#include "nvq_layout.h"
#include "pair_unit.h"

namespace mfqb {

static uint16_t bf16_of_small_int(int v) {   // exact for |v| <= 256
    float f = (float)v;
    uint32_t u;
    memcpy(&u, &f, 4);
    return (uint16_t)(u >> 16);
}

// Four sign bits of vector `vec` (0..) of a row: weight k = 4*vec + e takes bit (k % 8) of its
// block's 7-bit mask, the eighth weight of a block the parity of the seven.
static uint32_t sign_nibble(const HostNvq& t, int64_t row, int64_t vec) {
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

NvqPacked pack_nvq_device(const HostNvq& t) {
    NvqPacked p;
    NvqDev& d = p.d;
    d.n = (int)t.n;
    d.k = (int)t.k;
    d.ng = (int)t.ng;
    d.nrb = (d.n + 15) / 16;
    d.nchunks = (d.ng + kNvqChunkGroups - 1) / kNvqChunkGroups;
    d.index_bits = t.index_bits;
    d.fb = t.index_bits + 4;
    d.wc = (24 * d.fb + 31) / 32;
    d.rec_words = d.wc * 32 + 16;
    d.entries = t.entries;
    d.banks = t.banks;
    d.jsc = t.jsc ? 1 : 0;
    d.bankmap = 0;
    for (int s = 0; s < 16; ++s) {
        d.lut[s] = t.jsc ? f16_to_f32(t.lut_h[s]) : (float)s;
        d.bankmap |= (uint32_t)(t.jsc ? t.bank_for_state[s] : 0) << (2 * s);
    }
    p.cb.resize((size_t)t.banks * t.entries * 2);
    for (size_t e = 0; e < (size_t)t.banks * t.entries; ++e) {
        const int8_t* m = &t.codebooks[e * 4];
        p.cb[2 * e] = (uint32_t)bf16_of_small_int(m[0]) | ((uint32_t)bf16_of_small_int(m[1]) << 16);
        p.cb[2 * e + 1] = (uint32_t)bf16_of_small_int(m[2]) | ((uint32_t)bf16_of_small_int(m[3]) << 16);
    }
    p.items.assign((size_t)d.nrb * d.nchunks * d.rec_words, 0u);
    p.anchors.assign((size_t)d.nrb * 16, 0u);
    for (int64_t r = 0; r < t.n; ++r) p.anchors[r] = t.anchors[r];

    std::vector<uint32_t> lane_words(d.wc + 1), quad_words(2);
    for (int rb = 0; rb < d.nrb; ++rb)
        for (int ch = 0; ch < d.nchunks; ++ch) {
            uint32_t* rec = &p.items[((size_t)rb * d.nchunks + ch) * d.rec_words];
            for (int lane = 0; lane < 32; ++lane) {
                const int q = lane >> 2, c = lane & 3;
                std::fill(lane_words.begin(), lane_words.end(), 0u);
                for (int pr = 0; pr < 4; ++pr)
                    for (int r = 0; r < 2; ++r)
                        for (int u = 0; u < 3; ++u) {
                            int g, v;
                            nvq_slot(pr, u, c, g, v);
                            const int64_t row = (int64_t)rb * 16 + q + 8 * r;
                            const int64_t vec = ((int64_t)ch * kNvqChunkGroups + g) * 6 + v;
                            if (row >= t.n || vec >= t.nvec) continue;
                            const uint32_t field = (uint32_t)t.idx[row * t.nvec + vec] | (sign_nibble(t, row, vec) << d.index_bits);
                            put_bits(lane_words, ((pr * 2 + r) * 3 + u) * d.fb, d.fb, field);
                        }
                for (int w = 0; w < d.wc; ++w) rec[w * 32 + lane] = lane_words[w];
            }
            for (int q = 0; q < 8; ++q) {
                quad_words[0] = quad_words[1] = 0u;
                for (int g = 0; g < 8; ++g) {
                    const int64_t grp = (int64_t)ch * kNvqChunkGroups + g;
                    uint32_t lo = 0, hi = 0;
                    if (grp < t.ng) {
                        const int64_t r0 = (int64_t)rb * 16 + q, r1 = r0 + 8;
                        if (r0 < t.n) lo = t.sub[r0 * t.ng + grp];
                        if (r1 < t.n) hi = t.sub[r1 * t.ng + grp];
                    }
                    pair_put(4, quad_words.data(), g, lo, hi);
                }
                rec[d.wc * 32 + q] = quad_words[0];
                rec[d.wc * 32 + 8 + q] = quad_words[1];
            }
        }
    return p;
}

uint64_t selfcheck_nvq_layout(const HostNvq& t) {
    NvqPacked p = pack_nvq_device(t);
    const NvqDev& d = p.d;
    uint64_t bad = 0;
    std::vector<uint32_t> lane_words(d.wc + 1, 0u);
    for (int64_t row = 0; row < t.n; ++row) {
        const int rb = (int)(row / 16), q = (int)(row % 8), r = (int)((row % 16) / 8);
        if ((p.anchors[row] & 0xFFFFu) != t.anchors[row]) ++bad;
        for (int64_t grp = 0; grp < t.ng; ++grp) {
            const int ch = (int)(grp / kNvqChunkGroups), g = (int)(grp % kNvqChunkGroups);
            const uint32_t* rec = &p.items[((size_t)rb * d.nchunks + ch) * d.rec_words];
            const uint32_t sw[2] = {rec[d.wc * 32 + q], rec[d.wc * 32 + 8 + q]};
            const uint32_t sp = pair_get(4, sw, g);
            if ((r ? (sp >> 16) : (sp & 0xFFFFu)) != t.sub[row * t.ng + grp]) ++bad;
            for (int v = 0; v < 6; ++v) {
                const int64_t vec = grp * 6 + v;
                if (vec >= t.nvec) break;
                // invert nvq_slot
                const int pr = g / 2, h = g % 2;
                int c, u;
                if (h == 0) { if (v < 4) { c = v; u = 0; } else { c = v - 4; u = 1; } }
                else { if (v < 2) { c = v + 2; u = 1; } else { c = v - 2; u = 2; } }
                for (int w = 0; w < d.wc; ++w) lane_words[w] = rec[w * 32 + 4 * q + c];
                const uint32_t f = get_bits(lane_words.data(), ((pr * 2 + r) * 3 + u) * d.fb, d.fb);
                if ((f & ((1u << d.index_bits) - 1u)) != t.idx[row * t.nvec + vec]) ++bad;
                if ((f >> d.index_bits) != sign_nibble(t, row, vec)) ++bad;
            }
        }
    }
    return bad;
}

}  // namespace mfqb
