// Host-side packer: HostNint -> lane-stream device layout (see nint_layout.h).
#include "common.h"
#include "nint_layout.h"
#include "pair_unit.h"

namespace mfqb {

NintPacked pack_nint_device(const HostNint& t) {
    NintPacked p;
    NintDev& d = p.d;
    d.n = (int)t.n;
    d.k = (int)t.k;
    d.ng = (int)t.ng;
    d.bits = t.bits;
    d.gs = t.gs;
    d.sub_bits = t.sub_bits;
    d.per = nint_per(t.gs);
    d.sw = nint_stored_sub_width(t.bits, t.sub_bits);
    d.nrb = (d.n + 15) / 16;
    d.nchunks = (d.ng + kChunkGroups - 1) / kChunkGroups;
    const int half = d.per / 2, npairs = kChunkGroups * d.per;
    d.wc = pair_unit_words(d.bits, npairs);
    const int swords_per = pair_unit_words(d.sw, 16);
    d.swc = swords_per;
    d.rec_words = d.wc * 32 + d.swc * 8;
    p.items.assign((size_t)d.nrb * d.nchunks * d.rec_words, 0u);
    p.anchors.assign((size_t)d.nrb * 16, 0u);
    for (int64_t r = 0; r < t.n; ++r) p.anchors[r] = (uint32_t)t.ns[r] | ((uint32_t)t.nm[r] << 16);

    std::vector<uint32_t> lane_words(d.wc), quad_words(swords_per);
    for (int rb = 0; rb < d.nrb; ++rb) {
        for (int ch = 0; ch < d.nchunks; ++ch) {
            const size_t item = (size_t)rb * d.nchunks + ch;
            for (int lane = 0; lane < 32; ++lane) {
                const int q = lane >> 2, c = lane & 3;
                std::fill(lane_words.begin(), lane_words.end(), 0u);
                for (int g = 0; g < kChunkGroups; ++g) {
                    const int64_t grp = (int64_t)ch * kChunkGroups + g;
                    if (grp >= t.ng) break;
                    for (int r = 0; r < 2; ++r) {
                        const int64_t row = (int64_t)rb * 16 + q + 8 * r;
                        if (row >= t.n) continue;
                        const uint8_t* codes = &t.q[(row * t.ng + grp) * t.gs];
                        for (int j = 0; j < half; ++j) {
                            const int i0 = c * d.per + 2 * j;
                            const uint32_t lo = i0 < t.gs ? codes[i0] : 0u;
                            const uint32_t hi = i0 + 1 < t.gs ? codes[i0 + 1] : 0u;
                            if (lo | hi) pair_put(d.bits, lane_words.data(), (g * 2 + r) * half + j, lo, hi);
                        }
                    }
                }
                for (int w = 0; w < d.wc; ++w) p.items[item * d.rec_words + (size_t)w * 32 + lane] = lane_words[w];
            }
            for (int q = 0; q < 8; ++q) {
                std::fill(quad_words.begin(), quad_words.end(), 0u);
                const int64_t rows[2] = {(int64_t)rb * 16 + q, (int64_t)rb * 16 + q + 8};
                auto sub = [&](const std::vector<uint8_t>& a, int r, int g) -> uint32_t {
                    const int64_t grp = (int64_t)ch * kChunkGroups + g;
                    return (rows[r] < t.n && grp < t.ng) ? a[rows[r] * t.ng + grp] : 0u;
                };
                for (int g = 0; g < 8; ++g) pair_put(d.sw, quad_words.data(), g, sub(t.ss, 0, g), sub(t.ss, 1, g));
                for (int r = 0; r < 2; ++r)
                    for (int j = 0; j < 4; ++j)
                        pair_put(d.sw, quad_words.data(), 8 + 4 * r + j, sub(t.sm, r, 2 * j), sub(t.sm, r, 2 * j + 1));
                for (int w = 0; w < swords_per; ++w) p.items[item * d.rec_words + (size_t)d.wc * 32 + (size_t)w * 8 + q] = quad_words[w];
            }
        }
    }
    return p;
}

// Reads every field back through the kernels' accessors; returns the mismatch count.
uint64_t selfcheck_nint_layout(const HostNint& t) {
    NintPacked p = pack_nint_device(t);
    const NintDev& d = p.d;
    const int half = d.per / 2, swords_per = pair_unit_words(d.sw, 16);
    uint64_t bad = 0;
    std::vector<uint32_t> lane_words(d.wc), quad_words(swords_per);
    for (int64_t row = 0; row < t.n; ++row) {
        const int rb = (int)(row / 16), q = (int)(row % 8), r = (int)((row % 16) / 8);
        if (p.anchors[row] != ((uint32_t)t.ns[row] | ((uint32_t)t.nm[row] << 16))) ++bad;
        for (int64_t grp = 0; grp < t.ng; ++grp) {
            const int ch = (int)(grp / kChunkGroups), g = (int)(grp % kChunkGroups);
            const size_t item = (size_t)rb * d.nchunks + ch;
            for (int w = 0; w < swords_per; ++w) quad_words[w] = p.items[item * d.rec_words + (size_t)d.wc * 32 + (size_t)w * 8 + q];
            const uint32_t sp = pair_get(d.sw, quad_words.data(), g);
            const uint32_t ssv = r ? (sp >> 16) : (sp & 0xFFFF);
            const uint32_t mp = pair_get(d.sw, quad_words.data(), 8 + 4 * r + g / 2);
            const uint32_t smv = (g & 1) ? (mp >> 16) : (mp & 0xFFFF);
            if (ssv != t.ss[row * t.ng + grp]) ++bad;
            if (smv != t.sm[row * t.ng + grp]) ++bad;
            for (int c = 0; c < 4; ++c) {
                const int lane = 4 * q + c;
                for (int w = 0; w < d.wc; ++w) lane_words[w] = p.items[item * d.rec_words + (size_t)w * 32 + lane];
                for (int j = 0; j < half; ++j) {
                    const uint32_t pr = pair_get(d.bits, lane_words.data(), (g * 2 + r) * half + j);
                    const int i0 = c * d.per + 2 * j;
                    const uint8_t* codes = &t.q[(row * t.ng + grp) * t.gs];
                    if (i0 < t.gs && (pr & 0xFFFF) != codes[i0]) ++bad;
                    if (i0 + 1 < t.gs && (pr >> 16) != codes[i0 + 1]) ++bad;
                }
            }
        }
    }
    return bad;
}

}  // namespace mfqb
