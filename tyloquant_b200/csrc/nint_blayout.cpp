// Host-side packer: HostNint -> byte-lane device layout (see nint_blayout.h).
#include "nint_blayout.h"

#include "common.h"
#include "lane_unit.h"

namespace mfqb {

NintPackedB pack_nint_bytes(const HostNint& t) {
    NintPackedB p;
    NintDevB& d = p.d;
    d.n = (int)t.n;
    d.k = (int)t.k;
    d.ng = (int)t.ng;
    d.bits = t.bits;
    d.gs = t.gs;
    d.sub_bits = t.sub_bits;
    d.t8 = (t.gs + 7) / 8;
    d.nrb = (d.n + 15) / 16;
    d.nchunks = (d.ng + kChunkGroupsB - 1) / kChunkGroupsB;
    const int nregs = 8 * d.t8;
    d.wc = byte_unit_words(d.bits, nregs);
    d.rec_words = (d.wc + 2) * 32;
    p.items.assign((size_t)d.nrb * d.nchunks * d.rec_words, 0u);
    p.anchors.assign((size_t)d.nrb * 16, 0u);
    for (int64_t r = 0; r < t.n; ++r) p.anchors[r] = (uint32_t)t.ns[r] | ((uint32_t)t.nm[r] << 16);

    std::vector<uint32_t> lane_words(d.wc);
    for (int rb = 0; rb < d.nrb; ++rb) {
        for (int ch = 0; ch < d.nchunks; ++ch) {
            uint32_t* rec = p.items.data() + ((size_t)rb * d.nchunks + ch) * d.rec_words;
            for (int lane = 0; lane < 32; ++lane) {
                std::fill(lane_words.begin(), lane_words.end(), 0u);
                for (int reg = 0; reg < nregs; ++reg) {
                    const NintRegCoord rc = nint_reg_coord(d.t8, lane, reg);
                    const int64_t row = (int64_t)rb * 16 + rc.row, grp = (int64_t)ch * kChunkGroupsB + rc.group;
                    if (row >= t.n || grp >= t.ng) continue;
                    const uint8_t* codes = &t.q[(row * t.ng + grp) * t.gs];
                    uint32_t v = 0;
                    for (int i = 0; i < 4; ++i)
                        if (rc.slot + i < t.gs) v |= (uint32_t)codes[rc.slot + i] << (8 * i);
                    if (v) byte_unit_put(d.bits, lane_words.data(), reg, v);
                }
                for (int w = 0; w < d.wc; ++w) rec[(size_t)w * 32 + lane] = lane_words[w];
                const int q = lane >> 2, c = lane & 3;
                uint32_t s0 = 0, s1 = 0;
                for (int i = 0; i < 4; ++i) {
                    const int64_t row = (int64_t)rb * 16 + q + 8 * (i >> 1), grp = (int64_t)ch * kChunkGroupsB + 2 * c + (i & 1);
                    if (row >= t.n || grp >= t.ng) continue;
                    s0 |= (uint32_t)t.ss[row * t.ng + grp] << (8 * i);
                    s1 |= (uint32_t)t.sm[row * t.ng + grp] << (8 * i);
                }
                rec[(size_t)d.wc * 32 + lane] = s0;
                rec[(size_t)(d.wc + 1) * 32 + lane] = s1;
            }
        }
    }
    return p;
}

// Reads every field back through the kernels' accessors; returns the mismatch count.
uint64_t selfcheck_nint_bytes(const HostNint& t) {
    NintPackedB p = pack_nint_bytes(t);
    const NintDevB& d = p.d;
    uint64_t bad = 0, seen = 0;
    std::vector<uint32_t> lane_words(d.wc);
    for (int64_t row = 0; row < t.n; ++row)
        if (p.anchors[row] != ((uint32_t)t.ns[row] | ((uint32_t)t.nm[row] << 16))) ++bad;
    for (int rb = 0; rb < d.nrb; ++rb) {
        for (int ch = 0; ch < d.nchunks; ++ch) {
            const uint32_t* rec = p.items.data() + ((size_t)rb * d.nchunks + ch) * d.rec_words;
            for (int lane = 0; lane < 32; ++lane) {
                for (int w = 0; w < d.wc; ++w) lane_words[w] = rec[(size_t)w * 32 + lane];
                for (int reg = 0; reg < 8 * d.t8; ++reg) {
                    const NintRegCoord rc = nint_reg_coord(d.t8, lane, reg);
                    const int64_t row = (int64_t)rb * 16 + rc.row, grp = (int64_t)ch * kChunkGroupsB + rc.group;
                    const uint32_t v = byte_unit_get(d.bits, lane_words.data(), reg);
                    for (int i = 0; i < 4; ++i) {
                        const uint32_t got = (v >> (8 * i)) & 0xFF;
                        const bool live = row < t.n && grp < t.ng && rc.slot + i < t.gs;
                        const uint32_t want = live ? t.q[(row * t.ng + grp) * t.gs + rc.slot + i] : 0u;
                        if (got != want) ++bad;
                        if (live) ++seen;
                    }
                }
                const int q = lane >> 2, c = lane & 3;
                for (int i = 0; i < 4; ++i) {
                    const int64_t row = (int64_t)rb * 16 + q + 8 * (i >> 1), grp = (int64_t)ch * kChunkGroupsB + 2 * c + (i & 1);
                    const bool live = row < t.n && grp < t.ng;
                    const uint32_t ss = (rec[(size_t)d.wc * 32 + lane] >> (8 * i)) & 0xFF, sm = (rec[(size_t)(d.wc + 1) * 32 + lane] >> (8 * i)) & 0xFF;
                    if (ss != (live ? t.ss[row * t.ng + grp] : 0u)) ++bad;
                    if (sm != (live ? t.sm[row * t.ng + grp] : 0u)) ++bad;
                }
            }
        }
    }
    if (seen != (uint64_t)t.n * t.ng * t.gs) ++bad;   // every code of the tensor is stored exactly once
    return bad;
}

}  // namespace mfqb
