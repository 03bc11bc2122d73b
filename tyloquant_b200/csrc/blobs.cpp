// Host-side decoding of tensor blobs into plain arrays, and packed-domain slicing.
//   NINT  : mfq/formats/io.py:191-248, cpp_runtime/mfq_decode.cpp:1546-1589
//   NVQ   : mfq/formats/nvq.py:586-820, cpp_runtime/mfq_decode.cpp:3756-4013
//   NINTM : mfq/formats/io.py:304-446, cpp_runtime/mfq_decode.cpp:2367-2478
//   slices: cpp_runtime/mfq_decode.cpp:1663-1744, 3579-3677
#include <algorithm>

#include "common.h"
#include "nvq_d4_256.h"

namespace mfqb {

void unpack_bits(const uint8_t* src, uint64_t count, int bits, uint8_t* dst) {
    if (bits == 8) {
        memcpy(dst, src, count);
        return;
    }
    const uint32_t mask = (1u << bits) - 1u;
    uint64_t acc = 0;
    int have = 0;
    for (uint64_t i = 0; i < count; ++i) {
        while (have < bits) {
            acc |= (uint64_t)(*src++) << have;
            have += 8;
        }
        dst[i] = (uint8_t)(acc & mask);
        acc >>= bits;
        have -= bits;
    }
}

void unpack_bits16(const uint8_t* src, uint64_t count, int bits, uint16_t* dst) {
    const uint32_t mask = (1u << bits) - 1u;
    uint64_t acc = 0;
    int have = 0;
    for (uint64_t i = 0; i < count; ++i) {
        while (have < bits) {
            acc |= (uint64_t)(*src++) << have;
            have += 8;
        }
        dst[i] = (uint16_t)(acc & mask);
        acc >>= bits;
        have -= bits;
    }
}

bool dtype_is_nint(const std::string& d) {
    return d.size() == 5 && d.compare(0, 4, "NINT") == 0 && d[4] >= '1' && d[4] <= '8';
}
bool dtype_is_nvq(const std::string& d) {
    return d == "NVQ3" || d == "NIQ3" || d == "NVQ3J" || d == "NVQ3J-512" || d == "NVQ3J-L";
}

HostNint parse_nint(const void* blob, uint64_t nbytes) {
    Cursor c(blob, nbytes);
    HostNint t;
    t.bits = c.get<uint8_t>("NINT header");
    t.sub_bits = c.get<uint8_t>("NINT header");
    t.gs = c.get<int32_t>("NINT header");
    const int32_t axis = c.get<int32_t>("NINT header");
    const int32_t neuron_len = c.get<int32_t>("NINT header");
    const uint32_t ndim = c.get<uint32_t>("NINT ndim");
    if (ndim == 0 || ndim > 8) fail(MFQB_ERR_FORMAT, "NINT blob: implausible rank %u", ndim);
    std::vector<int64_t> shape(ndim);
    for (auto& s : shape) s = c.get<int64_t>("NINT shape");
    const uint32_t out = c.get<uint32_t>("NINT out");
    const uint32_t ng = c.get<uint32_t>("NINT ng");
    if (t.bits < 1 || t.bits > 8 || t.sub_bits < 1 || t.sub_bits > 8 || t.gs <= 0 || neuron_len <= 0)
        fail(MFQB_ERR_FORMAT, "NINT blob: invalid profile bits=%d sub_bits=%d gs=%d len=%d", t.bits, t.sub_bits, t.gs,
             neuron_len);
    if ((int64_t)ng != ((int64_t)neuron_len + t.gs - 1) / t.gs)
        fail(MFQB_ERR_FORMAT, "NINT blob: ng=%u does not match neuron_len=%d / gs=%d", ng, neuron_len, t.gs);
    if (axis != 0 || ndim != 2 || shape[0] != (int64_t)out || shape[1] != neuron_len)
        fail(MFQB_ERR_UNSUPPORTED, "NINT blob: only rank-2 tensors quantized along axis 0 are executable");
    t.n = out;
    t.k = neuron_len;
    t.ng = ng;
    const uint64_t nsub = (uint64_t)out * ng, nq = nsub * (uint64_t)t.gs;
    const uint8_t* ns = c.take(2ull * out, "NINT neuron_scale");
    const uint8_t* nm = c.take(2ull * out, "NINT neuron_min");
    t.ns.resize(out);
    t.nm.resize(out);
    memcpy(t.ns.data(), ns, 2ull * out);
    memcpy(t.nm.data(), nm, 2ull * out);
    const uint64_t packed_tail = 2 * packed_nbytes(nsub, t.sub_bits) + packed_nbytes(nq, t.bits);
    const uint64_t legacy_tail = 2 * nsub + nq;  // whole-uint8 storage of older writers
    const uint64_t remaining = nbytes - c.off;
    // sizes come from the header: nothing is allocated for them before the tail length has confirmed them
    if (remaining != legacy_tail && remaining != packed_tail)
        fail(MFQB_ERR_FORMAT, "invalid NINT blob tail: remaining=%llu packed=%llu legacy=%llu",
             (unsigned long long)remaining, (unsigned long long)packed_tail, (unsigned long long)legacy_tail);
    t.ss.resize(nsub);
    t.sm.resize(nsub);
    t.q.resize(nq);
    if (remaining == legacy_tail) {
        memcpy(t.ss.data(), c.take(nsub, "NINT sub_scale"), nsub);
        memcpy(t.sm.data(), c.take(nsub, "NINT sub_min"), nsub);
        memcpy(t.q.data(), c.take(nq, "NINT q"), nq);
    } else if (remaining == packed_tail) {
        unpack_bits(c.take(packed_nbytes(nsub, t.sub_bits), "NINT sub_scale"), nsub, t.sub_bits, t.ss.data());
        unpack_bits(c.take(packed_nbytes(nsub, t.sub_bits), "NINT sub_min"), nsub, t.sub_bits, t.sm.data());
        unpack_bits(c.take(packed_nbytes(nq, t.bits), "NINT q"), nq, t.bits, t.q.data());
    } else {
        fail(MFQB_ERR_FORMAT, "invalid NINT blob tail: remaining=%llu packed=%llu legacy=%llu",
             (unsigned long long)remaining, (unsigned long long)packed_tail, (unsigned long long)legacy_tail);
    }
    return t;
}

uint64_t nint_payload_bytes(const HostNint& t) {
    const uint64_t nsub = (uint64_t)t.n * t.ng;
    return 4ull * t.n + 2 * packed_nbytes(nsub, t.sub_bits) + packed_nbytes(nsub * t.gs, t.bits);
}

HostNint slice_nint(const HostNint& t, int axis, int64_t begin, int64_t end) {
    if (axis == 0) {
        if (end < 0) end = t.n;
        if (begin < 0 || begin >= end || end > t.n) fail(MFQB_ERR_ARG, "NINT row slice [%lld,%lld) out of range", (long long)begin, (long long)end);
        HostNint r = t;
        r.n = end - begin;
        r.ns.assign(t.ns.begin() + begin, t.ns.begin() + end);
        r.nm.assign(t.nm.begin() + begin, t.nm.begin() + end);
        r.ss.assign(t.ss.begin() + begin * t.ng, t.ss.begin() + end * t.ng);
        r.sm.assign(t.sm.begin() + begin * t.ng, t.sm.begin() + end * t.ng);
        r.q.assign(t.q.begin() + begin * t.ng * t.gs, t.q.begin() + end * t.ng * t.gs);
        return r;
    }
    if (axis != 1) fail(MFQB_ERR_ARG, "slice axis must be 0 (rows) or 1 (columns)");
    if (end < 0) end = t.k;
    if (begin < 0 || begin >= end || end > t.k) fail(MFQB_ERR_ARG, "NINT column slice [%lld,%lld) out of range", (long long)begin, (long long)end);
    if (begin % t.gs != 0 || (end != t.k && end % t.gs != 0))
        fail(MFQB_ERR_ARG, "NINT column slices must start and end on group boundaries (gs=%d)", t.gs);
    const int64_t g0 = begin / t.gs, g1 = (end + t.gs - 1) / t.gs, ngs = g1 - g0;
    HostNint r;
    r.bits = t.bits;
    r.sub_bits = t.sub_bits;
    r.gs = t.gs;
    r.n = t.n;
    r.k = end - begin;
    r.ng = ngs;
    r.ns = t.ns;
    r.nm = t.nm;
    r.ss.resize((size_t)t.n * ngs);
    r.sm.resize((size_t)t.n * ngs);
    r.q.resize((size_t)t.n * ngs * t.gs);
    for (int64_t row = 0; row < t.n; ++row) {
        memcpy(&r.ss[row * ngs], &t.ss[row * t.ng + g0], ngs);
        memcpy(&r.sm[row * ngs], &t.sm[row * t.ng + g0], ngs);
        memcpy(&r.q[row * ngs * t.gs], &t.q[(row * t.ng + g0) * t.gs], (size_t)ngs * t.gs);
    }
    return r;
}

HostNvq parse_nvq(const void* blob, uint64_t nbytes) {
    Cursor c(blob, nbytes);
    const uint8_t* magic = c.take(4, "NVQ magic");
    if (memcmp(magic, "NVQ1", 4) != 0 && memcmp(magic, "NIQ1", 4) != 0) fail(MFQB_ERR_FORMAT, "invalid NVQ magic");
    const uint8_t prof = c.get<uint8_t>("NVQ header");
    HostNvq t;
    t.sub_bits = c.get<uint8_t>("NVQ header");
    t.gs = c.get<uint16_t>("NVQ header");
    const int32_t axis = c.get<int32_t>("NVQ header");
    const int32_t neuron_len = c.get<int32_t>("NVQ header");
    const uint32_t ndim = c.get<uint32_t>("NVQ header");
    const bool index_parity = prof & 0x80, custom = prof & 0x40;
    t.jsc = prof & 0x20;
    const int cid = prof & 0x1F;
    switch (cid) {
        case 2: t.index_bits = 8; break;   // d4_256
        case 3: t.index_bits = 9; break;   // d4_512
        case 6: t.index_bits = 10; break;  // d4_1024
        case 1: case 4: case 5:
            fail(MFQB_ERR_UNSUPPORTED, "NVQ2 (E8 lattice) tensors are outside the NVQ3 execution path");
        default: fail(MFQB_ERR_FORMAT, "unknown NVQ codebook id %d", cid);
    }
    if (index_parity) fail(MFQB_ERR_FORMAT, "index-parity signs require the E8 codebook");
    t.vec = 4;
    t.entries = 1 << t.index_bits;
    if (ndim == 0 || ndim > 8) fail(MFQB_ERR_FORMAT, "NVQ blob: implausible rank %u", ndim);
    std::vector<int64_t> shape(ndim);
    for (auto& s : shape) s = c.get<int64_t>("NVQ shape");
    const uint32_t out = c.get<uint32_t>("NVQ out");
    if (neuron_len <= 0 || t.gs <= 0 || t.gs % 8 || t.sub_bits < 1 || t.sub_bits > 8)
        fail(MFQB_ERR_FORMAT, "NVQ blob: invalid profile gs=%d sub_bits=%d len=%d", t.gs, t.sub_bits, neuron_len);
    if (axis != 0 || ndim != 2 || shape[0] != (int64_t)out || shape[1] != neuron_len)
        fail(MFQB_ERR_UNSUPPORTED, "NVQ blob: only rank-2 tensors quantized along axis 0 are executable");
    if (t.gs != 24) fail(MFQB_ERR_UNSUPPORTED, "NVQ blob: the execution path requires groupsize 24, got %d", t.gs);
    if (t.jsc) {
        if (custom || t.sub_bits != 4) fail(MFQB_ERR_FORMAT, "invalid NVQ-JSC profile flags");
        const uint8_t* h = c.take(64, "NVQ-JSC metadata header");
        const int version = h[0], banks = h[1], states = h[2], mode = h[3];
        if (version != 1) fail(MFQB_ERR_FORMAT, "unsupported NVQ-JSC metadata version %d", version);
        if ((banks != 1 && banks != 2 && banks != 4) || states != 16 || (mode != 0 && mode != 1))
            fail(MFQB_ERR_FORMAT, "invalid NVQ-JSC table dimensions");
        for (int i = 52; i < 64; ++i)
            if (h[i]) fail(MFQB_ERR_FORMAT, "NVQ-JSC reserved metadata bytes must be zero");
        memcpy(t.lut_h, h + 4, 32);
        memcpy(t.bank_for_state, h + 36, 16);
        for (int i = 0; i < 16; ++i)
            if (t.bank_for_state[i] >= banks) fail(MFQB_ERR_FORMAT, "invalid NVQ-JSC state-to-bank map");
        t.banks = banks;
        const uint64_t nb = (uint64_t)banks * t.entries * t.vec;
        const uint8_t* cb = c.take(nb, "NVQ-JSC codebook banks");
        t.codebooks.assign(reinterpret_cast<const int8_t*>(cb), reinterpret_cast<const int8_t*>(cb) + nb);
        for (int8_t v : t.codebooks)
            if (v < 0) fail(MFQB_ERR_FORMAT, "NVQ-JSC codebook entries must be in [0,127]");
        t.table_bytes = 64 + nb;
    } else {
        t.banks = 1;
        t.codebooks.resize((size_t)t.entries * 4);
        if (custom) {
            const uint8_t* cb = c.take(2ull * t.entries, "NVQ custom codebook");
            for (int e = 0; e < t.entries; ++e) {
                uint16_t enc;
                memcpy(&enc, cb + 2 * e, 2);
                for (int j = 0; j < 4; ++j) t.codebooks[e * 4 + j] = (int8_t)(2 * ((enc >> (3 * j)) & 7) + 1);
            }
            t.table_bytes = 2ull * t.entries;
        } else {
            if (cid != 2) fail(MFQB_ERR_UNSUPPORTED, "only the 256-entry D4 grid is built in; larger grids travel as NVQ-JSC banks");
            for (int e = 0; e < 256; ++e)
                for (int j = 0; j < 4; ++j) t.codebooks[e * 4 + j] = (int8_t)(2 * ((kD4_256_packed[e] >> (3 * j)) & 7) + 1);
        }
    }
    t.n = out;
    t.k = neuron_len;
    t.ng = (t.k + t.gs - 1) / t.gs;
    t.nvec = (t.k + 3) / 4;
    t.nsign = (t.k + 7) / 8;
    const uint8_t* an = c.take(2ull * out, "NVQ anchors");
    t.anchors.resize(out);
    memcpy(t.anchors.data(), an, 2ull * out);
    const uint64_t nsub = (uint64_t)out * t.ng, nidx = (uint64_t)out * t.nvec, nsg = (uint64_t)out * t.nsign;
    t.sub.resize(nsub);
    t.idx.resize(nidx);
    t.signs.resize(nsg);
    unpack_bits(c.take(packed_nbytes(nsub, t.sub_bits), "NVQ sub-scales"), nsub, t.sub_bits, t.sub.data());
    unpack_bits16(c.take(packed_nbytes(nidx, t.index_bits), "NVQ indices"), nidx, t.index_bits, t.idx.data());
    unpack_bits(c.take(packed_nbytes(nsg, 7), "NVQ signs"), nsg, 7, t.signs.data());
    if (c.off != nbytes) fail(MFQB_ERR_FORMAT, "invalid NVQ blob tail: consumed=%llu size=%llu", (unsigned long long)c.off, (unsigned long long)nbytes);
    if (t.jsc)
        for (uint8_t s : t.sub)
            if (s > 15) fail(MFQB_ERR_FORMAT, "NVQ-JSC state out of range");
    return t;
}

uint64_t nvq_payload_bytes(const HostNvq& t) {
    return 2ull * t.n + packed_nbytes((uint64_t)t.n * t.ng, t.sub_bits) + packed_nbytes((uint64_t)t.n * t.nvec, t.index_bits) +
           packed_nbytes((uint64_t)t.n * t.nsign, 7) + t.table_bytes;
}

HostNvq slice_nvq(const HostNvq& t, int axis, int64_t begin, int64_t end) {
    HostNvq r = t;
    if (axis == 0) {
        if (end < 0) end = t.n;
        if (begin < 0 || begin >= end || end > t.n) fail(MFQB_ERR_ARG, "NVQ row slice out of range");
        r.n = end - begin;
        r.anchors.assign(t.anchors.begin() + begin, t.anchors.begin() + end);
        r.sub.assign(t.sub.begin() + begin * t.ng, t.sub.begin() + end * t.ng);
        r.idx.assign(t.idx.begin() + begin * t.nvec, t.idx.begin() + end * t.nvec);
        r.signs.assign(t.signs.begin() + begin * t.nsign, t.signs.begin() + end * t.nsign);
        return r;
    }
    if (axis != 1) fail(MFQB_ERR_ARG, "slice axis must be 0 (rows) or 1 (columns)");
    if (end < 0) end = t.k;
    if (begin < 0 || begin >= end || end > t.k) fail(MFQB_ERR_ARG, "NVQ column slice out of range");
    // Groups (24), index vectors (4) and sign blocks (8) all restart at multiples of 24.
    if (begin % 24 != 0 || (end != t.k && end % 24 != 0))
        fail(MFQB_ERR_ARG, "NVQ column slices must start and end on multiples of 24");
    r.k = end - begin;
    r.ng = (r.k + 23) / 24;
    r.nvec = (r.k + 3) / 4;
    r.nsign = (r.k + 7) / 8;
    r.sub.resize((size_t)t.n * r.ng);
    r.idx.resize((size_t)t.n * r.nvec);
    r.signs.resize((size_t)t.n * r.nsign);
    for (int64_t row = 0; row < t.n; ++row) {
        memcpy(&r.sub[row * r.ng], &t.sub[row * t.ng + begin / 24], r.ng);
        memcpy(&r.idx[row * r.nvec], &t.idx[row * t.nvec + begin / 4], 2 * (size_t)r.nvec);
        memcpy(&r.signs[row * r.nsign], &t.signs[row * t.nsign + begin / 8], r.nsign);
    }
    return r;
}

HostNintm parse_nintm(const void* blob, uint64_t nbytes) {
    Cursor c(blob, nbytes);
    const uint8_t* magic = c.take(4, "NINTM header");
    const bool v1 = memcmp(magic, "NIM1", 4) == 0, v2 = memcmp(magic, "NIM2", 4) == 0;
    if (!v1 && !v2) fail(MFQB_ERR_FORMAT, "invalid NINTM magic");
    HostNintm t;
    t.n_experts = c.get<uint32_t>("NINTM header");
    t.out_per_expert = c.get<uint32_t>("NINTM header");
    t.k = c.get<uint32_t>("NINTM header");
    const uint32_t pool_count = c.get<uint32_t>("NINTM header");
    if (pool_count == 0 || pool_count > t.n_experts) fail(MFQB_ERR_FORMAT, "invalid NINTM pool count");
    std::vector<int> owner((size_t)t.n_experts, -1);
    for (uint32_t p = 0; p < pool_count; ++p) {
        uint32_t count, dlen = 0;
        uint64_t payload, runtime = 0;
        if (v1) {
            count = c.get<uint32_t>("NINTM pool header");
            payload = c.get<uint64_t>("NINTM pool header");
        } else {
            count = c.get<uint32_t>("NINTM pool header");
            dlen = c.get<uint32_t>("NINTM pool header");
            payload = c.get<uint64_t>("NINTM pool header");
            runtime = c.get<uint64_t>("NINTM pool header");
            if (dlen == 0 || dlen > 32) fail(MFQB_ERR_FORMAT, "invalid NINTM v2 pool metadata");
        }
        if (count == 0) fail(MFQB_ERR_FORMAT, "NINTM precision pools cannot be empty");
        HostNintmPool pool;
        pool.expert_ids.resize(count);
        memcpy(pool.expert_ids.data(), c.take(4ull * count, "NINTM expert ids"), 4ull * count);
        if (v2) {
            const uint8_t* d = c.take(dlen, "NINTM cohort dtype");
            pool.dtype.assign(reinterpret_cast<const char*>(d), dlen);
            c.take(runtime, "NINTM runtime metadata");
        }
        const uint8_t* pl = c.take(payload, "NINTM pool payload");
        if (v1) pool.dtype = "NINT" + std::to_string(payload ? pl[0] : 0);
        if (!dtype_is_nint(pool.dtype))
            fail(MFQB_ERR_UNSUPPORTED, "NINTM cohort dtype '%s' is outside the NINT execution path", pool.dtype.c_str());
        if (runtime) fail(MFQB_ERR_FORMAT, "unexpected NINTM cohort runtime metadata for a NINT cohort");
        pool.tensor = parse_nint(pl, payload);
        if (pool.tensor.n != (int64_t)count * t.out_per_expert || pool.tensor.k != t.k)
            fail(MFQB_ERR_FORMAT, "NINTM pool %u tensor shape does not match its expert count", p);
        for (int32_t e : pool.expert_ids) {
            if (e < 0 || e >= t.n_experts) fail(MFQB_ERR_FORMAT, "NINTM pool %u contains an invalid expert id", p);
            if (owner[e] >= 0) fail(MFQB_ERR_FORMAT, "an expert belongs to multiple NINTM pools");
            owner[e] = (int)p;
        }
        t.pools.push_back(std::move(pool));
    }
    if (c.off != nbytes) fail(MFQB_ERR_FORMAT, "invalid NINTM tail: %llu extra bytes", (unsigned long long)(nbytes - c.off));
    for (int64_t e = 0; e < t.n_experts; ++e)
        if (owner[e] < 0) fail(MFQB_ERR_FORMAT, "NINTM pools do not cover expert %lld", (long long)e);
    return t;
}

}  // namespace mfqb
