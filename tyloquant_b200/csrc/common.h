// Shared host-side declarations: status/error plumbing, parsed (host) tensors, bit reader.
#pragma once
#include <cstdarg>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <stdexcept>
#include <string>
#include <vector>

#include "../../include/mfqb200.h"

namespace mfqb {

// Thrown inside the library, translated to a status + message at the C boundary.
struct Error : std::runtime_error {
    int code;
    Error(int c, const std::string& m) : std::runtime_error(m), code(c) {}
};

[[noreturn]] inline void fail(int code, const char* fmt, ...) {
    char buf[512];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof buf, fmt, ap);
    va_end(ap);
    throw Error(code, buf);
}

void set_last_error(const std::string& msg);

template <class F>
int guarded(F&& f) noexcept {
    try {
        f();
        return MFQB_OK;
    } catch (const Error& e) {
        set_last_error(e.what());
        return e.code;
    } catch (const std::bad_alloc&) {
        set_last_error("out of host memory");
        return MFQB_ERR_ARG;
    } catch (const std::exception& e) {
        set_last_error(e.what());
        return MFQB_ERR_ARG;
    }
}

// ---- little-endian cursor over a byte range -------------------------------------------
struct Cursor {
    const uint8_t* p;
    uint64_t n, off = 0;
    Cursor(const void* d, uint64_t len) : p(static_cast<const uint8_t*>(d)), n(len) {}
    void need(uint64_t k, const char* what) const {
        if (k > n - off) fail(MFQB_ERR_FORMAT, "truncated %s (need %llu bytes at %llu of %llu)", what,
                              (unsigned long long)k, (unsigned long long)off, (unsigned long long)n);
    }
    template <class T>
    T get(const char* what) {
        need(sizeof(T), what);
        T v;
        memcpy(&v, p + off, sizeof(T));
        off += sizeof(T);
        return v;
    }
    const uint8_t* take(uint64_t k, const char* what) {
        need(k, what);
        const uint8_t* r = p + off;
        off += k;
        return r;
    }
};

// LSB-first bitstream: value i of width b occupies stream bits [i*b, i*b+b).
// (mfq/formats/io.py:144-188, mfq/formats/nvq.py:559-583)
void unpack_bits(const uint8_t* src, uint64_t count, int bits, uint8_t* dst);
void unpack_bits16(const uint8_t* src, uint64_t count, int bits, uint16_t* dst);
inline uint64_t packed_nbytes(uint64_t count, int bits) { return (count * (uint64_t)bits + 7) / 8; }

// ---- parsed tensors (host) ------------------------------------------------------------
struct HostNint {
    int bits = 0, sub_bits = 0, gs = 0;
    int64_t n = 0, k = 0, ng = 0;          // rows, columns (neuron_len), groups per row
    std::vector<uint16_t> ns, nm;          // f16 bit patterns [n]
    std::vector<uint8_t> ss, sm;           // [n*ng]
    std::vector<uint8_t> q;                // [n*ng*gs]
};

struct HostNvq {
    int index_bits = 0, vec = 4, sub_bits = 4, gs = 24;
    bool jsc = false;
    int banks = 1, entries = 256;
    int64_t n = 0, k = 0, ng = 0, nvec = 0, nsign = 0;
    std::vector<uint16_t> anchors;         // f16 bits [n]
    std::vector<uint8_t> sub;              // [n*ng] sub-scale (plain) or state (JSC)
    std::vector<uint16_t> idx;             // [n*nvec]
    std::vector<uint8_t> signs;            // [n*nsign] 7-bit masks
    std::vector<int8_t> codebooks;         // [banks*entries*vec]
    uint16_t lut_h[16] = {0};              // JSC: f16 scale LUT
    uint8_t bank_for_state[16] = {0};      // JSC
    uint64_t table_bytes = 0;              // bytes of in-blob tables (JSC header+banks / custom codebook)
};

struct HostNintmPool {
    std::vector<int32_t> expert_ids;
    std::string dtype;
    HostNint tensor;                       // rows = expert_ids.size() * out_per_expert
};
struct HostNintm {
    int64_t n_experts = 0, out_per_expert = 0, k = 0;
    std::vector<HostNintmPool> pools;
};

HostNint parse_nint(const void* blob, uint64_t nbytes);
HostNvq parse_nvq(const void* blob, uint64_t nbytes);
HostNintm parse_nintm(const void* blob, uint64_t nbytes);
HostNint slice_nint(const HostNint& t, int axis, int64_t begin, int64_t end);
HostNvq slice_nvq(const HostNvq& t, int axis, int64_t begin, int64_t end);
uint64_t nint_payload_bytes(const HostNint& t);
uint64_t nvq_payload_bytes(const HostNvq& t);

bool dtype_is_nint(const std::string& dtype);
bool dtype_is_nvq(const std::string& dtype);

inline float f16_to_f32(uint16_t h) {
    const uint32_t s = (uint32_t)(h & 0x8000) << 16;
    uint32_t e = (h >> 10) & 0x1F, m = h & 0x3FF, bits;
    if (e == 0) {
        if (m == 0) bits = s;
        else {
            int sh = 0;
            while (!(m & 0x400)) { m <<= 1; ++sh; }
            bits = s | ((uint32_t)(113 - sh) << 23) | ((m & 0x3FF) << 13);
        }
    } else if (e == 31) bits = s | 0x7F800000u | (m << 13);
    else bits = s | ((e + 112) << 23) | (m << 13);
    float f;
    memcpy(&f, &bits, 4);
    return f;
}

}  // namespace mfqb
