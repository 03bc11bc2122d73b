// MFQ container reader: header, record table, blob access, shard sets.
// Mirrors MfqFile (cpp_runtime/mfq_decode.cpp:1294-1527) and the Python reader
// (mfq/formats/io.py:782-831).
#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <memory>
#include <utility>

#include "common.h"

namespace mfqb {

static thread_local std::string g_last_error;
void set_last_error(const std::string& msg) { g_last_error = msg; }
const char* last_error_cstr() { return g_last_error.c_str(); }

struct Source {                 // one physical file (or memory image)
    const uint8_t* data = nullptr;
    uint64_t size = 0;
    bool mapped = false;
    std::vector<uint8_t> owned;
    ~Source() {
        if (mapped && data) munmap(const_cast<uint8_t*>(data), size);
    }
};

struct Record {
    std::string name, dtype;
    uint64_t offset = 0, nbytes = 0;
    int source = 0;
};

}  // namespace mfqb

struct mfqb_file {
    uint32_t version = 0;
    std::string arch;
    std::vector<std::pair<std::string, std::string>> extra;
    std::vector<mfqb::Record> records;
    std::vector<std::unique_ptr<mfqb::Source>> sources;
};

namespace mfqb {

static std::string read_str(Cursor& c, const char* what) {
    const uint32_t n = c.get<uint32_t>(what);
    const uint8_t* p = c.take(n, what);
    return std::string(reinterpret_cast<const char*>(p), n);
}

// Parse one image; appends its records (pointing at source index `si`).
static void parse_image(mfqb_file& f, int si, bool first) {
    const Source& s = *f.sources[si];
    Cursor c(s.data, s.size);
    const uint8_t* magic = c.take(4, "MFQ magic");
    if (memcmp(magic, "MFQ1", 4) != 0) fail(MFQB_ERR_FORMAT, "not an MFQ file (bad magic)");
    const uint32_t version = c.get<uint32_t>("version");
    std::string arch = read_str(c, "arch");
    std::vector<std::pair<std::string, std::string>> extra;
    if (version >= 2) {
        const uint32_t n_extra = c.get<uint32_t>("extra count");
        for (uint32_t i = 0; i < n_extra; ++i) {
            std::string k = read_str(c, "extra key");
            std::string v = read_str(c, "extra value");
            extra.emplace_back(std::move(k), std::move(v));
        }
    }
    const uint32_t nrec = c.get<uint32_t>("record count");
    // a table entry is at least two empty strings and a size (16 bytes): a larger count cannot be true
    if (nrec > (s.size - c.off) / 16) fail(MFQB_ERR_FORMAT, "MFQ record count %u does not fit the file", nrec);
    std::vector<Record> recs;
    recs.reserve(nrec);
    for (uint32_t i = 0; i < nrec; ++i) {
        Record r;
        r.name = read_str(c, "record name");
        r.dtype = read_str(c, "record dtype");
        r.nbytes = c.get<uint64_t>("record size");
        r.source = si;
        recs.push_back(std::move(r));
    }
    uint64_t off = c.off;
    for (auto& r : recs) {
        if (r.nbytes > s.size - off)
            fail(MFQB_ERR_FORMAT, "record '%s' runs past the end of the file", r.name.c_str());
        r.offset = off;
        off += r.nbytes;
    }
    if (off != s.size)
        fail(MFQB_ERR_FORMAT, "MFQ length mismatch: record table ends at %llu, file has %llu bytes",
             (unsigned long long)off, (unsigned long long)s.size);
    if (first) {
        f.version = version;
        f.arch = std::move(arch);
        f.extra = std::move(extra);
    }
    for (auto& r : recs) f.records.push_back(std::move(r));
}

static std::unique_ptr<Source> map_file(const std::string& path) {
    const int fd = open(path.c_str(), O_RDONLY);
    if (fd < 0) fail(MFQB_ERR_IO, "cannot open '%s'", path.c_str());
    struct stat st;
    if (fstat(fd, &st) != 0) {
        close(fd);
        fail(MFQB_ERR_IO, "cannot stat '%s'", path.c_str());
    }
    auto s = std::make_unique<Source>();
    s->size = (uint64_t)st.st_size;
    if (s->size == 0) {
        close(fd);
        fail(MFQB_ERR_FORMAT, "'%s' is empty", path.c_str());
    }
    void* p = mmap(nullptr, s->size, PROT_READ, MAP_PRIVATE, fd, 0);
    close(fd);
    if (p == MAP_FAILED) fail(MFQB_ERR_IO, "cannot map '%s'", path.c_str());
    s->data = static_cast<const uint8_t*>(p);
    s->mapped = true;
    return s;
}

// "<stem>-00001-of-00003.mfq" -> (stem, 1, 3); returns false when the name is not a shard.
static bool split_shard_name(const std::string& path, std::string& stem, int& no, int& count) {
    const size_t n = path.size();
    // "-ddddd-of-ddddd.mfq" is 19 characters
    if (n < 19 || path.compare(n - 4, 4, ".mfq") != 0) return false;
    const std::string tail = path.substr(n - 19, 15);  // "-ddddd-of-ddddd"
    if (tail[0] != '-' || tail.compare(6, 4, "-of-") != 0) return false;
    for (int i : {1, 2, 3, 4, 5, 10, 11, 12, 13, 14})
        if (tail[i] < '0' || tail[i] > '9') return false;
    stem = path.substr(0, n - 19);
    no = std::stoi(tail.substr(1, 5));
    count = std::stoi(tail.substr(10, 5));
    return count >= 1 && no >= 1 && no <= count;
}

static const std::string* find_extra(const mfqb_file& f, const char* key) {
    for (auto& kv : f.extra)
        if (kv.first == key) return &kv.second;
    return nullptr;
}

}  // namespace mfqb

using namespace mfqb;

extern "C" {
#pragma GCC visibility push(default)

const char* mfqb_last_error(void) { return mfqb::last_error_cstr(); }
int mfqb_version(void) { return 100; }

// Unsigned integer stored as JSON text in the extras (plain digits, optionally quoted).
static uint64_t extra_uint(const mfqb_file& f, const char* key, uint64_t fallback) {
    const std::string* v = find_extra(f, key);
    if (!v) return fallback;
    size_t i = 0;
    while (i < v->size() && ((*v)[i] == ' ' || (*v)[i] == '"')) ++i;
    if (i >= v->size() || (*v)[i] < '0' || (*v)[i] > '9') return fallback;
    uint64_t r = 0;
    for (; i < v->size() && (*v)[i] >= '0' && (*v)[i] <= '9'; ++i) r = r * 10 + (uint64_t)((*v)[i] - '0');
    return r;
}

int mfqb_file_open(const char* path, mfqb_file** out) {
    return guarded([&] {
        if (!path || !out) fail(MFQB_ERR_ARG, "mfqb_file_open: null argument");
        auto f = std::make_unique<mfqb_file>();
        f->sources.push_back(map_file(path));
        parse_image(*f, 0, true);
        const uint64_t split_no = extra_uint(*f, "split.no", 0);
        const uint64_t split_count = extra_uint(*f, "split.count", 1);
        if (split_count < 1 || split_count > 99999 || split_no >= split_count)
            fail(MFQB_ERR_FORMAT, "invalid MFQ split metadata in '%s'", path);
        if (split_count > 1) {
            // The shard set is named "<stem>-%05d-of-%05d.mfq" (1-based); the file name must
            // agree with the zero-based split.no / split.count stored in the file.
            std::string stem;
            int no = 0, count = 0;
            if (!split_shard_name(path, stem, no, count) || (uint64_t)no != split_no + 1 ||
                (uint64_t)count != split_count)
                fail(MFQB_ERR_FORMAT, "MFQ shard filename/metadata mismatch: '%s'", path);
            auto set = std::make_unique<mfqb_file>();
            uint64_t want_records = UINT64_MAX, want_tensors = UINT64_MAX;
            for (uint64_t i = 0; i < split_count; ++i) {
                char name[32];
                snprintf(name, sizeof name, "-%05d-of-%05d.mfq", (int)i + 1, count);
                mfqb_file one;
                one.sources.push_back(map_file(stem + name));
                parse_image(one, 0, true);
                if (extra_uint(one, "split.no", split_count) != i || extra_uint(one, "split.count", 0) != split_count)
                    fail(MFQB_ERR_FORMAT, "MFQ shard metadata mismatch: '%s%s'", stem.c_str(), name);
                if (one.version != f->version || one.arch != f->arch)
                    fail(MFQB_ERR_FORMAT, "MFQ shard architecture/version mismatch: '%s%s'", stem.c_str(), name);
                for (auto key_total : {std::make_pair("split.records.count", &want_records),
                                       std::make_pair("split.tensors.count", &want_tensors)}) {
                    const uint64_t v = extra_uint(one, key_total.first, UINT64_MAX);
                    if (*key_total.second == UINT64_MAX) *key_total.second = v;
                    else if (v != UINT64_MAX && v != *key_total.second)
                        fail(MFQB_ERR_FORMAT, "MFQ shard %s mismatch: '%s%s'", key_total.first, stem.c_str(), name);
                }
                if (i == 0) {
                    set->version = one.version;
                    set->arch = one.arch;
                    set->extra = one.extra;
                }
                for (auto& r : one.records) {
                    r.source = (int)i;
                    set->records.push_back(std::move(r));
                }
                set->sources.push_back(std::move(one.sources[0]));
            }
            uint64_t tensors = 0;
            for (auto& r : set->records)
                if (r.name.rfind("__mfq_asset__/", 0) != 0) ++tensors;
            if (want_records != UINT64_MAX && want_records != set->records.size())
                fail(MFQB_ERR_FORMAT, "MFQ shard record total mismatch");
            if (want_tensors != UINT64_MAX && want_tensors != tensors)
                fail(MFQB_ERR_FORMAT, "MFQ shard tensor total mismatch");
            f = std::move(set);
        }
        *out = f.release();
    });
}

int mfqb_file_open_memory(const void* image, uint64_t nbytes, mfqb_file** out) {
    return guarded([&] {
        if (!image || !out) fail(MFQB_ERR_ARG, "mfqb_file_open_memory: null argument");
        auto f = std::make_unique<mfqb_file>();
        auto s = std::make_unique<Source>();
        s->owned.assign(static_cast<const uint8_t*>(image), static_cast<const uint8_t*>(image) + nbytes);
        s->data = s->owned.data();
        s->size = nbytes;
        f->sources.push_back(std::move(s));
        parse_image(*f, 0, true);
        *out = f.release();
    });
}

int mfqb_file_close(mfqb_file* f) {
    delete f;
    return MFQB_OK;
}

int mfqb_file_header(const mfqb_file* f, uint32_t* version, const char** arch, int* n_extra, int* n_records) {
    return guarded([&] {
        if (!f) fail(MFQB_ERR_ARG, "null file handle");
        if (version) *version = f->version;
        if (arch) *arch = f->arch.c_str();
        if (n_extra) *n_extra = (int)f->extra.size();
        if (n_records) *n_records = (int)f->records.size();
    });
}

int mfqb_file_extra(const mfqb_file* f, int i, const char** key, const char** json) {
    return guarded([&] {
        if (!f || i < 0 || i >= (int)f->extra.size()) fail(MFQB_ERR_ARG, "extra index out of range");
        if (key) *key = f->extra[i].first.c_str();
        if (json) *json = f->extra[i].second.c_str();
    });
}

int mfqb_file_record(const mfqb_file* f, int i, const char** name, const char** dtype, uint64_t* nbytes) {
    return guarded([&] {
        if (!f || i < 0 || i >= (int)f->records.size()) fail(MFQB_ERR_ARG, "record index out of range");
        if (name) *name = f->records[i].name.c_str();
        if (dtype) *dtype = f->records[i].dtype.c_str();
        if (nbytes) *nbytes = f->records[i].nbytes;
    });
}

int mfqb_file_find(const mfqb_file* f, const char* name, int* index) {
    return guarded([&] {
        if (!f || !name || !index) fail(MFQB_ERR_ARG, "mfqb_file_find: null argument");
        *index = -1;
        for (size_t i = 0; i < f->records.size(); ++i)
            if (f->records[i].name == name) {
                *index = (int)i;
                break;
            }
    });
}

int mfqb_file_blob(const mfqb_file* f, int i, const void** data, uint64_t* nbytes) {
    return guarded([&] {
        if (!f || i < 0 || i >= (int)f->records.size() || !data) fail(MFQB_ERR_ARG, "record index out of range");
        const Record& r = f->records[i];
        *data = f->sources[r.source]->data + r.offset;
        if (nbytes) *nbytes = r.nbytes;
    });
}

#pragma GCC visibility pop
}  // extern "C"
