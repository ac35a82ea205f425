// GGUF expert reader and bank packer (host code): finds the stacked 3-D expert tensors of a GGUF checkpoint
// ([cols, rows, experts], e.g. blk.N.ffn_gate_exps.weight), addresses one expert or a block of experts without touching
// the rest, and packs the block straight into the library's bank layout, ready for one upload.
// Replaces the part of the reference's reader that serves the expert path: gguf_expert_slice / gguf_expert_count
// (src/core/gguf.hpp:77-91, src/core/gguf.cpp:174-213), the block table for the five expert formats (gguf.cpp:116-152) and
// the loaders' repack (src/formats/weight/q4.cpp:295-325,495-607,802-832); like the packed expert file of
// src/experts/packed_experts.hpp:2-5 the result is a bank that needs no repack on the device. The file is mapped
// read-only; nothing is copied until a bank is packed. Inconsistent files are refused, never guessed at (a wrong slice
// reads a neighbouring expert's weights and still produces plausible numbers).
//
// GGUF (version 2 and 3, little-endian): magic "GGUF", u32 version, u64 tensor count, u64 key/value count; key/value pairs
// (string key, u32 value type, value); tensor infos (string name, u32 rank, u64 dims, u32 type, u64 offset into the data
// section); the data section starts at the next multiple of general.alignment (default 32).
#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <cstring>
#include <string>
#include <vector>

#include "common.cuh"

namespace b2 {
namespace {

struct GgufTensorInfo {
    std::string name;
    uint32_t type = 0, rank = 0;
    uint64_t ne[4] = {1, 1, 1, 1};
    uint64_t offset = 0;          // from the start of the file
};
struct GgufFile {
    const uint8_t * map = nullptr;
    size_t bytes = 0;
    std::vector<GgufTensorInfo> tensors;
};

struct Cursor {
    const uint8_t * p;
    size_t left;
    bool ok = true;
    template <class T> T get() {
        T v{};
        if (left < sizeof(T)) { ok = false; left = 0; return v; }
        std::memcpy(&v, p, sizeof(T));
        p += sizeof(T); left -= sizeof(T);
        return v;
    }
    void skip(uint64_t n) {
        if (n > left) { ok = false; left = 0; return; }
        p += n; left -= size_t(n);
    }
    std::string str() {
        const uint64_t n = get<uint64_t>();
        if (!ok || n > left) { ok = false; return std::string(); }
        std::string s(reinterpret_cast<const char *>(p), size_t(n));
        skip(n);
        return s;
    }
};
// bytes of one scalar of a GGUF value type, 0 for strings / arrays / unknown types
size_t scalar_bytes(uint32_t t) {
    switch (t) {
        case 0: case 1: case 7: return 1;
        case 2: case 3: return 2;
        case 4: case 5: case 6: return 4;
        case 10: case 11: case 12: return 8;
        default: return 0;
    }
}
bool skip_value(Cursor & c, uint32_t type, int depth = 0) {
    if (type == 8) { c.str(); return c.ok; }
    if (type == 9) {
        if (depth > 2) return false;
        const uint32_t et = c.get<uint32_t>();
        const uint64_t n = c.get<uint64_t>();
        if (!c.ok) return false;
        if (const size_t sb = scalar_bytes(et)) {
            if (n > c.left / sb) return false;
            c.skip(n * sb);
            return c.ok;
        }
        for (uint64_t i = 0; i < n && c.ok; ++i)
            if (!skip_value(c, et, depth + 1)) return false;
        return c.ok;
    }
    const size_t sb = scalar_bytes(type);
    if (!sb) return false;
    c.skip(sb);
    return c.ok;
}

const GgufTensorInfo * find(const GgufFile * f, const char * name) {
    for (const auto & t : f->tensors)
        if (t.name == name) return &t;
    return nullptr;
}
// raw bytes of `rows` rows of `cols` weights of a block format the library knows, 0 otherwise
uint64_t expert_bytes(uint32_t type, uint64_t rows, uint64_t cols) {
    if (rows == 0 || cols == 0 || rows > 0x7fffffffull || cols > 0x7fffffffull) return 0;
    return b2moe_raw_bytes(type, int32_t(rows), int32_t(cols));
}

}  // namespace
}  // namespace b2

using namespace b2;

extern "C" B2MOE_API int32_t b2moe_gguf_open(const char * path, void ** handle) {
    if (!path || !handle) return B2MOE_ERR_NULL;
    *handle = nullptr;
    const int fd = ::open(path, O_RDONLY);
    if (fd < 0) return B2MOE_ERR_FORMAT;
    struct stat st;
    if (::fstat(fd, &st) != 0 || st.st_size < 24) { ::close(fd); return B2MOE_ERR_FORMAT; }
    void * m = ::mmap(nullptr, size_t(st.st_size), PROT_READ, MAP_PRIVATE, fd, 0);
    ::close(fd);
    if (m == MAP_FAILED) return B2MOE_ERR_FORMAT;
    GgufFile * f = new GgufFile;
    f->map = static_cast<const uint8_t *>(m);
    f->bytes = size_t(st.st_size);
    auto fail = [&]() { ::munmap(m, f->bytes); delete f; return int32_t(B2MOE_ERR_FORMAT); };
    Cursor c{f->map, f->bytes};
    if (c.get<uint32_t>() != 0x46554747u) return fail();                       // "GGUF"
    const uint32_t version = c.get<uint32_t>();
    if (version != 2 && version != 3) return fail();
    const uint64_t n_tensors = c.get<uint64_t>(), n_kv = c.get<uint64_t>();
    if (!c.ok || n_tensors > (1ull << 24) || n_kv > (1ull << 24)) return fail();
    uint64_t alignment = 32;
    for (uint64_t i = 0; i < n_kv; ++i) {
        const std::string key = c.str();
        const uint32_t vt = c.get<uint32_t>();
        if (!c.ok) return fail();
        if (key == "general.alignment" && vt == 4) {
            alignment = c.get<uint32_t>();
            if (!c.ok || alignment == 0 || (alignment & (alignment - 1))) return fail();
        } else if (!skip_value(c, vt)) return fail();
    }
    f->tensors.reserve(size_t(n_tensors));
    for (uint64_t i = 0; i < n_tensors; ++i) {
        GgufTensorInfo t;
        t.name = c.str();
        t.rank = c.get<uint32_t>();
        if (!c.ok || t.rank == 0 || t.rank > 4) return fail();
        for (uint32_t d = 0; d < t.rank; ++d) t.ne[d] = c.get<uint64_t>();
        t.type = c.get<uint32_t>();
        t.offset = c.get<uint64_t>();                                          // relative to the data section for now
        if (!c.ok) return fail();
        f->tensors.push_back(std::move(t));
    }
    const uint64_t consumed = f->bytes - c.left, data0 = (consumed + alignment - 1) / alignment * alignment;
    if (data0 > f->bytes) return fail();
    for (auto & t : f->tensors) {
        if (t.offset % alignment || t.offset > f->bytes - data0) return fail();
        t.offset += data0;
    }
    *handle = f;
    return B2MOE_OK;
}

extern "C" B2MOE_API void b2moe_gguf_close(void * handle) {
    GgufFile * f = static_cast<GgufFile *>(handle);
    if (!f) return;
    ::munmap(const_cast<uint8_t *>(f->map), f->bytes);
    delete f;
}

extern "C" B2MOE_API int32_t b2moe_gguf_tensor_count(const void * handle) {
    return handle ? int32_t(static_cast<const GgufFile *>(handle)->tensors.size()) : 0;
}

extern "C" B2MOE_API int32_t b2moe_gguf_tensor_name(const void * handle, int32_t index, char * name, int32_t name_bytes) {
    const GgufFile * f = static_cast<const GgufFile *>(handle);
    if (!f || !name) return B2MOE_ERR_NULL;
    if (index < 0 || size_t(index) >= f->tensors.size() || name_bytes <= 0) return B2MOE_ERR_SHAPE;
    const std::string & s = f->tensors[size_t(index)].name;
    if (s.size() + 1 > size_t(name_bytes)) return B2MOE_ERR_CAPACITY;
    std::memcpy(name, s.c_str(), s.size() + 1);
    return B2MOE_OK;
}

// type, dims (cols, rows, experts; 1 beyond the tensor's rank) and the byte range of a tensor inside the file
extern "C" B2MOE_API int32_t b2moe_gguf_tensor(const void * handle, const char * name, uint32_t * type, int64_t dims[3], uint64_t * offset,
                                               uint64_t * bytes) {
    const GgufFile * f = static_cast<const GgufFile *>(handle);
    if (!f || !name) return B2MOE_ERR_NULL;
    const GgufTensorInfo * t = find(f, name);
    if (!t) return B2MOE_ERR_SHAPE;
    if (t->rank > 3) return B2MOE_ERR_SHAPE;
    if (type) *type = t->type;
    if (dims) for (int d = 0; d < 3; ++d) dims[d] = int64_t(t->ne[d]);
    if (offset) *offset = t->offset;
    if (bytes) {
        const uint64_t per = expert_bytes(t->type, t->ne[1], t->ne[0]);
        *bytes = per * t->ne[2];                                               // 0 for a block format the library does not know
    }
    return B2MOE_OK;
}

// experts [first, first + count) of the 3-D expert tensor `name` (or the one matrix of a 2-D tensor): a pointer into the mapped
// file (raw GGUF rows, expert-major) and its length. Refuses a tensor of another rank, an expert range outside it, a block format the library does
// not serve, a row length that is not whole blocks, and a byte range that leaves the file.
extern "C" B2MOE_API int32_t b2moe_gguf_expert_slice(const void * handle, const char * name, int32_t first, int32_t count, uint32_t * type,
                                                     int32_t * rows, int32_t * cols, const void ** raw, uint64_t * raw_bytes) {
    const GgufFile * f = static_cast<const GgufFile *>(handle);
    if (!f || !name || !raw || !raw_bytes) return B2MOE_ERR_NULL;
    const GgufTensorInfo * t = find(f, name);
    if (!t || t->rank < 2 || t->rank > 3 || t->ne[2] == 0) return B2MOE_ERR_SHAPE;      // a 2-D matrix (a shared expert) counts as one expert
    if (first < 0 || count <= 0 || uint64_t(first) + uint64_t(count) > t->ne[2]) return B2MOE_ERR_SHAPE;
    const uint64_t per = expert_bytes(t->type, t->ne[1], t->ne[0]);
    if (per == 0) return B2MOE_ERR_FORMAT;
    const uint64_t begin = t->offset + per * uint64_t(first), len = per * uint64_t(count);
    if (per * t->ne[2] > f->bytes - t->offset) return B2MOE_ERR_FORMAT;        // the whole tensor must lie inside the file
    if (type) *type = t->type;
    if (rows) *rows = int32_t(t->ne[1]);
    if (cols) *cols = int32_t(t->ne[0]);
    *raw = f->map + begin;
    *raw_bytes = len;
    return B2MOE_OK;
}

// The same experts packed into the bank layout of `bank_type` (the tensor's own type, or B2MOE_IQ3_S_X4 for an IQ3_S
// tensor): data / aux are host buffers of b2moe_bank_bytes / b2moe_bank_aux_bytes(bank_type, count * rows, cols) bytes,
// ready for one upload as a bank of `count` experts. rows must be a multiple of 16 (stacked experts keep whole row tiles).
extern "C" B2MOE_API int32_t b2moe_gguf_expert_bank(const void * handle, const char * name, int32_t first, int32_t count, uint32_t bank_type,
                                                    void * data, void * aux) {
    uint32_t type = 0;
    int32_t rows = 0, cols = 0;
    const void * raw = nullptr;
    uint64_t raw_bytes = 0;
    if (int32_t rc = b2moe_gguf_expert_slice(handle, name, first, count, &type, &rows, &cols, &raw, &raw_bytes)) return rc;
    if (bank_type != type && !(bank_type == B2MOE_IQ3_S_X4 && type == B2MOE_IQ3_S)) return B2MOE_ERR_FORMAT;
    if (rows % 16) return B2MOE_ERR_SHAPE;
    return b2moe_bank_pack_host(bank_type, raw, count, rows, cols, data, aux);
}
