// GGUF reader and its flat C-ABI (include/b200_llama.h, "model files").
//
// Layout (ggml/include/gguf.h:1-46): magic "GGUF", u32 version, u64 tensor count, u64 key/value count; the
// key/value pairs (string key, u32 gguf_type, value; an array value is u32 element type, u64 count, elements);
// the tensor infos (string name, u32 n_dims, u64 dims[n_dims], u32 ggml_type, u64 offset); padding to
// `general.alignment` (32 when the key is absent); the tensor data.  Strings are u64 length + bytes.
// Every read is bounds-checked against the mapping: a truncated or corrupt file gives an error, not a fault.
#include "gguf_load.h"
#include "ggml_compat.h"

#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

namespace b200 {

namespace {

// gguf_type (ggml/include/gguf.h:53-68)
enum : uint32_t { G_U8 = 0, G_I8, G_U16, G_I16, G_U32, G_I32, G_F32, G_BOOL, G_STR, G_ARR, G_U64, G_I64, G_F64, G_COUNT };

size_t scalar_size(uint32_t t) {
    switch (t) {
        case G_U8: case G_I8: case G_BOOL: return 1;
        case G_U16: case G_I16: return 2;
        case G_U32: case G_I32: case G_F32: return 4;
        case G_U64: case G_I64: case G_F64: return 8;
        default: return 0;
    }
}

struct Cursor {
    const uint8_t * p; size_t size, pos = 0; bool ok = true;
    bool need(size_t n) { if (!ok || n > size - pos) { ok = false; return false; } return true; }
    template <typename T> T get() { T v{}; if (need(sizeof(T))) { memcpy(&v, p + pos, sizeof(T)); pos += sizeof(T); } return v; }
    std::string str() {
        const uint64_t n = get<uint64_t>();
        if (!ok || n > size - pos) { ok = false; return std::string(); }
        std::string s((const char *) p + pos, (size_t) n);
        pos += (size_t) n;
        return s;
    }
    void skip(uint64_t n) { if (!ok || n > size - pos) ok = false; else pos += (size_t) n; }
};

bool read_scalar(Cursor & c, uint32_t t, GgufValue & v) {
    switch (t) {
        case G_U8:   v.inum = c.get<uint8_t>();  break;
        case G_I8:   v.inum = c.get<int8_t>();   break;
        case G_U16:  v.inum = c.get<uint16_t>(); break;
        case G_I16:  v.inum = c.get<int16_t>();  break;
        case G_U32:  v.inum = c.get<uint32_t>(); break;
        case G_I32:  v.inum = c.get<int32_t>();  break;
        case G_BOOL: v.inum = c.get<uint8_t>() != 0; break;
        case G_U64:  v.inum = (int64_t) c.get<uint64_t>(); break;
        case G_I64:  v.inum = c.get<int64_t>();  break;
        case G_F32:  v.num = c.get<float>();  v.inum = (int64_t) v.num; return c.ok;
        case G_F64:  v.num = c.get<double>(); v.inum = (int64_t) v.num; return c.ok;
        default: return false;
    }
    v.num = (double) v.inum;
    return c.ok;
}

}  // namespace

GgufFile::~GgufFile() { if (base) munmap((void *) base, size); }

bool GgufFile::open(const char * path_, std::string & err) {
    path = path_ ? path_ : "";
    const int fd = ::open(path.c_str(), O_RDONLY);
    if (fd < 0) { err = "cannot open " + path; return false; }
    struct stat st;
    if (fstat(fd, &st) != 0 || st.st_size < 24) { ::close(fd); err = path + ": not a GGUF file (too short)"; return false; }
    size = (size_t) st.st_size;
    void * m = mmap(nullptr, size, PROT_READ, MAP_PRIVATE, fd, 0);
    ::close(fd);
    if (m == MAP_FAILED) { err = "mmap failed for " + path; return false; }
    base = (const uint8_t *) m;

    Cursor c{base, size};
    if (memcmp(base, "GGUF", 4) != 0) { err = path + ": bad magic"; return false; }
    c.pos = 4;
    version = c.get<uint32_t>();
    if (version < 2 || version > 3) { err = path + ": unsupported GGUF version " + std::to_string(version); return false; }
    const uint64_t n_tensors = c.get<uint64_t>(), n_kv = c.get<uint64_t>();
    // every key/value pair takes at least 13 bytes and every tensor info at least 24
    if (!c.ok || n_kv > size / 13 || n_tensors > size / 24) { err = path + ": implausible header counts"; return false; }

    for (uint64_t i = 0; i < n_kv; ++i) {
        std::string key = c.str();
        GgufValue v;
        v.type = c.get<uint32_t>();
        if (!c.ok || v.type >= G_COUNT) { err = path + ": bad key/value pair " + std::to_string(i); return false; }
        if (v.type == G_STR) {
            v.str = c.str();
        } else if (v.type == G_ARR) {
            v.elem_type = c.get<uint32_t>();
            v.count = c.get<uint64_t>();
            if (!c.ok || v.elem_type >= G_COUNT || v.elem_type == G_ARR) { err = path + ": bad array for key " + key; return false; }
            if (v.elem_type == G_STR) {
                for (uint64_t e = 0; e < v.count && c.ok; ++e) { const uint64_t n = c.get<uint64_t>(); c.skip(n); }
            } else {
                const size_t es = scalar_size(v.elem_type);
                if (v.count > (size - c.pos) / es) c.ok = false; else c.skip(v.count * es);
            }
        } else if (!read_scalar(c, v.type, v)) {
            c.ok = false;
        }
        if (!c.ok) { err = path + ": truncated in the metadata (key " + key + ")"; return false; }
        if (kv.count(key)) { err = path + ": duplicate key " + key; return false; }
        keys.push_back(key);
        kv[key] = v;
    }
    {
        uint32_t a = 0;
        if (get_u32("general.alignment", a)) alignment = a;
        if (alignment == 0 || (alignment & (alignment - 1))) { err = path + ": general.alignment is not a power of two"; return false; }
    }

    tensors.reserve((size_t) n_tensors);
    for (uint64_t i = 0; i < n_tensors; ++i) {
        GgufTensor t;
        t.name = c.str();
        t.n_dims = c.get<uint32_t>();
        if (!c.ok || t.n_dims > 4) { err = path + ": bad tensor info " + std::to_string(i); return false; }
        for (uint32_t d = 0; d < t.n_dims; ++d) t.ne[d] = (int64_t) c.get<uint64_t>();
        t.type = (int32_t) c.get<uint32_t>();
        t.offset = c.get<uint64_t>();
        if (!c.ok) { err = path + ": truncated in the tensor infos"; return false; }
        const int64_t blck = t_blck(t.type);
        if (blck <= 0) { err = path + ": tensor " + t.name + " has unknown type " + std::to_string(t.type); return false; }
        int64_t rows = 1;
        for (int d = 0; d < 4; ++d) {
            if (t.ne[d] < 0 || (d > 0 && t.ne[d] > 0 && rows > INT64_MAX / t.ne[d])) { err = path + ": tensor " + t.name + " has a bad shape"; return false; }
            if (d > 0) rows *= t.ne[d];
        }
        if (t.ne[0] % blck) { err = path + ": row length of " + t.name + " is not a multiple of its block size"; return false; }
        const size_t row_size = t_row_size(t.type, t.ne[0]);
        if (row_size && (size_t) rows > SIZE_MAX / row_size) { err = path + ": tensor " + t.name + " is larger than the address space"; return false; }
        t.nbytes = row_size * (size_t) rows;
        if (t.offset % alignment) { err = path + ": tensor " + t.name + " is not aligned"; return false; }
        if (by_name.count(t.name)) { err = path + ": duplicate tensor " + t.name; return false; }
        by_name[t.name] = tensors.size();
        tensors.push_back(t);
    }
    data_offset = (c.pos + alignment - 1) / alignment * alignment;
    for (const GgufTensor & t : tensors) {
        if (data_offset > size || t.offset > size - data_offset || t.nbytes > size - data_offset - t.offset) {
            err = path + ": data of tensor " + t.name + " lies outside the file";
            return false;
        }
    }
    return true;
}

const GgufTensor * GgufFile::find(const std::string & name) const {
    auto it = by_name.find(name);
    return it == by_name.end() ? nullptr : &tensors[it->second];
}
bool GgufFile::get_u32(const std::string & key, uint32_t & v) const {
    auto it = kv.find(key);
    if (it == kv.end() || it->second.type == G_STR || it->second.type == G_ARR || it->second.type == G_F32 || it->second.type == G_F64) return false;
    if (it->second.inum < 0 || it->second.inum > (int64_t) UINT32_MAX) return false;
    v = (uint32_t) it->second.inum;
    return true;
}
bool GgufFile::get_f32(const std::string & key, float & v) const {
    auto it = kv.find(key);
    if (it == kv.end() || it->second.type == G_STR || it->second.type == G_ARR) return false;
    v = (float) it->second.num;
    return true;
}
bool GgufFile::get_str(const std::string & key, std::string & v) const {
    auto it = kv.find(key);
    if (it == kv.end() || it->second.type != G_STR) return false;
    v = it->second.str;
    return true;
}

}  // namespace b200

// ---- flat C-ABI ----
using b200::GgufFile;
struct b200_gguf { GgufFile f; };
static thread_local std::string g_gguf_error;

extern "C" {
#define API __attribute__((visibility("default")))

API const char * b200_gguf_error(void) { return g_gguf_error.c_str(); }

API b200_gguf * b200_gguf_open(const char * path) {
    b200_gguf * g = new b200_gguf;
    if (!g->f.open(path, g_gguf_error)) { delete g; return nullptr; }
    return g;
}
API void b200_gguf_close(b200_gguf * g) { delete g; }
API uint32_t b200_gguf_version(const b200_gguf * g) { return g->f.version; }
API uint32_t b200_gguf_alignment(const b200_gguf * g) { return g->f.alignment; }
API uint64_t b200_gguf_data_offset(const b200_gguf * g) { return g->f.data_offset; }
API int64_t  b200_gguf_n_kv(const b200_gguf * g) { return (int64_t) g->f.keys.size(); }
API int64_t  b200_gguf_n_tensors(const b200_gguf * g) { return (int64_t) g->f.tensors.size(); }

API int32_t b200_gguf_key(const b200_gguf * g, int64_t i, char * key, size_t cap, uint32_t * type, uint32_t * elem_type, uint64_t * count) {
    if (i < 0 || (size_t) i >= g->f.keys.size()) return -1;
    const std::string & k = g->f.keys[(size_t) i];
    const b200::GgufValue & v = g->f.kv.at(k);
    if (key && cap) snprintf(key, cap, "%s", k.c_str());
    if (type) *type = v.type;
    if (elem_type) *elem_type = v.elem_type;
    if (count) *count = v.count;
    return 0;
}
API int32_t b200_gguf_get_u32(const b200_gguf * g, const char * key, uint32_t * v) { return g->f.get_u32(key, *v) ? 0 : -1; }
API int32_t b200_gguf_get_f32(const b200_gguf * g, const char * key, float * v) { return g->f.get_f32(key, *v) ? 0 : -1; }
API int32_t b200_gguf_get_str(const b200_gguf * g, const char * key, char * v, size_t cap) {
    std::string s;
    if (!g->f.get_str(key, s)) return -1;
    if (v && cap) snprintf(v, cap, "%s", s.c_str());
    return 0;
}
API int32_t b200_gguf_tensor_info(const b200_gguf * g, int64_t i, char * name, size_t cap, int32_t * type, int32_t * n_dims,
                                  int64_t * ne, uint64_t * offset, size_t * nbytes) {
    if (i < 0 || (size_t) i >= g->f.tensors.size()) return -1;
    const b200::GgufTensor & t = g->f.tensors[(size_t) i];
    if (name && cap) snprintf(name, cap, "%s", t.name.c_str());
    if (type) *type = t.type;
    if (n_dims) *n_dims = (int32_t) t.n_dims;
    if (ne) for (int d = 0; d < 4; ++d) ne[d] = t.ne[d];
    if (offset) *offset = t.offset;
    if (nbytes) *nbytes = t.nbytes;
    return 0;
}
API int64_t b200_gguf_find_tensor(const b200_gguf * g, const char * name) {
    auto it = g->f.by_name.find(name);
    return it == g->f.by_name.end() ? -1 : (int64_t) it->second;
}
/* host address of tensor i's bytes inside the read-only mapping (valid until b200_gguf_close) */
API const void * b200_gguf_tensor_data(const b200_gguf * g, int64_t i) {
    if (i < 0 || (size_t) i >= g->f.tensors.size()) return nullptr;
    return g->f.data(g->f.tensors[(size_t) i]);
}

}  // extern "C"
