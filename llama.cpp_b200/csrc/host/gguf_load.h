// Reader of GGUF model files (the reference's on-disk format: ggml/include/gguf.h:1-46 for the layout,
// :53-68 for the value types; reader ggml/src/gguf.cpp:288-640).  The file is mapped read-only; metadata
// scalars and strings are kept, arrays are measured and skipped (their element type and count are kept),
// tensor infos give name, shape, ggml_type and the offset into the aligned data section.
#pragma once

#include <cstddef>
#include <cstdint>
#include <map>
#include <string>
#include <vector>

namespace b200 {

struct GgufValue {
    uint32_t type = 0;            // gguf_type of the key (9 = array)
    uint32_t elem_type = 0;       // arrays: type of the elements
    uint64_t count = 0;           // arrays: number of elements
    double   num = 0;             // integer / float / bool values
    int64_t  inum = 0;            // integer values, exact
    std::string str;              // string values
};

struct GgufTensor {
    std::string name;
    uint32_t n_dims = 0;
    int64_t  ne[4] = {1, 1, 1, 1};
    int32_t  type = 0;            // ggml_type
    uint64_t offset = 0;          // relative to the data section
    size_t   nbytes = 0;
};

struct GgufFile {
    std::string path;
    const uint8_t * base = nullptr;   // the mapping
    size_t   size = 0;
    uint32_t version = 0;
    uint32_t alignment = 32;
    size_t   data_offset = 0;         // start of the data section in the file
    std::vector<std::string> keys;    // in file order
    std::map<std::string, GgufValue> kv;
    std::vector<GgufTensor> tensors;
    std::map<std::string, size_t> by_name;

    ~GgufFile();
    // returns false and sets err on a malformed, truncated or unsupported file
    bool open(const char * path, std::string & err);
    const GgufTensor * find(const std::string & name) const;
    const uint8_t * data(const GgufTensor & t) const { return base + data_offset + t.offset; }
    bool get_u32(const std::string & key, uint32_t & v) const;
    bool get_f32(const std::string & key, float & v) const;
    bool get_str(const std::string & key, std::string & v) const;
};

}  // namespace b200
