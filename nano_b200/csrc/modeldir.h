// modeldir.h -- reader of a model folder: config.json (a small JSON value tree) and model.safetensors (8-byte little-endian header
// length, a JSON directory name -> {dtype, shape, data_offsets}, then the tensor bytes; the file is memory-mapped).
#pragma once
#include <stdint.h>

#include <map>
#include <string>
#include <utility>
#include <vector>

namespace nb {

struct Json {
    enum Type { Null, Bool, Num, Str, Arr, Obj } t = Null;
    double num = 0.0;
    bool b = false;
    std::string str;
    std::vector<Json> arr;
    std::vector<std::pair<std::string, Json>> obj;

    const Json *get(const char *key) const {        // member of an object, nullptr when absent (or when this is no object)
        if (t != Obj) return nullptr;
        for (const auto &kv : obj) if (kv.first == key) return &kv.second;
        return nullptr;
    }
    bool present(const char *key) const { const Json *j = get(key); return j && j->t != Null; }
    bool number(const char *key, double *v) const { const Json *j = get(key); if (!j || j->t != Num) return false; *v = j->num; return true; }
};

// parses one JSON document; returns false and a message with the byte offset on malformed input
bool json_parse(const char *s, size_t n, Json *out, std::string *err);

struct StTensor {
    std::string dtype;               // "BF16", "F32", "I32", ...
    std::vector<uint64_t> shape;
    const uint8_t *data = nullptr;   // into the mapping
    uint64_t bytes = 0;
    uint64_t count() const { uint64_t c = 1; for (uint64_t s : shape) c *= s; return c; }
};

struct ModelDir {
    std::string path;
    Json config;
    std::map<std::string, StTensor> tensors;
    void *map = nullptr; size_t map_bytes = 0;
    ~ModelDir();
    ModelDir() = default;
    ModelDir(const ModelDir &) = delete;
    ModelDir &operator=(const ModelDir &) = delete;
};

// 0 on success; otherwise a message in *err
int modeldir_open(const char *path, ModelDir *out, std::string *err);

}  // namespace nb
