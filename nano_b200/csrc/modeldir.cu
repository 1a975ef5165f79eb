// modeldir.cu -- config.json / model.safetensors reader (host code only; see modeldir.h)
#include "modeldir.h"

#include <fcntl.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

namespace nb {

namespace {

struct Parser {
    const char *s; size_t n, i = 0; std::string err; int depth = 0;
    bool bad(const char *what) { char b[96]; snprintf(b, sizeof b, "%s at byte %zu", what, i); err = b; return false; }
    void ws() { while (i < n && (s[i] == ' ' || s[i] == '\t' || s[i] == '\n' || s[i] == '\r')) i++; }
    bool lit(const char *w) { size_t l = strlen(w); if (i + l <= n && memcmp(s + i, w, l) == 0) { i += l; return true; } return false; }
    bool string(std::string *out) {
        if (i >= n || s[i] != '"') return bad("expected a string");
        i++;
        while (i < n && s[i] != '"') {
            char c = s[i++];
            if (c == '\\') {
                if (i >= n) return bad("unterminated escape");
                char e = s[i++];
                switch (e) {
                    case 'n': out->push_back('\n'); break; case 't': out->push_back('\t'); break; case 'r': out->push_back('\r'); break;
                    case 'b': out->push_back('\b'); break; case 'f': out->push_back('\f'); break;
                    case 'u': {
                        if (i + 4 > n) return bad("short \\u escape");
                        unsigned v = (unsigned)strtoul(std::string(s + i, 4).c_str(), nullptr, 16); i += 4;
                        if (v < 0x80) out->push_back((char)v);
                        else if (v < 0x800) { out->push_back((char)(0xC0 | (v >> 6))); out->push_back((char)(0x80 | (v & 0x3F))); }
                        else { out->push_back((char)(0xE0 | (v >> 12))); out->push_back((char)(0x80 | ((v >> 6) & 0x3F))); out->push_back((char)(0x80 | (v & 0x3F))); }
                        break;
                    }
                    default: out->push_back(e);
                }
            } else out->push_back(c);
        }
        if (i >= n) return bad("unterminated string");
        i++;
        return true;
    }
    bool value(Json *v) {
        if (++depth > 64) return bad("nesting too deep");
        ws();
        if (i >= n) return bad("unexpected end");
        bool ok = true;
        const char c = s[i];
        if (c == '{') {
            i++; v->t = Json::Obj; ws();
            if (i < n && s[i] == '}') i++;
            else for (;;) {
                ws();
                std::string k; if (!string(&k)) return false;
                ws(); if (i >= n || s[i] != ':') return bad("expected ':'");
                i++;
                Json child; if (!value(&child)) return false;
                v->obj.emplace_back(std::move(k), std::move(child));
                ws();
                if (i < n && s[i] == ',') { i++; continue; }
                if (i < n && s[i] == '}') { i++; break; }
                return bad("expected ',' or '}'");
            }
        } else if (c == '[') {
            i++; v->t = Json::Arr; ws();
            if (i < n && s[i] == ']') i++;
            else for (;;) {
                Json child; if (!value(&child)) return false;
                v->arr.push_back(std::move(child));
                ws();
                if (i < n && s[i] == ',') { i++; continue; }
                if (i < n && s[i] == ']') { i++; break; }
                return bad("expected ',' or ']'");
            }
        } else if (c == '"') { v->t = Json::Str; ok = string(&v->str); }
        else if (lit("true")) { v->t = Json::Bool; v->b = true; }
        else if (lit("false")) { v->t = Json::Bool; v->b = false; }
        else if (lit("null")) { v->t = Json::Null; }
        else {
            char *end = nullptr;
            std::string tmp(s + i, n - i < 64 ? n - i : 64);
            const double d = strtod(tmp.c_str(), &end);
            if (end == tmp.c_str()) return bad("unexpected character");
            i += (size_t)(end - tmp.c_str());
            v->t = Json::Num; v->num = d;
        }
        depth--;
        return ok;
    }
};

bool read_file(const std::string &p, std::string *out) {
    FILE *f = fopen(p.c_str(), "rb");
    if (!f) return false;
    char buf[65536]; size_t k;
    while ((k = fread(buf, 1, sizeof buf, f)) > 0) out->append(buf, k);
    fclose(f);
    return true;
}

}  // namespace

bool json_parse(const char *s, size_t n, Json *out, std::string *err) {
    Parser p{s, n};
    if (!p.value(out)) { if (err) *err = p.err; return false; }
    p.ws();
    if (p.i != n) { if (err) *err = "trailing bytes after the JSON value"; return false; }
    return true;
}

ModelDir::~ModelDir() { if (map) munmap(map, map_bytes); }

int modeldir_open(const char *path, ModelDir *out, std::string *err) {
    out->path = path;
    std::string txt, perr;
    if (!read_file(out->path + "/config.json", &txt)) { *err = "cannot read " + out->path + "/config.json"; return -1; }
    if (!json_parse(txt.data(), txt.size(), &out->config, &perr)) { *err = "config.json: " + perr; return -1; }
    const std::string sp = out->path + "/model.safetensors";
    const int fd = open(sp.c_str(), O_RDONLY);
    if (fd < 0) { *err = "cannot open " + sp; return -1; }
    struct stat st;
    if (fstat(fd, &st) != 0 || st.st_size < 8) { close(fd); *err = sp + ": too short"; return -1; }
    void *m = mmap(nullptr, (size_t)st.st_size, PROT_READ, MAP_PRIVATE, fd, 0);
    close(fd);
    if (m == MAP_FAILED) { *err = "mmap of " + sp + " failed"; return -1; }
    out->map = m; out->map_bytes = (size_t)st.st_size;
    const uint8_t *b = static_cast<const uint8_t *>(m);
    uint64_t hl = 0; memcpy(&hl, b, 8);
    if (hl > out->map_bytes - 8) { *err = sp + ": header length beyond the file"; return -1; }
    Json hdr;
    if (!json_parse(reinterpret_cast<const char *>(b + 8), (size_t)hl, &hdr, &perr) || hdr.t != Json::Obj) { *err = sp + ": header: " + perr; return -1; }
    const uint8_t *data = b + 8 + hl;
    const uint64_t data_bytes = out->map_bytes - 8 - hl;
    for (const auto &kv : hdr.obj) {
        if (kv.first == "__metadata__") continue;
        const Json *dt = kv.second.get("dtype"), *sh = kv.second.get("shape"), *off = kv.second.get("data_offsets");
        if (!dt || dt->t != Json::Str || !sh || sh->t != Json::Arr || !off || off->t != Json::Arr || off->arr.size() != 2) { *err = sp + ": bad entry " + kv.first; return -1; }
        StTensor t;
        t.dtype = dt->str;
        for (const Json &d : sh->arr) t.shape.push_back((uint64_t)d.num);
        const uint64_t lo = (uint64_t)off->arr[0].num, hi = (uint64_t)off->arr[1].num;
        if (lo > hi || hi > data_bytes) { *err = sp + ": offsets of " + kv.first + " beyond the file"; return -1; }
        t.data = data + lo; t.bytes = hi - lo;
        const uint64_t esz = (t.dtype == "BF16" || t.dtype == "F16") ? 2 : (t.dtype == "F64" || t.dtype == "I64") ? 8 : (t.dtype == "I8" || t.dtype == "U8") ? 1 : 4;
        if (t.count() * esz != t.bytes) { *err = sp + ": size of " + kv.first + " does not fit its shape"; return -1; }
        out->tensors.emplace(kv.first, std::move(t));
    }
    return 0;
}

}  // namespace nb
