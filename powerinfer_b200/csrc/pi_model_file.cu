// Host-only reader for the reference's files: PowerInfer model files and GPU-index (placement) files.
//
// Both are GGUF v2 / v3 containers whose magic is PWRI instead of GGUF (ggml.h:247, ggml.c:19481-19495): a header
// {magic u32, version u32, n_tensors u64, n_kv u64}, the key / value table (ggml.c:19497-19600), the tensor directory
// {name, n_dims u32, ne[n_dims] u64, type u32, offset u64} (ggml.c:19603-19640) and, from the next multiple of
// general.alignment (default 32), the tensor data.  Nothing here touches a device; every read is bounds-checked, so a
// truncated or corrupt file gives an error status instead of a fault.
#include "pi_common.cuh"

#include <cstring>
#include <fcntl.h>
#include <string>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>
#include <unordered_map>
#include <vector>

namespace pi {
namespace {

enum : uint32_t { T_U8 = 0, T_I8, T_U16, T_I16, T_U32, T_I32, T_F32, T_BOOL, T_STR, T_ARR, T_U64, T_I64, T_F64 };
static const size_t SCALAR_SIZE[13] = {1, 1, 2, 2, 4, 4, 4, 1, 0, 0, 8, 8, 8};

struct Value { uint32_t type; size_t pos; size_t len; };              // pos: offset of the value (string: of its bytes)
struct Tensor { std::string name; int type; int64_t ne[4]; size_t offset; size_t nbytes; };

// bytes of a tensor of a type this reader knows (enum ggml_type, ggml.h:307-333); 0 for other types; SIZE_MAX when the
// element count or the byte count does not fit 64 bits (four extents of up to 2^40 each can wrap the product, and a wrapped
// size would pass the end-of-file check while the extents still advertise a huge tensor)
size_t tensor_bytes(int type, const int64_t ne[4]) {
    uint64_t n = 1;
    for (int k = 0; k < 4; k++)
        if (__builtin_mul_overflow(n, (uint64_t)ne[k], &n)) return SIZE_MAX;
    if (n > (UINT64_MAX >> 3)) return SIZE_MAX;                       // n * 4 below must not wrap either
    switch (type) {
        case 0:  return n * 4;                                        // F32
        case 1:  return n * 2;                                        // F16
        case 2:  return ne[0] % 32 == 0 ? n / 32 * 18 : 0;            // Q4_0
        case 16: return n;                                            // I8
        case 17: return n * 2;                                        // I16
        case 18: return n * 4;                                        // I32
        default: return 0;
    }
}

}  // namespace
}  // namespace pi

struct pi_model_file {
    const unsigned char * base = nullptr;
    size_t size = 0;
    bool powerinfer = false;
    size_t data_start = 0;
    std::unordered_map<std::string, pi::Value> kv;
    std::vector<pi::Tensor> tensors;
    std::unordered_map<std::string, size_t> by_name;
};

namespace pi {
namespace {

struct Cursor {
    const unsigned char * base; size_t size; size_t pos; bool ok;
    bool need(size_t n) { if (!ok || n > size || pos > size - n) { ok = false; return false; } return true; }
    template <typename T> T take() { T v{}; if (need(sizeof(T))) { memcpy(&v, base + pos, sizeof(T)); pos += sizeof(T); } return v; }
    bool string(size_t * at, size_t * len) {
        const uint64_t n = take<uint64_t>();
        if (!need((size_t)n)) return false;
        *at = pos; *len = (size_t)n; pos += (size_t)n;
        return true;
    }
    // skips a value of `type`; records where it is
    bool value(uint32_t type, Value * out, int depth) {
        out->type = type; out->pos = pos; out->len = 0;
        if (type == T_STR) return string(&out->pos, &out->len);
        if (type == T_ARR) {
            if (depth > 0) { ok = false; return false; }               // the format has no nested arrays
            const uint32_t et = take<uint32_t>();
            const uint64_t n = take<uint64_t>();
            out->len = (size_t)n;
            if (et > T_F64 || et == T_ARR) { ok = false; return false; }
            if (et == T_STR) {
                for (uint64_t i = 0; i < n && ok; i++) { size_t a, l; string(&a, &l); }
                return ok;
            }
            const size_t es = SCALAR_SIZE[et];
            if (n > (uint64_t)(size / (es ? es : 1))) { ok = false; return false; }
            if (!need((size_t)n * es)) return false;
            pos += (size_t)n * es;
            return true;
        }
        if (type > T_F64) { ok = false; return false; }
        if (!need(SCALAR_SIZE[type])) return false;
        pos += SCALAR_SIZE[type];
        return true;
    }
};

int parse(pi_model_file * f) {
    Cursor c{f->base, f->size, 0, true};
    if (!c.need(24)) { set_error("model_file: shorter than a GGUF header"); return PI_ERR_INVALID; }
    const bool pwri = memcmp(f->base, "PWRI", 4) == 0;
    if (!pwri && memcmp(f->base, "GGUF", 4) != 0) { set_error("model_file: magic is neither PWRI nor GGUF"); return PI_ERR_INVALID; }
    f->powerinfer = pwri;
    c.pos = 4;
    const uint32_t version = c.take<uint32_t>();
    if (version != 2 && version != 3) { set_error("model_file: GGUF version %u is not supported (2 and 3 are)", version); return PI_ERR_INVALID; }
    const uint64_t n_tensors = c.take<uint64_t>(), n_kv = c.take<uint64_t>();
    if (n_tensors > f->size / 24 || n_kv > f->size / 12) { set_error("model_file: implausible header counts"); return PI_ERR_INVALID; }
    for (uint64_t i = 0; i < n_kv; i++) {
        size_t at, len;
        if (!c.string(&at, &len)) break;
        std::string key((const char *)f->base + at, len);
        const uint32_t type = c.take<uint32_t>();
        Value v;
        if (!c.value(type, &v, 0)) break;
        f->kv.emplace(std::move(key), v);
    }
    if (!c.ok) { set_error("model_file: truncated or malformed key / value table"); return PI_ERR_INVALID; }
    f->tensors.reserve((size_t)n_tensors);
    for (uint64_t i = 0; i < n_tensors; i++) {
        size_t at, len;
        if (!c.string(&at, &len)) break;
        Tensor t;
        t.name.assign((const char *)f->base + at, len);
        const uint32_t nd = c.take<uint32_t>();
        if (nd > 4) { c.ok = false; break; }
        for (int k = 0; k < 4; k++) t.ne[k] = 1;
        for (uint32_t k = 0; k < nd; k++) {
            const uint64_t e = c.take<uint64_t>();
            if (e > ((uint64_t)1 << 40)) { c.ok = false; break; }
            t.ne[k] = (int64_t)e;
        }
        t.type = (int)c.take<uint32_t>();
        t.offset = (size_t)c.take<uint64_t>();
        t.nbytes = tensor_bytes(t.type, t.ne);
        if (t.nbytes == SIZE_MAX) c.ok = false;
        if (!c.ok) break;
        f->by_name.emplace(t.name, f->tensors.size());
        f->tensors.push_back(std::move(t));
    }
    if (!c.ok) { set_error("model_file: truncated or malformed tensor directory"); return PI_ERR_INVALID; }
    uint64_t align = 32;
    { auto it = f->kv.find("general.alignment"); if (it != f->kv.end() && it->second.type == T_U32) { uint32_t a; memcpy(&a, f->base + it->second.pos, 4); if (a) align = a; } }
    f->data_start = (c.pos + align - 1) / align * align;
    for (const Tensor & t : f->tensors) {
        if (f->data_start > f->size || t.offset > f->size - f->data_start || t.nbytes > f->size - f->data_start - t.offset) {
            set_error("model_file: tensor %s reaches beyond the end of the file", t.name.c_str());
            return PI_ERR_INVALID;
        }
    }
    return PI_OK;
}

const Value * find(const pi_model_file * f, const char * key) {
    if (!f || !key) return nullptr;
    auto it = f->kv.find(key);
    return it == f->kv.end() ? nullptr : &it->second;
}

}  // namespace
}  // namespace pi

using namespace pi;

extern "C" {
#pragma GCC visibility push(default)

int pi_model_file_open(const char * path, pi_model_file ** out) {
    PI_REQUIRE(path && out, "model_file_open: null argument");
    *out = nullptr;
    const int fd = open(path, O_RDONLY);
    if (fd < 0) { set_error("model_file_open: cannot open %s", path); return PI_ERR_INVALID; }
    struct stat st;
    if (fstat(fd, &st) != 0 || st.st_size <= 0) { close(fd); set_error("model_file_open: cannot stat %s (or it is empty)", path); return PI_ERR_INVALID; }
    void * m = mmap(nullptr, (size_t)st.st_size, PROT_READ, MAP_PRIVATE, fd, 0);
    close(fd);
    if (m == MAP_FAILED) { set_error("model_file_open: cannot map %s", path); return PI_ERR_INVALID; }
    pi_model_file * f = new (std::nothrow) pi_model_file();
    if (!f) { munmap(m, (size_t)st.st_size); set_error("model_file_open: out of host memory"); return PI_ERR_INVALID; }
    f->base = (const unsigned char *)m; f->size = (size_t)st.st_size;
    const int rc = parse(f);
    if (rc != PI_OK) { pi_model_file_close(f); return rc; }
    *out = f;
    return PI_OK;
}

void pi_model_file_close(pi_model_file * f) {
    if (!f) return;
    if (f->base) munmap((void *)f->base, f->size);
    delete f;
}

int pi_model_file_is_powerinfer(const pi_model_file * f) { return f && f->powerinfer ? 1 : 0; }

int pi_model_file_get_u64(const pi_model_file * f, const char * key, uint64_t * value) {
    PI_REQUIRE(f && key && value, "model_file_get_u64: null argument");
    const Value * v = find(f, key);
    PI_REQUIRE(v, "model_file: no key %s", key);
    const unsigned char * p = f->base + v->pos;
    int64_t s = 0;
    switch (v->type) {
        case T_U8: case T_BOOL: *value = *p; return PI_OK;
        case T_U16: { uint16_t x; memcpy(&x, p, 2); *value = x; return PI_OK; }
        case T_U32: { uint32_t x; memcpy(&x, p, 4); *value = x; return PI_OK; }
        case T_U64: { uint64_t x; memcpy(&x, p, 8); *value = x; return PI_OK; }
        case T_I8:  s = (int8_t)*p; break;
        case T_I16: { int16_t x; memcpy(&x, p, 2); s = x; break; }
        case T_I32: { int32_t x; memcpy(&x, p, 4); s = x; break; }
        case T_I64: { int64_t x; memcpy(&x, p, 8); s = x; break; }
        default: set_error("model_file: key %s is not an integer", key); return PI_ERR_INVALID;
    }
    PI_REQUIRE(s >= 0, "model_file: key %s is negative", key);
    *value = (uint64_t)s;
    return PI_OK;
}

int pi_model_file_get_f32(const pi_model_file * f, const char * key, float * value) {
    PI_REQUIRE(f && key && value, "model_file_get_f32: null argument");
    const Value * v = find(f, key);
    PI_REQUIRE(v, "model_file: no key %s", key);
    if (v->type == T_F32) { memcpy(value, f->base + v->pos, 4); return PI_OK; }
    if (v->type == T_F64) { double d; memcpy(&d, f->base + v->pos, 8); *value = (float)d; return PI_OK; }
    set_error("model_file: key %s is not a float", key);
    return PI_ERR_INVALID;
}

int pi_model_file_get_str(const pi_model_file * f, const char * key, const char ** str, size_t * len) {
    PI_REQUIRE(f && key && str && len, "model_file_get_str: null argument");
    const Value * v = find(f, key);
    PI_REQUIRE(v && v->type == T_STR, "model_file: no string key %s", key);
    *str = (const char *)f->base + v->pos; *len = v->len;
    return PI_OK;
}

int64_t pi_model_file_n_tensors(const pi_model_file * f) { return f ? (int64_t)f->tensors.size() : 0; }

int pi_model_file_tensor_at(const pi_model_file * f, int64_t i, const char ** name, int * ggml_type, int64_t ne[4],
                            const void ** data, size_t * nbytes) {
    PI_REQUIRE(f && i >= 0 && (size_t)i < f->tensors.size(), "model_file_tensor_at: index out of range");
    const Tensor & t = f->tensors[(size_t)i];
    if (name) *name = t.name.c_str();
    if (ggml_type) *ggml_type = t.type;
    if (ne) for (int k = 0; k < 4; k++) ne[k] = t.ne[k];
    if (data) *data = t.nbytes ? f->base + f->data_start + t.offset : nullptr;
    if (nbytes) *nbytes = t.nbytes;
    return PI_OK;
}

int pi_model_file_tensor(const pi_model_file * f, const char * name, int * ggml_type, int64_t ne[4],
                         const void ** data, size_t * nbytes) {
    PI_REQUIRE(f && name, "model_file_tensor: null argument");
    auto it = f->by_name.find(name);
    PI_REQUIRE(it != f->by_name.end(), "model_file: no tensor %s", name);
    return pi_model_file_tensor_at(f, (int64_t)it->second, nullptr, ggml_type, ne, data, nbytes);
}

int pi_model_file_engine_config(const pi_model_file * f, pi_engine_config * cfg) {
    PI_REQUIRE(f && cfg, "model_file_engine_config: null argument");
    const char * a; size_t alen;
    int rc = pi_model_file_get_str(f, "general.architecture", &a, &alen);
    if (rc) return rc;
    const std::string arch(a, alen);
    memset(cfg, 0, sizeof *cfg);
    if (arch == "llama") cfg->arch = PI_ARCH_LLAMA;
    else if (arch == "bamboo") cfg->arch = PI_ARCH_BAMBOO;
    else if (arch == "falcon") cfg->arch = PI_ARCH_FALCON;
    else if (arch == "opt") cfg->arch = PI_ARCH_OPT;
    else { set_error("model_file: architecture %s is not one of llama / bamboo / falcon / opt", arch.c_str()); return PI_ERR_INVALID; }
    int type; int64_t ne[4];
    for (const char * need : {"blk.0.ffn_down_t.weight", "blk.0.fc1.weight", "blk.0.fc2.weight", "blk.0.ffn_up.weight", "token_embd.weight"}) {
        if (pi_model_file_tensor(f, need, &type, ne, nullptr, nullptr) != PI_OK) {
            set_error("model_file: %s is missing: not a PowerInfer (sparse) model file", need);
            return PI_ERR_INVALID;
        }
    }
    pi_model_file_tensor(f, "blk.0.ffn_up.weight", &type, ne, nullptr, nullptr);
    PI_REQUIRE(type == 1 || type == 2, "model_file: blk.0.ffn_up.weight has ggml type %d; F16 and Q4_0 are on the decode path", type);
    cfg->wtype = type == 2 ? PI_TYPE_Q4_0 : PI_TYPE_F16;
    pi_model_file_tensor(f, "blk.0.fc1.weight", &type, ne, nullptr, nullptr);
    cfg->rank = (int)ne[1];
    pi_model_file_tensor(f, "token_embd.weight", &type, ne, nullptr, nullptr);
    cfg->n_vocab = (int)ne[1];
    auto u = [&](const char * suffix, uint64_t fallback, bool required, int * dst) -> int {
        uint64_t v = fallback;
        const std::string key = arch + "." + suffix;
        if (find(f, key.c_str())) { const int r = pi_model_file_get_u64(f, key.c_str(), &v); if (r) return r; }
        else if (required) { set_error("model_file: no key %s", key.c_str()); return PI_ERR_INVALID; }
        *dst = (int)v;
        return PI_OK;
    };
    if ((rc = u("embedding_length", 0, true, &cfg->d))) return rc;
    if ((rc = u("block_count", 0, true, &cfg->n_layer))) return rc;
    if ((rc = u("feed_forward_length", 0, true, &cfg->n_ff))) return rc;
    if ((rc = u("attention.head_count", 0, true, &cfg->n_head))) return rc;
    if ((rc = u("attention.head_count_kv", (uint64_t)cfg->n_head, false, &cfg->n_head_kv))) return rc;
    if ((rc = u("context_length", 512, false, &cfg->n_ctx))) return rc;
    const bool rms = cfg->arch == PI_ARCH_LLAMA || cfg->arch == PI_ARCH_BAMBOO;
    const std::string eps_key = arch + (rms ? ".attention.layer_norm_rms_epsilon" : ".attention.layer_norm_epsilon");
    cfg->norm_eps = cfg->arch == PI_ARCH_OPT ? 0.0f : 1e-5f;
    if (find(f, eps_key.c_str()) && (rc = pi_model_file_get_f32(f, eps_key.c_str(), &cfg->norm_eps))) return rc;
    cfg->rope_base = 10000.0f;
    const std::string rope_key = arch + ".rope.freq_base";
    if (find(f, rope_key.c_str()) && (rc = pi_model_file_get_f32(f, rope_key.c_str(), &cfg->rope_base))) return rc;
    cfg->threshold = 0.0f;
    if (find(f, "powerinfer.sparse_threshold") && (rc = pi_model_file_get_f32(f, "powerinfer.sparse_threshold", &cfg->threshold))) return rc;
    cfg->n_pos = 0;
    if (cfg->arch == PI_ARCH_OPT && pi_model_file_tensor(f, "position_embd.weight", &type, ne, nullptr, nullptr) == PI_OK) cfg->n_pos = (int)ne[1];
    cfg->max_batch = 1; cfg->n_ranks = 1; cfg->rank_id = 0;
    return PI_OK;
}

#pragma GCC visibility pop
}
