// GGUF reader and model loader on the C ABI: what crates/gguf (reader.rs, value.rs, types.rs) and
// ModelConfig::from_gguf (crates/core/src/config.rs:107-264) do for the reference's CudaModel::load_with
// (crates/core/src/cuda/load.rs:166-417).  Host code only; no CUDA call happens before tfr_load_gguf.
//
// Semantics kept from the reference reader: little-endian; magic "GGUF"; versions 2 and 3; at most
// 1e6 tensors / metadata pairs; at most 4 dims; tensor types must be known; the data section starts
// at the header's end rounded up to general.alignment (default 32); every tensor's byte range must
// lie inside the file.  Integer metadata is read leniently (u8/u16/u32/u64 and non-negative i32/i64
// all answer a u64 query; f64 answers an f32 query), as Value::as_u32 / as_u64 / as_f32 do.
#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <map>
#include <string>
#include <vector>

#include "../../include/tarafer_b200.h"

namespace {

struct TypeInfo {
    int id;
    const char* name;
    int block;  // elements per block
    int bytes;  // bytes per block
};
// crates/gguf/src/types.rs:7-160 (ggml type ids, block sizes, block byte sizes)
const TypeInfo kTypes[] = {
    {0, "F32", 1, 4},      {1, "F16", 1, 2},       {2, "Q4_0", 32, 18},     {3, "Q4_1", 32, 20},    {6, "Q5_0", 32, 22},
    {7, "Q5_1", 32, 24},   {8, "Q8_0", 32, 34},    {9, "Q8_1", 32, 36},     {10, "Q2_K", 256, 84},  {11, "Q3_K", 256, 110},
    {12, "Q4_K", 256, 144}, {13, "Q5_K", 256, 176}, {14, "Q6_K", 256, 210}, {15, "Q8_K", 256, 292}, {16, "IQ2_XXS", 256, 66},
    {17, "IQ2_XS", 256, 74}, {18, "IQ3_XXS", 256, 98}, {19, "IQ1_S", 256, 50}, {20, "IQ4_NL", 32, 18}, {21, "IQ3_S", 256, 110},
    {22, "IQ2_S", 256, 82}, {23, "IQ4_XS", 256, 136}, {24, "I8", 1, 1},     {25, "I16", 1, 2},      {26, "I32", 1, 4},
    {27, "I64", 1, 8},     {28, "F64", 1, 8},      {29, "IQ1_M", 256, 56},  {30, "BF16", 1, 2},
};
const TypeInfo* type_info(uint32_t id) {
    for (const TypeInfo& t : kTypes)
        if ((uint32_t)t.id == id) return &t;
    return nullptr;
}

enum ValueKind { V_U8 = 0, V_I8, V_U16, V_I16, V_U32, V_I32, V_F32, V_BOOL, V_STRING, V_ARRAY, V_U64, V_I64, V_F64 };

struct Value {
    int kind = -1;
    uint64_t u = 0;   // unsigned / bool payload
    int64_t i = 0;    // signed payload
    double f = 0.0;   // float payload
    std::string s;    // string payload
    uint64_t count = 0;  // arrays: element count
    int item_kind = -1;
    // array payloads the tokenizer needs (tokenizer/mod.rs:27-106): strings (tokens, merges), floats (scores),
    // integers (token types).  Other item kinds are parsed to stay in step and dropped.
    std::vector<std::string> items_s;
    std::vector<double> items_f;
    std::vector<int64_t> items_i;
};

struct Tensor {
    std::string name;
    int n_dims = 0;
    int64_t dims[4] = {1, 1, 1, 1};
    uint32_t type = 0;
    uint64_t offset = 0, nbytes = 0;
};

struct Cursor {
    const uint8_t* p;
    size_t n, at = 0;
    bool ok = true;
    const char* eof_ctx = nullptr;
    template <class T>
    T get(const char* ctx) {
        T v{};
        if (!ok) return v;
        if (at + sizeof(T) > n) {
            ok = false;
            eof_ctx = ctx;
            return v;
        }
        memcpy(&v, p + at, sizeof(T));
        at += sizeof(T);
        return v;
    }
    const char* malformed = nullptr;  // set with ok = false: a limit of value.rs was exceeded
    uint64_t bad_len = 0;
    std::string str(const char* ctx) {
        const uint64_t len = get<uint64_t>("string length");
        if (!ok) return {};
        if (len > 64ull * 1024 * 1024) {  // value.rs:163-183
            ok = false;
            malformed = "string length %llu is unreasonably large";
            bad_len = len;
            return {};
        }
        if (len > n - at) {
            ok = false;
            eof_ctx = ctx;
            return {};
        }
        std::string s(reinterpret_cast<const char*>(p + at), (size_t)len);
        at += (size_t)len;
        if (!valid_utf8(s)) {  // String::from_utf8 in read_string
            ok = false;
            malformed = "invalid UTF-8 in a string (offset %llu)";
            bad_len = at - len;
        }
        return s;
    }
    static bool valid_utf8(const std::string& s) {
        const unsigned char* b = reinterpret_cast<const unsigned char*>(s.data());
        const size_t m = s.size();
        for (size_t i = 0; i < m;) {
            const unsigned c = b[i];
            int extra;
            unsigned cp;
            if (c < 0x80) { i++; continue; }
            else if ((c & 0xe0) == 0xc0) extra = 1, cp = c & 0x1f;
            else if ((c & 0xf0) == 0xe0) extra = 2, cp = c & 0x0f;
            else if ((c & 0xf8) == 0xf0) extra = 3, cp = c & 0x07;
            else return false;
            if (i + (size_t)extra >= m) return false;  // truncated sequence
            for (int k = 1; k <= extra; k++) {
                if ((b[i + k] & 0xc0) != 0x80) return false;
                cp = (cp << 6) | (b[i + k] & 0x3f);
            }
            if ((extra == 1 && cp < 0x80) || (extra == 2 && cp < 0x800) || (extra == 3 && cp < 0x10000) || cp > 0x10ffff ||
                (cp >= 0xd800 && cp <= 0xdfff))
                return false;
            i += extra + 1;
        }
        return true;
    }
};

}  // namespace

struct tfr_gguf {
    std::string path;
    int fd = -1;
    const uint8_t* map = nullptr;
    size_t size = 0;
    uint32_t version = 0;
    uint64_t data_offset = 0;
    std::map<std::string, Value> meta;
    std::vector<Tensor> tensors;
    std::map<std::string, size_t> index;
};

namespace {

int set_err(char* err, size_t cap, int code, const char* fmt, ...) {
    if (err && cap) {
        va_list ap;
        va_start(ap, fmt);
        vsnprintf(err, cap, fmt, ap);
        va_end(ap);
    }
    return code;
}

bool read_value(Cursor& c, int kind, Value& v, int depth) {
    v.kind = kind;
    switch (kind) {
        case V_U8: v.u = c.get<uint8_t>("value"); break;
        case V_I8: v.i = c.get<int8_t>("value"); break;
        case V_U16: v.u = c.get<uint16_t>("value"); break;
        case V_I16: v.i = c.get<int16_t>("value"); break;
        case V_U32: v.u = c.get<uint32_t>("value"); break;
        case V_I32: v.i = c.get<int32_t>("value"); break;
        case V_F32: v.f = c.get<float>("value"); break;
        case V_BOOL: v.u = c.get<uint8_t>("value") != 0; break;
        case V_STRING: v.s = c.str("string value"); break;
        case V_U64: v.u = c.get<uint64_t>("value"); break;
        case V_I64: v.i = c.get<int64_t>("value"); break;
        case V_F64: v.f = c.get<double>("value"); break;
        case V_ARRAY: {
            const uint32_t item = c.get<uint32_t>("array item type");
            const uint64_t count = c.get<uint64_t>("array length");
            if (!c.ok) return false;
            if (item > V_F64 || depth > 4) return false;
            if (count > 10000000ull) {  // value.rs:246-262
                c.ok = false;
                c.malformed = "array length %llu is unreasonably large";
                c.bad_len = count;
                return false;
            }
            v.item_kind = (int)item;
            v.count = count;
            for (uint64_t k = 0; k < count && c.ok; k++) {
                Value it;
                if (!read_value(c, (int)item, it, depth + 1)) return false;
                if (depth == 0) {
                    if (item == V_STRING) v.items_s.push_back(std::move(it.s));
                    else if (item == V_F32 || item == V_F64) v.items_f.push_back(it.f);
                    else if (item == V_I8 || item == V_I16 || item == V_I32 || item == V_I64) v.items_i.push_back(it.i);
                    else if (item != V_ARRAY) v.items_i.push_back((int64_t)it.u);
                }
            }
            break;
        }
        default: return false;
    }
    return c.ok;
}

const Value* find(const tfr_gguf* g, const char* key) {
    auto it = g->meta.find(key);
    return it == g->meta.end() ? nullptr : &it->second;
}
bool as_u64(const Value* v, uint64_t& out) {  // value.rs: as_u32 / as_u64
    if (!v) return false;
    switch (v->kind) {
        case V_U8: case V_U16: case V_U32: case V_U64: out = v->u; return true;
        case V_I32: case V_I64:
            if (v->i < 0) return false;
            out = (uint64_t)v->i;
            return true;
        default: return false;
    }
}
bool as_f32(const Value* v, float& out) {
    if (!v || (v->kind != V_F32 && v->kind != V_F64)) return false;
    out = (float)v->f;
    return true;
}

}  // namespace

extern "C" int tfr_gguf_open(const char* path, tfr_gguf** out, char* err, size_t err_cap) {
    if (!path || !out) return TFR_E_INVALID;
    *out = nullptr;
    tfr_gguf* g = new tfr_gguf();
    g->path = path;
    g->fd = open(path, O_RDONLY);
    struct stat st {};
    if (g->fd < 0 || fstat(g->fd, &st) != 0) {
        tfr_gguf_close(g);
        return set_err(err, err_cap, TFR_E_INVALID, "cannot open %s", path);
    }
    g->size = (size_t)st.st_size;
    void* m = g->size ? mmap(nullptr, g->size, PROT_READ, MAP_PRIVATE, g->fd, 0) : MAP_FAILED;
    if (m == MAP_FAILED) {
        tfr_gguf_close(g);
        return set_err(err, err_cap, TFR_E_INVALID, "cannot map %s", path);
    }
    g->map = static_cast<const uint8_t*>(m);
    Cursor c{g->map, g->size};
    auto bad = [&](const char* fmt, auto... a) {
        const int rc = set_err(err, err_cap, TFR_E_INVALID, fmt, a...);
        tfr_gguf_close(g);
        return rc;
    };
    auto eof = [&]() {
        if (c.malformed) {
            char fmt[96];
            snprintf(fmt, sizeof fmt, "malformed file: %s", c.malformed);
            return bad(fmt, (unsigned long long)c.bad_len);
        }
        return bad("unexpected end of file in %s", c.eof_ctx);
    };
    const uint32_t magic = c.get<uint32_t>("magic");
    if (!c.ok) return eof();
    if (magic != 0x46554747u) return bad("bad magic 0x%08x (not a GGUF file)", magic);
    g->version = c.get<uint32_t>("version");
    if (!c.ok) return bad("unexpected end of file in %s", c.eof_ctx);
    if (g->version != 2 && g->version != 3) return bad("unsupported GGUF version %u", g->version);
    const uint64_t n_tensors = c.get<uint64_t>("tensor count"), n_kv = c.get<uint64_t>("metadata kv count");
    if (!c.ok) return bad("unexpected end of file in %s", c.eof_ctx);
    if (n_tensors > 1000000 || n_kv > 1000000)
        return bad("unreasonable counts: tensors=%llu kv=%llu", (unsigned long long)n_tensors, (unsigned long long)n_kv);
    for (uint64_t k = 0; k < n_kv; k++) {
        const std::string key = c.str("metadata key");
        const uint32_t ty = c.get<uint32_t>("metadata value type");
        if (!c.ok) return eof();
        if (ty > V_F64) return bad("unknown metadata value type %u", ty);
        Value v;
        if (!read_value(c, (int)ty, v, 0)) return c.ok ? bad("malformed metadata value for key %s", key.c_str()) : eof();
        g->meta[key] = std::move(v);
    }
    g->tensors.reserve((size_t)n_tensors);
    for (uint64_t i = 0; i < n_tensors; i++) {
        Tensor t;
        t.name = c.str("tensor name");
        const uint32_t nd = c.get<uint32_t>("tensor n_dims");
        if (!c.ok) return eof();
        if (nd > 4) return bad("tensor %s: n_dims=%u > 4", t.name.c_str(), nd);
        t.n_dims = (int)nd;
        uint64_t elems = 1;
        for (uint32_t d = 0; d < nd; d++) {
            const uint64_t v = c.get<uint64_t>("tensor dim");
            t.dims[d] = (int64_t)v;
            elems = v && elems > UINT64_MAX / v ? UINT64_MAX : elems * v;
        }
        t.type = c.get<uint32_t>("tensor type");
        t.offset = c.get<uint64_t>("tensor offset");
        if (!c.ok) return eof();
        const TypeInfo* ti = type_info(t.type);
        if (!ti) return bad("unknown tensor type %u (tensor %s)", t.type, t.name.c_str());
        const uint64_t blocks = elems / (uint64_t)ti->block;
        t.nbytes = (elems == UINT64_MAX || blocks > UINT64_MAX / (uint64_t)ti->bytes) ? UINT64_MAX
                                                                                      : blocks * (uint64_t)ti->bytes;  // types.rs: nbytes()
        g->index[t.name] = g->tensors.size();
        g->tensors.push_back(std::move(t));
    }
    uint64_t alignment = 32;
    as_u64(find(g, "general.alignment"), alignment);
    g->data_offset = alignment ? (c.at + alignment - 1) / alignment * alignment : c.at;
    for (const Tensor& t : g->tensors) {
        const uint64_t start = g->data_offset + t.offset < t.offset ? UINT64_MAX : g->data_offset + t.offset;
        const uint64_t end = start + t.nbytes < start ? UINT64_MAX : start + t.nbytes;
        if (end > g->size)
            return bad("tensor %s data [%llu, %llu) exceeds file size %llu", t.name.c_str(), (unsigned long long)start,
                       (unsigned long long)end, (unsigned long long)g->size);
    }
    *out = g;
    return TFR_OK;
}

extern "C" void tfr_gguf_close(tfr_gguf* g) {
    if (!g) return;
    if (g->map) munmap(const_cast<uint8_t*>(g->map), g->size);
    if (g->fd >= 0) close(g->fd);
    delete g;
}

extern "C" int tfr_gguf_version(const tfr_gguf* g) { return g ? (int)g->version : TFR_E_INVALID; }
extern "C" uint64_t tfr_gguf_data_offset(const tfr_gguf* g) { return g ? g->data_offset : 0; }
extern "C" int64_t tfr_gguf_tensor_count(const tfr_gguf* g) { return g ? (int64_t)g->tensors.size() : TFR_E_INVALID; }
extern "C" int64_t tfr_gguf_find_tensor(const tfr_gguf* g, const char* name) {
    if (!g || !name) return -1;
    auto it = g->index.find(name);
    return it == g->index.end() ? -1 : (int64_t)it->second;
}
extern "C" int tfr_gguf_tensor_info(const tfr_gguf* g, int64_t i, const char** name, int* ggml_type, int* n_dims, int64_t dims[4],
                                    uint64_t* offset, uint64_t* nbytes) {
    if (!g || i < 0 || i >= (int64_t)g->tensors.size()) return TFR_E_INVALID;
    const Tensor& t = g->tensors[(size_t)i];
    if (name) *name = t.name.c_str();
    if (ggml_type) *ggml_type = (int)t.type;
    if (n_dims) *n_dims = t.n_dims;
    if (dims)
        for (int d = 0; d < 4; d++) dims[d] = t.dims[d];
    if (offset) *offset = t.offset;
    if (nbytes) *nbytes = t.nbytes;
    return TFR_OK;
}
extern "C" const void* tfr_gguf_tensor_data(const tfr_gguf* g, int64_t i) {
    if (!g || i < 0 || i >= (int64_t)g->tensors.size()) return nullptr;
    return g->map + g->data_offset + g->tensors[(size_t)i].offset;
}
extern "C" int tfr_gguf_meta_u64(const tfr_gguf* g, const char* key, uint64_t* out) {
    uint64_t v = 0;
    if (!g || !key || !as_u64(find(g, key), v)) return TFR_E_INVALID;
    if (out) *out = v;
    return TFR_OK;
}
extern "C" int tfr_gguf_meta_f32(const tfr_gguf* g, const char* key, float* out) {
    float v = 0.f;
    if (!g || !key || !as_f32(find(g, key), v)) return TFR_E_INVALID;
    if (out) *out = v;
    return TFR_OK;
}
extern "C" int tfr_gguf_meta_str(const tfr_gguf* g, const char* key, const char** out) {
    const Value* v = g && key ? find(g, key) : nullptr;
    if (!v || v->kind != V_STRING) return TFR_E_INVALID;
    if (out) *out = v->s.c_str();
    return TFR_OK;
}
extern "C" int64_t tfr_gguf_meta_array_len(const tfr_gguf* g, const char* key) {
    const Value* v = g && key ? find(g, key) : nullptr;
    return v && v->kind == V_ARRAY ? (int64_t)v->count : -1;
}
extern "C" int tfr_gguf_meta_array_str(const tfr_gguf* g, const char* key, int64_t i, const char** out, uint64_t* len) {
    const Value* v = g && key ? find(g, key) : nullptr;
    if (!v || v->kind != V_ARRAY || v->item_kind != V_STRING || i < 0 || (uint64_t)i >= v->items_s.size()) return TFR_E_INVALID;
    if (out) *out = v->items_s[(size_t)i].data();
    if (len) *len = v->items_s[(size_t)i].size();
    return TFR_OK;
}
extern "C" int tfr_gguf_meta_array_f32(const tfr_gguf* g, const char* key, int64_t i, float* out) {
    const Value* v = g && key ? find(g, key) : nullptr;
    if (!v || v->kind != V_ARRAY || i < 0 || (uint64_t)i >= v->items_f.size()) return TFR_E_INVALID;
    if (out) *out = (float)v->items_f[(size_t)i];
    return TFR_OK;
}
extern "C" int tfr_gguf_meta_array_i64(const tfr_gguf* g, const char* key, int64_t i, int64_t* out) {
    const Value* v = g && key ? find(g, key) : nullptr;
    if (!v || v->kind != V_ARRAY || i < 0 || (uint64_t)i >= v->items_i.size()) return TFR_E_INVALID;
    if (out) *out = v->items_i[(size_t)i];
    return TFR_OK;
}

// ModelConfig::from_gguf, crates/core/src/config.rs:107-264.
extern "C" int tfr_gguf_model_config(const tfr_gguf* g, tfr_model_config* c, char* err, size_t err_cap) {
    if (!g || !c) return TFR_E_INVALID;
    memset(c, 0, sizeof *c);
    const Value* av = find(g, "general.architecture");
    if (!av || av->kind != V_STRING) return set_err(err, err_cap, TFR_E_INVALID, "missing general.architecture");
    const std::string arch = av->s;
    // Families whose layer schedule differs from the ones built here are refused instead of decoded wrongly:
    // smollm3 skips RoPE on every fourth layer (config.rs:150, layer.rs:417-418); mixture-of-experts models
    // (config.rs is_moe, backend.rs:19-27) run on kernels outside this library.
    if (arch == "smollm3") return set_err(err, err_cap, TFR_E_UNSUPPORTED, "architecture smollm3 is not supported (no-RoPE layers)");
    if (arch == "tara_moe_141" || arch.find("moe") != std::string::npos)
        return set_err(err, err_cap, TFR_E_UNSUPPORTED, "architecture %s is not supported (mixture of experts)", arch.c_str());
    {
        uint64_t experts = 0;
        if (as_u64(find(g, (arch + ".expert_count").c_str()), experts) && experts > 0)
            return set_err(err, err_cap, TFR_E_UNSUPPORTED, "architecture %s with %llu experts is not supported (mixture of experts)",
                           arch.c_str(), (unsigned long long)experts);
    }
    const std::string key_arch = (arch == "llama" || arch == "llama2" || arch == "llama3") ? "llama" : arch;
    auto k = [&](const char* s) { return key_arch + "." + s; };
    auto get = [&](const char* s, uint64_t& v) { return as_u64(find(g, k(s).c_str()), v); };
    uint64_t n_embd = 0, n_layer = 0, n_head = 0, n_ff = 0;
    if (!get("embedding_length", n_embd)) return set_err(err, err_cap, TFR_E_INVALID, "missing %s", k("embedding_length").c_str());
    if (!get("block_count", n_layer)) return set_err(err, err_cap, TFR_E_INVALID, "missing %s", k("block_count").c_str());
    if (!get("attention.head_count", n_head) || n_head == 0)
        return set_err(err, err_cap, TFR_E_INVALID, "missing %s", k("attention.head_count").c_str());
    if (!get("feed_forward_length", n_ff)) return set_err(err, err_cap, TFR_E_INVALID, "missing %s", k("feed_forward_length").c_str());
    uint64_t n_kv = n_head, hd = n_embd / n_head, vhd = 0, ctx = 4096, vocab = 0;
    get("attention.head_count_kv", n_kv);
    get("attention.key_length", hd);
    vhd = hd;
    get("attention.value_length", vhd);
    if (vhd != hd)
        return set_err(err, err_cap, TFR_E_UNSUPPORTED, "different attention key/value lengths are unsupported: key=%llu, value=%llu",
                       (unsigned long long)hd, (unsigned long long)vhd);
    get("context_length", ctx);
    if (!get("vocab_size", vocab)) {
        auto it = g->index.find("token_embd.weight");
        if (it == g->index.end() || g->tensors[it->second].n_dims < 2) return set_err(err, err_cap, TFR_E_INVALID, "vocab size");
        vocab = (uint64_t)g->tensors[it->second].dims[1];
    }
    float theta = key_arch == "llama" ? 10000.0f : 1000000.0f, eps = 1e-6f;
    as_f32(find(g, k("rope.freq_base").c_str()), theta);
    as_f32(find(g, k("attention.layer_norm_rms_epsilon").c_str()), eps);
    c->n_layer = (int32_t)n_layer;
    c->n_embd = (int32_t)n_embd;
    c->n_head = (int32_t)n_head;
    c->n_kv_head = (int32_t)n_kv;
    c->head_dim = (int32_t)hd;
    c->n_ff = (int32_t)n_ff;
    c->n_vocab = (int32_t)vocab;
    c->context_length = (int32_t)ctx;
    c->rope_theta = theta;
    c->rms_eps = eps;
    c->tp_rank = 0;
    c->tp_size = 1;
    if (arch == "qwen35" || arch == "qwen3_5") {
        uint64_t rope_dim = hd, conv = 4, state = 0, nk = 0, nv = 0, inner = 0, interval = 4;
        get("rope.dimension_count", rope_dim);
        get("ssm.conv_kernel", conv);
        if (!get("ssm.state_size", state)) return set_err(err, err_cap, TFR_E_INVALID, "missing %s.ssm.state_size", arch.c_str());
        if (!get("ssm.group_count", nk)) return set_err(err, err_cap, TFR_E_INVALID, "missing %s.ssm.group_count", arch.c_str());
        if (!get("ssm.time_step_rank", nv)) return set_err(err, err_cap, TFR_E_INVALID, "missing %s.ssm.time_step_rank", arch.c_str());
        inner = state * nv;
        get("ssm.inner_size", inner);
        get("full_attention_interval", interval);
        c->hybrid = 1;
        c->rope_dim = (int32_t)rope_dim;
        c->ssm_conv_kernel = (int32_t)conv;
        c->ssm_state_size = (int32_t)state;
        c->ssm_group_count = (int32_t)nk;
        c->ssm_time_step_rank = (int32_t)nv;
        c->ssm_inner_size = (int32_t)inner;
        c->full_attention_interval = (int32_t)(interval ? interval : 1);
    }
    return TFR_OK;
}

// Tensor names the decode path looks up (load.rs:280-417); everything else in the file is ignored.
static bool wanted(const std::string& n) {
    static const char* top[] = {"token_embd.weight", "output.weight", "output_norm.weight"};
    for (const char* t : top)
        if (n == t) return true;
    if (n.compare(0, 4, "blk.") != 0) return false;
    const size_t dot = n.find('.', 4);
    if (dot == std::string::npos) return false;
    const std::string rest = n.substr(dot + 1);
    static const char* layer[] = {"attn_q.weight", "attn_k.weight", "attn_v.weight", "attn_output.weight", "attn_q.bias", "attn_k.bias",
                                  "attn_v.bias", "attn_norm.weight", "ffn_norm.weight", "post_attention_norm.weight", "ffn_gate.weight",
                                  "ffn_up.weight", "ffn_down.weight", "attn_q_norm.weight", "attn_k_norm.weight", "attn_qkv.weight",
                                  "attn_gate.weight", "ssm_beta.weight", "ssm_alpha.weight", "ssm_out.weight", "ssm_conv1d.weight", "ssm_a",
                                  "ssm_dt.bias", "ssm_norm.weight"};
    for (const char* t : layer)
        if (rest == t) return true;
    return false;
}

// CudaModel::load_with (load.rs:166-417): configuration from the metadata, then every tensor of the decode
// path from the mapped file, then the one-off preparation.  tp_size > 1: this engine keeps its shard.
extern "C" int tfr_load_gguf(tfr_engine* e, const tfr_gguf* g, int tp_rank, int tp_size) {
    if (!e || !g) return TFR_E_INVALID;
    tfr_model_config c;
    char msg[256] = "";
    int rc = tfr_gguf_model_config(g, &c, msg, sizeof msg);
    if (rc) {
        fprintf(stderr, "tfr_load_gguf: %s\n", msg);
        return rc;
    }
    c.tp_rank = tp_rank;
    c.tp_size = tp_size < 1 ? 1 : tp_size;
    rc = tfr_set_config(e, &c);
    if (rc) return rc;
    {
        // load.rs:285-352: TARAFER_VOCAB_LIMIT, else 49 152 for a hybrid with more than 100 000 tokens unless
        // TARAFER_FULL_VOCAB is set; limits below 1024 or not below n_vocab are ignored; the end-of-sequence
        // token keeps a row of its own when it lies outside the shortlist.  Not combined with tensor parallelism.
        long long limit = 0;
        if (const char* v = getenv("TARAFER_VOCAB_LIMIT")) {
            char* end = nullptr;
            const long long n = strtoll(v, &end, 10);
            if (end != v && *end == 0 && n > 0) limit = n;
        }
        if (!limit && !getenv("TARAFER_VOCAB_LIMIT") && c.hybrid && c.n_vocab > 100000 && !getenv("TARAFER_FULL_VOCAB")) limit = 49152;
        if (limit >= 1024 && limit < c.n_vocab && c.tp_size == 1) {
            uint64_t eos = 0;
            const bool has_eos = tfr_gguf_meta_u64(g, "tokenizer.ggml.eos_token_id", &eos) == TFR_OK;
            limit &= ~1ll;
            rc = tfr_set_vocab_shortlist(e, (int)limit, has_eos && eos < (uint64_t)c.n_vocab ? (int)eos : -1);
            if (rc) return rc;
            fprintf(stderr, "approximation | active_vocab=%lld/%d (low-id shortlist)\n", limit, c.n_vocab);
        }
    }
    for (size_t i = 0; i < g->tensors.size(); i++) {
        const Tensor& t = g->tensors[i];
        if (!wanted(t.name)) continue;
        const void* data = g->map + g->data_offset + t.offset;
        if (t.type == TFR_TYPE_F32) {
            int64_t n = 1;
            for (int d = 0; d < t.n_dims; d++) n *= t.dims[d];
            rc = tfr_upload_tensor(e, t.name.c_str(), TFR_TYPE_F32, n, 1, data, (size_t)t.nbytes);
        } else {
            rc = tfr_upload_tensor(e, t.name.c_str(), (int)t.type, t.dims[0], t.n_dims > 1 ? t.dims[1] : 1, data, (size_t)t.nbytes);
        }
        if (rc) return rc;
    }
    return tfr_finalize_load(e);
}
