// GGUF v3 reader and the file-backed loader of the resident model: the host side of
// crates/llamd-gguf/src/lib.rs:116-286 (open, parse, tensor, tensor_data),
// crates/llamd-models/src/hparams.rs:78-186 (from_gguf, validate),
// crates/llamd-models/src/model.rs:43-160 (layer tensor names, verify_present) and the checks and upload order of
// DeviceModel::load_batched (crates/llamd-runtime/src/device.rs:225-471).
//
// The file is mapped read-only; tensors are handed to llamd_model_set_tensor straight from the mapping, in slices,
// so that a 23 GiB model never needs a second copy in host memory. No device code in this file.
#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <cerrno>
#include <cstdio>
#include <cstring>
#include <map>
#include <string>
#include <vector>

#include "../../include/llamd_cuda.h"
#include "../../include/llamd_gguf.h"

namespace {

// llamd_core::Error as (kind, message); thrown inside the parser, turned into a return code at the ABI.
struct Failure {
    int kind;
    std::string msg;
};
[[noreturn]] void fail(int kind, const std::string &what, const std::string &detail) { throw Failure{kind, what + ": " + detail}; }

void put_err(char *err, size_t len, const std::string &msg) {
    if (!err || !len) return;
    const size_t n = msg.size() < len - 1 ? msg.size() : len - 1;
    memcpy(err, msg.data(), n);
    err[n] = 0;
}

// Value (lib.rs:23-38). Scalars keep their declared type so that the as_* conversions can refuse like the reference.
struct Value {
    uint32_t type = 0;
    uint64_t u = 0;  // U8..U64, Bool
    int64_t i = 0;   // I8..I64
    double f = 0;    // F32 (exactly representable), F64
    std::string s;
    uint32_t inner = 0;       // element type of an array
    std::vector<Value> arr;
};

enum { T_U8, T_I8, T_U16, T_I16, T_U32, T_I32, T_F32, T_BOOL, T_STRING, T_ARRAY, T_U64, T_I64, T_F64 };

struct TensorInfo {
    std::string name;
    std::vector<uint64_t> dims;
    uint32_t ggml_type;
    uint64_t offset;
    // elems (lib.rs:98-101); a product that overflows u64 is reported when the data is asked for
    bool elems(uint64_t *out) const {
        uint64_t n = 1;
        for (uint64_t d : dims)
            if (__builtin_mul_overflow(n, d, &n)) return false;
        *out = n;
        return true;
    }
};

struct Reader {
    const uint8_t *b;
    size_t len, p = 0;
    const uint8_t *take(size_t n) {
        if (n > len - p) fail(LLAMD_E_MALFORMED, "gguf", "truncated: wanted " + std::to_string(n) + " bytes at " + std::to_string(p) + ", file has " + std::to_string(len));
        const uint8_t *s = b + p;
        p += n;
        return s;
    }
    template <class T>
    T le() {
        T v;
        memcpy(&v, take(sizeof(T)), sizeof(T));  // the format is little-endian and so is every host this library runs on
        return v;
    }
    std::string string() {
        const uint64_t n = le<uint64_t>();
        if (n > len - p) fail(LLAMD_E_MALFORMED, "gguf", "truncated: wanted " + std::to_string(n) + " bytes at " + std::to_string(p) + ", file has " + std::to_string(len));
        const uint8_t *s = take((size_t)n);
        return std::string((const char *)s, (size_t)n);  // bytes kept as they are; the reference replaces invalid UTF-8, keys on the path are ASCII
    }
    Value value(uint32_t ty) {
        Value v;
        v.type = ty;
        switch (ty) {
        case T_U8: v.u = le<uint8_t>(); break;
        case T_I8: v.i = le<int8_t>(); break;
        case T_U16: v.u = le<uint16_t>(); break;
        case T_I16: v.i = le<int16_t>(); break;
        case T_U32: v.u = le<uint32_t>(); break;
        case T_I32: v.i = le<int32_t>(); break;
        case T_F32: v.f = le<float>(); break;
        case T_BOOL: v.u = le<uint8_t>() != 0; break;
        case T_STRING: v.s = string(); break;
        case T_ARRAY: {
            v.inner = le<uint32_t>();
            const uint64_t n = le<uint64_t>();
            if (v.inner == T_ARRAY) fail(LLAMD_E_UNSUPPORTED, "gguf array", "nested arrays");
            // every element takes at least one byte: a count beyond the rest of the file is a lie, refused before any reservation
            if (n > len - p) fail(LLAMD_E_MALFORMED, "gguf array", std::to_string(n) + " elements declared, only " + std::to_string(len - p) + " bytes remain");
            v.arr.reserve((size_t)(n < 65536 ? n : 65536));
            for (uint64_t k = 0; k < n; k++) v.arr.push_back(value(v.inner));
        } break;
        case T_U64: v.u = le<uint64_t>(); break;
        case T_I64: v.i = le<int64_t>(); break;
        case T_F64: v.f = le<double>(); break;
        default: fail(LLAMD_E_MALFORMED, "gguf value", "unknown type " + std::to_string(ty));
        }
        return v;
    }
};

}  // namespace

struct llamd_gguf {
    uint32_t version = 0;
    std::map<std::string, Value> metadata;  // sorted, like the reference's BTreeMap
    std::vector<const std::string *> keys;  // metadata keys in map order, for llamd_gguf_metadata_key
    std::vector<TensorInfo> tensors;
    uint64_t data_offset = 0, alignment = 32;
    const uint8_t *map = nullptr;
    size_t len = 0;
    bool owned = false;  // mapping made by llamd_gguf_open (munmap on close)

    const Value *get(const std::string &k) const {
        auto it = metadata.find(k);
        return it == metadata.end() ? nullptr : &it->second;
    }
    const TensorInfo *tensor(const std::string &name) const {
        for (const TensorInfo &t : tensors)
            if (t.name == name) return &t;
        return nullptr;
    }
};

namespace {

bool as_u64(const Value *v, uint64_t *out) {
    if (!v) return false;
    switch (v->type) {
    case T_U8: case T_U16: case T_U32: case T_U64: *out = v->u; return true;
    case T_I8: case T_I16: case T_I32: case T_I64:
        if (v->i < 0) return false;
        *out = (uint64_t)v->i;
        return true;
    default: return false;
    }
}
bool as_f32(const Value *v, float *out) {
    if (!v || (v->type != T_F32 && v->type != T_F64)) return false;
    *out = (float)v->f;  // F64 rounds once to f32, as `as f32` does
    return true;
}

void parse_into(llamd_gguf &g) {
    Reader r{g.map, g.len};
    const uint8_t *magic = r.take(4);
    if (memcmp(magic, "GGUF", 4)) {
        char shown[64];
        snprintf(shown, sizeof shown, "[%u, %u, %u, %u]", magic[0], magic[1], magic[2], magic[3]);
        fail(LLAMD_E_MALFORMED, "gguf header", std::string("magic is ") + shown + ", expected \"GGUF\"");
    }
    g.version = r.le<uint32_t>();
    if (g.version != 3) fail(LLAMD_E_UNSUPPORTED, "gguf version", "version " + std::to_string(g.version) + "; this parser implements 3");
    const uint64_t n_tensors = r.le<uint64_t>(), n_kv = r.le<uint64_t>();
    if (n_tensors > g.len || n_kv > g.len)
        fail(LLAMD_E_MALFORMED, "gguf header", std::to_string(n_kv) + " kv / " + std::to_string(n_tensors) + " tensors exceeds the " + std::to_string(g.len) + "-byte file");
    for (uint64_t k = 0; k < n_kv; k++) {
        std::string key = r.string();
        const uint32_t ty = r.le<uint32_t>();
        g.metadata[key] = r.value(ty);  // a repeated key keeps its last value (BTreeMap::insert)
    }
    g.tensors.reserve((size_t)(n_tensors < 4096 ? n_tensors : 4096));
    for (uint64_t k = 0; k < n_tensors; k++) {
        TensorInfo t;
        t.name = r.string();
        const uint32_t n_dims = r.le<uint32_t>();
        if (n_dims > 4) fail(LLAMD_E_MALFORMED, "tensor info", t.name + " claims " + std::to_string(n_dims) + " dimensions; ggml allows at most 4");
        for (uint32_t d = 0; d < n_dims; d++) t.dims.push_back(r.le<uint64_t>());
        t.ggml_type = r.le<uint32_t>();
        t.offset = r.le<uint64_t>();
        g.tensors.push_back(std::move(t));
    }
    uint64_t a = 32;
    if (as_u64(g.get("general.alignment"), &a)) {}
    if (a == 0 || (a & (a - 1))) fail(LLAMD_E_MALFORMED, "general.alignment", std::to_string(a) + " is not a power of two");
    g.alignment = a;
    const uint64_t pos = r.p;
    uint64_t off;
    if (__builtin_add_overflow(pos, a - 1, &off)) fail(LLAMD_E_MALFORMED, "gguf layout", "data section offset overflows");
    off &= ~(a - 1);
    if (off > g.len) fail(LLAMD_E_MALFORMED, "gguf layout", "data section starts at " + std::to_string(off) + ", past the " + std::to_string(g.len) + "-byte file");
    g.data_offset = off;
    for (auto &kv : g.metadata) g.keys.push_back(&kv.first);
}

// QuantType::from_ggml + bytes_for (crates/llamd-quant/src/lib.rs:58-102)
const char *type_name(uint32_t t) {
    switch (t) {
    case LLAMD_GGML_F32: return "F32";
    case LLAMD_GGML_F16: return "F16";
    case LLAMD_GGML_Q8_0: return "Q8_0";
    case LLAMD_GGML_Q6_K: return "Q6K";
    default: return "?";
    }
}
uint64_t bytes_for(uint32_t ggml_type, uint64_t n) {
    uint64_t be, bb;
    switch (ggml_type) {
    case LLAMD_GGML_F32: be = 1, bb = 4; break;
    case LLAMD_GGML_F16: be = 1, bb = 2; break;
    case LLAMD_GGML_Q8_0: be = 32, bb = 34; break;
    case LLAMD_GGML_Q6_K: be = 256, bb = 210; break;
    default: fail(LLAMD_E_UNSUPPORTED, "ggml quantization type", "type " + std::to_string(ggml_type) + " is not implemented yet");
    }
    if (n % be) fail(LLAMD_E_MALFORMED, "tensor length", std::to_string(n) + " elements is not a multiple of the " + std::to_string(be) + "-element block for " + type_name(ggml_type));
    uint64_t out;
    if (__builtin_mul_overflow(n / be, bb, &out)) fail(LLAMD_E_MALFORMED, "tensor", "byte length overflows");
    return out;
}

// Gguf::tensor_data (lib.rs:231-256)
const uint8_t *tensor_bytes(const llamd_gguf &g, const TensorInfo &t, size_t *n_bytes) {
    uint64_t n;
    if (!t.elems(&n)) fail(LLAMD_E_MALFORMED, "tensor", t.name + " has too many elements");
    const uint64_t len = bytes_for(t.ggml_type, n);
    uint64_t start, end;
    if (__builtin_add_overflow(g.data_offset, t.offset, &start)) fail(LLAMD_E_MALFORMED, "tensor", "offset does not fit in usize");
    if (__builtin_add_overflow(start, len, &end)) fail(LLAMD_E_MALFORMED, "tensor", t.name + " extent overflows");
    if (end > g.len)
        fail(LLAMD_E_MALFORMED, "tensor", t.name + " spans " + std::to_string(start) + ".." + std::to_string(end) + ", past the " + std::to_string(g.len) + "-byte file");
    *n_bytes = (size_t)len;
    return g.map + start;
}

struct Hp {
    llamd_hparams hp{};
    bool moe = false;
    uint64_t n_ff = 0, n_ctx_train = 0;
};

// Hparams::from_gguf (hparams.rs:78-149) and validate (:151-175)
Hp read_hparams(const llamd_gguf &g) {
    const Value *av = g.get("general.architecture");
    if (!av || av->type != T_STRING) fail(LLAMD_E_MALFORMED, "hparams", "general.architecture is absent");
    Hp h;
    if (av->s == "qwen3") h.moe = false;
    else if (av->s == "qwen3moe") h.moe = true;
    else fail(LLAMD_E_UNSUPPORTED, "architecture", av->s + "; LLAMD implements qwen3 and qwen3moe");
    const std::string p = av->s;
    auto req_u = [&](const char *suffix) -> uint64_t {
        const std::string k = p + "." + suffix;
        uint64_t v;
        if (!as_u64(g.get(k), &v)) fail(LLAMD_E_MALFORMED, "hparams", k + " is absent");
        return v;
    };
    auto req_f = [&](const char *suffix) -> float {
        const std::string k = p + "." + suffix;
        float v;
        if (!as_f32(g.get(k), &v)) fail(LLAMD_E_MALFORMED, "hparams", k + " is absent");
        return v;
    };
    const uint64_t n_embd = req_u("embedding_length"), n_head = req_u("attention.head_count"), n_head_kv = req_u("attention.head_count_kv");
    // head_dim: the explicit key, else the K projection's output width over the kv heads, else n_embd / n_head
    uint64_t hd;
    if (!as_u64(g.get(p + ".attention.key_length"), &hd)) {
        const TensorInfo *k = g.tensor("blk.0.attn_k.weight");
        if (k && k->dims.size() > 1) hd = k->dims[1] / (n_head_kv ? n_head_kv : 1);
        else hd = n_embd / (n_head ? n_head : 1);
    }
    const TensorInfo *te = g.tensor("token_embd.weight");
    if (!te || te->dims.size() < 2) fail(LLAMD_E_MALFORMED, "hparams", "token_embd.weight is absent");
    const uint64_t n_vocab = te->dims[1];
    uint64_t n_expert = 0, n_used = 0, n_ffe = 0;
    if (h.moe) {
        n_expert = req_u("expert_count");
        n_used = req_u("expert_used_count");
        n_ffe = req_u("expert_feed_forward_length");
    }
    const uint64_t n_layer = req_u("block_count");
    h.n_ff = req_u("feed_forward_length");
    h.n_ctx_train = req_u("context_length");
    const float freq_base = req_f("rope.freq_base"), eps = req_f("attention.layer_norm_rms_epsilon");
    if (n_head_kv == 0 || n_head % n_head_kv) fail(LLAMD_E_MALFORMED, "hparams", std::to_string(n_head) + " query heads do not divide into " + std::to_string(n_head_kv) + " kv heads");
    if (hd % 2) fail(LLAMD_E_MALFORMED, "hparams", "head_dim " + std::to_string(hd) + " must be even for RoPE");
    if (h.moe && (n_used == 0 || n_used > n_expert)) fail(LLAMD_E_MALFORMED, "hparams", std::to_string(n_used) + " experts used of " + std::to_string(n_expert) + " available");
    for (uint64_t v : {n_layer, n_embd, n_head, n_head_kv, hd, n_expert, n_used, n_ffe, n_vocab})
        if (v > 0x7fffffffu) fail(LLAMD_E_MALFORMED, "hparams", "a dimension of " + std::to_string(v) + " does not fit the device model");
    h.hp.n_layer = (int32_t)n_layer;
    h.hp.n_embd = (int32_t)n_embd;
    h.hp.n_head = (int32_t)n_head;
    h.hp.n_head_kv = (int32_t)n_head_kv;
    h.hp.head_dim = (int32_t)hd;
    h.hp.n_expert = (int32_t)n_expert;
    h.hp.n_expert_used = (int32_t)n_used;
    h.hp.n_ff_expert = (int32_t)n_ffe;
    h.hp.n_vocab = (int32_t)n_vocab;
    h.hp.rope_freq_base = freq_base;
    h.hp.rms_eps = eps;
    return h;
}

// LayerNames (model.rs:24-98): which tensors a layer needs and which are optional
struct LayerTensor {
    const char *suffix;
    int id;         // LLAMD_T_*; -1 = a dense-FFN tensor the device model has no slot for
    bool f32;       // uploaded as f32 (norms, the router); otherwise a Q6_K matrix
    bool optional;  // attn_q_norm / attn_k_norm
    bool moe_only, dense_only;
};
const LayerTensor kLayerTensors[] = {
    {"attn_norm.weight", LLAMD_T_ATTN_NORM, true, false, false, false},
    {"attn_q.weight", LLAMD_T_ATTN_Q, false, false, false, false},
    {"attn_k.weight", LLAMD_T_ATTN_K, false, false, false, false},
    {"attn_v.weight", LLAMD_T_ATTN_V, false, false, false, false},
    {"attn_q_norm.weight", LLAMD_T_ATTN_Q_NORM, true, true, false, false},
    {"attn_k_norm.weight", LLAMD_T_ATTN_K_NORM, true, true, false, false},
    {"attn_output.weight", LLAMD_T_ATTN_OUT, false, false, false, false},
    {"ffn_norm.weight", LLAMD_T_FFN_NORM, true, false, false, false},
    {"ffn_gate.weight", -1, false, false, false, true},
    {"ffn_up.weight", -1, false, false, false, true},
    {"ffn_down.weight", -1, false, false, false, true},
    {"ffn_gate_inp.weight", LLAMD_T_FFN_GATE_INP, true, false, true, false},
    {"ffn_gate_exps.weight", LLAMD_T_FFN_GATE_EXPS, false, false, true, false},
    {"ffn_up_exps.weight", LLAMD_T_FFN_UP_EXPS, false, false, true, false},
    {"ffn_down_exps.weight", LLAMD_T_FFN_DOWN_EXPS, false, false, true, false},
};
std::string blk(int il, const char *suffix) { return "blk." + std::to_string(il) + "." + suffix; }

// Model::verify_present (model.rs:133-160)
void verify_present(const llamd_gguf &g, const Hp &h) {
    std::vector<std::string> missing;
    for (const char *n : {"token_embd.weight", "output_norm.weight"})
        if (!g.tensor(n)) missing.push_back(n);
    for (int il = 0; il < h.hp.n_layer; il++)
        for (const LayerTensor &t : kLayerTensors) {
            if (t.optional || (t.moe_only && !h.moe) || (t.dense_only && h.moe)) continue;
            const std::string n = blk(il, t.suffix);
            if (!g.tensor(n)) missing.push_back(n);
        }
    if (missing.empty()) return;
    std::string first = "[";
    for (size_t i = 0; i < missing.size() && i < 3; i++) first += (i ? ", \"" : "\"") + missing[i] + "\"";
    fail(LLAMD_E_MALFORMED, "model", std::to_string(missing.size()) + " tensors missing, first: " + first + "]");
}

// IEEE binary16 -> f32, exact (subnormals included): for norm vectors stored as F16
float half_to_float(uint16_t h) {
    const uint32_t sign = (uint32_t)(h & 0x8000) << 16, exp = (h >> 10) & 31, man = h & 1023;
    uint32_t bits;
    if (exp == 0) {
        if (man == 0) bits = sign;
        else {
            int e = -1;
            uint32_t m = man;
            do { m <<= 1; e++; } while (!(m & 1024));
            bits = sign | ((uint32_t)(112 - e) << 23) | ((m & 1023) << 13);
        }
    } else if (exp == 31) bits = sign | 0x7f800000u | (man << 13);
    else bits = sign | ((exp + 112) << 23) | (man << 13);
    float f;
    memcpy(&f, &bits, 4);
    return f;
}

const TensorInfo &need_tensor(const llamd_gguf &g, const std::string &name) {
    const TensorInfo *t = g.tensor(name);
    if (!t) fail(LLAMD_E_MALFORMED, "model", "tensor " + name + " is absent");
    return *t;
}

// A Q6_K matrix as DeviceModel's up_planar takes it (device.rs:236-249): k = dims[0], rows = elems / k, Q6_K only.
// `rows` and `k` are what the hyperparameters say the tensor must be.
const uint8_t *q6k_matrix(const llamd_gguf &g, const std::string &name, uint64_t rows, uint64_t k, size_t *n_bytes) {
    const TensorInfo &t = need_tensor(g, name);
    if (t.ggml_type != LLAMD_GGML_Q6_K) {
        bytes_for(t.ggml_type, 0);  // an unknown type id is reported as such
        fail(LLAMD_E_UNSUPPORTED, "planar upload", name + " is " + type_name(t.ggml_type) + ", not Q6_K");
    }
    uint64_t n;
    if (!t.elems(&n) || t.dims.empty() || t.dims[0] != k || n != rows * k) {
        std::string d;
        for (uint64_t v : t.dims) d += (d.empty() ? "" : ", ") + std::to_string(v);
        fail(LLAMD_E_MALFORMED, "shape", name + " is [" + d + "], the hyperparameters want " + std::to_string(rows) + " rows of " + std::to_string(k));
    }
    return tensor_bytes(g, t, n_bytes);
}

// An f32 vector or matrix (up_f32, device.rs:253-256): stored F32, or F16 widened exactly.
std::vector<float> f32_tensor(const llamd_gguf &g, const std::string &name, uint64_t want) {
    const TensorInfo &t = need_tensor(g, name);
    size_t nb;
    const uint8_t *p = tensor_bytes(g, t, &nb);
    uint64_t n = 0;
    t.elems(&n);
    if (n != want) fail(LLAMD_E_MALFORMED, "shape", name + " has " + std::to_string(n) + " elements, the hyperparameters want " + std::to_string(want));
    std::vector<float> out((size_t)n);
    if (t.ggml_type == LLAMD_GGML_F32) memcpy(out.data(), p, nb);
    else if (t.ggml_type == LLAMD_GGML_F16)
        for (size_t i = 0; i < out.size(); i++) {
            uint16_t h;
            memcpy(&h, p + 2 * i, 2);
            out[i] = half_to_float(h);
        }
    else fail(LLAMD_E_UNSUPPORTED, "f32 upload", name + " is " + type_name(t.ggml_type) + "; norms and the router are read as F32 or F16");
    return out;
}

llamd_model *load_model(const llamd_gguf &g, int max_kv, int max_seq) {
    const Hp h = read_hparams(g);
    verify_present(g, h);
    if (!h.moe) fail(LLAMD_E_UNSUPPORTED, "device model", "only MoE models are wired up; a dense FFN has no expert path");
    if (max_kv <= 0) fail(LLAMD_E_MALFORMED, "device model", "max_kv of 0");
    const llamd_hparams &hp = h.hp;
    const uint64_t E = hp.n_embd, qd = (uint64_t)hp.n_head * hp.head_dim, kvd = (uint64_t)hp.n_head_kv * hp.head_dim;
    const uint64_t ffe = hp.n_ff_expert, ne = hp.n_expert, V = hp.n_vocab;
    const int world = llamd_cuda_ep_world() > 0 ? llamd_cuda_ep_world() : 1, rank = world > 1 ? llamd_cuda_ep_rank() : 0;
    const bool tied = g.tensor("output.weight") == nullptr;  // the head then reads the embedding table (model.rs:117-121)

    // Pass 1: every matrix is looked up, type- and shape-checked, and sized, before anything is uploaded
    // (device.rs:292-323: refuse early and legibly rather than partway through a 23 GiB upload).
    struct Mat {
        int layer, id;
        std::string name;
        const uint8_t *p;
        size_t bytes;
    };
    std::vector<Mat> mats;
    uint64_t need = 0;
    auto add = [&](int layer, int id, const std::string &name, uint64_t rows, uint64_t k, bool expert) {
        size_t nb;
        const uint8_t *p = q6k_matrix(g, name, rows, k, &nb);
        mats.push_back({layer, id, name, p, nb});
        need += expert ? nb / world : nb;
    };
    add(-1, LLAMD_T_TOK_EMBD, "token_embd.weight", V, E, false);
    if (!tied) add(-1, LLAMD_T_OUTPUT, "output.weight", V, E, false);
    for (int il = 0; il < hp.n_layer; il++) {
        add(il, LLAMD_T_ATTN_Q, blk(il, "attn_q.weight"), qd, E, false);
        add(il, LLAMD_T_ATTN_K, blk(il, "attn_k.weight"), kvd, E, false);
        add(il, LLAMD_T_ATTN_V, blk(il, "attn_v.weight"), kvd, E, false);
        add(il, LLAMD_T_ATTN_OUT, blk(il, "attn_output.weight"), E, qd, false);
        add(il, LLAMD_T_FFN_GATE_EXPS, blk(il, "ffn_gate_exps.weight"), ne * ffe, E, true);
        add(il, LLAMD_T_FFN_UP_EXPS, blk(il, "ffn_up_exps.weight"), ne * ffe, E, true);
        add(il, LLAMD_T_FFN_DOWN_EXPS, blk(il, "ffn_down_exps.weight"), ne * E, ffe, true);
    }
    const uint64_t free_b = llamd_cuda_free_mem();
    if (free_b > 0 && need + (1ull << 30) > free_b) {
        char buf[160];
        snprintf(buf, sizeof buf, "model needs about %.1f GiB of weights but only %.1f GiB is free", need / 1073741824.0, free_b / 1073741824.0);
        throw Failure{LLAMD_E_OTHER, buf};
    }

    llamd_model *m = llamd_model_create(&hp, max_kv, max_seq);
    if (!m) throw Failure{LLAMD_E_OTHER, std::string("device model: ") + llamd_cuda_last_error_string()};
    try {
        auto check = [&](int rc, const std::string &name) {
            if (rc) throw Failure{LLAMD_E_OTHER, name + ": " + llamd_model_error(m)};
        };
        auto up_f32 = [&](int layer, int id, const std::string &name, uint64_t n) {
            const std::vector<float> v = f32_tensor(g, name, n);
            check(llamd_model_set_tensor(m, layer, id, 0, v.data(), v.size()), name);
        };
        for (const Mat &t : mats) {
            const size_t blocks = t.bytes / LLAMD_Q6K_BLOCK_BYTES;
            const bool expert = t.id == LLAMD_T_FFN_GATE_EXPS || t.id == LLAMD_T_FFN_UP_EXPS || t.id == LLAMD_T_FFN_DOWN_EXPS;
            // expert e is a contiguous block range (model.rs:182-227): with expert parallelism only this rank's range is read
            const size_t lo = expert ? blocks / world * rank : 0, cnt = expert ? blocks / world : blocks;
            // 64 MiB at a time: the staging and re-layout on the device side stay small whatever the tensor's size
            const size_t step = (64u << 20) / LLAMD_Q6K_BLOCK_BYTES;
            for (size_t b0 = 0; b0 < cnt; b0 += step) {
                const size_t c = cnt - b0 < step ? cnt - b0 : step;
                check(llamd_model_set_tensor(m, t.layer, t.id, lo + b0, t.p + (lo + b0) * LLAMD_Q6K_BLOCK_BYTES, c), t.name);
            }
        }
        up_f32(-1, LLAMD_T_OUTPUT_NORM, "output_norm.weight", E);
        for (int il = 0; il < hp.n_layer; il++) {
            up_f32(il, LLAMD_T_ATTN_NORM, blk(il, "attn_norm.weight"), E);
            up_f32(il, LLAMD_T_FFN_NORM, blk(il, "ffn_norm.weight"), E);
            if (g.tensor(blk(il, "attn_q_norm.weight"))) up_f32(il, LLAMD_T_ATTN_Q_NORM, blk(il, "attn_q_norm.weight"), hp.head_dim);
            if (g.tensor(blk(il, "attn_k_norm.weight"))) up_f32(il, LLAMD_T_ATTN_K_NORM, blk(il, "attn_k_norm.weight"), hp.head_dim);
            up_f32(il, LLAMD_T_FFN_GATE_INP, blk(il, "ffn_gate_inp.weight"), ne * E);
        }
    } catch (...) {
        llamd_model_free(m);
        throw;
    }
    return m;
}

}  // namespace

// ---- C ABI -------------------------------------------------------------------------------------------------------
namespace {
template <class F>
int guarded(char *err, size_t err_len, F &&f) {
    try {
        f();
        return LLAMD_E_OK;
    } catch (const Failure &e) {
        put_err(err, err_len, e.msg);
        return e.kind;
    } catch (const std::exception &e) {
        put_err(err, err_len, e.what());
        return LLAMD_E_OTHER;
    }
}
}  // namespace

extern "C" {

llamd_gguf *llamd_gguf_parse(const void *bytes, size_t len, int *kind, char *err, size_t err_len) {
    llamd_gguf *g = new llamd_gguf;
    g->map = (const uint8_t *)bytes;
    g->len = len;
    const int rc = bytes ? guarded(err, err_len, [&] { parse_into(*g); }) : LLAMD_E_MALFORMED;
    if (kind) *kind = rc;
    if (rc) {
        delete g;
        return nullptr;
    }
    return g;
}

llamd_gguf *llamd_gguf_open(const char *path, int *kind, char *err, size_t err_len) {
    auto io_fail = [&](const char *what) -> llamd_gguf * {
        put_err(err, err_len, std::string(what) + " " + (path ? path : "(null)") + ": " + strerror(errno));
        if (kind) *kind = LLAMD_E_IO;
        return nullptr;
    };
    if (!path) {
        errno = EINVAL;
        return io_fail("open");
    }
    const int fd = open(path, O_RDONLY | O_CLOEXEC);
    if (fd < 0) return io_fail("open");
    struct stat st;
    if (fstat(fd, &st)) {
        close(fd);
        return io_fail("stat");
    }
    if (st.st_size == 0) {  // an empty file cannot be mapped; it is a truncated header
        close(fd);
        static const uint8_t none = 0;
        return llamd_gguf_parse(&none, 0, kind, err, err_len);
    }
    void *p = mmap(nullptr, (size_t)st.st_size, PROT_READ, MAP_PRIVATE, fd, 0);
    close(fd);  // the mapping keeps the file
    if (p == MAP_FAILED) return io_fail("mmap");
    llamd_gguf *g = llamd_gguf_parse(p, (size_t)st.st_size, kind, err, err_len);
    if (!g) munmap(p, (size_t)st.st_size);
    else g->owned = true;
    return g;
}

void llamd_gguf_close(llamd_gguf *g) {
    if (!g) return;
    if (g->owned) munmap((void *)g->map, g->len);
    delete g;
}

uint32_t llamd_gguf_version(const llamd_gguf *g) { return g ? g->version : 0; }
uint64_t llamd_gguf_alignment(const llamd_gguf *g) { return g ? g->alignment : 0; }
uint64_t llamd_gguf_data_offset(const llamd_gguf *g) { return g ? g->data_offset : 0; }
uint64_t llamd_gguf_file_size(const llamd_gguf *g) { return g ? g->len : 0; }
uint64_t llamd_gguf_n_metadata(const llamd_gguf *g) { return g ? g->metadata.size() : 0; }
uint64_t llamd_gguf_n_tensors(const llamd_gguf *g) { return g ? g->tensors.size() : 0; }

int llamd_gguf_get_u64(const llamd_gguf *g, const char *key, uint64_t *out) {
    uint64_t v;
    if (!g || !key || !as_u64(g->get(key), &v)) return LLAMD_E_ABSENT;
    if (out) *out = v;
    return LLAMD_E_OK;
}
int llamd_gguf_get_f32(const llamd_gguf *g, const char *key, float *out) {
    float v;
    if (!g || !key || !as_f32(g->get(key), &v)) return LLAMD_E_ABSENT;
    if (out) *out = v;
    return LLAMD_E_OK;
}
int llamd_gguf_get_str(const llamd_gguf *g, const char *key, char *out, size_t len, size_t *full_len) {
    const Value *v = g && key ? g->get(key) : nullptr;
    if (!v || v->type != T_STRING) return LLAMD_E_ABSENT;
    if (full_len) *full_len = v->s.size();
    put_err(out, len, v->s);
    return LLAMD_E_OK;
}
int llamd_gguf_get_array_len(const llamd_gguf *g, const char *key, uint64_t *out) {
    const Value *v = g && key ? g->get(key) : nullptr;
    if (!v || v->type != T_ARRAY) return LLAMD_E_ABSENT;
    if (out) *out = v->arr.size();
    return LLAMD_E_OK;
}
const char *llamd_gguf_metadata_key(const llamd_gguf *g, uint64_t i) { return g && i < g->keys.size() ? g->keys[i]->c_str() : nullptr; }

int64_t llamd_gguf_find_tensor(const llamd_gguf *g, const char *name) {
    if (!g || !name) return -1;
    for (size_t i = 0; i < g->tensors.size(); i++)
        if (g->tensors[i].name == name) return (int64_t)i;
    return -1;
}
const char *llamd_gguf_tensor_name(const llamd_gguf *g, uint64_t index) { return g && index < g->tensors.size() ? g->tensors[index].name.c_str() : nullptr; }
int llamd_gguf_tensor_info(const llamd_gguf *g, uint64_t index, uint32_t *ggml_type, int *n_dims, uint64_t dims[4], uint64_t *offset) {
    if (!g || index >= g->tensors.size()) return LLAMD_E_ABSENT;
    const TensorInfo &t = g->tensors[index];
    if (ggml_type) *ggml_type = t.ggml_type;
    if (n_dims) *n_dims = (int)t.dims.size();
    if (dims)
        for (size_t d = 0; d < 4; d++) dims[d] = d < t.dims.size() ? t.dims[d] : 1;
    if (offset) *offset = t.offset;
    return LLAMD_E_OK;
}
int llamd_gguf_tensor_data(const llamd_gguf *g, uint64_t index, const void **data, size_t *n_bytes, char *err, size_t err_len) {
    if (!g || index >= g->tensors.size()) return LLAMD_E_ABSENT;
    return guarded(err, err_len, [&] {
        size_t nb;
        const uint8_t *p = tensor_bytes(*g, g->tensors[index], &nb);
        if (data) *data = p;
        if (n_bytes) *n_bytes = nb;
    });
}

int llamd_gguf_hparams(const llamd_gguf *g, llamd_hparams *hp, int *is_moe, int32_t *n_ff, int32_t *n_ctx_train, char *err, size_t err_len) {
    if (!g) return LLAMD_E_ABSENT;
    return guarded(err, err_len, [&] {
        const Hp h = read_hparams(*g);
        if (hp) *hp = h.hp;
        if (is_moe) *is_moe = h.moe;
        if (n_ff) *n_ff = (int32_t)(h.n_ff < 0x7fffffffu ? h.n_ff : 0x7fffffffu);
        if (n_ctx_train) *n_ctx_train = (int32_t)(h.n_ctx_train < 0x7fffffffu ? h.n_ctx_train : 0x7fffffffu);
    });
}
int llamd_gguf_verify_present(const llamd_gguf *g, char *err, size_t err_len) {
    if (!g) return LLAMD_E_ABSENT;
    return guarded(err, err_len, [&] { verify_present(*g, read_hparams(*g)); });
}

llamd_model *llamd_model_load_gguf(const llamd_gguf *g, int max_kv, int max_seq, int *kind, char *err, size_t err_len) {
    llamd_model *m = nullptr;
    const int rc = g ? guarded(err, err_len, [&] { m = load_model(*g, max_kv, max_seq); }) : LLAMD_E_ABSENT;
    if (kind) *kind = rc;
    return rc ? nullptr : m;
}

}  // extern "C"
