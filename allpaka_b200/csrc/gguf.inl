// GGUF files on the host: the header and tensor table (crates/allpaka-gguf/src/metadata.rs:194-297,
// 369-466), tensor bytes straight out of a read-only mapping (crates/allpaka-gguf/src/tensors.rs:
// 183-217), and the dense-decoder view of a model that the decode path consumes
// (crates/allpaka-model/src/config.rs:184-310, crates/allpaka-model/src/model/loader.rs:100-260,
// 366-426, 558-580).  Pure host code: nothing here needs a GPU until apk_model_attach.

#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <map>

struct GgufValue {
    enum Kind { NONE, UINT, INT, FLOAT, STR, U32ARR, SKIPPED } kind = NONE;
    uint64_t u = 0;
    int64_t i = 0;
    double f = 0.0;
    std::string s;
    std::vector<uint32_t> arr;
};

struct GgufTensor {
    std::string name;
    uint32_t ty = 0, n_dims = 0;
    uint64_t dims[4] = {1, 1, 1, 1};
    uint64_t offset = 0;   // from the start of the data section
    uint64_t n_bytes = 0;  // 0: a type this library has no geometry for
};

struct apk_gguf {
    int fd = -1;
    const uint8_t *map = nullptr;
    size_t len = 0;
    uint32_t version = 0;
    uint64_t data_offset = 0;
    std::string arch;
    std::vector<std::pair<std::string, GgufValue>> fields;
    std::map<std::string, size_t> field_index;
    std::vector<GgufTensor> tensors;
    std::map<std::string, size_t> tensor_index;
    ~apk_gguf() {
        if (map) munmap((void *)map, len);
        if (fd >= 0) close(fd);
    }
};

namespace {

// Bytes of `elements` values of a GGML type: the block geometries of crates/allpaka-dtype/src/lib.rs:79-108
// that can appear in a decoder file this library serves (quantised matrices it has kernels for, f32/f16 vectors).
bool gguf_type_bytes(uint32_t ty, uint64_t elements, uint64_t *out) {
    uint32_t be, bb;
    if (ty == 0) { *out = elements * 4; return true; }  // F32
    if (ty == 1) { *out = elements * 2; return true; }  // F16
    if (ty == 30) { *out = elements * 2; return true; } // BF16
    if (!block_geom(ty, &be, &bb) || elements % be) return false;
    *out = elements / be * bb;
    return true;
}

struct GgufCursor {
    const uint8_t *p, *end;
    bool ok = true;
    bool need(uint64_t n) {
        if (!ok || (uint64_t)(end - p) < n) ok = false;
        return ok;
    }
    template <class T> T get() {
        T v{};
        if (need(sizeof(T))) {
            memcpy(&v, p, sizeof(T));
            p += sizeof(T);
        }
        return v;
    }
    std::string str() {
        const uint64_t n = get<uint64_t>();
        if (n > (1u << 20) || !need(n)) {  // "implausible GGUF string length" (metadata.rs:468-479)
            ok = false;
            return {};
        }
        std::string s((const char *)p, (size_t)n);
        p += n;
        return s;
    }
};

// width of a scalar value type, 0 for strings / arrays / unknown
int gguf_scalar_bytes(uint32_t kind) {
    switch (kind) {
        case 0: case 1: case 7: return 1;
        case 2: case 3: return 2;
        case 4: case 5: case 6: return 4;
        case 10: case 11: case 12: return 8;
        default: return 0;
    }
}

bool gguf_read_value(GgufCursor &c, GgufValue *v) {
    const uint32_t kind = c.get<uint32_t>();
    switch (kind) {
        case 0: v->kind = GgufValue::UINT; v->u = c.get<uint8_t>(); break;
        case 1: v->kind = GgufValue::INT; v->i = c.get<int8_t>(); break;
        case 2: v->kind = GgufValue::UINT; v->u = c.get<uint16_t>(); break;
        case 3: v->kind = GgufValue::INT; v->i = c.get<int16_t>(); break;
        case 4: v->kind = GgufValue::UINT; v->u = c.get<uint32_t>(); break;
        case 5: v->kind = GgufValue::INT; v->i = c.get<int32_t>(); break;
        case 6: v->kind = GgufValue::FLOAT; v->f = c.get<float>(); break;
        case 7: v->kind = GgufValue::INT; v->i = c.get<uint8_t>(); break;  // bools read as 0/1 ints
        case 8: v->kind = GgufValue::STR; v->s = c.str(); break;
        case 9: {
            const uint32_t et = c.get<uint32_t>();
            const uint64_t n = c.get<uint64_t>();
            if (et == 4 && n <= 1024) {  // small u32 arrays are kept (metadata.rs:403-409)
                v->kind = GgufValue::U32ARR;
                for (uint64_t i = 0; i < n && c.ok; ++i) v->arr.push_back(c.get<uint32_t>());
                break;
            }
            v->kind = GgufValue::SKIPPED;  // vocabulary, merges, scores...: walked over, not kept
            if (et == 8) {
                for (uint64_t i = 0; i < n && c.ok; ++i) {
                    const uint64_t sl = c.get<uint64_t>();
                    if (c.need(sl)) c.p += sl;
                }
            } else if (const int w = gguf_scalar_bytes(et)) {
                if (n > (uint64_t)(c.end - c.p) / (uint64_t)w) c.ok = false;
                else c.p += n * (uint64_t)w;
            } else {
                c.ok = false;  // nested arrays / unknown element types
            }
            break;
        }
        case 10: v->kind = GgufValue::UINT; v->u = c.get<uint64_t>(); break;
        case 11: v->kind = GgufValue::INT; v->i = c.get<int64_t>(); break;
        case 12: v->kind = GgufValue::FLOAT; v->f = c.get<double>(); break;
        default: c.ok = false;
    }
    return c.ok;
}

const GgufValue *gguf_field(const apk_gguf *f, const char *key) {
    auto it = f->field_index.find(key);
    return it == f->field_index.end() ? nullptr : &f->fields[it->second].second;
}

}  // namespace

int apk_gguf_open(const char *path, apk_gguf **out) {
    if (!path || !out) return fail(APK_ERR_INVALID_ARG, "gguf_open: null argument");
    auto f = std::make_unique<apk_gguf>();
    f->fd = open(path, O_RDONLY);
    if (f->fd < 0) return fail(APK_ERR_INVALID_ARG, "gguf_open: cannot open %s", path);
    struct stat st;
    if (fstat(f->fd, &st) != 0 || st.st_size < 24) return fail(APK_ERR_INVALID_ARG, "gguf_open: %s is not a GGUF file (too short)", path);
    f->len = (size_t)st.st_size;
    void *m = mmap(nullptr, f->len, PROT_READ, MAP_PRIVATE, f->fd, 0);
    if (m == MAP_FAILED) return fail(APK_ERR_INVALID_ARG, "gguf_open: mmap of %s failed", path);
    f->map = (const uint8_t *)m;
    GgufCursor c{f->map, f->map + f->len};
    if (memcmp(c.p, "GGUF", 4) != 0) return fail(APK_ERR_INVALID_ARG, "gguf_open: %s has no GGUF magic", path);
    c.p += 4;
    f->version = c.get<uint32_t>();
    if (f->version < 2) return fail(APK_ERR_INVALID_ARG, "gguf_open: GGUF version %u is not supported", f->version);
    const uint64_t n_tensors = c.get<uint64_t>(), n_kv = c.get<uint64_t>();
    uint64_t alignment = 32;  // when the file does not carry general.alignment
    for (uint64_t i = 0; i < n_kv; ++i) {
        std::string key = c.str();
        GgufValue v;
        if (!c.ok || !gguf_read_value(c, &v)) return fail(APK_ERR_INVALID_ARG, "gguf_open: metadata entry %llu is malformed or truncated", (unsigned long long)i);
        if (key == "general.architecture" && v.kind == GgufValue::STR) f->arch = v.s;
        if (key == "general.alignment" && v.kind == GgufValue::UINT && v.u > 0) alignment = v.u;
        f->field_index[key] = f->fields.size();
        f->fields.emplace_back(std::move(key), std::move(v));
    }
    for (uint64_t i = 0; i < n_tensors; ++i) {
        GgufTensor t;
        t.name = c.str();
        t.n_dims = c.get<uint32_t>();
        if (!c.ok || t.n_dims > 4) return fail(APK_ERR_INVALID_ARG, "gguf_open: tensor %llu claims %u dimensions; GGUF allows at most 4", (unsigned long long)i, t.n_dims);
        for (uint32_t d = 0; d < t.n_dims; ++d) t.dims[d] = c.get<uint64_t>();
        t.ty = c.get<uint32_t>();
        t.offset = c.get<uint64_t>();
        if (!c.ok) return fail(APK_ERR_INVALID_ARG, "gguf_open: the tensor table is truncated at entry %llu", (unsigned long long)i);
        uint64_t elements = 1;
        bool overflow = false;
        for (uint32_t d = 0; d < t.n_dims; ++d) {
            if (t.dims[d] != 0 && elements > UINT64_MAX / t.dims[d]) overflow = true;
            elements *= t.dims[d];
        }
        if (overflow) return fail(APK_ERR_INVALID_ARG, "gguf_open: tensor %s: size overflows", t.name.c_str());
        if (!gguf_type_bytes(t.ty, elements, &t.n_bytes)) t.n_bytes = 0;
        f->tensor_index[t.name] = f->tensors.size();
        f->tensors.push_back(std::move(t));
    }
    // the data section starts at the next aligned position after the header
    const uint64_t here = (uint64_t)(c.p - f->map);
    f->data_offset = (here + alignment - 1) / alignment * alignment;
    for (const GgufTensor &t : f->tensors) {
        // "claims bytes a..b, but the file has only n" (tensors.rs:199-213)
        if (t.offset > f->len || f->data_offset > f->len - t.offset || t.n_bytes > f->len - t.offset - f->data_offset)
            return fail(APK_ERR_INVALID_ARG, "gguf_open: tensor %s claims bytes %llu..%llu, but the file has only %zu", t.name.c_str(),
                        (unsigned long long)(f->data_offset + t.offset), (unsigned long long)(f->data_offset + t.offset + t.n_bytes), f->len);
    }
    *out = f.release();
    return APK_OK;
}

void apk_gguf_close(apk_gguf *f) { delete f; }

uint64_t apk_gguf_n_tensors(const apk_gguf *f) { return f ? f->tensors.size() : 0; }

static void gguf_fill(const apk_gguf *f, const GgufTensor &t, apk_gguf_tensor *out) {
    out->name = t.name.c_str();
    out->ty = t.ty;
    out->n_dims = t.n_dims;
    for (int d = 0; d < 4; ++d) out->dims[d] = t.dims[d];
    out->data = f->map + f->data_offset + t.offset;
    out->n_bytes = t.n_bytes;
}

int apk_gguf_tensor_at(const apk_gguf *f, uint64_t i, apk_gguf_tensor *out) {
    if (!f || !out || i >= f->tensors.size()) return fail(APK_ERR_INVALID_ARG, "gguf_tensor_at: index out of range");
    gguf_fill(f, f->tensors[i], out);
    return APK_OK;
}

int apk_gguf_find(const apk_gguf *f, const char *name, apk_gguf_tensor *out) {
    if (!f || !name || !out) return fail(APK_ERR_INVALID_ARG, "gguf_find: null argument");
    auto it = f->tensor_index.find(name);
    if (it == f->tensor_index.end()) return fail(APK_DECLINE_INVALID_STATE, "GGUF has no tensor \"%s\"", name);
    gguf_fill(f, f->tensors[it->second], out);
    return APK_OK;
}

const char *apk_gguf_architecture(const apk_gguf *f) { return f ? f->arch.c_str() : ""; }

int apk_gguf_meta_u32(const apk_gguf *f, const char *key, uint32_t *out) {
    const GgufValue *v = (f && key) ? gguf_field(f, key) : nullptr;
    if (!v || !out) return APK_DECLINE_INVALID_STATE;
    if (v->kind == GgufValue::UINT && v->u <= UINT32_MAX) *out = (uint32_t)v->u;
    else if (v->kind == GgufValue::INT && v->i >= 0 && v->i <= (int64_t)UINT32_MAX) *out = (uint32_t)v->i;
    else return APK_DECLINE_INVALID_STATE;
    return APK_OK;
}

int apk_gguf_meta_f32(const apk_gguf *f, const char *key, float *out) {
    const GgufValue *v = (f && key) ? gguf_field(f, key) : nullptr;
    if (!v || !out || v->kind != GgufValue::FLOAT) return APK_DECLINE_INVALID_STATE;
    *out = (float)v->f;
    return APK_OK;
}

const char *apk_gguf_meta_str(const apk_gguf *f, const char *key) {
    const GgufValue *v = (f && key) ? gguf_field(f, key) : nullptr;
    return (v && v->kind == GgufValue::STR) ? v->s.c_str() : nullptr;
}

const void *apk_gguf_mapping(const apk_gguf *f, uint64_t *len) {
    if (!f) return nullptr;
    if (len) *len = f->len;
    return f->map;
}

// ---------------------------------------------------------------- the dense-decoder view

struct apk_model {
    apk_gguf *file = nullptr;
    apk_model_info info{};
    std::vector<apk_token_layer> layers;
    const float *output_norm = nullptr;
    apk_mat output{}, embd{};
    std::vector<std::unique_ptr<uint8_t[]>> owned;       // reordered Q / K matrices
    std::vector<std::pair<const void *, size_t>> owned_spans;
    apk_ctx *attached_to = nullptr;
};

namespace {

int model_mat(const apk_gguf *f, const std::string &name, uint64_t n_out, uint64_t n_in, apk_mat *out) {
    // qmat (loader.rs:558-569): a silently transposed tensor produces plausible garbage; a named
    // shape error produces a fix
    auto it = f->tensor_index.find(name);
    if (it == f->tensor_index.end()) return fail(APK_DECLINE_INVALID_STATE, "GGUF has no tensor \"%s\"", name.c_str());
    const GgufTensor &t = f->tensors[it->second];
    if (t.n_dims != 2 || t.dims[0] != n_in || t.dims[1] != n_out)
        return fail(APK_DECLINE_UNSUPPORTED_SHAPE, "tensor \"%s\" has shape [%llu, %llu], expected [%llu, %llu]", name.c_str(),
                    (unsigned long long)t.dims[0], (unsigned long long)t.dims[1], (unsigned long long)n_in, (unsigned long long)n_out);
    uint32_t be, bb;
    if (!block_geom(t.ty, &be, &bb)) return fail(APK_DECLINE_UNSUPPORTED_TYPE, "tensor \"%s\": ggml type %u has no kernel", name.c_str(), t.ty);
    out->ty = t.ty;
    out->w = f->map + f->data_offset + t.offset;
    out->n_out = (uint32_t)n_out;
    return APK_OK;
}

int model_vec(const apk_gguf *f, const std::string &name, uint64_t n, const float **out, bool optional = false) {
    auto it = f->tensor_index.find(name);
    if (it == f->tensor_index.end()) {
        if (optional) { *out = nullptr; return APK_OK; }
        return fail(APK_DECLINE_INVALID_STATE, "GGUF has no tensor \"%s\"", name.c_str());
    }
    const GgufTensor &t = f->tensors[it->second];
    // norm_raw (loader.rs:573-580): the GPU binds F32 norm vectors directly out of the mapping
    if (t.ty != 0) return fail(APK_DECLINE_UNSUPPORTED_TYPE, "tensor \"%s\" is not F32", name.c_str());
    uint64_t elements = 1;
    for (uint32_t d = 0; d < t.n_dims; ++d) elements *= t.dims[d];
    if (elements != n) return fail(APK_DECLINE_UNSUPPORTED_SHAPE, "tensor \"%s\" has %llu elements, expected %llu", name.c_str(),
                                   (unsigned long long)elements, (unsigned long long)n);
    const uint8_t *p = f->map + f->data_offset + t.offset;
    if ((uintptr_t)p % 4) return fail(APK_DECLINE_INVALID_STATE, "tensor \"%s\" is not 4-byte aligned in the file", name.c_str());
    *out = (const float *)p;
    return APK_OK;
}

// reorder_head_rows (loader.rs:395-426): a copy of the matrix with the rows of every head taken in
// `order` (new row -> old row within the head).  Rows are whole quantised blocks, so this moves
// bytes and changes no value.
int reorder_head_rows(apk_model *M, apk_mat *m, uint64_t n_in, const std::vector<uint32_t> &order) {
    uint32_t be, bb;
    block_geom(m->ty, &be, &bb);
    const size_t row = (size_t)(n_in / be) * bb, hd = order.size();
    if (hd == 0 || m->n_out % hd) return fail(APK_DECLINE_UNSUPPORTED_SHAPE, "cannot reorder %u rows in heads of %zu", m->n_out, hd);
    const size_t bytes = row * m->n_out;
    std::unique_ptr<uint8_t[]> buf(new uint8_t[bytes]);
    const uint8_t *src = (const uint8_t *)m->w;
    for (size_t head = 0; head < m->n_out / hd; ++head)
        for (size_t nw = 0; nw < hd; ++nw)
            memcpy(buf.get() + (head * hd + nw) * row, src + (head * hd + order[nw]) * row, row);
    m->w = buf.get();
    M->owned_spans.emplace_back(buf.get(), bytes);
    M->owned.push_back(std::move(buf));
    return APK_OK;
}

}  // namespace

int apk_model_open(apk_gguf *f, apk_model **out) {
    if (!f || !out) return fail(APK_ERR_INVALID_ARG, "model_open: null argument");
    auto M = std::make_unique<apk_model>();
    M->file = f;
    apk_model_info &I = M->info;
    const std::string arch = f->arch;
    auto key = [&](const char *suffix) { return arch + "." + suffix; };
    auto need = [&](const char *suffix, uint32_t *v) {
        if (apk_gguf_meta_u32(f, key(suffix).c_str(), v) != APK_OK) return fail(APK_DECLINE_INVALID_STATE, "GGUF has no %s", key(suffix).c_str());
        return (int)APK_OK;
    };
    // Config::from_gguf (config.rs:184-310), the fields of a dense attention decoder
    APK_TRY(need("attention.head_count", &I.n_heads));
    APK_TRY(need("embedding_length", &I.hidden));
    if (I.n_heads == 0) return fail(APK_DECLINE_UNSUPPORTED_SHAPE, "attention.head_count is 0");
    if (apk_gguf_meta_u32(f, key("attention.key_length").c_str(), &I.head_dim) != APK_OK) I.head_dim = I.hidden / I.n_heads;
    auto e = f->tensor_index.find("token_embd.weight");
    if (e == f->tensor_index.end()) return fail(APK_DECLINE_INVALID_STATE, "GGUF has no token_embd.weight tensor");
    const GgufTensor &embd = f->tensors[e->second];
    if (embd.n_dims != 2 || embd.dims[0] != I.hidden)
        return fail(APK_DECLINE_UNSUPPORTED_SHAPE, "token_embd.weight has shape [%llu, %llu], expected [%u, vocab]",
                    (unsigned long long)embd.dims[0], (unsigned long long)embd.dims[1], I.hidden);
    I.vocab = (uint32_t)embd.dims[1];
    if (apk_gguf_meta_u32(f, key("rope.dimension_count").c_str(), &I.rot_dim) != APK_OK) I.rot_dim = I.head_dim;
    I.rot_dim = std::min(I.rot_dim, I.head_dim);
    if (I.rot_dim == 0 || I.rot_dim % 2) return fail(APK_DECLINE_UNSUPPORTED_SHAPE, "rope.dimension_count %u must be a positive even number", I.rot_dim);
    APK_TRY(need("block_count", &I.n_layers));
    // converters may count blocks whose tensors they do not write: trim them (config.rs:258-264)
    while (I.n_layers > 0 && !f->tensor_index.count("blk." + std::to_string(I.n_layers - 1) + ".attn_q.weight")) --I.n_layers;
    if (I.n_layers == 0) return fail(APK_DECLINE_INVALID_STATE, "GGUF has no attention blocks");
    if (apk_gguf_meta_u32(f, key("attention.head_count_kv").c_str(), &I.n_kv_heads) != APK_OK) I.n_kv_heads = I.n_heads;
    if (apk_gguf_meta_u32(f, key("feed_forward_length").c_str(), &I.ffn) != APK_OK) I.ffn = 0;
    if (apk_gguf_meta_f32(f, key("attention.layer_norm_rms_epsilon").c_str(), &I.eps) != APK_OK) I.eps = 1e-5f;
    if (apk_gguf_meta_f32(f, key("rope.freq_base").c_str(), &I.rope_base) != APK_OK) I.rope_base = 10000.0f;
    uint32_t n_expert = 0;
    if (apk_gguf_meta_u32(f, key("expert_count").c_str(), &n_expert) == APK_OK && n_expert > 0)
        return fail(APK_DECLINE_MISSING_CAPABILITY, "mixture-of-experts files are outside the dense decode path");
    if (f->tensor_index.count("blk.0.attn_q.bias")) return fail(APK_DECLINE_MISSING_CAPABILITY, "projection biases are outside the dense decode path");
    bool has_qk_norm = false;
    for (uint32_t l = 0; l < I.n_layers; ++l) has_qk_norm |= f->tensor_index.count("blk." + std::to_string(l) + ".attn_q_norm.weight") > 0;
    I.has_qk_norm = has_qk_norm ? 1 : 0;
    // neox_order (loader.rs:366-390): llama / mistral files store Q and K rows for pairwise (NORM) rotation;
    // taking them in the order 0, 2, 4, ..., 1, 3, 5, ... makes the same rotation the NEOX one the kernels apply
    const bool norm_style = arch == "llama" || arch == "mistral";
    const char *keep = getenv("ALLPAKA_ROPE_NORM");
    std::vector<uint32_t> order;
    if (norm_style && !has_qk_norm && !(keep && keep[0] == '1' && keep[1] == 0)) {
        const uint32_t half = I.rot_dim / 2;
        for (uint32_t nw = 0; nw < I.head_dim; ++nw)
            order.push_back(nw < half ? 2 * nw : (nw < I.rot_dim ? 2 * (nw - half) + 1 : nw));
    } else if (norm_style) {
        // the reference then rotates adjacent pairs at run time (per-head norms, or ALLPAKA_ROPE_NORM=1); the kernels here
        // rotate split halves only
        return fail(APK_DECLINE_MISSING_CAPABILITY, "pairwise rotary embedding kept in file order is outside the decode path");
    }
    I.neox_reordered = order.empty() ? 0 : 1;
    const uint64_t q_dim = (uint64_t)I.n_heads * I.head_dim, kv_dim = (uint64_t)I.n_kv_heads * I.head_dim;
    M->layers.resize(I.n_layers);
    for (uint32_t l = 0; l < I.n_layers; ++l) {
        apk_token_layer &L = M->layers[l];
        auto name = [&](const char *part) { return "blk." + std::to_string(l) + "." + part + ".weight"; };
        APK_TRY(model_vec(f, name("attn_norm"), I.hidden, &L.attn_norm));
        // GLM calls the pre-FFN norm "post_attention_norm" (loader.rs:107-113)
        const std::string ffn_norm = f->tensor_index.count(name("ffn_norm")) ? name("ffn_norm") : name("post_attention_norm");
        APK_TRY(model_vec(f, ffn_norm, I.hidden, &L.ffn_norm));
        APK_TRY(model_mat(f, name("attn_q"), q_dim, I.hidden, &L.wq));
        APK_TRY(model_mat(f, name("attn_k"), kv_dim, I.hidden, &L.wk));
        APK_TRY(model_mat(f, name("attn_v"), kv_dim, I.hidden, &L.wv));
        APK_TRY(model_mat(f, name("attn_output"), I.hidden, q_dim, &L.wo));
        if (!order.empty()) {
            APK_TRY(reorder_head_rows(M.get(), &L.wq, I.hidden, order));
            APK_TRY(reorder_head_rows(M.get(), &L.wk, I.hidden, order));
        }
        APK_TRY(model_vec(f, name("attn_q_norm"), I.head_dim, &L.q_norm, true));
        APK_TRY(model_vec(f, name("attn_k_norm"), I.head_dim, &L.k_norm, true));
        APK_TRY(model_mat(f, name("ffn_gate"), I.ffn, I.hidden, &L.gate));
        APK_TRY(model_mat(f, name("ffn_up"), I.ffn, I.hidden, &L.up));
        APK_TRY(model_mat(f, name("ffn_down"), I.hidden, I.ffn, &L.down));
    }
    APK_TRY(model_vec(f, "output_norm.weight", I.hidden, &M->output_norm));
    APK_TRY(model_mat(f, "token_embd.weight", I.vocab, I.hidden, &M->embd));
    // tied embeddings: no output.weight, the table is the LM head (loader.rs:207-211)
    if (f->tensor_index.count("output.weight")) {
        APK_TRY(model_mat(f, "output.weight", I.vocab, I.hidden, &M->output));
        I.tied = 0;
    } else {
        M->output = M->embd;
        I.tied = 1;
    }
    *out = M.release();
    return APK_OK;
}

const apk_model_info *apk_model_get_info(const apk_model *m) { return m ? &m->info : nullptr; }

int apk_model_token_req(const apk_model *m, apk_token_req *req) {
    if (!m || !req) return fail(APK_ERR_INVALID_ARG, "model_token_req: null argument");
    memset(req, 0, sizeof(*req));
    req->layers = m->layers.data();
    req->n_layers = m->info.n_layers;
    req->output_norm = m->output_norm;
    req->output = m->output;
    req->embd = m->embd;
    req->m = 1;
    req->rot_dim = m->info.rot_dim;
    req->eps = m->info.eps;
    req->hidden = m->info.hidden;
    req->head_dim = m->info.head_dim;
    req->n_heads = m->info.n_heads;
    req->n_kv_heads = m->info.n_kv_heads;
    req->attn_core = APK_ATTN_CAUSAL;
    req->scale = 1.0f / sqrtf((float)m->info.head_dim);
    return APK_OK;
}

int apk_model_attach(apk_ctx *c, apk_model *m) {
    if (!c || !m) return fail(APK_ERR_INVALID_ARG, "model_attach: null argument");
    if (m->attached_to) return fail(APK_DECLINE_INVALID_STATE, "model_attach: the model is attached already");
    // the whole mapping, like gpu::attach on the GgufFile's mmap (loader.rs:62-98), and every
    // reordered copy, offered to the GPU like any other weight (loader.rs:421)
    APK_TRY(apk_attach(c, m->file->map, m->file->len));
    for (auto &s : m->owned_spans) APK_TRY(apk_attach(c, s.first, s.second));
    m->attached_to = c;
    return APK_OK;
}

void apk_model_close(apk_model *m) {
    if (!m) return;
    if (m->attached_to) {
        apk_detach(m->attached_to, m->file->map, m->file->len);
        for (auto &s : m->owned_spans) apk_detach(m->attached_to, s.first, s.second);
    }
    delete m;
}
