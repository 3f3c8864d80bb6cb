// libapk_b200.so: host side of the C ABI declared in include/allpaka_b200.h.
//
// Plain CUDA runtime; no PyTorch, no CPU compute fallback.  One context = one
// GPU.  Weights are addressed by host pointer inside attached mappings, as the
// reference CUDA backend does (crates/allpaka-backend/src/gpu/cuda/runtime/
// select.rs:80-84, device.rs:588-621), and live on the device as the tiled
// stream described in kernels.cuh.
#include "../../include/allpaka_b200.h"
#include "kernels.cuh"
#include "mv_pick.h"

#include <dlfcn.h>

#include <algorithm>
#include <chrono>
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <map>
#include <memory>
#include <mutex>
#include <string>
#include <tuple>
#include <vector>

using namespace apk;

namespace {

thread_local char g_last_error[512] = "";  // fixed storage: reporting an error never touches the heap

int fail(int code, const char *fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_last_error, sizeof g_last_error, fmt, ap);
    va_end(ap);
    return code;
}

#define CUDA_TRY(expr)                                                                          \
    do {                                                                                        \
        cudaError_t e__ = (expr);                                                               \
        if (e__ != cudaSuccess)                                                                 \
            return fail(e__ == cudaErrorMemoryAllocation ? APK_ERR_OOM : APK_ERR_CUDA,          \
                        "%s: %s (%s:%d)", #expr, cudaGetErrorString(e__), __FILE__, __LINE__); \
    } while (0)

#define APK_TRY(expr)          \
    do {                       \
        int rc__ = (expr);     \
        if (rc__) return rc__; \
    } while (0)

uint64_t now_ns() {
    return (uint64_t)std::chrono::duration_cast<std::chrono::nanoseconds>(
               std::chrono::steady_clock::now().time_since_epoch())
        .count();
}

bool block_geom(uint32_t ty, uint32_t *be, uint32_t *bb) {
    // crates/allpaka-dtype/src/lib.rs:79-108
    if (ty == APK_TY_Q8_0) { *be = 32; *bb = 34; return true; }
    if (ty == APK_TY_Q5_0) { *be = 32; *bb = 22; return true; }
    if (ty == APK_TY_Q4_K) { *be = 256; *bb = 144; return true; }
    if (ty == APK_TY_Q5_K) { *be = 256; *bb = 176; return true; }
    if (ty == APK_TY_Q6_K) { *be = 256; *bb = 210; return true; }
    if (ty == APK_TY_Q3_K) { *be = 256; *bb = 110; return true; }
    if (ty == APK_TY_Q2_K) { *be = 256; *bb = 84; return true; }
    return false;
}

// The format a matrix has in device memory: Q3_K is rewritten into the Q6_K stream at load (same
// sub-block structure and arithmetic, see repack_q6_k_kernel<true>), every other type keeps its own.
uint32_t stream_ty(uint32_t ty) { return ty == APK_TY_Q3_K ? APK_TY_Q6_K : ty; }

// A device buffer that only ever grows (never while a graph that uses it exists).
struct DevBuf {
    void *p = nullptr;
    size_t cap = 0;
    int ensure(size_t bytes, bool zero = false) {
        if (bytes <= cap) return APK_OK;
        if (p) cudaFree(p);
        p = nullptr;
        cap = 0;
        const size_t want = std::max(bytes, (size_t)4096);
        CUDA_TRY(cudaMalloc(&p, want));
        cap = want;
        if (zero) CUDA_TRY(cudaMemset(p, 0, want));
        return APK_OK;
    }
    void release() {
        if (p) cudaFree(p);
        p = nullptr;
        cap = 0;
    }
    template <class T> T *as() const { return reinterpret_cast<T *>(p); }
};

// One source of rows for a device matrix: rows [row0, row0+rows) and 32-element
// blocks starting at kblk0 of the host matrix at `w`; segment row r lands at
// destination row (r / group) * stride + offset + r % group.
struct Segment {
    const void *w;
    uint32_t n_in_full;
    uint32_t row0, rows;
    uint32_t kblk0;
    int group, stride, offset;
};

struct DevMatrix {
    uint32_t ty = 0;      // format of the device stream (picks the kernel)
    uint32_t src_ty = 0;  // format of the host bytes it was built from
    uint32_t n_out = 0, n_in = 0;  // of the device matrix (after sharding / fusing)
    int nb = 0, n_tiles = 0, KS = 0;
    uint32_t tile_bytes = 0;
    size_t bytes = 0;
    uint8_t *d = nullptr;
    std::vector<std::pair<const uint8_t *, size_t>> host_spans;  // for detach
    ~DevMatrix() {
        if (d) cudaFree(d);
    }
};

// (kind, p0, p1, p2, ty, n_out, n_in, shard kind, shard index * 64 + world)
typedef std::tuple<int, const void *, const void *, const void *, uint32_t, uint32_t, uint32_t, int, int> MatKey;
enum { KIND_PLAIN = 0, KIND_QKV = 1, KIND_GATEUP = 2 };
enum { SHARD_NONE = 0, SHARD_ROWS = 1, SHARD_K = 2 };

// ---- NCCL through dlopen: only tensor-parallel runs need the library ---------
struct Nccl {
    void *h = nullptr;
    struct uid_t { char internal[128]; };
    int (*GetUniqueId)(uid_t *) = nullptr;
    int (*CommInitRank)(void **, int, uid_t, int) = nullptr;
    int (*CommDestroy)(void *) = nullptr;
    int (*AllReduce)(const void *, void *, size_t, int, int, void *, cudaStream_t) = nullptr;
    int (*AllGather)(const void *, void *, size_t, int, void *, cudaStream_t) = nullptr;
    const char *(*GetErrorString)(int) = nullptr;
    bool load() {
        if (h) return true;
        h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
        if (!h) return false;
        GetUniqueId = (decltype(GetUniqueId))dlsym(h, "ncclGetUniqueId");
        CommInitRank = (decltype(CommInitRank))dlsym(h, "ncclCommInitRank");
        CommDestroy = (decltype(CommDestroy))dlsym(h, "ncclCommDestroy");
        AllReduce = (decltype(AllReduce))dlsym(h, "ncclAllReduce");
        AllGather = (decltype(AllGather))dlsym(h, "ncclAllGather");
        GetErrorString = (decltype(GetErrorString))dlsym(h, "ncclGetErrorString");
        return GetUniqueId && CommInitRank && CommDestroy && AllReduce && AllGather && GetErrorString;
    }
};
Nccl g_nccl;
constexpr int NCCL_FLOAT32 = 7;  // ncclFloat32
constexpr int NCCL_SUM = 0;      // ncclSum

struct RecMeta { int ke, m_eff, two_level, launch; };

}  // namespace

// The f16 KV cache of a session (this rank's kv heads): K slabs of every layer, then the V slabs.
struct apk_kv {
    uint32_t n_layers = 0, kv_dim = 0, capacity = 0;  // kv_dim: this rank's
    __half *base = nullptr;
    size_t layer_stride() const { return (size_t)kv_dim * capacity; }
    __half *k(uint32_t layer) const { return base + layer_stride() * layer; }
    __half *v(uint32_t layer) const { return base + layer_stride() * (n_layers + layer); }
};

namespace {

struct PlanLayer {
    DevMatrix *qkv = nullptr, *wo = nullptr, *gateup = nullptr, *down = nullptr;
    DevMatrix *v = nullptr;  // V as a matrix of its own when its type differs from Q and K (qkv is then Q | K)
    const float *attn_norm = nullptr, *ffn_norm = nullptr, *q_norm = nullptr, *k_norm = nullptr;  // device
};

struct Plan {
    // identity of the request this plan was built for
    const apk_token_layer *layers_key = nullptr;
    uint32_t n_layers = 0;
    const void *output_key = nullptr;
    uint64_t desc_hash = 0;  // every layer's descriptors (weight and norm pointers, types, row counts)
    uint32_t hidden = 0, head_dim = 0, n_heads = 0, n_kv_heads = 0, rot_dim = 0, vocab = 0, ffn = 0;
    float eps = 0;
    uint32_t attn_core = 0;
    const apk_kv *kv = nullptr;
    float scale = 0;
    // local (per-rank) shapes
    uint32_t nq_l = 0, nkv_l = 0, ffn_l = 0, vocab_l = 0;
    std::vector<PlanLayer> L;
    DevMatrix *head = nullptr;
    DevMatrix *embd = nullptr;  // token embedding table (unsharded), when the request names one
    const float *out_norm = nullptr;
    DevBuf norms, xin, x[2], qkv, yp, act_h, act_q, act_d, logits, logits_all, amax, rope, sumsq, hidden_out;
    DevBuf chain;  // greedy chain state: token | step | hist[] | rope rows
    DevBuf pos, attn_part, attn_out;  // cache position of row 0; split partials and f32 rows of the attention core
    cudaGraphExec_t exec[APK_MAX_M + 1][2] = {};  // [m][argmax]
    int launches[APK_MAX_M + 1][2] = {};
    ~Plan() {
        for (auto &row : exec)
            for (auto &e : row)
                if (e) cudaGraphExecDestroy(e);
        for (DevBuf *b : {&norms, &xin, &x[0], &x[1], &qkv, &yp, &act_h, &act_q, &act_d, &logits, &logits_all, &amax, &rope, &sumsq, &hidden_out, &chain, &pos, &attn_part, &attn_out})
            b->release();
    }
};

}  // namespace

struct apk_ctx {
    std::mutex mu;
    int device = 0;
    int n_sm = 0;
    int smem_optin = 0;
    cudaStream_t stream = nullptr;
    // A V projection with a type of its own runs beside the Q | K launch on a few SMs of its own
    // (ALLPAKA_B200_FORK_V=0: after it, like every other launch): a second stream forked and joined
    // with events, which capture turns into two branches of the token graph.
    cudaStream_t side = nullptr;
    cudaEvent_t ev_fork = nullptr, ev_join = nullptr;
    cudaStream_t launch_stream = nullptr;  // where launch_ex puts the next kernels (null: stream)
    int grid_cap = 0;                      // most CTAs the next matvec launches may take (0: no cap)
    int fork_v = 4;                        // CTAs per V tile of that branch (0: no branch); measured 1 / 2 / 4: 168 / 175 / 178 tok/s
    cudaEvent_t ev0 = nullptr, ev1 = nullptr;
    std::map<std::pair<const uint8_t *, size_t>, int> attached;  // (base,len) -> refcount
    std::map<MatKey, std::unique_ptr<DevMatrix>> mats;
    DevBuf staging;             // raw GGUF rows on their way to the repack
    DevBuf partials;            // stream-K fix-up scratch
    int *d_err = nullptr;       // device error word
    int *h_err = nullptr;       // pinned mirror
    DevBuf x_dev, y_dev, act_a, act_b, misc, dump;
    unsigned long long *trace = nullptr;  // when set: every matvec launch stamps its own [n_sm][8] slab
    uint32_t trace_idx = 0, trace_cap = 0;
    apk_stats_t st{};
    int rank = 0, world = 1;
    // How a residual matvec (wo, down) helps the RMSNorm that reads its result (ALLPAKA_B200_FUSE_NORM):
    //  0 nothing; 1 (default) it leaves the per-block sums of squares, the reader still quantises
    //  f32(f64(x)*scale)*gamma itself (exact); 2 it also quantises x*gamma per tile and the reader only
    //  applies the row scale (cheaper; codes may differ by one at a .5 boundary); 3 like 2 for m > 1, like 1 at m = 1
    int fuse_norm = 1;
    long long wait_limit = WAIT_LIMIT_DEFAULT;  // cycle budget of the bounded device-side waits (apk_debug_set_wait_limit)
    bool self_xch = false;       // ALLPAKA_B200_SELF_XCH=1: a single rank runs the peer-exchange path on itself (one-GPU test of it)
    // parity instrumentation (apk_debug_token_records): one slab per matvec launch that reads the residual through a norm
    uint8_t *rec_dump = nullptr;
    size_t rec_slab = 0;
    uint32_t rec_idx = 0, rec_cap = 0;
    int32_t *dots_dump = nullptr;  // block dots of launch dots_launch
    size_t dots_cap = 0;
    int dots_launch = -1, launch_no = 0;
    int attn_tc = 1;             // ALLPAKA_B200_ATTN_TC=0: the attention core on CUDA cores instead of tensor cores
    bool attn_tc_ready = false;
    int attn_min_pos = 256;      // ALLPAKA_B200_ATTN_MIN_POS: fewest cache positions a split of the attention core is sized for
    int tl_alt = 0;              // ALLPAKA_B200_TL_ALT=1: the timeline stamps the closing of each CTA's last tile
    bool prev_mv_exclusive = false;  // the last matvec launched holds every SM to itself (see launch_matvec)
    int smem_per_sm = 0;
    std::vector<RecMeta> rec_meta;
    bool use_pdl = true;        // ALLPAKA_B200_PDL=0 turns programmatic dependent launch off
    void *comm = nullptr;
    std::unique_ptr<Plan> plan;
    float *xch_local = nullptr;     // this rank's exchange buffer (apk_dist_p2p_export)
    XchPeers xch{};                 // every rank's buffer, peer-mapped
    bool p2p_open = false;       // every rank's exchange buffer is mapped here
    bool p2p_ready = false;      // peer buffers are mapped and the peer exchange is switched on
    int inflight = 3;            // K-steps of weights a CTA keeps outstanding (ALLPAKA_B200_INFLIGHT overrides, for tuning)
    int inflight_pre = 2;        // ... while the previous kernel is still finishing (ALLPAKA_B200_INFLIGHT_PRE)
    // host address -> device-resident raw GGUF bytes written by apk_debug_synth_matrix
    std::map<const uint8_t *, std::pair<uint8_t *, size_t>> raw_dev;
};

namespace {

// ------------------------------------------------------------ kernel table

MvKernel pick_kernel(uint32_t ty, int m_eff, bool dump) {
    if (ty == APK_TY_Q8_0) return mv_pick_q8_0(m_eff, dump);
    if (ty == APK_TY_Q5_0) return mv_pick_q5_0(m_eff, dump);
    if (ty == APK_TY_Q4_K) return mv_pick_q4_k(m_eff, dump);
    if (ty == APK_TY_Q5_K) return mv_pick_q5_k(m_eff, dump);
    if (ty == APK_TY_Q6_K) return mv_pick_q6_k(m_eff, dump);
    if (ty == APK_TY_Q2_K) return mv_pick_q2_k(m_eff, dump);
    return nullptr;
}

int init_kernel_attrs(apk_ctx *c) {
    static const int ms[] = {1, 2, 3, 4, 5, 6, 7, 8, 10, 12, 14, 16};
    for (uint32_t ty : {APK_TY_Q8_0, APK_TY_Q5_0, APK_TY_Q2_K, APK_TY_Q4_K, APK_TY_Q5_K, APK_TY_Q6_K})
        for (int m : ms)
            for (int dump = 0; dump < 2; ++dump) {
                MvKernel k = pick_kernel(ty, m, dump != 0);
                CUDA_TRY(cudaFuncSetAttribute((const void *)k, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                              c->smem_optin));
            }
    return APK_OK;
}

int ke_of(uint32_t ty) { return ty_k45((int)ty) ? 512 : 256; }
// consumers whose min term multiplies the exact f32 block sums of the activations (q8_acts.rs:257-258, 296-297)
bool needs_sum(uint32_t ty) { return ty_k45((int)ty); }

// --------------------------------------------------------------- matrices

bool inside_attached(apk_ctx *c, const void *p, size_t len) {
    const uint8_t *b = (const uint8_t *)p;
    for (auto &kv : c->attached) {
        const uint8_t *base = kv.first.first;
        if (b >= base && b + len <= base + kv.first.second) return true;
    }
    return false;
}

size_t host_bytes(uint32_t ty, uint32_t n_out, uint32_t n_in) {
    uint32_t be, bb;
    if (!block_geom(ty, &be, &bb)) return 0;
    return (size_t)n_out * (n_in / be) * bb;
}

// Device-resident stand-in for host bytes [p, p+len), if a generator put one there.
const uint8_t *raw_lookup(apk_ctx *c, const uint8_t *p, size_t len) {
    auto it = c->raw_dev.upper_bound(p);
    if (it == c->raw_dev.begin()) return nullptr;
    --it;
    if (p >= it->first && p + len <= it->first + it->second.second) return it->second.first + (p - it->first);
    return nullptr;
}

// Build a device matrix of n_out x n_in from row segments of host matrices.
int build_matrix(apk_ctx *c, uint32_t ty, uint32_t n_out, uint32_t n_in, const std::vector<Segment> &segs,
                 std::unique_ptr<DevMatrix> *out) {
    uint32_t be, bb;
    if (!block_geom(ty, &be, &bb)) return fail(APK_DECLINE_UNSUPPORTED_TYPE, "ggml type %u has no kernel", ty);
    if (n_in == 0 || n_out == 0 || n_in % be)
        return fail(APK_DECLINE_UNSUPPORTED_SHAPE, "row length %u is not whole %u-element blocks", n_in, be);
    auto m = std::make_unique<DevMatrix>();
    m->src_ty = ty;
    const uint32_t src_ty = ty;
    ty = stream_ty(ty);
    m->ty = ty;
    m->n_out = n_out;
    m->n_in = n_in;
    m->nb = (int)(n_in / 32);
    m->n_tiles = (int)((n_out + TILE_ROWS - 1) / TILE_ROWS);
    const int kt = ty_k45((int)ty) ? Q4_KT_SB * 8 : Q8_KT;
    m->KS = (m->nb + kt - 1) / kt;
    m->tile_bytes = ty_b32((int)ty) ? (uint32_t)(m->nb / Q8_KT) * (uint32_t)b32_step_bytes((int)ty, Q8_KT) +
                                          (m->nb % Q8_KT ? (uint32_t)b32_step_bytes((int)ty, m->nb % Q8_KT) : 0u)
                                      : (uint32_t)(m->nb / 8) * (ty == APK_TY_Q4_K ? Q4_SB_UNIT : (ty == APK_TY_Q5_K ? Q5_SB_UNIT : (ty == APK_TY_Q2_K ? Q2_SB_UNIT : Q6_SB_UNIT)));
    m->bytes = (size_t)m->n_tiles * m->tile_bytes;
    CUDA_TRY(cudaMalloc((void **)&m->d, m->bytes));
    CUDA_TRY(cudaMemsetAsync(m->d, 0, m->bytes, c->stream));

    const size_t seg_row_bytes = (size_t)n_in / be * bb;
    for (const Segment &s : segs) {
        const size_t full_row_bytes = (size_t)s.n_in_full / be * bb;
        const uint8_t *src =
            (const uint8_t *)s.w + (size_t)s.row0 * full_row_bytes + (size_t)s.kblk0 * 32 / be * bb;
        m->host_spans.emplace_back((const uint8_t *)s.w + (size_t)s.row0 * full_row_bytes,
                                   (size_t)s.rows * full_row_bytes);
        // upload in slabs of whole rows through the staging buffer
        const size_t slab_rows = std::max<size_t>(1, ((size_t)256 << 20) / seg_row_bytes);
        APK_TRY(c->staging.ensure(std::min<size_t>(slab_rows, s.rows) * seg_row_bytes));
        for (size_t r0 = 0; r0 < s.rows; r0 += slab_rows) {
            const size_t nr = std::min<size_t>(slab_rows, s.rows - r0);
            const uint8_t *from = src + r0 * full_row_bytes;
            cudaMemcpyKind kind = cudaMemcpyHostToDevice;
            if (const uint8_t *dev = raw_lookup(c, from, (nr - 1) * full_row_bytes + seg_row_bytes)) {
                from = dev;
                kind = cudaMemcpyDeviceToDevice;
            }
            CUDA_TRY(cudaMemcpy2DAsync(c->staging.p, seg_row_bytes, from, full_row_bytes, seg_row_bytes, nr, kind,
                                       c->stream));
            RepackParams rp;
            rp.src = c->staging.as<uint8_t>();
            rp.src_row_bytes = seg_row_bytes;
            rp.src_rows = (int)nr;
            rp.row_base = (int)r0;
            rp.nb = m->nb;
            rp.dst = m->d;
            rp.dst_tile_bytes = m->tile_bytes;
            rp.group = s.group;
            rp.stride = s.stride;
            rp.offset = s.offset;
            const size_t total = ty_b32((int)ty) ? nr * (size_t)m->nb : nr * (size_t)(m->nb / 8);
            const int threads = 256;
            const unsigned blocks = (unsigned)((total + threads - 1) / threads);
            if (ty == APK_TY_Q8_0)
                repack_q8_0_kernel<<<blocks, threads, 0, c->stream>>>(rp);
            else if (ty == APK_TY_Q5_0)
                repack_q5_0_kernel<<<blocks, threads, 0, c->stream>>>(rp);
            else if (ty == APK_TY_Q4_K)
                repack_q45_k_kernel<false><<<blocks, threads, 0, c->stream>>>(rp);
            else if (ty == APK_TY_Q5_K)
                repack_q45_k_kernel<true><<<blocks, threads, 0, c->stream>>>(rp);
            else
                (src_ty == APK_TY_Q3_K ? repack_q6_k_kernel<3> : (src_ty == APK_TY_Q2_K ? repack_q6_k_kernel<2> : repack_q6_k_kernel<0>))
                    <<<blocks, threads, 0, c->stream>>>(rp);
            CUDA_TRY(cudaGetLastError());
            c->st.launches++;
            CUDA_TRY(cudaStreamSynchronize(c->stream));  // staging is reused by the next slab
        }
    }
    c->st.weight_bytes += m->bytes;
    *out = std::move(m);
    return APK_OK;
}

int check_host_matrix(apk_ctx *c, const char *what, const void *w, uint32_t ty, uint32_t n_out, uint32_t n_in) {
    uint32_t be, bb;
    if (!block_geom(ty, &be, &bb))
        return fail(APK_DECLINE_UNSUPPORTED_TYPE, "%s: tensor has unsupported type %u", what, ty);
    if (!w || n_out == 0 || n_in == 0) return fail(APK_ERR_INVALID_ARG, "%s: null or empty matrix", what);
    if (n_in % be)
        return fail(APK_DECLINE_UNSUPPORTED_SHAPE, "%s: row length %u is not whole %u-element blocks", what, n_in, be);
    if (!inside_attached(c, w, host_bytes(ty, n_out, n_in)))
        return fail(APK_DECLINE_FOREIGN_MEMORY, "%s: weights are outside attached mappings", what);
    return APK_OK;
}

int shard_plan(uint32_t kind, uint32_t ty, uint32_t n_out, uint32_t n_in, uint32_t row_granule, int rank, int world,
               uint32_t out[4]) {
    uint32_t be, bb;
    if (!block_geom(ty, &be, &bb)) return fail(APK_DECLINE_UNSUPPORTED_TYPE, "ggml type %u has no kernel", ty);
    if (world < 1 || rank < 0 || rank >= world) return fail(APK_ERR_INVALID_ARG, "rank %d of %d", rank, world);
    out[0] = 0; out[1] = n_out; out[2] = 0; out[3] = n_in;
    if (world == 1 || kind == SHARD_NONE) return APK_OK;
    if (row_granule == 0) row_granule = 1;
    if (kind == SHARD_ROWS) {
        if (n_out % ((uint32_t)world * row_granule))
            return fail(APK_DECLINE_UNSUPPORTED_SHAPE, "%u rows do not split over %d ranks in bands of %u", n_out, world, row_granule);
        out[1] = n_out / world;
        out[0] = rank * out[1];
    } else if (kind == SHARD_K) {
        if (n_in % ((uint32_t)world * be))
            return fail(APK_DECLINE_UNSUPPORTED_SHAPE, "row length %u does not split over %d ranks in %u-element blocks", n_in, world, be);
        out[3] = n_in / world;
        out[2] = rank * out[3];
    } else {
        return fail(APK_ERR_INVALID_ARG, "unknown shard kind %u", kind);
    }
    return APK_OK;
}

int shard_tag(apk_ctx *c, int kind) { return kind == SHARD_NONE ? 0 : c->rank * 64 + c->world; }

// A single host matrix, whole or sharded for this rank.
int resolve_plain(apk_ctx *c, const char *what, const void *w, uint32_t ty, uint32_t n_out, uint32_t n_in, int shard,
                  DevMatrix **out) {
    if (c->world == 1) shard = SHARD_NONE;
    MatKey key(KIND_PLAIN, w, nullptr, nullptr, ty, n_out, n_in, shard, shard_tag(c, shard));
    auto it = c->mats.find(key);
    if (it != c->mats.end()) { *out = it->second.get(); return APK_OK; }
    APK_TRY(check_host_matrix(c, what, w, ty, n_out, n_in));
    uint32_t be, bb;
    block_geom(ty, &be, &bb);
    uint32_t sl[4];
    APK_TRY(shard_plan((uint32_t)shard, ty, n_out, n_in, 1, c->rank, c->world, sl));
    Segment s{w, n_in, sl[0], sl[1], sl[2] / 32, 1 << 30, 0, 0};
    const uint32_t dn_out = sl[1], dn_in = sl[3];
    std::unique_ptr<DevMatrix> m;
    APK_TRY(build_matrix(c, ty, dn_out, dn_in, {s}, &m));
    *out = m.get();
    c->mats[key] = std::move(m);
    return APK_OK;
}

// wq | wk | wv as one matrix whose tiles are whole heads (head_dim 128); with
// tensor parallelism this rank's Q heads, then its K heads, then its V heads.
int resolve_qkv(apk_ctx *c, uint32_t ty, const void *wq, const void *wk, const void *wv, uint32_t hidden,
                uint32_t n_q, uint32_t n_kv, DevMatrix **out) {
    MatKey key(KIND_QKV, wq, wk, wv, ty, n_q + (wv ? 2 : 1) * n_kv, hidden, SHARD_ROWS, shard_tag(c, SHARD_ROWS));
    auto it = c->mats.find(key);
    if (it != c->mats.end()) { *out = it->second.get(); return APK_OK; }
    APK_TRY(check_host_matrix(c, "attn wq", wq, ty, n_q, hidden));
    APK_TRY(check_host_matrix(c, "attn wk", wk, ty, n_kv, hidden));
    if (wv) APK_TRY(check_host_matrix(c, "attn wv", wv, ty, n_kv, hidden));  // (null: Q | K only, V is a matrix of its own)
    uint32_t sq[4], sk[4];
    APK_TRY(shard_plan(SHARD_ROWS, ty, n_q, hidden, TILE_ROWS, c->rank, c->world, sq));
    APK_TRY(shard_plan(SHARD_ROWS, ty, n_kv, hidden, TILE_ROWS, c->rank, c->world, sk));
    const uint32_t ql = sq[1], kl = sk[1];
    std::vector<Segment> segs = {
        {wq, hidden, sq[0], ql, 0, 1 << 30, 0, 0},
        {wk, hidden, sk[0], kl, 0, 1 << 30, 0, (int)ql},
        {wv, hidden, sk[0], kl, 0, 1 << 30, 0, (int)(ql + kl)},
    };
    if (!wv) segs.pop_back();
    std::unique_ptr<DevMatrix> m;
    APK_TRY(build_matrix(c, ty, ql + (wv ? 2 : 1) * kl, hidden, segs, &m));
    *out = m.get();
    c->mats[key] = std::move(m);
    return APK_OK;
}

// gate and up interleaved in groups of 64 rows so one 128-row tile holds 64
// gate rows and the 64 matching up rows (the SwiGLU epilogue is then tile-local).
int resolve_gateup(apk_ctx *c, uint32_t ty, const void *gate, const void *up, uint32_t hidden, uint32_t ffn,
                   DevMatrix **out, uint32_t *ffn_local) {
    MatKey key(KIND_GATEUP, gate, up, nullptr, ty, ffn, hidden, SHARD_ROWS, shard_tag(c, SHARD_ROWS));
    // the band of ffn rows is also the band of `down` columns: split on 32-row (block) boundaries
    uint32_t sf[4];
    APK_TRY(shard_plan(SHARD_ROWS, ty, ffn, hidden, 32, c->rank, c->world, sf));
    const uint32_t fl = sf[1];
    *ffn_local = fl;
    auto it = c->mats.find(key);
    if (it != c->mats.end()) { *out = it->second.get(); return APK_OK; }
    APK_TRY(check_host_matrix(c, "ffn gate", gate, ty, ffn, hidden));
    APK_TRY(check_host_matrix(c, "ffn up", up, ty, ffn, hidden));
    std::vector<Segment> segs = {
        {gate, hidden, sf[0], fl, 0, 64, 128, 0},
        {up, hidden, sf[0], fl, 0, 64, 128, 64},
    };
    const uint32_t tiles = (fl + 63) / 64;
    std::unique_ptr<DevMatrix> m;
    APK_TRY(build_matrix(c, ty, tiles * TILE_ROWS, hidden, segs, &m));
    *out = m.get();
    c->mats[key] = std::move(m);
    return APK_OK;
}

// --------------------------------------------------------------- launches

// Launch with (optionally) a programmatic dependency on the previous kernel in
// the stream: the kernel may start early and calls griddepcontrol.wait itself.
template <class... Args>
cudaError_t launch_ex(apk_ctx *c, void (*kernel)(Args...), dim3 grid, dim3 block, size_t smem, bool pdl, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = c->launch_stream ? c->launch_stream : c->stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, args...);
}

ActLayout act_layout(void *base, uint32_t consumer_ty, int m_eff) {
    ActLayout L;
    L.base = (uint8_t *)base;
    L.ke = ke_of(consumer_ty);
    L.m_eff = m_eff;
    return L;
}

size_t act_bytes(uint32_t consumer_ty, int m_eff, uint32_t n_in) {
    ActLayout L = act_layout(nullptr, consumer_ty, m_eff);
    return L.total_bytes((int)n_in) + 256;
}

struct ActMode {
    int two_level;
    int m_eff;
};

ActMode resolve_mode(uint32_t act_mode, uint32_t m) {
    // QuantMat::matmul: m == 1 -> Q8 activations, m > 1 -> f32 dots (quantmat/mod.rs:142-169)
    const bool f32 = act_mode == APK_ACT_F32 || (act_mode == APK_ACT_AUTO && m > 1);
    return ActMode{f32 ? 1 : 0, (int)(f32 ? 2 * m : m)};
}

// x [m][n] (f32) -> prepared activations for a consumer matrix of type `cty`.
int launch_prep(apk_ctx *c, const float *x, int ldx, const float *add, int ldadd, float *xout,
                int ldxout, const float *gamma, float eps, float *hout, int ldh, uint32_t n, uint32_t m,
                uint32_t cty, ActMode mode, void *act_base, const double *sumsq = nullptr) {
    PrepParams p{};
    p.sumsq = sumsq;
    p.x = x; p.ldx = ldx;
    p.add = add; p.ldadd = ldadd;
    p.xout = xout; p.ldxout = ldxout;
    p.gamma = gamma; p.eps = eps;
    p.hout = hout; p.ldh = ldh;
    p.n = (int)n; p.m = (int)m;
    p.out = act_layout(act_base, cty, mode.m_eff);
    p.two_level = mode.two_level;
    p.need_sum = needs_sum(cty);
    dim3 grid((n / 32 + 7) / 8, m);
    CUDA_TRY(launch_ex(c, prep_acts_kernel, grid, dim3(256), 0, c->use_pdl, p, c->use_pdl ? 1 : 0));
    c->st.launches++;
    return APK_OK;
}

// Stages that fit next to the resident activations (0 = does not fit at all).
int pick_stages(apk_ctx *c, int ty, int m_eff, int pro, int KS, int act_rec) {
    int ns = 6;
    while (ns > 0 && mv_smem_total(ty, m_eff, pro, KS, act_rec, ns) > c->smem_optin) --ns;
    return ns;
}

// p.pro on entry is the prologue the caller would like; a resident prologue that
// does not leave room for a useful ring falls back to streaming records (the
// caller must then have prepared them: see want_resident()).
int launch_matvec(apk_ctx *c, const DevMatrix *W, MvParams p, ActMode mode, bool dump = false) {
    MvKernel k = pick_kernel(W->ty, mode.m_eff, dump);
    if (!k) return fail(APK_DECLINE_UNSUPPORTED_SHAPE, "no kernel for %d activation rows", mode.m_eff);
    p.W = W->d;
    p.ty = (int)W->ty;
    p.n_out = (int)W->n_out;
    p.nb = W->nb;
    p.n_tiles = W->n_tiles;
    p.KS = W->KS;
    p.tile_bytes = W->tile_bytes;
    p.two_level = mode.two_level;
    p.m_out = mode.two_level ? mode.m_eff / 2 : mode.m_eff;
    p.partials = c->partials.as<unsigned long long>() + (size_t)(c->launch_no & 1) * c->n_sm * 2 * MAX_M_EFF * TILE_ROWS;
    p.err = c->d_err;
    p.wait_limit = c->wait_limit;
    p.pdl = c->use_pdl ? 1 : 0;
    p.inflight = c->inflight;
    p.inflight_pre = c->inflight_pre;
    if (c->trace && c->trace_idx < c->trace_cap) p.timeline = c->trace + (size_t)(c->trace_idx++) * c->n_sm * 8;
    if (c->dots_dump && c->launch_no == c->dots_launch &&
        (size_t)mode.m_eff * W->n_out * W->nb <= c->dots_cap) {
        p.dump = c->dots_dump;
        dump = true;
        k = pick_kernel(W->ty, mode.m_eff, true);
    }
    p.launch_id = c->launch_no;
    p.tl_alt = c->tl_alt;
    c->launch_no++;
    const int act_rec = p.act.rec_bytes();
    const int ns = pick_stages(c, (int)W->ty, mode.m_eff, p.pro, W->KS, act_rec);
    if (ns < 2) return fail(APK_DECLINE_MISSING_CAPABILITY, "activations of %d rows x %u do not fit in shared memory", mode.m_eff, W->n_in);
    p.n_stages = ns;
    const int smem = mv_smem_total((int)W->ty, mode.m_eff, p.pro, W->KS, act_rec, ns);
    const long long U = (long long)W->n_tiles * W->KS;
    int grid = (int)std::min<long long>(c->n_sm, U);
    if (c->grid_cap > 0) grid = std::min(grid, c->grid_cap);
    if ((U + 1) * grid >= (1LL << 31)) return fail(APK_DECLINE_UNSUPPORTED_SHAPE, "matrix too large for 32-bit unit arithmetic");
    // A launch may defer its dependency wait (xin_late) only behind a matvec that holds every SM
    // to itself: one CTA per SM, too much shared memory for a second one.  Its own CTAs then start
    // only where a CTA of that matvec has left, i.e. after that matvec saw everything before it
    // complete -- the token counter included.  Smaller grids share the GPU with older launches.
    const bool exclusive = grid == c->n_sm && 2 * (smem + 1024) > c->smem_per_sm;
    if (p.xin_late && !c->prev_mv_exclusive) p.xin_late = 0;
    c->prev_mv_exclusive = exclusive;
    CUDA_TRY(launch_ex(c, k, dim3(grid), dim3(MV_THREADS), (size_t)smem, c->use_pdl, (const MvParams)p));
    c->st.launches++;
    return APK_OK;
}

// Can the whole activation buffer of this matvec live in shared memory with a ring of >= 4 stages?
bool want_resident(apk_ctx *c, const DevMatrix *W, int m_eff) {
    ActLayout L = act_layout(nullptr, W->ty, m_eff);
    return pick_stages(c, (int)W->ty, m_eff, PRO_LOAD, W->KS, L.rec_bytes()) >= 4;
}

// Activation source for a matvec on x (device, f32): at one token the
// kernel quantises in its own prologue (with the optional RMSNorm); otherwise
// the separate pass writes records that are then loaded whole or streamed.
int stage_acts(apk_ctx *c, const DevMatrix *W, const float *x, int ldx, const float *add, int ldadd,
               float *xout, int ldxout, const float *gamma, float eps, uint32_t m, ActMode mode, void *act_buf,
               MvParams *p, const double *sumsq = nullptr, float *hout = nullptr) {
    p->act = act_layout(act_buf, W->ty, mode.m_eff);
    if (m == 1 && W->n_in <= (uint32_t)(N_CONSUMERS * PRO_CH) && ((uintptr_t)x & 15) == 0 && want_resident(c, W, mode.m_eff)) {
        p->pro = PRO_QUANT;
        PrepParams &pp = p->prep;
        pp.x = x; pp.ldx = ldx;
        pp.add = add; pp.ldadd = ldadd;
        pp.xout = xout; pp.ldxout = ldxout;
        pp.gamma = gamma; pp.eps = eps;
        pp.hout = hout; pp.ldh = (int)W->n_in;
        pp.sumsq = sumsq;
        pp.n = (int)W->n_in; pp.m = (int)m;
        pp.out = p->act;
        pp.two_level = mode.two_level;
        pp.need_sum = needs_sum(W->ty);
        return APK_OK;
    }
    APK_TRY(launch_prep(c, x, ldx, add, ldadd, xout, ldxout, gamma, eps, hout, (int)W->n_in, W->n_in, m, W->ty, mode,
                        act_buf, sumsq));
    p->pro = want_resident(c, W, mode.m_eff) ? PRO_LOAD : PRO_STREAM;
    return APK_OK;
}

// Activation source for records an earlier epilogue already wrote.
void use_records(apk_ctx *c, const DevMatrix *W, ActMode mode, void *act_buf, MvParams *p) {
    p->act = act_layout(act_buf, W->ty, mode.m_eff);
    p->pro = want_resident(c, W, mode.m_eff) ? PRO_LOAD : PRO_STREAM;
}

MvParams mv_store(const ActLayout &act, float *y, int ldy) {
    MvParams p{};
    p.xin.index = -1;
    p.act = act;
    p.epi = EPI_STORE;
    p.y = y;
    p.ldy = ldy;
    return p;
}

// Wait for the stream, then surface any error word a kernel left behind.
int finish(apk_ctx *c) {
    const uint64_t t0 = now_ns();
    cudaError_t e = cudaMemcpyAsync(c->h_err, c->d_err, sizeof(int), cudaMemcpyDeviceToHost, c->stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(c->stream);
    c->st.wait_ns += now_ns() - t0;
    if (e != cudaSuccess) return fail(APK_ERR_CUDA, "stream: %s", cudaGetErrorString(e));
    if (*c->h_err != 0) {
        const int w = *c->h_err;
        cudaMemsetAsync(c->d_err, 0, sizeof(int), c->stream);
        // a kernel that gave up may have left tagged partial sums behind
        if (c->partials.p) cudaMemsetAsync(c->partials.p, 0, c->partials.cap, c->stream);
        cudaStreamSynchronize(c->stream);
        const int kind = w & 15;
        return fail(APK_ERR_TIMEOUT, "device-side wait expired (%s; site %d, launch %d)",
                    kind == ERRW_PRODUCER_TIMEOUT ? "copy producer"
                    : kind == ERRW_PEER_TIMEOUT   ? "a peer rank never delivered its partial sums"
                    : kind == ERRW_FINISHER_TIMEOUT ? "a tile piece of another CTA never arrived"
                                                    : "tile consumer",
                    (w >> 4) & 15, w >> 8);
    }
    return APK_OK;
}

int check_m(uint32_t m) {
    if (m == 0 || m > APK_MAX_M) return fail(APK_DECLINE_UNSUPPORTED_SHAPE, "m = %u is outside 1..%u", m, APK_MAX_M);
    return APK_OK;
}

// One matvec on device buffers (x already in x_dev): activations + kernel -> y (device).
int run_matvec_dev(apk_ctx *c, DevMatrix *W, const float *x_dev, uint32_t m, uint32_t act_mode, float *y_dev,
                   bool reuse_act, int32_t *dump) {
    const ActMode mode = resolve_mode(act_mode, m);
    MvParams p = mv_store(ActLayout{}, y_dev, (int)W->n_out);
    APK_TRY(c->act_a.ensure(act_bytes(W->ty, mode.m_eff, W->n_in)));
    if (reuse_act && m > 1)
        use_records(c, W, mode, c->act_a.p, &p);
    else
        APK_TRY(stage_acts(c, W, x_dev, (int)W->n_in, nullptr, 0, nullptr, 0, nullptr, 0.f, m, mode, c->act_a.p, &p));
    p.dump = dump;
    return launch_matvec(c, W, p, mode, dump != nullptr);
}


// One item of gpu::ffn_batch, resolved (matrices resident) and enqueued on device buffers:
// x in c->x_dev [m][hidden], y in c->y_dev.
struct FfnOp {
    DevMatrix *GU = nullptr, *D = nullptr;
    uint32_t m = 0, hidden = 0, ffn = 0;
};

int ffn_resolve(apk_ctx *c, const apk_ffn_req *r, FfnOp *op) {
    APK_TRY(check_m(r->m));
    if (r->gate_ty != r->up_ty)
        return fail(APK_DECLINE_UNSUPPORTED_TYPE, "ffn: gate (%u) and up (%u) must share a type", r->gate_ty, r->up_ty);
    if (c->world != 1) return fail(APK_DECLINE_INVALID_STATE, "ffn: stand-alone FFN runs on an unsharded context");
    uint32_t fl;
    APK_TRY(resolve_gateup(c, r->gate_ty, r->gate_w, r->up_w, r->hidden, r->ffn, &op->GU, &fl));
    APK_TRY(resolve_plain(c, "ffn down", r->down_w, r->down_ty, r->hidden, r->ffn, SHARD_NONE, &op->D));
    op->m = r->m; op->hidden = r->hidden; op->ffn = r->ffn;
    const ActMode q8{0, (int)r->m};
    const ActMode dmode = resolve_mode(APK_ACT_AUTO, r->m);
    APK_TRY(c->x_dev.ensure((size_t)r->m * r->hidden * sizeof(float)));
    APK_TRY(c->y_dev.ensure((size_t)r->m * r->hidden * sizeof(float)));
    APK_TRY(c->act_a.ensure(act_bytes(op->GU->ty, q8.m_eff, r->hidden)));
    APK_TRY(c->act_b.ensure(act_bytes(op->D->ty, dmode.m_eff, r->ffn)));
    return APK_OK;
}

int ffn_enqueue(apk_ctx *c, const FfnOp &op) {
    const uint32_t m = op.m;
    const ActMode q8{0, (int)m};
    const ActMode dmode = resolve_mode(APK_ACT_AUTO, m);  // w_down.matmul(&gate, m): model/moe.rs:128
    MvParams p{};
    APK_TRY(stage_acts(c, op.GU, c->x_dev.as<float>(), (int)op.hidden, nullptr, 0, nullptr, 0, nullptr, 0.f, m, q8, c->act_a.p, &p));
    p.epi = EPI_SWIGLU;
    p.act_next = act_layout(c->act_b.p, op.D->ty, dmode.m_eff);
    p.next_two_level = dmode.two_level;
    p.next_need_sum = needs_sum(op.D->ty);
    p.ffn = (int)op.ffn;
    APK_TRY(launch_matvec(c, op.GU, p, q8));
    MvParams pd = mv_store(ActLayout{}, c->y_dev.as<float>(), (int)op.hidden);
    use_records(c, op.D, dmode, c->act_b.p, &pd);
    return launch_matvec(c, op.D, pd, dmode);
}

// The input half of gpu::attn_block: x in c->x_dev, side inputs in c->misc, [q | k | v] rows in c->y_dev.
struct AttnInOp {
    DevMatrix *W = nullptr;
    uint32_t m = 0, H = 0, nq = 0, nkv = 0, half = 0;
};

int attn_in_resolve(apk_ctx *c, const apk_attn_in_req *r, AttnInOp *op) {
    APK_TRY(check_m(r->m));
    if (r->head_dim != TILE_ROWS)
        return fail(APK_DECLINE_UNSUPPORTED_SHAPE, "attn_in: head_dim %u (the fused epilogue is written for 128)", r->head_dim);
    if (r->rot_dim > r->head_dim || r->rot_dim % 2)
        return fail(APK_DECLINE_UNSUPPORTED_SHAPE, "attn_in: rot_dim %u", r->rot_dim);
    if (c->world != 1) return fail(APK_DECLINE_INVALID_STATE, "attn_in: stand-alone call runs on an unsharded context");
    op->m = r->m; op->H = r->hidden; op->nq = r->n_heads * r->head_dim; op->nkv = r->n_kv_heads * r->head_dim;
    op->half = r->rot_dim / 2;
    APK_TRY(resolve_qkv(c, r->ty, r->wq, r->wk, r->wv, op->H, op->nq, op->nkv, &op->W));
    APK_TRY(c->x_dev.ensure((size_t)op->m * op->H * sizeof(float)));
    APK_TRY(c->y_dev.ensure((size_t)op->m * (op->nq + 2 * op->nkv) * sizeof(float)));
    APK_TRY(c->act_a.ensure(act_bytes(op->W->ty, (int)op->m, op->H)));
    // misc: gamma[H] | q_norm[128] | k_norm[128] | rope[m][half][2]
    APK_TRY(c->misc.ensure(((size_t)op->H + 256 + (size_t)op->m * op->half * 2) * sizeof(float)));
    return APK_OK;
}

int attn_in_upload(apk_ctx *c, const apk_attn_in_req *r, const AttnInOp &op) {
    float *misc = c->misc.as<float>();
    const size_t H = op.H;
    CUDA_TRY(cudaMemcpyAsync(c->x_dev.p, r->x, (size_t)op.m * H * sizeof(float), cudaMemcpyHostToDevice, c->stream));
    if (r->gamma) CUDA_TRY(cudaMemcpyAsync(misc, r->gamma, H * sizeof(float), cudaMemcpyHostToDevice, c->stream));
    if (r->q_norm) CUDA_TRY(cudaMemcpyAsync(misc + H, r->q_norm, 128 * sizeof(float), cudaMemcpyHostToDevice, c->stream));
    if (r->k_norm) CUDA_TRY(cudaMemcpyAsync(misc + H + 128, r->k_norm, 128 * sizeof(float), cudaMemcpyHostToDevice, c->stream));
    if (op.half) CUDA_TRY(cudaMemcpyAsync(misc + H + 256, r->rope, (size_t)op.m * op.half * 2 * sizeof(float), cudaMemcpyHostToDevice, c->stream));
    return APK_OK;
}

int attn_in_enqueue(apk_ctx *c, const apk_attn_in_req *r, const AttnInOp &op) {
    float *misc = c->misc.as<float>();
    const size_t H = op.H;
    const ActMode q8{0, (int)op.m};
    MvParams p{};
    APK_TRY(stage_acts(c, op.W, c->x_dev.as<float>(), (int)H, nullptr, 0, nullptr, 0, r->gamma ? misc : nullptr, r->eps, op.m, q8,
                       c->act_a.p, &p));
    p.epi = EPI_QKV_ROPE;
    p.y = c->y_dev.as<float>();
    p.ldy = (int)(op.nq + 2 * op.nkv);
    p.n_q_tiles = (int)r->n_heads;
    p.n_k_tiles = (int)r->n_kv_heads;
    p.q_norm = r->q_norm ? misc + H : nullptr;
    p.k_norm = r->k_norm ? misc + H + 128 : nullptr;
    p.eps = r->eps;
    p.rope = misc + H + 256;
    p.half = (int)op.half;
    return launch_matvec(c, op.W, p, q8);
}

}  // namespace

// =========================================================== the C ABI

extern "C" {

int apk_init(apk_ctx **out, int device) {
    if (!out) return fail(APK_ERR_INVALID_ARG, "apk_init: null out pointer");
    *out = nullptr;
    int n_dev = 0;
    if (cudaGetDeviceCount(&n_dev) != cudaSuccess || n_dev == 0)
        return fail(APK_DECLINE_NO_DEVICE, "no accelerator device");
    if (device < 0) {
        const char *lr = getenv("LOCAL_RANK");
        device = lr ? atoi(lr) % n_dev : 0;
    }
    if (device >= n_dev) return fail(APK_ERR_INVALID_ARG, "device %d of %d", device, n_dev);
    CUDA_TRY(cudaSetDevice(device));
    cudaDeviceProp prop;
    CUDA_TRY(cudaGetDeviceProperties(&prop, device));
    if (prop.major != 10)
        return fail(APK_DECLINE_MISSING_CAPABILITY, "device is sm_%d%d; this library is built for sm_100a only",
                    prop.major, prop.minor);
    auto c = std::make_unique<apk_ctx>();
    c->device = device;
    c->n_sm = prop.multiProcessorCount;
    c->smem_optin = (int)prop.sharedMemPerBlockOptin;
    c->smem_per_sm = (int)prop.sharedMemPerMultiprocessor;
    CUDA_TRY(cudaStreamCreateWithFlags(&c->stream, cudaStreamNonBlocking));
    CUDA_TRY(cudaStreamCreateWithFlags(&c->side, cudaStreamNonBlocking));
    CUDA_TRY(cudaEventCreateWithFlags(&c->ev_fork, cudaEventDisableTiming));
    CUDA_TRY(cudaEventCreateWithFlags(&c->ev_join, cudaEventDisableTiming));
    if (const char *e = getenv("ALLPAKA_B200_FORK_V")) c->fork_v = std::max(0, std::min(atoi(e), 8));
    CUDA_TRY(cudaEventCreate(&c->ev0));
    CUDA_TRY(cudaEventCreate(&c->ev1));
    CUDA_TRY(cudaMalloc((void **)&c->d_err, sizeof(int)));
    CUDA_TRY(cudaMemset(c->d_err, 0, sizeof(int)));
    CUDA_TRY(cudaMallocHost((void **)&c->h_err, sizeof(int)));
    *c->h_err = 0;
    // two copies, used by alternate launches: a launch that takes its input from the peer exchange
    // starts before the launch in front of it has drained
    APK_TRY(c->partials.ensure(2 * (size_t)c->n_sm * 2 * MAX_M_EFF * TILE_ROWS * sizeof(unsigned long long), true));
    APK_TRY(init_kernel_attrs(c.get()));
    if (const char *e = getenv("ALLPAKA_B200_PDL")) c->use_pdl = atoi(e) != 0;
    if (const char *e = getenv("ALLPAKA_B200_FUSE_NORM")) c->fuse_norm = atoi(e);
    if (const char *e = getenv("ALLPAKA_B200_INFLIGHT")) c->inflight = std::max(1, std::min(atoi(e), MAX_STAGES));
    if (const char *e = getenv("ALLPAKA_B200_INFLIGHT_PRE")) c->inflight_pre = std::max(1, std::min(atoi(e), MAX_STAGES));
    if (const char *e = getenv("ALLPAKA_B200_SELF_XCH")) c->self_xch = atoi(e) != 0;
    if (const char *e = getenv("ALLPAKA_B200_TL_ALT")) c->tl_alt = atoi(e) != 0;
    if (const char *e = getenv("ALLPAKA_B200_ATTN_TC")) c->attn_tc = atoi(e) != 0;
    if (const char *e = getenv("ALLPAKA_B200_ATTN_MIN_POS")) c->attn_min_pos = std::max(16, std::min(atoi(e), 4096));
    if (c->self_xch) {
        // one rank exchanging with itself: the peer-store epilogue and the collecting prologue on one GPU
        CUDA_TRY(cudaMalloc((void **)&c->xch_local, XCH_BYTES));
        CUDA_TRY(cudaMemset(c->xch_local, 0, XCH_BYTES));
        c->xch.slots[0] = c->xch_local;
        c->xch.rank = 0;
        c->xch.world = 1;
        c->p2p_ready = true;  // (p2p_open stays false: nothing was mapped from a peer)
    }
    *out = c.release();
    return APK_OK;
}

void apk_shutdown(apk_ctx *c) {
    if (!c) return;
    cudaSetDevice(c->device);
    if (c->stream) cudaStreamSynchronize(c->stream);
    c->plan.reset();
    c->mats.clear();
    for (auto &kv : c->raw_dev) cudaFree(kv.second.first);
    c->raw_dev.clear();
    if (c->p2p_open)
        for (int r = 0; r < c->world; ++r)
            if (r != c->rank && c->xch.slots[r]) cudaIpcCloseMemHandle(c->xch.slots[r]);
    if (c->xch_local) cudaFree(c->xch_local);
    if (c->comm && g_nccl.CommDestroy) g_nccl.CommDestroy(c->comm);
    for (DevBuf *b : {&c->staging, &c->partials, &c->x_dev, &c->y_dev, &c->act_a, &c->act_b, &c->misc, &c->dump})
        b->release();
    if (c->d_err) cudaFree(c->d_err);
    if (c->h_err) cudaFreeHost(c->h_err);
    if (c->ev0) cudaEventDestroy(c->ev0);
    if (c->ev1) cudaEventDestroy(c->ev1);
    if (c->ev_fork) cudaEventDestroy(c->ev_fork);
    if (c->ev_join) cudaEventDestroy(c->ev_join);
    if (c->side) cudaStreamDestroy(c->side);
    if (c->stream) cudaStreamDestroy(c->stream);
    delete c;
}

int apk_attach(apk_ctx *c, const void *host_base, size_t len) {
    if (!c || !host_base || len == 0) return fail(APK_ERR_INVALID_ARG, "attach: null or empty mapping");
    std::lock_guard<std::mutex> g(c->mu);
    c->attached[{(const uint8_t *)host_base, len}]++;
    return APK_OK;
}

int apk_detach(apk_ctx *c, const void *host_base, size_t len) {
    if (!c || !host_base) return fail(APK_ERR_INVALID_ARG, "detach: null mapping");
    std::lock_guard<std::mutex> g(c->mu);
    auto it = c->attached.find({(const uint8_t *)host_base, len});
    if (it == c->attached.end()) return fail(APK_DECLINE_INVALID_STATE, "detach: mapping was never attached");
    if (--it->second > 0) return APK_OK;
    c->attached.erase(it);
    cudaSetDevice(c->device);
    cudaStreamSynchronize(c->stream);
    c->plan.reset();  // a plan may point at matrices about to go
    const uint8_t *b = (const uint8_t *)host_base;
    for (auto mi = c->mats.begin(); mi != c->mats.end();) {
        bool hit = false;
        for (auto &sp : mi->second->host_spans)
            if (sp.first < b + len && sp.first + sp.second > b) hit = true;
        if (hit) {
            c->st.weight_bytes -= mi->second->bytes;
            mi = c->mats.erase(mi);
        } else {
            ++mi;
        }
    }
    return APK_OK;
}

int apk_is_attached(apk_ctx *c) {
    if (!c) return 0;
    std::lock_guard<std::mutex> g(c->mu);
    return c->attached.empty() ? 0 : 1;
}

int apk_register_matrix(apk_ctx *c, const void *w, uint32_t ty, uint32_t n_out, uint32_t n_in) {
    if (!c) return fail(APK_ERR_INVALID_ARG, "null context");
    std::lock_guard<std::mutex> g(c->mu);
    CUDA_TRY(cudaSetDevice(c->device));
    DevMatrix *m;
    return resolve_plain(c, "register", w, ty, n_out, n_in, SHARD_NONE, &m);
}

int apk_matvec_batch(apk_ctx *c, const apk_matvec_req *reqs, uint32_t n_reqs, uint32_t act_mode,
                     float *const *ys) {
    if (!c || (n_reqs && (!reqs || !ys))) return fail(APK_ERR_INVALID_ARG, "matvec_batch: null argument");
    if (n_reqs == 0) return APK_OK;
    std::lock_guard<std::mutex> g(c->mu);
    CUDA_TRY(cudaSetDevice(c->device));
    const uint64_t t0 = now_ns();
    size_t y_total = 0, x_max = 0;
    std::vector<DevMatrix *> mats(n_reqs);
    for (uint32_t i = 0; i < n_reqs; ++i) {
        const apk_matvec_req &r = reqs[i];
        APK_TRY(check_m(r.m));
        if (!r.x || !ys[i]) return fail(APK_ERR_INVALID_ARG, "matvec: null x or y");
        APK_TRY(resolve_plain(c, "matvec", r.w, r.ty, r.n_out, r.n_in, SHARD_NONE, &mats[i]));
        y_total += (size_t)r.m * r.n_out;
        x_max = std::max(x_max, (size_t)r.m * r.n_in);
    }
    APK_TRY(c->x_dev.ensure(x_max * sizeof(float)));
    APK_TRY(c->y_dev.ensure(y_total * sizeof(float)));
    size_t y_off = 0;
    const float *last_x = nullptr;
    uint32_t last_m = 0, last_n = 0, last_ty = 0;
    std::vector<size_t> offs(n_reqs);
    for (uint32_t i = 0; i < n_reqs; ++i) {
        const apk_matvec_req &r = reqs[i];
        // items that share x share one activation quantisation (quantmat/mod.rs:372-388)
        const bool same = last_x == r.x && last_m == r.m && last_n == r.n_in && ke_of(last_ty) == ke_of(r.ty) &&
                          needs_sum(last_ty) == needs_sum(r.ty);
        if (!same)
            CUDA_TRY(cudaMemcpyAsync(c->x_dev.p, r.x, (size_t)r.m * r.n_in * sizeof(float), cudaMemcpyHostToDevice,
                                     c->stream));
        offs[i] = y_off;
        APK_TRY(run_matvec_dev(c, mats[i], c->x_dev.as<float>(), r.m, act_mode, c->y_dev.as<float>() + y_off, same,
                               nullptr));
        y_off += (size_t)r.m * r.n_out;
        last_x = r.x; last_m = r.m; last_n = r.n_in; last_ty = r.ty;
    }
    for (uint32_t i = 0; i < n_reqs; ++i)
        CUDA_TRY(cudaMemcpyAsync(ys[i], c->y_dev.as<float>() + offs[i],
                                 (size_t)reqs[i].m * reqs[i].n_out * sizeof(float), cudaMemcpyDeviceToHost, c->stream));
    c->st.encode_ns += now_ns() - t0;
    c->st.calls++;
    return finish(c);
}

int apk_matvec(apk_ctx *c, const void *w, uint32_t ty, uint32_t n_in, uint32_t n_out, const float *x, uint32_t m,
               uint32_t act_mode, float *y) {
    apk_matvec_req r{ty, w, n_in, n_out, x, m};
    float *ys[1] = {y};
    return apk_matvec_batch(c, &r, 1, act_mode, ys);
}

int apk_debug_block_dots(apk_ctx *c, const void *w, uint32_t ty, uint32_t n_in, uint32_t n_out, const float *x,
                         uint32_t m, int32_t *dots) {
    if (!c || !x || !dots) return fail(APK_ERR_INVALID_ARG, "block_dots: null argument");
    std::lock_guard<std::mutex> g(c->mu);
    CUDA_TRY(cudaSetDevice(c->device));
    APK_TRY(check_m(m));
    DevMatrix *W;
    APK_TRY(resolve_plain(c, "block_dots", w, ty, n_out, n_in, SHARD_NONE, &W));
    const size_t nd = (size_t)m * n_out * (n_in / 32);
    APK_TRY(c->x_dev.ensure((size_t)m * n_in * sizeof(float)));
    APK_TRY(c->y_dev.ensure((size_t)m * n_out * sizeof(float)));
    APK_TRY(c->dump.ensure(nd * sizeof(int32_t)));
    CUDA_TRY(cudaMemcpyAsync(c->x_dev.p, x, (size_t)m * n_in * sizeof(float), cudaMemcpyHostToDevice, c->stream));
    CUDA_TRY(cudaMemsetAsync(c->dump.p, 0xff, nd * sizeof(int32_t), c->stream));
    APK_TRY(run_matvec_dev(c, W, c->x_dev.as<float>(), m, APK_ACT_Q8, c->y_dev.as<float>(), false,
                           c->dump.as<int32_t>()));
    CUDA_TRY(cudaMemcpyAsync(dots, c->dump.p, nd * sizeof(int32_t), cudaMemcpyDeviceToHost, c->stream));
    c->st.calls++;
    return finish(c);
}

int apk_debug_matvec_timeline(apk_ctx *c, const void *w, uint32_t ty, uint32_t n_in, uint32_t n_out, const float *x,
                              uint32_t m, uint64_t *stamps, uint32_t max_ctas, uint32_t *n_ctas) {
    if (!c || !x || !stamps || !n_ctas) return fail(APK_ERR_INVALID_ARG, "timeline: null argument");
    std::lock_guard<std::mutex> g(c->mu);
    CUDA_TRY(cudaSetDevice(c->device));
    APK_TRY(check_m(m));
    DevMatrix *W;
    APK_TRY(resolve_plain(c, "timeline", w, ty, n_out, n_in, SHARD_NONE, &W));
    const long long U = (long long)W->n_tiles * W->KS;
    const uint32_t grid = (uint32_t)std::min<long long>(c->n_sm, U);
    if (grid > max_ctas) return fail(APK_ERR_INVALID_ARG, "timeline: room for %u CTAs, need %u", max_ctas, grid);
    *n_ctas = grid;
    const ActMode mode{0, (int)m};
    APK_TRY(c->x_dev.ensure((size_t)m * n_in * sizeof(float)));
    APK_TRY(c->y_dev.ensure((size_t)m * n_out * sizeof(float)));
    APK_TRY(c->dump.ensure((size_t)grid * 8 * sizeof(uint64_t)));
    APK_TRY(c->act_a.ensure(act_bytes(W->ty, mode.m_eff, W->n_in)));
    CUDA_TRY(cudaMemcpyAsync(c->x_dev.p, x, (size_t)m * n_in * sizeof(float), cudaMemcpyHostToDevice, c->stream));
    MvParams p = mv_store(ActLayout{}, c->y_dev.as<float>(), (int)n_out);
    APK_TRY(stage_acts(c, W, c->x_dev.as<float>(), (int)n_in, nullptr, 0, nullptr, 0, nullptr, 0.f, m, mode, c->act_a.p, &p));
    // Four launches back to back (programmatic dependencies chain them like the layers of
    // a token); every launch rewrites all stamps, so the last one is what is reported.
    CUDA_TRY(cudaMemsetAsync(c->dump.p, 0, (size_t)grid * 8 * sizeof(uint64_t), c->stream));
    p.timeline = c->dump.as<unsigned long long>();
    for (int rep = 0; rep < 4; ++rep) APK_TRY(launch_matvec(c, W, p, mode));
    CUDA_TRY(cudaMemcpyAsync(stamps, c->dump.p, (size_t)grid * 8 * sizeof(uint64_t), cudaMemcpyDeviceToHost, c->stream));
    c->st.calls++;
    return finish(c);
}

int apk_debug_q8_acts(apk_ctx *c, const float *x, uint32_t n, const float *gamma, float eps, float *d, float *sum,
                      int8_t *q) {
    if (!c || !x || !d || !sum || !q) return fail(APK_ERR_INVALID_ARG, "q8_acts: null argument");
    if (n == 0 || n % 32) return fail(APK_DECLINE_UNSUPPORTED_SHAPE, "q8_acts: %u is not whole 32-element blocks", n);
    std::lock_guard<std::mutex> g(c->mu);
    CUDA_TRY(cudaSetDevice(c->device));
    const ActMode mode{0, 1};
    const size_t ab = act_bytes(APK_TY_Q4_K, 1, n);
    APK_TRY(c->x_dev.ensure((size_t)n * sizeof(float)));
    APK_TRY(c->misc.ensure((size_t)n * sizeof(float)));
    APK_TRY(c->act_a.ensure(ab));
    CUDA_TRY(cudaMemcpyAsync(c->x_dev.p, x, (size_t)n * sizeof(float), cudaMemcpyHostToDevice, c->stream));
    if (gamma) CUDA_TRY(cudaMemcpyAsync(c->misc.p, gamma, (size_t)n * sizeof(float), cudaMemcpyHostToDevice, c->stream));
    CUDA_TRY(cudaMemsetAsync(c->act_a.p, 0, ab, c->stream));
    // the Q4_K flavour of the record carries the block sums as well
    APK_TRY(launch_prep(c, c->x_dev.as<float>(), (int)n, nullptr, 0, nullptr, 0, gamma ? c->misc.as<float>() : nullptr, eps,
                        nullptr, 0, n, 1, APK_TY_Q4_K, mode, c->act_a.p));
    std::vector<uint8_t> host(ab);
    CUDA_TRY(cudaMemcpyAsync(host.data(), c->act_a.p, ab, cudaMemcpyDeviceToHost, c->stream));
    c->st.calls++;
    APK_TRY(finish(c));
    // one-row record of the Q4_K flavour: q [block][half][16], d [block][2], sum [block][2]
    const ActLayout L = act_layout(nullptr, APK_TY_Q4_K, 1);
    const int kt = L.kt(), mp = L.mp(), rec = L.rec_bytes();
    for (uint32_t b = 0; b < n / 32; ++b) {
        const uint8_t *r = host.data() + (size_t)(b / kt) * rec;
        const int bl = (int)(b % kt);
        memcpy(q + (size_t)b * 32, r + bl * 32, 32);
        memcpy(&d[b], r + L.q_bytes() + (bl * mp) * 4, 4);
        memcpy(&sum[b], r + L.q_bytes() + (kt * mp + bl * mp) * 4, 4);
    }
    return APK_OK;
}

int apk_ffn(apk_ctx *c, const apk_ffn_req *r, float *y) {
    if (!c || !r || !y || !r->x) return fail(APK_ERR_INVALID_ARG, "ffn: null argument");
    std::lock_guard<std::mutex> g(c->mu);
    CUDA_TRY(cudaSetDevice(c->device));
    const uint64_t t0 = now_ns();
    FfnOp op;
    APK_TRY(ffn_resolve(c, r, &op));
    CUDA_TRY(cudaMemcpyAsync(c->x_dev.p, r->x, (size_t)op.m * op.hidden * sizeof(float), cudaMemcpyHostToDevice, c->stream));
    APK_TRY(ffn_enqueue(c, op));
    CUDA_TRY(cudaMemcpyAsync(y, c->y_dev.p, (size_t)op.m * op.hidden * sizeof(float), cudaMemcpyDeviceToHost, c->stream));
    c->st.encode_ns += now_ns() - t0;
    c->st.calls++;
    return finish(c);
}

int apk_attn_in(apk_ctx *c, const apk_attn_in_req *r, float *q, float *k, float *v) {
    if (!c || !r || !q || !k || !v || !r->x || !r->rope) return fail(APK_ERR_INVALID_ARG, "attn_in: null argument");
    std::lock_guard<std::mutex> g(c->mu);
    CUDA_TRY(cudaSetDevice(c->device));
    const uint64_t t0 = now_ns();
    AttnInOp op;
    APK_TRY(attn_in_resolve(c, r, &op));
    APK_TRY(attn_in_upload(c, r, op));
    APK_TRY(attn_in_enqueue(c, r, op));
    const uint32_t m = op.m, nq = op.nq, nkv = op.nkv, ld = nq + 2 * nkv;
    const float *yd = c->y_dev.as<float>();
    CUDA_TRY(cudaMemcpy2DAsync(q, nq * sizeof(float), yd, ld * sizeof(float), nq * sizeof(float), m, cudaMemcpyDeviceToHost, c->stream));
    CUDA_TRY(cudaMemcpy2DAsync(k, nkv * sizeof(float), yd + nq, ld * sizeof(float), nkv * sizeof(float), m, cudaMemcpyDeviceToHost, c->stream));
    CUDA_TRY(cudaMemcpy2DAsync(v, nkv * sizeof(float), yd + nq + nkv, ld * sizeof(float), nkv * sizeof(float), m, cudaMemcpyDeviceToHost, c->stream));
    c->st.encode_ns += now_ns() - t0;
    c->st.calls++;
    return finish(c);
}

int apk_bench_ring(apk_ctx *c, const apk_bench_req *b, uint32_t reps, float *us_per_pass) {
    if (!c || !b || !us_per_pass || reps == 0 || b->n_copies == 0) return fail(APK_ERR_INVALID_ARG, "bench_ring: null argument");
    std::lock_guard<std::mutex> g(c->mu);
    CUDA_TRY(cudaSetDevice(c->device));
    const uint32_t n = b->n_copies;
    std::vector<DevMatrix *> mats(n);
    std::vector<FfnOp> ffns(n);
    std::vector<AttnInOp> attns(n);
    if (b->op == APK_BENCH_MATVEC) {
        if (!b->mv) return fail(APK_ERR_INVALID_ARG, "bench_ring: no matvec requests");
        for (uint32_t i = 0; i < n; ++i) {
            const apk_matvec_req &r = b->mv[i];
            APK_TRY(check_m(r.m));
            if (r.m != b->mv[0].m || r.n_in != b->mv[0].n_in || r.n_out != b->mv[0].n_out)
                return fail(APK_ERR_INVALID_ARG, "bench_ring: copies differ in shape");
            APK_TRY(resolve_plain(c, "bench", r.w, r.ty, r.n_out, r.n_in, SHARD_NONE, &mats[i]));
        }
        const apk_matvec_req &r0 = b->mv[0];
        if (!r0.x) return fail(APK_ERR_INVALID_ARG, "bench_ring: no input rows");
        APK_TRY(c->x_dev.ensure((size_t)r0.m * r0.n_in * sizeof(float)));
        APK_TRY(c->y_dev.ensure((size_t)r0.m * r0.n_out * sizeof(float)));
        CUDA_TRY(cudaMemcpyAsync(c->x_dev.p, r0.x, (size_t)r0.m * r0.n_in * sizeof(float), cudaMemcpyHostToDevice, c->stream));
    } else if (b->op == APK_BENCH_FFN) {
        if (!b->ffn || !b->ffn[0].x) return fail(APK_ERR_INVALID_ARG, "bench_ring: no ffn requests");
        for (uint32_t i = 0; i < n; ++i) APK_TRY(ffn_resolve(c, &b->ffn[i], &ffns[i]));
        CUDA_TRY(cudaMemcpyAsync(c->x_dev.p, b->ffn[0].x, (size_t)ffns[0].m * ffns[0].hidden * sizeof(float),
                                 cudaMemcpyHostToDevice, c->stream));
    } else if (b->op == APK_BENCH_ATTN_IN) {
        if (!b->attn || !b->attn[0].x || !b->attn[0].rope) return fail(APK_ERR_INVALID_ARG, "bench_ring: no attn_in requests");
        for (uint32_t i = 0; i < n; ++i) APK_TRY(attn_in_resolve(c, &b->attn[i], &attns[i]));
        APK_TRY(attn_in_upload(c, &b->attn[0], attns[0]));
    } else {
        return fail(APK_ERR_INVALID_ARG, "bench_ring: unknown op %u", b->op);
    }
    auto pass = [&](uint32_t i) -> int {
        if (b->op == APK_BENCH_MATVEC)
            return run_matvec_dev(c, mats[i], c->x_dev.as<float>(), b->mv[0].m, b->act_mode, c->y_dev.as<float>(), false, nullptr);
        if (b->op == APK_BENCH_FFN) return ffn_enqueue(c, ffns[i]);
        return attn_in_enqueue(c, &b->attn[0], attns[i]);
    };
    for (uint32_t i = 0; i < n; ++i) APK_TRY(pass(i));  // warm: every copy once
    APK_TRY(finish(c));
    CUDA_TRY(cudaEventRecord(c->ev0, c->stream));
    for (uint32_t rep = 0; rep < reps; ++rep)
        for (uint32_t i = 0; i < n; ++i) APK_TRY(pass(i));
    CUDA_TRY(cudaEventRecord(c->ev1, c->stream));
    c->st.calls++;
    APK_TRY(finish(c));
    float ms = 0.f;
    CUDA_TRY(cudaEventElapsedTime(&ms, c->ev0, c->ev1));
    *us_per_pass = ms * 1e3f / (float)(reps * n);
    return APK_OK;
}

int apk_debug_synth_matrix(apk_ctx *c, void *w, uint32_t ty, uint32_t n_out, uint32_t n_in, uint64_t seed,
                           int write_host) {
    if (!c || !w) return fail(APK_ERR_INVALID_ARG, "synth: null argument");
    std::lock_guard<std::mutex> g(c->mu);
    CUDA_TRY(cudaSetDevice(c->device));
    APK_TRY(check_host_matrix(c, "synth", w, ty, n_out, n_in));
    const size_t bytes = host_bytes(ty, n_out, n_in);
    uint32_t be = 0, bb = 0;
    block_geom(ty, &be, &bb);
    const size_t n_blocks = bytes / bb;
    uint8_t *d = nullptr;
    CUDA_TRY(cudaMalloc((void **)&d, bytes));
    const unsigned blocks = (unsigned)((n_blocks + 255) / 256);
    if (ty == APK_TY_Q8_0)
        synth_q8_0_kernel<<<blocks, 256, 0, c->stream>>>(d, n_blocks, seed);
    else if (ty == APK_TY_Q5_0)
        synth_q5_0_kernel<<<blocks, 256, 0, c->stream>>>(d, n_blocks, seed);
    else if (ty == APK_TY_Q3_K)
        synth_q3_k_kernel<<<blocks, 256, 0, c->stream>>>(d, n_blocks, seed);
    else if (ty == APK_TY_Q2_K)
        synth_q2_k_kernel<<<blocks, 256, 0, c->stream>>>(d, n_blocks, seed);
    else if (ty == APK_TY_Q4_K)
        synth_q4_k_kernel<<<blocks, 256, 0, c->stream>>>(d, n_blocks, seed);
    else if (ty == APK_TY_Q5_K)
        synth_q5_k_kernel<<<blocks, 256, 0, c->stream>>>(d, n_blocks, seed);
    else
        synth_q6_k_kernel<<<blocks, 256, 0, c->stream>>>(d, n_blocks, seed);
    c->st.launches++;
    cudaError_t e = cudaGetLastError();
    if (e == cudaSuccess && write_host) e = cudaMemcpyAsync(w, d, bytes, cudaMemcpyDeviceToHost, c->stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(c->stream);
    if (e != cudaSuccess) {
        cudaFree(d);
        return fail(APK_ERR_CUDA, "synth: %s", cudaGetErrorString(e));
    }
    auto old = c->raw_dev.find((const uint8_t *)w);
    if (old != c->raw_dev.end()) {
        cudaFree(old->second.first);
        c->raw_dev.erase(old);
    }
    c->raw_dev[(const uint8_t *)w] = {d, bytes};
    return APK_OK;
}

int apk_debug_synth_release(apk_ctx *c) {
    if (!c) return fail(APK_ERR_INVALID_ARG, "null context");
    std::lock_guard<std::mutex> g(c->mu);
    CUDA_TRY(cudaSetDevice(c->device));
    CUDA_TRY(cudaStreamSynchronize(c->stream));
    for (auto &kv : c->raw_dev) cudaFree(kv.second.first);
    c->raw_dev.clear();
    return APK_OK;
}

void apk_stats(apk_ctx *c, apk_stats_t *out) {
    if (!c || !out) return;
    std::lock_guard<std::mutex> g(c->mu);
    *out = c->st;
}

const char *apk_last_error(apk_ctx *) { return g_last_error; }

int apk_shard_plan(uint32_t kind, uint32_t ty, uint32_t n_out, uint32_t n_in, uint32_t row_granule, int rank, int world,
                   uint32_t out[4]) {
    if (!out) return fail(APK_ERR_INVALID_ARG, "shard_plan: null out");
    return shard_plan(kind, ty, n_out, n_in, row_granule, rank, world, out);
}

int apk_dist_p2p_export(apk_ctx *c, void *handle_out) {
    if (!c || !handle_out) return fail(APK_ERR_INVALID_ARG, "p2p_export: null argument");
    std::lock_guard<std::mutex> g(c->mu);
    CUDA_TRY(cudaSetDevice(c->device));
    if (c->world > XCH_MAX_RANKS) return fail(APK_DECLINE_UNSUPPORTED_SHAPE, "p2p exchange is built for at most %d ranks", XCH_MAX_RANKS);
    if (!c->xch_local) {
        CUDA_TRY(cudaMalloc((void **)&c->xch_local, XCH_BYTES));
        CUDA_TRY(cudaMemset(c->xch_local, 0, XCH_BYTES));
    }
    static_assert(sizeof(cudaIpcMemHandle_t) == APK_IPC_HANDLE_BYTES, "IPC handle size");
    cudaIpcMemHandle_t h;
    CUDA_TRY(cudaIpcGetMemHandle(&h, c->xch_local));
    memcpy(handle_out, &h, sizeof h);
    return APK_OK;
}

int apk_dist_p2p_open(apk_ctx *c, const void *handles) {
    if (!c || !handles) return fail(APK_ERR_INVALID_ARG, "p2p_open: null argument");
    std::lock_guard<std::mutex> g(c->mu);
    CUDA_TRY(cudaSetDevice(c->device));
    if (!c->xch_local) return fail(APK_DECLINE_INVALID_STATE, "p2p_open before p2p_export");
    if (c->p2p_open) return APK_OK;
    if (c->world > XCH_MAX_RANKS) return fail(APK_DECLINE_UNSUPPORTED_SHAPE, "p2p exchange is built for at most %d ranks", XCH_MAX_RANKS);
    c->xch.rank = c->rank;
    c->xch.world = c->world;
    for (int r = 0; r < c->world; ++r) {
        if (r == c->rank) { c->xch.slots[r] = c->xch_local; continue; }
        cudaIpcMemHandle_t h;
        memcpy(&h, (const uint8_t *)handles + (size_t)r * APK_IPC_HANDLE_BYTES, sizeof h);
        void *ptr = nullptr;
        CUDA_TRY(cudaIpcOpenMemHandle(&ptr, h, cudaIpcMemLazyEnablePeerAccess));
        c->xch.slots[r] = (float *)ptr;
    }
    c->plan.reset();  // graphs captured with NCCL reductions are rebuilt
    c->p2p_open = true;
    c->p2p_ready = true;
    return APK_OK;
}

int apk_dist_set_exchange(apk_ctx *c, int peer_stores) {
    if (!c) return fail(APK_ERR_INVALID_ARG, "null context");
    std::lock_guard<std::mutex> g(c->mu);
    CUDA_TRY(cudaSetDevice(c->device));
    if (peer_stores && !c->p2p_open) return fail(APK_DECLINE_INVALID_STATE, "set_exchange: no peer buffers are open");
    CUDA_TRY(cudaStreamSynchronize(c->stream));
    c->p2p_ready = peer_stores != 0;
    c->plan.reset();  // captured graphs carry the other kind of reduction
    return APK_OK;
}

int apk_dist_unique_id(void *id_out) {
    if (!id_out) return fail(APK_ERR_INVALID_ARG, "null id buffer");
    if (!g_nccl.load()) return fail(APK_ERR_NCCL, "libnccl.so.2 could not be loaded: %s", dlerror());
    Nccl::uid_t id;
    const int rc = g_nccl.GetUniqueId(&id);
    if (rc) return fail(APK_ERR_NCCL, "ncclGetUniqueId: %s", g_nccl.GetErrorString(rc));
    memcpy(id_out, &id, sizeof id);
    return APK_OK;
}

int apk_dist_init(apk_ctx *c, int rank, int world, const void *unique_id) {
    if (!c || !unique_id || world < 1 || rank < 0 || rank >= world)
        return fail(APK_ERR_INVALID_ARG, "dist_init: bad rank %d / world %d", rank, world);
    std::lock_guard<std::mutex> g(c->mu);
    if (!c->mats.empty()) return fail(APK_DECLINE_INVALID_STATE, "dist_init must precede the first weight upload");
    CUDA_TRY(cudaSetDevice(c->device));
    if (world > 1) {
        if (!g_nccl.load()) return fail(APK_ERR_NCCL, "libnccl.so.2 could not be loaded");
        Nccl::uid_t id;
        memcpy(&id, unique_id, sizeof id);
        const int rc = g_nccl.CommInitRank(&c->comm, world, id, rank);
        if (rc) return fail(APK_ERR_NCCL, "ncclCommInitRank: %s", g_nccl.GetErrorString(rc));
    }
    c->rank = rank;
    c->world = world;
    return APK_OK;
}

}  // extern "C"

#include "decode.inl"
#include "noalloc.inl"
#include "gguf.inl"
