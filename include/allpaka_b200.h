/*
 * allpaka_b200.h -- C ABI of libapk_b200.so, the sm_100a decode dequant-matvec
 * path for the allpaka engine.
 *
 * Every entry point is what an `allpaka-b200-sys` FFI crate binds so that
 * allpaka-backend's accelerator module (`crate::gpu::*`, the free-function
 * surface every backend implements: crates/allpaka-backend/src/gpu/mod.rs:9-26,
 * spelled out by gpu/stub.rs:37-217) can forward to it.  Conventions follow the
 * engine's existing native shim (third_party/allpaka_ggml/allpaka_ggml.h:16-152):
 * `extern "C"`, plain pointers and sizes, int status, no callbacks, no
 * unwinding, nothing allocated here is freed by the caller.
 *
 * Ownership: all pointer arguments are borrowed HOST memory, valid only for the
 * call.  Weights are identified by their host address inside an attached
 * mapping, exactly like the reference CUDA backend (gpu/cuda/runtime/
 * select.rs:80-84); the library keeps a repacked device copy until the mapping
 * is detached.  There is no CPU fallback: a supported request either runs on
 * the GPU or returns an error.
 *
 * Threading: one internal mutex per context; calls may come from any thread and
 * are serialised (the reference: one process-wide Mutex<CudaGpu>,
 * gpu/cuda/runtime/device.rs:267, 944-948).
 */
#ifndef ALLPAKA_B200_H
#define ALLPAKA_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- status codes -------------------------------------------------------
 * 0 = executed.  1..7 = declined, nothing happened; the values are the
 * variants of allpaka-backend's DeclineReason (src/accel.rs:10-36).
 * Negative = a hard error; the context stays usable unless stated. */
#define APK_OK 0
#define APK_DECLINE_NO_DEVICE 1
#define APK_DECLINE_UNSUPPORTED_TYPE 2
#define APK_DECLINE_UNSUPPORTED_SHAPE 3
#define APK_DECLINE_FOREIGN_MEMORY 4
#define APK_DECLINE_MISSING_CAPABILITY 5
#define APK_DECLINE_INVALID_STATE 6
#define APK_DECLINE_BACKEND 7
#define APK_ERR_INVALID_ARG (-1)
#define APK_ERR_CUDA (-2)
#define APK_ERR_TIMEOUT (-3) /* a bounded device-side wait expired */
#define APK_ERR_NCCL (-4)
#define APK_ERR_OOM (-5)

/* GGML type ids (crates/allpaka-dtype/src/lib.rs:61-75). */
#define APK_TY_Q5_0 6u
#define APK_TY_Q8_0 8u
#define APK_TY_Q2_K 10u
#define APK_TY_Q3_K 11u
#define APK_TY_Q4_K 12u
#define APK_TY_Q5_K 13u
#define APK_TY_Q6_K 14u

/* How activations meet the integer weights.  The reference picks this by call
 * site, not by dtype (crates/allpaka-backend/src/quantmat/mod.rs):
 *   APK_ACT_Q8   Q8Acts::from_f32 per row + int32 block dots: every m == 1
 *                matvec (mod.rs:224-267) and every matmul_many item at any m
 *                (mod.rs:314-419).  Block dots are bit-exact.
 *   APK_ACT_F32  f32 row dots: QuantMat::matmul with m > 1 (mod.rs:156-213).
 *                Computed here with two-level int8 activations (error ~2e-5
 *                relative, far inside the 2e-3 bar).
 *   APK_ACT_AUTO what QuantMat::matmul does: m == 1 -> Q8, m > 1 -> F32. */
#define APK_ACT_Q8 0u
#define APK_ACT_F32 1u
#define APK_ACT_AUTO 2u

#define APK_MAX_M 8u /* speculative verify batches are m = K+1 <= 8 (model/decode.rs:140-225) */

typedef struct apk_ctx apk_ctx;

/* One context = one GPU (one process per GPU; ranks of a tensor-parallel
 * group each own one).  device < 0 picks LOCAL_RANK or 0.
 * Replaces the lazy GPU singleton, gpu/cuda/runtime/device.rs:934-948. */
int apk_init(apk_ctx **out, int device);
void apk_shutdown(apk_ctx *ctx);

/* gpu::attach / detach / is_attached (stub.rs:37-45; cuda/mod.rs:41-66).
 * Attach is refcounted per (base,len) and uploads nothing; matrices inside the
 * range are repacked and uploaded at their first use or by
 * apk_register_matrix.  Detach at refcount 0 frees every device copy whose
 * host bytes lie in the range. */
int apk_attach(apk_ctx *ctx, const void *host_base, size_t len);
int apk_detach(apk_ctx *ctx, const void *host_base, size_t len);
int apk_is_attached(apk_ctx *ctx);

/* Optional eager form of what the first matvec does lazily: repack the
 * [n_out, n_in] matrix at w (raw GGUF blocks, crates/allpaka-backend/src/
 * quantmat/mod.rs:39-65 geometry rules) into the tiled device stream. */
int apk_register_matrix(apk_ctx *ctx, const void *w, uint32_t ty, uint32_t n_out, uint32_t n_in);

/* gpu::matvec (stub.rs:87-95) and one item of gpu::matvec_batch
 * (stub.rs:97-99, MatvecReq gpu/types.rs:9-16): y[m][n_out] = x[m][n_in] . W^T. */
int apk_matvec(apk_ctx *ctx, const void *w, uint32_t ty, uint32_t n_in, uint32_t n_out,
               const float *x, uint32_t m, uint32_t act_mode, float *y);

typedef struct {
    uint32_t ty;
    const void *w;
    uint32_t n_in, n_out;
    const float *x; /* m * n_in */
    uint32_t m;
} apk_matvec_req; /* MatvecReq, gpu/types.rs:9-16 */

/* gpu::matvec_batch (stub.rs:97-99): several matmuls, one submission.  Items
 * that share x (QKV, gate/up) share one activation quantisation, as the CPU
 * path does (quantmat/mod.rs:372-388).  act_mode applies to every item
 * (matmul_many -> APK_ACT_Q8; a single matmul -> APK_ACT_AUTO). */
int apk_matvec_batch(apk_ctx *ctx, const apk_matvec_req *reqs, uint32_t n_reqs, uint32_t act_mode,
                     float *const *ys);

typedef struct {
    uint32_t gate_ty; const void *gate_w;
    uint32_t up_ty; const void *up_w;
    uint32_t down_ty; const void *down_w;
    uint32_t hidden, ffn;
    const float *x; /* m * hidden */
    uint32_t m;
} apk_ffn_req; /* FfnReq, gpu/types.rs:20-31 */

/* One item of gpu::ffn_batch (stub.rs:101-103): y = swiglu(x.G^T, x.U^T).D^T.
 * gate/up: Q8 activations (matmul_many); down: Q8 at m == 1, F32 at m > 1
 * (model/moe.rs:120-128).  y is m * hidden. */
int apk_ffn(apk_ctx *ctx, const apk_ffn_req *req, float *y);

typedef struct {
    uint32_t ty; /* wq, wk, wv share a type */
    const void *wq, *wk, *wv;
    uint32_t hidden, head_dim, n_heads, n_kv_heads;
    const float *x;      /* m * hidden (the layer input; normed here when gamma != NULL) */
    uint32_t m;
    const float *gamma;  /* attn_norm weight [hidden] or NULL */
    float eps;
    const float *q_norm; /* per-head norms [head_dim] or NULL */
    const float *k_norm;
    const float *rope;   /* (sin, cos) pairs: m rows of rot_dim/2 entries */
    uint32_t rot_dim;    /* <= head_dim; NeoX split-half pairing */
} apk_attn_in_req;

/* The input half of gpu::attn_block (stub.rs:146-148, AttnBlockReq
 * gpu/types.rs:54-80): RMSNorm -> fused Q/K/V matvec -> per-head norm -> NeoX
 * RoPE, the part of the block that is dequant-matvec work
 * (model/decode.rs:478, 548-552; model/attention.rs:131-165).
 * q is m * n_heads*head_dim, k and v are m * n_kv_heads*head_dim. */
int apk_attn_in(apk_ctx *ctx, const apk_attn_in_req *req, float *q, float *k, float *v);

typedef struct {
    uint32_t ty;
    const void *w;
    uint32_t n_out;
} apk_mat; /* the (GgmlType, bytes, n_out) descriptor tuple, quantmat/mod.rs:499-502 */

typedef struct {
    const float *attn_norm, *ffn_norm; /* hidden floats each */
    apk_mat wq, wk, wv, wo;
    const float *q_norm, *k_norm;      /* optional, head_dim floats */
    apk_mat gate, up, down;            /* TokenFfn::Dense */
} apk_token_layer; /* TokenLayer, gpu/types.rs:111-150 (dense attention layers) */

#define APK_ATTN_IDENTITY 1u /* attention core = identity on the roped Q slice (the synthetic benchmark stack) */
#define APK_ATTN_CAUSAL 2u   /* causal GQA attention over the f16 KV cache named by the request */

/* The f16 KV cache of a session on the device: per layer a K slab and a V slab of
 * [capacity][kv_dim] halves (KvCache, crates/allpaka-model/src/kv.rs:507-535, 682-697, 815-824).
 * kv_dim = n_kv_heads * head_dim of the whole model; a rank of a tensor-parallel group keeps its
 * own kv heads only.  apk_kv_read / apk_kv_write move rows pos0..pos0+n_pos of one layer between
 * the host and this rank's slabs (this rank's kv heads, f16 bits), e.g. to hand over a prefill. */
typedef struct apk_kv apk_kv;
int apk_kv_create(apk_ctx *ctx, uint32_t n_layers, uint32_t kv_dim, uint32_t capacity, apk_kv **out);
void apk_kv_destroy(apk_ctx *ctx, apk_kv *kv);
int apk_kv_read(apk_ctx *ctx, const apk_kv *kv, uint32_t layer, uint32_t pos0, uint32_t n_pos, uint16_t *k, uint16_t *v);
int apk_kv_write(apk_ctx *ctx, apk_kv *kv, uint32_t layer, uint32_t pos0, uint32_t n_pos, const uint16_t *k,
                 const uint16_t *v);

/* gpu::attend_batch (AttnReq, gpu/types.rs:34-52): m query rows of n_heads * 128 floats attend over
 * one layer of the cache, row i over positions 0..=pos+i, GQA group = n_heads / kv heads, scores
 * scaled by `scale`; out is m * n_heads * 128 (model/attention.rs:337-428).  Unsharded contexts. */
int apk_attend(apk_ctx *ctx, const apk_kv *kv, uint32_t layer, const float *q, uint32_t m, uint32_t n_heads,
               uint32_t pos, float scale, float *out);

typedef struct {
    const apk_token_layer *layers;
    uint32_t n_layers;
    const float *output_norm; /* hidden floats */
    apk_mat output;           /* LM head, n_out = vocab */
    const float *x;           /* m * hidden input rows */
    uint32_t m;               /* 1 = decode, 2..8 = speculative verify */
    const float *rope;        /* m rows of rot_dim/2 (sin,cos) pairs */
    uint32_t rot_dim;
    float eps;
    uint32_t hidden, head_dim, n_heads, n_kv_heads;
    uint32_t attn_core;       /* APK_ATTN_IDENTITY or APK_ATTN_CAUSAL */
    int argmax;               /* 1: return the greedy token per row instead of logits */
    /* TokenReq.embd + token_id (gpu/types.rs:187-192): when embd.w != NULL, use_token != 0 and
     * m == 1, the input row is the embedding row of token_id, dequantised on the GPU at the head
     * of the submission, and x is ignored.  embd = (type, table bytes, vocab rows); its row length
     * is `hidden`.  With tied embeddings pass the LM head's bytes: the resident copy is shared. */
    apk_mat embd;
    uint32_t token_id;
    int use_token;
    /* APK_ATTN_CAUSAL (TokenReq.cache / pos / scale, gpu/types.rs:207-226): the layer's K and V rows
     * of the m tokens are stored at positions pos..pos+m-1 of kv (f16), row i attends over
     * 0..=pos+i.  kv must have at least n_layers layers and pos + m <= its capacity. */
    apk_kv *kv;
    uint32_t pos;
    float scale;              /* 1/sqrt(head_dim) */
} apk_token_req; /* TokenReq, gpu/types.rs:183-238 */

/* TokenOut, gpu/types.rs:228-238.  Logits(Vec<f32>): logits set, argmax == 0.
 * Argmax(u32): argmax set, argmax == 1, m == 1.  Rows { argmax, hidden }, what
 * the speculative verify consumes (model/decode.rs:212-217): argmax and hidden
 * both set, argmax == 1, any m.  `hidden` may accompany either form. */
typedef struct {
    float *logits;    /* m * vocab, written when argmax == 0 */
    uint32_t *argmax; /* m ids, written when argmax == 1 (ties go to the higher id, model/decode.rs:604-608) */
    float *hidden;    /* optional, m * hidden: the output-normed rows (rmsnorm(x, output_norm), the LM head's input) */
} apk_token_out;

/* gpu::decode_token_checked (stub.rs:150-157): the whole token as one
 * submission (a replayed CUDA graph).  Layer weights are resolved, fused
 * (Q|K|V rows, gate/up row interleave) and uploaded at the first call that
 * names them.  The plan built then is keyed on every descriptor of the request
 * (layer array address, each weight and norm pointer, types, row counts); the
 * norm weights are copied at that point, so the borrowed tensors must keep
 * their contents until the mapping is detached. */
int apk_decode_token(apk_ctx *ctx, const apk_token_req *req, apk_token_out *out);

/* gpu::decode_token with argmax followed by gpu::decode_greedy_continue
 * (gpu/cuda/decode.rs:93-227): n_tokens greedy steps with one synchronisation at the end.  Step 0
 * embeds req->token_id; every step's winner (ties to the higher id) is embedded on the device as
 * the next step's input, and nothing returns to the host in between.  rope holds one row of
 * rot_dim/2 (sin, cos) pairs per step (positions pos, pos+1, ...), built by the host as for
 * apk_decode_token; req->rope is ignored.  Needs req->embd, m == 1.  tokens_out receives the
 * n_tokens winners. */
int apk_decode_greedy(apk_ctx *ctx, const apk_token_req *req, uint32_t n_tokens, const float *rope,
                      uint32_t *tokens_out);

/* Same work with the m*hidden input already in device memory and the result
 * left there: what a caller that keeps the residual stream on the GPU between
 * tokens uses, and what the benchmark times as the device-resident number.
 * `iters` back-to-back replays; returns the elapsed GPU time of all of them
 * (CUDA events on the launching stream). */
int apk_decode_replay(apk_ctx *ctx, const apk_token_req *req, uint32_t iters, float *elapsed_ms);

/* Parity instrumentation: the int32 dot of every 32-element block,
 * dots[(i*n_out + j)*(n_in/32) + b], for Q8-activation mode.  For Q4_K and Q5_K
 * block b = 8*superblock + sub-block; for Q6_K and Q3_K the entry is sc0*dot0 + sc1*dot1
 * of the block's two 16-element halves, the integer the reference scales
 * (quantmat/q8_acts.rs:338-342, 206-210), for Q2_K the same with its 4-bit scales (its min
 * term is not a dot with the weights); for Q5_0 the dot with the values q - 16. */
int apk_debug_block_dots(apk_ctx *ctx, const void *w, uint32_t ty, uint32_t n_in, uint32_t n_out,
                         const float *x, uint32_t m, int32_t *dots);

/* Parity instrumentation: the Q8 activation blocks the kernels consume
 * (Q8Acts::from_f32 semantics, quantmat/q8_acts.rs:26-63), optionally after
 * the fused RMSNorm (gamma != NULL).  d and sum are n/32 floats, q n bytes. */
int apk_debug_q8_acts(apk_ctx *ctx, const float *x, uint32_t n, const float *gamma, float eps,
                      float *d, float *sum, int8_t *q);

/* Parity instrumentation for the whole-token path: the token of apk_decode_token
 * is enqueued launch by launch and every matvec that reads the residual stream
 * through an RMSNorm (Q|K|V, gate/up, LM head) hands back what it worked on:
 * record i = the m residual rows it normalised, x[(i*8 + row)*hidden ..], and
 * the activation records its tensor-core loop consumed, unpacked to
 * d, sum [(i*16 + r)*(hidden/32) ..] and q [(i*16 + r)*hidden ..] for r < rows;
 * meta[4i..] = {rows, two-level flag, index of the launch in the token, K-step}.
 * With dots != NULL the int32 block dots of matvec launch number dots_launch
 * (0-based in issue order; layout [rows][device rows of that matrix][n_in/32])
 * are written too, if they fit dots_elems.  Single-GPU contexts only. */
int apk_debug_token_records(apk_ctx *ctx, const apk_token_req *req, uint32_t max_records, float *x, float *d,
                            float *sum, int8_t *q, int32_t *meta, uint32_t *n_records, int dots_launch,
                            int32_t *dots, size_t dots_elems);

/* Every wait inside a kernel (on a copy, on another CTA's tile piece, on a
 * peer rank's partial sums) gives up after a cycle budget, records which wait
 * it was and lets the kernel end; the call then returns APK_ERR_TIMEOUT and
 * the context stays usable.  This sets the budget in SM clock cycles (0
 * restores the default of 4e9, about two seconds), for tests that make a wait
 * run out on purpose. */
int apk_debug_set_wait_limit(apk_ctx *ctx, uint64_t cycles);

/* Test of that path which needs one GPU only: the kernel that collects a
 * tensor-parallel exchange is run against a second local buffer standing for a
 * peer that never delivers.  Returns what the call that hit it would return
 * (APK_ERR_TIMEOUT once the budget has run out). */
int apk_debug_xch_timeout(apk_ctx *ctx);

/* A matvec that allocates nothing.  It has no counterpart in the reference.
 *
 * For callers that cannot call cudaMalloc at this point: every byte of device
 * memory was budgeted and handed out at start-up (a late allocation would
 * simply fail), or the call sits in a latency-bounded decode loop where the
 * device-wide stall of an allocation is not acceptable.  They own x and y already; the kernel's
 * private scratch (stream-K partial sums, error word,
 * quantised-activation records) lives in a fixed ~5.9 MB array inside the
 * library's device image, which every GPU that loads the library holds until
 * the process exits.
 *
 *   w        host address of a matrix that is ALREADY resident (apk_register_matrix or any
 *            earlier call); otherwise APK_DECLINE_INVALID_STATE, because uploading would allocate
 *   x_dev    device pointer, m * n_in floats;  y_dev  device pointer, m * n_out floats
 *   stream   the CUDA stream (cudaStream_t) to enqueue on; wait != 0 also synchronises it and
 *            reports an expired device-side wait
 * Limits: n_in <= APK_NOALLOC_MAX_N_IN, n_out <= APK_NOALLOC_MAX_N_OUT, m <= APK_MAX_M, at most 160
 * SMs; larger requests are declined with APK_DECLINE_UNSUPPORTED_SHAPE / _MISSING_CAPABILITY.
 * No cudaMalloc, cudaFree or other allocating call is made, on any path.
 *
 * The first call on a device resolves the array's device address
 * (cudaGetSymbolAddress); make that first call before starting a stream capture.
 * All calls on a device share the one array, from whichever context, and it
 * keeps the last call's contents (the error word is cleared at the start of
 * every call; the tagged partial sums are left all-zero by a kernel that ran to
 * its end and are cleared again after any call on that device that was not
 * seen to end cleanly): two calls whose kernels overlap on the GPU, on
 * different streams or contexts of the same device, race.  With wait == 0
 * nobody reads the error word, so an expired device-side wait of that call
 * goes unreported.  Results are identical to apk_matvec's. */
#define APK_NOALLOC_MAX_N_IN 32768u
#define APK_NOALLOC_MAX_N_OUT 524288u
int apk_matvec_noalloc(apk_ctx *ctx, const void *w, uint32_t ty, uint32_t n_in, uint32_t n_out, const float *x_dev,
                       uint32_t m, uint32_t act_mode, float *y_dev, void *stream, int wait);

/* Trace: per-CTA timestamps (GPU global timer, ns) of one matvec launch on
 * activations already quantised: stamps[cta][8] = {kernel entry, first unit in
 * shared memory, second unit, last unit, a tile finished, last tile finished,
 * 0, 0}.  n_ctas receives the grid size. */
int apk_debug_matvec_timeline(apk_ctx *ctx, const void *w, uint32_t ty, uint32_t n_in, uint32_t n_out,
                              const float *x, uint32_t m, uint64_t *stamps, uint32_t max_ctas, uint32_t *n_ctas);

/* Trace of a whole token: the token of apk_decode_token is enqueued launch by
 * launch (no graph) and every matvec launch writes the same eight stamps per
 * CTA into its own slab: stamps[launch][n_ctas][8], launches in issue order
 * (per layer Q|K|V, wo, gate/up, down; then the LM head).  At most
 * max_launches slabs are written; n_launches receives how many were. */
int apk_debug_token_timeline(apk_ctx *ctx, const apk_token_req *req, uint64_t *stamps, uint32_t max_launches,
                             uint32_t *n_launches, uint32_t *n_ctas);

/* Benchmark utility: a seeded synthetic tensor without host-side generation.
 * The raw GGUF blocks of the [n_out, n_in] matrix whose host address is w are
 * produced by a counter-based generator on the device and kept there as the
 * stand-in for the host bytes: later uploads of (parts of) that host range
 * copy from it instead of from w.  With write_host != 0 the same bytes are
 * also stored to w, so a CPU reference can read them.  w must lie inside an
 * attached mapping.  apk_debug_synth_release drops the stand-ins once every
 * matrix that needs them has been uploaded. */
int apk_debug_synth_matrix(apk_ctx *ctx, void *w, uint32_t ty, uint32_t n_out, uint32_t n_in, uint64_t seed,
                           int write_host);
int apk_debug_synth_release(apk_ctx *ctx);

/* Benchmark utility: average GPU time of each matvec kernel launch of one
 * token, by kind, with the kernels launched back to back over all layers
 * between one CUDA-event pair per kind (no graph).  ms[0..4] = Q|K|V, wo,
 * gate/up, down, LM head (per launch); bytes[0..4] = algorithmic bytes of one
 * such launch (original GGUF weight bytes + activations in + results out). */
int apk_decode_profile(apk_ctx *ctx, const apk_token_req *req, uint32_t reps, float *ms, double *bytes);

/* Benchmark utility: one operator timed over a ring of distinct weight copies,
 * inputs resident on the device, launches chained back to back like the layers
 * of a token, one CUDA-event pair on the launching stream around reps * n_copies
 * passes (after one untimed pass over every copy).  A ring larger than L2
 * measures HBM-cold; a single copy measures L2-hot.  Ops: a plain matvec
 * (mv[i], x of mv[0]), the input half of the attention block (attn[i]: RMSNorm
 * -> Q|K|V -> per-head norm -> RoPE; x, norm weights and RoPE table of attn[0]),
 * or one FFN (ffn[i]; x of ffn[0]).  Copies must share one shape. */
#define APK_BENCH_MATVEC 0u
#define APK_BENCH_ATTN_IN 1u
#define APK_BENCH_FFN 2u
typedef struct {
    uint32_t op;
    uint32_t n_copies;
    const apk_matvec_req *mv;
    const apk_attn_in_req *attn;
    const apk_ffn_req *ffn;
    uint32_t act_mode; /* matvec only */
} apk_bench_req;
int apk_bench_ring(apk_ctx *ctx, const apk_bench_req *req, uint32_t reps, float *us_per_pass);

typedef struct {
    uint64_t calls;      /* entry-point submissions (gpu::stats().0, gpu/common.rs:24-31) */
    uint64_t launches;   /* kernels launched by this library (".1 dispatches") */
    uint64_t encode_ns;  /* host time spent building submissions */
    uint64_t wait_ns;    /* host time blocked on the GPU */
    uint64_t weight_bytes;   /* repacked device bytes resident */
    uint64_t decode_attempts, decode_successes, decode_declines; /* DecodePathStats, gpu/types.rs:258-285 */
} apk_stats_t;

/* Benchmark helper: the attention core of apk_attend over every layer of the cache in turn (distinct
 * memory per layer), `reps` rounds timed with CUDA events; microseconds per layer. */
int apk_bench_attend(apk_ctx *ctx, const apk_kv *kv, const float *q, uint32_t m, uint32_t n_heads, uint32_t pos, float scale,
                     uint32_t reps, float *us_per_layer);

void apk_stats(apk_ctx *ctx, apk_stats_t *out);

/* Human-readable reason for the last non-zero status on this thread
 * (gpu::init_error, stub.rs:51-53; DecodeDecline{stage,reason} gpu/types.rs:247-252). */
const char *apk_last_error(apk_ctx *ctx);

/* ---- model files ---------------------------------------------------------
 * GGUF on the host: header, metadata and tensor table parsed out of a read-only mapping of the
 * file (crates/allpaka-gguf/src/metadata.rs:194-297, tensors.rs:183-217).  Versions >= 2;
 * general.alignment honoured (default 32); arrays other than short u32 ones are walked over.
 * Tensor bytes are pointers into the mapping: attach it (apk_gguf_mapping + apk_attach, or
 * apk_model_attach) and hand them to any entry point above.  No GPU is needed to read a file. */
typedef struct apk_gguf apk_gguf;
typedef struct {
    const char *name;   /* owned by the file handle */
    uint32_t ty;        /* GGML type id */
    uint32_t n_dims;
    uint64_t dims[4];   /* dims[0] is the row length (n_in), dims[1] the rows (n_out) */
    const void *data;
    uint64_t n_bytes;   /* 0 for types this library has no block geometry for */
} apk_gguf_tensor;
int apk_gguf_open(const char *path, apk_gguf **out);
void apk_gguf_close(apk_gguf *f);
uint64_t apk_gguf_n_tensors(const apk_gguf *f);
int apk_gguf_tensor_at(const apk_gguf *f, uint64_t i, apk_gguf_tensor *out);
int apk_gguf_find(const apk_gguf *f, const char *name, apk_gguf_tensor *out); /* GgufFile::tensor + data */
const char *apk_gguf_architecture(const apk_gguf *f);
/* metadata by full key (GgufFile::meta_u32 / meta_f32 / meta_str, tensors.rs:143-166);
 * APK_DECLINE_INVALID_STATE / NULL when absent or of another kind */
int apk_gguf_meta_u32(const apk_gguf *f, const char *key, uint32_t *out);
int apk_gguf_meta_f32(const apk_gguf *f, const char *key, float *out);
const char *apk_gguf_meta_str(const apk_gguf *f, const char *key);
const void *apk_gguf_mapping(const apk_gguf *f, uint64_t *len);

/* The dense-decoder view of a file: Config::from_gguf (crates/allpaka-model/src/config.rs:184-310)
 * and the tensor binding of Model::load (model/loader.rs:100-260) for attention + dense-FFN blocks.
 * Every matrix is checked against the shape the graph expects (qmat, loader.rs:558-569); norm
 * vectors must be F32 (norm_raw, loader.rs:573-580); llama / mistral files get the rows of every
 * Q and K head reordered for NEOX rotation (neox_order + reorder_head_rows, loader.rs:366-426;
 * ALLPAKA_ROPE_NORM=1 declines that); mixture-of-experts, projection biases and other block kinds
 * are declined.  The file handle must outlive the model. */
typedef struct apk_model apk_model;
typedef struct {
    uint32_t n_layers, hidden, n_heads, n_kv_heads, head_dim, ffn, vocab, rot_dim;
    float eps, rope_base;
    int has_qk_norm, neox_reordered, tied;
} apk_model_info;
int apk_model_open(apk_gguf *f, apk_model **out);
const apk_model_info *apk_model_get_info(const apk_model *m);
/* A request template over the model's tensors (layers, norms, LM head, embedding table, shapes,
 * causal attention, scale = 1/sqrt(head_dim), m = 1); the caller adds the input (x or token_id),
 * the rope rows, the cache and the position. */
int apk_model_token_req(const apk_model *m, apk_token_req *req);
/* gpu::attach of the file's mapping and of every reordered copy (loader.rs:62-98, 421). */
int apk_model_attach(apk_ctx *ctx, apk_model *m);
void apk_model_close(apk_model *m);

/* ---- tensor parallelism over one NVLink domain ----------------------------
 * No counterpart in the reference (its only multi-device scheme is layer
 * pipelining over TCP, crates/allpaka-model/src/pipeline.rs).  Every rank
 * calls the same entry points with the same host tensors; each uploads only
 * its shard (column-parallel Q|K|V and gate/up, row-parallel wo and down) and
 * the partial sums are combined across ranks after wo and down. */
#define APK_SHARD_ROWS 1u /* column-parallel: a contiguous band of output rows (whole 128-row heads for Q|K|V) */
#define APK_SHARD_K 2u    /* row-parallel: a contiguous band of input columns, on quantisation-block boundaries */
/* The slice of an [n_out, n_in] matrix that `rank` of `world` holds: out[0..3] =
 * {first row, rows, first column, columns}.  `row_granule` is 1, or 128 when rows
 * are attention heads.  Pure host arithmetic (no GPU needed); the uploads use
 * exactly this function.  Returns APK_DECLINE_UNSUPPORTED_SHAPE when the
 * matrix does not divide. */
int apk_shard_plan(uint32_t kind, uint32_t ty, uint32_t n_out, uint32_t n_in, uint32_t row_granule, int rank,
                   int world, uint32_t out[4]);
/* Optional low-latency exchange for the two per-layer reductions: each rank
 * exports one device buffer (CUDA IPC handle, APK_IPC_HANDLE_BYTES), the host
 * gathers the handles of all ranks in rank order and every rank opens them.
 * From then on the CTA that closes a tile of a row-parallel matvec stores its
 * partial sums straight into every rank's buffer over NVLink, each value as a
 * 64-bit word that carries the exchange's number; the next matvec polls those
 * words in its own prologue (bounded), adds them in rank order onto the residual
 * row, normalises and quantises: four launches per layer, no fence, no flag, no
 * NCCL all-reduce.  At most 8 ranks, m * hidden <= 131072.  Every rank must
 * issue the same sequence of decode calls. */
#define APK_IPC_HANDLE_BYTES 64
int apk_dist_p2p_export(apk_ctx *ctx, void *handle_out);
int apk_dist_p2p_open(apk_ctx *ctx, const void *handles /* world * APK_IPC_HANDLE_BYTES */);
/* Switch between the peer-store exchange (1; needs apk_dist_p2p_open) and NCCL
 * all-reduce (0) for the per-layer reductions.  Every rank must make the same call. */
int apk_dist_set_exchange(apk_ctx *ctx, int peer_stores);
#define APK_UNIQUE_ID_BYTES 128
int apk_dist_unique_id(void *id_out /* APK_UNIQUE_ID_BYTES */);
int apk_dist_init(apk_ctx *ctx, int rank, int world, const void *unique_id);

#ifdef __cplusplus
}
#endif
#endif
