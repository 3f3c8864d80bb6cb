/*
 * apk_oracle.h -- CPU restatement of allpaka's reference dequant-matvec path.
 *
 * TEST INFRASTRUCTURE ONLY.  This library is the checker for the CUDA path and
 * the timed CPU baseline; nothing in the product library links, loads or calls
 * it.  Every function cites the reference file:line whose arithmetic (operand
 * order, accumulation type, rounding) it follows.  Always the x86_64 /
 * not(aarch64) arms of the reference.
 *
 * Parity pin: the reference is Rust and cannot be compiled where this is
 * built, so the restatement is pinned by the reference's own known-answer
 * tests (block-layout KATs, hand-computed matmuls, LCG row tests and their
 * tolerances), restated in tests/test_oracle_kats.py.
 *
 * Build with -ffp-contract=off and without -ffast-math: Rust never contracts
 * a*b+c and never reassociates float sums.
 */
#ifndef APK_ORACLE_H
#define APK_ORACLE_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* GGML type ids (crates/allpaka-dtype/src/lib.rs:61-75). */
#define ORC_TY_Q8_0 8u
#define ORC_TY_Q4_K 12u
#define ORC_TY_Q5_K 13u
#define ORC_TY_Q6_K 14u
#define ORC_TY_Q5_0 6u
#define ORC_TY_Q3_K 11u
#define ORC_TY_Q2_K 10u

/* crates/allpaka-dtype/src/lib.rs:129-201 */
float orc_f16_to_f32(uint16_t h);
uint16_t orc_f32_to_f16(float x);
float orc_bf16_to_f32(uint16_t h);
uint16_t orc_f32_to_bf16(float x);

/* crates/allpaka-dtype/src/lib.rs:382-390 */
void orc_scale_min_k4(int j, const uint8_t *packed, float *sc, float *mn);

/* crates/allpaka-dtype/src/lib.rs:79-124.  Returns 0 on unsupported type or
 * ragged element count (the reference returns Err). */
size_t orc_expected_bytes(uint32_t ty, size_t elements);

/* crates/allpaka-gguf/src/dequant.rs:26-91, 94-126, 211-231.
 * Returns 0 on success, -1 on a byte-count / type error. */
int orc_dequant(uint32_t ty, const uint8_t *bytes, size_t n_bytes, float *out, size_t n);

/* crates/allpaka-backend/src/quantmat/q8_acts.rs:26-63 */
void orc_q8acts_from_f32(const float *x, size_t n, float *d, float *sum, int8_t *q);

/* crates/allpaka-backend/src/quantmat/q8_acts.rs:353-365 */
int32_t orc_dot_i8(const int8_t *a, const int8_t *b, size_t n);

/* q8_acts.rs:86-96, 267-301 and dot_f32.rs:140-160, 166-210: one row. */
float orc_dot_q8_0_i8(const uint8_t *row, size_t n_in, const float *d, const int8_t *q);
float orc_dot_q4_k_i8(const uint8_t *row, size_t n_in, const float *d, const float *sum,
                      const int8_t *q);
float orc_dot_q8_0(const uint8_t *row, size_t n_in, const float *x);
float orc_dot_q4_k(const uint8_t *row, size_t n_in, const float *x);
/* q8_acts.rs:223-262 and dot_f32.rs:97-135: one Q5_K row. */
float orc_dot_q5_k_i8(const uint8_t *row, size_t n_in, const float *d, const float *sum, const int8_t *q);
float orc_dot_q5_k(const uint8_t *row, size_t n_in, const float *x);
/* q8_acts.rs:100-124 and dot_f32.rs:39-55: one Q5_0 row. */
float orc_dot_q5_0_i8(const uint8_t *row, size_t n_in, const float *d, const int8_t *q);
float orc_dot_q5_0(const uint8_t *row, size_t n_in, const float *x);
/* q8_acts.rs:127-174 and dot_f32.rs:214-248: one Q2_K row. */
float orc_dot_q2_k_i8(const uint8_t *row, size_t n_in, const float *d, const int8_t *q);
float orc_dot_q2_k(const uint8_t *row, size_t n_in, const float *x);
/* q8_acts.rs:178-218 and dot_f32.rs:58-94: one Q3_K row. */
float orc_dot_q3_k_i8(const uint8_t *row, size_t n_in, const float *d, const int8_t *q);
float orc_dot_q3_k(const uint8_t *row, size_t n_in, const float *x);
/* q8_acts.rs:307-346 and dot_f32.rs:252-289: one Q6_K row. */
float orc_dot_q6_k_i8(const uint8_t *row, size_t n_in, const float *d, const int8_t *q);
float orc_dot_q6_k(const uint8_t *row, size_t n_in, const float *x);

/* The int32 dot of every 32-element block of every row against Q8 acts:
 * dots[(i*n_out + j)*(n_in/32) + b].  For Q4_K block b = 8*superblock +
 * sub-block (lo nibbles = even sub-blocks, q8_acts.rs:288-295); for Q6_K the entry is
 * sc0*dot0 + sc1*dot1 of the block's two 16-element halves (q8_acts.rs:338-342). */
int orc_block_dots(uint32_t ty, const uint8_t *w, size_t n_out, size_t n_in, const int8_t *q,
                   size_t m, int32_t *dots);

/* Activation handling at the call site (quantmat/mod.rs):
 *   ORC_ACT_Q8  - Q8Acts::from_f32 per row, integer dots (matvec mod.rs:224-267,
 *                 matmul_many mod.rs:314-419 at any m)
 *   ORC_ACT_F32 - f32 row_dot (matmul with m>1, mod.rs:156-213, 706-735)
 *   ORC_ACT_AUTO- what QuantMat::matmul does: m==1 -> Q8, m>1 -> F32. */
#define ORC_ACT_Q8 0
#define ORC_ACT_F32 1
#define ORC_ACT_AUTO 2

/* y[m][n_out] = x[m][n_in] . W^T.  threads<=0 -> all cores.  Follows the
 * reference threading rule: contiguous row chunks (thread_pool.rs:207-230),
 * only when n_out*n_in >= 2<<20 (mod.rs:241-243).  Returns 0 / -1. */
int orc_matmul(uint32_t ty, const uint8_t *w, size_t w_bytes, size_t n_out, size_t n_in,
               const float *x, size_t m, int act_mode, float *y, int threads);

/* crates/allpaka-backend/src/ops/norm.rs:6-109 (AVX2 lane order), 115-187, 193-269 */
double orc_sum_sq_f64(const float *x, size_t n);
void orc_rmsnorm(float *x, const float *w, size_t n, float eps);
void orc_rmsnorm_into(float *dst, const float *src, const float *w, size_t n, float eps);

/* crates/allpaka-backend/src/ops/rope.rs:8-22, 70-81, 104-117 */
void orc_rope_inv_freq(size_t head_dim, float base, float *out);
void orc_rope_sin_cos(uint32_t pos, const float *inv_freq, size_t n, float *table /*[n][2]*/);
void orc_rope_neox_table(float *x, size_t len, const float *table, size_t half);
void orc_rope_neox(float *x, size_t d, uint32_t pos, float base);

/* crates/allpaka-backend/src/ops/activation.rs:20-22, 116-119 */
float orc_silu(float x);
void orc_swiglu(float *gate, const float *up, size_t n);

/* rmsnorm_into -> matmul_many(wq,wk,wv) -> per-head [rmsnorm] + NeoX rope on q
 * and k (model/decode.rs:478, 548-552; model/attention.rs:131-165).
 * x[m][hidden]; gamma NULL = no input norm; q_norm/k_norm NULL = no per-head
 * norm; rope table [m][half][2].  Outputs q[m][n_q], k[m][n_kv], v[m][n_kv]. */
int orc_attn_in(uint32_t ty, const uint8_t *wq, const uint8_t *wk, const uint8_t *wv,
                size_t hidden, size_t n_q, size_t n_kv, size_t head_dim, const float *x, size_t m,
                const float *gamma, float eps, const float *q_norm, const float *k_norm,
                const float *rope, size_t half, float *q, float *k, float *v, int threads);

/* Dense FFN: matmul_many(gate, up) -> swiglu -> down.matmul(act, m)
 * (model/moe.rs:120-128).  act_out (may be NULL) receives the swiglu rows. */
int orc_ffn(uint32_t gate_ty, const uint8_t *gate, uint32_t up_ty, const uint8_t *up,
            uint32_t down_ty, const uint8_t *down, size_t hidden, size_t ffn, const float *x,
            size_t m, float *y, float *act_out, int threads);

/* One decoder layer of the shape the benchmark uses, attention core replaced
 * by the identity on the roped Q slice (model/decode.rs:435-591, 755-777):
 *   h = rmsnorm(x, attn_norm); q,k,v = qkv(h); rope(q,k);
 *   x += wo . q;  h = rmsnorm(x, ffn_norm); x += down . swiglu(gate.h, up.h)
 * All matrices share one type.  x is updated in place ([hidden], m = 1). */
typedef struct {
    const uint8_t *wq, *wk, *wv, *wo, *gate, *up, *down;
    const float *attn_norm, *ffn_norm;
    const float *q_norm, *k_norm; /* optional per-head norms */
} orc_layer;

int orc_decode_layers(uint32_t ty, const orc_layer *layers, size_t n_layers, size_t hidden,
                      size_t n_q, size_t n_kv, size_t head_dim, size_t ffn, float eps,
                      const float *rope, size_t half, float *x, int threads);

/* finish_hidden: rmsnorm(x, output_norm) then output.matmul(x,1)
 * (model/decode.rs:594-602). */
int orc_lm_head(uint32_t ty, const uint8_t *w, size_t vocab, size_t hidden, const float *x,
                const float *output_norm, float eps, float *logits, int threads);

/* ---- decode attention over the f16 KV cache (model/attention.rs:337-399; model/kv.rs:682-697) */
/* K or V row of one position into the cache: f32 -> f16, round to nearest even (kv.rs:695-696). */
void orc_kv_store(const float *row, size_t n, uint16_t *dst);
/* One kv head attending for its whole GQA group over positions first..=pos, online softmax in one
 * K/V pass (attend_group, attention.rs:337-399).  kcache/vcache: this layer's [capacity][kv_dim] f16. */
void orc_attend_group(const float *q_group, const uint16_t *kcache, const uint16_t *vcache, size_t kv_dim,
                      size_t kv_head, size_t head_dim, size_t group, size_t first, size_t pos, float scale,
                      float *out_group);
/* All heads of one row (attend_one, attention.rs:403-428). */
void orc_attend_one(const float *q_row, const uint16_t *kcache, const uint16_t *vcache, size_t kv_dim,
                    size_t n_kv_heads, size_t head_dim, size_t group, size_t first, size_t pos, float scale,
                    float *out_row);
/* The naive formulation the reference pins attend_group against (attend_head, attention.rs:430-465):
 * one q head, buffered softmax (ops/activation.rs:5-16).  out accumulates. */
void orc_attend_head(const float *qh, const uint16_t *kcache, const uint16_t *vcache, size_t kv_dim,
                     size_t kv_head, size_t head_dim, size_t pos, float scale, float *out);

int orc_cpu_threads(void);

#ifdef __cplusplus
}
#endif
#endif
