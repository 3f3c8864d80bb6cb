/*
 * apk_oracle.c -- CPU restatement of allpaka's reference dequant-matvec path.
 * TEST INFRASTRUCTURE ONLY (see apk_oracle.h).  Plain C, no intrinsics: the
 * statement order below is the arithmetic contract; the compiler may
 * vectorise integer sums but, without -ffast-math, no float sum is reordered.
 */
#include "apk_oracle.h"

#include <float.h>
#include <math.h>
#include <pthread.h>
#include <stdlib.h>
#include <string.h>
#include <unistd.h>

/* ------------------------------------------------------------------ dtype */

static inline uint32_t f32_bits(float x) { uint32_t b; memcpy(&b, &x, 4); return b; }
static inline float bits_f32(uint32_t b) { float x; memcpy(&x, &b, 4); return x; }

/* crates/allpaka-dtype/src/lib.rs:129-147 */
float orc_f16_to_f32(uint16_t h) {
    uint32_t sign = (h >> 15) & 1u, exp = (h >> 10) & 0x1fu, frac = h & 0x3ffu, bits;
    if (exp == 0 && frac == 0) {
        bits = sign << 31;
    } else if (exp == 0) {
        uint32_t p = 31u - (uint32_t)__builtin_clz(frac);
        uint32_t e = 127u - 24u + p;
        uint32_t f = (frac << (23u - p)) & 0x7fffffu;
        bits = (sign << 31) | (e << 23) | f;
    } else if (exp == 0x1f) {
        bits = (sign << 31) | 0x7f800000u | (frac << 13);
    } else {
        bits = (sign << 31) | ((exp + 127u - 15u) << 23) | (frac << 13);
    }
    return bits_f32(bits);
}

/* crates/allpaka-dtype/src/lib.rs:151-184 */
uint16_t orc_f32_to_f16(float x) {
    uint32_t bits = f32_bits(x);
    uint16_t sign = (uint16_t)((bits >> 16) & 0x8000u);
    uint32_t mag = bits & 0x7fffffffu;
    if (mag >= 0x7f800000u) {
        uint16_t man = mag > 0x7f800000u ? 0x200 : 0;
        return sign | 0x7c00 | man;
    }
    int exp = (int)(mag >> 23) - 127;
    if (exp >= 16) return sign | 0x7c00;
    if (exp >= -14) {
        uint32_t man = mag & 0x7fffffu;
        uint16_t h = (uint16_t)(((uint32_t)(exp + 15) << 10) | (man >> 13));
        uint32_t rest = man & 0x1fffu;
        if (rest > 0x1000u || (rest == 0x1000u && (h & 1))) h += 1;
        return sign | h;
    }
    if (exp < -25) return sign;
    uint32_t man = (mag & 0x7fffffu) | 0x800000u;
    uint32_t shift = (uint32_t)(-exp - 14);
    uint16_t h = (uint16_t)(man >> (13 + shift));
    uint32_t rest = man & ((1u << (13 + shift)) - 1u);
    uint32_t halfway = 1u << (12 + shift);
    if (rest > halfway || (rest == halfway && (h & 1))) h += 1;
    return sign | h;
}

/* crates/allpaka-dtype/src/lib.rs:188-190 */
float orc_bf16_to_f32(uint16_t h) { return bits_f32((uint32_t)h << 16); }

/* crates/allpaka-dtype/src/lib.rs:194-201 */
uint16_t orc_f32_to_bf16(float x) {
    uint32_t bits = f32_bits(x);
    if ((bits & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((bits >> 16) | 0x0040u);
    uint32_t bias = 0x00007fffu + ((bits >> 16) & 1u);
    return (uint16_t)((bits + bias) >> 16);
}

/* crates/allpaka-dtype/src/lib.rs:382-390 */
void orc_scale_min_k4(int j, const uint8_t *p, float *sc, float *mn) {
    if (j < 4) {
        *sc = (float)(p[j] & 63);
        *mn = (float)(p[j + 4] & 63);
    } else {
        uint8_t s = (uint8_t)((p[j + 4] & 0xf) | ((p[j - 4] >> 6) << 4));
        uint8_t m = (uint8_t)((p[j + 4] >> 4) | ((p[j] >> 6) << 4));
        *sc = (float)s;
        *mn = (float)m;
    }
}

static int block_geom(uint32_t ty, size_t *be, size_t *bb) {
    /* crates/allpaka-dtype/src/lib.rs:79-108 */
    if (ty == ORC_TY_Q8_0) { *be = 32; *bb = 34; return 0; }
    if (ty == ORC_TY_Q5_0) { *be = 32; *bb = 22; return 0; }
    if (ty == ORC_TY_Q3_K) { *be = 256; *bb = 110; return 0; }
    if (ty == ORC_TY_Q2_K) { *be = 256; *bb = 84; return 0; }
    if (ty == ORC_TY_Q4_K) { *be = 256; *bb = 144; return 0; }
    if (ty == ORC_TY_Q5_K) { *be = 256; *bb = 176; return 0; }
    if (ty == ORC_TY_Q6_K) { *be = 256; *bb = 210; return 0; }
    return -1;
}

size_t orc_expected_bytes(uint32_t ty, size_t elements) {
    size_t be, bb;
    if (block_geom(ty, &be, &bb) || elements % be) return 0;
    return elements / be * bb;
}

/* ---------------------------------------------------------------- dequant */

static inline uint16_t le16(const uint8_t *p) { return (uint16_t)(p[0] | (p[1] << 8)); }

/* crates/allpaka-gguf/src/dequant.rs:94-126 (scalar arm 122-125) */
static void dequant_q8_0_block(const uint8_t *b, float *out) {
    float d = orc_f16_to_f32(le16(b));
    for (int i = 0; i < 32; i++) out[i] = d * (float)(int8_t)b[2 + i];
}

/* The 32 values q - 16 of a Q5_0 block {f16 d; u32 qh; u8 qs[16]}: element j takes the low nibble of
 * qs[j] and bit j of qh, element j + 16 the high nibble and bit j + 16
 * (crates/allpaka-backend/src/quantmat/q8_acts.rs:115-120, dequant.rs:135-138). */
static void q5_0_values(const uint8_t *b, int8_t out[32]) {
    uint32_t qh = (uint32_t)b[2] | ((uint32_t)b[3] << 8) | ((uint32_t)b[4] << 16) | ((uint32_t)b[5] << 24);
    const uint8_t *qs = b + 6;
    for (int j = 0; j < 16; j++) {
        out[j] = (int8_t)((int)((qs[j] & 0x0f) | (((qh >> j) & 1u) << 4)) - 16);
        out[j + 16] = (int8_t)((int)((qs[j] >> 4) | (((qh >> (j + 16)) & 1u) << 4)) - 16);
    }
}

/* crates/allpaka-gguf/src/dequant.rs:131-141 */
static void dequant_q5_0_block(const uint8_t *b, float *out) {
    float d = orc_f16_to_f32(le16(b));
    int8_t q[32];
    q5_0_values(b, q);
    for (int i = 0; i < 32; i++) out[i] = d * (float)q[i];
}

/* The 32 two-bit values of block blk (0..7) of a Q2_K super-block {u8 scales[16]; u8 qs[64]; f16 d; f16 dmin}:
 * qs[32 * (blk / 4) + l] at shift 2 * (blk % 4) (q8_acts.rs:148-152, dequant.rs:158-166). */
static void q2_k_values(const uint8_t *block, int blk, int8_t out[32]) {
    const uint8_t *q = block + 16 + (blk / 4) * 32;
    int shift = 2 * (blk % 4);
    for (int l = 0; l < 32; l++) out[l] = (int8_t)((q[l] >> shift) & 3);
}

/* crates/allpaka-gguf/src/dequant.rs:150-174: x = d * (sc & 15) * q - dmin * (sc >> 4) per 16-element sub-block */
static void dequant_q2_k_block(const uint8_t *b, float *out) {
    float d = orc_f16_to_f32(le16(b + 80)), dmin = orc_f16_to_f32(le16(b + 82));
    for (int blk = 0; blk < 8; blk++) {
        int8_t q[32];
        q2_k_values(b, blk, q);
        for (int group = 0; group < 2; group++) {
            uint8_t sc = b[2 * blk + group];
            float dl = d * (float)(sc & 0xf), ml = dmin * (float)(sc >> 4);
            for (int l = 0; l < 16; l++) out[blk * 32 + group * 16 + l] = dl * (float)q[group * 16 + l] - ml;
        }
    }
}

/* Q3_K block {u8 hmask[32]; u8 qs[64]; u8 scales[12]; f16 d}: the 16 six-bit sub-block scales, still
 * biased by 32 (crates/allpaka-dtype/src/lib.rs:395-404). */
static void q3_k_scales_raw(const uint8_t *packed, int raw[16]) {
    for (int i = 0; i < 4; i++) {
        raw[i] = (packed[i] & 0x0f) | ((packed[8 + i] & 3) << 4);
        raw[4 + i] = (packed[4 + i] & 0x0f) | (((packed[8 + i] >> 2) & 3) << 4);
        raw[8 + i] = (packed[i] >> 4) | (((packed[8 + i] >> 4) & 3) << 4);
        raw[12 + i] = (packed[4 + i] >> 4) | (((packed[8 + i] >> 6) & 3) << 4);
    }
}

/* The 32 signed 3-bit values of block blk (0..7) of a super-block: two bits from qs at shift
 * 2 * (blk % 4), minus 4 where bit blk of hmask is clear (q8_acts.rs:203-205, dequant.rs:193-195). */
static void q3_k_values(const uint8_t *block, int blk, int8_t out[32]) {
    const uint8_t *hmask = block, *q = block + 32 + (blk / 4) * 32;
    int shift = 2 * (blk % 4);
    uint8_t m = (uint8_t)(1u << blk);
    for (int l = 0; l < 32; l++) out[l] = (int8_t)(((q[l] >> shift) & 3) - ((hmask[l] & m) ? 0 : 4));
}

/* crates/allpaka-gguf/src/dequant.rs:176-204 */
static void dequant_q3_k_block(const uint8_t *b, float *out) {
    float d_all = orc_f16_to_f32(le16(b + 108));
    int raw[16];
    q3_k_scales_raw(b + 96, raw);
    for (int blk = 0; blk < 8; blk++) {
        int8_t q[32];
        q3_k_values(b, blk, q);
        for (int group = 0; group < 2; group++) {
            float dl = d_all * (float)(raw[2 * blk + group] - 32);
            for (int l = 0; l < 16; l++) out[blk * 32 + group * 16 + l] = dl * (float)q[group * 16 + l];
        }
    }
}

/* crates/allpaka-gguf/src/dequant.rs:211-231 */
static void dequant_q4_k_block(const uint8_t *b, float *out) {
    float d = orc_f16_to_f32(le16(b));
    float dmin = orc_f16_to_f32(le16(b + 2));
    const uint8_t *packed = b + 4, *qs = b + 16;
    for (int pair = 0; pair < 4; pair++) {
        const uint8_t *q = qs + pair * 32;
        float sc1, mn1, sc2, mn2;
        orc_scale_min_k4(pair * 2, packed, &sc1, &mn1);
        orc_scale_min_k4(pair * 2 + 1, packed, &sc2, &mn2);
        float d_sc1 = d * sc1, dm1 = dmin * mn1, d_sc2 = d * sc2, dm2 = dmin * mn2;
        int base = pair * 64;
        for (int l = 0; l < 32; l++) {
            out[base + l] = d_sc1 * (float)(q[l] & 0xf) - dm1;
            out[base + 32 + l] = d_sc2 * (float)(q[l] >> 4) - dm2;
        }
    }
}

/* crates/allpaka-gguf/src/dequant.rs:238-263 */
static void dequant_q5_k_block(const uint8_t *b, float *out) {
    float d = orc_f16_to_f32(le16(b));
    float dmin = orc_f16_to_f32(le16(b + 2));
    const uint8_t *packed = b + 4, *qh = b + 16, *qs = b + 48;
    for (int pair = 0; pair < 4; pair++) {
        const uint8_t *q = qs + pair * 32;
        float sc1, mn1, sc2, mn2;
        orc_scale_min_k4(pair * 2, packed, &sc1, &mn1);
        orc_scale_min_k4(pair * 2 + 1, packed, &sc2, &mn2);
        float d_sc1 = d * sc1, dm1 = dmin * mn1, d_sc2 = d * sc2, dm2 = dmin * mn2;
        uint8_t bit1 = (uint8_t)(1u << (pair * 2)), bit2 = (uint8_t)(1u << (pair * 2 + 1));
        int base = pair * 64;
        for (int l = 0; l < 32; l++) {
            int hi1 = (qh[l] & bit1) ? 16 : 0, hi2 = (qh[l] & bit2) ? 16 : 0;
            out[base + l] = d_sc1 * (float)((q[l] & 0xf) + hi1) - dm1;
            out[base + 32 + l] = d_sc2 * (float)((q[l] >> 4) + hi2) - dm2;
        }
    }
}

/* The four 6-bit values that share index l of one 128-element half: ql low/high nibbles of bytes
 * l and l+32, high bits from successive 2-bit fields of qh[l], each minus 32
 * (crates/allpaka-gguf/src/dequant.rs:285-289; the same lines in q8_acts.rs:329-333). */
static inline void q6_k_four(const uint8_t *ql, const uint8_t *qh, int l, int q[4]) {
    q[0] = (int)(int8_t)((ql[l] & 0xf) | ((qh[l] & 3) << 4)) - 32;
    q[1] = (int)(int8_t)((ql[l + 32] & 0xf) | (((qh[l] >> 2) & 3) << 4)) - 32;
    q[2] = (int)(int8_t)((ql[l] >> 4) | (((qh[l] >> 4) & 3) << 4)) - 32;
    q[3] = (int)(int8_t)((ql[l + 32] >> 4) | (((qh[l] >> 6) & 3) << 4)) - 32;
}

/* crates/allpaka-gguf/src/dequant.rs:271-296 */
static void dequant_q6_k_block(const uint8_t *b, float *out) {
    const uint8_t *scales = b + 192;
    float d = orc_f16_to_f32(le16(b + 208));
    for (int half = 0; half < 2; half++) {
        const uint8_t *ql = b + half * 64, *qh = b + 128 + half * 32;
        const int8_t *sc = (const int8_t *)scales + half * 8;
        float *o = out + half * 128;
        for (int l = 0; l < 32; l++) {
            int is = l / 16, q[4];
            q6_k_four(ql, qh, l, q);
            o[l] = d * (float)sc[is] * (float)q[0];
            o[32 + l] = d * (float)sc[is + 2] * (float)q[1];
            o[64 + l] = d * (float)sc[is + 4] * (float)q[2];
            o[96 + l] = d * (float)sc[is + 6] * (float)q[3];
        }
    }
}

int orc_dequant(uint32_t ty, const uint8_t *bytes, size_t n_bytes, float *out, size_t n) {
    size_t be, bb;
    if (block_geom(ty, &be, &bb) || n % be || n / be * bb != n_bytes) return -1;
    for (size_t i = 0; i < n / be; i++) {
        if (ty == ORC_TY_Q8_0) dequant_q8_0_block(bytes + i * bb, out + i * be);
        else if (ty == ORC_TY_Q5_0) dequant_q5_0_block(bytes + i * bb, out + i * be);
        else if (ty == ORC_TY_Q3_K) dequant_q3_k_block(bytes + i * bb, out + i * be);
        else if (ty == ORC_TY_Q2_K) dequant_q2_k_block(bytes + i * bb, out + i * be);
        else if (ty == ORC_TY_Q4_K) dequant_q4_k_block(bytes + i * bb, out + i * be);
        else if (ty == ORC_TY_Q5_K) dequant_q5_k_block(bytes + i * bb, out + i * be);
        else dequant_q6_k_block(bytes + i * bb, out + i * be);
    }
    return 0;
}

/* --------------------------------------------------------- Q8 activations */

/* f32 -> i8 the way Rust's `as i8` does it: saturating, NaN -> 0. */
static inline int8_t sat_i8(float v) {
    if (v != v) return 0;
    if (v >= 127.0f) return 127;
    if (v <= -128.0f) return -128;
    return (int8_t)v;
}

/* crates/allpaka-backend/src/quantmat/q8_acts.rs:26-63 (arms 38-41, 56-58) */
void orc_q8acts_from_f32(const float *x, size_t n, float *d, float *sum, int8_t *q) {
    size_t blocks = n / 32;
    for (size_t b = 0; b < blocks; b++) {
        const float *xs = x + b * 32;
        float amax = 0.0f, block_sum = 0.0f;
        /* fold(0, |m,v| m.max(v.abs())): f32::max ignores a NaN operand */
        for (int i = 0; i < 32; i++) amax = fmaxf(amax, fabsf(xs[i]));
        /* iter().sum::<f32>() folds from +0.0... Rust's f32 Sum starts at -0.0
         * since 1.83?  Either start gives identical results unless every term
         * is a zero, where the sign of zero is immaterial to every consumer. */
        for (int i = 0; i < 32; i++) block_sum += xs[i];
        float db = isfinite(amax) ? amax / 127.0f : 0.0f;
        float id = (db > 0.0f && isfinite(db)) ? 1.0f / db : 0.0f;
        for (int i = 0; i < 32; i++) q[b * 32 + i] = sat_i8(roundf(xs[i] * id));
        d[b] = db;
        sum[b] = block_sum;
    }
}

/* crates/allpaka-backend/src/quantmat/q8_acts.rs:353-365 (scalar arm 364) */
int32_t orc_dot_i8(const int8_t *a, const int8_t *b, size_t n) {
    int32_t s = 0;
    for (size_t i = 0; i < n; i++) s += (int32_t)a[i] * (int32_t)b[i];
    return s;
}

static inline int32_t dot_i8_32(const int8_t *a, const int8_t *b) {
    int32_t s = 0;
    for (int i = 0; i < 32; i++) s += (int32_t)a[i] * (int32_t)b[i];
    return s;
}

/* crates/allpaka-backend/src/quantmat/q8_acts.rs:86-96 */
float orc_dot_q8_0_i8(const uint8_t *row, size_t n_in, const float *d, const int8_t *q) {
    float total = 0.0f;
    size_t nb = n_in / 32;
    for (size_t bi = 0; bi < nb; bi++) {
        const uint8_t *block = row + bi * 34;
        float dw = orc_f16_to_f32(le16(block));
        /* total += d * acts.d[bi] * dot as f32  ==  total + ((d*dx)*dot) */
        total += dw * d[bi] * (float)dot_i8_32((const int8_t *)(block + 2), q + bi * 32);
    }
    return total;
}

/* crates/allpaka-backend/src/quantmat/q8_acts.rs:267-301 */
float orc_dot_q4_k_i8(const uint8_t *row, size_t n_in, const float *dx, const float *sum,
                      const int8_t *q8) {
    float total = 0.0f;
    size_t nsb = n_in / 256;
    for (size_t bi = 0; bi < nsb; bi++) {
        const uint8_t *block = row + bi * 144;
        float d = orc_f16_to_f32(le16(block));
        float dmin = orc_f16_to_f32(le16(block + 2));
        const uint8_t *packed = block + 4, *qs = block + 16;
        for (int pair = 0; pair < 4; pair++) {
            const uint8_t *q = qs + pair * 32;
            float sc1, mn1, sc2, mn2;
            orc_scale_min_k4(pair * 2, packed, &sc1, &mn1);
            orc_scale_min_k4(pair * 2 + 1, packed, &sc2, &mn2);
            int8_t lo[32], hi[32];
            for (int l = 0; l < 32; l++) {
                lo[l] = (int8_t)(q[l] & 0xf);
                hi[l] = (int8_t)(q[l] >> 4);
            }
            size_t b_lo = bi * 8 + (size_t)pair * 2, b_hi = b_lo + 1;
            float dot_lo = (float)dot_i8_32(lo, q8 + b_lo * 32) * dx[b_lo];
            float dot_hi = (float)dot_i8_32(hi, q8 + b_hi * 32) * dx[b_hi];
            total += d * sc1 * dot_lo - dmin * mn1 * sum[b_lo];
            total += d * sc2 * dot_hi - dmin * mn2 * sum[b_hi];
        }
    }
    return total;
}

/* crates/allpaka-backend/src/quantmat/q8_acts.rs:100-124 (the not(aarch64) arm): total += d * d_x[b] * dot */
float orc_dot_q5_0_i8(const uint8_t *row, size_t n_in, const float *dx, const int8_t *q8) {
    float total = 0.0f;
    for (size_t bi = 0; bi < n_in / 32; bi++) {
        const uint8_t *block = row + bi * 22;
        float d = orc_f16_to_f32(le16(block));
        int8_t qw[32];
        q5_0_values(block, qw);
        total += d * dx[bi] * (float)dot_i8_32(qw, q8 + bi * 32);
    }
    return total;
}

/* crates/allpaka-backend/src/quantmat/dot_f32.rs:39-55: per block s += x0 * xs[j] + x1 * xs[j + 16], total += d * s */
float orc_dot_q5_0(const uint8_t *row, size_t n_in, const float *x) {
    float total = 0.0f;
    for (size_t bi = 0; bi < n_in / 32; bi++) {
        const uint8_t *block = row + bi * 22;
        float d = orc_f16_to_f32(le16(block));
        int8_t q[32];
        q5_0_values(block, q);
        const float *xs = x + bi * 32;
        float s = 0.0f;
        for (int j = 0; j < 16; j++) s += (float)q[j] * xs[j] + (float)q[j + 16] * xs[j + 16];
        total += d * s;
    }
    return total;
}

/* crates/allpaka-backend/src/quantmat/q8_acts.rs:127-174 (the not(aarch64) arm): per 16-element sub-block
 * total += dl * dotq - ml * sum_x, dotq and sum_x over the activation codes, each times d_x of the block */
float orc_dot_q2_k_i8(const uint8_t *row, size_t n_in, const float *dx_all, const int8_t *q8) {
    float total = 0.0f;
    for (size_t bi = 0; bi < n_in / 256; bi++) {
        const uint8_t *block = row + bi * 84;
        float d = orc_f16_to_f32(le16(block + 80)), dmin = orc_f16_to_f32(le16(block + 82));
        for (int b = 0; b < 8; b++) {
            size_t blk = bi * 8 + (size_t)b;
            const int8_t *xq = q8 + blk * 32;
            float dx = dx_all[blk];
            int8_t qw[32];
            q2_k_values(block, b, qw);
            for (int group = 0; group < 2; group++) {
                uint8_t sc = block[2 * b + group];
                float dl = d * (float)(sc & 0xf);
                float ml = dmin * (float)(sc >> 4);
                float dotq = (float)orc_dot_i8(qw + group * 16, xq + group * 16, 16) * dx;
                int32_t s = 0;
                for (int l = 0; l < 16; l++) s += xq[group * 16 + l];
                float sum_x = (float)s * dx;
                total += dl * dotq - ml * sum_x;
            }
        }
    }
    return total;
}

/* crates/allpaka-backend/src/quantmat/dot_f32.rs:214-248 */
float orc_dot_q2_k(const uint8_t *row, size_t n_in, const float *x) {
    float total = 0.0f;
    for (size_t bi = 0; bi < n_in / 256; bi++) {
        const uint8_t *block = row + bi * 84;
        float d = orc_f16_to_f32(le16(block + 80)), dmin = orc_f16_to_f32(le16(block + 82));
        const float *xb = x + bi * 256;
        float acc_d = 0.0f, acc_m = 0.0f;
        for (int b = 0; b < 8; b++) {
            int8_t q[32];
            q2_k_values(block, b, q);
            for (int group = 0; group < 2; group++) {
                uint8_t sc = block[2 * b + group];
                const float *xs = xb + b * 32 + group * 16;
                float dotq = 0.0f, sum = 0.0f;
                for (int l = 0; l < 16; l++) {
                    dotq += (float)q[group * 16 + l] * xs[l];
                    sum += xs[l];
                }
                acc_d += (float)(sc & 0xf) * dotq;
                acc_m += (float)(sc >> 4) * sum;
            }
        }
        total += d * acc_d - dmin * acc_m;
    }
    return total;
}

/* crates/allpaka-backend/src/quantmat/q8_acts.rs:178-218 (the not(aarch64) arm):
 * total += d_all * dx * (sc0 * dot0 + sc1 * dot1) per 32-element block */
float orc_dot_q3_k_i8(const uint8_t *row, size_t n_in, const float *dx, const int8_t *q8) {
    float total = 0.0f;
    for (size_t bi = 0; bi < n_in / 256; bi++) {
        const uint8_t *block = row + bi * 110;
        float d_all = orc_f16_to_f32(le16(block + 108));
        int raw[16];
        q3_k_scales_raw(block + 96, raw);
        for (int b = 0; b < 8; b++) {
            size_t blk = bi * 8 + (size_t)b;
            int8_t qw[32];
            q3_k_values(block, b, qw);
            float dot0 = (float)orc_dot_i8(qw, q8 + blk * 32, 16);
            float dot1 = (float)orc_dot_i8(qw + 16, q8 + blk * 32 + 16, 16);
            float sc0 = (float)(raw[2 * b] - 32), sc1 = (float)(raw[2 * b + 1] - 32);
            total += d_all * dx[blk] * (sc0 * dot0 + sc1 * dot1);
        }
    }
    return total;
}

/* crates/allpaka-backend/src/quantmat/dot_f32.rs:58-94: sub-block sums weighted by their scales, one
 * multiplication by d per super-block */
float orc_dot_q3_k(const uint8_t *row, size_t n_in, const float *x) {
    float total = 0.0f;
    for (size_t bi = 0; bi < n_in / 256; bi++) {
        const uint8_t *block = row + bi * 110;
        float d_all = orc_f16_to_f32(le16(block + 108));
        const float *xb = x + bi * 256;
        int raw[16];
        q3_k_scales_raw(block + 96, raw);
        float blk_sum = 0.0f;
        for (int b = 0; b < 8; b++) {
            int8_t q[32];
            q3_k_values(block, b, q);
            for (int group = 0; group < 2; group++) {
                float sub = 0.0f;
                for (int l = 0; l < 16; l++) sub += (float)q[group * 16 + l] * xb[b * 32 + group * 16 + l];
                blk_sum += (float)(raw[2 * b + group] - 32) * sub;
            }
        }
        total += d_all * blk_sum;
    }
    return total;
}

/* The 5-bit values of the two sub-blocks of pair `pair` (q8_acts.rs:247-252). */
static void q5_k_pair(const uint8_t *q, const uint8_t *qh, int pair, int8_t lo[32], int8_t hi[32]) {
    for (int l = 0; l < 32; l++) {
        uint8_t h1 = (uint8_t)(((qh[l] >> (pair * 2)) & 1) << 4), h2 = (uint8_t)(((qh[l] >> (pair * 2 + 1)) & 1) << 4);
        lo[l] = (int8_t)((q[l] & 0x0f) | h1);
        hi[l] = (int8_t)((q[l] >> 4) | h2);
    }
}

/* crates/allpaka-backend/src/quantmat/q8_acts.rs:223-262 */
float orc_dot_q5_k_i8(const uint8_t *row, size_t n_in, const float *dx, const float *sum, const int8_t *q8) {
    float total = 0.0f;
    size_t nsb = n_in / 256;
    for (size_t bi = 0; bi < nsb; bi++) {
        const uint8_t *block = row + bi * 176;
        float d = orc_f16_to_f32(le16(block));
        float dmin = orc_f16_to_f32(le16(block + 2));
        const uint8_t *packed = block + 4, *qh = block + 16, *qs = block + 48;
        for (int pair = 0; pair < 4; pair++) {
            float sc1, mn1, sc2, mn2;
            orc_scale_min_k4(pair * 2, packed, &sc1, &mn1);
            orc_scale_min_k4(pair * 2 + 1, packed, &sc2, &mn2);
            int8_t lo[32], hi[32];
            q5_k_pair(qs + pair * 32, qh, pair, lo, hi);
            size_t b_lo = bi * 8 + (size_t)pair * 2, b_hi = b_lo + 1;
            float dot_lo = (float)dot_i8_32(lo, q8 + b_lo * 32) * dx[b_lo];
            float dot_hi = (float)dot_i8_32(hi, q8 + b_hi * 32) * dx[b_hi];
            total += d * sc1 * dot_lo - dmin * mn1 * sum[b_lo];
            total += d * sc2 * dot_hi - dmin * mn2 * sum[b_hi];
        }
    }
    return total;
}

/* crates/allpaka-backend/src/quantmat/dot_f32.rs:97-135 */
float orc_dot_q5_k(const uint8_t *row, size_t n_in, const float *x) {
    float total = 0.0f;
    size_t nsb = n_in / 256;
    for (size_t bi = 0; bi < nsb; bi++) {
        const uint8_t *block = row + bi * 176;
        float d = orc_f16_to_f32(le16(block));
        float dmin = orc_f16_to_f32(le16(block + 2));
        const uint8_t *packed = block + 4, *qh = block + 16, *qs = block + 48;
        const float *xb = x + bi * 256;
        float acc_d = 0.0f, acc_m = 0.0f;
        for (int pair = 0; pair < 4; pair++) {
            const uint8_t *q = qs + pair * 32;
            const float *x_lo = xb + pair * 64, *x_hi = xb + pair * 64 + 32;
            float sc1, mn1, sc2, mn2;
            orc_scale_min_k4(pair * 2, packed, &sc1, &mn1);
            orc_scale_min_k4(pair * 2 + 1, packed, &sc2, &mn2);
            uint8_t bit1 = (uint8_t)(1u << (pair * 2)), bit2 = (uint8_t)(1u << (pair * 2 + 1));
            float dot_lo = 0.0f, sum_lo = 0.0f, dot_hi = 0.0f, sum_hi = 0.0f;
            for (int l = 0; l < 32; l++) {
                int hi1 = (qh[l] & bit1) ? 16 : 0, hi2 = (qh[l] & bit2) ? 16 : 0;
                dot_lo += (float)((q[l] & 0xf) + hi1) * x_lo[l];
                sum_lo += x_lo[l];
                dot_hi += (float)((q[l] >> 4) + hi2) * x_hi[l];
                sum_hi += x_hi[l];
            }
            acc_d += sc1 * dot_lo + sc2 * dot_hi;
            acc_m += mn1 * sum_lo + mn2 * sum_hi;
        }
        total += d * acc_d - dmin * acc_m;
    }
    return total;
}

/* The signed 6-bit values of quarter qi (0..3) of one half, in element order. */
static void q6_k_quarter(const uint8_t *ql, const uint8_t *qh, int qi, int8_t out[32]) {
    for (int l = 0; l < 32; l++) {
        int q[4];
        q6_k_four(ql, qh, l, q);
        out[l] = (int8_t)q[qi];
    }
}

/* crates/allpaka-backend/src/quantmat/q8_acts.rs:307-346 (the non-aarch64 arm 328-334) */
float orc_dot_q6_k_i8(const uint8_t *row, size_t n_in, const float *dx, const int8_t *q8) {
    float total = 0.0f;
    size_t nsb = n_in / 256;
    for (size_t bi = 0; bi < nsb; bi++) {
        const uint8_t *block = row + bi * 210;
        float d = orc_f16_to_f32(le16(block + 208));
        for (int half = 0; half < 2; half++) {
            const uint8_t *ql = block + half * 64, *qh = block + 128 + half * 32;
            const int8_t *sc = (const int8_t *)block + 192 + half * 8;
            for (int qi = 0; qi < 4; qi++) {
                int8_t qq[32];
                q6_k_quarter(ql, qh, qi, qq);
                size_t blk = bi * 8 + (size_t)half * 4 + (size_t)qi;
                const int8_t *xq = q8 + blk * 32;
                float dot0 = (float)orc_dot_i8(qq, xq, 16);
                float dot1 = (float)orc_dot_i8(qq + 16, xq + 16, 16);
                float sc0 = (float)sc[2 * qi], sc1 = (float)sc[2 * qi + 1];
                total += d * dx[blk] * (sc0 * dot0 + sc1 * dot1);
            }
        }
    }
    return total;
}

/* crates/allpaka-backend/src/quantmat/dot_f32.rs:252-289 */
float orc_dot_q6_k(const uint8_t *row, size_t n_in, const float *x) {
    float total = 0.0f;
    size_t nsb = n_in / 256;
    for (size_t bi = 0; bi < nsb; bi++) {
        const uint8_t *block = row + bi * 210;
        float d = orc_f16_to_f32(le16(block + 208));
        const float *xb = x + bi * 256;
        float blk_sum = 0.0f;
        for (int half = 0; half < 2; half++) {
            const uint8_t *ql = block + half * 64, *qh = block + 128 + half * 32;
            const int8_t *sc = (const int8_t *)block + 192 + half * 8;
            const float *xh = xb + half * 128;
            float acc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
            for (int is = 0; is < 2; is++) {
                for (int l = is * 16; l < is * 16 + 16; l++) {
                    int q[4];
                    q6_k_four(ql, qh, l, q);
                    acc[is] += (float)q[0] * xh[l];
                    acc[2 + is] += (float)q[1] * xh[l + 32];
                    acc[4 + is] += (float)q[2] * xh[l + 64];
                    acc[6 + is] += (float)q[3] * xh[l + 96];
                }
            }
            for (int g = 0; g < 8; g++) blk_sum += (float)sc[g] * acc[g];
        }
        total += d * blk_sum;
    }
    return total;
}

/* crates/allpaka-backend/src/quantmat/dot_f32.rs:140-160 (scalar arm 150-156) */
float orc_dot_q8_0(const uint8_t *row, size_t n_in, const float *x) {
    float total = 0.0f;
    size_t nb = n_in / 32;
    for (size_t bi = 0; bi < nb; bi++) {
        const uint8_t *block = row + bi * 34;
        float d = orc_f16_to_f32(le16(block));
        const float *xs = x + bi * 32;
        float s = 0.0f;
        for (int i = 0; i < 32; i++) s += (float)(int8_t)block[2 + i] * xs[i];
        total += d * s;
    }
    return total;
}

/* crates/allpaka-backend/src/quantmat/dot_f32.rs:166-210 */
float orc_dot_q4_k(const uint8_t *row, size_t n_in, const float *x) {
    float total = 0.0f;
    size_t nsb = n_in / 256;
    for (size_t bi = 0; bi < nsb; bi++) {
        const uint8_t *block = row + bi * 144;
        float d = orc_f16_to_f32(le16(block));
        float dmin = orc_f16_to_f32(le16(block + 2));
        const uint8_t *packed = block + 4, *qs = block + 16;
        const float *xb = x + bi * 256;
        float acc_d = 0.0f, acc_m = 0.0f;
        for (int pair = 0; pair < 4; pair++) {
            const uint8_t *q = qs + pair * 32;
            const float *x_lo = xb + pair * 64, *x_hi = xb + pair * 64 + 32;
            float sc1, mn1, sc2, mn2;
            orc_scale_min_k4(pair * 2, packed, &sc1, &mn1);
            orc_scale_min_k4(pair * 2 + 1, packed, &sc2, &mn2);
            float dot_lo = 0.0f, sum_lo = 0.0f, dot_hi = 0.0f, sum_hi = 0.0f;
            for (int l = 0; l < 32; l++) {
                dot_lo += (float)(q[l] & 0xf) * x_lo[l];
                sum_lo += x_lo[l];
            }
            for (int l = 0; l < 32; l++) {
                dot_hi += (float)(q[l] >> 4) * x_hi[l];
                sum_hi += x_hi[l];
            }
            acc_d += sc1 * dot_lo + sc2 * dot_hi;
            acc_m += mn1 * sum_lo + mn2 * sum_hi;
        }
        total += d * acc_d - dmin * acc_m;
    }
    return total;
}

int orc_block_dots(uint32_t ty, const uint8_t *w, size_t n_out, size_t n_in, const int8_t *q,
                   size_t m, int32_t *dots) {
    size_t be, bb;
    if (block_geom(ty, &be, &bb) || n_in % be) return -1;
    size_t nb = n_in / 32, row_bytes = n_in / be * bb;
    for (size_t i = 0; i < m; i++) {
        const int8_t *qi = q + i * n_in;
        for (size_t j = 0; j < n_out; j++) {
            const uint8_t *row = w + j * row_bytes;
            int32_t *o = dots + (i * n_out + j) * nb;
            if (ty == ORC_TY_Q8_0) {
                for (size_t b = 0; b < nb; b++)
                    o[b] = dot_i8_32((const int8_t *)(row + b * 34 + 2), qi + b * 32);
            } else if (ty == ORC_TY_Q2_K) {
                /* per 32-element block the integer that d * d_x multiplies: sc0*dot0 + sc1*dot1 with the
                 * 4-bit scales (q8_acts.rs:156-168; the min term is not a dot with the weights) */
                for (size_t sb = 0; sb < n_in / 256; sb++) {
                    const uint8_t *block = row + sb * 84;
                    for (int b = 0; b < 8; b++) {
                        int8_t qw[32];
                        q2_k_values(block, b, qw);
                        size_t blk = sb * 8 + (size_t)b;
                        o[blk] = (int32_t)(block[2 * b] & 0xf) * orc_dot_i8(qw, qi + blk * 32, 16) +
                                 (int32_t)(block[2 * b + 1] & 0xf) * orc_dot_i8(qw + 16, qi + blk * 32 + 16, 16);
                    }
                }
            } else if (ty == ORC_TY_Q3_K) {
                /* per 32-element block the integer the f32 scales multiply: sc0*dot0 + sc1*dot1
                 * (q8_acts.rs:206-210; exact in f32 there) */
                for (size_t sb = 0; sb < n_in / 256; sb++) {
                    const uint8_t *block = row + sb * 110;
                    int raw[16];
                    q3_k_scales_raw(block + 96, raw);
                    for (int b = 0; b < 8; b++) {
                        int8_t qw[32];
                        q3_k_values(block, b, qw);
                        size_t blk = sb * 8 + (size_t)b;
                        o[blk] = (int32_t)(raw[2 * b] - 32) * orc_dot_i8(qw, qi + blk * 32, 16) +
                                 (int32_t)(raw[2 * b + 1] - 32) * orc_dot_i8(qw + 16, qi + blk * 32 + 16, 16);
                    }
                }
            } else if (ty == ORC_TY_Q5_0) {
                for (size_t b = 0; b < nb; b++) {
                    int8_t qw[32];
                    q5_0_values(row + b * 22, qw);
                    o[b] = dot_i8_32(qw, qi + b * 32);
                }
            } else if (ty == ORC_TY_Q5_K) {
                for (size_t sb = 0; sb < n_in / 256; sb++) {
                    const uint8_t *block = row + sb * 176;
                    for (int pair = 0; pair < 4; pair++) {
                        int8_t lo[32], hi[32];
                        q5_k_pair(block + 48 + pair * 32, block + 16, pair, lo, hi);
                        size_t b_lo = sb * 8 + (size_t)pair * 2;
                        o[b_lo] = dot_i8_32(lo, qi + b_lo * 32);
                        o[b_lo + 1] = dot_i8_32(hi, qi + (b_lo + 1) * 32);
                    }
                }
            } else if (ty == ORC_TY_Q6_K) {
                /* per 32-element block the integer the f32 scale multiplies: sc0*dot0 + sc1*dot1
                 * (q8_acts.rs:338-342; exact in f32 there, |value| < 2^24) */
                for (size_t sb = 0; sb < n_in / 256; sb++) {
                    const uint8_t *block = row + sb * 210;
                    for (int half = 0; half < 2; half++) {
                        const int8_t *sc = (const int8_t *)block + 192 + half * 8;
                        for (int qr = 0; qr < 4; qr++) {
                            int8_t qq[32];
                            q6_k_quarter(block + half * 64, block + 128 + half * 32, qr, qq);
                            size_t blk = sb * 8 + (size_t)half * 4 + (size_t)qr;
                            o[blk] = (int32_t)sc[2 * qr] * orc_dot_i8(qq, qi + blk * 32, 16) +
                                     (int32_t)sc[2 * qr + 1] * orc_dot_i8(qq + 16, qi + blk * 32 + 16, 16);
                        }
                    }
                }
            } else {
                for (size_t sb = 0; sb < n_in / 256; sb++) {
                    const uint8_t *qs = row + sb * 144 + 16;
                    for (int pair = 0; pair < 4; pair++) {
                        int8_t lo[32], hi[32];
                        for (int l = 0; l < 32; l++) {
                            lo[l] = (int8_t)(qs[pair * 32 + l] & 0xf);
                            hi[l] = (int8_t)(qs[pair * 32 + l] >> 4);
                        }
                        size_t b_lo = sb * 8 + (size_t)pair * 2;
                        o[b_lo] = dot_i8_32(lo, qi + b_lo * 32);
                        o[b_lo + 1] = dot_i8_32(hi, qi + (b_lo + 1) * 32);
                    }
                }
            }
        }
    }
    return 0;
}

/* ------------------------------------------------------------- threading */

/* ---------------------------------------------------------------- decode attention
 * crates/allpaka-model/src/model/attention.rs:337-399 (attend_group), 403-428 (attend_one),
 * 430-465 (attend_head, the test-only naive form); crates/allpaka-backend/src/ops/f16.rs scalar
 * arms of dot (63-69) and axpy (118-121); crates/allpaka-model/src/kv.rs:682-697 (store_at). */
void orc_kv_store(const float *row, size_t n, uint16_t *dst) {
    for (size_t i = 0; i < n; ++i) dst[i] = orc_f32_to_f16(row[i]);
}

static float f16_dot(const float *a, const uint16_t *b, size_t n) {
    float total = 0.0f;
    for (size_t k = 0; k < n; ++k) total += a[k] * orc_f16_to_f32(b[k]);
    return total;
}

void orc_attend_group(const float *q_group, const uint16_t *kcache, const uint16_t *vcache, size_t kv_dim,
                      size_t kv_head, size_t head_dim, size_t group, size_t first, size_t pos, float scale,
                      float *out_group) {
    float *maxes = (float *)malloc(group * sizeof(float));
    float *denoms = (float *)malloc(group * sizeof(float));
    for (size_t h = 0; h < group; ++h) {
        maxes[h] = -INFINITY;
        denoms[h] = 0.0f;
    }
    for (size_t t = first; t <= pos; ++t) {
        const uint16_t *kt = kcache + t * kv_dim + kv_head * head_dim;
        const uint16_t *vt = vcache + t * kv_dim + kv_head * head_dim;
        for (size_t h = 0; h < group; ++h) {
            const float *qh = q_group + h * head_dim;
            const float s = f16_dot(qh, kt, head_dim) * scale;
            float *acc = out_group + h * head_dim;
            if (s > maxes[h]) {
                if (denoms[h] > 0.0f) {
                    const float rescale = expf(maxes[h] - s);
                    for (size_t i = 0; i < head_dim; ++i) acc[i] *= rescale;
                    denoms[h] *= rescale;
                }
                maxes[h] = s;
            }
            const float p = expf(s - maxes[h]);
            denoms[h] += p;
            for (size_t i = 0; i < head_dim; ++i) acc[i] += p * orc_f16_to_f32(vt[i]);
        }
    }
    for (size_t h = 0; h < group; ++h) {
        const float dn = denoms[h] > FLT_MIN ? denoms[h] : FLT_MIN;  /* denom.max(f32::MIN_POSITIVE) */
        const float inv_d = 1.0f / dn;
        float *acc = out_group + h * head_dim;
        for (size_t i = 0; i < head_dim; ++i) acc[i] *= inv_d;
    }
    free(maxes);
    free(denoms);
}

void orc_attend_one(const float *q_row, const uint16_t *kcache, const uint16_t *vcache, size_t kv_dim,
                    size_t n_kv_heads, size_t head_dim, size_t group, size_t first, size_t pos, float scale,
                    float *out_row) {
    for (size_t kvh = 0; kvh < n_kv_heads; ++kvh) {
        const size_t at = kvh * group * head_dim;
        orc_attend_group(q_row + at, kcache, vcache, kv_dim, kvh, head_dim, group, first, pos, scale, out_row + at);
    }
}

void orc_attend_head(const float *qh, const uint16_t *kcache, const uint16_t *vcache, size_t kv_dim,
                     size_t kv_head, size_t head_dim, size_t pos, float scale, float *out) {
    float *scores = (float *)malloc((pos + 1) * sizeof(float));
    for (size_t t = 0; t <= pos; ++t) {
        const uint16_t *kt = kcache + t * kv_dim + kv_head * head_dim;
        float s = 0.0f;
        for (size_t i = 0; i < head_dim; ++i) s += qh[i] * orc_f16_to_f32(kt[i]);
        scores[t] = s * scale;
    }
    /* ops::softmax (ops/activation.rs:5-16) */
    float mx = -INFINITY;
    for (size_t t = 0; t <= pos; ++t) mx = scores[t] > mx ? scores[t] : mx;
    float sum = 0.0f;
    for (size_t t = 0; t <= pos; ++t) {
        scores[t] = expf(scores[t] - mx);
        sum += scores[t];
    }
    const float inv_sum = 1.0f / sum;
    for (size_t t = 0; t <= pos; ++t) scores[t] *= inv_sum;
    for (size_t t = 0; t <= pos; ++t) {
        const uint16_t *vt = vcache + t * kv_dim + kv_head * head_dim;
        for (size_t i = 0; i < head_dim; ++i) out[i] += scores[t] * orc_f16_to_f32(vt[i]);
    }
    free(scores);
}

int orc_cpu_threads(void) {
    /* std::thread::available_parallelism (runtime.rs:361-365) */
    long n = sysconf(_SC_NPROCESSORS_ONLN);
    return n > 0 ? (int)n : 1;
}

typedef void (*chunk_fn)(void *ctx, size_t start, size_t end);
typedef struct { chunk_fn f; void *ctx; size_t start, end; } chunk_job;

static void *chunk_tramp(void *p) {
    chunk_job *j = (chunk_job *)p;
    j->f(j->ctx, j->start, j->end);
    return NULL;
}

/* crates/allpaka-backend/src/thread_pool.rs:207-230: up to n_workers
 * contiguous chunks of ceil(total/nt) items; worker 0 is the caller. */
static void par_for_chunks(size_t total, int n_workers, chunk_fn f, void *ctx) {
    if (total == 0 || n_workers <= 0) return;
    size_t nt = (size_t)n_workers < total ? (size_t)n_workers : total;
    if (nt <= 1) { f(ctx, 0, total); return; }
    size_t per = (total + nt - 1) / nt;
    size_t chunks = (total + per - 1) / per;
    pthread_t *th = (pthread_t *)malloc(sizeof(pthread_t) * chunks);
    chunk_job *jobs = (chunk_job *)malloc(sizeof(chunk_job) * chunks);
    for (size_t t = 0; t < chunks; t++) {
        jobs[t].f = f; jobs[t].ctx = ctx;
        jobs[t].start = t * per;
        jobs[t].end = (t + 1) * per < total ? (t + 1) * per : total;
        if (t > 0) pthread_create(&th[t], NULL, chunk_tramp, &jobs[t]);
    }
    chunk_tramp(&jobs[0]);
    for (size_t t = 1; t < chunks; t++) pthread_join(th[t], NULL);
    free(th);
    free(jobs);
}

/* ---------------------------------------------------------------- matmul */

typedef struct {
    uint32_t ty;
    const uint8_t *w;
    size_t n_out, n_in, row_bytes, m;
    const float *x;     /* [m][n_in] */
    const float *d, *sum;
    const int8_t *q;    /* Q8 acts, or NULL for the f32 path */
    float *y;           /* [m][n_out] */
} mm_ctx;

/* row_dot_dispatch (mod.rs:288-305) / row_dot (mod.rs:706-735) */
static inline float row_dot_any(const mm_ctx *c, size_t i, size_t j) {
    const uint8_t *row = c->w + j * c->row_bytes;
    size_t nb = c->n_in / 32;
    if (c->q) {
        if (c->ty == ORC_TY_Q8_0)
            return orc_dot_q8_0_i8(row, c->n_in, c->d + i * nb, c->q + i * c->n_in);
        if (c->ty == ORC_TY_Q5_0)
            return orc_dot_q5_0_i8(row, c->n_in, c->d + i * nb, c->q + i * c->n_in);
        if (c->ty == ORC_TY_Q3_K)
            return orc_dot_q3_k_i8(row, c->n_in, c->d + i * nb, c->q + i * c->n_in);
        if (c->ty == ORC_TY_Q2_K)
            return orc_dot_q2_k_i8(row, c->n_in, c->d + i * nb, c->q + i * c->n_in);
        if (c->ty == ORC_TY_Q6_K)
            return orc_dot_q6_k_i8(row, c->n_in, c->d + i * nb, c->q + i * c->n_in);
        if (c->ty == ORC_TY_Q5_K)
            return orc_dot_q5_k_i8(row, c->n_in, c->d + i * nb, c->sum + i * nb, c->q + i * c->n_in);
        return orc_dot_q4_k_i8(row, c->n_in, c->d + i * nb, c->sum + i * nb, c->q + i * c->n_in);
    }
    const float *xi = c->x + i * c->n_in;
    if (c->ty == ORC_TY_Q5_0) return orc_dot_q5_0(row, c->n_in, xi);
    if (c->ty == ORC_TY_Q3_K) return orc_dot_q3_k(row, c->n_in, xi);
    if (c->ty == ORC_TY_Q2_K) return orc_dot_q2_k(row, c->n_in, xi);
    if (c->ty == ORC_TY_Q6_K) return orc_dot_q6_k(row, c->n_in, xi);
    if (c->ty == ORC_TY_Q5_K) return orc_dot_q5_k(row, c->n_in, xi);
    return c->ty == ORC_TY_Q8_0 ? orc_dot_q8_0(row, c->n_in, xi) : orc_dot_q4_k(row, c->n_in, xi);
}

/* chunk over output rows j for every activation row i (matvec mod.rs:253-265;
 * matmul_many's inner loops mod.rs:408-413 visit the same (i,j) pairs) */
static void mm_rows_chunk(void *p, size_t start, size_t end) {
    const mm_ctx *c = (const mm_ctx *)p;
    for (size_t i = 0; i < c->m; i++)
        for (size_t j = start; j < end; j++) c->y[i * c->n_out + j] = row_dot_any(c, i, j);
}

/* chunk over the flat (i,j) space (matmul m>1, m<threads: mod.rs:194-211) */
static void mm_flat_chunk(void *p, size_t start, size_t end) {
    const mm_ctx *c = (const mm_ctx *)p;
    for (size_t flat = start; flat < end; flat++)
        c->y[flat] = row_dot_any(c, flat / c->n_out, flat % c->n_out);
}

int orc_matmul(uint32_t ty, const uint8_t *w, size_t w_bytes, size_t n_out, size_t n_in,
               const float *x, size_t m, int act_mode, float *y, int threads) {
    size_t be, bb;
    /* QuantMat::new (mod.rs:39-65) */
    if (block_geom(ty, &be, &bb) || n_in % be) return -1;
    size_t row_bytes = n_in / be * bb;
    if (row_bytes * n_out != w_bytes) return -1;
    if (n_out == 0 || n_in == 0 || m == 0) return 0;
    if (threads <= 0) threads = orc_cpu_threads();
    if (act_mode == ORC_ACT_AUTO) act_mode = m == 1 ? ORC_ACT_Q8 : ORC_ACT_F32;

    mm_ctx c = {ty, w, n_out, n_in, row_bytes, m, x, NULL, NULL, NULL, y};
    float *d = NULL, *sum = NULL;
    int8_t *q = NULL;
    if (act_mode == ORC_ACT_Q8) {
        /* quantized_acts (mod.rs:271-286): one from_f32 over all m rows */
        size_t nb = m * n_in / 32;
        d = (float *)malloc(nb * sizeof(float));
        sum = (float *)malloc(nb * sizeof(float));
        q = (int8_t *)malloc(m * n_in);
        orc_q8acts_from_f32(x, m * n_in, d, sum, q);
        c.d = d; c.sum = sum; c.q = q;
    }
    const size_t PARALLEL_THRESHOLD_ELEMENTS = (size_t)2 << 20;
    if (m * n_out * n_in < PARALLEL_THRESHOLD_ELEMENTS || threads <= 1) {
        mm_rows_chunk(&c, 0, n_out);
    } else if (act_mode == ORC_ACT_F32 && m > 1 && m < (size_t)threads) {
        par_for_chunks(m * n_out, threads, mm_flat_chunk, &c);
    } else {
        /* results do not depend on how (i,j) pairs are spread over threads */
        par_for_chunks(n_out, threads, mm_rows_chunk, &c);
    }
    free(d); free(sum); free(q);
    return 0;
}

/* ------------------------------------------------------------------ norm */

/* crates/allpaka-backend/src/ops/norm.rs:6-109, AVX2+FMA arm (43-73): two
 * 4-lane f64 accumulators over strides of 8, folded lane-wise then
 * (lo+hi), then the scalar tail.  f32 squares are exact in f64, so the fused
 * multiply-add of the reference equals the separate multiply and add here. */
double orc_sum_sq_f64(const float *x, size_t n) {
    double acc0[4] = {0, 0, 0, 0}, acc1[4] = {0, 0, 0, 0};
    size_t i = 0;
    while (i + 8 <= n) {
        for (int l = 0; l < 4; l++) {
            double a = (double)x[i + l], b = (double)x[i + 4 + l];
            acc0[l] = a * a + acc0[l];
            acc1[l] = b * b + acc1[l];
        }
        i += 8;
    }
    double s[4];
    for (int l = 0; l < 4; l++) s[l] = acc0[l] + acc1[l];
    double p0 = s[0] + s[2], p1 = s[1] + s[3];
    double total = p0 + p1;
    while (i < n) {
        double v = (double)x[i];
        total += v * v;
        i++;
    }
    return total;
}

/* crates/allpaka-backend/src/ops/norm.rs:115-187 */
void orc_rmsnorm(float *x, const float *w, size_t n, float eps) {
    double mean_sq = orc_sum_sq_f64(x, n) / (double)n;
    double scale = 1.0 / sqrt(mean_sq + (double)eps);
    for (size_t i = 0; i < n; i++) x[i] = (float)((double)x[i] * scale) * w[i];
}

/* crates/allpaka-backend/src/ops/norm.rs:193-269 */
void orc_rmsnorm_into(float *dst, const float *src, const float *w, size_t n, float eps) {
    double mean_sq = orc_sum_sq_f64(src, n) / (double)n;
    double scale = 1.0 / sqrt(mean_sq + (double)eps);
    for (size_t i = 0; i < n; i++) dst[i] = (float)((double)src[i] * scale) * w[i];
}

/* ------------------------------------------------------------------ rope */

/* crates/allpaka-backend/src/ops/rope.rs:8-12 */
void orc_rope_inv_freq(size_t head_dim, float base, float *out) {
    for (size_t i = 0; i < head_dim / 2; i++)
        out[i] = powf(base, -2.0f * (float)i / (float)head_dim);
}

/* crates/allpaka-backend/src/ops/rope.rs:18-22; table rows are [sin, cos] */
void orc_rope_sin_cos(uint32_t pos, const float *inv_freq, size_t n, float *table) {
    for (size_t i = 0; i < n; i++) {
        float t = (float)pos * inv_freq[i];
        table[2 * i] = sinf(t);
        table[2 * i + 1] = cosf(t);
    }
}

/* crates/allpaka-backend/src/ops/rope.rs:70-81: `half` table entries rotate
 * (x[i], x[i+half]); channels past 2*half pass through. */
void orc_rope_neox_table(float *x, size_t len, const float *table, size_t half) {
    (void)len;
    for (size_t i = 0; i < half; i++) {
        float sn = table[2 * i], cs = table[2 * i + 1];
        float a = x[i], b = x[i + half];
        x[i] = a * cs - b * sn;
        x[i + half] = a * sn + b * cs;
    }
}

/* crates/allpaka-backend/src/ops/rope.rs:104-117 */
void orc_rope_neox(float *x, size_t d, uint32_t pos, float base) {
    size_t half = d / 2;
    for (size_t i = 0; i < half; i++) {
        float theta = (float)pos * powf(base, -2.0f * (float)i / (float)d);
        float sn = sinf(theta), cs = cosf(theta);
        float a = x[i], b = x[i + half];
        x[i] = a * cs - b * sn;
        x[i + half] = a * sn + b * cs;
    }
}

/* ------------------------------------------------------------ activation */

/* crates/allpaka-backend/src/ops/activation.rs:20-22 */
float orc_silu(float x) { return x / (1.0f + expf(-x)); }

/* crates/allpaka-backend/src/ops/activation.rs:116-119 */
void orc_swiglu(float *gate, const float *up, size_t n) {
    for (size_t i = 0; i < n; i++) gate[i] = orc_silu(gate[i]) * up[i];
}

/* ------------------------------------------------------------- composites */

int orc_attn_in(uint32_t ty, const uint8_t *wq, const uint8_t *wk, const uint8_t *wv,
                size_t hidden, size_t n_q, size_t n_kv, size_t head_dim, const float *x, size_t m,
                const float *gamma, float eps, const float *q_norm, const float *k_norm,
                const float *rope, size_t half, float *q, float *k, float *v, int threads) {
    float *h = (float *)malloc(m * hidden * sizeof(float));
    for (size_t i = 0; i < m; i++) {
        if (gamma) orc_rmsnorm_into(h + i * hidden, x + i * hidden, gamma, hidden, eps);
        else memcpy(h + i * hidden, x + i * hidden, hidden * sizeof(float));
    }
    /* matmul_many: Q8 acts per row at any m (mod.rs:372-388, 408-413) */
    int rc = 0;
    rc |= orc_matmul(ty, wq, orc_expected_bytes(ty, hidden) * n_q, n_q, hidden, h, m, ORC_ACT_Q8, q, threads);
    rc |= orc_matmul(ty, wk, orc_expected_bytes(ty, hidden) * n_kv, n_kv, hidden, h, m, ORC_ACT_Q8, k, threads);
    rc |= orc_matmul(ty, wv, orc_expected_bytes(ty, hidden) * n_kv, n_kv, hidden, h, m, ORC_ACT_Q8, v, threads);
    free(h);
    if (rc) return -1;
    /* model/attention.rs:131-165: per row, per head: optional rmsnorm then rope */
    for (size_t i = 0; i < m; i++) {
        const float *tab = rope + i * half * 2;
        for (size_t hd = 0; hd < n_q / head_dim; hd++) {
            float *head = q + i * n_q + hd * head_dim;
            if (q_norm) orc_rmsnorm(head, q_norm, head_dim, eps);
            orc_rope_neox_table(head, head_dim, tab, half);
        }
        for (size_t hd = 0; hd < n_kv / head_dim; hd++) {
            float *head = k + i * n_kv + hd * head_dim;
            if (k_norm) orc_rmsnorm(head, k_norm, head_dim, eps);
            orc_rope_neox_table(head, head_dim, tab, half);
        }
    }
    return 0;
}

int orc_ffn(uint32_t gate_ty, const uint8_t *gate, uint32_t up_ty, const uint8_t *up,
            uint32_t down_ty, const uint8_t *down, size_t hidden, size_t ffn, const float *x,
            size_t m, float *y, float *act_out, int threads) {
    float *g = (float *)malloc(m * ffn * sizeof(float));
    float *u = (float *)malloc(m * ffn * sizeof(float));
    int rc = 0;
    /* moe.rs:120: matmul_many -> Q8 acts per row */
    rc |= orc_matmul(gate_ty, gate, orc_expected_bytes(gate_ty, hidden) * ffn, ffn, hidden, x, m, ORC_ACT_Q8, g, threads);
    rc |= orc_matmul(up_ty, up, orc_expected_bytes(up_ty, hidden) * ffn, ffn, hidden, x, m, ORC_ACT_Q8, u, threads);
    if (!rc) {
        orc_swiglu(g, u, m * ffn);
        if (act_out) memcpy(act_out, g, m * ffn * sizeof(float));
        /* moe.rs:128: w_down.matmul(&gate, m): Q8 acts at m==1, f32 dots at m>1 */
        rc |= orc_matmul(down_ty, down, orc_expected_bytes(down_ty, ffn) * hidden, hidden, ffn, g, m, ORC_ACT_AUTO, y, threads);
    }
    free(g); free(u);
    return rc ? -1 : 0;
}

int orc_decode_layers(uint32_t ty, const orc_layer *layers, size_t n_layers, size_t hidden,
                      size_t n_q, size_t n_kv, size_t head_dim, size_t ffn, float eps,
                      const float *rope, size_t half, float *x, int threads) {
    float *q = (float *)malloc(n_q * sizeof(float));
    float *k = (float *)malloc(n_kv * sizeof(float));
    float *v = (float *)malloc(n_kv * sizeof(float));
    float *h = (float *)malloc(hidden * sizeof(float));
    float *y = (float *)malloc(hidden * sizeof(float));
    int rc = 0;
    for (size_t l = 0; l < n_layers && !rc; l++) {
        const orc_layer *L = &layers[l];
        rc |= orc_attn_in(ty, L->wq, L->wk, L->wv, hidden, n_q, n_kv, head_dim, x, 1, L->attn_norm,
                          eps, L->q_norm, L->k_norm, rope, half, q, k, v, threads);
        /* identity attention core: attn_out = roped q; wo.matmul(attn_out, 1) */
        rc |= orc_matmul(ty, L->wo, orc_expected_bytes(ty, n_q) * hidden, hidden, n_q, q, 1, ORC_ACT_AUTO, y, threads);
        for (size_t i = 0; i < hidden; i++) x[i] += y[i];
        orc_rmsnorm_into(h, x, L->ffn_norm, hidden, eps);
        rc |= orc_ffn(ty, L->gate, ty, L->up, ty, L->down, hidden, ffn, h, 1, y, NULL, threads);
        for (size_t i = 0; i < hidden; i++) x[i] += y[i];
    }
    free(q); free(k); free(v); free(h); free(y);
    return rc ? -1 : 0;
}

int orc_lm_head(uint32_t ty, const uint8_t *w, size_t vocab, size_t hidden, const float *x,
                const float *output_norm, float eps, float *logits, int threads) {
    float *h = (float *)malloc(hidden * sizeof(float));
    memcpy(h, x, hidden * sizeof(float));
    orc_rmsnorm(h, output_norm, hidden, eps);
    int rc = orc_matmul(ty, w, orc_expected_bytes(ty, hidden) * vocab, vocab, hidden, h, 1, ORC_ACT_AUTO, logits, threads);
    free(h);
    return rc;
}
