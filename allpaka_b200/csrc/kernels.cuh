// Device code of the B200 decode dequant-matvec path.
//
// Data layout in HBM ("tiled stream").  A [n_out, n_in] matrix is cut into
// tiles of 128 output rows; a tile's K extent is cut into K-steps of 256
// elements (Q8_0: 8 blocks; Q6_K: 1 super-block) or 512 elements (Q4_K, Q5_K: 2 super-blocks).  One
// (tile, K-step) "unit" is ONE contiguous span of at most 36 KiB that a single
// bulk async copy (cp.async.bulk + mbarrier complete_tx) brings into shared
// memory.  Inside a unit the bytes sit in the order the tensor-core fragments
// want them, so a warp feeds `mma.sync.m16n8k32.s8` (16 rows x one 32-element
// block x up to 8 activation rows -> int32 block dots) with conflict-free
// 16-byte shared loads and no shuffles.  The repack is a pure permutation of
// the GGUF blocks (zero rows pad the last tile; Q4_K's packed 6-bit scale/min
// fields are split into bytes): quants and f16 scales are untouched.
//
//   Q8_0 unit with kb blocks:  quants [b][row group 0..3][16-row half][lane][16 B], i.e. the
//                              A fragments of mma.m16n8k32 (lane = 4*g + t holds rows g, g+8
//                              and k bytes 4t.., 16+4t..), kb*4096 B; then the f16 scales
//                              [b][row group][g][rows g, g+8, g+16, g+24], kb*256 B
//   Q4_K unit with ns super-blocks: per super-block and row group, the nibble bytes in the
//        same fragment order (one 16-byte chunk per pair, 16-row half and lane: masking
//        gives the low-nibble sub-block, shifting the high one), 4096 B, then the header
//        with the 6-bit scales and mins already split out into bytes: {d, dmin} f16 pairs
//        [g][4 rows], scales [g][half of the sub-blocks][4 rows][4], mins likewise, 640 B
//   Q5_K: as Q4_K, with the qh bytes (one high bit per element: sub-block j reads bit j) in the
//        same fragment order between the nibbles and the header, 1024 B per row group
//   Q6_K unit (one super-block): per row group, the ql bytes as nibble fragments like Q4_K's
//        (chunk (half, byte group c): low nibbles = quarter c, high = quarter c + 2 of that half),
//        4096 B; the qh bytes of each half in the same fragment order (quarter qi takes bits
//        2qi, 2qi+1 of every byte), 2048 B; the sixteen int8 sub-block scales [g][4 rows][16],
//        512 B; the f16 d [g][4 rows], 64 B.  6720 B = 32 rows x 210 B: nothing is widened.
//
// Work split ("stream-K"): the flat unit sequence of the whole matrix is cut
// into equal contiguous ranges, one per CTA (one CTA per SM), so every SM
// streams the same number of bytes regardless of n_out.  A tile whose units
// straddle CTAs is finished by the CTA that holds its last units: the others
// publish their partial sums as tagged 64-bit words, it adds them in CTA order
// (deterministic; no float atomics; its only wait, on CTAs of lower index of
// the same grid, is bounded).
// (The kernels that are not templates are `static`: this header is compiled into several
// translation units, one per weight format for the matvec kernel, which are built side by side.)
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace apk {

constexpr int TILE_ROWS = 128;
constexpr int Q8_KT = 8;             // Q8_0 blocks per K-step (256 elements)
constexpr int Q8_BLOCK_UNIT = 4352;  // 128 rows * 34 B
constexpr int Q4_SB_RG = 4736;       // one row group of a super-block: 4096 B nibbles + 640 B header
constexpr int Q4_SB_UNIT = 4 * Q4_SB_RG;  // 128 rows: 18944 B (18432 B of GGUF blocks + split scale bytes)
constexpr int Q4_KT_SB = 2;          // Q4_K super-blocks per K-step (512 elements)
constexpr int Q5_SB_RG = 5760;       // Q5_K: 4096 B nibbles + 1024 B high bits + 640 B header
constexpr int Q5_SB_UNIT = 4 * Q5_SB_RG;  // 128 rows: 23040 B (22528 B of GGUF blocks + split scale bytes)
constexpr int Q6_SB_RG = 6720;       // one row group of a Q6_K super-block: 4096 B ql + 2048 B qh + 512 B scales + 64 B d
constexpr int Q6_SB_UNIT = 4 * Q6_SB_RG;  // 128 rows: 26880 B = 128 * 210 B
// Q2_K rides on the Q6_K stream (code q + 32, the 4-bit sub-block scales as int8) with its second half appended to
// each row group: the 4-bit sub-block mins, laid out like the scales, and the f16 dmin, laid out like d.
constexpr int Q2_SB_RG = Q6_SB_RG + 512 + 64;   // 7296
constexpr int Q2_SB_UNIT = 4 * Q2_SB_RG;        // 29184
__host__ __device__ constexpr bool ty_k6(int ty) { return ty == 14 || ty == 10; }
__host__ __device__ constexpr int k6_sb_rg(int ty) { return ty == 10 ? Q2_SB_RG : Q6_SB_RG; }
constexpr int Q50_BLOCK_UNIT = 2816; // Q5_0, 128 rows * 22 B: 2048 B nibbles + 512 B of the K-step's fifth-bit plane + 256 B scales
__host__ __device__ constexpr int stage_w_bytes(int ty) {  // one full K-step of weights
    return ty == 8 ? 8 * 4352 : (ty == 6 ? 8 * 2816 : (ty == 14 ? 26880 : (ty == 10 ? 29184 : (ty == 13 ? 2 * 23040 : 2 * 18944))));
}
// Q8_0 and Q5_0: 32-element blocks with one f16 scale, eight blocks per K-step.  A K-step of kb
// blocks holds kb fragment arrays (4096 B of int8 for Q8_0, 2048 B of nibbles for Q5_0), for Q5_0
// then ONE 4096-byte plane of fifth bits (bit j of a byte = block j of the K-step, bytes in
// fragment order), then kb arrays of 128 scales.
__host__ __device__ constexpr bool ty_b32(int ty) { return ty == 8 || ty == 6; }
__host__ __device__ constexpr int b32_step_bytes(int ty, int kb) { return ty == 6 ? kb * 2304 + 4096 : kb * 4352; }
__host__ __device__ constexpr int b32_scale_off(int ty, int kb) { return ty == 6 ? kb * 2048 + 4096 : kb * 4096; }
// Q4_K and Q5_K share everything but the fifth bit: row-group size and header offset of a super-block
__host__ __device__ constexpr bool ty_k45(int ty) { return ty == 12 || ty == 13; }
__host__ __device__ constexpr int k45_sb_rg(int ty) { return ty == 13 ? Q5_SB_RG : Q4_SB_RG; }
__host__ __device__ constexpr int k45_hdr(int ty) { return ty == 13 ? 5120 : 4096; }
constexpr int N_CONSUMER_WARPS = 16; // 4 row groups x 4 quarters of a K-step
constexpr int K_SPLIT = 4;
constexpr int N_CONSUMERS = N_CONSUMER_WARPS * 32;
constexpr int N_FINISH_WARPS = 3;     // close tiles (cross-CTA hand-off, epilogue) while the consumers stream on
constexpr int N_FINISHERS = N_FINISH_WARPS * 32;
constexpr int MV_THREADS = N_CONSUMERS + 32 + N_FINISHERS;  // consumers | producer warp | finisher warps
constexpr int MAX_M_EFF = 16;
constexpr int MAX_STAGES = 8;
constexpr int TY_Q5_0 = 6;
constexpr int TY_Q8_0 = 8;
constexpr int TY_Q2_K = 10;  // the Q6_K stream plus sub-block mins and dmin (see repack_q6_k_kernel<2>)
constexpr int TY_Q3_K = 11;  // carried in the Q6_K stream (see repack_q6_k_kernel<true>)
constexpr int TY_Q4_K = 12;
constexpr int TY_Q5_K = 13;
constexpr int TY_Q6_K = 14;

// Error words written by kernels (never a trap): which bounded wait gave up.  The matvec kernel
// records kind | site << 4 | launch number << 8 (the first one to give up wins): sites 1-3 the
// copy producer (a landed stage, the prologue scratch, an empty stage), 5 another CTA's tile
// piece, 6 the finishers waiting for a hand-off, 8-10 the consumers (activation records, a full
// stage, the hand-off buffer).
constexpr int ERRW_PRODUCER_TIMEOUT = 1;
constexpr int ERRW_CONSUMER_TIMEOUT = 2;
constexpr int ERRW_PEER_TIMEOUT = 3;
constexpr int ERRW_FINISHER_TIMEOUT = 4;

// Default spin budget of one bounded wait, in SM clock cycles (~2 s).  Kernels take the
// budget as a parameter so that a test can make a wait run out in a millisecond.
constexpr long long WAIT_LIMIT_DEFAULT = 4000000000LL;

enum Epilogue : int {
    EPI_STORE = 0,   // y[m][row] = v
    EPI_ADD = 1,     // y[m][row] = resid[m][row] + v   (residual stream update)
    EPI_QKV_ROPE = 2,// tile = one head: optional per-head RMSNorm, NeoX RoPE on Q and K heads
    EPI_SWIGLU = 3,  // tile = 64 gate rows + 64 up rows: act = silu(g)*u, optionally packed for `down`
    EPI_PEERS = 4,   // tensor parallel: this rank's partial sums stored straight into every rank's exchange buffer
};

// One-shot exchange of row-parallel partial sums between the ranks of a
// tensor-parallel group over peer-mapped memory (plain stores across NVLink, one
// per peer).  Every rank owns one buffer, laid out
//   slots [2 parity][XCH_MAX_RANKS][XCH_ROW_FLOATS] 64-bit words | tok u32
// Exchanges are numbered e = 1, 2, ... for the life of the group (every rank runs the
// same sequence).  The CTA of rank s that closes a 128-row tile of the row-parallel matvec
// stores the tile's partial sums into slot (e & 1, s) of EVERY rank's buffer, each value as
// one 64-bit word {e, f32}: a naturally aligned 64-bit access is single-copy atomic, so a
// reader that sees tag e has the value -- no fence, no flag, no second round trip, and the
// storing CTA leaves at once.  The kernel that consumes the sum polls the words of its own
// buffer (bounded) until all world slots carry tag e and adds them in rank order 0..world-1:
// deterministic, one NVLink hop, no extra launch.  Old words carry older tags, so nothing is
// ever cleared.  Two parities suffice: a rank can run at most one exchange ahead of the
// slowest one, because passing exchange e + 1 needs every rank's words for e + 1.
// `tok` counts decoded tokens; e = (tok - 1) * exchanges per token + index in the token + 1.
constexpr int XCH_MAX_RANKS = 8;
constexpr int XCH_ROW_FLOATS = 8 * 16384;  // m * hidden values per slot
constexpr size_t XCH_SLOTS_BYTES = (size_t)2 * XCH_MAX_RANKS * XCH_ROW_FLOATS * sizeof(unsigned long long);
constexpr size_t XCH_BYTES = XCH_SLOTS_BYTES + 256;

struct XchPeers {
    float *slots[XCH_MAX_RANKS];  // peer-mapped base of each rank's buffer (own included)
    int rank, world;
};
__host__ __device__ inline unsigned long long *xch_words(float *base) { return reinterpret_cast<unsigned long long *>(base); }
__host__ __device__ inline uint32_t *xch_tok(float *base) { return reinterpret_cast<uint32_t *>(reinterpret_cast<uint8_t *>(base) + XCH_SLOTS_BYTES); }
// Where a kernel stands in the exchange sequence of its token.
struct XchSeq {
    int index = -1;     // exchange index within the token (0-based); -1 = this launch takes no part
    int per_token = 0;  // exchanges per token
};

// Prepared activations as the matvec kernel consumes them: per K-step of `ke`
// elements (kt = ke/32 blocks) one record
//   q   [block][16-element half][row 0..m_eff-1][16 B]   int8, the B fragments of the mma
//   d   [block][mp] f32      (mp = m_eff rounded up to even)
//   sum [block][mp] f32
struct ActLayout {
    uint8_t *base;
    int ke;        // elements per K-step: 256 (Q8_0 or Q6_K consumer) or 512 (Q4_K consumer)
    int m_eff;     // rows in the record (2 per token in two-level mode)
    __host__ __device__ int kt() const { return ke >> 5; }
    __host__ __device__ int mp() const { return (m_eff + 1) & ~1; }
    __host__ __device__ int q_bytes() const { return ke * m_eff; }
    __host__ __device__ int rec_bytes() const { return ke * m_eff + kt() * mp() * 8; }
    __host__ __device__ size_t total_bytes(int n_in) const {
        return (size_t)((n_in + ke - 1) / ke) * rec_bytes();
    }
};

struct MvParams;
__device__ __forceinline__ void note_timeout(const MvParams &p, int kind, int site);

struct PrepParams {
    const float *x; int ldx;                 // [m][n] activations
    const float *add; int ldadd;             // optional addend (residual / combined partial sums)
    float *xout; int ldxout;                 // optional: store x + add
    const float *gamma; float eps;           // optional RMSNorm weight
    float *hout; int ldh;                    // optional: store the normed f32 row
    int n, m;
    ActLayout out;
    int two_level, need_sum;
    // optional: f64 sums of squares of the 32-element blocks of x, [m][n / 32], left by the
    // kernel that produced x; the RMSNorm then adds those instead of re-reading the row
    const double *sumsq;
};

// How the kernel gets its activations.
enum Prologue : int {
    PRO_STREAM = 0,  // prepared records streamed with every unit (any m, any K)
    PRO_LOAD = 1,    // the whole prepared buffer bulk-loaded once into shared memory
    PRO_QUANT = 2,   // x (f32) [+ addend] -> optional RMSNorm -> Q8 blocks, computed in the CTA
};

struct MvParams {
    const uint8_t *W;   // tiled stream
    ActLayout act;      // prepared activations (m_eff rows)
    int ty;
    int n_out, nb;      // real rows; 32-element blocks per row
    int n_tiles, KS;    // tiles; K-steps per tile
    uint32_t tile_bytes;
    int n_stages;
    int m_out;          // tokens written by the epilogue (m_eff, or m_eff/2 in two-level mode)
    int two_level;
    int pro;            // Prologue
    PrepParams prep;    // PRO_QUANT inputs (prep.out is ignored: blocks go to shared memory)
    int pdl;            // launched with a programmatic dependency on the previous kernel
    unsigned long long *partials;  // [gridDim.x][2][MAX_M_EFF][128] tagged partial sums (see part_store)
    int *err;           // error word
    int launch_id;
    int tl_alt;     // timeline: stamp the closing of the last tile (1: handed over, 4: crew complete, 7: pieces added) instead of 1 and 4      // number of this launch within its submission (goes into the error word)
    long long wait_limit;  // cycle budget of every bounded wait in this launch
    int32_t *dump;      // optional [m_eff][n_out][nb] int32 block dots
    uint8_t *act_dump;  // optional: CTA 0 copies its resident activation records here (parity instrumentation)
    int inflight;       // K-steps of weights one CTA keeps in flight at a time (>= 1)
    int inflight_pre;   // the same while the previous kernel has not finished yet (>= 1)
    unsigned long long *timeline;  // optional [gridDim.x][8] globaltimer stamps (trace)
    // epilogue
    int epi;
    float *y; int ldy;
    const float *resid; int ldr;
    // EPI_QKV_ROPE
    int n_q_tiles, n_k_tiles;          // tiles (heads) that are Q, then K; the rest are V
    const float *q_norm, *k_norm;      // optional [128]
    float eps;
    const float *rope; int half;       // [m][half][2] (sin, cos)
    ActLayout q_next;                  // optional: roped Q heads packed as the next matvec's activations
    int q_next_two_level, q_next_need_sum;
    int qkv_tile_base;  // EPI_QKV_ROPE: stack index of this matrix's first head (n_q_tiles + n_k_tiles for a V matrix of its own)
    __half *kv_k, *kv_v;               // optional: this layer's f16 cache slabs [capacity][kv_dim]; K and V rows go there too
    int kv_dim;                        // (this rank's) kv heads * 128
    const uint32_t *pos_dev; uint32_t pos;  // cache position of row 0: on the device (greedy chain) or with the launch
    // Tensor-parallel exchange (see XchPeers).  xout: EPI_PEERS, this launch feeds exchange
    // xout.index.  xin: PRO_QUANT, the input row is prep.x + the rank-ordered sum of exchange
    // xin.index (CTA 0 stores it to prep.xout).  tok_inc: CTA 0 advances the token counter
    // (set on the first launch of a token, which takes part in no exchange).
    XchPeers xch; int xch_row;         // floats per token row in a slot (= hidden)
    XchSeq xin, xout;
    int xin_late;   // xin: start on the tagged words alone, make up for the dependency wait at the end (token order only:
                    // the launch in front must be a row-parallel matvec that did wait for its own predecessor)
    int tok_inc;
    // EPI_SWIGLU
    float *act_f32; int ld_act;        // optional f32 swiglu rows [m][ffn]
    ActLayout act_next;                // optional packed activations for the down projection
    int next_two_level, next_need_sum;
    int ffn;                           // real ffn rows (gate rows)
    // EPI_ADD, optional: the updated residual rows feed an RMSNorm and a matvec next.
    //  nq_sumsq: each tile leaves the f64 sums of squares of its four blocks, [m_out][n_out / 32];
    //    the next kernel adds them up instead of reducing the row again (exact: the quantisation
    //    itself happens there, on f32(f64(x) * scale) * gamma as ops::rmsnorm_into orders it).
    //  nq_gamma (with nq_sumsq): the tile also quantises its 128 elements times the norm weight
    //    right away, before the row-wide scale exists, and the next kernel multiplies the block
    //    scales by 1/sqrt(mean + eps) (norm_sumsq).  Cheaper, but codes can differ from the exact
    //    order by one where v/d lands on a .5 boundary: an opt-in approximation.
    const float *nq_gamma;             // [n_out] weight of the next norm; null = off
    ActLayout nq_act;                  // the next matvec's activation records
    int nq_two_level, nq_need_sum;
    double *nq_sumsq;                  // [m_out][n_out / 32]
    // PRO_LOAD, optional: records prepared that way by the previous kernel
    const double *norm_sumsq;          // [m_out][norm_blocks]; null = records are final
    int norm_blocks;                   // 32-element blocks per row
    float norm_eps;
};

__device__ __forceinline__ void note_timeout(const MvParams &p, int kind, int site) {
    atomicCAS(p.err, 0, kind | (site << 4) | (p.launch_id << 8));
}

// ------------------------------------------------------------------ PTX glue

__device__ __forceinline__ uint32_t smem_u32(const void *p) {
    return (uint32_t)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ void mbar_init(uint64_t *bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void fence_mbar_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t *bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t *bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t *bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
// Wait for a phase with a cycle budget.  false = gave up (caller records it).
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t *bar, uint32_t parity, long long limit) {
    if (mbar_try_wait(bar, parity)) return true;
    const long long t0 = clock64();
    for (;;) {
#pragma unroll 1
        for (int i = 0; i < 256; ++i)
            if (mbar_try_wait(bar, parity)) return true;
        if (clock64() - t0 > limit) return false;
    }
}
// Same, for the producer lane: it has nothing else to do, so it backs off between
// polls instead of competing with the consumer warps for issue slots.
__device__ __forceinline__ bool mbar_wait_bounded_relaxed(uint64_t *bar, uint32_t parity, long long limit) {
    if (mbar_try_wait(bar, parity)) return true;
    const long long t0 = clock64();
    for (;;) {
#pragma unroll 1
        for (int i = 0; i < 64; ++i) {
            if (mbar_try_wait(bar, parity)) return true;
            __nanosleep(40);
        }
        if (clock64() - t0 > limit) return false;
    }
}
// Partial sums of a tile shared by several CTAs travel as one 64-bit word per
// element: the f32 value below a "valid" tag.  A naturally aligned 64-bit scalar
// access is single-copy atomic, so a reader that sees the tag has the value: no
// fence, no counter, no second round trip.  The reader clears what it has read,
// so every word is back to zero when the kernel ends.
constexpr unsigned long long PART_VALID = 1ull << 32;
__device__ __forceinline__ void part_store(unsigned long long *p, float v) {
    const unsigned long long w = PART_VALID | (unsigned long long)__float_as_uint(v);
    asm volatile("st.relaxed.gpu.global.b64 [%0], %1;" ::"l"(p), "l"(w) : "memory");
}
__device__ __forceinline__ void part_clear(unsigned long long *p) {
    asm volatile("st.relaxed.gpu.global.b64 [%0], %1;" ::"l"(p), "l"(0ull) : "memory");
}
__device__ __forceinline__ unsigned long long part_load(const unsigned long long *p) {
    unsigned long long w;
    asm volatile("ld.relaxed.gpu.global.b64 %0, [%1];" : "=l"(w) : "l"(p) : "memory");
    return w;
}
__device__ __forceinline__ uint64_t l2_policy_evict_first() {
    uint64_t p;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(p));
    return p;
}
__device__ __forceinline__ uint64_t l2_policy_evict_last() {
    uint64_t p;
    asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(p));
    return p;
}
// 1-D bulk async copy global -> shared, completion counted on an mbarrier.
// dst, src 16-byte aligned; bytes a multiple of 16.
__device__ __forceinline__ void bulk_g2s(void *dst, const void *src, uint32_t bytes, uint64_t *bar,
                                         uint64_t policy) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint "
        "[%0], [%1], %2, [%3], %4;" ::"r"(smem_u32(dst)),
        "l"(src), "r"(bytes), "r"(smem_u32(bar)), "l"(policy)
        : "memory");
}
// Programmatic dependent launch: let the next kernel in the stream start its
// independent work (weight prefetch) early / wait for the previous kernel's results.
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ unsigned long long globaltimer_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
__device__ __forceinline__ void consumer_bar() { asm volatile("bar.sync 1, %0;" ::"n"(N_CONSUMERS) : "memory"); }
__device__ __forceinline__ void finisher_bar() { asm volatile("bar.sync 2, %0;" ::"n"(N_FINISHERS) : "memory"); }
// The threads that close a tile together: the finisher warps (barrier 2), joined for a CTA's
// last tile by the consumer warps, which have nothing left to do by then (barrier 3).
struct Crew {
    int t, n, bar;  // this thread's index in the crew, crew size, named barrier
    __device__ __forceinline__ void sync() const { asm volatile("bar.sync %0, %1;" ::"r"(bar), "r"(n) : "memory"); }
};
constexpr int N_CREW_ALL = N_FINISHERS + N_CONSUMERS;

// D[16 rows x 8 cols] = A[16 x 32] . B[32 x 8], int8 operands, int32 result: one
// 32-element quantisation block of 16 weight rows against up to 8 activation rows.
__device__ __forceinline__ void mma_block_s8(int (&d)[4], const uint4 &a, uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
        : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
        : "r"(a.x), "r"(a.y), "r"(a.z), "r"(a.w), "r"(b0), "r"(b1), "r"(0));
}

// The same, accumulating onto d.
__device__ __forceinline__ void mma_block_s8_acc(int (&d)[4], const uint4 &a, uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
        : "r"(a.x), "r"(a.y), "r"(a.z), "r"(a.w), "r"(b0), "r"(b1));
}

// Half of that: 16 rows x 16 k-values x 8 columns, accumulating.  a0/a1 are registers 0, 1
// (or 2, 3) of the k32 A fragment, b the matching B register.
// the same with unsigned A bytes (weights as 0..255) and signed B bytes
__device__ __forceinline__ void mma_block_u8s8_acc(int (&d)[4], const uint4 &a, uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
        : "r"(a.x), "r"(a.y), "r"(a.z), "r"(a.w), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void mma_half_s8_acc(int (&d)[4], uint32_t a0, uint32_t a1, uint32_t b) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5}, {%6}, {%0,%1,%2,%3};"
        : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
        : "r"(a0), "r"(a1), "r"(b));
}

// Q6_K: the 6-bit values of quarter qi (0..3) of one half as int8 fragment words, (ql nibble | two
// qh bits << 4) per byte, WITHOUT the -32 of crates/allpaka-backend/src/quantmat/q8_acts.rs:329-333:
// dot(q - 32, x) = dot(q, x) - 32 * sum(x), and the sums of the activation codes come out of one
// extra mma against an all-ones fragment (see the consumers), which is cheaper than a byte-wise
// subtraction per register.  ql: the chunk of byte group qi & 1; qh: the half's chunk.
__device__ __forceinline__ uint4 q6_k_unpack(const uint4 &ql, const uint4 &qh, int qi) {
    const int sh = 2 * qi;
    uint4 v;
    if (qi & 2) {
        v.x = (ql.x >> 4) & 0x0f0f0f0fu; v.y = (ql.y >> 4) & 0x0f0f0f0fu;
        v.z = (ql.z >> 4) & 0x0f0f0f0fu; v.w = (ql.w >> 4) & 0x0f0f0f0fu;
    } else {
        v.x = ql.x & 0x0f0f0f0fu; v.y = ql.y & 0x0f0f0f0fu; v.z = ql.z & 0x0f0f0f0fu; v.w = ql.w & 0x0f0f0f0fu;
    }
    v.x |= ((qh.x >> sh) & 0x03030303u) << 4;
    v.y |= ((qh.y >> sh) & 0x03030303u) << 4;
    v.z |= ((qh.z >> sh) & 0x03030303u) << 4;
    v.w |= ((qh.w >> sh) & 0x03030303u) << 4;
    return v;
}
// Q5_K: the fifth bit of the two sub-blocks of pair pr (low nibbles: bit 2*pr of each qh byte, high
// nibbles: bit 2*pr + 1) onto the nibble fragments (crates/allpaka-backend/src/quantmat/q8_acts.rs:247-252)
__device__ __forceinline__ void q5_k_high(uint4 &lo, uint4 &hi, const uint4 &qh, int pr) {
    const int s = 2 * pr;
    lo.x |= ((qh.x >> s) & 0x01010101u) << 4; lo.y |= ((qh.y >> s) & 0x01010101u) << 4;
    lo.z |= ((qh.z >> s) & 0x01010101u) << 4; lo.w |= ((qh.w >> s) & 0x01010101u) << 4;
    hi.x |= ((qh.x >> (s + 1)) & 0x01010101u) << 4; hi.y |= ((qh.y >> (s + 1)) & 0x01010101u) << 4;
    hi.z |= ((qh.z >> (s + 1)) & 0x01010101u) << 4; hi.w |= ((qh.w >> (s + 1)) & 0x01010101u) << 4;
}

// Q5_0: the codes q = nibble | fifth bit << 4 (0..31) of block b as an A fragment, WITHOUT the - 16 of
// crates/allpaka-backend/src/quantmat/q8_acts.rs:115-120: dot(q - 16, x) = dot(q, x) - 16 * sum(x), and the
// sums of the activation codes come out of one mma against an all-0x10 fragment (see the consumers).
// nib: the row pair's nibble words (low nibbles = elements 0..15, the first k-half); qh: this lane's
// bytes of the K-step's fifth-bit plane, bit b of each byte belonging to block b.
__device__ __forceinline__ uint4 q5_0_unpack(const uint2 nib, const uint4 &qh, int b) {
    uint4 a;
    a.x = (nib.x & 0x0f0f0f0fu) | (((qh.x >> b) & 0x01010101u) << 4);
    a.y = (nib.y & 0x0f0f0f0fu) | (((qh.y >> b) & 0x01010101u) << 4);
    a.z = ((nib.x >> 4) & 0x0f0f0f0fu) | (((qh.z >> b) & 0x01010101u) << 4);
    a.w = ((nib.y >> 4) & 0x0f0f0f0fu) | (((qh.w >> b) & 0x01010101u) << 4);
    return a;
}
// the A fragment of 16 rows (row group rg, half h16) of block b in a staged K-step of kb blocks
// (Q5_0: codes 0..31, see q5_0_unpack)
template <int TY>
__device__ __forceinline__ uint4 b32_frag(const uint8_t *sw, int kb, int b, int rg, int h16, int lane) {
    if constexpr (TY == TY_Q5_0) {
        const uint2 nib = *reinterpret_cast<const uint2 *>(sw + b * 2048 + rg * 512 + h16 * 256 + lane * 8);
        const uint4 qh = *reinterpret_cast<const uint4 *>(sw + kb * 2048 + ((rg * 2 + h16) * 32 + lane) * 16);
        return q5_0_unpack(nib, qh, b);
    } else {
        return *reinterpret_cast<const uint4 *>(sw + b * 4096 + rg * 1024 + h16 * 512 + lane * 16);
    }
}

// ----------------------------------------------------- activation quantiser
//
// One warp quantises one 32-element block; lane = element.  Arithmetic of
// Q8Acts::from_f32 (crates/allpaka-backend/src/quantmat/q8_acts.rs:26-63):
// d = amax/127 (0 when amax is not finite), id = 1/d (IEEE division),
// q = round-half-away(v*id) saturated to i8, sum = sequential f32 sum.
// q = round-half-away-from-zero(x * id) saturated to i8, i.e. `(x * id).round() as i8`
// (quantmat/q8_acts.rs:57).  For |r| <= 129 (always: |x * id| <= 127 up to rounding),
// trunc(r + copysign(0.5, r)) with |r| < 0.5 -> 0 equals roundf(r) for every f32
// (checked exhaustively); NaN converts to 0 like the Rust cast.
__device__ __forceinline__ int q8_round(float x, float id) {
    const float r = __fmul_rn(x, id);
    const int q = __float2int_rz(__fadd_rn(r, copysignf(0.5f, r)));
    return fabsf(r) < 0.5f ? 0 : max(-128, min(127, q));
}

struct QBlock { float d; float sum; int q; };

__device__ __forceinline__ QBlock quantize_block(float v, bool need_sum) {
    float amax = fabsf(v);
    if (amax != amax) amax = 0.0f;  // f32::max drops a NaN operand
    // non-negative floats order like their bit patterns: one warp-wide integer max
    amax = __uint_as_float(__reduce_max_sync(0xffffffffu, __float_as_uint(amax)));
    const bool fin = amax <= 3.402823466e+38f;
    const float db = fin ? __fdiv_rn(amax, 127.0f) : 0.0f;
    const float id = (db > 0.0f) ? __frcp_rn(db) : 0.0f;  // IEEE 1.0/db
    const int q = q8_round(v, id);
    float s = 0.0f;
    if (need_sum) {
        // xs.iter().sum::<f32>(): strictly left to right
#pragma unroll
        for (int i = 0; i < 32; ++i) s = __fadd_rn(s, __shfl_sync(0xffffffffu, v, i));
    }
    QBlock o;
    o.d = db; o.sum = s; o.q = q;
    return o;
}

// Store one quantised block (lane = element) into a prepared-activation buffer.
__device__ __forceinline__ void store_act_block(const ActLayout &L, int row, int k_block, int lane,
                                                const QBlock &qb) {
    const int kt = L.kt();
    const int ks = k_block / kt, bl = k_block - ks * kt;
    uint8_t *rec = L.base + (size_t)ks * L.rec_bytes();
    rec[((bl * 2 + (lane >> 4)) * L.m_eff + row) * 16 + (lane & 15)] = (uint8_t)(int8_t)qb.q;
    if (lane == 0) {
        float *d = reinterpret_cast<float *>(rec + L.q_bytes());
        d[bl * L.mp() + row] = qb.d;
        d[kt * L.mp() + bl * L.mp() + row] = qb.sum;
    }
}

// Quantise value v (lane = element) of token m, block k_block, in Q8 mode
// (one row per token) or two-level mode (rows 2m = value, 2m+1 = residual:
// x = d1*q1 + d2*q2, d2 = d1/256, to ~2^-16 of the block maximum, which is how the f32
// activation call sites of the reference are served by the integer kernels).
__device__ __forceinline__ void quantize_store(const ActLayout &L, int two_level, int need_sum, int m,
                                               int k_block, int lane, float v) {
    QBlock q1 = quantize_block(v, need_sum && !two_level);
    if (!two_level) {
        store_act_block(L, m, k_block, lane, q1);
        return;
    }
    // residual is exact in one fused operation; its scale is d1 / 256 exactly, so that the
    // consumer can merge the two digits as integers: d1*dot1 + d2*dot2 = d2 * (256*dot1 + dot2)
    const float r = __fmaf_rn(-q1.d, (float)q1.q, v);
    QBlock q2;
    q2.d = q1.d * 0.00390625f;
    q2.sum = 0.0f;
    q2.q = max(-127, min(127, q8_round(r, q2.d > 0.0f ? __frcp_rn(q2.d) : 0.0f)));
    if (need_sum) {
        // the min term needs sum(x) once: carry the exact block sum on the first row
        float s = 0.0f;
#pragma unroll
        for (int i = 0; i < 32; ++i) s = __fadd_rn(s, __shfl_sync(0xffffffffu, v, i));
        q1.sum = s;
        q2.sum = 0.0f;
    }
    store_act_block(L, 2 * m, k_block, lane, q1);
    store_act_block(L, 2 * m + 1, k_block, lane, q2);
}

__device__ __forceinline__ float load_x(const PrepParams &p, int m, int i) {
    float v = p.x[(size_t)m * p.ldx + i];
    if (p.add) v = __fadd_rn(v, p.add[(size_t)m * p.ldadd + i]);
    return v;
}

// The sum of squares of a row from the per-block f64 sums its producer left: lane-strided
// partial sums, then a butterfly.  One fixed order, used by every kernel that takes the
// hand-off, so they all get the same scale.
__device__ __forceinline__ double sumsq_total(const double *sq, int nblk, int lane) {
    double ss = 0.0;
    for (int i = lane; i < nblk; i += 32) ss += sq[i];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    return ss;
}

// RMSNorm scale exactly as ops::rmsnorm_into does it (crates/allpaka-backend/
// src/ops/norm.rs:193-198): f64 sum of squares, f64 1/sqrt(mean + eps).  The
// f64 sum order differs from the reference's 8-lane walk; the difference is
// confined to the last bits of an f64 that is then rounded to f32.
__device__ __forceinline__ double block_rms_scale(const PrepParams &p, int m, double *red) {
    if (p.sumsq) {
        const double tot = sumsq_total(p.sumsq + (size_t)m * (p.n >> 5), p.n >> 5, threadIdx.x & 31);
        return 1.0 / sqrt(tot / (double)p.n + (double)p.eps);
    }
    double ss = 0.0;
    for (int i = threadIdx.x; i < p.n; i += blockDim.x) {
        const double v = (double)load_x(p, m, i);
        ss = fma(v, v, ss);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    const int w = threadIdx.x >> 5, nw = blockDim.x >> 5;
    if ((threadIdx.x & 31) == 0) red[w] = ss;
    __syncthreads();
    double tot = 0.0;
    for (int i = 0; i < nw; ++i) tot += red[i];
    return 1.0 / sqrt(tot / (double)p.n + (double)p.eps);
}

// grid = (ceil(blocks / 8), m), 256 threads: each warp quantises one block.
static __global__ void __launch_bounds__(256) prep_acts_kernel(PrepParams p, int pdl) {
    __shared__ double red[8];
    if (pdl) {
        pdl_launch_dependents();
        pdl_wait();
    }
    const int m = blockIdx.y;
    double scale = 1.0;
    if (p.gamma) scale = block_rms_scale(p, m, red);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int blk = blockIdx.x * 8 + warp;
    if (blk * 32 >= p.n) return;
    const int i = blk * 32 + lane;
    float v = load_x(p, m, i);
    if (p.xout) p.xout[(size_t)m * p.ldxout + i] = v;
    if (p.gamma) v = __fmul_rn((float)((double)v * scale), p.gamma[i]);
    if (p.hout) p.hout[(size_t)m * p.ldh + i] = v;
    quantize_store(p.out, p.two_level, p.need_sum, m, blk, lane, v);
}

// ------------------------------------------------- tensor-parallel exchange

// Number of the exchange a launch takes part in (see XchPeers).
__device__ __forceinline__ uint32_t xch_number(float *mine, const XchSeq &s) {
    return (__ldcg(xch_tok(mine)) - 1u) * (uint32_t)s.per_token + (uint32_t)s.index + 1u;
}
__device__ __forceinline__ void st_relaxed_sys_b64(unsigned long long *p, unsigned long long v) {
    asm volatile("st.relaxed.sys.global.b64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ void ld_relaxed_sys_v2b64(const unsigned long long *p, unsigned long long &a, unsigned long long &b) {
    asm volatile("ld.relaxed.sys.global.v2.b64 {%0, %1}, [%2];" : "=l"(a), "=l"(b) : "l"(p) : "memory");
}
// (slot 0 + slot 1 + ...)[i..i+3] in rank order: the one summation order of an exchange (rank 0's
// slot already holds the residual row plus its partial sums, see EPI_PEERS), for NJ groups of
// four consecutive values per thread (group j at word offset off[j]; live[j] = false: skipped).
// Polls (bounded) until the words carry tag e; *ok = false when the budget ran out (the sums then
// hold whatever was there).  Nothing but tagged words is read, so a caller needs no other
// ordering with the kernels that produced them.
// The loads of XCH_RB ranks and all NJ groups are in flight together: once the words are there,
// the gather costs world / XCH_RB round trips to L2, not world * NJ.
constexpr int XCH_RB = 2;
template <int NJ>
__device__ __forceinline__ void xch_gather(float *mine, uint32_t e, int world, const size_t (&off)[NJ], const bool (&live)[NJ],
                                           long long limit, bool *ok, float4 (&sum)[NJ]) {
    const unsigned long long *s0 = xch_words(mine) + (size_t)(e & 1u) * XCH_MAX_RANKS * XCH_ROW_FLOATS;
    const long long t0 = clock64();
#pragma unroll
    for (int j = 0; j < NJ; ++j) sum[j] = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int r0 = 0; r0 < world; r0 += XCH_RB) {
        unsigned long long w[XCH_RB][NJ][4];
        for (;;) {
            bool all = true;
#pragma unroll
            for (int rr = 0; rr < XCH_RB; ++rr)
#pragma unroll
                for (int j = 0; j < NJ; ++j)
                    if (r0 + rr < world && live[j]) {
                        const unsigned long long *src = s0 + (size_t)(r0 + rr) * XCH_ROW_FLOATS + off[j];
                        ld_relaxed_sys_v2b64(src, w[rr][j][0], w[rr][j][1]);
                        ld_relaxed_sys_v2b64(src + 2, w[rr][j][2], w[rr][j][3]);
                    }
#pragma unroll
            for (int rr = 0; rr < XCH_RB; ++rr)
#pragma unroll
                for (int j = 0; j < NJ; ++j)
                    if (r0 + rr < world && live[j])
                        all = all && (uint32_t)(w[rr][j][0] >> 32) == e && (uint32_t)(w[rr][j][1] >> 32) == e &&
                              (uint32_t)(w[rr][j][2] >> 32) == e && (uint32_t)(w[rr][j][3] >> 32) == e;
            if (all) break;
            if (clock64() - t0 > limit) {
                *ok = false;
                break;
            }
        }
#pragma unroll
        for (int rr = 0; rr < XCH_RB; ++rr)
#pragma unroll
            for (int j = 0; j < NJ; ++j)
                if (r0 + rr < world && live[j]) {
                    const float4 v = make_float4(__uint_as_float((uint32_t)w[rr][j][0]), __uint_as_float((uint32_t)w[rr][j][1]),
                                                 __uint_as_float((uint32_t)w[rr][j][2]), __uint_as_float((uint32_t)w[rr][j][3]));
                    if (r0 + rr == 0) sum[j] = v;
                    else {
                        sum[j].x = __fadd_rn(sum[j].x, v.x); sum[j].y = __fadd_rn(sum[j].y, v.y);
                        sum[j].z = __fadd_rn(sum[j].z, v.z); sum[j].w = __fadd_rn(sum[j].w, v.w);
                    }
                }
    }
}

struct XchReduceParams {
    XchPeers xch;
    XchSeq seq;                // which exchange to collect
    float *xout; int ldxout;   // residual stream out [m][n] = sum over ranks of the slots (rank 0's holds the old rows too)
    int n, m;
    int *err;
    int pdl;
    long long wait_limit;
};

// Stand-alone form of the collecting side (batches of m > 1 rows, whose activations are
// quantised by a separate pass): grid = ceil(m*n / 1024), 256 threads, four floats per
// thread.  Waits (bounded) for every rank's tagged words of the exchange and adds them in
// rank order into the new residual rows.
static __global__ void __launch_bounds__(256) xch_reduce_kernel(XchReduceParams p) {
    if (p.pdl) {
        pdl_launch_dependents();
        pdl_wait();  // this rank's matvec (and its peer stores) is complete
    }
    float *mine = p.xch.slots[p.xch.rank];
    const uint32_t e = xch_number(mine, p.seq);
    const size_t total = (size_t)p.m * p.n;
    const size_t i = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) * 4;
    if (i < total) {
        const int m = (int)(i / p.n), col = (int)(i % p.n);
        bool ok = true;
        const size_t off[1] = {(size_t)m * p.n + col};
        const bool live[1] = {true};
        float4 accs[1];
        xch_gather<1>(mine, e, p.xch.world, off, live, p.wait_limit, &ok, accs);
        const float4 acc = accs[0];
        if (!ok) atomicCAS(p.err, 0, ERRW_PEER_TIMEOUT);  // a peer never delivered: record it and finish normally
        *reinterpret_cast<float4 *>(p.xout + (size_t)m * p.ldxout + col) = acc;
    }
}

// ------------------------------------------------------------------ repack

struct RepackParams {
    const uint8_t *src;      // raw GGUF rows (device staging copy)
    size_t src_row_bytes;    // bytes from one staged row to the next
    int src_rows;            // rows in the staging copy
    int row_base;            // segment-relative index of the staging copy's first row
    int nb;                  // 32-element blocks per (sharded) row
    uint8_t *dst;            // tiled stream of the destination matrix
    uint32_t dst_tile_bytes;
    // destination row of source row r: (r / group) * stride + offset + r % group
    int group, stride, offset;
};

__device__ __forceinline__ int map_row(const RepackParams &p, int r) {
    r += p.row_base;
    return (r / p.group) * p.stride + p.offset + (r % p.group);
}

// Where the fragment order puts things.  A tile row r (0..127) is row group
// rg = r/32, 16-row half h16 = (r%32)/16, fragment row g = r%8, upper = (r%16)/8
// (rows g and g+8 of a 16-row mma tile share a lane).  Within a 32-byte block,
// k-word w (bytes 4w..4w+3) belongs to lane column t = w%4 and k-half w/4; the
// A-fragment register index is 2*(w/4) + upper.
__device__ __forceinline__ void frag_pos(int r, int &rg, int &h16, int &g, int &upper) {
    rg = r >> 5;
    h16 = (r >> 4) & 1;
    g = r & 7;
    upper = (r >> 3) & 1;
}

// One thread per (row, block): 34 unaligned source bytes -> eight fragment words + scale.
static __global__ void repack_q8_0_kernel(RepackParams p) {
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const size_t total = (size_t)p.src_rows * p.nb;
    if (idx >= total) return;
    const int r = (int)(idx / p.nb), b = (int)(idx % p.nb);
    const uint8_t *s = p.src + (size_t)r * p.src_row_bytes + (size_t)b * 34;
    const int dr = map_row(p, r);
    const int tile = dr / TILE_ROWS, rt = dr % TILE_ROWS;
    int rg, h16, g, upper;
    frag_pos(rt, rg, h16, g, upper);
    const int ks = b / Q8_KT, bl = b % Q8_KT;
    const int kb = min(Q8_KT, p.nb - ks * Q8_KT);
    uint8_t *unit = p.dst + (size_t)tile * p.dst_tile_bytes + (size_t)ks * Q8_KT * Q8_BLOCK_UNIT;
    uint8_t *frag = unit + (size_t)(((bl * 4 + rg) * 2 + h16) * 32) * 16;
#pragma unroll
    for (int w = 0; w < 8; ++w) {
        const uint32_t v = (uint32_t)s[2 + 4 * w] | ((uint32_t)s[3 + 4 * w] << 8) | ((uint32_t)s[4 + 4 * w] << 16) |
                           ((uint32_t)s[5 + 4 * w] << 24);
        const int lane = g * 4 + (w & 3), reg = 2 * (w >> 2) + upper;
        *reinterpret_cast<uint32_t *>(frag + lane * 16 + reg * 4) = v;
    }
    uint16_t *sc = reinterpret_cast<uint16_t *>(unit + kb * 4096 + ((bl * 4 + rg) * 8 + g) * 8 + (h16 * 2 + upper) * 2);
    *sc = (uint16_t)(s[0] | (s[1] << 8));
}

// Q5_0, one thread per (row, block): 22 source bytes {f16 d, u32 qh, 16 B nibbles} -> four nibble words
// (byte j = elements j and j + 16, as in the file), this block's bit in the K-step's fifth-bit plane
// (eight blocks share each byte, hence the atomic OR into the zero-filled destination), scale.
static __global__ void repack_q5_0_kernel(RepackParams p) {
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const size_t total = (size_t)p.src_rows * p.nb;
    if (idx >= total) return;
    const int r = (int)(idx / p.nb), b = (int)(idx % p.nb);
    const uint8_t *s = p.src + (size_t)r * p.src_row_bytes + (size_t)b * 22;
    const int dr = map_row(p, r);
    const int tile = dr / TILE_ROWS, rt = dr % TILE_ROWS;
    int rg, h16, g, upper;
    frag_pos(rt, rg, h16, g, upper);
    const int ks = b / Q8_KT, bl = b % Q8_KT;
    const int kb = min(Q8_KT, p.nb - ks * Q8_KT);
    uint8_t *unit = p.dst + (size_t)tile * p.dst_tile_bytes + (size_t)ks * b32_step_bytes(TY_Q5_0, Q8_KT);
    const uint32_t qh = (uint32_t)s[2] | ((uint32_t)s[3] << 8) | ((uint32_t)s[4] << 16) | ((uint32_t)s[5] << 24);
#pragma unroll
    for (int w = 0; w < 4; ++w) {
        const uint32_t v = (uint32_t)s[6 + 4 * w] | ((uint32_t)s[7 + 4 * w] << 8) | ((uint32_t)s[8 + 4 * w] << 16) |
                           ((uint32_t)s[9 + 4 * w] << 24);
        *reinterpret_cast<uint32_t *>(unit + bl * 2048 + rg * 512 + h16 * 256 + (g * 4 + w) * 8 + upper * 4) = v;
    }
#pragma unroll
    for (int w = 0; w < 8; ++w) {  // k-word w: elements 4w..4w+3, lane column w % 4, fragment register 2 * (w / 4) + upper
        uint32_t bits = 0;
#pragma unroll
        for (int k = 0; k < 4; ++k) bits |= ((qh >> (4 * w + k)) & 1u) << (8 * k + bl);
        if (bits)
            atomicOr(reinterpret_cast<unsigned int *>(unit + kb * 2048 + ((rg * 2 + h16) * 32 + g * 4 + (w & 3)) * 16 +
                                                      (2 * (w >> 2) + upper) * 4),
                     bits);
    }
    uint16_t *sc = reinterpret_cast<uint16_t *>(unit + b32_scale_off(TY_Q5_0, kb) + ((bl * 4 + rg) * 8 + g) * 8 + (h16 * 2 + upper) * 2);
    *sc = (uint16_t)(s[0] | (s[1] << 8));
}

// One thread per (row, super-block): 144 (Q4_K) or 176 (Q5_K) source bytes -> nibble fragments
// [+ high-bit fragments] + split header.
template <bool K5>
__global__ void repack_q45_k_kernel(RepackParams p) {
    constexpr int TY = K5 ? TY_Q5_K : TY_Q4_K;
    constexpr int SB_RG = k45_sb_rg(TY), SB_UNIT = 4 * SB_RG;
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const int nsb = p.nb / 8;
    const size_t total = (size_t)p.src_rows * nsb;
    if (idx >= total) return;
    const int sb = (int)(idx % nsb), r = (int)(idx / nsb);
    const uint8_t *s = p.src + (size_t)r * p.src_row_bytes + (size_t)sb * (K5 ? 176 : 144);
    const int dr = map_row(p, r);
    const int tile = dr / TILE_ROWS, rt = dr % TILE_ROWS;
    int rg, h16, g, upper;
    frag_pos(rt, rg, h16, g, upper);
    const int ks = sb / Q4_KT_SB, sl = sb % Q4_KT_SB;
    uint8_t *base = p.dst + (size_t)tile * p.dst_tile_bytes + (size_t)ks * Q4_KT_SB * SB_UNIT +
                    (size_t)sl * SB_UNIT + (size_t)rg * SB_RG;
    // nibble bytes: pair pr holds qs[32*pr .. 32*pr+31]; word w of the pair -> lane column w%4, k-half w/4
    const uint8_t *qs = s + (K5 ? 48 : 16);
    if (K5) {
        // high bits: qh[0..31] in the same order (element l of sub-block j reads bit j of qh[l])
        uint8_t *frag = base + 4096 + (size_t)(h16 * 32) * 16;
        for (int w = 0; w < 8; ++w) {
            const uint8_t *q = s + 16 + 4 * w;
            const uint32_t v = (uint32_t)q[0] | ((uint32_t)q[1] << 8) | ((uint32_t)q[2] << 16) | ((uint32_t)q[3] << 24);
            const int lane = g * 4 + (w & 3), reg = 2 * (w >> 2) + upper;
            *reinterpret_cast<uint32_t *>(frag + lane * 16 + reg * 4) = v;
        }
    }
#pragma unroll 4
    for (int pr = 0; pr < 4; ++pr) {
        uint8_t *frag = base + (size_t)((pr * 2 + h16) * 32) * 16;
        for (int w = 0; w < 8; ++w) {
            const uint8_t *q = qs + pr * 32 + 4 * w;
            const uint32_t v = (uint32_t)q[0] | ((uint32_t)q[1] << 8) | ((uint32_t)q[2] << 16) | ((uint32_t)q[3] << 24);
            const int lane = g * 4 + (w & 3), reg = 2 * (w >> 2) + upper;
            *reinterpret_cast<uint32_t *>(frag + lane * 16 + reg * 4) = v;
        }
    }
    // header: {d, dmin} [g][4 rows] | scales [g][j half][4 rows][4] | mins likewise
    uint8_t *hdr = base + k45_hdr(TY);
    const int row4 = h16 * 2 + upper;  // which of rows g, g+8, g+16, g+24
    *reinterpret_cast<uint32_t *>(hdr + (g * 4 + row4) * 4) =
        (uint32_t)s[0] | ((uint32_t)s[1] << 8) | ((uint32_t)s[2] << 16) | ((uint32_t)s[3] << 24);
    const uint8_t *pk = s + 4;
    for (int j = 0; j < 8; ++j) {
        // scale_min_k4 (crates/allpaka-dtype/src/lib.rs:382-390), kept as integers
        uint8_t sc, mn;
        if (j < 4) {
            sc = pk[j] & 63;
            mn = pk[j + 4] & 63;
        } else {
            sc = (uint8_t)((pk[j + 4] & 0xf) | ((pk[j - 4] >> 6) << 4));
            mn = (uint8_t)((pk[j + 4] >> 4) | ((pk[j] >> 6) << 4));
        }
        hdr[128 + ((g * 2 + (j >> 2)) * 4 + row4) * 4 + (j & 3)] = sc;
        hdr[384 + ((g * 2 + (j >> 2)) * 4 + row4) * 4 + (j & 3)] = mn;
    }
}

// A Q3_K super-block {u8 hmask[32]; u8 qs[64]; u8 scales[12]; f16 d} rewritten as the Q6_K
// super-block with the same values.  Both are 16 sub-blocks of 16 elements in natural order with an
// integer scale each and one f16 d, x = d * sc * q (crates/allpaka-gguf/src/dequant.rs:176-204 and
// 265-296), and both dots are d * dx * (sc0 * dot0 + sc1 * dot1) per 32-element block
// (crates/allpaka-backend/src/quantmat/q8_acts.rs:206-210 and 338-342): the signed 3-bit value q
// becomes the 6-bit code q + 32, the 6-bit scale minus 32 the int8 scale.
__device__ inline void q3_k_as_q6_k(const uint8_t *s, uint8_t (&o)[210]) {
    for (int i = 0; i < 192; ++i) o[i] = 0;
    for (int e = 0; e < 256; ++e) {
        const int blk = e >> 5, l = e & 31, half = e >> 7, quarter = blk & 3;
        const int q = ((s[32 + half * 32 + l] >> (2 * quarter)) & 3) - ((s[l] >> blk) & 1 ? 0 : 4);
        const int code = q + 32;  // 28..35
        // Q6_K: quarter qr of a half takes the low (qr < 2) or high nibbles of ql[64*half + 32*(qr&1) + l]
        // and bits 2qr, 2qr+1 of qh[32*half + l]
        o[half * 64 + (quarter & 1) * 32 + l] |= (uint8_t)((code & 15) << (quarter < 2 ? 0 : 4));
        o[128 + half * 32 + l] |= (uint8_t)((code >> 4) << (2 * quarter));
    }
    const uint8_t *pk = s + 96;
    for (int i = 0; i < 4; ++i) {  // crates/allpaka-dtype/src/lib.rs:395-404
        o[192 + i] = (uint8_t)(int8_t)(((pk[i] & 0x0f) | ((pk[8 + i] & 3) << 4)) - 32);
        o[196 + i] = (uint8_t)(int8_t)(((pk[4 + i] & 0x0f) | (((pk[8 + i] >> 2) & 3) << 4)) - 32);
        o[200 + i] = (uint8_t)(int8_t)(((pk[i] >> 4) | (((pk[8 + i] >> 4) & 3) << 4)) - 32);
        o[204 + i] = (uint8_t)(int8_t)(((pk[4 + i] >> 4) | (((pk[8 + i] >> 6) & 3) << 4)) - 32);
    }
    o[208] = s[108];
    o[209] = s[109];
}

// A Q2_K super-block {u8 scales[16]; u8 qs[64]; f16 d; f16 dmin}, x = d * (sc & 15) * q - dmin * (sc >> 4)
// (crates/allpaka-gguf/src/dequant.rs:150-174): its first term as a Q6_K super-block (code q + 32, scale sc & 15),
// the 16 mins sc >> 4 and dmin on the side.
__device__ inline void q2_k_as_q6_k(const uint8_t *s, uint8_t (&o)[210], uint8_t (&mins)[16], uint16_t *dmin) {
    for (int i = 0; i < 192; ++i) o[i] = 0;
    for (int e = 0; e < 256; ++e) {
        const int l = e & 31, half = e >> 7, quarter = (e >> 5) & 3;
        const int code = ((s[16 + half * 32 + l] >> (2 * quarter)) & 3) + 32;
        o[half * 64 + (quarter & 1) * 32 + l] |= (uint8_t)((code & 15) << (quarter < 2 ? 0 : 4));
        o[128 + half * 32 + l] |= (uint8_t)((code >> 4) << (2 * quarter));
    }
    for (int i = 0; i < 16; ++i) {
        o[192 + i] = (uint8_t)(s[i] & 15);
        mins[i] = (uint8_t)(s[i] >> 4);
    }
    o[208] = s[80];
    o[209] = s[81];
    *dmin = (uint16_t)(s[82] | (s[83] << 8));
}

// One thread per (row, super-block): 210 source bytes -> nibble and high-bit fragments, scales, d.
// FROM = 3: the source is Q3_K (110 bytes per super-block), FROM = 2: Q2_K (84 bytes), rewritten on the fly.
template <int FROM>
__global__ void repack_q6_k_kernel(RepackParams p) {
    constexpr bool FROM_Q3 = FROM == 3, FROM_Q2 = FROM == 2;
    constexpr int RG = FROM_Q2 ? Q2_SB_RG : Q6_SB_RG;
    const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const int nsb = p.nb / 8;
    const size_t total = (size_t)p.src_rows * nsb;
    if (idx >= total) return;
    const int sb = (int)(idx % nsb), r = (int)(idx / nsb);
    const uint8_t *s = p.src + (size_t)r * p.src_row_bytes + (size_t)sb * (FROM_Q3 ? 110 : (FROM_Q2 ? 84 : 210));
    uint8_t tmp[210], mins[16];
    uint16_t dmin = 0;
    if (FROM_Q3) {
        q3_k_as_q6_k(s, tmp);
        s = tmp;
    }
    if (FROM_Q2) {
        q2_k_as_q6_k(s, tmp, mins, &dmin);
        s = tmp;
    }
    const int dr = map_row(p, r);
    const int tile = dr / TILE_ROWS, rt = dr % TILE_ROWS;
    int rg, h16, g, upper;
    frag_pos(rt, rg, h16, g, upper);
    uint8_t *base = p.dst + (size_t)tile * p.dst_tile_bytes + (size_t)sb * (4 * RG) + (size_t)rg * RG;
    auto word = [](const uint8_t *q) {
        return (uint32_t)q[0] | ((uint32_t)q[1] << 8) | ((uint32_t)q[2] << 16) | ((uint32_t)q[3] << 24);
    };
    // ql: chunk (half, c) holds ql[64*half + 32*c .. +31]; word w -> lane column w%4, k-half w/4
    for (int pr = 0; pr < 4; ++pr) {
        uint8_t *frag = base + (size_t)((pr * 2 + h16) * 32) * 16;
        for (int w = 0; w < 8; ++w) {
            const int lane = g * 4 + (w & 3), reg = 2 * (w >> 2) + upper;
            *reinterpret_cast<uint32_t *>(frag + lane * 16 + reg * 4) = word(s + pr * 32 + 4 * w);
        }
    }
    // qh: chunk `half` holds qh[32*half .. +31] in the same order
    for (int half = 0; half < 2; ++half) {
        uint8_t *frag = base + 4096 + (size_t)((half * 2 + h16) * 32) * 16;
        for (int w = 0; w < 8; ++w) {
            const int lane = g * 4 + (w & 3), reg = 2 * (w >> 2) + upper;
            *reinterpret_cast<uint32_t *>(frag + lane * 16 + reg * 4) = word(s + 128 + half * 32 + 4 * w);
        }
    }
    const int row4 = h16 * 2 + upper;  // which of rows g, g+8, g+16, g+24
    uint8_t *sc = base + 6144 + (g * 4 + row4) * 16;
    for (int j = 0; j < 16; ++j) sc[j] = s[192 + j];
    *reinterpret_cast<uint16_t *>(base + 6656 + (g * 4 + row4) * 2) = (uint16_t)(s[208] | (s[209] << 8));
    if (FROM_Q2) {
        uint8_t *mn = base + Q6_SB_RG + (g * 4 + row4) * 16;
        for (int j = 0; j < 16; ++j) mn[j] = mins[j];
        *reinterpret_cast<uint16_t *>(base + Q6_SB_RG + 512 + (g * 4 + row4) * 2) = dmin;
    }
}

// ------------------------------------------------------ decode attention over the f16 KV cache
//
// What sits between the Q|K|V matvec and the output projection of a decoder layer
// (crates/allpaka-model/src/model/attention.rs:337-399): per kv head, its GQA group of q heads
// attends over cache positions 0..=pos with an online softmax; K and V live in the cache as f16
// (model/kv.rs), scores and sums are f32.  HBM-bound on the cache bytes and far smaller than the
// weight stream next to it at short contexts (2 * positions * kv_dim * 2 B per layer; as large as a
// layer's Q|K|V weights from ~13k positions on), plain SIMT in f32 like the reference: the positions
// are split over CTAs, a warp walks its share four positions at a time, the splits are merged by a
// second small kernel that also packs the result as the Q8 (or two-level) blocks the output
// projection consumes.
constexpr int ATT_WARPS = 8;
constexpr int ATT_MAX_GROUP = 8;       // q heads per kv head handled by one CTA pass
constexpr int ATT_PART = TILE_ROWS + 4;  // floats per partial: acc[128], running max, denominator, pad (16-byte rows)
static_assert(ATT_PART % 4 == 0, "partials are moved as float4");

struct AttnParams {
    const float *q; int ldq;           // [m][ldq] roped q heads (head h at column h * 128)
    const __half *kc, *vc;             // this layer's cache slabs, [capacity][kv_dim]
    int kv_dim, n_kv_heads, group;     // local (per rank) kv heads, q heads per kv head
    const uint32_t *pos_dev; uint32_t pos;  // position of row 0: on the device (greedy chain) or with the launch
    int m, n_splits;
    float scale;
    float *part;                       // [m][q heads][n_splits][ATT_PART]
    // second kernel
    float *out; int ldo;               // optional f32 rows [m][q heads * 128]
    ActLayout next;                    // the output projection's activation records
    int next_two_level, next_need_sum;
};

// grid (kv heads, splits, m), ATT_WARPS warps.  head_dim is 128.
// A warp serves ATT_HPW q heads of the kv head's group and takes four positions per step: eight
// lanes per position, 16 head dimensions (two 16-byte loads of K, two of V) per lane, so a score
// needs three shuffle rounds, the loads of the next step are in flight while this one is reduced,
// and the running state (max, denominator, 16 x ATT_HPW accumulators) stays in registers.  The
// warps of a CTA are (pair of heads) x (position slot); the K and V rows a CTA touches are read
// by its head-pair warps out of L1 after the first.
constexpr int ATT_HPW = 2;
static __global__ void __launch_bounds__(ATT_WARPS * 32) attn_split_kernel(AttnParams p, int pdl) {
    if (pdl) {
        pdl_launch_dependents();
        pdl_wait();
    }
    // one state per (warp, position subgroup, head of the warp)
    __shared__ float sm[ATT_WARPS * 4 * ATT_HPW][ATT_PART];
    const int kvh = blockIdx.x, split = blockIdx.y, row = blockIdx.z;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int sg = lane >> 3, c = lane & 7;  // position within the step, 16-dimension chunk
    const uint32_t pos = (p.pos_dev ? *p.pos_dev : p.pos) + (uint32_t)row;  // this row sees positions 0..=pos
    const uint32_t n_pos = pos + 1u;
    const uint32_t per = (n_pos + (uint32_t)p.n_splits - 1u) / (uint32_t)p.n_splits;
    const uint32_t t0 = (uint32_t)split * per, t1 = min(n_pos, t0 + per);
    for (int g0 = 0; g0 < p.group; g0 += ATT_MAX_GROUP) {
        const int G = min(ATT_MAX_GROUP, p.group - g0);
        const int n_hp = (G + ATT_HPW - 1) / ATT_HPW, n_pp = ATT_WARPS / n_hp;  // head pairs, position slots
        const int hp = warp % n_hp, pp = warp / n_hp;
        const bool busy = pp < n_pp;
        float q[ATT_HPW][16], acc[ATT_HPW][16], mx[ATT_HPW], dn[ATT_HPW];
#pragma unroll
        for (int hh = 0; hh < ATT_HPW; ++hh) {
            const int h = ATT_HPW * hp + hh;
            const bool on = busy && h < G;
            const float *qp = p.q + (size_t)row * p.ldq + (size_t)(kvh * p.group + g0 + (on ? h : 0)) * TILE_ROWS + 16 * c;
#pragma unroll
            for (int i = 0; i < 16; i += 4) {
                const float4 v = on ? *reinterpret_cast<const float4 *>(qp + i) : make_float4(0.f, 0.f, 0.f, 0.f);
                q[hh][i] = v.x; q[hh][i + 1] = v.y; q[hh][i + 2] = v.z; q[hh][i + 3] = v.w;
            }
#pragma unroll
            for (int i = 0; i < 16; ++i) acc[hh][i] = 0.0f;
            mx[hh] = -INFINITY;
            dn[hh] = 0.0f;
        }
        if (busy) {
            const size_t col = (size_t)kvh * TILE_ROWS + 16 * c;
            const uint32_t stride = (uint32_t)n_pp * 4u;
            // the rows of the next step are requested before this step's are used
            uint4 kn0, kn1, vn0, vn1;
            auto fetch = [&](uint32_t tb) {
                const uint32_t t = tb + (uint32_t)sg;
                const size_t off = (size_t)(t < t1 ? t : t0) * p.kv_dim + col;
                kn0 = __ldg(reinterpret_cast<const uint4 *>(p.kc + off));
                kn1 = __ldg(reinterpret_cast<const uint4 *>(p.kc + off + 8));
                vn0 = __ldg(reinterpret_cast<const uint4 *>(p.vc + off));
                vn1 = __ldg(reinterpret_cast<const uint4 *>(p.vc + off + 8));
            };
            const uint32_t tb0 = t0 + (uint32_t)pp * 4u;
            if (tb0 < t1) fetch(tb0);
            for (uint32_t tb = tb0; tb < t1; tb += stride) {
                const bool valid = tb + (uint32_t)sg < t1;
                const uint32_t kw[8] = {kn0.x, kn0.y, kn0.z, kn0.w, kn1.x, kn1.y, kn1.z, kn1.w};
                const uint32_t vw[8] = {vn0.x, vn0.y, vn0.z, vn0.w, vn1.x, vn1.y, vn1.z, vn1.w};
                if (tb + stride < t1) fetch(tb + stride);
                float k[16], v[16];
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    const float2 kf = __half22float2(*reinterpret_cast<const __half2 *>(&kw[i]));
                    const float2 vf = __half22float2(*reinterpret_cast<const __half2 *>(&vw[i]));
                    k[2 * i] = kf.x; k[2 * i + 1] = kf.y;
                    v[2 * i] = vf.x; v[2 * i + 1] = vf.y;
                }
#pragma unroll
                for (int hh = 0; hh < ATT_HPW; ++hh) {
                    float s = 0.0f;
#pragma unroll
                    for (int i = 0; i < 16; ++i) s = fmaf(q[hh][i], k[i], s);
                    s += __shfl_xor_sync(0xffffffffu, s, 1);
                    s += __shfl_xor_sync(0xffffffffu, s, 2);
                    s += __shfl_xor_sync(0xffffffffu, s, 4);
                    s *= p.scale;
                    // online softmax without a branch: a maximum that stays gives r = exp(0) = 1 exactly,
                    // so this is attend_group's update (model/attention.rs:366-388) value for value
                    const float m_new = valid ? fmaxf(mx[hh], s) : mx[hh];
                    const float r = mx[hh] == -INFINITY ? 0.0f : expf(mx[hh] - m_new);
                    const float pr = valid ? expf(s - m_new) : 0.0f;
                    dn[hh] = fmaf(dn[hh], r, pr);
#pragma unroll
                    for (int i = 0; i < 16; ++i) acc[hh][i] = fmaf(pr, v[i], acc[hh][i] * r);
                    mx[hh] = m_new;
                }
            }
        }
        // every (warp, subgroup, head) state into shared memory, then one warp per head merges them
        __syncthreads();
#pragma unroll
        for (int hh = 0; hh < ATT_HPW; ++hh) {
            float *st = sm[(warp * 4 + sg) * ATT_HPW + hh];
#pragma unroll
            for (int i = 0; i < 16; i += 4)
                *reinterpret_cast<float4 *>(st + 16 * c + i) = make_float4(acc[hh][i], acc[hh][i + 1], acc[hh][i + 2], acc[hh][i + 3]);
            if (c == 0) {
                st[TILE_ROWS] = busy ? mx[hh] : -INFINITY;
                st[TILE_ROWS + 1] = busy ? dn[hh] : 0.0f;
            }
        }
        __syncthreads();
        for (int h = warp; h < G; h += ATT_WARPS) {
            const int hp_h = h / ATT_HPW, hh = h % ATT_HPW;
            float M = -INFINITY;
            for (int w = hp_h; w < n_hp * n_pp; w += n_hp)
#pragma unroll
                for (int s4 = 0; s4 < 4; ++s4) M = fmaxf(M, sm[(w * 4 + s4) * ATT_HPW + hh][TILE_ROWS]);
            float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
            float d = 0.0f;
            for (int w = hp_h; w < n_hp * n_pp; w += n_hp)
#pragma unroll
                for (int s4 = 0; s4 < 4; ++s4) {
                    const float *st = sm[(w * 4 + s4) * ATT_HPW + hh];
                    const float mw = st[TILE_ROWS];
                    const float r = mw == -INFINITY ? 0.0f : expf(mw - M);
                    const float4 aw = *reinterpret_cast<const float4 *>(st + 4 * lane);
                    a.x += r * aw.x; a.y += r * aw.y; a.z += r * aw.z; a.w += r * aw.w;
                    d += r * st[TILE_ROWS + 1];
                }
            float *dst = p.part + (((size_t)row * (p.n_kv_heads * p.group) + (size_t)(kvh * p.group + g0 + h)) * p.n_splits + split) * ATT_PART;
            *reinterpret_cast<float4 *>(dst + 4 * lane) = a;
            if (lane == 0) {
                dst[TILE_ROWS] = M;
                dst[TILE_ROWS + 1] = d;
            }
        }
        __syncthreads();  // the states are rewritten by the next group of heads
    }
}

// The same on tensor cores, for the long contexts where the cache is the larger stream.  K and V
// are f16 in the cache already; q and the softmax weights are f32, so each is fed as two f16
// fragments (value = hi + lo, lo = f16(value - hi)): the products are exact in the f32
// accumulator and the split costs one more mma, which keeps the result at f32 rounding level
// (the reference computes f32 x f16 in f32).  grid (kv heads, splits, m), ATC_WARPS warps; a warp
// takes 16 positions per step: cp.async brings their K and V rows (2 x 4 KB) into its own
// double-buffered stage, ldmatrix (transposed for V) forms the B fragments, S = Q K^T is 8 k-steps
// x 2 position tiles x {hi, lo}, the online softmax runs on the accumulator fragments (rows =
// the group's heads, four lanes per row), O += P V is 16 dimension tiles x {hi, lo}.  Rows 8..15 of
// the 16-row mma stay zero (a GQA group has at most 8 heads per pass).
constexpr int ATC_WARPS = 4;
constexpr int ATC_ROW = TILE_ROWS + 8;   // halves per staged row: 272 B, so the eight rows of an ldmatrix hit distinct banks
constexpr int ATC_STAGE = 2 * 16 * ATC_ROW;  // halves per stage: K tile, then V tile
constexpr int ATC_STAGES = 2;            // per warp: one step of K and V rows in flight while it works on the other (a third stage measured slower: 33.4 against 31.5 us at 32768 positions)
constexpr int ATC_SMEM = ATC_WARPS * ATC_STAGES * ATC_STAGE * 2;  // 68 KB (the merge buffer reuses the stages); two CTAs per SM by registers
static_assert(ATC_WARPS * 16 * ATT_PART * 4 <= ATC_SMEM, "the merge buffer lives in the stage memory");

__device__ __forceinline__ void mma_f16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void split_f16x2(float x, float y, uint32_t &hi, uint32_t &lo) {
    const __half2 h = __floats2half2_rn(x, y);
    const float2 hf = __half22float2(h);
    const __half2 l = __floats2half2_rn(x - hf.x, y - hf.y);
    hi = *reinterpret_cast<const uint32_t *>(&h);
    lo = *reinterpret_cast<const uint32_t *>(&l);
}

// PAIR = false: one query row per CTA, rows 8..15 of the mma stay zero (decode).  PAIR = true (verify
// batches): consecutive query rows share the K and V stream.  Each half of the 16 fragment rows holds
// 8 / Gp query rows of Gp heads (Gp = the group size rounded up to a power of two, at most 8), each
// row with its own causal limit and softmax state; grid.x = ceil(m / atc_rows(group)).
// the group size (at most 8 heads per pass) rounded up to a power of two, and the query rows one CTA of
// the PAIR kernel takes
__host__ __device__ inline int atc_group_pow2(int group) { return group <= 1 ? 1 : group <= 2 ? 2 : group <= 4 ? 4 : 8; }
__host__ __device__ inline int atc_rows(int group) { return 16 / atc_group_pow2(group); }

template <bool PAIR>
static __global__ void __launch_bounds__(ATC_WARPS * 32) attn_split_tc_kernel(AttnParams p, int pdl) {
    if (pdl) {
        pdl_launch_dependents();
        pdl_wait();
    }
    constexpr int NR = PAIR ? 2 : 1;
    extern __shared__ __align__(16) uint8_t att_smem[];
    __half *stages = reinterpret_cast<__half *>(att_smem);
    float *merge = reinterpret_cast<float *>(att_smem);  // [warp][row of the pair][head][ATT_PART], over the stages once every warp is through with them
    const int Gp = PAIR ? atc_group_pow2(p.group) : 8, RH = 8 / Gp, NRC = NR * RH;  // rows per half, rows per CTA
    // grid (kv heads, splits, 1), or for PAIR (row groups, kv heads, splits): the CTAs that walk the same K and V rows are neighbours
    const int kvh = PAIR ? blockIdx.y : blockIdx.x, split = PAIR ? blockIdx.z : blockIdx.y, row0 = PAIR ? NRC * blockIdx.x : 0;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    const int hh = g % Gp, sr = g / Gp;                    // this lane's head of the group and row of the half
    const uint32_t base = p.pos_dev ? *p.pos_dev : p.pos;  // query row r sees positions 0..=base + r
    const uint32_t n_pos = base + (uint32_t)min(row0 + NRC, p.m);  // what the last row of this CTA sees
    // positions per split: whole steps of the CTA (16 positions per warp), so that no warp idles through a ragged
    // last step; the splits this leaves empty publish an empty partial
    constexpr uint32_t STEP = 16u * ATC_WARPS;
    const uint32_t per = ((n_pos + (uint32_t)p.n_splits - 1u) / (uint32_t)p.n_splits + STEP - 1u) / STEP * STEP;
    const uint32_t t0 = (uint32_t)split * per, t1 = min(n_pos, t0 + per);
    __half *my = stages + (size_t)warp * ATC_STAGES * ATC_STAGE;
    const uint32_t my_s = (uint32_t)__cvta_generic_to_shared(my);
    // this warp's 16 positions of step i: t0 + 16 * (warp + ATC_WARPS * i)
    auto stage_load = [&](uint32_t p0, int st) {
        // 16 rows x 256 B of K and of V: 512 16-byte chunks, 16 per lane
#pragma unroll
        for (int j = 0; j < 16; ++j) {
            const int ch = j * 32 + lane, kvsel = ch >> 8, r = (ch >> 4) & 15, cc = ch & 15;
            const uint32_t tr = min(p0 + (uint32_t)r, t1 - 1u);  // rows past the end repeat the last one; their scores are masked
            const __half *src = (kvsel ? p.vc : p.kc) + (size_t)tr * p.kv_dim + (size_t)kvh * TILE_ROWS + 8 * cc;
            const uint32_t dst = my_s + (uint32_t)((st * ATC_STAGE + kvsel * 16 * ATC_ROW + r * ATC_ROW + 8 * cc) * 2);
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    const uint32_t first = t0 + 16u * (uint32_t)warp, stride = 16u * ATC_WARPS;
    for (int g0 = 0; g0 < p.group; g0 += ATT_MAX_GROUP) {
        const int G = min(ATT_MAX_GROUP, p.group - g0);
        // the K and V rows of the first two steps are on their way while q is fetched and split
        if (first < t1) stage_load(first, 0);
        if (ATC_STAGES > 2 && first + stride < t1) stage_load(first + stride, 1);
        // q of this lane's (row, head) in each half as A fragments, hi and lo, eight k-steps of 16 dimensions
        uint32_t qh[8][2 * NR], ql[8][2 * NR];
        uint32_t lim[NR];
#pragma unroll
        for (int rr = 0; rr < NR; ++rr) {
            const int qrow = row0 + rr * RH + sr;
            const bool on = hh < G && qrow < p.m;
            lim[rr] = min(t1, base + (uint32_t)qrow + 1u);
            const float *qp = p.q + (size_t)(on ? qrow : 0) * p.ldq + (size_t)(kvh * p.group + g0 + (on ? hh : 0)) * TILE_ROWS;
#pragma unroll
            for (int ks = 0; ks < 8; ++ks) {
                float2 x0 = make_float2(0.f, 0.f), x1 = make_float2(0.f, 0.f);
                if (on) {
                    x0 = *reinterpret_cast<const float2 *>(qp + 16 * ks + 2 * t);
                    x1 = *reinterpret_cast<const float2 *>(qp + 16 * ks + 2 * t + 8);
                }
                // fragment registers: a0 (row g, k 2t..), a1 (row g+8, k 2t..), a2 (row g, k 2t+8..), a3 (row g+8, k 2t+8..)
                split_f16x2(x0.x, x0.y, qh[ks][rr], ql[ks][rr]);
                split_f16x2(x1.x, x1.y, qh[ks][NR + rr], ql[ks][NR + rr]);
            }
        }
        float o[16][4];
#pragma unroll
        for (int nt = 0; nt < 16; ++nt)
#pragma unroll
            for (int i = 0; i < 4; ++i) o[nt][i] = 0.0f;
        float mx[NR], dn[NR];
#pragma unroll
        for (int rr = 0; rr < NR; ++rr) {
            mx[rr] = -INFINITY;
            dn[rr] = 0.0f;
        }
        int st = 0;
        for (uint32_t p0 = first; p0 < t1; p0 += stride, st = st == ATC_STAGES - 1 ? 0 : st + 1) {
            // ATC_STAGES - 1 steps ahead of this one are in flight; the step fetched now goes to the stage of the step before this one
            constexpr int AHEAD = ATC_STAGES - 1;
            if (p0 + AHEAD * stride < t1) {
                stage_load(p0 + AHEAD * stride, st == 0 ? ATC_STAGES - 1 : st - 1);
                if (AHEAD == 2) asm volatile("cp.async.wait_group 2;" ::: "memory");
                else asm volatile("cp.async.wait_group 1;" ::: "memory");
            } else if (AHEAD == 2 && p0 + stride < t1) {
                asm volatile("cp.async.wait_group 1;" ::: "memory");
            } else {
                asm volatile("cp.async.wait_group 0;" ::: "memory");
            }
            __syncwarp();
            const uint32_t ks_base = my_s + (uint32_t)(st * ATC_STAGE * 2);
            const uint32_t vs_base = ks_base + 16 * ATC_ROW * 2;
            // S = Q K^T for two tiles of 8 positions.  Four accumulator chains (tile x {hi, lo} part of q), so
            // that consecutive mmas do not wait on each other, and the K fragments of the next k-step are
            // fetched while this one multiplies.
            float s0[4] = {0.f, 0.f, 0.f, 0.f}, s1[4] = {0.f, 0.f, 0.f, 0.f};
            {
                float s0l[4] = {0.f, 0.f, 0.f, 0.f}, s1l[4] = {0.f, 0.f, 0.f, 0.f};
                uint32_t kb[2][4];
                const uint32_t addr0 = ks_base + (uint32_t)((((lane >> 4) * 8 + (lane & 7)) * ATC_ROW + ((lane >> 3) & 1) * 8) * 2);
                asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                             : "=r"(kb[0][0]), "=r"(kb[0][1]), "=r"(kb[0][2]), "=r"(kb[0][3]) : "r"(addr0));
#pragma unroll
                for (int ks = 0; ks < 8; ++ks) {
                    if (ks < 7)
                        asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                                     : "=r"(kb[(ks + 1) & 1][0]), "=r"(kb[(ks + 1) & 1][1]), "=r"(kb[(ks + 1) & 1][2]), "=r"(kb[(ks + 1) & 1][3])
                                     : "r"(addr0 + 32u * (uint32_t)(ks + 1)));
                    const uint32_t(&b)[4] = kb[ks & 1];
                    const uint32_t h1 = PAIR ? qh[ks][1] : 0u, h3 = PAIR ? qh[ks][NR + 1] : 0u;
                    const uint32_t l1 = PAIR ? ql[ks][1] : 0u, l3 = PAIR ? ql[ks][NR + 1] : 0u;
                    mma_f16(s0, qh[ks][0], h1, qh[ks][NR], h3, b[0], b[1]);
                    mma_f16(s1, qh[ks][0], h1, qh[ks][NR], h3, b[2], b[3]);
                    mma_f16(s0l, ql[ks][0], l1, ql[ks][NR], l3, b[0], b[1]);
                    mma_f16(s1l, ql[ks][0], l1, ql[ks][NR], l3, b[2], b[3]);
                }
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    s0[i] += s0l[i];
                    s1[i] += s1l[i];
                }
            }
            // online softmax: fragment row g (and g+8 in the other half); this lane holds positions p0 + 2t, +1 and p0 + 8 + 2t, +1
            float pr[NR][4], rs[NR];
#pragma unroll
            for (int rr = 0; rr < NR; ++rr) {
                float sc[4];
                sc[0] = (p0 + 2 * t < lim[rr]) ? s0[2 * rr] * p.scale : -INFINITY;
                sc[1] = (p0 + 2 * t + 1 < lim[rr]) ? s0[2 * rr + 1] * p.scale : -INFINITY;
                sc[2] = (p0 + 8 + 2 * t < lim[rr]) ? s1[2 * rr] * p.scale : -INFINITY;
                sc[3] = (p0 + 8 + 2 * t + 1 < lim[rr]) ? s1[2 * rr + 1] * p.scale : -INFINITY;
                float mt = fmaxf(fmaxf(sc[0], sc[1]), fmaxf(sc[2], sc[3]));
                mt = fmaxf(mt, __shfl_xor_sync(0xffffffffu, mt, 1));
                mt = fmaxf(mt, __shfl_xor_sync(0xffffffffu, mt, 2));
                const float m_new = fmaxf(mx[rr], mt);
                // (a row may have nothing in this step: the last positions belong to later rows alone)
                rs[rr] = mx[rr] == -INFINITY ? 0.0f : expf(mx[rr] - m_new);
#pragma unroll
                for (int i = 0; i < 4; ++i) pr[rr][i] = sc[i] == -INFINITY ? 0.0f : expf(sc[i] - m_new);
                float ps = (pr[rr][0] + pr[rr][1]) + (pr[rr][2] + pr[rr][3]);
                ps += __shfl_xor_sync(0xffffffffu, ps, 1);
                ps += __shfl_xor_sync(0xffffffffu, ps, 2);
                dn[rr] = fmaf(dn[rr], rs[rr], ps);
                mx[rr] = m_new;
            }
            uint32_t ph[4] = {0u, 0u, 0u, 0u}, pl[4] = {0u, 0u, 0u, 0u};  // A fragment registers a0..a3 of P
#pragma unroll
            for (int rr = 0; rr < NR; ++rr) {
                split_f16x2(pr[rr][0], pr[rr][1], ph[rr], pl[rr]);
                split_f16x2(pr[rr][2], pr[rr][3], ph[2 + rr], pl[2 + rr]);
            }
            // O = O * r + P V, 16 tiles of 8 dimensions; the V fragments of the next pair of tiles are fetched
            // while this pair multiplies
            {
                uint32_t vb[2][4];
                const uint32_t addr0 = vs_base + (uint32_t)(((((lane >> 3) & 1) * 8 + (lane & 7)) * ATC_ROW + (lane >> 4) * 8) * 2);
                asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                             : "=r"(vb[0][0]), "=r"(vb[0][1]), "=r"(vb[0][2]), "=r"(vb[0][3]) : "r"(addr0));
#pragma unroll
                for (int nt = 0; nt < 16; nt += 2) {
                    if (nt < 14)
                        asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                                     : "=r"(vb[((nt >> 1) + 1) & 1][0]), "=r"(vb[((nt >> 1) + 1) & 1][1]), "=r"(vb[((nt >> 1) + 1) & 1][2]),
                                       "=r"(vb[((nt >> 1) + 1) & 1][3])
                                     : "r"(addr0 + 16u * (uint32_t)(nt + 2)));
                    const uint32_t(&b)[4] = vb[(nt >> 1) & 1];
#pragma unroll
                    for (int u = 0; u < 2; ++u) {
                        o[nt + u][0] *= rs[0]; o[nt + u][1] *= rs[0];
                        if (PAIR) { o[nt + u][2] *= rs[NR - 1]; o[nt + u][3] *= rs[NR - 1]; }
                    }
                    mma_f16(o[nt], ph[0], ph[1], ph[2], ph[3], b[0], b[1]);
                    mma_f16(o[nt + 1], ph[0], ph[1], ph[2], ph[3], b[2], b[3]);
                    mma_f16(o[nt], pl[0], pl[1], pl[2], pl[3], b[0], b[1]);
                    mma_f16(o[nt + 1], pl[0], pl[1], pl[2], pl[3], b[2], b[3]);
                }
            }
            __syncwarp();  // the stage is refilled two steps from now
        }
        // this warp's state per fragment row, then one warp per live fragment row merges the warps
        __syncthreads();
#pragma unroll
        for (int rr = 0; rr < NR; ++rr) {
            if (hh < G && row0 + rr * RH + sr < p.m) {
                float *stt = merge + (size_t)(warp * 8 * NR + rr * 8 + g) * ATT_PART;
#pragma unroll
                for (int nt = 0; nt < 16; ++nt) *reinterpret_cast<float2 *>(stt + nt * 8 + 2 * t) = make_float2(o[nt][2 * rr], o[nt][2 * rr + 1]);
                if (t == 0) {
                    stt[TILE_ROWS] = mx[rr];
                    stt[TILE_ROWS + 1] = dn[rr];
                }
            }
        }
        __syncthreads();
        for (int fr = warp; fr < 8 * NR; fr += ATC_WARPS) {
            const int h = (fr & 7) % Gp, qrow = row0 + (fr >> 3) * RH + (fr & 7) / Gp;
            if (h >= G || qrow >= p.m) continue;
            float M = -INFINITY;
#pragma unroll
            for (int w = 0; w < ATC_WARPS; ++w) M = fmaxf(M, merge[(size_t)(w * 8 * NR + fr) * ATT_PART + TILE_ROWS]);
            float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
            float d = 0.0f;
#pragma unroll
            for (int w = 0; w < ATC_WARPS; ++w) {
                const float *stt = merge + (size_t)(w * 8 * NR + fr) * ATT_PART;
                const float mw = stt[TILE_ROWS];
                const float wgt = mw == -INFINITY ? 0.0f : expf(mw - M);
                const float4 aw = *reinterpret_cast<const float4 *>(stt + 4 * lane);
                a.x += wgt * aw.x; a.y += wgt * aw.y; a.z += wgt * aw.z; a.w += wgt * aw.w;
                d += wgt * stt[TILE_ROWS + 1];
            }
            float *dst = p.part + (((size_t)qrow * (p.n_kv_heads * p.group) + (size_t)(kvh * p.group + g0 + h)) * p.n_splits + split) * ATT_PART;
            *reinterpret_cast<float4 *>(dst + 4 * lane) = a;
            if (lane == 0) {
                dst[TILE_ROWS] = M;
                dst[TILE_ROWS + 1] = d;
            }
        }
        __syncthreads();
    }
}

// grid (q heads, m), 128 threads: merge the splits of one head, normalise (attention.rs:391-398),
// keep the f32 row and pack the head's four 32-element blocks for the output projection.
static __global__ void __launch_bounds__(TILE_ROWS) attn_combine_kernel(AttnParams p, int pdl) {
    if (pdl) {
        pdl_launch_dependents();
        pdl_wait();
    }
    __shared__ float w[TILE_ROWS];   // weight of each split: exp(its maximum - the common maximum)
    __shared__ float red[8];
    const int head = blockIdx.x, row = blockIdx.y, i = threadIdx.x, lane = i & 31, warp = i >> 5;
    const float *src = p.part + ((size_t)row * (p.n_kv_heads * p.group) + head) * p.n_splits * ATT_PART;
    // thread s looks at split s (at most 128 splits): common maximum, weights, denominator
    const float ms = i < p.n_splits ? src[(size_t)i * ATT_PART + TILE_ROWS] : -INFINITY;
    float M = ms;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) M = fmaxf(M, __shfl_xor_sync(0xffffffffu, M, o));
    if (lane == 0) red[warp] = M;
    __syncthreads();
    M = fmaxf(fmaxf(red[0], red[1]), fmaxf(red[2], red[3]));
    const float ws = ms == -INFINITY ? 0.0f : expf(ms - M);
    w[i] = ws;
    float d = i < p.n_splits ? ws * src[(size_t)i * ATT_PART + TILE_ROWS + 1] : 0.0f;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) d += __shfl_xor_sync(0xffffffffu, d, o);
    if (lane == 0) red[4 + warp] = d;
    __syncthreads();
    d = (red[4] + red[5]) + (red[6] + red[7]);
    float a = 0.0f;
#pragma unroll 8
    for (int s = 0; s < p.n_splits; ++s) a = fmaf(w[s], src[(size_t)s * ATT_PART + i], a);
    const float o = a * (1.0f / fmaxf(d, 1.17549435e-38f));  // denom.max(f32::MIN_POSITIVE)
    if (p.out) p.out[(size_t)row * p.ldo + (size_t)head * TILE_ROWS + i] = o;
    if (p.next.base) quantize_store(p.next, p.next_two_level, p.next_need_sum, row, head * 4 + (i >> 5), i & 31, o);
}

// ------------------------------------------------------ token ends (embedding row, greedy chain)
//
// The embedding row of a token, dequantised straight out of the tiled stream (the LM head of a
// model with tied embeddings is the same resident matrix): x[i] = d * q for Q8_0
// (crates/allpaka-gguf/src/dequant.rs:93-126), d*sc*q - dmin*mn for Q4_K (dequant.rs:211-231),
// the same with the fifth bit for Q5_K (dequant.rs:238-263), d*sc*(q-32) for Q6_K (dequant.rs:271-296),
// with the reference's operation order (two roundings, no fused multiply-add).
struct EmbedParams {
    const uint8_t *W;         // tiled stream of the [vocab, hidden] table
    int ty, nb, n_rows;       // nb: 32-element blocks per row
    uint32_t tile_bytes;
    const uint32_t *token_dev;  // the token id lives on the device (greedy chain) ...
    uint32_t token;             // ... or comes with the launch
    float *x;                 // [hidden]
    int *err;
};

static __global__ void __launch_bounds__(256) embed_row_kernel(EmbedParams p) {
    uint32_t tok = p.token_dev ? *p.token_dev : p.token;
    if (tok >= (uint32_t)p.n_rows) tok = (uint32_t)p.n_rows - 1;  // (the host checks ids it can see; a chained id is an argmax over n_rows)
    const int tile = (int)(tok / TILE_ROWS), rt = (int)(tok % TILE_ROWS);
    int rg, h16, g, upper;
    frag_pos(rt, rg, h16, g, upper);
    const int idx = blockIdx.x * blockDim.x + threadIdx.x;
    if (p.ty == TY_Q8_0) {
        const int b = idx >> 3, w = idx & 7;
        if (b >= p.nb) return;
        const int ks = b / Q8_KT, bl = b % Q8_KT;
        const int kb = min(Q8_KT, p.nb - ks * Q8_KT);
        const uint8_t *unit = p.W + (size_t)tile * p.tile_bytes + (size_t)ks * Q8_KT * Q8_BLOCK_UNIT;
        const uint8_t *frag = unit + (size_t)(((bl * 4 + rg) * 2 + h16) * 32) * 16;
        const int lane = g * 4 + (w & 3), reg = 2 * (w >> 2) + upper;
        const uint32_t v = *reinterpret_cast<const uint32_t *>(frag + lane * 16 + reg * 4);
        const float d = __half2float(*reinterpret_cast<const __half *>(unit + kb * 4096 + ((bl * 4 + rg) * 8 + g) * 8 + (h16 * 2 + upper) * 2));
        float4 o;
        o.x = __fmul_rn(d, (float)(int8_t)(v & 0xffu));
        o.y = __fmul_rn(d, (float)(int8_t)((v >> 8) & 0xffu));
        o.z = __fmul_rn(d, (float)(int8_t)((v >> 16) & 0xffu));
        o.w = __fmul_rn(d, (float)(int8_t)(v >> 24));
        *reinterpret_cast<float4 *>(p.x + b * 32 + 4 * w) = o;
    } else if (p.ty == TY_Q5_0) {
        // one thread per (block, four elements): x = d * (q - 16) (dequant.rs:131-141)
        const int b = idx >> 3, w = idx & 7;
        if (b >= p.nb) return;
        const int ks = b / Q8_KT, bl = b % Q8_KT;
        const int kb = min(Q8_KT, p.nb - ks * Q8_KT);
        const uint8_t *unit = p.W + (size_t)tile * p.tile_bytes + (size_t)ks * b32_step_bytes(TY_Q5_0, Q8_KT);
        const int lane = g * 4 + (w & 3), reg = 2 * (w >> 2) + upper;
        uint32_t nib = *reinterpret_cast<const uint32_t *>(unit + bl * 2048 + rg * 512 + h16 * 256 + lane * 8 + upper * 4);
        if (w >= 4) nib >>= 4;
        const uint32_t qh = *reinterpret_cast<const uint32_t *>(unit + kb * 2048 + ((rg * 2 + h16) * 32 + lane) * 16 + reg * 4);
        const uint32_t v = (nib & 0x0f0f0f0fu) | (((qh >> bl) & 0x01010101u) << 4);
        const float d = __half2float(*reinterpret_cast<const __half *>(unit + b32_scale_off(TY_Q5_0, kb) + ((bl * 4 + rg) * 8 + g) * 8 + (h16 * 2 + upper) * 2));
        float4 o;
        o.x = __fmul_rn(d, (float)((int)(v & 0xffu) - 16));
        o.y = __fmul_rn(d, (float)((int)((v >> 8) & 0xffu) - 16));
        o.z = __fmul_rn(d, (float)((int)((v >> 16) & 0xffu) - 16));
        o.w = __fmul_rn(d, (float)((int)(v >> 24) - 16));
        *reinterpret_cast<float4 *>(p.x + b * 32 + 4 * w) = o;
    } else if (ty_k6(p.ty)) {
        // one thread per (super-block, half, 4-byte word): four values of each of the half's quarters,
        // x = d * sc * q in that order (dequant.rs:290-293); Q2_K: x = d * sc * q - dmin * mn (dequant.rs:163-168)
        const int sb = idx >> 4, half = (idx >> 3) & 1, w = idx & 7;
        if (sb >= p.nb / 8) return;
        const bool k2 = p.ty == TY_Q2_K;
        const int k6_rg = k2 ? Q2_SB_RG : Q6_SB_RG;
        const uint8_t *base = p.W + (size_t)tile * p.tile_bytes + (size_t)sb * (4 * k6_rg) + (size_t)rg * k6_rg;
        const int lane = g * 4 + (w & 3), reg = 2 * (w >> 2) + upper, row4 = h16 * 2 + upper;
        const uint32_t qh = *reinterpret_cast<const uint32_t *>(base + 4096 + (size_t)((half * 2 + h16) * 32) * 16 + lane * 16 + reg * 4);
        const float d = __half2float(*reinterpret_cast<const __half *>(base + 6656 + (g * 4 + row4) * 2));
        const int8_t *sc = reinterpret_cast<const int8_t *>(base + 6144 + (g * 4 + row4) * 16) + half * 8;
        const int is = w >> 2;  // elements 4w..4w+3 of a quarter lie in its 16-element half `is`
        const float dmin = k2 ? __half2float(*reinterpret_cast<const __half *>(base + Q6_SB_RG + 512 + (g * 4 + row4) * 2)) : 0.0f;
        const uint8_t *mn = base + Q6_SB_RG + (g * 4 + row4) * 16 + half * 8;
        float *o = p.x + sb * 256 + half * 128 + 4 * w;
#pragma unroll
        for (int qi = 0; qi < 4; ++qi) {
            const uint32_t ql = *reinterpret_cast<const uint32_t *>(base + (size_t)(((half * 2 + (qi & 1)) * 2 + h16) * 32) * 16 + lane * 16 + reg * 4);
            const float dsc = __fmul_rn(d, (float)sc[2 * qi + is]);
            const float ml = k2 ? __fmul_rn(dmin, (float)mn[2 * qi + is]) : 0.0f;
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const uint32_t nib = ((qi & 2) ? (ql >> (8 * k + 4)) : (ql >> (8 * k))) & 0xfu;
                const int q = (int)(nib | (((qh >> (8 * k + 2 * qi)) & 3u) << 4)) - 32;
                o[32 * qi + k] = k2 ? __fsub_rn(__fmul_rn(dsc, (float)q), ml) : __fmul_rn(dsc, (float)q);
            }
        }
    } else {
        // one thread per (super-block, pair of sub-blocks, 4-byte word of nibbles)
        const int sb = idx >> 5, pr = (idx >> 3) & 3, w = idx & 7;
        if (sb >= p.nb / 8) return;
        const int ks = sb / Q4_KT_SB, sl = sb % Q4_KT_SB;
        const bool k5 = p.ty == TY_Q5_K;
        const int sb_rg = k5 ? Q5_SB_RG : Q4_SB_RG, sb_unit = 4 * sb_rg;
        const uint8_t *base = p.W + (size_t)tile * p.tile_bytes + (size_t)ks * Q4_KT_SB * sb_unit + (size_t)sl * sb_unit +
                              (size_t)rg * sb_rg;
        const uint8_t *frag = base + (size_t)((pr * 2 + h16) * 32) * 16;
        const int lane = g * 4 + (w & 3), reg = 2 * (w >> 2) + upper;
        const uint32_t v = *reinterpret_cast<const uint32_t *>(frag + lane * 16 + reg * 4);
        // Q5_K: bit 2*pr of qh[l] adds 16 to the low-nibble sub-block's element l, bit 2*pr+1 to the high one's (dequant.rs:253-260)
        const uint32_t qh = k5 ? *reinterpret_cast<const uint32_t *>(base + 4096 + (size_t)(h16 * 32) * 16 + lane * 16 + reg * 4) : 0u;
        const uint8_t *hdr = base + (k5 ? 5120 : 4096);
        const int row4 = h16 * 2 + upper;
        const uint32_t dd = *reinterpret_cast<const uint32_t *>(hdr + (g * 4 + row4) * 4);
        const float d = __half2float(__ushort_as_half((unsigned short)(dd & 0xffffu)));
        const float dmin = __half2float(__ushort_as_half((unsigned short)(dd >> 16)));
        const int j1 = 2 * pr, j2 = 2 * pr + 1;
        const float sc1 = (float)hdr[128 + ((g * 2 + (j1 >> 2)) * 4 + row4) * 4 + (j1 & 3)];
        const float mn1 = (float)hdr[384 + ((g * 2 + (j1 >> 2)) * 4 + row4) * 4 + (j1 & 3)];
        const float sc2 = (float)hdr[128 + ((g * 2 + (j2 >> 2)) * 4 + row4) * 4 + (j2 & 3)];
        const float mn2 = (float)hdr[384 + ((g * 2 + (j2 >> 2)) * 4 + row4) * 4 + (j2 & 3)];
        const float d_sc1 = __fmul_rn(d, sc1), dm1 = __fmul_rn(dmin, mn1);
        const float d_sc2 = __fmul_rn(d, sc2), dm2 = __fmul_rn(dmin, mn2);
        float *o = p.x + sb * 256 + pr * 64 + 4 * w;
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const uint32_t byte = (v >> (8 * k)) & 0xffu, hb = (qh >> (8 * k + 2 * pr)) & 3u;
            o[k] = __fsub_rn(__fmul_rn(d_sc1, (float)((byte & 0xfu) + ((hb & 1u) << 4))), dm1);
            o[32 + k] = __fsub_rn(__fmul_rn(d_sc2, (float)((byte >> 4) + ((hb >> 1) << 4))), dm2);
        }
    }
}

// One step of the greedy chain, after the token's graph: keep the winner, make it the next
// input token, and put the next position's RoPE row in place.  One CTA.
struct ChainParams {
    const uint32_t *amax;  // the step's greedy winner
    uint32_t *token;       // next input token
    uint32_t *hist;        // [steps] winners so far
    uint32_t *step;        // steps done
    const float *rope_tab; // [steps][row] (sin, cos) rows, one per position
    float *rope;           // the row the token graph reads
    int row;               // floats per row
    int n_steps;
    uint32_t *pos;         // cache position of the next token (advanced here)
};
static __global__ void __launch_bounds__(128) chain_advance_kernel(ChainParams p) {
    const uint32_t s = *p.step;
    if (threadIdx.x == 0) {
        p.hist[s] = *p.amax;
        *p.token = *p.amax;
        if (p.pos) *p.pos += 1u;
    }
    if (s + 1 < (uint32_t)p.n_steps)
        for (int i = threadIdx.x; i < p.row; i += blockDim.x) p.rope[i] = p.rope_tab[(size_t)(s + 1) * p.row + i];
    __syncthreads();
    if (threadIdx.x == 0) *p.step = s + 1;
}

// ------------------------------------------------- synthetic weights (bench)
//
// Counter-based generator for benchmark tensors: raw GGUF blocks are produced
// on the device so a multi-gigabyte synthetic model needs no host generation.
// Q8_0: quants uniform in [-127,127], scale f16(|N(0,0.02)|/127).
// Q4_K: nibbles, 6-bit scales and mins uniform, d and dmin f16(|N(0,0.002)|).
// Q6_K: see synth_q6_k_kernel.
__device__ __forceinline__ uint64_t splitmix64(uint64_t x) {
    x += 0x9E3779B97F4A7C15ull;
    x = (x ^ (x >> 30)) * 0xBF58476D1CE4E5B9ull;
    x = (x ^ (x >> 27)) * 0x94D049BB133111EBull;
    return x ^ (x >> 31);
}
__device__ __forceinline__ float absnormal(uint64_t h, float sigma) {
    const float u1 = ((float)(uint32_t)(h >> 40) + 1.0f) * (1.0f / 16777217.0f);
    const float u2 = (float)(uint32_t)(h & 0xffffffu) * (1.0f / 16777216.0f);
    return fabsf(sqrtf(-2.0f * logf(u1)) * cospif(2.0f * u2)) * sigma;
}
// Q2_K: uniform bytes for the packed scales / mins and the quants, d and dmin ~ |N(0, 4e-4)|
static __global__ void synth_q2_k_kernel(uint8_t *dst, size_t n_blocks, uint64_t seed) {
    const size_t b = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (b >= n_blocks) return;
    uint8_t *o = dst + b * 84;
    const uint64_t base = splitmix64(seed) ^ (b * 0x9E3779B97F4A7C15ull);
    for (int i = 0; i < 10; ++i) {
        const uint64_t h = splitmix64(base + (uint64_t)i + 1);
        for (int j = 0; j < 8; ++j) o[i * 8 + j] = (uint8_t)(h >> (8 * j));
    }
    const unsigned short db = __half_as_ushort(__float2half_rn(absnormal(splitmix64(base ^ 0x51ull), 4e-4f)));
    const unsigned short mb = __half_as_ushort(__float2half_rn(absnormal(splitmix64(base ^ 0x52ull), 4e-4f)));
    o[80] = (uint8_t)(db & 0xff);
    o[81] = (uint8_t)(db >> 8);
    o[82] = (uint8_t)(mb & 0xff);
    o[83] = (uint8_t)(mb >> 8);
}
// Q3_K: uniform bytes for the masks, quants and packed scales, d ~ |N(0, 1e-4)|
static __global__ void synth_q3_k_kernel(uint8_t *dst, size_t n_blocks, uint64_t seed) {
    const size_t b = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (b >= n_blocks) return;
    uint8_t *o = dst + b * 110;
    const uint64_t base = splitmix64(seed) ^ (b * 0x9E3779B97F4A7C15ull);
    for (int i = 0; i < 14; ++i) {
        const uint64_t h = splitmix64(base + (uint64_t)i + 1);
        for (int j = 0; j < 8; ++j)
            if (i * 8 + j < 108) o[i * 8 + j] = (uint8_t)(h >> (8 * j));
    }
    const unsigned short db = __half_as_ushort(__float2half_rn(absnormal(splitmix64(base ^ 0x51ull), 1e-4f)));
    o[108] = (uint8_t)(db & 0xff);
    o[109] = (uint8_t)(db >> 8);
}
// Q5_0: scale |N(0, 0.02)| / 15, uniform fifth bits and nibbles
static __global__ void synth_q5_0_kernel(uint8_t *dst, size_t n_blocks, uint64_t seed) {
    const size_t b = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (b >= n_blocks) return;
    uint8_t *o = dst + b * 22;
    const uint64_t base = splitmix64(seed) ^ (b * 0x9E3779B97F4A7C15ull);
    const unsigned short db = __half_as_ushort(__float2half_rn(absnormal(splitmix64(base ^ 0x51ull), 0.02f) / 15.0f));
    o[0] = (uint8_t)(db & 0xff);
    o[1] = (uint8_t)(db >> 8);
#pragma unroll
    for (int i = 0; i < 3; ++i) {
        const uint64_t h = splitmix64(base + (uint64_t)i + 1);
#pragma unroll
        for (int j = 0; j < 8; ++j)
            if (2 + i * 8 + j < 22) o[2 + i * 8 + j] = (uint8_t)(h >> (8 * j));
    }
}
// one thread per block of the raw row-major GGUF layout
static __global__ void synth_q8_0_kernel(uint8_t *dst, size_t n_blocks, uint64_t seed) {
    const size_t b = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (b >= n_blocks) return;
    uint8_t *o = dst + b * 34;
    const uint64_t base = splitmix64(seed) ^ (b * 0x9E3779B97F4A7C15ull);
    const __half d = __float2half_rn(absnormal(splitmix64(base ^ 0x51ull), 0.02f) / 127.0f);
    const unsigned short db = __half_as_ushort(d);
    o[0] = (uint8_t)(db & 0xff);
    o[1] = (uint8_t)(db >> 8);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const uint64_t h = splitmix64(base + (uint64_t)i + 1);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const uint32_t u16 = (uint32_t)(h >> (16 * j)) & 0xffffu;
            o[2 + i * 4 + j] = (uint8_t)(int8_t)((int)((u16 * 255u) >> 16) - 127);
        }
    }
}
static __global__ void synth_q4_k_kernel(uint8_t *dst, size_t n_blocks, uint64_t seed) {
    const size_t b = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (b >= n_blocks) return;
    uint8_t *o = dst + b * 144;
    const uint64_t base = splitmix64(seed) ^ (b * 0x9E3779B97F4A7C15ull);
    const unsigned short d = __half_as_ushort(__float2half_rn(absnormal(splitmix64(base ^ 0x51ull), 0.002f)));
    const unsigned short dm = __half_as_ushort(__float2half_rn(absnormal(splitmix64(base ^ 0x52ull), 0.002f)));
    o[0] = (uint8_t)(d & 0xff); o[1] = (uint8_t)(d >> 8);
    o[2] = (uint8_t)(dm & 0xff); o[3] = (uint8_t)(dm >> 8);
    for (int i = 0; i < 140 / 4; ++i) {
        const uint32_t h = (uint32_t)splitmix64(base + (uint64_t)i + 1);
        o[4 + i * 4 + 0] = (uint8_t)h; o[4 + i * 4 + 1] = (uint8_t)(h >> 8);
        o[4 + i * 4 + 2] = (uint8_t)(h >> 16); o[4 + i * 4 + 3] = (uint8_t)(h >> 24);
    }
}

// Q5_K: as Q4_K with 32 more uniform bytes (the high bits).
static __global__ void synth_q5_k_kernel(uint8_t *dst, size_t n_blocks, uint64_t seed) {
    const size_t b = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (b >= n_blocks) return;
    uint8_t *o = dst + b * 176;
    const uint64_t base = splitmix64(seed) ^ (b * 0x9E3779B97F4A7C15ull);
    const unsigned short d = __half_as_ushort(__float2half_rn(absnormal(splitmix64(base ^ 0x53ull), 0.001f)));
    const unsigned short dm = __half_as_ushort(__float2half_rn(absnormal(splitmix64(base ^ 0x54ull), 0.001f)));
    o[0] = (uint8_t)(d & 0xff); o[1] = (uint8_t)(d >> 8);
    o[2] = (uint8_t)(dm & 0xff); o[3] = (uint8_t)(dm >> 8);
    for (int i = 0; i < 172 / 4; ++i) {
        const uint32_t h = (uint32_t)splitmix64(base + (uint64_t)i + 1);
        o[4 + i * 4 + 0] = (uint8_t)h; o[4 + i * 4 + 1] = (uint8_t)(h >> 8);
        o[4 + i * 4 + 2] = (uint8_t)(h >> 16); o[4 + i * 4 + 3] = (uint8_t)(h >> 24);
    }
}

// Q6_K: every ql/qh byte and every int8 sub-block scale uniform, d f16(|N(0,2.5e-5)|).
static __global__ void synth_q6_k_kernel(uint8_t *dst, size_t n_blocks, uint64_t seed) {
    const size_t b = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (b >= n_blocks) return;
    uint8_t *o = dst + b * 210;
    const uint64_t base = splitmix64(seed) ^ (b * 0x9E3779B97F4A7C15ull);
    for (int i = 0; i < 208 / 4; ++i) {
        const uint32_t h = (uint32_t)splitmix64(base + (uint64_t)i + 1);
        o[i * 4 + 0] = (uint8_t)h; o[i * 4 + 1] = (uint8_t)(h >> 8);
        o[i * 4 + 2] = (uint8_t)(h >> 16); o[i * 4 + 3] = (uint8_t)(h >> 24);
    }
    const unsigned short d = __half_as_ushort(__float2half_rn(absnormal(splitmix64(base ^ 0x61ull), 2.5e-5f)));
    o[208] = (uint8_t)(d & 0xff); o[209] = (uint8_t)(d >> 8);
}

// ------------------------------------------------------------ the matvec

// Shared memory map of the matvec kernel (dynamic, 128-byte aligned base):
//   [0, 64)      full barriers       [64, 128) empty barriers
//   [128, 136)   barrier of the resident-activation load    [136, 144) prologue scratch released
//   [144, 152)   red full (consumers -> finishers)          [152, 160) red empty (finishers -> consumers)
//   [160, 192)   flags: tile and last-tile mark of the hand-off, finisher-local words
//   [256 ..)     red[4][M][128] f32  K-quarter partials of the tile the consumers just left
//   [..]         fin[M][128] f32     the finishers' working copy (tile result), then the slot table
//   [..]         resident activation records (PRO_LOAD / PRO_QUANT), all K-steps
//   [..]         stages: n_stages * (one K-step of weights [+ one activation record when streaming])
constexpr int SLOT_TAB_BYTES = 640;  // one int per CTA that can share a tile (grids of up to 160 CTAs)
template <int M>
struct MvSmem {
    static constexpr int RED_OFF = 256;
    static constexpr int RED_BYTES = K_SPLIT * M * TILE_ROWS * 4;
    static constexpr int FIN_OFF = RED_OFF + RED_BYTES;
    static constexpr int SLOT_OFF = FIN_OFF + M * TILE_ROWS * 4;
    static constexpr int RES_OFF = SLOT_OFF + SLOT_TAB_BYTES;
};
__host__ __device__ inline int mv_resident_bytes(int pro, int KS, int act_rec) {
    return pro == PRO_STREAM ? 0 : ((KS * act_rec + 127) & ~127);
}
__host__ __device__ inline int mv_stage_bytes(int ty, int pro, int act_rec) {
    return stage_w_bytes(ty) + (pro == PRO_STREAM ? ((act_rec + 127) & ~127) : 0);
}
__host__ __device__ inline int mv_smem_total(int ty, int m_eff, int pro, int KS, int act_rec, int n_stages) {
    return 256 + (K_SPLIT + 1) * m_eff * TILE_ROWS * 4 + SLOT_TAB_BYTES + mv_resident_bytes(pro, KS, act_rec) + n_stages * mv_stage_bytes(ty, pro, act_rec);
}

// The order in which a CTA walks its range [u_begin, u_end) of the flat unit
// sequence: the tile pieces it shares with neighbours first (tail piece, then
// head piece), whole tiles after.  A shared tile's cross-CTA hand-off (publish,
// count, last arriver sums) then overlaps the streaming of the whole tiles
// instead of sitting at the very end of the kernel.
// (All unit arithmetic is 32-bit: the host checks tiles * K-steps * grid < 2^31.)
struct UnitOrder {
    uint32_t u_begin, u_end;
    int n_total, len_tail, len_head;
    __device__ UnitOrder(uint32_t ub, uint32_t ue, uint32_t KS) : u_begin(ub), u_end(ue) {
        n_total = (int)(ue - ub);
        const uint32_t t_first = ub / KS, t_last = (ue - 1) / KS;
        const uint32_t h_end = (t_first + 1) * KS < ue ? (t_first + 1) * KS : ue;
        const bool head_partial = (ub % KS) != 0 || (h_end - ub) < KS;
        len_head = head_partial ? (int)(h_end - ub) : 0;
        len_tail = (t_last > t_first && (ue % KS) != 0) ? (int)(ue - t_last * KS) : 0;
    }
    __device__ __forceinline__ uint32_t at(int it) const {
        if (it < len_tail) return u_end - len_tail + it;
        if (it < len_tail + len_head) return u_begin + (it - len_tail);
        return u_begin + it - len_tail;  // = u_begin + len_head + (it - len_tail - len_head)
    }
};

template <int M>
__device__ __forceinline__ void epilogue_tile(const MvParams &p, const Crew &cw, int tile, float *out /*[M][128] smem*/,
                                              const float *pre, const float *rope_pre, float gam_pre);
constexpr int EPI_PRE = 2;  // residual values a finisher thread fetches ahead of the EPI_ADD epilogue

// In-CTA activation prologue (PRO_QUANT): the consumer threads turn one row
// x (n <= N_CONSUMERS * PRO_CH elements) into Q8 blocks in shared memory, after the
// optional RMSNorm, entirely in registers.
//  * The norm weight does not depend on the previous kernel: it is loaded
//    BEFORE the dependency wait (prologue_gamma).
//  * The row itself is read by the consumer threads with plain 16-byte loads right
//    after the wait (they return sooner than a copy staged through shared memory).
//    The last ring stage stays free until pro_bar completes: the exact block sums
//    of the Q4_K flavour use it as scratch.
//  * Thread t owns elements 4t..4t+3 of every 2048-element chunk j, so the 8
//    lanes t&~7 .. t|7 hold one 32-element block: block maximum = 3 shuffles,
//    then the IEEE divide / reciprocal, rounding and one packed 32-bit store,
//    the PRO_J chunks being independent chains that overlap.
// Arithmetic is Q8Acts::from_f32 (quantmat/q8_acts.rs:26-63) exactly; the
// left-to-right f32 block sum (needed by Q4_K consumers only) is done one block
// per thread over a padded copy of the row.
constexpr int PRO_J = 3;            // chunks of 4 * N_CONSUMERS = 2048 elements
constexpr int PRO_CH = 4 * PRO_J;   // elements per thread
constexpr int PRO_CHUNK = 4 * N_CONSUMERS;
constexpr int PRO_MAX_N = PRO_J * PRO_CHUNK;  // longest row the in-CTA prologue takes (6144)

__device__ __forceinline__ void prologue_gamma(const MvParams &p, int tid, float (&g)[PRO_CH]) {
    const PrepParams &pp = p.prep;
#pragma unroll
    for (int j = 0; j < PRO_J; ++j) {
        const int e = 4 * tid + PRO_CHUNK * j;
        float4 w = make_float4(1.0f, 1.0f, 1.0f, 1.0f);
        if (pp.gamma && e < pp.n) w = *reinterpret_cast<const float4 *>(pp.gamma + e);
        g[4 * j] = w.x; g[4 * j + 1] = w.y; g[4 * j + 2] = w.z; g[4 * j + 3] = w.w;
    }
}

template <int M>
__device__ __forceinline__ void prologue_quant(const MvParams &p, uint8_t *res, float *hs, float *red, int tid,
                                               const float (&g)[PRO_CH], double ssq_in, const float4 (&xr)[PRO_J]) {
    const PrepParams &pp = p.prep;
    const int warp = tid >> 5, lane = tid & 31;
    const int n = pp.n, nb = n >> 5;
    ActLayout L = p.act;
    L.base = res;
    L.m_eff = M;
    const int ke = L.ke, kt_shift = ke == 256 ? 3 : 4, kt = 1 << kt_shift, mp = L.mp();
    const int rec_bytes = L.rec_bytes(), q_bytes = L.q_bytes();
    double *dred = reinterpret_cast<double *>(red);
    float v[PRO_CH];
    if (p.xin.index >= 0) {
        // Tensor parallel: the row is the sum of what every rank stored into this rank's
        // exchange buffer as tagged words (rank 0: old residual + its partial sums, the others:
        // their partial sums).  Poll them (bounded) and add the slots in rank order; CTA 0
        // keeps the new residual row.
        float *mine = p.xch.slots[p.xch.rank];
        const uint32_t e = xch_number(mine, p.xin);
        bool ok = true;
        size_t off[PRO_J];
        bool live[PRO_J];
        float4 xs[PRO_J];
#pragma unroll
        for (int j = 0; j < PRO_J; ++j) {
            off[j] = (size_t)(4 * tid + PRO_CHUNK * j);
            live[j] = 4 * tid + PRO_CHUNK * j < n;
        }
        xch_gather<PRO_J>(mine, e, p.xch.world, off, live, p.wait_limit, &ok, xs);
#pragma unroll
        for (int j = 0; j < PRO_J; ++j) {
            const int el = 4 * tid + PRO_CHUNK * j;
            const float4 x = xs[j];
            if (el < n && pp.xout && blockIdx.x == 0) *reinterpret_cast<float4 *>(pp.xout + el) = x;
            v[4 * j] = x.x; v[4 * j + 1] = x.y; v[4 * j + 2] = x.z; v[4 * j + 3] = x.w;
        }
        if (!ok) atomicCAS(p.err, 0, ERRW_PEER_TIMEOUT | (p.launch_id << 8));  // goes on with what is there; the host reports the error
    } else {
#pragma unroll
        for (int j = 0; j < PRO_J; ++j) {
            const int e = 4 * tid + PRO_CHUNK * j;
            float4 x = xr[j];  // loaded by the caller right after the dependency resolved
            if (e < n) {
                if (pp.add) {
                    const float4 a = __ldcg(reinterpret_cast<const float4 *>(pp.add + e));
                    x.x = __fadd_rn(x.x, a.x); x.y = __fadd_rn(x.y, a.y); x.z = __fadd_rn(x.z, a.z); x.w = __fadd_rn(x.w, a.w);
                }
                if (pp.xout && blockIdx.x == 0) *reinterpret_cast<float4 *>(pp.xout + e) = x;
            }
            v[4 * j] = x.x; v[4 * j + 1] = x.y; v[4 * j + 2] = x.z; v[4 * j + 3] = x.w;
        }
    }
    if (pp.gamma) {
        // ops::rmsnorm_into (ops/norm.rs:193-198): f64 sum of squares, f64 1/sqrt(mean + eps)
        double tot;
        if (pp.sumsq) {
            tot = ssq_in;  // the producer of the row left the per-block sums (added up by the caller)
        } else {
            double ss = 0.0;
#pragma unroll
            for (int j = 0; j < PRO_CH; ++j) ss = fma((double)v[j], (double)v[j], ss);
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
            if (lane == 0) dred[warp] = ss;
            consumer_bar();
            tot = 0.0;
#pragma unroll
            for (int i = 0; i < N_CONSUMER_WARPS; ++i) tot += dred[i];
        }
        // one lane per warp does the f64 division and square root (the double-precision pipe is
        // narrow: 512 threads doing it side by side cost more than the broadcast)
        double scale = 0.0;
        if (lane == 0) scale = 1.0 / sqrt(tot / (double)n + (double)pp.eps);
        scale = __shfl_sync(0xffffffffu, scale, 0);
#pragma unroll
        for (int j = 0; j < PRO_CH; ++j) v[j] = __fmul_rn((float)((double)v[j] * scale), g[j]);
        if (pp.hout && blockIdx.x == 0) {
#pragma unroll
            for (int j = 0; j < PRO_J; ++j) {
                const int e = 4 * tid + PRO_CHUNK * j;
                if (e < n) *reinterpret_cast<float4 *>(pp.hout + e) = make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
            }
        }
    }
    if (p.timeline && tid == 0) p.timeline[(size_t)blockIdx.x * 8 + 7] = globaltimer_ns();  // row normalised
    if (pp.need_sum) {
        // exact sequential block sums: padded copy of the row, one block per thread
        consumer_bar();  // everyone has read the raw row
#pragma unroll
        for (int j = 0; j < PRO_J; ++j) {
            const int e = 4 * tid + PRO_CHUNK * j;
            if (e < n) {
                float *h4 = hs + e + (e >> 5);
                h4[0] = v[4 * j]; h4[1] = v[4 * j + 1]; h4[2] = v[4 * j + 2]; h4[3] = v[4 * j + 3];
            }
        }
        consumer_bar();
        for (int b = tid; b < nb; b += N_CONSUMERS) {
            const float *hb = hs + b * 33;
            float sum = 0.0f;
#pragma unroll 8
            for (int k = 0; k < 32; ++k) sum = __fadd_rn(sum, hb[k]);  // strictly left to right
            float *d = reinterpret_cast<float *>(res + (size_t)(b >> kt_shift) * rec_bytes + q_bytes);
            d[kt * mp + (b & (kt - 1)) * mp] = sum;           // row 0 carries sum(x)
            if (pp.two_level) d[kt * mp + (b & (kt - 1)) * mp + 1] = 0.0f;  // the residual row adds nothing to the min term
        }
    }
    const int levels = pp.two_level ? 2 : 1;
    // Stage by stage across the PRO_J chunks (not chunk by chunk): the warp shuffles
    // order the instruction stream, so independent work has to sit side by side for
    // the chains of the five blocks to overlap.
    float dprev[PRO_J];
#pragma unroll
    for (int lv = 0; lv < 2; ++lv) {
        if (lv < levels) {
            float amax[PRO_J], db[PRO_J], id[PRO_J];
            int q[PRO_CH];
            if (lv == 0) {
#pragma unroll
                for (int j = 0; j < PRO_J; ++j) {
                    amax[j] = fmaxf(fmaxf(fabsf(v[4 * j]), fabsf(v[4 * j + 1])), fmaxf(fabsf(v[4 * j + 2]), fabsf(v[4 * j + 3])));
                    if (amax[j] != amax[j]) amax[j] = 0.0f;  // all four NaN: f32::max drops NaN operands
                }
#pragma unroll
                for (int o = 1; o <= 4; o <<= 1) {
                    float t[PRO_J];
#pragma unroll
                    for (int j = 0; j < PRO_J; ++j) t[j] = __shfl_xor_sync(0xffffffffu, amax[j], o);
#pragma unroll
                    for (int j = 0; j < PRO_J; ++j) amax[j] = fmaxf(amax[j], t[j]);
                }
#pragma unroll
                for (int j = 0; j < PRO_J; ++j) db[j] = amax[j] <= 3.402823466e+38f ? __fdiv_rn(amax[j], 127.0f) : 0.0f;
            } else {
                // the residual's scale is d1 / 256 exactly (see quantize_store)
#pragma unroll
                for (int j = 0; j < PRO_J; ++j) db[j] = dprev[j] * 0.00390625f;
            }
#pragma unroll
            for (int j = 0; j < PRO_J; ++j) {
                id[j] = (db[j] > 0.0f) ? __frcp_rn(db[j]) : 0.0f;  // IEEE 1.0/db
                dprev[j] = db[j];
            }
#pragma unroll
            for (int k = 0; k < PRO_CH; ++k) {
                q[k] = q8_round(v[k], id[k >> 2]);
                if (lv == 1) q[k] = max(-127, min(127, q[k]));
            }
#pragma unroll
            for (int j = 0; j < PRO_J; ++j) {
                const int e = 4 * tid + PRO_CHUNK * j;
                const int b = e >> 5;
                if (e < n) {
                    uint8_t *rec = res + (size_t)(b >> kt_shift) * rec_bytes;
                    const int bl = b & (kt - 1);
                    *reinterpret_cast<uint32_t *>(rec + ((bl * 2 + ((e >> 4) & 1)) * M + lv) * 16 + (e & 15)) =
                        (uint32_t)(q[4 * j] & 0xff) | ((uint32_t)(q[4 * j + 1] & 0xff) << 8) |
                        ((uint32_t)(q[4 * j + 2] & 0xff) << 16) | ((uint32_t)(q[4 * j + 3] & 0xff) << 24);
                    if ((tid & 7) == 0) {
                        float *d = reinterpret_cast<float *>(rec + q_bytes);
                        d[bl * mp + lv] = db[j];
                        if (!pp.need_sum) d[kt * mp + bl * mp + lv] = 0.0f;
                    }
                }
            }
            if (lv + 1 < levels) {
                // residual for the second digit, exact in one fused operation
#pragma unroll
                for (int k = 0; k < PRO_CH; ++k) v[k] = __fmaf_rn(-db[k >> 2], (float)q[k], v[k]);
            }
        }
    }
    consumer_bar();
}

template <int TY, int M, bool DUMP>
__global__ void __launch_bounds__(MV_THREADS, 1) matvec_streamk_kernel(const MvParams p) {
    extern __shared__ __align__(128) uint8_t smem[];
    uint64_t *full = reinterpret_cast<uint64_t *>(smem);
    uint64_t *empty = full + MAX_STAGES;
    uint64_t *acts_bar = reinterpret_cast<uint64_t *>(smem + 128);
    uint64_t *pro_bar = reinterpret_cast<uint64_t *>(smem + 136);  // PRO_QUANT scratch (last stage) released
    uint64_t *red_full = reinterpret_cast<uint64_t *>(smem + 144);   // a tile's K-quarter partials are in red
    uint64_t *red_empty = reinterpret_cast<uint64_t *>(smem + 152);  // the finishers have taken them
    int *s_flags = reinterpret_cast<int *>(smem + 160);
    float *red = reinterpret_cast<float *>(smem + MvSmem<M>::RED_OFF);
    const int act_rec = p.act.rec_bytes();
    const bool streaming = p.pro == PRO_STREAM;
    uint8_t *res = smem + MvSmem<M>::RES_OFF;
    const int stage_bytes = mv_stage_bytes(TY, p.pro, act_rec);
    uint8_t *stages = res + mv_resident_bytes(p.pro, p.KS, act_rec);
    const int NS = p.n_stages;

    // Few activation rows (M <= 4): the eight result columns of an mma are shared out among
    // 8 / MP2 consecutive blocks x MP2 rows ("chained columns", see the consumers below); the
    // two halves of the consumer warps then take alternate K-steps.
    constexpr bool CH = M <= 4;
    constexpr int MP2 = M <= 1 ? 1 : (M <= 2 ? 2 : 4);  // result columns per block
    constexpr int BPC = 8 / MP2;                        // blocks per mma chain
    constexpr int KQ = CH ? 2 : K_SPLIT;                // partial sums per tile row handed to the finishers

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    unsigned long long *tl = p.timeline ? p.timeline + (size_t)blockIdx.x * 8 : nullptr;
    if (tl && tid == 0) tl[0] = globaltimer_ns();
    // prepared records arrive by bulk copy; a row still to be quantised is read straight into
    // registers by the consumer threads (plain loads return sooner than a copy through shared memory)
    const bool acts_copy = p.pro == PRO_LOAD;
    if (tid == 0) {
        for (int s = 0; s < NS; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], CH ? N_CONSUMER_WARPS / 2 : N_CONSUMER_WARPS);
        }
        mbar_init(acts_bar, 1);
        mbar_init(pro_bar, N_CONSUMER_WARPS);
        mbar_init(red_full, N_CONSUMER_WARPS);
        mbar_init(red_empty, 1);
        fence_mbar_init();
    }
    __syncthreads();
    if (p.pdl) pdl_launch_dependents();

    // this CTA's contiguous range of the flat unit sequence
    const uint32_t U = (uint32_t)p.n_tiles * (uint32_t)p.KS;
    const uint32_t G = gridDim.x;
    const UnitOrder order(blockIdx.x * U / G, (blockIdx.x + 1) * U / G, (uint32_t)p.KS);
    const int n_total = order.n_total;
    const int kt = ty_k45(TY) ? Q4_KT_SB * 8 : Q8_KT;  // 32-element blocks per full K-step
    constexpr int K45_RG = k45_sb_rg(TY), K45_UNIT = 4 * K45_RG, K45_HDR = k45_hdr(TY);  // (meaningful for Q4_K / Q5_K)
    constexpr bool K5 = TY == TY_Q5_K;

    if (warp == N_CONSUMER_WARPS) {
        // ------------------------------------------------ producer (one lane)
        if (lane == 0) {
            const uint64_t pol_w = l2_policy_evict_first();
            const uint64_t pol_a = l2_policy_evict_last();
            auto issue_weights = [&](int it) {
                const uint32_t u = order.at(it);
                const int s = it % NS;
                const int t = (int)(u / p.KS), ks = (int)(u % p.KS);
                const int kb = min(kt, p.nb - ks * kt);
                uint32_t wbytes, woff;
                if (ty_b32(TY)) {
                    wbytes = (uint32_t)b32_step_bytes(TY, kb);
                    woff = (uint32_t)ks * (uint32_t)b32_step_bytes(TY, Q8_KT);
                } else if (ty_k6(TY)) {
                    wbytes = (uint32_t)(4 * k6_sb_rg(TY));
                    woff = (uint32_t)ks * (uint32_t)(4 * k6_sb_rg(TY));
                } else {
                    wbytes = (uint32_t)(kb / 8) * K45_UNIT;
                    woff = (uint32_t)ks * Q4_KT_SB * K45_UNIT;
                }
                mbar_arrive_expect_tx(&full[s], wbytes + (streaming ? (uint32_t)act_rec : 0u));
                bulk_g2s(stages + (size_t)s * stage_bytes, p.W + (size_t)t * p.tile_bytes + woff, wbytes, &full[s], pol_w);
            };
            auto issue_acts = [&](int it) {
                const int s = it % NS;
                const int ks = (int)(order.at(it) % p.KS);
                bulk_g2s(stages + (size_t)s * stage_bytes + stage_w_bytes(TY), p.act.base + (size_t)ks * act_rec,
                         (uint32_t)act_rec, &full[s], pol_a);
            };
            // Weights depend on nothing: fill the ring before waiting for the previous kernel.
            // (The in-CTA prologue borrows the last stage buffer as scratch until pro_bar.)
            // Only `inflight` K-steps are outstanding at a time: a K-step or two per SM already
            // saturate HBM, and everything beyond that just queues in the memory system, in
            // front of the small latency-critical loads (activation rows, tile pieces of other
            // CTAs) of the kernel that is finishing on the other SMs.
            // While the previous kernel is still closing its tiles the budget is smaller still
            // (inflight_pre): there is no hurry, the dependency wait comes next.
            const int D = p.inflight < NS - 1 ? p.inflight : NS - 1;  // D < NS: the stage asked about has not been re-armed since
            const int D0 = p.inflight_pre < D ? p.inflight_pre : D;
            bool stuck = false;
            auto landed = [&](int j) {  // K-step j of this CTA's walk is in shared memory
                if (j >= 0 && !stuck && !mbar_wait_bounded_relaxed(&full[j % NS], (uint32_t)((j / NS) & 1), p.wait_limit)) {
                    stuck = true;
                    note_timeout(p, ERRW_PRODUCER_TIMEOUT, 1);
                }
            };
            // (the in-CTA prologue of a Q4_K consumer uses the last stage as scratch for its exact block sums)
            const bool scratch = p.pro == PRO_QUANT && p.prep.need_sum;
            int ring0 = scratch ? NS - 1 : NS;
            const int pre = n_total < ring0 ? n_total : ring0;
            for (int it = 0; it < pre; ++it) {
                // (a streamed stage completes only with its activation record, which cannot be
                // asked for yet: no metering there)
                if (!streaming) landed(it - D0);
                issue_weights(it);
            }
            // (The resident activations are fetched by the first consumer thread, which is not
            // held up by the metering above.)
            if (streaming) {
                if (p.pdl) pdl_wait();
                for (int it = 0; it < pre; ++it) issue_acts(it);
            }
            // the in-CTA prologue borrows the last stage until it is done
            if (scratch && !mbar_wait_bounded_relaxed(pro_bar, 0u, p.wait_limit)) note_timeout(p, ERRW_PRODUCER_TIMEOUT, 2);
            int it = pre;
            for (; it < n_total; ++it) {
                const int s = it % NS;
                const uint32_t ph = (uint32_t)((it / NS) & 1);
                if (stuck || !mbar_wait_bounded_relaxed(&empty[s], ph ^ 1u, p.wait_limit)) {
                    note_timeout(p, ERRW_PRODUCER_TIMEOUT, 3);
                    break;
                }
                landed(it - D);
                issue_weights(it);
                if (streaming) issue_acts(it);
            }
            // Every copy issued above lands before this lane leaves: wait (bounded)
            // for the stages still in flight so no bulk write outlives the CTA.
            const int pending = it < NS ? it : NS;
            for (int j = it - pending; j < it; ++j) (void)mbar_wait_bounded(&full[j % NS], (uint32_t)((j / NS) & 1), p.wait_limit);
            if (acts_copy) (void)mbar_wait_bounded(acts_bar, 0u, p.wait_limit);
        }
        return;
    }

    // Close one tile (or tile piece) that the consumers left in red: add the K-quarters; for a tile
    // shared with other CTAs publish the partial sum, or - in the CTA that holds the tile's last
    // units - collect the others' and add them in CTA order; run the epilogue.
    float *fin = reinterpret_cast<float *>(smem + MvSmem<M>::FIN_OFF);
    int *slot_tab = reinterpret_cast<int *>(smem + MvSmem<M>::SLOT_OFF);
    const int my_first_tile = (int)(order.u_begin / (uint32_t)p.KS);
    auto close_tile = [&](const Crew &cw, int t_cur, bool final_tile, const float *rope_pre) {
            // Two-level activations: the consumers merged the digit pairs, everything sits in the
            // even rows; from here on the tile has one row per token.
            const int R = p.two_level ? M / 2 : M;
            const int RN = R * TILE_ROWS;
            for (int i = cw.t; i < RN; i += cw.n) {
                const int src = p.two_level ? 2 * (i / TILE_ROWS) * TILE_ROWS + i % TILE_ROWS : i;
                float v = red[src] + red[M * TILE_ROWS + src];
                if (KQ == 4) v += red[2 * M * TILE_ROWS + src] + red[3 * M * TILE_ROWS + src];
                fin[i] = v;
            }
            cw.sync();  // red and the flags have been read
            if (cw.t == 0) mbar_arrive(red_empty);
            const uint32_t ua = (uint32_t)t_cur * (uint32_t)p.KS, ub = ua + (uint32_t)p.KS - 1;
            const int c_first = (int)(((ua + 1) * G - 1) / U), c_last = (int)(((ub + 1) * G - 1) / U);
            if (c_first != c_last && (int)blockIdx.x != c_last) {
                // a piece of a tile that a later CTA closes: publish and move on
                unsigned long long *slot =
                    p.partials + ((size_t)blockIdx.x * 2 + (my_first_tile == t_cur ? 0 : 1)) * (MAX_M_EFF * TILE_ROWS);
                for (int i = cw.t; i < RN; i += cw.n) part_store(&slot[i], fin[i]);
            } else {
                // EPI_ADD: the residual is known since the dependency resolved; fetch it now so
                // that its round trip overlaps the wait for the other pieces
                float pre[EPI_PRE];
                const bool use_pre = p.epi == EPI_ADD && RN <= EPI_PRE * cw.n;
                if (use_pre) {
#pragma unroll
                    for (int j = 0; j < EPI_PRE; ++j) {
                        const int i = cw.t + j * cw.n;
                        const int m = i / TILE_ROWS, row = t_cur * TILE_ROWS + i % TILE_ROWS;
                        pre[j] = (i < RN && row < p.n_out) ? p.resid[(size_t)m * p.ldr + row] : 0.0f;
                    }
                }
                // likewise the weight of the next norm for the first block this warp will quantise
                float gam_pre = 0.0f;
                if (p.epi == EPI_ADD && p.nq_gamma) {
                    const int w = cw.t >> 5;
                    const int row = t_cur * TILE_ROWS + 32 * (w & 3) + (cw.t & 31);
                    if (w < R * 4 && row < p.n_out) gam_pre = p.nq_gamma[row];
                }
                if (c_first != c_last) {
                    // This CTA holds the last units of the tile: it adds the pieces of CTAs
                    // c_first .. c_last-1 (lower block indices, so they were scheduled no later
                    // than this one) in CTA order, then its own.  Where each left its piece:
                    // head piece -> slot 0, else slot 1.
                    const int nparts = c_last - c_first;
                    for (int k = cw.t; k < nparts; k += cw.n) {
                        const int c = c_first + k;
                        const int cf = (int)(((uint32_t)c * U / G) / (uint32_t)p.KS);
                        slot_tab[k] = (c * 2 + (cf == t_cur ? 0 : 1)) * (MAX_M_EFF * TILE_ROWS);
                    }
                    cw.sync();
                    const long long t_wait = clock64();
                    bool gave_up = false;
                    for (int i = cw.t; i < RN; i += 2 * cw.n) {
                        // two elements x eight pieces per round trip; poll until every tag is there (bounded)
                        const int i2 = i + cw.n;
                        const bool two = i2 < RN;
                        float v = 0.0f, v2 = 0.0f;
                        for (int k0 = 0; k0 < nparts; k0 += 8) {
                            unsigned long long w[8], w2[8];
                            for (;;) {
                                bool all = true;
#pragma unroll
                                for (int j = 0; j < 8; ++j) {
                                    const bool on = k0 + j < nparts;
                                    w[j] = on ? part_load(p.partials + slot_tab[k0 + j] + i) : PART_VALID;
                                    w2[j] = (on && two) ? part_load(p.partials + slot_tab[k0 + j] + i2) : PART_VALID;
                                    all = all && (w[j] & w2[j] & PART_VALID) != 0;
                                }
                                if (all || gave_up) break;
                                if (clock64() - t_wait > p.wait_limit) gave_up = true;
                            }
#pragma unroll
                            for (int j = 0; j < 8; ++j)
                                if (k0 + j < nparts) {
                                    v += __uint_as_float((uint32_t)w[j]);
                                    part_clear(p.partials + slot_tab[k0 + j] + i);
                                    if (two) {
                                        v2 += __uint_as_float((uint32_t)w2[j]);
                                        part_clear(p.partials + slot_tab[k0 + j] + i2);
                                    }
                                }
                        }
                        fin[i] = v + fin[i];
                        if (two) fin[i2] = v2 + fin[i2];
                    }
                    if (gave_up) note_timeout(p, ERRW_FINISHER_TIMEOUT, 5);
                    cw.sync();
                }
                if (tl && cw.t == 0 && final_tile && (p.pro != PRO_QUANT || p.tl_alt)) tl[7] = globaltimer_ns();  // pieces added
                epilogue_tile<M>(p, cw, t_cur, fin, use_pre ? pre : nullptr, rope_pre, gam_pre);
            }
    };

    if (warp > N_CONSUMER_WARPS) {
        // ------------------------------------------------------- finishers
        // Take each tile (or tile piece) the consumers leave in red, and close it: add the
        // four K-quarters; for a tile shared with other CTAs publish the partial sum, count
        // arrivals, and if this CTA is the last to arrive add all pieces in CTA order; run
        // the epilogue.  None of this stalls the consumers, who are already on the next tile.
        const int ftid = tid - (N_CONSUMERS + 32);
        // The RoPE table comes from the host, not from the previous kernel: the sin/cos pairs
        // lane, lane+32 of the first token this warp rotates are fetched before any tile is due.
        float rope_pre[4] = {0.f, 0.f, 0.f, 0.f};
        const bool has_rope_pre = p.epi == EPI_QKV_ROPE && (p.half == 32 || p.half == 64) && (ftid >> 5) < p.m_out;
        if (has_rope_pre) {
            const float *tab = p.rope + (size_t)(ftid >> 5) * p.half * 2;
            const int l = ftid & 31;
            rope_pre[0] = tab[2 * l];
            rope_pre[1] = tab[2 * l + 1];
            if (l + 32 < p.half) {
                rope_pre[2] = tab[2 * (l + 32)];
                rope_pre[3] = tab[2 * (l + 32) + 1];
            }
        }
        for (uint32_t n = 0;; ++n) {
            // one thread waits (bounded) and tells the others, so all of them leave together
            if (ftid == 0) {
                const bool ok = mbar_wait_bounded(red_full, n & 1u, p.wait_limit);
                if (!ok) note_timeout(p, ERRW_CONSUMER_TIMEOUT, 6);
                s_flags[2] = ok ? 1 : 0;
            }
            finisher_bar();
            // (after an expired wait the error word is set and the walk goes on: every wait in
            // this kernel is bounded, and leaving here would strand the consumers at the barrier
            // they share with the finishers for the last tile)
            const int t_cur = s_flags[0];
            const bool final_tile = s_flags[1] != 0;
            Crew cw{ftid, final_tile ? N_CREW_ALL : N_FINISHERS, final_tile ? 3 : 2};
            if (final_tile) cw.sync();  // the consumers join for the CTA's last tile
            close_tile(cw, t_cur, final_tile, has_rope_pre ? rope_pre : nullptr);
            if (final_tile) break;
            finisher_bar();  // fin, the slot table and the flags are reused by the next tile
        }
        if (tl && ftid == 0) tl[5] = globaltimer_ns();  // the last tile done
        return;
    }

    // ---------------------------------------------------------- consumers
    // Warp = (row group of 32 rows, quarter of the K-step).  Lane = 4*lg + lt: fragment rows
    // lg, lg+8 of each 16-row half, activation rows (tokens) 2*lt, 2*lt+1 of each group of 8.
    const int rg = warp & 3;
    const int kq = warp >> 2;
    const int lg = lane >> 2, lt = lane & 3;
    constexpr int NG = (M + 7) / 8;   // groups of 8 activation rows
    constexpr int MP = (M + 1) & ~1;  // row stride of the d / sum arrays
    float acc[2][NG][4];              // [16-row half][group][rows g,g / g+8,g+8 x tokens 2t,2t+1]
#pragma unroll
    for (int h = 0; h < 2; ++h)
#pragma unroll
        for (int j = 0; j < NG; ++j)
#pragma unroll
            for (int i = 0; i < 4; ++i) acc[h][j][i] = 0.0f;
    // chained columns: warp = (16-row half-group, parity of the K-steps it takes)
    const int hg = warp & 7, ug = warp >> 3;
    const int rgc = hg >> 1, h16c = hg & 1;
    const int my_blk = lg / MP2;                          // block of a chain whose activations this lane feeds (B column lg)
    const int my_tok = (lg % MP2) < M ? (lg % MP2) : M - 1;  // ... and which activation row (clamped)
    float cacc[4] = {0.0f, 0.0f, 0.0f, 0.0f};             // rows lg, lg, lg+8, lg+8 x result columns 2lt, 2lt+1
    bool aborted = false;

    float gam[PRO_CH];
    if (p.pro == PRO_QUANT) prologue_gamma(p, tid, gam);  // independent of the previous kernel
    // A launch whose row comes out of the exchange needs nothing else of the previous kernel:
    // the tagged words say when the row is complete, on this rank and on the others, so it does
    // not wait for that grid to drain (its peer stores take microseconds to be acknowledged).
    // The wait is made up for after the last unit, when it costs nothing.
    const bool late_dep = p.pro == PRO_QUANT && p.xin.index >= 0 && p.xin_late;
    if (p.pdl && !late_dep) pdl_wait();
    // first launch of a token in a tensor-parallel group: advance the token counter that numbers
    // the exchanges.  Single writer, after every launch of the previous token has completed
    // (this launch never defers its wait); later launches read it after this grid has completed.
    if (p.tok_inc && blockIdx.x == 0 && tid == 0) *xch_tok(p.xch.slots[p.xch.rank]) += 1u;
    if (tl && tid == 0) tl[2] = globaltimer_ns();  // dependency satisfied
    if (tid == 0 && acts_copy) {
        // the activations, as soon as they exist
        const uint64_t pol_a = l2_policy_evict_last();
        const uint32_t bytes = (uint32_t)(p.KS * act_rec);
        mbar_arrive_expect_tx(acts_bar, bytes);
        for (uint32_t o = 0; o < bytes; o += 32768u)
            bulk_g2s(res + o, p.act.base + o, min(32768u, bytes - o), acts_bar, pol_a);
    }
    float4 xr[PRO_J];
#pragma unroll
    for (int j = 0; j < PRO_J; ++j) {
        const int e = 4 * tid + PRO_CHUNK * j;
        xr[j] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (p.pro == PRO_QUANT && p.xin.index < 0 && e < p.prep.n) xr[j] = __ldcg(reinterpret_cast<const float4 *>(p.prep.x + e));
    }
    float *s_scale = red;  // [m_out] row scales of the block below; red is free until the first tile closes
    if (p.pro == PRO_LOAD && p.norm_sumsq) {
        // Records quantised before the row-wide RMSNorm scale was known: finish them.  Warp w
        // adds the per-block sums of squares of token w (fixed order), ops::rmsnorm_into's
        // f64 1/sqrt(mean + eps) (ops/norm.rs:193-198); below, every block scale and block sum
        // of that token's rows is multiplied by it.
        for (int tok = warp; tok < p.m_out; tok += N_CONSUMER_WARPS) {
            const double ss = sumsq_total(p.norm_sumsq + (size_t)tok * p.norm_blocks, p.norm_blocks, lane);
            if (lane == 0) s_scale[tok] = (float)(1.0 / sqrt(ss / (double)(p.norm_blocks * 32) + (double)p.norm_eps));
        }
    }
    // the row's sum of squares, when its producer left the per-block sums: the loads fly
    // while the row itself is on its way
    double ssq_in = 0.0;
    if (p.pro == PRO_QUANT && p.prep.gamma && p.prep.sumsq) ssq_in = sumsq_total(p.prep.sumsq, p.prep.n >> 5, lane);
    if (acts_copy && !mbar_wait_bounded(acts_bar, 0u, p.wait_limit)) {
        aborted = true;
        if (lane == 0) note_timeout(p, ERRW_CONSUMER_TIMEOUT, 8);
    }
    if (p.pro == PRO_LOAD && p.norm_sumsq) {
        consumer_bar();
        const int kt_r = p.act.kt(), mp_r = p.act.mp(), qb_r = p.act.q_bytes();
        const int per_rec = kt_r * mp_r;
        for (int i = tid; i < p.KS * per_rec; i += N_CONSUMERS) {
            const int ksr = i / per_rec, e = i - ksr * per_rec;
            const int row = e % mp_r;
            if (row < M) {
                float *d = reinterpret_cast<float *>(res + (size_t)ksr * act_rec + qb_r);
                const float sc = s_scale[p.two_level ? row >> 1 : row];
                d[e] = __fmul_rn(d[e], sc);
                d[per_rec + e] = __fmul_rn(d[per_rec + e], sc);
            }
        }
        consumer_bar();
    }
    if (p.pro == PRO_QUANT) {
        if (tl && tid == 0) tl[4] = globaltimer_ns();  // raw row requested
        prologue_quant<M>(p, res, reinterpret_cast<float *>(stages + (size_t)(NS - 1) * stage_bytes), red, tid, gam, ssq_in, xr);
        // generic-proxy accesses to the scratch are done; the bulk-copy engine may overwrite it
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        __syncwarp();
        if (lane == 0) mbar_arrive(pro_bar);
    }
    if (tl && tid == 0) tl[6] = globaltimer_ns();  // activations ready
    if (p.act_dump && blockIdx.x == 0 && p.pro != PRO_STREAM) {
        // parity instrumentation: the records exactly as the mma loop is about to read them
        const uint32_t *src = reinterpret_cast<const uint32_t *>(res);
        uint32_t *dst = reinterpret_cast<uint32_t *>(p.act_dump);
        for (int i = tid; i < (p.KS * act_rec) >> 2; i += N_CONSUMERS) dst[i] = src[i];
    }

    // (tile, K-step) of the walk, kept incrementally: the order has one jump
    // (after the tail piece) and otherwise advances by one unit.
    int t, ks;
    {
        const uint32_t u0 = order.at(0);
        t = (int)(u0 / p.KS);
        ks = (int)(u0 % p.KS);
    }
    int s = 0;
    uint32_t ph = 0;
    uint32_t n_handoff = 0;  // tiles (or tile pieces) passed to the finishers so far
    int t_last = 0;          // the tile of the last hand-off
    for (int it = 0; it < n_total; ++it) {
        // where the next unit lies (decides whether this one closes its tile)
        int t_next = t, ks_next = ks + 1;
        if (it + 1 == order.len_tail) {
            t_next = (int)(order.u_begin / p.KS);
            ks_next = (int)(order.u_begin % p.KS);
        } else if (ks_next == p.KS) {
            ks_next = 0;
            t_next = t + 1;
        }
        const bool mine = !CH || (it & 1) == ug;
        if (mine && !aborted && !mbar_wait_bounded(&full[s], ph, p.wait_limit)) {
            aborted = true;
            if (lane == 0) note_timeout(p, ERRW_CONSUMER_TIMEOUT, 9);
        }
        if (tl && mine && lane == 0 && (warp & 7) == 0) {
            if (it == 0 && !p.tl_alt) tl[1] = globaltimer_ns();   // first unit landed
            if (it + 1 == n_total) tl[3] = globaltimer_ns();  // last unit landed
        }
        if (mine && !aborted) {
            const uint8_t *sw = stages + (size_t)s * stage_bytes;
            const uint8_t *sa = streaming ? sw + stage_w_bytes(TY) : res + (size_t)ks * act_rec;
            const int kb = min(kt, p.nb - ks * kt);
            const float *ad = reinterpret_cast<const float *>(sa + M * p.act.ke);  // d[block][MP], then sum[block][MP]
            const float *as = ad + kt * MP;
            // parity instrumentation: the int32 block dots of fragment (h16, group j), global block gb
            auto dump4 = [&](const int (&d)[4], int h16, int j, int gb) {
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const int row = t * TILE_ROWS + rg * 32 + h16 * 16 + lg + (i >> 1) * 8;
                    const int tok = 8 * j + 2 * lt + (i & 1);
                    if (tok < M && row < p.n_out) p.dump[((size_t)tok * p.n_out + row) * p.nb + gb] = d[i];
                }
            };
            if constexpr (CH) {
                // Chained columns.  One mma gives 16 rows x 8 columns, and with a single activation
                // row seven columns would repeat the first.  Instead a chain of BPC mmas runs over BPC
                // consecutive blocks into ONE accumulator, block i of the chain feeding only columns
                // i*MP2 .. i*MP2+MP2-1 of the B operand (zero elsewhere): column c of the result is the
                // block dot of block c / MP2 with activation row c % MP2.  Every lane then holds four
                // distinct dots (rows lg, lg+8 x columns 2lt, 2lt+1) and the fp32 scaling is done once
                // per dot instead of eight times.
                auto dumpc = [&](const int (&d)[4], int gb0) {  // gb0: global index of the chain's first block
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const int c = 2 * lt + (i & 1);
                        const int row = t * TILE_ROWS + hg * 16 + lg + (i >> 1) * 8;
                        const int tok = c % MP2, gb = gb0 + c / MP2;
                        if (tok < M && gb < p.nb && row < p.n_out) p.dump[((size_t)tok * p.n_out + row) * p.nb + gb] = d[i];
                    }
                };
                if (ty_b32(TY)) {
                    const uint8_t *ws = sw + b32_scale_off(TY, kb) + (rgc * 8 + lg) * 8 + h16c * 4;  // + b*256: scales of rows lg, lg+8
#pragma unroll
                    for (int cb = 0; cb < Q8_KT; cb += BPC) {
                        if (cb < kb) {
                            const int xblk = cb + my_blk;
                            uint32_t xb0 = 0u, xb1 = 0u;
                            if (xblk < kb) {
                                const uint8_t *xb = sa + xblk * (32 * M) + my_tok * 16 + 4 * lt;
                                xb0 = *reinterpret_cast<const uint32_t *>(xb);
                                xb1 = *reinterpret_cast<const uint32_t *>(xb + 16 * M);
                            }
                            int d[4] = {0, 0, 0, 0}, e[4] = {0, 0, 0, 0};  // two chains, so consecutive mmas do not wait on each other
#pragma unroll
                            for (int i = 0; i < BPC; ++i) {
                                if (cb + i < kb) {
                                    const uint4 a = b32_frag<TY>(sw, kb, cb + i, rgc, h16c, lane);
                                    const uint32_t b0 = my_blk == i ? xb0 : 0u, b1 = my_blk == i ? xb1 : 0u;
                                    if (i & 1) mma_block_s8_acc(e, a, b0, b1);
                                    else mma_block_s8_acc(d, a, b0, b1);
                                }
                            }
                            if (BPC > 1) {
#pragma unroll
                                for (int i = 0; i < 4; ++i) d[i] += e[i];
                            }
                            if (TY == TY_Q5_0) {
                                // the codes went in as 0..31: take 16 x the sum of the column's activation codes off
                                int sd[4] = {0, 0, 0, 0};
                                mma_block_s8_acc(sd, make_uint4(0x10101010u, 0x10101010u, 0x10101010u, 0x10101010u), xb0, xb1);
#pragma unroll
                                for (int i = 0; i < 4; ++i) d[i] -= sd[i];
                            }
                            if (MP2 > 1 && p.two_level) {
                                // columns 2lt, 2lt+1 are the two digits of one token of one block, d2 = d1 / 256:
                                // merge them as integers, scale once
                                const int c = 2 * lt;
                                const int b = cb + c / MP2, tok = c % MP2 + 1;
                                if (b < kb) {
                                    const __half2 sc = *reinterpret_cast<const __half2 *>(ws + b * 256);
                                    const float dx = ad[b * MP + tok];
                                    cacc[0] = fmaf(__fmul_rn(__low2float(sc), dx), (float)((d[0] << 8) + d[1]), cacc[0]);
                                    cacc[2] = fmaf(__fmul_rn(__high2float(sc), dx), (float)((d[2] << 8) + d[3]), cacc[2]);
                                }
                            } else {
#pragma unroll
                                for (int i = 0; i < 4; ++i) {
                                    const int c = 2 * lt + (i & 1);
                                    const int b = cb + c / MP2;
                                    const int tok = (c % MP2) < M ? (c % MP2) : M - 1;
                                    if (b < kb) {
                                        const __half2 sc = *reinterpret_cast<const __half2 *>(ws + b * 256);
                                        const float dw = (i >> 1) ? __high2float(sc) : __low2float(sc);
                                        cacc[i] = fmaf(__fmul_rn(dw, ad[b * MP + tok]), (float)d[i], cacc[i]);
                                    }
                                }
                            }
                            if (DUMP) dumpc(d, ks * Q8_KT + cb);
                        }
                    }
                } else if (ty_k6(TY)) {
                    // One super-block per K-step.  Sub-block scales cover 16 elements, so a block's
                    // dot is two 16-deep mmas (one per half of the block, each in its own chain) and
                    // sc0*dot0 + sc1*dot1 is formed in integers: exactly what the reference forms in
                    // f32 (q8_acts.rs:338-342; |value| < 2^24).
                    // Q2_K adds its min term: - dmin * dx * (mn0 * sum0 + mn1 * sum1) over the sums of the
                    // activation codes of the two halves (q8_acts.rs:160-168), which the -32 correction has already.
                    constexpr bool K2 = TY == TY_Q2_K;
                    const uint8_t *base = sw + rgc * k6_sb_rg(TY);
                    // the 16 sub-block scales of row lg, then of row lg+8: a lane reads the two bytes of the block
                    // whose dot it holds (a 16-bit load at a lane-dependent offset, no byte selection in registers)
                    const uint8_t *sc_rows = base + 6144 + (lg * 4 + 2 * h16c) * 16;
                    const uint8_t *mn_rows = base + Q6_SB_RG + (lg * 4 + 2 * h16c) * 16;  // Q2_K: the mins, same layout
                    const __half2 dd = *reinterpret_cast<const __half2 *>(base + 6656 + (lg * 4 + 2 * h16c) * 2);
                    const float dwl = __low2float(dd), dwh = __high2float(dd);
                    float dml = 0.0f, dmh = 0.0f;
                    if (K2) {
                        const __half2 dm = *reinterpret_cast<const __half2 *>(base + Q6_SB_RG + 512 + (lg * 4 + 2 * h16c) * 2);
                        dml = __low2float(dm);
                        dmh = __high2float(dm);
                    }
#pragma unroll
                    for (int ch = 0; ch < 8 / BPC; ++ch) {
                        const int xs = ch * BPC + my_blk;
                        const uint8_t *xb = sa + xs * (32 * M) + my_tok * 16 + 4 * lt;
                        const uint32_t xb0 = *reinterpret_cast<const uint32_t *>(xb);
                        const uint32_t xb1 = *reinterpret_cast<const uint32_t *>(xb + 16 * M);
                        int d[4] = {0, 0, 0, 0}, e[4] = {0, 0, 0, 0};
                        // column c of these two: the sum of the activation codes of the chain's block c / MP2
                        // (row c % MP2) over its first and second 16 elements, times 32
                        int sd[4] = {0, 0, 0, 0}, se[4] = {0, 0, 0, 0};
                        mma_half_s8_acc(sd, 0x20202020u, 0x20202020u, xb0);
                        mma_half_s8_acc(se, 0x20202020u, 0x20202020u, xb1);
#pragma unroll
                        for (int i = 0; i < BPC; ++i) {
                            const int blk = ch * BPC + i, half = blk >> 2, qi = blk & 3;
                            const uint4 ql = *reinterpret_cast<const uint4 *>(base + (((half * 2 + (qi & 1)) * 2 + h16c) * 32 + lane) * 16);
                            const uint4 qh = *reinterpret_cast<const uint4 *>(base + 4096 + ((half * 2 + h16c) * 32 + lane) * 16);
                            const uint4 a = q6_k_unpack(ql, qh, qi);
                            mma_half_s8_acc(d, a.x, a.y, my_blk == i ? xb0 : 0u);
                            mma_half_s8_acc(e, a.z, a.w, my_blk == i ? xb1 : 0u);
                        }
                        int I[4];
                        int J[4] = {0, 0, 0, 0};  // Q2_K: mn0 * sum0 + mn1 * sum1 (sd, se are 32 x the sums)
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            const int b = ch * BPC + (2 * lt + (i & 1)) / MP2;
                            const uint32_t w = *reinterpret_cast<const unsigned short *>(sc_rows + (i >> 1) * 16 + 2 * b);
                            I[i] = ((int)(w << 24) >> 24) * (d[i] - sd[i]) + ((int)(w << 16) >> 24) * (e[i] - se[i]);
                            if (K2) {
                                const uint32_t wm = *reinterpret_cast<const unsigned short *>(mn_rows + (i >> 1) * 16 + 2 * b);
                                J[i] = (int)(wm & 0xffu) * (sd[i] >> 5) + (int)(wm >> 8) * (se[i] >> 5);
                            }
                        }
                        if (MP2 > 1 && p.two_level) {
                            // columns 2lt, 2lt+1 are the two digits of one token of one block, d2 = d1 / 256
                            const int c = 2 * lt;
                            const int b = ch * BPC + c / MP2, tok = c % MP2 + 1;
                            const float dx = ad[b * MP + tok];
                            cacc[0] = fmaf(__fmul_rn(dwl, dx), (float)(((long long)I[0] << 8) + I[1]), cacc[0]);
                            cacc[2] = fmaf(__fmul_rn(dwh, dx), (float)(((long long)I[2] << 8) + I[3]), cacc[2]);
                            if (K2) {
                                cacc[0] = fmaf(-__fmul_rn(dml, dx), (float)((J[0] << 8) + J[1]), cacc[0]);
                                cacc[2] = fmaf(-__fmul_rn(dmh, dx), (float)((J[2] << 8) + J[3]), cacc[2]);
                            }
                        } else {
#pragma unroll
                            for (int i = 0; i < 4; ++i) {
                                const int c = 2 * lt + (i & 1);
                                const int b = ch * BPC + c / MP2;
                                const int tok = (c % MP2) < M ? (c % MP2) : M - 1;
                                // total += d * acts.d[blk] * (sc0*dot0 + sc1*dot1)  (q8_acts.rs:342)
                                cacc[i] = fmaf(__fmul_rn((i >> 1) ? dwh : dwl, ad[b * MP + tok]), (float)I[i], cacc[i]);
                                if (K2) cacc[i] = fmaf(-__fmul_rn((i >> 1) ? dmh : dml, ad[b * MP + tok]), (float)J[i], cacc[i]);
                            }
                        }
                        if (DUMP) dumpc(I, ks * 8 + ch * BPC);
                    }
                } else {
#pragma unroll
                    for (int sbi = 0; sbi < Q4_KT_SB; ++sbi) {
                        if (sbi * 8 < kb) {
                            const uint8_t *base = sw + sbi * K45_UNIT + rgc * K45_RG;
                            const uint8_t *hdr = base + K45_HDR;
                            // Q5_K: the fifth bits of this 16-row half, all eight sub-blocks (sub-block j: bit j of every byte)
                            uint4 qh5 = make_uint4(0u, 0u, 0u, 0u);
                            if (K5) qh5 = *reinterpret_cast<const uint4 *>(base + 4096 + (h16c * 32 + lane) * 16);
                            // {d, dmin} of rows lg, lg+8 of this half
                            const uint2 dd = *reinterpret_cast<const uint2 *>(hdr + (lg * 4 + 2 * h16c) * 4);
                            float U[4] = {0.0f, 0.0f, 0.0f, 0.0f}, V[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
                            for (int ch = 0; ch < 8 / BPC; ++ch) {  // sub-blocks ch*BPC .. ch*BPC+BPC-1 of the super-block
                                const int xs = sbi * 8 + ch * BPC + my_blk;
                                const uint8_t *xb = sa + xs * (32 * M) + my_tok * 16 + 4 * lt;
                                const uint32_t xb0 = *reinterpret_cast<const uint32_t *>(xb);
                                const uint32_t xb1 = *reinterpret_cast<const uint32_t *>(xb + 16 * M);
                                int d[4] = {0, 0, 0, 0}, e[4] = {0, 0, 0, 0};
#pragma unroll
                                for (int pi = 0; pi < BPC / 2; ++pi) {  // a byte holds sub-blocks 2*pr (low nibble), 2*pr+1 (high)
                                    const int pr = ch * (BPC / 2) + pi;
                                    const uint4 q = *reinterpret_cast<const uint4 *>(base + ((pr * 2 + h16c) * 32 + lane) * 16);
                                    uint4 lo = make_uint4(q.x & 0x0f0f0f0fu, q.y & 0x0f0f0f0fu, q.z & 0x0f0f0f0fu, q.w & 0x0f0f0f0fu);
                                    if constexpr (K5) {
                                        uint4 hi = make_uint4((q.x >> 4) & 0x0f0f0f0fu, (q.y >> 4) & 0x0f0f0f0fu,
                                                              (q.z >> 4) & 0x0f0f0f0fu, (q.w >> 4) & 0x0f0f0f0fu);
                                        q5_k_high(lo, hi, qh5, pr);
                                        mma_block_s8_acc(d, lo, my_blk == 2 * pi ? xb0 : 0u, my_blk == 2 * pi ? xb1 : 0u);
                                        mma_block_s8_acc(e, hi, my_blk == 2 * pi + 1 ? xb0 : 0u, my_blk == 2 * pi + 1 ? xb1 : 0u);
                                    } else {
                                        // Q4_K: the high nibbles stay where they are and go in as unsigned bytes 16 * q; the
                                        // chain's sum is 16 x the dots, exactly, and is shifted back once (below)
                                        const uint4 hi16 = make_uint4(q.x & 0xf0f0f0f0u, q.y & 0xf0f0f0f0u, q.z & 0xf0f0f0f0u, q.w & 0xf0f0f0f0u);
                                        mma_block_s8_acc(d, lo, my_blk == 2 * pi ? xb0 : 0u, my_blk == 2 * pi ? xb1 : 0u);
                                        mma_block_u8s8_acc(e, hi16, my_blk == 2 * pi + 1 ? xb0 : 0u, my_blk == 2 * pi + 1 ? xb1 : 0u);
                                    }
                                }
#pragma unroll
                                for (int i = 0; i < 4; ++i) d[i] += K5 ? e[i] : (e[i] >> 4);
#pragma unroll
                                for (int i = 0; i < 4; ++i) {
                                    const int c = 2 * lt + (i & 1);
                                    const int sbk = ch * BPC + c / MP2;  // sub-block of the super-block
                                    const int tok = (c % MP2) < M ? (c % MP2) : M - 1;
                                    // 6-bit scale and min of row lg (i < 2) or lg+8 (split out at repack, four sub-blocks per
                                    // word): one byte load each at the lane's own offset, nothing selected in registers
                                    const int hoff = ((lg * 2 + (sbk >> 2)) * 4 + 2 * h16c + (i >> 1)) * 4 + (sbk & 3);
                                    const float sc = (float)hdr[128 + hoff];
                                    const float mn = (float)hdr[384 + hoff];
                                    const int b = sbi * 8 + sbk;
                                    if (MP2 > 1 && p.two_level) {
                                        // digits merged as integers (d2 = d1 / 256); odd columns carry nothing
                                        if (!(i & 1)) {
                                            U[i] = fmaf(sc, __fmul_rn((float)((d[i] << 8) + d[i + 1]), ad[b * MP + tok + 1]), U[i]);
                                            V[i] = fmaf(mn, as[b * MP + tok], V[i]);
                                        }
                                    } else {
                                        U[i] = fmaf(sc, __fmul_rn((float)d[i], ad[b * MP + tok]), U[i]);
                                        V[i] = fmaf(mn, as[b * MP + tok], V[i]);
                                    }
                                }
                                if (DUMP) dumpc(d, ks * 16 + sbi * 8 + ch * BPC);
                            }
                            // total += d * sum(sc*dot*dx) - dmin * sum(mn*sum)  (q8_acts.rs:296-297, regrouped per super-block)
#pragma unroll
                            for (int i = 0; i < 4; ++i) {
                                const uint32_t w = (i >> 1) ? dd.y : dd.x;
                                const float dq = __half2float(__ushort_as_half((unsigned short)(w & 0xffffu)));
                                const float dmin = __half2float(__ushort_as_half((unsigned short)(w >> 16)));
                                cacc[i] += __fsub_rn(__fmul_rn(dq, U[i]), __fmul_rn(dmin, V[i]));
                            }
                        }
                    }
                }
            } else
            if (ty_b32(TY)) {
                // this warp: blocks kq, kq+4 of the K-step.  Activation rows past M are clamped to
                // row M-1: their results are computed but never stored, which keeps predicates
                // out of the loop.
                const uint8_t *ws = sw + b32_scale_off(TY, kb) + (rg * 8 + lg) * 8;   // + b*256
                auto block = [&](int b) {
                    const uint4 a0 = b32_frag<TY>(sw, kb, b, rg, 0, lane);
                    const uint4 a1 = b32_frag<TY>(sw, kb, b, rg, 1, lane);
                    const uint2 sc = *reinterpret_cast<const uint2 *>(ws + b * 256);
                    const __half2 s01 = *reinterpret_cast<const __half2 *>(&sc.x);
                    const __half2 s23 = *reinterpret_cast<const __half2 *>(&sc.y);
                    const float2 f01 = __half22float2(s01), f23 = __half22float2(s23);
                    const uint8_t *xb = sa + b * (32 * M);
                    const float *xd = ad + b * MP;
#pragma unroll
                    for (int j = 0; j < NG; ++j) {
                        const int tb = min(8 * j + lg, M - 1);      // B-fragment row
                        const int t0 = min(8 * j + 2 * lt, M - 1);  // result columns
                        const int t1 = min(8 * j + 2 * lt + 1, M - 1);
                        const uint32_t b0 = *reinterpret_cast<const uint32_t *>(xb + tb * 16 + 4 * lt);
                        const uint32_t b1 = *reinterpret_cast<const uint32_t *>(xb + 16 * M + tb * 16 + 4 * lt);
                        int d0[4], d1[4];
                        mma_block_s8(d0, a0, b0, b1);
                        mma_block_s8(d1, a1, b0, b1);
                        if (TY == TY_Q5_0) {
                            // the codes went in as 0..31: take 16 x the sum of the column's activation codes off
                            int sd[4];
                            mma_block_s8(sd, make_uint4(0x10101010u, 0x10101010u, 0x10101010u, 0x10101010u), b0, b1);
#pragma unroll
                            for (int i = 0; i < 4; ++i) {
                                d0[i] -= sd[i];
                                d1[i] -= sd[i];
                            }
                        }
                        const float dx0 = xd[t0];
                        // total += d_w * d_x * dot (q8_acts.rs:93), per (row, token)
                        if (M > 8 || (M > 1 && p.two_level)) {
                            // columns 2lt, 2lt+1 are the two digits of one token, d2 = d1 / 256:
                            // merge them as integers, scale once
                            const float dx1 = xd[t1];
                            acc[0][j][0] = fmaf(__fmul_rn(f01.x, dx1), (float)((d0[0] << 8) + d0[1]), acc[0][j][0]);
                            acc[0][j][2] = fmaf(__fmul_rn(f01.y, dx1), (float)((d0[2] << 8) + d0[3]), acc[0][j][2]);
                            acc[1][j][0] = fmaf(__fmul_rn(f23.x, dx1), (float)((d1[0] << 8) + d1[1]), acc[1][j][0]);
                            acc[1][j][2] = fmaf(__fmul_rn(f23.y, dx1), (float)((d1[2] << 8) + d1[3]), acc[1][j][2]);
                        } else if constexpr (M <= 8) {
                            acc[0][j][0] = fmaf(__fmul_rn(f01.x, dx0), (float)d0[0], acc[0][j][0]);
                            acc[0][j][2] = fmaf(__fmul_rn(f01.y, dx0), (float)d0[2], acc[0][j][2]);
                            acc[1][j][0] = fmaf(__fmul_rn(f23.x, dx0), (float)d1[0], acc[1][j][0]);
                            acc[1][j][2] = fmaf(__fmul_rn(f23.y, dx0), (float)d1[2], acc[1][j][2]);
                            if (M > 1) {  // a single activation row never has an odd column
                                const float dx1 = xd[t1];
                                acc[0][j][1] = fmaf(__fmul_rn(f01.x, dx1), (float)d0[1], acc[0][j][1]);
                                acc[0][j][3] = fmaf(__fmul_rn(f01.y, dx1), (float)d0[3], acc[0][j][3]);
                                acc[1][j][1] = fmaf(__fmul_rn(f23.x, dx1), (float)d1[1], acc[1][j][1]);
                                acc[1][j][3] = fmaf(__fmul_rn(f23.y, dx1), (float)d1[3], acc[1][j][3]);
                            }
                        }
                        if (DUMP) {
                            dump4(d0, 0, j, ks * Q8_KT + b);
                            dump4(d1, 1, j, ks * Q8_KT + b);
                        }
                    }
                };
                if (kb == Q8_KT) {
                    block(kq);
                    block(kq + K_SPLIT);
                } else {
                    for (int b = kq; b < kb; b += K_SPLIT) block(b);
                }
            } else if (ty_k6(TY)) {
                // this warp: quarter kq of both halves of the super-block (blocks kq and kq + 4)
                constexpr bool K2 = TY == TY_Q2_K;
                const uint8_t *base = sw + rg * k6_sb_rg(TY);
                const uint2 ddw = *reinterpret_cast<const uint2 *>(base + 6656 + lg * 8);  // d of rows lg, lg+8, lg+16, lg+24
                const float2 f01 = __half22float2(*reinterpret_cast<const __half2 *>(&ddw.x));
                const float2 f23 = __half22float2(*reinterpret_cast<const __half2 *>(&ddw.y));
                const float dwr[4] = {f01.x, f01.y, f23.x, f23.y};
                float dmr[4] = {0.0f, 0.0f, 0.0f, 0.0f};  // Q2_K: dmin of the same rows
                if (K2) {
                    const uint2 dmw = *reinterpret_cast<const uint2 *>(base + Q6_SB_RG + 512 + lg * 8);
                    const float2 g01 = __half22float2(*reinterpret_cast<const __half2 *>(&dmw.x));
                    const float2 g23 = __half22float2(*reinterpret_cast<const __half2 *>(&dmw.y));
                    dmr[0] = g01.x; dmr[1] = g01.y; dmr[2] = g23.x; dmr[3] = g23.y;
                }
#pragma unroll
                for (int half = 0; half < 2; ++half) {
                    const int b = half * 4 + kq;
                    uint4 a[2];
#pragma unroll
                    for (int h = 0; h < 2; ++h) {
                        const uint4 ql = *reinterpret_cast<const uint4 *>(base + (((half * 2 + (kq & 1)) * 2 + h) * 32 + lane) * 16);
                        const uint4 qh = *reinterpret_cast<const uint4 *>(base + 4096 + ((half * 2 + h) * 32 + lane) * 16);
                        a[h] = q6_k_unpack(ql, qh, kq);
                    }
                    int s0[4], s1[4];  // the block's two sub-block scales for rows lg, lg+8, lg+16, lg+24
                    int m0[4] = {0, 0, 0, 0}, m1[4] = {0, 0, 0, 0};  // Q2_K: and its two sub-block mins
#pragma unroll
                    for (int r4 = 0; r4 < 4; ++r4) {
                        const uint32_t w = *reinterpret_cast<const unsigned short *>(base + 6144 + (lg * 4 + r4) * 16 + 2 * b);
                        s0[r4] = (int)(w << 24) >> 24;
                        s1[r4] = (int)(w << 16) >> 24;
                        if (K2) {
                            const uint32_t wm = *reinterpret_cast<const unsigned short *>(base + Q6_SB_RG + (lg * 4 + r4) * 16 + 2 * b);
                            m0[r4] = (int)(wm & 0xffu);
                            m1[r4] = (int)(wm >> 8);
                        }
                    }
                    const uint8_t *xb = sa + b * (32 * M);
                    const float *xd = ad + b * MP;
#pragma unroll
                    for (int j = 0; j < NG; ++j) {
                        // rows past M are clamped to row M-1: computed, never stored
                        const int tb = min(8 * j + lg, M - 1);
                        const int t0 = min(8 * j + 2 * lt, M - 1), t1 = min(8 * j + 2 * lt + 1, M - 1);
                        const uint32_t b0 = *reinterpret_cast<const uint32_t *>(xb + tb * 16 + 4 * lt);
                        const uint32_t b1 = *reinterpret_cast<const uint32_t *>(xb + 16 * M + tb * 16 + 4 * lt);
                        int I[2][4], J[2][4];
                        int sd[4] = {0, 0, 0, 0}, se[4] = {0, 0, 0, 0};  // 32 * the sums of the activation codes, per column
                        mma_half_s8_acc(sd, 0x20202020u, 0x20202020u, b0);
                        mma_half_s8_acc(se, 0x20202020u, 0x20202020u, b1);
#pragma unroll
                        for (int h = 0; h < 2; ++h) {
                            int d[4] = {0, 0, 0, 0}, e[4] = {0, 0, 0, 0};
                            mma_half_s8_acc(d, a[h].x, a[h].y, b0);
                            mma_half_s8_acc(e, a[h].z, a[h].w, b1);
#pragma unroll
                            for (int i = 0; i < 4; ++i) {
                                I[h][i] = s0[2 * h + (i >> 1)] * (d[i] - sd[i]) + s1[2 * h + (i >> 1)] * (e[i] - se[i]);
                                J[h][i] = K2 ? m0[2 * h + (i >> 1)] * (sd[i] >> 5) + m1[2 * h + (i >> 1)] * (se[i] >> 5) : 0;
                            }
                        }
                        const float dx0 = xd[t0], dx1 = xd[t1];
#pragma unroll
                        for (int h = 0; h < 2; ++h) {
                            if (M > 8 || (M > 1 && p.two_level)) {
                                // columns 2lt, 2lt+1 are the two digits of one token, d2 = d1 / 256
#pragma unroll
                                for (int i = 0; i < 4; i += 2) {
                                    acc[h][j][i] = fmaf(__fmul_rn(dwr[2 * h + (i >> 1)], dx1), (float)(((long long)I[h][i] << 8) + I[h][i + 1]),
                                                        acc[h][j][i]);
                                    if (K2)
                                        acc[h][j][i] = fmaf(-__fmul_rn(dmr[2 * h + (i >> 1)], dx1), (float)((J[h][i] << 8) + J[h][i + 1]), acc[h][j][i]);
                                }
                            } else if constexpr (M <= 8) {
#pragma unroll
                                for (int i = 0; i < 4; ++i) {
                                    if (M == 1 && (i & 1)) continue;  // a single activation row has no odd column
                                    acc[h][j][i] = fmaf(__fmul_rn(dwr[2 * h + (i >> 1)], (i & 1) ? dx1 : dx0), (float)I[h][i], acc[h][j][i]);
                                    if (K2)
                                        acc[h][j][i] = fmaf(-__fmul_rn(dmr[2 * h + (i >> 1)], (i & 1) ? dx1 : dx0), (float)J[h][i], acc[h][j][i]);
                                }
                            }
                        }
                        if (DUMP) {
                            dump4(I[0], 0, j, ks * 8 + b);
                            dump4(I[1], 1, j, ks * 8 + b);
                        }
                    }
                }
            } else {
                // this warp: super-block kq/2 of the K-step, sub-blocks 4*(kq&1) .. +3 (pairs 2*(kq&1), +1)
                const int sb = kq >> 1, jh = kq & 1;
                if (sb * 8 < kb) {
                    const uint8_t *base = sw + sb * K45_UNIT + rg * K45_RG;
                    const uint8_t *hdr = base + K45_HDR;
                    const uint4 dd = *reinterpret_cast<const uint4 *>(hdr + lg * 16);                   // {d, dmin} of 4 rows
                    const uint4 scw = *reinterpret_cast<const uint4 *>(hdr + 128 + (lg * 2 + jh) * 16);  // 4 scales x 4 rows
                    const uint4 mnw = *reinterpret_cast<const uint4 *>(hdr + 384 + (lg * 2 + jh) * 16);  // 4 mins x 4 rows
                    const uint32_t ddw[4] = {dd.x, dd.y, dd.z, dd.w};
                    const uint32_t scr[4] = {scw.x, scw.y, scw.z, scw.w};
                    const uint32_t mnr[4] = {mnw.x, mnw.y, mnw.z, mnw.w};
                    float U[2][NG][4], V[2][NG][4];  // sum_j sc_j * (dot_j * dx_j), sum_j mn_j * sum_j
#pragma unroll
                    for (int h = 0; h < 2; ++h)
#pragma unroll
                        for (int j = 0; j < NG; ++j)
#pragma unroll
                            for (int i = 0; i < 4; ++i) U[h][j][i] = V[h][j][i] = 0.0f;
#pragma unroll
                    for (int pi = 0; pi < 2; ++pi) {
                        const int pr = 2 * jh + pi;
                        uint4 lo[2], hi[2];
#pragma unroll
                        for (int h = 0; h < 2; ++h) {
                            const uint4 q = *reinterpret_cast<const uint4 *>(base + ((pr * 2 + h) * 32 + lane) * 16);
                            lo[h] = make_uint4(q.x & 0x0f0f0f0fu, q.y & 0x0f0f0f0fu, q.z & 0x0f0f0f0fu, q.w & 0x0f0f0f0fu);
                            hi[h] = make_uint4((q.x >> 4) & 0x0f0f0f0fu, (q.y >> 4) & 0x0f0f0f0fu, (q.z >> 4) & 0x0f0f0f0fu,
                                               (q.w >> 4) & 0x0f0f0f0fu);
                            if (K5) q5_k_high(lo[h], hi[h], *reinterpret_cast<const uint4 *>(base + 4096 + (h * 32 + lane) * 16), pr);
                        }
#pragma unroll
                        for (int nib = 0; nib < 2; ++nib) {
                            const int jj = 2 * pi + nib;         // sub-block within this warp's four
                            const int b = sb * 8 + 2 * pr + nib;  // activation block within the K-step
                            float scf[4], mnf[4];
#pragma unroll
                            for (int r4 = 0; r4 < 4; ++r4) {
                                scf[r4] = (float)((scr[r4] >> (8 * jj)) & 0xffu);
                                mnf[r4] = (float)((mnr[r4] >> (8 * jj)) & 0xffu);
                            }
                            const uint8_t *xb = sa + b * (32 * M);
#pragma unroll
                            for (int j = 0; j < NG; ++j) {
                                // rows past M are clamped to row M-1: computed, never stored
                                const int tb = min(8 * j + lg, M - 1);
                                const int t0 = min(8 * j + 2 * lt, M - 1), t1 = min(8 * j + 2 * lt + 1, M - 1);
                                const uint32_t b0 = *reinterpret_cast<const uint32_t *>(xb + tb * 16 + 4 * lt);
                                const uint32_t b1 = *reinterpret_cast<const uint32_t *>(xb + 16 * M + tb * 16 + 4 * lt);
                                int d0[4], d1[4];
                                mma_block_s8(d0, nib ? hi[0] : lo[0], b0, b1);
                                mma_block_s8(d1, nib ? hi[1] : lo[1], b0, b1);
                                const float dx0 = ad[b * MP + t0], dx1 = ad[b * MP + t1];
                                const float sx0 = as[b * MP + t0], sx1 = as[b * MP + t1];
                                // (more than 8 rows only ever are digit pairs: the other form is not compiled for them,
                                // which halves the live accumulators of the instantiations that used to spill)
                                if (M > 8 || (M > 1 && p.two_level)) {
                                    // digits merged as integers (d2 = d1 / 256); the min term rides on the first digit's row
#pragma unroll
                                    for (int i = 0; i < 4; i += 2) {
                                        U[0][j][i] = fmaf(scf[i >> 1], __fmul_rn((float)((d0[i] << 8) + d0[i + 1]), dx1), U[0][j][i]);
                                        U[1][j][i] = fmaf(scf[2 + (i >> 1)], __fmul_rn((float)((d1[i] << 8) + d1[i + 1]), dx1), U[1][j][i]);
                                        V[0][j][i] = fmaf(mnf[i >> 1], sx0, V[0][j][i]);
                                        V[1][j][i] = fmaf(mnf[2 + (i >> 1)], sx0, V[1][j][i]);
                                    }
                                } else if constexpr (M <= 8) {
#pragma unroll
                                    for (int i = 0; i < 4; ++i) {
                                        if (M == 1 && (i & 1)) continue;  // a single activation row has no odd column
                                        const float dx = (i & 1) ? dx1 : dx0, sx = (i & 1) ? sx1 : sx0;
                                        U[0][j][i] = fmaf(scf[i >> 1], __fmul_rn((float)d0[i], dx), U[0][j][i]);
                                        U[1][j][i] = fmaf(scf[2 + (i >> 1)], __fmul_rn((float)d1[i], dx), U[1][j][i]);
                                        V[0][j][i] = fmaf(mnf[i >> 1], sx, V[0][j][i]);
                                        V[1][j][i] = fmaf(mnf[2 + (i >> 1)], sx, V[1][j][i]);
                                    }
                                }
                                if (DUMP) {
                                    dump4(d0, 0, j, ks * 16 + b);
                                    dump4(d1, 1, j, ks * 16 + b);
                                }
                            }
                        }
                    }
                    // total += d * sum(sc*dot*dx) - dmin * sum(mn*sum)  (q8_acts.rs:296-297, regrouped per super-block)
#pragma unroll
                    for (int h = 0; h < 2; ++h)
#pragma unroll
                        for (int j = 0; j < NG; ++j)
#pragma unroll
                            for (int i = 0; i < 4; ++i) {
                                const uint32_t w = ddw[2 * h + (i >> 1)];
                                const float d = __half2float(__ushort_as_half((unsigned short)(w & 0xffffu)));
                                const float dmin = __half2float(__ushort_as_half((unsigned short)(w >> 16)));
                                acc[h][j][i] += __fsub_rn(__fmul_rn(d, U[h][j][i]), __fmul_rn(dmin, V[h][j][i]));
                            }
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&empty[s]);
        }

        // ---- end of this CTA's share of tile t: combine and finish the tile
        const bool tile_done = (it + 1 == n_total) || t_next != t;
        const int t_cur = t;
        t = t_next;
        ks = ks_next;
        if (++s == NS) {
            s = 0;
            ph ^= 1u;
        }
        if (!tile_done) continue;
        // Hand the tile's partial sums to the finisher warps and stream on.  red is a single
        // buffer: the finishers copy it out at once, so this wait only bites when two tiles
        // close within a fraction of a microsecond.
        if (n_handoff > 0 && !aborted && !mbar_wait_bounded(red_empty, (n_handoff - 1u) & 1u, p.wait_limit)) {
            aborted = true;
            if (lane == 0) note_timeout(p, ERRW_CONSUMER_TIMEOUT, 10);
        }
        if constexpr (CH) {
            // columns of the same activation row sit in different lt lanes: add them up
            float v[4] = {cacc[0], cacc[1], cacc[2], cacc[3]};
            if (MP2 == 1) {  // all eight columns are row 0
                v[0] += v[1];
                v[2] += v[3];
            }
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                if (MP2 <= 2) v[i] += __shfl_xor_sync(0xffffffffu, v[i], 1);
                v[i] += __shfl_xor_sync(0xffffffffu, v[i], 2);
            }
            // after that lane lt = 0 (MP2 <= 2) or lanes lt = 0, 1 (MP2 = 4) hold rows 2lt, 2lt+1
            if (lt < (MP2 == 4 ? 2 : 1)) {
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    const int tok = MP2 == 1 ? 0 : (2 * lt + (i & 1)) % MP2;
                    if ((MP2 > 1 || !(i & 1)) && tok < M)
                        red[(ug * M + tok) * TILE_ROWS + hg * 16 + lg + (i >> 1) * 8] = v[i];
                }
            }
#pragma unroll
            for (int i = 0; i < 4; ++i) cacc[i] = 0.0f;
        } else {
#pragma unroll
            for (int h = 0; h < 2; ++h)
#pragma unroll
                for (int j = 0; j < NG; ++j)
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const int tok = 8 * j + 2 * lt + (i & 1);
                        if (tok < M) red[(kq * M + tok) * TILE_ROWS + rg * 32 + h * 16 + lg + (i >> 1) * 8] = acc[h][j][i];
                        acc[h][j][i] = 0.0f;
                    }
        }
        if (tid == 0) {
            s_flags[0] = t_cur;
            s_flags[1] = (it + 1 == n_total) ? 1 : 0;
            if (tl && p.tl_alt && it + 1 == n_total) tl[1] = globaltimer_ns();  // (alternative stamps) the last tile handed over
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(red_full);
        ++n_handoff;
        t_last = t_cur;
    }
    if (p.pdl && late_dep) pdl_wait();  // keeps the chain of completions whole for the launches behind this one
    // Nothing left to stream: help the finishers close this CTA's last tile.
    {
        const Crew cw{N_FINISHERS + tid, N_CREW_ALL, 3};
        cw.sync();
        if (tl && p.tl_alt && tid == 0) tl[4] = globaltimer_ns();  // (alternative stamps) the closing crew is complete
        close_tile(cw, t_last, true, nullptr);
    }
}

// tile result out[m][r] (m < M rows of the activation record) -> global.
// Called by all threads of the crew that closes the tile.
template <int M>
__device__ __forceinline__ void epilogue_tile(const MvParams &p, const Crew &cw, int tile, float *out, const float *pre,
                                              const float *rope_pre, float gam_pre) {
    const int tid = cw.t;
    const int MO = p.m_out;
    // one row per token (the digit pairs of two-level activations are merged by now)
    auto val = [&](int m, int r) -> float { return out[m * TILE_ROWS + r]; };
    const int row0 = tile * TILE_ROWS;
    if (p.epi == EPI_STORE || p.epi == EPI_ADD) {
        for (int i = tid, j = 0; i < MO * TILE_ROWS; i += cw.n, ++j) {
            const int m = i / TILE_ROWS, r = i % TILE_ROWS;
            const int row = row0 + r;
            if (row >= p.n_out) continue;
            float v = val(m, r);
            if (p.epi == EPI_ADD) v = __fadd_rn(pre ? pre[j] : p.resid[(size_t)m * p.ldr + row], v);
            p.y[(size_t)m * p.ldy + row] = v;
            if (p.nq_sumsq) out[i] = v;
        }
        if (p.epi == EPI_ADD && p.nq_sumsq) {
            // the start of the next RMSNorm, as far as this tile can take it (see MvParams)
            cw.sync();
            const int warp = tid >> 5, lane = tid & 31;
            const int nblk = p.n_out >> 5;
            for (int w = warp; w < MO * 4; w += (cw.n >> 5)) {
                const int m = w >> 2, jb = w & 3;
                const int row = row0 + 32 * jb + lane;
                if (row0 + 32 * jb >= p.n_out) continue;
                const float v = out[m * TILE_ROWS + 32 * jb + lane];
                double ss = (double)v * (double)v;
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
                if (lane == 0) p.nq_sumsq[(size_t)m * nblk + (row >> 5)] = ss;
                if (p.nq_gamma) {
                    const float gam = w == warp ? gam_pre : p.nq_gamma[row];
                    quantize_store(p.nq_act, p.nq_two_level, p.nq_need_sum, m, row >> 5, lane, __fmul_rn(v, gam));
                }
            }
        }
        return;
    }
    if (p.epi == EPI_PEERS) {
        float *mine = p.xch.slots[p.xch.rank];
        const uint32_t e = xch_number(mine, p.xout);
        const size_t slot = ((size_t)(e & 1u) * XCH_MAX_RANKS + p.xch.rank) * XCH_ROW_FLOATS;
        for (int i = tid; i < MO * TILE_ROWS; i += cw.n) {
            const int m = i / TILE_ROWS, r = i % TILE_ROWS;
            const int row = row0 + r;
            if (row >= p.n_out) continue;
            // rank 0 carries the residual rows into the sum (every rank holds the same rows)
            const float v = (p.resid && p.xch.rank == 0) ? __fadd_rn(__ldcg(p.resid + (size_t)m * p.ldr + row), val(m, r)) : val(m, r);
            const unsigned long long w = ((unsigned long long)e << 32) | (unsigned long long)__float_as_uint(v);
            for (int k = 0; k < p.xch.world; ++k) {
                const int dst = (p.xch.rank + k) % p.xch.world;  // start with the local copy, spread the links
                st_relaxed_sys_b64(xch_words(p.xch.slots[dst]) + slot + (size_t)m * p.xch_row + row, w);
            }
        }
        // (nothing to publish separately: every word carries the exchange number next to its value)
        return;
    }
    if (p.epi == EPI_QKV_ROPE) {
        // one head per tile (head_dim 128): warp w serves tokens w, w+8, ...
        const int warp = tid >> 5, lane = tid & 31;
        const int vt = tile + p.qkv_tile_base;  // the head's index in the Q | K | V stack (V may be a matrix, and a launch, of its own)
        const float *nw = vt < p.n_q_tiles ? p.q_norm : (vt < p.n_q_tiles + p.n_k_tiles ? p.k_norm : nullptr);
        const bool rot = vt < p.n_q_tiles + p.n_k_tiles;
        for (int m = warp; m < MO; m += (cw.n >> 5)) {
            float v[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) v[j] = val(m, lane + 32 * j);
            if (nw) {
                // ops::rmsnorm on the head (model/attention.rs:134-137; ops/norm.rs:115-118)
                double ss = 0.0;
#pragma unroll
                for (int j = 0; j < 4; ++j) ss = fma((double)v[j], (double)v[j], ss);
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
                const double scale = 1.0 / sqrt(ss / 128.0 + (double)p.eps);
#pragma unroll
                for (int j = 0; j < 4; ++j)
                    v[j] = __fmul_rn((float)((double)v[j] * scale), nw[lane + 32 * j]);
            }
            // stage the (normed) head so rotation partners can be read back
            __syncwarp();
            float *hs = out + m * TILE_ROWS;
#pragma unroll
            for (int j = 0; j < 4; ++j) hs[lane + 32 * j] = v[j];
            __syncwarp();
            const int half = p.half;
            const float *tab = p.rope + (size_t)m * half * 2;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int c = lane + 32 * j;
                float o = v[j];
                if (rot) {
                    // ops::rope_neox_cached_from_array (ops/rope.rs:70-81); pair i = lane or lane + 32
                    // when half is 32 or 64, which is what the prefetched values cover
                    const bool from_pre = rope_pre != nullptr && m == warp;
                    if (c < half) {
                        const float sn = from_pre ? (j == 0 ? rope_pre[0] : rope_pre[2]) : tab[2 * c];
                        const float cs = from_pre ? (j == 0 ? rope_pre[1] : rope_pre[3]) : tab[2 * c + 1];
                        o = __fsub_rn(__fmul_rn(v[j], cs), __fmul_rn(hs[c + half], sn));
                    } else if (c < 2 * half) {
                        const int i = c - half;
                        const bool first = i < 32;  // pair `lane`, else pair `lane + 32`
                        const float sn = from_pre ? (first ? rope_pre[0] : rope_pre[2]) : tab[2 * i];
                        const float cs = from_pre ? (first ? rope_pre[1] : rope_pre[3]) : tab[2 * i + 1];
                        o = __fadd_rn(__fmul_rn(hs[i], sn), __fmul_rn(v[j], cs));
                    }
                }
                const int row = row0 + c;
                if (row < p.n_out) p.y[(size_t)m * p.ldy + row] = o;
                if (p.kv_k && vt >= p.n_q_tiles) {
                    // K (roped) and V of this position into the f16 cache, round to nearest even
                    // (KvCache::store_at, crates/allpaka-model/src/kv.rs:682-697)
                    const uint32_t pos = (p.pos_dev ? *p.pos_dev : p.pos) + (uint32_t)m;
                    const bool is_k = vt < p.n_q_tiles + p.n_k_tiles;
                    const int col = (vt - p.n_q_tiles - (is_k ? 0 : p.n_k_tiles)) * TILE_ROWS + c;
                    (is_k ? p.kv_k : p.kv_v)[(size_t)pos * p.kv_dim + col] = __float2half_rn(o);
                }
                v[j] = o;
            }
            if (p.q_next.base && vt < p.n_q_tiles) {
                // keep the roped head in shared memory for the packing pass below
                __syncwarp();
#pragma unroll
                for (int j = 0; j < 4; ++j) hs[lane + 32 * j] = v[j];
            }
        }
        // identity attention core: the roped Q head is what the output projection consumes.
        // One warp per (token, 32-element block): the four blocks of a head go in parallel.
        if (p.q_next.base && vt < p.n_q_tiles) {
            cw.sync();
            for (int w = warp; w < MO * 4; w += (cw.n >> 5)) {
                const int m = w >> 2, j = w & 3;
                const float *hs = out + m * TILE_ROWS;
                quantize_store(p.q_next, p.q_next_two_level, p.q_next_need_sum, m, vt * 4 + j, lane, hs[lane + 32 * j]);
            }
        }
        return;
    }
    if (p.epi == EPI_SWIGLU) {
        // rows 0..63 = gate rows [64*tile, 64*tile+64), rows 64..127 = the matching up rows.
        // Work item = (token, 32-row half) = one activation block of the down projection.
        const int warp = tid >> 5, lane = tid & 31;
        for (int w = warp; w < MO * 2; w += (cw.n >> 5)) {
            const int m = w >> 1, h = w & 1;
            const int r = h * 32 + lane;
            const float g = val(m, r), uu = val(m, 64 + r);
            // ops::silu / swiglu (ops/activation.rs:20-22, 116-119)
            const float a = __fmul_rn(__fdiv_rn(g, __fadd_rn(1.0f, expf(-g))), uu);
            const int k = tile * 64 + r;  // column of the down projection
            const bool live = k < p.ffn;
            if (p.act_f32 && live) p.act_f32[(size_t)m * p.ld_act + k] = a;
            if (p.act_next.base && (tile * 64 + h * 32) < p.ffn)
                quantize_store(p.act_next, p.next_two_level, p.next_need_sum, m, k >> 5, lane, live ? a : 0.0f);
        }
        return;
    }
}

}  // namespace apk
