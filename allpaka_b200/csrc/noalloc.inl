// apk_matvec_noalloc: a matvec entry point that allocates nothing.
//
// Who needs it: a host loop that has already handed out every byte of device
// memory it is willing to spend (the engine leases VRAM to weights, KV cache
// and arenas up front and treats a later allocation failure as fatal), or that
// sits somewhere cudaMalloc is off the table because it would stall the device
// or fail outright: a latency-bounded decode thread, a process whose allocator
// has been frozen after start-up.  Such a caller owns the
// input and output buffers already; what it cannot supply is the kernel's
// private scratch (stream-K partial sums, the error word, and the
// quantised-activation records).  Here that scratch is a fixed
// array in the library's own device image.
//
// Included at the end of apk_b200.cu: same translation unit as the kernels, so
// the array's symbol is resolved with cudaGetSymbolAddress in this file.

namespace {

constexpr uint32_t NOALLOC_MAX_CTAS = 160;       // one CTA per SM
constexpr size_t NOALLOC_PARTIALS_BYTES = (size_t)NOALLOC_MAX_CTAS * 2 * MAX_M_EFF * TILE_ROWS * sizeof(unsigned long long);
constexpr size_t NOALLOC_ERR_BYTES = 256;
constexpr size_t NOALLOC_ACTS_BYTES = (size_t)MAX_M_EFF * APK_NOALLOC_MAX_N_IN * 5 / 4 + 256;
constexpr size_t NOALLOC_OFF_ERR = NOALLOC_PARTIALS_BYTES;
constexpr size_t NOALLOC_OFF_ACTS = NOALLOC_OFF_ERR + NOALLOC_ERR_BYTES;
constexpr size_t NOALLOC_TOTAL = NOALLOC_OFF_ACTS + NOALLOC_ACTS_BYTES;  // about 5.9 MB

// Held by every GPU that loads the library, until the process exits.  In host
// code this name is only a stand-in for the symbol, never a device address.
static __device__ __align__(256) unsigned char g_noalloc_scratch[NOALLOC_TOTAL];

// The array exists once per DEVICE, not per context: its address and whether its last
// user was seen to leave it clean are kept per device, under one lock, so that contexts
// sharing a GPU see each other's calls.
constexpr int NOALLOC_MAX_DEVICES = 64;
struct NoallocDev {
    unsigned char *ptr = nullptr;
    bool dirty = true;  // until a call is seen to end cleanly the tagged partial sums are cleared first
};
NoallocDev g_noalloc_dev[NOALLOC_MAX_DEVICES];
std::mutex g_noalloc_mu;

// Device address of the array on the context's device (that device is current).
int noalloc_setup(apk_ctx *c, NoallocDev **out) {
    if (c->device < 0 || c->device >= NOALLOC_MAX_DEVICES) return fail(APK_ERR_INVALID_ARG, "device %d", c->device);
    NoallocDev *d = &g_noalloc_dev[c->device];
    if (!d->ptr) {
        void *ptr = nullptr;
        const cudaError_t e = cudaGetSymbolAddress(&ptr, g_noalloc_scratch);
        if (e != cudaSuccess || !ptr)
            return fail(APK_ERR_CUDA, "cudaGetSymbolAddress(scratch): %s", cudaGetErrorString(e));
        d->ptr = (unsigned char *)ptr;
    }
    *out = d;
    return APK_OK;
}

}  // namespace

extern "C" int apk_matvec_noalloc(apk_ctx *c, const void *w, uint32_t ty, uint32_t n_in, uint32_t n_out,
                                  const float *x_dev, uint32_t m, uint32_t act_mode, float *y_dev, void *stream,
                                  int wait) {
    if (!c || !w || !x_dev || !y_dev) return fail(APK_ERR_INVALID_ARG, "matvec_noalloc: null argument");
    std::lock_guard<std::mutex> g(c->mu);
    CUDA_TRY(cudaSetDevice(c->device));
    APK_TRY(check_m(m));
    if (n_in > APK_NOALLOC_MAX_N_IN || n_out > APK_NOALLOC_MAX_N_OUT)
        return fail(APK_DECLINE_UNSUPPORTED_SHAPE,
                    "matvec_noalloc: %u x %u exceeds the built-in scratch (n_in <= %u, n_out <= %u)", n_out, n_in,
                    APK_NOALLOC_MAX_N_IN, APK_NOALLOC_MAX_N_OUT);
    if ((uint32_t)c->n_sm > NOALLOC_MAX_CTAS)
        return fail(APK_DECLINE_MISSING_CAPABILITY, "matvec_noalloc: %d SMs exceed the built-in scratch (%u)", c->n_sm,
                    NOALLOC_MAX_CTAS);
    // the weights must be resident already: uploading them here would allocate
    auto it = c->mats.find(MatKey(KIND_PLAIN, w, nullptr, nullptr, ty, n_out, n_in, SHARD_NONE, 0));
    if (it == c->mats.end())
        return fail(APK_DECLINE_INVALID_STATE,
                    "matvec_noalloc: matrix is not resident; call apk_register_matrix first (this entry point never allocates)");
    const DevMatrix *W = it->second.get();
    std::lock_guard<std::mutex> gdev(g_noalloc_mu);
    NoallocDev *dev = nullptr;
    APK_TRY(noalloc_setup(c, &dev));  // first call on this device: resolves the scratch symbol
    cudaStream_t st = (cudaStream_t)stream;
    unsigned char *base = dev->ptr;
    unsigned long long *partials = reinterpret_cast<unsigned long long *>(base);
    int *err = reinterpret_cast<int *>(base + NOALLOC_OFF_ERR);
    void *acts = base + NOALLOC_OFF_ACTS;
    // The array keeps the previous call's contents: the error word must start at zero.
    CUDA_TRY(cudaMemsetAsync(err, 0, NOALLOC_ERR_BYTES, st));
    // So must the tagged partial sums.  A kernel that ran to its end leaves them zero; only a
    // call that was seen to end cleanly (wait != 0, no error) proves that, so after any other
    // call on this device, from whichever context, the region is cleared again.
    if (dev->dirty) CUDA_TRY(cudaMemsetAsync(base, 0, NOALLOC_PARTIALS_BYTES, st));
    dev->dirty = true;

    const ActMode mode = resolve_mode(act_mode, m);
    MvKernel k = pick_kernel(W->ty, mode.m_eff, false);
    if (!k) return fail(APK_DECLINE_UNSUPPORTED_SHAPE, "no kernel for %d activation rows", mode.m_eff);
    MvParams p{};
    p.act = act_layout(acts, W->ty, mode.m_eff);
    const bool in_cta = m == 1 && W->n_in <= (uint32_t)(N_CONSUMERS * PRO_CH) && ((uintptr_t)x_dev & 15) == 0 &&
                        want_resident(c, W, mode.m_eff);
    if (in_cta) {
        p.pro = PRO_QUANT;
        PrepParams &pp = p.prep;
        pp.x = x_dev; pp.ldx = (int)n_in;
        pp.n = (int)n_in; pp.m = 1;
        pp.out = p.act;
        pp.two_level = mode.two_level;
        pp.need_sum = needs_sum(W->ty);
    } else {
        PrepParams pp{};
        pp.x = x_dev; pp.ldx = (int)n_in;
        pp.n = (int)n_in; pp.m = (int)m;
        pp.out = p.act;
        pp.two_level = mode.two_level;
        pp.need_sum = needs_sum(W->ty);
        prep_acts_kernel<<<dim3((n_in / 32 + 7) / 8, m), 256, 0, st>>>(pp, 0);
        CUDA_TRY(cudaGetLastError());
        c->st.launches++;
        p.pro = want_resident(c, W, mode.m_eff) ? PRO_LOAD : PRO_STREAM;
    }
    p.W = W->d;
    p.ty = (int)W->ty;
    p.n_out = (int)W->n_out;
    p.nb = W->nb;
    p.n_tiles = W->n_tiles;
    p.KS = W->KS;
    p.tile_bytes = W->tile_bytes;
    p.two_level = mode.two_level;
    p.m_out = mode.two_level ? mode.m_eff / 2 : mode.m_eff;
    p.partials = partials;
    p.err = err;
    p.wait_limit = c->wait_limit;
    p.xin.index = -1;
    p.pdl = 0;
    p.inflight = c->inflight;
    p.inflight_pre = c->inflight_pre;
    p.epi = EPI_STORE;
    p.y = y_dev;
    p.ldy = (int)n_out;
    const int act_rec = p.act.rec_bytes();
    const int ns = pick_stages(c, (int)W->ty, mode.m_eff, p.pro, W->KS, act_rec);
    if (ns < 2) return fail(APK_DECLINE_MISSING_CAPABILITY, "activations do not fit in shared memory");
    p.n_stages = ns;
    const int smem = mv_smem_total((int)W->ty, mode.m_eff, p.pro, W->KS, act_rec, ns);
    const long long U = (long long)W->n_tiles * W->KS;
    const int grid = (int)std::min<long long>(c->n_sm, U);
    k<<<grid, MV_THREADS, smem, st>>>(p);
    CUDA_TRY(cudaGetLastError());
    c->st.launches++;
    c->st.calls++;
    if (!wait) return APK_OK;
    int herr = 0;  // plain stack word: a synchronous copy needs no pinned staging of ours
    CUDA_TRY(cudaMemcpyAsync(&herr, err, sizeof herr, cudaMemcpyDeviceToHost, st));
    CUDA_TRY(cudaStreamSynchronize(st));
    if (herr != 0)
        return fail(APK_ERR_TIMEOUT, "device-side wait expired (%s)",
                    (herr & 15) == ERRW_PRODUCER_TIMEOUT   ? "copy producer"
                    : (herr & 15) == ERRW_FINISHER_TIMEOUT ? "a tile piece of another CTA never arrived"
                                                    : "tile consumer");
    dev->dirty = false;
    return APK_OK;
}
