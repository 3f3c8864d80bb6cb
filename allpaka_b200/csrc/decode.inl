// Whole-token decode: the per-layer call order of the reference
// (crates/allpaka-model/src/model/decode.rs:435-591, 755-777; finish_hidden
// 594-602) as one captured CUDA graph, replayed per token.  Included at the end
// of apk_b200.cu (same translation unit).
//
// Per layer (m tokens, all on the GPU):
//   prep    h = rmsnorm(x, attn_norm) -> Q8 blocks
//   matvec  [Q|K|V] rows, epilogue: per-head norm + NeoX RoPE          -> qkv
//   prep    attention-core stand-in: the roped Q slice is the core's output
//   matvec  wo, epilogue x += .           (tensor parallel: partial sums -> all-reduce,
//                                          the add moves into the next prep)
//   prep    h = rmsnorm(x, ffn_norm) -> Q8 blocks
//   matvec  gate/up interleaved, epilogue swiglu -> blocks for `down`
//   matvec  down, epilogue x += .
// then rmsnorm(x, output_norm) + LM head (+ argmax).

namespace {

__global__ void __launch_bounds__(1024) argmax_rows_kernel(const float *logits, int vocab_l, int world, int m,
                                                           uint32_t *out) {
    // logits laid out [rank][m][vocab_l]; token = blockIdx.x.  Ties go to the
    // higher index, as the CPU greedy pick does (model/decode.rs:604-608).
    __shared__ float sv[32];
    __shared__ int si[32];
    const int tok = blockIdx.x;
    float best = -INFINITY;
    int bi = -1;
    const int vocab = vocab_l * world;
    for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
        const int r = i / vocab_l, j = i % vocab_l;
        const float v = logits[((size_t)r * m + tok) * vocab_l + j];
        if (v > best || (v == best && i > bi) || bi < 0) { best = v; bi = i; }
    }
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (oi >= 0 && (bi < 0 || ov > best || (ov == best && oi > bi))) { best = ov; bi = oi; }
    }
    if ((threadIdx.x & 31) == 0) { sv[threadIdx.x >> 5] = best; si[threadIdx.x >> 5] = bi; }
    __syncthreads();
    if (threadIdx.x < 32) {
        best = sv[threadIdx.x];
        bi = si[threadIdx.x];
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, best, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (oi >= 0 && (bi < 0 || ov > best || (ov == best && oi > bi))) { best = ov; bi = oi; }
        }
        if (threadIdx.x == 0) out[tok] = (uint32_t)(bi < 0 ? 0 : bi);
    }
}

int decline_decode(apk_ctx *c, int code, const char *fmt, ...) {
    char buf[400];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof buf, fmt, ap);
    va_end(ap);
    c->st.decode_declines++;
    return fail(code, "stage=backend-decode reason=%s", buf);
}

// FNV-1a over every descriptor of the request that the plan bakes in: a caller that
// rewrites the layer array in place, or reuses its address for another model, gets a
// new plan instead of the old weights.
uint64_t desc_hash(const apk_token_req *r) {
    uint64_t h = 1469598103934665603ull;
    auto mix = [&](uint64_t v) {
        for (int i = 0; i < 8; ++i) {
            h ^= (v >> (8 * i)) & 0xffu;
            h *= 1099511628211ull;
        }
    };
    auto mat = [&](const apk_mat &m) {
        mix((uint64_t)(uintptr_t)m.w);
        mix(((uint64_t)m.ty << 32) | m.n_out);
    };
    for (uint32_t l = 0; l < r->n_layers; ++l) {
        const apk_token_layer &t = r->layers[l];
        mix((uint64_t)(uintptr_t)t.attn_norm); mix((uint64_t)(uintptr_t)t.ffn_norm);
        mix((uint64_t)(uintptr_t)t.q_norm); mix((uint64_t)(uintptr_t)t.k_norm);
        mat(t.wq); mat(t.wk); mat(t.wv); mat(t.wo); mat(t.gate); mat(t.up); mat(t.down);
    }
    mix((uint64_t)(uintptr_t)r->output_norm);
    mat(r->output);
    mat(r->embd);
    return h;
}

bool plan_matches(const Plan *p, const apk_token_req *r) {
    return p && p->attn_core == r->attn_core && p->kv == r->kv && p->scale == r->scale &&
           p->layers_key == r->layers && p->n_layers == r->n_layers && p->output_key == r->output.w &&
           p->hidden == r->hidden && p->head_dim == r->head_dim && p->n_heads == r->n_heads &&
           p->n_kv_heads == r->n_kv_heads && p->rot_dim == r->rot_dim && p->vocab == r->output.n_out &&
           p->eps == r->eps && p->desc_hash == desc_hash(r);
}

int nccl_allreduce(apk_ctx *c, float *buf, size_t n) {
    const int rc = g_nccl.AllReduce(buf, buf, n, NCCL_FLOAT32, NCCL_SUM, c->comm, c->stream);
    if (rc) return fail(APK_ERR_NCCL, "ncclAllReduce: %s", g_nccl.GetErrorString(rc));
    return APK_OK;
}

bool uses_xch(const apk_ctx *c) { return c->p2p_ready && (c->world > 1 || c->self_xch); }

// Position splits of the attention core: fixed per cache (the launch shape is captured), and sized
// in whole steps of a CTA (64 positions) so that the splits come out even.  Long caches: at least 256
// positions per split (four steps per warp: the pipeline fills, the per-CTA prologue and merge
// amortise), and kv heads x splits at most one wave of two CTAs per SM (measured at 32768 positions:
// 37 splits 30 us, 43 splits 40 us, 128 splits 43 us).  Short caches are latency: fewer steps per
// split while the grid stays within one CTA per SM (measured, 64 q / 8 kv heads: 1024 positions
// 6.9 us with 16 splits against 11.5 us with 4; 2048 positions 8.1 against 10.7 us with 8; more CTAs
// than SMs lose again: 4096 positions 11.4 us with 64 splits against 9.9 us with 16).
int attn_splits(const apk_ctx *c, const apk_kv *kv) {
    const uint32_t n_kv = std::max<uint32_t>(1, kv->kv_dim / TILE_ROWS);
    const uint32_t wave = std::max<uint32_t>(1, 2u * (uint32_t)c->n_sm / n_kv);
    const uint32_t one_per_sm = std::max<uint32_t>(1, (uint32_t)c->n_sm / n_kv);
    const uint32_t steps = (kv->capacity + 63) / 64;
    const uint32_t long_steps = std::max<uint32_t>(1, (uint32_t)c->attn_min_pos / 64);
    uint32_t per = (steps + one_per_sm - 1) / one_per_sm;                        // steps per split, one CTA per SM
    if (per >= long_steps) per = std::max(long_steps, (steps + wave - 1) / wave);  // two per SM
    return (int)std::max<uint32_t>(1, std::min<uint32_t>((steps + per - 1) / per, 128));
}

// q [m][ldq] -> attention over one layer of the cache -> optional f32 rows, optional records for wo.
int launch_attention(apk_ctx *c, const apk_kv *kv, uint32_t layer, const float *q, int ldq, uint32_t m, uint32_t n_heads_l,
                     const uint32_t *pos_dev, uint32_t pos, float scale, float *part, float *out, int ldo,
                     const ActLayout *next, int next_two_level, int next_need_sum) {
    AttnParams ap{};
    ap.q = q; ap.ldq = ldq;
    ap.kc = kv->k(layer); ap.vc = kv->v(layer);
    ap.kv_dim = (int)kv->kv_dim;
    ap.n_kv_heads = (int)(kv->kv_dim / TILE_ROWS);
    ap.group = (int)(n_heads_l / (kv->kv_dim / TILE_ROWS));
    ap.pos_dev = pos_dev; ap.pos = pos;
    ap.m = (int)m;
    ap.n_splits = attn_splits(c, kv);
    ap.scale = scale;
    ap.part = part;
    ap.out = out; ap.ldo = ldo;
    if (next) ap.next = *next;
    ap.next_two_level = next_two_level;
    ap.next_need_sum = next_need_sum;
    const int pdl = c->use_pdl ? 1 : 0;
    if (c->attn_tc) {
        if (!c->attn_tc_ready) {
            CUDA_TRY(cudaFuncSetAttribute((const void *)attn_split_tc_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, ATC_SMEM));
            CUDA_TRY(cudaFuncSetAttribute((const void *)attn_split_tc_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, ATC_SMEM));
            c->attn_tc_ready = true;
        }
        // verify batches: 16 / group consecutive rows share one pass over K and V.  Batches of more rows
        // than that take several CTAs per (kv head, split): they sit next to each other in the grid, so
        // that they stream the same K and V rows at the same time and all but one hit in L2, and the
        // splits shrink to keep the whole grid within one wave.
        if (m > 1) {
            const int nz = ((int)m + atc_rows(ap.group) - 1) / atc_rows(ap.group);
            ap.n_splits = std::min(ap.n_splits, std::max(1, 2 * c->n_sm / (ap.n_kv_heads * nz)));
            CUDA_TRY(launch_ex(c, attn_split_tc_kernel<true>, dim3(nz, ap.n_kv_heads, ap.n_splits), dim3(ATC_WARPS * 32), (size_t)ATC_SMEM, c->use_pdl, ap, pdl));
        } else
            CUDA_TRY(launch_ex(c, attn_split_tc_kernel<false>, dim3(ap.n_kv_heads, ap.n_splits, 1), dim3(ATC_WARPS * 32), (size_t)ATC_SMEM, c->use_pdl, ap, pdl));
    } else {
        CUDA_TRY(launch_ex(c, attn_split_kernel, dim3(ap.n_kv_heads, ap.n_splits, m), dim3(ATT_WARPS * 32), 0, c->use_pdl, ap, pdl));
    }
    CUDA_TRY(launch_ex(c, attn_combine_kernel, dim3(n_heads_l, m), dim3(TILE_ROWS), 0, c->use_pdl, ap, pdl));
    c->st.launches += 2;
    return APK_OK;
}

int build_plan(apk_ctx *c, const apk_token_req *r) {
    c->plan.reset();
    auto P = std::make_unique<Plan>();
    const uint32_t H = r->hidden, nq = r->n_heads * r->head_dim, nkv = r->n_kv_heads * r->head_dim;
    if (r->n_layers == 0 || !r->layers || !r->output.w || !r->output_norm)
        return decline_decode(c, APK_ERR_INVALID_ARG, "empty layer list or missing output head");
    if (r->head_dim != TILE_ROWS) return decline_decode(c, APK_DECLINE_UNSUPPORTED_SHAPE, "head_dim %u (fused QKV epilogue is written for 128)", r->head_dim);
    if (r->rot_dim > r->head_dim || r->rot_dim % 2) return decline_decode(c, APK_DECLINE_UNSUPPORTED_SHAPE, "rot_dim %u", r->rot_dim);
    const uint32_t ffn = r->layers[0].gate.n_out;
    P->layers_key = r->layers; P->n_layers = r->n_layers; P->output_key = r->output.w;
    P->desc_hash = desc_hash(r);
    P->hidden = H; P->head_dim = r->head_dim; P->n_heads = r->n_heads; P->n_kv_heads = r->n_kv_heads;
    P->rot_dim = r->rot_dim; P->vocab = r->output.n_out; P->eps = r->eps; P->ffn = ffn;
    P->attn_core = r->attn_core; P->kv = r->kv; P->scale = r->scale;
    if (uses_xch(c) && ((size_t)APK_MAX_M * H > (size_t)XCH_ROW_FLOATS || H % 4))
        return decline_decode(c, APK_DECLINE_UNSUPPORTED_SHAPE, "hidden %u exceeds the peer exchange buffer", H);
    if (P->vocab % c->world) return decline_decode(c, APK_DECLINE_UNSUPPORTED_SHAPE, "vocab %u does not split over %d ranks", P->vocab, c->world);
    P->nq_l = nq / c->world; P->nkv_l = nkv / c->world; P->vocab_l = P->vocab / c->world;

    // norm weights: one device array
    const size_t per_layer = 2 * (size_t)H + 2 * 128;
    std::vector<float> norms(per_layer * r->n_layers + H, 0.f);
    for (uint32_t l = 0; l < r->n_layers; ++l) {
        const apk_token_layer &tl = r->layers[l];
        if (!tl.attn_norm || !tl.ffn_norm) return decline_decode(c, APK_ERR_INVALID_ARG, "layer %u: missing norm weights", l);
        float *b = norms.data() + per_layer * l;
        memcpy(b, tl.attn_norm, H * sizeof(float));
        memcpy(b + H, tl.ffn_norm, H * sizeof(float));
        if (tl.q_norm) memcpy(b + 2 * H, tl.q_norm, 128 * sizeof(float));
        if (tl.k_norm) memcpy(b + 2 * H + 128, tl.k_norm, 128 * sizeof(float));
    }
    memcpy(norms.data() + per_layer * r->n_layers, r->output_norm, H * sizeof(float));
    APK_TRY(P->norms.ensure(norms.size() * sizeof(float)));
    CUDA_TRY(cudaMemcpy(P->norms.p, norms.data(), norms.size() * sizeof(float), cudaMemcpyHostToDevice));

    P->L.resize(r->n_layers);
    for (uint32_t l = 0; l < r->n_layers; ++l) {
        const apk_token_layer &tl = r->layers[l];
        PlanLayer &pl = P->L[l];
        if (tl.wq.ty != tl.wk.ty) return decline_decode(c, APK_DECLINE_UNSUPPORTED_TYPE, "layer %u: wq/wk types differ", l);
        // V in a type of its own (the Q4_K_M recipe keeps it in Q6_K): a second matrix and launch
        const bool own_v = tl.wv.ty != tl.wq.ty;
        if (own_v && c->world > 1) return decline_decode(c, APK_DECLINE_UNSUPPORTED_TYPE, "layer %u: wv in a type of its own on a sharded context", l);
        if (tl.gate.ty != tl.up.ty) return decline_decode(c, APK_DECLINE_UNSUPPORTED_TYPE, "layer %u: gate/up types differ", l);
        if (tl.wq.n_out != nq || tl.wk.n_out != nkv || tl.wv.n_out != nkv || tl.wo.n_out != H || tl.gate.n_out != ffn ||
            tl.up.n_out != ffn || tl.down.n_out != H)
            return decline_decode(c, APK_DECLINE_UNSUPPORTED_SHAPE, "layer %u: projection shapes disagree with the request", l);
        int rc;
        if ((rc = resolve_qkv(c, tl.wq.ty, tl.wq.w, tl.wk.w, own_v ? nullptr : tl.wv.w, H, nq, nkv, &pl.qkv))) { c->st.decode_declines++; return rc; }
        pl.v = nullptr;
        if (own_v && (rc = resolve_plain(c, "attn wv", tl.wv.w, tl.wv.ty, nkv, H, SHARD_NONE, &pl.v))) { c->st.decode_declines++; return rc; }
        if ((rc = resolve_plain(c, "attn wo", tl.wo.w, tl.wo.ty, H, nq, SHARD_K, &pl.wo))) { c->st.decode_declines++; return rc; }
        if ((rc = resolve_gateup(c, tl.gate.ty, tl.gate.w, tl.up.w, H, ffn, &pl.gateup, &P->ffn_l))) { c->st.decode_declines++; return rc; }
        if ((rc = resolve_plain(c, "ffn down", tl.down.w, tl.down.ty, H, ffn, SHARD_K, &pl.down))) { c->st.decode_declines++; return rc; }
        const float *b = P->norms.as<float>() + per_layer * l;
        pl.attn_norm = b;
        pl.ffn_norm = b + H;
        pl.q_norm = tl.q_norm ? b + 2 * H : nullptr;
        pl.k_norm = tl.k_norm ? b + 2 * H + 128 : nullptr;
    }
    {
        int rc;
        if ((rc = resolve_plain(c, "output", r->output.w, r->output.ty, P->vocab, H, SHARD_ROWS, &P->head))) { c->st.decode_declines++; return rc; }
    }
    P->out_norm = P->norms.as<float>() + per_layer * r->n_layers;
    if (r->embd.w) {
        // the embedding table stays whole on every rank (a row is looked up, not multiplied); at one
        // rank a tied LM head resolves to the same resident matrix
        int rc;
        if ((rc = resolve_plain(c, "token embedding", r->embd.w, r->embd.ty, r->embd.n_out, H, SHARD_NONE, &P->embd))) { c->st.decode_declines++; return rc; }
    }

    const uint32_t M = APK_MAX_M, ldq = P->nq_l + 2 * P->nkv_l;
    const uint32_t big = APK_TY_Q4_K;  // the larger record flavour bounds every buffer
    APK_TRY(P->xin.ensure((size_t)M * H * 4));
    APK_TRY(P->x[0].ensure((size_t)M * H * 4));
    APK_TRY(P->x[1].ensure((size_t)M * H * 4));
    APK_TRY(P->qkv.ensure((size_t)M * ldq * 4));
    APK_TRY(P->yp.ensure((size_t)M * H * 4));
    APK_TRY(P->act_h.ensure(act_bytes(big, 2 * M, H)));
    APK_TRY(P->act_q.ensure(act_bytes(big, 2 * M, P->nq_l)));
    APK_TRY(P->act_d.ensure(act_bytes(big, 2 * M, P->ffn_l)));
    APK_TRY(P->logits.ensure((size_t)M * P->vocab_l * 4));
    if (c->world > 1) APK_TRY(P->logits_all.ensure((size_t)M * P->vocab * 4));
    APK_TRY(P->amax.ensure(M * sizeof(uint32_t)));
    APK_TRY(P->rope.ensure((size_t)M * (r->rot_dim / 2 + 1) * 2 * 4));
    APK_TRY(P->sumsq.ensure((size_t)M * (H / 32 + 1) * sizeof(double), true));
    APK_TRY(P->hidden_out.ensure((size_t)M * H * 4));
    APK_TRY(P->pos.ensure(256, true));
    if (r->attn_core == APK_ATTN_CAUSAL) {
        if (nq % c->world || nkv % c->world || (nq / nkv) * nkv != nq)
            return decline_decode(c, APK_DECLINE_UNSUPPORTED_SHAPE, "heads do not split over the ranks");
        if (!r->kv || r->kv->n_layers < r->n_layers || r->kv->kv_dim != P->nkv_l)
            return decline_decode(c, APK_ERR_INVALID_ARG, "the KV cache does not fit the request (layers, kv_dim)");
        APK_TRY(P->attn_part.ensure((size_t)M * (P->nq_l / TILE_ROWS) * attn_splits(c, r->kv) * ATT_PART * 4));
        APK_TRY(P->attn_out.ensure((size_t)M * P->nq_l * 4));
    }
    if (uses_xch(c)) {
        // A new plan restarts the exchange numbering (its exchanges per token may differ): clear
        // this rank's tagged words and token counter, then meet the other ranks, so that nobody's
        // first token runs against a peer that is still uploading or against old tags.  (The bounded
        // device-side waits are for a peer that died, not for one that is a few seconds behind.)
        if (c->world > 1) APK_TRY(nccl_allreduce(c, P->yp.as<float>(), 1));  // every rank's previous token is over
        CUDA_TRY(cudaStreamSynchronize(c->stream));
        CUDA_TRY(cudaMemsetAsync(c->xch_local, 0, XCH_BYTES, c->stream));
    }
    if (c->world > 1) {
        APK_TRY(nccl_allreduce(c, P->yp.as<float>(), 1));
        CUDA_TRY(cudaStreamSynchronize(c->stream));
    }
    c->plan = std::move(P);
    return APK_OK;
}

// The matvecs of a layer and the head, as launches on the context stream.
struct TokenLaunch {
    apk_ctx *c;
    Plan *P;
    uint32_t m;
    ActMode q8, autom;
    int cur = 0;
    bool pending_add = false;  // NCCL reductions: yp holds a combined delta not yet added to x
    int pending_xch = -1;      // peer exchange: index of the exchange whose sum is not yet added to x
    int n_xch = 0;             // exchanges launched so far in this token
    bool first = true;         // the next matvec launch is the token's first
    bool in_token = true;      // launches follow the token's order (false: one kind replayed in isolation)
    bool have_sumsq = false;   // the last residual matvec left the per-block sums of squares of x[cur]
    // the previous residual matvec already quantised x * gamma for this (matrix, mode): its
    // records sit in act_h and only lack the row-wide RMSNorm scale (opt-in approximation)
    const DevMatrix *prenormed_for = nullptr;
    int prenormed_m_eff = 0;

    TokenLaunch(apk_ctx *c_, Plan *P_, uint32_t m_) : c(c_), P(P_), m(m_), q8{0, (int)m_}, autom(resolve_mode(APK_ACT_AUTO, m_)) {}

    int per_token() const { return 2 * (int)P->n_layers; }
    // Can the residual epilogue in front of matvec W (through an RMSNorm) do the quantisation?
    bool can_prenorm(const DevMatrix *W, ActMode mode) const {
        const bool on = c->fuse_norm == 2 || (c->fuse_norm == 3 && m > 1);
        return on && W != P->head && !uses_xch(c) && c->world == 1 && P->hidden % 32 == 0 && want_resident(c, W, mode.m_eff);
    }
    int launch(const DevMatrix *W, MvParams &p, ActMode mode, const DevMatrix *Wn) {
        if (first && uses_xch(c)) {
            p.xch = c->xch;
            p.tok_inc = 1;
        }
        first = false;
        (void)Wn;
        return launch_matvec(c, W, p, mode);
    }
    // Parity instrumentation: keep the rows this launch normalises and the records it consumes.
    void record_hook(const float *x_in, ActMode mode, MvParams *p) {
        if (!c->rec_dump || c->rec_idx >= c->rec_cap) return;
        uint8_t *slab = c->rec_dump + (size_t)c->rec_idx * c->rec_slab;
        cudaMemcpyAsync(slab, x_in, (size_t)m * P->hidden * 4, cudaMemcpyDeviceToDevice, c->stream);
        p->act_dump = slab + (size_t)APK_MAX_M * P->hidden * 4;
        c->rec_meta.push_back({p->act.ke, mode.m_eff, mode.two_level, c->launch_no});
        c->rec_idx++;
    }
    // activations of a matvec that reads the residual stream through an RMSNorm
    int normed_input(const DevMatrix *W, const float *gamma, ActMode mode, MvParams *p, bool advance, float *hout = nullptr) {
        const uint32_t H = P->hidden;
        p->xin.index = -1;
        if (prenormed_for == W && prenormed_m_eff == mode.m_eff) {
            p->act = act_layout(P->act_h.p, W->ty, mode.m_eff);
            p->pro = PRO_LOAD;
            p->norm_sumsq = P->sumsq.as<double>();
            p->norm_blocks = (int)(H / 32);
            p->norm_eps = P->eps;
            record_hook(P->x[cur].as<float>(), mode, p);
            if (advance) prenormed_for = nullptr;
            return APK_OK;
        }
        float *xc = P->x[cur].as<float>();
        if (pending_xch >= 0) {
            float *xn = P->x[cur ^ 1].as<float>();
            const bool in_cta = m == 1 && H <= (uint32_t)(N_CONSUMERS * PRO_CH) && want_resident(c, W, mode.m_eff);
            if (in_cta) {
                // the kernel gathers the row itself: residual + rank-ordered sum of the slots
                APK_TRY(stage_acts(c, W, xc, (int)H, nullptr, 0, xn, (int)H, gamma, P->eps, m, mode, P->act_h.p, p, nullptr, hout));
                p->xch = c->xch;
                p->xin = XchSeq{pending_xch, per_token()};
                p->xin_late = in_token ? 1 : 0;
                if (advance) { cur ^= 1; pending_xch = -1; }
                return APK_OK;
            }
            XchReduceParams rp{};
            rp.xch = c->xch;
            rp.seq = XchSeq{pending_xch, per_token()};
            rp.xout = xn; rp.ldxout = (int)H;
            rp.n = (int)H; rp.m = (int)m;
            rp.err = c->d_err;
            rp.pdl = c->use_pdl ? 1 : 0;
            rp.wait_limit = c->wait_limit;
            const unsigned grid = (unsigned)(((size_t)m * H + 1023) / 1024);
            CUDA_TRY(launch_ex(c, xch_reduce_kernel, dim3(grid), dim3(256), 0, c->use_pdl, rp));
            c->st.launches++;
            if (advance) { cur ^= 1; pending_xch = -1; xc = xn; }
            else xc = xn;
            return stage_acts(c, W, xc, (int)H, nullptr, 0, nullptr, 0, gamma, P->eps, m, mode, P->act_h.p, p, nullptr, hout);
        }
        if (pending_add) {
            float *xn = P->x[cur ^ 1].as<float>();
            APK_TRY(stage_acts(c, W, xc, (int)H, P->yp.as<float>(), (int)H, xn, (int)H, gamma, P->eps, m, mode, P->act_h.p, p, nullptr, hout));
            if (advance) { cur ^= 1; pending_add = false; }
            return APK_OK;
        }
        APK_TRY(stage_acts(c, W, xc, (int)H, nullptr, 0, nullptr, 0, gamma, P->eps, m, mode, P->act_h.p, p,
                           have_sumsq ? P->sumsq.as<double>() : nullptr, hout));
        record_hook(xc, mode, p);
        return APK_OK;
    }
    int qkv(PlanLayer &L, bool advance = true, uint32_t layer = 0) {
        if (L.v) {
            const int v_base = (int)((P->nq_l + P->nkv_l) / TILE_ROWS);
            // One token row on one GPU, nothing pending on the residual stream: V (a few tiles, its row
            // normalised and quantised inside its own CTAs) runs on SMs of its own beside Q | K instead of
            // as a whole launch after it.  A few CTAs per V tile, the other SMs for Q | K; the kernel behind
            // them depends on both branches (and keeps its programmatic edge: it may start early and waits
            // itself, like every other launch of the token).
            // (at most a quarter of the SMs go to V)
            const int v_ctas = L.v->n_tiles * std::min(c->fork_v, c->n_sm / (4 * std::max(1, L.v->n_tiles)));
            const bool beside = v_ctas > 0 && c->world == 1 && !uses_xch(c) && m == 1 && !pending_add && pending_xch < 0 &&
                                P->hidden <= (uint32_t)(N_CONSUMERS * PRO_CH) && want_resident(c, L.v, q8.m_eff);
            if (!beside) {
                APK_TRY(qkv_part(L, L.qkv, false, layer, 0));
                return qkv_part(L, L.v, advance, layer, v_base);
            }
            CUDA_TRY(cudaEventRecord(c->ev_fork, c->stream));
            CUDA_TRY(cudaStreamWaitEvent(c->side, c->ev_fork, 0));
            c->launch_stream = c->side;
            c->grid_cap = v_ctas;
            int rc = qkv_part(L, L.v, false, layer, v_base);
            c->launch_stream = nullptr;
            if (rc == APK_OK) rc = cudaEventRecord(c->ev_join, c->side) == cudaSuccess ? APK_OK : fail(APK_ERR_CUDA, "event record on the side branch");
            c->grid_cap = c->n_sm - v_ctas;
            if (rc == APK_OK) rc = qkv_part(L, L.qkv, advance, layer, 0);
            c->grid_cap = 0;
            // (joined even after an error above, so that a capture in progress can end)
            const cudaError_t je = cudaStreamWaitEvent(c->stream, c->ev_join, 0);
            if (rc == APK_OK && je != cudaSuccess) rc = fail(APK_ERR_CUDA, "joining the side branch: %s", cudaGetErrorString(je));
            return rc;
        }
        return qkv_part(L, L.qkv, advance, layer, 0);
    }
    // W: the Q | K | V stack, or Q | K and then V when V has a type of its own (tile_base: V's first head in the stack)
    int qkv_part(PlanLayer &L, DevMatrix *W, bool advance, uint32_t layer, int tile_base) {
        MvParams p{};
        APK_TRY(normed_input(W, L.attn_norm, q8, &p, advance));
        p.epi = EPI_QKV_ROPE;
        p.qkv_tile_base = tile_base;
        p.y = P->qkv.as<float>() + (size_t)tile_base * TILE_ROWS;
        p.ldy = (int)(P->nq_l + 2 * P->nkv_l);
        p.n_q_tiles = (int)(P->nq_l / TILE_ROWS);
        p.n_k_tiles = (int)(P->nkv_l / TILE_ROWS);
        p.q_norm = L.q_norm;
        p.k_norm = L.k_norm;
        p.eps = P->eps;
        p.rope = P->rope.as<float>();
        p.half = (int)(P->rot_dim / 2);
        if (P->attn_core == APK_ATTN_CAUSAL) {
            // K (roped) and V rows go into the f16 cache at the rows' positions; the attention core reads them there
            p.kv_k = P->kv->k(layer);
            p.kv_v = P->kv->v(layer);
            p.kv_dim = (int)P->kv->kv_dim;
            p.pos_dev = P->pos.as<uint32_t>();
        } else {
            // attention core stand-in (identity): the roped Q slice, packed here, is wo's input
            p.q_next = act_layout(P->act_q.p, L.wo->ty, autom.m_eff);
            p.q_next_two_level = autom.two_level;
            p.q_next_need_sum = needs_sum(L.wo->ty);
        }
        return launch(W, p, q8, L.wo);
    }
    // the attention core over the cache: its result, packed, is wo's input
    int attention(PlanLayer &L, uint32_t layer) {
        const ActLayout next = act_layout(P->act_q.p, L.wo->ty, autom.m_eff);
        return launch_attention(c, P->kv, layer, P->qkv.as<float>(), (int)(P->nq_l + 2 * P->nkv_l), m, P->nq_l / TILE_ROWS,
                                P->pos.as<uint32_t>(), 0u, P->scale, P->attn_part.as<float>(), P->attn_out.as<float>(),
                                (int)P->nq_l, &next, autom.two_level, needs_sum(L.wo->ty));
    }
    // next_*: the matvec that will read the updated rows through an RMSNorm (null: none)
    int residual(DevMatrix *W, void *records, const DevMatrix *next_W = nullptr, const float *next_gamma = nullptr,
                 ActMode next_mode = ActMode{0, 1}) {
        const uint32_t H = P->hidden;
        MvParams p{};
        use_records(c, W, autom, records, &p);
        p.xin.index = -1;
        have_sumsq = false;
        if (uses_xch(c)) {
            // partial sums straight into every rank's exchange buffer; the kernel that reads the
            // residual next gathers them in its prologue
            p.epi = EPI_PEERS;
            p.xch = c->xch;
            p.xch_row = (int)H;
            p.resid = P->x[cur].as<float>();  // rank 0 adds the old rows into its slot
            p.ldr = (int)H;
            p.xout = XchSeq{n_xch, per_token()};
            pending_xch = n_xch++;
            return launch(W, p, autom, next_W);
        }
        if (c->world > 1) {
            p.epi = EPI_STORE;
            p.y = P->yp.as<float>();
            p.ldy = (int)H;
            APK_TRY(launch(W, p, autom, nullptr));
            APK_TRY(nccl_allreduce(c, P->yp.as<float>(), (size_t)m * H));
            pending_add = true;
            return APK_OK;
        }
        p.epi = EPI_ADD;
        p.y = P->x[cur].as<float>();
        p.ldy = (int)H;
        p.resid = P->x[cur].as<float>();
        p.ldr = (int)H;
        if (next_W && c->fuse_norm != 0 && H % 32 == 0) {
            p.nq_sumsq = P->sumsq.as<double>();
            have_sumsq = true;
            if (can_prenorm(next_W, next_mode)) {
                p.nq_gamma = next_gamma;
                p.nq_act = act_layout(P->act_h.p, next_W->ty, next_mode.m_eff);
                p.nq_two_level = next_mode.two_level;
                p.nq_need_sum = needs_sum(next_W->ty);
                prenormed_for = next_W;
                prenormed_m_eff = next_mode.m_eff;
            }
        }
        return launch(W, p, autom, next_W);
    }
    int wo(PlanLayer &L) { return residual(L.wo, P->act_q.p, L.gateup, L.ffn_norm, q8); }
    int gateup(PlanLayer &L, bool advance = true) {
        MvParams p{};
        APK_TRY(normed_input(L.gateup, L.ffn_norm, q8, &p, advance));
        p.epi = EPI_SWIGLU;
        p.act_next = act_layout(P->act_d.p, L.down->ty, autom.m_eff);
        p.next_two_level = autom.two_level;
        p.next_need_sum = needs_sum(L.down->ty);
        p.ffn = (int)P->ffn_l;
        return launch(L.gateup, p, q8, L.down);
    }
    // after down comes the next layer's Q|K|V, or the output head
    int down(PlanLayer &L, PlanLayer *next) {
        if (next) return residual(L.down, P->act_d.p, next->qkv, next->attn_norm, q8);
        return residual(L.down, P->act_d.p, P->head, P->out_norm, autom);
    }
    int head(bool advance = true) {
        // finish_hidden: rmsnorm + output.matmul(x, m) (QuantMat::matmul: Q8 at m == 1, f32 dots above);
        // the output-normed rows are kept: TokenOut::Rows hands them to the caller
        MvParams p{};
        APK_TRY(normed_input(P->head, P->out_norm, autom, &p, advance, P->hidden_out.as<float>()));
        p.epi = EPI_STORE;
        p.y = P->logits.as<float>();
        p.ldy = (int)P->vocab_l;
        return launch(P->head, p, autom, nullptr);
    }
};

// x <- embedding row of a token (id on the device, or given).
int launch_embed(apk_ctx *c, Plan *P, const uint32_t *token_dev, uint32_t token, float *x) {
    const DevMatrix *E = P->embd;
    if (!E) return fail(APK_ERR_INVALID_ARG, "the request names no embedding table");
    EmbedParams ep{};
    ep.W = E->d;
    ep.ty = (int)E->ty;
    ep.nb = E->nb;
    ep.n_rows = (int)E->n_out;
    ep.tile_bytes = E->tile_bytes;
    ep.token_dev = token_dev;
    ep.token = token;
    ep.x = x;
    ep.err = c->d_err;
    const int threads = ty_b32((int)E->ty) ? E->nb * 8 : (E->nb / 8) * (ty_k45((int)E->ty) ? 32 : 16);
    embed_row_kernel<<<(threads + 255) / 256, 256, 0, c->stream>>>(ep);
    CUDA_TRY(cudaGetLastError());
    c->st.launches++;
    return APK_OK;
}

// Enqueue one token's work on the stream (called under capture).
int enqueue_token(apk_ctx *c, Plan *P, uint32_t m, int argmax, int *n_launches) {
    const uint64_t l0 = c->st.launches;
    c->launch_no = 0;  // launches are numbered within the token (error reports, parity instrumentation)
    c->prev_mv_exclusive = false;
    TokenLaunch T(c, P, m);
    CUDA_TRY(cudaMemcpyAsync(P->x[0].p, P->xin.p, (size_t)m * P->hidden * 4, cudaMemcpyDeviceToDevice, c->stream));
    for (uint32_t l = 0; l < P->n_layers; ++l) {
        PlanLayer &L = P->L[l];
        APK_TRY(T.qkv(L, true, l));
        if (P->attn_core == APK_ATTN_CAUSAL) APK_TRY(T.attention(L, l));
        APK_TRY(T.wo(L));
        APK_TRY(T.gateup(L));
        APK_TRY(T.down(L, l + 1 < P->n_layers ? &P->L[l + 1] : nullptr));
    }
    APK_TRY(T.head());
    const float *lg = P->logits.as<float>();
    if (c->world > 1) {
        const int rc = g_nccl.AllGather(P->logits.p, P->logits_all.p, (size_t)m * P->vocab_l, NCCL_FLOAT32, c->comm, c->stream);
        if (rc) return fail(APK_ERR_NCCL, "ncclAllGather: %s", g_nccl.GetErrorString(rc));
        lg = P->logits_all.as<float>();
    }
    if (argmax) {
        argmax_rows_kernel<<<m, 1024, 0, c->stream>>>(lg, (int)P->vocab_l, c->world, (int)m, P->amax.as<uint32_t>());
        CUDA_TRY(cudaGetLastError());
        c->st.launches++;
    }
    *n_launches = (int)(c->st.launches - l0);
    return APK_OK;
}

int ensure_graph(apk_ctx *c, const apk_token_req *r) {
    if (!plan_matches(c->plan.get(), r)) APK_TRY(build_plan(c, r));
    Plan *P = c->plan.get();
    const int am = r->argmax ? 1 : 0;
    if (P->exec[r->m][am]) return APK_OK;
    cudaGraph_t graph = nullptr;
    const uint64_t launches_before = c->st.launches;
    CUDA_TRY(cudaStreamBeginCapture(c->stream, cudaStreamCaptureModeThreadLocal));
    int n_launch = 0;
    const int rc = enqueue_token(c, P, r->m, am, &n_launch);
    const cudaError_t e = cudaStreamEndCapture(c->stream, &graph);
    c->st.launches = launches_before;  // capture launched nothing
    if (rc) {
        if (graph) cudaGraphDestroy(graph);
        return rc;
    }
    if (e != cudaSuccess) return fail(APK_ERR_CUDA, "graph capture: %s", cudaGetErrorString(e));
    const cudaError_t ie = cudaGraphInstantiate(&P->exec[r->m][am], graph, 0);
    cudaGraphDestroy(graph);
    if (ie != cudaSuccess) return fail(APK_ERR_CUDA, "graph instantiate: %s", cudaGetErrorString(ie));
    P->launches[r->m][am] = n_launch;
    return APK_OK;
}

int validate_token_req(apk_ctx *c, const apk_token_req *r) {
    if (!r) return fail(APK_ERR_INVALID_ARG, "decode: null request");
    c->st.decode_attempts++;
    if (r->m == 0 || r->m > APK_MAX_M) return decline_decode(c, APK_DECLINE_UNSUPPORTED_SHAPE, "m = %u is outside 1..8", r->m);
    if (r->attn_core != APK_ATTN_IDENTITY && r->attn_core != APK_ATTN_CAUSAL)
        return decline_decode(c, APK_DECLINE_MISSING_CAPABILITY, "attention core %u is not built into this library", r->attn_core);
    if (r->attn_core == APK_ATTN_CAUSAL && !r->kv) return decline_decode(c, APK_ERR_INVALID_ARG, "attention core without a KV cache");
    if (r->attn_core == APK_ATTN_CAUSAL && (uint64_t)r->pos + r->m > r->kv->capacity)  // the caller's CPU path grows its own cache
        return decline_decode(c, APK_DECLINE_INVALID_STATE, "positions %u..%u are past the cache capacity %u", r->pos, r->pos + r->m - 1,
                              r->kv->capacity);
    const bool by_token = r->use_token && r->embd.w && r->m == 1;
    if ((!r->x && !by_token) || (r->rot_dim && !r->rope)) return decline_decode(c, APK_ERR_INVALID_ARG, "missing input rows or rope table");
    return APK_OK;
}

}  // namespace

extern "C" {

int apk_decode_token(apk_ctx *c, const apk_token_req *r, apk_token_out *out) {
    if (!c || !out) return fail(APK_ERR_INVALID_ARG, "decode: null argument");
    std::lock_guard<std::mutex> g(c->mu);
    CUDA_TRY(cudaSetDevice(c->device));
    APK_TRY(validate_token_req(c, r));
    if (r->argmax ? !out->argmax : !out->logits) return decline_decode(c, APK_ERR_INVALID_ARG, "missing output buffer");
    const bool by_token = r->use_token && r->embd.w && r->m == 1;
    if (by_token && r->token_id >= r->embd.n_out)
        return decline_decode(c, APK_ERR_INVALID_ARG, "token %u out of vocabulary %u", r->token_id, r->embd.n_out);
    const uint64_t t0 = now_ns();
    APK_TRY(ensure_graph(c, r));
    Plan *P = c->plan.get();
    const uint32_t m = r->m, H = P->hidden;
    if (by_token)
        APK_TRY(launch_embed(c, P, nullptr, r->token_id, P->xin.as<float>()));
    else
        CUDA_TRY(cudaMemcpyAsync(P->xin.p, r->x, (size_t)m * H * 4, cudaMemcpyHostToDevice, c->stream));
    if (r->rot_dim)
        CUDA_TRY(cudaMemcpyAsync(P->rope.p, r->rope, (size_t)m * (r->rot_dim / 2) * 2 * 4, cudaMemcpyHostToDevice, c->stream));
    CUDA_TRY(cudaMemcpyAsync(P->pos.p, &r->pos, sizeof(uint32_t), cudaMemcpyHostToDevice, c->stream));
    CUDA_TRY(cudaGraphLaunch(P->exec[m][r->argmax ? 1 : 0], c->stream));
    c->st.launches += P->launches[m][r->argmax ? 1 : 0];
    std::vector<float> gathered;
    // TokenOut::Rows: the output-normed hidden rows next to the per-row winners (or logits)
    if (out->hidden)
        CUDA_TRY(cudaMemcpyAsync(out->hidden, P->hidden_out.p, (size_t)m * H * 4, cudaMemcpyDeviceToHost, c->stream));
    if (r->argmax) {
        CUDA_TRY(cudaMemcpyAsync(out->argmax, P->amax.p, m * sizeof(uint32_t), cudaMemcpyDeviceToHost, c->stream));
    } else if (c->world == 1 || m == 1) {
        const void *src = c->world == 1 ? P->logits.p : P->logits_all.p;
        CUDA_TRY(cudaMemcpyAsync(out->logits, src, (size_t)m * P->vocab * 4, cudaMemcpyDeviceToHost, c->stream));
    } else {
        gathered.resize((size_t)m * P->vocab);
        CUDA_TRY(cudaMemcpyAsync(gathered.data(), P->logits_all.p, gathered.size() * 4, cudaMemcpyDeviceToHost, c->stream));
    }
    c->st.encode_ns += now_ns() - t0;
    c->st.calls++;
    APK_TRY(finish(c));
    if (!gathered.empty())  // [rank][m][vocab_l] -> [m][vocab]
        for (int rk = 0; rk < c->world; ++rk)
            for (uint32_t i = 0; i < m; ++i)
                memcpy(out->logits + (size_t)i * P->vocab + (size_t)rk * P->vocab_l,
                       gathered.data() + ((size_t)rk * m + i) * P->vocab_l, (size_t)P->vocab_l * 4);
    c->st.decode_successes++;
    return APK_OK;
}

int apk_decode_profile(apk_ctx *c, const apk_token_req *r, uint32_t reps, float *ms, double *bytes) {
    if (!c || !ms || !bytes || reps == 0) return fail(APK_ERR_INVALID_ARG, "profile: null argument");
    std::lock_guard<std::mutex> g(c->mu);
    CUDA_TRY(cudaSetDevice(c->device));
    APK_TRY(validate_token_req(c, r));
    if (!r->x) return fail(APK_ERR_INVALID_ARG, "this entry point takes its input rows from x");
    APK_TRY(ensure_graph(c, r));
    Plan *P = c->plan.get();
    CUDA_TRY(cudaMemcpyAsync(P->pos.p, &r->pos, sizeof(uint32_t), cudaMemcpyHostToDevice, c->stream));
    const uint32_t m = r->m, H = P->hidden;
    // one real token first, so every activation buffer the kernels read holds sane data
    CUDA_TRY(cudaMemcpyAsync(P->xin.p, r->x, (size_t)m * H * 4, cudaMemcpyHostToDevice, c->stream));
    if (r->rot_dim)
        CUDA_TRY(cudaMemcpyAsync(P->rope.p, r->rope, (size_t)m * (r->rot_dim / 2) * 2 * 4, cudaMemcpyHostToDevice, c->stream));
    CUDA_TRY(cudaGraphLaunch(P->exec[m][r->argmax ? 1 : 0], c->stream));
    APK_TRY(finish(c));
    auto orig_bytes = [](const DevMatrix *W) {
        uint32_t be = 32, bb = 34;
        block_geom(W->src_ty, &be, &bb);
        return (double)W->n_out * (W->n_in / be) * bb;
    };
    for (int kind = 0; kind < 5; ++kind) {
        const uint32_t n_launch = kind == 4 ? 1 : P->n_layers;
        CUDA_TRY(cudaEventRecord(c->ev0, c->stream));
        for (uint32_t rep = 0; rep < reps; ++rep)
            for (uint32_t l = 0; l < n_launch; ++l) {
                PlanLayer &L = P->L[l];
                TokenLaunch T(c, P, m);  // fresh state: reads x[0], never flips buffers
                T.first = false;         // the token counter stays where the token above left it
                T.in_token = false;
                if (uses_xch(c)) {
                    // As in the real token, Q|K|V, gate/up and the head gather an exchange in front of
                    // them.  The slots keep the tagged words of the token's last two exchanges only,
                    // so every gathering launch here reads the last one (its words are there on every
                    // rank, whatever the ranks' relative progress) and the storing launches rewrite
                    // the last two with their own numbers: no wait of this loop depends on a peer.
                    const int last = T.per_token() - 1;
                    T.n_xch = kind == 1 ? last - 1 : last;
                    if ((kind == 0 && l > 0) || kind == 2 || kind == 4) T.pending_xch = last;
                } else if (c->world == 1 && c->fuse_norm != 0 && (kind == 0 ? l > 0 : (kind == 2 || kind == 4))) {
                    T.have_sumsq = true;  // left in place by the token above
                }
                // the launch variants of the real token: inputs that a residual epilogue prepared
                const DevMatrix *nw = kind == 0 ? L.qkv : kind == 2 ? L.gateup : kind == 4 ? P->head : nullptr;
                const ActMode nm = kind == 4 ? T.autom : T.q8;
                if (nw && T.can_prenorm(nw, nm)) {
                    T.prenormed_for = nw;
                    T.prenormed_m_eff = nm.m_eff;
                }
                if (kind == 0) APK_TRY(T.qkv(L, false, l));
                else if (kind == 1) APK_TRY(T.wo(L));
                else if (kind == 2) APK_TRY(T.gateup(L, false));
                else if (kind == 3) APK_TRY(T.down(L, l + 1 < P->n_layers ? &P->L[l + 1] : nullptr));
                else APK_TRY(T.head(false));
            }
        CUDA_TRY(cudaEventRecord(c->ev1, c->stream));
        APK_TRY(finish(c));
        float t = 0.f;
        CUDA_TRY(cudaEventElapsedTime(&t, c->ev0, c->ev1));
        ms[kind] = t / (float)(reps * n_launch);
        const PlanLayer &L0 = P->L[0];
        const DevMatrix *W = kind == 0 ? L0.qkv : kind == 1 ? L0.wo : kind == 2 ? L0.gateup : kind == 3 ? L0.down : P->head;
        // weights as stored in the GGUF file (padding rows of the tiled stream are not counted)
        double wb = orig_bytes(W);
        if (kind == 0 && L0.v) wb += orig_bytes(L0.v);
        if (kind == 2) {
            uint32_t be = 32, bb = 34;
            block_geom(W->src_ty, &be, &bb);
            wb = 2.0 * (double)P->ffn_l * (H / be) * bb;
        }
        const double in_b = (double)m * W->n_in * 4.0;
        const double out_b = kind == 2 ? (double)m * P->ffn_l * 4.0 : (double)m * W->n_out * 4.0;
        bytes[kind] = wb + in_b + out_b;
    }
    c->st.calls++;
    return APK_OK;
}

int apk_debug_token_timeline(apk_ctx *c, const apk_token_req *r, uint64_t *stamps, uint32_t max_launches,
                             uint32_t *n_launches, uint32_t *n_ctas) {
    if (!c || !stamps || !n_launches || !n_ctas || max_launches == 0) return fail(APK_ERR_INVALID_ARG, "timeline: null argument");
    std::lock_guard<std::mutex> g(c->mu);
    CUDA_TRY(cudaSetDevice(c->device));
    APK_TRY(validate_token_req(c, r));
    if (!r->x) return fail(APK_ERR_INVALID_ARG, "this entry point takes its input rows from x");
    APK_TRY(ensure_graph(c, r));
    Plan *P = c->plan.get();
    CUDA_TRY(cudaMemcpyAsync(P->pos.p, &r->pos, sizeof(uint32_t), cudaMemcpyHostToDevice, c->stream));
    const size_t words = (size_t)max_launches * c->n_sm * 8;
    APK_TRY(c->dump.ensure(words * sizeof(uint64_t)));
    CUDA_TRY(cudaMemcpyAsync(P->xin.p, r->x, (size_t)r->m * P->hidden * 4, cudaMemcpyHostToDevice, c->stream));
    if (r->rot_dim)
        CUDA_TRY(cudaMemcpyAsync(P->rope.p, r->rope, (size_t)r->m * (r->rot_dim / 2) * 2 * 4, cudaMemcpyHostToDevice, c->stream));
    CUDA_TRY(cudaMemsetAsync(c->dump.p, 0, words * sizeof(uint64_t), c->stream));
    int nl = 0;
    APK_TRY(enqueue_token(c, P, r->m, 0, &nl));  // untraced pass first: caches and clocks warm
    c->trace = c->dump.as<unsigned long long>();
    c->trace_idx = 0;
    c->trace_cap = max_launches;
    const int rc = enqueue_token(c, P, r->m, 0, &nl);
    c->trace = nullptr;
    *n_launches = c->trace_idx;
    *n_ctas = (uint32_t)c->n_sm;
    if (rc) return rc;
    CUDA_TRY(cudaMemcpyAsync(stamps, c->dump.p, words * sizeof(uint64_t), cudaMemcpyDeviceToHost, c->stream));
    c->st.calls++;
    return finish(c);
}

int apk_decode_replay(apk_ctx *c, const apk_token_req *r, uint32_t iters, float *elapsed_ms) {
    if (!c || !elapsed_ms) return fail(APK_ERR_INVALID_ARG, "replay: null argument");
    std::lock_guard<std::mutex> g(c->mu);
    CUDA_TRY(cudaSetDevice(c->device));
    APK_TRY(validate_token_req(c, r));
    if (!r->x) return fail(APK_ERR_INVALID_ARG, "this entry point takes its input rows from x");
    APK_TRY(ensure_graph(c, r));
    Plan *P = c->plan.get();
    CUDA_TRY(cudaMemcpyAsync(P->pos.p, &r->pos, sizeof(uint32_t), cudaMemcpyHostToDevice, c->stream));
    const int am = r->argmax ? 1 : 0;
    CUDA_TRY(cudaMemcpyAsync(P->xin.p, r->x, (size_t)r->m * P->hidden * 4, cudaMemcpyHostToDevice, c->stream));
    if (r->rot_dim)
        CUDA_TRY(cudaMemcpyAsync(P->rope.p, r->rope, (size_t)r->m * (r->rot_dim / 2) * 2 * 4, cudaMemcpyHostToDevice, c->stream));
    CUDA_TRY(cudaStreamSynchronize(c->stream));
    CUDA_TRY(cudaEventRecord(c->ev0, c->stream));
    for (uint32_t i = 0; i < iters; ++i) CUDA_TRY(cudaGraphLaunch(P->exec[r->m][am], c->stream));
    CUDA_TRY(cudaEventRecord(c->ev1, c->stream));
    c->st.launches += (uint64_t)iters * P->launches[r->m][am];
    c->st.calls++;
    APK_TRY(finish(c));
    CUDA_TRY(cudaEventElapsedTime(elapsed_ms, c->ev0, c->ev1));
    c->st.decode_successes++;
    return APK_OK;
}

int apk_debug_set_wait_limit(apk_ctx *c, uint64_t cycles) {
    if (!c) return fail(APK_ERR_INVALID_ARG, "null context");
    std::lock_guard<std::mutex> g(c->mu);
    CUDA_TRY(cudaSetDevice(c->device));
    CUDA_TRY(cudaStreamSynchronize(c->stream));
    c->wait_limit = cycles ? (long long)std::min<uint64_t>(cycles, (uint64_t)1 << 62) : WAIT_LIMIT_DEFAULT;
    c->plan.reset();  // captured launches carry the old budget
    return APK_OK;
}

int apk_debug_xch_timeout(apk_ctx *c) {
    if (!c) return fail(APK_ERR_INVALID_ARG, "null context");
    std::lock_guard<std::mutex> g(c->mu);
    CUDA_TRY(cudaSetDevice(c->device));
    // Two exchange buffers on this one GPU stand for ranks 0 and 1.  Rank 0's own words carry the
    // exchange's tag, "rank 1" never delivers: the collecting kernel must give up after the wait
    // budget, leave an error word and end normally.
    const int n = 256;
    float *buf[2] = {nullptr, nullptr};
    for (auto &b : buf) {
        CUDA_TRY(cudaMalloc((void **)&b, XCH_BYTES));
        CUDA_TRY(cudaMemsetAsync(b, 0, XCH_BYTES, c->stream));
    }
    APK_TRY(c->y_dev.ensure(n * sizeof(float)));
    const uint32_t one = 1u;
    CUDA_TRY(cudaMemcpyAsync(xch_tok(buf[0]), &one, 4, cudaMemcpyHostToDevice, c->stream));
    std::vector<unsigned long long> own(n, 1ull << 32);  // rank 0's words of exchange 1 (parity 1): tag 1, value 0
    CUDA_TRY(cudaMemcpyAsync(xch_words(buf[0]) + (size_t)1 * XCH_MAX_RANKS * XCH_ROW_FLOATS, own.data(), n * 8,
                             cudaMemcpyHostToDevice, c->stream));
    XchReduceParams rp{};
    rp.xch.slots[0] = buf[0];
    rp.xch.slots[1] = buf[1];
    rp.xch.rank = 0;
    rp.xch.world = 2;
    rp.seq = XchSeq{0, 1};
    rp.xout = c->y_dev.as<float>(); rp.ldxout = n;
    rp.n = n; rp.m = 1;
    rp.err = c->d_err;
    rp.pdl = 0;
    rp.wait_limit = c->wait_limit;
    xch_reduce_kernel<<<1, 256, 0, c->stream>>>(rp);
    cudaError_t e = cudaGetLastError();
    c->st.launches++;
    c->st.calls++;
    const int rc = e == cudaSuccess ? finish(c) : fail(APK_ERR_CUDA, "launch: %s", cudaGetErrorString(e));
    cudaStreamSynchronize(c->stream);
    for (auto &b : buf) cudaFree(b);
    return rc;
}

int apk_debug_token_records(apk_ctx *c, const apk_token_req *r, uint32_t max_records, float *x, float *d, float *sum,
                            int8_t *q, int32_t *meta, uint32_t *n_records, int dots_launch, int32_t *dots,
                            size_t dots_elems) {
    if (!c || !x || !d || !sum || !q || !meta || !n_records || max_records == 0)
        return fail(APK_ERR_INVALID_ARG, "token_records: null argument");
    std::lock_guard<std::mutex> g(c->mu);
    CUDA_TRY(cudaSetDevice(c->device));
    APK_TRY(validate_token_req(c, r));
    if (!r->x) return fail(APK_ERR_INVALID_ARG, "this entry point takes its input rows from x");
    if (c->world != 1 || uses_xch(c)) return fail(APK_DECLINE_INVALID_STATE, "token_records runs on an unsharded context");
    APK_TRY(ensure_graph(c, r));
    Plan *P = c->plan.get();
    CUDA_TRY(cudaMemcpyAsync(P->pos.p, &r->pos, sizeof(uint32_t), cudaMemcpyHostToDevice, c->stream));
    const uint32_t m = r->m, H = P->hidden, nblk = H / 32;
    const size_t x_bytes = (size_t)APK_MAX_M * H * 4;
    const size_t slab = (x_bytes + act_bytes(APK_TY_Q4_K, MAX_M_EFF, H) + 255) & ~(size_t)255;
    APK_TRY(c->dump.ensure(slab * max_records));
    if (dots && dots_elems) {
        APK_TRY(c->misc.ensure(dots_elems * sizeof(int32_t)));
        CUDA_TRY(cudaMemsetAsync(c->misc.p, 0xff, dots_elems * sizeof(int32_t), c->stream));
    }
    CUDA_TRY(cudaMemsetAsync(c->dump.p, 0, slab * max_records, c->stream));
    CUDA_TRY(cudaMemcpyAsync(P->xin.p, r->x, (size_t)m * H * 4, cudaMemcpyHostToDevice, c->stream));
    if (r->rot_dim)
        CUDA_TRY(cudaMemcpyAsync(P->rope.p, r->rope, (size_t)m * (r->rot_dim / 2) * 2 * 4, cudaMemcpyHostToDevice, c->stream));
    c->rec_dump = c->dump.as<uint8_t>();
    c->rec_slab = slab;
    c->rec_idx = 0;
    c->rec_cap = max_records;
    c->rec_meta.clear();
    c->launch_no = 0;
    c->dots_launch = dots && dots_elems ? dots_launch : -1;
    c->dots_dump = dots && dots_elems ? c->misc.as<int32_t>() : nullptr;
    c->dots_cap = dots_elems;
    int nl = 0;
    const int rc = enqueue_token(c, P, m, 0, &nl);
    c->rec_dump = nullptr;
    c->dots_dump = nullptr;
    c->dots_launch = -1;
    const uint32_t n = c->rec_idx;
    *n_records = n;
    if (rc) {
        cudaStreamSynchronize(c->stream);
        return rc;
    }
    std::vector<uint8_t> host(slab * n);
    CUDA_TRY(cudaMemcpyAsync(host.data(), c->dump.p, host.size(), cudaMemcpyDeviceToHost, c->stream));
    if (dots && dots_elems)
        CUDA_TRY(cudaMemcpyAsync(dots, c->misc.p, dots_elems * sizeof(int32_t), cudaMemcpyDeviceToHost, c->stream));
    c->st.calls++;
    APK_TRY(finish(c));
    // per record: x [APK_MAX_M][H] | d, sum [MAX_M_EFF][H/32] | q [MAX_M_EFF][H]; meta = {rows, two-level, launch, K-step}
    for (uint32_t i = 0; i < n; ++i) {
        const RecMeta &mt = c->rec_meta[i];
        const uint8_t *sl = host.data() + slab * i;
        memcpy(x + (size_t)i * APK_MAX_M * H, sl, (size_t)m * H * 4);
        ActLayout L;
        L.base = nullptr; L.ke = mt.ke; L.m_eff = mt.m_eff;
        const int kt = L.kt(), mp = L.mp(), rec = L.rec_bytes(), qb = L.q_bytes();
        const uint8_t *recs = sl + x_bytes;
        for (int row = 0; row < mt.m_eff; ++row)
            for (uint32_t b = 0; b < nblk; ++b) {
                const uint8_t *rr = recs + (size_t)(b / kt) * rec;
                const int bl = (int)(b % kt);
                int8_t *qo = q + ((size_t)i * MAX_M_EFF + row) * H + (size_t)b * 32;
                memcpy(qo, rr + ((bl * 2 + 0) * mt.m_eff + row) * 16, 16);
                memcpy(qo + 16, rr + ((bl * 2 + 1) * mt.m_eff + row) * 16, 16);
                memcpy(d + ((size_t)i * MAX_M_EFF + row) * nblk + b, rr + qb + (bl * mp + row) * 4, 4);
                memcpy(sum + ((size_t)i * MAX_M_EFF + row) * nblk + b, rr + qb + (kt * mp + bl * mp + row) * 4, 4);
            }
        meta[4 * i] = mt.m_eff; meta[4 * i + 1] = mt.two_level; meta[4 * i + 2] = mt.launch; meta[4 * i + 3] = mt.ke;
    }
    return APK_OK;
}

int apk_decode_greedy(apk_ctx *c, const apk_token_req *r, uint32_t n_tokens, const float *rope, uint32_t *tokens_out) {
    if (!c || !r || !tokens_out || (r->rot_dim && !rope)) return fail(APK_ERR_INVALID_ARG, "greedy: null argument");
    if (n_tokens == 0) return APK_OK;
    std::lock_guard<std::mutex> g(c->mu);
    CUDA_TRY(cudaSetDevice(c->device));
    apk_token_req q = *r;  // the chain is argmax decode by token id, whatever the caller left in those fields
    q.argmax = 1;
    q.use_token = 1;
    q.rope = rope;
    APK_TRY(validate_token_req(c, &q));
    if (q.m != 1 || !q.embd.w) return decline_decode(c, APK_DECLINE_UNSUPPORTED_SHAPE, "the greedy chain takes one row and an embedding table");
    if (q.token_id >= q.embd.n_out) return decline_decode(c, APK_ERR_INVALID_ARG, "token %u out of vocabulary %u", q.token_id, q.embd.n_out);
    if (n_tokens > 65536) return decline_decode(c, APK_DECLINE_UNSUPPORTED_SHAPE, "at most 65536 chained tokens per call");
    if (q.attn_core == APK_ATTN_CAUSAL && (uint64_t)q.pos + n_tokens > q.kv->capacity)
        return decline_decode(c, APK_DECLINE_INVALID_STATE, "the chain of %u tokens from position %u runs past the cache capacity %u", n_tokens,
                              q.pos, q.kv->capacity);
    const uint64_t t0 = now_ns();
    APK_TRY(ensure_graph(c, &q));
    Plan *P = c->plan.get();
    const int row = (int)(q.rot_dim / 2) * 2;
    // chain state: token | step | hist[n] | rope rows [n][row]
    const size_t hist_off = 64, rope_off = (hist_off + (size_t)n_tokens * 4 + 255) & ~(size_t)255;
    const size_t need = rope_off + (size_t)n_tokens * std::max(row, 1) * 4;
    if (need > P->chain.cap) {
        CUDA_TRY(cudaStreamSynchronize(c->stream));
        APK_TRY(P->chain.ensure(need));
    }
    uint8_t *base = P->chain.as<uint8_t>();
    uint32_t *d_token = reinterpret_cast<uint32_t *>(base), *d_step = d_token + 1;
    uint32_t *d_hist = reinterpret_cast<uint32_t *>(base + hist_off);
    float *d_rope = reinterpret_cast<float *>(base + rope_off);
    const uint32_t init[2] = {q.token_id, 0u};
    CUDA_TRY(cudaMemcpyAsync(d_token, init, sizeof init, cudaMemcpyHostToDevice, c->stream));
    CUDA_TRY(cudaMemcpyAsync(P->pos.p, &q.pos, sizeof(uint32_t), cudaMemcpyHostToDevice, c->stream));
    if (row) {
        CUDA_TRY(cudaMemcpyAsync(d_rope, rope, (size_t)n_tokens * row * 4, cudaMemcpyHostToDevice, c->stream));
        CUDA_TRY(cudaMemcpyAsync(P->rope.p, d_rope, (size_t)row * 4, cudaMemcpyDeviceToDevice, c->stream));
    }
    ChainParams cp{};
    cp.amax = P->amax.as<uint32_t>();
    cp.token = d_token;
    cp.hist = d_hist;
    cp.step = d_step;
    cp.rope_tab = d_rope;
    cp.rope = P->rope.as<float>();
    cp.row = row;
    cp.n_steps = (int)n_tokens;
    cp.pos = P->pos.as<uint32_t>();
    for (uint32_t i = 0; i < n_tokens; ++i) {
        APK_TRY(launch_embed(c, P, d_token, 0u, P->xin.as<float>()));
        CUDA_TRY(cudaGraphLaunch(P->exec[1][1], c->stream));
        chain_advance_kernel<<<1, 128, 0, c->stream>>>(cp);
        CUDA_TRY(cudaGetLastError());
        c->st.launches += P->launches[1][1] + 1;
    }
    CUDA_TRY(cudaMemcpyAsync(tokens_out, d_hist, (size_t)n_tokens * 4, cudaMemcpyDeviceToHost, c->stream));
    c->st.encode_ns += now_ns() - t0;
    c->st.calls++;
    c->st.decode_attempts += n_tokens - 1;
    APK_TRY(finish(c));
    c->st.decode_successes += n_tokens;
    return APK_OK;
}

int apk_kv_create(apk_ctx *c, uint32_t n_layers, uint32_t kv_dim, uint32_t capacity, apk_kv **out) {
    if (!c || !out || n_layers == 0 || capacity == 0) return fail(APK_ERR_INVALID_ARG, "kv_create: null or empty");
    std::lock_guard<std::mutex> g(c->mu);
    CUDA_TRY(cudaSetDevice(c->device));
    if (kv_dim == 0 || kv_dim % (TILE_ROWS * (uint32_t)c->world))
        return fail(APK_DECLINE_UNSUPPORTED_SHAPE, "kv_dim %u is not whole 128-wide heads per rank", kv_dim);
    auto kv = std::make_unique<apk_kv>();
    kv->n_layers = n_layers;
    kv->kv_dim = kv_dim / (uint32_t)c->world;
    kv->capacity = capacity;
    const size_t bytes = 2 * kv->layer_stride() * n_layers * sizeof(__half);
    CUDA_TRY(cudaMalloc((void **)&kv->base, bytes));
    CUDA_TRY(cudaMemsetAsync(kv->base, 0, bytes, c->stream));
    CUDA_TRY(cudaStreamSynchronize(c->stream));
    *out = kv.release();
    return APK_OK;
}

void apk_kv_destroy(apk_ctx *c, apk_kv *kv) {
    if (!c || !kv) return;
    std::lock_guard<std::mutex> g(c->mu);
    cudaSetDevice(c->device);
    cudaStreamSynchronize(c->stream);
    if (c->plan && c->plan->kv == kv) c->plan.reset();  // its graphs point into the cache
    if (kv->base) cudaFree(kv->base);
    delete kv;
}

static int kv_rows(apk_ctx *c, const apk_kv *kv, uint32_t layer, uint32_t pos0, uint32_t n_pos, uint16_t *k, uint16_t *v, bool write) {
    if (!c || !kv || !k || !v) return fail(APK_ERR_INVALID_ARG, "kv rows: null argument");
    if (layer >= kv->n_layers || (uint64_t)pos0 + n_pos > kv->capacity) return fail(APK_ERR_INVALID_ARG, "kv rows: layer or positions out of range");
    std::lock_guard<std::mutex> g(c->mu);
    CUDA_TRY(cudaSetDevice(c->device));
    const size_t bytes = (size_t)n_pos * kv->kv_dim * sizeof(__half);
    __half *kd = kv->k(layer) + (size_t)pos0 * kv->kv_dim, *vd = kv->v(layer) + (size_t)pos0 * kv->kv_dim;
    if (write) {
        CUDA_TRY(cudaMemcpyAsync(kd, k, bytes, cudaMemcpyHostToDevice, c->stream));
        CUDA_TRY(cudaMemcpyAsync(vd, v, bytes, cudaMemcpyHostToDevice, c->stream));
    } else {
        CUDA_TRY(cudaMemcpyAsync(k, kd, bytes, cudaMemcpyDeviceToHost, c->stream));
        CUDA_TRY(cudaMemcpyAsync(v, vd, bytes, cudaMemcpyDeviceToHost, c->stream));
    }
    CUDA_TRY(cudaStreamSynchronize(c->stream));
    return APK_OK;
}

int apk_kv_read(apk_ctx *c, const apk_kv *kv, uint32_t layer, uint32_t pos0, uint32_t n_pos, uint16_t *k, uint16_t *v) {
    return kv_rows(c, kv, layer, pos0, n_pos, k, v, false);
}

int apk_kv_write(apk_ctx *c, apk_kv *kv, uint32_t layer, uint32_t pos0, uint32_t n_pos, const uint16_t *k, const uint16_t *v) {
    return kv_rows(c, kv, layer, pos0, n_pos, const_cast<uint16_t *>(k), const_cast<uint16_t *>(v), true);
}

int apk_attend(apk_ctx *c, const apk_kv *kv, uint32_t layer, const float *q, uint32_t m, uint32_t n_heads, uint32_t pos,
               float scale, float *out) {
    if (!c || !kv || !q || !out) return fail(APK_ERR_INVALID_ARG, "attend: null argument");
    std::lock_guard<std::mutex> g(c->mu);
    CUDA_TRY(cudaSetDevice(c->device));
    APK_TRY(check_m(m));
    if (c->world != 1) return fail(APK_DECLINE_INVALID_STATE, "attend: stand-alone call runs on an unsharded context");
    const uint32_t n_kv = kv->kv_dim / TILE_ROWS;
    if (layer >= kv->n_layers || n_heads == 0 || n_heads % n_kv || (uint64_t)pos + m > kv->capacity)
        return fail(APK_DECLINE_UNSUPPORTED_SHAPE, "attend: layer %u, %u heads over %u kv heads, positions to %u", layer, n_heads, n_kv, pos + m - 1);
    const size_t qn = (size_t)m * n_heads * TILE_ROWS;
    APK_TRY(c->x_dev.ensure(qn * 4));
    APK_TRY(c->y_dev.ensure(qn * 4));
    APK_TRY(c->misc.ensure((size_t)m * n_heads * attn_splits(c, kv) * ATT_PART * 4));
    CUDA_TRY(cudaMemcpyAsync(c->x_dev.p, q, qn * 4, cudaMemcpyHostToDevice, c->stream));
    APK_TRY(launch_attention(c, kv, layer, c->x_dev.as<float>(), (int)(n_heads * TILE_ROWS), m, n_heads, nullptr, pos, scale,
                             c->misc.as<float>(), c->y_dev.as<float>(), (int)(n_heads * TILE_ROWS), nullptr, 0, 0));
    CUDA_TRY(cudaMemcpyAsync(out, c->y_dev.p, qn * 4, cudaMemcpyDeviceToHost, c->stream));
    c->st.calls++;
    return finish(c);
}

// Benchmark helper: apk_attend's launches over every layer of the cache in turn (distinct memory per
// layer, so a cache larger than L2 is read from HBM), `reps` rounds between one pair of events.
int apk_bench_attend(apk_ctx *c, const apk_kv *kv, const float *q, uint32_t m, uint32_t n_heads, uint32_t pos, float scale,
                     uint32_t reps, float *us_per_layer) {
    if (!c || !kv || !q || !us_per_layer || reps == 0) return fail(APK_ERR_INVALID_ARG, "bench_attend: null argument");
    std::lock_guard<std::mutex> g(c->mu);
    CUDA_TRY(cudaSetDevice(c->device));
    APK_TRY(check_m(m));
    const uint32_t n_kv = kv->kv_dim / TILE_ROWS;
    if (c->world != 1 || n_heads == 0 || n_heads % n_kv || (uint64_t)pos + m > kv->capacity)
        return fail(APK_DECLINE_UNSUPPORTED_SHAPE, "bench_attend: %u heads over %u kv heads, positions to %u", n_heads, n_kv, pos + m - 1);
    const size_t qn = (size_t)m * n_heads * TILE_ROWS;
    APK_TRY(c->x_dev.ensure(qn * 4));
    APK_TRY(c->y_dev.ensure(qn * 4));
    APK_TRY(c->misc.ensure((size_t)m * n_heads * attn_splits(c, kv) * ATT_PART * 4));
    CUDA_TRY(cudaMemcpyAsync(c->x_dev.p, q, qn * 4, cudaMemcpyHostToDevice, c->stream));
    auto pass = [&](uint32_t layer) {
        return launch_attention(c, kv, layer, c->x_dev.as<float>(), (int)(n_heads * TILE_ROWS), m, n_heads, nullptr, pos, scale,
                                c->misc.as<float>(), c->y_dev.as<float>(), (int)(n_heads * TILE_ROWS), nullptr, 0, 0);
    };
    for (uint32_t l = 0; l < kv->n_layers; ++l) APK_TRY(pass(l));
    APK_TRY(finish(c));
    CUDA_TRY(cudaEventRecord(c->ev0, c->stream));
    for (uint32_t r = 0; r < reps; ++r)
        for (uint32_t l = 0; l < kv->n_layers; ++l) APK_TRY(pass(l));
    CUDA_TRY(cudaEventRecord(c->ev1, c->stream));
    APK_TRY(finish(c));
    float ms = 0.f;
    CUDA_TRY(cudaEventElapsedTime(&ms, c->ev0, c->ev1));
    *us_per_layer = ms * 1e3f / (float)(reps * kv->n_layers);
    c->st.calls++;
    return APK_OK;
}

}  // extern "C"
