// Engine methods of the Degavik family (see degavik.cuh): weight upload and the per-layer launch sequence.  The step function,
// step metadata, cache pages, slot / snapshot interface and CUDA graphs are the ones of kemirax_engine.cuh.  Included by
// engine.cu after it.
#pragma once

using namespace b200;

void b200rwkv_engine::dg_load(const StFile& st, KxSizes& z) {
    SeqModel& m = *kx;
    const int W = m.W, nl = (int)m.cfg.layers.size();
    m.embed = kx_up16(kx_host_bf16(st, "embed", m.V, W));
    m.head = kx_up16(kx_host_bf16(st, "head", m.V, W));
    m.final_w = kx_up32(kx_host_f32(st, "final.norm", W));
    m.layers.resize(nl);
    auto rank_of = [&](const std::string& name) {
        const StTensor* t = st.find(name);
        REQUIRE(t && t->shape.size() == 2, B200RWKV_ERR_INVALID, "missing tensor: " + name);
        return (int)t->shape[0];
    };
    // ---- tensors of the layers that own some ----
    for (int i = 0; i < nl; ++i) {
        KxLayer& l = m.layers[i];
        l.c = m.cfg.layers[i];
        const KxLayerCfg& c = l.c;
        if (c.weights_of >= 0) continue;
        const std::string p = "l" + std::to_string(i) + ".";
        const int H_ = c.heads, G_ = c.kv_heads, dk = c.dim, dv = c.vdim;
        REQUIRE(H_ >= 1 && dk >= 1 && dv >= 1, B200RWKV_ERR_INVALID, "config: bad mixer sizes");
        l.norm1_w = kx_up32(kx_host_f32(st, p + "norm1", W));
        l.o = kx_up16(kx_host_bf16(st, p + "mix.o", W, (int64_t)H_ * dv));
        if (c.mixer == KX_RETENTION) {
            auto w = kx_host_bf16(st, p + "mix.q", (int64_t)H_ * dk, W);
            kx_cat(w, kx_host_bf16(st, p + "mix.k", (int64_t)H_ * dk, W));
            kx_cat(w, kx_host_bf16(st, p + "mix.v", (int64_t)H_ * dv, W));
            kx_cat(w, kx_host_bf16(st, p + "mix.g", (int64_t)H_ * dv, W));
            l.proj_n = 2 * H_ * dk + 2 * H_ * dv;
            l.proj = kx_up16(w);
        } else if (c.mixer == KX_DELTA) {
            l.a_rank = rank_of(p + "mix.a1");
            l.g_rank = rank_of(p + "mix.g1");
            l.conv_C = 2 * G_ * dk + H_ * dv;
            auto w = kx_host_bf16(st, p + "mix.q", (int64_t)G_ * dk, W);
            kx_cat(w, kx_host_bf16(st, p + "mix.k", (int64_t)G_ * dk, W));
            kx_cat(w, kx_host_bf16(st, p + "mix.v", (int64_t)H_ * dv, W));
            kx_cat(w, kx_host_bf16(st, p + "mix.b", H_, W));
            kx_cat(w, kx_host_bf16(st, p + "mix.a1", l.a_rank, W));
            kx_cat(w, kx_host_bf16(st, p + "mix.g1", l.g_rank, W));
            l.proj_n = l.conv_C + H_ + l.a_rank + l.g_rank;
            l.proj = kx_up16(w);
            l.a2 = kx_up16(kx_host_bf16(st, p + "mix.a2", (int64_t)H_ * dk, l.a_rank));
            l.a2_b = kx_up32(kx_host_f32(st, p + "mix.dt_bias", (int64_t)H_ * dk));
            l.g2 = kx_up16(kx_host_bf16(st, p + "mix.g2", (int64_t)H_ * dv, l.g_rank));
            l.a_log = kx_up32(kx_host_f32(st, p + "mix.A_log", H_));
            l.norm_w = kx_up32(kx_host_f32(st, p + "mix.norm", dv));
            auto cw = kx_host_f32(st, p + "mix.q.conv", (int64_t)G_ * dk * c.taps);
            auto ck = kx_host_f32(st, p + "mix.k.conv", (int64_t)G_ * dk * c.taps);
            auto cvv = kx_host_f32(st, p + "mix.v.conv", (int64_t)H_ * dv * c.taps);
            cw.insert(cw.end(), ck.begin(), ck.end());
            cw.insert(cw.end(), cvv.begin(), cvv.end());
            l.conv_w = kx_up32(cw);
        } else {
            auto w = kx_host_bf16(st, p + "mix.q", (int64_t)H_ * dk, W);
            kx_cat(w, kx_host_bf16(st, p + "mix.k", (int64_t)G_ * dk, W));
            kx_cat(w, kx_host_bf16(st, p + "mix.v", (int64_t)G_ * dv, W));
            l.proj_n = H_ * dk + G_ * dk + G_ * dv;
            l.proj = kx_up16(w);
            l.qn_w = kx_up32(kx_host_f32(st, p + "mix.q.norm", dk));
            l.kn_w = kx_up32(kx_host_f32(st, p + "mix.k.norm", dk));
            l.talk = kx_up32(kx_host_f32(st, p + "mix.talk", (int64_t)H_ * H_));
            l.temp = kx_up32(kx_host_f32(st, p + "mix.temp", H_));
        }
        if (c.has_mlp) {
            l.norm2_w = kx_up32(kx_host_f32(st, p + "norm2", W));
            if (c.mlp_dense) {        // one gated unit: kept where a routed layer keeps its always-on expert
                l.sh_gu = kx_up16(kx_interleave(kx_host_bf16(st, p + "mlp.gate", c.ff, W), kx_host_bf16(st, p + "mlp.up", c.ff, W), c.ff, W));
                l.sh_down = kx_up16(kx_host_bf16(st, p + "mlp.down", W, c.ff));
            } else {
                const int E = c.experts, ff = c.ff;
                REQUIRE(E >= 1 && E <= 2048 && c.top >= 1 && c.top <= MOE_MAX_TOP && c.top <= E, B200RWKV_ERR_UNSUPPORTED,
                        "config: router sizes out of range (1 <= top <= 8, top <= experts <= 2048)");
                l.router = kx_up16(kx_host_bf16(st, p + "mlp.router", E, W));
                l.corr = kx_up32(kx_host_f32(st, p + "mlp.router.b", E));
                std::vector<uint16_t> gu, dw;
                for (int e = 0; e < E; ++e) {
                    const std::string q = p + "mlp.e" + std::to_string(e) + ".";
                    kx_cat(gu, kx_interleave(kx_host_bf16(st, q + "gate", ff, W), kx_host_bf16(st, q + "up", ff, W), ff, W));
                    kx_cat(dw, kx_host_bf16(st, q + "down", W, ff));
                }
                l.gu = kx_up16(gu); l.down = kx_up16(dw);
                if (c.has_shared) {
                    l.sh_gu = kx_up16(kx_interleave(kx_host_bf16(st, p + "mlp.shared.gate", c.sff, W), kx_host_bf16(st, p + "mlp.shared.up", c.sff, W),
                                                    c.sff, W));
                    l.sh_down = kx_up16(kx_host_bf16(st, p + "mlp.shared.down", W, c.sff));
                }
            }
        }
    }
    // ---- layers that use another layer's tensors; constants and sequence memory of every layer ----
    int qb = 4;
    for (int i = 0; i < nl; ++i) {
        KxLayer& l = m.layers[i];
        const KxLayerCfg own = m.cfg.layers[i];
        if (own.weights_of >= 0) {
            const KxLayerCfg& s = m.cfg.layers[own.weights_of];
            REQUIRE(s.heads == own.heads && s.kv_heads == own.kv_heads && s.dim == own.dim && s.vdim == own.vdim && s.taps == own.taps &&
                        s.has_mlp == own.has_mlp && s.mlp_dense == own.mlp_dense && s.ff == own.ff && s.experts == own.experts &&
                        s.has_shared == own.has_shared && s.sff == own.sff,
                    B200RWKV_ERR_INVALID, "config: a layer with weights_of must have the sizes of the layer it names");
            l = m.layers[own.weights_of];      // the tensors (device pointers); the source has no sequence memory yet or gets its own below
            l.fixed.clear(); l.cache = nullptr; l.cache_D = 0; l.rec_state = nullptr; l.conv_tail = nullptr;
            l.c = own;
        }
    }
    for (int i = 0; i < nl; ++i) {
        KxLayer& l = m.layers[i];
        const KxLayerCfg& c = l.c;
        const int H_ = c.heads, G_ = c.kv_heads, dk = c.dim, dv = c.vdim;
        REQUIRE(dv <= 1024, B200RWKV_ERR_UNSUPPORTED, "vdim must be <= 1024");
        if (c.mixer == KX_RETENTION || c.mixer == KX_DELTA) {
            REQUIRE(std::max(retention_smem_bytes(dk, dv), delta_rule_smem_bytes(dk, dv)) <= 200 * 1024, B200RWKV_ERR_UNSUPPORTED,
                    "head state too large for shared memory");
            l.rec_state = (float*)dalloc((size_t)S * H_ * dk * dv * 4);
            l.fixed.push_back({l.rec_state, (size_t)H_ * dk * dv});
        }
        if (c.mixer == KX_RETENTION) {
            std::vector<float> d(H_);
            for (int h = 0; h < H_; ++h) d[h] = (float)c.decay[h];
            l.decay = kx_up32(d);
        }
        if (c.mixer == KX_RETENTION || c.mixer == KX_WINDOW) {
            std::vector<double> fr(std::max(c.rot.dims / 2, 1), 0.0);
            for (int f = 0; f < c.rot.dims / 2; ++f) fr[f] = std::pow(c.rot.base, -2.0 * f / c.rot.dims);
            l.freq_d = (double*)dalloc(fr.size() * 8, false);
            CK(cudaMemcpy(l.freq_d, fr.data(), fr.size() * 8, cudaMemcpyHostToDevice));
        }
        if (c.mixer == KX_DELTA) {
            const size_t tail = (size_t)(c.taps - 1) * l.conv_C;
            l.conv_tail = (float*)dalloc(std::max<size_t>((size_t)S * tail, 1) * 4);
            l.fixed.push_back({l.conv_tail, tail});
            z.n_cv = std::max(z.n_cv, (size_t)l.conv_C); z.n_z = std::max(z.n_z, (size_t)H_ * dk);
            z.n_gl = std::max(z.n_gl, (size_t)H_ * dv);
        }
        if (c.mixer == KX_WINDOW) {
            l.cache_D = G_ * (dk + dv);
            l.cache = (float*)dalloc((size_t)m.npages * m.page * l.cache_D * 4);
            while (qb > 1 && window_attn_smem(qb, H_, dk, dv, 1) > 128 * 1024) qb /= 2;
            REQUIRE(window_attn_smem(1, H_, dk, dv, 1) <= 200 * 1024, B200RWKV_ERR_UNSUPPORTED, "attention heads too large for shared memory");
            z.n_q = std::max(z.n_q, (size_t)H_ * dk);
        }
        z.n_pr = std::max(z.n_pr, (size_t)l.proj_n); z.n_vout = std::max(z.n_vout, (size_t)H_ * dv);
        if (c.has_mlp) {
            if (c.mlp_dense) z.n_ys = std::max(z.n_ys, (size_t)c.ff);
            else {
                z.n_yc = std::max(z.n_yc, (size_t)c.ff); z.n_rl = std::max(z.n_rl, (size_t)c.experts);
                z.max_top = std::max(z.max_top, c.top); z.max_E = std::max(z.max_E, c.experts);
                if (c.has_shared) z.n_ys = std::max(z.n_ys, (size_t)c.sff);
            }
        }
    }
    m.qb_prompt = qb;
    for (KxLayer& l : m.layers)
        if (l.c.mixer == KX_WINDOW) {              // as many key / value heads per tile load as fit beside the chunk's rows
            l.wa_gt = l.c.kv_heads;
            while (l.wa_gt > 1 && window_attn_smem(qb, l.c.heads, l.c.dim, l.c.vdim, l.wa_gt) > 160 * 1024) l.wa_gt = (l.wa_gt + 1) / 2;
        }
    CK(cudaFuncSetAttribute(retention_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
    CK(cudaFuncSetAttribute(delta_rule_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
    CK(cudaFuncSetAttribute(window_attn_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
    // the largest cluster the attention launch may ask for: what the device can co-schedule at this layer's shared memory
    m.max_split = 8;
    for (const KxLayer& l : m.layers) {
        if (l.c.mixer != KX_WINDOW) continue;
        int cl = 8;
        for (; cl > 1; cl >>= 1) {
            cudaLaunchConfig_t cfg;
            memset(&cfg, 0, sizeof(cfg));
            cfg.gridDim = dim3(cl); cfg.blockDim = dim3(WA_THREADS);
            cfg.dynamicSmemBytes = window_attn_smem(qb, l.c.heads, l.c.dim, l.c.vdim, l.wa_gt);
            cudaLaunchAttribute at;
            at.id = cudaLaunchAttributeClusterDimension;
            at.val.clusterDim.x = (unsigned)cl; at.val.clusterDim.y = 1; at.val.clusterDim.z = 1;
            cfg.attrs = &at; cfg.numAttrs = 1;
            int n = 0;
            if (cudaOccupancyMaxActiveClusters(&n, window_attn_kernel, &cfg) == cudaSuccess && n > 0) break;
            cudaGetLastError();
        }
        m.max_split = std::min(m.max_split, cl);
    }
    m.wa_ctas_prompt = m.wa_ctas_decode = 8;
    for (const KxLayer& l : m.layers) {
        if (l.c.mixer != KX_WINDOW) continue;
        const int G_ = l.c.kv_heads, H_ = l.c.heads;
        const int thr_p = std::min(l.wa_gt, G_) * cdiv(qb * (H_ / G_), WA_RB) >= 16 ? WA_THREADS : 256;
        const int thr_d = std::min(l.wa_gt, G_) * cdiv(H_ / G_, WA_RB) >= 16 ? WA_THREADS : 256;
        int np = 1, nd = 1;
        CK(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&np, window_attn_kernel, thr_p, window_attn_smem(qb, H_, l.c.dim, l.c.vdim, l.wa_gt)));
        CK(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&nd, window_attn_kernel, thr_d, window_attn_smem(1, H_, l.c.dim, l.c.vdim, l.wa_gt)));
        m.wa_ctas_prompt = std::max(1, std::min(m.wa_ctas_prompt, np));
        m.wa_ctas_decode = std::max(1, std::min(m.wa_ctas_decode, nd));
    }
    REQUIRE((size_t)W * 4 <= 200 * 1024, B200RWKV_ERR_UNSUPPORTED, "width too large for the output-norm kernel");
    CK(cudaFuncSetAttribute(norm_add_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
}

// one layer: x += rms(mixer(x)) * w1, then x += rms(ff(x)) * w2
void b200rwkv_engine::dg_enqueue_layer(cudaStream_t s, KxLayer& l, int rows, int nslot_grid, bool decode, int nsplit, Profiler* prof) {
    SeqModel& m = *kx;
    const int W = m.W;
    MetaView mv{d_meta, maxT, S};
    const int* cntT = d_meta;
    const KxLayerCfg& c = l.c;
    const int H_ = c.heads, G_ = c.kv_heads, dk = c.dim, dv = c.vdim;
    auto lin = [&](const float* X, int ldx, const __nv_bfloat16* Wt, float* Y, int ldy, int N_, int K_, int epi = LE_STORE, const float* bias = nullptr) {
        LinParams p;
        memset(&p, 0, sizeof(p));
        p.X = X; p.ldx = ldx; p.W = Wt; p.Y = Y; p.ldy = ldy; p.N = N_; p.K = K_; p.cnt = cntT; p.epi = epi; p.bias = bias;
        return p;
    };
    const int PN = l.proj_n;
    kx_lin(s, prof, lin(m.x, W, l.proj, m.pr, PN, PN, W), rows, 1);
    if (c.mixer == KX_RETENTION) {
        RetentionParams rp{m.pr, m.pr + H_ * dk, m.pr + 2 * H_ * dk, m.pr + 2 * H_ * dk + H_ * dv, PN, l.rec_state, m.vout, H_ * dv, l.decay, l.freq_d,
                           H_, dk, dv, c.rot.dims, 1.f / sqrtf((float)dk), m.cfg.eps, mv, m.sm};
        if (dk <= RET_REG_MAX_DK && dv <= RET_REG_MAX_DV) {       // usual head sizes: the state column lives in registers
            auto kern = dk <= 32 ? retention_reg_kernel<32> : (dk <= 64 ? retention_reg_kernel<64> : retention_reg_kernel<128>);
            launch_k(kern, dim3(H_, nslot_grid), dim3(rup(dv, 32)), 0, rp, KC_WKV, s, prof);
        } else {
            launch_k(retention_kernel, dim3(H_, nslot_grid), dim3(rup(dv, 32)), retention_smem_bytes(dk, dv), rp, KC_WKV, s, prof);
        }
    } else if (c.mixer == KX_DELTA) {
        const int C_ = l.conv_C;
        ShortConvParams cp{m.pr, PN, m.cv, C_, l.conv_w, l.conv_tail, C_, c.taps, mv};
        launch_k(short_conv_kernel, dim3(rows, cdiv(C_, 256)), dim3(256), 0, cp, KC_OTHER, s, prof);
        if (c.taps > 1) launch_k(conv_commit_kernel, dim3(nslot_grid, cdiv(C_, 256)), dim3(256), 0, cp, KC_OTHER, s, prof);
        kx_lin(s, prof, lin(m.pr + C_ + H_, PN, l.a2, m.z, H_ * dk, H_ * dk, l.a_rank, LE_STORE, l.a2_b), rows, 1);
        kx_lin(s, prof, lin(m.pr + C_ + H_ + l.a_rank, PN, l.g2, m.gl, H_ * dv, H_ * dv, l.g_rank), rows, 1);
        DeltaRuleParams dp{m.cv, m.cv + G_ * dk, m.cv + 2 * G_ * dk, C_, m.z, H_ * dk, m.pr + C_, PN, m.gl, H_ * dv, l.a_log, l.norm_w, l.rec_state,
                           m.vout, H_ * dv, H_, G_, dk, dv, 1.f / sqrtf((float)dk), 1e-6f, m.cfg.eps, mv};
        if (dk <= DR_REG_MAX_DK && dv <= DR_REG_MAX_DV) {
            auto kern = dk <= 32 ? delta_rule_reg_kernel<32> : (dk <= 64 ? delta_rule_reg_kernel<64> : delta_rule_reg_kernel<128>);
            launch_k(kern, dim3(H_, nslot_grid), dim3(rup(dv, 32)), 0, dp, KC_WKV, s, prof);
        } else {
            launch_k(delta_rule_kernel, dim3(H_, nslot_grid), dim3(rup(dv, 32)), delta_rule_smem_bytes(dk, dv), dp, KC_WKV, s, prof);
        }
    } else {
        AttnPrepParams ap{m.pr, m.pr + H_ * dk, m.pr + H_ * dk + G_ * dk, PN, m.q, H_ * dk, l.cache, m.d_table, m.npages, m.page, l.qn_w, l.kn_w,
                          l.temp, l.freq_d, H_, G_, dk, dv, c.rot.dims, c.scale, m.cfg.eps, mv, m.sm};
        launch_k(attn_prep_kernel, dim3(rows), dim3(128), 0, ap, KC_OTHER, s, prof);
        const int qb = decode ? 1 : m.qb_prompt;
        WindowAttnParams wp{m.q, H_ * dk, l.cache, m.d_table, m.npages, m.page, m.vout, H_ * dv, l.talk, H_, G_, dk, dv, c.window, c.keep_first,
                            c.softcap, qb, l.wa_gt, nsplit, mv, m.sm};
        launch_cluster = nsplit;
        // 16 warps where the score / value phases have a work item (four rows of one key head) for each, 8 otherwise
        const int items = std::min(l.wa_gt, G_) * cdiv(qb * (H_ / G_), WA_RB);      // qb = 1 in decode steps
        launch_k(window_attn_kernel, dim3((decode ? rows : cdiv(rows, qb) + nslot_grid) * nsplit), dim3(items >= 16 ? WA_THREADS : 256),
                 window_attn_smem(qb, H_, dk, dv, l.wa_gt), wp, KC_WKV, s, prof);
    }
    kx_lin(s, prof, lin(m.vout, H_ * dv, l.o, m.y, W, W, H_ * dv), rows, 1);
    {
        NormAddParams na{m.x, m.y, nullptr, nullptr, nullptr, 0, nullptr, l.norm1_w, m.cfg.eps, W, mv};
        launch_k(norm_add_kernel, dim3(rows), dim3(NORM_THREADS), 0, na, KC_LN, s, prof);
    }
    if (!c.has_mlp) return;
    if (c.mlp_dense) {
        kx_lin(s, prof, lin(m.x, W, l.sh_gu, m.ys, c.ff, 2 * c.ff, W, LE_GLU_SILU), rows, 1);
        kx_lin(s, prof, lin(m.ys, c.ff, l.sh_down, m.y, W, W, c.ff), rows, 1);
        NormAddParams na{m.x, m.y, nullptr, nullptr, nullptr, 0, nullptr, l.norm2_w, m.cfg.eps, W, mv};
        launch_k(norm_add_kernel, dim3(rows), dim3(NORM_THREADS), 0, na, KC_LN, s, prof);
        return;
    }
    const int E = c.experts, ff = c.ff;
    MoeRouteParams rp{m.x, W, l.router, W, l.corr, E, c.top, m.sel, m.wgt, mv, MOE_TOP_LOGITS};
    launch_k(moe_route_kernel, dim3(rows), dim3(MOE_ROUTE_THREADS), moe_route_smem(W, E), rp, KC_OTHER, s, prof);
    MoeGroupParams gp{m.sel, c.top, E, m.cnt, m.off, m.list, m.row_of, mv};
    launch_k(moe_group_kernel, dim3(1), dim3(256), ((size_t)E * 2 + (size_t)maxT * c.top) * 4, gp, KC_OTHER, s, prof);
    LinParams p1 = lin(m.x, W, l.gu, m.yc, ff, 2 * ff, W, LE_GLU_SILU);
    p1.w_gstride = (long long)2 * ff * W; p1.cnt = m.cnt; p1.cnt_gstride = 1; p1.off = m.off; p1.xlist = m.list;
    kx_lin(s, prof, p1, rows, E);
    LinParams p2 = lin(m.yc, ff, l.down, m.dn, W, W, ff);
    p2.w_gstride = (long long)W * ff; p2.cnt = m.cnt; p2.cnt_gstride = 1; p2.off = m.off;
    kx_lin(s, prof, p2, rows, E);
    if (c.has_shared) {
        kx_lin(s, prof, lin(m.x, W, l.sh_gu, m.ys, c.sff, 2 * c.sff, W, LE_GLU_SILU), rows, 1);
        kx_lin(s, prof, lin(m.ys, c.sff, l.sh_down, m.ds, W, W, c.sff), rows, 1);
    }
    NormAddParams na{m.x, nullptr, m.dn, m.row_of, m.wgt, c.top, c.has_shared ? m.ds : nullptr, l.norm2_w, m.cfg.eps, W, mv};
    launch_k(norm_add_kernel, dim3(rows), dim3(NORM_THREADS), (size_t)W * 4, na, KC_LN, s, prof);
}
