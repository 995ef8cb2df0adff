// Softmax attention over a paged key / value cache with a sliding window that keeps the first tokens, capped scores and a
// mix of the heads' attention weights.
//
// H query heads, G key / value heads (query head h reads head h / (H / G)).  Per layer and token the cache row holds the G
// keys (normed and rotated) followed by the G values: D = G (dk + dv) floats.  For query position i and key position j
//     visible(i, j) = j <= i and (i - j < window or j < keep_first)                       (kept tokens keep their positions)
//     s_h(i, j) = cap * tanh((q_h(i) . k(j)) * scale * temp_h / cap)                      (cap <= 0: no cap)
//     p_h(i, .) = softmax over the visible j;    p'_h = sum_g M[h, g] p_g;    o_h(i) = sum_j p'_h(i, j) v(j)
// Because the mix needs every head's NORMALISED weight of a key, a CTA owns all heads of its query tokens and walks the
// visible keys twice: first the running maximum and sum of every (token, head) row, then the weights themselves, mixed and
// applied to the values tile by tile.  Keys outside the window are never touched: the walk covers the kept prefix and the
// window of the chunk's tokens (one range when they meet).
//
//   attn_prep_kernel     per token: q heads = rms(q) * w_q, rotated, times scale * temp_h -> q buffer;  k heads = rms(k) * w_k,
//                        rotated, and v -> the cache row of (slot, position).  Rotation pairs entry 2i with 2i + 1 on the first
//                        `dims` entries of a head; angle = position * frequency in f32.
//   window_attn_kernel   one CTA per chunk of consecutive tokens of one sequence (SeqMeta chunks), all heads; 32-key tiles of one
//                        key / value head at a time in shared memory; scores, softmax, mix and the weighted sums in f32.
#pragma once
#include <cuda_runtime.h>
#include <math_constants.h>
#include "common.cuh"
#include "latent_attn.cuh"

namespace b200 {

struct AttnPrepParams {
    const float* q; const float* k; const float* v; int ld;      // projection rows: q [H * dk], k [G * dk], v [G * dv]
    float* qo; int ldq;                           // [T, H * dk]
    float* cache;                                 // [pages][page][G * dk + G * dv]
    const int* table; int stride; int page;
    const float* wq; const float* wk;             // [dk] norm weights
    const float* temp;                            // [H]
    const float* freq;                            // [dims / 2]
    int H, G, dk, dv, dims;
    float scale, eps;
    MetaView meta; SeqMeta sm;
};

__global__ void __launch_bounds__(128) attn_prep_kernel(const AttnPrepParams p) {
    const int t = blockIdx.x;
    if (t >= p.meta.T()) return;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
    const int slot = p.meta.tok_slot()[t], ipos = p.sm.tok_pos()[t];
    const float pos = (float)ipos;
    const int D = p.G * (p.dk + p.dv);
    float* row = p.cache + ((size_t)p.table[(size_t)slot * p.stride + ipos / p.page] * p.page + ipos % p.page) * D;
    for (int hh = warp; hh < p.H + p.G; hh += nw) {
        const bool isq = hh < p.H;
        const int h = isq ? hh : hh - p.H;
        const float* src = (isq ? p.q : p.k) + (size_t)t * p.ld + (size_t)h * p.dk;
        float* dst = isq ? p.qo + (size_t)t * p.ldq + (size_t)h * p.dk : row + (size_t)h * p.dk;
        const float* w = isq ? p.wq : p.wk;
        float ss = 0.f;
        for (int i = lane; i < p.dk; i += 32) ss = fmaf(src[i], src[i], ss);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
        const float r = 1.f / sqrtf(ss / (float)p.dk + p.eps);
        const float mul = isq ? p.scale * p.temp[h] : 1.f;
        for (int i = lane; i < p.dk; i += 32) {
            float val;
            if (i < p.dims) {
                const int e = i & ~1;
                const float a = pos * p.freq[i >> 1];
                const float cs = cosf(a), sn = sinf(a);
                const float u = src[e] * r * w[e], v = src[e + 1] * r * w[e + 1];
                val = (i & 1) ? v * cs + u * sn : u * cs - v * sn;
            } else {
                val = src[i] * r * w[i];
            }
            dst[i] = val * mul;
        }
    }
    float* vdst = row + (size_t)p.G * p.dk;
    const float* vsrc = p.v + (size_t)t * p.ld;
    for (int i = threadIdx.x; i < p.G * p.dv; i += blockDim.x) vdst[i] = vsrc[i];
}

struct WindowAttnParams {
    const float* q; int ldq;                      // [T, H * dk] prepared queries
    const float* cache;
    const int* table; int stride; int page;
    float* out; int ldo;                          // [T, H * dv]
    const float* mix;                             // [H][H] weight mix (row = output head)
    int H, G, dk, dv;
    int window, keep;
    float cap;
    int qb;                                       // tokens per chunk the shared memory was sized for
    MetaView meta; SeqMeta sm;
};

constexpr int WA_KT = 32;                          // keys per tile (one per lane in the score phase)
constexpr int WA_THREADS = 256;

__host__ __device__ inline size_t window_attn_smem(int qb, int H, int dk, int dv) {
    const size_t R = (size_t)qb * H, dmax = dk > dv ? dk : dv;
    return (R * dk + R * dv + 2 * R * WA_KT + (size_t)WA_KT * (dmax + 1) + 2 * R + (size_t)H * H + 8) * sizeof(float);
}

__global__ void __launch_bounds__(WA_THREADS) window_attn_kernel(const WindowAttnParams p) {
    const int ch = blockIdx.x;
    if (ch >= p.sm.n_chunks()) return;
    const int t0 = p.sm.chunk_start()[ch], nq = p.sm.chunk_count()[ch];
    const int slot = p.meta.tok_slot()[t0];
    const int pos0 = p.sm.tok_pos()[t0], pos1 = pos0 + nq - 1;
    const int H = p.H, G = p.G, dk = p.dk, dv = p.dv, rep = H / G, R = nq * H;
    const int dmax = dk > dv ? dk : dv, ts = dmax + 1, D = G * (dk + dv);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = WA_THREADS / 32;
    extern __shared__ __align__(16) float wa_smem[];
    const int Rcap = p.qb * H;
    float* sQ = wa_smem;                          // [R][dk]
    float* sO = sQ + (size_t)Rcap * dk;           // [R][dv]
    float* sP = sO + (size_t)Rcap * dv;           // [R][KT] normalised weights of the tile
    float* sM = sP + (size_t)Rcap * WA_KT;        // [R][KT] mixed weights
    float* sT = sM + (size_t)Rcap * WA_KT;        // [KT][ts] key or value tile of one head
    float* sMax = sT + (size_t)WA_KT * ts;        // [R]
    float* sSum = sMax + Rcap;                    // [R]
    float* sMix = sSum + Rcap;                    // [H][H]
    for (int e = threadIdx.x; e < R * dk; e += WA_THREADS) {
        const int r = e / dk, i = e % dk;
        sQ[e] = p.q[(size_t)(t0 + r / H) * p.ldq + (size_t)(r % H) * dk + i];
    }
    for (int e = threadIdx.x; e < R * dv; e += WA_THREADS) sO[e] = 0.f;
    for (int e = threadIdx.x; e < R; e += WA_THREADS) { sMax[e] = -CUDART_INF_F; sSum[e] = 0.f; }
    for (int e = threadIdx.x; e < H * H; e += WA_THREADS) sMix[e] = p.mix[e];
    // key ranges: the kept prefix [0, a_hi) and the window [b_lo, pos1]; one range when they touch
    int seg_lo[2], seg_hi[2], nseg = 1;
    {
        const int a_hi = min(p.keep, pos1 + 1), b_lo = max(0, pos0 - p.window + 1);
        if (a_hi <= 0) { seg_lo[0] = b_lo; seg_hi[0] = pos1 + 1; }
        else if (b_lo <= a_hi) { seg_lo[0] = 0; seg_hi[0] = pos1 + 1; }
        else { seg_lo[0] = 0; seg_hi[0] = a_hi; seg_lo[1] = b_lo; seg_hi[1] = pos1 + 1; nseg = 2; }
    }
    const int* tbl = p.table + (size_t)slot * p.stride;
    __syncthreads();
    for (int pass = 0; pass < 2; ++pass) {
        for (int sg = 0; sg < nseg; ++sg) {
            for (int j0 = seg_lo[sg]; j0 < seg_hi[sg]; j0 += WA_KT) {
                const int nk = min(WA_KT, seg_hi[sg] - j0);
                const int jl = j0 + lane;
                for (int c = 0; c < G; ++c) {
                    __syncthreads();               // the tile buffer is free
                    for (int kt = warp; kt < nk; kt += nw) {
                        const int j = j0 + kt;
                        const float* src = p.cache + ((size_t)tbl[j / p.page] * p.page + j % p.page) * D + (size_t)c * dk;
                        for (int i = lane; i < dk; i += 32) sT[kt * ts + i] = src[i];
                    }
                    __syncthreads();
                    for (int rr = warp; rr < nq * rep; rr += nw) {
                        const int qi = rr / rep, r = qi * H + c * rep + rr % rep;
                        const int pq = pos0 + qi;
                        float s = 0.f;
                        if (lane < nk) {
                            const float* qv = sQ + (size_t)r * dk;
                            const float* kv = sT + lane * ts;
#pragma unroll 4
                            for (int i = 0; i < dk; ++i) s = fmaf(qv[i], kv[i], s);
                            if (p.cap > 0.f) s = p.cap * tanhf(s / p.cap);
                        }
                        const bool vis = lane < nk && jl <= pq && (pq - jl < p.window || jl < p.keep);
                        if (pass == 0) {
                            float mx = vis ? s : -CUDART_INF_F;
#pragma unroll
                            for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
                            if (mx > -CUDART_INF_F) {          // warp-uniform
                                const float mo = sMax[r], mn = fmaxf(mo, mx);
                                float e = vis ? expf(s - mn) : 0.f;
#pragma unroll
                                for (int o = 16; o > 0; o >>= 1) e += __shfl_xor_sync(0xffffffffu, e, o);
                                if (lane == 0) { sSum[r] = sSum[r] * (mo > -CUDART_INF_F ? expf(mo - mn) : 0.f) + e; sMax[r] = mn; }
                                __syncwarp();
                            }
                        } else {
                            sP[r * WA_KT + lane] = vis ? expf(s - sMax[r]) / sSum[r] : 0.f;
                        }
                    }
                }
                if (pass == 0) continue;
                __syncthreads();
                for (int e = threadIdx.x; e < R * WA_KT; e += WA_THREADS) {
                    const int r = e / WA_KT, kt = e % WA_KT, qi = r / H, h = r % H;
                    float a = 0.f;
                    for (int g = 0; g < H; ++g) a = fmaf(sMix[h * H + g], sP[(qi * H + g) * WA_KT + kt], a);
                    sM[e] = a;
                }
                for (int c = 0; c < G; ++c) {
                    __syncthreads();               // mixed weights written / the tile buffer is free
                    for (int kt = warp; kt < nk; kt += nw) {
                        const int j = j0 + kt;
                        const float* src = p.cache + ((size_t)tbl[j / p.page] * p.page + j % p.page) * D + (size_t)G * dk + (size_t)c * dv;
                        for (int i = lane; i < dv; i += 32) sT[kt * ts + i] = src[i];
                    }
                    __syncthreads();
                    for (int rr = warp; rr < nq * rep; rr += nw) {
                        const int qi = rr / rep, r = qi * H + c * rep + rr % rep;
                        const float* w = sM + r * WA_KT;
                        for (int d = lane; d < dv; d += 32) {
                            float acc = sO[(size_t)r * dv + d];
                            for (int kt = 0; kt < nk; ++kt) acc = fmaf(w[kt], sT[kt * ts + d], acc);
                            sO[(size_t)r * dv + d] = acc;
                        }
                    }
                }
            }
        }
        __syncthreads();
    }
    for (int e = threadIdx.x; e < R * dv; e += WA_THREADS) {
        const int r = e / dv, d = e % dv;
        p.out[(size_t)(t0 + r / H) * p.ldo + (size_t)(r % H) * dv + d] = sO[e];
    }
}

}  // namespace b200
