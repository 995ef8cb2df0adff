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
//                        `dims` entries of a head.
//   window_attn_kernel   a cluster of 1..8 CTAs per chunk of consecutive tokens of one sequence (SeqMeta chunks), all heads; the
//                        32-key tiles of the walk are dealt out among the cluster's CTAs (decode steps and short steps would
//                        otherwise run on a handful of SMs); the per-row maxima / sums after the first walk and the partial
//                        outputs after the second are combined through distributed shared memory in rank order.  A warp scores
//                        four rows of one key / value head against a key at a time.  Scores, softmax, mix and sums in f32.
#pragma once
#include <cooperative_groups.h>
#include <cuda_runtime.h>
#include <math_constants.h>
#include "common.cuh"
#include "latent_attn.cuh"
#include "linear.cuh"

namespace b200 {

struct AttnPrepParams {
    const float* q; const float* k; const float* v; int ld;      // projection rows: q [H * dk], k [G * dk], v [G * dv]
    float* qo; int ldq;                           // [T, H * dk]
    float* cache;                                 // [pages][page][G * dk + G * dv]
    const int* table; int stride; int page;
    const float* wq; const float* wk;             // [dk] norm weights
    const float* temp;                            // [H]
    const double* freq;                           // [dims / 2]
    int H, G, dk, dv, dims;
    float scale, eps;
    MetaView meta; SeqMeta sm;
};

__global__ void __launch_bounds__(128) attn_prep_kernel(const AttnPrepParams p) {
    const int t = blockIdx.x;
    if (t >= p.meta.T()) return;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
    const int slot = p.meta.tok_slot()[t], ipos = p.sm.tok_pos()[t];
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
                float cs, sn;
                rot_cos_sin(ipos, p.freq[i >> 1], cs, sn);
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
    int gt;                                       // key / value heads per tile load
    int cl;                                       // CTAs per chunk (cluster size): the key tiles are dealt out among them
    MetaView meta; SeqMeta sm;
};

constexpr int WA_KT = 32;                          // keys per tile (one per lane in the score phase)
constexpr int WA_THREADS = 512;                     // most threads per CTA; the host launches 256 where fewer warps find work
constexpr int WA_RB = 4;                           // most rows of one key / value head a warp works on together

__host__ __device__ inline size_t window_attn_smem(int qb, int H, int dk, int dv, int gt) {
    const size_t R = (size_t)qb * H, dmax = dk > dv ? dk : dv;
    return (R * dk + R * dv + 2 * R * WA_KT + (size_t)gt * WA_KT * (dmax + 4) + 4 * R + (size_t)H * H + 8) * sizeof(float);
}

// `nk` cache rows from position j0 on, `w` floats at offset `off` of each of `gn` consecutive heads -> tile[head][key][ts].  vec:
// 16-byte cp.async copies issued by all threads at once (every row address comes from the page table first, so the copies of a
// tile are in flight together); otherwise plain loads.  Ends with the data visible to the whole CTA.
__device__ __forceinline__ void wa_load_tile(const float* cache, const int* tbl, int page, int D, size_t off, int w, float* tile, int ts, int gn,
                                             int nk, int j0, bool vec) {
    if (vec) {
        const int w4 = w >> 2, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
        for (int kt = warp; kt < nk; kt += (int)(blockDim.x >> 5)) {      // a warp per cache row: one page lookup, then 16 bytes per lane
            const int j = j0 + kt, pg = j / page;
            const float* src = cache + ((size_t)tbl[pg] * page + (j - pg * page)) * D + off;
            float* dst = tile + (size_t)kt * ts;
            for (int cl_ = 0; cl_ < gn; ++cl_)
                for (int v4 = lane; v4 < w4; v4 += 32) cp_async16(dst + (size_t)cl_ * WA_KT * ts + v4 * 4, src + (size_t)cl_ * w + v4 * 4);
        }
        asm volatile("cp.async.commit_group;\n" ::: "memory");
        asm volatile("cp.async.wait_group 0;\n" ::: "memory");
    } else {
        const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
        for (int e = warp; e < gn * nk; e += (int)(blockDim.x >> 5)) {
            const int cl_ = e / nk, kt = e % nk, j = j0 + kt;
            const float* src = cache + ((size_t)tbl[j / page] * page + j % page) * D + off + (size_t)cl_ * w;
            float* dst = tile + ((size_t)cl_ * WA_KT + kt) * ts;
            for (int i = lane; i < w; i += 32) dst[i] = src[i];
        }
    }
    __syncthreads();
}

// the tile `ti` of the key walk: segment 0 first, then segment 1
__device__ __forceinline__ void wa_tile(int ti, int n0, const int* lo, const int* hi, int& j0, int& nk) {
    const int sg = ti < n0 ? 0 : 1, k = ti < n0 ? ti : ti - n0;
    j0 = lo[sg] + k * WA_KT;
    nk = min(WA_KT, hi[sg] - j0);
}

__global__ void __launch_bounds__(WA_THREADS) window_attn_kernel(const WindowAttnParams p) {
    namespace cg = cooperative_groups;
    cg::cluster_group cluster = cg::this_cluster();
    const int CL = p.cl, rank = blockIdx.x % CL, ch = blockIdx.x / CL;
    if (ch >= p.sm.n_chunks()) return;             // the same for every CTA of a cluster
    const int t0 = p.sm.chunk_start()[ch], nq = p.sm.chunk_count()[ch];
    const int slot = p.meta.tok_slot()[t0];
    const int pos0 = p.sm.tok_pos()[t0], pos1 = pos0 + nq - 1;
    const int H = p.H, G = p.G, dk = p.dk, dv = p.dv, rep = H / G, R = nq * H;
    // head sizes that are multiples of four: rows of the tile buffer start on 16 bytes (stride dmax + 4: a quarter warp's 16-byte
    // reads of eight different rows fall into different banks), tiles arrive by cp.async and the score loop reads four floats at
    // a time; otherwise stride dmax + 1 and scalar loads
    const bool vec = (dk % 4 == 0) && (dv % 4 == 0);
    const int dmax = dk > dv ? dk : dv, ts = dmax + (vec ? 4 : 1), D = G * (dk + dv);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
    extern __shared__ __align__(16) float wa_smem[];
    const int Rcap = p.qb * H;
    float* sQ = wa_smem;                          // [R][dk]
    float* sO = sQ + (size_t)Rcap * dk;           // [R][dv]
    float* sP = sO + (size_t)Rcap * dv;           // [R][KT] normalised weights of the tile
    float* sM = sP + (size_t)Rcap * WA_KT;        // [R][KT] mixed weights
    float* sT = sM + (size_t)Rcap * WA_KT;        // [gt][KT][ts] key or value tiles of gt heads
    float* sMax = sT + (size_t)p.gt * WA_KT * ts; // [R] this CTA's running maximum / sum
    float* sSum = sMax + Rcap;
    float* sGMax = sSum + Rcap;                   // [R] the chunk's (all CTAs of the cluster)
    float* sGSum = sGMax + Rcap;
    float* sMix = sGSum + Rcap;                   // [H][H]
    for (int e = threadIdx.x; e < R * dk; e += (int)blockDim.x) {
        const int r = e / dk, i = e % dk;
        sQ[e] = p.q[(size_t)(t0 + r / H) * p.ldq + (size_t)(r % H) * dk + i];
    }
    for (int e = threadIdx.x; e < R * dv; e += (int)blockDim.x) sO[e] = 0.f;
    for (int e = threadIdx.x; e < R; e += (int)blockDim.x) { sMax[e] = -CUDART_INF_F; sSum[e] = 0.f; }
    for (int e = threadIdx.x; e < H * H; e += (int)blockDim.x) sMix[e] = p.mix[e];
    // key ranges: the kept prefix [0, a_hi) and the window [b_lo, pos1]; one range when they touch
    int seg_lo[2] = {0, 0}, seg_hi[2] = {0, 0};
    {
        const int a_hi = min(p.keep, pos1 + 1), b_lo = max(0, pos0 - p.window + 1);
        if (a_hi <= 0) { seg_lo[0] = b_lo; seg_hi[0] = pos1 + 1; }
        else if (b_lo <= a_hi) { seg_lo[0] = 0; seg_hi[0] = pos1 + 1; }
        else { seg_lo[0] = 0; seg_hi[0] = a_hi; seg_lo[1] = b_lo; seg_hi[1] = pos1 + 1; }
    }
    const int n0 = (seg_hi[0] - seg_lo[0] + WA_KT - 1) / WA_KT, ntiles = n0 + (seg_hi[1] - seg_lo[1] + WA_KT - 1) / WA_KT;
    const int* tbl = p.table + (size_t)slot * p.stride;
    const int nrg = nq * rep;                      // rows of one key / value head
    const int rb = WA_RB;                          // rows a warp takes together: they share every key / value operand
    const int nblk = (nrg + rb - 1) / rb;          // row blocks of one head
    __syncthreads();
    for (int pass = 0; pass < 2; ++pass) {
        for (int ti = rank; ti < ntiles; ti += CL) {
            int j0, nk;
            wa_tile(ti, n0, seg_lo, seg_hi, j0, nk);
            const int jl = j0 + lane;
            for (int c0 = 0; c0 < G; c0 += p.gt) {
                const int gn = min(p.gt, G - c0);
                __syncthreads();                   // the tile buffer is free
                wa_load_tile(p.cache, tbl, p.page, D, (size_t)c0 * dk, dk, sT, ts, gn, nk, j0, vec);
                for (int it = warp; it < gn * nblk; it += nw) {
                    const int cl_ = it / nblk, c = c0 + cl_, rr0 = (it % nblk) * rb, nr = min(rb, nrg - rr0);
                    int rows[WA_RB];
                    const float* qv[WA_RB];
#pragma unroll
                    for (int b = 0; b < WA_RB; ++b) {
                        const int rr = rr0 + min(b, nr - 1);
                        rows[b] = (rr / rep) * H + c * rep + rr % rep;
                        qv[b] = sQ + (size_t)rows[b] * dk;
                    }
                    float sc[WA_RB] = {0.f, 0.f, 0.f, 0.f};
                    if (lane < nk) {
                        const float* kv = sT + ((size_t)cl_ * WA_KT + lane) * ts;
                        if (vec) {
                            const float4* k4 = reinterpret_cast<const float4*>(kv);
#pragma unroll 4
                            for (int i = 0; i < dk / 4; ++i) {
                                const float4 kx = k4[i];
#pragma unroll
                                for (int b = 0; b < WA_RB; ++b) {
                                    const float4 qx = reinterpret_cast<const float4*>(qv[b])[i];
                                    sc[b] = fmaf(qx.x, kx.x, sc[b]); sc[b] = fmaf(qx.y, kx.y, sc[b]);
                                    sc[b] = fmaf(qx.z, kx.z, sc[b]); sc[b] = fmaf(qx.w, kx.w, sc[b]);
                                }
                            }
                        } else {
#pragma unroll 4
                            for (int i = 0; i < dk; ++i) {
                                const float kx = kv[i];
#pragma unroll
                                for (int b = 0; b < WA_RB; ++b) sc[b] = fmaf(qv[b][i], kx, sc[b]);
                            }
                        }
                    }
#pragma unroll
                    for (int b = 0; b < WA_RB; ++b) {
                        if (b >= nr) break;
                        const int r = rows[b], pq = pos0 + r / H;
                        float s = sc[b];
                        if (p.cap > 0.f) s = p.cap * tanhf(s / p.cap);
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
                            sP[r * WA_KT + lane] = vis ? expf(s - sGMax[r]) / sGSum[r] : 0.f;
                        }
                    }
                }
            }
            if (pass == 0) continue;
            __syncthreads();
            for (int e = threadIdx.x; e < R * WA_KT; e += (int)blockDim.x) {
                const int r = e / WA_KT, kt = e % WA_KT, qi = r / H, h = r % H;
                float a = 0.f;
                for (int g = 0; g < H; ++g) a = fmaf(sMix[h * H + g], sP[(qi * H + g) * WA_KT + kt], a);
                sM[e] = a;
            }
            for (int c0 = 0; c0 < G; c0 += p.gt) {
                const int gn = min(p.gt, G - c0);
                __syncthreads();                   // mixed weights written / the tile buffer is free
                wa_load_tile(p.cache, tbl, p.page, D, (size_t)G * dk + (size_t)c0 * dv, dv, sT, ts, gn, nk, j0, vec);
                for (int it = warp; it < gn * nblk; it += nw) {
                    const int cl_ = it / nblk, c = c0 + cl_, rr0 = (it % nblk) * rb, nr = min(rb, nrg - rr0);
                    int rows[WA_RB];
#pragma unroll
                    for (int b = 0; b < WA_RB; ++b) {
                        const int rr = rr0 + min(b, nr - 1);
                        rows[b] = (rr / rep) * H + c * rep + rr % rep;
                    }
                    const float* vt = sT + (size_t)cl_ * WA_KT * ts;
                    for (int d = lane; d < dv; d += 32) {
                        float acc[WA_RB];
#pragma unroll
                        for (int b = 0; b < WA_RB; ++b) acc[b] = sO[(size_t)rows[b] * dv + d];
#pragma unroll 4
                        for (int kt = 0; kt < nk; ++kt) {
                            const float vx = vt[kt * ts + d];
#pragma unroll
                            for (int b = 0; b < WA_RB; ++b) acc[b] = fmaf(sM[rows[b] * WA_KT + kt], vx, acc[b]);
                        }
#pragma unroll
                        for (int b = 0; b < WA_RB; ++b)
                            if (b < nr) sO[(size_t)rows[b] * dv + d] = acc[b];
                    }
                }
            }
        }
        __syncthreads();
        if (pass == 0) {
            // the chunk's maximum and sum of every row: the CTAs' partial results combined in rank order (the same in every CTA)
            cluster.sync();
            for (int e = threadIdx.x; e < R; e += (int)blockDim.x) {
                float m = -CUDART_INF_F;
                for (int rk = 0; rk < CL; ++rk) m = fmaxf(m, cluster.map_shared_rank(sMax, rk)[e]);
                float l = 0.f;
                for (int rk = 0; rk < CL; ++rk) {
                    const float mr = cluster.map_shared_rank(sMax, rk)[e];
                    if (mr > -CUDART_INF_F) l += cluster.map_shared_rank(sSum, rk)[e] * expf(mr - m);
                }
                sGMax[e] = m; sGSum[e] = l;
            }
            __syncthreads();
        }
    }
    // the CTAs' partial sums added in rank order; every CTA finishes its share of the outputs
    cluster.sync();
    for (int e = rank * (int)blockDim.x + threadIdx.x; e < R * dv; e += CL * (int)blockDim.x) {
        float a = 0.f;
        for (int rk = 0; rk < CL; ++rk) a += cluster.map_shared_rank(sO, rk)[e];
        const int r = e / dv, d = e % dv;
        p.out[(size_t)(t0 + r / H) * p.ldo + (size_t)(r % H) * dv + d] = a;
    }
    cluster.sync();                                // nobody leaves while its shared memory is still being read
}

}  // namespace b200
