// Gated linear attention: per head a [dk, dv] f32 state with a per-key-channel decay,
//     S_t = diag(alpha_t) S_{t-1} + k_t v_t^T,    o_t = S_t^T q_t,    alpha = sigmoid(z)^(1/tau) = exp(logsigmoid(z) / tau)
// followed by an RMS norm of o over dv (weight shared by heads) and an output gate silu(g).  One CTA per (head, sequence of the
// step): the state lives in shared memory for the sequence's tokens of this step (column j of S belongs to thread j, so the
// decay, the rank-1 update and the read-out are one pass over a column with no cross-thread traffic), is loaded from and
// stored to the sequence's slot once per step.  Decay, state, read-out and norm are f32.
#pragma once
#include <cuda_runtime.h>
#include "common.cuh"

namespace b200 {

struct GlaParams {
    const float* q; const float* k; const float* v; const float* g;   // rows of the fused projection output, row stride ld
    int ld;
    const float* z; int ldz;                      // decay logits [T, H * dk] (bias already added)
    float* state;                                 // [S][H][dk][dv] of this layer
    float* out; int ldo;                          // [T, H * dv]: normed, gated
    const float* norm_w;                          // [dv]
    int H, dk, dv;
    float inv_tau, q_scale, eps;
    MetaView meta;
};

__host__ __device__ inline size_t gla_smem_bytes(int dk, int dv) { return ((size_t)dk * dv + 3 * (size_t)dk + 32) * sizeof(float); }

__global__ void gla_kernel(const GlaParams p) {
    const int h = blockIdx.x, si = blockIdx.y;
    if (si >= p.meta.nslots()) return;
    const int slot = p.meta.slot_id()[si], t0 = p.meta.slot_start()[si], nt = p.meta.slot_count()[si];
    const int dk = p.dk, dv = p.dv, j = threadIdx.x;
    extern __shared__ __align__(16) float gla_smem[];
    float* S = gla_smem;                             // [dk][dv]
    float* sq = S + (size_t)dk * dv;              // [dk]
    float* skk = sq + dk;
    float* sa = skk + dk;
    float* red = sa + dk;                         // [32]
    float* gS = p.state + ((size_t)slot * p.H + h) * dk * dv;
    const int nst = dk * dv;
    const bool vec = (nst % 4) == 0;                  // slot records then start on 16-byte boundaries
    if (vec) {
#pragma unroll 8
        for (int e = j; e < nst / 4; e += blockDim.x) reinterpret_cast<float4*>(S)[e] = __ldg(reinterpret_cast<const float4*>(gS) + e);
    } else {
        for (int e = j; e < nst; e += blockDim.x) S[e] = gS[e];
    }
    for (int t = t0; t < t0 + nt; ++t) {
        __syncthreads();
        for (int i = j; i < dk; i += blockDim.x) {
            const size_t c = (size_t)h * dk + i;
            sq[i] = p.q[(size_t)t * p.ld + c] * p.q_scale;
            skk[i] = p.k[(size_t)t * p.ld + c];
            const float zz = p.z[(size_t)t * p.ldz + c];
            const float ls = fminf(zz, 0.f) - log1pf(expf(-fabsf(zz)));      // log sigmoid(z)
            sa[i] = expf(ls * p.inv_tau);
        }
        __syncthreads();
        float o = 0.f;
        if (j < dv) {
            const float vj = p.v[(size_t)t * p.ld + (size_t)h * dv + j];
            for (int i = 0; i < dk; ++i) {
                const float s = fmaf(sa[i], S[(size_t)i * dv + j], skk[i] * vj);
                S[(size_t)i * dv + j] = s;
                o = fmaf(s, sq[i], o);
            }
        }
        // RMS over dv
        float ss = j < dv ? o * o : 0.f;
#pragma unroll
        for (int of = 16; of > 0; of >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, of);
        if ((j & 31) == 0) red[j >> 5] = ss;
        __syncthreads();
        ss = 0.f;
        for (int w = 0; w < (int)((blockDim.x + 31) >> 5); ++w) ss += red[w];
        if (j < dv) {
            const float gg = p.g[(size_t)t * p.ld + (size_t)h * dv + j];
            const float gate = gg / (1.f + expf(-gg));
            p.out[(size_t)t * p.ldo + (size_t)h * dv + j] = o / sqrtf(ss / (float)dv + p.eps) * p.norm_w[j] * gate;
        }
    }
    __syncthreads();
    if (vec) {
#pragma unroll 8
        for (int e = j; e < nst / 4; e += blockDim.x) reinterpret_cast<float4*>(gS)[e] = reinterpret_cast<const float4*>(S)[e];
    } else {
        for (int e = j; e < nst; e += blockDim.x) gS[e] = S[e];
    }
}

}  // namespace b200
