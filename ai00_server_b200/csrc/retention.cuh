// Retention: linear attention with one fixed decay per head, no softmax and no denominator,
//     S_t = lambda_h S_{t-1} + k_t v_t^T,    o_t = S_t^T q_t,
// q and k rotated by position first (rotate-half pairing: entry i with entry i + dims / 2, on the first `dims` entries of a
// head), k scaled after the rotation.  The read-out is divided by its root mean square over the value width (no weight) and
// multiplied by silu of a gate projection.  One CTA per (head, sequence of the step): the [dk, dv] f32 state stays in shared
// memory for the sequence's tokens of this step, column j belongs to thread j (decay, rank-1 update and read-out in one pass
// over the column, no cross-thread traffic), and is loaded from / stored to the sequence's slot once per step.  State,
// read-out and norm are f32; the rotation angle is formed and reduced in double (rot_cos_sin).
#pragma once
#include <cuda_runtime.h>
#include "common.cuh"
#include "latent_attn.cuh"

namespace b200 {

struct RetentionParams {
    const float* q; const float* k; const float* v; const float* g;   // rows of the fused projection output, row stride ld
    int ld;
    float* state;                                 // [S][H][dk][dv] of this layer
    float* out; int ldo;                          // [T, H * dv]: normed, gated
    const float* decay;                           // [H]
    const double* freq;                           // [rot_dims / 2]
    int H, dk, dv, rot_dims;
    float k_scale, eps;
    MetaView meta; SeqMeta sm;
};

__host__ __device__ inline size_t retention_smem_bytes(int dk, int dv) { return ((size_t)dk * dv + 2 * (size_t)dk + 32) * sizeof(float); }

__global__ void retention_kernel(const RetentionParams p) {
    const int h = blockIdx.x, si = blockIdx.y;
    if (si >= p.meta.nslots()) return;
    const int slot = p.meta.slot_id()[si], t0 = p.meta.slot_start()[si], nt = p.meta.slot_count()[si];
    const int dk = p.dk, dv = p.dv, j = threadIdx.x, half = p.rot_dims >> 1;
    extern __shared__ __align__(16) float ret_smem[];
    float* S = ret_smem;                          // [dk][dv]
    float* sq = S + (size_t)dk * dv;              // [dk]
    float* sk = sq + dk;                          // [dk]
    float* red = sk + dk;                         // [32]
    float* gS = p.state + ((size_t)slot * p.H + h) * dk * dv;
    const int nst = dk * dv;
    const bool vec = (nst % 4) == 0;
    if (vec) {
#pragma unroll 8
        for (int e = j; e < nst / 4; e += blockDim.x) reinterpret_cast<float4*>(S)[e] = __ldg(reinterpret_cast<const float4*>(gS) + e);
    } else {
        for (int e = j; e < nst; e += blockDim.x) S[e] = gS[e];
    }
    const float lam = p.decay[h];
    for (int t = t0; t < t0 + nt; ++t) {
        __syncthreads();
        const int ipos = p.sm.tok_pos()[t];
        const float* qr = p.q + (size_t)t * p.ld + (size_t)h * dk;
        const float* kr = p.k + (size_t)t * p.ld + (size_t)h * dk;
        for (int i = j; i < dk; i += blockDim.x) {
            if (i >= p.rot_dims) { sq[i] = qr[i]; sk[i] = kr[i] * p.k_scale; continue; }
            const int f = i < half ? i : i - half;
            float cs, sn;
            rot_cos_sin(ipos, p.freq[f], cs, sn);
            const float qu = qr[f], qv = qr[f + half], ku = kr[f], kv = kr[f + half];
            sq[i] = i < half ? qu * cs - qv * sn : qv * cs + qu * sn;
            sk[i] = (i < half ? ku * cs - kv * sn : kv * cs + ku * sn) * p.k_scale;
        }
        __syncthreads();
        float o = 0.f;
        if (j < dv) {
            const float vj = p.v[(size_t)t * p.ld + (size_t)h * dv + j];
            for (int i = 0; i < dk; ++i) {
                const float s = fmaf(lam, S[(size_t)i * dv + j], sk[i] * vj);
                S[(size_t)i * dv + j] = s;
                o = fmaf(s, sq[i], o);
            }
        }
        float ss = j < dv ? o * o : 0.f;
#pragma unroll
        for (int of = 16; of > 0; of >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, of);
        if ((j & 31) == 0) red[j >> 5] = ss;
        __syncthreads();
        ss = 0.f;
        for (int w = 0; w < (int)((blockDim.x + 31) >> 5); ++w) ss += red[w];
        if (j < dv) {
            const float gg = p.g[(size_t)t * p.ld + (size_t)h * dv + j];
            p.out[(size_t)t * p.ldo + (size_t)h * dv + j] = o / sqrtf(ss / (float)dv + p.eps) * (gg / (1.f + expf(-gg)));
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

// The same recurrence with the state column in REGISTERS (dk <= DKC <= 128, dv <= 256): thread j keeps S[0..dk)[j] for the whole
// step; decay, rank-1 update and read-out are straight-line FMAs on registers fed by broadcast reads of q and k from shared memory.
constexpr int RET_REG_MAX_DK = 128, RET_REG_MAX_DV = 256;

template <int DKC>
__global__ void __launch_bounds__(RET_REG_MAX_DV) retention_reg_kernel(const RetentionParams p) {
    const int h = blockIdx.x, si = blockIdx.y;
    if (si >= p.meta.nslots()) return;
    const int slot = p.meta.slot_id()[si], t0 = p.meta.slot_start()[si], nt = p.meta.slot_count()[si];
    const int dk = p.dk, dv = p.dv, j = threadIdx.x, half = p.rot_dims >> 1;
    __shared__ __align__(16) float sq[DKC], sk[DKC];
    __shared__ float red[32];
    float* gS = p.state + ((size_t)slot * p.H + h) * dk * dv;
    float s[DKC];
#pragma unroll
    for (int i = 0; i < DKC; ++i) s[i] = (i < dk && j < dv) ? gS[(size_t)i * dv + j] : 0.f;
    const float lam = p.decay[h];
    for (int t = t0; t < t0 + nt; ++t) {
        __syncthreads();
        const int ipos = p.sm.tok_pos()[t];
        const float* qr = p.q + (size_t)t * p.ld + (size_t)h * dk;
        const float* kr = p.k + (size_t)t * p.ld + (size_t)h * dk;
        for (int i = j; i < DKC; i += blockDim.x) {
            if (i >= dk) { sq[i] = 0.f; sk[i] = 0.f; continue; }
            if (i >= p.rot_dims) { sq[i] = qr[i]; sk[i] = kr[i] * p.k_scale; continue; }
            const int f = i < half ? i : i - half;
            float cs, sn;
            rot_cos_sin(ipos, p.freq[f], cs, sn);
            const float qu = qr[f], qv = qr[f + half], ku = kr[f], kv = kr[f + half];
            sq[i] = i < half ? qu * cs - qv * sn : qv * cs + qu * sn;
            sk[i] = (i < half ? ku * cs - kv * sn : kv * cs + ku * sn) * p.k_scale;
        }
        __syncthreads();
        float o = 0.f;
        if (j < dv) {
            const float vj = p.v[(size_t)t * p.ld + (size_t)h * dv + j];
            float o0 = 0.f, o1 = 0.f, o2 = 0.f, o3 = 0.f;
#pragma unroll
            for (int i = 0; i < DKC; i += 4) {
                s[i] = fmaf(lam, s[i], sk[i] * vj); s[i + 1] = fmaf(lam, s[i + 1], sk[i + 1] * vj);
                s[i + 2] = fmaf(lam, s[i + 2], sk[i + 2] * vj); s[i + 3] = fmaf(lam, s[i + 3], sk[i + 3] * vj);
                o0 = fmaf(s[i], sq[i], o0); o1 = fmaf(s[i + 1], sq[i + 1], o1);
                o2 = fmaf(s[i + 2], sq[i + 2], o2); o3 = fmaf(s[i + 3], sq[i + 3], o3);
            }
            o = (o0 + o1) + (o2 + o3);
        }
        float ss = j < dv ? o * o : 0.f;
#pragma unroll
        for (int of = 16; of > 0; of >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, of);
        if ((j & 31) == 0) red[j >> 5] = ss;
        __syncthreads();
        ss = 0.f;
        for (int w = 0; w < (int)((blockDim.x + 31) >> 5); ++w) ss += red[w];
        if (j < dv) {
            const float gg = p.g[(size_t)t * p.ld + (size_t)h * dv + j];
            p.out[(size_t)t * p.ldo + (size_t)h * dv + j] = o / sqrtf(ss / (float)dv + p.eps) * (gg / (1.f + expf(-gg)));
        }
    }
    if (j < dv) {
#pragma unroll
        for (int i = 0; i < DKC; ++i)
            if (i < dk) gS[(size_t)i * dv + j] = s[i];
    }
}

}  // namespace b200
