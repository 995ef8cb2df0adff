// Root-mean-square normalisation stages on f32 rows (every norm of this family is computed in 32-bit):
//   embed_rows_kernel      x[t] = table[token[t]]                                   (bf16 table -> f32 residual)
//   norm_shift_kernel      h = x / rms(x) * g (one scalar gain);  hs = h + (h_prev - h) * mu  (token shift on the NORMED row;
//                          h_prev = the previous token's h: the row before it in this step, or the sequence's shift state);
//   shift_commit_kernel    the last token of every sequence in the step leaves its h as the new shift state
//   rms_rows_kernel        y[r, c*w .. c*w+w) = x / rms(x over the w-wide chunk) * weight[w]   (per-chunk norm with a weight vector)
//   final_norm_kernel      rows that want logits: x[out_tok[r]] / rms * g  -> compact [R, W] head operand (+ all hidden rows)
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include "common.cuh"

namespace b200 {

constexpr int NORM_THREADS = 256;

__device__ __forceinline__ float rms_block_sum(float v, float* red /* [32] */) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    __syncthreads();                       // red may still be read from a previous call
    if (lane == 0) red[warp] = v;
    __syncthreads();
    float s = 0.f;
    for (int i = 0; i < nw; ++i) s += red[i];      // same order in every thread
    return s;
}

struct EmbedRowsParams {
    const __nv_bfloat16* table;
    float* x;
    int W;
    MetaView meta;
};

__global__ void __launch_bounds__(NORM_THREADS) embed_rows_kernel(const EmbedRowsParams p) {
    const int t = blockIdx.x;
    if (t >= p.meta.T()) return;
    const __nv_bfloat16* src = p.table + (size_t)p.meta.tok()[t] * p.W;
    float* dst = p.x + (size_t)t * p.W;
    for (int c = threadIdx.x; c < p.W; c += blockDim.x) dst[c] = __bfloat162float(src[c]);
}

struct NormShiftParams {
    const float* x;          // [T, W] residual
    float* h;                // [T, W] normed row (feed-forward, gates)
    float* hs;               // [T, W] token-shifted normed row (mixer); nullptr: no shift
    const float* mu;         // [W]
    float* shift_state;      // [S, W] of this layer
    float gain, eps;
    int W;
    MetaView meta;
};

__global__ void __launch_bounds__(NORM_THREADS) norm_shift_kernel(const NormShiftParams p) {
    __shared__ float red[32];
    const int t = blockIdx.x;
    if (t >= p.meta.T()) return;
    const int W = p.W;
    const float* xr = p.x + (size_t)t * W;
    const int prev = p.meta.tok_prev()[t];
    const int slot = p.meta.tok_slot()[t];
    float ss = 0.f, sp = 0.f;
    for (int c = threadIdx.x; c < W; c += blockDim.x) {
        const float v = xr[c];
        ss = fmaf(v, v, ss);
        if (prev >= 0) { const float u = p.x[(size_t)prev * W + c]; sp = fmaf(u, u, sp); }
    }
    ss = rms_block_sum(ss, red);
    const float r = p.gain / sqrtf(ss / (float)W + p.eps);
    float rp = 0.f;
    if (prev >= 0) { sp = rms_block_sum(sp, red); rp = p.gain / sqrtf(sp / (float)W + p.eps); }
    for (int c = threadIdx.x; c < W; c += blockDim.x) {
        const float hv = xr[c] * r;
        p.h[(size_t)t * W + c] = hv;
        if (p.hs) {
            const float hp = prev >= 0 ? p.x[(size_t)prev * W + c] * rp : p.shift_state[(size_t)slot * W + c];
            p.hs[(size_t)t * W + c] = hv + (hp - hv) * p.mu[c];
        }
    }
}

// shift-state commit, run after norm_shift_kernel of the same layer (a first token of the sequence may still be reading the
// old row while the last token's CTA would overwrite it, so the commit is its own launch)
__global__ void __launch_bounds__(NORM_THREADS) shift_commit_kernel(const NormShiftParams p) {
    const int i = blockIdx.x;
    if (i >= p.meta.nslots()) return;
    const int t = p.meta.slot_start()[i] + p.meta.slot_count()[i] - 1;
    const int slot = p.meta.slot_id()[i];
    for (int c = threadIdx.x; c < p.W; c += blockDim.x) p.shift_state[(size_t)slot * p.W + c] = p.h[(size_t)t * p.W + c];
}

struct RmsRowsParams {
    const float* x; int ldx;
    float* y; int ldy;
    const float* weight;     // [w]
    int w, chunks;           // `chunks` chunks of width w per row
    float eps;
    const int* nrows;
};

__global__ void __launch_bounds__(128) rms_rows_kernel(const RmsRowsParams p) {
    __shared__ float red[32];
    const int r = blockIdx.x, c = blockIdx.y;
    if (r >= *p.nrows) return;
    const float* x = p.x + (size_t)r * p.ldx + (size_t)c * p.w;
    float* y = p.y + (size_t)r * p.ldy + (size_t)c * p.w;
    float ss = 0.f;
    for (int i = threadIdx.x; i < p.w; i += blockDim.x) ss = fmaf(x[i], x[i], ss);
    ss = rms_block_sum(ss, red);
    const float s = 1.f / sqrtf(ss / (float)p.w + p.eps);
    for (int i = threadIdx.x; i < p.w; i += blockDim.x) y[i] = x[i] * s * p.weight[i];
}

struct FinalNormParams {
    const float* x;          // [T, W]
    float* y;                // [R, W]
    float* hidden;           // [T, W] copy of the residual (embeddings route); may be nullptr
    float gain, eps;
    int W;
    MetaView meta;
};

__global__ void __launch_bounds__(NORM_THREADS) final_norm_kernel(const FinalNormParams p) {
    __shared__ float red[32];
    const int t = blockIdx.x;
    if (t >= p.meta.T()) return;
    const int W = p.W;
    const float* xr = p.x + (size_t)t * W;
    const int row = p.meta.tok_outrow()[t];
    if (p.hidden)
        for (int c = threadIdx.x; c < W; c += blockDim.x) p.hidden[(size_t)t * W + c] = xr[c];
    if (row < 0) return;
    float ss = 0.f;
    for (int c = threadIdx.x; c < W; c += blockDim.x) ss = fmaf(xr[c], xr[c], ss);
    ss = rms_block_sum(ss, red);
    const float r = p.gain / sqrtf(ss / (float)W + p.eps);
    for (int c = threadIdx.x; c < W; c += blockDim.x) p.y[(size_t)row * W + c] = xr[c] * r;
}

}  // namespace b200
