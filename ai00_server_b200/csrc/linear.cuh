// Grouped linear layers over row-major f32 activations and bf16 weights stored [out, in]:  Y[r, n] = epi(sum_k X[r, k] W[n, k]).
//
// One launch covers `groups` independent problems that share N and K (blockIdx.z): the heads of a per-head projection (column
// offsets into X / Y), or the experts of a routed feed-forward (row lists built on the device).  Row counts come from device
// memory (the step metadata, the router's per-expert counts), so a captured step graph never changes.
//
//   lin_tile_kernel<EXACT>   steps of many rows.  EXACT = false: bf16 operands on the tensor cores (mma.sync m16n8k16, f32
//                            accumulate), activations rounded to bf16 while they are staged; EXACT = true: plain f32 FMA on
//                            the f32 activations (bf16 weights widen exactly), no reduced-precision product anywhere.
//   lin_skinny_kernel        decode-shaped steps (a few rows): one warp per output (pair), the weight row streamed once as
//                            16-byte loads, f32 FMA for either precision -- the launch is bound by the weight bytes.
//
// Epilogues (fused): bias, sigmoid / silu, a per-row scale, accumulate-into-residual through a gate, and the clamped gated
// unit of the experts on interleaved (gate, up) output pairs.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace b200 {

enum LinEpi {
    LE_STORE = 0,       // Y = acc (+ bias)
    LE_SIGMOID = 1,     // Y = sigmoid(acc + bias)
    LE_GATED_ADD = 2,   // Y += gate[r, n] * acc          (residual accumulate; every element has one writer)
    LE_GLU_CLAMP = 3,   // outputs (2i, 2i+1) = (g, u): Y[r, i] = min(g, lim) * sigmoid(1.702 min(g, lim)) * (clamp(u, -lim, lim) + 1)
};

struct LinParams {
    const float* X; int ldx; long long x_gstride;      // X + g * x_gstride, row stride ldx (floats)
    const __nv_bfloat16* W; long long w_gstride;       // W + g * w_gstride, row n at n * K
    float* Y; int ldy; long long y_gstride;
    int N, K;
    const int* cnt; int cnt_gstride;                   // rows of group g = cnt[g * cnt_gstride]
    const int* off;                                    // first compact row of group g (nullptr: 0)
    const int* xlist;                                  // X row of compact row i (nullptr: i)
    const float* bias;                                 // [N] (nullptr: none); group g adds g * N
    const float* gate; int ldg;                        // LE_GATED_ADD
    float limit;                                       // LE_GLU_CLAMP
    int epi;
    int max_rows;                                      // upper bound of any group's rows (grid sizing)
};

__device__ __forceinline__ float lin_sigmoid(float z) { return 1.f / (1.f + expf(-z)); }

__device__ __forceinline__ float lin_glu(float g, float u, float lim) {
    g = fminf(g, lim);
    u = fminf(fmaxf(u, -lim), lim);
    return g * lin_sigmoid(1.702f * g) * (u + 1.f);
}

// one finished output element (or pair) -> memory
__device__ __forceinline__ void lin_store(const LinParams& p, int g, int yrow, int n, float a0, float a1, bool has1) {
    float* Y = p.Y + g * p.y_gstride;
    if (p.epi == LE_GLU_CLAMP) {                       // n is even: (gate, up) pair -> column n / 2
        Y[(size_t)yrow * p.ldy + (n >> 1)] = lin_glu(a0, a1, p.limit);
        return;
    }
    const float* b = p.bias ? p.bias + (size_t)g * p.N : nullptr;
#pragma unroll
    for (int j = 0; j < 2; ++j) {
        if (j == 1 && !has1) break;
        float a = j ? a1 : a0;
        const int nn = n + j;
        if (b) a += b[nn];
        float* y = Y + (size_t)yrow * p.ldy + nn;
        if (p.epi == LE_SIGMOID) *y = lin_sigmoid(a);
        else if (p.epi == LE_GATED_ADD) *y += p.gate[(size_t)yrow * p.ldg + nn] * a;
        else *y = a;
    }
}

// ------------------------------------------------------------------------------------------------------------------
// tiled kernel: 64 rows x 64 outputs per CTA, k in slabs of 32; 128 threads
// ------------------------------------------------------------------------------------------------------------------
constexpr int LIN_BM = 64, LIN_BN = 64, LIN_BK = 32, LIN_THREADS = 128;

__device__ __forceinline__ void mma_bf16_16816(float c[4], const uint32_t a[4], const uint32_t b[2]) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}

template <bool EXACT>
__global__ void __launch_bounds__(LIN_THREADS) lin_tile_kernel(const LinParams p) {
    const int g = blockIdx.z;
    const int rows = p.cnt[(size_t)g * p.cnt_gstride];
    const int r0 = blockIdx.y * LIN_BM;
    if (r0 >= rows) return;
    const int n0 = blockIdx.x * LIN_BN;
    const int base = p.off ? p.off[g] : 0;
    const float* X = p.X + g * p.x_gstride;
    const __nv_bfloat16* W = p.W + g * p.w_gstride;
    const int tid = threadIdx.x, K = p.K, N = p.N;

    __shared__ int s_xrow[LIN_BM];
    for (int i = tid; i < LIN_BM; i += LIN_THREADS) {
        const int r = r0 + i;
        s_xrow[i] = r < rows ? (p.xlist ? p.xlist[base + r] : base + r) : -1;
    }

    if constexpr (EXACT) {
        __shared__ float sA[LIN_BK][LIN_BM + 1];       // k-major: the inner product walks k, threads differ in row / column
        __shared__ float sB[LIN_BK][LIN_BN + 1];
        const int ty = tid >> 3, tx = tid & 7;         // 16 x 8 threads: 4 rows x 8 columns each
        float acc[4][8];
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
            for (int j = 0; j < 8; ++j) acc[i][j] = 0.f;
        __syncthreads();
        for (int k0 = 0; k0 < K; k0 += LIN_BK) {
            for (int e = tid; e < LIN_BM * LIN_BK; e += LIN_THREADS) {
                const int r = e / LIN_BK, k = e % LIN_BK;
                const int xr = s_xrow[r];
                sA[k][r] = (xr >= 0 && k0 + k < K) ? X[(size_t)xr * p.ldx + k0 + k] : 0.f;
                const int n = n0 + r;
                sB[k][r] = (n < N && k0 + k < K) ? __bfloat162float(W[(size_t)n * K + k0 + k]) : 0.f;
            }
            __syncthreads();
#pragma unroll 8
            for (int k = 0; k < LIN_BK; ++k) {
                float a[4], b[8];
#pragma unroll
                for (int i = 0; i < 4; ++i) a[i] = sA[k][ty * 4 + i];
#pragma unroll
                for (int j = 0; j < 8; ++j) b[j] = sB[k][tx * 8 + j];
#pragma unroll
                for (int i = 0; i < 4; ++i)
#pragma unroll
                    for (int j = 0; j < 8; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
            }
            __syncthreads();
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int r = r0 + ty * 4 + i;
            if (r >= rows) continue;
#pragma unroll
            for (int j = 0; j < 8; j += 2) {
                const int n = n0 + tx * 8 + j;
                if (n < N) lin_store(p, g, base + r, n, acc[i][j], acc[i][j + 1], n + 1 < N);
            }
        }
    } else {
        constexpr int LDS = LIN_BK + 8;                // 80-byte rows: fragment loads fall into distinct banks
        __shared__ __align__(16) __nv_bfloat16 sA[LIN_BM][LDS];
        __shared__ __align__(16) __nv_bfloat16 sB[LIN_BN][LDS];
        const int warp = tid >> 5, lane = tid & 31;
        const int wm = (warp >> 1) * 32, wn = (warp & 1) * 32;      // 2 x 2 warps, 32 x 32 each
        const int gq = lane >> 2, tq = lane & 3;
        float acc[2][4][4];
#pragma unroll
        for (int i = 0; i < 2; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j)
#pragma unroll
                for (int c = 0; c < 4; ++c) acc[i][j][c] = 0.f;
        const bool vecW = (K % 8 == 0) && ((reinterpret_cast<uintptr_t>(W) & 15) == 0);
        const bool vecX = (p.ldx % 4 == 0) && ((reinterpret_cast<uintptr_t>(X) & 15) == 0);
        __syncthreads();
        for (int k0 = 0; k0 < K; k0 += LIN_BK) {
            // activations: 64 rows x 32 k, 4 consecutive k per thread and pass
            for (int e = tid; e < LIN_BM * (LIN_BK / 4); e += LIN_THREADS) {
                const int r = e / (LIN_BK / 4), k = (e % (LIN_BK / 4)) * 4;
                const int xr = s_xrow[r];
                float v[4] = {0.f, 0.f, 0.f, 0.f};
                if (xr >= 0) {
                    const float* src = X + (size_t)xr * p.ldx + k0 + k;
                    if (vecX && k0 + k + 3 < K) {
                        const float4 q = *reinterpret_cast<const float4*>(src);
                        v[0] = q.x; v[1] = q.y; v[2] = q.z; v[3] = q.w;
                    } else {
#pragma unroll
                        for (int j = 0; j < 4; ++j)
                            if (k0 + k + j < K) v[j] = src[j];
                    }
                }
                __nv_bfloat162 lo = __floats2bfloat162_rn(v[0], v[1]), hi = __floats2bfloat162_rn(v[2], v[3]);
                *reinterpret_cast<__nv_bfloat162*>(&sA[r][k]) = lo;
                *reinterpret_cast<__nv_bfloat162*>(&sA[r][k + 2]) = hi;
            }
            // weights: 64 outputs x 32 k, 8 consecutive k per thread and pass
            for (int e = tid; e < LIN_BN * (LIN_BK / 8); e += LIN_THREADS) {
                const int r = e / (LIN_BK / 8), k = (e % (LIN_BK / 8)) * 8;
                const int n = n0 + r;
                uint4 q = make_uint4(0, 0, 0, 0);
                if (n < N) {
                    const __nv_bfloat16* src = W + (size_t)n * K + k0 + k;
                    if (vecW && k0 + k + 7 < K) {
                        q = *reinterpret_cast<const uint4*>(src);
                    } else {
                        __nv_bfloat16 t[8];
#pragma unroll
                        for (int j = 0; j < 8; ++j) t[j] = (k0 + k + j < K) ? src[j] : __float2bfloat16(0.f);
                        q = *reinterpret_cast<const uint4*>(t);
                    }
                }
                *reinterpret_cast<uint4*>(&sB[r][k]) = q;
            }
            __syncthreads();
#pragma unroll
            for (int kk = 0; kk < LIN_BK; kk += 16) {
                uint32_t a[2][4], b[4][2];
#pragma unroll
                for (int i = 0; i < 2; ++i) {
                    const int r = wm + i * 16 + gq;
                    a[i][0] = *reinterpret_cast<const uint32_t*>(&sA[r][kk + tq * 2]);
                    a[i][1] = *reinterpret_cast<const uint32_t*>(&sA[r + 8][kk + tq * 2]);
                    a[i][2] = *reinterpret_cast<const uint32_t*>(&sA[r][kk + 8 + tq * 2]);
                    a[i][3] = *reinterpret_cast<const uint32_t*>(&sA[r + 8][kk + 8 + tq * 2]);
                }
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const int n = wn + j * 8 + gq;
                    b[j][0] = *reinterpret_cast<const uint32_t*>(&sB[n][kk + tq * 2]);
                    b[j][1] = *reinterpret_cast<const uint32_t*>(&sB[n][kk + 8 + tq * 2]);
                }
#pragma unroll
                for (int i = 0; i < 2; ++i)
#pragma unroll
                    for (int j = 0; j < 4; ++j) mma_bf16_16816(acc[i][j], a[i], b[j]);
            }
            __syncthreads();
        }
#pragma unroll
        for (int i = 0; i < 2; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int n = n0 + wn + j * 8 + tq * 2;
                if (n >= N) continue;
#pragma unroll
                for (int hrow = 0; hrow < 2; ++hrow) {
                    const int r = r0 + wm + i * 16 + gq + hrow * 8;
                    if (r < rows) lin_store(p, g, base + r, n, acc[i][j][hrow * 2], acc[i][j][hrow * 2 + 1], n + 1 < N);
                }
            }
    }
}

// ------------------------------------------------------------------------------------------------------------------
// skinny kernel: up to LIN_SK_ROWS rows per pass, one warp per output pair
// ------------------------------------------------------------------------------------------------------------------
constexpr int LIN_SK_ROWS = 8, LIN_SK_WARPS = 8;

__global__ void __launch_bounds__(LIN_SK_WARPS * 32) lin_skinny_kernel(const LinParams p) {
    const int g = blockIdx.z;
    const int rows = p.cnt[(size_t)g * p.cnt_gstride];
    if (rows <= 0) return;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n = (blockIdx.x * LIN_SK_WARPS + warp) * 2;
    if (n >= p.N) return;
    const bool has1 = n + 1 < p.N;
    const int base = p.off ? p.off[g] : 0;
    const float* X = p.X + g * p.x_gstride;
    const __nv_bfloat16* w0 = p.W + g * p.w_gstride + (size_t)n * p.K;
    const __nv_bfloat16* w1 = has1 ? w0 + p.K : w0;
    const int K = p.K;
    const bool vec = (K % 8 == 0) && ((reinterpret_cast<uintptr_t>(w0) & 15) == 0) && (p.ldx % 4 == 0) &&
                     ((reinterpret_cast<uintptr_t>(X) & 15) == 0);
    for (int rb = 0; rb < rows; rb += LIN_SK_ROWS) {
        const int nr = min(LIN_SK_ROWS, rows - rb);
        const float* xr[LIN_SK_ROWS];
#pragma unroll
        for (int i = 0; i < LIN_SK_ROWS; ++i) {
            const int r = rb + min(i, nr - 1);
            xr[i] = X + (size_t)(p.xlist ? p.xlist[base + r] : base + r) * p.ldx;
        }
        float a0[LIN_SK_ROWS], a1[LIN_SK_ROWS];
#pragma unroll
        for (int i = 0; i < LIN_SK_ROWS; ++i) a0[i] = a1[i] = 0.f;
        if (vec) {
            for (int k = lane * 8; k < K; k += 256) {
                const uint4 q0 = *reinterpret_cast<const uint4*>(w0 + k);
                const uint4 q1 = *reinterpret_cast<const uint4*>(w1 + k);
                const __nv_bfloat162* h0 = reinterpret_cast<const __nv_bfloat162*>(&q0);
                const __nv_bfloat162* h1 = reinterpret_cast<const __nv_bfloat162*>(&q1);
                float f0[8], f1[8];
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const float2 u = __bfloat1622float2(h0[j]), v = __bfloat1622float2(h1[j]);
                    f0[2 * j] = u.x; f0[2 * j + 1] = u.y; f1[2 * j] = v.x; f1[2 * j + 1] = v.y;
                }
#pragma unroll
                for (int i = 0; i < LIN_SK_ROWS; ++i) {
                    if (i >= nr) break;
                    const float4 xa = *reinterpret_cast<const float4*>(xr[i] + k);
                    const float4 xb = *reinterpret_cast<const float4*>(xr[i] + k + 4);
                    const float xv[8] = {xa.x, xa.y, xa.z, xa.w, xb.x, xb.y, xb.z, xb.w};
#pragma unroll
                    for (int j = 0; j < 8; ++j) { a0[i] = fmaf(xv[j], f0[j], a0[i]); a1[i] = fmaf(xv[j], f1[j], a1[i]); }
                }
            }
        } else {
            for (int k = lane; k < K; k += 32) {
                const float f0 = __bfloat162float(w0[k]), f1 = __bfloat162float(w1[k]);
#pragma unroll
                for (int i = 0; i < LIN_SK_ROWS; ++i) {
                    if (i >= nr) break;
                    const float xv = xr[i][k];
                    a0[i] = fmaf(xv, f0, a0[i]); a1[i] = fmaf(xv, f1, a1[i]);
                }
            }
        }
#pragma unroll
        for (int i = 0; i < LIN_SK_ROWS; ++i) {
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                a0[i] += __shfl_xor_sync(0xffffffffu, a0[i], o);
                a1[i] += __shfl_xor_sync(0xffffffffu, a1[i], o);
            }
        }
        if (lane == 0) {
#pragma unroll
            for (int i = 0; i < LIN_SK_ROWS; ++i)
                if (i < nr) lin_store(p, g, base + rb + i, n, a0[i], a1[i], has1);
        }
    }
}

}  // namespace b200
