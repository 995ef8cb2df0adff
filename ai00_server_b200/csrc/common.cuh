// Device-side helpers shared by all kernels (sm_100a only).
#pragma once
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace b200 {

// ---------------------------------------------------------------------------------------
// Per-step metadata, one flat int array in HBM (rewritten by a single H2D copy per step so
// the captured CUDA graph never changes).  Layout: header, then arrays sized by the
// engine's token_chunk (maxT) and max_batch (maxS).
// ---------------------------------------------------------------------------------------
struct MetaView {
    const int* base;
    int maxT, maxS;
    __host__ __device__ int T() const { return base[0]; }        // tokens this step
    __host__ __device__ int nslots() const { return base[1]; }   // active slots this step
    __host__ __device__ int R() const { return base[2]; }        // logits rows this step
    __host__ __device__ const int* tok() const { return base + 8; }                       // [maxT] token ids
    __host__ __device__ const int* tok_slot() const { return base + 8 + maxT; }           // [maxT] state slot of token
    __host__ __device__ const int* tok_prev() const { return base + 8 + 2 * maxT; }       // [maxT] t-1 or -1 (take shift state)
    __host__ __device__ const int* tok_last() const { return base + 8 + 3 * maxT; }       // [maxT] 1 if last token of its slot in this step
    __host__ __device__ const int* out_tok() const { return base + 8 + 4 * maxT; }        // [maxT] logits row r -> token index
    __host__ __device__ const int* tok_outrow() const { return base + 8 + 5 * maxT; }     // [maxT] token -> logits row or -1
    __host__ __device__ const int* slot_id() const { return base + 8 + 6 * maxT; }        // [maxS] active slot -> state slot
    __host__ __device__ const int* slot_start() const { return base + 8 + 6 * maxT + maxS; }
    __host__ __device__ const int* slot_count() const { return base + 8 + 6 * maxT + 2 * maxS; }
    __host__ __device__ static size_t ints(int maxT, int maxS) { return 8 + 6 * (size_t)maxT + 3 * (size_t)maxS; }
};

// cosine and sine of position * frequency: the product and its reduction to [-pi, pi] in double (a float product is off by
// 1e-4 rad at a few thousand tokens), the functions themselves in f32 on the reduced angle
__device__ __forceinline__ void rot_cos_sin(int pos, double freq, float& cs, float& sn) {
    double a = (double)pos * freq;
    a -= 6.283185307179586 * rint(a * 0.15915494309189535);
    sincosf((float)a, &sn, &cs);
}

// ---------------------------------------------------------------------------------------
// "A16" activation layout: the f16 operand of every projection, stored so that (a) the slice a GEMM stage needs -- one
// 128-wide k block of ALL tokens of the step -- is ONE contiguous run (one bulk TMA copy) and (b) that run IS the UMMA
// canonical K-major / no-swizzle operand of `th` token rows, which ONE tcgen05.mma with N = th consumes:
//   [k block (128 k)][k8 chunk 16][th token rows][8 halves]      (8 rows x 16 B = one 128-byte core matrix)
// th = 16 x (token tiles of the step) = 16 / 32 / 64 / 128; a step's producers and consumers agree on it (the engine passes
// it to every launch).  Measured (profiles/r02_findings.md §8): a tcgen05.mma with N = 16 costs ~80 cycles whatever N is, so
// eight N = 16 MMAs per k step (128-token steps) made the projections MMA-bound; one N = 128 MMA does not.
// Split operands (precision 1): th = 32, rows 0-15 hold the hi halves of the 16 tokens, rows 16-31 the lo halves.
// Every buffer reserves 128 token rows per k block and K padded to whole k blocks (padding k is multiplied by zero weights).
// ---------------------------------------------------------------------------------------
constexpr int A16_MAX_ROWS = 128;                      // token rows per k block: steps of up to 128 tokens
constexpr int A16_KB_HALVES = A16_MAX_ROWS * 128;      // halves per k block of a buffer
__host__ __device__ inline size_t a16_index(int m, int k, int th) {
    return (size_t)(k >> 7) * A16_KB_HALVES + ((size_t)((k >> 3) & 15) * th + m) * 8 + (k & 7);
}

__device__ __forceinline__ __half f2h_sat(float v) {
    v = fminf(fmaxf(v, -65504.f), 65504.f);
    return __float2half_rn(v);
}
// Split operand (precision 1 = f32 activations): a projection input v travels as two f16 numbers hi + lo = v
// (to ~2^-22 relative); hi sits at token row t, lo at row t + 16 of the same A16 buffer (the second 16-token tile), the
// projection multiplies both tiles and its epilogue adds the two accumulator tiles.
__device__ __forceinline__ void split_h(const float v, __half& hi, __half& lo) {
    hi = f2h_sat(v);
    lo = __float2half_rn(v - __half2float(hi));
}
__device__ __forceinline__ uint32_t pack_h2(float a, float b) {
    __half2 h = __halves2half2(f2h_sat(a), f2h_sat(b));
    return *reinterpret_cast<uint32_t*>(&h);
}

__device__ __forceinline__ void split_pack_h2(const float a, const float b, uint32_t& hi, uint32_t& lo) {
    __half ah, al, bh, bl;
    split_h(a, ah, al);
    split_h(b, bh, bl);
    __half2 h = __halves2half2(ah, bh), l = __halves2half2(al, bl);
    hi = *reinterpret_cast<uint32_t*>(&h);
    lo = *reinterpret_cast<uint32_t*>(&l);
}

// ---------------------------------------------------------------------------------------
// mbarrier + 1-D bulk TMA (cp.async.bulk)
// ---------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_fence_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
// ---------------------------------------------------------------------------------------
// Watchdog: every spin-wait in this library gives up after ~2 s, writes a record to mapped pinned
// host memory (so it survives the dead context) and traps: a protocol bug becomes a CUDA error
// with a diagnosis instead of a hung GPU.  g_watchdog is set once per process by the host.
// record: [0]=0xDEAD0000|code [1]=blockIdx.x [2]=threadIdx.x [3]=arg0 [4]=arg1 [5]=arg2
// ---------------------------------------------------------------------------------------
__device__ unsigned* g_watchdog = nullptr;
constexpr unsigned long long WATCHDOG_NS = 2000000000ull;
__device__ __forceinline__ unsigned long long globaltimer_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}
__device__ __noinline__ void watchdog_fire(unsigned code, unsigned a0, unsigned a1, unsigned a2) {
    unsigned* w = g_watchdog;
    if (w) {
        w[1] = blockIdx.x; w[2] = threadIdx.x; w[3] = a0; w[4] = a1; w[5] = a2;
        __threadfence_system();
        w[0] = 0xDEAD0000u | code;
        __threadfence_system();
    }
    __trap();
}
struct SpinGuard {          // poll(): call once per spin iteration
    unsigned n = 0;
    unsigned long long t0 = 0;
    __device__ __forceinline__ void poll(unsigned code, unsigned a0, unsigned a1, unsigned a2) {
        if ((++n & 0x3FFu) == 0) {
            const unsigned long long t = globaltimer_ns();
            if (t0 == 0) t0 = t;
            else if (t - t0 > ((code == 2u || code == 3u) ? 2 * WATCHDOG_NS : WATCHDOG_NS)) watchdog_fire(code, a0, a1, a2);   // passive waiters (grid barrier, phase start) wait longest: the culprit reports first
        }
    }
};
enum WatchCode : unsigned { WD_MBAR = 1, WD_GRIDBAR = 2 };

__device__ __forceinline__ bool mbar_try(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
// `tag` identifies the call site in watchdog reports
__device__ __forceinline__ void mbar_wait(uint32_t bar, uint32_t parity, unsigned tag = 0) {
    if (mbar_try(bar, parity)) return;
    SpinGuard g;
    while (!mbar_try(bar, parity)) g.poll(WD_MBAR, bar, parity, tag);
}
// fire-and-forget request to bring [p, p + bytes) into L2 (bytes % 16 == 0)
__device__ __forceinline__ void bulk_prefetch_l2(const void* p, uint32_t bytes) {
    asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(p), "r"(bytes) : "memory");
}
// L2 policy for streamed-once weights
__device__ __forceinline__ uint64_t l2_policy_evict_first() {
    uint64_t pol;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(pol));
    return pol;
}
__device__ __forceinline__ uint64_t l2_policy_evict_last() {
    uint64_t pol;
    asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(pol));
    return pol;
}
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
                 "l"(src), "r"(bytes), "r"(bar)
                 : "memory");
}
__device__ __forceinline__ void bulk_g2s_hint(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar,
                                              uint64_t policy) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;" ::"r"(
            dst),
        "l"(src), "r"(bytes), "r"(bar), "l"(policy)
        : "memory");
}
__device__ __forceinline__ bool mbar_test(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async;" ::: "memory"); }
// fire-and-forget arrival: no value comes back, so the arriving thread pays a one-way trip
__device__ __forceinline__ void red_add_release_gpu(unsigned* p, unsigned v) {
    asm volatile("red.release.gpu.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned ld_acquire_gpu(const unsigned* p) {
    unsigned v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_release_gpu(unsigned* p, unsigned v) {
    asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned atom_add_acq_rel_gpu(unsigned* p, unsigned v) {
    unsigned old;
    asm volatile("atom.add.acq_rel.gpu.global.u32 %0, [%1], %2;" : "=r"(old) : "l"(p), "r"(v) : "memory");
    return old;
}
__device__ __forceinline__ unsigned ld_relaxed_gpu(const unsigned* p) {
    unsigned v;
    asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_relaxed_gpu(unsigned* p, unsigned v) {
    asm volatile("st.relaxed.gpu.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint4 lds128(uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
    return v;
}
__device__ __forceinline__ void named_bar_sync(int id, int nthreads) {
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(nthreads) : "memory");
}

// D[16x8] += A[16x16] * B[16x8], f16 operands, f32 accumulate (legacy tensor path: HMMA)
__device__ __forceinline__ void mma_16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                          uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// ---------------------------------------------------------------------------------------
// tcgen05 (5th-gen tensor core) wrappers: TMEM allocation, single-thread MMA issue, commit to an
// mbarrier, TMEM -> register loads.
// ---------------------------------------------------------------------------------------
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
// whole warp; writes the TMEM base address to shared memory at `smem_dst`
__device__ __forceinline__ void tc_alloc(uint32_t smem_dst, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_dst), "r"(ncols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tc_dealloc(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
// shared-memory matrix descriptor, K-major, no swizzle: core matrix = 8 rows x 16 bytes (128 B
// contiguous); lbo = byte distance between the two 16-byte k chunks of one k16 step, sbo = byte
// distance between 8-row groups.  Bits [46,48) = 1: Blackwell descriptor version.
__device__ __forceinline__ uint64_t umma_desc(uint32_t saddr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
    return (uint64_t)((saddr & 0x3FFFFu) >> 4) | ((uint64_t)((lbo_bytes >> 4) & 0x3FFFu) << 16) |
           ((uint64_t)((sbo_bytes >> 4) & 0x3FFFu) << 32) | (1ull << 46);
}
// instruction descriptor, kind::f16: f16 x f16 -> f32, both operands K-major
__host__ __device__ constexpr uint32_t umma_idesc_f16(int M, int N) {
    return (1u << 4) | ((uint32_t)(N >> 3) << 17) | ((uint32_t)(M >> 4) << 24);
}
__device__ __forceinline__ void tc_mma_f16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
        "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// same, A operand (M = 128 rows x K = 16) read from tensor memory: lane m = row m, 8 columns of two f16 each (k even in the low half)
__device__ __forceinline__ void tc_mma_f16_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}" ::"r"(d_tmem),
        "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// 16 registers per thread -> 32 lanes x 16 consecutive 32-bit columns (lane i of the warp = TMEM lane base+i)
__device__ __forceinline__ void tc_st16(uint32_t taddr, const uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};" ::"r"(taddr),
        "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]),
        "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
        : "memory");
}
__device__ __forceinline__ void tc_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
// arrive on an mbarrier once all previously issued MMAs of this thread have completed
__device__ __forceinline__ void tc_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
// 32 lanes x 16 consecutive 32-bit columns -> 16 registers per thread (lane i of the warp = TMEM lane base+i)
__device__ __forceinline__ void tc_ld16(uint32_t taddr, float (&v)[16]) {
    uint32_t r[16];
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr)
        : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(r[i]);
}

// Programmatic dependent launch: everything before griddepcontrol.wait may overlap the tail of the preceding kernel in the
// stream / graph (weights and step metadata are immutable while a step runs, so prefetching them may).
// profiling aid: globaltimer stamp i of this launch's trace row (CTA 0, thread 0 only; `tr` is null in production)
__device__ __forceinline__ void trace_stamp(unsigned long long* tr, const int i) {
    if (tr && blockIdx.x == 0 && blockIdx.y == 0 && threadIdx.x == 0) {
        unsigned long long t;
        asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
        tr[i] = t;
    }
}
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// ---------------------------------------------------------------------------------------
// reductions
// ---------------------------------------------------------------------------------------
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}
// block-wide sum over 256 threads; `red` is >= 8 floats of shared memory; result broadcast
constexpr int CONSUMER_THREADS = 256;
__device__ __forceinline__ float block_sum(float v, float* red) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    v = warp_sum(v);
    __syncthreads();   // protect `red` from the previous use
    if (lane == 0) red[warp] = v;
    __syncthreads();
    float t = (lane < CONSUMER_THREADS / 32) ? red[lane] : 0.f;
    t = warp_sum(t);
    return t;
}
// generic versions for kernels with other block sizes (softmax)
__device__ __forceinline__ float block_sum_any(float v, float* red) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    __syncthreads();
    if (lane == 0) red[warp] = v;
    __syncthreads();
    float t = (lane < nw) ? red[lane] : 0.f;
    t = warp_sum(t);
    return t;
}
__device__ __forceinline__ float block_max_any(float v, float* red) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
    v = warp_max(v);
    __syncthreads();
    if (lane == 0) red[warp] = v;
    __syncthreads();
    float t = (lane < nw) ? red[lane] : -INFINITY;
    t = warp_max(t);
    return t;
}

// ---------------------------------------------------------------------------------------
// activations (exact-ish: expf/tanhf, not the fast intrinsics, to stay inside the 1e-3 budget)
// ---------------------------------------------------------------------------------------
enum Act : int { ACT_NONE = 0, ACT_TANH, ACT_SIGMOID, ACT_SILU, ACT_RELU2, ACT_EXPNEGEXP, ACT_V7DECAY };

__device__ __forceinline__ float sigmoidf_(float x) { return 1.f / (1.f + expf(-x)); }
__device__ __forceinline__ float apply_act(float v, int act) {
    switch (act) {
        case ACT_TANH: return tanhf(v);
        case ACT_SIGMOID: return sigmoidf_(v);
        case ACT_SILU: return v * sigmoidf_(v);
        case ACT_RELU2: { float r = fmaxf(v, 0.f); return r * r; }
        case ACT_EXPNEGEXP: return expf(-expf(v));                       // v6 decay
        case ACT_V7DECAY: return expf(-0.606531f * sigmoidf_(v));        // v7 decay, exp(-0.5)
        default: return v;
    }
}

}  // namespace b200
