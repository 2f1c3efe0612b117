// Shared device helpers for the sm_100a kernels: bulk asynchronous copies with mbarrier completion, programmatic
// dependent launch, bounded waits, and small numeric utilities.
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace tb {

// Error words a kernel can leave in the context's device status word (0 = fine).
enum : uint32_t { ERR_NONE = 0, ERR_WAIT_FULL = 1, ERR_WAIT_EMPTY = 2, ERR_DRAIN = 3, ERR_GRID = 4 };

// Longest a thread polls one barrier before it gives up and reports: two seconds of %globaltimer.
constexpr unsigned long long WAIT_LIMIT_NS = 2000000000ull;

__device__ __forceinline__ uint32_t smem_addr(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

__device__ __forceinline__ unsigned long long global_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_addr(bar)), "r"(count) : "memory");
}

__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_addr(bar)), "r"(bytes) : "memory");
}

__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_addr(bar)) : "memory");
}

// mbarrier.arrive counting for `count` arrivals at once.
__device__ __forceinline__ void mbar_arrive_n(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0], %1;" ::"r"(smem_addr(bar)), "r"(count) : "memory");
}

// Adds to a counter with release semantics and without waiting for the old value.
__device__ __forceinline__ void red_release_add(uint32_t* p, uint32_t v) {
    asm volatile("red.release.gpu.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

__device__ __forceinline__ uint32_t ld_acquire_u32(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.b32 %0, 1, 0, p;\n\t}"
        : "=r"(done)
        : "r"(smem_addr(bar)), "r"(parity)
        : "memory");
    return done != 0;
}

// Waits for the phase with `parity` to complete, at most `limit` nanoseconds (WAIT_LIMIT_NS unless a caller has a reason
// for less); false when it gave up.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, unsigned long long limit = WAIT_LIMIT_NS) {
    if (mbar_try_wait(bar, parity)) return true;
    const unsigned long long start = global_ns();
    for (uint32_t spins = 0;; ++spins) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((spins & 255u) == 255u && global_ns() - start > limit) return false;
    }
}

// One-dimensional bulk copy global -> shared; `bytes` a multiple of 16, both addresses 16-byte aligned.  Completion
// is counted in bytes on `bar`.
__device__ __forceinline__ void bulk_load(void* dst_smem, const void* src_gmem, uint32_t bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(smem_addr(dst_smem)),
                 "l"(src_gmem), "r"(bytes), "r"(smem_addr(bar))
                 : "memory");
}

// An L2 policy that marks what is fetched with it as the first to evict: for data that is streamed once.
__device__ __forceinline__ uint64_t policy_evict_first() {
    uint64_t p;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(p));
    return p;
}

// bulk_load with an L2 cache policy.
__device__ __forceinline__ void bulk_load_hint(void* dst_smem, const void* src_gmem, uint32_t bytes, uint64_t* bar, uint64_t policy) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;" ::"r"(smem_addr(dst_smem)),
                 "l"(src_gmem), "r"(bytes), "r"(smem_addr(bar)), "l"(policy)
                 : "memory");
}

// Prefetch a range into L2 without a destination.
__device__ __forceinline__ void bulk_prefetch_l2(const void* src_gmem, uint32_t bytes) {
    asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(src_gmem), "r"(bytes) : "memory");
}

// One 128-byte line into the L2, through the load/store unit (it does not queue behind the bulk copies).
__device__ __forceinline__ void prefetch_line_l2(const void* p) { asm volatile("prefetch.global.L2 [%0];" ::"l"(p)); }

// Issues the L2 prefetches of a hint (see Prefetch in internal.h) for the later kernel's blocks b = first, first +
// step, ...  Called by one thread.
template <typename P>
__device__ __forceinline__ void prefetch_hint(const P& pf, uint32_t first, uint32_t step) {
    if (pf.w == nullptr || pf.bytes == 0) return;
    const uint32_t units = pf.rows / pf.unit;
    for (uint32_t b = first; b < pf.grid; b += step) {
        const uint32_t q0 = static_cast<uint32_t>((uint64_t)units * b / pf.grid) * pf.unit;
        const uint32_t q1 = static_cast<uint32_t>((uint64_t)units * (b + 1) / pf.grid) * pf.unit;
        const size_t total = (size_t)(q1 - q0) * pf.cols;
        size_t lo = pf.skip < total ? pf.skip : total, hi = lo + pf.bytes < total ? lo + pf.bytes : total;
        const char* base = reinterpret_cast<const char*>(pf.w) + (size_t)q0 * pf.cols;
        for (size_t o = lo; o < hi; o += 16384) bulk_prefetch_l2(base + o, (uint32_t)(hi - o < 16384 ? hi - o : 16384));
        const char* sb = reinterpret_cast<const char*>(pf.s) + (size_t)q0 * (pf.cols / 16);
        lo = (lo / 16) & ~(size_t)15;
        hi = ((hi / 16) + 15) & ~(size_t)15;
        if (hi > total / 16) hi = total / 16;
        for (size_t o = lo; o < hi; o += 16384) bulk_prefetch_l2(sb + o, (uint32_t)(hi - o < 16384 ? hi - o : 16384));
    }
}

// Asks the L2 for `rows` rows of a matrix from `row` on: row_bytes of codes and srow_bytes of scales a row.  One thread.
__device__ __forceinline__ void prefetch_rows_l2(const void* w, const void* s, uint32_t row, uint32_t rows, uint32_t row_bytes, uint32_t srow_bytes) {
    const char* wb = reinterpret_cast<const char*>(w) + (size_t)row * row_bytes;
    const size_t wn = (size_t)rows * row_bytes;
    for (size_t o = 0; o < wn; o += 16384) bulk_prefetch_l2(wb + o, (uint32_t)(wn - o < 16384 ? wn - o : 16384));
    const char* sb = reinterpret_cast<const char*>(s) + (size_t)row * srow_bytes;
    const size_t sn = (size_t)rows * srow_bytes;
    for (size_t o = 0; o < sn; o += 16384) bulk_prefetch_l2(sb + o, (uint32_t)(sn - o < 16384 ? sn - o : 16384));
}

// The stage form of a hint (see Prefetch in internal.h) for the block with index b.
template <typename P>
__device__ __forceinline__ void prefetch_stages(const P& pf, uint32_t b) {
    if (pf.w == nullptr || pf.stages == 0) return;
    for (uint32_t k = 0; k < pf.stages; k++) {
        const uint32_t row = (b + k * pf.grid) * pf.stage_rows;
        if (row >= pf.rows) break;
        prefetch_rows_l2(pf.w, pf.s, row, min(pf.stage_rows, pf.rows - row), pf.row_bytes, pf.srow_bytes);
    }
}

// Programmatic dependent launch: let the next kernel in the stream start its independent prologue / wait for the
// kernels before this one to have finished and their writes to be visible.
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

__device__ __forceinline__ void named_bar_sync(uint32_t id, uint32_t threads) {
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}

// The same barrier, also telling every participant whether any of them passed a true `pred`.
__device__ __forceinline__ bool named_bar_or(uint32_t id, uint32_t threads, bool pred) {
    uint32_t any;
    asm volatile(
        "{\n\t.reg .pred p, q;\n\tsetp.ne.u32 p, %1, 0;\n\tbarrier.red.or.pred q, %2, %3, p;\n\tselp.u32 %0, 1, 0, q;\n\t}"
        : "=r"(any)
        : "r"((uint32_t)pred), "r"(id), "r"(threads)
        : "memory");
    return any != 0;
}

// dp4a with signed weights: against signed / unsigned activation bytes.
__device__ __forceinline__ int dp4a_ss(uint32_t a, uint32_t b, int c) {
    int d;
    asm("dp4a.s32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}
__device__ __forceinline__ uint32_t dp4a_uu(uint32_t a, uint32_t b, uint32_t c) {
    uint32_t d;
    asm("dp4a.u32.u32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}
__device__ __forceinline__ int dp4a_su(uint32_t a, uint32_t b, int c) {
    int d;
    asm("dp4a.s32.u32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}

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

// Loads that bypass L1: activations written by an earlier (possibly overlapping) kernel.
__device__ __forceinline__ float4 ld_cg_f4(const void* p) { return __ldcg(reinterpret_cast<const float4*>(p)); }
__device__ __forceinline__ uint4 ld_cg_u4(const void* p) { return __ldcg(reinterpret_cast<const uint4*>(p)); }
__device__ __forceinline__ float ld_cg_f(const float* p) { return __ldcg(p); }
__device__ __forceinline__ uint32_t ld_cg_u(const uint32_t* p) { return __ldcg(p); }

// tanh-form GELU, as the reference's decoder computes it (crates/tachyon/src/ptx/mod.rs:376-390):
// x / (1 + 2^(-2*sqrt(2/pi)*log2(e)*(x + 0.044715 x^3))).
// Value x of element i -> the reference's Q8 (crates/tachyon/src/ptx/mod.rs:191-212): the 32 lanes of a warp hold 32
// consecutive values, one block; scale amax / 127, codes rounded to nearest even, the pair [s, s * sum q] from lane 0.
__device__ __forceinline__ void q8_store(float x, uint32_t i, int8_t* q, float2* s) {
    float amax = fabsf(x);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    const float d = __fdiv_rn(amax, 127.0f);
    const float inv = amax > 0.0f ? __fdiv_rn(127.0f, amax) : 0.0f;
    const int code = __float2int_rn(__fmul_rn(x, inv));
    q[i] = static_cast<int8_t>(code);
    int sum = code;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
    if ((i & 31u) == 0) s[i >> 5] = make_float2(d, __fmul_rn(static_cast<float>(sum), d));
}

// 0.5 x (1 + tanh(u)) = x / (1 + e^(-2u)), u = sqrt(2/pi) (x + 0.044715 x^3); the quotient by the hardware's reciprocal (2 ulp).
__device__ __forceinline__ float gelu_tanh(float x) {
    const float u = x + 0.044715f * x * x * x;
    return __fdividef(x, 1.0f + exp2f(-2.0f * 0.7978845608028654f * 1.4426950408889634f * u));
}

// erf to 1.5e-7 (Abramowitz and Stegun 7.1.26) and the exact-form GELU built on it, as the reference's encoder
// computes them (crates/tachyon/src/ptx/encoder.rs:807-841).
__device__ __forceinline__ float erf_as(float x) {
    const float t = __fdividef(1.0f, 1.0f + 0.3275911f * fabsf(x));
    const float p = t * (0.2548296f + t * (-0.28449674f + t * (1.4214137f + t * (-1.4531521f + t * 1.0614054f))));
    return copysignf(1.0f - p * __expf(-x * x), x);
}
__device__ __forceinline__ float gelu_erf(float x) { return 0.5f * x * (1.0f + erf_as(x * 0.70710678118f)); }
// The same function in thirteen instructions for the products' epilogues, which are bound by issue slots at short K:
// x Phi(x) with Phi = 1 - q (x >= 0) or q (x < 0), q = 0.5 p(t) e^(-x^2 / 2), t = 1 / (1 + 0.3275911 |x| / sqrt 2), so
// x Phi(x) = max(x, 0) - |x| q.  The 0.5 and the 1 / sqrt 2 are folded into the constants; within 5e-7 of gelu_erf.
__device__ __forceinline__ float gelu_erf_lean(float x) {
    const float a = fabsf(x);
    const float t = __fdividef(1.0f, fmaf(a, 0.3275911f * 0.70710678118f, 1.0f));
    const float p = t * (0.5f * 0.2548296f + t * (0.5f * -0.28449674f + t * (0.5f * 1.4214137f + t * (0.5f * -1.4531521f + t * (0.5f * 1.0614054f)))));
    float e;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"((x * x) * (-0.5f * 1.4426950408889634f)));
    return fmaf(-a, p * e, fmaxf(x, 0.0f));
}

// A float's bits as an unsigned key with the same order (for atomicMax on values).
__device__ __forceinline__ uint32_t float_key(float v) {
    const uint32_t b = __float_as_uint(v);
    return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}

}  // namespace tb
