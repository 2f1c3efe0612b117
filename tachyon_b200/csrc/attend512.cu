// Decode attention for the shapes attend.cu's tensor-core kernel does not take: heads of 512 (Gemma 4's global layers,
// the reference's attend_512, crates/tachyon/src/ptx/attend.rs:1-32, 423-466) and, at either head size, eight query
// heads to a key-value head (E2B: two blocks of four heads share each key-value head, the reference's `group` 2).
// Semantics are attend.cu's.  No benchmark configuration has these shapes, so the kernel is written for clarity rather
// than for the last microsecond: no shared-memory tiles, every warp walks its share of the block's positions straight
// from the cache with its own running softmax (maximum, sum, weighted values for the G query heads, DH / 32 dimensions
// a lane), the eight warps' results meet in shared memory, and splits meet as in attend.cu: partial results in scratch,
// the last block to arrive (atomic counter, no spin) merges them.
#include "common.cuh"
#include "internal.h"

#include <string>

namespace tb {

namespace {

constexpr int THREADS = 256, WARPS = THREADS / 32, MIN_SPAN = 16;

// A lane holds NV = DH / 32 values of a head: element j < NV/2 is dim (NV/2) lane + j, element NV/2 + j its RoPE partner
// DH/2 + (NV/2) lane + j.
template <int DH>
struct Wide {
    float q[4][DH];
    float kf[DH], vf[DH];
    float m[WARPS][4], l[WARPS][4];
    float acc[WARPS][4][DH];
    float mm[4], ll[4];
    uint32_t last;
};

template <int DH>
__device__ __forceinline__ int dim_of(int i, int lane) {
    constexpr int H2 = DH / 64;
    return i < H2 ? H2 * lane + i : DH / 2 + H2 * lane + i - H2;
}
// From global memory (ld.global.cg: must not be given a shared address).
template <int DH>
__device__ __forceinline__ void load_lane(const float* src, float (&x)[DH / 32], int lane) {
    constexpr int H2 = DH / 64;
#pragma unroll
    for (int half = 0; half < 2; half++)
#pragma unroll
        for (int v = 0; v < H2 / 4; v++) {
            const float4 t = ld_cg_f4(src + half * (DH / 2) + H2 * lane + 4 * v);
            x[half * H2 + v * 4] = t.x, x[half * H2 + v * 4 + 1] = t.y, x[half * H2 + v * 4 + 2] = t.z, x[half * H2 + v * 4 + 3] = t.w;
        }
}
template <int DH>
__device__ __forceinline__ void load_lane_shared(const float* src, float (&x)[DH / 32], int lane) {
    constexpr int H2 = DH / 64;
#pragma unroll
    for (int half = 0; half < 2; half++)
#pragma unroll
        for (int v = 0; v < H2 / 4; v++) {
            const float4 t = *reinterpret_cast<const float4*>(src + half * (DH / 2) + H2 * lane + 4 * v);
            x[half * H2 + v * 4] = t.x, x[half * H2 + v * 4 + 1] = t.y, x[half * H2 + v * 4 + 2] = t.z, x[half * H2 + v * 4 + 3] = t.w;
        }
}
template <int DH>
__device__ __forceinline__ void store_lane(float* dst, const float (&x)[DH / 32], int lane) {
    constexpr int H2 = DH / 64;
#pragma unroll
    for (int half = 0; half < 2; half++)
#pragma unroll
        for (int v = 0; v < H2 / 4; v++)
            *reinterpret_cast<float4*>(dst + half * (DH / 2) + H2 * lane + 4 * v) =
                make_float4(x[half * H2 + v * 4], x[half * H2 + v * 4 + 1], x[half * H2 + v * 4 + 2], x[half * H2 + v * 4 + 3]);
}
// f16 rows of the cache, four values (8 bytes) a load.
template <int DH>
__device__ __forceinline__ void load_lane_f16(const __half* src, float (&x)[DH / 32], int lane) {
    constexpr int H2 = DH / 64;
#pragma unroll
    for (int half = 0; half < 2; half++)
#pragma unroll
        for (int v = 0; v < H2 / 4; v++) {
            const uint2 t = __ldcg(reinterpret_cast<const uint2*>(src + half * (DH / 2) + H2 * lane + 4 * v));
            const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&t.x)), b = __half22float2(*reinterpret_cast<const __half2*>(&t.y));
            x[half * H2 + v * 4] = a.x, x[half * H2 + v * 4 + 1] = a.y, x[half * H2 + v * 4 + 2] = b.x, x[half * H2 + v * 4 + 3] = b.y;
        }
}
template <int DH>
__device__ __forceinline__ void store_lane_f16(__half* dst, const float (&x)[DH / 32], int lane) {
    constexpr int H2 = DH / 64;
#pragma unroll
    for (int half = 0; half < 2; half++)
#pragma unroll
        for (int v = 0; v < H2 / 4; v++) {
            const __half2 a = __floats2half2_rn(x[half * H2 + v * 4], x[half * H2 + v * 4 + 1]), b = __floats2half2_rn(x[half * H2 + v * 4 + 2], x[half * H2 + v * 4 + 3]);
            *reinterpret_cast<uint2*>(dst + half * (DH / 2) + H2 * lane + 4 * v) = make_uint2(*reinterpret_cast<const uint32_t*>(&a), *reinterpret_cast<const uint32_t*>(&b));
        }
}
// RMS norm (optional weights) and RoPE (optional; pairs (i, i + DH/2), f32 angle as tests/common/mod.rs:127-134) of a head.
template <int DH>
__device__ __forceinline__ void norm_rope_lane(float (&x)[DH / 32], bool norm, const float* w, const float* freq, uint32_t pos, float eps, int lane) {
    constexpr int NV = DH / 32, H2 = DH / 64;
    if (norm) {
        float s = 0.0f;
#pragma unroll
        for (int i = 0; i < NV; i++) s = fmaf(x[i], x[i], s);
        const float r = rsqrtf(warp_sum(s) / (float)DH + eps);
#pragma unroll
        for (int i = 0; i < NV; i++) x[i] *= r * (w ? __ldg(w + dim_of<DH>(i, lane)) : 1.0f);
    }
    if (freq != nullptr) {
#pragma unroll
        for (int i = 0; i < H2; i++) {
            float s, c;
            sincosf((float)pos * __ldg(freq + H2 * lane + i), &s, &c);
            const float a = x[i], b = x[i + H2];
            x[i] = a * c - b * s;
            x[i + H2] = b * c + a * s;
        }
    }
}

template <int DH, int G>
__global__ void __launch_bounds__(THREADS) attend_wide_kernel(const AttendParams p) {
    constexpr int NV = DH / 32;
    extern __shared__ __align__(16) uint8_t raw[];
    Wide<DH>& sm = *reinterpret_cast<Wide<DH>*>(raw);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    // Block b takes G query heads of one key-value head; with 8 query heads to a key-value head two blocks share it
    // (the reference's `group`, attend.rs:3-5) and the first of them stores the new key and value.
    const uint32_t b = blockIdx.x, sp = blockIdx.y, per_kv = p.heads / (p.kv_heads * G), g = b / per_kv;
    const bool stores = b % per_kv == 0;
    pdl_wait();
    pdl_launch_dependents();
    const uint32_t pos = ld_cg_u(p.pos), n = min(pos + 1, p.window), cur = pos % p.cap;
    // Positions per block as in attend.cu (whole multiples of 64 once a span is longer than that).
    uint32_t span = max((n + p.splits - 1) / p.splits, (uint32_t)MIN_SPAN);
    if (span > 64u) span = (span + 63u) / 64u * 64u;
    const uint32_t used = (n + span - 1) / span;
    if (sp >= used) return;
    const uint32_t a_begin = sp * span, a_end = min(n, a_begin + span);  // ages: 0 is the new token
    const bool fresh_here = p.fresh != 0 && sp == 0, norms = p.q_norm != nullptr;
    const float qscale = p.scale * 1.4426950408889634f;  // scores in base 2

    if (warp < G) {
        float x[NV];
        load_lane<DH>(p.qkv + (size_t)(b * G + warp) * DH, x, lane);
        norm_rope_lane<DH>(x, norms, p.q_norm, p.freq, pos, p.eps, lane);
#pragma unroll
        for (int i = 0; i < NV; i++) x[i] *= qscale;
        store_lane<DH>(sm.q[warp], x, lane);
    } else if (fresh_here && warp == G) {
        float x[NV];
        load_lane<DH>(p.qkv + (size_t)(p.heads + g) * DH, x, lane);
        norm_rope_lane<DH>(x, norms, p.k_norm, p.freq, pos, p.eps, lane);
        store_lane<DH>(sm.kf, x, lane);
        if (stores) store_lane_f16<DH>(p.kc + ((size_t)g * p.cap + cur) * DH, x, lane);
    } else if (fresh_here && warp == G + 1) {
        float x[NV];
        load_lane<DH>(p.qkv + (size_t)(p.heads + p.kv_heads + g) * DH, x, lane);
        norm_rope_lane<DH>(x, norms, nullptr, nullptr, pos, p.eps, lane);
        store_lane<DH>(sm.vf, x, lane);
        if (stores) store_lane_f16<DH>(p.vc + ((size_t)g * p.cap + cur) * DH, x, lane);
    }
    __syncthreads();

    // Every warp: its own running softmax over ages a_begin + warp, + 8, ...
    float qr[G][NV], acc[G][NV], m[G], l[G];
#pragma unroll
    for (int h = 0; h < G; h++) {
        load_lane_shared<DH>(sm.q[h], qr[h], lane);
        m[h] = -INFINITY, l[h] = 0.0f;
#pragma unroll
        for (int i = 0; i < NV; i++) acc[h][i] = 0.0f;
    }
    const __half* kb = p.kc + (size_t)g * p.cap * DH;
    const __half* vb = p.vc + (size_t)g * p.cap * DH;
    for (uint32_t age = a_begin + warp; age < a_end; age += WARPS) {
        const uint32_t slot = (cur + p.cap - age) % p.cap;
        const bool is_new = fresh_here && age == 0;
        float kv[NV];
        if (is_new) load_lane_shared<DH>(sm.kf, kv, lane);
        else load_lane_f16<DH>(kb + (size_t)slot * DH, kv, lane);
        float sc[G];
#pragma unroll
        for (int h = 0; h < G; h++) {
            float s = 0.0f;
#pragma unroll
            for (int i = 0; i < NV; i++) s = fmaf(qr[h][i], kv[i], s);
            sc[h] = warp_sum(s);
        }
        if (is_new) load_lane_shared<DH>(sm.vf, kv, lane);
        else load_lane_f16<DH>(vb + (size_t)slot * DH, kv, lane);
#pragma unroll
        for (int h = 0; h < G; h++) {
            const float mn = fmaxf(m[h], sc[h]), c = exp2f(m[h] - mn), e = exp2f(sc[h] - mn);
            l[h] = fmaf(l[h], c, e);
#pragma unroll
            for (int i = 0; i < NV; i++) acc[h][i] = fmaf(acc[h][i], c, e * kv[i]);
            m[h] = mn;
        }
    }
    // The eight warps' results meet: weights 2^(m_w - M).
#pragma unroll
    for (int h = 0; h < G; h++) {
        if (lane == 0) sm.m[warp][h] = m[h], sm.l[warp][h] = l[h];
        store_lane<DH>(sm.acc[warp][h], acc[h], lane);
    }
    __syncthreads();
    if (tid < G) {
        float M = -INFINITY, L = 0.0f;
        for (int w = 0; w < WARPS; w++) M = fmaxf(M, sm.m[w][tid]);
        for (int w = 0; w < WARPS; w++) L += sm.m[w][tid] == -INFINITY ? 0.0f : exp2f(sm.m[w][tid] - M) * sm.l[w][tid];
        sm.mm[tid] = M, sm.ll[tid] = L;
    }
    __syncthreads();
    float o[G][DH / THREADS];  // this thread's dims tid and tid + 256 of every head
#pragma unroll
    for (int h = 0; h < G; h++)
#pragma unroll
        for (int e = 0; e < DH / THREADS; e++) {
            float v = 0.0f;
            for (int w = 0; w < WARPS; w++)
                if (sm.m[w][h] != -INFINITY) v = fmaf(exp2f(sm.m[w][h] - sm.mm[h]), sm.acc[w][h][tid + e * THREADS], v);
            o[h][e] = v;
        }

    const uint32_t stride = 2 * G + G * DH;  // floats per partial: maxima, sums, outputs
    auto write_out = [&](int h, int e, float v) {
        const size_t at = (size_t)(b * G + h) * DH + tid + e * THREADS;
        if (p.out_f16 == 2) q8_store(v, (uint32_t)at, static_cast<int8_t*>(p.out), reinterpret_cast<float2*>(p.out_pairs));
        else if (p.out_f16) static_cast<__half*>(p.out)[at] = __float2half_rn(v);
        else static_cast<float*>(p.out)[at] = v;
    };
    if (used == 1) {
#pragma unroll
        for (int h = 0; h < G; h++)
#pragma unroll
            for (int e = 0; e < DH / THREADS; e++) write_out(h, e, o[h][e] / sm.ll[h]);
        return;
    }
    float* mine = p.partial + (size_t)(b * p.splits + sp) * stride;
    if (tid < G) mine[tid] = sm.mm[tid], mine[G + tid] = sm.ll[tid];
#pragma unroll
    for (int h = 0; h < G; h++)
#pragma unroll
        for (int e = 0; e < DH / THREADS; e++) mine[2 * G + h * DH + tid + e * THREADS] = o[h][e];
    __threadfence();
    __syncthreads();
    if (tid == 0) sm.last = (atomicAdd(p.count + b, 1u) == used - 1) ? 1u : 0u;
    __syncthreads();
    if (sm.last == 0) return;
    __threadfence();
    // Combine (attend.rs:371-405): weights 2^(m_s - M) over the splits that ran.
    const float* base = p.partial + (size_t)b * p.splits * stride;
    if (tid < G) {
        float M = -INFINITY, L = 0.0f;
        for (uint32_t s2 = 0; s2 < used; s2++) M = fmaxf(M, __ldcg(base + (size_t)s2 * stride + tid));
        for (uint32_t s2 = 0; s2 < used; s2++) L = fmaf(exp2f(__ldcg(base + (size_t)s2 * stride + tid) - M), __ldcg(base + (size_t)s2 * stride + G + tid), L);
        sm.mm[tid] = M, sm.ll[tid] = L;
    }
    __syncthreads();
#pragma unroll
    for (int h = 0; h < G; h++)
#pragma unroll
        for (int e = 0; e < DH / THREADS; e++) {
            float v = 0.0f;
            for (uint32_t s2 = 0; s2 < used; s2++)
                v = fmaf(exp2f(__ldcg(base + (size_t)s2 * stride + h) - sm.mm[h]), __ldcg(base + (size_t)s2 * stride + 2 * G + h * DH + tid + e * THREADS), v);
            write_out(h, e, v / sm.ll[h]);
        }
    if (tid == 0) p.count[b] = 0;
}

template <int DH>
int launch_wide(tb_context* ctx, const AttendParams& p, const char* who) {
    const std::string name(who);
    if (p.kv_heads == 0 || p.heads % p.kv_heads != 0) return fail(OUT_OF_RANGE, name + ": heads must be a multiple of kv_heads");
    const uint32_t ratio = p.heads / p.kv_heads, group = ratio < 4 ? ratio : 4;  // query heads per block
    if (ratio != 1 && ratio != 2 && ratio != 4 && ratio != 8) return fail(UNSUPPORTED, name + ": 1, 2, 4 or 8 query heads per key-value head");
    if (p.cap == 0 || p.window == 0 || p.window > p.cap) return fail(OUT_OF_RANGE, name + ": need 0 < window <= cap");
    if (p.splits == 0 || p.splits > 1024) return fail(OUT_OF_RANGE, name + ": splits out of range");
    if (!p.qkv || !p.kc || !p.vc || !p.pos || !p.out || !p.count || (p.splits > 1 && !p.partial)) return fail(OUT_OF_RANGE, name + ": null argument");
    if (p.out_f16 == 2 && !p.out_pairs) return fail(OUT_OF_RANGE, name + ": Q8 output needs its pairs");
    if ((p.q_norm == nullptr) != (p.k_norm == nullptr)) return fail(OUT_OF_RANGE, name + ": q_norm and k_norm go together");
    if ((reinterpret_cast<uintptr_t>(p.kc) | reinterpret_cast<uintptr_t>(p.vc) | reinterpret_cast<uintptr_t>(p.qkv)) & 15) return fail(OUT_OF_RANGE, name + ": buffers must be 16-byte aligned");
    const dim3 grid(p.heads / group, p.splits), block(THREADS);
    constexpr size_t SMEM = sizeof(Wide<DH>);
    static bool configured[16] = {};
    if (!configured[ctx->gpu & 15]) {
        TB_CUDA(cudaFuncSetAttribute(attend_wide_kernel<DH, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM));
        TB_CUDA(cudaFuncSetAttribute(attend_wide_kernel<DH, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM));
        TB_CUDA(cudaFuncSetAttribute(attend_wide_kernel<DH, 4>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM));
        configured[ctx->gpu & 15] = true;
    }
    if (group == 4) TB_CUDA(launch_kernel(ctx, attend_wide_kernel<DH, 4>, grid, block, SMEM, true, p));
    else if (group == 2) TB_CUDA(launch_kernel(ctx, attend_wide_kernel<DH, 2>, grid, block, SMEM, true, p));
    else TB_CUDA(launch_kernel(ctx, attend_wide_kernel<DH, 1>, grid, block, SMEM, true, p));
    return OK;
}

}  // namespace

int launch_attend_512(tb_context* ctx, const AttendParams& p) { return launch_wide<512>(ctx, p, "attend_512"); }
int launch_attend_256_shared(tb_context* ctx, const AttendParams& p) { return launch_wide<256>(ctx, p, "attend_256"); }

}  // namespace tb
