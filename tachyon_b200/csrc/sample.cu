// The sampler: the reference's `sample` kernel (crates/tachyon/src/ptx/sample.rs:1-27, 91-417) with its arguments, its
// 40-byte Sampling block read from device memory (sample.rs:38-78), its transform, its hash and its exact filtered draw.
//
//   x' = softcap * tanh(x / softcap); -inf when `allowed` excludes the token; x' / penalty (x' * penalty when negative)
//   when the token was seen; x' / temperature.  Temperature 0: the largest, lowest index among equals.  Otherwise every
//   block writes its share transformed to `work`, keeps its maximum, its sum of exp(x' - max) and its Gumbel candidate
//   argmax(x' + G), G = -ln(-ln U), U from murmur3's finaliser over (seed, step, round, token) exactly as
//   sample.rs:81-88, 113-121 hash it; the last block to finish merges the blocks' results.  With top_k / top_p / min_p
//   the last block counts the tokens above the candidate and their probability mass (sample.rs:318-336: strictly greater
//   logits; kept when count < top_k, mass < top_p * Z or mass == 0, and x' >= max + ln(min_p)); a candidate that fails
//   is replaced by a fresh draw among the tokens above it, so the token follows the filtered distribution exactly;
//   after 32 failed draws the largest is taken.
//
// The approximate instructions the reference uses (ex2, lg2, rcp .approx) are used here too, through inline PTX, so a
// draw depends on the same bits of noise.  Reductions keep "greater, or equal with a lower index".
#include "common.cuh"
#include "internal.h"

namespace tb {

namespace {

constexpr int THREADS = 1024;  // sample.rs:36

__device__ __forceinline__ float ex2(float x) {
    float y;
    asm("ex2.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ float lg2(float x) {
    float y;
    asm("lg2.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ float rcp_approx(float x) {
    float y;
    asm("rcp.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ uint32_t fmix(uint32_t h) {  // sample.rs:81-82
    h ^= h >> 16, h *= 0x85EBCA6Bu, h ^= h >> 13, h *= 0xC2B2AE35u, h ^= h >> 16;
    return h;
}
// The hash of seed, step and draw every token's noise starts from (sample.rs:85-88).
__device__ __forceinline__ uint32_t noise_base(uint32_t step, uint32_t round, uint32_t seedlo, uint32_t seedhi) {
    uint32_t h = step * 0x9E3779B9u + seedhi;
    h = round * 0x85EBCA77u + h;
    return fmix(fmix(h) ^ seedlo);
}
// Token i's Gumbel noise (sample.rs:113-121): U = ((hash >> 9) + 0.5) * 2^-23, G = -ln 2 * lg2(-ln 2 * lg2 U).
__device__ __forceinline__ float gumbel(uint32_t i, uint32_t base) {
    const uint32_t h = fmix((i * 0x9E3779B9u) ^ base) >> 9;
    float u = __fmul_rn(__fadd_rn(static_cast<float>(h), 0.5f), 1.1920928955078125e-07f);
    u = __fmul_rn(lg2(u), -0.693147182464599609375f);
    return __fmul_rn(lg2(u), -0.693147182464599609375f);
}

struct Pick {
    float v;
    uint32_t i;
};
__device__ __forceinline__ void better(float v, uint32_t i, Pick& b) {  // sample.rs:91-97
    if (v > b.v || (v == b.v && i < b.i)) b.v = v, b.i = i;
}
// The block's best (value, index) in every thread (sample.rs:100-109).
__device__ __forceinline__ Pick block_argmax(Pick p, float* sv, uint32_t* si) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) better(__shfl_xor_sync(0xffffffffu, p.v, o), __shfl_xor_sync(0xffffffffu, p.i, o), p);
    if (lane == 0) sv[warp] = p.v, si[warp] = p.i;
    __syncthreads();
    p.v = sv[lane], p.i = si[lane];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) better(__shfl_xor_sync(0xffffffffu, p.v, o), __shfl_xor_sync(0xffffffffu, p.i, o), p);
    __syncthreads();
    return p;
}
__device__ __forceinline__ float block_sum(float v, float* sv) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    v = warp_sum(v);
    if (lane == 0) sv[warp] = v;
    __syncthreads();
    v = warp_sum(sv[lane]);
    __syncthreads();
    return v;
}

struct Sampling {  // sample.rs:38-78
    float softcap, temperature, top_p, min_p, penalty;
    uint32_t top_k;
    unsigned long long allowed, seed;
};
static_assert(sizeof(Sampling) == 40, "the reference's layout");

constexpr float LOG2E = 1.44269502162933349609375f;  // 0f3FB8AA3B

// trace (optional, not in the reference's list): trace[step & trace_mask] = token, for the decoder's chained runs.
__global__ void __launch_bounds__(THREADS) sample_kernel(const float* __restrict__ logits, float* work, uint32_t vocab, const Sampling* cfg, uint32_t* state,
                                                         uint32_t* seen, uint32_t* out, float* partial, uint32_t* count, uint32_t* trace, uint32_t trace_mask) {
    __shared__ float sv[32];
    __shared__ uint32_t si[32];
    __shared__ uint32_t flag;
    pdl_wait();
    const uint32_t th = threadIdx.x, nb = gridDim.x;
    const Sampling c = *cfg;
    const uint32_t step = state[0], seedlo = static_cast<uint32_t>(c.seed), seedhi = static_cast<uint32_t>(c.seed >> 32);
    const bool hcap = c.softcap > 0.0f, greedy = c.temperature <= 0.0f;
    const float isc = __fmul_rn(__frcp_rn(c.softcap), 2.8853900432586669921875f);  // 2 log2(e) / softcap
    const float sc2 = __fmul_rn(c.softcap, -2.0f);
    const float itemp = greedy ? 1.0f : __frcp_rn(c.temperature), ipen = __frcp_rn(c.penalty);
    const uint32_t* allow = reinterpret_cast<const uint32_t*>(c.allowed);
    const bool filter = c.top_k != 0 || c.top_p < 1.0f || c.min_p > 0.0f;
    uint32_t round = 0;
    uint32_t base = noise_base(step, round, seedlo, seedhi);

    Pick best{-INFINITY, 0xffffffffu}, key{-INFINITY, 0xffffffffu};
    float m = -INFINITY, z = 0.0f;
    // Transform: four tokens a thread and turn (vocab is a multiple of 4, sample.rs:26).
    for (uint32_t e = (blockIdx.x * THREADS + th) * 4; e < vocab; e += nb * THREADS * 4) {
        float4 x4 = *reinterpret_cast<const float4*>(logits + e);
        float x[4] = {x4.x, x4.y, x4.z, x4.w};
        const uint32_t sw = seen[e >> 5], aw = allow ? allow[e >> 5] : 0xffffffffu, sh = e & 31;
#pragma unroll
        for (uint32_t k = 0; k < 4; k++) {
            if (hcap) {  // softcap * tanh(x / softcap) = softcap - 2 softcap / (1 + 2^(x * 2 log2 e / softcap))
                float t = ex2(__fmul_rn(x[k], isc));
                t = rcp_approx(__fadd_rn(t, 1.0f));
                x[k] = __fmaf_rn(t, sc2, c.softcap);
            }
            if (((aw >> (sh + k)) & 1u) == 0) x[k] = -INFINITY;
            if ((sw >> (sh + k)) & 1u) x[k] = __fmul_rn(x[k], x[k] > 0.0f ? ipen : c.penalty);
            x[k] = __fmul_rn(x[k], itemp);
            const float mn = fmaxf(m, x[k]);
            if (x[k] != -INFINITY) {
                z = __fmaf_rn(z, ex2(__fmul_rn(__fsub_rn(m, mn), LOG2E)), ex2(__fmul_rn(__fsub_rn(x[k], mn), LOG2E)));
                m = mn;
            }
            better(x[k], e + k, best);
            if (!greedy) better(__fadd_rn(x[k], gumbel(e + k, base)), e + k, key);  // the threshold is -inf in the first round
        }
        *reinterpret_cast<float4*>(work + e) = make_float4(x[0], x[1], x[2], x[3]);
    }
    // Merge inside the block, publish, and let the last block merge the blocks (sample.rs:244-306).
    best = block_argmax(best, sv, si);
    z = m == -INFINITY ? 0.0f : __fmul_rn(z, ex2(__fmul_rn(__fsub_rn(m, best.v), LOG2E)));
    z = block_sum(z, sv);
    key = block_argmax(key, sv, si);
    if (th == 0) {
        float* p = partial + 8 * blockIdx.x;
        p[0] = best.v, p[1] = __uint_as_float(best.i), p[2] = z, p[3] = key.v, p[4] = __uint_as_float(key.i);
        __threadfence();
        const bool last = atomicAdd(count, 1u) == nb - 1;
        if (last) *count = 0;
        __threadfence();
        flag = last ? 1u : 0u;
    }
    __syncthreads();
    if (flag == 0) return;
    best = Pick{-INFINITY, 0xffffffffu}, key = Pick{-INFINITY, 0xffffffffu}, z = 0.0f;
    if (th < nb) {
        const float* p = partial + 8 * th;
        best.v = __ldcg(p), best.i = __float_as_uint(__ldcg(p + 1)), z = __ldcg(p + 2), key.v = __ldcg(p + 3), key.i = __float_as_uint(__ldcg(p + 4));
    }
    m = best.v;
    best = block_argmax(best, sv, si);
    z = m == -INFINITY ? 0.0f : __fmul_rn(z, ex2(__fmul_rn(__fsub_rn(m, best.v), LOG2E)));
    z = block_sum(z, sv);
    key = block_argmax(key, sv, si);
    uint32_t token = greedy ? best.i : key.i;
    if (!greedy && filter) {
        // sample.rs:307-316: the thresholds the candidate is held against.
        const float least = __fmaf_rn(lg2(c.min_p), 0.693147182464599609375f, best.v);
        const float most_mass = c.top_p >= 1.0f ? INFINITY : __fmul_rn(c.top_p, z);
        const float most = c.top_k == 0 ? INFINITY : static_cast<float>(c.top_k);
        for (;;) {
            const float lj = __ldcg(work + token);
            float cnt = 0.0f, mass = 0.0f;
            for (uint32_t e = th * 4; e < vocab; e += THREADS * 4) {
                const float4 x4 = __ldcg(reinterpret_cast<const float4*>(work + e));
                const float x[4] = {x4.x, x4.y, x4.z, x4.w};
#pragma unroll
                for (int k = 0; k < 4; k++)
                    if (x[k] > lj) cnt += 1.0f, mass = __fadd_rn(mass, ex2(__fmul_rn(__fsub_rn(x[k], best.v), LOG2E)));
            }
            cnt = block_sum(cnt, sv), mass = block_sum(mass, sv);
            const bool ok = cnt < most && (mass < most_mass || mass == 0.0f) && lj >= least;
            if (ok) break;
            round++;
            token = best.i;
            if (round >= 32) break;
            base = noise_base(step, round, seedlo, seedhi);
            key = Pick{-INFINITY, 0xffffffffu};
            for (uint32_t e = th * 4; e < vocab; e += THREADS * 4) {
                const float4 x4 = __ldcg(reinterpret_cast<const float4*>(work + e));
                const float x[4] = {x4.x, x4.y, x4.z, x4.w};
#pragma unroll
                for (uint32_t k = 0; k < 4; k++)
                    if (x[k] > lj) better(__fadd_rn(x[k], gumbel(e + k, base)), e + k, key);
            }
            key = block_argmax(key, sv, si);
            token = key.i;
        }
    }
    if (th == 0) {
        if (trace != nullptr) trace[step & trace_mask] = token;
        state[1] = token;
        state[0] = step + 1;
        atomicOr(seen + (token >> 5), 1u << (token & 31));
        if (out != nullptr) *out = token;
    }
}

}  // namespace

int launch_sample_draw(tb_context* ctx, const float* logits, float* work, uint32_t vocab, const void* cfg, uint32_t* state, uint32_t* seen, uint32_t* out,
                       float* partial, uint32_t* count, uint32_t blocks, uint32_t* trace, uint32_t trace_mask) {
    if (!logits || !work || !cfg || !state || !seen || !partial || !count) return fail(OUT_OF_RANGE, "sample: null argument");
    if (vocab == 0 || vocab % 4 != 0) return fail(OUT_OF_RANGE, "sample: the vocabulary must be a positive multiple of 4");
    if ((reinterpret_cast<uintptr_t>(logits) | reinterpret_cast<uintptr_t>(work)) & 15) return fail(OUT_OF_RANGE, "sample: logits and work must be 16-byte aligned");
    if (reinterpret_cast<uintptr_t>(cfg) & 7) return fail(OUT_OF_RANGE, "sample: the settings must be 8-byte aligned");
    // sample.rs:26-27: at most min(1024, ceil(vocab / 4096)) blocks; one per multiprocessor is enough.
    uint32_t grid = (vocab + 4 * THREADS - 1) / (4 * THREADS);
    const uint32_t most = blocks ? blocks : (uint32_t)ctx->sms;
    if (grid > most) grid = most;
    if (grid > 1024) grid = 1024;
    TB_CUDA(launch_kernel(ctx, sample_kernel, dim3(grid), dim3(THREADS), 0, true, logits, work, vocab, static_cast<const Sampling*>(cfg), state, seen, out, partial,
                          count, trace, trace_mask));
    return OK;
}

}  // namespace tb
