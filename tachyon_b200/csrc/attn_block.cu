// The attention half of a decode layer as ONE kernel: the residual step and RMS-norm, the query/key/value product, the
// head norms and rotation, the cache append, attention over the window, and the output projection
// (crates/tachyon/src/model/decode.rs:596-630: norm_q8 + gemv_q4 on qkv, attend_256, gemv_q4 on o).
//
// Why: as three launches those phases take 15.8 us of a 35.5 us layer for 11 MB of the layer's 119 MB; what they spend is
// three hand-overs through the L2 (a dependent launch seeing its predecessor's end, then a chain of L2 round trips to
// fetch what it wrote), not bandwidth.  Here the hand-overs stay on chip: one thread-block cluster of 16 blocks per
// key-value head (two clusters, 32 SMs) runs all three phases and passes vectors between its blocks through distributed
// shared memory, with `barrier.cluster` (hardware, nothing spins) between phases.  The 116 other SMs are free for the
// gate/up product behind it to move in and fill its rings.
//
//   before the wait  every warp loads its three rows of the group's q/k/v matrix slice into registers (96 rows a block: 64 of
//                    q, 16 of k, 16 of v), the block's 128 rows x 1024 columns of the output projection go to shared memory
//                    by cp.async, and the first tile of old cache rows is fetched (position and cache do not depend on
//                    the kernel in front);
//   phase A          x = the residual step + RMS-norm as planes (every block, redundantly); three dot products a warp;
//                    every result is written into all 16 blocks' shared memory; cluster barrier;
//   phase B          head norms + RoPE (every block), block 0 appends the new key/value row to the cache; the window is
//                    cut into 16 runs of positions, one a block: a warp a position for the scores, a thread an output
//                    dimension for the values, passes of 32 positions with a running maximum;
//   merge            reduce-scatter: block o receives every block's maxima, sums and 64 of the 1024 outputs, merges
//                    them and writes the normalised 64 values to all blocks; two cluster barriers;
//   phase C          the group's 1024 attention outputs as planes; 128 rows of the output projection over the group's
//                    1024 columns from shared memory; the partial product goes to y[group]: the product behind adds the two.
// Shapes: hidden 2048, 8 query heads and 2 key-value heads of 256, eight-bit weights, a layer with a cache of its own.
// Anything else keeps the three launches.
#include <cuda.h>

#include "attend_body.cuh"
#include "common.cuh"
#include "internal.h"
#include "planes.cuh"

namespace tb {

namespace {

namespace ab {

constexpr int CL = 16;                     // blocks of a cluster
constexpr int NT = 1024, NW = NT / 32;     // threads and warps of a block
constexpr int HID = 2048, HD = 256, GQ = 4, KVH = 2;
constexpr int QROWS = GQ * HD / CL;        // 64 rows of q a block
constexpr int KROWS = HD / CL;             // 16 rows of k, and of v
constexpr int AROWS = QROWS + 2 * KROWS;   // 96 rows of phase A a block: three a warp
constexpr int OROWS = HID / CL;            // 128 rows of the output projection a block: four a warp
constexpr int OCOLS = GQ * HD;             // 1024 columns: the group's heads
constexpr int PASS = 32;                   // positions a pass: one a warp
static_assert(AROWS == 3 * NW && OROWS == 4 * NW && OCOLS == 32 * 32, "the work is cut for 32 warps");

struct Smem {
    // planes of the phase's input vector (2048 values in phase A, 1024 in phase C): a word per four values
    uint32_t hi[HID / 4], mid[HID / 4], lo[HID / 4];
    float mul[HID / 32];
    float4 sums[NW];
    float qkv[GQ * HD + 2 * HD];  // phase A's results of the group, from all blocks: q [1024], k [256], v [256]
    float q[GQ][HD];              // after norm, rotation and scale
    float kf[HD], vf[HD];         // the new key and value, f32
    float s[PASS][GQ];            // scores of a pass, then its probabilities
    float mrun[GQ], lrun[GQ], corr[GQ];
    float in_ml[CL][2 * GQ];      // merge: every block's maxima and sums
    float in_acc[CL][OCOLS / CL]; // merge: every block's 64 outputs of this block's slice
    float att[OCOLS];             // the group's normalised attention outputs, from the 16 owners
    __half v[2][PASS][HD];        // value rows of a pass, double-buffered
    __half so[OROWS][OCOLS / 32]; // scales of the output projection's slice
    alignas(16) int8_t wo[OROWS][OCOLS];  // its codes
};
static_assert(sizeof(Smem) <= 232448 - 1024, "over the 227 KiB a block may use");

__device__ __forceinline__ uint32_t cluster_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void cluster_sync() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// The address, in the cluster's shared window, of this block's shared address `local` in block `cta`.
__device__ __forceinline__ uint32_t in_cta(const void* local, uint32_t cta) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr(local)), "r"(cta));
    return r;
}
__device__ __forceinline__ void st_cluster(uint32_t addr, float v) { asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(addr), "f"(v) : "memory"); }

// The global row of the q/k/v matrix behind local row r of block `rank` in group g.
__device__ __forceinline__ uint32_t qkv_row(uint32_t g, uint32_t rank, uint32_t r) {
    if (r < QROWS) return g * (GQ * HD) + rank * QROWS + r;
    if (r < QROWS + KROWS) return KVH * GQ * HD + g * HD + rank * KROWS + (r - QROWS);
    return KVH * GQ * HD + KVH * HD + g * HD + rank * KROWS + (r - QROWS - KROWS);
}
// Where that row's result lies in Smem::qkv.
__device__ __forceinline__ uint32_t qkv_slot(uint32_t rank, uint32_t r) {
    if (r < QROWS) return rank * QROWS + r;
    if (r < QROWS + KROWS) return GQ * HD + rank * KROWS + (r - QROWS);
    return GQ * HD + HD + rank * KROWS + (r - QROWS - KROWS);
}

// Four values of the vector into the planes (virtual thread idx of len / 4; eight neighbours share a block of 32).
__device__ __forceinline__ void store_planes4(Smem& sm, int idx, float v0, float v1, float v2, float v3) {
    float amax = fmaxf(fmaxf(fabsf(v0), fabsf(v1)), fmaxf(fabsf(v2), fabsf(v3)));
#pragma unroll
    for (int o = 4; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    const uint32_t eb = min(__float_as_uint(amax) >> 23, 254u);
    const bool zero = eb < 22u;
    const float sc = zero ? 0.0f : __uint_as_float((275u - eb) << 23);
    const int x0 = __float2int_rn(v0 * sc), x1 = __float2int_rn(v1 * sc), x2 = __float2int_rn(v2 * sc), x3 = __float2int_rn(v3 * sc);
    sm.hi[idx] = pack_bytes(x0, x1, x2, x3, 0x0062);
    sm.mid[idx] = pack_bytes(x0, x1, x2, x3, 0x0051);
    sm.lo[idx] = pack_bytes(x0, x1, x2, x3, 0x0040);
    if ((idx & 7) == 0) sm.mul[idx >> 3] = zero ? 0.0f : __uint_as_float((eb - 21u) << 23);
}

// The same with two values a thread (thread idx of len / 2; sixteen neighbours share a block of 32): the even thread of a pair
// packs the pair's four values into the planes' word idx / 2.  All 32 lanes call it.
__device__ __forceinline__ void store_planes2(Smem& sm, int idx, float v0, float v1) {
    float amax = fmaxf(fabsf(v0), fabsf(v1));
#pragma unroll
    for (int o = 8; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    const uint32_t eb = min(__float_as_uint(amax) >> 23, 254u);
    const bool zero = eb < 22u;
    const float sc = zero ? 0.0f : __uint_as_float((275u - eb) << 23);
    const int x0 = __float2int_rn(v0 * sc), x1 = __float2int_rn(v1 * sc);
    const int x2 = __shfl_down_sync(0xffffffffu, x0, 1), x3 = __shfl_down_sync(0xffffffffu, x1, 1);
    if ((idx & 1) == 0) {
        sm.hi[idx >> 1] = pack_bytes(x0, x1, x2, x3, 0x0062);
        sm.mid[idx >> 1] = pack_bytes(x0, x1, x2, x3, 0x0051);
        sm.lo[idx >> 1] = pack_bytes(x0, x1, x2, x3, 0x0040);
    }
    if ((idx & 15) == 0) sm.mul[idx >> 4] = zero ? 0.0f : __uint_as_float((eb - 21u) << 23);
}

// The integer dot product of 32 codes (two 16-byte chunks) with block b's planes, plane by plane to keep registers few.
__device__ __forceinline__ float dot_block(const Smem& sm, int b, const uint4& a, const uint4& c) {
    const uint32_t w[8] = {a.x, a.y, a.z, a.w, c.x, c.y, c.z, c.w};
    int h = 0, m = 0, l = 0;
    {
        const uint4 p0 = reinterpret_cast<const uint4*>(sm.hi)[2 * b], p1 = reinterpret_cast<const uint4*>(sm.hi)[2 * b + 1];
        const uint32_t p[8] = {p0.x, p0.y, p0.z, p0.w, p1.x, p1.y, p1.z, p1.w};
#pragma unroll
        for (int k = 0; k < 8; k++) h = dp4a_ss(w[k], p[k], h);
    }
    {
        const uint4 p0 = reinterpret_cast<const uint4*>(sm.mid)[2 * b], p1 = reinterpret_cast<const uint4*>(sm.mid)[2 * b + 1];
        const uint32_t p[8] = {p0.x, p0.y, p0.z, p0.w, p1.x, p1.y, p1.z, p1.w};
#pragma unroll
        for (int k = 0; k < 8; k++) m = dp4a_su(w[k], p[k], m);
    }
    {
        const uint4 p0 = reinterpret_cast<const uint4*>(sm.lo)[2 * b], p1 = reinterpret_cast<const uint4*>(sm.lo)[2 * b + 1];
        const uint32_t p[8] = {p0.x, p0.y, p0.z, p0.w, p1.x, p1.y, p1.z, p1.w};
#pragma unroll
        for (int k = 0; k < 8; k++) l = dp4a_su(w[k], p[k], l);
    }
    return fmaf(static_cast<float>(h), 65536.0f, static_cast<float>(m * 256 + l));
}

// The same for two rows at once (one set of plane words serves both).
__device__ __forceinline__ void dot_block2(const Smem& sm, int b, const uint4& a0, const uint4& c0, const uint4& a1, const uint4& c1, float& r0, float& r1) {
    const uint32_t w0[8] = {a0.x, a0.y, a0.z, a0.w, c0.x, c0.y, c0.z, c0.w}, w1[8] = {a1.x, a1.y, a1.z, a1.w, c1.x, c1.y, c1.z, c1.w};
    int h0 = 0, m0 = 0, l0 = 0, h1 = 0, m1 = 0, l1 = 0;
    {
        const uint4 p0 = reinterpret_cast<const uint4*>(sm.hi)[2 * b], p1 = reinterpret_cast<const uint4*>(sm.hi)[2 * b + 1];
        const uint32_t p[8] = {p0.x, p0.y, p0.z, p0.w, p1.x, p1.y, p1.z, p1.w};
#pragma unroll
        for (int k = 0; k < 8; k++) h0 = dp4a_ss(w0[k], p[k], h0), h1 = dp4a_ss(w1[k], p[k], h1);
    }
    {
        const uint4 p0 = reinterpret_cast<const uint4*>(sm.mid)[2 * b], p1 = reinterpret_cast<const uint4*>(sm.mid)[2 * b + 1];
        const uint32_t p[8] = {p0.x, p0.y, p0.z, p0.w, p1.x, p1.y, p1.z, p1.w};
#pragma unroll
        for (int k = 0; k < 8; k++) m0 = dp4a_su(w0[k], p[k], m0), m1 = dp4a_su(w1[k], p[k], m1);
    }
    {
        const uint4 p0 = reinterpret_cast<const uint4*>(sm.lo)[2 * b], p1 = reinterpret_cast<const uint4*>(sm.lo)[2 * b + 1];
        const uint32_t p[8] = {p0.x, p0.y, p0.z, p0.w, p1.x, p1.y, p1.z, p1.w};
#pragma unroll
        for (int k = 0; k < 8; k++) l0 = dp4a_su(w0[k], p[k], l0), l1 = dp4a_su(w1[k], p[k], l1);
    }
    r0 = fmaf(static_cast<float>(h0), 65536.0f, static_cast<float>(m0 * 256 + l0));
    r1 = fmaf(static_cast<float>(h1), 65536.0f, static_cast<float>(m1 * 256 + l1));
}

}  // namespace ab

using namespace ab;
using attend::cp_async_16;
using attend::cp_async_commit;
using attend::cp_async_wait_all;
using attend::norm_rope;
using attend::rope_trig;
using attend::store_head;
using attend::store_head_f16;
using attend::Trig;

__global__ void __launch_bounds__(NT, 1) attn_block_kernel(const AttnBlockParams p) {
    extern __shared__ __align__(128) uint8_t raw[];
    Smem& sm = *reinterpret_cast<Smem*>(raw);
    const int t = threadIdx.x, warp = t >> 5, lane = t & 31;
    const uint32_t rank = cluster_rank(), g = blockIdx.y;
    pdl_launch_dependents();  // nothing it writes is read before a kernel's own wait

    // ---- before the wait: weights, the position, the first tile of old rows ------------------------------------------
    // Rows warp and warp + 32 of the block's 96 go to registers, row warp + 64 (a key or value row) to shared memory, where the
    // second half of the output projection's slice will lie later: the register file cannot hold all three and a working set.
    uint4 w[2][4];
    float ws[3][2];
#pragma unroll
    for (int j = 0; j < 3; j++) {
        const uint32_t row = qkv_row(g, rank, warp + 32 * j);
        const uint4* wr = reinterpret_cast<const uint4*>(p.wqkv + (size_t)row * HID);
        if (j < 2) {
            w[j][0] = __ldcs(wr + 2 * lane), w[j][1] = __ldcs(wr + 2 * lane + 1);
            w[j][2] = __ldcs(wr + 64 + 2 * lane), w[j][3] = __ldcs(wr + 64 + 2 * lane + 1);
        } else {
            int8_t* dst = &sm.wo[OROWS / 2][0] + (size_t)warp * HID;
#pragma unroll
            for (int c = 0; c < 4; c++) cp_async_16(dst + (lane + 32 * c) * 16, reinterpret_cast<const int8_t*>(wr) + (lane + 32 * c) * 16);
        }
        const __half* sr = p.sqkv + (size_t)row * (HID / 32);
        ws[j][0] = __half2float(__ldcs(sr + lane)), ws[j][1] = __half2float(__ldcs(sr + lane + 32));
    }
    // The block's slice of the output projection: rows rank * 128 .., columns g * 1024 ..: its first 64 rows and all its
    // scales now, the other 64 rows once phase A has read its third rows (asked into the L2 now).
#pragma unroll
    for (int i = 0; i < (OROWS / 2) * (OCOLS / 16) / NT; i++) {
        const int id = t + NT * i, r = id / (OCOLS / 16), c = id % (OCOLS / 16);
        cp_async_16(&sm.wo[r][c * 16], p.wo + (size_t)(rank * OROWS + r) * HID + g * OCOLS + c * 16);
    }
    if (t < OROWS * 4) {
        const int r = t / 4, c = t % 4;
        cp_async_16(&sm.so[r][c * 8], p.so + (size_t)(rank * OROWS + r) * (HID / 32) + g * (OCOLS / 32) + c * 8);
    }
    cp_async_commit();
    if (t < (OROWS / 2) * (OCOLS / 128)) prefetch_line_l2(p.wo + (size_t)(rank * OROWS + OROWS / 2 + t / (OCOLS / 128)) * HID + g * OCOLS + (t % (OCOLS / 128)) * 128);
    // The window's positions by age (0 is the new token), cut into CL runs; this block's run is [a_begin, a_end).
    const uint32_t pos = ld_cg_u(p.pos), n = min(pos + 1, p.window), cur = pos % p.cap;
    const uint32_t span = (n + CL - 1) / CL;
    const uint32_t a_begin = min(n, rank * span), a_end = min(n, a_begin + span);
    const __half* kb = p.kc + (size_t)g * p.cap * HD;
    const __half* vb = p.vc + (size_t)g * p.cap * HD;
    auto slot_of = [&](uint32_t age) { return (cur + p.cap - age) % p.cap; };
    // A pass's key row of this warp into registers, its value rows into sm.v[buf] (a thread a 16-byte piece); the new
    // token's row (age 0) is not in the cache yet and comes from kf / vf.
    auto fetch_pass = [&](uint32_t a0, int buf, uint4& kreg) {
        const uint32_t age = a0 + (uint32_t)warp;
        kreg = make_uint4(0u, 0u, 0u, 0u);
        if (age < a_end && age != 0) kreg = __ldg(reinterpret_cast<const uint4*>(kb + (size_t)slot_of(age) * HD) + lane);
        if (age < a_end && age != 0) cp_async_16(&sm.v[buf][warp][lane * 8], vb + (size_t)slot_of(age) * HD + lane * 8);
        cp_async_commit();
    };
    uint4 kreg;
    fetch_pass(a_begin, 0, kreg);
    unsigned long long* stamp = nullptr;
    if (p.stamps != nullptr && t == 0 && ((g == 0 && rank == 0) || (g == KVH - 1 && rank == CL - 1))) stamp = p.stamps + (g == 0 ? 0 : 4);
    if (stamp) stamp[0] = global_ns();
    pdl_wait();
    if (stamp) stamp[1] = global_ns();

    // ---- phase A: the residual step and RMS-norm as planes (ptx/mod.rs:24-30), two values a thread; then three rows a warp
    {
        const size_t at = (size_t)t * 2;
        const float2 h = __ldcg(reinterpret_cast<const float2*>(p.h + at));
        float2 a = make_float2(0.0f, 0.0f);
        float sy = 0.0f;
        if (p.yres != nullptr) {
            const float2 y = __ldcg(reinterpret_cast<const float2*>(p.yres + at)), w1 = __ldg(reinterpret_cast<const float2*>(p.w1 + at));
            a = make_float2(y.x * w1.x, y.y * w1.y);
            sy = y.x * y.x + y.y * y.y;
        }
        float sh = h.x * h.x + h.y * h.y, sha = h.x * a.x + h.y * a.y, sa = a.x * a.x + a.y * a.y;
        sy = warp_sum(sy), sh = warp_sum(sh), sha = warp_sum(sha), sa = warp_sum(sa);
        if (lane == 0) sm.sums[warp] = make_float4(sy, sh, sha, sa);
        __syncthreads();
        sy = sh = sha = sa = 0.0f;
#pragma unroll 8
        for (int k = 0; k < NW; k++) {
            const float4 u = sm.sums[k];
            sy += u.x, sh += u.y, sha += u.z, sa += u.w;
        }
        const float nn = (float)HID;
        const float ry = p.yres != nullptr ? rsqrtf(sy / nn + p.eps) : 0.0f;
        const float hs = p.yres != nullptr ? p.hscale : 1.0f;
        const float sq = hs * hs * (sh + 2.0f * ry * sha + ry * ry * sa);
        const float rh = rsqrtf(fmaxf(sq, 0.0f) / nn + p.eps);
        const float v0 = fmaf(a.x, ry, h.x) * hs, v1 = fmaf(a.y, ry, h.y) * hs;
        if (g == 0 && rank == 0 && p.h_out != nullptr) *reinterpret_cast<float2*>(p.h_out + at) = make_float2(v0, v1);
        const float2 w2 = __ldg(reinterpret_cast<const float2*>(p.w2 + at));
        store_planes2(sm, t, v0 * rh * w2.x, v1 * rh * w2.y);
        __syncthreads();
    }
    if (stamp && p.stamp_at == 0) stamp[2] = global_ns();
    cp_async_wait_all();  // this thread's pieces of the third rows (and whatever else it asked for)
    __syncwarp();         // a warp's row was copied by its own lanes
    {
        // The two rows in registers together, block by block and plane by plane; then the row in shared memory.  The fences keep
        // the compiler from pulling all the planes and the third row in at once, which would not fit the registers.
        float r0, r1, u0, u1;
        dot_block2(sm, lane, w[0][0], w[0][1], w[1][0], w[1][1], r0, r1);
        asm volatile("" ::: "memory");
        dot_block2(sm, lane + 32, w[0][2], w[0][3], w[1][2], w[1][3], u0, u1);
        asm volatile("" ::: "memory");
        const float mul0 = sm.mul[lane], mul1 = sm.mul[lane + 32];
        float v0 = fmaf(u0, ws[0][1] * mul1, r0 * (ws[0][0] * mul0)), v1 = fmaf(u1, ws[1][1] * mul1, r1 * (ws[1][0] * mul0));
        v0 = warp_sum(v0), v1 = warp_sum(v1);
        // every block of the cluster gets every result: lane i writes block i's copy
        if (lane < CL) st_cluster(in_cta(&sm.qkv[qkv_slot(rank, warp)], lane), v0), st_cluster(in_cta(&sm.qkv[qkv_slot(rank, warp + 32)], lane), v1);
        asm volatile("" ::: "memory");
        const uint4* row = reinterpret_cast<const uint4*>(&sm.wo[OROWS / 2][0] + (size_t)warp * HID);
        float v2 = dot_block(sm, lane, row[2 * lane], row[2 * lane + 1]) * (ws[2][0] * mul0);
        asm volatile("" ::: "memory");
        v2 = fmaf(dot_block(sm, lane + 32, row[64 + 2 * lane], row[64 + 2 * lane + 1]), ws[2][1] * mul1, v2);
        v2 = warp_sum(v2);
        if (lane < CL) st_cluster(in_cta(&sm.qkv[qkv_slot(rank, warp + 64)], lane), v2);
    }
    Trig trig;  // the rotation's cosines and sines, on their way while the cluster meets
    if (warp <= GQ) trig = rope_trig(nullptr, pos, lane, p.trig);
    cluster_sync();
    if (stamp && p.stamp_at == 1) stamp[2] = global_ns();

    // ---- phase B: head norms and rotation; the cache row; attention over this block's run of positions --------------
    if (warp < GQ + 2) {
        const float* src = warp < GQ ? sm.qkv + warp * HD : sm.qkv + GQ * HD + (warp - GQ) * HD;
        float x[8];
        const float4 a = *reinterpret_cast<const float4*>(src + 4 * lane), b = *reinterpret_cast<const float4*>(src + 128 + 4 * lane);
        x[0] = a.x, x[1] = a.y, x[2] = a.z, x[3] = a.w, x[4] = b.x, x[5] = b.y, x[6] = b.z, x[7] = b.w;
        if (warp < GQ) {
            norm_rope(x, true, p.q_norm, &trig, p.head_eps, lane);
            const float qscale = p.scale * 1.4426950408889634f;  // scores in base 2
#pragma unroll
            for (int i = 0; i < 8; i++) x[i] *= qscale;
            store_head(sm.q[warp], x, lane);
        } else if (warp == GQ) {
            norm_rope(x, true, p.k_norm, &trig, p.head_eps, lane);
            store_head(sm.kf, x, lane);
            if (rank == 0) store_head_f16(p.kc + ((size_t)g * p.cap + cur) * HD, x, lane);
        } else {
            norm_rope(x, true, nullptr, nullptr, p.head_eps, lane);
            store_head(sm.vf, x, lane);
            if (rank == 0) store_head_f16(p.vc + ((size_t)g * p.cap + cur) * HD, x, lane);
        }
    }
    if (t < GQ) sm.mrun[t] = -INFINITY, sm.lrun[t] = 0.0f;
    __syncthreads();

    float acc = 0.0f;  // thread t: head t / 256, dimension t % 256
    int buf = 0;
    for (uint32_t a0 = a_begin; a0 < a_end; a0 += PASS) {  // the same trip count for every thread of the block
        const uint32_t cnt = min((uint32_t)PASS, a_end - a0);
        if ((uint32_t)warp < cnt) {
            float k8[8];
            if (a0 + (uint32_t)warp == 0) {
                const float4 ka = *reinterpret_cast<const float4*>(&sm.kf[8 * lane]), kc2 = *reinterpret_cast<const float4*>(&sm.kf[8 * lane + 4]);
                k8[0] = ka.x, k8[1] = ka.y, k8[2] = ka.z, k8[3] = ka.w, k8[4] = kc2.x, k8[5] = kc2.y, k8[6] = kc2.z, k8[7] = kc2.w;
            } else {
                const uint32_t kw[4] = {kreg.x, kreg.y, kreg.z, kreg.w};
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&kw[i]));
                    k8[2 * i] = f.x, k8[2 * i + 1] = f.y;
                }
            }
#pragma unroll
            for (int hq = 0; hq < GQ; hq++) {
                const float4 qa = *reinterpret_cast<const float4*>(&sm.q[hq][8 * lane]), qb = *reinterpret_cast<const float4*>(&sm.q[hq][8 * lane + 4]);
                float sc = k8[0] * qa.x + k8[1] * qa.y + k8[2] * qa.z + k8[3] * qa.w + k8[4] * qb.x + k8[5] * qb.y + k8[6] * qb.z + k8[7] * qb.w;
                sc = warp_sum(sc);
                if (lane == 0) sm.s[warp][hq] = sc;
            }
        }
        // the next pass's rows are asked for now; this pass's value rows must have arrived
        const bool more = a0 + PASS < a_end;
        uint4 knext = make_uint4(0u, 0u, 0u, 0u);
        if (more) {
            fetch_pass(a0 + PASS, buf ^ 1, knext);
            asm volatile("cp.async.wait_group 1;" ::: "memory");
        } else {
            cp_async_wait_all();
        }
        __syncthreads();
        if (warp < GQ) {  // the softmax statistics of head `warp`: a lane a position
            const float v = (uint32_t)lane < cnt ? sm.s[lane][warp] : -INFINITY;
            const float m = warp_max(v);
            const float mold = sm.mrun[warp], mnew = fmaxf(mold, m);
            const float e = (uint32_t)lane < cnt ? exp2f(v - mnew) : 0.0f;
            const float l = warp_sum(e);
            sm.s[lane][warp] = e;
            if (lane == 0) {
                const float c = exp2f(mold - mnew);  // 0 on the first pass (mold = -inf)
                sm.corr[warp] = c, sm.mrun[warp] = mnew, sm.lrun[warp] = sm.lrun[warp] * c + l;
            }
        }
        __syncthreads();
        {
            const int hq = t >> 8, d = t & 255;
            acc *= sm.corr[hq];
            for (uint32_t j = 0; j < cnt; j++) {
                const float vv = a0 + j == 0 ? sm.vf[d] : __half2float(sm.v[buf][j][d]);
                acc = fmaf(sm.s[j][hq], vv, acc);
            }
        }
        __syncthreads();  // sm.s and sm.v[buf] are free for the pass after next
        kreg = knext, buf ^= 1;
    }

    if (stamp && p.stamp_at == 2) stamp[2] = global_ns();
    // The other 64 rows of the output projection's slice, over phase A's third rows (every warp has long read its own).
#pragma unroll
    for (int i = 0; i < (OROWS / 2) * (OCOLS / 16) / NT; i++) {
        const int id = t + NT * i, r = OROWS / 2 + id / (OCOLS / 16), c = id % (OCOLS / 16);
        cp_async_16(&sm.wo[r][c * 16], p.wo + (size_t)(rank * OROWS + r) * HID + g * OCOLS + c * 16);
    }
    cp_async_commit();

    // ---- merge: block o gets every block's statistics and its 64 of the 1024 outputs ----------------------------------
    st_cluster(in_cta(&sm.in_acc[rank][t & 63], (uint32_t)t >> 6), acc);
    if (t < CL * 2 * GQ) st_cluster(in_cta(&sm.in_ml[rank][t & 7], (uint32_t)t >> 3), (t & 7) < GQ ? sm.mrun[t & 7] : sm.lrun[(t & 7) - GQ]);
    cluster_sync();
    if (t < OCOLS / CL) {
        const uint32_t hq = rank / (CL / GQ);  // the head this block's 64 outputs belong to
        float M = -INFINITY;
#pragma unroll
        for (int r = 0; r < CL; r++) M = fmaxf(M, sm.in_ml[r][hq]);
        float Lsum = 0.0f, A = 0.0f;
#pragma unroll
        for (int r = 0; r < CL; r++) {
            const float wgt = exp2f(sm.in_ml[r][hq] - M);  // 0 for a block without positions (its maximum is -inf)
            Lsum = fmaf(wgt, sm.in_ml[r][GQ + hq], Lsum);
            A = fmaf(wgt, sm.in_acc[r][t], A);
        }
        const float out = A / Lsum;
#pragma unroll
        for (int r = 0; r < CL; r++) st_cluster(in_cta(&sm.att[rank * (OCOLS / CL) + t], (uint32_t)r), out);
    }
    cluster_sync();  // the last access to another block's shared memory is behind this
    if (stamp && p.stamp_at == 3) stamp[2] = global_ns();

    // ---- phase C: the group's columns of the output projection, 128 rows a block ----------------------------------------
    if (t < OCOLS / 4) {
        const float4 v = *reinterpret_cast<const float4*>(&sm.att[4 * t]);
        store_planes4(sm, t, v.x, v.y, v.z, v.w);
    }
    cp_async_wait_all();
    __syncthreads();
    float* y = (g == 0 ? p.y[0] : p.y[1]) + rank * OROWS;
#pragma unroll
    for (int j = 0; j < 4; j++) {
        const int r = warp + 32 * j;
        const uint4 a = *reinterpret_cast<const uint4*>(&sm.wo[r][32 * lane]), c = *reinterpret_cast<const uint4*>(&sm.wo[r][32 * lane + 16]);
        float v = dot_block(sm, lane, a, c) * (__half2float(sm.so[r][lane]) * sm.mul[lane]);
        v = warp_sum(v);
        if (lane == 0) y[r] = v;
    }
    if (stamp) stamp[3] = global_ns();
}

}  // namespace

bool attn_block_available(tb_context* ctx) {
    static int known[16] = {};  // 0 unknown, 1 yes, 2 no
    int& k = known[ctx->gpu & 15];
    if (k == 0) {
        k = 2;
        cudaSetDevice(ctx->gpu);
        if (cudaFuncSetAttribute(attn_block_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sizeof(Smem) + 128) == cudaSuccess &&
            cudaFuncSetAttribute(attn_block_kernel, cudaFuncAttributeNonPortableClusterSizeAllowed, 1) == cudaSuccess) {
            cudaLaunchConfig_t cfg = {};
            cfg.gridDim = dim3(CL, KVH), cfg.blockDim = dim3(NT), cfg.dynamicSmemBytes = sizeof(Smem) + 128;
            cudaLaunchAttribute attr[1];
            attr[0].id = cudaLaunchAttributeClusterDimension;
            attr[0].val.clusterDim.x = CL, attr[0].val.clusterDim.y = 1, attr[0].val.clusterDim.z = 1;
            cfg.attrs = attr, cfg.numAttrs = 1;
            int clusters = 0;
            if (cudaOccupancyMaxActiveClusters(&clusters, attn_block_kernel, &cfg) == cudaSuccess && clusters >= KVH) k = 1;
        }
        cudaGetLastError();
    }
    return k == 1;
}

int launch_attn_block(tb_context* ctx, const AttnBlockParams& p) {
    if (!p.h || !p.w2 || !p.wqkv || !p.sqkv || !p.q_norm || !p.k_norm || !p.trig || !p.pos || !p.kc || !p.vc || !p.wo || !p.so || !p.y[0] || !p.y[1])
        return fail(OUT_OF_RANGE, "attention block: null argument");
    if (p.yres != nullptr && p.w1 == nullptr) return fail(OUT_OF_RANGE, "attention block: a residual needs its norm weights");
    if (p.cap == 0 || p.window == 0 || p.window > p.cap) return fail(OUT_OF_RANGE, "attention block: window and cache size");
    if (!attn_block_available(ctx)) return fail(UNSUPPORTED, "attention block: this GPU does not run two clusters of 16 blocks");
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(CL, KVH), cfg.blockDim = dim3(NT), cfg.dynamicSmemBytes = sizeof(Smem) + 128, cfg.stream = ctx->stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = CL, attr[0].val.clusterDim.y = 1, attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = ctx->pdl ? 1 : 0;
    cfg.attrs = attr, cfg.numAttrs = 2;
    TB_CUDA(cudaLaunchKernelEx(&cfg, attn_block_kernel, p));
    return OK;
}

}  // namespace tb
