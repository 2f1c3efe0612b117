// Prefill GEMM on the fifth-generation tensor cores: D[M, N] = A[M, K] (f16 activations) x W[N, K]^T with W in the
// decode path's Q8 layout (int8 codes + one f16 scale per 32 along K), f32 accumulation in tensor memory.
// Stands in for the reference's gemm_q4 (crates/tachyon/src/ptx/gemm.rs:225-259: integer mma.sync on Q4 x Q8P) and its
// split-K sum (gemm.rs:287-325), which the TMEM accumulator makes unnecessary: a block owns one output tile
// over the whole K (128 or 256 tokens x 256 outputs).
//
// One block, ten warps:
//   warp 0      one thread issues the TMA loads of the activation tile (128 rows x 64 halves, 128-byte swizzle);
//   warp 1      allocates tensor memory; one thread issues tcgen05.mma (M128 N256 K16: the widest shape, so that the
//               operand reads from shared memory stay below the tensor core's rate) and commits;
//   warps 2-9   dequantise the weight tile: thread j reads row j's 64 codes and two scales, turns the codes into f16
//               exactly (0x6400 | (code ^ 0x80) is 1024 + code + 128; minus 1152), multiplies by the scale and stores
//               the row in the same swizzled K-major layout TMA would have produced; after the main loop the same
//               warps read the accumulator back (tcgen05.ld) and write the output (f32, f16, or GeGLU of column pairs).
// Stages hand over on mbarriers: full = TMA bytes + the dequantising warps, empty = tcgen05.commit.
// With f16 weights (tb_gemm_f16, and the f16 copies of quantised matrices that prefill and the encoder keep) the weight tile
// comes by TMA like the activations' and those warps only run the epilogue.
// Operands are f16 rather than bf16: the code -> f16 step is exact and costs one instruction per two weights, the
// tensor rate is the same, and the activations that reach this kernel are normalised.
#include <cuda.h>

#include <algorithm>

#include "common.cuh"
#include "internal.h"

namespace tb {

namespace {

constexpr int BM = 128, BN = 256, BK = 64;  // MMA shape M128 N256; BK halves = one 128-byte swizzle row
constexpr int stages(int mt) { return mt == 2 ? 3 : 4; }
constexpr int DW = 16;                  // dequantising / epilogue warps: with two per scheduler the loads' latency showed
constexpr int DT = DW * 32, PIECES = 1024 / DT;  // a weight tile is 1024 pieces of 16 codes
constexpr int THREADS = 64 + DT;        // TMA warp, MMA warp, the dequantising / epilogue warps
constexpr int WALK_EW = DW;             // epilogue warps of the kernel that walks tiles of f16 weights (28, seven a quarter at 64 registers, measured slower: 203 against 198 us)
constexpr int A_BYTES = BM * BK * 2, B_BYTES = BN * BK * 2;  // per 128-row sub-tile of activations, per weight tile
constexpr int smem_bytes(int mt) { return 1024 + stages(mt) * (mt * A_BYTES + B_BYTES) + 256; }

// tcgen05.mma instruction descriptor, kind::f16: f32 accumulator, f16 A and B, both K-major, N = 128, M = 128.
constexpr uint32_t IDESC = (1u << 4) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);

// Shared-memory matrix descriptor: K-major tile of 128-byte rows, 128-byte swizzle, 1024 bytes between 8-row groups.
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr) {
    const uint32_t lo = ((addr & 0x3ffffu) >> 4) | (1u << 16);
    const uint32_t hi = (1024u >> 4) | (1u << 14) | (2u << 29);
    return ((uint64_t)hi << 32) | lo;
}

__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, int x, int y, uint64_t* bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(smem_addr(dst)),
                 "l"(map), "r"(x), "r"(y), "r"(smem_addr(bar))
                 : "memory");
}

__device__ __forceinline__ void mma_f16(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(IDESC), "r"(accumulate)
        : "memory");
}

__device__ __forceinline__ void mma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_addr(bar)) : "memory");
}

// 32 consecutive accumulator columns of this thread's row.
__device__ __forceinline__ void tmem_load32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, %17, %18, %19, %20, %21, "
        "%22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]),
          "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]),
          "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr));
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// Four codes (one word) -> four f16 of code * scale, as two half2.
__device__ __forceinline__ void dequant4(uint32_t w, __half2 scale, uint32_t& lo, uint32_t& hi) {
    const uint32_t x = w ^ 0x80808080u;                 // code + 128 in every byte
    uint32_t a = __byte_perm(x, 0x64646464u, 0x5140);  // {0x64, b1, 0x64, b0}: 1024 + b1, 1024 + b0
    uint32_t b = __byte_perm(x, 0x64646464u, 0x7362);  // bytes 2 and 3
    const __half2 bias = __floats2half2_rn(1152.0f, 1152.0f);
    const __half2 va = __hmul2(__hsub2(*reinterpret_cast<__half2*>(&a), bias), scale);
    const __half2 vb = __hmul2(__hsub2(*reinterpret_cast<__half2*>(&b), bias), scale);
    lo = *reinterpret_cast<const uint32_t*>(&va);
    hi = *reinterpret_cast<const uint32_t*>(&vb);
}

// Eight four-bit weights (one word of the reference's Q4: bytes' low nibbles are weights 0..3, high nibbles 4..7,
// crates/tachyon/src/quant.rs:60-66) -> eight f16 of (n - 8) * scale, in order, as four half2.
__device__ __forceinline__ void dequant8_q4(uint32_t w, __half2 scale, uint32_t (&out)[4]) {
    const uint32_t lo = w & 0x0F0F0F0Fu, hi = (w >> 4) & 0x0F0F0F0Fu;
    const __half2 bias = __floats2half2_rn(1032.0f, 1032.0f);  // 0x6400 | n is 1024 + n
    uint32_t p[4] = {__byte_perm(lo, 0x64646464u, 0x4140), __byte_perm(lo, 0x64646464u, 0x4342), __byte_perm(hi, 0x64646464u, 0x4140),
                     __byte_perm(hi, 0x64646464u, 0x4342)};
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const __half2 v = __hmul2(__hsub2(*reinterpret_cast<__half2*>(&p[i]), bias), scale);
        out[i] = *reinterpret_cast<const uint32_t*>(&v);
    }
}

struct GemmArgs {
    const int8_t* w;
    const __half* s;
    void* out;
    uint32_t M, N, K;
    int mode;  // 0: f32 [M, N]; 1: f16 [M, N]; 2: GeGLU (tanh) of column pairs, f16 [M, N / 2]; 3: f32 [M, N] += D;
               // 4: GeGLU (erf) of column pairs, f16 [M, N / 2]; 5: GELU (erf), f16 [M, N]; 7: ReLU, f16 [M, N];
               // 8: SiLU(even) * odd of column pairs, f16 [M, N / 2] (the reference's store modes 3 and 5, ptx/encoder.rs:5-9)
    const float* bias;  // f32 [N] added to every token's sums before the mode's store, or null (ptx/encoder.rs:418-436)
};

__device__ __forceinline__ float silu(float v) { return v / (1.0f + exp2f(-1.4426950408889634f * v)); }

// The epilogue of one tile: the accumulator's rows are tokens, its columns weight rows; warp `warp` (2 .. 2 + DW) reads the lanes of
// its quarter, 32 columns at a time, adds the bias, applies the mode and stores.  (m0, n0): the tile's first token and weight row.
template <int MT, int EW = DW>
__device__ __forceinline__ void epilogue_tile(const GemmArgs& g, uint32_t tmem, int warp, int lane, uint32_t m0, uint32_t n0, bool ok) {
    // EW / 4 warps share each quarter of the accumulator's lanes and take the column blocks in turn.
    const uint32_t q = warp & 3, rrow = 32 * q + lane;
#pragma unroll 1
    for (int cbi = (warp - 2) >> 2; cbi < MT * (BN / 32); cbi += EW / 4) {
        const int mt = cbi / (BN / 32), cb = cbi % (BN / 32);
        const uint32_t m = m0 + mt * BM + rrow;
        uint32_t r[32];
        tmem_load32(tmem + ((32 * q) << 16) + mt * BN + cb * 32, r);
        if (m < g.M && ok) {
            const uint32_t col = n0 + cb * 32;
            if (g.bias != nullptr && col < g.N) {
#pragma unroll
                for (int i = 0; i < 8; i++) {
                    const float4 b = __ldg(reinterpret_cast<const float4*>(g.bias + col) + i);
                    r[4 * i] = __float_as_uint(__uint_as_float(r[4 * i]) + b.x), r[4 * i + 1] = __float_as_uint(__uint_as_float(r[4 * i + 1]) + b.y);
                    r[4 * i + 2] = __float_as_uint(__uint_as_float(r[4 * i + 2]) + b.z), r[4 * i + 3] = __float_as_uint(__uint_as_float(r[4 * i + 3]) + b.w);
                }
            }
            if (g.mode == 3) {
                float4* dst = reinterpret_cast<float4*>(static_cast<float*>(g.out) + (size_t)m * g.N + col);
#pragma unroll
                for (int i = 0; i < 8; i++)
                    if (col + 4 * i < g.N) {
                        float4 t = dst[i];
                        t.x += __uint_as_float(r[4 * i]), t.y += __uint_as_float(r[4 * i + 1]), t.z += __uint_as_float(r[4 * i + 2]), t.w += __uint_as_float(r[4 * i + 3]);
                        dst[i] = t;
                    }
            } else if (g.mode == 0) {
                float4* dst = reinterpret_cast<float4*>(static_cast<float*>(g.out) + (size_t)m * g.N + col);
#pragma unroll
                for (int i = 0; i < 8; i++)
                    if (col + 4 * i < g.N) dst[i] = make_float4(__uint_as_float(r[4 * i]), __uint_as_float(r[4 * i + 1]), __uint_as_float(r[4 * i + 2]), __uint_as_float(r[4 * i + 3]));
            } else if (g.mode == 1 || g.mode == 5 || g.mode == 7) {
                uint4* dst = reinterpret_cast<uint4*>(static_cast<__half*>(g.out) + (size_t)m * g.N + col);
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    uint32_t h[4];
#pragma unroll
                    for (int e = 0; e < 4; e++) {
                        float f0 = __uint_as_float(r[8 * i + 2 * e]), f1 = __uint_as_float(r[8 * i + 2 * e + 1]);
                        if (g.mode == 5) f0 = gelu_erf_lean(f0), f1 = gelu_erf_lean(f1);
                        if (g.mode == 7) f0 = fmaxf(f0, 0.0f), f1 = fmaxf(f1, 0.0f);
                        const __half2 t = __floats2half2_rn(f0, f1);
                        h[e] = *reinterpret_cast<const uint32_t*>(&t);
                    }
                    if (col + 8 * i < g.N) dst[i] = make_uint4(h[0], h[1], h[2], h[3]);
                }
            } else {
                // columns (2j, 2j+1) are (gate_j, up_j): gelu_tanh(gate) * up, 16 results per 32 columns
                uint4* dst = reinterpret_cast<uint4*>(static_cast<__half*>(g.out) + (size_t)m * (g.N / 2) + col / 2);
#pragma unroll
                for (int i = 0; i < 2; i++) {
                    uint32_t h[4];
#pragma unroll
                    for (int e = 0; e < 4; e++) {
                        const float g0 = __uint_as_float(r[16 * i + 4 * e]), g1 = __uint_as_float(r[16 * i + 4 * e + 2]);
                        const float a0 = (g.mode == 2 ? gelu_tanh(g0) : g.mode == 8 ? silu(g0) : gelu_erf_lean(g0)) * __uint_as_float(r[16 * i + 4 * e + 1]);
                        const float a1 = (g.mode == 2 ? gelu_tanh(g1) : g.mode == 8 ? silu(g1) : gelu_erf_lean(g1)) * __uint_as_float(r[16 * i + 4 * e + 3]);
                        const __half2 t = __floats2half2_rn(a0, a1);
                        h[e] = *reinterpret_cast<const uint32_t*>(&t);
                    }
                    if (col + 16 * i < g.N) dst[i] = make_uint4(h[0], h[1], h[2], h[3]);
                }
            }
        }
    }
}

// MT: 128-row sub-tiles of activations a block multiplies with each dequantised weight tile (1 or 2): with two, the
// dequantisation is shared by twice the tensor-core work.
// WB: bits per weight, 8 (codes, an f16 scale per 32), 4 (the reference's Q4, a scale per 64 = one per row and K tile) or 16
// (f16 weights as they are, the reference's gemm_f16, ptx/encoder.rs:498-525: the weight tile then comes by TMA through
// w_map like the activations', and the sixteen warps only run the epilogue).
template <int MT, int WB = 8>
__global__ void __launch_bounds__(THREADS, 1) gemm_q8_kernel(const __grid_constant__ CUtensorMap a_map, const __grid_constant__ CUtensorMap w_map,
                                                             const GemmArgs g, uint32_t* status) {
    constexpr int AS = MT * A_BYTES, STAGES = stages(MT);
    extern __shared__ uint8_t raw_unaligned[];
    uint8_t* raw = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(raw_unaligned) + 1023) & ~uintptr_t(1023));
    uint8_t* As = raw;
    uint8_t* Bs = raw + STAGES * AS;
    uint64_t* full = reinterpret_cast<uint64_t*>(raw + STAGES * (AS + B_BYTES));
    uint64_t* empty = full + STAGES;
    uint64_t* acc_full = empty + STAGES;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_full + 1);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // Consecutive blocks share a weight tile (their reads of it meet in the L2) and differ in the token tile.
    const uint32_t m0 = blockIdx.x * (MT * BM), n0 = blockIdx.y * BN, nk = g.K / BK;

    if (threadIdx.x == 0) {
        for (int i = 0; i < STAGES; i++) mbar_init(&full[i], WB == 16 ? 1 : DW + 1), mbar_init(&empty[i], 1);
        mbar_init(acc_full, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_addr(tmem_slot)), "r"((uint32_t)(MT * BN)) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = *tmem_slot;
    // Tensor memory, barriers and descriptors are set up: the kernel behind may be scheduled, and this one reads and writes only
    // once the kernel in front is done (both do nothing where a launch is not programmatic).
    pdl_launch_dependents();
    pdl_wait();
    bool ok = true;

    if (warp == 0) {
        if (lane == 0) {
            for (uint32_t kt = 0; kt < nk && ok; kt++) {
                const uint32_t s = kt % STAGES;
                if (kt >= STAGES && !mbar_wait(&empty[s], ((kt / STAGES) - 1) & 1)) {
                    atomicCAS(status, ERR_NONE, ERR_WAIT_EMPTY);
                    ok = false;
                    break;
                }
                mbar_expect_tx(&full[s], WB == 16 ? AS + B_BYTES : AS);
                tma_load_2d(As + s * AS, &a_map, (int)(kt * BK), (int)m0, &full[s]);
                if constexpr (WB == 16) tma_load_2d(Bs + s * B_BYTES, &w_map, (int)(kt * BK), (int)n0, &full[s]);
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            for (uint32_t kt = 0; kt < nk && ok; kt++) {
                const uint32_t s = kt % STAGES;
                if (!mbar_wait(&full[s], (kt / STAGES) & 1)) {
                    atomicCAS(status, ERR_NONE, ERR_WAIT_FULL);
                    ok = false;
                    break;
                }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t a = smem_addr(As + s * AS), b = smem_addr(Bs + s * B_BYTES);
#pragma unroll
                for (int mt = 0; mt < MT; mt++)
#pragma unroll
                    for (int k = 0; k < BK / 16; k++)
                        mma_f16(tmem + mt * BN, smem_desc(a + mt * A_BYTES + k * 32), smem_desc(b + k * 32), (kt > 0 || k > 0) ? 1u : 0u);
                mma_commit(&empty[s]);
            }
            mma_commit(acc_full);  // arrives when every MMA above has finished (also after an early exit)
        }
    } else {
        // Weight tile: 256 rows x 64 codes = 1024 pieces of 16 codes; thread j takes pieces j, j + 512 (with sixteen warps)
        // (piece p: row p / 4, quarter p % 4), so a warp's load covers eight rows' whole 64-byte segments instead of
        // thirty-two separate lines.  A row's scales for four tiles come in one 16-byte load every fourth tile.  The
        // next tile's codes are fetched before this one's are stored.
        const int j = threadIdx.x - 64, qtr = j & 3;
        uint4 c[PIECES];
        uint4 sc8[PIECES];  // per piece: the row's eight scales covering tiles kt & ~3 ... + 3
        auto fetch = [&](uint32_t kt) {
#pragma unroll
            for (int it = 0; it < PIECES; it++) {
                const uint32_t row = it * (DT / 4) + (j >> 2), n = n0 + row;
                const bool live = n < g.N;
                if constexpr (WB == 4) {
                    // A piece is 16 weights = 8 bytes; a row's tile 32 bytes; its one scale per tile comes eight tiles at a time.
                    const uint2 t = live ? __ldg(reinterpret_cast<const uint2*>(g.w + (size_t)n * (g.K / 2) + (size_t)kt * (BK / 2) + qtr * 8))
                                         : make_uint2(0x88888888u, 0x88888888u);
                    c[it] = make_uint4(t.x, t.y, 0u, 0u);
                    if ((kt & 7) == 0) {
                        const __half* sp = g.s + (size_t)n * (g.K / 64) + kt;
                        if (live && kt + 8 <= g.K / 64 && (g.K / 64) % 8 == 0) {
                            sc8[it] = __ldg(reinterpret_cast<const uint4*>(sp));
                        } else {
                            __half t8[8];
#pragma unroll
                            for (int e = 0; e < 8; e++) t8[e] = (live && kt + e < g.K / 64) ? sp[e] : __float2half(0.0f);
                            sc8[it] = *reinterpret_cast<const uint4*>(t8);
                        }
                    }
                    continue;
                }
                c[it] = live ? __ldg(reinterpret_cast<const uint4*>(g.w + (size_t)n * g.K + (size_t)kt * BK + qtr * 16))
                             : make_uint4(0x80808080u, 0x80808080u, 0x80808080u, 0x80808080u);
                if ((kt & 3) == 0) {
                    // K is a multiple of 64: the last group of four tiles may be short, a 16-byte load still stays
                    // inside the row when K is a multiple of 256; otherwise fall back to single scales.
                    const __half* sp = g.s + (size_t)n * (g.K / 32) + kt * 2;
                    if (live && kt * 2 + 8 <= g.K / 32 && (g.K / 32) % 8 == 0) {
                        sc8[it] = __ldg(reinterpret_cast<const uint4*>(sp));
                    } else {
                        __half t[8];
#pragma unroll
                        for (int e = 0; e < 8; e++) t[e] = (live && kt * 2 + e < g.K / 32) ? sp[e] : __float2half(0.0f);
                        sc8[it] = *reinterpret_cast<const uint4*>(t);
                    }
                }
            }
        };
        if (WB != 16 && nk > 0) fetch(0);
        for (uint32_t kt = 0; WB != 16 && kt < nk; kt++) {
            const uint32_t s = kt % STAGES;
            uint32_t v[PIECES][8];  // per piece 16 halves
#pragma unroll
            for (int it = 0; it < PIECES; it++) {
                // scale of this piece's group of 32: tile kt's two scales are halves 2*(kt&3) and 2*(kt&3)+1
                const uint32_t words[4] = {sc8[it].x, sc8[it].y, sc8[it].z, sc8[it].w};
                if constexpr (WB == 4) {
                    const uint32_t pair = words[(kt & 7) >> 1];
                    const __half2 s2 = __half2half2(__ushort_as_half((unsigned short)((kt & 1) ? (pair >> 16) : (pair & 0xffffu))));
                    uint32_t a[4], b[4];
                    dequant8_q4(c[it].x, s2, a), dequant8_q4(c[it].y, s2, b);
#pragma unroll
                    for (int e = 0; e < 4; e++) v[it][e] = a[e], v[it][4 + e] = b[e];
                    continue;
                }
                const uint32_t pair = words[kt & 3];
                const __half sh = __ushort_as_half((unsigned short)((qtr & 2) ? (pair >> 16) : (pair & 0xffffu)));
                const __half2 s2 = __half2half2(sh);
                dequant4(c[it].x, s2, v[it][0], v[it][1]);
                dequant4(c[it].y, s2, v[it][2], v[it][3]);
                dequant4(c[it].z, s2, v[it][4], v[it][5]);
                dequant4(c[it].w, s2, v[it][6], v[it][7]);
            }
            if (kt + 1 < nk) fetch(kt + 1);
            if (ok && kt >= STAGES && !mbar_wait(&empty[s], ((kt / STAGES) - 1) & 1)) {
                atomicCAS(status, ERR_NONE, ERR_WAIT_EMPTY);
                ok = false;
            }
#pragma unroll
            for (int it = 0; it < PIECES; it++) {
                const uint32_t row = it * (DT / 4) + (j >> 2);
                uint8_t* base = Bs + s * B_BYTES + row * 128;
                *reinterpret_cast<uint4*>(base + (((2 * qtr) ^ (row & 7)) << 4)) = make_uint4(v[it][0], v[it][1], v[it][2], v[it][3]);
                *reinterpret_cast<uint4*>(base + (((2 * qtr + 1) ^ (row & 7)) << 4)) = make_uint4(v[it][4], v[it][5], v[it][6], v[it][7]);
            }
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // the tensor core reads through the async proxy
            __syncwarp();
            if (lane == 0) mbar_arrive(&full[s]);
        }
        // Epilogue: this warp's quarter of the accumulator rows.
        if (!mbar_wait(acc_full, 0)) {
            atomicCAS(status, ERR_NONE, ERR_WAIT_FULL);
            ok = false;
        }
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        epilogue_tile<MT>(g, tmem, warp, lane, m0, n0, ok);
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 1) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"((uint32_t)(MT * BN)) : "memory");
}

// The same product for f16 weights as a persistent kernel: a block walks the output tiles t = blockIdx.x, + gridDim.x, ...
// (token tile t % tiles_m, weight tile t / tiles_m, so that blocks running together share weight tiles in the L2).  The
// accumulator fills all of tensor memory (MT x 256 columns), so a tile's epilogue cannot overlap the next tile's products; what
// the loop buys is that the copies of the next tile's first stages are under way during the epilogue (the ring is free
// then), and that tensor memory, barriers and descriptors are set up once a block instead of once a tile.
template <int MT, int EW>
__global__ void __launch_bounds__(64 + 32 * EW, 1) gemm_f16_persistent_tile_kernel(const __grid_constant__ CUtensorMap a_map, const __grid_constant__ CUtensorMap w_map,
                                                                              const GemmArgs g, uint32_t* status) {
    constexpr int AS = MT * A_BYTES, STAGES = stages(MT);
    extern __shared__ uint8_t raw_unaligned[];
    uint8_t* raw = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(raw_unaligned) + 1023) & ~uintptr_t(1023));
    uint8_t* As = raw;
    uint8_t* Bs = raw + STAGES * AS;
    uint64_t* full = reinterpret_cast<uint64_t*>(raw + STAGES * (AS + B_BYTES));
    uint64_t* empty = full + STAGES;
    uint64_t* acc_full = empty + STAGES;
    uint64_t* acc_empty = acc_full + 1;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 1);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t nk = g.K / BK, tiles_m = (g.M + MT * BM - 1) / (MT * BM), tiles = tiles_m * ((g.N + BN - 1) / BN);

    if (threadIdx.x == 0) {
        for (int i = 0; i < STAGES; i++) mbar_init(&full[i], 1), mbar_init(&empty[i], 1);
        mbar_init(acc_full, 1), mbar_init(acc_empty, EW);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_addr(tmem_slot)), "r"((uint32_t)(MT * BN)) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = *tmem_slot;
    // Tensor memory, barriers and descriptors are set up: the kernel behind may be scheduled, and this one reads and writes only
    // once the kernel in front is done (both do nothing where a launch is not programmatic).
    pdl_launch_dependents();
    pdl_wait();

    if (warp == 0) {
        if (lane == 0) {
            uint32_t it = 0;
            for (uint32_t t = blockIdx.x; t < tiles; t += gridDim.x) {
                const uint32_t m0 = (t % tiles_m) * (MT * BM), n0 = (t / tiles_m) * BN;
                for (uint32_t kt = 0; kt < nk; kt++, it++) {
                    const uint32_t s = it % STAGES;
                    if (it >= STAGES && !mbar_wait(&empty[s], ((it / STAGES) - 1) & 1)) {
                        atomicCAS(status, ERR_NONE, ERR_WAIT_EMPTY);
                        t = tiles;
                        break;
                    }
                    mbar_expect_tx(&full[s], AS + B_BYTES);
                    tma_load_2d(As + s * AS, &a_map, (int)(kt * BK), (int)m0, &full[s]);
                    tma_load_2d(Bs + s * B_BYTES, &w_map, (int)(kt * BK), (int)n0, &full[s]);
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            uint32_t it = 0, ti = 0;
            bool ok = true;
            for (uint32_t t = blockIdx.x; t < tiles && ok; t += gridDim.x, ti++) {
                // the epilogue of the tile before has read the accumulator
                if (ti > 0 && !mbar_wait(acc_empty, (ti - 1) & 1)) {
                    atomicCAS(status, ERR_NONE, ERR_WAIT_EMPTY);
                    break;
                }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                for (uint32_t kt = 0; kt < nk; kt++, it++) {
                    const uint32_t s = it % STAGES;
                    if (!mbar_wait(&full[s], (it / STAGES) & 1)) {
                        atomicCAS(status, ERR_NONE, ERR_WAIT_FULL);
                        ok = false;
                        break;
                    }
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const uint32_t a = smem_addr(As + s * AS), b = smem_addr(Bs + s * B_BYTES);
#pragma unroll
                    for (int mt = 0; mt < MT; mt++)
#pragma unroll
                        for (int k = 0; k < BK / 16; k++)
                            mma_f16(tmem + mt * BN, smem_desc(a + mt * A_BYTES + k * 32), smem_desc(b + k * 32), (kt > 0 || k > 0) ? 1u : 0u);
                    mma_commit(&empty[s]);
                }
                mma_commit(acc_full);  // arrives when the tile's products have finished (also after an early exit)
            }
        }
    } else {
        uint32_t ti = 0;
        for (uint32_t t = blockIdx.x; t < tiles; t += gridDim.x, ti++) {
            const uint32_t m0 = (t % tiles_m) * (MT * BM), n0 = (t / tiles_m) * BN;
            bool ok = true;
            if (!mbar_wait(acc_full, ti & 1)) {
                atomicCAS(status, ERR_NONE, ERR_WAIT_FULL);
                ok = false;
            }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            epilogue_tile<MT, EW>(g, tmem, warp, lane, m0, n0, ok);
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(acc_empty);
            if (!ok) break;
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 1) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"((uint32_t)(MT * BN)) : "memory");
}

// Codes to f16 weights once, with the arithmetic of the product's own conversion (dequant4, dequant8_q4), so that a product on
// the copy has the operands the converting kernel would have made: a thread a piece of sixteen weights.  The scales lie
// [rows][cols / group] behind one another, so a piece's scale is at piece / (group / 16).
template <int WB>
__global__ void __launch_bounds__(256) dequant_f16_kernel(const uint8_t* __restrict__ w, const __half* __restrict__ s, size_t pieces, __half* __restrict__ out) {
    const size_t stride = (size_t)gridDim.x * 256;
    for (size_t p = (size_t)blockIdx.x * 256 + threadIdx.x; p < pieces; p += stride) {
        uint32_t v[8];
        if constexpr (WB == 8) {
            const uint4 c = __ldcs(reinterpret_cast<const uint4*>(w) + p);
            const __half2 s2 = __half2half2(__ldg(s + p / 2));
            dequant4(c.x, s2, v[0], v[1]), dequant4(c.y, s2, v[2], v[3]), dequant4(c.z, s2, v[4], v[5]), dequant4(c.w, s2, v[6], v[7]);
        } else {
            const uint2 c = __ldcs(reinterpret_cast<const uint2*>(w) + p);
            const __half2 s2 = __half2half2(__ldg(s + p / 4));
            uint32_t a[4], b[4];
            dequant8_q4(c.x, s2, a), dequant8_q4(c.y, s2, b);
#pragma unroll
            for (int e = 0; e < 4; e++) v[e] = a[e], v[4 + e] = b[e];
        }
        uint4* dst = reinterpret_cast<uint4*>(out) + 2 * p;
        dst[0] = make_uint4(v[0], v[1], v[2], v[3]), dst[1] = make_uint4(v[4], v[5], v[6], v[7]);
    }
}

typedef CUresult (*EncodeTiled)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiled encode_tiled() {
    static EncodeTiled fn = [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess) p = nullptr;
        return reinterpret_cast<EncodeTiled>(p);
    }();
    return fn;
}

}  // namespace

int launch_dequant_f16(tb_context* ctx, const int8_t* w, const __half* s, uint32_t rows, uint32_t cols, uint32_t wbits, __half* out) {
    if (!w || !s || !out || rows == 0 || cols == 0) return fail(OUT_OF_RANGE, "dequantise: null or empty argument");
    if (wbits != 8 && wbits != 4) return fail(OUT_OF_RANGE, "dequantise: weights are 8 or 4 bits");
    if (cols % (wbits == 4 ? 64 : 32) != 0) return fail(OUT_OF_RANGE, "dequantise: ragged scale groups");
    if ((reinterpret_cast<uintptr_t>(w) | reinterpret_cast<uintptr_t>(out)) & 15) return fail(OUT_OF_RANGE, "dequantise: buffers must be 16-byte aligned");
    const size_t pieces = (size_t)rows * cols / 16;
    const unsigned blocks = (unsigned)std::min<size_t>((pieces + 1023) / 1024, (size_t)ctx->sms * 16);
    if (wbits == 8) dequant_f16_kernel<8><<<blocks, 256, 0, ctx->stream>>>(reinterpret_cast<const uint8_t*>(w), s, pieces, out);
    else dequant_f16_kernel<4><<<blocks, 256, 0, ctx->stream>>>(reinterpret_cast<const uint8_t*>(w), s, pieces, out);
    TB_CUDA(cudaGetLastError());
    return OK;
}

int launch_gemm_q8(tb_context* ctx, const int8_t* w, const __half* s, const __half* a, uint32_t M, uint32_t N, uint32_t K, void* out, int mode,
                   uint32_t wbits, const float* mul, uint32_t mul_stride, const float* bias) {
    if (!w || (!s && wbits != 16) || !a || !out || M == 0 || N == 0 || K == 0) return fail(OUT_OF_RANGE, "gemm: null or empty argument");
    if (K % BK != 0) return fail(OUT_OF_RANGE, "gemm: K must be a multiple of 64");
    if (N % 32 != 0 || ((mode == 2 || mode == 4 || mode == 8) && N % 64 != 0)) return fail(OUT_OF_RANGE, "gemm: N must be a multiple of 32 (64 with a gated output)");
    if (mode < 0 || mode > 8) return fail(OUT_OF_RANGE, "gemm: unknown output mode");
    if (mode == 6) {  // only the persistent schedule has this epilogue
        if (bias != nullptr) return fail(UNSUPPORTED, "gemm: a bias has no place beside a multiplier");
        if (!mul || mul_stride < N || (reinterpret_cast<uintptr_t>(mul) & 15) || mul_stride % 4 != 0) return fail(OUT_OF_RANGE, "gemm: the multiplier must be present, 16-byte aligned and at least N wide");
        if (!gemm_persistent_supports(N, K, wbits)) return fail(UNSUPPORTED, "gemm: no kernel for this shape with a multiplier");
        if (wbits != 8 && wbits != 4) return fail(OUT_OF_RANGE, "gemm: weights are 8 or 4 bits");
        if ((reinterpret_cast<uintptr_t>(w) | reinterpret_cast<uintptr_t>(s) | reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(out)) & 15)
            return fail(OUT_OF_RANGE, "gemm: buffers must be 16-byte aligned");
        return launch_gemm_persistent(ctx, w, s, a, M, N, K, out, mode, wbits, mul, mul_stride);
    }
    if (wbits != 8 && wbits != 4 && wbits != 16) return fail(OUT_OF_RANGE, "gemm: weights are 16, 8 or 4 bits");
    if ((reinterpret_cast<uintptr_t>(w) | reinterpret_cast<uintptr_t>(s) | reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(out)) & 15)
        return fail(OUT_OF_RANGE, "gemm: buffers must be 16-byte aligned");
    if (bias != nullptr && (reinterpret_cast<uintptr_t>(bias) & 15)) return fail(OUT_OF_RANGE, "gemm: the bias must be 16-byte aligned");
    if (mode != 7 && mode != 8 && bias == nullptr) {  // a bias and the two rarer outputs: this file's kernel only
        // Schedules: this file's one tile per block; gemm2.cu's persistent blocks, whose epilogue overlaps the next tile's
        // products and whose MMAs read less shared memory per FLOP; gemm3.cu's pairs of SMs.  Measured on the benchmark's
        // shapes the persistent one wins where the epilogue stores f32 (plain or added to the output: 1.2 to 1.7 times
        // the rate), and loses where it stores f16 or computes a GELU per output.  tb_context_set_gemm_schedule (or
        // TACHYON_B200_GEMM=1..4 when the context is created) forces one, so a test can run all.  Up to 128 tokens the
        // persistent tile of 256 would be half empty.
        const int which = ctx->gemm_schedule;
        // 3 and 4: the pair schedule of gemm3.cu with tiles of 256 and 128 weight rows.
        if ((which == 3 || which == 4) && gemm_pair_supports(N, K, wbits, mode)) return launch_gemm_pair(ctx, w, s, a, M, N, K, out, mode, wbits, which == 4);
        // With f16 weights (no conversion: sixteen more warps drain accumulators) the persistent one wins everywhere but on
        // the gated outputs over a long K, where this file's larger tile reads less per FLOP (measured at 2048 tokens:
        // 32768 x 2048 gated 206 against 220 us; 3072 x 2048 33 against 42; at 16384 tokens, 3072 x 768 with a GELU 109 against 121).
        const bool stores_only = (mode == 0 || mode == 3) && M > 128;
        const bool prefer = wbits == 16 ? (M > 128 && !((mode == 2 || mode == 4) && K >= 1536)) : stores_only;
        if ((which == 2 || (which == 0 && prefer)) && gemm_persistent_supports(N, K, wbits)) return launch_gemm_persistent(ctx, w, s, a, M, N, K, out, mode, wbits);
    }
    EncodeTiled enc = encode_tiled();
    if (!enc) return fail(NO_DRIVER, "gemm: the driver does not export cuTensorMapEncodeTiled");
    CUtensorMap map;
    const cuuint64_t dims[2] = {K, M};
    const cuuint64_t strides[1] = {(cuuint64_t)K * 2};
    // Two token sub-tiles share a dequantised weight tile when that still leaves enough blocks for the machine.
    const int mt = (M > (uint32_t)BM && (uint64_t)((M + 255) / 256) * ((N + BN - 1) / BN) >= (uint64_t)ctx->sms * 3 / 4) ? 2 : 1;
    const cuuint32_t box[2] = {BK, (cuuint32_t)(mt * BM)}, elem[2] = {1, 1};
    const CUresult r = enc(&map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<__half*>(a), dims, strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE,
                           CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(CUDA, "gemm: cuTensorMapEncodeTiled failed (" + std::to_string((int)r) + ")");
    static bool configured[16] = {};
    if (!configured[ctx->gpu & 15]) {
        TB_CUDA(cudaFuncSetAttribute(gemm_q8_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes(1)));
        TB_CUDA(cudaFuncSetAttribute(gemm_q8_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes(2)));
        TB_CUDA(cudaFuncSetAttribute((gemm_q8_kernel<1, 4>), cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes(1)));
        TB_CUDA(cudaFuncSetAttribute((gemm_q8_kernel<2, 4>), cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes(2)));
        TB_CUDA(cudaFuncSetAttribute((gemm_q8_kernel<1, 16>), cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes(1)));
        TB_CUDA(cudaFuncSetAttribute((gemm_q8_kernel<2, 16>), cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes(2)));
        TB_CUDA(cudaFuncSetAttribute((gemm_f16_persistent_tile_kernel<1, WALK_EW>), cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes(1)));
        TB_CUDA(cudaFuncSetAttribute((gemm_f16_persistent_tile_kernel<2, WALK_EW>), cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes(2)));
        configured[ctx->gpu & 15] = true;
    }
    CUtensorMap wmap = map;  // f16 weights: [N, K] in tiles of 256 rows x 64 halves; unused otherwise
    if (wbits == 16) {
        const cuuint64_t wdims[2] = {K, N};
        const cuuint32_t wbox[2] = {BK, BN};
        const CUresult rw = enc(&wmap, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<int8_t*>(w), wdims, strides, wbox, elem, CU_TENSOR_MAP_INTERLEAVE_NONE,
                                CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (rw != CUDA_SUCCESS) return fail(CUDA, "gemm: cuTensorMapEncodeTiled failed for the weights (" + std::to_string((int)rw) + ")");
    }
    GemmArgs g{w, s, out, M, N, K, mode, bias};
    const dim3 grid((M + mt * BM - 1) / (mt * BM), (N + BN - 1) / BN);
    // f16 weights and more tiles than SMs: one block an SM walks the tiles (schedule 5 asks for the walk whatever the count).
    const uint32_t tiles = grid.x * grid.y, walkers = tiles < (uint32_t)ctx->sms ? tiles : (uint32_t)ctx->sms;
    const bool walk = wbits == 16 && ((ctx->gemm_walk && tiles > (uint32_t)ctx->sms) || ctx->gemm_schedule == 5);
    cudaError_t le;
    if (walk && mt == 2) le = launch_kernel(ctx, gemm_f16_persistent_tile_kernel<2, WALK_EW>, dim3(walkers), dim3(64 + 32 * WALK_EW), (size_t)smem_bytes(2), true, map, wmap, g, ctx->status);
    else if (walk) le = launch_kernel(ctx, gemm_f16_persistent_tile_kernel<1, WALK_EW>, dim3(walkers), dim3(64 + 32 * WALK_EW), (size_t)smem_bytes(1), true, map, wmap, g, ctx->status);
    else if (wbits == 16 && mt == 2) le = launch_kernel(ctx, gemm_q8_kernel<2, 16>, dim3(grid), dim3(THREADS), (size_t)smem_bytes(2), true, map, wmap, g, ctx->status);
    else if (wbits == 16) le = launch_kernel(ctx, gemm_q8_kernel<1, 16>, dim3(grid), dim3(THREADS), (size_t)smem_bytes(1), true, map, wmap, g, ctx->status);
    else if (wbits == 4 && mt == 2) le = launch_kernel(ctx, gemm_q8_kernel<2, 4>, dim3(grid), dim3(THREADS), (size_t)smem_bytes(2), true, map, wmap, g, ctx->status);
    else if (wbits == 4) le = launch_kernel(ctx, gemm_q8_kernel<1, 4>, dim3(grid), dim3(THREADS), (size_t)smem_bytes(1), true, map, wmap, g, ctx->status);
    else if (mt == 2) le = launch_kernel(ctx, gemm_q8_kernel<2>, dim3(grid), dim3(THREADS), (size_t)smem_bytes(2), true, map, wmap, g, ctx->status);
    else le = launch_kernel(ctx, gemm_q8_kernel<1>, dim3(grid), dim3(THREADS), (size_t)smem_bytes(1), true, map, wmap, g, ctx->status);
    TB_CUDA(le);
    return OK;
}

}  // namespace tb
