// The prefill / encoder product as a persistent kernel: D[M, N] = A[M, K] (f16) x W[N, K]^T with W quantised (int8 codes
// and an f16 scale per 32, or the reference's Q4 nibbles and a scale per 64), f32 accumulation in tensor memory.
// Stands in for the reference's gemm_q4 (crates/tachyon/src/ptx/gemm.rs:225-259) and gemm_q8* (ptx/encoder.rs:315-375);
// same results as gemm.cu's kernel, different schedule, built on what measuring that kernel showed: its tensor pipe
// waits for operands (the codes' trip from the L2, the conversion, the swizzled stores, and shared-memory bandwidth
// itself), and between tiles for the epilogue.  Here
//   * one block per SM walks the output tiles (256 tokens x 128 weight rows), tiles that share weight rows running at
//     the same time on neighbouring SMs so that their code reads meet in the L2;
//   * the codes come through their own ring of eight bulk tensor copies, far enough ahead that no warp waits for the L2;
//   * sixteen warps turn a stage's codes into f16 in the K-major swizzled layout the tensor core reads;
//   * the weight tile is the MMA's M operand and the 256 tokens its N operand, so a product of M128 N256 K16 reads
//     12 KiB of shared memory where two of M128 N128 read 16;
//   * the accumulator (lanes: weight rows, columns: tokens) is double-buffered (2 x 256 columns of tensor memory): eight
//     epilogue warps drain one tile, writing whole 128-byte segments of output rows, while the next is multiplied.
// Warps: 0 activation copies, 1 code copies, 2 MMA issue, 3..18 dequantisation, 19..26 epilogue.  Every wait is
// bounded; a warp that gives up records it in the context's status word and leaves its loops.
#include <cuda.h>

#include <string>

#include "common.cuh"
#include "internal.h"

namespace tb {

namespace {

constexpr int BM = 128, BN = 128, BK = 64, MT = 2;   // MMA M128 N128; two token sub-tiles share a weight tile
constexpr int ST = 3;                                // stages of f16 operands
constexpr int ST16 = 4;                              // the same with f16 weights, which need no ring of codes
constexpr int stages_of(int wb) { return wb == 16 ? ST16 : ST; }
constexpr int CS = 8;                                // stages of codes
constexpr int DW = 16, EW = 8;                       // dequantising and epilogue warps (a multiple of four: TMEM lane quarters)
constexpr int FIRST_DW = 3, FIRST_EW = FIRST_DW + DW;
constexpr int THREADS = 32 * (FIRST_EW + EW);
constexpr int A_BYTES = MT * BM * BK * 2, B_BYTES = BN * BK * 2, C_BYTES = BN * BK;  // per stage; codes at 8 bits
constexpr int OFF_A = 0, OFF_B = OFF_A + ST * A_BYTES, OFF_C = OFF_B + ST * B_BYTES, OFF_BAR = OFF_C + CS * C_BYTES;
constexpr int SMEM_BYTES = 1024 + OFF_BAR + 512;
static_assert(SMEM_BYTES <= 232448, "over the 227 KiB a block may use");

// kind::f16, f32 accumulator, K-major operands.  The weight tile is the MMA's A operand (M = 128 weight rows) and the token
// tile its B operand (N = 256 tokens): one M128 N256 product reads 12 KiB of shared memory per 16 of K where two M128 N128
// products with the roles the other way round read 16, and shared-memory bandwidth is what the tensor pipe waits for.
__host__ __device__ constexpr uint32_t idesc_for(uint32_t tokens) { return (1u << 4) | ((tokens >> 3) << 17) | ((uint32_t)(BN >> 4) << 24); }

__device__ __forceinline__ uint64_t smem_desc(uint32_t addr) {  // K-major, 128-byte rows, SWIZZLE_128B, 1024 bytes between 8-row groups
    const uint32_t lo = ((addr & 0x3ffffu) >> 4) | (1u << 16);
    const uint32_t hi = (1024u >> 4) | (1u << 14) | (2u << 29);
    return ((uint64_t)hi << 32) | lo;
}
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, int x, int y, uint64_t* bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(smem_addr(dst)),
                 "l"(map), "r"(x), "r"(y), "r"(smem_addr(bar))
                 : "memory");
}
__device__ __forceinline__ void mma_f16(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem_d),
        "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void mma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_addr(bar)) : "memory");
}
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

// Four int8 codes (one word) -> four f16 of code * scale: 0x6400 | (code ^ 0x80) is the f16 1024 + code + 128.
__device__ __forceinline__ void dequant4(uint32_t w, __half2 scale, uint32_t& lo, uint32_t& hi) {
    const uint32_t x = w ^ 0x80808080u;
    uint32_t a = __byte_perm(x, 0x64646464u, 0x5140), b = __byte_perm(x, 0x64646464u, 0x7362);
    const __half2 bias = __floats2half2_rn(1152.0f, 1152.0f);
    const __half2 va = __hmul2(__hsub2(*reinterpret_cast<__half2*>(&a), bias), scale), vb = __hmul2(__hsub2(*reinterpret_cast<__half2*>(&b), bias), scale);
    lo = *reinterpret_cast<const uint32_t*>(&va), hi = *reinterpret_cast<const uint32_t*>(&vb);
}
// Eight four-bit weights (quant.rs:60-66: low nibbles are weights 0..3, high nibbles 4..7) -> eight f16 of (n - 8) * scale.
__device__ __forceinline__ void dequant8_q4(uint32_t w, __half2 scale, uint32_t (&out)[4]) {
    const uint32_t lo = w & 0x0F0F0F0Fu, hi = (w >> 4) & 0x0F0F0F0Fu;
    const __half2 bias = __floats2half2_rn(1032.0f, 1032.0f);
    uint32_t p[4] = {__byte_perm(lo, 0x64646464u, 0x4140), __byte_perm(lo, 0x64646464u, 0x4342), __byte_perm(hi, 0x64646464u, 0x4140),
                     __byte_perm(hi, 0x64646464u, 0x4342)};
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const __half2 v = __hmul2(__hsub2(*reinterpret_cast<__half2*>(&p[i]), bias), scale);
        out[i] = *reinterpret_cast<const uint32_t*>(&v);
    }
}

struct Args {
    const __half* s;   // scales [N][K / 32] (8-bit codes) or [N][K / 64] (4-bit)
    void* out;
    uint32_t M, N, K;
    int mode;          // as gemm.cu: 0 f32, 1 f16, 2 GeGLU(tanh) pairs, 3 f32 +=, 4 GeGLU(erf) pairs, 5 GELU(erf) f16, 6 GELU(tanh) * mul f16
    const float* mul;  // mode 6: f32 [M][mul_stride], the factor of output (m, n) at m * mul_stride + n
    uint32_t mul_stride;
    // Tokens a tile (the MMA's N): 256, 192 or 128, picked by the launcher so that the tiles fill whole rounds of the machine's
    // SMs (192 tiles of 256 tokens are two rounds of 148 at 65 %; 264 tiles of 192 tokens are two shorter rounds at 89 %).
    uint32_t tn;
    int red;           // mode 3: the sums added at the L2 by reductions, no load in the epilogue
    GemmRope rope;     // mode 1: table != null turns the pairs of the first rope.cols weight rows (internal.h)
};

struct Bars {
    uint64_t full[ST16], empty[ST16], c_full[CS], c_empty[CS], acc_full[2], acc_empty[2];
    uint32_t tmem;
};

template <int WB, bool ROPE = false>
__global__ void __launch_bounds__(THREADS, 1) gemm_persistent_kernel(const __grid_constant__ CUtensorMap a_map, const __grid_constant__ CUtensorMap w_map, const Args g,
                                                                     uint32_t* status) {
    extern __shared__ uint8_t raw_unaligned[];
    uint8_t* raw = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(raw_unaligned) + 1023) & ~uintptr_t(1023));
    // WB == 16: the weights are f16 already; their tiles come by TMA (warp 0) into the operand stages, of which there are four
    // in place of three and the ring of codes; warp 1 and the dequantising warps have nothing to do.
    constexpr int ST = stages_of(WB);
    static_assert(stages_of(16) * (A_BYTES + B_BYTES) <= OFF_BAR, "the f16 stages must end before the barriers");
    uint8_t *As = raw + OFF_A, *Bs = raw + OFF_A + ST * A_BYTES, *Cs = raw + OFF_C;
    Bars& bar = *reinterpret_cast<Bars*>(raw + OFF_BAR);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t nk = g.K / BK, tiles_m = (g.M + g.tn - 1) / g.tn, tiles_n = (g.N + BN - 1) / BN, tiles = tiles_m * tiles_n;
    const uint32_t a_bytes = g.tn * BK * 2;  // what a stage's copy of the activations brings: g.tn rows of 128 bytes

    if (threadIdx.x == 0) {
        for (int i = 0; i < ST; i++) mbar_init(&bar.full[i], WB == 16 ? 1 : DW + 1), mbar_init(&bar.empty[i], 1);
        for (int i = 0; i < CS; i++) mbar_init(&bar.c_full[i], 1), mbar_init(&bar.c_empty[i], DW);
        for (int i = 0; i < 2; i++) mbar_init(&bar.acc_full[i], 1), mbar_init(&bar.acc_empty[i], WB == 16 ? DW + EW : EW);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 2) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_addr(&bar.tmem)), "r"(512u) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = bar.tmem;
    // Set up: the kernel behind may be scheduled; this one reads and writes only once the kernel in front is done (both do
    // nothing where a launch is not programmatic).
    pdl_launch_dependents();
    pdl_wait();

    // Tile t: token tile t % tiles_m, weight tile t / tiles_m: blocks that run together share weight rows.
    if (warp == 0) {
        if (lane == 0) {
            uint32_t it = 0;
            for (uint32_t t = blockIdx.x; t < tiles; t += gridDim.x) {
                const uint32_t m0 = (t % tiles_m) * g.tn, n0 = (t / tiles_m) * BN;
                for (uint32_t kt = 0; kt < nk; kt++, it++) {
                    const uint32_t s = it % ST;
                    if (it >= ST && !mbar_wait(&bar.empty[s], ((it / ST) - 1) & 1)) {
                        atomicCAS(status, ERR_NONE, ERR_WAIT_EMPTY);
                        t = tiles;
                        break;
                    }
                    mbar_expect_tx(&bar.full[s], WB == 16 ? a_bytes + B_BYTES : a_bytes);
                    tma_load_2d(As + s * A_BYTES, &a_map, (int)(kt * BK), (int)m0, &bar.full[s]);
                    if constexpr (WB == 16) tma_load_2d(Bs + s * B_BYTES, &w_map, (int)(kt * BK), (int)n0, &bar.full[s]);
                }
            }
        }
    } else if (warp == 1) {
        if (WB != 16 && lane == 0) {
            uint32_t ic = 0;
            for (uint32_t t = blockIdx.x; t < tiles; t += gridDim.x) {
                const uint32_t n0 = (t / tiles_m) * BN;
                for (uint32_t kt = 0; kt < nk; kt++, ic++) {
                    const uint32_t c = ic % CS;
                    if (ic >= CS && !mbar_wait(&bar.c_empty[c], ((ic / CS) - 1) & 1)) {
                        atomicCAS(status, ERR_NONE, ERR_WAIT_EMPTY);
                        t = tiles;
                        break;
                    }
                    mbar_expect_tx(&bar.c_full[c], C_BYTES * WB / 8);
                    tma_load_2d(Cs + c * C_BYTES, &w_map, (int)(kt * BK * WB / 8), (int)n0, &bar.c_full[c]);
                }
            }
        }
    } else if (warp == 2) {
        if (lane == 0) {
            uint32_t it = 0, ti = 0;
            bool ok = true;
            for (uint32_t t = blockIdx.x; t < tiles && ok; t += gridDim.x, ti++) {
                const uint32_t b = ti & 1;
                if (ti >= 2 && !mbar_wait(&bar.acc_empty[b], ((ti >> 1) - 1) & 1)) {
                    atomicCAS(status, ERR_NONE, ERR_WAIT_EMPTY);
                    break;
                }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                for (uint32_t kt = 0; kt < nk; kt++, it++) {
                    const uint32_t s = it % ST;
                    if (!mbar_wait(&bar.full[s], (it / ST) & 1)) {
                        atomicCAS(status, ERR_NONE, ERR_WAIT_FULL);
                        ok = false;
                        break;
                    }
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const uint32_t a = smem_addr(As + s * A_BYTES), bb = smem_addr(Bs + s * B_BYTES);
#pragma unroll
                    for (int k = 0; k < BK / 16; k++) mma_f16(tmem + b * (MT * BM), smem_desc(bb + k * 32), smem_desc(a + k * 32), idesc_for(g.tn), (kt > 0 || k > 0) ? 1u : 0u);
                    mma_commit(&bar.empty[s]);
                }
                mma_commit(&bar.acc_full[b]);  // arrives when the tile's products have finished
            }
        }
    } else if (WB != 16 && warp < FIRST_EW) {
        // Dequantisation: thread j takes the 16 codes of piece (row j / 4, quarter j % 4) of every stage.
        const int j = threadIdx.x - 32 * FIRST_DW, row = j >> 2, qtr = j & 3;
        constexpr uint32_t GS = WB == 4 ? 8 : 4;               // k tiles one 16-byte load of scales covers
        const uint32_t spr = g.K / (WB == 4 ? 64 : 32);        // scales per row
        uint32_t it = 0, ic = 0;
        bool ok = true;
        for (uint32_t t = blockIdx.x; t < tiles && ok; t += gridDim.x) {
            const uint32_t n = (t / tiles_m) * BN + row;
            const bool live = n < g.N;
            const __half* srow = g.s + (size_t)n * spr;
            auto scales_from = [&](uint32_t kt) -> uint4 {  // the row's eight scales from k tile `kt` on
                const uint32_t at = kt * (WB == 4 ? 1 : 2);
                if (live && at + 8 <= spr && spr % 8 == 0) return __ldg(reinterpret_cast<const uint4*>(srow + at));
                uint32_t w[4] = {0u, 0u, 0u, 0u};
#pragma unroll
                for (uint32_t e = 0; e < 8; e++)
                    if (live && at + e < spr) w[e >> 1] |= (uint32_t)__half_as_ushort(srow[at + e]) << (16 * (e & 1));
                return make_uint4(w[0], w[1], w[2], w[3]);
            };
            uint4 sc = scales_from(0), sc_next = sc;
            for (uint32_t kt = 0; kt < nk; kt++, it++, ic++) {
                if (kt % GS == 0) {
                    if (kt > 0) sc = sc_next;
                    if (kt + GS < nk) sc_next = scales_from(kt + GS);  // one group ahead
                }
                const uint32_t c = ic % CS, s = it % ST;
                if (!mbar_wait(&bar.c_full[c], (ic / CS) & 1)) {
                    atomicCAS(status, ERR_NONE, ERR_WAIT_FULL);
                    ok = false;
                    break;
                }
                uint32_t v[8];
                const uint32_t h = WB == 4 ? (kt & 7u) : 2u * (kt & 3u) + (uint32_t)(qtr >> 1);  // which of the eight scales
                const uint32_t word = (h >> 1) == 0 ? sc.x : (h >> 1) == 1 ? sc.y : (h >> 1) == 2 ? sc.z : sc.w;
                const __half2 s2 = __half2half2(__ushort_as_half((unsigned short)((h & 1u) ? (word >> 16) : (word & 0xffffu))));
                if constexpr (WB == 4) {
                    const uint2 cw = *reinterpret_cast<const uint2*>(Cs + c * C_BYTES + row * (BK / 2) + qtr * 8);
                    uint32_t a[4], b[4];
                    dequant8_q4(cw.x, s2, a), dequant8_q4(cw.y, s2, b);
#pragma unroll
                    for (int e = 0; e < 4; e++) v[e] = a[e], v[4 + e] = b[e];
                } else {
                    const uint4 cw = *reinterpret_cast<const uint4*>(Cs + c * C_BYTES + row * BK + qtr * 16);
                    dequant4(cw.x, s2, v[0], v[1]), dequant4(cw.y, s2, v[2], v[3]), dequant4(cw.z, s2, v[4], v[5]), dequant4(cw.w, s2, v[6], v[7]);
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(&bar.c_empty[c]);  // the codes are in registers
                if (it >= ST && !mbar_wait(&bar.empty[s], ((it / ST) - 1) & 1)) {
                    atomicCAS(status, ERR_NONE, ERR_WAIT_EMPTY);
                    ok = false;
                    break;
                }
                uint8_t* base = Bs + s * B_BYTES + row * 128;
                *reinterpret_cast<uint4*>(base + (((2 * qtr) ^ (row & 7)) << 4)) = make_uint4(v[0], v[1], v[2], v[3]);
                *reinterpret_cast<uint4*>(base + (((2 * qtr + 1) ^ (row & 7)) << 4)) = make_uint4(v[4], v[5], v[6], v[7]);
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // the tensor core reads through the async proxy
                __syncwarp();
                if (lane == 0) mbar_arrive(&bar.full[s]);
            }
        }
    } else {
        // Epilogue: the accumulator's lanes are weight rows, its columns tokens.  A warp reads the lanes of its quarter
        // q = warp % 4, 32 tokens at a time (the EW / 4 warps of a quarter take alternate blocks of tokens); for each token
        // its 32 lanes then hold 32 consecutive outputs of that token's row, which go out as one 128-byte (f32) store.
        // With f16 weights the sixteen warps that would convert codes drain accumulators too: six warps a quarter.
        constexpr int FIRST = WB == 16 ? FIRST_DW : FIRST_EW, PARTS = (WB == 16 ? DW + EW : EW) / 4;
        const uint32_t q = warp & 3, part = (warp - FIRST) >> 2;
        uint32_t ti = 0;
        for (uint32_t t = blockIdx.x; t < tiles; t += gridDim.x, ti++) {
            const uint32_t b = ti & 1, m0 = (t % tiles_m) * g.tn, n = (t / tiles_m) * BN + 32 * q + lane;
            if (!mbar_wait(&bar.acc_full[b], (ti >> 1) & 1)) {
                atomicCAS(status, ERR_NONE, ERR_WAIT_FULL);
                break;
            }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const bool row_ok = n < g.N;  // the same for the whole warp: N is a multiple of 32
#pragma unroll 1
            for (int cb = part; cb < (int)(g.tn / 32); cb += PARTS) {
                uint32_t r[32];
                tmem_load32(tmem + ((32 * q) << 16) + b * (MT * BM) + cb * 32, r);
                if (!row_ok) continue;
                const uint32_t mb = m0 + cb * 32;
                if (g.mode == 0) {
                    float* dst = static_cast<float*>(g.out) + (size_t)mb * g.N + n;
#pragma unroll
                    for (int i = 0; i < 32; i++)
                        if (mb + i < g.M) dst[(size_t)i * g.N] = __uint_as_float(r[i]);
                } else if (g.mode == 3) {
                    // The old values first, sixteen loads in flight, then the sums (a load after a store to the same array
                    // would wait for it).
                    float* dst = static_cast<float*>(g.out) + (size_t)mb * g.N + n;
                    if (g.red) {
                        // x += D as 32 reductions at the L2: the same single f32 addition per element, but the epilogue waits
                        // for no load (16384 x 768 x 768: 25.9 against 34.0 us; the encoder's batch 2 % shorter).
#pragma unroll
                        for (int i = 0; i < 32; i++)
                            if (mb + i < g.M) asm volatile("red.global.add.f32 [%0], %1;" ::"l"(dst + (size_t)i * g.N), "f"(__uint_as_float(r[i])) : "memory");
                        continue;
                    }
#pragma unroll
                    for (int half = 0; half < 2; half++) {
                        float old[16];
#pragma unroll
                        for (int i = 0; i < 16; i++) old[i] = mb + 16 * half + i < g.M ? __ldcg(dst + (size_t)(16 * half + i) * g.N) : 0.0f;
#pragma unroll
                        for (int i = 0; i < 16; i++)
                            if (mb + 16 * half + i < g.M) dst[(size_t)(16 * half + i) * g.N] = old[i] + __uint_as_float(r[16 * half + i]);
                    }
                } else if (g.mode == 1 || g.mode == 5 || g.mode == 6) {
                    // Two lanes (weight rows n, n + 1) trade values so that each writes a pair of halves: the even lane
                    // the even tokens of a pair of tokens, the odd lane the odd ones.
                    const uint32_t odd = lane & 1u;
                    __half* dst = static_cast<__half*>(g.out) + (size_t)(mb + odd) * g.N + (n - odd);
                    const float* mrow = g.mode == 6 ? g.mul + (size_t)mb * g.mul_stride + n : nullptr;
                    // Rotary embedding in the store: after the trade below a lane holds rows (n - odd, n - odd + 1) of its token,
                    // the pair (a, b) of rotation j; each is rounded to f16 first, then (a c - b s, b c + a s) as a product and one
                    // fused multiply-add, so the bits are those of a rotation kernel run on the stored halves.
                    // (A kernel of its own, ROPE: with this in the common kernel every mode's epilogue paid for it.)
                    bool turn = false;
                    uint32_t my_pos = 0, rot = 0;
                    if constexpr (ROPE) {
                        turn = n < g.rope.cols;
                        my_pos = turn && mb + lane < g.M ? __ldg(g.rope.pos + mb + lane) : 0u;
                        rot = ((n - odd) % g.rope.head) / 2;
                    }
#pragma unroll
                    for (int k = 0; k < 16; k++) {
                        float v0 = __uint_as_float(r[2 * k]), v1 = __uint_as_float(r[2 * k + 1]);
                        if (g.mode == 5) v0 = gelu_erf_lean(v0), v1 = gelu_erf_lean(v1);
                        if (g.mode == 6) {
                            v0 = mb + 2 * k < g.M ? gelu_tanh(v0) * __ldg(mrow + (size_t)(2 * k) * g.mul_stride) : 0.0f;
                            v1 = mb + 2 * k + 1 < g.M ? gelu_tanh(v1) * __ldg(mrow + (size_t)(2 * k + 1) * g.mul_stride) : 0.0f;
                        }
                        const float got = __shfl_xor_sync(0xffffffffu, odd ? v0 : v1, 1);  // the neighbour's value for my token
                        __half2 pair = odd ? __floats2half2_rn(got, v1) : __floats2half2_rn(v0, got);
                        if constexpr (ROPE) {  // every lane reaches the shuffle
                            const uint32_t p = __shfl_sync(0xffffffffu, my_pos, 2 * k + odd);
                            if (turn) {
                                const float2 cs = __ldg(g.rope.table + (size_t)p * (g.rope.head / 2) + rot);
                                const float2 ab = __half22float2(pair);
                                pair = __floats2half2_rn(__fmaf_rn(ab.y, -cs.y, __fmul_rn(ab.x, cs.x)), __fmaf_rn(ab.x, cs.y, __fmul_rn(ab.y, cs.x)));
                            }
                        }
                        if (mb + 2 * k + odd < g.M) *reinterpret_cast<__half2*>(dst + (size_t)(2 * k) * g.N) = pair;
                    }
                } else {
                    // Weight rows (2j, 2j + 1) are (gate_j, up_j): an even lane holds gate_j of two tokens, the odd lane beside it
                    // up_j.  They trade one value each, so that the even lane has (gate, up) of the even token and the odd lane
                    // those of the odd token, and every lane computes one output.  Lanes 4c .. 4c + 3 then hold outputs j and j + 1
                    // of two tokens: lanes 4c and 4c + 1 take their neighbour pair's and write two halves each.
                    const bool odd = (lane & 1u) != 0, second = (lane & 2u) != 0;
                    __half* dst = static_cast<__half*>(g.out) + (size_t)(mb + (odd ? 1 : 0)) * (g.N / 2) + (n - (lane & 3u)) / 2;
#pragma unroll
                    for (int k = 0; k < 16; k++) {
                        const float v0 = __uint_as_float(r[2 * k]), v1 = __uint_as_float(r[2 * k + 1]);
                        const float got = __shfl_xor_sync(0xffffffffu, odd ? v0 : v1, 1);  // even: up of the even token; odd: gate of the odd token
                        const float gate = odd ? got : v0, up = odd ? v1 : got;
                        const float a = (g.mode == 2 ? gelu_tanh(gate) : gelu_erf_lean(gate)) * up;
                        const float other = __shfl_xor_sync(0xffffffffu, a, 2);  // output j + 1 (or j) of the same token
                        const __half2 pair = second ? __floats2half2_rn(other, a) : __floats2half2_rn(a, other);
                        if (!second && mb + 2 * k + (odd ? 1 : 0) < g.M) *reinterpret_cast<__half2*>(dst + (size_t)(2 * k) * (g.N / 2)) = pair;
                    }
                }
            }
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(&bar.acc_empty[b]);
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 2) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512u) : "memory");
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

// The shapes this schedule takes: everything gemm.cu's kernel takes with whole 16-byte rows of codes.
bool gemm_persistent_supports(uint32_t N, uint32_t K, uint32_t wbits) { return K % BK == 0 && (K * wbits / 8) % 16 == 0 && N > 0; }  // wbits 16: f16 weights

int launch_gemm_persistent(tb_context* ctx, const int8_t* w, const __half* s, const __half* a, uint32_t M, uint32_t N, uint32_t K, void* out, int mode,
                           uint32_t wbits, const float* mul, uint32_t mul_stride, const GemmRope* rope) {
    EncodeTiled enc = encode_tiled();
    if (rope && (mode != 1 || wbits != 16 || rope->head == 0 || rope->head % 2 != 0 || rope->cols % 32 != 0 || rope->cols > N)) return fail(OUT_OF_RANGE, "gemm: a rotation wants the f16 store, an even head size and whole groups of 32 rows");
    if (!enc) return fail(NO_DRIVER, "gemm: the driver does not export cuTensorMapEncodeTiled");
    // Tokens a tile: 256, or 192 or 128 where that fills whole rounds of the SMs so much better that it pays (a tenth at least by
    // rounds x (tokens + 32), the 32 standing for what a tile costs whatever its size).  Other sizes leave the epilogue's six
    // warps a quarter unevenly loaded, and where the epilogue is what a tile waits for (few K tiles) smaller tiles lose:
    // measured with 224 tokens on the encoder's 16384 x 3072 x 768 with a GELU, 114 against 109 us.
    uint32_t tn = MT * BM;
    {
        const uint64_t tiles_n = (N + BN - 1) / BN;
        auto cost = [&](uint32_t c) {
            const uint64_t tiles = (uint64_t)((M + c - 1) / c) * tiles_n, rounds = (tiles + ctx->sms - 1) / ctx->sms;
            return rounds * (c + 32);
        };
        const uint64_t whole = cost(MT * BM);
        uint64_t best = whole - whole / 10;
        for (uint32_t c : {192u, 128u})
            if (cost(c) < best) best = cost(c), tn = c;
    }
    CUtensorMap amap, wmap;
    {
        const cuuint64_t dims[2] = {K, M};
        const cuuint64_t strides[1] = {(cuuint64_t)K * 2};
        const cuuint32_t box[2] = {BK, tn}, elem[2] = {1, 1};
        const CUresult r = enc(&amap, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<__half*>(a), dims, strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE,
                               CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) return fail(CUDA, "gemm: cuTensorMapEncodeTiled (activations) failed (" + std::to_string((int)r) + ")");
    }
    {
        const cuuint64_t row = (cuuint64_t)K * wbits / 8;  // bytes of codes (or of f16 weights) per weight row
        const cuuint64_t dims[2] = {wbits == 16 ? (cuuint64_t)K : row, N};
        const cuuint64_t strides[1] = {row};
        const cuuint32_t box[2] = {(cuuint32_t)(wbits == 16 ? BK : BK * wbits / 8), BN}, elem[2] = {1, 1};
        // f16 weights go straight into the operand stage: halves, 128-byte swizzle, like the activations
        const CUresult r = enc(&wmap, wbits == 16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<int8_t*>(w), dims, strides, box, elem,
                               CU_TENSOR_MAP_INTERLEAVE_NONE, wbits == 16 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                               CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) return fail(CUDA, "gemm: cuTensorMapEncodeTiled (codes) failed (" + std::to_string((int)r) + ")");
    }
    static bool configured[16] = {};
    if (!configured[ctx->gpu & 15]) {
        TB_CUDA(cudaFuncSetAttribute(gemm_persistent_kernel<8>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES));
        TB_CUDA(cudaFuncSetAttribute(gemm_persistent_kernel<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES));
        TB_CUDA(cudaFuncSetAttribute(gemm_persistent_kernel<16>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES));
        TB_CUDA(cudaFuncSetAttribute((gemm_persistent_kernel<16, true>), cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES));
        configured[ctx->gpu & 15] = true;
    }
    const uint32_t tiles = ((M + tn - 1) / tn) * ((N + BN - 1) / BN);
    const uint32_t grid = tiles < (uint32_t)ctx->sms ? tiles : (uint32_t)ctx->sms;
    const Args g{s, out, M, N, K, mode, mul, mul_stride, tn, ctx->gemm_red ? 1 : 0, rope ? *rope : GemmRope{nullptr, nullptr, 0, 2}};
    cudaError_t le;
    if (wbits == 16 && rope) le = launch_kernel(ctx, gemm_persistent_kernel<16, true>, dim3(grid), dim3(THREADS), (size_t)SMEM_BYTES, true, amap, wmap, g, ctx->status);
    else if (wbits == 16) le = launch_kernel(ctx, gemm_persistent_kernel<16>, dim3(grid), dim3(THREADS), (size_t)SMEM_BYTES, true, amap, wmap, g, ctx->status);
    else if (wbits == 4) le = launch_kernel(ctx, gemm_persistent_kernel<4>, dim3(grid), dim3(THREADS), (size_t)SMEM_BYTES, true, amap, wmap, g, ctx->status);
    else le = launch_kernel(ctx, gemm_persistent_kernel<8>, dim3(grid), dim3(THREADS), (size_t)SMEM_BYTES, true, amap, wmap, g, ctx->status);
    TB_CUDA(le);
    return OK;
}

}  // namespace tb
