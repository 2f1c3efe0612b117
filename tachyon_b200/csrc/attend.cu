// Decode attention for one new token: grouped queries over an f16 key/value cache, split over blocks along the
// positions and merged by the last block to finish.  Replaces the reference's attend_256 family
// (crates/tachyon/src/ptx/attend.rs:423-466; setup 281-330, step 213-225, partial 334-367, combine 371-405).
//
// Per key-value head there are `splits` blocks; each takes a span of the newest min(pos + 1, window) positions,
// brings their keys and values into shared memory with asynchronous 16-byte copies (into padded rows, so that the
// tensor-core fragment loads meet no bank conflicts), and keeps running softmax statistics for the query heads of its group.  Optional per-head RMS-norms and
// RoPE on the new query/key/value (the reference's Gemma-4 semantics) and a plain mode (no norms, no rotation, caller's
// scale) are parameters.  The new token's key/value are written to slot pos % cap by the first block of each group and
// used from f32, as the reference does.
//
// Scratch: per (kv head, split) the block's maxima, sums and unnormalised outputs; a counter per kv head that is zero
// between launches.  Blocks never wait on one another: a block that is not the last to finish just exits.
#include "attend_body.cuh"

#include <mutex>
#include <string>

namespace tb {

using namespace attend;

namespace {

template <int G>
__global__ void __launch_bounds__(THREADS) attend_kernel(const AttendParams p) {
    extern __shared__ __align__(128) uint8_t raw[];
    ClusterSmem& cs = *reinterpret_cast<ClusterSmem*>(raw);
    Smem& sm = cs.body;
    const int tid = threadIdx.x;
    // The hint is about weights no kernel writes: ask for them before waiting for the previous kernel.
    if (tid == 0) prefetch_hint(p.pf, blockIdx.y * gridDim.x + blockIdx.x, gridDim.x * gridDim.y);
    // The norm weights and the RoPE table are model constants (2.5 KiB): ask the L2 for them ahead of the wait.
    if (tid < 8 && p.q_norm != nullptr) prefetch_line_l2(p.q_norm + tid * 32);
    else if (tid >= 8 && tid < 16 && p.k_norm != nullptr) prefetch_line_l2(p.k_norm + (tid - 8) * 32);
    else if (tid >= 16 && tid < 20 && p.freq != nullptr) prefetch_line_l2(p.freq + (tid - 16) * 32);
    // The decoder's caches and position do not depend on the kernel right before this one: ask for the first tile now,
    // and have the rotation's cosines and sines ready.
    uint32_t pos = 0;
    bool sent = false;
    Trig trig;
    if (p.early) {
        pos = ld_cg_u(p.pos);
        sent = load_first_tile(p, sm, blockIdx.x, blockIdx.y, pos, tid);
        trig = rope_trig(p.freq, pos, tid & 31, p.trig);
    }
    unsigned long long* stamp = nullptr;
    if (p.stamps != nullptr && tid == 0) {
        const uint32_t b = blockIdx.y * gridDim.x + blockIdx.x;
        if (b == 0 || b == gridDim.x * gridDim.y - 1) stamp = p.stamps + (b == 0 ? 0 : 4);
    }
    if (stamp) stamp[0] = global_ns();
    // Nothing this kernel does before its wait depends on the kernels in front of it, and nothing it writes is read
    // before a kernel's own wait: the kernel behind it may start at once.
    pdl_launch_dependents();
    pdl_wait();
    if (stamp) stamp[1] = global_ns();
    if (!p.early) {
        pos = ld_cg_u(p.pos);
        trig = rope_trig(p.freq, pos, tid & 31, p.trig);
    }
    if (p.cluster > 1) attend_cluster_body<G>(p, cs, tid, blockIdx.x, blockIdx.y, pos, sent, trig);
    else attend_body<G, false>(p, sm, tid, blockIdx.x, blockIdx.y, pos, sent, trig);
    if (stamp) stamp[3] = global_ns();
}

// table[pos][i] = cos(pos * freq[i]), table[pos][128 + i] = sin(pos * freq[i]): sincosf of the f32 product, as rope_trig.
__global__ void rope_table_kernel(const float* freq, uint32_t positions, float* table) {
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= positions * (D / 2)) return;
    const uint32_t pos = i / (D / 2), k = i % (D / 2);
    float s, c;
    sincosf((float)pos * freq[k], &s, &c);
    table[(size_t)pos * D + k] = c, table[(size_t)pos * D + D / 2 + k] = s;
}

}  // namespace

int launch_rope_table(tb_context* ctx, const float* freq, uint32_t positions, float* table) {
    if (!freq || !table || positions == 0) return fail(OUT_OF_RANGE, "rope table: bad arguments");
    const uint32_t n = positions * (D / 2);
    rope_table_kernel<<<(n + 255) / 256, 256, 0, ctx->stream>>>(freq, positions, table);
    TB_CUDA(cudaGetLastError());
    return OK;
}

size_t attend_partial_floats(uint32_t heads, uint32_t kv_heads, uint32_t splits) {
    const uint32_t group = heads / kv_heads;
    return (size_t)kv_heads * splits * (attend_header(group) + (size_t)group * D);
}

int launch_attend(tb_context* ctx, const AttendParams& p) {
    if (p.kv_heads == 0 || p.heads % p.kv_heads != 0) return fail(OUT_OF_RANGE, "attend: heads must be a multiple of kv_heads");
    const uint32_t group = p.heads / p.kv_heads;
    if (group != 1 && group != 2 && group != 4) return fail(UNSUPPORTED, "attend: 1, 2 or 4 query heads per key-value head");
    if (p.cap == 0 || p.window == 0 || p.window > p.cap) return fail(OUT_OF_RANGE, "attend: need 0 < window <= cap");
    if (p.splits == 0 || p.splits > 1024) return fail(OUT_OF_RANGE, "attend: splits out of range");
    if (!p.qkv || !p.kc || !p.vc || !p.pos || (!p.defer && (!p.out || !p.count)) || ((p.splits > 1 || p.defer) && !p.partial)) return fail(OUT_OF_RANGE, "attend: null argument");
    if ((p.q_norm == nullptr) != (p.k_norm == nullptr)) return fail(OUT_OF_RANGE, "attend: q_norm and k_norm go together");
    if (p.cluster != 1 && ((p.cluster != 2 && p.cluster != 4 && p.cluster != 8) || p.splits % p.cluster != 0 || !p.defer))
        return fail(OUT_OF_RANGE, "attend: clusters of 2, 4 or 8 splits, dividing the splits, and only with the merge left to the next kernel");
    if ((reinterpret_cast<uintptr_t>(p.kc) | reinterpret_cast<uintptr_t>(p.vc) | reinterpret_cast<uintptr_t>(p.qkv)) & 15) return fail(OUT_OF_RANGE, "attend: buffers must be 16-byte aligned");
    const dim3 grid(p.kv_heads, p.splits), block(THREADS);
    {
        // Per device, once; threads that own contexts on different GPUs may get here together.
        static std::mutex guard;
        static bool configured[64] = {};
        std::lock_guard<std::mutex> lock(guard);
        if (!configured[ctx->gpu & 63]) {
            TB_CUDA(cudaFuncSetAttribute(attend_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sizeof(ClusterSmem)));
            TB_CUDA(cudaFuncSetAttribute(attend_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sizeof(ClusterSmem)));
            TB_CUDA(cudaFuncSetAttribute(attend_kernel<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)sizeof(ClusterSmem)));
            // As much of each SM as possible to shared memory: in a decode step this kernel's blocks move in beside blocks
            // of the products around it, and an SM's split cannot change while blocks run on it.
            TB_CUDA(cudaFuncSetAttribute(attend_kernel<1>, cudaFuncAttributePreferredSharedMemoryCarveout, (int)cudaSharedmemCarveoutMaxShared));
            TB_CUDA(cudaFuncSetAttribute(attend_kernel<2>, cudaFuncAttributePreferredSharedMemoryCarveout, (int)cudaSharedmemCarveoutMaxShared));
            TB_CUDA(cudaFuncSetAttribute(attend_kernel<4>, cudaFuncAttributePreferredSharedMemoryCarveout, (int)cudaSharedmemCarveoutMaxShared));
            configured[ctx->gpu & 63] = true;
        }
    }
    const dim3 cluster(1, p.cluster, 1);
    if (group == 4) TB_CUDA(launch_kernel(ctx, attend_kernel<4>, grid, block, sizeof(ClusterSmem), true, cluster, p));
    else if (group == 2) TB_CUDA(launch_kernel(ctx, attend_kernel<2>, grid, block, sizeof(ClusterSmem), true, cluster, p));
    else TB_CUDA(launch_kernel(ctx, attend_kernel<1>, grid, block, sizeof(ClusterSmem), true, cluster, p));
    return OK;
}

// ---- the variant that allocates nothing ---------------------------------------------------------------------------
//
// tb_attend_decode needs scratch from its caller (the per-split partial results and the per-head counters).  Some
// callers have no way to provide it: an engine whose device memory was carved up once at start-up and has nothing left
// to hand out, or a latency-critical loop that may not call cudaMalloc because that call synchronises the whole device.
// For them the scratch lives here, in the library's own image: a fixed array every GPU that loads the library holds
// until the process exits.  Its size covers up to STATIC_KV_HEADS key-value heads with up to STATIC_SPLITS blocks each
// and four query heads per key-value head (1,057,024 bytes, about 1.01 MiB); anything larger is refused.
constexpr uint32_t STATIC_KV_HEADS = 4;
constexpr uint32_t STATIC_SPLITS = 64;
constexpr size_t STATIC_FLOATS = (size_t)STATIC_KV_HEADS * STATIC_SPLITS * (2 * MAXG + MAXG * D);
constexpr size_t STATIC_COUNTERS = 64;  // words, after the partials

namespace {
static __device__ __align__(256) float g_attend_scratch[STATIC_FLOATS + STATIC_COUNTERS];
// Device address of the array on each GPU ordinal, resolved on first use.  The name above is only a handle on the host:
// it must go through cudaGetSymbolAddress before a kernel can be given it.
float* g_attend_scratch_ptr[64] = {};
}  // namespace

int launch_attend_static(tb_context* ctx, AttendParams p) {
    if (p.kv_heads == 0 || p.heads % p.kv_heads != 0 || p.heads / p.kv_heads > (uint32_t)MAXG)
        return fail(OUT_OF_RANGE, "attend (static scratch): at most 4 query heads per key-value head");
    if (p.kv_heads > STATIC_KV_HEADS || p.splits > STATIC_SPLITS)
        return fail(OUT_OF_RANGE, "attend (static scratch): the built-in scratch holds at most 4 key-value heads x 64 splits; got " +
                                      std::to_string(p.kv_heads) + " x " + std::to_string(p.splits) + " (use tb_attend_decode with caller scratch)");
    if (ctx->gpu < 0 || ctx->gpu >= 64) return fail(OUT_OF_RANGE, "attend (static scratch): GPU ordinal out of range");
    float* base = nullptr;
    {
        // Once per device, with that device current; under a lock, since threads with contexts on different GPUs share
        // the table.
        static std::mutex guard;
        std::lock_guard<std::mutex> lock(guard);
        if (g_attend_scratch_ptr[ctx->gpu] == nullptr) {
            TB_CUDA(cudaSetDevice(ctx->gpu));
            void* ptr = nullptr;
            TB_CUDA(cudaGetSymbolAddress(&ptr, g_attend_scratch));
            g_attend_scratch_ptr[ctx->gpu] = static_cast<float*>(ptr);
        }
        base = g_attend_scratch_ptr[ctx->gpu];
    }
    p.partial = base;
    p.count = reinterpret_cast<uint32_t*>(base + STATIC_FLOATS);
    // The array keeps whatever the last call left.  The partials are overwritten before they are read; the counters must
    // start at zero, so they are cleared on the stream ahead of the kernel.
    TB_CUDA(cudaMemsetAsync(p.count, 0, STATIC_COUNTERS * sizeof(uint32_t), ctx->stream));
    return launch_attend(ctx, p);
}

}  // namespace tb
