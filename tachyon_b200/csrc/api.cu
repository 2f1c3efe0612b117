// The C ABI's context, memory, event and per-kernel entry points (include/tachyon_b200.h).  Each validates its
// descriptor on the host and launches nothing when validation fails, as the reference's `within()` checks do
// (crates/tachyon/src/cuda/mod.rs:377-379).
#include "../../include/tachyon_b200.h"
#include "common.cuh"
#include "internal.h"

#include <dlfcn.h>

#include <mutex>
#include <string>

namespace tb {

static thread_local std::string g_error;

int fail(int status, const std::string& what) {
    g_error = what;
    return status;
}

int cuda_fail(cudaError_t e, const char* where) {
    cudaGetLastError();  // clear the sticky "last error" of non-fatal failures
    const int status = e == cudaErrorMemoryAllocation ? OUT_OF_MEMORY
                       : (e == cudaErrorInsufficientDriver || e == cudaErrorNoDevice || e == cudaErrorInitializationError) ? NO_DRIVER
                                                                                                                           : CUDA;
    return fail(status, std::string(where) + ": " + cudaGetErrorName(e) + " (" + cudaGetErrorString(e) + ")");
}

cudaError_t pool_alloc(tb_context* ctx, void** out, size_t bytes) {
    if (ctx->pool == nullptr) return cudaMalloc(out, bytes);
    return cudaMallocFromPoolAsync(out, bytes, ctx->pool, ctx->stream);
}

void pool_free(tb_context* ctx, void* p) {
    if (p == nullptr) return;
    if (ctx->pool == nullptr) cudaFree(p);
    else cudaFreeAsync(p, ctx->stream);
}

// The driver seam (crates/tachyon/src/cuda/driver.rs:138-167): the driver library is looked for at $TACHYON_LIBCUDA when that
// is set, else under its usual names; it must export cuDriverGetVersion and cuGetProcAddress_v2 and support CUDA 12.0.  The
// outcome is kept for the life of the process, as the reference keeps it.  The statically linked CUDA runtime then finds the
// same library (already loaded under its name); all this layer adds is the reference's search order and its clean errors.
static int driver_probe() {
    static std::once_flag once;
    static int outcome = OK;
    static std::string message;
    std::call_once(once, [] {
        const char* custom = getenv("TACHYON_LIBCUDA");
        const char* search[] = {"libcuda.so.1", "/usr/lib/wsl/lib/libcuda.so.1"};
        void* lib = nullptr;
        if (custom != nullptr && custom[0] != 0) {
            lib = dlopen(custom, RTLD_NOW | RTLD_GLOBAL);
        } else {
            for (const char* p : search)
                if ((lib = dlopen(p, RTLD_NOW | RTLD_GLOBAL)) != nullptr) break;
        }
        if (lib == nullptr || dlsym(lib, "cuDriverGetVersion") == nullptr) {
            outcome = NO_DRIVER;
            message = "the NVIDIA driver (libcuda.so.1) was not found; install it or set TACHYON_LIBCUDA to its path";  // error.rs:58
            return;
        }
        int version = 0;
        reinterpret_cast<int (*)(int*)>(dlsym(lib, "cuDriverGetVersion"))(&version);
        if (version < 12000 || dlsym(lib, "cuGetProcAddress_v2") == nullptr) {
            outcome = NO_DRIVER;
            message = "the NVIDIA driver supports CUDA " + std::to_string(version / 1000) + "." + std::to_string(version % 1000 / 10) +
                      "; tachyon needs 12.0 or newer (driver R525+)";  // error.rs:59 (Error::DriverTooOld)
        }
    });
    return outcome == OK ? OK : fail(outcome, message);
}

}  // namespace tb

using namespace tb;

struct tb_event {
    cudaEvent_t ev = nullptr;
};

extern "C" {

const char* tb_last_error(void) { return g_error.c_str(); }

int tb_devices(int* count) {
    if (count == nullptr) return fail(OUT_OF_RANGE, "tb_devices: null count");
    *count = 0;
    TB_TRY(driver_probe());
    TB_CUDA(cudaGetDeviceCount(count));
    return OK;
}

int tb_context_new(int gpu, tb_context** out) {
    if (out == nullptr) return fail(OUT_OF_RANGE, "tb_context_new: null out");
    *out = nullptr;
    TB_TRY(driver_probe());
    int count = 0;
    TB_CUDA(cudaGetDeviceCount(&count));
    if (gpu < 0 || gpu >= count) return fail(OUT_OF_RANGE, "tb_context_new: no such GPU");
    cudaDeviceProp prop;
    TB_CUDA(cudaGetDeviceProperties(&prop, gpu));
    if (prop.major != 10) return fail(UNSUPPORTED_GPU, std::string("tb_context_new: ") + prop.name + " is not an sm_100 device; this library has no other code path");
    TB_CUDA(cudaSetDevice(gpu));
    tb_context* ctx = new tb_context();
    ctx->gpu = gpu;
    ctx->sms = prop.multiProcessorCount;
    cudaError_t e = cudaStreamCreateWithFlags(&ctx->stream, cudaStreamNonBlocking);
    if (e == cudaSuccess) {
        // The pool the decoders' memory comes from: it never gives memory back by itself (tb_context_trim does).
        cudaMemPoolProps props = {};
        props.allocType = cudaMemAllocationTypePinned, props.handleTypes = cudaMemHandleTypeNone;
        props.location.type = cudaMemLocationTypeDevice, props.location.id = gpu;
        if (cudaMemPoolCreate(&ctx->pool, &props) == cudaSuccess) {
            uint64_t keep = UINT64_MAX;
            cudaMemPoolSetAttribute(ctx->pool, cudaMemPoolAttrReleaseThreshold, &keep);
        } else {
            ctx->pool = nullptr;  // no pools on this driver: plain allocations
            cudaGetLastError();
        }
    }
    if (e == cudaSuccess) e = cudaMalloc(&ctx->status, 256);
    if (e == cudaSuccess) e = cudaMemset(ctx->status, 0, 256);
    if (e == cudaSuccess) e = cudaHostAlloc(&ctx->status_host, 256, cudaHostAllocDefault);
    if (e == cudaSuccess) e = cudaMalloc(&ctx->sched, 64 * 2 * sizeof(uint32_t));
    if (e == cudaSuccess) e = cudaMemset(ctx->sched, 0, 64 * 2 * sizeof(uint32_t));
    if (e != cudaSuccess) {
        tb_context_free(ctx);
        return cuda_fail(e, "tb_context_new");
    }
    const char* env = getenv("TACHYON_B200_NO_OVERLAP");
    ctx->pdl = !(env != nullptr && env[0] == '1');
    env = getenv("TACHYON_B200_NO_PREFETCH");
    ctx->prefetch = !(env != nullptr && env[0] == '1');
    env = getenv("TACHYON_B200_STATIC");
    ctx->dynamic = !(env != nullptr && env[0] == '1');
    env = getenv("TACHYON_B200_NO_LEAN");
    ctx->lean = (env != nullptr && env[0] == '1') ? 0 : 1;
    env = getenv("TACHYON_B200_LATE_TRIGGER");
    ctx->early_trigger = !(env != nullptr && env[0] == '1');
    env = getenv("TACHYON_B200_LEAN_QKV");
    ctx->lean_qkv = env != nullptr && env[0] == '1';
    env = getenv("TACHYON_B200_L2_AHEAD");
    ctx->l2_ahead = env != nullptr ? (uint32_t)atoi(env) : 1u;  // one stage a block: measured 1 % of a decode step; two and more bring nothing
    env = getenv("TACHYON_B200_L2_NEXT");
    ctx->l2_next = env != nullptr ? (uint32_t)atoi(env) : 0u;
    env = getenv("TACHYON_B200_NO_CLUSTER");
    ctx->cluster = !(env != nullptr && env[0] == '1');
    env = getenv("TACHYON_B200_ATTN_BLOCK");
    ctx->attn_block = env != nullptr && env[0] == '1';
    env = getenv("TACHYON_B200_GEMM_WALK");
    ctx->gemm_walk = !(env != nullptr && env[0] == '0');
    env = getenv("TACHYON_B200_L2_SIDE");
    ctx->l2_side = env != nullptr && env[0] == '1';
    env = getenv("TACHYON_B200_GEMM_RED");
    ctx->gemm_red = !(env != nullptr && env[0] == '0');
    env = getenv("TACHYON_B200_FLASH");
    ctx->flash_tc = !(env != nullptr && env[0] == '0');
    env = getenv("TACHYON_B200_GEMM");
    ctx->gemm_schedule = env != nullptr ? atoi(env) : 0;
    *out = ctx;
    return OK;
}

void tb_context_free(tb_context* ctx) {
    if (ctx == nullptr) return;
    cudaSetDevice(ctx->gpu);
    if (ctx->stream) cudaStreamSynchronize(ctx->stream);
    if (ctx->pool) cudaMemPoolDestroy(ctx->pool);
    if (ctx->stream) cudaStreamDestroy(ctx->stream);
    if (ctx->status) cudaFree(ctx->status);
    if (ctx->sched) cudaFree(ctx->sched);
    if (ctx->status_host) cudaFreeHost(ctx->status_host);
    delete ctx;
}

int tb_context_sms(const tb_context* ctx) { return ctx ? ctx->sms : 0; }

int tb_context_set_overlap(tb_context* ctx, int on) {
    if (!ctx) return fail(OUT_OF_RANGE, "null context");
    ctx->pdl = on != 0;
    return OK;
}

int tb_context_set_gemm_schedule(tb_context* ctx, int which) {
    if (!ctx) return fail(OUT_OF_RANGE, "null context");
    if (which < 0 || which > 5) return fail(OUT_OF_RANGE, "tb_context_set_gemm_schedule: 0 (automatic) or 1..5");
    ctx->gemm_schedule = which;
    return OK;
}

int tb_context_set_lean(tb_context* ctx, int mode) {
    if (!ctx) return fail(OUT_OF_RANGE, "null context");
    if (mode < 0 || mode > 2) return fail(OUT_OF_RANGE, "tb_context_set_lean: 0, 1 or 2");
    ctx->lean = mode;
    return OK;
}

int tb_context_set_dynamic(tb_context* ctx, int on) {
    if (!ctx) return fail(OUT_OF_RANGE, "null context");
    ctx->dynamic = on != 0;
    return OK;
}

int tb_context_trim(tb_context* ctx) {
    if (!ctx) return fail(OUT_OF_RANGE, "null context");
    if (ctx->pool == nullptr) return OK;
    TB_CUDA(cudaSetDevice(ctx->gpu));
    TB_CUDA(cudaStreamSynchronize(ctx->stream));  // frees in the stream's order have to have happened
    TB_CUDA(cudaMemPoolTrimTo(ctx->pool, 0));
    return OK;
}

int tb_context_set_attn_block(tb_context* ctx, int on) {
    if (!ctx) return fail(OUT_OF_RANGE, "null context");
    if (on != 0 && on != 1) return fail(OUT_OF_RANGE, "tb_context_set_attn_block: 0 or 1");
    ctx->attn_block = on != 0;
    return OK;
}

int tb_context_memory(tb_context* ctx, size_t* free_bytes, size_t* total_bytes) {
    if (!ctx || !free_bytes || !total_bytes) return fail(OUT_OF_RANGE, "tb_context_memory: null argument");
    TB_CUDA(cudaSetDevice(ctx->gpu));
    TB_CUDA(cudaMemGetInfo(free_bytes, total_bytes));
    return OK;
}

int tb_context_set_flash(tb_context* ctx, int which) {
    if (!ctx) return fail(OUT_OF_RANGE, "null context");
    if (which != 0 && which != 1) return fail(OUT_OF_RANGE, "tb_context_set_flash: 0 (mma.sync kernel) or 1 (tcgen05 where the shape allows)");
    ctx->flash_tc = which != 0;
    return OK;
}

int tb_status(tb_context* ctx, uint32_t* word) {
    if (!ctx) return fail(OUT_OF_RANGE, "null context");
    TB_CUDA(cudaMemcpyAsync(ctx->status_host, ctx->status, 4, cudaMemcpyDeviceToHost, ctx->stream));
    TB_CUDA(cudaStreamSynchronize(ctx->stream));
    if (word) *word = *ctx->status_host;
    if (*ctx->status_host != 0) return fail(DEVICE_WAIT, "a kernel gave up a bounded wait (code " + std::to_string(*ctx->status_host) + ")");
    return OK;
}

int tb_alloc(tb_context* ctx, size_t bytes, void** dev) {
    if (!ctx || !dev) return fail(OUT_OF_RANGE, "tb_alloc: null argument");
    TB_CUDA(cudaSetDevice(ctx->gpu));
    TB_CUDA(cudaMalloc(dev, bytes ? bytes : 1));
    return OK;
}

int tb_free(tb_context* ctx, void* dev) {
    if (!ctx) return fail(OUT_OF_RANGE, "tb_free: null context");
    TB_CUDA(cudaStreamSynchronize(ctx->stream));
    TB_CUDA(cudaFree(dev));
    return OK;
}

int tb_alloc_host(tb_context* ctx, size_t bytes, void** host) {
    if (!ctx || !host) return fail(OUT_OF_RANGE, "tb_alloc_host: null argument");
    TB_CUDA(cudaSetDevice(ctx->gpu));
    TB_CUDA(cudaHostAlloc(host, bytes ? bytes : 1, cudaHostAllocMapped));
    return OK;
}

int tb_host_device_ptr(tb_context* ctx, void* host, void** dev) {
    if (!ctx || !host || !dev) return fail(OUT_OF_RANGE, "tb_host_device_ptr: null argument");
    TB_CUDA(cudaSetDevice(ctx->gpu));
    TB_CUDA(cudaHostGetDevicePointer(dev, host, 0));
    return OK;
}

int tb_free_host(tb_context* ctx, void* host) {
    if (!ctx) return fail(OUT_OF_RANGE, "tb_free_host: null context");
    TB_CUDA(cudaFreeHost(host));
    return OK;
}

int tb_upload(tb_context* ctx, void* dev, const void* host, size_t bytes) {
    if (!ctx || (bytes && (!dev || !host))) return fail(OUT_OF_RANGE, "tb_upload: null argument");
    TB_CUDA(cudaMemcpyAsync(dev, host, bytes, cudaMemcpyHostToDevice, ctx->stream));
    return OK;
}

int tb_download(tb_context* ctx, void* host, const void* dev, size_t bytes) {
    if (!ctx || (bytes && (!dev || !host))) return fail(OUT_OF_RANGE, "tb_download: null argument");
    TB_CUDA(cudaMemcpyAsync(host, dev, bytes, cudaMemcpyDeviceToHost, ctx->stream));
    return OK;
}

int tb_fill(tb_context* ctx, void* dev, int byte, size_t bytes) {
    if (!ctx || (bytes && !dev)) return fail(OUT_OF_RANGE, "tb_fill: null argument");
    TB_CUDA(cudaMemsetAsync(dev, byte, bytes, ctx->stream));
    return OK;
}

int tb_sync(tb_context* ctx) {
    if (!ctx) return fail(OUT_OF_RANGE, "null context");
    TB_CUDA(cudaStreamSynchronize(ctx->stream));
    return OK;
}

int tb_event_new(tb_context* ctx, tb_event** out) {
    if (!ctx || !out) return fail(OUT_OF_RANGE, "tb_event_new: null argument");
    tb_event* ev = new tb_event();
    cudaError_t e = cudaEventCreate(&ev->ev);
    if (e != cudaSuccess) {
        delete ev;
        return cuda_fail(e, "cudaEventCreate");
    }
    *out = ev;
    return OK;
}

void tb_event_free(tb_event* ev) {
    if (!ev) return;
    cudaEventDestroy(ev->ev);
    delete ev;
}

int tb_event_record(tb_context* ctx, tb_event* ev) {
    if (!ctx || !ev) return fail(OUT_OF_RANGE, "tb_event_record: null argument");
    TB_CUDA(cudaEventRecord(ev->ev, ctx->stream));
    return OK;
}

int tb_event_sync(tb_event* ev) {
    if (!ev) return fail(OUT_OF_RANGE, "tb_event_sync: null event");
    TB_CUDA(cudaEventSynchronize(ev->ev));
    return OK;
}

int tb_event_elapsed_ms(tb_event* start, tb_event* end, float* ms) {
    if (!start || !end || !ms) return fail(OUT_OF_RANGE, "tb_event_elapsed_ms: null argument");
    TB_CUDA(cudaEventElapsedTime(ms, start->ev, end->ev));
    return OK;
}

// ---- kernels ----------------------------------------------------------------------------------------------------

static int dtype_ok(int d) { return d == TB_F32 || d == TB_F16; }

int tb_gemv_q8(tb_context* ctx, const int8_t* w, const uint16_t* scales, const void* x, int x_dtype, void* y, int y_dtype, uint32_t rows, uint32_t cols) {
    if (!ctx) return fail(OUT_OF_RANGE, "null context");
    if (!dtype_ok(x_dtype) || !dtype_ok(y_dtype)) return fail(OUT_OF_RANGE, "tb_gemv_q8: unknown dtype");
    GemvParams p;
    p.w = w, p.s = reinterpret_cast<const __half*>(scales), p.rows = rows, p.cols = cols;
    p.xmode = x_dtype == TB_F16 ? X_F16 : X_F32, p.x = x;
    p.epi = y_dtype == TB_F16 ? EPI_F16 : EPI_F32, p.y = y;
    return launch_gemv(ctx, p);
}

int tb_quant_q8(tb_context* ctx, const float* x, uint32_t n, int8_t* q, float* pairs) {
    if (!ctx) return fail(OUT_OF_RANGE, "null context");
    return launch_quant_q8(ctx, x, q, pairs, n);
}

int tb_gemv_q4(tb_context* ctx, const uint8_t* packed, const uint16_t* scales, const int8_t* q, const float* pairs, float* y, uint32_t rows, uint32_t cols) {
    if (!ctx) return fail(OUT_OF_RANGE, "null context");
    return launch_gemv_q4(ctx, packed, scales, q, pairs, y, rows, cols);
}

int tb_geglu_q8(tb_context* ctx, const float* a, const float* b, uint32_t n, int8_t* q, float* pairs) {
    if (!ctx) return fail(OUT_OF_RANGE, "null context");
    return launch_geglu_q8(ctx, a, b, q, pairs, n);
}

int tb_norm_q8(tb_context* ctx, const float* h, float* h_out, const float* y, const float* w1, const float* w2, int8_t* q, float* pairs, uint32_t len,
               uint32_t chunks, float eps, float scale) {
    if (!ctx) return fail(OUT_OF_RANGE, "null context");
    return launch_norm_q8(ctx, h, h_out, y, w1, w2, q, pairs, len, chunks, eps, scale);
}

int tb_embed_q4(tb_context* ctx, const uint8_t* packed, const uint16_t* scales, const uint32_t* tokens, uint32_t rows, float* out, uint32_t cols, float scale) {
    if (!ctx) return fail(OUT_OF_RANGE, "null context");
    return launch_embed_q4_rows(ctx, packed, scales, tokens, rows, out, cols, scale);
}

// Stream::launch by kernel name (cuda/mod.rs:417-425, ptx/mod.rs:7-41): args[i] points at argument i's value, as the
// reference's `arg(&x)` and the driver's kernelParams do.
int tb_launch(tb_context* ctx, const char* kernel, const uint32_t grid[3], const uint32_t block[3], uint32_t shared_bytes, void* const* args, size_t nargs) {
    if (!ctx || !kernel || !grid || !block || (nargs && !args)) return fail(OUT_OF_RANGE, "tb_launch: null argument");
    const std::string name(kernel);
    auto ptr = [&](size_t i) { return reinterpret_cast<void*>(*static_cast<const uintptr_t*>(args[i])); };
    auto u32 = [&](size_t i) { return *static_cast<const uint32_t*>(args[i]); };
    auto f32 = [&](size_t i) { return *static_cast<const float*>(args[i]); };
    auto shape = [&](size_t want, uint32_t threads) -> int {
        if (nargs != want) return fail(OUT_OF_RANGE, "tb_launch: " + name + " takes " + std::to_string(want) + " arguments");
        if (block[0] != threads || block[1] != 1 || block[2] != 1) return fail(OUT_OF_RANGE, "tb_launch: " + name + " runs blocks of " + std::to_string(threads));
        if (shared_bytes != 0) return fail(OUT_OF_RANGE, "tb_launch: " + name + " takes no dynamic shared memory");
        return OK;
    };
    for (size_t i = 0; i < nargs; i++)
        if (!args[i]) return fail(OUT_OF_RANGE, "tb_launch: null argument slot");
    if (name == "quant_q8") {  // x, q, s, len
        TB_TRY(shape(4, 256));
        return launch_quant_q8(ctx, static_cast<const float*>(ptr(0)), static_cast<int8_t*>(ptr(1)), static_cast<float*>(ptr(2)), u32(3));
    }
    if (name == "geglu_q8") {  // a, b, q, s, len
        TB_TRY(shape(5, 256));
        return launch_geglu_q8(ctx, static_cast<const float*>(ptr(0)), static_cast<const float*>(ptr(1)), static_cast<int8_t*>(ptr(2)), static_cast<float*>(ptr(3)), u32(4));
    }
    if (name == "norm_q8") {  // h, h_out, y, w1, w2, q, s, len, eps, scale; grid (len / 256, chunks)
        TB_TRY(shape(10, 256));
        if (grid[0] != u32(7) / 256) return fail(OUT_OF_RANGE, "tb_launch: norm_q8 runs len / 256 blocks per chunk");
        return launch_norm_q8(ctx, static_cast<const float*>(ptr(0)), static_cast<float*>(ptr(1)), static_cast<const float*>(ptr(2)), static_cast<const float*>(ptr(3)),
                              static_cast<const float*>(ptr(4)), static_cast<int8_t*>(ptr(5)), static_cast<float*>(ptr(6)), u32(7), grid[1], f32(8), f32(9));
    }
    if (name == "quant_q8p") {  // x, q, s, len (ptx/mod.rs:253-287); grid len / 256 (rounded up) blocks of 256
        TB_TRY(shape(4, 256));
        return launch_quant_q8p(ctx, static_cast<const float*>(ptr(0)), static_cast<int8_t*>(ptr(1)), static_cast<float*>(ptr(2)), u32(3));
    }
    if (name == "geglu_q8p") {  // a, b, q, s, len, width, sa, sb, so: value i is row i / width, read at strides sa, sb, stored at stride so
        TB_TRY(shape(9, 256));
        return launch_geglu_q8p(ctx, static_cast<const float*>(ptr(0)), static_cast<const float*>(ptr(1)), static_cast<int8_t*>(ptr(2)), static_cast<float*>(ptr(3)),
                                u32(4), u32(5), u32(6), u32(7), u32(8));
    }
    if (name == "norm_q8p") {  // norm_q8's arguments; grid (len / 256, tokens)
        TB_TRY(shape(10, 256));
        if (grid[0] != u32(7) / 256) return fail(OUT_OF_RANGE, "tb_launch: norm_q8p runs len / 256 blocks per token");
        return launch_norm_q8p(ctx, static_cast<const float*>(ptr(0)), static_cast<float*>(ptr(1)), static_cast<const float*>(ptr(2)), static_cast<const float*>(ptr(3)),
                               static_cast<const float*>(ptr(4)), static_cast<int8_t*>(ptr(5)), static_cast<float*>(ptr(6)), u32(7), grid[1], f32(8), f32(9));
    }
    if (name == "gemm_q4") {
        // ptx/gemm.rs:18-23: w, ws, q, s (Q8P), y, rows, cols, tokens; grid (tokens / 128 rounded up, rows / 64, slices).  Only the
        // number of slices is taken from the grid: this build tiles the tokens and rows its own way.
        if (nargs != 8) return fail(OUT_OF_RANGE, "tb_launch: gemm_q4 takes 8 arguments");
        return launch_gemm_q4_ref(ctx, static_cast<const uint8_t*>(ptr(0)), static_cast<const uint16_t*>(ptr(1)), static_cast<const int8_t*>(ptr(2)),
                                  static_cast<const float*>(ptr(3)), static_cast<float*>(ptr(4)), u32(5), u32(6), u32(7), grid[2]);
    }
    if (name == "sum_slices") {  // y, len, slices (ptx/gemm.rs:31-34)
        TB_TRY(shape(3, 256));
        return launch_sum_slices(ctx, static_cast<float*>(ptr(0)), u32(1), u32(2));
    }
    if (name == "embed_q4") {  // packed, scales, token, out, cols, scale; grid (cols / 256, rows)
        TB_TRY(shape(6, 256));
        return launch_embed_q4_rows(ctx, static_cast<const uint8_t*>(ptr(0)), static_cast<const uint16_t*>(ptr(1)), static_cast<const uint32_t*>(ptr(2)), grid[1],
                                    static_cast<float*>(ptr(3)), u32(4), f32(5));
    }
    if (name == "gemv_q4") {  // w, ws, q, s, y, rows, cols; this build chooses its own grid
        if (nargs != 7) return fail(OUT_OF_RANGE, "tb_launch: gemv_q4 takes 7 arguments");
        return launch_gemv_q4(ctx, static_cast<const uint8_t*>(ptr(0)), static_cast<const uint16_t*>(ptr(1)), static_cast<const int8_t*>(ptr(2)),
                              static_cast<const float*>(ptr(3)), static_cast<float*>(ptr(4)), u32(5), u32(6));
    }
    if (name == "gemv_q4_narrow") {  // gemv_q4's arguments, rows of at most 256 weights; rows / 16 (rounded up) blocks of 128 (gemv.rs:7-9)
        TB_TRY(shape(7, 128));
        if (grid[0] != (u32(5) + 15) / 16) return fail(OUT_OF_RANGE, "tb_launch: gemv_q4_narrow runs rows / 16 (rounded up) blocks");
        return launch_gemv_q4_narrow(ctx, static_cast<const uint8_t*>(ptr(0)), static_cast<const uint16_t*>(ptr(1)), static_cast<const int8_t*>(ptr(2)),
                                     static_cast<const float*>(ptr(3)), static_cast<float*>(ptr(4)), u32(5), u32(6));
    }
    if (name == "sample") {  // logits, work, vocab, cfg, state, seen, out, partial, count; grid[0] blocks of 1024
        TB_TRY(shape(9, 1024));
        return launch_sample_draw(ctx, static_cast<const float*>(ptr(0)), static_cast<float*>(ptr(1)), u32(2), ptr(3), static_cast<uint32_t*>(ptr(4)),
                                  static_cast<uint32_t*>(ptr(5)), static_cast<uint32_t*>(ptr(6)), static_cast<float*>(ptr(7)), static_cast<uint32_t*>(ptr(8)), grid[0]);
    }
    if (name == "attend_256" || name == "attend_256_2") {
        // attend.rs:21-32: qkv, qn, kn, freq, k_cache, v_cache, pos, cap, window, fresh, group, partial, count, Q8 out (q, s);
        // grid (H / per, S) blocks of 256, per = 4 query heads a block (2 for attend_256_2), `group` blocks per key-value head.
        TB_TRY(shape(15, 256));
        const uint32_t per = name == "attend_256" ? 4u : 2u, group = u32(10);
        if (group != 1 && !(group == 2 && per == 4)) return fail(UNSUPPORTED, "tb_launch: " + name + " with that many blocks per key-value head has no kernel here");
        if (grid[0] % group != 0) return fail(OUT_OF_RANGE, "tb_launch: " + name + " runs `group` blocks per key-value head");
        AttendParams a;
        a.qkv = static_cast<const float*>(ptr(0)), a.q_norm = static_cast<const float*>(ptr(1)), a.k_norm = static_cast<const float*>(ptr(2));
        a.freq = static_cast<const float*>(ptr(3)), a.kc = static_cast<__half*>(ptr(4)), a.vc = static_cast<__half*>(ptr(5));
        a.pos = static_cast<const uint32_t*>(ptr(6)), a.cap = u32(7), a.window = u32(8), a.fresh = u32(9);
        a.kv_heads = grid[0] / group, a.heads = per * grid[0], a.splits = grid[1], a.scale = 1.0f, a.eps = 1e-6f;
        a.partial = static_cast<float*>(ptr(11)), a.count = static_cast<uint32_t*>(ptr(12));
        a.out = ptr(13), a.out_pairs = static_cast<float*>(ptr(14)), a.out_f16 = 2;
        if (!a.q_norm || !a.k_norm || !a.out || !a.out_pairs) return fail(OUT_OF_RANGE, "tb_launch: " + name + " needs its norm weights and its Q8 output");
        return group == 2 ? launch_attend_256_shared(ctx, a) : launch_attend(ctx, a);  // eight query heads to a key-value head: E2B
    }
    if (name == "attend_512") {
        // attend.rs:21-32 at head size 512: grid (H / 4, S), four query heads a block, `group` blocks per key-value head.
        TB_TRY(shape(15, 256));
        const uint32_t group = u32(10);
        if (group != 1 && group != 2) return fail(UNSUPPORTED, "tb_launch: attend_512 with more than two blocks per key-value head has no kernel here");
        if (grid[0] % group != 0) return fail(OUT_OF_RANGE, "tb_launch: attend_512 runs `group` blocks per key-value head");
        AttendParams a;
        a.qkv = static_cast<const float*>(ptr(0)), a.q_norm = static_cast<const float*>(ptr(1)), a.k_norm = static_cast<const float*>(ptr(2));
        a.freq = static_cast<const float*>(ptr(3)), a.kc = static_cast<__half*>(ptr(4)), a.vc = static_cast<__half*>(ptr(5));
        a.pos = static_cast<const uint32_t*>(ptr(6)), a.cap = u32(7), a.window = u32(8), a.fresh = u32(9);
        a.kv_heads = grid[0] / group, a.heads = 4 * grid[0], a.splits = grid[1], a.scale = 1.0f, a.eps = 1e-6f;
        a.partial = static_cast<float*>(ptr(11)), a.count = static_cast<uint32_t*>(ptr(12));
        a.out = ptr(13), a.out_pairs = static_cast<float*>(ptr(14)), a.out_f16 = 2;
        if (!a.q_norm || !a.k_norm || !a.out || !a.out_pairs) return fail(OUT_OF_RANGE, "tb_launch: attend_512 needs its norm weights and its Q8 output");
        return launch_attend_512(ctx, a);
    }
    const bool wide = name.size() > 4 && name.compare(name.size() - 4, 4, "_512") == 0;  // heads of 512
    if (name == "kv_256" || name == "kv_512") {
        // attend.rs:472-511: qkv, kn, freq, k_cache, v_cache, pos, cap, ratio; grid (Hkv, tokens) blocks of 32.
        TB_TRY(shape(8, 32));
        const uint32_t kv = grid[0], tokens = grid[1], ratio = u32(7), d = wide ? 512u : 256u;
        PrefillRows rows;
        rows.first = ratio * kv, rows.count = 2 * kv, rows.stride = (ratio + 2) * kv * d, rows.pos = static_cast<const uint32_t*>(ptr(5));
        if (!ptr(0) || !ptr(1) || !ptr(2) || !ptr(3) || !ptr(4) || !rows.pos || kv == 0 || tokens == 0 || ratio == 0 || u32(6) == 0)
            return fail(OUT_OF_RANGE, "tb_launch: " + name + ": null or empty argument");
        return launch_prefill_rows(ctx, static_cast<const float*>(ptr(0)), nullptr, static_cast<const float*>(ptr(1)), static_cast<const float*>(ptr(2)), nullptr,
                                   static_cast<__half*>(ptr(3)), static_cast<__half*>(ptr(4)), tokens, 0, u32(6), ratio * kv, kv, 1e-6f, 1.0f, d, rows);
    }
    if (name == "query_256" || name == "query_512") {
        // attend.rs:514-556: qkv, qn, freq, out, pos, row (floats per token of qkv); grid (H, tokens) blocks of 32.
        TB_TRY(shape(6, 32));
        const uint32_t heads = grid[0], tokens = grid[1], d = wide ? 512u : 256u;
        PrefillRows rows;
        rows.first = 0, rows.count = heads, rows.stride = u32(5), rows.pos = static_cast<const uint32_t*>(ptr(4));
        if (!ptr(0) || !ptr(1) || !ptr(2) || !ptr(3) || !rows.pos || heads == 0 || tokens == 0 || rows.stride < heads * d)
            return fail(OUT_OF_RANGE, "tb_launch: " + name + ": null, empty or short argument");
        // kv_heads 0: no row is a key or a value; cap 1 is not used.  The queries are stored as they are (scale 1, no log2 e).
        return launch_prefill_rows(ctx, static_cast<const float*>(ptr(0)), static_cast<const float*>(ptr(1)), nullptr, static_cast<const float*>(ptr(2)),
                                   static_cast<__half*>(ptr(3)), nullptr, nullptr, tokens, 0, 1, heads, 0, 1e-6f, 1.0f, d, rows);
    }
    if (name == "flash_256" || name == "flash_256_2" || name == "flash_512") {
        // flash.rs:19-22: q, k_cache, v_cache, pos, cap, window, group, tokens, y (f32); grid (tiles of tokens, H / P).  This build
        // chooses its own tiles, block and shared memory: grid[0], block and shared_bytes are not used.
        if (nargs != 9) return fail(OUT_OF_RANGE, "tb_launch: " + name + " takes 9 arguments");
        const uint32_t per = name == "flash_256_2" ? 2u : 4u, group = u32(6), heads = per * grid[1], tokens = u32(7), d = wide ? 512u : 256u;
        if (!ptr(0) || !ptr(1) || !ptr(2) || !ptr(3) || !ptr(8) || group == 0 || grid[1] % group != 0 || tokens == 0 || u32(4) == 0 || u32(5) == 0)
            return fail(OUT_OF_RANGE, "tb_launch: " + name + ": null, empty or ragged argument");
        return launch_prefill_flash(ctx, static_cast<const __half*>(ptr(0)), static_cast<const __half*>(ptr(1)), static_cast<const __half*>(ptr(2)), ptr(8), tokens, 0,
                                    u32(4), u32(5), heads, grid[1] / group, d, static_cast<const uint32_t*>(ptr(3)), 1.4426950408889634f, 1);
    }
    // ---- the encoder's kernels (ptx/encoder.rs:5-38) ----
    if (name == "quant_f16") {  // a (f16 rows), q, scales, cols; grid (cols / 64 / 8 rounded up, tokens)
        TB_TRY(shape(4, 256));
        return launch_quant_f16(ctx, static_cast<const __half*>(ptr(0)), static_cast<int8_t*>(ptr(1)), static_cast<float*>(ptr(2)), u32(3), grid[1]);
    }
    if (name == "norm_f16") {  // x, gamma, beta (or 0), a, xo (or 0), h, eps; one block a row, of any size: this build runs 256 threads
        if (nargs != 7) return fail(OUT_OF_RANGE, "tb_launch: norm_f16 takes 7 arguments");
        return launch_norm_f16(ctx, static_cast<const float*>(ptr(0)), static_cast<const float*>(ptr(1)), static_cast<const float*>(ptr(2)), static_cast<__half*>(ptr(3)),
                               static_cast<float*>(ptr(4)), u32(5), f32(6), grid[0]);
    }
    if (name == "embed_f16" || name == "add_rows" || name == "add_rows_f16" || name == "gather_rows") {  // table, idx, out, h; grid (h / 256 rounded up, n)
        TB_TRY(shape(4, 256));
        if (grid[0] != (u32(3) + 255) / 256) return fail(OUT_OF_RANGE, "tb_launch: " + name + " runs h / 256 (rounded up) blocks a row");
        const int kind = name == "embed_f16" ? 0 : name == "add_rows" ? 1 : name == "add_rows_f16" ? 2 : 3;
        return launch_rows(ctx, kind, ptr(0), static_cast<const uint32_t*>(ptr(1)), static_cast<float*>(ptr(2)), u32(3), grid[1]);
    }
    if (name == "gelu_f16") {  // x, out, width, len, gated
        TB_TRY(shape(5, 256));
        return launch_gelu_f16(ctx, static_cast<const float*>(ptr(0)), static_cast<__half*>(ptr(1)), u32(2), u32(3), u32(4));
    }
    if (name == "rope_f16") {  // qkv, table, pos, h, d; grid (h / 2 / 256 rounded up, n)
        TB_TRY(shape(5, 256));
        return launch_rope_f16(ctx, static_cast<__half*>(ptr(0)), static_cast<const float*>(ptr(1)), static_cast<const uint32_t*>(ptr(2)), u32(3), u32(4), grid[1]);
    }
    if (name == "attend_f16" || name == "attend_f16_32") {  // qkv, out, tiles, h, window (0: all), scale; grid (tiles, h / d) blocks of 128
        TB_TRY(shape(6, 128));
        const uint32_t d = name == "attend_f16" ? 64u : 32u, h = u32(3), window = u32(4);
        if (h == 0 || h % d != 0 || grid[1] != h / d) return fail(OUT_OF_RANGE, "tb_launch: " + name + " runs a block per tile and head");
        return launch_enc_attend(ctx, static_cast<const __half*>(ptr(0)), static_cast<const uint32_t*>(ptr(2)), static_cast<__half*>(ptr(1)), h, d,
                                 window == 0 ? -1 : (int)window, f32(5), grid[0]);
    }
    if (name == "gemm_f16" || name == "gemm_f16_128" || name == "gemm_f16_tall" || name == "gemm_q8" || name == "gemm_q8_128" || name == "gemm_q8_tall") {
        // a, w, bias (or 0), y, rows, cols, tokens, mode; the 8-bit ones also a's and w's scales.  The three names of each are
        // the reference's three block shapes of one product; here one kernel each, which tiles its own way: grid and block
        // are not used.
        const bool q8 = name.compare(0, 7, "gemm_q8") == 0;
        if (nargs != (q8 ? 10u : 8u)) return fail(OUT_OF_RANGE, "tb_launch: " + name + " takes " + (q8 ? "10" : "8") + " arguments");
        const uint32_t rows = u32(4), cols = u32(5), tokens = u32(6), mode = u32(7);
        if (mode > 5) return fail(OUT_OF_RANGE, "tb_launch: " + name + " has modes 0 to 5");
        if (rows % 64 != 0 || cols % 64 != 0) return fail(OUT_OF_RANGE, "tb_launch: " + name + " takes rows and cols in multiples of 64");
        if (q8) return launch_gemm_q8e(ctx, static_cast<const int8_t*>(ptr(0)), static_cast<const int8_t*>(ptr(1)), static_cast<const float*>(ptr(2)), ptr(3), rows, cols,
                                       tokens, mode, static_cast<const float*>(ptr(8)), static_cast<const float*>(ptr(9)));
        static const int store[6] = {TB_GEMM_F32, TB_GEMM_ADD, TB_GEMM_F16, TB_GEMM_RELU, TB_GEMM_GEGLU_ERF, TB_GEMM_GATED_SILU};
        return launch_gemm_q8(ctx, static_cast<const int8_t*>(ptr(1)), nullptr, static_cast<const __half*>(ptr(0)), tokens, rows, cols, ptr(3), store[mode], 16, nullptr, 0,
                              static_cast<const float*>(ptr(2)));
    }
    return fail(NO_MODEL, "tb_launch: no kernel named " + name);
}

int tb_gemv_q4x(tb_context* ctx, const uint8_t* packed, const uint16_t* scales, const void* x, int x_dtype, float* y, uint32_t rows, uint32_t cols) {
    if (!ctx) return fail(OUT_OF_RANGE, "null context");
    if (!dtype_ok(x_dtype)) return fail(OUT_OF_RANGE, "tb_gemv_q4x: unknown dtype");
    GemvParams p;
    p.w = reinterpret_cast<const int8_t*>(packed), p.s = reinterpret_cast<const __half*>(scales), p.rows = rows, p.cols = cols, p.wbits = 4;
    p.xmode = x_dtype == TB_F16 ? X_F16 : X_F32, p.x = x;
    p.epi = EPI_F32, p.y = y;
    return launch_gemv(ctx, p);
}

int tb_sample(tb_context* ctx, const float* logits, float* work, uint32_t vocab, const tb_sampling* cfg, uint32_t* state, uint32_t* seen, uint32_t* out,
              void* partial, uint32_t* count, uint32_t blocks) {
    if (!ctx) return fail(OUT_OF_RANGE, "null context");
    return launch_sample_draw(ctx, logits, work, vocab, cfg, state, seen, out, static_cast<float*>(partial), count, blocks);
}

int tb_gemv_q8_norm(tb_context* ctx, const int8_t* w, const uint16_t* scales, const float* h, const float* y_res, const float* w1, const float* w2, float eps,
                    float hscale, float* h_out, float* y, uint32_t rows, uint32_t cols, int geglu) {
    if (!ctx) return fail(OUT_OF_RANGE, "null context");
    GemvParams p;
    p.w = w, p.s = reinterpret_cast<const __half*>(scales), p.rows = rows, p.cols = cols;
    p.xmode = X_NORM, p.h = h, p.yres = y_res, p.w1 = w1, p.w2 = w2, p.eps = eps, p.hscale = hscale, p.h_out = h_out;
    p.epi = geglu ? EPI_GEGLU : EPI_F32, p.y = y;
    return launch_gemv(ctx, p);
}

int tb_selftest_wait(tb_context* ctx, uint64_t limit_ns) {
    if (!ctx) return fail(OUT_OF_RANGE, "tb_selftest_wait: null context");
    if (limit_ns == 0 || limit_ns > 100000000ull) return fail(OUT_OF_RANGE, "tb_selftest_wait: a limit between 1 ns and 100 ms");
    // Two rows of 2048 columns: one block, whose producer is told to post nothing.
    const uint32_t rows = 2, cols = 2048;
    char* buf = nullptr;
    TB_CUDA(cudaSetDevice(ctx->gpu));
    TB_CUDA(cudaMalloc(&buf, rows * cols + 4096 + cols * 4 + 256));
    cudaError_t e = cudaMemsetAsync(buf, 0, rows * cols + 4096 + cols * 4 + 256, ctx->stream);
    int st = OK;
    if (e == cudaSuccess) {
        GemvParams p;
        p.w = reinterpret_cast<const int8_t*>(buf), p.s = reinterpret_cast<const __half*>(buf + rows * cols), p.rows = rows, p.cols = cols;
        p.xmode = X_F32, p.x = buf + rows * cols + 4096, p.epi = EPI_F32, p.y = buf + rows * cols + 4096 + cols * 4;
        p.silent = 1, p.wait_ns = limit_ns;
        st = launch_gemv(ctx, p);
    }
    if (e == cudaSuccess) e = cudaStreamSynchronize(ctx->stream);
    cudaFree(buf);
    if (e != cudaSuccess) return cuda_fail(e, "tb_selftest_wait");
    return st;
}

int tb_status_clear(tb_context* ctx) {
    if (!ctx) return fail(OUT_OF_RANGE, "null context");
    TB_CUDA(cudaMemsetAsync(ctx->status, 0, 4, ctx->stream));
    TB_CUDA(cudaStreamSynchronize(ctx->stream));
    return OK;
}

int tb_gemv_f16(tb_context* ctx, const uint16_t* w, const void* x, int x_dtype, void* y, int y_dtype, uint32_t rows, uint32_t cols) {
    if (!ctx) return fail(OUT_OF_RANGE, "tb_gemv_f16: null context");
    if (!dtype_ok(x_dtype) || !dtype_ok(y_dtype)) return fail(OUT_OF_RANGE, "tb_gemv_f16: unknown dtype");
    GemvF16Params p;
    p.w = reinterpret_cast<const __half*>(w), p.rows = rows, p.cols = cols;
    p.xmode = x_dtype == TB_F16 ? X_F16 : X_F32, p.x = x;
    p.epi = y_dtype == TB_F16 ? EPI_F16 : EPI_F32, p.y = y;
    return launch_gemv_f16(ctx, p);
}

int tb_gemv_f16_norm(tb_context* ctx, const uint16_t* w, const float* h, const float* y_res, const float* w1, const float* w2, float eps, float hscale,
                     float* h_out, void* y, int y_dtype, uint32_t rows, uint32_t cols) {
    if (!ctx) return fail(OUT_OF_RANGE, "tb_gemv_f16_norm: null context");
    if (!dtype_ok(y_dtype)) return fail(OUT_OF_RANGE, "tb_gemv_f16_norm: unknown dtype");
    GemvF16Params p;
    p.w = reinterpret_cast<const __half*>(w), p.rows = rows, p.cols = cols;
    p.xmode = X_NORM, p.h = h, p.yres = y_res, p.w1 = w1, p.w2 = w2, p.eps = eps, p.hscale = hscale, p.h_out = h_out;
    p.epi = y_dtype == TB_F16 ? EPI_F16 : EPI_F32, p.y = y;
    return launch_gemv_f16(ctx, p);
}

int tb_gemv_q8_argmax(tb_context* ctx, const int8_t* w, const uint16_t* scales, const void* x, int x_dtype, float* logits, uint32_t rows, uint32_t cols,
                      void* scratch, uint32_t* state, uint32_t* token_out) {
    if (!ctx) return fail(OUT_OF_RANGE, "null context");
    if (!dtype_ok(x_dtype) || !scratch || (reinterpret_cast<uintptr_t>(scratch) & 7)) return fail(OUT_OF_RANGE, "tb_gemv_q8_argmax: bad dtype or scratch");
    GemvParams p;
    p.w = w, p.s = reinterpret_cast<const __half*>(scales), p.rows = rows, p.cols = cols;
    p.xmode = x_dtype == TB_F16 ? X_F16 : X_F32, p.x = x;
    p.epi = EPI_ARGMAX, p.y = logits;
    p.best = static_cast<unsigned long long*>(scratch), p.count = reinterpret_cast<uint32_t*>(static_cast<char*>(scratch) + 8);
    p.state = state, p.token_out = token_out;
    return launch_gemv(ctx, p);
}

int tb_gemm_q8(tb_context* ctx, const int8_t* w, const uint16_t* scales, const uint16_t* a, uint32_t m, uint32_t n, uint32_t k, void* out, int mode) {
    if (!ctx) return fail(OUT_OF_RANGE, "null context");
    return launch_gemm_q8(ctx, w, reinterpret_cast<const __half*>(scales), reinterpret_cast<const __half*>(a), m, n, k, out, mode);
}

int tb_gemm_q4(tb_context* ctx, const uint8_t* packed, const uint16_t* scales, const uint16_t* a, uint32_t m, uint32_t n, uint32_t k, void* out, int mode) {
    if (!ctx) return fail(OUT_OF_RANGE, "null context");
    return launch_gemm_q8(ctx, reinterpret_cast<const int8_t*>(packed), reinterpret_cast<const __half*>(scales), reinterpret_cast<const __half*>(a), m, n, k, out, mode, 4);
}

int tb_gemm_f16(tb_context* ctx, const uint16_t* w, const uint16_t* a, uint32_t m, uint32_t n, uint32_t k, void* out, int mode) {
    if (!ctx) return fail(OUT_OF_RANGE, "null context");
    if (mode == 6) return fail(OUT_OF_RANGE, "tb_gemm_f16: unknown output mode");
    return launch_gemm_q8(ctx, reinterpret_cast<const int8_t*>(w), nullptr, reinterpret_cast<const __half*>(a), m, n, k, out, mode, 16);
}

int tb_dequant_f16(tb_context* ctx, const void* w, const uint16_t* scales, uint32_t rows, uint32_t cols, uint32_t bits, uint16_t* out) {
    if (!ctx) return fail(OUT_OF_RANGE, "null context");
    return launch_dequant_f16(ctx, static_cast<const int8_t*>(w), reinterpret_cast<const __half*>(scales), rows, cols, bits, reinterpret_cast<__half*>(out));
}

int tb_norm(tb_context* ctx, const float* h, const float* y_res, const float* w1, const float* w2, uint32_t n, float eps, float hscale, float* h_out,
            float* x_out) {
    if (!ctx) return fail(OUT_OF_RANGE, "null context");
    return launch_norm(ctx, h, y_res, w1, w2, n, eps, hscale, h_out, x_out);
}

int tb_prefill_norm(tb_context* ctx, float* h, const float* y, const float* w1, const float* w2, uint32_t tokens, uint32_t n, float eps, float hscale, uint16_t* x) {
    if (!ctx) return fail(OUT_OF_RANGE, "null context");
    if (!h || !x || tokens == 0 || (y != nullptr && w1 == nullptr)) return fail(OUT_OF_RANGE, "tb_prefill_norm: null or empty argument");
    return launch_prefill_norm(ctx, h, y, w1, w2, tokens, n, eps, hscale, reinterpret_cast<__half*>(x));
}

int tb_embed_q8(tb_context* ctx, const int8_t* w, const uint16_t* scales, const uint32_t* token, uint32_t cols, float scale, float* out) {
    if (!ctx) return fail(OUT_OF_RANGE, "null context");
    return launch_embed_q8(ctx, w, reinterpret_cast<const __half*>(scales), token, cols, scale, out);
}

int tb_prefill_attend(tb_context* ctx, const uint16_t* q, const uint16_t* k_cache, const uint16_t* v_cache, uint16_t* out, uint32_t tokens, uint32_t pos0,
                      uint32_t cap, uint32_t window, uint32_t heads, uint32_t kv_heads, uint32_t head_dim) {
    if (!ctx || !q || !k_cache || !v_cache || !out) return fail(OUT_OF_RANGE, "tb_prefill_attend: null argument");
    if (tokens == 0 || cap == 0 || window == 0 || kv_heads == 0 || heads % kv_heads != 0) return fail(OUT_OF_RANGE, "tb_prefill_attend: empty or ragged shape");
    if ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k_cache) | reinterpret_cast<uintptr_t>(v_cache) | reinterpret_cast<uintptr_t>(out)) & 15)
        return fail(OUT_OF_RANGE, "tb_prefill_attend: buffers must be 16-byte aligned");
    return launch_prefill_flash(ctx, reinterpret_cast<const __half*>(q), reinterpret_cast<const __half*>(k_cache), reinterpret_cast<const __half*>(v_cache),
                                reinterpret_cast<__half*>(out), tokens, pos0, cap, window, heads, kv_heads, head_dim);
}

int tb_prefill_qkv(tb_context* ctx, const float* qkv, const float* q_norm, const float* k_norm, const float* freq, uint16_t* q_out, uint16_t* k_cache,
                   uint16_t* v_cache, uint32_t tokens, uint32_t pos0, uint32_t cap, uint32_t heads, uint32_t kv_heads, float eps, float scale, uint32_t head_dim) {
    if (!ctx || !qkv || !q_norm || !freq || !q_out) return fail(OUT_OF_RANGE, "tb_prefill_qkv: null argument");
    if (kv_heads != 0 && (!k_norm || !k_cache || !v_cache)) return fail(OUT_OF_RANGE, "tb_prefill_qkv: keys and values need their norm weights and caches");
    if (tokens == 0 || cap == 0 || heads == 0) return fail(OUT_OF_RANGE, "tb_prefill_qkv: empty shape");
    return launch_prefill_qkv(ctx, qkv, q_norm, k_norm, freq, reinterpret_cast<__half*>(q_out), reinterpret_cast<__half*>(k_cache), reinterpret_cast<__half*>(v_cache),
                              tokens, pos0, cap, heads, kv_heads, eps, scale, head_dim);
}

size_t tb_attend_scratch_bytes(uint32_t heads, uint32_t kv_heads, uint32_t splits) {
    if (kv_heads == 0) return 0;
    return attend_partial_floats(heads, kv_heads, splits) * sizeof(float);
}

int tb_attend_decode(tb_context* ctx, const tb_attend* a) {
    if (!ctx || !a) return fail(OUT_OF_RANGE, "tb_attend_decode: null argument");
    if (!dtype_ok(a->out_dtype)) return fail(OUT_OF_RANGE, "tb_attend_decode: unknown dtype");
    AttendParams p;
    p.qkv = a->qkv, p.q_norm = a->q_norm, p.k_norm = a->k_norm, p.freq = a->freq;
    p.kc = reinterpret_cast<__half*>(a->k_cache), p.vc = reinterpret_cast<__half*>(a->v_cache);
    p.pos = a->pos, p.cap = a->cap, p.window = a->window, p.fresh = a->fresh, p.heads = a->heads, p.kv_heads = a->kv_heads;
    p.scale = a->scale, p.eps = a->eps, p.partial = a->partial, p.count = a->count, p.splits = a->splits;
    p.out = a->out, p.out_f16 = a->out_dtype == TB_F16;
    if (a->kv_heads != 0 && a->heads == 8 * a->kv_heads) return launch_attend_256_shared(ctx, p);  // two blocks of four heads per key-value head
    return launch_attend(ctx, p);
}

int tb_attend_project(tb_context* ctx, const tb_attend* a, uint32_t cluster, const int8_t* w, const uint16_t* scales, uint32_t rows, float* y) {
    if (!ctx || !a || !w || !scales || !y) return fail(OUT_OF_RANGE, "tb_attend_project: null argument");
    if (a->kv_heads == 0 || a->heads * 256 != 2048) return fail(UNSUPPORTED, "tb_attend_project: heads * 256 must be 2048");
    AttendParams p;
    p.qkv = a->qkv, p.q_norm = a->q_norm, p.k_norm = a->k_norm, p.freq = a->freq;
    p.kc = reinterpret_cast<__half*>(a->k_cache), p.vc = reinterpret_cast<__half*>(a->v_cache);
    p.pos = a->pos, p.cap = a->cap, p.window = a->window, p.fresh = a->fresh, p.heads = a->heads, p.kv_heads = a->kv_heads;
    p.scale = a->scale, p.eps = a->eps, p.partial = a->partial, p.splits = a->splits;
    p.defer = 1, p.cluster = cluster;
    TB_TRY(launch_attend(ctx, p));
    GemvParams g;
    g.w = w, g.s = reinterpret_cast<const __half*>(scales), g.rows = rows, g.cols = 2048;
    g.xmode = X_ATTN, g.att_partial = a->partial, g.att_pos = a->pos, g.att_splits = a->splits, g.att_window = a->window;
    g.att_heads = a->heads, g.att_kv = a->kv_heads, g.att_cluster = cluster;
    g.epi = EPI_F32, g.y = y, g.lean = 1;
    return launch_gemv(ctx, g);
}

size_t tb_attend_512_scratch_bytes(uint32_t heads, uint32_t splits) { return (size_t)heads * splits * (2 + 512) * sizeof(float); }

int tb_attend_decode_512(tb_context* ctx, const tb_attend* a) {
    if (!ctx || !a) return fail(OUT_OF_RANGE, "tb_attend_decode_512: null argument");
    if (!dtype_ok(a->out_dtype)) return fail(OUT_OF_RANGE, "tb_attend_decode_512: unknown dtype");
    AttendParams p;
    p.qkv = a->qkv, p.q_norm = a->q_norm, p.k_norm = a->k_norm, p.freq = a->freq;
    p.kc = reinterpret_cast<__half*>(a->k_cache), p.vc = reinterpret_cast<__half*>(a->v_cache);
    p.pos = a->pos, p.cap = a->cap, p.window = a->window, p.fresh = a->fresh, p.heads = a->heads, p.kv_heads = a->kv_heads;
    p.scale = a->scale, p.eps = a->eps, p.partial = a->partial, p.count = a->count, p.splits = a->splits;
    p.out = a->out, p.out_f16 = a->out_dtype == TB_F16;
    return launch_attend_512(ctx, p);
}

int tb_attend_decode_static(tb_context* ctx, const tb_attend* a) {
    if (!ctx || !a) return fail(OUT_OF_RANGE, "tb_attend_decode_static: null argument");
    if (!dtype_ok(a->out_dtype)) return fail(OUT_OF_RANGE, "tb_attend_decode_static: unknown dtype");
    AttendParams p;
    p.qkv = a->qkv, p.q_norm = a->q_norm, p.k_norm = a->k_norm, p.freq = a->freq;
    p.kc = reinterpret_cast<__half*>(a->k_cache), p.vc = reinterpret_cast<__half*>(a->v_cache);
    p.pos = a->pos, p.cap = a->cap, p.window = a->window, p.fresh = a->fresh, p.heads = a->heads, p.kv_heads = a->kv_heads;
    p.scale = a->scale, p.eps = a->eps, p.splits = a->splits;
    p.out = a->out, p.out_f16 = a->out_dtype == TB_F16;
    return launch_attend_static(ctx, p);
}

int tb_sample_greedy(tb_context* ctx, const float* logits, uint32_t vocab, float softcap, float penalty, uint32_t* seen, const uint32_t* allowed,
                     void* scratch, uint32_t* state, uint32_t* token_out) {
    if (!ctx || !scratch || (reinterpret_cast<uintptr_t>(scratch) & 7)) return fail(OUT_OF_RANGE, "tb_sample_greedy: bad scratch");
    return launch_sample(ctx, logits, vocab, softcap, penalty, seen, allowed, static_cast<unsigned long long*>(scratch),
                         reinterpret_cast<uint32_t*>(static_cast<char*>(scratch) + 8), state, seen, token_out);
}

int tb_topk(tb_context* ctx, const float* logits, uint32_t vocab, uint32_t k, uint32_t* idx, float* val) {
    if (!ctx) return fail(OUT_OF_RANGE, "null context");
    return launch_topk(ctx, logits, vocab, k, idx, val, nullptr);
}

int tb_fill_codes(tb_context* ctx, uint64_t seed, uint64_t stream_id, int8_t* dev, size_t n) {
    if (!ctx || !dev) return fail(OUT_OF_RANGE, "tb_fill_codes: null argument");
    return launch_fill_codes(ctx, seed, stream_id, dev, n);
}
int tb_fill_scales(tb_context* ctx, uint64_t seed, uint64_t stream_id, uint16_t* dev, size_t n, float mul) {
    if (!ctx || !dev) return fail(OUT_OF_RANGE, "tb_fill_scales: null argument");
    return launch_fill_scales(ctx, seed, stream_id, reinterpret_cast<__half*>(dev), n, mul);
}
int tb_fill_gauss_f16(tb_context* ctx, uint64_t seed, uint64_t stream_id, uint16_t* dev, size_t n, float mul) {
    if (!ctx || !dev) return fail(OUT_OF_RANGE, "tb_fill_gauss_f16: null argument");
    return launch_fill_gauss_f16(ctx, seed, stream_id, reinterpret_cast<__half*>(dev), n, mul);
}
int tb_fill_uniform(tb_context* ctx, uint64_t seed, uint64_t stream_id, float* dev, size_t n, float lo, float hi) {
    if (!ctx || !dev) return fail(OUT_OF_RANGE, "tb_fill_uniform: null argument");
    return launch_fill_uniform(ctx, seed, stream_id, dev, n, lo, hi);
}

}  // extern "C"
