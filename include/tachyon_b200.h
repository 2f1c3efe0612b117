/*
 * tachyon_b200 -- C ABI of the B200 (sm_100a) decode / prefill hot path.
 *
 * Every entry point returns an int status (TB_OK == 0) and never aborts; tb_last_error() gives the calling thread's
 * last failure as text.  Pointers named `dev_*` or documented as device memory must come from tb_alloc (or any CUDA
 * allocation of the same device); everything else is host memory.  One host thread owns a context; nothing here is
 * thread-safe across contexts sharing a GPU stream, as in the reference (crates/tachyon/src/cuda/mod.rs:3-6).
 *
 * Each declaration cites the reference interface it stands in for (paths relative to the reference repository).
 */
#ifndef TACHYON_B200_H
#define TACHYON_B200_H

#include <stddef.h>
#include <stdint.h>

#if defined(__GNUC__)
#define TB_API __attribute__((visibility("default")))
#else
#define TB_API
#endif

#ifdef __cplusplus
extern "C" {
#endif

/* Status codes; mirror crates/tachyon/src/error.rs:8-50. */
enum {
    TB_OK = 0,
    TB_NO_DRIVER = 1,       /* Error::NoDriver */
    TB_UNSUPPORTED_GPU = 2, /* Error::UnsupportedGpu: not compute capability 10.x */
    TB_OUT_OF_RANGE = 3,    /* Error::OutOfRange: a launch descriptor failed validation, nothing was launched */
    TB_CUDA = 4,            /* Error::Cuda(code) */
    TB_FORMAT = 5,          /* Error::Format */
    TB_TOO_LONG = 6,        /* Error::TooLong: the sequence would pass the context */
    TB_OUT_OF_MEMORY = 7,   /* Error::OutOfMemory */
    TB_NO_MODEL = 8,        /* Error::NoModel: a tensor is missing */
    TB_UNSUPPORTED = 9,     /* Error::Unsupported: a shape this build has no kernel for */
    TB_DEVICE_WAIT = 10,    /* a kernel gave up a bounded wait; see tb_status */
    TB_IO = 11              /* Error::Io(errno): a file could not be opened or read; tb_last_error() has the errno text */
};

typedef struct tb_context tb_context;
typedef struct tb_decoder tb_decoder;
typedef struct tb_parked tb_parked;
typedef struct tb_engine tb_engine;
typedef struct tb_event tb_event;

/* The calling thread's last error message ("" when none). */
TB_API const char* tb_last_error(void);

/* ---- context, memory, stream: crates/tachyon/src/cuda/mod.rs:157-458 (Context, DevBuf, HostBuf, Stream, Event) ---- */

/* Context::new (cuda/mod.rs:177-187): binds GPU `gpu`, requires compute capability 10.x, creates the stream. */
TB_API int tb_context_new(int gpu, tb_context** out);
TB_API void tb_context_free(tb_context* ctx);
/* cuda::devices() (crates/tachyon/src/cuda/mod.rs): how many GPUs the driver offers.  This call and tb_context_new load the
 * driver the way the reference does (cuda/driver.rs:138-167): the library named by $TACHYON_LIBCUDA when that is set, else
 * libcuda.so.1 (then the WSL path); once per process.  TB_NO_DRIVER with the reference's message when it is not found,
 * lacks cuDriverGetVersion / cuGetProcAddress_v2, or supports less than CUDA 12.0 (the reference's DriverTooOld). */
TB_API int tb_devices(int* count);
/* Context::info().sms */
TB_API int tb_context_sms(const tb_context* ctx);
/* Turns programmatic dependent launch on (default) or off for kernels launched after the call. */
TB_API int tb_context_set_overlap(tb_context* ctx, int on);
/* Which schedule tb_gemm_q8 / tb_gemm_q4 use from now on: 0 picks by shape and epilogue (default), 1 one tile per block,
 * 2 persistent blocks, 3 and 4 pairs of SMs with tiles of 256 and 128 weight rows, 5 the first's tile with one block an SM walking
 * the tiles (f16 weights; automatic takes it when there are more tiles than SMs).  The environment variable
 * TACHYON_B200_GEMM gives the value a new context starts with.  (The reference races its tile shapes per product,
 * crates/tachyon/src/encoder/race.rs:56-88; this is the knob such a race turns.) */
TB_API int tb_context_set_gemm_schedule(tb_context* ctx, int which);
/* The small-footprint matrix-vector kernel (no shared-memory ring, dependents released at once; for the short products of a
 * decode step, so that the large product behind them is resident early): 0 never, 1 where the decoder marks a product as
 * short (default), 2 wherever the shape allows (2048 columns, f32 out, at most 32 rows a block), which lets tb_gemv_q8 and
 * tb_gemv_q8_norm reach it.  TACHYON_B200_NO_LEAN=1 starts a context at 0. */
TB_API int tb_context_set_lean(tb_context* ctx, int mode);
/* Whether large matrix-vector products hand their stages of rows to the blocks through a counter (default) or split the
 * rows evenly beforehand (0).  Results are the same bits either way.  TACHYON_B200_STATIC=1 starts a context at 0. */
TB_API int tb_context_set_dynamic(tb_context* ctx, int on);
/* Which kernel tb_prefill_attend, prefill inside the decoder and "flash_256" use for heads of 256 with four query heads to a
 * key-value head and a ring of a multiple of 64 slots: 1 the tcgen05 kernel (S = Q K^T and O = P V in tensor memory;
 * default), 0 the mma.sync kernel every other shape takes.  An encoder with heads of 64 opened while this is 1 runs its
 * attention on tcgen05 as well (tiles of 128 queries of a sequence and head).  TACHYON_B200_FLASH=0 starts a context at 0. */
TB_API int tb_context_set_flash(tb_context* ctx, int which);
/* 1: decoders recorded from now on run the attention half of a layer (norm, q/k/v product, attention, output projection) as one
 * kernel on two thread-block clusters of 16 blocks, where the layer has the shape for it (hidden 2048, 8 query and 2 key-value
 * heads of 256, eight-bit matrices, a cache of its own) and the GPU gives it the clusters; same results to rounding.  Off by
 * default: measured slower than the three launches (the clusters start late and fetch through two GPCs only).
 * TACHYON_B200_ATTN_BLOCK=1 starts a context with it on. */
TB_API int tb_context_set_attn_block(tb_context* ctx, int on);
/* Context::trim (cuda/mod.rs): decoders take their device memory from a pool that keeps what they free, so that the next
 * model to come into VRAM finds it at once (a parked or closed decoder's memory stays with this process); this gives the
 * pool's unused memory back to the system.  The engine calls it when a model is unloaded or expires, as the reference does. */
TB_API int tb_context_trim(tb_context* ctx);
/* Context::memory (cuda/mod.rs:194-198): free and total device memory, in bytes. */
TB_API int tb_context_memory(tb_context* ctx, size_t* free_bytes, size_t* total_bytes);
/* First error word a kernel left on the device (0 = none); synchronises the stream.  *word may be NULL. */
TB_API int tb_status(tb_context* ctx, uint32_t* word);
/* Clears that word (after an error has been looked at). */
TB_API int tb_status_clear(tb_context* ctx);
/*
 * Self-test of the bounded waits, for a deployment that wants to see the failure path work before it relies on it: one
 * block of the matrix-vector kernel whose producer is told to copy nothing, so its consumers' wait runs out after limit_ns
 * (at most 100 ms).  The kernel returns normally; afterwards tb_status reports TB_DEVICE_WAIT with word 1 (a wait for a full
 * stage), and the context keeps working once tb_status_clear has run.  Nothing traps, faults or waits without a limit.
 * The reference's last-block counters never wait (crates/tachyon/src/ptx/attend.rs:334-367), so it has no counterpart.
 */
TB_API int tb_selftest_wait(tb_context* ctx, uint64_t limit_ns);

/* Context::alloc / DevBuf drop (cuda/mod.rs:292-298, 337-375). */
TB_API int tb_alloc(tb_context* ctx, size_t bytes, void** dev);
TB_API int tb_free(tb_context* ctx, void* dev);
/* Context::alloc_host: pinned, device-mapped host memory.  tb_host_device_ptr is HostBuf::device_ptr (cuda/mod.rs:337-375):
 * the address kernels read it at. */
TB_API int tb_alloc_host(tb_context* ctx, size_t bytes, void** host);
TB_API int tb_host_device_ptr(tb_context* ctx, void* host, void** dev);
TB_API int tb_free_host(tb_context* ctx, void* host);
/* Stream::upload / download / fill / sync (cuda/mod.rs:382-411).  Copies are queued on the context's stream; the
 * caller keeps host memory alive until tb_sync. */
TB_API int tb_upload(tb_context* ctx, void* dev, const void* host, size_t bytes);
TB_API int tb_download(tb_context* ctx, void* host, const void* dev, size_t bytes);
TB_API int tb_fill(tb_context* ctx, void* dev, int byte, size_t bytes);
TB_API int tb_sync(tb_context* ctx);
/* Event (cuda/mod.rs:427-458). */
TB_API int tb_event_new(tb_context* ctx, tb_event** out);
TB_API void tb_event_free(tb_event* ev);
TB_API int tb_event_record(tb_context* ctx, tb_event* ev);
TB_API int tb_event_sync(tb_event* ev);
TB_API int tb_event_elapsed_ms(tb_event* start, tb_event* end, float* ms);

/* ---- kernels, one call per launch: the (name, grid, block, args) seam of Stream::launch (cuda/mod.rs:417-425) ---- */

enum { TB_F32 = 0, TB_F16 = 1 };

/*
 * y = W x.  W: device int8 [rows, cols] row-major; scales: device f16 [rows, cols/32]; x: device [cols] of x_dtype;
 * y: device [rows] of y_dtype; f32 accumulation.  Stands in for gemv_q4 / gemv_q4_narrow
 * (crates/tachyon/src/ptx/gemv.rs:1-27, 156-195) with this build's Q8 weights and unquantised activations.
 * cols must be a multiple of 32; 2048, 4096, 8192 and 16384 take the staged kernel.
 */
TB_API int tb_gemv_q8(tb_context* ctx, const int8_t* w, const uint16_t* scales, const void* x, int x_dtype, void* y, int y_dtype, uint32_t rows, uint32_t cols);

/*
 * The same product with f16 weights: w device f16 [rows, cols] row-major, x and y as in tb_gemv_q8, f32 accumulation.
 * The reference keeps f16 weights for models too small for 8-bit codes to pay (gemm_f16, crates/tachyon/src/ptx/
 * encoder.rs:498-525, chosen by encoder/convert.rs:26-29); this is that product for one token.  cols: a multiple of 256,
 * at most 16384.  tb_gemv_f16_norm puts the residual / RMS-norm step of tb_gemv_q8_norm in front (any such cols).
 */
TB_API int tb_gemv_f16(tb_context* ctx, const uint16_t* w, const void* x, int x_dtype, void* y, int y_dtype, uint32_t rows, uint32_t cols);
TB_API int tb_gemv_f16_norm(tb_context* ctx, const uint16_t* w, const float* h, const float* y_res, const float* w1, const float* w2, float eps, float hscale,
                            float* h_out, void* y, int y_dtype, uint32_t rows, uint32_t cols);

/*
 * The residual / RMS-norm step fused in front of the product: h' = (h + w1 * rmsnorm(y_res)) * hscale (y_res NULL:
 * h' = h), x = w2 * rmsnorm(h') (w2 NULL: x = h'), y = W x; h_out (may be NULL) receives h'.  cols must be 2048.
 * Stands in for norm_q8 followed by gemv_q4 (ptx/mod.rs:24-30, 404-511).  `geglu` != 0: rows are (gate_j, up_j) pairs
 * and y (f32 [rows/2]) receives gelu_tanh(gate_j) * up_j -- geglu_q8 (ptx/mod.rs:376-393).
 */
TB_API int tb_gemv_q8_norm(tb_context* ctx, const int8_t* w, const uint16_t* scales, const float* h, const float* y_res, const float* w1, const float* w2,
                    float eps, float hscale, float* h_out, float* y, uint32_t rows, uint32_t cols, int geglu);

/*
 * LM head and greedy pick in one launch: logits = W x (written to `logits` when not NULL), token = argmax with the lowest
 * index among equals; writes state[1] = token, state[0] += 1 and *token_out (device-visible, may be NULL).
 * scratch: 16 bytes of device memory, zero before the first launch, left zero.  Stands in for gemv_q4 over the tied
 * embedding followed by sample in greedy mode (ptx/sample.rs:21-27, 91-97).
 */
TB_API int tb_gemv_q8_argmax(tb_context* ctx, const int8_t* w, const uint16_t* scales, const void* x, int x_dtype, float* logits, uint32_t rows, uint32_t cols,
                      void* scratch, uint32_t* state, uint32_t* token_out);

/*
 * Prefill product on the tensor cores: D[m, n] = A[m, k] x W[n, k]^T.  A: device f16 [m, k] row-major; W, scales: as
 * tb_gemv_q8; f32 accumulation.  mode TB_GEMM_F32: out f32 [m, n]; TB_GEMM_F16: out f16 [m, n]; TB_GEMM_GEGLU: columns
 * (2j, 2j+1) are (gate_j, up_j) and out is f16 [m, n/2] of gelu_tanh(gate) * up.  k a multiple of 64, n of 32.
 * TB_GEMM_ADD: out f32 [m, n] += D (residual); TB_GEMM_GEGLU_ERF / TB_GEMM_GELU_ERF: the encoder's exact-form GELU, gated on
 * column pairs (f16 [m, n/2]) or plain (f16 [m, n]) -- the store modes of gemm_q8 / gemm_f16 (ptx/encoder.rs:418-492).
 * Stands in for gemm_q4 with its split-K slices and sum_slices (crates/tachyon/src/ptx/gemm.rs:18-23, 225-259,
 * 287-325) and, in GeGLU mode, geglu_q8p (ptx/mod.rs:217-249).
 */
enum { TB_GEMM_F32 = 0, TB_GEMM_F16 = 1, TB_GEMM_GEGLU = 2, TB_GEMM_ADD = 3, TB_GEMM_GEGLU_ERF = 4, TB_GEMM_GELU_ERF = 5,
       /* 6: internal (a product times a per-token vector, the per-layer inputs' gate) */
       TB_GEMM_RELU = 7,        /* out f16 [m, n] = max(D, 0): the reference's store mode 3 (ptx/encoder.rs:5-9) */
       TB_GEMM_GATED_SILU = 8   /* out f16 [m, n/2] = silu(D[2j]) * D[2j+1]: its store mode 5 */ };
TB_API int tb_gemm_q8(tb_context* ctx, const int8_t* w, const uint16_t* scales, const uint16_t* a, uint32_t m, uint32_t n, uint32_t k, void* out, int mode);
/* The same product on the reference's Q4 weights (packed u8 [n, k/2], scales f16 [n, k/64], quant.rs:47-82): the nibbles
 * become f16 (n - 8) * scale in the operand path; stands in for gemm_q4 (ptx/gemm.rs:225-259) on a converted model. */
TB_API int tb_gemm_q4(tb_context* ctx, const uint8_t* packed, const uint16_t* scales, const uint16_t* a, uint32_t m, uint32_t n, uint32_t k, void* out, int mode);
/* The same product on f16 weights (w: device f16 [n, k] row-major, as PyTorch's Linear holds them): gemm_f16 and its store
 * modes (ptx/encoder.rs:5-9, 498-525), which the reference uses for encoders too narrow for 8-bit weights (encoder/convert.rs:
 * 26-29).  The weight tile goes to the tensor cores as it is. */
TB_API int tb_gemm_f16(tb_context* ctx, const uint16_t* w, const uint16_t* a, uint32_t m, uint32_t n, uint32_t k, void* out, int mode);
/* out f16 [rows, cols] = code * scale, rounded once to f16 as tb_gemm_q8 / tb_gemm_q4 round it in their operand path (bits 8:
 * codes int8 with an f16 scale per 32; bits 4: the reference's nibbles, (n - 8) * scale with a scale per 64): tb_gemm_f16 on the
 * result is tb_gemm_q8 on the codes.  The decoder's prefill copy is made with it.  No counterpart in the reference. */
TB_API int tb_dequant_f16(tb_context* ctx, const void* w, const uint16_t* scales, uint32_t rows, uint32_t cols, uint32_t bits, uint16_t* out);

/*
 * The reference's own decode formats, for callers that hold a model converted by the reference (quant.rs:47-130):
 * Q4 weights, two per byte in the order of quant.rs:60-66 with one f16 scale per 64, and Q8 activations, i8 codes with
 * a pair [s, s * sum q] per 32.  Both kernels repeat the reference kernels' f32 operations one by one (round to
 * nearest throughout, the same order of sums), so the outputs are the reference's bit for bit.
 *   tb_quant_q8 = quant_q8 (ptx/mod.rs:191-212, 393-399): x f32 [n] -> q i8 [n], pairs f32 [n / 32][2]; n % 32 == 0.
 *   tb_gemv_q4  = gemv_q4 (ptx/gemv.rs:156-195): y f32 [rows] = W (packed [rows][cols / 2], scales f16 [rows][cols / 64])
 *                 times (q, pairs); cols a multiple of 64 (powers of two from 512 to 16384 stream through shared memory).
 */
TB_API int tb_quant_q8(tb_context* ctx, const float* x, uint32_t n, int8_t* q, float* pairs);
TB_API int tb_gemv_q4(tb_context* ctx, const uint8_t* packed, const uint16_t* scales, const int8_t* q, const float* pairs, float* y, uint32_t rows, uint32_t cols);
/*
 * The rest of the reference's small decode kernels, in its formats and with its arithmetic (the approximate instructions
 * too: ex2.approx, rsqrt.approx):
 *   tb_geglu_q8 = geglu_q8 (ptx/mod.rs:376-393): q, pairs <- Q8 of gelu_tanh(a[i]) * b[i]; n % 32 == 0.
 *   tb_norm_q8  = norm_q8 (ptx/mod.rs:404-511): per chunk of `len` values (a multiple of 256 up to 6144): when y is not
 *                 NULL, h_out <- (h + w1 * rmsnorm(y)) * scale; then, when q is not NULL, Q8 of w2 * rmsnorm(h') (of h'
 *                 itself when w2 is NULL).  h is left alone; w1, w2 hold one chunk.
 *   tb_embed_q4 = embed_q4 (ptx/mod.rs:531-598): out[r][i] = (nibble - 8) * scale_f16 * scale for row tokens[r] of the table.
 * tb_launch is Stream::launch by kernel name (cuda/mod.rs:417-425): the names "quant_q8", "geglu_q8", "norm_q8",
 * "embed_q4", "gemv_q4", "sample", "attend_256" / "attend_256_2" / "attend_512" (group 1, or 2 for attend_256 and
 * attend_512; Q8 out), and prefill's "kv_256" / "kv_512", "query_256" / "query_512" (attend.rs:472-556) and "flash_256" /
 * "flash_256_2" / "flash_512" (flash.rs:19-22: f32 out; tiles, block and shared memory are this build's own),
 * prefill's formats "quant_q8p", "geglu_q8p", "norm_q8p", "gemm_q4" (the slices taken from grid[2]) and "sum_slices"
 * (ptx/gemm.rs:18-34), and the encoder's "quant_f16", "norm_f16", "embed_f16", "add_rows", "add_rows_f16", "gather_rows",
 * "gelu_f16", "rope_f16", "attend_f16" / "attend_f16_32", "gemm_f16" / "gemm_f16_128" / "gemm_f16_tall" and "gemm_q8" /
 * "gemm_q8_128" / "gemm_q8_tall" (ptx/encoder.rs:5-38; the three names of a product are one kernel here),
 * with the argument lists of ptx/mod.rs:7-41, gemv.rs:1-16, sample.rs:21-27, attend.rs:21-32 and encoder.rs:5-38;
 * args[i] points at argument i's value (a u64 device address, u32 or f32), as the driver's kernelParams do.  Grid and block
 * are checked against the kernel's documented launch shape where it has a meaning here (chunks, rows and block counts
 * are taken from the grid).  An unknown name is TB_NO_MODEL.
 */
TB_API int tb_geglu_q8(tb_context* ctx, const float* a, const float* b, uint32_t n, int8_t* q, float* pairs);
TB_API int tb_norm_q8(tb_context* ctx, const float* h, float* h_out, const float* y, const float* w1, const float* w2, int8_t* q, float* pairs, uint32_t len,
                      uint32_t chunks, float eps, float scale);
TB_API int tb_embed_q4(tb_context* ctx, const uint8_t* packed, const uint16_t* scales, const uint32_t* tokens, uint32_t rows, float* out, uint32_t cols, float scale);
TB_API int tb_launch(tb_context* ctx, const char* kernel, const uint32_t grid[3], const uint32_t block[3], uint32_t shared_bytes, void* const* args, size_t nargs);
/*
 * The same Q4 weights, read as they are by this build's decode product: the activation (f16 or f32, device) is not
 * rounded to Q8 but split into the exact fixed-point planes tb_gemv_q8 uses, so y = sum_g d_g sum_k (n_k - 8) x_k to
 * f32 accuracy.  This is the product a decoder opened with TB_WEIGHTS_Q4 runs.  cols: 2048, 4096, 8192 or 16384.
 */
TB_API int tb_gemv_q4x(tb_context* ctx, const uint8_t* packed, const uint16_t* scales, const void* x, int x_dtype, float* y, uint32_t rows, uint32_t cols);

/* Stand-alone residual / RMS-norm step (norm_q8 without its Q8 output, ptx/mod.rs:404-511). All device f32 [n]. */
TB_API int tb_norm(tb_context* ctx, const float* h, const float* y_res, const float* w1, const float* w2, uint32_t n, float eps, float hscale, float* h_out,
            float* x_out);
/* The same step for a chunk of prefill (norm_q8p's place, ptx/mod.rs:217-249, model/prefill.rs:144-196), a warp a token:
 * h [tokens, n] f32 is updated in place to (h + w1 * rmsnorm(y)) * hscale (y null: h stays), x [tokens, n] f16 receives
 * w2 * rmsnorm(h') (w2 null: h' itself), the next product's operand.  n = 2048. */
TB_API int tb_prefill_norm(tb_context* ctx, float* h, const float* y, const float* w1, const float* w2, uint32_t tokens, uint32_t n, float eps, float hscale,
                           uint16_t* x);

/* Row *token of a Q8 table times `scale` as f32 [cols]: embed_q4 (ptx/mod.rs:531-598). token: device word. */
TB_API int tb_embed_q8(tb_context* ctx, const int8_t* w, const uint16_t* scales, const uint32_t* token, uint32_t cols, float scale, float* out);

/*
 * Prefill attention on tensor cores: flash_256 / flash_512 (crates/tachyon/src/ptx/flash.rs:1-23).  Token t of the chunk,
 * at position pos0 + t, attends positions p - window < j <= p of the cache (f16 [kv_heads][cap][head_dim], position j in
 * slot j % cap, the chunk's own keys and values already stored).  q: device f16 [tokens][heads][head_dim] as the query
 * kernel leaves them, already multiplied by scale * log2(e); out: device f16 [tokens][heads * head_dim].
 * head_dim 256 or 512; heads / kv_heads in {1, 2, 4, 8}.  Key tiles start at multiples of their size (32 positions; 64 in the
 * tcgen05 kernel, see tb_context_set_flash), so a token's sums do not depend on how the prompt was cut into chunks.
 */
TB_API int tb_prefill_attend(tb_context* ctx, const uint16_t* q, const uint16_t* k_cache, const uint16_t* v_cache, uint16_t* out, uint32_t tokens,
                             uint32_t pos0, uint32_t cap, uint32_t window, uint32_t heads, uint32_t kv_heads, uint32_t head_dim);
/*
 * What prefill does to a chunk's projected rows before that: kv_256 / kv_512 and query_256 / query_512 (ptx/attend.rs:
 * 472-556) in one launch.  qkv: device f32 [tokens][(heads + 2 kv_heads) * head_dim]; queries are normalised (q_norm),
 * rotated at pos0 + t, multiplied by scale * log2(e) and stored as f16 [tokens][heads][head_dim]; keys normalised
 * (k_norm) and rotated, values normalised without weights, both stored as f16 in cache slot (pos0 + t) % cap.
 * kv_heads 0: a layer that shares another layer's cache projects queries only.  freq: f32 [head_dim / 2].
 */
TB_API int tb_prefill_qkv(tb_context* ctx, const float* qkv, const float* q_norm, const float* k_norm, const float* freq, uint16_t* q_out, uint16_t* k_cache,
                          uint16_t* v_cache, uint32_t tokens, uint32_t pos0, uint32_t cap, uint32_t heads, uint32_t kv_heads, float eps, float scale,
                          uint32_t head_dim);

/*
 * Decode attention for one new token; argument meaning follows attend_256 (crates/tachyon/src/ptx/attend.rs:21-32).
 * head size 256; heads / kv_heads in {1, 2, 4}, or 8 (E2B: two blocks of four query heads share a key-value head, the
 * reference's `group` 2; a simpler, slower kernel serves it).
 */
typedef struct tb_attend {
    const float* qkv;      /* device f32 [(heads + 2*kv_heads) * 256]: queries, new keys, new values */
    const float* q_norm;   /* device f32 [256] or NULL: NULL (with k_norm NULL) = plain mode, no norms */
    const float* k_norm;
    const float* freq;     /* device f32 [128] RoPE frequencies, or NULL for no rotation */
    uint16_t* k_cache;     /* device f16 [kv_heads][cap][256] */
    uint16_t* v_cache;
    const uint32_t* pos;   /* device word: position of the new token */
    uint32_t cap;          /* slots per kv head; the new token goes to slot pos % cap */
    uint32_t window;       /* attends the newest min(pos + 1, window) positions; window <= cap */
    uint32_t fresh;        /* != 0: normalise/rotate the new key and value, store them, use them unrounded */
    uint32_t heads, kv_heads;
    float scale;           /* softmax scale (1 in Gemma 4, 1/sqrt(256) in the plain configuration) */
    float eps;
    float* partial;        /* device scratch, tb_attend_scratch_bytes(...) bytes; NULL allowed when splits == 1 */
    uint32_t* count;       /* device, kv_heads words (heads / 4 when heads = 8 kv_heads), zero before the first launch, left zero */
    uint32_t splits;       /* blocks per kv head */
    void* out;             /* device [heads * 256], f32 or f16 */
    int out_dtype;
} tb_attend;
TB_API size_t tb_attend_scratch_bytes(uint32_t heads, uint32_t kv_heads, uint32_t splits);
TB_API int tb_attend_decode(tb_context* ctx, const tb_attend* args);
/*
 * Attention and the output projection as a decode step chains them (model/decode.rs:603-618: attend_*, then gemv(o)):
 * the attention kernel only leaves its splits' results in args->partial, merged `cluster` neighbouring splits at a time
 * inside a thread-block cluster (1: not at all; 2, 4 or 8, dividing splits), and the projection's prologue finishes the merge
 * (the reference merges in its attention kernel's last block, ptx/attend.rs:334-405).  y: device f32 [rows] = W . out with
 * W int8 [rows, heads * 256] and scales f16 [rows, heads * 8]; heads * 256 must be 2048.  args->out, out_dtype and count
 * are not used.
 */
TB_API int tb_attend_project(tb_context* ctx, const tb_attend* args, uint32_t cluster, const int8_t* w, const uint16_t* scales, uint32_t rows, float* y);
/*
 * The same for heads of 512: attend_512 (crates/tachyon/src/ptx/attend.rs:1-32, 37-38), Gemma 4's global layers.  The
 * struct's 256s read 512 (freq: f32 [256]); heads / kv_heads in {1, 2, 4, 8}.  A block takes up to four query heads, so
 * with 8 to a key-value head two blocks share it (the reference's `group` 2).  count: heads / min(heads / kv_heads, 4)
 * words; partial: tb_attend_512_scratch_bytes(heads, splits) bytes.
 */
TB_API size_t tb_attend_512_scratch_bytes(uint32_t heads, uint32_t splits);
TB_API int tb_attend_decode_512(tb_context* ctx, const tb_attend* args);
/*
 * tb_attend_decode for callers that cannot allocate device memory (no counterpart in the reference, which always carves
 * this scratch out of its decoder's arena): an engine whose memory plan is fixed at start-up, or a loop that must not
 * call cudaMalloc because it synchronises the device.  args->partial and args->count are ignored; the scratch is a
 * fixed array inside the library (1,057,024 bytes, about 1.01 MiB, held by every GPU that loads the library, until the process exits).
 * Limits: kv_heads <= 4, splits <= 64, heads / kv_heads <= 4; anything larger returns TB_OUT_OF_RANGE and launches
 * nothing.  The call itself makes no cudaMalloc, cudaFree or other allocating call.
 * The first call on a GPU resolves the array's device address (once per device); make that first call before any
 * stream capture begins.  All calls share the one array: calls that overlap on the GPU (two streams, two contexts on
 * one GPU) race; serialise them.  The array keeps the last call's contents; the call clears the words that must be
 * zero itself.
 */
TB_API int tb_attend_decode_static(tb_context* ctx, const tb_attend* args);

/*
 * Greedy sampler over f32 logits with the reference's transform (soft cap, allowed mask, repetition penalty):
 * sample in greedy mode (ptx/sample.rs:21-27; Sampling, :38-78).  seen / allowed: device bitmaps or NULL.
 * scratch as in tb_gemv_q8_argmax.  Sets the token's bit in `seen` when given.
 */
TB_API int tb_sample_greedy(tb_context* ctx, const float* logits, uint32_t vocab, float softcap, float penalty, uint32_t* seen, const uint32_t* allowed,
                     void* scratch, uint32_t* state, uint32_t* token_out);
/*
 * Sampling (ptx/sample.rs:38-78), laid out as the kernel reads it from DEVICE memory, so that one recorded decode step
 * serves every setting: soft cap (0: none), temperature (0: the most likely token), nucleus size (1: no limit), least
 * probability relative to the most likely token (0: no limit), repetition penalty (1: none), most tokens kept (0: no
 * limit), device address of a bitmap of allowed tokens (0: all), seed of the draws.
 */
typedef struct tb_sampling {
    float softcap, temperature, top_p, min_p, penalty;
    uint32_t top_k;
    uint64_t allowed;
    uint64_t seed;
} tb_sampling;
/*
 * sample (ptx/sample.rs:1-27), argument for argument: logits f32 [vocab] (left unchanged), work f32 [vocab], cfg (device),
 * state = [step, token] (the kernel writes the token and advances the step, which seeds the next draw), seen (bitmap of
 * vocab bits; the token's bit is set), out (NULL or a word that also receives the token, e.g. mapped pinned memory),
 * partial (8 words per block), count (zero before the first launch, left zero).  vocab is a multiple of 4.  The draw
 * is exact under top_k / top_p / min_p: Gumbel-max over the tokens, the candidate checked against the filters by the
 * last block and redrawn among the tokens above it when it fails (32 rounds at most, then the largest).
 * blocks: 0, or the most blocks to launch (the reference's tests use 7 so that a block walks several shares).
 */
TB_API int tb_sample(tb_context* ctx, const float* logits, float* work, uint32_t vocab, const tb_sampling* cfg, uint32_t* state, uint32_t* seen,
                     uint32_t* out, void* partial, uint32_t* count, uint32_t blocks);
/* The k largest logits, largest first, lowest index first among equals. idx, val: device [k]. */
TB_API int tb_topk(tb_context* ctx, const float* logits, uint32_t vocab, uint32_t k, uint32_t* idx, float* val);

/* Seeded synthetic tensors (this build's generators; the reference's benches are synthetic too, benches/gemv.rs:8-9). */
TB_API int tb_fill_codes(tb_context* ctx, uint64_t seed, uint64_t stream_id, int8_t* dev, size_t n);
TB_API int tb_fill_scales(tb_context* ctx, uint64_t seed, uint64_t stream_id, uint16_t* dev, size_t n, float mul);
TB_API int tb_fill_gauss_f16(tb_context* ctx, uint64_t seed, uint64_t stream_id, uint16_t* dev, size_t n, float mul);
TB_API int tb_fill_uniform(tb_context* ctx, uint64_t seed, uint64_t stream_id, float* dev, size_t n, float lo, float hi);

/* ---- decoder: crates/tachyon/src/model/decode.rs (Decoder, Settings) and model/mod.rs:27-61 (Config) ---- */

typedef struct tb_config {
    uint32_t hidden, ffn, heads, kv_heads, head_dim, vocab, layers, window;
    const uint8_t* global;  /* [layers], != 0 where a layer attends globally (Config::global); NULL: use global_every */
    uint32_t global_every;  /* with global == NULL: layer i is global iff (i + 1) % global_every == 0; 0 = none */
    float theta_sliding, theta_global, fraction_global; /* Config::theta, Config::fraction */
    float eps, softcap;
    float attn_scale;       /* softmax scale; Gemma 4 uses 1 */
    uint32_t shared;        /* Config::shared: the last `shared` layers project no keys or values and attend over the cache of the
                               last earlier layer of their kind (Config::source, model/mod.rs:138-143); their qkv matrix holds
                               the query rows only */
    uint32_t global_head_dim; /* Config::head_dim[1]: head size of global layers, 256 or 512; 0 = head_dim */
    uint32_t global_kv_heads; /* Config::kv_heads[1]: key-value heads of global layers; 0 = kv_heads */
    uint32_t per_layer;       /* Config::per_layer: width of each layer's per-layer input (256 in Gemma 4's E models); 0 = none.
                                 Tensors: embed_per_layer [vocab, layers * per_layer], per_layer_proj [layers * per_layer, hidden],
                                 per_layer_norm [per_layer], {i}.per_layer_gate [per_layer, hidden], {i}.per_layer_proj [hidden,
                                 per_layer], {i}.post_per_layer_input_norm [hidden] (model/mod.rs:180-186, 199-201, 228-236).  Eight-bit weights only;
                                 the table lives in device memory (the reference keeps it in pinned host memory) */
} tb_config;

/* model::Settings (decode.rs:64-76) plus what this build adds. */
typedef struct tb_settings {
    uint32_t context;      /* positions a global layer keeps */
    uint32_t chunk;        /* extra ring slots of sliding layers (the reference's prefill chunk) */
    uint32_t keep_logits;  /* != 0: every step also stores the f32 logits for tb_decoder_logits */
    uint32_t fused;        /* != 0: the whole step as one persistent kernel with grid barriers instead of 2 + 5*layers launches */
    uint32_t weight_bits;  /* 0 or 8: int8 codes with an f16 scale per 32 (TB_WEIGHTS_Q8); 4: the reference's converted Q4
                              matrices as they are in weights.wpk, u8 [rows, cols/2] and f16 [rows, cols/64] (TB_WEIGHTS_Q4) */
    uint32_t host_table;   /* != 0: the per-layer table (embed_per_layer, the reference's host.wpk) stays in pinned, mapped host
                              memory and every step reads its token's row from there (decode.rs:477-483, 572-573); 0: in HBM */
    uint32_t prefill_copy; /* the layers' qkv, o, gate/up and down matrices once more as f16 (2 bytes a weight beside the codes),
                              which prefill's products on 256 tokens and more read by TMA instead of converting codes in their
                              loop; the values are the codes' own (tb_dequant_f16), decode keeps reading the codes.
                              0: automatic (when chunk >= 256 and a quarter of the device's memory stays free after it;
                              TACHYON_B200_PREFILL_COPY=0 turns it off), 1: none, 2: always (TB_OUT_OF_MEMORY without room) */
} tb_settings;
enum { TB_WEIGHTS_Q8 = 8, TB_WEIGHTS_Q4 = 4 };

/* Decoder::open without the file loader: allocates weights, caches and step buffers for `cfg`. */
TB_API int tb_decoder_open(tb_context* ctx, const tb_config* cfg, const tb_settings* settings, tb_decoder** out);
TB_API void tb_decoder_close(tb_decoder* dec);
/*
 * Uploads one tensor by its converted-model name (model/mod.rs:178-286): matrices as `<name>.w` (int8 codes; with
 * TB_WEIGHTS_Q4 the reference's packed nibbles) and `<name>.s` (f16 scales, one per 32 along a row; per 64 with Q4) for embed, {i}.qkv, {i}.o, {i}.gate_up (gate rows, then up rows),
 * {i}.down; f32 vectors {i}.q_norm, {i}.k_norm, {i}.input_layernorm, {i}.post_attention_layernorm,
 * {i}.pre_feedforward_layernorm, {i}.post_feedforward_layernorm, {i}.layer_scalar, norm.
 */
TB_API int tb_decoder_load(tb_decoder* dec, const char* name, const void* data, size_t bytes);
/* Fills every tensor from the seeded generators (stream ids documented in decoder.cu). */
TB_API int tb_decoder_fill_random(tb_decoder* dec, uint64_t seed);
/* Fills the first `positions` positions of every cache with seeded N(0,1) values and sets the position. */
TB_API int tb_decoder_fill_cache(tb_decoder* dec, uint64_t seed, uint32_t positions);
/* Records the step's graphs (Decoder::build, decode.rs:250-272); call after loading, before stepping. */
TB_API int tb_decoder_build(tb_decoder* dec);
/* Decoder::reset (decode.rs:297-301): position 0. */
TB_API int tb_decoder_reset(tb_decoder* dec);
/* Decoder::step (decode.rs:305-310): host token in, sampled token out, one graph launch, waits for it. */
TB_API int tb_decoder_step(tb_decoder* dec, uint32_t token, uint32_t* next);
/* Decoder::start / next_token / stop (decode.rs:313-345): keeps one step queued behind the running one. */
TB_API int tb_decoder_start(tb_decoder* dec, uint32_t token);
TB_API int tb_decoder_next_token(tb_decoder* dec, uint32_t* token);
TB_API int tb_decoder_stop(tb_decoder* dec);
/* Queues `steps` chained steps (each feeds the token the one before sampled) without touching the host between
 * them, starting from `token`; for throughput measurement.  tokens_out (host, may be NULL) receives them after a sync. */
TB_API int tb_decoder_run(tb_decoder* dec, uint32_t token, uint32_t steps, uint32_t* tokens_out);
/* Decoder::prefill (decode.rs:346-364): feeds `n` prompt tokens, no sampling result kept. */
TB_API int tb_decoder_prefill(tb_decoder* dec, const uint32_t* tokens, uint32_t n);
/* Decoder::logits (decode.rs:439-445): the last step's logits, needs settings.keep_logits. */
TB_API int tb_decoder_logits(tb_decoder* dec, float* host_out);
/* Current position. */
TB_API int tb_decoder_position(tb_decoder* dec, uint32_t* pos);
/*
 * How the next steps pick their token (the engine's Request -> Sampling, sample.rs:38-78; NULL: Sampling::default, the
 * largest logit).  While the settings ask for no more than the largest logit (temperature 0, penalty 1, no mask) the
 * step's LM head picks it itself; otherwise the step ends in the head's logits and tb_sample's kernel, recorded once:
 * the settings live in device memory, so changing them records nothing.  `allowed` is a device address the caller keeps
 * alive.  The bitmap of seen tokens starts empty at tb_decoder_reset and gains every generated token.  Draws are a
 * function of (seed, position).  Not with the fused step.
 */
TB_API int tb_decoder_set_sampling(tb_decoder* dec, const tb_sampling* sampling);
/* Bytes of weights and of key/value cache one step reads at the current position (the roofline's numerator). */
TB_API int tb_decoder_step_bytes(tb_decoder* dec, uint64_t* weight_bytes, uint64_t* cache_bytes);
/* Kernels one step launches. */
TB_API int tb_decoder_step_launches(tb_decoder* dec, uint32_t* launches);
/*
 * Decoder::timeline (decode.rs:424-436): runs one step on `token` outside the two step graphs and returns, for the
 * first and for the last block of every phase (embedding, per layer qkv / attention / o / gate_up / down, head),
 * four %globaltimer stamps in ns.  One launch per phase: kernel entry, after the wait for the previous kernel, after
 * the prologue (0 for attention and the embedding, which has no stamps at all), end of the block's work.  Fused
 * step: start, after the prologue, end of work, after the barrier behind it.
 * host_out: [2 blocks][phases][4] words; call with host_out NULL to learn `phases`.
 */
TB_API int tb_decoder_timeline(tb_decoder* dec, uint32_t token, uint64_t* host_out, uint32_t* phases);
/* ---- weights.wpk: crates/tachyon/src/wpk/mod.rs (Wpk::open, tensors, verify) ---- */

typedef struct tb_wpk tb_wpk;
/* wpk::Tensor (wpk/mod.rs:74-89).  dtype: 0 F32, 1 F16, 2 BF16, 3 F8E4M3, 4 I8, 5 U8 (wpk/mod.rs:44-62). */
typedef struct tb_wpk_info {
    const char* name;      /* owned by the file handle */
    uint32_t dtype, rank;
    uint64_t shape[8];
    uint64_t offset;       /* in the data region, which starts at byte 4096 of the file */
    uint64_t bytes;
    uint32_t crc32c;
} tb_wpk_info;
/* CRC32C (Castagnoli) of `bytes` bytes continuing from `crc` (wpk/mod.rs:105-123); tb_crc32c(0, "123456789", 9) is 0xE3069283. */
TB_API uint32_t tb_crc32c(uint32_t crc, const void* data, size_t bytes);
/* CRC32C of A followed by B from tb_crc32c(0, A), tb_crc32c(0, B) and B's length: pieces of a tensor checked apart. */
TB_API uint32_t tb_crc32c_combine(uint32_t crc_a, uint32_t crc_b, uint64_t len_b);
/* Wpk::open (wpk/mod.rs:190-213): checks the header, the table's checksum and every table entry; TB_FORMAT with the
 * reference's message when a check fails, TB_IO when the file cannot be read. */
TB_API int tb_wpk_open(const char* path, tb_wpk** out);
TB_API void tb_wpk_close(tb_wpk* wpk);
TB_API uint32_t tb_wpk_count(const tb_wpk* wpk);
TB_API int tb_wpk_tensor(const tb_wpk* wpk, uint32_t index, tb_wpk_info* out);
/* Reads tensor `index` into `host` (`bytes` must be its size); verify != 0 also checks its CRC32C (Wpk::verify). */
TB_API int tb_wpk_read(const tb_wpk* wpk, uint32_t index, void* host, size_t bytes, int verify);
/*
 * Decoder::open's loading step (decode.rs:225-247) for a converted model's weights.wpk: every tensor of the file goes
 * to tb_decoder_load under its own name.  The decoder must have been opened with the file's format (TB_WEIGHTS_Q4 for
 * a model converted by the reference).  A tensor the decoder has no place for (per-layer inputs, experts) ends the
 * load with TB_NO_MODEL; a size that does not fit with TB_FORMAT.
 */
TB_API int tb_decoder_load_wpk(tb_decoder* dec, const char* path, int verify);

/*
 * The host-RAM tier (Decoder::park, Parked::resume, Decoder::{shadow_bytes, drop_shadow, parked_bytes}: decode.rs:235-247,
 * 275-295, 452-463).  tb_decoder_park stops a running generation, copies the weights into pinned host memory (unless the decoder
 * still holds the pinned copy it was resumed from), frees the decoder and every byte of its device memory, and hands back the
 * parked model; on failure the decoder is untouched.  tb_parked_resume takes the parked model (on success) and gives a built
 * decoder with `settings` (context and chunk may differ; weight_bits and host_table are the parked model's): one copy of the
 * weights over the link, then the step's graphs are recorded; the pinned copy stays with the decoder as its shadow.  The
 * per-layer table in host memory moves along as it is.  Positions, caches and sampler state do not survive: the decoder
 * starts at position 0 with greedy sampling.
 */
TB_API int tb_decoder_park(tb_decoder* dec, tb_parked** out);
TB_API int tb_parked_resume(tb_parked* parked, const tb_settings* settings, tb_decoder** out);
TB_API size_t tb_parked_bytes(const tb_parked* parked);   /* pinned host memory it holds: weights + table */
TB_API void tb_parked_close(tb_parked* parked);
TB_API size_t tb_decoder_bytes(const tb_decoder* dec);          /* device memory it holds: arena + prefill copy */
/* The device memory a decoder of this shape and these settings takes, without allocating it (the engine's `need`,
 * engine.rs:214; an automatic prefill copy is counted whenever chunk >= 256). */
TB_API int tb_decoder_footprint(tb_context* ctx, const tb_config* cfg, const tb_settings* settings, size_t* bytes);
TB_API size_t tb_decoder_parked_bytes(tb_decoder* dec);         /* pinned memory parking it would hold */
TB_API size_t tb_decoder_shadow_bytes(const tb_decoder* dec);   /* pinned memory it keeps from its last resume */
TB_API void tb_decoder_drop_shadow(tb_decoder* dec);

/*
 * Model residency: the reference engine's tiers (engine.rs:62-130 Limits / Load / Loaded / Tier, 203-223 load, 243-250 unload,
 * 271-283 tier, 309-325 expire, 386-453 resident / room / evict).  Decoders only; names are the caller's.  A model is loaded
 * from its converted files (weights.wpk, and host.wpk for a per-layer table); asking for it brings it into VRAM, moving
 * out the least recently used models that may go (not pinned, not the one asked for) until `vram_limit` holds; a model
 * moved out is parked in pinned host memory if `host_limit` allows, after the least recently used pinned memory has given
 * way (a resident model's kept copy is dropped, a parked model goes to disk), else it goes to disk and is read again when
 * asked for.  A keep-alive that has run out sends a model to disk at the next call.  Limits of 0 mean 70 % of the GPU's
 * memory and half the machine's RAM.  tb_decoder_footprint gives a model's VRAM `need`.
 */
enum { TB_TIER_VRAM = 0, TB_TIER_HOST = 1, TB_TIER_DISK = 2 };  /* engine.rs:110-118 */
typedef struct tb_load {   /* engine.rs:72-90 */
    tb_settings settings;
    uint64_t keep_alive_ms;  /* how long it stays in memory after its last use; 0: out at the next call; UINT64_MAX: for good */
    uint32_t pin;            /* != 0: never moves out of VRAM, by keep-alive or to make room */
} tb_load;
typedef struct tb_loaded { /* engine.rs:93-107 */
    char name[64];
    int tier;
    size_t vram;             /* the VRAM it takes where it is: 0 out of VRAM */
    uint64_t left_ms;        /* what is left of its keep-alive; UINT64_MAX: no end (pinned or kept for good) */
} tb_loaded;
TB_API int tb_engine_new(tb_context* ctx, size_t vram_limit, size_t host_limit, tb_engine** out);
TB_API void tb_engine_close(tb_engine* eng);
/* Engine::load: a model of that name is unloaded first; TB_OUT_OF_MEMORY (nothing loaded) when it cannot be made to fit. */
TB_API int tb_engine_load(tb_engine* eng, const char* name, const tb_config* cfg, const tb_load* load, const char* weights_path, const char* host_path);
TB_API int tb_engine_unload(tb_engine* eng, const char* name, int* was_loaded);
/* The model's decoder, in VRAM (Engine::resident), its keep-alive started again.  The pointer is the engine's and holds
 * until the next call that may move the model.  TB_NO_MODEL for a name that is not loaded. */
TB_API int tb_engine_decoder(tb_engine* eng, const char* name, tb_decoder** out);
/* feed (engine.rs:458-465) without the tokenizer: from position 0, every prompt token but the last through prefill, the
 * last through a step; *first is the answer's first token.  tb_decoder_next_token etc. on tb_engine_decoder's pointer go on. */
TB_API int tb_engine_feed(tb_engine* eng, const char* name, const uint32_t* tokens, uint32_t n, uint32_t* first);
TB_API int tb_engine_tier(const tb_engine* eng, const char* name, int* tier);
TB_API int tb_engine_models(const tb_engine* eng, tb_loaded* out, size_t capacity, size_t* count);
TB_API int tb_engine_expire(tb_engine* eng);
TB_API int tb_engine_usage(const tb_engine* eng, size_t* vram, size_t* host);   /* Engine::used, Engine::hosted */

/* Hidden state after the last step, f32 [hidden] (for layer-wise parity checks). */
TB_API int tb_decoder_hidden(tb_decoder* dec, float* host_out);

/* ---- encoder: crates/tachyon/src/encoder/{mod,run}.rs (Config, Encoder) ---- */

typedef struct tb_encoder tb_encoder;

/* encoder::Config (encoder/mod.rs:36-90) plus the benchmark's variants. */
typedef struct tb_encoder_config {
    uint32_t hidden, heads, inter, vocab, layers;
    uint32_t window;        /* a sliding layer sees |i - j| <= window (Config::window = local_attention / 2) */
    const uint8_t* global;  /* [layers] != 0 where a layer attends globally; NULL: every global_every-th from layer 0 */
    uint32_t global_every;  /* with global == NULL (0 means 3, as the reference's default) */
    float theta_global, theta_local, eps;
    uint32_t gated;         /* 1: Wi is [2*inter, hidden], MLP = gelu(first half) * second half (the reference); 2: the same with a
                             * SiLU for the GELU (Config::silu, encoder/mod.rs:55-56); 0: Wi is [inter, hidden], plain GELU */
    uint32_t mean_pool;     /* != 0: mean over a sequence's tokens; 0: its first token (the reference, run.rs:160-173) */
    uint32_t dims;          /* leading dimensions kept (Matryoshka, encoder/text.rs:56-63); hidden keeps all */
} tb_encoder_config;

/* Encoder::open without the file loader: room for `tokens` packed tokens and `sequences` sequences a batch
 * (encoder::Settings::tokens, encoder/mod.rs:23-33).  A batch runs padded to whole tiles of 64 tokens as a CUDA graph
 * recorded the first time its padded shape is seen, sixteen shapes kept (Encoder::encode, encoder/run.rs:379-410);
 * TACHYON_B200_ENCODER_GRAPHS=0 in the environment at this call launches kernel by kernel instead. */
TB_API int tb_encoder_open(tb_context* ctx, const tb_encoder_config* cfg, uint32_t tokens, uint32_t sequences, tb_encoder** out);
TB_API void tb_encoder_close(tb_encoder* enc);
/* Tensors by converted-model name (encoder/convert.rs:79-105): embed (f16 [vocab, hidden]), embed_norm, final_norm,
 * {l}.attn_norm (layer 0's is unused), {l}.mlp_norm (f32 [hidden]); matrices {l}.qkv, {l}.o, {l}.up, {l}.down either as
 * a converted model holds them, under the plain name: f16 [rows, cols], or Q8E codes i8 [rows, cols] with <name>.scale,
 * f32 [rows, cols / 64] (quant.rs:107-115; which of the two is told by the size; the scales are kept as f16, one per 32);
 * or in this build's Q8: <name>.w (int8 codes) and <name>.s (f16 scale per 32 along a row).  The gated Wi ({l}.up) comes
 * as the file has it, the activation's rows then the gate's, and is interleaved on the device (Encoder::interleave,
 * encoder/run.rs:449-466). */
TB_API int tb_encoder_load(tb_encoder* enc, const char* name, const void* data, size_t bytes);
TB_API int tb_encoder_fill_random(tb_encoder* enc, uint64_t seed);
/* Every tensor of a converted encoder's file (weights.wpk, host.wpk: encoder/convert.rs) through tb_encoder_load, as
 * tb_decoder_load_wpk does for a decoder; verify != 0 checks each tensor's CRC32C first. */
TB_API int tb_encoder_load_wpk(tb_encoder* enc, const char* path, int verify);
/* Encoder::embeddings (run.rs:161-175): ids packed back to back, lens[s] tokens each; out_host: dims f32 per sequence,
 * L2-normalised.  More tokens (or sequences) than the encoder was opened for go in several batches, in order, a batch
 * closed by the first sequence that no longer fits (Encoder::batches, run.rs:207-221); one sequence longer than the
 * capacity is TB_TOO_LONG. */
TB_API int tb_encoder_embed(tb_encoder* enc, const uint32_t* ids, const uint32_t* lens, uint32_t sequences, float* out_host);
/* The last batch's final hidden states, f32 [tb_encoder_batch_tokens, hidden] (for parity checks). */
TB_API int tb_encoder_hidden(tb_encoder* enc, float* out_host);
TB_API uint32_t tb_encoder_batch_tokens(const tb_encoder* enc);
/* Padded shapes whose graph is held at the moment. */
TB_API uint32_t tb_encoder_graphs(const tb_encoder* enc);
/* Encoder::bytes (encoder/run.rs:144-147): the VRAM the encoder holds.  encoder::footprint (encoder/run.rs:613-619): what
 * tb_encoder_open will take for this shape and capacity; f16_matrices != 0 counts the layers' matrices in f16 too, which a
 * converted f16 model loads beside the arena. */
TB_API size_t tb_encoder_bytes(const tb_encoder* enc);
TB_API int tb_encoder_footprint(tb_context* ctx, const tb_encoder_config* cfg, uint32_t tokens, uint32_t sequences, int f16_matrices, size_t* bytes);

/* Encoders in the engine (engine.rs:54-55, 225-232, 244-262): held by name, always in VRAM and counted against the VRAM limit
 * (tb_engine_usage, tb_engine_models list them after the decoders, tier TB_TIER_VRAM), dropped by tb_engine_expire when their
 * keep-alive has run out (keep_alive_ms as in tb_load; pin != 0: never).  Loading one moves decoders out to make room, as
 * loading a decoder does; an encoder never moves out.  tb_engine_unload and tb_engine_tier take an encoder's name too.
 * tb_engine_encoder starts the keep-alive again; its pointer is the engine's.  tb_engine_embed is Engine::embed from token
 * ids (the tokenizer stays with the caller): tb_encoder_embed on the held encoder. */
TB_API int tb_engine_load_encoder(tb_engine* eng, const char* name, const tb_encoder_config* cfg, uint32_t tokens, uint32_t sequences, uint64_t keep_alive_ms, int pin,
                                  const char* weights_path, const char* host_path);
TB_API int tb_engine_encoder(tb_engine* eng, const char* name, tb_encoder** out);
TB_API int tb_engine_embed(tb_engine* eng, const char* name, const uint32_t* ids, const uint32_t* lens, uint32_t sequences, float* out_host);

/* ---- Text to token ids and back (host code; crates/tachyon/src/token/mod.rs, token/chat.rs) ------------------------------------
 * Tokenizer::from_json (mod.rs:97-127) reads a Hugging Face tokenizer.json of Gemma's kind (BPE with byte fallback, spaces
 * as U+2581), of the Metaspace kind, or byte-level BPE cut by GPT-2's, cl100k's or o200k's pattern, with an NFC normalizer
 * or none; anything else is refused (TB_FORMAT, "... is not supported").  Tokenizer::to_bytes /
 * from_bytes (mod.rs:422-455) are the reference's stored form, word for word: a converted model's tokenizer.tok loads as it
 * is.  Tokenizer::encode (mod.rs:272-301) encodes text literally: a special token's text stays text; special tokens enter by
 * id, from the chat template.  Output buffers: *count (or *bytes) is always what the whole result needs; with capacity 0
 * nothing is written and the call only counts; a capacity that is too small is TB_OUT_OF_RANGE.  A tokenizer is not changed
 * by any call after it is made: threads may encode with one at the same time; a detokenizer belongs to one stream of tokens. */
typedef struct tb_tokenizer tb_tokenizer;
typedef struct tb_detokenizer tb_detokenizer;
TB_API int tb_tokenizer_from_json(const void* json, size_t bytes, tb_tokenizer** out);
TB_API int tb_tokenizer_from_bytes(const void* data, size_t bytes, tb_tokenizer** out);
TB_API int tb_tokenizer_to_bytes(const tb_tokenizer* tok, void* out, size_t capacity, size_t* bytes);
TB_API void tb_tokenizer_close(tb_tokenizer* tok);
TB_API size_t tb_tokenizer_len(const tb_tokenizer* tok);                                           /* Tokenizer::len */
TB_API int tb_tokenizer_encode(const tb_tokenizer* tok, const char* text, size_t bytes, uint32_t* ids, size_t capacity, size_t* count);
/* Tokenizer::bytes (mod.rs:241-245): the text token `id` decodes to; a byte token is one byte, maybe part of a character.
 * The pointer is the tokenizer's. */
TB_API int tb_tokenizer_token(const tb_tokenizer* tok, uint32_t id, const uint8_t** text, size_t* bytes);
TB_API int tb_tokenizer_is_special(const tb_tokenizer* tok, uint32_t id);                          /* Tokenizer::is_special */
TB_API int tb_tokenizer_special(const tb_tokenizer* tok, const char* text, uint32_t* id);          /* Tokenizer::special; TB_NO_MODEL if none */
/* Tokenizer::frame (mod.rs:232-234): the special tokens the post-processor puts before and after a text; UINT32_MAX: none. */
TB_API void tb_tokenizer_frame(const tb_tokenizer* tok, uint32_t* before, uint32_t* after);
/* Detokenizer (mod.rs:603-648): generated tokens back into text as they come, whole characters only: a character split across
 * byte tokens appears once its last byte arrives; special tokens add nothing; finish gives what is left, an unfinished
 * character as U+FFFD.  A call whose text does not fit consumes nothing. */
TB_API int tb_detokenizer_new(tb_detokenizer** out);
TB_API void tb_detokenizer_close(tb_detokenizer* det);
TB_API int tb_detokenizer_push(tb_detokenizer* det, const tb_tokenizer* tok, uint32_t id, char* out, size_t capacity, size_t* bytes);
TB_API int tb_detokenizer_finish(tb_detokenizer* det, char* out, size_t capacity, size_t* bytes);
/* Gemma 4's chat template (token/chat.rs:1-16, 57-72, 124-163), text messages only: <bos>, the system turn when the first
 * message is a system message or thinking is on (<|think|> switches it on), each message trimmed and closed by <turn|>,
 * consecutive model messages sharing one turn, then the opening of the model's turn; with `closed` set (Chat::with_template,
 * chat.rs:97-107: told from the model's chat_template.jinja) an empty thinking block follows when thinking is off. */
enum { TB_ROLE_SYSTEM = 0, TB_ROLE_USER = 1, TB_ROLE_MODEL = 2 };
typedef struct tb_chat {
    uint32_t bos, turn, end, think;
    uint32_t closed[2];      /* <|channel>, <channel|>, or UINT32_MAX twice */
} tb_chat;
typedef struct tb_message {
    int role;
    const char* text;
    size_t bytes;
} tb_message;
TB_API int tb_chat_gemma4(const tb_tokenizer* tok, tb_chat* out);                                  /* TB_FORMAT: not Gemma 4's tokenizer */
TB_API int tb_chat_with_template(const tb_tokenizer* tok, tb_chat* chat, const char* template_text, size_t bytes);
TB_API int tb_chat_encode(const tb_tokenizer* tok, const tb_chat* chat, const tb_message* messages, size_t n, int think, uint32_t* ids, size_t capacity, size_t* count);

#ifdef __cplusplus
}
#endif
#endif
