"""tachyon_b200: the B200 (sm_100a) decode hot path of the tachyon engine behind a C ABI.

This package is a thin host-side mirror of the reference's Rust API names (``Context``, ``DevBuf``, ``Decoder``,
``Config``, ``Settings``; crates/tachyon/src/cuda/mod.rs, crates/tachyon/src/model/decode.rs) over
``libtachyon_b200.so``.  All computation happens in the library's CUDA kernels; nothing here computes on the CPU and
nothing falls back when the library or a GPU is missing.
"""
from __future__ import annotations

import ctypes as C
import os

import numpy as np

from . import _lib
from ._lib import Attend, Config, EncoderConfig, Load, Loaded, Settings

F32, F16 = 0, 1


class Error(RuntimeError):
    """A non-zero status from the library; ``status`` is the TB_* code."""

    def __init__(self, status: int, message: str):
        super().__init__(f"tachyon_b200 status {status}: {message}")
        self.status = status


def check(status: int) -> None:
    if status != 0:
        raise Error(status, _lib.load().tb_last_error().decode())


class HostBuf:
    """Pinned, device-mapped host memory (cuda/mod.rs HostBuf): ``array`` is the host's view of it as bytes, ``ptr`` the address
    kernels read it at."""

    def __init__(self, ctx: "Context", nbytes: int):
        self.ctx, self.nbytes = ctx, nbytes
        p, d = C.c_void_p(), C.c_void_p()
        check(ctx.lib.tb_alloc_host(ctx.handle, nbytes, C.byref(p)))
        self.host = p.value
        check(ctx.lib.tb_host_device_ptr(ctx.handle, self.host, C.byref(d)))
        self.ptr = d.value
        self.array = np.ctypeslib.as_array((C.c_uint8 * nbytes).from_address(self.host))

    def free(self) -> None:
        if self.host is not None and self.ctx.handle:
            self.array = None
            self.ctx.lib.tb_free_host(self.ctx.handle, self.host)
        self.host = None

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass


class DevBuf:
    """Device memory owned by a context (cuda/mod.rs DevBuf): freed on ``free`` or with the object."""

    def __init__(self, ctx: "Context", nbytes: int):
        self.ctx, self.nbytes = ctx, nbytes
        p = C.c_void_p()
        check(ctx.lib.tb_alloc(ctx.handle, nbytes, C.byref(p)))
        self.ptr = p.value

    def free(self) -> None:
        if self.ptr is not None and self.ctx.handle:
            self.ctx.lib.tb_free(self.ctx.handle, self.ptr)
        self.ptr = None

    def __del__(self):
        try:
            self.free()
        except Exception:
            pass

    def upload(self, a: np.ndarray) -> "DevBuf":
        a = np.ascontiguousarray(a)
        assert a.nbytes <= self.nbytes
        check(self.ctx.lib.tb_upload(self.ctx.handle, self.ptr, a.ctypes.data, a.nbytes))
        self.ctx.sync()
        return self

    def download(self, dtype, count: int | None = None) -> np.ndarray:
        dtype = np.dtype(dtype)
        n = self.nbytes // dtype.itemsize if count is None else count
        out = np.empty(n, dtype)
        check(self.ctx.lib.tb_download(self.ctx.handle, out.ctypes.data, self.ptr, out.nbytes))
        self.ctx.sync()
        return out

    def zero(self) -> "DevBuf":
        check(self.ctx.lib.tb_fill(self.ctx.handle, self.ptr, 0, self.nbytes))
        return self


class Context:
    """One GPU and its stream (cuda/mod.rs Context + Stream)."""

    def __init__(self, gpu: int = 0):
        self.lib = _lib.load()
        h = C.c_void_p()
        check(self.lib.tb_context_new(gpu, C.byref(h)))
        self.handle = h.value
        self.gpu = gpu

    def close(self) -> None:
        if self.handle:
            self.lib.tb_context_free(self.handle)
            self.handle = None

    @property
    def sms(self) -> int:
        return self.lib.tb_context_sms(self.handle)

    def set_overlap(self, on: bool) -> None:
        check(self.lib.tb_context_set_overlap(self.handle, int(on)))

    def sync(self) -> None:
        check(self.lib.tb_sync(self.handle))

    def status(self) -> int:
        w = C.c_uint32(0)
        check(self.lib.tb_status(self.handle, C.byref(w)))
        return w.value

    def alloc(self, nbytes: int) -> DevBuf:
        return DevBuf(self, nbytes)

    def alloc_host(self, nbytes: int) -> HostBuf:
        return HostBuf(self, nbytes)

    def upload(self, a: np.ndarray) -> DevBuf:
        a = np.ascontiguousarray(a)
        return DevBuf(self, max(a.nbytes, 16)).upload(a)

    def zeros(self, nbytes: int) -> DevBuf:
        b = DevBuf(self, nbytes).zero()
        self.sync()
        return b

    # ---- events ----
    def event(self) -> "Event":
        return Event(self)

    # ---- kernels (one launch each) ----
    def gemv_q8(self, w: DevBuf, s: DevBuf, x: DevBuf, x_dtype: int, y: DevBuf, y_dtype: int, rows: int, cols: int) -> None:
        check(self.lib.tb_gemv_q8(self.handle, w.ptr, s.ptr, x.ptr, x_dtype, y.ptr, y_dtype, rows, cols))

    def gemv_f16(self, w: DevBuf, x: DevBuf, x_dtype: int, y: DevBuf, y_dtype: int, rows: int, cols: int) -> None:
        """tb_gemv_f16: f16 weights [rows, cols] times an f16/f32 vector, f32 accumulation."""
        check(self.lib.tb_gemv_f16(self.handle, w.ptr, x.ptr, x_dtype, y.ptr, y_dtype, rows, cols))

    def gemv_f16_norm(self, w, h, y_res, w1, w2, eps, hscale, h_out, y, y_dtype, rows, cols) -> None:
        p = lambda b: None if b is None else b.ptr
        check(self.lib.tb_gemv_f16_norm(self.handle, w.ptr, h.ptr, p(y_res), p(w1), p(w2), eps, hscale, p(h_out), y.ptr, y_dtype, rows, cols))

    def quant_q8(self, x: DevBuf, n: int, q: DevBuf, pairs: DevBuf) -> None:
        """tb_quant_q8 (the reference's quant_q8): f32 x [n] -> i8 codes [n] and f32 pairs [n / 32][2]."""
        check(self.lib.tb_quant_q8(self.handle, x.ptr, n, q.ptr, pairs.ptr))

    def gemv_q4(self, packed: DevBuf, scales: DevBuf, q: DevBuf, pairs: DevBuf, y: DevBuf, rows: int, cols: int) -> None:
        """tb_gemv_q4 (the reference's gemv_q4): Q4 weights x Q8 activations -> f32 y [rows]."""
        check(self.lib.tb_gemv_q4(self.handle, packed.ptr, scales.ptr, q.ptr, pairs.ptr, y.ptr, rows, cols))

    def geglu_q8(self, a, b, n, q, pairs) -> None:
        check(self.lib.tb_geglu_q8(self.handle, a.ptr, b.ptr, n, q.ptr, pairs.ptr))

    def norm_q8(self, h, h_out, y, w1, w2, q, pairs, length, chunks, eps, scale) -> None:
        p = lambda b: None if b is None else b.ptr
        check(self.lib.tb_norm_q8(self.handle, h.ptr, p(h_out), p(y), p(w1), p(w2), p(q), p(pairs), length, chunks, eps, scale))

    def embed_q4(self, packed, scales, tokens, rows, out, cols, scale) -> None:
        check(self.lib.tb_embed_q4(self.handle, packed.ptr, scales.ptr, tokens.ptr, rows, out.ptr, cols, scale))

    def launch(self, kernel: str, grid, block, shared_bytes, args) -> None:
        """tb_launch: the reference's Stream::launch by kernel name; args: ("p", address) | ("u", int) | ("f", float)."""
        slots = [C.c_uint64(v or 0) if k == "p" else C.c_uint32(v) if k == "u" else C.c_float(v) for k, v in args]
        table = (C.c_void_p * len(slots))(*[C.addressof(s) for s in slots])
        g, b = (C.c_uint32 * 3)(*grid), (C.c_uint32 * 3)(*block)
        check(self.lib.tb_launch(self.handle, kernel.encode(), g, b, shared_bytes, table, len(slots)))

    def gemv_q4x(self, packed: DevBuf, scales: DevBuf, x: DevBuf, x_dtype: int, y: DevBuf, rows: int, cols: int) -> None:
        """tb_gemv_q4x: Q4 weights x an f16/f32 activation that is not rounded to Q8 -> f32 y [rows]."""
        check(self.lib.tb_gemv_q4x(self.handle, packed.ptr, scales.ptr, x.ptr, x_dtype, y.ptr, rows, cols))

    def gemv_q8_norm(self, w, s, h, y_res, w1, w2, eps, hscale, h_out, y, rows, cols, geglu=False) -> None:
        p = lambda b: None if b is None else b.ptr
        check(self.lib.tb_gemv_q8_norm(self.handle, w.ptr, s.ptr, h.ptr, p(y_res), p(w1), p(w2), eps, hscale, p(h_out), y.ptr, rows, cols, int(geglu)))

    def gemv_q8_argmax(self, w, s, x, x_dtype, logits, rows, cols, scratch, state, token_out=None) -> None:
        p = lambda b: None if b is None else b.ptr
        check(self.lib.tb_gemv_q8_argmax(self.handle, w.ptr, s.ptr, x.ptr, x_dtype, p(logits), rows, cols, scratch.ptr, state.ptr, p(token_out)))

    def gemm_q8(self, w, s, a, m, n, k, out, mode=0) -> None:
        """tb_gemm_q8: out[m, n] = a[m, k] (f16) x w[n, k]^T on the tensor cores; mode 0 f32, 1 f16, 2 GeGLU."""
        check(self.lib.tb_gemm_q8(self.handle, w.ptr, s.ptr, a.ptr, m, n, k, out.ptr, mode))

    def dequant_f16(self, w, s, rows, cols, bits, out) -> None:
        """tb_dequant_f16: out f16 [rows, cols] = code * scale as the tensor-core products round it."""
        check(self.lib.tb_dequant_f16(self.handle, w.ptr, s.ptr, rows, cols, bits, out.ptr))

    def gemm_f16(self, w, a, m, n, k, out, mode=0) -> None:
        """tb_gemm_f16: the same product on f16 weights [n, k]."""
        check(self.lib.tb_gemm_f16(self.handle, w.ptr, a.ptr, m, n, k, out.ptr, mode))

    def gemm_q4(self, packed, s, a, m, n, k, out, mode=0) -> None:
        """tb_gemm_q4: the same product on the reference's Q4 weights."""
        check(self.lib.tb_gemm_q4(self.handle, packed.ptr, s.ptr, a.ptr, m, n, k, out.ptr, mode))

    def sample(self, logits, work, vocab, cfg, state, seen, out, partial, count, blocks=0) -> None:
        """tb_sample: the reference's sampler; cfg is a device buffer holding the 40-byte Sampling."""
        check(self.lib.tb_sample(self.handle, logits.ptr, work.ptr, vocab, cfg.ptr, state.ptr, seen.ptr, None if out is None else out.ptr, partial.ptr,
                                 count.ptr, blocks))

    def norm(self, h, y_res, w1, w2, n, eps, hscale, h_out, x_out) -> None:
        p = lambda b: None if b is None else b.ptr
        check(self.lib.tb_norm(self.handle, h.ptr, p(y_res), p(w1), p(w2), n, eps, hscale, p(h_out), p(x_out)))

    def embed_q8(self, w, s, token, cols, scale, out) -> None:
        check(self.lib.tb_embed_q8(self.handle, w.ptr, s.ptr, token.ptr, cols, scale, out.ptr))

    def prefill_attend(self, q, kc, vc, out, tokens, pos0, cap, window, heads, kv_heads, head_dim=256) -> None:
        """tb_prefill_attend: a chunk's tokens over their windows of the cache (the reference's flash_256 / flash_512)."""
        check(self.lib.tb_prefill_attend(self.handle, q.ptr, kc.ptr, vc.ptr, out.ptr, tokens, pos0, cap, window, heads, kv_heads, head_dim))

    def prefill_qkv(self, qkv, q_norm, k_norm, freq, q_out, kc, vc, tokens, pos0, cap, heads, kv_heads, eps, scale, head_dim=256) -> None:
        """tb_prefill_qkv: norms, RoPE, cache append and f16 queries for a chunk (kv_256/512 and query_256/512 in one launch)."""
        p = lambda b: None if b is None else b.ptr
        check(self.lib.tb_prefill_qkv(self.handle, qkv.ptr, q_norm.ptr, p(k_norm), freq.ptr, q_out.ptr, p(kc), p(vc), tokens, pos0, cap, heads, kv_heads, eps, scale,
                                      head_dim))

    def attend_decode(self, args: Attend) -> None:
        check(self.lib.tb_attend_decode(self.handle, C.byref(args)))

    def attend_project(self, args: Attend, cluster: int, w: DevBuf, s: DevBuf, rows: int, y: DevBuf) -> None:
        """tb_attend_project: attention leaving its splits (merged `cluster` at a time), then the output projection."""
        check(self.lib.tb_attend_project(self.handle, C.byref(args), cluster, w.ptr, s.ptr, rows, y.ptr))

    def set_lean(self, mode: int) -> None:
        check(self.lib.tb_context_set_lean(self.handle, mode))

    def set_dynamic(self, on: bool) -> None:
        check(self.lib.tb_context_set_dynamic(self.handle, int(on)))

    def memory(self) -> tuple[int, int]:
        """Context::memory: free and total device memory in bytes."""
        f, t = C.c_size_t(0), C.c_size_t(0)
        check(self.lib.tb_context_memory(self.handle, C.byref(f), C.byref(t)))
        return f.value, t.value

    def trim(self) -> None:
        """Context::trim: the pool's unused device memory back to the system."""
        check(self.lib.tb_context_trim(self.handle))

    def set_attn_block(self, on: bool) -> None:
        """tb_context_set_attn_block: a layer's attention half as one kernel on clusters of 16 blocks (off by default)."""
        check(self.lib.tb_context_set_attn_block(self.handle, int(on)))

    def set_flash(self, which: int) -> None:
        """tb_context_set_flash: 1 prefill attention on tcgen05 where the shape allows (default), 0 the mma.sync kernel."""
        check(self.lib.tb_context_set_flash(self.handle, which))

    def attend_decode_512(self, args: Attend) -> None:
        """tb_attend_decode_512: heads of 512 (the reference's attend_512)."""
        check(self.lib.tb_attend_decode_512(self.handle, C.byref(args)))

    def attend_512_scratch_bytes(self, heads: int, splits: int) -> int:
        return self.lib.tb_attend_512_scratch_bytes(heads, splits)

    def attend_decode_static(self, args: Attend) -> None:
        """tb_attend_decode_static: the scratch lives inside the library; nothing is allocated."""
        check(self.lib.tb_attend_decode_static(self.handle, C.byref(args)))

    def attend_scratch_bytes(self, heads: int, kv_heads: int, splits: int) -> int:
        return self.lib.tb_attend_scratch_bytes(heads, kv_heads, splits)

    def sample_greedy(self, logits, vocab, softcap, penalty, seen, allowed, scratch, state, token_out=None) -> None:
        p = lambda b: None if b is None else b.ptr
        check(self.lib.tb_sample_greedy(self.handle, logits.ptr, vocab, softcap, penalty, p(seen), p(allowed), scratch.ptr, state.ptr, p(token_out)))

    def topk(self, logits, vocab, k, idx, val) -> None:
        check(self.lib.tb_topk(self.handle, logits.ptr, vocab, k, idx.ptr, val.ptr))


class Event:
    def __init__(self, ctx: Context):
        self.ctx = ctx
        h = C.c_void_p()
        check(ctx.lib.tb_event_new(ctx.handle, C.byref(h)))
        self.handle = h.value

    def record(self) -> "Event":
        check(self.ctx.lib.tb_event_record(self.ctx.handle, self.handle))
        return self

    def sync(self) -> None:
        check(self.ctx.lib.tb_event_sync(self.handle))

    def elapsed_ms(self, end: "Event") -> float:
        ms = C.c_float(0)
        check(self.ctx.lib.tb_event_elapsed_ms(self.handle, end.handle, C.byref(ms)))
        return ms.value

    def __del__(self):
        try:
            if self.handle:
                self.ctx.lib.tb_event_free(self.handle)
        except Exception:
            pass


def gemma4_e4b_shape(layers: int = 35, ffn: int = 16384, vocab: int = 262144) -> Config:
    """The benchmark's Gemma-4-E4B-shaped configuration: 35 layers, width 2048, 8 query / 2 key-value heads of 256,
    GeGLU 16384, four sliding-window (512) layers to one global, tied vocabulary of 262144."""
    return Config(hidden=2048, ffn=ffn, heads=8, kv_heads=2, head_dim=256, vocab=vocab, layers=layers, window=512, global_=None, global_every=5,
                  theta_sliding=1e4, theta_global=1e6, fraction_global=0.25, eps=1e-6, softcap=30.0, attn_scale=1.0)


def config_from_json(text: bytes) -> Config:
    """model::Config::from_json (crates/tachyon/src/model/mod.rs:63-105): a converted model's (Hugging Face's) config.json, the
    decoder's part under `text_config` when the model is multimodal.  What this build does not run is refused as the
    reference refuses what it does not: a double-wide MLP, a mixture of experts."""
    import json

    doc = json.loads(text)
    c = doc.get("text_config", doc)
    need = ["hidden_size", "intermediate_size", "num_attention_heads", "num_key_value_heads", "head_dim", "global_head_dim", "hidden_size_per_layer_input",
            "vocab_size", "sliding_window", "rms_norm_eps"]
    for k in need:
        if not isinstance(c.get(k), (int, float)):
            raise Error(5, f"config.json: no {k}")
    heads, kv = int(c["num_attention_heads"]), int(c["num_key_value_heads"])
    global_kv = int(c.get("num_global_key_value_heads") or kv)
    for k in (kv, global_kv):
        if k == 0 or heads % k != 0 or (heads // k) % 2 != 0:
            raise Error(9, "a key-value head serving fewer than two query heads, or an odd number")
    if c.get("use_double_wide_mlp") or int(c.get("num_experts") or 0) > 0:
        raise Error(9, "a double-wide MLP or a mixture of experts")
    rope = c.get("rope_parameters") or {}
    types = c.get("layer_types") or []
    glob = np.array([t == "full_attention" for t in types], np.uint8)
    cfg = Config(hidden=int(c["hidden_size"]), ffn=int(c["intermediate_size"]), heads=heads, kv_heads=kv, head_dim=int(c["head_dim"]), vocab=int(c["vocab_size"]),
                 layers=len(types), window=int(c["sliding_window"]), global_=glob.ctypes.data if len(types) else None, global_every=0,
                 theta_sliding=float((rope.get("sliding_attention") or {}).get("rope_theta", 1e4)), theta_global=float((rope.get("full_attention") or {}).get("rope_theta", 1e6)),
                 fraction_global=float((rope.get("full_attention") or {}).get("partial_rotary_factor", 1.0)), eps=float(c["rms_norm_eps"]),
                 softcap=float(c.get("final_logit_softcapping") or 0.0), attn_scale=1.0, shared=int(c.get("num_kv_shared_layers") or 0),
                 global_head_dim=int(c["global_head_dim"]), global_kv_heads=global_kv, per_layer=int(c["hidden_size_per_layer_input"]))
    cfg._global = glob  # the structure points into it
    return cfg


def encoder_config_from_json(text: bytes, mean_pool: bool = False, dims: int = 0) -> EncoderConfig:
    """encoder::Config::from_json (crates/tachyon/src/encoder/mod.rs:61-117): a ModernBERT's config.json; GELU or SiLU gates, no
    attention biases."""
    import json

    c = json.loads(text)
    if c.get("model_type") != "modernbert":
        raise Error(9, "an encoder other than ModernBERT")
    act = c.get("hidden_activation")
    if act not in ("gelu", "silu") or c.get("attention_bias") is True:
        raise Error(9, "a ModernBERT with another activation or with biases")
    hidden, heads, inter, vocab, layers = (int(c.get(k) or 0) for k in ("hidden_size", "num_attention_heads", "intermediate_size", "vocab_size", "num_hidden_layers"))
    if not (heads > 0 and hidden % heads == 0 and (hidden // heads) % 2 == 0 and inter * vocab * layers > 0):
        raise Error(5, "config.json: an inconsistent ModernBERT shape")
    every = max(int(c.get("global_attn_every_n_layers") or 3), 1)
    types = c.get("layer_types")
    glob = np.array([t == "full_attention" for t in types] if types else [i % every == 0 for i in range(layers)], np.uint8)
    rope = c.get("rope_parameters") or {}

    def theta(kind, legacy, default):
        v = (rope.get(kind) or {}).get("rope_theta")
        return float(v if v is not None else c.get(legacy, default))

    cfg = EncoderConfig(hidden=hidden, heads=heads, inter=inter, vocab=vocab, layers=len(glob), window=int(c.get("local_attention", 128)) // 2, global_=glob.ctypes.data,
                        global_every=0, theta_global=theta("full_attention", "global_rope_theta", 160000.0), theta_local=theta("sliding_attention", "local_rope_theta", 10000.0),
                        eps=float(c.get("norm_eps", 1e-5)), gated=2 if act == "silu" else 1, mean_pool=int(mean_pool), dims=dims or hidden)
    cfg._global = glob
    return cfg


class Wpk:
    """wpk::Wpk (crates/tachyon/src/wpk/mod.rs): an open weights.wpk, its table checked; no GPU involved."""

    DTYPES = {0: np.float32, 1: np.float16, 2: np.uint16, 3: np.uint8, 4: np.int8, 5: np.uint8}  # bf16 and f8 as raw bits

    def __init__(self, path: str):
        self.lib = _lib.load()
        h = C.c_void_p()
        check(self.lib.tb_wpk_open(os.fsencode(path), C.byref(h)))
        self.handle = h.value

    def close(self) -> None:
        if self.handle:
            self.lib.tb_wpk_close(self.handle)
            self.handle = None

    def tensors(self):
        out = []
        for i in range(self.lib.tb_wpk_count(self.handle)):
            info = _lib.WpkInfo()
            check(self.lib.tb_wpk_tensor(self.handle, i, C.byref(info)))
            out.append((info.name.decode(), info.dtype, tuple(info.shape[: info.rank]), info.offset, info.bytes, info.crc32c))
        return out

    def read(self, index: int, verify: bool = True) -> np.ndarray:
        name, dtype, shape, _, nbytes, _ = self.tensors()[index]
        raw = np.zeros(nbytes, np.uint8)
        check(self.lib.tb_wpk_read(self.handle, index, raw.ctypes.data, nbytes, int(verify)))
        return raw.view(self.DTYPES[dtype]).reshape(shape)


def crc32c(data: bytes, crc: int = 0) -> int:
    buf = np.frombuffer(data, np.uint8)
    return int(_lib.load().tb_crc32c(crc, buf.ctypes.data if buf.size else None, buf.size))


def crc32c_combine(crc_a: int, crc_b: int, len_b: int) -> int:
    """tb_crc32c_combine: the checksum of A followed by B from the two checksums and B's length."""
    return int(_lib.load().tb_crc32c_combine(crc_a, crc_b, len_b))


def framed(tok: "Tokenizer", texts, capacity: int) -> list[list[int]]:
    """Encoder::embed's sequences (encoder/text.rs:40-55): the token the post-processor puts first (else <bos> or [CLS]), the
    text's tokens cut to the capacity, and the token it puts last, if any."""
    before, after = tok.frame()
    if before is None:
        for name in ("<bos>", "[CLS]"):
            try:
                before = tok.special(name)
                break
            except Error:
                pass
        if before is None:
            raise Error(5, "the tokenizer has none of ['<bos>', '[CLS]']")
    out = []
    for t in texts:
        ids = ([before] + tok.encode(t))[: capacity - (after is not None)]
        out.append(ids + ([after] if after is not None else []))
    return out


class Tokenizer:
    """token::Tokenizer (crates/tachyon/src/token/mod.rs): text to token ids and back.  Host code, no GPU."""

    def __init__(self, handle: int):
        self.lib, self.handle = _lib.load(), handle

    @classmethod
    def from_json(cls, json: bytes) -> "Tokenizer":
        h = C.c_void_p()
        check(_lib.load().tb_tokenizer_from_json(json, len(json), C.byref(h)))
        return cls(h.value)

    @classmethod
    def from_bytes(cls, data: bytes) -> "Tokenizer":
        h = C.c_void_p()
        check(_lib.load().tb_tokenizer_from_bytes(data, len(data), C.byref(h)))
        return cls(h.value)

    def to_bytes(self) -> bytes:
        n = C.c_size_t(0)
        check(self.lib.tb_tokenizer_to_bytes(self.handle, None, 0, C.byref(n)))
        buf = C.create_string_buffer(n.value)
        check(self.lib.tb_tokenizer_to_bytes(self.handle, buf, n.value, C.byref(n)))
        return buf.raw[: n.value]

    def close(self) -> None:
        if self.handle:
            self.lib.tb_tokenizer_close(self.handle)
            self.handle = None

    def __len__(self) -> int:
        return int(self.lib.tb_tokenizer_len(self.handle))

    def encode(self, text: str) -> list[int]:
        raw = text.encode("utf-8", "surrogatepass")
        ids = np.empty(len(raw) + 16, np.uint32)  # a token per byte at most, but for the spaces a pre-tokenizer prepends
        n = C.c_size_t(0)
        if self.lib.tb_tokenizer_encode(self.handle, raw, len(raw), ids.ctypes.data, ids.size, C.byref(n)) != 0 and n.value > ids.size:
            ids = np.empty(n.value, np.uint32)
            check(self.lib.tb_tokenizer_encode(self.handle, raw, len(raw), ids.ctypes.data, ids.size, C.byref(n)))
        return ids[: n.value].tolist()

    def token(self, id: int) -> bytes:
        p, n = C.c_void_p(), C.c_size_t(0)
        check(self.lib.tb_tokenizer_token(self.handle, id, C.byref(p), C.byref(n)))
        return C.string_at(p.value, n.value) if n.value else b""

    def is_special(self, id: int) -> bool:
        return bool(self.lib.tb_tokenizer_is_special(self.handle, id))

    def special(self, text: str) -> int:
        v = C.c_uint32(0)
        check(self.lib.tb_tokenizer_special(self.handle, text.encode(), C.byref(v)))
        return v.value

    def frame(self) -> tuple[int | None, int | None]:
        a, b = C.c_uint32(0), C.c_uint32(0)
        self.lib.tb_tokenizer_frame(self.handle, C.byref(a), C.byref(b))
        return tuple(None if v.value == 0xFFFFFFFF else v.value for v in (a, b))

    def decode(self, ids) -> str:
        d = Detokenizer(self)
        out = "".join(d.push(i) for i in ids) + d.finish()
        d.close()
        return out


class Detokenizer:
    """token::Detokenizer (mod.rs:603-648): tokens back into text as they come, whole characters only."""

    def __init__(self, tok: Tokenizer):
        self.tok, self.lib = tok, tok.lib
        h = C.c_void_p()
        check(self.lib.tb_detokenizer_new(C.byref(h)))
        self.handle, self.buf = h.value, C.create_string_buffer(1 << 16)

    def close(self) -> None:
        if self.handle:
            self.lib.tb_detokenizer_close(self.handle)
            self.handle = None

    def push(self, id: int) -> str:
        n = C.c_size_t(0)
        check(self.lib.tb_detokenizer_push(self.handle, self.tok.handle, id, self.buf, len(self.buf), C.byref(n)))
        return self.buf.raw[: n.value].decode("utf-8")

    def finish(self) -> str:
        n = C.c_size_t(0)
        check(self.lib.tb_detokenizer_finish(self.handle, self.buf, len(self.buf), C.byref(n)))
        return self.buf.raw[: n.value].decode("utf-8")


ROLES = {"system": 0, "user": 1, "model": 2, "assistant": 2}


class ChatTemplate:
    """token::Chat (token/chat.rs): Gemma 4's chat template over a tokenizer, text messages only."""

    def __init__(self, tok: Tokenizer, template: str | None = None):
        self.tok, self.lib, self.chat = tok, tok.lib, _lib.Chat()
        check(self.lib.tb_chat_gemma4(tok.handle, C.byref(self.chat)))
        if template is not None:
            raw = template.encode()
            check(self.lib.tb_chat_with_template(tok.handle, C.byref(self.chat), raw, len(raw)))

    def end_of_turn(self) -> int:
        return self.chat.end

    def encode(self, messages, think: bool = False) -> list[int]:
        """messages: [(role, text)] with role "system", "user", "model" (or "assistant")."""
        raws = [text.encode("utf-8") for _, text in messages]
        arr = (_lib.Message * max(len(messages), 1))()
        for i, ((role, _), raw) in enumerate(zip(messages, raws)):
            arr[i].role, arr[i].text, arr[i].bytes = ROLES[role], C.cast(C.c_char_p(raw), C.c_void_p), len(raw)
        n = C.c_size_t(0)
        check(self.lib.tb_chat_encode(self.tok.handle, C.byref(self.chat), arr, len(messages), int(think), None, 0, C.byref(n)))
        ids = np.empty(max(n.value, 1), np.uint32)
        check(self.lib.tb_chat_encode(self.tok.handle, C.byref(self.chat), arr, len(messages), int(think), ids.ctypes.data, ids.size, C.byref(n)))
        return ids[: n.value].tolist()


class WpkWriter:
    """wpk::Writer (crates/tachyon/src/wpk/mod.rs:270-337): writes a `.wpk` tensor by tensor, each on a 4 KiB boundary, then the
    table and the header.  Host code; the checksums come from tb_crc32c."""

    ALIGN = 4096
    DTYPES = {"f32": (0, 4), "f16": (1, 2), "bf16": (2, 2), "f8e4m3": (3, 1), "i8": (4, 1), "u8": (5, 1)}

    def __init__(self, path: str):
        self.f = open(path, "wb")
        self.f.write(b"\0" * self.ALIGN)
        self.table, self.data_len = [], 0

    def add(self, name: str, dtype: str, shape, raw) -> None:
        import struct

        raw = memoryview(raw).cast("B")
        code, size = self.DTYPES[dtype]
        n = size
        for d in shape:
            n *= int(d)
        if n != len(raw):
            raise ValueError(f"{name}: {len(raw)} bytes for {dtype} {tuple(shape)}")
        entry = struct.pack("<H", len(name.encode())) + name.encode() + bytes([code, len(shape)])
        entry += b"".join(struct.pack("<Q", int(v)) for v in list(shape) + [self.data_len, len(raw)]) + struct.pack("<I", crc32c(raw))
        self.table.append(entry)
        self.f.write(raw)
        pad = -len(raw) % self.ALIGN
        self.f.write(b"\0" * pad)
        self.data_len += len(raw) + pad

    def close(self) -> None:
        import struct

        table = b"".join(self.table)
        self.f.write(table)
        head = b"TACHYWPK" + struct.pack("<QQQQ", 1 | len(self.table) << 32, self.data_len, self.ALIGN + self.data_len, len(table))
        head += struct.pack("<I", crc32c(table))
        head += struct.pack("<I", crc32c(head))
        self.f.seek(0)
        self.f.write(head)
        self.f.close()

    def __enter__(self):
        return self

    def __exit__(self, *exc):
        self.close()


class Parked:
    """model::Parked (decode.rs:101-109, 449-469): a model in the host-RAM tier."""

    def __init__(self, ctx: Context, cfg: Config, settings: Settings, handle: int):
        self.ctx, self.cfg, self.settings, self.lib, self.handle = ctx, cfg, settings, ctx.lib, handle

    def bytes(self) -> int:
        return int(self.lib.tb_parked_bytes(self.handle))

    def resume(self, context: int | None = None, chunk: int | None = None, keep_logits: bool | None = None, prefill_copy: int | None = None) -> "Decoder":
        """Parked::resume: back to VRAM with these settings (those not given stay as they were); this object is spent on success."""
        old = self.settings
        st = Settings(context=old.context if context is None else context, chunk=old.chunk if chunk is None else chunk,
                      keep_logits=old.keep_logits if keep_logits is None else int(keep_logits), fused=old.fused, weight_bits=old.weight_bits,
                      host_table=old.host_table, prefill_copy=old.prefill_copy if prefill_copy is None else prefill_copy)
        h = C.c_void_p()
        check(self.lib.tb_parked_resume(self.handle, C.byref(st), C.byref(h)))
        self.handle = None
        return Decoder._adopt(self.ctx, self.cfg, st, h.value)

    def close(self) -> None:
        if self.handle:
            self.lib.tb_parked_close(self.handle)
            self.handle = None


TIER_VRAM, TIER_HOST, TIER_DISK = 0, 1, 2
FOR_GOOD = 2**64 - 1


class Engine:
    """Engine's model residency (crates/tachyon/src/engine.rs:190-453): load, decoder, feed, tier, models, unload, expire; encoders
    held by name with load_encoder, embed."""

    def __init__(self, ctx: Context, vram_limit: int = 0, host_limit: int = 0):
        self.ctx, self.lib = ctx, ctx.lib
        h = C.c_void_p()
        check(self.lib.tb_engine_new(ctx.handle, vram_limit, host_limit, C.byref(h)))
        self.handle = h.value
        self.loaded: dict[str, tuple[Config, Settings]] = {}

    def close(self) -> None:
        if self.handle:
            self.lib.tb_engine_close(self.handle)
            self.handle = None

    def load(self, name: str, cfg: Config, weights: str, host: str | None = None, context: int = 4096, chunk: int = 512, keep_alive_ms: int = 300_000,
             pin: bool = False, keep_logits: bool = False, weight_bits: int = 8, host_table: bool = False, prefill_copy: int = 0) -> None:
        st = Settings(context=context, chunk=chunk, keep_logits=int(keep_logits), fused=0, weight_bits=weight_bits, host_table=int(host_table), prefill_copy=prefill_copy)
        load = Load(settings=st, keep_alive_ms=keep_alive_ms, pin=int(pin))
        check(self.lib.tb_engine_load(self.handle, name.encode(), C.byref(cfg), C.byref(load), os.fsencode(weights), os.fsencode(host) if host else None))
        self.loaded[name] = (cfg, st)

    def load_dir(self, name: str, directory: str, **how):
        """Engine::load of a converted model's directory (engine.rs:203-232): config.json tells a decoder from an encoder; weights.wpk,
        host.wpk if there is one, tokenizer.tok.  A decoder comes in the reference's converted format (four-bit weights, the
        per-layer table in pinned host memory).  Returns the model's tokenizer, or None if the directory has none; a decoder's
        chat template is kept for Engine.chat."""
        import json

        def read(file):
            path = os.path.join(directory, file)
            return open(path, "rb").read() if os.path.exists(path) else None

        config = read("config.json")
        if config is None:
            raise Error(11, f"{directory}: no config.json")
        stored = read("tokenizer.tok")
        tok = Tokenizer.from_bytes(stored) if stored is not None else None
        weights, host = os.path.join(directory, "weights.wpk"), os.path.join(directory, "host.wpk")
        host = host if os.path.exists(host) else None
        if json.loads(config).get("model_type") == "modernbert":
            self.load_encoder(name, encoder_config_from_json(config, mean_pool=how.pop("mean_pool", False), dims=how.pop("dims", 0)), weights, host, **how)
            return tok
        cfg = config_from_json(config)
        self.load(name, cfg, weights, host, weight_bits=how.pop("weight_bits", 4), host_table=how.pop("host_table", host is not None and cfg.per_layer > 0), **how)
        if tok is not None:
            template = read("chat_template.jinja")
            self.templates = getattr(self, "templates", {})
            self.templates[name] = ChatTemplate(tok, template.decode("utf-8") if template is not None else None)
        return tok

    def unload(self, name: str) -> bool:
        was = C.c_int(0)
        check(self.lib.tb_engine_unload(self.handle, name.encode(), C.byref(was)))
        self.loaded.pop(name, None)
        return bool(was.value)

    def decoder(self, name: str) -> "Decoder":
        h = C.c_void_p()
        check(self.lib.tb_engine_decoder(self.handle, name.encode(), C.byref(h)))
        cfg, st = self.loaded[name]
        return Decoder._adopt(self.ctx, cfg, st, h.value, owned=False)

    def feed(self, name: str, tokens) -> int:
        t = np.ascontiguousarray(tokens, np.uint32)
        first = C.c_uint32(0)
        check(self.lib.tb_engine_feed(self.handle, name.encode(), t.ctypes.data, t.size, C.byref(first)))
        return first.value

    def tier(self, name: str) -> int:
        t = C.c_int(0)
        check(self.lib.tb_engine_tier(self.handle, name.encode(), C.byref(t)))
        return t.value

    def models(self) -> list[dict]:
        n = C.c_size_t(0)
        check(self.lib.tb_engine_models(self.handle, None, 0, C.byref(n)))
        arr = (Loaded * max(n.value, 1))()
        check(self.lib.tb_engine_models(self.handle, arr, n.value, C.byref(n)))
        return [{"name": arr[i].name.decode(), "tier": arr[i].tier, "vram": arr[i].vram, "left_ms": arr[i].left_ms} for i in range(n.value)]

    def expire(self) -> None:
        check(self.lib.tb_engine_expire(self.handle))

    def chat(self, name: str, tok: "Tokenizer", messages, think: bool = False, max_tokens: int = 256, template: "ChatTemplate | None" = None):
        """Engine::chat and TokenStream::next_text (engine.rs:326-337, 515-536): the conversation through the chat template, every
        prompt token but the last through prefill and the last through a step, then the answer's text piece by piece, whole
        characters only, until the model ends its turn, `max_tokens` are out or the context is full."""
        chat = template or getattr(self, "templates", {}).get(name) or ChatTemplate(tok)
        prompt = chat.encode(messages, think=think)
        context = self.loaded[name][1].context
        if len(prompt) >= context:
            raise Error(3, f"the prompt's {len(prompt)} tokens do not fit the context of {context}")
        ends = {chat.end_of_turn()}
        for mark in ("<eos>", "<end_of_turn>"):
            try:
                ends.add(tok.special(mark))
            except Error:
                pass
        token = self.feed(name, prompt)
        dec, detok, left = self.decoder(name), Detokenizer(tok), min(max_tokens, context - len(prompt))
        try:
            while left > 0 and token not in ends:
                left -= 1
                text = detok.push(token) if token < len(tok) else ""
                if text:
                    yield text
                if left > 0:
                    token = dec.step(token)
            text = detok.finish()
            if text:
                yield text
        finally:
            detok.close()

    def load_encoder(self, name: str, cfg: EncoderConfig, weights: str, host: str | None = None, tokens: int = 4096, sequences: int = 64,
                     keep_alive_ms: int = 300_000, pin: bool = False) -> None:
        """tb_engine_load_encoder: the encoder of these files held as `name`, decoders moved out to make room."""
        check(self.lib.tb_engine_load_encoder(self.handle, name.encode(), C.byref(cfg), tokens, sequences, keep_alive_ms, int(pin), os.fsencode(weights),
                                              os.fsencode(host) if host else None))
        self.dims = getattr(self, "dims", {})
        self.dims[name] = cfg.dims
        self.capacity = getattr(self, "capacity", {})
        self.capacity[name] = tokens

    def embed_texts(self, name: str, tok: "Tokenizer", texts) -> np.ndarray:
        """Engine::embed (engine.rs:258-262) from texts: framed and cut as Encoder::embed does (encoder/text.rs:40-55)."""
        return self.embed(name, framed(tok, texts, self.capacity[name]))

    def embed(self, name: str, sequences) -> np.ndarray:
        """tb_engine_embed: embeddings [len(sequences), dims] of lists of token ids by the held encoder `name`."""
        lens = np.array([len(q) for q in sequences], np.uint32)
        ids = np.concatenate([np.asarray(q, np.uint32) for q in sequences])
        out = np.zeros((len(sequences), getattr(self, "dims", {}).get(name, 0)), np.float32)
        check(self.lib.tb_engine_embed(self.handle, name.encode(), ids.ctypes.data, lens.ctypes.data, len(sequences), out.ctypes.data if out.size else None))
        return out

    def usage(self) -> tuple[int, int]:
        v, h = C.c_size_t(0), C.c_size_t(0)
        check(self.lib.tb_engine_usage(self.handle, C.byref(v), C.byref(h)))
        return v.value, h.value


def decoder_footprint(ctx: Context, cfg: Config, context: int = 4096, chunk: int = 512, keep_logits: bool = False, weight_bits: int = 8,
                      host_table: bool = False, prefill_copy: int = 0) -> int:
    """tb_decoder_footprint: the device memory such a decoder takes, nothing allocated."""
    st = Settings(context=context, chunk=chunk, keep_logits=int(keep_logits), fused=0, weight_bits=weight_bits, host_table=int(host_table), prefill_copy=prefill_copy)
    n = C.c_size_t(0)
    check(ctx.lib.tb_decoder_footprint(ctx.handle, C.byref(cfg), C.byref(st), C.byref(n)))
    return n.value


def encoder_footprint(ctx: Context, cfg: EncoderConfig, tokens: int = 4096, sequences: int = 64, f16_matrices: bool = False) -> int:
    """tb_encoder_footprint: the device memory such an encoder takes, nothing allocated."""
    n = C.c_size_t(0)
    check(ctx.lib.tb_encoder_footprint(ctx.handle, C.byref(cfg), tokens, sequences, int(f16_matrices), C.byref(n)))
    return n.value


class Decoder:
    """model::Decoder (crates/tachyon/src/model/decode.rs:79-99): open, load or fill, build, then step."""

    def __init__(self, ctx: Context, cfg: Config, context: int = 4096, chunk: int = 0, keep_logits: bool = False, fused: bool = False,
                 weight_bits: int = 8, host_table: bool = False, prefill_copy: int = 0):
        self.ctx, self.cfg, self.lib = ctx, cfg, ctx.lib
        self.settings = Settings(context=context, chunk=chunk, keep_logits=int(keep_logits), fused=int(fused), weight_bits=weight_bits,
                                 host_table=int(host_table), prefill_copy=prefill_copy)
        h = C.c_void_p()
        check(self.lib.tb_decoder_open(ctx.handle, C.byref(cfg), C.byref(self.settings), C.byref(h)))
        self.handle = h.value

    @classmethod
    def _adopt(cls, ctx: Context, cfg: Config, settings: Settings, handle: int, owned: bool = True) -> "Decoder":
        """A decoder the library made (tb_parked_resume, tb_engine_decoder); `owned` False: the engine's, never closed here."""
        d = cls.__new__(cls)
        d.ctx, d.cfg, d.lib, d.settings, d.handle, d.owned = ctx, cfg, ctx.lib, settings, handle, owned
        return d

    def close(self) -> None:
        if self.handle and getattr(self, "owned", True):
            self.lib.tb_decoder_close(self.handle)
        self.handle = None

    def park(self) -> "Parked":
        """Decoder::park (decode.rs:235-247): weights to pinned host memory, the device memory freed; this object is spent."""
        h = C.c_void_p()
        check(self.lib.tb_decoder_park(self.handle, C.byref(h)))
        self.handle = None
        return Parked(self.ctx, self.cfg, self.settings, h.value)

    def bytes(self) -> int:
        return int(self.lib.tb_decoder_bytes(self.handle))

    def parked_bytes(self) -> int:
        return int(self.lib.tb_decoder_parked_bytes(self.handle))

    def shadow_bytes(self) -> int:
        return int(self.lib.tb_decoder_shadow_bytes(self.handle))

    def drop_shadow(self) -> None:
        self.lib.tb_decoder_drop_shadow(self.handle)

    def load(self, name: str, a: np.ndarray) -> None:
        a = np.ascontiguousarray(a)
        check(self.lib.tb_decoder_load(self.handle, name.encode(), a.ctypes.data, a.nbytes))

    def set_sampling(self, softcap=0.0, temperature=0.0, top_p=1.0, min_p=0.0, penalty=1.0, top_k=0, allowed: int = 0, seed=0) -> None:
        """tb_decoder_set_sampling with the reference's Sampling fields (defaults: the largest logit)."""
        raw = np.zeros(40, np.uint8)
        raw[:20].view(np.float32)[:] = [softcap, temperature, top_p, min_p, penalty]
        raw[20:24].view(np.uint32)[0] = top_k
        raw[24:40].view(np.uint64)[:] = [allowed, seed]
        check(self.lib.tb_decoder_set_sampling(self.handle, raw.ctypes.data))

    def load_wpk(self, path: str, verify: bool = True) -> None:
        """tb_decoder_load_wpk: every tensor of a converted model's weights.wpk, by its name."""
        check(self.lib.tb_decoder_load_wpk(self.handle, os.fsencode(path), int(verify)))

    def fill_random(self, seed: int) -> None:
        check(self.lib.tb_decoder_fill_random(self.handle, seed))

    def fill_cache(self, seed: int, positions: int) -> None:
        check(self.lib.tb_decoder_fill_cache(self.handle, seed, positions))

    def build(self) -> None:
        check(self.lib.tb_decoder_build(self.handle))

    def reset(self) -> None:
        check(self.lib.tb_decoder_reset(self.handle))

    def step(self, token: int) -> int:
        out = C.c_uint32(0)
        check(self.lib.tb_decoder_step(self.handle, token, C.byref(out)))
        return out.value

    def start(self, token: int) -> None:
        check(self.lib.tb_decoder_start(self.handle, token))

    def next_token(self) -> int:
        out = C.c_uint32(0)
        check(self.lib.tb_decoder_next_token(self.handle, C.byref(out)))
        return out.value

    def stop(self) -> None:
        check(self.lib.tb_decoder_stop(self.handle))

    def run(self, token: int, steps: int, want_tokens: bool = True):
        out = np.zeros(steps, np.uint32) if want_tokens else None
        check(self.lib.tb_decoder_run(self.handle, token, steps, None if out is None else out.ctypes.data))
        return out

    def prefill(self, tokens) -> None:
        t = np.ascontiguousarray(tokens, np.uint32)
        check(self.lib.tb_decoder_prefill(self.handle, t.ctypes.data, t.size))

    def logits(self) -> np.ndarray:
        out = np.empty(self.cfg.vocab, np.float32)
        check(self.lib.tb_decoder_logits(self.handle, out.ctypes.data))
        return out

    def hidden(self) -> np.ndarray:
        out = np.empty(self.cfg.hidden, np.float32)
        check(self.lib.tb_decoder_hidden(self.handle, out.ctypes.data))
        return out

    def timeline(self, token: int) -> np.ndarray:
        """One step outside the graphs; returns ns stamps [2 blocks, phases, 4] (start, -, end of work, after barrier)."""
        n = C.c_uint32(0)
        check(self.lib.tb_decoder_timeline(self.handle, token, None, C.byref(n)))
        out = np.zeros((2, n.value, 4), np.uint64)
        check(self.lib.tb_decoder_timeline(self.handle, token, out.ctypes.data, C.byref(n)))
        return out

    @property
    def position(self) -> int:
        p = C.c_uint32(0)
        check(self.lib.tb_decoder_position(self.handle, C.byref(p)))
        return p.value

    def step_bytes(self) -> tuple[int, int]:
        w, kv = C.c_uint64(0), C.c_uint64(0)
        check(self.lib.tb_decoder_step_bytes(self.handle, C.byref(w), C.byref(kv)))
        return w.value, kv.value

    @property
    def step_launches(self) -> int:
        n = C.c_uint32(0)
        check(self.lib.tb_decoder_step_launches(self.handle, C.byref(n)))
        return n.value


def granite_311m_shape(layers: int = 22, vocab: int = 50368) -> EncoderConfig:
    """The benchmark's Granite-embedding-311m-shaped encoder: 22 layers, width 768, 12 heads of 64, plain GELU FFN of 3072,
    every third layer global and the others within 64 positions either way, mean-pooled, 256 dimensions kept."""
    return EncoderConfig(hidden=768, heads=12, inter=3072, vocab=vocab, layers=layers, window=64, global_=None, global_every=3, theta_global=160000.0,
                         theta_local=10000.0, eps=1e-5, gated=0, mean_pool=1, dims=256)


class Encoder:
    """encoder::Encoder (crates/tachyon/src/encoder/run.rs:68-90): open, load or fill, then embed packed batches."""

    def __init__(self, ctx: Context, cfg: EncoderConfig, tokens: int = 4096, sequences: int = 64):
        self.ctx, self.cfg, self.lib = ctx, cfg, ctx.lib
        h = C.c_void_p()
        check(self.lib.tb_encoder_open(ctx.handle, C.byref(cfg), tokens, sequences, C.byref(h)))
        self.handle, self.tokens = h.value, tokens

    def close(self) -> None:
        if self.handle:
            self.lib.tb_encoder_close(self.handle)
            self.handle = None

    def load(self, name: str, a: np.ndarray) -> None:
        a = np.ascontiguousarray(a)
        check(self.lib.tb_encoder_load(self.handle, name.encode(), a.ctypes.data, a.nbytes))

    def fill_random(self, seed: int) -> None:
        check(self.lib.tb_encoder_fill_random(self.handle, seed))

    def bytes(self) -> int:
        """tb_encoder_bytes: the VRAM the encoder holds."""
        return int(self.lib.tb_encoder_bytes(self.handle))

    def load_wpk(self, path: str, verify: bool = True) -> None:
        """tb_encoder_load_wpk: every tensor of a converted encoder's file, by its name."""
        check(self.lib.tb_encoder_load_wpk(self.handle, os.fsencode(path), int(verify)))

    def embed(self, sequences) -> np.ndarray:
        """Embeddings [len(sequences), dims] of lists of token ids, packed into batches of at most the capacity."""
        lens = np.array([len(q) for q in sequences], np.uint32)
        ids = np.concatenate([np.asarray(q, np.uint32) for q in sequences])
        out = np.zeros((len(sequences), self.cfg.dims), np.float32)
        check(self.lib.tb_encoder_embed(self.handle, ids.ctypes.data, lens.ctypes.data, len(sequences), out.ctypes.data))
        return out

    def embed_texts(self, tok: "Tokenizer", texts) -> np.ndarray:
        """Encoder::embed (encoder/text.rs:40-65): the texts framed and cut to the capacity, then embed."""
        return self.embed(framed(tok, texts, self.tokens))

    def graphs(self) -> int:
        return int(self.lib.tb_encoder_graphs(self.handle))

    def hidden(self) -> np.ndarray:
        """The last batch's final hidden states [its tokens, hidden]."""
        out = np.zeros((int(self.lib.tb_encoder_batch_tokens(self.handle)), self.cfg.hidden), np.float32)
        check(self.lib.tb_encoder_hidden(self.handle, out.ctypes.data))
        return out
