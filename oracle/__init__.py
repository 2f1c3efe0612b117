"""ctypes binding of the CPU oracle (``oracle/tachyon_oracle.c``).

Test infrastructure only: imported by ``tests/``, by ``__graft_entry__.smoke()`` and by the CPU-baseline legs of
``bench.py``.  The shipped package never imports it.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "_build", "liboracle.so")


def build(force: bool = False) -> str:
    """Compiles the oracle with gcc when the library is missing or older than its source."""
    src = os.path.join(_HERE, "tachyon_oracle.c")
    if force or not os.path.exists(_SO) or os.path.getmtime(_SO) < os.path.getmtime(src):
        subprocess.run(["make", "-C", _HERE, "-s", "-B"], check=True)
    return _SO


_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        _lib = C.CDLL(build())
        _declare(_lib)
    return _lib


class Config(C.Structure):
    _fields_ = [(n, C.c_int32) for n in ("hidden", "ffn", "heads", "kv_heads", "head_dim", "vocab", "layers", "window", "context")] + [
        (n, C.c_float) for n in ("theta_sliding", "theta_global", "fraction_global", "eps", "softcap", "attn_scale", "embed_scale")
    ] + [("weight_bits", C.c_int32), ("global_head_dim", C.c_int32), ("global_kv_heads", C.c_int32), ("per_layer", C.c_int32)]


class Layer(C.Structure):
    _fields_ = (
        [(n, C.c_void_p) for n in ("qkv", "o", "gate_up", "down", "qkv_s", "o_s", "gate_up_s", "down_s")]
        + [(n, C.c_void_p) for n in ("q_norm", "k_norm", "input_ln", "post_attn_ln", "pre_ffn_ln", "post_ffn_ln")]
        + [("layer_scalar", C.c_float), ("global_", C.c_int32), ("kc", C.c_void_p), ("vc", C.c_void_p), ("cap", C.c_int32), ("shared", C.c_int32)]
        + [(n, C.c_void_p) for n in ("pl_gate", "pl_proj", "pl_gate_s", "pl_proj_s", "post_pl_ln")]
    )


class Model(C.Structure):
    _fields_ = [("cfg", Config), ("embed", C.c_void_p), ("embed_s", C.c_void_p), ("norm", C.c_void_p), ("layers", C.POINTER(Layer))] + [
        (n, C.c_void_p) for n in ("embed_pl", "pl_model_proj", "embed_pl_s", "pl_model_proj_s", "pl_norm")]


class EncConfig(C.Structure):
    _fields_ = [(n, C.c_int32) for n in ("hidden", "heads", "inter", "vocab", "layers", "window", "gated")] + [
        (n, C.c_float) for n in ("theta_global", "theta_local", "eps")] + [("global_", C.c_void_p)]


class EncLayer(C.Structure):
    _fields_ = [(n, C.c_void_p) for n in ("attn_norm", "qkv", "o", "mlp_norm", "up", "down")]


def _declare(l: C.CDLL) -> None:
    vp, sz, u32, u64, i32, f32, f64 = C.c_void_p, C.c_size_t, C.c_uint32, C.c_uint64, C.c_int, C.c_float, C.c_double
    sig = {
        "tbo_f16_bits": (C.c_uint16, [f32]),
        "tbo_f16_value": (f32, [C.c_uint16]),
        "tbo_q4": (None, [vp, sz, vp, vp]),
        "tbo_q8_blocks": (None, [vp, sz, i32, vp, vp]),
        "tbo_q8p_pairs": (None, [vp, sz]),
        "tbo_product_q4": (None, [vp, vp, vp, sz, sz, vp, vp]),
        "tbo_sample_draw": (C.c_uint32, [vp, sz, vp, C.c_uint32, vp, vp, vp]),
        "tbo_gemv_q4": (None, [vp, vp, vp, vp, sz, sz, vp]),
        "tbo_gemv_q4x": (None, [vp, vp, vp, sz, sz, vp, vp]),
        "tbo_gemv_q8": (None, [vp, vp, vp, sz, sz, vp, vp, vp]),
        "tbo_normalize": (None, [vp, sz, vp, f64]),
        "tbo_rotate": (None, [vp, sz, vp, u32]),
        "tbo_rope_freq": (None, [f32, i32, f32, vp]),
        "tbo_gelu_tanh": (f64, [f64]),
        "tbo_norm_step": (None, [vp, vp, vp, vp, sz, f64, f64, vp, vp]),
        "tbo_attend_decode": (None, [vp, vp, vp, vp, vp, vp, u32, u32, u32, i32, i32, i32, i32, f64, f64, vp]),
        "tbo_sample_transform": (f64, [f32, sz, f32, f32, f32, vp, vp]),
        "tbo_sample_greedy": (u32, [vp, sz, f32, f32, vp, vp, vp]),
        "tbo_sample_topk": (None, [vp, sz, i32, vp, vp]),
        "tbo_fill_codes": (None, [u64, u64, vp, sz]),
        "tbo_fill_scales": (None, [u64, u64, vp, sz, f32]),
        "tbo_fill_uniform": (None, [u64, u64, vp, sz, f32, f32]),
        "tbo_fill_gauss_f16": (None, [u64, u64, vp, sz, f32]),
        "tbo_fill_gauss_f32": (None, [u64, u64, vp, sz, f32]),
        "tbo_decoder_step": (C.c_int32, [C.POINTER(Model), u32, u32, vp, i32, vp]),
        "tbo_gemv_q4_narrow": (None, [vp, vp, vp, vp, sz, sz, vp]),
        "tbo_gemm_q8e": (None, [vp, vp, vp, vp, vp, sz, sz, sz, vp]),
        "tbo_encoder_forward": (None, [C.POINTER(EncConfig), vp, vp, C.POINTER(EncLayer), vp, vp, sz, vp]),
        "tbo_erf_as": (f32, [f32]),
        "tbo_threads": (i32, []),
        "tbo_set_threads": (None, [i32]),
    }
    for name, (res, args) in sig.items():
        f = getattr(l, name)
        f.restype, f.argtypes = res, args


def ptr(a):
    """Address of a C-contiguous numpy array, or None."""
    if a is None:
        return None
    assert a.flags["C_CONTIGUOUS"]
    return a.ctypes.data


# ---------------------------------------------------------------------------------------------------------------
# numpy-facing helpers
# ---------------------------------------------------------------------------------------------------------------

def f16_bits(v: float) -> int:
    return int(lib().tbo_f16_bits(float(np.float32(v))))


def f16_value(h: int) -> float:
    return float(lib().tbo_f16_value(int(h)))


def q4(w: np.ndarray):
    w = np.ascontiguousarray(w, dtype=np.float32).ravel()
    packed, scales = np.zeros(w.size // 2, np.uint8), np.zeros(w.size // 64, np.uint16)
    lib().tbo_q4(ptr(w), w.size, ptr(packed), ptr(scales))
    return packed, scales


def q8(x: np.ndarray, block: int = 32):
    x = np.ascontiguousarray(x, dtype=np.float32).ravel()
    q, pairs = np.zeros(x.size, np.int8), np.zeros((x.size // block, 2), np.float32)
    lib().tbo_q8_blocks(ptr(x), x.size, block, ptr(q), ptr(pairs))
    return q, pairs


def q8p(x: np.ndarray):
    q, pairs = q8(x, 64)
    lib().tbo_q8p_pairs(ptr(pairs), pairs.shape[0])
    return q, pairs


def q8e(x: np.ndarray):
    """quant::q8e (crates/tachyon/src/quant.rs:107-115): int8 codes and an f32 scale per block of 64, amax / 127, ties to
    even; what quant_f16 computes from f16 rows (ptx/encoder.rs:670-743)."""
    q, pairs = q8(x, 64)
    return q, np.ascontiguousarray(pairs[:, 0])


def gemm_q8e(aq, sa, wq, sw, rows: int, bias=None) -> np.ndarray:
    """The reference's gemm_q8 sums, bit for bit: f32 [tokens, rows] from Q8E activations and weights, bias added."""
    aq, wq = np.ascontiguousarray(aq, np.int8), np.ascontiguousarray(wq, np.int8)
    sa, sw = np.ascontiguousarray(sa, np.float32), np.ascontiguousarray(sw, np.float32)
    cols = wq.size // rows
    tokens = aq.size // cols
    b = None if bias is None else np.ascontiguousarray(bias, np.float32)
    y = np.zeros((tokens, rows), np.float32)
    lib().tbo_gemm_q8e(ptr(aq), ptr(sa), ptr(wq), ptr(sw), ptr(b) if b is not None else None, tokens, rows, cols, ptr(y))
    return y


def rope_table(theta: float, positions: int, d: int) -> np.ndarray:
    """rope_tables (crates/tachyon/src/encoder/run.rs:523-537): f32 [positions, d/2, 2] of cos and sin of p * theta^(-2j/d),
    computed in f64 and rounded once."""
    j = np.arange(d // 2, dtype=np.float64)
    angle = np.arange(positions, dtype=np.float64)[:, None] * np.float64(np.float32(theta)) ** (-2.0 * j / d)[None, :]
    return np.stack([np.cos(angle), np.sin(angle)], axis=2).astype(np.float32)


def product_q4(packed, scales, x, rows):
    x = np.ascontiguousarray(x, dtype=np.float32)
    s, b = np.zeros(rows, np.float64), np.zeros(rows, np.float64)
    lib().tbo_product_q4(ptr(packed), ptr(scales), ptr(x), rows, x.size, ptr(s), ptr(b))
    return s, b


def gemv_q4(packed, scales, q, pairs, rows: int):
    """The reference's gemv_q4 kernel, bit for bit: f32 y [rows] from Q4 weights and Q8 activations (codes, pairs)."""
    q = np.ascontiguousarray(q, np.int8)
    pairs = np.ascontiguousarray(pairs, np.float32)
    y = np.zeros(rows, np.float32)
    lib().tbo_gemv_q4(ptr(packed), ptr(scales), ptr(q), ptr(pairs), rows, q.size, ptr(y))
    return y


def gemv_q4_narrow(packed, scales, q, pairs, rows: int):
    """The reference's gemv_q4_narrow kernel, bit for bit: rows of at most 256 weights, eight lanes a row."""
    q = np.ascontiguousarray(q, np.int8)
    pairs = np.ascontiguousarray(pairs, np.float32)
    y = np.zeros(rows, np.float32)
    lib().tbo_gemv_q4_narrow(ptr(packed), ptr(scales), ptr(q), ptr(pairs), rows, q.size, ptr(y))
    return y


def gemv_q4x(packed, scales, x, rows: int):
    """(f64 y, bound) of Q4 weights times an f32 vector that is not rounded to Q8."""
    x = np.ascontiguousarray(x, np.float32)
    y, b = np.zeros(rows, np.float64), np.zeros(rows, np.float64)
    lib().tbo_gemv_q4x(ptr(packed), ptr(scales), ptr(x), rows, x.size, ptr(y), ptr(b))
    return y, b


def gemv_q8(w: np.ndarray, scales: np.ndarray, x: np.ndarray):
    """(f32-accumulated y, f64 y, bound) for int8 ``w`` [rows, cols], f16-bit ``scales`` [rows, cols/32], f32 ``x``."""
    rows, cols = w.shape
    w, scales = np.ascontiguousarray(w, np.int8), np.ascontiguousarray(scales, np.uint16)
    x = np.ascontiguousarray(x, np.float32)
    y, e, b = np.zeros(rows, np.float32), np.zeros(rows, np.float64), np.zeros(rows, np.float64)
    lib().tbo_gemv_q8(ptr(w), ptr(scales), ptr(x), rows, cols, ptr(y), ptr(e), ptr(b))
    return y, e, b


def gemv_f16(w_bits: np.ndarray, x: np.ndarray):
    """(f64 y, bound) for f16 weights given as their bits [rows, cols] and an f32 vector: the product the reference's gemm_f16
    computes for one token (crates/tachyon/src/ptx/encoder.rs:157-203), restated as a plain f64 sum; bound is the sum of the
    terms' magnitudes, the measure the reference's tolerance is stated in (tests/common/mod.rs:95-112)."""
    w = np.ascontiguousarray(w_bits, np.uint16).view(np.float16).astype(np.float64)
    x = np.asarray(x, np.float32).astype(np.float64)
    return w @ x, np.abs(w) @ np.abs(x)


def rope_freq(theta: float, d: int, fraction: float) -> np.ndarray:
    f = np.zeros(d // 2, np.float32)
    lib().tbo_rope_freq(theta, d, fraction, ptr(f))
    return f


def norm_step(h, y, w1, w2, eps, scale):
    h = np.ascontiguousarray(h, np.float32)
    ho, xo = np.zeros(h.size, np.float64), np.zeros(h.size, np.float64)
    cv = lambda a: None if a is None else np.ascontiguousarray(a, np.float32)
    y, w1, w2 = cv(y), cv(w1), cv(w2)
    lib().tbo_norm_step(ptr(h), ptr(y), ptr(w1), ptr(w2), h.size, eps, scale, ptr(ho), ptr(xo))
    return ho, xo


def attend_decode(qkv, qn, kn, freq, kc, vc, pos, cap, window, fresh, heads, kv_heads, d, scale, eps=1e-6):
    """Returns f64 out [heads*d]; ``kc``/``vc`` (uint16 f16 bits, [kv_heads, cap, d]) are updated in place when fresh."""
    qkv = np.ascontiguousarray(qkv, np.float32)
    out = np.zeros(heads * d, np.float64)
    cv = lambda a: None if a is None else np.ascontiguousarray(a, np.float32)
    qn, kn, freq = cv(qn), cv(kn), cv(freq)
    assert kc.dtype == np.uint16 and vc.dtype == np.uint16
    lib().tbo_attend_decode(ptr(qkv), ptr(qn), ptr(kn), ptr(freq), ptr(kc), ptr(vc), pos, cap, window, int(fresh), heads, kv_heads, d,
                            scale, eps, ptr(out))
    return out


def sample_greedy(logits, softcap=0.0, penalty=1.0, seen=None, allowed=None):
    logits = np.ascontiguousarray(logits, np.float32)
    gap = C.c_double(0)
    t = lib().tbo_sample_greedy(ptr(logits), logits.size, softcap, penalty, ptr(seen), ptr(allowed), C.byref(gap))
    return int(t), gap.value


class Sampling(C.Structure):
    """ptx/sample.rs:38-78: the 40 bytes the sampler reads."""
    _fields_ = [("softcap", C.c_float), ("temperature", C.c_float), ("top_p", C.c_float), ("min_p", C.c_float), ("penalty", C.c_float),
                ("top_k", C.c_uint32), ("allowed", C.c_uint64), ("seed", C.c_uint64)]


def sampling(softcap=0.0, temperature=0.0, top_p=1.0, min_p=0.0, penalty=1.0, top_k=0, allowed=0, seed=0) -> Sampling:
    """Sampling::default (sample.rs:58-63) with overrides."""
    return Sampling(softcap, temperature, top_p, min_p, penalty, top_k, allowed, seed)


def sample_draw(logits, cfg: Sampling, step: int, seen=None, allowed=None):
    """(token, failed draws) of one draw at `step`, hash and filters as the reference's kernel, transcendental steps in double."""
    logits = np.ascontiguousarray(logits, np.float32)
    rounds = C.c_int(0)
    t = lib().tbo_sample_draw(ptr(logits), logits.size, C.byref(cfg), step, ptr(seen), ptr(allowed), C.byref(rounds))
    return int(t), rounds.value


def sample_topk(logits, k):
    logits = np.ascontiguousarray(logits, np.float32)
    idx, val = np.zeros(k, np.uint32), np.zeros(k, np.float32)
    lib().tbo_sample_topk(ptr(logits), logits.size, k, ptr(idx), ptr(val))
    return idx, val


def fill_codes(seed, stream, n):
    w = np.zeros(n, np.int8)
    lib().tbo_fill_codes(seed, stream, ptr(w), n)
    return w


def fill_scales(seed, stream, n, mul):
    s = np.zeros(n, np.uint16)
    lib().tbo_fill_scales(seed, stream, ptr(s), n, mul)
    return s


def fill_uniform(seed, stream, n, lo, hi):
    x = np.zeros(n, np.float32)
    lib().tbo_fill_uniform(seed, stream, ptr(x), n, lo, hi)
    return x


def fill_gauss_f16(seed, stream, n, mul=1.0):
    x = np.zeros(n, np.uint16)
    lib().tbo_fill_gauss_f16(seed, stream, ptr(x), n, mul)
    return x


def fill_gauss_f32(seed, stream, n, mul=1.0):
    x = np.zeros(n, np.float32)
    lib().tbo_fill_gauss_f32(seed, stream, ptr(x), n, mul)
    return x


def encoder_forward(cfg: dict, weights: dict, ids) -> np.ndarray:
    """Last hidden states [n, hidden] of one sequence.  cfg: hidden, heads, inter, vocab, window, gated, theta_global,
    theta_local, eps, global (list of bool).  weights: f32 arrays named embed, embed_norm, {l}.attn_norm (absent in
    layer 0), {l}.qkv, {l}.o, {l}.mlp_norm, {l}.up, {l}.down, final_norm."""
    layers = len(cfg["global"])
    keep = {k: np.ascontiguousarray(v, np.float32) for k, v in weights.items()}
    glob = np.array([1 if g else 0 for g in cfg["global"]], np.uint8)
    c = EncConfig(hidden=cfg["hidden"], heads=cfg["heads"], inter=cfg["inter"], vocab=cfg["vocab"], layers=layers, window=cfg["window"],
                  gated=int(cfg.get("gated", 1)), theta_global=cfg["theta_global"], theta_local=cfg["theta_local"], eps=cfg["eps"], global_=glob.ctypes.data)
    arr = (EncLayer * layers)()
    for l in range(layers):
        arr[l].attn_norm = keep[f"{l}.attn_norm"].ctypes.data if f"{l}.attn_norm" in keep else None
        for name in ("qkv", "o", "mlp_norm", "up", "down"):
            setattr(arr[l], name, keep[f"{l}.{name}"].ctypes.data)
    ids = np.ascontiguousarray(ids, np.uint32)
    out = np.zeros((ids.size, cfg["hidden"]), np.float32)
    lib().tbo_encoder_forward(C.byref(c), ptr(keep["embed"]), ptr(keep["embed_norm"]), C.cast(arr, C.POINTER(EncLayer)), ptr(keep["final_norm"]),
                              ptr(ids), ids.size, ptr(out))
    return out
