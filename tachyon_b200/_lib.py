"""ctypes declarations of ``libtachyon_b200.so`` (see ``include/tachyon_b200.h``).

There is no fallback: if the library has not been built (``python -m tachyon_b200.build``) loading raises.
"""
from __future__ import annotations

import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
# TACHYON_B200_LIBRARY names another build of the same library (a developer comparing two builds in one process tree).
PATH = os.environ.get("TACHYON_B200_LIBRARY") or os.path.join(HERE, "_native", "libtachyon_b200.so")

u32, u64, i32, f32, vp, sz, cp = C.c_uint32, C.c_uint64, C.c_int, C.c_float, C.c_void_p, C.c_size_t, C.c_char_p
pp = C.POINTER(C.c_void_p)


class Attend(C.Structure):
    _fields_ = [
        ("qkv", vp), ("q_norm", vp), ("k_norm", vp), ("freq", vp), ("k_cache", vp), ("v_cache", vp), ("pos", vp),
        ("cap", u32), ("window", u32), ("fresh", u32), ("heads", u32), ("kv_heads", u32),
        ("scale", f32), ("eps", f32), ("partial", vp), ("count", vp), ("splits", u32), ("out", vp), ("out_dtype", i32),
    ]


class Config(C.Structure):
    _fields_ = [
        ("hidden", u32), ("ffn", u32), ("heads", u32), ("kv_heads", u32), ("head_dim", u32), ("vocab", u32), ("layers", u32), ("window", u32),
        ("global_", vp), ("global_every", u32),
        ("theta_sliding", f32), ("theta_global", f32), ("fraction_global", f32), ("eps", f32), ("softcap", f32), ("attn_scale", f32),
        ("shared", u32), ("global_head_dim", u32), ("global_kv_heads", u32), ("per_layer", u32),
    ]


class EncoderConfig(C.Structure):
    _fields_ = [("hidden", u32), ("heads", u32), ("inter", u32), ("vocab", u32), ("layers", u32), ("window", u32), ("global_", vp), ("global_every", u32),
                ("theta_global", f32), ("theta_local", f32), ("eps", f32), ("gated", u32), ("mean_pool", u32), ("dims", u32)]


class WpkInfo(C.Structure):
    _fields_ = [("name", cp), ("dtype", u32), ("rank", u32), ("shape", u64 * 8), ("offset", u64), ("bytes", u64), ("crc32c", u32)]


class Chat(C.Structure):
    """tb_chat (token/chat.rs:57-72): the ids of Gemma 4's chat marks."""
    _fields_ = [("bos", u32), ("turn", u32), ("end", u32), ("think", u32), ("closed", u32 * 2)]


class Message(C.Structure):
    """tb_message: a role (0 system, 1 user, 2 model) and a text."""
    _fields_ = [("role", i32), ("text", vp), ("bytes", sz)]


class Load(C.Structure):
    """tb_load (engine.rs:72-90): settings, keep-alive in ms (2**64 - 1: for good), pin."""
    pass


class Loaded(C.Structure):
    """tb_loaded (engine.rs:93-107)."""
    _fields_ = [("name", C.c_char * 64), ("tier", C.c_int), ("vram", C.c_size_t), ("left_ms", C.c_uint64)]


class Settings(C.Structure):
    _fields_ = [("context", u32), ("chunk", u32), ("keep_logits", u32), ("fused", u32), ("weight_bits", u32), ("host_table", u32), ("prefill_copy", u32)]


Load._fields_ = [("settings", Settings), ("keep_alive_ms", C.c_uint64), ("pin", C.c_uint32)]


# name -> (restype, argtypes); every symbol the header declares.
SIGNATURES = {
    "tb_last_error": (cp, []),
    "tb_context_new": (i32, [i32, pp]),
    "tb_context_free": (None, [vp]),
    "tb_context_sms": (i32, [vp]),
    "tb_devices": (i32, [C.POINTER(i32)]),
    "tb_context_set_overlap": (i32, [vp, i32]),
    "tb_context_set_gemm_schedule": (i32, [vp, i32]),
    "tb_context_set_lean": (i32, [vp, i32]),
    "tb_context_set_dynamic": (i32, [vp, i32]),
    "tb_context_set_flash": (i32, [vp, i32]),
    "tb_context_memory": (i32, [vp, C.POINTER(sz), C.POINTER(sz)]),
    "tb_context_trim": (i32, [vp]),
    "tb_context_set_attn_block": (i32, [vp, i32]),
    "tb_status": (i32, [vp, C.POINTER(u32)]),
    "tb_status_clear": (i32, [vp]),
    "tb_selftest_wait": (i32, [vp, u64]),
    "tb_alloc": (i32, [vp, sz, pp]),
    "tb_free": (i32, [vp, vp]),
    "tb_alloc_host": (i32, [vp, sz, pp]),
    "tb_free_host": (i32, [vp, vp]),
    "tb_host_device_ptr": (i32, [vp, vp, pp]),
    "tb_upload": (i32, [vp, vp, vp, sz]),
    "tb_download": (i32, [vp, vp, vp, sz]),
    "tb_fill": (i32, [vp, vp, i32, sz]),
    "tb_sync": (i32, [vp]),
    "tb_event_new": (i32, [vp, pp]),
    "tb_event_free": (None, [vp]),
    "tb_event_record": (i32, [vp, vp]),
    "tb_event_sync": (i32, [vp]),
    "tb_event_elapsed_ms": (i32, [vp, vp, C.POINTER(f32)]),
    "tb_gemv_q8": (i32, [vp, vp, vp, vp, i32, vp, i32, u32, u32]),
    "tb_quant_q8": (i32, [vp, vp, u32, vp, vp]),
    "tb_gemv_q4": (i32, [vp, vp, vp, vp, vp, vp, u32, u32]),
    "tb_geglu_q8": (i32, [vp, vp, vp, u32, vp, vp]),
    "tb_norm_q8": (i32, [vp, vp, vp, vp, vp, vp, vp, vp, u32, u32, f32, f32]),
    "tb_embed_q4": (i32, [vp, vp, vp, vp, u32, vp, u32, f32]),
    "tb_launch": (i32, [vp, cp, vp, vp, u32, vp, sz]),
    "tb_gemv_q4x": (i32, [vp, vp, vp, vp, i32, vp, u32, u32]),
    "tb_sample": (i32, [vp, vp, vp, u32, vp, vp, vp, vp, vp, vp, u32]),
    "tb_gemv_f16": (i32, [vp, vp, vp, i32, vp, i32, u32, u32]),
    "tb_gemv_f16_norm": (i32, [vp, vp, vp, vp, vp, vp, f32, f32, vp, vp, i32, u32, u32]),
    "tb_gemv_q8_norm": (i32, [vp, vp, vp, vp, vp, vp, vp, f32, f32, vp, vp, u32, u32, i32]),
    "tb_gemv_q8_argmax": (i32, [vp, vp, vp, vp, i32, vp, u32, u32, vp, vp, vp]),
    "tb_gemm_q8": (i32, [vp, vp, vp, vp, u32, u32, u32, vp, i32]),
    "tb_gemm_f16": (i32, [vp, vp, vp, u32, u32, u32, vp, i32]),
    "tb_dequant_f16": (i32, [vp, vp, vp, u32, u32, u32, vp]),
    "tb_gemm_q4": (i32, [vp, vp, vp, vp, u32, u32, u32, vp, i32]),
    "tb_norm": (i32, [vp, vp, vp, vp, vp, u32, f32, f32, vp, vp]),
    "tb_prefill_norm": (i32, [vp, vp, vp, vp, vp, u32, u32, f32, f32, vp]),
    "tb_embed_q8": (i32, [vp, vp, vp, vp, u32, f32, vp]),
    "tb_prefill_attend": (i32, [vp, vp, vp, vp, vp, u32, u32, u32, u32, u32, u32, u32]),
    "tb_prefill_qkv": (i32, [vp, vp, vp, vp, vp, vp, vp, vp, u32, u32, u32, u32, u32, f32, f32, u32]),
    "tb_attend_scratch_bytes": (sz, [u32, u32, u32]),
    "tb_attend_decode": (i32, [vp, C.POINTER(Attend)]),
    "tb_attend_project": (i32, [vp, C.POINTER(Attend), u32, vp, vp, u32, vp]),
    "tb_attend_decode_static": (i32, [vp, C.POINTER(Attend)]),
    "tb_attend_decode_512": (i32, [vp, C.POINTER(Attend)]),
    "tb_attend_512_scratch_bytes": (C.c_size_t, [u32, u32]),
    "tb_sample_greedy": (i32, [vp, vp, u32, f32, f32, vp, vp, vp, vp, vp]),
    "tb_topk": (i32, [vp, vp, u32, u32, vp, vp]),
    "tb_fill_codes": (i32, [vp, u64, u64, vp, sz]),
    "tb_fill_scales": (i32, [vp, u64, u64, vp, sz, f32]),
    "tb_fill_gauss_f16": (i32, [vp, u64, u64, vp, sz, f32]),
    "tb_fill_uniform": (i32, [vp, u64, u64, vp, sz, f32, f32]),
    "tb_decoder_open": (i32, [vp, C.POINTER(Config), C.POINTER(Settings), pp]),
    "tb_decoder_close": (None, [vp]),
    "tb_decoder_load": (i32, [vp, cp, vp, sz]),
    "tb_decoder_fill_random": (i32, [vp, u64]),
    "tb_decoder_fill_cache": (i32, [vp, u64, u32]),
    "tb_decoder_build": (i32, [vp]),
    "tb_decoder_reset": (i32, [vp]),
    "tb_decoder_step": (i32, [vp, u32, C.POINTER(u32)]),
    "tb_decoder_start": (i32, [vp, u32]),
    "tb_decoder_next_token": (i32, [vp, C.POINTER(u32)]),
    "tb_decoder_stop": (i32, [vp]),
    "tb_decoder_run": (i32, [vp, u32, u32, vp]),
    "tb_decoder_prefill": (i32, [vp, vp, u32]),
    "tb_decoder_logits": (i32, [vp, vp]),
    "tb_decoder_position": (i32, [vp, C.POINTER(u32)]),
    "tb_decoder_step_bytes": (i32, [vp, C.POINTER(u64), C.POINTER(u64)]),
    "tb_decoder_step_launches": (i32, [vp, C.POINTER(u32)]),
    "tb_decoder_hidden": (i32, [vp, vp]),
    "tb_decoder_set_sampling": (i32, [vp, vp]),
    "tb_crc32c": (u32, [u32, vp, sz]),
    "tb_crc32c_combine": (u32, [u32, u32, u64]),
    "tb_wpk_open": (i32, [cp, pp]),
    "tb_wpk_close": (None, [vp]),
    "tb_wpk_count": (u32, [vp]),
    "tb_wpk_tensor": (i32, [vp, u32, vp]),
    "tb_wpk_read": (i32, [vp, u32, vp, sz, i32]),
    "tb_decoder_load_wpk": (i32, [vp, cp, i32]),
    "tb_encoder_load_wpk": (i32, [vp, cp, i32]),
    "tb_decoder_park": (i32, [vp, pp]),
    "tb_parked_resume": (i32, [vp, C.POINTER(Settings), pp]),
    "tb_parked_bytes": (sz, [vp]),
    "tb_parked_close": (None, [vp]),
    "tb_decoder_bytes": (sz, [vp]),
    "tb_decoder_parked_bytes": (sz, [vp]),
    "tb_decoder_shadow_bytes": (sz, [vp]),
    "tb_decoder_drop_shadow": (None, [vp]),
    "tb_decoder_footprint": (i32, [vp, C.POINTER(Config), C.POINTER(Settings), C.POINTER(sz)]),
    "tb_engine_new": (i32, [vp, sz, sz, pp]),
    "tb_engine_close": (None, [vp]),
    "tb_engine_load": (i32, [vp, cp, C.POINTER(Config), C.POINTER(Load), cp, cp]),
    "tb_engine_unload": (i32, [vp, cp, C.POINTER(i32)]),
    "tb_engine_decoder": (i32, [vp, cp, pp]),
    "tb_engine_feed": (i32, [vp, cp, vp, u32, C.POINTER(u32)]),
    "tb_engine_tier": (i32, [vp, cp, C.POINTER(i32)]),
    "tb_engine_models": (i32, [vp, C.POINTER(Loaded), sz, C.POINTER(sz)]),
    "tb_engine_expire": (i32, [vp]),
    "tb_engine_usage": (i32, [vp, C.POINTER(sz), C.POINTER(sz)]),
    "tb_tokenizer_from_json": (i32, [vp, sz, pp]),
    "tb_tokenizer_from_bytes": (i32, [vp, sz, pp]),
    "tb_tokenizer_to_bytes": (i32, [vp, vp, sz, C.POINTER(sz)]),
    "tb_tokenizer_close": (None, [vp]),
    "tb_tokenizer_len": (sz, [vp]),
    "tb_tokenizer_encode": (i32, [vp, vp, sz, vp, sz, C.POINTER(sz)]),
    "tb_tokenizer_token": (i32, [vp, u32, pp, C.POINTER(sz)]),
    "tb_tokenizer_is_special": (i32, [vp, u32]),
    "tb_tokenizer_special": (i32, [vp, cp, C.POINTER(u32)]),
    "tb_tokenizer_frame": (None, [vp, C.POINTER(u32), C.POINTER(u32)]),
    "tb_detokenizer_new": (i32, [pp]),
    "tb_detokenizer_close": (None, [vp]),
    "tb_detokenizer_push": (i32, [vp, vp, u32, vp, sz, C.POINTER(sz)]),
    "tb_detokenizer_finish": (i32, [vp, vp, sz, C.POINTER(sz)]),
    "tb_chat_gemma4": (i32, [vp, C.POINTER(Chat)]),
    "tb_chat_with_template": (i32, [vp, C.POINTER(Chat), vp, sz]),
    "tb_chat_encode": (i32, [vp, C.POINTER(Chat), C.POINTER(Message), sz, i32, vp, sz, C.POINTER(sz)]),
    "tb_engine_load_encoder": (i32, [vp, cp, C.POINTER(EncoderConfig), u32, u32, u64, i32, cp, cp]),
    "tb_engine_encoder": (i32, [vp, cp, pp]),
    "tb_engine_embed": (i32, [vp, cp, vp, vp, u32, vp]),
    "tb_encoder_bytes": (sz, [vp]),
    "tb_encoder_footprint": (i32, [vp, C.POINTER(EncoderConfig), u32, u32, i32, C.POINTER(sz)]),
    "tb_encoder_open": (i32, [vp, C.POINTER(EncoderConfig), u32, u32, pp]),
    "tb_encoder_close": (None, [vp]),
    "tb_encoder_load": (i32, [vp, cp, vp, sz]),
    "tb_encoder_fill_random": (i32, [vp, u64]),
    "tb_encoder_embed": (i32, [vp, vp, vp, u32, vp]),
    "tb_encoder_hidden": (i32, [vp, vp]),
    "tb_encoder_batch_tokens": (u32, [vp]),
    "tb_encoder_graphs": (u32, [vp]),
    "tb_decoder_timeline": (i32, [vp, u32, vp, C.POINTER(u32)]),
}

_lib = None


def load() -> C.CDLL:
    """The library, loaded once.  Raises when it is missing: there is no other code path."""
    global _lib
    if _lib is None:
        if not os.path.exists(PATH):
            raise ImportError(f"{PATH} is not built; run `python -m tachyon_b200.build` (needs nvcc). There is no CPU or PyTorch fallback.")
        lib = C.CDLL(PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(lib, name)
            fn.restype, fn.argtypes = res, args
        _lib = lib
    return _lib
