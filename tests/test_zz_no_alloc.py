"""tb_attend_decode_static: decode attention for callers that cannot allocate device memory (their memory plan is
fixed at start-up, or cudaMalloc's device-wide synchronisation is not acceptable where they call from).  The scratch
is an array inside the library, so the results must equal those of tb_attend_decode with caller-provided scratch.

This file is collected last on purpose: a run that stops at the first failure has then already run everything else.
"""
import numpy as np
import pytest

import tachyon_b200 as tb
from util import f16, f16_to_f32, values_fast

pytestmark = pytest.mark.gpu
D = 256


def make_args(ctx, *, heads, kv, cap, window, pos, splits, seed, with_scratch):
    qkv = values_fast((heads + 2 * kv) * D, seed)
    qn = (0.2 + 0.1 * values_fast(D, seed + 1)).astype(np.float32)
    kn = (0.2 + 0.1 * values_fast(D, seed + 2)).astype(np.float32)
    freq = (10000.0 ** (-np.arange(D // 2, dtype=np.float32) * 2 / D)).astype(np.float32)
    kc, vc = f16(0.3 * values_fast(kv * cap * D, seed + 3)), f16(0.3 * values_fast(kv * cap * D, seed + 4))
    keep = dict(qkv=ctx.upload(qkv), qn=ctx.upload(qn), kn=ctx.upload(kn), freq=ctx.upload(freq), k=ctx.upload(kc), v=ctx.upload(vc),
                pos=ctx.upload(np.array([pos], np.uint32)), out=ctx.zeros(heads * D * 4))
    if with_scratch:
        keep["part"] = ctx.zeros(ctx.attend_scratch_bytes(heads, kv, splits))
        keep["count"] = ctx.zeros(4 * kv)
    a = tb.Attend(qkv=keep["qkv"].ptr, q_norm=keep["qn"].ptr, k_norm=keep["kn"].ptr, freq=keep["freq"].ptr, k_cache=keep["k"].ptr, v_cache=keep["v"].ptr,
                  pos=keep["pos"].ptr, cap=cap, window=window, fresh=1, heads=heads, kv_heads=kv, scale=1.0, eps=1e-6,
                  partial=keep["part"].ptr if with_scratch else None, count=keep["count"].ptr if with_scratch else None, splits=splits,
                  out=keep["out"].ptr, out_dtype=tb.F32)
    return a, keep


CASES = [dict(heads=8, kv=2, cap=4096, window=4096, pos=3000, splits=64, seed=5),   # many splits, big partials
         dict(heads=8, kv=2, cap=512, window=512, pos=700, splits=16, seed=9),      # right after: fewer splits, stale partials beyond them
         dict(heads=4, kv=4, cap=256, window=256, pos=40, splits=2, seed=13)]       # four kv heads: every counter word in use


def test_static_scratch_matches_caller_scratch_on_calls_in_a_row(ctx):
    for case in CASES:
        a_ref, keep_ref = make_args(ctx, with_scratch=True, **case)
        ctx.attend_decode(a_ref)
        want = keep_ref["out"].download(np.float32, case["heads"] * D)
        a_new, keep_new = make_args(ctx, with_scratch=False, **case)
        for _ in range(2):  # twice in a row on the same shared array
            keep_new["out"].zero()
            ctx.attend_decode_static(a_new)
            got = keep_new["out"].download(np.float32, case["heads"] * D)
            assert np.abs(got - want).max() <= 1e-3 * np.abs(want).max()
        # the new token's key/value landed in the cache exactly as with the other entry point
        n = case["kv"] * case["cap"] * D
        assert np.array_equal(keep_new["k"].download(np.uint16, n), keep_ref["k"].download(np.uint16, n))
        assert np.array_equal(keep_new["v"].download(np.uint16, n), keep_ref["v"].download(np.uint16, n))
    assert ctx.status() == 0


def test_sizes_beyond_the_built_in_scratch_are_refused(ctx):
    a, keep = make_args(ctx, with_scratch=False, heads=8, kv=2, cap=8192, window=8192, pos=100, splits=65, seed=1)
    with pytest.raises(tb.Error) as e:
        ctx.attend_decode_static(a)
    assert e.value.status == 3 and "64 splits" in str(e.value)
    a, keep = make_args(ctx, with_scratch=False, heads=8, kv=8, cap=64, window=64, pos=10, splits=2, seed=1)
    with pytest.raises(tb.Error) as e:
        ctx.attend_decode_static(a)
    assert e.value.status == 3
