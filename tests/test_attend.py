"""Decode attention on the GPU against the f64 oracle.  Cases follow crates/tachyon/tests/decode.rs:185-334 (short
context, full sliding window, ring longer than the window, shared cache, 1/2/4 query heads per key-value head) at head
size 256, plus the benchmark's plain configuration (scale 1/16, no norms, f16 output, 4096 positions); head size 512
(rope(1e6, 512, 0.25), decode.rs:212, 329-334) and eight query heads to a key-value head (decode.rs:313-314)."""
import numpy as np
import pytest

import oracle
import tachyon_b200 as tb
from util import f16, f16_to_f32, values_fast

pytestmark = pytest.mark.gpu
D = 256


def run_case(ctx, *, cap, win, pos, splits, fresh, heads, kv, plain=False, out_f16=False, times=2, scale=1.0, seed=0, D=256):
    blocks = heads // min(heads // kv, 4)  # blocks per split: the counters
    rng_seed = seed + pos + cap
    rows = heads + 2 * kv
    qkv = values_fast(rows * D, rng_seed)
    if plain:
        qkv = np.random.default_rng(rng_seed).standard_normal(rows * D).astype(np.float32)
    qn = (0.2 + 0.1 * values_fast(D, rng_seed + 1)).astype(np.float32)
    kn = (0.2 + 0.1 * values_fast(D, rng_seed + 2)).astype(np.float32)
    freq = oracle.rope_freq(10000.0, D, 1.0) if D == 256 else oracle.rope_freq(1e6, D, 0.25)
    mul = 1.0 if plain else 0.3
    kc = f16(mul * (np.random.default_rng(rng_seed + 3).standard_normal(kv * cap * D) if plain else values_fast(kv * cap * D, rng_seed + 3)))
    vc = f16(mul * (np.random.default_rng(rng_seed + 4).standard_normal(kv * cap * D) if plain else values_fast(kv * cap * D, rng_seed + 4)))
    kc0, vc0 = kc.copy(), vc.copy()
    want = oracle.attend_decode(qkv, None if plain else qn, None if plain else kn, None if plain else freq, kc0, vc0, pos, cap, win, fresh, heads, kv, D, scale)

    bufs = dict(qkv=ctx.upload(qkv), qn=ctx.upload(qn), kn=ctx.upload(kn), freq=ctx.upload(freq), k=ctx.upload(kc), v=ctx.upload(vc),
                pos=ctx.upload(np.array([pos], np.uint32)), part=ctx.zeros(max(ctx.attend_scratch_bytes(heads, kv, splits) * (D // 256), 16)),
                count=ctx.zeros(4 * blocks), out=ctx.zeros(heads * D * 4))
    a = tb.Attend(qkv=bufs["qkv"].ptr, q_norm=None if plain else bufs["qn"].ptr, k_norm=None if plain else bufs["kn"].ptr,
                  freq=None if plain else bufs["freq"].ptr, k_cache=bufs["k"].ptr, v_cache=bufs["v"].ptr, pos=bufs["pos"].ptr, cap=cap, window=win,
                  fresh=int(fresh), heads=heads, kv_heads=kv, scale=scale, eps=1e-6, partial=bufs["part"].ptr, count=bufs["count"].ptr, splits=splits,
                  out=bufs["out"].ptr, out_dtype=tb.F16 if out_f16 else tb.F32)
    for _ in range(times):
        ctx.attend_decode(a) if D == 256 else ctx.attend_decode_512(a)
    assert not bufs["count"].download(np.uint32, blocks).any(), "the counters are left at zero"
    got = f16_to_f32(bufs["out"].download(np.uint16, heads * D)) if out_f16 else bufs["out"].download(np.float32, heads * D)
    tol = (2e-3 if out_f16 else 1e-3) * np.abs(want).max()
    assert np.abs(got - want).max() <= tol, (np.abs(got - want).max(), tol)
    # the caches: untouched when shared, the new token's slot rewritten when fresh
    k_after, v_after = bufs["k"].download(np.uint16, kv * cap * D), bufs["v"].download(np.uint16, kv * cap * D)
    if not fresh:
        assert np.array_equal(k_after, kc) and np.array_equal(v_after, vc)
    else:
        slot = pos % cap
        mask = np.ones(kv * cap * D, bool)
        for g in range(kv):
            mask[(g * cap + slot) * D:(g * cap + slot + 1) * D] = False
        assert np.array_equal(k_after[mask], kc[mask]) and np.array_equal(v_after[mask], vc[mask]), "only the new slot changes"
        for got_c, want_c in ((k_after, kc0), (v_after, vc0)):
            g_, w_ = f16_to_f32(got_c[~mask]), f16_to_f32(want_c[~mask])
            assert np.all(np.abs(g_ - w_) <= 1e-3 * np.abs(w_) + 1e-4)


def test_attention_over_a_short_context(ctx):
    run_case(ctx, cap=512, win=512, pos=0, splits=16, fresh=True, heads=8, kv=2)
    run_case(ctx, cap=512, win=512, pos=100, splits=16, fresh=True, heads=8, kv=2)
    run_case(ctx, cap=512, win=512, pos=100, splits=16, fresh=True, heads=4, kv=2)  # two query heads per kv head
    run_case(ctx, cap=512, win=512, pos=100, splits=16, fresh=True, heads=2, kv=2)  # one
    run_case(ctx, cap=512, win=512, pos=17, splits=1, fresh=True, heads=8, kv=2)    # a single block, no scratch used


def test_attention_over_a_full_sliding_window(ctx):
    run_case(ctx, cap=512, win=512, pos=700, splits=16, fresh=True, heads=8, kv=2)
    run_case(ctx, cap=1024, win=512, pos=1700, splits=16, fresh=True, heads=8, kv=2)  # a ring longer than the window
    run_case(ctx, cap=2048, win=1024, pos=3000, splits=32, fresh=True, heads=4, kv=2)
    run_case(ctx, cap=600, win=512, pos=5999, splits=7, fresh=True, heads=8, kv=2)    # ragged spans, wrap inside a tile


def test_global_attention_with_its_own_or_a_shared_cache(ctx):
    run_case(ctx, cap=2048, win=2048, pos=1500, splits=32, fresh=True, heads=8, kv=2)
    run_case(ctx, cap=2048, win=2048, pos=1500, splits=128, fresh=False, heads=8, kv=2)
    run_case(ctx, cap=4096, win=4096, pos=4095, splits=4, fresh=True, heads=8, kv=2)  # several tiles per block


def test_heads_of_512(ctx):
    """decode.rs:329-334: global layers' heads of 512, their own cache or a shared one, four or eight query heads to a key-value head."""
    assert ctx.attend_512_scratch_bytes(8, 32) == 8 * 32 * 514 * 4
    run_case(ctx, D=512, cap=2048, win=2048, pos=1500, splits=32, fresh=True, heads=8, kv=2)
    run_case(ctx, D=512, cap=2048, win=2048, pos=1500, splits=256, fresh=False, heads=8, kv=2)
    run_case(ctx, D=512, cap=2048, win=2048, pos=1500, splits=32, fresh=True, heads=16, kv=2)
    run_case(ctx, D=512, cap=512, win=512, pos=0, splits=8, fresh=True, heads=4, kv=2)
    run_case(ctx, D=512, cap=600, win=512, pos=5999, splits=7, fresh=True, heads=2, kv=2, out_f16=True)
    run_case(ctx, D=512, cap=512, win=512, pos=17, splits=1, fresh=True, heads=8, kv=2)


def test_eight_query_heads_to_a_key_value_head(ctx):
    """decode.rs:313-314 (E2B): two blocks share each key-value head and the first stores the new key and value."""
    run_case(ctx, cap=512, win=512, pos=100, splits=16, fresh=True, heads=16, kv=2)
    run_case(ctx, cap=1024, win=512, pos=1700, splits=16, fresh=True, heads=8, kv=1)
    run_case(ctx, cap=2048, win=2048, pos=1500, splits=64, fresh=False, heads=16, kv=2)


def test_plain_configuration_of_the_benchmark(ctx):
    """8 query heads, 2 kv heads, 4096 positions ~N(0,1), scale 1/sqrt(256), f16 out: global and sliding-512."""
    run_case(ctx, cap=4096, win=4096, pos=4095, splits=64, fresh=False, heads=8, kv=2, plain=True, out_f16=True, scale=1 / 16.0)
    run_case(ctx, cap=4096, win=512, pos=4095, splits=16, fresh=False, heads=8, kv=2, plain=True, out_f16=True, scale=1 / 16.0)
    run_case(ctx, cap=4096, win=4096, pos=4095, splits=64, fresh=True, heads=8, kv=2, plain=True, out_f16=False, scale=1 / 16.0)


def test_attention_rejects_bad_descriptors(ctx):
    z = ctx.zeros(64)
    a = tb.Attend(qkv=z.ptr, k_cache=z.ptr, v_cache=z.ptr, pos=z.ptr, cap=16, window=32, fresh=1, heads=8, kv_heads=2, scale=1.0, eps=1e-6,
                  partial=z.ptr, count=z.ptr, splits=1, out=z.ptr, out_dtype=tb.F32)
    with pytest.raises(tb.Error) as e:
        ctx.attend_decode(a)  # window larger than the ring
    assert e.value.status == 3
    a.window, a.heads = 16, 6
    with pytest.raises(tb.Error):
        ctx.attend_decode(a)  # three query heads per kv head: no kernel


@pytest.mark.parametrize("cluster", [1, 2, 4, 8])
@pytest.mark.parametrize("lean", [1, 0])
@pytest.mark.parametrize("cap,win,pos,splits,fresh,kv", [(640, 512, 2048, 8, True, 2), (640, 512, 100, 8, True, 2), (640, 512, 40, 8, True, 2), (4096, 4096, 2048, 32, True, 2),
                                                          (4096, 4096, 4095, 32, False, 2), (4096, 4096, 300, 32, True, 4), (640, 512, 5999, 16, False, 8),
                                                          (640, 512, 0, 8, True, 2)])
def test_attention_then_projection_with_splits_merged_in_clusters(ctx, cluster, lean, cap, win, pos, splits, fresh, kv):
    """tb_attend_project: what a decode step does between its query/key/value and its gate/up products.  Whatever the
    cluster size (1: every split reaches the projection's prologue; 8: one entry per eight splits, merged in distributed
    shared memory), with empty splits inside a cluster, whole clusters without positions, and the small or the staged
    projection kernel, the result is the oracle's attention output times the dequantised matrix."""
    heads, rows = 8, 512
    seed = pos + cap + kv
    qkv = values_fast((heads + 2 * kv) * D, seed)
    qn, kn = (0.2 + 0.1 * values_fast(D, seed + 1)).astype(np.float32), (0.2 + 0.1 * values_fast(D, seed + 2)).astype(np.float32)
    freq = oracle.rope_freq(10000.0, D, 1.0)
    kc, vc = f16(0.3 * values_fast(kv * cap * D, seed + 3)), f16(0.3 * values_fast(kv * cap * D, seed + 4))
    att = oracle.attend_decode(qkv, qn, kn, freq, kc.copy(), vc.copy(), pos, cap, win, fresh, heads, kv, D, 1.0)
    from util import q8_weights

    w, s = q8_weights(rows, heads * D, 77)
    deq = w.astype(np.float64) * np.repeat(f16_to_f32(s).astype(np.float64), 32, axis=1)
    want, bound = deq @ att, np.abs(deq) @ np.abs(att)
    bufs = [ctx.upload(a) for a in (qkv, qn, kn, freq, kc, vc, np.array([pos], np.uint32), w, s)]
    part, y = ctx.zeros(ctx.attend_scratch_bytes(heads, kv, splits)), ctx.zeros(rows * 4)
    a = tb.Attend(qkv=bufs[0].ptr, q_norm=bufs[1].ptr, k_norm=bufs[2].ptr, freq=bufs[3].ptr, k_cache=bufs[4].ptr, v_cache=bufs[5].ptr, pos=bufs[6].ptr, cap=cap,
                  window=win, fresh=int(fresh), heads=heads, kv_heads=kv, scale=1.0, eps=1e-6, partial=part.ptr, count=None, splits=splits, out=None, out_dtype=tb.F32)
    ctx.set_lean(lean)
    try:
        for _ in range(2):
            ctx.attend_project(a, cluster, bufs[7], bufs[8], rows, y)
    finally:
        ctx.set_lean(1)
    got = y.download(np.float32, rows)
    assert np.all(np.abs(got - want) <= 1e-3 * bound + 1e-6), float(np.abs(got - want).max())
    assert ctx.status() == 0


def test_cluster_sizes_that_do_not_fit_are_refused(ctx):
    z = ctx.zeros(1 << 16)
    a = tb.Attend(qkv=z.ptr, k_cache=z.ptr, v_cache=z.ptr, pos=z.ptr, cap=64, window=64, fresh=1, heads=8, kv_heads=2, scale=1.0, eps=1e-6, partial=z.ptr,
                  count=None, splits=6, out=None, out_dtype=tb.F32)
    for cluster in (3, 4, 16):  # not a power of two up to 8, not a divisor of the splits, too large
        with pytest.raises(tb.Error) as e:
            ctx.attend_project(a, cluster, z, z, 64, z)
        assert e.value.status == 3
