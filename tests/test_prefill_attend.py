"""Prefill attention (tb_prefill_attend) against f64 on the CPU.  Cases follow crates/tachyon/tests/prefill.rs:199-209
(a chunk starting at position 600 over a sliding window of a ring, global attention, four or two query heads per
key-value head) at head sizes 256 and 512, plus ragged token counts and a window that starts before position 0; and the
chunk's key-value store and query preparation (tb_prefill_qkv; prefill.rs:213-236 launches kv_*, query_* before flash_*)."""
import numpy as np
import pytest

import oracle
import tachyon_b200 as tb
from util import f16, f16_to_f32, values_fast

pytestmark = pytest.mark.gpu
KV = 2


def reference(q, kc, vc, tokens, pos0, cap, window, heads, D):
    """q [tokens][heads][D] (base-2 scores), caches [KV][cap][D]; f64 out [tokens][heads * D]."""
    ratio = heads // KV
    out = np.zeros((tokens, heads, D))
    for t in range(tokens):
        p = pos0 + t
        js = np.arange(max(0, p - window + 1), p + 1)
        for h in range(heads):
            k, v = kc[h // ratio, js % cap], vc[h // ratio, js % cap]
            s = k @ q[t, h]
            w = np.exp2(s - s.max())
            out[t, h] = (w / w.sum()) @ v
    return out.reshape(tokens, heads * D)


@pytest.mark.parametrize("D,ratio,cap,window,pos0,tokens", [(256, 4, 1024, 512, 600, 100), (256, 2, 1024, 512, 600, 100), (256, 4, 700, 700, 600, 100),
                                                            (256, 1, 256, 64, 0, 37), (256, 4, 2048, 512, 0, 300), (256, 4, 640, 512, 1900, 129),
                                                            (512, 4, 700, 700, 600, 100), (512, 2, 1024, 512, 600, 70), (512, 1, 256, 64, 0, 37),
                                                            (512, 4, 2048, 2048, 0, 200), (256, 8, 1024, 512, 600, 50), (512, 8, 700, 700, 600, 50)])
def test_prefill_attention_matches_f64(ctx, D, ratio, cap, window, pos0, tokens):
    heads, seed = ratio * KV, cap + pos0 + tokens
    q = f16(0.25 * values_fast(tokens * heads * D, seed))
    kc, vc = f16(0.3 * values_fast(KV * cap * D, seed + 1)), f16(0.3 * values_fast(KV * cap * D, seed + 2))
    want = reference(f16_to_f32(q).astype(np.float64).reshape(tokens, heads, D), f16_to_f32(kc).astype(np.float64).reshape(KV, cap, D),
                     f16_to_f32(vc).astype(np.float64).reshape(KV, cap, D), tokens, pos0, cap, window, heads, D)
    qd, kd, vd = ctx.upload(q), ctx.upload(kc), ctx.upload(vc)
    out = ctx.alloc((tokens + 2) * heads * D * 2)
    out.upload(np.full((tokens + 2) * heads * D, 0x7BFF, np.uint16))
    ctx.prefill_attend(qd, kd, vd, out, tokens, pos0, cap, window, heads, KV, D)
    got = out.download(np.uint16, (tokens + 2) * heads * D)
    assert np.all(got[tokens * heads * D:] == 0x7BFF), "rows past the tokens were written"
    got = f16_to_f32(got[: tokens * heads * D]).reshape(tokens, heads * D)
    top = np.abs(want).max()
    assert np.abs(got - want).max() <= 1e-3 * top + 2.0**-11 * top, float(np.abs(got - want).max() / top)


@pytest.mark.parametrize("cap,window,pos0,tokens", [(1024, 512, 600, 100), (2048, 2048, 0, 300), (640, 512, 1900, 129), (4096, 512, 1000, 33), (128, 128, 0, 128),
                                                    (256, 64, 500, 31)])
def test_the_tcgen05_kernel_and_the_mma_sync_kernel_agree(ctx, cap, window, pos0, tokens):
    """tb_context_set_flash: heads of 256, four query heads to a key-value head and a ring of whole tiles of 64 run on tcgen05
    (scores and outputs in tensor memory, the running maximum moved only when a tile passes it by 2^8); every other shape, and
    setting 0, on mma.sync.  Both are the same attention: the same values to the rounding of the probabilities to f16, rows
    past the tokens left alone, f16 or f32 out (the "flash_256" launch stores f32)."""
    heads, D = 4 * KV, 256
    q = f16(0.25 * values_fast(tokens * heads * D, cap + tokens))
    kc, vc = f16(0.3 * values_fast(KV * cap * D, cap + 1)), f16(0.3 * values_fast(KV * cap * D, cap + 2))
    qd, kd, vd = ctx.upload(q), ctx.upload(kc), ctx.upload(vc)
    outs = []
    for which in (0, 1):
        ctx.set_flash(which)
        try:
            out = ctx.alloc((tokens + 2) * heads * D * 2)
            out.upload(np.full((tokens + 2) * heads * D, 0x7BFF, np.uint16))
            ctx.prefill_attend(qd, kd, vd, out, tokens, pos0, cap, window, heads, KV, D)
            got = out.download(np.uint16, (tokens + 2) * heads * D)
        finally:
            ctx.set_flash(1)
        assert np.all(got[tokens * heads * D:] == 0x7BFF), "rows past the tokens were written"
        outs.append(f16_to_f32(got[: tokens * heads * D]))
    top = np.abs(outs[0]).max()
    assert np.abs(outs[0] - outs[1]).max() <= 2e-3 * top, float(np.abs(outs[0] - outs[1]).max() / top)
    want = reference(f16_to_f32(q).astype(np.float64).reshape(tokens, heads, D), f16_to_f32(kc).astype(np.float64).reshape(KV, cap, D),
                     f16_to_f32(vc).astype(np.float64).reshape(KV, cap, D), tokens, pos0, cap, window, heads, D).ravel()
    for got in outs:
        assert np.abs(got - want).max() <= 1e-3 * top + 2.0**-11 * top
    assert ctx.status() == 0


def test_scores_far_apart_move_the_running_maximum(ctx):
    """Keys whose scores rise by more than 2^8 from tile to tile: the tcgen05 kernel rescales its sums and its output in tensor
    memory on those tiles, and only the last keys carry weight."""
    heads, D, cap, tokens, window = 4 * KV, 256, 1024, 64, 1024
    rng = np.random.default_rng(9)
    q = np.zeros((tokens, heads, D), np.float32)
    q[:, :, 0] = 1.0
    kc = 0.01 * rng.standard_normal((KV, cap, D)).astype(np.float32)
    kc[:, :, 0] = np.arange(cap, dtype=np.float32)[None, :] * 0.25  # the score of key j is j / 4: 32 more a tile
    vc = rng.standard_normal((KV, cap, D)).astype(np.float32)
    qh, kh, vh = f16(q), f16(kc), f16(vc)
    pos0 = 600
    want = reference(f16_to_f32(qh).astype(np.float64).reshape(tokens, heads, D), f16_to_f32(kh).astype(np.float64).reshape(KV, cap, D),
                     f16_to_f32(vh).astype(np.float64).reshape(KV, cap, D), tokens, pos0, cap, window, heads, D)
    out = ctx.zeros(tokens * heads * D * 2)
    ctx.prefill_attend(ctx.upload(qh), ctx.upload(kh), ctx.upload(vh), out, tokens, pos0, cap, window, heads, KV, D)
    got = f16_to_f32(out.download(np.uint16, tokens * heads * D)).reshape(tokens, heads * D)
    top = np.abs(want).max()
    assert np.abs(got - want).max() <= 2e-3 * top, float(np.abs(got - want).max() / top)
    assert ctx.status() == 0


@pytest.mark.parametrize("D", [256, 512])
def test_prefill_attention_does_not_depend_on_the_chunking(ctx, D):
    """flash.rs:9-12: key tiles start at multiples of their size, so a token's sums are the same whichever chunk it is in."""
    heads, cap, window, tokens = 8, 1024, 512, 96
    q = f16(0.25 * values_fast(tokens * heads * D, 5))
    kc, vc = f16(0.3 * values_fast(KV * cap * D, 6)), f16(0.3 * values_fast(KV * cap * D, 7))
    qd, kd, vd = ctx.upload(q), ctx.upload(kc), ctx.upload(vc)
    cut = 40  # not a multiple of the tile of 16 tokens
    whole, first, second = ctx.zeros(tokens * heads * D * 2), ctx.zeros(cut * heads * D * 2), ctx.zeros((tokens - cut) * heads * D * 2)
    ctx.prefill_attend(qd, kd, vd, whole, tokens, 200, cap, window, heads, KV, D)
    ctx.prefill_attend(qd, kd, vd, first, cut, 200, cap, window, heads, KV, D)
    ctx.prefill_attend(ctx.upload(q[cut * heads * D:]), kd, vd, second, tokens - cut, 200 + cut, cap, window, heads, KV, D)
    parts = np.concatenate([first.download(np.uint16, cut * heads * D), second.download(np.uint16, (tokens - cut) * heads * D)])
    assert np.array_equal(whole.download(np.uint16, tokens * heads * D), parts)


@pytest.mark.parametrize("D,heads,kv,theta,fraction", [(256, 8, 2, 1e4, 1.0), (512, 8, 2, 1e6, 0.25), (256, 8, 0, 1e4, 1.0), (512, 2, 1, 1e6, 0.25), (512, 8, 1, 1e6, 0.25)])
def test_prefill_qkv_stores_keys_values_and_queries(ctx, D, heads, kv, theta, fraction):
    """kv_256 / kv_512 and query_256 / query_512 (ptx/attend.rs:472-556): norms, RoPE at pos0 + t, ring slot (pos0 + t) % cap."""
    tokens, pos0, cap, eps, scale = 53, 990, 64, 1e-6, 0.5  # 53 x 10 rows: the last block is not full
    rows = heads + 2 * kv
    qkv = values_fast(tokens * rows * D, 11 + D).reshape(tokens, rows, D)
    qn, kn = (0.2 + 0.1 * values_fast(D, 12)).astype(np.float32), (0.2 + 0.1 * values_fast(D, 13)).astype(np.float32)
    freq = oracle.rope_freq(theta, D, fraction)

    def prepared(x, w, pos, rotate):
        x = x.astype(np.float64)
        x = x / np.sqrt((x * x).mean() + eps) * (1.0 if w is None else w.astype(np.float64))
        if rotate:
            ang = np.float32(pos) * freq  # f32 angle, as the reference's test model has it
            c, s_ = np.cos(ang.astype(np.float64)), np.sin(ang.astype(np.float64))
            a, b = x[: D // 2].copy(), x[D // 2:].copy()
            x = np.concatenate([a * c - b * s_, b * c + a * s_])
        return x

    kc0, vc0 = f16(0.3 * values_fast(max(kv, 1) * cap * D, 14)), f16(0.3 * values_fast(max(kv, 1) * cap * D, 15))
    bufs = [ctx.upload(a) for a in (qkv, qn, kn, freq, kc0, vc0)]
    q_out = ctx.zeros(tokens * heads * D * 2)
    ctx.prefill_qkv(bufs[0], bufs[1], bufs[2] if kv else None, bufs[3], q_out, bufs[4] if kv else None, bufs[5] if kv else None, tokens, pos0, cap, heads, kv, eps,
                    scale, D)
    got_q = f16_to_f32(q_out.download(np.uint16, tokens * heads * D)).reshape(tokens, heads, D)
    for t in (0, 17, tokens - 1):
        for h in (0, heads - 1):
            want = prepared(qkv[t, h], qn, pos0 + t, True) * scale * np.log2(np.e)
            assert np.abs(got_q[t, h] - want).max() <= 2.0**-10 * np.abs(want).max() + 1e-4
    got_k, got_v = bufs[4].download(np.uint16, kc0.size), bufs[5].download(np.uint16, vc0.size)
    if kv == 0:
        assert np.array_equal(got_k, kc0) and np.array_equal(got_v, vc0)
        return
    got_k, got_v = f16_to_f32(got_k).reshape(kv, cap, D), f16_to_f32(got_v).reshape(kv, cap, D)
    old_k = f16_to_f32(kc0).reshape(kv, cap, D)
    written = {(pos0 + t) % cap for t in range(tokens)}
    for slot in range(cap):
        if slot not in written:
            assert np.array_equal(got_k[:, slot], old_k[:, slot]), "a slot outside the chunk was written"
    for t in (0, 17, tokens - 1):
        for g in range(kv):
            slot = (pos0 + t) % cap
            wk, wv = prepared(qkv[t, heads + g], kn, pos0 + t, True), prepared(qkv[t, heads + kv + g], None, pos0 + t, False)
            assert np.abs(got_k[g, slot] - wk).max() <= 2.0**-10 * np.abs(wk).max() + 1e-4
            assert np.abs(got_v[g, slot] - wv).max() <= 2.0**-10 * np.abs(wv).max() + 1e-4


def test_prefill_attention_rejects_bad_shapes(ctx):
    z = ctx.zeros(4096)
    with pytest.raises(tb.Error) as e:
        ctx.prefill_attend(z, z, z, z, 4, 0, 16, 16, 6, 4, 256)
    assert e.value.status == 3
    with pytest.raises(tb.Error):
        ctx.prefill_attend(z, z, z, z, 4, 0, 16, 16, 32, 2, 256)  # sixteen query heads to a key-value head: no kernel
    with pytest.raises(tb.Error):
        ctx.prefill_attend(z, z, z, z, 4, 0, 16, 16, 8, 2, 128)  # heads of 128: no kernel
