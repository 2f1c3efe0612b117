"""The reference's small decode kernels in its own formats, launched by name: crates/tachyon/tests/decode.rs:31-177
(geglu_q8, norm_q8, embed_q4) through tb_launch, the kernel-launch seam a caller of the reference's Stream::launch binds."""
import numpy as np
import pytest

import oracle
import tachyon_b200 as tb
from util import f16_to_f32, values

pytestmark = pytest.mark.gpu


def assert_q8(q, pairs, want, slack):
    """tests/common/mod.rs:81-91: every value within half a quantum of its block plus slack; the stored sums exact."""
    scale = np.repeat(pairs[:, 0].astype(np.float64), 32)
    got = q.astype(np.float64) * scale
    assert np.all(np.abs(got - want) <= 0.5 * scale * 1.001 + slack), float(np.abs(got - want).max())
    sums = q.reshape(-1, 32).astype(np.int32).sum(axis=1).astype(np.float32)
    assert np.array_equal((sums * pairs[:, 0]).view(np.uint32), pairs[:, 1].view(np.uint32)), "the stored sums"


def q8_out(ctx, n):
    return ctx.zeros(n), ctx.zeros(n // 32 * 8)


def q8_read(q, s, n):
    return q.download(np.int8, n), s.download(np.float32, n // 16).reshape(-1, 2)


def test_geglu_gates_then_quantizes(ctx):
    n = 10_240
    a, b = (6.0 * values(n, 1)).astype(np.float32), values(n, 2)
    ad, bd, (q, s) = ctx.upload(a), ctx.upload(b), q8_out(ctx, n)
    ctx.launch("geglu_q8", (n // 256, 1, 1), (256, 1, 1), 0, [("p", ad.ptr), ("p", bd.ptr), ("p", q.ptr), ("p", s.ptr), ("u", n)])
    x = a.astype(np.float64)
    want = 0.5 * x * (1.0 + np.tanh(np.sqrt(2.0 / np.pi) * (x + 0.044715 * x ** 3))) * b.astype(np.float64)
    assert_q8(*q8_read(q, s, n), want, 1e-5)


def rms(v, eps):
    return 1.0 / np.sqrt(np.mean(v * v) + eps)


def run_norm(ctx, h, y, w1, w2, quantize, eps, scale, length):
    n = h.size
    hd, ho = ctx.upload(h), ctx.upload(h)
    yd = None if y is None else ctx.upload(y)
    w1d, w2d = ctx.upload(w1), None if w2 is None else ctx.upload(w2)
    q, s = q8_out(ctx, n) if quantize else (None, None)
    p = lambda b: 0 if b is None else b.ptr
    ctx.launch("norm_q8", (length // 256, n // length, 1), (256, 1, 1), 0,
               [("p", hd.ptr), ("p", ho.ptr), ("p", p(yd)), ("p", w1d.ptr), ("p", p(w2d)), ("p", p(q)), ("p", p(s)), ("u", length), ("f", eps), ("f", scale)])
    assert np.array_equal(hd.download(np.float32, n), h), "the input is left alone"
    got_h = ho.download(np.float32, n)
    # the same in f64 (tests/decode.rs:83-97)
    want_h = h.astype(np.float64).copy()
    want_x = []
    for c in range(n // length):
        chunk = want_h[c * length:(c + 1) * length]
        if y is not None:
            yc = y[c * length:(c + 1) * length].astype(np.float64)
            chunk[:] = (chunk + yc * rms(yc, eps) * w1.astype(np.float64)) * np.float64(np.float32(scale))
        r = rms(chunk, eps) if w2 is not None else 1.0
        want_x.append(chunk * r * (w2.astype(np.float64) if w2 is not None else 1.0))
    want_x = np.concatenate(want_x)
    assert np.all(np.abs(got_h - want_h) <= 1e-5 * np.maximum(np.abs(want_h), 1.0))
    if quantize:
        assert_q8(*q8_read(q, s, n), want_x, 1e-5 * np.abs(want_x).max())
        return q8_read(q, s, n)


def test_norm_adds_the_residual_and_quantizes_the_next_input(ctx):
    n = 2560
    w1, w2 = (1.0 + values(n, 3)).astype(np.float32), (0.5 + values(n, 4)).astype(np.float32)
    h, y = (20.0 * values(n, 5)).astype(np.float32), (300.0 * values(n, 6)).astype(np.float32)
    run_norm(ctx, h, y, w1, w2, True, 1e-6, 0.75, n)
    run_norm(ctx, h, None, w1, w2, True, 1e-6, 1.0, n)


def test_norm_works_per_chunk_without_quantizing(ctx):
    length, chunks = 256, 42
    w1 = (1.0 + values(length, 7)).astype(np.float32)
    h, y = values(length * chunks, 8), (1e-3 * values(length * chunks, 9)).astype(np.float32)
    run_norm(ctx, h, y, w1, None, False, 1e-6 * 2560.0, float(np.float32(np.sqrt(0.5))), length)


def test_norm_without_inputs_quantizes_exactly_as_quant_q8(ctx):
    n = 2560
    h = (7.0 * values(n, 10)).astype(np.float32)
    q, s = run_norm(ctx, h, None, np.zeros(n, np.float32), None, True, 1e-6, 1.0, n)
    cq, cs = oracle.q8(h)
    assert np.array_equal(q, cq) and np.array_equal(s.view(np.uint32), cs.view(np.uint32))
    xd, (q2, s2) = ctx.upload(h), q8_out(ctx, n)
    ctx.launch("quant_q8", (n // 256, 1, 1), (256, 1, 1), 0, [("p", xd.ptr), ("p", q2.ptr), ("p", s2.ptr), ("u", n)])
    g2, p2 = q8_read(q2, s2, n)
    assert np.array_equal(g2, q) and np.array_equal(p2.view(np.uint32), s.view(np.uint32))


def test_embed_decodes_rows_of_a_q4_table(ctx):
    rows, cols = 7, 2560
    packed, scales = oracle.q4(values(rows * cols, 11).reshape(rows, cols))
    tokens = np.array([5, 0, 6], np.uint32)
    at = (tokens[:, None].astype(np.int64) * cols + np.arange(cols)[None, :])
    g, k = at // 64, at % 64
    nib = ((packed[g * 32 + k // 8 * 4 + k % 4] >> (k % 8 // 4 * 4).astype(np.uint8)) & 15).astype(np.int32) - 8
    want = nib.astype(np.float32) * f16_to_f32(scales)[g] * np.float32(50.5)
    pd, sd, td, out = ctx.upload(packed), ctx.upload(scales), ctx.upload(tokens), ctx.zeros(tokens.size * cols * 4)
    ctx.launch("embed_q4", (cols // 256, tokens.size, 1), (256, 1, 1), 0, [("p", pd.ptr), ("p", sd.ptr), ("p", td.ptr), ("p", out.ptr), ("u", cols), ("f", 50.5)])
    assert np.array_equal(out.download(np.float32, tokens.size * cols).reshape(tokens.size, cols).view(np.uint32), want.view(np.uint32))


def test_gemv_and_sampler_launch_by_name_and_bad_launches_are_refused(ctx):
    rows, cols = 64, 2048
    packed, scales = oracle.q4(values(rows * cols, 12).reshape(rows, cols))
    x = values(cols, 13)
    q, pairs = oracle.q8(x)
    wd, sd, qd, pd, yd = ctx.upload(packed), ctx.upload(scales), ctx.upload(q), ctx.upload(pairs), ctx.zeros(rows * 4)
    ctx.launch("gemv_q4", (rows // 4, 1, 1), (128, 1, 1), 0, [("p", wd.ptr), ("p", sd.ptr), ("p", qd.ptr), ("p", pd.ptr), ("p", yd.ptr), ("u", rows), ("u", cols)])
    assert np.array_equal(yd.download(np.float32, rows).view(np.uint32), oracle.gemv_q4(packed, scales, q, pairs, rows).view(np.uint32))
    vocab = 4096
    logits = (3.0 * values(vocab, 14)).astype(np.float32)
    cfg = oracle.sampling()
    ld, work, cd = ctx.upload(logits), ctx.zeros(vocab * 4), ctx.upload(np.frombuffer(bytes(cfg), np.uint8))
    state, seen, part, count = ctx.zeros(8), ctx.zeros(vocab // 8), ctx.zeros(32 * 4), ctx.zeros(4)
    ctx.launch("sample", (1, 1, 1), (1024, 1, 1), 0, [("p", ld.ptr), ("p", work.ptr), ("u", vocab), ("p", cd.ptr), ("p", state.ptr), ("p", seen.ptr), ("p", 0),
                                                    ("p", part.ptr), ("p", count.ptr)])
    assert [int(v) for v in state.download(np.uint32, 2)] == [1, int(np.argmax(logits))]
    with pytest.raises(tb.Error) as e:
        ctx.launch("attend_1024", (1, 1, 1), (32, 1, 1), 0, [])
    assert e.value.status == 8
    with pytest.raises(tb.Error) as e:
        ctx.launch("quant_q8", (1, 1, 1), (128, 1, 1), 0, [("p", ld.ptr), ("p", work.ptr), ("p", part.ptr), ("u", 32)])
    assert e.value.status == 3
    with pytest.raises(tb.Error):
        ctx.launch("geglu_q8", (1, 1, 1), (256, 1, 1), 0, [("p", ld.ptr)])


@pytest.mark.parametrize("name,per,cap,win,pos,splits,fresh,group", [(n, p, c, w, at, s, f, 1) for n, p, c, w, at, s, f in [
    ("attend_256", 4, 512, 512, 0, 16, True), ("attend_256", 4, 512, 512, 100, 16, True), ("attend_256_2", 2, 512, 512, 100, 16, True),
    ("attend_256", 4, 512, 512, 700, 16, True), ("attend_256", 4, 1024, 512, 1700, 16, True), ("attend_256_2", 2, 2048, 1024, 3000, 32, True),
    ("attend_256", 4, 2048, 2048, 1500, 64, False), ("attend_512", 4, 2048, 2048, 1500, 32, True), ("attend_512", 4, 2048, 2048, 1500, 256, False)]] + [
    ("attend_256", 4, 512, 512, 100, 16, True, 2), ("attend_512", 4, 2048, 2048, 1500, 32, True, 2)])
def test_attention_by_name_writes_q8(ctx, name, per, cap, win, pos, splits, fresh, group):
    """tests/decode.rs:185-334 through the launch seam: fifteen arguments, Q8 out, counters left at zero; `group` blocks per key-value head."""
    from util import f16, values_fast

    D, kv = 512 if name == "attend_512" else 256, 2
    heads, seed, blocks = per * group * kv, pos + 256, group * kv
    qkv = values_fast((heads + 2 * kv) * D, seed)
    qn, kn = (0.2 + 0.1 * values_fast(D, seed + 1)).astype(np.float32), (0.2 + 0.1 * values_fast(D, seed + 2)).astype(np.float32)
    freq = oracle.rope_freq(10000.0, D, 1.0) if D == 256 else oracle.rope_freq(1e6, D, 0.25)
    kc, vc = f16(0.3 * values_fast(kv * cap * D, seed + 3)), f16(0.3 * values_fast(kv * cap * D, seed + 4))
    want = oracle.attend_decode(qkv, qn, kn, freq, kc.copy(), vc.copy(), pos, cap, win, fresh, heads, kv, D, 1.0).astype(np.float64)
    b = [ctx.upload(a) for a in (qkv, qn, kn, freq, kc, vc, np.array([pos], np.uint32))]
    part, count, (q, s) = ctx.zeros(blocks * splits * (8 + per * D) * 4), ctx.zeros(4 * blocks), q8_out(ctx, heads * D)
    args = [("p", x.ptr) for x in b] + [("u", cap), ("u", win), ("u", int(fresh)), ("u", group), ("p", part.ptr), ("p", count.ptr), ("p", q.ptr), ("p", s.ptr)]
    for _ in range(2):
        ctx.launch(name, (blocks, splits, 1), (256, 1, 1), 0, args)
    assert not count.download(np.uint32, blocks).any(), "the counters are left at zero"
    assert_q8(*q8_read(q, s, heads * D), want, 1e-3 * np.abs(want).max())
    if not fresh:
        assert np.array_equal(b[4].download(np.uint16, kc.size), kc) and np.array_equal(b[5].download(np.uint16, vc.size), vc)
    with pytest.raises(tb.Error) as e:
        ctx.launch(name, (4 * blocks, splits, 1), (256, 1, 1), 0, args[:10] + [("u", 4)] + args[11:])
    assert e.value.status == 9  # sixteen query heads to one key-value head: no kernel here


@pytest.mark.parametrize("d,ratio,cap,win,p0", [(256, 4, 1024, 512, 600), (512, 4, 700, 700, 600), (256, 2, 1024, 512, 600)])
def test_prefill_attention_by_name(ctx, d, ratio, cap, win, p0):
    """tests/prefill.rs:199-236 (flash_attention_matches_the_reference): kv_* stores a chunk's keys and values, query_* the
    queries as f16, flash_* gives every token's heads over its window in f32, within a thousandth of the largest output."""
    from util import f16, f16_to_f32, values_fast

    KV, TOKENS = 2, 40
    heads, rows = ratio * KV, (ratio + 2) * KV
    qkv = values_fast(TOKENS * rows * d, 3).reshape(TOKENS, rows, d)
    qn, kn = (0.2 + 0.1 * values_fast(d, 4)).astype(np.float32), (0.2 + 0.1 * values_fast(d, 5)).astype(np.float32)
    freq = oracle.rope_freq(10000.0, d, 1.0) if d == 256 else oracle.rope_freq(1e6, d, 0.25)
    kc, vc = f16(0.3 * values_fast(KV * cap * d, 6)), f16(0.3 * values_fast(KV * cap * d, 7))

    def prepared(x, w, pos, rotate):
        x = x.astype(np.float64)
        x = x / np.sqrt((x * x).mean() + 1e-6) * (1.0 if w is None else w.astype(np.float64))
        if rotate:
            ang = (np.float32(pos) * freq).astype(np.float64)
            a, b = x[: d // 2].copy(), x[d // 2:].copy()
            x = np.concatenate([a * np.cos(ang) - b * np.sin(ang), b * np.cos(ang) + a * np.sin(ang)])
        return x

    keys, vals = f16_to_f32(kc).astype(np.float64).reshape(KV, cap, d), f16_to_f32(vc).astype(np.float64).reshape(KV, cap, d)
    for t in range(TOKENS):  # the chunk's own keys and values, unrounded (prefill.rs:161-171)
        for g in range(KV):
            keys[g, (p0 + t) % cap] = prepared(qkv[t, heads + g], kn, p0 + t, True)
            vals[g, (p0 + t) % cap] = prepared(qkv[t, heads + KV + g], None, p0 + t, False)
    want = np.zeros((TOKENS, heads, d))
    for t in range(TOKENS):
        p = p0 + t
        js = np.arange(max(0, p - win + 1), p + 1)
        for h in range(heads):
            q = prepared(qkv[t, h], qn, p, True)
            s = keys[h // ratio, js % cap] @ q
            w = np.exp(s - s.max())
            want[t, h] = (w / w.sum()) @ vals[h // ratio, js % cap]

    b = [ctx.upload(a) for a in (qkv, qn, kn, freq, kc, vc, np.array([p0], np.uint32))]
    qh, y = ctx.zeros(48 * heads * d * 2), ctx.zeros(TOKENS * heads * d * 4)
    sfx = "512" if d == 512 else "256"
    ctx.launch("kv_" + sfx, (KV, TOKENS, 1), (32, 1, 1), 0, [("p", b[0].ptr), ("p", b[2].ptr), ("p", b[3].ptr), ("p", b[4].ptr), ("p", b[5].ptr), ("p", b[6].ptr),
                                                          ("u", cap), ("u", ratio)])
    ctx.launch("query_" + sfx, (heads, TOKENS, 1), (32, 1, 1), 0, [("p", b[0].ptr), ("p", b[1].ptr), ("p", b[3].ptr), ("p", qh.ptr), ("p", b[6].ptr), ("u", rows * d)])
    name = "flash_512" if d == 512 else ("flash_256_2" if ratio == 2 else "flash_256")
    per, tile = (2, 32) if ratio == 2 else (4, 8 if d == 512 else 16)
    ctx.launch(name, (-(-TOKENS // tile), heads // per, 1), (256, 1, 1), 0, [("p", qh.ptr), ("p", b[4].ptr), ("p", b[5].ptr), ("p", b[6].ptr), ("u", cap), ("u", win),
                                                                            ("u", 1), ("u", TOKENS), ("p", y.ptr)])
    got = y.download(np.float32, TOKENS * heads * d).reshape(TOKENS, heads, d)
    top = np.abs(want).max()
    assert np.abs(got - want).max() <= 1e-3 * top, float(np.abs(got - want).max() / top)
    # the stored keys: the chunk's slots rewritten, every other slot as it was
    k_after = f16_to_f32(b[4].download(np.uint16, kc.size)).reshape(KV, cap, d)
    slots = {(p0 + t) % cap for t in range(TOKENS)}
    untouched = [s for s in range(cap) if s not in slots]
    assert np.array_equal(k_after[:, untouched], f16_to_f32(kc).reshape(KV, cap, d)[:, untouched])
    assert np.abs(k_after[:, sorted(slots)] - keys[:, sorted(slots)]).max() <= 2.0**-10 * np.abs(keys).max()
    with pytest.raises(tb.Error):
        ctx.launch("flash_256", (3, 2, 1), (256, 1, 1), 0, [("p", qh.ptr), ("p", b[4].ptr)])  # nine arguments
