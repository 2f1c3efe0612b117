"""Greedy sampling and top-k on the GPU against the oracle (crates/tachyon/tests/sample.rs:92-110), plus the embedding
row and the stand-alone norm step (crates/tachyon/tests/decode.rs:100-177)."""
import numpy as np
import pytest

import oracle
import tachyon_b200 as tb
from util import f16_to_f32, q8_weights, values_fast

pytestmark = pytest.mark.gpu


def test_greedy_picks_the_largest_transformed_logit(ctx):
    vocab = 262_144
    logits = (40.0 * values_fast(vocab, 1)).astype(np.float32)
    seen = np.array([0xF0F0F0F0 if i % 3 == 0 else 0 for i in range(vocab // 32)], np.uint32)
    allowed = np.array([0 if i % 5 == 0 else 0xFFFFFFFF for i in range(vocab // 32)], np.uint32)
    want, gap = oracle.sample_greedy(logits, softcap=30.0, penalty=1.3, seen=seen, allowed=allowed)
    ld, sd, ad = ctx.upload(logits), ctx.upload(seen), ctx.upload(allowed)
    scratch, state, out = ctx.zeros(16), ctx.zeros(8), ctx.zeros(4)
    for step in (1, 2):
        sd.upload(seen)
        ctx.sample_greedy(ld, vocab, 30.0, 1.3, sd, ad, scratch, state, out)
        st = state.download(np.uint32, 2)
        if gap > 1e-4:  # bit-exact whenever the top-2 gap exceeds the float noise of tanh
            assert (int(st[0]), int(st[1])) == (step, want)
            assert int(out.download(np.uint32, 1)[0]) == want
            assert (int(sd.download(np.uint32, vocab // 32)[want // 32]) >> (want % 32)) & 1 == 1, "token marked as seen"
        assert not scratch.download(np.uint32, 4).any()


def test_greedy_without_transform_and_ties(ctx):
    vocab = 5000
    logits = values_fast(vocab, 3)
    logits[[77, 4000]] = 5.0
    ld, scratch, state = ctx.upload(logits), ctx.zeros(16), ctx.zeros(8)
    ctx.sample_greedy(ld, vocab, 0.0, 1.0, None, None, scratch, state, None)
    assert int(state.download(np.uint32, 2)[1]) == 77


def test_topk_orders_by_value_then_index(ctx):
    vocab = 262_144
    logits = (40.0 * values_fast(vocab, 7)).astype(np.float32)
    logits[[5, 9000]] = 39.99
    k = 40
    idx, val = ctx.zeros(4 * k), ctx.zeros(4 * k)
    ctx.topk(ctx.upload(logits), vocab, k, idx, val)
    want_i, want_v = oracle.sample_topk(logits, k)
    assert np.array_equal(idx.download(np.uint32, k), want_i)
    assert np.array_equal(val.download(np.float32, k), want_v)


def test_embed_row_is_dequantised_and_scaled(ctx):
    vocab, cols = 300, 2048
    w, s = q8_weights(vocab, cols, 4)
    out = ctx.zeros(cols * 4)
    for token in (0, 123, 299):
        ctx.embed_q8(ctx.upload(w), ctx.upload(s), ctx.upload(np.array([token], np.uint32)), cols, 45.25, out)
        want = w[token].astype(np.float32) * np.repeat(f16_to_f32(s[token]), 32) * np.float32(45.25)
        assert np.allclose(out.download(np.float32, cols), want, rtol=1e-6, atol=0)


def test_norm_adds_the_residual_and_normalises_the_next_input(ctx):
    n = 2560
    rng = np.random.default_rng(5)
    w1, w2 = (1 + rng.uniform(-1, 1, n)).astype(np.float32), (0.5 + rng.uniform(-1, 1, n)).astype(np.float32)
    h, y = (20 * rng.uniform(-1, 1, n)).astype(np.float32), (300 * rng.uniform(-1, 1, n)).astype(np.float32)
    for yres, scale, use_w2 in [(y, 0.75, True), (None, 1.0, True), (y, 1.0, False)]:
        h_want, x_want = oracle.norm_step(h, yres, w1 if yres is not None else None, w2 if use_w2 else None, 1e-6, scale)
        ho, xo = ctx.zeros(n * 4), ctx.zeros(n * 4)
        ctx.norm(ctx.upload(h), None if yres is None else ctx.upload(y), None if yres is None else ctx.upload(w1), ctx.upload(w2) if use_w2 else None, n, 1e-6,
                 scale, ho, xo)
        assert np.all(np.abs(ho.download(np.float32, n) - h_want) <= 1e-5 * np.maximum(np.abs(h_want), 1.0))
        assert np.all(np.abs(xo.download(np.float32, n) - x_want) <= 1e-5 * np.maximum(np.abs(x_want).max(), 1.0))


def test_device_fills_match_the_cpu_generators_bit_for_bit(ctx):
    import ctypes as C

    n = 100_003
    lib = ctx.lib
    codes, scales, gauss, uni = ctx.zeros(n), ctx.zeros(2 * n), ctx.zeros(2 * n), ctx.zeros(4 * n)
    tb.check(lib.tb_fill_codes(ctx.handle, 7, 3, codes.ptr, n))
    tb.check(lib.tb_fill_scales(ctx.handle, 7, 4, scales.ptr, n, C.c_float(0.02 / 127)))
    tb.check(lib.tb_fill_gauss_f16(ctx.handle, 7, 5, gauss.ptr, n, C.c_float(1.0)))
    tb.check(lib.tb_fill_uniform(ctx.handle, 7, 6, uni.ptr, n, C.c_float(0.15), C.c_float(0.35)))
    assert np.array_equal(codes.download(np.int8, n), oracle.fill_codes(7, 3, n))
    assert np.array_equal(scales.download(np.uint16, n), oracle.fill_scales(7, 4, n, 0.02 / 127))
    assert np.array_equal(gauss.download(np.uint16, n), oracle.fill_gauss_f16(7, 5, n, 1.0))
    assert np.array_equal(uni.download(np.float32, n), oracle.fill_uniform(7, 6, n, 0.15, 0.35))


# ---- the sampler with draws: crates/tachyon/tests/sample.rs:74-183 ----

BLOCKS = 7  # tests/sample.rs:13: fewer blocks than the vocabulary needs, so each walks several shares


class Slot:
    """A device address inside a buffer someone else owns."""

    def __init__(self, ptr):
        self.ptr = ptr


class Sampler:
    def __init__(self, ctx, logits, seen, allowed, cfg):
        self.ctx, self.vocab, self.seen0 = ctx, logits.size, seen
        self.allowed = ctx.upload(allowed)
        if cfg.allowed:
            cfg.allowed = self.allowed.ptr
        self.cfg_host = cfg
        self.logits, self.work = ctx.upload(logits), ctx.zeros(logits.size * 4)
        self.cfg = ctx.upload(np.frombuffer(bytes(cfg), np.uint8))
        self.state, self.seen = ctx.zeros(8), ctx.upload(seen)
        self.partial, self.count = ctx.zeros(32 * BLOCKS), ctx.zeros(4)

    def draw(self, out=None, reset_seen=True):
        if reset_seen:
            self.seen.upload(self.seen0)
        self.ctx.sample(self.logits, self.work, self.vocab, self.cfg, self.state, self.seen, out, self.partial, self.count, BLOCKS)


def transform(logits, cfg, seen, allowed):
    """tests/sample.rs:61-72 in f64."""
    i = np.arange(logits.size)
    bit = lambda m: ((m[i // 32] >> (i % 32).astype(np.uint32)) & 1) == 1
    v = logits.astype(np.float64)
    if cfg.softcap > 0:
        v = cfg.softcap * np.tanh(v / cfg.softcap)
    s = bit(seen)
    v = np.where(s, np.where(v > 0, v / cfg.penalty, v * cfg.penalty), v)
    if cfg.allowed:
        v = np.where(bit(allowed), v, -np.inf)
    return v / cfg.temperature if cfg.temperature > 0 else v


def expected(x, cfg):
    """tests/sample.rs:75-88: softmax over the tokens every filter keeps."""
    m = x.max()
    p = np.exp(x - m)
    z = p.sum()
    keep = np.zeros(x.size, bool)
    for i in range(x.size):
        above = x > x[i]
        count, mass = int(above.sum()), float(p[above].sum())
        keep[i] = (cfg.top_k == 0 or count < cfg.top_k) and (cfg.top_p >= 1.0 or mass < float(np.float32(cfg.top_p)) * z or mass == 0.0) \
            and (x[i] - m >= (np.log(np.float64(np.float32(cfg.min_p))) if cfg.min_p > 0 else -np.inf))
    kept = np.where(keep, p, 0.0)
    return kept / kept.sum()


def test_sampler_in_greedy_mode_advances_the_step_and_marks_the_token(ctx):
    vocab = 262_144
    logits = (40.0 * values_fast(vocab, 1)).astype(np.float32)
    seen = np.array([0xF0F0F0F0 if i % 3 == 0 else 0 for i in range(vocab // 32)], np.uint32)
    allowed = np.array([0 if i % 5 == 0 else 0xFFFFFFFF for i in range(vocab // 32)], np.uint32)
    cfg = oracle.sampling(softcap=30.0, penalty=1.3, allowed=1)
    x = transform(logits, cfg, seen, allowed)
    want = int(np.argmax(x))
    order = np.sort(x)
    s = Sampler(ctx, logits, seen, allowed, cfg)
    out = ctx.zeros(4)
    for step in (1, 2):
        s.draw(out)
        if order[-1] - order[-2] > 1e-4:
            assert [int(v) for v in s.state.download(np.uint32, 2)] == [step, want]
            assert int(out.download(np.uint32, 1)[0]) == want
            assert (int(s.seen.download(np.uint32, vocab // 32)[want // 32]) >> (want % 32)) & 1 == 1
        assert int(s.count.download(np.uint32, 1)[0]) == 0


def check_draws(ctx, vocab, cfg, n=60_000):
    from util import values

    logits = (3.0 * values(vocab, cfg.top_k + 7)).astype(np.float32)
    seen = np.array([(0x01010101 << (i % 8)) & 0xFFFFFFFF for i in range(vocab // 32)], np.uint32)
    allowed = np.array([0x00FFFF00 if i % 4 == 1 else 0xFFFFFFFF for i in range(vocab // 32)], np.uint32)
    x = transform(logits, cfg, seen, allowed)
    p = expected(x, cfg)
    s = Sampler(ctx, logits, seen, allowed, cfg)
    tokens = ctx.zeros(4 * n)
    for i in range(n):
        s.draw(Slot(tokens.ptr + 4 * i), reset_seen=cfg.penalty != 1.0)  # every draw leaves its token in a slot of its own
    got = np.bincount(tokens.download(np.uint32, n), minlength=vocab)
    assert not got[p == 0].any(), "a filtered token was drawn"
    e = p[p > 0] * n
    chi2 = float((((got[p > 0] - e) ** 2) / e).sum())
    df = int((p > 0).sum()) - 1
    assert chi2 < df + 6.0 * np.sqrt(2.0 * df) + 10.0, (chi2, df)
    # the oracle restates hash and filters: the first draws are the same tokens (noise differs in the last bits only)
    first = tokens.download(np.uint32, 64)
    want = [oracle.sample_draw(logits, s.cfg_host, step, seen, allowed if cfg.allowed else None)[0] for step in range(64)]
    assert sum(int(a) != b for a, b in zip(first, want)) <= 1
    return got


def test_draws_follow_the_temperature_distribution(ctx):
    check_draws(ctx, 256, oracle.sampling(temperature=1.0, seed=1))


def test_draws_follow_top_k_across_blocks(ctx):
    got = check_draws(ctx, 8192, oracle.sampling(temperature=0.7, top_k=10, seed=2), n=30_000)
    assert (got > 0).sum() <= 10


def test_draws_follow_top_p(ctx):
    check_draws(ctx, 256, oracle.sampling(temperature=1.3, top_p=0.8, seed=3))


def test_draws_follow_min_p_softcap_penalty_and_mask(ctx):
    check_draws(ctx, 256, oracle.sampling(temperature=1.0, min_p=0.05, softcap=5.0, penalty=1.5, allowed=1, seed=4), n=30_000)


def test_draws_are_a_function_of_seed_and_step(ctx):
    vocab = 4096
    logits = (3.0 * values_fast(vocab, 11)).astype(np.float32)
    zeros = np.zeros(vocab // 32, np.uint32)
    runs = []
    for seed in (5, 5, 6):
        s = Sampler(ctx, logits, zeros, zeros, oracle.sampling(temperature=1.0, top_p=0.95, seed=seed))
        toks = []
        for _ in range(24):
            s.draw()
            toks.append(int(s.state.download(np.uint32, 2)[1]))
        runs.append(toks)
    assert runs[0] == runs[1] and runs[0] != runs[2] and len(set(runs[0])) > 4
