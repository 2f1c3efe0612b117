"""Kernel-level parity of two kernels the model tests only reach through whole forward passes: the prefill chunk's residual /
RMS-norm step (`prefill_norm_kernel`, the place of the reference's norm_q8p: crates/tachyon/src/ptx/mod.rs:217-249) against
f64, and the encoder's pooling (`enc_pool_part_kernel` + `enc_pool_kernel`, encoder/run.rs:160-173, encoder/text.rs:56-63)
against numpy on the hidden states the encoder hands out."""
import numpy as np
import pytest

import tachyon_b200 as tb
from util import f16_to_f32

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("tokens", [1, 7, 300])
@pytest.mark.parametrize("residual,weights", [(True, True), (False, True), (True, False), (False, False)])
def test_prefill_norm_against_f64(ctx, tokens, residual, weights):
    n, eps, hscale = 2048, 1e-6, 0.75
    rng = np.random.default_rng(tokens + 2 * residual + weights)
    h = (20.0 * rng.standard_normal((tokens, n))).astype(np.float32)
    y = (300.0 * rng.standard_normal((tokens, n))).astype(np.float32)
    w1 = (1.0 + 0.2 * rng.standard_normal(n)).astype(np.float32)
    w2 = (0.5 + 0.2 * rng.standard_normal(n)).astype(np.float32)
    hd, yd, w1d, w2d = ctx.upload(h), ctx.upload(y), ctx.upload(w1), ctx.upload(w2)
    x = ctx.alloc((tokens + 1) * n * 2)
    x.upload(np.full((tokens + 1) * n, 0x3C00, np.uint16))
    tb.check(ctx.lib.tb_prefill_norm(ctx.handle, hd.ptr, yd.ptr if residual else None, w1d.ptr if residual else None, w2d.ptr if weights else None, tokens, n, eps,
                                     hscale, x.ptr))
    h64 = h.astype(np.float64)
    if residual:
        y64 = y.astype(np.float64)
        h64 = (h64 + y64 / np.sqrt((y64 * y64).mean(axis=1, keepdims=True) + eps) * w1) * hscale
    want = h64 / np.sqrt((h64 * h64).mean(axis=1, keepdims=True) + eps) * w2 if weights else h64
    got_h = hd.download(np.float32, tokens * n).reshape(tokens, n)
    assert np.abs(got_h - h64).max() <= 2e-6 * np.abs(h64).max(), "the residual stream, updated in place (or left as it was)"
    got = x.download(np.uint16, (tokens + 1) * n)
    assert np.all(got[tokens * n:] == 0x3C00), "the row past the tokens was written"
    got_x = f16_to_f32(got[: tokens * n]).reshape(tokens, n)
    assert np.all(np.abs(got_x - want) <= 2.0**-10 * np.abs(want) + 1e-6 * np.abs(want).max()), "f16 of the normalised row"
    assert ctx.status() == 0


def test_prefill_norm_refuses_other_widths(ctx):
    h, x = ctx.zeros(4 * 1024 * 4), ctx.zeros(4 * 1024 * 2)
    assert ctx.lib.tb_prefill_norm(ctx.handle, h.ptr, None, None, None, 4, 1024, 1e-6, 1.0, x.ptr) == 9  # TB_UNSUPPORTED
    assert ctx.lib.tb_prefill_norm(ctx.handle, h.ptr, h.ptr, None, None, 4, 2048, 1e-6, 1.0, x.ptr) == 3  # a residual without its weights


@pytest.mark.parametrize("mean,dims", [(1, 256), (1, 96), (0, 256), (0, 64)])
def test_pooling_from_the_hidden_states(ctx, mean, dims):
    """Sequences of 1 to 70 tokens (fewer tokens than parts of the sum, exactly as many, and more), mean or first token,
    all dimensions or a truncated embedding."""
    cfg = tb.EncoderConfig(vocab=512, hidden=256, layers=1, heads=4, inter=256, window=8, global_=None, global_every=1, theta_global=10000.0, theta_local=10000.0,
                           eps=1e-5, gated=0, mean_pool=mean, dims=dims)
    enc = tb.Encoder(ctx, cfg, tokens=512, sequences=16)
    enc.fill_random(5)
    lens = [1, 3, 8, 9, 33, 70, 16, 64]
    rng = np.random.default_rng(7)
    got = enc.embed([rng.integers(0, cfg.vocab, size=n).astype(np.uint32) for n in lens])
    hidden = enc.hidden().astype(np.float64)
    at = 0
    for s, n in enumerate(lens):
        v = hidden[at:at + n].mean(axis=0) if mean else hidden[at]
        v = v / max(np.sqrt((v * v).sum()), 1e-12)
        v = v[:dims]
        if dims < cfg.hidden:
            v = v / max(np.sqrt((v * v).sum()), 1e-12)
        assert np.abs(got[s] - v).max() <= 2e-6, (s, n)
        at += n
    enc.close()
