"""Prefill GEMM (tcgen05, Q8 weights dequantised to f16 in the operand path) against f64 on the CPU.  Shapes follow
crates/tachyon/tests/gemm.rs:17 in spirit (ragged token counts, one and several K tiles) at this build's widths."""
import numpy as np
import pytest

import oracle
import tachyon_b200 as tb
from util import f16, f16_to_f32, q8_weights

pytestmark = pytest.mark.gpu

# (tokens, rows, cols)
SHAPES = [(128, 128, 64), (128, 128, 256), (1, 128, 2048), (37, 256, 2048), (300, 3072, 2048), (512, 2048, 2048), (129, 2048, 16384), (256, 96, 128)]


SCHEDULES = {"one tile per block": "1", "persistent": "2", "pairs of SMs, tiles of 256 weight rows": "3", "pairs of SMs, tiles of 128 weight rows": "4",
             "one tile at a time, blocks walking the tiles (f16 weights; as the first otherwise)": "5"}


@pytest.fixture(params=list(SCHEDULES))
def schedule(request, ctx):
    """Every schedule of the GEMM (tb_context_set_gemm_schedule); left to itself the library picks by shape."""
    tb.check(ctx.lib.tb_context_set_gemm_schedule(ctx.handle, int(SCHEDULES[request.param])))
    yield request.param
    tb.check(ctx.lib.tb_context_set_gemm_schedule(ctx.handle, 0))


def reference(w, s, a):
    deq = w.astype(np.float64) * np.repeat(f16_to_f32(s).astype(np.float64), 32, axis=1)
    a64 = a.astype(np.float64)
    return a64 @ deq.T, np.abs(a64) @ np.abs(deq).T


@pytest.mark.parametrize("m,n,k", SHAPES)
def test_gemm_matches_f64(ctx, schedule, m, n, k):
    w, s = q8_weights(n, k, 7 + n + k)
    a = f16_to_f32(f16(np.random.default_rng(m + k).standard_normal((m, k)).astype(np.float32)))
    want, bound = reference(w, s, a)
    wd, sd, ad = ctx.upload(w), ctx.upload(s), ctx.upload(f16(a))
    out = ctx.alloc((m + 3) * n * 4)
    canary = np.full((m + 3) * n, 12345.0, np.float32)
    out.upload(canary)
    ctx.gemm_q8(wd, sd, ad, m, n, k, out, 0)
    got = out.download(np.float32, (m + 3) * n)
    assert np.all(got[m * n:] == 12345.0), "rows past the tokens were written"
    got = got[: m * n].reshape(m, n)
    # weights are rounded to f16 after scaling (2^-11 relative each); the accumulation is f32
    assert np.all(np.abs(got - want) <= 1e-3 * bound + 1e-6), float(np.abs(got - want).max())
    # f16 output
    out16 = ctx.zeros(m * n * 2)
    ctx.gemm_q8(wd, sd, ad, m, n, k, out16, 1)
    got16 = f16_to_f32(out16.download(np.uint16, m * n)).reshape(m, n)
    assert np.all(np.abs(got16 - want) <= 2.0**-10 * np.abs(want) + 1e-3 * bound + 1e-6)
    assert ctx.status() == 0


def test_gemm_geglu_epilogue(ctx, schedule):
    m, n, k = 200, 1024, 2048
    w, s = q8_weights(n, k, 3)
    a = f16_to_f32(f16(np.random.default_rng(5).standard_normal((m, k)).astype(np.float32)))
    want, bound = reference(w, s, a)
    gate, up = want[:, 0::2], want[:, 1::2]
    gelu = np.vectorize(lambda v: oracle.lib().tbo_gelu_tanh(float(v)))
    ref = gelu(gate) * up
    out = ctx.zeros(m * n)
    ctx.gemm_q8(ctx.upload(w), ctx.upload(s), ctx.upload(f16(a)), m, n, k, out, 2)
    got = f16_to_f32(out.download(np.uint16, m * n // 2)).reshape(m, n // 2)
    tol = 2.0**-9 * np.abs(ref) + 2e-3 * (bound[:, 0::2] * (1 + np.abs(up)) + bound[:, 1::2] * (1 + np.abs(gate))) * 0.05 + 1e-4
    assert np.all(np.abs(got - ref) <= tol), float(np.abs(got - ref).max())


def test_gemm_rejects_bad_shapes(ctx):
    z = ctx.zeros(4096)
    with pytest.raises(tb.Error) as e:
        ctx.gemm_q8(z, z, z, 4, 32, 48, z, 0)  # K not a multiple of 64
    assert e.value.status == 3
    with pytest.raises(tb.Error):
        ctx.gemm_q8(z, z, z, 4, 32, 64, z, 9)


@pytest.mark.parametrize("m,n,k", [(128, 128, 64), (37, 256, 2048), (300, 3072, 2048), (129, 2048, 16384), (256, 96, 128), (64, 64, 576)])
def test_gemm_q4_matches_f64(ctx, schedule, m, n, k):
    """The reference's Q4 weights (quant.rs:47-82) through the same tensor-core product: (n - 8) * scale as f16 operands."""
    wf = np.random.default_rng(n + k).uniform(-1, 1, (n, k)).astype(np.float32)
    packed, scales = oracle.q4(wf)
    nib = np.zeros((n * k // 64, 64), np.float64)
    pk = packed.reshape(-1, 32)
    for j in range(64):  # weight j of a group: nibble j % 8 / 4 of byte j / 8 * 4 + j % 4
        nib[:, j] = (pk[:, j // 8 * 4 + j % 4] >> (j % 8 // 4 * 4)) & 15
    deq = ((nib - 8) * f16_to_f32(scales).astype(np.float64)[:, None]).reshape(n, k)
    a = f16_to_f32(f16(np.random.default_rng(m + k).standard_normal((m, k)).astype(np.float32)))
    a64 = a.astype(np.float64)
    want, bound = a64 @ deq.T, np.abs(a64) @ np.abs(deq).T
    out = ctx.alloc((m + 1) * n * 4)
    out.upload(np.full((m + 1) * n, 12345.0, np.float32))
    ctx.gemm_q4(ctx.upload(packed), ctx.upload(scales), ctx.upload(f16(a)), m, n, k, out, 0)
    got = out.download(np.float32, (m + 1) * n)
    assert np.all(got[m * n:] == 12345.0)
    got = got[: m * n].reshape(m, n)
    assert np.all(np.abs(got - want) <= 1e-3 * bound + 1e-6), float(np.abs(got - want).max())
    assert ctx.status() == 0


@pytest.mark.parametrize("m,n,k", [(128, 128, 64), (37, 256, 768), (300, 2304, 768), (512, 768, 3072), (129, 3072, 768), (64, 64, 576)])
def test_gemm_f16_weights_and_every_store_mode(ctx, schedule, m, n, k):
    """tb_gemm_f16: f16 weights as they are (the reference's gemm_f16, tests/encoder.rs:240-355: all modes, rows past the
    tokens untouched), against f64; and the store modes the Q8 test above does not reach: residual add, exact-form GELU plain
    and gated, ReLU, gated SiLU."""
    rng = np.random.default_rng(m + n + k)
    w = f16(rng.standard_normal((n, k)).astype(np.float32) * np.float32(0.05))
    a = f16(rng.standard_normal((m, k)).astype(np.float32))
    w64, a64 = f16_to_f32(w).astype(np.float64), f16_to_f32(a).astype(np.float64)
    want, bound = a64 @ w64.T, np.abs(a64) @ np.abs(w64).T
    wd, ad = ctx.upload(w), ctx.upload(a)
    erf = np.vectorize(lambda v: float(oracle.lib().tbo_erf_as(np.float32(v))))
    gelu = lambda v: 0.5 * v * (1.0 + erf(v * 0.70710678118))
    silu = lambda v: v / (1.0 + np.exp(-v))
    out = ctx.alloc((m + 2) * n * 4)
    # f32 store, then the residual add on top of it
    out.upload(np.full((m + 2) * n, 9.0, np.float32))
    ctx.gemm_f16(wd, ad, m, n, k, out, 0)
    got = out.download(np.float32, (m + 2) * n)
    assert np.all(got[m * n:] == 9.0), "rows past the tokens were written"
    assert np.all(np.abs(got[: m * n].reshape(m, n) - want) <= 1e-5 * bound + 1e-6), float(np.abs(got[: m * n].reshape(m, n) - want).max())
    ctx.gemm_f16(wd, ad, m, n, k, out, 3)
    assert np.all(np.abs(out.download(np.float32, m * n).reshape(m, n) - 2 * want) <= 2e-5 * bound + 2e-6)
    tol16 = lambda ref, b: 2.0**-9 * np.abs(ref) + 1e-4 * b + 1e-5
    for mode, ref in ((1, want), (5, gelu(want)), (7, np.maximum(want, 0.0))):
        o16 = ctx.zeros(m * n * 2)
        ctx.gemm_f16(wd, ad, m, n, k, o16, mode)
        got16 = f16_to_f32(o16.download(np.uint16, m * n)).reshape(m, n)
        assert np.all(np.abs(got16 - ref) <= tol16(ref, bound)), (mode, float(np.abs(got16 - ref).max()))
    if n % 64 == 0:
        even, odd, be, bo = want[:, 0::2], want[:, 1::2], bound[:, 0::2], bound[:, 1::2]
        for mode, ref in ((4, gelu(even) * odd), (8, silu(even) * odd)):
            o16 = ctx.zeros(m * n)
            ctx.gemm_f16(wd, ad, m, n, k, o16, mode)
            got16 = f16_to_f32(o16.download(np.uint16, m * n // 2)).reshape(m, n // 2)
            tol = 2.0**-9 * np.abs(ref) + 1e-4 * (be * (1 + np.abs(odd)) + bo * (1 + np.abs(even))) + 1e-5
            assert np.all(np.abs(got16 - ref) <= tol), (mode, float(np.abs(got16 - ref).max()))
    assert ctx.status() == 0


def test_gemm_q8_relu_and_gated_silu(ctx):
    m, n, k = 200, 512, 768
    w, s = q8_weights(n, k, 9)
    a = f16_to_f32(f16(np.random.default_rng(10).standard_normal((m, k)).astype(np.float32)))
    want, bound = reference(w, s, a)
    wd, sd, ad = ctx.upload(w), ctx.upload(s), ctx.upload(f16(a))
    o = ctx.zeros(m * n * 2)
    ctx.gemm_q8(wd, sd, ad, m, n, k, o, 7)
    got = f16_to_f32(o.download(np.uint16, m * n)).reshape(m, n)
    assert np.all(np.abs(got - np.maximum(want, 0.0)) <= 2.0**-9 * np.abs(want) + 1e-3 * bound + 1e-5)
    ctx.gemm_q8(wd, sd, ad, m, n, k, o, 8)
    even, odd = want[:, 0::2], want[:, 1::2]
    ref = even / (1.0 + np.exp(-even)) * odd
    got = f16_to_f32(o.download(np.uint16, m * n // 2)).reshape(m, n // 2)
    tol = 2.0**-9 * np.abs(ref) + 1e-3 * (bound[:, 0::2] * (1 + np.abs(odd)) + bound[:, 1::2] * (1 + np.abs(even))) + 1e-5
    assert np.all(np.abs(got - ref) <= tol)


@pytest.mark.parametrize("bits", [8, 4])
@pytest.mark.parametrize("m,n,k", [(300, 2304, 768), (512, 768, 3072), (37, 96, 128)])
def test_dequantised_copy_holds_the_products_own_operands(ctx, bits, m, n, k):
    """tb_dequant_f16 writes code * scale rounded once to f16, the value the Q8 / Q4 products build in their operand path, so
    tb_gemm_f16 on the copy gives tb_gemm_q8 / tb_gemm_q4's bits (the decoder's prefill copy leans on exactly that)."""
    rng = np.random.default_rng(bits + m + n + k)
    if bits == 8:
        w, s = q8_weights(n, k, 21 + n + k)
        exact = w.astype(np.float32) * np.repeat(f16_to_f32(s), 32, axis=1)
        wd, sd = ctx.upload(w), ctx.upload(s)
    else:
        packed, s = oracle.q4((rng.standard_normal((n, k)) * 0.05).astype(np.float32))
        packed, s = np.asarray(packed, np.uint8).reshape(n, k // 2), np.asarray(s, np.uint16).reshape(n, k // 64)
        nib = np.empty((n, k // 8, 8), np.float32)  # a word of four bytes: low nibbles are weights 0..3, high nibbles 4..7
        words = packed.reshape(n, k // 8, 4)
        nib[:, :, :4], nib[:, :, 4:] = words & 15, words >> 4
        exact = (nib.reshape(n, k) - 8.0) * np.repeat(f16_to_f32(s), 64, axis=1)
        wd, sd = ctx.upload(packed), ctx.upload(s)
    copy = ctx.zeros(n * k * 2)
    ctx.dequant_f16(wd, sd, n, k, bits, copy)
    got = copy.download(np.uint16, n * k).reshape(n, k)
    assert np.array_equal(got, f16(exact)), "code * scale, rounded once"
    a = ctx.upload(f16(rng.standard_normal((m, k)).astype(np.float32)))
    o1, o2 = ctx.zeros(m * n * 4), ctx.zeros(m * n * 4)
    tb.check(ctx.lib.tb_context_set_gemm_schedule(ctx.handle, 1))
    try:
        if bits == 8:
            ctx.gemm_q8(wd, sd, a, m, n, k, o1, 0)
        else:
            tb.check(ctx.lib.tb_gemm_q4(ctx.handle, wd.ptr, sd.ptr, a.ptr, m, n, k, o1.ptr, 0))
    finally:
        tb.check(ctx.lib.tb_context_set_gemm_schedule(ctx.handle, 0))
    ctx.gemm_f16(copy, a, m, n, k, o2, 0)
    assert np.array_equal(o1.download(np.uint32, m * n), o2.download(np.uint32, m * n)), "the same operands, the same sums"
    assert ctx.status() == 0
