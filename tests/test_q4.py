"""The reference's own decode formats: Q8 activation quantisation and the Q4 x Q8 matrix-vector product.

Mirrors crates/tachyon/tests/gemv.rs: `quant_q8_matches_the_cpu_exactly` and `gemv_matches_the_reference_on_every_shape`
(same seeded values, same shapes, same bound `1e-5 * bound + 1e-6` against the f64 product of tests/common/mod.rs:95-112),
plus what this build can add: the oracle repeats the reference kernel's f32 operations in the kernel's order, and the GPU
must give the oracle's bits."""
import numpy as np
import pytest

import oracle
import tachyon_b200 as tb
from util import values, values_fast

# crates/tachyon/tests/gemv.rs:16 and the decode projections of the benchmark's model (staged path: 2048, 4096, 16384 wide).
SHAPES = [(512, 2560), (512, 2048), (512, 4096), (256, 10240), (37, 2560), (5, 64), (3, 192), (2560, 256), (36, 64),
          (3072, 2048), (37, 2048), (1, 2048), (300, 512), (96, 1024), (64, 8192), (2048, 16384), (37, 16384)]


def inputs(rows, cols, i):
    gen = values if rows * cols <= 1 << 16 else values_fast  # the reference's xorshift generator is a Python loop here
    return gen(rows * cols, 11 + i), gen(cols, 99 + i)


@pytest.mark.parametrize("i,shape", list(enumerate(SHAPES[:9] + [(64, 2048), (8, 16384)])))
def test_oracle_kernel_order_meets_the_reference_bound(i, shape):
    """CPU only: the kernel-order restatement stays within the reference test's bound of the f64 product."""
    rows, cols = shape
    wf, x = inputs(rows, cols, i)
    packed, scales = oracle.q4(wf.reshape(rows, cols))
    q, pairs = oracle.q8(x)
    y = oracle.gemv_q4(packed, scales, q, pairs, rows)
    want, bound = oracle.product_q4(packed, scales, x, rows)
    assert np.all(np.abs(y.astype(np.float64) - want) <= 1e-5 * bound + 1e-6)


NARROW = [(2560, 256), (36, 64), (4, 192), (16, 128), (260, 256)]  # gemv.rs:7-9: rows a multiple of 4, at most 256 weights each


@pytest.mark.parametrize("i,shape", list(enumerate(NARROW)))
def test_oracle_narrow_order_meets_the_reference_bound(i, shape):
    """CPU only: eight lanes a row add in another order than thirty-two; both stay within the reference's bound."""
    rows, cols = shape
    wf, x = inputs(rows, cols, 40 + i)
    packed, scales = oracle.q4(wf.reshape(rows, cols))
    q, pairs = oracle.q8(x)
    narrow, wide = oracle.gemv_q4_narrow(packed, scales, q, pairs, rows), oracle.gemv_q4(packed, scales, q, pairs, rows)
    want, bound = oracle.product_q4(packed, scales, x, rows)
    assert np.all(np.abs(narrow.astype(np.float64) - want) <= 1e-5 * bound + 1e-6)
    assert np.all(np.abs(narrow.astype(np.float64) - wide) <= 2e-5 * bound + 2e-6)
    if cols == 64:  # two chunks: lanes 0 and 1 either way, one addition
        assert np.array_equal(narrow, wide)


@pytest.mark.gpu
@pytest.mark.parametrize("i,shape", list(enumerate(NARROW)))
def test_gemv_q4_narrow_gives_the_reference_kernels_bits(ctx, i, shape):
    rows, cols = shape
    wf, x = inputs(rows, cols, 40 + i)
    packed, scales = oracle.q4(wf.reshape(rows, cols))
    xd, qd, sd = ctx.upload(x), ctx.zeros(cols), ctx.zeros(cols // 32 * 8)
    ctx.quant_q8(xd, cols, qd, sd)
    wd, wsd, yd = ctx.upload(packed), ctx.upload(scales), ctx.zeros(rows * 4)
    ctx.launch("gemv_q4_narrow", ((rows + 15) // 16, 1, 1), (128, 1, 1), 0,
               [("p", wd.ptr), ("p", wsd.ptr), ("p", qd.ptr), ("p", sd.ptr), ("p", yd.ptr), ("u", rows), ("u", cols)])
    got = yd.download(np.float32, rows)
    q, pairs = oracle.q8(x)
    assert np.array_equal(got.view(np.uint32), oracle.gemv_q4_narrow(packed, scales, q, pairs, rows).view(np.uint32)), f"{rows}x{cols}"
    with pytest.raises(tb.Error):
        ctx.launch("gemv_q4_narrow", ((rows + 15) // 16, 1, 1), (128, 1, 1), 0,
                   [("p", wd.ptr), ("p", wsd.ptr), ("p", qd.ptr), ("p", sd.ptr), ("p", yd.ptr), ("u", rows), ("u", 512)])  # rows too long
    with pytest.raises(tb.Error):
        ctx.launch("gemv_q4_narrow", (1, 1, 1), (128, 1, 1), 0,
                   [("p", wd.ptr), ("p", wsd.ptr), ("p", qd.ptr), ("p", sd.ptr), ("p", yd.ptr), ("u", 6), ("u", cols)])  # rows not a multiple of 4


@pytest.mark.gpu
def test_quant_q8_matches_the_cpu_exactly(ctx):
    x = values(4096, 7)
    x[64:96] = 0.0
    x[100] = 1e-30
    xd, qd, sd = ctx.upload(x), ctx.zeros(x.size), ctx.zeros(x.size // 32 * 8)
    ctx.quant_q8(xd, x.size, qd, sd)
    cq, cs = oracle.q8(x)
    assert np.array_equal(qd.download(np.int8, x.size), cq), "Q8 values differ"
    assert np.array_equal(sd.download(np.float32, x.size // 16).view(np.uint32), cs.ravel().view(np.uint32)), "Q8 scales differ"


def gpu_gemv(ctx, packed, scales, x, rows):
    cols = x.size
    xd, qd, sd = ctx.upload(x), ctx.zeros(cols), ctx.zeros(cols // 32 * 8)
    ctx.quant_q8(xd, cols, qd, sd)
    wd, wsd, yd = ctx.upload(packed), ctx.upload(scales), ctx.zeros(rows * 4)
    ctx.gemv_q4(wd, wsd, qd, sd, yd, rows, cols)
    return yd.download(np.float32, rows)


@pytest.mark.gpu
@pytest.mark.parametrize("i,shape", list(enumerate(SHAPES)))
def test_gemv_q4_gives_the_reference_kernels_bits_on_every_shape(ctx, i, shape):
    rows, cols = shape
    wf, x = inputs(rows, cols, i)
    packed, scales = oracle.q4(wf.reshape(rows, cols))
    got = gpu_gemv(ctx, packed, scales, x, rows)
    q, pairs = oracle.q8(x)
    assert np.array_equal(got.view(np.uint32), oracle.gemv_q4(packed, scales, q, pairs, rows).view(np.uint32)), f"{rows}x{cols}"
    want, bound = oracle.product_q4(packed, scales, x, rows)
    assert np.all(np.abs(got.astype(np.float64) - want) <= 1e-5 * bound + 1e-6)


@pytest.mark.gpu
def test_gemv_q4_stays_close_to_the_unquantized_product(ctx):
    rows, cols = 512, 2560
    wf, x = values_fast(rows * cols, 3), values_fast(cols, 4)
    packed, scales = oracle.q4(wf.reshape(rows, cols))
    y = gpu_gemv(ctx, packed, scales, x, rows).astype(np.float64)
    exact = wf.reshape(rows, cols).astype(np.float64) @ x.astype(np.float64)
    assert np.linalg.norm(y - exact) / np.linalg.norm(exact) < 0.15


@pytest.mark.gpu
def test_gemv_q4_rejects_what_it_cannot_run(ctx):
    d = ctx.zeros(4096)
    with pytest.raises(tb.Error):
        ctx.gemv_q4(d, d, d, d, d, 4, 96)  # not whole groups of 64
    with pytest.raises(tb.Error):
        ctx.quant_q8(d, 48, d, d)


@pytest.mark.gpu
@pytest.mark.parametrize("rows,cols", [(3072, 2048), (37, 2048), (1, 2048), (300, 4096), (64, 8192), (2048, 16384), (37, 16384)])
def test_gemv_q4x_reads_q4_weights_with_an_unrounded_activation(ctx, rows, cols):
    """The decode product on the reference's converted weights: f32 accuracy against the f64 product."""
    wf, x = values_fast(rows * cols, 21 + rows), np.random.default_rng(cols + rows).standard_normal(cols).astype(np.float32)
    x[64:96] = 0.0
    x[100] = 1e-30
    packed, scales = oracle.q4(wf.reshape(rows, cols))
    want, bound = oracle.gemv_q4x(packed, scales, x, rows)
    wd, sd, xd, yd = ctx.upload(packed), ctx.upload(scales), ctx.upload(x), ctx.zeros(rows * 4)
    ctx.gemv_q4x(wd, sd, xd, tb.F32, yd, rows, cols)
    got = yd.download(np.float32, rows)
    assert np.all(np.abs(got.astype(np.float64) - want) <= 1e-5 * bound + 1e-6), np.abs(got - want).max()


@pytest.mark.gpu
def test_embed_decodes_a_row_from_device_or_host_memory(ctx):
    """crates/tachyon/tests/decode.rs:153-177: embed_q4 reads its table from VRAM or from pinned, mapped host memory (the
    per-layer table of host.wpk): the same row, exactly."""
    rows, cols, token = 7, 2560, 5
    packed, scales = oracle.q4(values_fast(rows * cols, 11).reshape(rows, cols))
    g = np.arange(cols)
    byte = packed.reshape(rows, cols // 64, 32)[token][g // 64, g % 64 // 8 * 4 + g % 4]
    nib = ((byte >> (g % 8 // 4 * 4)) & 15).astype(np.float32) - np.float32(8.0)
    want = nib * np.asarray(scales, np.uint16).view(np.float16).astype(np.float32).reshape(rows, cols // 64)[token][g // 64] * np.float32(50.5)
    tok, out = ctx.upload(np.array([token], np.uint32)), ctx.zeros(cols * 4)
    host = ctx.alloc_host(packed.nbytes + scales.nbytes)
    host.array[:packed.nbytes] = packed.view(np.uint8).ravel()
    host.array[packed.nbytes:] = scales.view(np.uint8).ravel()
    dp, ds = ctx.upload(packed), ctx.upload(scales)
    for pw, ps in ((dp.ptr, ds.ptr), (host.ptr, host.ptr + packed.nbytes)):
        out.zero()
        ctx.launch("embed_q4", ((cols + 255) // 256, 1, 1), (256, 1, 1), 0, [("p", pw), ("p", ps), ("p", tok.ptr), ("p", out.ptr), ("u", cols), ("f", 50.5)])
        assert np.array_equal(out.download(np.float32, cols), want)
    host.free()
