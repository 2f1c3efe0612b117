"""The CPU oracle against the reference's own known-answer tests (crates/tachyon/src/quant.rs:249-277) and against the
committed golden vectors under tests/golden/."""
import json
import os

import numpy as np

import oracle
from util import values

GOLDEN = os.path.join(os.path.dirname(__file__), "golden")


def test_f16_round_trips_every_value_and_rounds_to_even():
    # quant.rs:252-262
    lib = oracle.lib()
    for h in range(0x10000):
        if (h & 0x7C00) != 0x7C00 or (h & 0x3FF) == 0:
            assert lib.tbo_f16_bits(lib.tbo_f16_value(h)) == h, hex(h)
    cases = [(1.0, 0x3C00), (65504.0, 0x7BFF), (65520.0, 0x7C00), (2.0**-24, 1), (2.0**-25, 0), (0.1, 0x2E66), (-2.0, 0xC000)]
    for v, h in cases:
        assert oracle.f16_bits(v) == h, v
    assert oracle.f16_bits(1.0 + 2.0**-11) == 0x3C00  # a tie rounds to the even neighbour


def test_f16_matches_numpy_on_every_pattern():
    bits = np.arange(0x10000, dtype=np.uint16)
    finite = (bits & 0x7C00) != 0x7C00
    mine = np.array([oracle.f16_value(int(h)) for h in bits[finite]], np.float32)
    assert np.array_equal(mine, bits[finite].view(np.float16).astype(np.float32))


def test_q4_packs_weights_where_the_kernel_reads_them():
    # quant.rs:264-270
    w = np.array([(j % 15) - 7.0 for j in range(64)], np.float32)
    packed, scales = oracle.q4(w)
    assert oracle.f16_value(int(scales[0])) == 1.0
    nib = lambda j: (int(packed[j // 8 * 4 + j % 4]) >> (j % 8 // 4 * 4)) & 15
    assert all(nib(j) - 8.0 == w[j] for j in range(64))
    assert packed[0] == 0x51  # weights 0 and 4 share byte 0


def test_q8_keeps_block_sums():
    # quant.rs:272-277
    x = np.arange(64, dtype=np.float32) - 20.0
    q, pairs = oracle.q8(x)
    assert (q[0], q[20], q[63]) == (-127, 0, 127)
    scale = np.float32(20.0) / np.float32(127.0)
    assert pairs[0][0] == scale and pairs[0][1] == np.float32(int(q[:32].sum())) * scale


def test_q8p_pairs_follow_the_magic_offset():
    # quant.rs:102-105: z = fma(s, -MAGIC, -8 * s * sum)
    x = values(128, 3)
    q, pairs = oracle.q8(x, 64)
    _, pp = oracle.q8p(x)
    for b in range(2):
        s, ssum = pairs[b]
        want = np.float32(np.float64(s) * -12582912.0 + np.float64(np.float32(ssum * np.float32(-8.0))))
        assert pp[b][0] == s and abs(pp[b][1] - want) <= abs(want) * 2**-23


def test_golden_vectors_still_hold():
    """tests/golden/oracle_vectors.json was written by tests/golden/make_golden.py; the oracle must reproduce it."""
    with open(os.path.join(GOLDEN, "oracle_vectors.json")) as f:
        g = json.load(f)
    assert [int(v) for v in oracle.fill_codes(7, 3, 16)] == g["fill_codes_7_3"]
    assert [int(v) for v in oracle.fill_scales(7, 4, 8, 0.02 / 127)] == g["fill_scales_7_4"]
    x = values(64, 11)
    assert [float(v) for v in x[:4]] == g["values_11"][:4]
    w = oracle.fill_codes(5, 0, 4 * 64).reshape(4, 64)
    s = oracle.fill_scales(5, 1, 4 * 2, 0.02 / 127).reshape(4, 2)
    y, exact, _ = oracle.gemv_q8(w, s, x)
    assert np.allclose(exact, g["gemv_exact"], rtol=1e-12)
    assert [float(v) for v in y] == g["gemv_f32"]
    packed, scales = oracle.q4(values(128, 5))
    assert [int(v) for v in packed[:8]] == g["q4_packed"] and [int(v) for v in scales] == g["q4_scales"]
    t, gap = oracle.sample_greedy(values(4000, 9) * 40.0, softcap=30.0)
    assert t == g["greedy_token"]


def test_gemv_oracle_matches_plain_numpy():
    rng = np.random.default_rng(0)
    w = rng.integers(-127, 128, size=(9, 96), dtype=np.int8)
    s = (np.abs(rng.standard_normal((9, 3))) * 0.02 / 127).astype(np.float16)
    x = rng.standard_normal(96).astype(np.float32)
    _, exact, bound = oracle.gemv_q8(w, s.view(np.uint16), x)
    deq = w.astype(np.float64) * np.repeat(s.astype(np.float64), 32, axis=1)
    assert np.allclose(exact, deq @ x.astype(np.float64), rtol=1e-12, atol=1e-15)
    assert np.all(bound >= np.abs(exact) - 1e-12)


def test_attention_oracle_matches_plain_numpy_in_plain_mode():
    rng = np.random.default_rng(1)
    heads, kv, d, cap, pos, win = 4, 2, 256, 64, 40, 16
    qkv = rng.standard_normal((heads + 2 * kv) * d).astype(np.float32)
    kc = rng.standard_normal((kv, cap, d)).astype(np.float16)
    vc = rng.standard_normal((kv, cap, d)).astype(np.float16)
    kb, vb = kc.view(np.uint16).copy(), vc.view(np.uint16).copy()
    out = oracle.attend_decode(qkv, None, None, None, kb, vb, pos, cap, win, True, heads, kv, d, 1 / 16.0)
    # plain numpy: newest 16 positions, new k/v taken unrounded
    for h in range(heads):
        g = h // 2
        ks = [kc[g, (pos - a) % cap].astype(np.float64) if a else qkv[(heads + g) * d:][:d].astype(np.float64) for a in range(win)]
        vs = [vc[g, (pos - a) % cap].astype(np.float64) if a else qkv[(heads + kv + g) * d:][:d].astype(np.float64) for a in range(win)]
        q = qkv[h * d:][:d].astype(np.float64)
        sc = np.array([q @ k for k in ks]) / 16.0
        p = np.exp(sc - sc.max())
        want = (p[:, None] * np.array(vs)).sum(0) / p.sum()
        assert np.allclose(out[h * d:][:d], want, rtol=1e-10, atol=1e-12)
    # the new key/value landed in slot pos % cap, rounded to f16
    assert np.array_equal(kb.reshape(kv, cap, d)[0, pos % cap], qkv[heads * d:][:d].astype(np.float16).view(np.uint16))


def test_q8e_is_q8_in_blocks_of_64_with_the_scale_alone():
    # quant.rs:107-115 over the vector of quant.rs:272-277: the largest magnitude of a block over 127, ties to even
    x = np.concatenate([np.arange(64, dtype=np.float32) - 20.0, np.zeros(64, np.float32), np.full(64, 0.5, np.float32)])
    q, s = oracle.q8e(x)
    assert s.shape == (3,) and s[0] == np.float32(43.0) / np.float32(127.0) and s[1] == 0.0 and s[2] == np.float32(0.5) / np.float32(127.0)
    inv = np.float32(127.0) / np.float32(43.0)
    assert np.array_equal(q[:64], np.rint(x[:64] * inv).astype(np.int8)) and not q[64:128].any() and np.all(q[128:] == 127)


def test_the_q8e_product_is_the_sum_of_scaled_integer_sums():
    # crates/tachyon/tests/encoder.rs:329-331: the product of the dequantised values, within the test's bound
    rows, cols, tokens = 64, 192, 5
    (aq, sa), (wq, sw) = oracle.q8e(values(tokens * cols, 8)), oracle.q8e(values(rows * cols, 9))
    bias = values(rows, 10)
    got = oracle.gemm_q8e(aq, sa, wq, sw, rows, bias)
    a = aq.astype(np.float64).reshape(tokens, cols // 64, 64) * sa.astype(np.float64).reshape(tokens, cols // 64, 1)
    w = wq.astype(np.float64).reshape(rows, cols // 64, 64) * sw.astype(np.float64).reshape(rows, cols // 64, 1)
    want = a.reshape(tokens, cols) @ w.reshape(rows, cols).T + bias
    # -12582912 s is rounded before the fused multiply-add takes it (ptx/encoder.rs:362): each group carries up to half a unit
    # in the last place of 12582912 s, times the row's scale; the reference's own bound is 1e-3 + 2e-3 |want|
    assert np.abs(got - want).max() < 3e-4
    assert np.array_equal(oracle.gemm_q8e(aq, sa, wq, sw, rows), oracle.gemm_q8e(aq, sa, wq, sw, rows, np.zeros(rows, np.float32)))


def test_rope_table_holds_cos_and_sin_of_each_position():
    # encoder/run.rs:523-537
    t = oracle.rope_table(10000.0, 5, 8)
    assert t.shape == (5, 4, 2) and np.all(t[0, :, 0] == 1.0) and np.all(t[0, :, 1] == 0.0)
    assert t[3, 2, 0] == np.float32(np.cos(3 * 10000.0 ** -0.5)) and t[3, 2, 1] == np.float32(np.sin(3 * 10000.0 ** -0.5))
