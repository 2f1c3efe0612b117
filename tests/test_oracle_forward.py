"""A second, independent statement of the decoder's forward pass, in numpy f64, against the C oracle's (oracle/tachyon_oracle.c
tbo_decoder_step).  Both follow the reference's CPU test model (crates/tachyon/tests/common/tiny.rs:225-299: "Gemma 4's
forward pass ... as Hugging Face computes it"), written separately: this one from whole-matrix products and the layer
formulas, the C one as the loops every GPU parity test leans on.  It pins nothing to the reference itself (nothing in this
environment can run the reference); it catches a slip in either transcription.  No GPU involved."""
import numpy as np
import pytest

import oracle
import tachyon_b200 as tb
from oracle.model import OracleModel, bf16_round


def f16_round(a):
    return np.asarray(a, np.float64).astype(np.float16).astype(np.float64)


def dequant(model, name, bits=8):
    w, s = model.tensors[name + ".w"], model.tensors[name + ".s"]
    if bits == 8:
        return w.astype(np.float64) * np.repeat(s.view(np.float16).astype(np.float64), 32, axis=1)
    # crates/tachyon/src/quant.rs:47-82: weight k of a group of 64 is nibble k % 8 / 4 of byte k / 8 * 4 + k % 4, minus 8, times the
    # group's f16 scale
    rows = w.shape[0]
    pk = w.view(np.uint8).reshape(rows, -1, 32)
    k = np.arange(64)
    nib = (pk[:, :, k // 8 * 4 + k % 4] >> (k % 8 // 4 * 4)) & 15
    return ((nib.astype(np.float64) - 8.0) * s.view(np.float16).astype(np.float64)[:, :, None]).reshape(rows, -1)


def rms(x, w=None, eps=1e-6):
    y = x / np.sqrt((x * x).mean() + eps)  # tiny.rs:376-379
    return y if w is None else y * w


def rotate(x, pos, freq):
    """tiny.rs:382-391: rotate_half pairs (j, j + d/2); the angle is an f32 product, as the test model has it."""
    half = x.size // 2
    ang = (np.float32(pos) * freq.astype(np.float32)).astype(np.float64)
    c, s = np.cos(ang), np.sin(ang)
    a, b = x[:half], x[half:]
    return np.concatenate([a * c - b * s, b * c + a * s])


def gelu(x):
    return 0.5 * x * (1.0 + np.tanh(np.sqrt(2.0 / np.pi) * (x + 0.044715 * x ** 3)))  # tiny.rs:393-395


class Forward:
    """The forward pass over an OracleModel's tensors; caches hold f16-rounded keys and values, as the decoder keeps them."""

    def __init__(self, cfg, model: OracleModel, bits=8):
        self.cfg, self.m, self.bits = cfg, model, bits
        self.L = cfg.layers
        self.mats = {}
        self.cache = [dict() for _ in range(self.L)]  # position -> (k [kvh, D], v [kvh, D])
        self.glob = [bool(cfg.global_every) and (i + 1) % cfg.global_every == 0 for i in range(self.L)]

    def mat(self, name):
        if name not in self.mats:
            self.mats[name] = dequant(self.m, name, self.bits)
        return self.mats[name]

    def source(self, i):
        first_shared = self.L - self.cfg.shared
        if i < first_shared:
            return i
        return next(j for j in range(first_shared - 1, -1, -1) if self.glob[j] == self.glob[i])  # model/mod.rs:138-143

    def step(self, token, pos, context):
        c, t = self.cfg, self.m.tensors
        H = c.hidden
        x = self.mat("embed")[token] * bf16_round(float(np.sqrt(np.float32(H))))  # tiny.rs:233; decode.rs:571 rounds the factor to bf16
        pl = c.per_layer
        if pl:  # tiny.rs:239-252
            ple = self.mat("embed_per_layer")[token] * np.sqrt(pl)
            proj = self.mat("per_layer_proj") @ x / np.sqrt(H)
            pli = np.concatenate([(rms(proj[l * pl:(l + 1) * pl], t["per_layer_norm"].astype(np.float64), c.eps) + ple[l * pl:(l + 1) * pl]) / np.sqrt(2.0)
                                  for l in range(self.L)])
        for i in range(self.L):
            g = self.glob[i]
            D = (c.global_head_dim or c.head_dim) if g else c.head_dim
            kvh = (c.global_kv_heads or c.kv_heads) if g else c.kv_heads
            nq, nkv = c.heads * D, kvh * D
            freq = oracle.rope_freq(c.theta_global if g else c.theta_sliding, D, c.fraction_global if g else 1.0)
            w = lambda n: t[f"{i}.{n}"].astype(np.float64)
            h = rms(x, w("input_layernorm"), c.eps)
            qkv = self.mat(f"{i}.qkv") @ h
            q = np.stack([rotate(rms(qkv[k * D:(k + 1) * D], w("q_norm"), c.eps), pos, freq) for k in range(c.heads)])
            src = self.source(i)
            if src == i:
                k = np.stack([rotate(rms(qkv[nq + j * D: nq + (j + 1) * D], w("k_norm"), c.eps), pos, freq) for j in range(kvh)])
                v = np.stack([rms(qkv[nq + nkv + j * D: nq + nkv + (j + 1) * D], None, c.eps) for j in range(kvh)])
                self.cache[i][pos] = (f16_round(k), f16_round(v))
            window = context if g else c.window
            first = max(0, pos + 1 - window)
            ks = np.stack([self.cache[src][p][0] for p in range(first, pos + 1)])  # [n, kvh, D]
            vs = np.stack([self.cache[src][p][1] for p in range(first, pos + 1)])
            group = c.heads // kvh
            out = np.zeros((c.heads, D))
            for hq in range(c.heads):
                sc = ks[:, hq // group] @ q[hq] * c.attn_scale
                e = np.exp(sc - sc.max())
                out[hq] = (e / e.sum()) @ vs[:, hq // group]
            x = x + rms(self.mat(f"{i}.o") @ out.ravel(), w("post_attention_layernorm"), c.eps)
            hh = rms(x, w("pre_feedforward_layernorm"), c.eps)
            gu = self.mat(f"{i}.gate_up") @ hh  # gate rows, then up rows
            a = gelu(gu[:c.ffn]) * gu[c.ffn:]
            x = x + rms(self.mat(f"{i}.down") @ a, w("post_feedforward_layernorm"), c.eps)
            if pl:  # tiny.rs:298-300
                a2 = gelu(self.mat(f"{i}.per_layer_gate") @ x) * pli[i * pl:(i + 1) * pl]
                x = x + rms(self.mat(f"{i}.per_layer_proj") @ a2, w("post_per_layer_input_norm"), c.eps)
            x = x * float(t[f"{i}.layer_scalar"][0])
        return self.mat("embed") @ rms(x, t["norm"].astype(np.float64), c.eps), x


def config(**kw):
    c = tb.gemma4_e4b_shape(layers=kw.pop("layers", 3), ffn=kw.pop("ffn", 2048), vocab=kw.pop("vocab", 1024))
    c.window, c.global_every = 8, 3
    for k, v in kw.items():
        setattr(c, k, v)
    return c


@pytest.mark.parametrize("kw", [dict(), dict(layers=6, shared=3), dict(layers=6, global_head_dim=512, global_kv_heads=1, shared=2),
                                dict(layers=5, per_layer=256, global_head_dim=512, shared=1), dict(layers=3, kv_heads=1),
                                dict(layers=5, per_layer=256, global_head_dim=512, shared=1, bits=4)],
                         ids=["plain", "shared caches", "heads of 512", "per-layer inputs", "eight query heads to a key-value head",
                              "per-layer inputs in four bits"])
def test_the_c_oracle_and_the_numpy_forward_agree(kw):
    kw = dict(kw)
    bits = kw.pop("bits", 8)
    cfg = config(**kw)
    context = 32
    model = OracleModel(cfg, 4321, context=context, chunk=4, weight_bits=bits)
    fwd = Forward(cfg, model, bits)
    token = 7
    for pos in range(14):  # past the window of 8 and the ring of 12
        pick, logits, hidden = model.step(token, pos)
        want, want_hidden = fwd.step(token, pos, context)
        assert np.abs(hidden - want_hidden).max() <= 2e-4 * np.abs(want_hidden).max(), pos  # f32 loops against f64 products
        assert np.abs(logits - want).max() <= 2e-4 * np.abs(want).max(), pos
        capped = cfg.softcap * np.tanh(want / cfg.softcap)
        top = np.sort(capped)
        if top[-1] - top[-2] > 1e-3 * np.abs(want).max():
            assert pick == int(np.argmax(capped))
        token = (pos * 7919 + 13) % cfg.vocab
