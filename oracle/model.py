"""Test infrastructure (see oracle/__init__.py).  Builds the CPU oracle's copy of a seeded synthetic decoder: the same generator streams tb_decoder_fill_random uses
on the device (documented at the top of tachyon_b200/csrc/decoder.cu)."""
import ctypes as C

import numpy as np

import oracle


def bf16_round(v: float) -> float:
    b = np.array([v], np.float32).view(np.uint32)
    b = (b + 0x7FFF + ((b >> 16) & 1)) & 0xFFFF0000
    return float(b.view(np.float32)[0])


class OracleModel:
    """Weights (numpy, kept alive here), caches and the ctypes structs of oracle.tbo_decoder_step."""

    def __init__(self, cfg, seed: int, context: int, chunk: int = 0, layers: int | None = None, weight_bits: int = 8):
        self.cfg, self.keep = cfg, []
        H, F = cfg.hidden, cfg.ffn
        # Config::head_dim / Config::kv_heads of the two kinds of layer (model/mod.rs:34-37); 0 = as the sliding layers
        dims = (cfg.head_dim, getattr(cfg, "global_head_dim", 0) or cfg.head_dim)
        kvs = (cfg.kv_heads, getattr(cfg, "global_kv_heads", 0) or cfg.kv_heads)
        L = cfg.layers if layers is None else layers
        smul = 0.02 / 8 if weight_bits == 4 else 0.02 / 127
        group = 64 if weight_bits == 4 else 32
        self.tensors = {}

        def mat(name, stream, rows, cols):
            # Four-bit matrices: the same seeded bytes, each holding two weights (tb_decoder_fill_random does the same).
            w = oracle.fill_codes(seed, stream, rows * cols * weight_bits // 8).reshape(rows, cols * weight_bits // 8)
            s = oracle.fill_scales(seed, stream + 1, rows * cols // group, smul).reshape(rows, cols // group)
            self.tensors[name + ".w"], self.tensors[name + ".s"] = w, s
            return w, s

        def vec(name, stream, n, lo, hi):
            v = oracle.fill_uniform(seed, stream, n, lo, hi)
            self.tensors[name] = v
            return v

        self.embed, self.embed_s = mat("embed", 1 << 20, cfg.vocab, H)
        self.norm = vec("norm", (1 << 20) + 2, H, 0.5, 1.5)
        pl = getattr(cfg, "per_layer", 0)
        if pl:  # per-layer inputs: the table, the projection of the embedding, the norm (streams 2^20 + 4 .. 8)
            full = L  # the table holds one input per layer
            self.embed_pl, self.embed_pl_s = mat("embed_per_layer", (1 << 20) + 4, cfg.vocab, pl * full)
            self.pl_model_proj, self.pl_model_proj_s = mat("per_layer_proj", (1 << 20) + 6, pl * full, H)
            self.pl_norm = vec("per_layer_norm", (1 << 20) + 8, pl, 0.5, 1.5)
        self.layers = (oracle.Layer * L)()
        self.caches = []
        for i in range(L):
            b = 32 * i
            ly = self.layers[i]
            is_global = bool(cfg.global_every) and (i + 1) % cfg.global_every == 0
            D, kvh = dims[int(is_global)], kvs[int(is_global)]
            nq, nkv = cfg.heads * D, kvh * D
            # Config::source (model/mod.rs:138-143): the last `shared` layers reuse the cache of the last earlier layer of their kind
            first_shared = L - getattr(cfg, "shared", 0)
            source = i
            if i >= first_shared:
                source = next(j for j in range(first_shared - 1, -1, -1) if (bool(cfg.global_every) and (j + 1) % cfg.global_every == 0) == is_global)
            qkv, qkv_s = mat(f"{i}.qkv", b, nq + (2 * nkv if source == i else 0), H)
            o, o_s = mat(f"{i}.o", b + 2, H, nq)
            gu, gu_s = mat(f"{i}.gate_up", b + 4, 2 * F, H)
            dn, dn_s = mat(f"{i}.down", b + 6, H, F)
            vs = [vec(f"{i}.q_norm", b + 8, D, 0.15, 0.35), vec(f"{i}.k_norm", b + 9, D, 0.15, 0.35),
                  vec(f"{i}.input_layernorm", b + 10, H, 0.5, 1.5), vec(f"{i}.post_attention_layernorm", b + 11, H, 0.5, 1.5),
                  vec(f"{i}.pre_feedforward_layernorm", b + 12, H, 0.5, 1.5), vec(f"{i}.post_feedforward_layernorm", b + 13, H, 0.5, 1.5)]
            scalar = vec(f"{i}.layer_scalar", b + 14, 1, 0.95, 1.0)
            if pl:
                g, g_s = mat(f"{i}.per_layer_gate", b + 16, pl, H)
                pj, pj_s = mat(f"{i}.per_layer_proj", b + 18, H, pl)
                post = vec(f"{i}.post_per_layer_input_norm", b + 20, H, 0.5, 1.5)
                ly.pl_gate, ly.pl_gate_s, ly.pl_proj, ly.pl_proj_s, ly.post_pl_ln = (a.ctypes.data for a in (g, g_s, pj, pj_s, post))
            cap = context if is_global else cfg.window + chunk
            if source == i:
                kc, vc = np.zeros((kvh, cap, D), np.uint16), np.zeros((kvh, cap, D), np.uint16)
            else:
                kc, vc = self.caches[source]
            self.caches.append((kc, vc))
            for name, a in zip(("qkv", "o", "gate_up", "down", "qkv_s", "o_s", "gate_up_s", "down_s"), (qkv, o, gu, dn, qkv_s, o_s, gu_s, dn_s)):
                setattr(ly, name, a.ctypes.data)
            for name, a in zip(("q_norm", "k_norm", "input_ln", "post_attn_ln", "pre_ffn_ln", "post_ffn_ln"), vs):
                setattr(ly, name, a.ctypes.data)
            ly.layer_scalar, ly.global_, ly.kc, ly.vc, ly.cap = float(scalar[0]), int(is_global), kc.ctypes.data, vc.ctypes.data, cap
            ly.shared = int(source != i)
        oc = oracle.Config(hidden=H, ffn=F, heads=cfg.heads, kv_heads=cfg.kv_heads, head_dim=cfg.head_dim, vocab=cfg.vocab, layers=L, window=cfg.window,
                           context=context, theta_sliding=cfg.theta_sliding, theta_global=cfg.theta_global, fraction_global=cfg.fraction_global,
                           eps=cfg.eps, softcap=cfg.softcap, attn_scale=cfg.attn_scale, embed_scale=bf16_round(float(np.sqrt(np.float32(H)))),
                           weight_bits=weight_bits, global_head_dim=dims[1], global_kv_heads=kvs[1], per_layer=pl)
        self.model = oracle.Model(cfg=oc, embed=self.embed.ctypes.data, embed_s=self.embed_s.ctypes.data, norm=self.norm.ctypes.data,
                                  layers=C.cast(self.layers, C.POINTER(oracle.Layer)))
        if pl:
            self.model.embed_pl, self.model.embed_pl_s = self.embed_pl.ctypes.data, self.embed_pl_s.ctypes.data
            self.model.pl_model_proj, self.model.pl_model_proj_s = self.pl_model_proj.ctypes.data, self.pl_model_proj_s.ctypes.data
            self.model.pl_norm = self.pl_norm.ctypes.data

    def fill_cache(self, seed: int):
        """The same seeded N(0,1) cache contents tb_decoder_fill_cache writes."""
        for i, (kc, vc) in enumerate(self.caches):
            if self.layers[i].shared:
                continue  # the source layer's arrays
            kc[...] = oracle.fill_gauss_f16(seed, (1 << 21) + 2 * i, kc.size, 1.0).reshape(kc.shape)
            vc[...] = oracle.fill_gauss_f16(seed, (1 << 21) + 2 * i + 1, vc.size, 1.0).reshape(vc.shape)

    def step(self, token: int, pos: int, want_logits: bool = True, stop_layer: int = 0):
        logits = np.zeros(self.cfg.vocab, np.float32) if want_logits and stop_layer == 0 else None
        hidden = np.zeros(self.cfg.hidden, np.float32)
        t = oracle.lib().tbo_decoder_step(C.byref(self.model), token, pos, None if logits is None else logits.ctypes.data, stop_layer, hidden.ctypes.data)
        return t, logits, hidden
