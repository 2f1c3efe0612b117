"""Writes tests/golden/tiny_encoder.npz from the reference's tiny-encoder fixture
(crates/tachyon/tests/fixtures/tiny-encoder: a random 3-layer ModernBERT and PyTorch's hidden states for three
sequences, made by the reference's scripts/encoders.py).  The npz holds the encoder's tensors under this build's
names (float16, as the fixture stores them), its config and the cases' ids and hidden states, so that the oracle's encoder forward
stays pinned where the reference tree is absent.

Run from the repository root with the reference's tree at hand: python tests/golden/make_encoder_golden.py <reference root>
"""
import json
import os
import struct
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
if len(sys.argv) != 2:
    sys.exit(__doc__)
REF = sys.argv[1]
DIR = os.path.join(REF, "crates/tachyon/tests/fixtures/tiny-encoder")

raw = open(os.path.join(DIR, "model.safetensors"), "rb").read()
(hlen,) = struct.unpack("<Q", raw[:8])
head = json.loads(raw[8:8 + hlen])
data = raw[8 + hlen:]


def tensor(name):
    t = head["encoder." + name]
    a, b = t["data_offsets"]
    assert t["dtype"] == "F16", t["dtype"]  # the fixture is stored in half precision
    return np.frombuffer(data[a:b], np.float16).reshape(t["shape"]).copy()


cfg = json.load(open(os.path.join(DIR, "config.json")))
layers = cfg["num_hidden_layers"]
out = {"embed": tensor("embeddings.tok_embeddings.weight"), "embed_norm": tensor("embeddings.norm.weight"), "final_norm": tensor("final_norm.weight")}
for l in range(layers):
    p = f"layers.{l}."
    if l > 0:
        out[f"{l}.attn_norm"] = tensor(p + "attn_norm.weight")
    for ours, theirs in (("qkv", "attn.Wqkv"), ("o", "attn.Wo"), ("mlp_norm", "mlp_norm"), ("up", "mlp.Wi"), ("down", "mlp.Wo")):
        out[f"{l}.{ours}"] = tensor(p + theirs + ".weight")
config = {"hidden": cfg["hidden_size"], "heads": cfg["num_attention_heads"], "inter": cfg["intermediate_size"], "vocab": cfg["vocab_size"],
          "window": cfg["local_attention"] // 2, "gated": 1, "theta_global": cfg["rope_parameters"]["full_attention"]["rope_theta"],
          "theta_local": cfg["rope_parameters"]["sliding_attention"]["rope_theta"], "eps": cfg["norm_eps"],
          "global": [t == "full_attention" for t in cfg["layer_types"]]}
cases = [json.loads(line) for line in open(os.path.join(DIR, "outputs.ref")) if line.strip()]
out["config_json"] = np.frombuffer(json.dumps(config).encode(), np.uint8)
for i, c in enumerate(cases):
    out[f"case{i}.ids"] = np.array(c["ids"], np.uint32)
    out[f"case{i}.hidden"] = np.array(c["hidden"], np.float32)
out["cases"] = np.array([len(cases)], np.int32)
np.savez_compressed(os.path.join(HERE, "tiny_encoder.npz"), **out)
print("wrote tiny_encoder.npz:", len(cases), "cases,", {k: v.shape for k, v in list(out.items())[:4]})
