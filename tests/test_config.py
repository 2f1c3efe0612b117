"""config.json as the reference reads it: model::Config::from_json (crates/tachyon/src/model/mod.rs:63-105, 154-161) and
encoder::Config::from_json (crates/tachyon/src/encoder/mod.rs:61-117).  Host logic, no GPU."""
import json

import pytest

import tachyon_b200 as tb

TEXT = {"hidden_size": 2560, "intermediate_size": 10240, "num_attention_heads": 8, "num_key_value_heads": 2, "head_dim": 256, "global_head_dim": 512,
        "hidden_size_per_layer_input": 256, "vocab_size": 262144, "sliding_window": 512, "rms_norm_eps": 1e-6, "num_kv_shared_layers": 18, "final_logit_softcapping": 30.0,
        "num_global_key_value_heads": 2, "layer_types": (["sliding_attention"] * 5 + ["full_attention"]) * 7,
        "rope_parameters": {"full_attention": {"rope_theta": 1e6, "partial_rotary_factor": 0.25}, "sliding_attention": {"rope_theta": 1e4}}}


def test_a_multimodal_config_gives_the_decoders_shape():
    for doc in ({"model_type": "gemma4", "text_config": TEXT}, TEXT):
        c = tb.config_from_json(json.dumps(doc).encode())
        assert (c.hidden, c.ffn, c.heads, c.kv_heads, c.head_dim, c.global_head_dim, c.per_layer, c.vocab, c.window) == (2560, 10240, 8, 2, 256, 512, 256, 262144, 512)
        assert (c.layers, c.shared, c.global_kv_heads) == (42, 18, 2) and c.softcap == 30.0 and c.fraction_global == 0.25
        assert c.theta_sliding == 1e4 and c.theta_global == 1e6 and abs(c.eps - 1e-6) < 1e-12
        assert list(c._global) == [0, 0, 0, 0, 0, 1] * 7 and c.global_ == c._global.ctypes.data
    bare = {k: v for k, v in TEXT.items() if k not in ("rope_parameters", "final_logit_softcapping", "num_kv_shared_layers", "num_global_key_value_heads")}
    c = tb.config_from_json(json.dumps(bare).encode())
    assert (c.theta_sliding, c.theta_global, c.fraction_global, c.softcap, c.shared, c.global_kv_heads) == (1e4, 1e6, 1.0, 0.0, 0, 2)


def test_what_the_decoder_does_not_run_is_refused():
    for change, status in (({"num_key_value_heads": 8}, 9), ({"num_key_value_heads": 3}, 9), ({"use_double_wide_mlp": True}, 9), ({"num_experts": 8}, 9)):
        with pytest.raises(tb.Error) as e:
            tb.config_from_json(json.dumps({**TEXT, **change}).encode())
        assert e.value.status == status
    missing = {k: v for k, v in TEXT.items() if k != "head_dim"}
    with pytest.raises(tb.Error) as e:
        tb.config_from_json(json.dumps(missing).encode())
    assert e.value.status == 5 and "no head_dim" in str(e.value)


def test_a_modernbert_config_gives_the_encoders_shape():
    doc = {"model_type": "modernbert", "hidden_activation": "gelu", "hidden_size": 768, "num_attention_heads": 12, "intermediate_size": 1152, "vocab_size": 50368,
           "num_hidden_layers": 22, "local_attention": 128, "global_rope_theta": 160000.0, "local_rope_theta": 10000.0, "norm_eps": 1e-5}
    e = tb.encoder_config_from_json(json.dumps(doc).encode())
    assert (e.hidden, e.heads, e.inter, e.vocab, e.layers, e.window, e.gated, e.dims, e.mean_pool) == (768, 12, 1152, 50368, 22, 64, 1, 768, 0)
    assert list(e._global) == [int(i % 3 == 0) for i in range(22)] and e.theta_global == 160000.0 and e.theta_local == 10000.0
    typed = {**doc, "hidden_activation": "silu", "layer_types": ["full_attention", "sliding_attention"] * 11,
             "rope_parameters": {"full_attention": {"rope_theta": 5e5}, "sliding_attention": {"rope_theta": 2e4}}}
    e = tb.encoder_config_from_json(json.dumps(typed).encode(), mean_pool=True, dims=256)
    assert e.gated == 2 and list(e._global) == [1, 0] * 11 and (e.theta_global, e.theta_local, e.dims, e.mean_pool) == (5e5, 2e4, 256, 1)
    for change in ({"model_type": "bert"}, {"hidden_activation": "relu"}, {"attention_bias": True}):
        with pytest.raises(tb.Error) as err:
            tb.encoder_config_from_json(json.dumps({**doc, **change}).encode())
        assert err.value.status == 9
    with pytest.raises(tb.Error) as err:
        tb.encoder_config_from_json(json.dumps({**doc, "num_attention_heads": 7}).encode())
    assert err.value.status == 5
