"""Configuration: reading the architecture's own config.json keys, defaults, refusals, registry."""

import json

import pytest

from tiny_configs import TINY_A, TINY_B, TINY_C

from ninfer_amd_mi50_b200.config import ConfigError, EngineOptions
from ninfer_amd_mi50_b200.models.qwen2_moe import Qwen2MoeConfig
from ninfer_amd_mi50_b200.registry import architecture_names, architecture_of, get_architecture


def test_reads_every_key():
    c = Qwen2MoeConfig.from_dict(TINY_B)
    assert (c.num_hidden_layers, c.hidden_size, c.num_attention_heads, c.num_key_value_heads) == (3, 512, 4, 1)
    assert (c.head_dim, c.intermediate_size, c.moe_intermediate_size) == (128, 768, 96)
    assert (c.shared_expert_intermediate_size, c.num_experts, c.num_experts_per_tok) == (384, 16, 4)
    assert c.norm_topk_prob is True and c.mlp_only_layers == [1] and c.tie_word_embeddings is True
    assert c.rope_theta == 1e6 and c.rms_norm_eps == 1e-5 and c.vocab_size == 2003
    assert [c.layer_is_sparse(l) for l in range(3)] == [True, False, True]


def test_defaults_follow_the_reference_parser():
    d = {k: v for k, v in TINY_A.items() if k not in ("num_key_value_heads", "head_dim", "rope_theta",
                                                      "tie_word_embeddings", "norm_topk_prob")}
    c = Qwen2MoeConfig.from_dict(d)
    assert c.num_key_value_heads == c.num_attention_heads       # config.cpp:21-23
    assert c.head_dim == c.hidden_size // c.num_attention_heads  # config.cpp:25-27
    assert c.rope_theta == 1e6 and c.tie_word_embeddings is False and c.norm_topk_prob is False


def test_sparse_step_and_window_rules():
    c = Qwen2MoeConfig.from_dict(TINY_C)
    assert [c.layer_is_sparse(l) for l in range(4)] == [False, True, False, True]
    assert [c.layer_window(l) for l in range(4)] == [None, 40, 40, None]


def test_window_layers_must_be_named_layer_by_layer():
    d = dict(TINY_C)
    del d["layer_types"]
    d["max_window_layers"] = 2
    with pytest.raises(ConfigError, match="layer_types is absent"):
        Qwen2MoeConfig.from_dict(d)                     # never a guessed rule
    d = dict(TINY_C, layer_types=["full_attention"] * 3)
    with pytest.raises(ConfigError, match="3 entries for 4 layers"):
        Qwen2MoeConfig.from_dict(d)
    d = dict(TINY_C, layer_types=["full_attention", "chunked", "full_attention", "full_attention"])
    with pytest.raises(ConfigError, match="chunked"):
        Qwen2MoeConfig.from_dict(d)
    d = dict(TINY_C, use_sliding_window=False)
    with pytest.raises(ConfigError, match="use_sliding_window is not true"):
        Qwen2MoeConfig.from_dict(d)
    # a list of full_attention only, as newer exports of unwindowed models carry, is fine
    d = dict(TINY_A, layer_types=["full_attention"] * 2)
    assert [Qwen2MoeConfig.from_dict(d).layer_window(l) for l in range(2)] == [None, None]


def test_rope_theta_inside_rope_parameters():
    d = dict(TINY_A)
    del d["rope_theta"]
    d["rope_parameters"] = {"rope_type": "default", "rope_theta": 12345.0}
    assert Qwen2MoeConfig.from_dict(d).rope_theta == 12345.0
    d["rope_parameters"] = {"rope_type": "yarn", "rope_theta": 1.0, "factor": 4}
    with pytest.raises(ConfigError, match="rope_type"):
        Qwen2MoeConfig.from_dict(d)


@pytest.mark.parametrize("change,match", [
    ({"vocab_size": None}, "vocab_size"),
    ({"hidden_size": 0}, "hidden_size"),
    ({"num_key_value_heads": 3}, "multiple"),
    ({"head_dim": 33}, "even"),
    ({"num_experts_per_tok": 9}, "num_experts_per_tok"),
    ({"mlp_only_layers": [7]}, "mlp_only_layers"),
    ({"decoder_sparse_step": 0}, "decoder_sparse_step"),
    ({"hidden_act": "gelu"}, "hidden_act"),
    ({"use_sliding_window": True, "sliding_window": None}, "sliding_window"),
    ({"moe_intermediate_size": 0}, "moe_intermediate_size"),
    ({"norm_topk_prob": "yes"}, "norm_topk_prob"),
])
def test_refusals(change, match):
    d = dict(TINY_A)
    for k, v in change.items():
        if v is None:
            d.pop(k, None)
        else:
            d[k] = v
    with pytest.raises(ConfigError, match=match):
        Qwen2MoeConfig.from_dict(d)


def test_round_trip_through_json(tmp_path):
    c = Qwen2MoeConfig.from_dict(TINY_C)
    p = tmp_path / "config.json"
    p.write_text(json.dumps(c.to_dict()))
    assert Qwen2MoeConfig.from_file(str(p)) == c


def test_registry():
    assert "Qwen2MoeForCausalLM" in architecture_names()
    arch = architecture_of(TINY_A)
    plan = arch.build_plan(arch.parse_config(TINY_B))
    assert len(plan.layers) == 3 and [c.layer for c in plan.order] == [0, 1, 2]
    assert [l.feed_forward.kind for l in plan.layers] == ["sparse_moe_swiglu", "dense_swiglu", "sparse_moe_swiglu"]
    with pytest.raises(ConfigError, match="not registered"):
        get_architecture("LlamaForCausalLM")
    with pytest.raises(ConfigError, match="architectures"):
        architecture_of({"hidden_size": 4})


def test_engine_options():
    o = EngineOptions(max_context=0, prefill_chunk=-1, num_sequences=0)
    # the reference's defaults (c_api.cpp:54-82), but for the portion of a prompt: 2,048 instead of 512
    assert (o.max_context, o.prefill_chunk, o.num_sequences) == (32768, 2048, 1)
    assert EngineOptions(dtype="fp32").dtype == "float32"
    with pytest.raises(ValueError):
        EngineOptions(dtype="int4")
    with pytest.raises(ValueError):
        EngineOptions(page_size=24)


def test_shared_keys_agree_with_the_reference_parser():
    """The reference's own config parser, compiled from its sources, read the same three
    configurations (tests/golden/reference_config.json, made by
    tests/golden/make_reference_config_golden.sh)."""
    import os
    from tiny_configs import CONFIGS
    golden = json.load(open(os.path.join(os.path.dirname(__file__), "golden", "reference_config.json")))
    for name, (cfg, _) in CONFIGS.items():
        if name not in golden:
            continue
        ours, ref = Qwen2MoeConfig.from_dict(cfg), golden[name]
        assert ours.architecture == ref["arch"] and ours.model_type == ref["model_type"]
        for key in ("vocab_size", "hidden_size", "num_hidden_layers", "num_attention_heads",
                    "num_key_value_heads", "intermediate_size", "head_dim", "num_experts",
                    "num_experts_per_tok", "moe_intermediate_size", "tie_word_embeddings"):
            assert getattr(ours, key) == ref[key], (name, key)
        assert abs(ours.rms_norm_eps - ref["rms_norm_eps"]) <= 1e-7 * ours.rms_norm_eps * 10
        assert abs(ours.rope_theta - ref["rope_theta"]) <= 1e-6 * ours.rope_theta
        assert ref["is_moe"] is True and ref["ffn_inner"] == ours.moe_intermediate_size
