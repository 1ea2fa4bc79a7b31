"""Derupel's configuration and spec on the CPU: what config.json gives reaches the parts, and what it cannot describe is
refused with every problem listed."""
import copy

import pytest

from tests import derupel_util as du


def spec_of(cfg):
    from llmgen_b200.registry import config_from_dict
    arch, typed = config_from_dict(cfg)
    return arch.build_spec(typed)


def test_every_size_and_constant_reaches_the_specs():
    spec = spec_of(du.MIXED)
    assert spec.architecture == "Derupel" and spec.embedding_scale == 3.0 and spec.vocab_size == 97 and not spec.tied
    kinds = [(b.kind, b.mixer.kind, None if b.ffn is None else b.ffn.kind) for b in spec.layers]
    assert kinds == [("postnorm", "linear_attention", "dense_mlp"), ("postnorm", "latent_attention", "routed_mlp"),
                     ("postnorm", "latent_attention", None), ("postnorm", "linear_attention", "routed_mlp")]
    lin, lat, lat2, lin2 = (b.mixer for b in spec.layers)
    assert (lin.num_heads, lin.key_dim, lin.value_dim, lin.decay) == (2, 16, 24, (0.9, 1.0)) and lin.out_norm.dim == 48
    assert (lat.num_heads, lat.nope_dim, lat.rope_dim, lat.value_dim, lat.q_rank, lat.kv_rank, lat.scale) == (3, 16, 8, 24, 40, 32, 0.2)
    assert lat.position.pairing == "interleaved" and lat.position.theta == 100.0 and lat.position.rotary_dim == 8
    assert lat2.position.theta == 5000.0 and spec.layers[2].ffn_norm is None
    routed = spec.layers[1].ffn
    assert (len(routed.experts), routed.top_k, routed.experts[0].limit, routed.shared.limit, routed.shared.intermediate_size) == (5, 2, 0.8, 1.2, 32)
    assert routed.weight_on_input and not routed.renormalize and routed.scoring == "sigmoid"
    assert spec.layers[3].ffn.shared is None and spec.layers[3].ffn.top_k == 1
    assert all(b.mixer_norm.eps == 1e-5 for b in spec.layers)


def test_the_declared_tensors_are_the_model_folders_names():
    from llmgen_b200.parts.registry import model_weight_decls
    shapes = {d.name: tuple(d.shape) for d in model_weight_decls(spec_of(du.MIXED))}
    assert shapes["embed"] == (97, 64) and shapes["head"] == (97, 64) and shapes["final.norm"] == (64,)
    assert shapes["l0.mix.q"] == (32, 64) and shapes["l0.mix.v"] == (48, 64) and shapes["l0.mix.norm"] == (48,)
    assert shapes["l1.mix.dq"] == (40, 64) and shapes["l1.mix.uq"] == (72, 40) and shapes["l1.mix.dkv"] == (40, 64)
    assert shapes["l1.mix.dkv.norm"] == (32,) and shapes["l1.mix.uk"] == (48, 32) and shapes["l1.mix.uv"] == (72, 32)
    assert shapes["l1.mlp.router"] == (5, 64) and shapes["l1.mlp.e4.down"] == (64, 24) and shapes["l1.mlp.shared.gate"] == (32, 64)
    assert "l2.norm2" not in shapes and "l3.mlp.shared.up" not in shapes and shapes["l3.mlp.e2.up"] == (16, 64)


def test_a_config_that_cannot_run_lists_its_problems():
    from llmgen_b200.config.base import ConfigError
    bad = copy.deepcopy(du.MIXED)
    bad["layers"][0]["mixer"]["decay"] = [0.5]
    bad["layers"][1]["mlp"]["router"]["top"] = 9
    bad["layers"][2]["type"] = "convolution"
    del bad["norm"]
    with pytest.raises(ConfigError) as e:
        spec_of(bad)
    text = str(e.value)
    assert "decay" in text and "top" in text and "convolution" in text and "norm" in text


def test_the_architecture_is_found_by_the_singular_key():
    from llmgen_b200.config.base import architecture_name
    assert architecture_name({"architecture": "Derupel"}) == "Derupel"
    assert architecture_name({"architectures": ["Qwen3ForCausalLM"], "architecture": "x"}) == "Qwen3ForCausalLM"
