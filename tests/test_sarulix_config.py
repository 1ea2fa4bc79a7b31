"""Sarulix on the CPU: its typed configuration, the run list of a looped model, the tensors it declares, and the plain
implementation's own consistency (the scans against closed forms)."""
import copy

import pytest
import torch

from llmgen_b200.config.base import ConfigError
from llmgen_b200.parts.registry import model_weight_decls
from llmgen_b200.registry import config_from_dict
from tests import sarulix_util as su
from tests.plain import sarulix_plain as plain


def spec_of(cfg):
    arch, typed = config_from_dict(cfg)
    return arch.build_spec(typed)


def test_the_registry_finds_the_architecture_and_the_parts_it_is_made_of():
    spec = spec_of(su.MIXED)
    assert spec.architecture == "Sarulix" and spec.logit_scale == 0.7 and spec.embedding_scale == 3.0
    kinds = [layer.mixer.kind for layer in spec.layers]
    assert kinds == ["rglru", "gated_delta", "attention", "rglru"]
    assert [layer.ffn is not None for layer in spec.layers] == [False, False, True, True]
    att = spec.layers[2].mixer
    assert att.sink and att.softcap == 15.0 and att.v_head_dim == 24 and att.position.rotary_dim == 8 and att.position.pairing == "half"
    assert spec.layers[0].mixer_norm.weight_offset == 1.0 and spec.final_norm.weight_offset == 1.0
    assert spec.layers[1].mixer.decay_rank == 8 and spec.layers[1].mixer.gate_rank == 12


def test_a_loop_repeats_its_layers_with_caches_of_their_own_and_a_reentry_before_every_pass():
    spec = spec_of(su.MIXED)        # loop [1, 3) twice
    assert [item.layer for item in spec.run_order] == [0, 1, 2, 1, 2, 3]
    assert [item.cache for item in spec.run_order] == list(range(6))
    rows = [item.before.row if item.before is not None else None for item in spec.run_order]
    assert rows == [None, 0, None, 1, None, None]
    assert [plain_item[1] for plain_item in plain.run_list(su.MIXED)] == rows
    no_loop = spec_of(su.ODD)
    assert [item.layer for item in no_loop.run_order] == [0, 1, 2, 3] and all(item.before is None for item in no_loop.run_order)
    names = {d.name for d in model_weight_decls(no_loop)}
    assert "loop.in" not in names and "loop.step" not in names
    looped = {d.name: d.shape for d in model_weight_decls(spec)}
    assert looped["loop.in"] == (64, 128) and looped["loop.step"] == (2, 64)


def test_declared_tensors_have_the_design_s_names_and_shapes():
    shapes = {d.name: tuple(d.shape) for d in model_weight_decls(spec_of(su.MIXED))}
    assert shapes["l0.mix.ra"] == (3, 16, 16) and shapes["l0.mix.conv"] == (48, 4) and shapes["l0.mix.y"] == (48, 64)
    assert shapes["l1.mix.q.conv"] == (32, 3) and shapes["l1.mix.v.conv"] == (96, 3) and shapes["l1.mix.a2"] == (64, 8)
    assert shapes["l1.mix.b"] == (4, 64) and shapes["l1.mix.A_log"] == (4,) and shapes["l1.mix.norm"] == (24,)
    assert shapes["l2.mix.q"] == (64, 64) and shapes["l2.mix.v"] == (48, 64) and shapes["l2.mix.g"] == (96, 64)
    assert shapes["l2.mix.o"] == (64, 96) and shapes["l2.mix.o.b"] == (64,) and shapes["l2.mix.k.norm"] == (16,)
    assert "l0.norm2" not in shapes and shapes["l2.norm2"] == (64,) and shapes["l2.mlp.gate"] == (80, 64)


def test_low_ranks_come_from_the_folder_s_tensor_shapes_when_the_file_does_not_name_them():
    from llmgen_b200.config.sarulix import SarulixConfig
    cfg = copy.deepcopy(su.MIXED)
    for key in ("decay_rank", "gate_rank"):
        del cfg["layers"][1]["mixer"][key]
    filled = SarulixConfig.fill_from_tensor_shapes(cfg, {"l1.mix.a1": (5, 64), "l1.mix.g1": (7, 64)})
    m = spec_of(filled).layers[1].mixer
    assert (m.decay_rank, m.gate_rank) == (5, 7)
    assert "decay_rank" not in cfg["layers"][1]["mixer"]          # the caller's dict is left alone


def test_every_problem_of_a_configuration_is_listed_at_once():
    bad = copy.deepcopy(su.MIXED)
    del bad["norm"]
    bad["layers"][2]["mixer"]["kv_heads"] = 3
    bad["layers"][0]["mixer"]["blocks"] = 5
    bad["loop"]["stop"] = 9
    with pytest.raises(ConfigError) as e:
        config_from_dict(bad)
    text = str(e.value)
    assert "norm" in text and "kv_heads" in text and "blocks" in text and "loop" in text


def test_the_plain_scans_agree_with_their_closed_forms():
    torch.manual_seed(0)
    T, C = 9, 5
    u, r, i, lam = torch.randn(T, C, dtype=torch.float64), torch.rand(T, C, dtype=torch.float64), torch.rand(T, C, dtype=torch.float64), torch.randn(C, dtype=torch.float64)
    S = plain.rglru_scan(u, r, i, lam)
    a = torch.exp(-8.0 * r * torch.log1p(torch.exp(lam)))
    b = torch.sqrt(1 - a * a) * i * u
    want = sum(b[j] * a[j + 1:].prod(dim=0) for j in range(T))
    assert torch.allclose(S[-1], want, atol=1e-12)
    # the delta rule with beta = 1 and no decay stores v under a unit key exactly
    k = torch.nn.functional.normalize(torch.randn(1, 1, 6, dtype=torch.float64), dim=-1)
    v = torch.randn(1, 1, 4, dtype=torch.float64)
    o = plain.gated_delta_scan(k, k, v, torch.ones(1, 1, dtype=torch.float64), torch.ones(1, 1, 6, dtype=torch.float64))
    assert torch.allclose(o, v, atol=1e-12)
    # the sink: one key of score s has the weight e^s / (1 + e^s)
    q = torch.tensor([[[2.0, 0.0]]], dtype=torch.float64)
    out = plain.sink_softmax_attention(q, q, torch.ones(1, 1, 1, dtype=torch.float64), 1.0, 0.0)
    assert torch.allclose(out, torch.sigmoid(torch.tensor(4.0, dtype=torch.float64)).reshape(1, 1, 1))
