"""The Nulalorn configuration without a GPU: reading, the plan's order of executions, declared tensors, errors."""

import copy

import pytest
import torch

import plain_nulalorn as plain
from ondeviceinfer_b200.config.nulalorn import NulalornConfig
from ondeviceinfer_b200.config.specs import (CappedAttentionSpec, MLPSpec, NoPositionSpec, ReinjectSpec, RotarySpec,
                                             SandwichBlockSpec, TableExpertsSpec)
from ondeviceinfer_b200.engine.model import DecoderModel
from ondeviceinfer_b200.parts.position import scaled_frequencies
from ondeviceinfer_b200.registry import config_from_dict
from ondeviceinfer_b200.weights.tensors import RandomSource

CONFIGS = [plain.TINY_A, plain.TINY_B, plain.TINY_C, plain.SHARP, plain.PLAIN_STACK, plain.WIDE_HEADS] + [plain.random_config(s) for s in range(8)]


@pytest.mark.parametrize("cfg", CONFIGS)
def test_configuration_reads_back_and_declares_the_designs_tensors(cfg):
    config = config_from_dict(cfg)
    assert isinstance(config, NulalornConfig) and config_from_dict(config.to_dict()) == config
    declared = {d.name: tuple(d.shape) for d in DecoderModel(config.to_plan()).tensor_decls()}
    stored = {name: tuple(shape[:2]) if shape[-1] == "int" else tuple(shape) for name, shape in plain.tensor_shapes(cfg).items()}
    missing_norms = {f"l{i}.{n}" for i, layer in enumerate(cfg["layers"]) if layer["mlp"] is None for n in ("norm2", "norm2b")}
    assert declared == {k: v for k, v in stored.items() if k not in missing_norms}


@pytest.mark.parametrize("cfg", CONFIGS)
def test_order_of_executions_follows_the_loop(cfg):
    plan = config_from_dict(cfg).to_plan()
    runs = plain.layer_runs(cfg)
    order = list(plan.order)
    at = 0
    for layer, opens in runs:
        if opens is not None:
            spec = plan.layers[order[at].layer]
            assert isinstance(spec, ReinjectSpec) and spec.index == opens and spec.num_steps == cfg["loop"]["times"]
            at += 1
        assert order[at].layer == layer and isinstance(plan.layers[layer], SandwichBlockSpec)
        at += 1
    assert at == len(order) and all(entry.cache_from is None for entry in order)


def test_plan_carries_every_constant_of_the_layers():
    plan = config_from_dict(plain.TINY_A).to_plan()
    first, third, last = plan.layers[0], plan.layers[2], plan.layers[3]
    m = first.mixer
    assert isinstance(m, CappedAttentionSpec) and (m.num_heads, m.num_kv_heads, m.head_dim, m.value_dim) == (4, 2, 16, 8)
    assert (m.scale, m.softcap, m.window, m.unit_norm_eps) == (0.4, 9.0, 7, 1e-5)
    assert isinstance(m.position, RotarySpec) and m.position.interleaved and m.position.dim == 8
    assert m.position.scaling == (8.0, 1.0, 4.0, 64.0)
    assert isinstance(first.ffn, MLPSpec) and first.ffn.intermediate_size == 72 and first.ffn.activation == "gelu_erf"
    e = plan.layers[1].ffn
    assert isinstance(e, TableExpertsSpec) and (e.num_experts, e.top_k, e.expert_size, e.shared_size, e.vocab_size) == (5, 2, 24, 40, 61)
    assert third.ffn.shared_size == 0 and third.mixer.position.scaling is None
    assert last.ffn is None and last.ffn_norm is None and last.mixer.softcap is None
    assert plan.head.softcap == 12.0
    bare = config_from_dict(plain.PLAIN_STACK).to_plan()
    assert isinstance(bare.layers[0].mixer.position, NoPositionSpec) and bare.layers[0].mixer.window is None
    assert bare.head.softcap is None and not any(isinstance(spec, ReinjectSpec) for spec in bare.layers)


def test_frequency_scaling_has_three_branches():
    for dims, base, scaling in ((8, 100.0, plain.SCALED), (24, 5000.0, {"factor": 3.0, "low": 2.0, "high": 8.0, "original": 1000})):
        plain_f = [base ** (-2.0 * i / dims) for i in range(dims // 2)]
        want = plain.rotary_frequencies(dims, base, scaling)
        got = scaled_frequencies(plain_f, tuple(scaling[k] for k in ("factor", "low", "high", "original")))
        assert torch.allclose(torch.tensor(got, dtype=torch.float64), want, rtol=1e-12)
        ratio = [g / f for g, f in zip(got, plain_f)]
        assert ratio[0] == 1.0 and abs(ratio[-1] - 1.0 / scaling["factor"]) < 1e-12
        assert any(1.0 / scaling["factor"] + 1e-9 < r < 1.0 - 1e-9 for r in ratio)


def test_random_tables_hold_distinct_experts():
    decls = DecoderModel(config_from_dict(plain.TINY_C).to_plan()).tensor_decls()
    source = RandomSource(decls, 4, device="cpu")
    table = source.fetch("l0.mlp.table")
    assert table.dtype == torch.int32 and tuple(table.shape) == (33, 3) and source.stored()["l0.mlp.table"].dtype == torch.int32
    assert int(table.min()) >= 0 and int(table.max()) < 5
    assert all(len(set(row.tolist())) == 3 for row in table)


@pytest.mark.parametrize("change,error", [
    (lambda c: c["layers"][0].update(type="recurrent"), ValueError),
    (lambda c: c["layers"][0]["mlp"].update(kind="gated"), ValueError),
    (lambda c: c["loop"].update(stop=9), ValueError),
    (lambda c: c["loop"].update(times=0), ValueError),
    (lambda c: c.pop("width"), KeyError),
    (lambda c: c["layers"][1]["mixer"].pop("scale"), KeyError),
])
def test_bad_configurations_are_refused(change, error):
    cfg = copy.deepcopy(plain.TINY_A)
    change(cfg)
    with pytest.raises(error):
        config_from_dict(cfg).to_plan()
