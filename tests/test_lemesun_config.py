"""The Lemesun configuration, its plan and the cache groups it asks for (no GPU needed)."""

import copy

import pytest
import torch

import plain_lemesun as plain
from ondeviceinfer_b200 import KVNeed, LemesunConfig, SequenceCache, StateNeed
from ondeviceinfer_b200.config import ChannelDeltaSpec, LatentAttentionSpec, RoutedExpertsSpec
from ondeviceinfer_b200.engine.model import DecoderModel
from ondeviceinfer_b200.registry import architecture_name, config_from_dict
from ondeviceinfer_b200.weights import loader
from ondeviceinfer_b200.weights.tensors import StoredTensor


def stored_of(cfg, seed=0):
    return {name: StoredTensor(tuple(t.shape), t.dtype) for name, t in plain.random_weights(cfg, seed).items()}


def test_the_registry_reads_the_single_architecture_key():
    assert architecture_name(plain.TINY_A) == "Lemesun"
    assert isinstance(config_from_dict(plain.TINY_A), LemesunConfig)


def test_round_trip_and_plan_of_the_layer_list():
    config = LemesunConfig.from_dict(plain.TINY_A)
    assert LemesunConfig.from_dict(config.to_dict()) == config
    plan = config.plan_for(stored_of(plain.TINY_A))
    # five runs over three layers with tensors of their own; runs 2 and 4 use the tensors of runs 0 and 1
    assert [e.layer for e in plan.order] == [0, 1, 0, 2, 1] and len(plan.layers) == 3
    latent, delta, bare = plan.layers
    assert isinstance(latent.mixer, LatentAttentionSpec) and latent.mixer.position.interleaved
    assert (latent.mixer.num_heads, latent.mixer.qk_dim, latent.mixer.rot_dim, latent.mixer.kv_rank) == (3, 8, 4, 20)
    assert isinstance(delta.mixer, ChannelDeltaSpec) and (delta.mixer.decay_rank, delta.mixer.gate_rank) == plain.BOTTLENECKS
    assert isinstance(delta.ffn, RoutedExpertsSpec) and (delta.ffn.num_identity, delta.ffn.keep_groups) == (2, 2)
    assert delta.ffn.shared_size == 40 and delta.ffn.shared_limit == 0.7
    assert bare.ffn is None and bare.ffn_norm is None
    assert latent.mixer_norm.weight_offset == 1.0 and latent.mixer_norm.scale_in_fp32
    # every declared tensor is in the checkpoint and the other way round
    loader.check(DecoderModel(plan).tensor_decls(), stored_of(plain.TINY_A), plan.ignored_tensors)


def test_sizes_that_only_tensors_give():
    config = LemesunConfig.from_dict(plain.TINY_B)
    with pytest.raises(KeyError, match="bottlenecks"):
        config.to_plan()
    carried = copy.deepcopy(plain.TINY_B)
    for layer in carried["layers"]:
        if layer["type"] == "channel_delta":
            layer["mixer"].update(decay_rank=5, gate_rank=7)
    plan = LemesunConfig.from_dict(carried).to_plan()
    assert (plan.layers[0].mixer.decay_rank, plan.layers[0].mixer.gate_rank) == (5, 7)
    assert plan.layers[0].ffn.num_groups == 1 and plan.layers[0].ffn.shared_size == 0


@pytest.mark.parametrize("change,error", [
    (lambda c: c["layers"][0].update(type="convolution"), "known"),
    (lambda c: c["layers"][2].update(weights_of=7), "does not exist"),
    (lambda c: c["layers"][2].update(weights_of=1), "takes the weights of"),
    (lambda c: c["layers"][4].update(weights_of=2), "no tensors of its own"),
    (lambda c: c.pop("width"), "width"),
])
def test_bad_configurations_are_refused(change, error):
    cfg = copy.deepcopy(plain.TINY_A)
    change(cfg)
    with pytest.raises((ValueError, KeyError), match=error):
        LemesunConfig.from_dict(cfg)


def test_cache_groups_of_the_two_mixers():
    plan = LemesunConfig.from_dict(plain.TINY_A).plan_for(stored_of(plain.TINY_A))
    model = DecoderModel(plan)
    needs = [model.layers[e.layer].cache_needs() for e in plan.order]
    assert needs[0] == (KVNeed(1, 24, None, value_plane=False),)
    assert needs[1] == (StateNeed((4, 16, 8), torch.float32, "delta state"),
                        StateNeed((2, 96), torch.float32, "convolution inputs"))
    cache = SequenceCache(needs, [None] * len(needs), dtype=torch.float32, device="cpu", max_tokens=256, max_seqs=3)
    # the two runs of the latent layer share a group of single-plane rows, each with storage of its own
    (latent,) = cache.kv_groups
    assert latent.owners == [0, 2] and latent.pool.shape[:2] == (2, 1) and cache.view(0).values is None
    assert cache.view(0).keys.data_ptr() != cache.view(2).keys.data_ptr()
    # runs 1 and 4 keep states of the same shapes apart; run 3 has other sizes
    assert [g.owners for g in cache.state_groups] == [[1, 4], [1, 4], [3], [3]]
    first, second = cache.view(1).states
    assert first.shape == (4, 4, 16, 8) and second.shape == (4, 2, 96)
    assert cache.view(4).states[0].data_ptr() != first.data_ptr()
    # a slot that is used again starts from zero
    slot = cache.alloc()
    cache.view(1).states[0][slot].fill_(3.0)
    cache.view(4).states[1][slot].fill_(2.0)
    cache.free(slot)
    again = cache.alloc()
    assert again == slot and float(cache.view(1).states[0][slot].abs().sum()) == 0.0
    assert float(cache.view(4).states[1][slot].abs().sum()) == 0.0


def test_a_mixer_may_not_name_the_same_state_twice():
    need = StateNeed((2, 2))
    with pytest.raises(ValueError, match="twice"):
        SequenceCache([(need, need)], [None], dtype=torch.float32, device="cpu", max_tokens=64, max_seqs=1)


def test_the_plain_router_keeps_to_the_best_groups():
    g = torch.Generator().manual_seed(1)
    h = torch.randn(50, 8, generator=g)
    f = plain.moe(6, 2, 3, 4, 2, 8, 1.0)
    w = {"r.router": torch.randn(8, 8, generator=g), "r.correction": torch.randn(8, generator=g) * 0.1}
    chosen, weight = plain.route(h, w, "r.", f)
    groups = chosen // 2
    assert all(len(set(row.tolist())) <= 2 for row in groups) and float(weight.sum(-1).max()) <= 1.0 + 1e-6
