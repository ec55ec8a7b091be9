"""Typed configuration of the Lemesun decoder, read from its own ``config.json`` keys.

``config.json`` holds ``vocab``, ``width``, ``norm.eps`` and a list ``layers``; each entry has ``type``
(``latent_attention`` or ``channel_delta``), the mixer's sizes under ``mixer`` and its feed-forward under ``mlp``
(null: none).  An entry with ``weights_of: j`` runs layer j's tensors again with a cache or state of its own.
Tensor names: ``embed``, ``l<i>.norm1``, ``l<i>.norm2``, ``l<i>.mix.*``, ``l<i>.mlp.*``, ``final.norm``, ``head``.

Every norm of the block stores its weight as the deviation from one and scales in fp32; rotary pairs are
neighbouring lanes; the residual stream, scores, routing and recurrent state are fp32 in both compute dtypes.
"""

from __future__ import annotations

import copy
from dataclasses import dataclass
from typing import Any, List, Mapping, Optional, Tuple

from .specs import (ChannelDeltaSpec, EmbeddingSpec, HeadSpec, LatentAttentionSpec, ModelPlan, OrderEntry,
                    PreNormBlockSpec, RMSNormSpec, RotarySpec, RoutedExpertsSpec, names)

MIXERS = ("latent_attention", "channel_delta")


def _need(raw: Mapping[str, Any], key: str, where: str):
    if key not in raw:
        raise KeyError(f"config.json: {where} lacks {key!r}")
    return raw[key]


@dataclass(frozen=True)
class LemesunConfig:
    vocab_size: int
    hidden_size: int
    norm_eps: float
    layers: Tuple[Mapping[str, Any], ...]     # the entries of config.json["layers"], as read

    architecture = "Lemesun"

    # ------------------------------------------------------------------ construction

    @classmethod
    def from_dict(cls, raw: Mapping[str, Any]) -> "LemesunConfig":
        layers = _need(raw, "layers", "the model")
        if not isinstance(layers, list) or not layers:
            raise ValueError("config.json: 'layers' must be a non-empty list")
        config = cls(vocab_size=int(_need(raw, "vocab", "the model")), hidden_size=int(_need(raw, "width", "the model")),
                     norm_eps=float(_need(_need(raw, "norm", "the model"), "eps", "norm")),
                     layers=tuple(copy.deepcopy(layer) for layer in layers))
        config.validate()
        return config

    def to_dict(self) -> dict:
        return {"architecture": self.architecture, "layers": [copy.deepcopy(dict(layer)) for layer in self.layers],
                "norm": {"eps": self.norm_eps}, "vocab": self.vocab_size, "width": self.hidden_size}

    def validate(self) -> None:
        if self.vocab_size <= 0 or self.hidden_size <= 0 or self.norm_eps <= 0:
            raise ValueError("vocab, width and norm.eps must be positive")
        for i, layer in enumerate(self.layers):
            if layer.get("type") not in MIXERS:
                raise ValueError(f"layers[{i}].type is {layer.get('type')!r}; known: {MIXERS}")
            source = layer.get("weights_of")
            if source is not None:
                if not (isinstance(source, int) and 0 <= source < len(self.layers)) or source == i:
                    raise ValueError(f"layers[{i}].weights_of names layer {source!r}, which does not exist")
                if self.layers[source].get("weights_of") is not None:
                    raise ValueError(f"layers[{i}].weights_of names layer {source}, which has no tensors of its own")
                if self.layers[source].get("type") != layer.get("type"):
                    raise ValueError(f"layers[{i}] is a {layer.get('type')} but takes the weights of a "
                                     f"{self.layers[source].get('type')}")
            kind = (layer.get("mlp") or {}).get("kind", "moe")
            if kind != "moe":
                raise ValueError(f"layers[{i}].mlp.kind is {kind!r}; this design's feed-forward is 'moe'")

    @property
    def stop_token_ids(self) -> tuple:
        return ()

    # ------------------------------------------------------------------ the plan

    def _norm(self, name: str) -> RMSNormSpec:
        return RMSNormSpec(self.hidden_size, self.norm_eps, name, weight_offset=1.0, scale_in_fp32=True)

    def _mixer(self, i: int, layer: Mapping[str, Any]):
        m, p = _need(layer, "mixer", f"layers[{i}]"), f"l{i}.mix."
        where = f"layers[{i}].mixer"
        if layer["type"] == "latent_attention":
            rot = _need(m, "rot", where)
            rot_dim = int(_need(m, "rot_dim", where))
            return LatentAttentionSpec(
                hidden_size=self.hidden_size, num_heads=int(_need(m, "heads", where)), qk_dim=int(_need(m, "dim", where)),
                rot_dim=rot_dim, v_dim=int(_need(m, "vdim", where)), kv_rank=int(_need(m, "kv_rank", where)),
                scale=float(_need(m, "scale", where)), norm_eps=self.norm_eps,
                position=RotarySpec(head_dim=rot_dim, theta=float(_need(rot, "base", where + ".rot")),
                                    rotary_dim=int(_need(rot, "dims", where + ".rot")), interleaved=True),
                prefix=p, names=names(q="q", dkv="dkv", dkv_norm="dkv.norm", uk="uk", uv="uv", o="o"))
        heads = int(_need(m, "heads", where))
        return ChannelDeltaSpec(
            hidden_size=self.hidden_size, num_heads=heads, num_kv_heads=int(m.get("kv_heads", heads)),
            qk_dim=int(_need(m, "dim", where)), v_dim=int(_need(m, "vdim", where)), conv_taps=int(_need(m, "conv", where)),
            decay_rank=int(m["decay_rank"]), gate_rank=int(m["gate_rank"]), norm_eps=self.norm_eps, prefix=p,
            names=names(q="q", k="k", v="v", q_conv="q.conv", k_conv="k.conv", v_conv="v.conv", b="b", A_log="A_log",
                        dt_bias="dt_bias", a1="a1", a2="a2", g1="g1", g2="g2", norm="norm", o="o"))

    def _mlp(self, i: int, layer: Mapping[str, Any]) -> Optional[RoutedExpertsSpec]:
        f = layer.get("mlp")
        if f is None:
            return None
        where = f"layers[{i}].mlp"
        router, expert = _need(f, "router", where), _need(f, "expert", where)
        groups = router.get("groups") or {}
        shared = f.get("shared") or {}
        return RoutedExpertsSpec(
            hidden_size=self.hidden_size, expert_size=int(_need(expert, "ff", where + ".expert")),
            num_experts=int(_need(router, "experts", where + ".router")), num_identity=int(router.get("identity", 0)),
            top_k=int(_need(router, "top", where + ".router")), num_groups=int(groups.get("count", 1)),
            keep_groups=int(groups.get("keep", groups.get("count", 1))), limit=float(_need(expert, "limit", where + ".expert")),
            prefix=f"l{i}.mlp.", has_correction=True, shared_size=int(shared.get("ff", 0)),
            shared_limit=float(shared.get("limit", 0.0)))

    def to_plan(self, bottlenecks: Optional[Mapping[int, Tuple[int, int]]] = None) -> ModelPlan:
        """The layer table.  A layer's two low-rank widths (decay, output gate) are not in ``config.json``: they are
        the shapes of its ``a1`` and ``g1`` tensors, given here as ``bottlenecks[layer] = (decay, gate)``; a
        configuration may also carry them as ``mixer.decay_rank`` / ``mixer.gate_rank``."""
        layers: List[PreNormBlockSpec] = []
        index_of = {}
        ignored = []
        for i, layer in enumerate(self.layers):
            if layer.get("weights_of") is not None:
                continue
            if layer["type"] == "channel_delta":
                m = dict(layer["mixer"])
                given = (bottlenecks or {}).get(i)
                if given is not None:
                    m["decay_rank"], m["gate_rank"] = given
                elif "decay_rank" not in m or "gate_rank" not in m:
                    raise KeyError(f"layers[{i}]: the widths of the decay and gate bottlenecks are known neither "
                                   "from the checkpoint's tensors nor from mixer.decay_rank / mixer.gate_rank")
                layer = {**layer, "mixer": m}
            mlp = self._mlp(i, layer)
            index_of[i] = len(layers)
            layers.append(PreNormBlockSpec(mixer_norm=self._norm(f"l{i}.norm1"), mixer=self._mixer(i, layer),
                                           ffn_norm=self._norm(f"l{i}.norm2") if mlp is not None else None, ffn=mlp))
            if mlp is None:
                ignored.append(f"l{i}.norm2")
        order = tuple(OrderEntry(layer=index_of[layer.get("weights_of", i) if layer.get("weights_of") is not None else i])
                      for i, layer in enumerate(self.layers))
        plan = ModelPlan(embedding=EmbeddingSpec(self.vocab_size, self.hidden_size, "embed"), layers=tuple(layers),
                         order=order, final_norm=self._norm("final.norm"),
                         head=HeadSpec(self.vocab_size, self.hidden_size, "head"), ignored_tensors=tuple(ignored))
        plan.validate()
        return plan

    def plan_for(self, stored: Mapping[str, Any]) -> ModelPlan:
        """The plan for a checkpoint whose tensors are ``stored`` (name -> something with ``shape``): sizes that
        only the tensors give are read from them."""
        found = {}
        for i, layer in enumerate(self.layers):
            if layer["type"] == "channel_delta" and layer.get("weights_of") is None:
                a1, g1 = stored.get(f"l{i}.mix.a1"), stored.get(f"l{i}.mix.g1")
                if a1 is not None and g1 is not None:
                    found[i] = (int(a1.shape[0]), int(g1.shape[0]))
        return self.to_plan(found)
