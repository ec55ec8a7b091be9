"""Typed configuration of the Nulalorn decoder, read from its own ``config.json`` keys.

``config.json`` holds ``vocab``, ``width``, ``norm.eps``, ``logit_softcap``, a list ``layers`` and ``loop``.  Each
layer has ``type`` (``attention``), the mixer's sizes and constants under ``mixer`` (``heads``, ``kv_heads``,
``dim``, ``vdim``, ``scale``, ``softcap``, ``mask.size``, ``rot.base|dims|scaling``) and its feed-forward under
``mlp`` (null: none; ``kind`` ``dense`` with ``ff``, or ``moe`` with ``expert.ff``, ``router.experts|top`` and
``shared.ff``).  ``loop`` (``start``, ``stop``, ``times``) runs layers start..stop-1 ``times`` times in a row with
the same tensors and a cache of their own per pass; every pass opens with h <- W [h ; embedding] + step[pass].
A key that is absent switches its mechanism off (no window, no cap, no scaling, no shared expert, no loop).
Tensor names: ``embed``, ``loop.in``, ``loop.step``, ``l<i>.norm1|norm1b|norm2|norm2b``, ``l<i>.mix.q|k|v|o``,
``l<i>.mlp.up|down`` or ``l<i>.mlp.table``, ``l<i>.mlp.e<j>.up|down``, ``l<i>.mlp.shared.up|down|sg``,
``final.norm``, ``head``.

Norms scale in fp32 by the stored weight; rotary pairs are neighbouring lanes; the residual stream, the norms on
both sides of a sublayer, scores and softmax are fp32 in both compute dtypes.
"""

from __future__ import annotations

import copy
from dataclasses import dataclass
from typing import Any, List, Mapping, Optional, Tuple

from .specs import (CappedAttentionSpec, EmbeddingSpec, HeadSpec, MLPSpec, ModelPlan, NoPositionSpec, OrderEntry,
                    ReinjectSpec, RMSNormSpec, RotarySpec, SandwichBlockSpec, TableExpertsSpec, names)

MIXERS = ("attention",)
FEED_FORWARDS = ("dense", "moe")
ACTIVATION = "gelu_erf"         # the design fixes the exact (erf) GELU in every feed-forward


def _need(raw: Mapping[str, Any], key: str, where: str):
    if not isinstance(raw, Mapping) or key not in raw:
        raise KeyError(f"config.json: {where} lacks {key!r}")
    return raw[key]


@dataclass(frozen=True)
class NulalornConfig:
    vocab_size: int
    hidden_size: int
    norm_eps: float
    layers: Tuple[Mapping[str, Any], ...]     # the entries of config.json["layers"], as read
    loop: Optional[Tuple[int, int, int]] = None       # (start, stop, times)
    logit_softcap: Optional[float] = None

    architecture = "Nulalorn"

    # ------------------------------------------------------------------ construction

    @classmethod
    def from_dict(cls, raw: Mapping[str, Any]) -> "NulalornConfig":
        layers = _need(raw, "layers", "the model")
        if not isinstance(layers, list) or not layers:
            raise ValueError("config.json: 'layers' must be a non-empty list")
        loop = raw.get("loop")
        if loop is not None:
            loop = tuple(int(_need(loop, key, "loop")) for key in ("start", "stop", "times"))
        cap = raw.get("logit_softcap")
        config = cls(vocab_size=int(_need(raw, "vocab", "the model")), hidden_size=int(_need(raw, "width", "the model")),
                     norm_eps=float(_need(_need(raw, "norm", "the model"), "eps", "norm")),
                     layers=tuple(copy.deepcopy(layer) for layer in layers), loop=loop,
                     logit_softcap=None if cap is None else float(cap))
        config.validate()
        return config

    def to_dict(self) -> dict:
        out = {"architecture": self.architecture, "layers": [copy.deepcopy(dict(layer)) for layer in self.layers],
               "norm": {"eps": self.norm_eps}, "vocab": self.vocab_size, "width": self.hidden_size}
        if self.loop is not None:
            out["loop"] = dict(zip(("start", "stop", "times"), self.loop))
        if self.logit_softcap is not None:
            out["logit_softcap"] = self.logit_softcap
        return out

    def validate(self) -> None:
        if self.vocab_size <= 0 or self.hidden_size <= 0 or self.norm_eps <= 0:
            raise ValueError("vocab, width and norm.eps must be positive")
        if self.logit_softcap is not None and self.logit_softcap <= 0:
            raise ValueError("logit_softcap must be positive")
        for i, layer in enumerate(self.layers):
            if layer.get("type") not in MIXERS:
                raise ValueError(f"layers[{i}].type is {layer.get('type')!r}; known: {MIXERS}")
            f = layer.get("mlp")
            if f is not None and f.get("kind") not in FEED_FORWARDS:
                raise ValueError(f"layers[{i}].mlp.kind is {f.get('kind')!r}; known: {FEED_FORWARDS}")
        if self.loop is not None:
            start, stop, times = self.loop
            if not 0 <= start < stop <= len(self.layers) or times < 1:
                raise ValueError(f"loop {self.loop}: 0 <= start < stop <= {len(self.layers)} layers and times >= 1")

    @property
    def stop_token_ids(self) -> tuple:
        return ()

    # ------------------------------------------------------------------ the plan

    def _norm(self, name: str) -> RMSNormSpec:
        return RMSNormSpec(self.hidden_size, self.norm_eps, name, scale_in_fp32=True)

    def _mixer(self, i: int, layer: Mapping[str, Any]) -> CappedAttentionSpec:
        m, where = _need(layer, "mixer", f"layers[{i}]"), f"layers[{i}].mixer"
        head_dim = int(_need(m, "dim", where))
        rot = m.get("rot")
        position = NoPositionSpec()
        if rot is not None:
            scaling = rot.get("scaling")
            if scaling is not None:
                scaling = tuple(float(_need(scaling, key, where + ".rot.scaling"))
                                for key in ("factor", "low", "high", "original"))
            position = RotarySpec(head_dim=head_dim, theta=float(_need(rot, "base", where + ".rot")),
                                  rotary_dim=int(_need(rot, "dims", where + ".rot")), interleaved=True, scaling=scaling)
        heads = int(_need(m, "heads", where))
        window = (m.get("mask") or {}).get("size")
        cap = m.get("softcap")
        return CappedAttentionSpec(
            hidden_size=self.hidden_size, num_heads=heads, num_kv_heads=int(m.get("kv_heads", heads)), head_dim=head_dim,
            value_dim=int(m.get("vdim", head_dim)), scale=float(_need(m, "scale", where)), position=position,
            prefix=f"l{i}.mix.", names=names(q="q", k="k", v="v", o="o"), softcap=None if cap is None else float(cap),
            window=None if window is None else int(window), unit_norm_eps=self.norm_eps)

    def _mlp(self, i: int, layer: Mapping[str, Any]):
        f = layer.get("mlp")
        if f is None:
            return None
        where, prefix = f"layers[{i}].mlp", f"l{i}.mlp."
        if f["kind"] == "dense":
            return MLPSpec(self.hidden_size, int(_need(f, "ff", where)), ACTIVATION, prefix, names(up="up", down="down"))
        router = _need(f, "router", where)
        shared = f.get("shared") or {}
        return TableExpertsSpec(
            hidden_size=self.hidden_size, expert_size=int(_need(_need(f, "expert", where), "ff", where + ".expert")),
            num_experts=int(_need(router, "experts", where + ".router")), top_k=int(_need(router, "top", where + ".router")),
            vocab_size=self.vocab_size, prefix=prefix, activation=ACTIVATION, shared_size=int(shared.get("ff", 0)),
            shared_gated=True)

    def layer_runs(self) -> List[Tuple[int, Optional[int]]]:
        """The executions in order: (layer, the number of the pass that this execution opens, or None)."""
        n = len(self.layers)
        if self.loop is None:
            return [(i, None) for i in range(n)]
        start, stop, times = self.loop
        runs: List[Tuple[int, Optional[int]]] = [(i, None) for i in range(start)]
        for t in range(times):
            runs += [(i, t if i == start else None) for i in range(start, stop)]
        return runs + [(i, None) for i in range(stop, n)]

    def to_plan(self) -> ModelPlan:
        layers: List[object] = []
        ignored: List[str] = []
        for i, layer in enumerate(self.layers):
            mlp = self._mlp(i, layer)
            has = mlp is not None
            layers.append(SandwichBlockSpec(
                mixer_norm=self._norm(f"l{i}.norm1"), mixer=self._mixer(i, layer), mixer_post_norm=self._norm(f"l{i}.norm1b"),
                ffn_norm=self._norm(f"l{i}.norm2") if has else None, ffn=mlp,
                ffn_post_norm=self._norm(f"l{i}.norm2b") if has else None))
            if not has:
                ignored += [f"l{i}.norm2", f"l{i}.norm2b"]
        order: List[OrderEntry] = []
        for i, opens in self.layer_runs():
            if opens is not None:
                # the step that opens pass `opens`: a layer of its own in the plan (all passes bind the same tensors)
                layers.append(ReinjectSpec(self.hidden_size, "loop.in", "loop.step", self.loop[2], opens))
                order.append(OrderEntry(layer=len(layers) - 1))
            order.append(OrderEntry(layer=i))
        plan = ModelPlan(embedding=EmbeddingSpec(self.vocab_size, self.hidden_size, "embed"), layers=tuple(layers),
                         order=tuple(order), final_norm=self._norm("final.norm"),
                         head=HeadSpec(self.vocab_size, self.hidden_size, "head", softcap=self.logit_softcap),
                         ignored_tensors=tuple(ignored))
        plan.validate()
        return plan
