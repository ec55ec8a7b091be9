"""The gated delta rule with a decay per head and key channel: a recurrent mixer whose cache is a matrix
state per head and the last inputs of its short convolutions.

Steps of ``forward``: one product for q, k, v (before their convolutions) and the beta logits; one product for
the two low-rank bottlenecks (decay and output gate) and one, block-diagonal, for their second halves (fp32
out: what enters the recurrence besides q, k and v stays in 32 bits); then ``ops.delta_rule`` (convolutions with
SiLU and their state, unit vectors, decays, the recurrence over each sequence's tokens in order, the gated
per-head norm of the read-outs: ``csrc/delta.cu``); then the output projection with the residual add.

The state [heads, qk_dim, v_dim] and the convolution inputs [taps - 1, channels] are fp32 rows of the cache's
state groups, zero when a sequence starts, advanced over all tokens a sequence brings in a step.
"""

from __future__ import annotations

import torch

from ..cache import StateNeed
from ..config.specs import ChannelDeltaSpec
from ..kernels import ops
from ..weights.tensors import TensorDecl
from .base import Part, register_part
from .linear import linear


class ChannelDelta(Part):
    graph_safe = True   # no host work that depends on the step's values

    def __init__(self, spec: ChannelDeltaSpec) -> None:
        super().__init__(spec)
        for key in ("num_heads", "num_kv_heads", "qk_dim", "v_dim", "conv_taps", "decay_rank", "gate_rank"):
            if getattr(spec, key) <= 0:
                raise ValueError(f"{key} must be positive, got {getattr(spec, key)}")
        if spec.num_heads % spec.num_kv_heads != 0:
            raise ValueError("heads must be divisible by kv_heads")
        if spec.conv_taps > 16 or spec.qk_dim > ops.DELTA_MAX_DIM:
            raise ValueError(f"the delta rule kernels take up to 16 taps and key sizes up to {ops.DELTA_MAX_DIM}")
        self.qk_channels = spec.num_kv_heads * spec.qk_dim
        self.v_channels = spec.num_heads * spec.v_dim
        self.channels = 2 * self.qk_channels + self.v_channels

    def tensor_decls(self):
        s = self.spec
        H, qk, v = s.hidden_size, self.qk_channels, self.v_channels
        return [TensorDecl(s.name("q"), (qk, H)), TensorDecl(s.name("q_conv"), (qk, s.conv_taps)),
                TensorDecl(s.name("k"), (qk, H)), TensorDecl(s.name("k_conv"), (qk, s.conv_taps)),
                TensorDecl(s.name("v"), (v, H)), TensorDecl(s.name("v_conv"), (v, s.conv_taps)),
                TensorDecl(s.name("b"), (s.num_heads, H)), TensorDecl(s.name("A_log"), (s.num_heads,)),
                TensorDecl(s.name("norm"), (s.v_dim,), "one_plus_normal"),
                TensorDecl(s.name("a1"), (s.decay_rank, H)), TensorDecl(s.name("a2"), (s.num_heads * s.qk_dim, s.decay_rank)),
                TensorDecl(s.name("dt_bias"), (s.num_heads * s.qk_dim,)),
                TensorDecl(s.name("g1"), (s.gate_rank, H)), TensorDecl(s.name("g2"), (v, s.gate_rank)),
                TensorDecl(s.name("o"), (H, v))]

    def load(self, fetch, runtime) -> None:
        s = self.spec
        self.runtime = runtime
        self.w_in = torch.cat([fetch.matrix(s.name(r)) for r in ("q", "k", "v", "b")], 0)
        self.w_low = torch.cat([fetch.matrix(s.name("a1")), fetch.matrix(s.name("g1"))], 0)
        a2, g2 = fetch.matrix(s.name("a2")), fetch.matrix(s.name("g2"))
        # [a2 0; 0 g2]: one product gives the decay's inner term and the gate's logits side by side
        self.w_high = torch.zeros((a2.shape[0] + g2.shape[0], s.decay_rank + s.gate_rank), dtype=a2.dtype, device=a2.device)
        self.w_high[:a2.shape[0], :s.decay_rank] = a2
        self.w_high[a2.shape[0]:, s.decay_rank:] = g2
        self.taps = torch.cat([fetch.vector(s.name(r)) for r in ("q_conv", "k_conv", "v_conv")], 0)
        self.a_log = fetch.vector(s.name("A_log"))
        self.dt_bias = fetch.vector(s.name("dt_bias"))
        self.out_norm = fetch.vector(s.name("norm"))
        self.w_o = fetch.matrix(s.name("o"))

    def cache_needs(self):
        s = self.spec
        needs = [StateNeed((s.num_heads, s.qk_dim, s.v_dim), torch.float32, "delta state")]
        if s.conv_taps > 1:
            needs.append(StateNeed((s.conv_taps - 1, self.channels), torch.float32, "convolution inputs"))
        return tuple(needs)

    def forward(self, x, ctx, view, residual) -> None:
        s = self.spec
        proj = linear(x, self.w_in)
        inner = linear(linear(x, self.w_low), self.w_high, out_dtype=torch.float32)
        out = torch.empty((x.shape[0], self.v_channels), dtype=proj.dtype, device=proj.device)
        ops.delta_rule(proj, inner, self.taps, self.a_log, self.dt_bias, self.out_norm,
                       view.states[1] if s.conv_taps > 1 else None, view.states[0], out, ctx.cu_q, ctx.tok_seq,
                       ctx.slots, n_seqs=ctx.n_seqs, heads=s.num_heads, kv_heads=s.num_kv_heads, d=s.qk_dim,
                       dv=s.v_dim, eps=s.norm_eps, unit_eps=s.unit_eps)
        linear(out, self.w_o, residual=residual, track=ctx)


register_part(ChannelDeltaSpec, ChannelDelta)
