"""Mixture of experts: a grouped top-k router, clamped gated experts, identity outputs and a shared expert.

Steps of ``forward`` (no step waits for the host):

1. router logits in fp32 (one product), then ``ops.moe_route``: softmax over all outputs, the correction for the
   choice only, the best groups, the top-k outputs and their scores as weights;
2. ``ops.moe_group``: the (token, choice) pairs that go to real experts, sorted by expert on the device;
3. two grouped products over that order (``csrc/grouped_gemm.cu``): gate and up with the clamped activation,
   then down into fp32 rows; in bfloat16, when the experts get many rows each (prompts), the rows are gathered
   side by side instead and the two products go to the tensor cores: the vendor library's grouped product
   over the experts' row ranges where it has one, else every expert's products through ``linear``, for which the
   host reads the experts' offsets once (the only wait of the part, and never inside a graph capture);
4. ``ops.moe_combine``: each token adds its weighted rows, in the order of its choices, and its own input for
   an identity output;
5. the shared expert, if any: gate/up product, the same activation with its own limit, down with the residual add.
"""

from __future__ import annotations

import torch

from ..config.specs import RoutedExpertsSpec
from ..kernels import ops
from ..weights.tensors import TensorDecl
from .base import Part, register_part
from .linear import linear


# From this many rows per expert on (on average) a bfloat16 step runs each expert's products through linear().
ROWS_PER_EXPERT_FOR_TENSOR_CORES = 32


class RoutedExperts(Part):
    graph_safe = True   # the grouped products wait for no one; the per-expert form is not chosen while capturing
    _library_groups = True      # until the vendor library's grouped product has refused once

    def __init__(self, spec: RoutedExpertsSpec) -> None:
        super().__init__(spec)
        n_all = spec.num_experts + spec.num_identity
        if spec.num_experts < 0 or spec.num_identity < 0 or n_all <= 0:
            raise ValueError("a router needs at least one output")
        if spec.num_groups <= 0 or n_all % spec.num_groups != 0:
            raise ValueError(f"{n_all} router outputs do not form {spec.num_groups} equal groups")
        if not 0 < spec.keep_groups <= spec.num_groups:
            raise ValueError("keep_groups must be between 1 and the number of groups")
        if not 0 < spec.top_k <= spec.keep_groups * (n_all // spec.num_groups):
            raise ValueError("top_k exceeds the outputs that the kept groups hold")
        self.n_all = n_all

    def tensor_decls(self):
        s = self.spec
        decls = [TensorDecl(s.prefix + "router", (self.n_all, s.hidden_size))]
        if s.has_correction:
            decls.append(TensorDecl(s.prefix + "correction", (self.n_all,), "zeros"))
        for e in range(s.num_experts):
            decls += [TensorDecl(f"{s.prefix}e{e}.gate", (s.expert_size, s.hidden_size)),
                      TensorDecl(f"{s.prefix}e{e}.up", (s.expert_size, s.hidden_size)),
                      TensorDecl(f"{s.prefix}e{e}.down", (s.hidden_size, s.expert_size))]
        if s.shared_size > 0:
            decls += [TensorDecl(s.prefix + "shared.gate", (s.shared_size, s.hidden_size)),
                      TensorDecl(s.prefix + "shared.up", (s.shared_size, s.hidden_size)),
                      TensorDecl(s.prefix + "shared.down", (s.hidden_size, s.shared_size))]
        return decls

    def load(self, fetch, runtime) -> None:
        s = self.spec
        self.runtime = runtime
        self.w_router = fetch.matrix(s.prefix + "router")
        self.correction = fetch.vector(s.prefix + "correction") if s.has_correction else None
        if s.num_experts > 0:
            # per expert: gate rows then up rows, so that one grouped product yields both
            self.w_gate_up = torch.stack([torch.cat([fetch.matrix(f"{s.prefix}e{e}.gate"), fetch.matrix(f"{s.prefix}e{e}.up")], 0)
                                          for e in range(s.num_experts)])
            self.w_down = torch.stack([fetch.matrix(f"{s.prefix}e{e}.down") for e in range(s.num_experts)])
            self.counts = torch.zeros(s.num_experts, dtype=torch.int32, device=runtime.device)
        if s.shared_size > 0:
            self.w_shared_gate_up = torch.cat([fetch.matrix(s.prefix + "shared.gate"), fetch.matrix(s.prefix + "shared.up")], 0)
            self.w_shared_down = fetch.matrix(s.prefix + "shared.down")

    def forward(self, x, ctx, residual) -> None:
        s = self.spec
        n, dev = x.shape[0], x.device
        logits = linear(x, self.w_router, out_dtype=torch.float32)
        ids = torch.empty((n, s.top_k), dtype=torch.int32, device=dev)
        weights = torch.empty((n, s.top_k), dtype=torch.float32, device=dev)
        ops.moe_route(logits, self.correction, ids, weights, n_groups=s.num_groups, keep=s.keep_groups)
        # single-token steps, a few rows per expert: the grouped product that streams weights through registers
        few_ok = ops.grouped_few_rows_ok((s.hidden_size, s.expert_size), x.dtype)
        table = ops.RoutingTable(n, s.top_k, max(s.num_experts, 1), dev, few_rows_ok=few_ok)
        expert_out = torch.empty((table.n_pairs, s.hidden_size), dtype=torch.float32, device=dev)
        if s.num_experts > 0:
            ops.moe_group(ids, self.counts, table)
            act = torch.empty((table.n_pairs, s.expert_size), dtype=x.dtype, device=dev)
            if (x.dtype == torch.bfloat16 and table.n_pairs >= ROWS_PER_EXPERT_FOR_TENSOR_CORES * s.num_experts
                    and not torch.cuda.is_current_stream_capturing()):
                expert_out = self._experts_one_by_one(x, table, act, expert_out)
            else:
                ops.grouped_gemm_routed(x, self.w_gate_up, act, table, gather=True, epi=ops.GROUPED_GATED_CLAMP,
                                        limit=s.limit, alpha=s.gate_alpha)
                ops.grouped_gemm_routed(act, self.w_down, expert_out, table, gather=False, epi=ops.GROUPED_STORE_F32)
        ops.moe_combine(residual, expert_out, x, ids, weights, table)
        if s.shared_size > 0:
            act = torch.empty((n, s.shared_size), dtype=x.dtype, device=dev)
            ops.gated_clamp(linear(x, self.w_shared_gate_up), act, s.shared_limit, s.gate_alpha)
            linear(act, self.w_shared_down, residual=residual, track=ctx)


    def _experts_one_by_one(self, x, table, act, expert_out):
        """The experts' outputs in the sorted order of pairs: ``expert_out``, or a tensor of the library's own."""
        s = self.spec
        rows = torch.empty((table.n_pairs, s.hidden_size), dtype=x.dtype, device=x.device)
        ops.moe_gather(x, table, rows)
        if self._library_groups and s.hidden_size % 8 == 0 and s.expert_size % 8 == 0:
            # the vendor library's grouped product: the experts' row ranges stay on the device, nothing waits
            try:
                ends = table.offsets[1:]
                gate_up = torch._grouped_mm(rows, self.w_gate_up.transpose(1, 2), offs=ends)
                ops.gated_clamp(gate_up, act, s.limit, s.gate_alpha)
                down = torch._grouped_mm(act, self.w_down.transpose(1, 2), offs=ends)
                ops.LAUNCHES["library"] += 2
                return down                                   # rounded to the compute dtype; the combine widens it
            except (RuntimeError, AttributeError, TypeError, NotImplementedError) as error:
                RoutedExperts._library_groups = False           # this build of the library has none: one by one
                import sys
                print(f"[ondeviceinfer_b200] no grouped product in the vendor library ({type(error).__name__}); "
                      "routed experts run one by one", file=sys.stderr)
        bounds = table.offsets.tolist()                     # waits for the device
        for e in range(s.num_experts):
            lo, hi = bounds[e], bounds[e + 1]
            if hi > lo:
                ops.gated_clamp(linear(rows[lo:hi], self.w_gate_up[e]), act[lo:hi], s.limit, s.gate_alpha)
                expert_out[lo:hi].copy_(linear(act[lo:hi], self.w_down[e], out_dtype=torch.float32))
        return expert_out


register_part(RoutedExpertsSpec, RoutedExperts)
