"""Mixture of experts whose choice is a table row per token id, with plain (ungated) experts and a shared expert
that a number per token scales.

Steps of ``forward`` (no step waits for the host):

1. ``ops.moe_table_route``: the token's experts are row ``token id`` of the table, each weighted 1 / top;
2. ``ops.moe_group``: the (token, choice) pairs sorted by expert on the device;
3. two grouped products over that order (``csrc/grouped_gemm.cu``): up with the activation in its epilogue, then
   down into fp32 rows; in bfloat16, when the experts get many rows each (prompts), the rows are gathered side by
   side and the vendor library's grouped product runs over the experts' row ranges;
4. ``ops.moe_combine``: each token adds its weighted rows in the order of its choices;
5. the shared expert, if any: up, activation, down, then ``ops.gated_row_add``: added times sigmoid(sg . x).
"""

from __future__ import annotations

import torch

from ..config.specs import TableExpertsSpec
from ..kernels import ops
from ..weights.tensors import TensorDecl
from .base import Part, register_part
from .linear import activated_linear, linear
from .routed_experts import ROWS_PER_EXPERT_FOR_TENSOR_CORES

GROUPED_EPILOGUE = {"gelu_erf": ops.GROUPED_GELU_ERF, "gelu_tanh": ops.GROUPED_GELU_TANH}


class TableExperts(Part):
    graph_safe = True
    returns_output = True   # forward(..., residual=None) returns the fp32 output instead of adding it
    _library_groups = True      # until the vendor library's grouped product has refused once

    def __init__(self, spec: TableExpertsSpec) -> None:
        super().__init__(spec)
        if spec.num_experts <= 0 or not 0 < spec.top_k <= spec.num_experts:
            raise ValueError("top_k must be between 1 and the number of experts")
        if spec.activation not in GROUPED_EPILOGUE:
            raise ValueError(f"activation {spec.activation!r} is not implemented ({sorted(GROUPED_EPILOGUE)} are)")

    def tensor_decls(self):
        s = self.spec
        decls = [TensorDecl(s.prefix + "table", (s.vocab_size, s.top_k), f"distinct_below:{s.num_experts}")]
        for e in range(s.num_experts):
            decls += [TensorDecl(f"{s.prefix}e{e}.up", (s.expert_size, s.hidden_size)),
                      TensorDecl(f"{s.prefix}e{e}.down", (s.hidden_size, s.expert_size))]
        if s.shared_size > 0:
            decls += [TensorDecl(s.prefix + "shared.up", (s.shared_size, s.hidden_size)),
                      TensorDecl(s.prefix + "shared.down", (s.hidden_size, s.shared_size))]
            if s.shared_gated:
                decls.append(TensorDecl(s.prefix + "shared.sg", (1, s.hidden_size)))
        return decls

    def load(self, fetch, runtime) -> None:
        s = self.spec
        self.runtime = runtime
        self.table = fetch.integer(s.prefix + "table")
        self.w_up = torch.stack([fetch.matrix(f"{s.prefix}e{e}.up") for e in range(s.num_experts)])
        self.w_down = torch.stack([fetch.matrix(f"{s.prefix}e{e}.down") for e in range(s.num_experts)])
        self.counts = torch.zeros(s.num_experts, dtype=torch.int32, device=runtime.device)
        if s.shared_size > 0:
            self.w_shared_up = fetch.matrix(s.prefix + "shared.up")
            self.w_shared_down = fetch.matrix(s.prefix + "shared.down")
            self.w_shared_gate = fetch.matrix(s.prefix + "shared.sg").reshape(-1).contiguous() if s.shared_gated else None

    def forward(self, x, ctx, residual):
        """Adds to ``residual`` (fp32); with ``residual`` None returns the output as a new fp32 tensor."""
        s = self.spec
        n, dev = x.shape[0], x.device
        ids = torch.empty((n, s.top_k), dtype=torch.int32, device=dev)
        weights = torch.empty((n, s.top_k), dtype=torch.float32, device=dev)
        ops.moe_table_route(self.table, ctx.token_ids, ids, weights, n_experts=s.num_experts, weight=1.0 / s.top_k)
        few_ok = ops.grouped_few_rows_ok((s.hidden_size, s.expert_size), x.dtype)
        table = ops.RoutingTable(n, s.top_k, s.num_experts, dev, few_rows_ok=few_ok)
        ops.moe_group(ids, self.counts, table)
        act = torch.empty((table.n_pairs, s.expert_size), dtype=x.dtype, device=dev)
        expert_out = None
        if (x.dtype == torch.bfloat16 and table.n_pairs >= ROWS_PER_EXPERT_FOR_TENSOR_CORES * s.num_experts
                and TableExperts._library_groups and s.hidden_size % 8 == 0 and s.expert_size % 8 == 0
                and not torch.cuda.is_current_stream_capturing()):
            expert_out = self._library_products(x, table, act)
        if expert_out is None:
            expert_out = torch.empty((table.n_pairs, s.hidden_size), dtype=torch.float32, device=dev)
            ops.grouped_gemm_routed(x, self.w_up, act, table, gather=True, epi=GROUPED_EPILOGUE[s.activation])
            ops.grouped_gemm_routed(act, self.w_down, expert_out, table, gather=False, epi=ops.GROUPED_STORE_F32)
        assign = residual is None
        if assign:
            residual = torch.empty((n, s.hidden_size), dtype=torch.float32, device=dev)
        ops.moe_combine(residual, expert_out, x, ids, weights, table, assign=assign)
        if s.shared_size > 0:
            shared = activated_linear(x, self.w_shared_up, s.activation)
            if self.w_shared_gate is None:
                linear(shared, self.w_shared_down, residual=residual)
            else:
                ops.gated_row_add(residual, linear(shared, self.w_shared_down, out_dtype=torch.float32), x, self.w_shared_gate)
        if ctx is not None:
            ctx.residual_sumsq = None
        return residual if assign else None

    def _library_products(self, x, table, act):
        """bfloat16 prompts: the experts' products by the vendor library's grouped product over rows gathered side
        by side (the experts' row ranges stay on the device); None if this build of the library has none."""
        s = self.spec
        rows = torch.empty((table.n_pairs, s.hidden_size), dtype=x.dtype, device=x.device)
        ops.moe_gather(x, table, rows)
        try:
            ends = table.offsets[1:]
            up = torch._grouped_mm(rows, self.w_up.transpose(1, 2), offs=ends)
            ops.activation(up, act, s.activation)
            down = torch._grouped_mm(act, self.w_down.transpose(1, 2), offs=ends)
            ops.LAUNCHES["library"] += 2
            return down                                   # rounded to the compute dtype; the combine widens it
        except (RuntimeError, AttributeError, TypeError, NotImplementedError) as error:
            TableExperts._library_groups = False
            import sys
            print(f"[ondeviceinfer_b200] no grouped product in the vendor library ({type(error).__name__}); "
                  "table-routed experts use this library's grouped kernels", file=sys.stderr)
            return None


register_part(TableExpertsSpec, TableExperts)
