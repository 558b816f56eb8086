"""A per-layer input that depends on the token's id: every layer owns a slice
of a second embedding table and adds, after its feed-forward,

    e = table[token][offset : offset + dim]
    g = gelu_tanh(W_gate x) * e
    y = W_proj g
    x <- x + y / sqrt(mean(y^2) + eps) * gain

to the stream x (an RMS norm with a plain gain, whatever the model's norm is).
In float32 both products read and write 32-bit values; in bfloat16 they read
bfloat16 roundings of the stream and of g and accumulate in 32-bit.
"""
from __future__ import annotations

import torch

from .. import ops
from ..ops import hybrid
from .base import Part, TensorDecl, VECTOR, register_part
from .runner import Eager, Planned, Runner, keep, stream_tensor


class GatedTokenInput(Part):
    category = "token_input"

    @classmethod
    def declare(cls, params):
        h, d = params["hidden"], params["dim"]
        return {"table": TensorDecl.of(params["vocab"], params["table_width"]), "gate": TensorDecl.of(d, h),
                "proj": TensorDecl.of(h, d), "norm": TensorDecl.of(h, role=VECTOR)}

    def __init__(self, params, tensors, rt):
        super().__init__(params, tensors, rt)
        self.hidden, self.dim, self.offset = int(params["hidden"]), int(params["dim"]), int(params["offset"])
        self.vocab, self.eps = int(params["vocab"]), float(params["eps"])
        self.table = tensors["table"]                      # shared by every layer: one copy in memory
        if self.offset + self.dim > self.table.shape[1]:
            raise ValueError(f"columns {self.offset}..{self.offset + self.dim} of a table {self.table.shape[1]} wide")
        self.gate, self.proj = tensors["gate"].contiguous(), tensors["proj"].contiguous()
        self.gain = tensors["norm"].to(torch.float32).contiguous()

    def kernel_libraries(self):
        return ("core", hybrid.LIBRARY)

    def step_weight_bytes(self, n_tokens: int, seen: set) -> int:
        # (the table's rows a step gathers are not counted, as for the token embedding)
        return (self.gate.numel() + self.proj.numel()) * self.gate.element_size() + self.gain.numel() * 4

    def run(self, rn: Runner, x: torch.Tensor, x_rows: torch.Tensor = None) -> None:
        """``x``: the stream (float32), which receives the result; ``x_rows``: the same rows in
        bfloat16 when the caller has them (the products then run on the tensor cores)."""
        g = rn.buffer("token_input_gate", self.dim, torch.float32)
        rn.linear(x if x_rows is None else x_rows, self.gate, None, g, role="token_input_gate")
        g16 = None if x_rows is None else rn.buffer("token_input_gated", self.dim, torch.bfloat16)
        rn.op("gelu_mul_rows", [g.data_ptr(), g.stride(0), keep(rn, self.table), ops.dtype_code(self.table.dtype),
                                self.table.stride(0), self.offset, rn.token_ids, rn.N, self.dim, self.vocab,
                                0 if g16 is None else g16.data_ptr()])
        y = rn.buffer("branch", self.hidden, torch.float32)
        rn.linear(g if g16 is None else g16, self.proj, None, y, role="token_input_proj")
        rn.op("norm_add", [x.data_ptr(), x.stride(0), y.data_ptr(), y.stride(0), keep(rn, self.gain), rn.N,
                           self.hidden, hybrid.NORM_RMS], [self.eps], label="norm_add")

    def forward(self, x, step) -> None:
        self.run(Eager(self.rt, step), stream_tensor(x))

    def plan_ops(self, plan) -> None:
        self.run(Planned(plan), plan.residual)


register_part("token_input", "gated_token_input", GatedTokenInput)
