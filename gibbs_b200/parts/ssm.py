"""A selective state-space mixer with scalar decay per head (the
"state-space duality" form), with its short causal convolution, gate and
grouped RMS norm.

With inner = heads * vdim, N = state, G = groups, the input projection gives
[z: inner | x: inner | B: G*N | C: G*N | dt: heads].  x, B and C pass a causal
convolution per channel (``conv`` taps, the last one on the current token, zeros
before the start) and silu.  Then per head h (group g = h // (heads / G)):

    dt_t = softplus(dt_t + dt_bias_h)
    S_t  = exp(-exp(A_log_h) * dt_t) * S_(t-1) + dt_t * B_t x_t^T        S: [N, vdim]
    y_t  = S_t^T C_t + D_h x_t

y (heads side by side) is multiplied by silu(z), RMS-normed in ``norm_groups``
equal parts, multiplied by a gain, and projected out.  Per request a slot
holds the convolution's last conv - 1 inputs and S, both in 32-bit; the
recurrence, decays, step sizes and the norm are 32-bit in every compute dtype
(csrc/ssm.cu, csrc/norms.cu).
"""
from __future__ import annotations

import torch

from .. import ops
from ..ops import hybrid
from .base import Mixer, SlotState, TensorDecl, VECTOR, register_part
from .runner import BranchPart, Runner, keep


class StateSpaceMixer(BranchPart, Mixer):
    @classmethod
    def declare(cls, params):
        d, H, P, N, G, K = (params[k] for k in ("hidden", "heads", "vdim", "state", "groups", "conv"))
        inner, ch = H * P, H * P + 2 * G * N
        return {"in": TensorDecl.of(2 * inner + 2 * G * N + H, d), "conv": TensorDecl.of(ch, K, role=VECTOR),
                "conv.b": TensorDecl.of(ch, role=VECTOR), "dt_bias": TensorDecl.of(H, role=VECTOR),
                "A_log": TensorDecl.of(H, role=VECTOR), "D": TensorDecl.of(H, role=VECTOR),
                "norm": TensorDecl.of(inner, role=VECTOR), "o": TensorDecl.of(d, inner)}

    def __init__(self, params, tensors, rt):
        super().__init__(params, tensors, rt)
        p = params
        self.hidden, self.heads, self.P, self.N = int(p["hidden"]), int(p["heads"]), int(p["vdim"]), int(p["state"])
        self.G, self.K, self.norm_groups = int(p["groups"]), int(p["conv"]), int(p.get("norm_groups", 1))
        self.eps = float(p["eps"])
        self.inner = self.heads * self.P
        self.channels = self.inner + 2 * self.G * self.N
        if self.heads % self.G or self.inner % self.norm_groups or self.K < 1:
            raise ValueError(f"{self.heads} heads in {self.G} groups, {self.inner} columns in {self.norm_groups} norm "
                             f"groups, {self.K} taps")
        f32 = lambda n: tensors[n].to(torch.float32).contiguous()
        self.w_in, self.w_out = tensors["in"].contiguous(), tensors["o"].contiguous()
        self.taps = f32("conv").reshape(self.channels, self.K).contiguous()
        self.conv_bias, self.dt_bias, self.a_log, self.d_skip, self.gain = (f32(n) for n in
                                                                           ("conv.b", "dt_bias", "A_log", "D", "norm"))

    def kernel_libraries(self):
        return tuple(set(ops.linear_libraries(self.w_in.dtype, self.rt.dtype)) | {"core", hybrid.LIBRARY})

    def cache_needs(self):
        # (a convolution of one tap has nothing to remember; its slot is one unused row)
        return [SlotState((max(self.K - 1, 1), self.channels), torch.float32),
                SlotState((self.heads, self.P, self.N), torch.float32)]

    def run(self, rn: Runner, h, out, caches):
        conv, rec = caches[0], caches[1]
        inner, ch, H, G, N = self.inner, self.channels, self.heads, self.G, self.N
        width = 2 * inner + 2 * G * N + H
        u = rn.buffer("ssm_in", width, torch.float32)
        rn.linear(h, self.w_in, None, u, role="ssm_in")
        xbc = rn.buffer("ssm_conv", ch, torch.float32)
        slots = rn.slots(conv)
        rn.op("causal_conv_silu", [u.data_ptr() + 4 * inner, u.stride(0), keep(rn, self.taps), keep(rn, self.conv_bias),
                                   keep(rn, conv.state), conv.state.stride(0), slots, rn.tok_req, rn.q_start, rn.q_len,
                                   xbc.data_ptr(), xbc.stride(0), rn.N, ch, self.K, rn.R])
        y = rn.buffer("ssm_y", inner, torch.float32)
        rn.op("ssm_scan", [xbc.data_ptr(), xbc.stride(0), u.data_ptr() + 4 * (2 * inner + 2 * G * N), u.stride(0),
                           keep(rn, self.dt_bias), keep(rn, self.a_log), keep(rn, self.d_skip), keep(rn, rec.state),
                           rec.state.stride(0), slots, rn.q_start, rn.q_len, y.data_ptr(), y.stride(0), rn.R, H, self.P,
                           N, G])
        o = rn.buffer("ssm_gated", inner)
        rn.op("gated_group_norm", [y.data_ptr(), y.stride(0), u.data_ptr(), u.stride(0), keep(rn, self.gain),
                                   o.data_ptr(), ops.dtype_code(o.dtype), o.stride(0), rn.N, inner, self.norm_groups],
              [self.eps])
        rn.linear(o, self.w_out, None, out, role="ssm_out")


register_part("mixer", "state_space", StateSpaceMixer)
