"""Arrangements of norm, mixer and feed-forward around the residual stream."""
from __future__ import annotations

import torch

from .base import Block, plan_ops_of, register_part
from .norm import RowNorm
from .runner import Eager, Planned, stream_tensor


class PreNormResidual(Block):
    """x += mixer(norm(x)); x += ffn(norm(x))
    (MisterTK/gibbs arch/families/lfm2.json5:76-89)."""
    ROLES = (("mixer_norm", "norm"), ("mixer", "mixer"), ("ffn_norm", "norm"), ("ffn", "feed_forward"))
    OPTIONAL_ROLES = ("ffn_norm", "ffn")       # a layer may have no feed-forward (then neither its norm)

    # A mixer or feed-forward that says ``fuses_norm`` hands its input straight to a product
    # (``parts.linear.Linear``), which may then run the norm itself.

    def forward(self, x, step, caches):
        h = self.mixer_norm.lazy(x) if getattr(self.mixer, "fuses_norm", False) else self.mixer_norm.forward(x)
        self.mixer.forward(h, x, step, self.caches_of("mixer", caches))
        if "ffn" not in self.parts:
            return
        h = self.ffn_norm.lazy(x) if getattr(self.ffn, "fuses_norm", False) else self.ffn_norm.forward(x)
        self.ffn.forward(h, x, step)

    def plan_ops(self, plan, caches):
        h = self._norm_ops(plan, self.mixer_norm, self.mixer)
        plan_ops_of(self.mixer)(plan, h, self.caches_of("mixer", caches))
        if "ffn" not in self.parts:
            return
        h = self._norm_ops(plan, self.ffn_norm, self.ffn)
        plan_ops_of(self.ffn)(plan, h)

    @staticmethod
    def _norm_ops(plan, norm, consumer):
        if getattr(consumer, "fuses_norm", False) and getattr(norm, "lazy", None) is not None:
            try:
                return plan_ops_of(norm)(plan, lazy=True)
            except TypeError:            # a norm from outside whose plan_ops knows no such option
                pass
        return plan_ops_of(norm)(plan)


register_part("block", "prenorm_residual", PreNormResidual)


class SandwichResidual(Block):
    """A norm in front of AND behind every sublayer:

        x += post_norm(mixer(norm(x)));  x += post_norm(ffn(norm(x)));  token_input(x)

    The feed-forward (with its two norms) and the token input are optional.  Sublayers write
    their output for the norm behind them (``parts.runner.BranchPart``); the norms behind are
    ``RowNorm`` kinds, whose ``add_normed`` adds into the stream."""
    ROLES = (("mixer_norm", "norm"), ("mixer", "mixer"), ("mixer_post_norm", "norm"), ("ffn_norm", "norm"),
             ("ffn", "feed_forward"), ("ffn_post_norm", "norm"), ("token_input", "token_input"))
    OPTIONAL_ROLES = ("ffn_norm", "ffn", "ffn_post_norm", "token_input")

    def __init__(self, parts, rt, params=None):
        super().__init__(parts, rt, params)
        have = set(self.parts)
        if len(have & {"ffn_norm", "ffn", "ffn_post_norm"}) not in (0, 3):
            raise ValueError("a feed-forward comes with the norm in front of it and the norm behind it")
        for role in ("mixer", "ffn"):
            if role in have and not getattr(self.parts[role], "writes_branch", False):
                raise ValueError(f"the {role} of this arrangement must be able to write its output for the norm "
                                 f"behind it; {type(self.parts[role]).__name__} only adds into the stream")
        for role in ("mixer_post_norm", "ffn_post_norm"):
            if role in have and not hasattr(self.parts[role], "add_normed"):
                raise ValueError(f"the {role} must be a norm that can add into the stream (a RowNorm kind)")

    def _run(self, rn, x, caches, h_of):
        hidden = x.shape[1]
        y = rn.buffer("branch", hidden, torch.float32)
        # a token input reads the stream through a product: in bfloat16 the norm that completes the
        # stream also leaves the rows in that type
        copy = None
        if "token_input" in self.parts and self.rt.dtype == torch.bfloat16:
            copy = rn.buffer("stream_rows", hidden, torch.bfloat16)
        has_ffn = "ffn" in self.parts
        self.mixer.run(rn, h_of(self.mixer_norm), y, self.caches_of("mixer", caches))
        # the norm in front of the feed-forward is taken in the kernel that completes the stream behind the mixer
        fuse = has_ffn and isinstance(self.ffn_norm, RowNorm) and self.ffn_norm.dim == hidden
        h = self.mixer_post_norm.add_normed(rn, x, y, None if has_ffn else copy, self.ffn_norm if fuse else None)
        if has_ffn:
            self.ffn.run(rn, h if fuse else h_of(self.ffn_norm), y, None)
            self.ffn_post_norm.add_normed(rn, x, y, copy)
        if "token_input" in self.parts:
            self.token_input.run(rn, x, copy)

    def forward(self, x, step, caches):
        rn, xt = Eager(self.rt, step), stream_tensor(x)
        self._run(rn, xt, caches, lambda norm: norm.forward(xt))

    def plan_ops(self, plan, caches):
        self._run(Planned(plan), plan.residual, caches, lambda norm: plan_ops_of(norm)(plan))


register_part("block", "sandwich_residual", SandwichResidual)
