"""Two mixers side by side that read the same input; their outputs are added with a factor each."""

from __future__ import annotations

from dataclasses import dataclass

import torch

from .base import MIXERS, Runtime, TensorReq, graph_safe, linear, tensor_bytes, weight_bytes


@dataclass(frozen=True)
class ParallelMixerSpec:
    """``left`` and ``right`` are mixer specs; their tensors lie under ``left_prefix`` / ``right_prefix`` behind the
    part's own prefix; the result is ``left_scale * left(h) + right_scale * right(h)``."""

    left: object
    right: object
    left_scale: float
    right_scale: float
    left_prefix: str = "left."
    right_prefix: str = "right."
    kind: str = "parallel"


@MIXERS.register("parallel")
class ParallelMixer:
    """Both halves must offer ``branch(h, step, cache_view, out, out_scale)`` (the rows in front of their
    output projection, times a factor, written into a column range of a buffer), ``out_width`` and ``w_o``:
    the two output projections are stacked along their inputs once, so that

        ``left_scale * W_l y_l + right_scale * W_r y_r = [W_l | W_r] [left_scale y_l ; right_scale y_r]``

    is one product.  The factors are applied in float32 before the rows are rounded to the engine's dtype.
    The cache need is the dictionary of the halves' needs.

    Halves that declare ``TAKES_PROJ = True`` keep their stacked input projection in ``w_in`` and take
    ``branch(..., proj=, proj_off=)``: the two input projections are then stacked too and run as one product of
    the shared input, each half reading its columns of the result from ``proj_off`` on.
    """

    def __init__(self, spec: ParallelMixerSpec, prefix: str, tensors: dict[str, torch.Tensor], rt: Runtime):
        self.spec = spec
        self.rt = rt
        self.left = MIXERS.get(spec.left.kind)(spec.left, prefix + spec.left_prefix, tensors, rt)
        self.right = MIXERS.get(spec.right.kind)(spec.right, prefix + spec.right_prefix, tensors, rt)
        for half in (self.left, self.right):
            if not (hasattr(half, "branch") and hasattr(half, "out_width") and hasattr(half, "w_o")):
                raise ValueError(f"a {type(half).__name__} cannot be half of a parallel mixer: it has no branch()")
        self.w_o = torch.cat([self.left.w_o, self.right.w_o], dim=1).contiguous()
        self.w_in = None
        if all(getattr(half, "TAKES_PROJ", False) for half in (self.left, self.right)):
            n_left = self.left.w_in.shape[0]
            self.w_in = torch.cat([self.left.w_in, self.right.w_in], dim=0).contiguous()
            self.left.w_in, self.right.w_in = self.w_in[:n_left], self.w_in[n_left:]      # one copy in memory
        self.prefill_heads = getattr(self.left, "prefill_heads", None) or getattr(self.right, "prefill_heads", None)

    @staticmethod
    def expected_tensors(spec: ParallelMixerSpec, prefix: str) -> dict[str, TensorReq]:
        out = dict(MIXERS.get(spec.left.kind).expected_tensors(spec.left, prefix + spec.left_prefix))
        out.update(MIXERS.get(spec.right.kind).expected_tensors(spec.right, prefix + spec.right_prefix))
        return out

    def cache_need(self) -> dict:
        return {"left": self.left.cache_need(), "right": self.right.cache_need()}

    def GRAPH_SAFE(self) -> bool:
        return graph_safe(self.left, self.right)

    def weight_bytes(self) -> int:
        return weight_bytes(self.left, self.right)

    def forward(self, h, step, cache_view):
        n, wl, wr = h.shape[0], self.left.out_width, self.right.out_width
        y = torch.empty((n, wl + wr), dtype=h.dtype, device=h.device)
        if self.w_in is not None:
            proj = linear(h, self.w_in, err=step.err)
            self.left.branch(h, step, cache_view["left"], out=y[:, :wl], out_scale=self.spec.left_scale, proj=proj)
            self.right.branch(h, step, cache_view["right"], out=y[:, wl:], out_scale=self.spec.right_scale, proj=proj,
                              proj_off=self.left.w_in.shape[0])
        else:
            self.left.branch(h, step, cache_view["left"], out=y[:, :wl], out_scale=self.spec.left_scale)
            self.right.branch(h, step, cache_view["right"], out=y[:, wl:], out_scale=self.spec.right_scale)
        return linear(y, self.w_o, err=step.err)
