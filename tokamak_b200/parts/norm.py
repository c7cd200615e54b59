"""RMSNorm, fused with the residual sum that precedes it."""

from __future__ import annotations

from dataclasses import dataclass

import torch

from ..csrc import ops
from .base import NORMS, HyperBranch, NormedBranch, OwedNorm, Runtime, TensorReq


@dataclass(frozen=True)
class RMSNormSpec:
    dim: int
    eps: float
    kind: str = "rmsnorm"


@NORMS.register("rmsnorm")
class RMSNorm:
    """``weight * x * rsqrt(mean(x^2) + eps)`` with 32-bit statistics
    (src/tokamak/model/layers.py:16-33).

    The residual stream is float32; ``add_norm`` first adds the pending branch
    output to it (a 32-bit sum) and then normalises the sum, in one kernel.
    """

    GRAPH_SAFE = True

    def __init__(self, spec: RMSNormSpec, name: str, tensors: dict[str, torch.Tensor], rt: Runtime):
        self.spec = spec
        self.rt = rt
        self.weight = tensors[name]

    @staticmethod
    def expected_tensors(spec: RMSNormSpec, name: str) -> dict[str, TensorReq]:
        return {name: TensorReq((spec.dim,), role="vector")}

    def weight_bytes(self) -> int:
        return self.weight.numel() * self.weight.element_size()

    def owed_norm_params(self) -> tuple[torch.Tensor, float] | None:
        """Weight and eps for a product kernel that prepares this norm's input itself."""
        return self.weight, self.spec.eps

    def add_norm(self, resid: torch.Tensor, delta, rows: torch.Tensor | None = None):
        """Normalised rows in the engine's dtype.

        Without ``rows`` the sum ``resid + delta`` is written back to ``resid`` and
        every row is normalised.  With ``rows`` only those rows are summed and
        normalised and ``resid`` is left as it is.  ``delta`` may be an
        :class:`OwedNorm`: the branch has been added to ``resid`` already; if it was
        prepared for this norm it is handed on as it is (its consumer pays the scale).
        A :class:`NormedBranch` is normalised, scaled and added by the same kernel.
        """
        if isinstance(delta, NormedBranch):
            n = rows.numel() if rows is not None else resid.shape[0]
            out = torch.empty((n, self.spec.dim), dtype=self.rt.dtype, device=resid.device)
            ops.branch_norm_add(resid, delta.x, delta.weight, delta.layer_scale, delta.eps, self.weight, out,
                                self.spec.eps, rows, branch_groups=delta.groups)
            return out
        if isinstance(delta, OwedNorm):
            if delta.norm is self:
                return delta if rows is None else delta.rows(rows)
            delta = None
        n = rows.numel() if rows is not None else resid.shape[0]
        out = torch.empty((n, self.spec.dim), dtype=self.rt.dtype, device=resid.device)
        ops.add_rmsnorm(resid, delta, self.weight, out, self.spec.eps, rows)
        return out


@dataclass(frozen=True)
class OffsetRMSNormSpec:
    """An RMS norm whose weight is stored around zero: the factor is ``1 + w``."""

    dim: int
    eps: float
    kind: str = "rmsnorm_offset"


@NORMS.register("rmsnorm_offset")
class OffsetRMSNorm(RMSNorm):
    """``(1 + w) * x * rsqrt(mean(x^2) + eps)``: the stored tensor is the weight's distance from one.
    ``1 + w`` is formed once, in float32, when the part is built; everything else is :class:`RMSNorm`."""

    def __init__(self, spec: OffsetRMSNormSpec, name: str, tensors: dict[str, torch.Tensor], rt: Runtime):
        self.spec = spec
        self.rt = rt
        self.weight = (1.0 + tensors[name].float()).contiguous()

    @staticmethod
    def expected_tensors(spec: OffsetRMSNormSpec, name: str) -> dict[str, TensorReq]:
        return {name: TensorReq((spec.dim,), role="bias")}


@dataclass(frozen=True)
class CastNormSpec:
    """No normalisation: the seat of a norm in front of a sublayer that reads the residual stream itself."""

    dim: int
    kind: str = "cast"


@NORMS.register("cast")
class CastNorm:
    """Joins the pending branch to the float32 residual stream and hands the rows on unnormalised,
    rounded to the engine's dtype (the sublayer's products read that type).  It has no tensor."""

    GRAPH_SAFE = True

    def __init__(self, spec: CastNormSpec, name: str, tensors: dict[str, torch.Tensor], rt: Runtime):
        self.spec = spec
        self.rt = rt

    @staticmethod
    def expected_tensors(spec: CastNormSpec, name: str) -> dict[str, TensorReq]:
        return {}

    def weight_bytes(self) -> int:
        return 0

    def join(self, resid: torch.Tensor, delta) -> None:
        """Only the first half: the pending branch joins the float32 stream, nothing is handed on (for a
        block whose sublayer reads the stream through a kernel of its own)."""
        if isinstance(delta, NormedBranch):
            ops.branch_norm_add(resid, delta.x, delta.weight, delta.layer_scale, delta.eps, None, None, 0.0, None,
                                branch_groups=delta.groups)
        elif delta is not None and not isinstance(delta, OwedNorm):
            from .base import sum_parts
            resid.add_(sum_parts(delta, torch.float32))

    def add_norm(self, resid: torch.Tensor, delta, rows: torch.Tensor | None = None):
        if isinstance(delta, OwedNorm):
            delta = None        # its branch is in the stream already
        if isinstance(delta, NormedBranch):
            n = rows.numel() if rows is not None else resid.shape[0]
            out = torch.empty((n, self.spec.dim), dtype=self.rt.dtype, device=resid.device)
            ops.branch_norm_add(resid, delta.x, delta.weight, delta.layer_scale, delta.eps, None, out, 0.0, rows,
                                branch_groups=delta.groups)
            return out
        if delta is not None:
            from .base import sum_parts
            delta = sum_parts(delta, torch.float32)
            if rows is None:
                resid.add_(delta)
            else:
                return (resid.index_select(0, rows.long()) + delta.index_select(0, rows.long())).to(self.rt.dtype)
        x = resid if rows is None else resid.index_select(0, rows.long())
        return x.to(self.rt.dtype, copy=True)


@dataclass(frozen=True)
class GroupRMSNormSpec:
    """An RMS norm in ``groups`` equal consecutive parts of the row: every part is divided by its own
    root mean square, the whole is multiplied by one weight per channel."""

    dim: int
    eps: float
    groups: int
    kind: str = "rmsnorm_groups"


@NORMS.register("rmsnorm_groups")
class GroupRMSNorm:
    """``w * x / sqrt(mean_part(x^2) + eps)`` with the mean taken over the part of the row that the channel
    lies in; statistics are float32.  Behind a sublayer it rides in the :class:`NormedBranch` (``groups``);
    in front of one, or as a model's last norm, it joins the pending branch and normalises in one kernel."""

    GRAPH_SAFE = True

    def __init__(self, spec: GroupRMSNormSpec, name: str, tensors: dict[str, torch.Tensor], rt: Runtime):
        if spec.groups < 1 or spec.dim % spec.groups:
            raise ValueError(f"a row of {spec.dim} does not split into {spec.groups} equal groups")
        self.spec = spec
        self.rt = rt
        self.weight = tensors[name]
        self.groups = spec.groups

    @staticmethod
    def expected_tensors(spec: GroupRMSNormSpec, name: str) -> dict[str, TensorReq]:
        return {name: TensorReq((spec.dim,), role="vector")}

    def weight_bytes(self) -> int:
        return self.weight.numel() * self.weight.element_size()

    def owed_norm_params(self) -> tuple[torch.Tensor, float]:
        return self.weight, self.spec.eps

    def add_norm(self, resid: torch.Tensor, delta, rows: torch.Tensor | None = None):
        if isinstance(delta, OwedNorm):
            delta = None        # its branch is in the stream already
        n = rows.numel() if rows is not None else resid.shape[0]
        out = torch.empty((n, self.spec.dim), dtype=self.rt.dtype, device=resid.device)
        if isinstance(delta, NormedBranch):
            ops.branch_norm_add(resid, delta.x, delta.weight, delta.layer_scale, delta.eps, self.weight, out,
                                self.spec.eps, rows, branch_groups=delta.groups, next_groups=self.spec.groups)
            return out
        if delta is not None:
            from .base import sum_parts
            if rows is not None:
                raise ValueError("a plain branch cannot join selected rows only")
            resid.add_(sum_parts(delta, torch.float32))
        ops.branch_norm_add(resid, None, None, None, 0.0, self.weight, out, self.spec.eps, rows,
                            next_groups=self.spec.groups)
        return out


@dataclass(frozen=True)
class LayerNormSpec:
    """A layer norm with a weight and, with ``bias``, a bias (the tensor's name with ``bias_suffix``)."""

    dim: int
    eps: float
    bias: bool = True
    bias_suffix: str = ".b"
    kind: str = "layernorm"


@NORMS.register("layernorm")
class LayerNorm:
    """``(x - mean) / sqrt(var + eps) * w + b`` with the variance the mean of the squared deviations; statistics
    are float32 and taken in two passes over the row.

    The residual stream it reads may be kept in several float32 copies ``[S, tokens, width]`` (a 2-D stream is
    one copy): ``add_norm`` writes the pending sublayer output to all copies (a
    :class:`~tokamak_b200.parts.base.HyperBranch`; a plain tensor joins every copy as it is), reads the row
    ``sum_s read[s] x_s`` (``read=None``: the sum of the copies) and normalises it, in one kernel
    (``csrc/hyper.cu``)."""

    GRAPH_SAFE = True

    def __init__(self, spec: LayerNormSpec, name: str, tensors: dict[str, torch.Tensor], rt: Runtime):
        self.spec = spec
        self.rt = rt
        self.weight = tensors[name]
        self.bias = tensors[name + spec.bias_suffix] if spec.bias else None

    @staticmethod
    def expected_tensors(spec: LayerNormSpec, name: str) -> dict[str, TensorReq]:
        out = {name: TensorReq((spec.dim,), role="vector")}
        if spec.bias:
            out[name + spec.bias_suffix] = TensorReq((spec.dim,), role="bias")
        return out

    def weight_bytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in (self.weight, self.bias) if t is not None)

    def add_norm(self, resid: torch.Tensor, delta, rows: torch.Tensor | None = None, read: torch.Tensor | None = None):
        """Normalised rows in the engine's dtype.  Without ``rows`` the pending branch is written to the stream
        and every row is normalised; with ``rows`` only those rows are, and the stream is left as it is."""
        streams = resid if resid.dim() == 3 else resid.unsqueeze(0)
        if isinstance(delta, OwedNorm):
            delta = None        # its branch is in the stream already
        if isinstance(delta, NormedBranch):
            raise ValueError("a layer norm does not join a branch that is normalised on the way out")
        if delta is not None and not isinstance(delta, HyperBranch):
            delta = HyperBranch(delta)
        branch = delta.x if delta is not None else None
        out, _ = ops.hyper_mix_norm(streams, branch, mix=delta.mix if delta else None,
                                    write=delta.write if delta else None, read=read,
                                    mult=delta.mult if delta else 1.0, norm_w=self.weight, norm_b=self.bias,
                                    eps=self.spec.eps, dtype=self.rt.dtype, rows=rows)
        return out
