"""A state-space layer with a scalar decay per head (Mamba-2, state-space duality)."""

from __future__ import annotations

from dataclasses import dataclass

import torch

from ..cache.manager import StateNeed
from ..csrc import ops
from .base import MIXERS, Runtime, TensorReq, linear, tensor_bytes


@dataclass(frozen=True)
class StateSpaceDualSpec:
    """``num_heads`` heads of ``value_dim`` channels (``inner = num_heads * value_dim``), a state of
    ``state_dim`` rows per head, ``num_groups`` groups of heads that share their B and C, a convolution of
    ``conv_taps`` taps on x, B and C, an output norm in ``norm_groups`` equal parts.  The ``*_name`` fields are
    the tensors' names after the part's prefix."""

    hidden_size: int
    num_heads: int
    value_dim: int
    state_dim: int
    num_groups: int
    conv_taps: int
    norm_groups: int
    norm_eps: float
    in_name: str = "in"
    conv_name: str = "conv"
    conv_bias_name: str = "conv.b"
    dt_bias_name: str = "dt_bias"
    decay_log_name: str = "A_log"
    skip_name: str = "D"
    norm_name: str = "norm"
    o_name: str = "o"
    kind: str = "ssd"


@MIXERS.register("ssd")
class StateSpaceDual:
    """The input projection is laid out ``[z: inner | x: inner | B: groups state | C: groups state | dt: heads]``.
    x, B and C pass a causal convolution per channel with a bias, then silu; ``dt = softplus(dt + dt_bias)``;
    per head (with B and C of its group), ``S`` being ``[state, value_dim]``:

        ``S_t = exp(-exp(A_log) dt) S_(t-1) + dt B_t x_t^T``,   ``y_t = S_t^T C_t + D x_t``;

    ``y`` (heads concatenated) is multiplied by ``silu(z)``, RMS-normed in ``norm_groups`` equal parts with a
    weight per channel, and projected out.

    The request's state is two float32 records: the matrix per head and the convolution's last
    ``conv_taps - 1`` inputs.  The convolution's sums, ``dt``, the decay, the state, the recurrence and the
    norm are float32 in every dtype (``csrc/short_conv.cu``, ``csrc/state_mixers.cu``; the recurrence is gated
    linear attention's kernel with B as the key, C as the query and ``dt x`` as the value).

    :meth:`branch` writes the rows in front of the output projection into a buffer of the caller's, times
    a factor, so that a mixer made of several can run one output product over all of them.
    """

    GRAPH_SAFE = True

    def __init__(self, spec: StateSpaceDualSpec, prefix: str, tensors: dict[str, torch.Tensor], rt: Runtime):
        if spec.num_heads % spec.num_groups:
            raise ValueError(f"{spec.num_heads} heads are not a multiple of {spec.num_groups} groups")
        if spec.state_dim > 256:
            raise ValueError(f"a state of {spec.state_dim} rows is beyond the recurrence kernel's limit of 256")
        if not 1 <= spec.conv_taps <= 8:
            raise ValueError(f"a convolution of {spec.conv_taps} taps is not taken (1 to 8)")
        self.spec = spec
        self.rt = rt
        self.inner = spec.num_heads * spec.value_dim
        if self.inner % spec.norm_groups:
            raise ValueError(f"{self.inner} channels do not split into {spec.norm_groups} equal groups")
        self.conv_channels = self.inner + 2 * spec.num_groups * spec.state_dim
        t = lambda name: tensors[prefix + name]
        self.w_in = t(spec.in_name)
        self.z_off, self.xbc_off, self.dt_off = 0, self.inner, self.inner + self.conv_channels
        self.taps = t(spec.conv_name).float().contiguous()
        self.conv_bias = t(spec.conv_bias_name).contiguous()
        self.dt_bias = t(spec.dt_bias_name).contiguous()
        self.a_log = t(spec.decay_log_name).contiguous()
        self.skip = t(spec.skip_name).contiguous()
        self.norm_w = t(spec.norm_name).contiguous()
        self.w_o = t(spec.o_name)
        self.out_width = self.inner

    @staticmethod
    def expected_tensors(spec: StateSpaceDualSpec, prefix: str) -> dict[str, TensorReq]:
        w, inner = spec.hidden_size, spec.num_heads * spec.value_dim
        ch = inner + 2 * spec.num_groups * spec.state_dim
        return {
            prefix + spec.in_name: TensorReq((inner + ch + spec.num_heads, w)),
            prefix + spec.conv_name: TensorReq((ch, spec.conv_taps), role="bias"),
            prefix + spec.conv_bias_name: TensorReq((ch,), role="bias"),
            prefix + spec.dt_bias_name: TensorReq((spec.num_heads,), role="bias"),
            prefix + spec.decay_log_name: TensorReq((spec.num_heads,), role="bias"),
            prefix + spec.skip_name: TensorReq((spec.num_heads,), role="vector"),
            prefix + spec.norm_name: TensorReq((inner,), role="vector"),
            prefix + spec.o_name: TensorReq((w, inner)),
        }

    def cache_need(self) -> dict:
        s = self.spec
        need = {"state": StateNeed((s.num_heads, s.state_dim, s.value_dim), "float32")}
        if s.conv_taps > 1:
            need["conv"] = StateNeed((s.conv_taps - 1, self.conv_channels), "float32")
        return need

    def weight_bytes(self) -> int:
        return tensor_bytes(self.w_in, self.taps, self.conv_bias, self.dt_bias, self.a_log, self.skip, self.norm_w,
                            self.w_o)

    def branch(self, h, step, cache_view, out: torch.Tensor | None = None, out_scale: float = 1.0) -> torch.Tensor:
        """The rows that the output projection reads, times ``out_scale``, into ``out`` (``[tokens, inner]``,
        rows of any stride) or a new tensor."""
        spec = self.spec
        proj = linear(h, self.w_in, err=step.err)
        tail = cache_view["conv"].records if "conv" in cache_view else None
        xbc = ops.short_conv(proj, self.taps, tail, step, dtype=h.dtype, in_off=self.xbc_off,
                             channels=self.conv_channels, bias=self.conv_bias, silu=True, out_f32=True)
        prep = ops.ssd_prepare(xbc, proj, self.dt_off, self.dt_bias, self.a_log, dtype=h.dtype, heads=spec.num_heads,
                               groups=spec.num_groups, state=spec.state_dim, value_dim=spec.value_dim)
        o = ops.gla_scan(prep, cache_view["state"].records, step.req_q_start, step.req_q_len, step.req_slot, step.err)
        return ops.ssd_out(o, xbc, proj, self.z_off, self.skip, self.norm_w, spec.norm_groups, spec.norm_eps, h.dtype,
                           out=out, out_scale=out_scale)

    def forward(self, h, step, cache_view):
        return linear(self.branch(h, step, cache_view), self.w_o, err=step.err)
