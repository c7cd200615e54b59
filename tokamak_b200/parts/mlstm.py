"""A matrix memory with exponential input and forget gates (the mLSTM of xLSTM), held stable by a running
maximum of the gates' logarithms."""

from __future__ import annotations

from dataclasses import dataclass

import torch

from ..cache.manager import StateNeed
from ..csrc import ops
from .base import MIXERS, Runtime, TensorReq, linear, tensor_bytes


@dataclass(frozen=True)
class MlstmSpec:
    """``num_heads`` heads with ``key_dim`` query/key channels and ``value_dim`` value channels; ``gate_cap``
    bounds the gates' pre-activations (``cap * tanh(z / cap)``); ``denominator_eps`` is added to the
    normaliser; the ``*_name`` fields are the tensors' names after the part's prefix."""

    hidden_size: int
    num_heads: int
    key_dim: int
    value_dim: int
    gate_cap: float
    norm_eps: float
    denominator_eps: float = 1e-6
    q_name: str = "q"
    k_name: str = "k"
    v_name: str = "v"
    gate_name: str = "g"
    i_name: str = "i"
    i_bias_name: str = "i.b"
    f_name: str = "f"
    f_bias_name: str = "f.b"
    norm_name: str = "norm"
    o_name: str = "o"
    kind: str = "mlstm"


@MIXERS.register("mlstm")
class Mlstm:
    """Per head, with the logarithms ``i = cap tanh((W_i h + b_i) / cap)`` of the input gate and
    ``f = logsigmoid(cap tanh((W_f h + b_f) / cap))`` of the forget gate and a running maximum
    ``m_t = max(f + m_(t-1), i)`` that starts at zero:

        ``S_t = exp(f + m_(t-1) - m_t) S_(t-1) + exp(i - m_t) k v^T``,  ``n_t`` likewise with ``k`` alone,
        ``o = S_t^T q / (max(|n_t . q|, exp(-m_t)) + 1e-6)``,

    ``q = W_q h / sqrt(key_dim)``, ``k = W_k h``, ``v = W_v h``.  Every head's ``o`` is scaled to unit root mean
    square; the concatenated heads are multiplied by a weight per channel and by ``sigmoid(W_g h)`` and
    projected out.

    The request's state is three float32 records: the matrix with the normaliser as one more value column
    (``[heads, key_dim, value_dim + 1]``: the values get a column of ones, so ``n . q`` is the last column of
    the read-out) and the running maximum ``[heads]``.  Gates, maximum, state, recurrence and norm are
    float32 in every dtype; the recurrence is gated linear attention's kernel.
    """

    GRAPH_SAFE = True

    def __init__(self, spec: MlstmSpec, prefix: str, tensors: dict[str, torch.Tensor], rt: Runtime):
        if spec.key_dim > 256:
            raise ValueError(f"key_dim {spec.key_dim} is beyond the recurrence kernel's limit of 256")
        if not spec.gate_cap > 0 or spec.denominator_eps != 1e-6:
            raise ValueError("gate_cap must be > 0 and the normaliser's eps is the kernel's 1e-6")
        self.spec = spec
        self.rt = rt
        hk, hv, hh = spec.num_heads * spec.key_dim, spec.num_heads * spec.value_dim, spec.num_heads
        t = lambda name: tensors[prefix + name]
        self.w_in = torch.cat([t(spec.q_name), t(spec.k_name), t(spec.v_name), t(spec.gate_name), t(spec.i_name),
                               t(spec.f_name)], dim=0).contiguous()
        self.q_off, self.k_off, self.v_off = 0, hk, 2 * hk
        self.g_off, self.i_off, self.f_off = 2 * hk + hv, 2 * hk + 2 * hv, 2 * hk + 2 * hv + hh
        self.i_bias = t(spec.i_bias_name).contiguous()
        self.f_bias = t(spec.f_bias_name).contiguous()
        self.norm_w = t(spec.norm_name).contiguous()
        self.w_o = t(spec.o_name)

    @staticmethod
    def expected_tensors(spec: MlstmSpec, prefix: str) -> dict[str, TensorReq]:
        w, hk, hv, hh = spec.hidden_size, spec.num_heads * spec.key_dim, spec.num_heads * spec.value_dim, spec.num_heads
        return {
            prefix + spec.q_name: TensorReq((hk, w)),
            prefix + spec.k_name: TensorReq((hk, w)),
            prefix + spec.v_name: TensorReq((hv, w)),
            prefix + spec.gate_name: TensorReq((hv, w)),
            prefix + spec.o_name: TensorReq((w, hv)),
            prefix + spec.norm_name: TensorReq((hv,), role="vector"),
            prefix + spec.i_name: TensorReq((hh, w)),
            prefix + spec.i_bias_name: TensorReq((hh,), role="bias"),
            prefix + spec.f_name: TensorReq((hh, w)),
            prefix + spec.f_bias_name: TensorReq((hh,), role="bias"),
        }

    def cache_need(self) -> dict:
        s = self.spec
        return {"memory": StateNeed((s.num_heads, s.key_dim, s.value_dim + 1), "float32"),
                "maximum": StateNeed((s.num_heads,), "float32")}

    def weight_bytes(self) -> int:
        return tensor_bytes(self.w_in, self.i_bias, self.f_bias, self.norm_w, self.w_o)

    def forward(self, h, step, cache_view):
        spec = self.spec
        proj = linear(h, self.w_in, err=step.err)
        prep, gates = ops.mlstm_prepare(proj, self.i_bias, self.f_bias, cache_view["maximum"].records, step,
                                        dtype=h.dtype, q_off=self.q_off, k_off=self.k_off, v_off=self.v_off,
                                        i_off=self.i_off, f_off=self.f_off, heads=spec.num_heads, key_dim=spec.key_dim,
                                        value_dim=spec.value_dim, cap=spec.gate_cap, q_scale=spec.key_dim ** -0.5)
        o = ops.gla_scan(prep, cache_view["memory"].records, step.req_q_start, step.req_q_len, step.req_slot, step.err)
        y = ops.mlstm_out(o, gates, proj, self.g_off, self.norm_w, spec.norm_eps, h.dtype)
        return linear(y, self.w_o, err=step.err)
