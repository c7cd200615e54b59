"""Linear attention whose forget gate also decides what is written (HGRN2): a matrix-valued state per
request and head, with the complement of the gate in the key's place."""

from __future__ import annotations

from dataclasses import dataclass

import torch

from ..cache.manager import StateNeed
from ..csrc import ops
from .base import MIXERS, Runtime, TensorReq, linear, tensor_bytes


@dataclass(frozen=True)
class Hgrn2Spec:
    """``num_heads`` heads with ``key_dim`` gate/query channels and ``value_dim`` value channels each; the
    ``*_name`` fields are the tensors' names after the part's prefix."""

    hidden_size: int
    num_heads: int
    key_dim: int
    value_dim: int
    norm_eps: float
    q_name: str = "q"
    f_name: str = "f"
    f_bias_name: str = "f.b"
    lower_name: str = "lower"
    v_name: str = "v"
    norm_name: str = "norm"
    o_name: str = "o"
    kind: str = "hgrn2"


@MIXERS.register("hgrn2")
class Hgrn2:
    """Per head, with ``S`` the ``[key_dim, value_dim]`` state: ``S_t = diag(f_t) S_(t-1) + (1 - f_t) v_t^T``,
    ``o_t = S_t^T q_t``, where ``q = silu(W_q h)``, ``v = W_v h`` and the forget gate per head and channel is
    ``f = l + (1 - l) sigmoid(W_f h + b)`` with a learned lower bound ``l``.  Every head's ``o`` is RMS-normed
    over ``value_dim`` (one weight vector for all heads), the heads are concatenated and projected out.

    The state is a float32 record per request (:class:`~tokamak_b200.cache.manager.StateNeed`), cleared
    when the slot is handed out.  The three input projections are one stacked operand; gate, state,
    recurrence and norm are float32 in every dtype (``csrc/state_mixers.cu`` lays the inputs out, the
    recurrence and the output stage are gated linear attention's kernels).
    """

    GRAPH_SAFE = True

    def __init__(self, spec: Hgrn2Spec, prefix: str, tensors: dict[str, torch.Tensor], rt: Runtime):
        if spec.key_dim > 256:
            raise ValueError(f"key_dim {spec.key_dim} is beyond the recurrence kernel's limit of 256")
        self.spec = spec
        self.rt = rt
        hk = spec.num_heads * spec.key_dim
        t = lambda name: tensors[prefix + name]
        self.w_in = torch.cat([t(spec.q_name), t(spec.f_name), t(spec.v_name)], dim=0).contiguous()
        self.q_off, self.f_off, self.v_off = 0, hk, 2 * hk
        self.f_bias = t(spec.f_bias_name).contiguous()
        self.lower = t(spec.lower_name).contiguous()
        self.norm_w = t(spec.norm_name)
        self.w_o = t(spec.o_name)

    @staticmethod
    def expected_tensors(spec: Hgrn2Spec, prefix: str) -> dict[str, TensorReq]:
        w, hk, hv = spec.hidden_size, spec.num_heads * spec.key_dim, spec.num_heads * spec.value_dim
        return {
            prefix + spec.q_name: TensorReq((hk, w)),
            prefix + spec.f_name: TensorReq((hk, w)),
            prefix + spec.f_bias_name: TensorReq((hk,), role="bias"),
            prefix + spec.lower_name: TensorReq((hk,), role="fraction"),
            prefix + spec.v_name: TensorReq((hv, w)),
            prefix + spec.norm_name: TensorReq((spec.value_dim,), role="vector"),
            prefix + spec.o_name: TensorReq((w, hv)),
        }

    def cache_need(self) -> StateNeed:
        return StateNeed((self.spec.num_heads, self.spec.key_dim, self.spec.value_dim), "float32")

    def weight_bytes(self) -> int:
        return tensor_bytes(self.w_in, self.f_bias, self.lower, self.norm_w, self.w_o)

    def forward(self, h, step, cache_view):
        spec = self.spec
        proj = linear(h, self.w_in, err=step.err)
        prep = ops.hgrn2_prepare(proj, self.f_bias, self.lower, dtype=h.dtype, q_off=self.q_off, f_off=self.f_off,
                                 v_off=self.v_off, heads=spec.num_heads, key_dim=spec.key_dim, value_dim=spec.value_dim)
        o = ops.gla_scan(prep, cache_view.records, step.req_q_start, step.req_q_len, step.req_slot, step.err)
        y = ops.gla_out(o, None, 0, self.norm_w, spec.norm_eps, h.dtype)
        return linear(y, self.w_o, err=step.err)
