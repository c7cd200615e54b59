"""Retention: linear attention with a fixed decay per head, a mixer whose memory is a matrix per request and head."""

from __future__ import annotations

from dataclasses import dataclass

import torch

from ..cache.manager import StateNeed
from ..csrc import ops
from .base import MIXERS, POSITIONS, Runtime, TensorReq, graph_safe, linear, tensor_bytes


@dataclass(frozen=True)
class RetentionSpec:
    """``num_heads`` heads of ``key_dim`` query/key and ``value_dim`` value channels; ``decay`` holds one number in
    (0, 1] per head; ``position`` is a position spec whose part rotates q and k (halves or neighbouring pairs) or
    ``none``; ``k_scale`` multiplies the rotated keys (``None``: ``key_dim ** -0.5``); ``norm_eps`` is the eps of the
    weightless RMS norm of every head's output.  The ``*_name`` fields are the tensors' names after the part's
    prefix."""

    hidden_size: int
    num_heads: int
    key_dim: int
    value_dim: int
    decay: tuple
    position: object
    norm_eps: float
    k_scale: float | None = None
    q_name: str = "q"
    k_name: str = "k"
    v_name: str = "v"
    gate_name: str = "g"
    o_name: str = "o"
    kind: str = "retention"


@MIXERS.register("retention")
class Retention:
    """``S_t = decay_h S_(t-1) + k_t v_t^T``, ``o_t = S_t^T q_t`` per head, without softmax or denominator; q and k are
    rotated by the token's position, k is then scaled; every head's ``o`` is divided by its root mean square,
    the heads are concatenated, multiplied by ``silu(W_g h)`` and projected out.

    The state ``[heads, key_dim, value_dim]`` is a float32 record in the request's slot of the cache
    (:class:`~tokamak_b200.cache.manager.StateNeed`): zero when the slot is handed out, read at the start of a
    step's portion and stored at its end.  The four input projections are one stacked operand; a step is
    that product, the kernel that lays out the recurrence's float32 inputs (rotation, scale, decays:
    ``csrc/state_mixers.cu``), the recurrence and the output stage of gated linear attention (``csrc/gla.cu``)
    and the output product.  Angles, rotation, decays, state, recurrence and norm are float32 in every dtype.

    :meth:`branch` writes the rows in front of the output projection into a buffer of the caller's, times a
    factor (see :class:`~tokamak_b200.parts.parallel.ParallelMixer`)."""

    def __init__(self, spec: RetentionSpec, prefix: str, tensors: dict[str, torch.Tensor], rt: Runtime):
        if len(spec.decay) != spec.num_heads:
            raise ValueError(f"{len(spec.decay)} decays for {spec.num_heads} heads")
        if any(not 0.0 < float(a) <= 1.0 for a in spec.decay):
            raise ValueError("a decay must lie in (0, 1]")
        if spec.key_dim > 256:
            raise ValueError(f"a key size of {spec.key_dim} is beyond the recurrence kernel's limit of 256")
        self.spec = spec
        self.rt = rt
        t = lambda name: tensors[prefix + name]
        self.w_in = torch.cat([t(spec.q_name), t(spec.k_name), t(spec.v_name), t(spec.gate_name)], dim=0).contiguous()
        hk, hv = spec.num_heads * spec.key_dim, spec.num_heads * spec.value_dim
        self.q_off, self.k_off, self.v_off, self.g_off = 0, hk, 2 * hk, 2 * hk + hv
        self.decay = torch.tensor([float(a) for a in spec.decay], dtype=torch.float32, device=rt.device)
        self.position = POSITIONS.get(spec.position.kind)(spec.position, tensors, rt)
        if not hasattr(self.position, "rotary_table"):
            raise ValueError(f"position encoding {spec.position.kind!r} does not rotate queries and keys")
        self.halves = getattr(self.position, "PAIRING", "halves") == "halves"
        self.k_scale = spec.k_scale if spec.k_scale is not None else spec.key_dim ** -0.5
        self.w_o = t(spec.o_name)
        self.out_width = hv

    @staticmethod
    def expected_tensors(spec: RetentionSpec, prefix: str) -> dict[str, TensorReq]:
        h = spec.hidden_size
        hk, hv = spec.num_heads * spec.key_dim, spec.num_heads * spec.value_dim
        out = {
            prefix + spec.q_name: TensorReq((hk, h)),
            prefix + spec.k_name: TensorReq((hk, h)),
            prefix + spec.v_name: TensorReq((hv, h)),
            prefix + spec.gate_name: TensorReq((hv, h)),
            prefix + spec.o_name: TensorReq((h, hv)),
        }
        out.update(POSITIONS.get(spec.position.kind).expected_tensors(spec.position))
        return out

    def cache_need(self) -> StateNeed:
        return StateNeed((self.spec.num_heads, self.spec.key_dim, self.spec.value_dim), "float32")

    def GRAPH_SAFE(self) -> bool:
        return graph_safe(self.position)

    def weight_bytes(self) -> int:
        return tensor_bytes(self.w_in, self.w_o)

    TAKES_PROJ = True      # the stacked input projection may be part of a wider product (see ParallelMixer)

    def branch(self, h, step, cache_view, out: torch.Tensor | None = None, out_scale: float = 1.0, proj=None,
               proj_off: int = 0) -> torch.Tensor:
        """``proj``: a product of ``h`` that holds this part's input projection in its columns from ``proj_off`` on."""
        spec = self.spec
        if proj is None:
            proj, proj_off = linear(h, self.w_in, err=step.err), 0
        table, rotary_dim = self.position.rotary_table(step)
        prep = ops.retention_prepare(proj, self.decay, table, dtype=h.dtype, q_off=proj_off + self.q_off,
                                     k_off=proj_off + self.k_off, v_off=proj_off + self.v_off, heads=spec.num_heads, key_dim=spec.key_dim,
                                     value_dim=spec.value_dim, rotary_dim=rotary_dim, halves=self.halves,
                                     k_scale=self.k_scale)
        o = ops.gla_scan(prep, cache_view.records, step.req_q_start, step.req_q_len, step.req_slot, step.err)
        return ops.gla_out(o, proj, proj_off + self.g_off, None, spec.norm_eps, h.dtype, out=out, out_scale=out_scale)

    def forward(self, h, step, cache_view):
        return linear(self.branch(h, step, cache_view), self.w_o, err=step.err)
