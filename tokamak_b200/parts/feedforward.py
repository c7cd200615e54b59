"""Feed-forward parts."""

from __future__ import annotations

from dataclasses import dataclass

import torch

from ..csrc import ops
from .base import (FEED_FORWARDS, SWAPPED_GEMM_MAX_TOKENS, OwedNorm, Runtime, TensorReq, chain_of, linear,
                   tensor_bytes)


@dataclass(frozen=True)
class SwiGLUSpec:
    """A gated unit ``down(act(gate(x)) * up(x))``; ``activation`` is ``silu`` (SwiGLU) or
    ``gelu_tanh``; the three names are the tensors' names after the part's prefix."""

    hidden_size: int
    intermediate_size: int
    kind: str = "swiglu"
    activation: str = "silu"
    gate_name: str = "gate_proj.weight"
    up_name: str = "up_proj.weight"
    down_name: str = "down_proj.weight"


@FEED_FORWARDS.register("swiglu")
class SwiGLU:
    """``down(silu(gate(x)) * up(x))`` without biases (src/tokamak/model/layers.py:92-104).

    The gate and up matrices are stacked into one ``[2I, H]`` operand so that one
    product feeds the activation.  Where the intermediate size allows it, their rows
    alternate in blocks of 64 (64 gate rows, then the 64 up rows of the same outputs): a
    128-row tile of the decode product then holds both halves of 64 outputs, and the block
    that adds its K splits up applies the activation itself, so that decoding needs no
    activation kernel and no float32 round trip of the ``[tokens, 2I]`` sums.

    ``activation`` (silu, or the tanh form of gelu) is applied by the same epilogues.
    """

    def __init__(self, spec: SwiGLUSpec, prefix: str, tensors: dict[str, torch.Tensor], rt: Runtime):
        self.spec = spec
        self.rt = rt
        if spec.activation not in ops.GLU_ACTIVATIONS:
            raise ValueError(f"unknown activation {spec.activation!r}; known: {', '.join(ops.GLU_ACTIVATIONS)}")
        self.fused_act = True      # the products' fused epilogues know every activation of ops.GLU_ACTIVATIONS
        gate, up = tensors[prefix + spec.gate_name], tensors[prefix + spec.up_name]
        i, h = spec.intermediate_size, spec.hidden_size
        b = ops.SWIGLU_TILE_BLOCK
        if i % b == 0:
            self.block = b
            self.w_gate_up = torch.stack((gate.view(i // b, b, h), up.view(i // b, b, h)), dim=1).reshape(2 * i, h)
        else:
            self.block = i
            self.w_gate_up = torch.cat((gate, up), dim=0)
        self.w_gate_up = self.w_gate_up.contiguous()
        self.w_down = tensors[prefix + spec.down_name]

    @staticmethod
    def expected_tensors(spec: SwiGLUSpec, prefix: str) -> dict[str, TensorReq]:
        h, i = spec.hidden_size, spec.intermediate_size
        return {
            prefix + spec.gate_name: TensorReq((i, h)),
            prefix + spec.up_name: TensorReq((i, h)),
            prefix + spec.down_name: TensorReq((h, i)),
        }

    GRAPH_SAFE = True

    def weight_bytes(self) -> int:
        return tensor_bytes(self.w_gate_up, self.w_down)

    TAKES_OWED_NORM = True     # the gate/up product pays an owed norm scale in its epilogue
    TAKES_THEN_NORM = True     # the down product can add itself to the residual stream

    def forward(self, h, step, then_norm=None):
        err = step.err if step is not None else None
        chain = chain_of(step)
        n = h.shape[0]
        if (self.fused_act and h.dtype == torch.bfloat16 and err is not None and n <= SWAPPED_GEMM_MAX_TOKENS
                and self.block == ops.SWIGLU_TILE_BLOCK and self.spec.hidden_size % 8 == 0):
            splits, stages, cluster = ops.swapped_gemm_plan(2 * self.spec.intermediate_size, self.spec.hidden_size, n)
            colscale = None
            if isinstance(h, OwedNorm):
                colscale, h = (h.sumsq, h.dim, h.eps), h.xb
            act = ops.gemm_tc_swapped(self.w_gate_up, h, err, splits, max_stages=stages, cluster=cluster,
                                      swiglu=True, activation=self.spec.activation, colscale=colscale, chain=chain)
        else:
            if isinstance(h, OwedNorm):
                h = h.materialize()
            if (self.fused_act and h.dtype == torch.bfloat16 and err is not None and self.block == ops.SWIGLU_TILE_BLOCK
                    and ops.pair_gemm_takes(n, 2 * self.spec.intermediate_size, self.spec.hidden_size, fused=True)):
                # many tokens: the product on pairs of SMs applies the activation to its accumulators
                act = ops.gemm_pair(h, self.w_gate_up, err, swiglu=True, activation=self.spec.activation)
            else:
                gate_up = linear(h, self.w_gate_up, err=err)
                act = torch.empty((n, self.spec.intermediate_size), dtype=h.dtype, device=h.device)
                ops.swiglu(gate_up, act, block=self.block, activation=self.spec.activation)
        return linear(act, self.w_down, err=err, then_norm=then_norm, chain=chain)


@dataclass(frozen=True)
class MlpSpec:
    """An ungated unit ``down(act(up(x)))``; ``activation`` is ``relu2`` (the square of relu), ``gelu_tanh`` or
    ``silu``; the names are the tensors' names after the part's prefix."""

    hidden_size: int
    intermediate_size: int
    activation: str = "relu2"
    up_name: str = "up"
    down_name: str = "down"
    kind: str = "mlp"


@FEED_FORWARDS.register("mlp")
class Mlp:
    """``W_down act(W_up x)`` without biases.  In bfloat16 the activation rides in the epilogue of the first
    product (steps of few tokens: the tcgen05 product whose cluster adds its splits up; many tokens: the product
    on pairs of SMs), where the sizes allow; otherwise, and in float32, it is a kernel of its own that also adds
    up the float32 partial sums of a split product (``csrc/elementwise.cu``)."""

    GRAPH_SAFE = True

    def __init__(self, spec: MlpSpec, prefix: str, tensors: dict[str, torch.Tensor], rt: Runtime):
        if spec.activation not in ops.UNARY_ACTIVATIONS:
            raise ValueError(f"unknown activation {spec.activation!r}; known: {', '.join(ops.UNARY_ACTIVATIONS)}")
        self.spec = spec
        self.rt = rt
        self.w_up = tensors[prefix + spec.up_name]
        self.w_down = tensors[prefix + spec.down_name]

    @staticmethod
    def expected_tensors(spec: MlpSpec, prefix: str) -> dict[str, TensorReq]:
        h, i = spec.hidden_size, spec.intermediate_size
        return {prefix + spec.up_name: TensorReq((i, h)), prefix + spec.down_name: TensorReq((h, i))}

    def weight_bytes(self) -> int:
        return tensor_bytes(self.w_up, self.w_down)

    def forward(self, h, step):
        err = step.err if step is not None else None
        if isinstance(h, OwedNorm):
            h = h.materialize()
        n, name = h.shape[0], self.spec.activation
        ff, width = self.spec.intermediate_size, self.spec.hidden_size
        if h.dtype == torch.bfloat16 and err is not None and n <= SWAPPED_GEMM_MAX_TOKENS and ff % 128 == 0 and width % 8 == 0:
            # few tokens: the cluster that adds the product's splits up applies the activation
            splits, stages, cluster = ops.swapped_gemm_plan(ff, width, n)
            act = ops.gemm_tc_swapped(self.w_up, h, err, splits, max_stages=stages, cluster=cluster, unary=name)
        elif h.dtype == torch.bfloat16 and err is not None and ops.pair_gemm_takes(n, ff, width, fused=True):
            # many tokens: the product on pairs of SMs applies it to its accumulators
            act = ops.gemm_pair(h, self.w_up, err, unary=name)
        else:
            act = ops.unary_act(linear(h, self.w_up, err=err), h.dtype, name)
        return linear(act, self.w_down, err=err)


@dataclass(frozen=True)
class MoESpec:
    """A mixture of ``num_experts`` gated units of inner size ``intermediate_size`` of which every token uses
    ``top``.  The experts form ``num_groups`` equal groups of neighbours and only experts of the ``keep_groups``
    best groups can be chosen (``num_groups = keep_groups = 1``: no restriction).  ``correction``: a learned
    number per expert that is added to the scores for the choice only.  The ``*_name`` fields are the
    tensors' names after the part's prefix; expert ``e``'s matrices lie under ``expert_prefix.format(e)``."""

    hidden_size: int
    intermediate_size: int
    num_experts: int
    top: int
    num_groups: int = 1
    keep_groups: int = 1
    correction: bool = True
    activation: str = "silu"
    router_name: str = "router"
    correction_name: str = "correction"
    expert_prefix: str = "e{}."
    gate_name: str = "gate"
    up_name: str = "up"
    down_name: str = "down"
    kind: str = "moe"


@FEED_FORWARDS.register("moe")
class MixtureOfExperts:
    """Router scores are sigmoids of 32-bit logits, ``s = sigmoid(W_r h)``; the choice is made on
    ``s + correction``: a group's score is the sum of its two largest choice scores, experts outside the best
    groups cannot be chosen, and the ``top`` largest of the rest are; the weights are the chosen experts'
    plain scores, not renormalised; the output is the weighted sum of the chosen experts'
    ``W_down (act(W_gate h) * (W_up h))``.  Experts have no biases.

    The experts' matrices are stacked ``[experts, ...]`` at load.  A step's (token, choice) pairs are laid
    out expert by expert on the device, so nothing is read back and a step of single tokens can be
    replayed from a CUDA graph; the products run over tiles of one expert's rows (``csrc/moe.cu``).  The
    result is float32 and does not depend on what else is in the batch.
    """

    GRAPH_SAFE = True

    def __init__(self, spec: MoESpec, prefix: str, tensors: dict[str, torch.Tensor], rt: Runtime):
        if spec.activation not in ops.GLU_ACTIVATIONS:
            raise ValueError(f"unknown activation {spec.activation!r}; known: {', '.join(ops.GLU_ACTIVATIONS)}")
        if spec.num_experts % spec.num_groups or not 1 <= spec.keep_groups <= spec.num_groups:
            raise ValueError(f"{spec.num_experts} experts do not form {spec.num_groups} equal groups of which "
                             f"{spec.keep_groups} are kept")
        if not 1 <= spec.top <= spec.keep_groups * (spec.num_experts // spec.num_groups):
            raise ValueError(f"{spec.top} experts cannot be chosen from {spec.keep_groups} groups of "
                             f"{spec.num_experts // spec.num_groups}")
        self.spec = spec
        self.rt = rt
        self.router = tensors[prefix + spec.router_name].float().contiguous()
        self.correction = tensors[prefix + spec.correction_name].contiguous() if spec.correction else None
        stack = lambda name: torch.stack([tensors[prefix + spec.expert_prefix.format(e) + name]
                                          for e in range(spec.num_experts)]).contiguous()
        self.w_gate, self.w_up, self.w_down = stack(spec.gate_name), stack(spec.up_name), stack(spec.down_name)
        # bfloat16 at sizes the product on pairs of SMs takes: gate and up rows alternate in blocks, so that
        # the activation is the product's epilogue; the two matrices are then kept only in that form
        self.w_gate_up = None
        if ops.moe_tc_takes(self.w_gate.dtype, spec.hidden_size, spec.intermediate_size):
            self.w_gate_up = ops.moe_stack_gate_up(self.w_gate, self.w_up)
            self.w_gate = self.w_up = None

    @staticmethod
    def expected_tensors(spec: MoESpec, prefix: str) -> dict[str, TensorReq]:
        h, i = spec.hidden_size, spec.intermediate_size
        out = {}
        for e in range(spec.num_experts):
            p = prefix + spec.expert_prefix.format(e)
            out[p + spec.gate_name] = TensorReq((i, h))
            out[p + spec.up_name] = TensorReq((i, h))
            out[p + spec.down_name] = TensorReq((h, i))
        out[prefix + spec.router_name] = TensorReq((spec.num_experts, h), role="matrix_f32")
        if spec.correction:
            out[prefix + spec.correction_name] = TensorReq((spec.num_experts,), role="bias")
        return out

    def weight_bytes(self) -> int:
        """What a step of one token reads: the router and ``top`` experts (a large step reads all)."""
        per_expert = tensor_bytes(self.w_gate, self.w_up, self.w_gate_up, self.w_down) // self.spec.num_experts
        return tensor_bytes(self.router, self.correction) + self.spec.top * per_expert

    def forward(self, h, step):
        spec = self.spec
        if isinstance(h, OwedNorm):
            h = h.materialize()
        tc = self.w_gate_up is not None
        routing = ops.moe_route(h, self.router, self.correction, top=spec.top, n_groups=spec.num_groups,
                                keep=spec.keep_groups, padded=tc)
        if tc and ops.moe_small_takes(h.shape[0], spec.top, spec.hidden_size, spec.intermediate_size):
            out = ops.moe_experts_small(h, routing, self.w_gate_up, self.w_down, activation=spec.activation)
        elif tc:
            out = ops.moe_experts_tc(h, routing, self.w_gate_up, self.w_down, step.err, activation=spec.activation)
        else:
            out = ops.moe_experts(h, routing, self.w_gate, self.w_up, self.w_down, activation=spec.activation)
        return out.unsqueeze(0)         # float32 sums, one part: the consuming norm reads them as they are
