"""Position encodings.  A rotary position part hands the mixer a table of (cos, sin) pairs for
the tokens of the step; the rotation itself happens in the mixer's fused kernel.  An absolute
encoding would instead implement ``add_to_embedding`` (see ``parts/base.py``)."""

from __future__ import annotations

from dataclasses import dataclass

import torch

from ..csrc import ops
from .base import POSITIONS, Runtime, TensorReq


@dataclass(frozen=True)
class RopeSpec:
    head_dim: int
    theta: float
    kind: str = "rope_neox"


@dataclass(frozen=True)
class NoPositionSpec:
    kind: str = "none"


@POSITIONS.register("rope_neox")
class RopeNeox:
    """Half-rotation rotary embedding over the whole head
    (src/tokamak/model/layers.py:36-89).

    ``inv_freq[j] = 1 / theta ** (2j / d)`` is formed in float32 from a float32
    ``arange`` exactly as the reference does (layers.py:47); a kernel multiplies it by
    the float32 position and takes cosine and sine in float32, once per step: every
    layer with the same spec reads the same table.
    """

    GRAPH_SAFE = True

    def __init__(self, spec: RopeSpec, tensors: dict, rt: Runtime):
        if spec.head_dim % 2:
            raise ValueError(f"rotary embedding needs an even head_dim, got {spec.head_dim}")
        self.spec = spec
        inv_freq = 1.0 / (spec.theta ** (torch.arange(0, spec.head_dim, 2, dtype=torch.float32)
                                         / spec.head_dim))
        self.inv_freq = inv_freq.to(rt.device)

    @staticmethod
    def expected_tensors(spec: RopeSpec) -> dict:
        return {}

    def rotary_table(self, step) -> tuple[torch.Tensor | None, int]:
        """``([tokens, head_dim / 2, 2] float32 of (cos, sin), rotary_dim)`` for the step's tokens."""
        key = ("rope_table", self.spec)
        table = step.scratch.get(key)
        if table is None:
            table = ops.rope_table(step.positions, self.inv_freq)
            step.scratch[key] = table
        return table, self.spec.head_dim


@dataclass(frozen=True)
class YarnScaling:
    """Stretching of a rotary encoding beyond the length it was trained for: pairs that turn fewer
    than ``slow`` times over ``original`` positions have their frequency divided by ``factor``, pairs
    that turn more than ``fast`` times keep it, a linear ramp over the pair index lies between; cosine
    and sine are multiplied by ``0.1 ln(factor) + 1``."""

    factor: float
    original: float
    fast: float
    slow: float


@dataclass(frozen=True)
class RopePairsSpec:
    """Rotation of neighbouring pairs (elements 2i and 2i+1) over the first ``rotary_dim``
    elements of a head; the rest passes unrotated.  ``yarn`` stretches the frequencies."""

    rotary_dim: int
    theta: float
    yarn: YarnScaling | None = None
    kind: str = "rope_pairs"
    linear_factor: float = 1.0     # every frequency is divided by it (linear position scaling)


def yarn_frequencies(rotary_dim: int, theta: float, yarn: YarnScaling | None) -> tuple[torch.Tensor, float]:
    """``(float64 frequencies [rotary_dim / 2], factor on cosine and sine)``.  With
    ``where(t) = rotary_dim ln(original / (2 pi t)) / (2 ln theta)``, the pair index at which a pair turns
    ``t`` times over the original length, the ramp runs from ``lo = max(floor(where(fast)), 0)`` to
    ``hi = min(ceil(where(slow)), rotary_dim - 1)``: ``ramp = clamp((i - lo) / max(hi - lo, 0.001), 0, 1)`` and
    ``f = f0 / factor * ramp + f0 * (1 - ramp)``."""
    import math
    idx = torch.arange(0, rotary_dim, 2, dtype=torch.float64)
    freq = float(theta) ** (-idx / max(rotary_dim, 1))
    if yarn is None:
        return freq, 1.0
    where = lambda turns: rotary_dim * math.log(yarn.original / (2.0 * math.pi * turns)) / (2.0 * math.log(theta))
    lo = max(math.floor(where(yarn.fast)), 0)
    hi = min(math.ceil(where(yarn.slow)), rotary_dim - 1)
    ramp = ((idx / 2 - lo) / max(hi - lo, 0.001)).clamp(0.0, 1.0)
    return freq / yarn.factor * ramp + freq * (1.0 - ramp), 0.1 * math.log(yarn.factor) + 1.0


@POSITIONS.register("rope_pairs")
class RopePairs:
    """Rotary embedding in the interleaved layout: pair ``i`` of a head, ``(x[2i], x[2i+1])``,
    turns by ``position * theta ** (-2i / rotary_dim)``.  The frequencies are rounded to
    float32 once; position times frequency, cosine and sine are float32, once per step."""

    GRAPH_SAFE = True
    PAIRING = "neighbours"       # the mixer hands the table to a kernel that rotates (2i, 2i+1)

    def __init__(self, spec: RopePairsSpec, tensors: dict, rt: Runtime):
        if spec.rotary_dim % 2 or spec.rotary_dim < 0:
            raise ValueError(f"the rotated part of a head must be even, got {spec.rotary_dim}")
        self.spec = spec
        freq, self.magnitude = yarn_frequencies(spec.rotary_dim, spec.theta, spec.yarn)
        self.inv_freq = (freq / spec.linear_factor).to(torch.float32).to(rt.device)

    @staticmethod
    def expected_tensors(spec: RopePairsSpec) -> dict:
        return {}

    def rotary_table(self, step) -> tuple[torch.Tensor | None, int]:
        if self.spec.rotary_dim == 0:
            return None, 0
        key = ("rope_table", self.spec)
        table = step.scratch.get(key)
        if table is None:
            table = ops.rope_table(step.positions, self.inv_freq, self.magnitude)
            step.scratch[key] = table
        return table, self.spec.rotary_dim


@dataclass(frozen=True)
class RopeHalvesSpec:
    """Rotation of halves (elements i and i + rotary_dim / 2) over the first ``rotary_dim`` elements of a head;
    the rest passes unrotated.  ``linear_factor`` divides every frequency."""

    rotary_dim: int
    theta: float
    linear_factor: float = 1.0
    kind: str = "rope_halves"


@POSITIONS.register("rope_halves")
class RopeHalves:
    """Rotary embedding in the half-split layout on part of the head: element ``i < rotary_dim / 2`` and element
    ``i + rotary_dim / 2`` turn by ``position * theta ** (-2i / rotary_dim) / linear_factor``.  The frequencies are
    formed in float64 and rounded to float32 once; position times frequency, cosine and sine are float32, once
    per step.  The mixer's kernel does the rotation (``PAIRING`` tells it which elements pair up)."""

    GRAPH_SAFE = True
    PAIRING = "halves"

    def __init__(self, spec: RopeHalvesSpec, tensors: dict, rt: Runtime):
        if spec.rotary_dim % 2 or spec.rotary_dim < 0:
            raise ValueError(f"the rotated part of a head must be even, got {spec.rotary_dim}")
        self.spec = spec
        freq, _ = yarn_frequencies(spec.rotary_dim, spec.theta, None)
        self.inv_freq = (freq / spec.linear_factor).to(torch.float32).to(rt.device)

    @staticmethod
    def expected_tensors(spec: RopeHalvesSpec) -> dict:
        return {}

    def rotary_table(self, step) -> tuple[torch.Tensor | None, int]:
        if self.spec.rotary_dim == 0:
            return None, 0
        key = ("rope_table", self.spec)
        table = step.scratch.get(key)
        if table is None:
            table = ops.rope_table(step.positions, self.inv_freq)
            step.scratch[key] = table
        return table, self.spec.rotary_dim


@POSITIONS.register("none")
class NoPosition:
    """No position encoding: queries and keys pass unrotated."""

    GRAPH_SAFE = True

    def __init__(self, spec: NoPositionSpec, tensors: dict, rt: Runtime):
        self.spec = spec

    @staticmethod
    def expected_tensors(spec: NoPositionSpec) -> dict:
        return {}

    def rotary_table(self, step) -> tuple[torch.Tensor | None, int]:
        return None, 0


@dataclass(frozen=True)
class LearnedPositionSpec:
    """An absolute encoding: row ``position`` of a learned table ``[max_positions, hidden_size]`` joins the
    embedded token, times ``scale``."""

    max_positions: int
    hidden_size: int
    name: str = "pos"
    scale: float = 1.0
    kind: str = "learned_absolute"


@POSITIONS.register("learned_absolute")
class LearnedPosition:
    """For the model's ``embedding_position`` seat: ``x[t] += scale * table[position[t]]`` in the float32
    stream (the embedding's gather kernel, accumulating).  A position beyond the table is reported through
    the step's error word."""

    GRAPH_SAFE = True

    def __init__(self, spec: LearnedPositionSpec, tensors: dict, rt: Runtime):
        self.spec = spec
        self.table = tensors[spec.name]

    @staticmethod
    def expected_tensors(spec: LearnedPositionSpec) -> dict:
        return {spec.name: TensorReq((spec.max_positions, spec.hidden_size))}

    def weight_bytes(self) -> int:
        return 0          # read by row

    def add_to_embedding(self, resid: torch.Tensor, step) -> None:
        ops.embed_gather(self.table, step.positions, resid, step.err, scale=self.spec.scale, accumulate=True)
