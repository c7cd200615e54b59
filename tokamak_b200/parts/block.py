"""Arrangements of a mixer, a feed-forward and their norms in one block."""

from __future__ import annotations

from dataclasses import dataclass

import torch

from .base import (BLOCKS, FEED_FORWARDS, MIXERS, NORMS, HyperBranch, NormedBranch, OwedNorm, Runtime, TensorReq,
                   graph_safe, weight_bytes)


@dataclass(frozen=True)
class PreNormBlockSpec:
    """One block and the checkpoint names of its tensors.

    ``mixer_prefix`` and ``ffn_prefix`` end with a dot; ``norm1_name`` and
    ``norm2_name`` are full tensor names.
    """

    name: str
    norm1: object
    mixer: object
    norm2: object
    feed_forward: object
    norm1_name: str
    mixer_prefix: str
    norm2_name: str
    ffn_prefix: str
    kind: str = "pre_norm"


@BLOCKS.register("pre_norm")
class PreNormBlock:
    """``x = x + mixer(norm1(x)); x = x + ffn(norm2(x))``
    (src/tokamak/model/transformer.py:89-109).

    The block receives the float32 residual stream and the branch output that
    has not been added to it yet; each norm call adds the pending branch and
    normalises the sum in one kernel.  The second branch's output is returned as
    the new pending value, to be added by whoever normalises next.

    Where a branch can, its last product adds itself to the residual stream and prepares
    the input of the norm after it (see ``parts/base.py``, owed norms): the mixer for
    ``norm2``, the feed-forward for ``next_norm``, the norm that will consume what this
    block leaves pending.
    """

    TAKES_NEXT_NORM = True

    def __init__(self, spec: PreNormBlockSpec, tensors: dict[str, torch.Tensor], rt: Runtime):
        self.spec = spec
        self.norm1 = NORMS.get(spec.norm1.kind)(spec.norm1, spec.norm1_name, tensors, rt)
        self.mixer = MIXERS.get(spec.mixer.kind)(spec.mixer, spec.mixer_prefix, tensors, rt)
        self.norm2 = NORMS.get(spec.norm2.kind)(spec.norm2, spec.norm2_name, tensors, rt)
        self.feed_forward = FEED_FORWARDS.get(spec.feed_forward.kind)(
            spec.feed_forward, spec.ffn_prefix, tensors, rt)

    @staticmethod
    def expected_tensors(spec: PreNormBlockSpec) -> dict[str, TensorReq]:
        out: dict[str, TensorReq] = {}
        out.update(NORMS.get(spec.norm1.kind).expected_tensors(spec.norm1, spec.norm1_name))
        out.update(MIXERS.get(spec.mixer.kind).expected_tensors(spec.mixer, spec.mixer_prefix))
        out.update(NORMS.get(spec.norm2.kind).expected_tensors(spec.norm2, spec.norm2_name))
        out.update(FEED_FORWARDS.get(spec.feed_forward.kind).expected_tensors(
            spec.feed_forward, spec.ffn_prefix))
        return out

    def cache_need(self):
        return self.mixer.cache_need()

    def GRAPH_SAFE(self) -> bool:
        return graph_safe(self.norm1, self.mixer, self.norm2, self.feed_forward)

    @property
    def prefill_heads(self) -> int | None:
        """The mixer's hint for the work list of prompt portions, if it gives one."""
        return getattr(self.mixer, "prefill_heads", None)

    def weight_bytes(self) -> int:
        return weight_bytes(self.norm1, self.mixer, self.norm2, self.feed_forward)

    @property
    def entry_norm(self):
        return self.norm1

    @staticmethod
    def _branch(part, h, args: tuple, then_norm):
        if isinstance(h, OwedNorm) and not getattr(part, "TAKES_OWED_NORM", False):
            h = h.materialize()
        if then_norm is not None and getattr(part, "TAKES_THEN_NORM", False):
            return part.forward(h, *args, then_norm=then_norm)
        return part.forward(h, *args)

    def forward(self, resid: torch.Tensor, pending, step, cache_view, next_norm=None):
        h = self.norm1.add_norm(resid, pending)
        a = self._branch(self.mixer, h, (step, cache_view), (resid, self.norm2))
        h = self.norm2.add_norm(resid, a)
        out = self._branch(self.feed_forward, h, (step,), (resid, next_norm) if next_norm is not None else None)
        return resid, out


@dataclass(frozen=True)
class SandwichBlockSpec:
    """A block whose sublayers are normalised on the way in and on the way out, with a learned
    per-channel scale on what joins the residual stream.  ``feed_forward`` of ``None`` is a
    block of one sublayer.  The ``*_name`` fields are full tensor names (``None``: no layer
    scale); the prefixes end with a dot.

    ``conv_taps > 0`` gives every sublayer an *input convolution*: what the sublayer reads, ``h``, is
    replaced by ``h + conv(h)``, a causal convolution over time on every channel with the taps
    ``conv1_name`` / ``conv2_name`` (``[width, conv_taps]``, the last column weighing the current token).
    The last ``conv_taps - 1`` inputs are part of a request's state.
    """

    name: str
    norm_in1: object
    mixer: object
    norm_out1: object
    norm_in1_name: str
    mixer_prefix: str
    norm_out1_name: str
    scale1_name: str | None = None
    norm_in2: object = None
    feed_forward: object = None
    norm_out2: object = None
    norm_in2_name: str | None = None
    ffn_prefix: str | None = None
    norm_out2_name: str | None = None
    scale2_name: str | None = None
    conv_taps: int = 0
    conv1_name: str | None = None
    conv2_name: str | None = None
    kind: str = "sandwich"


@BLOCKS.register("sandwich")
class SandwichBlock:
    """``x = x + s1 * norm_out1(mixer(norm_in1(x)))``, then, if the block has a feed-forward,
    ``x = x + s2 * norm_out2(ffn(norm_in2(x)))``, with ``s1`` and ``s2`` per-channel scales.

    A sublayer's output is left as a :class:`NormedBranch`; the norm in front of the next
    sublayer (this block's, the next block's, or the model's last norm) normalises it, scales
    it, adds it to the float32 residual stream and normalises the sum, in one kernel.

    With input convolutions the block keeps state of its own beside its mixer's: one float32 record
    ``[conv_taps - 1, width]`` per sublayer and request (``cache_need`` is then a dictionary, and so is the
    view that ``forward`` is given).  Where the seat in front of a sublayer has no norm (``join``), the
    convolution reads the float32 stream itself and its result is rounded once.
    """

    def __init__(self, spec: SandwichBlockSpec, tensors: dict[str, torch.Tensor], rt: Runtime):
        self.spec = spec
        self.norm_in1 = NORMS.get(spec.norm_in1.kind)(spec.norm_in1, spec.norm_in1_name, tensors, rt)
        self.mixer = MIXERS.get(spec.mixer.kind)(spec.mixer, spec.mixer_prefix, tensors, rt)
        self.norm_out1 = NORMS.get(spec.norm_out1.kind)(spec.norm_out1, spec.norm_out1_name, tensors, rt)
        self.scale1 = tensors[spec.scale1_name] if spec.scale1_name else None
        self.feed_forward = self.norm_in2 = self.norm_out2 = self.scale2 = None
        if spec.feed_forward is not None:
            self.norm_in2 = NORMS.get(spec.norm_in2.kind)(spec.norm_in2, spec.norm_in2_name, tensors, rt)
            self.feed_forward = FEED_FORWARDS.get(spec.feed_forward.kind)(spec.feed_forward, spec.ffn_prefix, tensors, rt)
            self.norm_out2 = NORMS.get(spec.norm_out2.kind)(spec.norm_out2, spec.norm_out2_name, tensors, rt)
            self.scale2 = tensors[spec.scale2_name] if spec.scale2_name else None
        for norm in (self.norm_out1, self.norm_out2):
            if norm is not None and not hasattr(norm, "owed_norm_params"):
                raise ValueError("the norm after a sublayer must hand out its weight and eps (owed_norm_params)")
        self.rt = rt
        self.conv1 = self.conv2 = None
        if spec.conv_taps > 0:
            if not 1 <= spec.conv_taps <= 8:
                raise ValueError(f"an input convolution of {spec.conv_taps} taps is not taken (1 to 8)")
            self.conv1 = tensors[spec.conv1_name].float().contiguous()
            if spec.feed_forward is not None:
                self.conv2 = tensors[spec.conv2_name].float().contiguous()

    @staticmethod
    def expected_tensors(spec: SandwichBlockSpec) -> dict[str, TensorReq]:
        out: dict[str, TensorReq] = {}
        out.update(NORMS.get(spec.norm_in1.kind).expected_tensors(spec.norm_in1, spec.norm_in1_name))
        out.update(MIXERS.get(spec.mixer.kind).expected_tensors(spec.mixer, spec.mixer_prefix))
        out.update(NORMS.get(spec.norm_out1.kind).expected_tensors(spec.norm_out1, spec.norm_out1_name))
        if spec.scale1_name:
            out[spec.scale1_name] = TensorReq((spec.norm_out1.dim,), role="vector")
        if spec.feed_forward is not None:
            out.update(NORMS.get(spec.norm_in2.kind).expected_tensors(spec.norm_in2, spec.norm_in2_name))
            out.update(FEED_FORWARDS.get(spec.feed_forward.kind).expected_tensors(spec.feed_forward, spec.ffn_prefix))
            out.update(NORMS.get(spec.norm_out2.kind).expected_tensors(spec.norm_out2, spec.norm_out2_name))
            if spec.scale2_name:
                out[spec.scale2_name] = TensorReq((spec.norm_out2.dim,), role="vector")
        if spec.conv_taps > 0:
            width = spec.norm_out1.dim
            out[spec.conv1_name] = TensorReq((width, spec.conv_taps), role="bias")
            if spec.feed_forward is not None:
                out[spec.conv2_name] = TensorReq((width, spec.conv_taps), role="bias")
        return out

    def cache_need(self):
        need = self.mixer.cache_need()
        if self.spec.conv_taps <= 1:
            return need
        from ..cache.manager import StateNeed
        tail = StateNeed((self.spec.conv_taps - 1, self.spec.norm_out1.dim), "float32")
        out = {"conv1": tail}
        if need is not None:
            out["mixer"] = need
        if self.conv2 is not None:
            out["conv2"] = tail
        return out

    def _parts(self) -> list:
        return [p for p in (self.norm_in1, self.mixer, self.norm_out1, self.norm_in2, self.feed_forward,
                            self.norm_out2) if p is not None]

    def GRAPH_SAFE(self) -> bool:
        return graph_safe(*self._parts())

    @property
    def prefill_heads(self) -> int | None:
        return getattr(self.mixer, "prefill_heads", None)

    def weight_bytes(self) -> int:
        extra = sum(t.numel() * t.element_size() for t in (self.scale1, self.scale2, self.conv1, self.conv2)
                    if t is not None)
        return weight_bytes(*self._parts()) + extra

    @property
    def entry_norm(self):
        return self.norm_in1

    @staticmethod
    def _leave(x, norm, scale) -> NormedBranch:
        weight, eps = norm.owed_norm_params()
        return NormedBranch(x, weight, eps, scale, getattr(norm, "groups", 1))

    def _read(self, norm_in, taps, tail_view, resid, pending, step):
        """What a sublayer reads: the rows of the seat in front of it, through the input convolution if
        the block has one."""
        if taps is None:
            h = norm_in.add_norm(resid, pending)
            return h.materialize() if isinstance(h, OwedNorm) else h
        from ..csrc import ops
        if hasattr(norm_in, "join"):
            norm_in.join(resid, pending)
            rows = resid
        else:
            rows = norm_in.add_norm(resid, pending)
            rows = rows.materialize() if isinstance(rows, OwedNorm) else rows
        tail = tail_view.records if tail_view is not None else None
        return ops.short_conv(rows, taps, tail, step, dtype=self.rt.dtype, add_input=True)

    def forward(self, resid: torch.Tensor, pending, step, cache_view):
        # with input convolutions of more than one tap the view is this block's dictionary (see cache_need);
        # otherwise it is the mixer's own, which may be a dictionary too
        views = cache_view if self.spec.conv_taps > 1 else {"mixer": cache_view}
        h = self._read(self.norm_in1, self.conv1, views.get("conv1"), resid, pending, step)
        pending = self._leave(self.mixer.forward(h, step, views.get("mixer")), self.norm_out1, self.scale1)
        if self.feed_forward is not None:
            h = self._read(self.norm_in2, self.conv2, views.get("conv2"), resid, pending, step)
            pending = self._leave(self.feed_forward.forward(h, step), self.norm_out2, self.scale2)
        return resid, pending


@dataclass(frozen=True)
class HyperBlockSpec:
    """A pre-norm block over a residual stream kept in ``streams`` copies.  Sublayer ``q`` (1: the mixer, 2: the
    feed-forward, which may be absent) has three tensors under ``hc<q>_prefix``: ``in`` ``[streams]`` (how the copies
    are read), ``out`` ``[streams]`` (how its output is written to each copy) and ``mix`` ``[streams, streams]``
    (how the copies are mixed meanwhile, indexed [from, to]).  ``connections=False``: no such tensors; the block
    is then ``x <- x + mult * sublayer(norm(x))`` on the one copy it is given.  ``mult`` scales what a sublayer
    adds.  The ``*_name`` fields are full tensor names; the prefixes end with a dot."""

    name: str
    norm1: object
    mixer: object
    norm1_name: str
    mixer_prefix: str
    streams: int = 1
    connections: bool = True
    mult: float = 1.0
    norm2: object = None
    feed_forward: object = None
    norm2_name: str | None = None
    ffn_prefix: str | None = None
    hc1_prefix: str | None = None
    hc2_prefix: str | None = None
    in_name: str = "in"
    out_name: str = "out"
    mix_name: str = "mix"
    kind: str = "hyper"


@BLOCKS.register("hyper")
class HyperBlock:
    """For each sublayer: ``u = sum_s in[s] x_s``, ``y = sublayer(norm(u))``, then, all copies at once from the old
    ones, ``x_t <- sum_s mix[s, t] x_s + mult * out[t] * y``.

    The write is left pending as a :class:`~tokamak_b200.parts.base.HyperBranch`; the norm in front of the next
    sublayer (this block's, the next block's, the model's last) does it together with its own read and
    normalisation, so the copies cross memory once per sublayer.  The norms must take a ``read`` argument
    (:class:`~tokamak_b200.parts.norm.LayerNorm`)."""

    def __init__(self, spec: HyperBlockSpec, tensors: dict[str, torch.Tensor], rt: Runtime):
        if spec.streams < 1 or (not spec.connections and spec.streams != 1):
            raise ValueError(f"{spec.streams} copies of the stream without connections between them")
        self.spec = spec
        self.rt = rt
        self.norm1 = NORMS.get(spec.norm1.kind)(spec.norm1, spec.norm1_name, tensors, rt)
        self.mixer = MIXERS.get(spec.mixer.kind)(spec.mixer, spec.mixer_prefix, tensors, rt)
        self.norm2 = self.feed_forward = None
        if spec.feed_forward is not None:
            self.norm2 = NORMS.get(spec.norm2.kind)(spec.norm2, spec.norm2_name, tensors, rt)
            self.feed_forward = FEED_FORWARDS.get(spec.feed_forward.kind)(spec.feed_forward, spec.ffn_prefix, tensors, rt)
        self.hc1 = self._connections(spec.hc1_prefix, tensors)
        self.hc2 = self._connections(spec.hc2_prefix, tensors) if spec.feed_forward is not None else None

    def _connections(self, prefix, tensors):
        if not self.spec.connections:
            return None, None, None
        s = self.spec
        return tuple(tensors[prefix + n].float().contiguous() for n in (s.in_name, s.out_name, s.mix_name))

    @staticmethod
    def expected_tensors(spec: HyperBlockSpec) -> dict[str, TensorReq]:
        out: dict[str, TensorReq] = {}
        out.update(NORMS.get(spec.norm1.kind).expected_tensors(spec.norm1, spec.norm1_name))
        out.update(MIXERS.get(spec.mixer.kind).expected_tensors(spec.mixer, spec.mixer_prefix))
        prefixes = [spec.hc1_prefix]
        if spec.feed_forward is not None:
            out.update(NORMS.get(spec.norm2.kind).expected_tensors(spec.norm2, spec.norm2_name))
            out.update(FEED_FORWARDS.get(spec.feed_forward.kind).expected_tensors(spec.feed_forward, spec.ffn_prefix))
            prefixes.append(spec.hc2_prefix)
        if spec.connections:
            for prefix in prefixes:
                out[prefix + spec.in_name] = TensorReq((spec.streams,), role="fraction")
                out[prefix + spec.out_name] = TensorReq((spec.streams,), role="vector")
                out[prefix + spec.mix_name] = TensorReq((spec.streams, spec.streams), role="fraction")
        return out

    def cache_need(self):
        return self.mixer.cache_need()

    def _parts(self) -> list:
        return [p for p in (self.norm1, self.mixer, self.norm2, self.feed_forward) if p is not None]

    def GRAPH_SAFE(self) -> bool:
        return graph_safe(*self._parts())

    @property
    def prefill_heads(self) -> int | None:
        return getattr(self.mixer, "prefill_heads", None)

    def weight_bytes(self) -> int:
        return weight_bytes(*self._parts())

    @property
    def entry_norm(self):
        return self.norm1

    def forward(self, resid: torch.Tensor, pending, step, cache_view):
        copies = resid.shape[0] if resid.dim() == 3 else 1
        if copies != self.spec.streams:
            raise ValueError(f"the block works on {self.spec.streams} copies of the stream and is given {copies}")
        read, write, mix = self.hc1
        h = self.norm1.add_norm(resid, pending, read=read)
        pending = HyperBranch(self.mixer.forward(h, step, cache_view), mix, write, self.spec.mult)
        if self.feed_forward is not None:
            read, write, mix = self.hc2
            h = self.norm2.add_norm(resid, pending, read=read)
            pending = HyperBranch(self.feed_forward.forward(h, step), mix, write, self.spec.mult)
        return resid, pending
