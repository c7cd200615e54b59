"""The attention mixer: grouped-query attention over paged keys and values."""

from __future__ import annotations

import contextlib
from dataclasses import dataclass

import torch

from ..cache.manager import KVPagesNeed
from ..csrc import ops
from .base import (MIXERS, POSITIONS, SWAPPED_GEMM_MAX_TOKENS, OwedNorm, Runtime, TensorReq, chain_of,
                   graph_safe, linear, tensor_bytes)


@dataclass(frozen=True)
class AttentionSpec:
    """Sizes and constants of one attention mixer.

    ``qk_norm_eps`` of ``None`` switches the per-head norm of q and k off;
    ``window`` of ``None`` means every earlier key is seen; ``own_kv=False``
    describes a layer without key and value projections that reads the pages
    another layer wrote (the schedule names which).
    """

    hidden_size: int
    num_heads: int
    num_kv_heads: int
    head_dim: int
    position: object                       # a position spec (kind, ...)
    qk_norm_eps: float | None = None
    window: int | None = None
    own_kv: bool = True
    softmax_scale: float | None = None     # default head_dim ** -0.5
    kind: str = "attention"


@MIXERS.register("attention")
class Attention:
    """Projections, per-head q/k norm, rotation, page write and attention
    (src/tokamak/model/transformer.py:22-86 with the step context's
    store-then-attend order, src/tokamak/model/step_context.py:88).

    The q, k and v matrices are stacked into one ``[(Hq + 2 Hkv) d, H]`` operand.
    """

    def __init__(self, spec: AttentionSpec, prefix: str, tensors: dict[str, torch.Tensor], rt: Runtime):
        if spec.num_heads % spec.num_kv_heads:
            raise ValueError(f"{spec.num_heads} query heads are not a multiple of "
                             f"{spec.num_kv_heads} key/value heads")
        if spec.head_dim > 256 or spec.head_dim % 4:
            raise ValueError(f"head_dim {spec.head_dim} is not taken by the attention kernels: "
                             f"they need a multiple of 4 up to 256")
        self.spec = spec
        self.rt = rt
        mats = [tensors[prefix + "q_proj.weight"]]
        if spec.own_kv:
            mats += [tensors[prefix + "k_proj.weight"], tensors[prefix + "v_proj.weight"]]
        self.w_qkv = torch.cat(mats, dim=0).contiguous() if len(mats) > 1 else mats[0]
        self.w_o = tensors[prefix + "o_proj.weight"]
        self.q_norm_w = tensors.get(prefix + "q_norm.weight") if spec.qk_norm_eps is not None else None
        self.k_norm_w = tensors.get(prefix + "k_norm.weight") if spec.qk_norm_eps is not None else None
        self.position = POSITIONS.get(spec.position.kind)(spec.position, tensors, rt)
        if not hasattr(self.position, "rotary_table"):
            raise ValueError(f"position encoding {spec.position.kind!r} does not rotate queries and keys "
                             f"(no rotary_table); give it the model's embedding_position seat instead")
        self.scale = spec.softmax_scale if spec.softmax_scale is not None else spec.head_dim ** -0.5
        self.prefill_heads = spec.num_heads      # work items per block of prompt tokens (see parts/base.py)

    @staticmethod
    def expected_tensors(spec: AttentionSpec, prefix: str) -> dict[str, TensorReq]:
        h, d = spec.hidden_size, spec.head_dim
        out = {
            prefix + "q_proj.weight": TensorReq((spec.num_heads * d, h)),
            prefix + "o_proj.weight": TensorReq((h, spec.num_heads * d)),
        }
        if spec.own_kv:
            out[prefix + "k_proj.weight"] = TensorReq((spec.num_kv_heads * d, h))
            out[prefix + "v_proj.weight"] = TensorReq((spec.num_kv_heads * d, h))
        if spec.qk_norm_eps is not None:
            out[prefix + "q_norm.weight"] = TensorReq((d,), role="vector")
            if spec.own_kv:
                out[prefix + "k_norm.weight"] = TensorReq((d,), role="vector")
        out.update(POSITIONS.get(spec.position.kind).expected_tensors(spec.position))
        return out

    def cache_need(self) -> KVPagesNeed:
        return KVPagesNeed(self.spec.num_kv_heads, self.spec.head_dim, self.spec.window)

    def GRAPH_SAFE(self) -> bool:
        return graph_safe(self.position)

    def weight_bytes(self) -> int:
        return tensor_bytes(self.w_qkv, self.w_o, self.q_norm_w, self.k_norm_w)

    TAKES_OWED_NORM = True     # the q|k|v product pays an owed norm scale in its epilogue
    TAKES_THEN_NORM = True     # the output product can add itself to the residual stream

    def forward(self, h, step, cache_view, then_norm=None):
        spec = self.spec
        n = h.shape[0]
        q = torch.empty((n, spec.num_heads, spec.head_dim), dtype=h.dtype, device=h.device)
        table, rotary_dim = self.position.rotary_table(step)
        if (h.dtype == torch.bfloat16 and n <= SWAPPED_GEMM_MAX_TOKENS and spec.own_kv
                and spec.head_dim == ops.QKV_ROPE_HEAD_DIM and rotary_dim in (0, spec.head_dim)
                and spec.hidden_size % 8 == 0 and cache_view.k.dtype == torch.bfloat16):
            # few tokens and heads that are whole tiles: norm, rotation and page write ride in
            # the product's epilogue
            splits, stages, _ = ops.swapped_gemm_plan(self.w_qkv.shape[0], spec.hidden_size, n)
            colscale, x = ((h.sumsq, h.dim, h.eps), h.xb) if isinstance(h, OwedNorm) else (None, h)
            ops.gemm_qkv_rope(self.w_qkv, x, step.err, splits, q, cache_view.k, cache_view.v, step.positions,
                              step.tok_req, step.req_slot, cache_view.table, self.q_norm_w, self.k_norm_w,
                              table, n_q_heads=spec.num_heads, n_kv_heads=spec.num_kv_heads,
                              eps=spec.qk_norm_eps or 0.0, max_stages=stages, colscale=colscale,
                              req_q_len=step.req_q_len, req_kv_len=step.req_kv_len, chain=chain_of(step))
        else:
            self._project_and_rotate(h, q, table, rotary_dim, step, cache_view)
        out = torch.empty_like(q)
        paged_attention(q, out, cache_view, step, scale=self.scale, window=spec.window)
        return linear(out.view(n, spec.num_heads * spec.head_dim), self.w_o, err=step.err, then_norm=then_norm,
                      chain=chain_of(step))

    def _project_and_rotate(self, h, q, table, rotary_dim, step, cache_view) -> None:
        """The q|k|v product, then norm, rotation and page write in a kernel of their own."""
        spec = self.spec
        qkv = linear(h, self.w_qkv, err=step.err)
        ops.rope_kv(qkv, q, cache_view.k if spec.own_kv else None,
                    cache_view.v if spec.own_kv else None,
                    step.positions, step.tok_req, step.req_slot, cache_view.table,
                    self.q_norm_w, self.k_norm_w, table, step.err,
                    n_q_heads=spec.num_heads, n_kv_heads=spec.num_kv_heads, head_dim=spec.head_dim,
                    rotary_dim=rotary_dim, eps=spec.qk_norm_eps or 0.0, write_kv=spec.own_kv,
                    req_q_len=step.req_q_len, req_kv_len=step.req_kv_len)


@dataclass(frozen=True)
class CappedAttentionSpec:
    """Sizes and constants of an attention mixer with the options of :class:`CappedAttention`.

    ``head_dim`` is the size of a query or key head, ``v_head_dim`` of a value head.
    ``unit_norm_eps`` switches the weightless RMS norm of the rotated q and k heads on.
    ``softcap`` of ``None``: scores are not capped.  ``sinks``: one learned number per query head
    joins the softmax denominator.  ``value_mix`` is ``None``, ``"source"`` (this layer's raw
    values are kept for later layers of the step under the key ``value_mix_key``) or ``"blend"``
    (this layer's values are blended with the kept ones by its learned ``mix`` scalar).
    The ``*_name`` fields are the tensors' names after the part's prefix.
    """

    hidden_size: int
    num_heads: int
    num_kv_heads: int
    head_dim: int
    v_head_dim: int
    position: object
    softmax_scale: float
    unit_norm_eps: float | None = None
    window: int | None = None
    softcap: float | None = None
    sinks: bool = False
    value_mix: str | None = None
    value_mix_key: str = "value_mix"
    q_name: str = "q"
    k_name: str = "k"
    v_name: str = "v"
    o_name: str = "o"
    sink_name: str = "sink"
    mix_name: str = "vmix"
    kind: str = "attention_capped"


@MIXERS.register("attention_capped")
class CappedAttention:
    """Grouped-query attention over paged keys and values with a set of options that several
    designs share: value heads of their own size, rotation of neighbouring pairs over part of the
    head, a unit RMS norm of q and k after the rotation, scores bounded by ``cap * tanh(s / cap)``,
    a sliding window, a sink in the softmax denominator, and values blended with those of the
    first blending layer (``v <- (1 - lambda) v + lambda v_first``; the blended values are what
    the pages hold).  Query head ``h`` reads key/value head ``h // (Hq / Hkv)``.

    The q, k and v matrices are stacked into one operand.  Rotation, norm, blend and page write
    are one kernel (``csrc/qkv_pairs.cu``); scores, softmax and the weighted sum run in float32
    inside the attention kernels.
    """

    def __init__(self, spec: CappedAttentionSpec, prefix: str, tensors: dict[str, torch.Tensor], rt: Runtime):
        if spec.num_heads % spec.num_kv_heads:
            raise ValueError(f"{spec.num_heads} query heads are not a multiple of "
                             f"{spec.num_kv_heads} key/value heads")
        if max(spec.head_dim, spec.v_head_dim) > 256 or spec.head_dim % 2 or spec.v_head_dim % 2:
            raise ValueError(f"head sizes {spec.head_dim} / {spec.v_head_dim} are not taken by the attention "
                             f"kernels: they need even sizes up to 256")
        if spec.value_mix not in (None, "source", "blend"):
            raise ValueError(f"value_mix must be None, 'source' or 'blend', got {spec.value_mix!r}")
        self.spec = spec
        self.rt = rt
        self.w_qkv = torch.cat([tensors[prefix + spec.q_name], tensors[prefix + spec.k_name],
                                tensors[prefix + spec.v_name]], dim=0).contiguous()
        self.w_o = tensors[prefix + spec.o_name]
        self.sinks = tensors[prefix + spec.sink_name].contiguous() if spec.sinks else None
        self.mix = tensors[prefix + spec.mix_name].reshape(1).contiguous() if spec.value_mix == "blend" else None
        self.position = POSITIONS.get(spec.position.kind)(spec.position, tensors, rt)
        if getattr(self.position, "PAIRING", None) != "neighbours":
            raise ValueError(f"position encoding {spec.position.kind!r} does not rotate neighbouring pairs")
        self.prefill_heads = spec.num_heads

    @staticmethod
    def expected_tensors(spec: CappedAttentionSpec, prefix: str) -> dict[str, TensorReq]:
        h, d, dv = spec.hidden_size, spec.head_dim, spec.v_head_dim
        out = {
            prefix + spec.q_name: TensorReq((spec.num_heads * d, h)),
            prefix + spec.k_name: TensorReq((spec.num_kv_heads * d, h)),
            prefix + spec.v_name: TensorReq((spec.num_kv_heads * dv, h)),
            prefix + spec.o_name: TensorReq((h, spec.num_heads * dv)),
        }
        if spec.sinks:
            out[prefix + spec.sink_name] = TensorReq((spec.num_heads,), role="bias")
        if spec.value_mix is not None:
            # the source layer's scalar is stored too; it is loaded and never read
            out[prefix + spec.mix_name] = TensorReq((), role="fraction")
        out.update(POSITIONS.get(spec.position.kind).expected_tensors(spec.position))
        return out

    def cache_need(self) -> KVPagesNeed:
        s = self.spec
        return KVPagesNeed(s.num_kv_heads, s.head_dim, s.window, None if s.v_head_dim == s.head_dim else s.v_head_dim)

    def GRAPH_SAFE(self) -> bool:
        return graph_safe(self.position)

    def weight_bytes(self) -> int:
        return tensor_bytes(self.w_qkv, self.w_o, self.sinks, self.mix)

    def forward(self, h, step, cache_view):
        spec = self.spec
        n = h.shape[0]
        qkv = linear(h, self.w_qkv, err=step.err)
        q = torch.empty((n, spec.num_heads, spec.head_dim), dtype=h.dtype, device=h.device)
        table, rotary_dim = self.position.rotary_table(step)
        v_in = v_out = None
        key = ("value_mix", spec.value_mix_key)
        if spec.value_mix == "source":
            v_out = torch.empty((n, spec.num_kv_heads * spec.v_head_dim), dtype=torch.float32, device=h.device)
            step.scratch[key] = v_out
        elif spec.value_mix == "blend":
            v_in = step.scratch.get(key)
            if v_in is None or v_in.shape != (n, spec.num_kv_heads * spec.v_head_dim):
                raise RuntimeError("a blending attention layer ran before the layer whose values it blends with, "
                                   "or their value heads differ in number or size")
        ops.qkv_pairs(qkv, q, cache_view.k, cache_view.v, step.positions, step.tok_req, step.req_slot,
                      cache_view.table, table, step.err, n_q_heads=spec.num_heads, n_kv_heads=spec.num_kv_heads,
                      rotary_dim=rotary_dim, unit_norm_eps=spec.unit_norm_eps, v_first_in=v_in, v_lambda=self.mix,
                      v_first_out=v_out, req_q_len=step.req_q_len, req_kv_len=step.req_kv_len)
        out = torch.empty((n, spec.num_heads, spec.v_head_dim), dtype=h.dtype, device=h.device)
        paged_attention(q, out, cache_view, step, scale=spec.softmax_scale, window=spec.window,
                        softcap=spec.softcap, sinks=self.sinks)
        return linear(out.view(n, spec.num_heads * spec.v_head_dim), self.w_o, err=step.err)


@dataclass(frozen=True)
class RowNormAttentionSpec:
    """Sizes and constants of an attention mixer with the options of :class:`RowNormAttention`.

    ``bias``: q, k and v projections have biases.  ``row_norm_eps`` switches the RMS norm over the *whole*
    query projection of a token (all heads at once, a weight per channel) and over the whole key projection
    on.  ``chunk``: a query sees only the keys of its own block of that many positions.  ``slope_exponent``:
    the score of a key ``n`` positions behind the query loses ``slope_h * n`` with
    ``slope_h = 2 ** (-slope_exponent * (h + 1) / heads)`` (``None``: no distance bias).  ``sinks``: a learned
    number per query head joins the softmax denominator.  ``gate``: the concatenated heads are multiplied by
    ``sigmoid(W_g h)``.  The ``*_name`` fields are the tensors' names after the part's prefix.
    """

    hidden_size: int
    num_heads: int
    num_kv_heads: int
    head_dim: int
    v_head_dim: int
    softmax_scale: float
    bias: bool = True
    row_norm_eps: float | None = None
    chunk: int | None = None
    window: int | None = None
    slope_exponent: float | None = None
    sinks: bool = False
    gate: bool = False
    q_name: str = "q"
    k_name: str = "k"
    v_name: str = "v"
    o_name: str = "o"
    gate_name: str = "g"
    bias_suffix: str = ".b"
    norm_suffix: str = ".norm"
    sink_name: str = "sink"
    kind: str = "attention_rownorm"


@MIXERS.register("attention_rownorm")
class RowNormAttention:
    """Grouped-query attention over paged keys and values without rotation: positions enter through a
    distance bias on the scores and through a chunked mask.  Query head ``h`` reads key/value head
    ``h // (Hq / Hkv)``; ``score = (q . k) * scale - slope_h * (i - j)``; position ``i`` sees ``j <= i`` of its own
    chunk (chunks are counted from position 0 of the sequence, wherever a prompt was cut); the softmax
    denominator also holds ``exp(sink_h)``.

    The q, k, v and gate matrices are one stacked operand.  Biases, row norms and the page write are one
    kernel (``csrc/qkv_rownorm.cu``); scores, bias, softmax and the weighted sum run in float32 inside the
    attention kernel; the gate and the caller's factor are one kernel.  :meth:`branch` writes the rows in
    front of the output projection into a buffer of the caller's (see :class:`~tokamak_b200.parts.parallel.ParallelMixer`).
    """

    GRAPH_SAFE = True

    def __init__(self, spec: RowNormAttentionSpec, prefix: str, tensors: dict[str, torch.Tensor], rt: Runtime):
        if spec.num_heads % spec.num_kv_heads:
            raise ValueError(f"{spec.num_heads} query heads are not a multiple of "
                             f"{spec.num_kv_heads} key/value heads")
        if max(spec.head_dim, spec.v_head_dim) > 1024:
            raise ValueError(f"head sizes {spec.head_dim} / {spec.v_head_dim} are beyond the attention kernel's 1024")
        if spec.chunk is not None and spec.chunk < 1:
            raise ValueError(f"a chunk of {spec.chunk} positions is none")
        self.spec = spec
        self.rt = rt
        t = lambda name: tensors[prefix + name]
        mats = [t(spec.q_name), t(spec.k_name), t(spec.v_name)] + ([t(spec.gate_name)] if spec.gate else [])
        self.w_in = torch.cat(mats, dim=0).contiguous()
        nq, nk = spec.num_heads * spec.head_dim, spec.num_kv_heads * spec.head_dim
        self.q_off, self.k_off, self.v_off = 0, nq, nq + nk
        self.g_off = nq + nk + spec.num_kv_heads * spec.v_head_dim
        vec = lambda name: t(name).contiguous()
        self.q_bias = vec(spec.q_name + spec.bias_suffix) if spec.bias else None
        self.k_bias = vec(spec.k_name + spec.bias_suffix) if spec.bias else None
        self.v_bias = vec(spec.v_name + spec.bias_suffix) if spec.bias else None
        self.q_norm = vec(spec.q_name + spec.norm_suffix) if spec.row_norm_eps is not None else None
        self.k_norm = vec(spec.k_name + spec.norm_suffix) if spec.row_norm_eps is not None else None
        self.sinks = vec(spec.sink_name) if spec.sinks else None
        self.slopes = None
        if spec.slope_exponent is not None:
            heads = torch.arange(1, spec.num_heads + 1, dtype=torch.float64)
            self.slopes = torch.pow(2.0, -spec.slope_exponent * heads / spec.num_heads).to(torch.float32).to(rt.device)
        self.w_o = t(spec.o_name)
        self.out_width = spec.num_heads * spec.v_head_dim
        self.prefill_heads = spec.num_heads

    @staticmethod
    def expected_tensors(spec: RowNormAttentionSpec, prefix: str) -> dict[str, TensorReq]:
        h, d, dv = spec.hidden_size, spec.head_dim, spec.v_head_dim
        nq, nk, nv = spec.num_heads * d, spec.num_kv_heads * d, spec.num_kv_heads * dv
        out = {}
        for name, rows in ((spec.q_name, nq), (spec.k_name, nk), (spec.v_name, nv)):
            out[prefix + name] = TensorReq((rows, h))
            if spec.bias:
                out[prefix + name + spec.bias_suffix] = TensorReq((rows,), role="bias")
        if spec.row_norm_eps is not None:
            out[prefix + spec.q_name + spec.norm_suffix] = TensorReq((nq,), role="vector")
            out[prefix + spec.k_name + spec.norm_suffix] = TensorReq((nk,), role="vector")
        if spec.sinks:
            out[prefix + spec.sink_name] = TensorReq((spec.num_heads,), role="bias")
        if spec.gate:
            out[prefix + spec.gate_name] = TensorReq((spec.num_heads * dv, h))
        out[prefix + spec.o_name] = TensorReq((h, spec.num_heads * dv))
        return out

    def cache_need(self) -> KVPagesNeed:
        s = self.spec
        return KVPagesNeed(s.num_kv_heads, s.head_dim, s.window, None if s.v_head_dim == s.head_dim else s.v_head_dim)

    def weight_bytes(self) -> int:
        return tensor_bytes(self.w_in, self.w_o, self.q_bias, self.k_bias, self.v_bias, self.q_norm, self.k_norm,
                            self.sinks)

    def branch(self, h, step, cache_view, out: torch.Tensor | None = None, out_scale: float = 1.0) -> torch.Tensor:
        spec = self.spec
        n = h.shape[0]
        proj = linear(h, self.w_in, err=step.err)
        q = torch.empty((n, spec.num_heads, spec.head_dim), dtype=h.dtype, device=h.device)
        ops.qkv_rownorm(proj, q, cache_view.k, cache_view.v, step, cache_view.table, q_off=self.q_off,
                        k_off=self.k_off, v_off=self.v_off, q_bias=self.q_bias, k_bias=self.k_bias,
                        v_bias=self.v_bias, q_norm=self.q_norm, k_norm=self.k_norm, eps=spec.row_norm_eps or 0.0)
        att = torch.empty((n, spec.num_heads, spec.v_head_dim), dtype=h.dtype, device=h.device)
        paged_attention(q, att, cache_view, step, scale=spec.softmax_scale, window=spec.window, sinks=self.sinks,
                        chunk=spec.chunk, slopes=self.slopes)
        att = att.view(n, self.out_width)
        if not spec.gate:
            if out is None and out_scale == 1.0:
                return att
            res = att.float().mul_(out_scale).to(h.dtype)
            if out is None:
                return res
            out.copy_(res)
            return out
        return ops.gate_scale(att, proj, self.g_off, out=out, scale=out_scale)

    def forward(self, h, step, cache_view):
        return linear(self.branch(h, step, cache_view), self.w_o, err=step.err)


def bucketed_distance_table(rel: torch.Tensor, far: int) -> torch.Tensor:
    """A learned bias by bucketed distance, laid out distance by distance: ``[heads, far + 1]`` float32 with
    ``out[h, n] = rel[bucket(n), h]``.  ``rel`` has ``B`` rows; distances below ``B / 2`` have a bucket each, the
    further ones share the rest on a logarithmic scale that reaches the last bucket at ``far``:
    ``bucket(n) = B/2 + floor(ln(n / (B/2)) / ln(far / (B/2)) * (B - B/2))``, at most ``B - 1``; every distance from
    ``far`` on has the last bucket, so a reader clamps the distance to the table's last column."""
    import math
    rows, heads = rel.shape
    half = rows // 2
    if half < 1 or far <= half:
        raise ValueError(f"{rows} buckets up to distance {far}: the logarithmic part is empty")
    idx = []
    for n in range(far + 1):
        if n < half:
            idx.append(n)
        else:
            idx.append(min(rows - 1, half + int(math.floor(math.log(n / half) / math.log(far / half) * (rows - half)))))
    index = torch.tensor(idx, dtype=torch.long, device=rel.device)
    return rel.float().index_select(0, index).t().contiguous()


@dataclass(frozen=True)
class GatedAttentionSpec:
    """Sizes and constants of an attention mixer with the options of :class:`GatedAttention`.

    ``bias``: the q, k and v projections have biases.  ``values_from_keys``: there is no value projection; the
    values are the key projection as it is before norm and rotation.  ``head_norm_eps``: q and k heads are RMS
    normed, with a weight of one head's size shared by all heads (``head_norm_weight``) or none.  ``position``: a
    position spec whose part rotates neighbouring pairs or halves, or ``none``.  ``q_temp`` ``(coef, every)``: the
    query at position ``p`` is multiplied by ``1 + coef * ln(floor((p + 1) / every) + 1)``.  ``softcap``: scores
    are bounded by ``cap * tanh(s / cap)``.  ``unit_sink``: one is added to every softmax denominator (a sink of
    score 0 without a value).  ``rel_far``: a learned bias ``rel[bucket(i - j), h]`` joins the score, see
    :func:`bucketed_distance_table`; the table's rows are read from the checkpoint.  ``gate``: ``"head"`` (one
    sigmoid gate per head) or ``"channel"`` (one per output channel) or ``None``.  The ``*_name`` fields are the
    tensors' names after the part's prefix."""

    hidden_size: int
    num_heads: int
    num_kv_heads: int
    head_dim: int
    v_head_dim: int
    softmax_scale: float
    position: object
    bias: bool = False
    values_from_keys: bool = False
    head_norm_eps: float | None = None
    head_norm_weight: bool = True
    q_temp: tuple | None = None
    softcap: float | None = None
    unit_sink: bool = False
    rel_far: int | None = None
    rel_rows: int | None = None
    gate: str | None = None
    window: int | None = None
    q_name: str = "q"
    k_name: str = "k"
    v_name: str = "v"
    o_name: str = "o"
    gate_name: str = "g"
    rel_name: str = "rel"
    bias_suffix: str = ".b"
    norm_suffix: str = ".norm"
    kind: str = "attention_gated"


@MIXERS.register("attention_gated")
class GatedAttention:
    """Grouped-query attention over paged keys and values; query head ``h`` reads key/value head
    ``h // (Hq / Hkv)``; ``score = (q . k) * scale``, capped, plus the distance bias; causal; the softmax
    denominator may hold one more term ``exp(0)``; the heads are gated by ``sigmoid(W_g h)`` before the output
    projection.

    The q, k, v and gate matrices are one stacked operand.  Biases, head norms, the query temperature, the
    rotation and the page write are one kernel (``csrc/qkv_heads.cu``); scores, cap, bias, softmax and the
    weighted sum run in float32 inside the attention kernel; gate and the caller's factor are one kernel.
    :meth:`branch` writes the rows in front of the output projection into a buffer of the caller's (see
    :class:`~tokamak_b200.parts.parallel.ParallelMixer`)."""

    def __init__(self, spec: GatedAttentionSpec, prefix: str, tensors: dict[str, torch.Tensor], rt: Runtime):
        if spec.num_heads % spec.num_kv_heads:
            raise ValueError(f"{spec.num_heads} query heads are not a multiple of "
                             f"{spec.num_kv_heads} key/value heads")
        if max(spec.head_dim, spec.v_head_dim) > 512:
            raise ValueError(f"head sizes {spec.head_dim} / {spec.v_head_dim} are beyond the kernels' 512")
        if spec.values_from_keys and spec.v_head_dim != spec.head_dim:
            raise ValueError("values that are the keys have the keys' size")
        if spec.gate not in (None, "head", "channel"):
            raise ValueError(f"gate must be None, 'head' or 'channel', got {spec.gate!r}")
        self.spec = spec
        self.rt = rt
        t = lambda name: tensors[prefix + name]
        mats = [t(spec.q_name), t(spec.k_name)] + ([] if spec.values_from_keys else [t(spec.v_name)])
        nq, nk = spec.num_heads * spec.head_dim, spec.num_kv_heads * spec.head_dim
        nv = 0 if spec.values_from_keys else spec.num_kv_heads * spec.v_head_dim
        self.q_off, self.k_off = 0, nq
        self.v_off = None if spec.values_from_keys else nq + nk
        self.g_off = nq + nk + nv
        if spec.gate is not None:
            mats.append(t(spec.gate_name))
        self.w_in = torch.cat(mats, dim=0).contiguous()
        vec = lambda name: t(name).contiguous()
        self.q_bias = vec(spec.q_name + spec.bias_suffix) if spec.bias else None
        self.k_bias = vec(spec.k_name + spec.bias_suffix) if spec.bias else None
        self.v_bias = vec(spec.v_name + spec.bias_suffix) if spec.bias and not spec.values_from_keys else None
        normed = spec.head_norm_eps is not None and spec.head_norm_weight
        self.q_norm = vec(spec.q_name + spec.norm_suffix) if normed else None
        self.k_norm = vec(spec.k_name + spec.norm_suffix) if normed else None
        self.sinks = torch.zeros(spec.num_heads, dtype=torch.float32, device=rt.device) if spec.unit_sink else None
        self.dist_bias = bucketed_distance_table(t(spec.rel_name), spec.rel_far) if spec.rel_far is not None else None
        self.position = POSITIONS.get(spec.position.kind)(spec.position, tensors, rt)
        if not hasattr(self.position, "rotary_table"):
            raise ValueError(f"position encoding {spec.position.kind!r} does not rotate queries and keys")
        self.halves = getattr(self.position, "PAIRING", "halves") == "halves"
        self.w_o = t(spec.o_name)
        self.out_width = spec.num_heads * spec.v_head_dim
        self.prefill_heads = spec.num_heads

    @staticmethod
    def expected_tensors(spec: GatedAttentionSpec, prefix: str) -> dict[str, TensorReq]:
        h, d, dv = spec.hidden_size, spec.head_dim, spec.v_head_dim
        sizes = [(spec.q_name, spec.num_heads * d), (spec.k_name, spec.num_kv_heads * d)]
        if not spec.values_from_keys:
            sizes.append((spec.v_name, spec.num_kv_heads * dv))
        out = {}
        for name, rows in sizes:
            out[prefix + name] = TensorReq((rows, h))
            if spec.bias:
                out[prefix + name + spec.bias_suffix] = TensorReq((rows,), role="bias")
        if spec.head_norm_eps is not None and spec.head_norm_weight:
            out[prefix + spec.q_name + spec.norm_suffix] = TensorReq((d,), role="vector")
            out[prefix + spec.k_name + spec.norm_suffix] = TensorReq((d,), role="vector")
        if spec.rel_far is not None:
            out[prefix + spec.rel_name] = TensorReq((spec.rel_rows, spec.num_heads), role="bias")
        if spec.gate is not None:
            out[prefix + spec.gate_name] = TensorReq((spec.num_heads if spec.gate == "head" else spec.num_heads * dv, h))
        out[prefix + spec.o_name] = TensorReq((h, spec.num_heads * dv))
        out.update(POSITIONS.get(spec.position.kind).expected_tensors(spec.position))
        return out

    def cache_need(self) -> KVPagesNeed:
        s = self.spec
        return KVPagesNeed(s.num_kv_heads, s.head_dim, s.window, None if s.v_head_dim == s.head_dim else s.v_head_dim)

    def GRAPH_SAFE(self) -> bool:
        return graph_safe(self.position)

    def weight_bytes(self) -> int:
        return tensor_bytes(self.w_in, self.w_o, self.q_bias, self.k_bias, self.v_bias, self.q_norm, self.k_norm,
                            self.dist_bias)

    TAKES_PROJ = True      # the stacked input projection may be part of a wider product (see ParallelMixer)

    def branch(self, h, step, cache_view, out: torch.Tensor | None = None, out_scale: float = 1.0, proj=None,
               proj_off: int = 0) -> torch.Tensor:
        """The rows in front of the output projection, times ``out_scale``, into ``out`` or a new tensor.  ``proj``:
        a product of ``h`` that holds this part's input projection in its columns from ``proj_off`` on."""
        spec = self.spec
        n = h.shape[0]
        if proj is None:
            proj, proj_off = linear(h, self.w_in, err=step.err), 0
        q = torch.empty((n, spec.num_heads, spec.head_dim), dtype=h.dtype, device=h.device)
        table, rotary_dim = self.position.rotary_table(step)
        coef, every = spec.q_temp if spec.q_temp is not None else (0.0, 0)
        ops.qkv_heads(proj, q, cache_view.k, cache_view.v, step, cache_view.table, q_off=proj_off + self.q_off,
                      k_off=proj_off + self.k_off, v_off=None if self.v_off is None else proj_off + self.v_off,
                      q_bias=self.q_bias, k_bias=self.k_bias, v_bias=self.v_bias,
                      head_norm_eps=spec.head_norm_eps, q_norm=self.q_norm, k_norm=self.k_norm, table=table,
                      rotary_dim=rotary_dim, halves=self.halves, temp_coef=coef, temp_every=every)
        att = torch.empty((n, spec.num_heads, spec.v_head_dim), dtype=h.dtype, device=h.device)
        paged_attention(q, att, cache_view, step, scale=spec.softmax_scale, window=spec.window, softcap=spec.softcap,
                        sinks=self.sinks, dist_bias=self.dist_bias)
        att = att.view(n, self.out_width)
        if spec.gate is None:
            if out is None and out_scale == 1.0:
                return att
            res = att.float().mul_(out_scale).to(h.dtype)
            if out is None:
                return res
            out.copy_(res)
            return out
        return ops.gate_scale(att, proj, proj_off + self.g_off, out=out, scale=out_scale,
                              gate_group=spec.v_head_dim if spec.gate == "head" else 1)

    def forward(self, h, step, cache_view):
        return linear(self.branch(h, step, cache_view), self.w_o, err=step.err)


_SIDE: dict = {}


def _side_stream(device: torch.device):
    """A second stream of the device and the two events that fork to it and join from it."""
    entry = _SIDE.get(device)
    if entry is None:
        entry = (torch.cuda.Stream(device), torch.cuda.Event(), torch.cuda.Event())
        _SIDE[device] = entry
    return entry


def paged_attention(q: torch.Tensor, out: torch.Tensor, cache_view, step, *, scale: float,
                    window: int | None, softcap: float | None = None, sinks: torch.Tensor | None = None,
                    chunk: int | None = None, slopes: torch.Tensor | None = None,
                    dist_bias: torch.Tensor | None = None) -> None:
    """Attention of every token of the step over the pages of its own request.

    ``softcap`` bounds the scaled scores by ``cap * tanh(score / cap)``; ``sinks`` (float32, one per
    query head) adds ``exp(sink)`` to every softmax denominator.  ``out`` is ``[N, Hq, dv]`` where
    the value heads have a size of their own.  ``chunk`` (a query sees only its own block of that many
    positions) and ``slopes`` (a distance bias per query head) are known to the general kernel, the decode
    kernels and the tcgen05 prefill kernel.  ``dist_bias`` (float32 ``[Hq, L]``: the score of the key ``n``
    positions back gains ``dist_bias[h, min(n, L - 1)]``) is known to the same kernels.

    Chooses the kernels.  A latent cache in bfloat16 goes to the tensor-core kernel that stacks the heads
    of a token (``csrc/attention_latent.cu``).  bfloat16 with a head_dim the tiled kernels take: single next
    tokens go to the split-K decode kernel, portions of prompts to the tcgen05 flash
    prefill kernel (or to the mma.sync one for page sizes it does not take).  float32,
    and every other shape, runs on the general kernel.
    """
    ops.flush_chains()     # q and the pages may come from a product that is still queued: launch it on this stream
    n, hq, d = q.shape
    hkv, page = cache_view.k.shape[1], cache_view.k.shape[2]
    bf16 = q.dtype == torch.bfloat16
    n_dec = step.decode_items.numel()
    n_pf = step.prefill_items.numel()
    dv = cache_view.v.shape[3]
    if (hkv == 1 and cache_view.k.dtype == torch.bfloat16 and cache_view.v.data_ptr() == cache_view.k.data_ptr()
            and cache_view.v.stride(2) == d and softcap is None and ops.latent_kernel_takes(d, dv)):
        # a latent cache (one row a position for all heads, the values inside the keys): the heads of a
        # token are rows of one tile of the tensor-core kernel, which reads every key once for all of them
        if n_dec:
            ops.attention_latent(q, out, cache_view.k, dv, step, cache_view.table, scale=scale, window=window, sinks=sinks,
                                 items=step.decode_items,
                                 n_splits=ops.latent_decode_splits(q.device, n_dec, step.max_kv_len, window))
        if n_pf:
            ops.attention_latent(q, out, cache_view.k, dv, step, cache_view.table, scale=scale, window=window, sinks=sinks,
                                 tiles=step.prefill_tiles)
        return
    # the tiled kernels take heads of one size for keys and values; of the two prefill kernels the
    # tcgen05 one knows caps and sinks
    same_size = cache_view.v.shape[3] == d
    extras = (softcap is not None or sinks is not None or chunk is not None or slopes is not None
              or dist_bias is not None)
    # a single token sees no more keys than its chunk holds: the kernels' work is planned for that many
    dec_span = step.max_kv_len if chunk is None else min(step.max_kv_len, chunk)
    tiled = bf16 and same_size
    dec_tiled = tiled and n_dec > 0 and ops.decode_kernel_takes(hq, hkv, d, page)
    pf_tiled = (tiled and n_pf > 0 and ops.prefill_kernel_takes(hq, hkv, d, page)
                and (not extras or ops.prefill_tc_kernel_takes(hq, hkv, d, page)))
    # In a mixed step the two kernels touch different tokens.  One portion against a long context
    # is few blocks (one per pair of 128-row query tiles and head), so the decode kernel runs
    # beside it on a second stream instead of after it.
    beside = dec_tiled and pf_tiled and not torch.cuda.is_current_stream_capturing()
    if beside:
        side, fork, join = _side_stream(q.device)
        fork.record()
        side.wait_event(fork)
    if dec_tiled:
        with torch.cuda.stream(side) if beside else contextlib.nullcontext():
            if ops.decode_uses_balanced(q.device, n_dec, hkv, dec_span):
                ops.attention_decode_balanced(q, out, cache_view.k, cache_view.v, step.decode_items, step.positions,
                                              step.tok_req, step.req_slot, cache_view.table, step.err, scale=scale,
                                              window=window, softcap=softcap, sinks=sinks, chunk=chunk, slopes=slopes,
                                              dist_bias=dist_bias, blocks=ops.decode_balanced_blocks(q.device, n_dec, hkv, dec_span))
            else:
                ops.attention_decode(q, out, cache_view.k, cache_view.v, step.decode_items, step.positions,
                                     step.tok_req, step.req_slot, cache_view.table, step.err, scale=scale,
                                     window=window, softcap=softcap, sinks=sinks, chunk=chunk, slopes=slopes,
                                     dist_bias=dist_bias, n_splits=ops.decode_splits(n_dec, hkv, dec_span))
            if beside:
                join.record()
    if pf_tiled and ops.prefill_tc_kernel_takes(hq, hkv, d, page):
        ops.attention_prefill_tc(q, out, cache_view.k, cache_view.v, step.prefill_tc,
                                 cache_view.table, step.err, scale=scale, window=window, softcap=softcap,
                                 sinks=sinks, chunk=chunk, slopes=slopes, dist_bias=dist_bias)
    elif pf_tiled:
        ops.attention_prefill(q, out, cache_view.k, cache_view.v, step.prefill_tiles,
                              step.req_q_start, step.req_q_len, step.req_kv_len, step.req_slot,
                              cache_view.table, step.err, scale=scale, window=window)
    if beside:
        torch.cuda.current_stream().wait_event(join)
    dec_rest = n_dec > 0 and not dec_tiled
    pf_rest = n_pf > 0 and not pf_tiled
    if dec_rest or pf_rest:
        items = None if (dec_rest and pf_rest) else (step.decode_items if dec_rest else step.prefill_items)
        ops.attention_plain(q, out, cache_view.k, cache_view.v, step.positions, step.tok_req,
                            step.req_slot, cache_view.table, step.err, scale=scale, window=window,
                            items=items, softcap=softcap, sinks=sinks, chunk=chunk, slopes=slopes,
                            dist_bias=dist_bias)
