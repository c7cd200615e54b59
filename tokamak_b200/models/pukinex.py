"""The Pukinex decoder as a :class:`ModelSpec`.

A stack of pre-norm blocks (layer norms with weight and bias) whose residual stream may be kept in
several copies with learned connections between them (``streams``: every sublayer reads a weighted sum of
the copies and writes its output, times ``residual_mult``, back to all of them while they are mixed among
themselves); a span of the layers may run several times in a row with the same weights and a cache of its
own per pass (``loop``).  The embedding is scaled, the head untied, the logits scaled and capped.  The
mixers, listed layer by layer in ``config.json``:

* ``attention``: grouped-query attention whose values are the unrotated keys (no value projection),
  neighbouring-pair rotation on part of the head with linearly scaled positions, capped scores, one added
  to the softmax denominator, a sigmoid gate per head.
* ``parallel``: two mixers side by side, added with a factor each.  Left: attention without rotation, with
  biases, q and k normed per head (one weight for all heads), a query temperature that grows with the
  logarithm of the position, a learned bias by bucketed distance, one added to the denominator, a sigmoid
  gate per channel.  Right: retention (a fixed decay per head, half-split rotation, scaled keys, unit
  root mean square per head, a silu gate).

Feed-forwards are ungated, ``W_down relu(W_up h)^2``; a layer may lack its feed-forward.

    {"architecture": "Pukinex", "vocab": V, "width": W, "norm": {"eps": e}, "embedding": {"scale": s},
     "residual_mult": m, "streams": S, "loop": {"start": a, "stop": b, "times": n},
     "logit_scale": c, "logit_softcap": cap,
     "layers": [{"type": "attention", "mixer": {"heads", "kv_heads", "dim", "vdim", "scale", "softcap",
                                                "rot": {"base", "dims", "scaling": {"factor"}}}, "mlp": ...},
                {"type": "parallel", "mixer": {"left": {"heads", "kv_heads", "dim", "vdim", "scale", "bias_max",
                                                        "q_temp": {"coef", "every"}},
                                               "right": {"heads", "dim", "vdim", "decay": [...], "rot": {"base", "dims"}},
                                               "left_scale", "right_scale"}, "mlp": ...}]}
    mlp: {"kind": "dense", "ff": F} | null

Tensors are ``embed``, ``head``, ``final.norm`` (+ ``.b``) and, for layer ``i``, ``l<i>.norm1``, ``l<i>.norm2`` (+ ``.b``),
``l<i>.mix.*``, ``l<i>.mlp.up`` / ``down`` and, with ``streams``, ``l<i>.hc1.*`` / ``l<i>.hc2.*`` (``in``, ``out``, ``mix``).
The number of distance buckets of a left half is the row count of its ``rel`` table: it is read from the
checkpoint's header or, for a folder of random weights, from the optional key ``left.bias_buckets``.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Mapping

from ..config.model_config import ConfigError
from ..parts.attention import GatedAttentionSpec
from ..parts.block import HyperBlockSpec
from ..parts.embedding import EmbeddingSpec, HeadSpec
from ..parts.feedforward import MlpSpec
from ..parts.norm import LayerNormSpec
from ..parts.parallel import ParallelMixerSpec
from ..parts.position import NoPositionSpec, RopeHalvesSpec, RopePairsSpec
from ..parts.retention import RetentionSpec
from .decoder import LayerCall, ModelSpec

ARCHITECTURE = "Pukinex"
DEFAULT_MAX_POSITIONS = 1 << 17     # the design has no limit of its own
DEFAULT_BUCKETS = 16
MAX_STREAMS = 8


@dataclass(frozen=True)
class Rotation:
    dims: int
    base: float
    factor: float


@dataclass(frozen=True)
class AttentionLayer:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    softcap: float | None
    rot: Rotation | None


@dataclass(frozen=True)
class LeftHalf:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    bias_max: int
    buckets: int
    q_temp: tuple | None          # (coef, every)


@dataclass(frozen=True)
class RightHalf:
    heads: int
    dim: int
    vdim: int
    decay: tuple
    rot: Rotation | None


@dataclass(frozen=True)
class ParallelLayer:
    left: LeftHalf
    right: RightHalf
    left_scale: float
    right_scale: float


@dataclass(frozen=True)
class PukinexLayer:
    type: str                     # "attention" or "parallel"
    mixer: Any
    ff: int | None


@dataclass(frozen=True)
class PukinexConfig:
    """Typed configuration; the first four fields are what the engine reads."""

    architecture: str
    vocab_size: int
    max_position_embeddings: int
    eos_token_ids: tuple
    hidden_size: int
    norm_eps: float
    embedding_scale: float
    residual_mult: float
    streams: int | None           # None: one stream without connection tensors
    loop: tuple                   # (start, stop, times)
    logit_scale: float
    logit_softcap: float | None
    layers: tuple


def _need(raw: Mapping[str, Any], key: str, where: str) -> Any:
    if not isinstance(raw, Mapping) or key not in raw or raw[key] is None:
        raise ConfigError(f"config.json is missing {where}{key!r}")
    return raw[key]


def _positive(value: Any, what: str) -> int:
    if isinstance(value, bool) or not isinstance(value, (int, float)) or int(value) != value or int(value) < 1:
        raise ConfigError(f"{what} must be a positive integer, got {value!r}")
    return int(value)


def _number(value: Any, what: str) -> float:
    if isinstance(value, bool) or not isinstance(value, (int, float)):
        raise ConfigError(f"{what} must be a number, got {value!r}")
    return float(value)


def _rotation(raw: Any, dim: int, where: str) -> Rotation | None:
    if raw is None:
        return None
    dims = _need(raw, "dims", where)
    if isinstance(dims, bool) or not isinstance(dims, int) or dims < 0 or dims % 2 or dims > dim:
        raise ConfigError(f"{where}dims must be an even number up to the head size {dim}, got {dims!r}")
    if dims == 0:
        return None
    base = _number(_need(raw, "base", where), where + "base")
    factor = _number((raw.get("scaling") or {}).get("factor", 1.0), where + "scaling.factor")
    if not base > 0.0 or not factor > 0.0:
        raise ConfigError(f"{where}base and scaling.factor must be > 0")
    return Rotation(dims=dims, base=base, factor=factor)


def _heads(m: Mapping[str, Any], w: str) -> tuple[int, int, int, int]:
    heads = _positive(_need(m, "heads", w), w + "heads")
    kv = _positive(m.get("kv_heads", heads), w + "kv_heads")
    if heads % kv:
        raise ConfigError(f"{w}heads ({heads}) must be a multiple of kv_heads ({kv})")
    dim = _positive(_need(m, "dim", w), w + "dim")
    return heads, kv, dim, _positive(m.get("vdim", dim), w + "vdim")


def _parse_layer(i: int, raw: Mapping[str, Any], buckets: Mapping[int, int]) -> PukinexLayer:
    where = f"layers[{i}]."
    kind = _need(raw, "type", where)
    m = _need(raw, "mixer", where)
    w = where + "mixer."
    if kind == "attention":
        heads, kv, dim, vdim = _heads(m, w)
        if vdim != dim:
            raise ConfigError(f"{w}vdim ({vdim}) must equal dim ({dim}): the values are the keys")
        cap = m.get("softcap")
        if cap is not None and not _number(cap, w + "softcap") > 0.0:
            raise ConfigError(f"{w}softcap must be > 0, got {cap}")
        mixer = AttentionLayer(heads=heads, kv_heads=kv, dim=dim, vdim=vdim,
                               scale=_number(_need(m, "scale", w), w + "scale"),
                               softcap=None if cap is None else float(cap), rot=_rotation(m.get("rot"), dim, w + "rot."))
    elif kind == "parallel":
        l, r = _need(m, "left", w), _need(m, "right", w)
        wl, wr = w + "left.", w + "right."
        heads, kv, dim, vdim = _heads(l, wl)
        far = _positive(_need(l, "bias_max", wl), wl + "bias_max")
        rows = _positive(buckets.get(i, l.get("bias_buckets", DEFAULT_BUCKETS)), wl + "bias_buckets")
        if rows < 2 or far <= rows // 2:
            raise ConfigError(f"{wl}{rows} distance buckets do not reach up to bias_max ({far})")
        qt = l.get("q_temp")
        if qt is not None:
            qt = (_number(_need(qt, "coef", wl + "q_temp."), wl + "q_temp.coef"),
                  _positive(_need(qt, "every", wl + "q_temp."), wl + "q_temp.every"))
        left = LeftHalf(heads=heads, kv_heads=kv, dim=dim, vdim=vdim, scale=_number(_need(l, "scale", wl), wl + "scale"),
                        bias_max=far, buckets=rows, q_temp=qt)
        rh = _positive(_need(r, "heads", wr), wr + "heads")
        rd = _positive(_need(r, "dim", wr), wr + "dim")
        decay = _need(r, "decay", wr)
        if not isinstance(decay, (list, tuple)) or len(decay) != rh:
            raise ConfigError(f"{wr}decay must list one number per head ({rh})")
        decay = tuple(_number(a, wr + "decay") for a in decay)
        if any(not 0.0 < a <= 1.0 for a in decay):
            raise ConfigError(f"{wr}decay must lie in (0, 1]")
        right = RightHalf(heads=rh, dim=rd, vdim=_positive(r.get("vdim", rd), wr + "vdim"), decay=decay,
                          rot=_rotation(r.get("rot"), rd, wr + "rot."))
        mixer = ParallelLayer(left=left, right=right, left_scale=_number(m.get("left_scale", 1.0), w + "left_scale"),
                              right_scale=_number(m.get("right_scale", 1.0), w + "right_scale"))
    else:
        raise ConfigError(f"{where}type {kind!r} is not a mixer of this design (attention, parallel)")
    ff = None
    mlp = raw.get("mlp")
    if mlp is not None:
        if mlp.get("kind", "dense") != "dense":
            raise ConfigError(f"{where}mlp.kind {mlp.get('kind')!r} is not a feed-forward of this design (dense)")
        ff = _positive(_need(mlp, "ff", where + "mlp."), where + "mlp.ff")
    return PukinexLayer(type=kind, mixer=mixer, ff=ff)


def parse_config(raw: Mapping[str, Any], eos_token_ids=None, tensor_shapes: Mapping[str, tuple] | None = None
                 ) -> PukinexConfig:
    """The typed configuration of a ``config.json`` dictionary.  ``tensor_shapes`` (name -> shape, from the
    checkpoint's header) supplies the number of distance buckets of every left half."""
    layers_raw = _need(raw, "layers", "")
    if not isinstance(layers_raw, (list, tuple)) or not layers_raw:
        raise ConfigError("config.json: layers must be a non-empty list")
    buckets = {}
    for i in range(len(layers_raw)):
        shape = (tensor_shapes or {}).get(f"l{i}.mix.left.rel")
        if shape is not None and len(shape) == 2:
            buckets[i] = int(shape[0])
    eps = _number(_need(_need(raw, "norm", ""), "eps", "norm."), "norm.eps")
    if not eps > 0.0:
        raise ConfigError(f"norm.eps must be > 0, got {eps}")
    n = len(layers_raw)
    loop = raw.get("loop")
    if loop is None:
        loop_t = (0, 0, 1)
    else:
        start, stop, times = (_need(loop, k, "loop.") for k in ("start", "stop", "times"))
        for k, v in (("start", start), ("stop", stop)):
            if isinstance(v, bool) or not isinstance(v, int) or not 0 <= v <= n:
                raise ConfigError(f"loop.{k} must be a layer index from 0 to {n}, got {v!r}")
        if stop < start:
            raise ConfigError(f"loop.stop ({stop}) lies before loop.start ({start})")
        loop_t = (start, stop, _positive(times, "loop.times"))
    streams = raw.get("streams")
    if streams is not None:
        streams = _positive(streams, "streams")
        if streams > MAX_STREAMS:
            raise ConfigError(f"streams must be at most {MAX_STREAMS}, got {streams}")
    cap = raw.get("logit_softcap")
    if cap is not None and not _number(cap, "logit_softcap") > 0.0:
        raise ConfigError(f"logit_softcap must be > 0, got {cap}")
    return PukinexConfig(
        architecture=ARCHITECTURE,
        vocab_size=_positive(_need(raw, "vocab", ""), "vocab"),
        max_position_embeddings=_positive(raw.get("max_position_embeddings", DEFAULT_MAX_POSITIONS),
                                          "max_position_embeddings"),
        eos_token_ids=tuple(int(e) for e in (eos_token_ids or ())),
        hidden_size=_positive(_need(raw, "width", ""), "width"),
        norm_eps=eps,
        embedding_scale=_number((raw.get("embedding") or {}).get("scale", 1.0), "embedding.scale"),
        residual_mult=_number(raw.get("residual_mult", 1.0), "residual_mult"),
        streams=streams,
        loop=loop_t,
        logit_scale=_number(raw.get("logit_scale", 1.0), "logit_scale"),
        logit_softcap=None if cap is None else float(cap),
        layers=tuple(_parse_layer(i, lay, buckets) for i, lay in enumerate(layers_raw)),
    )


def layer_order(cfg: PukinexConfig) -> list[tuple[int, int]]:
    """``(layer, pass)`` in the order in which the layers run: the layers before the loop, the looped span
    ``times`` times, the rest."""
    start, stop, times = cfg.loop
    order = [(i, 0) for i in range(start)]
    order += [(i, p) for p in range(times) for i in range(start, stop)]
    return order + [(i, 0) for i in range(stop, len(cfg.layers))]


def _position(rot: Rotation | None, halves: bool):
    if rot is None:
        return NoPositionSpec()
    if halves:
        return RopeHalvesSpec(rot.dims, rot.base, linear_factor=rot.factor)
    return RopePairsSpec(rot.dims, rot.base, linear_factor=rot.factor)


def model_spec(cfg: PukinexConfig) -> ModelSpec:
    """Blocks and schedule: a block per layer; a layer of the looped span is called once per pass, each call
    with a cache of its own (pages for attention, a state record for retention)."""
    width, eps = cfg.hidden_size, cfg.norm_eps
    norm = LayerNormSpec(width, eps)
    blocks = []
    for i, lay in enumerate(cfg.layers):
        prefix = f"l{i}."
        m = lay.mixer
        if lay.type == "attention":
            mixer = GatedAttentionSpec(hidden_size=width, num_heads=m.heads, num_kv_heads=m.kv_heads, head_dim=m.dim,
                                       v_head_dim=m.vdim, softmax_scale=m.scale, position=_position(m.rot, halves=False),
                                       values_from_keys=True, softcap=m.softcap, unit_sink=True, gate="head")
        else:
            l, r = m.left, m.right
            left = GatedAttentionSpec(hidden_size=width, num_heads=l.heads, num_kv_heads=l.kv_heads, head_dim=l.dim,
                                      v_head_dim=l.vdim, softmax_scale=l.scale, position=NoPositionSpec(), bias=True,
                                      head_norm_eps=eps, q_temp=l.q_temp, unit_sink=True, rel_far=l.bias_max,
                                      rel_rows=l.buckets, gate="channel")
            right = RetentionSpec(hidden_size=width, num_heads=r.heads, key_dim=r.dim, value_dim=r.vdim, decay=r.decay,
                                  position=_position(r.rot, halves=True), norm_eps=eps)
            mixer = ParallelMixerSpec(left=left, right=right, left_scale=m.left_scale, right_scale=m.right_scale)
        ffn = {}
        if lay.ff is not None:
            ffn = dict(norm2=norm, feed_forward=MlpSpec(width, lay.ff, activation="relu2"), norm2_name=prefix + "norm2",
                       ffn_prefix=prefix + "mlp.", hc2_prefix=prefix + "hc2.")
        blocks.append(HyperBlockSpec(name=f"l{i}", norm1=norm, mixer=mixer, norm1_name=prefix + "norm1",
                                     mixer_prefix=prefix + "mix.", streams=cfg.streams or 1,
                                     connections=cfg.streams is not None, mult=cfg.residual_mult,
                                     hc1_prefix=prefix + "hc1.", **ffn))
    schedule = tuple(LayerCall(block=f"l{i}", cache=f"l{i}" if p == 0 else f"l{i}.pass{p}")
                     for i, p in layer_order(cfg))
    return ModelSpec(
        embedding=EmbeddingSpec(cfg.vocab_size, width, name="embed", scale=cfg.embedding_scale),
        blocks=tuple(blocks),
        schedule=schedule,
        final_norm=norm,
        final_norm_name="final.norm",
        head=HeadSpec(cfg.vocab_size, width, tied=False, name="head", scale=cfg.logit_scale,
                      softcap=cfg.logit_softcap),
        streams=cfg.streams or 1,
    )
