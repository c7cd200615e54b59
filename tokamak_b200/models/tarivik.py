"""The Tarivik decoder as a :class:`ModelSpec`.

A stack of blocks whose sublayers read the residual stream itself, through a short causal convolution
(``h + conv(h)``, its last inputs part of a request's state), and are normalised only on the way out by an RMS
norm in equal groups of channels: ``x <- x + norm1(mixer(x)); x <- x + norm2(ff(x))``.  A learned position
table joins the embedding.  The mixers, listed layer by layer in ``config.json``: forget-gated linear
attention (``hgrn2``), a matrix memory with exponential gates (``mlstm``), and two mixers side by side
(``parallel``): chunked grouped-query attention with biases, a norm over the whole q and k projections, a
distance bias, sinks and an output gate on the left, a state-space layer with scalar decays on the right,
added with a factor each.  Feed-forwards are mixtures of silu-gated experts with a sigmoid router that
chooses inside the best groups of experts; a layer may lack its feed-forward.

    {"architecture": "Tarivik", "vocab": V, "width": W, "max_positions": P, "norm": {"eps": e, "groups": g},
     "canon": {"taps": k},
     "layers": [{"type": "hgrn2", "mixer": {"heads", "dim", "vdim"}, "mlp": {...} | null},
                {"type": "mlstm", "mixer": {"heads", "dim", "vdim", "gate_cap"}, "mlp": ...},
                {"type": "parallel", "mixer": {"left": {"heads", "kv_heads", "dim", "vdim", "scale", "mask": {"size"}},
                                                "right": {"heads", "vdim", "state", "groups", "conv", "norm_groups"},
                                                "left_scale", "right_scale"}, "mlp": ...}, ...]}
    mlp: {"kind": "moe", "expert": {"ff"}, "router": {"experts", "top", "groups": {"count", "keep"}}}

Tensors are ``embed``, ``pos``, ``head``, ``final.norm`` and, for layer ``i``, ``l<i>.norm1``, ``l<i>.canon1``,
``l<i>.mix.*`` and, with a feed-forward, ``l<i>.norm2``, ``l<i>.canon2`` and ``l<i>.mlp.*``.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Mapping

from ..config.model_config import ConfigError
from ..parts.attention import RowNormAttentionSpec
from ..parts.block import SandwichBlockSpec
from ..parts.embedding import EmbeddingSpec, HeadSpec
from ..parts.feedforward import MoESpec
from ..parts.hgrn2 import Hgrn2Spec
from ..parts.mlstm import MlstmSpec
from ..parts.norm import CastNormSpec, GroupRMSNormSpec
from ..parts.parallel import ParallelMixerSpec
from ..parts.position import LearnedPositionSpec
from ..parts.ssd import StateSpaceDualSpec
from .decoder import LayerCall, ModelSpec

ARCHITECTURE = "Tarivik"
SLOPE_EXPONENT = 8.0        # head h's distance slope is 2 ** (-8 (h + 1) / heads)


@dataclass(frozen=True)
class Hgrn2Layer:
    heads: int
    dim: int
    vdim: int


@dataclass(frozen=True)
class MlstmLayer:
    heads: int
    dim: int
    vdim: int
    gate_cap: float


@dataclass(frozen=True)
class ChunkedAttentionHalf:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    chunk: int


@dataclass(frozen=True)
class StateSpaceHalf:
    heads: int
    vdim: int
    state: int
    groups: int
    conv: int
    norm_groups: int


@dataclass(frozen=True)
class ParallelLayer:
    left: ChunkedAttentionHalf
    right: StateSpaceHalf
    left_scale: float
    right_scale: float


@dataclass(frozen=True)
class MoELayer:
    ff: int
    experts: int
    top: int
    groups: int
    keep: int


@dataclass(frozen=True)
class TarivikLayer:
    type: str                      # "hgrn2", "mlstm" or "parallel"
    mixer: Any
    mlp: MoELayer | None


@dataclass(frozen=True)
class TarivikConfig:
    """Typed configuration; the first four fields are what the engine reads."""

    architecture: str
    vocab_size: int
    max_position_embeddings: int
    eos_token_ids: tuple
    hidden_size: int
    norm_eps: float
    norm_groups: int
    canon_taps: int
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


def _parse_mlp(raw: Any, where: str) -> MoELayer | None:
    if raw is None:
        return None
    if raw.get("kind", "moe") != "moe":
        raise ConfigError(f"{where}kind {raw.get('kind')!r} is not a feed-forward of this design (moe)")
    router = _need(raw, "router", where)
    w = where + "router."
    experts, top = _positive(_need(router, "experts", w), w + "experts"), _positive(_need(router, "top", w), w + "top")
    groups = router.get("groups") or {}
    count = _positive(groups.get("count", 1), w + "groups.count")
    keep = _positive(groups.get("keep", count), w + "groups.keep")
    if experts % count or keep > count:
        raise ConfigError(f"{w}{experts} experts do not form {count} equal groups of which {keep} are kept")
    if top > keep * (experts // count):
        raise ConfigError(f"{w}top ({top}) is more than the {keep} kept groups of {experts // count} experts hold")
    return MoELayer(ff=_positive(_need(_need(raw, "expert", where), "ff", where + "expert."), where + "expert.ff"),
                    experts=experts, top=top, groups=count, keep=keep)


def _parse_layer(i: int, raw: Mapping[str, Any]) -> TarivikLayer:
    where = f"layers[{i}]."
    kind = _need(raw, "type", where)
    m = _need(raw, "mixer", where)
    w = where + "mixer."
    if kind == "hgrn2":
        num = lambda key: _positive(_need(m, key, w), w + key)
        dim = num("dim")
        mixer = Hgrn2Layer(heads=num("heads"), dim=dim, vdim=_positive(m.get("vdim", dim), w + "vdim"))
    elif kind == "mlstm":
        num = lambda key: _positive(_need(m, key, w), w + key)
        dim = num("dim")
        cap = _number(_need(m, "gate_cap", w), w + "gate_cap")
        if not cap > 0:
            raise ConfigError(f"{w}gate_cap must be > 0, got {cap}")
        mixer = MlstmLayer(heads=num("heads"), dim=dim, vdim=_positive(m.get("vdim", dim), w + "vdim"), gate_cap=cap)
    elif kind == "parallel":
        l, r = _need(m, "left", w), _need(m, "right", w)
        wl, wr = w + "left.", w + "right."
        ln = lambda key: _positive(_need(l, key, wl), wl + key)
        rn = lambda key: _positive(_need(r, key, wr), wr + key)
        heads = ln("heads")
        kv = _positive(l.get("kv_heads", heads), wl + "kv_heads")
        if heads % kv:
            raise ConfigError(f"{wl}heads ({heads}) must be a multiple of kv_heads ({kv})")
        dim = ln("dim")
        left = ChunkedAttentionHalf(heads=heads, kv_heads=kv, dim=dim, vdim=_positive(l.get("vdim", dim), wl + "vdim"),
                                    scale=_number(_need(l, "scale", wl), wl + "scale"),
                                    chunk=_positive(_need(_need(l, "mask", wl), "size", wl + "mask."), wl + "mask.size"))
        rh, rg = rn("heads"), _positive(r.get("groups", 1), wr + "groups")
        if rh % rg:
            raise ConfigError(f"{wr}heads ({rh}) must be a multiple of groups ({rg})")
        right = StateSpaceHalf(heads=rh, vdim=rn("vdim"), state=rn("state"), groups=rg, conv=rn("conv"),
                               norm_groups=_positive(r.get("norm_groups", 1), wr + "norm_groups"))
        if (right.heads * right.vdim) % right.norm_groups:
            raise ConfigError(f"{wr}heads * vdim ({right.heads * right.vdim}) does not split into "
                              f"{right.norm_groups} norm groups")
        mixer = ParallelLayer(left=left, right=right, left_scale=_number(m.get("left_scale", 1.0), w + "left_scale"),
                              right_scale=_number(m.get("right_scale", 1.0), w + "right_scale"))
    else:
        raise ConfigError(f"{where}type {kind!r} is not a mixer of this design (hgrn2, mlstm, parallel)")
    return TarivikLayer(type=kind, mixer=mixer, mlp=_parse_mlp(raw.get("mlp"), where + "mlp."))


def parse_config(raw: Mapping[str, Any], eos_token_ids=None) -> TarivikConfig:
    """The typed configuration of a ``config.json`` dictionary."""
    layers_raw = _need(raw, "layers", "")
    if not isinstance(layers_raw, (list, tuple)) or not layers_raw:
        raise ConfigError("config.json: layers must be a non-empty list")
    norm = _need(raw, "norm", "")
    eps = _number(_need(norm, "eps", "norm."), "norm.eps")
    if not eps > 0.0:
        raise ConfigError(f"norm.eps must be > 0, got {eps}")
    width = _positive(_need(raw, "width", ""), "width")
    groups = _positive(norm.get("groups", 1), "norm.groups")
    if width % groups:
        raise ConfigError(f"width ({width}) does not split into norm.groups ({groups}) equal parts")
    taps = _positive(_need(_need(raw, "canon", ""), "taps", "canon."), "canon.taps")
    if taps > 8:
        raise ConfigError(f"canon.taps must be at most 8, got {taps}")
    return TarivikConfig(
        architecture=ARCHITECTURE,
        vocab_size=_positive(_need(raw, "vocab", ""), "vocab"),
        max_position_embeddings=_positive(_need(raw, "max_positions", ""), "max_positions"),
        eos_token_ids=tuple(int(e) for e in (eos_token_ids or ())),
        hidden_size=width,
        norm_eps=eps,
        norm_groups=groups,
        canon_taps=taps,
        layers=tuple(_parse_layer(i, lay) for i, lay in enumerate(layers_raw)),
    )


def model_spec(cfg: TarivikConfig) -> ModelSpec:
    """Blocks and schedule: every layer once, with caches of its own (pages for an attention half, state
    records for the recurrent mixers and for the blocks' input convolutions).  A block is the sandwich
    arrangement without a norm in front of its sublayers, with input convolutions and without layer scales."""
    width, eps = cfg.hidden_size, cfg.norm_eps
    norm, front = GroupRMSNormSpec(width, eps, cfg.norm_groups), CastNormSpec(width)
    blocks, schedule = [], []
    for i, lay in enumerate(cfg.layers):
        prefix = f"l{i}."
        m = lay.mixer
        if lay.type == "hgrn2":
            mixer = Hgrn2Spec(hidden_size=width, num_heads=m.heads, key_dim=m.dim, value_dim=m.vdim, norm_eps=eps)
        elif lay.type == "mlstm":
            mixer = MlstmSpec(hidden_size=width, num_heads=m.heads, key_dim=m.dim, value_dim=m.vdim,
                              gate_cap=m.gate_cap, norm_eps=eps)
        else:
            l, r = m.left, m.right
            left = RowNormAttentionSpec(hidden_size=width, num_heads=l.heads, num_kv_heads=l.kv_heads, head_dim=l.dim,
                                        v_head_dim=l.vdim, softmax_scale=l.scale, bias=True, row_norm_eps=eps,
                                        chunk=l.chunk, slope_exponent=SLOPE_EXPONENT, sinks=True, gate=True)
            right = StateSpaceDualSpec(hidden_size=width, num_heads=r.heads, value_dim=r.vdim, state_dim=r.state,
                                       num_groups=r.groups, conv_taps=r.conv, norm_groups=r.norm_groups, norm_eps=eps)
            mixer = ParallelMixerSpec(left=left, right=right, left_scale=m.left_scale, right_scale=m.right_scale)
        ffn = {}
        if lay.mlp is not None:
            f = lay.mlp
            ffn = dict(norm_in2=front, norm_out2=norm,
                       feed_forward=MoESpec(hidden_size=width, intermediate_size=f.ff, num_experts=f.experts, top=f.top,
                                            num_groups=f.groups, keep_groups=f.keep),
                       norm_in2_name="", ffn_prefix=prefix + "mlp.", norm_out2_name=prefix + "norm2",
                       conv2_name=prefix + "canon2")
        blocks.append(SandwichBlockSpec(name=f"l{i}", norm_in1=front, mixer=mixer, norm_out1=norm, norm_in1_name="",
                                        mixer_prefix=prefix + "mix.", norm_out1_name=prefix + "norm1",
                                        conv_taps=cfg.canon_taps, conv1_name=prefix + "canon1", **ffn))
        schedule.append(LayerCall(block=f"l{i}", cache=f"l{i}"))
    return ModelSpec(
        embedding=EmbeddingSpec(cfg.vocab_size, width, name="embed"),
        blocks=tuple(blocks),
        schedule=tuple(schedule),
        final_norm=norm,
        final_norm_name="final.norm",
        head=HeadSpec(cfg.vocab_size, width, tied=False, name="head"),
        embedding_position=LearnedPositionSpec(cfg.max_position_embeddings, width, name="pos"),
    )
