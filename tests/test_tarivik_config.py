"""The Tarivik design without a GPU: the reader of config.json and its refusals, the tensors it expects,
the cache needs of its parts, and the plain implementation's own consistency."""

from __future__ import annotations

import copy

import pytest
import torch

import tarivik_configs as tc
from plain import tarivik_plain as plain
from tokamak_b200.cache.manager import KVPagesNeed, StateNeed
from tokamak_b200.config.model_config import ConfigError
from tokamak_b200.config.registry import architecture_of, supported_architectures
from tokamak_b200.models.decoder import DecoderModel, flat_needs


def spec_of(raw):
    arch = architecture_of(raw)
    return arch.build_spec(arch.parse(raw))


def test_registered_and_parsed():
    assert "Tarivik" in supported_architectures()
    arch = architecture_of(tc.TV_A)
    cfg = arch.parse(tc.TV_A)
    assert (cfg.vocab_size, cfg.hidden_size, cfg.norm_eps, cfg.norm_groups, cfg.canon_taps) == (211, 64, 1e-5, 2, 4)
    assert cfg.max_position_embeddings == 256
    assert [l.type for l in cfg.layers] == [l["type"] for l in tc.TV_A["layers"]]
    par = cfg.layers[1].mixer
    assert (par.left.heads, par.left.kv_heads, par.left.chunk, par.left.scale) == (6, 3, 24, 0.25)
    assert (par.right.state, par.right.groups, par.right.conv, par.right.norm_groups) == (16, 3, 3, 3)
    assert (par.left_scale, par.right_scale) == (0.7, 1.3)
    assert cfg.layers[2].mlp is None and cfg.layers[2].mixer.gate_cap == 8.0
    moe = cfg.layers[0].mlp
    assert (moe.ff, moe.experts, moe.top, moe.groups, moe.keep) == (48, 6, 2, 3, 2)
    assert cfg.layers[3].mlp.groups == 1 and cfg.layers[3].mlp.keep == 1
    with pytest.raises(ConfigError):
        arch.build_spec(cfg, window=8)


def test_expected_tensors_and_cache_needs():
    spec = spec_of(tc.TV_A)
    names = DecoderModel.expected_tensors(spec)
    assert names["embed"].shape == (211, 64) and names["pos"].shape == (256, 64) and names["head"].shape == (211, 64)
    assert names["final.norm"].shape == (64,) and names["l0.canon1"].shape == (64, 4) and names["l0.canon2"].shape == (64, 4)
    assert names["l0.mix.q"].shape == (48, 64) and names["l0.mix.f.b"].shape == (48,) and names["l0.mix.lower"].shape == (48,)
    assert names["l0.mix.v"].shape == (80, 64) and names["l0.mix.norm"].shape == (20,) and names["l0.mix.o"].shape == (64, 80)
    assert names["l0.mlp.e5.gate"].shape == (48, 64) and names["l0.mlp.e0.down"].shape == (64, 48)
    assert names["l0.mlp.router"].shape == (6, 64) and names["l0.mlp.router"].role == "matrix_f32"
    assert names["l0.mlp.correction"].shape == (6,) and "l0.mlp.e6.gate" not in names
    assert names["l1.mix.left.q"].shape == (96, 64) and names["l1.mix.left.k.b"].shape == (48,)
    assert names["l1.mix.left.v"].shape == (72, 64) and names["l1.mix.left.q.norm"].shape == (96,)
    assert names["l1.mix.left.k.norm"].shape == (48,) and names["l1.mix.left.sink"].shape == (6,)
    assert names["l1.mix.left.g"].shape == (144, 64) and names["l1.mix.left.o"].shape == (64, 144)
    assert names["l1.mix.right.in"].shape == (48 + 48 + 96 + 6, 64) and names["l1.mix.right.conv"].shape == (144, 3)
    assert names["l1.mix.right.conv.b"].shape == (144,) and names["l1.mix.right.A_log"].shape == (6,)
    assert names["l1.mix.right.norm"].shape == (48,) and names["l1.mix.right.o"].shape == (64, 48)
    assert names["l2.mix.i"].shape == (2, 64) and names["l2.mix.f.b"].shape == (2,) and names["l2.mix.norm"].shape == (32,)
    assert "l2.norm2" not in names and "l2.canon2" not in names and "l2.mlp.router" not in names
    # what a request keeps: pages for the attention half, records for every recurrence and every convolution
    from tokamak_b200.parts.base import BLOCKS, Runtime
    shapes = {k: torch.zeros(r.shape) for k, r in names.items()}
    rt = Runtime(device=torch.device("cpu"), dtype=torch.float32)
    needs = {}
    for b in spec.blocks:
        needs.update(dict(flat_needs(b.name, BLOCKS.get(b.kind)(b, shapes, rt).cache_need())))
    tail = StateNeed((3, 64), "float32")
    assert needs["l0/conv1"] == tail and needs["l0/conv2"] == tail and needs["l2/conv1"] == tail and "l2/conv2" not in needs
    assert needs["l0/mixer"] == StateNeed((4, 12, 20), "float32")
    assert needs["l1/mixer/left"] == KVPagesNeed(3, 16, None, 24)
    assert needs["l1/mixer/right/state"] == StateNeed((6, 16, 8), "float32")
    assert needs["l1/mixer/right/conv"] == StateNeed((2, 144), "float32")
    assert needs["l2/mixer/memory"] == StateNeed((2, 24, 17), "float32") and needs["l2/mixer/maximum"] == StateNeed((2,), "float32")
    assert needs["l3/mixer/left"] == KVPagesNeed(1, 8, None, None)
    # one tap: no tail; a state-space half without a convolution: no tail either
    spec_c = spec_of(tc.TV_C)
    shapes = {k: torch.zeros(r.shape) for k, r in DecoderModel.expected_tensors(spec_c).items()}
    need = BLOCKS.get("sandwich")(spec_c.blocks[1], shapes, rt).cache_need()
    assert set(need) == {"left", "right"} and set(need["right"]) == {"state"}


def _broken(path, value):
    raw = copy.deepcopy(tc.TV_A)
    at = raw
    for key in path[:-1]:
        at = at[key]
    if value is None:
        del at[path[-1]]
    else:
        at[path[-1]] = value
    return raw


@pytest.mark.parametrize("path,value", [
    (("width",), None), (("vocab",), 0), (("max_positions",), None), (("norm", "eps"), 0.0), (("norm", "groups"), 5),
    (("canon",), None), (("canon", "taps"), 9), (("layers",), []), (("layers", 0, "type"), "attention"),
    (("layers", 0, "mixer", "heads"), 0), (("layers", 2, "mixer", "gate_cap"), -1.0),
    (("layers", 1, "mixer", "left", "kv_heads"), 4), (("layers", 1, "mixer", "left", "mask"), None),
    (("layers", 1, "mixer", "left", "scale"), None), (("layers", 1, "mixer", "right", "groups"), 4),
    (("layers", 1, "mixer", "right", "norm_groups"), 5), (("layers", 1, "mixer", "right"), None),
    (("layers", 0, "mlp", "kind"), "dense"), (("layers", 0, "mlp", "router", "top"), 5),
    (("layers", 0, "mlp", "router", "groups", "count"), 4), (("layers", 0, "mlp", "router", "groups", "keep"), 4),
    (("layers", 0, "mlp", "expert"), None),
])
def test_refusals(path, value):
    with pytest.raises(ConfigError):
        architecture_of(tc.TV_A).parse(_broken(path, value))


def test_random_folder_round_trip(tmp_path):
    """A folder of seeded random weights is written under the checkpoint's names and read back by the plain
    implementation; the router is stored like a matrix."""
    folder = tc.write_folder(tmp_path / "m", "TD", "bfloat16")
    cfg, w = plain.load_folder(folder)
    assert cfg["architecture"] == "Tarivik" and w["l1.mlp.router"].dtype == torch.bfloat16
    assert set(w) == set(DecoderModel.expected_tensors(spec_of(tc.TV_D)))
    logits = plain.forward(cfg, w, [1, 2, 3, 4, 5])
    assert logits.shape == (5, 120) and torch.isfinite(logits).all()


def test_plain_implementation_is_causal_and_stateful_pieces_agree():
    """The plain implementation against itself: a prefix's logits do not depend on what follows, the
    convolution and the recurrences continue where they stopped, and rounding changes little."""
    folder_cfg = tc.TV_B
    from tokamak_b200.weights.random_init import random_tensors
    w = random_tensors(DecoderModel.expected_tensors(spec_of(folder_cfg)), seed=3, std=0.1, dtype=torch.float32)
    toks = list(range(1, 30))
    full = plain.forward(folder_cfg, w, toks)
    assert (plain.forward(folder_cfg, w, toks[:17]) - full[:17]).abs().max() < 1e-9
    rounded = plain.forward(folder_cfg, w, toks, round_to=torch.bfloat16)
    assert 0 < (rounded - full).abs().mean() < 0.05 * full.std()      # (a flipped expert moves single rows further)
    x = torch.randn(12, 5, dtype=torch.float64)
    taps = torch.randn(5, 3, dtype=torch.float64)
    whole = plain.causal_conv(x, taps)
    by_hand = sum(taps[:, j] * (x[9 - 2 + j]) for j in range(3))
    assert (whole[9] - by_hand).abs().max() < 1e-12 and (whole[0] - taps[:, 2] * x[0]).abs().max() < 1e-12
    # chunked mask: with a chunk of one position every query sees itself only
    q, k, v = torch.randn(6, 2, 4, dtype=torch.float64), torch.randn(6, 1, 4, dtype=torch.float64), torch.randn(6, 1, 3, dtype=torch.float64)
    alone = plain.chunked_attention(q, k, v, 0.5, 1, torch.full((2,), -1e9, dtype=torch.float64))
    assert (alone - v.expand(6, 2, 3)).abs().max() < 1e-9
