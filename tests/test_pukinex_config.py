"""The Pukinex design without a GPU: the reader of config.json and its refusals, the tensors it expects, the
order in which looped layers run and the caches they get, the distance table, and the plain
implementation's own consistency."""

from __future__ import annotations

import copy
import math

import pytest
import torch

import pukinex_configs as pc
from plain import pukinex_plain as plain
from tokamak_b200.cache.manager import KVPagesNeed, StateNeed
from tokamak_b200.config.model_config import ConfigError
from tokamak_b200.config.registry import architecture_of, supported_architectures
from tokamak_b200.models.decoder import DecoderModel, flat_needs


def spec_of(raw, shapes=None):
    arch = architecture_of(raw)
    return arch.build_spec(arch.parse(raw, tensor_shapes=shapes))


def test_registered_and_parsed():
    assert "Pukinex" in supported_architectures()
    arch = architecture_of(pc.PX_A)
    cfg = arch.parse(pc.PX_A)
    assert (cfg.vocab_size, cfg.hidden_size, cfg.norm_eps, cfg.streams, cfg.loop) == (197, 48, 1e-5, 3, (1, 3, 2))
    assert (cfg.embedding_scale, cfg.residual_mult, cfg.logit_scale, cfg.logit_softcap) == (3.0, 0.8, 0.5, 12.0)
    assert [l.type for l in cfg.layers] == [l["type"] for l in pc.PX_A["layers"]]
    att = cfg.layers[0].mixer
    assert (att.heads, att.kv_heads, att.dim, att.softcap) == (4, 2, 12, 9.0)
    assert (att.rot.dims, att.rot.base, att.rot.factor) == (8, 10000.0, 4.0)
    par = cfg.layers[1].mixer
    assert (par.left.heads, par.left.kv_heads, par.left.dim, par.left.vdim, par.left.bias_max, par.left.buckets) == (4, 2, 10, 6, 20, 8)
    assert par.left.q_temp == (0.5, 16) and par.right.decay == (0.9, 0.96, 0.99) and par.right.rot.factor == 1.0
    assert (par.left_scale, par.right_scale) == (0.7, 0.4)
    assert cfg.layers[2].ff is None and cfg.layers[2].mixer.softcap is None and cfg.layers[3].mixer.right.rot is None
    assert cfg.layers[3].mixer.left.q_temp is None
    # without the optional keys: one stream without connection tensors, no loop, plain logits
    cfg_b = arch.parse(pc.PX_B)
    assert cfg_b.streams is None and cfg_b.loop == (0, 0, 1) and cfg_b.logit_softcap is None and cfg_b.logit_scale == 1.0
    # the number of buckets comes from the checkpoint where there is one
    assert arch.parse(pc.PX_A, tensor_shapes={"l1.mix.left.rel": (14, 4)}).layers[1].mixer.left.buckets == 14
    with pytest.raises(ConfigError):
        arch.build_spec(cfg, window=8)


def test_layers_of_a_loop_run_in_order_with_a_cache_per_pass():
    from tokamak_b200.models.pukinex import layer_order
    arch = architecture_of(pc.PX_A)
    cfg = arch.parse(pc.PX_A)
    assert layer_order(cfg) == [(0, 0), (1, 0), (2, 0), (1, 1), (2, 1), (3, 0)]
    spec = arch.build_spec(cfg)
    assert [(c.block, c.cache) for c in spec.schedule] == [
        ("l0", "l0"), ("l1", "l1"), ("l2", "l2"), ("l1", "l1.pass1"), ("l2", "l2.pass1"), ("l3", "l3")]
    assert [c.block for c in spec_of(pc.PX_C).schedule] == ["l0", "l0", "l0", "l1", "l2"]
    assert [c.block for c in spec_of(pc.PX_D).schedule] == ["l0", "l1", "l1"]
    assert [c.block for c in spec_of(pc.PX_B).schedule] == ["l0", "l1", "l2"]
    assert len({c.cache for c in spec_of(pc.PX_C).schedule}) == 5
    assert spec.streams == 3 and spec_of(pc.PX_B).streams == 1


def test_expected_tensors_and_cache_needs():
    spec = spec_of(pc.PX_A)
    names = DecoderModel.expected_tensors(spec)
    assert names["embed"].shape == (197, 48) and names["head"].shape == (197, 48)
    assert names["final.norm"].shape == (48,) and names["final.norm.b"].shape == (48,)
    assert names["l0.norm1"].shape == (48,) and names["l0.norm2.b"].shape == (48,)
    assert names["l0.mix.q"].shape == (48, 48) and names["l0.mix.k"].shape == (24, 48) and "l0.mix.v" not in names
    assert names["l0.mix.g"].shape == (4, 48) and names["l0.mix.o"].shape == (48, 48)
    assert names["l0.mlp.up"].shape == (40, 48) and names["l0.mlp.down"].shape == (48, 40)
    for q in ("hc1", "hc2"):
        assert names[f"l0.{q}.in"].shape == (3,) and names[f"l0.{q}.out"].shape == (3,) and names[f"l0.{q}.mix"].shape == (3, 3)
    assert names["l1.mix.left.q"].shape == (40, 48) and names["l1.mix.left.q.b"].shape == (40,)
    assert names["l1.mix.left.k"].shape == (20, 48) and names["l1.mix.left.v"].shape == (12, 48)
    assert names["l1.mix.left.v.b"].shape == (12,) and names["l1.mix.left.q.norm"].shape == (10,)
    assert names["l1.mix.left.k.norm"].shape == (10,) and names["l1.mix.left.rel"].shape == (8, 4)
    assert names["l1.mix.left.g"].shape == (24, 48) and names["l1.mix.left.o"].shape == (48, 24)
    assert names["l1.mix.right.q"].shape == (36, 48) and names["l1.mix.right.v"].shape == (30, 48)
    assert names["l1.mix.right.g"].shape == (30, 48) and names["l1.mix.right.o"].shape == (48, 30)
    assert "l2.norm2" not in names and "l2.mlp.up" not in names and "l2.hc2.in" not in names and "l2.hc1.mix" in names
    assert not [n for n in DecoderModel.expected_tensors(spec_of(pc.PX_B)) if ".hc" in n]
    # what a request keeps: pages for attention (values of their own size), a record for retention
    from tokamak_b200.parts.base import BLOCKS, Runtime
    shapes = {k: torch.zeros(r.shape) for k, r in names.items()}
    rt = Runtime(device=torch.device("cpu"), dtype=torch.float32)
    needs = {}
    for b in spec.blocks:
        needs.update(dict(flat_needs(b.name, BLOCKS.get(b.kind)(b, shapes, rt).cache_need())))
    assert needs["l0"] == KVPagesNeed(2, 12, None, None)
    assert needs["l1/left"] == KVPagesNeed(2, 10, None, 6) and needs["l1/right"] == StateNeed((3, 12, 10), "float32")
    assert needs["l3/left"] == KVPagesNeed(3, 8, None, 12) and needs["l3/right"] == StateNeed((2, 6, 14), "float32")


def _broken(path, value):
    raw = copy.deepcopy(pc.PX_A)
    at = raw
    for key in path[:-1]:
        at = at[key]
    if value is None:
        del at[path[-1]]
    else:
        at[path[-1]] = value
    return raw


@pytest.mark.parametrize("path,value", [
    (("width",), None), (("vocab",), 0), (("norm", "eps"), 0.0), (("norm",), None), (("layers",), []),
    (("layers", 0, "type"), "retention"), (("layers", 0, "mixer", "heads"), 0), (("layers", 0, "mixer", "kv_heads"), 3),
    (("layers", 0, "mixer", "vdim"), 10), (("layers", 0, "mixer", "softcap"), -1.0), (("layers", 0, "mixer", "rot", "dims"), 7),
    (("layers", 0, "mixer", "rot", "dims"), 14), (("layers", 0, "mixer", "rot", "scaling", "factor"), 0.0),
    (("layers", 0, "mixer", "scale"), None), (("layers", 1, "mixer", "left", "bias_max"), None),
    (("layers", 1, "mixer", "left", "bias_max"), 4), (("layers", 1, "mixer", "left", "q_temp", "every"), 0),
    (("layers", 1, "mixer", "right", "decay"), [0.9, 0.9]), (("layers", 1, "mixer", "right", "decay"), [0.9, 1.5, 0.9]),
    (("layers", 1, "mixer", "right"), None), (("layers", 0, "mlp", "kind"), "moe"), (("layers", 0, "mlp", "ff"), None),
    (("streams",), 9), (("streams",), 0), (("loop", "stop"), 5), (("loop", "start"), 4), (("loop", "times"), 0),
    (("logit_softcap",), 0.0),
])
def test_refusals(path, value):
    with pytest.raises(ConfigError):
        architecture_of(pc.PX_A).parse(_broken(path, value))


def test_distance_table_follows_the_bucket_formula():
    from tokamak_b200.parts.attention import bucketed_distance_table
    gen = torch.Generator().manual_seed(1)
    for rows, far in ((16, 100), (8, 20), (4, 9), (12, 60), (6, 1000), (2, 2), (32, 17)):
        rel = torch.randn(rows, 3, generator=gen)
        tab = bucketed_distance_table(rel, far)
        assert tab.shape == (3, far + 1)
        half = rows // 2
        for n in range(far + 1):
            b = n if n < half else min(rows - 1, half + math.floor(math.log(n / half) / math.log(far / half) * (rows - half)))
            assert b == plain.bucket_of(n, rows, far) and torch.equal(tab[:, n], rel[b]), (rows, far, n)
        assert plain.bucket_of(far, rows, far) == rows - 1 == plain.bucket_of(far * 7, rows, far)
    with pytest.raises(ValueError):
        bucketed_distance_table(torch.zeros(8, 2), 4)


def test_random_folder_round_trip(tmp_path):
    folder = pc.write_folder(tmp_path / "m", "PD", "bfloat16")
    cfg, w = plain.load_folder(folder)
    assert cfg["architecture"] == "Pukinex"
    from tokamak_b200.weights.loader import checkpoint_shapes
    shapes = checkpoint_shapes(folder)
    assert set(w) == set(DecoderModel.expected_tensors(spec_of(pc.PX_D, shapes)))
    logits = plain.forward(cfg, w, [1, 2, 3, 4, 5])
    assert logits.shape == (5, 90) and torch.isfinite(logits).all()


def test_plain_implementation_is_causal_and_stateful_pieces_agree():
    """The plain implementation against itself: a prefix's logits do not depend on what follows, retention
    continues where it stopped and equals its sum form, both rotations keep lengths and depend on distance
    only, the added unit in the denominator takes its share, and rounding changes little."""
    from tokamak_b200.weights.random_init import random_tensors
    raw = pc.PX_A
    w = {k: v.double() for k, v in random_tensors(DecoderModel.expected_tensors(spec_of(raw)), seed=3, std=0.1,
                                                  dtype=torch.float32).items()}
    toks = list(range(1, 30))
    full = plain.forward(raw, w, toks)
    assert (plain.forward(raw, w, toks[:17]) - full[:17]).abs().max() < 1e-9
    rounded = plain.forward(raw, w, toks, ROUND=plain.bf16_round)
    assert 0 < (rounded - full).abs().mean() < 0.05 * full.std()
    gen = torch.Generator().manual_seed(0)
    q, k = torch.randn(9, 2, 6, generator=gen, dtype=torch.float64), torch.randn(9, 2, 6, generator=gen, dtype=torch.float64)
    v = torch.randn(9, 2, 3, generator=gen, dtype=torch.float64)
    o, S = plain.retention_scan(q, k, v, [0.9, 0.5])
    o1, S1 = plain.retention_scan(q[:4], k[:4], v[:4], [0.9, 0.5])
    o2, S2 = plain.retention_scan(q[4:], k[4:], v[4:], [0.9, 0.5], S1)
    assert (torch.cat([o1, o2]) - o).abs().max() < 1e-12 and (S2 - S).abs().max() < 1e-12
    by_sum = sum(0.9 ** (8 - j) * (q[8, 0] @ k[j, 0]) * v[j, 0] for j in range(9))
    assert (o[8, 0] - by_sum).abs().max() < 1e-12
    for turn in (plain.rotate_neighbours, plain.rotate_halves):
        a = turn(q, plain.rope_angles(torch.arange(9), 4, 100.0, 2.0))
        b = turn(k, plain.rope_angles(torch.arange(9), 4, 100.0, 2.0))
        assert (a.norm(dim=-1) - q.norm(dim=-1)).abs().max() < 1e-12 and (a[..., 4:] - q[..., 4:]).abs().max() == 0
        a5 = turn(q, plain.rope_angles(torch.arange(9) + 5, 4, 100.0, 2.0))
        b5 = turn(k, plain.rope_angles(torch.arange(9) + 5, 4, 100.0, 2.0))
        assert ((a[7] * b[3]).sum() - (a5[7] * b5[3]).sum()).abs() < 1e-12
    p = plain.softmax_plus_one(torch.zeros(1, 3, 3, dtype=torch.float64), torch.tril(torch.ones(3, 3, dtype=torch.bool)))
    assert torch.allclose(p[0, 2], torch.full((3,), 0.25, dtype=torch.float64)) and p[0, 0, 1] == 0
