"""Tiny Tarivik configurations for the tests.  They differ in every size and option: widths (also one that
is no multiple of 4), norm groups (1 to 6), input convolutions of 1 to 4 taps, layer orders (every mixer
comes first somewhere, layers without a feed-forward), head counts and groups of the attention half (all
heads on one key head, every head its own), key and value sizes that differ, chunks from 1 position to longer
than a request, state-space halves with 1 to 3 groups and convolutions of 1 to 5 taps, mixtures with groups
of one expert, with one group, with every group kept, and the cache's page size."""

from __future__ import annotations


def _moe(ff, experts, top, count=1, keep=None):
    return {"kind": "moe", "expert": {"ff": ff},
            "router": {"experts": experts, "top": top, "groups": {"count": count, "keep": count if keep is None else keep}}}


def _hgrn2(heads, dim, vdim):
    return {"heads": heads, "dim": dim, "vdim": vdim}


def _mlstm(heads, dim, vdim, cap):
    return {"heads": heads, "dim": dim, "vdim": vdim, "gate_cap": cap}


def _parallel(left, right, ls, rs):
    return {"left": left, "right": right, "left_scale": ls, "right_scale": rs}


def _left(heads, kv, dim, vdim, scale, chunk):
    return {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": scale, "mask": {"size": chunk}}


def _right(heads, vdim, state, groups, conv, norm_groups):
    return {"heads": heads, "vdim": vdim, "state": state, "groups": groups, "conv": conv, "norm_groups": norm_groups}


def _layer(kind, mixer, mlp):
    return {"type": kind, "mixer": mixer, "mlp": mlp}


TV_A = {
    "architecture": "Tarivik", "vocab": 211, "width": 64, "max_positions": 256, "norm": {"eps": 1e-5, "groups": 2},
    "canon": {"taps": 4},
    "layers": [
        _layer("hgrn2", _hgrn2(4, 12, 20), _moe(48, 6, 2, 3, 2)),
        _layer("parallel", _parallel(_left(6, 3, 16, 24, 0.25, 24), _right(6, 8, 16, 3, 3, 3), 0.7, 1.3), _moe(32, 4, 2, 4, 2)),
        _layer("mlstm", _mlstm(2, 24, 16, 8.0), None),
        _layer("parallel", _parallel(_left(4, 1, 8, 8, 0.35, 7), _right(2, 24, 8, 1, 5, 1), 1.0, 0.25), _moe(40, 5, 3)),
    ],
}
TV_B = {
    "architecture": "Tarivik", "vocab": 157, "width": 54, "max_positions": 200, "norm": {"eps": 1e-6, "groups": 3},
    "canon": {"taps": 2},
    "layers": [
        _layer("parallel", _parallel(_left(3, 3, 12, 10, 0.3, 1), _right(3, 10, 12, 3, 2, 2), 0.5, 0.5), None),
        _layer("mlstm", _mlstm(3, 10, 22, 15.0), _moe(24, 8, 4, 2, 1)),
        _layer("hgrn2", _hgrn2(1, 40, 6), _moe(56, 3, 1, 3, 3)),
        _layer("parallel", _parallel(_left(2, 1, 20, 12, 0.2, 400), _right(4, 6, 20, 2, 4, 4), 1.5, 0.8), _moe(16, 12, 5, 4, 3)),
    ],
}
# sizes that the products' own kernels take (widths and inner sizes in steps of 64), a state wider than one
# block of value channels, no input convolution to speak of (one tap), a state-space half without a convolution
TV_C = {
    "architecture": "Tarivik", "vocab": 300, "width": 128, "max_positions": 256, "norm": {"eps": 1e-6, "groups": 1},
    "canon": {"taps": 1},
    "layers": [
        _layer("mlstm", _mlstm(4, 32, 48, 10.0), _moe(64, 8, 2, 2, 2)),
        _layer("parallel", _parallel(_left(4, 2, 64, 32, 0.125, 40), _right(4, 32, 64, 2, 1, 2), 1.0, 1.0), _moe(128, 4, 1)),
        _layer("hgrn2", _hgrn2(2, 130, 80), None),
        _layer("parallel", _parallel(_left(8, 2, 32, 64, 0.18, 33), _right(8, 16, 32, 4, 4, 8), 0.9, 0.6), _moe(64, 16, 6, 8, 4)),
    ],
}
# a width that is no multiple of 4, six norm groups, one layer of each kind without any feed-forward but one
TV_D = {
    "architecture": "Tarivik", "vocab": 120, "width": 42, "max_positions": 192, "norm": {"eps": 1e-5, "groups": 6},
    "canon": {"taps": 3},
    "layers": [
        _layer("hgrn2", _hgrn2(3, 6, 14), None),
        _layer("mlstm", _mlstm(1, 18, 42, 20.0), _moe(30, 2, 2)),
        _layer("parallel", _parallel(_left(5, 5, 6, 6, 0.4, 16), _right(1, 14, 6, 1, 3, 1), 2.0, 1.0), None),
    ],
}
# (configuration, how the random weights are drawn, page size)
ALL = {
    "TA": (TV_A, {"seed": 31, "std": 0.08, "norm_std": 0.1}, 16),
    "TB": (TV_B, {"seed": 32, "std": 0.1, "norm_std": 0.1}, 8),
    "TC": (TV_C, {"seed": 33, "std": 0.06, "norm_std": 0.1}, 32),
    "TD": (TV_D, {"seed": 34, "std": 0.1, "norm_std": 0.1}, 16),
}


def write_folder(folder, tag: str, dtype: str):
    """A model folder of configuration ``tag``: seeded random weights, with the tensors that random draws
    leave without effect redrawn so that every mechanism matters: routers that spread the scores, corrections
    that change a choice now and then, position rows as large as the embedding's."""
    import torch
    from safetensors.torch import load_file, save_file

    from tokamak_b200.weights import write_random_model

    raw, init, _ = ALL[tag]
    write_random_model(folder, raw, dtype=dtype, **init)
    path = str(folder) + "/model.safetensors"
    tensors = load_file(path)
    gen = torch.Generator().manual_seed(init["seed"] + 1000)
    for name, t in tensors.items():
        draw = lambda std: (std * torch.randn(t.shape, generator=gen)).to(t.dtype)
        if name.endswith(".router"):
            tensors[name] = draw(1.2 / raw["width"] ** 0.5 / init["std"])
        elif name.endswith(".correction"):
            tensors[name] = draw(0.08)
        elif name.endswith(("canon1", "canon2")):
            tensors[name] = draw(0.4)
        elif name.endswith(".A_log"):
            tensors[name] = draw(0.7) - 1.0
    save_file({k: v.contiguous() for k, v in tensors.items()}, path)
    return folder
