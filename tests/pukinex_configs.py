"""Tiny Pukinex configurations for the tests.  They differ in every size and option: the number of copies of
the residual stream (none declared, 1, 2, 3, 4), loops (none, from the first layer, in the middle, three passes, a
span of one layer), layer orders (each mixer first somewhere, layers without a feed-forward), head counts and
groups (every head its own key head, all heads on one), key and value sizes that differ, rotation over the
whole head and over part of it, with and without position scaling and score caps, retention with rotation
over part of the head and without any, distance tables of 4 to 12 buckets that reach 9 to 60 positions back,
query temperatures that change every 5 to 32 positions or are absent, logits with and without scale and cap,
and the cache's page size."""

from __future__ import annotations


def _attention(heads, kv, dim, scale, softcap=None, rot=None):
    m = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": dim, "scale": scale}
    if softcap is not None:
        m["softcap"] = softcap
    if rot is not None:
        m["rot"] = rot
    return m


def _rot(dims, base, factor=None):
    r = {"base": base, "dims": dims}
    if factor is not None:
        r["scaling"] = {"factor": factor}
    return r


def _left(heads, kv, dim, vdim, scale, far, buckets, q_temp=None):
    m = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": scale, "bias_max": far,
         "bias_buckets": buckets}
    if q_temp is not None:
        m["q_temp"] = {"coef": q_temp[0], "every": q_temp[1]}
    return m


def _right(heads, dim, vdim, decay, rot=None):
    m = {"heads": heads, "dim": dim, "vdim": vdim, "decay": decay}
    if rot is not None:
        m["rot"] = rot
    return m


def _parallel(left, right, ls, rs):
    return {"left": left, "right": right, "left_scale": ls, "right_scale": rs}


def _layer(kind, mixer, ff):
    return {"type": kind, "mixer": mixer, "mlp": None if ff is None else {"kind": "dense", "ff": ff}}


PX_A = {
    "architecture": "Pukinex", "vocab": 197, "width": 48, "norm": {"eps": 1e-5}, "embedding": {"scale": 3.0},
    "residual_mult": 0.8, "streams": 3, "loop": {"start": 1, "stop": 3, "times": 2},
    "logit_scale": 0.5, "logit_softcap": 12.0,
    "layers": [
        _layer("attention", _attention(4, 2, 12, 0.3, softcap=9.0, rot=_rot(8, 10000.0, 4.0)), 40),
        _layer("parallel", _parallel(_left(4, 2, 10, 6, 0.3, 20, 8, (0.5, 16)),
                                     _right(3, 12, 10, [0.9, 0.96, 0.99], _rot(8, 5000.0)), 0.7, 0.4), 56),
        _layer("attention", _attention(2, 1, 16, 0.25, rot=_rot(16, 300.0)), None),
        _layer("parallel", _parallel(_left(3, 3, 8, 12, 0.35, 9, 4, None),
                                     _right(2, 6, 14, [0.97, 1.0], None), 1.2, 0.5), 24),
    ],
}
PX_B = {
    "architecture": "Pukinex", "vocab": 131, "width": 54, "norm": {"eps": 1e-6}, "embedding": {"scale": 1.0},
    "residual_mult": 1.0,
    "layers": [
        _layer("parallel", _parallel(_left(2, 1, 14, 14, 0.27, 60, 12, (1.5, 5)),
                                     _right(1, 20, 6, [0.95], _rot(20, 100.0, 2.0)), 0.5, 1.0), 30),
        _layer("attention", _attention(3, 3, 10, 0.32, softcap=30.0), 70),
        _layer("parallel", _parallel(_left(6, 2, 6, 4, 0.4, 12, 6, (0.25, 32)),
                                     _right(4, 8, 8, [0.8, 0.9, 0.95, 0.98], _rot(4, 777.0)), 1.0, 1.0), None),
    ],
}
# sizes that the products' own kernels take (widths and inner sizes in steps of 64), head sizes the tiled attention
# kernels take, one copy of the stream with connection tensors, a loop of three passes over one layer
PX_C = {
    "architecture": "Pukinex", "vocab": 320, "width": 128, "norm": {"eps": 1e-5}, "embedding": {"scale": 8.0},
    "residual_mult": 0.5, "streams": 1, "loop": {"start": 0, "stop": 1, "times": 3}, "logit_softcap": 20.0,
    "layers": [
        _layer("attention", _attention(4, 2, 64, 0.125, softcap=20.0, rot=_rot(32, 10000.0, 2.0)), 192),
        _layer("parallel", _parallel(_left(4, 2, 64, 64, 0.125, 40, 10, (0.4, 24)),
                                     _right(4, 32, 48, [0.9, 0.95, 0.98, 0.995], _rot(32, 10000.0)), 0.6, 0.8), 128),
        _layer("attention", _attention(2, 2, 128, 0.09, rot=_rot(128, 50000.0)), None),
    ],
}
# four copies, a loop that ends with the model, a width that is no multiple of 4
PX_D = {
    "architecture": "Pukinex", "vocab": 90, "width": 42, "norm": {"eps": 1e-5}, "embedding": {"scale": 2.0},
    "residual_mult": 0.6, "streams": 4, "loop": {"start": 1, "stop": 2, "times": 2}, "logit_scale": 2.0,
    "layers": [
        _layer("parallel", _parallel(_left(5, 5, 6, 8, 0.4, 33, 8, (0.7, 9)),
                                     _right(2, 10, 4, [0.999, 0.9], _rot(6, 64.0)), 0.9, 0.9), 20),
        _layer("attention", _attention(6, 1, 8, 0.35, softcap=5.0, rot=_rot(2, 20.0, 1.5)), 36),
    ],
}
# (configuration, how the random weights are drawn, page size)
ALL = {
    "PA": (PX_A, {"seed": 41, "std": 0.1, "norm_std": 0.1}, 16),
    "PB": (PX_B, {"seed": 42, "std": 0.1, "norm_std": 0.1}, 8),
    "PC": (PX_C, {"seed": 43, "std": 0.06, "norm_std": 0.1}, 32),
    "PD": (PX_D, {"seed": 44, "std": 0.12, "norm_std": 0.1}, 16),
}


def write_folder(folder, tag: str, dtype: str):
    """A model folder of configuration ``tag``: seeded random weights, with the tensors that random draws leave
    without effect redrawn so that every mechanism matters: distance tables that move scores by several units,
    connections between the copies of the stream that keep their size (columns of the mixing matrix that sum
    to about one), head gates that are not all half open."""
    import torch
    from safetensors.torch import load_file, save_file

    from tokamak_b200.weights import write_random_model

    raw, init, _ = ALL[tag]
    write_random_model(folder, raw, dtype=dtype, **init)
    path = str(folder) + "/model.safetensors"
    tensors = load_file(path)
    gen = torch.Generator().manual_seed(init["seed"] + 1000)
    for name, t in tensors.items():
        draw = lambda std: std * torch.randn(t.shape, generator=gen)
        if name.endswith(".rel"):
            tensors[name] = draw(1.5).to(t.dtype)
        elif name.endswith(".mix") and ".hc" in name:
            s = t.shape[0]
            tensors[name] = (torch.eye(s) * 0.7 + 0.3 / s + draw(0.1)).to(t.dtype)
        elif name.endswith(".in") and ".hc" in name:
            tensors[name] = (1.0 / t.shape[0] + draw(0.2)).to(t.dtype)
        elif name.endswith("mix.g"):
            tensors[name] = draw(4.0 * init["std"]).to(t.dtype)
    save_file({k: v.contiguous() for k, v in tensors.items()}, path)
    return folder
