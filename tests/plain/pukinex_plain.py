"""A slow, plain implementation of the Pukinex design, one function per mechanism, written from the
design's equations.  It shares no code with the package: tensors in, tensors out, a whole sequence at
a time, float64 unless the caller says otherwise.  ``ROUND`` (a function tensor -> tensor) rounds
where an engine of 16 bits rounds: the results of matrix products and the rows that feed them.

Notation: ``x`` rows are tokens ``[T, width]``; ``W`` matrices are ``[out, in]`` and applied as ``x @ W.T``.
"""

from __future__ import annotations

import math

import torch

DT = torch.float64


def no_round(t):
    return t


def bf16_round(t):
    return t.to(torch.bfloat16).to(t.dtype)


def layer_norm(x, w, b, eps):
    mu = x.mean(-1, keepdim=True)
    var = ((x - mu) ** 2).mean(-1, keepdim=True)
    return (x - mu) / torch.sqrt(var + eps) * w + b


def rms_unit(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def rope_angles(positions, dims, base, factor=1.0):
    """[T, dims / 2] angles: position * base^(-2i / dims) / factor."""
    i = torch.arange(dims // 2, dtype=DT)
    freq = base ** (-2.0 * i / dims) / factor
    return positions.to(DT)[:, None] * freq[None, :]


def rotate_neighbours(x, ang):
    """x [T, H, d]: elements (2i, 2i + 1) of the first 2 * ang.shape[1] turn by ang[:, i]."""
    r = 2 * ang.shape[1]
    out = x.clone()
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    u, v = x[..., 0:r:2], x[..., 1:r:2]
    out[..., 0:r:2] = u * c - v * s
    out[..., 1:r:2] = v * c + u * s
    return out


def rotate_halves(x, ang):
    """x [T, H, d]: elements (i, i + r / 2) of the first r = 2 * ang.shape[1] turn by ang[:, i]."""
    half = ang.shape[1]
    out = x.clone()
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    u, v = x[..., :half], x[..., half:2 * half]
    out[..., :half] = u * c - v * s
    out[..., half:2 * half] = v * c + u * s
    return out


def softmax_plus_one(scores, mask):
    """Rows of probabilities whose denominator holds one more term, exp(0): [.., T, T]."""
    s = scores.masked_fill(~mask, -math.inf)
    m = torch.clamp(s.max(-1, keepdim=True).values, min=0.0)
    e = torch.exp(s - m)
    return e / (torch.exp(-m) + e.sum(-1, keepdim=True))


def bucket_of(n: int, rows: int, far: int) -> int:
    half = rows // 2
    if n < half:
        return n
    return min(rows - 1, half + int(math.floor(math.log(n / half) / math.log(far / half) * (rows - half))))


def distance_bias(T, rel, far, positions):
    """[H, T, T] bias rel[bucket(i - j), h] (zero above the diagonal)."""
    rows, heads = rel.shape
    pos = torch.as_tensor(positions)
    dist = pos[:, None] - pos[None, :]
    buckets = torch.tensor([bucket_of(n, rows, far) for n in range(int(dist.max()) + 1)])
    out = rel[buckets[dist.clamp_min(0)]].permute(2, 0, 1)
    return out * (dist >= 0)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def attention_mixer(h, w, m, positions, ROUND=no_round):
    """The 'attention' mixer: values are the unrotated keys, neighbour-pair rotation on part of the head,
    capped scores, one added to the denominator, a gate per head."""
    T = h.shape[0]
    H, G, d = m["heads"], m["kv_heads"], m["dim"]
    q = ROUND(h @ w["q"].T).view(T, H, d)
    k = ROUND(h @ w["k"].T).view(T, G, d)
    v = k.clone()
    rot = m.get("rot")
    if rot:
        ang = rope_angles(positions, rot["dims"], rot["base"], (rot.get("scaling") or {}).get("factor", 1.0))
        q, k = ROUND(rotate_neighbours(q, ang)), ROUND(rotate_neighbours(k, ang))
    rep = H // G
    kk, vv = k.repeat_interleave(rep, dim=1), v.repeat_interleave(rep, dim=1)
    s = torch.einsum("ihd,jhd->hij", q, kk) * m["scale"]
    cap = m.get("softcap")
    if cap:
        s = cap * torch.tanh(s / cap)
    mask = torch.tril(torch.ones(T, T, dtype=torch.bool))
    p = softmax_plus_one(s, mask)
    o = torch.einsum("hij,jhd->ihd", p, vv)
    g = torch.sigmoid(ROUND(h @ w["g"].T))                    # [T, H]
    o = ROUND(o * g[:, :, None]).reshape(T, H * d)
    return ROUND(o @ w["o"].T)


def left_half(h, w, m, eps, positions, ROUND=no_round):
    """Attention without rotation: biases, q and k normed per head with a shared weight, a query
    temperature that grows with the position, a learned bias by bucketed distance, one added to the
    denominator, a gate per channel.  Returns the rows in front of the output projection."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (ROUND(h @ w["q"].T) + w["q.b"]).view(T, H, d)
    k = (ROUND(h @ w["k"].T) + w["k.b"]).view(T, G, d)
    v = ROUND(ROUND(h @ w["v"].T) + w["v.b"]).view(T, G, dv)
    q = rms_unit(q, eps) * w["q.norm"]
    k = ROUND(rms_unit(k, eps) * w["k.norm"])
    qt = m.get("q_temp")
    if qt:
        temp = 1.0 + qt["coef"] * torch.log(torch.floor((positions.to(DT) + 1.0) / qt["every"]) + 1.0)
        q = q * temp[:, None, None]
    q = ROUND(q)
    rep = H // G
    kk, vv = k.repeat_interleave(rep, dim=1), v.repeat_interleave(rep, dim=1)
    s = torch.einsum("ihd,jhd->hij", q, kk) * m["scale"]
    s = s + distance_bias(T, w["rel"], m["bias_max"], positions)
    mask = torch.tril(torch.ones(T, T, dtype=torch.bool))
    p = softmax_plus_one(s, mask)
    o = torch.einsum("hij,jhd->ihd", p, vv).reshape(T, H * dv)
    return o * torch.sigmoid(ROUND(h @ w["g"].T))


def retention_scan(q, k, v, decay, state=None):
    """S_t = decay_h S_(t-1) + k_t v_t^T, o_t = S_t^T q_t; q, k [T, H, d], v [T, H, dv]; returns (o, S)."""
    T, H, d = q.shape
    dv = v.shape[2]
    S = torch.zeros((H, d, dv), dtype=q.dtype) if state is None else state.clone()
    o = torch.zeros((T, H, dv), dtype=q.dtype)
    dec = torch.as_tensor(decay, dtype=q.dtype)[:, None, None]
    for t in range(T):
        S = dec * S + k[t][:, :, None] * v[t][:, None, :]
        o[t] = torch.einsum("hdv,hd->hv", S, q[t])
    return o, S


def right_half(h, w, m, eps, positions, ROUND=no_round, state=None):
    """Retention: rotated q and k (halves), k scaled, a fixed decay per head, each head's output divided
    by its root mean square, a silu gate.  Returns the rows in front of the output projection and the state."""
    T = h.shape[0]
    H, d, dv = m["heads"], m["dim"], m["vdim"]
    q = ROUND(h @ w["q"].T).view(T, H, d)
    k = ROUND(h @ w["k"].T).view(T, H, d)
    v = ROUND(h @ w["v"].T).view(T, H, dv)
    rot = m.get("rot")
    if rot:
        ang = rope_angles(positions, rot["dims"], rot["base"], (rot.get("scaling") or {}).get("factor", 1.0))
        q, k = rotate_halves(q, ang), rotate_halves(k, ang)
    k = k * d ** -0.5
    o, S = retention_scan(q, k, v, m["decay"], state)
    o = rms_unit(o, eps).reshape(T, H * dv)
    g = ROUND(h @ w["g"].T)
    return o * (g * torch.sigmoid(g)), S


def parallel_mixer(h, w, m, eps, positions, ROUND=no_round):
    lw = {k[5:]: t for k, t in w.items() if k.startswith("left.")}
    rw = {k[6:]: t for k, t in w.items() if k.startswith("right.")}
    left = ROUND(left_half(h, lw, m["left"], eps, positions, ROUND) * m["left_scale"])
    right, _ = right_half(h, rw, m["right"], eps, positions, ROUND)
    right = ROUND(right * m["right_scale"])
    # the engine forms both output projections as one product over the stacked rows
    return ROUND(left @ lw["o"].T + right @ rw["o"].T)


def dense_ff(h, w, ROUND=no_round):
    a = torch.relu(ROUND(h @ w["up"].T))
    return ROUND(ROUND(a * a) @ w["down"].T)


def layer_weights(weights, prefix):
    return {k[len(prefix):]: t for k, t in weights.items() if k.startswith(prefix)}


def sublayer_streams(xs, hc, mult, fn, norm_w, norm_b, eps, ROUND):
    """One sublayer over the streams xs [S, T, W]: read, norm, sublayer, mix and write."""
    u = torch.einsum("s,stw->tw", hc["in"], xs)
    y = fn(ROUND(layer_norm(u, norm_w, norm_b, eps)))
    return torch.einsum("st,snw->tnw", hc["mix"], xs) + mult * hc["out"][:, None, None] * y[None]


def forward(cfg, weights, tokens, ROUND=no_round, layers_out=None):
    """Logits [T, vocab] of one sequence from position 0; ``weights`` maps names to float64 tensors.
    ``layers_out``: a list that receives the residual stream (sum of the streams) after every layer run."""
    T = len(tokens)
    positions = torch.arange(T)
    eps = cfg["norm"]["eps"]
    mult = cfg.get("residual_mult", 1.0)
    x = weights["embed"][torch.as_tensor(tokens)] * cfg["embedding"]["scale"]
    streams = cfg.get("streams")
    xs = x[None].repeat(streams or 1, 1, 1)
    loop = cfg.get("loop") or {"start": 0, "stop": 0, "times": 1}
    n = len(cfg["layers"])
    order = list(range(loop["start"])) + list(range(loop["start"], loop["stop"])) * loop["times"] + \
        list(range(loop["stop"], n))
    for i in order:
        lay = cfg["layers"][i]
        w = layer_weights(weights, f"l{i}.")
        mw = layer_weights(w, "mix.")
        if lay["type"] == "attention":
            mix = lambda h: attention_mixer(h, mw, lay["mixer"], positions, ROUND)
        elif lay["type"] == "parallel":
            mix = lambda h: parallel_mixer(h, mw, lay["mixer"], eps, positions, ROUND)
        else:
            raise ValueError(lay["type"])
        ones = {"in": torch.ones(1, dtype=DT), "out": torch.ones(1, dtype=DT), "mix": torch.ones(1, 1, dtype=DT)}
        hc1 = layer_weights(w, "hc1.") if streams else ones
        hc2 = layer_weights(w, "hc2.") if streams else ones
        xs = sublayer_streams(xs, hc1, mult, mix, w["norm1"], w["norm1.b"], eps, ROUND)
        if lay.get("mlp") is not None:
            ff = lambda h: dense_ff(h, layer_weights(w, "mlp."), ROUND)
            xs = sublayer_streams(xs, hc2, mult, ff, w["norm2"], w["norm2.b"], eps, ROUND)
        if layers_out is not None:
            layers_out.append(xs.sum(0))
    x = xs.sum(0)
    h = ROUND(layer_norm(x, weights["final.norm"], weights["final.norm.b"], eps))
    logits = (h @ weights["head"].T) * cfg.get("logit_scale", 1.0)
    cap = cfg.get("logit_softcap")
    if cap:
        logits = cap * torch.tanh(logits / cap)
    return logits


def load_folder(folder):
    """``(config dictionary, name -> float64 tensor)`` of a model folder."""
    import json
    from pathlib import Path

    from safetensors.torch import load_file
    cfg = json.loads((Path(folder) / "config.json").read_text())
    return cfg, {k: v.to(DT) for k, v in load_file(str(Path(folder) / "model.safetensors")).items()}


def greedy_generate(cfg, weights, prompt, n_new):
    seq, out = list(prompt), []
    for _ in range(n_new):
        tok = int(forward(cfg, weights, seq)[-1].argmax())
        out.append(tok)
        seq.append(tok)
    return out
