"""A slow float64 implementation of every mechanism of the Tarivik design, one function each,
written from the equations.  It shares nothing with the package: tests compare the engine with it.

All functions take and return ``torch.float64`` tensors on the CPU; a sequence is processed whole
(``[T, ...]``), position ``t`` of the sequence being row ``t``.
"""

from __future__ import annotations

import json
import math
from pathlib import Path

import torch

F64 = torch.float64

# ``ROUND`` is applied wherever an engine that keeps activations in 16 bits rounds them: at the input
# and the output of every matrix product.  The identity by default; :func:`forward` with ``round_to``
# swaps it for the duration of a call.
ROUND = lambda x: x


def rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    """``x / sqrt(mean(x^2) + eps)`` over the last axis."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def group_norm(x: torch.Tensor, w: torch.Tensor, groups: int, eps: float) -> torch.Tensor:
    """The last axis in ``groups`` equal consecutive parts, each divided by its own root mean square,
    the whole multiplied by ``w``."""
    shape = x.shape
    return rms(x.reshape(*shape[:-1], groups, shape[-1] // groups), eps).reshape(shape) * w


def silu(z: torch.Tensor) -> torch.Tensor:
    return z / (1.0 + torch.exp(-z))


def softplus(z: torch.Tensor) -> torch.Tensor:
    return torch.where(z > 30.0, z, torch.log1p(torch.exp(torch.clamp(z, max=30.0))))


def log_sigmoid(z: torch.Tensor) -> torch.Tensor:
    return -softplus(-z)


def causal_conv(x: torch.Tensor, taps: torch.Tensor) -> torch.Tensor:
    """``y[t, c] = sum_j taps[c, j] x[t - (K - 1) + j, c]``, zeros before the start (the last column
    weighs the current token)."""
    T, _ = x.shape
    K = taps.shape[1]
    y = torch.zeros_like(x)
    for j in range(K):
        back = K - 1 - j
        if back < T:
            y[back:] += taps[:, j] * x[:T - back]
    return y


def input_conv(x: torch.Tensor, taps: torch.Tensor) -> torch.Tensor:
    """What a sublayer reads: the stream plus its own short causal convolution."""
    return x + causal_conv(x, taps)


def linear_state_scan(q, k, v, decay):
    """``S_t = diag(decay_t) S_(t-1) + k_t v_t^T``, ``o_t = S_t^T q_t`` for one head.  ``q, k, decay``
    ``[T, dk]`` (a decay per row of the state), ``v`` ``[T, dv]``."""
    T, dk = k.shape
    S = torch.zeros(dk, v.shape[1], dtype=F64)
    out = torch.zeros(T, v.shape[1], dtype=F64)
    for t in range(T):
        S = decay[t][:, None] * S + torch.outer(k[t], v[t])
        out[t] = S.T @ q[t]
    return out


def hgrn2_mixer(h, w, m, eps):
    """Linear attention whose forget gate also decides what is written: the key is ``1 - f``."""
    T = h.shape[0]
    H, dk, dv = m["heads"], m["dim"], m["vdim"]
    h = ROUND(h)
    q = silu(ROUND(h @ w["q"].T)).view(T, H, dk)
    v = ROUND(h @ w["v"].T).view(T, H, dv)
    lower = w["lower"]
    f = (lower + (1.0 - lower) * torch.sigmoid(ROUND(h @ w["f"].T) + w["f.b"])).view(T, H, dk)
    o = torch.stack([linear_state_scan(q[:, i], 1.0 - f[:, i], v[:, i], f[:, i]) for i in range(H)], 1)
    y = ROUND(rms(o, eps) * w["norm"])
    return ROUND(y.reshape(T, H * dv) @ w["o"].T)


def mlstm_scan(q, k, v, gi, gf):
    """Matrix memory with exponential gates held stable by a running maximum that starts at zero.
    ``gi``, ``gf`` are the logarithms of the input and forget gates, ``[T]``."""
    T, dk = k.shape
    S = torch.zeros(dk, v.shape[1], dtype=F64)
    n = torch.zeros(dk, dtype=F64)
    m = torch.zeros((), dtype=F64)
    out = torch.zeros(T, v.shape[1], dtype=F64)
    for t in range(T):
        m_new = torch.maximum(gf[t] + m, gi[t])
        a, b = torch.exp(gf[t] + m - m_new), torch.exp(gi[t] - m_new)
        S = a * S + b * torch.outer(k[t], v[t])
        n = a * n + b * k[t]
        m = m_new
        out[t] = S.T @ q[t] / (torch.maximum((n @ q[t]).abs(), torch.exp(-m)) + 1e-6)
    return out


def mlstm_mixer(h, w, m, eps):
    T = h.shape[0]
    H, dk, dv, cap = m["heads"], m["dim"], m["vdim"], float(m["gate_cap"])
    h = ROUND(h)
    q = (ROUND(h @ w["q"].T) * dk ** -0.5).view(T, H, dk)
    k = ROUND(h @ w["k"].T).view(T, H, dk)
    v = ROUND(h @ w["v"].T).view(T, H, dv)
    gi = cap * torch.tanh((ROUND(h @ w["i"].T) + w["i.b"]) / cap)
    gf = log_sigmoid(cap * torch.tanh((ROUND(h @ w["f"].T) + w["f.b"]) / cap))
    o = torch.stack([mlstm_scan(q[:, i], k[:, i], v[:, i], gi[:, i], gf[:, i]) for i in range(H)], 1)
    y = rms(o, eps).reshape(T, H * dv) * w["norm"] * torch.sigmoid(ROUND(h @ w["g"].T))
    return ROUND(ROUND(y) @ w["o"].T)


def head_slopes(heads: int) -> torch.Tensor:
    return torch.tensor([2.0 ** (-8.0 * (i + 1) / heads) for i in range(heads)], dtype=F64)


def chunked_attention(q, k, v, scale, chunk, sinks):
    """``q`` ``[T, H, d]``, ``k`` ``[T, G, d]``, ``v`` ``[T, G, dv]``.  A query sees the keys of its own
    chunk of ``chunk`` positions up to itself; a score loses ``slope_h * distance``; ``exp(sink_h)``
    joins the denominator."""
    T, H, _ = q.shape
    G = k.shape[1]
    pos = torch.arange(T)
    dist = (pos[:, None] - pos[None, :]).to(F64)
    seen = (pos[None, :] <= pos[:, None]) & ((pos[:, None] // chunk) == (pos[None, :] // chunk))
    slopes = head_slopes(H)
    out = torch.zeros(T, H, v.shape[2], dtype=F64)
    for i in range(H):
        g = i // (H // G)
        s = (q[:, i] @ k[:, g].T) * scale - slopes[i] * dist
        s = torch.where(seen, s, torch.full_like(s, -math.inf))
        top = torch.maximum(s.max(-1).values, sinks[i])
        e = torch.exp(s - top[:, None])
        out[:, i] = (e @ v[:, g]) / (e.sum(-1) + torch.exp(sinks[i] - top))[:, None]
    return out


def attention_branch(h, w, m, eps):
    """The left half of a parallel mixer."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    h = ROUND(h)
    q = rms(ROUND(h @ w["q"].T + w["q.b"]), eps) * w["q.norm"]
    k = rms(ROUND(h @ w["k"].T + w["k.b"]), eps) * w["k.norm"]
    v = ROUND(h @ w["v"].T + w["v.b"])
    o = chunked_attention(ROUND(q).view(T, H, d), ROUND(k).view(T, G, d), v.view(T, G, dv), float(m["scale"]),
                          int(m["mask"]["size"]), w["sink"])
    y = o.reshape(T, H * dv) * torch.sigmoid(ROUND(h @ w["g"].T))
    return ROUND(ROUND(y) @ w["o"].T)


def ssd_branch(h, w, m, eps):
    """The right half of a parallel mixer: a state-space layer with a scalar decay per head."""
    T = h.shape[0]
    H, dv, N, G = m["heads"], m["vdim"], m["state"], m["groups"]
    inner = H * dv
    h = ROUND(h)
    proj = ROUND(h @ w["in"].T)
    z, xbc, dt = proj[:, :inner], proj[:, inner:2 * inner + 2 * G * N], proj[:, 2 * inner + 2 * G * N:]
    xbc = silu(causal_conv(xbc, w["conv"]) + w["conv.b"])
    x = xbc[:, :inner].view(T, H, dv)
    B = xbc[:, inner:inner + G * N].view(T, G, N)
    C = xbc[:, inner + G * N:].view(T, G, N)
    dt = softplus(dt + w["dt_bias"])
    decay = torch.exp(-torch.exp(w["A_log"]) * dt)
    ys = []
    for i in range(H):
        g = i // (H // G)
        y = linear_state_scan(C[:, g], B[:, g], dt[:, i, None] * x[:, i], decay[:, i, None].expand(T, N))
        ys.append(y + w["D"][i] * x[:, i])
    y = torch.stack(ys, 1).reshape(T, inner) * silu(z)
    y = group_norm(y, w["norm"], int(m["norm_groups"]), eps)
    return ROUND(ROUND(y) @ w["o"].T)


def parallel_mixer(h, w, m, eps):
    left = {k[len("left."):]: t for k, t in w.items() if k.startswith("left.")}
    right = {k[len("right."):]: t for k, t in w.items() if k.startswith("right.")}
    return (float(m["left_scale"]) * attention_branch(h, left, m["left"], eps)
            + float(m["right_scale"]) * ssd_branch(h, right, m["right"], eps))


def route(h, router, correction, top, n_groups, keep):
    """``(chosen experts [T, top], their weights [T, top])``.  Scores are sigmoids of the router's
    logits; the choice is made on score plus correction, inside the ``keep`` groups of neighbouring
    experts whose two best choice scores add up highest; the weights are the plain scores."""
    s = torch.sigmoid(h @ router.T)
    choice = s + correction
    T, E = s.shape
    size = E // n_groups
    grouped = choice.view(T, n_groups, size)
    group_score = grouped.topk(min(2, size), dim=-1).values.sum(-1)
    kept = group_score.topk(keep, dim=-1).indices
    allowed = torch.zeros(T, n_groups, dtype=torch.bool)
    allowed.scatter_(1, kept, True)
    masked = torch.where(allowed[:, :, None].expand(T, n_groups, size).reshape(T, E), choice,
                         torch.full_like(choice, -math.inf))
    chosen = masked.topk(top, dim=-1).indices
    return chosen, s.gather(1, chosen)


def route_margin(h, router, correction, top, n_groups, keep) -> torch.Tensor:
    """How far every token is from another choice, ``[T]``: the smaller of the gap between the last group
    kept and the best one left out and the gap between the last expert chosen and the best one left out
    among the kept groups (infinite where nothing is left out)."""
    choice = torch.sigmoid(h @ router.T) + correction
    T, E = choice.shape
    size = E // n_groups
    group_score = choice.view(T, n_groups, size).topk(min(2, size), dim=-1).values.sum(-1)
    ranked = group_score.sort(-1, descending=True)
    margin = torch.full((T,), math.inf, dtype=F64)
    if keep < n_groups:
        margin = ranked.values[:, keep - 1] - ranked.values[:, keep]
    allowed = torch.zeros(T, n_groups, dtype=torch.bool)
    allowed.scatter_(1, ranked.indices[:, :keep], True)
    masked = torch.where(allowed[:, :, None].expand(T, n_groups, size).reshape(T, E), choice,
                         torch.full_like(choice, -math.inf)).sort(-1, descending=True).values
    if top < keep * size:
        margin = torch.minimum(margin, masked[:, top - 1] - masked[:, top])
    return margin


def moe(h, w, m, margins_out: list | None = None):
    """A mixture of silu-gated experts; the output is the weighted sum of the chosen experts'."""
    r = m["router"]
    h = ROUND(h)
    if margins_out is not None:
        margins_out.append(route_margin(h, w["router"], w["correction"], int(r["top"]), int(r["groups"]["count"]),
                                        int(r["groups"]["keep"])))
    chosen, weights = route(h, w["router"], w["correction"], int(r["top"]), int(r["groups"]["count"]),
                            int(r["groups"]["keep"]))
    out = torch.zeros_like(h)
    for e in range(int(r["experts"])):
        hit = chosen == e
        rows = hit.any(-1)
        if not rows.any():
            continue
        x = h[rows]
        act = ROUND(silu(ROUND(x @ w[f"e{e}.gate"].T)) * ROUND(x @ w[f"e{e}.up"].T))
        y = ROUND(act @ w[f"e{e}.down"].T)
        out[rows] += (weights * hit)[rows].sum(-1, keepdim=True) * y
    return out


MIXERS = {"hgrn2": hgrn2_mixer, "mlstm": mlstm_mixer, "parallel": parallel_mixer}


def _sub(tensors: dict, prefix: str) -> dict:
    return {k[len(prefix):]: t for k, t in tensors.items() if k.startswith(prefix)}


def forward(cfg: dict, tensors: dict, tokens, round_to: torch.dtype | None = None, layers_out: list | None = None,
            margins_out: list | None = None):
    """Float64 logits ``[T, vocab]`` of one whole sequence; ``layers_out`` collects the stream after
    every layer, ``margins_out`` every router's distance from another choice, token by token.  ``round_to``
    rounds where an engine with 16-bit activations rounds."""
    global ROUND
    keep = ROUND
    if round_to is not None:
        ROUND = lambda x: x.to(round_to).to(F64)
    try:
        w = {k: t.to(F64) for k, t in tensors.items()}
        eps, groups = float(cfg["norm"]["eps"]), int(cfg["norm"]["groups"])
        tokens = torch.as_tensor(tokens, dtype=torch.long)
        T = tokens.numel()
        x = w["embed"][tokens] + w["pos"][:T]
        for i, lay in enumerate(cfg["layers"]):
            p = f"l{i}."
            h = input_conv(x, w[p + "canon1"])
            x = x + group_norm(MIXERS[lay["type"]](h, _sub(w, p + "mix."), lay["mixer"], eps), w[p + "norm1"], groups, eps)
            if lay.get("mlp") is not None:
                h = input_conv(x, w[p + "canon2"])
                x = x + group_norm(moe(h, _sub(w, p + "mlp."), lay["mlp"], margins_out), w[p + "norm2"], groups, eps)
            if layers_out is not None:
                layers_out.append(x.clone())
        return ROUND(group_norm(x, w["final.norm"], groups, eps)) @ w["head"].T
    finally:
        ROUND = keep


def load_folder(folder) -> tuple[dict, dict]:
    """``(config dictionary, name -> tensor)`` of a model folder."""
    from safetensors.torch import load_file
    folder = Path(folder)
    return json.loads((folder / "config.json").read_text()), load_file(str(folder / "model.safetensors"))


def greedy_generate(cfg: dict, tensors: dict, prompt, n: int) -> list[int]:
    """The ``n`` tokens that always taking the largest logit gives."""
    seq, out = list(prompt), []
    for _ in range(n):
        tok = int(forward(cfg, tensors, seq)[-1].argmax())
        out.append(tok)
        seq.append(tok)
    return out
