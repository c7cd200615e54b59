"""The Pukinex design on the GPU: every mechanism's kernels against the plain implementation, then whole
models under every way of cutting and batching their requests, and generation through the engine's entry
point."""

from __future__ import annotations

import functools
import json
import math
import subprocess
import sys
import tempfile
from pathlib import Path
from types import SimpleNamespace

import numpy as np
import pytest
import torch

import pukinex_configs as pc
import traces
from helpers import assert_logits_close, random_tokens
from plain import pukinex_plain as plain

pytestmark = pytest.mark.gpu

ROOT = Path(__file__).resolve().parent.parent
DTYPES = ["float32", "bfloat16"]
TORCH = {"float32": torch.float32, "bfloat16": torch.bfloat16}
_TMP = []


@functools.lru_cache(maxsize=None)
def folder_of(tag: str, dtype: str) -> Path:
    tmp = tempfile.TemporaryDirectory(prefix=f"px_{tag}_{dtype}_")
    _TMP.append(tmp)
    return Path(pc.write_folder(tmp.name, tag, dtype))


@functools.lru_cache(maxsize=None)
def _truth(folder: str, tokens: tuple) -> torch.Tensor:
    cfg, w = plain.load_folder(folder)
    return plain.forward(cfg, w, list(tokens))


# bfloat16: a row is judged against what rounding alone costs in its request (the plain implementation
# rounding at every product's input and output): the level is the worst row of the request, the limit four
# times that and never below the level of a well-conditioned row.  A wrong key, state, bucket or copy of the
# stream moves a row by about its spread.
BF16_FLOOR_RMS, BF16_FLOOR_MAX, BF16_TIMES = 0.04, 0.16, 4.0


@functools.lru_cache(maxsize=None)
def _rounding_level(folder: str, tokens: tuple) -> tuple[float, float]:
    cfg, w = plain.load_folder(folder)
    want = _truth(folder, tokens)
    rounded = plain.forward(cfg, w, list(tokens), ROUND=plain.bf16_round)
    rel = (rounded - want).abs() / want.std(dim=-1, keepdim=True).clamp_min(1e-6)
    return rel.pow(2).mean(-1).sqrt().max().item(), rel.max().item()


def check_rows(results, rows, reqs, folder, dtype, what) -> int:
    n = 0
    for step in sorted(rows):
        got = torch.from_numpy(np.asarray(results[step])).double()
        for i, (rid, p) in enumerate(rows[step]):
            where = f"{what}: step {step}, request {rid!r}, position {p}"
            toks = tuple(int(t) for t in reqs[rid])
            want = _truth(str(folder), toks)[p]
            n += 1
            if dtype == "float32":
                assert_logits_close(got[i:i + 1], want[None], dtype, where)
                continue
            assert torch.isfinite(got[i]).all(), where
            mine = (got[i] - want).abs() / want.std().clamp_min(1e-6)
            base_rms, base_max = _rounding_level(str(folder), toks)
            rms = mine.pow(2).mean().sqrt().item()
            assert (rms <= max(BF16_FLOOR_RMS, BF16_TIMES * base_rms)
                    and mine.max().item() <= max(BF16_FLOOR_MAX, BF16_TIMES * base_max)), (
                f"{where}: off by {rms:.3e} (rms) and {mine.max().item():.3e} (max) of the row's spread; "
                f"rounding alone costs up to {base_rms:.3e} and {base_max:.3e}")
    return n


def dev(x, dtype=None):
    return x.to("cuda", dtype) if dtype is not None else x.to("cuda")


def i32(v):
    return torch.tensor(list(v), dtype=torch.int32, device="cuda")


def close(got, want, dtype, scale=1.0):
    got, want = got.detach().cpu().double(), want.double()
    tol = (2e-5 if dtype == "float32" else 2e-2) * scale
    err = (got - want).abs().max().item()
    assert err <= tol * max(1.0, want.abs().max().item()), f"off by {err:.3e}"


def fake_step(q_lens, slots, starts):
    """What a kernel reads of a step: requests of ``q_lens`` tokens in ``slots``, continuing at ``starts``."""
    tok_req, pos, q_start = [], [], []
    at = 0
    for r, (n, s) in enumerate(zip(q_lens, starts)):
        q_start.append(at)
        tok_req += [r] * n
        pos += list(range(s, s + n))
        at += n
    return SimpleNamespace(tok_req=i32(tok_req), positions=i32(pos), req_q_start=i32(q_start), req_q_len=i32(q_lens),
                           req_slot=i32(slots), req_kv_len=i32([s + n for s, n in zip(starts, q_lens)]),
                           err=torch.zeros(4, dtype=torch.int32, device="cuda"), max_q_len=max(q_lens), n_tokens=at,
                           scratch={})


def run_in_steps(seqs, slots, cuts, fn):
    """Feed sequences (``[T, ...]`` each, one per request) through ``fn(rows of the step, step)`` cut into steps:
    ``cuts[r]`` lists request r's portion sizes, step by step (0: the request sits the step out).  Returns
    the outputs put together again per request."""
    outs = [[] for _ in seqs]
    fed = [0] * len(seqs)
    for s in range(max(len(c) for c in cuts)):
        live = [r for r in range(len(seqs)) if s < len(cuts[r]) and cuts[r][s] > 0]
        step = fake_step([cuts[r][s] for r in live], [slots[r] for r in live], [fed[r] for r in live])
        rows = torch.cat([seqs[r][fed[r]:fed[r] + cuts[r][s]] for r in live])
        y = fn(rows, step)
        assert step.err.tolist()[0] == 0
        at = 0
        for r in live:
            outs[r].append(y[at:at + cuts[r][s]].detach().cpu())
            at += cuts[r][s]
            fed[r] += cuts[r][s]
    assert fed == [len(x) for x in seqs]
    return [torch.cat(o) for o in outs]


CUTS = [[5, 1, 1, 0, 2, 7, 1], [1, 1, 3, 9, 0, 2], [16, 1, 0, 0, 1, 1, 2]]      # the second step is single tokens only
SLOTS = [2, 0, 3]


# ======================================================================= mechanisms alone

@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("copies,width,parts", [(1, 42, 0), (2, 256, 2), (3, 48, 1), (8, 130, 0), (4, 1100, 3)])
def test_copies_of_the_stream_written_read_and_normed(dtype, copies, width, parts):
    """The write of a pending sublayer output to all copies from the old ones, the weighted read and the
    layer norm, against the equations; with a list of rows the copies stay as they are."""
    from tokamak_b200.csrc import ops
    gen = torch.Generator().manual_seed(copies * 1000 + width)
    n = 11
    xs = torch.randn(copies, n, width, generator=gen) * 2.0 + 0.5
    mix = torch.randn(copies, copies, generator=gen)
    write, read = torch.randn(copies, generator=gen), torch.randn(copies, generator=gen)
    w, b = 1.0 + 0.2 * torch.randn(width, generator=gen), torch.randn(width, generator=gen)
    y = torch.randn(max(parts, 1), n, width, generator=gen)
    branch = y if parts else y[0].to(TORCH[dtype])
    y_sum = y.double().sum(0) if parts else branch.double()
    mult, eps = 0.7, 1e-5
    new = torch.einsum("st,snw->tnw", mix.double(), xs.double()) + mult * write.double()[:, None, None] * y_sum[None]
    u = torch.einsum("s,snw->nw", read.double(), new)
    want = plain.layer_norm(u, w.double(), b.double(), eps)
    streams = dev(xs.clone())
    out, got_u = ops.hyper_mix_norm(streams, dev(branch), mix=dev(mix), write=dev(write), read=dev(read), mult=mult,
                                    norm_w=dev(w), norm_b=dev(b), eps=eps, dtype=TORCH[dtype], want_sum=True)
    close(streams, new, "float32")
    close(got_u, u, "float32")
    close(out, want, dtype)
    # nothing pending: only read and norm; defaults are the sum of the copies
    out2, _ = ops.hyper_mix_norm(streams, None, norm_w=dev(w), norm_b=None, eps=eps, dtype=TORCH[dtype])
    close(out2, plain.layer_norm(new.sum(0), w.double(), torch.zeros(width, dtype=torch.float64), eps), dtype)
    close(streams, new, "float32")
    # selected rows: the write is formed for them and not stored
    streams = dev(xs.clone())
    rows = [7, 0, 3]
    out3, _ = ops.hyper_mix_norm(streams, dev(branch), mix=dev(mix), write=dev(write), read=dev(read), mult=mult,
                                 norm_w=dev(w), norm_b=dev(b), eps=eps, dtype=TORCH[dtype], rows=i32(rows))
    close(out3, want[rows], dtype)
    assert torch.equal(streams.cpu(), xs)


def test_one_copy_without_connections_is_the_plain_residual_sum():
    from tokamak_b200.csrc import ops
    gen = torch.Generator().manual_seed(3)
    x, y = torch.randn(1, 6, 20, generator=gen), torch.randn(6, 20, generator=gen)
    streams = dev(x.clone())
    ops.hyper_mix_norm(streams, dev(y), mult=0.25)
    close(streams[0], x[0].double() + 0.25 * y.double(), "float32")


def _pages(n_pages, G, page, d, dv, dtype):
    kc = torch.full((n_pages, G, page, d), float("nan"), dtype=TORCH[dtype], device="cuda")
    vc = torch.full((n_pages, G, page, dv), float("nan"), dtype=TORCH[dtype], device="cuda")
    return kc, vc


def _read_pages(cache, table_row, T, page):
    return torch.stack([cache[table_row[p // page], :, p % page] for p in range(T)]).cpu().double()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H,G,d,dv,rot,halves,norm,weight,bias,temp,from_keys", [
    (4, 2, 12, 12, 8, False, False, False, False, None, True),       # the attention layers' use
    (6, 3, 10, 6, 0, False, True, True, True, (0.5, 4), False),      # the left halves' use
    (3, 1, 70, 33, 70, True, True, False, True, (2.0, 1), False),    # halves over the whole head, unit norm
    (2, 2, 16, 16, 6, True, False, False, True, None, True),
    (5, 5, 7, 9, 0, False, True, True, False, None, False),          # an odd head size
    (4, 2, 64, 32, 0, False, True, True, True, (0.5, 3), False),     # sizes in steps of 4: 16-byte accesses
    (2, 1, 128, 128, 64, False, False, False, False, None, True),
    (3, 3, 20, 8, 12, True, True, True, True, None, False),
])
def test_queries_keys_and_values_head_by_head(dtype, H, G, d, dv, rot, halves, norm, weight, bias, temp, from_keys):
    """Biases, head norms, temperature, both rotations over part of a head, values that are the unrotated
    keys, and the page and slot of every token, over two steps of two requests."""
    from tokamak_b200.csrc import ops
    gen = torch.Generator().manual_seed(H * 100 + d)
    page, T, eps = 4, 13, 1e-5
    nq, nk, nv = H * d, G * d, 0 if from_keys else G * dv
    seqs = [torch.randn(T, nq + nk + nv + (4 if d % 4 == 0 else 5), generator=gen).to(TORCH[dtype]) for _ in range(2)]
    qb = torch.randn(nq, generator=gen) if bias else None
    kb = torch.randn(nk, generator=gen) if bias else None
    vb = torch.randn(nv, generator=gen) if bias and not from_keys else None
    qw = 1.0 + 0.3 * torch.randn(d, generator=gen) if weight else None
    kw = 1.0 + 0.3 * torch.randn(d, generator=gen) if weight else None
    inv_freq = torch.tensor([50.0 ** (-2.0 * i / max(rot, 1)) for i in range(rot // 2)], dtype=torch.float32)
    kc, vc = _pages(12, G, page, d, dv, dtype)
    table = torch.full((3, 5), -1, dtype=torch.int32)
    table[2, :4] = torch.tensor([7, 1, 10, 3])
    table[0, :4] = torch.tensor([4, 11, 0, 8])
    table_d = dev(table)
    q_got = [[], []]
    for lens, starts in (([9, 2], [0, 0]), ([4, 11], [9, 2])):
        step = fake_step(lens, [2, 0], starts)
        rows = torch.cat([seqs[r][s:s + n] for r, (n, s) in enumerate(zip(lens, starts))])
        tab = ops.rope_table(step.positions, dev(inv_freq)) if rot else None
        q = torch.empty(rows.shape[0], H, d, dtype=TORCH[dtype], device="cuda")
        ops.qkv_heads(dev(rows), q, kc, vc, step, table_d, q_off=0, k_off=nq, v_off=None if from_keys else nq + nk,
                      q_bias=dev(qb) if bias else None, k_bias=dev(kb) if bias else None,
                      v_bias=dev(vb) if vb is not None else None, head_norm_eps=eps if norm else None,
                      q_norm=dev(qw) if weight else None, k_norm=dev(kw) if weight else None, table=tab, rotary_dim=rot,
                      halves=halves, temp_coef=temp[0] if temp else 0.0, temp_every=temp[1] if temp else 0)
        assert step.err.tolist()[0] == 0
        q_got[0].append(q[:lens[0]].cpu())
        q_got[1].append(q[lens[0]:].cpu())
    for r, slot in ((0, 2), (1, 0)):
        x = seqs[r].double()
        pos = torch.arange(T)
        qq = (x[:, :nq] + (qb.double() if bias else 0.0)).view(T, H, d)
        kk = (x[:, nq:nq + nk] + (kb.double() if bias else 0.0)).view(T, G, d)
        vv = kk.clone() if from_keys else (x[:, nq + nk:nq + nk + nv] + (vb.double() if vb is not None else 0.0)).view(T, G, dv)
        if norm:
            qq = plain.rms_unit(qq, eps) * (qw.double() if weight else 1.0)
            kk = plain.rms_unit(kk, eps) * (kw.double() if weight else 1.0)
        if temp:
            qq = qq * (1.0 + temp[0] * torch.log(torch.floor((pos.double() + 1.0) / temp[1]) + 1.0))[:, None, None]
        if rot:
            ang = plain.rope_angles(pos, rot, 50.0)
            turn = plain.rotate_halves if halves else plain.rotate_neighbours
            qq, kk = turn(qq, ang), turn(kk, ang)
        close(torch.cat(q_got[r]), qq, dtype, scale=2.0)
        close(_read_pages(kc, table[slot], T, page), kk, dtype, scale=2.0)
        close(_read_pages(vc, table[slot], T, page), vv, dtype, scale=2.0)
    # the rest of the last page of each request was cleared, pages of nobody were not touched
    assert (kc[3, :, 1:] == 0).all() and (vc[8, :, 1:] == 0).all()
    assert torch.isnan(kc[[2, 5, 6, 9]]).all()


def test_distance_table_follows_the_bucket_formula():
    from tokamak_b200.parts.attention import bucketed_distance_table
    gen = torch.Generator().manual_seed(1)
    for rows, far in ((16, 120), (8, 20), (4, 9), (12, 60), (6, 1000), (2, 2), (32, 17)):
        rel = torch.randn(rows, 3, generator=gen)
        tab = bucketed_distance_table(dev(rel), far).cpu()
        assert tab.shape == (3, far + 1)
        for n in range(far + 1):
            assert torch.equal(tab[:, n], rel[plain.bucket_of(n, rows, far)]), (rows, far, n)
        assert plain.bucket_of(far, rows, far) == rows - 1 == plain.bucket_of(far * 7, rows, far)
        assert [plain.bucket_of(n, rows, far) for n in range(rows // 2 + 1)] == list(range(rows // 2 + 1))


def _paged(k, v, page, gen, n_pages):
    T, G, d = k.shape
    ids = torch.randperm(n_pages, generator=gen)[:-(-T // page)]
    kc = torch.full((n_pages, G, page, d), float("nan"), dtype=k.dtype)
    vc = torch.full((n_pages, G, page, v.shape[2]), float("nan"), dtype=v.dtype)
    for p in range(T):
        kc[ids[p // page], :, p % page] = k[p]
        vc[ids[p // page], :, p % page] = v[p]
    table = torch.full((3, 64), -1, dtype=torch.int32)
    table[1, :len(ids)] = ids.int()
    return dev(kc), dev(vc), dev(table)


def _biased_attention(q, k, v, scale, rel, far, cap=None):
    """Plain causal attention of one sequence with the bucketed bias and one added to the denominator."""
    T, H, _ = q.shape
    rep = H // k.shape[1]
    kk, vv = k.repeat_interleave(rep, dim=1), v.repeat_interleave(rep, dim=1)
    s = torch.einsum("ihd,jhd->hij", q, kk) * scale
    if cap:
        s = cap * torch.tanh(s / cap)
    if rel is not None:
        s = s + plain.distance_bias(T, rel, far, torch.arange(T))
    p = plain.softmax_plus_one(s, torch.tril(torch.ones(T, T, dtype=torch.bool)))
    return torch.einsum("hij,jhd->ihd", p, vv)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("rows,far,page", [(8, 20, 16), (16, 120, 8), (4, 9, 4), (12, 60, 16)])
def test_attention_with_a_bias_by_bucketed_distance_and_keys_that_stand_out(dtype, rows, far, page):
    """The learned bias is made so large for one bucket at a time that the keys of that bucket take the whole
    weight: the last distance of a bucket and the first of the next must fall on different sides, also at
    ``far`` and beyond it, across page borders, in a prompt's portion and for single tokens; elsewhere a key far
    back is made to stand out by its score.  One is added to every denominator."""
    from tokamak_b200.csrc import ops
    from tokamak_b200.parts.attention import bucketed_distance_table
    gen = torch.Generator().manual_seed(rows * 100 + far)
    T, H, G, d, dv = 170, 4, 2, 12, 20
    q = torch.randn(T, H, d, generator=gen).to(TORCH[dtype])
    k = torch.randn(T, G, d, generator=gen).to(TORCH[dtype])
    v = torch.randn(T, G, dv, generator=gen).to(TORCH[dtype])
    rel = torch.randn(rows, H, generator=gen)
    for h in range(H):
        rel[(rows // 2 + 3 * h) % rows, h] += 14.0          # a bucket of its own for every head
    q[T - 1] *= 3.0                                           # and a key 160 back that stands out by its score
    k[T - 161] = (q[T - 1, ::H // G].float() * 1.5).to(k.dtype)
    want = _biased_attention(q.double(), k.double(), v.double(), 0.3, rel.double(), far)
    kc, vc, table = _paged(k, v, page, gen, -(-T // page) + 5)
    tab = bucketed_distance_table(dev(rel), far)
    zeros = torch.zeros(H, device="cuda")
    err = torch.zeros(4, dtype=torch.int32, device="cuda")
    pos = list(range(T - 90, T))
    out = torch.empty(90, H, dv, dtype=TORCH[dtype], device="cuda")
    ops.attention_plain(dev(q[pos]), out, kc, vc, i32(pos), i32([0] * 90), i32([1]), table, err, scale=0.3, sinks=zeros,
                        dist_bias=tab)
    close(out, want[pos], dtype, scale=4.0)
    for i in (0, 1, rows // 2, far - 1, far, far + 1, T - 1):
        out = torch.empty(1, H, dv, dtype=TORCH[dtype], device="cuda")
        ops.attention_plain(dev(q[i:i + 1]), out, kc, vc, i32([i]), i32([0]), i32([1]), table, err, scale=0.3,
                            sinks=zeros, dist_bias=tab)
        close(out, want[i:i + 1], dtype, scale=4.0)
    assert err.tolist()[0] == 0
    # the unit in the denominator shows: without any key that scores well the weights do not sum to one
    lone = _biased_attention(q[:1].double() * 0.0, k[:1].double(), v[:1].double(), 0.3, None, far)
    assert torch.allclose(lone[0, 0], 0.5 * v[0, 0].double())


def _tiled_step(q_lens, slots, starts, heads):
    """:func:`fake_step` with what the attention mixer's choice of kernels reads besides."""
    from tokamak_b200.csrc import ops
    step = fake_step(q_lens, slots, starts)
    q_start = step.req_q_start.tolist()
    kv_len = [s + n for s, n in zip(starts, q_lens)]
    rec, n_parts, n_split = ops.prefill_tc_records(q_start, q_lens, kv_len, slots, heads=heads,
                                                   sms=ops.sm_count(torch.device("cuda", 0)))
    step.prefill_tc = ops.PrefillItems(torch.from_numpy(rec).cuda(), n_parts, n_split)
    step.decode_items = i32([q_start[r] for r, n in enumerate(q_lens) if n == 1])
    step.prefill_items = i32([q_start[r] + j for r, n in enumerate(q_lens) if n > 1 for j in range(n)])
    step.prefill_tiles = i32([])
    step.max_kv_len = max(kv_len)
    return step


@pytest.mark.parametrize("rows,far,cap", [(16, 100, None), (8, 300, 12.0), (32, 650, None), (4, 9, None)])
@pytest.mark.parametrize("H,G,d", [(8, 2, 64), (4, 4, 128), (6, 1, 128)])
def test_bucketed_distance_bias_on_the_tiled_kernels(rows, far, cap, H, G, d):
    """bfloat16 heads of 64 and 128 channels go to the tensor-core kernels, which know the distance table too: a
    whole prompt (key tiles wholly beyond the table's last distance, tiles that straddle it, the diagonal), a
    portion that begins inside a page and a key tile, single tokens around every bucket's first distance (equal
    splits and tiles dealt out), and both kinds in one step; every head has a bucket that takes the whole weight."""
    from tokamak_b200.csrc import ops
    from tokamak_b200.cache.device import KVView
    from tokamak_b200.parts.attention import bucketed_distance_table, paged_attention
    gen = torch.Generator().manual_seed(rows * 10 + H)
    T, page = 700, 16
    q = torch.randn(T, H, d, generator=gen).to(torch.bfloat16)
    k = torch.randn(T, G, d, generator=gen).to(torch.bfloat16)
    v = torch.randn(T, G, d, generator=gen).to(torch.bfloat16)
    rel = torch.randn(rows, H, generator=gen)
    for h in range(H):
        rel[(rows // 2 + 3 * h) % rows, h] += 12.0
    edges = sorted({n for n in range(1, far + 1) if plain.bucket_of(n, rows, far) != plain.bucket_of(n - 1, rows, far)})
    probes = sorted({min(T - 1, max(0, e + j)) for e in edges[-6:] + [far] for j in (-1, 0, 1)} | {0, 1, T - 1})
    q[T - 1] *= 2.0
    k[3] = (q[T - 1, ::H // G].float() * 1.5).to(k.dtype)       # a key far back that stands out by its score
    want = _biased_attention(q.double(), k.double(), v.double(), 0.2, rel.double(), far, cap)
    n_pages = -(-T // page) + 7
    ids = torch.randperm(n_pages, generator=gen)[:-(-T // page)]
    kc = torch.full((n_pages, G, page, d), float("nan"), dtype=torch.bfloat16)
    vc = torch.full((n_pages, G, page, d), float("nan"), dtype=torch.bfloat16)
    kc[ids[-1]] = 0.0                            # the rest of a request's last page is cleared by the kernel that writes it
    vc[ids[-1]] = 0.0
    for p in range(T):
        kc[ids[p // page], :, p % page] = k[p]
        vc[ids[p // page], :, p % page] = v[p]
    table = torch.full((3, 64), -1, dtype=torch.int32)
    table[1, :len(ids)] = ids.int()
    view = KVView(dev(kc), dev(vc), dev(table), page, None)
    kw = dict(scale=0.2, window=None, softcap=cap, sinks=torch.zeros(H, device="cuda"),
              dist_bias=bucketed_distance_table(dev(rel), far))

    def run(q_lens, starts):
        step = _tiled_step(q_lens, [1] * len(q_lens), starts, H)
        x = torch.cat([q[s:s + n] for n, s in zip(q_lens, starts)])
        out = torch.full((len(x), H, d), float("nan"), dtype=torch.bfloat16, device="cuda")
        paged_attention(dev(x), out, view, step, **kw)
        torch.cuda.synchronize()
        assert step.err.tolist()[0] == 0
        close(out, torch.cat([want[s:s + n] for n, s in zip(q_lens, starts)]), "bfloat16", scale=4.0)
        return step

    assert ops.decode_kernel_takes(H, G, d, page) and ops.prefill_tc_kernel_takes(H, G, d, page)
    run([T], [0])
    run([T - 130], [130])
    run([1] * len(probes), probes)
    run([1, T - 333, 1, 1], [probes[-2], 333, probes[1], probes[len(probes) // 2]])
    step = _tiled_step([1] * len(probes), [1] * len(probes), probes, H)
    x = dev(torch.cat([q[i:i + 1] for i in probes]))
    ref = torch.cat([want[i:i + 1] for i in probes])
    args = (view.k, view.v, step.decode_items, step.positions, step.tok_req, step.req_slot, view.table, step.err)
    for n_splits in (1, 3, 16):
        out = torch.full_like(x, float("nan"))
        ops.attention_decode(x, out, *args, n_splits=n_splits, **kw)
        close(out, ref, "bfloat16", scale=4.0)
    for blocks in (1, 5, 64):
        out = torch.full_like(x, float("nan"))
        ops.attention_decode_balanced(x, out, *args, blocks=blocks, **kw)
        close(out, ref, "bfloat16", scale=4.0)
    assert step.err.tolist()[0] == 0


def _mixer_part(kind, spec, weights, dtype):
    from tokamak_b200.parts.base import MIXERS, Runtime
    rt = Runtime(device=torch.device("cuda"), dtype=TORCH[dtype])
    cls = MIXERS.get(kind)
    tensors = {}
    for name, req in cls.expected_tensors(spec, "m.").items():
        t = weights[name[2:]]
        tensors[name] = dev(t, torch.float32 if req.role != "matrix" else TORCH[dtype])
    return cls(spec, "m.", tensors, rt)


def _random_weights(shapes, gen, dtype):
    out = {}
    for name, (shape, std, mean) in shapes.items():
        t = torch.randn(*shape, generator=gen) * std + mean
        out[name] = t.to(TORCH[dtype]).float() if len(shape) == 2 else t
    return out


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads,dk,dv,rot", [(3, 12, 20, 8), (1, 70, 9, 70), (2, 130, 64, 0), (4, 16, 16, 2)])
def test_retention_alone_with_its_state_carried_over_steps(dtype, heads, dk, dv, rot):
    from tokamak_b200.cache.device import StateView
    from tokamak_b200.parts.position import NoPositionSpec, RopeHalvesSpec
    from tokamak_b200.parts.retention import RetentionSpec
    gen = torch.Generator().manual_seed(dk)
    width = 40
    w = _random_weights({"q": ((heads * dk, width), 0.3, 0), "k": ((heads * dk, width), 0.3, 0),
                         "v": ((heads * dv, width), 0.3, 0), "g": ((heads * dv, width), 0.3, 0),
                         "o": ((width, heads * dv), 0.2, 0)}, gen, dtype)
    decay = [1.0 - 0.5 ** (h + 2) for h in range(heads)]
    position = RopeHalvesSpec(rot, 200.0, linear_factor=2.0) if rot else NoPositionSpec()
    part = _mixer_part("retention", RetentionSpec(width, heads, dk, dv, tuple(decay), position, 1e-5), w, dtype)
    rec = torch.full((4, heads, dk, dv), float("nan"), device="cuda")
    rec[SLOTS] = 0.0
    view = StateView(rec)
    seqs = [torch.randn(sum(c), width, generator=gen).to(TORCH[dtype]) for c in CUTS]
    got = run_in_steps(seqs, SLOTS, CUTS, lambda rows, step: torch.as_tensor(
        part.forward(dev(rows), step, view)).float().reshape(-1, rows.shape[0], width).sum(0))
    m = {"heads": heads, "dim": dk, "vdim": dv, "decay": decay}
    if rot:
        m["rot"] = {"dims": rot, "base": 200.0, "scaling": {"factor": 2.0}}
    for g, x in zip(got, seqs):
        rows, state = plain.right_half(x.double(), {k: v.double() for k, v in w.items()}, m, 1e-5, torch.arange(len(x)))
        close(g, rows @ w["o"].double().T, dtype, scale=3.0)
    # the state that is left is the plain one's; the slot nobody used was not touched
    close(rec[SLOTS[2]], state, "float32" if dtype == "float32" else dtype, scale=3.0)
    assert torch.isnan(rec[1]).all()


def test_retention_decay_of_a_write_far_back_float32():
    """One token writes, three hundred later ones write nothing: what the last one reads is the write times
    decay ** 300, and with a decay of one the write itself."""
    from tokamak_b200.csrc import ops
    heads, dk, dv, n = 2, 4, 4, 301
    proj = torch.zeros(n, heads * (2 * dk + dv))
    vals = torch.tensor([1.0, -2.0, 3.0, 0.5])
    for h in range(heads):
        proj[0, heads * dk + h * dk:heads * dk + (h + 1) * dk] = 1.0          # the first token's key
        proj[0, 2 * heads * dk + h * dv:2 * heads * dk + (h + 1) * dv] = vals  # and value
        proj[-1, h * dk:(h + 1) * dk] = 0.25                                  # the last token's query
    decay = torch.tensor([0.99, 1.0])
    prep = ops.retention_prepare(dev(proj), dev(decay), None, dtype=torch.float32, q_off=0, k_off=heads * dk,
                                 v_off=2 * heads * dk, heads=heads, key_dim=dk, value_dim=dv, k_scale=0.5)
    rec = torch.zeros(2, heads, dk, dv, device="cuda")
    step = fake_step([n], [1], [0])
    o = ops.gla_scan(prep, rec, step.req_q_start, step.req_q_len, step.req_slot, step.err).cpu().double()
    for h, a in enumerate((0.99, 1.0)):
        want = vals.double() * 0.5 * dk * 0.25 * a ** 300
        assert (o[-1, h] - want).abs().max() <= 1e-4 * want.abs().max()


@pytest.mark.parametrize("activation", ["relu2", "gelu_tanh", "silu"])
@pytest.mark.parametrize("width,ff,n", [(128, 256, 9), (64, 384, 64), (256, 3072, 2048), (128, 200, 700)])
def test_ungated_activation_in_the_products_epilogues(activation, width, ff, n):
    """bfloat16: few tokens take the tcgen05 product whose cluster applies the activation to its summed splits,
    many tokens the product on pairs of SMs that applies it to its accumulators; other sizes the kernel of its
    own.  All against the plain product and activation."""
    from tokamak_b200.csrc import ops
    from tokamak_b200.parts.base import FEED_FORWARDS, Runtime
    from tokamak_b200.parts.feedforward import MlpSpec
    gen = torch.Generator().manual_seed(width + n)
    w = _random_weights({"up": ((ff, width), width ** -0.5, 0), "down": ((width, ff), ff ** -0.5, 0)}, gen, "bfloat16")
    rt = Runtime(device=torch.device("cuda"), dtype=torch.bfloat16)
    part = FEED_FORWARDS.get("mlp")(MlpSpec(width, ff, activation=activation), "f.",
                                    {"f." + k: dev(v, torch.bfloat16) for k, v in w.items()}, rt)
    x = torch.randn(n, width, generator=gen).to(torch.bfloat16)
    step = SimpleNamespace(err=torch.zeros(4, dtype=torch.int32, device="cuda"), scratch={}, n_tokens=n)
    before = ops.LAUNCHES
    got = torch.as_tensor(part.forward(dev(x), step)).float().reshape(-1, n, width).sum(0)
    fused = ff % 128 == 0 and (n <= 64 or ops.pair_gemm_takes(n, ff, width, fused=True))
    assert step.err.tolist()[0] == 0
    z = x.double() @ w["up"].double().T
    act = {"relu2": torch.relu(z) ** 2, "gelu_tanh": plain.gelu_tanh(z), "silu": z * torch.sigmoid(z)}[activation]
    close(got, plain.bf16_round(act) @ w["down"].double().T, "bfloat16", scale=2.0)
    if fused and n <= 64:
        assert ops.LAUNCHES - before == 2        # two products, no kernel between them


@pytest.mark.parametrize("dtype", DTYPES)
def test_ungated_feed_forward_and_capped_logits(dtype):
    from tokamak_b200.csrc import ops
    from tokamak_b200.parts.base import FEED_FORWARDS, Runtime
    from tokamak_b200.parts.feedforward import MlpSpec
    gen = torch.Generator().manual_seed(8)
    width, ff, n = 40, 72, 9
    w = _random_weights({"up": ((ff, width), 0.3, 0), "down": ((width, ff), 0.3, 0)}, gen, dtype)
    rt = Runtime(device=torch.device("cuda"), dtype=TORCH[dtype])
    part = FEED_FORWARDS.get("mlp")(MlpSpec(width, ff), "f.", {"f." + k: dev(v, TORCH[dtype]) for k, v in w.items()}, rt)
    x = torch.randn(n, width, generator=gen).to(TORCH[dtype])
    step = SimpleNamespace(err=torch.zeros(4, dtype=torch.int32, device="cuda"), scratch={}, n_tokens=n)
    got = torch.as_tensor(part.forward(dev(x), step)).float().reshape(-1, n, width).sum(0)
    close(got, plain.dense_ff(x.double(), {k: v.double() for k, v in w.items()}), dtype, scale=3.0)
    # the activation over the partial sums of a split product
    parts = torch.randn(3, n, ff, generator=gen)
    close(ops.unary_act(dev(parts), TORCH[dtype], "relu2"), torch.relu(parts.double().sum(0)) ** 2, dtype, scale=2.0)
    close(ops.unary_act(dev(parts), TORCH[dtype], "gelu_tanh"), plain.gelu_tanh(parts.double().sum(0)), dtype)
    logits = torch.randn(5, 77, generator=gen) * 40.0
    close(ops.logits_scale_cap(dev(logits.clone()), 0.25, 6.0), 6.0 * torch.tanh(logits.double() * 0.25 / 6.0), "float32")
    close(ops.logits_scale_cap(dev(logits.clone()), 3.0, None), logits.double() * 3.0, "float32")


# ======================================================================= whole models

LENGTHS = {"PA": [5, 17, 33, 70, 130, 96, 41, 128], "PB": [1, 7, 31, 64, 100, 143, 52, 90],
           "PC": [3, 40, 77, 150, 64, 110, 25, 95], "PD": [2, 66, 129, 20, 90, 151, 47, 80]}
TAGS = ["PA", "PB", "PC", "PD"]


def requests_for(tag):
    vocab = pc.ALL[tag][0]["vocab"]
    return {f"r{i}": random_tokens(vocab, n, seed=100 * i + n) for i, n in enumerate(LENGTHS[tag])}


def make_core(tag, dtype, max_tokens, max_live=4):
    from tokamak_b200.engine.replay import build_core
    return build_core(folder_of(tag, dtype), dtype, max_tokens, page_size=pc.ALL[tag][2], max_live=max_live)


def replay(tag, dtype, builder, max_tokens, poison=False, max_live=4, **kw):
    from tokamak_b200.engine.replay import run_step
    reqs = requests_for(tag)
    if builder is traces.mixed:
        kw.update(max_tokens=max_tokens, max_live=max_live)
    records, rows = builder(reqs, **kw)
    core = make_core(tag, dtype, max_tokens, max_live)
    results = {}
    for rec in records:
        if poison:
            core.cache.poison_free_pages()
            core.cache.poison_free_state()
        out = run_step(core, rec)
        if out is not None:
            results[rec["step"]] = out
        core.manager.check_invariants()
    assert not core.manager.live_requests()
    assert all(g.num_free == g.num_pages for g in core.manager.kv_groups)
    n = check_rows(results, rows, reqs, folder_of(tag, dtype), dtype, f"{tag}/{dtype}")
    assert n == sum(len(v) for v in rows.values())
    return core


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("tag", TAGS)
def test_whole_prompts(tag, dtype):
    replay(tag, dtype, traces.whole, max_tokens=192)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("tag", TAGS)
def test_tail_decoded_one_by_one_across_every_bucket_and_temperature_step(tag, dtype):
    replay(tag, dtype, traces.tail_one_by_one, max_tokens=192, tail=70)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("tag", TAGS)
def test_portions_of_changing_size(tag, dtype):
    replay(tag, dtype, traces.portions, max_tokens=192)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("tag", TAGS)
def test_mixed_batches_with_pages_and_slots_used_again(tag, dtype):
    replay(tag, dtype, traces.mixed, max_tokens=384, poison=True, seed=7)
    assert sum(LENGTHS[tag]) > 384


@pytest.mark.parametrize("seed", [1, 2])
@pytest.mark.parametrize("tag,dtype", [("PA", "float32"), ("PB", "bfloat16"), ("PC", "bfloat16"), ("PD", "float32")])
def test_mixed_batches_in_other_orders_with_two_slots(tag, dtype, seed):
    replay(tag, dtype, traces.mixed, max_tokens=320, poison=True, seed=seed, max_live=2)


@pytest.mark.parametrize("dtype", DTYPES)
def test_first_tokens_and_long_decode(dtype):
    """Positions 0, 1, 2 one by one, then 220 more decoded one by one: over many pages, beyond the farthest
    bucket and through many steps of the query temperature, with every state carried through every one."""
    from tokamak_b200.engine.replay import run_trace
    tag = "PA"
    reqs = {"long": random_tokens(pc.ALL[tag][0]["vocab"], 224, seed=5)}
    records, rows = traces.tail_one_by_one(reqs, tail=223)
    results = run_trace(make_core(tag, dtype, 256), records)
    check_rows(results, rows, reqs, folder_of(tag, dtype), dtype, f"long/{dtype}")


def test_same_logits_however_cut_float32():
    from tokamak_b200.engine.replay import run_trace
    tag = "PB"
    reqs = requests_for(tag)
    got = {}
    for name, builder in (("whole", traces.whole), ("portions", traces.portions)):
        records, rows = builder(reqs)
        res = run_trace(make_core(tag, "float32", 192), records)
        got[name] = {rp: res[s][i] for s in rows for i, rp in enumerate(rows[s])}
    for rp, a in got["whole"].items():
        b = got["portions"][rp]
        assert np.abs(a - b).max() <= 2e-5 * max(1.0, np.abs(a).max()), rp


@pytest.mark.parametrize("tag", ["PA", "PD", "PB"])
def test_residual_stream_after_every_layer_run_float32(tag):
    """Layer run by layer run (a looped layer counts every time): the sum of the copies of the stream with
    what the block leaves pending written to them, against the plain implementation."""
    from tokamak_b200.csrc import ops
    from tokamak_b200.engine.step import StepEntry
    core = make_core(tag, "float32", 64)
    caught = []
    for block in core.model.blocks.values():
        def wrapped(resid, pending, step, view, fwd=block.forward):
            r, p = fwd(resid, pending, step, view)
            streams = r if r.dim() == 3 else r.unsqueeze(0)
            rows = torch.arange(streams.shape[1], dtype=torch.int32, device="cuda")
            _, u = ops.hyper_mix_norm(streams, p.x, mix=p.mix, write=p.write, mult=p.mult, rows=rows, want_sum=True,
                                      dtype=torch.float32)
            caught.append(u.double().cpu())
            return r, p
        block.forward = wrapped
    toks = random_tokens(pc.ALL[tag][0]["vocab"], 40, seed=9)
    core.step.run([StepEntry("a", toks, [39])])
    cfg, w = plain.load_folder(folder_of(tag, "float32"))
    want = []
    plain.forward(cfg, w, toks, layers_out=want)
    assert len(caught) == len(want) == len(core.model.spec.schedule)
    for i, got in enumerate(caught):
        err = (got - want[i]).abs().max().item()
        assert err <= 2e-4 * max(1.0, want[i].abs().max().item()), f"layer run {i} is off by {err:.3e}"


@pytest.mark.parametrize("tag", ["PA", "PB"])
def test_greedy_generation_through_the_entry_point_float32(tag):
    """LLM.generate with its scheduler: prompts in portions beside decoding requests, fewer slots
    than requests, a pool that is used again; the tokens are the plain implementation's."""
    from tokamak_b200 import LLM, SamplingParams
    folder = folder_of(tag, "float32")
    llm = LLM(folder, dtype="float32", block_size=pc.ALL[tag][2], max_seq_len=128, kv_pool_tokens=256,
              prefill_chunk=24, max_num_batched_tokens=40, max_batch_size=3)
    vocab = pc.ALL[tag][0]["vocab"]
    prompts = [random_tokens(vocab, n, seed=7 * n + 1) for n in (5, 33, 1, 61, 18)]
    outs = llm.generate(prompt_token_ids=prompts, sampling_params=SamplingParams(temperature=0.0, max_new_tokens=10))
    assert llm.last_stats["mixed_steps"] > 0
    cfg, w = plain.load_folder(folder)
    for p, o in zip(prompts, outs):
        assert o.output_token_ids == plain.greedy_generate(cfg, w, p, 10), len(p)


def test_greedy_generation_bfloat16_with_graphs_picks_top_tokens():
    """Decode steps replayed from CUDA graphs (every part of the design declares them safe): the tokens are
    those of the same engine with every step laid out by the host, and nearly the plain implementation's best
    for their prefix."""
    from tokamak_b200 import LLM, SamplingParams
    tag = "PC"
    folder = folder_of(tag, "bfloat16")
    llm = LLM(folder, dtype="bfloat16", block_size=pc.ALL[tag][2], max_seq_len=128, max_batch_size=4)
    assert llm.core.model.graph_safe()
    prompts = [random_tokens(pc.ALL[tag][0]["vocab"], n, seed=n) for n in (9, 40, 70)]
    params = SamplingParams(temperature=0.0, max_new_tokens=12)
    outs = llm.generate(prompt_token_ids=prompts, sampling_params=params)
    replays = llm.core.step.graph_replays
    assert replays > 0
    llm.plain_steps = True
    slow = llm.generate(prompt_token_ids=prompts, sampling_params=params)
    assert llm.core.step.graph_replays == replays
    assert [o.output_token_ids for o in outs] == [o.output_token_ids for o in slow]
    near = total = 0
    for p, o in zip(prompts, outs):
        seq = list(p)
        for tok in o.output_token_ids:
            logits = _truth(str(folder), tuple(seq))[-1]
            near += bool(logits[tok] >= logits.max() - 0.05 * logits.std())
            total += 1
            seq.append(tok)
    assert near >= 0.8 * total


def test_trace_run_program_on_this_design(tmp_path):
    tag, dtype = "PD", "float32"
    reqs = {k: v for k, v in list(requests_for(tag).items())[:4]}
    records, rows = traces.mixed(reqs, max_tokens=256, seed=3)
    folder = folder_of(tag, dtype)
    out = tmp_path / "out"
    proc = subprocess.run(
        [sys.executable, str(ROOT / "bin" / "trace_run"), "--model", str(folder), "--dtype", dtype,
         "--out", str(out), "--max-tokens", "256", "--page-size", "8"],
        input="".join(json.dumps(r) + "\n" for r in records), text=True, capture_output=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert proc.stdout.split() == [w for r in records for w in ("done", str(r["step"]))]
    vocab = pc.ALL[tag][0]["vocab"]
    results = {s: np.fromfile(out / f"{s}.f32", dtype="<f4").reshape(-1, vocab) for s in rows}
    check_rows(results, rows, reqs, folder, dtype, "trace_run")


def test_generation_from_the_command_line(capsys):
    from tokamak_b200.cli import main
    folder = folder_of("PA", "float32")
    argv = ["--model", str(folder), "--dtype", "float32", "--prompt-len", "21", "--temperature", "0",
            "--max-new-tokens", "9", "--ignore-eos", "--block-size", "16", "--max-seq-len", "64", "--kv-pool-tokens", "256"]
    assert main(argv) == 0
    first = capsys.readouterr().out
    assert main(argv) == 0
    assert capsys.readouterr().out == first and first.strip()
