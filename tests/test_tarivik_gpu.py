"""The Tarivik design on the GPU: every mechanism's kernels against the plain implementation, then whole
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

import tarivik_configs as tc
import traces
from helpers import assert_logits_close, random_tokens
from plain import tarivik_plain as plain

pytestmark = pytest.mark.gpu

ROOT = Path(__file__).resolve().parent.parent
DTYPES = ["float32", "bfloat16"]
TORCH = {"float32": torch.float32, "bfloat16": torch.bfloat16}
F64 = torch.float64
_TMP = []


@functools.lru_cache(maxsize=None)
def folder_of(tag: str, dtype: str) -> Path:
    tmp = tempfile.TemporaryDirectory(prefix=f"tk_{tag}_{dtype}_")
    _TMP.append(tmp)
    return Path(tc.write_folder(tmp.name, tag, dtype))


@functools.lru_cache(maxsize=None)
def _truth(folder: str, tokens: tuple):
    """Logits of the whole sequence, and for every position how close any router came to another choice at
    or before it (a choice made otherwise early in a sequence reaches later positions through the states)."""
    cfg, w = plain.load_folder(folder)
    margins = []
    logits = plain.forward(cfg, w, list(tokens), margins_out=margins)
    risk = torch.stack(margins).min(0).values.cummin(0).values if margins else torch.full((len(tokens),), math.inf)
    return logits, risk


def truth(folder, tokens) -> torch.Tensor:
    return _truth(str(folder), tuple(int(t) for t in tokens))[0]


# bfloat16: a row is judged against what rounding alone costs in its request (the plain implementation
# rounding at every product's input and output, which now and then tips a router to another expert): the
# level is the worst row of the request, the limit four times that and never below the level of a
# well-conditioned row.  A wrong key, state, expert or mask moves a row by about its spread.  So does a router
# that rounding tips elsewhere than in the plain implementation: no row rests on such a close call, and the
# few rows beyond the limit that have a router within CLOSE of another choice, at or before them, are let
# through, counted.
BF16_FLOOR_RMS, BF16_FLOOR_MAX, BF16_TIMES = 0.05, 0.2, 4.0
CLOSE, TIPPED_ROWS, TIPPED_SHARE = 0.03, 2, 0.06


@functools.lru_cache(maxsize=None)
def _rounding_level(folder: str, tokens: tuple) -> tuple[float, float]:
    cfg, w = plain.load_folder(folder)
    want = _truth(folder, tokens)[0]
    rounded = plain.forward(cfg, w, list(tokens), round_to=torch.bfloat16)
    rel = (rounded - want).abs() / want.std(dim=-1, keepdim=True).clamp_min(1e-6)
    return rel.pow(2).mean(-1).sqrt().max().item(), rel.max().item()


def check_rows(results, rows, reqs, folder, dtype, what) -> int:
    n, tipped = 0, []
    for step in sorted(rows):
        got = torch.from_numpy(np.asarray(results[step])).double()
        for i, (rid, p) in enumerate(rows[step]):
            where = f"{what}: step {step}, request {rid!r}, position {p}"
            want, risk = _truth(str(folder), tuple(int(t) for t in reqs[rid]))
            want = want[p]
            n += 1
            if dtype == "float32":
                assert_logits_close(got[i:i + 1], want[None], dtype, where)
                continue
            mine = (got[i] - want).abs() / want.std().clamp_min(1e-6)
            base_rms, base_max = _rounding_level(str(folder), tuple(int(t) for t in reqs[rid]))
            assert torch.isfinite(got[i]).all(), where
            rms = mine.pow(2).mean().sqrt().item()
            ok = (rms <= max(BF16_FLOOR_RMS, BF16_TIMES * base_rms)
                  and mine.max().item() <= max(BF16_FLOOR_MAX, BF16_TIMES * base_max))
            if not ok and risk[p].item() < CLOSE:
                tipped.append((rid, p))
                continue
            assert ok, (f"{where}: off by {rms:.3e} (rms) and {mine.max().item():.3e} (max) of the row's spread; "
                        f"rounding alone costs up to {base_rms:.3e} and {base_max:.3e}")
    assert len(tipped) <= max(TIPPED_ROWS, TIPPED_SHARE * n), f"{what}: {len(tipped)} of {n} rows are off: {tipped}"
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
@pytest.mark.parametrize("width,groups_b,groups_n", [(42, 6, 3), (64, 1, 4), (1032, 4, 1), (96, 2, 2)])
def test_norm_in_groups_behind_a_sublayer_and_in_front_of_the_head(dtype, width, groups_b, groups_n):
    from tokamak_b200.csrc import ops
    gen = torch.Generator().manual_seed(width)
    n = 9
    resid = torch.randn(n, width, generator=gen, dtype=F64) * 3
    branch = (torch.randn(n, width, generator=gen) * torch.linspace(0.01, 30, width)).to(TORCH[dtype])
    wb, wn = torch.rand(width, generator=gen) + 0.5, torch.rand(width, generator=gen) + 0.5
    x = resid + plain.group_norm(branch.double(), wb.double(), groups_b, 1e-5)
    r = dev(resid, torch.float32)
    ops.branch_norm_add(r, dev(branch), dev(wb), None, 1e-5, None, None, branch_groups=groups_b)      # the join alone
    close(r, x, "float32")
    # the same with the partial sums of a split product, the next norm over selected rows: nothing is written back
    r2 = dev(resid, torch.float32)
    parts = torch.stack([branch.float() * 0.25, branch.float() * 0.75])
    rows = i32([7, 0, 3])
    out = torch.empty(3, width, dtype=TORCH[dtype], device="cuda")
    ops.branch_norm_add(r2, dev(parts), dev(wb), None, 1e-5, dev(wn), out, 1e-6, rows, branch_groups=groups_b,
                        next_groups=groups_n)
    close(out, plain.group_norm(x[[7, 0, 3]], wn.double(), groups_n, 1e-6), dtype)
    assert torch.equal(r2.cpu(), resid.float())
    # no branch: the norm in front alone
    out = torch.empty(n, width, dtype=TORCH[dtype], device="cuda")
    ops.branch_norm_add(r, None, None, None, 0.0, dev(wn), out, 1e-6, None, next_groups=groups_n)
    close(out, plain.group_norm(r.cpu().double(), wn.double(), groups_n, 1e-6), dtype)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("taps", [1, 2, 3, 5, 8])
def test_input_convolution_across_steps_slots_and_single_tokens(dtype, taps):
    """h + conv(h) over requests cut into steps of every size: the tail in the request's slot carries the
    last inputs across, also through steps in which every request brings one token (the kernel then moves
    the tail on itself) and steps that a request sits out."""
    from tokamak_b200.csrc import ops
    gen = torch.Generator().manual_seed(taps)
    width = 37
    w = torch.randn(width, taps, generator=gen) * 0.5
    seqs = [torch.randn(sum(c), width, generator=gen) for c in CUTS]
    tail = torch.full((4, max(taps - 1, 1), width), float("nan"), device="cuda")
    tail[SLOTS] = 0.0                                           # a slot is cleared when it is handed out
    tail = tail[:, :taps - 1].contiguous() if taps > 1 else None
    got = run_in_steps(seqs, SLOTS, CUTS, lambda rows, step: ops.short_conv(
        dev(rows), dev(w), tail, step, dtype=TORCH[dtype], add_input=True))
    for g, x in zip(got, seqs):
        close(g, plain.input_conv(x.double(), w.double()), dtype)
    if taps > 1:
        for r, slot in enumerate(SLOTS):                        # the tail is the request's last inputs
            assert torch.equal(tail[slot].cpu(), seqs[r][-(taps - 1):]) or len(seqs[r]) < taps - 1
        assert torch.isnan(tail[1]).all()                       # nobody's slot is nobody's business


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("taps,width", [(2, 64), (4, 520), (7, 36)])
def test_input_convolution_in_steps_of_many_tokens(dtype, taps, width):
    """Steps of 64 tokens and more, where a thread forms several tokens of four channels: requests that begin
    and end anywhere inside such a group of tokens, single tokens among long portions, a request whose window
    reaches back into the tail for its first tokens; bit for bit the results of the steps of few tokens."""
    from tokamak_b200.csrc import ops
    gen = torch.Generator().manual_seed(taps * width)
    w = torch.randn(width, taps, generator=gen) * 0.5
    cuts = [[70, 1, 3, 129, 2], [3, 66, 1, 1, 70], [1, 0, 61, 5, 9]]
    slots = [2, 0, 3]
    seqs = [torch.randn(sum(c), width, generator=gen).to(TORCH[dtype]).float() for c in cuts]

    def run(cuts_of):
        tail = torch.full((4, taps - 1, width), float("nan"), device="cuda")
        tail[slots] = 0.0
        got = run_in_steps(seqs, slots, cuts_of, lambda rows, step: ops.short_conv(
            dev(rows), dev(w), tail, step, dtype=TORCH[dtype], add_input=True))
        return got, tail
    got, tail = run(cuts)
    for g, x in zip(got, seqs):
        close(g, plain.input_conv(x.double(), w.double()), dtype)
    for r, slot in enumerate(slots):
        assert torch.equal(tail[slot].cpu(), seqs[r][-(taps - 1):])
    assert torch.isnan(tail[1]).all()
    small, _ = run([[7] * (len(x) // 7) + [len(x) % 7] for x in seqs])      # every step below 64 tokens
    for a, b in zip(got, small):
        assert torch.equal(a, b)


def _ref_moe(h, w, m):
    return plain.moe(h.double(), {k: v.double() for k, v in w.items()}, m)


@pytest.mark.parametrize("experts,count,keep,top", [(6, 3, 2, 3), (4, 4, 2, 2), (5, 1, 1, 3), (12, 4, 3, 5), (2, 1, 1, 2)])
def test_router_chooses_inside_the_best_groups(experts, count, keep, top):
    """Scores that are laid out by hand: the router is the identity, so a token's logits are its own first
    channels.  A group wins by the sum of its two best choice scores, not by its best; an expert outside
    the kept groups is never chosen, however large its score, also when every choice score inside is
    negative; the weights are the scores without the correction."""
    from tokamak_b200.csrc import ops
    gen = torch.Generator().manual_seed(experts * 10 + top)
    n, width = 64, 16
    h = torch.randn(n, width, generator=gen) * 2.0
    size = experts // count
    if count > 1 and size > 1:
        h[0, :experts] = -3.0
        h[0, 0] = 6.0                            # the best single expert, in a group whose second best is poor
        h[0, size:2 * size] = 1.0                # a group of good ones
    router = torch.zeros(experts, width)
    router[:, :experts] = torch.eye(experts)
    correction = torch.randn(experts, generator=gen) * 0.3
    correction[-1] = -4.0                        # choice scores of the last expert are all negative
    got = ops.moe_route(dev(h), dev(router), dev(correction), top=top, n_groups=count, keep=keep)
    chosen, weights = plain.route(h.double(), router.double(), correction.double(), top, count, keep)
    mine, mine_w = got.chosen.cpu().long(), got.weights.cpu().double()
    assert torch.equal(mine.sort(-1).values, chosen.sort(-1).values)
    order, ref_order = mine.argsort(-1), chosen.argsort(-1)
    assert (mine_w.gather(1, order) - weights.gather(1, ref_order)).abs().max() < 1e-6
    # every pair lies in its expert's stretch of the order, the tiles cover the pairs once
    pairs = got.order.cpu().tolist()
    assert sorted(pairs) == list(range(n * top))
    flat = mine.reshape(-1)
    covered = []
    for e, first, rows in got.tiles[:int(got.n_tiles.item())].cpu().tolist():
        assert 1 <= rows <= ops.moe_tile_rows() and all(int(flat[p]) == e for p in pairs[first:first + rows])
        covered += pairs[first:first + rows]
    assert sorted(covered) == list(range(n * top))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("n,width,ff,experts,count,keep,top", [(70, 48, 40, 6, 3, 2, 3), (1, 64, 72, 4, 1, 1, 2),
                                                                (300, 30, 130, 9, 3, 3, 4)])
def test_mixture_of_experts_against_the_plain_sum(dtype, n, width, ff, experts, count, keep, top):
    from tokamak_b200.csrc import ops
    gen = torch.Generator().manual_seed(n)
    rnd = lambda *s, std=1.0: (torch.randn(*s, generator=gen) * std).to(TORCH[dtype])
    h = rnd(n, width)
    w = {"router": rnd(experts, width, std=0.3).float(), "correction": torch.randn(experts, generator=gen) * 0.1}
    for e in range(experts):
        w[f"e{e}.gate"], w[f"e{e}.up"], w[f"e{e}.down"] = rnd(ff, width, std=0.2), rnd(ff, width, std=0.2), rnd(width, ff, std=0.2)
    m = {"router": {"experts": experts, "top": top, "groups": {"count": count, "keep": keep}}}
    stack = lambda name: dev(torch.stack([w[f"e{e}.{name}"] for e in range(experts)]))
    routing = ops.moe_route(dev(h), dev(w["router"]), dev(w["correction"]), top=top, n_groups=count, keep=keep)
    got = ops.moe_experts(dev(h), routing, stack("gate"), stack("up"), stack("down"))
    close(got, _ref_moe(h, w, m), dtype, scale=2.0)
    # a token's result does not depend on the batch: the same tokens alone and in another order
    pick = torch.randperm(n, generator=gen)[:max(1, n // 3)]
    r2 = ops.moe_route(dev(h[pick]), dev(w["router"]), dev(w["correction"]), top=top, n_groups=count, keep=keep)
    again = ops.moe_experts(dev(h[pick]), r2, stack("gate"), stack("up"), stack("down"))
    assert torch.equal(again.cpu(), got.cpu()[pick])


@pytest.mark.parametrize("n,width,ff,experts,count,keep,top", [(70, 64, 128, 6, 3, 2, 3), (1, 72, 64, 4, 1, 1, 2),
                                                                (700, 136, 192, 9, 3, 3, 4), (5, 256, 320, 16, 4, 2, 1)])
def test_mixture_of_experts_on_the_tensor_cores(n, width, ff, experts, count, keep, top):
    """bfloat16 at sizes the grouped product takes: experts with no row, with a few rows and with more rows
    than a tile; a token's result is the same bit for bit whatever else is in the batch."""
    from tokamak_b200.csrc import ops
    gen = torch.Generator().manual_seed(n + width)
    rnd = lambda *s, std=1.0: (torch.randn(*s, generator=gen) * std).to(torch.bfloat16)
    h = rnd(n, width)
    w = {"router": rnd(experts, width, std=0.3).float(), "correction": torch.randn(experts, generator=gen) * 0.1}
    for e in range(experts):
        w[f"e{e}.gate"], w[f"e{e}.up"], w[f"e{e}.down"] = rnd(ff, width, std=0.2), rnd(ff, width, std=0.2), rnd(width, ff, std=0.2)
    m = {"router": {"experts": experts, "top": top, "groups": {"count": count, "keep": keep}}}
    stack = lambda name: dev(torch.stack([w[f"e{e}.{name}"] for e in range(experts)]))
    assert ops.moe_tc_takes(torch.bfloat16, width, ff)
    gate_up, down = ops.moe_stack_gate_up(stack("gate"), stack("up")), stack("down")
    err = torch.zeros(4, dtype=torch.int32, device="cuda")
    route = lambda x: ops.moe_route(dev(x), dev(w["router"]), dev(w["correction"]), top=top, n_groups=count, keep=keep,
                                    padded=True)
    got = ops.moe_experts_tc(dev(h), route(h), gate_up, down, err)
    close(got, _ref_moe(h, w, m), "bfloat16", scale=2.0)
    pick = torch.randperm(n, generator=gen)[:max(1, n // 3)]
    again = ops.moe_experts_tc(dev(h[pick]), route(h[pick]), gate_up, down, err)
    assert torch.equal(again.cpu(), got.cpu()[pick])
    assert err.tolist()[0] == 0


@pytest.mark.parametrize("n,width,ff,experts,count,keep,top", [(1, 72, 64, 4, 1, 1, 2), (8, 256, 320, 16, 4, 2, 2),
                                                                (16, 64, 128, 2, 1, 1, 2), (5, 136, 192, 9, 3, 3, 4),
                                                                (10, 64, 64, 3, 1, 1, 3), (3, 520, 1088, 8, 4, 2, 2)])
def test_mixture_of_experts_in_steps_of_few_tokens(monkeypatch, n, width, ff, experts, count, keep, top):
    """bfloat16 steps of few tokens, where the chosen experts' weights are streamed once: experts nobody
    chose, experts chosen by more tokens than are worked on at a time (every token takes every expert), rows
    longer than one sweep of a warp; a token's result is the same bit for bit whatever else is in the step.
    The kernel is tried beyond the number of pairs up to which the engine prefers it."""
    from tokamak_b200.csrc import ops
    monkeypatch.setattr(ops, "MOE_SMALL_PAIRS", 64)
    gen = torch.Generator().manual_seed(n * 7 + width)
    rnd = lambda *s, std=1.0: (torch.randn(*s, generator=gen) * std).to(torch.bfloat16)
    h = rnd(n, width)
    w = {"router": rnd(experts, width, std=0.3).float(), "correction": torch.randn(experts, generator=gen) * 0.1}
    for e in range(experts):
        w[f"e{e}.gate"], w[f"e{e}.up"], w[f"e{e}.down"] = rnd(ff, width, std=0.2), rnd(ff, width, std=0.2), rnd(width, ff, std=0.2)
    m = {"router": {"experts": experts, "top": top, "groups": {"count": count, "keep": keep}}}
    stack = lambda name: dev(torch.stack([w[f"e{e}.{name}"] for e in range(experts)]))
    assert ops.moe_small_takes(n, top, width, ff)
    gate_up, down = ops.moe_stack_gate_up(stack("gate"), stack("up")), stack("down")
    route = lambda x: ops.moe_route(dev(x), dev(w["router"]), dev(w["correction"]), top=top, n_groups=count, keep=keep,
                                    padded=True)
    got = ops.moe_experts_small(dev(h), route(h), gate_up, down)
    close(got, _ref_moe(h, w, m), "bfloat16", scale=2.0)
    for keep_rows in (slice(0, 1), slice(n // 2, n), torch.randperm(n, generator=gen)):
        again = ops.moe_experts_small(dev(h[keep_rows]), route(h[keep_rows]), gate_up, down)
        assert torch.equal(again.cpu(), got.cpu()[keep_rows])
    # and beside the tensor-core path over the same weights, which rounds elsewhere
    err = torch.zeros(4, dtype=torch.int32, device="cuda")
    close(ops.moe_experts_tc(dev(h), route(h), gate_up, down, err), got.cpu().double(), "bfloat16", scale=2.0)
    assert err.tolist()[0] == 0


def _attention_setup(dtype, T, H, G, d, dv, page, gen):
    """Random q, k, v of one sequence, and k, v laid into shuffled pages."""
    q = torch.randn(T, H, d, generator=gen).to(TORCH[dtype])
    k = torch.randn(T, G, d, generator=gen).to(TORCH[dtype])
    v = torch.randn(T, G, dv, generator=gen).to(TORCH[dtype])
    return q, k, v


def _paged(k, v, page, gen, n_pages):
    T, G, d = k.shape
    ids = torch.randperm(n_pages, generator=gen)[:-(-T // page)]
    kc = torch.full((n_pages, G, page, d), float("nan"), dtype=k.dtype)
    vc = torch.full((n_pages, G, page, v.shape[2]), float("nan"), dtype=v.dtype)
    for p in range(T):
        kc[ids[p // page], :, p % page] = k[p]
        vc[ids[p // page], :, p % page] = v[p]
    table = torch.full((3, 40), -1, dtype=torch.int32)
    table[1, :len(ids)] = ids.int()
    return dev(kc), dev(vc), dev(table)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("chunk,page", [(24, 16), (16, 16), (7, 8), (200, 16), (1, 4)])
def test_chunked_attention_with_keys_that_stand_out(dtype, chunk, page):
    """One key is made to stand out (query and key scaled so that its score dwarfs the others): the first key
    of the query's chunk must be seen, the last key of the chunk before must not, wherever pages end, in a
    prompt's portion and for a single token; far keys in a long chunk; the sink and the distance bias ride
    along."""
    from tokamak_b200.csrc import ops
    gen = torch.Generator().manual_seed(chunk * 100 + page)
    T, H, G, d, dv = 150, 6, 2, 20, 12
    q, k, v = _attention_setup(dtype, T, H, G, d, dv, page, gen)
    probes = sorted({min(T - 1, i) for i in (T - 1, (T // chunk) * chunk, max(0, (T // chunk) * chunk - 1), chunk - 1, chunk,
                                             2 * chunk + 1)})
    for i in probes:                         # the key that must be seen, and the one that must not
        first = i - i % chunk
        q[i] *= 3.0
        k[first] = (q[i, ::H // G].float() * 0.5).to(k.dtype) if first != i else k[first]
        if first > 0:
            k[first - 1] = (q[i, ::H // G].float() * 2.0).to(k.dtype)
    sinks = torch.randn(H, generator=gen)
    slopes = plain.head_slopes(H).float()
    want = plain.chunked_attention(q.double(), k.double(), v.double(), 0.3, chunk, sinks.double())
    kc, vc, table = _paged(k, v, page, gen, -(-T // page) + 5)
    err = torch.zeros(4, dtype=torch.int32, device="cuda")
    # a portion of a prompt: the last 70 positions in one step
    pos = list(range(T - 70, T))
    out = torch.empty(70, H, dv, dtype=TORCH[dtype], device="cuda")
    ops.attention_plain(dev(q[pos]), out, kc, vc, i32(pos), i32([0] * 70), i32([1]), table, err, scale=0.3,
                        sinks=dev(sinks), chunk=chunk, slopes=dev(slopes))
    close(out, want[pos], dtype, scale=4.0)
    # single tokens, each a request of its own step
    for i in probes:
        out = torch.empty(1, H, dv, dtype=TORCH[dtype], device="cuda")
        ops.attention_plain(dev(q[i:i + 1]), out, kc, vc, i32([i]), i32([0]), i32([1]), table, err, scale=0.3,
                            sinks=dev(sinks), chunk=chunk, slopes=dev(slopes))
        close(out, want[i:i + 1], dtype, scale=4.0)
    assert err.tolist()[0] == 0


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


@pytest.mark.parametrize("chunk", [24, 64, 100, 256, 1000])
@pytest.mark.parametrize("H,G,d", [(8, 2, 64), (4, 4, 128), (6, 1, 128)])
def test_chunked_attention_on_the_tiled_kernels(chunk, H, G, d):
    """bfloat16 heads of 64 and 128 channels go to the tensor-core kernels, which know the chunks, the distance
    bias and the sinks too: a prompt's portion that crosses chunks and blocks of 256 rows, single tokens at the
    chunks' edges (equal splits and tiles dealt out), and both kinds in one step, with keys that stand out just
    inside and just outside every probe's chunk."""
    from tokamak_b200.csrc import ops
    from tokamak_b200.cache.device import KVView
    from tokamak_b200.parts.attention import paged_attention
    gen = torch.Generator().manual_seed(chunk * 10 + H)
    T, page = 700, 16
    q, k, v = _attention_setup("bfloat16", T, H, G, d, d, page, gen)
    probes = sorted({min(T - 1, max(0, i)) for c in range(0, T + chunk, chunk) for i in (c - 1, c, c + 1)} | {T - 1, 0})
    probes = probes[:6] + probes[-12:] if len(probes) > 18 else probes
    for i in probes:
        first = i - i % chunk
        q[i] *= 3.0
        if first != i:
            k[first] = (q[i, ::H // G].float() * 0.5).to(k.dtype)
        if first > 0 and (first - 1) not in probes:
            k[first - 1] = (q[i, ::H // G].float() * 2.0).to(k.dtype)
    sinks = torch.randn(H, generator=gen)
    slopes = plain.head_slopes(H).float()
    want = plain.chunked_attention(q.double(), k.double(), v.double(), 0.3, chunk, sinks.double())
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
    kw = dict(scale=0.3, window=None, sinks=dev(sinks), chunk=chunk, slopes=dev(slopes))

    def run(q_lens, starts):
        step = _tiled_step(q_lens, [1] * len(q_lens), starts, H)
        rows = torch.cat([q[s:s + n] for n, s in zip(q_lens, starts)])
        out = torch.full((len(rows), H, d), float("nan"), dtype=torch.bfloat16, device="cuda")
        paged_attention(dev(rows), out, view, step, **kw)
        torch.cuda.synchronize()
        assert step.err.tolist()[0] == 0
        close(out, torch.cat([want[s:s + n] for n, s in zip(q_lens, starts)]), "bfloat16", scale=4.0)
        return step

    assert ops.decode_kernel_takes(H, G, d, page) and ops.prefill_tc_kernel_takes(H, G, d, page)
    run([T], [0])                                # the whole prompt
    run([T - 130], [130])                        # a portion that begins inside a chunk, a page and a key tile
    run([1] * len(probes), probes)               # single tokens
    run([1, T - 333, 1, 1], [probes[-2], 333, probes[1], probes[len(probes) // 2]])      # both kinds in one step
    # the two decode kernels by name, with few and many splits
    step = _tiled_step([1] * len(probes), [1] * len(probes), probes, H)
    rows = dev(torch.cat([q[i:i + 1] for i in probes]))
    ref = torch.cat([want[i:i + 1] for i in probes])
    args = (view.k, view.v, step.decode_items, step.positions, step.tok_req, step.req_slot, view.table, step.err)
    for n_splits in (1, 3, 16):
        out = torch.full_like(rows, float("nan"))
        ops.attention_decode(rows, out, *args, n_splits=n_splits, **kw)
        close(out, ref, "bfloat16", scale=4.0)
    for blocks in (1, 5, 64):
        out = torch.full_like(rows, float("nan"))
        ops.attention_decode_balanced(rows, out, *args, blocks=blocks, **kw)
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


def _state_views(part, slots=4):
    from tokamak_b200.cache.device import KVView, StateView
    from tokamak_b200.cache.manager import StateNeed

    def build(need):
        if isinstance(need, dict):
            return {k: build(v) for k, v in need.items()}
        assert isinstance(need, StateNeed)
        rec = torch.full((slots, *need.shape), float("nan"), device="cuda")
        rec[SLOTS] = 0.0
        return StateView(rec)
    return build(part.cache_need())


def _random_weights(shapes, gen, dtype):
    out = {}
    for name, (shape, std, mean) in shapes.items():
        t = torch.randn(*shape, generator=gen) * std + mean
        out[name] = t.to(TORCH[dtype]).float() if len(shape) == 2 and name not in ("conv",) else t
    return out


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads,dk,dv", [(3, 12, 20), (1, 70, 9), (2, 130, 64)])
def test_hgrn2_mixer_alone_with_its_state_carried_over_steps(dtype, heads, dk, dv):
    from tokamak_b200.parts.hgrn2 import Hgrn2Spec
    gen = torch.Generator().manual_seed(dk)
    width = 40
    w = _random_weights({"q": ((heads * dk, width), 0.3, 0), "f": ((heads * dk, width), 0.3, 0), "f.b": ((heads * dk,), 1.0, 1.0),
                         "lower": ((heads * dk,), 0.0, 0.0), "v": ((heads * dv, width), 0.3, 0),
                         "norm": ((dv,), 0.2, 1.0), "o": ((width, heads * dv), 0.2, 0)}, gen, dtype)
    w["lower"] = torch.rand(heads * dk, generator=gen) * 0.9
    part = _mixer_part("hgrn2", Hgrn2Spec(width, heads, dk, dv, 1e-5), w, dtype)
    view = _state_views(part)
    seqs = [torch.randn(sum(c), width, generator=gen).to(TORCH[dtype]) for c in CUTS]
    got = run_in_steps(seqs, SLOTS, CUTS, lambda rows, step: torch.as_tensor(
        part.forward(dev(rows), step, view)).float().reshape(-1, rows.shape[0], width).sum(0))
    m = {"heads": heads, "dim": dk, "vdim": dv}
    for g, x in zip(got, seqs):
        close(g, plain.hgrn2_mixer(x.double(), {k: v.double() for k, v in w.items()}, m, 1e-5), dtype, scale=3.0)
    assert torch.isnan(view.records[1]).all()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads,dk,dv,cap", [(2, 16, 24, 12.0), (1, 50, 7, 3.0), (3, 8, 64, 30.0)])
def test_mlstm_mixer_alone_with_memory_normaliser_and_maximum_carried(dtype, heads, dk, dv, cap):
    """Gate biases that drive the running maximum far from zero in both directions: a forget gate near one
    with large input gates (the maximum grows), and input gates far below zero (the maximum stays at its
    start, zero, and exp(-m) bounds the normaliser)."""
    from tokamak_b200.parts.mlstm import MlstmSpec
    gen = torch.Generator().manual_seed(dk + 1)
    width = 32
    w = _random_weights({"q": ((heads * dk, width), 0.4, 0), "k": ((heads * dk, width), 0.4, 0), "v": ((heads * dv, width), 0.3, 0),
                         "g": ((heads * dv, width), 0.3, 0), "o": ((width, heads * dv), 0.2, 0), "norm": ((heads * dv,), 0.2, 1.0),
                         "i": ((heads, width), 0.6, 0), "i.b": ((heads,), 0.0, 0.0), "f": ((heads, width), 0.6, 0),
                         "f.b": ((heads,), 0.0, 3.0)}, gen, dtype)
    w["i.b"] = torch.tensor([4.0, -9.0, 0.5][:heads])
    part = _mixer_part("mlstm", MlstmSpec(width, heads, dk, dv, cap, 1e-6), w, dtype)
    view = _state_views(part)
    seqs = [torch.randn(sum(c), width, generator=gen).to(TORCH[dtype]) for c in CUTS]
    got = run_in_steps(seqs, SLOTS, CUTS, lambda rows, step: torch.as_tensor(
        part.forward(dev(rows), step, view)).float().reshape(-1, rows.shape[0], width).sum(0))
    m = {"heads": heads, "dim": dk, "vdim": dv, "gate_cap": cap}
    for g, x in zip(got, seqs):
        close(g, plain.mlstm_mixer(x.double(), {k: v.double() for k, v in w.items()}, m, 1e-6), dtype, scale=3.0)


@pytest.mark.parametrize("dtype", DTYPES)
def test_mlstm_running_maximum_over_long_portions(dtype):
    """Portions longer than one stretch of the gates' scan, ending inside a stretch and inside a lane's share
    of it, beside a single token; the maximum rises in one head and stays at its start in another."""
    from tokamak_b200.parts.mlstm import MlstmSpec
    gen = torch.Generator().manual_seed(77)
    width, heads, dk, dv, cap = 32, 2, 16, 24, 8.0
    w = _random_weights({"q": ((heads * dk, width), 0.4, 0), "k": ((heads * dk, width), 0.4, 0), "v": ((heads * dv, width), 0.3, 0),
                         "g": ((heads * dv, width), 0.3, 0), "o": ((width, heads * dv), 0.2, 0), "norm": ((heads * dv,), 0.2, 1.0),
                         "i": ((heads, width), 0.6, 0), "i.b": ((heads,), 0.0, 0.0), "f": ((heads, width), 0.6, 0),
                         "f.b": ((heads,), 0.0, 3.0)}, gen, dtype)
    w["i.b"] = torch.tensor([3.0, -9.0])
    part = _mixer_part("mlstm", MlstmSpec(width, heads, dk, dv, cap, 1e-6), w, dtype)
    view = _state_views(part)
    cuts = [[150, 1, 137, 1, 2], [1, 1101, 0, 530, 1]]
    seqs = [torch.randn(sum(c), width, generator=gen).to(TORCH[dtype]) for c in cuts]
    got = run_in_steps(seqs, [3, 0], cuts, lambda rows, step: torch.as_tensor(
        part.forward(dev(rows), step, view)).float().reshape(-1, rows.shape[0], width).sum(0))
    m = {"heads": heads, "dim": dk, "vdim": dv, "gate_cap": cap}
    # Hundreds of tokens with a head whose memory stays tiny: the unit norm magnifies what 16-bit products cost,
    # so bfloat16 is judged against the plain implementation rounding where an engine of 16 bits rounds.
    keep = plain.ROUND
    try:
        if dtype == "bfloat16":
            plain.ROUND = lambda t: t.to(torch.bfloat16).double()
        want = [plain.mlstm_mixer(x.double(), {k: v.double() for k, v in w.items()}, m, 1e-6) for x in seqs]
    finally:
        plain.ROUND = keep
    for g, x in zip(got, want):
        close(g, x, dtype, scale=3.0)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads,dv,state,groups,conv,norm_groups", [(4, 8, 16, 2, 4, 2), (3, 10, 5, 3, 1, 1), (2, 32, 70, 1, 5, 4)])
def test_state_space_mixer_alone_with_state_and_convolution_tail_carried(dtype, heads, dv, state, groups, conv, norm_groups):
    from tokamak_b200.parts.ssd import StateSpaceDualSpec
    gen = torch.Generator().manual_seed(state)
    width, inner = 48, heads * dv
    ch = inner + 2 * groups * state
    w = _random_weights({"in": ((inner + ch + heads, width), 0.3, 0), "conv": ((ch, conv), 0.4, 0), "conv.b": ((ch,), 0.3, 0),
                         "dt_bias": ((heads,), 0.5, 0), "A_log": ((heads,), 0.7, -1.0), "D": ((heads,), 0.3, 1.0),
                         "norm": ((inner,), 0.2, 1.0), "o": ((width, inner), 0.2, 0)}, gen, dtype)
    part = _mixer_part("ssd", StateSpaceDualSpec(width, heads, dv, state, groups, conv, norm_groups, 1e-5), w, dtype)
    view = _state_views(part)
    seqs = [torch.randn(sum(c), width, generator=gen).to(TORCH[dtype]) for c in CUTS]
    got = run_in_steps(seqs, SLOTS, CUTS, lambda rows, step: torch.as_tensor(
        part.forward(dev(rows), step, view)).float().reshape(-1, rows.shape[0], width).sum(0))
    m = {"heads": heads, "vdim": dv, "state": state, "groups": groups, "norm_groups": norm_groups}
    for g, x in zip(got, seqs):
        close(g, plain.ssd_branch(x.double(), {k: v.double() for k, v in w.items()}, m, 1e-5), dtype, scale=3.0)


def test_state_space_decay_of_a_write_far_back_float32():
    """One token writes, three hundred later ones neither write nor decay anything but by the known factor:
    what is read out at the end is the write times decay ** 300."""
    from tokamak_b200.csrc import ops
    heads, dv, state, n = 1, 4, 4, 301
    xbc = torch.zeros(n, dv + 2 * state)
    xbc[0, :dv] = torch.tensor([1.0, -2.0, 3.0, 0.5])          # x of the first token
    xbc[0, dv:dv + state] = 1.0                                # its B
    xbc[-1, dv + state:] = 0.25                                # the last token's C
    proj = torch.zeros(n, 1)                                   # dt = softplus(0) = ln 2 everywhere
    a_log = torch.tensor([math.log(0.01)])
    prep = ops.ssd_prepare(dev(xbc), dev(proj), 0, dev(torch.zeros(1)), dev(a_log), dtype=torch.float32, heads=heads,
                           groups=1, state=state, value_dim=dv)
    rec = torch.zeros(2, heads, state, dv, device="cuda")
    step = fake_step([n], [1], [0])
    o = ops.gla_scan(prep, rec, step.req_q_start, step.req_q_len, step.req_slot, step.err).cpu().double()
    dt = math.log(2.0)
    want = xbc[0, :dv].double() * dt * state * 0.25 * math.exp(-0.01 * dt) ** 300
    assert (o[-1, 0] - want).abs().max() <= 1e-4 * want.abs().max()      # three hundred float32 products


# ======================================================================= whole models

LENGTHS = {"TA": [5, 17, 33, 70, 130, 96, 41, 128], "TB": [1, 7, 31, 64, 100, 143, 52, 90],
           "TC": [3, 40, 77, 150, 64, 110, 25, 95], "TD": [2, 66, 129, 20, 90, 151, 47, 80]}
TAGS = ["TA", "TB", "TC", "TD"]


def requests_for(tag):
    vocab = tc.ALL[tag][0]["vocab"]
    return {f"r{i}": random_tokens(vocab, n, seed=100 * i + n) for i, n in enumerate(LENGTHS[tag])}


def make_core(tag, dtype, max_tokens, max_live=4):
    from tokamak_b200.engine.replay import build_core
    return build_core(folder_of(tag, dtype), dtype, max_tokens, page_size=tc.ALL[tag][2], max_live=max_live)


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
def test_tail_decoded_one_by_one_across_every_chunk_border(tag, dtype):
    replay(tag, dtype, traces.tail_one_by_one, max_tokens=192, tail=60)


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
@pytest.mark.parametrize("tag,dtype", [("TA", "float32"), ("TB", "bfloat16"), ("TC", "bfloat16"), ("TD", "float32")])
def test_mixed_batches_in_other_orders_with_two_slots(tag, dtype, seed):
    replay(tag, dtype, traces.mixed, max_tokens=320, poison=True, seed=seed, max_live=2)


@pytest.mark.parametrize("dtype", DTYPES)
def test_first_tokens_and_long_decode(dtype):
    """Positions 0, 1, 2 one by one, then 220 more decoded one by one: over many pages and chunks, with every
    state and every convolution tail carried through every one of them."""
    from tokamak_b200.engine.replay import run_trace
    tag = "TA"
    reqs = {"long": random_tokens(tc.ALL[tag][0]["vocab"], 224, seed=5)}
    records, rows = traces.tail_one_by_one(reqs, tail=223)
    results = run_trace(make_core(tag, dtype, 256), records)
    check_rows(results, rows, reqs, folder_of(tag, dtype), dtype, f"long/{dtype}")


def test_same_logits_however_cut_float32():
    from tokamak_b200.engine.replay import run_trace
    tag = "TB"
    reqs = requests_for(tag)
    got = {}
    for name, builder in (("whole", traces.whole), ("portions", traces.portions)):
        records, rows = builder(reqs)
        res = run_trace(make_core(tag, "float32", 192), records)
        got[name] = {rp: res[s][i] for s in rows for i, rp in enumerate(rows[s])}
    for rp, a in got["whole"].items():
        b = got["portions"][rp]
        assert np.abs(a - b).max() <= 2e-5 * max(1.0, np.abs(a).max()), rp


@pytest.mark.parametrize("tag", ["TA", "TC"])
def test_residual_stream_after_every_layer_float32(tag):
    """Layer by layer: what each block leaves, joined to the stream, against the plain implementation."""
    from tokamak_b200.engine.step import StepEntry
    core = make_core(tag, "float32", 64)
    caught = []
    for block in core.model.blocks.values():
        def wrapped(resid, pending, step, view, fwd=block.forward):
            r, p = fwd(resid, pending, step, view)
            x = (p.x.float() if p.x.dim() == 2 else p.x.sum(0)).double().cpu()
            assert p.layer_scale is None
            caught.append(r.double().cpu() + plain.group_norm(x, p.weight.double().cpu(), p.groups, p.eps))
            return r, p
        block.forward = wrapped
    toks = random_tokens(tc.ALL[tag][0]["vocab"], 40, seed=9)
    core.step.run([StepEntry("a", toks, [39])])
    cfg, w = plain.load_folder(folder_of(tag, "float32"))
    want = []
    plain.forward(cfg, w, toks, layers_out=want)
    assert len(caught) == len(want)
    for i, got in enumerate(caught):
        err = (got - want[i]).abs().max().item()
        assert err <= 2e-4 * max(1.0, want[i].abs().max().item()), f"layer {i} is off by {err:.3e}"


@pytest.mark.parametrize("tag", ["TA", "TB"])
def test_greedy_generation_through_the_entry_point_float32(tag):
    """LLM.generate with its scheduler: prompts in portions beside decoding requests, fewer slots
    than requests, a pool that is used again; the tokens are the plain implementation's."""
    from tokamak_b200 import LLM, SamplingParams
    folder = folder_of(tag, "float32")
    llm = LLM(folder, dtype="float32", block_size=tc.ALL[tag][2], max_seq_len=128, kv_pool_tokens=256,
              prefill_chunk=24, max_num_batched_tokens=40, max_batch_size=3)
    vocab = tc.ALL[tag][0]["vocab"]
    prompts = [random_tokens(vocab, n, seed=7 * n + 1) for n in (5, 33, 1, 61, 18)]
    outs = llm.generate(prompt_token_ids=prompts, sampling_params=SamplingParams(temperature=0.0, max_new_tokens=10))
    assert llm.last_stats["mixed_steps"] > 0
    cfg, w = plain.load_folder(folder)
    for p, o in zip(prompts, outs):
        assert o.output_token_ids == plain.greedy_generate(cfg, w, p, 10), len(p)


def test_greedy_generation_bfloat16_with_graphs_picks_top_tokens():
    """Decode steps replayed from CUDA graphs (every part of the design declares them safe): the tokens are
    those of the same engine with every step laid out by the host, and nearly the plain implementation's best
    for their prefix, unless a router stood close to another choice on the way."""
    from tokamak_b200 import LLM, SamplingParams
    tag = "TC"
    folder = folder_of(tag, "bfloat16")
    llm = LLM(folder, dtype="bfloat16", block_size=tc.ALL[tag][2], max_seq_len=128, max_batch_size=4)
    assert llm.core.model.graph_safe()
    prompts = [random_tokens(tc.ALL[tag][0]["vocab"], n, seed=n) for n in (9, 40, 70)]
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
            logits, risk = _truth(str(folder), tuple(seq))
            logits = logits[-1]
            good = bool(logits[tok] >= logits.max() - 0.05 * logits.std())
            assert good or risk[-1].item() < CLOSE, (len(p), len(seq))
            near += good
            total += 1
            seq.append(tok)
    assert near >= 0.7 * total


def test_trace_run_program_on_this_design(tmp_path):
    tag, dtype = "TB", "float32"
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
    vocab = tc.ALL[tag][0]["vocab"]
    results = {s: np.fromfile(out / f"{s}.f32", dtype="<f4").reshape(-1, vocab) for s in rows}
    check_rows(results, rows, reqs, folder, dtype, "trace_run")


def test_generation_from_the_command_line(capsys):
    from tokamak_b200.cli import main
    folder = folder_of("TA", "float32")
    argv = ["--model", str(folder), "--dtype", "float32", "--prompt-len", "21", "--temperature", "0",
            "--max-new-tokens", "9", "--ignore-eos", "--block-size", "16", "--max-seq-len", "64", "--kv-pool-tokens", "256"]
    assert main(argv) == 0
    first = capsys.readouterr().out
    assert main(argv) == 0
    assert capsys.readouterr().out == first and first.strip()
