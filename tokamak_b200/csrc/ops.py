"""Python entry points of the CUDA kernels: argument checks, then one C call each.

Every function takes CUDA tensors and launches on PyTorch's current stream, so
the calls can be recorded into a CUDA graph like any other stream work.  There
is no CPU path: a tensor that is not on a CUDA device is an error.
"""

from __future__ import annotations

import os
from dataclasses import dataclass

import numpy as np
import torch

from .lib import library

DTYPE_CODE = {torch.float32: 0, torch.bfloat16: 1}


class KernelError(RuntimeError):
    """A kernel launch failed or refused its arguments."""


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream() -> int:
    """The current stream's handle.  Every launch asks for it, so the fast accessor is used where
    this torch has it (no Stream object is built)."""
    if _raw_stream is not None:
        return _raw_stream(torch.cuda.current_device())
    return torch.cuda.current_stream().cuda_stream


LAUNCHES = 0     # kernels of this library launched (or recorded into a graph) so far
_ACTIVE_CHAINS: list = []      # product chains with queued products (see ProductChain)


def _check(code: int, what: str) -> None:
    global LAUNCHES
    if code != 0:
        raise KernelError(f"{what}: CUDA error {code}")
    LAUNCHES += 1


def _lib():
    """The library, for a wrapper that is about to launch: products that are still queued in a
    chain are launched first, so that no kernel reads a result that does not exist yet."""
    if _ACTIVE_CHAINS:
        flush_chains()
    return library()


def _ptr(t: torch.Tensor | None) -> int | None:
    return None if t is None else t.data_ptr()


def _want(t: torch.Tensor, dtype: torch.dtype | None, name: str) -> None:
    if not t.is_cuda:
        raise KernelError(f"{name} must be a CUDA tensor (the engine has no CPU path)")
    if not t.is_contiguous():
        raise KernelError(f"{name} must be contiguous")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{name} must be {dtype}, got {t.dtype}")


def dtype_code(dtype: torch.dtype) -> int:
    try:
        return DTYPE_CODE[dtype]
    except KeyError:
        raise KernelError(f"unsupported element type {dtype}; the kernels take float32 and bfloat16")


def embed_gather(table: torch.Tensor, ids: torch.Tensor, resid: torch.Tensor, err: torch.Tensor,
                 scale: float = 1.0, accumulate: bool = False) -> None:
    """resid[t] = float32(table[ids[t]]) * scale; with ``accumulate`` the rows are added to what
    ``resid`` holds (a second table, looked up by position)."""
    _want(table, None, "table"); _want(ids, torch.int32, "ids"); _want(resid, torch.float32, "resid")
    n = ids.numel()
    vocab, hidden = table.shape
    if resid.shape[-1] != hidden or resid.numel() < n * hidden:
        raise KernelError("resid is too small for the tokens")
    _check(_lib().tk_embed_gather(table.data_ptr(), dtype_code(table.dtype), ids.data_ptr(),
                                     resid.data_ptr(), n, hidden, vocab, float(scale), int(accumulate), err.data_ptr(),
                                     _stream()),
           "embed_gather")


class UpdateBuffers:
    """Device side of the update list that the kernels opening a step apply (``step_state.cu``):
    the list itself, the engine's slot records and the flat block tables it writes into."""

    def __init__(self, ctl: torch.Tensor, max_rec: int, max_tab: int, records: torch.Tensor,
                 tables: torch.Tensor):
        _want(ctl, torch.int32, "ctl"); _want(records, torch.int32, "records"); _want(tables, torch.int32, "tables")
        if ctl.numel() < 2 + 9 * max_rec + 2 * max_tab:
            raise KernelError("the update list is too small for its limits")
        if records.dim() != 2 or records.shape[1] != library().tk_slot_words():
            raise KernelError(f"slot records must be [slots, {library().tk_slot_words()}]")
        self.ctl, self.max_rec, self.max_tab, self.records, self.tables = ctl, max_rec, max_tab, records, tables

    def args(self) -> tuple:
        return (self.ctl.data_ptr(), self.max_rec, self.max_tab, self.records.data_ptr(),
                self.records.shape[0], self.tables.data_ptr(), self.tables.numel())


def step_begin(upd: UpdateBuffers, token_ids: torch.Tensor, req_q_start: torch.Tensor,
               req_kv_len: torch.Tensor, req_slot: torch.Tensor, req_fed: torch.Tensor | None,
               err: torch.Tensor) -> None:
    """Open a step laid out by the host: apply the pending updates, put the last sampled token of
    every request marked in ``req_fed`` at its place in ``token_ids``, and note in each request's
    record that the cache will hold ``req_kv_len`` positions."""
    for name, t in (("token_ids", token_ids), ("req_q_start", req_q_start), ("req_kv_len", req_kv_len),
                    ("req_slot", req_slot)):
        _want(t, torch.int32, name)
    n = req_slot.numel()
    if req_q_start.numel() < n or req_kv_len.numel() < n or (req_fed is not None and req_fed.numel() < n):
        raise KernelError("a per-request array is shorter than the batch")
    _check(_lib().tk_step_begin(*upd.args(), token_ids.data_ptr(), req_q_start.data_ptr(),
                                   req_kv_len.data_ptr(), req_slot.data_ptr(), _ptr(req_fed), n,
                                   token_ids.numel(), err.data_ptr(), _stream()), "step_begin")


def decode_begin(upd: UpdateBuffers, dec_slots: torch.Tensor, n_reqs: int, max_positions: int,
                 token_ids: torch.Tensor, positions: torch.Tensor, req_kv_len: torch.Tensor,
                 err: torch.Tensor) -> None:
    """Open a step of single next tokens from the slot records alone: token, position and cache
    length of the request in slot ``dec_slots[r]`` go to row ``r`` and its record moves on."""
    for name, t in (("dec_slots", dec_slots), ("token_ids", token_ids), ("positions", positions),
                    ("req_kv_len", req_kv_len)):
        _want(t, torch.int32, name)
        if t.numel() < n_reqs:
            raise KernelError(f"{name} is shorter than the batch")
    _check(_lib().tk_decode_begin(*upd.args(), dec_slots.data_ptr(), n_reqs, max_positions,
                                     token_ids.data_ptr(), positions.data_ptr(), req_kv_len.data_ptr(),
                                     err.data_ptr(), _stream()), "decode_begin")


SAMPLING_MAX_VOCAB = 1 << 21      # the pieces of the first histograms of sampling.cu hold vocab / 8 masses
SAMPLING_MAX_ROWS = 65535


def _sampling_takes(rows: int, vocab: int) -> None:
    if vocab > SAMPLING_MAX_VOCAB or rows > SAMPLING_MAX_ROWS:
        raise KernelError(f"the sampling kernel takes up to {SAMPLING_MAX_ROWS} rows of up to {SAMPLING_MAX_VOCAB} "
                          f"logits, got {rows} x {vocab}")


def sample_slots(logits: torch.Tensor, records: torch.Tensor, row_slot: torch.Tensor,
                 out_tokens: torch.Tensor, err: torch.Tensor) -> None:
    """One token per row of float32 logits, with the parameters, seed and counter of the slot
    record ``records[row_slot[r]]``; the token is also written into the record and its counter
    advanced (see sampling.cu)."""
    _want(logits, torch.float32, "logits"); _want(records, torch.int32, "records")
    _want(row_slot, torch.int32, "row_slot"); _want(out_tokens, torch.int32, "out_tokens")
    rows, vocab = logits.shape
    if row_slot.numel() < rows or out_tokens.numel() < rows:
        raise KernelError("a per-row sampling tensor is shorter than the batch")
    _sampling_takes(rows, vocab)
    _check(_lib().tk_sample_slots(logits.data_ptr(), logits.stride(0), records.data_ptr(),
                                     row_slot.data_ptr(), records.shape[0], out_tokens.data_ptr(), rows, vocab,
                                     err.data_ptr(), _stream()), "sample_slots")


def wait_probe(limit: int, err: torch.Tensor) -> None:
    """Test aid: one block waits on a barrier that nobody arrives at, gives up after ``limit``
    polls and reports it through the error word exactly as the tcgen05 kernels would."""
    _want(err, torch.int32, "err")
    _check(_lib().tk_wait_probe(int(limit), err.data_ptr(), _stream()), "wait_probe")


def probe_mma_issue(mode: int, n: int, reps: int = 96) -> list[dict]:
    """Measurement aid (csrc/tcgen05_probe.cu): what ``reps`` tcgen05.mma of M 128 x N ``n`` x K 16
    cost the issuing thread.  ``mode`` 0: both operands in shared memory; 1: A in tensor memory;
    2 / 3: the same with two issuing threads; 4: eight of N ``n`` from shared memory, then four of
    N 128 with A in tensor memory, as the prefill attention kernel issues them.  Per issuing thread:
    clocks and nanoseconds per product until issued and until done."""
    out = torch.zeros(8, dtype=torch.int64, device="cuda")
    err = torch.zeros(4, dtype=torch.int32, device="cuda")
    _check(_lib().tk_probe_mma_issue(int(mode), int(n), int(reps), out.data_ptr(), err.data_ptr(), _stream()),
           "probe_mma_issue")
    torch.cuda.synchronize()
    if int(err[0]) != 0:
        raise KernelError(f"probe_mma_issue: a bounded wait ran out (code {int(err[0])})")
    host = out.tolist()
    threads = 2 if mode in (2, 3) else 1
    return [{"issue_clk": host[4 * i] / reps, "done_clk": host[4 * i + 1] / reps,
             "issue_ns": host[4 * i + 2] / reps, "done_ns": host[4 * i + 3] / reps} for i in range(threads)]


def probe_softmax_tile(variant: int, warpgroups: int, tiles: int = 400) -> dict:
    """Measurement aid (csrc/tcgen05_probe.cu): clocks per 64-key tile of one softmax warp, with
    ``warpgroups`` warps on every scheduler (1 or 2), in one of the loop's forms (0: as the prefill
    attention kernel has it; 1: four chains for the maximum; 2: the second half of the scores
    loaded under the first half's maximum; 3: both; 4 / 5 / 6: one, two, all four of every four
    exponentials by a polynomial on the multiply-add pipe)."""
    out = torch.zeros(16, dtype=torch.int32, device="cuda")
    _check(_lib().tk_probe_softmax_tile(int(variant), int(warpgroups), int(tiles), sm_count(out.device),
                                        out.data_ptr(), _stream()), "probe_softmax_tile")
    torch.cuda.synchronize()
    h = [int(x) & 0xFFFFFFFF for x in out.tolist()]
    names = ["load", "maximum", "exponentials_store", "store_arrived", "fence"]
    res = {k: h[i] / tiles for i, k in enumerate(names)}
    res["tile"] = h[5] / tiles
    return res


def add_rmsnorm(resid: torch.Tensor, delta: torch.Tensor | None, weight: torch.Tensor,
                out: torch.Tensor, eps: float, rows: torch.Tensor | None = None) -> None:
    """x = resid (+ delta), written back unless ``rows`` is given; out = weight * x * rsqrt(mean x^2 + eps).

    ``delta`` is the branch output in the activation type, or a 3-D float32 tensor of partial
    sums ``[parts, tokens, hidden]`` (from a split-K product) that the kernel adds up."""
    _want(resid, torch.float32, "resid"); _want(weight, torch.float32, "weight"); _want(out, None, "out")
    hidden = resid.shape[-1]
    if weight.numel() != hidden or out.shape[-1] != hidden:
        raise KernelError("norm width mismatch")
    parts, n_parts, part_stride = None, 0, 0
    if delta is not None and delta.dim() == 3:
        _want(delta, torch.float32, "delta partial sums")
        if delta.shape[1:] != resid.shape:
            raise KernelError("partial sums and resid differ in shape")
        parts, n_parts, part_stride, delta = delta, delta.shape[0], delta.stride(0), None
    elif delta is not None:
        _want(delta, out.dtype, "delta")
        if delta.shape != resid.shape:
            raise KernelError("delta and resid differ in shape")
    if rows is not None:
        _want(rows, torch.int32, "rows")
        n_rows = rows.numel()
    else:
        n_rows = resid.numel() // hidden
    if out.numel() < n_rows * hidden:
        raise KernelError("out is too small")
    _check(_lib().tk_add_rmsnorm(resid.data_ptr(), _ptr(delta), _ptr(parts), n_parts, part_stride,
                                    weight.data_ptr(), out.data_ptr(), _ptr(rows), n_rows, hidden,
                                    float(eps), dtype_code(out.dtype), _stream()), "add_rmsnorm")


GLU_ACTIVATIONS = {"silu": 0, "gelu_tanh": 1}


def swiglu(gate_up: torch.Tensor, out: torch.Tensor, block: int = 0, activation: str = "silu") -> None:
    """out[t, j] = act(gate[t, j]) * up[t, j] with act = silu or the tanh form of gelu; a row of ``gate_up`` holds ``block`` gate values,
    then the ``block`` up values of the same outputs, and so on (``block = 0``: all I gate values,
    then all up values).  ``gate_up`` may be float32 partial sums ``[parts, tokens, 2I]`` that the
    kernel adds up first."""
    _want(gate_up, None, "gate_up"); _want(out, None, "out")
    parts, n_parts, part_stride = None, 0, 0
    if gate_up.dim() == 3:
        _want(gate_up, torch.float32, "gate_up partial sums")
        parts, n_parts, part_stride = gate_up, gate_up.shape[0], gate_up.stride(0)
        n, two_i = gate_up.shape[1:]
        gate_up = None
    else:
        if gate_up.dtype != out.dtype:
            raise KernelError("gate_up and out differ in element type")
        n, two_i = gate_up.shape
    if two_i % 2 or out.shape != (n, two_i // 2):
        raise KernelError("swiglu shape mismatch")
    block = block or two_i // 2
    if (two_i // 2) % block:
        raise KernelError("the gate/up block must divide the intermediate size")
    if activation not in GLU_ACTIVATIONS:
        raise KernelError(f"unknown activation {activation!r}; known: {', '.join(GLU_ACTIVATIONS)}")
    _check(_lib().tk_swiglu(_ptr(gate_up), _ptr(parts), n_parts, part_stride, out.data_ptr(), n,
                               two_i // 2, block, dtype_code(out.dtype), GLU_ACTIVATIONS[activation], _stream()),
           "swiglu")


def rope_table(positions: torch.Tensor, inv_freq: torch.Tensor, magnitude: float = 1.0) -> torch.Tensor:
    """``[tokens, len(inv_freq), 2]`` float32: ``magnitude`` times (cos, sin) of ``float(position) * inv_freq[j]``."""
    _want(positions, torch.int32, "positions"); _want(inv_freq, torch.float32, "inv_freq")
    n, half = positions.numel(), inv_freq.numel()
    table = torch.empty((n, half, 2), dtype=torch.float32, device=positions.device)
    _check(_lib().tk_rope_table(positions.data_ptr(), inv_freq.data_ptr(), table.data_ptr(), n, 2 * half,
                                   float(magnitude), _stream()), "rope_table")
    return table


def rope_kv(qkv: torch.Tensor, q_out: torch.Tensor, k_cache: torch.Tensor | None,
            v_cache: torch.Tensor | None, positions: torch.Tensor, tok_req: torch.Tensor,
            req_slot: torch.Tensor, block_table: torch.Tensor, q_norm_w: torch.Tensor | None,
            k_norm_w: torch.Tensor | None, table: torch.Tensor | None, err: torch.Tensor, *,
            n_q_heads: int, n_kv_heads: int, head_dim: int, rotary_dim: int, eps: float,
            write_kv: bool = True, req_q_len: torch.Tensor | None = None,
            req_kv_len: torch.Tensor | None = None) -> None:
    """Per-head norm of q and k, rotation, and the write of k and v into their pages.

    ``qkv`` is ``[tokens, (Hq + 2 Hkv) d]`` in the activation type, or float32 partial sums
    ``[parts, tokens, (Hq + 2 Hkv) d]`` that the kernel adds up.  With ``req_q_len`` and
    ``req_kv_len`` the last token of every request also clears the rest of a page begun in
    this step (the tcgen05 attention kernel loads whole pages and relies on it)."""
    _want(qkv, None, "qkv"); _want(q_out, None, "q_out")
    parts, n_parts = None, 0
    if qkv.dim() == 3:
        _want(qkv, torch.float32, "qkv partial sums")
        parts, n_parts = qkv, qkv.shape[0]
        n, row = qkv.shape[1:]
        qkv = None
    else:
        if qkv.dtype != q_out.dtype:
            raise KernelError("qkv and q_out differ in element type")
        n, row = qkv.shape
    need = (n_q_heads + (2 * n_kv_heads if write_kv else 0)) * head_dim
    if row < need:
        raise KernelError(f"qkv rows hold {row} values, {need} needed")
    for name, t in (("positions", positions), ("tok_req", tok_req), ("req_slot", req_slot),
                    ("block_table", block_table)):
        _want(t, torch.int32, name)
    for name, t in (("q_norm_w", q_norm_w), ("k_norm_w", k_norm_w), ("table", table)):
        if t is not None:
            _want(t, torch.float32, name)
    if head_dim % 4 or rotary_dim % 4 or rotary_dim > head_dim:
        raise KernelError(f"head_dim {head_dim} and rotary_dim {rotary_dim} must be multiples of 4 "
                          f"with rotary_dim <= head_dim")
    if q_norm_w is not None and q_norm_w.numel() != head_dim:
        raise KernelError("q_norm weight does not match head_dim")
    if k_norm_w is not None and k_norm_w.numel() != head_dim:
        raise KernelError("k_norm weight does not match head_dim")
    if table is not None and table.shape != (n, rotary_dim // 2, 2):
        raise KernelError(f"the rotation table must be [{n}, {rotary_dim // 2}, 2], got {tuple(table.shape)}")
    if table is None and rotary_dim != 0:
        raise KernelError("rotary_dim without a rotation table")
    if write_kv:
        _want(k_cache, q_out.dtype, "k_cache"); _want(v_cache, q_out.dtype, "v_cache")
        num_pages, hkv, page_size, d = k_cache.shape
        if hkv != n_kv_heads or d != head_dim or v_cache.shape != k_cache.shape:
            raise KernelError("cache pages do not match the heads")
    else:
        num_pages, page_size = 0, 1
    _check(_lib().tk_rope_kv(_ptr(qkv), _ptr(parts), n_parts, q_out.data_ptr(), _ptr(k_cache), _ptr(v_cache),
                                positions.data_ptr(), tok_req.data_ptr(), req_slot.data_ptr(),
                                block_table.data_ptr(), _ptr(req_q_len), _ptr(req_kv_len),
                                _ptr(q_norm_w), _ptr(k_norm_w), _ptr(table),
                                err.data_ptr(), n, req_slot.numel(), n_q_heads, n_kv_heads, head_dim,
                                rotary_dim, row, page_size, block_table.shape[1], num_pages,
                                1 if write_kv else 0, float(eps), dtype_code(q_out.dtype), _stream()),
           "rope_kv")


def attention_plain(q: torch.Tensor, out: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                    positions: torch.Tensor, tok_req: torch.Tensor, req_slot: torch.Tensor,
                    block_table: torch.Tensor, err: torch.Tensor, *, scale: float,
                    window: int | None = None, items: torch.Tensor | None = None,
                    softcap: float | None = None, sinks: torch.Tensor | None = None,
                    chunk: int | None = None, slopes: torch.Tensor | None = None,
                    dist_bias: torch.Tensor | None = None) -> None:
    """Paged attention of a mixed batch; q is [N, Hq, d], out [N, Hq, dv] with dv the size of a
    value head (``v_cache`` is ``[pages, Hkv, page, dv]``).

    ``q`` is in the pages' type or float32, and may be any view whose last axis is dense (a
    ``[Hq, N, d]`` tensor seen as ``[N, Hq, d]``).  ``v_cache`` may be a view of the leading ``dv``
    elements of the key rows (a cache whose values are part of its keys).  ``items`` restricts the
    work to the listed token indices (rows of q and out).  ``softcap`` bounds the scaled scores
    (``cap * tanh(score / cap)``); ``sinks`` is one float32 per query head whose exponential joins
    the softmax denominator.  ``chunk``: a query sees only the keys of its own block of ``chunk``
    positions (blocks counted from position 0).  ``slopes`` (float32, one per query head): the score of
    the key at distance ``n`` behind the query loses ``slope * n``.  ``dist_bias`` (float32 ``[Hq, L]``): the score
    of the key at distance ``n`` gains ``dist_bias[h, min(n, L - 1)]``."""
    _want(out, k_cache.dtype, "out"); _want(k_cache, None, "k_cache")
    if dist_bias is not None:
        _want(dist_bias, torch.float32, "dist_bias")
        if dist_bias.dim() != 2 or dist_bias.shape[0] != q.shape[1] or dist_bias.shape[1] < 1:
            raise KernelError("the distance bias must be [query heads, distances]")
    if slopes is not None:
        _want(slopes, torch.float32, "slopes")
        if slopes.numel() != q.shape[1]:
            raise KernelError("one slope per query head is needed")
    if not q.is_cuda or q.dtype not in (k_cache.dtype, torch.float32) or q.stride(2) != 1:
        raise KernelError("q must be a CUDA tensor in the pages' type or float32 with a dense last axis")
    n, hq, d = q.shape
    num_pages, hkv, page_size, dk = k_cache.shape
    dv = v_cache.shape[3]
    if dk != d or v_cache.shape[:3] != k_cache.shape[:3] or out.shape != (n, hq, dv) or v_cache.dtype != k_cache.dtype:
        raise KernelError("attention shape mismatch")
    v_stride = v_cache.stride(2)
    if (not v_cache.is_cuda or v_cache.stride(3) != 1 or v_cache.stride(1) != page_size * v_stride
            or v_cache.stride(0) != hkv * page_size * v_stride):
        raise KernelError("v_cache must be laid out like pages, with a row stride of its own at most")
    if max(d, dv) > 1024:
        raise KernelError(f"head sizes {d} / {dv} are beyond the kernel's limit of 1024")
    if sinks is not None:
        _want(sinks, torch.float32, "sinks")
        if sinks.numel() != hq:
            raise KernelError("one sink per query head is needed")
    if hq % hkv:
        raise KernelError(f"{hq} query heads are not a multiple of {hkv} key/value heads")
    _check(_lib().tk_attention_plain(q.data_ptr(), out.data_ptr(), k_cache.data_ptr(),
                                        v_cache.data_ptr(), positions.data_ptr(), tok_req.data_ptr(),
                                        req_slot.data_ptr(), block_table.data_ptr(), _ptr(items),
                                        err.data_ptr(), n if items is None else items.numel(),
                                        req_slot.numel(), hq, hkv, d, page_size,
                                        block_table.shape[1], num_pages, int(window or 0),
                                        float(scale), dtype_code(k_cache.dtype), dv, float(softcap or 0.0),
                                        _ptr(sinks), dtype_code(q.dtype), q.stride(0), q.stride(1), d, v_stride,
                                        int(chunk or 0), _ptr(slopes), _ptr(dist_bias),
                                        dist_bias.shape[1] if dist_bias is not None else 0, _stream()),
           "attention_plain")


def latent_kernel_takes(d: int, dv: int) -> bool:
    """Whether :func:`attention_latent` takes cache rows of ``d`` elements whose leading ``dv`` are the values."""
    return bool(library().tk_attention_latent_takes(d, dv))


def latent_decode_splits(device: torch.device, n_items: int, max_kv_len: int, window: int | None) -> int:
    """Shares that the keys of a single token are cut into: enough blocks for one round over the SMs,
    at least two 64-key tiles a share.  It follows from the step's bucket, not from its lengths."""
    tiles = -(-min(max_kv_len, window or max_kv_len) // 64) + 1
    want = sm_count(device) // max(1, n_items)
    return max(1, min(want, tiles // 2, 128))


def attention_latent(q: torch.Tensor, out: torch.Tensor, cache: torch.Tensor, dv: int, step, block_table: torch.Tensor,
                     *, scale: float, window: int | None = None, sinks: torch.Tensor | None = None,
                     tiles: torch.Tensor | None = None, items: torch.Tensor | None = None, n_splits: int = 1) -> None:
    """Attention over a latent cache on the tensor cores: ``cache`` is ``[pages, 1, page, d]`` bfloat16, the
    values are the rows' leading ``dv`` elements, ``q`` is ``[N, H, d]`` (float32 or bfloat16, any view with a
    dense last axis), ``out`` ``[N, H, dv]`` bfloat16.  Either ``tiles`` (int32 pairs of request row and
    64-token tile: prompt portions) or ``items`` (token indices of requests that bring one token, whose
    keys are cut into ``n_splits`` shares) says what to work on; ``step`` is the batch description."""
    _want(out, torch.bfloat16, "out"); _want(cache, torch.bfloat16, "cache")
    n, heads, d = q.shape
    num_pages, one, page_size, dk = cache.shape
    if one != 1 or dk != d or out.shape != (n, heads, dv) or not latent_kernel_takes(d, dv):
        raise KernelError("the latent attention kernel does not take these sizes")
    if not q.is_cuda or q.dtype not in (torch.float32, torch.bfloat16) or q.stride(2) != 1:
        raise KernelError("q must be a CUDA tensor, float32 or bfloat16, with a dense last axis")
    _want_sinks(sinks, heads)
    if (tiles is None) == (items is None):
        raise KernelError("either tiles or items")
    part_o = part_ml = None
    if tiles is not None:
        _want(tiles, torch.int32, "tiles")
        n_work, n_splits = tiles.numel() // 2, 1
    else:
        _want(items, torch.int32, "items")
        n_work = items.numel()
        if n_splits > 1:
            part_o = torch.empty((n_work, heads, n_splits, dv), dtype=torch.float32, device=q.device)
            part_ml = torch.empty((n_work, heads, n_splits, 2), dtype=torch.float32, device=q.device)
    global LAUNCHES
    _check(_lib().tk_attention_latent(q.data_ptr(), out.data_ptr(), cache.data_ptr(), _ptr(sinks), _ptr(tiles), _ptr(items),
                                         step.positions.data_ptr(), step.tok_req.data_ptr(), step.req_q_start.data_ptr(),
                                         step.req_q_len.data_ptr(), step.req_kv_len.data_ptr(), step.req_slot.data_ptr(),
                                         block_table.data_ptr(), _ptr(part_o), _ptr(part_ml), step.err.data_ptr(),
                                         q.stride(0), q.stride(1), dtype_code(q.dtype), n_work, step.req_slot.numel(),
                                         heads, d, dv, page_size, block_table.shape[1], num_pages, int(window or 0),
                                         int(n_splits), float(scale), _stream()), "attention_latent")
    LAUNCHES += 1 if n_splits > 1 else 0        # the kernel that adds the shares up


def _want_sinks(sinks: torch.Tensor | None, n_q_heads: int) -> None:
    if sinks is not None:
        _want(sinks, torch.float32, "sinks")
        if sinks.numel() != n_q_heads:
            raise KernelError("one sink per query head is needed")


def _want_dist_bias(dist_bias: torch.Tensor | None, n_q_heads: int) -> int:
    """Checks a distance table ``[query heads, distances]`` and returns its number of distances (0: none)."""
    if dist_bias is None:
        return 0
    _want(dist_bias, torch.float32, "dist_bias")
    if dist_bias.dim() != 2 or dist_bias.shape[0] != n_q_heads or dist_bias.shape[1] < 1:
        raise KernelError("the distance bias must be [query heads, distances]")
    return dist_bias.shape[1]


def _parts_of(x: torch.Tensor, like: torch.dtype, name: str):
    """(tensor | None, partial sums | None, number of parts, tokens, row length) of a product's
    result: a 2-D tensor in the activation type, or 3-D float32 partial sums."""
    if x.dim() == 3:
        _want(x, torch.float32, name + " partial sums")
        return None, x, x.shape[0], x.shape[1], x.shape[2]
    _want(x, like, name)
    return x, None, 0, x.shape[0], x.shape[1]


def branch_norm_add(resid: torch.Tensor, branch: torch.Tensor | None, post_weight: torch.Tensor | None,
                    layer_scale: torch.Tensor | None, branch_eps: float, next_weight: torch.Tensor | None,
                    out: torch.Tensor | None, next_eps: float = 0.0, rows: torch.Tensor | None = None,
                    branch_groups: int = 1, next_groups: int = 1) -> None:
    """``x = resid + rmsnorm(branch) * post_weight * layer_scale`` (written back unless ``rows``
    selects rows), then, if ``out`` is given, ``out = rmsnorm(x) * next_weight`` or, without
    ``next_weight``, ``out = x`` in the activation type.  ``branch`` is in the activation type or
    float32 partial sums ``[parts, tokens, hidden]``; ``None``: nothing joins, only the norm in front
    runs.  ``branch_groups`` / ``next_groups``: the norm works on that many equal consecutive parts of
    a row, each with a root mean square of its own."""
    _want(resid, torch.float32, "resid")
    hidden = resid.shape[-1]
    if hidden % branch_groups or hidden % next_groups:
        raise KernelError(f"a row of {hidden} does not split into {branch_groups} / {next_groups} equal groups")
    if branch is None:
        if out is None:
            return
        dtype, b, parts, n_parts = out.dtype, None, None, 0
    else:
        dtype = out.dtype if out is not None else (branch.dtype if branch.dim() == 2 else torch.float32)
        b, parts, n_parts, n, width = _parts_of(branch, dtype, "branch")
        if width != hidden or n != resid.shape[0]:
            raise KernelError("branch and resid differ in shape")
    n = resid.shape[0]
    for name, t in (("post_weight", post_weight), ("layer_scale", layer_scale), ("next_weight", next_weight)):
        if t is not None:
            _want(t, torch.float32, name)
            if t.numel() != hidden:
                raise KernelError(f"{name} does not match the width")
    if rows is not None:
        _want(rows, torch.int32, "rows")
    n_rows = rows.numel() if rows is not None else n
    if out is not None:
        _want(out, None, "out")
        if out.numel() < n_rows * hidden:
            raise KernelError("out needs room for the rows")
    _check(_lib().tk_branch_norm_add(resid.data_ptr(), _ptr(b), _ptr(parts), n_parts,
                                        parts.stride(0) if parts is not None else 0, _ptr(post_weight),
                                        _ptr(layer_scale), _ptr(next_weight), _ptr(out), _ptr(rows), n_rows, hidden,
                                        float(branch_eps), float(next_eps), int(branch_groups), int(next_groups),
                                        dtype_code(dtype), _stream()),
           "branch_norm_add")


def qkv_pairs(qkv: torch.Tensor, q_out: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
              positions: torch.Tensor, tok_req: torch.Tensor, req_slot: torch.Tensor, block_table: torch.Tensor,
              table: torch.Tensor | None, err: torch.Tensor, *, n_q_heads: int, n_kv_heads: int, rotary_dim: int,
              unit_norm_eps: float | None, v_first_in: torch.Tensor | None = None,
              v_lambda: torch.Tensor | None = None, v_first_out: torch.Tensor | None = None,
              req_q_len: torch.Tensor | None = None, req_kv_len: torch.Tensor | None = None) -> None:
    """Rotation of neighbouring pairs, unit norm of the rotated heads, blend of the values with an
    earlier layer's, and the page write, for key heads of size ``d`` and value heads of size ``dv``.

    ``qkv`` rows hold ``Hq d | Hkv d | Hkv dv`` values (activation type, or float32 partial sums).
    ``v_first_in`` / ``v_first_out`` are float32 ``[tokens, Hkv dv]``; ``v_lambda`` one float32."""
    _want(q_out, None, "q_out")
    x, parts, n_parts, n, row = _parts_of(qkv, q_out.dtype, "qkv")
    _want(k_cache, q_out.dtype, "k_cache"); _want(v_cache, q_out.dtype, "v_cache")
    num_pages, hkv, page_size, d = k_cache.shape
    dv = v_cache.shape[3]
    if hkv != n_kv_heads or v_cache.shape[:3] != k_cache.shape[:3] or q_out.shape != (n, n_q_heads, d):
        raise KernelError("cache pages or q_out do not match the heads")
    if row < (n_q_heads + n_kv_heads) * d + n_kv_heads * dv:
        raise KernelError("qkv rows are too short for the heads")
    for name, t in (("positions", positions), ("tok_req", tok_req), ("req_slot", req_slot),
                    ("block_table", block_table)):
        _want(t, torch.int32, name)
    if table is not None:
        _want(table, torch.float32, "table")
        if table.shape != (n, rotary_dim // 2, 2):
            raise KernelError(f"the rotation table must be [{n}, {rotary_dim // 2}, 2], got {tuple(table.shape)}")
    elif rotary_dim:
        raise KernelError("rotary_dim without a rotation table")
    for name, t in (("v_first_in", v_first_in), ("v_first_out", v_first_out)):
        if t is not None:
            _want(t, torch.float32, name)
            if t.shape != (n, n_kv_heads * dv):
                raise KernelError(f"{name} must be [{n}, {n_kv_heads * dv}]")
    if v_first_in is not None:
        _want(v_lambda, torch.float32, "v_lambda")
    _check(_lib().tk_qkv_pairs(_ptr(x), _ptr(parts), n_parts, q_out.data_ptr(), k_cache.data_ptr(),
                                  v_cache.data_ptr(), positions.data_ptr(), tok_req.data_ptr(), req_slot.data_ptr(),
                                  block_table.data_ptr(), _ptr(req_q_len), _ptr(req_kv_len), _ptr(table),
                                  _ptr(v_first_in), _ptr(v_lambda), _ptr(v_first_out), err.data_ptr(), n,
                                  req_slot.numel(), n_q_heads, n_kv_heads, d, dv, rotary_dim, row, page_size,
                                  block_table.shape[1], num_pages, 0 if unit_norm_eps is None else 1,
                                  float(unit_norm_eps or 0.0), dtype_code(q_out.dtype), _stream()), "qkv_pairs")


def gla_prepared_row(key_dim: int, value_dim: int) -> tuple[int, int]:
    """``(dks, dvs)``: key and value sizes rounded up to 16 bytes of float32, as :func:`gla_prepare` lays a row out."""
    return (key_dim + 3) // 4 * 4, (value_dim + 3) // 4 * 4


def gla_prepare(proj: torch.Tensor, q_off: int, k_off: int, v_off: int, a_off: int, w2: torch.Tensor,
                bias: torch.Tensor | None, *, heads: int, key_dim: int, value_dim: int, tau: float,
                q_scale: float) -> torch.Tensor:
    """The recurrence's inputs in float32 from the columns of the stacked projection ``proj``
    (activation type, or float32 partial sums), as one flat tensor that :func:`gla_prepared_views`
    takes apart: ``q * q_scale``, ``k`` and ``alpha = sigmoid(a W2^T + bias) ** (1 / tau)`` (``a``: the
    ``rank`` columns from ``a_off`` on) in pieces of four key channels, and ``v``; head by head, so
    that a head's tokens follow one another."""
    _want(w2, None, "w2")
    channels, rank = w2.shape
    if channels != heads * key_dim:
        raise KernelError("the decay projection must have heads * key_dim rows")
    x, parts, n_parts, n, row = _parts_of(proj, w2.dtype, "proj")
    for off, size in ((q_off, heads * key_dim), (k_off, heads * key_dim), (v_off, heads * value_dim), (a_off, rank)):
        if off < 0 or off + size > row:
            raise KernelError("a column range lies outside the row")
    if bias is not None:
        _want(bias, torch.float32, "bias")
        if bias.numel() != channels:
            raise KernelError("one bias per channel is needed")
    dks, dvs = gla_prepared_row(key_dim, value_dim)
    out = torch.empty(n * heads * (3 * dks + dvs), dtype=torch.float32, device=w2.device)
    _check(_lib().tk_gla_prepare(_ptr(x), _ptr(parts), n_parts, row, q_off, k_off, v_off, a_off, w2.data_ptr(),
                                    _ptr(bias), out.data_ptr(), n, heads, key_dim, value_dim, rank, float(tau),
                                    float(q_scale), dtype_code(w2.dtype), _stream()), "gla_prepare")
    return out


def gla_prepared_views(prep: torch.Tensor, heads: int, key_dim: int, value_dim: int) -> tuple[torch.Tensor, torch.Tensor]:
    """``(pieces, values)`` of what :func:`gla_prepare` returned: ``pieces[h, t, i, 0 / 1 / 2, :]`` are
    ``q * q_scale``, ``k`` and ``alpha`` of the key channels ``4 i .. 4 i + 3``, ``values[h, t, :]`` is ``v``
    (both padded with zeros up to ``dks``, ``dvs``)."""
    dks, dvs = gla_prepared_row(key_dim, value_dim)
    n = prep.numel() // (heads * (3 * dks + dvs))
    split = heads * n * 3 * dks
    return prep[:split].view(heads, n, dks // 4, 3, 4), prep[split:].view(heads, n, dvs)


def gla_scan(prep: torch.Tensor, state: torch.Tensor, req_q_start: torch.Tensor, req_q_len: torch.Tensor,
             req_slot: torch.Tensor, err: torch.Tensor, *, cols: int = 0) -> torch.Tensor:
    """The recurrence ``S = diag(alpha) S + k v^T, o = S^T q`` over every request's tokens of the
    step, from the rows of :func:`gla_prepare`; ``state`` is float32 ``[slots, heads, key_dim, value_dim]``
    and is advanced in place.  Returns ``o`` float32 ``[tokens, heads, value_dim]``.  ``cols`` is the
    number of value channels a block takes (32, 16 or 8; 0 lets the kernel's launcher cover the SMs);
    the result is the same bit for bit under every split."""
    _want(state, torch.float32, "state"); _want(prep, torch.float32, "prep")
    n_slots, heads, dk, dv = state.shape
    dks, dvs = gla_prepared_row(dk, dv)
    if prep.dim() != 1 or prep.numel() % (heads * (3 * dks + dvs)) != 0:
        raise KernelError("prep must be the flat tensor that gla_prepare returns for this state's sizes")
    if dk > 256:
        raise KernelError(f"key size {dk} is beyond the kernel's limit of 256")
    for name, t in (("req_q_start", req_q_start), ("req_q_len", req_q_len), ("req_slot", req_slot)):
        _want(t, torch.int32, name)
    n, n_reqs = prep.numel() // (heads * (3 * dks + dvs)), req_slot.numel()
    out = torch.empty((n, heads, dv), dtype=torch.float32, device=state.device)
    _check(_lib().tk_gla_scan(prep.data_ptr(), state.data_ptr(), out.data_ptr(), req_q_start.data_ptr(),
                                 req_q_len.data_ptr(), req_slot.data_ptr(), err.data_ptr(), n, n_reqs, n_slots, heads,
                                 dk, dv, int(cols), _stream()), "gla_scan")
    return out


def gla_out(o: torch.Tensor, proj: torch.Tensor | None, g_off: int, weight: torch.Tensor | None, eps: float,
            dtype: torch.dtype, out: torch.Tensor | None = None, out_scale: float = 1.0) -> torch.Tensor:
    """``rmsnorm(o) * weight * silu(gate) * out_scale`` per (token, head) in the activation type
    ``[tokens, heads * value_dim]``; the gate is read from ``proj`` at column ``g_off`` (``proj=None``: no gate);
    ``weight=None``: the heads are only divided by their root mean square.  ``out`` may be a column range of
    wider rows."""
    _want(o, torch.float32, "o")
    n, heads, dv = o.shape
    x = parts = None
    n_parts, row = 0, 0
    if proj is not None:
        x, parts, n_parts, n2, row = _parts_of(proj, dtype, "proj")
        if n2 != n or g_off < 0 or g_off + heads * dv > row:
            raise KernelError("the gate columns lie outside the row")
    else:
        g_off = -1
    if weight is not None:
        _want(weight, torch.float32, "weight")
        if weight.numel() != dv:
            raise KernelError("the norm weight does not match the value size")
    y = out if out is not None else torch.empty((n, heads * dv), dtype=dtype, device=o.device)
    if y.dtype != dtype or y.shape != (n, heads * dv) or y.stride(1) != 1:
        raise KernelError("out must be [tokens, heads * value_dim] in the activation type with dense rows")
    _check(_lib().tk_gla_out(o.data_ptr(), _ptr(x), _ptr(parts), n_parts, row, g_off, _ptr(weight), y.data_ptr(),
                                y.stride(0), float(out_scale), n, heads, dv, float(eps), dtype_code(dtype), _stream()),
           "gla_out")
    return y



def _stacked_args(proj: torch.Tensor, like: torch.dtype, name: str) -> tuple:
    """``(x pointer, parts pointer, parts, stride of a part, row length, tokens)`` of a product's result."""
    x, parts, n_parts, n, row = _parts_of(proj, like, name)
    return _ptr(x), _ptr(parts), n_parts, parts.stride(0) if parts is not None else 0, row, n


def short_conv(rows: torch.Tensor, taps: torch.Tensor, tail: torch.Tensor | None, step, *, dtype: torch.dtype,
               in_off: int = 0, channels: int | None = None, bias: torch.Tensor | None = None,
               add_input: bool = False, silu: bool = False, out_f32: bool = False) -> torch.Tensor:
    """A causal convolution of ``taps.shape[1]`` taps per channel over every request's tokens of the step,
    continued from the request's *tail*: ``tail[slot]`` is float32 ``[taps - 1, channels]``, the inputs of
    the positions before the step (zeros before the sequence), and is moved on to the step's last inputs.

    ``rows`` is the float32 residual stream ``[tokens, width]``, a product's result in ``dtype`` or its
    float32 partial sums; the channels are the columns from ``in_off`` on.  ``y = [x +] [bias +] conv(x)``,
    then silu if asked; float32 sums; the result is ``[tokens, channels]`` in ``dtype`` (or float32)."""
    _want(taps, torch.float32, "taps")
    ch, k = taps.shape
    channels = ch if channels is None else channels
    if channels != ch:
        raise KernelError("one row of taps per channel is needed")
    rows_f32 = None
    if rows.dim() == 2 and rows.dtype == torch.float32 and dtype != torch.float32:
        _want(rows, torch.float32, "rows")
        rows_f32, x, parts, n_parts, part_stride, row, n = rows.data_ptr(), None, None, 0, 0, rows.shape[1], rows.shape[0]
    else:
        x, parts, n_parts, part_stride, row, n = _stacked_args(rows, dtype, "rows")
    if bias is not None:
        _want(bias, torch.float32, "bias")
    if k > 1:
        _want(tail, torch.float32, "tail")
        if tail.shape[1:] != (k - 1, channels):
            raise KernelError("the tail must be [slots, taps - 1, channels]")
    out = torch.empty((n, channels), dtype=torch.float32 if out_f32 else dtype, device=taps.device)
    move = 1 if step.max_q_len == 1 else 2
    _check(_lib().tk_short_conv(x, parts, n_parts, part_stride, rows_f32, row, in_off, taps.data_ptr(), _ptr(bias),
                                   _ptr(tail), out.data_ptr(), step.tok_req.data_ptr(), step.req_q_start.data_ptr(),
                                   step.req_q_len.data_ptr(), step.req_slot.data_ptr(), step.err.data_ptr(), n,
                                   step.req_slot.numel(), tail.shape[0] if tail is not None else 0, channels, k,
                                   int(add_input), int(silu), int(out_f32), move, dtype_code(dtype), _stream()),
           "short_conv")
    return out


def _prep_buffer(n: int, heads: int, dk: int, dv: int, device) -> torch.Tensor:
    dks, dvs = gla_prepared_row(dk, dv)
    return torch.empty(n * heads * (3 * dks + dvs), dtype=torch.float32, device=device)


def hgrn2_prepare(proj: torch.Tensor, f_bias: torch.Tensor, lower: torch.Tensor, *, dtype: torch.dtype, q_off: int,
                  f_off: int, v_off: int, heads: int, key_dim: int, value_dim: int) -> torch.Tensor:
    """The inputs of :func:`gla_scan` for linear attention whose forget gate is also its key:
    ``q = silu(z_q)``, ``f = lower + (1 - lower) sigmoid(z_f + f_bias)``, ``alpha = f``, ``k = 1 - f``, ``v = z_v``."""
    _want(f_bias, torch.float32, "f_bias"); _want(lower, torch.float32, "lower")
    x, parts, n_parts, part_stride, row, n = _stacked_args(proj, dtype, "proj")
    prep = _prep_buffer(n, heads, key_dim, value_dim, f_bias.device)
    _check(_lib().tk_hgrn2_prepare(x, parts, n_parts, part_stride, row, q_off, f_off, v_off, f_bias.data_ptr(),
                                      lower.data_ptr(), prep.data_ptr(), n, heads, key_dim, value_dim,
                                      dtype_code(dtype), _stream()), "hgrn2_prepare")
    return prep


def mlstm_prepare(proj: torch.Tensor, i_bias: torch.Tensor, f_bias: torch.Tensor, m_state: torch.Tensor, step, *,
                  dtype: torch.dtype, q_off: int, k_off: int, v_off: int, i_off: int, f_off: int, heads: int,
                  key_dim: int, value_dim: int, cap: float, q_scale: float) -> tuple[torch.Tensor, torch.Tensor]:
    """``(prep, gates)``: the inputs of :func:`gla_scan` for a matrix memory with exponential gates whose
    normaliser rides as one more value column (the state is ``[heads, key_dim, value_dim + 1]``), and
    ``gates`` float32 ``[tokens, heads, 3]`` = ``(alpha, exp(i - m), exp(-m))``.  ``m_state`` ``[slots, heads]``
    holds every request's running maximum and is moved on."""
    for name, t in (("i_bias", i_bias), ("f_bias", f_bias), ("m_state", m_state)):
        _want(t, torch.float32, name)
    x, parts, n_parts, part_stride, row, n = _stacked_args(proj, dtype, "proj")
    prep = _prep_buffer(n, heads, key_dim, value_dim + 1, m_state.device)
    gates = torch.empty((n, heads, 3), dtype=torch.float32, device=m_state.device)
    _check(_lib().tk_mlstm_prepare(x, parts, n_parts, part_stride, row, q_off, k_off, v_off, i_off, f_off,
                                      i_bias.data_ptr(), f_bias.data_ptr(), float(cap), float(q_scale),
                                      m_state.data_ptr(), gates.data_ptr(), prep.data_ptr(),
                                      step.req_q_start.data_ptr(), step.req_q_len.data_ptr(), step.req_slot.data_ptr(),
                                      step.err.data_ptr(), n, step.req_slot.numel(), m_state.shape[0], heads, key_dim,
                                      value_dim, dtype_code(dtype), _stream()), "mlstm_prepare")
    return prep, gates


def mlstm_out(o: torch.Tensor, gates: torch.Tensor, proj: torch.Tensor, g_off: int, weight: torch.Tensor, eps: float,
              dtype: torch.dtype, out: torch.Tensor | None = None, out_scale: float = 1.0) -> torch.Tensor:
    """``o`` is ``[tokens, heads, dv + 1]`` with ``n . q`` in the last column: every head's
    ``o / (max(|n . q|, exp(-m)) + 1e-6)`` is scaled to unit root mean square, multiplied by ``weight``
    (one per channel of all heads) and by ``sigmoid(gate)``, the gate read from ``proj`` at ``g_off``."""
    _want(o, torch.float32, "o"); _want(gates, torch.float32, "gates"); _want(weight, torch.float32, "weight")
    n, heads, dv1 = o.shape
    dv = dv1 - 1
    x, parts, n_parts, part_stride, row, n2 = _stacked_args(proj, dtype, "proj")
    if n2 != n or weight.numel() != heads * dv or g_off < 0 or g_off + heads * dv > row:
        raise KernelError("mlstm_out shape mismatch")
    if out is None:
        out = torch.empty((n, heads * dv), dtype=dtype, device=o.device)
    _check(_lib().tk_mlstm_out(o.data_ptr(), gates.data_ptr(), x, parts, n_parts, part_stride, row, g_off,
                                  weight.data_ptr(), out.data_ptr(), out.stride(0), n, heads, dv, float(eps),
                                  float(out_scale), dtype_code(dtype), _stream()), "mlstm_out")
    return out


def ssd_prepare(xbc: torch.Tensor, proj: torch.Tensor, dt_off: int, dt_bias: torch.Tensor, a_log: torch.Tensor, *,
                dtype: torch.dtype, heads: int, groups: int, state: int, value_dim: int) -> torch.Tensor:
    """The inputs of :func:`gla_scan` for a state-space layer with a scalar decay per head.  ``xbc`` is
    float32 ``[tokens, heads * value_dim + 2 * groups * state]`` (x | B | C after their convolution);
    ``dt = softplus(proj[:, dt_off + h] + dt_bias)``, ``alpha = exp(-exp(a_log) dt)``, ``k = B``, ``q = C`` of the
    head's group, ``v = dt x``."""
    for name, t in (("xbc", xbc), ("dt_bias", dt_bias), ("a_log", a_log)):
        _want(t, torch.float32, name)
    x, parts, n_parts, part_stride, row, n = _stacked_args(proj, dtype, "proj")
    if xbc.shape != (n, heads * value_dim + 2 * groups * state):
        raise KernelError("ssd_prepare shape mismatch")
    prep = _prep_buffer(n, heads, state, value_dim, xbc.device)
    _check(_lib().tk_ssd_prepare(xbc.data_ptr(), x, parts, n_parts, part_stride, row, dt_off, dt_bias.data_ptr(),
                                    a_log.data_ptr(), prep.data_ptr(), n, heads, groups, state, value_dim,
                                    dtype_code(dtype), _stream()), "ssd_prepare")
    return prep


def ssd_out(o: torch.Tensor, xbc: torch.Tensor, proj: torch.Tensor, z_off: int, skip: torch.Tensor,
            weight: torch.Tensor, norm_groups: int, eps: float, dtype: torch.dtype, out: torch.Tensor | None = None,
            out_scale: float = 1.0) -> torch.Tensor:
    """``norm((o + skip_h x) * silu(z)) * weight`` with the RMS norm over ``norm_groups`` equal parts of the
    row; ``x`` are the leading columns of ``xbc``, ``z`` the columns of ``proj`` from ``z_off`` on."""
    for name, t in (("o", o), ("xbc", xbc), ("skip", skip), ("weight", weight)):
        _want(t, torch.float32, name)
    n, heads, dv = o.shape
    x, parts, n_parts, part_stride, row, n2 = _stacked_args(proj, dtype, "proj")
    if n2 != n or weight.numel() != heads * dv or skip.numel() != heads or (heads * dv) % norm_groups:
        raise KernelError("ssd_out shape mismatch")
    if out is None:
        out = torch.empty((n, heads * dv), dtype=dtype, device=o.device)
    _check(_lib().tk_ssd_out(o.data_ptr(), xbc.data_ptr(), xbc.stride(0), x, parts, n_parts, part_stride, row, z_off,
                                skip.data_ptr(), weight.data_ptr(), out.data_ptr(), out.stride(0), n, heads, dv,
                                int(norm_groups), float(eps), float(out_scale), dtype_code(dtype), _stream()), "ssd_out")
    return out


def gate_scale(x: torch.Tensor, proj: torch.Tensor, g_off: int, out: torch.Tensor | None = None,
               scale: float = 1.0, gate_group: int = 1) -> torch.Tensor:
    """``x * sigmoid(gate) * scale`` with the gate read from ``proj`` at column ``g_off``; ``out`` may be a
    column range of wider rows.  ``gate_group`` neighbouring columns of ``x`` share one gate column (a gate per
    head: the head's size)."""
    _want(x, None, "x")
    n, cols = x.shape
    g, parts, n_parts, part_stride, row, n2 = _stacked_args(proj, x.dtype, "proj")
    if gate_group < 1 or n2 != n or g_off < 0 or g_off + -(-cols // gate_group) > row:
        raise KernelError("the gate columns lie outside the row")
    if out is None:
        out = torch.empty_like(x)
    _check(_lib().tk_gate_scale(x.data_ptr(), g, parts, n_parts, part_stride, row, g_off, out.data_ptr(),
                                   out.stride(0), n, cols, float(scale), int(gate_group), dtype_code(x.dtype), _stream()),
           "gate_scale")
    return out


def qkv_rownorm(proj: torch.Tensor, q_out: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, step,
                block_table: torch.Tensor, *, q_off: int, k_off: int, v_off: int, q_bias, k_bias, v_bias, q_norm,
                k_norm, eps: float) -> None:
    """Biases, an RMS norm over a token's whole query projection and over its whole key projection (one
    weight per channel; ``None``: no norm), queries to ``q_out`` ``[tokens, Hq, d]``, keys and values into
    their pages."""
    n, hq, d = q_out.shape
    num_pages, hkv, page_size, dk = k_cache.shape
    dv = v_cache.shape[3]
    if dk != d or not q_out.is_contiguous():
        raise KernelError("qkv_rownorm shape mismatch")
    for name, t, size in (("q_bias", q_bias, hq * d), ("k_bias", k_bias, hkv * d), ("v_bias", v_bias, hkv * dv),
                          ("q_norm", q_norm, hq * d), ("k_norm", k_norm, hkv * d)):
        if t is not None:
            _want(t, torch.float32, name)
            if t.numel() != size:
                raise KernelError(f"{name} does not match the projection")
    x, parts, n_parts, part_stride, row, n2 = _stacked_args(proj, q_out.dtype, "proj")
    if n2 != n:
        raise KernelError("proj and q_out differ in tokens")
    _check(_lib().tk_qkv_rownorm(x, parts, n_parts, part_stride, row, q_off, k_off, v_off, _ptr(q_bias), _ptr(k_bias),
                                    _ptr(v_bias), _ptr(q_norm), _ptr(k_norm), q_out.data_ptr(), k_cache.data_ptr(),
                                    v_cache.data_ptr(), step.positions.data_ptr(), step.tok_req.data_ptr(),
                                    step.req_slot.data_ptr(), block_table.data_ptr(), step.req_q_len.data_ptr(),
                                    step.req_kv_len.data_ptr(), step.err.data_ptr(), n, step.req_slot.numel(), hq, hkv,
                                    d, dv, page_size, block_table.shape[1], num_pages, float(eps),
                                    dtype_code(q_out.dtype), _stream()), "qkv_rownorm")


UNARY_ACTIVATIONS = {"silu": 0, "gelu_tanh": 1, "relu2": 2}


def unary_act(x: torch.Tensor, dtype: torch.dtype, activation: str) -> torch.Tensor:
    """``act(x)`` element by element in the activation type: ``silu``, ``gelu_tanh`` or ``relu2`` (the square of
    relu).  ``x`` is ``[tokens, cols]`` in ``dtype`` or the float32 partial sums of a split product."""
    if activation not in UNARY_ACTIVATIONS:
        raise KernelError(f"unknown activation {activation!r}; known: {', '.join(UNARY_ACTIVATIONS)}")
    xp, parts, n_parts, n, cols = _parts_of(x, dtype, "x")
    out = torch.empty((n, cols), dtype=dtype, device=x.device)
    _check(_lib().tk_unary_act(_ptr(xp), _ptr(parts), n_parts, parts.stride(0) if parts is not None else 0,
                                  out.data_ptr(), n * cols, dtype_code(dtype), UNARY_ACTIVATIONS[activation], _stream()),
           "unary_act")
    return out


def logits_scale_cap(logits: torch.Tensor, scale: float = 1.0, cap: float | None = None) -> torch.Tensor:
    """``cap * tanh(scale * logits / cap)`` in place on float32 logits (``cap=None``: only the scale)."""
    _want(logits, torch.float32, "logits")
    _check(_lib().tk_logits_scale_cap(logits.data_ptr(), logits.numel(), float(scale), float(cap or 0.0), _stream()),
           "logits_scale_cap")
    return logits


HYPER_MAX_STREAMS = 8


def hyper_mix_norm(streams: torch.Tensor, branch: torch.Tensor | None, *, mix: torch.Tensor | None = None,
                   write: torch.Tensor | None = None, read: torch.Tensor | None = None, mult: float = 1.0,
                   norm_w: torch.Tensor | None = None, norm_b: torch.Tensor | None = None, eps: float = 0.0,
                   dtype: torch.dtype | None = None, rows: torch.Tensor | None = None,
                   want_sum: bool = False):
    """A residual stream in ``S`` float32 copies ``[S, tokens, width]``: the pending sublayer output ``branch``
    (activation type or float32 partial sums; ``None``: nothing pending) is written to all copies,
    ``x_t <- sum_s mix[s, t] x_s + mult * write[t] * branch``, then the row ``u = sum_s read[s] x_s`` is read and, with
    ``norm_w``, layer-normed (``norm_b`` optional) into a new ``[rows, width]`` tensor of ``dtype``.  ``mix``, ``write``
    and ``read`` default to the identity and ones.  With ``rows`` (int32) only those rows are read and the copies
    stay as they are.  Returns ``(normed rows | None, u float32 | None)``; ``u`` only with ``want_sum``."""
    _want(streams, torch.float32, "streams")
    if streams.dim() != 3 or streams.shape[0] > HYPER_MAX_STREAMS:
        raise KernelError(f"the stream must be [copies <= {HYPER_MAX_STREAMS}, tokens, width]")
    S, n, width = streams.shape
    b = parts = None
    n_parts = part_stride = row = 0
    if branch is not None:
        like = dtype if dtype is not None else (branch.dtype if branch.dim() == 2 else torch.float32)
        b, parts, n_parts, n2, row = _parts_of(branch, like, "branch")
        if n2 != n or row != width:
            raise KernelError("branch and stream differ in shape")
        part_stride = parts.stride(0) if parts is not None else 0
        dtype = like
    for name, t, size in (("mix", mix, S * S), ("write", write, S), ("read", read, S), ("norm_w", norm_w, width),
                          ("norm_b", norm_b, width)):
        if t is not None:
            _want(t, torch.float32, name)
            if t.numel() != size:
                raise KernelError(f"{name} has {t.numel()} elements, not {size}")
    if rows is not None:
        _want(rows, torch.int32, "rows")
    n_rows = rows.numel() if rows is not None else n
    out = u = None
    if norm_w is not None:
        if dtype is None:
            raise KernelError("the normed rows need an element type")
        out = torch.empty((n_rows, width), dtype=dtype, device=streams.device)
    if want_sum:
        u = torch.empty((n_rows, width), dtype=torch.float32, device=streams.device)
    if out is None and u is None and (branch is None or rows is not None):
        return None, None
    _check(_lib().tk_hyper_mix_norm(streams.data_ptr(), _ptr(b), _ptr(parts), n_parts, part_stride, row, _ptr(mix),
                                       _ptr(write), _ptr(read), _ptr(norm_w), _ptr(norm_b), _ptr(out), _ptr(u),
                                       _ptr(rows), n_rows, n, width, S, float(mult), float(eps),
                                       dtype_code(dtype if dtype is not None else torch.float32), _stream()),
           "hyper_mix_norm")
    return out, u


def qkv_heads(proj: torch.Tensor, q_out: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, step,
              block_table: torch.Tensor, *, q_off: int, k_off: int, v_off: int | None, q_bias=None, k_bias=None,
              v_bias=None, head_norm_eps: float | None = None, q_norm=None, k_norm=None, table=None,
              rotary_dim: int = 0, halves: bool = False, temp_coef: float = 0.0, temp_every: int = 0) -> None:
    """Queries, keys and values head by head from the columns of a stacked projection (activation type or
    float32 partial sums): biases, an RMS norm of every q and k head (``head_norm_eps``; ``q_norm`` / ``k_norm``: a
    weight of one head's size shared by all heads, or none), the query temperature
    ``1 + temp_coef * ln(floor((p + 1) / temp_every) + 1)``, rotation over the first ``rotary_dim`` elements of the q
    and k heads by ``table`` (``[tokens, rotary_dim / 2, 2]`` float32; neighbouring pairs, or ``halves``); queries
    to ``q_out`` ``[tokens, Hq, d]``, keys and values into their pages.  ``v_off=None``: the values are the key
    projection as it was before norm and rotation."""
    n, hq, d = q_out.shape
    num_pages, hkv, page_size, dk = k_cache.shape
    dv = v_cache.shape[3]
    if dk != d or not q_out.is_contiguous() or v_cache.shape[:3] != k_cache.shape[:3]:
        raise KernelError("qkv_heads shape mismatch")
    if max(d, dv) > 512:
        raise KernelError(f"head sizes {d} / {dv} are beyond the kernel's limit of 512")
    for name, t, size in (("q_bias", q_bias, hq * d), ("k_bias", k_bias, hkv * d), ("v_bias", v_bias, hkv * dv),
                          ("q_norm", q_norm, d), ("k_norm", k_norm, d)):
        if t is not None:
            _want(t, torch.float32, name)
            if t.numel() != size:
                raise KernelError(f"{name} does not match the projection")
    x, parts, n_parts, part_stride, row, n2 = _stacked_args(proj, q_out.dtype, "proj")
    if n2 != n:
        raise KernelError("proj and q_out differ in tokens")
    if v_off is None and dv != d:
        raise KernelError("values that are the keys have the keys' size")
    spans = [(q_off, hq * d), (k_off, hkv * d)] + ([(v_off, hkv * dv)] if v_off is not None else [])
    if any(off < 0 or off + size > row for off, size in spans):
        raise KernelError("a column range lies outside the row")
    if table is not None:
        _want(table, torch.float32, "table")
        if table.shape != (n, rotary_dim // 2, 2):
            raise KernelError(f"the rotation table must be [{n}, {rotary_dim // 2}, 2], got {tuple(table.shape)}")
    elif rotary_dim:
        raise KernelError("rotary_dim without a rotation table")
    _check(_lib().tk_qkv_heads(x, parts, n_parts, part_stride, row, q_off, k_off, -1 if v_off is None else v_off,
                                  _ptr(q_bias), _ptr(k_bias), _ptr(v_bias), _ptr(q_norm), _ptr(k_norm),
                                  0 if head_norm_eps is None else 1, float(head_norm_eps or 0.0), _ptr(table),
                                  int(rotary_dim), int(bool(halves)), float(temp_coef), int(temp_every),
                                  q_out.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), step.positions.data_ptr(),
                                  step.tok_req.data_ptr(), step.req_slot.data_ptr(), block_table.data_ptr(),
                                  step.req_q_len.data_ptr(), step.req_kv_len.data_ptr(), step.err.data_ptr(), n,
                                  step.req_slot.numel(), hq, hkv, d, dv, page_size, block_table.shape[1], num_pages,
                                  dtype_code(q_out.dtype), _stream()), "qkv_heads")


def retention_prepare(proj: torch.Tensor, decay: torch.Tensor, table: torch.Tensor | None, *, dtype: torch.dtype,
                      q_off: int, k_off: int, v_off: int, heads: int, key_dim: int, value_dim: int, rotary_dim: int = 0,
                      halves: bool = True, q_scale: float = 1.0, k_scale: float = 1.0) -> torch.Tensor:
    """The inputs of :func:`gla_scan` for retention: q and k rotated over their first ``rotary_dim`` elements by
    ``table`` (``[tokens, rotary_dim / 2, 2]`` float32; halves or neighbouring pairs), then scaled; every row of head
    ``h`` decays by ``decay[h]`` (float32 ``[heads]``); v as projected."""
    _want(decay, torch.float32, "decay")
    x, parts, n_parts, part_stride, row, n = _stacked_args(proj, dtype, "proj")
    if decay.numel() != heads:
        raise KernelError("one decay per head is needed")
    for off, size in ((q_off, heads * key_dim), (k_off, heads * key_dim), (v_off, heads * value_dim)):
        if off < 0 or off + size > row:
            raise KernelError("a column range lies outside the row")
    if table is not None:
        _want(table, torch.float32, "table")
        if table.shape != (n, rotary_dim // 2, 2):
            raise KernelError(f"the rotation table must be [{n}, {rotary_dim // 2}, 2], got {tuple(table.shape)}")
    elif rotary_dim:
        raise KernelError("rotary_dim without a rotation table")
    prep = _prep_buffer(n, heads, key_dim, value_dim, decay.device)
    _check(_lib().tk_retention_prepare(x, parts, n_parts, part_stride, row, q_off, k_off, v_off, decay.data_ptr(),
                                          _ptr(table), int(rotary_dim), int(bool(halves)), float(q_scale),
                                          float(k_scale), prep.data_ptr(), n, heads, key_dim, value_dim,
                                          dtype_code(dtype), _stream()), "retention_prepare")
    return prep


def moe_tile_rows() -> int:
    return _lib().tk_moe_tile_rows()


class MoeRouting:
    """What :func:`moe_route` leaves on the device: ``chosen`` / ``weights`` ``[tokens, top]``, the pairs
    ``token * top + choice`` laid out expert by expert (``order``), and the products' row tiles.  With
    ``padded``: also every pair's row in the layout whose experts start on whole tiles of
    :func:`moe_pad_rows` rows (``pair_row``) and every such tile's expert (``tile_expert``, -1: unused)."""

    def __init__(self, chosen, weights, order, tiles, n_tiles, max_tiles, pair_row=None, tile_expert=None):
        self.chosen, self.weights, self.order, self.tiles, self.n_tiles, self.max_tiles = (
            chosen, weights, order, tiles, n_tiles, max_tiles)
        self.pair_row, self.tile_expert = pair_row, tile_expert


def moe_pad_rows() -> int:
    return _lib().tk_moe_pad_rows()


def moe_route(h: torch.Tensor, router: torch.Tensor, correction: torch.Tensor | None, *, top: int, n_groups: int,
              keep: int, padded: bool = False) -> MoeRouting:
    """Scores ``sigmoid(h router^T)`` in float32, choice by score plus ``correction`` among the ``keep`` groups
    of neighbouring experts whose two best choice scores add up highest, weights the plain scores."""
    _want(h, None, "h"); _want(router, torch.float32, "router")
    n, width = h.shape
    experts = router.shape[0]
    if correction is not None:
        _want(correction, torch.float32, "correction")
    if router.shape[1] != width or experts % n_groups or not 1 <= keep <= n_groups or not 1 <= top <= keep * (experts // n_groups):
        raise KernelError("moe_route: sizes do not fit")
    dev = h.device
    pairs = n * top
    max_tiles = min(pairs, -(-pairs // moe_tile_rows()) + experts)
    chosen = torch.empty((n, top), dtype=torch.int32, device=dev)
    weights = torch.empty((n, top), dtype=torch.float32, device=dev)
    order = torch.empty(pairs, dtype=torch.int32, device=dev)
    tiles = torch.empty((max_tiles, 3), dtype=torch.int32, device=dev)
    n_tiles = torch.empty(1, dtype=torch.int32, device=dev)
    pair_row = tile_expert = None
    if padded:
        pair_row = torch.empty(pairs, dtype=torch.int32, device=dev)
        tile_expert = torch.empty(min(pairs, pairs // moe_pad_rows() + experts), dtype=torch.int32, device=dev)
    _check(_lib().tk_moe_route(h.data_ptr(), router.data_ptr(), _ptr(correction), chosen.data_ptr(), weights.data_ptr(),
                                  order.data_ptr(), tiles.data_ptr(), n_tiles.data_ptr(), _ptr(pair_row), _ptr(tile_expert),
                                  tile_expert.numel() if padded else 0, n, width, experts, n_groups,
                                  keep, top, dtype_code(h.dtype), _stream()), "moe_route")
    return MoeRouting(chosen, weights, order, tiles, n_tiles, max_tiles, pair_row, tile_expert)


def moe_tc_takes(dtype: torch.dtype, width: int, ff: int) -> bool:
    """Whether :func:`moe_experts_tc` runs these sizes: bfloat16, an inner size in whole blocks of the fused
    activation, rows that TMA and 16-byte stores can address."""
    return dtype == torch.bfloat16 and ff % SWIGLU_TILE_BLOCK == 0 and width % 8 == 0 and PAIR_GEMM_POLICY != "off"


def moe_stack_gate_up(w_gate: torch.Tensor, w_up: torch.Tensor) -> torch.Tensor:
    """``[experts, 2 ff, width]`` with every expert's gate and up rows alternating in blocks of
    ``SWIGLU_TILE_BLOCK``, as the fused activation of the product wants them."""
    experts, ff, width = w_gate.shape
    b = SWIGLU_TILE_BLOCK
    return torch.stack([w_gate.view(experts, ff // b, b, width), w_up.view(experts, ff // b, b, width)],
                       dim=2).reshape(experts, 2 * ff, width).contiguous()


def moe_experts_tc(h: torch.Tensor, routing: MoeRouting, w_gate_up: torch.Tensor, w_down: torch.Tensor, err: torch.Tensor,
                   activation: str = "silu") -> torch.Tensor:
    """:func:`moe_experts` on the tensor cores (bfloat16): the tokens' rows are copied into the padded layout
    of ``routing``, the grouped product on pairs of SMs forms ``act(gate) * up`` in its epilogue and then the
    down product, row for row, and the weighted sum reads the pairs' rows.  ``w_gate_up`` is what
    :func:`moe_stack_gate_up` returns, ``w_down`` ``[experts, width, ff]``.  float32 ``[tokens, width]``."""
    _want(h, torch.bfloat16, "h"); _want(w_gate_up, torch.bfloat16, "w_gate_up"); _want(w_down, torch.bfloat16, "w_down")
    n, width = h.shape
    experts, ff2, _ = w_gate_up.shape
    ff = ff2 // 2
    top = routing.chosen.shape[1]
    if routing.pair_row is None or w_gate_up.shape != (experts, 2 * ff, width) or w_down.shape != (experts, width, ff):
        raise KernelError("moe_experts_tc: the routing must be padded and the weights stacked for these sizes")
    if not moe_tc_takes(h.dtype, width, ff) or h.stride(1) != 1 or h.stride(0) % 8:
        raise KernelError("moe_experts_tc does not take these sizes")
    if activation not in GLU_ACTIVATIONS:
        raise KernelError(f"unknown activation {activation!r}")
    flush_chains()
    lib, r = _lib(), routing
    rows = r.tile_expert.numel() * moe_pad_rows()
    xs = torch.empty((rows, width), dtype=torch.bfloat16, device=h.device)
    act = torch.empty((rows, ff), dtype=torch.bfloat16, device=h.device)
    y = torch.empty((rows, width), dtype=torch.bfloat16, device=h.device)
    out = torch.empty((n, width), dtype=torch.float32, device=h.device)
    _check(lib.tk_moe_gather(h.data_ptr(), h.stride(0), xs.data_ptr(), r.pair_row.data_ptr(), n, top, width, _stream()),
           "moe_gather")
    _check(lib.tk_gemm_bf16_pair_grouped(xs.data_ptr(), w_gate_up.data_ptr(), act.data_ptr(), err.data_ptr(),
                                         r.tile_expert.data_ptr(), rows, experts, 2 * ff, width, width, width, ff,
                                         1 + GLU_ACTIVATIONS[activation], _stream()), "gemm_pair_grouped (gate, up)")
    _check(lib.tk_gemm_bf16_pair_grouped(act.data_ptr(), w_down.data_ptr(), y.data_ptr(), err.data_ptr(),
                                         r.tile_expert.data_ptr(), rows, experts, width, ff, ff, ff, width, 0, _stream()),
           "gemm_pair_grouped (down)")
    _check(lib.tk_moe_combine_rows(y.data_ptr(), r.weights.data_ptr(), r.pair_row.data_ptr(), out.data_ptr(), n, width,
                                   top, _stream()), "moe_combine_rows")
    return out


def moe_small_takes(n_tokens: int, top: int, width: int, ff: int) -> bool:
    """Whether :func:`moe_experts_small` runs a step of these sizes: few enough (token, choice) pairs that an
    expert's weights are better streamed once past them than multiplied in whole tiles."""
    return (n_tokens * top <= MOE_SMALL_PAIRS and width % 8 == 0 and ff % 8 == 0 and ff % SWIGLU_TILE_BLOCK == 0
            and 65536 + 8 * max(width, ff) <= 200 * 1024)


def moe_experts_small(h: torch.Tensor, routing: MoeRouting, w_gate_up: torch.Tensor, w_down: torch.Tensor,
                      activation: str = "silu") -> torch.Tensor:
    """:func:`moe_experts` for steps of few tokens (bfloat16): only the experts that some token chose are
    read, once, a warp an output row; the sums are float32, the rows between the two products bfloat16.
    ``w_gate_up`` is what :func:`moe_stack_gate_up` returns.  float32 ``[tokens, width]``."""
    _want(h, torch.bfloat16, "h"); _want(w_gate_up, torch.bfloat16, "w_gate_up"); _want(w_down, torch.bfloat16, "w_down")
    n, width = h.shape
    experts, ff2, _ = w_gate_up.shape
    ff = ff2 // 2
    top = routing.chosen.shape[1]
    if w_gate_up.shape != (experts, 2 * ff, width) or w_down.shape != (experts, width, ff):
        raise KernelError("moe_experts_small: the weights must be stacked for these sizes")
    if not moe_small_takes(n, top, width, ff) or h.stride(1) != 1 or h.stride(0) % 8:
        raise KernelError("moe_experts_small does not take these sizes")
    if activation not in GLU_ACTIVATIONS:
        raise KernelError(f"unknown activation {activation!r}")
    flush_chains()
    lib, pairs = _lib(), n * top
    act = torch.empty((pairs, ff), dtype=torch.bfloat16, device=h.device)
    y = torch.empty((pairs, width), dtype=torch.float32, device=h.device)
    out = torch.empty((n, width), dtype=torch.float32, device=h.device)
    _check(lib.tk_moe_small(h.data_ptr(), h.stride(0), top, w_gate_up.data_ptr(), act.data_ptr(),
                            routing.chosen.data_ptr(), pairs, experts, ff, width, GLU_ACTIVATIONS[activation],
                            SWIGLU_TILE_BLOCK, _stream()), "moe_small (gate, up)")
    _check(lib.tk_moe_small(act.data_ptr(), ff, 1, w_down.data_ptr(), y.data_ptr(), routing.chosen.data_ptr(), pairs,
                            experts, width, ff, 0, 0, _stream()), "moe_small (down)")
    _check(lib.tk_moe_combine(y.data_ptr(), routing.weights.data_ptr(), out.data_ptr(), n, width, top, _stream()),
           "moe_combine")
    return out


def moe_experts(h: torch.Tensor, routing: MoeRouting, w_gate: torch.Tensor, w_up: torch.Tensor, w_down: torch.Tensor,
                activation: str = "silu") -> torch.Tensor:
    """The weighted sum of the chosen experts' gated units, float32 ``[tokens, width]``.  ``w_gate`` and
    ``w_up`` are ``[experts, ff, width]``, ``w_down`` ``[experts, width, ff]``, all in the type of ``h``."""
    n, width = h.shape
    experts, ff, _ = w_gate.shape
    top = routing.chosen.shape[1]
    for name, t, shape in (("w_gate", w_gate, (experts, ff, width)), ("w_up", w_up, (experts, ff, width)),
                           ("w_down", w_down, (experts, width, ff))):
        _want(t, h.dtype, name)
        if t.shape != shape:
            raise KernelError(f"{name} must be {shape}")
    pairs = n * top
    act = torch.empty((pairs, ff), dtype=h.dtype, device=h.device)
    y = torch.empty((pairs, width), dtype=torch.float32, device=h.device)
    out = torch.empty((n, width), dtype=torch.float32, device=h.device)
    lib, r = _lib(), routing
    _check(lib.tk_moe_ffn(h.data_ptr(), h.stride(0), top, w_gate.data_ptr(), w_up.data_ptr(), act.data_ptr(),
                          r.order.data_ptr(), r.tiles.data_ptr(), r.n_tiles.data_ptr(), r.max_tiles, ff, width,
                          GLU_ACTIVATIONS[activation], dtype_code(h.dtype), _stream()), "moe_ffn (gate, up)")
    _check(lib.tk_moe_ffn(act.data_ptr(), ff, 1, w_down.data_ptr(), None, y.data_ptr(), r.order.data_ptr(),
                          r.tiles.data_ptr(), r.n_tiles.data_ptr(), r.max_tiles, width, ff, 0, dtype_code(h.dtype),
                          _stream()), "moe_ffn (down)")
    _check(lib.tk_moe_combine(y.data_ptr(), r.weights.data_ptr(), out.data_ptr(), n, width, top, _stream()),
           "moe_combine")
    return out


def decode_splits(n_items: int, n_kv_heads: int, max_kv_len: int) -> int:
    """How many key splits the decode kernel gets.

    Two blocks of three stages fit an SM, or three blocks of two stages (the kernel takes two
    stages when its grid is larger than two blocks per SM), so up to 444 run at a time.  A second,
    partly filled wave costs as much as the first (measured at Qwen3-8B head sizes with two
    blocks to an SM: batch 8 takes 30 us with 4 splits = 256 blocks and 43 us with 5), so the
    splits are chosen to stay within one wave.  A block keeps at least eight 16-key tiles, and a
    multiple of four, so that each of its four warps has the same number (one sequence of 4,096
    keys: 9.6 us with 16 splits, 10.1 with 18, 8.8 with 32).  Where three blocks per SM do not
    give more blocks than two per SM hold, the splits are those of two per SM."""
    tiles = max(1, -(-max_kv_len // 16))
    pairs = max(1, n_items * n_kv_heads)

    def splits_for(slots: int) -> int:
        most = max(1, min(slots // pairs, 128))
        per_split = max(8, -(-(-(-tiles // most)) // 4) * 4)
        return max(1, min(-(-tiles // per_split), most))

    wide = splits_for(444)
    return wide if pairs * wide > 296 else splits_for(296)


def attention_decode(q: torch.Tensor, out: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                     items: torch.Tensor, positions: torch.Tensor, tok_req: torch.Tensor,
                     req_slot: torch.Tensor, block_table: torch.Tensor, err: torch.Tensor, *,
                     scale: float, window: int | None, n_splits: int,
                     scratch: torch.Tensor | None = None, softcap: float | None = None,
                     sinks: torch.Tensor | None = None, chunk: int | None = None,
                     slopes: torch.Tensor | None = None,
                     dist_bias: torch.Tensor | None = None) -> None:
    """Split-K paged attention for the single next tokens listed in ``items`` (bfloat16 only).
    ``softcap``, ``sinks``, ``chunk``, ``slopes`` and ``dist_bias`` as in :func:`attention_plain`."""
    _want_sinks(sinks, q.shape[1])
    _want_sinks(slopes, q.shape[1])
    _want(q, torch.bfloat16, "q"); _want(out, torch.bfloat16, "out")
    _want(k_cache, torch.bfloat16, "k_cache"); _want(v_cache, torch.bfloat16, "v_cache")
    _want(items, torch.int32, "items")
    n, hq, d = q.shape
    num_pages, hkv, page_size, dk = k_cache.shape
    if not decode_kernel_takes(hq, hkv, d, page_size):
        raise KernelError(f"the split-K decode kernel does not take heads {hq}/{hkv}, head_dim {d}, "
                          f"page size {page_size}")
    n_items = items.numel()
    counters = _decode_counters(q.device, n_items * hkv)
    need = n_items * hq * n_splits * (d + 2)
    if scratch is None:
        scratch = torch.empty(need, dtype=torch.float32, device=q.device)
    else:
        _want(scratch, torch.float32, "scratch")
        if scratch.numel() < need:
            raise KernelError(f"scratch holds {scratch.numel()} floats, {need} needed")
    _check(_lib().tk_attention_decode(q.data_ptr(), out.data_ptr(), k_cache.data_ptr(),
                                         v_cache.data_ptr(), scratch.data_ptr(), counters.data_ptr(),
                                         items.data_ptr(),
                                         positions.data_ptr(), tok_req.data_ptr(), req_slot.data_ptr(),
                                         block_table.data_ptr(), err.data_ptr(), n_items,
                                         req_slot.numel(), hq, hkv, d, page_size, block_table.shape[1],
                                         num_pages, int(window or 0), n_splits, float(scale),
                                         float(softcap or 0.0), _ptr(sinks), int(chunk or 0), _ptr(slopes),
                                         _ptr(dist_bias), _want_dist_bias(dist_bias, hq), _stream()),
           "attention_decode")


# Which decode attention kernel the mixer uses: "balanced" deals the key tiles of all (token, kv head)
# pairs out evenly over two blocks per SM; "split" gives every pair the same number of splits; "auto"
# takes the balanced kernel where there are more pairs than blocks that run at a time (equal splits
# would run as a full wave and a partly filled one) or where a block gets some 320 tiles or more, so
# that its one or two merged parts weigh little.  Inside the decode step at the Qwen3-8B head sizes:
# batch 64, context 4,096: 6,700 against 6,300 tokens/s; batch 8, context 32,768: 895 against 864;
# batch 8, context 16,384: 1,313 against 1,327; batch 8, context 4,096: 2,010 against 2,090.
DECODE_ATTENTION = os.environ.get("TOKAMAK_B200_DECODE_ATTENTION", "auto")
DECODE_BALANCED_MAX_ITEMS = 1024
DECODE_BALANCED_MAX_BLOCKS = 512
_SM_COUNT: dict = {}
_BALANCED_SCRATCH: dict = {}


def decode_balanced_blocks(device: torch.device, n_items: int, n_kv_heads: int, max_kv_len: int) -> int:
    """Blocks of the balanced decode kernel: two per SM, fewer where that would leave a block with
    less than eight 16-key tiles (``max_kv_len`` bounds the longest context)."""
    sms = _SM_COUNT.get(device)
    if sms is None:
        sms = _SM_COUNT[device] = torch.cuda.get_device_properties(device).multi_processor_count
    tiles = n_items * n_kv_heads * max(1, -(-max_kv_len // 16))
    return max(1, min(2 * sms, DECODE_BALANCED_MAX_BLOCKS, tiles // 8))


def decode_uses_balanced(device: torch.device, n_items: int, n_kv_heads: int, max_kv_len: int) -> bool:
    """Whether the mixer should take the balanced decode kernel for this many single tokens whose
    longest context is at most ``max_kv_len``."""
    if DECODE_ATTENTION == "split" or n_items > DECODE_BALANCED_MAX_ITEMS:
        return False
    if DECODE_ATTENTION == "balanced":
        return True
    decode_balanced_blocks(device, 1, 1, 16)           # makes sure the SM count is known
    blocks = 2 * _SM_COUNT[device]
    pairs = n_items * n_kv_heads
    if pairs > blocks:
        return True
    # Fewer pairs than that: equal splits fill the SMs three blocks deep (batch 8 at contexts of
    # 16,384 and 32,768: 1,369 and 911 tokens/s against 1,325 and 891 with the tiles dealt out),
    # unless there are too many pairs to split at all and a long context to stream
    return decode_splits(n_items, n_kv_heads, max_kv_len) == 1 and pairs * -(-max_kv_len // 16) >= 320 * blocks


def attention_decode_balanced(q: torch.Tensor, out: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                              items: torch.Tensor, positions: torch.Tensor, tok_req: torch.Tensor,
                              req_slot: torch.Tensor, block_table: torch.Tensor, err: torch.Tensor, *,
                              scale: float, window: int | None, blocks: int, softcap: float | None = None,
                              sinks: torch.Tensor | None = None, chunk: int | None = None,
                              slopes: torch.Tensor | None = None,
                     dist_bias: torch.Tensor | None = None) -> None:
    """Paged attention for the single next tokens listed in ``items`` (bfloat16 only), the key tiles of
    all (token, kv head) pairs dealt out evenly over ``blocks`` blocks.  ``softcap``, ``sinks``, ``chunk``
    and ``slopes`` as in :func:`attention_plain`."""
    _want_sinks(sinks, q.shape[1])
    _want_sinks(slopes, q.shape[1])
    _want(q, torch.bfloat16, "q"); _want(out, torch.bfloat16, "out")
    _want(k_cache, torch.bfloat16, "k_cache"); _want(v_cache, torch.bfloat16, "v_cache")
    _want(items, torch.int32, "items")
    n, hq, d = q.shape
    num_pages, hkv, page_size, dk = k_cache.shape
    n_items = items.numel()
    if (not decode_kernel_takes(hq, hkv, d, page_size) or n_items > DECODE_BALANCED_MAX_ITEMS
            or not 1 <= blocks <= DECODE_BALANCED_MAX_BLOCKS):
        raise KernelError(f"the balanced decode kernel does not take heads {hq}/{hkv}, head_dim {d}, "
                          f"page size {page_size}, {n_items} tokens, {blocks} blocks")
    lib = _lib()
    need = lib.tk_attention_decode_balanced_scratch_floats(blocks, d)
    scratch = _BALANCED_SCRATCH.get(q.device)
    if scratch is None or scratch.numel() < need:
        if scratch is not None:
            _RETIRED_COUNTERS.append(scratch)        # captured graphs still hold its address
        scratch = _BALANCED_SCRATCH[q.device] = torch.empty(max(need, 1 << 20), dtype=torch.float32, device=q.device)
    counters = _decode_counters(q.device, n_items * hkv)
    _check(lib.tk_attention_decode_balanced(q.data_ptr(), out.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(),
                                            scratch.data_ptr(), counters.data_ptr(), items.data_ptr(),
                                            positions.data_ptr(), tok_req.data_ptr(), req_slot.data_ptr(),
                                            block_table.data_ptr(), err.data_ptr(), n_items, req_slot.numel(),
                                            hq, hkv, d, page_size, block_table.shape[1], num_pages,
                                            int(window or 0), blocks, float(scale), float(softcap or 0.0),
                                            _ptr(sinks), int(chunk or 0), _ptr(slopes), _ptr(dist_bias),
                                            _want_dist_bias(dist_bias, hq), _stream()),
           "attention_decode_balanced")


def attention_prefill(q: torch.Tensor, out: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                      tiles: torch.Tensor, req_q_start: torch.Tensor, req_q_len: torch.Tensor,
                      req_kv_len: torch.Tensor, req_slot: torch.Tensor, block_table: torch.Tensor,
                      err: torch.Tensor, *, scale: float, window: int | None) -> None:
    """Paged flash attention for the 64-token query tiles listed in ``tiles`` (bfloat16 only).

    ``tiles`` is int32 ``[n_tiles, 2]``: the request's row in the per-request arrays and the
    index of the tile within the tokens that the request brings to this step."""
    _want(q, torch.bfloat16, "q"); _want(out, torch.bfloat16, "out")
    _want(k_cache, torch.bfloat16, "k_cache"); _want(v_cache, torch.bfloat16, "v_cache")
    _want(tiles, torch.int32, "tiles")
    n, hq, d = q.shape
    num_pages, hkv, page_size, dk = k_cache.shape
    if not prefill_kernel_takes(hq, hkv, d, page_size) or dk != d:
        raise KernelError(f"the flash prefill kernel does not take heads {hq}/{hkv}, head_dim {d}")
    _check(_lib().tk_attention_prefill(q.data_ptr(), out.data_ptr(), k_cache.data_ptr(),
                                          v_cache.data_ptr(), tiles.data_ptr(), req_q_start.data_ptr(),
                                          req_q_len.data_ptr(), req_kv_len.data_ptr(),
                                          req_slot.data_ptr(), block_table.data_ptr(), err.data_ptr(),
                                          tiles.numel() // 2, req_slot.numel(), hq, hkv, d, page_size,
                                          block_table.shape[1], num_pages, int(window or 0),
                                          float(scale), _stream()), "attention_prefill")


PREFILL_TC_ROWS = 256     # query tokens per item of the tcgen05 prefill kernel (two tiles of 128)
PREFILL_TC_KEYS = 64      # keys per tile
PREFILL_TC_RECORD = 12    # int32 fields of an item record
PREFILL_TC_MAX_PARTS = 64
PREFILL_TC_MIN_PART = 8   # key tiles: shorter parts cost more in hand-overs than they balance


@dataclass
class PrefillItems:
    """Work list of :func:`attention_prefill_tc`, made by :func:`prefill_tc_records` and uploaded by
    the caller: ``records`` int32 ``[n, PREFILL_TC_RECORD]`` on the device, and how many parts of cut
    token blocks and how many cut token blocks it holds (sizes of the scratch memory)."""
    records: torch.Tensor
    n_parts: int
    n_split: int


def prefill_tc_records(q_start, q_len, kv_len, slots, *, heads: int, sms: int,
                       parts: int | None = None) -> tuple[np.ndarray, int, int]:
    """Item records of the tcgen05 prefill kernel for the requests that bring more than one token.

    The tokens of a request are cut into blocks of :data:`PREFILL_TC_ROWS`; block ``b`` visits the
    64-key tiles ``0 .. (pos0 + rows - 1) // 64`` (``pos0 = kv_len - q_len + 256 b``; a window
    shortens the walk inside the kernel).  Every block is one item per query head.  The kernel deals
    items out longest first to one thread block per SM.  Where there are fewer items than half the
    SMs (one short portion against a long context), every block is cut along its keys into parts of
    equal length (at least :data:`PREFILL_TC_MIN_PART` tiles each), as many as keep all items in one
    round over the SMs; the kernel adds the parts up.  Measured on a B200: a cut costs a part about
    as much as writing its rows out, and the part that adds up a few microseconds more, so with a
    round of items or more to deal out, cutting loses.  ``heads`` is the number of query heads the
    list is balanced for (the kernel takes any).

    Returns ``(records, n_parts, n_split)``: int32 ``[n, PREFILL_TC_RECORD]`` with the fields
    ``tok0, rows, pos0, slot, kt_begin, kt_end, part, n_parts, poff, split, merger`` longest first, the total
    number of parts of cut blocks, and the number of cut blocks."""
    blocks = []
    for r in range(len(q_len)):
        if q_len[r] <= 1:
            continue
        base = kv_len[r] - q_len[r]
        for b in range(-(-q_len[r] // PREFILL_TC_ROWS)):
            rows = min(PREFILL_TC_ROWS, q_len[r] - PREFILL_TC_ROWS * b)
            pos0 = base + PREFILL_TC_ROWS * b
            blocks.append((q_start[r] + PREFILL_TC_ROWS * b, rows, pos0, slots[r],
                           (pos0 + rows - 1) // PREFILL_TC_KEYS + 1))
    # cutting pays only where the SMs would otherwise stand idle: with fewer items than half the SMs,
    # every block is cut into as many parts as keeps all items in one round over the SMs
    n_items = len(blocks) * max(1, heads)
    parts_all = min(max(1, sms) // n_items, PREFILL_TC_MAX_PARTS) if n_items else 1
    if parts is not None:
        parts_all = parts        # a measurement's own choice
    records, poff, split = [], 0, 0
    for tok0, rows, pos0, slot, n_kt in blocks:
        n_cut = max(1, min(parts_all, n_kt // PREFILL_TC_MIN_PART))
        for i in range(n_cut):
            records.append((tok0, rows, pos0, slot, n_kt * i // n_cut, n_kt * (i + 1) // n_cut, i, n_cut,
                            poff if n_cut > 1 else 0, split if n_cut > 1 else 0, 0, 0))
        if n_cut > 1:
            poff += n_cut
            split += 1
    records.sort(key=lambda rec: rec[4] - rec[5])          # longest first; equal lengths keep their order
    out = np.asarray(records, dtype=np.int32).reshape(-1, PREFILL_TC_RECORD)
    # the part of a cut block that comes last in the list adds the parts up: the kernel hands items
    # out in list order, so all the others are running or done when it gets there
    last_of = {}
    for i, rec in enumerate(records):
        if rec[7] > 1:
            last_of[rec[9]] = i
    for i in last_of.values():
        out[i, 10] = 1
    return out, poff, split


_PREFILL_TC_WS: dict = {}


def _prefill_tc_workspace(device: torch.device, part_slots: int, counters: int, head_dim: int) -> dict:
    """Counters (zero between launches) and scratch of the tcgen05 prefill kernel, one set per device."""
    ws = _PREFILL_TC_WS.get(device)
    if ws is None:
        ws = _PREFILL_TC_WS[device] = {"sched": torch.zeros(2, dtype=torch.int32, device=device),
                                       "count": torch.zeros(1024, dtype=torch.int32, device=device),
                                       "o": None, "ml": None}
    if ws["count"].numel() < counters:
        ws["count"] = torch.zeros(max(counters, 2 * ws["count"].numel()), dtype=torch.int32, device=device)
    floats = part_slots * 128 * head_dim
    if floats > 0 and (ws["o"] is None or ws["o"].numel() < floats):
        ws["o"] = torch.empty(floats, dtype=torch.float32, device=device)
        ws["ml"] = torch.empty(part_slots * 128 * 2, dtype=torch.float32, device=device)
    return ws


def attention_prefill_tc(q: torch.Tensor, out: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                         items: PrefillItems, block_table: torch.Tensor, err: torch.Tensor, *,
                         scale: float, window: int | None, softcap: float | None = None,
                         sinks: torch.Tensor | None = None, chunk: int | None = None,
                         slopes: torch.Tensor | None = None,
                     dist_bias: torch.Tensor | None = None) -> None:
    """Paged flash attention on tcgen05 for the work list ``items`` (see :func:`prefill_tc_records`),
    a persistent kernel that deals the items out to one block per SM.  Loads whole pages: the cache
    must have been written by :func:`rope_kv` with ``req_q_len`` and ``req_kv_len`` given.  One call
    at a time per device: the calls share counters and scratch."""
    _want(q, torch.bfloat16, "q"); _want(out, torch.bfloat16, "out")
    _want(k_cache, torch.bfloat16, "k_cache"); _want(v_cache, torch.bfloat16, "v_cache")
    _want(items.records, torch.int32, "items.records")
    n, hq, d = q.shape
    num_pages, hkv, page_size, dk = k_cache.shape
    if not prefill_tc_kernel_takes(hq, hkv, d, page_size) or dk != d:
        raise KernelError(f"the tcgen05 prefill kernel does not take heads {hq}/{hkv}, head_dim {d}, "
                          f"page size {page_size}")
    if items.records.dim() != 2 or items.records.shape[1] != PREFILL_TC_RECORD:
        raise KernelError(f"item records want {PREFILL_TC_RECORD} fields, got shape {tuple(items.records.shape)}")
    ws = _prefill_tc_workspace(q.device, items.n_parts * hq * 2, items.n_split * hq * 2, d)
    part_o = ws["o"].data_ptr() if items.n_parts > 0 else 0
    part_ml = ws["ml"].data_ptr() if items.n_parts > 0 else 0
    _check(_lib().tk_attention_prefill_tc(q.data_ptr(), out.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(),
                                          items.records.data_ptr(), block_table.data_ptr(), err.data_ptr(),
                                          ws["sched"].data_ptr(), part_o, part_ml, ws["count"].data_ptr(),
                                          n, items.records.shape[0], hq, hkv, d, page_size,
                                          block_table.shape[1], num_pages, int(window or 0),
                                          float(scale), float(softcap or 0.0), _ptr(sinks), int(chunk or 0),
                                          _ptr(slopes), _ptr(dist_bias), _want_dist_bias(dist_bias, hq), _stream()),
           "attention_prefill_tc")


def sm_count(device: torch.device) -> int:
    """Streaming multiprocessors of the device."""
    sms = _SM_COUNT.get(device)
    if sms is None:
        sms = _SM_COUNT[device] = torch.cuda.get_device_properties(device).multi_processor_count
    return sms


def prefill_tc_kernel_takes(n_q_heads: int, n_kv_heads: int, head_dim: int, page_size: int) -> bool:
    """Shapes of the tcgen05 prefill kernel."""
    return bool(library().tk_attention_prefill_tc_takes(n_q_heads, n_kv_heads, head_dim, page_size))


def prefill_kernel_takes(n_q_heads: int, n_kv_heads: int, head_dim: int, page_size: int) -> bool:
    """Shapes of the tensor-core prefill kernel; everything else goes to the general kernel."""
    return head_dim in (64, 128) and n_q_heads % n_kv_heads == 0 and page_size >= 1


_DECODE_COUNTERS: dict = {}
_RETIRED_COUNTERS: list = []


def _decode_counters(device: torch.device, n: int) -> torch.Tensor:
    """Arrival counters of the decode kernel: zero between calls, one buffer per device.  A call
    that needs more than the buffer holds gets a larger one; the smaller one is kept alive for
    good, because CUDA graphs captured earlier still hold its address."""
    buf = _DECODE_COUNTERS.get(device)
    if buf is None or buf.numel() < n:
        if buf is not None:
            _RETIRED_COUNTERS.append(buf)
        buf = torch.zeros(max(65536, n), dtype=torch.int32, device=device)
        _DECODE_COUNTERS[device] = buf
    return buf


def decode_kernel_takes(n_q_heads: int, n_kv_heads: int, head_dim: int, page_size: int) -> bool:
    """Shapes of the tensor-core decode kernel; everything else goes to the general kernel."""
    return (head_dim in (64, 128) and page_size % 16 == 0 and n_q_heads % n_kv_heads == 0
            and n_q_heads // n_kv_heads <= 16)


def gemm_f32(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    """out[M, N] = a[M, K] @ w[N, K]^T in true float32 (FFMA, ascending k)."""
    _want(a, torch.float32, "a"); _want(w, torch.float32, "w")
    m, k = a.shape
    n, kw = w.shape
    if k != kw:
        raise KernelError(f"inner sizes differ: {k} and {kw}")
    if out is None:
        out = torch.empty((m, n), dtype=torch.float32, device=a.device)
    else:
        _want(out, torch.float32, "out")
        if out.shape != (m, n):
            raise KernelError("out has the wrong shape")
    _check(_lib().tk_gemm_f32(a.data_ptr(), w.data_ptr(), out.data_ptr(), m, n, k, k, k, n,
                                 _stream()), "gemm_f32")
    return out


def gemm_f32_heads(x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """``out[h, t, :] = w[h] @ x[t, h, :]`` in true float32: ``x`` is a ``[tokens, heads, K]`` view with a
    dense last axis, ``w`` ``[heads, M, K]`` contiguous; returns ``[heads, tokens, M]``."""
    _want(w, torch.float32, "w")
    n, heads, k = x.shape
    if x.dtype != torch.float32 or not x.is_cuda or x.stride(2) != 1 or w.shape[0] != heads or w.shape[2] != k:
        raise KernelError("x must be float32 [tokens, heads, K] with a dense last axis and w [heads, M, K]")
    m = w.shape[1]
    out = torch.empty((heads, n, m), dtype=torch.float32, device=x.device)
    _check(_lib().tk_gemm_f32_batched(x.data_ptr(), w.data_ptr(), out.data_ptr(), n, m, k, x.stride(0), k, m, heads,
                                         x.stride(1), m * k, n * m, _stream()), "gemm_f32_heads")
    return out


def _stacked(x: torch.Tensor, like: torch.dtype, name: str) -> tuple:
    """(pointer | None, parts pointer | None, parts, part stride, tokens, row length) of a product's result."""
    t, parts, n_parts, n, row = _parts_of(x, like, name)
    return _ptr(t), _ptr(parts), n_parts, (parts.stride(0) if parts is not None else 0), n, row


def latent_prepare(proj: torch.Tensor, cache: torch.Tensor, positions: torch.Tensor, tok_req: torch.Tensor,
                   req_slot: torch.Tensor, block_table: torch.Tensor, err: torch.Tensor, *, kv_off: int, rank: int,
                   rot: int, kv_norm_w: torch.Tensor, eps: float, table: torch.Tensor | None = None,
                   q_abs: torch.Tensor | None = None, q_off: int = 0, q_head_cols: int = 0, q_rot_off: int = 0,
                   cq_off: int = 0, cq_norm_w: torch.Tensor | None = None,
                   req_q_len: torch.Tensor | None = None, req_kv_len: torch.Tensor | None = None):
    """A latent cache's rows for the step's tokens, and what the queries need, from the columns of the
    stacked projection ``proj`` (the cache's type, or float32 partial sums).

    Columns ``kv_off .. + rank`` are RMS-normed with ``kv_norm_w`` (the latent), the ``rot`` columns
    behind them are the shared key part, whose first ``2 * table.shape[1]`` elements turn as
    neighbouring pairs by the (cos, sin) of ``table``; both go to the token's row of ``cache``
    ``[pages, 1, page, rank + rot]``.  With ``q_abs`` (float32 ``[heads, tokens, rank]``) the query rows
    ``[tokens, heads, rank + rot]`` are returned in float32: ``q_abs`` and the turned columns
    ``q_off + h * q_head_cols + q_rot_off .. + rot``.  With ``cq_norm_w`` the columns ``cq_off .. +
    len(cq_norm_w)`` are RMS-normed into a second result ``[tokens, len(cq_norm_w)]``.
    Returns ``(query rows | None, normed query latent | None)``."""
    _want(cache, None, "cache"); _want(kv_norm_w, torch.float32, "kv_norm_w")
    x, parts, n_parts, part_stride, n, row = _stacked(proj, cache.dtype, "proj")
    num_pages, one, page_size, width = cache.shape
    if one != 1 or width != rank + rot or kv_norm_w.numel() != rank or kv_off < 0 or kv_off + width > row:
        raise KernelError("the cache rows or the latent's columns do not match the sizes")
    pairs = 0
    if table is not None:
        _want(table, torch.float32, "table")
        pairs = table.shape[1]
        if table.shape[0] != n or 2 * pairs > rot:
            raise KernelError("the rotation table does not match the tokens or the rotated part")
    heads, q_lat = 0, None
    if q_abs is not None:
        _want(q_abs, torch.float32, "q_abs")
        heads = q_abs.shape[0]
        if q_abs.shape != (heads, n, rank) or q_off < 0 or q_off + (heads - 1) * q_head_cols + q_rot_off + rot > row:
            raise KernelError("q_abs must be [heads, tokens, rank] and the rotated query columns inside the row")
        q_lat = torch.empty((n, heads, width), dtype=torch.float32, device=cache.device)
    cq, cq_rank = None, 0
    if cq_norm_w is not None:
        _want(cq_norm_w, torch.float32, "cq_norm_w")
        cq_rank = cq_norm_w.numel()
        if cq_off < 0 or cq_off + cq_rank > row:
            raise KernelError("the query latent's columns lie outside the row")
        cq = torch.empty((n, cq_rank), dtype=cache.dtype, device=cache.device)
    for name, t in (("positions", positions), ("tok_req", tok_req), ("req_slot", req_slot), ("block_table", block_table)):
        _want(t, torch.int32, name)
    _check(_lib().tk_latent_prepare(x, parts, n_parts, part_stride, row, kv_off, q_off, q_head_cols, q_rot_off, cq_off,
                                       cq_rank, kv_norm_w.data_ptr(), _ptr(cq_norm_w), _ptr(cq), _ptr(q_abs), _ptr(q_lat),
                                       cache.data_ptr(), _ptr(table), positions.data_ptr(), tok_req.data_ptr(),
                                       req_slot.data_ptr(), block_table.data_ptr(), _ptr(req_q_len), _ptr(req_kv_len),
                                       err.data_ptr(), n, req_slot.numel(), heads, rank, rot, pairs, page_size,
                                       block_table.shape[1], num_pages, float(eps), dtype_code(cache.dtype), _stream()),
           "latent_prepare")
    return q_lat, cq


def heads_gate(x: torch.Tensor, proj: torch.Tensor | None = None, g_off: int = 0) -> torch.Tensor:
    """``y[t, h * dv + e] = x[h, t, e] * sigmoid(proj[t, g_off + h * dv + e])`` (``proj=None``: no gate):
    per-head results ``[heads, tokens, dv]`` back as token rows ``[tokens, heads * dv]``."""
    _want(x, None, "x")
    heads, n, dv = x.shape
    gx = gparts = None
    n_parts, part_stride, row = 0, 0, 0
    if proj is not None:
        gx, gparts, n_parts, part_stride, n2, row = _stacked(proj, x.dtype, "proj")
        if n2 != n or g_off < 0 or g_off + heads * dv > row:
            raise KernelError("the gate columns lie outside the row")
    else:
        g_off = -1
    y = torch.empty((n, heads * dv), dtype=x.dtype, device=x.device)
    _check(_lib().tk_heads_gate(x.data_ptr(), gx, gparts, n_parts, part_stride, row, g_off, y.data_ptr(), n, heads, dv,
                                   dtype_code(x.dtype), _stream()), "heads_gate")
    return y


def delta_record_floats(heads: int, kv_heads: int, key_dim: int, value_dim: int, taps: int) -> tuple[int, int]:
    """``(floats of a request's record, where the convolution's tail starts)``: the state of every head,
    then the last ``taps - 1`` inputs of every q, k and v channel."""
    state = heads * key_dim * value_dim
    return state + (taps - 1) * (2 * kv_heads * key_dim + heads * value_dim), state


def delta_prepare(proj: torch.Tensor, taps: torch.Tensor, a_log: torch.Tensor, dt_bias: torch.Tensor,
                  records: torch.Tensor, tok_req: torch.Tensor, req_q_start: torch.Tensor, req_q_len: torch.Tensor,
                  req_slot: torch.Tensor, err: torch.Tensor, *, dtype: torch.dtype, q_off: int, k_off: int, v_off: int,
                  b_off: int, a_off: int, heads: int, kv_heads: int, key_dim: int, value_dim: int, unit_eps: float,
                  q_scale: float, shape: int = 0) -> tuple:
    """The float32 inputs of the delta-rule recurrence from the columns of the stacked projection
    ``proj`` (type ``dtype``, or float32 partial sums): short causal convolution (``taps`` float32
    ``[channels, K]``, channels in the order q, k, v) and silu on q, k and v, q and k heads scaled to
    unit length (q also by ``q_scale``), ``beta = sigmoid(b)`` and ``g = exp(-exp(a_log) softplus(a +
    dt_bias))`` per head.  The convolution reads the inputs before the step from the tail of the
    requests' ``records`` (float32 ``[slots, floats]``, see :func:`delta_record_floats`) and moves the tail on
    (every request must bring at least one token: with as many tokens as requests the same kernel does both).
    ``shape``: 0 lets the launcher choose a warp (many tokens) or a block (few) per head, 1 and 2 force one;
    the results are the same bits.
    Returns ``(q [N, Hk, dk], k [N, Hk, dk], v [N, H, dv], beta [N, H], g [N, H])``."""
    _want(taps, torch.float32, "taps"); _want(a_log, torch.float32, "a_log"); _want(dt_bias, torch.float32, "dt_bias")
    _want(records, torch.float32, "records")
    x, parts, n_parts, part_stride, n, row = _stacked(proj, dtype, "proj")
    hk, hv = kv_heads * key_dim, heads * value_dim
    channels, k_taps = taps.shape
    floats, tail_off = delta_record_floats(heads, kv_heads, key_dim, value_dim, k_taps)
    if channels != 2 * hk + hv or records.dim() != 2 or records.shape[1] != floats:
        raise KernelError("taps must be [q + k + v channels, K] and the records sized by delta_record_floats")
    if a_log.numel() != heads or dt_bias.numel() != heads:
        raise KernelError("one A_log and one dt_bias per head are needed")
    for off, size in ((q_off, hk), (k_off, hk), (v_off, hv), (b_off, heads), (a_off, heads)):
        if off < 0 or off + size > row:
            raise KernelError("a column range lies outside the row")
    for name, t in (("tok_req", tok_req), ("req_q_start", req_q_start), ("req_q_len", req_q_len), ("req_slot", req_slot)):
        _want(t, torch.int32, name)
    dev = records.device
    q = torch.empty((n, kv_heads, key_dim), dtype=torch.float32, device=dev)
    k = torch.empty_like(q)
    v = torch.empty((n, heads, value_dim), dtype=torch.float32, device=dev)
    beta = torch.empty((n, heads), dtype=torch.float32, device=dev)
    g = torch.empty_like(beta)
    _check(_lib().tk_delta_prepare(x, parts, n_parts, part_stride, row, q_off, k_off, v_off, b_off, a_off,
                                      taps.data_ptr(), a_log.data_ptr(), dt_bias.data_ptr(), records.data_ptr(), floats,
                                      tail_off, tok_req.data_ptr(), req_q_start.data_ptr(), req_q_len.data_ptr(),
                                      req_slot.data_ptr(), q.data_ptr(), k.data_ptr(), v.data_ptr(), beta.data_ptr(),
                                      g.data_ptr(), err.data_ptr(), n, req_slot.numel(), records.shape[0], heads,
                                      kv_heads, key_dim, value_dim, k_taps, float(unit_eps), float(q_scale),
                                      dtype_code(dtype), 1, int(shape), _stream()), "delta_prepare")
    global LAUNCHES
    LAUNCHES += 1 if k_taps > 1 and n != req_slot.numel() else 0       # the kernel that moves the tail on
    return q, k, v, beta, g


def delta_scan(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, beta: torch.Tensor, g: torch.Tensor,
               records: torch.Tensor, req_q_start: torch.Tensor, req_q_len: torch.Tensor, req_slot: torch.Tensor,
               err: torch.Tensor, *, cols: int = 0) -> torch.Tensor:
    """The gated delta rule ``S = g S; u = beta (v - S^T k); S += k u^T; o = S^T q`` over every request's
    tokens of the step; the states ``[heads, dk, dv]`` lead the requests' float32 ``records`` and are
    advanced in place.  Returns ``o`` float32 ``[tokens, heads, dv]``.  ``cols`` is the number of value
    channels a block takes (64, 32 or 16: eight warps of 8, 4 or 2 columns; 0: what the sizes of the heads suggest)."""
    for name, t in (("q", q), ("k", k), ("v", v), ("beta", beta), ("g", g), ("records", records)):
        _want(t, torch.float32, name)
    n, kv_heads, dk = q.shape
    _, heads, dv = v.shape
    if k.shape != q.shape or v.shape[0] != n or beta.shape != (n, heads) or g.shape != (n, heads) or heads % kv_heads:
        raise KernelError("the recurrence's inputs do not match one another")
    if records.dim() != 2 or records.shape[1] < heads * dk * dv:
        raise KernelError("a record is too short for the state")
    if dk > 256:
        raise KernelError(f"key size {dk} is beyond the kernel's limit of 256")
    for name, t in (("req_q_start", req_q_start), ("req_q_len", req_q_len), ("req_slot", req_slot)):
        _want(t, torch.int32, name)
    out = torch.empty((n, heads, dv), dtype=torch.float32, device=records.device)
    _check(_lib().tk_delta_scan(q.data_ptr(), k.data_ptr(), v.data_ptr(), beta.data_ptr(), g.data_ptr(),
                                   records.data_ptr(), records.shape[1], out.data_ptr(), req_q_start.data_ptr(),
                                   req_q_len.data_ptr(), req_slot.data_ptr(), err.data_ptr(), req_slot.numel(),
                                   records.shape[0], heads, kv_heads, dk, dv, int(cols), _stream()), "delta_scan")
    return out


SWIGLU_TILE_BLOCK = 64     # gate/up rows alternate in blocks of this many for the fused activation
# Most (token, choice) pairs of a step whose experts are streamed by the CUDA cores (the kernel takes up to 64).
# Measured at 8 experts of 4,096 x 2,048, two per token: 1 token 31 us against 65 us on the tensor cores'
# padded tiles, 4 tokens 87 against 125, 8 tokens 147 against 152, 16 tokens 281 against 157: a pair costs the
# CUDA cores as much arithmetic as the weights cost to fetch, from about three pairs an expert on.
MOE_SMALL_PAIRS = 8


def gemm_tc_swapped(weight: torch.Tensor, x: torch.Tensor, err: torch.Tensor, n_splits: int,
                    out: torch.Tensor | None = None, max_stages: int = 0, cluster: int = 0,
                    swiglu: bool = False, activation: str = "silu", colscale: tuple | None = None,
                    residual_norm: tuple | None = None, chain: "ProductChain | None" = None,
                    unary: str | None = None):
    """``x @ weight^T`` on tcgen05, the weight being the 128-row operand (for few tokens: every
    weight byte is streamed once by TMA), as float32 partial sums ``[parts, tokens, N_out]`` for
    the caller to add up.  ``parts = n_splits``, or ``n_splits / cluster`` with ``cluster`` in
    2..8 (a divisor of ``n_splits``): that many consecutive splits of a tile form a thread-block
    cluster that adds its partials up itself.

    ``swiglu=True``: the weight is a stacked gate/up matrix whose rows alternate in blocks of
    ``SWIGLU_TILE_BLOCK`` (gate rows, then the up rows of the same outputs); all splits form one
    cluster and the result is bfloat16 ``[tokens, N_out / 2] = silu(gate) * up``.

    ``unary`` (a name of ``UNARY_ACTIVATIONS``; ``N_out`` a multiple of 128, all splits in one cluster): the result
    is bfloat16 ``[tokens, N_out] = act(sums)``.

    ``colscale=(sumsq, dim, eps)`` with ``sumsq`` float32 ``[tiles, tokens]``: every token's sums
    are multiplied by ``rsqrt(sum over tiles / dim + eps)`` (all splits in one cluster): ``x``
    then holds activations whose RMS scale is still owed.

    ``residual_norm=(resid, norm_weight)`` (all splits in one cluster, ``N_out`` a multiple of
    128): the sums are added to the float32 residual stream ``resid [tokens, N_out]`` in place and
    ``(xb, sumsq)`` is returned: ``xb = bf16(resid * norm_weight)`` and the tiles' sums of squares
    ``[N_out / 128, tokens]``, ready to be the ``x`` and ``colscale`` of the next product.

    ``chain``: a :class:`ProductChain`; a product whose result is a single part is queued in it
    instead of launched (the result tensors are returned all the same, to be filled at the flush)."""
    _want(weight, torch.bfloat16, "weight"); _want(x, torch.bfloat16, "x")
    n_out, k = weight.shape
    tokens, kx = x.shape
    if k != kx or k % 8:
        raise KernelError(f"inner sizes {k} and {kx} must agree and be a multiple of 8")
    if tokens > 256:
        raise KernelError("the swapped product takes at most 256 tokens")
    if cluster > 1 and (cluster > 8 or n_splits % cluster):
        raise KernelError("a cluster holds 2..8 splits and must divide their count")
    bn = 16
    while bn < tokens:
        bn *= 2
    parts = n_splits // cluster if cluster > 1 else n_splits
    cs_ptr, cs_n, cs_inv, cs_eps = None, 0, 0.0, 0.0
    if colscale is not None:
        sumsq, dim, eps = colscale
        _want(sumsq, torch.float32, "colscale sums")
        if parts != 1 or sumsq.dim() != 2 or sumsq.shape[1] != tokens:
            raise KernelError("colscale wants one cluster and sums of squares [tiles, tokens]")
        cs_ptr, cs_n, cs_inv, cs_eps = sumsq.data_ptr(), sumsq.shape[0], 1.0 / dim, float(eps)
    epilogue, resid_ptr, w_ptr, xb, sums_out, result = 0, None, None, None, None, None
    if residual_norm is not None:
        resid, norm_w = residual_norm
        _want(resid, torch.float32, "resid"); _want(norm_w, torch.float32, "norm weight")
        if swiglu or parts != 1 or n_out % 128 or resid.shape != (tokens, n_out) or norm_w.numel() != n_out:
            raise KernelError("residual_norm wants one cluster, N_out a multiple of 128 and resid [tokens, N_out]")
        xb = torch.empty((tokens, n_out), dtype=torch.bfloat16, device=x.device)
        sums_out = torch.empty((n_out // 128, tokens), dtype=torch.float32, device=x.device)
        epilogue, resid_ptr, w_ptr, result = 2, resid.data_ptr(), norm_w.data_ptr(), (xb, sums_out)
        out_ptr = None
    elif swiglu:
        if n_out % (2 * SWIGLU_TILE_BLOCK) or parts != 1:
            raise KernelError("the fused activation wants rows in blocks of 64 gate + 64 up and one cluster")
        if out is None:
            out = torch.empty((tokens, n_out // 2), dtype=torch.bfloat16, device=x.device)
        if activation not in GLU_ACTIVATIONS:
            raise KernelError(f"unknown activation {activation!r}")
        epilogue, out_ptr, result = (1 if activation == "silu" else 4), out.data_ptr(), out
    elif unary is not None:
        if n_out % 128 or parts != 1 or unary not in UNARY_ACTIVATIONS:
            raise KernelError("the fused ungated activation wants rows in steps of 128, one cluster and a known name")
        if out is None:
            out = torch.empty((tokens, n_out), dtype=torch.bfloat16, device=x.device)
        epilogue, out_ptr, result, chain = 5 + UNARY_ACTIVATIONS[unary], out.data_ptr(), out, None
    else:
        if out is None:
            out = torch.empty((parts, tokens, n_out), dtype=torch.float32, device=x.device)
        out_ptr, result = out.data_ptr(), out
    def alone():
        _check(library().tk_gemm_bf16_tcgen05(weight.data_ptr(), x.data_ptr(), out_ptr, err.data_ptr(),
                                              n_out, tokens, k, k, k, bn, n_splits, max_stages,
                                              cluster if cluster > 1 else 0, epilogue, cs_ptr, cs_n, cs_inv, cs_eps,
                                              resid_ptr, w_ptr, _ptr(xb), _ptr(sums_out), _stream()),
               "gemm_tc_swapped")

    if chain is not None and parts == 1 and ProductChain.takes(tokens, n_out):
        a = _ChainPhaseArgs()
        a.w, a.x, a.ld_w, a.ld_x, a.rows, a.k, a.epilogue = weight.data_ptr(), x.data_ptr(), k, k, n_out, k, epilogue
        a.out, a.colscale_parts, a.n_colscale_parts = out_ptr, cs_ptr, cs_n
        a.colscale_inv_dim, a.colscale_eps = cs_inv, cs_eps
        a.resid, a.norm_w, a.xb_out, a.sumsq_out = resid_ptr, w_ptr, _ptr(xb), _ptr(sums_out)
        chain.add(a, alone, (weight, x, result, colscale, residual_norm))
        return result
    flush_chains()
    alone()
    return result


QKV_ROPE_HEAD_DIM = 128    # the head size whose heads are whole 128-row tiles of the swapped product


# ---- chains of decode products ---------------------------------------------------------------------

CHAIN_MAX_TOKENS = 64
# Whether the parts queue their decode products into chains ("on") or launch every product as a kernel
# of its own ("off").  Measured at the Qwen3-8B sizes, batch 8: 4.9 ms a step chained against 3.8 ms
# with one kernel per product, so the default is "off"; gemm_chain.cu says where the time goes.
CHAIN_POLICY = os.environ.get("TOKAMAK_B200_CHAIN", "off")


class _ChainPhaseArgs(__import__("ctypes").Structure):
    """``TkChainPhaseArgs`` of gemm_chain.cu."""
    import ctypes as _c
    _fields_ = [("w", _c.c_void_p), ("x", _c.c_void_p), ("ld_w", _c.c_longlong), ("ld_x", _c.c_longlong),
                ("rows", _c.c_int), ("k", _c.c_int), ("epilogue", _c.c_int), ("n_colscale_parts", _c.c_int),
                ("out", _c.c_void_p), ("colscale_parts", _c.c_void_p),
                ("colscale_inv_dim", _c.c_float), ("colscale_eps", _c.c_float),
                ("resid", _c.c_void_p), ("norm_w", _c.c_void_p), ("xb_out", _c.c_void_p), ("sumsq_out", _c.c_void_p),
                ("q_out", _c.c_void_p), ("k_cache", _c.c_void_p), ("v_cache", _c.c_void_p),
                ("positions", _c.c_void_p), ("tok_req", _c.c_void_p), ("req_slot", _c.c_void_p),
                ("block_table", _c.c_void_p), ("req_q_len", _c.c_void_p), ("req_kv_len", _c.c_void_p),
                ("q_norm_w", _c.c_void_p), ("k_norm_w", _c.c_void_p), ("rope_table", _c.c_void_p),
                ("n_reqs", _c.c_int), ("n_q_heads", _c.c_int), ("n_kv_heads", _c.c_int), ("page_size", _c.c_int),
                ("max_pages", _c.c_int), ("num_pages", _c.c_int), ("eps", _c.c_float), ("reserved", _c.c_int)]
    del _c


_CHAIN_WORKSPACES: dict = {}
_CHAIN_MAX_TILES = 2048          # most 128-row tiles of one product (a head of 262,144 rows)


def _chain_workspace(device: torch.device) -> tuple[torch.Tensor, torch.Tensor]:
    """Scratch for the parts of tiles and the (zero) counters of the chain kernel, one per device."""
    ws = _CHAIN_WORKSPACES.get(device)
    if ws is None:
        lib = library()
        scratch = torch.empty(lib.tk_gemm_chain_scratch_floats(CHAIN_MAX_TOKENS), dtype=torch.float32, device=device)
        counters = torch.zeros(lib.tk_gemm_chain_counter_ints(_CHAIN_MAX_TILES), dtype=torch.int32, device=device)
        ws = _CHAIN_WORKSPACES[device] = (scratch, counters)
    return ws


def reset_workspaces() -> None:
    """Put the counters that kernels expect at zero back to zero (after a kernel reported an error
    and may have left them otherwise)."""
    for _, counters in _CHAIN_WORKSPACES.values():
        counters.zero_()
    for buf in _DECODE_COUNTERS.values():
        buf.zero_()
    for ws in _PREFILL_TC_WS.values():
        ws["sched"].zero_()
        ws["count"].zero_()


class ProductChain:
    """Decode products whose launch is put off so that consecutive ones run as ONE persistent
    kernel (gemm_chain.cu): the weights of the next product stream in while the sums of the one
    before are added up and stored.

    :func:`gemm_tc_swapped` and :func:`gemm_qkv_rope` take a chain; with one, a product that ends
    in a single part is queued instead of launched, and its result tensors are returned at once,
    not yet computed.  :meth:`flush` launches what is queued; every other kernel wrapper of this
    module calls it first, so a kernel of this library never reads a result that is still queued.
    Code that reads such a tensor in any other way must call :meth:`flush` itself.
    """

    def __init__(self, tokens: int, err: torch.Tensor):
        self.tokens = tokens
        self.err = err
        self.phases: list[tuple[_ChainPhaseArgs, object]] = []     # (arguments, launch on its own)
        self.keep: list = []
        self.max_phases = library().tk_gemm_chain_max_phases()

    @staticmethod
    def takes(tokens: int, n_out: int) -> bool:
        return 1 <= tokens <= CHAIN_MAX_TOKENS and -(-n_out // 128) <= _CHAIN_MAX_TILES

    def add(self, args: _ChainPhaseArgs, alone, keep: tuple) -> None:
        if len(self.phases) == self.max_phases:
            self.flush()
        if not self.phases:
            self.stream = _stream()
        self.phases.append((args, alone))
        self.keep.append(keep)               # operands stay allocated until the launch
        if self not in _ACTIVE_CHAINS:
            _ACTIVE_CHAINS.append(self)

    def flush(self) -> None:
        if not self.phases:
            return
        phases, self.phases, self.keep = self.phases, [], []
        if _stream() != self.stream:
            raise KernelError("queued products are being launched on another stream than they were queued on; "
                              "call ops.flush_chains() before changing the stream")
        if len(phases) == 1:
            phases[0][1]()                     # a single product: the kernel tuned for it
            return
        arr = (_ChainPhaseArgs * len(phases))(*[a for a, _ in phases])
        scratch, counters = _chain_workspace(self.err.device)
        _check(library().tk_gemm_chain(arr, len(phases), self.tokens, self.err.data_ptr(), scratch.data_ptr(),
                                       counters.data_ptr(), _CHAIN_MAX_TILES, _stream()), "gemm_chain")


def flush_chains() -> None:
    chains = list(_ACTIVE_CHAINS)
    _ACTIVE_CHAINS.clear()
    for chain in chains:
        chain.flush()


def gemm_qkv_rope(weight: torch.Tensor, x: torch.Tensor, err: torch.Tensor, n_splits: int, q_out: torch.Tensor,
                  k_cache: torch.Tensor, v_cache: torch.Tensor, positions: torch.Tensor, tok_req: torch.Tensor,
                  req_slot: torch.Tensor, block_table: torch.Tensor, q_norm_w: torch.Tensor | None,
                  k_norm_w: torch.Tensor | None, table: torch.Tensor | None, *, n_q_heads: int, n_kv_heads: int,
                  eps: float, max_stages: int = 0, colscale: tuple | None = None,
                  req_q_len: torch.Tensor | None = None, req_kv_len: torch.Tensor | None = None,
                  chain: "ProductChain | None" = None) -> None:
    """The stacked q|k|v projection of few tokens with :func:`rope_kv`'s work in its epilogue, for
    heads of 128 elements: ``weight`` is ``[(Hq + 2 Hkv) 128, K]``, ``x`` ``[tokens, K]``; ``q_out``
    receives the normed and rotated queries, the keys and values go to their pages.  All
    ``n_splits`` (at most 8) blocks of a head form one cluster.  ``colscale`` as in
    :func:`gemm_tc_swapped`; ``table`` is the rotation table ``[tokens, 64, 2]`` or None."""
    _want(weight, torch.bfloat16, "weight"); _want(x, torch.bfloat16, "x"); _want(q_out, torch.bfloat16, "q_out")
    _want(k_cache, torch.bfloat16, "k_cache"); _want(v_cache, torch.bfloat16, "v_cache")
    d = QKV_ROPE_HEAD_DIM
    n_out, k = weight.shape
    tokens, kx = x.shape
    if k != kx or k % 8:
        raise KernelError(f"inner sizes {k} and {kx} must agree and be a multiple of 8")
    if n_out != (n_q_heads + 2 * n_kv_heads) * d:
        raise KernelError(f"the weight has {n_out} rows, {(n_q_heads + 2 * n_kv_heads) * d} needed for heads of {d}")
    if tokens > 256 or not 1 <= n_splits <= 8:
        raise KernelError("the swapped product takes at most 256 tokens and 8 splits in a cluster")
    if q_out.shape != (tokens, n_q_heads, d):
        raise KernelError(f"q_out must be [{tokens}, {n_q_heads}, {d}]")
    num_pages, hkv, page_size, dk = k_cache.shape
    if hkv != n_kv_heads or dk != d or v_cache.shape != k_cache.shape:
        raise KernelError("cache pages do not match the heads")
    for name, t in (("positions", positions), ("tok_req", tok_req), ("req_slot", req_slot),
                    ("block_table", block_table)):
        _want(t, torch.int32, name)
    for name, t in (("q_norm_w", q_norm_w), ("k_norm_w", k_norm_w), ("table", table)):
        if t is not None:
            _want(t, torch.float32, name)
    for name, t in (("q_norm_w", q_norm_w), ("k_norm_w", k_norm_w)):
        if t is not None and t.numel() != d:
            raise KernelError(f"{name} does not match head_dim {d}")
    if table is not None and table.shape != (tokens, d // 2, 2):
        raise KernelError(f"the rotation table must be [{tokens}, {d // 2}, 2], got {tuple(table.shape)}")
    if (req_q_len is None) != (req_kv_len is None):
        raise KernelError("req_q_len and req_kv_len come together")
    cs_ptr, cs_n, cs_inv, cs_eps = None, 0, 0.0, 0.0
    if colscale is not None:
        sumsq, dim, cs_eps = colscale
        _want(sumsq, torch.float32, "colscale sums")
        if sumsq.dim() != 2 or sumsq.shape[1] != tokens:
            raise KernelError("colscale wants sums of squares [tiles, tokens]")
        cs_ptr, cs_n, cs_inv, cs_eps = sumsq.data_ptr(), sumsq.shape[0], 1.0 / dim, float(cs_eps)
    bn = 16
    while bn < tokens:
        bn *= 2
    def alone():
        _check(library().tk_gemm_qkv_rope(weight.data_ptr(), x.data_ptr(), err.data_ptr(), tokens, k, k, k, bn,
                                          n_splits, max_stages, cs_ptr, cs_n, cs_inv, cs_eps,
                                          q_out.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(),
                                          positions.data_ptr(), tok_req.data_ptr(), req_slot.data_ptr(),
                                          block_table.data_ptr(), _ptr(req_q_len), _ptr(req_kv_len),
                                          _ptr(q_norm_w), _ptr(k_norm_w), _ptr(table), req_slot.numel(),
                                          n_q_heads, n_kv_heads, page_size, block_table.shape[1], num_pages,
                                          float(eps), _stream()), "gemm_qkv_rope")

    if chain is not None and ProductChain.takes(tokens, n_out):
        a = _ChainPhaseArgs()
        a.w, a.x, a.ld_w, a.ld_x, a.rows, a.k, a.epilogue = weight.data_ptr(), x.data_ptr(), k, k, n_out, k, 3
        a.colscale_parts, a.n_colscale_parts, a.colscale_inv_dim, a.colscale_eps = cs_ptr, cs_n, cs_inv, cs_eps
        a.q_out, a.k_cache, a.v_cache = q_out.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr()
        a.positions, a.tok_req, a.req_slot = positions.data_ptr(), tok_req.data_ptr(), req_slot.data_ptr()
        a.block_table, a.req_q_len, a.req_kv_len = block_table.data_ptr(), _ptr(req_q_len), _ptr(req_kv_len)
        a.q_norm_w, a.k_norm_w, a.rope_table = _ptr(q_norm_w), _ptr(k_norm_w), _ptr(table)
        a.n_reqs, a.n_q_heads, a.n_kv_heads, a.page_size = req_slot.numel(), n_q_heads, n_kv_heads, page_size
        a.max_pages, a.num_pages, a.eps = block_table.shape[1], num_pages, float(eps)
        chain.add(a, alone, (weight, x, q_out, colscale, table, q_norm_w, k_norm_w, positions))
        return
    flush_chains()
    alone()


def swapped_gemm_plan(n_out: int, k: int, tokens: int = 8) -> tuple[int, int, int]:
    """(K splits, pipeline stages, cluster size) of the swapped product.

    About 2.5 to 3 blocks per SM, each with at least four 64-wide k blocks, so that several
    blocks share an SM and one block's start-up hides behind another's streaming; the splits of
    a tile (at most 8) form one cluster that adds its partials up, so the consumer sees a single
    part.  Rings of three stages; four where the grid is short enough that its blocks still all
    fit: with at most 16 tokens a single split or up to about 2.7 blocks per SM (three such
    blocks fit an SM), with more tokens (larger stages) up to two blocks per SM.  Measured on
    the Qwen3-8B decode step: 16 splits in two clusters, deeper rings and other block counts were
    all slower, and so were four stages for the long gate/up grid, and for the q|k|v and head
    products at 32 and 64 tokens (head at 64 tokens: 195 us with three stages, 212 with four)."""
    tiles = -(-n_out // 128)
    k_blocks = -(-k // 64)
    splits = max(1, min(round(448 / tiles), max(1, k_blocks // 4), 8))
    if tokens <= 16:
        stages = 4 if splits == 1 or tiles * splits <= 400 else 3
    else:
        stages = 4 if tiles * splits <= 296 else 3
    return splits, stages, splits


# Which products of many tokens run on the engine's own kernel for pairs of SMs: "all" of them,
# only the gate/up product with the "fused" activation, or none ("off": the library everywhere).
PAIR_GEMM_POLICY = os.environ.get("TOKAMAK_B200_PAIR_GEMM", "all")
PAIR_GEMM_MIN_TILES = 96     # below this the grid of SM pairs is too empty and the library is faster


def pair_gemm_takes(tokens: int, n_out: int, k: int, fused: bool = False) -> bool:
    """Whether :func:`gemm_pair` is the product to use: the policy allows it, there are enough
    256 x 256 tiles to keep the 74 pairs of SMs busy, and its TMA maps and 16-byte stores can
    address the sizes."""
    if PAIR_GEMM_POLICY == "off" or (PAIR_GEMM_POLICY == "fused" and not fused):
        return False
    tiles = -(-tokens // 256) * -(-n_out // 256)
    return tiles >= PAIR_GEMM_MIN_TILES and k % 8 == 0 and n_out % 8 == 0


def gemm_pair(x: torch.Tensor, weight: torch.Tensor, err: torch.Tensor, swiglu: bool = False,
              activation: str = "silu", unary: str | None = None) -> torch.Tensor:
    """``x @ weight^T`` for many tokens on pairs of SMs (tcgen05.mma.cta_group::2, persistent grid);
    bfloat16 ``[tokens, N_out]``.  ``swiglu=True``: the weight is a stacked gate/up matrix whose rows
    alternate in blocks of ``SWIGLU_TILE_BLOCK``; the result is ``[tokens, N_out / 2] = silu(gate) * up``.
    ``unary`` (a name of ``UNARY_ACTIVATIONS``): the result is ``act(x @ weight^T)``."""
    _want(weight, torch.bfloat16, "weight"); _want(x, torch.bfloat16, "x")
    n_out, k = weight.shape
    tokens, kx = x.shape
    if k != kx or k % 8:
        raise KernelError(f"inner sizes {k} and {kx} must agree and be a multiple of 8")
    if swiglu and n_out % (2 * SWIGLU_TILE_BLOCK):
        raise KernelError("the fused activation wants rows in blocks of 64 gate + 64 up")
    width = n_out // 2 if swiglu else n_out
    if swiglu and activation not in GLU_ACTIVATIONS:
        raise KernelError(f"unknown activation {activation!r}")
    mode = 1 + GLU_ACTIVATIONS[activation] if swiglu else 0
    if unary is not None:
        if swiglu or unary not in UNARY_ACTIVATIONS:
            raise KernelError(f"an ungated activation {unary!r} beside a gated one, or unknown")
        mode = 3 + UNARY_ACTIVATIONS[unary]
    if width % 8:
        raise KernelError("the output width must be a multiple of 8")
    out = torch.empty((tokens, width), dtype=torch.bfloat16, device=x.device)
    _check(_lib().tk_gemm_bf16_pair(x.data_ptr(), weight.data_ptr(), out.data_ptr(), err.data_ptr(), tokens,
                                       n_out, k, k, k, width, mode, _stream()), "gemm_pair")
    return out


def sample(logits: torch.Tensor, temperature: torch.Tensor, top_k: torch.Tensor, top_p: torch.Tensor,
           seed: torch.Tensor, counter: torch.Tensor, out_tokens: torch.Tensor) -> None:
    """One token per row of float32 logits; see sampling.cu for the exact rule."""
    _want(logits, torch.float32, "logits"); _want(temperature, torch.float32, "temperature")
    _want(top_k, torch.int32, "top_k"); _want(top_p, torch.float32, "top_p")
    _want(seed, torch.int64, "seed"); _want(counter, torch.int32, "counter")
    _want(out_tokens, torch.int32, "out_tokens")
    rows, vocab = logits.shape
    for t in (temperature, top_k, top_p, seed, counter, out_tokens):
        if t.numel() < rows:
            raise KernelError("a per-row sampling tensor is shorter than the batch")
    _sampling_takes(rows, vocab)
    _check(_lib().tk_sample(logits.data_ptr(), logits.stride(0), temperature.data_ptr(),
                               top_k.data_ptr(), top_p.data_ptr(), seed.data_ptr(), counter.data_ptr(),
                               out_tokens.data_ptr(), rows, vocab, _stream()), "sample")


_TIMELINE_FILES = ("gemm_tcgen05", "gemm_chain", "attention_decode", "attention_prefill_tc", "sampling", "step_state",
                   "elementwise")


def timeline_start(capacity: int = 1 << 20) -> torch.Tensor:
    """Hand the kernels a buffer for their time stamps (a library built with -DTK_TIMELINE only,
    see timeline.cuh) and return it; :func:`timeline_read` decodes it."""
    import ctypes
    lib = library()
    if not hasattr(lib, "tk_timeline_set_gemm_tcgen05"):
        raise KernelError("the library was built without -DTK_TIMELINE (set TOKAMAK_B200_NVCC_FLAGS)")
    buf = torch.zeros(1 + 2 * capacity, dtype=torch.int64, device="cuda")
    for name in _TIMELINE_FILES:
        fn = getattr(lib, "tk_timeline_set_" + name)
        fn.argtypes = [ctypes.c_void_p, ctypes.c_uint]
        fn.restype = ctypes.c_int
        code = fn(buf.data_ptr(), capacity)
        if code != 0:
            raise KernelError(f"timeline_set_{name}: CUDA error {code}")
    return buf


def timeline_read(buf: torch.Tensor) -> list[tuple[int, int, int, int, int]]:
    """(time in ns, kernel, phase, SM, block) records in the order of time; clears the buffer."""
    torch.cuda.synchronize()
    host = buf.cpu()
    n = min(int(host[0]), (host.numel() - 1) // 2)
    out = []
    for i in range(n):
        t, rec = int(host[1 + 2 * i]), int(host[2 + 2 * i]) & 0xFFFFFFFFFFFFFFFF
        out.append((t, (rec >> 56) & 0xFF, (rec >> 48) & 0xFF, (rec >> 32) & 0xFFFF, rec & 0xFFFFFFFF))
    buf.zero_()
    return sorted(out)


def philox_u32(seed: int, counter: int) -> int:
    """First word of the generator's block for (seed, counter), computed on the host."""
    import ctypes
    out = (ctypes.c_uint * 4)()
    library().tk_philox_u32(seed & 0xFFFFFFFFFFFFFFFF, counter & 0xFFFFFFFF, out)
    return int(out[0])
