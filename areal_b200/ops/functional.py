"""Tensor-level ops of the framework.

Each op has two implementations with identical semantics:

* ``*_ref``: plain PyTorch (fp32 math), used on CPU tensors and as the numerical oracle in
  tests;
* the sm_100a kernel from ``libab2_kernels.so`` for CUDA tensors (bf16 activations), wrapped
  in ``torch.autograd.Function`` where the op is differentiable.

Public entry points dispatch on ``tensor.is_cuda`` only: CPU -> reference, CUDA -> kernel
(raising if the library cannot be loaded; there is no silent CUDA fallback).
"""
from __future__ import annotations

import math
import os
from typing import Optional

import torch
import torch.nn.functional as F

from . import lib as _lib

EPI_BF16, EPI_F32, EPI_F32_ACC, EPI_BF16_RESID = 0, 1, 2, 3
# 2-CTA (cta_group::2) GEMM for large products (measured 1.56-1.58 against 1.43-1.44 PFLOP/s of the one-CTA kernel at
# 8192^3 and 32768 x 4096 x 4096, same bits): AB2_GEMM_2SM=0 keeps everything on the one-CTA kernel
GEMM_2SM = os.environ.get("AB2_GEMM_2SM", "1") == "1"
GEMM_2SM_MIN_M = 1024


def _L():
    return _lib.get_lib()


def _s():
    return _lib.stream_ptr()


# ----------------------------------------------------------------------------- GEMM
def gemm(a: torch.Tensor, b: torch.Tensor, *, a_mn: bool = False, b_mn: bool = False,
         out: Optional[torch.Tensor] = None, epi: int = EPI_BF16, resid: Optional[torch.Tensor] = None,
         bn: int = 0) -> torch.Tensor:
    """``C = op(A) @ op(B)`` on tcgen05 tensor cores (bf16 in, fp32 accumulate).

    ``a``: ``[M,K]`` (or ``[K,M]`` when ``a_mn``); ``b``: ``[N,K]`` (or ``[K,N]`` when
    ``b_mn``). ``epi``: EPI_BF16 store, EPI_F32 store, EPI_F32_ACC accumulate into ``out``,
    EPI_BF16_RESID store of ``acc + resid``.
    """
    assert a.dtype == torch.bfloat16 and b.dtype == torch.bfloat16
    assert a.stride(-1) == 1 and b.stride(-1) == 1 and a.dim() == 2 and b.dim() == 2
    M, K = (a.shape[1], a.shape[0]) if a_mn else (a.shape[0], a.shape[1])
    N, Kb = (b.shape[1], b.shape[0]) if b_mn else (b.shape[0], b.shape[1])
    assert K == Kb, f"inner dims differ: {K} vs {Kb}"
    if out is None:
        assert epi != EPI_F32_ACC
        out = torch.empty(M, N, device=a.device, dtype=torch.float32 if epi == EPI_F32 else torch.bfloat16)
    assert out.shape == (M, N) and out.stride(1) == 1
    if not a.is_cuda:
        A = (a.t() if a_mn else a).float()
        B = (b if b_mn else b.t()).float()
        acc = A @ B
        if epi == EPI_F32_ACC:
            out += acc
        elif epi == EPI_BF16_RESID:
            out.copy_((acc + resid.float()).to(out.dtype))
        else:
            out.copy_(acc.to(out.dtype))
        return out
    if epi == EPI_BF16_RESID:
        assert resid is not None and resid.shape == out.shape and resid.stride() == out.stride()
    if GEMM_2SM and bn == 0 and M >= GEMM_2SM_MIN_M and N >= 512 and K >= 256:
        # large products: 256 x 256 tiles on CTA pairs (tcgen05 cta_group::2), half the B traffic per SM
        rc = _L().ab2_gemm_bf16_2sm(a.data_ptr(), b.data_ptr(), out.data_ptr(), _lib.ptr(resid), M, N, K, a.stride(0), b.stride(0),
                                    out.stride(0), int(a_mn), int(b_mn), epi, _s())
        _lib.check(rc, "ab2_gemm_bf16_2sm")
        return out
    rc = _L().ab2_gemm_bf16(a.data_ptr(), b.data_ptr(), out.data_ptr(), _lib.ptr(resid), M, N, K, a.stride(0),
                            b.stride(0), out.stride(0), int(a_mn), int(b_mn), epi, bn, _s())
    _lib.check(rc, "ab2_gemm_bf16")
    return out


# ----------------------------------------------------------------------------- grouped (expert) GEMM
def grouped_tile_table(counts, n_cols: int, bn: int, device) -> torch.Tensor:
    """int32 [num_tiles, 4] = (expert, first row, valid rows, n-block) for row groups of sizes
    ``counts`` (rows sorted by expert)."""
    rows = []
    off = 0
    nb = (n_cols + bn - 1) // bn
    for e, n in enumerate(counts):
        n = int(n)
        for r0 in range(0, n, 128):
            valid = min(128, n - r0)
            for b in range(nb):
                rows.append((e, off + r0, valid, b))
        off += n
    if not rows:
        return torch.zeros(0, 4, dtype=torch.int32, device=device)
    return torch.tensor(rows, dtype=torch.int32).to(device, non_blocking=True)


def grouped_gemm_ref(x, w, counts, b_mn: bool = False):
    outs, off = [], 0
    for e, n in enumerate(counts):
        n = int(n)
        if n:
            we = w[e].float()
            outs.append(x[off:off + n].float() @ (we if b_mn else we.t()))
        off += n
    n_out = w.shape[2] if b_mn else w.shape[1]
    return (torch.cat(outs, 0) if outs else x.new_zeros(0, n_out)).to(x.dtype)


def grouped_gemm(x: torch.Tensor, w: torch.Tensor, counts, b_mn: bool = False, tiles: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Rows of ``x`` [R, K] are grouped by expert (``counts[e]`` rows each, in order); returns
    ``y`` [R, N] with ``y[group e] = x[group e] @ w[e]^T`` (``w``: [E, N, K]) or ``@ w[e]``
    (``b_mn``; ``w``: [E, K, N]). One persistent kernel for all experts."""
    if not x.is_cuda:
        return grouped_gemm_ref(x, w, counts, b_mn)
    assert x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and x.stride(1) == 1 and w.is_contiguous()
    R, K = x.shape
    E = w.shape[0]
    N = w.shape[2] if b_mn else w.shape[1]
    assert (w.shape[1] if b_mn else w.shape[2]) == K and sum(int(c) for c in counts) == R
    bn = 256 if N % 256 == 0 else 128
    if tiles is None:
        tiles = grouped_tile_table(counts, N, bn, x.device)
    y = torch.empty(R, N, device=x.device, dtype=torch.bfloat16)
    if tiles.shape[0]:
        rc = _L().ab2_gemm_grouped(x.data_ptr(), w.data_ptr(), y.data_ptr(), tiles.data_ptr(), tiles.shape[0], R, N, K, E, x.stride(0),
                                   y.stride(0), int(b_mn), bn, _s())
        _lib.check(rc, "ab2_gemm_grouped")
    return y


class Routing:
    """Expert assignment of a batch of tokens, made on the device (:func:`moe_route`).

    ``order[r]`` is the (token * k + slot) entry on row ``r`` of the expert-sorted layout, ``token_of[r]``
    its token, ``inv`` the inverse of ``order``; ``counts`` / ``offs`` are the group sizes and starts;
    ``row_tiles`` / ``num_row_tiles`` feed the grouped GEMM. ``host_counts()`` gives the group sizes as
    a list; the copy was started when the routing was made, so a caller that asks late (the weight
    gradients in backward) does not stall the stream."""

    def __init__(self, tope, topw, probs, counts, offs, order, token_of, inv, row_tiles, num_row_tiles, k):
        self.tope, self.topw, self.probs = tope, topw, probs
        self.counts, self.offs, self.order, self.token_of, self.inv = counts, offs, order, token_of, inv
        self.row_tiles, self.num_row_tiles, self.k = row_tiles, num_row_tiles, k
        self.rows = order.shape[0]
        self._host = None
        self._event = None
        if counts.is_cuda:
            self._host = torch.empty(counts.shape, dtype=counts.dtype, pin_memory=True)
            self._host.copy_(counts, non_blocking=True)
            self._event = torch.cuda.Event()
            self._event.record()

    def host_counts(self) -> list:
        if self._host is None:
            return self.counts.tolist()
        self._event.synchronize()
        return self._host.tolist()


def moe_route_ref(logits, k: int, bias=None, sigmoid: bool = False, norm: bool = True, scale: float = 1.0, tope=None):
    """PyTorch statement of :func:`moe_route` (ties between equal scores may resolve differently)."""
    T, E = logits.shape
    probs = torch.sigmoid(logits.float()) if sigmoid else torch.softmax(logits.float(), dim=-1)
    topw = None
    if tope is None:
        choice = probs if bias is None else probs + bias
        tope = torch.topk(choice, k, dim=-1).indices
        topw = probs.gather(1, tope)
        if norm:
            topw = topw / topw.sum(-1, keepdim=True).clamp(min=1e-20)
        topw = topw * scale
    flat = tope.reshape(-1).long()
    order = torch.argsort(flat, stable=True)
    counts = torch.bincount(flat, minlength=E)
    offs = torch.cat([counts.new_zeros(1), counts.cumsum(0)])
    inv = torch.empty_like(order)
    inv[order] = torch.arange(order.numel(), device=order.device)
    tiles = [(e, int(offs[e]) + r0, min(128, int(counts[e]) - r0), 0) for e in range(E) for r0 in range(0, int(counts[e]), 128)]
    rt = torch.tensor(tiles, dtype=torch.int32, device=logits.device).view(-1, 4)
    return Routing(tope.int(), topw, probs, counts.int(), offs.int(), order.int(), (order // k).int(), inv.int(), rt,
                   torch.tensor([rt.shape[0]], dtype=torch.int32, device=logits.device), k)


def moe_route(logits: torch.Tensor, k: int, bias: Optional[torch.Tensor] = None, sigmoid: bool = False, norm: bool = True,
              scale: float = 1.0, tope: Optional[torch.Tensor] = None, want_probs: bool = True) -> Routing:
    """Scores, top-k choice, stable sort by expert, group sizes and the grouped-GEMM tile list from fp32
    router logits [T, E], in four small launches and without a host read. With ``tope`` given (the choice
    was made elsewhere, e.g. group-limited routing) only the sort / counts / tiles are produced."""
    T, E = logits.shape
    if not logits.is_cuda or E > 256 or k > 16:
        return moe_route_ref(logits, k, bias, sigmoid, norm, scale, tope)
    dev = logits.device
    logits = logits.float().contiguous()
    n = T * k
    i32 = dict(dtype=torch.int32, device=dev)
    given = tope is not None
    tope_ = tope.to(torch.int32).contiguous() if given else torch.empty(T, k, **i32)
    topw = None if given else torch.empty(T, k, dtype=torch.float32, device=dev)
    probs = None if (given or not want_probs) else torch.empty(T, E, dtype=torch.float32, device=dev)
    counts, offs = torch.empty(E, **i32), torch.empty(E + 1, **i32)
    order, token_of, inv = torch.empty(n, **i32), torch.empty(n, **i32), torch.empty(n, **i32)
    max_rt = n // 128 + E
    row_tiles = torch.empty(max_rt, 4, **i32)
    num_rt = torch.empty(1, **i32)
    L = _L()
    ws = torch.empty(int(L.ab2_moe_route_workspace(n, E)), **i32)
    b = bias.float().contiguous() if bias is not None else None
    flags = (1 if sigmoid else 0) | (2 if norm else 0) | (4 if given else 0)
    rc = L.ab2_moe_route(logits.data_ptr(), _lib.ptr(b), T, E, k, flags, float(scale), _lib.ptr(probs), _lib.ptr(topw),
                         tope_.data_ptr(), counts.data_ptr(), offs.data_ptr(), order.data_ptr(), token_of.data_ptr(),
                         inv.data_ptr(), row_tiles.data_ptr(), num_rt.data_ptr(), max_rt, ws.data_ptr(), _s())
    _lib.check(rc, "ab2_moe_route")
    return Routing(tope_, topw, probs, counts, offs, order, token_of, inv, row_tiles, num_rt, k)


def grouped_gemm_rt(x: torch.Tensor, w: torch.Tensor, routing: Routing, b_mn: bool = False) -> torch.Tensor:
    """:func:`grouped_gemm` with the tile list of a device-made :class:`Routing` (no host copy of the group sizes)."""
    if not x.is_cuda:
        return grouped_gemm_ref(x, w, routing.host_counts(), b_mn)
    assert x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and x.stride(1) == 1 and w.is_contiguous()
    R, K = x.shape
    E = w.shape[0]
    N = w.shape[2] if b_mn else w.shape[1]
    assert (w.shape[1] if b_mn else w.shape[2]) == K and R == routing.rows
    bn = 256 if N % 256 == 0 else 128
    y = torch.empty(R, N, device=x.device, dtype=torch.bfloat16)
    if R:
        rc = _L().ab2_gemm_grouped_rt(x.data_ptr(), w.data_ptr(), y.data_ptr(), routing.row_tiles.data_ptr(),
                                      routing.num_row_tiles.data_ptr(), routing.row_tiles.shape[0], R, N, K, E, x.stride(0),
                                      y.stride(0), int(b_mn), bn, _s())
        _lib.check(rc, "ab2_gemm_grouped_rt")
    return y


class _GroupedLinear(torch.autograd.Function):
    """``y[group e] = x[group e] @ W[e]^T`` for stacked expert weights ``W`` [E, N, K]. Forward and
    input gradient are one grouped kernel each; weight gradients accumulate per expert in fp32
    (into ``W.main_grad`` when present)."""

    @staticmethod
    def forward(ctx, x, w, counts):
        ctx.routing = counts if isinstance(counts, Routing) else None
        ctx.counts = None if ctx.routing is not None else [int(c) for c in counts]
        ctx.save_for_backward(x, w)
        if ctx.routing is not None:
            return grouped_gemm_rt(x, w, ctx.routing)
        return grouped_gemm(x, w, ctx.counts)

    @staticmethod
    def backward(ctx, dy):
        x, w = ctx.saved_tensors
        dy = dy.contiguous()
        if ctx.routing is not None:
            dx = grouped_gemm_rt(dy, w, ctx.routing, b_mn=True) if ctx.needs_input_grad[0] else None
            counts = ctx.routing.host_counts()      # copied to the host since the forward pass: no stall here
        else:
            counts = ctx.counts
            dx = grouped_gemm(dy, w, counts, b_mn=True) if ctx.needs_input_grad[0] else None
        dw = None
        if ctx.needs_input_grad[1]:
            mg = getattr(w, "main_grad", None)

            def wgrad(acc):
                off = 0
                for e, n in enumerate(counts):
                    if n:
                        if x.is_cuda:
                            gemm(dy[off:off + n], x[off:off + n], a_mn=True, b_mn=True, out=acc[e], epi=EPI_F32_ACC)
                        else:
                            acc[e] += dy[off:off + n].float().t() @ x[off:off + n].float()
                    off += n
                return acc
            if _WGRAD_QUEUE is not None:
                # split backward: per-expert products run when the caller flushes the queue
                _WGRAD_QUEUE.append(lambda: wgrad(mg) if mg is not None else _accumulate_wgrad(
                    w, wgrad(torch.zeros(w.shape, device=w.device, dtype=torch.float32))))
            else:
                acc = wgrad(mg if mg is not None else torch.zeros(w.shape, device=w.device, dtype=torch.float32))
                dw = None if mg is not None else acc.to(w.dtype)
        return dx, dw, None


def grouped_linear(x: torch.Tensor, w: torch.Tensor, counts) -> torch.Tensor:
    """``counts``: group sizes as a list of ints, or a :class:`Routing` made on the device."""
    return _GroupedLinear.apply(x, w, counts)


SKINNY_MAX_TOKENS = 256
_skinny_ws: dict = {}


def _skinny_workspace(device, n_out: int):
    """Zeroed split-K workspace and tile counters, one set per (device, stream): launches on
    one stream are ordered, launches on different streams must not share them. The kernel
    leaves both zeroed."""
    key = (device.index, _s())
    ent = _skinny_ws.get(key)
    need = SKINNY_MAX_TOKENS * n_out
    if ent is None or ent[0].numel() < need:
        ws = torch.zeros(max(need, SKINNY_MAX_TOKENS * 32768), device=device, dtype=torch.float32)
        cnt = torch.zeros(4096, device=device, dtype=torch.int32)
        ent = _skinny_ws[key] = (ws, cnt)
    return ent


_SPLITK_WS: dict = {}
DECODE_SPLITK = os.environ.get("AB2_DECODE_SPLITK", "0") == "1"     # route decode-sized linear() calls through gemm_decode
DECODE_GEMM_MAX_ROWS = 128


def decode_gemm_plan(M: int, N: int, K: int, n_sms: int = 148) -> tuple[int, int]:
    """(tile width, K splits) for a decode-shaped product: the widest tile whose count, times the
    split, comes closest to one CTA per SM without exceeding it; at least 8 k-blocks per piece."""
    best = (128, 1, 0.0)
    for bn in (256, 128):
        if N % bn and N > bn:
            continue
        tiles = -(-N // bn) * -(-M // 128)
        max_split = max(1, (K // 64) // 8)
        split = max(1, min(max_split, n_sms // tiles if tiles <= n_sms else 1))
        fill = min(1.0, tiles * split / n_sms)
        # wider tiles re-read the activations less often: prefer them at equal fill
        score = fill + (0.05 if bn == 256 else 0.0)
        if score > best[2]:
            best = (bn, split, score)
    return best[0], best[1]


def gemm_decode(x: torch.Tensor, w: torch.Tensor, resid: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``x @ w^T (+ resid)`` for a handful of rows (decode): output tiles alone cannot fill the
    machine, so K is split over CTAs as well (fp32 pieces in a static workspace, one reduce
    kernel). Falls back to :func:`gemm` when no split is worth it."""
    M, K = x.shape
    N = w.shape[0]
    if not x.is_cuda:
        y = x.float() @ w.float().t()
        return (y + resid.float() if resid is not None else y).to(x.dtype)
    bn, splits = decode_gemm_plan(M, N, K)
    if splits <= 1 or N % 4 or x.stride(1) != 1 or w.stride(1) != 1:
        return gemm(x, w, epi=EPI_BF16_RESID, resid=resid) if resid is not None else gemm(x, w)
    need = splits * M * N
    key = (x.device.index, torch.cuda.current_stream(x.device).cuda_stream)
    ws = _SPLITK_WS.get(key)
    if ws is None or ws.numel() < need:
        ws = _SPLITK_WS[key] = torch.empty(max(need, 4 * DECODE_GEMM_MAX_ROWS * 32768), dtype=torch.float32, device=x.device)
    y = torch.empty(M, N, dtype=torch.bfloat16, device=x.device)
    if resid is not None:
        assert resid.shape == y.shape and resid.is_contiguous() and resid.dtype == torch.bfloat16
    rc = _L().ab2_gemm_splitk(x.data_ptr(), w.data_ptr(), y.data_ptr(), _lib.ptr(resid), ws.data_ptr(), M, N, K, x.stride(0), w.stride(0),
                              splits, bn, _s())
    _lib.check(rc, "ab2_gemm_splitk")
    return y


def gemm_skinny(x: torch.Tensor, w: torch.Tensor, resid: Optional[torch.Tensor] = None, out_dtype=torch.bfloat16,
                split_k: int = 0) -> torch.Tensor:
    """``x @ w^T (+ resid)`` for at most 256 rows of ``x``: the decode-shaped product, bound
    by streaming ``w`` once (swap-AB tcgen05 tiles, split-K reduced in L2)."""
    assert x.dim() == 2 and w.dim() == 2 and x.shape[1] == w.shape[1] and x.shape[0] <= SKINNY_MAX_TOKENS
    assert x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and x.stride(1) == 1 and w.stride(1) == 1
    M, K = x.shape
    N = w.shape[0]
    if not x.is_cuda:
        y = x.float() @ w.float().t()
        if resid is not None:
            y = y + resid.float()
        return y.to(out_dtype)
    y = torch.empty(M, N, device=x.device, dtype=out_dtype)
    if resid is not None:
        assert resid.shape == y.shape and resid.stride() == y.stride() and resid.dtype == torch.bfloat16
    ws, cnt = _skinny_workspace(x.device, N) if N <= 65536 else (None, None)
    rc = _L().ab2_gemm_skinny(x.data_ptr(), w.data_ptr(), y.data_ptr(), _lib.ptr(resid), _lib.ptr(ws), _lib.ptr(cnt), M, N, K,
                              x.stride(0), w.stride(0), y.stride(0), int(out_dtype == torch.float32),
                              split_k if ws is not None else 1, _s())
    _lib.check(rc, "ab2_gemm_skinny")
    return y


# ---- split backward (zero-bubble pipeline schedules): while a queue is installed, the backward of a
# linear layer computes only the input gradient and appends its weight-gradient product to the queue;
# the caller runs the queue later (after it has handed the input gradient to the previous stage).
_WGRAD_QUEUE: Optional[list] = None
SPLIT_BACKWARD = False          # set while a schedule that splits backward is running (selects the deferrable CPU path)


class deferred_wgrad:
    """``with deferred_wgrad() as q: loss.backward()`` leaves the weight-gradient work of every
    ``linear`` in ``q``; ``flush_wgrad(q)`` performs it."""

    def __enter__(self):
        global _WGRAD_QUEUE
        self.prev, self.queue = _WGRAD_QUEUE, []
        _WGRAD_QUEUE = self.queue
        return self.queue

    def __exit__(self, *exc):
        global _WGRAD_QUEUE
        _WGRAD_QUEUE = self.prev
        return False


def flush_wgrad(queue: list) -> None:
    with torch.no_grad():
        for fn in queue:
            fn()
    queue.clear()


def _accumulate_wgrad(w, g32):
    mg = getattr(w, "main_grad", None)
    if mg is not None:
        mg.add_(g32.to(mg.dtype))
    elif w.grad is None:
        w.grad = g32.to(w.dtype)
    else:
        w.grad.add_(g32.to(w.dtype))


class _LinearSplit(torch.autograd.Function):
    """Plain-PyTorch linear whose weight gradient can be deferred (the CPU counterpart of ``_Linear``)."""

    @staticmethod
    def forward(ctx, x, w, resid):
        ctx.save_for_backward(x, w)
        ctx.has_resid = resid is not None
        y = F.linear(x, w)
        return y + resid if resid is not None else y

    @staticmethod
    def backward(ctx, dy):
        x, w = ctx.saved_tensors
        dx = (dy @ w) if ctx.needs_input_grad[0] else None
        dw = None
        if ctx.needs_input_grad[1]:
            dy2, x2 = dy.reshape(-1, dy.shape[-1]), x.reshape(-1, x.shape[-1])
            if not w.is_leaf and getattr(w, "main_grad", None) is None:
                # a view of a parameter (one expert of a stack): its gradient has to travel on through autograd, so it
                # cannot wait in the queue
                dw = (dy2.float().t() @ x2.float()).to(w.dtype)
            else:
                def wgrad(dy2=dy2, x2=x2, w=w):
                    _accumulate_wgrad(w, dy2.float().t() @ x2.float())
                if _WGRAD_QUEUE is not None:
                    _WGRAD_QUEUE.append(wgrad)
                else:
                    wgrad()
        return dx, dw, (dy if ctx.has_resid else None)


class _Linear(torch.autograd.Function):
    """y = x @ W^T (+ residual). Weight gradients accumulate in fp32 into ``w.main_grad``
    when the parameter carries one (flat-shard training), else are returned in bf16."""

    @staticmethod
    def forward(ctx, x, w, resid, grad_buf=None):
        ctx.save_for_backward(x, w)
        ctx.has_resid = resid is not None
        ctx.grad_buf = grad_buf
        x2 = x.reshape(-1, x.shape[-1])
        if resid is not None:
            y = gemm(x2, w, epi=EPI_BF16_RESID, resid=resid.reshape(-1, w.shape[0]))
        else:
            y = gemm(x2, w)
        return y.view(*x.shape[:-1], w.shape[0])

    @staticmethod
    def backward(ctx, dy):
        x, w = ctx.saved_tensors
        dy2 = dy.reshape(-1, dy.shape[-1])
        if not dy2.is_contiguous():
            dy2 = dy2.contiguous()
        x2 = x.reshape(-1, x.shape[-1])
        dx = dw = None
        if ctx.needs_input_grad[0]:
            dx = gemm(dy2, w, b_mn=True).view_as(x)
        if ctx.grad_buf is not None:
            gemm(dy2, x2, a_mn=True, b_mn=True, out=ctx.grad_buf, epi=EPI_F32_ACC)
        elif ctx.needs_input_grad[1]:
            mg = getattr(w, "main_grad", None)
            if _WGRAD_QUEUE is not None and (mg is not None or w.is_leaf):
                # split backward: the product runs when the caller flushes the queue (a view of a parameter without
                # its own gradient buffer cannot wait: its gradient travels on through autograd)
                def wgrad(dy2=dy2, x2=x2, w=w, mg=mg):
                    if mg is not None:
                        gemm(dy2, x2, a_mn=True, b_mn=True, out=mg, epi=EPI_F32_ACC)
                    else:
                        _accumulate_wgrad(w, gemm(dy2, x2, a_mn=True, b_mn=True, epi=EPI_F32))
                _WGRAD_QUEUE.append(wgrad)
            elif mg is not None:
                gemm(dy2, x2, a_mn=True, b_mn=True, out=mg, epi=EPI_F32_ACC)
                dw = None
            else:
                dw = gemm(dy2, x2, a_mn=True, b_mn=True)
        return dx, dw, (dy if ctx.has_resid else None), None


def linear(x: torch.Tensor, w: torch.Tensor, resid: Optional[torch.Tensor] = None,
           grad_buf: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``x @ w^T (+ resid)``. ``grad_buf`` (fp32, shape of ``w``): the weight gradient is
    accumulated there even when ``w`` is a detached view (slices of stacked expert weights)."""
    if not x.is_cuda:
        if SPLIT_BACKWARD and torch.is_grad_enabled() and grad_buf is None:
            return _LinearSplit.apply(x, w, resid)
        y = F.linear(x, w)
        return y + resid if resid is not None else y
    # The swap-AB split-K kernel (gemm_skinny) is NOT routed here: in isolation (L2 flushed) it
    # beats the general kernel for <= 64 tokens on three of the four decode shapes of an 8B
    # model, but inside the decode CUDA graph the whole step came out slower (13.2 ms vs 10.1 ms
    # per step at 64 sequences), so decode keeps the general kernel; callers can use
    # gemm_skinny() explicitly.
    if DECODE_SPLITK and x.dim() == 2 and x.shape[0] <= DECODE_GEMM_MAX_ROWS and not torch.is_grad_enabled() and x.dtype == torch.bfloat16:
        return gemm_decode(x, w, resid)      # decode: split K as well, the output alone has too few tiles
    return _Linear.apply(x, w, resid, grad_buf)


# ----------------------------------------------------------------------------- RMSNorm
def rmsnorm_ref(x, w, eps, resid=None):
    if resid is not None:
        x = (x.float() + resid.float()).to(x.dtype)
    xf = x.float()
    y = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps) * w.float()
    return y.to(x.dtype), x


class _RMSNorm(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, resid, eps):
        H = x.shape[-1]
        x2 = x.reshape(-1, H)
        rows = x2.shape[0]
        y = torch.empty_like(x2)
        rstd = torch.empty(rows, device=x.device, dtype=torch.float32)
        if resid is not None:
            r2 = resid.reshape(-1, H)
            new_res = torch.empty_like(x2)
            rc = _L().ab2_rmsnorm_fwd(x2.data_ptr(), r2.data_ptr(), w.data_ptr(), y.data_ptr(), new_res.data_ptr(),
                                      rstd.data_ptr(), rows, H, eps, _s())
            saved_x = new_res
        else:
            rc = _L().ab2_rmsnorm_fwd(x2.data_ptr(), None, w.data_ptr(), y.data_ptr(), None, rstd.data_ptr(), rows, H,
                                      eps, _s())
            new_res = None
            saved_x = x2
        _lib.check(rc, "ab2_rmsnorm_fwd")
        ctx.save_for_backward(saved_x, w, rstd)
        ctx.has_resid = resid is not None
        ctx.shape = x.shape
        if new_res is None:  # the residual stream is the input itself; the caller keeps using it
            return y.view(x.shape), x2.new_empty(0)
        return y.view(x.shape), new_res.view(x.shape)

    @staticmethod
    def backward(ctx, dy, dres):
        x2, w, rstd = ctx.saved_tensors
        rows, H = x2.shape
        dy2 = dy.reshape(rows, H).contiguous()
        dr2 = dres.reshape(rows, H).contiguous() if (dres is not None and ctx.has_resid) else None
        dx = torch.empty_like(x2)
        mg = getattr(w, "main_grad", None)
        dw32 = mg if mg is not None else torch.zeros(H, device=x2.device, dtype=torch.float32)
        rc = _L().ab2_rmsnorm_bwd(x2.data_ptr(), w.data_ptr(), dy2.data_ptr(), _lib.ptr(dr2), rstd.data_ptr(),
                                  dx.data_ptr(), dw32.data_ptr(), rows, H, _s())
        _lib.check(rc, "ab2_rmsnorm_bwd")
        dxv = dx.view(ctx.shape)
        return dxv, (None if mg is not None else dw32.to(w.dtype)), (dxv if ctx.has_resid else None), None


def rmsnorm(x, w, eps: float = 1e-6, resid=None):
    """Returns ``(normed, residual_stream)`` where ``residual_stream = x (+ resid)``."""
    if not x.is_cuda:
        return rmsnorm_ref(x, w, eps, resid)
    x = x.contiguous()
    if resid is None:
        y, _ = _RMSNorm.apply(x, w, None, eps)
        return y, x
    return _RMSNorm.apply(x, w, resid.contiguous(), eps)


# ----------------------------------------------------------------------------- RoPE
def rope_tables(max_pos: int, dim: int, theta: float, device) -> tuple[torch.Tensor, torch.Tensor]:
    inv = 1.0 / (theta ** (torch.arange(0, dim, 2, dtype=torch.float32, device=device) / dim))
    ang = torch.arange(max_pos, dtype=torch.float32, device=device)[:, None] * inv[None, :]
    return ang.cos().contiguous(), ang.sin().contiguous()


def rope_ref(x, pos, cos, sin, backward=False):
    # x: [T, h, D]; rotate-half convention (HF Qwen/Llama)
    D = x.shape[-1]
    c = cos[pos][:, None, :]
    s = sin[pos][:, None, :]
    if backward:
        s = -s
    xf = x.float()
    a, b = xf[..., : D // 2], xf[..., D // 2:]
    return torch.cat([a * c - b * s, b * c + a * s], dim=-1).to(x.dtype)


class _Rope(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, pos, cos, sin):
        ctx.save_for_backward(pos, cos, sin)
        y = x.clone() if x.is_contiguous() else x.contiguous()
        T, h, D = y.shape
        rc = _L().ab2_rope(y.data_ptr(), pos.data_ptr(), cos.data_ptr(), sin.data_ptr(), T, h, D, y.stride(0), 0, _s())
        _lib.check(rc, "ab2_rope")
        return y

    @staticmethod
    def backward(ctx, dy):
        pos, cos, sin = ctx.saved_tensors
        g = dy.clone() if dy.is_contiguous() else dy.contiguous()
        T, h, D = g.shape
        rc = _L().ab2_rope(g.data_ptr(), pos.data_ptr(), cos.data_ptr(), sin.data_ptr(), T, h, D, g.stride(0), 1, _s())
        _lib.check(rc, "ab2_rope")
        return g, None, None, None


def rope(x, pos, cos, sin):
    """x: [T, heads, D] bf16; pos: [T] int32; cos/sin: [max_pos, D/2] fp32."""
    if not x.is_cuda:
        return rope_ref(x, pos.long(), cos, sin)
    return _Rope.apply(x, pos, cos, sin)


def rope_inplace_(x, pos, cos, sin):
    """In-place rotary embedding on a (possibly strided) ``[T, heads, D]`` view. No autograd."""
    if not x.is_cuda:
        x.copy_(rope_ref(x, pos.long(), cos, sin))
        return x
    T, h, D = x.shape
    assert x.stride(2) == 1 and x.stride(1) == D
    rc = _L().ab2_rope(x.data_ptr(), pos.data_ptr(), cos.data_ptr(), sin.data_ptr(), T, h, D, x.stride(0), 0, _s())
    _lib.check(rc, "ab2_rope")
    return x


# ----------------------------------------------------------------------------- SwiGLU
def swiglu_ref(gu):
    I = gu.shape[-1] // 2
    g, u = gu[..., :I].float(), gu[..., I:].float()
    return (F.silu(g) * u).to(gu.dtype)


class _SwiGLU(torch.autograd.Function):
    @staticmethod
    def forward(ctx, gu):
        ctx.save_for_backward(gu)
        I = gu.shape[-1] // 2
        g2 = gu.reshape(-1, 2 * I)
        out = torch.empty(g2.shape[0], I, device=gu.device, dtype=gu.dtype)
        _lib.check(_L().ab2_swiglu_fwd(g2.data_ptr(), out.data_ptr(), g2.shape[0], I, _s()), "ab2_swiglu_fwd")
        return out.view(*gu.shape[:-1], I)

    @staticmethod
    def backward(ctx, dout):
        (gu,) = ctx.saved_tensors
        I = gu.shape[-1] // 2
        g2 = gu.reshape(-1, 2 * I)
        d2 = dout.reshape(-1, I).contiguous()
        dgu = torch.empty_like(g2)
        _lib.check(_L().ab2_swiglu_bwd(g2.data_ptr(), d2.data_ptr(), dgu.data_ptr(), g2.shape[0], I, _s()),
                   "ab2_swiglu_bwd")
        return dgu.view_as(gu)


def swiglu(gu):
    """``silu(gu[..., :I]) * gu[..., I:]``."""
    if not gu.is_cuda:
        return swiglu_ref(gu)
    return _SwiGLU.apply(gu.contiguous())


# ----------------------------------------------------------------------------- embedding
class _Embedding(torch.autograd.Function):
    @staticmethod
    def forward(ctx, ids, W):
        ctx.save_for_backward(ids)
        ctx.W = W
        T = ids.numel()
        V, H = W.shape
        out = torch.empty(T, H, device=W.device, dtype=W.dtype)
        _lib.check(_L().ab2_embed_fwd(W.data_ptr(), ids.data_ptr(), out.data_ptr(), T, H, V, _s()), "ab2_embed_fwd")
        return out.view(*ids.shape, H)

    @staticmethod
    def backward(ctx, dy):
        (ids,) = ctx.saved_tensors
        W = ctx.W
        V, H = W.shape
        d2 = dy.reshape(-1, H).contiguous()
        mg = getattr(W, "main_grad", None)
        dW = mg if mg is not None else torch.zeros(V, H, device=W.device, dtype=torch.float32)
        _lib.check(_L().ab2_embed_bwd(d2.data_ptr(), ids.data_ptr(), dW.data_ptr(), d2.shape[0], H, V, _s()),
                   "ab2_embed_bwd")
        return None, (None if mg is not None else dW.to(W.dtype))


def embedding(ids, W):
    if not W.is_cuda:
        return F.embedding(ids.long(), W)
    return _Embedding.apply(ids.to(torch.int32).contiguous(), W)


# ----------------------------------------------------------------------------- attention
# --------------------------------------------------------------------------- fp8 (e4m3) GEMM
FP8_MAX = 448.0
FP8_ROW, FP8_BLOCK_1x128, FP8_BLOCK_128x128 = 0, 1, 2


def quant_fp8_ref(x: torch.Tensor, mode: int, pow2: bool = False):
    """Plain PyTorch statement of :func:`quant_fp8` (any device): returns (e4m3 tensor, fp32 scales)."""
    R, K = x.shape
    xf = x.float()
    kb = (K + 127) // 128
    if mode == FP8_ROW:
        amax = xf.abs().amax(1)
    elif mode == FP8_BLOCK_1x128:
        pad = torch.zeros(R, kb * 128, device=x.device)
        pad[:, :K] = xf.abs()
        amax = pad.view(R, kb, 128).amax(-1).t().contiguous()              # [kb, R]
    else:
        rb = (R + 127) // 128
        pad = torch.zeros(rb * 128, kb * 128, device=x.device)
        pad[:R, :K] = xf.abs()
        amax = pad.view(rb, 128, kb, 128).amax((1, 3))                      # [rb, kb]
    s = amax.clamp(min=1e-12) / FP8_MAX
    if pow2:
        s = torch.exp2(torch.ceil(torch.log2(s)))
    if mode == FP8_ROW:
        full = s[:, None]
    elif mode == FP8_BLOCK_1x128:
        full = s.t().repeat_interleave(128, dim=1)[:, :K]
    else:
        full = s.repeat_interleave(128, 0).repeat_interleave(128, 1)[:R, :K]
    q = (xf / full).clamp(-FP8_MAX, FP8_MAX).to(torch.float8_e4m3fn)
    return q, s.float()


def quant_fp8(x: torch.Tensor, mode: int = FP8_BLOCK_1x128, pow2: bool = False):
    """bf16 ``[R, K]`` -> (e4m3 ``[R, K]``, fp32 scales). ``mode``: ``FP8_ROW`` one scale per row
    (``[R]``); ``FP8_BLOCK_1x128`` one per row and 128-wide K block (``[ceil(K/128), R]``, the
    activation layout); ``FP8_BLOCK_128x128`` one per 128 x 128 block (``[ceil(R/128), ceil(K/128)]``,
    the weight layout). ``x = q * scale`` up to rounding; ``pow2`` rounds scales up to powers of two."""
    if not x.is_cuda:
        return quant_fp8_ref(x, mode, pow2)
    R, K = x.shape
    assert x.dtype == torch.bfloat16 and x.stride(1) == 1
    q = torch.empty(R, K, dtype=torch.float8_e4m3fn, device=x.device)
    kb = (K + 127) // 128
    shape = (R,) if mode == FP8_ROW else ((kb, R) if mode == FP8_BLOCK_1x128 else ((R + 127) // 128, kb))
    s = torch.empty(shape, dtype=torch.float32, device=x.device)
    rc = _L().ab2_quant_fp8(x.data_ptr(), q.data_ptr(), s.data_ptr(), R, K, x.stride(0), q.stride(0), mode, int(pow2), _s())
    _lib.check(rc, "ab2_quant_fp8")
    return q, s


def dequant_fp8(q: torch.Tensor, s: torch.Tensor, mode: int) -> torch.Tensor:
    R, K = q.shape
    if mode == FP8_ROW:
        full = s[:, None]
    elif mode == FP8_BLOCK_1x128:
        full = s.t().repeat_interleave(128, dim=1)[:, :K]
    else:
        full = s.repeat_interleave(128, 0).repeat_interleave(128, 1)[:R, :K]
    return q.float() * full


def gemm_fp8(a_q: torch.Tensor, a_s: torch.Tensor, b_q: torch.Tensor, b_s: torch.Tensor, block_scaled: bool = True,
             out_dtype=torch.bfloat16) -> torch.Tensor:
    """``[M, K] x [N, K]^T`` on e4m3 operands with fp32 accumulation. Block-scaled: ``a_s``
    ``[ceil(K/128), M]`` and ``b_s`` ``[ceil(N/128), ceil(K/128)]``; otherwise row scales ``[M]`` / ``[N]``."""
    M, K = a_q.shape
    N = b_q.shape[0]
    if not a_q.is_cuda:
        am = FP8_BLOCK_1x128 if block_scaled else FP8_ROW
        bm = FP8_BLOCK_128x128 if block_scaled else FP8_ROW
        return (dequant_fp8(a_q, a_s, am) @ dequant_fp8(b_q, b_s, bm).t()).to(out_dtype)
    assert a_q.stride(1) == 1 and b_q.stride(1) == 1 and a_s.is_contiguous() and b_s.is_contiguous()
    c = torch.empty(M, N, dtype=out_dtype, device=a_q.device)
    rc = _L().ab2_gemm_fp8(a_q.data_ptr(), b_q.data_ptr(), c.data_ptr(), a_s.data_ptr(), b_s.data_ptr(), M, N, K, a_q.stride(0),
                           b_q.stride(0), c.stride(0), int(block_scaled), int(out_dtype == torch.float32), _s())
    _lib.check(rc, "ab2_gemm_fp8")
    return c


class _Fp8Linear(torch.autograd.Function):
    """``y = x @ W^T`` with block-scaled fp8 operands in the forward and in the input gradient
    (activations 1 x 128, weights 128 x 128 blocks, scales recomputed from the current values);
    the weight gradient stays in bf16 / fp32 (it accumulates over micro-batches)."""

    @staticmethod
    def forward(ctx, x, w):
        xq, xs = quant_fp8(x.contiguous(), FP8_BLOCK_1x128)
        wq, ws = quant_fp8(w, FP8_BLOCK_128x128)
        ctx.save_for_backward(x, w)
        return gemm_fp8(xq, xs, wq, ws, True, x.dtype)

    @staticmethod
    def backward(ctx, dy):
        x, w = ctx.saved_tensors
        dy = dy.contiguous()
        dx = None
        if ctx.needs_input_grad[0]:
            # dx = dy @ W: contraction over the output features, so W is needed K-major in that dimension
            dq, ds = quant_fp8(dy, FP8_BLOCK_1x128)
            wtq, wts = quant_fp8(w.t().contiguous(), FP8_BLOCK_128x128)
            dx = gemm_fp8(dq, ds, wtq, wts, True, x.dtype)
        dw = None
        if ctx.needs_input_grad[1]:
            mg = getattr(w, "main_grad", None)
            if mg is not None and x.is_cuda:
                gemm(dy, x, a_mn=True, b_mn=True, out=mg, epi=EPI_F32_ACC)
            else:
                dw = (dy.float().t() @ x.float()).to(w.dtype)
        return dx, dw


def fp8_linear(x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    return _Fp8Linear.apply(x, w)


def attention_ref(q, k, v, cu_seqlens, causal=True, scale=None):
    """Packed varlen attention, fp32 math. q: [T,Hq,D], k/v: [T,Hkv,D]. Returns (o, lse[Hq,T])."""
    T, Hq, D = q.shape
    Hkv = k.shape[1]
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    o = torch.zeros_like(q, dtype=torch.float32)
    lse = torch.zeros(Hq, T, dtype=torch.float32, device=q.device)
    cu = cu_seqlens.tolist()
    rep = Hq // Hkv
    for i in range(len(cu) - 1):
        a, b = cu[i], cu[i + 1]
        if b <= a:
            continue
        qi = q[a:b].float().transpose(0, 1)  # [Hq, L, D]
        ki = k[a:b].float().transpose(0, 1).repeat_interleave(rep, dim=0)
        vi = v[a:b].float().transpose(0, 1).repeat_interleave(rep, dim=0)
        s = qi @ ki.transpose(1, 2) * scale
        if causal:
            L = b - a
            mask = torch.ones(L, L, dtype=torch.bool, device=q.device).tril()
            s = s.masked_fill(~mask, float("-inf"))
        lse[:, a:b] = torch.logsumexp(s, dim=-1)
        o[a:b] = (torch.softmax(s, dim=-1) @ vi).transpose(0, 1)
    return o.to(q.dtype), lse


def attn_tile_table(cu_seqlens: torch.Tensor, total_tokens: int, tile: int = 128) -> torch.Tensor:
    """Device-side (sync-free) table ``[n,2]`` of (sequence index | -1, query block) for the
    attention kernels; ``n = ceil(T/tile) + num_seqs`` is an upper bound on the tile count."""
    B = cu_seqlens.numel() - 1
    n = (total_tokens + tile - 1) // tile + B
    lens = (cu_seqlens[1:] - cu_seqlens[:-1]).to(torch.int64)
    blocks = (lens + tile - 1) // tile
    ends = torch.cumsum(blocks, 0)
    starts = ends - blocks
    idx = torch.arange(n, device=cu_seqlens.device)
    seq = torch.searchsorted(ends, idx, right=True)
    valid = seq < B
    seqc = seq.clamp(max=B - 1)
    qb = idx - starts[seqc]
    # heaviest (latest) query blocks first: better tail behaviour under causal masking
    info = torch.stack([torch.where(valid, seqc, torch.full_like(seqc, -1)), qb], dim=1)
    order = torch.argsort(torch.where(valid, qb, torch.full_like(qb, -1)), descending=True, stable=True)
    return info[order].to(torch.int32).contiguous()


def attention_fwd(q, k, v, cu_seqlens, causal=True, scale=None, tile_info=None, out=None):
    """Kernel forward; returns (o, lse). q/k/v may be strided slices of a fused projection."""
    T, Hq, D = q.shape
    Hkv = k.shape[1]
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    if not q.is_cuda:
        return attention_ref(q, k, v, cu_seqlens, causal, scale)
    for t in (q, k, v):
        assert t.stride(2) == 1 and t.stride(1) == D and t.dtype == torch.bfloat16
    if tile_info is None:
        tile_info = attn_tile_table(cu_seqlens, T)
    o = out if out is not None else torch.empty(T, Hq, D, device=q.device, dtype=q.dtype)
    lse = torch.empty(Hq, T, device=q.device, dtype=torch.float32)
    cu = cu_seqlens.to(torch.int32)
    rc = _L().ab2_attn_fwd(q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), lse.data_ptr(), cu.data_ptr(),
                           tile_info.data_ptr(), tile_info.shape[0], T, Hq, Hkv, D, q.stride(0), k.stride(0),
                           v.stride(0), o.stride(0), scale, int(causal), _s())
    _lib.check(rc, "ab2_attn_fwd")
    return o, lse


def attention_bwd_ref(q, k, v, o, lse, do, cu_seqlens, causal, scale):
    """Reference backward (recomputes probabilities from lse), fp32 math, per sequence."""
    T, Hq, D = q.shape
    Hkv = k.shape[1]
    rep = Hq // Hkv
    dq = torch.zeros_like(q, dtype=torch.float32)
    dk = torch.zeros_like(k, dtype=torch.float32)
    dv = torch.zeros_like(v, dtype=torch.float32)
    cu = cu_seqlens.tolist()
    for i in range(len(cu) - 1):
        a, b = cu[i], cu[i + 1]
        if b <= a:
            continue
        L = b - a
        qi = q[a:b].float().transpose(0, 1)
        ki = k[a:b].float().transpose(0, 1).repeat_interleave(rep, dim=0)
        vi = v[a:b].float().transpose(0, 1).repeat_interleave(rep, dim=0)
        doi = do[a:b].float().transpose(0, 1)
        oi = o[a:b].float().transpose(0, 1)
        s = qi @ ki.transpose(1, 2) * scale
        if causal:
            mask = torch.ones(L, L, dtype=torch.bool, device=q.device).tril()
            s = s.masked_fill(~mask, float("-inf"))
        p = torch.exp(s - lse[:, a:b].unsqueeze(-1))
        dvi = p.transpose(1, 2) @ doi
        dp = doi @ vi.transpose(1, 2)
        delta = (doi * oi).sum(-1, keepdim=True)
        ds = p * (dp - delta) * scale
        dq[a:b] = (ds @ ki).transpose(0, 1)
        dki = ds.transpose(1, 2) @ qi
        dk[a:b] = dki.view(Hkv, rep, L, D).sum(1).transpose(0, 1)
        dv[a:b] = dvi.view(Hkv, rep, L, D).sum(1).transpose(0, 1)
    return dq.to(q.dtype), dk.to(k.dtype), dv.to(v.dtype)


def attention_bwd_into(q, k, v, o, lse, do, cu_seqlens, causal, scale, tile_info, dk, dv):
    """Kernel backward writing dk / dv into caller-provided (possibly strided) ``[T, Hkv, D]``
    views; returns the fp32 dq reduction buffer ``[T, Hq, D]``."""
    T, Hq, D = q.shape
    Hkv = k.shape[1]
    for t in (q, k, v, o, do, dk, dv):
        assert t.stride(2) == 1 and t.stride(1) == D and t.dtype == torch.bfloat16
    if tile_info is None:
        tile_info = attn_tile_table(cu_seqlens, T)
    # heaviest key blocks (most query blocks to visit under causal masking) first
    tiles_bwd = tile_info.flip(0).contiguous()
    cu = cu_seqlens.to(torch.int32)
    delta = torch.empty(Hq, T, device=q.device, dtype=torch.float32)
    _lib.check(_L().ab2_attn_delta(o.data_ptr(), do.data_ptr(), delta.data_ptr(), T, Hq, D, o.stride(0), do.stride(0), _s()),
               "ab2_attn_delta")
    dq32 = torch.zeros(T, Hq, D, device=q.device, dtype=torch.float32)
    rc = _L().ab2_attn_bwd(q.data_ptr(), k.data_ptr(), v.data_ptr(), do.data_ptr(), lse.data_ptr(), delta.data_ptr(),
                           dq32.data_ptr(), dk.data_ptr(), dv.data_ptr(), cu.data_ptr(), tiles_bwd.data_ptr(),
                           tiles_bwd.shape[0], T, Hq, Hkv, D, q.stride(0), k.stride(0), v.stride(0), do.stride(0),
                           dk.stride(0), dv.stride(0), scale, int(causal), _s())
    _lib.check(rc, "ab2_attn_bwd")
    return dq32


def attention_bwd(q, k, v, o, lse, do, cu_seqlens, causal, scale, tile_info=None):
    """Kernel backward: returns (dq, dk, dv) in the dtype of q. ``lse``: [Hq, T] from the forward."""
    T, Hq, D = q.shape
    Hkv = k.shape[1]
    for t in (q, k, v, o, do):
        assert t.stride(2) == 1 and t.stride(1) == D and t.dtype == torch.bfloat16
    if tile_info is None:
        tile_info = attn_tile_table(cu_seqlens, T)
    # heaviest key blocks (most query blocks to visit under causal masking) first
    tiles_bwd = tile_info.flip(0).contiguous()
    cu = cu_seqlens.to(torch.int32)
    delta = torch.empty(Hq, T, device=q.device, dtype=torch.float32)
    _lib.check(_L().ab2_attn_delta(o.data_ptr(), do.data_ptr(), delta.data_ptr(), T, Hq, D, o.stride(0), do.stride(0), _s()),
               "ab2_attn_delta")
    dq32 = torch.zeros(T, Hq, D, device=q.device, dtype=torch.float32)
    # every token of the packed batch belongs to one key block, so dk / dv are fully written
    dk = torch.empty(T, Hkv, D, device=q.device, dtype=q.dtype)
    dv = torch.empty(T, Hkv, D, device=q.device, dtype=q.dtype)
    rc = _L().ab2_attn_bwd(q.data_ptr(), k.data_ptr(), v.data_ptr(), do.data_ptr(), lse.data_ptr(), delta.data_ptr(),
                           dq32.data_ptr(), dk.data_ptr(), dv.data_ptr(), cu.data_ptr(), tiles_bwd.data_ptr(),
                           tiles_bwd.shape[0], T, Hq, Hkv, D, q.stride(0), k.stride(0), v.stride(0), do.stride(0),
                           dk.stride(0), dv.stride(0), scale, int(causal), _s())
    _lib.check(rc, "ab2_attn_bwd")
    return dq32.to(q.dtype), dk, dv


_ATTN_BWD_IMPL = attention_bwd  # set to None to fall back to the fp32 reference backward


class _Attention(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, cu_seqlens, causal, scale, tile_info):
        o, lse = attention_fwd(q, k, v, cu_seqlens, causal, scale, tile_info)
        ctx.save_for_backward(q, k, v, o, lse, cu_seqlens)
        ctx.causal, ctx.scale, ctx.tile_info = causal, scale, tile_info
        return o

    @staticmethod
    def backward(ctx, do):
        q, k, v, o, lse, cu = ctx.saved_tensors
        do = do.contiguous()
        if not o.is_contiguous():
            o = o.contiguous()
        if _ATTN_BWD_IMPL is not None:
            dq, dk, dv = _ATTN_BWD_IMPL(q, k, v, o, lse, do, cu, ctx.causal, ctx.scale, ctx.tile_info)
        else:
            dq, dk, dv = attention_bwd_ref(q, k, v, o, lse, do, cu, ctx.causal, ctx.scale)
        return dq, dk, dv, None, None, None, None


def attention(q, k, v, cu_seqlens, causal=True, scale=None, tile_info=None):
    """Differentiable packed varlen attention. q: [T,Hq,D]; k,v: [T,Hkv,D]."""
    D = q.shape[-1]
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    if not q.is_cuda:
        # autograd through the reference math
        T, Hq, _ = q.shape
        Hkv = k.shape[1]
        rep = Hq // Hkv
        outs = []
        cu = cu_seqlens.tolist()
        for i in range(len(cu) - 1):
            a, b = cu[i], cu[i + 1]
            if b <= a:
                continue
            qi = q[a:b].transpose(0, 1)
            ki = k[a:b].transpose(0, 1).repeat_interleave(rep, dim=0)
            vi = v[a:b].transpose(0, 1).repeat_interleave(rep, dim=0)
            oi = F.scaled_dot_product_attention(qi[None], ki[None], vi[None], is_causal=causal, scale=scale)[0]
            outs.append(oi.transpose(0, 1))
        return torch.cat(outs, dim=0) if outs else torch.zeros_like(q)
    return _Attention.apply(q, k, v, cu_seqlens, causal, scale, tile_info)


# ----------------------------------------------------------------------------- fused attention block
def qknorm_rope_fwd(qkv: torch.Tensor, wq, wk, pos, cos, sin, nq: int, nkv: int, D: int, eps: float):
    """q/k heads of a fused projection -> normalised (optional) and rotated ``[T, nq+nkv, D]``
    plus the per-row rstd (``None`` without norm). No autograd."""
    T = qkv.shape[0]
    assert qkv.stride(1) == 1 and qkv.dtype == torch.bfloat16
    qk = torch.empty(T, nq + nkv, D, device=qkv.device, dtype=qkv.dtype)
    rstd = torch.empty(T * (nq + nkv), device=qkv.device, dtype=torch.float32) if wq is not None else None
    rc = _L().ab2_qknorm_rope_fwd(qkv.data_ptr(), _lib.ptr(wq), _lib.ptr(wk), pos.data_ptr(), cos.data_ptr(), sin.data_ptr(),
                                  qk.data_ptr(), _lib.ptr(rstd), T, nq, nkv, D, qkv.stride(0), eps, _s())
    _lib.check(rc, "ab2_qknorm_rope_fwd")
    return qk, rstd


class _QKNormRopeAttention(torch.autograd.Function):
    """QK-norm + RoPE + varlen causal attention on a fused QKV projection: the forward reads q/k
    heads straight from the projection output and v through its row stride; the backward has
    the attention kernel write dk / dv into the projection-gradient buffer and finishes dq / dk
    in place (inverse rotation + norm backward), so no slice, copy or zero-fill op runs."""

    @staticmethod
    def forward(ctx, qkv, wq, wk, pos, cos, sin, cu_seqlens, scale, tile_info, nq, nkv, D, eps):
        T = qkv.shape[0]
        qk, rstd = qknorm_rope_fwd(qkv, wq, wk, pos, cos, sin, nq, nkv, D, eps)
        q, k = qk[:, :nq], qk[:, nq:]
        v = qkv[:, (nq + nkv) * D:].view(T, nkv, D)
        o, lse = attention_fwd(q, k, v, cu_seqlens, True, scale, tile_info)
        ctx.save_for_backward(qkv, qk, rstd, o, lse, wq, wk, pos, cos, sin, cu_seqlens)
        ctx.meta = (scale, tile_info, nq, nkv, D)
        return o

    @staticmethod
    def backward(ctx, do):
        qkv, qk, rstd, o, lse, wq, wk, pos, cos, sin, cu = ctx.saved_tensors
        scale, tile_info, nq, nkv, D = ctx.meta
        T = qkv.shape[0]
        do = do.contiguous()
        dqkv = torch.empty(T, (nq + 2 * nkv) * D, device=qkv.device, dtype=qkv.dtype)
        dk = dqkv[:, nq * D:(nq + nkv) * D].view(T, nkv, D)
        dv = dqkv[:, (nq + nkv) * D:].view(T, nkv, D)
        v = qkv[:, (nq + nkv) * D:].view(T, nkv, D)
        dq32 = attention_bwd_into(qk[:, :nq], qk[:, nq:], v, o, lse, do, cu, True, scale, tile_info, dk, dv)
        dwq = dwk = None
        ret_q = ret_k = None
        if wq is not None:
            mq, mk = getattr(wq, "main_grad", None), getattr(wk, "main_grad", None)
            dwq = mq if mq is not None else torch.zeros(D, device=qkv.device, dtype=torch.float32)
            dwk = mk if mk is not None else torch.zeros(D, device=qkv.device, dtype=torch.float32)
        rc = _L().ab2_qknorm_rope_bwd(qkv.data_ptr(), _lib.ptr(wq), _lib.ptr(wk), pos.data_ptr(), cos.data_ptr(), sin.data_ptr(),
                                      _lib.ptr(rstd), dq32.data_ptr(), dqkv.data_ptr(), _lib.ptr(dwq), _lib.ptr(dwk), T, nq, nkv,
                                      D, qkv.stride(0), dqkv.stride(0), _s())
        _lib.check(rc, "ab2_qknorm_rope_bwd")
        if wq is not None:
            ret_q = None if getattr(wq, "main_grad", None) is not None else dwq.to(wq.dtype)
            ret_k = None if getattr(wk, "main_grad", None) is not None else dwk.to(wk.dtype)
        return dqkv, ret_q, ret_k, None, None, None, None, None, None, None, None, None, None


def qknorm_rope_attention(qkv, wq, wk, pos, cos, sin, cu_seqlens, nq: int, nkv: int, D: int, eps: float, scale=None,
                          tile_info=None):
    """``attention(rope(norm(q)), rope(norm(k)), v)`` for ``qkv = [q heads | k heads | v heads]``
    (``[T, (nq + 2 nkv) D]``). CUDA: fused kernels; CPU: the unfused reference ops."""
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    T = qkv.shape[0]
    if qkv.is_cuda and D in (64, 128):
        return _QKNormRopeAttention.apply(qkv, wq, wk, pos, cos, sin, cu_seqlens, scale, tile_info, nq, nkv, D, eps)
    q = qkv[:, : nq * D].view(T, nq, D)
    k = qkv[:, nq * D: (nq + nkv) * D].view(T, nkv, D)
    v = qkv[:, (nq + nkv) * D:].view(T, nkv, D)
    if wq is not None:
        q = rmsnorm(q.reshape(T * nq, D), wq, eps)[0].view(T, nq, D)
        k = rmsnorm(k.reshape(T * nkv, D), wk, eps)[0].view(T, nkv, D)
    q, k = rope(q, pos, cos, sin), rope(k, pos, cos, sin)
    return attention(q, k.contiguous(), v.contiguous(), cu_seqlens, True, scale, tile_info)


# ----------------------------------------------------------------------------- logprob / entropy
def logprob_entropy_ref(logits, labels, temperature=1.0):
    z = logits.float() / temperature
    lp = torch.log_softmax(z, dim=-1)
    logp = lp.gather(-1, labels.long().unsqueeze(-1)).squeeze(-1)
    ent = -(lp.exp() * lp).sum(-1)
    return logp, ent


def logprob_entropy_from_logits(logits: torch.Tensor, labels: torch.Tensor, temperature: float = 1.0):
    """(logp, entropy, lse) per row from fp32 logits; no autograd."""
    if not logits.is_cuda:
        logp, ent = logprob_entropy_ref(logits, labels, temperature)
        return logp, ent, torch.logsumexp(logits.float() / temperature, -1)
    assert logits.dtype == torch.float32 and logits.stride(1) == 1
    rows, V = logits.shape
    logp = torch.empty(rows, device=logits.device, dtype=torch.float32)
    ent = torch.empty_like(logp)
    lse = torch.empty_like(logp)
    lab = labels.to(torch.int32).contiguous()
    rc = _L().ab2_logprob_fwd(logits.data_ptr(), lab.data_ptr(), logp.data_ptr(), ent.data_ptr(), lse.data_ptr(), None,
                              rows, V, logits.stride(0), temperature, 0, 0, _s())
    _lib.check(rc, "ab2_logprob_fwd")
    return logp, ent, lse


class _LMHeadLogprob(torch.autograd.Function):
    """Chunked LM head + log-softmax gather + entropy without keeping ``[T, V]`` alive.

    Forward: per chunk of rows, logits = h @ W^T (fp32 out) -> per-row (logp, entropy, lse).
    Backward: logits are recomputed per chunk, turned in one pass into bf16 dlogits, and fed
    to the dgrad / wgrad GEMMs (wgrad accumulates in fp32)."""

    @staticmethod
    def forward(ctx, h, W, labels, temperature, chunk):
        T, H = h.shape
        V = W.shape[0]
        logp = torch.empty(T, device=h.device, dtype=torch.float32)
        ent = torch.empty_like(logp)
        lse = torch.empty_like(logp)
        lab = labels.to(torch.int32).contiguous()
        Vp = (V + 3) // 4 * 4
        buf = torch.empty(min(chunk, T), Vp, device=h.device, dtype=torch.float32)
        for a in range(0, T, chunk):
            b = min(T, a + chunk)
            lg = buf[: b - a, :V] if Vp == V else buf[: b - a]
            out = buf[: b - a].as_strided((b - a, V), (Vp, 1))
            gemm(h[a:b], W, out=out, epi=EPI_F32)
            rc = _L().ab2_logprob_fwd(out.data_ptr(), lab[a:b].data_ptr(), logp[a:b].data_ptr(), ent[a:b].data_ptr(),
                                      lse[a:b].data_ptr(), None, b - a, V, Vp, temperature, 0, 0, _s())
            _lib.check(rc, "ab2_logprob_fwd")
        ctx.save_for_backward(h, W, lab, lse, ent)
        ctx.temperature, ctx.chunk = temperature, chunk
        return logp, ent

    @staticmethod
    def backward(ctx, g_logp, g_ent):
        h, W, lab, lse, ent = ctx.saved_tensors
        T, H = h.shape
        V = W.shape[0]
        chunk = ctx.chunk
        Vp = (V + 7) // 8 * 8
        buf = torch.empty(min(chunk, T), Vp, device=h.device, dtype=torch.float32)
        dbuf = torch.zeros(min(chunk, T), Vp, device=h.device, dtype=torch.bfloat16)
        g_logp = g_logp.contiguous().float() if g_logp is not None else None
        g_ent = g_ent.contiguous().float() if g_ent is not None else None
        dh = torch.empty_like(h) if ctx.needs_input_grad[0] else None
        mg = getattr(W, "main_grad", None)
        dW = None
        if ctx.needs_input_grad[1]:
            dW = mg if mg is not None else torch.zeros(V, H, device=h.device, dtype=torch.float32)
        for a in range(0, T, chunk):
            b = min(T, a + chunk)
            n = b - a
            out = buf[:n].as_strided((n, V), (Vp, 1))
            gemm(h[a:b], W, out=out, epi=EPI_F32)
            dl = dbuf[:n].as_strided((n, V), (Vp, 1))
            rc = _L().ab2_logprob_bwd(out.data_ptr(), lab[a:b].data_ptr(), lse[a:b].data_ptr(), ent[a:b].data_ptr(),
                                      _lib.ptr(g_logp[a:b]) if g_logp is not None else None,
                                      _lib.ptr(g_ent[a:b]) if g_ent is not None else None, dl.data_ptr(), n, V, Vp,
                                      Vp, ctx.temperature, 0, _s())
            _lib.check(rc, "ab2_logprob_bwd")
            if dh is not None:
                gemm(dl, W, b_mn=True, out=dh[a:b])
            if dW is not None:
                gemm(dl, h[a:b], a_mn=True, b_mn=True, out=dW, epi=EPI_F32_ACC)
        if dW is not None and mg is None:
            dW = dW.to(W.dtype)
        elif mg is not None:
            dW = None
        return dh, dW, None, None, None


def lm_head_logprob(h: torch.Tensor, W: torch.Tensor, labels: torch.Tensor, temperature: float = 1.0,
                    chunk: int = 2048):
    """Per-token ``(logp[label], entropy)`` of ``softmax(h @ W^T / temperature)``.

    Mirrors the chunked ``gather_logprobs_entropy`` of the reference
    (areal/utils/functional/vocab_parallel.py:16-82) but folds the LM-head GEMM in, so the
    full ``[T, V]`` logits never exist."""
    if not h.is_cuda:
        outs_lp, outs_e = [], []
        for a in range(0, h.shape[0], chunk):
            lg = F.linear(h[a:a + chunk], W)
            lp, e = logprob_entropy_ref(lg, labels[a:a + chunk], temperature)
            outs_lp.append(lp)
            outs_e.append(e)
        return torch.cat(outs_lp), torch.cat(outs_e)
    return _LMHeadLogprob.apply(h.contiguous(), W, labels, float(temperature), int(chunk))


# ----------------------------------------------------------------------------- optimizer pieces
def sqnorm_accumulate_(x: torch.Tensor, state: torch.Tensor) -> None:
    """state[0] += sum(x^2) for a flat fp32 tensor (device-side, no sync)."""
    if not x.is_cuda:
        state[0] += x.float().pow(2).sum()
        return
    assert x.dtype == torch.float32 and x.is_contiguous()
    _lib.check(_L().ab2_sqnorm_f32(x.data_ptr(), x.numel(), state.data_ptr(), _s()), "ab2_sqnorm_f32")


def clip_coef_(state: torch.Tensor, max_norm: float, inv_scale: float = 1.0) -> None:
    """From state[0] = sum of squares: state[1] = grad multiplier, state[2] = finite flag,
    state[3] = norm."""
    if not state.is_cuda:
        norm = math.sqrt(float(state[0])) * inv_scale if math.isfinite(float(state[0])) else float("nan")
        finite = math.isfinite(norm)
        coef = inv_scale
        if max_norm > 0 and finite and norm > max_norm:
            coef = inv_scale * max_norm / (norm + 1e-6)
        state[1] = coef if finite else 0.0
        state[2] = 1.0 if finite else 0.0
        state[3] = norm
        return
    _lib.check(_L().ab2_clip_coef(state.data_ptr(), max_norm, inv_scale, _s()), "ab2_clip_coef")


def adamw_step_(p32, m, v, g, p_bf16, state, lr, beta1, beta2, eps, wd, step) -> None:
    """Fused decoupled-weight-decay Adam on flat buffers; reads the clip coefficient and the
    skip flag from ``state`` on the device; also refreshes the bf16 compute copy."""
    if not p32.is_cuda:
        coef = float(state[1]) if state is not None else 1.0
        go = (float(state[2]) != 0.0) if state is not None else True
        if not go:
            return
        gi = g.float() * coef
        m.mul_(beta1).add_(gi, alpha=1 - beta1)
        v.mul_(beta2).addcmul_(gi, gi, value=1 - beta2)
        bc1, bc2 = 1 - beta1 ** step, 1 - beta2 ** step
        p32.mul_(1 - lr * wd)
        p32.addcdiv_(m / bc1, (v / bc2).sqrt() + eps, value=-lr)
        if p_bf16 is not None:
            p_bf16.copy_(p32.to(p_bf16.dtype))
        return
    assert p32.is_contiguous() and m.is_contiguous() and v.is_contiguous() and g.is_contiguous()
    rc = _L().ab2_adamw(p32.data_ptr(), m.data_ptr(), v.data_ptr(), g.data_ptr(), int(g.dtype == torch.bfloat16),
                        _lib.ptr(p_bf16), _lib.ptr(state), p32.numel(), lr, beta1, beta2, eps, wd, int(step), _s())
    _lib.check(rc, "ab2_adamw")


# ----------------------------------------------------------------------------- RL losses
class _PPOTokenLoss(torch.autograd.Function):
    """``sum over kept tokens of the clipped surrogate / n_valid`` with the gradient taken from the
    same kernel pass (the loss is an elementwise function of the new log-probs)."""

    @staticmethod
    def forward(ctx, logp, prox, old, adv, mask, params_bytes, prox_is_logp):
        n = logp.numel()
        dev = logp.device
        dlogp = torch.empty(n, dtype=torch.float32, device=dev)
        loss_tok = torch.empty(n, dtype=torch.float32, device=dev)
        ratio = torch.empty(n, dtype=torch.float32, device=dev)
        behave_w = torch.empty(n, dtype=torch.float32, device=dev)
        flags = torch.empty(n, dtype=torch.uint8, device=dev)
        sums = torch.zeros(8, dtype=torch.float64, device=dev)
        rc = _L().ab2_ppo_token_loss(logp.data_ptr(), None if prox_is_logp else prox.data_ptr(), old.data_ptr(), adv.data_ptr(),
                                     mask.data_ptr(), n, params_bytes, dlogp.data_ptr(), loss_tok.data_ptr(), ratio.data_ptr(),
                                     behave_w.data_ptr(), flags.data_ptr(), sums.data_ptr(), _s())
        _lib.check(rc, "ab2_ppo_token_loss")
        denom = sums[1].clamp(min=1.0)
        ctx.save_for_backward(dlogp, denom)
        ctx.shape = logp.shape
        ctx.mark_non_differentiable(loss_tok, ratio, behave_w, flags, sums)
        return (sums[0] / denom).float(), loss_tok, ratio, behave_w, flags, sums

    @staticmethod
    def backward(ctx, g, *unused):
        dlogp, denom = ctx.saved_tensors
        return (dlogp * (g / denom).float()).view(ctx.shape), None, None, None, None, None, None


def ppo_token_loss(logp: torch.Tensor, prox: Optional[torch.Tensor], old: torch.Tensor, adv: torch.Tensor, mask: torch.Tensor,
                   eps_clip: float, eps_clip_higher: Optional[float] = None, c_clip: Optional[float] = None,
                   rs_action: int = 0, rs_metric: int = 0, rs_lower: Optional[float] = None, rs_upper: Optional[float] = None):
    """Token-level decoupled PPO loss with token-level rejection sampling in ONE kernel (CUDA, fp32
    inputs of identical shape; ``prox=None``: the proximal policy is the current one). Returns
    ``(loss, per_token_loss, ratio, behave_weight, flags, sums)``; ``flags`` bits: 1 clipped, 2 dual
    clipped, 4 behaviour weight > 0, 8 kept after rejection; ``sums`` (fp64): loss, valid, kept,
    filtered, clipped, dual clipped, behave tokens."""
    import struct

    assert logp.is_cuda and logp.dtype == torch.float32
    hi = eps_clip if eps_clip_higher is None else eps_clip_higher
    params = struct.pack("fffiiffiii", float(eps_clip), float(hi), float(c_clip or 0.0), int(rs_action), int(rs_metric),
                         float(rs_lower or 0.0), float(rs_upper or 0.0), int(rs_lower is not None), int(rs_upper is not None),
                         int(prox is None))
    f = lambda t: t.detach().to(torch.float32).contiguous().reshape(-1)
    m = mask.to(torch.uint8).contiguous().reshape(-1) if mask.dtype != torch.uint8 else mask.contiguous().reshape(-1)
    lp = logp.contiguous()
    out = _PPOTokenLoss.apply(lp.reshape(-1) if lp.dim() > 1 else lp, None if prox is None else f(prox), f(old), f(adv), m, params, prox is None)
    return out


def gae_scan(rewards: torch.Tensor, values: torch.Tensor, loss_mask: torch.Tensor, seq_no_eos_mask: torch.Tensor, discount: float,
             gae_lambda) -> tuple[torch.Tensor, torch.Tensor]:
    """Token-level GAE over ``[B, L]`` CUDA tensors: one thread per sequence walks its row backwards."""
    B, L = rewards.shape
    dev = rewards.device
    lam = gae_lambda.float().to(dev).contiguous() if torch.is_tensor(gae_lambda) else torch.full((B,), float(gae_lambda), device=dev)
    adv = torch.empty(B, L, dtype=torch.float32, device=dev)
    ret = torch.empty(B, L, dtype=torch.float32, device=dev)
    # converted copies stay referenced until the launch is queued (a freed block could be handed to the next conversion)
    r32, v32 = rewards.float().contiguous(), values.float().contiguous()
    m8, e8 = loss_mask.to(torch.uint8).contiguous(), seq_no_eos_mask.to(torch.uint8).contiguous()
    rc = _L().ab2_gae_scan(r32.data_ptr(), v32.data_ptr(), m8.data_ptr(), e8.data_ptr(), lam.data_ptr(), float(discount), B, L,
                           adv.data_ptr(), ret.data_ptr(), _s())
    _lib.check(rc, "ab2_gae_scan")
    return adv, ret
