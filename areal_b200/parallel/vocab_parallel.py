"""Vocabulary-parallel LM head: every rank of a group holds ``V / P`` rows of the output
embedding and computes log-prob-of-label and entropy without any rank ever holding a full
``[T, V]`` logits row.

Forward per chunk of rows: local logits (fp32) -> per-row partial ``(max, sum exp, sum exp*z,
label logit)`` (``ab2_logprob_fwd`` in partial mode) -> ONE all-gather of the ``[rows, 4]``
partials -> combine (``ab2_logprob_combine``). Backward: local logits are recomputed, turned
into bf16 dlogits with the *global* lse / entropy (``ab2_logprob_bwd`` with the shard's vocab
offset), fed to the dgrad / wgrad GEMMs; the hidden-state gradient is summed over the group.
Reference: ``areal/utils/functional/vocab_parallel.py:120-195`` (2-4 all-reduces per chunk:
MAX, SUM(exp), SUM(target), SUM(exp*z)); here one gather of 16 bytes per row. With a
:class:`PartialsExchange` the gather is not a library collective either: every rank stores its
partials straight into every peer's slot (peer memory over NVLink), a flag barrier follows, and the
combine kernel reads the slots in place.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.distributed as dist

from ..ops import functional as OF
from ..ops import lib as oplib


def _partials_ref(z: torch.Tensor, labels: torch.Tensor, vocab_start: int) -> torch.Tensor:
    """[rows, 4] = (max, sumexp, sum exp*z, label z or 0) of a logits shard ``z`` (already / T)."""
    m = z.max(-1).values
    e = torch.exp(z - m[:, None])
    V = z.shape[1]
    loc = labels.long() - vocab_start
    inside = (loc >= 0) & (loc < V)
    tz = torch.where(inside, z.gather(1, loc.clamp(0, V - 1)[:, None])[:, 0], torch.zeros_like(m))
    return torch.stack([m, e.sum(-1), (e * z).sum(-1), tz], dim=1)


def combine_partials(parts: torch.Tensor):
    """parts: [P, rows, 4] -> (logp, entropy, lse)."""
    m = parts[:, :, 0].max(0).values
    scale = torch.exp(parts[:, :, 0] - m[None])
    s = (parts[:, :, 1] * scale).sum(0)
    sz = (parts[:, :, 2] * scale).sum(0)
    lse = m + torch.log(s)
    tz = parts[:, :, 3].sum(0)
    return tz - lse, lse - sz / s, lse


class PartialsExchange:
    """Peer-memory gather of the ``[rows, 4]`` partials of one chunk. Every rank owns a symmetric buffer of
    ``2 x P x max_rows x 4`` floats; ``gather`` stores this rank's partials into slot ``rank`` of the current half
    on every peer (one ``push_copy`` launch, 16-byte stores over NVLink), passes a bounded flag barrier and returns
    the local half ``[P, max_rows, 4]``. The halves alternate: a rank that runs ahead writes the other half while a
    slower peer still reads this one, and it cannot come back to this half before that peer has reached the next
    barrier, i.e. finished reading."""

    def __init__(self, group, device, max_rows: int = 4096):
        from .symm import SymmComm, ptr_array, symm_empty

        self.group = group
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        self.max_rows = int(max_rows)
        self.half = self.world * self.max_rows * 4
        self.buf, hdl = symm_empty(2 * self.half, torch.float32, device, group)
        self.buf.zero_()
        self.comm = SymmComm(group, device)
        self.ptrs = ptr_array(list(hdl.buffer_ptrs))
        self.parity = 0

    def gather(self, part: torch.Tensor) -> tuple[torch.Tensor, int]:
        """part: [n, 4] fp32 (n <= max_rows). Returns (slots [P, max_rows, 4] of this chunk, floats between ranks)."""
        n = part.shape[0]
        if n > self.max_rows:
            raise ValueError(f"chunk of {n} rows exceeds the exchange's {self.max_rows}")
        off = self.parity * self.half + self.rank * self.max_rows * 4          # in floats
        # the copy kernel moves 16-byte vectors of 2-byte elements: a float is two of them
        rc = oplib.get_lib().ab2_push_copy(part.contiguous().data_ptr(), self.ptrs, self.world, 2 * off, 2 * n * 4, oplib.stream_ptr())
        oplib.check(rc, "ab2_push_copy(partials)")
        self.comm.barrier(3)
        view = self.buf[self.parity * self.half:(self.parity + 1) * self.half].view(self.world, self.max_rows, 4)
        self.parity ^= 1
        return view, self.max_rows * 4


class _VocabParallelLogprob(torch.autograd.Function):
    @staticmethod
    def forward(ctx, h, W_shard, labels, temperature, chunk, group, vocab_start, exchange=None):
        T = h.shape[0]
        Vl = W_shard.shape[0]
        P = dist.get_world_size(group)
        cuda = h.is_cuda
        logp = torch.empty(T, device=h.device, dtype=torch.float32)
        ent, lse = torch.empty_like(logp), torch.empty_like(logp)
        lab = labels.to(torch.int32).contiguous()
        Vp = (Vl + 3) // 4 * 4
        L = oplib.get_lib() if cuda else None
        for a in range(0, T, chunk):
            b = min(T, a + chunk)
            n = b - a
            if cuda:
                buf = torch.empty(n, Vp, device=h.device, dtype=torch.float32)
                out = buf.as_strided((n, Vl), (Vp, 1))
                OF.gemm(h[a:b], W_shard, out=out, epi=OF.EPI_F32)
                part = torch.empty(n, 4, device=h.device, dtype=torch.float32)
                oplib.check(L.ab2_logprob_fwd(out.data_ptr(), lab[a:b].data_ptr(), None, None, None, part.data_ptr(), n, Vl, Vp,
                                              temperature, vocab_start, 1, oplib.stream_ptr()), "ab2_logprob_fwd(partial)")
            else:
                z = (h[a:b].float() @ W_shard.float().t()) / temperature
                part = _partials_ref(z, lab[a:b], vocab_start)
            stride = n * 4
            allp = None
            if cuda and exchange is not None:
                allp, stride = exchange.gather(part)
            elif cuda:
                allp = torch.empty(P, n, 4, device=h.device, dtype=torch.float32)
                dist.all_gather_into_tensor(allp.view(P * n, 4), part, group=group)
            else:
                gathered = [torch.empty_like(part) for _ in range(P)]
                dist.all_gather(gathered, part.contiguous(), group=group)
                allp = torch.stack(gathered)
            if cuda:
                oplib.check(L.ab2_logprob_combine(allp.data_ptr(), P, stride, logp[a:b].data_ptr(), ent[a:b].data_ptr(),
                                                  lse[a:b].data_ptr(), n, oplib.stream_ptr()), "ab2_logprob_combine")
            else:
                logp[a:b], ent[a:b], lse[a:b] = combine_partials(allp)
        ctx.save_for_backward(h, W_shard, lab, lse, ent)
        ctx.meta = (temperature, chunk, group, vocab_start)
        return logp, ent

    @staticmethod
    def backward(ctx, g_logp, g_ent):
        h, W, lab, lse, ent = ctx.saved_tensors
        temperature, chunk, group, vocab_start = ctx.meta
        T, H = h.shape
        Vl = W.shape[0]
        cuda = h.is_cuda
        g_logp = g_logp.contiguous().float() if g_logp is not None else torch.zeros(T, device=h.device)
        g_ent = g_ent.contiguous().float() if g_ent is not None else torch.zeros(T, device=h.device)
        dh = torch.zeros_like(h, dtype=torch.float32 if not cuda else h.dtype)
        mg = getattr(W, "main_grad", None)
        dW = mg if mg is not None else torch.zeros(Vl, H, device=h.device, dtype=torch.float32)
        Vp = (Vl + 7) // 8 * 8
        L = oplib.get_lib() if cuda else None
        for a in range(0, T, chunk):
            b = min(T, a + chunk)
            n = b - a
            if cuda:
                buf = torch.empty(n, Vp, device=h.device, dtype=torch.float32)
                out = buf.as_strided((n, Vl), (Vp, 1))
                OF.gemm(h[a:b], W, out=out, epi=OF.EPI_F32)
                dbuf = torch.zeros(n, Vp, device=h.device, dtype=torch.bfloat16)
                dl = dbuf.as_strided((n, Vl), (Vp, 1))
                oplib.check(L.ab2_logprob_bwd(out.data_ptr(), lab[a:b].data_ptr(), lse[a:b].data_ptr(), ent[a:b].data_ptr(),
                                              g_logp[a:b].data_ptr(), g_ent[a:b].data_ptr(), dl.data_ptr(), n, Vl, Vp, Vp, temperature,
                                              vocab_start, oplib.stream_ptr()), "ab2_logprob_bwd")
                OF.gemm(dl, W, b_mn=True, out=dh[a:b])
                OF.gemm(dl, h[a:b], a_mn=True, b_mn=True, out=dW, epi=OF.EPI_F32_ACC)
            else:
                z = (h[a:b].float() @ W.float().t()) / temperature
                p = torch.exp(z - lse[a:b, None])
                onehot = torch.zeros_like(z)
                loc = lab[a:b].long() - vocab_start
                inside = (loc >= 0) & (loc < Vl)
                onehot[torch.arange(n)[inside], loc[inside]] = 1.0
                logpj = z - lse[a:b, None]
                dz = (g_logp[a:b, None] * (onehot - p) - g_ent[a:b, None] * p * (logpj + ent[a:b, None])) / temperature
                dh[a:b] = dz @ W.float()
                dW += dz.t() @ h[a:b].float()
        dist.all_reduce(dh, group=group)                    # every shard contributes to d hidden
        dW_ret = None if mg is not None else dW.to(W.dtype)
        return dh.to(h.dtype), dW_ret, None, None, None, None, None, None


def vocab_parallel_lm_head_logprob(h: torch.Tensor, W_shard: torch.Tensor, labels: torch.Tensor, group, temperature: float = 1.0,
                                   chunk: int = 2048, vocab_start: Optional[int] = None, exchange: Optional[PartialsExchange] = None):
    """``(logp[label], entropy)`` of ``softmax(h @ W^T / temperature)`` with ``W`` split by rows
    over ``group`` (rank r holds rows ``[r * V/P, (r+1) * V/P)`` unless ``vocab_start`` says
    otherwise). ``h`` and ``labels`` are identical on every rank of the group."""
    if vocab_start is None:
        vocab_start = dist.get_rank(group) * W_shard.shape[0]
    if exchange is not None and chunk > exchange.max_rows:
        chunk = exchange.max_rows
    return _VocabParallelLogprob.apply(h, W_shard, labels, temperature, chunk, group, vocab_start, exchange)
