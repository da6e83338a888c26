"""Trainer -> rollout weight push over NVLink peer memory.

Every trainer rank owns a contiguous shard of the flat bf16 parameter space. On an update it
writes exactly that shard into the parameter buffers of every rollout replica with one kernel
(:func:`ab2_push_copy`), so all trainer GPUs push concurrently, nothing is gathered to rank 0 and
no tensor is touched twice. For tensor-parallel rollout replicas the plan below cuts every
parameter into the row / column slices each TP rank owns; the whole plan (1-D and 2-D strided
copies, optionally cast to block-scaled e4m3 on the way) runs as ONE launch (:func:`ab2_push_plan`).

Compared with the reference's ``xccl`` path (``areal/engine/fsdp_engine.py:1596-1692``: full
``full_tensor()`` all-gather on every trainer rank, then per-tensor NCCL broadcast from rank 0
in 1 GiB buckets with an HTTP round-trip per bucket) the bytes crossing NVLink drop from
``(world-1)/world * P`` (gather) ``+ P`` per replica from one source port to ``P / n_train``
per trainer per replica, spread over all ports. The NCCL broadcast path is kept as
:class:`BroadcastWeightPusher` for baseline measurements.
"""
from __future__ import annotations

import time
from dataclasses import dataclass
from typing import Optional

import torch
import torch.distributed as dist

from ..api.io_struct import WeightUpdateMeta
from ..ops import lib as oplib
from ..utils import logging as alog
from .symm import ptr_array

logger = alog.getLogger("weight_push")


# --------------------------------------------------------------------------- reshard plan
@dataclass
class CopyOp:
    src_off: int        # element offset in the trainer's flat buffer
    dst_tp: int         # destination TP rank inside a replica
    dst_off: int        # element offset in that TP rank's flat buffer
    rows: int
    cols: int
    ld_src: int
    ld_dst: int

    @property
    def contiguous(self) -> bool:
        return self.rows == 1 or (self.cols == self.ld_src and self.cols == self.ld_dst)


def tp_layout_of(cfg, name: str, shape: tuple, tp: int):
    """How a native parameter is split for tensor-parallel inference.

    Returns a list (one entry per TP rank) of lists of ``(row0, row1, col0, col1)`` source
    blocks that are concatenated (along rows) into the rank-local tensor."""
    if tp == 1 or len(shape) == 1 and not name.endswith("qkv_bias"):
        return [[(0, shape[0], 0, shape[1] if len(shape) > 1 else 1)] for _ in range(tp)]
    D, nq, nkv = cfg.head_dim, cfg.num_heads, cfg.num_kv_heads
    R = shape[0]
    C = shape[1] if len(shape) > 1 else 1
    out = []
    for j in range(tp):
        if name.endswith("qkv_proj") or name.endswith("qkv_bias"):
            qr, kr = nq * D, nkv * D
            q0, q1 = j * qr // tp, (j + 1) * qr // tp
            k0, k1 = j * kr // tp, (j + 1) * kr // tp
            out.append([(q0, q1, 0, C), (qr + k0, qr + k1, 0, C), (qr + kr + k0, qr + kr + k1, 0, C)])
        elif name.endswith("gate_up_proj"):
            I = R // 2
            a, b = j * I // tp, (j + 1) * I // tp
            out.append([(a, b, 0, C), (I + a, I + b, 0, C)])
        elif name.endswith("o_proj") or name.endswith("down_proj"):
            a, b = j * C // tp, (j + 1) * C // tp
            out.append([(0, R, a, b)])
        else:       # norms, embeddings and the LM head are replicated on every TP rank (as in parallel.tp.shard_tensor)
            out.append([(0, R, 0, C)])
    return out


def build_push_plan(cfg, names, offsets, shapes, shard_range, tp: int, dst_offsets: list[dict]) -> list[CopyOp]:
    """Copy operations that move the part of ``[shard_range)`` of the trainer's flat buffer that
    each TP rank needs. ``dst_offsets[j][name]`` is the element offset of ``name`` in TP rank
    j's flat buffer."""
    lo, hi = shard_range
    ops: list[CopyOp] = []
    for name, off, shape in zip(names, offsets, shapes):
        numel = 1
        for s in shape:
            numel *= s
        if off + numel <= lo or off >= hi:
            continue
        C = shape[1] if len(shape) > 1 else 1
        if len(shape) > 2:  # stacked experts: treat as [E*rows, cols]
            C = shape[-1]
        R = numel // C
        layout = tp_layout_of(cfg, name, (R, C), tp) if len(shape) <= 2 else [[(0, R, 0, C)] for _ in range(tp)]
        for j, blocks in enumerate(layout):
            drow = 0
            ldd = None
            for (r0, r1, c0, c1) in blocks:
                w = c1 - c0
                ldd = w
                # rows of this block that intersect the shard (a row is cut at most at its ends)
                for r in _row_segments(off, C, r0, r1, c0, c1, lo, hi):
                    (ra, rb, ca, cb) = r
                    src = off + ra * C + ca
                    dst = dst_offsets[j][name] + (drow + ra - r0) * w + (ca - c0)
                    ops.append(CopyOp(src, j, dst, rb - ra, cb - ca, C, w))
                drow += r1 - r0
    return ops


def _row_segments(off, C, r0, r1, c0, c1, lo, hi):
    """Splits block rows [r0,r1) x cols [c0,c1) of a tensor at flat offset ``off`` (row width
    ``C``) into pieces fully inside the flat range [lo, hi): at most one partial row before and
    one after a run of full rows. Returns ``(row_a, row_b, col_a, col_b)`` tuples."""
    def ceil_div(a, b):
        return -((-a) // b)

    full_a = max(r0, ceil_div(lo - off - c0, C))
    full_b = min(r1, (hi - off - c1) // C + 1)
    out = []
    cand = set()
    if full_a < full_b:
        cand.update((full_a - 1, full_b))
    else:
        base = max(r0, (max(lo, off) - off) // C - 1)
        cand.update(range(base, min(r1, base + 4)))
    pre, post = [], []
    for r in sorted(cand):
        if r < r0 or r >= r1 or (full_a < full_b and full_a <= r < full_b):
            continue
        a, b = max(off + r * C + c0, lo), min(off + r * C + c1, hi)
        if a < b:
            seg = (r, r + 1, a - off - r * C, b - off - r * C)
            (pre if (full_a >= full_b or r < full_a) else post).append(seg)
    out += pre
    if full_a < full_b:
        out.append((full_a, full_b, c0, c1))
    out += post
    return out


class TPPushPlan:
    """A re-shard plan in device memory, executed by ONE launch of ``ab2_push_plan`` per push: the
    op table (``CopyOp`` rows), the prefix sum of the ops' work chunks and, per call, the table of
    destination buffers (replica-major: entry ``k * tp + j`` is TP rank ``j`` of replica ``k``)."""

    CHUNK = 4096          # 16-byte vectors per work item; must equal PLAN_CHUNK in ops/csrc/comm.cu

    def __init__(self, ops: list, tp: int, device):
        import numpy as np

        self.ops, self.tp, self.device = list(ops), tp, torch.device(device)
        rec = np.zeros(len(self.ops), dtype=[("src_off", "<i8"), ("dst_off", "<i8"), ("dst", "<i4"), ("rows", "<i4"), ("cols", "<i4"),
                                             ("ld_src", "<i4"), ("ld_dst", "<i4"), ("pad", "<i4")])
        starts, total = [], 0
        for i, op in enumerate(self.ops):
            if op.contiguous and op.rows * op.cols < 2 ** 31:      # one long row: 1-D tensors, whole row blocks
                op = self.ops[i] = CopyOp(op.src_off, op.dst_tp, op.dst_off, 1, op.rows * op.cols, op.rows * op.cols, op.rows * op.cols)
            if op.cols % 8 or op.src_off % 8 or op.dst_off % 8 or op.ld_src % 8 or op.ld_dst % 8:
                raise ValueError(f"re-shard op {op} is not 16-byte aligned")
            rec[i] = (op.src_off, op.dst_off, op.dst_tp, op.rows, op.cols, op.ld_src, op.ld_dst, 0)
            starts.append(total)
            total += -(-(op.rows * (op.cols // 8)) // self.CHUNK)
        self.total_chunks = total
        self.bytes = sum(op.rows * op.cols for op in self.ops) * 2
        if self.device.type == "cuda" and self.ops:
            self.d_ops = torch.from_numpy(rec.view(np.uint8).reshape(-1).copy()).to(self.device)
            self.d_starts = torch.tensor(starts, dtype=torch.int32, device=self.device)
        self._tables: dict = {}

    @classmethod
    def build(cls, cfg, store, tp: int, dst_offsets: list[dict], device=None) -> "TPPushPlan":
        """Plan for the shard of ``store`` (a trainer's :class:`FlatParamStore`)."""
        shapes = [tuple(p.shape) for p in store.params]
        ops = build_push_plan(cfg, store.names, store.offsets, shapes, store.shard_range, tp, dst_offsets)
        return cls(ops, tp, device if device is not None else store.device)

    def _table(self, ptrs: list[int]) -> torch.Tensor:
        key = tuple(ptrs)
        t = self._tables.get(key)
        if t is None:
            t = self._tables[key] = torch.tensor(list(ptrs), dtype=torch.int64, device=self.device)
        return t

    def run(self, src_flat: torch.Tensor, dst_ptrs: list[int], n_rep: int, scale_ptrs: Optional[list[int]] = None,
            pow2: bool = False) -> None:
        """Copies (``scale_ptrs`` given: casts to block-scaled e4m3) on the current stream."""
        if not self.ops:
            return
        assert len(dst_ptrs) == n_rep * self.tp
        if self.device.type != "cuda":
            raise RuntimeError("the plan kernel runs on CUDA; use apply_plan_reference on the CPU")
        tab = self._table(dst_ptrs)
        stab = self._table(scale_ptrs) if scale_ptrs is not None else None
        rc = oplib.get_lib().ab2_push_plan(src_flat.data_ptr(), self.d_ops.data_ptr(), len(self.ops), self.d_starts.data_ptr(),
                                           self.total_chunks, tab.data_ptr(), stab.data_ptr() if stab is not None else None, n_rep,
                                           self.tp, int(scale_ptrs is not None), int(pow2), oplib.stream_ptr())
        oplib.check(rc, "ab2_push_plan")


def apply_plan_reference(ops: list, src_flat: torch.Tensor, dst_flats: list[torch.Tensor]) -> None:
    """Plain PyTorch execution of a plan (CPU deployments and tests): ``dst_flats[j]`` is TP rank j's buffer."""
    for op in ops:
        src = torch.as_strided(src_flat, (op.rows, op.cols), (op.ld_src, 1), op.src_off)
        torch.as_strided(dst_flats[op.dst_tp], (op.rows, op.cols), (op.ld_dst, 1), op.dst_off).copy_(src)


def tp_dst_layout(model_cfg, tp: int, dtype=torch.bfloat16) -> list[dict]:
    """``{name: element offset}`` of every parameter in the flat buffer of a TP rank (identical for
    all ranks of a replica): the layout :class:`~areal_b200.engine.flat_params.FlatParamStore`
    gives a rank-local model, computed from shapes alone."""
    from ..engine.flat_params import flat_layout
    from ..models.decoder import build_model
    from . import tp as TP

    local = build_model(TP.local_config(model_cfg, tp), dtype=dtype, device="meta")
    names = [n for n, _ in local.named_parameters()]
    offs, _ = flat_layout([p.numel() for _, p in local.named_parameters()], 1)
    d = dict(zip(names, offs))
    return [d for _ in range(tp)]


# --------------------------------------------------------------------------- pushers
class TPWeightPusher:
    """Shard-direct push into tensor-parallel rollout replicas: every trainer rank re-shards ITS part
    of the flat parameter space into the row / column slices each TP rank owns and writes them over
    NVLink into every replica, all in one kernel launch (``ab2_push_plan``). Nothing is gathered on
    the trainer side and no rollout rank receives bytes it does not keep (except the replicated
    embeddings / norms, which every TP rank holds in full).

    The rollout ranks' flat buffers are symmetric allocations of the world group (same size as the
    trainer's); ``dst_layout[j]`` gives the element offset of each parameter inside TP rank j's buffer."""

    def __init__(self, train_engine, rollout_client, meta: WeightUpdateMeta, tp: int):
        self.train, self.client, self.meta, self.tp = train_engine, rollout_client, meta, tp
        self.bus, self.split = rollout_client.bus, rollout_client.split
        eng = train_engine
        if eng.store.flat_param.data_ptr() not in eng._symm_handles:
            raise RuntimeError("the trainer's parameter buffer is not in symmetric memory; cannot push peer to peer")
        layout = tp_dst_layout(eng.model_config, tp, eng.store.dtype)
        self.plan = TPPushPlan.build(eng.model_config, eng.store, tp, layout)
        # replica-major table: replica k occupies rollout ranks [k * tp, (k + 1) * tp)
        self.dst_ptrs = eng.peer_ptrs(eng.store.flat_param, self.split.rollout_ranks)
        self.n_rep = len(self.split.rollout_ranks) // tp
        self.seq = 0
        self.last_ms = self.last_dev_ms = self.last_gbps = 0.0

    def push(self, meta: Optional[WeightUpdateMeta] = None) -> float:
        meta = meta or self.meta
        eng = self.train
        head = eng.local_index == 0
        t0 = time.perf_counter()
        if head:
            self.bus.put(f"wu/{self.seq}/pause", 1)
        for r in self.split.rollout_ranks:
            self.bus.get(f"wu/{self.seq}/ack/{r}")
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        ev0.record()
        self.plan.run(eng.store.flat_param, self.dst_ptrs, self.n_rep)
        ev1.record()
        torch.cuda.current_stream().synchronize()
        dev_ms = ev0.elapsed_time(ev1)
        if eng.cpu_group is not None:
            dist.barrier(group=eng.cpu_group)
        if head:
            self.bus.put(f"wu/{self.seq}/done", {"version": meta.version if meta.version is not None else eng.get_version() + 1})
        self.seq += 1
        self.last_ms = (time.perf_counter() - t0) * 1e3
        self.last_dev_ms = dev_ms
        self.last_gbps = self.plan.bytes * self.n_rep / max(dev_ms, 1e-6) / 1e6
        return self.last_ms


class DistributedWeightPusher:
    """Shard-direct push from every trainer rank into every rollout rank (replicas with the
    trainer's flat layout; TP = 1)."""

    def __init__(self, train_engine, rollout_client, meta: WeightUpdateMeta):
        self.train, self.client, self.meta = train_engine, rollout_client, meta
        self.bus = rollout_client.bus
        self.split = rollout_client.split
        if train_engine.store.flat_param.data_ptr() not in train_engine._symm_handles:
            raise RuntimeError("the trainer's parameter buffer is not in symmetric memory; cannot push peer to peer")
        self.dst_ptrs = train_engine.peer_ptrs(train_engine.store.flat_param, self.split.rollout_ranks)
        self.seq = 0
        self.last_ms = 0.0
        self.last_gbps = 0.0

    def push(self, meta: Optional[WeightUpdateMeta] = None) -> float:
        meta = meta or self.meta
        eng = self.train
        head = eng.local_index == 0
        t0 = time.perf_counter()
        if head:
            self.bus.put(f"wu/{self.seq}/pause", 1)
        for r in self.split.rollout_ranks:
            self.bus.get(f"wu/{self.seq}/ack/{r}")
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        ev0.record()
        sh = eng.store.param_shard
        rc = oplib.get_lib().ab2_push_copy(sh.data_ptr(), ptr_array(self.dst_ptrs), len(self.dst_ptrs),
                                           eng.store.shard_range[0], sh.numel(), oplib.stream_ptr())
        oplib.check(rc, "ab2_push_copy")
        ev1.record()
        torch.cuda.current_stream().synchronize()
        dev_ms = ev0.elapsed_time(ev1)
        if eng.cpu_group is not None:
            dist.barrier(group=eng.cpu_group)
        if head:
            self.bus.put(f"wu/{self.seq}/done", {"version": meta.version if meta.version is not None else eng.get_version() + 1})
        self.seq += 1
        self.last_ms = (time.perf_counter() - t0) * 1e3
        self.last_dev_ms = dev_ms
        self.last_gbps = sh.numel() * 2 * len(self.dst_ptrs) / max(dev_ms, 1e-6) / 1e6
        return self.last_ms


class BroadcastWeightPusher:
    """Collective baseline: the trainer head broadcasts the whole flat parameter buffer to the
    rollout ranks in buckets (the data movement of the reference's xccl path, minus its HTTP
    round trips). Works on NCCL and on gloo (CPU deployments).

    Delta transfer (``actor.enable_delta_weight_update`` or ``weight_update_delta_method: exact``): after a
    small-learning-rate step most bf16 values keep their bit pattern, so from the second push on the head compares the
    buffer with a snapshot of what the receivers hold and, when fewer than a third of the elements changed, broadcasts
    only (index, value) pairs: 6 bytes per changed element instead of 2 per element. Every
    ``weight_update_anchor_interval``-th push (default 20) is a full one again. Reference:
    ``areal/v2/weight_update/awex/delta_detect.py``, the ``dte`` example (sparse deltas with periodic anchors)."""

    def __init__(self, train_engine, rollout_client, group, bucket_mb: int = 1024):
        self.train, self.client, self.group = train_engine, rollout_client, group
        self.bucket = bucket_mb * 1024 * 1024 // max(1, train_engine.store.flat_param.element_size())
        self.bus, self.split, self.seq = rollout_client.bus, rollout_client.split, 0
        self.last_ms = 0.0
        cfg = getattr(train_engine, "config", None)
        self.delta = bool(getattr(cfg, "enable_delta_weight_update", False)) or getattr(cfg, "weight_update_delta_method", "none") == "exact"
        self.anchor_every = int(getattr(cfg, "weight_update_anchor_interval", 0) or 20)
        self.snapshot: Optional[torch.Tensor] = None
        self.deltas_since_anchor = 0
        self.last_fraction = 1.0               # bytes sent / bytes of a full push

    def _sparse_update(self, flat: torch.Tensor):
        """(indices, values) of the elements whose bits differ from the receivers' copy, or ``None`` for a full push."""
        if not self.delta or self.snapshot is None or self.deltas_since_anchor >= self.anchor_every:
            return None
        view = {2: torch.int16, 4: torch.int32, 1: torch.int8}[flat.element_size()]
        idx = (flat.view(view) != self.snapshot.view(view)).nonzero().flatten()
        isz = 4 if flat.numel() < 2 ** 31 else 8
        if idx.numel() * (isz + flat.element_size()) >= flat.numel() * flat.element_size():
            return None                        # dense is cheaper
        return (idx.to(torch.int32) if isz == 4 else idx), flat[idx]

    def push(self, meta: Optional[WeightUpdateMeta] = None) -> float:
        eng = self.train
        head = eng.local_index <= 0
        t0 = time.perf_counter()
        src = self.split.train_ranks[0]
        flat = eng.store.flat_param
        sparse = self._sparse_update(flat) if head else None
        if head:
            cmd = {"mode": "broadcast", "bucket": self.bucket, "src": src}
            if sparse is not None:
                cmd.update(sparse=int(sparse[0].numel()), index_dtype=str(sparse[0].dtype).replace("torch.", ""))
            self.bus.put(f"wu/{self.seq}/pause", cmd)
        for r in self.split.rollout_ranks:
            self.bus.get(f"wu/{self.seq}/ack/{r}")
        if head:
            if sparse is not None:
                idx, vals = sparse
                for a in range(0, idx.numel(), self.bucket):
                    dist.broadcast(idx[a:a + self.bucket], src=src, group=self.group)
                    dist.broadcast(vals[a:a + self.bucket], src=src, group=self.group)
                self.snapshot[idx.long()] = vals
                self.deltas_since_anchor += 1
                self.last_fraction = idx.numel() * (idx.element_size() + vals.element_size()) / max(1, flat.numel() * flat.element_size())
            else:
                for a in range(0, flat.numel(), self.bucket):
                    dist.broadcast(flat[a:a + self.bucket], src=src, group=self.group)
                if self.delta:
                    self.snapshot = flat.detach().clone()
                    self.deltas_since_anchor = 0
                self.last_fraction = 1.0
            if flat.is_cuda:
                torch.cuda.current_stream().synchronize()
        if eng.cpu_group is not None:
            dist.barrier(group=eng.cpu_group)
        if head:
            version = meta.version if meta is not None and meta.version is not None else eng.get_version() + 1
            self.bus.put(f"wu/{self.seq}/done", {"version": version})
        self.seq += 1
        self.last_ms = (time.perf_counter() - t0) * 1e3
        return self.last_ms
