"""Sharded engine checkpoints for recovery: every rank writes its own slice of the flat
parameter space (weights in compute dtype, fp32 master, Adam moments) as one safetensors file
plus a small JSON manifest; loading re-assembles by flat offsets, so a checkpoint can be read
back under the same sharding without any gather, and under ANOTHER data-parallel world size by
reading, from every saved shard, the part of its range that overlaps the new rank's range (tensor
offsets in the flat space do not depend on the world size; only the tail padding does). HF export is separate
(:mod:`areal_b200.models.hf_io`). Plays the role of the DCP checkpoints of the reference
(``areal/engine/fsdp_engine.py:1834-1881``)."""
from __future__ import annotations

import json
import os

import torch
import torch.distributed as dist


def save_sharded(engine, path: str, with_optim: bool = True) -> None:
    from safetensors.torch import save_file

    os.makedirs(path, exist_ok=True)
    st = engine.store
    r = max(engine.local_index, 0)
    tensors = {"param_shard": st.param_shard.detach().cpu().contiguous()}
    meta = dict(numel=st.numel, padded=st.padded, world_size=st.world_size, shard_range=list(st.shard_range),
                names=st.names, offsets=st.offsets, version=engine.get_version(), dtype=str(st.dtype))
    opt = engine.optimizer
    if with_optim and opt is not None:
        tensors.update(master=opt.master.cpu(), exp_avg=opt.exp_avg.cpu(), exp_avg_sq=opt.exp_avg_sq.cpu())
        meta.update(step_count=opt.step_count, sched_step=opt.sched_step)
    es, eo = getattr(engine, "expert_store", None), getattr(engine, "expert_optimizer", None)
    if es is not None:
        # expert parallelism: the experts' own flat space (sharded over the replicas of the same experts)
        tensors["expert_param_shard"] = es.param_shard.detach().cpu().contiguous()
        meta["expert"] = dict(padded=es.padded, world_size=es.world_size, shard_range=list(es.shard_range), names=es.names)
        if with_optim and eo is not None:
            tensors.update(expert_master=eo.master.cpu(), expert_exp_avg=eo.exp_avg.cpu(), expert_exp_avg_sq=eo.exp_avg_sq.cpu())
    save_file(tensors, os.path.join(path, f"shard-{r:05d}-of-{st.world_size:05d}.safetensors"))
    with open(os.path.join(path, f"shard-{r:05d}.json"), "w") as f:
        json.dump(meta, f)
    if r == 0 and engine.model_config is not None:
        engine.model_config.save_pretrained(path)
    if engine.cpu_group is not None:
        dist.barrier(group=engine.cpu_group)


def _load_resharded(engine, path: str, with_optim: bool) -> None:
    """The checkpoint was written by another number of data-parallel ranks: every rank fills its range of the flat
    space from the saved shards that overlap it."""
    import glob

    from safetensors.torch import load_file

    st = engine.store
    if getattr(engine, "expert_store", None) is not None:
        raise ValueError("an expert-parallel checkpoint must be reloaded under the layout that wrote it; export to HF instead")
    metas = []
    for fn in sorted(glob.glob(os.path.join(path, "shard-*.json"))):
        with open(fn) as f:
            metas.append((int(os.path.basename(fn)[6:11]), json.load(f)))
    if not metas:
        raise FileNotFoundError(f"no sharded checkpoint under {path}")
    m0 = metas[0][1]
    if m0["names"] != st.names or m0["offsets"] != st.offsets or m0["numel"] != st.numel:
        raise ValueError("sharded checkpoint holds another model or another model-parallel slice; export to HF and reload instead")
    if len(metas) != m0["world_size"]:
        raise ValueError(f"sharded checkpoint is incomplete: {len(metas)} of {m0['world_size']} shards")
    lo, hi = st.shard_range
    opt = engine.optimizer
    want_opt = with_optim and opt is not None
    st.param_shard.zero_()
    got_opt = True
    if want_opt:
        for t in (opt.master, opt.exp_avg, opt.exp_avg_sq):
            t.zero_()
    for r, meta in metas:
        a, b = meta["shard_range"]
        x, y = max(a, lo), min(b, hi)
        if x >= y:
            continue
        tensors = load_file(os.path.join(path, f"shard-{r:05d}-of-{meta['world_size']:05d}.safetensors"))
        st.param_shard[x - lo:y - lo].copy_(tensors["param_shard"][x - a:y - a].to(st.dtype))
        if want_opt and "master" in tensors:
            for name, dst in (("master", opt.master), ("exp_avg", opt.exp_avg), ("exp_avg_sq", opt.exp_avg_sq)):
                dst[x - lo:y - lo].copy_(tensors[name][x - a:y - a].to(dst.dtype))
        else:
            got_opt = False
    if st.world_size > 1 and st.flat_param is not None:         # (sharded parameters have no replicated copy to refresh)
        dist.all_gather_into_tensor(st.flat_param, st.param_shard.clone(), group=engine._shard_group)
    if opt is not None:
        if want_opt and got_opt:
            opt.step_count, opt.sched_step = int(m0.get("step_count", 0)), int(m0.get("sched_step", 0))
        else:
            opt.resync_master()
    engine.set_version(int(m0.get("version", 0)))


def load_sharded(engine, path: str, with_optim: bool = True) -> None:
    from safetensors.torch import load_file

    st = engine.store
    r = max(engine.local_index, 0)
    mine = os.path.join(path, f"shard-{r:05d}.json")
    if not os.path.exists(mine):
        return _load_resharded(engine, path, with_optim)          # more ranks now than wrote the checkpoint
    with open(mine) as f:
        meta = json.load(f)
    if meta["world_size"] != st.world_size or meta["padded"] != st.padded:
        return _load_resharded(engine, path, with_optim)
    tensors = load_file(os.path.join(path, f"shard-{r:05d}-of-{st.world_size:05d}.safetensors"))
    st.param_shard.copy_(tensors["param_shard"].to(st.dtype))
    if st.world_size > 1 and st.flat_param is not None:         # (sharded parameters have no replicated copy to refresh)
        dist.all_gather_into_tensor(st.flat_param, st.param_shard.clone(), group=engine._shard_group)
    opt = engine.optimizer
    if opt is not None:
        if with_optim and "master" in tensors:
            opt.master.copy_(tensors["master"])
            opt.exp_avg.copy_(tensors["exp_avg"])
            opt.exp_avg_sq.copy_(tensors["exp_avg_sq"])
            opt.step_count, opt.sched_step = int(meta.get("step_count", 0)), int(meta.get("sched_step", 0))
        else:
            opt.resync_master()
    es, eo = getattr(engine, "expert_store", None), getattr(engine, "expert_optimizer", None)
    if es is not None:
        em = meta.get("expert")
        if em is None or em["world_size"] != es.world_size or em["padded"] != es.padded:
            raise ValueError("sharded checkpoint has no matching expert-parallel section")
        es.param_shard.copy_(tensors["expert_param_shard"].to(es.dtype))
        if es.world_size > 1:
            dist.all_gather_into_tensor(es.flat_param, es.param_shard.clone(), group=engine._edp_group)
        if eo is not None:
            if with_optim and "expert_master" in tensors:
                eo.master.copy_(tensors["expert_master"])
                eo.exp_avg.copy_(tensors["expert_exp_avg"])
                eo.exp_avg_sq.copy_(tensors["expert_exp_avg_sq"])
                eo.step_count, eo.sched_step = int(meta.get("step_count", 0)), int(meta.get("sched_step", 0))
            else:
                eo.resync_master()
    engine.set_version(int(meta.get("version", 0)))
