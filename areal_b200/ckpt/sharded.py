"""Sharded engine checkpoints for recovery: every rank writes its own slice of the flat
parameter space (weights in compute dtype, fp32 master, Adam moments) as one safetensors file
plus a small JSON manifest; loading re-assembles by flat offsets, so a checkpoint can be read
back under the same sharding without any gather. HF export is separate
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


def load_sharded(engine, path: str, with_optim: bool = True) -> None:
    from safetensors.torch import load_file

    st = engine.store
    r = max(engine.local_index, 0)
    with open(os.path.join(path, f"shard-{r:05d}.json")) as f:
        meta = json.load(f)
    if meta["world_size"] != st.world_size or meta["padded"] != st.padded:
        raise ValueError("sharded checkpoint was written with a different layout; export to HF and reload instead")
    tensors = load_file(os.path.join(path, f"shard-{r:05d}-of-{st.world_size:05d}.safetensors"))
    st.param_shard.copy_(tensors["param_shard"].to(st.dtype))
    if st.world_size > 1:
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
