"""Pipeline-parallel parity (gloo ranks on CPU): 1F1B, GPipe and the split-backward ZBH1 schedule over 2 and 3 stages against the
unsplit model. Prints PP_OK per rank."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

from areal_b200.models.config import preset  # noqa: E402
from areal_b200.models.decoder import PackedBatch, build_model  # noqa: E402
from areal_b200.parallel.pp import (InterleavedStages, PipelineRunner, PipelineStage, ScheduledPipelineRunner,  # noqa: E402
                                    build_timetable, split_layers)


def main():
    dist.init_process_group("gloo")
    rank, world = dist.get_rank(), dist.get_world_size()
    for name, tie in (("tiny-qwen3", False), ("tiny-qwen2", True)):
        cfg = preset(name, num_layers=6 if world == 3 else 4)
        assert cfg.tie_word_embeddings == tie
        full = build_model(cfg, dtype=torch.float32, device="cpu", seed=3)
        stage = PipelineStage(cfg, rank, world, dtype=torch.float32, device="cpu", seed=3)
        g = torch.Generator().manual_seed(1)
        mbs = []
        for lens in ([20, 12], [7, 30, 5], [16], [9, 9, 9]):
            T = sum(lens)
            ids = torch.randint(0, cfg.vocab_size, (T,), generator=g)
            cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32)
            pos = torch.cat([torch.arange(n) for n in lens]).int()
            mbs.append(dict(input_ids=ids, pb=PackedBatch(cu, pos, T, max(lens)), labels=torch.roll(ids, -1), cu=cu, max_len=max(lens)))

        def loss_of(model):
            def fn(hidden, mb):
                lp, _ = model.logprobs_entropy(hidden, mb["labels"])
                return -lp.float().mean() / len(mbs)
            return fn
        for schedule in ("1F1B", "GPipe", "ZBH1"):
            stage.zero_grad(set_to_none=True)
            full.zero_grad(set_to_none=True)
            full.train(); stage.train()
            runner = PipelineRunner(stage, dist.group.WORLD, schedule)
            losses = runner.run(mbs, loss_of(stage))
            ref_losses = []
            for mb in mbs:
                l = loss_of(full)(full(mb["input_ids"], mb["cu"], max_seqlen=mb["max_len"]), mb)
                l.backward()
                ref_losses.append(l.detach())
            tot = runner.broadcast_loss(torch.stack(losses).sum() if losses else None)
            assert abs(tot.item() - torch.stack(ref_losses).sum().item()) < 1e-5, (name, schedule)
            ref_grads = {n: p.grad for n, p in full.named_parameters()}
            for n, p in stage.named_parameters():
                want = ref_grads[stage.native_name(n)]
                assert p.grad is not None, n
                err = (p.grad - want).abs().max().item()
                assert err < 2e-5, f"{name} {schedule} stage {rank}: grad of {n} off by {err}"
            fo = runner.run(mbs, loss_of(stage), forward_only=True)
            assert (len(fo) == len(mbs)) == stage.is_last
        # ---- virtual pipeline: two chunks per rank, interleaved 1F1B on the tick-synchronous runner
        if cfg.num_layers % (2 * world) == 0 or cfg.num_layers >= 2 * world:
            inter = InterleavedStages(cfg, rank, world, 2, dtype=torch.float32, device="cpu", seed=3)
            mbs_i = (mbs * world)[: 2 * world]                     # a multiple of the pipeline size
            for schedule in ("Interleaved1F1B", "GPipe", "InterleavedZeroBubble"):
                inter.zero_grad(set_to_none=True)
                full.zero_grad(set_to_none=True)
                inter.train()
                runner = ScheduledPipelineRunner(inter, dist.group.WORLD, schedule)

                def loss_i(hidden, mb):
                    lp, _ = inter.logprobs_entropy(hidden, mb["labels"])
                    return -lp.float().mean() / len(mbs_i)
                losses = runner.run(mbs_i, loss_i)
                ref_losses = []
                for mb in mbs_i:
                    lp, _ = full.logprobs_entropy(full(mb["input_ids"], mb["cu"], max_seqlen=mb["max_len"]), mb["labels"])
                    l = -lp.float().mean() / len(mbs_i)
                    l.backward()
                    ref_losses.append(l.detach())
                tot = runner.broadcast_loss(torch.stack(losses).sum() if losses else None)
                assert abs(tot.item() - torch.stack(ref_losses).sum().item()) < 1e-5, (name, schedule)
                ref_grads = {n: p.grad for n, p in full.named_parameters()}
                checked = 0
                for n, p in inter.named_parameters():
                    want = ref_grads[inter.native_name(n)]
                    assert p.grad is not None, n
                    err = (p.grad - want).abs().max().item()
                    assert err < 2e-5, f"{name} {schedule} rank {rank}: grad of {n} off by {err}"
                    checked += 1
                assert checked > 0
                fo = runner.run(mbs_i, loss_i, forward_only=True)
                assert (len(fo) == len(mbs_i)) == (rank == world - 1)
    t = build_timetable(4, 2, 8)
    assert sum(1 for row, _ in t for o in row if o is not None) == 4 * 2 * 8 * 2 and len(t) < 2 * 8 * 2 + 2 * (4 - 1) * 2
    assert [list(r) for r in split_layers(36, 4)] == [list(range(0, 9)), list(range(9, 18)), list(range(18, 27)), list(range(27, 36))]
    assert sum(len(r) for r in split_layers(10, 3, first_extra=1, last_extra=2)) == 10
    print("PP_OK", flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
