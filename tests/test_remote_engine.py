"""HTTP inference server + remote client engine on CPU (tiny model)."""
import asyncio
import threading
import time

import pytest
import torch

from areal_b200.api.cli_args import GenerationHyperparameters, InferenceEngineConfig, NativeInferConfig
from areal_b200.api.io_struct import ModelRequest, SaveLoadMeta, WeightUpdateMeta
from areal_b200.engine.infer_engine import NativeInferenceEngine
from areal_b200.engine.remote_engine import RemoteInfEngine
from areal_b200.engine.server import InferenceServer, gconfig_from_sampling_params
from areal_b200.models import hf_io
from areal_b200.models.config import preset
from areal_b200.models.decoder import build_model


@pytest.fixture()
def served():
    mc = preset("tiny-qwen2", vocab_size=64, num_layers=2)
    engs, srvs = [], []
    for i in range(2):
        e = NativeInferenceEngine(InferenceEngineConfig(), NativeInferConfig(), model_config=mc)
        e.initialize(device="cpu", seed=1, start_executor=False)
        engs.append(e)
        srvs.append(InferenceServer(e).start())
    yield mc, engs, srvs
    for s in srvs:
        s.stop()
    for e in engs:
        e.destroy()


def test_sampling_params_mapping():
    g = gconfig_from_sampling_params({"temperature": 0.0, "max_new_tokens": 5, "top_k": -1, "stop_token_ids": [3]})
    assert g.greedy and g.max_new_tokens == 5 and g.top_k >= 10 ** 7 and g.stop_token_ids == [3]


def test_remote_generation_matches_local_and_round_robins(served):
    mc, engs, srvs = served
    cl = RemoteInfEngine(InferenceEngineConfig(setup_timeout=20), [s.address for s in srvs]).initialize(start_executor=False)
    g = GenerationHyperparameters(max_new_tokens=6, greedy=True, max_tokens=64)
    prompts = [[1, 2, 3, 4], [5, 6, 7], [9, 9, 1, 2, 3]]

    async def both():
        remote = await asyncio.gather(*[cl.agenerate(ModelRequest(rid=f"r{i}", input_ids=p, gconfig=g)) for i, p in enumerate(prompts)])
        local = await asyncio.gather(*[engs[0].agenerate(ModelRequest(input_ids=p, gconfig=g)) for p in prompts])
        return remote, local
    remote, local = asyncio.run(both())
    for r, l in zip(remote, local):
        assert r.output_tokens == l.output_tokens and r.stop_reason == l.stop_reason
        assert r.output_logprobs == pytest.approx(l.output_logprobs, abs=1e-5) and len(r.output_versions) == r.output_len
    assert cl.choose_server("r0") == srvs[0].address and cl.choose_server("r1") == srvs[1].address   # affinity + round robin
    cl.destroy()


def test_remote_weight_update_from_disk_pause_and_versions(served, tmp_path):
    mc, engs, srvs = served
    cl = RemoteInfEngine(InferenceEngineConfig(setup_timeout=20), [s.address for s in srvs]).initialize(start_executor=False)
    other = build_model(mc, dtype=torch.float32, device="cpu", seed=7)
    hf_io.save_model_hf(other, str(tmp_path / "ckpt"))
    cl.pause_generation()
    cl.update_weights_from_disk(WeightUpdateMeta(type="disk", path=str(tmp_path / "ckpt"), version=4)).result(timeout=60)
    cl.set_version(4)
    cl.continue_generation()
    assert cl.get_version() == 4 and all(e.get_version() == 4 for e in engs)
    k, v = next(iter(other.named_parameters()))
    assert torch.allclose(dict(engs[1].model.named_parameters())[k], v)
    g = GenerationHyperparameters(max_new_tokens=4, greedy=True, max_tokens=64)
    r = asyncio.run(cl.agenerate(ModelRequest(input_ids=[1, 2, 3], gconfig=g)))
    assert r.output_versions == [4] * r.output_len
    cl.destroy()


def test_generation_interrupted_by_pause_is_resumed_with_new_version(served):
    mc, engs, srvs = served
    cl = RemoteInfEngine(InferenceEngineConfig(setup_timeout=20), [srvs[0].address]).initialize(start_executor=False)
    g = GenerationHyperparameters(max_new_tokens=48, greedy=True, max_tokens=128, ignore_eos=True)

    def bump():
        time.sleep(0.15)
        cl.pause_generation()
        cl.set_version(9)
        cl.continue_generation()
    t = threading.Thread(target=bump)
    t.start()
    r = asyncio.run(cl.agenerate(ModelRequest(input_ids=[1, 2, 3, 4, 5], gconfig=g)))
    t.join()
    assert r.output_len == 48 and len(r.output_versions) == 48 and r.stop_reason == "length"
    assert set(r.output_versions) <= {0, 9} and r.output_versions == sorted(r.output_versions)
    cl.destroy()
