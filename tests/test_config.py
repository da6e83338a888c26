"""YAML + override loader and dataclass validation."""
import os

import pytest
import yaml

from areal_b200.api import cli_args as C

YAML = """
experiment_name: exp
trial_name: t0
seed: 3
tokenizer_path: ${actor.path}
cluster:
  fileroot: /tmp/areal_cfg_test
gconfig:
  n_samples: 4
  max_new_tokens: 128
rollout:
  backend: "native:d1"
  consumer_batch_size: ${train_dataset.batch_size}
  max_head_offpolicyness: 2
actor:
  backend: "fsdp:d1"
  path: /models/x
  optimizer:
    lr: 1.0e-5
  reward_norm:
    mean_level: group
    std_level: group
    group_size: ${gconfig.n_samples}
  max_new_tokens: ${gconfig.max_new_tokens}
ref:
  backend: ${actor.backend}
  path: ${actor.path}
train_dataset:
  batch_size: 32
  path: synthetic/arithmetic
"""


def _load(tmp_path, extra=()):
    p = tmp_path / "c.yaml"
    p.write_text(YAML)
    raw, f = C.parse_cli_args(["--config", str(p), *extra])
    return C.to_structured_cfg(raw, C.GRPOConfig)


def test_yaml_interpolation_and_types(tmp_path):
    cfg = _load(tmp_path)
    assert cfg.tokenizer_path == "/models/x" and cfg.ref.path == "/models/x" and cfg.ref.backend == "fsdp:d1"
    assert cfg.rollout.consumer_batch_size == 32 and isinstance(cfg.rollout.consumer_batch_size, int)
    assert cfg.actor.reward_norm.group_size == 4 and cfg.actor.max_new_tokens == 128
    assert cfg.actor.optimizer.lr == pytest.approx(1e-5)
    assert cfg.actor.eps_clip == 0.2 and cfg.actor.ppo_n_minibatches == 4      # defaults survive


def test_overrides_and_plus_keys(tmp_path):
    cfg = _load(tmp_path, ["actor.optimizer.lr=3e-4", "+actor.eps_clip_higher=0.28", "gconfig.n_samples=8", "seed=7"])
    assert cfg.actor.optimizer.lr == pytest.approx(3e-4) and cfg.actor.eps_clip_higher == pytest.approx(0.28)
    assert cfg.gconfig.n_samples == 8 and cfg.actor.reward_norm.group_size == 8 and cfg.seed == 7


def test_unknown_key_and_type_errors(tmp_path):
    with pytest.raises(C.ConfigError):
        _load(tmp_path, ["actor.not_a_field=1"])
    with pytest.raises(C.ConfigError):
        _load(tmp_path, ["seed=abc"])
    with pytest.raises(C.ConfigError):
        _load(tmp_path, ["actor.c_clip=0.5"])          # __post_init__ validation


def test_reference_yaml_loads():
    root = os.environ.get("AREAL_REFERENCE_ROOT", "")
    ref = os.path.join(root, "examples", "math", "gsm8k_grpo.yaml")
    if not root or not os.path.exists(ref):
        pytest.skip("set AREAL_REFERENCE_ROOT to a checkout of the reference to check its stock YAML")
    raw, _ = C.parse_cli_args(["--config", ref])
    cfg = C.to_structured_cfg(raw, C.GRPOConfig)
    assert cfg.actor.use_decoupled_loss and cfg.actor.rejection_sampling.upper == 5.0
    assert cfg.rollout.max_head_offpolicyness == 2


def test_save_config_roundtrip(tmp_path):
    cfg = _load(tmp_path)
    path = C.save_config(cfg, str(tmp_path / "out"))
    again = C.to_structured_cfg(yaml.safe_load(open(path)), C.GRPOConfig)
    assert again.actor.optimizer.lr == cfg.actor.optimizer.lr and again.gconfig.n_samples == 4


def test_rejection_sampling_config_validation():
    with pytest.raises(ValueError):
        C.RejectionSamplingConfig(level="word")
    with pytest.raises(ValueError):
        C.RejectionSamplingConfig(upper=None, lower=None)
    with pytest.raises(ValueError):
        C.PPOActorConfig(use_sapo_loss=True, use_decoupled_loss=True)


def test_example_configs_parse_and_backend_extras_are_kept():
    import glob
    import os

    from areal_b200.api.cli_args import GRPOConfig, PPOConfig, SFTConfig, parse_cli_args, to_structured_cfg

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    files = sorted(glob.glob(os.path.join(root, "examples", "**", "*.yaml"), recursive=True))
    assert len(files) >= 5
    for f in files:
        cls = SFTConfig if "sft" in os.path.basename(f) else (PPOConfig if "ppo" in os.path.basename(f) else GRPOConfig)
        raw, _ = parse_cli_args(["--config", f])
        cfg = to_structured_cfg(raw, cls)
        assert cfg.experiment_name
    # keys that configure a backend of the reference (SGLang server flags, Megatron switches) are accepted and kept
    raw, _ = parse_cli_args(["--config", files[0], "+sglang.enable_dp_attention=true", "+actor.megatron.recompute_method=uniform",
                             "+actor.use_kernels=false", "+rollout.poll_interval=0.1"])
    cfg = to_structured_cfg(raw, GRPOConfig)
    assert cfg.sglang.extra == {"enable_dp_attention": True} and cfg.actor.megatron.extra == {"recompute_method": "uniform"}
    assert cfg.actor.use_kernels is False and cfg.rollout.poll_interval == 0.1


def test_config_reference_is_generated_from_the_dataclasses():
    from areal_b200.tools import generate_cli_docs as G

    text = G.render()
    assert "## PPOActorConfig" in text and "`prox_logp_method`" in text and "`context_parallel`" in text
    assert G.main(["--check"]) == 0, "docs/config_reference.md is out of date: python -m areal_b200.tools.generate_cli_docs"
