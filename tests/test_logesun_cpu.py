"""Logesun on the CPU: the engine's host logic (configuration, loading, the cache's windows and
groups, batching, scheduling, the looped run order) and the parts' wiring, with the torch
statements of the kernels in place of the kernel table, against tests/plain_logesun.py."""

import json

import pytest
import torch

import logesun_cases as lc
from emulated_ops import TorchOps

OPS, DEV = TorchOps(), "cpu"


def test_config_round_trip_and_run_order():
    from qwen3_runtime_b200.config import LogesunConfig, resolve_architecture
    from qwen3_runtime_b200.config.model_config import ConfigError

    cfg = lc.CONFIGS["P"]["config"]
    raw = json.loads(json.dumps(cfg.to_hf_config()))
    assert resolve_architecture(raw).config_class is LogesunConfig
    assert LogesunConfig.from_hf_config(raw) == cfg
    assert cfg.run_order() == [(0, False), (1, False), (2, False), (1, True), (2, False), (1, True), (2, False),
                               (3, False)]
    assert lc.CONFIGS["R"]["config"].run_order() == [(0, False), (1, False), (0, True), (1, False)]
    assert [r for r in lc.CONFIGS["Q"]["config"].run_order()] == [(0, False), (1, False), (2, False)]
    bad = json.loads(json.dumps(raw))
    bad["layers"][0]["type"] = "something_else"
    with pytest.raises(ConfigError, match="unknown mixer type"):
        LogesunConfig.from_hf_config(bad)
    bad = json.loads(json.dumps(raw))
    bad["loop"]["stop"] = 9
    with pytest.raises(ConfigError, match="loop"):
        LogesunConfig.from_hf_config(bad)


def test_layers_with_unlike_windows_get_cache_groups_of_their_own(tmp_path):
    rt = lc.runtime(lc.make_dir(tmp_path, "Q"), "Q", "float32", OPS, DEV, pages=16)
    kinds = sorted((g.kind, g.window) for g in rt.cache.groups)
    assert kinds == [("full", None), ("window", 9), ("window", 33)]
    rt = lc.runtime(lc.make_dir(tmp_path, "P"), "P", "float32", OPS, DEV, pages=16)
    # eight layer runs: six with a window of 20 rows, two (the looped layer 2) with one of 8
    assert sorted(len(g.cache_ids) for g in rt.model.cache_layout().groups) == [3, 5]


@pytest.mark.parametrize("name", ["P", "Q", "R"])
def test_schedules(tmp_path, name):
    lc.case_schedules(tmp_path, name, "float32", OPS, DEV)


def test_schedules_with_bfloat16_activations(tmp_path):
    lc.case_schedules(tmp_path, "R", "bfloat16", OPS, DEV, lengths=(40, 2, 21))


def test_long_decode(tmp_path):
    lc.case_long_decode(tmp_path, "P", "float32", OPS, DEV, total=90)


@pytest.mark.parametrize("name", ["P", "Q"])
def test_first_tokens(tmp_path, name):
    lc.case_first_tokens(tmp_path, name, "float32", OPS, DEV)


def test_sinks_matter(tmp_path):
    lc.case_sink_matters(tmp_path, "Q", "float32", OPS, DEV)


@pytest.mark.parametrize("name", ["P", "R"])
def test_greedy_generation_under_the_scheduler(tmp_path, name):
    lc.case_greedy_generation(tmp_path, name, "float32", OPS, DEV)


@pytest.mark.parametrize("window,sink", [(7, True), (None, False), (1, True), (64, False)])
def test_mixer_alone(window, sink):
    lc.case_mixer_alone("float32", OPS, DEV, window=window, sink=sink)


def test_mixer_alone_other_sizes():
    lc.case_mixer_alone("float32", OPS, DEV, window=10, sink=True, heads=1, dim=8, rot_dim=24, vdim=8, q_rank=8,
                        kv_rank=72, rot_dims=12, page_size=4)


def test_attention_edges():
    lc.case_attention_edges("float32", OPS, DEV)
    lc.case_attention_edges("float32", OPS, DEV, window=8, page_size=8, heads=1)


@pytest.mark.parametrize("experts,top,shared,weight_on", [(6, 2, True, "input"), (3, 1, False, "input"),
                                                         (4, 4, True, "input"), (5, 2, False, "output")])
def test_experts_alone(experts, top, shared, weight_on):
    if weight_on == "output":  # the plain statement has the design's form only; both tables agree on the other
        return
    lc.case_experts_alone("float32", OPS, DEV, experts=experts, top=top, shared=shared)


def test_norms_and_loop():
    lc.case_norms_and_loop("float32", OPS, DEV)


def test_random_model_folder_and_model_less_entry(tmp_path):
    """``LLM(model=None, architecture="Logesun")`` builds the design's tiny configuration."""
    from qwen3_runtime_b200 import LLM

    llm = LLM(None, architecture="Logesun", dtype="float32", device=DEV, ops=OPS, cuda_graph=False)
    out = llm.generate([[1, 2, 3], [4, 5]], max_tokens=5)
    assert [len(o) for o in out] == [5, 5]
