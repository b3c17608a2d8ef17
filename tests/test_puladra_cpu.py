"""Puladra on the CPU: the engine's host logic (configuration, loading, cache layers made of several
parts, state slots, batching, scheduling, the looped run order) and the parts' wiring, with the torch
statements of the kernels in place of the kernel table, against tests/plain_puladra.py."""

import json

import pytest

import puladra_cases as pc
from emulated_ops import TorchOps

OPS, DEV = TorchOps(), "cpu"


def test_config_round_trip_run_order_and_sizes_from_tensor_shapes(tmp_path):
    from qwen3_runtime_b200.config import PuladraConfig, load_config, resolve_architecture
    from qwen3_runtime_b200.config.model_config import ConfigError
    from qwen3_runtime_b200.weights.loader import SafetensorsDir

    cfg = pc.CONFIGS["U"]["config"]
    raw = json.loads(json.dumps(cfg.to_hf_config()))
    assert resolve_architecture(raw).config_class is PuladraConfig
    folder = pc.make_dir(tmp_path, "U")
    _arch, read = load_config(folder)
    assert read != cfg  # the decay's rank is not in config.json ...
    assert read.with_tensor_shapes(SafetensorsDir(folder).shape) == cfg  # ... the stored tensor gives it
    assert cfg.run_order() == [(0, None), (1, 0), (2, None), (1, 1), (2, None), (1, 2), (2, None), (3, None)]
    assert pc.CONFIGS["W"]["config"].run_order() == [(0, 0), (1, None), (0, 1), (1, None)]
    assert pc.CONFIGS["V"]["config"].run_order() == [(0, None), (1, None), (2, None)]
    for key, value, match in ((("layers", 0, "type"), "something_else", "unknown mixer type"),
                              (("loop", "stop"), 9, "loop"), (("layers", 0, "mlp", "kind"), "dense", "feed-forward")):
        bad = json.loads(json.dumps(raw))
        at = bad
        for k in key[:-1]:
            at = at[k]
        at[key[-1]] = value
        with pytest.raises(ConfigError, match=match):
            PuladraConfig.from_hf_config(bad)


def test_cache_layers_of_a_parallel_mixer(tmp_path):
    """Pages with a window, the convolution's rows and the retention state of one mixer are three cache
    layers in three groups; layers with unlike windows or sizes get groups of their own."""
    rt = pc.runtime(pc.make_dir(tmp_path, "U"), "U", "float32", OPS, DEV, pages=16)
    kinds = sorted((g.kind, g.window) for g in rt.cache.groups)
    assert [k for k in kinds if k[0] == "window"] == [("window", 8), ("window", 20)]
    assert sum(1 for k in kinds if k[0] == "state") >= 4  # gla states, retention states, two convolutions
    view = rt.storage.view(0)
    (pages, conv), state = view
    assert pages.k_pages.shape[-1] == 24 and pages.v_pages.shape[-1] == 40 and pages.window == 20
    assert tuple(conv.state.shape[1:]) == (3, 6 * 24 + 3 * 24 + 3 * 40)
    assert tuple(state.state.shape[1:]) == (3, 12, 20)
    rt = pc.runtime(pc.make_dir(tmp_path, "V"), "V", "float32", OPS, DEV, pages=16)
    (pages, conv), _state = rt.storage.view(1)
    assert conv is None and pages.window is None


@pytest.mark.parametrize("name", ["U", "V", "W", "X", "Y", "Z"])
def test_schedules(tmp_path, name):
    pc.case_schedules(tmp_path, name, "float32", OPS, DEV)


def test_schedules_with_bfloat16_activations(tmp_path):
    pc.case_schedules(tmp_path, "W", "bfloat16", OPS, DEV, lengths=(40, 2, 21))


def test_long_decode(tmp_path):
    pc.case_long_decode(tmp_path, "U", "float32", OPS, DEV, total=90)


@pytest.mark.parametrize("name", ["U", "W"])
def test_first_tokens(tmp_path, name):
    pc.case_first_tokens(tmp_path, name, "float32", OPS, DEV)


@pytest.mark.parametrize("name", ["U", "V"])
def test_greedy_generation_under_the_scheduler(tmp_path, name):
    pc.case_greedy_generation(tmp_path, name, "float32", OPS, DEV)


def test_mixers_alone():
    pc.case_mixer_alone("float32", OPS, DEV, "gla")
    pc.case_mixer_alone("float32", OPS, DEV, "gla", heads=1, dim=40, vdim=8, tau=1.0)
    pc.case_mixer_alone("float32", OPS, DEV, "parallel")
    pc.case_mixer_alone("float32", OPS, DEV, "parallel", page_size=4,
                        left=dict(heads=2, kv_heads=2, dim=16, vdim=8, conv=0, rot=None, mask=None),
                        right=dict(heads=1, dim=8, vdim=24, decay=[0.99], rot=None))


def test_state_scan_and_a_far_token():
    pc.case_state_scan("float32", OPS, DEV, gated=True)
    pc.case_state_scan("float32", OPS, DEV, gated=False, rot=12)
    pc.case_state_remembers_a_far_token("float32", OPS, DEV)


def test_attention_edges_and_convolution():
    pc.case_attention_edges("float32", OPS, DEV)
    pc.case_attention_edges("float32", OPS, DEV, window=8, page_size=8, heads=1, kv_heads=1, D=20, Dv=8)
    pc.case_convolution_across_portions("float32", OPS, DEV)
    pc.case_convolution_across_portions("float32", OPS, DEV, taps=2, heads=1, D=12, Dv=4, rot=4)


@pytest.mark.parametrize("experts,top,shared", [(6, 2, 24), (3, 1, 0), (4, 4, 8)])
def test_experts_alone(experts, top, shared):
    pc.case_experts_alone("float32", OPS, DEV, experts=experts, top=top, shared=shared)
    pc.case_router_scores("float32", OPS, DEV)


def test_stream_extras():
    pc.case_stream_extras("float32", OPS, DEV)


def test_model_less_entry():
    """``LLM(model=None, architecture="Puladra")`` builds the design's tiny configuration."""
    from qwen3_runtime_b200 import LLM

    llm = LLM(None, architecture="Puladra", dtype="float32", device=DEV, ops=OPS, cuda_graph=False)
    out = llm.generate([[1, 2, 3], [4, 5]], max_tokens=5)
    assert [len(o) for o in out] == [5, 5]
