"""Logesun on the GPU with the engine's kernels, in float32 and bfloat16, against
tests/plain_logesun.py: each mechanism alone, then whole models under every kind of schedule."""

import pytest
import torch

import logesun_cases as lc

pytestmark = pytest.mark.gpu
DEV = "cuda"


@pytest.fixture(scope="module")
def ops():
    from qwen3_runtime_b200.ops.cuda import CudaOps

    return CudaOps()


DTYPES = ["float32", "bfloat16"]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("window,sink", [(7, True), (None, False), (1, True), (64, False)])
def test_mixer_alone(ops, dtype, window, sink):
    lc.case_mixer_alone(dtype, ops, DEV, window=window, sink=sink)


@pytest.mark.parametrize("dtype", DTYPES)
def test_mixer_alone_other_sizes(ops, dtype):
    lc.case_mixer_alone(dtype, ops, DEV, window=10, sink=True, heads=1, dim=8, rot_dim=24, vdim=8, q_rank=8,
                        kv_rank=72, rot_dims=12, page_size=4)
    lc.case_mixer_alone(dtype, ops, DEV, window=40, sink=True, heads=9, dim=32, rot_dim=32, vdim=16, q_rank=64,
                        kv_rank=128, T=130, page_size=16)


@pytest.mark.parametrize("dtype", DTYPES)
def test_attention_edges(ops, dtype):
    lc.case_attention_edges(dtype, ops, DEV)
    lc.case_attention_edges(dtype, ops, DEV, window=8, page_size=8, heads=1)
    lc.case_attention_edges(dtype, ops, DEV, window=33, page_size=16, heads=3, width=96, dv=64, T=80)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("experts,top,shared", [(6, 2, True), (3, 1, False), (4, 4, True), (40, 3, False)])
def test_experts_alone(ops, dtype, experts, top, shared):
    lc.case_experts_alone(dtype, ops, DEV, experts=experts, top=top, shared=shared)
    lc.case_experts_alone(dtype, ops, DEV, experts=experts, top=top, shared=shared, T=300)


@pytest.mark.parametrize("dtype", DTYPES)
def test_kernels_against_their_torch_statements(ops, dtype):
    """The router, the grouped products with the weight on the output, the clamped unit and the
    per-head product at sizes the models above do not have, against tests/emulated_ops.py."""
    from emulated_ops import TorchOps

    ref = TorchOps()
    dt = lc.TORCH[dtype]
    g = torch.Generator().manual_seed(1)
    T, W, E, F, top = 70, 72, 9, 20, 4
    h = torch.randn((T, W), generator=g).to(dt).cuda()
    router = (0.1 * torch.randn((E, W), generator=g)).cuda()  # small enough that no sigmoid saturates to a tie
    chosen, weights = ops.route_top(h, router, top, renormalize=True)
    rc, rw = ref.route_top(h, router, top, renormalize=True)
    assert torch.equal(chosen, rc)
    assert float((weights - rw).abs().max()) < 1e-5
    gate_up = (0.2 * torch.randn((E, 2 * F, W), generator=g)).to(dt).cuda()
    down = (0.2 * torch.randn((E, W, F), generator=g)).to(dt).cuda()
    shared = torch.randn((T, W), generator=g).to(dt).cuda()
    tol = 3e-5 if dtype == "float32" else 6e-2
    for weight_on in ("input", "output"):
        kw = dict(limit=0.7, alpha=1.3, up_offset=0.5, weight_on=weight_on, shared=shared)
        got = ops.routed_experts(h, chosen, weights, gate_up, down, **kw).float()
        want = ref.routed_experts(h, chosen, weights, gate_up, down, **kw).float()
        assert float((got - want).abs().max()) <= tol * max(1.0, float(want.abs().max()))
    x = torch.randn((T, 5, 44), generator=g).to(dt).cuda()
    w = torch.randn((5, 31, 24), generator=g).to(dt).cuda()
    out = torch.zeros((T, 5, 40), dtype=dt, device="cuda")
    ops.head_linear(x[:, :, 3:27], w, out[:, :, 2:33])
    want = torch.zeros_like(out)
    ref.head_linear(x[:, :, 3:27], w, want[:, :, 2:33])
    assert float((out.float() - want.float()).abs().max()) <= tol * float(want.float().abs().max())
    assert float(out[:, :, :2].abs().max()) == 0 and float(out[:, :, 33:].abs().max()) == 0


@pytest.mark.parametrize("dtype", DTYPES)
def test_norms_and_loop(ops, dtype):
    lc.case_norms_and_loop(dtype, ops, DEV)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["P", "Q", "R"])
def test_schedules(tmp_path, ops, name, dtype):
    lc.case_schedules(tmp_path, name, dtype, ops, DEV)


@pytest.mark.parametrize("name", ["P", "Q"])
def test_schedules_through_captured_decode_steps(tmp_path, ops, name):
    lc.case_schedules(tmp_path, name, "bfloat16", ops, DEV, cuda_graph=True)
    lc.case_schedules(tmp_path, name, "float32", ops, DEV, cuda_graph=True, lengths=(40, 5, 33))


@pytest.mark.parametrize("dtype", DTYPES)
def test_long_decode(tmp_path, ops, dtype):
    lc.case_long_decode(tmp_path, "P", dtype, ops, DEV, total=200, cuda_graph=True)
    lc.case_long_decode(tmp_path, "Q", dtype, ops, DEV, total=120)


@pytest.mark.parametrize("dtype", DTYPES)
def test_first_tokens_and_sinks(tmp_path, ops, dtype):
    lc.case_first_tokens(tmp_path, "P", dtype, ops, DEV)
    lc.case_first_tokens(tmp_path, "Q", dtype, ops, DEV)
    lc.case_sink_matters(tmp_path, "Q", dtype, ops, DEV)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("cuda_graph", [False, True])
def test_greedy_generation_under_the_scheduler(tmp_path, ops, dtype, cuda_graph):
    lc.case_greedy_generation(tmp_path, "P", dtype, ops, DEV, cuda_graph=cuda_graph)
    lc.case_greedy_generation(tmp_path, "R", dtype, ops, DEV, cuda_graph=cuda_graph)


def test_trace_replay_program_on_a_logesun_folder(tmp_path, ops):
    """bin/trace_run as a subprocess: the model class is chosen by config.json."""
    import json
    import os
    import subprocess
    import sys

    import numpy as np

    folder = lc.make_dir(tmp_path, "R")
    toks = lc.requests_for("R", (20,))["r0"]
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": toks[:13], "want": [0, 12]}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": toks[13:], "want": [6]}], "end": ["a"]}]
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    out = tmp_path / "out"
    proc = subprocess.run([sys.executable, os.path.join(root, "bin", "trace_run"), "--model", str(folder), "--dtype",
                           "float32", "--out", str(out), "--max-tokens", "64"],
                          input="\n".join(json.dumps(s) for s in steps) + "\n", capture_output=True, text=True,
                          timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert [l for l in proc.stdout.splitlines() if l.startswith("done")] == ["done 0", "done 1"]
    want, tol = lc.expected(folder, {"a": toks}, "float32")
    V = lc.CONFIGS["R"]["config"].vocab
    got0 = torch.from_numpy(np.fromfile(out / "0.f32", dtype="<f4").reshape(2, V))
    got1 = torch.from_numpy(np.fromfile(out / "1.f32", dtype="<f4").reshape(1, V))
    assert float((got0 - want["a"][[0, 12]]).abs().max()) <= tol
    assert float((got1 - want["a"][[19]]).abs().max()) <= tol
