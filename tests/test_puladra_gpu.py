"""Puladra on the GPU with the engine's kernels, in float32 and bfloat16, against
tests/plain_puladra.py: each mechanism alone, then whole models under every kind of schedule."""

import pytest
import torch

import puladra_cases as pc

pytestmark = pytest.mark.gpu
DEV = "cuda"


@pytest.fixture(scope="module")
def ops():
    from qwen3_runtime_b200.ops.cuda import CudaOps

    return CudaOps()


DTYPES = ["float32", "bfloat16"]


@pytest.mark.parametrize("dtype", DTYPES)
def test_mixers_alone(ops, dtype):
    pc.case_mixer_alone(dtype, ops, DEV, "gla")
    pc.case_mixer_alone(dtype, ops, DEV, "gla", heads=1, dim=40, vdim=8, tau=1.0)
    pc.case_mixer_alone(dtype, ops, DEV, "gla", heads=2, dim=128, vdim=72, tau=16.0, T=80, cuts=(33, 1, 2, 44))
    pc.case_mixer_alone(dtype, ops, DEV, "parallel")
    pc.case_mixer_alone(dtype, ops, DEV, "parallel", page_size=4,
                        left=dict(heads=2, kv_heads=2, dim=16, vdim=8, conv=0, rot=None, mask=None),
                        right=dict(heads=1, dim=8, vdim=24, decay=[0.99], rot=None))
    pc.case_mixer_alone(dtype, ops, DEV, "parallel", page_size=16, T=150, cuts=(70, 1, 2, 77),
                        left=dict(heads=8, kv_heads=2, dim=64, vdim=64, conv=3, rot=dict(dims=64, base=1e4),
                                  mask=dict(size=40)),
                        right=dict(heads=2, dim=64, vdim=128, decay=[0.97, 0.999], rot=dict(dims=32, base=1e5)))


@pytest.mark.parametrize("dtype", DTYPES)
def test_state_scan_and_a_far_token(ops, dtype):
    pc.case_state_scan(dtype, ops, DEV, gated=True)
    pc.case_state_scan(dtype, ops, DEV, gated=False, rot=12)
    pc.case_state_scan(dtype, ops, DEV, gated=True, H=2, D=128, Dv=40)
    pc.case_state_scan(dtype, ops, DEV, gated=False, H=1, D=7, Dv=33, rot=6)
    pc.case_state_remembers_a_far_token(dtype, ops, DEV)


@pytest.mark.parametrize("dtype", DTYPES)
def test_attention_edges_and_convolution(ops, dtype):
    pc.case_attention_edges(dtype, ops, DEV)
    pc.case_attention_edges(dtype, ops, DEV, window=8, page_size=8, heads=1, kv_heads=1, D=20, Dv=8)
    pc.case_attention_edges(dtype, ops, DEV, window=16, page_size=16, heads=6, kv_heads=2, D=48, Dv=96, T=70)
    pc.case_convolution_across_portions(dtype, ops, DEV)
    pc.case_convolution_across_portions(dtype, ops, DEV, taps=2, heads=1, D=12, Dv=4, rot=4)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("experts,top,shared", [(6, 2, 24), (3, 1, 0), (4, 4, 8)])
def test_experts_alone(ops, dtype, experts, top, shared):
    pc.case_experts_alone(dtype, ops, DEV, experts=experts, top=top, shared=shared)
    pc.case_experts_alone(dtype, ops, DEV, experts=experts, top=top, shared=shared, T=300)
    pc.case_router_scores(dtype, ops, DEV)


def test_kernels_against_their_torch_statements(ops):
    """The small new kernels with sizes the engine's tests do not reach."""
    from emulated_ops import TorchOps

    ref = TorchOps()
    g = torch.Generator().manual_seed(6)
    for dt, tol in ((torch.float32, 2e-6), (torch.bfloat16, 1e-2)):
        x = torch.randn((33, 50), generator=g).to(dt).cuda()
        out, want = torch.empty((33, 43), dtype=dt, device="cuda"), torch.empty((33, 43), dtype=dt, device="cuda")
        ops.relu_squared(x, out)
        ref.relu_squared(x, want)
        assert float((out.float() - want.float()).abs().max()) <= tol * float(want.float().abs().max())
        gate = torch.randn((33, 10), generator=g).to(dt).cuda()
        table = torch.randn((17, 40), generator=g).to(dt).cuda()
        ids = torch.randint(0, 17, (33,), generator=g).to(torch.int32).cuda()
        out, want = torch.empty_like(gate), torch.empty_like(gate)
        ops.gelu_gate_rows(gate, ids, table, 20, out)
        ref.gelu_gate_rows(gate, ids, table, 20, want)
        assert float((out.float() - want.float()).abs().max()) <= tol * max(1.0, float(want.float().abs().max()))
        o = torch.randn((33, 3, 21), generator=g).cuda()
        gates = torch.randn((33, 70), generator=g).to(dt).cuda()
        w = torch.randn(21, generator=g).cuda()
        for weight in (w, None):
            out, want = torch.zeros((33, 80), dtype=dt, device="cuda"), torch.zeros((33, 80), dtype=dt, device="cuda")
            ops.head_norm_gate(o, gates[:, 4:67].unflatten(1, (3, 21)), out[:, 8:71].unflatten(1, (3, 21)), weight=weight,
                               eps=1e-5, out_scale=0.8)
            ref.head_norm_gate(o, gates[:, 4:67].unflatten(1, (3, 21)), want[:, 8:71].unflatten(1, (3, 21)),
                               weight=weight, eps=1e-5, out_scale=0.8)
            assert float((out.float() - want.float()).abs().max()) <= tol * max(1.0, float(want.float().abs().max()))


@pytest.mark.parametrize("dtype", DTYPES)
def test_stream_extras(ops, dtype):
    pc.case_stream_extras(dtype, ops, DEV)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["U", "V", "W", "X", "Y", "Z"])
def test_schedules(tmp_path, ops, name, dtype):
    pc.case_schedules(tmp_path, name, dtype, ops, DEV)


@pytest.mark.parametrize("name", ["U", "V", "X", "Y"])
def test_schedules_through_captured_decode_steps(tmp_path, ops, name):
    pc.case_schedules(tmp_path, name, "bfloat16", ops, DEV, cuda_graph=True)
    pc.case_schedules(tmp_path, name, "float32", ops, DEV, cuda_graph=True, lengths=(40, 5, 33))


@pytest.mark.parametrize("dtype", DTYPES)
def test_long_decode(tmp_path, ops, dtype):
    pc.case_long_decode(tmp_path, "U", dtype, ops, DEV, total=200, cuda_graph=True)
    pc.case_long_decode(tmp_path, "V", dtype, ops, DEV, total=120)
    pc.case_long_decode(tmp_path, "X", dtype, ops, DEV, total=120, cuda_graph=True)


@pytest.mark.parametrize("dtype", DTYPES)
def test_first_tokens(tmp_path, ops, dtype):
    pc.case_first_tokens(tmp_path, "U", dtype, ops, DEV)
    pc.case_first_tokens(tmp_path, "W", dtype, ops, DEV)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("cuda_graph", [False, True])
def test_greedy_generation_under_the_scheduler(tmp_path, ops, dtype, cuda_graph):
    pc.case_greedy_generation(tmp_path, "U", dtype, ops, DEV, cuda_graph=cuda_graph)
    pc.case_greedy_generation(tmp_path, "W", dtype, ops, DEV, cuda_graph=cuda_graph)


def test_trace_replay_program_on_a_puladra_folder(tmp_path, ops):
    """bin/trace_run as a subprocess: the model class is chosen by config.json."""
    import json
    import os
    import subprocess
    import sys

    import numpy as np

    folder = pc.make_dir(tmp_path, "W")
    toks = pc.requests_for("W", (20,))["r0"]
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
    want, tol = pc.expected(folder, {"a": toks}, "float32")
    V = pc.CONFIGS["W"]["config"].vocab
    got0 = torch.from_numpy(np.fromfile(out / "0.f32", dtype="<f4").reshape(2, V))
    got1 = torch.from_numpy(np.fromfile(out / "1.f32", dtype="<f4").reshape(1, V))
    assert float((got0 - want["a"][[0, 12]]).abs().max()) <= tol
    assert float((got1 - want["a"][[19]]).abs().max()) <= tol
