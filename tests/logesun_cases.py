"""Logesun: engine and parts against the plain statement (tests/plain_logesun.py), written once
and run on the CPU with the torch statements of the kernels and on the GPU with the kernels."""

from __future__ import annotations

import json

import torch

import plain_logesun as pl
from helpers import (first_mismatch, max_abs_diff, peak_tokens, random_ids, run_trace, trace_mixed, trace_portions,
                     trace_tail_decode, trace_whole)
from qwen3_runtime_b200.config import LogesunConfig, PartSpec
from qwen3_runtime_b200.config.logesun_config import (ExpertConfig, FeedForwardConfig, LatentAttentionConfig,
                                                      LogesunLayerConfig)
from qwen3_runtime_b200.engine.factory import build_engine, build_runtime, load_model
from qwen3_runtime_b200.parts import BuildContext, ResidualStream, StepContext, build_part
from qwen3_runtime_b200.weights import write_random_model

TORCH = {"float32": torch.float32, "bfloat16": torch.bfloat16}


def _mixer(**kw):
    base = dict(heads=3, dim=24, rot_dim=16, vdim=40, q_rank=48, kv_rank=56, scale=0.17, rot_dims=16, rot_base=5000.0,
                window=20)
    base.update(kw)
    return LatentAttentionConfig(**base)


def _moe(experts, top, ff, limit, shared=None):
    return FeedForwardConfig(kind="moe", experts=experts, top=top, expert=ExpertConfig(ff, limit),
                             shared=ExpertConfig(*shared) if shared else None)


def _layer(mixer, mlp):
    return LogesunLayerConfig("latent_attention", mixer, mlp)


# Sizes that no two of which are equal where the design lets them differ: value size and key sizes,
# the two ranks, a latent that is no multiple of 32, windows that are no multiple of the page, a
# window of one page exactly, top 1 / top 2 / every expert, with and without a shared expert, a
# layer without a feed-forward, a loop of three passes, no loop, a loop from layer 0.
CONFIGS = {
    # a loop of three passes over two layers, one of them routed
    "P": dict(page_size=8, seed=21, config=LogesunConfig(
        vocab=200, width=96, norm_eps=1e-5, loop_start=1, loop_stop=3, loop_times=3, layers=(
            _layer(_mixer(), FeedForwardConfig(kind="dense", ff=112)),
            _layer(_mixer(), _moe(6, 2, 40, 1.5, shared=(72, 2.5))),
            _layer(_mixer(window=8), None),
            _layer(_mixer(), _moe(3, 1, 56, 3.0))))),
    # no loop; every layer its own sizes and window (one without a window): three cache groups
    "Q": dict(page_size=4, seed=22, config=LogesunConfig(
        vocab=131, width=64, norm_eps=1e-6, layers=(
            _layer(_mixer(heads=5, dim=16, rot_dim=8, vdim=8, q_rank=24, kv_rank=32, rot_dims=8, window=9, scale=0.2),
                   _moe(4, 4, 24, 2.0, shared=(16, 1.0))),
            _layer(_mixer(heads=1, dim=32, rot_dim=32, vdim=64, q_rank=40, kv_rank=24, rot_dims=32, window=None,
                          scale=0.12, rot_base=123456.0),
                   FeedForwardConfig(kind="dense", ff=80)),
            _layer(_mixer(heads=2, dim=8, rot_dim=24, vdim=16, q_rank=16, kv_rank=40, rot_dims=24, window=33, scale=0.3),
                   _moe(5, 3, 8, 4.0))))),
    # the loop starts at layer 0 and covers everything; a window of one token in one layer
    "R": dict(page_size=16, seed=23, config=LogesunConfig(
        vocab=90, width=48, norm_eps=1e-5, loop_start=0, loop_stop=2, loop_times=2, layers=(
            _layer(_mixer(heads=2, dim=16, rot_dim=16, vdim=24, q_rank=32, kv_rank=32, window=1),
                   FeedForwardConfig(kind="dense", ff=64)),
            _layer(_mixer(heads=2, dim=16, rot_dim=16, vdim=24, q_rank=32, kv_rank=32, window=16),
                   _moe(2, 1, 32, 2.0, shared=(32, 2.0)))))),
}

STD = 0.15  # spread of the random matrices: attention and the experts' clamps have to matter


ROUTER_GAIN = 3.0  # routers are made decisive (a choice should not hang on a score's last bit) but do not saturate


def make_dir(tmp_path, name, sink_scale=1.0):
    spec = CONFIGS[name]
    folder = tmp_path / f"logesun_{name}_{sink_scale}"
    if not (folder / "model.safetensors").exists():
        from safetensors.torch import load_file, save_file

        write_random_model(spec["config"], folder, spec["seed"], std=STD, vector_std=0.1)
        t = load_file(str(folder / "model.safetensors"))
        for k in t:
            if k.endswith(".sink"):
                t[k] = (t[k].float() * sink_scale).to(t[k].dtype)
            if k.endswith(".router"):
                t[k] = (t[k].float() * ROUTER_GAIN).to(t[k].dtype)
        save_file(t, str(folder / "model.safetensors"))
    return folder


def read_dir(folder):
    from safetensors.torch import load_file

    return json.loads((folder / "config.json").read_text()), load_file(str(folder / "model.safetensors"))


def expected(folder, requests, dtype):
    """Plain logits per request and the tolerance: float32 a few 1e-5 of the logits' size;
    bfloat16 three times the distance between the plain bfloat16 and the plain float32 logits."""
    raw, t = read_dir(folder)
    exact = {rid: pl.forward(toks, t, raw) for rid, toks in requests.items()}
    scale = max(float(v.abs().max()) for v in exact.values())
    if dtype == "float32":
        return exact, 5e-5 * max(1.0, scale)
    rounded = {rid: pl.forward(toks, t, raw, act=torch.bfloat16) for rid, toks in requests.items()}
    noise = max(float((rounded[r] - exact[r]).abs().max()) for r in exact)
    return rounded, 3.0 * noise


def runtime(folder, name, dtype, ops, device, pages, max_live=4, cuda_graph=False):
    model, _cfg, _ = load_model(folder, dtype=dtype, device=device, ops=ops)
    return build_runtime(model, block_size=CONFIGS[name]["page_size"], num_kv_blocks=pages, max_num_seqs=max_live,
                         cuda_graph=cuda_graph)


def requests_for(name, lengths, seed=0):
    vocab = CONFIGS[name]["config"].vocab
    return {f"r{i}": random_ids(vocab, n, 1000 * seed + i) for i, n in enumerate(lengths)}


def check(got, want, tol, what):
    bad = first_mismatch(got, want, tol)
    assert bad is None, f"{what}: request {bad[0]} position {bad[1]} differs by {bad[2]:.3g} (tolerance {tol:.3g})"
    print(f"{what}: worst difference {max_abs_diff(got, want):.3g} (tolerance {tol:.3g})")


def case_schedules(tmp_path, name, dtype, ops, device, lengths=(75, 9, 41, 2, 58, 1, 30), cuda_graph=False):
    """Whole prompts; the tail decoded token by token; portions down to two tokens; unequal
    requests side by side with pages and slots freed and used again (poisoned in between)."""
    folder = make_dir(tmp_path, name)
    requests = requests_for(name, lengths)
    want, tol = expected(folder, requests, dtype)
    ps = CONFIGS[name]["page_size"]
    results = {}
    for kind, steps in (("whole", trace_whole(requests)), ("tail", trace_tail_decode(requests, tail=30)),
                        ("portions", trace_portions(requests, seed=3)), ("mixed", trace_mixed(requests, seed=5))):
        rt = runtime(folder, name, dtype, ops, device, pages=-(-peak_tokens(steps, 64) // ps), cuda_graph=cuda_graph)
        results[kind] = run_trace(rt, steps, poison=True)
        check(results[kind], want, tol, f"{name} {dtype} {kind}")
        assert rt.cache.num_free_pages == rt.cache.num_pages
        assert sum(len(v) for v in results[kind].values()) == sum(lengths)
    # how the tokens were cut and what else was in the batch changes nothing beyond rounding
    whole = {rid: torch.stack([rows[p] for p in sorted(rows)]) for rid, rows in results["whole"].items()}
    cut_tol = tol if dtype == "bfloat16" else 2e-5 * max(1.0, max(float(v.abs().max()) for v in whole.values()))
    for kind in ("tail", "portions", "mixed"):
        check(results[kind], whole, cut_tol, f"{name} {dtype} {kind} against whole")


def case_long_decode(tmp_path, name, dtype, ops, device, total=150, cuda_graph=False):
    """A short prompt and then one token at a time, far beyond every window and over many pages."""
    folder = make_dir(tmp_path, name)
    requests = requests_for(name, (total,), seed=7)
    want, tol = expected(folder, requests, dtype)
    toks = requests["r0"]
    steps = [{"step": 0, "entries": [{"id": "r0", "tokens": toks[:3], "want": [0, 1, 2]}], "end": []}]
    steps += [{"step": i - 2, "entries": [{"id": "r0", "tokens": [toks[i]], "want": [0]}],
               "end": ["r0"] if i == total - 1 else []} for i in range(3, total)]
    rt = runtime(folder, name, dtype, ops, device, pages=-(-(total + 63) // CONFIGS[name]["page_size"]),
                 cuda_graph=cuda_graph)
    check(run_trace(rt, steps), want, tol, f"{name} {dtype} long decode")
    assert rt.cache.num_free_pages == rt.cache.num_pages


def case_first_tokens(tmp_path, name, dtype, ops, device):
    """One-token and two-token sequences, alone and side by side: the first positions, where a
    window is not full yet and a sink weighs most."""
    folder = make_dir(tmp_path, name)
    requests = requests_for(name, (1, 2, 3, 1), seed=9)
    want, tol = expected(folder, requests, dtype)
    steps = [{"step": 0, "entries": [{"id": r, "tokens": t, "want": list(range(len(t)))} for r, t in requests.items()],
              "end": list(requests)}]
    rt = runtime(folder, name, dtype, ops, device, pages=32)
    check(run_trace(rt, steps), want, tol, f"{name} {dtype} first tokens")


def case_sink_matters(tmp_path, name, dtype, ops, device):
    """With sinks ten times as large the logits move by far more than the tolerance, and the engine
    follows: a sink that was left out, scaled, or counted per key would show."""
    requests = requests_for(name, (40,), seed=11)
    base, _ = expected(make_dir(tmp_path, name), requests, "float32")
    folder = make_dir(tmp_path, name, sink_scale=10.0)
    want, tol = expected(folder, requests, dtype)
    exact, tol32 = expected(folder, requests, "float32")
    assert float((exact["r0"] - base["r0"]).abs().max()) > 1000 * tol32, "the sinks hardly change this model"
    rt = runtime(folder, name, dtype, ops, device, pages=32)
    check(run_trace(rt, trace_portions(requests, seed=2)), want, tol, f"{name} {dtype} large sinks")


def case_greedy_generation(tmp_path, name, dtype, ops, device, cuda_graph=False, steps=12):
    """Greedy generation through the engine's own entry point, scheduler and sampler: unequal
    prompts side by side in a small pool, every token checked at its own place against the plain
    model given the tokens before it."""
    folder = make_dir(tmp_path, name)
    raw, t = read_dir(folder)
    prompts = list(requests_for(name, (17, 3, 29, 8), seed=13).values())
    engine = build_engine(folder, dtype=dtype, device=device, ops=ops, block_size=CONFIGS[name]["page_size"],
                          num_kv_blocks=-(-4 * 64 // CONFIGS[name]["page_size"]), max_num_seqs=3,
                          max_num_batched_tokens=24, cuda_graph=cuda_graph)
    outs = engine.generate_batch(prompts, max_tokens=steps)
    for prompt, out in zip(prompts, outs):
        assert len(out) == steps
        seq = list(prompt) + list(out[:-1])
        exact = pl.forward(seq, t, raw)[len(prompt) - 1:]
        if dtype == "float32":
            rows, tol = exact, 1e-4 * max(1.0, float(exact.abs().max()))
        else:
            rows = pl.forward(seq, t, raw, act=torch.bfloat16)[len(prompt) - 1:]
            tol = 2 * 3.0 * float((rows - exact).abs().max())
        for i, tok in enumerate(out):
            gap = float(rows[i].max() - rows[i][tok])
            assert gap <= tol, f"token {i} ({tok}) is {gap:.3g} below the plain argmax (allowed {tol:.3g})"
    engine.runtime.cache.check_invariants()
    assert engine.runtime.cache.num_free_pages == engine.runtime.cache.num_pages


# ---- parts alone ---------------------------------------------------------------------------------

def _step(positions, seqs, tables, device, page_size):
    T = len(positions)
    i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=device)  # noqa: E731
    B = len(tables)
    cu = [0]
    for b in range(B):
        cu.append(cu[-1] + sum(1 for s in seqs if s == b))
    kv = [max(p for p, s in zip(positions, seqs) if s == b) + 1 for b in range(B)]
    width = max(len(t) for t in tables)
    bt = [list(t) + [0] * (width - len(t)) for t in tables]
    return StepContext(num_tokens=T, num_seqs=B, token_ids=i32([0] * T), positions=i32(positions), token_seq=i32(seqs),
                       cu_seqlens=i32(cu), kv_lens=i32(kv), state_slots=i32([0] * B), block_tables=[i32(bt)],
                       logit_rows=i32([]), num_logit_rows=0, max_query_len=T, max_kv_len=max(kv), decode_only=False,
                       host_cu_seqlens=cu, host_kv_lens=kv)


def _random_tensors(part, gen, dtype, device, std=0.3):
    out = {}
    for name, ps in part.param_specs().items():
        t = torch.randn(ps.shape, generator=gen) * std
        if ps.kind == "vector":
            t = 1.0 + t
        stored = t.to(torch.bfloat16)  # as a checkpoint holds it
        out[name] = stored.to(device=device, dtype=torch.float32 if ps.kind in ("vector", "matrix_f32") else dtype)
    return out


def _tolerance(dtype, want):
    return (3e-5 if dtype == "float32" else 4e-2) * max(1.0, float(want.abs().max()))


def case_mixer_alone(dtype, ops, device, *, window, sink, heads=3, dim=24, rot_dim=16, vdim=40, q_rank=48, kv_rank=56,
                     rot_dims=None, T=45, page_size=8):
    """The mixer on one sequence in two portions through a paged cache whose pages are out of order,
    against the plain statement on the whole sequence."""
    dt = TORCH[dtype]
    gen = torch.Generator().manual_seed(5)
    m = dict(heads=heads, dim=dim, rot_dim=rot_dim, vdim=vdim, q_rank=q_rank, kv_rank=kv_rank, scale=0.2,
             rot=dict(dims=rot_dims or rot_dim, base=777.0), mask=dict(size=window) if window else None)
    width = 64
    position = PartSpec("rope_interleaved", dict(rotary_dim=rot_dims or rot_dim, theta=777.0))
    spec = PartSpec("latent_attention", dict(hidden_size=width, num_heads=heads, dim=dim, rot_dim=rot_dim, vdim=vdim,
                                             q_rank=q_rank, kv_rank=kv_rank, eps=1e-5, scale=0.2, window=window,
                                             sink=sink, position=position))
    part = build_part("mixer", spec, BuildContext(dt, torch.device(device), ops))
    tensors = _random_tensors(part, gen, dt, device)
    part.load(tensors)
    h = torch.randn((T, width), generator=gen).to(torch.bfloat16).float()
    plain_t = {"mix." + k: v.float().cpu() for k, v in tensors.items()}
    want = pl.latent_attention(h, plain_t, "mix.", m, 1e-5, dt).float()
    from qwen3_runtime_b200.cache.storage import CacheLayerView

    pages_needed = -(-T // page_size)
    table = list(reversed(range(1, pages_needed + 1)))  # not in order, page 0 unused
    pages = torch.full((pages_needed + 2, page_size, kv_rank + rot_dim), float("nan"), dtype=dt, device=device)
    view = CacheLayerView(0, 0, page_size, window, None, None, None, True, latent_pages=pages)
    cut = T // 2 + 1
    got = []
    for lo, hi in ((0, cut), (cut, T)):
        step = _step(list(range(lo, hi)), [0] * (hi - lo), [table], device, page_size)
        got.append(part.forward(h[lo:hi].to(device=device, dtype=dt), step, view).float().cpu())
    got = torch.cat(got)
    tol = _tolerance(dtype, want)
    diff = float((got - want).abs().max())
    assert diff <= tol, f"latent attention ({dtype}, window {window}, sink {sink}): off by {diff:.3g} (allowed {tol:.3g})"
    return got, want


def case_attention_edges(dtype, ops, device, *, window=12, page_size=8, heads=3, width=40, dv=24, T=50):
    """The attention over cached rows alone, with one key that takes all the weight when it is seen:
    just inside the window (distance window - 1) it decides the output, just outside (distance
    window) it does not; for queries inside a prompt portion and for a single decoded token, with
    the key at a page's last row, at a page's first row and inside a page; and a key 48 rows back
    when there is no window.  Pages are out of order and unused rows hold NaN."""
    dt = TORCH[dtype]
    gen = torch.Generator().manual_seed(17)
    pages_needed = -(-T // page_size)
    table = list(reversed(range(1, pages_needed + 1)))
    sink = torch.tensor([0.5, -1.0, 2.0][:heads])
    cases = [(win, qi, qi - dist) for win in (window,) for qi in (win + 19, win + 20, win + 24, T - 1)
             for dist in (win - 1, win)]
    cases += [(None, T - 1, 1), (None, 20, 0)]
    for win, qi, kj in cases:
        rows = (0.3 * torch.randn((T, width), generator=gen))
        q = 0.3 * torch.randn((T, heads, width), generator=gen)
        unit = torch.zeros(width)
        unit[width - 3] = 1.0  # in the part of a row that is key only
        rows[kj] = rows[kj] + 6.0 * unit
        q[qi] = q[qi] + 6.0 * unit
        rows, q = rows.to(torch.bfloat16).float(), q.to(torch.bfloat16).float()
        k = rows[:, None, :].expand(T, heads, width)
        want = pl.window_sink_attention(q, k, k[..., :dv], 1.0, win, sink)
        seen = win is None or qi - kj < win
        weight_on_key = float((want[qi] - rows[kj, :dv]).abs().max())
        assert (weight_on_key < 0.05) == seen, "the marked key does not stand out as intended"
        pages = torch.full((pages_needed + 2, page_size, width), float("nan"), dtype=dt, device=device)
        for j in range(T):
            pages[table[j // page_size], j % page_size] = rows[j].to(dt)
        for lo, hi in ((0, T), (qi, qi + 1)):  # a whole prompt; the query as a single decoded token
            step = _step(list(range(lo, hi)), [0] * (hi - lo), [table], device, page_size)
            out = torch.empty((hi - lo, heads, dv), dtype=dt, device=device)
            ops.latent_attention(q[lo:hi].to(device=device, dtype=dt), pages=pages, value_dim=dv,
                                 block_table=step.block_tables[0], token_seq=step.token_seq, positions=step.positions,
                                 sink=sink.to(device), out=out, page_size=page_size, scale=1.0, window=win, step=step)
            diff = float((out.float().cpu() - want[lo:hi]).abs().max())
            tol = 2e-5 if dtype == "float32" else 2e-2
            assert diff <= tol, f"window {win}, query {qi}, key {kj}, tokens {lo}..{hi}: off by {diff:.3g}"


def case_experts_alone(dtype, ops, device, *, experts=6, top=2, shared=True, T=37, weight_on="input"):
    dt = TORCH[dtype]
    gen = torch.Generator().manual_seed(8)
    width, ff = 48, 40
    spec = PartSpec("routed_experts", dict(hidden_size=width, num_experts=experts, top=top, expert_size=ff, limit=1.0,
                                           shared_size=24 if shared else 0, shared_limit=0.5, weight_on=weight_on))
    part = build_part("feed_forward", spec, BuildContext(dt, torch.device(device), ops))
    tensors = _random_tensors(part, gen, dt, device, std=0.4)
    part.load(tensors)
    h = torch.randn((T, width), generator=gen).to(torch.bfloat16).float()
    mlp = dict(router=dict(experts=experts, top=top), expert=dict(ff=ff, limit=1.0),
               shared=dict(ff=24, limit=0.5) if shared else None)
    want = pl.routed_feed_forward(h, {"mlp." + k: v.float().cpu() for k, v in tensors.items()}, "mlp.", mlp, dt).float()
    got = part.forward(h.to(device=device, dtype=dt), None).float().cpu()
    tol = _tolerance(dtype, want)
    diff = float((got - want).abs().max())
    assert diff <= tol, f"routed experts ({dtype}, top {top} of {experts}): off by {diff:.3g} (allowed {tol:.3g})"
    # the clamps are reached: without them the result would differ
    assert float(want.abs().max()) > 0


def case_norms_and_loop(dtype, ops, device):
    """The stream through norms that also normalise what is pending and add the embedding again."""
    dt = TORCH[dtype]
    gen = torch.Generator().manual_seed(3)
    H, T, V = 40, 7, 19
    ctx = BuildContext(dt, torch.device(device), ops)
    norm = build_part("norm", PartSpec("rmsnorm", dict(size=H, eps=1e-5, weight_name="")), ctx)
    w = (1 + 0.2 * torch.randn(H, generator=gen)).to(device)
    post = (1 + 0.2 * torch.randn(H, generator=gen)).to(device)
    norm.load({"": w})
    table = torch.randn((V, H), generator=gen).to(torch.bfloat16).to(device=device, dtype=dt)
    ids = torch.randint(0, V, (T,), generator=gen).to(device=device, dtype=torch.int32)
    y = torch.randn((T, H), generator=gen).to(torch.bfloat16).to(device=device, dtype=dt)
    stream = ResidualStream(T, H, ids=ids, table=table)
    out0 = norm.add_norm(stream)
    x = table[ids.long()].float()
    assert float((out0.float() - pl.rms_norm(x, w, 1e-5).to(dt).float()).abs().max()) <= _tolerance(dtype, x)
    stream.pending, stream.pending_norm, stream.add_source = y, (post, 1e-5), True
    out1 = norm.add_norm(stream)
    x = x + pl.rms_norm(y, post, 1e-5) + table[ids.long()].float()
    assert float((stream.resid - x).abs().max()) <= 1e-5 * float(x.abs().max())
    assert float((out1.float() - pl.rms_norm(x, w, 1e-5).to(dt).float()).abs().max()) <= _tolerance(dtype, x)
    # the final norm: some rows only, the sum left as it is
    stream.pending, stream.pending_norm = y, (post, 1e-5)
    rows = torch.tensor([5, 0], dtype=torch.int32, device=device)
    out2 = norm.add_norm(stream, rows=rows)
    x2 = (x + pl.rms_norm(y, post, 1e-5))[rows.long()]
    assert float((out2.float() - pl.rms_norm(x2, w, 1e-5).to(dt).float()).abs().max()) <= _tolerance(dtype, x2)
    assert float((stream.resid - x).abs().max()) <= 1e-5 * float(x.abs().max())
