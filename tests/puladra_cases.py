"""Puladra: engine and parts against the plain statement (tests/plain_puladra.py), written once
and run on the CPU with the torch statements of the kernels and on the GPU with the kernels."""

from __future__ import annotations

import json

import torch

import plain_puladra as pl
from helpers import (first_mismatch, max_abs_diff, peak_tokens, random_ids, run_trace, trace_mixed, trace_portions,
                     trace_tail_decode, trace_whole)
from qwen3_runtime_b200.cache.storage import CacheLayerView
from qwen3_runtime_b200.config import PartSpec, PuladraConfig
from qwen3_runtime_b200.config.puladra_config import (GlaConfig, MoeConfig, ParallelConfig, PuladraLayerConfig,
                                                      RetentionConfig, RotationConfig, WindowAttentionConfig)
from qwen3_runtime_b200.engine.factory import build_engine, build_runtime, load_model
from qwen3_runtime_b200.parts import BuildContext, ResidualStream, StepContext, build_part
from qwen3_runtime_b200.weights import write_random_model

TORCH = {"float32": torch.float32, "bfloat16": torch.bfloat16}


def _gla(**kw):
    base = dict(heads=3, dim=20, vdim=36, tau=4.0, decay_rank=6)
    base.update(kw)
    return GlaConfig(**base)


def _left(**kw):
    base = dict(heads=6, kv_heads=3, dim=24, vdim=40, scale=0.2, conv=4, rot=RotationConfig(16, 5000.0), window=20)
    base.update(kw)
    return WindowAttentionConfig(**base)


def _right(**kw):
    base = dict(heads=3, dim=12, vdim=20, decay=(0.9, 0.97, 0.999), rot=RotationConfig(12, 300.0))
    base.update(kw)
    return RetentionConfig(**base)


def _par(left=None, right=None, left_scale=0.7, right_scale=1.3):
    return ParallelConfig(left or _left(), right or _right(), left_scale, right_scale)


# Sizes that no two of which are equal where the design lets them differ: key and value sizes, head
# counts, a head size that is no multiple of 8, a rotation of part of a head, windows that are no
# multiple of the page, a window of one page exactly and of one token, convolutions of 4, 2 and no
# taps, top 1 / 2 / every expert, with and without a shared expert, a layer without a feed-forward,
# a loop of three passes in the middle, a loop from layer 0 over everything, no loop, with and
# without the per-layer token input.
CONFIGS = {
    "U": dict(page_size=8, seed=31, config=PuladraConfig(
        vocab=150, width=72, norm_eps=1e-5, logit_scale=1.7, side_dim=10, loop_start=1, loop_stop=3, loop_times=3,
        layers=(PuladraLayerConfig("parallel", _par(), MoeConfig(6, 2, 40, 24)),
                PuladraLayerConfig("gla", _gla(), MoeConfig(5, 3, 24, 0)),
                PuladraLayerConfig("parallel", _par(left=_left(window=8, conv=2, heads=3, kv_heads=3)), None),
                PuladraLayerConfig("gla", _gla(heads=1, dim=40, vdim=8, tau=16.0, decay_rank=3),
                                   MoeConfig(3, 1, 56, 16))))),
    "V": dict(page_size=4, seed=32, config=PuladraConfig(
        vocab=131, width=64, norm_eps=1e-6, logit_scale=1.0, side_dim=0, layers=(
            PuladraLayerConfig("gla", _gla(heads=2, dim=32, vdim=64, tau=2.0, decay_rank=16), MoeConfig(4, 4, 24, 16)),
            PuladraLayerConfig("parallel", _par(left=_left(heads=4, kv_heads=1, dim=32, vdim=16, conv=0, rot=None,
                                                           window=None, scale=0.12),
                                                right=_right(heads=1, dim=16, vdim=48, decay=(0.95,), rot=None),
                                                left_scale=1.0, right_scale=0.25),
                               MoeConfig(5, 2, 8, 0)),
            PuladraLayerConfig("parallel", _par(left=_left(window=33, rot=RotationConfig(24, 1e6))),
                               MoeConfig(2, 1, 16, 40))))),
    "W": dict(page_size=16, seed=33, config=PuladraConfig(
        vocab=90, width=48, norm_eps=1e-5, logit_scale=0.5, side_dim=6, loop_start=0, loop_stop=2, loop_times=2,
        layers=(PuladraLayerConfig("parallel", _par(left=_left(heads=2, kv_heads=2, dim=16, vdim=24, window=1, conv=3,
                                                               rot=RotationConfig(16, 10000.0)),
                                                    right=_right(heads=2, dim=8, vdim=8, decay=(0.5, 0.9921875),
                                                                 rot=RotationConfig(4, 50.0))),
                                   MoeConfig(2, 1, 32, 32)),
                PuladraLayerConfig("gla", _gla(heads=2, dim=16, vdim=24, tau=8.0, decay_rank=8), None)))),
    # keys and values of one size (64) in groups of four query heads: in bfloat16 the specialised attention
    # kernels (split-KV decode, tensor-core prompt portions) take the windowed branch
    "X": dict(page_size=16, seed=34, config=PuladraConfig(
        vocab=210, width=128, norm_eps=1e-5, logit_scale=1.2, side_dim=16, loop_start=0, loop_stop=1, loop_times=2,
        layers=(PuladraLayerConfig("parallel", _par(left=_left(heads=8, kv_heads=2, dim=64, vdim=64, conv=3, window=40,
                                                               rot=RotationConfig(64, 10000.0), scale=0.125),
                                                    right=_right(heads=2, dim=32, vdim=64, decay=(0.97, 0.999),
                                                                 rot=RotationConfig(32, 1e5))),
                                   MoeConfig(4, 2, 64, 32)),
                PuladraLayerConfig("gla", _gla(heads=2, dim=64, vdim=128, tau=16.0, decay_rank=16),
                                   MoeConfig(8, 3, 32, 0))))),
    # no layer with pages at all, a loop of a single pass over the last layer, more experts than a warp's
    # worth of lanes would suggest (9, five chosen)
    "Y": dict(page_size=16, seed=35, config=PuladraConfig(
        vocab=64, width=40, norm_eps=1e-5, logit_scale=1.0, side_dim=0, loop_start=1, loop_stop=2, loop_times=1,
        layers=(PuladraLayerConfig("gla", _gla(heads=2, dim=16, vdim=24, tau=8.0, decay_rank=8), MoeConfig(9, 5, 16, 0)),
                PuladraLayerConfig("gla", _gla(heads=2, dim=16, vdim=24, tau=8.0, decay_rank=8), None)))),
    # every layer parallel, a convolution of one tap (nothing is carried), a rotation of one pair, as many
    # key/value heads as query heads, a window shorter than a page
    "Z": dict(page_size=16, seed=36, config=PuladraConfig(
        vocab=64, width=40, norm_eps=1e-5, logit_scale=2.0, side_dim=3, layers=(
            PuladraLayerConfig("parallel", _par(left=_left(conv=1, heads=4, kv_heads=4, dim=8, vdim=8,
                                                           rot=RotationConfig(2, 10.0), window=5)), None),
            PuladraLayerConfig("parallel", _par(left=_left(conv=1, heads=4, kv_heads=4, dim=8, vdim=8,
                                                           rot=RotationConfig(2, 10.0), window=5)),
                               MoeConfig(9, 5, 16, 0))))),
}

STD = 0.15  # spread of the random matrices: attention, states and experts have to matter
ROUTER_GAIN = 3.0  # routers are made decisive: a choice should not hang on a logit's last bit


def _every_expert(cfg: PuladraConfig) -> PuladraConfig:
    """The same model with every expert chosen for every token (the weights are then the softmax over
    all router logits).  Whole models in bfloat16 are tested in this form: with many tokens, layers
    and passes some router logit pair always lies within bfloat16 rounding, the choice between two
    experts then goes either way, both are right, and the logits differ by far more than rounding.
    The choice itself is tested in float32 on whole models and in bfloat16 on the feed-forward alone."""
    import dataclasses

    layers = tuple(dataclasses.replace(l, mlp=dataclasses.replace(l.mlp, top=l.mlp.experts)) if l.mlp else l
                   for l in cfg.layers)
    return dataclasses.replace(cfg, layers=layers)


for _name in ("U", "V", "W", "X", "Y", "Z"):
    CONFIGS[_name + "all"] = dict(CONFIGS[_name], config=_every_expert(CONFIGS[_name]["config"]))


def model_for(name, dtype):
    return name + "all" if dtype == "bfloat16" and not name.endswith("all") else name


def make_dir(tmp_path, name):
    spec = CONFIGS[name]
    folder = tmp_path / f"puladra_{name}"
    if not (folder / "model.safetensors").exists():
        from safetensors.torch import load_file, save_file

        write_random_model(spec["config"], folder, spec["seed"], std=STD, vector_std=0.1)
        t = load_file(str(folder / "model.safetensors"))
        for k in t:
            if k.endswith(".router"):
                t[k] = (t[k].float() * ROUTER_GAIN).to(t[k].dtype)
            if k.endswith((".norm1", ".norm2")) or k == "final.norm":  # these are stored as deviations from one
                t[k] = (t[k].float() - 1.0).to(t[k].dtype)
            if k.endswith(".conv"):
                t[k] = (t[k].float() * 3.0).to(torch.bfloat16)
            if k == "loop.step":
                t[k] = (t[k].float() * 4.0).to(torch.bfloat16)
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
    requests side by side with pages and slots freed and used again (pages poisoned in between)."""
    name = model_for(name, dtype)
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
        assert rt.cache.slots.num_free == rt.cache.slots.num_slots
        assert sum(len(v) for v in results[kind].values()) == sum(lengths)
    # how the tokens were cut and what else was in the batch changes nothing beyond rounding
    whole = {rid: torch.stack([rows[p] for p in sorted(rows)]) for rid, rows in results["whole"].items()}
    cut_tol = tol if dtype == "bfloat16" else 2e-5 * max(1.0, max(float(v.abs().max()) for v in whole.values()))
    for kind in ("tail", "portions", "mixed"):
        check(results[kind], whole, cut_tol, f"{name} {dtype} {kind} against whole")


def case_long_decode(tmp_path, name, dtype, ops, device, total=150, cuda_graph=False):
    """A short prompt and then one token at a time, far beyond every window and over many pages."""
    name = model_for(name, dtype)
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
    """One-token and two-token sequences, alone and side by side, and a sequence fed one token at a
    time from its first: the first positions, where a window is not full, the convolution reads
    zeros and the states start from zero in slots that others used before."""
    name = model_for(name, dtype)
    folder = make_dir(tmp_path, name)
    requests = requests_for(name, (1, 2, 3, 1), seed=9)
    want, tol = expected(folder, requests, dtype)
    steps = [{"step": 0, "entries": [{"id": r, "tokens": t, "want": list(range(len(t)))} for r, t in requests.items()],
              "end": list(requests)}]
    rt = runtime(folder, name, dtype, ops, device, pages=32)
    check(run_trace(rt, steps), want, tol, f"{name} {dtype} first tokens")
    # the same slots again, now token by token from position 0
    again = requests_for(name, (6, 5), seed=10)
    want, tol = expected(folder, again, dtype)
    steps = [{"step": i, "entries": [{"id": r, "tokens": [t[i]], "want": [0]} for r, t in again.items() if i < len(t)],
              "end": [r for r, t in again.items() if i == len(t) - 1]} for i in range(6)]
    check(run_trace(rt, steps), want, tol, f"{name} {dtype} first tokens one by one in used slots")


def case_greedy_generation(tmp_path, name, dtype, ops, device, cuda_graph=False, steps=12):
    """Greedy generation through the engine's own entry point, scheduler and sampler: unequal
    prompts side by side in a small pool, every token checked at its own place against the plain
    model given the tokens before it."""
    name = model_for(name, dtype)
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


# ---- parts and kernels alone ---------------------------------------------------------------------

def _step(positions, seqs, tables, device, slots=None, ids=None):
    T = len(positions)
    i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=device)  # noqa: E731
    B = len(tables)
    cu = [0]
    for b in range(B):
        cu.append(cu[-1] + sum(1 for s in seqs if s == b))
    kv = [max(p for p, s in zip(positions, seqs) if s == b) + 1 for b in range(B)]
    width = max(len(t) for t in tables)
    bt = [list(t) + [0] * (width - len(t)) for t in tables]
    qlen = max(cu[b + 1] - cu[b] for b in range(B))
    return StepContext(num_tokens=T, num_seqs=B, token_ids=i32(ids if ids is not None else [0] * T),
                       positions=i32(positions), token_seq=i32(seqs), cu_seqlens=i32(cu), kv_lens=i32(kv),
                       state_slots=i32(slots if slots is not None else list(range(B))), block_tables=[i32(bt)],
                       logit_rows=i32([]), num_logit_rows=0, max_query_len=qlen, max_kv_len=max(kv),
                       decode_only=qlen == 1, host_cu_seqlens=cu, host_kv_lens=kv)


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


def _views_for(spec, device, dt, page_size, pages, slots, poison=True):
    """Cache views for a (possibly nested) cache spec, pages and state rows filled with NaN where
    nothing may be read before it is written (state slots start from zero, as the engine leaves them)."""
    from qwen3_runtime_b200.cache.layout import KVLayerSpec, StateLayerSpec

    if isinstance(spec, tuple):
        return tuple(_views_for(s, device, dt, page_size, pages, slots) for s in spec)
    if spec is None:
        return None
    if isinstance(spec, KVLayerSpec):
        fill = float("nan") if poison else 0.0
        k = torch.full((pages, spec.num_kv_heads, page_size, spec.head_dim), fill, dtype=dt, device=device)
        v = torch.full((pages, spec.num_kv_heads, page_size, spec.value_dim or spec.head_dim), fill, dtype=dt,
                       device=device)
        return CacheLayerView(0, 0, page_size, spec.window, k, v, None, True)
    assert isinstance(spec, StateLayerSpec)
    return CacheLayerView(0, None, page_size, None, None, None,
                          torch.zeros((slots, *spec.shape), dtype=torch.float32, device=device), True)


def case_mixer_alone(dtype, ops, device, kind, *, T=45, page_size=8, cuts=(24, 1, 2, 18), **sizes):
    """A mixer on one sequence in portions (one of a single token, one of two) through a paged cache
    whose pages are out of order and a state slot that is not the first, against the plain statement
    on the whole sequence."""
    dt = TORCH[dtype]
    gen = torch.Generator().manual_seed(5)
    width, eps = 64, 1e-5
    ctx = BuildContext(dt, torch.device(device), ops)
    if kind == "gla":
        m = dict(heads=3, dim=20, vdim=36, tau=4.0)
        m.update(sizes)
        spec = PartSpec("gla", dict(hidden_size=width, num_heads=m["heads"], dim=m["dim"], vdim=m["vdim"], tau=m["tau"],
                                    eps=eps, decay_rank=6))
        plain = lambda h, t: pl.gla_mixer(h, t, "mix.", m, eps, dt)  # noqa: E731
    else:
        left = dict(heads=6, kv_heads=3, dim=24, vdim=40, scale=0.2, conv=4, rot=dict(dims=16, base=5000.0),
                    mask=dict(size=20))
        left.update(sizes.get("left", {}))
        right = dict(heads=3, dim=12, vdim=20, decay=[0.9, 0.97, 0.999], rot=dict(dims=12, base=300.0))
        right.update(sizes.get("right", {}))
        m = dict(left=left, right=right, left_scale=0.7, right_scale=1.3)

        def pos(r):
            return PartSpec("rope_neox", dict(rotary_dim=r["dims"], theta=r["base"])) if r else PartSpec("none")

        window = (left.get("mask") or {}).get("size")
        attention = PartSpec("conv_window_attention", dict(
            hidden_size=width, num_heads=left["heads"], num_kv_heads=left["kv_heads"], dim=left["dim"],
            vdim=left["vdim"], scale=left["scale"], taps=left.get("conv") or 0, window=window,
            position=pos(left.get("rot"))))
        retention = PartSpec("retention", dict(hidden_size=width, num_heads=right["heads"], dim=right["dim"],
                                               vdim=right["vdim"], decay=tuple(right["decay"]), eps=eps,
                                               position=pos(right.get("rot"))))
        spec = PartSpec("parallel", dict(branches=(("left.", attention, 0.7), ("right.", retention, 1.3))))
        plain = lambda h, t: pl.parallel_mixer(h, t, "mix.", m, eps, dt)  # noqa: E731
    part = build_part("mixer", spec, ctx)
    tensors = _random_tensors(part, gen, dt, device)
    part.load(tensors)
    h = torch.randn((T, width), generator=gen).to(torch.bfloat16).float()
    want = plain(h, {"mix." + k: v.float().cpu() for k, v in tensors.items()}).float()
    pages_needed = -(-T // page_size)
    table = list(reversed(range(1, pages_needed + 1)))  # not in order, page 0 unused
    cache = _views_for(part.cache_spec(), device, dt, page_size, pages_needed + 2, slots=3)
    got, lo = [], 0
    assert sum(cuts) == T
    for n in cuts:
        step = _step(list(range(lo, lo + n)), [0] * n, [table], device, slots=[2])
        got.append(part.forward(h[lo:lo + n].to(device=device, dtype=dt), step, cache).float().cpu())
        lo += n
    got = torch.cat(got)
    tol = _tolerance(dtype, want)
    diff = float((got - want).abs().max())
    assert diff <= tol, f"{kind} mixer ({dtype}, {sizes}): off by {diff:.3g} (allowed {tol:.3g})"


def case_state_scan(dtype, ops, device, *, H=3, D=20, Dv=36, T=70, gated=True, rot=0):
    """The decayed-state kernel alone: two sequences side by side in portions, states in slots that
    held other sequences' states before, against the plain recurrence; with decays from logits and a
    bias (and a temperature), or one decay per head with rotated q and k."""
    dt = TORCH[dtype]
    gen = torch.Generator().manual_seed(11)
    B = 2
    rnd = lambda *shape: (0.5 * torch.randn(shape, generator=gen)).to(torch.bfloat16).float()  # noqa: E731
    q, k, v, z = rnd(B, T, H, D), rnd(B, T, H, D), rnd(B, T, H, Dv), 2.0 * rnd(B, T, H, D)
    bias = rnd(H * D)
    decay = torch.tensor([0.5, 0.97, 0.999, 0.9][:H])
    inv = (100.0 ** (-torch.arange(rot // 2, dtype=torch.float32) * 2 / rot)) if rot else None
    want = []
    for b in range(B):
        if gated:
            a = torch.exp(torch.nn.functional.logsigmoid(z[b] + bias.reshape(1, H, D)) / 3.0)
            want.append(pl.decayed_state_scan(q[b] * 0.25, k[b], v[b], a))
        else:
            pos = torch.arange(T)
            qq = pl.rotate_halves(q[b], pos, rot, 100.0) if rot else q[b]
            kk = pl.rotate_halves(k[b], pos, rot, 100.0) if rot else k[b]
            want.append(pl.decayed_state_scan(qq, kk * 0.5, v[b], decay[None, :, None].expand(T, H, D)))
    state = torch.full((4, H, D, Dv), float("nan"), dtype=torch.float32, device=device)
    slots = [3, 1]
    state[slots] = 0.0
    got = [[], []]
    at = [0, 0]
    for portions in ((9, 1), (1, 30), (2, 7), (58, 32)):  # unequal portions side by side
        rows, seqs, positions = [], [], []
        for b, n in enumerate(portions):
            rows += [(b, at[b] + i) for i in range(n)]
            seqs += [b] * n
            positions += list(range(at[b], at[b] + n))
        step = _step(positions, seqs, [[0], [0]], device, slots=slots)
        pick = lambda x: torch.stack([x[b, t] for b, t in rows]).to(device=device, dtype=dt)  # noqa: E731
        # q, k, v (and the logits) as slices of wider rows, as the fused projection leaves them
        wide = torch.cat([pick(q).flatten(1), pick(k).flatten(1), pick(v).flatten(1)], dim=1)
        qv, kv = wide[:, :H * D].unflatten(1, (H, D)), wide[:, H * D:2 * H * D].unflatten(1, (H, D))
        vv = wide[:, 2 * H * D:].unflatten(1, (H, Dv))
        kw = dict(state=state, cu_seqlens=step.cu_seqlens, state_slots=step.state_slots, num_seqs=B)
        if gated:
            o = ops.decayed_state_scan(qv, kv, vv, decay_logits=pick(z), decay_bias=bias.to(device), tau=3.0,
                                       q_scale=0.25, **kw)
        else:
            o = ops.decayed_state_scan(qv, kv, vv, head_decay=decay.to(device), k_scale=0.5,
                                       inv_freq=inv.to(device) if rot else None, positions=step.positions, **kw)
        o = o.cpu()
        for i, (b, _t) in enumerate(rows):
            got[b].append(o[i])
        for b, n in enumerate(portions):
            at[b] += n
    for b in range(B):
        g = torch.stack(got[b])
        diff = float((g - want[b]).abs().max())
        tol = 3e-5 * max(1.0, float(want[b].abs().max()))
        assert diff <= tol, f"state scan ({dtype}, gated {gated}, rot {rot}) sequence {b}: off by {diff:.3g}"
    assert torch.isnan(state[0]).all() and torch.isnan(state[2]).all(), "a slot of another request was touched"


def case_state_remembers_a_far_token(dtype, ops, device, *, T=400, H=2, D=16, Dv=8):
    """One key far back (hundreds of tokens, in an earlier portion) that the last query asks for: with
    a decay near one its value comes through the state, and a state that was lost, reset or mixed up
    between portions would show."""
    dt = TORCH[dtype]
    gen = torch.Generator().manual_seed(2)
    q, k = 0.05 * torch.randn((T, H, D), generator=gen), 0.05 * torch.randn((T, H, D), generator=gen)
    v = 0.05 * torch.randn((T, H, Dv), generator=gen)
    far = 7
    k[far, :, 3] += 4.0
    q[T - 1, :, 3] += 4.0
    v[far] = torch.arange(1, Dv + 1).float()[None, :].expand(H, Dv)
    q, k, v = (x.to(torch.bfloat16).float() for x in (q, k, v))
    decay = torch.tensor([0.9990234375, 0.96875][:H])
    want = pl.decayed_state_scan(q, k, v, decay[None, :, None].expand(T, H, D))
    assert float(want[T - 1, 0].abs().max()) > 50 * float(want[T - 2, 0].abs().max()), "the far token does not stand out"
    state = torch.zeros((2, H, D, Dv), dtype=torch.float32, device=device)
    outs, lo = [], 0
    for n in (100, 1, 150, 2, T - 253 - 1, 1):
        step = _step(list(range(lo, lo + n)), [0] * n, [[0]], device, slots=[1])
        cut = lambda x: x[lo:lo + n].to(device=device, dtype=dt)  # noqa: E731
        outs.append(ops.decayed_state_scan(cut(q), cut(k), cut(v), state=state, cu_seqlens=step.cu_seqlens,
                                           state_slots=step.state_slots, num_seqs=1,
                                           head_decay=decay.to(device)).cpu())
        lo += n
    got = torch.cat(outs)
    diff = float((got - want).abs().max())
    assert diff <= 3e-5 * float(want.abs().max()), f"far token through the state ({dtype}): off by {diff:.3g}"


def case_attention_edges(dtype, ops, device, *, window=12, page_size=8, heads=4, kv_heads=2, D=24, Dv=40, T=50):
    """The windowed attention alone with one key that takes all the weight when it is seen: just inside
    the window (distance window - 1) it decides the output, just outside (distance window) it does
    not; for queries inside a prompt portion and for a single decoded token, with the key at a page's
    last row, at a page's first row and inside a page; and a key 48 rows back when there is no window.
    Keys and values have unlike sizes, pages are out of order and unused rows hold NaN; the output goes
    into a slice of wider rows."""
    dt = TORCH[dtype]
    gen = torch.Generator().manual_seed(17)
    pages_needed = -(-T // page_size)
    table = list(reversed(range(1, pages_needed + 1)))
    cases = [(win, qi, qi - dist) for win in (window,) for qi in (win + 19, win + 20, win + 24, T - 1)
             for dist in (win - 1, win)]
    cases += [(None, T - 1, 1), (None, 20, 0)]
    for win, qi, kj in cases:
        k = 0.3 * torch.randn((T, kv_heads, D), generator=gen)
        v = torch.randn((T, kv_heads, Dv), generator=gen)
        q = 0.3 * torch.randn((T, heads, D), generator=gen)
        k[kj, :, D - 3] += 8.0
        q[qi, :, D - 3] += 8.0
        q, k, v = (x.to(torch.bfloat16).float() for x in (q, k, v))
        want = pl.window_attention(q, k, v, 1.0, win)
        seen = win is None or qi - kj < win
        on_key = float((want[qi, 0] - v[kj, 0]).abs().max())
        assert (on_key < 0.05) == seen, "the marked key does not stand out as intended"
        k_pages = torch.full((pages_needed + 2, kv_heads, page_size, D), float("nan"), dtype=dt, device=device)
        v_pages = torch.full((pages_needed + 2, kv_heads, page_size, Dv), float("nan"), dtype=dt, device=device)
        for j in range(T):
            k_pages[table[j // page_size], :, j % page_size] = k[j].to(dt)
            v_pages[table[j // page_size], :, j % page_size] = v[j].to(dt)
        for lo, hi in ((0, T), (qi, qi + 1)):  # a whole prompt; the query as a single decoded token
            step = _step(list(range(lo, hi)), [0] * (hi - lo), [table], device)
            wide = torch.zeros((hi - lo, heads * Dv + 16), dtype=dt, device=device)
            qd = q[lo:hi].reshape(hi - lo, heads * D).to(device=device, dtype=dt).contiguous()
            ops.paged_attention(qd, qd.stride(0), num_heads=heads, num_kv_heads=kv_heads, head_dim=D, k_pages=k_pages,
                                v_pages=v_pages, block_table=step.block_tables[0], token_seq=step.token_seq,
                                positions=step.positions, out=wide[:, 8:8 + heads * Dv], page_size=page_size, scale=1.0,
                                window=win, step=step, value_dim=Dv)
            out = wide[:, 8:8 + heads * Dv].float().cpu().reshape(hi - lo, heads, Dv)
            diff = float((out - want[lo:hi]).abs().max())
            tol = 2e-5 if dtype == "float32" else 3e-2
            assert diff <= tol, f"window {win}, query {qi}, key {kj}, tokens {lo}..{hi}: off by {diff:.3g}"
            assert float(wide[:, :8].abs().max()) == 0 and float(wide[:, 8 + heads * Dv:].abs().max()) == 0


def case_convolution_across_portions(dtype, ops, device, *, taps=4, heads=2, kv_heads=1, D=8, Dv=12, rot=8):
    """The short convolution, rotation and cache write alone: two sequences in portions shorter than
    the convolution (one and two tokens), its state in slots that held other values before; the
    first tokens of a sequence read zeros."""
    dt = TORCH[dtype]
    gen = torch.Generator().manual_seed(23)
    C = heads * D + kv_heads * D + kv_heads * Dv
    T, page_size = 21, 4
    u = torch.randn((2, T, C), generator=gen).to(torch.bfloat16).float()
    w = torch.randn((C, taps), generator=gen).to(torch.bfloat16).float()
    inv = 1000.0 ** (-torch.arange(rot // 2, dtype=torch.float32) * 2 / rot)
    tables = [[5, 2, 7, 1, 9, 3], [4, 8, 0, 6, 10, 11]]
    k_pages = torch.full((13, kv_heads, page_size, D), float("nan"), dtype=dt, device=device)
    v_pages = torch.full((13, kv_heads, page_size, Dv), float("nan"), dtype=dt, device=device)
    state = torch.full((4, taps - 1, C), float("nan"), dtype=torch.float32, device=device)
    slots = [2, 0]
    state[slots] = 0.0
    want = []
    for b in range(2):
        y = pl.short_convolution(u[b], w, torch.float32)
        pos = torch.arange(T)
        qw = pl.rotate_halves(y[:, :heads * D].reshape(T, heads, D), pos, rot, 1000.0)
        kw = pl.rotate_halves(y[:, heads * D:(heads + kv_heads) * D].reshape(T, kv_heads, D), pos, rot, 1000.0)
        want.append((qw, kw, 0.5 * y[:, (heads + kv_heads) * D:].reshape(T, kv_heads, Dv)))
    at = [0, 0]
    tol = 2e-5 if dtype == "float32" else 6e-2
    for portions in ((1, 2), (2, 1), (1, 1), (9, 3), (8, 14)):
        seqs, positions, rows = [], [], []
        for b, n in enumerate(portions):
            seqs += [b] * n
            positions += list(range(at[b], at[b] + n))
            rows += [(b, at[b] + i) for i in range(n)]
        step = _step(positions, seqs, tables, device, slots=slots)
        x = torch.stack([u[b, t] for b, t in rows]).to(device=device, dtype=dt)
        q_out = torch.empty((len(rows), heads * D), dtype=dt, device=device)
        ops.conv_rope_store(x, num_heads=heads, num_kv_heads=kv_heads, head_dim=D, value_dim=Dv,
                            conv_weight=w.t().contiguous().to(device), conv_state=state, inv_freq=inv.to(device),
                            positions=step.positions, token_seq=step.token_seq, cu_seqlens=step.cu_seqlens,
                            state_slots=step.state_slots, num_seqs=2, block_table=step.block_tables[0],
                            k_pages=k_pages, v_pages=v_pages, page_size=page_size, q_out=q_out, value_scale=0.5)
        for i, (b, t) in enumerate(rows):
            page, off = tables[b][t // page_size], t % page_size
            for got, ref, what in ((q_out[i].reshape(heads, D), want[b][0][t], "q"),
                                   (k_pages[page, :, off], want[b][1][t], "k"), (v_pages[page, :, off], want[b][2][t], "v")):
                diff = float((got.float().cpu() - ref).abs().max())
                assert diff <= tol * max(1.0, float(ref.abs().max())), f"{what} of sequence {b} token {t}: off by {diff:.3g}"
        for b, n in enumerate(portions):
            at[b] += n
    assert torch.isnan(state[1]).all() and torch.isnan(state[3]).all(), "a slot of another request was touched"


def case_experts_alone(dtype, ops, device, *, experts=6, top=2, shared=24, T=37):
    dt = TORCH[dtype]
    gen = torch.Generator().manual_seed(8)
    width, ff = 48, 40
    spec = PartSpec("routed_experts", dict(hidden_size=width, num_experts=experts, top=top, expert_size=ff,
                                           activation="relu2", score="softmax_chosen", weight_on="output",
                                           shared_size=shared, shared_gate="sigmoid" if shared else None))
    part = build_part("feed_forward", spec, BuildContext(dt, torch.device(device), ops))
    tensors = _random_tensors(part, gen, dt, device, std=0.4)
    part.load(tensors)
    h = torch.randn((T, width), generator=gen).to(torch.bfloat16).float()
    mlp = dict(router=dict(experts=experts, top=top), expert=dict(ff=ff), shared=dict(ff=shared) if shared else None)
    want = pl.routed_feed_forward(h, {"mlp." + k: v.float().cpu() for k, v in tensors.items()}, "mlp.", mlp, dt).float()
    got = part.forward(h.to(device=device, dtype=dt), None).float().cpu()
    tol = _tolerance(dtype, want)
    diff = float((got - want).abs().max())
    assert diff <= tol, f"routed experts ({dtype}, top {top} of {experts}): off by {diff:.3g} (allowed {tol:.3g})"


def case_stream_extras(dtype, ops, device):
    """The stream through a norm that multiplies by 1 + w: a vector added to every row, the stream read
    without a norm, the token input's output normalised with a plain weight before it is added, and
    partial-sum planes as what is pending in each of these."""
    dt = TORCH[dtype]
    gen = torch.Generator().manual_seed(3)
    H, T, V, dim = 40, 7, 19, 6
    ctx = BuildContext(dt, torch.device(device), ops)
    norm = build_part("norm", PartSpec("rmsnorm", dict(size=H, eps=1e-5, weight_name="", weight_offset=1.0)), ctx)
    w = (0.2 * torch.randn(H, generator=gen)).to(device)
    norm.load({"": w})
    table = torch.randn((V, H), generator=gen).to(torch.bfloat16).to(device=device, dtype=dt)
    side_table = torch.randn((V, 3 * dim), generator=gen).to(torch.bfloat16).to(device=device, dtype=dt)
    ctx.shared["side.table"] = side_table
    ids = torch.randint(0, V, (T,), generator=gen).to(device=device, dtype=torch.int32)
    vec = torch.randn(H, generator=gen).to(device)
    stream = ResidualStream(T, H, ids=ids, table=table)
    stream.add_vector = vec
    out0 = norm.add_norm(stream)
    x = table[ids.long()].float() + vec
    tol = _tolerance(dtype, x)
    assert float((out0.float() - pl.offset_norm(x, w, 1e-5).to(dt).float()).abs().max()) <= tol
    assert stream.add_vector is None
    # the token input after a sublayer whose output comes as partial-sum planes
    side = build_part("side_input", PartSpec("gated_token_input", dict(hidden_size=H, dim=dim, offset=dim,
                                                                       table="side.table", eps=1e-5)), ctx)
    st = _random_tensors(side, gen, dt, device)
    side.load(st)
    planes = torch.randn((3, T, H), generator=gen).to(device)
    stream.pending = planes
    step = _step(list(range(T)), [0] * T, [[0]], device, ids=ids.tolist())
    side.forward(stream, step, lambda s: norm.add_norm(s, normalise=False))
    x = x + planes.sum(0)
    assert float((stream.resid - x).abs().max()) <= 1e-5 * float(x.abs().max())
    t = {"side.embed": side_table.float().cpu(), **{"l1.side." + k: v.float().cpu() for k, v in st.items()}}
    y = pl.token_side_input(x.cpu(), ids.long().cpu(), t, 1, dim, 1e-5, dt)
    stream.add_vector = vec
    out1 = norm.add_norm(stream)
    x = x + y.to(device) + vec
    assert float((stream.resid - x).abs().max()) <= (2e-5 if dtype == "float32" else 5e-2) * float(x.abs().max())
    assert float((out1.float() - pl.offset_norm(x, w, 1e-5).to(dt).float()).abs().max()) <= 3 * tol


def case_router_scores(dtype, ops, device):
    """The weights are the softmax over the chosen logits only: they sum to one whatever the others are."""
    dt = TORCH[dtype]
    gen = torch.Generator().manual_seed(4)
    T, W, E, top = 33, 40, 9, 4
    h = torch.randn((T, W), generator=gen).to(dt).to(device)
    router = (0.3 * torch.randn((E, W), generator=gen)).to(device)
    chosen, weights = ops.route_top(h, router, top, score="softmax_chosen")
    z = h.float() @ router.t()
    best = torch.topk(z, top, dim=-1)
    assert torch.equal(chosen.long().cpu(), best.indices.cpu())
    assert float((weights.cpu() - torch.softmax(best.values, -1).cpu()).abs().max()) < 1e-5
    assert float((weights.sum(-1) - 1).abs().max()) < 1e-5
