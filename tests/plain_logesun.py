"""A plain, slow statement of the Logesun design: whole sequences, no cache, no batching,
one function per mechanism.  It is the oracle of the Logesun tests and shares no code with
the engine.  ``tensors`` maps checkpoint names to tensors, ``cfg`` is the raw ``config.json``
dictionary.

Precision: with ``act=torch.float32`` everything is float32.  With ``act=torch.bfloat16``
matrix products round their results to bfloat16 (float32 accumulation) while norms, angles,
scores, softmax, router and the residual sum stay in float32, which is how the engine serves
the model.
"""

from __future__ import annotations

import torch


def _mm(x: torch.Tensor, w: torch.Tensor, act) -> torch.Tensor:
    """``W x`` for every row of ``x``; operands and result in the activation type."""
    return (x.to(act).float() @ w.to(act).float().t()).to(act)


def rms_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    x = x.float()
    return x / torch.sqrt(x.pow(2).mean(-1, keepdim=True) + eps) * w.float()


def rotate_interleaved(x: torch.Tensor, positions: torch.Tensor, dims: int, base: float) -> torch.Tensor:
    """Pairs (2i, 2i+1) of the first ``dims`` elements of the last axis turn by p * base^(-2i/dims);
    ``x`` is ``[tokens, ..., n]`` and ``positions`` ``[tokens]``."""
    x = x.float()
    i = torch.arange(dims // 2, dtype=torch.float32)
    freq = 1.0 / (base ** (2.0 * i / dims))
    ang = positions.float()[:, None] * freq[None, :]
    shape = [x.shape[0]] + [1] * (x.dim() - 2) + [dims // 2]
    c, s = ang.cos().reshape(shape), ang.sin().reshape(shape)
    u, v = x[..., 0:dims:2], x[..., 1:dims:2]
    out = x.clone()
    out[..., 0:dims:2] = u * c - v * s
    out[..., 1:dims:2] = v * c + u * s
    return out


def window_sink_attention(q, k, v, scale: float, window: int | None, sink: torch.Tensor | None) -> torch.Tensor:
    """``q, k`` ``[T, H, Dk]``, ``v`` ``[T, H, Dv]`` of one sequence from position 0.  The query at
    position p reads keys max(0, p - window + 1) .. p; exp(sink_h) is one more term of the softmax
    denominator and brings no value."""
    T, H, _ = q.shape
    scores = torch.einsum("ihd,jhd->hij", q.float(), k.float()) * scale
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    seen = (j <= i) if not window else (j <= i) & (i - j < window)
    scores = scores.masked_fill(~seen[None], float("-inf"))
    if sink is not None:
        scores = torch.cat([scores, sink.float()[:, None, None].expand(H, T, 1)], dim=-1)
    p = torch.softmax(scores, dim=-1)
    if sink is not None:
        p = p[..., :-1]
    return torch.einsum("hij,jhd->ihd", p, v.float())


def latent_attention(h, t, prefix: str, m: dict, eps: float, act) -> torch.Tensor:
    """The 'latent_attention' mixer on normalised input ``h`` ``[T, width]``."""
    T = h.shape[0]
    H, dim, rot, vdim, rank = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    pos = torch.arange(T)
    cq = rms_norm(_mm(h, t[prefix + "dq"], act), t[prefix + "dq.norm"], eps).to(act)
    q = _mm(cq, t[prefix + "uq"], act).reshape(T, H, dim + rot)
    dkv = _mm(h, t[prefix + "dkv"], act)
    c = rms_norm(dkv[:, :rank], t[prefix + "dkv.norm"], eps).to(act)
    k_rot = rotate_interleaved(dkv[:, None, rank:], pos, m["rot"]["dims"], m["rot"]["base"]).to(act)
    q_rot = rotate_interleaved(q[..., dim:], pos, m["rot"]["dims"], m["rot"]["base"]).to(act)
    k_plain = _mm(c, t[prefix + "uk"], act).reshape(T, H, dim)
    val = _mm(c, t[prefix + "uv"], act).reshape(T, H, vdim)
    qq = torch.cat([q[..., :dim].float(), q_rot.float()], dim=-1)
    kk = torch.cat([k_plain.float(), k_rot.float().expand(T, H, rot)], dim=-1)
    window = (m.get("mask") or {}).get("size")
    ctx = window_sink_attention(qq, kk, val, m["scale"], window, t.get(prefix + "sink")).to(act)
    return _mm(ctx.reshape(T, H * vdim), t[prefix + "o"], act)


def dense_feed_forward(h, t, prefix: str, act) -> torch.Tensor:
    g = _mm(h, t[prefix + "gate"], act).float()
    u = _mm(h, t[prefix + "up"], act).float()
    return _mm((g * torch.sigmoid(g) * u).to(act), t[prefix + "down"], act)


def clamped_expert(h, t, prefix: str, limit: float, act) -> torch.Tensor:
    g = _mm(h, t[prefix + "gate"], act).float().clamp(max=limit)
    u = _mm(h, t[prefix + "up"], act).float().clamp(-limit, limit)
    y = g * torch.sigmoid(1.702 * g) * (u + 1.0)
    return _mm(y.to(act), t[prefix + "down"], act)


def routed_feed_forward(h, t, prefix: str, mlp: dict, act) -> torch.Tensor:
    """Sigmoid scores, the ``top`` largest chosen, not renormalised; the score multiplies the
    expert's input; a shared expert is added for every token."""
    T = h.shape[0]
    n, top = mlp["router"]["experts"], mlp["router"]["top"]
    scores = torch.sigmoid(h.to(act).float() @ t[prefix + "router"].float().t())
    best = torch.topk(scores, top, dim=-1)
    out = torch.zeros(T, t[prefix + "e0.down"].shape[0], dtype=torch.float32)
    for tok in range(T):
        for w, e in zip(best.values[tok].tolist(), best.indices[tok].tolist()):
            x = (h[tok:tok + 1].float() * w).to(act)
            out[tok] += clamped_expert(x, t, f"{prefix}e{e}.", mlp["expert"]["limit"], act)[0].float()
    if mlp.get("shared"):
        out = out + clamped_expert(h, t, prefix + "shared.", mlp["shared"]["limit"], act).float()
    return out.to(act)


def run_order(cfg: dict) -> list[tuple[int, bool]]:
    """(layer, whether the embedding output is added right before it) for every layer run."""
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop or loop.get("times", 1) <= 1 or loop["start"] >= loop["stop"]:
        return [(i, False) for i in range(n)]
    start, stop, times = loop["start"], loop["stop"], loop["times"]
    order = [(i, False) for i in range(start)]
    for rep in range(times):
        order += [(i, rep > 0 and i == start) for i in range(start, stop)]
    return order + [(i, False) for i in range(stop, n)]


def forward(tokens: list[int], t: dict, cfg: dict, act=torch.float32, want_layers: bool = False):
    """Float32 logits ``[T, vocab]`` of one sequence (and the residual stream after every layer
    run when asked)."""
    eps = cfg["norm"]["eps"]
    ids = torch.tensor(tokens, dtype=torch.long)
    embedded = t["embed"].to(act)[ids].float()
    x = embedded.clone()
    layers = []
    for i, add_embedding in run_order(cfg):
        layer, p = cfg["layers"][i], f"l{i}."
        if add_embedding:
            x = x + embedded
        if layer["type"] != "latent_attention":
            raise ValueError(layer["type"])
        h = rms_norm(x, t[p + "norm1"], eps).to(act)
        y = latent_attention(h, t, p + "mix.", layer["mixer"], eps, act)
        x = x + rms_norm(y, t[p + "norm1b"], eps)
        mlp = layer.get("mlp")
        if mlp:
            h = rms_norm(x, t[p + "norm2"], eps).to(act)
            if mlp["kind"] == "dense":
                y = dense_feed_forward(h, t, p + "mlp.", act)
            elif mlp["kind"] == "moe":
                y = routed_feed_forward(h, t, p + "mlp.", mlp, act)
            else:
                raise ValueError(mlp["kind"])
            x = x + rms_norm(y, t[p + "norm2b"], eps)
        layers.append(x.clone())
    h = rms_norm(x, t["final.norm"], eps).to(act)
    logits = h.float() @ t["head"].to(act).float().t()
    return (logits, torch.stack(layers)) if want_layers else logits
