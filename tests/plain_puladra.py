"""A plain, slow statement of the Puladra design: whole sequences, no cache, no batching, one
function per mechanism.  It is the oracle of the Puladra tests and shares no code with the
engine.  ``t`` maps checkpoint names to tensors, ``cfg`` is the raw ``config.json`` dictionary.

Precision: with ``act=torch.float32`` everything is float32.  With ``act=torch.bfloat16``
matrix products and short convolutions round their results to bfloat16 (float32 accumulation)
while norms, angles, scores, softmax, routers, decays, recurrent states and the residual sum stay
in float32, which is how the engine serves the model.
"""

from __future__ import annotations

import math

import torch


def _mm(x: torch.Tensor, w: torch.Tensor, act) -> torch.Tensor:
    """``W x`` for every row of ``x``; operands and result in the activation type."""
    return (x.to(act).float() @ w.to(act).float().t()).to(act)


def unit_rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    x = x.float()
    return x / torch.sqrt(x.pow(2).mean(-1, keepdim=True) + eps)


def offset_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """The model's norm multiplies by one plus the stored tensor."""
    return unit_rms(x, eps) * (1.0 + w.float())


def plain_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    return unit_rms(x, eps) * w.float()


def gelu_tanh(z: torch.Tensor) -> torch.Tensor:
    z = z.float()
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def rotate_halves(x: torch.Tensor, positions: torch.Tensor, dims: int, base: float) -> torch.Tensor:
    """Element i of the first ``dims`` of the last axis is paired with element i + dims/2; the pair
    turns by p * base^(-2i/dims).  ``x`` is ``[tokens, heads, n]``, ``positions`` ``[tokens]``."""
    x = x.float()
    half = dims // 2
    i = torch.arange(half, dtype=torch.float32)
    freq = base ** (-2.0 * i / dims)
    ang = positions.float()[:, None] * freq[None, :]
    c, s = ang.cos()[:, None, :], ang.sin()[:, None, :]
    u, v = x[..., :half], x[..., half:dims]
    out = x.clone()
    out[..., :half] = u * c - v * s
    out[..., half:dims] = v * c + u * s
    return out


def short_convolution(u: torch.Tensor, w: torch.Tensor, act) -> torch.Tensor:
    """``u`` ``[T, channels]``, ``w`` ``[channels, taps]``: y_t = sum_j w[:, j] u_(t - taps + 1 + j),
    zeros before the sequence's start."""
    T, taps = u.shape[0], w.shape[1]
    padded = torch.cat([torch.zeros(taps - 1, u.shape[1]), u.to(act).float()])
    y = torch.zeros(T, u.shape[1])
    for j in range(taps):
        y = y + w.to(act).float()[:, j][None, :] * padded[j:j + T]
    return y.to(act)


def window_attention(q, k, v, scale: float, window: int | None) -> torch.Tensor:
    """``q`` ``[T, H, D]``, ``k`` ``[T, G, D]``, ``v`` ``[T, G, Dv]`` of one sequence from position 0;
    query head h reads key/value head h // (H / G); position i sees j with 0 <= i - j < window."""
    T, H, _ = q.shape
    G = k.shape[1]
    k = k.float().repeat_interleave(H // G, dim=1)
    v = v.float().repeat_interleave(H // G, dim=1)
    scores = torch.einsum("ihd,jhd->hij", q.float(), k) * scale
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    seen = (j <= i) if not window else (j <= i) & (i - j < window)
    p = torch.softmax(scores.masked_fill(~seen[None], float("-inf")), dim=-1)
    return torch.einsum("hij,jhd->ihd", p, v)


def decayed_state_scan(q, k, v, decay) -> torch.Tensor:
    """S_t = diag(decay_t) S_(t-1) + k_t v_t^T,  o_t = S_t^T q_t, per head, from a zero state, all in
    float32.  ``q, k`` ``[T, H, D]``, ``v`` ``[T, H, Dv]``, ``decay`` ``[T, H, D]`` (per key channel)."""
    T, H, D = q.shape
    S = torch.zeros(H, D, v.shape[-1])
    out = torch.zeros(T, H, v.shape[-1])
    for step in range(T):
        S = decay[step].float()[:, :, None] * S + k[step].float()[:, :, None] * v[step].float()[:, None, :]
        out[step] = torch.einsum("hdv,hd->hv", S, q[step].float())
    return out


def softmax_attention_branch(h, t, p: str, m: dict, act) -> torch.Tensor:
    """Windowed softmax attention with a short convolution on q, k and v before the rotation."""
    T = h.shape[0]
    H, G, D, Dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    pos = torch.arange(T)
    q, k, v = (_mm(h, t[p + n], act) for n in "qkv")
    if m.get("conv"):
        q, k, v = (short_convolution(x, t[p + n + ".conv"], act) for x, n in ((q, "q"), (k, "k"), (v, "v")))
    q, k, v = q.reshape(T, H, D), k.reshape(T, G, D), v.reshape(T, G, Dv)
    if m.get("rot"):
        q = rotate_halves(q, pos, m["rot"]["dims"], m["rot"]["base"]).to(act)
        k = rotate_halves(k, pos, m["rot"]["dims"], m["rot"]["base"]).to(act)
    window = (m.get("mask") or {}).get("size")
    ctx = window_attention(q, k, v, m["scale"], window).to(act)
    return _mm(ctx.reshape(T, H * Dv), t[p + "o"], act)


def retention_branch(h, t, p: str, m: dict, eps: float, act) -> torch.Tensor:
    """Linear attention with one fixed decay per head, no softmax and no denominator."""
    T = h.shape[0]
    H, D, Dv = m["heads"], m["dim"], m["vdim"]
    pos = torch.arange(T)
    q = _mm(h, t[p + "q"], act).reshape(T, H, D)
    k = _mm(h, t[p + "k"], act).reshape(T, H, D)
    v = _mm(h, t[p + "v"], act).reshape(T, H, Dv)
    if m.get("rot"):
        q = rotate_halves(q, pos, m["rot"]["dims"], m["rot"]["base"])
        k = rotate_halves(k, pos, m["rot"]["dims"], m["rot"]["base"])
    k = k.float() * D ** -0.5
    decay = torch.tensor(m["decay"], dtype=torch.float32)[None, :, None].expand(T, H, D)
    o = unit_rms(decayed_state_scan(q, k, v, decay), eps)
    g = _mm(h, t[p + "g"], act).float()
    y = o.reshape(T, H * Dv) * (g * torch.sigmoid(g))
    return _mm(y.to(act), t[p + "o"], act)


def parallel_mixer(h, t, p: str, m: dict, eps: float, act) -> torch.Tensor:
    left = softmax_attention_branch(h, t, p + "left.", m["left"], act).float()
    right = retention_branch(h, t, p + "right.", m["right"], eps, act).float()
    return (m["left_scale"] * left + m["right_scale"] * right).to(act)


def gla_mixer(h, t, p: str, m: dict, eps: float, act) -> torch.Tensor:
    """Gated linear attention: one decay per key channel and token, sigmoid(z)^(1/tau)."""
    T = h.shape[0]
    H, D, Dv = m["heads"], m["dim"], m["vdim"]
    q = _mm(h, t[p + "q"], act).float().reshape(T, H, D) * D ** -0.5
    k = _mm(h, t[p + "k"], act).reshape(T, H, D)
    v = _mm(h, t[p + "v"], act).reshape(T, H, Dv)
    z = _mm(_mm(h, t[p + "a1"], act), t[p + "a2"], act).float() + t[p + "a2.b"].float()
    decay = torch.exp(torch.nn.functional.logsigmoid(z) / m["tau"]).reshape(T, H, D)
    o = plain_norm(decayed_state_scan(q, k, v, decay), t[p + "norm"], eps)
    g = _mm(h, t[p + "g"], act).float()
    y = o.reshape(T, H * Dv) * (g * torch.sigmoid(g))
    return _mm(y.to(act), t[p + "o"], act)


def squared_relu_expert(h, t, p: str, act) -> torch.Tensor:
    u = _mm(h, t[p + "up"], act).float()
    return _mm((torch.relu(u) ** 2).to(act), t[p + "down"], act)


def routed_feed_forward(h, t, p: str, mlp: dict, act) -> torch.Tensor:
    """The ``top`` experts with the largest router logits; weights: softmax over the chosen logits;
    the weight multiplies the expert's output.  The shared expert runs for every token, times
    sigmoid(W_sg h)."""
    T = h.shape[0]
    top = mlp["router"]["top"]
    z = h.to(act).float() @ t[p + "router"].float().t()
    best = torch.topk(z, top, dim=-1)
    weights = torch.softmax(best.values, dim=-1)
    out = torch.zeros(T, t[p + "e0.down"].shape[0], dtype=torch.float32)
    for tok in range(T):
        for w, e in zip(weights[tok].tolist(), best.indices[tok].tolist()):
            out[tok] += w * squared_relu_expert(h[tok:tok + 1], t, f"{p}e{e}.", act)[0].float()
    if mlp.get("shared"):
        gate = torch.sigmoid(_mm(h, t[p + "shared.sg"], act).float())
        out = out + gate * squared_relu_expert(h, t, p + "shared.", act).float()
    return out.to(act)


def token_side_input(x, ids, t, layer: int, dim: int, eps: float, act) -> torch.Tensor:
    """What a layer adds to the stream from the token itself: a slice of a second embedding, gated by
    the stream, projected up and RMS-normalised with a plain weight."""
    p = f"l{layer}.side."
    e = t["side.embed"].to(act)[ids][:, layer * dim:(layer + 1) * dim].float()
    g = (gelu_tanh(_mm(x, t[p + "gate"], act)) * e).to(act)
    y = _mm(g, t[p + "proj"], act)
    return plain_norm(y, t[p + "norm"], eps)


def layer_passes(cfg: dict) -> list[tuple[int, int | None]]:
    """``(layer, pass number if this run starts a pass of the loop, else None)`` for every layer run."""
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return [(i, None) for i in range(n)]
    start, stop, times = loop["start"], loop["stop"], loop["times"]
    order = [(i, None) for i in range(start)]
    for rep in range(times):
        order += [(i, rep if i == start else None) for i in range(start, stop)]
    return order + [(i, None) for i in range(stop, n)]


def forward(tokens: list[int], t: dict, cfg: dict, act=torch.float32, want_layers: bool = False):
    """Float32 logits ``[T, vocab]`` of one sequence (and the residual stream after every layer run
    when asked)."""
    eps = cfg["norm"]["eps"]
    ids = torch.tensor(tokens, dtype=torch.long)
    x = t["embed"].to(act)[ids].float()
    side = (cfg.get("token_side") or {}).get("dim")
    layers = []
    for i, loop_pass in layer_passes(cfg):
        layer, p = cfg["layers"][i], f"l{i}."
        if loop_pass is not None:
            x = x + t["loop.step"][loop_pass].float()
        h = offset_norm(x, t[p + "norm1"], eps).to(act)
        if layer["type"] == "gla":
            y = gla_mixer(h, t, p + "mix.", layer["mixer"], eps, act)
        elif layer["type"] == "parallel":
            y = parallel_mixer(h, t, p + "mix.", layer["mixer"], eps, act)
        else:
            raise ValueError(layer["type"])
        x = x + y.float()
        mlp = layer.get("mlp")
        if mlp:
            if mlp["kind"] != "moe":
                raise ValueError(mlp["kind"])
            h = offset_norm(x, t[p + "norm2"], eps).to(act)
            x = x + routed_feed_forward(h, t, p + "mlp.", mlp, act).float()
        if side:
            x = x + token_side_input(x, ids, t, i, side, eps, act)
        layers.append(x.clone())
    h = offset_norm(x, t["final.norm"], eps).to(act)
    logits = (h.float() @ t["embed"].to(act).float().t()) * cfg.get("logit_scale", 1.0)
    return (logits, torch.stack(layers)) if want_layers else logits
