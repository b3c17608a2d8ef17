"""Mixers that keep a decayed matrix state per (request, head) instead of keys and values, and
the shape that lets several mixers run side by side on one input.

    S_t = diag(a_t) S_(t-1) + k_t v_t^T        o_t = S_t^T q_t        (float32, in a state slot)

``gla`` (gated linear attention): q = W_q h * dim^(-1/2), k = W_k h, v = W_v h; a decay per key
channel and token, a_t = sigmoid(W_a2 (W_a1 h) + b)^(1 / tau); each head's o is RMS-normalised
over its value size with a weight shared by the heads, multiplied by silu(W_g h) and projected.
``retention``: one fixed decay per head; q and k may be rotated (pairs (i, i + dims / 2)), k is
multiplied by dim^(-1/2) after the rotation; each head's o is divided by its root mean square (no
weight), multiplied by silu(W_g h) and projected.

:class:`BranchMixer` is what such a mixer (and any other that wants to be usable inside the
``parallel`` mixer) implements: it names the matrix that holds all products of its input
(:meth:`input_weight`), writes what its output projection reads into a slice of a buffer
(:meth:`context`) and names that projection (:meth:`output_weight`).  Alone, its ``forward`` is
product, context, product; side by side, the ``parallel`` mixer fuses the branches' input
matrices into one product and their output projections into another.
"""

from __future__ import annotations

import torch

from ..cache.layout import StateLayerSpec
from ..config.spec import PartSpec
from .base import BuildContext, ParamSpec, Part, StepContext, build_part, register_part


def heads_view(rows: torch.Tensor, start: int, heads: int, size: int) -> torch.Tensor:
    """Columns ``start .. start + heads * size`` of ``rows`` ``[T, n]`` as ``[T, heads, size]`` (a view)."""
    return rows[:, start:start + heads * size].unflatten(1, (heads, size))


class BranchMixer(Part):
    category = "mixer"

    def input_weight(self) -> torch.Tensor:
        """``[n, hidden]``: every matrix that multiplies the mixer's input, row blocks in the order
        :meth:`context` expects its ``proj`` columns."""
        raise NotImplementedError

    def release_input_weight(self) -> None:
        """Called by whoever fused :meth:`input_weight` into a larger matrix: the own copy may go."""

    def context_size(self) -> int:
        raise NotImplementedError

    def output_weight(self) -> torch.Tensor:
        """``[hidden, context_size]``."""
        raise NotImplementedError

    def context(self, proj: torch.Tensor, step: StepContext, cache, out: torch.Tensor, out_scale: float) -> None:
        """``proj`` ``[T, n]`` (a view of wider rows allowed) is ``input_weight() @ h``; write
        ``out_scale`` times what the output projection reads into ``out`` ``[T, context_size]`` (a view
        of wider rows allowed)."""
        raise NotImplementedError

    def forward(self, h: torch.Tensor, step: StepContext, cache) -> torch.Tensor:
        proj = self.ops.linear(h, self.input_weight())
        ctx = torch.empty((h.shape[0], self.context_size()), dtype=h.dtype, device=h.device)
        self.context(proj, step, cache, ctx, 1.0)
        return self.ops.linear(ctx, self.output_weight(), partial_sums=self.partial_sums_ok)


def _pad_rows(blocks: list[torch.Tensor], multiple: int = 8) -> tuple[torch.Tensor, list[int]]:
    """Row blocks stacked, each starting at a multiple of ``multiple`` rows (zero rows between them,
    so that every block's columns of the product start at a 16-byte boundary); and the starts."""
    parts, starts, at = [], [], 0
    for b in blocks:
        starts.append(at)
        parts.append(b)
        at += b.shape[0]
        pad = -at % multiple
        if pad:
            parts.append(b.new_zeros((pad, b.shape[1])))
            at += pad
    return torch.cat(parts, dim=0).contiguous(), starts


class _DecayedStateMixer(BranchMixer):
    """What ``gla`` and ``retention`` share: sizes, the state slot, the gate and the projections."""

    def __init__(self, spec, ctx: BuildContext):
        super().__init__(spec, ctx)
        self.hidden_size = int(spec["hidden_size"])
        self.num_heads = int(spec["num_heads"])
        self.dim = int(spec["dim"])
        self.vdim = int(spec["vdim"])
        self.eps = float(spec["eps"])
        if self.dim > 256:
            raise ValueError(f"dim={self.dim} is not supported: the state kernel keeps up to 256 key rows per head")
        self.names = dict(q="q", k="k", v="v", g="g", o="o")
        self.names.update(spec.get("names") or {})
        self.in_weight = self.o_weight = None
        self.starts: list[int] = []

    def _base_specs(self):
        H, D, Dv, W = self.num_heads, self.dim, self.vdim, self.hidden_size
        n = self.names
        return {n["q"]: ParamSpec((H * D, W)), n["k"]: ParamSpec((H * D, W)), n["v"]: ParamSpec((H * Dv, W)),
                n["g"]: ParamSpec((H * Dv, W)), n["o"]: ParamSpec((W, H * Dv))}

    def _fuse(self, tensors, extra=()):
        n = self.names
        self.in_weight, self.starts = _pad_rows([tensors[n["q"]], tensors[n["k"]], tensors[n["v"]], tensors[n["g"]],
                                                 *extra])
        self.o_weight = tensors[n["o"]].contiguous()

    def input_weight(self):
        return self.in_weight

    def release_input_weight(self):
        self.in_weight = None

    def context_size(self):
        return self.num_heads * self.vdim

    def output_weight(self):
        return self.o_weight

    def kernel_groups(self):
        groups = ["linear_state"]
        groups += ["gemm_f32"] if self.ctx.dtype == torch.float32 else ["gemm_small_m", "gemm_stream"]
        return groups

    def cache_spec(self):
        return StateLayerSpec((self.num_heads, self.dim, self.vdim))

    def _views(self, proj):
        H, D, Dv = self.num_heads, self.dim, self.vdim
        s = self.starts
        return (heads_view(proj, s[0], H, D), heads_view(proj, s[1], H, D), heads_view(proj, s[2], H, Dv),
                heads_view(proj, s[3], H, Dv))


class GatedLinearAttention(_DecayedStateMixer):
    def __init__(self, spec, ctx: BuildContext):
        super().__init__(spec, ctx)
        self.tau = float(spec["tau"])
        self.decay_rank = int(spec["decay_rank"])
        self.a2 = self.a2_bias = self.norm_weight = None

    def param_specs(self):
        H, D, W = self.num_heads, self.dim, self.hidden_size
        specs = self._base_specs()
        specs.update({"norm": ParamSpec((self.vdim,), "vector"), "a1": ParamSpec((self.decay_rank, W)),
                      "a2": ParamSpec((H * D, self.decay_rank)), "a2.b": ParamSpec((H * D,), "vector")})
        return specs

    def load(self, tensors):
        self._fuse(tensors, extra=[tensors["a1"]])
        self.a2 = tensors["a2"].contiguous()
        self.a2_bias = tensors["a2.b"].contiguous()
        self.norm_weight = tensors["norm"].contiguous()

    def context(self, proj, step, cache, out, out_scale):
        ops = self.ops
        H, D, Dv = self.num_heads, self.dim, self.vdim
        q, k, v, g = self._views(proj)
        low = proj[:, self.starts[4]:self.starts[4] + self.decay_rank]
        z = ops.linear(low, self.a2).unflatten(1, (H, D))
        o = ops.decayed_state_scan(q, k, v, state=cache.state, cu_seqlens=step.cu_seqlens, state_slots=step.state_slots,
                                   num_seqs=step.num_seqs, decay_logits=z, decay_bias=self.a2_bias, tau=self.tau,
                                   q_scale=D ** -0.5)
        ops.head_norm_gate(o, g, out.unflatten(1, (H, Dv)), weight=self.norm_weight, eps=self.eps, out_scale=out_scale)


class Retention(_DecayedStateMixer):
    def __init__(self, spec, ctx: BuildContext):
        super().__init__(spec, ctx)
        self.decay = [float(d) for d in spec["decay"]]
        if len(self.decay) != self.num_heads:
            raise ValueError("retention: one decay per head")
        pos_spec = spec.get("position") or PartSpec("none")
        self.position = build_part("position", pos_spec, ctx)
        if self.position.style == "rotary" and getattr(self.position, "pairing", "half") != "half":
            raise ValueError("retention rotates pairs (i, i + dims / 2)")
        self.decay_dev = None

    def param_specs(self):
        return self._base_specs()

    def load(self, tensors):
        self._fuse(tensors)
        self.decay_dev = torch.tensor(self.decay, dtype=torch.float32, device=self.ctx.device)

    def context(self, proj, step, cache, out, out_scale):
        ops = self.ops
        H, D, Dv = self.num_heads, self.dim, self.vdim
        q, k, v, g = self._views(proj)
        inv = self.position.device_inverse_frequencies() if self.position.style == "rotary" else None
        o = ops.decayed_state_scan(q, k, v, state=cache.state, cu_seqlens=step.cu_seqlens, state_slots=step.state_slots,
                                   num_seqs=step.num_seqs, head_decay=self.decay_dev, inv_freq=inv,
                                   positions=step.positions, k_scale=D ** -0.5)
        ops.head_norm_gate(o, g, out.unflatten(1, (H, Dv)), weight=None, eps=self.eps, out_scale=out_scale)


class ParallelMixer(Part):
    """Several mixers side by side on the same input; the result is the sum of their outputs, each
    times its own scale.  The branches' input matrices are one product.  Every branch writes
    ``scale * (what its output projection reads)``; where the norm that takes the mixer's output adds
    partial sums, each branch's output projection is a product of its own into one float32 plane and
    the norm adds the planes (no kernel adds the branches up, and every branch has a dense buffer,
    which the specialised attention kernels want); else the branches write into their columns of one
    buffer and the projections, laid side by side, multiply that buffer once.
    ``branches``: ``[(prefix, PartSpec of a BranchMixer, scale), ...]``."""

    category = "mixer"

    def __init__(self, spec, ctx: BuildContext):
        super().__init__(spec, ctx)
        self.branches = []
        for prefix, part_spec, scale in spec["branches"]:
            part = build_part("mixer", part_spec, ctx)
            if not isinstance(part, BranchMixer):
                raise ValueError(f"mixer {part_spec.kind!r} cannot run as a branch of a parallel mixer")
            self.branches.append((str(prefix), part, float(scale)))
        self._owners = {prefix + name: (part, name) for prefix, part, _ in self.branches for name in part.param_specs()}
        self.in_weight = self.o_weight = None
        self.in_starts: list[int] = []
        self.out_starts: list[int] = []

    def param_specs(self):
        return {full: part.param_specs()[name] for full, (part, name) in self._owners.items()}

    def load(self, tensors):
        for prefix, part, _ in self.branches:
            part.load({name: tensors[prefix + name] for name in part.param_specs()})
        self.in_weight, self.in_starts = _pad_rows([part.input_weight() for _, part, _ in self.branches])
        self.o_weight = None  # the projections side by side; made when first needed
        self.in_sizes = [part.input_weight().shape[0] for _, part, _ in self.branches]
        at = 0
        for _, part, _ in self.branches:
            self.out_starts.append(at)
            at += part.context_size()
            part.release_input_weight()

    def kernel_groups(self):
        return [g for _, part, _ in self.branches for g in part.kernel_groups()]

    def step_choosers(self):
        return {name: fn for _, part, _ in self.branches for name, fn in part.step_choosers().items()}

    def position_limit(self):
        limits = [n for n in (part.position_limit() for _, part, _ in self.branches) if n is not None]
        return min(limits) if limits else None

    def cache_spec(self):
        return tuple(part.cache_spec() for _, part, _ in self.branches)

    def forward(self, h: torch.Tensor, step: StepContext, cache) -> torch.Tensor:
        proj = self.ops.linear(h, self.in_weight)
        T = h.shape[0]
        if self.partial_sums_ok:
            planes = torch.empty((len(self.branches), T, self.in_weight.shape[1]), dtype=torch.float32, device=h.device)
            for i, ((_, part, scale), a, n, view) in enumerate(zip(self.branches, self.in_starts, self.in_sizes, cache)):
                ctx = torch.empty((T, part.context_size()), dtype=h.dtype, device=h.device)
                part.context(proj[:, a:a + n], step, view, ctx, scale)
                self.ops.linear(ctx, part.output_weight(), out=planes[i], out_dtype=torch.float32)
            return planes
        if self.o_weight is None:
            self.o_weight = torch.cat([part.output_weight() for _, part, _ in self.branches], dim=1).contiguous()
        ctx = torch.empty((T, self.o_weight.shape[1]), dtype=h.dtype, device=h.device)
        for (_, part, scale), a, n, b, view in zip(self.branches, self.in_starts, self.in_sizes, self.out_starts, cache):
            part.context(proj[:, a:a + n], step, view, ctx[:, b:b + part.context_size()], scale)
        return self.ops.linear(ctx, self.o_weight)


register_part("mixer", "gla", GatedLinearAttention)
register_part("mixer", "retention", Retention)
register_part("mixer", "parallel", ParallelMixer)
