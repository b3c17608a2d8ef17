"""RMSNorm: y = x * rsqrt(mean(x^2) + eps) * w, all in float32, one rounding at the end
(qwen3_runtime/layers/ops.py:17-20; residual form :28-37).  ``weight_offset``: the stored weight
is the deviation from this value, which is added to it when it is loaded (y = ... * (offset + w))."""

from __future__ import annotations

import torch

from .base import BuildContext, ParamSpec, Part, ResidualStream, register_part


class RMSNorm(Part):
    category = "norm"
    adds_partial_sums = True

    def __init__(self, spec, ctx: BuildContext):
        super().__init__(spec, ctx)
        self.size = int(spec["size"])
        self.eps = float(spec["eps"])
        # the stored tensor's name after the part's prefix ("" when the prefix is the whole name)
        self.weight_name = str(spec.get("weight_name", "weight"))
        self.weight_offset = float(spec.get("weight_offset", 0.0))
        self.weight: torch.Tensor | None = None

    def param_specs(self):
        return {self.weight_name: ParamSpec((self.size,), "vector")}

    def load(self, tensors):
        self.weight = tensors[self.weight_name]
        if self.weight_offset:
            self.weight = (self.weight.float() + self.weight_offset).contiguous()

    def pending_scale(self) -> tuple[torch.Tensor, float]:
        """This norm as something the next norm applies to what is pending (``ResidualStream.pending_norm``)."""
        return self.weight, self.eps

    def kernel_groups(self):
        return ["norm"]

    def add_norm(self, stream: ResidualStream, rows: torch.Tensor | None = None,
                 num_rows: int | None = None, normalise: bool = True) -> torch.Tensor:
        """Fold what is pending into the residual sum and return its normalised rows.

        With ``rows`` only those rows are normalised and the residual sum is left as
        it is (the final norm before the output head).  ``normalise=False``: the rows of the sum
        itself, rounded to the activation type (the stream as the input of a product)."""
        n = stream.num_tokens if rows is None else (num_rows if num_rows is not None else rows.numel())
        out = torch.empty((n, self.size), dtype=self.ctx.dtype, device=self.ctx.device)
        keep = rows is None
        extra = {}
        if stream.pending is not None and stream.pending_norm is not None:
            extra.update(post_weight=stream.pending_norm[0], post_eps=stream.pending_norm[1])
        if stream.add_source:
            if stream.embed is not None:
                raise ValueError("the embedding cannot be added again before it was read once")
            extra.update(add_ids=stream.source[0], add_table=stream.source[1])
        if stream.add_vector is not None:
            extra.update(add_vector=stream.add_vector)
        weight = self.weight if normalise else None
        if stream.embed is not None:
            ids, table = stream.embed
            if keep:
                stream.resid = torch.empty((stream.num_tokens, self.size), dtype=torch.float32,
                                           device=self.ctx.device)
            self.ops.fused_norm(out, weight, self.eps, resid=stream.resid if keep else None,
                                pending=stream.pending, ids=ids, table=table, rows=rows, write_resid=keep,
                                num_rows=n, **extra)
            if keep:
                stream.embed = None
        else:
            self.ops.fused_norm(out, weight, self.eps, resid=stream.resid, pending=stream.pending,
                                rows=rows, write_resid=keep, num_rows=n, **extra)
        if keep:
            stream.pending = None
            stream.pending_norm = None
            stream.add_source = False
            stream.add_vector = None
        return out


register_part("norm", "rmsnorm", RMSNorm)
