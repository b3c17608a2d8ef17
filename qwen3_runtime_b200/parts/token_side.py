"""A per-layer input from the token itself, added to the stream after the block's sublayers.

    e = table[token][offset : offset + dim]          a slice of a second embedding, one slice per layer
    g = gelu_tanh(W_gate x) * e                       x: the stream (the residual sum, not normalised)
    y = W_proj g                                      x <- x + y / sqrt(mean(y^2) + eps) * w

The part folds what is pending into the residual sum, reads the sum in the activation type, and
leaves ``y`` on the stream as the pending output together with the norm that is to be applied to it
(``ResidualStream.pending_norm``): whichever norm reads the stream next normalises it, adds it and
normalises the sum in one kernel.  The table is a shared table of the model
(``ModelSpec.shared_tables``), found under ``table`` in ``BuildContext.shared``.
"""

from __future__ import annotations

import torch

from .base import BuildContext, ParamSpec, Part, ResidualStream, StepContext, register_part


class GatedTokenInput(Part):
    category = "side_input"

    def __init__(self, spec, ctx: BuildContext):
        super().__init__(spec, ctx)
        self.hidden_size = int(spec["hidden_size"])
        self.dim = int(spec["dim"])
        self.offset = int(spec["offset"])
        self.table_name = str(spec["table"])
        self.eps = float(spec["eps"])
        self.gate = self.proj = self.norm_weight = None

    def param_specs(self):
        return {"gate": ParamSpec((self.dim, self.hidden_size)), "proj": ParamSpec((self.hidden_size, self.dim)),
                "norm": ParamSpec((self.hidden_size,), "vector")}

    def load(self, tensors):
        self.gate = tensors["gate"].contiguous()
        self.proj = tensors["proj"].contiguous()
        self.norm_weight = tensors["norm"].contiguous()

    def kernel_groups(self):
        return ["norm"] + (["gemm_f32"] if self.ctx.dtype == torch.float32 else ["gemm_small_m", "gemm_stream"])

    def forward(self, stream: ResidualStream, step: StepContext, fold) -> None:
        """``fold(stream)`` adds what is pending to the residual sum and returns the sum in the
        activation type (a norm part's ``add_norm(stream, normalise=False)``)."""
        ops = self.ops
        x = fold(stream)
        gate = ops.linear(x, self.gate)
        g = torch.empty_like(gate)
        ops.gelu_gate_rows(gate, step.token_ids, self.ctx.shared[self.table_name], self.offset, g)
        stream.pending = ops.linear(g, self.proj)
        stream.pending_norm = (self.norm_weight, self.eps)


register_part("side_input", "gated_token_input", GatedTokenInput)
