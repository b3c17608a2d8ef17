"""Softmax attention over a sliding window with a short causal convolution on q, k and v.

    q, k, v = W_q h, W_k h, W_v h                      (one product)
    y_t[c] = sum_j w[c, j] * u_(t - taps + 1 + j)[c]    on every channel of q, k and v
    q, k rotated: pairs (i, i + dims / 2) of the first ``dims`` elements of a head
    score = (q . k) * scale;  position i sees j with 0 <= i - j < window;  softmax;  W_o

Query heads share key/value heads in groups; keys and values may have unlike sizes per head.  The
cache holds the rotated keys and the values in pages (only a window of them) and, in a state slot,
the last ``taps - 1`` rows of the q/k/v product of every request, so that a step continues the
convolution where the last one stopped.  One kernel does convolution, rotation and cache write.
The part is a :class:`BranchMixer`: it runs alone or as a branch of the ``parallel`` mixer.
"""

from __future__ import annotations

import torch

from ..cache.layout import KVLayerSpec, StateLayerSpec
from ..config.spec import PartSpec
from .base import BuildContext, ParamSpec, StepContext, build_part, register_part
from .linear_state import BranchMixer


class ConvWindowAttention(BranchMixer):
    def __init__(self, spec, ctx: BuildContext):
        super().__init__(spec, ctx)
        self.hidden_size = int(spec["hidden_size"])
        self.num_heads = int(spec["num_heads"])
        self.num_kv_heads = int(spec["num_kv_heads"])
        self.dim = int(spec["dim"])
        self.vdim = int(spec["vdim"])
        self.scale = float(spec["scale"])
        self.taps = int(spec.get("taps") or 0)
        self.window = spec.get("window") or None
        if self.num_heads % self.num_kv_heads:
            raise ValueError("num_heads must be a multiple of num_kv_heads")
        if self.dim > 256 or self.vdim > 256:
            raise ValueError(f"dim={self.dim}, vdim={self.vdim}: the attention kernels take sizes up to 256")
        if self.taps > 16:
            raise ValueError(f"taps={self.taps}: the convolution kernel takes up to 16")
        pos_spec = spec.get("position") or PartSpec("none")
        self.position = build_part("position", pos_spec, ctx)
        if self.position.style == "rotary" and getattr(self.position, "pairing", "half") != "half":
            raise ValueError("conv_window_attention rotates pairs (i, i + dims / 2)")
        self.channels = (self.num_heads + self.num_kv_heads) * self.dim + self.num_kv_heads * self.vdim
        self.in_weight = self.o_weight = self.conv_weight = None

    def param_specs(self):
        H, G, D, Dv, W = self.num_heads, self.num_kv_heads, self.dim, self.vdim, self.hidden_size
        specs = {"q": ParamSpec((H * D, W)), "k": ParamSpec((G * D, W)), "v": ParamSpec((G * Dv, W)),
                 "o": ParamSpec((W, H * Dv))}
        if self.taps:
            specs.update({"q.conv": ParamSpec((H * D, self.taps), "matrix_f32"),
                          "k.conv": ParamSpec((G * D, self.taps), "matrix_f32"),
                          "v.conv": ParamSpec((G * Dv, self.taps), "matrix_f32")})
        return specs

    def load(self, tensors):
        self.in_weight = torch.cat([tensors["q"], tensors["k"], tensors["v"]], dim=0).contiguous()
        self.o_weight = tensors["o"].contiguous()
        if self.taps:
            # tap-major [taps, channels]: the kernel's neighbouring channels read neighbouring weights
            self.conv_weight = torch.cat([tensors["q.conv"], tensors["k.conv"], tensors["v.conv"]], dim=0).t().contiguous()

    def input_weight(self):
        return self.in_weight

    def release_input_weight(self):
        self.in_weight = None

    def context_size(self):
        return self.num_heads * self.vdim

    def output_weight(self):
        return self.o_weight

    def kernel_groups(self):
        groups = ["short_conv", "attention_generic"]
        groups += ["gemm_f32"] if self.ctx.dtype == torch.float32 else ["gemm_small_m", "gemm_stream"]
        if self._specialised():
            groups += ["attention_decode", "attention_prefill"]
        return groups

    def _specialised(self) -> bool:
        """Keys and values of one size that the split-KV decode kernel and the tensor-core prompt kernel
        take (ops.paged_attention sends a dense output there)."""
        return (self.ctx.dtype == torch.bfloat16 and self.dim == self.vdim and self.dim in (64, 128)
                and self.num_heads // self.num_kv_heads <= 16)

    def step_choosers(self):
        """Into how many slices the split-KV decode kernel cuts the longest sequence's keys."""
        model = getattr(self.ops, "decode_slices_for", None)
        if model is None or not self._specialised():
            return {}
        nkv, D, window = self.num_kv_heads, self.dim, self.window
        return {("decode_slices", nkv, D, window): lambda kv_lens: model(kv_lens, nkv, D, window)}

    def cache_spec(self):
        pages = KVLayerSpec(self.num_kv_heads, self.dim, self.window, value_dim=self.vdim)
        state = StateLayerSpec((self.taps - 1, self.channels)) if self.taps > 1 else None
        return (pages, state)

    def position_limit(self):
        return self.position.position_limit()

    def context(self, proj, step: StepContext, cache, out, out_scale):
        ops = self.ops
        pages, conv = cache
        T = proj.shape[0]
        H, G, D, Dv = self.num_heads, self.num_kv_heads, self.dim, self.vdim
        q = torch.empty((T, H * D), dtype=proj.dtype, device=proj.device)
        block_table = step.block_tables[pages.paged_index]
        inv = self.position.device_inverse_frequencies() if self.position.style == "rotary" else None
        # the values are stored times the output scale: a weighted sum of them is the scaled context
        ops.conv_rope_store(proj, num_heads=H, num_kv_heads=G, head_dim=D, value_dim=Dv, conv_weight=self.conv_weight,
                            conv_state=conv.state if conv is not None else None, inv_freq=inv,
                            positions=step.positions, token_seq=step.token_seq, cu_seqlens=step.cu_seqlens,
                            state_slots=step.state_slots, num_seqs=step.num_seqs, block_table=block_table,
                            k_pages=pages.k_pages, v_pages=pages.v_pages, page_size=pages.page_size, q_out=q,
                            value_scale=out_scale, write_kv=pages.writes)
        ops.paged_attention(q, q.stride(0), num_heads=H, num_kv_heads=G, head_dim=D, k_pages=pages.k_pages,
                            v_pages=pages.v_pages, block_table=block_table, token_seq=step.token_seq,
                            positions=step.positions, out=out, page_size=pages.page_size, scale=self.scale,
                            window=self.window, step=step, value_dim=Dv,
                            decode_slices=step.choices.get(("decode_slices", G, D, self.window)))


register_part("mixer", "conv_window_attention", ConvWindowAttention)
