"""Puladra expressed as data for the generic decoder.

Pre-norm blocks whose norms multiply by ``1 + w``, w being the stored tensor.  The mixer of a layer is
gated linear attention (``gla``) or two mixers side by side on the same input (``parallel``:
windowed softmax attention with a short convolution on q, k and v, and retention), the
feed-forward routed squared-ReLU experts with a gated shared one, or absent.  After its sublayers a
layer adds an input from the token itself (a slice of a second embedding, gated by the stream).  A
run of layers may be repeated with the same weights: every pass has cache layers of its own, and a
learned vector per pass is added to the stream before the pass's first layer.  The output head is
the embedding table, the logits are multiplied by ``logit_scale``.
Tensor names: ``embed``, ``loop.step``, ``side.embed``, ``l<i>.norm1 | norm2``, ``l<i>.mix.*``,
``l<i>.mlp.*``, ``l<i>.side.*``, ``final.norm``.
"""

from __future__ import annotations

from ..config.puladra_config import (GlaConfig, MoeConfig, ParallelConfig, PuladraConfig, PuladraLayerConfig,
                                     RetentionConfig, RotationConfig, WindowAttentionConfig)
from ..config.registry import register_architecture
from ..config.spec import LayerRun, ModelSpec, PartSpec

LOOP_TABLE = "loop.step"
SIDE_TABLE = "side.embed"


def _position(rot: RotationConfig | None) -> PartSpec:
    if rot is None:
        return PartSpec("none")
    return PartSpec("rope_neox", dict(rotary_dim=rot.dims, theta=rot.base))  # no table: any position


def _mixer_spec(cfg: PuladraConfig, layer: PuladraLayerConfig) -> PartSpec:
    m = layer.mixer
    if isinstance(m, GlaConfig):
        if not m.decay_rank:
            raise ValueError("gla: the decay's rank is not known yet; it is the row count of the stored a1 "
                             "(PuladraConfig.with_tensor_shapes)")
        return PartSpec("gla", dict(hidden_size=cfg.width, num_heads=m.heads, dim=m.dim, vdim=m.vdim, tau=m.tau,
                                    eps=cfg.norm_eps, decay_rank=m.decay_rank))
    left, right = m.left, m.right
    attention = PartSpec("conv_window_attention", dict(
        hidden_size=cfg.width, num_heads=left.heads, num_kv_heads=left.kv_heads, dim=left.dim, vdim=left.vdim,
        scale=left.scale, taps=left.conv, window=left.window, position=_position(left.rot)))
    retention = PartSpec("retention", dict(
        hidden_size=cfg.width, num_heads=right.heads, dim=right.dim, vdim=right.vdim, decay=tuple(right.decay),
        eps=cfg.norm_eps, position=_position(right.rot)))
    return PartSpec("parallel", dict(branches=(("left.", attention, m.left_scale), ("right.", retention, m.right_scale))))


def _feed_forward_spec(cfg: PuladraConfig, f: MoeConfig) -> PartSpec:
    return PartSpec("routed_experts", dict(
        hidden_size=cfg.width, num_experts=f.experts, top=f.top, expert_size=f.ff, activation="relu2",
        score="softmax_chosen", weight_on="output", shared_size=f.shared_ff,
        shared_gate="sigmoid" if f.shared_ff else None))


def puladra_spec(cfg: PuladraConfig) -> ModelSpec:
    norm = PartSpec("rmsnorm", dict(size=cfg.width, eps=cfg.norm_eps, weight_name="", weight_offset=1.0))
    blocks = []
    for i, layer in enumerate(cfg.layers):
        params = dict(mixer=_mixer_spec(cfg, layer), mixer_norm=norm, mixer_prefix="mix.", mixer_norm_prefix="norm1")
        if layer.mlp is not None:
            params.update(feed_forward=_feed_forward_spec(cfg, layer.mlp), feed_forward_norm=norm,
                          feed_forward_prefix="mlp.", feed_forward_norm_prefix="norm2")
        if cfg.side_dim:
            params.update(side_input=PartSpec("gated_token_input", dict(
                hidden_size=cfg.width, dim=cfg.side_dim, offset=i * cfg.side_dim, table=SIDE_TABLE, eps=cfg.norm_eps)),
                side_input_prefix="side.")
        blocks.append(PartSpec("pre_norm", params))
    order = tuple(LayerRun(block=layer, cache=run, add_row=(LOOP_TABLE, rep) if rep is not None else None)
                  for run, (layer, rep) in enumerate(cfg.run_order()))
    tables = []
    if cfg.loop_times:
        tables.append((LOOP_TABLE, (cfg.loop_times, cfg.width), "matrix_f32"))
    if cfg.side_dim:
        tables.append((SIDE_TABLE, (cfg.vocab, len(cfg.layers) * cfg.side_dim), "matrix"))
    return ModelSpec(vocab_size=cfg.vocab, hidden_size=cfg.width, blocks=tuple(blocks), order=order,
                     final_norm=norm, tie_word_embeddings=True, embed_name="embed", head_name="head",
                     block_prefix="l{index}.", final_norm_prefix="final.norm", logit_scale=cfg.logit_scale,
                     shared_tables=tuple(tables))


def tiny_puladra_config() -> PuladraConfig:
    """A small model with every branch of the design: both mixers, a layer without a feed-forward,
    a loop, the per-layer token input."""
    gla = GlaConfig(heads=2, dim=16, vdim=24, tau=8.0, decay_rank=8)
    par = ParallelConfig(
        left=WindowAttentionConfig(heads=4, kv_heads=2, dim=16, vdim=24, scale=0.25, conv=3,
                                   rot=RotationConfig(8, 10000.0), window=24),
        right=RetentionConfig(heads=2, dim=16, vdim=8, decay=(0.9, 0.99), rot=RotationConfig(16, 1000.0)),
        left_scale=0.7, right_scale=0.6)
    moe = MoeConfig(experts=4, top=2, ff=16, shared_ff=24)
    layers = (PuladraLayerConfig("gla", gla, moe), PuladraLayerConfig("parallel", par, moe),
              PuladraLayerConfig("gla", gla, None))
    return PuladraConfig(vocab=64, width=40, norm_eps=1e-5, layers=layers, logit_scale=1.5, side_dim=8,
                         loop_start=0, loop_stop=2, loop_times=2)


register_architecture(PuladraConfig.architecture, PuladraConfig, puladra_spec, tiny_config=tiny_puladra_config)
