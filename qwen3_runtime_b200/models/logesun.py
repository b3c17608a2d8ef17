"""Logesun expressed as data for the generic decoder.

Blocks norm both the input and the output of each sublayer (``sandwich_norm``).  The mixer is
attention through a low-rank latent with a sliding window and a sink, rotating interleaved pairs
of a shared key part; the feed-forward is a dense SwiGLU layer or routed clamped experts with a
shared one, or absent.  A run of layers may be repeated with the same weights: every pass has a
cache layer of its own and every pass but the first starts from the stream plus the embedding.
Tensor names: ``embed``, ``l<i>.norm1 | norm1b | norm2 | norm2b``, ``l<i>.mix.*``, ``l<i>.mlp.*``,
``final.norm``, ``head``.
"""

from __future__ import annotations

from ..config.logesun_config import (ExpertConfig, FeedForwardConfig, LatentAttentionConfig, LogesunConfig,
                                     LogesunLayerConfig)
from ..config.registry import register_architecture
from ..config.spec import LayerRun, ModelSpec, PartSpec


def _mixer_spec(cfg: LogesunConfig, m: LatentAttentionConfig) -> PartSpec:
    position = PartSpec("rope_interleaved", dict(rotary_dim=m.rot_dims, theta=m.rot_base))
    return PartSpec("latent_attention", dict(
        hidden_size=cfg.width, num_heads=m.heads, dim=m.dim, rot_dim=m.rot_dim, vdim=m.vdim, q_rank=m.q_rank,
        kv_rank=m.kv_rank, eps=cfg.norm_eps, scale=m.scale, window=m.window, sink=True, position=position))


def _feed_forward_spec(cfg: LogesunConfig, f: FeedForwardConfig) -> PartSpec:
    if f.kind == "dense":
        return PartSpec("gated_mlp", dict(hidden_size=cfg.width, intermediate_size=f.ff, activation="silu",
                                          names=dict(gate="gate", up="up", down="down")))
    return PartSpec("routed_experts", dict(
        hidden_size=cfg.width, num_experts=f.experts, top=f.top, expert_size=f.expert.ff, limit=f.expert.limit,
        alpha=1.702, up_offset=1.0, score="sigmoid", renormalize=False, weight_on="input",
        shared_size=f.shared.ff if f.shared else 0, shared_limit=f.shared.limit if f.shared else None))


def logesun_spec(cfg: LogesunConfig) -> ModelSpec:
    norm = PartSpec("rmsnorm", dict(size=cfg.width, eps=cfg.norm_eps, weight_name=""))
    blocks = []
    for layer in cfg.layers:
        params = dict(mixer=_mixer_spec(cfg, layer.mixer), mixer_norm=norm, mixer_out_norm=norm,
                      mixer_prefix="mix.", mixer_norm_prefix="norm1", mixer_out_norm_prefix="norm1b",
                      feed_forward=None)
        if layer.mlp is not None:
            params.update(feed_forward=_feed_forward_spec(cfg, layer.mlp), feed_forward_norm=norm,
                          feed_forward_out_norm=norm, feed_forward_prefix="mlp.", feed_forward_norm_prefix="norm2",
                          feed_forward_out_norm_prefix="norm2b")
        blocks.append(PartSpec("sandwich_norm", params))
    order = tuple(LayerRun(block=layer, cache=run, add_embedding=again)
                  for run, (layer, again) in enumerate(cfg.run_order()))
    return ModelSpec(vocab_size=cfg.vocab, hidden_size=cfg.width, blocks=tuple(blocks), order=order,
                     final_norm=norm, tie_word_embeddings=False, embed_name="embed", head_name="head",
                     block_prefix="l{index}.", final_norm_prefix="final.norm")


def tiny_logesun_config() -> LogesunConfig:
    """A small model with every branch of the design: a dense and a routed feed-forward, a layer
    without one, and a loop."""
    mixer = LatentAttentionConfig(heads=2, dim=16, rot_dim=8, vdim=24, q_rank=24, kv_rank=32, scale=0.2,
                                  rot_dims=8, rot_base=10000.0, window=24)
    moe = FeedForwardConfig(kind="moe", experts=4, top=2, expert=ExpertConfig(16, 3.0), shared=ExpertConfig(24, 2.0))
    layers = (LogesunLayerConfig("latent_attention", mixer, FeedForwardConfig(kind="dense", ff=48)),
              LogesunLayerConfig("latent_attention", mixer, moe),
              LogesunLayerConfig("latent_attention", mixer, None))
    return LogesunConfig(vocab=64, width=40, norm_eps=1e-5, layers=layers, loop_start=1, loop_stop=3, loop_times=2)


register_architecture(LogesunConfig.architecture, LogesunConfig, logesun_spec, tiny_config=tiny_logesun_config)
