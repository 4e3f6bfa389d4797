"""Nizazen as a blueprint of parts.

A decoder whose residual stream has several lanes: every sub-layer reads a
learned mixture of the lanes through an RMS norm and writes its output, scaled
per channel, back into all of them while the lanes are mixed among themselves
(``parts/lanes.py``).  Layers differ: the mixer is windowed attention with q and
k normed over their whole projection, or latent attention; the feed-forward is
a dense gated one (tanh-form GELU, biases), a mixture of clamped gated experts,
or absent.  At the end the lanes are added, normed, and the logits squashed by
a tanh.  Tensor names: ``embed``, ``l<i>.norm1`` / ``.norm2`` / ``.ls1`` /
``.ls2`` / ``.hc1.*`` / ``.hc2.*`` / ``.mix.*`` / ``.mlp.*``, ``final.norm``,
``head``.
"""

from __future__ import annotations

from ..config.nizazen import (DenseMLPConfig, ExpertsMLPConfig, LatentAttentionConfig, NizazenConfig,
                              WindowAttentionConfig)
from ..engine.blueprint import LayerSpec, ModelBlueprint, PartSpec, RunSpec
from ..registry import register_architecture

# The configuration gives no longest sequence, and nothing in the design depends on one.
NO_POSITION_LIMIT = 1 << 30


def nizazen_blueprint(cfg: NizazenConfig) -> ModelBlueprint:
    H, eps = cfg.width, cfg.norm_eps
    lanes = cfg.streams or 1

    def connection(p: str, q: int) -> PartSpec:
        """The connection of sub-layer q (1 mixer, 2 feed-forward) of layer p to the lanes; without ``streams`` in
        the configuration only the norm and the per-channel scale exist."""
        names = dict(tensor=f"{p}.norm{q}", gain=f"{p}.ls{q}")
        if cfg.streams is not None:
            names.update(read=f"{p}.hc{q}.in", mix=f"{p}.hc{q}.mix", back=f"{p}.hc{q}.out")
        return PartSpec("norm", "lanes_rmsnorm", dict(size=H, eps=eps, lanes=lanes, **names))

    layers = []
    for i, L in enumerate(cfg.layers):
        p, m = f"l{i}", L.mixer
        if isinstance(m, WindowAttentionConfig):
            mixer = PartSpec("mixer", "qk_normed_attention",
                             dict(hidden_size=H, n_heads=m.heads, n_kv_heads=m.kv_heads, head_dim=m.dim,
                                  v_head_dim=m.vdim, scale=m.scale, eps=eps, window=m.window), f"{p}.mix")
        elif isinstance(m, LatentAttentionConfig):
            mixer = PartSpec("mixer", "latent_attention",
                             dict(hidden_size=H, n_heads=m.heads, head_dim=m.dim, v_head_dim=m.vdim, kv_rank=m.kv_rank,
                                  scale=m.scale, eps=eps, window=m.window), f"{p}.mix")
        else:
            raise TypeError(f"layer {i}: unknown mixer configuration {type(m).__name__}")
        parts = dict(norm1=connection(p, 1), mixer=mixer)
        f = L.mlp
        if isinstance(f, DenseMLPConfig):
            parts["feed_forward"] = PartSpec("feed_forward", "gated_mlp",
                                             dict(hidden_size=H, intermediate_size=f.ff, activation="gelu_tanh", bias=True),
                                             f"{p}.mlp")
        elif isinstance(f, ExpertsMLPConfig):
            parts["feed_forward"] = PartSpec("feed_forward", "routed_experts",
                                             dict(hidden_size=H, n_experts=f.experts, top=f.top, expert_ff=f.ff,
                                                  correction=False, expert_act="clamped_swish", limit=f.limit,
                                                  router_bias=True), f"{p}.mlp")
        if f is not None:
            parts["norm2"] = connection(p, 2)
        layers.append(LayerSpec("lanes_prenorm", parts))
    return ModelBlueprint(
        hidden_size=H,
        vocab_size=cfg.vocab,
        embedding=PartSpec("embedding", "token_table", dict(vocab_size=cfg.vocab, hidden_size=H, tensor="embed")),
        positions={},
        layers=layers,
        schedule=[RunSpec(i) for i in range(len(layers))],
        # the final norm reads the lanes added up
        final_norm=PartSpec("norm", "lanes_rmsnorm", dict(size=H, eps=eps, lanes=lanes, tensor="final.norm")),
        head=PartSpec("head", "linear_head", dict(vocab_size=cfg.vocab, hidden_size=H, tensor="head",
                                                  softcap=cfg.logit_softcap)),
        max_positions=NO_POSITION_LIMIT,
        lanes=lanes,
    )


register_architecture("Nizazen", NizazenConfig, nizazen_blueprint)
