"""Lonasun as a blueprint of parts.

A decoder of pre-norm layers (RMS norm whose gain is kept as an offset from one);
every layer's mixer is attention with a short convolution on q, k and v, a
partial rotation, chunked visibility and an output gate; its feed-forward is a
mixture of relu^2 experts with identity experts and a shared expert, or absent.
A span of layers may run several times in a row with the same weights, each run
with a cache of its own; every pass of the span starts by sending the residual
stream and the embedding output through one matrix.  Tensor names: ``embed``,
``loop.in``, ``l<i>.norm1`` / ``.norm2`` / ``.mix.*`` / ``.mlp.*``,
``final.norm``, ``head``.
"""

from __future__ import annotations

from ..config.lonasun import LonasunConfig
from ..engine.blueprint import LayerSpec, ModelBlueprint, PartSpec, RunSpec
from ..registry import register_architecture

# The configuration gives no longest sequence: the rotation tables are built for what the first cache asks for.
NO_POSITION_LIMIT = 1 << 30


def lonasun_blueprint(cfg: LonasunConfig) -> ModelBlueprint:
    H = cfg.width
    positions = {}
    layers = []
    for i, L in enumerate(cfg.layers):
        p, m = f"l{i}", L.mixer
        rope = None
        if m.rot_dims:
            rope = f"rot{m.rot_dims}@{m.rot_base!r}"
            positions.setdefault(rope, PartSpec("position", "rotary_half",
                                                dict(head_dim=m.rot_dims, theta=m.rot_base,
                                                     max_positions=NO_POSITION_LIMIT)))
        parts = dict(
            norm1=PartSpec("norm", "rmsnorm", dict(size=H, eps=cfg.norm_eps, unit_offset=True, tensor=f"{p}.norm1")),
            mixer=PartSpec("mixer", "conv_gated_attention",
                           dict(hidden_size=H, n_heads=m.heads, n_kv_heads=m.kv_heads, head_dim=m.dim, v_head_dim=m.vdim,
                                taps=m.conv, scale=m.scale, position=rope, rot_dims=m.rot_dims, chunk=m.chunk),
                           f"{p}.mix"),
            # a layer without a feed-forward may or may not carry its second norm's weight; it never runs
            norm2=PartSpec("norm", "rmsnorm", dict(size=H, eps=cfg.norm_eps, unit_offset=True, tensor=f"{p}.norm2",
                                                   optional=L.mlp is None)),
        )
        if L.mlp is not None:
            f = L.mlp
            parts["feed_forward"] = PartSpec("feed_forward", "routed_experts",
                                             dict(hidden_size=H, n_experts=f.experts, n_identity=f.identity, top=f.top,
                                                  expert_ff=f.expert_ff, shared_ff=f.shared_ff), f"{p}.mlp")
        layers.append(LayerSpec("prenorm", parts))
    stream_ops = {}
    if cfg.loop_times:
        stream_ops["loop_in"] = PartSpec("stream_op", "reinject_embedding", dict(hidden_size=H, tensor="loop.in"))
    schedule = [RunSpec(i, before="loop_in" if starts else None) for i, starts in cfg.layer_runs()]
    return ModelBlueprint(
        hidden_size=H,
        vocab_size=cfg.vocab,
        embedding=PartSpec("embedding", "token_table", dict(vocab_size=cfg.vocab, hidden_size=H, tensor="embed")),
        positions=positions,
        layers=layers,
        schedule=schedule,
        final_norm=PartSpec("norm", "rmsnorm", dict(size=H, eps=cfg.norm_eps, unit_offset=True, tensor="final.norm")),
        head=PartSpec("head", "linear_head", dict(vocab_size=cfg.vocab, hidden_size=H, tensor="head")),
        max_positions=NO_POSITION_LIMIT,
        stream_ops=stream_ops,
    )


register_architecture("Lonasun", LonasunConfig, lonasun_blueprint)
