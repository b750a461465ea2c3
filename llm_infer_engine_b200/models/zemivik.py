"""The Zemivik design as a `ModelSpec`.

Embedding stage: the token embedding times a constant plus a learned position vector, then an RMS norm. Every
layer is h += norm(mixer(h)) and, where the layer has a feed-forward, h += norm(ff(h)): the norms sit on the
branch outputs and the branches read the stream itself. The one mixer is gated grouped-query attention without
rotation (whole-projection query/key norms, a window that keeps the sequence's first tokens, a softmax with a
sink, values blended with those of the first blending layer, an output gate); the feed-forward is
down(relu(up x + b)^2) + b. Then a final norm and a head of its own. Layers are listed one by one in the
configuration, each with its own sizes. Checkpoint names: `embed`, `pos`, `embed.norm`, `l<i>.norm1|norm2`,
`l<i>.mix.{q,k,v,g,o,q.norm,k.norm,vmix}`, `l<i>.mlp.{up,up.b,down,down.b}`, `final.norm`, `head`.
"""
from __future__ import annotations

from ..config.registry import register_architecture
from ..config.spec import LayerCall, LayerSpec, ModelSpec, PartSpec
from ..config.zemivik import ZemivikConfig


def zemivik_spec(cfg: ZemivikConfig) -> ModelSpec:
    norm = PartSpec("rmsnorm", {"size": cfg.width, "eps": cfg.norm_eps, "weight_name": ""})
    layers = []
    seen_blend = False
    for layer in cfg.layers:
        m = layer.mixer
        blend = None
        if m.v_mix:
            blend = "blend" if seen_blend else "first"
            seen_blend = True
        mixer = PartSpec("gated_attention", {
            "hidden": cfg.width, "n_heads": m.heads, "n_kv_heads": m.kv_heads, "head_dim": m.dim, "v_head_dim": m.vdim,
            "scale": m.scale, "window": m.mask.size if m.mask else 0, "keep_first": m.mask.keep_first if m.mask else 0,
            "sink": True, "qk_norm_eps": cfg.norm_eps, "gate": True, "value_blend": blend})
        if layer.mlp is None:
            layers.append(LayerSpec("branch_norm_mixer", parts={"mixer": mixer, "mixer_norm": norm},
                                    names={"mixer": "mix", "mixer_norm": "norm1"}))
        else:
            ff = PartSpec("dense_mlp", {"hidden": cfg.width, "intermediate": layer.mlp.ff, "activation": "relu2",
                                        "bias": True})
            layers.append(LayerSpec("branch_norm", mixer=mixer, feed_forward=ff, mixer_norm=norm, feed_forward_norm=norm,
                                    names={"mixer": "mix", "feed_forward": "mlp", "mixer_norm": "norm1",
                                           "feed_forward_norm": "norm2"}))
    stage = PartSpec("embedding_stage", {"size": cfg.width, "scale": cfg.embedding_scale, "positions": cfg.max_positions,
                                         "norm_eps": cfg.norm_eps, "names": {"positions": "pos", "norm": "embed.norm"}})
    return ModelSpec(
        hidden_size=cfg.width, vocab_size=cfg.vocab, max_position=cfg.max_positions, layers=layers,
        schedule=[LayerCall(i) for i in range(len(layers))], final_norm=norm, tie_head=False, embedding_name="embed",
        layer_prefix="l{i}.", final_norm_name="final.norm", head_name="head", after_embedding=stage,
        after_embedding_name="",
        # a checkpoint may hold the blend scalar of a layer that does not blend; nothing reads it
        ignore_unexpected=(r"l\d+\.mix\.vmix$",))


register_architecture("Zemivik", ZemivikConfig, zemivik_spec)
