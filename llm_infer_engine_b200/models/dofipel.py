"""The Dofipel design as a `ModelSpec`.

x = E[token]; every layer is u = dyt(x), x += mixer(u) + ff(u) with ONE Dynamic-Tanh norm (tanh(alpha x) w + b, no
mean, no variance) whose output both branches read; logits = E dyt(x) * logit_scale. Two mixers: grouped-query
attention without rotation (capped scores, a learned bias by bucketed distance, a sliding window, a learned sink per
head) and latent attention (keys and values made from a cached low-rank latent plus one rotated key part shared by
all heads, causal, sigmoid output gate), whose layers may read an earlier layer's latent. Two feed-forwards: a gated
one with the tanh form of gelu, and routed experts (silu) with a shared expert. Layers are listed one by one in the
configuration, each with its own sizes. Checkpoint names: `embed`, `l<i>.norm1{,.alpha,.b}`,
`l<i>.mix.{q,k,v,rel,sink,o}` or `l<i>.mix.{q,dkv,dkv.norm,uk,uv,g,o}`, `l<i>.mlp.{gate,up,down}` or
`l<i>.mlp.{router,router.b,e<j>.{gate,up,down},shared.{gate,up,down}}`, `final.norm{,.alpha,.b}`.
"""
from __future__ import annotations

from ..config.dofipel import DenseFF, DofipelConfig, LatentAttention, WindowAttention
from ..config.registry import register_architecture
from ..config.spec import LayerCall, LayerSpec, ModelSpec, PartSpec

NO_POSITION_LIMIT = 1 << 20       # the design has no table of positions; the engine's own limit decides


def dofipel_spec(cfg: DofipelConfig) -> ModelSpec:
    norm = PartSpec("dynamic_tanh", {"size": cfg.width, "weight_name": "", "alpha_name": "alpha", "bias_name": "b"})
    gated_names = {"gate": "gate", "up": "up", "down": "down"}
    layers, schedule = [], []
    for i, layer in enumerate(cfg.layers):
        m = layer.mixer
        if isinstance(m, WindowAttention):
            mixer = PartSpec("gated_attention", {
                "hidden": cfg.width, "n_heads": m.heads, "n_kv_heads": m.kv_heads, "head_dim": m.dim, "v_head_dim": m.vdim,
                "scale": m.scale, "window": m.window, "sink": "learned", "softcap": m.softcap,
                "distance_bias": {"rows": None, "far": m.bias_max}})
            schedule.append(LayerCall(i))
        else:
            assert isinstance(m, LatentAttention)
            mixer = PartSpec("latent_attention", {
                "hidden": cfg.width, "n_heads": m.heads, "head_dim": m.dim, "rot_dim": m.rot_dim, "v_head_dim": m.vdim,
                "kv_rank": m.kv_rank, "scale": m.scale, "rot_base": m.rot_base, "rot_dims": m.rot_dims,
                "norm_eps": cfg.norm_eps, "gate": True, "owns_latent": m.kv_from is None, "out_float32": True})
            schedule.append(LayerCall(i, cache_of=m.kv_from))
        parts = {"mixer": mixer, "norm": norm}
        names = {"mixer": "mix", "norm": "norm1"}
        if layer.mlp is not None:
            if isinstance(layer.mlp, DenseFF):
                parts["feed_forward"] = PartSpec("swiglu", {"hidden": cfg.width, "intermediate": layer.mlp.ff,
                                                            "activation": "gelu_tanh", "names": gated_names,
                                                            "out_float32": True})
            else:
                f = layer.mlp
                parts["feed_forward"] = PartSpec("routed_experts", {
                    "hidden": cfg.width, "n_experts": f.experts, "top": f.top, "expert_ff": f.expert_ff,
                    "activation": "silu", "router_bias": True, "shared_ff": f.shared_ff})
            names["feed_forward"] = "mlp"
        layers.append(LayerSpec("parallel" if layer.mlp is not None else "parallel_mixer", parts=parts, names=names))
    return ModelSpec(
        hidden_size=cfg.width, vocab_size=cfg.vocab, max_position=NO_POSITION_LIMIT, layers=layers, schedule=schedule,
        final_norm=norm, tie_head=True, embedding_name="embed", layer_prefix="l{i}.", final_norm_name="final.norm",
        head_name="head", after_head=PartSpec("scale", {"factor": cfg.logit_scale}))


register_architecture("Dofipel", DofipelConfig, dofipel_spec)
