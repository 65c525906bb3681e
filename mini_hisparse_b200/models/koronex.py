"""Koronex as data: the ModelSpec of a KoronexConfig and its registry entry.

The embedding is scaled; every layer is a post-norm block (the norm follows the residual addition, and the
stream is scaled inside it) whose mixer is lightning attention (linear attention with a decay per head, a state per
request) or windowed grouped-query attention with a norm over the whole q and k projections, partial
rotation, a softmax sink and an output gate; a layer may have a relu-squared feed-forward, and ends
with an input from the token itself (a slice of a table shared by all layers).  An attention layer
with ``kv_from`` has no keys of its own: its run entry reads the cache of the layer it names.
Tensor names: embed, side.embed, l<i>.{norm1,norm2,mix.*,mlp.*,side.*}, final.norm, head.
"""
from __future__ import annotations

from ..config.koronex import KoronexConfig
from ..config.registry import register_architecture
from ..parts.spec import LayerSpec, ModelSpec, PartSpec, RunEntry


def koronex_spec(cfg: KoronexConfig) -> ModelSpec:
    W = cfg.width
    norm = PartSpec.make("rmsnorm", width=W, eps=cfg.eps, weight_name="")
    # how many positions an attention cache keeps: the widest window among its owner and its readers
    keep = {}
    for i, layer in enumerate(cfg.layers):
        if layer.type == "attention":
            owner = i if layer.mixer.kv_from is None else layer.mixer.kv_from
            keep[owner] = max(keep.get(owner, 0), layer.mixer.window)
    layers, order, entry_of = [], [], {}
    for i, layer in enumerate(cfg.layers):
        m = layer.mixer
        if layer.type == "lightning":
            mixer = PartSpec.make("lightning_attention", hidden_size=W, heads=m.heads, dim=m.dim, vdim=m.vdim,
                                  decay=m.decay, eps=cfg.eps)
            entry = RunEntry(i)
        else:
            owner = i if m.kv_from is None else m.kv_from
            position = (PartSpec.make("rotary", head_dim=m.dim, theta=m.rot_base, rotary_dim=m.rot_dims)
                        if m.rot_dims else PartSpec.make("none"))
            mixer = PartSpec.make("sink_attention", hidden_size=W, q_heads=m.heads, kv_heads=m.kv_heads, dim=m.dim,
                                  vdim=m.vdim, scale=m.scale, window=m.window, keep=keep[owner], eps=cfg.eps,
                                  position=position, own_kv=m.kv_from is None)
            entry = RunEntry(i) if m.kv_from is None else RunEntry(i, cache_of=entry_of[m.kv_from])
        entry_of[i] = len(order)
        order.append(entry)
        parts = {"mixer_norm": norm, "mixer": mixer}
        if layer.ff is not None:
            parts["ff_norm"] = norm
            parts["feed_forward"] = PartSpec.make("mlp_act", hidden_size=W, intermediate_size=layer.ff,
                                                  activation="relu2")
        if cfg.side_dim is not None:
            parts["side"] = PartSpec.make("token_side", hidden_size=W, dim=cfg.side_dim, column0=i * cfg.side_dim,
                                          eps=cfg.eps, table="side")
        layers.append(LayerSpec.make(f"l{i}", "post_norm", parts,
                                     {"mixer_norm": "norm1", "mixer": "mix", "ff_norm": "norm2",
                                      "feed_forward": "mlp", "side": "side"},
                                     {"alpha": cfg.alpha}))
    shared = ()
    if cfg.side_dim is not None:
        shared = (("side", PartSpec.make("token_table", vocab_size=cfg.vocab, width=len(cfg.layers) * cfg.side_dim,
                                         weight_name="embed"), "side"),)
    return ModelSpec(
        architecture="Koronex", vocab_size=cfg.vocab, hidden_size=W,
        embedding=PartSpec.make("token_embedding", vocab_size=cfg.vocab, hidden_size=W, scale=cfg.embedding_scale,
                                copy=True, weight_name=""),
        embedding_name="embed", layers=tuple(layers), order=tuple(order),
        final_norm=norm, final_norm_name="final.norm",
        head=PartSpec.make("lm_head", vocab_size=cfg.vocab, hidden_size=W, tied=False, weight_name=""),
        head_name="head", shared=shared,
    )


register_architecture("Koronex", KoronexConfig, koronex_spec, replace=True)
