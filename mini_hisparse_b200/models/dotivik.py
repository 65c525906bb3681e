"""Dotivik as data: the ModelSpec of a DotivikConfig and its registry entry.

Every layer is a parallel block: one layer norm (weight, no bias) whose output both the mixer and the
gated gelu feed-forward read, their outputs added to the stream together.  The mixer is attention with
two score maps per head (the second subtracted from the first; capped scores, interleaved rotation) or
latent attention (a low-rank row per position, a rotated key part shared by the heads, a sliding
window).  A run of layers may repeat: every pass has caches of its own (a run entry each) and opens with
x <- W_in [x ; embedding output], a part of the model as a whole that the first entry of the pass runs
first.  The output head is the embedding table.  Tensor names: embed, loop.in,
l<i>.{norm1, mix.*, mlp.{gate,up,down}}, final.norm.
"""
from __future__ import annotations

from ..config.dotivik import DotivikConfig
from ..config.registry import register_architecture
from ..parts.spec import LayerSpec, ModelSpec, PartSpec, RunEntry

STREAM_BUFFER = "stream_cat"


def dotivik_spec(cfg: DotivikConfig) -> ModelSpec:
    W = cfg.width
    norm = PartSpec.make("layernorm", width=W, eps=cfg.eps, weight_name="")
    layers = []
    for i, layer in enumerate(cfg.layers):
        m = layer.mixer
        if layer.type == "attention":
            position = (PartSpec.make("rotary", head_dim=m.dim, theta=m.rot_base, rotary_dim=m.rot_dims,
                                      style="interleaved") if m.rot_dims else PartSpec.make("none"))
            mixer = PartSpec.make("diff_attention", hidden_size=W, heads=m.heads, kv_heads=m.kv_heads, dim=m.dim,
                                  vdim=m.vdim, scale=m.scale, softcap=m.softcap, lambda_init=m.diff, eps=cfg.eps,
                                  window=m.window, position=position)
        else:
            position = (PartSpec.make("rotary", head_dim=m.rot_dim, theta=m.rot_base, rotary_dim=m.rot_dim,
                                      style="half_split") if m.rot_dim else PartSpec.make("none"))
            mixer = PartSpec.make("latent_attention", hidden_size=W, heads=m.heads, dim=m.dim, rot_dim=m.rot_dim,
                                  vdim=m.vdim, kv_rank=m.kv_rank, scale=m.scale, window=m.window, eps=cfg.eps,
                                  position=position)
        parts = {"norm": norm, "mixer": mixer}
        if layer.ff is not None:
            parts["feed_forward"] = PartSpec.make("glu", hidden_size=W, intermediate_size=layer.ff,
                                                  activation="gelu_tanh")
        layers.append(LayerSpec.make(f"l{i}", "parallel", parts,
                                     {"norm": "norm1", "mixer": "mix", "feed_forward": "mlp"}))
    n = len(cfg.layers)
    loop = cfg.loop
    if loop is None or loop.start == loop.stop:
        order = [RunEntry(i) for i in range(n)]
        looped = False
    else:
        order = [RunEntry(i) for i in range(loop.start)]
        for _ in range(loop.times):           # the same weights, a cache of its own for every pass
            order += [RunEntry(i, before="loop" if i == loop.start else None) for i in range(loop.start, loop.stop)]
        order += [RunEntry(i) for i in range(loop.stop, n)]
        looped = True
    shared = ()
    embedding = dict(vocab_size=cfg.vocab, hidden_size=W, weight_name="")
    if looped:
        shared = (("loop", PartSpec.make("stream_input", width=W, buffer=STREAM_BUFFER, weight_name="in"), "loop"),)
        embedding["keep"] = (STREAM_BUFFER, 2 * W, W)
    return ModelSpec(
        architecture="Dotivik", vocab_size=cfg.vocab, hidden_size=W,
        embedding=PartSpec.make("token_embedding", **embedding), embedding_name="embed",
        layers=tuple(layers), order=tuple(order), final_norm=norm, final_norm_name="final.norm",
        head=PartSpec.make("lm_head", vocab_size=cfg.vocab, hidden_size=W, tied=True, weight_name="weight"),
        head_name="head", shared=shared,
    )


register_architecture("Dotivik", DotivikConfig, dotivik_spec, replace=True)
