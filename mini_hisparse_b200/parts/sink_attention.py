"""Grouped-query attention with a norm over the whole q and k projections, a sliding window, a
softmax sink per head and an output gate, over keys and values of different widths."""
from __future__ import annotations

import torch

from ..kernels import api as K
from .attention import ITEM_INTS, ROW_TILE, AttentionPlanner, AttentionShape
from .base import CacheView, Mixer, Product, StepContext
from .registry import POSITIONS, register_mixer
from .spec import PagedKVNeed, ParamSpec, PartSpec


@register_mixer("sink_attention")
class SinkAttention(Mixer):
    """q = W_q h [q_heads x dim], k = W_k h [kv_heads x dim], v = W_v h [kv_heads x vdim], no biases.

    * q and k are each RMS-normalised as ONE vector spanning every head (the statistic is not per head; the
      weight is a plain multiplier as long as that vector), and only then cut into heads and rotated by the
      position part.
    * score = (q . k) * scale; a query at position i sees the keys at positions i - window + 1 ... i.
    * The softmax's denominator has one more term, exp(sink_h): a learned per-head logit that stands for no
      position (it brings neither a key nor a value) and is used as stored, without the score scale.
    * The heads' outputs are multiplied by sigmoid(W_g h) and projected by W_o.
    * ``own_kv`` False: the layer has no k and v tensors; it reads the cache of another run entry
      (RunEntry.cache_of) with its own queries, window, sink and gate.

    Parameters: hidden_size, q_heads, kv_heads, dim, vdim, scale, window (None: all keys), keep
    (how many positions the CACHE keeps: at least the window of every reader of the cache; None:
    all), eps, position (a PartSpec), own_kv.  Tensors: q, k, v, q.norm, k.norm, sink, g, o.
    Scores, softmax, norms and angles are float32; q, k and v are kept in the compute dtype.
    """

    def __init__(self, spec: PartSpec, rt=None):
        super().__init__(spec, rt)
        self.hidden = int(spec["hidden_size"])
        self.nq, self.nkv = int(spec["q_heads"]), int(spec["kv_heads"])
        self.dk, self.dv = int(spec["dim"]), int(spec["vdim"])
        self.scale = float(spec["scale"])
        self.window = spec.get("window")
        self.keep = spec.get("keep", self.window)
        self.eps = float(spec["eps"])
        self.own_kv = bool(spec.get("own_kv", True))
        if self.nq % self.nkv:
            raise ValueError(f"{self.nq} query heads cannot be grouped over {self.nkv} KV heads")
        if self.keep is not None and (self.window is None or self.keep < self.window):
            raise ValueError(f"the cache keeps {self.keep} positions, fewer than the window of {self.window or 'all'}")
        if self.dv > 256:
            raise ValueError(f"values {self.dv} wide: the attention kernels take up to 256")
        self.position = POSITIONS.build(spec["position"], rt=rt)
        if getattr(self.position, "interleaved", False):
            raise ValueError("sink_attention rotates half-split pairs only")
        self.qw, self.kw, self.vw, self.ow = self.nq * self.dk, self.nkv * self.dk, self.nkv * self.dv, self.nq * self.dv
        self.weight = self.o_weight = self.q_norm = self.k_norm = self.sink = None

    def kernel_family(self, page_size: int | None = None) -> str:
        """Which attention kernels serve this layer over pages of ``page_size`` keys (None: whatever the
        page size).  "tc": tcgen05 128-row tiles for long portions (bfloat16, keys and values both 64 or
        both 128 wide, pages that divide 64) and mma.sync 16-row tiles for the rest; "mma": mma.sync tiles
        of 64 and 16 rows (bfloat16, widths that are multiples of 8 up to 128); "simt": the CUDA cores
        (float32, and every other width)."""
        if self.rt is None or self.rt.dtype != torch.bfloat16 or not K.attention_mma_ext_supports(self.dk, self.dv):
            return "simt"
        if not self.scale > 0.0:        # the tensor-core kernels keep the sink in the raw products' units, sink / scale
            return "simt"
        if page_size is not None and self.dk == self.dv and K.attention_tma_supports(self.dk, page_size):
            return "tc"
        return "mma"

    def kernel_modules(self):
        if self.kernel_family() == "simt":
            return ("attention_simt", "postnorm")
        if self.dk == self.dv and self.dk in (64, 128):
            return ("attention_simt", "attention_mma_ext", "attention_tma", "attention_tc", "postnorm")
        return ("attention_simt", "attention_mma_ext", "postnorm")

    def cache_need(self):
        return PagedKVNeed(kv_heads=self.nkv, head_dim=self.dk, window=self.keep, v_dim=self.dv)

    def plan_key(self):
        return ("sink_attention", self.nq, self.nkv, self.window)

    def planner(self, page_size: int, sm_count: int):
        rows = {"tc": 128, "mma": 64, "simt": ROW_TILE}[self.kernel_family(page_size)]
        return AttentionPlanner(AttentionShape(self.nq, self.nkv, self.window, rows), sm_count)

    def parameters(self):
        p = {"q": ParamSpec((self.qw, self.hidden)), "g": ParamSpec((self.ow, self.hidden)),
             "o": ParamSpec((self.hidden, self.ow)),
             "q.norm": ParamSpec((self.qw,), role="vector", init=("normal", 1.0, 0.1)),
             "sink": ParamSpec((self.nq,), role="vector", init=("normal", 0.0, 1.0))}
        if self.own_kv:
            p.update({"k": ParamSpec((self.kw, self.hidden)), "v": ParamSpec((self.vw, self.hidden)),
                      "k.norm": ParamSpec((self.kw,), role="vector", init=("normal", 1.0, 0.1))})
        return p

    def load(self, tensors):
        rows = [tensors["q"]] + ([tensors["k"], tensors["v"]] if self.own_kv else []) + [tensors["g"]]
        self.weight = torch.cat(rows, 0).contiguous()           # one product: [q | k | v | g]
        self.o_weight = tensors["o"].contiguous()
        self.q_norm, self.k_norm = tensors["q.norm"], tensors.get("k.norm")
        self.sink = tensors["sink"]

    def forward(self, h, ctx: StepContext, cache: CacheView) -> Product:
        rt, ws, T = ctx.rt, ctx.ws, h.shape[0]
        meta = cache.meta
        if cache.writable != self.own_kv:
            raise ValueError("a sink_attention layer with tensors for k and v owns its cache, one without reads another's")
        proj = rt.linear(h, self.weight, ws, "sa_proj", out_dtype=torch.float32)
        p = proj.tensor
        q = ws.get("sa_q", (T, self.qw), rt.dtype)
        rdim = int(getattr(self.position, "rotary_dim", 0) or 0)
        K.qknorm_rope_append(p, self.q_norm, self.k_norm, self.eps, ctx.positions, ctx.tok_seg, meta["block_table"],
                             self.position.inv_freq, rdim, q, cache.storage, nq=self.nq, nkv=self.nkv, dk=self.dk,
                             dv=self.dv, page_size=cache.page_size, has_kv=self.own_kv, nsplit=proj.nsplit,
                             split_stride=proj.split_stride, status=ctx.status)
        g0 = self.qw + (self.kw + self.vw if self.own_kv else 0)
        gate = dict(gate=(p[0] if proj.nsplit > 1 else p)[:, g0:], gate_nsplit=proj.nsplit,
                    gate_split_stride=proj.split_stride)
        attn = ws.get("sa_attn", (T, self.ow), rt.dtype)
        part_rows = max(1, meta["part_rows_cap"])
        part_acc = ws.get("attn_part_acc", (part_rows, self.nq, self.dv), torch.float32)
        part_ml = ws.get("attn_part_ml", (part_rows, self.nq, 2), torch.float32)
        n_small, n_big = meta["n_small"], meta["n_big"]
        n = n_small + n_big
        family = self.kernel_family(cache.page_size)
        if family != "simt":
            args = (q, cache.storage, attn, part_acc, part_ml)
            tail = (ctx.positions, meta["block_table"], meta["tok_part_row"])
            common = dict(nq=self.nq, nkv=self.nkv, d=self.dk, dv=self.dv, page_size=cache.page_size,
                          window=self.window or 0, scale=self.scale, sink=self.sink, **gate)
            if n_small:          # decoded tokens and short portions: 16-row tiles, key splits merged by the last CTA
                chunks = -(-(self.nq // self.nkv) // ROW_TILE)
                counters = ws.get_zeroed("attn_counters", (T * self.nkv * chunks,), torch.int32)
                if family == "tc":      # TMA-fed tiles (keys and values of one width, pages that divide 64)
                    K.attention_tma_ext(*args, meta["items"], n_small, 16, *tail, nq=self.nq, nkv=self.nkv, d=self.dk,
                                        page_size=cache.page_size, window=self.window or 0, scale=self.scale,
                                        sink=self.sink, **gate, tok_nsplit=meta["tok_nsplit"], counters=counters,
                                        status=ctx.status)
                else:
                    K.attention_mma_ext(*args, meta["items"], n_small, 16, *tail, **common,
                                        tok_nsplit=meta["tok_nsplit"], counters=counters)
            big_items = meta["items"][n_small * ITEM_INTS:]
            if n_big and family == "tc":       # long portions: tcgen05 128-row tiles, split along the keys when few
                K.attention_tc_ext(q, cache.storage, attn, big_items, n_big, ctx.positions, meta["block_table"],
                                   nq=self.nq, nkv=self.nkv, d=self.dk, page_size=cache.page_size,
                                   window=self.window or 0, scale=self.scale, status=ctx.status, part_acc=part_acc,
                                   part_ml=part_ml, tok_part_row=meta["tok_part_row"], sink=self.sink, **gate)
                if meta.get("big_split"):
                    K.attention_combine(part_acc, part_ml, meta["tok_part_row"], meta["tok_nsplit"], attn,
                                        nq=self.nq, d=self.dv, **gate)
            elif n_big:          # long portions: 64-row tiles
                K.attention_mma_ext(*args, big_items, n_big, 64, *tail, **common)
            return rt.linear(attn, self.o_weight, ws, "mix_out", out_dtype=torch.float32)
        if n:
            K.attention_simt(q, cache.storage, attn, part_acc, part_ml, meta["items"], n, n, ctx.positions,
                             meta["block_table"], meta["tok_part_row"], nq=self.nq, nkv=self.nkv, d=self.dk,
                             dv=self.dv, page_size=cache.page_size, window=self.window or 0, scale=self.scale,
                             sink=self.sink, **gate)
        if meta["any_split"]:
            K.attention_combine(part_acc, part_ml, meta["tok_part_row"], meta["tok_nsplit"], attn, nq=self.nq,
                                d=self.dv, **gate)
        return rt.linear(attn, self.o_weight, ws, "mix_out", out_dtype=torch.float32)
