"""Attention whose heads each hold several score maps over shared values (differential attention: two
maps, the second subtracted from the first), with capped scores, a unit-RMS norm per head and a gate
per head."""
from __future__ import annotations

import torch

from ..kernels import api as K
from .attention import ITEM_INTS, ROW_TILE, AttentionPlanner, AttentionShape
from .base import CacheView, Mixer, Product, StepContext
from .registry import POSITIONS, register_mixer
from .spec import PagedKVNeed, ParamSpec, PartSpec

MAPS = 2


def _pad_rows(w: torch.Tensor, multiple: int = 16) -> torch.Tensor:
    """The stacked weight with zero rows up to a multiple of ``multiple`` (the product's row stride
    then suits every kernel that reads it)."""
    extra = -w.shape[0] % multiple
    if not extra:
        return w.contiguous()
    return torch.cat((w, w.new_zeros(extra, w.shape[1])), 0).contiguous()


@register_mixer("diff_attention")
class DifferentialAttention(Mixer):
    """q = W_q h [heads x 2 x dim], k = W_k h [kv_heads x 2 x dim], v = W_v h [kv_heads x vdim], no biases;
    a head's q and k are laid out [map 1 | map 2].

    * Every map of q and k is rotated by the position part on its own first ``rotary_dim`` elements.
    * Per map: s = (q . k) * scale, then s <- softcap * tanh(s / softcap) if there is a cap; a causal
      softmax (over the last ``window`` keys, if there is a window) times the head's shared values gives
      a1 and a2.
    * o = a1 - lambda * a2 with lambda = exp(lq1 . lk1) - exp(lq2 . lk2) + lambda_init, one number for the
      layer; o <- o / sqrt(mean(o^2) + eps) over the head's values, times (1 - lambda_init).
    * The head's output is multiplied by sigmoid(W_g h)_head (one gate per head) and projected by W_o.

    Query head h reads KV head h // (heads // kv_heads).  The cache keeps, per position and KV head, the
    two key maps side by side and the values: PagedKVNeed(kv_heads, 2 * dim, v_dim=vdim).
    Parameters: hidden_size, heads, kv_heads, dim, vdim, scale, softcap (None: no cap), lambda_init, eps,
    window (None: all keys), position (a PartSpec).  Tensors: q, k, v, lq1, lk1, lq2, lk2, g, o.
    Scores, softmax, the maps' outputs and their difference, the norm and the gate are float32.
    """

    def __init__(self, spec: PartSpec, rt=None):
        super().__init__(spec, rt)
        self.hidden = int(spec["hidden_size"])
        self.heads, self.nkv = int(spec["heads"]), int(spec["kv_heads"])
        self.d, self.dv = int(spec["dim"]), int(spec["vdim"])
        self.scale = float(spec["scale"])
        self.softcap = float(spec.get("softcap") or 0.0)
        self.lambda_init = float(spec["lambda_init"])
        self.eps = float(spec["eps"])
        self.window = spec.get("window")
        if self.heads % self.nkv:
            raise ValueError(f"{self.heads} query heads cannot be grouped over {self.nkv} KV heads")
        if self.dv > 512:
            raise ValueError(f"values {self.dv} wide: the attention kernels take up to 512")
        self.position = POSITIONS.build(spec["position"], rt=rt)
        self.nq = self.heads * MAPS                       # query maps: what the attention kernels call heads
        self.qw, self.kw, self.vw = self.nq * self.d, self.nkv * MAPS * self.d, self.nkv * self.dv
        self.ow = self.heads * self.dv
        self.weight = self.o_weight = None
        self.lam = None

    def kernel_family(self, page_size: int | None = None) -> str:
        """"tc": the two maps' keys of a KV head lie side by side and are as wide together as its values (64 or 128,
        bfloat16, pages that divide 64): every q map is padded with zeros to that width, at its own map's columns,
        so a map's score is the product with the WHOLE key row and the kernels see plain grouped-query attention
        with 2 x heads query heads: tcgen05 128-row tiles for long portions, TMA-fed 16-row tiles for the rest.
        "mma": mma.sync tiles of 64 and 16 rows that read a map's keys at its columns (bfloat16, widths that are
        multiples of 8 up to 128); "simt": the CUDA cores (float32, and every other width)."""
        if (self.rt is None or self.rt.dtype != torch.bfloat16 or not self.scale > 0.0
                or not K.attention_mma_ext_supports(self.d, self.dv)):
            return "simt"
        if (page_size is not None and MAPS * self.d == self.dv and self.dv in (64, 128)
                and K.attention_tma_supports(self.dv, page_size)):
            return "tc"
        return "mma"

    def kernel_modules(self):
        if self.kernel_family() == "simt":
            return ("attention_simt", "mixparts")
        if MAPS * self.d == self.dv and self.dv in (64, 128):
            return ("attention_simt", "attention_mma_ext", "attention_tma", "attention_tc", "mixparts")
        return ("attention_simt", "attention_mma_ext", "mixparts")

    def cache_need(self):
        return PagedKVNeed(kv_heads=self.nkv, head_dim=MAPS * self.d, window=self.window, v_dim=self.dv)

    def plan_key(self):
        return ("diff_attention", self.heads, self.nkv, self.window, self.d, self.dv, self.rt is not None and self.rt.dtype)

    def planner(self, page_size: int, sm_count: int):
        family = self.kernel_family(page_size)
        if family == "tc":       # plain grouped-query attention over 2 x heads padded query maps
            return AttentionPlanner(AttentionShape(self.nq, self.nkv, self.window, 128), sm_count)
        rows = {"mma": 64, "simt": ROW_TILE}[family]
        return AttentionPlanner(AttentionShape(self.heads, self.nkv, self.window, rows), sm_count)

    def parameters(self):
        vec = dict(role="vector", init=("normal", 0.0, 0.1))
        return {"q": ParamSpec((self.qw, self.hidden)), "k": ParamSpec((self.kw, self.hidden)),
                "v": ParamSpec((self.vw, self.hidden)), "g": ParamSpec((self.heads, self.hidden)),
                "o": ParamSpec((self.hidden, self.ow)),
                "lq1": ParamSpec((self.d,), **vec), "lk1": ParamSpec((self.d,), **vec),
                "lq2": ParamSpec((self.d,), **vec), "lk2": ParamSpec((self.d,), **vec)}

    def load(self, tensors):
        self.weight = _pad_rows(torch.cat((tensors["q"], tensors["k"], tensors["v"], tensors["g"]), 0))   # [q | k | v | g]
        self.o_weight = tensors["o"].contiguous()
        f = {k: tensors[k].float() for k in ("lq1", "lk1", "lq2", "lk2")}
        lam = torch.exp((f["lq1"] * f["lk1"]).sum()) - torch.exp((f["lq2"] * f["lk2"]).sum()) + self.lambda_init
        self.lam = float(lam.item())          # a constant of the layer, taken in float32 once

    def forward(self, h, ctx: StepContext, cache: CacheView) -> Product:
        rt, ws, T = ctx.rt, ctx.ws, h.shape[0]
        meta = cache.meta
        proj = rt.linear(h, self.weight, ws, "mm_proj", out_dtype=torch.float32)
        p = proj.tensor
        family = self.kernel_family(cache.page_size)
        padded = family == "tc"
        q = ws.get("mm_q", (T, self.qw * (MAPS if padded else 1)), rt.dtype)
        rdim = int(getattr(self.position, "rotary_dim", 0) or 0)
        K.rope_append_maps(p, ctx.positions, ctx.tok_seg, meta["block_table"], self.position.inv_freq, rdim,
                           bool(getattr(self.position, "interleaved", False)), q, cache.storage, nq=self.nq,
                           nkv=self.nkv, kparts=MAPS, d=self.d, dv=self.dv, page_size=cache.page_size,
                           nsplit=proj.nsplit, split_stride=proj.split_stride, status=ctx.status, q_pad=padded)
        maps = ws.get("mm_maps", (T, self.heads, MAPS, self.dv), torch.float32)     # a1, a2 of every head
        part_rows = max(1, meta["part_rows_cap"])
        part_acc = ws.get("attn_part_acc", (part_rows, self.nq, self.dv), torch.float32)
        part_ml = ws.get("attn_part_ml", (part_rows, self.nq, 2), torch.float32)
        n_small, n_big = meta["n_small"], meta["n_big"]
        common = dict(nq=self.nq, nkv=self.nkv, d=self.d, dv=self.dv, page_size=cache.page_size,
                      window=self.window or 0, scale=self.scale, kparts=MAPS, softcap=self.softcap)
        args = (q, cache.storage, maps, part_acc, part_ml)
        tail = (ctx.positions, meta["block_table"], meta["tok_part_row"])
        big_items = meta["items"][n_small * ITEM_INTS:]
        if family == "tc":
            if n_small:          # decoded tokens and short portions: TMA-fed 16-row tiles, key splits merged by the last CTA
                chunks = -(-(self.nq // self.nkv) // ROW_TILE)
                counters = ws.get_zeroed("attn_counters", (T * self.nkv * chunks,), torch.int32)
                K.attention_tma_ext(*args, meta["items"], n_small, 16, *tail, nq=self.nq, nkv=self.nkv, d=self.dv,
                                    page_size=cache.page_size, window=self.window or 0, scale=self.scale,
                                    softcap=self.softcap, tok_nsplit=meta["tok_nsplit"], counters=counters,
                                    status=ctx.status)
            if n_big:
                K.attention_tc_ext(q, cache.storage, maps, big_items, n_big, ctx.positions, meta["block_table"],
                                   nq=self.nq, nkv=self.nkv, d=self.dv, page_size=cache.page_size,
                                   window=self.window or 0, scale=self.scale, status=ctx.status, part_acc=part_acc,
                                   part_ml=part_ml, tok_part_row=meta["tok_part_row"], softcap=self.softcap)
                if meta.get("big_split"):
                    K.attention_combine(part_acc, part_ml, meta["tok_part_row"], meta["tok_nsplit"], maps,
                                        nq=self.nq, d=self.dv)
        elif family == "mma":
            if n_small:          # decoded tokens and short portions: 16-row tiles, key splits merged by the last CTA
                chunks = -(-(self.heads // self.nkv) // ROW_TILE)
                counters = ws.get_zeroed("attn_counters", (T * self.nkv * MAPS * chunks,), torch.int32)
                K.attention_mma_ext(*args, meta["items"], n_small, 16, *tail, **common,
                                    tok_nsplit=meta["tok_nsplit"], counters=counters)
            if n_big:            # long portions: 64-row tiles
                K.attention_mma_ext(*args, big_items, n_big, 64, *tail, **common)
        else:
            n = n_small + n_big
            if n:
                K.attention_simt(*args, meta["items"], n, n, *tail, **common)
            if meta["any_split"]:
                K.attention_combine(part_acc, part_ml, meta["tok_part_row"], meta["tok_nsplit"], maps, nq=self.nq,
                                    d=self.dv)
        g0 = self.qw + self.kw + self.vw
        gate = (p[0] if proj.nsplit > 1 else p)[:, g0:g0 + self.heads]
        attn = ws.get("mm_attn", (T, self.ow), rt.dtype)
        K.maps_combine(maps, self.lam, self.eps, 1.0 - self.lambda_init, attn, gate=gate, gate_nsplit=proj.nsplit,
                       gate_split_stride=proj.split_stride)
        return rt.linear(attn, self.o_weight, ws, "mix_out", out_dtype=torch.float32)
