"""Linear attention with a fixed decay per head over a state that is carried from step to step."""
from __future__ import annotations

import numpy as np
import torch

from ..kernels import api as K
from .base import CacheView, Mixer, Product, StepContext, StepPlanner
from .registry import register_mixer
from .spec import ParamSpec, PartSpec, StateNeed

SCAN_MAX_TOKENS = 16       # segments up to this long are walked token by token; longer ones go in chunks
CHUNK_INTS = 4
SMEM_LIMIT = 200 * 1024


class ChunkPlanner(StepPlanner):
    """Cuts the long segments of a step into chunks for the chunked route of csrc/lightning.cu.

    ``chunks``: {segment, first token in the batch, tokens, index of the chunk in its segment};
    ``seg_chunks``: {segment, first chunk, chunks, first token} for every long segment.  A step of
    single tokens has none of either, captured in a graph or not."""

    def __init__(self, chunk: int):
        self.chunk = chunk

    def capacity(self, max_tokens, max_segments, fixed=None):
        if fixed is not None:
            return {"chunks": 0, "seg_chunks": 0}
        return {"chunks": (max_tokens // self.chunk + max_segments) * CHUNK_INTS, "seg_chunks": max_segments * CHUNK_INTS}

    def plan(self, segments, T, fixed=None):
        chunks, segs = [], []
        for si, seg in enumerate(segments):
            if seg.count <= SCAN_MAX_TOKENS or fixed is not None:
                continue
            first = len(chunks)
            for ci, a in enumerate(range(0, seg.count, self.chunk)):
                chunks.append((si, seg.offset + a, min(self.chunk, seg.count - a), ci))
            segs.append((si, first, len(chunks) - first, seg.offset))
        arrays = {"chunks": np.asarray(chunks, np.int32).reshape(-1), "seg_chunks": np.asarray(segs, np.int32).reshape(-1)}
        return arrays, {"num_chunks": len(chunks), "num_long": len(segs)}

    def decode_fixed(self, segments_count, max_positions):
        return ("scan",)

    def plan_decode(self, starts, fixed):
        empty = np.zeros(0, np.int32)
        return {"chunks": empty, "seg_chunks": empty}, {"num_chunks": 0, "num_long": 0}


@register_mixer("lightning_attention")
class LightningAttention(Mixer):
    """q = silu(W_q h), k = silu(W_k h) [heads x dim], v = silu(W_v h) [heads x vdim];
    per head S_t = decay_h S_(t-1) + k_t v_t^T and o_t = S_t^T q_t, with no other scale; the heads'
    outputs are RMS-normalised TOGETHER (one norm over heads x vdim, plain weight), multiplied by
    sigmoid(W_g h) and projected by W_o.

    The state [heads, dim, vdim] is float32, one per request slot, zero for a new request; silu, the
    recurrence, the norm and the gate are float32 (the q/k/v/g product writes float32).  Parameters:
    hidden_size, heads, dim, vdim, decay (one number per head), eps.  Tensors: q, k, v, g, o, norm.
    """

    def __init__(self, spec: PartSpec, rt=None):
        super().__init__(spec, rt)
        self.hidden = int(spec["hidden_size"])
        self.heads = int(spec["heads"])
        self.dk = int(spec["dim"])
        self.dv = int(spec["vdim"])
        self.eps = float(spec["eps"])
        self.decay_values = tuple(float(d) for d in spec["decay"])
        if len(self.decay_values) != self.heads:
            raise ValueError(f"{len(self.decay_values)} decays for {self.heads} heads")
        self.qw, self.vw = self.heads * self.dk, self.heads * self.dv
        self.weight = self.o_weight = self.norm = self.decay = None
        self.chunk = 0

    def kernel_modules(self):
        return ("lightning", "postnorm")

    def cache_need(self):
        return StateNeed(shape=(self.heads, self.dk, self.dv), dtype="float32")

    def plan_key(self):
        return ("lightning_attention", self.dk, self.dv)

    def planner(self, page_size: int, sm_count: int):
        return ChunkPlanner(self._chunk())

    @property
    def tensor_cores(self) -> bool:
        """The chunked route on the tensor cores: the bfloat16 runtime and widths up to 128."""
        return (self.rt is not None and self.rt.dtype == torch.bfloat16
                and K.lightning_chunked_tc_supports(self.dk, self.dv))

    def _chunk(self) -> int:
        """Tokens per chunk of the chunked route: the tensor-core kernels' 64, or on the CUDA cores the
        largest of 64, 32, 16 whose tiles fit an SM."""
        if self.tensor_cores:
            return K.LIGHTNING_TC_CHUNK
        if not self.chunk:
            self.chunk = 16
            for c in (64, 32):
                if 4 * (2 * c * (self.dk + 1) + c * self.dv + c * (c + 1) + c + 1) <= SMEM_LIMIT:
                    self.chunk = c
                    break
        return self.chunk

    def parameters(self):
        return {"q": ParamSpec((self.qw, self.hidden)), "k": ParamSpec((self.qw, self.hidden)),
                "v": ParamSpec((self.vw, self.hidden)), "g": ParamSpec((self.vw, self.hidden)),
                "o": ParamSpec((self.hidden, self.vw)),
                "norm": ParamSpec((self.vw,), role="vector", init=("normal", 1.0, 0.1))}

    def load(self, tensors):
        self.weight = torch.cat((tensors["q"], tensors["k"], tensors["v"], tensors["g"]), 0).contiguous()
        self.o_weight = tensors["o"].contiguous()
        self.norm = tensors["norm"]
        self.decay = torch.tensor(self.decay_values, dtype=torch.float32, device=self.o_weight.device)

    def forward(self, h, ctx: StepContext, cache: CacheView) -> Product:
        rt, ws, T = ctx.rt, ctx.ws, h.shape[0]
        proj = rt.linear(h, self.weight, ws, "la_proj", out_dtype=torch.float32)
        p = proj.tensor
        o = ws.get("la_o", (T, self.vw), torch.float32)
        args = (p, 0, self.qw, 2 * self.qw, self.decay, cache.storage, o, ctx.tok_seg, ctx.seg_slot, ctx.positions)
        common = dict(heads=self.heads, dk=self.dk, dv=self.dv, nsplit=proj.nsplit, split_stride=proj.split_stride,
                      writable=cache.writable)
        meta = cache.meta
        n_chunks = meta.get("num_chunks", 0)
        short = any(s.count <= SCAN_MAX_TOKENS for s in ctx.segments) if n_chunks else True
        if short:
            K.lightning_scan(*args, **common, max_tokens=SCAN_MAX_TOKENS if n_chunks else 0)
        if n_chunks:
            scratch = ws.get("la_chunk_states", (n_chunks * self.heads * self.dk * self.dv,), torch.float32)
            if self.tensor_cores:
                K.lightning_chunked_tc(*args, meta["chunks"], n_chunks, meta["seg_chunks"], meta["num_long"], scratch,
                                       **common)
            else:
                K.lightning_chunked(*args, meta["chunks"], n_chunks, meta["seg_chunks"], meta["num_long"], scratch,
                                    self._chunk(), **common)
        gate = (p[0] if proj.nsplit > 1 else p)[:, 2 * self.qw + self.vw:]
        out = ws.get("la_normed", (T, self.vw), rt.dtype)
        K.gated_rmsnorm(o, self.norm, self.eps, out, gate=gate, gate_nsplit=proj.nsplit,
                        gate_split_stride=proj.split_stride)
        return rt.linear(out, self.o_weight, ws, "mix_out", out_dtype=torch.float32)      # it joins a float32 sum
