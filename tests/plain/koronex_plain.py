"""A plain, slow Koronex: one function per mechanism, whole sequences at once, no cache.

Written from the design's equations with torch on the CPU; it shares no code with the engine and
is the oracle of the tests.  Notation: x is the residual stream [T, W]; W_name are matrices
stored [out, in] and applied as ``h @ W.T``; positions are 0 .. T-1.

    embedding        x = E[token] * s
    layer            x = N1(a x + mixer(x));  x = N2(a x + ff(x)) if the layer has a feed-forward;
                     x = x + rms(P (gelu_tanh(G x) * S[token, i d : (i+1) d])) * w_side
    norm             N(x) = x / sqrt(mean(x^2) + eps) * w
    lightning mixer  q, k, v = silu(W h); S_t = lambda_h S_(t-1) + k_t v_t^T; o_t = S_t^T q_t;
                     out = W_o (N(concat o) * sigmoid(W_g h))
    attention mixer  q, k normalised over the whole projection, rotated on the first r elements of
                     each head, softmax over the last `window` keys with one extra term exp(sink_h)
                     in the denominator, heads gated by sigmoid(W_g h), then W_o
    feed-forward     W_down relu(W_up h)^2
    output           logits = W_head N_final(x)
"""
from __future__ import annotations

import json
import math
import struct
from pathlib import Path

import torch


# ---- files ---------------------------------------------------------------------------------------
def read_safetensors(path) -> dict[str, torch.Tensor]:
    data = Path(path).read_bytes()
    (n,) = struct.unpack("<Q", data[:8])
    header = json.loads(data[8:8 + n])
    kinds = {"BF16": torch.bfloat16, "F32": torch.float32, "I32": torch.int32, "F16": torch.float16}
    out = {}
    for name, info in header.items():
        if name == "__metadata__":
            continue
        a, b = info["data_offsets"]
        buf = bytearray(data[8 + n + a: 8 + n + b])
        out[name] = torch.frombuffer(buf, dtype=kinds[info["dtype"]]).reshape(info["shape"]).clone()
    return out


def load_folder(folder, dtype=torch.float64):
    folder = Path(folder)
    cfg = json.loads((folder / "config.json").read_text())
    w = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in read_safetensors(folder / "model.safetensors").items()}
    return cfg, w


# ---- small functions -------------------------------------------------------------------------------
def rms(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def silu(z):
    return z * torch.sigmoid(z)


def embed(cfg, w, tokens):
    return w["embed"][torch.as_tensor(tokens)] * cfg["embedding"]["scale"]


# ---- mixers ----------------------------------------------------------------------------------------
def lightning(cfg, w, p, m, h):
    """Linear attention with a fixed decay per head, token by token."""
    T = h.shape[0]
    H, d, dv = m["heads"], m["dim"], m["vdim"]
    q = silu(h @ w[p + "q"].T).view(T, H, d)
    k = silu(h @ w[p + "k"].T).view(T, H, d)
    v = silu(h @ w[p + "v"].T).view(T, H, dv)
    out = torch.zeros(T, H, dv, dtype=h.dtype)
    for hd in range(H):
        S = torch.zeros(d, dv, dtype=h.dtype)
        lam = m["decay"][hd]
        for t in range(T):
            S = lam * S + torch.outer(k[t, hd], v[t, hd])
            out[t, hd] = S.T @ q[t, hd]
    o = rms(out.reshape(T, H * dv), cfg["norm"]["eps"]) * w[p + "norm"]
    return (o * torch.sigmoid(h @ w[p + "g"].T)) @ w[p + "o"].T


def rotate(t, positions, r, base):
    """t [T, heads, d]: element i of a head is paired with element i + r/2, i < r/2; the rest passes."""
    if not r:
        return t
    half = r // 2
    f = torch.tensor([base ** (-2.0 * i / r) for i in range(half)], dtype=t.dtype)
    a = positions.to(t.dtype)[:, None] * f[None, :]
    c, s = a.cos()[:, None, :], a.sin()[:, None, :]
    u, v = t[..., :half], t[..., half:r]
    return torch.cat((u * c - v * s, v * c + u * s, t[..., r:]), -1)


def attention_keys(cfg, w, p, m, h, positions):
    """Keys (normalised, rotated) and values of an attention layer with projections of its own."""
    T = h.shape[0]
    G, d, dv = m["kv_heads"], m["dim"], m["vdim"]
    k = rms(h @ w[p + "k"].T, cfg["norm"]["eps"]) * w[p + "k.norm"]
    k = rotate(k.view(T, G, d), positions, m["rot"]["dims"], m["rot"]["base"])
    v = (h @ w[p + "v"].T).view(T, G, dv)
    return k, v


def attention(cfg, w, p, m, h, positions, kv):
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    k, v = kv
    q = rms(h @ w[p + "q"].T, cfg["norm"]["eps"]) * w[p + "q.norm"]
    q = rotate(q.view(T, H, d), positions, m["rot"]["dims"], m["rot"]["base"])
    win = m["mask"]["size"]
    diff = positions[:, None] - positions[None, :]
    seen = (diff >= 0) & (diff < win)
    out = torch.zeros(T, H, dv, dtype=h.dtype)
    for hd in range(H):
        g = hd // (H // G)
        s = (q[:, hd] @ k[:, g].T) * m["scale"]
        s = s.masked_fill(~seen, -math.inf)
        sink = w[p + "sink"][hd]
        top = torch.maximum(s.max(-1).values, sink)
        e = torch.exp(s - top[:, None])
        den = e.sum(-1) + torch.exp(sink - top)
        out[:, hd] = (e / den[:, None]) @ v[:, g]
    gate = torch.sigmoid(h @ w[p + "g"].T)
    return (out.reshape(T, H * dv) * gate) @ w[p + "o"].T


# ---- feed-forward and the per-layer token input --------------------------------------------------
def feed_forward(w, p, h):
    return torch.relu(h @ w[p + "up"].T) ** 2 @ w[p + "down"].T


def token_side(cfg, w, i, x, tokens):
    d = cfg["token_side"]["dim"]
    p = f"l{i}.side."
    e = w["side.embed"][torch.as_tensor(tokens)][:, i * d:(i + 1) * d]
    y = (gelu_tanh(x @ w[p + "gate"].T) * e) @ w[p + "proj"].T
    return x + rms(y, cfg["norm"]["eps"]) * w[p + "norm"]


# ---- the model ---------------------------------------------------------------------------------------
def forward(cfg, w, tokens, layers_out: list | None = None):
    """Logits [T, vocab] of one whole sequence; ``layers_out`` collects the stream after every layer."""
    T = len(tokens)
    positions = torch.arange(T)
    eps, alpha = cfg["norm"]["eps"], cfg["postln_alpha"]
    x = embed(cfg, w, tokens)
    kept = {}
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}.mix.", layer["mixer"]
        if layer["type"] == "lightning":
            y = lightning(cfg, w, p, m, x)
        elif layer["type"] == "attention":
            if "kv_from" in m and m["kv_from"] is not None:
                kv = kept[m["kv_from"]]
            else:
                kv = kept[i] = attention_keys(cfg, w, p, m, x, positions)
            y = attention(cfg, w, p, m, x, positions, kv)
        else:
            raise ValueError(layer["type"])
        x = rms(alpha * x + y, eps) * w[f"l{i}.norm1"]
        if layer["mlp"] is not None:
            x = rms(alpha * x + feed_forward(w, f"l{i}.mlp.", x), eps) * w[f"l{i}.norm2"]
        if cfg.get("token_side"):
            x = token_side(cfg, w, i, x, tokens)
        if layers_out is not None:
            layers_out.append(x.clone())
    return (rms(x, eps) * w["final.norm"]) @ w["head"].T


def generate(cfg, w, prompt, n):
    """Greedy continuation (lowest index wins ties), recomputing the whole sequence every time."""
    seq = list(prompt)
    for _ in range(n):
        seq.append(int(forward(cfg, w, seq)[-1].argmax()))
    return seq[len(prompt):]
