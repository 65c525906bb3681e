"""A plain, slow Dotivik: one function per mechanism, whole sequences at once, no cache.

Written from the design's equations with torch on the CPU; it shares no code with the engine and
is the oracle of the tests.  Notation: x is the residual stream [T, W]; matrices are stored
[out, in] and applied as ``h @ W.T``; positions are 0 .. T-1.

    embedding        x = E[token];  x0 = x
    run order        layers 0 .. start-1, then `times` passes over layers start .. stop-1 (each pass
                     opens with x = W_in [x ; x0]), then layers stop ..
    layer            h = LN(x);  x = x + mixer(h) + ff(h)             (both sublayers read the same h)
    norm             LN(x) = (x - mean) / sqrt(var + eps) * w         (no bias)
    attention        every head has two score maps over shared values; q and k rotated in interleaved
                     pairs on the first r elements of each map; s = cap tanh(q.k scale / cap); causal
                     softmax per map; o = a1 - lambda a2 with lambda = exp(lq1.lk1) - exp(lq2.lk2) + diff;
                     o = o / rms(o) * (1 - diff); heads gated by sigmoid(W_g h); then W_o
    latent attention [c ; kr] = W_dkv h;  c = c / rms(c) * w_c;  kr rotated (half-split pairs) and shared
                     by the heads;  k_h = [W_uk c ; kr],  v_h = W_uv c;  q_h = [unrotated ; rotated];
                     softmax over the last `size` keys; heads gated by sigmoid(W_g h); then W_o
    feed-forward     W_down (gelu_tanh(W_gate h) * (W_up h))
    output           logits = E LN_final(x)
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
    w = {k: (v.to(dtype) if v.is_floating_point() else v)
         for k, v in read_safetensors(folder / "model.safetensors").items()}
    return cfg, w


# ---- small functions -------------------------------------------------------------------------------
def layer_norm(x, weight, eps):
    mean = x.mean(-1, keepdim=True)
    var = ((x - mean) ** 2).mean(-1, keepdim=True)
    return (x - mean) / torch.sqrt(var + eps) * weight


def unit_rms(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def angles(positions, dims, base, dtype):
    """[T, dims / 2]: position times base^(-2i / dims)."""
    i = torch.arange(dims // 2, dtype=dtype)
    return positions.to(dtype)[:, None] * base ** (-2.0 * i / dims)[None, :]


def rotate_interleaved(t, positions, dims, base):
    """t [T, n, d]: the pairs (2i, 2i + 1) of the first ``dims`` elements turn by the position's angles."""
    a = angles(positions, dims, base, t.dtype)
    cos, sin = a.cos()[:, None, :], a.sin()[:, None, :]
    u, v = t[..., 0:dims:2], t[..., 1:dims:2]
    out = t.clone()
    out[..., 0:dims:2] = u * cos - v * sin
    out[..., 1:dims:2] = v * cos + u * sin
    return out


def rotate_half_split(t, positions, dims, base):
    """t [T, n, d]: the pairs (i, i + dims / 2) of the first ``dims`` elements turn."""
    a = angles(positions, dims, base, t.dtype)
    cos, sin = a.cos()[:, None, :], a.sin()[:, None, :]
    half = dims // 2
    u, v = t[..., :half], t[..., half:dims]
    out = t.clone()
    out[..., :half] = u * cos - v * sin
    out[..., half:dims] = v * cos + u * sin
    return out


def visible(T, window=None):
    """[T, T] bool: query i sees key j when j <= i (and i - j < window, if there is one)."""
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    ok = j <= i
    if window is not None:
        ok &= (i - j) < window
    return ok


def softmax_over(scores, mask):
    return torch.softmax(scores.masked_fill(~mask, float("-inf")), -1)


# ---- mechanisms --------------------------------------------------------------------------------------
def embed(w, tokens):
    return w["embed"][torch.as_tensor(tokens, dtype=torch.long)]


def differential_attention(cfg, w, p, m, h, positions):
    """h [T, W] -> [T, W].  p: the layer's tensor prefix, m: the layer's mixer sizes."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    eps = cfg["norm"]["eps"]
    q = (h @ w[p + "q"].T).view(T, H, 2, d)
    k = (h @ w[p + "k"].T).view(T, G, 2, d)
    v = (h @ w[p + "v"].T).view(T, G, dv)
    r, base = m["rot"]["dims"], m["rot"]["base"]
    q = rotate_interleaved(q.reshape(T, 2 * H, d), positions, r, base).view(T, H, 2, d)
    k = rotate_interleaved(k.reshape(T, 2 * G, d), positions, r, base).view(T, G, 2, d)
    lam = (torch.exp((w[p + "lq1"] * w[p + "lk1"]).sum()) - torch.exp((w[p + "lq2"] * w[p + "lk2"]).sum())
           + m["diff"])
    mask = visible(T, (m.get("mask") or {}).get("size"))       # causal; a window only if the layer names one
    gate = torch.sigmoid(h @ w[p + "g"].T)                     # [T, H]
    cap = m.get("softcap")                                       # absent or null: the scores are not capped
    heads = []
    for hd in range(H):
        g = hd // (H // G)
        maps = []
        for which in range(2):
            s = (q[:, hd, which] @ k[:, g, which].T) * m["scale"]
            if cap is not None:
                s = cap * torch.tanh(s / cap)
            maps.append(softmax_over(s, mask) @ v[:, g])
        o = maps[0] - lam * maps[1]
        o = unit_rms(o, eps) * (1.0 - m["diff"])
        heads.append(o * gate[:, hd:hd + 1])
    return torch.cat(heads, -1) @ w[p + "o"].T


def latent_attention(cfg, w, p, m, h, positions):
    T = h.shape[0]
    H, d, dr, dv, rank = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    eps = cfg["norm"]["eps"]
    base = m["rot"]["base"]
    q = (h @ w[p + "q"].T).view(T, H, d + dr)
    down = h @ w[p + "dkv"].T
    c = unit_rms(down[:, :rank], eps) * w[p + "dkv.norm"]
    kr = rotate_half_split(down[:, None, rank:], positions, dr, base)[:, 0]      # [T, dr], one for all heads
    qr = rotate_half_split(q[..., d:], positions, dr, base)                      # [T, H, dr]
    ku = (c @ w[p + "uk"].T).view(T, H, d)
    v = (c @ w[p + "uv"].T).view(T, H, dv)
    mask = visible(T, (m.get("mask") or {}).get("size"))
    gate = torch.sigmoid(h @ w[p + "g"].T)
    heads = []
    for hd in range(H):
        s = (q[:, hd, :d] @ ku[:, hd].T + qr[:, hd] @ kr.T) * m["scale"]
        heads.append((softmax_over(s, mask) @ v[:, hd]) * gate[:, hd:hd + 1])
    return torch.cat(heads, -1) @ w[p + "o"].T


def feed_forward(w, p, h):
    return (gelu_tanh(h @ w[p + "gate"].T) * (h @ w[p + "up"].T)) @ w[p + "down"].T


def run_order(cfg):
    """[(layer, opens a pass)] in the order the layers run."""
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return [(i, False) for i in range(n)]
    start, stop, times = loop["start"], loop["stop"], loop["times"]
    order = [(i, False) for i in range(start)]
    for _ in range(times):
        order += [(i, i == start) for i in range(start, stop)]
    return order + [(i, False) for i in range(stop, n)]


def layer(cfg, w, i, x, positions):
    spec = cfg["layers"][i]
    h = layer_norm(x, w[f"l{i}.norm1"], cfg["norm"]["eps"])
    mixer = {"attention": differential_attention, "latent_attention": latent_attention}[spec["type"]]
    out = mixer(cfg, w, f"l{i}.mix.", spec["mixer"], h, positions)
    if spec.get("mlp") is not None:
        assert spec["mlp"]["kind"] == "dense"
        out = out + feed_forward(w, f"l{i}.mlp.", h)
    return x + out


def forward(cfg, w, tokens, layers_out: list | None = None):
    """Logits [T, vocab] of one whole sequence; ``layers_out`` receives the stream after every layer run."""
    positions = torch.arange(len(tokens))
    x = embed(w, tokens)
    x0 = x
    for i, opens in run_order(cfg):
        if opens:
            x = torch.cat((x, x0), -1) @ w["loop.in"].T
        x = layer(cfg, w, i, x, positions)
        if layers_out is not None:
            layers_out.append(x.clone())
    return layer_norm(x, w["final.norm"], cfg["norm"]["eps"]) @ w["embed"].T


def generate(cfg, w, prompt, n):
    """Greedy continuation of ``prompt`` by n tokens (lowest index wins ties), whole sequence each time."""
    tokens = list(prompt)
    for _ in range(n):
        tokens.append(int(forward(cfg, w, tokens)[-1].argmax()))
    return tokens[len(prompt):]
