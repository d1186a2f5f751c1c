"""Plain, slow implementation of the Tifapel decoder, for tests only.

Written from the design's equations, one function per mechanism, whole
sequences token by token where a recurrence is involved, no cache, float64 on
the CPU (so that it sits inside the float32 rounding of any right
implementation).  It shares no code with ``llmoxide_b200``: it has its own
reader for the model folder and its own handling of the configuration.

Notation: x [T, d] is the residual stream of one sequence, positions 0..T-1;
weights are stored [out, in] and applied as W x.
"""

from __future__ import annotations

import json
import math
import struct
from pathlib import Path

import numpy as np
import torch

F = torch.float64


# --------------------------------------------------------------------------
# Model folder
# --------------------------------------------------------------------------

def read_safetensors(path) -> dict:
    raw = Path(path).read_bytes()
    (n,) = struct.unpack("<Q", raw[:8])
    header = json.loads(raw[8 : 8 + n])
    out = {}
    for name, info in header.items():
        if name == "__metadata__":
            continue
        lo, hi = info["data_offsets"]
        buf = raw[8 + n + lo : 8 + n + hi]
        if info["dtype"] == "BF16":
            bits = np.frombuffer(buf, dtype=np.uint16).astype(np.uint32) << 16
            arr = bits.view(np.float32)
        else:
            arr = np.frombuffer(buf, dtype={"F32": np.float32, "F16": np.float16, "I32": np.int32}[info["dtype"]])
        out[name] = torch.from_numpy(arr.reshape(info["shape"]).copy()).to(F)
    return out


def read_model(folder):
    folder = Path(folder)
    return json.loads((folder / "config.json").read_text()), read_safetensors(folder / "model.safetensors")


# --------------------------------------------------------------------------
# Mechanisms
# --------------------------------------------------------------------------

def rms(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def rms_norm(x, gain, eps):
    return rms(x, eps) * gain


def silu(z):
    return z * torch.sigmoid(z)


def rotate_half(x, positions, dims, base):
    """x [T, heads, D]: dimension i of the first ``dims`` is paired with i + dims/2 and the pair is turned
    by the angle position * base^(-2i/dims); the other dimensions pass."""
    half = dims // 2
    freq = torch.tensor([base ** (-2.0 * i / dims) for i in range(half)], dtype=F)
    ang = positions.to(F)[:, None] * freq[None, :]            # [T, half]
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    u, v = x[..., :half], x[..., half:dims]
    return torch.cat([u * c - v * s, v * c + u * s, x[..., dims:]], dim=-1)


def decayed_outer_product_scan(q, k, v, decay):
    """S_t = decay_h S_{t-1} + k_t v_t^T;  o_t = S_t^T q_t.  q, k [T, H, D]; v [T, H, Dv]; decay [H]."""
    T, H, D = q.shape
    S = torch.zeros(H, D, v.shape[-1], dtype=F)
    out = torch.zeros(T, H, v.shape[-1], dtype=F)
    g = torch.as_tensor(decay, dtype=F)[:, None, None]
    for t in range(T):
        S = g * S + k[t][:, :, None] * v[t][:, None, :]
        out[t] = torch.einsum("hdv,hd->hv", S, q[t])
    return out


def retention(h, w, p, m, eps):
    """Linear attention with a fixed decay per head, rotary positions on q and k, k scaled by D^-1/2
    after the rotation, every head's output divided by its own root mean square, a SiLU gate."""
    T = h.shape[0]
    H, D, Dv = m["heads"], m["dim"], m["vdim"]
    q = (h @ w[p + "q"].T).view(T, H, D)
    k = (h @ w[p + "k"].T).view(T, H, D)
    v = (h @ w[p + "v"].T).view(T, H, Dv)
    rot = m.get("rot")
    if rot:
        pos = torch.arange(T)
        q, k = rotate_half(q, pos, rot["dims"], rot["base"]), rotate_half(k, pos, rot["dims"], rot["base"])
    k = k * D ** -0.5
    o = rms(decayed_outer_product_scan(q, k, v, m["decay"]), eps)
    return (o.reshape(T, H * Dv) * silu(h @ w[p + "g"].T)) @ w[p + "o"].T


def lightning(h, w, p, m, eps):
    """The same recurrence on SiLU-activated q, k and v with no other scale; the heads are normed together
    with a gain, then a sigmoid gate."""
    T = h.shape[0]
    H, D, Dv = m["heads"], m["dim"], m["vdim"]
    q = silu(h @ w[p + "q"].T).view(T, H, D)
    k = silu(h @ w[p + "k"].T).view(T, H, D)
    v = silu(h @ w[p + "v"].T).view(T, H, Dv)
    o = decayed_outer_product_scan(q, k, v, m["decay"]).reshape(T, H * Dv)
    return (rms_norm(o, w[p + "norm"], eps) * torch.sigmoid(h @ w[p + "g"].T)) @ w[p + "o"].T


def visible(i, j, mask):
    """Whether the query at position i sees the key at position j."""
    if j > i:
        return False
    if mask is None:
        return True
    return i - j < mask["size"] or j < mask.get("keep_first", 0)


def attention_keys_values(h, w, p, m):
    T = h.shape[0]
    G = m["kv_heads"]
    return (h @ w[p + "k"].T).view(T, G, m["dim"]), (h @ w[p + "v"].T).view(T, G, m["vdim"])


def attention(h, w, p, m, k, v):
    """Softmax attention without positions, grouped heads, a sliding window that also keeps the first
    tokens; k, v are this layer's own or another layer's."""
    T = h.shape[0]
    H, G, D = m["heads"], m["kv_heads"], m["dim"]
    q = (h @ w[p + "q"].T).view(T, H, D)
    out = torch.zeros(T, H, m["vdim"], dtype=F)
    for i in range(T):
        js = [j for j in range(T) if visible(i, j, m.get("mask"))]
        for hq in range(H):
            g = hq // (H // G)
            s = (k[js, g] @ q[i, hq]) * m["scale"]
            out[i, hq] = torch.softmax(s, 0) @ v[js, g]
    return out.reshape(T, -1) @ w[p + "o"].T


def route(h, w_router, r):
    """Per token: the picked experts and their weights.  s = sigmoid(logits); with groups, the expert axis is cut
    into ``count`` equal contiguous blocks, a block ranks by the sum of its top-2 s, and picks are limited to the
    ``keep`` top-ranked blocks."""
    s = torch.sigmoid(h @ w_router.T)                   # [T, E]
    T, E = s.shape
    allowed = torch.ones(T, E, dtype=torch.bool)
    groups = r.get("groups")
    if groups:
        n, keep = groups["count"], groups["keep"]
        per = E // n
        gs = s.view(T, n, per).topk(min(2, per), dim=-1).values.sum(-1)         # [T, n]
        best = gs.topk(keep, dim=-1).indices
        gmask = torch.zeros(T, n, dtype=torch.bool).scatter_(1, best, True)
        allowed = gmask[:, :, None].expand(T, n, per).reshape(T, E)
    chosen = s.masked_fill(~allowed, -1.0).topk(r["top"], dim=-1).indices       # [T, top]
    sc = s.gather(1, chosen)
    return chosen, sc / (sc.sum(-1, keepdim=True) + 1e-20) * r["scale"]


def experts(h, w, p, mlp):
    chosen, weight = route(h, w[p + "router"], mlp["router"])
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e, a in zip(chosen[t].tolist(), weight[t]):
            q = f"{p}e{e}."
            out[t] += a * ((silu(h[t] @ w[q + "gate"].T) * (h[t] @ w[q + "up"].T)) @ w[q + "down"].T)
    return out


# --------------------------------------------------------------------------
# The decoder
# --------------------------------------------------------------------------

def forward(cfg, w, tokens, return_layers=False):
    """Logits [T, vocab] (float64) of one whole sequence; with ``return_layers`` also the residual stream
    after every layer [L, T, d]."""
    eps = cfg["norm"]["eps"]
    x = w["embed"][torch.as_tensor(tokens, dtype=torch.long)]
    kv, after = {}, []
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        h = rms_norm(x, w[p + "norm1"], eps)
        if layer["type"] == "retention":
            a = retention(h, w, p + "mix.", m, eps)
        elif layer["type"] == "lightning":
            a = lightning(h, w, p + "mix.", m, eps)
        elif layer["type"] == "attention":
            src = m.get("kv_from")
            if src is None:
                kv[i] = attention_keys_values(h, w, p + "mix.", m)
                src = i
            a = attention(h, w, p + "mix.", m, *kv[src])
        else:
            raise ValueError(layer["type"])
        f = experts(h, w, p + "mlp.", layer["mlp"]) if layer.get("mlp") else 0.0
        x = x + (a + f)
        after.append(x)
    logits = rms_norm(x, w["final.norm"], eps) @ w["head"].T
    return (logits, torch.stack(after)) if return_layers else logits


def argmax(row) -> int:
    return int(np.argmax(np.asarray(row)))
