"""Plain, slow implementation of the Voserax decoder, for tests only.

Written from the design's equations, one function per mechanism, whole
sequences, no cache, float64 on the CPU (so that it sits inside the float32
rounding of any right implementation).  It shares no code with
``llmoxide_b200``: it has its own reader for the model folder and its own
handling of the configuration.

Notation: a sequence has T tokens at positions 0..T-1; weights are stored
[out, in] and applied as W x; S residual streams X [S, T, d].
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
            arr = (np.frombuffer(buf, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)
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

def rms_norm(x, gain, eps):
    """x / sqrt(mean(x^2) + eps) * gain over the last axis."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * gain


def short_convolution(u, w):
    """u [T, C], w [C, taps]: y_t = sum_j w[:, j] u_(t - taps + 1 + j), zeros before the sequence."""
    T, taps = u.shape[0], w.shape[1]
    padded = torch.cat([torch.zeros((taps - 1, u.shape[1]), dtype=F), u], dim=0)
    y = torch.zeros_like(u)
    for j in range(taps):
        y = y + padded[j : j + T] * w[:, j][None, :]
    return y


def scaled_frequencies(dims, base, scaling):
    """The rotation's frequencies f_i = base^(-2i/dims), i < dims/2, and the factor on cos and sin.  With
    ``scaling`` (factor, original, fast, slow) the frequencies of slow pairs are divided by ``factor``,
    with a linear ramp between the pair indices at which ``original`` positions hold ``fast`` and ``slow``
    turns."""
    half = dims // 2
    f = [base ** (-2.0 * i / dims) for i in range(half)]
    if not scaling:
        return torch.tensor(f, dtype=F), 1.0
    factor, original = float(scaling["factor"]), float(scaling["original"])

    def pair_index(turns):
        return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(pair_index(float(scaling["fast"]))), 0)
    hi = min(math.ceil(pair_index(float(scaling["slow"]))), dims - 1)
    out = []
    for i in range(half):
        ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
        out.append(f[i] / factor * ramp + f[i] * (1.0 - ramp))
    return torch.tensor(out, dtype=F), 0.1 * math.log(factor) + 1.0


def rotate_half(x, positions, dims, base, scaling=None):
    """x [T, heads, D]: dimension i of the first ``dims`` is paired with i + dims/2 and the pair (u, v) is
    turned to (u cos a - v sin a, v cos a + u sin a); the other dimensions pass."""
    half = dims // 2
    freq, mult = scaled_frequencies(dims, base, scaling)
    ang = positions.to(F)[:, None] * freq[None, :]
    c, s = (torch.cos(ang) * mult)[:, None, :], (torch.sin(ang) * mult)[:, None, :]
    u, v = x[..., :half], x[..., half:dims]
    return torch.cat([u * c - v * s, v * c + u * s, x[..., dims:]], dim=-1)


def sink_softmax_attention(q, k, v, scale, window):
    """q [T, H, D], k [T, G, D], v [T, G, Dv].  Position i sees j with 0 <= i - j < window (all j <= i
    without one); the weights are exp(s_j) / (1 + sum exp(s_j)).  Returns [T, H * Dv]."""
    T, H, _ = q.shape
    G = k.shape[1]
    out = torch.zeros((T, H, v.shape[2]), dtype=F)
    for h in range(H):
        g = h // (H // G)
        s = (q[:, h] @ k[:, g].T) * scale
        i = torch.arange(T)
        seen = (i[:, None] >= i[None, :])
        if window is not None:
            seen &= (i[:, None] - i[None, :]) < window
        s = s.masked_fill(~seen, -math.inf)
        m = torch.clamp(s.max(dim=1, keepdim=True).values, min=0.0)
        e = torch.exp(s - m)
        p = e / (torch.exp(-m) + e.sum(dim=1, keepdim=True))
        out[:, h] = p @ v[:, g]
    return out.reshape(T, -1)


def attention_mixer(h, W, prefix, m, first_values):
    """One attention mixer on h [T, d].  ``first_values`` is a one-element list holding the values of the
    first layer that mixes values (None until that layer has run).  Returns the mixer's output."""
    T = h.shape[0]
    H, G, D, Dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q, k, v = h @ W[prefix + "q"].T, h @ W[prefix + "k"].T, h @ W[prefix + "v"].T
    if m.get("conv"):
        q = short_convolution(q, W[prefix + "q.conv"])
        k = short_convolution(k, W[prefix + "k.conv"])
        v = short_convolution(v, W[prefix + "v.conv"])
    q, k, v = q.view(T, H, D), k.view(T, G, D), v.view(T, G, Dv)
    rot = m.get("rot")
    if rot:
        pos = torch.arange(T)
        q = rotate_half(q, pos, rot["dims"], float(rot["base"]), rot.get("scaling"))
        k = rotate_half(k, pos, rot["dims"], float(rot["base"]), rot.get("scaling"))
    if m.get("v_mix"):
        if first_values[0] is None:
            first_values[0] = v
        else:
            lam = W[prefix + "vmix"]
            v = (1.0 - lam) * v + lam * first_values[0]
    mask = m.get("mask")
    o = sink_softmax_attention(q, k, v, float(m["scale"]), mask["size"] if mask else None)
    return o @ W[prefix + "o"].T


def relu_gated(h, W, prefix):
    return (torch.relu(h @ W[prefix + "gate"].T) * (h @ W[prefix + "up"].T)) @ W[prefix + "down"].T


def clamped_expert(h, W, prefix, limit):
    """g = min(W_gate h, limit), u = clamp(W_up h, -limit, limit); W_down (g sigmoid(1.702 g) (u + 1))."""
    g = torch.clamp(h @ W[prefix + "gate"].T, max=limit)
    u = torch.clamp(h @ W[prefix + "up"].T, min=-limit, max=limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ W[prefix + "down"].T


def route(h, W, prefix, r):
    """Softmax scores over experts + identity experts; the ``top`` largest of score + correction are chosen,
    weighted by their scores.  Returns (ids [T, top], weights [T, top], scores)."""
    s = torch.softmax(h @ W[prefix + "router"].T, dim=-1)
    choice = s + W[prefix + "correction"] if prefix + "correction" in W else s
    ids = torch.topk(choice, r["top"], dim=-1).indices
    return ids, torch.gather(s, 1, ids), s


def mixture(h, W, prefix, mlp):
    r = mlp["router"]
    E, limit = r["experts"], float(mlp["expert"]["limit"])
    ids, w, _ = route(h, W, prefix, r)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e, wt in zip(ids[t].tolist(), w[t]):
            y = h[t : t + 1] if e >= E else clamped_expert(h[t : t + 1], W, f"{prefix}e{e}.", limit)
            out[t] += wt * y[0]
    sh = mlp.get("shared")
    if sh:
        gate = torch.sigmoid(h @ W[prefix + "shared.sg"].T)           # [T, 1]
        out = out + gate * clamped_expert(h, W, prefix + "shared.", float(sh["limit"]))
    return out


def feed_forward(h, W, prefix, mlp):
    return relu_gated(h, W, prefix, ) if mlp.get("kind", "dense") == "dense" else mixture(h, W, prefix, mlp)


def hyper_sublayer(X, W, prefix, mult, norm_gain, eps, fn):
    """X [S, T, d].  u = sum_s in[s] X_s; y = fn(norm(u)); X_t <- sum_s mix[s, t] X_s + mult out[t] y."""
    u = torch.einsum("s,std->td", W[prefix + "in"], X)
    y = fn(rms_norm(u, norm_gain, eps))
    return torch.einsum("sr,std->rtd", W[prefix + "mix"], X) + mult * W[prefix + "out"][:, None, None] * y[None]


# --------------------------------------------------------------------------
# The model
# --------------------------------------------------------------------------

def forward(cfg, W, tokens, layer_outputs=None):
    """Logits [T, vocab] of one whole sequence.  ``layer_outputs``: a list that receives the sum of the
    streams after every layer."""
    tokens = torch.as_tensor(tokens, dtype=torch.long)
    T = tokens.shape[0]
    eps, mult = float(cfg["norm"]["eps"]), float(cfg.get("residual_mult", 1.0))
    x = W["embed"][tokens]
    if "pos" in W:
        x = x + W["pos"][:T]
    S = cfg.get("streams")
    X = x[None].repeat(S or 1, 1, 1)
    first_values = [None]
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        mixer = lambda h: attention_mixer(h, W, p + "mix.", layer["mixer"], first_values)
        ff = (lambda h: feed_forward(h, W, p + "mlp.", layer["mlp"])) if layer.get("mlp") else None
        if S:
            X = hyper_sublayer(X, W, p + "hc1.", mult, W[p + "norm1"], eps, mixer)
            if ff:
                X = hyper_sublayer(X, W, p + "hc2.", mult, W[p + "norm2"], eps, ff)
        else:
            X = X + mult * mixer(rms_norm(X[0], W[p + "norm1"], eps))[None]
            if ff:
                X = X + mult * ff(rms_norm(X[0], W[p + "norm2"], eps))[None]
        if layer_outputs is not None:
            layer_outputs.append(X.sum(0))
    return rms_norm(X.sum(0), W["final.norm"], eps) @ W["embed"].T


def greedy(cfg, W, prompt, n_new):
    """Greedy continuation without a cache: the whole sequence again for every token."""
    seq = list(prompt)
    for _ in range(n_new):
        seq.append(int(forward(cfg, W, seq)[-1].argmax()))
    return seq[len(prompt):]
