"""Linear attention with a fixed decay per head as a mixer: no softmax and no
denominator, a float32 state of fixed size per sequence instead of keys and
values.

    q, k: [heads, D], v: [heads, Dv], gate: [heads * Dv]     one fused projection of the layer's input
    q, k, v <- act(q), act(k), act(v)                         ``qkv_activation``: none or silu
    q, k <- rotate(q), rotate(k)                              when the block has a position encoding
    k <- k * k_scale
    S_t = decay_h S_{t-1} + k_t v_t^T,  o_t = S_t^T q_t       per head; S starts at zero
    o <- o / sqrt(mean(o^2) + eps) [* gain]                   ``out_norm``: per_head or all_heads (with a gain)
    y = W_o (o * gate_act(gate))                              ``gate``: silu or sigmoid

The state, the decays, the rotation's angles, the recurrence and the norm are
float32 whatever the compute dtype; the projections and their activations
follow the compute dtype.  Two designs of this family differ in the
parameters only (a retention layer: no activation, rotation, k scaled by
D^-1/2, per-head unit norm, SiLU gate; a lightning-attention layer: SiLU on
q, k and v, no rotation, one norm over all heads with a gain, sigmoid gate).
"""

from __future__ import annotations

import torch

from .. import kernels
from ..cache import StateNeed
from ..errors import ConfigError, Unsupported
from .linear import Linear
from .registry import register_mixer


@register_mixer("decay_linear_attention")
class DecayLinearAttention:
    def __init__(self, spec, position, weights: dict, rt):
        self.rt = rt
        self.H, self.D, self.Dv = spec["n_heads"], spec["head_dim"], spec["v_head_dim"]
        if self.D > 256:
            raise Unsupported(f"head_dim {self.D}: the recurrence kernel takes sizes up to 256")
        decay = [float(g) for g in spec["decay"]]
        if len(decay) != self.H:
            raise ConfigError(f"{len(decay)} decays for {self.H} heads")
        self.decay = torch.tensor(decay, dtype=torch.float32, device=rt.device)
        self.eps = float(spec["eps"])
        self.activation = spec.get("qkv_activation", "none")
        self.k_scale = float(spec.get("k_scale", 1.0))
        self.per_head = {"per_head": True, "all_heads": False}[spec.get("out_norm", "per_head")]
        self.gate = spec.get("gate", "silu")
        if self.activation not in ("none", "silu") or self.gate not in ("none", "silu", "sigmoid"):
            raise ConfigError(f"activation {self.activation!r} / gate {self.gate!r} are not built")
        t = spec.tensors
        ws = [weights.pop(t[r].name) for r in ("q", "k", "v", "g")]
        if len({w.dtype for w in ws}) > 1:
            ws = [w.float() for w in ws]
        # one matrix product for q, k, v and the gate: rows in that order
        self.qkvg = Linear(torch.cat(ws, dim=0), rt)
        del ws
        self.o = Linear(weights.pop(t["o"].name), rt)
        self.gain = weights.pop(t["norm"].name).to(torch.float32).contiguous() if "norm" in t else None
        self.position = position
        HD, HDv = self.H * self.D, self.H * self.Dv
        self.q_off, self.k_off, self.v_off, self.g_off = 0, HD, 2 * HD, 2 * HD + HDv

    def cache_need(self):
        return None, StateNeed((self.H, self.D, self.Dv))

    def libraries(self) -> set:
        return {"linear_attention"} | self.qkvg.libraries() | self.o.libraries()

    adds_to_residual = True      # forward() takes ``residual`` and may return None: "already added"

    def forward(self, x, ctx, view, writes_cache=True, residual=None):
        if not writes_cache:
            raise Unsupported("a recurrent state has one writer: the layer that owns it")
        T = x.shape[0]
        tables = self.position.rotary_tables() if self.position is not None else None
        cos, sin, n_rot = tables if tables is not None else (None, None, 0)
        proj = self.qkvg(x, splits_ok=True)
        o = torch.empty((T, self.H * self.Dv), dtype=torch.float32, device=x.device)
        kernels.decay_scan(proj, o, view.state, ctx.seq_start, ctx.token_pos, ctx.seq_slot, self.decay, cos, sin, n_rot,
                           self.activation, self.k_scale, self.H, self.D, self.Dv, self.q_off, self.k_off, self.v_off,
                           max_new=ctx.max_new)
        y = torch.empty((T, self.H * self.Dv), dtype=self.rt.act_dtype, device=x.device)
        kernels.gated_norm(o, proj, self.g_off, self.gain, self.eps, self.gate, self.per_head, y, self.H, self.Dv)
        if residual is not None and self.o.add_into(y, residual):
            return None
        return self.o(y, splits_ok=True)
