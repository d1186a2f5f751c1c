"""RMSNorm with a plain multiplicative gain: x / sqrt(mean(x^2) + eps) * g
(crates/model/src/ops.rs:40-59), fused with the residual add that precedes it.

Several copies of the residual stream (h [S,T,d], "hyper-connections").  The
norm of a sublayer then reads u = sum_s read[s] h_s, and what the sublayer
returns joins the copies as h_r <- sum_s mix[s,r] h_s + mult * out[r] * y.  The
three weights ride with the norm (tensors ``hc_in`` [S], ``hc_out`` [S],
``hc_mix`` [S,S] indexed [from, to]; ``residual_mult`` is the parameter
``mult``); without them the norm reads the plain sum and the result is added
to every copy times ``mult``.  As with one stream, the update is applied by
the next norm's kernel: ``owed(y)`` wraps a sublayer's result into the
``StreamUpdate`` that the next ``add_forward`` (or ``add``) takes as ``delta``."""

from __future__ import annotations

import torch

from .. import kernels
from .row_scaled import RowScaled
from .registry import register_norm


class StreamUpdate:
    """What a sublayer owes the copies of the residual stream: h_r <- sum_s mix[s,r] h_s + write[r] * delta."""

    __slots__ = ("delta", "mix", "write")

    def __init__(self, delta, mix, write):
        self.delta, self.mix, self.write = delta, mix, write


@register_norm("rms_norm")
class RMSNorm:
    def __init__(self, spec, weights: dict, rt):
        self.size, self.eps, self.rt = spec["size"], float(spec["eps"]), rt
        self.gain = weights[spec.tensors["gain"].name].to(torch.float32).contiguous()
        self.mult = float(spec.get("residual_mult", 1.0))
        self.read = self.mix = self.write = None
        if "hc_mix" in spec.tensors:
            t = spec.tensors
            self.read = weights.pop(t["hc_in"].name).to(torch.float32).contiguous()
            self.mix = weights.pop(t["hc_mix"].name).to(torch.float32).contiguous()
            self.write = (weights.pop(t["hc_out"].name).to(torch.float32) * self.mult).contiguous()
        self._plain: dict = {}

    def libraries(self) -> set:
        return {"elementwise", "stream_mix"}

    def owed(self, delta, n_streams: int):
        """The update by which a sublayer's result ``delta`` (None: nothing) joins ``n_streams`` copies."""
        if delta is None:
            return None
        if self.mix is None:        # no connection weights: every copy keeps itself and gets mult * delta
            if n_streams not in self._plain:
                self._plain[n_streams] = (torch.eye(n_streams, dtype=torch.float32, device=self.gain.device).contiguous(),
                                          torch.full((n_streams,), self.mult, dtype=torch.float32, device=self.gain.device))
            return StreamUpdate(delta, *self._plain[n_streams])
        return StreamUpdate(delta, self.mix, self.write)

    def _streams(self, h, delta, out, rows, write_h):
        if delta is None:
            d, mix, write = None, None, None
        elif isinstance(delta, StreamUpdate):
            d, mix, write = delta.delta, delta.mix, delta.write
        else:
            upd = RMSNorm.owed(self, delta, h.shape[0]) if self.mix is None else None
            if upd is None:
                raise ValueError("a result that joins several copies of the residual stream comes as a StreamUpdate")
            d, mix, write = upd.delta, upd.mix, upd.write
        kernels.stream_mix_norm(h, d, mix, write, self.read if out is not None else None, self.gain, self.eps, out,
                                rows=rows, write_h=write_h)

    ROW_SCALE_MAX_TOKENS = 64      # what the products' epilogues take

    def add(self, h, delta) -> None:
        """h += delta (``delta`` [T,d] or split partials [S,T,d], added in order); nothing is normed."""
        if h.dim() == 2 and isinstance(delta, StreamUpdate):
            h = h.unsqueeze(0)       # one copy, with connection weights of its own
        if h.dim() == 3:
            if delta is not None:
                self._streams(h, delta, None, None, True)
            return
        kernels.add_rms_norm(h, delta, self.gain, self.eps, None)

    def add_forward(self, h, delta, rows=None, write_h=True, out_dtype=None, row_scales_ok=False):
        """With ``row_scales_ok`` the caller's next products apply the norm's scale themselves; for a step of
        few tokens the result is then ``RowScaled`` (the norm in two halves, see ``parts.row_scaled``)."""
        if h.dim() == 2 and isinstance(delta, StreamUpdate):
            h = h.unsqueeze(0)       # one copy, with connection weights of its own
        if h.dim() == 3:
            n = h.shape[1] if rows is None else rows.numel()
            out = torch.empty((n, self.size), dtype=out_dtype or self.rt.act_dtype, device=h.device)
            self._streams(h, delta, out, rows, write_h)
            return out
        if (row_scales_ok and rows is None and write_h and out_dtype in (None, torch.bfloat16)
                and self.rt.act_dtype == torch.bfloat16 and h.shape[0] <= self.ROW_SCALE_MAX_TOKENS
                and self.size % 4 == 0):
            T = h.shape[0]
            parts = (self.size + kernels.ADD_SLICE - 1) // kernels.ADD_SLICE
            x = torch.empty((T, self.size), dtype=torch.bfloat16, device=h.device)
            sumsq = torch.empty((parts, max(T, 8)), dtype=torch.float32, device=h.device)
            kernels.add_gain_sumsq(h, delta, self.gain, x, sumsq)
            return RowScaled(x, sumsq, parts, self.eps, self.size)
        n = h.shape[0] if rows is None else rows.numel()
        out = torch.empty((n, self.size), dtype=out_dtype or self.rt.act_dtype, device=h.device)
        kernels.add_rms_norm(h, delta, self.gain, self.eps, out, rows=rows, write_h=write_h)
        return out
