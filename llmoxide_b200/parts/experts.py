"""Routed experts as a feed-forward: every token uses ``top`` of ``n_experts``
small gated layers, down(act(gate x) * (up x)), weighted by the router.

Router logits z = W_r x are float32 (the router's matrix is kept in float32;
x may be the compute dtype's rounding).  ``score``: s = sigmoid(z), or a
softmax over z.  With ``n_groups`` > 1 the expert indices are cut into
``n_groups`` contiguous blocks of equal length; every block is ranked by the
sum of its ``group_score_top`` highest s, and a token's choice is restricted
to the ``keep_groups`` top-ranked blocks.  The ``top`` highest s among the
eligible experts are taken; their weights are those s, over (their sum +
``normalize_eps``) when ``normalize``, times ``scale``.

The step's (token, choice) pairs are ordered by expert on the device and the
two products run grouped over that order (csrc/moe.cu), so nothing is read
back to the host and a decode step stays inside a CUDA graph.  The result is
handed on as one float32 partial per choice, [top, T, d], which the norm that
adds it to the residual stream sums in order.
"""

from __future__ import annotations

import torch

from .. import kernels
from ..errors import ConfigError, Unsupported
from .registry import register_feed_forward


@register_feed_forward("none")
class NoFeedForward:
    """A layer without a feed-forward."""

    def __init__(self, spec, weights: dict, rt):
        pass

    def libraries(self) -> set:
        return set()

    def forward(self, x, ctx, residual=None):
        return None


@register_feed_forward("routed_experts")
class RoutedExperts:
    def __init__(self, spec, weights: dict, rt):
        if spec.get("activation", "silu") != "silu":
            raise Unsupported(f"routed_experts activation {spec.get('activation')!r}: only 'silu' is built")
        self.rt = rt
        self.E, self.top, self.F = spec["n_experts"], spec["top"], spec["intermediate_size"]
        self.n_groups, self.keep_groups = spec.get("n_groups", 1), spec.get("keep_groups", 1)
        self.group_top = spec.get("group_score_top", 2)
        self.score = spec.get("score", "sigmoid")
        self.normalize, self.norm_eps = bool(spec.get("normalize", True)), float(spec.get("normalize_eps", 0.0))
        self.scale = float(spec.get("scale", 1.0))
        if self.E % self.n_groups or self.top > self.E // self.n_groups * self.keep_groups:
            raise ConfigError(f"{self.E} experts in {self.n_groups} groups, {self.keep_groups} kept, top {self.top}")
        if self.E > 1024 or self.top > 16:
            raise Unsupported(f"{self.E} experts / top {self.top}: the routing kernel takes up to 1024 / 16")
        t = spec.tensors
        # the router decides in float32 whatever the compute dtype
        self.router = weights.pop(t["router"].name).to(torch.float32).contiguous()
        dt = rt.act_dtype
        gate_up = [torch.cat([weights.pop(t[f"gate{e}"].name), weights.pop(t[f"up{e}"].name)], dim=0).to(dt)
                   for e in range(self.E)]
        self.gate_up = torch.stack(gate_up).contiguous()             # [E, 2F, d]: gate rows, then up rows
        del gate_up
        self.down = torch.stack([weights.pop(t[f"down{e}"].name).to(dt) for e in range(self.E)]).contiguous()  # [E, d, F]

        # bfloat16 with sizes the TMA takes: the grouped products run on tcgen05 (csrc/moe_tc.cu)
        self.tensor_cores = bool(rt.tensor_cores and dt == torch.bfloat16 and self.gate_up.shape[2] % 8 == 0
                                 and self.F % 8 == 0)

    def libraries(self) -> set:
        return {"moe"} | ({"moe_tc"} if self.tensor_cores else set())

    def tile_rows(self, n_pairs: int) -> int:
        """Rows per tile of the grouped products: narrow tiles when an expert gets few rows (a decode step streams
        the weights), wide ones for prompts."""
        per_expert = n_pairs / self.E
        return 16 if per_expert <= 16 else 64 if per_expert <= 96 else 128

    def forward(self, x, ctx, residual=None):
        T, dev = x.shape[0], x.device
        P = T * self.top
        ids = torch.empty((T, self.top), dtype=torch.int32, device=dev)
        pair_w = torch.empty((T, self.top), dtype=torch.float32, device=dev)
        kernels.moe_router(x, self.router, ids, pair_w, self.n_groups, self.keep_groups, self.group_top, self.score,
                           self.normalize, self.norm_eps, self.scale)
        perm = torch.empty((P,), dtype=torch.int32, device=dev)
        fast = self.tensor_cores and x.dtype == torch.bfloat16 and kernels.moe_tc_supports(x, self.gate_up)
        rows = self.tile_rows(P) if fast else kernels.MOE_TILE
        tiles = torch.empty((kernels.moe_max_tiles(P, self.E, rows), 3), dtype=torch.int32, device=dev)
        act = torch.empty((P, self.F), dtype=self.rt.act_dtype, device=dev)
        y = torch.empty((self.top, T, self.down.shape[1]), dtype=torch.float32, device=dev)
        if fast:
            dest = torch.empty((P,), dtype=torch.int32, device=dev)
            sorted_w = torch.empty((P,), dtype=torch.float32, device=dev)
            kernels.moe_sort(ids, self.E, perm, tiles, rows, pair_w, dest, sorted_w)
            xs = torch.empty((P, x.shape[1]), dtype=torch.bfloat16, device=dev)
            kernels.moe_gather_rows(x, perm, self.top, xs)
            kernels.moe_grouped_tc(xs, self.gate_up, act, tiles, rows, dest, sorted_w, gated=True)
            kernels.moe_grouped_tc(act, self.down, y, tiles, rows, dest, sorted_w, gated=False)
        else:
            kernels.moe_sort(ids, self.E, perm, tiles, rows)
            kernels.moe_grouped(x, self.gate_up, act, perm, tiles, pair_w, self.top, T, gated=True)
            kernels.moe_grouped(act, self.down, y, perm, tiles, pair_w, self.top, T, gated=False)
        return y
