"""Token embedding: h[t,:] = E[tok_t,:] widened to float32, times ``scale``
when the description gives one (the reference's dense Qwen3 path has none,
crates/model/src/qwen35/cpu.rs:129-136).  With a tensor ``positions`` a learned
vector per position is added (not scaled): h[t,:] += P[pos_t,:], the sum in
float32.  When the model keeps several copies of the residual stream
(h [S,T,d]) every copy gets the same rows."""

from __future__ import annotations

from .. import kernels
from .registry import register_embedding


@register_embedding("gather")
class GatherEmbedding:
    def __init__(self, spec, weights: dict, rt):
        self.table = weights[spec.tensors["table"].name]       # left in ``weights``: a tied head shares it
        scale = spec.get("scale")
        self.scale = 1.0 if scale is None else float(scale)
        self.positions = None
        if "positions" in spec.tensors:
            self.positions = weights.pop(spec.tensors["positions"].name)
            if self.positions.dtype != self.table.dtype:
                self.positions = self.positions.to(self.table.dtype)

    needs_context = True         # forward() takes the step's context (token positions)

    def libraries(self) -> set:
        return {"elementwise"}

    def forward(self, tokens, h, ctx=None) -> None:
        if self.positions is None and h.dim() == 2:
            kernels.embed(self.table, tokens, h, self.scale)
        else:
            kernels.embed_positions(self.table, self.positions, tokens, None if ctx is None else ctx.token_pos, h,
                                    self.scale)
