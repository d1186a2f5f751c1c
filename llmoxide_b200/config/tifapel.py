"""Typed configuration of the Tifapel decoder and its description as a
``ModelSpec``.

config.json of this design is nested: ``vocab``, ``width``, ``norm.eps`` and a
list ``layers``; every layer names its mixer (``type``: ``attention``,
``retention`` or ``lightning``) with the mixer's sizes (``mixer``) and its
feed-forward (``mlp``: a routed mixture of experts, or null for none).  A
layer has a single norm that feeds mixer and feed-forward alike, and adds the
two results to the residual stream together.  Tensors: ``embed``, ``l<i>.norm1``,
``l<i>.mix.*``, ``l<i>.mlp.*``, ``final.norm``, ``head``.

An attention layer with ``kv_from: j`` has no key/value projections; it reads
layer j's cache entry with its own queries and its own mask.  The entry keeps
what the widest mask among its readers can still see.
"""

from __future__ import annotations

import copy
import math
from dataclasses import dataclass, field

from ..errors import ConfigError
from .spec import BlockSpec, LayerCall, ModelSpec, PartSpec, TensorSpec

_MIXERS = ("attention", "retention", "lightning")


def _need(d: dict, key: str, where: str):
    if not isinstance(d, dict) or d.get(key) is None:
        raise ConfigError(f"config.json: {where} lacks '{key}'")
    return d[key]


def _positive_int(v, what: str) -> int:
    if not isinstance(v, int) or isinstance(v, bool) or v <= 0:
        raise ConfigError(f"{what} must be a positive integer, got {v!r}")
    return v


@dataclass
class TifapelConfig:
    vocab: int
    width: int
    eps: float
    layers: list                       # as in config.json: dicts with type / mixer / mlp
    max_positions: int = 1 << 20       # the design has no limit of its own; the cache's size is the limit
    torch_dtype: str = "bfloat16"
    extra: dict = field(default_factory=dict)
    generation: dict = field(default_factory=dict)

    # ---- reading -----------------------------------------------------------

    @classmethod
    def from_dict(cls, d: dict) -> "TifapelConfig":
        norm = _need(d, "norm", "the top level")
        known = {"architecture", "architectures", "vocab", "width", "norm", "layers", "max_positions", "torch_dtype"}
        cfg = cls(vocab=_need(d, "vocab", "the top level"), width=_need(d, "width", "the top level"),
                  eps=float(_need(norm, "eps", "norm")), layers=copy.deepcopy(_need(d, "layers", "the top level")),
                  max_positions=int(d.get("max_positions") or (1 << 20)),
                  torch_dtype=d.get("torch_dtype") or "bfloat16",
                  extra={k: v for k, v in d.items() if k not in known})
        cfg.validate()
        return cfg

    def to_dict(self) -> dict:
        d = dict(self.extra)
        d.update(architecture="Tifapel", vocab=self.vocab, width=self.width, norm={"eps": self.eps},
                 layers=copy.deepcopy(self.layers), torch_dtype=self.torch_dtype)
        if self.max_positions != 1 << 20:
            d["max_positions"] = self.max_positions
        return d

    # ---- checks ------------------------------------------------------------

    def validate(self) -> None:
        _positive_int(self.vocab, "vocab")
        _positive_int(self.width, "width")
        if not (self.eps > 0 and math.isfinite(self.eps)):
            raise ConfigError(f"norm.eps must be positive, got {self.eps!r}")
        if not isinstance(self.layers, list) or not self.layers:
            raise ConfigError("'layers' must be a non-empty list")
        if self.torch_dtype not in ("bfloat16", "float32"):
            raise ConfigError(f"torch_dtype {self.torch_dtype!r}: supported are bfloat16 and float32")
        for i, layer in enumerate(self.layers):
            where = f"layers[{i}]"
            kind = _need(layer, "type", where)
            if kind not in _MIXERS:
                raise ConfigError(f"{where}.type {kind!r}: this design has {', '.join(_MIXERS)}")
            m = _need(layer, "mixer", where)
            for key in ("heads", "dim", "vdim"):
                _positive_int(_need(m, key, where + ".mixer"), f"{where}.mixer.{key}")
            if kind == "attention":
                self._check_attention(i, m, where + ".mixer")
            else:
                decay = _need(m, "decay", where + ".mixer")
                if not isinstance(decay, list) or len(decay) != m["heads"]:
                    raise ConfigError(f"{where}.mixer.decay must list one decay per head ({m['heads']})")
                if any(not (isinstance(g, (int, float)) and 0.0 <= g <= 1.0) for g in decay):
                    raise ConfigError(f"{where}.mixer.decay: every decay lies in [0, 1]")
                rot = m.get("rot")
                if rot is not None:
                    if kind != "retention":
                        raise ConfigError(f"{where}.mixer.rot: only the retention mixer rotates")
                    dims = _positive_int(_need(rot, "dims", where + ".mixer.rot"), f"{where}.mixer.rot.dims")
                    if dims % 2 or dims > m["dim"]:
                        raise ConfigError(f"{where}.mixer.rot.dims {dims} must be even and at most dim {m['dim']}")
                    if not float(_need(rot, "base", where + ".mixer.rot")) > 0:
                        raise ConfigError(f"{where}.mixer.rot.base must be positive")
            mlp = layer.get("mlp")
            if mlp is not None:
                self._check_mlp(mlp, where + ".mlp")

    def _check_attention(self, i: int, m: dict, where: str) -> None:
        G = _positive_int(_need(m, "kv_heads", where), where + ".kv_heads")
        if m["heads"] % G:
            raise ConfigError(f"{where}: {m['heads']} heads are not a multiple of {G} kv_heads")
        if not math.isfinite(float(_need(m, "scale", where))):
            raise ConfigError(f"{where}.scale must be a number")
        mask = m.get("mask")
        if mask is not None:
            _positive_int(_need(mask, "size", where + ".mask"), where + ".mask.size")
            keep = mask.get("keep_first", 0)
            if not isinstance(keep, int) or keep < 0:
                raise ConfigError(f"{where}.mask.keep_first must be a non-negative integer")
        src = m.get("kv_from")
        if src is not None:
            if not isinstance(src, int) or not (0 <= src < i):
                raise ConfigError(f"{where}.kv_from {src!r} must name an earlier layer")
            other = self.layers[src]
            om = other.get("mixer", {})
            if other.get("type") != "attention" or om.get("kv_from") is not None:
                raise ConfigError(f"{where}.kv_from {src}: that layer has no keys and values of its own")
            for key in ("kv_heads", "dim", "vdim"):
                if om.get(key) != m.get(key):
                    raise ConfigError(f"{where}.kv_from {src}: '{key}' differs ({m.get(key)} against {om.get(key)})")

    @staticmethod
    def _check_mlp(mlp: dict, where: str) -> None:
        kind = mlp.get("kind", "moe")
        if kind != "moe":
            raise ConfigError(f"{where}.kind {kind!r}: this design's feed-forward is 'moe' (or null for none)")
        _positive_int(_need(_need(mlp, "expert", where), "ff", where + ".expert"), where + ".expert.ff")
        r = _need(mlp, "router", where)
        E = _positive_int(_need(r, "experts", where + ".router"), where + ".router.experts")
        top = _positive_int(_need(r, "top", where + ".router"), where + ".router.top")
        if not math.isfinite(float(_need(r, "scale", where + ".router"))):
            raise ConfigError(f"{where}.router.scale must be a number")
        groups = r.get("groups")
        allowed = E
        if groups is not None:
            n = _positive_int(_need(groups, "count", where + ".router.groups"), where + ".router.groups.count")
            keep = _positive_int(_need(groups, "keep", where + ".router.groups"), where + ".router.groups.keep")
            if E % n or keep > n:
                raise ConfigError(f"{where}.router.groups: {E} experts in {n} equal groups of which {keep} are kept")
            allowed = E // n * keep
        if top > allowed:
            raise ConfigError(f"{where}.router.top {top} exceeds the {allowed} experts a token may choose from")

    # ---- derived ----------------------------------------------------------------

    def n_params(self) -> int:
        return sum(math.prod(t.shape) for t in self.to_spec().tensors())

    def summary(self) -> str:
        kinds = [layer["type"][0] for layer in self.layers]
        return (f"tifapel: {len(self.layers)} layers ({''.join(kinds)}), width {self.width}, vocab {self.vocab}, "
                f"eps {self.eps:g}, {self.n_params() / 1e6:.1f} M params, {self.torch_dtype}")

    # ---- description as parts ------------------------------------------------

    def _entry_masks(self) -> dict:
        """Per attention layer that owns keys and values: (window, keep_first) its cache entry must hold,
        which is what the widest mask among the layers that read the entry sees (window None: everything)."""
        out = {}
        for i, layer in enumerate(self.layers):
            if layer["type"] != "attention":
                continue
            m = layer["mixer"]
            owner = m.get("kv_from", None)
            owner = i if owner is None else owner
            mask = m.get("mask")
            window, keep = (mask["size"], mask.get("keep_first", 0)) if mask else (None, 0)
            if owner in out:
                w0, k0 = out[owner]
                window = None if (w0 is None or window is None) else max(w0, window)
                keep = max(k0, keep)
            out[owner] = (window, keep)
        return out

    def to_spec(self) -> ModelSpec:
        d, eps = self.width, self.eps
        entry_masks = self._entry_masks()
        blocks, schedule, entry_of = [], [], {}
        for i, layer in enumerate(self.layers):
            p, m, kind = f"l{i}.", layer["mixer"], layer["type"]
            H, D, Dv = m["heads"], m["dim"], m["vdim"]
            position = None
            if kind == "attention":
                G, src = m["kv_heads"], m.get("kv_from")
                mask = m.get("mask")
                owner = i if src is None else src
                tensors = dict(q=TensorSpec(p + "mix.q", (H * D, d)), o=TensorSpec(p + "mix.o", (d, H * Dv)))
                if src is None:
                    tensors.update(k=TensorSpec(p + "mix.k", (G * D, d)), v=TensorSpec(p + "mix.v", (G * Dv, d)))
                mixer = PartSpec("gqa_attention", dict(
                    hidden_size=d, n_heads=H, n_kv_heads=G, head_dim=D, v_head_dim=Dv, scale=float(m["scale"]),
                    window=mask["size"] if mask else None, keep_first=mask.get("keep_first", 0) if mask else 0,
                    cache_window=entry_masks[owner][0], cache_keep_first=entry_masks[owner][1],
                    qk_norm_eps=None, own_kv=src is None), tensors)
            else:
                rot = m.get("rot") if kind == "retention" else None
                if rot:
                    position = PartSpec("rope_neox", dict(n_rot=rot["dims"], base=float(rot["base"]), angles="float32"))
                tensors = dict(q=TensorSpec(p + "mix.q", (H * D, d)), k=TensorSpec(p + "mix.k", (H * D, d)),
                               v=TensorSpec(p + "mix.v", (H * Dv, d)), g=TensorSpec(p + "mix.g", (H * Dv, d)),
                               o=TensorSpec(p + "mix.o", (d, H * Dv)))
                if kind == "lightning":
                    tensors["norm"] = TensorSpec(p + "mix.norm", (H * Dv,), "vector")
                # retention: plain q, k, v; k scaled by D^-1/2 after the rotation; every head divided by its own
                # root mean square; SiLU gate.  lightning: SiLU on q, k, v; all heads normed together with a
                # gain; sigmoid gate.
                mixer = PartSpec("decay_linear_attention", dict(
                    hidden_size=d, n_heads=H, head_dim=D, v_head_dim=Dv, decay=tuple(float(g) for g in m["decay"]),
                    eps=eps,
                    qkv_activation="silu" if kind == "lightning" else "none",
                    k_scale=1.0 if kind == "lightning" else float(D) ** -0.5,
                    out_norm="all_heads" if kind == "lightning" else "per_head",
                    gate="sigmoid" if kind == "lightning" else "silu"), tensors)
            mlp = layer.get("mlp")
            if mlp is None:
                ffn = PartSpec("none", {}, {})
            else:
                r, F = mlp["router"], mlp["expert"]["ff"]
                E, groups = r["experts"], r.get("groups")
                tensors = {"router": TensorSpec(p + "mlp.router", (E, d))}
                for e in range(E):
                    tensors[f"gate{e}"] = TensorSpec(f"{p}mlp.e{e}.gate", (F, d))
                    tensors[f"up{e}"] = TensorSpec(f"{p}mlp.e{e}.up", (F, d))
                    tensors[f"down{e}"] = TensorSpec(f"{p}mlp.e{e}.down", (d, F))
                ffn = PartSpec("routed_experts", dict(
                    hidden_size=d, intermediate_size=F, n_experts=E, top=r["top"], score="sigmoid",
                    n_groups=groups["count"] if groups else 1, keep_groups=groups["keep"] if groups else 1,
                    group_score_top=2, normalize=True, normalize_eps=1e-20, scale=float(r["scale"]),
                    activation="silu"), tensors)
            norms = dict(shared=PartSpec("rms_norm", dict(size=d, eps=eps),
                                         dict(gain=TensorSpec(p + "norm1", (d,), "vector"))))
            blocks.append(BlockSpec("parallel", mixer, ffn, norms, position))
            if kind == "attention" and m.get("kv_from") is not None:
                schedule.append(LayerCall(layer=i, cache=entry_of[m["kv_from"]], writes_cache=False))
            else:
                entry_of[i] = len(entry_of)
                schedule.append(LayerCall(layer=i, cache=entry_of[i]))
        return ModelSpec(
            architecture="Tifapel", hidden_size=d, vocab_size=self.vocab,
            embedding=PartSpec("gather", dict(scale=None), dict(table=TensorSpec("embed", (self.vocab, d)))),
            blocks=tuple(blocks), schedule=tuple(schedule),
            final_norm=PartSpec("rms_norm", dict(size=d, eps=eps), dict(gain=TensorSpec("final.norm", (d,), "vector"))),
            head=PartSpec("linear", dict(softcap=None), dict(weight=TensorSpec("head", (self.vocab, d)))),
            max_positions=self.max_positions, stop_ids=(), storage_dtype=self.torch_dtype,
            default_sampling={},
        )
