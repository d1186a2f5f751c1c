"""Typed configuration of the Voserax decoder and its description as a
``ModelSpec``.

config.json of this design is nested: ``vocab``, ``width``, ``norm.eps``,
``residual_mult``, ``streams`` and a list ``layers``; every layer names its
mixer (``type``: ``attention``) with the mixer's sizes (``mixer``) and its
feed-forward (``mlp``: ``kind`` ``dense`` or ``moe``, or null for none).

What the design is made of, in this package's parts:

* embedding ``gather`` with a learned position table (``pos``), tied ``linear`` head;
* arrangement ``hyper_connections``: ``streams`` copies of the residual stream; a sublayer reads a weighted sum
  of them through an RMS norm, and its result, times ``residual_mult`` and a per-stream factor, joins the
  streams after they have been mixed with a [from, to] matrix (``l<i>.hc1.*`` for the mixer, ``hc2`` for the
  feed-forward); the model's output is the sum of the streams;
* mixer ``gqa_attention`` with a short causal convolution over time on every channel of q, k and v (``conv``
  taps), a rotation of the first ``rot.dims`` dims with scaled frequencies (``rope_neox`` with ``scaling``), a
  sliding window, a softmax whose denominator has one added (``sink``), and values mixed with those of the
  first layer that mixes (``v_mix``);
* feed-forward ``gated_mlp`` with ReLU, or ``routed_experts`` with softmax scores, a choice correction,
  identity experts, a clamped gated activation and a shared expert behind a sigmoid gate.

Tensors: ``embed``, ``pos``, ``l<i>.norm1/norm2``, ``l<i>.mix.*``, ``l<i>.mlp.*``, ``l<i>.hc1/hc2.*``, ``final.norm``.
"""

from __future__ import annotations

import copy
import math
from dataclasses import dataclass, field

from ..errors import ConfigError
from .spec import BlockSpec, LayerCall, ModelSpec, PartSpec, TensorSpec

# Constants the design fixes (parameters of the parts; the configuration below sets them).
EXPERT_GATE_SLOPE = 1.702       # g * sigmoid(1.702 g)
EXPERT_UP_SHIFT = 1.0           # (u + 1)
SINK_WEIGHT = 1.0               # the one added to the softmax's denominator
ROT_AMPLITUDE_SLOPE = 0.1       # cos and sin times 0.1 ln(factor) + 1


def _need(d, key: str, where: str):
    if not isinstance(d, dict) or d.get(key) is None:
        raise ConfigError(f"config.json: {where} lacks '{key}'")
    return d[key]


def _positive_int(v, what: str) -> int:
    if not isinstance(v, int) or isinstance(v, bool) or v <= 0:
        raise ConfigError(f"{what} must be a positive integer, got {v!r}")
    return v


def _number(v, what: str) -> float:
    if isinstance(v, bool) or not isinstance(v, (int, float)) or not math.isfinite(float(v)):
        raise ConfigError(f"{what} must be a number, got {v!r}")
    return float(v)


@dataclass
class VoseraxConfig:
    vocab: int
    width: int
    eps: float
    layers: list                       # as in config.json: dicts with type / mixer / mlp
    residual_mult: float = 1.0
    streams: int = 0                   # 0: no hyper-connections (one stream, plain residual sums)
    max_positions: int = 0             # 0: config.json gives none; the position table's rows are what the file has
    learned_positions: bool = True
    torch_dtype: str = "bfloat16"
    extra: dict = field(default_factory=dict)
    generation: dict = field(default_factory=dict)

    # ---- reading -----------------------------------------------------------

    @classmethod
    def from_dict(cls, d: dict) -> "VoseraxConfig":
        norm = _need(d, "norm", "the top level")
        known = {"architecture", "architectures", "vocab", "width", "norm", "layers", "max_positions", "torch_dtype",
                 "residual_mult", "streams", "learned_positions"}
        cfg = cls(vocab=_need(d, "vocab", "the top level"), width=_need(d, "width", "the top level"),
                  eps=float(_need(norm, "eps", "norm")), layers=copy.deepcopy(_need(d, "layers", "the top level")),
                  residual_mult=1.0 if d.get("residual_mult") is None else d["residual_mult"],
                  streams=d.get("streams") or 0,
                  max_positions=int(d.get("max_positions") or 0),
                  learned_positions=bool(d.get("learned_positions", True)),
                  torch_dtype=d.get("torch_dtype") or "bfloat16",
                  extra={k: v for k, v in d.items() if k not in known})
        cfg.validate()
        return cfg

    def to_dict(self) -> dict:
        d = dict(self.extra)
        d.update(architecture="Voserax", vocab=self.vocab, width=self.width, norm={"eps": self.eps},
                 residual_mult=self.residual_mult, layers=copy.deepcopy(self.layers), torch_dtype=self.torch_dtype)
        if self.max_positions:
            d["max_positions"] = self.max_positions
        if self.streams:
            d["streams"] = self.streams
        if not self.learned_positions:
            d["learned_positions"] = False
        return d

    # ---- checks ------------------------------------------------------------

    def validate(self) -> None:
        _positive_int(self.vocab, "vocab")
        _positive_int(self.width, "width")
        if self.max_positions:
            _positive_int(self.max_positions, "max_positions")
        if not (self.eps > 0 and math.isfinite(self.eps)):
            raise ConfigError(f"norm.eps must be positive, got {self.eps!r}")
        self.residual_mult = _number(self.residual_mult, "residual_mult")
        if not isinstance(self.streams, int) or isinstance(self.streams, bool) or not (0 <= self.streams <= 8):
            raise ConfigError(f"streams must be an integer from 1 to 8, got {self.streams!r}")
        if not isinstance(self.layers, list) or not self.layers:
            raise ConfigError("'layers' must be a non-empty list")
        if self.torch_dtype not in ("bfloat16", "float32"):
            raise ConfigError(f"torch_dtype {self.torch_dtype!r}: supported are bfloat16 and float32")
        mixed = None
        for i, layer in enumerate(self.layers):
            where = f"layers[{i}]"
            kind = _need(layer, "type", where)
            if kind != "attention":
                raise ConfigError(f"{where}.type {kind!r}: this design's mixer is 'attention'")
            m = _need(layer, "mixer", where)
            self._check_attention(m, where + ".mixer")
            if m.get("v_mix"):
                sizes = (m["kv_heads"], m["vdim"])
                if mixed is not None and sizes != mixed:
                    raise ConfigError(f"{where}.mixer.v_mix: its values ({sizes[0]} heads of {sizes[1]}) differ in size "
                                      f"from those of the first layer that mixes ({mixed[0]} of {mixed[1]})")
                mixed = sizes
            mlp = layer.get("mlp")
            if mlp is not None:
                self._check_mlp(mlp, where + ".mlp")

    @staticmethod
    def _check_attention(m: dict, where: str) -> None:
        for key in ("heads", "kv_heads", "dim", "vdim"):
            _positive_int(_need(m, key, where), f"{where}.{key}")
        if m["heads"] % m["kv_heads"]:
            raise ConfigError(f"{where}: {m['heads']} heads are not a multiple of {m['kv_heads']} kv_heads")
        _number(_need(m, "scale", where), where + ".scale")
        if m.get("conv") is not None and m["conv"] != 0:
            taps = _positive_int(m["conv"], where + ".conv")
            if taps > 16:
                raise ConfigError(f"{where}.conv {taps}: the convolution kernel takes up to 16 taps")
        mask = m.get("mask")
        if mask is not None:
            _positive_int(_need(mask, "size", where + ".mask"), where + ".mask.size")
        rot = m.get("rot")
        if rot is not None:
            dims = _positive_int(_need(rot, "dims", where + ".rot"), where + ".rot.dims")
            if dims % 2 or dims > m["dim"]:
                raise ConfigError(f"{where}.rot.dims {dims} must be even and at most dim {m['dim']}")
            if not _number(_need(rot, "base", where + ".rot"), where + ".rot.base") > 0:
                raise ConfigError(f"{where}.rot.base must be positive")
            sc = rot.get("scaling")
            if sc is not None:
                for key in ("factor", "original", "fast", "slow"):
                    if not _number(_need(sc, key, where + ".rot.scaling"), f"{where}.rot.scaling.{key}") > 0:
                        raise ConfigError(f"{where}.rot.scaling.{key} must be positive")

    @staticmethod
    def _check_mlp(mlp: dict, where: str) -> None:
        kind = mlp.get("kind", "dense")
        if kind == "dense":
            _positive_int(_need(mlp, "ff", where), where + ".ff")
            return
        if kind != "moe":
            raise ConfigError(f"{where}.kind {kind!r}: this design's feed-forward is 'dense' or 'moe' (or null for none)")
        ex = _need(mlp, "expert", where)
        _positive_int(_need(ex, "ff", where + ".expert"), where + ".expert.ff")
        _number(_need(ex, "limit", where + ".expert"), where + ".expert.limit")
        r = _need(mlp, "router", where)
        E = _positive_int(_need(r, "experts", where + ".router"), where + ".router.experts")
        top = _positive_int(_need(r, "top", where + ".router"), where + ".router.top")
        ident = r.get("identity") or 0
        if not isinstance(ident, int) or ident < 0:
            raise ConfigError(f"{where}.router.identity must be a non-negative integer")
        if top > E + ident:
            raise ConfigError(f"{where}.router.top {top} exceeds the {E + ident} experts")
        sh = mlp.get("shared")
        if sh is not None:
            _positive_int(_need(sh, "ff", where + ".shared"), where + ".shared.ff")
            _number(_need(sh, "limit", where + ".shared"), where + ".shared.limit")

    # ---- derived ----------------------------------------------------------------

    def n_params(self) -> int:
        return sum(math.prod(t.shape) for t in self.to_spec().tensors() if -1 not in t.shape)   # (a table of unknown length is left out)

    def summary(self) -> str:
        kinds = "".join("-" if not l.get("mlp") else l["mlp"].get("kind", "dense")[0] for l in self.layers)
        return (f"voserax: {len(self.layers)} attention layers (feed-forwards {kinds}), width {self.width}, "
                f"{self.streams or 1} streams, vocab {self.vocab}, eps {self.eps:g}, "
                f"{self.n_params() / 1e6:.1f} M params, {self.torch_dtype}")

    # ---- description as parts ------------------------------------------------

    def _mixer(self, i: int, m: dict, first_mixing):
        d, p = self.width, f"l{i}.mix."
        H, G, D, Dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
        taps = int(m.get("conv") or 0)
        mask = m.get("mask")
        tensors = dict(q=TensorSpec(p + "q", (H * D, d)), k=TensorSpec(p + "k", (G * D, d)),
                       v=TensorSpec(p + "v", (G * Dv, d)), o=TensorSpec(p + "o", (d, H * Dv)))
        if taps:
            tensors.update(q_conv=TensorSpec(p + "q.conv", (H * D, taps), "vector", (0.0, 0.5)),
                           k_conv=TensorSpec(p + "k.conv", (G * D, taps), "vector", (0.0, 0.5)),
                           v_conv=TensorSpec(p + "v.conv", (G * Dv, taps), "vector", (0.0, 0.5)))
        v_mix = None
        if m.get("v_mix"):
            # the first layer that mixes gives its values to the later ones; its own weight, if a file stores one, is
            # unused (and ignored)
            v_mix = "source" if first_mixing is None else "mix"
            if v_mix == "mix":
                tensors["v_mix"] = TensorSpec(p + "vmix", (), "vector", (0.5, 0.1))
        mixer = PartSpec("gqa_attention", dict(
            hidden_size=d, n_heads=H, n_kv_heads=G, head_dim=D, v_head_dim=Dv, scale=float(m["scale"]),
            window=mask["size"] if mask else None, keep_first=0, qk_norm_eps=None, own_kv=True,
            conv_taps=taps, sink=SINK_WEIGHT, v_mix=v_mix, v_mix_key="values of the first mixing layer"), tensors)
        position = None
        rot = m.get("rot")
        if rot:
            params = dict(n_rot=rot["dims"], base=float(rot["base"]), angles="float32")
            sc = rot.get("scaling")
            if sc:
                params["scaling"] = dict(factor=float(sc["factor"]), original=float(sc["original"]),
                                         fast=float(sc["fast"]), slow=float(sc["slow"]),
                                         amplitude_slope=ROT_AMPLITUDE_SLOPE)
            position = PartSpec("rope_neox", params)
        return mixer, position

    def _feed_forward(self, i: int, mlp):
        d, p = self.width, f"l{i}.mlp."
        if mlp is None:
            return PartSpec("none", {}, {})
        if mlp.get("kind", "dense") == "dense":
            F = mlp["ff"]
            return PartSpec("gated_mlp", dict(hidden_size=d, intermediate_size=F, activation="relu"),
                            dict(gate=TensorSpec(p + "gate", (F, d)), up=TensorSpec(p + "up", (F, d)),
                                 down=TensorSpec(p + "down", (d, F))))
        r, F, limit = mlp["router"], mlp["expert"]["ff"], float(mlp["expert"]["limit"])
        E, ident = r["experts"], int(r.get("identity") or 0)
        tensors = {"router": TensorSpec(p + "router", (E + ident, d)),
                   "correction": TensorSpec(p + "correction", (E + ident,), "vector", (0.0, 0.01))}
        for e in range(E):
            tensors[f"gate{e}"] = TensorSpec(f"{p}e{e}.gate", (F, d))
            tensors[f"up{e}"] = TensorSpec(f"{p}e{e}.up", (F, d))
            tensors[f"down{e}"] = TensorSpec(f"{p}e{e}.down", (d, F))
        params = dict(hidden_size=d, intermediate_size=F, n_experts=E, n_identity=ident, top=r["top"], score="softmax",
                      n_groups=1, keep_groups=1, group_score_top=1, normalize=False, normalize_eps=0.0, scale=1.0,
                      activation="clamped_swish", act_slope=EXPERT_GATE_SLOPE, act_limit=limit,
                      act_up_shift=EXPERT_UP_SHIFT)
        sh = mlp.get("shared")
        if sh:
            Fs = sh["ff"]
            params.update(shared_size=Fs, shared_limit=float(sh["limit"]), shared_gate="sigmoid")
            tensors.update(shared_gate=TensorSpec(p + "shared.gate", (Fs, d)), shared_up=TensorSpec(p + "shared.up", (Fs, d)),
                           shared_down=TensorSpec(p + "shared.down", (d, Fs)),
                           shared_sg=TensorSpec(p + "shared.sg", (1, d)))
        return PartSpec("routed_experts", params, tensors)

    def to_spec(self) -> ModelSpec:
        d, eps, S = self.width, self.eps, self.streams
        blocks, first_mixing = [], None
        for i, layer in enumerate(self.layers):
            p = f"l{i}."
            mixer, position = self._mixer(i, layer["mixer"], first_mixing)
            if layer["mixer"].get("v_mix") and first_mixing is None:
                first_mixing = i
            ffn = self._feed_forward(i, layer.get("mlp"))
            norms = dict(mixer=PartSpec("rms_norm", dict(size=d, eps=eps), dict(gain=TensorSpec(p + "norm1", (d,), "vector"))))
            if ffn.kind != "none":
                norms["feed_forward"] = PartSpec("rms_norm", dict(size=d, eps=eps),
                                                 dict(gain=TensorSpec(p + "norm2", (d,), "vector")))
            if S:
                # the connection weights ride with the norm of their sublayer
                for role, q in (("mixer", "hc1"), ("feed_forward", "hc2")):
                    if role in norms:
                        n = norms[role]
                        norms[role] = PartSpec("rms_norm", n.params, dict(
                            n.tensors, hc_in=TensorSpec(f"{p}{q}.in", (S,), "vector", (0.5, 0.2)),
                            hc_out=TensorSpec(f"{p}{q}.out", (S,), "vector", (1.0, 0.2)),
                            hc_mix=TensorSpec(f"{p}{q}.mix", (S, S), "vector", (1.0 / S, 0.1 / S))))
            blocks.append(BlockSpec("hyper_connections", mixer, ffn, norms, position,
                                    dict(streams=max(1, S), residual_mult=self.residual_mult)))
        # What a file may carry although this configuration does not use it (a weight of a switched-off option):
        # left alone, not an error.
        used = {t.name for b in blocks for part in (b.mixer, b.feed_forward, *b.norms.values()) for t in part.tensors.values()}
        optional = []
        for i in range(len(blocks)):
            p = f"l{i}."
            optional += [p + "mix.vmix", p + "mix.q.conv", p + "mix.k.conv", p + "mix.v.conv", p + "norm2", p + "mlp.correction"]
            optional += [f"{p}{q}.{w}" for q in ("hc1", "hc2") for w in ("in", "out", "mix")]
        ignored = tuple(n for n in optional if n not in used) + (() if self.learned_positions else ("pos",))
        emb_tensors = dict(table=TensorSpec("embed", (self.vocab, d)))
        if self.learned_positions:
            emb_tensors["positions"] = TensorSpec("pos", (self.max_positions or -1, d))
        return ModelSpec(
            architecture="Voserax", hidden_size=d, vocab_size=self.vocab,
            embedding=PartSpec("gather", dict(scale=None), emb_tensors),
            blocks=tuple(blocks), schedule=tuple(LayerCall(layer=i, cache=i) for i in range(len(blocks))),
            final_norm=PartSpec("rms_norm", dict(size=d, eps=eps), dict(gain=TensorSpec("final.norm", (d,), "vector"))),
            head=PartSpec("linear", dict(tied=True, softcap=None), {}),
            max_positions=self.max_positions or (1 << 20), stop_ids=(), storage_dtype=self.torch_dtype,
            default_sampling={}, residual_streams=max(1, S), ignored_tensors=ignored,
        )
