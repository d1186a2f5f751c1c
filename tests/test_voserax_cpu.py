"""CPU: the Voserax configuration and its description as parts, the scaled rotation table's frequencies, and the
plain implementation's own mechanisms against closed forms."""

import copy
import math

import pytest
import torch

import plain_voserax as plain
from voserax_configs import ALL, VX_A, VX_B, VX_D

from llmoxide_b200.config import VoseraxConfig, read_config
from llmoxide_b200.errors import ConfigError


def test_config_is_chosen_by_name_and_round_trips():
    for raw in ALL.values():
        cfg = read_config(copy.deepcopy(raw))
        assert isinstance(cfg, VoseraxConfig)
        again = read_config(cfg.to_dict())
        assert again.to_dict() == cfg.to_dict()
        assert "voserax" in cfg.summary()


def test_description_names_every_tensor_once_with_the_shapes_of_the_configuration():
    spec = read_config(copy.deepcopy(VX_A)).to_spec()
    names = [t.name for t in spec.tensors()]
    assert len(names) == len(set(names))
    shapes = {t.name: tuple(t.shape) for t in spec.tensors()}
    assert shapes["embed"] == (211, 96) and shapes["pos"] == (512, 96) and "head" not in shapes
    assert shapes["l0.mix.q"] == (4 * 32, 96) and shapes["l0.mix.v"] == (2 * 16, 96) and shapes["l0.mix.o"] == (96, 4 * 16)
    assert shapes["l0.mix.q.conv"] == (128, 3) and shapes["l2.mix.k.conv"] == (48, 2) and shapes["l2.mix.v.conv"] == (32, 2)
    assert shapes["l3.mix.vmix"] == () and not any(f"l{i}.mix.vmix" in shapes for i in (0, 1, 2))   # 1 is the source
    assert spec.is_ignored("l1.mix.vmix") and spec.is_ignored("l2.norm2") and not spec.is_ignored("l3.mix.vmix")
    assert shapes["l0.mlp.gate"] == (72, 96) and shapes["l1.mlp.router"] == (8, 96) and shapes["l1.mlp.correction"] == (8,)
    assert shapes["l1.mlp.e5.down"] == (96, 40) and "l1.mlp.e6.gate" not in shapes          # 6 experts + 2 identity
    assert shapes["l1.mlp.shared.sg"] == (1, 96) and shapes["l1.mlp.shared.up"] == (24, 96)
    assert "l3.mlp.shared.gate" not in shapes and shapes["l3.mlp.router"] == (5, 96)
    assert shapes["l0.hc1.in"] == (3,) and shapes["l0.hc2.mix"] == (3, 3) and "l2.hc2.in" not in shapes and "l2.norm2" not in shapes
    assert spec.residual_streams == 3 and spec.head.get("tied")
    # the first layer that mixes values is their source; the later ones mix
    assert [b.mixer.get("v_mix") for b in spec.blocks] == [None, "source", None, "mix"]
    assert [b.mixer["conv_taps"] for b in spec.blocks] == [3, 3, 2, 3] and spec.blocks[0].mixer["sink"] == 1.0
    assert spec.blocks[0].position["scaling"]["factor"] == 4.0 and spec.blocks[1].position.get("scaling") is None
    assert spec.blocks[3].position is None and spec.blocks[2].feed_forward.kind == "none"
    ff = spec.blocks[1].feed_forward
    assert (ff["n_experts"], ff["n_identity"], ff["top"], ff["score"], ff["normalize"]) == (6, 2, 2, "softmax", False)
    assert ff["act_limit"] == 1.5 and ff["shared_limit"] == 0.8 and ff["act_slope"] == 1.702
    # without 'streams' there are no connection weights and one copy of the stream
    spec_d = read_config(copy.deepcopy(VX_D)).to_spec()
    assert spec_d.residual_streams == 1 and not any(".hc" in t.name for t in spec_d.tensors())
    assert spec_d.blocks[0].mixer["conv_taps"] == 0 and spec_d.blocks[0].mixer["window"] is None


@pytest.mark.parametrize("change, word", [
    (lambda c: c["layers"][0].__setitem__("type", "retention"), "type"),
    (lambda c: c["layers"][0]["mixer"].__setitem__("kv_heads", 3), "multiple"),
    (lambda c: c["layers"][0]["mixer"]["rot"].__setitem__("dims", 34), "rot.dims"),
    (lambda c: c["layers"][0]["mixer"]["rot"]["scaling"].pop("slow"), "slow"),
    (lambda c: c["layers"][3]["mixer"].__setitem__("vdim", 8), "v_mix"),
    (lambda c: c["layers"][1]["mlp"]["router"].__setitem__("top", 9), "top"),
    (lambda c: c["layers"][1]["mlp"]["expert"].pop("limit"), "limit"),
    (lambda c: c["layers"][0]["mlp"].__setitem__("kind", "conv"), "kind"),
    (lambda c: c.__setitem__("streams", 9), "streams"),
    (lambda c: c.pop("norm"), "norm"),
    (lambda c: c["layers"][0]["mixer"].pop("scale"), "scale"),
    (lambda c: c["layers"][0]["mixer"].__setitem__("conv", 17), "taps"),
])
def test_inconsistent_configurations_are_refused(change, word):
    raw = copy.deepcopy(VX_A)
    change(raw)
    with pytest.raises(ConfigError) as e:
        read_config(raw)
    assert word in str(e.value)


def test_scaled_frequencies_of_the_rotation_part_are_the_plain_ones():
    """The package's table frequencies (``RotaryNeox._scaling``) against the oracle's, and the ramp's ends: pairs that
    turn fast keep their frequency, pairs that turn slowly have it divided by the factor."""
    from llmoxide_b200.config.spec import PartSpec
    from llmoxide_b200.parts.position import RotaryNeox
    from llmoxide_b200.parts.runtime import Runtime

    rt = Runtime(dtype="float32", device=torch.device("cpu"), max_positions=8)
    for dims, base, sc in ((16, 10000.0, (4.0, 64, 8.0, 1.0)), (48, 500.0, (2.0, 128, 16.0, 2.0)), (64, 10000.0, (2.0, 256, 32.0, 1.0)),
                           (12, 10000.0, (8.0, 32, 4.0, 1.0)), (32, 10000.0, None)):
        params = dict(n_rot=dims, base=base, angles="float32")
        scaling = None
        if sc:
            scaling = dict(factor=sc[0], original=sc[1], fast=sc[2], slow=sc[3])
            params["scaling"] = dict(scaling, amplitude_slope=0.1)
        part = RotaryNeox(PartSpec("rope_neox", params), {}, rt)
        freqs, amp = part._scaling()
        want, want_amp = plain.scaled_frequencies(dims, base, scaling)
        assert torch.allclose(torch.tensor(freqs, dtype=torch.float64), want, rtol=1e-15, atol=0)
        assert amp == pytest.approx(want_amp, rel=1e-15)
        plain_f = [base ** (-2.0 * i / dims) for i in range(dims // 2)]
        if sc:
            assert freqs[0] == plain_f[0] and freqs[-1] == pytest.approx(plain_f[-1] / sc[0], rel=1e-12)
            assert amp == pytest.approx(0.1 * math.log(sc[0]) + 1.0)
        cos, sin, n = part.rotary_tables()
        p = 5
        assert torch.allclose(cos[p].double(), torch.cos(p * want) * want_amp, atol=2e-6)
        assert torch.allclose(sin[p].double(), torch.sin(p * want) * want_amp, atol=2e-6)


def test_plain_sink_softmax_and_window_against_closed_forms():
    # one query, one key: the weight is e^s / (1 + e^s)
    q = torch.tensor([[[2.0, 0.0]]], dtype=plain.F)
    k = torch.tensor([[[1.5, 0.0]]], dtype=plain.F)
    v = torch.tensor([[[4.0]]], dtype=plain.F)
    out = plain.sink_softmax_attention(q, k, v, 0.5, None)
    s = 2.0 * 1.5 * 0.5
    assert out[0, 0].item() == pytest.approx(4.0 * math.exp(s) / (1.0 + math.exp(s)), rel=1e-14)
    # zero scores over a window of 3: every seen key weighs 1 / (1 + seen)
    T = 6
    q = torch.zeros((T, 1, 2), dtype=plain.F)
    k = torch.zeros((T, 1, 2), dtype=plain.F)
    v = torch.arange(1.0, T + 1, dtype=plain.F).view(T, 1, 1)
    out = plain.sink_softmax_attention(q, k, v, 1.0, 3)
    for i in range(T):
        seen = list(range(max(0, i - 2), i + 1))
        assert out[i, 0].item() == pytest.approx(sum(j + 1.0 for j in seen) / (1 + len(seen)), rel=1e-14)


def test_plain_convolution_and_hyper_connections_against_closed_forms():
    u = torch.arange(1.0, 6.0, dtype=plain.F).view(5, 1)
    w = torch.tensor([[100.0, 10.0, 1.0]], dtype=plain.F)          # the last tap is the token itself
    assert plain.short_convolution(u, w).view(-1).tolist() == [1.0, 12.0, 123.0, 234.0, 345.0]
    # identity mixing, unit weights: the streams all get mult * y, and the read is their sum
    S, T, d = 3, 4, 8
    X = torch.randn(S, T, d, dtype=plain.F)
    W = {"hc.in": torch.ones(S, dtype=plain.F), "hc.out": torch.ones(S, dtype=plain.F), "hc.mix": torch.eye(S, dtype=plain.F)}
    seen = []
    new = plain.hyper_sublayer(X, W, "hc.", 0.5, torch.ones(d, dtype=plain.F), 1e-6, lambda h: (seen.append(h), 2.0 * h)[1])
    u = X.sum(0)
    assert torch.allclose(seen[0], plain.rms_norm(u, torch.ones(d, dtype=plain.F), 1e-6))
    assert torch.allclose(new, X + 0.5 * 2.0 * seen[0][None])
    # [from, to]: a mix that moves stream 0 to stream 1 only
    W["hc.mix"] = torch.zeros(S, S, dtype=plain.F)
    W["hc.mix"][0, 1] = 1.0
    new = plain.hyper_sublayer(X, W, "hc.", 0.0, torch.ones(d, dtype=plain.F), 1e-6, lambda h: h)
    assert torch.equal(new[1], X[0]) and not new[0].any() and not new[2].any()


def test_plain_routing_and_experts_against_closed_forms():
    d = 4
    W = {"m.router": torch.zeros(5, d, dtype=plain.F), "m.correction": torch.tensor([0.0, 0.3, 0.0, 0.2, 0.0], dtype=plain.F)}
    h = torch.ones(2, d, dtype=plain.F)
    ids, w, s = plain.route(h, W, "m.", dict(top=2))
    assert ids.tolist() == [[1, 3], [1, 3]] and torch.allclose(w, torch.full((2, 2), 0.2, dtype=plain.F))  # weights without the correction
    # an identity expert returns its input times the weight; the clamps act on gate and up
    W.update({"m.e0.gate": torch.eye(d, dtype=plain.F) * 5, "m.e0.up": -torch.eye(d, dtype=plain.F) * 5,
              "m.e0.down": torch.eye(d, dtype=plain.F)})
    y = plain.clamped_expert(h, W, "m.e0.", 2.0)
    g = 2.0
    assert torch.allclose(y, torch.full((2, d), g / (1 + math.exp(-1.702 * g)) * (-2.0 + 1.0), dtype=plain.F))
    W["m.router"] = torch.zeros(3, d, dtype=plain.F)
    W["m.correction"] = torch.tensor([-1.0, 0.0, 1.0], dtype=plain.F)
    out = plain.mixture(h, W, "m.", dict(router=dict(experts=1, top=2, identity=2), expert=dict(ff=d, limit=2.0)))
    assert torch.allclose(out, 2 * h / 3)       # the two identity experts, each with weight 1/3


def test_without_max_positions_the_position_table_has_the_rows_the_file_has():
    from llmoxide_b200.weights.loader import check_checkpoint

    raw = copy.deepcopy(VX_D)
    raw.pop("max_positions")
    cfg = read_config(raw)
    spec = cfg.to_spec()
    assert [t.shape for t in spec.tensors() if t.name == "pos"] == [(-1, 64)] and "max_positions" not in cfg.to_dict()
    assert "voserax" in cfg.summary()

    class Entry:
        def __init__(self, shape):
            self.shape, self.dtype = shape, "BF16"

    entries = {t.name: Entry(tuple(300 if n == -1 else n for n in t.shape)) for t in spec.tensors()}
    assert check_checkpoint(spec, entries) == []
    entries["pos"] = Entry((300, 65))
    from llmoxide_b200.errors import WeightsError
    with pytest.raises(WeightsError):
        check_checkpoint(spec, entries)
