"""CPU: the Tifapel configuration and its description as parts, the cache's bookkeeping for windows that keep
their first tokens, and the plain implementation's own mechanisms against closed forms."""

import copy

import numpy as np
import pytest
import torch

import plain_tifapel as plain
from tifapel_configs import ALL, TF_A, TF_B

from llmoxide_b200.cache import PAGE, CacheAllocator
from llmoxide_b200.config import TifapelConfig, read_config
from llmoxide_b200.errors import ConfigError


def test_config_is_chosen_by_name_and_round_trips():
    for raw in ALL.values():
        cfg = read_config(copy.deepcopy(raw))
        assert isinstance(cfg, TifapelConfig)
        again = read_config(cfg.to_dict())
        assert again.to_dict() == cfg.to_dict()
        assert "tifapel" in cfg.summary()


def test_description_names_every_tensor_once_and_shares_cache_entries():
    spec = read_config(copy.deepcopy(TF_A)).to_spec()
    names = [t.name for t in spec.tensors()]
    assert len(names) == len(set(names))
    assert "l3.mix.k" not in names and "l3.mix.v" not in names and "l0.mix.k" in names      # the reader has no k/v
    assert "l2.mlp.router" not in names and "l1.mix.norm" in names and "l2.mix.norm" not in names
    shapes = {t.name: tuple(t.shape) for t in spec.tensors()}
    assert shapes["l0.mix.q"] == (4 * 32, 96) and shapes["l0.mix.v"] == (2 * 16, 96) and shapes["l0.mix.o"] == (96, 4 * 16)
    assert shapes["l2.mix.g"] == (2 * 40, 96) and shapes["l1.mlp.e7.down"] == (96, 40) and shapes["head"] == (211, 96)
    calls = spec.schedule
    assert calls[3].cache == calls[0].cache and not calls[3].writes_cache and calls[0].writes_cache
    assert len({c.cache for c in calls}) == 3
    # the shared entry keeps what the wider of the two masks sees
    m0, m3 = spec.blocks[0].mixer, spec.blocks[3].mixer
    assert (m0["window"], m0["keep_first"], m3["window"], m3["keep_first"]) == (20, 3, 33, 1)
    assert m0["cache_window"] == m3["cache_window"] == 33 and m0["cache_keep_first"] == m3["cache_keep_first"] == 3
    # a reader without a mask keeps everything
    spec_b = read_config(copy.deepcopy(TF_B)).to_spec()
    assert spec_b.blocks[2].mixer["cache_window"] is None and spec_b.blocks[1].mixer["cache_window"] == 130


@pytest.mark.parametrize("change, word", [
    (lambda c: c["layers"][0].__setitem__("type", "conv"), "type"),
    (lambda c: c["layers"][3]["mixer"].__setitem__("kv_from", 3), "earlier"),
    (lambda c: c["layers"][3]["mixer"].__setitem__("kv_from", 1), "keys and values"),
    (lambda c: c["layers"][3]["mixer"].__setitem__("dim", 16), "differs"),
    (lambda c: c["layers"][1]["mixer"].__setitem__("decay", [0.5]), "decay"),
    (lambda c: c["layers"][2]["mixer"]["rot"].__setitem__("dims", 34), "rot.dims"),
    (lambda c: c["layers"][0]["mlp"]["router"].__setitem__("top", 5), "top"),
    (lambda c: c["layers"][0]["mlp"]["router"]["groups"].__setitem__("count", 3), "groups"),
    (lambda c: c.pop("norm"), "norm"),
    (lambda c: c["layers"][0]["mixer"].pop("scale"), "scale"),
])
def test_inconsistent_configurations_are_refused(change, word):
    raw = copy.deepcopy(TF_A)
    change(raw)
    with pytest.raises(ConfigError, match=word):
        read_config(raw)


def test_window_pages_are_given_back_but_never_the_kept_first_ones():
    # one group with a window of 70 that keeps its first 70 tokens (two pages), one plain window of 70
    al = CacheAllocator(n_slots=2, n_pages=32, windows=[70, 70], keep_first=[70, 0])
    s = al.acquire()
    al.reserve(s, 5 * PAGE)
    al.commit(s, 5 * PAGE)
    kept, plain_row = al.page_row(s, 0), al.page_row(s, 1)
    # the next query sits at 320 and sees keys from 251 on: pages 0..2 are dead for the plain window
    assert [p >= 0 for p in plain_row] == [False, False, False, True, True]
    assert [p >= 0 for p in kept] == [True, True, False, True, True]
    for _ in range(3 * PAGE):
        al.reserve(s, 1)
        al.commit(s, 1)
    assert [p >= 0 for p in al.page_row(s, 0)] == [True, True] + [False] * 4 + [True, True, True][:2]
    al.check_consistent()
    al.release(s)
    assert al.pages_held(0) == 0 and al.pages_held(1) == 0
    # keep_first within the first page
    al = CacheAllocator(n_slots=1, n_pages=8, windows=[10], keep_first=[4])
    s = al.acquire()
    al.reserve(s, 200)
    al.commit(s, 200)
    assert [p >= 0 for p in al.page_row(s, 0)] == [True, False, True, True]      # the next query (200) sees 191 on: page 2


def test_plain_recurrence_equals_its_closed_form():
    torch.manual_seed(0)
    T, H, D, Dv = 9, 2, 3, 4
    q, k, v = (torch.randn(T, H, n, dtype=plain.F) for n in (D, D, Dv))
    decay = [0.5, 0.9]
    got = plain.decayed_outer_product_scan(q, k, v, decay)
    for h in range(H):
        for t in range(T):
            want = sum(decay[h] ** (t - j) * (q[t, h] @ k[j, h]) * v[j, h] for j in range(t + 1))
            assert torch.allclose(got[t, h], want, atol=1e-12)


def test_plain_rotation_turns_pairs_and_keeps_the_rest():
    x = torch.arange(1.0, 7.0, dtype=plain.F).view(1, 1, 6).repeat(3, 1, 1)
    y = plain.rotate_half(x, torch.arange(3), 4, 100.0)
    assert torch.equal(y[0], x[0]) and torch.equal(y[..., 4:], x[..., 4:])
    a0, a1 = 2 * 1.0, 2 * 100.0 ** -0.5            # position 2; pairs (0, 2) and (1, 3)
    want = [1 * np.cos(a0) - 3 * np.sin(a0), 2 * np.cos(a1) - 4 * np.sin(a1),
            3 * np.cos(a0) + 1 * np.sin(a0), 4 * np.cos(a1) + 2 * np.sin(a1)]
    assert np.allclose(y[2, 0, :4].numpy(), want, atol=1e-12)


def test_plain_mask_and_router_rules():
    mask = dict(size=3, keep_first=2)
    assert [j for j in range(8) if plain.visible(6, j, mask)] == [0, 1, 4, 5, 6]
    assert [j for j in range(8) if plain.visible(1, j, mask)] == [0, 1]
    assert [j for j in range(5) if plain.visible(3, j, None)] == [0, 1, 2, 3]
    # scores 0.9 and 0.1 | 0.6 and 0.55 | 0.7 and 0.2: group sums 1.0, 1.15, 0.9 -> group 1 alone may be chosen from
    s = torch.tensor([[0.9, 0.1, 0.6, 0.55, 0.7, 0.2]], dtype=plain.F)
    z = torch.log(s / (1 - s))
    ids, w = plain.route(z, torch.eye(6, dtype=plain.F), dict(top=2, scale=3.0, groups=dict(count=3, keep=1)))
    assert ids.tolist() == [[2, 3]]
    assert np.allclose(w.numpy(), [[3.0 * 0.6 / 1.15, 3.0 * 0.55 / 1.15]])
    ids, _ = plain.route(z, torch.eye(6, dtype=plain.F), dict(top=2, scale=1.0, groups=dict(count=3, keep=2)))
    assert ids.tolist() == [[0, 2]]
    ids, _ = plain.route(z, torch.eye(6, dtype=plain.F), dict(top=3, scale=1.0))
    assert ids.tolist() == [[0, 4, 2]]
