"""GPU: the Tifapel decoder's mechanisms one by one against the plain implementation (tests/plain_tifapel.py),
then whole models under every way of cutting the same requests into steps, and greedy generation through the
package's own entry point."""

import copy

import numpy as np
import pytest
import torch

import plain_tifapel as plain
import replay_util as ru
from tifapel_configs import ALL, make_folder
from tiny_configs import prompts

pytestmark = pytest.mark.gpu

DEV = "cuda:0"
F32_TOL, BF16_TOL = 2e-5, 3e-2


def _rel(got, want):
    want = np.asarray(want, dtype=np.float64)
    return float(np.abs(np.asarray(got, dtype=np.float64) - want).max() / max(np.abs(want).max(), 1e-30))


def _bf16_exact(t):
    return t.to(torch.bfloat16).to(torch.float64)


# ---------------------------------------------------------------------------------------------------------
# routing
# ---------------------------------------------------------------------------------------------------------

@pytest.mark.parametrize("E, top, groups", [(12, 2, (2, 1)), (8, 3, (4, 2)), (6, 2, (6, 3)), (6, 1, None),
                                            (4, 4, None), (10, 2, (5, 2)), (64, 6, (8, 3)), (33, 5, (3, 3))])
def test_routing_matches_the_plain_rule(E, top, groups):
    from llmoxide_b200 import kernels

    torch.manual_seed(E * 100 + top)
    T = 301
    z = (torch.randn(T, E, dtype=torch.float64) * 2.0).float()
    r = dict(top=top, scale=1.7)
    if groups:
        r["groups"] = dict(count=groups[0], keep=groups[1])
    want_ids, want_w = plain.route(z.double(), torch.eye(E, dtype=torch.float64), r)
    ids = torch.empty((T, top), dtype=torch.int32, device=DEV)
    w = torch.empty((T, top), dtype=torch.float32, device=DEV)
    kernels.moe_route(z.to(DEV), ids, w, top, groups[0] if groups else 1, groups[1] if groups else 1, 2, "sigmoid",
                      True, 1e-20, 1.7)
    assert torch.equal(ids.cpu().long(), want_ids)
    assert _rel(w.cpu().numpy(), want_w.numpy()) < 1e-6


def test_the_sort_puts_every_pair_into_its_experts_tiles():
    from llmoxide_b200 import kernels

    torch.manual_seed(3)
    for T, top, E in ((1, 2, 12), (77, 3, 8), (5000, 2, 5)):
        ids = torch.stack([torch.randperm(E)[:top] for _ in range(T)]).to(torch.int32).to(DEV)
        P = T * top
        perm = torch.empty(P, dtype=torch.int32, device=DEV)
        tiles = torch.empty((kernels.moe_max_tiles(P, E), 3), dtype=torch.int32, device=DEV)
        kernels.moe_sort(ids, E, perm, tiles)
        perm, tiles, flat = perm.cpu().numpy(), tiles.cpu().numpy(), ids.cpu().numpy().reshape(-1)
        assert sorted(perm.tolist()) == list(range(P))
        seen = 0
        for e, row0, n in tiles[tiles[:, 0] >= 0]:
            assert 0 < n <= kernels.MOE_TILE and row0 == seen
            assert (flat[perm[row0 : row0 + n]] == e).all()
            seen += n
        assert seen == P


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_routed_experts_part_against_the_plain_experts(dtype):
    from llmoxide_b200.config.spec import PartSpec, TensorSpec
    from llmoxide_b200.parts import Runtime
    from llmoxide_b200.parts.experts import RoutedExperts

    torch.manual_seed(5)
    d, F, E, top = 72, 40, 6, 2
    w = {"r": torch.randn(E, d) * 0.3}
    for e in range(E):
        w[f"g{e}"], w[f"u{e}"], w[f"d{e}"] = torch.randn(F, d) * 0.2, torch.randn(F, d) * 0.2, torch.randn(d, F) * 0.2
    w = {k: _bf16_exact(v) for k, v in w.items()}
    tensors = {"router": TensorSpec("r", (E, d))}
    for e in range(E):
        tensors.update({f"gate{e}": TensorSpec(f"g{e}", (F, d)), f"up{e}": TensorSpec(f"u{e}", (F, d)),
                        f"down{e}": TensorSpec(f"d{e}", (d, F))})
    spec = PartSpec("routed_experts", dict(hidden_size=d, intermediate_size=F, n_experts=E, top=top, score="sigmoid",
                                           n_groups=3, keep_groups=2, group_score_top=2, normalize=True,
                                           normalize_eps=1e-20, scale=1.5, activation="silu"), tensors)
    rt = Runtime(dtype="float32" if dtype == torch.float32 else "bfloat16", device=torch.device(DEV), max_positions=64)
    part = RoutedExperts(spec, {k: v.to(dtype).to(DEV) for k, v in w.items()}, rt)
    for T in (1, 3, 130, 1300):      # one row, a few, rows for tiles of 16, 64 and 128
        x = _bf16_exact(torch.randn(T, d))
        y = part.forward(x.to(dtype).to(DEV), None)
        assert y.shape == (top, T, d) and y.dtype == torch.float32
        pw = {"router": w["r"]}
        for e in range(E):
            pw.update({f"e{e}.gate": w[f"g{e}"], f"e{e}.up": w[f"u{e}"], f"e{e}.down": w[f"d{e}"]})
        want = plain.experts(x, pw, "", dict(router=dict(top=top, scale=1.5, groups=dict(count=3, keep=2))))
        assert _rel(y.sum(0).cpu().numpy(), want.numpy()) < (1e-5 if dtype == torch.float32 else 1e-2)


# ---------------------------------------------------------------------------------------------------------
# the recurrence
# ---------------------------------------------------------------------------------------------------------

def _scan_inputs(T, H, D, Dv, seed):
    g = torch.Generator().manual_seed(seed)
    N = 2 * H * D + 2 * H * Dv
    return _bf16_exact(torch.randn(T, N, generator=g))


@pytest.mark.parametrize("H, D, Dv, n_rot, act, per_head", [
    (2, 32, 64, 0, "silu", False), (3, 20, 12, 20, "none", True), (2, 64, 40, 16, "none", True),
    (1, 128, 128, 128, "none", True), (2, 6, 5, 4, "silu", False), (1, 200, 33, 0, "none", False)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_recurrence_norm_and_gate_against_the_plain_functions(H, D, Dv, n_rot, act, per_head, dtype):
    """Three sequences of unequal lengths in one step, then continued in portions (two tokens, one token, the
    rest): every cutting gives the same bits, and all agree with the plain recurrence."""
    from llmoxide_b200 import kernels

    lens, decay, base, eps = [37, 1, 70], [0.5, 0.97, 0.999][:H], 10000.0, 1e-5
    k_scale = D ** -0.5 if act == "none" else 1.0
    gate = "silu" if per_head else "sigmoid"
    half = n_rot // 2
    pos = np.arange(128, dtype=np.float32)
    freq = np.array([np.float32(base ** (-2.0 * i / n_rot)) for i in range(half)], dtype=np.float32)
    ang = (pos[:, None] * freq[None, :]).astype(np.float64) if half else np.zeros((128, 0))
    cos = torch.tensor(np.cos(ang), dtype=torch.float32, device=DEV) if half else None
    sin = torch.tensor(np.sin(ang), dtype=torch.float32, device=DEV) if half else None
    gain = None if per_head else (1 + 0.1 * torch.randn(H * Dv, generator=torch.Generator().manual_seed(1))).float()
    projs = [_scan_inputs(n, H, D, Dv, 10 + i) for i, n in enumerate(lens)]
    HD, HDv = H * D, H * Dv

    def plain_out(p):
        T = p.shape[0]
        q, k, v, g = p[:, :HD], p[:, HD : 2 * HD], p[:, 2 * HD : 2 * HD + HDv], p[:, 2 * HD + HDv :]
        if act == "silu":
            q, k, v = plain.silu(q), plain.silu(k), plain.silu(v)
        q, k, v = q.reshape(T, H, D), k.reshape(T, H, D), v.reshape(T, H, Dv)
        if n_rot:
            # the same float32 angles as the tables hold
            c, s = torch.tensor(np.cos(ang[:T]))[:, None, :], torch.tensor(np.sin(ang[:T]))[:, None, :]
            rot = lambda x: torch.cat([x[..., :half] * c - x[..., half:n_rot] * s,
                                       x[..., half:n_rot] * c + x[..., :half] * s, x[..., n_rot:]], -1)
            q, k = rot(q), rot(k)
        o = plain.decayed_outer_product_scan(q, k * k_scale, v, decay)
        if per_head:
            o = plain.rms(o, eps).reshape(T, HDv) * plain.silu(g)
        else:
            o = plain.rms_norm(o.reshape(T, HDv), gain.double(), eps) * torch.sigmoid(g)
        return o

    def run(cuts, seg_len=0):
        """cuts[i]: the portions sequence i arrives in; portion j of every sequence that still has one forms step j."""
        state = torch.zeros((4, H, D, Dv), dtype=torch.float32, device=DEV)
        slots = [2, 0, 3]
        outs = [[] for _ in lens]
        fed = [0] * len(lens)
        for j in range(max(len(c) for c in cuts)):
            live = [i for i in range(len(lens)) if j < len(cuts[i])]
            rows = torch.cat([projs[i][fed[i] : fed[i] + cuts[i][j]] for i in live]).to(dtype).to(DEV)
            counts = [cuts[i][j] for i in live]
            start = torch.tensor(np.concatenate([[0], np.cumsum(counts)]), dtype=torch.int32, device=DEV)
            past = torch.tensor(np.concatenate([np.arange(fed[i], fed[i] + cuts[i][j]) for i in live]),
                                dtype=torch.int32, device=DEV)             # every token's position
            slot = torch.tensor([slots[i] for i in live], dtype=torch.int32, device=DEV)
            o = torch.empty((rows.shape[0], HDv), dtype=torch.float32, device=DEV)
            kernels.decay_scan(rows, o, state, start, past, slot, torch.tensor(decay, device=DEV), cos, sin, n_rot, act,
                               k_scale, H, D, Dv, 0, HD, 2 * HD, max_new=max(counts), seg_len=seg_len)
            y = torch.empty((rows.shape[0], HDv), dtype=dtype, device=DEV)
            kernels.gated_norm(o, rows, 2 * HD + HDv, None if gain is None else gain.to(DEV), eps, gate, per_head, y, H, Dv)
            at = 0
            for i, n in zip(live, counts):
                outs[i].append(y[at : at + n].float().cpu())
                at += n
                fed[i] += n
        return [torch.cat(o) for o in outs]

    whole = run([[n] for n in lens])
    for got, p in zip(whole, projs):
        assert _rel(got.numpy(), plain_out(p).numpy()) < (2e-5 if dtype == torch.float32 else 1e-2)
    cut = run([[2, 1, 16, 17, 1], [1], [33, 2, 2, 1, 32]])
    single = run([[1] * n for n in lens])
    for a, b, c in zip(whole, cut, single):
        assert torch.equal(a, b) and torch.equal(a, c)
    # long prompts are walked in segments side by side and put together in a second pass: the same sums, rounded
    # in another order (segments of 16 and of 24 tokens here; a later portion of a prompt in segments as well)
    for seg_len, cuts in ((16, [[n] for n in lens]), (24, [[30, 7], [1], [5, 65]])):
        for got, p in zip(run(cuts, seg_len), projs):
            assert _rel(got.numpy(), plain_out(p).numpy()) < (2e-5 if dtype == torch.float32 else 1e-2)


# ---------------------------------------------------------------------------------------------------------
# attention: a window that keeps its first tokens, values of another size
# ---------------------------------------------------------------------------------------------------------

@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("D, Dv, H, G, window, keep", [(16, 48, 6, 3, 64, 70), (32, 16, 4, 2, 20, 3), (64, 64, 8, 1, 130, 4),
                                                        (48, 48, 3, 3, 0, 0), (40, 24, 2, 1, 5, 1)])
def test_one_key_stands_out_at_every_edge_of_the_mask(D, Dv, H, G, window, keep, dtype):
    """Queries at several positions; for each, one key is made to carry nearly all the weight if it is visible:
    the last key inside the window, the first outside it, the last kept first token, the first not kept, a key
    at a page border.  The values say which key was seen."""
    from llmoxide_b200 import kernels

    torch.manual_seed(D + Dv)
    n_pos, page = 400, kernels.PAGE
    n_pages = (n_pos + page - 1) // page
    table = torch.randperm(n_pages + 3)[:n_pages].to(torch.int32)           # pages in any order
    k = _bf16_exact(torch.randn(n_pos, G, D) * 0.1)
    v = _bf16_exact(torch.randn(n_pos, G, Dv))
    queries = []
    for p in (0, 1, keep, window + keep + 1, 199, 255, 256, 399):
        if p >= n_pos or p < 0:
            continue
        targets = {p, max(0, p - 1), (p // page) * page, max(0, (p // page) * page - 1)}
        if window:
            targets |= {max(0, p - window + 1), max(0, p - window), max(0, keep - 1), min(p, keep)}
        queries += [(p, j) for j in sorted(targets) if j <= p]
    q = _bf16_exact(torch.randn(len(queries), H, D) * 0.1)
    for i, (p, j) in enumerate(queries):        # the target's key points along this query's first head of its group
        for g in range(G):
            k_dir = q[i, g * (H // G)] / q[i, g * (H // G)].norm()
            q[i, g * (H // G)] = _bf16_exact(k_dir * 6.0)
    kc = torch.zeros((n_pages + 3, G, page, D), dtype=torch.float64)
    vc = torch.zeros((n_pages + 3, G, page, Dv), dtype=torch.float64)
    outs, wants = [], []
    for i, (p, j) in enumerate(queries):
        kk = k.clone()
        for g in range(G):
            kk[j, g] = _bf16_exact(q[i, g * (H // G)] / 6.0 * 8.0)
        for pos in range(n_pos):
            kc[table[pos // page], :, pos % page] = kk[pos]
            vc[table[pos // page], :, pos % page] = v[pos]
        out = torch.empty((1, H * Dv), dtype=dtype, device=DEV)
        kernels.attention_paged(q[i].reshape(1, H * D).to(dtype).to(DEV), out, kc.to(dtype).to(DEV), vc.to(dtype).to(DEV),
                                table.view(1, -1).to(DEV), torch.zeros(1, dtype=torch.int32, device=DEV),
                                torch.tensor([p], dtype=torch.int32, device=DEV), H, G, D, window or None, 0.9,
                                v_head_dim=Dv, keep_first=keep)
        mask = dict(size=window, keep_first=keep) if window else None
        js = [x for x in range(p + 1) if plain.visible(p, x, mask)]
        want = torch.zeros(H, Dv, dtype=torch.float64)
        for hq in range(H):
            g = hq // (H // G)
            want[hq] = torch.softmax((kk[js, g] @ q[i, hq]) * 0.9, 0) @ v[js, g]
        outs.append(out.float().cpu().view(H, Dv))
        wants.append(want)
    err = _rel(torch.stack(outs).numpy(), torch.stack(wants).numpy())
    assert err < (1e-5 if dtype == torch.float32 else 1.5e-2), err


# ---------------------------------------------------------------------------------------------------------
# whole models
# ---------------------------------------------------------------------------------------------------------

LENGTHS = {"A": [5, 70, 1, 41, 150, 23], "B": [300, 7, 66, 131, 2, 200], "C": [260, 65, 1, 129], "D": [210, 33, 64, 1, 90]}


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    base = tmp_path_factory.mktemp("tifapel")
    return {(n, d): make_folder(base, n, d) for n in ALL for d in ("float32", "bfloat16")}


def _engine(folder, dtype, max_tokens=4096, **kw):
    from llmoxide_b200.engine.engine import Engine, LoadOptions

    return Engine.load(folder, LoadOptions(dtype=dtype, max_tokens=max_tokens, max_batch=8, **kw))


def _requests(name):
    toks = prompts(ALL[name]["vocab"], LENGTHS[name], seed=21)
    return {f"r{i}": t for i, t in enumerate(toks)}


def _expected(folder, reqs):
    cfg, w = plain.read_model(folder)
    return {rid: plain.forward(cfg, w, toks).numpy() for rid, toks in reqs.items()}


def _compare(got, want, dtype, what):
    """float32: every logit of every position within rounding (largest difference against the largest logit).
    bfloat16: a position's error is the root mean square over the vocabulary of the difference (its mean taken
    off) against that of the logits; a token whose best experts nearly tie may choose another one than the plain
    implementation does, so a few positions may lie outside the tolerance."""
    worst, n, over = 0.0, 0, 0
    for rid in want:
        assert got[rid].shape == want[rid].shape, (what, rid)
        if dtype == "float32":
            e = np.abs(got[rid] - want[rid]).max(axis=1) / np.abs(want[rid]).max()
        else:
            d = got[rid] - want[rid]
            w = want[rid] - want[rid].mean(axis=1, keepdims=True)
            e = (d - d.mean(axis=1, keepdims=True)).std(axis=1) / np.sqrt((w * w).mean())
        worst = max(worst, float(e.max()))
        n += len(e)
        over += int((e > (F32_TOL if dtype == "float32" else BF16_TOL)).sum())
    if dtype == "float32":
        assert over == 0, f"{what}: {over} of {n} positions differ from the plain implementation, worst {worst:.3e}"
    else:
        assert over <= max(2, 0.1 * n) and worst < 0.3, f"{what}: {over} of {n} positions beyond {BF16_TOL}, worst {worst:.3e}"
    return worst


def _rms_err(got, want):
    d = got - want
    w = want - want.mean(axis=1, keepdims=True)
    return (d - d.mean(axis=1, keepdims=True)).std(axis=1) / np.sqrt((w * w).mean())


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
def test_every_cutting_matches_the_plain_implementation(folders, tmp_path, name, dtype):
    folder = folders[(name, dtype)]
    reqs = _requests(name)
    want = _expected(folder, reqs)
    vocab = ALL[name]["vocab"]
    eng = _engine(folder, dtype)
    results = {}
    # the same engine runs every trace: slots, pages and state rows are freed and used again from trace to trace
    for what, steps in (("whole", ru.trace_whole(reqs)),
                        ("last 48 one by one", ru.trace_tail_decode(reqs, 48)),
                        ("all but the first token one by one", ru.trace_tail_decode(reqs, 10 ** 6)),
                        ("unequal batches", ru.trace_batches(reqs, 4)),
                        ("unequal batches of 3, short prompts", ru.trace_batches(reqs, 3, 0.2)),
                        ("portions of 2", ru.trace_chunks({k: v for k, v in reqs.items() if len(v) <= 70}, 2, 3, tail=3)),
                        ("portions of 5", ru.trace_chunks(reqs, 5, 6, tail=4)),
                        ("portions of 48", ru.trace_chunks(reqs, 48, 3)),
                        ("portions of 64", ru.trace_chunks(reqs, 64, 4)),
                        ("portions of 100 beside single tokens", ru.trace_chunks(reqs, 100, 6, tail=40, mixed=True))):
        out = tmp_path / what.replace(" ", "_").replace(",", "")
        ru.run_in_process(eng, steps, out)
        got = ru.collect(steps, out, vocab)
        sub = {rid: want[rid] for rid in got}
        worst = _compare(got, sub, dtype, f"{name}/{dtype}/{what}")
        print(f"{name}/{dtype}/{what}: worst rel err {worst:.2e}")
        results[what] = got
    if dtype == "float32":      # how a prompt is cut changes the products' rows per launch, nothing else
        for what, got in results.items():
            for rid in got:
                assert ru.rel_err(got[rid], results["whole"][rid]) < 4e-6, (what, rid)
    else:
        # bfloat16, cutting against cutting: most tokens whose experts nearly tie choose alike under every cutting
        # (a prompt step and a decode step round differently, so a few do not); a fault of the cache, the state
        # or the batch would move every later position
        for what, got in results.items():
            e = np.concatenate([_rms_err(got[rid], results["whole"][rid]) for rid in got])
            assert (e > BF16_TOL).sum() <= max(2, 0.05 * len(e)) and np.median(e) < 1.5e-2, \
                (what, int((e > BF16_TOL).sum()), float(np.median(e)), float(e.max()))
    eng.check_status()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_replay_as_a_user_runs_it(folders, tmp_path, dtype):
    """``bin/trace_run`` as a subprocess on a Tifapel folder: unequal batches whose requests end at different steps,
    with ``--max-tokens`` the bare sum of the live requests' tokens (the pages' padding is the runner's business)."""
    folder = folders[("A", dtype)]
    reqs = _requests("A")
    steps = ru.trace_batches(reqs, 3, 0.6)
    ru.run_trace_run(folder, dtype, steps, tmp_path / "out", max_tokens=sum(len(t) for t in reqs.values()))
    got = ru.collect(steps, tmp_path / "out", ALL["A"]["vocab"])
    _compare(got, _expected(folder, reqs), dtype, f"trace_run/{dtype}")


def test_a_slot_used_again_starts_from_an_empty_state(folders):
    """One slot: a long request, then a short one in the same slot; the second must not see the first's
    recurrent state, keys or kept first tokens."""
    folder = folders[("A", "float32")]
    eng = _engine(folder, "float32", max_tokens=512)
    cfg, w = plain.read_model(folder)
    long_req, short_req = prompts(ALL["A"]["vocab"], [200, 30], seed=5)
    for toks in (long_req, short_req, long_req[:90]):
        slot = eng.acquire()
        assert slot == 0
        got = eng.step([(slot, toks)], [list(range(len(toks)))]).cpu().numpy()
        eng.release(slot)
        assert ru.rel_err(got, plain.forward(cfg, w, toks).numpy()) < F32_TOL
    eng.cache.alloc.check_consistent()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_past_every_window(folders, dtype):
    """A short prompt and 330 single-token steps: the window of every layer, the kept first tokens and several
    page borders pass under decoded tokens; decode steps replay a CUDA graph."""
    folder = folders[("B", dtype)]
    eng = _engine(folder, dtype, max_tokens=1024)
    cfg, w = plain.read_model(folder)
    toks = prompts(ALL["B"]["vocab"], [340], seed=9)[0]
    want = plain.forward(cfg, w, toks).numpy()
    slot = eng.acquire()
    rows = [eng.step([(slot, toks[:10])], [list(range(10))]).cpu().numpy()]
    for t in toks[10:]:
        rows.append(eng.step([(slot, [t])], [[0]]).cpu().numpy())
    eng.release(slot)
    _compare({"r": np.concatenate(rows)}, {"r": want}, dtype, f"long decoding/{dtype}")
    eng.check_status()


@pytest.mark.parametrize("name, dtype", [("A", "float32"), ("C", "float32"), ("C", "bfloat16")])
def test_greedy_generation_through_the_session(folders, name, dtype):
    from llmoxide_b200 import LoadOptions, Request, Sampling, Session

    folder = folders[(name, dtype)]
    cfg, w = plain.read_model(folder)
    session = Session.load(folder, LoadOptions(dtype=dtype, max_tokens=2048, max_batch=4))
    reqs = prompts(ALL[name]["vocab"], [9, 1, 140, 40], seed=3)
    outs = session.generate([Request(p, 24, Sampling.greedy(), stop_ids=()) for p in reqs])
    for p, o in zip(reqs, outs):
        assert len(o.tokens) == 24
        ids = list(p)
        for tok in o.tokens:
            logits = plain.forward(cfg, w, ids)[-1].numpy()
            if dtype == "float32":
                assert tok == plain.argmax(logits), (name, p[:4], o.tokens)
            else:       # bfloat16 may differ only where the plain logits nearly tie
                assert logits.max() - logits[tok] <= 3e-2 * np.abs(logits).max(), (name, p[:4], o.tokens)
            ids.append(tok)
    info = session.info()
    assert info["architecture"] == "Tifapel" and info["n_layers"] == len(ALL[name]["layers"])


def test_random_weights_on_the_device_equal_the_folder(folders):
    """``Session.random`` makes the same model as the folder written from the same seed."""
    from llmoxide_b200 import Engine, LoadOptions, read_config

    folder = folders[("A", "float32")]
    toks = prompts(ALL["A"]["vocab"], [50], seed=1)[0]
    opts = dict(dtype="float32", max_tokens=256, max_batch=2)
    a = Engine.load(folder, LoadOptions(**opts))
    b = Engine.random(read_config(dict(copy.deepcopy(ALL["A"]), torch_dtype="float32")), 4321, LoadOptions(**opts))
    la = a.step([(a.acquire(), toks)], [[49]])
    lb = b.step([(b.acquire(), toks)], [[49]])
    assert torch.equal(la, lb)


# ---------------------------------------------------------------------------------------------------------
# the tiled bfloat16 kernels under a window that keeps its first keys
# ---------------------------------------------------------------------------------------------------------

def _paged_case(lens, G, D, seed):
    """A cache of random keys and values for sequences of the given lengths, pages dealt out in any order."""
    from llmoxide_b200 import kernels

    g = torch.Generator().manual_seed(seed)
    page = kernels.PAGE
    per = [(n + page - 1) // page for n in lens]
    order = torch.randperm(sum(per) + 2, generator=g).tolist()
    width = max(per)
    table = torch.full((len(lens), width), -1, dtype=torch.int32)
    kc = torch.randn((sum(per) + 2, G, page, D), generator=g) * 0.3
    vc = torch.randn((sum(per) + 2, G, page, D), generator=g)
    at = 0
    for b, n in enumerate(per):
        table[b, :n] = torch.tensor(order[at : at + n], dtype=torch.int32)
        at += n
    return table, kc.to(torch.bfloat16), vc.to(torch.bfloat16)


@pytest.mark.parametrize("D, H, G", [(64, 8, 1), (128, 4, 2), (48, 3, 3)])
@pytest.mark.parametrize("window, keep", [(40, 3), (130, 70), (20, 33), (64, 0), (0, 0)])
def test_decode_attention_with_kept_first_keys_equals_the_general_kernel(D, H, G, window, keep):
    """One token per sequence at lengths around the window's and the pages' edges; the key just outside the
    window (or the last kept one, or the first that is not kept) is made to stand out, so that a mask that is
    one key off changes the result beyond any tolerance.  Every split of the keys gives the same answer."""
    from llmoxide_b200 import kernels

    lens = [1, 2, keep + 1, window + 1, window + 2, window + keep + 3, 64, 65, 200, 399, 129, 257]
    lens = [n for n in lens if n >= 1]
    table, kc, vc = _paged_case(lens, G, D, seed=D + window)
    B = len(lens)
    q = (torch.randn(B, H, D, generator=torch.Generator().manual_seed(1)) * 0.3).to(torch.bfloat16)
    page = kernels.PAGE
    for b, n in enumerate(lens):
        p = n - 1
        spots = [p - window, p - window + 1, keep - 1, keep] if window else [0, p]
        j = spots[b % len(spots)]
        if 0 <= j <= p:
            for g in range(G):
                kc[table[b, j // page], g, j % page] = (q[b, g * (H // G)].float() * 6.0).to(torch.bfloat16)
    past = torch.tensor([n - 1 for n in lens], dtype=torch.int32, device=DEV)
    seq = torch.arange(B, dtype=torch.int32, device=DEV)
    qd, kd, vd, td = q.view(B, H * D).to(DEV), kc.to(DEV), vc.to(DEV), table.to(DEV)
    want = torch.empty((B, H * D), dtype=torch.bfloat16, device=DEV)
    kernels.attention_paged(qd, want, kd, vd, td, seq, past, H, G, D, window or None, 0.7, keep_first=keep)
    for n_chunks in (0, 1, 3, 8, 11):
        got = torch.empty_like(want)
        kernels.attention_decode(qd, got, kd, vd, td, past, H, G, D, window or None, 0.7, n_chunks=n_chunks,
                                 keep_first=keep)
        assert _rel(got.float().cpu().numpy(), want.float().cpu().numpy()) < 1.5e-2, (n_chunks,)
    kernels.check_status()


@pytest.mark.parametrize("D, H, G", [(64, 8, 1), (128, 4, 2)])
@pytest.mark.parametrize("window, keep", [(40, 3), (130, 70), (20, 33), (64, 0)])
def test_prompt_attention_with_kept_first_keys_equals_the_general_kernel(D, H, G, window, keep):
    """Whole prompts and later portions (129 and 2 tokens after a cached prefix) in one launch."""
    from llmoxide_b200 import kernels

    lens = [1, 70, 200, 399, 257, 66]
    new = [1, 70, 200, 129, 2, 65]              # the last `new` tokens of each are this step's
    table, kc, vc = _paged_case(lens, G, D, seed=3 * D + window)
    T = sum(new)
    q = (torch.randn(T, H, D, generator=torch.Generator().manual_seed(2)) * 0.3).to(torch.bfloat16)
    start = np.concatenate([[0], np.cumsum(new)]).astype(np.int32)
    tok_seq = np.concatenate([[b] * n for b, n in enumerate(new)]).astype(np.int32)
    tok_pos = np.concatenate([np.arange(L - n, L) for L, n in zip(lens, new)]).astype(np.int32)
    page = kernels.PAGE
    for b, L in enumerate(lens):                # a key that stands out for the sequence's last query
        p = L - 1
        j = [p - window, p - window + 1, keep - 1, keep][b % 4]
        if 0 <= j <= p:
            for g in range(G):
                kc[table[b, j // page], g, j % page] = (q[start[b + 1] - 1, g * (H // G)].float() * 6.0).to(torch.bfloat16)
    qd, kd, vd, td = q.view(T, H * D).to(DEV), kc.to(DEV), vc.to(DEV), table.to(DEV)
    want = torch.empty((T, H * D), dtype=torch.bfloat16, device=DEV)
    kernels.attention_paged(qd, want, kd, vd, td, torch.tensor(tok_seq, device=DEV), torch.tensor(tok_pos, device=DEV),
                            H, G, D, window, 0.7, keep_first=keep)
    got = torch.empty_like(want)
    kernels.attention_prefill(qd, got, kd, vd, td, torch.tensor(start, device=DEV),
                              torch.tensor([L - n for L, n in zip(lens, new)], dtype=torch.int32, device=DEV),
                              len(lens), max(new), H, G, D, window, 0.7, keep_first=keep)
    assert _rel(got.float().cpu().numpy(), want.float().cpu().numpy()) < 1.5e-2
    if D == 128:            # the tcgen05 kernel of that head size
        got = torch.empty_like(want)
        kernels.attention_prefill_tc(qd, got, kd, vd, td, torch.tensor(start, device=DEV),
                                     torch.tensor([L - n for L, n in zip(lens, new)], dtype=torch.int32, device=DEV),
                                     len(lens), max(new), H, G, D, window, 0.7, keep_first=keep)
        assert _rel(got.float().cpu().numpy(), want.float().cpu().numpy()) < 1.5e-2
        kernels.check_status()
