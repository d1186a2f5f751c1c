"""GPU: the Voserax decoder's mechanisms one by one against the plain implementation (tests/plain_voserax.py),
then whole models under every way of cutting the same requests into steps, and greedy generation through the
package's own entry point."""

import copy
from types import SimpleNamespace

import numpy as np
import pytest
import torch

import plain_voserax as plain
import replay_util as ru
from tiny_configs import prompts
from voserax_configs import ALL, make_folder

pytestmark = pytest.mark.gpu

DEV = "cuda:0"
F32_TOL, BF16_TOL = 2e-5, 3e-2


def _rel(got, want):
    want = np.asarray(want, dtype=np.float64)
    return float(np.abs(np.asarray(got, dtype=np.float64) - want).max() / max(np.abs(want).max(), 1e-30))


def _bf16_exact(t):
    return t.to(torch.bfloat16).to(torch.float64)


def _i32(x):
    return torch.tensor(x, dtype=torch.int32, device=DEV)


# ---------------------------------------------------------------------------------------------------------
# copies of the residual stream
# ---------------------------------------------------------------------------------------------------------

@pytest.mark.parametrize("S, d, n_split", [(1, 40, 1), (2, 96, 3), (4, 200, 5), (5, 1000, 2), (8, 64, 1), (3, 50, 6), (2, 2050, 1), (4, 2048, 3)])
@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
def test_stream_update_and_norm_against_the_plain_sublayer(S, d, n_split, out_dtype):
    from llmoxide_b200 import kernels

    torch.manual_seed(S * 7 + d)
    T, eps = 37, 1e-5
    X = torch.randn(S, T, d, dtype=torch.float64).float().double()
    parts = torch.randn(n_split, T, d, dtype=torch.float64).float().double()
    W = {"a.in": torch.randn(S, dtype=torch.float64).float().double(), "a.out": torch.randn(S, dtype=torch.float64).float().double(),
         "a.mix": torch.randn(S, S, dtype=torch.float64).float().double(), "b.in": torch.randn(S, dtype=torch.float64).float().double()}
    gain = torch.randn(d, dtype=torch.float64).float().double()
    mult = 0.7
    # the update that sublayer a owes (its result: the sum of the partials), then the read of sublayer b
    new = plain.hyper_sublayer(X, W, "a.", mult, gain, eps, lambda h: parts.sum(0))
    want_x = plain.rms_norm(torch.einsum("s,std->td", W["b.in"], new), gain, eps)
    h = X.float().to(DEV).contiguous()
    out = torch.empty((T, d), dtype=out_dtype, device=DEV)
    kernels.stream_mix_norm(h, parts.float().to(DEV), W["a.mix"].float().to(DEV).contiguous(),
                            (W["a.out"] * mult).float().to(DEV), W["b.in"].float().to(DEV), gain.float().to(DEV), eps, out)
    assert _rel(h.cpu().numpy(), new.numpy()) < 2e-6
    assert _rel(out.float().cpu().numpy(), want_x.numpy()) < (3e-6 if out_dtype == torch.float32 else 6e-3)
    # some rows only, nothing stored, the plain sum as the read (what the model's last norm does)
    h2 = X.float().to(DEV).contiguous()
    rows = _i32([T - 1, 0, 5])
    out2 = torch.empty((3, d), dtype=torch.float32, device=DEV)
    kernels.stream_mix_norm(h2, parts.float().to(DEV), W["a.mix"].float().to(DEV).contiguous(),
                            (W["a.out"] * mult).float().to(DEV), None, gain.float().to(DEV), eps, out2, rows=rows, write_h=False)
    assert torch.equal(h2.cpu(), X.float())
    assert _rel(out2.cpu().numpy(), plain.rms_norm(new.sum(0), gain, eps)[[T - 1, 0, 5]].numpy()) < 3e-6
    # no update owed: only the read
    out3 = torch.empty((T, d), dtype=torch.float32, device=DEV)
    kernels.stream_mix_norm(h2, None, None, None, W["b.in"].float().to(DEV), gain.float().to(DEV), eps, out3)
    assert _rel(out3.cpu().numpy(), plain.rms_norm(torch.einsum("s,std->td", W["b.in"], X), gain, eps).numpy()) < 3e-6


def test_embedding_with_learned_positions_fills_every_copy():
    from llmoxide_b200 import kernels

    torch.manual_seed(2)
    for dtype in (torch.float32, torch.bfloat16):
        table, pos = torch.randn(50, 24).to(dtype), torch.randn(70, 24).to(dtype)
        tokens, where = [3, 49, 0, 7], [0, 69, 5, 5]
        h = torch.empty((3, 4, 24), dtype=torch.float32, device=DEV)
        kernels.embed_positions(table.to(DEV), pos.to(DEV), _i32(tokens), _i32(where), h, 1.0)
        want = table.float()[tokens] + pos.float()[where]
        assert all(torch.equal(h[s].cpu(), want) for s in range(3))


# ---------------------------------------------------------------------------------------------------------
# the short convolution with rotation, value mixing and the cache write
# ---------------------------------------------------------------------------------------------------------

def _conv_case(cuts, H, G, D, Dv, taps, n_rot, mode, dtype, n_split=1, seed=0):
    """Two sequences of unequal lengths through ``conv_rope_cache`` + ``conv_state_update``, cut into steps as
    ``cuts`` says (tokens per step and sequence); returns q, k, v of every position as the kernels left them (k and
    v read back from the cache) beside what the plain functions give."""
    from llmoxide_b200 import kernels

    g = torch.Generator().manual_seed(seed)
    lens = [sum(c[b] for c in cuts) for b in range(2)]
    C = (H + G) * D + G * Dv
    page = kernels.PAGE
    u = [_bf16_exact(torch.randn(n, C, generator=g)) for n in lens]
    w = _bf16_exact(torch.randn(C, max(taps, 1), generator=g) * 0.5)
    first = [_bf16_exact(torch.randn(n, G * Dv, generator=g)) for n in lens]
    lam = 0.3
    cos = sin = None
    if n_rot:
        freq, amp = plain.scaled_frequencies(n_rot, 100.0, dict(factor=2.0, original=16, fast=4.0, slow=1.0))
        ang = torch.arange(max(lens), dtype=torch.float64)[:, None] * freq[None]
        cos, sin = (torch.cos(ang) * amp).float().to(DEV), (torch.sin(ang) * amp).float().to(DEV)
    per = [(n + page - 1) // page for n in lens]
    table = torch.full((2, max(per)), 0, dtype=torch.int32)
    order = torch.randperm(sum(per) + 1, generator=g).tolist()
    table[0, : per[0]] = torch.tensor(order[: per[0]], dtype=torch.int32)
    table[1, : per[1]] = torch.tensor(order[per[0] : per[0] + per[1]], dtype=torch.int32)
    kc = torch.zeros((sum(per) + 1, G, page, D), dtype=dtype, device=DEV)
    vc = torch.zeros((sum(per) + 1, G, page, Dv), dtype=dtype, device=DEV)
    state = torch.full((5, max(taps - 1, 1), C), 7.0, dtype=torch.float32, device=DEV)     # slots 3 and 1 are the sequences'
    slots = [3, 1]
    state[slots] = 0.0
    got_q = [torch.zeros(n, H * D) for n in lens]
    past = [0, 0]
    for c in cuts:
        live = [b for b in range(2) if c[b] > 0]
        rows = torch.cat([u[b][past[b] : past[b] + c[b]] for b in live])
        T = rows.shape[0]
        token_seq = [i for i, b in enumerate(live) for _ in range(c[b])]
        token_pos = [past[b] + j for b in live for j in range(c[b])]
        starts = np.cumsum([0] + [c[b] for b in live]).tolist()
        ctx = SimpleNamespace(token_seq=_i32(token_seq), token_pos=_i32(token_pos), seq_start=_i32(starts),
                              seq_past=_i32([past[b] for b in live]), seq_slot=_i32([slots[b] for b in live]), n_seqs=len(live))
        if n_split > 1:       # float32 partials that add up to the rows
            a = _bf16_exact(torch.randn(n_split - 1, T, C, generator=g))
            proj = torch.cat([a, (rows - a.sum(0))[None]]).float().to(DEV).contiguous()
        else:
            proj = rows.to(dtype).to(DEV).contiguous()
        q = torch.empty((T, H * D), dtype=dtype, device=DEV)
        vf = None
        if mode == 1:
            vf = torch.zeros((T, G * Dv), dtype=torch.float32, device=DEV)
        elif mode == 2:
            vf = torch.cat([first[b][past[b] : past[b] + c[b]] for b in live]).float().to(DEV).contiguous()
        single = all(c[b] == 1 for b in live)       # a step of single tokens: the first kernel moves the state on itself
        kernels.conv_rope_cache(proj, state, w.float().t().contiguous().to(DEV) if taps else None, taps, q, kc, vc,
                                table[live].to(DEV).contiguous(), ctx, cos, sin, n_rot, vf,
                                torch.tensor([lam], dtype=torch.float32, device=DEV) if mode == 2 else None, mode, H, G, D, Dv,
                                inline_state=single)
        if not single:
            kernels.conv_state_update(proj, state, taps, ctx)
        at = 0
        for b in live:
            got_q[b][past[b] : past[b] + c[b]] = q[at : at + c[b]].float().cpu()
            if mode == 1:      # the values left for later layers are the convolved ones
                first[b][past[b] : past[b] + c[b]] = vf[at : at + c[b]].double().cpu()
            at += c[b]
            past[b] += c[b]
    assert torch.equal(state[[0, 2, 4]].cpu(), torch.full((3, max(taps - 1, 1), C), 7.0)), "another slot's state was written"
    out = []
    for b in range(2):
        n = lens[b]
        y = plain.short_convolution(u[b], w) if taps else u[b]
        qw, kw, vw = y[:, : H * D].view(n, H, D), y[:, H * D : (H + G) * D].view(n, G, D), y[:, (H + G) * D :].view(n, G, Dv)
        if n_rot:
            sc = dict(factor=2.0, original=16, fast=4.0, slow=1.0)
            qw, kw = (plain.rotate_half(t, torch.arange(n), n_rot, 100.0, sc) for t in (qw, kw))
        if mode == 2:
            vw = (1 - lam) * vw + lam * first[b].view(n, G, Dv)
        pages = table[b].long()
        kg = torch.stack([kc[pages[p // page], :, p % page] for p in range(n)]).float().cpu()
        vg = torch.stack([vc[pages[p // page], :, p % page] for p in range(n)]).float().cpu()
        out.append((got_q[b].view(n, H, D), kg, vg, qw, kw, vw, first[b].view(n, G, Dv), y))
        if taps > 1:           # the state: the last taps-1 projected rows, zeros before the start
            want_state = torch.cat([torch.zeros(taps - 1, C, dtype=torch.float64), u[b]])[-(taps - 1):]
            assert torch.equal(state[slots[b]].double().cpu(), want_state)
    return out


CUTTINGS = {
    "whole": [(70, 131)],
    "token by token": [(1, 1)] * 9 + [(0, 1)] * 3,
    "portions of two, then single tokens": [(2, 2)] * 4 + [(1, 1)] * 3,
    "portions that straddle a page": [(60, 3), (7, 61), (1, 1), (5, 0), (0, 70)],
}


@pytest.mark.parametrize("cutting", list(CUTTINGS))
@pytest.mark.parametrize("H, G, D, Dv, taps, n_rot, mode, n_split", [
    (4, 1, 32, 16, 4, 16, 0, 1), (3, 3, 16, 48, 2, 16, 1, 1), (2, 2, 40, 24, 3, 0, 2, 3), (2, 1, 128, 128, 5, 64, 2, 1),
    (1, 1, 8, 8, 0, 8, 2, 1), (6, 2, 16, 16, 16, 4, 1, 2)])
def test_convolution_rotation_and_value_mixing_under_every_cutting(cutting, H, G, D, Dv, taps, n_rot, mode, n_split):
    cuts = CUTTINGS[cutting]
    ref = _conv_case([tuple(sum(c[b] for c in cuts) for b in range(2))], H, G, D, Dv, taps, n_rot, mode, torch.float32, 1, seed=5)
    for dtype in (torch.float32, torch.bfloat16):
        if n_split > 1 and dtype == torch.bfloat16:
            continue
        res = _conv_case(cuts, H, G, D, Dv, taps, n_rot, mode, dtype, n_split, seed=5)
        tol = 3e-6 if dtype == torch.float32 else 8e-3
        for b, (q, k, v, qw, kw, vw, first, _) in enumerate(res):
            assert _rel(q.numpy(), qw.numpy()) < tol and _rel(k.numpy(), kw.numpy()) < tol and _rel(v.numpy(), vw.numpy()) < tol, \
                (cutting, dtype, b)
            if mode == 1:
                assert _rel(first.numpy(), res[b][7][:, (H + G) * D :].reshape(first.shape).numpy()) < 3e-6
            if dtype == torch.float32 and n_split == 1:       # a cutting changes nothing at all
                assert torch.equal(q, ref[b][0]) and torch.equal(k, ref[b][1]) and torch.equal(v, ref[b][2]), (cutting, b)


# ---------------------------------------------------------------------------------------------------------
# attention with a sink under a window
# ---------------------------------------------------------------------------------------------------------

@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("D, Dv, H, G, window", [(16, 48, 6, 3, 64), (32, 16, 4, 2, 20), (64, 64, 8, 1, 130),
                                                 (48, 48, 3, 3, 0), (40, 24, 2, 1, 1), (80, 48, 5, 1, 37)])
def test_one_key_stands_out_at_every_edge_of_the_window_with_a_sink(D, Dv, H, G, window, dtype):
    """Queries at several positions; for each, one key is made to carry nearly all the weight if it is visible: the
    last key inside the window, the first outside it, the first token, a key at a page border, a far key among
    hundreds.  The values say which key was seen, and the sink takes its share where no key stands out."""
    from llmoxide_b200 import kernels

    torch.manual_seed(D + Dv)
    n_pos, page = 400, kernels.PAGE
    n_pages = (n_pos + page - 1) // page
    table = torch.randperm(n_pages + 3)[:n_pages].to(torch.int32)
    k = _bf16_exact(torch.randn(n_pos, G, D) * 0.1)
    v = _bf16_exact(torch.randn(n_pos, G, Dv))
    queries = []
    for p in (0, 1, 2, window, window + 1, 199, 255, 256, 399):
        if p >= n_pos or p < 0:
            continue
        targets = {p, max(0, p - 1), 0, (p // page) * page, max(0, (p // page) * page - 1), p // 2}
        if window:
            targets |= {max(0, p - window + 1), max(0, p - window)}
        queries += [(p, j) for j in sorted(targets) if j <= p]
    q = _bf16_exact(torch.randn(len(queries), H, D) * 0.1)
    for i in range(len(queries)):
        for g in range(G):
            k_dir = q[i, g * (H // G)] / q[i, g * (H // G)].norm()
            q[i, g * (H // G)] = _bf16_exact(k_dir * 6.0)
    outs, wants = [], []
    for i, (p, j) in enumerate(queries):
        kk = k.clone()
        for g in range(G):
            kk[j, g] = _bf16_exact(q[i, g * (H // G)] / 6.0 * 8.0)
        kc = torch.zeros((n_pages + 3, G, page, D), dtype=torch.float64)
        vc = torch.zeros((n_pages + 3, G, page, Dv), dtype=torch.float64)
        for pos in range(p + 1):
            kc[table[pos // page], :, pos % page] = kk[pos]
            vc[table[pos // page], :, pos % page] = v[pos]
        out = torch.empty((1, H * Dv), dtype=dtype, device=DEV)
        kernels.attention_paged(q[i].reshape(1, H * D).to(dtype).to(DEV), out, kc.to(dtype).to(DEV), vc.to(dtype).to(DEV),
                                table.view(1, -1).to(DEV), torch.zeros(1, dtype=torch.int32, device=DEV),
                                torch.tensor([p], dtype=torch.int32, device=DEV), H, G, D, window or None, 0.9,
                                v_head_dim=Dv, sink=1.0)
        # the plain function on the whole sequence up to p; its last row is this query (the others use their own q)
        qq = torch.zeros(p + 1, H, D, dtype=torch.float64)
        qq[p] = q[i]
        want = plain.sink_softmax_attention(qq, kk[: p + 1], v[: p + 1], 0.9, window or None)[p].view(H, Dv)
        outs.append(out.float().cpu().view(H, Dv))
        wants.append(want)
    err = max(_rel(o.numpy(), w.numpy()) for o, w in zip(outs, wants))
    assert err < (1e-5 if dtype == torch.float32 else 1.5e-2), err
    # the sink is there: with one key of score 0 the output is half the value
    out = torch.empty((1, H * Dv), dtype=torch.float32, device=DEV)
    kc = torch.zeros((1, G, page, D), dtype=torch.float32, device=DEV)
    vc = torch.ones((1, G, page, Dv), dtype=torch.float32, device=DEV)
    kernels.attention_paged(torch.ones((1, H * D), device=DEV), out, kc, vc, _i32([[0]]), _i32([0]), _i32([0]), H, G, D,
                            window or None, 0.9, v_head_dim=Dv, sink=1.0)
    assert torch.allclose(out.cpu(), torch.full((1, H * Dv), 0.5))


def _paged_case(lens, G, D, seed):
    """A cache of random keys and values for sequences of the given lengths, pages dealt out in any order."""
    from llmoxide_b200 import kernels

    g = torch.Generator().manual_seed(seed)
    page = kernels.PAGE
    per = [(n + page - 1) // page for n in lens]
    order = torch.randperm(sum(per) + 2, generator=g).tolist()
    table = torch.full((len(lens), max(per)), -1, dtype=torch.int32)
    kc = torch.randn((sum(per) + 2, G, page, D), generator=g) * 0.3
    vc = torch.randn((sum(per) + 2, G, page, D), generator=g)
    at = 0
    for b, n in enumerate(per):
        table[b, :n] = torch.tensor(order[at : at + n], dtype=torch.int32)
        at += n
    return table, kc.to(torch.bfloat16), vc.to(torch.bfloat16)


@pytest.mark.parametrize("D, H, G", [(64, 8, 1), (128, 4, 2), (48, 3, 3), (96, 6, 2)])
@pytest.mark.parametrize("window", [37, 130, 1, 64, 0])
def test_decode_attention_with_a_sink_equals_the_general_kernel(D, H, G, window):
    """One token per sequence at lengths around the window's and the pages' edges; the key just outside or just
    inside the window is made to stand out, so that a mask that is one key off changes the result beyond any
    tolerance; where no key stands out (short sequences, small scores) the sink holds a large share of the
    denominator.  Every split of the keys gives the same answer: the sink joins the merged denominator once."""
    from llmoxide_b200 import kernels

    lens = [n for n in [1, 2, 3, window + 1, window + 2, window + 3, 64, 65, 200, 399, 129, 257] if n >= 1]
    table, kc, vc = _paged_case(lens, G, D, seed=D + window)
    B = len(lens)
    q = (torch.randn(B, H, D, generator=torch.Generator().manual_seed(1)) * 0.3).to(torch.bfloat16)
    page = kernels.PAGE
    for b, n in enumerate(lens):
        p = n - 1
        spots = [p - window, p - window + 1, None] if window else [0, p, None]
        j = spots[b % 3]
        if j is not None and 0 <= j <= p:
            for g in range(G):
                kc[table[b, j // page], g, j % page] = (q[b, g * (H // G)].float() * 6.0).to(torch.bfloat16)
    past = torch.tensor([n - 1 for n in lens], dtype=torch.int32, device=DEV)
    seq = torch.arange(B, dtype=torch.int32, device=DEV)
    qd, kd, vd, td = q.view(B, H * D).to(DEV), kc.to(DEV), vc.to(DEV), table.to(DEV)
    want = torch.empty((B, H * D), dtype=torch.bfloat16, device=DEV)
    kernels.attention_paged(qd, want, kd, vd, td, seq, past, H, G, D, window or None, 0.7, sink=1.0)
    without = torch.empty_like(want)
    kernels.attention_paged(qd, without, kd, vd, td, seq, past, H, G, D, window or None, 0.7)
    assert _rel(without.float().cpu().numpy(), want.float().cpu().numpy()) > 0.1       # the sink shows
    for n_chunks in (0, 1, 3, 8, 11):
        got = torch.empty_like(want)
        kernels.attention_decode(qd, got, kd, vd, td, past, H, G, D, window or None, 0.7, n_chunks=n_chunks, sink=1.0)
        assert _rel(got.float().cpu().numpy(), want.float().cpu().numpy()) < 1.5e-2, (n_chunks,)
    kernels.check_status()


@pytest.mark.parametrize("D, H, G", [(64, 8, 1), (128, 4, 2)])
@pytest.mark.parametrize("window", [37, 130, 1, 64, 0])
def test_prompt_attention_with_a_sink_equals_the_general_kernel(D, H, G, window):
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
        j = [p - window, p - window + 1][b % 2] if window else [0, p][b % 2]
        if 0 <= j <= p:
            for g in range(G):
                kc[table[b, j // page], g, j % page] = (q[start[b + 1] - 1, g * (H // G)].float() * 6.0).to(torch.bfloat16)
    qd, kd, vd, td = q.view(T, H * D).to(DEV), kc.to(DEV), vc.to(DEV), table.to(DEV)
    want = torch.empty((T, H * D), dtype=torch.bfloat16, device=DEV)
    kernels.attention_paged(qd, want, kd, vd, td, torch.tensor(tok_seq, device=DEV), torch.tensor(tok_pos, device=DEV),
                            H, G, D, window or None, 0.7, sink=1.0)
    pasts = torch.tensor([L - n for L, n in zip(lens, new)], dtype=torch.int32, device=DEV)
    got = torch.empty_like(want)
    kernels.attention_prefill(qd, got, kd, vd, td, torch.tensor(start, device=DEV), pasts, len(lens), max(new), H, G, D,
                              window or None, 0.7, sink=1.0)
    assert _rel(got.float().cpu().numpy(), want.float().cpu().numpy()) < 1.5e-2
    if D == 128:            # the tcgen05 kernel of that head size
        got = torch.empty_like(want)
        kernels.attention_prefill_tc(qd, got, kd, vd, td, torch.tensor(start, device=DEV), pasts, len(lens), max(new), H, G,
                                     D, window or None, 0.7, sink=1.0)
        assert _rel(got.float().cpu().numpy(), want.float().cpu().numpy()) < 1.5e-2
        kernels.check_status()


# ---------------------------------------------------------------------------------------------------------
# feed-forwards
# ---------------------------------------------------------------------------------------------------------

@pytest.mark.parametrize("E, ident, top", [(8, 2, 2), (4, 3, 3), (5, 0, 1), (1, 4, 2), (30, 2, 6)])
def test_routing_with_a_correction_matches_the_plain_rule(E, ident, top):
    from llmoxide_b200 import kernels

    torch.manual_seed(E * 10 + top)
    T, n = 301, E + ident
    z = (torch.randn(T, n, dtype=torch.float64) * 2.0).float()
    W = {"m.router": torch.eye(n, dtype=torch.float64), "m.correction": (torch.randn(n, dtype=torch.float64) * 0.2).float().double()}
    want_ids, want_w, _ = plain.route(z.double(), W, "m.", dict(top=top))
    ids = torch.empty((T, top), dtype=torch.int32, device=DEV)
    w = torch.empty((T, top), dtype=torch.float32, device=DEV)
    kernels.moe_route(z.to(DEV), ids, w, top, 1, 1, 1, "softmax", False, 0.0, 1.0, bias=W["m.correction"].float().to(DEV))
    assert torch.equal(ids.cpu().long(), want_ids)
    assert _rel(w.cpu().numpy(), want_w.numpy()) < 1e-6


def test_a_row_of_nan_scores_is_reported_and_routed_to_experts_that_exist():
    """A token whose logits are NaN wins no comparison; the kernel reports it in its status word and hands out experts
    that exist, and the sort takes whatever ids it is given without leaving its arrays (both report, neither faults)."""
    from llmoxide_b200 import kernels
    from llmoxide_b200.errors import KernelError

    E, top, T = 7, 3, 5
    z = torch.randn(T, E)
    z[2] = float("nan")
    ids = torch.empty((T, top), dtype=torch.int32, device=DEV)
    w = torch.empty((T, top), dtype=torch.float32, device=DEV)
    kernels.moe_route(z.to(DEV), ids, w, top, 1, 1, 1, "softmax", False, 0.0, 1.0)
    got = ids.cpu()
    assert ((got >= 0) & (got < E)).all() and len(set(got[2].tolist())) == top
    with pytest.raises(KernelError, match="moe"):
        kernels.check_status()
    bad = got.clone()
    bad[1, 0] = 1 << 30
    perm = torch.empty(T * top, dtype=torch.int32, device=DEV)
    tiles = torch.empty((kernels.moe_max_tiles(T * top, E), 3), dtype=torch.int32, device=DEV)
    kernels.moe_sort(bad.to(DEV), E, perm, tiles)
    assert sorted(perm.cpu().tolist()) == list(range(T * top))
    with pytest.raises(KernelError, match="moe"):
        kernels.check_status()
    kernels.check_status()          # reported once, then clean


def _experts_part(d, F, E, ident, top, limit, shared, dtype, seed):
    from llmoxide_b200.config.spec import PartSpec, TensorSpec
    from llmoxide_b200.parts import Runtime
    from llmoxide_b200.parts.experts import RoutedExperts

    g = torch.Generator().manual_seed(seed)
    n = E + ident
    W = {"m.router": torch.randn(n, d, generator=g) * 0.3, "m.correction": torch.randn(n, generator=g) * 0.05}
    tensors = {"router": TensorSpec("m.router", (n, d)), "correction": TensorSpec("m.correction", (n,), "vector")}
    for e in range(E):
        for r, shape in (("gate", (F, d)), ("up", (F, d)), ("down", (d, F))):
            W[f"m.e{e}.{r}"] = torch.randn(*shape, generator=g) * 0.3
            tensors[f"{r}{e}"] = TensorSpec(f"m.e{e}.{r}", shape)
    params = dict(hidden_size=d, intermediate_size=F, n_experts=E, n_identity=ident, top=top, score="softmax", n_groups=1,
                  keep_groups=1, group_score_top=1, normalize=False, normalize_eps=0.0, scale=1.0, activation="clamped_swish",
                  act_slope=1.702, act_limit=limit, act_up_shift=1.0)
    mlp = dict(router=dict(experts=E, top=top, identity=ident), expert=dict(ff=F, limit=limit))
    if shared:
        Fs, lim = shared
        for r, shape in (("gate", (Fs, d)), ("up", (Fs, d)), ("down", (d, Fs)), ("sg", (1, d))):
            W[f"m.shared.{r}"] = torch.randn(*shape, generator=g) * 0.3
            tensors[f"shared_{r}"] = TensorSpec(f"m.shared.{r}", shape)
        params.update(shared_size=Fs, shared_limit=lim, shared_gate="sigmoid")
        mlp["shared"] = dict(ff=Fs, limit=lim)
    W = {k: _bf16_exact(v) for k, v in W.items()}
    rt = Runtime(dtype="float32" if dtype == torch.float32 else "bfloat16", device=torch.device(DEV), max_positions=64)
    part = RoutedExperts(PartSpec("routed_experts", params, tensors), {k: v.to(dtype).to(DEV) for k, v in W.items()}, rt)
    return part, W, mlp


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("d, F, E, ident, top, limit, shared", [(72, 40, 6, 2, 2, 1.0, (24, 0.8)), (64, 16, 3, 0, 3, 0.3, None),
                                                                (96, 64, 4, 3, 4, 7.0, (128, 0.5)), (40, 8, 1, 2, 1, 1.0, None)])
def test_clamped_experts_with_identity_and_shared_experts_against_the_plain_mixture(d, F, E, ident, top, limit, shared, dtype):
    part, W, mlp = _experts_part(d, F, E, ident, top, limit, shared, dtype, seed=d + E)
    torch.manual_seed(1)
    for T in (1, 3, 130, 700):
        x = _bf16_exact(torch.randn(T, d) * 2.0)
        y = part.forward(x.to(dtype).to(DEV), None)
        assert y.shape == (top + (1 if shared else 0), T, d) and y.dtype == torch.float32
        want = plain.mixture(x, W, "m.", mlp)
        err = np.abs(y.sum(0).cpu().numpy() - want.numpy()).max(axis=1) / np.abs(want.numpy()).max()
        if dtype == torch.float32:
            assert err.max() < 1e-5, (T, err.max())
        else:       # a token whose choice scores nearly tie may choose otherwise once x W_r is rounded differently
            assert (err > 1.5e-2).sum() <= max(1, 0.05 * T), (T, err.max())


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("activation", ["relu", ("clamped_swish", 1.702, 0.6, 1.0)])
def test_gated_feed_forward_with_other_activations(activation, dtype):
    from llmoxide_b200.config.spec import PartSpec, TensorSpec
    from llmoxide_b200.parts import Runtime
    from llmoxide_b200.parts.feed_forward import GatedMLP

    torch.manual_seed(9)
    d, F = 96, 80
    W = {"m.gate": _bf16_exact(torch.randn(F, d) * 0.2), "m.up": _bf16_exact(torch.randn(F, d) * 0.2),
         "m.down": _bf16_exact(torch.randn(d, F) * 0.2)}
    spec = PartSpec("gated_mlp", dict(hidden_size=d, intermediate_size=F, activation=activation),
                    dict(gate=TensorSpec("m.gate", (F, d)), up=TensorSpec("m.up", (F, d)), down=TensorSpec("m.down", (d, F))))
    rt = Runtime(dtype="float32" if dtype == torch.float32 else "bfloat16", device=torch.device(DEV), max_positions=64)
    part = GatedMLP(spec, {k: v.to(dtype).to(DEV) for k, v in W.items()}, rt)
    for T in (1, 5, 70, 300):
        x = _bf16_exact(torch.randn(T, d))
        y = part.forward(x.to(dtype).to(DEV), None)
        y = y.float().sum(0) if y.dim() == 3 else y.float()
        want = plain.relu_gated(x, W, "m.") if activation == "relu" else plain.clamped_expert(x, W, "m.", activation[2])
        assert _rel(y.cpu().numpy(), want.numpy()) < (1e-5 if dtype == torch.float32 else 1.2e-2), T


# ---------------------------------------------------------------------------------------------------------
# whole models
# ---------------------------------------------------------------------------------------------------------

LENGTHS = {"A": [5, 70, 1, 41, 150, 23], "B": [300, 7, 66, 131, 2, 200], "C": [260, 65, 1, 129], "D": [90, 3, 64, 1],
           "E": [210, 33, 64, 1, 90]}


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    base = tmp_path_factory.mktemp("voserax")
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


def _rms_err(got, want):
    d = got - want
    w = want - want.mean(axis=1, keepdims=True)
    return (d - d.mean(axis=1, keepdims=True)).std(axis=1) / np.sqrt((w * w).mean())


def _compare(got, want, dtype, what):
    """float32: every logit of every position within rounding (largest difference against the largest logit).
    bfloat16: a position's error is the root mean square over the vocabulary of the difference (its mean taken
    off) against that of the logits; a token whose choice scores nearly tie (with random weights the scores are
    close to one another and the small correction decides) may choose another expert than the plain implementation
    does, which moves that position's logits by as much as an expert's whole output, so a few positions may lie
    outside the tolerance; a fault of the cache, the state or the batch would move every later position."""
    worst, n, over = 0.0, 0, 0
    for rid in want:
        assert got[rid].shape == want[rid].shape, (what, rid)
        e = (np.abs(got[rid] - want[rid]).max(axis=1) / np.abs(want[rid]).max() if dtype == "float32"
             else _rms_err(got[rid], want[rid]))
        worst = max(worst, float(e.max()))
        n += len(e)
        over += int((e > (F32_TOL if dtype == "float32" else BF16_TOL)).sum())
    if dtype == "float32":
        assert over == 0, f"{what}: {over} of {n} positions differ from the plain implementation, worst {worst:.3e}"
    else:
        assert over <= max(2, 0.1 * n) and worst < 1.0, f"{what}: {over} of {n} positions beyond {BF16_TOL}, worst {worst:.3e}"
    return worst


def test_layer_by_layer_against_the_plain_streams(folders):
    """The sum of the streams after every layer, as the step's named intermediates report it."""
    for name in ("A", "E"):
        folder = folders[(name, "float32")]
        cfg, w = plain.read_model(folder)
        toks = prompts(ALL[name]["vocab"], [75], seed=4)[0]
        layers = []
        plain.forward(cfg, w, toks, layers)
        eng = _engine(folder, "float32", max_tokens=512)
        got = {}
        eng.step([(eng.acquire(), toks)], [[0]], probe=lambda n, t: got.__setitem__(n, t.detach().float().cpu().numpy()))
        for i, want in enumerate(layers):
            assert _rel(got[f"l_out-{i}"], want.numpy()) < 5e-6, (name, i)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(ALL))
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
        worst = _compare(got, {rid: want[rid] for rid in got}, dtype, f"{name}/{dtype}/{what}")
        print(f"{name}/{dtype}/{what}: worst rel err {worst:.2e}")
        results[what] = got
    if dtype == "float32":      # how a prompt is cut changes the products' rows per launch, nothing else
        for what, got in results.items():
            for rid in got:
                assert ru.rel_err(got[rid], results["whole"][rid]) < 4e-6, (what, rid)
    else:
        for what, got in results.items():
            e = np.concatenate([_rms_err(got[rid], results["whole"][rid]) for rid in got])
            assert (e > BF16_TOL).sum() <= max(2, 0.05 * len(e)) and np.median(e) < 1.5e-2, \
                (what, int((e > BF16_TOL).sum()), float(np.median(e)), float(e.max()))
    eng.check_status()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_replay_as_a_user_runs_it(folders, tmp_path, dtype):
    """``bin/trace_run`` as a subprocess on a Voserax folder: unequal batches whose requests end at different steps,
    with ``--max-tokens`` the bare sum of the live requests' tokens."""
    folder = folders[("A", dtype)]
    reqs = _requests("A")
    steps = ru.trace_batches(reqs, 3, 0.6)
    ru.run_trace_run(folder, dtype, steps, tmp_path / "out", max_tokens=sum(len(t) for t in reqs.values()))
    got = ru.collect(steps, tmp_path / "out", ALL["A"]["vocab"])
    _compare(got, _expected(folder, reqs), dtype, f"trace_run/{dtype}")


def test_a_slot_used_again_starts_from_an_empty_state(folders):
    """One slot: a long request, then a short one in the same slot; the second must see neither the first's
    keys nor the rows its convolution kept."""
    folder = folders[("A", "float32")]
    eng = _engine(folder, "float32", max_tokens=512)
    cfg, w = plain.read_model(folder)
    long_req, short_req = prompts(ALL["A"]["vocab"], [200, 30], seed=5)
    for toks in (long_req, short_req, long_req[:90]):
        slot = eng.acquire()
        assert slot == 0
        got = eng.step([(slot, toks[:-2])], [list(range(len(toks) - 2))]).cpu().numpy()
        got = np.concatenate([got] + [eng.step([(slot, [t])], [[0]]).cpu().numpy() for t in toks[-2:]])
        eng.release(slot)
        assert ru.rel_err(got, plain.forward(cfg, w, toks).numpy()) < F32_TOL
    eng.cache.alloc.check_consistent()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_past_every_window(folders, dtype):
    """A short prompt and 330 single-token steps: the window of every layer and several page borders pass under
    decoded tokens; decode steps replay a CUDA graph."""
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


def test_a_far_key_and_the_windows_edge_show_in_the_logits(folders):
    """Whole model, float32: changing one token changes the logits of the positions whose window still holds it (in
    a model of n layers the change travels n windows far) and of none before it, as in the plain implementation."""
    folder = folders[("E", "float32")]
    cfg, w = plain.read_model(folder)
    eng = _engine(folder, "float32", max_tokens=1024)
    toks = prompts(ALL["E"]["vocab"], [260], seed=12)[0]
    other = list(toks)
    other[100] = (toks[100] + 1) % ALL["E"]["vocab"]
    outs = []
    for seq in (toks, other):
        slot = eng.acquire()
        a = eng.step([(slot, seq[:150])], [list(range(150))]).cpu().numpy()
        b = [eng.step([(slot, [t])], [[0]]).cpu().numpy() for t in seq[150:]]
        eng.release(slot)
        outs.append(np.concatenate([a] + b))
        assert ru.rel_err(outs[-1], plain.forward(cfg, w, seq).numpy()) < F32_TOL
    moved = np.abs(outs[0] - outs[1]).max(axis=1) > 0
    reach = 100 + (41 - 1) + (41 - 1) + (5 - 1) + 3 * 3        # three layers' windows and their convolutions' taps
    assert not moved[:100].any() and moved[100] and not moved[reach + 1 :].any()


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
                assert logits.max() - logits[tok] <= 1e-5 * np.abs(logits).max(), (name, p[:4], o.tokens)
            else:       # bfloat16 may differ only where the plain logits nearly tie
                assert logits.max() - logits[tok] <= 3e-2 * np.abs(logits).max(), (name, p[:4], o.tokens)
            ids.append(tok)
    info = session.info()
    assert info["architecture"] == "Voserax" and info["n_layers"] == len(ALL[name]["layers"])


def test_random_weights_on_the_device_equal_the_folder(folders):
    """``Engine.random`` makes the same model as the folder written from the same seed."""
    from llmoxide_b200 import Engine, LoadOptions, read_config

    folder = folders[("A", "float32")]
    toks = prompts(ALL["A"]["vocab"], [50], seed=1)[0]
    opts = dict(dtype="float32", max_tokens=256, max_batch=2)
    a = Engine.load(folder, LoadOptions(**opts))
    b = Engine.random(read_config(dict(copy.deepcopy(ALL["A"]), torch_dtype="float32")), 977, LoadOptions(**opts))
    la = a.step([(a.acquire(), toks)], [[49]])
    lb = b.step([(b.acquire(), toks)], [[49]])
    assert torch.equal(la, lb)
