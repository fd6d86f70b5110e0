"""Darolix on the GPU against the plain implementation (tests/plain_darolix.py).

Mechanisms alone (kernel against the plain function of the same mechanism):
the scaled embedding with its position vector, the short convolution and its
carried inputs, the recurrence with one decay per head and with one per key
channel (portions, reused slots, a far token whose trace must survive), the
gated norms, the capped attention (far keys, page borders, key and value sizes
that differ), the sum of normed branches, the router with its correction and
identity experts.  Then whole models of three configurations, in 32-bit and
bfloat16: whole prompts, prefill against token-by-token decoding, portions
down to two tokens, batches of unequal requests in a pool so small that pages
and slots are used again, long decoding from the first token, the stream after
every layer run, and greedy generation through the engine and the programs."""
import json
import subprocess
import sys

import numpy as np
import pytest
import torch

import plain_darolix as plain
import replay
import tiny_darolix as tiny
from gpu_util import assert_close, dev, paged_from_sequences, rounded

pytestmark = pytest.mark.gpu

F32, BF16 = torch.float32, torch.bfloat16
TOL = {"float32": 2e-5, "bfloat16": 9e-2}
KERNEL_TOL = {F32: 1e-5, BF16: 2e-2}
LENGTHS = {"A": [1, 2, 37, 64, 65, 130], "B": [3, 16, 17, 33, 80], "C": [5, 63, 129, 200], "D": [2, 64, 150, 300]}
DECODED = 12


# ---------------------------------------------------------------------------------------------------
# mechanisms alone
# ---------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("width,scale", [(96, 3.0), (33, 1.0), (128, 11.3)])
def test_embedding_is_scaled_and_gets_its_position_vector(width, scale):
    from alofa_b200.csrc import ops

    rng = np.random.default_rng(1)
    table = rounded(rng.standard_normal((50, width)), BF16)
    ids = rng.integers(0, 50, size=9).astype(np.int32)
    positions = np.array([0, 1, 2, 63, 64, 500, 4095, 7, 30000], dtype=np.int32)
    freq = (10000.0 ** (-2.0 * np.arange((width + 1) // 2) / width)).astype(np.float32)
    out = torch.empty((9, width), dtype=F32, device="cuda")
    ops.embed_scaled(out, dev(table, BF16), dev(ids), dev(positions), scale, dev(freq))
    want = np.stack([plain.embedding(table, [i], scale, first_position=int(p))[0] for i, p in zip(ids, positions)])
    # the angle is an fp32 product: at position p it carries an error of about p * 6e-8
    assert_close(out.cpu(), want, 1e-5 + 2e-7 * 30000 / max(1.0, np.abs(want).max()), "embedding")


def scan_setup(n_slots, words):
    return torch.full((n_slots, words), 0.0, dtype=F32, device="cuda")


def meta(counts, slots):
    q_start = np.concatenate([[0], np.cumsum(counts)]).astype(np.int32)
    seq = np.concatenate([np.full(c, s, dtype=np.int32) for s, c in enumerate(counts)])
    return dev(q_start), dev(np.asarray(slots, dtype=np.int32)), dev(seq)


@pytest.mark.parametrize("channels,taps", [(40, 4), (300, 2), (7, 3), (16, 1)])
def test_short_convolution_carries_its_last_inputs(channels, taps):
    """Two requests in portions of 1, 2 and many tokens, slots used in another order; against the whole sequences."""
    from alofa_b200.csrc import ops

    rng = np.random.default_rng(2)
    lengths = [23, 9]
    offset, ld = 5, channels + 11
    u = [rounded(rng.standard_normal((n, ld)), F32) for n in lengths]
    w, b = rounded(rng.standard_normal((channels, taps)), F32), rounded(rng.standard_normal(channels), F32)
    want = [plain.short_convolution(x[:, offset : offset + channels], w, b) for x in u]
    state = scan_setup(4, max(1, (taps - 1) * channels) + 3)
    got = [[], []]
    at = [0, 0]
    for cuts in ([1, 2], [2, 1], [5, 6], [1, 0], [14, 0]):
        live = [r for r in (0, 1) if cuts[r] and at[r] < lengths[r]]
        rows = np.concatenate([u[r][at[r] : at[r] + cuts[r]] for r in live])
        counts = [min(cuts[r], lengths[r] - at[r]) for r in live]
        q_start, slots, seq = meta(counts, [3 if r == 0 else 1 for r in live])
        out = torch.empty((rows.shape[0], channels), dtype=F32, device="cuda")
        ops.causal_conv(out, dev(rows, F32), offset, dev(w, F32), dev(b, F32), state[:, 3:], q_start, slots, seq, len(live))
        o = out.cpu().numpy()
        k = 0
        for r, c in zip(live, counts):
            got[r].append(o[k : k + c])
            k += c
            at[r] += c
    for r in (0, 1):
        assert at[r] == lengths[r]
        assert_close(np.concatenate(got[r]), want[r], 1e-5, f"request {r}")
    assert (state[[0, 2]] == 0).all() and (state[:, :3] == 0).all(), "state of another slot, or words before the convolution's, were written"


def run_scan(mode, lengths, cuts, H, G, N, P, tau=1.0, seed=3, boost=None):
    """The recurrence over requests cut into portions, against the plain whole-sequence form."""
    from alofa_b200.csrc import ops

    rng = np.random.default_rng(seed)
    f = lambda *s: rounded(rng.standard_normal(s), F32)
    data, want = [], []
    a_log, d_skip, dt_bias = rounded(np.log(rng.uniform(0.3, 3.0, H)), F32), f(H), rounded(rng.uniform(-2, 0.5, H), F32)
    for n in lengths:
        v, b, c = f(n, H * P), f(n, G * N), f(n, G * N)
        dec = f(n, H) if mode == 0 else 2.0 + f(n, H * N)
        if boost is not None and n > boost[1]:  # one early token written large, read back by one late query alone
            v[boost[0]] *= 30.0
        data.append((v, b, c, dec))
        if mode == 0:
            want.append(plain.scalar_decay_recurrence(v.reshape(n, H, P), b.reshape(n, G, N), c.reshape(n, G, N), plain.softplus(dec + dt_bias), a_log, d_skip, G).reshape(n, H * P))
        else:
            alpha = (1.0 / (1.0 + np.exp(-dec))) ** (1.0 / tau)
            want.append(plain.channel_decay_recurrence(c.reshape(n, H, N) * N ** -0.5, b.reshape(n, H, N), v.reshape(n, H, P), alpha.reshape(n, H, N)).reshape(n, H * P))
    state = scan_setup(5, H * P * N + 2)
    slots_of = [4, 0, 2][: len(lengths)]
    got = [[] for _ in lengths]
    at = [0] * len(lengths)
    step = 0
    while any(at[r] < lengths[r] for r in range(len(lengths))):
        live = [r for r in range(len(lengths)) if at[r] < lengths[r] and (step + r) % 3 != 2]  # requests sit steps out
        step += 1
        if not live:
            continue
        counts = [min(cuts[(step + r) % len(cuts)], lengths[r] - at[r]) for r in live]
        cat = lambda i: dev(np.concatenate([data[r][i][at[r] : at[r] + c] for r, c in zip(live, counts)]), F32)
        v, b, c, dec = cat(0), cat(1), cat(2), cat(3)
        q_start, slots, _ = meta(counts, [slots_of[r] for r in live])
        y = torch.empty((v.shape[0], H * P), dtype=F32, device="cuda")
        if mode == 0:
            ops.linear_scan(y, v, 0, b, 0, c, 0, dec, 0, state, q_start, slots, len(live), H, G, N, P, 0, dt_bias=dev(dt_bias, F32), a_log=dev(a_log, F32), d_skip=dev(d_skip, F32))
        else:
            ops.linear_scan(y, v, 0, b, 0, c, 0, dec, 0, state, q_start, slots, len(live), H, G, N, P, 1, tau=tau, q_scale=N ** -0.5)
        o = y.cpu().numpy()
        k = 0
        for r, cnt in zip(live, counts):
            got[r].append(o[k : k + cnt])
            k += cnt
            at[r] += cnt
    for r in range(len(lengths)):
        assert_close(np.concatenate(got[r]), want[r], 2e-5, f"mode {mode}, request {r} of {lengths[r]} tokens")
    assert (state[[1, 3]] == 0).all() and (state[:, H * P * N :] == 0).all()
    return state


@pytest.mark.parametrize("H,G,N,P", [(5, 1, 16, 24), (6, 3, 24, 12), (4, 4, 40, 8), (2, 1, 128, 64), (3, 3, 300, 5), (1, 1, 1, 1)])
def test_recurrence_with_one_decay_per_head(H, G, N, P):
    run_scan(0, [70, 33, 1], [1, 2, 17, 1, 40], H, G, N, P)


@pytest.mark.parametrize("H,N,P,tau", [(3, 16, 40, 4.0), (2, 8, 8, 9.0), (5, 20, 4, 1.0), (2, 64, 64, 16.0), (1, 520, 3, 2.0)])
def test_recurrence_with_one_decay_per_key_channel(H, N, P, tau):
    run_scan(1, [70, 33, 1], [2, 1, 17, 1, 40], H, H, N, P, tau=tau)


def test_recurrence_keeps_a_far_token_and_a_freed_slot_starts_anew():
    """400 tokens decoded one by one after a prompt of two: the state carries what token 1 wrote (scaled up so
    that losing it shows); then the slot is zeroed for another request, which must not see the old state."""
    from alofa_b200.csrc import ops

    state = run_scan(1, [402], [2] + [1] * 7, 2, 2, 16, 8, tau=40.0, seed=5, boost=(1, 300))
    assert float(state[4].abs().max()) > 0
    state[4].zero_()
    rng = np.random.default_rng(6)
    v, b, c, dec = (dev(rounded(rng.standard_normal((3, w)), F32), F32) for w in (16, 32, 32, 32))
    q_start, slots, _ = meta([3], [4])
    y = torch.empty((3, 16), dtype=F32, device="cuda")
    ops.linear_scan(y, v, 0, b, 0, c, 0, dec, 0, state, q_start, slots, 1, 2, 2, 16, 8, 1, tau=40.0, q_scale=0.25)
    alpha = (1.0 / (1.0 + np.exp(-dec.cpu().numpy().astype(np.float64)))) ** (1.0 / 40.0)
    want = plain.channel_decay_recurrence(c.cpu().numpy().astype(np.float64).reshape(3, 2, 16) * 0.25, b.cpu().numpy().astype(np.float64).reshape(3, 2, 16),
                                          v.cpu().numpy().astype(np.float64).reshape(3, 2, 8), alpha.reshape(3, 2, 16)).reshape(3, 16)
    assert_close(y.cpu(), want, 2e-5, "a request in a slot that another one left")


@pytest.mark.parametrize("dtype", [F32, BF16])
@pytest.mark.parametrize("width,groups,wlen,gate_first", [(120, 3, 120, True), (96, 1, 96, True), (120, 3, 40, False), (24, 24, 1, False)])
def test_gated_norms_in_both_orders(dtype, width, groups, wlen, gate_first):
    from alofa_b200.csrc import ops

    rng = np.random.default_rng(7)
    n, eps, g_off = 5, 1e-3, 9
    y, gate, w = rounded(3 * rng.standard_normal((n, width)), F32), rounded(rng.standard_normal((n, width + 20)), F32), rounded(1 + 0.2 * rng.standard_normal(wlen), F32)
    out = torch.empty((n, width), dtype=dtype, device="cuda")
    ops.gated_group_norm(out, dev(y, F32), dev(gate, F32), g_off, dev(w, F32), groups, eps, gate_first)
    g = plain.silu(gate[:, g_off : g_off + width])
    wide = np.tile(w, width // wlen)
    if gate_first:
        want = plain.unit_rms((y * g).reshape(n, groups, -1), eps).reshape(n, width) * wide
    else:
        want = plain.unit_rms(y.reshape(n, groups, -1), eps).reshape(n, width) * wide * g
    assert_close(out.float().cpu(), want, KERNEL_TOL[dtype], "gated norm")


@pytest.mark.parametrize("hidden", [96, 100, 1030])
def test_normed_branches_are_averaged_into_the_stream(hidden):
    from alofa_b200.csrc import ops

    rng = np.random.default_rng(8)
    h, a, b = (rounded(rng.standard_normal((4, hidden)) * s, F32) for s in (10.0, 0.3, 50.0))
    wa, wb = rounded(1 + 0.1 * rng.standard_normal(hidden), F32), rounded(1 + 0.1 * rng.standard_normal(hidden), F32)
    hd = dev(h, F32)
    ops.branch_norm_add(hd, dev(a, F32), dev(wa, F32), dev(b, F32), dev(wb, F32), 1e-5, 0.5)
    assert_close(hd.cpu(), h + 0.5 * (plain.unit_rms(a, 1e-5) * wa + plain.unit_rms(b, 1e-5) * wb), 1e-6, "two branches")
    hd = dev(h, F32)
    ops.branch_norm_add(hd, dev(a, F32), dev(wa, F32), None, None, 1e-5, 1.0)
    assert_close(hd.cpu(), h + plain.unit_rms(a, 1e-5) * wa, 1e-6, "one branch")


def attention_case(rng, lengths, H, G, d, dv, dtype, page, coef, every, eps, far=None):
    """Raw projections per request -> prepared queries, paged caches written by the kernel itself, plain outputs' inputs."""
    from alofa_b200.csrc import ops

    blocks = [-(-n // page) for n in lengths]
    total = sum(blocks) + 3
    order = rng.permutation(total)
    table = np.full((len(lengths), max(blocks) + 1), -1, dtype=np.int32)
    k_cache = torch.full((total * page, G, d), 7.0, dtype=dtype, device="cuda")
    v_cache = torch.full((total * page, G, dv), -7.0, dtype=dtype, device="cuda")
    raws, queries, at = [], [], 0
    for r, n in enumerate(lengths):
        table[r, : blocks[r]] = order[at : at + blocks[r]]
        at += blocks[r]
        raw = rounded(rng.standard_normal((n, H * d + G * d + G * dv)), F32)
        if far is not None and n > far[1]:  # key `far[0]` and the last query made parallel and long: one score stands out
            direction = rng.standard_normal(d)
            raw[far[0], H * d : H * d + d] = 6.0 * direction
            raw[n - 1, :d] = 6.0 * direction
        raws.append(raw)
        slot_map = np.array([table[r, j // page] * page + j % page for j in range(n)], dtype=np.int32)
        q = torch.empty((n, H * d), dtype=dtype, device="cuda")
        ops.qkv_prepare(q, k_cache, v_cache, dev(raw, F32), dev(np.arange(n, dtype=np.int32)), dev(slot_map), H, G, d, dv, True, eps, coef, every)
        queries.append(q)
    return raws, queries, k_cache, v_cache, dev(table)


def plain_attention_of(raw, H, G, d, dv, eps, coef, every, scale, softcap, dtype):
    n = raw.shape[0]
    q = plain.unit_rms(raw[:, : H * d].reshape(n, H, d), eps) * plain.query_temperature(np.arange(n), coef, every)[:, None, None]
    k = plain.unit_rms(raw[:, H * d : (H + G) * d].reshape(n, G, d), eps)
    v = raw[:, (H + G) * d :].reshape(n, G, dv)
    return plain.capped_attention(rounded(q, dtype), rounded(k, dtype), rounded(v, dtype), scale, softcap).reshape(n, H * dv)


@pytest.mark.parametrize("dtype", [F32, BF16])
@pytest.mark.parametrize("H,G,d,dv,softcap,coef,every", [(6, 3, 16, 24, 5.0, 0.5, 4), (2, 1, 24, 8, 0.0, 0.0, 1), (5, 5, 12, 12, 30.0, 0.2, 7), (4, 2, 64, 64, 20.0, 0.3, 16), (1, 1, 40, 200, 2.0, 0.0, 1)])
def test_capped_attention_over_paged_keys(dtype, H, G, d, dv, softcap, coef, every):
    """Prompts and decoding, lengths at page borders (16) and at the kernel's chunk borders (128); queries normed and
    scaled by position, scores capped, values of another width than keys."""
    from alofa_b200.csrc import ops

    rng = np.random.default_rng(9)
    lengths = [1, 2, 15, 16, 17, 127, 128, 129, 300]
    page, eps, scale = 16, 1e-5, 0.3
    raws, queries, k_cache, v_cache, table = attention_case(rng, lengths, H, G, d, dv, dtype, page, coef, every, eps)
    want = [plain_attention_of(raw, H, G, d, dv, eps, coef, every, scale, softcap, dtype) for raw in raws]
    for last_only in (False, True):
        picks = [[n - 1] if last_only else list(range(n)) for n in lengths]
        q = torch.cat([queries[r][picks[r]] for r in range(len(lengths))]).contiguous()
        positions = dev(np.concatenate([np.array(p, dtype=np.int32) for p in picks]))
        seq = dev(np.concatenate([np.full(len(p), r, dtype=np.int32) for r, p in enumerate(picks)]))
        out = torch.empty((q.shape[0], H * dv), dtype=dtype, device="cuda")
        ops.paged_attention_generic(out, q, k_cache, v_cache, positions, seq, table, page, H, G, d, None, scale, softcap, dv)
        got, at = out.float().cpu().numpy(), 0
        for r, p in enumerate(picks):
            assert_close(got[at : at + len(p)], want[r][p], KERNEL_TOL[dtype], f"request {r} ({lengths[r]} keys), decoding={last_only}")
            at += len(p)


@pytest.mark.parametrize("dtype", [F32, BF16])
def test_one_far_key_among_hundreds(dtype):
    """Key 3 of 700 and the last query point the same way: after norm, scale and cap that key holds most of the
    weight; the output must be (nearly) its value, which a lost page or a wrong position would not give."""
    from alofa_b200.csrc import ops

    rng = np.random.default_rng(10)
    H, G, d, dv, page, eps, scale, softcap = 2, 1, 32, 16, 16, 1e-6, 0.5, 14.0
    raws, queries, k_cache, v_cache, table = attention_case(rng, [700], H, G, d, dv, dtype, page, 0.0, 1, eps, far=(3, 600))
    want = plain_attention_of(raws[0], H, G, d, dv, eps, 0.0, 1, scale, softcap, dtype)
    out = torch.empty((1, H * dv), dtype=dtype, device="cuda")
    ops.paged_attention_generic(out, queries[0][699:].contiguous(), k_cache, v_cache, dev(np.array([699], dtype=np.int32)), dev(np.array([0], dtype=np.int32)), table, page,
                                H, G, d, None, scale, softcap, dv)
    assert_close(out.float().cpu(), want[699:], KERNEL_TOL[dtype], "last query")
    value3 = rounded(raws[0][3, (H + G) * d :], dtype)
    assert np.abs(want[699, :dv] - value3).max() < 0.2 * np.abs(value3).max(), "the test's far key does not stand out"


@pytest.mark.parametrize("experts,identity,top", [(5, 2, 3), (7, 0, 2), (4, 3, 4), (3, 0, 1), (40, 9, 6)])
def test_router_with_correction_and_identity_experts(experts, identity, top):
    """Choices by score + correction, weights from the scores alone over their sum; identity choices get no row
    of the sorted matrix and come back as the token's own input."""
    from alofa_b200.csrc import ops

    rng = np.random.default_rng(11)
    n, hidden, routed = 37, 48, experts + identity
    x = rounded(rng.standard_normal((n, hidden)), F32)
    wr = rounded(2 * rng.standard_normal((routed, hidden)) / np.sqrt(hidden), F32)
    corr = rounded(0.3 * rng.standard_normal(routed), F32)  # large enough to change the choice often
    chosen, weight, margin = plain.route(x, wr, corr, top)
    plain_nocorr, _, _ = plain.route(x, wr, np.zeros(routed), top)
    assert (np.sort(chosen, 1) != np.sort(plain_nocorr, 1)).any(), "the test's correction changes no choice"
    choice = torch.empty((n, top), dtype=torch.int32, device="cuda")
    wgt = torch.empty((n, top), dtype=F32, device="cuda")
    ops.moe_router(choice, wgt, None, dev(x, F32), dev(wr, F32), routed, top, True, True, dev(corr, F32), 1e-20)
    sure = margin > 1e-5
    assert (choice.cpu().numpy()[sure] == chosen[sure]).all()
    assert_close(wgt.cpu().numpy()[sure], weight[sure], 1e-5, "weights")
    tile = 64
    tiles = -(-n * top // tile) + experts
    dest = torch.empty((n, top), dtype=torch.int32, device="cuda")
    tile_expert = torch.empty((tiles,), dtype=torch.int32, device="cuda")
    ops.moe_sort(dest, tile_expert, choice, experts, tile)
    d, c = dest.cpu().numpy(), choice.cpu().numpy()
    assert ((d < 0) == (c >= experts)).all()
    te = tile_expert.cpu().numpy()
    assert all(te[d[t, k] // tile] == c[t, k] for t in range(n) for k in range(top) if d[t, k] >= 0)
    assert len(set(d[d >= 0].tolist())) == int((d >= 0).sum())
    ys = rounded(rng.standard_normal((tiles * tile, hidden)), F32)
    y = dev(np.ones((n, hidden)), F32)
    ops.moe_combine(y, dev(ys, F32), dest, wgt, None, None, top, dev(x, F32), add=True)
    w = wgt.cpu().numpy().astype(np.float64)
    want = 1.0 + sum(w[:, k : k + 1] * np.where(d[:, k : k + 1] >= 0, ys[np.maximum(d[:, k], 0)], x) for k in range(top))
    assert_close(y.cpu(), want, 1e-5, "combined")


@pytest.mark.parametrize("hidden,ff", [(64, 72), (128, 320), (192, 64)])
def test_gated_products_by_tile_on_the_tcgen05_kernel(hidden, ff):
    """Tiles of 128 sorted rows, each multiplied by its expert's gate and up rows with silu(gate) * up in the
    epilogue; a tile that names no expert is left alone."""
    from alofa_b200.csrc import ops

    rng = np.random.default_rng(12)
    experts, tiles = 3, 5
    tile_expert = np.array([2, 0, -1, 1, 2], dtype=np.int32)
    x = rounded(rng.standard_normal((tiles * 128, hidden)), BF16)
    w = rounded(rng.standard_normal((experts, 2 * ff, hidden)) / np.sqrt(hidden), BF16)
    out = torch.full((tiles * 128, ff), 3.0, dtype=BF16, device="cuda")
    assert ops.gemm_by_tile_gated(out, dev(x, BF16), dev(w, BF16), dev(tile_expert), 128)
    got = out.float().cpu().numpy()
    for i, e in enumerate(tile_expert):
        rows = slice(i * 128, (i + 1) * 128)
        if e < 0:
            assert (got[rows] == 3.0).all()
            continue
        want = plain.silu(x[rows] @ w[e, :ff].T) * (x[rows] @ w[e, ff:].T)
        assert_close(got[rows], want, KERNEL_TOL[BF16], f"tile {i}")


# ---------------------------------------------------------------------------------------------------
# whole models
# ---------------------------------------------------------------------------------------------------
@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    base = tmp_path_factory.mktemp("darolix_gpu")
    return {name: tiny.write(base / name, name, seed=20 + i) for i, name in enumerate(tiny.CONFIGS)}


def make_requests(name):
    reqs, prompts = {}, {}
    for i, n in enumerate(LENGTHS[name]):
        reqs[f"r{i}"] = tiny.tokens(name, n + DECODED, seed=i)
        prompts[f"r{i}"] = n
    return reqs, prompts


@pytest.fixture(scope="module")
def plain_logits(folders):
    """name -> (request -> logits, request -> positions before the first close call of a router)."""
    out = {}
    for name, folder in folders.items():
        w, cfg = plain.load(folder)
        logits, sure = {}, {}
        for rid, toks in make_requests(name)[0].items():
            margins = []
            logits[rid] = plain.forward(toks, w, cfg, margins=margins)
            sure[rid] = plain.sure_prefix(margins, len(toks))
        out[name] = (logits, sure)
    return out


def runner_for(folder, dtype, block, pages, max_requests=4, graphs=True):
    from alofa_b200.engine.loading import load_model
    from alofa_b200.engine.step import StepRunner

    model, *_ = load_model(folder, dtype)
    return StepRunner(model, block_size=block, num_pages=pages, max_requests=max_requests, max_tokens=pages * block, max_step_tokens=512, cuda_graphs=graphs)


def assert_most_close(errors, tol, what):
    errors = np.asarray(errors)
    assert (errors > tol).mean() <= 0.25 and np.median(errors) <= tol / 3, \
        f"{what}: {(errors > tol).sum()} of {len(errors)} positions beyond {tol:.1e}, median {np.median(errors):.3e}, worst {errors.max():.3e}"


def compare(steps, outputs, want, vocab, tol, what, sure=None):
    """Every position within ``tol`` in 32-bit.  In bfloat16 strictly up to a request's first close call of a
    router (``sure``): a routed feed-forward is not continuous, and where two choice scores lie within
    rounding bfloat16 may rightly take the other expert; that position, and through state and cache the
    ones after it, then differ by more than rounding.  Over all positions three quarters keep the bound and
    the median a third of it: a lost state, a wrong key or page moves every position by order one."""
    got = replay.collect(steps, outputs, vocab)
    errors = []
    for rid, rows in got.items():
        ref = want[rid][: len(rows)]
        assert rows.shape == ref.shape, f"{what} {rid}: {rows.shape} vs {ref.shape}"
        err = np.abs(rows - ref).max(axis=-1) / max(1.0, float(np.abs(ref).max()))
        n = len(rows) if sure is None else min(len(rows), sure[rid])
        if n:
            assert err[:n].max() <= tol, f"{what} {rid}: position {int(err[:n].argmax())} differs by {err[:n].max():.3e} > {tol:.1e}"
        errors.append(err)
    assert_most_close(np.concatenate(errors), tol, what)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(tiny.CONFIGS))
def test_whole_decoded_portions_and_mixed_batches(folders, plain_logits, name, dtype):
    """The same requests whole, with the last tokens decoded one by one, in portions down to two tokens, and
    mixed (portions beside single tokens, four live at most, four state slots) in a pool that holds two of
    the longest: pages and slots are given back and used again.  Every position against plain."""
    reqs, prompts = make_requests(name)
    vocab = tiny.CONFIGS[name]["vocab"]
    block = 16 if name == "B" else 64
    per_request = -(-max(len(t) for t in reqs.values()) // block)
    schedules = {
        "whole": (replay.whole(reqs), per_request),
        "decoded": (replay.tail_decoded(reqs, tail=DECODED + 20), per_request),
        "portions": (replay.portions(reqs), per_request),
        "mixed": (replay.mixed(reqs, prompts, 2 * per_request * block + block, block, seed=3), 2 * per_request + 1),
    }
    for what, (steps, pages) in schedules.items():
        runner = runner_for(folders[name], dtype, block, pages, max_requests=4)
        out = replay.run_inprocess(runner, steps)
        compare(steps, out, plain_logits[name][0], vocab, TOL[dtype], f"{name}/{dtype}/{what}", sure=plain_logits[name][1] if dtype == "bfloat16" else None)
        assert runner.manager.free_pages() == [pages] and runner.manager.live_requests() == 0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_from_the_first_token(folders, dtype):
    """One prompt token, then 150 tokens one by one (past two page borders and past every step of the query
    temperature), two requests side by side that started 40 steps apart; decode steps are replayed as graphs."""
    from alofa_b200.engine.step import StepEntry

    name = "A"
    w, cfg = plain.load(folders[name])
    a, b = tiny.tokens(name, 151, seed=50), tiny.tokens(name, 111, seed=51)
    ma, mb = [], []
    want_a, want_b = plain.forward(a, w, cfg, margins=ma), plain.forward(b, w, cfg, margins=mb)
    sure_a, sure_b = (plain.sure_prefix(ma, 151), plain.sure_prefix(mb, 111)) if dtype == "bfloat16" else (151, 111)
    runner = runner_for(folders[name], dtype, 64, 5, max_requests=2)
    sa = runner.admit(0)
    sb, errors = None, []
    for i in range(151):
        entries = [StepEntry(sa, [a[i]], [0])]
        if i >= 40:
            if sb is None:
                sb = runner.admit(1)
            entries.append(StepEntry(sb, [b[i - 40]], [0]))
        rows = runner.forward(entries).float().cpu().numpy()
        for row, want, k, sure, who in ((rows[0], want_a, i, sure_a, "first"),) + (((rows[1], want_b, i - 40, sure_b, "second"),) if i >= 40 else ()):
            if k < sure:
                assert_close(row, want[k], TOL[dtype], f"{who} request, token {k}")
            errors.append(np.abs(row - want[k]).max() / max(1.0, float(np.abs(want).max())))
    assert_most_close(errors, TOL[dtype], "long decoding")
    runner.check_status()
    assert runner.manager.defects() == 0


def test_batches_and_cuts_do_not_change_a_request(folders):
    """float32: a request's logits in a mixed batch, and in portions, equal those it gets alone and whole, up to
    the rounding of sums taken in another order."""
    name = "B"
    reqs, prompts = make_requests(name)
    vocab = tiny.CONFIGS[name]["vocab"]
    alone = replay.collect(replay.whole(reqs), replay.run_inprocess(runner_for(folders[name], "float32", 16, 10), replay.whole(reqs)), vocab)
    steps = replay.mixed(reqs, prompts, 400, 16, seed=9)
    together = replay.collect(steps, replay.run_inprocess(runner_for(folders[name], "float32", 16, 25), steps), vocab)
    cut = replay.portions(reqs)
    in_portions = replay.collect(cut, replay.run_inprocess(runner_for(folders[name], "float32", 16, 10), cut), vocab)
    for rid in reqs:
        for other, what in ((together, "mixed"), (in_portions, "portions")):
            assert np.abs(alone[rid] - other[rid]).max() <= 3e-6 * max(1.0, np.abs(alone[rid]).max()), (rid, what)


def test_the_stream_after_every_layer_run(folders):
    """float32: the residual stream after each run of a layer (looped layers count each time)."""
    import alofa_b200.parts.block as block
    from alofa_b200.engine.step import StepEntry

    name = "A"
    w, cfg = plain.load(folders[name])
    ids = tiny.tokens(name, 30, seed=77)
    want = []
    plain.forward(ids, w, cfg, streams=want)
    seen, original = [], block.ParallelResidual.forward

    def recording(self, ctx, h, cache, writes=True):
        original(self, ctx, h, cache, writes)
        ctx.flush_pending()
        seen.append(h.clone())

    block.ParallelResidual.forward = recording
    try:
        runner = runner_for(folders[name], "float32", 64, 1, graphs=False)
        runner.forward([StepEntry(runner.admit(0), ids, [0])])
    finally:
        block.ParallelResidual.forward = original
    assert len(seen) == len(want) == 6
    for k, (got, ref) in enumerate(zip(seen, want)):
        assert_close(got.cpu(), ref, 1e-5, f"after layer run {k}")


@pytest.mark.parametrize("name", list(tiny.CONFIGS))
def test_greedy_generation_through_the_engine(folders, name):
    """Engine.generate (scheduler, chunked prefill, decode graphs): float32 tokens equal plain greedy; bfloat16
    tokens are each within rounding of the plain maximum, up to a router's first close call."""
    from alofa_b200.engine.engine import Engine

    w, cfg = plain.load(folders[name])
    prompts = [tiny.tokens(name, n, seed=200 + i) for i, n in enumerate([1, 7, 40, 90, 18])]
    want = [plain.greedy(p, 6, w, cfg) for p in prompts]
    eng = Engine(str(folders[name]), dtype="float32", block_size=16, max_batch=3, token_budget=48, max_chunk=32, max_tokens=128)
    assert eng.generate(prompts, max_new_tokens=6) == want
    assert eng.stats()["defects"] == 0
    eng16 = Engine(str(folders[name]), dtype="bfloat16", block_size=16, max_batch=3, token_budget=48, max_chunk=32, max_tokens=128)
    for p, out in zip(prompts, eng16.generate(prompts, max_new_tokens=6)):
        seq = list(p)
        for tok in out:
            margins = []
            row = plain.forward(seq, w, cfg, margins=margins)[-1]
            if plain.sure_prefix(margins, len(seq)) < len(seq):
                break
            assert row.max() - row[tok] <= 8e-2 * max(1.0, float(np.abs(row).max())), "a bfloat16 token is not near the plain maximum"
            seq.append(tok)
    eng16.runner.check_status()


def test_the_programs_take_the_architecture(folders, tmp_path):
    """bin/trace_run replays a schedule and bin/generate generates, both choosing the model by config.json."""
    name = "C"
    reqs, _ = make_requests(name)
    reqs = {k: reqs[k] for k in ("r0", "r2")}
    w, cfg = plain.load(folders[name])
    want = {rid: plain.forward(t, w, cfg) for rid, t in reqs.items()}
    steps = replay.portions(reqs, sizes=(40, 2, 3, 64, 1))
    out = replay.run_trace_program(folders[name], "float32", steps, tmp_path / "out", 512)
    compare(steps, out, want, cfg["vocab"], TOL["float32"], "trace_run")
    prompt = tiny.tokens(name, 12, seed=5)
    done = subprocess.run([sys.executable, str(replay.ROOT / "bin" / "generate"), "--model", str(folders[name]), "--dtype", "float32", "--prompt-ids",
                           ",".join(map(str, prompt)), "--max-new-tokens", "5", "--max-tokens", "64", "--json"], capture_output=True, text=True, timeout=600)
    assert done.returncode == 0, done.stderr[-2000:]
    assert json.loads(done.stdout.strip().splitlines()[-1])["out_ids"] == [plain.greedy(prompt, 5, w, cfg)]
