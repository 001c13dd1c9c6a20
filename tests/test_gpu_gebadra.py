"""Gebadra on the GPU against the plain implementation: every mechanism alone, then whole models
under every way of cutting and batching (whole, last tokens decoded, portions down to two tokens,
mixed batches with pages and state slots used again), long decoding, generation through the
entry point, and the trace runner itself; float32 and bfloat16, three tiny configurations."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

from tests import replay_util as ru
from tests.helpers import GEBADRA, load_plain, make_gebadra_folder
from tests.plain import plain_gebadra as pg

pytestmark = pytest.mark.gpu
ROOT = os.path.abspath(os.path.join(os.path.dirname(__file__), ".."))
DEV = "cuda:0"
TOL_F32_REL = 3e-5          # max |dlogit| over the largest logit: summation order only
# bfloat16: activations between kernels carry 8 bits of mantissa, and these models are made
# sensitive on purpose (sharp softmaxes, gates away from one half, mixed streams); the bound is on
# a row's root-mean-square difference over the root mean square of the logits, on average over
# the rows and for the worst row (measured 0.023 to 0.1 for the worst row, mostly among a
# request's first tokens; it follows the size of the weights), and on the largest single
# difference.  The float32 runs are the sharp test of every schedule; the bfloat16 runs cover the
# 16-bit kernels and caches, and the stand-out keys above show a wrong key in 16 bits too.
TOL_BF16_RMS_MEAN = 0.03
TOL_BF16_RMS = 0.15
TOL_BF16_MAX = 0.12


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    return {name: make_gebadra_folder(tmp_path_factory.mktemp(f"geb_{name}"), cfg, seed)
            for name, (cfg, seed, _) in GEBADRA.items()}


def _ops():
    from paged_batch_engine_b200.csrc import ops
    return ops


# ================================================================ mechanisms alone
@pytest.mark.parametrize("S, W, ydt", [(1, 64, torch.float32), (3, 200, torch.bfloat16), (8, 96, torch.float32)])
def test_stream_norm_folds_collapses_and_normalises(S, W, ydt):
    ops = _ops()
    g = torch.Generator().manual_seed(S * 100 + W)
    T = 7
    r = torch.randn(T, S, W, generator=g)
    y = torch.randn(T, W, generator=g).to(ydt)
    mix, beta, alpha = torch.randn(S, S, generator=g), torch.randn(S, generator=g), torch.randn(S, generator=g)
    gain, bias = torch.randn(W, generator=g), torch.randn(W, generator=g)
    new = torch.einsum("st,nsw->ntw", mix.double(), r.double()) + beta.double()[None, :, None] * y.double()[:, None, :]
    a = torch.einsum("t,ntw->nw", alpha.double(), new)
    want = pg.layer_norm(a, gain.double(), bias.double(), 1e-5)
    dev = lambda t: t.to(DEV).contiguous()
    streams = dev(r)
    out = torch.empty(T, W, dtype=torch.float32, device=DEV)
    ops.stream_norm(streams, dev(y), dev(mix), dev(beta), dev(alpha), dev(gain), dev(bias), out, 1e-5)
    assert torch.allclose(out.cpu().double(), want, atol=2e-5, rtol=1e-5)
    assert torch.allclose(streams.cpu().double(), new, atol=1e-5)             # the streams were updated
    # gathered rows: the streams are left alone; root-mean-square mode; nothing pending
    streams2 = dev(r)
    rows = torch.tensor([5, 0, 5], dtype=torch.int32, device=DEV)
    out2 = torch.empty(3, W, dtype=torch.float32, device=DEV)
    ops.stream_norm(streams2, None, dev(mix), dev(beta), dev(alpha), dev(gain), None, out2, 1e-5, rows, rms=True)
    a2 = torch.einsum("t,ntw->nw", alpha.double(), r.double())[[5, 0, 5]]
    assert torch.allclose(out2.cpu().double(), pg.rms_unit(a2, 1e-5) * gain.double(), atol=2e-5, rtol=1e-5)
    assert torch.equal(streams2.cpu(), r)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_gated_rms_and_branch_mean(dtype):
    ops = _ops()
    g = torch.Generator().manual_seed(3)
    T, H, E = 5, 3, 20
    o = torch.randn(T, H * E, generator=g) * 4
    wide = torch.randn(T, 100 + H * E, generator=g).to(dtype)
    gate = wide[:, 100:]
    gain = torch.randn(H * E, generator=g)
    tol = 1e-5 if dtype == torch.float32 else 2e-2
    joint = ops.gated_rms(o.to(DEV), wide.to(DEV)[:, 100:], gain.to(DEV), H, 1e-6, False, "sigmoid", dtype)
    want = pg.rms_unit(o.double(), 1e-6) * gain.double() * torch.sigmoid(gate.double())
    assert torch.allclose(joint.cpu().double(), want, atol=tol, rtol=tol)
    heads = ops.gated_rms(o.to(DEV), wide.to(DEV)[:, 100:], None, H, 1e-6, True, "silu", dtype)
    want = pg.rms_unit(o.double().reshape(T, H, E), 1e-6).reshape(T, H * E) * pg.silu(gate.double())
    assert torch.allclose(heads.cpu().double(), want, atol=tol, rtol=tol)
    a, b = torch.randn(T, 72, generator=g).to(dtype), (torch.randn(T, 72, generator=g) * 9).to(dtype)
    ga, gb = torch.randn(72, generator=g), torch.randn(72, generator=g)
    got = ops.branch_rms_mean([a.to(DEV), b.to(DEV)], [ga.to(DEV), gb.to(DEV)], 1e-6)
    want = 0.5 * (pg.rms_unit(a.double(), 1e-6) * ga.double() + pg.rms_unit(b.double(), 1e-6) * gb.double())
    assert torch.allclose(got.cpu().double(), want, atol=tol, rtol=tol)


@pytest.mark.parametrize("H, D, E, silu", [(2, 16, 8, True), (3, 24, 40, False), (1, 48, 33, True), (2, 160, 16, False),
                                           (1, 300, 12, True), (2, 128, 64, False)])
def test_linear_attention_recurrence_state_and_batches(H, D, E, silu):
    """Three requests of unequal length in one launch equal each alone; a request cut in two
    launches (its state carried in its row) equals it whole; a state row used again after it was
    zeroed holds nothing of its former owner."""
    ops = _ops()
    g = torch.Generator().manual_seed(H * 1000 + D)
    lens = [13, 1, 30]
    T = sum(lens)
    wide = torch.randn(T, 2 * H * D + H * E + 5, generator=g)
    decay = torch.tensor([0.5, 0.97, 0.999][:H])
    scale = 0.37
    def plain(rows):
        x = wide[rows].double()
        act = pg.silu if silu else (lambda z: z)
        q = act(x[:, :H * D]).reshape(-1, H, D)
        k = act(x[:, H * D:2 * H * D]).reshape(-1, H, D) * scale
        v = act(x[:, 2 * H * D:2 * H * D + H * E]).reshape(-1, H, E)
        return pg.decayed_linear_attention(q, k, v, decay.double().tolist()).reshape(-1, H * E)
    w = wide.to(DEV)
    q, k, v = w[:, :H * D], w[:, H * D:2 * H * D], w[:, 2 * H * D:2 * H * D + H * E]
    state = torch.full((5, H, D, E), float("nan"), device=DEV)
    i32 = lambda a: torch.tensor(a, dtype=torch.int32, device=DEV)
    starts = [0, lens[0], lens[0] + lens[1]]
    slots = [3, 0, 1]
    state[slots] = 0
    out = ops.linear_attention(q, k, v, state, decay.to(DEV), i32(starts), i32(lens), i32(slots), 3, H, scale, silu)
    for s, n in zip(starts, lens):
        want = plain(slice(s, s + n))
        assert torch.allclose(out[s:s + n].cpu().double(), want, atol=2e-4, rtol=2e-4), (s, n)
    # the third request again, in two launches, in slot 3 (used by the first request before)
    s, n = starts[2], lens[2]
    state[3] = 0
    cut = 11
    a = ops.linear_attention(q[s:s + cut], k[s:s + cut], v[s:s + cut], state, decay.to(DEV), i32([0]), i32([cut]),
                             i32([3]), 1, H, scale, silu)
    b = ops.linear_attention(q[s + cut:s + n], k[s + cut:s + n], v[s + cut:s + n], state, decay.to(DEV), i32([0]),
                             i32([n - cut]), i32([3]), 1, H, scale, silu)
    assert torch.allclose(torch.cat([a, b]).cpu(), out[s:s + n].cpu(), atol=1e-4, rtol=1e-4)
    assert torch.allclose(state[3].cpu(), state[1].cpu(), atol=1e-4, rtol=1e-4)
    assert torch.isnan(state[2]).all() and torch.isnan(state[4]).all()          # no other row was touched


@pytest.mark.parametrize("chunk", [64, 16, 5])
def test_linear_attention_long_portions_run_as_chunks(chunk):
    """Requests cut into chunks that run side by side (own contributions, a scan over the chunks,
    then every chunk from its start state) against the plain recurrence: a long request that
    starts from a state it left earlier, a single token, a request of exactly two chunks."""
    from paged_batch_engine_b200.engine.batch import RecurrencePlan, recurrence_plan_arrays
    ops = _ops()
    H, D, E = 3, 40, 24
    g = torch.Generator().manual_seed(chunk)
    lens = [4 * chunk + 3, 1, 2 * chunk]
    head = 9                                    # rows of the first request that ran in an earlier step
    T = head + sum(lens)
    wide = torch.randn(T, 2 * H * D + H * E, generator=g) * 0.7
    decay = torch.tensor([0.6, 0.95, 0.999])

    def plain(rows):
        x = wide[rows].double()
        q, k = x[:, :H * D].reshape(-1, H, D), x[:, H * D:2 * H * D].reshape(-1, H, D)
        return pg.decayed_linear_attention(q, k, x[:, 2 * H * D:].reshape(-1, H, E), decay.double().tolist())
    w = wide.to(DEV)
    q, k, v = w[:, :H * D], w[:, H * D:2 * H * D], w[:, 2 * H * D:]
    i32 = lambda a: torch.tensor(a, dtype=torch.int32, device=DEV)
    state = torch.zeros(4, H, D, E, device=DEV)
    ops.linear_attention(q[:head], k[:head], v[:head], state, decay.to(DEV), i32([0]), i32([head]), i32([2]), 1, H)
    starts = [0, lens[0], lens[0] + lens[1]]
    slots = [2, 0, 3]
    first, scan, second, entries = recurrence_plan_arrays(starts, lens, slots, chunk)
    assert entries == 5 + 2 and len(scan) == 2
    plan = RecurrencePlan(entries, i32(first), len(first), i32(scan), len(scan), i32(second), len(second))
    out = ops.linear_attention(q[head:], k[head:], v[head:], state, decay.to(DEV), i32(starts), i32(lens),
                               i32(slots), 3, H, plan=plan).cpu().double()
    want0 = plain(slice(0, head + lens[0]))[head:].reshape(lens[0], H * E)
    assert torch.allclose(out[:lens[0]], want0, atol=3e-4, rtol=3e-4)
    for s, n in zip(starts[1:], lens[1:]):
        want = plain(slice(head + s, head + s + n)).reshape(n, H * E)
        assert torch.allclose(out[s:s + n], want, atol=3e-4, rtol=3e-4)
    # the states left behind equal those of the uncut recurrence
    ref = torch.zeros(4, H, D, E, device=DEV)
    ops.linear_attention(q[:head + lens[0]], k[:head + lens[0]], v[:head + lens[0]], ref, decay.to(DEV), i32([0]),
                         i32([head + lens[0]]), i32([2]), 1, H)
    assert torch.allclose(state[2].cpu(), ref[2].cpu(), atol=3e-4, rtol=3e-4)


def _attention_part(H, G, D, E, window, pool, dtype, talk, rotary=None, qk_norm=False, seed=0):
    """The attention part with identity projections: its input rows ARE q, k and v, and the first
    H*E columns of its output are the attention's."""
    from paged_batch_engine_b200.parts import PooledWindowAttention
    hidden = max((H + G) * D + G * E, H * E)
    part = PooledWindowAttention(hidden, H, G, D, E, scale=0.5, window=window, eps=1e-6, dtype=dtype, device=DEV,
                                 pool=pool, rotary=rotary, qk_norm=qk_norm, talking_heads=talk is not None,
                                 tensor_names=dict(q="q", k="k", v="v", o="o", q_norm="qn", k_norm="kn", talk="talk"),
                                 weight_suffix="")
    eye = torch.eye(hidden)
    n_in = (H + G) * D + G * E
    g = torch.Generator().manual_seed(seed)
    t = {"p.q": eye[:H * D], "p.k": eye[H * D:(H + G) * D], "p.v": eye[(H + G) * D:n_in], "p.o": eye[:, :H * E]}
    if talk is not None:
        t["p.talk"] = talk
    gains = None
    if qk_norm:
        gains = (1 + 0.3 * torch.randn(H * D, generator=g), 1 + 0.3 * torch.randn(G * D, generator=g))
        t["p.qn"], t["p.kn"] = gains
    part.load({k: v.to(DEV).to(dtype if v.dim() == 2 and k != "p.talk" else torch.float32) for k, v in t.items()}, "p.")
    return part, hidden, gains


def _run_attention(part, x, cuts, page, num_pages, dtype):
    """Feeds rows x of one request through the part in portions of the given sizes."""
    from paged_batch_engine_b200.cache.storage import CacheStorage
    from paged_batch_engine_b200.engine.batch import StepContext, StepEntry
    st = CacheStorage([part.cache_need()], page, num_pages, 2, dtype, DEV, poison=True)
    h = st.manager.add_request()
    outs, i = [], 0
    for n in cuts:
        assert st.manager.reserve(h, n)
        ctx = StepContext(st.manager, [StepEntry(h, [0] * n, [])], torch.device(DEV), [])
        outs.append(part.forward(x[i:i + n].to(DEV).to(dtype), ctx, st.layer(0)).float().cpu())
        st.manager.commit(h, n)
        i += n
    st.manager.check_invariants()
    return torch.cat(outs)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H, G, D, E, window, pool, page", [(4, 2, 16, 8, 9, 4, 4), (2, 1, 8, 24, 5, 8, 16),
                                                            (3, 3, 32, 32, 17, 3, 8), (8, 2, 64, 16, 40, 16, 16)])
def test_window_and_pooled_blocks_with_a_stand_out_key(H, G, D, E, window, pool, page, dtype):
    """One key that every query scores far above all others, placed in turn where a fault would
    show: just inside and just outside the window, in the block that is just seen or not yet, at
    a page's edge, at the very start; the request runs as a prompt portion and then token by token."""
    T = 3 * window + 4 * pool + 7
    g = torch.Generator().manual_seed(window * 10 + pool)
    talk = torch.eye(H) * 0.6 + 0.4 * torch.rand(H, H, generator=g)
    part, hidden, _ = _attention_part(H, G, D, E, window, pool, dtype, talk)
    marks = sorted({0, 1, pool - 1, pool, page - 1, page, window - 1, window, window + pool, T - window - 1,
                    T - window, T - window + 1, T - 2 * window, 2 * pool - 1} & set(range(T)))
    u = torch.zeros(D)
    u[0] = 1.0
    for m in marks[:: (1 if dtype == torch.float32 else 2)]:
        x = torch.zeros(T, hidden)
        n_in = (H + G) * D + G * E
        x[:, :n_in] = torch.randn(T, n_in, generator=g) * 0.3
        x[:, :H * D] += (u * 3.0).repeat(H)                       # every query looks along u
        x[m, H * D:(H + G) * D] += (u * (20.0 * max(1, pool))).repeat(G)    # the stand-out key, also after pooling
        x[m, (H + G) * D:n_in] = 5.0                                  # and a value that shows
        xs = x.to(dtype).float()
        q = xs[:, :H * D].reshape(T, H, D)
        k = xs[:, H * D:(H + G) * D].reshape(T, G, D)
        v = xs[:, (H + G) * D:n_in].reshape(T, G, E)
        if dtype == torch.bfloat16:       # pooled entries are held in the cache's dtype
            want = _plain_attention_rounded_pool(q, k, v, talk, 0.5, window, pool)
        else:
            want = pg.pooled_window_attention(q, k, v, talk, 0.5, window, pool)
        head = T - window - 3
        cuts = [head] + [1] * (T - head)
        got = _run_attention(part, x, cuts, page, (T + page - 1) // page + 1, dtype)[:, :H * E]
        tol = 2e-5 if dtype == torch.float32 else 4e-2
        err = (got - want.reshape(T, H * E)).abs().max(dim=1).values
        assert float(err.max()) <= tol, (m, int(err.argmax()), float(err.max()))


def _plain_attention_rounded_pool(q, k, v, talk, scale, window, pool):
    """The plain attention with the pooled keys and values rounded to bfloat16, as a bfloat16
    cache holds them."""
    T = q.shape[0]
    nb = T // pool
    kp = k[:nb * pool].reshape(nb, pool, *k.shape[1:]).mean(1).bfloat16().float()
    vp = v[:nb * pool].reshape(nb, pool, *v.shape[1:]).mean(1).bfloat16().float()
    H, G = q.shape[1], k.shape[1]
    out = torch.zeros(T, H, v.shape[-1])
    for t in range(T):
        n_seen, first = pg.visible_keys(t, window, pool)
        keys, vals = torch.cat([kp[:n_seen], k[first:t + 1]]), torch.cat([vp[:n_seen], v[first:t + 1]])
        w = torch.stack([torch.softmax((keys[:, h // (H // G)] @ q[t, h]) * scale, 0) for h in range(H)])
        w = talk @ w
        for h in range(H):
            out[t, h] = w[h] @ vals[:, h // (H // G)]
    return out


def test_query_key_norm_and_partial_rotation_in_portions_of_two():
    """The norm over the whole projection, the rotation of neighbouring pairs on part of each head
    with a scaled frequency, positions far from zero in later portions; portions of two tokens."""
    H, G, D, E, window, pool, page = 2, 2, 16, 8, 11, 4, 8
    rotary = dict(base=50.0, dims=8, factor=4.0)
    part, hidden, gains = _attention_part(H, G, D, E, window, pool, torch.float32, None, rotary, True, seed=4)
    T = 61
    g = torch.Generator().manual_seed(8)
    x = torch.zeros(T, hidden)
    n_in = (H + G) * D + G * E
    x[:, :n_in] = torch.randn(T, n_in, generator=g) * 2
    q = pg.rms_unit(x[:, :H * D], 1e-6) * gains[0]
    k = pg.rms_unit(x[:, H * D:(H + G) * D], 1e-6) * gains[1]
    pos = torch.arange(T)
    q = pg.rotate_pairs(q.reshape(T, H, D), pos, 50.0, 8, 4.0)
    k = pg.rotate_pairs(k.reshape(T, G, D), pos, 50.0, 8, 4.0)
    want = pg.pooled_window_attention(q, k, x[:, (H + G) * D:n_in].reshape(T, G, E), torch.eye(H), 0.5, window, pool)
    cuts = [2] * 20 + [7, 2, 3, 2, 5, 2]
    got = _run_attention(part, x, cuts, page, 12, torch.float32)[:, :H * E]
    assert float((got - want.reshape(T, H * E)).abs().max()) <= 2e-5


# ================================================================ whole models
LENGTHS = {"A": [3, 41, 97, 150], "B": [1, 30, 75, 131], "C": [2, 52, 110, 171]}


def requests_for(name, vocab):
    g = torch.Generator().manual_seed(sum(map(ord, name)) + 77)
    return {f"{name}{i}": torch.randint(0, vocab, (n,), generator=g).tolist() for i, n in enumerate(LENGTHS[name])}


_plain_cache = {}


def plain_logits(folder, reqs):
    cfg, w = load_plain(folder)
    out = {}
    for rid, toks in reqs.items():
        key = (folder, tuple(toks))
        if key not in _plain_cache:
            _plain_cache[key] = pg.forward(cfg, w, toks)
        out[rid] = _plain_cache[key]
    return out


def make_runner(folder, dtype, page, pool_tokens, max_requests=4):
    from paged_batch_engine_b200.engine.runner import ModelRunner
    return ModelRunner.from_folder(folder, dtype=dtype, device=DEV, page_tokens=page,
                                   max_cache_tokens=pool_tokens, max_requests=max_requests, poison=True)


def check(got, want, dtype, label):
    worst, where, scale = ru.max_error(got, want)
    tol = (TOL_F32_REL if dtype == "float32" else TOL_BF16_MAX) * max(scale, 1.0)
    rms_all = float(torch.cat([v.flatten() for v in want.values()]).pow(2).mean().sqrt())
    per_row = [float((row - want[rid][pos]).pow(2).mean().sqrt()) / rms_all for rid, rows in got.items()
               for pos, row in rows.items()]
    row_rms, mean_rms = max(per_row), sum(per_row) / len(per_row)
    print(f"\n[gebadra] {label} {dtype}: max|dlogit| = {worst:.3e} at {where}, max|logit| = {scale:.3f}, "
          f"tol = {tol:.3e}, row rms / logit rms: worst {row_rms:.3e}, mean {mean_rms:.3e}")
    assert worst <= tol, (label, dtype, worst, where, "first beyond tolerance:", ru.first_wrong(got, want, tol))
    if dtype != "float32":
        assert row_rms <= TOL_BF16_RMS and mean_rms <= TOL_BF16_RMS_MEAN, (label, row_rms, mean_rms)
    assert sum(len(v) for v in got.values()) == sum(v.shape[0] for v in want.values()), label


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_schedules_agree_with_plain(folders, name, dtype):
    cfg, _, page = GEBADRA[name]
    folder = folders[name]
    reqs = requests_for(name, cfg["vocab"])
    want = plain_logits(folder, reqs)
    schedules = {"whole": ru.whole(reqs), "tail": ru.tail_decoded(reqs, 40), "portions": ru.portions(reqs),
                 "mixed": ru.mixed(reqs, max_live=3, seed=5)}
    for label, recs in schedules.items():
        # the smallest pool the trace may be given and three request slots: pages and state rows
        # of finished requests are used again (the pool is poisoned with NaN at the start)
        runner = make_runner(folder, dtype, page, ru.pool_tokens_needed(recs), max_requests=3)
        got = ru.run_records(runner, recs)
        check(got, want, dtype, f"{name}/{label}")
        runner.cache.check_invariants()
        assert runner.cache.num_live_requests == 0
        for gi in range(len(runner.cache.groups)):
            assert runner.cache.num_free_pages(gi) == runner.cache.pools[gi].num_pages


def test_batch_of_unequal_requests_equals_each_alone_and_slots_are_used_again(folders):
    """Eight requests through two request slots, two at a time, against each alone: a state row
    or a page that kept something of its former owner would show."""
    cfg, _, page = GEBADRA["A"]
    folder = folders["A"]
    g = torch.Generator().manual_seed(1)
    reqs = {f"s{i}": torch.randint(0, cfg["vocab"], (n,), generator=g).tolist()
            for i, n in enumerate([50, 9, 33, 64, 2, 71, 18, 40])}
    want = plain_logits(folder, reqs)
    recs = ru.mixed(reqs, max_live=2, seed=9)
    runner = make_runner(folder, "float32", page, ru.pool_tokens_needed(recs), max_requests=2)
    check(ru.run_records(runner, recs), want, "float32", "A/two slots")
    assert runner.cache.state_slot_assignments == 8


@pytest.mark.parametrize("name", ["B", "C"])
def test_long_decoding_token_by_token(folders, name):
    """Every token decoded alone from the first on: the window and several pooled blocks pass
    over decoded tokens; in B the window is shorter than a block."""
    cfg, _, page = GEBADRA[name]
    g = torch.Generator().manual_seed(2)
    toks = torch.randint(0, cfg["vocab"], (140,), generator=g).tolist()
    want = plain_logits(folders[name], {"r": toks})
    recs = [{"step": i, "entries": [{"id": "r", "tokens": [t], "want": [0]}], "end": []} for i, t in enumerate(toks)]
    runner = make_runner(folders[name], "float32", page, 192)
    check(ru.run_records(runner, recs), want, "float32", f"{name}/all decoded")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_captured_decode_steps(folders, dtype):
    """Steps of single tokens through the captured decode step (a replayed CUDA graph), with
    request counts that leave padding rows (3 live in a step of 4, then fewer as they end)."""
    cfg, _, page = GEBADRA["A"]
    g = torch.Generator().manual_seed(6)
    reqs = {f"g{i}": torch.randint(0, cfg["vocab"], (n,), generator=g).tolist() for i, n in enumerate([70, 45, 58])}
    want = plain_logits(folders["A"], reqs)
    recs = ru.batch_decode(reqs, decode_tokens=30, prefill_group=3, portion=24)
    runner = make_runner(folders["A"], dtype, page, 256, max_requests=4)
    from paged_batch_engine_b200.engine.replay import TraceReplayer
    rp = TraceReplayer(runner, decode_graphs=True)
    got = ru.run_records(runner, recs, replayer=rp)
    assert rp.graph_steps >= 30
    check(got, want, dtype, "A/captured decode")


def test_greedy_generation_through_the_entry_point(folders):
    from paged_batch_engine_b200.engine.engine import Engine
    from paged_batch_engine_b200.sampling.params import SamplingParams
    cfg, _, page = GEBADRA["C"]
    c, w = load_plain(folders["C"])
    g = torch.Generator().manual_seed(3)
    prompts = [torch.randint(0, cfg["vocab"], (n,), generator=g).tolist() for n in (5, 37, 60)]
    eng = Engine(folders["C"], dtype="float32", device=DEV, page_size=page, num_pages=64, max_num_seqs=2,
                 max_num_batched_tokens=48, prefill_chunk_cap=24)
    res = eng.generate(prompts, SamplingParams(max_new_tokens=12, temperature=0.0, ignore_eos=True))
    for p, r in zip(prompts, res):
        toks = list(p)
        for _ in range(12):
            lg = pg.forward(c, w, toks)[-1]
            top2 = lg.topk(2).values
            nxt = int(lg.argmax())
            got = r.output_tokens[len(toks) - len(p)]
            if float(top2[0] - top2[1]) > 1e-4:
                assert got == nxt, (len(toks), got, nxt)
            toks.append(got)


def test_command_line_generates_greedily(folders):
    cfg, _, page = GEBADRA["B"]
    c, w = load_plain(folders["B"])
    prompt = [7, 100, 33, 2, 150, 9, 81, 64, 5, 199, 12]
    p = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "pbe-qwen"), folders["B"], "--prompt-ids",
                        ",".join(map(str, prompt)), "--max-new-tokens", "6", "--dtype", "float32", "--ignore-eos",
                        "--page-size", str(page), "--kv-cache-blocks-per-layer", "32", "--max-num-seqs", "2"],
                       capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, p.stderr[-2000:]
    line = [json.loads(l) for l in p.stdout.splitlines() if l.startswith("{")][0]
    toks = list(prompt)
    for got in line["output_ids"]:
        lg = pg.forward(c, w, toks)[-1]
        top2 = lg.topk(2).values
        if float(top2[0] - top2[1]) > 1e-4:
            assert got == int(lg.argmax()), (len(toks), got, int(lg.argmax()))
        toks.append(got)
    assert len(line["output_ids"]) == 6


@pytest.mark.parametrize("M, N, K", [(1, 70, 72), (5, 33, 40), (8, 250, 104), (20, 70, 72), (3, 66, 100)])
def test_projections_of_widths_that_divide_nothing(M, N, K):
    """The fused projections of a model with odd sizes: every route of the engine's product."""
    ops = _ops()
    g = torch.Generator().manual_seed(M * N)
    x, w = torch.randn(M, K, generator=g), torch.randn(N, K, generator=g)
    for dt, tol in ((torch.float32, 1e-4), (torch.bfloat16, 0.15)):
        y = ops.linear(x.to(DEV).to(dt), w.to(DEV).to(dt), None, out_dtype=dt).float().cpu()
        want = x.to(dt).double() @ w.to(dt).double().T
        assert float((y.double() - want).abs().max()) <= tol, (dt, M, N, K)


def test_trace_runner_program(folders, tmp_path):
    cfg, _, page = GEBADRA["A"]
    reqs = requests_for("A", cfg["vocab"])
    want = plain_logits(folders["A"], reqs)
    recs = ru.mixed(reqs, max_live=4, seed=2)
    out = tmp_path / "out"
    p = subprocess.run([os.path.join(ROOT, "bin", "trace_run"), "--model", folders["A"], "--dtype", "float32",
                        "--out", str(out), "--max-tokens", str(ru.pool_tokens_needed(recs))],
                       input="\n".join(json.dumps(r) for r in recs) + "\n", capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, p.stderr[-2000:]
    assert [l for l in p.stdout.splitlines() if l.startswith("done ")] == [f"done {r['step']}" for r in recs]
    progress, worst = {}, 0.0
    for r in recs:
        rows = np.fromfile(out / f"{r['step']}.f32", dtype="<f4").reshape(-1, cfg["vocab"])
        i = 0
        for e in r["entries"]:
            base = progress.get(e["id"], 0)
            for wpos in e["want"]:
                worst = max(worst, float(np.abs(rows[i] - want[e["id"]][base + wpos].numpy()).max()))
                i += 1
            progress[e["id"]] = base + len(e["tokens"])
    assert worst <= TOL_F32_REL * max(1.0, max(float(v.abs().max()) for v in want.values()))
