"""Bavetar on the GPU against the plain implementation: every mechanism alone, then whole models
under every way of cutting and batching (whole, last tokens decoded, portions down to two tokens,
mixed batches with pages and state slots used again), long decoding, captured decode steps,
generation through the entry point, and the trace runner itself; float32 and bfloat16, three tiny
configurations."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

from tests import replay_util as ru
from tests.helpers import BAVETAR, load_plain, make_bavetar_folder
from tests.plain import plain_bavetar as pb

pytestmark = pytest.mark.gpu
ROOT = os.path.abspath(os.path.join(os.path.dirname(__file__), ".."))
DEV = "cuda:0"
TOL_F32_REL = 3e-5          # max |dlogit| over the largest logit: summation order only
# bfloat16: a row's root-mean-square difference over the root mean square of all logits.  A router
# may choose another expert for a token whose scores lie within the rounding of 16-bit activations
# (the float32 runs are the sharp test of every schedule), so a few rows may lie beyond the bound.
TOL_BF16_RMS_MEAN = 0.03
TOL_BF16_RMS = 0.12
BF16_ROWS_BEYOND = 0.03


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    return {name: make_bavetar_folder(tmp_path_factory.mktemp(f"bav_{name}"), cfg, seed)
            for name, (cfg, seed, _) in BAVETAR.items()}


def _ops():
    from paged_batch_engine_b200.csrc import ops
    return ops


def i32(a):
    return torch.tensor(a, dtype=torch.int32, device=DEV)


# ================================================================ mechanisms alone
@pytest.mark.parametrize("W, dt", [(64, torch.float32), (200, torch.bfloat16), (37, torch.float32)])
def test_two_norms_of_one_sum(W, dt):
    ops = _ops()
    g = torch.Generator().manual_seed(W)
    T = 6
    x = torch.randn(T, W, generator=g) * 3
    a, b = torch.randn(T, W, generator=g).to(dt), torch.randn(T, W, generator=g).to(dt)
    g1, g2 = torch.randn(W, generator=g), torch.randn(W, generator=g)
    total = x.double() + (a.double() + b.double())
    res = x.to(DEV)
    o1, o2 = ops.add2_rmsnorm2(res, a.to(DEV), b.to(DEV), g1.to(DEV), g2.to(DEV), 1e-5, torch.float32)
    assert torch.allclose(res.cpu().double(), total, atol=1e-5)
    assert torch.allclose(o1.cpu().double(), pb.rms_unit(total, 1e-5) * g1.double(), atol=3e-5, rtol=1e-5)
    assert torch.allclose(o2.cpu().double(), pb.rms_unit(total, 1e-5) * g2.double(), atol=3e-5, rtol=1e-5)
    # gathered rows leave the residual alone; one branch absent; one norm only
    res2 = x.to(DEV)
    rows = i32([4, 0, 4])
    o, none = ops.add2_rmsnorm2(res2, a.to(DEV), None, g1.to(DEV), None, 1e-5, torch.float32, rows)
    assert none is None and torch.equal(res2.cpu(), x)
    want = pb.rms_unit(x.double() + a.double(), 1e-5)[[4, 0, 4]] * g1.double()
    assert torch.allclose(o.cpu().double(), want, atol=3e-5, rtol=1e-5)


@pytest.mark.parametrize("taps, C, dt", [(4, 40, torch.float32), (2, 300, torch.bfloat16), (3, 7, torch.float32),
                                         (1, 33, torch.float32), (16, 20, torch.float32)])
def test_short_convolution_carries_its_last_inputs(taps, C, dt):
    """Unequal requests in one launch equal each alone; a request cut into launches of 1, 2 and
    more rows (fewer rows than taps too) equals it whole; a zeroed state row holds nothing of its
    former owner."""
    ops = _ops()
    g = torch.Generator().manual_seed(taps * 100 + C)
    lens = [11, 1, 25]
    T = sum(lens)
    wide = torch.randn(T, C + 9, generator=g).to(dt)
    w, b = torch.randn(C, taps, generator=g), torch.randn(C, generator=g)
    u = wide[:, 4:4 + C]
    want = torch.cat([pb.silu(pb.causal_conv(u[s:s + n].double(), w.double(), b.double()))
                      for s, n in zip([0, 11, 12], lens)])
    tol = 2e-5 if dt == torch.float32 else 3e-2
    dev = wide.to(DEV)[:, 4:4 + C]
    state = torch.full((5, taps - 1, C), float("nan"), device=DEV)
    slots = [3, 0, 4]
    state[slots] = 0
    rows = i32([0] * 11 + [1] + [2] * 25)
    got = ops.short_conv(dev, w.to(DEV), b.to(DEV), state, rows, i32([0, 11, 12]), i32(lens), i32(slots), 3,
                         weight_t=w.t().contiguous().to(DEV))
    assert torch.allclose(got.float().cpu().double(), want, atol=tol, rtol=tol)
    # the third request again, in pieces, in the row the first one used
    state[3] = 0
    outs, at = [], 12
    for n in [1, 2, 1, 7, 1, 1, 12]:
        outs.append(ops.short_conv(dev[at:at + n], w.to(DEV), b.to(DEV), state, i32([0] * n), i32([0]), i32([n]),
                                   i32([3]), 1))
        at += n
    assert torch.allclose(torch.cat(outs).float().cpu().double(), want[12:], atol=tol, rtol=tol)
    if taps > 1:       # both ways leave the same inputs behind
        assert torch.equal(state[3].cpu(), state[4].cpu())


def _scan_inputs(H, G, N, P, T, seed, dt=torch.float32):
    g = torch.Generator().manual_seed(seed)
    wide = (torch.randn(T, H * P + 2 * G * N + 3, generator=g)).to(dt)
    step = 0.05 + torch.rand(T, H, generator=g)
    a_log = torch.log(0.1 + 2 * torch.rand(H, generator=g))
    decay = torch.exp(-torch.exp(a_log) * step)
    skip = torch.randn(H, generator=g)
    return wide, step, a_log, decay, skip


def _scan_plain(wide, step, a_log, skip, H, G, N, P, rows):
    x = wide[rows].double()
    n = x.shape[0]
    return pb.selective_scan(x[:, :H * P].reshape(n, H, P), step[rows].double(), a_log.double(),
                             x[:, H * P:H * P + G * N].reshape(n, G, N),
                             x[:, H * P + G * N:H * P + 2 * G * N].reshape(n, G, N), skip.double()).reshape(n, H * P)


@pytest.mark.parametrize("H, G, N, P", [(4, 2, 16, 8), (6, 1, 40, 33), (3, 3, 130, 16), (2, 2, 24, 64), (8, 4, 300, 4)])
def test_selective_recurrence_state_groups_and_batches(H, G, N, P):
    ops = _ops()
    lens = [13, 1, 30]
    T = sum(lens)
    wide, step, a_log, decay, skip = _scan_inputs(H, G, N, P, T, H * 1000 + N)
    w = wide.to(DEV)
    xs, B, C = w[:, :H * P], w[:, H * P:H * P + G * N], w[:, H * P + G * N:H * P + 2 * G * N]
    run = lambda lo, hi, state, qs, ql, sl, R: ops.linear_attention(
        C[lo:hi], B[lo:hi], xs[lo:hi], state, None, i32(qs), i32(ql), i32(sl), R, H, tok_decay=decay[lo:hi].to(DEV).contiguous(),
        tok_scale=step[lo:hi].to(DEV).contiguous(), skip=skip.to(DEV), kq_share=H // G).cpu().double()
    state = torch.full((5, H, N, P), float("nan"), device=DEV)
    state[[3, 0, 4]] = 0
    got = run(0, T, state, [0, 13, 14], lens, [3, 0, 4], 3)
    for s, n in zip([0, 13, 14], lens):
        want = _scan_plain(wide, step, a_log, skip, H, G, N, P, slice(s, s + n))
        assert torch.allclose(got[s:s + n], want, atol=3e-4, rtol=3e-4), (s, n)
    # the third request cut in two launches, in a row that is used again
    state[3] = 0
    first = run(14, 14 + 11, state, [0], [11], [3], 1)
    second = run(14 + 11, T, state, [0], [19], [3], 1)
    want = _scan_plain(wide, step, a_log, skip, H, G, N, P, slice(14, T))
    assert torch.allclose(torch.cat([first, second]), want, atol=3e-4, rtol=3e-4)
    assert torch.allclose(state[3].cpu(), state[4].cpu(), atol=3e-4, rtol=3e-4)


@pytest.mark.parametrize("chunk", [64, 16, 5])
def test_selective_recurrence_in_chunks_side_by_side(chunk):
    from paged_batch_engine_b200.engine.batch import RecurrencePlan, recurrence_plan_arrays
    ops = _ops()
    H, G, N, P = 4, 2, 40, 24
    lens = [4 * chunk + 3, 2, 2 * chunk]
    starts = [0, lens[0], lens[0] + lens[1]]
    T = sum(lens)
    wide, step, a_log, decay, skip = _scan_inputs(H, G, N, P, T, chunk)
    w = wide.to(DEV)
    xs, B, C = w[:, :H * P], w[:, H * P:H * P + G * N], w[:, H * P + G * N:H * P + 2 * G * N]
    slots = [2, 0, 3]
    first, scan, second, entries = recurrence_plan_arrays(starts, lens, slots, chunk)
    assert entries == 5 + 2
    plan = RecurrencePlan(entries, i32(first), len(first), i32(scan), len(scan), i32(second), len(second))
    args = dict(tok_decay=decay.to(DEV), tok_scale=step.to(DEV), skip=skip.to(DEV), kq_share=H // G)
    state = torch.zeros(4, H, N, P, device=DEV)
    state[2] = torch.randn(H, N, P, generator=torch.Generator().manual_seed(1)).to(DEV)    # a request in progress
    ref = state.clone()
    got = ops.linear_attention(C, B, xs, state, None, i32(starts), i32(lens), i32(slots), 3, H, plan=plan, **args)
    seq = ops.linear_attention(C, B, xs, ref, None, i32(starts), i32(lens), i32(slots), 3, H, **args)
    assert torch.allclose(got.cpu(), seq.cpu(), atol=3e-4, rtol=3e-4)
    assert torch.allclose(state.cpu(), ref.cpu(), atol=3e-4, rtol=3e-4)
    want = _scan_plain(wide, step, a_log, skip, H, G, N, P, slice(starts[2], T))
    assert torch.allclose(got[starts[2]:].cpu().double(), want, atol=3e-4, rtol=3e-4)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_gate_inside_the_grouped_norm_and_step_sizes(dtype):
    ops = _ops()
    g = torch.Generator().manual_seed(5)
    T, parts, E = 5, 3, 20
    y = torch.randn(T, parts * E, generator=g) * 4
    wide = torch.randn(T, 50 + parts * E, generator=g).to(dtype)
    gain = torch.randn(parts * E, generator=g)
    got = ops.gated_rms(y.to(DEV), wide.to(DEV)[:, 50:], gain.to(DEV), parts, 1e-5, True, "silu", dtype, gate_first=True)
    want = pb.grouped_rms(y.double() * pb.silu(wide[:, 50:].double()), parts, gain.double(), 1e-5)
    tol = 1e-5 if dtype == torch.float32 else 2e-2
    assert torch.allclose(got.float().cpu().double(), want, atol=tol, rtol=tol)
    H = 7
    bias, a_log = torch.randn(H, generator=g), torch.randn(H, generator=g)
    u = (torch.randn(T, H + 3, generator=g) * 8).to(dtype)          # large values: the softplus is not clamped
    dt, decay = ops.step_sizes(u.to(DEV)[:, 3:], bias.to(DEV), a_log.to(DEV))
    want_dt = pb.softplus(u[:, 3:].double() + bias.double())
    assert torch.allclose(dt.cpu().double(), want_dt, atol=1e-5, rtol=1e-5)
    assert torch.allclose(decay.cpu().double(), torch.exp(-torch.exp(a_log.double()) * want_dt), atol=1e-6, rtol=1e-5)


@pytest.mark.parametrize("E, top, count, keep", [(6, 2, 1, 1), (15, 3, 3, 2), (10, 3, 5, 2), (8, 1, 4, 1), (40, 6, 8, 3),
                                                 (130, 8, 1, 1), (9, 4, 3, 2)])
def test_router_groups_and_weights(E, top, count, keep):
    ops = _ops()
    g = torch.Generator().manual_seed(E * 10 + top)
    logits = torch.randn(50, E, generator=g) * 3
    r = dict(experts=E, top=top, scale=1.7, groups=dict(count=count, keep=keep))
    picked, weights = pb.route(logits.double(), torch.eye(E, dtype=torch.float64), r)
    chosen, w = ops.route(logits.to(DEV), top, count, keep, 1.7)
    chosen, w = chosen.cpu().long(), w.cpu().double()
    order_got, order_want = chosen.sort(dim=1), picked.sort(dim=1)
    assert torch.equal(order_got.values, order_want.values)
    assert torch.allclose(w.gather(1, order_got.indices), weights.gather(1, order_want.indices), atol=1e-6, rtol=1e-5)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("W, F, E, top", [(64, 48, 6, 2), (100, 24, 9, 4), (40, 130, 3, 1)])
def test_expert_rows_and_rows_sorted_by_expert(W, F, E, top, dtype):
    from paged_batch_engine_b200.parts import RoutedExperts
    g = torch.Generator().manual_seed(W + F)
    T = 70
    part = RoutedExperts(W, F, E, top, dtype, DEV, groups=1, scale=1.3, many_rows=1 << 30)
    w = {"p.router": torch.randn(E, W, generator=g)}
    for e in range(E):
        w[f"p.e{e}.gate"], w[f"p.e{e}.up"] = torch.randn(F, W, generator=g) * 0.3, torch.randn(F, W, generator=g) * 0.3
        w[f"p.e{e}.down"] = torch.randn(W, F, generator=g) * 0.3
    w = {k: v.to(dtype) for k, v in w.items()}
    part.load({k: v.to(DEV) for k, v in w.items()}, "p.")
    x = torch.randn(T, W, generator=g).to(dtype)
    want = pb.routed_ff(x.double(), {k: v.double() for k, v in w.items()}, "p.",
                        dict(router=dict(experts=E, top=top, scale=1.3)))
    part.MANY_ROWS_TILED = 1 << 30                 # every row streams its experts' matrices
    by_rows = part.forward(x.to(DEV), None).float().cpu().double()
    part.many_rows = part.MANY_ROWS_TILED = 1      # rows sorted by expert (bfloat16: the tiled products)
    by_expert = part.forward(x.to(DEV), None).float().cpu().double()
    tol = 3e-5 if dtype == torch.float32 else 6e-2
    scale = float(want.abs().max())
    # a row whose router scores lie within 16-bit rounding may choose otherwise: compare the rest
    ok = lambda got: ((got - want).abs().max(dim=1).values <= tol * scale)
    assert ok(by_rows).float().mean() >= (1.0 if dtype == torch.float32 else 0.95)
    assert ok(by_expert).float().mean() >= (1.0 if dtype == torch.float32 else 0.95)
    assert float((by_rows - by_expert).abs().max()) <= (tol if dtype == torch.float32 else 4e-2) * scale


def _latent_part(H, D, R, rot_dims, V, rank, q_rank, hidden, dtype, seed, sink):
    """The latent attention part with random weights made so that every query looks along one
    direction of the part of the shared key that does not turn, and the weights it was given."""
    from paged_batch_engine_b200.parts import LatentAttention
    g = torch.Generator().manual_seed(seed)
    m = dict(heads=H, dim=D, rot_dim=R, vdim=V, kv_rank=rank, q_rank=q_rank, scale=0.3,
             rot=dict(base=300.0, dims=rot_dims))
    part = LatentAttention(hidden, H, D, R, V, rank, q_rank, 0.3, 1e-5, dtype, DEV, rotary=m["rot"])
    rnd = lambda *s: torch.randn(*s, generator=g)
    w = {"p.dq": rnd(q_rank, hidden) * 0.2, "p.dq.norm": 1 + 0.2 * rnd(q_rank), "p.uq": rnd(H * (D + R), q_rank) * 0.3,
         "p.dkv": rnd(rank + R, hidden) * 0.2, "p.dkv.norm": 1 + 0.2 * rnd(rank), "p.uk": rnd(H * D, rank) * 0.3,
         "p.uv": rnd(H * V, rank) * 0.3, "p.sink": sink.clone(), "p.g": rnd(H, hidden), "p.o": rnd(hidden, H * V) * 0.3}
    # input column 0 is a constant that dominates the query latent's first value, which every head's
    # last rotated-part value reads; input column 1 goes straight into the shared key's last value
    w["p.dq"][0] = 0
    w["p.dq"][0, 0] = 4.0
    w["p.uq"].view(H, D + R, q_rank)[:, D + R - 1, :] = 0
    w["p.uq"].view(H, D + R, q_rank)[:, D + R - 1, 0] = 3.0
    w["p.dkv"][rank + R - 1] = 0
    w["p.dkv"][rank + R - 1, 1] = 1.0
    w["p.dkv"][:, 0] = 0
    w = {k: v.to(dtype if v.dim() == 2 else torch.float32) for k, v in w.items()}
    part.load({k: v.to(DEV) for k, v in w.items()}, "p.")
    return part, m, {k: v.double() for k, v in w.items()}


def _run_part(part, x, cuts, page, num_pages, dtype):
    """Feeds rows x of one request through the part in portions of the given sizes."""
    from paged_batch_engine_b200.cache.storage import CacheStorage
    from paged_batch_engine_b200.engine.batch import StepContext, StepEntry
    st = CacheStorage([part.cache_need()], page, num_pages, 2, dtype, DEV, poison=True)
    keys = [(st.layer(0).group,) + k for k in part.work_keys()]
    h = st.manager.add_request()
    outs, i = [], 0
    for n in cuts:
        assert st.manager.reserve(h, n)
        ctx = StepContext(st.manager, [StepEntry(h, [0] * n, [])], torch.device(DEV), keys)
        outs.append(part.forward(x[i:i + n].to(DEV).to(dtype), ctx, st.layer(0)).float().cpu())
        st.manager.commit(h, n)
        i += n
    st.manager.check_invariants()
    return torch.cat(outs)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H, D, R, rot_dims, V, rank, q_rank, page, T", [
    (3, 16, 8, 4, 24, 40, 24, 8, 75), (20, 8, 4, 2, 8, 20, 16, 16, 90), (8, 32, 16, 8, 56, 48, 40, 16, 1100),
    (1, 24, 6, 4, 10, 33, 7, 4, 50)])
def test_latent_attention_with_a_stand_out_key_and_a_sink(H, D, R, rot_dims, V, rank, q_rank, page, T, dtype):
    """One key that every query scores far above all others, placed in turn where a fault would
    show: the first tokens, a page's edges, far back among hundreds (where the keys are split over
    blocks), next to the query; as a prompt portion and then token by token.  The sinks weigh from
    nothing to more than all keys together."""
    hidden = 48
    sink = torch.linspace(-6.0, 9.0, H)
    part, m, w = _latent_part(H, D, R, rot_dims, V, rank, q_rank, hidden, dtype, T + H, sink)
    g = torch.Generator().manual_seed(T)
    # 511, 512: where the keys of a long request are split over blocks
    marks = sorted({0, 1, page - 1, page, 2 * page - 1, 511, 512, T // 2, T - 20, T - 2} & set(range(T)))
    for mark in marks[:: (1 if dtype == torch.float32 and T < 500 else 3)]:
        x = torch.randn(T, hidden, generator=g) * 0.5
        x[:, 0] = 3.0                      # every query looks along the key's last value
        x[:, 1] = 0.1 * torch.randn(T, generator=g)
        x[mark, 1] = 25.0                  # the stand-out key
        x[mark, 2:] = 2.0                  # and a latent (so a value) that shows
        xs = x.to(dtype).double()
        want = pb.latent_attention_mixer(xs, w, "p.", m, 1e-5)
        head = T - 12
        cuts = ([head] if T < 500 else [500, head - 500]) + [1] * (T - head)
        got = _run_part(part, x, cuts, page, (T + page - 1) // page + 1, dtype).double()
        tol = (3e-5 if dtype == torch.float32 else 4e-2) * float(want.abs().max())
        err = (got - want).abs().max(dim=1).values
        assert float(err.max()) <= tol, (mark, int(err.argmax()), float(err.max()), tol)


def test_latent_attention_in_portions_of_two_and_other_requests_beside():
    """Rotation at positions far from the start of a portion, portions of two tokens, and two
    requests of unequal length in one step against each alone."""
    from paged_batch_engine_b200.cache.storage import CacheStorage
    from paged_batch_engine_b200.engine.batch import StepContext, StepEntry
    H, D, R, V, rank, q_rank, hidden, page = 5, 12, 8, 20, 28, 18, 40, 8
    part, m, w = _latent_part(H, D, R, 8, V, rank, q_rank, hidden, torch.float32, 3, torch.randn(H))
    g = torch.Generator().manual_seed(9)
    xa, xb = torch.randn(61, hidden, generator=g), torch.randn(30, hidden, generator=g)
    want_a = pb.latent_attention_mixer(xa.double(), w, "p.", m, 1e-5)
    want_b = pb.latent_attention_mixer(xb.double(), w, "p.", m, 1e-5)
    got = _run_part(part, xa, [2] * 20 + [7, 2, 3, 2, 5, 2], page, 12, torch.float32).double()
    assert float((got - want_a).abs().max()) <= 3e-5 * float(want_a.abs().max())
    st = CacheStorage([part.cache_need()], page, 16, 2, torch.float32, DEV, poison=True)
    keys = [(st.layer(0).group,) + k for k in part.work_keys()]
    ha, hb = st.manager.add_request(), st.manager.add_request()
    done = {ha: 0, hb: 0}
    outs = {ha: [], hb: []}
    for na, nb in [(40, 1), (1, 17), (20, 12)]:
        entries, rows = [], []
        for h, n, x in ((ha, na, xa), (hb, nb, xb)):
            assert st.manager.reserve(h, n)
            entries.append(StepEntry(h, [0] * n, []))
            rows.append(x[done[h]:done[h] + n])
        ctx = StepContext(st.manager, entries, torch.device(DEV), keys)
        y = part.forward(torch.cat(rows).to(DEV), ctx, st.layer(0)).cpu()
        outs[ha].append(y[:na]); outs[hb].append(y[na:])
        for h, n in ((ha, na), (hb, nb)):
            st.manager.commit(h, n)
            done[h] += n
    assert float((torch.cat(outs[ha]).double() - want_a).abs().max()) <= 3e-5 * float(want_a.abs().max())
    assert float((torch.cat(outs[hb]).double() - want_b).abs().max()) <= 3e-5 * float(want_b.abs().max())


# ================================================================ whole models
LENGTHS = {"A": [3, 41, 97, 150], "B": [1, 30, 75, 131], "C": [2, 52, 110, 171]}


def requests_for(name, vocab):
    g = torch.Generator().manual_seed(sum(map(ord, name)) + 177)
    return {f"{name}{i}": torch.randint(0, vocab, (n,), generator=g).tolist() for i, n in enumerate(LENGTHS[name])}


_plain_cache = {}


def plain_logits(folder, reqs):
    cfg, w = load_plain(folder)
    out = {}
    for rid, toks in reqs.items():
        key = (folder, tuple(toks))
        if key not in _plain_cache:
            _plain_cache[key] = pb.forward(cfg, w, toks).float()
        out[rid] = _plain_cache[key]
    return out


def make_runner(folder, dtype, page, pool_tokens, max_requests=4):
    from paged_batch_engine_b200.engine.runner import ModelRunner
    return ModelRunner.from_folder(folder, dtype=dtype, device=DEV, page_tokens=page,
                                   max_cache_tokens=pool_tokens, max_requests=max_requests, poison=True)


def check(got, want, dtype, label):
    worst, where, scale = ru.max_error(got, want)
    rms_all = float(torch.cat([v.flatten() for v in want.values()]).pow(2).mean().sqrt())
    per_row = sorted(float((row - want[rid][pos]).pow(2).mean().sqrt()) / rms_all for rid, rows in got.items()
                     for pos, row in rows.items())
    print(f"\n[bavetar] {label} {dtype}: max|dlogit| = {worst:.3e} at {where}, max|logit| = {scale:.3f}, "
          f"row rms / logit rms: worst {per_row[-1]:.3e}, mean {sum(per_row) / len(per_row):.3e}")
    assert sum(len(v) for v in got.values()) == sum(v.shape[0] for v in want.values()), label
    if dtype == "float32":
        tol = TOL_F32_REL * max(scale, 1.0)
        assert worst <= tol, (label, worst, where, "first beyond tolerance:", ru.first_wrong(got, want, tol))
        return
    beyond = sum(1 for e in per_row if not e <= TOL_BF16_RMS)
    assert beyond <= max(1, int(BF16_ROWS_BEYOND * len(per_row))), (label, beyond, len(per_row), per_row[-5:])
    kept = per_row[:len(per_row) - beyond]
    assert sum(kept) / len(kept) <= TOL_BF16_RMS_MEAN, (label, sum(kept) / len(kept))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_schedules_agree_with_plain(folders, name, dtype):
    cfg, _, page = BAVETAR[name]
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


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("which", ["state", "latent"])
def test_models_of_one_kind_of_layer(tmp_path, which, dtype):
    """A model with state rows and no paged cache at all, and one with pages and no state row."""
    from tests.helpers import BAV_LATENT_ONLY, BAV_STATE_ONLY
    cfg = BAV_STATE_ONLY if which == "state" else BAV_LATENT_ONLY
    folder = make_bavetar_folder(tmp_path / which, cfg, 31)
    g = torch.Generator().manual_seed(4)
    reqs = {f"q{i}": torch.randint(0, cfg["vocab"], (n,), generator=g).tolist() for i, n in enumerate([37, 5, 70])}
    want = plain_logits(folder, reqs)
    for label, recs in (("tail", ru.tail_decoded(reqs, 20)), ("mixed", ru.mixed(reqs, max_live=2, seed=3))):
        runner = make_runner(folder, dtype, 8, ru.pool_tokens_needed(recs), max_requests=2)
        check(ru.run_records(runner, recs), want, dtype, f"{which}/{label}")


def test_batch_of_unequal_requests_equals_each_alone_and_slots_are_used_again(folders):
    """Eight requests through two request slots, two at a time, against each alone: a state row
    or a page that kept something of its former owner would show."""
    cfg, _, page = BAVETAR["A"]
    folder = folders["A"]
    g = torch.Generator().manual_seed(1)
    reqs = {f"s{i}": torch.randint(0, cfg["vocab"], (n,), generator=g).tolist()
            for i, n in enumerate([50, 9, 33, 64, 2, 71, 18, 40])}
    want = plain_logits(folder, reqs)
    recs = ru.mixed(reqs, max_live=2, seed=9)
    runner = make_runner(folder, "float32", page, ru.pool_tokens_needed(recs), max_requests=2)
    check(ru.run_records(runner, recs), want, "float32", "A/two slots")
    assert runner.cache.state_slot_assignments == 8


def test_many_rows_take_the_experts_sorted_path(folders):
    """A prompt long enough that its routed feed-forward sorts the rows by expert, whole and cut
    so that one portion is below that size."""
    cfg, _, page = BAVETAR["C"]
    g = torch.Generator().manual_seed(12)
    toks = torch.randint(0, cfg["vocab"], (300,), generator=g).tolist()
    want = plain_logits(folders["C"], {"r": toks})
    for cuts in ([300], [200, 37, 63]):
        recs, at = [], 0
        for i, n in enumerate(cuts):
            recs.append({"step": i, "entries": [{"id": "r", "tokens": toks[at:at + n], "want": list(range(n))}], "end": []})
            at += n
        runner = make_runner(folders["C"], "float32", page, 320)
        check(ru.run_records(runner, recs), want, "float32", f"C/{cuts}")


@pytest.mark.parametrize("name", ["A", "B"])
def test_long_decoding_token_by_token(folders, name):
    """Every token decoded alone from the first on: the convolution starts from its zeros, the
    states and the cache grow a token at a time over many pages."""
    cfg, _, page = BAVETAR[name]
    g = torch.Generator().manual_seed(2)
    toks = torch.randint(0, cfg["vocab"], (140,), generator=g).tolist()
    want = plain_logits(folders[name], {"r": toks})
    recs = [{"step": i, "entries": [{"id": "r", "tokens": [t], "want": [0]}], "end": []} for i, t in enumerate(toks)]
    runner = make_runner(folders[name], "float32", page, 192)
    check(ru.run_records(runner, recs), want, "float32", f"{name}/all decoded")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B"])
def test_captured_decode_steps(folders, name, dtype):
    """Steps of single tokens through the captured decode step (a replayed CUDA graph), with
    request counts that leave padding rows (3 live in a step of 4, then fewer as they end)."""
    cfg, _, page = BAVETAR[name]
    g = torch.Generator().manual_seed(6)
    reqs = {f"g{i}": torch.randint(0, cfg["vocab"], (n,), generator=g).tolist() for i, n in enumerate([70, 45, 58])}
    want = plain_logits(folders[name], reqs)
    recs = ru.batch_decode(reqs, decode_tokens=30, prefill_group=3, portion=24)
    runner = make_runner(folders[name], dtype, page, 256, max_requests=4)
    from paged_batch_engine_b200.engine.replay import TraceReplayer
    rp = TraceReplayer(runner, decode_graphs=True)
    got = ru.run_records(runner, recs, replayer=rp)
    assert rp.graph_steps >= 30
    check(got, want, dtype, f"{name}/captured decode")


def test_greedy_generation_through_the_entry_point(folders):
    from paged_batch_engine_b200.engine.engine import Engine
    from paged_batch_engine_b200.sampling.params import SamplingParams
    cfg, _, page = BAVETAR["C"]
    c, w = load_plain(folders["C"])
    g = torch.Generator().manual_seed(3)
    prompts = [torch.randint(0, cfg["vocab"], (n,), generator=g).tolist() for n in (5, 37, 60)]
    eng = Engine(folders["C"], dtype="float32", device=DEV, page_size=page, num_pages=64, max_num_seqs=2,
                 max_num_batched_tokens=48, prefill_chunk_cap=24)
    res = eng.generate(prompts, SamplingParams(max_new_tokens=12, temperature=0.0, ignore_eos=True))
    for p, r in zip(prompts, res):
        toks = list(p)
        for _ in range(12):
            lg = pb.forward(c, w, toks)[-1]
            top2 = lg.topk(2).values
            nxt = int(lg.argmax())
            got = r.output_tokens[len(toks) - len(p)]
            if float(top2[0] - top2[1]) > 1e-4:
                assert got == nxt, (len(toks), got, nxt)
            toks.append(got)


def test_command_line_generates_greedily(folders):
    cfg, _, page = BAVETAR["B"]
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
        lg = pb.forward(c, w, toks)[-1]
        top2 = lg.topk(2).values
        if float(top2[0] - top2[1]) > 1e-4:
            assert got == int(lg.argmax()), (len(toks), got, int(lg.argmax()))
        toks.append(got)
    assert len(line["output_ids"]) == 6


def test_trace_runner_program(folders, tmp_path):
    cfg, _, page = BAVETAR["A"]
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
