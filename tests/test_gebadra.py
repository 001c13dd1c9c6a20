"""Gebadra without a GPU: the configuration reader, the model as data, the cache manager's
groups of one entry per block of tokens, composite cache needs, and the plain implementation's
mechanisms against closed forms."""
import copy
import math

import pytest
import torch

from paged_batch_engine_b200.cache import CacheManager, KVGroupSpec
from paged_batch_engine_b200.config import ConfigError, load_config
from paged_batch_engine_b200.engine.runner import build_model
from tests.helpers import GEB_A, GEB_B, GEB_C
from tests.plain import plain_gebadra as pg


# ---------------------------------------------------------------- configuration
def test_architecture_is_chosen_by_its_name_in_one_string():
    arch, cfg = load_config(GEB_A)
    assert arch.name == "Gebadra" and cfg.streams == 3 and cfg.width == 64


def test_model_as_data_run_order_and_shared_tensors():
    _, cfg = load_config(GEB_A)
    spec = cfg.model_spec()
    assert len(spec.blocks) == 2 and [s.block for s in spec.run_order] == [0, 1, 0, 1]
    assert [s.cache_layer for s in spec.run_order] == [0, 1, 2, 3]      # a cache and state of its own each
    assert spec.residual_streams == 3
    model = build_model(cfg, torch.float32, "cpu")
    names = {p.name: tuple(p.shape) for p in model.param_specs() if not p.optional}
    assert names["l0.mix.q"] == (32, 64) and names["l0.mix.v"] == (48, 64) and names["l0.mix.norm"] == (48,)
    assert names["l1.mix.left.q"] == (128, 64) and names["l1.mix.left.k"] == (32, 64)
    assert names["l1.mix.left.v"] == (16, 64) and names["l1.mix.left.o"] == (64, 64)
    assert names["l1.mix.left.q.norm"] == (128,) and names["l1.mix.left.talk"] == (4, 4)
    assert names["l1.mix.right.g"] == (64, 64) and names["l1.mix.left.out"] == (64,)
    assert names["l0.hc1.mix"] == (3, 3) and names["l1.hc2.in"] == (3,)
    assert names["l0.norm1"] == (64,) and names["l0.norm1.b"] == (64,) and names["final.norm.b"] == (64,)
    assert names["embed"] == (300, 64) and names["head"] == (300, 64)
    assert not any(n.startswith("l2.") or n.startswith("l3.") for n in names)


def test_a_layer_may_name_a_layer_that_names_another():
    cfg = copy.deepcopy(GEB_A)
    cfg["layers"].append(dict(cfg["layers"][2], weights_of=2))
    _, typed = load_config(cfg)
    spec = typed.model_spec()
    assert [s.block for s in spec.run_order] == [0, 1, 0, 1, 0] and len(spec.blocks) == 2


def test_no_streams_key_means_no_connection_tensors_and_null_mlp_no_feed_forward():
    _, cfg = load_config(GEB_B)
    model = build_model(cfg, torch.float32, "cpu")
    names = {p.name for p in model.param_specs() if not p.optional}
    assert not any(".hc" in n for n in names)
    assert not any(n.startswith("l1.mlp") or n.startswith("l1.norm2") for n in names)
    assert "l0.mlp.gate" in names and "l0.norm2.b" in names
    assert model.spec.residual_streams == 1


def test_one_stream_given_still_has_its_tensors():
    _, cfg = load_config(GEB_C)
    names = {p.name: tuple(p.shape) for p in build_model(cfg, torch.float32, "cpu").param_specs()}
    assert names["l0.hc1.mix"] == (1, 1) and names["l1.hc2.out"] == (1,)


@pytest.mark.parametrize("edit, message", [
    (lambda c: c["layers"][0].__setitem__("type", "conv"), "unknown layer type"),
    (lambda c: c["layers"][0]["mixer"].__setitem__("decay", [0.5]), "one decay per head"),
    (lambda c: c["layers"][1]["mixer"]["left"].__setitem__("kv_heads", 3), "multiple of kv_heads"),
    (lambda c: c["layers"][2].__setitem__("weights_of", 1), "another type"),
    (lambda c: c["layers"][3].__setitem__("weights_of", 3), "tensors of its own"),
    (lambda c: c["layers"][1].__setitem__("weights_of", 3), "tensors of its own"),
    (lambda c: c["layers"][1]["mlp"].__setitem__("kind", "routed"), "not supported"),
    (lambda c: c.pop("width"), "lacks 'width'"),
    (lambda c: c.__setitem__("streams", 0), "streams"),
])
def test_bad_configurations_are_refused(edit, message):
    cfg = copy.deepcopy(GEB_A)
    edit(cfg)
    with pytest.raises(ConfigError, match=message):
        load_config(cfg)


def test_cache_needs_of_the_layers():
    from paged_batch_engine_b200.parts import CompositeNeed, PagedNeed, StateNeed
    _, cfg = load_config(GEB_B)
    model = build_model(cfg, torch.float32, "cpu")
    par, lin = model.cache_needs
    assert isinstance(lin, StateNeed) and lin.shape == (1, 48, 64)
    assert isinstance(par, CompositeNeed)
    left = dict(dict(par.parts)["left"].parts)
    # the window (7) is shorter than a block (8): tokens are kept until their block is pooled
    assert isinstance(left["tokens"], PagedNeed) and left["tokens"].window == 8 and left["tokens"].stride == 1
    assert left["pooled"].window is None and left["pooled"].stride == 8
    assert [(t.heads, t.width) for t in left["tokens"].tensors] == [(3, 24), (3, 40)]
    assert dict(par.parts)["right"].shape == (3, 40, 8)


# ---------------------------------------------------------------- cache manager: one entry per block
def test_group_with_one_entry_per_block_of_tokens():
    groups = [KVGroupSpec((0,), 1, 8, window=6), KVGroupSpec((1,), 1, 8, window=None, stride=4)]
    m = CacheManager(groups, page_tokens=2, num_pages=[40, 6], max_requests=3)
    h = m.add_request()
    assert m.pages_needed(h, 9) == [5, 2]            # 9 tokens: 5 token pages; 3 entries: 2 pages
    assert m.reserve(h, 9)
    assert len(m.block_table(h, 1)) == 2
    m.commit(h, 9)
    assert m.slot_of_token(h, 1, 8) == m.block_table(h, 1)[1] * 2 + 0      # token 8 -> entry 2 -> page 1, offset 0
    assert m.slot_of_token(h, 1, 7) == m.block_table(h, 1)[0] * 2 + 1
    # the windowed group gave back what lies before token 9 - 6 + 1 = 4, the other group nothing
    assert m.block_table(h, 0)[:2] == [-1, -1] and m.block_table(h, 0)[2] >= 0
    assert all(p >= 0 for p in m.block_table(h, 1))
    assert m.reserve(h, 8) and len(m.block_table(h, 1)) == 3               # 17 tokens: 5 entries: 3 pages
    m.check_invariants()
    h2 = m.add_request()
    assert m.reserve(h2, 20) and not m.reserve(h2, 5)                      # 25 tokens need 4 pages, 3 are left
    m.check_invariants()
    m.free(h)
    assert m.reserve(h2, 5)                                                # pages of the first request again
    m.truncate(h2, 3)
    assert len(m.block_table(h2, 1)) == 1 and len(m.block_table(h2, 0)) == 2
    m.free(h2)
    m.check_invariants()
    assert m.num_free_pages(0) == 40 and m.num_free_pages(1) == 6


def test_composite_needs_become_pools_and_state_rows():
    from paged_batch_engine_b200.cache.storage import CacheStorage
    _, cfg = load_config(GEB_A)
    model = build_model(cfg, torch.float32, "cpu")
    st = CacheStorage(model.cache_needs, page_tokens=8, num_pages=10, max_requests=3, dtype=torch.float32,
                      device="cpu")
    # the two parallel layers share a token pool and a pool of pooled entries
    assert len(st.groups) == 2 and sorted(g.stride for g in st.groups) == [1, 4]
    pooled = [g for g in st.groups if g.stride == 4][0]
    assert len(pooled.layers) == 2
    assert st.manager.pools[st.groups.index(pooled)].num_pages == 3 + 3    # ceil(10 / 4) and a page a request
    lc = st.layer(1)
    left = lc.sub["left"]
    assert left.sub["tokens"].k.shape == (10, 1, 8, 32) and left.sub["tokens"].v.shape == (10, 1, 8, 16)
    assert left.sub["pooled"].k.shape == (6, 1, 8, 32)
    assert lc.sub["right"].state.shape == (4, 2, 16, 32)
    assert st.layer(0).state.shape == (4, 2, 16, 24)
    assert st.layer(3).sub["left"].sub["tokens"].k.data_ptr() != left.sub["tokens"].k.data_ptr()
    assert len(st.state) == 4          # a state per run of a layer, also for layers that share tensors


# ---------------------------------------------------------------- the plain mechanisms
def test_plain_recurrence_equals_the_sum_over_the_past():
    torch.manual_seed(0)
    T, H, d, e = 9, 2, 3, 4
    q, k, v = torch.randn(T, H, d, dtype=torch.float64), torch.randn(T, H, d, dtype=torch.float64), \
        torch.randn(T, H, e, dtype=torch.float64)
    decay = [0.5, 0.9]
    o = pg.decayed_linear_attention(q, k, v, decay)
    for t in range(T):
        for h in range(H):
            want = sum(decay[h] ** (t - j) * (q[t, h] @ k[j, h]) * v[j, h] for j in range(t + 1))
            assert torch.allclose(o[t, h], want, atol=1e-12)


def test_plain_visibility_rule():
    # window 5, blocks of 3: position 9 sees tokens 5..9; block 0 (0..2) since 2 <= 4; block 1 ends
    # at 5 > 4: its tokens 3 and 4 are not seen at all
    assert pg.visible_keys(9, 5, 3) == (1, 5)
    assert pg.visible_keys(4, 5, 3) == (0, 0)
    assert pg.visible_keys(7, 5, 3) == (1, 3)        # block 0 ends at 2 = 7 - 5
    assert pg.visible_keys(6, 5, 3) == (0, 2)
    assert pg.visible_keys(10, 5, 3) == (2, 6)


def test_plain_attention_is_ordinary_softmax_inside_the_window():
    torch.manual_seed(1)
    T, H, G, d, e = 6, 2, 1, 4, 3
    q, k, v = torch.randn(T, H, d), torch.randn(T, G, d), torch.randn(T, G, e)
    out = pg.pooled_window_attention(q, k, v, torch.eye(H), 0.5, window=100, pool=2)
    for t in range(T):
        for h in range(H):
            w = torch.softmax((k[:t + 1, 0] @ q[t, h]) * 0.5, dim=0)
            assert torch.allclose(out[t, h], w @ v[:t + 1, 0], atol=1e-6)
    # mixing: head 0 takes head 1's probabilities
    swap = torch.tensor([[0.0, 1.0], [1.0, 0.0]])
    mixed = pg.pooled_window_attention(q, k, v, swap, 0.5, window=100, pool=2)
    assert torch.allclose(mixed[:, 0], out[:, 1], atol=1e-6) and torch.allclose(mixed[:, 1], out[:, 0], atol=1e-6)


def test_plain_rotation_pairs_neighbours_and_leaves_the_rest():
    x = torch.arange(8, dtype=torch.float64).reshape(1, 1, 8) + 1
    y = pg.rotate_pairs(x, torch.tensor([3]), base=100.0, dims=4, factor=2.0)
    assert torch.equal(y[..., 4:], x[..., 4:])
    for i in range(2):
        a = 3 * 100.0 ** (-2 * i / 4) / 2.0
        u, v = x[0, 0, 2 * i], x[0, 0, 2 * i + 1]
        assert math.isclose(y[0, 0, 2 * i], u * math.cos(a) - v * math.sin(a), abs_tol=1e-12)
        assert math.isclose(y[0, 0, 2 * i + 1], v * math.cos(a) + u * math.sin(a), abs_tol=1e-12)


def test_plain_streams_with_identity_wiring_are_the_residual_sum(tmp_path):
    from tests.helpers import load_plain, make_gebadra_folder
    cfg = copy.deepcopy(GEB_C)
    folder = make_gebadra_folder(tmp_path / "m", cfg, 5)
    c, w = load_plain(folder)
    for k in list(w):
        if ".hc" in k:
            w[k] = torch.ones_like(w[k])
    toks = list(range(3, 30))
    a = pg.forward(c, w, toks)
    c2 = dict(c)
    c2.pop("streams")
    assert torch.allclose(a, pg.forward(c2, w, toks), atol=1e-5)
