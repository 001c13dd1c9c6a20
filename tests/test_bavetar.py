"""Bavetar without a GPU: the configuration reader, the model as data, what its mixers keep in the
cache, and the plain implementation's mechanisms against closed forms."""
import copy
import math

import pytest
import torch

from paged_batch_engine_b200.config import ConfigError, load_config
from paged_batch_engine_b200.engine.runner import build_model
from paged_batch_engine_b200.parts import CompositeNeed, PagedNeed, StateNeed
from tests.helpers import BAV_A, BAV_B, BAV_C
from tests.plain import plain_bavetar as pb


# ---------------------------------------------------------------- configuration
def test_architecture_and_constants_come_from_the_configuration():
    arch, cfg = load_config(BAV_A)
    assert arch.name == "Bavetar" and cfg.width == 64 and cfg.logit_scale == 0.7 and cfg.logit_softcap == 9.0
    _, b = load_config(BAV_B)
    assert b.logit_softcap is None and b.model_spec().logit_softcap is None and b.model_spec().logit_scale == 2.0


def test_model_as_data_names_and_shapes():
    _, cfg = load_config(BAV_A)
    spec = cfg.model_spec()
    assert [b.kind for b in spec.blocks] == ["parallel"] * 4 and spec.lm_head_name is None
    assert [b.mixer.kind for b in spec.blocks] == ["latent_attention", "selective_state_space"] * 2
    assert [b.feed_forward.kind if b.feed_forward else None for b in spec.blocks] == \
        ["activation_mlp", "routed_experts", None, "activation_mlp"]
    model = build_model(cfg, torch.float32, "cpu")
    names = {p.name: tuple(p.shape) for p in model.param_specs() if not p.optional}
    assert names["embed"] == (300, 64) and names["final.norm"] == (64,) and "head" not in names
    assert names["l0.mix.dq"] == (24, 64) and names["l0.mix.dq.norm"] == (24,) and names["l0.mix.uq"] == (72, 24)
    assert names["l0.mix.dkv"] == (48, 64) and names["l0.mix.dkv.norm"] == (40,)
    assert names["l0.mix.uk"] == (48, 40) and names["l0.mix.uv"] == (72, 40) and names["l0.mix.o"] == (64, 72)
    assert names["l0.mix.sink"] == (3,) and names["l0.mix.g"] == (3, 64)
    assert names["l0.mlp.up"] == (96, 64) and names["l0.mlp.down"] == (64, 96)
    assert names["l1.mix.in"] == (2 * 64 + 2 * 24 + 4, 64) and names["l1.mix.conv"] == (64 + 48, 4)
    assert names["l1.mix.conv.b"] == (112,) and names["l1.mix.A_log"] == (4,) and names["l1.mix.norm"] == (64,)
    assert names["l1.mlp.router"] == (6, 64) and names["l1.mlp.e5.gate"] == (48, 64) and names["l1.mlp.e0.down"] == (64, 48)
    assert not any(n.startswith("l2.mlp") or n.startswith("l2.norm2") for n in names)
    assert names["l3.mix.in"] == (2 * 80 + 2 * 2 * 80 + 2, 64)


def test_what_the_mixers_keep():
    model = build_model(load_config(BAV_C)[1], torch.float32, "cpu")
    lat, one_tap, four_taps = model.cache_needs
    assert isinstance(lat, PagedNeed) and [(t.name, t.heads, t.width) for t in lat.tensors] == [("latent", 1, 64)]
    assert lat.window is None and lat.stride == 1
    assert isinstance(one_tap, CompositeNeed) and dict(one_tap.parts) == {"ssm": StateNeed((8, 130, 8), torch.float32)}
    assert dict(four_taps.parts) == {"ssm": StateNeed((4, 32, 24), torch.float32),
                                     "conv": StateNeed((3, 96 + 2 * 4 * 32), torch.float32)}
    assert model.decode_capturable()


@pytest.mark.parametrize("path, value, word", [
    (("layers", 0, "type"), "mamba3", "unknown layer type"),
    (("layers", 0, "mixer", "rot_dim"), 7, "even"),
    (("layers", 0, "mixer", "rot", "dims"), 10, "at most rot_dim"),
    (("layers", 1, "mixer", "groups"), 3, "multiple of groups"),
    (("layers", 1, "mixer", "norm_groups"), 5, "norm_groups"),
    (("layers", 1, "mlp", "router", "top"), 7, "top"),
    (("layers", 0, "mlp", "kind"), "glu", "not supported"),
    (("norm", "eps"), 0.0, "positive"),
])
def test_configurations_that_cannot_run_are_refused(path, value, word):
    cfg = copy.deepcopy(BAV_A)
    d = cfg
    for key in path[:-1]:
        d = d[key]
    d[path[-1]] = value
    with pytest.raises(ConfigError, match=word):
        load_config(cfg)


def test_a_missing_key_is_named():
    cfg = copy.deepcopy(BAV_B)
    del cfg["layers"][1]["mixer"]["kv_rank"]
    with pytest.raises(ConfigError, match="kv_rank"):
        load_config(cfg)


# ---------------------------------------------------------------- the plain mechanisms against closed forms
def test_sink_takes_its_share_of_the_softmax():
    scores = torch.zeros(1, 1, 4, dtype=torch.float64)              # four equal scores of 0
    w = pb.sink_softmax_weights(scores, torch.tensor([math.log(4.0)], dtype=torch.float64))
    assert torch.allclose(w, torch.full((1, 1, 4), 1 / 8, dtype=torch.float64))       # the sink weighs as much as all four
    w = pb.sink_softmax_weights(scores, torch.tensor([-1e9], dtype=torch.float64))
    assert torch.allclose(w.sum(-1), torch.ones(1, 1, dtype=torch.float64))


def test_causal_convolution_uses_the_last_column_for_the_current_token():
    u = torch.arange(1.0, 6.0, dtype=torch.float64)[:, None]
    w = torch.tensor([[100.0, 10.0, 1.0]], dtype=torch.float64)
    y = pb.causal_conv(u, w, torch.tensor([0.5], dtype=torch.float64))
    assert y[:, 0].tolist() == [1.5, 12.5, 123.5, 234.5, 345.5]


def test_selective_scan_with_constant_inputs_is_a_geometric_sum():
    T, rate, dt = 6, 0.5, 0.3
    x = torch.ones(T, 1, 1, dtype=torch.float64)
    ones = torch.ones(T, 1, 1, dtype=torch.float64)
    y = pb.selective_scan(x, torch.full((T, 1), dt, dtype=torch.float64), torch.tensor([math.log(rate)], dtype=torch.float64),
                          ones, ones, torch.tensor([2.0], dtype=torch.float64))
    a = math.exp(-rate * dt)
    want = [dt * sum(a ** j for j in range(t + 1)) + 2.0 for t in range(T)]
    assert torch.allclose(y[:, 0, 0], torch.tensor(want, dtype=torch.float64))


def test_routing_keeps_to_the_best_groups_and_scales_the_weights():
    # scores: expert 5 is the best, its group (4, 5) is kept; the second-best group is (0, 1) through expert 0;
    # expert 2 scores above expert 1 but lies in a group that is not kept
    logits = torch.tensor([[2.0, 0.5, 1.5, 0.0, 0.1, 3.0]], dtype=torch.float64)
    r = dict(experts=6, top=3, scale=2.0, groups=dict(count=3, keep=2))
    picked, weights = pb.route(logits, torch.eye(6, dtype=torch.float64), r)
    assert sorted(picked[0].tolist()) == [0, 1, 5]
    s = torch.softmax(logits[0], 0)
    assert torch.allclose(weights.sum(), torch.tensor(2.0, dtype=torch.float64))
    assert torch.allclose(weights[0, picked[0].tolist().index(5)], 2.0 * s[5] / (s[0] + s[1] + s[5]))
    picked, _ = pb.route(logits, torch.eye(6, dtype=torch.float64), dict(experts=6, top=3, scale=1.0))
    assert sorted(picked[0].tolist()) == [0, 2, 5]


def test_rotation_turns_neighbouring_pairs_and_leaves_the_rest():
    x = torch.tensor([[[1.0, 0.0, 1.0, 0.0, 7.0, 9.0]]], dtype=torch.float64).repeat(2, 1, 1)
    y = pb.rotate_pairs(x, torch.tensor([0, 3]), 100.0, 4)
    assert torch.equal(y[0], x[0])
    f = [1.0, 100.0 ** -0.5]
    want = [math.cos(3 * f[0]), math.sin(3 * f[0]), math.cos(3 * f[1]), math.sin(3 * f[1]), 7.0, 9.0]
    assert torch.allclose(y[1, 0], torch.tensor(want, dtype=torch.float64))
