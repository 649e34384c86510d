"""Host-side parts of the Tonilix integration (no GPU): the configuration reader, sizes of caches and state, the family
registry, and sanity of the plain oracle the GPU tests compare against (cases worked out by hand)."""
import json
import math

import pytest
import torch

import tonilix_ref as R
import tonilix_util as U
from b200attn.model import ARCHITECTURES, resolve_config
from b200attn.tonilix import DeltaSpec, DenseSpec, ExpertsSpec, ParallelSpec, TonilixConfig, config_from_dict

F64 = torch.float64


# ------------------------------------------------------------------------------------------------ configuration
def test_config_reads_every_size():
    c = config_from_dict(U.strip(U.cfg_a()))
    assert (c.vocab, c.hidden, c.groups, c.eps, c.layers) == (97, 64, 2, 1e-5, 4)
    d = c.layer_specs[0].mixer
    assert isinstance(d, DeltaSpec) and (d.heads, d.kv_heads, d.dim, d.vdim, d.taps) == (4, 2, 16, 24, 3)
    f = c.layer_specs[0].mlp
    assert isinstance(f, ExpertsSpec) and (f.experts, f.top, f.ff, f.groups, f.keep, f.scale) == (6, 2, 40, 3, 2, 1.7)
    p = c.layer_specs[1].mixer
    assert isinstance(p, ParallelSpec) and (p.left_scale, p.right_scale) == (0.7, 1.4)
    assert (p.left.heads, p.left.kv_heads, p.left.dim, p.left.vdim, p.left.scale, p.left.temp_coef, p.left.temp_every) == \
        (4, 1, 24, 16, 0.3, 0.8, 7)
    assert (p.right.heads, p.right.dim, p.right.vdim, p.right.tau) == (2, 16, 8, 4.0)
    assert c.layer_specs[1].mlp is None and isinstance(c.layer_specs[2].mlp, DenseSpec) and c.layer_specs[2].mlp.ff == 72
    g = c.layer_specs[3].mlp
    assert (g.groups, g.keep) == (1, 1)                           # no groups in the file: one group, kept


def test_low_rank_sizes_come_from_the_checkpoint(tmp_path):
    cfg = U.cfg_a()
    W = R.random_model(cfg, seed=3)
    U.save_checkpoint(tmp_path, U.strip(cfg), W)
    c = resolve_config(str(tmp_path))
    assert isinstance(c, TonilixConfig) and "Tonilix" in ARCHITECTURES
    assert (c.layer_specs[0].mixer.decay_rank, c.layer_specs[0].mixer.gate_rank) == (5, 12)
    assert c.layer_specs[1].mixer.right.decay_rank == 6 and c.layer_specs[2].mixer.right.decay_rank == 8


def test_config_defaults_and_errors():
    c = config_from_dict(U.strip(U.cfg_b()))
    assert c.layer_specs[0].mixer.left.temp_coef == 0.0 and c.groups == 1 and c.layer_specs[1].mixer.taps == 1
    for path, value, match in ((("layers", 0, "type"), "conv", "mixer type"), (("layers", 0, "mlp", "kind"), "glu", "feed-forward"),
                               (("norm", "groups"), 5, "norm groups"), (("layers", 1, "mixer", "kv_heads"), 2, "kv_heads"),
                               (("layers", 1, "mlp", "router", "groups", "keep"), 3, "groups"),
                               (("layers", 0, "mixer", "right", "tau"), 0.0, "tau")):
        bad = U.strip(U.cfg_b())
        node = bad
        for k in path[:-1]:
            node = node[k]
        node[path[-1]] = value
        with pytest.raises(ValueError, match=match):
            config_from_dict(bad)
    bad = U.strip(U.cfg_d())
    bad["layers"][0]["mlp"]["router"]["top"] = 4          # one kept group of three experts cannot give four
    with pytest.raises(ValueError, match="cannot give"):
        config_from_dict(bad)


def test_cache_and_state_sizes():
    c = config_from_dict(U.strip(U.cfg_a()))
    # attention of layers 1 (G=1, 24+16) and 2 (G=2, 16+16), 2 bytes each
    assert c.kv_bytes_per_token(2) == 40 * 2 + 64 * 2
    # per layer the shift row (64 fp32); delta layers: state + conv tail; parallel layers: the linear-attention state
    want = 4 * 64 * 4 + (4 * 16 * 24 * 4 + 2 * (2 * 2 * 16 + 4 * 24) * 2) + 2 * 16 * 8 * 4 + 3 * 8 * 24 * 4 \
        + (2 * 32 * 16 * 4 + 1 * (2 * 32 + 2 * 16) * 2)
    assert c.state_bytes_per_seq(2) == want


def test_unknown_architecture_is_refused(tmp_path):
    (tmp_path / "config.json").write_text(json.dumps({"architecture": "Nope"}))
    with pytest.raises(ValueError, match="unknown architecture"):
        resolve_config(str(tmp_path))


# ------------------------------------------------------------------------------------------------ the oracle by hand
def test_group_norm_by_hand():
    x = torch.tensor([[3.0, 4.0, 0.0, 2.0]], dtype=F64)
    w = torch.tensor([1.0, 2.0, 3.0, 0.5], dtype=F64)
    got = R.group_rms_norm(x, w, 2, 0.0)
    a, b = math.sqrt(12.5), math.sqrt(2.0)
    assert torch.allclose(got, torch.tensor([[3 / a, 8 / a, 0.0, 1 / b]], dtype=F64))
    assert torch.allclose(R.group_rms_norm(x, w, 1, 0.0), x / math.sqrt(29 / 4) * w)


def test_sinusoid_and_shift_by_hand():
    pe = R.sinusoid([0, 3], 4)
    assert torch.allclose(pe[0], torch.tensor([0.0, 1.0, 0.0, 1.0], dtype=F64))
    assert torch.allclose(pe[1], torch.tensor([math.sin(3), math.cos(3), math.sin(0.03), math.cos(0.03)], dtype=F64))
    h = torch.tensor([[1.0, 2.0], [3.0, 6.0], [5.0, 0.0]], dtype=F64)
    got = R.token_shift(h, torch.tensor([0.5, 1.0], dtype=F64))
    assert torch.allclose(got, torch.tensor([[0.5, 0.0], [2.0, 2.0], [4.0, 6.0]], dtype=F64))


def test_query_temperature_steps():
    assert R.query_temperature(0, 0.5, 4) == 1.0 and R.query_temperature(2, 0.5, 4) == 1.0
    assert R.query_temperature(3, 0.5, 4) == pytest.approx(1 + 0.5 * math.log(2))     # (3 + 1) // 4 = 1
    assert R.query_temperature(10, 0.5, 4) == pytest.approx(1 + 0.5 * math.log(3))
    assert R.query_temperature(11, 0.5, 4) == pytest.approx(1 + 0.5 * math.log(4))


def test_grouped_route_by_hand():
    r = {"top": 2, "scale": 2.0, "groups": {"count": 3, "keep": 1}}
    z = torch.tensor([2.0, -9.0, 1.0, 1.0, 0.0, 0.0], dtype=F64)
    s = torch.sigmoid(z)
    # without a correction group 1 (two scores of 0.73) beats group 0 (0.88 + 0.0001) and group 2 (0.5 + 0.5)
    idx, w = R.grouped_route(z, torch.zeros(6, dtype=F64), r)
    assert idx == [2, 3] and torch.allclose(w, torch.tensor([1.0, 1.0], dtype=F64))
    # a correction lifts group 2; the weights stay the plain scores, normalised and scaled
    idx, w = R.grouped_route(z, torch.tensor([0, 0, 0, 0, 0.3, 0.4], dtype=F64), r)
    assert idx == [5, 4] and torch.allclose(w, torch.tensor([1.0, 1.0], dtype=F64))
    # negative choice scores: a group outside the kept ones is never chosen, although its scores are larger than those
    r2 = {"top": 2, "scale": 1.0, "groups": {"count": 2, "keep": 1}}
    z2 = torch.tensor([0.0, 0.1, 3.0, -8.0], dtype=F64)
    corr = torch.tensor([-2.0, -2.0, -0.9, 0.9], dtype=F64)       # choice: -1.5, -1.48 | 0.05, 0.9
    idx, w = R.grouped_route(z2, corr, r2)
    s2 = torch.sigmoid(z2)
    assert idx == [3, 2] and torch.allclose(w, torch.stack([s2[3], s2[2]]) / (s2[3] + s2[2]))
    idx, _ = R.grouped_route(z2, torch.tensor([1.0, 1.0, -3.0, -3.0], dtype=F64), r2)
    assert idx == [1, 0]
    assert s.shape == (6,)


def test_recurrences_by_hand():
    # one key channel, one value column: S is a number
    q = torch.tensor([[1.0], [1.0]], dtype=F64)
    k = torch.tensor([[1.0], [0.5]], dtype=F64)
    v = torch.tensor([[2.0], [4.0]], dtype=F64)
    g = torch.tensor([[1.0], [0.5]], dtype=F64)
    o = R.gated_linear_rule(q, k, v, g)
    assert torch.allclose(o, torch.tensor([[2.0], [0.5 * 2.0 + 0.5 * 4.0]], dtype=F64))
    beta = torch.tensor([1.0, 0.5], dtype=F64)
    o = R.channel_delta_rule(q, k, v, beta, g)
    # token 0: S = 2.  token 1: S <- 1; u = 0.5 (4 - 0.5) = 1.75; S <- 1 + 0.5 * 1.75
    assert torch.allclose(o, torch.tensor([[2.0], [1.875]], dtype=F64))


@pytest.mark.parametrize("make", [U.cfg_a, U.cfg_b, U.cfg_c, U.cfg_d])
def test_prefix_property_of_the_oracle(make):
    """Logits at a position depend on the tokens up to it only."""
    cfg = make()
    W = R.random_model(cfg, seed=1)
    toks = U.tokens(19, cfg["vocab"], 5)
    full = R.forward(cfg, W, toks)
    part = R.forward(cfg, W, toks[:11])
    assert torch.allclose(full[:11], part, atol=1e-9)
    assert bool(torch.isfinite(full).all()) and float(full.std()) > 0.05
