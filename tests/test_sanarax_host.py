"""Host-side pieces of the Sanarax family (no GPU): the configuration reader with its defaults and refusals, cache and
state sizes, which layers own tensors, and the plain oracle against cases worked out by hand."""
import copy
import json
import math

import pytest
import torch

import sanarax_ref as R
import sanarax_util as U

F64 = torch.float64


def _config(c):
    from b200attn import sanarax
    return sanarax.config_from_dict(c)


def test_registered_and_read_from_a_directory(tmp_path):
    from b200attn.model import ARCHITECTURES, resolve_config
    assert "Sanarax" in ARCHITECTURES
    cfg = U.cfg_a()
    (tmp_path / "config.json").write_text(json.dumps(cfg))
    c = resolve_config(str(tmp_path))
    assert c.family == "sanarax" and c.vocab == 97 and c.hidden == 64 and c.layers == 5
    assert (c.embed_scale, c.logit_scale, c.eps) == (2.5, 0.5, 1e-5)
    assert [L.weights for L in c.layer_specs] == [0, 1, 2, 1, 0]
    w = c.layer_specs[1].mixer
    assert (w.heads, w.kv_heads, w.dim, w.window, w.keep_first, w.rot_dims, w.rot_base) == (4, 1, 24, 9, 2, 12, 500.0)
    la = c.layer_specs[2].mixer
    assert (la.kv_rank, la.q_rank, la.rot_dim, la.rot_dims, la.row) == (24, 40, 8, 8, 32)
    assert c.layer_specs[0].mixer.decay == (0.5, 0.9, 0.97) and c.layer_specs[2].mlp.ff == 56


def test_cache_and_state_sizes_count_every_layer_run():
    c = _config(U.cfg_a())
    # two runs of the window layer (K and V pools of one key head of 24), one latent pool of 24 + 8; two lightning runs
    assert c.kv_bytes_per_token(2) == 2 * (2 * 1 * 24 * 2) + 32 * 2
    assert c.kv_bytes_per_token(4) == 2 * c.kv_bytes_per_token(2)
    assert c.state_bytes_per_seq() == 2 * 3 * 16 * 24 * 4
    assert c.activation_bytes(128, 4) > 0 and c.params > 0
    # tensors are counted once per owner
    one = copy.deepcopy(U.cfg_a())
    one["layers"] = one["layers"][:3]
    assert _config(one).params == c.params


def test_defaults():
    c = U.cfg_b()
    del c["embedding"], c["logit_scale"], c["norm"]
    del c["layers"][0]["mixer"]["rot"]
    c["layers"][0]["mixer"].pop("mask", None)
    s = _config(c)
    assert (s.embed_scale, s.logit_scale, s.eps) == (1.0, 1.0, 1e-6)
    m = s.layer_specs[0].mixer
    assert (m.window, m.keep_first, m.rot_dims) == (0, 0, 0)


def test_query_latent_size_from_the_checkpoint_header(tmp_path):
    from b200attn import sanarax
    cfg = U.cfg_d()
    W = R.random_model(cfg, 1)
    bare = copy.deepcopy(cfg)
    for L in bare["layers"]:
        L["mixer"].pop("q_rank", None)
    with pytest.raises(ValueError, match="q_rank"):
        sanarax.config_from_dict(bare)
    U.save_checkpoint(tmp_path, bare, W)
    assert sanarax.config_from_dir(tmp_path).layer_specs[1].mixer.q_rank == 10


@pytest.mark.parametrize("edit,match", [
    (lambda c: c["layers"][0].update(type="convolution"), "unknown mixer"),
    (lambda c: c["layers"][0]["mlp"].update(kind="moe"), "feed-forward"),
    (lambda c: c["layers"][0]["mixer"].update(decay=[0.5]), "decay"),
    (lambda c: c["layers"][1]["mixer"].update(vdim=8), "vdim"),
    (lambda c: c["layers"][1]["mixer"].update(kv_heads=3), "key/value heads"),
    (lambda c: c["layers"][1]["mixer"]["rot"].update(dims=13), "rot.dims"),
    (lambda c: c["layers"][2]["mixer"]["rot"].update(dims=10), "rot.dims"),
    (lambda c: c["layers"][3].update(weights_of=4), "tensors of its own"),
    (lambda c: c["layers"][3].update(weights_of=9), "tensors of its own"),
    (lambda c: c["layers"][3].update(weights_of=2), "differ"),
    (lambda c: c["layers"][3]["mixer"]["mask"].update(size=10), "differ"),
])
def test_refusals(edit, match):
    c = U.cfg_a()
    edit(c)
    with pytest.raises(ValueError, match=match):
        _config(c)


def test_a_layer_may_use_a_later_layers_tensors():
    c = _config(U.cfg_d())
    assert [L.weights for L in c.layer_specs] == [2, 1, 2, 3]
    assert "l0.norm1" not in R.tensor_shapes(U.cfg_d()) and "l2.norm1" in R.tensor_shapes(U.cfg_d())


# ------------------------------------------------------------------------------------------------ the oracle by hand
def test_mask_by_hand():
    see = lambda i, W, F: [j for j in range(i + 3) if R.visible(i, j, W, F)]      # noqa: E731
    assert see(7, 0, 0) == list(range(8))
    assert see(7, 3, 0) == [5, 6, 7]
    assert see(7, 3, 2) == [0, 1, 5, 6, 7]
    assert see(7, 1, 1) == [0, 7]
    assert see(2, 3, 2) == [0, 1, 2]
    assert see(4, 2, 9) == [0, 1, 2, 3, 4]          # a kept prefix longer than the window: plain causal until it ends
    assert see(10, 2, 9) == list(range(9)) + [9, 10]
    assert see(12, 2, 9) == list(range(9)) + [11, 12]


def test_rotation_layouts_by_hand():
    x = torch.tensor([1.0, 2.0, 3.0, 4.0, 5.0, 6.0], dtype=F64)
    f = R.rotary_frequencies(4, 100.0)
    assert f == [1.0, 0.1]
    a, b = 3 * 1.0, 3 * 0.1
    half = R.rotate(x, 3, 4, 100.0, "half")          # pairs (0, 2) and (1, 3); entries 4, 5 pass
    want = [1 * math.cos(a) - 3 * math.sin(a), 2 * math.cos(b) - 4 * math.sin(b), 3 * math.cos(a) + 1 * math.sin(a),
            4 * math.cos(b) + 2 * math.sin(b), 5.0, 6.0]
    assert torch.allclose(half, torch.tensor(want, dtype=F64))
    inter = R.rotate(x, 3, 4, 100.0, "interleaved")  # pairs (0, 1) and (2, 3)
    want = [1 * math.cos(a) - 2 * math.sin(a), 2 * math.cos(a) + 1 * math.sin(a), 3 * math.cos(b) - 4 * math.sin(b),
            4 * math.cos(b) + 3 * math.sin(b), 5.0, 6.0]
    assert torch.allclose(inter, torch.tensor(want, dtype=F64))
    assert torch.equal(R.rotate(x, 0, 4, 100.0, "half"), x) and torch.equal(R.rotate(x, 9, 0, 100.0, "half"), x)


def test_sink_softmax_by_hand():
    s = torch.tensor([0.0, math.log(3.0)], dtype=F64)
    assert torch.allclose(R.sink_softmax(s, None), torch.tensor([0.25, 0.75], dtype=F64))
    assert torch.allclose(R.sink_softmax(s, math.log(4.0)), torch.tensor([0.125, 0.375], dtype=F64))       # the sink takes half
    assert float(R.sink_softmax(s, 50.0).sum()) < 1e-20 * 1e3 + 1e-15
    assert torch.allclose(R.sink_softmax(s, -1e4), torch.tensor([0.25, 0.75], dtype=F64))


def test_decay_scan_by_hand():
    q = torch.ones(3, 1, 1, dtype=F64)
    k = torch.ones(3, 1, 1, dtype=F64)
    v = torch.tensor([1.0, 10.0, 100.0], dtype=F64).view(3, 1, 1)
    o, S = R.decay_scan(q, k, v, [0.5])
    assert o.flatten().tolist() == [1.0, 10.5, 105.25] and float(S) == 105.25
    o2, _ = R.decay_scan(q[2:], k[2:], v[2:], [0.5], state=torch.tensor([[[10.5]]]))
    assert float(o2) == 105.25                       # carried across a cut
    o3, _ = R.decay_scan(q, k, v, [0.0])
    assert o3.flatten().tolist() == [1.0, 10.0, 100.0]


def test_norm_weight_around_zero():
    x = torch.tensor([[3.0, 4.0]], dtype=F64)
    y = R.offset_norm(x, torch.tensor([0.0, 1.0], dtype=F64), 0.0)
    r = math.sqrt(12.5)
    assert torch.allclose(y, torch.tensor([[3.0 / r, 8.0 / r]], dtype=F64))


@pytest.mark.parametrize("make", [U.cfg_a, U.cfg_d])
def test_prefix_property_and_shared_tensors(make):
    """The logits of a position depend on the tokens before it only; a layer with weights_of equals the same layer written
    out with copies of the tensors."""
    cfg = make()
    W = R.random_model(cfg, 3)
    toks = U.tokens(23, cfg["vocab"], 5)
    full = R.forward(cfg, W, toks)
    assert torch.allclose(R.forward(cfg, W, toks[:11]), full[:11], atol=1e-9)
    flat, W2 = copy.deepcopy(cfg), dict(W)
    for i, L in enumerate(flat["layers"]):
        j = L.pop("weights_of", None)
        if j is not None:
            for k, t in W.items():
                if k.startswith(f"l{j}."):
                    W2[f"l{i}." + k.split(".", 1)[1]] = t
    assert torch.allclose(R.forward(flat, W2, toks), full, atol=1e-9)
    assert len(R.tensor_shapes(flat)) > len(R.tensor_shapes(cfg))
