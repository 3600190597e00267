"""Zasudra without a GPU: its configuration checks, its plan (layers, which run
reads whose cache, tensor names and shapes), the random-weights writer, and the
plain model's own mechanisms against hand-made cases."""
import copy
import math

import pytest
import torch

from kipp_b200.config import config_from_dict
from kipp_b200.config.base import ConfigError
from kipp_b200.config.registry import get_architecture
from tiny import read_weights
from zasudra_util import CONFIGS, INIT, random_tokens, write_folder

import plain_zasudra as P


def spec_of(cfg):
    c = config_from_dict(cfg)
    return get_architecture(c.architecture).build(c)


def test_the_model_class_is_chosen_by_the_architecture_key():
    c = config_from_dict(CONFIGS["A"])
    assert c.architecture == "Zasudra" and c.to_dict()["layers"][1]["type"] == "wkv"
    assert config_from_dict(c.to_dict()).to_dict() == c.to_dict()
    assert c.vocab_size == 300 and c.hidden_size == 64


def test_a_layer_that_borrows_reads_the_lenders_cache_and_writes_none():
    order = spec_of(CONFIGS["A"]).plan["order"]
    assert [(o["layer"], o["cache"], o["writes_cache"]) for o in order] == [
        (0, 0, True), (1, 1, True), (2, 2, True), (3, 2, False), (4, 4, True)]
    order = spec_of(CONFIGS["B"]).plan["order"]
    assert [(o["cache"], o["writes_cache"]) for o in order][1:3] == [(1, True), (1, False)]


def test_parts_and_their_constants():
    plan = spec_of(CONFIGS["A"]).plan
    stages = [s["part"]["kind"] for s in plan["embedding"]]
    assert stages == ["token_embedding", "hashed_pair_embedding"]
    assert plan["embedding"][1]["part"]["buckets"] == 97 and plan["embedding"][1]["part"]["mul_prev"] == 31
    blocks = [l["part"] for l in plan["layers"]]
    assert all(b["kind"] == "output_norm_block" and b["residual_mult"] == 0.7 for b in blocks)
    first, gated, borrower = blocks[0]["mixer"], blocks[2]["mixer"], blocks[3]["mixer"]
    assert first["chunk"] == 16 and first["sink"] == "learned" and first["values_are_keys"] and first["interleaved"]
    assert first["norm_whole"] and first["position"]["rotary_dim"] == 8 and not first["head_gate"]
    assert gated["chunk"] == 0 and gated["sink"] == "unit" and gated["head_gate"] and not gated["values_are_keys"]
    assert gated["position"]["kind"] == "no_position" and gated["value_dim"] == 24
    assert borrower["shared_kv"] and not gated["shared_kv"]
    assert blocks[1]["mixer"]["kind"] == "wkv" and blocks[1]["ffn"]["kind"] == "expert_mixture"
    assert blocks[1]["ffn"]["experts"] == 5 and blocks[1]["ffn"]["top"] == 2 and blocks[2]["ffn"] is None
    assert plan["head"]["part"]["logit_scale"] == 1.5
    # what the configuration leaves out: no pair table, multiplier and logit scale of one
    plan = spec_of(CONFIGS["B"]).plan
    assert [s["part"]["kind"] for s in plan["embedding"]] == ["token_embedding"]
    assert plan["layers"][0]["part"]["residual_mult"] == 1.0 and plan["head"]["part"]["logit_scale"] == 1.0
    assert plan["layers"][4]["part"]["mixer"]["position"]["kind"] == "no_position"


def test_tensor_names_and_shapes():
    specs = {s.name: tuple(s.shape) for s in spec_of(CONFIGS["A"]).tensor_specs()}
    assert specs["embed"] == (300, 64) and specs["bigram"] == (98, 64) and specs["head"] == (300, 64)
    assert specs["l0.mix.q"] == (64, 64) and specs["l0.mix.k"] == (32, 64) and "l0.mix.v" not in specs
    assert specs["l0.mix.q.norm"] == (64,) and specs["l0.mix.k.norm"] == (32,) and specs["l0.mix.sink"] == (4,)
    assert specs["l2.mix.v"] == (96, 64) and specs["l2.mix.g"] == (4, 64) and specs["l2.mix.o"] == (64, 96)
    assert "l2.mix.sink" not in specs and "l2.norm2" not in specs and "l2.mlp.router" not in specs
    # the borrower has queries, a gate and an output projection, and nothing of keys and values
    assert specs["l3.mix.q"] == (64, 64) and specs["l3.mix.g"] == (4, 64)
    assert not any(n in specs for n in ("l3.mix.k", "l3.mix.v", "l3.mix.k.norm"))
    assert specs["l1.mix.mu.w"] == (64,) and specs["l1.mix.w1"] == (8, 64) and specs["l1.mix.w2"] == (32, 8)
    assert specs["l1.mix.w0"] == (32,) and specs["l1.mix.u"] == (2, 16) and specs["l1.mix.norm"] == (32,)
    assert specs["l1.mlp.e4.up"] == (40, 64) and specs["l1.mlp.e4.down"] == (64, 40) and "l1.mlp.e5.up" not in specs
    assert specs["l1.mlp.router"] == (5, 64) and specs["l1.mlp.router.b"] == (5,)
    assert specs["l4.mix.w1"] == (5, 64) and specs["final.norm"] == (64,)


def test_the_width_of_the_decay_bottleneck_may_be_left_to_the_tensor():
    cfg = copy.deepcopy(CONFIGS["A"])
    del cfg["layers"][1]["mixer"]["decay_rank"]
    specs = {s.name: tuple(s.shape) for s in spec_of(cfg).tensor_specs()}
    assert specs["l1.mix.w1"] == (-1, 64) and specs["l1.mix.w2"] == (32, -1)


def _changed(name, path, value):
    cfg = copy.deepcopy(CONFIGS[name])
    o = cfg
    for key in path[:-1]:
        o = o[key]
    if value is KeyError:
        del o[path[-1]]
    else:
        o[path[-1]] = value
    return cfg


@pytest.mark.parametrize("name,path,value,message", [
    ("A", ("layers", 0, "type"), "conv", "unknown layer type"),
    ("A", ("layers", 0, "mixer", "heads"), 3, "multiple of kv_heads"),
    ("A", ("layers", 0, "mixer", "vdim"), 8, "must equal dim"),
    ("A", ("layers", 0, "mixer", "rot", "dims"), 7, "even"),
    ("A", ("layers", 0, "mixer", "scale"), KeyError, "scale"),
    ("A", ("layers", 3, "mixer", "kv_from"), 3, "earlier layer"),
    ("A", ("layers", 3, "mixer", "kv_from"), 1, "attention layer"),
    ("A", ("layers", 3, "mixer", "kv_heads"), 2, "differ in 'kv_heads'"),
    ("A", ("layers", 1, "mlp", "router", "top"), 6, "must not exceed"),
    ("A", ("layers", 1, "mlp", "kind"), "dense", "not supported"),
    ("A", ("layers", 1, "mlp", "expert"), KeyError, "expert"),
    ("A", ("embedding", "bigram", "buckets"), 0, "at least 1"),
    ("A", ("norm", "eps"), 0.0, "positive"),
    ("A", ("width",), KeyError, "width"),
])
def test_configurations_that_are_refused(name, path, value, message):
    with pytest.raises(ConfigError, match=message):
        config_from_dict(_changed(name, path, value))


def test_the_writer_makes_every_tensor_of_the_plan(tmp_path):
    folder = write_folder(str(tmp_path / "m"), CONFIGS["D"], INIT["D"])
    w = read_weights(folder)
    specs = {s.name: tuple(s.shape) for s in spec_of(CONFIGS["D"]).tensor_specs()}
    assert {k: tuple(v.shape) for k, v in w.items()} == specs
    with torch.no_grad():
        logits = P.forward(CONFIGS["D"], w, random_tokens(101, 12, seed=1))
    assert logits.shape == (12, 101) and bool(torch.isfinite(logits).all())


# ------------------------------------------------------------------ the plain model's mechanisms
def test_plain_pair_rows():
    b = {"buckets": 10, "mul_prev": 3, "mul_cur": 7}
    assert P.bigram_rows([4, 9, 0, 5], b) == [10, (4 * 3 + 9 * 7) % 10, (9 * 3) % 10, (5 * 7) % 10]


def test_plain_rotation_pairs_neighbours_and_keeps_the_rest():
    x = torch.arange(12, dtype=torch.float64).view(1, 1, 12).repeat(3, 1, 1)
    y = P.rotate_interleaved(x, torch.arange(3), 4, 100.0)
    assert torch.equal(y[0], x[0]) and torch.equal(y[:, :, 4:], x[:, :, 4:])
    a = 2 * 100.0 ** (-2.0 / 4)               # position 2, pair 1
    assert math.isclose(float(y[2, 0, 2]), 2 * math.cos(a) - 3 * math.sin(a), rel_tol=1e-12)
    assert math.isclose(float(y[2, 0, 3]), 3 * math.cos(a) + 2 * math.sin(a), rel_tol=1e-12)
    assert math.isclose(float(y[1, 0, 0]), -math.sin(1.0), rel_tol=1e-12)     # pair 0 turns by the position itself


def test_plain_blocks_are_counted_from_position_zero():
    vis = P.visible_chunked(7, 3)
    assert vis[2].tolist() == [True, True, True, False, False, False, False]
    assert vis[3].tolist() == [False, False, False, True, False, False, False]
    assert vis[5].tolist() == [False, False, False, True, True, True, False]
    assert P.visible_chunked(4, 0)[3].tolist() == [True] * 4


def test_plain_sink_counts_once_and_has_no_value():
    s = torch.tensor([[0.0, 1.0]], dtype=torch.float64)
    vis = torch.tensor([[True, True]])
    p = P.softmax_with_sink(s, vis, 2.0)
    z = math.exp(2.0) + 1.0 + math.e
    assert torch.allclose(p, torch.tensor([[1.0 / z, math.e / z]], dtype=torch.float64))
    p0 = P.softmax_with_sink(s, torch.tensor([[True, False]]), 0.0)
    assert torch.allclose(p0, torch.tensor([[0.5, 0.0]], dtype=torch.float64))


def test_plain_wkv_reads_the_old_state_and_the_bonus_once():
    H, D, W = 1, 2, 2
    eye = torch.eye(2, dtype=torch.float64)
    w = {"mu." + s: torch.zeros(W, dtype=torch.float64) for s in "rkvgw"}
    w.update({"r": eye, "k": eye, "v": eye, "g": eye, "w1": torch.zeros(1, W, dtype=torch.float64),
              "w2": torch.zeros(2, 1, dtype=torch.float64), "w0": torch.zeros(2, dtype=torch.float64),
              "u": torch.tensor([[2.0, 0.0]], dtype=torch.float64), "norm": torch.ones(2, dtype=torch.float64),
              "o": eye})
    h = torch.tensor([[1.0, 3.0], [5.0, 7.0]], dtype=torch.float64)
    d = math.exp(-1.0)                                   # exp(-exp(0)) on every channel
    # o_0 = (u k_0) . r_0 v_0 = (2 * 1 * 1) * v_0;  S_0 = k_0 v_0^T
    # o_1 = S_0^T r_1 + (2 * 5 * 5) v_1 = (1*5 + 3*7) v_0 + 50 v_1
    o0 = 2.0 * h[0]
    o1 = 26.0 * h[0] + 50.0 * h[1]
    gate = h * torch.sigmoid(h)
    want = torch.stack([P.rms_divide(o0, 1e-6), P.rms_divide(o1, 1e-6)]) * gate
    got = P.wkv({("p." + k): v for k, v in w.items()}, "p.", {"heads": H, "dim": D}, h, 1e-6)
    assert torch.allclose(got, want, rtol=1e-12)
    # a third token sees S_1 = d S_0 + k_1 v_1^T
    h3 = torch.cat([h, torch.tensor([[1.0, 0.0]], dtype=torch.float64)])
    got3 = P.wkv({("p." + k): v for k, v in w.items()}, "p.", {"heads": H, "dim": D}, h3, 1e-6)
    o2 = (d * 1.0) * h[0] + 5.0 * h[1] + 2.0 * h3[2]
    assert torch.allclose(got3[2], P.rms_divide(o2, 1e-6) * gate.new_tensor([1 / (1 + math.exp(-1.0)), 0.0]), rtol=1e-12)


def test_plain_router_weights_are_a_softmax_over_the_chosen_only():
    w = {"p.router": torch.eye(4, dtype=torch.float64), "p.router.b": torch.tensor([0.0, 0.0, 0.5, 0.0], dtype=torch.float64)}
    h = torch.tensor([[3.0, 1.0, 2.0, -5.0]], dtype=torch.float64)
    idx, wt = P.route(w, "p.", {"experts": 4, "top": 2}, h)
    assert idx.tolist() == [[0, 2]]
    assert torch.allclose(wt, torch.softmax(torch.tensor([[3.0, 2.5]], dtype=torch.float64), -1))
