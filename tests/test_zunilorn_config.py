"""Zunilorn without a GPU: its configuration checks, its plan (parts, constants, the
run order of a looped span, tensor names and shapes), the random-weights writer,
and the plain model's own mechanisms against hand-made cases."""
import copy
import math

import pytest
import torch

from kipp_b200.config import config_from_dict
from kipp_b200.config.base import ConfigError
from kipp_b200.config.registry import get_architecture
from tiny import read_weights
from zunilorn_util import CONFIGS, INIT, random_tokens, write_folder

import plain_zunilorn as P


def spec_of(cfg):
    c = config_from_dict(cfg)
    return get_architecture(c.architecture).build(c)


def test_the_model_class_is_chosen_by_the_architecture_key():
    c = config_from_dict(CONFIGS["A"])
    assert c.architecture == "Zunilorn" and c.to_dict()["layers"][0]["type"] == "mamba2"
    assert config_from_dict(c.to_dict()).to_dict() == c.to_dict()
    assert c.vocab_size == 300 and c.hidden_size == 64


def test_a_looped_span_runs_in_a_row_and_every_run_has_its_own_cache():
    order = spec_of(CONFIGS["A"]).plan["order"]
    assert [o["layer"] for o in order] == [0, 1, 2, 1, 2, 3] == P.run_order(CONFIGS["A"])
    assert [o["cache"] for o in order] == list(range(6)) and all(o["writes_cache"] for o in order)
    assert [o["layer"] for o in spec_of(CONFIGS["C"]).plan["order"]] == [0, 0, 0, 1, 2]
    assert [o["layer"] for o in spec_of(CONFIGS["B"]).plan["order"]] == [0, 1, 2, 3]
    empty = copy.deepcopy(CONFIGS["B"])
    empty["loop"] = {"start": 2, "stop": 2, "times": 4}           # an empty span changes nothing
    assert [o["layer"] for o in spec_of(empty).plan["order"]] == [0, 1, 2, 3]


def test_parts_and_their_constants():
    plan = spec_of(CONFIGS["A"]).plan
    assert plan["streams"] == 3
    blocks = [l["part"] for l in plan["layers"]]
    assert all(b["kind"] == "hyper_connection_block" and b["residual_mult"] == 0.6 and b["streams"] == 3 and
               b["connections"] for b in blocks)
    ssm, att = blocks[0]["mixer"], blocks[1]["mixer"]
    assert ssm["kind"] == "state_space" and (ssm["num_heads"], ssm["groups"], ssm["value_dim"], ssm["state_dim"],
                                             ssm["conv"], ssm["norm_groups"]) == (4, 2, 16, 24, 3, 2)
    assert att["kind"] == "attention" and att["sink"] == "learned" and att["head_gate"] and att["softcap"] == 15.0
    assert att["value_dim"] == 24 and att["scale"] == 0.3
    pos = att["position"]
    assert pos["kind"] == "yarn_rotary" and (pos["rotary_dim"], pos["theta"], pos["factor"], pos["original"], pos["fast"],
                                             pos["slow"]) == (8, 10000.0, 2.0, 64, 8.0, 1.0)
    assert blocks[0]["ffn"]["kind"] == "gated_mlp" and blocks[0]["ffn"]["bias"] and blocks[0]["ffn"]["limit"] == 1.5
    assert blocks[0]["ffn"]["alpha"] == 1.702 and not blocks[0]["ffn"]["row_gate"]
    ex = blocks[1]["ffn"]
    assert ex["kind"] == "expert_mixture" and ex["routing"] == "scores" and ex["gated"] and ex["correction"]
    assert (ex["experts"], ex["identity"], ex["top"], ex["weight_scale"], ex["limit"]) == (5, 3, 2, 2.0, 1.0)
    assert ex["shared"]["kind"] == "gated_mlp" and ex["shared"]["row_gate"] and not ex["shared"]["bias"]
    assert blocks[3]["ffn"] is None and blocks[3]["post_norm"] is None
    head = plan["head"]["part"]
    assert head["tied_to"] == "embed" and head["logit_softcap"] == 12.0
    # what the configuration leaves out: one stream without connections, no caps, no limits, a multiplier of one
    plan = spec_of(CONFIGS["B"]).plan
    b0 = plan["layers"][0]["part"]
    assert plan["streams"] == 1 and not b0["connections"] and b0["residual_mult"] == 1.0
    assert plan["head"]["part"]["logit_softcap"] == 0.0 and b0["mixer"]["softcap"] == 0.0
    assert b0["mixer"]["position"]["kind"] == "rotary" and b0["mixer"]["num_kv_heads"] == 3
    assert plan["layers"][2]["part"]["mixer"]["position"]["kind"] == "no_position"
    assert b0["ffn"]["identity"] == 0 and b0["ffn"].get("shared") is None and b0["ffn"]["limit"] == 0.0
    # one stream WITH its connections is not the plain sum
    assert spec_of(CONFIGS["D"]).plan["layers"][0]["part"]["connections"]


def test_tensor_names_and_shapes():
    specs = {s.name: tuple(s.shape) for s in spec_of(CONFIGS["A"]).tensor_specs()}
    inner, channels = 4 * 16, 4 * 16 + 2 * 2 * 24
    assert specs["l0.mix.in"] == (inner + channels + 4, 64) and specs["l0.mix.conv"] == (channels, 3)
    assert specs["l0.mix.conv.b"] == (channels,) and specs["l0.mix.norm"] == (inner,) and specs["l0.mix.o"] == (64, inner)
    assert specs["l0.mix.A_log"] == specs["l0.mix.D"] == specs["l0.mix.dt_bias"] == (4,)
    assert specs["l0.mlp.gate"] == (96, 64) and specs["l0.mlp.down.b"] == (64,) and specs["l0.mlp.up.b"] == (96,)
    assert specs["l1.mix.q"] == (64, 64) and specs["l1.mix.k"] == (32, 64) and specs["l1.mix.v"] == (48, 64)
    assert specs["l1.mix.o"] == (64, 96) and specs["l1.mix.sink"] == (4,) and specs["l1.mix.g"] == (4, 64)
    assert specs["l1.mlp.router"] == (8, 64) and specs["l1.mlp.correction"] == (8,)
    assert specs["l1.mlp.e4.gate"] == (40, 64) and specs["l1.mlp.e4.down"] == (64, 40) and "l1.mlp.e5.up" not in specs
    assert specs["l1.mlp.shared.up"] == (48, 64) and specs["l1.mlp.shared.sg"] == (1, 64)
    assert specs["l1.hc1.in"] == (3,) and specs["l1.hc2.mix"] == (3, 3) and specs["l3.hc1.out"] == (3,)
    assert "l3.hc2.in" not in specs and "l3.norm2" not in specs and specs["final.norm"] == (64,)
    assert "head" not in specs or True
    plain = {s.name for s in spec_of(CONFIGS["B"]).tensor_specs()}
    assert not any(".hc" in n for n in plain) and "l0.mlp.correction" in plain


@pytest.mark.parametrize("change,message", [
    (lambda c: c.pop("vocab"), "vocab"),
    (lambda c: c["norm"].update(eps=0), "norm.eps"),
    (lambda c: c["layers"][0].update(type="conv"), "unknown layer type"),
    (lambda c: c["layers"][1]["mixer"].update(heads=3), "multiple of kv_heads"),
    (lambda c: c["layers"][0]["mixer"].update(groups=3), "multiple of groups"),
    (lambda c: c["layers"][0]["mixer"].update(norm_groups=5), "norm_groups"),
    (lambda c: c["layers"][1]["mixer"]["rot"].update(dims=7), "rot.dims"),
    (lambda c: c["layers"][1]["mixer"]["rot"]["scaling"].update(factor=0), "rot.scaling.factor"),
    (lambda c: c["layers"][1]["mixer"]["rot"]["scaling"].pop("slow"), "rot.scaling.slow"),
    (lambda c: c["layers"][1]["mlp"]["router"].update(top=9), "router.top"),
    (lambda c: c["layers"][1]["mlp"].update(kind="other"), "mlp.kind"),
    (lambda c: c["layers"][0]["mlp"].pop("ff"), "mlp.ff"),
    (lambda c: c["loop"].update(stop=9), "loop"),
    (lambda c: c.update(streams=0), "streams"),
    (lambda c: c.update(logit_softcap=-1.0), "logit_softcap"),
])
def test_what_the_configuration_refuses(change, message):
    cfg = copy.deepcopy(CONFIGS["A"])
    change(cfg)
    with pytest.raises(ConfigError) as e:
        config_from_dict(cfg)
    assert message in str(e.value)


def test_random_weights_cover_every_declared_tensor(tmp_path):
    folder = write_folder(str(tmp_path / "m"), CONFIGS["D"], INIT["D"])
    w = read_weights(folder)
    specs = {s.name: tuple(s.shape) for s in spec_of(CONFIGS["D"]).tensor_specs() if not (s.optional and s.alias_of)}
    assert {k: tuple(v.shape) for k, v in w.items()} == specs
    with torch.no_grad():
        logits = P.forward(CONFIGS["D"], w, random_tokens(101, 12, seed=1))
    assert logits.shape == (12, 101) and bool(torch.isfinite(logits).all()) and float(logits.abs().max()) <= 8.0


def test_the_parts_can_be_described_from_python_for_another_design():
    """A model put together in Python from the descriptions of the same parts (the layers without experts) gives
    the tensors and the parts the library's own builder makes."""
    from kipp_b200.models.spec import LayerRun, ModelSpec
    from kipp_b200.parts import (AttentionMixer, GatedFeedForward, HyperConnectionBlock, OutputHead, RMSNorm,
                                 StateSpaceMixer, TokenEmbedding, YarnRotaryEncoding)
    cfg = copy.deepcopy(CONFIGS["A"])
    cfg["layers"] = [cfg["layers"][0], cfg["layers"][3]]
    cfg.pop("loop")
    eps, width, S = cfg["norm"]["eps"], cfg["width"], cfg["streams"]
    layers = []
    for i, layer in enumerate(cfg["layers"]):
        m = layer["mixer"]
        if layer["type"] == "mamba2":
            mixer = StateSpaceMixer(width, m["heads"], m["vdim"], m["state"], m["conv"], eps, groups=m["groups"],
                                    norm_groups=m["norm_groups"])
        else:
            sc = m["rot"]["scaling"]
            pos = YarnRotaryEncoding(m["dim"], m["rot"]["base"], sc["factor"], sc["original"], sc["fast"], sc["slow"], m["rot"]["dims"])
            mixer = AttentionMixer(width, m["heads"], m["kv_heads"], m["dim"], pos, None, 0, m["scale"], value_dim=m["vdim"],
                                   sink="learned", head_gate=True, softcap=m["softcap"],
                                   names={"q": "q", "k": "k", "v": "v", "o": "o", "sink": "sink", "gate": "g"})
        f = layer["mlp"]
        ffn = GatedFeedForward(width, f["ff"], limit=f["limit"], alpha=1.702, bias=True) if f else None
        layers.append((f"l{i}.", HyperConnectionBlock(RMSNorm(width, eps, "norm1"), mixer, RMSNorm(width, eps, "norm2") if f else None,
                                                      ffn, streams=S, residual_mult=cfg["residual_mult"])))
    spec = ModelSpec(config=None, hidden_size=width, vocab_size=cfg["vocab"], streams=S,
                     embedding=TokenEmbedding(cfg["vocab"], width, weight_name="embed"), layers=layers,
                     order=[LayerRun(i, i) for i in range(len(layers))], final_norm=("", RMSNorm(width, eps, "final.norm")),
                     head=("", OutputHead(cfg["vocab"], width, tied_to="embed", weight_name="head",
                                          logit_softcap=cfg["logit_softcap"])))
    mine = {s.name: tuple(s.shape) for s in spec.tensor_specs()}
    theirs_spec = spec_of(cfg)
    assert mine == {s.name: tuple(s.shape) for s in theirs_spec.tensor_specs()}
    plan, _ = spec.to_plan()
    assert plan["streams"] == theirs_spec.plan["streams"] == 3
    for a, b in zip(plan["layers"], theirs_spec.plan["layers"]):
        assert a["part"]["mixer"]["kind"] == b["part"]["mixer"]["kind"]
        for key in ("streams", "connections", "residual_mult"):
            assert a["part"][key] == b["part"][key]
    assert plan["layers"][1]["part"]["mixer"]["position"] == theirs_spec.plan["layers"][1]["part"]["mixer"]["position"]
    assert plan["head"]["part"]["logit_softcap"] == 12.0
    # a block on another number of copies than the plan's is refused
    spec.streams = 2
    with pytest.raises(Exception) as e:
        spec.tensor_specs()
    assert "copies of the residual stream" in str(e.value)


# ------------------------------------------------------------------ the plain model against hand-made cases
def test_plain_causal_convolution_and_its_start():
    x = torch.tensor([[1.0], [2.0], [4.0]], dtype=torch.float64)
    w = torch.tensor([[100.0, 10.0, 1.0]], dtype=torch.float64)        # the last column meets the current token
    got = P.causal_conv(x, w, torch.tensor([0.5], dtype=torch.float64))
    assert got.flatten().tolist() == [1.5, 12.5, 124.5]


def test_plain_state_space_of_one_head_by_hand():
    m = {"heads": 1, "groups": 1, "vdim": 1, "state": 1, "conv": 1, "norm_groups": 1}
    # the projection is the identity on [z, x, B, C, dt]; the convolution passes its input on
    w = {"in": torch.eye(5, dtype=torch.float64), "conv": torch.ones(3, 1, dtype=torch.float64),
         "conv.b": torch.zeros(3, dtype=torch.float64), "dt_bias": torch.zeros(1, dtype=torch.float64),
         "A_log": torch.zeros(1, dtype=torch.float64), "D": torch.tensor([0.25], dtype=torch.float64),
         "norm": torch.ones(1, dtype=torch.float64), "o": torch.ones(5, 1, dtype=torch.float64)}
    h = torch.tensor([[0.3, 1.0, 2.0, -1.0, 0.1], [-0.2, 0.5, 1.0, 3.0, 0.7]], dtype=torch.float64)
    silu = lambda v: v / (1 + math.exp(-v))                                  # noqa: E731
    S, ys = 0.0, []
    for z, x, B, C, dt in h.tolist():
        x, B, C = silu(x), silu(B), silu(C)
        dt = math.log1p(math.exp(dt))
        S = math.exp(-dt) * S + dt * B * x
        ys.append((S * C + 0.25 * x) * silu(z))
    got = P.mamba2(m, w, "", h, 1e-5)
    want = [y / math.sqrt(y * y + 1e-5) for y in ys]
    assert torch.allclose(got[:, 0], torch.tensor(want, dtype=torch.float64), atol=1e-12)


def test_plain_sink_joins_the_denominator_alone():
    m = {"heads": 1, "kv_heads": 1, "dim": 2, "vdim": 1, "scale": 1.0}
    w = {"q": torch.zeros(2, 2, dtype=torch.float64), "k": torch.zeros(2, 2, dtype=torch.float64),
         "v": torch.tensor([[1.0, 0.0]], dtype=torch.float64), "g": torch.zeros(1, 2, dtype=torch.float64),
         "sink": torch.tensor([math.log(2.0)], dtype=torch.float64), "o": torch.ones(2, 1, dtype=torch.float64)}
    h = torch.tensor([[3.0, 0.0], [5.0, 0.0]], dtype=torch.float64)
    got = P.attention(m, w, "", h)
    # scores are 0: weights 1 / (t + 1 + 2); the gate is one half
    assert torch.allclose(got[:, 0], torch.tensor([3.0 / 3 / 2, (3.0 + 5.0) / 4 / 2], dtype=torch.float64))


def test_plain_routing_by_scores():
    f = {"router": {"experts": 2, "identity": 1, "top": 2, "scale": 3.0}}
    w = {"router": torch.tensor([[1.0], [0.0], [2.0]], dtype=torch.float64),
         "correction": torch.tensor([0.0, 10.0, 0.0], dtype=torch.float64)}
    chosen, weights = P.route(f, w, "", torch.tensor([[1.0]], dtype=torch.float64))
    s = torch.softmax(torch.tensor([1.0, 0.0, 2.0], dtype=torch.float64), 0)
    assert chosen.tolist() == [[1, 2]]                   # the correction chooses, the scores weigh
    assert torch.allclose(weights[0], 3.0 * s[[1, 2]] / (s[1] + s[2]))


def test_plain_gated_activation_with_limits():
    g, u = torch.tensor([3.0, -4.0, 0.5], dtype=torch.float64), torch.tensor([9.0, -9.0, 0.2], dtype=torch.float64)
    got = P.glu(g, u, 2.0)
    gate = torch.tensor([2.0, -4.0, 0.5], dtype=torch.float64)            # the gate is bounded from above only
    up = torch.tensor([2.0, -2.0, 0.2], dtype=torch.float64)
    assert torch.allclose(got, gate * torch.sigmoid(1.702 * gate) * (up + 1))


def test_plain_hyper_connections_with_chosen_numbers():
    cfg = {"streams": 2, "residual_mult": 0.5, "norm": {"eps": 1e-5},
           "layers": [{"type": "attention", "mixer": {}, "mlp": None}]}
    xs = torch.tensor([[[1.0, 2.0]], [[10.0, 20.0]]], dtype=torch.float64)          # [streams, T, W]
    w = {"l0.hc1.in": torch.tensor([1.0, 0.1], dtype=torch.float64), "l0.hc1.out": torch.tensor([2.0, -1.0], dtype=torch.float64),
         "l0.hc1.mix": torch.tensor([[1.0, 3.0], [0.0, 1.0]], dtype=torch.float64), "l0.norm1": torch.ones(2, dtype=torch.float64)}
    seen = {}

    def fake(cfg_, w_, i, q, h):
        seen["h"] = h
        return torch.tensor([[100.0, 200.0]], dtype=torch.float64)
    real, P.sublayer = P.sublayer, fake
    try:
        out = P.layer_forward(cfg, w, 0, xs)
    finally:
        P.sublayer = real
    u = torch.tensor([[2.0, 4.0]], dtype=torch.float64)                               # 1 * x_1 + 0.1 * x_2
    assert torch.allclose(seen["h"], P.rms_divide(u, 1e-5))
    # mix is [from, to]: stream 1 keeps x_1; stream 2 gets 3 x_1 + x_2; then mult * out[t] * y
    assert torch.allclose(out[0], torch.tensor([[1.0 + 100.0, 2.0 + 200.0]], dtype=torch.float64))
    assert torch.allclose(out[1], torch.tensor([[13.0 - 50.0, 26.0 - 100.0]], dtype=torch.float64))
