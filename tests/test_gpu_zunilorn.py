"""Zunilorn on the GPU against the plain float64 model (plain_zunilorn.py): each
mechanism alone; whole prompts; token-by-token decoding from the first token;
portions down to two tokens; batches of unequal requests; pages and slots used
again; keys far away and at the edges of pages; the sink; the first tokens; a state
that remembers the first token through long decoding; long decoding through
graphs; drawn configurations; greedy generation through the scheduler; the command
line and the trace program."""
import json
import math
import os
import random
import subprocess
import sys

import pytest
import torch

import plain_zunilorn as P
from tiny import nmse, read_weights
from zunilorn_util import (CONFIGS, attention_layer, dense, mamba_layer, model_folder, moe, random_tokens, set_tensors,
                           write_folder, yarn)

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
# float32: the engine against the float64 plain model.  bfloat16: against the plain model with
# the matrices rounded to bfloat16 (activations are not rounded there, so the bound is that of
# 16-bit activations through a few layers).
BOUND = {"float32": 1e-9, "bfloat16": 2e-3}


def rounded(w, dtype):
    if dtype != "bfloat16":
        return w
    return {k: (v.to(torch.bfloat16).float() if v.is_floating_point() else v) for k, v in w.items()}


def weights_for(name, dtype):
    return rounded(read_weights(model_folder(name)), dtype)


def f64(w):
    return {k: (v.double() if v.is_floating_point() else v) for k, v in w.items()}


_plain = {}


def plain_logits(name, dtype, tokens, whole_model=False):
    key = (name, dtype, tuple(tokens))
    if key not in _plain:
        with torch.no_grad():
            _plain[key] = P.forward(CONFIGS[name], weights_for(name, dtype), list(tokens))
    return (_plain[key], None) if whole_model else _plain[key]


def engine_for(name, dtype, **kw):
    from kipp_b200.engine import Engine
    opts = dict(dtype=dtype, page_size=16, cache_tokens=1024, max_requests=4, max_batch_tokens=1024)
    opts.update(kw)
    return Engine.from_folder(model_folder(name), **opts)


def close(got, want, dtype, what="", factor=1.0):
    """`want` as a pair marks the logits of a whole model.  In bfloat16 a router's close call
    may go the other way than in the plain model, and what that token then leaves in the caches
    and states reaches later rows; so there the rows are judged one by one: half of them within
    the bound, three quarters within ten times the bound.  (32-bit: all of them together.)"""
    if isinstance(want, tuple):
        want = want[0]
        if dtype == "bfloat16":
            g, w = got.cpu().double(), want.double()
            w = w - w.mean(1, keepdim=True)
            g = g - g.mean(1, keepdim=True)
            rows = (((g - w) ** 2).sum(1) / (w ** 2).sum(1)).sort().values
            n = len(rows)
            median, upper = float(rows[(n - 1) // 2]), float(rows[(3 * (n - 1)) // 4])
            assert median <= BOUND[dtype] * factor and upper <= 10 * BOUND[dtype] * factor, \
                f"{what}: row NMSE median {median:.3e}, third quartile {upper:.3e}"
            return
    e = nmse(got.cpu(), want)
    assert e <= BOUND[dtype] * factor, f"{what}: NMSE {e:.3e} > {BOUND[dtype] * factor:.1e}"


def _inputs(name, T, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randn(T, CONFIGS[name]["width"], generator=g, dtype=torch.float64)


def _run_of(eng, layer):
    return [o["layer"] for o in eng.spec.plan["order"]].index(layer)


def layers_of(kind):
    return [(n, i) for n in sorted(CONFIGS) for i, l in enumerate(CONFIGS[n]["layers"]) if l["type"] == kind]


# ------------------------------------------------------------------ each mechanism alone
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name,layer", layers_of("attention"))
def test_attention_alone(name, layer, dtype):
    """Rotation (stretched, plain, none), capped scores, the sink, the gate: in three portions,
    the later ones read the cache the earlier ones left."""
    from kipp_b200.engine import StepEntry
    cfg = CONFIGS[name]
    eng = engine_for(name, dtype, cuda_graphs=False)
    T = 150
    h_dev = _inputs(name, T, 100 + layer).to("cuda", eng.dtype).contiguous()
    w = f64(weights_for(name, dtype))
    want = P.attention(cfg["layers"][layer]["mixer"], w, f"l{layer}.mix.", h_dev.double().cpu())
    out = torch.zeros(T, cfg["width"], device="cuda")
    at = 0
    for n in (70, 1, 79):
        eng.run_part([StepEntry("a", [0] * n, [])], _run_of(eng, layer), "mixer", input=h_dev[at:at + n].contiguous(),
                     residual=out[at:at + n])
        at += n
    close(out, want, dtype, f"{name} layer {layer}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name,layer", layers_of("mamba2"))
def test_state_space_alone(name, layer, dtype):
    """The state and the convolution's last inputs cross every cut: portions shorter than the
    convolution's reach, of one token, and long ones."""
    from kipp_b200.engine import StepEntry
    cfg = CONFIGS[name]
    eng = engine_for(name, dtype, cuda_graphs=False)
    T = 66
    h_dev = _inputs(name, T, 200 + layer).to("cuda", eng.dtype).contiguous()
    w = f64(weights_for(name, dtype))
    want = P.mamba2(cfg["layers"][layer]["mixer"], w, f"l{layer}.mix.", h_dev.double().cpu(), cfg["norm"]["eps"])
    out = torch.zeros(T, cfg["width"], device="cuda")
    at = 0
    for n in (1, 2, 1, 1, 3, 17, 2, 39):
        eng.run_part([StepEntry("d", [0] * n, [])], _run_of(eng, layer), "mixer", input=h_dev[at:at + n].contiguous(),
                     residual=out[at:at + n])
        at += n
    assert at == T
    close(out, want, dtype, f"{name} layer {layer}")


def test_the_convolution_starts_from_zeros_in_a_slot_used_again():
    """A second request in the slot the first one gave back: no input and no state of the first."""
    from kipp_b200.engine import StepEntry
    name, layer = "A", 0
    cfg = CONFIGS[name]
    eng = engine_for(name, "float32", cuda_graphs=False, max_requests=1)
    w = f64(weights_for(name, "float32"))
    for k, rid in enumerate(("first", "second")):
        h_dev = _inputs(name, 9, 700 + k).to("cuda", eng.dtype).contiguous()
        want = P.mamba2(cfg["layers"][layer]["mixer"], w, f"l{layer}.mix.", h_dev.double().cpu(), cfg["norm"]["eps"])
        out = torch.zeros(9, cfg["width"], device="cuda")
        eng.run_part([StepEntry(rid, [0] * 2, [])], _run_of(eng, layer), "mixer", input=h_dev[:2].contiguous(), residual=out[:2])
        eng.run_part([StepEntry(rid, [0] * 7, [])], _run_of(eng, layer), "mixer", input=h_dev[2:].contiguous(), residual=out[2:])
        close(out, want, "float32", rid)
        eng.finish(rid)


FEED_FORWARDS = [(n, i, T) for n in sorted(CONFIGS) for i, l in enumerate(CONFIGS[n]["layers"]) if l["mlp"]
                 for T in ((97, 640) if n == "C" else (97,))]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name,layer,T", FEED_FORWARDS)
def test_feed_forward_alone(name, layer, T, dtype):
    """Dense with biases and limits; experts chosen by score + correction with the weights from the
    scores alone, identity experts, the shared expert behind its gate.  An input whose two outputs
    around the cut lie closer than rounding is left out."""
    from kipp_b200.engine import StepEntry
    cfg = CONFIGS[name]
    eng = engine_for(name, dtype, cuda_graphs=False)
    h_dev = (1.5 * _inputs(name, T, 300 + layer)).to("cuda", eng.dtype).contiguous()
    h_ref = h_dev.double().cpu()
    w = f64(weights_for(name, dtype))
    mlp, p = cfg["layers"][layer]["mlp"], f"l{layer}.mlp."
    want = P.feed_forward(mlp, w, p, h_ref)
    sure = torch.ones(T, dtype=torch.bool)
    if mlp["kind"] == "moe":
        choice = (torch.softmax(h_ref @ w[p + "router"].T, -1) + w[p + "correction"]).sort(-1, descending=True).values
        top = mlp["router"]["top"]
        if top < choice.shape[1]:
            sure = (choice[:, top - 1] - choice[:, top]) > 1e-4
        assert int(sure.sum()) > T // 2
    out = torch.zeros(T, cfg["width"], device="cuda")
    eng.run_part([StepEntry("f", [0] * T, [])], _run_of(eng, layer), "feed_forward", input=h_dev, residual=out)
    close(out[sure.cuda()], want[sure], dtype, f"{name} layer {layer}")
    # in bfloat16, sizes that are multiples of 8 run the gated activation inside the products (dense and
    # shared: one each; the experts: their grouped product); 32-bit and odd sizes use the kernel of its own
    fused = eng.info()["counters"]["glu_epilogues"]
    if dtype == "bfloat16" and name in ("A", "C"):
        assert fused == (1 if mlp["kind"] == "dense" else (2 if mlp.get("shared") else 1))
    elif dtype == "float32":
        assert fused == 0


def test_the_limits_and_identity_experts_show(tmp_path):
    """Inputs large enough that gate and up pass their limits, a correction that sends every token
    to an identity expert and one real expert, and a shared gate far from one half."""
    from kipp_b200.engine import Engine, StepEntry
    cfg = {"architecture": "Zunilorn", "vocab": 50, "width": 32, "norm": {"eps": 1e-5}, "streams": 2,
           "layers": [mamba_layer(2, 1, 8, 4, 2, 1, moe(3, 2, 2, 16, 0.5, 3.0, {"ff": 8, "limit": 0.25}))]}
    folder = write_folder(str(tmp_path / "m"), cfg, dict(seed=4, sigma=0.5, norm_jitter=0.1))
    set_tensors(folder, {"l0.mlp.correction": torch.tensor([0.0, 5.0, 0.0, 0.0, 6.0])})
    w = f64(read_weights(folder))
    h = 3.0 * torch.randn(40, 32, generator=torch.Generator().manual_seed(1), dtype=torch.float64)
    chosen, weights = P.route(cfg["layers"][0]["mlp"], w, "l0.mlp.", h)
    # (the weights sum to the scale, but for the 1e-20 in the divisor where the chosen scores are tiny)
    assert set(chosen.flatten().tolist()) == {1, 4} and float((weights.sum(1) - 3.0).abs().max()) < 1e-3
    g = h @ w["l0.mlp.e1.gate"].T
    assert float((g > 0.5).float().mean()) > 0.2          # the limit is at work
    want = P.feed_forward(cfg["layers"][0]["mlp"], w, "l0.mlp.", h)
    eng = Engine.from_folder(folder, dtype="float32", page_size=16, cache_tokens=64, max_requests=1, max_batch_tokens=64,
                             cuda_graphs=False)
    out = torch.zeros(40, 32, device="cuda")
    eng.run_part([StepEntry("f", [0] * 40, [])], 0, "feed_forward", input=h.float().cuda().contiguous(), residual=out)
    close(out, want, "float32", "limits and identity", factor=10)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name,layer", [("A", 0), ("A", 1), ("A", 3), ("B", 1), ("C", 2), ("D", 0), ("D", 1)])
def test_a_layer_alone_on_streams_that_differ(name, layer, dtype):
    """Hyper-connections: the copies of the stream start unequal here, so that the read weights,
    the mix matrix ([from, to]) and the write weights each show; without connections the plain sum."""
    from kipp_b200.engine import StepEntry
    cfg = CONFIGS[name]
    S, W, T = cfg.get("streams") or 1, cfg["width"], 21
    eng = engine_for(name, dtype, cuda_graphs=False)
    g = torch.Generator().manual_seed(900 + layer)
    xs = torch.randn(S, T, W, generator=g, dtype=torch.float64)
    x_dev = xs.float().cuda().contiguous()
    w = f64(weights_for(name, dtype))
    with torch.no_grad():
        want = P.layer_forward(cfg, w, layer, x_dev.double().cpu())
    eng.run_part([StepEntry("b", [0] * T, [])], _run_of(eng, layer), "block", residual=x_dev)
    close(x_dev.reshape(S * T, W), want.reshape(S * T, W), dtype, f"{name} layer {layer}", factor=3 if dtype == "bfloat16" else 1)


def test_stretched_frequencies_as_the_kernels_use_them():
    """One attention layer with no other mechanism in the way (no cap, sink far down, gate wide
    open): its output is the plain rotation's only if the stretched frequencies and the factor on
    cos and sin are what the equations say."""
    import tempfile
    from kipp_b200.engine import Engine, StepEntry
    rot = yarn(3000.0, 12, 5.0, 40, 6.0, 0.7)
    freq, mag = P.rotary_frequencies(rot)
    plain, _ = P.rotary_frequencies({"base": 3000.0, "dims": 12})
    assert abs(mag - (0.1 * math.log(5.0) + 1)) < 1e-12
    assert float(freq[0]) == float(plain[0]) and abs(float(freq[-1]) - float(plain[-1]) / 5.0) < 1e-12     # both ends of the ramp
    assert any(1e-9 < float(plain[i] - freq[i]) < float(plain[i]) * (1 - 1 / 5.0) - 1e-9 for i in range(6))  # and between
    cfg = {"architecture": "Zunilorn", "vocab": 40, "width": 32, "norm": {"eps": 1e-5},
           "layers": [attention_layer(2, 2, 16, 16, None, 1.5, None, rot)]}
    with tempfile.TemporaryDirectory() as tmp:
        folder = write_folder(tmp, cfg, dict(seed=8, sigma=0.4, norm_jitter=0.1))
        toks = random_tokens(40, 120, seed=2)
        with torch.no_grad():
            want = P.forward(cfg, read_weights(folder), toks)
            other = P.forward({**cfg, "layers": [attention_layer(2, 2, 16, 16, None, 1.5, None, {"base": 3000.0, "dims": 12})]},
                              read_weights(folder), toks)
        assert nmse(other, want) > 1e-4                    # the stretch is not a detail here
        eng = Engine.from_folder(folder, dtype="float32", page_size=16, cache_tokens=128, max_requests=1, max_batch_tokens=128)
        got = eng.step([StepEntry("r", toks, list(range(120)))], check=True)
        close(got, want, "float32", "stretched rotation")


# ------------------------------------------------------------------ whole models
LENGTH = {"A": 90, "B": 131, "C": 330, "D": 70}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_whole_prompt_and_every_way_of_cutting_it(name, dtype):
    """Whole; token by token from the very first token; portions down to two
    tokens: every position against the plain model, and (32-bit) the ways of
    cutting against one another."""
    from kipp_b200.engine import StepEntry
    toks = random_tokens(CONFIGS[name]["vocab"], LENGTH[name], seed=1)
    want = plain_logits(name, dtype, toks, whole_model=True)
    eng = engine_for(name, dtype)
    n = len(toks)
    whole = eng.step([StepEntry("w", toks, list(range(n)))], check=True).clone()
    eng.finish("w")
    close(whole, want, dtype, "whole")
    rows = [eng.step([StepEntry("t", [t], [0])]).clone() for t in toks]
    eng.synchronize()
    eng.finish("t")
    single = torch.cat(rows)
    close(single, want, dtype, "token by token")
    cut, at, i = [], 0, 0
    sizes = [2, 7, 2, 19, 3, 33, 2, 16, 17, 5, 64]
    while at < n:
        k = min(sizes[i % len(sizes)], n - at)
        cut.append(eng.step([StepEntry("c", toks[at:at + k], list(range(k)))]).clone())
        at, i = at + k, i + 1
    eng.synchronize()
    eng.finish("c")
    cut = torch.cat(cut)
    close(cut, want, dtype, "portions")
    if dtype == "float32":
        assert nmse(single.cpu(), whole.cpu()) <= 1e-10 and nmse(cut.cpu(), whole.cpu()) <= 1e-10


def test_the_stream_after_every_layer_run():
    """The sum of the copies after each run of the order (a looped layer counts each time)."""
    from kipp_b200.engine import StepEntry
    name = "A"
    cfg = CONFIGS[name]
    toks = random_tokens(cfg["vocab"], 25, seed=3)
    w = weights_for(name, "float32")
    sums = []
    with torch.no_grad():
        P.forward(cfg, w, toks, sums)
    eng = engine_for(name, "float32", cuda_graphs=False)
    S, T, W = cfg["streams"], len(toks), cfg["width"]
    x = torch.zeros(S, T, W, device="cuda")
    eng.run_part([StepEntry("e", toks, [])], 0, "embedding", residual=x[0])
    eng.finish("e")
    x[1:] = x[0]
    order = eng.spec.plan["order"]
    assert [o["layer"] for o in order] == [0, 1, 2, 1, 2, 3] and len({o["cache"] for o in order}) == len(order)
    for r in range(len(order)):
        eng.run_part([StepEntry(f"s{r}", [0] * T, [])], r, "block", residual=x)
        eng.finish(f"s{r}")
        assert nmse(x.sum(0).cpu(), sums[r]) <= 1e-9, f"run {r}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B"])
def test_unequal_requests_in_one_batch_with_pages_and_slots_used_again(name, dtype):
    """Six requests through two slots and a cache that holds two of them: portions
    of one beside decoded tokens of another; every request's logits are those of
    the request alone (state, kept inputs and pages of a slot's last owner are gone)."""
    from kipp_b200.engine import StepEntry
    vocab = CONFIGS[name]["vocab"]
    lengths = [37, 64, 5, 90, 18, 71]
    seqs = {f"r{i}": random_tokens(vocab, n, seed=20 + i) for i, n in enumerate(lengths)}
    eng = engine_for(name, dtype, cache_tokens=256, max_requests=2, max_batch_tokens=256)
    waiting, live, got = list(seqs), {}, {r: [] for r in seqs}
    tick = 0
    while waiting or live:
        while waiting and len(live) < 2:
            live[waiting.pop(0)] = 0
        entries = []
        for j, (rid, at) in enumerate(live.items()):
            toks = seqs[rid]
            head = max(len(toks) - 9, 1)
            k = 1 if at >= head else min([13, 2, 30, 5][(tick + j) % 4], head - at)
            entries.append(StepEntry(rid, toks[at:at + k], list(range(k))))
        logits = eng.step(entries, check=True)
        row = 0
        for e in entries:
            k = len(e.tokens)
            got[e.request].append(logits[row:row + k].clone())
            row += k
            live[e.request] += k
            if live[e.request] == len(seqs[e.request]):
                eng.finish(e.request)
                del live[e.request]
        eng.cache.check()
        tick += 1
    # 32-bit: against the plain model.  bfloat16: against the same engine running the request
    # alone in one step (what the batch, the slots and the pages must not do is change a
    # request's own result).
    alone = engine_for(name, dtype) if dtype == "bfloat16" else None
    for rid, toks in seqs.items():
        if alone is None:
            close(torch.cat(got[rid]), plain_logits(name, dtype, toks, whole_model=True), dtype, rid)
        else:
            want = alone.step([StepEntry(rid, toks, list(range(len(toks))))], check=True).clone()
            alone.finish(rid)
            close(torch.cat(got[rid]), (want.cpu(), None), dtype, rid)
    info = eng.info()
    assert info["free_slots"] == 2 and all(g["free_pages"] == g["pages"] for g in info["cache_groups"])


def test_a_request_left_out_of_a_step_goes_on_later():
    """Requests take turns: the one that pauses finds its state, its kept inputs and its
    pages as it left them, whatever the others did meanwhile."""
    from kipp_b200.engine import StepEntry
    name = "A"
    a, b = random_tokens(300, 50, seed=31), random_tokens(300, 44, seed=32)
    eng = engine_for(name, "float32")
    got_a, got_b = [], []
    got_a.append(eng.step([StepEntry("a", a[:7], list(range(7)))]).clone())
    got_b.append(eng.step([StepEntry("b", b[:30], list(range(30)))]).clone())
    lg = eng.step([StepEntry("a", a[7:20], list(range(13))), StepEntry("b", b[30:31], [0])]).clone()
    got_a.append(lg[:13]); got_b.append(lg[13:])
    got_b.append(eng.step([StepEntry("b", b[31:], list(range(13)))]).clone())
    got_a.append(eng.step([StepEntry("a", a[20:], list(range(30)))], check=True).clone())
    close(torch.cat(got_a), plain_logits(name, "float32", a), "float32", "a")
    close(torch.cat(got_b), plain_logits(name, "float32", b), "float32", "b")


# ------------------------------------------------------------------ edges, made to show
def needle_attention(scale=4.0, softcap=None, rot=None, vocab=97):
    """One attention layer whose softmax is sharp (a large score scale), so that a key wrongly
    seen or wrongly dropped moves the logits far more than rounding."""
    return {"architecture": "Zunilorn", "vocab": vocab, "width": 48, "norm": {"eps": 1e-5}, "residual_mult": 2.0, "streams": 2,
            "layers": [attention_layer(4, 2, 16, 8, None, scale, softcap, rot)]}


def _needle_run(cfg, folder, dtype, toks, edges, first=11):
    from kipp_b200.engine import Engine, StepEntry
    w = rounded(read_weights(folder), dtype)
    with torch.no_grad():
        want = P.forward(cfg, w, toks)
    n = len(toks)
    eng = Engine.from_folder(folder, dtype=dtype, page_size=16, cache_tokens=2 * n + 64, max_requests=2,
                             max_batch_tokens=max(n, 64))
    whole = eng.step([StepEntry("w", toks, list(range(n)))], check=True).clone()
    close(whole, want, dtype, "prompt")
    # the same positions decoded one by one after a prompt portion that ends inside the first page
    head = eng.step([StepEntry("d", toks[:first], list(range(first)))]).clone()
    rows = torch.cat([head] + [eng.step([StepEntry("d", [t], [0])]).clone() for t in toks[first:]])
    eng.synchronize()
    close(rows, want, dtype, "decoded")
    row_bound = BOUND[dtype] * (10 if dtype == "bfloat16" else 1)
    for pos in set(edges) & set(range(n)):
        for what, got in (("prompt", whole), ("decoded", rows)):
            e = nmse(got[pos:pos + 1].cpu(), want[pos:pos + 1])
            assert e <= row_bound, f"{what} position {pos}: NMSE {e:.3e}"
    return w, want


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_far_key_among_hundreds_and_the_edges_of_pages(dtype, tmp_path):
    """600 different tokens.  The query projection is the key projection behind a shift of the
    width's coordinates, and the embeddings of ten tokens of the first page are the shifted
    embeddings of the last ten: each of the last queries meets ONE key hundreds of positions back
    with a score far above all others (another token, with a value of its own).  Rows at page
    borders are judged one by one."""
    cfg = needle_attention(scale=1.0, vocab=640)
    folder = write_folder(str(tmp_path / "m"), cfg, dict(seed=77, sigma=0.3, norm_jitter=0.1))
    toks = torch.randperm(640, generator=torch.Generator().manual_seed(9))[:600].tolist()
    w0 = read_weights(folder)
    k, embed = w0["l0.mix.k"], w0["embed"].clone()           # k: [2 kv heads x 16, width]; head h reads kv head h // 2
    embed[toks[3:13]] = torch.roll(embed[toks[590:600]], 1, dims=1)
    q = torch.roll(k, -1, dims=1).view(2, 1, 16, 48).expand(2, 2, 16, 48).reshape(64, 48).clone()
    set_tensors(folder, {"l0.mix.q": q, "embed": embed, "l0.norm1": torch.ones(48)})
    w, want = _needle_run(cfg, folder, dtype, toks, edges=[15, 16, 17, 31, 32, 63, 64, 511, 512, 590, 599])
    # the far keys matter: without the first page's keys the last rows are other rows
    if dtype == "float32":
        with torch.no_grad():
            cut = P.forward(cfg, w, toks[16:])
        assert nmse(cut[-5:], want[-5:]) > 1e-3


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_the_sink_takes_its_share_and_the_cap_bends_the_scores(dtype, tmp_path):
    """A sink far above every score, and scores far beyond their cap: leaving either out shows."""
    cfg = needle_attention(scale=2.0, softcap=1.5)
    folder = write_folder(str(tmp_path / "m"), cfg, dict(seed=21, sigma=0.3, norm_jitter=0.1))
    set_tensors(folder, {"l0.mix.sink": torch.tensor([3.0, -2.0, 0.5, 6.0])})
    toks = random_tokens(97, 80, seed=4)
    w, want = _needle_run(cfg, folder, dtype, toks, edges=[0, 1, 15, 16, 79])
    if dtype == "float32":
        with torch.no_grad():
            no_sink = P.forward(cfg, {**w, "l0.mix.sink": torch.full((4,), -1e9)}, toks)
            no_cap = P.forward({**cfg, "layers": [attention_layer(4, 2, 16, 8, None, 2.0)]}, w, toks)
        assert nmse(no_sink, want) > 1e-3 and nmse(no_cap, want) > 1e-3


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_the_first_tokens_of_a_sequence(dtype):
    """Positions 0, 1, 2: one key and the sink; a convolution that reaches back beyond position 0."""
    from kipp_b200.engine import StepEntry
    for name in ("A", "D"):
        toks = random_tokens(CONFIGS[name]["vocab"], 3, seed=70)
        want = plain_logits(name, dtype, toks, whole_model=True)
        eng = engine_for(name, dtype)
        for cuts in ([3], [1, 1, 1], [1, 2], [2, 1]):
            rows, at = [], 0
            for k in cuts:
                rows.append(eng.step([StepEntry("f", toks[at:at + k], list(range(k)))], check=True).clone())
                at += k
            eng.finish("f")
            close(torch.cat(rows), want, dtype, f"{name} {cuts}", factor=5 if dtype == "bfloat16" else 1)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_state_that_keeps_the_first_token_through_long_decoding(dtype, tmp_path):
    """Decays next to one (A_log far down): what the first token wrote is still in the state 300
    tokens on, so a state lost, reset or carried to the wrong slot shows at the end."""
    from kipp_b200.engine import Engine, StepEntry
    cfg = {"architecture": "Zunilorn", "vocab": 60, "width": 32, "norm": {"eps": 1e-5}, "streams": 2, "residual_mult": 1.5,
           "layers": [mamba_layer(2, 1, 16, 8, 3, 2, None)]}
    folder = write_folder(str(tmp_path / "m"), cfg, dict(seed=6, sigma=0.4, norm_jitter=0.1))
    set_tensors(folder, {"l0.mix.A_log": torch.tensor([-9.0, -7.0]), "l0.mix.dt_bias": torch.tensor([-1.0, 0.5])})
    w = rounded(read_weights(folder), dtype)
    toks = random_tokens(60, 300, seed=13)
    other = [(toks[0] + 1) % 60] + toks[1:]
    with torch.no_grad():
        want, moved = P.forward(cfg, w, toks), P.forward(cfg, w, other)
    assert nmse(moved[-1:], want[-1:]) > 1e-5              # the first token still counts at the end
    eng = Engine.from_folder(folder, dtype=dtype, page_size=16, cache_tokens=1024, max_requests=2, max_batch_tokens=64)
    # two requests decode side by side; the second one's state must not leak into the first
    rows = []
    for i, t in enumerate(toks):
        lg = eng.step([StepEntry("x", [t], [0]), StepEntry("y", [other[i]], [0])]).clone()
        rows.append(lg)
    eng.synchronize()
    got = torch.stack(rows)                                 # [T, 2, vocab]
    close(got[:, 0], want, dtype, "first request")
    close(got[:, 1], moved, dtype, "second request")
    e = nmse(got[-1:, 0].cpu(), want[-1:])
    assert e <= BOUND[dtype] * (10 if dtype == "bfloat16" else 1), f"last row {e:.3e}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_of_a_batch_through_graphs(dtype):
    """Three requests of unequal prompts decode 150 tokens each in one batch (decode steps are
    graph replays); every row against the plain model."""
    from kipp_b200.engine import StepEntry
    name = "A"
    vocab = CONFIGS[name]["vocab"]
    seqs = [random_tokens(vocab, n, seed=40 + n) for n in (155, 171, 190)]
    heads = [5, 21, 40]
    eng = engine_for(name, dtype)
    got = [[] for _ in seqs]
    for i, (s, h) in enumerate(zip(seqs, heads)):
        got[i].append(eng.step([StepEntry(i, s[:h], list(range(h)))]).clone())
    for k in range(150):
        lg = eng.step([StepEntry(i, [s[h + k]], [0]) for i, (s, h) in enumerate(zip(seqs, heads))]).clone()
        for i in range(3):
            got[i].append(lg[i:i + 1])
    eng.synchronize()
    assert eng.graph_replays > 100
    for i, (s, h) in enumerate(zip(seqs, heads)):
        close(torch.cat(got[i]), plain_logits(name, dtype, s[:h + 150], whole_model=True), dtype, f"request {i}")


# ------------------------------------------------------------------ sizes nobody chose
def _drawn_config(seed):
    r = random.Random(seed)
    width = r.choice([32, 40, 48, 64, 72])
    streams = r.choice([None, 1, 2, 3, 5])
    cfg = {"architecture": "Zunilorn", "vocab": r.choice([64, 99, 130]), "width": width,
           "norm": {"eps": r.choice([1e-5, 1e-6])}}
    if streams is not None:
        cfg["streams"] = streams
    if r.random() < 0.7:
        cfg["residual_mult"] = r.choice([0.5, 0.9, 1.4])
    if r.random() < 0.7:
        cfg["logit_softcap"] = r.choice([5.0, 15.0, 40.0])

    def mlp():
        kind = r.choice(["none", "dense", "moe", "moe"])
        if kind == "none":
            return None
        if kind == "dense":
            return dense(r.choice([8, 20, 48]), r.choice([None, 0.8, 2.0]))
        experts, identity = r.choice([1, 2, 4, 7]), r.choice([None, 0, 1, 3])
        top = r.randint(1, min(3, experts + (identity or 0)))
        shared = r.choice([None, {"ff": r.choice([8, 24]), "limit": r.choice([1.0, 3.0])}])
        return moe(experts, identity, top, r.choice([8, 12, 32]), r.choice([None, 0.7, 1.5]), r.choice([None, 0.5, 2.0]), shared)

    layers = []
    for _ in range(r.randint(2, 4)):
        if r.random() < 0.5:
            kv = r.choice([1, 2])
            heads = kv * r.choice([1, 2, 3])
            dim = r.choice([4, 6, 8, 16, 32])
            rd = r.choice([0, 2, dim // 2 // 2 * 2, dim])
            rot = None
            if rd:
                rot = {"base": r.choice([100.0, 1e4, 5e5]), "dims": rd}
                if r.random() < 0.6:
                    rot = yarn(rot["base"], rd, r.choice([2.0, 8.0]), r.choice([16, 64, 512]), r.choice([4.0, 32.0]), r.choice([0.5, 1.0]))
            layers.append(attention_layer(heads, kv, dim, r.choice([dim, 4, 12, 24]), mlp(),
                                          r.choice([0.5, 1.0, 2.0]) * dim ** -0.5, r.choice([None, 3.0, 30.0]), rot))
        else:
            groups = r.choice([1, 2])
            heads = groups * r.choice([1, 2])
            vdim = r.choice([4, 6, 16, 32])
            parts = r.choice([p for p in (1, 2, heads, heads * 2) if (heads * vdim) % p == 0])
            layers.append(mamba_layer(heads, groups, vdim, r.choice([3, 8, 16, 24]), r.choice([1, 2, 3, 4]), parts, mlp()))
    cfg["layers"] = layers
    if r.random() < 0.6:
        a = r.randint(0, len(layers) - 1)
        cfg["loop"] = {"start": a, "stop": r.randint(a, len(layers)), "times": r.randint(1, 3)}
    return cfg


@pytest.mark.parametrize("seed", range(10))
def test_drawn_configurations(seed, tmp_path):
    """Ten configurations nobody chose: 32-bit against the plain model (whole, in portions, and two
    requests in one batch through one cache), bfloat16 whole against the plain model row by row."""
    from kipp_b200.engine import Engine, StepEntry
    cfg = _drawn_config(2000 + seed)
    folder = write_folder(str(tmp_path / "m"), cfg, dict(seed=seed, sigma=0.15, norm_jitter=0.15))
    a, b = random_tokens(cfg["vocab"], 75, seed=seed), random_tokens(cfg["vocab"], 40, seed=100 + seed)
    for dtype in ("float32", "bfloat16"):
        w = rounded(read_weights(folder), dtype)
        with torch.no_grad():
            want_a, want_b = P.forward(cfg, w, a), P.forward(cfg, w, b)
        eng = Engine.from_folder(folder, dtype=dtype, page_size=16, cache_tokens=192, max_requests=2, max_batch_tokens=128)
        whole = eng.step([StepEntry("w", a, list(range(len(a))))], check=True).clone()
        eng.finish("w")
        close(whole, (want_a, None), dtype, f"{cfg} whole")
        if dtype == "bfloat16":
            continue
        got_a, got_b, at_a, at_b, i = [], [], 0, 0, 0
        sizes_a, sizes_b = [2, 21, 1, 9, 30, 5, 7], [3, 1, 1, 17, 2, 16]
        while at_a < len(a) or at_b < len(b):
            entries = []
            if at_a < len(a):
                k = min(sizes_a[i % len(sizes_a)], len(a) - at_a)
                entries.append(StepEntry("a", a[at_a:at_a + k], list(range(k))))
            if at_b < len(b):
                k = min(sizes_b[i % len(sizes_b)], len(b) - at_b)
                entries.append(StepEntry("b", b[at_b:at_b + k], list(range(k))))
            lg, row = eng.step(entries, check=True), 0
            for e in entries:
                k = len(e.tokens)
                (got_a if e.request == "a" else got_b).append(lg[row:row + k].clone())
                row += k
                if e.request == "a":
                    at_a += k
                else:
                    at_b += k
            i += 1
        close(torch.cat(got_a), want_a, dtype, "a in portions beside b")
        close(torch.cat(got_b), want_b, dtype, "b in portions beside a")
        assert nmse(torch.cat(got_a).cpu(), whole.cpu()) <= 1e-10


# ------------------------------------------------------------------ the framework's entry points
@pytest.mark.parametrize("name", ["A", "C"])
def test_greedy_generation_through_the_scheduler(name):
    from kipp_b200.engine.llm import LLM
    vocab = CONFIGS[name]["vocab"]
    prompts = [random_tokens(vocab, n, seed=60 + n) for n in (3, 41, 17, 1, 26)]
    llm = LLM(model_folder(name), dtype="float32", kv_tokens=512, max_requests=3, max_batch_tokens=64, chunk=16)
    out = llm.generate(prompts, decode=12)
    w = weights_for(name, "float32")
    for prompt, result in zip(prompts, out):
        seq = list(prompt)
        with torch.no_grad():
            for _ in range(12):
                seq.append(int(P.forward(CONFIGS[name], w, seq)[-1].argmax()))
        assert result.tokens == seq[len(prompt):]


def test_the_command_line_generates_greedily_and_samples():
    name = "D"
    vocab = CONFIGS[name]["vocab"]
    a, b = random_tokens(vocab, 9, seed=5), random_tokens(vocab, 27, seed=6)
    proc = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "kipp"), "--model", model_folder(name),
                           "--prompt-ids", ",".join(map(str, a)), "--prompt-ids", ",".join(map(str, b)),
                           "--decode", "5", "--dtype", "float32", "--chunk", "16", "--top", "0"],
                          capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-2000:]
    got = [[int(t) for t in line.split("\t")[1].split()] for line in proc.stdout.strip().splitlines()]
    w = weights_for(name, "float32")
    for prompt, tokens in zip((a, b), got):
        seq = list(prompt)
        with torch.no_grad():
            for _ in range(5):
                seq.append(int(P.forward(CONFIGS[name], w, seq)[-1].argmax()))
        assert tokens == seq[len(prompt):]
    assert "prefill_tokens=36" in proc.stderr and "decode_tokens=10" in proc.stderr
    sampled = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "kipp"), "--random", "zunilorn-tiny",
                              "--prompt-ids", "1,2,3,4,5", "--decode", "8", "--temperature", "0.8", "--top-k", "20",
                              "--seed", "3", "--top", "0"], capture_output=True, text=True, timeout=600)
    assert sampled.returncode == 0, sampled.stderr[-2000:]
    tokens = [int(t) for t in sampled.stdout.strip().splitlines()[0].split("\t")[1].split()]
    assert len(tokens) == 8 and all(0 <= t < 320 for t in tokens)


def test_the_trace_program_runs_the_model_step_by_step(tmp_path):
    import numpy as np
    name = "A"
    vocab = CONFIGS[name]["vocab"]
    toks = random_tokens(vocab, 50, seed=77)
    steps = [{"step": 0, "entries": [{"id": "x", "tokens": toks[:30], "want": [0, 29]}], "end": []},
             {"step": 1, "entries": [{"id": "x", "tokens": toks[30:49], "want": []},
                                     {"id": "y", "tokens": toks[:2], "want": [1]}], "end": ["y"]},
             {"step": 2, "entries": [{"id": "x", "tokens": toks[49:], "want": [0]},
                                     {"id": "z", "tokens": toks[:3], "want": [2]}], "end": ["x", "z"]}]
    out = str(tmp_path / "out")
    proc = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", model_folder(name),
                           "--dtype", "float32", "--out", out, "--max-tokens", "128"],
                          input="".join(json.dumps(s) + "\n" for s in steps), capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stderr[-3000:]
    assert [l for l in proc.stdout.splitlines() if l.startswith("done")] == ["done 0", "done 1", "done 2"]
    want = plain_logits(name, "float32", toks)
    read = lambda i: torch.from_numpy(np.fromfile(os.path.join(out, f"{i}.f32"), dtype="<f4").reshape(-1, vocab))   # noqa: E731
    close(read(0), want[[0, 29]], "float32", "step 0")
    close(read(1), want[[1]], "float32", "step 1")
    close(read(2), want[[49, 2]], "float32", "step 2")
