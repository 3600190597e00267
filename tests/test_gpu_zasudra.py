"""Zasudra on the GPU against the plain float64 model (plain_zasudra.py): each
mechanism alone; whole prompts; token-by-token decoding from the first token;
portions down to two tokens; batches of unequal requests; pages and slots used
again; keys at the edges of blocks and of pages and far away; the sink; the
first tokens; long decoding through graphs; greedy generation through the
scheduler; the trace program."""
import json
import os
import subprocess
import sys

import pytest
import torch

import plain_zasudra as P
from tiny import nmse, read_weights
from zasudra_util import (CONFIGS, INIT, blocks_layer, gated_layer, model_folder, moe, random_tokens, set_tensors,
                          wkv_layer, write_folder)

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
# float32: the engine against the float64 plain model.  bfloat16: against the plain model with
# the matrices rounded to bfloat16 (activations are not rounded there, so the bound is that of
# 16-bit activations through a few layers).
BOUND = {"float32": 1e-9, "bfloat16": 2e-3}


def rounded(w, dtype):
    return {k: v.to(torch.bfloat16).float() for k, v in w.items()} if dtype == "bfloat16" else w


def weights_for(name, dtype):
    return rounded(read_weights(model_folder(name)), dtype)


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


# ------------------------------------------------------------------ each mechanism alone
ATTENTION_LAYERS = [(n, i) for n in sorted(CONFIGS) for i, l in enumerate(CONFIGS[n]["layers"])
                    if l["type"] != "wkv" and l["mixer"].get("kv_from") is None]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name,layer", ATTENTION_LAYERS)
def test_attention_mixers_alone(name, layer, dtype):
    """Both kinds of attention with keys of their own, in three portions: the later
    ones read the cache the earlier ones left."""
    from kipp_b200.engine import StepEntry
    cfg = CONFIGS[name]
    eng = engine_for(name, dtype, cuda_graphs=False)
    T = 150
    h_dev = _inputs(name, T, 100 + layer).to("cuda", eng.dtype).contiguous()
    h_ref = h_dev.double().cpu()
    w = {k: v.double() for k, v in weights_for(name, dtype).items()}
    mx, kind, eps, p = cfg["layers"][layer]["mixer"], cfg["layers"][layer]["type"], cfg["norm"]["eps"], f"l{layer}.mix."
    k, v = P.keys_and_values(w, p, mx, kind, h_ref, eps)
    want = P.attention(w, p, mx, kind, h_ref, eps, k, v)
    out = torch.zeros(T, cfg["width"], device="cuda")
    at = 0
    for n in (70, 1, 79):
        eng.run_part([StepEntry("a", [0] * n, [])], _run_of(eng, layer), "mixer", input=h_dev[at:at + n].contiguous(),
                     residual=out[at:at + n])
        at += n
    close(out, want, dtype, f"{name} layer {layer}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name,layer", [(n, i) for n in sorted(CONFIGS) for i, l in enumerate(CONFIGS[n]["layers"])
                                        if l["type"] == "wkv"])
def test_wkv_alone(name, layer, dtype):
    from kipp_b200.engine import StepEntry
    cfg = CONFIGS[name]
    eng = engine_for(name, dtype, cuda_graphs=False)
    T = 60
    h_dev = _inputs(name, T, 200 + layer).to("cuda", eng.dtype).contiguous()
    w = {k: v.double() for k, v in weights_for(name, dtype).items()}
    want = P.wkv(w, f"l{layer}.mix.", cfg["layers"][layer]["mixer"], h_dev.double().cpu(), cfg["norm"]["eps"])
    out = torch.zeros(T, cfg["width"], device="cuda")
    at = 0
    for n in (17, 1, 2, 40):                 # the state and the row before cross every cut
        eng.run_part([StepEntry("d", [0] * n, [])], _run_of(eng, layer), "mixer", input=h_dev[at:at + n].contiguous(),
                     residual=out[at:at + n])
        at += n
    close(out, want, dtype, f"{name} layer {layer}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name,layer,T", [("A", 0, 97), ("A", 3, 97), ("B", 0, 97), ("B", 1, 97), ("C", 0, 97), ("C", 4, 97),
                                          ("D", 0, 97), ("D", 1, 97),
                                          # long portions: in bfloat16 the experts' rows are sorted and padded
                                          # into tiles of one expert each (a grouped product); 641 leaves ragged tiles
                                          ("C", 0, 641), ("C", 3, 900), ("C", 4, 1024), ("B", 0, 300), ("D", 1, 400)])
def test_expert_mixture_alone(name, layer, T, dtype):
    """Top-k of all experts, of some, of one; the weights over the chosen only.  An input
    whose two best logits of the wanted rank lie closer than rounding is left out."""
    from kipp_b200.engine import StepEntry
    cfg = CONFIGS[name]
    eng = engine_for(name, dtype, cuda_graphs=False)
    h_dev = _inputs(name, T, 300 + layer).to("cuda", eng.dtype).contiguous()
    h_ref = h_dev.double().cpu()
    w = {k: v.double() for k, v in weights_for(name, dtype).items()}
    mlp, p = cfg["layers"][layer]["mlp"], f"l{layer}.mlp."
    want = P.expert_mixture(w, p, mlp, h_ref)
    z = (h_ref @ w[p + "router"].T + w[p + "router.b"]).sort(-1, descending=True).values
    top = mlp["router"]["top"]
    sure = torch.ones(T, dtype=torch.bool) if top == z.shape[1] else (z[:, top - 1] - z[:, top]) > 1e-4
    assert int(sure.sum()) > T // 2
    out = torch.zeros(T, cfg["width"], device="cuda")
    eng.run_part([StepEntry("f", [0] * T, [])], _run_of(eng, layer), "feed_forward", input=h_dev, residual=out)
    close(out[sure.cuda()], want[sure], dtype, f"{name} layer {layer}")


@pytest.mark.parametrize("name", ["A", "D"])
def test_pair_table_and_the_token_before_across_steps(name):
    """x = embed[token] + pair row; the row of a step's first token comes from the token
    the request's slot kept, the extra last row at position 0 only."""
    from kipp_b200.engine import StepEntry
    cfg = CONFIGS[name]
    eng = engine_for(name, "float32", cuda_graphs=False)
    toks = random_tokens(cfg["vocab"], 23, seed=5)
    w = {k: (v.double() if v.is_floating_point() else v) for k, v in weights_for(name, "float32").items()}
    want = P.embed(cfg, w, toks)
    x = torch.zeros(23, cfg["width"], device="cuda")
    at = 0
    for n in (1, 1, 9, 2, 10):
        eng.run_part([StepEntry("e", toks[at:at + n], [])], 0, "embedding", residual=x[at:at + n])
        at += n
    assert float((x.cpu().double() - want).abs().max()) <= 1e-6
    # another request in the slot the first one gave back starts from the extra row again
    eng.finish("e")
    y = torch.zeros(2, cfg["width"], device="cuda")
    eng.run_part([StepEntry("e2", toks[5:7], [])], 0, "embedding", residual=y)
    assert float((y.cpu().double() - P.embed(cfg, w, toks[5:7])).abs().max()) <= 1e-6


# ------------------------------------------------------------------ whole models
LENGTH = {"A": 90, "B": 131, "C": 560, "D": 70}


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


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B"])
def test_unequal_requests_in_one_batch_with_pages_and_slots_used_again(name, dtype):
    """Six requests through two slots and a cache that holds two of them: portions
    of one beside decoded tokens of another; every request's logits are those of
    the request alone (state, token before and pages of a slot's last owner are gone)."""
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
    # alone in one step (16-bit rounding through the routers makes some of these sequences move
    # by more than the bound under any small change, the plain model under weight noise too;
    # what the batch, the slots and the pages must not do is change a request's own result).
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
    """Requests take turns: the one that pauses finds its state, its token before and
    its pages as it left them, whatever the others did meanwhile."""
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
def needle_blocks(block, rot_dims=8):
    """One blocks layer whose attention is sharp (a large score scale), so that a key
    wrongly seen or wrongly dropped moves the logits far more than rounding."""
    return {"architecture": "Zasudra", "vocab": 97, "width": 48, "norm": {"eps": 1e-5}, "residual_mult": 2.0,
            "layers": [blocks_layer(3, 1, 16, block, rot_dims, None, scale=6.0)]}


def needle_causal(kv_from_too=False):
    layers = [gated_layer(4, 2, 16, 8, None, scale=3.0)]
    if kv_from_too:
        layers.append(gated_layer(4, 2, 16, 8, None, scale=2.0, kv_from=0))
    return {"architecture": "Zasudra", "vocab": 97, "width": 48, "norm": {"eps": 1e-5}, "residual_mult": 2.0, "layers": layers}


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
    # each position on its own: the edges are single rows.  (In bfloat16 the sharp scores that make
    # a wrong key show also magnify the rounding of q and k: ten times the bound for a single row.)
    row_bound = BOUND[dtype] * (10 if dtype == "bfloat16" else 1)
    for pos in set(edges) & set(range(n)):
        for what, got in (("prompt", whole), ("decoded", rows)):
            e = nmse(got[pos:pos + 1].cpu(), want[pos:pos + 1])
            assert e <= row_bound, f"{what} position {pos}: NMSE {e:.3e}"
    return w, want


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("block", [16, 17, 7, 33, 1, 64, 100])
def test_keys_just_inside_and_outside_a_block(block, dtype, tmp_path):
    cfg = needle_blocks(block)
    folder = write_folder(str(tmp_path / "m"), cfg, dict(seed=block * 100, sigma=0.3, norm_jitter=0.1))
    toks = random_tokens(97, 140, seed=block)
    edges = [0, 1, block - 1, block, block + 1, 2 * block - 1, 2 * block, 15, 16, 17, 139]
    w, want = _needle_run(cfg, folder, dtype, toks, edges)
    with torch.no_grad():
        # the oracle itself tells blocks that are one token off, or counted from elsewhere
        off = P.forward(needle_blocks(block + 1), w, toks)
        assert nmse(off[block:], want[block:]) > 3 * BOUND[dtype]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_many_narrow_heads(dtype, tmp_path):
    """36 heads in all (28 query, 4 key, 4 value) of 8 dims, seven query heads on a key head: the
    whole-projection norm over many heads; both kinds of layer."""
    cfg = {"architecture": "Zasudra", "vocab": 97, "width": 56, "norm": {"eps": 1e-5}, "residual_mult": 0.8,
           "layers": [blocks_layer(28, 4, 8, 24, 6, None, scale=0.6), gated_layer(28, 4, 8, 16, None, scale=0.5)]}
    folder = write_folder(str(tmp_path / "m"), cfg, dict(seed=19, sigma=0.25, norm_jitter=0.2))
    _needle_run(cfg, folder, dtype, random_tokens(97, 80, seed=9), [0, 1, 23, 24, 25, 79])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_far_key_among_hundreds_and_a_borrowed_cache(dtype, tmp_path):
    """Causal attention over 400 keys, sharp; the second layer reads the first one's keys
    and values with queries and a scale of its own."""
    cfg = needle_causal(kv_from_too=True)
    folder = write_folder(str(tmp_path / "m"), cfg, dict(seed=77, sigma=0.3, norm_jitter=0.1))
    toks = random_tokens(97, 400, seed=3)
    w, want = _needle_run(cfg, folder, dtype, toks, [0, 1, 2, 15, 16, 17, 255, 256, 257, 399], first=3)
    with torch.no_grad():
        # dropping the first 100 keys of every query would show
        far = P.forward(cfg, w, toks[100:])
        assert nmse(far[200:], want[300:]) > 3 * BOUND[dtype]


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("kind", ["learned", "unit"])
def test_the_sink_takes_its_share(kind, dtype, tmp_path):
    """Scores far below the sink: nearly all of the weight goes to the sink, which has no
    value.  A kernel without the sink, or with a scaled one, is off by a large factor."""
    cfg = needle_blocks(32) if kind == "learned" else needle_causal()
    cfg["layers"][0]["mixer"]["scale"] = 0.05
    cfg["layers"].append(wkv_layer(1, 8, 4, None))        # so that the size of layer 0's output matters
    cfg["residual_mult"] = 0.3
    folder = write_folder(str(tmp_path / "m"), cfg, dict(seed=8, sigma=0.3, norm_jitter=0.1))
    if kind == "learned":
        set_tensors(folder, {"l0.mix.sink": torch.tensor([4.0, -3.0, 1.5])})
    toks = random_tokens(97, 70, seed=4)
    _needle_run(cfg, folder, dtype, toks, [0, 1, 31, 32, 33, 69])


def _steady_tokens(name, n, seed):
    """n random tokens whose logits in the plain model move by less than a quarter of the 16-bit
    bound when every weight moves by a 16-bit rounding: with one or two tokens in the state, a
    head of the recurrence whose few terms cancel is divided by a root mean square near zero, and
    such a sequence tells nothing about the engine."""
    w = weights_for(name, "bfloat16")
    g = torch.Generator().manual_seed(seed)
    moved = {k: (v * (1 + 2.0 ** -9 * torch.randn(v.shape, generator=g)) if v.is_floating_point() else v) for k, v in w.items()}
    for s in range(seed, seed + 400, 10):
        toks = random_tokens(CONFIGS[name]["vocab"], n, seed=s)
        with torch.no_grad():
            if nmse(P.forward(CONFIGS[name], moved, toks), P.forward(CONFIGS[name], w, toks)) <= BOUND["bfloat16"] / 4:
                return toks
    raise AssertionError("no steady sequence found")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_the_first_tokens_of_a_sequence(dtype):
    """Prompts of one, two and three tokens, alone and in one batch: the extra pair row,
    the zero row before the first token, an empty state, a sink with a single key."""
    from kipp_b200.engine import StepEntry
    for name in ("A", "D"):
        vocab = CONFIGS[name]["vocab"]
        seqs = [_steady_tokens(name, n, 50 + n) for n in (1, 2, 3)]
        eng = engine_for(name, dtype)
        lg = eng.step([StepEntry(i, s, list(range(len(s)))) for i, s in enumerate(seqs)], check=True).clone()
        at = 0
        for i, s in enumerate(seqs):
            close(lg[at:at + len(s)], plain_logits(name, dtype, s, whole_model=True), dtype, f"{name} batch {i}")
            at += len(s)
            eng.finish(i)
        for i, s in enumerate(seqs):
            alone = eng.step([StepEntry("x", s, list(range(len(s))))], check=True).clone()
            eng.finish("x")
            close(alone, plain_logits(name, dtype, s, whole_model=True), dtype, f"{name} alone {i}")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_of_a_batch_through_graphs(dtype):
    """Two requests of unequal length decoded together for 150 steps (the steps are
    graph replays after the first); state, token before and blocks move with every token."""
    from kipp_b200.engine import StepEntry
    name = "B"
    vocab = CONFIGS[name]["vocab"]
    a, b = random_tokens(vocab, 170, seed=41), random_tokens(vocab, 155, seed=42)
    eng = engine_for(name, dtype)
    eng.step([StepEntry("a", a[:20], []), StepEntry("b", b[:5], [])])
    got_a, got_b = [], []
    for i in range(150):
        logits = eng.step([StepEntry("a", [a[20 + i]], [0]), StepEntry("b", [b[5 + i]], [0])])
        got_a.append(logits[0:1].clone())
        got_b.append(logits[1:2].clone())
    eng.synchronize()
    assert eng.graph_replays > 100
    close(torch.cat(got_a), (plain_logits(name, dtype, a)[20:], None), dtype, "a")
    close(torch.cat(got_b), (plain_logits(name, dtype, b)[5:], None), dtype, "b")


def _drawn_config(seed):
    """A configuration drawn from a seed: layer order, head counts, head sizes (odd ones too), value
    sizes, blocks, rotated dims, experts and choices, borrowed caches, optional keys left out."""
    import random
    r = random.Random(seed)
    width = r.choice([40, 52, 64, 72, 96])
    cfg = {"architecture": "Zasudra", "vocab": r.choice([89, 130, 257]), "width": width, "norm": {"eps": r.choice([1e-6, 1e-5, 3e-5])}}
    if r.random() < 0.7:
        cfg["residual_mult"] = r.choice([0.4, 0.9, 1.7])
    if r.random() < 0.7:
        cfg["logit_scale"] = r.choice([0.3, 2.0])
    if r.random() < 0.7:
        cfg["embedding"] = {"bigram": {"buckets": r.choice([1, 13, 211]), "mul_prev": r.choice([1, 29, 1000003]), "mul_cur": r.choice([1, 5, 40009])}}

    def mlp():
        if r.random() < 0.25:
            return None
        experts = r.choice([1, 2, 3, 7, 10])
        return moe(experts, r.randint(1, experts), r.choice([6, 16, 24, 40]))
    layers, lenders = [], []
    for i in range(r.randint(3, 6)):
        kind = r.choice(["attention", "attention_2", "wkv"])
        if kind == "wkv":
            layers.append(wkv_layer(r.choice([1, 2, 3]), r.choice([4, 6, 8, 16, 32]), r.choice([2, 5, 8]), mlp()))
            continue
        if kind == "attention_2" and lenders and r.random() < 0.5:
            j = r.choice(lenders)
            m = layers[j]["mixer"]
            layers.append(gated_layer(m["heads"], m["kv_heads"], m["dim"], m["vdim"], mlp(), scale=r.choice([0.2, 0.5]), kv_from=j))
            continue
        kv = r.choice([1, 2, 3])
        heads = kv * r.choice([1, 2, 4])
        dim = r.choice([4, 6, 8, 10, 16, 32, 64])
        scale = r.choice([0.5, 1.0, 2.0]) * dim ** -0.5
        if kind == "attention":
            rot = r.choice([0, 2, dim // 2 // 2 * 2, dim])
            layers.append(blocks_layer(heads, kv, dim, r.choice([0, 1, 3, 16, 21, 50]), rot, mlp(), base=r.choice([100.0, 1e4, 5e5]), scale=scale))
        else:
            layers.append(gated_layer(heads, kv, dim, r.choice([dim, 4, 12, 24]), mlp(), scale=scale))
            lenders.append(i)
    cfg["layers"] = layers
    return cfg


@pytest.mark.parametrize("seed", range(10))
def test_drawn_configurations(seed, tmp_path):
    """Ten configurations nobody chose: 32-bit against the plain model (whole, in portions, and two
    requests in one batch through one cache), bfloat16 whole against the plain model row by row."""
    from kipp_b200.engine import Engine, StepEntry
    cfg = _drawn_config(1000 + seed)
    folder = write_folder(str(tmp_path / "m"), cfg, dict(seed=seed, sigma=0.15, norm_jitter=0.15))
    a, b = random_tokens(cfg["vocab"], 75, seed=seed), random_tokens(cfg["vocab"], 40, seed=100 + seed)
    for dtype in ("float32", "bfloat16"):
        w = rounded(read_weights(folder), dtype)
        with torch.no_grad():
            want_a, want_b = P.forward(cfg, w, a), P.forward(cfg, w, b)
        eng = Engine.from_folder(folder, dtype=dtype, page_size=16, cache_tokens=192, max_requests=2, max_batch_tokens=128)
        whole = eng.step([StepEntry("w", a, list(range(len(a))))], check=True).clone()
        eng.finish("w")
        close(whole, (want_a, None), dtype, f"{cfg['layers']} whole")
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
    sampled = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "kipp"), "--random", "zasudra-tiny",
                              "--prompt-ids", "1,2,3,4,5", "--decode", "8", "--temperature", "0.8", "--top-k", "20",
                              "--seed", "3", "--top", "0"], capture_output=True, text=True, timeout=600)
    assert sampled.returncode == 0, sampled.stderr[-2000:]
    tokens = [int(t) for t in sampled.stdout.strip().splitlines()[0].split("\t")[1].split()]
    assert len(tokens) == 8 and all(0 <= t < 384 for t in tokens)


def test_the_trace_program_runs_the_model_step_by_step(tmp_path):
    import numpy as np
    name = "B"
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
