"""Small Zunilorn configurations for the tests (sizes of their own, each unlike the
others in head counts, head sizes, streams, loops, rotation, experts and layer order)
and helpers to write them as model folders with random weights."""
from __future__ import annotations

import functools
import os
import tempfile

import torch


def moe(experts, identity, top, ff, limit=None, scale=None, shared=None) -> dict:
    router = {"experts": experts, "top": top}
    if identity is not None:
        router["identity"] = identity
    if scale is not None:
        router["scale"] = scale
    expert = {"ff": ff}
    if limit is not None:
        expert["limit"] = limit
    out = {"kind": "moe", "expert": expert, "router": router}
    if shared is not None:
        out["shared"] = shared
    return out


def dense(ff, limit=None) -> dict:
    out = {"kind": "dense", "ff": ff}
    if limit is not None:
        out["limit"] = limit
    return out


def attention_layer(heads, kv_heads, dim, vdim, mlp, scale, softcap=None, rot=None) -> dict:
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if softcap is not None:
        m["softcap"] = softcap
    if rot is not None:
        m["rot"] = rot
    return {"type": "attention", "mixer": m, "mlp": mlp}


def yarn(base, dims, factor, original, fast, slow) -> dict:
    return {"base": base, "dims": dims, "scaling": {"factor": factor, "original": original, "fast": fast, "slow": slow}}


def mamba_layer(heads, groups, vdim, state, conv, norm_groups, mlp) -> dict:
    return {"type": "mamba2", "mlp": mlp,
            "mixer": {"heads": heads, "groups": groups, "vdim": vdim, "state": state, "conv": conv, "norm_groups": norm_groups}}


CONFIGS = {
    # three streams, a looped span that holds both kinds of mixer, identity experts and a shared
    # expert, value heads wider than key heads, a part of every head rotated with stretched pairs
    "A": {"architecture": "Zunilorn", "vocab": 300, "width": 64, "norm": {"eps": 1e-5}, "residual_mult": 0.6,
          "streams": 3, "logit_softcap": 12.0, "loop": {"start": 1, "stop": 3, "times": 2},
          "layers": [mamba_layer(4, 2, 16, 24, 3, 2, dense(96, 1.5)),
                     attention_layer(4, 2, 16, 24, moe(5, 3, 2, 40, 1.0, 2.0, {"ff": 48, "limit": 2.0}), 0.3, 15.0,
                                     yarn(10000.0, 8, 2.0, 64, 8.0, 1.0)),
                     mamba_layer(2, 1, 32, 16, 4, 1, moe(5, 3, 2, 40, 1.0, 2.0, {"ff": 48, "limit": 2.0})),
                     attention_layer(2, 1, 32, 16, None, 0.2, 30.0, yarn(500.0, 32, 8.0, 32, 4.0, 0.5))]},
    # no streams (the plain residual sum), no loop, no caps, no multiplier, no limits; experts without
    # identity experts or a shared one; as many key heads as heads; a plain rotation and none; every
    # head its own group
    "B": {"architecture": "Zunilorn", "vocab": 257, "width": 96, "norm": {"eps": 3e-6},
          "layers": [attention_layer(3, 3, 16, 16, moe(6, None, 3, 32), 0.25, None, {"base": 77.0, "dims": 16}),
                     mamba_layer(3, 3, 32, 8, 2, 1, None),
                     attention_layer(6, 2, 16, 32, dense(64), 0.3),
                     mamba_layer(6, 1, 16, 40, 5, 6, moe(1, 2, 1, 24, 0.7, 0.5))]},
    # head sizes of 64 and 128, four streams, sixteen experts, a whole-head rotation, a loop of
    # one layer three times
    "C": {"architecture": "Zunilorn", "vocab": 512, "width": 128, "norm": {"eps": 1e-6}, "residual_mult": 0.4,
          "streams": 4, "logit_softcap": 25.0, "loop": {"start": 0, "stop": 1, "times": 3},
          "layers": [mamba_layer(4, 2, 64, 64, 4, 4, moe(16, 4, 4, 64, 1.2, 1.0, {"ff": 128, "limit": 3.0})),
                     attention_layer(4, 2, 64, 128, moe(16, 0, 4, 64, 1.0, 2.5), 0.125, 50.0,
                                     yarn(1e6, 64, 4.0, 128, 32.0, 1.0)),
                     attention_layer(2, 1, 128, 64, dense(256, 4.0), 0.09, 20.0, {"base": 10000.0, "dims": 128})]},
    # sizes that fit no vector width: an odd vocabulary, a width that is no multiple of 8, heads of
    # 6 and 5, a state of 5 rows, five taps, one stream with its connections, a router that takes
    # every output
    "D": {"architecture": "Zunilorn", "vocab": 101, "width": 100, "norm": {"eps": 2e-5}, "residual_mult": 1.3,
          "streams": 1, "logit_softcap": 8.0,
          "layers": [attention_layer(3, 1, 6, 5, moe(2, 1, 3, 7, 0.8, 1.0, {"ff": 9, "limit": 1.1}), 0.7, 5.0,
                                     yarn(100.0, 2, 3.0, 16, 2.0, 1.0)),
                     mamba_layer(3, 1, 7, 5, 5, 3, dense(11, 0.9)),
                     mamba_layer(2, 2, 9, 3, 1, 2, moe(4, 0, 1, 7, 1.0))]},
}
INIT = {"A": dict(seed=3, sigma=0.15, norm_jitter=0.2), "B": dict(seed=5, sigma=0.12, norm_jitter=0.1),
        "C": dict(seed=9, sigma=0.08, norm_jitter=0.15), "D": dict(seed=12, sigma=0.2, norm_jitter=0.1)}

_tmp = tempfile.TemporaryDirectory(prefix="kipp_b200_zunilorn_")


def write_folder(folder: str, cfg: dict, init: dict, dtype=torch.bfloat16) -> str:
    """Weights are stored in bfloat16, as this design's checkpoints are: the 32-bit engine, the
    16-bit engine (which keeps the small tensors of routers, sinks, decays and connections in
    float32) and the plain model then all start from the same numbers."""
    from kipp_b200.config import config_from_dict
    from kipp_b200.weights import write_random_model
    return write_random_model(folder, config_from_dict(cfg), init["seed"], sigma=init["sigma"],
                              norm_jitter=init["norm_jitter"], dtype=dtype)


@functools.lru_cache(maxsize=None)
def model_folder(name: str) -> str:
    return write_folder(os.path.join(_tmp.name, name), CONFIGS[name], INIT[name])


def random_tokens(vocab: int, n: int, seed: int) -> list:
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()


def set_tensors(folder: str, changed: dict) -> None:
    """Rewrite ``folder/model.safetensors`` with some tensors replaced."""
    from kipp_b200.weights.safetensors_io import write_safetensors
    from tiny import read_weights
    w = read_weights(folder)
    for name, t in changed.items():
        assert tuple(w[name].shape) == tuple(t.shape), name
        w[name] = t.to(w[name].dtype)
    write_safetensors(os.path.join(folder, "model.safetensors"), list(w.items()), metadata={"format": "pt"})
