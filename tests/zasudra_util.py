"""Small Zasudra configurations for the tests (sizes of their own, each unlike the
others in head counts, head sizes, blocks, rotation, experts and layer order) and
helpers to write them as model folders with random weights."""
from __future__ import annotations

import functools
import os
import tempfile

import torch


def moe(experts: int, top: int, ff: int) -> dict:
    return {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}


def blocks_layer(heads, kv_heads, dim, block, rot_dims, mlp, base=10000.0, scale=None, kv_from=None) -> dict:
    """type 'attention': the values are the keys, blocks of positions, a learned sink."""
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim,
         "scale": scale if scale is not None else dim ** -0.5}
    if block:
        m["mask"] = {"size": block}
    if rot_dims:
        m["rot"] = {"base": base, "dims": rot_dims}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return {"type": "attention", "mixer": m, "mlp": mlp}


def gated_layer(heads, kv_heads, dim, vdim, mlp, scale=None, kv_from=None) -> dict:
    """type 'attention_2': W_v, every earlier key, a sink of score 0, a gate per head."""
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim,
         "scale": scale if scale is not None else dim ** -0.5}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return {"type": "attention_2", "mixer": m, "mlp": mlp}


def wkv_layer(heads, dim, rank, mlp) -> dict:
    return {"type": "wkv", "mixer": {"heads": heads, "dim": dim, "decay_rank": rank}, "mlp": mlp}


CONFIGS = {
    # a block of one page, value heads wider than key heads, a layer that borrows keys and values,
    # a router that takes every expert, layers without a feed-forward
    "A": {"architecture": "Zasudra", "vocab": 300, "width": 64, "norm": {"eps": 1e-5}, "residual_mult": 0.7,
          "logit_scale": 1.5, "embedding": {"bigram": {"buckets": 97, "mul_prev": 31, "mul_cur": 7}},
          "layers": [blocks_layer(4, 2, 16, 16, 8, moe(5, 2, 40), scale=0.3),
                     wkv_layer(2, 16, 8, moe(5, 2, 40)),
                     gated_layer(4, 4, 16, 24, None, scale=0.25),
                     gated_layer(4, 4, 16, 24, moe(3, 3, 24), scale=0.4, kv_from=2),
                     wkv_layer(1, 32, 5, None)]},
    # no pair table, no multiplier and no logit scale (both 1); one expert; blocks that fit no page;
    # a blocks layer without rotation, and one that borrows rotated keys under a mask of its own
    "B": {"architecture": "Zasudra", "vocab": 257, "width": 96, "norm": {"eps": 3e-6},
          "layers": [gated_layer(2, 1, 8, 8, moe(1, 1, 40), scale=0.5),
                     blocks_layer(6, 2, 16, 7, 12, moe(9, 4, 16), base=77.0, scale=0.3),
                     blocks_layer(6, 2, 16, 20, 12, None, base=77.0, scale=0.2, kv_from=1),
                     wkv_layer(3, 8, 16, moe(2, 1, 8)),
                     blocks_layer(3, 3, 8, 0, 0, moe(9, 4, 16), scale=0.4)]},
    # head sizes of 64 and 128, blocks of 64, a whole-head rotation, sixteen experts
    "C": {"architecture": "Zasudra", "vocab": 512, "width": 128, "norm": {"eps": 1e-6}, "residual_mult": 0.25,
          "logit_scale": 0.8, "embedding": {"bigram": {"buckets": 1021, "mul_prev": 1, "mul_cur": 1}},
          "layers": [blocks_layer(4, 2, 64, 64, 64, moe(16, 4, 64), base=1e6, scale=0.125),
                     gated_layer(2, 1, 128, 64, moe(16, 4, 64), scale=0.09),
                     wkv_layer(2, 64, 32, None),
                     blocks_layer(2, 2, 128, 48, 32, moe(4, 2, 128), scale=0.1),
                     gated_layer(2, 1, 128, 64, moe(16, 1, 64), scale=0.2, kv_from=1)]},
    # sizes that fit no vector width: an odd vocabulary, a width that is no multiple of 8, head
    # sizes of 6 and 5, three heads on one key/value head, a table of one bucket
    "D": {"architecture": "Zasudra", "vocab": 101, "width": 100, "norm": {"eps": 2e-5}, "residual_mult": 1.3,
          "embedding": {"bigram": {"buckets": 1, "mul_prev": 5, "mul_cur": 3}},
          "layers": [blocks_layer(3, 1, 6, 9, 2, moe(4, 1, 7), scale=0.7),
                     gated_layer(3, 3, 6, 5, moe(4, 3, 7), scale=0.9),
                     wkv_layer(2, 6, 3, moe(3, 2, 10))]},
}
INIT = {"A": dict(seed=3, sigma=0.15, norm_jitter=0.2), "B": dict(seed=5, sigma=0.12, norm_jitter=0.1),
        "C": dict(seed=9, sigma=0.08, norm_jitter=0.15), "D": dict(seed=12, sigma=0.2, norm_jitter=0.1)}

_tmp = tempfile.TemporaryDirectory(prefix="kipp_b200_zasudra_")


def write_folder(folder: str, cfg: dict, init: dict, dtype=torch.float32) -> str:
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
