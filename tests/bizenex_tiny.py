"""Small Bizenex configurations for the tests, and helpers around them.

BZ_A and BZ_B differ in every size and constant: widths, head counts and group sizes (1, 2
and 3 query heads per key/value head), key sizes smaller and larger than value sizes, latent
ranks, scales, temperature steps below a page and across pages, experts in one, two and four
groups, layers with and without a feed-forward, readers of an earlier layer's latent rows
with other head counts than their source, eps, vocabulary, with and without a cap on the
logits.  BZ_C has sizes that no vector access divides.
"""
import copy
import os

import numpy as np
import torch

from rvllm_b200.config import config_from_dict
from rvllm_b200.weights import write_random_model


def _latent(heads, dim, vdim, rank, scale, kv_from=None):
    m = {"heads": heads, "dim": dim, "vdim": vdim, "kv_rank": rank, "scale": scale}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return m


def _attn(heads, kv, dim, vdim, scale, temp=None):
    m = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": scale}
    if temp is not None:
        m["q_temp"] = {"coef": temp[0], "every": temp[1]}
    return m


def _moe(ff, experts, top, groups=None):
    if ff is None:
        return None
    router = {"experts": experts, "top": top}
    if groups is not None:
        router["groups"] = {"count": groups[0], "keep": groups[1]}
    return {"kind": "moe", "expert": {"ff": ff}, "router": router}


BZ_A = {
    "architecture": "Bizenex", "vocab": 300, "width": 96, "norm": {"eps": 1e-5},
    "logit_softcap": 8.0,
    "layers": [
        {"type": "latent_attention", "mixer": _latent(4, 16, 24, 32, 0.3),
         "mlp": _moe(64, 6, 2, (3, 2))},
        {"type": "attention", "mixer": _attn(6, 2, 32, 16, 0.4, (0.7, 5)),
         "mlp": _moe(48, 4, 1)},
        {"type": "latent_attention", "mixer": _latent(2, 24, 8, 32, 0.2, kv_from=0), "mlp": None},
        {"type": "attention", "mixer": _attn(3, 3, 16, 32, 0.5), "mlp": _moe(32, 8, 3, (4, 2))},
        {"type": "latent_attention", "mixer": _latent(4, 16, 24, 32, 0.3, kv_from=0),
         "mlp": _moe(64, 6, 4, (2, 2))},
    ],
}

BZ_B = {
    "architecture": "Bizenex", "vocab": 257, "width": 64, "norm": {"eps": 1e-3},
    "layers": [
        {"type": "attention", "mixer": _attn(4, 1, 16, 48, 1.5, (0.25, 21)),
         "mlp": _moe(96, 9, 3, (3, 1))},
        {"type": "latent_attention", "mixer": _latent(3, 32, 16, 48, 0.15),
         "mlp": _moe(32, 2, 2)},
        {"type": "latent_attention", "mixer": _latent(5, 8, 40, 16, 0.4), "mlp": None},
    ],
}

# sizes that no vector access divides: keys of 10, values of 6, a rank of 14, a width of 50
BZ_C = {
    "architecture": "Bizenex", "vocab": 99, "width": 50, "norm": {"eps": 1e-5},
    "logit_softcap": 30.0,
    "layers": [
        {"type": "latent_attention", "mixer": _latent(3, 10, 6, 14, 0.3),
         "mlp": _moe(34, 5, 2, (5, 3))},
        {"type": "attention", "mixer": _attn(3, 3, 10, 6, 0.6, (1.0, 1)), "mlp": _moe(22, 3, 3)},
    ],
}

# sizes the tensor-core kernels take in bfloat16
BZ_D = {
    "architecture": "Bizenex", "vocab": 200, "width": 128, "norm": {"eps": 1e-6},
    "logit_softcap": 20.0,
    "layers": [
        {"type": "latent_attention", "mixer": _latent(8, 32, 48, 64, 0.18),
         "mlp": _moe(128, 8, 2, (4, 2))},
        {"type": "attention", "mixer": _attn(12, 3, 64, 64, 0.2, (0.4, 16)),
         "mlp": _moe(64, 16, 4, (4, 3))},
        {"type": "latent_attention", "mixer": _latent(4, 64, 32, 64, 0.12, kv_from=0),
         "mlp": _moe(128, 4, 2)},
        {"type": "attention", "mixer": _attn(4, 4, 32, 32, 0.3), "mlp": None},
    ],
}

# larger heads and ranks: a rank beyond the tensor-core kernels' head sizes, key and value heads of
# 128, many experts of a size that no tile divides, a reader right after its source and one later
BZ_E = {
    "architecture": "Bizenex", "vocab": 500, "width": 256, "norm": {"eps": 1e-6},
    "logit_softcap": 10.0,
    "layers": [
        {"type": "attention", "mixer": _attn(4, 4, 128, 128, 0.3, (0.3, 50)),
         "mlp": _moe(200, 32, 6, (8, 4))},
        {"type": "latent_attention", "mixer": _latent(8, 64, 64, 192, 0.1),
         "mlp": _moe(72, 64, 8, (4, 1))},
        {"type": "latent_attention", "mixer": _latent(3, 32, 96, 192, 0.2, kv_from=1), "mlp": None},
        {"type": "attention", "mixer": _attn(16, 2, 32, 64, 0.25), "mlp": _moe(200, 32, 6, (8, 4))},
        {"type": "latent_attention", "mixer": _latent(8, 64, 64, 192, 0.1, kv_from=1),
         "mlp": _moe(128, 3, 1)},
    ],
}

CONFIGS = {"A": BZ_A, "B": BZ_B, "C": BZ_C, "D": BZ_D, "E": BZ_E}
SEEDS = {"A": 21, "B": 22, "C": 23, "D": 24, "E": 25}


def config(name: str) -> dict:
    return copy.deepcopy(CONFIGS[name])


def write(folder: str, name: str) -> str:
    return write_random_model(os.path.join(folder, "bz_" + name), config_from_dict(config(name)),
                              SEEDS[name])


def read_tensors(folder: str):
    """The file's tensors by name as float64 arrays, through the package's format reader."""
    from rvllm_b200.weights.safetensors_io import SafetensorsFile
    f = SafetensorsFile(os.path.join(folder, "model.safetensors"))
    return {n: f.tensor(n).to(torch.float64).numpy().copy() for n in f.names()}


def plain_logits(folder: str, name: str, tokens, cfg=None, tensors=None):
    import plain_bizenex
    out = plain_bizenex.forward(cfg or config(name), tensors or read_tensors(folder), tokens)
    return torch.from_numpy(np.asarray(out))
