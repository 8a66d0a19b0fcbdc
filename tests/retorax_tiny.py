"""Small Retorax configurations for the tests, and helpers around them.

RX_A and RX_B differ in every size and constant: widths of the model and of the recurrences,
head counts and group sizes (1, 2 and 3 query heads per key/value head), key and value sizes
(smaller, larger), how many dimensions turn (a few, all), chunk sizes (below a page, across
pages, different between a layer and the layer whose keys it reads), layers with and without
a feed-forward, eps, vocabulary.  RX_C has one key/value head, no mask and a chunk of one page.
"""
import copy
import os

import torch

from rvllm_b200.config import config_from_dict
from rvllm_b200.weights import write_random_model


def _attn(heads, kv, dim, vdim, scale, rot, base, mask, kv_from=None):
    m = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": scale,
         "rot": {"dims": rot, "base": base}}
    if mask is not None:
        m["mask"] = {"size": mask}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return m


def _ff(n):
    return None if n is None else {"kind": "dense", "ff": n}


RX_A = {
    "architecture": "Retorax", "vocab": 300, "width": 96, "norm": {"eps": 1e-5},
    "layers": [
        {"type": "mingru", "mixer": {"width": 80}, "mlp": _ff(160)},
        {"type": "attention", "mixer": _attn(6, 2, 32, 16, 0.2, 8, 5000.0, 24), "mlp": _ff(128)},
        {"type": "attention", "mixer": _attn(6, 2, 32, 16, 0.3, 8, 5000.0, 40, kv_from=1),
         "mlp": None},
        {"type": "mingru", "mixer": {"width": 64}, "mlp": None},
        {"type": "attention", "mixer": _attn(6, 2, 32, 16, 0.2, 8, 5000.0, 24, kv_from=1),
         "mlp": _ff(64)},
    ],
}

RX_B = {
    "architecture": "Retorax", "vocab": 257, "width": 64, "norm": {"eps": 1e-3},
    "layers": [
        {"type": "attention", "mixer": _attn(4, 4, 16, 48, 0.31, 16, 100.0, 7), "mlp": _ff(96)},
        {"type": "mingru", "mixer": {"width": 128}, "mlp": _ff(32)},
        {"type": "attention", "mixer": _attn(4, 4, 16, 48, 0.25, 16, 100.0, 7, kv_from=0),
         "mlp": _ff(96)},
        {"type": "attention", "mixer": _attn(3, 1, 24, 8, 0.15, 4, 777.0, 33), "mlp": None},
    ],
}

RX_C = {
    "architecture": "Retorax", "vocab": 128, "width": 32, "norm": {"eps": 1e-6},
    "layers": [
        {"type": "attention", "mixer": _attn(2, 1, 64, 64, 0.125, 32, 10000.0, None), "mlp": _ff(48)},
        {"type": "mingru", "mixer": {"width": 32}, "mlp": _ff(48)},
        {"type": "attention", "mixer": _attn(5, 5, 8, 24, 0.35, 2, 50.0, 16), "mlp": _ff(48)},
    ],
}

# head counts in multiples of 8: in bfloat16 its prompt portions take the tensor-core kernel
RX_D = {
    "architecture": "Retorax", "vocab": 200, "width": 64, "norm": {"eps": 1e-5},
    "layers": [
        {"type": "attention", "mixer": _attn(8, 2, 32, 16, 0.2, 16, 3000.0, 48), "mlp": _ff(64)},
        {"type": "mingru", "mixer": {"width": 48}, "mlp": None},
        {"type": "attention", "mixer": _attn(8, 2, 32, 16, 0.2, 16, 3000.0, 48, kv_from=0), "mlp": None},
        {"type": "attention", "mixer": _attn(16, 16, 16, 32, 0.3, 8, 99.0, 20), "mlp": _ff(96)},
    ],
}

# sizes that no vector access divides: keys of 10, values of 6, three heads, a width of 50
RX_E = {
    "architecture": "Retorax", "vocab": 99, "width": 50, "norm": {"eps": 1e-5},
    "layers": [
        {"type": "mingru", "mixer": {"width": 30}, "mlp": _ff(70)},
        {"type": "attention", "mixer": _attn(3, 3, 10, 6, 0.3, 2, 10.0, 19), "mlp": _ff(34)},
    ],
}

CONFIGS = {"A": RX_A, "B": RX_B, "C": RX_C, "D": RX_D, "E": RX_E}
SEEDS = {"A": 11, "B": 12, "C": 13, "D": 14, "E": 15}


def config(name: str) -> dict:
    return copy.deepcopy(CONFIGS[name])


def write(folder: str, name: str) -> str:
    return write_random_model(os.path.join(folder, "rx_" + name), config_from_dict(config(name)),
                              SEEDS[name])


def read_tensors(folder: str):
    """The file's tensors by name, through the package's reader (a format reader, no model)."""
    from rvllm_b200.weights.safetensors_io import SafetensorsFile
    f = SafetensorsFile(os.path.join(folder, "model.safetensors"))
    return {n: f.tensor(n).clone() for n in f.names()}


def plain_logits(folder: str, name: str, tokens, dtype=torch.float64):
    import plain_retorax
    return plain_retorax.forward(config(name), read_tensors(folder), tokens, dtype)
