"""The Retorax configuration: a list of layers, each a minGRU recurrence or an attention
whose heads are mixed, each with an optional dense feed-forward.

config.json of this design is nested:

    {"architecture": "Retorax", "vocab": V, "width": W, "norm": {"eps": e},
     "layers": [{"type": "mingru", "mixer": {"width": w}, "mlp": {"kind": "dense", "ff": F}},
                {"type": "attention",
                 "mixer": {"heads": H, "kv_heads": G, "dim": d, "vdim": dv, "scale": s,
                           "rot": {"dims": r, "base": b}, "mask": {"size": c},
                           "kv_from": j},            # optional: read layer j's keys and values
                 "mlp": null}]}

Every size and constant is read from the file; a key that is absent means the thing does
not exist (no mask: every earlier position is seen; no kv_from: the layer projects its own
keys and values; mlp null: the layer is its mixer alone).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, Optional, Tuple

from ..errors import ConfigError
from .base import Reader

MINGRU = "mingru"
ATTENTION = "attention"


@dataclass(frozen=True)
class RetoraxMlp:
    kind: str
    ff: int


@dataclass(frozen=True)
class RetoraxLayer:
    type: str
    mlp: Optional[RetoraxMlp]
    # mingru
    width: int = 0
    # attention
    heads: int = 0
    kv_heads: int = 0
    dim: int = 0
    vdim: int = 0
    scale: float = 0.0
    rot_dims: int = 0
    rot_base: float = 0.0
    mask_size: Optional[int] = None
    kv_from: Optional[int] = None


@dataclass(frozen=True)
class RetoraxConfig:
    architecture: str
    vocab: int
    width: int
    norm_eps: float
    layers: Tuple[RetoraxLayer, ...]
    torch_dtype: str = "bfloat16"
    extra: Dict[str, Any] = field(default_factory=dict, compare=False, hash=False)

    @classmethod
    def from_dict(cls, data: Dict[str, Any], where: str = "config.json") -> "RetoraxConfig":
        r = Reader(data, where)
        if not isinstance(data.get("layers"), list) or not data["layers"]:
            raise ConfigError(f"{where}: key 'layers' must be a non-empty list")
        if not isinstance(data.get("norm"), dict):
            raise ConfigError(f"{where}: missing key 'norm' (an object with 'eps')")
        layers = []
        for i, entry in enumerate(data["layers"]):
            at = f"{where}: layers[{i}]"
            lr = Reader(entry, at)
            kind = lr.str("type")
            mlp = None
            if entry.get("mlp") is not None:
                mr = Reader(entry["mlp"], at + ".mlp")
                mlp = RetoraxMlp(mr.str("kind"), mr.int("ff", minimum=1))
                if mlp.kind != "dense":
                    raise ConfigError(f"{at}.mlp: unknown kind {mlp.kind!r} (known: 'dense')")
            if not isinstance(entry.get("mixer"), dict):
                raise ConfigError(f"{at}: missing key 'mixer'")
            m = Reader(entry["mixer"], at + ".mixer")
            if kind == MINGRU:
                layers.append(RetoraxLayer(kind, mlp, width=m.int("width", minimum=1)))
            elif kind == ATTENTION:
                heads, kv = m.int("heads", minimum=1), m.int("kv_heads", minimum=1)
                if heads % kv:
                    raise ConfigError(f"{at}: invalid attention head counts: {heads} query, {kv} KV")
                dim = m.int("dim", minimum=1)
                rot_dims, rot_base = 0, 0.0
                if entry["mixer"].get("rot") is not None:
                    rr = Reader(entry["mixer"]["rot"], at + ".mixer.rot")
                    rot_dims, rot_base = rr.int("dims", minimum=0), rr.float("base")
                    if rot_dims % 2 or rot_dims > dim:
                        raise ConfigError(f"{at}: rot.dims {rot_dims} must be even and at most "
                                          f"dim {dim}")
                mask = None
                if entry["mixer"].get("mask") is not None:
                    mask = Reader(entry["mixer"]["mask"], at + ".mixer.mask").int("size", minimum=1)
                kv_from = m.optional_int("kv_from", minimum=0)
                if kv_from is not None:
                    if kv_from >= i or layers[kv_from].type != ATTENTION or \
                            layers[kv_from].kv_from is not None:
                        raise ConfigError(f"{at}: kv_from {kv_from} must name an earlier attention "
                                          f"layer with keys and values of its own")
                    src = layers[kv_from]
                    if (src.kv_heads, src.dim, src.vdim) != (kv, dim, m.int("vdim", minimum=1)):
                        raise ConfigError(f"{at}: kv_from {kv_from} has other head sizes")
                layers.append(RetoraxLayer(
                    kind, mlp, heads=heads, kv_heads=kv, dim=dim, vdim=m.int("vdim", minimum=1),
                    scale=m.float("scale"), rot_dims=rot_dims, rot_base=rot_base,
                    mask_size=mask, kv_from=kv_from))
            else:
                raise ConfigError(f"{at}: unknown type {kind!r} (known: {MINGRU!r}, {ATTENTION!r})")
        known = {"architecture", "architectures", "vocab", "width", "norm", "layers", "torch_dtype"}
        return cls(architecture=_name(data, where), vocab=r.int("vocab", minimum=1),
                   width=r.int("width", minimum=1),
                   norm_eps=Reader(data["norm"], where + ": norm").float("eps"),
                   layers=tuple(layers), torch_dtype=r.str("torch_dtype", "bfloat16"),
                   extra={k: v for k, v in data.items() if k not in known})

    def to_dict(self) -> Dict[str, Any]:
        d = dict(self.extra)
        layers = []
        for l in self.layers:
            if l.type == MINGRU:
                mixer: Dict[str, Any] = {"width": l.width}
            else:
                mixer = {"heads": l.heads, "kv_heads": l.kv_heads, "dim": l.dim, "vdim": l.vdim,
                         "scale": l.scale}
                if l.rot_dims:
                    mixer["rot"] = {"dims": l.rot_dims, "base": l.rot_base}
                if l.mask_size is not None:
                    mixer["mask"] = {"size": l.mask_size}
                if l.kv_from is not None:
                    mixer["kv_from"] = l.kv_from
            layers.append({"type": l.type, "mixer": mixer,
                           "mlp": None if l.mlp is None else {"kind": l.mlp.kind, "ff": l.mlp.ff}})
        d.update(architecture=self.architecture, vocab=self.vocab, width=self.width,
                 norm={"eps": self.norm_eps}, layers=layers, torch_dtype=self.torch_dtype)
        return d


def _name(data, where) -> str:
    name = data.get("architecture")
    if isinstance(name, str):
        return name
    archs = data.get("architectures")
    if isinstance(archs, list) and archs and isinstance(archs[0], str):
        return archs[0]
    raise ConfigError(f"{where}: missing key 'architecture'")
