"""The Bizenex configuration: a list of layers, each a latent attention or a grouped-query
attention without positions, each with an optional mixture-of-experts feed-forward.

config.json of this design is nested:

    {"architecture": "Bizenex", "vocab": V, "width": W, "norm": {"eps": e}, "logit_softcap": c,
     "layers": [{"type": "latent_attention",
                 "mixer": {"heads": H, "dim": d, "vdim": dv, "kv_rank": R, "scale": s,
                           "kv_from": j},            # optional: read layer j's latent rows
                 "mlp": {"kind": "moe", "expert": {"ff": F},
                         "router": {"experts": E, "top": k, "groups": {"count": g, "keep": m}}}},
                {"type": "attention",
                 "mixer": {"heads": H, "kv_heads": G, "dim": d, "vdim": dv, "scale": s,
                           "q_temp": {"coef": a, "every": n}},
                 "mlp": null}]}

Every size and constant is read from the file; a key that is absent means the thing does not
exist (no q_temp: queries keep their length; no kv_from: the layer makes its own latent rows;
no groups: every expert can be chosen; mlp null: the layer is its mixer alone; no
logit_softcap: logits stay as they are).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, Optional, Tuple

from ..errors import ConfigError
from .base import Reader

LATENT = "latent_attention"
ATTENTION = "attention"


@dataclass(frozen=True)
class BizenexMoe:
    ff: int
    experts: int
    top: int
    groups: int = 1
    keep: int = 1
    grouped: bool = False            # whether config.json had a "groups" object


@dataclass(frozen=True)
class BizenexLayer:
    type: str
    mlp: Optional[BizenexMoe]
    heads: int
    dim: int
    vdim: int
    scale: float
    # latent attention
    kv_rank: int = 0
    kv_from: Optional[int] = None
    # attention
    kv_heads: int = 0
    q_temp_coef: Optional[float] = None
    q_temp_every: int = 0


def _moe(entry, at) -> BizenexMoe:
    mr = Reader(entry, at)
    kind = mr.str("kind")
    if kind != "moe":
        raise ConfigError(f"{at}: unknown kind {kind!r} (known: 'moe')")
    if not isinstance(entry.get("expert"), dict) or not isinstance(entry.get("router"), dict):
        raise ConfigError(f"{at}: a mixture needs the objects 'expert' and 'router'")
    ff = Reader(entry["expert"], at + ".expert").int("ff", minimum=1)
    rr = Reader(entry["router"], at + ".router")
    experts = rr.int("experts", minimum=1)
    top = rr.int("top", minimum=1)
    groups, keep, grouped = 1, 1, False
    if entry["router"].get("groups") is not None:
        gr = Reader(entry["router"]["groups"], at + ".router.groups")
        groups, keep, grouped = gr.int("count", minimum=1), gr.int("keep", minimum=1), True
    if top > experts:
        raise ConfigError(f"{at}: top {top} is more than the {experts} experts")
    if experts % groups or keep > groups or keep * (experts // groups) < top:
        raise ConfigError(f"{at}: {experts} experts in {groups} groups of which {keep} are kept "
                          f"cannot give {top} experts a token")
    return BizenexMoe(ff, experts, top, groups, keep, grouped)


@dataclass(frozen=True)
class BizenexConfig:
    architecture: str
    vocab: int
    width: int
    norm_eps: float
    layers: Tuple[BizenexLayer, ...]
    logit_softcap: Optional[float] = None
    torch_dtype: str = "bfloat16"
    extra: Dict[str, Any] = field(default_factory=dict, compare=False, hash=False)

    @classmethod
    def from_dict(cls, data: Dict[str, Any], where: str = "config.json") -> "BizenexConfig":
        r = Reader(data, where)
        if not isinstance(data.get("layers"), list) or not data["layers"]:
            raise ConfigError(f"{where}: key 'layers' must be a non-empty list")
        if not isinstance(data.get("norm"), dict):
            raise ConfigError(f"{where}: missing key 'norm' (an object with 'eps')")
        layers = []
        for i, entry in enumerate(data["layers"]):
            at = f"{where}: layers[{i}]"
            kind = Reader(entry, at).str("type")
            mlp = _moe(entry["mlp"], at + ".mlp") if entry.get("mlp") is not None else None
            if not isinstance(entry.get("mixer"), dict):
                raise ConfigError(f"{at}: missing key 'mixer'")
            m = Reader(entry["mixer"], at + ".mixer")
            common = dict(heads=m.int("heads", minimum=1), dim=m.int("dim", minimum=1),
                          vdim=m.int("vdim", minimum=1), scale=m.float("scale"))
            if kind == LATENT:
                rank = m.int("kv_rank", minimum=1)
                kv_from = m.optional_int("kv_from", minimum=0)
                if kv_from is not None:
                    if kv_from >= i or layers[kv_from].type != LATENT or \
                            layers[kv_from].kv_from is not None:
                        raise ConfigError(f"{at}: kv_from {kv_from} must name an earlier latent "
                                          f"attention layer with latent rows of its own")
                    if layers[kv_from].kv_rank != rank:
                        raise ConfigError(f"{at}: kv_from {kv_from} has another kv_rank")
                layers.append(BizenexLayer(kind, mlp, kv_rank=rank, kv_from=kv_from, **common))
            elif kind == ATTENTION:
                kv = m.int("kv_heads", minimum=1)
                if common["heads"] % kv:
                    raise ConfigError(f"{at}: invalid attention head counts: {common['heads']} "
                                      f"query, {kv} KV")
                coef, every = None, 0
                if entry["mixer"].get("q_temp") is not None:
                    tr = Reader(entry["mixer"]["q_temp"], at + ".mixer.q_temp")
                    coef, every = tr.float("coef"), tr.int("every", minimum=1)
                layers.append(BizenexLayer(kind, mlp, kv_heads=kv, q_temp_coef=coef,
                                           q_temp_every=every, **common))
            else:
                raise ConfigError(f"{at}: unknown type {kind!r} (known: {LATENT!r}, {ATTENTION!r})")
        known = {"architecture", "architectures", "vocab", "width", "norm", "layers",
                 "logit_softcap", "torch_dtype"}
        name = data.get("architecture")
        if not isinstance(name, str):
            archs = data.get("architectures")
            if not (isinstance(archs, list) and archs and isinstance(archs[0], str)):
                raise ConfigError(f"{where}: missing key 'architecture'")
            name = archs[0]
        return cls(architecture=name, vocab=r.int("vocab", minimum=1),
                   width=r.int("width", minimum=1),
                   norm_eps=Reader(data["norm"], where + ": norm").float("eps"),
                   layers=tuple(layers), logit_softcap=r.optional_float("logit_softcap"),
                   torch_dtype=r.str("torch_dtype", "bfloat16"),
                   extra={k: v for k, v in data.items() if k not in known})

    def to_dict(self) -> Dict[str, Any]:
        d = dict(self.extra)
        layers = []
        for l in self.layers:
            mixer: Dict[str, Any] = {"heads": l.heads, "dim": l.dim, "vdim": l.vdim,
                                     "scale": l.scale}
            if l.type == LATENT:
                mixer["kv_rank"] = l.kv_rank
                if l.kv_from is not None:
                    mixer["kv_from"] = l.kv_from
            else:
                mixer["kv_heads"] = l.kv_heads
                if l.q_temp_coef is not None:
                    mixer["q_temp"] = {"coef": l.q_temp_coef, "every": l.q_temp_every}
            mlp = None
            if l.mlp is not None:
                router: Dict[str, Any] = {"experts": l.mlp.experts, "top": l.mlp.top}
                if l.mlp.grouped:
                    router["groups"] = {"count": l.mlp.groups, "keep": l.mlp.keep}
                mlp = {"kind": "moe", "expert": {"ff": l.mlp.ff}, "router": router}
            layers.append({"type": l.type, "mixer": mixer, "mlp": mlp})
        d.update(architecture=self.architecture, vocab=self.vocab, width=self.width,
                 norm={"eps": self.norm_eps}, layers=layers, torch_dtype=self.torch_dtype)
        if self.logit_softcap is not None:
            d["logit_softcap"] = self.logit_softcap
        return d
