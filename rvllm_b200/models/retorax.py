"""Retorax: from its configuration to a `ModelSpec`.

Every layer is a pre-norm block with a layer norm (weight and bias) before and after each
sub-layer: x <- x + norm1b(mixer(norm1(x))), then, when the layer has a feed-forward,
x <- x + norm2b(ff(norm2(x))).  The mixer is a minGRU recurrence or a grouped-query
attention with a partial rotation, scores mixed over the heads, a sink term in the softmax,
chunks that do not see one another, and a sigmoid gate before the output product; an
attention layer may read the keys and values of an earlier one.  The feed-forward is
down(xielu(up(x))).  The head is the embedding table, after the model's layer norm.

Tensor names: `embed`; `l<i>.norm1`, `.norm1b`, `.norm2`, `.norm2b` with the bias under the
same name plus `.b`; `l<i>.mix.*`, `l<i>.mlp.*`; `final.norm`, `final.norm.b`.
"""
from __future__ import annotations

from ..config.registry import register_architecture
from ..config.retorax import ATTENTION, MINGRU, RetoraxConfig
from ..parts.spec import (BlockSpec, DenseSpec, LayerCall, MinGRUSpec, MixedAttentionSpec,
                          ModelSpec, NormSpec, PositionSpec)

# the design has no longest context: positions are bounded only by what float32 counts exactly
MAX_POSITION = 1 << 24


def _norm_names(name):
    return {"weight": name, "bias": name + ".b"}


def build_spec(cfg: RetoraxConfig) -> ModelSpec:
    hidden = cfg.width
    norm = NormSpec("layernorm", hidden, cfg.norm_eps)
    layers, order = [], []
    for i, l in enumerate(cfg.layers):
        p = f"l{i}."
        if l.type == MINGRU:
            mixer = MinGRUSpec("mingru", hidden, width=l.width)
        else:
            position = PositionSpec("rope_partial", l.dim, l.rot_base, MAX_POSITION, l.rot_dims) \
                if l.rot_dims else PositionSpec("none")
            mixer = MixedAttentionSpec(
                "attention_mixed", hidden, num_heads=l.heads, num_kv_heads=l.kv_heads,
                head_dim=l.dim, position=position, scale=l.scale, v_head_dim=l.vdim,
                chunk=l.mask_size, head_mix=True, sinks=True, out_gate=True)
        ffn = None
        norms = {"mixer": (norm, _norm_names(p + "norm1")),
                 "post_mixer": (norm, _norm_names(p + "norm1b"))}
        if l.mlp is not None:
            ffn = DenseSpec("dense", hidden, ffn_dim=l.mlp.ff, activation="xielu",
                            names={"up": "up", "down": "down", "act": "act"})
            norms["ffn"] = (norm, _norm_names(p + "norm2"))
            norms["post_ffn"] = (norm, _norm_names(p + "norm2b"))
        layers.append(BlockSpec("pre_norm", mixer, ffn, norms, mixer_prefix=p + "mix.",
                                ffn_prefix=p + "mlp."))
        order.append(LayerCall(i, l.kv_from if l.type == ATTENTION else None))
    return ModelSpec(
        architecture=cfg.architecture, vocab_size=cfg.vocab, hidden=hidden,
        max_position=MAX_POSITION, layers=tuple(layers), order=tuple(order),
        final_norm=norm, embedding_name="embed", final_norm_name=_norm_names("final.norm"),
        head_name=None)


register_architecture("Retorax", RetoraxConfig, build_spec, replace=True)
