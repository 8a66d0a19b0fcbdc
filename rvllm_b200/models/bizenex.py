"""Bizenex: from its configuration to a `ModelSpec`.

Every layer is a pre-norm block with a layer norm (weight and bias) before each sub-layer:
x <- x + mixer(norm1(x)), then, when the layer has a feed-forward, x <- x + ff(norm2(x)).
The mixer is a latent attention (one cached latent row per token, learned sinks, a sigmoid
gate before the output product; a layer may read the latent rows of an earlier one) or a
grouped-query attention without positions (unit-norm queries and keys, a query temperature
that grows with the logarithm of the position, one added to the softmax's denominator).  The
feed-forward is a mixture of SwiGLU experts with a sigmoid router and groups of experts.
The head is a matrix of its own after the model's layer norm; logits pass c tanh(. / c).

Tensor names: `embed`; `l<i>.norm1`, `.norm2` with the bias under the same name plus `.b`;
`l<i>.mix.*`, `l<i>.mlp.*`; `final.norm`, `final.norm.b`; `head`.
"""
from __future__ import annotations

from ..config.bizenex import ATTENTION, LATENT, BizenexConfig
from ..config.registry import register_architecture
from ..parts.spec import (AttentionSpec, BlockSpec, LatentAttentionSpec, LayerCall, ModelSpec,
                          MoESpec, NormSpec)

# the design has no longest context: positions are bounded only by what float32 counts exactly
MAX_POSITION = 1 << 24

_ATTENTION_NAMES = {"q_proj": "q", "k_proj": "k", "v_proj": "v", "out_proj": "o"}
_LATENT_NAMES = {"dkv_norm": "dkv.norm"}


def _norm_names(name):
    return {"weight": name, "bias": name + ".b"}


def build_spec(cfg: BizenexConfig) -> ModelSpec:
    hidden = cfg.width
    norm = NormSpec("layernorm", hidden, cfg.norm_eps)
    layers, order = [], []
    for i, l in enumerate(cfg.layers):
        p = f"l{i}."
        if l.type == LATENT:
            mixer = LatentAttentionSpec(
                "attention_latent", hidden, num_heads=l.heads, head_dim=l.dim, v_head_dim=l.vdim,
                kv_rank=l.kv_rank, scale=l.scale, norm_eps=cfg.norm_eps, sinks=True,
                out_gate=True, names=_LATENT_NAMES)
        else:
            mixer = AttentionSpec(
                "attention", hidden, num_heads=l.heads, num_kv_heads=l.kv_heads, head_dim=l.dim,
                qk_norm=NormSpec("rms_unit", l.dim, cfg.norm_eps), scale=l.scale,
                names=_ATTENTION_NAMES, v_head_dim=l.vdim, sink_score=0.0,
                q_temp=None if l.q_temp_coef is None else (l.q_temp_coef, l.q_temp_every))
        ffn = None
        norms = {"mixer": (norm, _norm_names(p + "norm1"))}
        if l.mlp is not None:
            ffn = MoESpec("moe", hidden, ffn_dim=l.mlp.ff, experts=l.mlp.experts, top=l.mlp.top,
                          groups=l.mlp.groups, keep=l.mlp.keep, group_top=2, score="sigmoid",
                          weight_eps=1e-20)
            norms["ffn"] = (norm, _norm_names(p + "norm2"))
        layers.append(BlockSpec("pre_norm", mixer, ffn, norms, mixer_prefix=p + "mix.",
                                ffn_prefix=p + "mlp."))
        order.append(LayerCall(i, l.kv_from if l.type == LATENT else None))
    return ModelSpec(
        architecture=cfg.architecture, vocab_size=cfg.vocab, hidden=hidden,
        max_position=MAX_POSITION, layers=tuple(layers), order=tuple(order),
        final_norm=norm, embedding_name="embed", final_norm_name=_norm_names("final.norm"),
        head_name="head", logit_softcap=cfg.logit_softcap)


register_architecture("Bizenex", BizenexConfig, build_spec, replace=True)
