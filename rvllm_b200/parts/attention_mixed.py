"""Grouped-query attention over a paged cache whose heads talk to one another, with the
options of `MixedAttentionSpec`: a value size of its own, a rotation of only the first
dimensions of a head, scores mixed over the heads before the softmax, a learned extra
term in the softmax's denominator, chunks that do not see one another, and a sigmoid gate
on the concatenated heads.

For a query at position p of head h, over the visible keys j (j <= p, j > p - window when
there is a window, floor(j / chunk) = floor(p / chunk) when there are chunks):

    s_g[j]  = scale * <q_g, k_kv(g)[j]>                      every head g
    s'_h[j] = sum_g M[h, g] s_g[j]                           (head_mix)
    w_h[j]  = exp(s'_h[j]) / (sum_j' exp(s'_h[j']) + exp(sink_h))        (sinks)
    o_h     = sum_j w_h[j] v_kv(h)[j]
    y       = W_o (concat_h o_h * sigmoid(W_g x))             (out_gate)

Because of the mixing a query's heads cannot be computed apart, so the kernels take all heads
of a query token together (`ops.paged_attention_mixed`); scores, mixing and softmax are
float32.  q, k, v and the gate are one matrix product; rotation and the cache write are one
kernel.  A call whose cache belongs to another call projects q and the gate only and reads the
other call's rotated keys and values with its own mask.
"""
from __future__ import annotations

import math

import torch

from .base import Mixer, PagedNeed, position_class, register_mixer
from .spec import MixedAttentionSpec, ParamDecl


class MixedAttention(Mixer):
    LOCAL = ("q", "k", "v", "o", "talk", "sink", "g")

    @staticmethod
    def _names(spec):
        return {k: spec.names.get(k, k) for k in MixedAttention.LOCAL}

    @staticmethod
    def _vd(spec):
        return spec.v_head_dim or spec.head_dim

    @staticmethod
    def params(spec: MixedAttentionSpec, owns_cache: bool = True):
        n = MixedAttention._names(spec)
        H, G, d, dv = spec.num_heads, spec.num_kv_heads, spec.head_dim, MixedAttention._vd(spec)
        p = {n["q"]: ParamDecl((H * d, spec.hidden), "linear"),
             n["o"]: ParamDecl((spec.hidden, H * dv), "linear")}
        if owns_cache:
            p[n["k"]] = ParamDecl((G * d, spec.hidden), "linear")
            p[n["v"]] = ParamDecl((G * dv, spec.hidden), "linear")
        if spec.head_mix:
            p[n["talk"]] = ParamDecl((H, H), "normal", mean=0.0, std=0.4)
        if spec.sinks:
            p[n["sink"]] = ParamDecl((H,), "normal", mean=0.0, std=1.0)
        if spec.out_gate:
            p[n["g"]] = ParamDecl((H * dv, spec.hidden), "linear")
        return p

    @staticmethod
    def cache_need(spec: MixedAttentionSpec):
        dv = MixedAttention._vd(spec)
        return PagedNeed(spec.num_kv_heads, spec.head_dim, spec.window, spec.chunk,
                         dv if dv != spec.head_dim else None)

    @staticmethod
    def workspace_bytes(spec: MixedAttentionSpec, ops, max_requests: int, max_context: int) -> int:
        sizer = getattr(ops, "attention_mixed_scratch_bytes", None)
        if sizer is None:
            return 0
        span = min(x for x in (max_context, spec.window, spec.chunk) if x)
        return sizer(max_requests, spec.num_heads, MixedAttention._vd(spec), span)

    def __init__(self, spec: MixedAttentionSpec, tensors, ops, dtype):
        if spec.num_heads % spec.num_kv_heads:
            raise ValueError(f"invalid attention head counts: {spec.num_heads} query, "
                             f"{spec.num_kv_heads} KV")
        self.spec = spec
        self.ops = ops
        self.dtype = dtype
        n = self._names(spec)
        H, G, d, dv = spec.num_heads, spec.num_kv_heads, spec.head_dim, self._vd(spec)
        q = tensors[n["q"]]
        self.has_kv = n["k"] in tensors
        gate = [tensors[n["g"]].to(q.dtype)] if spec.out_gate else []
        if self.has_kv:
            self.w_all = torch.cat([q, tensors[n["k"]].to(q.dtype), tensors[n["v"]].to(q.dtype)]
                                   + gate, dim=0).contiguous()
        else:
            self.w_all = None
        # without a cache of its own a call needs the queries and the gate only
        self.w_q_gate = torch.cat([q] + gate, dim=0).contiguous() \
            if (gate or not self.has_kv) else q.contiguous()
        self.w_out = tensors[n["o"]].contiguous()
        f32 = torch.float32
        self.head_mix = tensors[n["talk"]].to(f32).contiguous() if spec.head_mix else None
        self.sinks = tensors[n["sink"]].to(f32).contiguous() if spec.sinks else None
        self.position = position_class(spec.position.kind)(spec.position, q.device)
        if spec.position.kind not in ("rope_partial", "none"):
            raise ValueError("mixed attention takes a rope_partial rotation or none")
        self.scale = spec.scale if spec.scale is not None else 1.0 / math.sqrt(d)
        self.sizes = (H, G, d, dv)

    def forward(self, normed, ctx, cache):
        s = self.spec
        H, G, d, dv = self.sizes
        owns = cache.owns
        if owns and not self.has_kv:
            raise ValueError("attention: this call owns a cache but the block has no "
                             "key and value projections")
        group = ctx.groups[cache.group]
        rows = self.ops.linear(normed, self.w_all if owns else self.w_q_gate,
                               out_dtype=self.dtype)
        kv = G if owns else 0
        gate_off = (H * d + kv * (d + dv)) if s.out_gate else -1
        freq = self.position.frequencies() if s.position.kind == "rope_partial" else None
        self.ops.rope_partial_write(rows, H, kv, d, dv, freq, ctx.positions, group.slot_mapping,
                                    cache.k if owns else None, cache.v if owns else None)
        out = self.ops.new_rows(normed.shape[0], H * dv, self.dtype, normed.device)
        self.ops.paged_attention_mixed(rows, gate_off, H, G, d, dv, cache.k, cache.v, ctx, group,
                                       self.scale, s.window, s.chunk, self.head_mix, self.sinks,
                                       out)
        return self.ops.linear(out, self.w_out, out_dtype=self.dtype)


register_mixer("attention_mixed", MixedAttention)
