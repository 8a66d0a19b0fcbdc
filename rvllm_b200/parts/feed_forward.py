"""SwiGLU feed-forward: down(silu(gate(x)) * up(x)) (the reference's `swiglu_ffn`,
src/model.rs:320-335).

gate and up are stored as one [2F, hidden] matrix so that they are one matrix
product; the activation kernel reads both halves of its output row.  (The reference
runs two products and `silu_gate_multiply.cu`, src/cuda/model.rs:740-760.)
"""
from __future__ import annotations

import torch

from .base import FeedForward, register_feed_forward
from .spec import DenseSpec, ParamDecl, SwiGLUSpec


class SwiGLU(FeedForward):
    @staticmethod
    def params(spec: SwiGLUSpec):
        n = spec.names
        return {
            n.get("gate", "gate.weight"): ParamDecl((spec.ffn_dim, spec.hidden), "linear"),
            n.get("up", "up.weight"): ParamDecl((spec.ffn_dim, spec.hidden), "linear"),
            n.get("down", "down.weight"): ParamDecl((spec.hidden, spec.ffn_dim), "linear"),
        }

    def __init__(self, spec: SwiGLUSpec, tensors, ops, dtype):
        self.spec = spec
        self.ops = ops
        self.dtype = dtype
        n = spec.names
        gate = tensors[n.get("gate", "gate.weight")]
        up = tensors[n.get("up", "up.weight")]
        self.gate_up = torch.cat([gate, up.to(gate.dtype)], dim=0).contiguous()
        self.down = tensors[n.get("down", "down.weight")].contiguous()

    def forward(self, normed, ctx):
        gate_up = self.ops.linear(normed, self.gate_up, out_dtype=self.dtype)
        act = self.ops.new_rows(normed.shape[0], self.spec.ffn_dim, self.dtype, normed.device)
        self.ops.swiglu(gate_up, act)
        return self.ops.linear(act, self.down, out_dtype=self.dtype)


register_feed_forward("swiglu", SwiGLU)


class Dense(FeedForward):
    """down(act(up(x))).  Activations by name:

    "xielu": with two learned numbers p, q (tensor "act" [2]),
        z > 0:   softplus(p) z^2 + z/2
        z <= 0:  (1/2 + softplus(q)) (e^z - 1 - z) + z/2
    so the slope at 0 is 1/2 from both sides.
    """
    ACTIVATIONS = {"xielu": 2}          # name -> how many learned numbers it has

    @staticmethod
    def params(spec: DenseSpec):
        n = spec.names
        if spec.activation not in Dense.ACTIVATIONS:
            raise ValueError(f"unknown activation {spec.activation!r} "
                             f"(known: {sorted(Dense.ACTIVATIONS)})")
        p = {n.get("up", "up.weight"): ParamDecl((spec.ffn_dim, spec.hidden), "linear"),
             n.get("down", "down.weight"): ParamDecl((spec.hidden, spec.ffn_dim), "linear")}
        k = Dense.ACTIVATIONS[spec.activation]
        if k:
            p[n.get("act", "act")] = ParamDecl((k,), "normal", mean=0.0, std=0.5)
        return p

    def __init__(self, spec: DenseSpec, tensors, ops, dtype):
        self.spec = spec
        self.ops = ops
        self.dtype = dtype
        n = spec.names
        self.up = tensors[n.get("up", "up.weight")].contiguous()
        self.down = tensors[n.get("down", "down.weight")].contiguous()
        self.act = tensors[n.get("act", "act")].to(torch.float32).contiguous()

    def forward(self, normed, ctx):
        z = self.ops.linear(normed, self.up, out_dtype=self.dtype)
        act = self.ops.new_rows(normed.shape[0], self.spec.ffn_dim, self.dtype, normed.device)
        self.ops.xielu(z, self.act, act)
        return self.ops.linear(act, self.down, out_dtype=self.dtype)


register_feed_forward("dense", Dense)
