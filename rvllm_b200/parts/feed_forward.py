"""SwiGLU feed-forward: down(silu(gate(x)) * up(x)) (the reference's `swiglu_ffn`,
src/model.rs:320-335).

gate and up are stored as one [2F, hidden] matrix so that they are one matrix
product; the activation kernel reads both halves of its output row.  (The reference
runs two products and `silu_gate_multiply.cu`, src/cuda/model.rs:740-760.)
"""
from __future__ import annotations

import torch

from .base import FeedForward, register_feed_forward
from .spec import DenseSpec, MoESpec, ParamDecl, SwiGLUSpec


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


class MoE(FeedForward):
    """A mixture of SwiGLU experts (`MoESpec`).  For a token x:

        s       = sigmoid(W_router x)                           float32
        allowed = experts of the `keep` groups whose `group_top` best scores sum highest
        chosen  = the `top` allowed experts with the largest s  (ties: the lower index)
        y       = sum_{e chosen} s_e / (sum_chosen s + weight_eps) * down_e(silu(gate_e x) * up_e x)

    The router matrix is kept in float32 and its product is formed in float32 whatever the
    compute type, in the kernel that also makes the choice (`ops.moe_route`).  The experts' matrices are stacked ([experts, 2 ffn, hidden] with gate and up rows
    alternating, so that a pair lies in neighbouring rows of a product's tile, and
    [experts, hidden, ffn]); `ops.moe_experts` chooses between a kernel that walks each token's
    experts (few tokens) and grouped matrix products over the tokens sorted by expert.  A
    token's result is a sum over its own experts in the order they were chosen, so it does not
    depend on what else is in the batch.
    """
    SCORES = ("sigmoid",)

    @staticmethod
    def _names(spec):
        n = spec.names
        out = {"router": n.get("router", "router")}
        for e in range(spec.experts):
            for k in ("gate", "up", "down"):
                out[(e, k)] = n.get("expert", "e{e}.{k}").format(e=e, k=k)
        return out

    @staticmethod
    def _check(spec: MoESpec):
        if spec.score not in MoE.SCORES:
            raise ValueError(f"unknown router score {spec.score!r} (known: {MoE.SCORES})")
        if spec.experts < 1 or not 1 <= spec.top <= spec.experts:
            raise ValueError(f"a mixture of {spec.experts} experts cannot use {spec.top} a token")
        if spec.groups < 1 or spec.experts % spec.groups or not 1 <= spec.keep <= spec.groups:
            raise ValueError(f"{spec.experts} experts do not form {spec.groups} equal groups "
                             f"of which {spec.keep} are kept")
        if spec.keep * (spec.experts // spec.groups) < spec.top:
            raise ValueError(f"{spec.keep} groups of {spec.experts // spec.groups} experts "
                             f"cannot give {spec.top} experts")

    @staticmethod
    def params(spec: MoESpec):
        MoE._check(spec)
        n = MoE._names(spec)
        p = {n["router"]: ParamDecl((spec.experts, spec.hidden), "normal", mean=0.0,
                                    std=spec.hidden ** -0.5)}
        for e in range(spec.experts):
            p[n[(e, "gate")]] = ParamDecl((spec.ffn_dim, spec.hidden), "linear")
            p[n[(e, "up")]] = ParamDecl((spec.ffn_dim, spec.hidden), "linear")
            p[n[(e, "down")]] = ParamDecl((spec.hidden, spec.ffn_dim), "linear")
        return p

    def __init__(self, spec: MoESpec, tensors, ops, dtype):
        self._check(spec)
        self.spec = spec
        self.ops = ops
        self.dtype = dtype
        n = self._names(spec)
        self.router = tensors[n["router"]].to(torch.float32).contiguous()
        first = tensors[n[(0, "gate")]]
        self.gate_up = torch.stack([
            torch.stack([tensors[n[(e, "gate")]].to(first.dtype),
                         tensors[n[(e, "up")]].to(first.dtype)], dim=1).reshape(
                             2 * spec.ffn_dim, spec.hidden)
            for e in range(spec.experts)]).contiguous()          # [E, 2F, W]: gate f, up f, ...
        self.down = torch.stack([tensors[n[(e, "down")]].to(first.dtype)
                                 for e in range(spec.experts)]).contiguous()   # [E, W, F]

    def forward(self, normed, ctx):
        s = self.spec
        n = normed.shape[0]
        ids = torch.empty((n, s.top), dtype=torch.int32, device=normed.device)
        weights = torch.empty((n, s.top), dtype=torch.float32, device=normed.device)
        # the router's product and the choice: one kernel
        self.ops.moe_route(normed, self.router, s.groups, s.keep, s.group_top, s.weight_eps,
                           ids, weights)
        out = self.ops.new_rows(n, s.hidden, self.dtype, normed.device)
        self.ops.moe_experts(normed, ids, weights, self.gate_up, self.down, out)
        return out


register_feed_forward("moe", MoE)
