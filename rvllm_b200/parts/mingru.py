"""minGRU: a gated recurrence whose gate and candidate read only the current token, so
that a prompt's states are a linear scan.

    z_t = sigmoid(W_z h_t + b_z)            u_t = W_x h_t + b_x
    c_t = u_t + 1/2  (u_t >= 0),  sigmoid(u_t)  (u_t < 0)
    S_t = (1 - z_t) S_(t-1) + z_t c_t       y_t = W_o (S_t * silu(W_g h_t))

(The recurrence of "Were RNNs All We Needed?", Feng et al., with the candidate kept
positive.)  W_z, W_x and W_g are one [3 width, hidden] product whose result stays float32;
gate, candidate, scan and state are float32.  The state is one float32 record [width] per
request in a slot of the cache manager; one kernel serves any mixture of prompt portions
and single tokens.
"""
from __future__ import annotations

import torch

from .base import Mixer, StateNeed, register_mixer
from .spec import MinGRUSpec, ParamDecl


class MinGRU(Mixer):
    @staticmethod
    def _names(spec):
        n = spec.names
        return {k: n.get(k, k) for k in ("z", "z.b", "x", "x.b", "g", "o")}

    @staticmethod
    def params(spec: MinGRUSpec, owns_cache: bool = True):
        n = MinGRU._names(spec)
        w, h = spec.width, spec.hidden
        return {n["z"]: ParamDecl((w, h), "linear"), n["z.b"]: ParamDecl((w,), "bias"),
                n["x"]: ParamDecl((w, h), "linear"), n["x.b"]: ParamDecl((w,), "bias"),
                n["g"]: ParamDecl((w, h), "linear"), n["o"]: ParamDecl((h, w), "linear")}

    @staticmethod
    def cache_need(spec: MinGRUSpec):
        return StateNeed((spec.width,))

    def __init__(self, spec: MinGRUSpec, tensors, ops, dtype):
        self.spec = spec
        self.ops = ops
        self.dtype = dtype
        n = self._names(spec)
        z = tensors[n["z"]]
        self.w_in = torch.cat([z, tensors[n["x"]].to(z.dtype), tensors[n["g"]].to(z.dtype)],
                              dim=0).contiguous()
        self.b_in = torch.cat([tensors[n["z.b"]].to(torch.float32),
                               tensors[n["x.b"]].to(torch.float32)]).contiguous()
        self.w_out = tensors[n["o"]].contiguous()

    def forward(self, normed, ctx, cache):
        if cache is None or not cache.owns:
            raise ValueError("mingru: a recurrent state cannot be shared between calls")
        proj = self.ops.linear(normed, self.w_in, out_dtype=torch.float32)
        y = self.ops.new_rows(normed.shape[0], self.spec.width, self.dtype, normed.device)
        self.ops.mingru_scan(proj, self.b_in, cache.state, ctx, y)
        return self.ops.linear(y, self.w_out, out_dtype=self.dtype)


register_mixer("mingru", MinGRU)
