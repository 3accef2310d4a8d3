"""The Mamba-2 (state-space duality) mixer.

With inner = heads * head_dim, N = state and G = groups, the input projection gives [z: inner | x: inner | B: G N |
C: G N | dt: heads].  x, B and C pass a causal convolution over `conv` tokens per channel (with bias) and silu;
dt <- softplus(dt + dt_bias); per head (head h reads group h / (heads / G)):

    S_t = exp(-exp(A_log) dt_t) S_{t-1} + dt_t B_t x_t^T      (S is N x head_dim),      y_t = S_t^T C_t + D x_t;

y * silu(z) is divided by its root mean square in `norm_groups` equal parts (the gate comes first), multiplied by a
weight, and projected back: residual += Wo (...).  The recurrence, its decays and step sizes and the norm are 32-bit.

What a sequence carries from token to token, S and the convolution's last `conv` - 1 inputs, is one float32 row of
the cache's per-sequence state (zero when the sequence starts); a prompt cut anywhere, or fed token by token, walks
the same recurrence.

Tensor names: prefix + "mix.{in,conv,conv.b,dt_bias,A_log,D,norm,o}" unless `params["tensor_names"]` gives others.
"""
from __future__ import annotations

from typing import List, Optional

import torch

from ..cache.sequence_cache import StateRequest
from ..kernels import ops
from .base import Mixer, WeightSpec
from .linear import linear
from .registry import register

_NAMES = {"in": "mix.in", "conv": "mix.conv", "conv_bias": "mix.conv.b", "dt_bias": "mix.dt_bias", "a_log": "mix.A_log",
          "d": "mix.D", "norm": "mix.norm", "o": "mix.o"}


@register("mixer", "mamba2")
class Mamba2(Mixer):
    def __init__(self, params, prefix=""):
        super().__init__(params, prefix)
        self.hidden = int(params["hidden_size"])
        self.heads = int(params["heads"])
        self.head_dim = int(params["head_dim"])
        self.n_state = int(params["state"])
        self.groups = int(params["groups"])
        self.taps = int(params["conv"])
        self.norm_groups = int(params["norm_groups"])
        self.eps = float(params["eps"])
        if self.heads % self.groups:
            raise ValueError(f"{self.heads} heads do not divide into {self.groups} groups")
        self.inner = self.heads * self.head_dim
        if self.inner % self.norm_groups:
            raise ValueError(f"{self.inner} values do not divide into {self.norm_groups} norm groups")
        if self.taps < 1:
            raise ValueError("the convolution needs at least one tap")
        self.channels = self.inner + 2 * self.groups * self.n_state
        self.proj_width = 2 * self.inner + 2 * self.groups * self.n_state + self.heads
        self.s_floats = self.heads * self.n_state * self.head_dim
        self.names = {k: self.tensor_name(k, v) for k, v in _NAMES.items()}

    def weights(self) -> List[WeightSpec]:
        n = self.names
        return [WeightSpec(n["in"], (self.proj_width, self.hidden)), WeightSpec(n["conv"], (self.channels, self.taps)),
                WeightSpec(n["conv_bias"], (self.channels,)), WeightSpec(n["dt_bias"], (self.heads,)),
                WeightSpec(n["a_log"], (self.heads,)), WeightSpec(n["d"], (self.heads,)),
                WeightSpec(n["norm"], (self.inner,), "ones"), WeightSpec(n["o"], (self.hidden, self.inner))]

    def state_request(self) -> Optional[StateRequest]:
        return StateRequest((self.s_floats + (self.taps - 1) * self.channels,), torch.float32)

    def bind(self, tensors, rt) -> None:
        super().bind(tensors, rt)
        n = self.names
        self.w_in = rt.place(tensors[n["in"]])
        self.w_o = rt.place(tensors[n["o"]])
        self.conv_w = rt.place(tensors[n["conv"]])
        self.conv_b = rt.place(tensors[n["conv_bias"]]).to(self.conv_w.dtype)
        # the recurrence's constants enter 32-bit arithmetic: kept as 32-bit values
        self.dt_bias, self.a_log, self.d_skip = (tensors[n[k]].to(device=rt.device, dtype=torch.float32).contiguous()
                                                 for k in ("dt_bias", "a_log", "d"))
        self.norm_w = rt.place(tensors[n["norm"]])

    def forward(self, h, residual, step, memory) -> None:
        if memory.state is None:
            raise RuntimeError("the state-space mixer was given no per-sequence state")
        with ops.bucket("qkv matmul"):
            proj = linear(h, self.w_in, out_dtype=self.rt.dtype)
        with ops.bucket("conv"):
            xbc = ops.mamba2_conv(proj, self.conv_w, self.conv_b, memory.state, step, self.inner, self.channels, self.taps,
                                  self.s_floats)
        with ops.bucket("scan"):
            y = ops.mamba2_scan(xbc, proj, self.dt_bias, self.a_log, self.d_skip, memory.state, step, self.heads,
                                self.head_dim, self.n_state, self.groups, self.taps)
        with ops.bucket("gated norm"):
            g = ops.mamba2_gate_norm(y, proj, self.norm_w, self.norm_groups, self.eps, self.rt.dtype)
        with ops.bucket("out matmul"):
            linear(g, self.w_o, out=residual, accumulate=True)
