"""Causal grouped-query attention without rotation, with the options some designs add to it.

q, k, v = Wq h, Wk h, Wv h (one product over the three matrices stacked by rows); the keys are `head_dim` wide and
the values `v_head_dim`, which need not be equal; score = (q . k) * scale, then, with `softcap` = c > 0,
score <- c * tanh(score / c); a query at position i sees keys j <= i, with `chunk` = s only those of its own chunk
(floor(i / s) == floor(j / s), chunks counted from position 0 of the sequence, wherever a prompt was cut), with
`window` = w only the last w; softmax, with `sink` a learned number per head whose exponential joins the denominator
without key or value (it is not scaled and not capped); residual += Wo (heads concatenated).

Value blending across layers (`value_mix`): the first layer that blends ("source") publishes its values for the
step's tokens; every later one ("blend") replaces its own by (1 - lambda) v + lambda v_source, lambda a learned
scalar, before they go to the cache.  Scores, softmax and the blend are 32-bit.

Tensor names: prefix + "mix.{q,k,v,o,sink,vmix}" unless `params["tensor_names"]` gives others.
"""
from __future__ import annotations

from typing import List, Optional

import torch

from ..cache.sequence_cache import CacheRequest
from ..kernels import ops
from .base import Mixer, WeightSpec
from .linear import linear
from .registry import register


@register("mixer", "sink_attention")
class SinkAttention(Mixer):
    def __init__(self, params, prefix=""):
        super().__init__(params, prefix)
        self.hidden = int(params["hidden_size"])
        self.n_heads = int(params["num_heads"])
        self.n_kv = int(params["num_kv_heads"])
        self.head_dim = int(params["head_dim"])
        self.v_dim = int(params.get("v_head_dim") or self.head_dim)
        self.scale = float(params["scale"])
        self.softcap = float(params.get("softcap") or 0.0)
        self.has_sink = bool(params.get("sink", False))
        self.chunk = int(params["chunk"]) if params.get("chunk") else None
        self.window = int(params["window"]) if params.get("window") else None
        self.value_mix = params.get("value_mix")            # None, "source" or "blend"
        self.value_mix_key = params.get("value_mix_key", "value_mix")
        if self.value_mix not in (None, "source", "blend"):
            raise ValueError(f"value_mix must be None, \"source\" or \"blend\", got {self.value_mix!r}")
        if self.n_heads % self.n_kv:
            raise ValueError(f"{self.n_heads} heads do not divide into {self.n_kv} kv heads")
        if self.chunk and self.window:
            raise ValueError("an attention is cut into chunks or sees a window, not both")
        self.q_dim, self.k_dim, self.v_width = self.n_heads * self.head_dim, self.n_kv * self.head_dim, self.n_kv * self.v_dim
        self.names = {k: self.tensor_name(k, f"mix.{k}") for k in ("q", "k", "v", "o", "sink", "vmix")}

    def weights(self) -> List[WeightSpec]:
        n = self.names
        out = [WeightSpec(n["q"], (self.q_dim, self.hidden)), WeightSpec(n["k"], (self.k_dim, self.hidden)),
               WeightSpec(n["v"], (self.v_width, self.hidden)), WeightSpec(n["o"], (self.hidden, self.n_heads * self.v_dim))]
        if self.has_sink:
            out.append(WeightSpec(n["sink"], (self.n_heads,)))
        if self.value_mix is not None:
            out.append(WeightSpec(n["vmix"], ()))     # the source layer stores one too; it has no use for it
        return out

    def cache_request(self) -> Optional[CacheRequest]:
        v = None if self.v_dim == self.head_dim else self.v_dim
        if self.chunk:
            return CacheRequest("chunk", self.n_kv, self.head_dim, self.chunk, v)
        if self.window:
            return CacheRequest("window", self.n_kv, self.head_dim, self.window, v)
        return CacheRequest("full", self.n_kv, self.head_dim, None, v)

    def decode_plan(self, n_seqs: int, max_kv_len: int, sm_count: int, kv_lens=None):
        return ops.attn_general_decode_plan(n_seqs, max_kv_len, sm_count, self.n_heads, self.n_kv, self.window, self.chunk,
                                            self.rt.dtype, self.head_dim, self.v_dim, kv_lens)

    def bind(self, tensors, rt) -> None:
        super().bind(tensors, rt)
        q, k, v = (rt.place(tensors[self.names[x]]) for x in ("q", "k", "v"))
        if not (q.dtype == k.dtype == v.dtype):
            q, k, v = (t.to(torch.float32) for t in (q, k, v))
        self.w_qkv = torch.cat([q, k, v], dim=0).contiguous()
        del q, k, v
        self.w_o = rt.place(tensors[self.names["o"]])
        # what enters the softmax and the blend is 32-bit whatever the file stores
        self.sinks = tensors[self.names["sink"]].to(device=rt.device, dtype=torch.float32).contiguous() if self.has_sink else None
        self.blend = None
        if self.value_mix == "blend":
            self.blend = tensors[self.names["vmix"]].to(device=rt.device, dtype=torch.float32).reshape(1).contiguous()

    def forward(self, h, residual, step, memory) -> None:
        with ops.bucket("qkv matmul"):
            qkv = linear(h, self.w_qkv, out_dtype=self.rt.dtype)
        with ops.bucket("rope+cache"):
            first = copy_to = None
            if self.value_mix == "source":
                copy_to = torch.empty((qkv.shape[0], self.v_width), dtype=qkv.dtype, device=qkv.device)
                step.shared[self.value_mix_key] = copy_to
            elif self.value_mix == "blend":
                first = step.shared.get(self.value_mix_key)
                if first is None:
                    raise RuntimeError("a layer that blends values ran before the layer whose values it blends in")
            ops.kv_store(qkv, step.positions, step.token_slots, memory, self.n_heads, self.n_kv, self.head_dim, self.v_dim,
                         first, self.blend, copy_to)
        with ops.bucket("attention"):
            att = torch.empty((qkv.shape[0], self.n_heads * self.v_dim), dtype=self.rt.dtype, device=qkv.device)
            ops.attention_general(qkv, memory, step, self.n_heads, self.n_kv, self.head_dim, self.v_dim, self.scale, att,
                                  window=self.window, chunk=self.chunk, softcap=self.softcap, sinks=self.sinks,
                                  plan=step.plan_of(self))
        with ops.bucket("out matmul"):
            linear(att, self.w_o, out=residual, accumulate=True)
