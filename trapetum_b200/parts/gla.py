"""Gated linear attention: a recurrent mixer whose state is a matrix per head with a decay per key channel.

Between a fused input product ``[q | k | v | g] = W h`` and an output product ``W_o``:

* per head (key channels d, value channels v): ``S <- diag(decay_t) S + k_t v_t^T`` and ``o_t = S^T (q_t * q_scale)``;
* the decay has low rank: ``decay_t = sigmoid(A2 (A1 h_t) + bias)^(1 / tau)``, one number per head and key channel;
* every head's ``o_t`` is divided by its root mean square (eps inside the root), multiplied by a weight of
  ``value_dim`` numbers that the heads share and by ``silu(g_t)``.

A sequence's state ``[heads, key_dim, value_dim]`` is one float32 row of the cache's state area, addressed by slot,
zero when the sequence starts, carried from step to step.  32-bit: the decay's pre-activation from its first
product on, the decay, the state, ``o`` and its norm.  The products and the gate's silu input are of the compute
dtype.  The kernels are in ``csrc/gla.cu``; a step of whole prompts and a step of one token each run the same ones.

Parameters (none is fixed in code): ``hidden_size``, ``heads``, ``key_dim``, ``value_dim``, ``tau``, ``q_scale``,
``eps``, ``decay_rank`` (optional: the weight file's shapes decide it when it is absent) and the tensor names ``q``, ``k``, ``v``, ``g``, ``o``, ``norm``, ``a1``, ``a2``, ``a2_bias``.
"""
from __future__ import annotations

from typing import Dict

import torch

from ..csrc import ops
from ..weights.loader import TensorSpec
from .base import Mixer, StateNeed, register_part
from .linear import kernel_files as linear_kernels
from .linear import linear, linear_partials


class GatedLinearAttention(Mixer):
    graph_safe = True          # sequences, slots and lengths are read on the device

    def __init__(self, params, prefix, rt):
        super().__init__(params, prefix, rt)
        p = params
        self.hidden = int(p["hidden_size"])
        self.heads = int(p["heads"])
        self.D = int(p["key_dim"])
        self.V = int(p["value_dim"])
        self.tau = float(p["tau"])
        self.q_scale = float(p["q_scale"])
        self.eps = float(p["eps"])
        if min(self.heads, self.D, self.V) < 1 or not self.tau > 0:
            raise ValueError(f"gla: heads={self.heads} key_dim={self.D} value_dim={self.V} tau={self.tau}")
        # the decay's rank: the a1 tensor's first size, read from the file's shape when bound, unless it is given
        self.rank = int(p["decay_rank"]) if p.get("decay_rank") else -1

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        HD, HV = self.heads * self.D, self.heads * self.V
        return {
            self._name("q"): TensorSpec((HD, self.hidden)),
            self._name("k"): TensorSpec((HD, self.hidden)),
            self._name("v"): TensorSpec((HV, self.hidden)),
            self._name("g"): TensorSpec((HV, self.hidden)),
            self._name("o"): TensorSpec((self.hidden, HV)),
            self._name("norm"): TensorSpec((self.V,), "gain"),
            self._name("a1"): TensorSpec((self.rank, self.hidden)),
            self._name("a2"): TensorSpec((HD, self.rank)),
            self._name("a2_bias"): TensorSpec((HD,), "norm"),
        }

    def bind(self, tensors) -> None:
        mats = [tensors[self._name(n)] for n in ("q", "k", "v", "g")]
        dt = mats[0].dtype if all(m.dtype == mats[0].dtype for m in mats) else torch.float32
        self.w_in = torch.cat([m.to(dt) for m in mats], dim=0).contiguous()
        self.w_a1 = tensors[self._name("a1")]
        self.rank = int(self.w_a1.shape[0])
        a2 = tensors[self._name("a2")]
        if tuple(a2.shape) != (self.heads * self.D, self.rank):
            raise ValueError(f"gla: {self._name('a2')} is {tuple(a2.shape)}, but {self._name('a1')} has rank {self.rank}")
        # what enters the decay is 32-bit from the first product's sums on
        self.w_a2 = a2.float().contiguous()
        self.b_a2 = tensors[self._name("a2_bias")].float().contiguous()
        self.w_norm = tensors[self._name("norm")].float().contiguous()
        self.w_o = tensors[self._name("o")]

    def kernel_files(self):
        return linear_kernels(self.rt.dtype) + ("gla",)

    def cache_need(self):
        return StateNeed((self.heads * self.D * self.V,), torch.float32)

    def forward(self, x, ctx, state):
        proj = linear(x, self.w_in, self.rt.dtype)
        low = linear_partials(x, self.w_a1)              # [splits, T, rank] float32, added up by the decay's kernel
        y = ops.gla(proj, low, self.w_a2, self.b_a2, self.tau, self.q_scale, self.w_norm, self.eps, self.heads, self.D,
                    self.V, state.data, ctx.seq_start, ctx.token_seq, ctx.slot_ids, ctx.batch,
                    max_seq_len=ctx.max_seq_len if ctx.is_prefill else 0)
        return linear_partials(y, self.w_o)


register_part("mixer", "gla", GatedLinearAttention)
