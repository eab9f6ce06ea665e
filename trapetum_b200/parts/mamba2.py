"""A selective state-space mixer: the Mamba-2 recurrence with its short convolution and gated norm.

Between an input product ``[z | x B C | dt] = W_in h`` (inner = heads * head_dim columns of z and of x,
groups * state columns of B and of C, one dt per head) and an output product ``W_o``:

* x, B and C pass a causal convolution over ``conv`` taps per channel (with bias; the last tap is the current
  token's) and silu;
* ``dt = softplus(dt + dt_bias)``; per head, with B and C of its group, the state S [head_dim, state] goes
  ``S <- exp(-exp(A_log) dt) S + dt x B^T`` and the output is ``y = S C + D x``;
* ``y * silu(z)`` is RMS-normed in ``norm_groups`` equal parts (gating first, then the norm), times a weight.

A sequence's state (S and the last ``conv - 1`` convolution inputs) is one float32 row of the cache's state
area, addressed by slot, zero when the sequence starts.  The step sizes (they enter an exponential), softplus,
the decay, the state, y and the gated norm are 32-bit: dt comes from a product of its own with 32-bit output.
The other products and the convolution with its silu work in the compute dtype.  The kernels are in
``csrc/mamba2.cu``; a step of one token per sequence and a step of whole prompts use the same recurrence.

Parameters (none is fixed in code): ``hidden_size``, ``heads``, ``head_dim``, ``state``, ``groups``, ``conv``,
``norm_groups``, ``eps`` and the tensor names ``in``, ``conv_w``, ``conv_b``, ``dt_bias``, ``A_log``, ``D``,
``norm``, ``o``.
"""
from __future__ import annotations

from typing import Dict

import torch

from ..csrc import ops
from ..weights.loader import TensorSpec
from .base import Mixer, StateNeed, register_part
from .linear import kernel_files as linear_kernels
from .linear import linear, linear_partials


class Mamba2(Mixer):
    graph_safe = True          # sequences, slots and lengths are read on the device

    def __init__(self, params, prefix, rt):
        super().__init__(params, prefix, rt)
        p = params
        self.hidden = int(p["hidden_size"])
        self.heads = int(p["heads"])
        self.P = int(p["head_dim"])
        self.N = int(p["state"])
        self.groups = int(p["groups"])
        self.taps = int(p["conv"])
        self.norm_groups = int(p["norm_groups"])
        self.eps = float(p["eps"])
        if self.heads % self.groups:
            raise ValueError(f"mamba2: {self.heads} heads cannot share {self.groups} groups")
        self.inner = self.heads * self.P
        if self.inner % self.norm_groups:
            raise ValueError(f"mamba2: {self.inner} inner columns do not split into {self.norm_groups} norm groups")
        if self.taps < 1 or not (1 <= self.N <= 256):
            raise ValueError(f"mamba2: conv={self.taps}, state={self.N} (conv >= 1, state 1..256)")
        self.channels = self.inner + 2 * self.groups * self.N
        self.w = {}

    def tensor_specs(self) -> Dict[str, TensorSpec]:
        return {
            self._name("in"): TensorSpec((self.inner + self.channels + self.heads, self.hidden)),
            self._name("conv_w"): TensorSpec((self.channels, self.taps)),
            self._name("conv_b"): TensorSpec((self.channels,)),
            self._name("dt_bias"): TensorSpec((self.heads,)),
            self._name("A_log"): TensorSpec((self.heads,)),
            self._name("D"): TensorSpec((self.heads,), "gain"),
            self._name("norm"): TensorSpec((self.inner,), "gain"),
            self._name("o"): TensorSpec((self.hidden, self.inner)),
        }

    def bind(self, tensors) -> None:
        w_in = tensors[self._name("in")]
        self.w_in = w_in[:self.inner + self.channels]             # z, x, B, C: output in the compute dtype
        self.w_dt = w_in[self.inner + self.channels:]             # dt: output in 32-bit
        self.w_o = tensors[self._name("o")]
        # the small tensors enter 32-bit arithmetic: kept in 32 bits (exact for what a file stores in 16)
        self.w = {k: tensors[self._name(k)].float().contiguous()
                  for k in ("conv_w", "conv_b", "dt_bias", "A_log", "D", "norm")}

    def kernel_files(self):
        return linear_kernels(self.rt.dtype) + ("mamba2",)

    def cache_need(self):
        return StateNeed((ops.mamba2_state_size(self.heads, self.P, self.N, self.groups, self.taps),), torch.float32)

    def forward(self, x, ctx, state):
        proj = linear(x, self.w_in, self.rt.dtype)
        dt_raw = linear_partials(x, self.w_dt)              # [splits, T, heads], added up by the recurrence's kernel
        w = self.w
        y = ops.mamba2(proj, dt_raw, self.heads, self.P, self.N, self.groups, self.taps, self.norm_groups, w["conv_w"],
                       w["conv_b"], w["dt_bias"], w["A_log"], w["D"], w["norm"], self.eps, state.data, ctx.seq_start,
                       ctx.token_seq, ctx.slot_ids, ctx.batch, one_token_each=not ctx.is_prefill,
                       max_seq_len=ctx.max_seq_len if ctx.is_prefill else 0)
        return linear_partials(y, self.w_o)


register_part("mixer", "mamba2", Mamba2)
