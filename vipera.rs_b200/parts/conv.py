"""A short causal convolution over time, one filter per channel, with the last inputs of every
request kept between steps.

``out_t = act(sum_j w[:, j] x_(t - taps + 1 + j) + b) (+ x_t)``: the last column of ``w`` is
the current token's, inputs before a request's start are zero.  The state of a request is its
last ``taps - 1`` inputs, 32-bit, [taps - 1, channels]; a portion of a prompt continues from
it, so a prompt may be cut anywhere.  Used in front of sublayers (added to its input, no
bias, no activation) and inside Mamba (bias and silu).
"""
from __future__ import annotations

import torch

from ..kernels import ops
from ..weights import TensorSpec
from .base import FixedState


class CausalConv:
    """``weight`` [channels, taps] (any float type; kept in 32-bit), ``bias`` [channels] or None."""

    kernels = ("seqconv",)
    graph_safe = True

    def kernel_families(self):
        return self.kernels

    @staticmethod
    def schema(prefix: str, channels: int, taps: int, bias: bool = False):
        out = {f"{prefix}.weight": TensorSpec((channels, taps), init="filter")}
        if bias:
            out[f"{prefix}.bias"] = TensorSpec((channels,), init="bias")
        return out

    @staticmethod
    def state_request(channels: int, taps: int):
        """What the convolution keeps per request: nothing for a single tap."""
        return FixedState((taps - 1, channels), torch.float32) if taps > 1 else None

    def __init__(self, prefix, tensors, device, *, add_input: bool, activation: str = "none"):
        self.weight = tensors[f"{prefix}.weight"].to(device=device, dtype=torch.float32).contiguous()
        bias = tensors.get(f"{prefix}.bias")
        self.bias = None if bias is None else bias.to(device=device, dtype=torch.float32).contiguous()
        self.channels, self.taps = self.weight.shape
        self.add_input = bool(add_input)
        self.activation = ops.CONV_ACTIVATIONS[activation]

    def __call__(self, ctx, x, state, *, out=None, out_f32=None, clear=None):
        """``x`` float32 [tokens, >= channels] (the first ``channels`` columns count); ``state`` a
        StateView or None (one tap); ``out`` in the run's type and/or ``out_f32`` receive the
        result; ``clear`` (float32, any shape) is set to zero on the way."""
        ops.causal_conv(x, self.weight, self.bias, channels=self.channels, state=None if state is None else state.data,
                        entry_starts=ctx.entry_starts, token_entry=ctx.token_entry, state_slots=ctx.state_slots,
                        fresh=ctx.fresh, num_entries=ctx.num_entries, single=ctx.all_single,
                        add_input=self.add_input, activation=self.activation, out=out, out_f32=out_f32, clear=clear)
