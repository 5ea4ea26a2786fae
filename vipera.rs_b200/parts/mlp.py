"""SwiGLU feed-forward: ``down(up(h) * silu(gate(h)))``, no biases
(crates/vipera-backend-cpu/src/model.rs:1154-1198, 4368-4374).

The reference runs gate and up as two products and the activation as its own pass
(model.rs:1159-1183).  Here the two matrices are interleaved at load so that one product
yields both halves of every feature in one tile, the activation is that product's ending,
and the down product adds into the 32-bit residual stream.
"""
from __future__ import annotations

import torch

from ..config.registry import FEED_FORWARDS
from ..errors import UnsupportedError
from ..kernels import ops
from ..weights import TensorSpec
from .base import FeedForward
from .linear import SWIGLU_GROUP, Linear, interleave_gate_up


class SwiGLU(FeedForward):
    """A gated feed-forward, ``down(act(gate(h)) * up(h))``.  params: hidden_size,
    intermediate_size and, optionally, ``projection_names`` (defaults gate_proj, up_proj,
    down_proj), ``activation`` (``silu``, the default, or ``gelu_tanh``) and ``bias`` (all three
    projections then have one, ``<name>.bias``).  Registered as ``swiglu`` and ``gated_mlp``."""

    takes_lazy_input = True

    @staticmethod
    def _names(params):
        return params.get("projection_names", ("gate_proj", "up_proj", "down_proj"))

    @classmethod
    def schema(cls, params, prefix):
        hidden, inter = params["hidden_size"], params["intermediate_size"]
        gate, up, down = cls._names(params)
        schema = {
            f"{prefix}.{gate}.weight": TensorSpec((inter, hidden)),
            f"{prefix}.{up}.weight": TensorSpec((inter, hidden)),
            f"{prefix}.{down}.weight": TensorSpec((hidden, inter)),
        }
        if params.get("bias", False):
            schema[f"{prefix}.{gate}.bias"] = TensorSpec((inter,), init="bias")
            schema[f"{prefix}.{up}.bias"] = TensorSpec((inter,), init="bias")
            schema[f"{prefix}.{down}.bias"] = TensorSpec((hidden,), init="bias")
        return schema

    @classmethod
    def workspace_bytes(cls, params, tokens, element_bytes):
        return tokens * params["intermediate_size"] * element_bytes

    def __init__(self, params, prefix, tensors, dtype, device):
        super().__init__(params, prefix, tensors, dtype, device)
        self.hidden = int(params["hidden_size"])
        self.inter = int(params["intermediate_size"])
        gate, up, down = self._names(params)
        name = str(params.get("activation", "silu"))
        if name not in ops.ACTIVATIONS:
            raise UnsupportedError(f"activation {name!r}; the gated unit knows: " + ", ".join(sorted(ops.ACTIVATIONS)))
        self.activation = ops.ACTIVATIONS[name]
        gate_w, up_w, down_w = (tensors[f"{prefix}.{n}.weight"] for n in (gate, up, down))
        with_bias = bool(params.get("bias", False))
        gate_b = tensors[f"{prefix}.{gate}.bias"].to(torch.float32) if with_bias else None
        up_b = tensors[f"{prefix}.{up}.bias"].to(torch.float32) if with_bias else None
        spare = -self.inter % SWIGLU_GROUP
        if spare:
            # Gate and up rows are interleaved in groups of 16.  An inner size that is no multiple
            # of that is filled up with features whose rows, biases and down columns are zero: they
            # come out as act(0) * 0 = 0 and add nothing.
            where = gate_w.device
            rows = torch.zeros(spare, self.hidden, dtype=gate_w.dtype, device=where)
            gate_w, up_w = torch.cat([gate_w, rows]), torch.cat([up_w, rows])
            down_w = torch.cat([down_w, torch.zeros(self.hidden, spare, dtype=down_w.dtype, device=where)], dim=1)
            if with_bias:
                gate_b, up_b = (torch.cat([b, torch.zeros(spare, device=where)]) for b in (gate_b, up_b))
            self.inter += spare
        fused = interleave_gate_up(gate_w, up_w)
        fused_bias = down_bias = None
        if with_bias:
            # the bias of the interleaved rows, interleaved the same way
            fused_bias = interleave_gate_up(gate_b[:, None], up_b[:, None]).reshape(-1)
            down_bias = tensors[f"{prefix}.{down}.bias"]
        self.gate_up = Linear(fused, dtype, device, bias=fused_bias)
        self.down = Linear(down_w, dtype, device, bias=down_bias)

    def kernel_families(self):
        return tuple(dict.fromkeys(self.gate_up.kernel_families() + self.down.kernel_families()))

    def forward(self, ctx, h, residual):
        act = ctx.workspace.get("swiglu.act", (ctx.num_tokens, self.inter), ctx.dtype)
        self.gate_up(ctx, h, epilogue=ops.EPI_GATED, out=act, activation=self.activation)
        self.down(ctx, act, epilogue=ops.EPI_RESIDUAL, resid=residual)


FEED_FORWARDS.register("swiglu", SwiGLU)
FEED_FORWARDS.register("gated_mlp", SwiGLU)
