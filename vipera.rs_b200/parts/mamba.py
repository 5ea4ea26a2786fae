"""Mamba's selective scan as a mixer with a state of fixed size.

From the mixer's input h: ``[x | z] = W_in h``; x passes a causal convolution per channel (with
bias) and silu; ``[dt | B | C] = W_x x``; ``dt = softplus(W_dt dt + b_dt)`` per channel; with
``A = -exp(A_log)`` [inner, state], per channel c and state index n

    S[c, n] = exp(dt_c A[c, n]) S[c, n] + dt_c x_c B_n        y_c = sum_n S[c, n] C_n + D_c x_c

and the mixer's output is ``W_o (y * silu(z))``, added into the stream it is handed.  A request
keeps S (32-bit, zero at its start) and the convolution's last inputs.  The products run in the
run's type; their results stay 32-bit up to the scan (``csrc/kernels/mamba.cu``), whose
arithmetic is 32-bit throughout: softplus, exp(dt A), the state and the sums over it.
"""
from __future__ import annotations

import os

import torch

from ..config.registry import MIXERS
from ..kernels import ops
from ..weights import TensorSpec
from .base import CacheBundle, FixedState, Mixer
from .conv import CausalConv
from .linear import Linear


class Mamba1(Mixer):
    """params: hidden_size, inner (channels), state (states per channel), dt_rank, taps (of the
    convolution) and, optionally, ``out_scale`` (multiplies the mixer's output).  Tensors under
    ``<prefix>``: in, conv (+ bias), x, dt (+ bias), A_log, D, o."""

    kernels = ("mamba", "seqconv")
    # Steps of this many tokens and more run their chunks side by side (three launches, the
    # recurrence computed twice); shorter ones walk each entry's tokens in one launch.
    CHUNKED_FROM = int(os.environ.get("VIPERA_SCAN_CHUNKED_FROM", 256))

    @classmethod
    def schema(cls, params, prefix):
        hidden, inner, state = params["hidden_size"], params["inner"], params["state"]
        rank, taps = params["dt_rank"], params["taps"]
        schema = {
            f"{prefix}.in.weight": TensorSpec((2 * inner, hidden)),
            f"{prefix}.x.weight": TensorSpec((rank + 2 * state, inner)),
            f"{prefix}.dt.weight": TensorSpec((inner, rank), init="filter"),
            f"{prefix}.dt.bias": TensorSpec((inner,), init="bias"),
            f"{prefix}.A_log.weight": TensorSpec((inner, state), init="log_rate"),
            f"{prefix}.D.weight": TensorSpec((inner,), init="norm"),
            f"{prefix}.o.weight": TensorSpec((hidden, inner)),
        }
        schema.update(CausalConv.schema(f"{prefix}.conv", inner, taps, bias=True))
        schema[f"{prefix}.conv.weight"] = TensorSpec((inner, taps), init="filter")
        return schema

    def __init__(self, params, prefix, tensors, dtype, device):
        super().__init__(params, prefix, tensors, dtype, device)
        self.hidden, self.inner = int(params["hidden_size"]), int(params["inner"])
        self.state, self.rank, self.taps = int(params["state"]), int(params["dt_rank"]), int(params["taps"])
        self.out_scale = float(params.get("out_scale", 1.0))
        self.proj_in = Linear(tensors[f"{prefix}.in.weight"], dtype, device)
        x_weight = tensors[f"{prefix}.x.weight"]
        # the step-size rows and the B/C rows as two matrices, so that each product's result is dense
        self.proj_dt_low = Linear(x_weight[: self.rank], dtype, device)
        self.proj_bc = Linear(x_weight[self.rank:], dtype, device)
        self.proj_dt = Linear(tensors[f"{prefix}.dt.weight"], dtype, device, bias=tensors[f"{prefix}.dt.bias"],
                              min_tensor_core_inner=64)
        out_weight = tensors[f"{prefix}.o.weight"]
        if self.out_scale != 1.0:
            out_weight = (out_weight.to(torch.float32) * self.out_scale)
        self.out = Linear(out_weight, dtype, device)
        self.conv = CausalConv(f"{prefix}.conv", tensors, device, add_input=False, activation="silu")
        self.a = (-torch.exp(tensors[f"{prefix}.A_log.weight"].to(device=device, dtype=torch.float32))).contiguous()
        self.d = tensors[f"{prefix}.D.weight"].to(device=device, dtype=torch.float32).contiguous()

    def kernel_families(self):
        names = ("mamba", "seqconv")
        for linear in (self.proj_in, self.proj_dt_low, self.proj_bc, self.proj_dt, self.out):
            names += linear.kernel_families()
        return tuple(dict.fromkeys(names))

    @classmethod
    def cache_request_for(cls, params):
        inner, state, taps = int(params["inner"]), int(params["state"]), int(params["taps"])
        return CacheBundle.of(conv=CausalConv.state_request(inner, taps),
                              scan=FixedState((inner * state,), torch.float32))

    @classmethod
    def workspace_bytes(cls, params, tokens, element_bytes):
        inner, state, rank = params["inner"], params["state"], params["dt_rank"]
        return tokens * (inner * (8 + 4 + 4 + 2 * element_bytes) + (rank * element_bytes) + 2 * state * 4)

    def forward(self, ctx, h, residual, cache, writes_cache):
        count, ws = ctx.num_tokens, ctx.workspace
        xz = ws.get("mamba.xz", (count, 2 * self.inner), torch.float32)
        self.proj_in(ctx, h, epilogue=ops.EPI_STORE, out=xz)
        x32 = ws.get("mamba.x32", (count, self.inner), torch.float32)
        x = x32 if ctx.dtype == torch.float32 else ws.get("mamba.x", (count, self.inner), ctx.dtype)
        self.conv(ctx, xz, cache.get("conv"), out=None if x is x32 else x, out_f32=x32)
        dt_low = ws.get("mamba.dt_low", (count, self.rank), ctx.dtype)
        self.proj_dt_low(ctx, x, epilogue=ops.EPI_STORE, out=dt_low)
        bc = ws.get("mamba.bc", (count, 2 * self.state), torch.float32)
        self.proj_bc(ctx, x, epilogue=ops.EPI_STORE, out=bc)
        dt_pre = ws.get("mamba.dt", (count, self.inner), torch.float32)
        self.proj_dt(ctx, dt_low, epilogue=ops.EPI_STORE, out=dt_pre)
        y = ws.get("mamba.y", (count, self.inner), ctx.dtype)
        chunk_scratch = None
        if not ctx.all_single and count >= self.CHUNKED_FROM:
            jobs = ops.scan_jobs(count, ctx.num_entries)
            chunk_scratch = (ws.get("mamba.chunk_states", (jobs, self.inner * self.state), torch.float32),
                             ws.get("mamba.chunk_dt", (jobs, self.inner), torch.float32))
        ops.mamba_scan(x32, dt_pre, bc, xz, self.inner, a=self.a, d=self.d, state=cache["scan"].data,
                       entry_starts=ctx.entry_starts, state_slots=ctx.state_slots, fresh=ctx.fresh,
                       num_entries=ctx.num_entries, out=y, chunk_scratch=chunk_scratch)
        self.out(ctx, y, epilogue=ops.EPI_RESIDUAL, resid=residual)


MIXERS.register("mamba1", Mamba1)
