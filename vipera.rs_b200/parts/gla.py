"""Gated linear attention as a mixer with a state of fixed size.

Per head a matrix S [d, dv] in 32-bit floats, zero at a request's start.  From the mixer's input
h: ``q = W_q h * d^-1/2``, ``k = W_k h``, ``v = W_v h``, and one decay per key channel,
``alpha = sigmoid(W_a2 (W_a1 h) + b_a2)^(1 / tau)``; for each token

    S = diag(alpha) S + k v^T        o = S^T q

Each head's o is divided by its root mean square over dv and multiplied by a weight per value
(one vector shared by the heads); the concatenated heads are multiplied by ``silu(W_g h)`` and
sent through the output matrix, which adds into the stream the mixer is handed.  q, k, v and g
come from one product with the concatenated matrix; its result stays 32-bit, and the decays
(through log sigmoid), the state, the products with it and the norm are 32-bit arithmetic
(``csrc/kernels/gla.cu``).
"""
from __future__ import annotations

import os

import torch

from ..config.registry import MIXERS
from ..kernels import ops
from ..weights import TensorSpec
from .base import FixedState, Mixer
from .linear import Linear


class GatedLinearAttention(Mixer):
    """params: hidden_size, num_heads, head_dim (size of q and k per head), value_dim, tau, norm_eps
    and, optionally, ``decay_rank`` (the inner size of the decay's two matrices; None: the stored
    tensors decide) and ``out_scale`` (multiplies the mixer's output).  Tensors under ``<prefix>``:
    q, k, v, g, o, norm [value_dim], a1 [rank, hidden], a2 [heads * head_dim, rank] with a bias."""

    kernels = ("gla",)
    # Steps of this many tokens and more run their chunks side by side (the recurrence computed
    # twice); shorter ones walk each entry's tokens in one launch.
    CHUNKED_FROM = int(os.environ.get("VIPERA_SCAN_CHUNKED_FROM", 256))

    @classmethod
    def schema(cls, params, prefix):
        hidden, heads = params["hidden_size"], params["num_heads"]
        d, dv, rank = params["head_dim"], params["value_dim"], params.get("decay_rank")
        return {
            f"{prefix}.q.weight": TensorSpec((heads * d, hidden)),
            f"{prefix}.k.weight": TensorSpec((heads * d, hidden)),
            f"{prefix}.v.weight": TensorSpec((heads * dv, hidden)),
            f"{prefix}.g.weight": TensorSpec((heads * dv, hidden)),
            f"{prefix}.o.weight": TensorSpec((hidden, heads * dv)),
            f"{prefix}.norm.weight": TensorSpec((dv,), init="norm"),
            f"{prefix}.a1.weight": TensorSpec((rank, hidden)),
            f"{prefix}.a2.weight": TensorSpec((heads * d, rank), init="filter"),
            f"{prefix}.a2.bias": TensorSpec((heads * d,), init="bias"),
        }

    def __init__(self, params, prefix, tensors, dtype, device):
        super().__init__(params, prefix, tensors, dtype, device)
        self.hidden, self.heads = int(params["hidden_size"]), int(params["num_heads"])
        self.dim, self.vdim = int(params["head_dim"]), int(params["value_dim"])
        self.tau, self.norm_eps = float(params["tau"]), float(params["norm_eps"])
        self.out_scale = float(params.get("out_scale", 1.0))
        rows = [tensors[f"{prefix}.{n}.weight"] for n in ("q", "k", "v", "g")]
        widths = [r.shape[0] for r in rows]
        self.offsets = tuple(sum(widths[:i]) for i in range(4))
        self.proj = Linear(torch.cat(rows, dim=0), dtype, device)
        self.decay_in = Linear(tensors[f"{prefix}.a1.weight"], dtype, device)
        self.decay_out = Linear(tensors[f"{prefix}.a2.weight"], dtype, device, bias=tensors[f"{prefix}.a2.bias"],
                                min_tensor_core_inner=64)
        self.rank = self.decay_in.out_features
        if self.decay_out.in_features != self.rank:
            from ..errors import UnsupportedError
            raise UnsupportedError(f"{prefix}: the decay's two matrices disagree on their inner size")
        self.out = Linear(tensors[f"{prefix}.o.weight"], dtype, device)
        self.norm_weight = tensors[f"{prefix}.norm.weight"].to(device=device, dtype=torch.float32).contiguous()

    def kernel_families(self):
        names = ("gla",)
        for linear in (self.proj, self.decay_in, self.decay_out, self.out):
            names += linear.kernel_families()
        return tuple(dict.fromkeys(names))

    @classmethod
    def cache_request_for(cls, params):
        return FixedState((int(params["num_heads"]) * int(params["head_dim"]) * int(params["value_dim"]),), torch.float32)

    @classmethod
    def workspace_bytes(cls, params, tokens, element_bytes):
        heads, d, dv = params["num_heads"], params["head_dim"], params["value_dim"]
        shares = -(-d // 8)
        return tokens * (heads * (2 * d + 2 * dv) * 4 + heads * d * 4 + shares * heads * dv * 4 + heads * dv * element_bytes)

    def forward(self, ctx, h, residual, cache, writes_cache):
        count, ws = ctx.num_tokens, ctx.workspace
        proj = ws.get("gla.proj", (count, self.proj.out_features), torch.float32)
        self.proj(ctx, h, epilogue=ops.EPI_STORE, out=proj)
        low = ws.get("gla.decay_low", (count, self.rank), ctx.dtype)
        self.decay_in(ctx, h, epilogue=ops.EPI_STORE, out=low)
        z = ws.get("gla.decay", (count, self.heads * self.dim), torch.float32)
        self.decay_out(ctx, low, epilogue=ops.EPI_STORE, out=z)
        log_decay = ws.get("gla.log_decay", (count, self.heads * self.dim), torch.float32)
        partial = ws.get("gla.partial", (ops.gla_shares(self.dim), count, self.heads * self.vdim), torch.float32)
        mixed = ws.get("gla.out", (count, self.heads * self.vdim), ctx.dtype)
        chunk_scratch = None
        if not ctx.all_single and count >= self.CHUNKED_FROM:
            jobs = ops.scan_jobs(count, ctx.num_entries)
            chunk_scratch = (ws.get("gla.chunk_states", (jobs, self.heads * self.dim * self.vdim), torch.float32),
                             ws.get("gla.chunk_decays", (jobs, self.heads * self.dim), torch.float32))
        ops.gla(proj, z, offsets=self.offsets, heads=self.heads, dim=self.dim, vdim=self.vdim,
                q_scale=self.dim ** -0.5, tau=self.tau, norm_weight=self.norm_weight, norm_eps=self.norm_eps,
                out_scale=self.out_scale, state=cache.data, entry_starts=ctx.entry_starts,
                state_slots=ctx.state_slots, fresh=ctx.fresh, num_entries=ctx.num_entries, partial=partial, out=mixed,
                log_decay=log_decay, chunk_scratch=chunk_scratch)
        self.out(ctx, mixed, epilogue=ops.EPI_RESIDUAL, resid=residual)


MIXERS.register("gla", GatedLinearAttention)
