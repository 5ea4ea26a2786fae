"""The matrix-memory cell of xLSTM (mLSTM) as a mixer with a state of fixed size.

Per head the cell keeps a matrix S [d, dv], a vector n [d] and a running maximum m, all in
32-bit floats, zero at a request's start (m starts at 0).  For each token, with
``li = cap tanh(i / cap)`` and ``lf = logsigmoid(cap tanh(f / cap))`` the capped log gates:

    m' = max(lf + m, li)
    S' = exp(lf + m - m') S + exp(li - m') k v^T        n' likewise with k alone
    o  = S'^T q / (max(|n' . q|, exp(-m')) + denominator_eps),   q scaled by d^-1/2

Each head's o is divided by its root mean square, the concatenated heads are scaled by a
learned vector, gated with ``sigmoid(g)`` and sent through the output matrix, which adds
into the residual stream.  q, k, v, g and the two gates' pre-activations come from one
product with the concatenated matrix; its result stays in 32-bit, and everything from the
gates to the head norm is 32-bit arithmetic (``csrc/kernels/mlstm.cu``: portions of prompts
chunk by chunk, single tokens in one pass over the state).
"""
from __future__ import annotations

import os

import torch

from ..config.registry import MIXERS
from ..errors import UnsupportedError
from ..kernels import ops
from ..weights import TensorSpec
from .base import FixedState, Mixer
from .linear import Linear


class MLSTM(Mixer):
    """params: hidden_size, num_heads, head_dim (size of q and k per head), value_dim, gate_cap,
    norm_eps (of the head norm) and, optionally, ``denominator_eps`` (default 1e-6) and
    ``projection_names`` (defaults q, k, v, g, i, f, o, norm).  The gates i and f have biases."""

    kernels = ("mlstm",)
    takes_lazy_input = True
    # Steps of this many tokens and more compute all chunks at once, as long as the states at the
    # chunks' starts (32-bit, one per chunk and head) fit this many bytes.
    AT_ONCE_FROM = int(os.environ.get("VIPERA_MLSTM_AT_ONCE_FROM", 256))
    AT_ONCE_MOST_BYTES = 4 << 30

    @staticmethod
    def _names(params):
        return params.get("projection_names", ("q", "k", "v", "g", "i", "f", "o", "norm"))

    @classmethod
    def schema(cls, params, prefix):
        hidden, heads = params["hidden_size"], params["num_heads"]
        d, dv = params["head_dim"], params["value_dim"]
        q, k, v, g, i, f, o, norm = cls._names(params)
        return {
            f"{prefix}.{q}.weight": TensorSpec((heads * d, hidden)),
            f"{prefix}.{k}.weight": TensorSpec((heads * d, hidden)),
            f"{prefix}.{v}.weight": TensorSpec((heads * dv, hidden)),
            f"{prefix}.{g}.weight": TensorSpec((heads * dv, hidden)),
            f"{prefix}.{o}.weight": TensorSpec((hidden, heads * dv)),
            f"{prefix}.{norm}.weight": TensorSpec((heads * dv,), init="norm", store="float32"),
            f"{prefix}.{i}.weight": TensorSpec((heads, hidden)),
            f"{prefix}.{i}.bias": TensorSpec((heads,), init="bias"),
            f"{prefix}.{f}.weight": TensorSpec((heads, hidden)),
            f"{prefix}.{f}.bias": TensorSpec((heads,), init="bias"),
        }

    def __init__(self, params, prefix, tensors, dtype, device):
        super().__init__(params, prefix, tensors, dtype, device)
        self.hidden = int(params["hidden_size"])
        self.heads = int(params["num_heads"])
        self.dim = int(params["head_dim"])
        self.vdim = int(params["value_dim"])
        self.gate_cap = float(params["gate_cap"])
        self.norm_eps = float(params["norm_eps"])
        self.denominator_eps = float(params.get("denominator_eps", 1e-6))
        if not self.gate_cap > 0:
            raise UnsupportedError("the gates' cap must be positive")
        q, k, v, g, i, f, o, norm = self._names(params)
        names = (q, k, v, g, i, f)
        rows = [tensors[f"{prefix}.{n}.weight"] for n in names]
        widths = [r.shape[0] for r in rows]
        # Rows of q, k, v, g, then i and f, padded with zero rows to a multiple of 8.
        total = sum(widths)
        padded = (total + 7) // 8 * 8
        where = rows[0].device    # tensors may come from a file (host) or from a generator on the device
        spare = [torch.zeros(padded - total, self.hidden, dtype=rows[0].dtype, device=where)] if padded > total else []
        fused = torch.cat(rows + spare, dim=0)
        bias = torch.zeros(padded, dtype=torch.float32, device=where)
        offsets, at = [], 0
        for name, width in zip(names, widths):
            offsets.append(at)
            if name in (i, f):
                bias[at:at + width] = tensors[f"{prefix}.{name}.bias"].to(torch.float32)
            at += width
        self.offsets = tuple(offsets)
        self.proj = Linear(fused, dtype, device, bias=bias)
        self.out = Linear(tensors[f"{prefix}.{o}.weight"], dtype, device)
        self.norm_weight = tensors[f"{prefix}.{norm}.weight"].to(device=device, dtype=torch.float32).contiguous()

    def kernel_families(self):
        return tuple(dict.fromkeys(("mlstm",) + self.proj.kernel_families() + self.out.kernel_families()))

    @classmethod
    def cache_request_for(cls, params):
        return FixedState((ops.mlstm_state_floats(int(params["num_heads"]), int(params["head_dim"]),
                                                  int(params["value_dim"])),), torch.float32)

    @classmethod
    def workspace_bytes(cls, params, tokens, element_bytes):
        heads, d, dv = params["num_heads"], params["head_dim"], params["value_dim"]
        width = 2 * heads * (d + dv) + 2 * heads
        return tokens * (width * 4 + heads * dv * (4 + element_bytes)) + tokens * heads * (d + 1) * 4

    def forward(self, ctx, h, residual, cache, writes_cache):
        count = ctx.num_tokens
        ws = ctx.workspace
        proj = ws.get("mlstm.proj", (count, self.proj.out_features), torch.float32)
        self.proj(ctx, h, epilogue=ops.EPI_STORE, out=proj)
        o_raw = ws.get("mlstm.cell", (count, self.heads * self.vdim), torch.float32)
        scratch = ws.get("mlstm.nm", (ctx.num_entries, self.heads * (self.dim + 1)), torch.float32)
        mixed = ws.get("mlstm.out", (count, self.heads * self.vdim), ctx.dtype)
        chunk_scratch = None
        jobs = count // ops.MLSTM_CHUNK + ctx.num_entries
        if (ctx.dtype == torch.bfloat16 and not ctx.all_single and count >= self.AT_ONCE_FROM
                and ops.mlstm_tc_takes(self.dim, self.vdim) and self.vdim % 4 == 0
                and jobs * self.heads * self.dim * self.vdim * 4 <= self.AT_ONCE_MOST_BYTES):
            # a long step: all its chunks at once (a block per chunk) instead of each entry's one after another
            chunk_scratch = (ws.get("mlstm.chunk_states", (jobs, self.heads * self.dim * self.vdim), torch.float32),
                             ws.get("mlstm.chunk_n", (jobs, self.heads * self.dim), torch.float32),
                             ws.get("mlstm.chunk_aux", (jobs, self.heads * 4), torch.float32))
        ops.mlstm(proj, offsets=self.offsets, heads=self.heads, dim=self.dim, vdim=self.vdim,
                  q_scale=self.dim ** -0.5, gate_cap=self.gate_cap, denom_eps=self.denominator_eps,
                  entry_starts=ctx.entry_starts, state_slots=ctx.state_slots, fresh=ctx.fresh,
                  token_entry=ctx.token_entry, num_entries=ctx.num_entries, single=ctx.all_single,
                  state=cache.data, o_raw=o_raw, nm_scratch=scratch, norm_weight=self.norm_weight,
                  norm_eps=self.norm_eps, out=mixed, chunk_scratch=chunk_scratch)
        self.out(ctx, mixed, epilogue=ops.EPI_RESIDUAL, resid=residual)


MIXERS.register("mlstm", MLSTM)
