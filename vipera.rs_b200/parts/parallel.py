"""Mixers side by side: every branch reads the same input, and the layer's mixer output is the
sum of the branches' outputs, each times a constant.

A branch is any registered mixer that takes ``out_scale`` among its parameters (it multiplies
its own output, so the sum forms where the branches add into the stream they are handed).  The
tensors of branch ``name`` live under ``<prefix>.<name>``; what the branches keep between steps
is bundled under their names.
"""
from __future__ import annotations

from ..config.registry import MIXERS
from ..config.spec import PartSpec
from .base import CacheBundle, Mixer


class ParallelMixers(Mixer):
    """params: ``branches``, a sequence of (name, PartSpec of a mixer, scale)."""

    @staticmethod
    def _branches(params):
        for name, part, scale in params["branches"]:
            yield name, MIXERS.find(part.kind), {**part.params, "out_scale": float(scale) * float(part.params.get("out_scale", 1.0))}

    @classmethod
    def schema(cls, params, prefix):
        schema = {}
        for name, kind, branch_params in cls._branches(params):
            schema.update(kind.schema(branch_params, f"{prefix}.{name}"))
        return schema

    def __init__(self, params, prefix, tensors, dtype, device):
        super().__init__(params, prefix, tensors, dtype, device)
        self.branches = [(name, kind(branch_params, f"{prefix}.{name}", tensors, dtype, device))
                         for name, kind, branch_params in self._branches(params)]
        self.graph_safe = all(getattr(branch, "graph_safe", True) for _, branch in self.branches)

    def kernel_families(self):
        names = ()
        for _, branch in self.branches:
            names += tuple(branch.kernel_families())
        return tuple(dict.fromkeys(names))

    def prepare(self, max_positions: int) -> None:
        for _, branch in self.branches:
            prepare = getattr(branch, "prepare", None)
            if prepare is not None:
                prepare(max_positions)

    @classmethod
    def cache_request_for(cls, params):
        return CacheBundle.of(**{name: kind.cache_request_for(branch_params)
                                 for name, kind, branch_params in cls._branches(params)})

    @classmethod
    def workspace_bytes(cls, params, tokens, element_bytes):
        return sum(kind.workspace_bytes(branch_params, tokens, element_bytes)
                   for _, kind, branch_params in cls._branches(params))

    def forward(self, ctx, h, residual, cache, writes_cache):
        cache = cache or {}
        for name, branch in self.branches:
            branch.forward(ctx, h, residual, cache.get(name), writes_cache)


MIXERS.register("parallel", ParallelMixers)
