"""Arrangements of a layer's parts.

An arrangement declares its roles: which named parts it reads from the layer's description
and which registry each comes from.  ``Block`` builds them, so a new arrangement (four norms
around the two sub-layers, a mixer beside the feed-forward, one norm only) is a subclass
that names its roles and writes ``forward``; nothing else changes.

``prenorm``: ``x += mixer(norm(x))``, then ``x += ffn(norm(x))`` — the order of
crates/vipera-backend-cpu/src/model.rs:977-1198.  The residual stream is 32-bit; mixers
and feed-forwards add into it themselves, so that the addition can be the ending of their
last product.
"""
from __future__ import annotations

from typing import Dict

import torch

from ..config.registry import BLOCKS, FEED_FORWARDS, MIXERS, NORMS, Registry
from .base import CacheBundle, FixedState, StateView
from .conv import CausalConv
from .linear import NormedInput


class Block:
    """Base of all arrangements.  ``roles`` maps a role's name to the registry its part is
    looked up in; the built parts are attributes of the same names.  ``cache_role`` names the
    role whose part says what the layer keeps between steps (``cache_request()``); the layer's
    cache slot is handed to ``forward`` and the arrangement passes it on to that part."""

    roles: Dict[str, Registry] = {}
    cache_role = "mixer"

    def __init__(self, layer_spec, tensors, dtype, device):
        self.spec = layer_spec
        self.params = layer_spec.params
        self._parts = {}
        for role, registry in self.roles.items():
            part_spec = self._role_spec(layer_spec, role)
            part = registry.find(part_spec.kind)(part_spec.params, layer_spec.part_prefix(role), tensors, dtype, device)
            setattr(self, role, part)
            self._parts[role] = part

    @classmethod
    def _role_spec(cls, layer_spec, role):
        from ..errors import InvalidArgumentError

        try:
            return layer_spec.parts[role]
        except KeyError:
            raise InvalidArgumentError(
                f"the {layer_spec.block!r} arrangement needs a part for the role {role!r}; "
                f"layer {layer_spec.prefix} gives {sorted(layer_spec.parts)}") from None

    @classmethod
    def schema(cls, layer_spec):
        schema = {}
        for role, registry in cls.roles.items():
            part_spec = cls._role_spec(layer_spec, role)
            schema.update(registry.find(part_spec.kind).schema(part_spec.params, layer_spec.part_prefix(role)))
        return schema

    def parts(self):
        return tuple(self._parts.values())

    def cache_request(self):
        """What this layer keeps between steps: PagedKV, FixedState or None."""
        part = self._parts.get(self.cache_role)
        return None if part is None else part.cache_request()

    @classmethod
    def cache_request_for(cls, layer_spec):
        """The same from the description alone (no weights): for memory plans."""
        if cls.cache_role not in cls.roles:
            return None
        part_spec = cls._role_spec(layer_spec, cls.cache_role)
        return cls.roles[cls.cache_role].find(part_spec.kind).cache_request_for(part_spec.params)

    @classmethod
    def workspace_bytes(cls, layer_spec, tokens, element_bytes):
        """Workspace of one execution of the layer in a step of `tokens` tokens: what its parts
        ask for, together (their buffers have names of their own and live side by side)."""
        total = 0
        for role, registry in cls.roles.items():
            part_spec = cls._role_spec(layer_spec, role)
            total += registry.find(part_spec.kind).workspace_bytes(part_spec.params, tokens, element_bytes)
        return total

    def forward(self, ctx, residual, cache, writes_cache):
        raise NotImplementedError

    @staticmethod
    def _input(part, normed: NormedInput):
        """A part that sets ``takes_lazy_input`` receives the normalised input as a NormedInput
        and may fuse the norm into its first product; any other part receives a tensor."""
        return normed if getattr(part, "takes_lazy_input", False) else normed.tensor()


class PreNormBlock(Block):
    roles = {"mixer_norm": NORMS, "mixer": MIXERS, "ffn_norm": NORMS, "ffn": FEED_FORWARDS}

    def forward(self, ctx, residual, cache, writes_cache):
        h = NormedInput(ctx, self.mixer_norm, residual)
        self.mixer.forward(ctx, self._input(self.mixer, h), residual, cache, writes_cache)
        h = NormedInput(ctx, self.ffn_norm, residual)
        self.ffn.forward(ctx, self._input(self.ffn, h), residual)


class PreNormMixerBlock(Block):
    """A layer without a feed-forward: ``x += mixer(norm(x))`` and nothing more."""

    roles = {"mixer_norm": NORMS, "mixer": MIXERS}

    def forward(self, ctx, residual, cache, writes_cache):
        h = NormedInput(ctx, self.mixer_norm, residual)
        self.mixer.forward(ctx, self._input(self.mixer, h), residual, cache, writes_cache)


class OutNormConvBlock(Block):
    """``x += norm(mixer(c(x)))`` and, where the layer has a feed-forward, ``x += norm(ffn(c(x)))``:
    the norms act on the sublayers' outputs, and what a sublayer reads is the residual stream
    itself with a short causal convolution over time added to it, ``c(h) = h + conv(h)``
    (``params``: ``taps``, ``hidden_size``; tensors ``<layer>.<mixer_conv>.weight`` and
    ``<layer>.<ffn_conv>.weight``, [hidden, taps]).  The last ``taps - 1`` rows of the stream in
    front of each sublayer are kept per request beside what the mixer keeps.

    A sublayer adds its output into the 32-bit stream it is handed; here that is a cleared
    buffer of the stream's shape, which the norm then adds into the stream."""

    roles = {"mixer": MIXERS, "mixer_norm": NORMS}
    optional_roles = {"ffn": FEED_FORWARDS, "ffn_norm": NORMS}
    conv_roles = ("mixer_conv", "ffn_conv")

    def __init__(self, layer_spec, tensors, dtype, device):
        self.roles = self._roles_of(layer_spec)
        super().__init__(layer_spec, tensors, dtype, device)
        self.hidden = int(layer_spec.params["hidden_size"])
        self.has_ffn = "ffn" in layer_spec.parts
        self.mixer_conv = CausalConv(layer_spec.part_prefix("mixer_conv"), tensors, device, add_input=True)
        self.ffn_conv = (CausalConv(layer_spec.part_prefix("ffn_conv"), tensors, device, add_input=True)
                         if self.has_ffn else None)

    @classmethod
    def _roles_of(cls, layer_spec):
        roles = dict(cls.roles)
        if "ffn" in layer_spec.parts:
            roles.update(cls.optional_roles)
        return roles

    @classmethod
    def _conv_state(cls, layer_spec):
        convs = 2 if "ffn" in layer_spec.parts else 1
        taps, hidden = int(layer_spec.params["taps"]), int(layer_spec.params["hidden_size"])
        return FixedState((convs, taps - 1, hidden), torch.float32) if taps > 1 else None

    @classmethod
    def schema(cls, layer_spec):
        schema = {}
        for role, registry in cls._roles_of(layer_spec).items():
            part_spec = cls._role_spec(layer_spec, role)
            schema.update(registry.find(part_spec.kind).schema(part_spec.params, layer_spec.part_prefix(role)))
        taps, hidden = int(layer_spec.params["taps"]), int(layer_spec.params["hidden_size"])
        for role in cls.conv_roles[:2 if "ffn" in layer_spec.parts else 1]:
            schema.update(CausalConv.schema(layer_spec.part_prefix(role), hidden, taps))
        return schema

    def parts(self):
        return tuple(self._parts.values()) + (self.mixer_conv,)

    def cache_request(self):
        return CacheBundle.of(conv=self._conv_state(self.spec), mixer=self.mixer.cache_request())

    @classmethod
    def cache_request_for(cls, layer_spec):
        part_spec = cls._role_spec(layer_spec, "mixer")
        return CacheBundle.of(conv=cls._conv_state(layer_spec),
                              mixer=MIXERS.find(part_spec.kind).cache_request_for(part_spec.params))

    @classmethod
    def workspace_bytes(cls, layer_spec, tokens, element_bytes):
        total = tokens * int(layer_spec.params["hidden_size"]) * (4 + element_bytes)   # the cleared stream and c(x)
        for role, registry in cls._roles_of(layer_spec).items():
            part_spec = cls._role_spec(layer_spec, role)
            total += registry.find(part_spec.kind).workspace_bytes(part_spec.params, tokens, element_bytes)
        return total

    def forward(self, ctx, residual, cache, writes_cache):
        ws = ctx.workspace
        cache = cache or {}
        conv_state = cache.get("conv")
        branch = ws.get("block.branch", (ctx.num_tokens, self.hidden), torch.float32)
        h = ws.get("block.h", (ctx.num_tokens, self.hidden), ctx.dtype)
        self.mixer_conv(ctx, residual, None if conv_state is None else StateView(conv_state.data[:, 0]),
                        out=h, clear=branch)
        self.mixer.forward(ctx, h, branch, cache.get("mixer"), writes_cache)
        self.mixer_norm.add_into(ctx, branch, residual)
        if self.has_ffn:
            self.ffn_conv(ctx, residual, None if conv_state is None else StateView(conv_state.data[:, 1]),
                          out=h, clear=branch)
            self.ffn.forward(ctx, h, branch)
            self.ffn_norm.add_into(ctx, branch, residual)


BLOCKS.register("prenorm", PreNormBlock)
BLOCKS.register("outnorm_conv", OutNormConvBlock)
BLOCKS.register("prenorm_mixer", PreNormMixerBlock)
