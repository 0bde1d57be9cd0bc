"""Two mixers side by side on the same input: ``x += left_scale * left(h) + right_scale * right(h)``.

Either side is any registered mixer.  One cache entry serves both: the pages are the left side's (the right side must
keep nothing per position), and the entry's per-sequence state holds the left side's state and then the right side's,
which each side finds through its ``state_offset`` (both sides must say ``honours_state_offset``).  A side that can
scale its own result (``scales_output``) adds straight into the stream; the other stores its result into a scratch
buffer that ``add_scaled`` adds with its weight.
"""
from __future__ import annotations

import torch

from .base import CacheRequest, Mixer
from .registry import part_class, register_mixer


class _Positions:
    """The position tables of both sides, as the model prepares them before a graph capture."""

    def __init__(self, sides):
        self.sides = [side.position for side in sides if getattr(side, "position", None) is not None]

    def ensure(self, positions: int) -> None:
        for side in self.sides:
            side.ensure(positions)


class MixerPair(Mixer):
    stores_branch = True

    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        self.left = part_class("mixer", spec.left.kind)(spec.left, runtime)
        self.right = part_class("mixer", spec.right.kind)(spec.right, runtime)
        left_request, right_request = self._requests(spec)
        for side, request in ((self.left, left_request), (self.right, right_request)):
            if request.state_bytes and not getattr(side, "honours_state_offset", False):
                raise ValueError(f"mixer_pair: a '{side.spec.kind}' mixer cannot share a cache entry's state")
        self.left.state_offset = 0
        self.right.state_offset = left_request.state_bytes // 4
        self.graph_safe = self.left.graph_safe and self.right.graph_safe
        self.position = _Positions((self.left, self.right))
        for side, scale in ((self.left, spec.left_scale), (self.right, spec.right_scale)):
            if getattr(side, "scales_output", False):
                side.out_scale = float(scale)

    @staticmethod
    def _requests(spec):
        left = part_class("mixer", spec.left.kind).cache_request(spec.left)
        right = part_class("mixer", spec.right.kind).cache_request(spec.right)
        if right.kind != "none":
            raise ValueError("mixer_pair: the right side must keep nothing per position (the pages are the left side's)")
        if left.state_bytes % 4 or right.state_bytes % 4:
            raise ValueError("mixer_pair: per-sequence state is counted in whole floats")
        return left, right

    @classmethod
    def expected_tensors(cls, spec):
        wanted = dict(part_class("mixer", spec.left.kind).expected_tensors(spec.left))
        wanted.update(part_class("mixer", spec.right.kind).expected_tensors(spec.right))
        return wanted

    @classmethod
    def cache_request(cls, spec):
        left, right = cls._requests(spec)
        return CacheRequest(left.kind, left.num_kv_heads, left.head_dim, left.window,
                            state_bytes=left.state_bytes + right.state_bytes, v_head_dim=left.v_head_dim, extra=left.extra)

    def bind(self, tensors):
        self.left.bind(tensors)
        self.right.bind(tensors)

    @staticmethod
    def _direct(side, scale) -> bool:
        """True if the side can put its weighted result straight into the stream."""
        return side.stores_branch and (getattr(side, "scales_output", False) or scale == 1.0)

    @staticmethod
    def _into(side, step, h, target, cache_entry, writes_cache, store: bool) -> None:
        if store and not side.stores_branch:          # the side only knows how to add: hand it zeros
            target.zero_()
            store = False
        step.store_branch = store
        try:
            side.forward(step, h, target, cache_entry, writes_cache)
        finally:
            step.store_branch = False

    def forward(self, step, h, x, cache_entry, writes_cache=True):
        s, ops = self.spec, self.rt.kernels()
        storing = bool(getattr(step, "store_branch", False))      # the arrangement wants the result stored, not added
        if step.residual_stats is not None:
            step.residual_stats.invalidate()
        # a side that writes straight into the stream goes first, so that it may overwrite where the result is stored
        sides = sorted(((self.left, s.left_scale), (self.right, s.right_scale)),
                       key=lambda pair: not self._direct(*pair))
        written = False
        try:
            for side, scale in sides:
                if self._direct(side, scale):
                    self._into(side, step, h, x, cache_entry, writes_cache, store=storing and not written)
                else:
                    if storing and not written:
                        x.zero_()
                    branch = self.rt.workspace.get("pair_branch", tuple(x.shape), torch.float32)
                    self._into(side, step, h, branch, cache_entry, writes_cache, store=True)
                    ops.add_scaled(x, branch, scale)
                written = True
        finally:
            step.store_branch = storing


register_mixer("mixer_pair", MixerPair)
