"""Rotary position encoding with split-half pairs.

For pair ``i`` of a head: ``f_i = theta^(-2i/d)`` computed in double and stored
as float; ``angle = position * f_i`` in double; cos and sin in double, then
rounded to float; ``x[i], x[i+d/2] = x1*cos - x2*sin, x1*sin + x2*cos``
(``src/layers/attention.cpp:63-69, 96-135``).  The table of (cos, sin) is built
on the host with exactly those steps and grows when a longer position is asked
for; the kernel that applies it also writes keys and values into the cache.
"""
from __future__ import annotations

import math

import numpy as np
import torch

from .registry import register_position


def rope_table(head_dim: int, theta: float, positions: int) -> np.ndarray:
    """``[positions, head_dim/2, 2]`` float32 of (cos, sin)."""
    half = head_dim // 2
    exponent = -2.0 * np.arange(half, dtype=np.float64) / float(head_dim)
    inv_freq = np.power(np.float64(theta), exponent).astype(np.float32)
    angle = np.arange(positions, dtype=np.float64)[:, None] * inv_freq.astype(np.float64)[None, :]
    return np.stack([np.cos(angle), np.sin(angle)], axis=-1).astype(np.float32)


class RopeHalf:
    role = "position"

    def __init__(self, spec, runtime):
        self.spec = spec
        self.rt = runtime
        self.table = None
        self.length = 0
        self._retired = []          # earlier tables stay alive: captured graphs may still read them

    def ensure(self, positions: int) -> None:
        """Make the table cover positions ``0 .. positions-1`` (never inside a graph capture)."""
        if positions <= self.length:
            return
        length = max(positions, 2 * self.length, 256)
        if self.table is not None:
            self._retired.append(self.table)
        host = torch.from_numpy(rope_table(self.spec.head_dim, self.spec.theta, length))
        self.table = host.to(self.rt.device).contiguous()
        self.length = length

    def fusion_table(self, max_positions: int):
        """The (cos, sin) table for kernels that rotate queries and keys themselves."""
        self.ensure(max_positions)
        return self.table

    def rotate_and_store(self, step, qkv, q_out, k_cache, v_cache, block_table, num_heads, num_kv_heads,
                         head_dim, block_size, write_kv):
        if head_dim != self.spec.head_dim:
            raise ValueError("rotary table was built for another head size")
        self.ensure(step.max_ctx)
        self.rt.kernels(head_dim).rope_kv_write(
            qkv, self.table, step.positions, step.token_seq, block_table, q_out, k_cache, v_cache,
            num_heads, num_kv_heads, head_dim, block_size, write_kv)


class NoPosition:
    """No position encoding: queries and keys pass unrotated into the cache."""
    role = "position"

    def __init__(self, spec, runtime):
        self.spec = spec
        self.rt = runtime

    def ensure(self, positions: int) -> None:
        pass

    def fusion_table(self, max_positions: int):
        return None

    def rotate_and_store(self, step, qkv, q_out, k_cache, v_cache, block_table, num_heads, num_kv_heads,
                         head_dim, block_size, write_kv):
        self.rt.kernels(head_dim).rope_kv_write(
            qkv, None, step.positions, step.token_seq, block_table, q_out, k_cache, v_cache,
            num_heads, num_kv_heads, head_dim, block_size, write_kv)


def rotary_table(spec, positions: int) -> np.ndarray:
    """``[positions, dims/2, 2]`` float32 of (cos, sin) for a ``RotarySpec``: frequencies and angles in double, the
    stretch of the frequencies (``YarnSpec``) and its factor on cosines and sines included, rounded to float last."""
    dims, base = spec.dims, float(spec.base)
    half = dims // 2
    index = np.arange(half, dtype=np.float64)
    freq = np.power(np.float64(base), -2.0 * index / float(dims))
    magnitude = 1.0
    scaling = spec.scaling
    if scaling is not None:
        def pair_of(turns):
            return dims * math.log(scaling.original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))
        lo = max(math.floor(pair_of(scaling.fast)), 0)
        hi = min(math.ceil(pair_of(scaling.slow)), dims - 1)
        ramp = np.clip((index - lo) / max(hi - lo, 0.001), 0.0, 1.0)
        freq = freq / scaling.factor * ramp + freq * (1.0 - ramp)
        magnitude = 0.1 * math.log(scaling.factor) + 1.0
    angle = np.arange(positions, dtype=np.float64)[:, None] * freq[None, :]
    return (np.stack([np.cos(angle), np.sin(angle)], axis=-1) * magnitude).astype(np.float32)


class RotaryTable:
    """A (cos, sin) table for rotations over part of a vector, with or without stretched frequencies; the mixers
    that use it hand ``table`` and ``spec.dims`` to their kernels."""
    role = "position"

    def __init__(self, spec, runtime):
        self.spec = spec
        self.rt = runtime
        self.table = None
        self.length = 0
        self._retired = []          # earlier tables stay alive: captured graphs may still read them

    def ensure(self, positions: int) -> None:
        """Make the table cover positions ``0 .. positions-1`` (never inside a graph capture)."""
        if positions <= self.length:
            return
        length = max(positions, 2 * self.length, 256)
        if self.table is not None:
            self._retired.append(self.table)
        self.table = torch.from_numpy(rotary_table(self.spec, length)).to(self.rt.device).contiguous()
        self.length = length

    def fusion_table(self, max_positions: int):
        self.ensure(max_positions)
        return self.table


register_position("rotary_table", RotaryTable)
register_position("rope_half", RopeHalf)
register_position("none", NoPosition)
