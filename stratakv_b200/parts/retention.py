"""Retention: linear attention with a fixed decay per head, no softmax and no denominator.

For the mixer's input h, H heads, key size d and value size dv::

    q = rot(Wq h),  k = rot(Wk h) * d^-1/2,  v = Wv h          rot: rotary positions on the first rope.dims numbers
    S_t = decay_h S_(t-1) + k_t v_t^T                          a d x dv matrix per head, zero before the first token
    o_t = S_t^T q_t;   o / rms(o) per head;   x += Wo (o * silu(Wg h))

Kernels: one projection for q, k, v and the gate (float32 out), ``ops.retention`` (rotation, the recurrence in chunks
for prompts or in one fused kernel for one token a sequence, the heads' norm and the gate; all float32), the output
projection.  The cache keeps nothing per position: per sequence its state area holds S twice, in the half chosen by
the parity of the last position written (``csrc/retention.cu`` says why).
"""
from __future__ import annotations

import torch

from .. import ops as _ops
from .attention import _residual_mode, _residual_stats
from .base import CacheRequest, Mixer, TensorRequest
from .position import RotaryTable
from .registry import register_mixer


class Retention(Mixer):
    graph_safe = True
    stores_branch = True

    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        if len(spec.decay) != spec.num_heads:
            raise ValueError("retention: one decay per head is needed")
        if spec.rope is not None and (spec.rope.dims > spec.head_dim or spec.rope.dims % 2):
            raise ValueError("retention: the rotated numbers must be an even count within a head")
        if runtime.dtype == torch.bfloat16 and spec.hidden_size % 8 != 0:
            raise ValueError(f"retention: hidden size {spec.hidden_size} is not supported in bfloat16 "
                             "(rows of 16 bytes are needed: a multiple of 8); float32 takes any size")
        self.qk_dim = spec.num_heads * spec.head_dim
        self.v_dim = spec.num_heads * spec.v_head_dim
        self.fused_width = -(-(2 * self.qk_dim + 2 * self.v_dim) // 8) * 8
        self.out_width = -(-self.v_dim // 8) * 8            # whole 16 bytes for the output projection
        self.position = RotaryTable(spec.rope, runtime) if spec.rope is not None else None

    @classmethod
    def expected_tensors(cls, spec):
        qk, v = spec.num_heads * spec.head_dim, spec.num_heads * spec.v_head_dim
        return {spec.q_weight: TensorRequest((qk, spec.hidden_size)), spec.k_weight: TensorRequest((qk, spec.hidden_size)),
                spec.v_weight: TensorRequest((v, spec.hidden_size)), spec.gate_weight: TensorRequest((v, spec.hidden_size)),
                spec.o_weight: TensorRequest((spec.hidden_size, v))}

    @classmethod
    def cache_request(cls, spec):
        return CacheRequest(kind="none", state_bytes=4 * 2 * spec.num_heads * spec.head_dim * spec.v_head_dim)

    def bind(self, tensors):
        s, rt = self.spec, self.rt
        parts = [rt.upload(tensors[name]) for name in (s.q_weight, s.k_weight, s.v_weight, s.gate_weight)]
        rows = sum(part.shape[0] for part in parts)
        if rows < self.fused_width:                 # (zero rows: what they produce is never read)
            parts.append(parts[0].new_zeros(self.fused_width - rows, s.hidden_size))
        self.w_fused = torch.cat(parts, dim=0).contiguous()
        del parts
        self.decay = torch.tensor(list(s.decay), dtype=torch.float32).to(rt.device)
        w_o = rt.upload(tensors[s.o_weight])
        if self.out_width != self.v_dim:
            w_o = torch.cat([w_o, w_o.new_zeros(s.hidden_size, self.out_width - self.v_dim)], dim=1)
        self.w_o = w_o.contiguous()

    def forward(self, step, h, x, cache_entry, writes_cache=True):
        s, rt = self.spec, self.rt
        ops = rt.kernels()
        n = h.shape[0]
        fused = rt.workspace.get("qkv", (n, self.fused_width), torch.float32)
        ops.linear(h, self.w_fused, fused, _ops.MODE_STORE_F32)
        table = self.position.fusion_table(step.max_ctx) if self.position is not None else None
        state = step.cache.state(cache_entry).view(torch.float32)
        mixed = rt.workspace.get("retention_out", (n, self.out_width), rt.dtype)
        need = ops.retention_scratch(step.n_seqs, step.max_q_len, s.num_heads, s.head_dim, s.v_head_dim)
        scratch = rt.workspace.get("retention_chunks", (need,), torch.float32) if need else None
        ops.retention(fused, table, s.rope.dims if s.rope is not None else 0, self.decay, s.eps, mixed, state,
                      (step.positions, step.token_seq, step.cu_q, step.slot_ids), s.num_heads, s.head_dim,
                      s.v_head_dim, step.max_q_len, scratch)
        ops.linear(mixed, self.w_o, x, _residual_mode(step), stats=_residual_stats(step))


register_mixer("retention", Retention)
