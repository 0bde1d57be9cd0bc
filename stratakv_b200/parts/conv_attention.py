"""Causal grouped-query attention whose queries and keys pass a short convolution over time, with rotary positions, a
sliding window, a sink in the softmax, and values that are the keys.

For the mixer's input h, H query heads on G key heads of d numbers::

    q, k = conv(Wq h + bq), conv(Wk h + bk)      conv(u)_p = sum_j w[:, j] u_(p - taps + 1 + j), zeros before p = 0
    v    = k                                      the convolved keys, before rotation; there is no value projection
    q, k = rot(q), rot(k)                         rotary positions on the first rope.dims numbers of every head
    score(i, j) = (q_i . k_j) scale               over 0 <= i - j < window (window 0: every earlier key)
    out  = softmax with exp(sink_h) as one more term of the denominator, times v;   x += Wo out

Kernels: one projection ``[q | k]`` (float32 out), ``short_conv_rotary`` (bias, convolution, rotation, queries out, keys
and values into the paged cache; all float32), ``short_conv_remember`` (the state a sequence keeps: the biased
projections of its last ``taps - 1`` positions), attention over the cache (prompts of head size 64 or 128 in bfloat16 on
the tensor-core kernel and their one-token steps on the split kernel, everything else on the kernel with run-time head
sizes, its one-token steps with the keys cut into parts), the output projection.  ``state_offset`` (floats): where this mixer's state starts in its cache entry's rows, for
a mixer that shares the entry with another.
"""
from __future__ import annotations

import torch

from .. import ops as _ops
from .attention import _residual_mode, _residual_stats
from .base import CacheRequest, Mixer, TensorRequest
from .position import RotaryTable
from .registry import register_mixer


class ConvAttention(Mixer):
    graph_safe = True
    stores_branch = True
    honours_state_offset = True

    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        if spec.num_heads % spec.num_kv_heads != 0:
            raise ValueError("conv_attention: heads must be a multiple of kv heads")
        if spec.rope is not None and (spec.rope.dims > spec.head_dim or spec.rope.dims % 2):
            raise ValueError("conv_attention: the rotated numbers must be an even count within a head")
        if spec.head_dim > 256:
            raise ValueError(f"conv_attention: heads of {spec.head_dim} numbers are not supported (at most 256)")
        if spec.taps > 0 and not (spec.q_conv and spec.k_conv):
            raise ValueError("conv_attention: a convolution needs its two weights")
        if runtime.dtype == torch.bfloat16 and spec.hidden_size % 8 != 0:
            raise ValueError(f"conv_attention: hidden size {spec.hidden_size} is not supported in bfloat16 "
                             "(rows of 16 bytes are needed: a multiple of 8); float32 takes any size")
        self.q_dim = spec.num_heads * spec.head_dim
        self.k_dim = spec.num_kv_heads * spec.head_dim
        self.channels = self.q_dim + self.k_dim
        self.fused_width = -(-self.channels // 8) * 8
        self.ctx_width = -(-self.q_dim // 8) * 8           # whole 16 bytes for the output projection
        self.position = RotaryTable(spec.rope, runtime) if spec.rope is not None else None
        self.state_offset = 0

    @classmethod
    def expected_tensors(cls, spec):
        q_dim, k_dim = spec.num_heads * spec.head_dim, spec.num_kv_heads * spec.head_dim
        wanted = {spec.q_weight: TensorRequest((q_dim, spec.hidden_size)),
                  spec.k_weight: TensorRequest((k_dim, spec.hidden_size)),
                  spec.o_weight: TensorRequest((spec.hidden_size, q_dim))}
        if spec.taps > 0:
            wanted[spec.q_conv] = TensorRequest((q_dim, spec.taps), "conv_taps")
            wanted[spec.k_conv] = TensorRequest((k_dim, spec.taps), "conv_taps")
        for name, width in ((spec.q_bias, q_dim), (spec.k_bias, k_dim)):
            if name:
                wanted[name] = TensorRequest((width,))
        if spec.sink:
            wanted[spec.sink] = TensorRequest((spec.num_heads,))
        return wanted

    @classmethod
    def state_floats(cls, spec) -> int:
        return spec.taps * (spec.num_heads + spec.num_kv_heads) * spec.head_dim if spec.taps > 1 else 0

    @classmethod
    def cache_request(cls, spec):
        return CacheRequest("kv_window" if spec.window > 0 else "kv", spec.num_kv_heads, spec.head_dim, spec.window,
                            state_bytes=4 * cls.state_floats(spec))

    def bind(self, tensors):
        s, rt = self.spec, self.rt
        parts = [rt.upload(tensors[s.q_weight]), rt.upload(tensors[s.k_weight])]
        if self.channels < self.fused_width:          # (zero rows: what they produce is never read)
            parts.append(parts[0].new_zeros(self.fused_width - self.channels, s.hidden_size))
        self.w_qk = torch.cat(parts, dim=0).contiguous()
        del parts
        w_o = rt.upload(tensors[s.o_weight])
        if self.ctx_width != self.q_dim:
            w_o = torch.cat([w_o, w_o.new_zeros(s.hidden_size, self.ctx_width - self.q_dim)], dim=1)
        self.w_o = w_o.contiguous()
        as_float = lambda name: rt.upload(tensors[name], torch.float32).contiguous()
        self.bias = None
        if s.q_bias or s.k_bias:
            zeros = lambda width: torch.zeros(width, dtype=torch.float32, device=rt.device)
            self.bias = torch.cat([as_float(s.q_bias).reshape(-1) if s.q_bias else zeros(self.q_dim),
                                   as_float(s.k_bias).reshape(-1) if s.k_bias else zeros(self.k_dim)]).contiguous()
        self.conv_w = (torch.cat([as_float(s.q_conv), as_float(s.k_conv)], dim=0).contiguous() if s.taps > 0 else None)
        self.sink = as_float(s.sink).reshape(-1) if s.sink else None

    def forward(self, step, h, x, cache_entry, writes_cache=True):
        s, rt = self.spec, self.rt
        ops = rt.kernels()
        n = h.shape[0]
        fused = rt.workspace.get("qkv", (n, self.fused_width), torch.float32)
        ops.linear(h, self.w_qk, fused, _ops.MODE_STORE_F32)
        k_cache, v_cache = step.cache.entry_kv(cache_entry)
        table = step.block_tables[step.cache.entry_group_index(cache_entry)]
        state = step.cache.state(cache_entry).view(torch.float32) if s.taps > 1 else None
        meta = (step.positions, step.token_seq, step.cu_q, step.slot_ids)
        q = rt.workspace.get("q", (n, self.q_dim), rt.dtype)
        cos_sin = self.position.fusion_table(step.max_ctx) if self.position is not None else None
        rotated = s.rope.dims if s.rope is not None else 0
        ops.short_conv_rotary(fused, self.bias, self.conv_w, s.taps, cos_sin, rotated,
                              bool(s.rope is not None and s.rope.interleaved), table, q, k_cache, v_cache, s.num_heads,
                              s.num_kv_heads, s.head_dim, step.cache.block_size, writes_cache, meta, state,
                              self.state_offset)
        if writes_cache:
            ops.short_conv_remember(fused, self.bias, self.channels, s.taps, step.n_seqs, meta, state, self.state_offset)
        ctx = rt.workspace.get("attn_ctx", (n, self.ctx_width), rt.dtype)
        self._attend(step, q, ctx, k_cache, v_cache, table)
        ops.linear(ctx, self.w_o, x, _residual_mode(step), stats=_residual_stats(step))

    def _tensor_core_prompt(self, step) -> bool:
        s, rt = self.spec, self.rt
        block_size = step.cache.block_size
        return (rt.dtype == torch.bfloat16 and rt.device.type == "cuda" and s.head_dim in (64, 128)
                and self.ctx_width == self.q_dim and step.max_q_len > 32 and block_size & (block_size - 1) == 0
                and block_size >= 16 and step.n_seqs * -(-step.max_q_len // 128) <= 65535
                and rt.kernels(s.head_dim).has_attention_prefill_tc())

    def _attend(self, step, q, ctx, k_cache, v_cache, table):
        s, rt = self.spec, self.rt
        n = q.shape[0]
        block_size = step.cache.block_size
        if self._tensor_core_prompt(step):
            rt.kernels(s.head_dim).attention_prefill_tc(
                q, k_cache, v_cache, table, step.cu_q, step.ctx_after, ctx, step.max_q_len, s.num_heads, s.num_kv_heads,
                s.head_dim, block_size, s.scale, s.window, sink=self.sink)
            return
        if (step.is_decode and rt.dtype == torch.bfloat16 and rt.device.type == "cuda" and s.head_dim in (64, 128)
                and self.ctx_width == self.q_dim and block_size % 16 == 0):
            # one token a sequence at a head size the split kernel is built for: the query heads of a key head as
            # rows of a tensor-core product, the context in pieces, the sink in the merge
            from .attention import decode_splits
            blocks_per_seq = s.num_kv_heads * (-(-(s.num_heads // s.num_kv_heads) // 16))
            keys = min(step.max_ctx, s.window) if s.window > 0 else step.max_ctx
            splits = decode_splits(n, blocks_per_seq, keys, rt.sm_count)
            scratch_o = scratch_ml = None
            if splits > 1:
                scratch_o = rt.workspace.get("attn_split_o", (n * s.num_heads * splits * s.head_dim,), torch.float32)
                scratch_ml = rt.workspace.get("attn_split_ml", (n * s.num_heads * splits * 2,), torch.float32)
            rt.kernels(s.head_dim).attention_decode(q, k_cache, v_cache, table, step.ctx_after, ctx, s.num_heads,
                                                    s.num_kv_heads, s.head_dim, block_size, s.scale, s.window, splits,
                                                    scratch_o, scratch_ml, sink=self.sink)
            return
        splits, scratch_o, scratch_ml = 1, None, None
        if step.is_decode:
            # few tokens over long contexts: each (token, head)'s visible keys in parts that run side by side
            keys = min(step.max_ctx, s.window) if s.window > 0 else step.max_ctx
            splits = max(1, min(-(-rt.sm_count * 32 // (n * s.num_heads)), -(-keys // 64), 64))
            if splits > 1:
                scratch_o = rt.workspace.get("attn_split_o", (n * s.num_heads * splits * s.head_dim,), torch.float32)
                scratch_ml = rt.workspace.get("attn_split_ml", (n * s.num_heads * splits * 2,), torch.float32)
        rt.kernels().attention_general(q, k_cache, v_cache, table, step.positions, step.token_seq, ctx, s.num_heads,
                                       s.num_kv_heads, s.head_dim, s.head_dim, block_size, s.scale, s.window,
                                       sink=self.sink, splits=splits, scratch_o=scratch_o, scratch_ml=scratch_ml)


register_mixer("conv_attention", ConvAttention)
