"""Causal attention over one compressed vector per position.

``c = rmsnorm(Wdkv h) * w`` is what the cache keeps (``latent_dim`` numbers a position, cache kind ``latent``).
Head h's keys and values are ``Wuk[h] c`` and ``Wuv[h] c``; they are never made.  Since
``q . (Wuk[h] c) = (Wuk[h]^T q) . c`` and ``sum_j p_j Wuv[h] c_j = Wuv[h] (sum_j p_j c_j)``, the mixer folds the
keys' up-projection into the queries (``headwise_linear`` with the transposed matrices), attends with every head over
the same cached vectors as keys and as values (the attention kernels with one key/value head of ``latent_dim``), and
applies the values' up-projection to each head's result.  No position encoding.

A design may add (``LatentAttentionSpec``): a rotated part of ``rope_dim`` numbers on every query head and ONE rotated key
part per position that all heads share, cached behind the latent (the folded query of a head is then
``[Wuk[h]^T q_plain | q_rotated]`` against the cached ``[c | k_rotated]``, and the values are the first ``latent_dim``
numbers of the same cached row); a sink per head in the softmax's denominator; a gate per head on the output; and a
layer that attends over the cache another layer wrote.  Any of these takes the folded way on the general attention
kernel in both dtypes.

That is how one token a sequence runs, and every step in float32.  A prompt in bfloat16 whose heads have a size the
tensor-core prompt kernel is built for goes the other way round: the cached vectors of the step's sequences are
gathered, up-projected by one GEMM into keys and values of all heads, laid out as pages of a scratch cache, and
attended over as ordinary multi-head attention; the work per key is then ``head_dim`` and not ``latent_dim`` numbers.
"""
from __future__ import annotations

import numpy as np
import torch

from .. import ops as _ops
from ..cache.kinds import CacheKind, register_cache_kind
from .attention import _residual_mode, _residual_stats
from .base import CacheRequest, Mixer, TensorRequest
from .position import RotaryTable
from .registry import register_mixer

register_cache_kind(CacheKind("latent", paged=True, windowed=False,
                              block_tensors=lambda request, block_size: {"c": (1, block_size, request.head_dim)}))


def _extended(spec) -> bool:
    """True if the spec uses a mechanism beyond the plain latent: a rotated part, a sink, a gate, a borrowed cache."""
    return bool(getattr(spec, "rope_dim", 0) or getattr(spec, "sink", None) or getattr(spec, "gate_weight", None)
                or getattr(spec, "shares_kv", False))


class LatentAttention(Mixer):
    graph_safe = True
    stores_branch = True

    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        if runtime.dtype == torch.bfloat16 and spec.hidden_size % 8 != 0:
            raise ValueError(f"latent attention: hidden size {spec.hidden_size} is not supported in bfloat16 "
                             "(rows of 16 bytes are needed: a multiple of 8); float32 takes any size")
        if spec.latent_dim > 512:
            raise ValueError(f"latent attention: a latent of {spec.latent_dim} numbers is not supported (at most 512)")
        self.extended = _extended(spec)
        self.rope_dim = getattr(spec, "rope_dim", 0)
        if bool(self.rope_dim) != (getattr(spec, "rope", None) is not None) or (self.rope_dim and spec.rope.dims > self.rope_dim):
            raise ValueError("latent attention: a rotated part needs its rotation, over at most that many numbers")
        self.q_head = spec.head_dim + self.rope_dim         # a query head: unrotated numbers, then rotated ones
        self.key_dim = spec.latent_dim + self.rope_dim      # a cached row: the latent, then the shared rotated key part
        self.q_dim = spec.num_heads * self.q_head
        self.ctx_dim = spec.num_heads * spec.v_head_dim
        self.ctx_width = -(-self.ctx_dim // 8) * 8          # whole 16 bytes for the output projection
        # rows of the fused projection: queries, then (a layer with a cache of its own) the latent and the key part,
        # then the gate's logits
        self.shares_kv = bool(getattr(spec, "shares_kv", False))
        self.gate_offset = self.q_dim + (0 if self.shares_kv else self.key_dim)
        self.has_gate = getattr(spec, "gate_weight", None) is not None
        self.fused_width = -(-(self.gate_offset + (spec.num_heads if self.has_gate else 0)) // 8) * 8
        self.position = RotaryTable(spec.rope, runtime) if self.rope_dim else None

    @classmethod
    def expected_tensors(cls, spec):
        rope_dim = getattr(spec, "rope_dim", 0)
        wanted = {spec.q_weight: TensorRequest((spec.num_heads * (spec.head_dim + rope_dim), spec.hidden_size)),
                  spec.k_up_weight: TensorRequest((spec.num_heads * spec.head_dim, spec.latent_dim)),
                  spec.v_up_weight: TensorRequest((spec.num_heads * spec.v_head_dim, spec.latent_dim)),
                  spec.o_weight: TensorRequest((spec.hidden_size, spec.num_heads * spec.v_head_dim))}
        if not getattr(spec, "shares_kv", False):
            wanted[spec.down_weight] = TensorRequest((spec.latent_dim + rope_dim, spec.hidden_size))
            wanted[spec.latent_norm] = TensorRequest((spec.latent_dim,), "around_one")
        if getattr(spec, "sink", None) is not None:
            wanted[spec.sink] = TensorRequest((spec.num_heads,))
        if getattr(spec, "gate_weight", None) is not None:
            wanted[spec.gate_weight] = TensorRequest((spec.num_heads, spec.hidden_size))
        return wanted

    @classmethod
    def cache_request(cls, spec):
        return CacheRequest("latent", 1, spec.latent_dim + getattr(spec, "rope_dim", 0))

    def bind(self, tensors):
        s = self.spec
        parts = [self.rt.upload(tensors[s.q_weight])]
        if not self.shares_kv:
            parts.append(self.rt.upload(tensors[s.down_weight]))
        if self.has_gate:
            parts.append(self.rt.upload(tensors[s.gate_weight]))
        rows = sum(part.shape[0] for part in parts)
        if rows < self.fused_width:                 # (zero rows: what they produce is never read)
            parts.append(parts[0].new_zeros(self.fused_width - rows, s.hidden_size))
        self.w_q_down = torch.cat(parts, dim=0).contiguous()
        del parts
        self.latent_gamma = self.rt.upload(tensors[s.latent_norm], torch.float32) if not self.shares_kv else None
        self.sink = (self.rt.upload(tensors[s.sink], torch.float32).reshape(-1).contiguous()
                     if getattr(s, "sink", None) is not None else None)
        k_up = self.rt.upload(tensors[s.k_up_weight]).view(s.num_heads, s.head_dim, s.latent_dim)
        self.w_k_up_t = k_up.transpose(1, 2).contiguous()       # [heads, latent, head_dim]: q -> q in latent space
        self.w_v_up = self.rt.upload(tensors[s.v_up_weight]).view(s.num_heads, s.v_head_dim, s.latent_dim).contiguous()
        # keys' and values' up-projections as one matrix, for steps that make every head's keys and values
        self.w_kv_up = (torch.cat([self.rt.upload(tensors[s.k_up_weight]), self.rt.upload(tensors[s.v_up_weight])],
                                  dim=0).contiguous() if not self.extended else None)
        # the same for a layer with a rotated part: a cached row is [latent | rotated key part], and rows of the
        # identity copy the rotated part behind every head's unrotated keys (exactly: one product a number)
        self.w_kv_whole = None
        if (self.extended and self.rt.dtype == torch.bfloat16 and self.q_head == s.v_head_dim and self.q_head in (64, 128)
                and self.key_dim % 8 == 0):
            k_up = self.rt.upload(tensors[s.k_up_weight]).view(s.num_heads, s.head_dim, s.latent_dim)
            keys = k_up.new_zeros(s.num_heads, self.q_head, self.key_dim)
            keys[:, :s.head_dim, :s.latent_dim] = k_up
            if self.rope_dim:
                keys[:, s.head_dim:, s.latent_dim:] = torch.eye(self.rope_dim, dtype=k_up.dtype, device=k_up.device)
            values = k_up.new_zeros(s.num_heads * s.v_head_dim, self.key_dim)
            values[:, :s.latent_dim] = self.rt.upload(tensors[s.v_up_weight])
            self.w_kv_whole = torch.cat([keys.view(s.num_heads * self.q_head, self.key_dim), values], dim=0).contiguous()
        w_o = self.rt.upload(tensors[s.o_weight])
        if self.ctx_width != self.ctx_dim:
            w_o = torch.cat([w_o, w_o.new_zeros(s.hidden_size, self.ctx_width - self.ctx_dim)], dim=1)
        self.w_o = w_o.contiguous()

    def forward(self, step, h, x, cache_entry, writes_cache=True):
        s, rt = self.spec, self.rt
        ops = rt.kernels()
        n = h.shape[0]
        fused = rt.workspace.get("qkv", (n, self.fused_width), torch.float32)
        ops.linear(h, self.w_q_down, fused, _ops.MODE_STORE_F32)
        latents = step.cache.entry_storage(cache_entry)["c"]
        group = step.cache.entry_group_index(cache_entry)
        table = step.block_tables[group]
        block_size = step.cache.block_size
        if self.extended:
            self._forward_extended(step, fused, latents, table, writes_cache, group)
            ctx = rt.workspace.get("attn_ctx", (n, self.ctx_width), rt.dtype)
            ops.linear(ctx, self.w_o, x, _residual_mode(step), stats=_residual_stats(step))
            return
        q = rt.workspace.get("q", (n, self.q_dim), rt.dtype)
        # queries pass as they are; the one "key head" of a row is the latent, normed with its weight and cached
        ops.qkv_finish(fused, q, latents, None, step.positions, step.token_seq, table, s.num_heads, 1, s.head_dim, 0,
                       block_size, write_kv=writes_cache, k_norm=True, qk_norm_eps=s.eps,
                       k_norm_weight=self.latent_gamma, key_dim=s.latent_dim)
        ctx = rt.workspace.get("attn_ctx", (n, self.ctx_width), rt.dtype)
        if not self._attend_expanded(step, q, ctx, latents, table, group):
            self._attend_folded(step, q, ctx, latents, table)
        ops.linear(ctx, self.w_o, x, _residual_mode(step), stats=_residual_stats(step))

    def _forward_extended(self, step, fused, cached, table, writes_cache, group):
        """The folded way with a rotated part, a sink and a gate: finish the projection's rows (the latent's norm, the
        rotations, the cache write), fold the keys' up-projection into the unrotated queries, attend with all heads
        over the cached rows, apply the values' up-projection."""
        s, rt = self.spec, self.rt
        ops = rt.kernels()
        n = fused.shape[0]
        rotation = self.position.fusion_table(step.max_ctx) if self.position is not None else None
        gate = fused[:, self.gate_offset:] if self.has_gate else None
        if self.w_kv_whole is not None and self._expanded_serves(step, self.q_head):
            # a prompt in bfloat16: whole query heads [unrotated | rotated] against every head's keys made from the
            # cached rows; the sink and the gate are the tensor-core kernel's
            q_whole = rt.workspace.get("q", (n, self.q_dim), rt.dtype)
            ops.latent_finish(fused, None, None, cached, step.positions, step.token_seq, table, s.num_heads,
                              s.head_dim, self.rope_dim, s.latent_dim, step.cache.block_size,
                              rotation=rotation, rotated=s.rope.dims if rotation is not None else 0,
                              latent_offset=self.q_dim, latent_gamma=self.latent_gamma, eps=s.eps,
                              write_cache=writes_cache and not self.shares_kv, q_whole=q_whole)
            ctx = rt.workspace.get("attn_ctx", (n, self.ctx_width), rt.dtype)
            self._attend_expanded(step, q_whole, ctx, cached, table, group, head_dim=self.q_head, row_width=self.key_dim,
                                  weight=self.w_kv_whole, gate=gate, gate_stride=self.fused_width, sink=self.sink)
            return
        q_plain = rt.workspace.get("q", (n, s.num_heads * s.head_dim), rt.dtype)
        q_folded = rt.workspace.get("q_latent", (n, s.num_heads * self.key_dim), rt.dtype)
        ops.latent_finish(fused, q_plain, q_folded, cached, step.positions, step.token_seq, table, s.num_heads,
                          s.head_dim, self.rope_dim, s.latent_dim, step.cache.block_size,
                          rotation=rotation, rotated=s.rope.dims if rotation is not None else 0,
                          latent_offset=self.q_dim, latent_gamma=self.latent_gamma, eps=s.eps,
                          write_cache=writes_cache and not self.shares_kv)
        ops.headwise_linear(q_plain, self.w_k_up_t, q_folded, s.num_heads, out_head_stride=self.key_dim)
        mixed = rt.workspace.get("latent_ctx", (n, s.num_heads * s.latent_dim), rt.dtype)
        # one token a sequence: few (token, head) pairs over long contexts, so each pair's keys are cut into parts that
        # run side by side, enough to give every SM thirty-odd warps (a part is at least 64 keys)
        splits, scratch_o, scratch_ml = 1, None, None
        if step.is_decode and rt.device.type == "cuda":
            splits = max(1, min(-(-rt.sm_count * 32 // (n * s.num_heads)), -(-step.max_ctx // 64), 64))
            if splits > 1:
                scratch_o = rt.workspace.get("attn_split_o", (n * s.num_heads * splits * s.latent_dim,), torch.float32)
                scratch_ml = rt.workspace.get("attn_split_ml", (n * s.num_heads * splits * 2,), torch.float32)
        ops.attention_general(q_folded, cached, cached, table, step.positions, step.token_seq, mixed, s.num_heads, 1,
                              self.key_dim, s.latent_dim, step.cache.block_size, s.scale,
                              gate=gate, gate_stride=self.fused_width,
                              sink=self.sink, value_stride=self.key_dim, splits=splits, scratch_o=scratch_o,
                              scratch_ml=scratch_ml)
        ctx = rt.workspace.get("attn_ctx", (n, self.ctx_width), rt.dtype)
        ops.headwise_linear(mixed, self.w_v_up, ctx, s.num_heads, zero_pad=self.ctx_width != self.ctx_dim)

    def _attend_folded(self, step, q, ctx, latents, table):
        """The up-projections folded into queries and outputs; attention of all heads over the cached vectors."""
        s, rt = self.spec, self.rt
        ops = rt.kernels()
        n = q.shape[0]
        block_size = step.cache.block_size
        q_latent = rt.workspace.get("q_latent", (n, s.num_heads * s.latent_dim), rt.dtype)
        ops.headwise_linear(q, self.w_k_up_t, q_latent, s.num_heads)
        mixed = rt.workspace.get("latent_ctx", (n, s.num_heads * s.latent_dim), rt.dtype)
        if not (step.is_decode and self._decode_on_tensor_cores(step, q_latent, mixed, latents, table)):
            ops.attention_general(q_latent, latents, latents, table, step.positions, step.token_seq, mixed, s.num_heads, 1,
                                  s.latent_dim, s.latent_dim, block_size, s.scale)
        ops.headwise_linear(mixed, self.w_v_up, ctx, s.num_heads, zero_pad=self.ctx_width != self.ctx_dim)

    def _decode_on_tensor_cores(self, step, q_latent, mixed, latents, table) -> bool:
        """One token a sequence in bfloat16: the split decode kernel of the library built for a head as wide as the
        latent, with all query heads on the one key head.  False where no such library can be built."""
        s, rt = self.spec, self.rt
        if (rt.dtype != torch.bfloat16 or rt.device.type != "cuda" or s.latent_dim % 16 != 0 or s.latent_dim > 256
                or step.cache.block_size % 16 != 0):
            return False
        from .attention import decode_splits
        ops = rt.kernels(s.latent_dim)
        n = q_latent.shape[0]
        splits = decode_splits(n, -(-s.num_heads // 16), step.max_ctx, rt.sm_count)
        scratch_o = scratch_ml = None
        if splits > 1:
            scratch_o = rt.workspace.get("attn_split_o", (n * s.num_heads * splits * s.latent_dim,), torch.float32)
            scratch_ml = rt.workspace.get("attn_split_ml", (n * s.num_heads * splits * 2,), torch.float32)
        ops.attention_decode(q_latent, latents, latents, table, step.ctx_after, mixed, s.num_heads, 1, s.latent_dim,
                             step.cache.block_size, s.scale, 0, splits, scratch_o, scratch_ml)
        return True

    def _expanded_serves(self, step, head_dim) -> bool:
        """True if this step can make every head's keys and values and attend on the tensor-core prompt kernel."""
        s, rt = self.spec, self.rt
        block_size = step.cache.block_size
        if (step.is_decode or rt.dtype != torch.bfloat16 or rt.device.type != "cuda" or head_dim != s.v_head_dim
                or head_dim not in (64, 128) or step.max_q_len <= 32 or block_size & (block_size - 1) or block_size < 16
                or step.n_seqs * -(-step.max_q_len // 128) > 65535 or self.ctx_width != self.ctx_dim
                or s.latent_dim % 8 != 0):          # (the up-projection GEMM reads rows of whole 16 bytes)
            return False
        return rt.kernels(head_dim).has_attention_prefill_tc()

    def _attend_expanded(self, step, q, ctx, latents, table, group, head_dim=None, row_width=None, weight=None,
                         gate=None, gate_stride=0, sink=None) -> bool:
        """A prompt in bfloat16: every head's keys and values are made from the gathered cached vectors by one GEMM,
        written as pages of a scratch cache, and the tensor-core prompt kernel attends over them as multi-head
        attention.  False where that kernel does not serve (then the folded way does).  ``head_dim``, ``row_width``
        and ``weight``: the keys' size, the cached row's width and the matrix that makes ``[keys | values]`` of all
        heads from a row (default: the plain latent's)."""
        s, rt = self.spec, self.rt
        block_size = step.cache.block_size
        head_dim = head_dim or s.head_dim
        row_width = row_width or s.latent_dim
        weight = weight if weight is not None else self.w_kv_up
        if not self._expanded_serves(step, head_dim):
            return False
        ops_d = rt.kernels(head_dim)
        ops = rt.kernels()
        meta = step.scratch.get("expanded_context")
        if meta is None:
            # every cached position of the step's sequences (this step's included), and a table of scratch pages
            lengths = [before + new for before, new in zip(step.ctx_before, step.q_lens)]
            pages = [-(-length // block_size) for length in lengths]
            width = max(pages)
            scratch_table = np.zeros((step.n_seqs, width), dtype=np.int32)
            base = 0
            for row, count in enumerate(pages):
                scratch_table[row, :count] = np.arange(base, base + count)
                base += count
            host = np.concatenate([np.concatenate([np.arange(length) for length in lengths]),
                                   np.repeat(np.arange(step.n_seqs), lengths), scratch_table.reshape(-1)]).astype(np.int32)
            device = torch.from_numpy(host).to(rt.device)
            total = int(sum(lengths))
            meta = (total, base, device[:total], device[total:2 * total], device[2 * total:].view(step.n_seqs, width))
            step.scratch["expanded_context"] = meta
        total, pages, positions, seqs, scratch_table = meta
        gathered = rt.workspace.get("latent_rows", (total, row_width), rt.dtype)
        ops.paged_gather(latents, table, positions, seqs, gathered)
        kv_width = s.num_heads * (head_dim + s.v_head_dim)
        expanded = rt.workspace.get("latent_kv", (total, kv_width), torch.float32)
        ops.linear(gathered, weight, expanded, _ops.MODE_STORE_F32)
        keys = rt.workspace.get("latent_keys", (pages, s.num_heads, block_size, head_dim), rt.dtype)
        values = rt.workspace.get("latent_values", (pages, s.num_heads, block_size, s.v_head_dim), rt.dtype)
        # (rows of a sequence's last page beyond its length are never seen, but a weight of zero times whatever the
        # scratch held, a NaN perhaps, is not zero)
        values.zero_()
        ops.qkv_finish(expanded, None, keys, values, positions, seqs, scratch_table, 0, s.num_heads, head_dim,
                       s.v_head_dim, block_size)
        ops_d.attention_prefill_tc(q, keys, values, scratch_table, step.cu_q, step.ctx_after, ctx, step.max_q_len,
                                   s.num_heads, s.num_heads, head_dim, block_size, s.scale, gate=gate,
                                   gate_stride=gate_stride, sink=sink)
        return True


register_mixer("latent_attention", LatentAttention)
