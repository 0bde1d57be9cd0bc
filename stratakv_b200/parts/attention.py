"""Causal grouped-query attention over the paged cache.

``q, k, v = h.Wq^T, h.Wk^T, h.Wv^T`` (no bias); rotary encoding on every query
and key head before the key is cached; scores ``(q.k) * scale`` over the
sequence's own earlier positions and the token itself; softmax and the weighted
sum of values in float; ``x += ctx.Wo^T`` (``src/layers/attention.cpp:153-342``,
``src/models/transformer_block.cpp:301-309``).  The three projections are one
matrix ``[q | k | v]`` here, and the residual sum is the epilogue of the output
projection.

A spec may switch on further mechanisms (``parts/spec.py::AttentionSpec``): biases on the projections, values
of another width than keys, an RMS norm on every value head before it is cached, a bias on the scores by the
logarithm of the distance, and a gate per head on the output.  Such a mixer projects ``[q | k | v | gate]`` at
once, finishes the rows in ``qkv_finish`` (biases, value norm, cache write) and attends with the kernels
that carry the bias and the gate (``csrc/attention_general.cu``).  Further switches of that path: a unit norm on
every query and key head, a temperature on the queries that grows with the position, a cap on the scores
(``c * tanh(score / c)``), a gate for every output number instead of one per head, and a mixer without key and value
projections that attends over the cache entry another layer's run wrote.
"""
from __future__ import annotations

import math

import torch

from .. import ops as _ops
from .base import CacheRequest, Mixer, TensorRequest
from .registry import part_class, register_mixer


def decode_splits(n_seqs: int, blocks_per_seq: int, max_ctx: int, sms: int) -> int:
    """Into how many pieces a decode step cuts each context: enough blocks to fill the
    GPU twice over, at least 128 keys (one group of 16 per warp) a piece.  It depends on
    the step's sizes only, never on which sequences are live."""
    by_length = max(1, max_ctx // 128)
    by_count = -(-2 * sms // max(1, n_seqs * blocks_per_seq))
    return max(1, min(by_length, by_count, 64))


def fused_decode_splits(n_seqs: int, blocks_per_seq: int, max_ctx: int, sms: int, per_sm: int = 2) -> int:
    """The same for the fused kernel, whose pieces are the blocks of one cluster: the largest
    power of two (other cluster sizes measured slower), at most 8, that keeps the grid within
    ``per_sm`` blocks per SM (2 up to head size 64, 1 above: the staged keys of a block take
    shared memory in proportion).  Half as many if that gives every block an SM to itself and
    a piece of at most 512 keys, which such a block fetches whole before its inputs are ready."""
    pairs = max(1, n_seqs * blocks_per_seq)
    by_length = max(1, max_ctx // 128)
    wanted = max(1, min(by_length, per_sm * sms // pairs, 8))
    wanted = 1 << (wanted.bit_length() - 1)
    if wanted > 1 and pairs * wanted > sms >= pairs * wanted // 2 and max_ctx * 2 <= 512 * wanted:
        wanted //= 2
    return wanted


def wants_more_pieces(n_seqs: int, blocks_per_seq: int, max_ctx: int, cluster_splits: int, sms: int) -> bool:
    """A cluster holds at most 8 pieces of a context.  Few long sequences want more: when the fused kernel's
    grid leaves SMs idle, its pieces are 2,048 keys or longer and the path through scratch memory would cut
    at least twice as many (batch 1 at 32,000 keys: 1.14 ms a step with 64 pieces and a combine kernel,
    1.72 ms with 8 pieces in one cluster)."""
    return (n_seqs * blocks_per_seq * cluster_splits < sms and max_ctx >= 2048 * cluster_splits
            and decode_splits(n_seqs, blocks_per_seq, max_ctx, sms) >= 2 * cluster_splits)


def _residual_mode(step):
    """The epilogue of a mixer's last projection: add to the stream, or store into a branch buffer."""
    return _ops.MODE_STORE_F32 if getattr(step, "store_branch", False) else _ops.MODE_ADD_F32


def _residual_stats(step):
    return None if getattr(step, "store_branch", False) else step.residual_stats


class PagedAttention(Mixer):
    graph_safe = True
    folds_norm = True
    stores_branch = True

    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        if spec.num_heads % spec.num_kv_heads != 0:
            raise ValueError("attention: heads must be a multiple of kv heads")
        self.q_dim = spec.num_heads * spec.head_dim
        self.kv_dim = 0 if spec.shares_kv else spec.num_kv_heads * spec.head_dim
        self.v_dim = 0 if spec.shares_kv else spec.num_kv_heads * spec.value_dim
        self.ctx_dim = spec.num_heads * spec.value_dim
        if spec.gate_per_element and not spec.gate_weight:
            raise ValueError("attention: a gate per output number needs a gate weight")
        if spec.extended:
            if spec.position is not None:
                raise ValueError("attention: the extended mechanisms are built without a rotation")
            if spec.value_dim > 256:
                raise ValueError(f"attention: value heads of {spec.value_dim} numbers are not supported (at most 256)")
            if runtime.dtype == torch.bfloat16 and spec.hidden_size % 8 != 0:
                raise ValueError(f"attention: hidden size {spec.hidden_size} is not supported in bfloat16 "
                                 "(rows of 16 bytes are needed: a multiple of 8); float32 takes any size")
            # the attention output's rows, padded so that the output projection reads whole 16 bytes
            self.ctx_width = -(-self.ctx_dim // 8) * 8
            gate_rows = (self.ctx_dim if spec.gate_per_element else spec.num_heads) if spec.gate_weight else 0
            self.gate_rows = gate_rows
            self.gate_offset = self.q_dim + self.kv_dim + self.v_dim
            self.fused_width = -(-(self.gate_offset + gate_rows) // 8) * 8
            self.position = None
            return
        if spec.head_dim % 16 != 0:
            raise ValueError(f"attention: head size {spec.head_dim} is not supported "
                             "(the kernels take multiples of 16)")
        if runtime.dtype == torch.bfloat16 and spec.hidden_size % 8 != 0:
            raise ValueError(f"attention: hidden size {spec.hidden_size} is not supported in bfloat16 "
                             "(rows of 16 bytes are needed: a multiple of 8); float32 takes any size")
        position_spec = spec.position
        kind = position_spec.kind if position_spec is not None else "none"
        self.position = part_class("position", kind)(position_spec, runtime)

    @classmethod
    def expected_tensors(cls, spec):
        q_dim, kv_dim = spec.num_heads * spec.head_dim, spec.num_kv_heads * spec.head_dim
        v_dim, ctx_dim = spec.num_kv_heads * spec.value_dim, spec.num_heads * spec.value_dim
        wanted = {spec.q_weight: TensorRequest((q_dim, spec.hidden_size)),
                  spec.o_weight: TensorRequest((spec.hidden_size, ctx_dim))}
        if not spec.shares_kv:
            wanted[spec.k_weight] = TensorRequest((kv_dim, spec.hidden_size))
            wanted[spec.v_weight] = TensorRequest((v_dim, spec.hidden_size))
        for name, width in ((spec.q_bias, q_dim), (spec.k_bias, kv_dim), (spec.v_bias, v_dim)):
            if name:
                wanted[name] = TensorRequest((width,))
        if spec.distance_bias:
            wanted[spec.distance_bias.r1] = TensorRequest((spec.num_heads,), "positive")
            wanted[spec.distance_bias.r2] = TensorRequest((spec.num_heads,), "positive")
        if spec.gate_weight:
            wanted[spec.gate_weight] = TensorRequest((ctx_dim if spec.gate_per_element else spec.num_heads,
                                                      spec.hidden_size))
        if getattr(spec, "q_norm_weight", None):
            wanted[spec.q_norm_weight] = TensorRequest((q_dim,), "around_one")
        if getattr(spec, "k_norm_weight", None) and not spec.shares_kv:
            wanted[spec.k_norm_weight] = TensorRequest((kv_dim,), "around_one")
        return wanted

    @classmethod
    def cache_request(cls, spec):
        kind = "kv_window" if spec.window > 0 else "kv"
        v_head_dim = spec.v_head_dim if spec.v_head_dim != spec.head_dim else 0
        return CacheRequest(kind, spec.num_kv_heads, spec.head_dim, spec.window, v_head_dim=v_head_dim)

    def bind(self, tensors):
        s = self.spec
        names = ([s.q_weight] + ([] if s.shares_kv else [s.k_weight, s.v_weight])
                 + ([s.gate_weight] if s.extended and s.gate_weight else []))
        parts = [self.rt.upload(tensors[name]) for name in names]
        if s.extended:
            rows = sum(part.shape[0] for part in parts)
            if rows < self.fused_width:            # (zero rows: what they produce is never read)
                parts.append(parts[0].new_zeros(self.fused_width - rows, s.hidden_size))
        self.w_qkv = torch.cat(parts, dim=0).contiguous()
        del parts
        self.w_o = self.rt.upload(tensors[s.o_weight])
        if not s.extended:
            return
        if self.ctx_width != self.ctx_dim:
            self.w_o = torch.cat([self.w_o, self.w_o.new_zeros(s.hidden_size, self.ctx_width - self.ctx_dim)], dim=1).contiguous()
        as_float = lambda name: self.rt.upload(tensors[name], torch.float32) if name else None
        self.q_bias, self.k_bias, self.v_bias = as_float(s.q_bias), as_float(s.k_bias), as_float(s.v_bias)
        # a norm over a whole projection (all heads together) runs right after the projection and adds that
        # projection's bias itself; the kernels behind it then see rows that need neither
        self.norm_segments = []
        if getattr(s, "q_norm_weight", None):
            self.norm_segments.append((0, self.q_dim, self.q_bias, as_float(s.q_norm_weight)))
            self.q_bias = None
        if getattr(s, "k_norm_weight", None) and not s.shares_kv:
            self.norm_segments.append((self.q_dim, self.kv_dim, self.k_bias, as_float(s.k_norm_weight)))
            self.k_bias = None
        self.r1 = as_float(s.distance_bias.r1) if s.distance_bias else None
        self.r2 = as_float(s.distance_bias.r2) if s.distance_bias else None
        self.bias_table = None
        if s.distance_bias and self._specialised():
            # what the bias takes off a score, by head and distance, for the kernels that look it up (they keep
            # scores in units of log2, so the table is in those units): as far as the window reaches, or as far as
            # the model's positions do
            reach = min(s.window or s.distance_bias.max_distance, s.distance_bias.max_distance or s.window)
            if reach > 0:
                r1 = tensors[s.distance_bias.r1].to(torch.float64)[:, None]
                r2 = tensors[s.distance_bias.r2].to(torch.float64)[:, None]
                r1, r2 = r1.cpu(), r2.cpu()         # (random weights may have been drawn on the device)
                table = r1 * torch.log1p(r2 * torch.arange(reach, dtype=torch.float64)[None, :]) * math.log2(math.e)
                self.bias_table = self.rt.upload(table.to(torch.float32).contiguous(), torch.float32)

    def _specialised(self) -> bool:
        """True if the kernels that are compiled for one head size can serve this mixer: bfloat16, keys and values
        of one width that a library can be built for, and a distance bias (if any) that fits a table."""
        s = self.spec
        return (self.rt.dtype == torch.bfloat16 and s.value_dim == s.head_dim and s.head_dim % 16 == 0
                and s.head_dim <= 256 and self.rt.device.type == "cuda"
                and (not s.distance_bias or s.window > 0 or s.distance_bias.max_distance > 0))

    def _forward_extended(self, step, h, x, cache_entry, writes_cache=True):
        """The mixer with any of the further mechanisms: one projection for queries, keys, values and the gates'
        logits (float32), ``qkv_finish``, attention with the bias and the gate, output projection."""
        s, rt = self.spec, self.rt
        ops = rt.kernels()
        n = h.shape[0]
        fused = rt.workspace.get("qkv", (n, self.fused_width), torch.float32)
        ops.linear(h, self.w_qkv, fused, _ops.MODE_STORE_F32)
        if self.norm_segments:
            ops.projection_norm(fused, s.projection_norm_eps, self.norm_segments)
        k_cache, v_cache = step.cache.entry_kv(cache_entry)
        table = step.block_tables[step.cache.entry_group_index(cache_entry)]
        if step.is_decode and self._specialised():
            ctx = rt.workspace.get("attn_ctx", (n, self.ctx_width), rt.dtype)
            if self._decode_fused(step, fused, ctx, k_cache, v_cache, table, writes_cache):
                ops.linear(ctx, self.w_o, x, _residual_mode(step), stats=_residual_stats(step))
                return
        q = rt.workspace.get("q", (n, self.q_dim), rt.dtype)
        temperature = (s.q_temperature.coef, s.q_temperature.every) if s.q_temperature else None
        ops.qkv_finish(fused, q, k_cache, v_cache, step.positions, step.token_seq, table, s.num_heads,
                       s.num_kv_heads, s.head_dim, s.value_dim, step.cache.block_size, self.q_bias, self.k_bias,
                       self.v_bias, s.value_norm_eps, writes_cache and not s.shares_kv,
                       q_norm=s.qk_norm_eps is not None, k_norm=s.qk_norm_eps is not None,
                       qk_norm_eps=s.qk_norm_eps or 0.0, q_temperature=temperature)
        ctx = rt.workspace.get("attn_ctx", (n, self.ctx_width), rt.dtype)
        gate = fused[:, self.gate_offset:] if s.gate_weight else None
        if self._specialised() and self._attend_specialised(step, q, ctx, k_cache, v_cache, table, gate):
            ops.linear(ctx, self.w_o, x, _residual_mode(step), stats=_residual_stats(step))
            return
        ops.attention_general(q, k_cache, v_cache, table, step.positions, step.token_seq, ctx, s.num_heads,
                              s.num_kv_heads, s.head_dim, s.value_dim, step.cache.block_size, s.scale, s.window,
                              self.r1, self.r2, gate, self.fused_width, softcap=s.softcap,
                              gate_per_element=s.gate_per_element)
        ops.linear(ctx, self.w_o, x, _residual_mode(step), stats=_residual_stats(step))

    def _decode_fused(self, step, fused, ctx, k_cache, v_cache, table, writes_cache) -> bool:
        """One token a sequence, in one kernel straight from the fused projection: biases, value norm, cache write,
        attention with the bias table over up to 8 pieces of the context, their merge, the gate.  False where
        that kernel does not serve (then ``qkv_finish`` and the split kernel do)."""
        s, rt = self.spec, self.rt
        ops = rt.kernels(s.head_dim)
        block_size = step.cache.block_size
        if not ops.has_attention_decode_fused() or s.head_dim > 128 or block_size % 16 != 0:
            return False
        if s.qk_norm_eps is not None and s.head_dim & (s.head_dim - 1):
            return False                            # (the kernel's unit norm wants a head size that is a power of two)
        n = fused.shape[0]
        blocks_per_seq = s.num_kv_heads * (-(-(s.num_heads // s.num_kv_heads) // 16))
        keys = min(step.max_ctx, s.window) if s.window > 0 else step.max_ctx
        splits = fused_decode_splits(n, blocks_per_seq, keys, rt.sm_count, per_sm=2 if s.head_dim <= 64 else 1)
        if wants_more_pieces(n, blocks_per_seq, keys, splits, rt.sm_count):
            return False
        ops.attention_decode_fused(fused, None, k_cache, v_cache, table, step.ctx_after, ctx, s.num_heads, s.num_kv_heads,
                                   s.head_dim, block_size, s.scale, s.window, splits, writes_cache and not s.shares_kv,
                                   q_bias=self.q_bias, k_bias=self.k_bias, v_bias=self.v_bias,
                                   value_norm_eps=s.value_norm_eps, bias=self.bias_table,
                                   gate=fused[:, self.gate_offset:] if s.gate_weight else None, gate_stride=self.fused_width,
                                   qk_norm_eps=s.qk_norm_eps,
                                   q_temperature=(s.q_temperature.coef, s.q_temperature.every) if s.q_temperature else None,
                                   softcap=s.softcap, gate_per_element=s.gate_per_element)
        return True

    def _attend_specialised(self, step, q, ctx, k_cache, v_cache, table, gate) -> bool:
        """Attention through the kernels of the head size's own library, which take the distance bias as a table and
        the gate's logits: split decode, or prefill on the tensor cores.  False if none of them serves this step."""
        s, rt = self.spec, self.rt
        ops = rt.kernels(s.head_dim)
        n = q.shape[0]
        extras = dict(bias=self.bias_table, gate=gate, gate_stride=self.fused_width, softcap=s.softcap,
                      gate_per_element=s.gate_per_element)
        block_size = step.cache.block_size
        if step.is_decode:
            if block_size % 16 != 0:
                return False
            blocks_per_seq = s.num_kv_heads * (-(-(s.num_heads // s.num_kv_heads) // 16))
            keys = min(step.max_ctx, s.window) if s.window > 0 else step.max_ctx
            splits = decode_splits(n, blocks_per_seq, keys, rt.sm_count)
            scratch_o = scratch_ml = None
            if splits > 1:
                scratch_o = rt.workspace.get("attn_split_o", (n * s.num_heads * splits * s.head_dim,), torch.float32)
                scratch_ml = rt.workspace.get("attn_split_ml", (n * s.num_heads * splits * 2,), torch.float32)
            ops.attention_decode(q, k_cache, v_cache, table, step.ctx_after, ctx, s.num_heads, s.num_kv_heads,
                                 s.head_dim, block_size, s.scale, s.window, splits, scratch_o, scratch_ml, **extras)
            return True
        if (ops.has_attention_prefill_tc() and step.max_q_len > 32 and block_size & (block_size - 1) == 0
                and block_size >= 16 and step.n_seqs * -(-step.max_q_len // 128) <= 65535):
            ops.attention_prefill_tc(q, k_cache, v_cache, table, step.cu_q, step.ctx_after, ctx, step.max_q_len,
                                     s.num_heads, s.num_kv_heads, s.head_dim, block_size, s.scale, s.window, **extras)
            return True
        if ops.has_attention_prefill() and s.num_heads <= 65535 and not s.softcap and not s.gate_per_element:
            del extras["softcap"], extras["gate_per_element"]
            ops.attention_prefill(q, k_cache, v_cache, table, step.cu_q, step.ctx_after, ctx, step.max_q_len,
                                  s.num_heads, s.num_kv_heads, s.head_dim, block_size, s.scale, s.window, **extras)
            return True
        return False

    def forward(self, step, h, x, cache_entry, writes_cache=True):
        if self.spec.extended:
            return self._forward_extended(step, h, x, cache_entry, writes_cache)
        s, rt = self.spec, self.rt
        ops = rt.kernels(s.head_dim)
        n = h.shape[0]
        ctx = rt.workspace.get("attn_ctx", (n, self.q_dim), rt.dtype)
        if (rt.dtype == torch.bfloat16 and n > 128 and s.head_dim in (64, 128) and torch.is_tensor(h)
                and hasattr(self.position, "fusion_table") and ops.has_linear_qkv_rope()):
            # many tokens: the projection's epilogue rotates queries and keys and writes the cache itself
            q = rt.workspace.get("q", (n, self.q_dim), rt.dtype)
            k_cache, v_cache = step.cache.entry_kv(cache_entry)
            table = step.block_tables[step.cache.entry_group_index(cache_entry)]
            ops.linear_qkv_rope(h, self.w_qkv, q, self.position.fusion_table(step.max_ctx), step.positions,
                                step.token_seq, table, k_cache, v_cache, s.num_heads, s.num_kv_heads, s.head_dim,
                                step.cache.block_size, writes_cache)
            self._attend_rotated(step, q, ctx, k_cache, v_cache, table)
        else:
            qkv = rt.workspace.get("qkv", (n, self.q_dim + 2 * self.kv_dim), torch.float32)
            ops.linear(h, self.w_qkv, qkv, _ops.MODE_STORE_F32)
            self.attend(step, qkv, ctx, cache_entry, writes_cache)
        ops.linear(ctx, self.w_o, x, _residual_mode(step), stats=_residual_stats(step))

    def attend(self, step, qkv, ctx, cache_entry, writes_cache=True):
        """From the float32 q|k|v rows of the step's tokens to the attention output ``ctx`` (compute dtype):
        position encoding, cache write, attention over each sequence's own keys."""
        s, rt = self.spec, self.rt
        ops = rt.kernels(s.head_dim)
        n = qkv.shape[0]
        k_cache, v_cache = step.cache.entry_kv(cache_entry)
        table = step.block_tables[step.cache.entry_group_index(cache_entry)]
        blocks_per_seq = s.num_kv_heads * (-(-(s.num_heads // s.num_kv_heads) // 16))
        fused = (step.is_decode and rt.dtype == torch.bfloat16 and hasattr(self.position, "fusion_table")
                 and ops.has_attention_decode_fused())
        if fused:
            splits = fused_decode_splits(n, blocks_per_seq, step.max_ctx, rt.sm_count, per_sm=2 if s.head_dim <= 64 else 1)
            fused = not wants_more_pieces(n, blocks_per_seq, step.max_ctx, splits, rt.sm_count)
        if fused:
            # one kernel: rotation, cache write, attention over the context in up to 8 pieces, merge
            ops.attention_decode_fused(qkv, self.position.fusion_table(step.max_ctx), k_cache, v_cache, table,
                                       step.ctx_after, ctx, s.num_heads, s.num_kv_heads, s.head_dim,
                                       step.cache.block_size, s.scale, s.window, splits, writes_cache)
            return
        q = rt.workspace.get("q", (n, self.q_dim), rt.dtype)
        self.position.rotate_and_store(step, qkv, q, k_cache, v_cache, table, s.num_heads, s.num_kv_heads,
                                       s.head_dim, step.cache.block_size, writes_cache)
        self._attend_rotated(step, q, ctx, k_cache, v_cache, table)

    def _attend_rotated(self, step, q, ctx, k_cache, v_cache, table):
        """Attention of the step's rotated queries ``q`` over the cache, which holds the step's keys and values."""
        s, rt = self.spec, self.rt
        ops = rt.kernels(s.head_dim)
        n = q.shape[0]
        blocks_per_seq = s.num_kv_heads * (-(-(s.num_heads // s.num_kv_heads) // 16))
        if step.is_decode and rt.dtype == torch.bfloat16:
            splits = decode_splits(n, blocks_per_seq, step.max_ctx, rt.sm_count)
            scratch_o = scratch_ml = None
            if splits > 1:
                scratch_o = rt.workspace.get("attn_split_o", (n * s.num_heads * splits * s.head_dim,), torch.float32)
                scratch_ml = rt.workspace.get("attn_split_ml", (n * s.num_heads * splits * 2,), torch.float32)
            ops.attention_decode(q, k_cache, v_cache, table, step.ctx_after, ctx, s.num_heads, s.num_kv_heads,
                                 s.head_dim, step.cache.block_size, s.scale, s.window, splits, scratch_o, scratch_ml)
        elif (rt.dtype == torch.bfloat16 and ops.has_attention_prefill_tc() and step.max_q_len > 32
              and step.cache.block_size & (step.cache.block_size - 1) == 0
              and step.n_seqs * -(-step.max_q_len // 128) <= 65535):
            ops.attention_prefill_tc(q, k_cache, v_cache, table, step.cu_q, step.ctx_after, ctx, step.max_q_len,
                                     s.num_heads, s.num_kv_heads, s.head_dim, step.cache.block_size, s.scale, s.window)
        elif rt.dtype == torch.bfloat16 and ops.has_attention_prefill():
            ops.attention_prefill(q, k_cache, v_cache, table, step.cu_q, step.ctx_after, ctx, step.max_q_len,
                                  s.num_heads, s.num_kv_heads, s.head_dim, step.cache.block_size, s.scale, s.window)
        else:
            ops.attention(q, k_cache, v_cache, table, step.positions, step.token_seq, ctx, s.num_heads,
                          s.num_kv_heads, s.head_dim, step.cache.block_size, s.scale, s.window)


register_mixer("attention", PagedAttention)
