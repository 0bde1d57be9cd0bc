"""Time mixing with a matrix state per head and a decay per token and key channel (the mixer of the RWKV family).

For the mixer's input h, h' the input of the token before (zeros for a sequence's first), H heads of d numbers::

    mix_s = h + (h' - h) mu_s                                for s in r, k, v, g, w
    r, k, v = Wr mix_r, Wk mix_k, Wv mix_v;   gate = silu(Wg mix_g);   w = exp(-exp(W2 tanh(W1 mix_w) + w0))
    o_t = (S_(t-1) + diag(u) k_t v_t^T)^T r_t;   S_t = diag(w_t) S_(t-1) + k_t v_t^T        per head, S = 0 at the start
    x += Wo (o / rms(o) per head * norm * gate) * out_scale

Kernels: ``token_shift_mix`` (the five mixes, compute dtype), five projections (float32 out), ``time_mix_decay``,
``time_mix_scan``, ``time_mix_finish`` (all float32 up to the rounding of the output projection's input), the output
projection.  Nothing is kept per position: per sequence the cache's state area holds S and the last input, each twice
(``csrc/time_mix.cu`` says why).  ``state_offset`` (floats): where this mixer's state starts in its cache entry's rows;
``out_scale``: a factor on the mixer's result, for a mixer that is one side of a weighted pair.
"""
from __future__ import annotations

import torch

from .. import ops as _ops
from .attention import _residual_mode, _residual_stats
from .base import CacheRequest, Mixer, TensorRequest
from .registry import register_mixer


class TimeMix(Mixer):
    graph_safe = True
    stores_branch = True
    honours_state_offset = True
    scales_output = True

    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        if len(spec.mix) != 5:
            raise ValueError("time_mix: one mix tensor for each of r, k, v, g, w is needed")
        if spec.head_dim > 512:
            raise ValueError(f"time_mix: heads of {spec.head_dim} numbers are not supported (at most 512)")
        if runtime.dtype == torch.bfloat16 and spec.hidden_size % 8 != 0:
            raise ValueError(f"time_mix: hidden size {spec.hidden_size} is not supported in bfloat16 "
                             "(rows of 16 bytes are needed: a multiple of 8); float32 takes any size")
        self.inner = spec.num_heads * spec.head_dim
        self.rank_padded = -(-spec.decay_rank // 8) * 8
        self.out_width = -(-self.inner // 8) * 8          # whole 16 bytes for the output projection
        self.state_offset = 0
        self.out_scale = 1.0

    @classmethod
    def expected_tensors(cls, spec):
        inner = spec.num_heads * spec.head_dim
        wanted = {name: TensorRequest((spec.hidden_size,), "unit_interval") for name in spec.mix}
        for name in (spec.r_weight, spec.k_weight, spec.v_weight, spec.g_weight):
            wanted[name] = TensorRequest((inner, spec.hidden_size))
        wanted[spec.w1_weight] = TensorRequest((spec.decay_rank, spec.hidden_size))
        wanted[spec.w2_weight] = TensorRequest((inner, spec.decay_rank))
        wanted[spec.w0] = TensorRequest((inner,), "decay_logit")
        wanted[spec.bonus] = TensorRequest((spec.num_heads, spec.head_dim), "half_normal")
        wanted[spec.norm] = TensorRequest((inner,), "around_one")
        wanted[spec.o_weight] = TensorRequest((spec.hidden_size, inner))
        return wanted

    @classmethod
    def state_floats(cls, spec) -> int:
        return 2 * spec.num_heads * spec.head_dim * spec.head_dim + 2 * spec.hidden_size

    @classmethod
    def cache_request(cls, spec):
        return CacheRequest(kind="none", state_bytes=4 * cls.state_floats(spec))

    def bind(self, tensors):
        s, rt = self.spec, self.rt
        as_float = lambda name: rt.upload(tensors[name], torch.float32).reshape(-1).contiguous()
        self.mu = torch.stack([as_float(name) for name in s.mix]).contiguous()             # [5, hidden]
        self.w_r, self.w_k, self.w_v, self.w_g = (rt.upload(tensors[name]).contiguous()
                                                  for name in (s.r_weight, s.k_weight, s.v_weight, s.g_weight))
        w1 = rt.upload(tensors[s.w1_weight])
        if self.rank_padded != s.decay_rank:          # (zero rows: the decay kernel reads the first decay_rank columns)
            w1 = torch.cat([w1, w1.new_zeros(self.rank_padded - s.decay_rank, s.hidden_size)], dim=0)
        self.w_1 = w1.contiguous()
        self.w_2 = rt.upload(tensors[s.w2_weight]).t().contiguous()      # [rank, inner]: the decay kernel reads it by rows
        self.w0, self.bonus, self.norm = as_float(s.w0), as_float(s.bonus), as_float(s.norm)
        w_o = rt.upload(tensors[s.o_weight])
        if self.out_width != self.inner:
            w_o = torch.cat([w_o, w_o.new_zeros(s.hidden_size, self.out_width - self.inner)], dim=1)
        self.w_o = w_o.contiguous()

    def forward(self, step, h, x, cache_entry, writes_cache=True):
        s, rt = self.spec, self.rt
        ops = rt.kernels()
        get = rt.workspace.get
        n = h.shape[0]
        state = step.cache.state(cache_entry).view(torch.float32)
        meta = (step.positions, step.token_seq, step.cu_q, step.slot_ids)
        mixes = get("time_mix_in", (5, n, s.hidden_size), rt.dtype)
        ops.token_shift_mix(h, self.mu, mixes, s.num_heads, s.head_dim, meta, state, self.state_offset)
        rows = get("time_mix_rows", (6, n, self.inner), torch.float32)       # r, k, v, gate, decay, o
        for index, weight in enumerate((self.w_r, self.w_k, self.w_v, self.w_g)):
            ops.linear(mixes[index], weight, rows[index], _ops.MODE_STORE_F32)
        lora = get("time_mix_lora", (n, self.rank_padded), torch.float32)
        ops.linear(mixes[4], self.w_1, lora, _ops.MODE_STORE_F32)
        ops.time_mix_decay(lora, s.decay_rank, self.w_2, self.w0, rows[4])
        ops.time_mix_scan(rows[0], rows[1], rows[2], rows[4], self.bonus, rows[5], h, step.n_seqs, s.num_heads,
                          s.head_dim, meta, state, self.state_offset)
        mixed = get("time_mix_out", (n, self.out_width), rt.dtype)
        ops.time_mix_finish(rows[5], rows[3], self.norm, s.eps, self.out_scale, mixed, s.num_heads, s.head_dim)
        ops.linear(mixed, self.w_o, x, _residual_mode(step), stats=_residual_stats(step))


register_mixer("time_mix", TimeMix)
