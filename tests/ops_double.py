"""A stand-in for the CUDA kernel library, used only by CPU tests of the engine's
bookkeeping (batch packing, cache slots and block tables, the order of parts).

It has the call signatures of ``stratakv_b200.ops.Kernels`` and computes each
call with plain torch on whatever device the tensors are on.  The package never
imports it; the product path has no CPU backend.
"""
from __future__ import annotations

import torch

MODE_STORE, MODE_STORE_F32, MODE_ADD_F32, MODE_GATED = 0, 1, 2, 3
MODE_ACT = 5
ACTIVATIONS = {"silu": lambda z: z * torch.sigmoid(z), "relu2": lambda z: torch.relu(z) ** 2,
               "gelu_tanh": lambda z: torch.nn.functional.gelu(z, approximate="tanh")}


class DoubleKernels:
    def __init__(self, dtype, head_dim):
        self.dtype = dtype
        self.head_dim = head_dim
        self.calls = []

    def embed(self, table, ids, out, flag=None, stats=None):
        self.calls.append("embed")
        out.copy_(table[ids.long()].float())

    def rmsnorm(self, x, gamma, eps, out, rows=None):
        self.calls.append("rmsnorm")
        src = x if rows is None else x[rows.long()]
        inv = 1.0 / torch.sqrt((src * src).mean(dim=-1, keepdim=True) + eps)
        out.copy_((src * inv * gamma).to(out.dtype))

    def linear(self, a, w, out, mode=MODE_STORE, activation="silu", flag=None, stats=None, activation_param=0.0):
        self.calls.append("linear")
        result = a.float() @ w.float().T
        if mode == MODE_GATED:
            tiles = result.view(result.shape[0], -1, 2, 8)
            gate, up = tiles[:, :, 0, :], tiles[:, :, 1, :]
            if activation == "swiglu_clamp":
                gate = gate.clamp(max=activation_param)
                product = gate * torch.sigmoid(1.702 * gate) * (up.clamp(-activation_param, activation_param) + 1.0)
            else:
                product = ACTIVATIONS[activation](gate) * up
            out.copy_(product.reshape(result.shape[0], -1).to(out.dtype))
        elif mode == MODE_ADD_F32:
            out.add_(result)
        elif mode == MODE_ACT:
            out.copy_(ACTIVATIONS[activation](result).to(out.dtype))
        else:
            out.copy_(result.to(out.dtype))

    def rope_kv_write(self, qkv, cos_sin, positions, token_seq, block_table, q_out, k_cache, v_cache,
                      num_heads, num_kv_heads, head_dim, block_size, write_kv):
        self.calls.append("rope_kv_write")
        n = qkv.shape[0]
        q_dim, kv_dim, half = num_heads * head_dim, num_kv_heads * head_dim, head_dim // 2
        q = qkv[:, :q_dim].view(n, num_heads, head_dim)
        k = qkv[:, q_dim:q_dim + kv_dim].view(n, num_kv_heads, head_dim)
        v = qkv[:, q_dim + kv_dim:].view(n, num_kv_heads, head_dim)

        def rotate(x):
            if cos_sin is None:
                return x
            cs = cos_sin[positions.long()]                        # [n, half, 2]
            c, s = cs[:, None, :, 0], cs[:, None, :, 1]
            x1, x2 = x[..., :half], x[..., half:]
            return torch.cat([x1 * c - x2 * s, x1 * s + x2 * c], dim=-1)

        q_out.copy_(rotate(q).reshape(n, q_dim).to(q_out.dtype))
        if write_kv:
            k = rotate(k)
            for t in range(n):
                pos = int(positions[t])
                block = int(block_table[int(token_seq[t]), pos // block_size])
                k_cache[block, :, pos % block_size, :] = k[t].to(k_cache.dtype)
                v_cache[block, :, pos % block_size, :] = v[t].to(v_cache.dtype)

    def attention(self, q, k_cache, v_cache, block_table, positions, token_seq, out, num_heads,
                  num_kv_heads, head_dim, block_size, scale, window=0):
        self.calls.append("attention")
        n = q.shape[0]
        group = num_heads // num_kv_heads
        qh = q.view(n, num_heads, head_dim).float()
        result = torch.zeros(n, num_heads, head_dim)
        for t in range(n):
            pos, seq = int(positions[t]), int(token_seq[t])
            lo = max(0, pos - window + 1) if window > 0 else 0
            keys = torch.stack([k_cache[int(block_table[seq, j // block_size]), :, j % block_size, :]
                                for j in range(lo, pos + 1)]).float()       # [ctx, kv_heads, d]
            values = torch.stack([v_cache[int(block_table[seq, j // block_size]), :, j % block_size, :]
                                  for j in range(lo, pos + 1)]).float()
            for h in range(num_heads):
                g = h // group
                weights = torch.softmax((keys[:, g, :] @ qh[t, h]) * scale, dim=0)
                result[t, h] = weights @ values[:, g, :]
        out.copy_(result.reshape(n, num_heads * head_dim).to(out.dtype))

    def embed_sum(self, table, ids, out, positions, token_seq, cu_q, slot_ids, flag=None, pair_table=None,
                  last_ids=None, mul_prev=0, mul_cur=0, position_table=None, position_scale=1.0, stats=None):
        self.calls.append("embed_sum")
        x = table[ids.long()].float()
        if pair_table is not None:
            buckets = pair_table.shape[0] - 1
            for t in range(ids.numel()):
                seq, pos, row = int(token_seq[t]), int(positions[t]), buckets
                if pos > 0:
                    slot = int(slot_ids[seq])
                    previous = int(ids[t - 1]) if t > int(cu_q[seq]) else int(last_ids[2 * slot + ((pos - 1) & 1)])
                    row = (previous * mul_prev + int(ids[t]) * mul_cur) % buckets
                x[t] += pair_table[row].float()
            for seq in range(slot_ids.numel()):
                last = int(cu_q[seq + 1]) - 1
                last_ids[2 * int(slot_ids[seq]) + (int(positions[last]) & 1)] = ids[last]
        if position_table is not None:
            x += position_table[positions.long()].float() * position_scale
        out.copy_(x)

    def qkv_finish(self, qkv, q_out, k_cache, v_cache, positions, token_seq, block_table, num_heads, num_kv_heads,
                   dim, vdim, block_size, q_bias=None, k_bias=None, v_bias=None, value_norm_eps=None, write_kv=True,
                   q_norm=False, k_norm=False, qk_norm_eps=0.0, k_norm_weight=None, q_temperature=None, key_dim=0):
        self.calls.append("qkv_finish")
        n = qkv.shape[0]
        key_dim = key_dim or dim
        unit = lambda x, eps: x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)
        a = num_heads * dim
        q = qkv[:, :a]
        q = (q + q_bias if q_bias is not None else q).view(n, num_heads, dim)
        if q_norm:
            q = unit(q, qk_norm_eps)
        if q_temperature is not None:
            coef, every = q_temperature
            steps = torch.div(positions.long() + 1, every, rounding_mode="floor").float()
            q = q * (1.0 + coef * torch.log(steps + 1.0))[:, None, None]
        q_out.copy_(q.reshape(n, a).to(q_out.dtype))
        if not write_kv:
            return
        b = a + num_kv_heads * key_dim
        k = qkv[:, a:b]
        k = (k + k_bias if k_bias is not None else k).view(n, num_kv_heads, key_dim)
        if k_norm:
            k = unit(k, qk_norm_eps)
            if k_norm_weight is not None:
                k = k * k_norm_weight.view(num_kv_heads, key_dim)
        v = None
        if vdim > 0:
            v = qkv[:, b:b + num_kv_heads * vdim]
            v = (v + v_bias if v_bias is not None else v).view(n, num_kv_heads, vdim)
            if value_norm_eps is not None:
                v = unit(v, value_norm_eps)
        for t in range(n):
            pos = int(positions[t])
            block = int(block_table[int(token_seq[t]), pos // block_size])
            k_cache[block, :, pos % block_size, :] = k[t].to(k_cache.dtype)
            if v is not None:
                v_cache[block, :, pos % block_size, :] = v[t].to(v_cache.dtype)

    def attention_general(self, q, k_cache, v_cache, block_table, positions, token_seq, out, num_heads, num_kv_heads,
                          dim, vdim, block_size, scale, window=0, r1=None, r2=None, gate=None, gate_stride=0,
                          softcap=0.0, gate_per_element=False, sink=None, value_stride=0, splits=1, scratch_o=None, scratch_ml=None):
        self.calls.append("attention_general")
        n = q.shape[0]
        group = num_heads // num_kv_heads
        qh = q.view(n, num_heads, dim).float()
        out.zero_()
        for t in range(n):
            pos, seq = int(positions[t]), int(token_seq[t])
            lo = max(0, pos - window + 1) if window > 0 else 0
            where = [(int(block_table[seq, j // block_size]), j % block_size) for j in range(lo, pos + 1)]
            keys = torch.stack([k_cache[b, :, r, :] for b, r in where]).float()
            values = torch.stack([v_cache[b, :, r, :vdim] for b, r in where]).float()
            distance = torch.arange(pos - lo, -1, -1, dtype=torch.float32)
            for h in range(num_heads):
                score = (keys[:, h // group, :] @ qh[t, h]) * scale
                if r1 is not None:
                    score = score - r1[h] * torch.log1p(r2[h] * distance)
                if softcap > 0.0:
                    score = softcap * torch.tanh(score / softcap)
                if sink is not None:                # one more term in the denominator, with no value
                    result = torch.softmax(torch.cat([score, sink[h].view(1)]), dim=0)[:-1] @ values[:, h // group, :]
                else:
                    result = torch.softmax(score, dim=0) @ values[:, h // group, :]
                if gate is not None and gate_per_element:
                    result = result * torch.sigmoid(gate[t, h * vdim:(h + 1) * vdim])
                elif gate is not None:
                    result = result * torch.sigmoid(gate[t, h])
                out[t, h * vdim:(h + 1) * vdim] = result.to(out.dtype)

    def rmsnorm_add(self, y, gamma, eps, x, next_gamma=None, next_eps=0.0, next_out=None):
        self.calls.append("rmsnorm_add")
        x.add_(y / torch.sqrt((y * y).mean(dim=-1, keepdim=True) + eps) * gamma)
        if next_out is not None:
            next_out.copy_((x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + next_eps) * next_gamma).to(next_out.dtype))

    def token_side(self, x, ids, table, offset, dim, gate_w, proj_t, norm_w, eps, next_gamma=None, next_eps=0.0,
                   next_out=None, branch=None, post_gamma=None, post_eps=0.0):
        self.calls.append("token_side")
        if branch is not None:
            self.rmsnorm_add(branch, post_gamma, post_eps, x)
        e = table[ids.long()][:, offset:offset + dim].float()
        g = torch.nn.functional.gelu(x @ gate_w.float().T, approximate="tanh") * e
        self.rmsnorm_add(g @ proj_t.float(), norm_w, eps, x, next_gamma, next_eps, next_out)

    def headwise_linear(self, x, w, out, heads, zero_pad=False, out_head_stride=0):
        self.calls.append("headwise_linear")
        n, out_dim, in_dim = x.shape[0], w.shape[1], w.shape[2]
        parts = x[:, :heads * in_dim].float().view(n, heads, in_dim)
        if zero_pad:
            out.zero_()
        result = torch.einsum("thi,hoi->tho", parts, w.float()).to(out.dtype)
        if out_head_stride and out_head_stride != out_dim:
            for h in range(heads):
                out[:, h * out_head_stride:h * out_head_stride + out_dim] = result[:, h]
        else:
            out[:, :heads * out_dim] = result.reshape(n, heads * out_dim)

    def stream_mix(self, streams, count, source=None, branch=None, mix=None, write=None, read=None, gamma=None,
                   eps=0.0, normed_out=None, sum_out=None):
        self.calls.append("stream_mix")
        old = streams.clone() if source is None else source[None].repeat(count, 1, 1)
        if branch is not None:
            old = torch.einsum("sr,stw->rtw", mix.view(count, count), old) + write[:, None, None] * branch[None]
            streams.copy_(old)
        if normed_out is not None:
            u = torch.einsum("s,stw->tw", read, old)
            normed_out.copy_((u / torch.sqrt((u * u).mean(dim=-1, keepdim=True) + eps) * gamma).to(normed_out.dtype))
        if sum_out is not None:
            sum_out.copy_(old.sum(dim=0))

    def retention_scratch(self, n_seqs, max_q_len, heads, dim, vdim):
        return 0

    @staticmethod
    def _turn(x, cos_sin, positions, rotated):
        """x [n, ..., width]: the first ``rotated`` numbers of the last axis turned by the table's angles."""
        if cos_sin is None or rotated == 0:
            return x
        half = rotated // 2
        cs = cos_sin[positions.long()]
        shape = (x.shape[0],) + (1,) * (x.dim() - 2) + (half,)
        c, s = cs[:, :, 0].view(shape), cs[:, :, 1].view(shape)
        u, v = x[..., :half], x[..., half:rotated]
        return torch.cat([u * c - v * s, v * c + u * s, x[..., rotated:]], dim=-1)

    def retention(self, fused, cos_sin, rotated, decay, eps, out, state, step_meta, heads, dim, vdim, max_q_len, scratch=None):
        self.calls.append("retention")
        positions, token_seq, cu_q, slot_ids = step_meta
        n = fused.shape[0]
        a, b = heads * dim, heads * vdim
        q = self._turn(fused[:, :a].view(n, heads, dim), cos_sin, positions, rotated)
        k = self._turn(fused[:, a:2 * a].view(n, heads, dim), cos_sin, positions, rotated) * dim ** -0.5
        v = fused[:, 2 * a:2 * a + b].view(n, heads, vdim)
        gate = fused[:, 2 * a + b:2 * a + 2 * b]
        size = heads * dim * vdim
        out.zero_()
        for s in range(slot_ids.numel()):
            first, last = int(cu_q[s]), int(cu_q[s + 1]) - 1
            row = state[int(slot_ids[s])]
            p_first = int(positions[first])
            S = (row[((p_first - 1) & 1) * size:][:size].clone().view(heads, dim, vdim) if p_first > 0
                 else torch.zeros(heads, dim, vdim))
            for t in range(first, last + 1):
                S = decay[:, None, None] * S + k[t][:, :, None] * v[t][:, None, :]
                o = torch.einsum("hde,hd->he", S, q[t])
                o = o / torch.sqrt((o * o).mean(dim=-1, keepdim=True) + eps)
                out[t, :b] = (o.reshape(b) * gate[t] * torch.sigmoid(gate[t])).to(out.dtype)
            row[((p_first + last - first) & 1) * size:][:size] = S.reshape(size)

    def latent_finish(self, fused, q_plain, q_folded, cache, positions, token_seq, block_table, heads, dim, rope_dim,
                      latent_dim, block_size, rotation=None, rotated=0, latent_offset=0, latent_gamma=None, eps=0.0,
                      write_cache=True, q_whole=None):
        self.calls.append("latent_finish")
        assert q_whole is None, "whole query heads are the bfloat16 prompt path's"
        n, key_dim = fused.shape[0], latent_dim + rope_dim
        q = fused[:, :heads * (dim + rope_dim)].view(n, heads, dim + rope_dim)
        q_plain.copy_(q[:, :, :dim].reshape(n, heads * dim).to(q_plain.dtype))
        if rope_dim:
            turned = self._turn(q[:, :, dim:], rotation, positions, rotated)
            q_folded.view(n, heads, key_dim)[:, :, latent_dim:] = turned.to(q_folded.dtype)
        if not write_cache:
            return
        c = fused[:, latent_offset:latent_offset + latent_dim]
        c = c / torch.sqrt((c * c).mean(dim=-1, keepdim=True) + eps) * latent_gamma
        rows = torch.cat([c, self._turn(fused[:, latent_offset + latent_dim:latent_offset + key_dim], rotation, positions,
                                        rotated)], dim=-1)
        for t in range(n):
            pos = int(positions[t])
            block = int(block_table[int(token_seq[t]), pos // block_size])
            cache[block, 0, pos % block_size, :] = rows[t].to(cache.dtype)

    def route_tokens(self, h, router_w, correction, top, scale, renormalize, chosen, weights, shared_gate_weight=None,
                     shared_gate_out=None, softmax=False, groups=0, keep=0, renorm_eps=0.0):
        self.calls.append("route_tokens")
        logits = h.float() @ router_w.float().T
        s = torch.softmax(logits, dim=-1) if softmax else torch.sigmoid(logits)
        choice = s + correction if correction is not None else s
        if groups > 1:
            size = s.shape[1] // groups
            best = choice.view(-1, groups, size).max(dim=-1).values
            kept = torch.zeros_like(best, dtype=torch.bool).scatter_(1, best.topk(keep, dim=-1).indices, True)
            choice = choice.masked_fill(~kept.repeat_interleave(size, dim=1), -float("inf"))
        picked = torch.topk(choice, top, dim=-1).indices
        w = torch.gather(s, 1, picked)
        if renormalize:
            w = w / (w.sum(dim=-1, keepdim=True) + renorm_eps)
        chosen.copy_(picked.to(torch.int32))
        weights.copy_(w * scale)
        if shared_gate_out is not None:
            shared_gate_out.copy_(torch.sigmoid(h.float() @ shared_gate_weight.float()))

    def sort_by_expert(self, chosen, experts, offsets, order, place):
        self.calls.append("sort_by_expert")
        flat = chosen.reshape(-1).long()
        sorted_pairs = torch.argsort(flat, stable=True)
        counts = torch.bincount(flat, minlength=experts)
        offsets[0] = 0
        offsets[1:] = torch.cumsum(counts, 0).to(torch.int32)
        order.copy_((sorted_pairs // chosen.shape[1]).to(torch.int32))
        place.view(-1)[sorted_pairs] = torch.arange(flat.numel(), dtype=torch.int32)

    def expert_rows_sorted_first(self, hidden):
        return False

    def expert_linear(self, a, w, offsets, out, rows=None, activation=None, flag=None, gated=False):
        self.calls.append("expert_linear")
        for e in range(w.shape[0]):
            lo, hi = int(offsets[e]), int(offsets[e + 1])
            if hi == lo:
                continue
            src = a[rows[lo:hi].long()] if rows is not None else a[lo:hi]
            result = src.float() @ w[e].float().T
            if gated:                               # tiles of 8 gate rows and their 8 up rows
                tiles = result.view(result.shape[0], -1, 2, 8)
                result = (ACTIVATIONS[activation](tiles[:, :, 0]) * tiles[:, :, 1]).reshape(result.shape[0], -1)
            elif activation is not None:
                result = ACTIVATIONS[activation](result)
            out[lo:hi] = result.to(out.dtype)

    def combine_experts(self, results, place, weights, shared, share, x, add=True):
        self.calls.append("combine_experts")
        total = (results[place.long()] * weights[:, :, None]).sum(dim=1)
        if shared is not None:
            total = total + (shared * share[:, None] if share is not None else shared)
        if add:
            x.add_(total)
        else:
            x.copy_(total)

    def rglru_conv(self, yx, x_offset, x_bias, conv_w, conv_b, u, step_meta, state):
        self.calls.append("rglru_conv")
        positions, token_seq, cu_q, slot_ids = step_meta
        channels, taps = conv_w.shape
        for t in range(u.shape[0]):
            p, s = int(positions[t]), int(token_seq[t])
            ring = state[int(slot_ids[s]), 2 * channels:(2 + taps) * channels].view(taps, channels)
            total = conv_b.clone()
            for k in range(taps):
                back = taps - 1 - k
                if p - back < 0:
                    continue
                inside = t - back >= int(cu_q[s])
                value = yx[t - back, x_offset:x_offset + channels] + x_bias if inside else ring[(p - back) % taps]
                total = total + conv_w[:, k] * value
            u[t] = total

    def rglru_rate(self, lam, rate):
        rate.copy_(8.0 * torch.nn.functional.softplus(lam))
        return rate

    def rglru_gates(self, gates, u, yx, y_bias, r_bias, i_bias, rate, part):
        self.calls.append("rglru_gates")
        n, channels = u.shape
        pairs = gates.view(n, channels // part, 2, part)
        r = torch.sigmoid(pairs[:, :, 0, :] + r_bias.view(-1, part))
        i = torch.sigmoid(pairs[:, :, 1, :] + i_bias.view(-1, part))
        a = torch.exp(-r * rate.view(-1, part))
        driven = torch.sqrt(1.0 - a * a) * i * u.view(n, -1, part)
        pairs[:, :, 0, :] = a
        pairs[:, :, 1, :] = driven
        yx[:, :channels] = torch.nn.functional.gelu(yx[:, :channels] + y_bias, approximate="tanh")

    def rglru_scan_scratch(self, n_seqs, max_q_len, channels):
        return 0

    def rglru_scan(self, gates, yx, x_offset, x_bias, out, part, taps, step_meta, state, max_q_len=0, summary=None):
        self.calls.append("rglru_scan")
        positions, token_seq, cu_q, slot_ids = step_meta
        n, channels = gates.shape[0], gates.shape[1] // 2
        pairs = gates.view(n, channels // part, 2, part)
        for s in range(slot_ids.numel()):
            first, last = int(cu_q[s]), int(cu_q[s + 1]) - 1
            row = state[int(slot_ids[s])]
            p_first = int(positions[first])
            S = row[((p_first - 1) & 1) * channels:][:channels].clone() if p_first > 0 else torch.zeros(channels)
            for t in range(first, last + 1):
                S = pairs[t, :, 0, :].reshape(-1) * S + pairs[t, :, 1, :].reshape(-1)
                out[t, :channels] = (S * yx[t, :channels]).to(out.dtype)
            p_last = p_first + last - first
            row[(p_last & 1) * channels:][:channels] = S
            ring = row[2 * channels:(2 + taps) * channels].view(taps, channels)
            for back in range(min(taps, last - first + 1)):
                ring[(p_last - back) % taps] = yx[last - back, x_offset:x_offset + channels] + x_bias

    def add_scaled(self, out, other, factor):
        self.calls.append("add_scaled")
        out.add_(other * factor)

    def projection_norm(self, rows, eps, segments):
        self.calls.append("projection_norm")
        for offset, width, bias, weight in segments:
            x = rows[:, offset:offset + width] + (bias if bias is not None else 0.0)
            rows[:, offset:offset + width] = x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps) * weight

    def short_conv_rotary(self, rows, bias, conv_w, taps, cos_sin, rotated, interleaved, block_table, q_out, k_cache,
                          v_cache, num_heads, num_kv_heads, dim, block_size, write_kv, step_meta, state, state_offset=0):
        self.calls.append("short_conv_rotary")
        positions, token_seq, cu_q, slot_ids = step_meta
        n, channels = rows.shape[0], (num_heads + num_kv_heads) * dim
        u = rows[:, :channels] + (bias if bias is not None else 0.0)
        y = torch.zeros(n, channels)
        for t in range(n):
            seq, p = int(token_seq[t]), int(positions[t])
            first = int(cu_q[seq])
            if taps == 0:
                y[t] = u[t]
                continue
            ring = (state[int(slot_ids[seq])][state_offset:state_offset + taps * channels].view(taps, channels)
                    if taps > 1 else None)
            for j in range(taps):
                back = taps - 1 - j
                if p - back >= 0:
                    y[t] += conv_w[:, j] * (u[t - back] if t - back >= first else ring[(p - back) % taps])
        heads = y.view(n, num_heads + num_kv_heads, dim)
        turned = heads.clone()
        if rotated:
            cs = cos_sin[positions.long()]                            # [n, rotated / 2, 2]
            c, sn = cs[:, None, :, 0], cs[:, None, :, 1]
            if interleaved:
                a, b = heads[..., 0:rotated:2], heads[..., 1:rotated:2]
                turned[..., 0:rotated:2], turned[..., 1:rotated:2] = a * c - b * sn, b * c + a * sn
            else:
                half = rotated // 2
                a, b = heads[..., :half], heads[..., half:rotated]
                turned[..., :half], turned[..., half:rotated] = a * c - b * sn, b * c + a * sn
        q_out.copy_(turned[:, :num_heads].reshape(n, num_heads * dim).to(q_out.dtype))
        if not write_kv:
            return
        for t in range(n):
            pos = int(positions[t])
            block = int(block_table[int(token_seq[t]), pos // block_size])
            k_cache[block, :, pos % block_size, :] = turned[t, num_heads:].to(k_cache.dtype)
            if v_cache is not None:
                v_cache[block, :, pos % block_size, :] = heads[t, num_heads:].to(v_cache.dtype)

    def short_conv_remember(self, rows, bias, channels, taps, n_seqs, step_meta, state, state_offset=0):
        self.calls.append("short_conv_remember")
        if taps <= 1:
            return
        positions, token_seq, cu_q, slot_ids = step_meta
        for seq in range(n_seqs):
            first, end = int(cu_q[seq]), int(cu_q[seq + 1])
            ring = state[int(slot_ids[seq])][state_offset:state_offset + taps * channels].view(taps, channels)
            for t in range(max(first, end - (taps - 1)), end):
                ring[int(positions[t]) % taps] = rows[t, :channels] + (bias if bias is not None else 0.0)

    def time_mix_state_floats(self, hidden, heads, dim):
        return 2 * heads * dim * dim + 2 * hidden

    def token_shift_mix(self, h, mu, mixes, heads, dim, step_meta, state, state_offset=0):
        self.calls.append("token_shift_mix")
        positions, token_seq, cu_q, slot_ids = step_meta
        hidden = h.shape[1]
        base = state_offset + 2 * heads * dim * dim
        for t in range(h.shape[0]):
            seq, p = int(token_seq[t]), int(positions[t])
            if t > int(cu_q[seq]):
                before = h[t - 1].float()
            elif p > 0:
                before = state[int(slot_ids[seq])][base + ((p - 1) & 1) * hidden:][:hidden]
            else:
                before = torch.zeros(hidden)
            now = h[t].float()
            for m in range(mixes.shape[0]):
                mixes[m, t] = (now + (before - now) * mu[m]).to(mixes.dtype)

    def time_mix_decay(self, lora, rank, w2, w0, decay):
        self.calls.append("time_mix_decay")
        decay.copy_(torch.exp(-torch.exp(torch.tanh(lora[:, :rank]) @ w2.float() + w0)))       # (w2 is [rank, channels])

    def time_mix_scan(self, r, k, v, decay, bonus, out, h, n_seqs, heads, dim, step_meta, state, state_offset=0):
        self.calls.append("time_mix_scan")
        positions, token_seq, cu_q, slot_ids = step_meta
        hidden, size = h.shape[1], heads * dim * dim
        u = bonus.view(heads, dim)
        for seq in range(n_seqs):
            first, end = int(cu_q[seq]), int(cu_q[seq + 1])
            if end <= first:
                continue
            row = state[int(slot_ids[seq])]
            p0 = int(positions[first])
            S = (row[state_offset + ((p0 - 1) & 1) * size:][:size].clone().view(heads, dim, dim) if p0 > 0
                 else torch.zeros(heads, dim, dim))
            for t in range(first, end):
                kv = k[t].view(heads, dim)[:, :, None] * v[t].view(heads, dim)[:, None, :]
                out[t] = torch.einsum("hi,hij->hj", r[t].view(heads, dim), S + u[:, :, None] * kv).reshape(-1)
                S = decay[t].view(heads, dim)[:, :, None] * S + kv
            last = p0 + end - first - 1
            row[state_offset + (last & 1) * size:][:size] = S.reshape(size)
            row[state_offset + 2 * size + (last & 1) * hidden:][:hidden] = h[end - 1].float()

    def time_mix_finish(self, o, gate, norm, eps, out_scale, out, heads, dim):
        self.calls.append("time_mix_finish")
        n = o.shape[0]
        heads_o = o.view(n, heads, dim)
        unit = heads_o / torch.sqrt((heads_o * heads_o).mean(dim=-1, keepdim=True) + eps)
        out.zero_()
        out[:, :heads * dim] = (unit.reshape(n, -1) * norm * gate * torch.sigmoid(gate) * out_scale).to(out.dtype)

    def scale_inplace(self, x, factor):
        x.mul_(factor)

    def add_inplace(self, out, other):
        out.add_(other)

    def argmax(self, logits, out, flag=None):
        out.copy_(torch.argmax(logits, dim=-1).to(torch.int32))


def double_loader():
    made = {}

    def load(dtype, head_dim):
        key = (dtype, head_dim)
        if key not in made:
            made[key] = DoubleKernels(dtype, head_dim)
        return made[key]
    return load
