"""The kernel library as Python calls: loads the compiled .so and checks arguments.

There is one backend: hand-written CUDA for sm_100a, loaded through ctypes.
If it cannot be compiled or loaded, or no CUDA device is present, the calls
raise; nothing falls back to the CPU or to library model code.
"""
from __future__ import annotations

import ctypes
import struct
from typing import Dict, Optional, Tuple

import torch

from .csrc.build import BuildError, build_library
from .residual import COLUMNS_PER_PARTIAL, KERNEL_FOLD_ROWS, NormedRows

MODE_STORE, MODE_STORE_F32, MODE_ADD_F32, MODE_GATED = 0, 1, 2, 3
MODE_QKV_ROPE = 4          # (linear_qkv_rope's own epilogue; named for Kernels.linear_form)
MODE_ACT = 5               # out = act(a . w^T) in the compute dtype: the first projection of a feed-forward without a gate
# activations that every projection kernel implements, on a gate or on what it stores (csrc/common.cuh)
ACTIVATIONS = {"silu": 0, "swish": 0, "gelu_tanh": 1, "gelu_pytorch_tanh": 1, "relu2": 2, "relu_squared": 2,
               "swiglu_clamp": 3}
# activations that take one number (``activation_param``): the clamp of both branches of "swiglu_clamp", a gated unit
# min(g, c) * sigmoid(1.702 min(g, c)) * (clamp(u, -c, c) + 1); it is an activation of gated projections only
PARAMETRIC_ACTIVATIONS = ("swiglu_clamp",)
# what the kernels of a routed feed-forward are built for (csrc/routed_mlp.cu)
MAX_EXPERTS, MAX_EXPERTS_PER_TOKEN = 1024, 16
MAX_STREAMS = 8            # copies of the residual stream that ``stream_mix`` takes (csrc/stream_mix.cu)


def activation_word(activation: str, param: float = 0.0):
    """An activation as the kernels take it: its code in the low bits, the bits of its float parameter in the high 32."""
    code = ACTIVATIONS[activation]
    if activation in PARAMETRIC_ACTIVATIONS:
        code |= struct.unpack("<I", struct.pack("<f", float(param)))[0] << 32
    return ctypes.c_longlong(code)


_DTYPE_NAMES = {torch.float32: "float32", torch.bfloat16: "bfloat16"}


class KernelError(RuntimeError):
    pass


def _ptr(tensor: Optional[torch.Tensor]):
    return ctypes.c_void_p(0 if tensor is None else tensor.data_ptr())


_NULL = ctypes.c_void_p(0)
_NO_FOLD = (_NULL, _NULL, _NULL, 0, _NULL, ctypes.c_float(0.0), _NULL)
_SCOPED_STREAM = None


def _stream():
    if _SCOPED_STREAM is not None:
        return _SCOPED_STREAM
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


class stream_scope:
    """Within the scope every kernel goes to the stream that was current when the scope began
    (asking torch for the current stream at each of a step's two hundred launches costs more
    than the launches themselves)."""

    def __enter__(self):
        global _SCOPED_STREAM
        self.previous = _SCOPED_STREAM
        _SCOPED_STREAM = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream) if torch.cuda.is_available() else None
        return self

    def __exit__(self, *exc):
        global _SCOPED_STREAM
        _SCOPED_STREAM = self.previous
        return False


class Kernels:
    """The kernels of one (compute dtype, head size) library."""

    launches = 0          # kernel launches issued through any library of this process

    def __init__(self, dtype: torch.dtype, head_dim: int, verbose: bool = True):
        if dtype not in _DTYPE_NAMES:
            raise KernelError(f"no kernels for dtype {dtype}")
        self.dtype = dtype
        self.head_dim = head_dim
        try:
            self.path = build_library(_DTYPE_NAMES[dtype], head_dim, verbose=verbose)
        except BuildError as error:
            raise KernelError(str(error)) from None
        try:
            self.lib = ctypes.CDLL(str(self.path))
        except OSError as error:
            raise KernelError(f"cannot load {self.path}: {error}") from None
        self.lib.skv_last_error.restype = ctypes.c_char_p
        if self.lib.skv_library_head_dim() != head_dim:
            raise KernelError(f"{self.path} was built for another head size")
        # A device word kernels raise bits in (4: a pipeline wait inside a kernel timed out).
        self.error_flag = torch.zeros(1, dtype=torch.int32, device="cuda") if torch.cuda.is_available() else None

    # ---- helpers -----------------------------------------------------------
    def _check(self, code: int, name: str) -> None:
        Kernels.launches += 1
        if code != 0:
            raise KernelError(f"{name}: {self.lib.skv_last_error().decode()}")

    def _want(self, tensor: torch.Tensor, dtype, name: str) -> None:
        if not tensor.is_cuda:
            raise KernelError(f"{name} must be a CUDA tensor: the kernels run on the GPU only")
        if tensor.dtype != dtype:
            raise KernelError(f"{name} must be {dtype}, got {tensor.dtype}")
        if not tensor.is_contiguous():
            raise KernelError(f"{name} must be contiguous")

    # ---- kernels -------------------------------------------------------------
    _KINDS = {torch.float32: 0, torch.bfloat16: 1, torch.float16: 2}

    def convert(self, src, out):
        """out = src in out's type (float32, bfloat16, float16), rounded to nearest even where bits are lost: how
        checkpoint tensors get from their stored type to the compute type once they are on the device."""
        if src.dtype not in self._KINDS or out.dtype not in self._KINDS:
            raise KernelError(f"convert: float32, bfloat16 and float16 only, not {src.dtype} -> {out.dtype}")
        if src.shape != out.shape or src.device != out.device or not src.is_cuda:
            raise KernelError("convert: source and result must have one shape and lie on the same GPU")
        if not (src.is_contiguous() and out.is_contiguous()):
            raise KernelError("convert: tensors must be contiguous")
        self.lib.skv_convert.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong,
                                         ctypes.c_void_p]
        self._check(self.lib.skv_convert(_ptr(src), self._KINDS[src.dtype], _ptr(out), self._KINDS[out.dtype],
                                         src.numel(), _stream()), "convert")
        return out

    def embed(self, table, ids, out, flag=None, stats=None):
        """out[t, :] = table[ids[t], :] as float32; with ``stats`` each row's sum of squares too."""
        self._want(table, self.dtype, "table"); self._want(ids, torch.int32, "ids")
        self._want(out, torch.float32, "out")
        n, hidden = out.shape
        vocab = table.shape[0]
        if table.shape[1] != hidden or ids.numel() != n:
            raise KernelError("embed: shapes do not agree")
        fold = self._fold_target(stats, n, hidden)
        self._check(self.lib.skv_embed(_ptr(table), _ptr(ids), _ptr(out), n, hidden, vocab, _ptr(flag),
                                       *(fold[:6] if fold else _NO_FOLD[:6]), _stream()), "embed")
        if stats is not None:
            stats.filled(1 if stats.consumer_sums else 0) if fold else stats.invalidate()

    def _fold_target(self, stats, rows: int, width: int):
        """Arguments (scaled rows, next norm's weight, partial sums, their stride, rows' factors, next norm's
        eps, counter) for a kernel that writes ``rows`` rows of the stream; None where it cannot fold."""
        if stats is None or stats.next_norm is None or self.dtype != torch.bfloat16 or rows > KERNEL_FOLD_ROWS:
            return None
        gamma = stats.next_norm.gamma
        self._want(gamma, torch.float32, "gamma"); self._want(stats.partials, torch.float32, "partials")
        self._want(stats.scaled, self.dtype, "scaled"); self._want(stats.row_scale, torch.float32, "row_scale")
        self._want(stats.counter, torch.int32, "counter")
        if (gamma.numel() != width or tuple(stats.scaled.shape) != (rows, width) or stats.row_scale.numel() != rows
                or stats.partials.shape[0] != rows
                or stats.partials.shape[1] * COLUMNS_PER_PARTIAL < width):
            raise KernelError("the buffers of the folded norm do not match the stream")
        return (_ptr(stats.scaled), _ptr(gamma), _ptr(stats.partials), stats.partials.shape[1], _ptr(stats.row_scale),
                ctypes.c_float(stats.next_norm.spec.eps), _NULL if stats.consumer_sums else _ptr(stats.counter))

    def rmsnorm(self, x, gamma, eps: float, out, rows=None):
        """out[r, :] = rmsnorm(x[rows[r] or r, :]) * gamma, in the compute dtype."""
        self._want(x, torch.float32, "x"); self._want(gamma, torch.float32, "gamma")
        self._want(out, self.dtype, "out")
        hidden = x.shape[-1]
        n_rows = out.shape[0]
        if gamma.numel() != hidden or out.shape[-1] != hidden:
            raise KernelError("rmsnorm: shapes do not agree")
        if rows is not None:
            self._want(rows, torch.int32, "rows")
            if rows.numel() != n_rows:
                raise KernelError("rmsnorm: one output row per index is needed")
        elif x.shape[0] != n_rows:
            raise KernelError("rmsnorm: shapes do not agree")
        self._check(self.lib.skv_rmsnorm(_ptr(x), _ptr(gamma), ctypes.c_float(eps), _ptr(out), _ptr(rows),
                                         n_rows, hidden, _stream()), "rmsnorm")

    def linear(self, a, w, out, mode: int = MODE_STORE, activation: str = "silu", flag=None, stats=None,
               activation_param: float = 0.0):
        """out = a[M,K] . w[N,K]^T with the epilogue ``mode``.

        ``a`` may be ``residual.NormedRows``: the norm is applied while the activations are
        loaded.  ``stats`` (residual-add mode): the statistics of ``out`` are brought up to date where
        the kernel can do that, and marked unknown where it cannot."""
        normed = a if isinstance(a, NormedRows) else None
        if normed is None:
            self._want(a, self.dtype, "a")
        else:
            self._want(normed.scaled, self.dtype, "scaled"); self._want(normed.row_scale, torch.float32, "row_scale")
            if normed.rows is not None:
                self._want(normed.rows, torch.int32, "rows")
            if normed.row_scale.numel() != normed.scaled.shape[0]:
                raise KernelError("linear: one factor per row of the normalised input is needed")
        self._want(w, self.dtype, "w")
        M, K = a.shape
        N = w.shape[0]
        if w.shape[1] != K:
            raise KernelError(f"linear: inner sizes differ ({K} and {w.shape[1]})")
        out_cols = N // 2 if mode == MODE_GATED else N
        out_dtype = self.dtype if mode in (MODE_STORE, MODE_GATED, MODE_ACT) else torch.float32
        self._want(out, out_dtype, "out")
        if tuple(out.shape) != (M, out_cols):
            raise KernelError(f"linear: out must be [{M}, {out_cols}], got {list(out.shape)}")
        if activation not in ACTIVATIONS:
            raise KernelError(f"linear: unknown activation '{activation}'")
        if activation in PARAMETRIC_ACTIVATIONS and mode == MODE_ACT:
            raise KernelError(f"linear: '{activation}' is an activation of gated projections")
        if stats is not None and mode != MODE_ADD_F32:
            raise KernelError("linear: statistics are kept by the residual-add mode only")
        if normed is not None:
            if stats is not None:
                raise KernelError("linear: a folded norm on the input and statistics of the output do not go together")
            if normed.n_partials > 0:
                self._want(normed.partials, torch.float32, "partials")
                if normed.partials.shape[0] != normed.scaled.shape[0] or normed.partials.shape[1] < normed.n_partials:
                    raise KernelError("linear: the partial sums do not match the normalised input")
                factor = (_NULL, _ptr(normed.partials), normed.n_partials, normed.partials.shape[1],
                          ctypes.c_float(normed.eps))
            else:
                factor = (_ptr(normed.row_scale), _NULL, 0, 0, ctypes.c_float(0.0))
            self._check(self.lib.skv_linear_normed(
                _ptr(normed.scaled), *factor, _ptr(normed.rows), _ptr(w), _ptr(out), M, N, K, mode,
                activation_word(activation, activation_param), _stream()), "linear")
            return
        fold = self._fold_target(stats, M, N)
        self._check(self.lib.skv_linear(_ptr(a), _ptr(w), _ptr(out), M, N, K, mode,
                                        activation_word(activation, activation_param),
                                        _ptr(flag if flag is not None else self.error_flag), *(fold or _NO_FOLD), _stream()),
                    "linear")
        if stats is not None:
            if fold:
                stats.filled((N + COLUMNS_PER_PARTIAL - 1) // COLUMNS_PER_PARTIAL if stats.consumer_sums else 0)
            else:
                stats.invalidate()

    def has_linear_qkv_rope(self) -> bool:
        return bool(self.lib.skv_has_linear_qkv_rope())

    def linear_form(self, M: int, N: int, K: int, mode: int) -> str:
        """Which tensor-memory kernel serves a projection of this shape and epilogue on this GPU (``mode`` 4 is the
        q|k|v projection with the rotary epilogue); for tests that must reach each of them."""
        code = int(self.lib.skv_linear_tcgen05_form(int(M), int(N), int(K), int(mode)))
        return {0: "few_tokens", 1: "tile_128", 2: "tile_160", 3: "tile_256", 4: "pair_256"}.get(code, "none")

    def linear_qkv_rope(self, a, w, q_out, cos_sin, positions, token_seq, block_table, k_cache, v_cache,
                        num_heads: int, num_kv_heads: int, head_dim: int, block_size: int, write_kv: bool, flag=None):
        """The q|k|v projection of a step of more than 128 tokens with ``rope_kv_write`` in its epilogue (bfloat16,
        head size 64 or 128): ``q_out`` [M, heads * head_dim] gets the rotated queries, the cache the rotated keys and
        the values of every token, at the row of its position in the block its sequence's table names."""
        self._want(a, self.dtype, "a"); self._want(w, self.dtype, "w"); self._want(q_out, self.dtype, "q_out")
        self._want(positions, torch.int32, "positions"); self._want(token_seq, torch.int32, "token_seq")
        self._want(block_table, torch.int32, "block_table")
        self._want(k_cache, self.dtype, "k_cache"); self._want(v_cache, self.dtype, "v_cache")
        if cos_sin is not None:
            self._want(cos_sin, torch.float32, "cos_sin")
        M, K = a.shape
        N = w.shape[0]
        if w.shape[1] != K or N != (num_heads + 2 * num_kv_heads) * head_dim:
            raise KernelError("linear_qkv_rope: the weight must be [(heads + 2 kv heads) * head_dim, K]")
        if tuple(q_out.shape) != (M, num_heads * head_dim) or positions.numel() != M or token_seq.numel() != M:
            raise KernelError("linear_qkv_rope: one query row, one position and one sequence index per token is needed")
        if tuple(k_cache.shape[1:]) != (num_kv_heads, block_size, head_dim) or k_cache.shape != v_cache.shape:
            raise KernelError("linear_qkv_rope: the cache must be [blocks, kv_heads, block_size, head_dim]")
        self._check(self.lib.skv_linear_qkv_rope(
            _ptr(a), _ptr(w), _ptr(q_out), M, N, K, _ptr(cos_sin), _ptr(positions), _ptr(token_seq), _ptr(block_table),
            block_table.shape[1], _ptr(k_cache), _ptr(v_cache), num_heads, num_kv_heads, head_dim, block_size,
            int(bool(write_kv)), _ptr(flag if flag is not None else self.error_flag), _stream()), "linear_qkv_rope")

    def rope_kv_write(self, qkv, cos_sin, positions, token_seq, block_table, q_out, k_cache, v_cache,
                      num_heads: int, num_kv_heads: int, head_dim: int, block_size: int, write_kv: bool):
        self._want(qkv, torch.float32, "qkv"); self._want(q_out, self.dtype, "q_out")
        self._want(positions, torch.int32, "positions"); self._want(token_seq, torch.int32, "token_seq")
        self._want(block_table, torch.int32, "block_table")
        self._want(k_cache, self.dtype, "k_cache"); self._want(v_cache, self.dtype, "v_cache")
        if cos_sin is not None:
            self._want(cos_sin, torch.float32, "cos_sin")
        n = qkv.shape[0]
        if qkv.shape[1] != (num_heads + 2 * num_kv_heads) * head_dim:
            raise KernelError("rope_kv_write: qkv width does not match the head counts")
        self._check(self.lib.skv_rope_kv_write(
            _ptr(qkv), _ptr(cos_sin), _ptr(positions), _ptr(token_seq), _ptr(block_table),
            block_table.shape[1], _ptr(q_out), _ptr(k_cache), _ptr(v_cache), n, num_heads, num_kv_heads,
            head_dim, block_size, int(bool(write_kv)), _stream()), "rope_kv_write")

    def attention(self, q, k_cache, v_cache, block_table, positions, token_seq, out, num_heads: int,
                  num_kv_heads: int, head_dim: int, block_size: int, scale: float, window: int = 0):
        self._want(q, self.dtype, "q"); self._want(out, self.dtype, "out")
        self._want(k_cache, self.dtype, "k_cache"); self._want(v_cache, self.dtype, "v_cache")
        self._want(block_table, torch.int32, "block_table")
        self._want(positions, torch.int32, "positions"); self._want(token_seq, torch.int32, "token_seq")
        n = q.shape[0]
        self._check(self.lib.skv_attention(
            _ptr(q), _ptr(k_cache), _ptr(v_cache), _ptr(block_table), block_table.shape[1], _ptr(positions),
            _ptr(token_seq), _ptr(out), n, num_heads, num_kv_heads, head_dim, block_size,
            ctypes.c_float(scale), window, _stream()), "attention")

    def _extras(self, bias, gate, gate_stride: int, num_heads: int, name: str, per_element_width: int = 0):
        """Arguments (bias table, its length, gate logits, their row stride) of the attention kernels' optional terms.
        ``per_element_width``: the gate holds a logit for every output number, that many a head."""
        bias_len = 0
        if bias is not None:
            self._want(bias, torch.float32, "bias")
            if bias.dim() != 2 or bias.shape[0] != num_heads or bias.shape[1] < 1:
                raise KernelError(f"{name}: the bias table must be [heads, distances]")
            bias_len = bias.shape[1]
        if gate is not None and (gate.dtype != torch.float32 or not gate.is_cuda
                                 or gate_stride < num_heads * max(1, per_element_width)):
            raise KernelError(f"{name}: the gate must be float32 on the GPU, a row at least heads wide")
        if per_element_width and gate is None:
            raise KernelError(f"{name}: a gate per output number needs the gate")
        return _ptr(bias), bias_len, _ptr(gate), int(gate_stride) if gate is not None else 0

    def has_attention_prefill(self) -> bool:
        return bool(self.lib.skv_has_attention_prefill())

    def attention_prefill(self, q, k_cache, v_cache, block_table, cu_q, ctx_after, out, max_q_len: int,
                          num_heads: int, num_kv_heads: int, head_dim: int, block_size: int, scale: float,
                          window: int = 0, bias=None, gate=None, gate_stride: int = 0):
        """Many new tokens per sequence (bfloat16 build, head size up to 128): sequence ``s`` owns rows
        ``cu_q[s]..cu_q[s+1]-1`` of ``q``/``out``; ``ctx_after[s]`` keys are cached, this step's included.
        ``bias`` (float32 ``[heads, distances]``, in units of log2: the natural bias times log2 e): ``bias[h, i - j]`` is
        taken off the score of query i and key j.
        ``gate`` (float32 logits, token t and head h at ``[t * gate_stride + h]``): the output times its sigmoid."""
        self._want(q, self.dtype, "q"); self._want(out, self.dtype, "out")
        self._want(k_cache, self.dtype, "k_cache"); self._want(v_cache, self.dtype, "v_cache")
        self._want(block_table, torch.int32, "block_table"); self._want(cu_q, torch.int32, "cu_q")
        self._want(ctx_after, torch.int32, "ctx_after")
        n_seqs = ctx_after.numel()
        if cu_q.numel() != n_seqs + 1 or block_table.shape[0] != n_seqs:
            raise KernelError("attention_prefill: one length, one offset pair and one table row per sequence is needed")
        self._check(self.lib.skv_attention_prefill_extras(
            _ptr(q), _ptr(k_cache), _ptr(v_cache), _ptr(block_table), block_table.shape[1], _ptr(cu_q),
            _ptr(ctx_after), _ptr(out), n_seqs, max_q_len, num_heads, num_kv_heads, head_dim, block_size,
            ctypes.c_float(scale), window, *self._extras(bias, gate, gate_stride, num_heads, "attention_prefill"),
            _stream()), "attention_prefill")

    def has_attention_prefill_tc(self) -> bool:
        return bool(self.lib.skv_has_attention_prefill_tc())

    def attention_prefill_tc(self, q, k_cache, v_cache, block_table, cu_q, ctx_after, out, max_q_len: int,
                             num_heads: int, num_kv_heads: int, head_dim: int, block_size: int, scale: float,
                             window: int = 0, flag=None, bias=None, gate=None, gate_stride: int = 0,
                             softcap: float = 0.0, gate_per_element: bool = False, sink=None):
        """``attention_prefill`` with both products on the tcgen05 tensor cores (bfloat16, head size 64 or 128).
        ``sink`` (float32 per head): ``exp(sink[h])`` counts once in the softmax's denominator.
        ``softcap`` c > 0: scores become ``c * tanh(score / c)``; ``gate_per_element``: a logit for every output
        number, at ``[t * gate_stride + h * head_dim + d]``."""
        self._want(q, self.dtype, "q"); self._want(out, self.dtype, "out")
        self._want(k_cache, self.dtype, "k_cache"); self._want(v_cache, self.dtype, "v_cache")
        self._want(block_table, torch.int32, "block_table"); self._want(cu_q, torch.int32, "cu_q")
        self._want(ctx_after, torch.int32, "ctx_after")
        n_seqs = ctx_after.numel()
        if cu_q.numel() != n_seqs + 1 or block_table.shape[0] != n_seqs:
            raise KernelError("attention_prefill_tc: one length, one offset pair and one table row per sequence is needed")
        if tuple(k_cache.shape[1:]) != (num_kv_heads, block_size, head_dim) or k_cache.shape != v_cache.shape:
            raise KernelError("attention_prefill_tc: the cache must be [blocks, kv_heads, block_size, head_dim]")
        if sink is not None:
            self._want(sink, torch.float32, "sink")
            if sink.numel() != num_heads:
                raise KernelError("attention_prefill_tc: the sink must hold one number per head")
        self._check(self.lib.skv_attention_prefill_tc_extras(
            _ptr(q), _ptr(k_cache), _ptr(v_cache), k_cache.shape[0], _ptr(block_table), block_table.shape[1],
            _ptr(cu_q), _ptr(ctx_after), _ptr(out), n_seqs, q.shape[0], max_q_len, num_heads, num_kv_heads, head_dim,
            block_size, ctypes.c_float(scale), window,
            *self._extras(bias, gate, gate_stride, num_heads, "attention_prefill_tc", head_dim if gate_per_element else 0),
            ctypes.c_float(softcap), int(bool(gate_per_element)), _ptr(sink),
            _ptr(flag if flag is not None else self.error_flag), _stream()), "attention_prefill_tc")

    def attention_decode(self, q, k_cache, v_cache, block_table, ctx_after, out, num_heads: int,
                         num_kv_heads: int, head_dim: int, block_size: int, scale: float, window: int = 0,
                         splits: int = 1, scratch_o=None, scratch_ml=None, bias=None, gate=None, gate_stride: int = 0,
                         softcap: float = 0.0, gate_per_element: bool = False, sink=None):
        """(``bias``, ``gate``: as in ``attention_prefill``; ``softcap``, ``gate_per_element``, ``sink``: as in
        ``attention_prefill_tc``.)
        One new token per sequence (bfloat16 build): ``ctx_after[s]`` keys are cached for sequence
        ``s``, the newest being the query's own.  ``splits`` > 1 cuts each context across blocks and
        needs float scratch: ``scratch_o`` [seqs*heads*splits*head_dim], ``scratch_ml`` [seqs*heads*splits*2]."""
        self._want(q, self.dtype, "q"); self._want(out, self.dtype, "out")
        self._want(k_cache, self.dtype, "k_cache"); self._want(v_cache, self.dtype, "v_cache")
        self._want(block_table, torch.int32, "block_table"); self._want(ctx_after, torch.int32, "ctx_after")
        n = q.shape[0]
        if ctx_after.numel() != n or block_table.shape[0] != n:
            raise KernelError("attention_decode: one length and one table row per sequence is needed")
        if splits > 1:
            self._want(scratch_o, torch.float32, "scratch_o"); self._want(scratch_ml, torch.float32, "scratch_ml")
            if scratch_o.numel() < n * num_heads * splits * head_dim or scratch_ml.numel() < n * num_heads * splits * 2:
                raise KernelError("attention_decode: scratch is too small for this many splits")
        if sink is not None:
            self._want(sink, torch.float32, "sink")
            if sink.numel() != num_heads:
                raise KernelError("attention_decode: the sink must hold one number per head")
        self._check(self.lib.skv_attention_decode_sink(
            _ptr(q), _ptr(k_cache), _ptr(v_cache), _ptr(block_table), block_table.shape[1], _ptr(ctx_after),
            _ptr(out), _ptr(scratch_o), _ptr(scratch_ml), n, num_heads, num_kv_heads, head_dim, block_size,
            ctypes.c_float(scale), window, splits,
            *self._extras(bias, gate, gate_stride, num_heads, "attention_decode", head_dim if gate_per_element else 0),
            ctypes.c_float(softcap), int(bool(gate_per_element)), _ptr(sink), _stream()), "attention_decode")

    def has_attention_decode_fused(self) -> bool:
        return bool(self.lib.skv_has_attention_decode_fused())

    def attention_decode_fused(self, qkv, cos_sin, k_cache, v_cache, block_table, ctx_after, out, num_heads: int,
                               num_kv_heads: int, head_dim: int, block_size: int, scale: float, window: int = 0,
                               splits: int = 1, write_kv: bool = True, q_bias=None, k_bias=None, v_bias=None,
                               value_norm_eps=None, bias=None, gate=None, gate_stride: int = 0, qk_norm_eps=None,
                               q_temperature=None, softcap: float = 0.0, gate_per_element: bool = False):
        """One new token per sequence (bfloat16 build), from the float32 q|k|v projection: rotates queries
        and the new key (``cos_sin`` table, or ``None`` for no rotation), writes the new key and value into
        the cache, attends over ``ctx_after[s]`` keys and merges ``splits`` (1..8) context pieces in-kernel.
        A row of ``qkv`` may be wider than its queries, keys and values.  Optional: float32 biases on the three,
        each value head divided by its root mean square (``value_norm_eps``), and ``bias``/``gate`` as in
        ``attention_prefill``; ``qk_norm_eps``: every query head and the new key head divided by its root mean square
        (head sizes that are powers of two); ``q_temperature`` ``(coef, every)``, ``softcap`` and ``gate_per_element`` as
        in ``qkv_finish`` and ``attention_prefill_tc``.  With ``write_kv`` false a row need hold its queries only."""
        self._want(qkv, torch.float32, "qkv"); self._want(out, self.dtype, "out")
        self._want(k_cache, self.dtype, "k_cache"); self._want(v_cache, self.dtype, "v_cache")
        self._want(block_table, torch.int32, "block_table"); self._want(ctx_after, torch.int32, "ctx_after")
        if cos_sin is not None:
            self._want(cos_sin, torch.float32, "cos_sin")
        n = qkv.shape[0]
        if qkv.shape[1] < (num_heads + (2 * num_kv_heads if write_kv else 0)) * head_dim:
            raise KernelError("attention_decode_fused: a row of qkv is shorter than its queries, keys and values")
        coef, every = q_temperature if q_temperature is not None else (0.0, 0)
        if ctx_after.numel() != n or block_table.shape[0] != n:
            raise KernelError("attention_decode_fused: one length and one table row per sequence is needed")
        for name, vector, width in (("q_bias", q_bias, num_heads * head_dim), ("k_bias", k_bias, num_kv_heads * head_dim),
                                    ("v_bias", v_bias, num_kv_heads * head_dim)):
            if vector is not None:
                self._want(vector, torch.float32, name)
                if vector.numel() != width:
                    raise KernelError(f"attention_decode_fused: {name} must hold {width} numbers")
        self._check(self.lib.skv_attention_decode_fused_extras(
            _ptr(qkv), qkv.shape[1], _ptr(cos_sin), _ptr(k_cache), _ptr(v_cache), _ptr(block_table), block_table.shape[1],
            _ptr(ctx_after), _ptr(out), n, num_heads, num_kv_heads, head_dim, block_size, ctypes.c_float(scale),
            window, splits, int(bool(write_kv)), _ptr(q_bias), _ptr(k_bias), _ptr(v_bias),
            int(value_norm_eps is not None), ctypes.c_float(value_norm_eps or 0.0),
            *self._extras(bias, gate, gate_stride, num_heads, "attention_decode_fused", head_dim if gate_per_element else 0),
            int(qk_norm_eps is not None), ctypes.c_float(qk_norm_eps or 0.0), ctypes.c_float(coef), int(every),
            ctypes.c_float(softcap), int(bool(gate_per_element)), _stream()), "attention_decode_fused")

    def embed_sum(self, table, ids, out, positions, token_seq, cu_q, slot_ids, flag=None, pair_table=None,
                  last_ids=None, mul_prev: int = 0, mul_cur: int = 0, position_table=None,
                  position_scale: float = 1.0, stats=None):
        """out[t, :] = table[ids[t]] + pair_table[bucket(previous id, ids[t])] + position_table[positions[t]] *
        position_scale, summed in float32; either of the two further tables may be None.  ``pair_table`` has one row
        per bucket and a last row for a sequence's first token; ``last_ids`` (int32, two per sequence slot: by the parity of the
        position) holds the last ids each sequence brought to its steps before and is brought up to date.
        ``stats``: as in ``embed`` (the first norm folded into the projection after it)."""
        self._want(table, self.dtype, "table"); self._want(ids, torch.int32, "ids")
        self._want(out, torch.float32, "out"); self._want(positions, torch.int32, "positions")
        self._want(token_seq, torch.int32, "token_seq"); self._want(cu_q, torch.int32, "cu_q")
        self._want(slot_ids, torch.int32, "slot_ids")
        n, hidden = out.shape
        n_seqs = slot_ids.numel()
        if table.shape[1] != hidden or ids.numel() != n or positions.numel() != n or cu_q.numel() != n_seqs + 1:
            raise KernelError("embed_sum: shapes do not agree")
        buckets = 0
        if pair_table is not None:
            self._want(pair_table, self.dtype, "pair_table"); self._want(last_ids, torch.int32, "last_ids")
            buckets = pair_table.shape[0] - 1
            if pair_table.shape[1] != hidden or buckets < 1:
                raise KernelError("embed_sum: the pair table must be [buckets + 1, hidden]")
        max_positions = 0
        if position_table is not None:
            self._want(position_table, self.dtype, "position_table")
            max_positions = position_table.shape[0]
            if position_table.shape[1] != hidden:
                raise KernelError("embed_sum: the position table must be [positions, hidden]")
        fold = self._fold_target(stats, n, hidden)
        self._check(self.lib.skv_embed_sum(
            _ptr(table), _ptr(pair_table), _ptr(position_table), _ptr(ids), _ptr(positions), _ptr(token_seq), _ptr(cu_q),
            _ptr(slot_ids), _ptr(last_ids), _ptr(out), n, n_seqs, hidden, table.shape[0], buckets,
            ctypes.c_longlong(mul_prev), ctypes.c_longlong(mul_cur), max_positions, ctypes.c_float(position_scale),
            _ptr(flag), *(fold[:6] if fold else _NO_FOLD[:6]), _stream()), "embed_sum")
        if pair_table is not None:
            Kernels.launches += 1              # (the second launch that remembers the last ids)
        if stats is not None:
            stats.filled(1 if stats.consumer_sums else 0) if fold else stats.invalidate()

    def qkv_finish(self, qkv, q_out, k_cache, v_cache, positions, token_seq, block_table, num_heads: int,
                   num_kv_heads: int, dim: int, vdim: int, block_size: int, q_bias=None, k_bias=None, v_bias=None,
                   value_norm_eps=None, write_kv: bool = True, q_norm: bool = False, k_norm: bool = False,
                   qk_norm_eps: float = 0.0, k_norm_weight=None, q_temperature=None, key_dim: int = 0):
        """From float32 rows ``[q | k | v | ...]`` of a fused projection: biases added, each value head divided by
        its root mean square (``value_norm_eps`` not None), queries to ``q_out`` and keys and values to the cache
        in the compute dtype.  Any head sizes; keys ``dim`` and values ``vdim`` wide.

        ``q_norm`` / ``k_norm``: every query / key head divided by its root mean square (``qk_norm_eps``), the keys
        then times ``k_norm_weight`` (float32 ``[kv_heads * dim]``) if given.  ``q_temperature`` ``(coef, every)``:
        the queries at position p times ``1 + coef * ln(floor((p + 1) / every) + 1)``.  ``vdim`` 0 with ``v_cache``
        None: the rows hold no values.  With ``write_kv`` false a row need hold its queries only.  ``key_dim``: the
        width of a key head where it is not a query head's (a compressed latent that is cached as the one key)."""
        key_dim = key_dim or dim
        self._want(qkv, torch.float32, "qkv")
        if num_heads > 0:
            self._want(q_out, self.dtype, "q_out")
        self._want(positions, torch.int32, "positions"); self._want(token_seq, torch.int32, "token_seq")
        self._want(block_table, torch.int32, "block_table")
        self._want(k_cache, self.dtype, "k_cache")
        if v_cache is not None:
            self._want(v_cache, self.dtype, "v_cache")
        for name, bias, width in (("q_bias", q_bias, num_heads * dim), ("k_bias", k_bias, num_kv_heads * (key_dim or dim)),
                                  ("v_bias", v_bias, num_kv_heads * vdim)):
            if bias is not None:
                self._want(bias, torch.float32, name)
                if bias.numel() != width:
                    raise KernelError(f"qkv_finish: {name} must hold {width} numbers")
        n = qkv.shape[0]
        if ((num_heads > 0 and tuple(q_out.shape) != (n, num_heads * dim)) or positions.numel() != n
                or token_seq.numel() != n):
            raise KernelError("qkv_finish: one query row, one position and one sequence index per token is needed")
        if (tuple(k_cache.shape[1:]) != (num_kv_heads, block_size, key_dim)
                or (v_cache is not None and tuple(v_cache.shape[1:]) != (num_kv_heads, block_size, vdim))):
            raise KernelError("qkv_finish: the cache must be [blocks, kv_heads, block_size, dim] and [.., vdim]")
        if (v_cache is None) != (vdim == 0):
            raise KernelError("qkv_finish: rows without values have vdim 0 and no value cache")
        if k_norm_weight is not None:
            self._want(k_norm_weight, torch.float32, "k_norm_weight")
            if k_norm_weight.numel() != num_kv_heads * key_dim:
                raise KernelError("qkv_finish: the keys' norm weight must hold kv_heads * dim numbers")
        coef, every = q_temperature if q_temperature is not None else (0.0, 0)
        self._check(self.lib.skv_qkv_finish(
            _ptr(qkv), qkv.shape[1], _ptr(q_bias), _ptr(k_bias), _ptr(v_bias), _ptr(positions), _ptr(token_seq),
            _ptr(block_table), block_table.shape[1], _ptr(q_out), _ptr(k_cache), _ptr(v_cache), n, num_heads,
            num_kv_heads, dim, vdim, block_size, int(value_norm_eps is not None),
            ctypes.c_float(value_norm_eps or 0.0), int(bool(write_kv)), int(bool(q_norm)), int(bool(k_norm)),
            ctypes.c_float(qk_norm_eps), _ptr(k_norm_weight), ctypes.c_float(coef), int(every), int(key_dim),
            _stream()), "qkv_finish")

    def attention_general(self, q, k_cache, v_cache, block_table, positions, token_seq, out, num_heads: int,
                          num_kv_heads: int, dim: int, vdim: int, block_size: int, scale: float, window: int = 0,
                          r1=None, r2=None, gate=None, gate_stride: int = 0, softcap: float = 0.0,
                          gate_per_element: bool = False, sink=None, value_stride: int = 0, splits: int = 1,
                          scratch_o=None, scratch_ml=None):
        """(``splits`` > 1: every (token, head)'s keys are cut into that many parts that run side by side, for steps of
        few tokens over long contexts; ``scratch_o`` float32 ``[tokens * heads * splits * vdim]`` and ``scratch_ml``
        ``[tokens * heads * splits * 2]`` hold the parts for the merge that follows.)
        (``sink``, float32 per head: ``exp(sink[h])`` counts once in the softmax's denominator, with no value.
        ``value_stride``: the values' rows are that many numbers apart where they are not ``vdim`` wide, so that the
        first ``vdim`` numbers of the cached keys can serve as the values.)
        (``softcap`` c > 0: scores become ``c * tanh(score / c)``.  ``gate_per_element``: the gate holds a logit for
        every output number, token t, head h, number d at ``[t * gate_stride + h * vdim + d]``.)
        Attention with run-time head sizes (keys ``dim``, values ``vdim``), a warp per (token, head), float math.
        ``r1``, ``r2`` (float32 per head): ``r1 * ln(1 + r2 * distance)`` is taken off each score.  ``gate``
        (float32, the logit of token t and head h at ``[t * gate_stride + h]``): the head's output times its sigmoid.
        ``out`` may be wider than ``heads * vdim``; the further columns are set to zero."""
        self._want(q, self.dtype, "q"); self._want(out, self.dtype, "out")
        self._want(k_cache, self.dtype, "k_cache"); self._want(v_cache, self.dtype, "v_cache")
        self._want(block_table, torch.int32, "block_table")
        self._want(positions, torch.int32, "positions"); self._want(token_seq, torch.int32, "token_seq")
        value_stride = value_stride or vdim
        if value_stride < vdim:
            raise KernelError("attention_general: the values' rows cannot be closer together than they are wide")
        if sink is not None:
            self._want(sink, torch.float32, "sink")
            if sink.numel() != num_heads:
                raise KernelError("attention_general: the sink must hold one number per head")
        for name, value in (("r1", r1), ("r2", r2)):
            if value is not None:
                self._want(value, torch.float32, name)
                if value.numel() != num_heads:
                    raise KernelError(f"attention_general: {name} must hold one number per head")
        if gate is not None and (gate.dtype != torch.float32 or not gate.is_cuda or gate.stride(-1) != 1
                                 or gate_stride < num_heads * (vdim if gate_per_element else 1)):
            raise KernelError("attention_general: the gate must be float32 on the GPU, a row at least heads wide")
        n = q.shape[0]
        if tuple(q.shape) != (n, num_heads * dim) or out.shape[0] != n or out.shape[1] < num_heads * vdim:
            raise KernelError("attention_general: q must be [tokens, heads * dim] and out [tokens, heads * vdim or wider]")
        if splits > 1:
            self._want(scratch_o, torch.float32, "scratch_o"); self._want(scratch_ml, torch.float32, "scratch_ml")
            if scratch_o.numel() < n * num_heads * splits * vdim or scratch_ml.numel() < n * num_heads * splits * 2:
                raise KernelError("attention_general: the scratch for the parts is too small")
        self._check(self.lib.skv_attention_general(
            _ptr(q), _ptr(k_cache), _ptr(v_cache), _ptr(block_table), block_table.shape[1], _ptr(positions),
            _ptr(token_seq), _ptr(out), n, num_heads, num_kv_heads, dim, vdim, block_size, ctypes.c_float(scale),
            window, _ptr(r1), _ptr(r2), _ptr(gate), gate_stride, out.shape[1], ctypes.c_float(softcap),
            int(bool(gate_per_element)), _ptr(sink), int(value_stride), int(splits),
            _ptr(scratch_o if splits > 1 else None), _ptr(scratch_ml if splits > 1 else None), _stream()),
            "attention_general")

    def paged_gather(self, cache, block_table, positions, seqs, out):
        """``out[i, :]`` = the row that a one-head paged cache (``[blocks, 1, block_size, width]``) holds for position
        ``positions[i]`` of sequence ``seqs[i]`` (a row of ``block_table``)."""
        self._want(cache, self.dtype, "cache"); self._want(out, self.dtype, "out")
        self._want(block_table, torch.int32, "block_table"); self._want(positions, torch.int32, "positions")
        self._want(seqs, torch.int32, "seqs")
        n, width = out.shape
        if cache.dim() != 4 or cache.shape[1] != 1 or cache.shape[3] != width or positions.numel() != n or seqs.numel() != n:
            raise KernelError("paged_gather: shapes do not agree")
        self._check(self.lib.skv_paged_gather(_ptr(cache), _ptr(block_table), block_table.shape[1], _ptr(positions),
                                              _ptr(seqs), _ptr(out), n, width, cache.shape[2], _stream()), "paged_gather")

    def rmsnorm_add(self, y, gamma, eps: float, x, next_gamma=None, next_eps: float = 0.0, next_out=None):
        """x += rmsnorm(y) * gamma on float32 rows (the norm after a sublayer); with ``next_gamma`` and ``next_out``
        (compute dtype) also ``next_out = rmsnorm(new x) * next_gamma``, the input of the sublayer after it."""
        self._want(y, torch.float32, "y"); self._want(x, torch.float32, "x"); self._want(gamma, torch.float32, "gamma")
        n, hidden = x.shape
        if tuple(y.shape) != (n, hidden) or gamma.numel() != hidden:
            raise KernelError("rmsnorm_add: shapes do not agree")
        if next_out is not None:
            self._want(next_out, self.dtype, "next_out"); self._want(next_gamma, torch.float32, "next_gamma")
            if tuple(next_out.shape) != (n, hidden) or next_gamma.numel() != hidden:
                raise KernelError("rmsnorm_add: the next norm's shapes do not agree")
        self._check(self.lib.skv_rmsnorm_add(_ptr(y), _ptr(gamma), ctypes.c_float(eps), _ptr(x), _ptr(next_gamma),
                                             ctypes.c_float(next_eps), _ptr(next_out), n, hidden, _stream()), "rmsnorm_add")

    def token_side(self, x, ids, table, offset: int, dim: int, gate_w, proj_t, norm_w, eps: float, next_gamma=None,
                   next_eps: float = 0.0, next_out=None, branch=None, post_gamma=None, post_eps: float = 0.0):
        """An input that depends on the token, added to the float32 stream: ``e = table[id, offset:offset + dim]``,
        ``g = gelu_tanh(gate_w . x) * e``, ``y = proj_t^T . g`` (``proj_t`` is the projection transposed,
        ``[dim, hidden]``), ``x += rmsnorm(y) * norm_w``; ``next_*`` as in ``rmsnorm_add``.  With ``branch`` (float32
        ``[tokens, hidden]``) and ``post_gamma``, ``x += rmsnorm(branch) * post_gamma`` (eps ``post_eps``) comes first: the
        sublayer in front of the token input is added in the same pass."""
        self._want(x, torch.float32, "x"); self._want(ids, torch.int32, "ids"); self._want(table, self.dtype, "table")
        self._want(gate_w, self.dtype, "gate_w"); self._want(proj_t, self.dtype, "proj_t")
        self._want(norm_w, torch.float32, "norm_w")
        n, hidden = x.shape
        if (ids.numel() != n or tuple(gate_w.shape) != (dim, hidden) or tuple(proj_t.shape) != (dim, hidden)
                or norm_w.numel() != hidden or table.dim() != 2):
            raise KernelError("token_side: shapes do not agree")
        if next_out is not None:
            self._want(next_out, self.dtype, "next_out"); self._want(next_gamma, torch.float32, "next_gamma")
            if tuple(next_out.shape) != (n, hidden) or next_gamma.numel() != hidden:
                raise KernelError("token_side: the next norm's shapes do not agree")
        if branch is not None:
            self._want(branch, torch.float32, "branch"); self._want(post_gamma, torch.float32, "post_gamma")
            if tuple(branch.shape) != (n, hidden) or post_gamma.numel() != hidden:
                raise KernelError("token_side: the branch's shapes do not agree")
        self._check(self.lib.skv_token_side(
            _ptr(x), _ptr(ids), _ptr(table), table.shape[1], int(offset), int(dim), table.shape[0], _ptr(gate_w),
            _ptr(proj_t), _ptr(norm_w), ctypes.c_float(eps), _ptr(next_gamma), ctypes.c_float(next_eps), _ptr(next_out),
            n, hidden, _ptr(branch), _ptr(post_gamma), ctypes.c_float(post_eps), _stream()), "token_side")

    def headwise_linear(self, x, w, out, heads: int, zero_pad: bool = False, out_head_stride: int = 0):
        """``out[t, h, :] = w[h] . x[t, h, :]`` with ``w`` ``[heads, out_dim, in_dim]`` in the compute dtype; ``x`` and
        ``out`` are 2-D, float32 or the compute dtype, head h at columns ``h * in_dim`` and ``h * out_dim`` (rows may be
        wider; ``zero_pad`` sets what lies beyond an out row's heads to zero).  Sums are float32.  ``out_head_stride``: head h
        of ``out`` starts at ``h * out_head_stride`` instead (what lies between the heads' results is left alone)."""
        self._want(w, self.dtype, "w")
        for name, tensor in (("x", x), ("out", out)):
            if not tensor.is_cuda or tensor.dtype not in (torch.float32, self.dtype) or tensor.dim() != 2 \
                    or tensor.stride(1) != 1:
                raise KernelError(f"headwise_linear: {name} must be a 2-D CUDA tensor, float32 or the compute dtype")
        if w.dim() != 3 or w.shape[0] != heads:
            raise KernelError("headwise_linear: the weight must be [heads, out_dim, in_dim]")
        out_dim, in_dim = w.shape[1], w.shape[2]
        n = x.shape[0]
        out_head_stride = out_head_stride or out_dim
        if (out.shape[0] != n or x.shape[1] < heads * in_dim or out_head_stride < out_dim
                or out.shape[1] < (heads - 1) * out_head_stride + out_dim):
            raise KernelError("headwise_linear: a row is shorter than its heads")
        if zero_pad and out_head_stride != out_dim:
            raise KernelError("headwise_linear: zero_pad goes with heads that lie side by side")
        self._check(self.lib.skv_headwise_linear(
            _ptr(x), int(x.dtype == torch.float32), x.stride(0), _ptr(w), _ptr(out), int(out.dtype == torch.float32),
            out.stride(0), n, heads, in_dim, out_dim, int(bool(zero_pad)), int(out_head_stride), _stream()),
            "headwise_linear")

    def _recurrent_batch(self, step_meta, state, channels: int, taps: int, name: str):
        positions, token_seq, cu_q, slot_ids = step_meta
        for label, tensor in (("positions", positions), ("token_seq", token_seq), ("cu_q", cu_q), ("slot_ids", slot_ids)):
            self._want(tensor, torch.int32, label)
        self._want(state, torch.float32, "state")
        if state.dim() != 2 or state.shape[1] < (2 + taps) * channels or cu_q.numel() != slot_ids.numel() + 1:
            raise KernelError(f"{name}: the state must be [slots, (2 + taps) * channels or wider] float32")
        return (_ptr(positions), _ptr(token_seq), _ptr(cu_q), _ptr(slot_ids), _ptr(state), state.shape[1])

    def rglru_conv(self, yx, x_offset: int, x_bias, conv_w, conv_b, u, step_meta, state):
        """The recurrent branch's causal convolution per channel: ``u[t] = conv_b + sum_k conv_w[:, k] * xb[t - (taps-1-k)]``
        with ``xb = yx[:, x_offset:x_offset + C] + x_bias``; inputs before this step come from ``state`` (float32
        ``[slots, (2 + taps) * C]``), positions before a sequence's start are zero.  ``step_meta``: the step's
        ``(positions, token_seq, cu_q, slot_ids)``."""
        self._want(yx, torch.float32, "yx"); self._want(u, torch.float32, "u")
        for label, tensor in (("x_bias", x_bias), ("conv_w", conv_w), ("conv_b", conv_b)):
            self._want(tensor, torch.float32, label)
        n, channels = u.shape
        taps = conv_w.shape[1]
        if yx.shape[0] != n or tuple(conv_w.shape) != (channels, taps) or x_bias.numel() != channels or conv_b.numel() != channels:
            raise KernelError("rglru_conv: shapes do not agree")
        self._check(self.lib.skv_rglru_conv(
            _ptr(yx), yx.shape[1], int(x_offset), _ptr(x_bias), _ptr(conv_w), _ptr(conv_b), _ptr(u), n, channels, taps,
            *self._recurrent_batch(step_meta, state, channels, taps, "rglru_conv"), _stream()), "rglru_conv")

    def rglru_rate(self, lam, rate):
        """``rate = 8 * softplus(lam)`` (float32, per channel): the token-independent part of the decay's exponent."""
        self._want(lam, torch.float32, "lam"); self._want(rate, torch.float32, "rate")
        if lam.numel() != rate.numel():
            raise KernelError("rglru_rate: sizes differ")
        self._check(self.lib.skv_rglru_rate(_ptr(lam), _ptr(rate), lam.numel(), _stream()), "rglru_rate")
        return rate

    def rglru_gates(self, gates, u, yx, y_bias, r_bias, i_bias, rate, part: int):
        """In place: ``gates`` (float32 ``[tokens, 2C]``, per part of ``part`` channels its r rows then its i rows, as
        ``headwise_linear`` leaves them) becomes the decay ``a = exp(-sigmoid(r + r_bias) rate)`` (``rate`` from
        ``rglru_rate``) and the driven input ``sqrt(1 - a^2) sigmoid(i + i_bias) u``; ``yx[:, :C]`` becomes
        ``gelu_tanh(yx[:, :C] + y_bias)``."""
        self._want(gates, torch.float32, "gates"); self._want(u, torch.float32, "u"); self._want(yx, torch.float32, "yx")
        for label, tensor in (("y_bias", y_bias), ("r_bias", r_bias), ("i_bias", i_bias), ("rate", rate)):
            self._want(tensor, torch.float32, label)
        n, channels = u.shape
        if tuple(gates.shape) != (n, 2 * channels) or yx.shape[0] != n or any(
                t.numel() != channels for t in (y_bias, r_bias, i_bias, rate)):
            raise KernelError("rglru_gates: shapes do not agree")
        self._check(self.lib.skv_rglru_gates(_ptr(gates), _ptr(u), _ptr(yx), yx.shape[1], _ptr(y_bias), _ptr(r_bias),
                                             _ptr(i_bias), _ptr(rate), n, channels, int(part), _stream()), "rglru_gates")

    def rglru_scan_scratch(self, n_seqs: int, max_q_len: int, channels: int) -> int:
        """Floats of scratch ``rglru_scan`` needs for a step whose longest sequence brings ``max_q_len`` tokens."""
        self.lib.skv_rglru_scan_scratch.restype = ctypes.c_longlong
        return int(self.lib.skv_rglru_scan_scratch(int(n_seqs), int(max_q_len), int(channels)))

    def rglru_scan(self, gates, yx, x_offset: int, x_bias, out, part: int, taps: int, step_meta, state,
                   max_q_len: int, summary=None):
        """``S_t = a_t S_(t-1) + driven_t`` along each sequence's tokens of this step, from and to ``state``;
        ``out[t, :C] = S_t * yx[t, :C]`` in the compute dtype; the convolution's last inputs go to ``state`` too.
        ``max_q_len``: the most tokens one sequence brings; long steps are walked in chunks side by side and need
        ``summary``, float32 scratch of ``rglru_scan_scratch`` numbers."""
        self._want(gates, torch.float32, "gates"); self._want(yx, torch.float32, "yx")
        self._want(out, self.dtype, "out"); self._want(x_bias, torch.float32, "x_bias")
        n, channels = gates.shape[0], gates.shape[1] // 2
        n_seqs = step_meta[3].numel()
        if yx.shape[0] != n or out.shape[0] != n or out.shape[1] < channels or x_bias.numel() != channels:
            raise KernelError("rglru_scan: shapes do not agree")
        if summary is not None:
            self._want(summary, torch.float32, "summary")
            if summary.numel() < self.rglru_scan_scratch(n_seqs, max_q_len, channels):
                raise KernelError("rglru_scan: the scratch for the chunks is too small")
        self._check(self.lib.skv_rglru_scan(
            _ptr(gates), _ptr(yx), yx.shape[1], int(x_offset), _ptr(x_bias), _ptr(out), out.shape[1], n_seqs, channels,
            int(part), int(taps), int(max_q_len), _ptr(summary),
            *self._recurrent_batch(step_meta, state, channels, taps, "rglru_scan"), _stream()), "rglru_scan")
        if summary is not None and self.rglru_scan_scratch(n_seqs, max_q_len, channels) > 0:
            Kernels.launches += 1              # (the pass that sums up the chunks)

    # ---- several copies of the residual stream ---------------------------------------
    def stream_mix(self, streams, count: int, source=None, branch=None, mix=None, write=None, read=None, gamma=None,
                   eps: float = 0.0, normed_out=None, sum_out=None):
        """One pass over ``count`` copies of the residual stream (float32 ``[count, tokens, hidden]``).  The old
        streams are ``streams``, or all equal to ``source`` (float32 ``[tokens, hidden]``) where they have not been
        written yet.  With ``branch`` (a sublayer's result), ``mix`` ``[from * count + to]`` and ``write``: every stream
        becomes ``sum_s mix[s, t] x_s + write[t] * branch`` and is written.  With ``read``, ``gamma`` and ``normed_out``
        (compute dtype): ``u = sum_t read[t] x_t`` of the (new) streams, ``normed_out = u / sqrt(mean(u^2) + eps) * gamma``.
        With ``sum_out``: the sum of the (new) streams."""
        self._want(streams, torch.float32, "streams")
        if streams.dim() != 3 or streams.shape[0] != count or not 1 <= count <= MAX_STREAMS:
            raise KernelError(f"stream_mix: the streams must be [count, tokens, hidden] with 1 to {MAX_STREAMS} copies")
        n, hidden = streams.shape[1], streams.shape[2]
        for name, tensor in (("source", source), ("branch", branch), ("sum_out", sum_out)):
            if tensor is not None:
                self._want(tensor, torch.float32, name)
                if tuple(tensor.shape) != (n, hidden):
                    raise KernelError(f"stream_mix: {name} must be [tokens, hidden]")
        if (branch is None) != (mix is None) or (branch is None) != (write is None):
            raise KernelError("stream_mix: an update needs the sublayer's result, the mixing matrix and the write weights")
        if branch is None and source is not None and normed_out is None and sum_out is None:
            raise KernelError("stream_mix: nothing to do")
        for name, tensor, size in (("mix", mix, count * count), ("write", write, count), ("read", read, count),
                                   ("gamma", gamma, hidden)):
            if tensor is not None:
                self._want(tensor, torch.float32, name)
                if tensor.numel() != size:
                    raise KernelError(f"stream_mix: {name} must hold {size} numbers")
        if (normed_out is None) != (read is None) or (normed_out is None) != (gamma is None):
            raise KernelError("stream_mix: a reading needs the read weights, the norm's weight and a place for the result")
        if normed_out is not None:
            self._want(normed_out, self.dtype, "normed_out")
            if tuple(normed_out.shape) != (n, hidden):
                raise KernelError("stream_mix: normed_out must be [tokens, hidden]")
        self._check(self.lib.skv_stream_mix(
            _ptr(streams), int(count), _ptr(source), _ptr(branch), _ptr(mix), _ptr(write), _ptr(read), _ptr(gamma),
            ctypes.c_float(eps), _ptr(normed_out), _ptr(sum_out), n, hidden, _stream()), "stream_mix")

    # ---- retention ----------------------------------------------------------------------
    def retention_scratch(self, n_seqs: int, max_q_len: int, heads: int, dim: int, vdim: int) -> int:
        """Floats of scratch ``retention`` needs for a step whose longest sequence brings ``max_q_len`` tokens."""
        self.lib.skv_retention_scratch.restype = ctypes.c_longlong
        return int(self.lib.skv_retention_scratch(int(n_seqs), int(max_q_len), int(heads), int(dim), int(vdim)))

    def retention(self, fused, cos_sin, rotated: int, decay, eps: float, out, state, step_meta, heads: int, dim: int,
                  vdim: int, max_q_len: int, scratch=None):
        """Retention over a packed step.  ``fused`` (float32 rows ``[q | k | v | gate]``: ``heads * dim`` twice, then
        ``heads * vdim`` twice; queries and keys are rotated in place): per head ``S <- decay S + k v^T`` with
        ``k = rot(k) * dim^-1/2`` from and to ``state`` (float32 ``[slots, 2 * heads * dim * vdim]``: S in the half of
        the last written position's parity), ``o = S^T rot(q)``, ``out = o / rms(o) * silu(gate)`` per head in the
        compute dtype (columns beyond the heads are set to zero).  ``cos_sin``: ``[positions, rotated / 2, 2]`` or None.
        ``step_meta``: the step's ``(positions, token_seq, cu_q, slot_ids)``; ``scratch``: ``retention_scratch`` floats."""
        self._want(fused, torch.float32, "fused"); self._want(decay, torch.float32, "decay")
        self._want(out, self.dtype, "out"); self._want(state, torch.float32, "state")
        positions, token_seq, cu_q, slot_ids = step_meta
        for label, tensor in (("positions", positions), ("token_seq", token_seq), ("cu_q", cu_q), ("slot_ids", slot_ids)):
            self._want(tensor, torch.int32, label)
        n, n_seqs = fused.shape[0], slot_ids.numel()
        if (fused.shape[1] < 2 * heads * (dim + vdim) or out.shape[0] != n or out.shape[1] < heads * vdim
                or decay.numel() != heads or positions.numel() != n or cu_q.numel() != n_seqs + 1):
            raise KernelError("retention: shapes do not agree")
        if state.dim() != 2 or state.shape[1] < 2 * heads * dim * vdim:
            raise KernelError("retention: the state must be [slots, 2 * heads * dim * vdim or wider] float32")
        if cos_sin is not None:
            self._want(cos_sin, torch.float32, "cos_sin")
            if rotated <= 0 or rotated % 2 or rotated > dim or tuple(cos_sin.shape[1:]) != (rotated // 2, 2):
                raise KernelError("retention: the rotation's table must be [positions, rotated / 2, 2]")
        need = self.retention_scratch(n_seqs, max_q_len, heads, dim, vdim)
        if need:
            self._want(scratch, torch.float32, "scratch")
            if scratch.numel() < need:
                raise KernelError("retention: the scratch for the chunks is too small")
        self._check(self.lib.skv_retention(
            _ptr(fused), fused.shape[1], _ptr(cos_sin), int(rotated if cos_sin is not None else 0),
            cos_sin.shape[0] if cos_sin is not None else 0, _ptr(decay), ctypes.c_float(eps), _ptr(out), out.shape[1],
            _ptr(scratch), n, n_seqs, heads, dim, vdim, int(max_q_len), _ptr(positions), _ptr(token_seq), _ptr(cu_q),
            _ptr(slot_ids), _ptr(state), state.shape[1], _stream()), "retention")

    # ---- latent attention with a rotated part ---------------------------------------------
    def latent_finish(self, fused, q_plain, q_folded, cache, positions, token_seq, block_table, heads: int, dim: int,
                      rope_dim: int, latent_dim: int, block_size: int, rotation=None, rotated: int = 0,
                      latent_offset: int = 0, latent_gamma=None, eps: float = 0.0, write_cache: bool = True,
                      q_whole=None):
        """From float32 rows of a fused projection ``[queries: heads x (dim | rope_dim) | latent_dim + rope_dim | ...]``:
        the unrotated query parts to ``q_plain`` ``[tokens, heads * dim]``, the rotated ones (first ``rotated`` numbers
        turned by ``rotation`` ``[positions, rotated / 2, 2]``) to the last ``rope_dim`` columns of every head of
        ``q_folded`` ``[tokens, heads * (latent_dim + rope_dim)]``; with ``write_cache`` the latent, divided by its root
        mean square and times ``latent_gamma``, and the rotated key part behind it go to the token's row of ``cache``
        ``[blocks, 1, block_size, latent_dim + rope_dim]``.  With ``q_whole`` ``[tokens, heads * (dim + rope_dim)]`` both
        query parts go there instead, head by head, and ``q_plain`` and ``q_folded`` may be None."""
        self._want(fused, torch.float32, "fused"); self._want(cache, self.dtype, "cache")
        n, key_dim = fused.shape[0], latent_dim + rope_dim
        if q_whole is not None:
            self._want(q_whole, self.dtype, "q_whole")
            if tuple(q_whole.shape) != (n, heads * (dim + rope_dim)):
                raise KernelError("latent_finish: q_whole must be [tokens, heads * (dim + rope_dim)]")
        else:
            self._want(q_plain, self.dtype, "q_plain"); self._want(q_folded, self.dtype, "q_folded")
            if tuple(q_plain.shape) != (n, heads * dim) or tuple(q_folded.shape) != (n, heads * key_dim):
                raise KernelError("latent_finish: shapes do not agree")
        self._want(positions, torch.int32, "positions"); self._want(token_seq, torch.int32, "token_seq")
        self._want(block_table, torch.int32, "block_table")
        if (tuple(cache.shape[1:]) != (1, block_size, key_dim) or positions.numel() != n or token_seq.numel() != n):
            raise KernelError("latent_finish: shapes do not agree")
        if fused.shape[1] < heads * (dim + rope_dim) + (key_dim if write_cache else 0) or (write_cache and latent_offset < heads * (dim + rope_dim)):
            raise KernelError("latent_finish: a row is shorter than its queries, latent and key part")
        if rotation is not None:
            self._want(rotation, torch.float32, "rotation")
            if rotated <= 0 or rotated % 2 or rotated > rope_dim or tuple(rotation.shape[1:]) != (rotated // 2, 2):
                raise KernelError("latent_finish: the rotation's table must be [positions, rotated / 2, 2]")
        if write_cache:
            self._want(latent_gamma, torch.float32, "latent_gamma")
            if latent_gamma.numel() != latent_dim:
                raise KernelError("latent_finish: the latent's norm weight must hold latent_dim numbers")
        self._check(self.lib.skv_latent_finish(
            _ptr(fused), fused.shape[1], _ptr(q_plain), _ptr(q_folded), _ptr(q_whole), _ptr(cache), _ptr(positions), _ptr(token_seq),
            _ptr(block_table), block_table.shape[1], n, heads, dim, rope_dim, latent_dim, block_size, _ptr(rotation),
            int(rotated if rotation is not None else 0), rotation.shape[0] if rotation is not None else 0,
            int(latent_offset), _ptr(latent_gamma), ctypes.c_float(eps), int(bool(write_cache)), _stream()), "latent_finish")

    # ---- routed feed-forward ------------------------------------------------------------------
    def route_tokens(self, h, router_w, correction, top: int, scale: float, renormalize: bool, chosen, weights,
                     shared_gate_weight=None, shared_gate_out=None, softmax: bool = False, groups: int = 0,
                     keep: int = 0, renorm_eps: float = 0.0):
        """(``softmax``: the scores are a softmax over all experts instead of sigmoids.  ``groups`` > 1: the experts form
        that many equal groups of neighbours, a group scores what its best expert does and only experts of the ``keep``
        best groups can be chosen.  ``renorm_eps`` is added to the chosen scores' sum before ``renormalize`` divides.)
        Per token: ``s = sigmoid(router_w . h)`` (float32 sums); the ``top`` experts with the largest
        ``s + correction`` (the lower index among equals) into ``chosen`` (int32 ``[tokens, top]``), their ``s * scale``
        into ``weights`` (``renormalize``: divided by the chosen scores' sum first).  With ``shared_gate_weight``
        ``[hidden]``: ``shared_gate_out[t] = sigmoid(shared_gate_weight . h[t])``."""
        self._want(h, self.dtype, "h"); self._want(router_w, self.dtype, "router_w")
        self._want(chosen, torch.int32, "chosen"); self._want(weights, torch.float32, "weights")
        n, hidden = h.shape
        experts = router_w.shape[0]
        if (router_w.shape[1] != hidden or tuple(chosen.shape) != (n, top) or tuple(weights.shape) != (n, top)
                or not 0 < top <= min(experts, MAX_EXPERTS_PER_TOKEN) or experts > MAX_EXPERTS):
            raise KernelError("route_tokens: shapes do not agree")
        if correction is not None:
            self._want(correction, torch.float32, "correction")
            if correction.numel() != experts:
                raise KernelError("route_tokens: one correction per expert is needed")
        if (shared_gate_weight is None) != (shared_gate_out is None):
            raise KernelError("route_tokens: the shared expert's gate needs its weight and a place for the result")
        if shared_gate_weight is not None:
            self._want(shared_gate_weight, self.dtype, "shared_gate_weight"); self._want(shared_gate_out, torch.float32, "shared_gate_out")
            if shared_gate_weight.numel() != hidden or shared_gate_out.numel() != n:
                raise KernelError("route_tokens: the shared expert's gate has the wrong size")
        if groups > 1 and (experts % groups or not 0 < keep <= groups or keep * (experts // groups) < top):
            raise KernelError("route_tokens: groups must divide the experts and the kept groups hold the choices")
        self._check(self.lib.skv_route_tokens(
            _ptr(h), _ptr(router_w), _ptr(correction), _ptr(shared_gate_weight), n, hidden, experts, int(top),
            ctypes.c_float(scale), int(bool(renormalize)), _ptr(chosen), _ptr(weights), _ptr(shared_gate_out),
            int(bool(softmax)), int(groups), int(keep), ctypes.c_float(renorm_eps), _stream()), "route_tokens")

    def sort_by_expert(self, chosen, experts: int, offsets, order, place):
        """A counting sort of the (token, choice) pairs by expert: ``offsets`` (int32 ``[experts + 1]``) bounds each
        expert's pairs in the sorted order, ``order[p]`` is the token of sorted pair p, ``place[t, k]`` where pair
        (t, k) went."""
        for name, tensor in (("chosen", chosen), ("offsets", offsets), ("order", order), ("place", place)):
            self._want(tensor, torch.int32, name)
        n, top = chosen.shape
        if offsets.numel() != experts + 1 or order.numel() != n * top or tuple(place.shape) != (n, top) or experts > MAX_EXPERTS:
            raise KernelError("sort_by_expert: shapes do not agree")
        self._check(self.lib.skv_sort_by_expert(_ptr(chosen), n * top, int(top), int(experts), _ptr(offsets), _ptr(order),
                                                _ptr(place), _stream()), "sort_by_expert")

    def gather_rows(self, a, rows, out):
        """``out[p] = a[rows[p]]`` (compute dtype, rows of whole 16 bytes)."""
        self._want(a, self.dtype, "a"); self._want(out, self.dtype, "out"); self._want(rows, torch.int32, "rows")
        if out.shape[0] != rows.numel() or out.shape[1] != a.shape[1]:
            raise KernelError("gather_rows: shapes do not agree")
        self._check(self.lib.skv_gather_rows(_ptr(a), a.stride(0), _ptr(rows), _ptr(out), out.shape[0], out.shape[1],
                                             _stream()), "gather_rows")

    def expert_rows_sorted_first(self, hidden: int) -> bool:
        """True if ``expert_linear`` is faster on rows that lie in sorted order (``gather_rows`` first): the bfloat16
        build's tensor-core form wants neighbouring rows of whole 16 bytes."""
        return self.dtype == torch.bfloat16 and hidden % 8 == 0

    def expert_linear(self, a, w, offsets, out, rows=None, activation: Optional[str] = None, flag=None,
                      gated: bool = False):
        """(``gated``: ``w`` is ``[experts, 2 N, K]`` in tiles of 8 gate rows and their 8 up rows, as ``pack_gate_up``
        lays them out, and ``out[p] = act(gate_e . a) * (up_e . a)``.)
        ``out[p] = act(w[e] . a[row(p)])`` for every sorted pair p of expert e (``offsets`` from ``sort_by_expert``);
        ``w`` ``[experts, N, K]``; ``row(p) = rows[p]`` (the first projection gathers its input from the tokens) or p.
        ``out`` ``[pairs, N]`` is the compute dtype (with ``activation``) or float32.  Sums are float32."""
        self._want(a, self.dtype, "a"); self._want(w, self.dtype, "w"); self._want(offsets, torch.int32, "offsets")
        if out.dtype not in (self.dtype, torch.float32) or not out.is_cuda or not out.is_contiguous():
            raise KernelError("expert_linear: out must be a contiguous CUDA tensor, float32 or the compute dtype")
        pairs = out.shape[0]
        experts, N, K = w.shape
        if gated:
            if N % 16 or activation is None:
                raise KernelError("expert_linear: a gated weight has whole tiles of 16 rows and an activation")
            N //= 2
        if a.shape[1] != K or out.shape[1] != N or offsets.numel() != experts + 1 or (rows is None and a.shape[0] != pairs):
            raise KernelError("expert_linear: shapes do not agree")
        if rows is not None:
            self._want(rows, torch.int32, "rows")
            if rows.numel() != pairs:
                raise KernelError("expert_linear: one row index per pair is needed")
        if activation is not None and (activation not in ACTIVATIONS or activation in PARAMETRIC_ACTIVATIONS):
            raise KernelError(f"expert_linear: activation '{activation}' is not supported")
        self._check(self.lib.skv_expert_linear(
            _ptr(a), a.stride(0), a.shape[0], _ptr(rows), _ptr(w), _ptr(offsets), _ptr(out),
            int(out.dtype == torch.float32), pairs, experts, N, K, ACTIVATIONS[activation] if activation is not None else -1,
            int(bool(gated)), _ptr(flag if flag is not None else self.error_flag), _stream()), "expert_linear")

    def combine_experts(self, results, place, weights, shared, share, x, add: bool = True):
        """``x[t] (+)= sum_k weights[t, k] * results[place[t, k]] + share[t] * shared[t]`` (float32; ``shared`` may be
        None, ``share`` None counts as one); ``add`` false stores instead of adding."""
        self._want(results, torch.float32, "results"); self._want(place, torch.int32, "place")
        self._want(weights, torch.float32, "weights"); self._want(x, torch.float32, "x")
        n, hidden = x.shape
        top = place.shape[1]
        if results.shape[1] != hidden or results.shape[0] != n * top or tuple(weights.shape) != (n, top) or place.shape[0] != n:
            raise KernelError("combine_experts: shapes do not agree")
        if shared is not None:
            self._want(shared, torch.float32, "shared")
            if tuple(shared.shape) != (n, hidden):
                raise KernelError("combine_experts: the shared expert's result must be [tokens, hidden]")
        if share is not None:
            self._want(share, torch.float32, "share")
            if shared is None or share.numel() != n:
                raise KernelError("combine_experts: one gate per token of the shared expert's result is needed")
        self._check(self.lib.skv_combine_experts(_ptr(results), _ptr(place), _ptr(weights), _ptr(shared), _ptr(share),
                                                 _ptr(x), n, hidden, top, int(bool(add)), _stream()), "combine_experts")

    def add_scaled(self, out, other, factor: float):
        """``out += factor * other`` (float32)."""
        self._want(out, torch.float32, "out"); self._want(other, torch.float32, "other")
        if out.numel() != other.numel():
            raise KernelError("add_scaled: sizes differ")
        self._check(self.lib.skv_add_scaled(_ptr(out), _ptr(other), ctypes.c_float(factor),
                                            ctypes.c_longlong(out.numel()), _stream()), "add_scaled")

    def projection_norm(self, rows, eps: float, segments):
        """An RMS norm with a weight over whole segments of a fused projection's float32 rows, in place: for each of one
        or two ``(offset, width, bias or None, weight)``, the columns ``[offset, offset + width)`` plus their bias are
        divided by their root mean square (eps inside the root) and multiplied by the weight (float32 ``[width]``)."""
        self._want(rows, torch.float32, "rows")
        if not 1 <= len(segments) <= 2:
            raise KernelError("projection_norm: one or two segments")
        flat = []
        for offset, width, bias, weight in segments:
            self._want(weight, torch.float32, "weight")
            if bias is not None:
                self._want(bias, torch.float32, "bias")
            if weight.numel() != width or (bias is not None and bias.numel() != width) or offset + width > rows.shape[1]:
                raise KernelError("projection_norm: a segment's sizes do not agree")
            flat += [int(offset), int(width), _ptr(bias), _ptr(weight)]
        if len(segments) == 1:
            flat += [0, 0, _NULL, _NULL]
        self._check(self.lib.skv_projection_norm(_ptr(rows), rows.shape[1], rows.shape[0], ctypes.c_float(eps), *flat,
                                                 _stream()), "projection_norm")

    @staticmethod
    def _state_args(step_meta, state, offset_floats: int):
        """Pointers of a step's packed batch and of a state area ``[slots, bytes]`` whose rows hold a part's floats from
        ``offset_floats`` on."""
        positions, token_seq, cu_q, slot_ids = step_meta
        if state is not None and (state.dtype != torch.float32 or state.dim() != 2 or not state.is_cuda
                                  or not state.is_contiguous()):
            raise KernelError("state must be a contiguous float32 [slots, floats] CUDA tensor")
        for name, tensor in (("positions", positions), ("token_seq", token_seq), ("cu_q", cu_q), ("slot_ids", slot_ids)):
            if tensor.dtype != torch.int32 or not tensor.is_cuda:
                raise KernelError(f"{name} must be int32 on the GPU")
        return (_ptr(positions), _ptr(token_seq), _ptr(cu_q), _ptr(slot_ids), _ptr(state),
                ctypes.c_longlong(state.shape[1] if state is not None else 0), ctypes.c_longlong(offset_floats))

    def short_conv_rotary(self, rows, bias, conv_w, taps: int, cos_sin, rotated: int, interleaved: bool, block_table,
                          q_out, k_cache, v_cache, num_heads: int, num_kv_heads: int, dim: int, block_size: int,
                          write_kv: bool, step_meta, state, state_offset: int = 0):
        """From float32 rows ``[queries | keys]`` of a fused projection: ``bias`` added, a causal convolution over time on
        every channel (``conv_w`` float32 ``[channels, taps]``; what lies before the step comes from ``state``), rotary
        positions on the first ``rotated`` numbers of every head (``cos_sin`` ``[positions, rotated / 2, 2]``; pairs
        ``(2i, 2i + 1)`` if ``interleaved`` else ``(i, i + rotated / 2)``); queries to ``q_out``, rotated keys to
        ``k_cache`` and, with ``v_cache``, the convolved keys before rotation there.  ``state`` float32
        ``[slots, floats]``: from ``state_offset`` a row holds ``[taps, channels]``; ``short_conv_remember`` writes it."""
        self._want(rows, torch.float32, "rows"); self._want(q_out, self.dtype, "q_out")
        self._want(k_cache, self.dtype, "k_cache"); self._want(block_table, torch.int32, "block_table")
        channels = (num_heads + num_kv_heads) * dim
        n = rows.shape[0]
        if v_cache is not None:
            self._want(v_cache, self.dtype, "v_cache")
            if v_cache.shape != k_cache.shape:
                raise KernelError("short_conv_rotary: values that are keys are cached in the keys' shape")
        if rows.shape[1] < channels or tuple(q_out.shape) != (n, num_heads * dim) or \
                tuple(k_cache.shape[1:]) != (num_kv_heads, block_size, dim):
            raise KernelError("short_conv_rotary: shapes do not agree")
        if bias is not None:
            self._want(bias, torch.float32, "bias")
            if bias.numel() != channels:
                raise KernelError("short_conv_rotary: one bias per channel is needed")
        if taps > 0:
            self._want(conv_w, torch.float32, "conv_w")
            if tuple(conv_w.shape) != (channels, taps):
                raise KernelError("short_conv_rotary: the convolution's weight must be [channels, taps]")
        if rotated > 0:
            self._want(cos_sin, torch.float32, "cos_sin")
            if cos_sin.dim() != 3 or cos_sin.shape[1] * 2 != rotated or rotated > dim:
                raise KernelError("short_conv_rotary: the rotation's table must be [positions, rotated / 2, 2]")
        if taps > 1 and (state is None or state_offset + taps * channels > state.shape[1]):
            raise KernelError("short_conv_rotary: the state's rows are too short")
        self._check(self.lib.skv_short_conv_rotary(
            _ptr(rows), rows.shape[1], _ptr(bias), _ptr(conv_w if taps > 0 else None), int(taps),
            _ptr(cos_sin if rotated > 0 else None), int(rotated), int(bool(interleaved)), _ptr(block_table),
            block_table.shape[1], _ptr(q_out), _ptr(k_cache), _ptr(v_cache), n, num_heads, num_kv_heads, dim, block_size,
            int(bool(write_kv)), *self._state_args(step_meta, state, state_offset), _stream()), "short_conv_rotary")

    def short_conv_remember(self, rows, bias, channels: int, taps: int, n_seqs: int, step_meta, state,
                            state_offset: int = 0):
        """The biased projections of every sequence's last ``taps - 1`` positions of the step into its state (row
        ``position mod taps``); it runs after ``short_conv_rotary`` has read the rows of the positions before the step."""
        self._want(rows, torch.float32, "rows")
        if taps <= 1:
            return
        self._check(self.lib.skv_short_conv_remember(
            _ptr(rows), rows.shape[1], _ptr(bias), int(channels), int(taps), int(n_seqs),
            *self._state_args(step_meta, state, state_offset), _stream()), "short_conv_remember")

    def time_mix_state_floats(self, hidden: int, heads: int, dim: int) -> int:
        self.lib.skv_time_mix_state_floats.restype = ctypes.c_longlong
        return int(self.lib.skv_time_mix_state_floats(int(hidden), int(heads), int(dim)))

    def token_shift_mix(self, h, mu, mixes, heads: int, dim: int, step_meta, state, state_offset: int = 0):
        """``mixes[s, t] = h[t] + (h[t - 1] - h[t]) * mu[s]`` in the compute dtype, with zeros before a sequence's first
        token and the last token of the step before from ``state`` (``csrc/time_mix.cu`` has its layout)."""
        self._want(h, self.dtype, "h"); self._want(mixes, self.dtype, "mixes"); self._want(mu, torch.float32, "mu")
        n, hidden = h.shape
        if mixes.dim() != 3 or tuple(mixes.shape[1:]) != (n, hidden) or tuple(mu.shape) != (mixes.shape[0], hidden):
            raise KernelError("token_shift_mix: shapes do not agree")
        self._check(self.lib.skv_token_shift_mix(
            _ptr(h), _ptr(mu), _ptr(mixes), n, hidden, mixes.shape[0], int(heads), int(dim),
            *self._state_args(step_meta, state, state_offset), _stream()), "token_shift_mix")

    def time_mix_decay(self, lora, rank: int, w2, w0, decay):
        """``decay[t, c] = exp(-exp(w0[c] + w2[:, c] . tanh(lora[t, :rank])))`` (float32; ``w2`` ``[rank, channels]``, the
        weight transposed, in the compute dtype)."""
        self._want(lora, torch.float32, "lora"); self._want(w2, self.dtype, "w2"); self._want(w0, torch.float32, "w0")
        self._want(decay, torch.float32, "decay")
        n, channels = decay.shape
        if lora.shape[0] != n or lora.shape[1] < rank or tuple(w2.shape) != (rank, channels) or w0.numel() != channels:
            raise KernelError("time_mix_decay: shapes do not agree")
        self._check(self.lib.skv_time_mix_decay(_ptr(lora), lora.shape[1], int(rank), _ptr(w2), _ptr(w0), _ptr(decay), n,
                                                channels, _stream()), "time_mix_decay")

    def time_mix_scan(self, r, k, v, decay, bonus, out, h, n_seqs: int, heads: int, dim: int, step_meta, state,
                      state_offset: int = 0):
        """Per head ``o_t = (S + diag(bonus) k_t v_t^T)^T r_t``, then ``S <- diag(decay_t) S + k_t v_t^T`` (all float32
        ``[tokens, heads * dim]``); S and the step's last row of ``h`` are kept in ``state``."""
        for name, tensor in (("r", r), ("k", k), ("v", v), ("decay", decay), ("out", out)):
            self._want(tensor, torch.float32, name)
            if tuple(tensor.shape) != tuple(r.shape):
                raise KernelError("time_mix_scan: r, k, v, decay and out have one shape")
        self._want(bonus, torch.float32, "bonus"); self._want(h, self.dtype, "h")
        if r.shape[1] != heads * dim or bonus.numel() != heads * dim or h.shape[0] != r.shape[0]:
            raise KernelError("time_mix_scan: shapes do not agree")
        if state_offset + self.time_mix_state_floats(h.shape[1], heads, dim) > state.shape[1]:
            raise KernelError("time_mix_scan: the state's rows are too short")
        self._check(self.lib.skv_time_mix_scan(
            _ptr(r), _ptr(k), _ptr(v), _ptr(decay), r.shape[1], _ptr(bonus), _ptr(out), _ptr(h), h.shape[1], int(n_seqs),
            int(heads), int(dim), *self._state_args(step_meta, state, state_offset), _stream()), "time_mix_scan")

    def time_mix_finish(self, o, gate, norm, eps: float, out_scale: float, out, heads: int, dim: int):
        """``out = o / rms(o) per head * norm * silu(gate) * out_scale`` in the compute dtype (``out`` may be wider than
        ``heads * dim``; the further columns are set to zero)."""
        self._want(o, torch.float32, "o"); self._want(gate, torch.float32, "gate"); self._want(norm, torch.float32, "norm")
        self._want(out, self.dtype, "out")
        n = o.shape[0]
        if tuple(o.shape) != (n, heads * dim) or tuple(gate.shape) != (n, heads * dim) or norm.numel() != heads * dim \
                or out.shape[0] != n or out.shape[1] < heads * dim:
            raise KernelError("time_mix_finish: shapes do not agree")
        self._check(self.lib.skv_time_mix_finish(_ptr(o), _ptr(gate), o.shape[1], _ptr(norm), ctypes.c_float(eps),
                                                 ctypes.c_float(out_scale), _ptr(out), out.shape[1], n, int(heads),
                                                 int(dim), _stream()), "time_mix_finish")

    def scale_inplace(self, x, factor: float):
        self._want(x, torch.float32, "x")
        self._check(self.lib.skv_scale_inplace(_ptr(x), ctypes.c_float(factor), ctypes.c_longlong(x.numel()), _stream()),
                    "scale_inplace")

    def add_inplace(self, out, other):
        self._want(out, torch.float32, "out"); self._want(other, torch.float32, "other")
        if out.numel() != other.numel():
            raise KernelError("add_inplace: sizes differ")
        self._check(self.lib.skv_add_inplace(_ptr(out), _ptr(other), ctypes.c_longlong(out.numel()), _stream()),
                    "add_inplace")

    def argmax(self, logits, out, flag=None):
        self._want(logits, torch.float32, "logits"); self._want(out, torch.int32, "out")
        rows, vocab = logits.shape
        self._check(self.lib.skv_argmax(_ptr(logits), _ptr(out), rows, vocab, _ptr(flag), _stream()), "argmax")

    def sample(self, logits, out, temperature: float, top_k: int, top_p: float, seed: int, streams, counters,
               flag=None):
        """Temperature / top-k / top-p draw per row; row r uses random number (seed, streams[r], counters[r])."""
        self._want(logits, torch.float32, "logits"); self._want(out, torch.int32, "out")
        self._want(streams, torch.int32, "streams"); self._want(counters, torch.int32, "counters")
        rows, vocab = logits.shape
        if streams.numel() != rows or counters.numel() != rows or out.numel() != rows:
            raise KernelError("sample: one stream, counter and output per row is needed")
        self._check(self.lib.skv_sample(_ptr(logits), _ptr(out), rows, vocab, ctypes.c_float(temperature),
                                        int(top_k), ctypes.c_float(top_p), ctypes.c_ulonglong(seed),
                                        _ptr(streams), _ptr(counters), _ptr(flag), _stream()), "sample")


_LOADED: Dict[Tuple[torch.dtype, int], Kernels] = {}


def kernels_for(dtype: torch.dtype, head_dim: int, verbose: bool = True) -> Kernels:
    key = (dtype, head_dim)
    if key not in _LOADED:
        _LOADED[key] = Kernels(dtype, head_dim, verbose=verbose)
    return _LOADED[key]


def require_cuda(device) -> torch.device:
    device = torch.device(device)
    if device.type != "cuda":
        raise KernelError(f"device {device}: this library runs on CUDA devices only")
    if not torch.cuda.is_available():
        raise KernelError("no CUDA device is available: this library has no CPU path")
    major, minor = torch.cuda.get_device_capability(device)
    if major != 10:
        raise KernelError(f"device {device} has compute capability {major}.{minor}; "
                          "the kernels are built for sm_100a only")
    return device
