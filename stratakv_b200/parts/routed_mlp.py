"""A mixture of experts: every token runs through the ``top`` experts that its router scores choose, and through a
shared expert if the layer has one.

    s = sigmoid(router h)                       float32, one score per expert (spec.score "softmax": a softmax over them)
    chosen: the `top` largest s + correction    (the correction chooses only; with spec.groups only experts of the
                                                 keep_groups best groups, a group scoring what its best expert does)
    y = sum over chosen e of s_e * route_scale * down_e act(up_e h)          (weights divided by their sum first if
                                                                               the spec says `renormalize`)
      + sigmoid(shared.gate . h) * shared.down act(shared.up h)

An expert may be gated (``spec.gate_weights``): ``down_e (act(gate_e h) * (up_e h))``, gate and up rows packed in tiles as
the dense gated feed-forward packs them.

Kernels (``csrc/routed_mlp.cu``): the router (scores, choice, weights, the shared expert's gate), a counting sort of
the (token, expert) pairs by expert, the two projections over the sorted pairs (each block of rows reads the
weights of the one expert that its rows chose; the first gathers its rows from the tokens), and the weighted sum,
which also adds the shared expert's result.  The shared expert's projections are the library's own.  Nothing is read
back to the host, so a step can be captured in a graph.
"""
from __future__ import annotations

import torch

from .. import ops as _ops
from .base import FeedForward, TensorRequest
from .ffn import pack_gate_up
from .registry import register_ffn


class RoutedMlp(FeedForward):
    graph_safe = True
    stores_branch = True

    def __init__(self, spec, runtime):
        super().__init__(spec, runtime)
        if spec.activation not in _ops.ACTIVATIONS or spec.activation in _ops.PARAMETRIC_ACTIVATIONS:
            raise ValueError(f"routed feed-forward: activation '{spec.activation}' is not supported")
        if not 0 < spec.top <= spec.experts or spec.experts > _ops.MAX_EXPERTS or spec.top > _ops.MAX_EXPERTS_PER_TOKEN:
            raise ValueError(f"routed feed-forward: {spec.top} of {spec.experts} experts is not supported (at most "
                             f"{_ops.MAX_EXPERTS_PER_TOKEN} of {_ops.MAX_EXPERTS})")
        if len(spec.up_weights) != spec.experts or len(spec.down_weights) != spec.experts:
            raise ValueError("routed feed-forward: one pair of tensor names per expert is needed")
        self.gated = getattr(spec, "gate_weights", None) is not None
        if self.gated and len(spec.gate_weights) != spec.experts:
            raise ValueError("routed feed-forward: one gate tensor per expert is needed")
        self.score = getattr(spec, "score", "sigmoid")
        if self.score not in ("sigmoid", "softmax"):
            raise ValueError(f"routed feed-forward: scores '{self.score}' are not supported (sigmoid, softmax)")
        self.groups, self.keep = getattr(spec, "groups", 0), getattr(spec, "keep_groups", 0)
        if self.groups > 1 and (spec.experts % self.groups or not 0 < self.keep <= self.groups
                                or self.keep * (spec.experts // self.groups) < spec.top):
            raise ValueError("routed feed-forward: the groups must divide the experts and the kept ones hold the choices")
        if runtime.dtype == torch.bfloat16 and spec.hidden_size % 8 != 0:
            raise ValueError(f"routed feed-forward: hidden size {spec.hidden_size} is not supported in bfloat16 "
                             "(rows of 16 bytes are needed: a multiple of 8); float32 takes any size")
        self.padded = -(-spec.intermediate_size // 8) * 8
        self.shared_padded = -(-spec.shared.intermediate_size // 8) * 8 if spec.shared is not None else 0

    @classmethod
    def expected_tensors(cls, spec):
        wanted = {spec.router_weight: TensorRequest((spec.experts, spec.hidden_size))}
        if spec.correction is not None:
            wanted[spec.correction] = TensorRequest((spec.experts,))
        for up, down in zip(spec.up_weights, spec.down_weights):
            wanted[up] = TensorRequest((spec.intermediate_size, spec.hidden_size))
            wanted[down] = TensorRequest((spec.hidden_size, spec.intermediate_size))
        for gate in getattr(spec, "gate_weights", None) or ():
            wanted[gate] = TensorRequest((spec.intermediate_size, spec.hidden_size))
        if spec.shared is not None:
            wanted[spec.shared.up_weight] = TensorRequest((spec.shared.intermediate_size, spec.hidden_size))
            wanted[spec.shared.down_weight] = TensorRequest((spec.hidden_size, spec.shared.intermediate_size))
            if spec.shared.gate_weight is not None:
                wanted[spec.shared.gate_weight] = TensorRequest((1, spec.hidden_size))
        return wanted

    @staticmethod
    def _padded(up, down, width):
        """Zero rows of up give act(0) = 0 for every activation here and meet zero columns of down."""
        missing = width - up.shape[0]
        if missing:
            up = torch.cat([up, up.new_zeros(missing, up.shape[1])], dim=0)
            down = torch.cat([down, down.new_zeros(down.shape[0], missing)], dim=1)
        return up.contiguous(), down.contiguous()

    def bind(self, tensors):
        s, rt = self.spec, self.rt
        self.w_router = rt.upload(tensors[s.router_weight]).contiguous()
        self.correction = (rt.upload(tensors[s.correction], torch.float32).reshape(-1).contiguous()
                           if s.correction is not None else None)
        ups, downs = [], []
        for index, (up_name, down_name) in enumerate(zip(s.up_weights, s.down_weights)):
            up, down = self._padded(rt.upload(tensors[up_name]), rt.upload(tensors[down_name]), self.padded)
            if self.gated:                          # [2 ff, hidden]: tiles of 8 gate rows and their 8 up rows
                up = pack_gate_up(rt.upload(tensors[s.gate_weights[index]]), up[:s.intermediate_size])
            ups.append(up)
            downs.append(down)
        self.w_up = torch.stack(ups).contiguous()            # [experts, ff, hidden]
        self.w_down = torch.stack(downs).contiguous()        # [experts, hidden, ff]
        del ups, downs
        self.shared_up = self.shared_down = self.shared_gate = None
        if s.shared is not None:
            self.shared_up, self.shared_down = self._padded(rt.upload(tensors[s.shared.up_weight]),
                                                            rt.upload(tensors[s.shared.down_weight]), self.shared_padded)
            if s.shared.gate_weight is not None:
                self.shared_gate = rt.upload(tensors[s.shared.gate_weight]).reshape(-1).contiguous()

    def forward(self, step, h, x):
        s, rt = self.spec, self.rt
        ops = rt.kernels()
        get = rt.workspace.get
        n, pairs = h.shape[0], h.shape[0] * s.top
        chosen = get("routed_chosen", (n, s.top), torch.int32)
        weights = get("routed_weights", (n, s.top), torch.float32)
        share = get("routed_share", (n,), torch.float32) if self.shared_gate is not None else None
        ops.route_tokens(h, self.w_router, self.correction, s.top, s.route_scale, s.renormalize, chosen, weights,
                         shared_gate_weight=self.shared_gate, shared_gate_out=share, softmax=self.score == "softmax",
                         groups=self.groups, keep=self.keep, renorm_eps=getattr(s, "renormalize_eps", 0.0))
        if step.choice_probe is not None:
            step.choice_probe(step.run_index, step, chosen)
        offsets = get("routed_offsets", (s.experts + 1,), torch.int32)
        order = get("routed_order", (pairs,), torch.int32)           # the token of every sorted pair
        place = get("routed_place", (n, s.top), torch.int32)         # where each (token, choice) went
        ops.sort_by_expert(chosen, s.experts, offsets, order, place)
        hidden = get("routed_hidden", (pairs, self.padded), rt.dtype)
        if ops.expert_rows_sorted_first(s.hidden_size):
            # the tensor-core projection reads tiles of neighbouring rows: bring the tokens' rows into sorted order first
            gathered = get("routed_rows", (pairs, s.hidden_size), rt.dtype)
            ops.gather_rows(h, order, gathered)
            ops.expert_linear(gathered, self.w_up, offsets, hidden, activation=s.activation, gated=self.gated)
        else:
            ops.expert_linear(h, self.w_up, offsets, hidden, rows=order, activation=s.activation, gated=self.gated)
        results = get("routed_results", (pairs, s.hidden_size), torch.float32)
        ops.expert_linear(hidden, self.w_down, offsets, results)
        shared_out = None
        if self.shared_up is not None:
            z = get("ffn_hidden", (n, self.shared_padded), rt.dtype)
            ops.linear(h, self.shared_up, z, _ops.MODE_ACT, s.activation)
            shared_out = get("routed_shared", (n, s.hidden_size), torch.float32)
            ops.linear(z, self.shared_down, shared_out, _ops.MODE_STORE_F32)
        ops.combine_experts(results, place, weights, shared_out, share, x, add=not getattr(step, "store_branch", False))


register_ffn("routed_mlp", RoutedMlp)
