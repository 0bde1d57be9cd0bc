"""How a sublayer is connected to several copies of the residual stream (hyper-connections).

With ``s`` streams ``x_1 .. x_s`` (all equal to the embedding's output before the first layer), a sublayer reads
``u = sum_s read[s] x_s`` and, once it has run on ``norm(u)``, every stream becomes
``x_t <- sum_s mix[s, t] x_s + write[t] * result``, all from the old ones.  The part holds the three small tensors in
float32; the ``multi_stream`` arrangement (``parts/block.py``) hands them to ``ops.stream_mix``.  A connection without
tensor names is the plain residual sum over one stream.
"""
from __future__ import annotations

import torch

from .base import Part, TensorRequest
from .registry import register_stream_mix


class StreamMix(Part):
    role = "stream_mix"
    graph_safe = True

    @classmethod
    def expected_tensors(cls, spec):
        if spec.read is None:
            return {}
        s = spec.streams
        return {spec.read: TensorRequest((s,), "around_one"), spec.write: TensorRequest((s,), "around_one"),
                spec.mix: TensorRequest((s, s), "around_identity")}

    def bind(self, tensors):
        s, rt = self.spec, self.rt
        if s.read is None:
            if s.streams != 1:
                raise ValueError("a connection without tensors is the plain sum over one stream")
            ones = torch.ones(1, dtype=torch.float32, device=rt.device)
            self.read, self.write, self.mix = ones, ones.clone(), ones.clone()
            return
        self.read = rt.upload(tensors[s.read], torch.float32).reshape(-1).contiguous()
        self.write = rt.upload(tensors[s.write], torch.float32).reshape(-1).contiguous()
        self.mix = rt.upload(tensors[s.mix], torch.float32).reshape(-1).contiguous()       # [from * streams + to]


register_stream_mix("stream_mix", StreamMix)
