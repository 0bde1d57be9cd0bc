"""The two ends of a model as parts: token embedding and output head.

``TokenEmbedding``: row ``ids[t]`` of the table becomes row ``t`` of the float32
residual stream (``src/generation/generator.cpp:520-529``).  ``LinearHead``:
``logits = y . W^T`` on the rows that the final norm was asked for, in float32
(``src/generation/generator.cpp:773-774``); its weight may be the embedding
table (tied), in which case both parts share one copy on the device.

Both are looked up by their spec's ``kind`` like every other part, so an
embedding with a scale factor or a head that caps its logits is another class
registered under another kind; the model only calls ``forward``.
"""
from __future__ import annotations

import torch

from .. import ops as _ops
from .base import CacheRequest, Part, TensorRequest
from .registry import register_embedding, register_head


class TokenEmbedding(Part):
    role = "embedding"
    graph_safe = True

    @classmethod
    def expected_tensors(cls, spec):
        return {spec.weight: TensorRequest((spec.vocab_size, spec.hidden_size))}

    def bind(self, tensors):
        self.table = self.rt.upload_shared(self.spec.weight, tensors[self.spec.weight])

    def forward(self, step, x, flags, stats=None) -> None:
        """Fill the stream ``x`` [tokens, hidden] for ``step.token_ids``; an id outside the table raises
        bit 0 of ``flags``.  ``stats``: see ``residual.ResidualStats`` (the kernel fills it where it can)."""
        # (a class that builds on this one for another kind of spec scales, or does not, by itself)
        scale = getattr(self.spec, "scale", 1.0) if getattr(self.spec, "kind", None) == "embedding" else 1.0
        # (a scaled row is not what the folded norm's statistics were taken of: the norm then runs as a kernel)
        self.rt.kernels().embed(self.table, step.token_ids, x, flags, stats=stats if scale == 1.0 else None)
        if scale != 1.0:
            self.rt.kernels().scale_inplace(x, scale)
            if stats is not None:
                stats.invalidate()


class SummedEmbedding(Part):
    """The token's row plus, where the spec names them, the row of a table of hashed token pairs and a learned
    vector for the position, summed in float32 (``csrc/elementwise.cu``).  The pair needs the token before: inside a
    step it is the neighbour, across steps it is what the sequence brought last, which is two int32 of state per
    sequence in the cache: the last id at an even and at an odd position, so that a step which is run twice
    reads the same id both times (``cache_request``; the model tells the part its cache entry as ``state_entry``)."""
    role = "embedding"
    graph_safe = True
    state_entry = None

    @classmethod
    def expected_tensors(cls, spec):
        wanted = {spec.weight: TensorRequest((spec.vocab_size, spec.hidden_size))}
        if spec.pair is not None:
            wanted[spec.pair.weight] = TensorRequest((spec.pair.buckets + 1, spec.hidden_size))
        if spec.positions is not None:
            wanted[spec.positions.weight] = TensorRequest((spec.positions.max_positions, spec.hidden_size))
        return wanted

    @classmethod
    def cache_request(cls, spec):
        """Per-sequence state this embedding keeps: the last token ids, if pairs are hashed; else None."""
        return CacheRequest(kind="none", state_bytes=8) if spec.pair is not None else None

    def bind(self, tensors):
        s = self.spec
        self.table = self.rt.upload_shared(s.weight, tensors[s.weight])
        self.pair_table = self.rt.upload(tensors[s.pair.weight]) if s.pair is not None else None
        self.position_table = self.rt.upload(tensors[s.positions.weight]) if s.positions is not None else None

    def forward(self, step, x, flags, stats=None) -> None:
        s = self.spec
        last_ids = None
        if s.pair is not None:
            last_ids = step.cache.state(self.state_entry).view(torch.int32).view(-1)
        self.rt.kernels().embed_sum(
            self.table, step.token_ids, x, step.positions, step.token_seq, step.cu_q, step.slot_ids, flags,
            pair_table=self.pair_table, last_ids=last_ids,
            mul_prev=s.pair.mul_prev if s.pair is not None else 0, mul_cur=s.pair.mul_cur if s.pair is not None else 0,
            position_table=self.position_table, position_scale=s.positions.scale if s.positions is not None else 1.0,
            stats=stats)


class LinearHead(Part):
    role = "head"
    graph_safe = True
    folds_norm = True

    @classmethod
    def expected_tensors(cls, spec):
        return {spec.weight: TensorRequest((spec.vocab_size, spec.hidden_size))}

    def bind(self, tensors):
        self.weight = self.rt.upload_shared(self.spec.weight, tensors[self.spec.weight])

    def forward(self, y, n_rows: int) -> torch.Tensor:
        """``y``: the normalised rows (or ``residual.NormedRows``); returns float32 ``[n_rows, vocab]``
        in scratch memory that the next step overwrites."""
        logits = self.rt.workspace.get("logits", (n_rows, self.spec.vocab_size), torch.float32)
        self.rt.kernels().linear(y, self.weight, logits, _ops.MODE_STORE_F32)
        scale = getattr(self.spec, "logit_scale", 1.0)         # (a head spec of another design may not have one)
        if scale != 1.0:
            self.rt.kernels().scale_inplace(logits, scale)
        return logits


register_embedding("embedding", TokenEmbedding)
register_embedding("summed_embedding", SummedEmbedding)
register_head("linear_head", LinearHead)
