"""Arrangements: how a layer's norms, mixer and feed-forward are strung together.

``pre_norm`` is the Llama block, ``x += mixer(norm(x)); x += ffn(norm(x))``
(``src/models/transformer_block.cpp:301-331``); ``parallel`` feeds one norm's output to
both branches.  Another arrangement is one more function registered under its name.
"""
from __future__ import annotations

import torch

from .registry import part_class, register_arrangement


class Layer:
    """The built parts of one ``LayerSpec``."""
    # the norm that reads the stream first, and the part it feeds (for the layer or embedding before)
    first_norm = property(lambda self: foldable(self.mixer_norm, self.mixer))

    def __init__(self, spec, runtime):
        self.spec = spec
        self.mixer_norm = self.mixer = self.ffn_norm = self.ffn = None
        self.extra = {}
        self._parts = []
        named = {"mixer_norm", "mixer", "ffn_norm", "ffn"}
        for name, role, part_spec in spec.named_parts():
            part = part_class(role, part_spec.kind)(part_spec, runtime)
            if name in named:
                setattr(self, name, part)
            else:
                self.extra[name] = part
            self._parts.append(part)
        self.run = part_class("arrangement", spec.arrangement)

    def parts(self):
        return tuple(self._parts)

    def forward(self, step, x, entry):
        self.run(self, step, x, entry)


def _normed(norm, consumer, step, x):
    stats = step.residual_stats
    if stats is not None and norm.folds_norm and consumer.folds_norm:
        return norm.forward(x, stats=stats)
    return norm.forward(x)


def foldable(norm, consumer):
    """The norm, if it can be folded into its consumer's first projection, else None."""
    return norm if norm is not None and consumer is not None and norm.folds_norm and consumer.folds_norm else None


def pre_norm(layer: Layer, step, x, entry) -> None:
    if layer.mixer_norm is None or layer.mixer is None or layer.ffn_norm is None or layer.ffn is None:
        raise ValueError("the pre_norm arrangement needs a norm and a mixer, and a norm and a feed-forward")
    stats = step.residual_stats
    h = _normed(layer.mixer_norm, layer.mixer, step, x)
    if stats is not None:
        stats.expect(foldable(layer.ffn_norm, layer.ffn))
    layer.mixer.forward(step, h, x, entry.cache, entry.writes_cache)
    if stats is not None and not layer.mixer.folds_norm:
        stats.invalidate()
    h = _normed(layer.ffn_norm, layer.ffn, step, x)
    if stats is not None:
        stats.expect(step.norm_after_layer)
    layer.ffn.forward(step, h, x)
    if stats is not None and not layer.ffn.folds_norm:
        stats.invalidate()


def parallel(layer: Layer, step, x, entry) -> None:
    """``h = norm(x); x += mixer(h) + ffn(h)``: one norm, and both branches read its output.  A layer
    without a feed-forward is ``x += mixer(norm(x))``."""
    if layer.mixer_norm is None or layer.mixer is None:
        raise ValueError("the parallel arrangement needs a norm and a mixer")
    stats = step.residual_stats
    folding = stats is not None and layer.mixer.folds_norm and (layer.ffn is None or layer.ffn.folds_norm)
    h = _normed(layer.mixer_norm, layer.mixer, step, x) if folding else layer.mixer_norm.forward(x)
    # Both branches add to the stream; the one that adds last leaves what the next norm's consumer needs.  A
    # norm handed over unfinished (``NormedRows``) stays readable for the second branch: the first one's
    # residual sum is told to expect nobody and so leaves the rows it was computed from alone.
    if stats is not None:
        stats.expect(step.norm_after_layer if folding and layer.ffn is None else None)
    layer.mixer.forward(step, h, x, entry.cache, entry.writes_cache)
    if layer.ffn is not None:
        if stats is not None:
            stats.expect(step.norm_after_layer if folding else None)
        layer.ffn.forward(step, h, x)
    if stats is not None and not folding:
        stats.invalidate()


def _fusable(norm):
    """True if the kernels that add to the stream can also apply this norm to their result (a plain RMS norm)."""
    return norm is not None and getattr(norm.spec, "kind", None) == "rmsnorm" and hasattr(norm, "gamma")


def _branch(part, step, h, shape, *cache_args):
    """Run a mixer or feed-forward into a float32 scratch buffer instead of the stream and return the buffer."""
    rt = part.rt
    out = rt.workspace.get("branch", shape, torch.float32)
    if part.stores_branch:
        step.store_branch = True
        try:
            part.forward(step, h, out, *cache_args)
        finally:
            step.store_branch = False
    else:                                           # the part only knows how to add: hand it zeros
        out.zero_()
        part.forward(step, h, out, *cache_args)
    return out


def sandwich(layer: Layer, step, x, entry) -> None:
    """``x += post1(mixer(norm1(x))); x += post2(ffn(norm2(x)))`` and then the layer's ``token_input``, if it has
    one.  The norms after the sublayers are the extras ``mixer_post_norm`` and ``ffn_post_norm``; a layer may have no
    feed-forward.  The kernel that adds a normed branch to the stream also applies the norm that reads the stream
    next (this layer's second, or the next layer's first), which the next reader then finds in ``step.scratch``."""
    post_mixer, post_ffn = layer.extra.get("mixer_post_norm"), layer.extra.get("ffn_post_norm")
    side = layer.extra.get("token_input")
    if layer.mixer_norm is None or layer.mixer is None or post_mixer is None:
        raise ValueError("the sandwich arrangement needs a norm, a mixer and a norm after it")
    if layer.ffn is not None and (layer.ffn_norm is None or post_ffn is None):
        raise ValueError("the sandwich arrangement needs a norm before and after its feed-forward")
    stats = step.residual_stats
    if stats is not None:
        stats.expect(None)                          # nothing here folds a norm into a projection
    rt = layer.mixer.rt
    ops = rt.kernels()

    def normed_ahead(norm, name):
        """The buffer for ``norm`` applied by the kernel in front, or None where that kernel cannot."""
        return rt.workspace.get(name, tuple(x.shape), rt.dtype) if _fusable(norm) else None

    def add_normed(branch, post, norm_ahead, name):
        ahead = normed_ahead(norm_ahead, name)
        ops.rmsnorm_add(branch, post.gamma, post.spec.eps, x,
                        next_gamma=norm_ahead.gamma if ahead is not None else None,
                        next_eps=norm_ahead.spec.eps if ahead is not None else 0.0, next_out=ahead)
        return ahead

    prepared = step.scratch.pop("normed_ahead", None)
    h = prepared[1] if prepared is not None and prepared[0] is layer.mixer_norm else layer.mixer_norm.forward(x)
    branch = _branch(layer.mixer, step, h, tuple(x.shape), entry.cache, entry.writes_cache)
    last = layer.ffn is None and side is None
    ahead_norm = layer.ffn_norm if layer.ffn is not None else (step.next_layer_norm if last else None)
    ahead = add_normed(branch, post_mixer, ahead_norm, "normed" if layer.ffn is not None else "normed_next")
    pending = None                                  # a branch that the token input's kernel adds on its way
    if layer.ffn is not None:
        h = ahead if ahead is not None else layer.ffn_norm.forward(x)
        branch = _branch(layer.ffn, step, h, tuple(x.shape))
        if side is not None and getattr(side, "adds_branch", False) and _fusable(post_ffn):
            pending = (branch, post_ffn)
        else:
            ahead_norm = step.next_layer_norm if side is None else None
            ahead = add_normed(branch, post_ffn, ahead_norm, "normed_next")
    if side is not None:
        ahead_norm = step.next_layer_norm
        ahead = normed_ahead(ahead_norm, "normed_next")
        more = dict(branch=pending[0], post_norm=pending[1]) if pending is not None else {}
        side.forward(step, x, ahead_norm if ahead is not None else None, ahead, **more)
    if ahead is not None and ahead_norm is not None:
        step.scratch["normed_ahead"] = (ahead_norm, ahead)
    if stats is not None:
        stats.invalidate()


def multi_stream(layer: Layer, step, x, entry) -> None:
    """The pre-norm block over several copies of the stream: each sublayer reads a mix of the streams through its
    norm and its result goes into every stream (``parts/stream_mix.py``).  The streams live in scratch memory
    ``[streams, tokens, hidden]``; before the first layer they all equal the embedding's output, which ``x`` holds,
    and after every layer ``x`` is their sum (what the last norm reads).  One kernel brings the streams up to date
    after a sublayer, reads them for the sublayer after it (this layer's feed-forward, or the next layer's mixer) and
    applies that one's norm."""
    link = layer.extra.get("mixer_streams")
    ffn_link = layer.extra.get("ffn_streams")
    if layer.mixer_norm is None or layer.mixer is None or link is None:
        raise ValueError("the multi_stream arrangement needs a norm, a mixer and the mixer's connection to the streams")
    if layer.ffn is not None and (layer.ffn_norm is None or ffn_link is None):
        raise ValueError("the multi_stream arrangement needs a norm and a connection for its feed-forward")
    stats = step.residual_stats
    if stats is not None:
        stats.expect(None)                          # nothing here folds a norm into a projection
    rt = layer.mixer.rt
    ops = rt.kernels()
    count = link.spec.streams
    shape = tuple(x.shape)
    streams = rt.workspace.get("streams", (count,) + shape, torch.float32)
    source = x if step.run_index == 0 else None     # the streams have not been written yet: they all equal x

    prepared = step.scratch.pop("normed_ahead", None)
    if prepared is not None and prepared[0] is layer.mixer_norm:
        h = prepared[1]
    else:
        h = rt.workspace.get("normed", shape, rt.dtype)
        ops.stream_mix(streams, count, source, read=link.read, gamma=layer.mixer_norm.gamma,
                       eps=layer.mixer_norm.spec.eps, normed_out=h)
    branch = _branch(layer.mixer, step, h, shape, entry.cache, entry.writes_cache)
    if layer.ffn is not None:
        h = rt.workspace.get("normed", shape, rt.dtype)
        ops.stream_mix(streams, count, source, branch=branch, mix=link.mix, write=link.write, read=ffn_link.read,
                       gamma=layer.ffn_norm.gamma, eps=layer.ffn_norm.spec.eps, normed_out=h)
        source = None
        branch = _branch(layer.ffn, step, h, shape)
        link = ffn_link
    # the layer's last update also leaves the sum of the streams in x and reads them for the next layer
    following = step.next_layer
    ahead = ahead_link = None
    if (following is not None and following.spec.arrangement == "multi_stream" and _fusable(following.mixer_norm)
            and following.extra["mixer_streams"].spec.streams == count):
        ahead_link = following.extra["mixer_streams"]
        ahead = rt.workspace.get("normed_next", shape, rt.dtype)
    ops.stream_mix(streams, count, source, branch=branch, mix=link.mix, write=link.write,
                   read=ahead_link.read if ahead is not None else None,
                   gamma=following.mixer_norm.gamma if ahead is not None else None,
                   eps=following.mixer_norm.spec.eps if ahead is not None else 0.0, normed_out=ahead, sum_out=x)
    if ahead is not None:
        step.scratch["normed_ahead"] = (following.mixer_norm, ahead)
    if stats is not None:
        stats.invalidate()


def parallel_pair(layer: Layer, step, x, entry) -> None:
    """``x += mixer(norm1(x)) + ffn(norm2(x))``: two norms of the same x, one for each branch, and then the layer's
    ``token_input`` if it has one.  A layer may have no feed-forward (then it has no second norm either)."""
    if layer.mixer_norm is None or layer.mixer is None:
        raise ValueError("the parallel_pair arrangement needs a norm and a mixer")
    if layer.ffn is not None and layer.ffn_norm is None:
        raise ValueError("the parallel_pair arrangement needs a norm of its own for the feed-forward")
    stats = step.residual_stats
    if stats is not None:
        stats.expect(None)                          # nothing here folds a norm into a projection
    # both norms read the stream before either branch has been added to it
    h_mixer = layer.mixer_norm.forward(x, name="normed")
    h_ffn = layer.ffn_norm.forward(x, name="normed_second") if layer.ffn is not None else None
    layer.mixer.forward(step, h_mixer, x, entry.cache, entry.writes_cache)
    if layer.ffn is not None:
        layer.ffn.forward(step, h_ffn, x)
    side = layer.extra.get("token_input")
    if side is not None:
        side.forward(step, x)
    if stats is not None:
        stats.invalidate()


register_arrangement("multi_stream", multi_stream)
register_arrangement("parallel_pair", parallel_pair)
register_arrangement("pre_norm", pre_norm)
register_arrangement("sandwich", sandwich)
register_arrangement("parallel", parallel)
