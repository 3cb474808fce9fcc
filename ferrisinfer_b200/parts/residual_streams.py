"""A layer over several residual streams (hyper-connections), as a block kind.

A token has ``streams`` residual rows x_1 .. x_S instead of one (the model keeps them as [T, S x H] fp32 and starts them
all from the embedding output; its result is their sum).  For each sublayer (1: the mixer, 2: the feed-forward), with
three learned tensors ``<hc>.in`` [S], ``<hc>.out`` [S] and ``<hc>.mix`` [S, S] (indexed [from, to]):

  u = sum_s in[s] x_s;   y = sublayer(norm(u));   x_r <- sum_s mix[s, r] x_s + out[r] y     (all r from the old streams)

The read with its RMS norm and the write of the sublayer before it are one pass over the streams
(``ops.streams_step``), also across layers: a layer leaves its last write to the first pass of the next one (the
model carries out what the last layer left).  Mixers and feed-forwards keep their interface: their result goes into an fp32 row buffer
(replacing what it held where the part can do that, added into zeroed rows otherwise), which the write then
distributes.  A layer may have no feed-forward.  ``learned`` False (one stream only): no
stream tensors are read and in = mix = out = 1, which is the plain pre-norm residual layer x <- x + sublayer(norm(x))
through the same kernels.
"""

from __future__ import annotations

import torch

from ..kernels import ops
from .base import Block, TensorSpec
from .plan import register_part


# key of ``ctx.shared``: the last write of a layer, (y, mix, out), which the next layer's first pass over the streams
# carries out (or ``flush_pending_write``, before anything else reads the streams)
PENDING_WRITE = "residual_streams_pending_write"


def flush_pending_write(ctx, h, streams: int) -> None:
    """Carry out the write that the last layer left for its successor."""
    pending = ctx.shared.pop(PENDING_WRITE, None)
    if pending is not None:
        ops.streams_step(h, streams, write=pending)


class ResidualStreamsBlock(Block):
    # the model hands this block [T, streams x H] rows
    def __init__(self, hidden_size: int, mixer, feed_forward, mixer_norm, feed_forward_norm, streams: int,
                 mixer_prefix: str = "mix", feed_forward_prefix: str = "mlp", mixer_norm_prefix: str = "norm1",
                 feed_forward_norm_prefix: str = "norm2", mixer_streams_prefix: str = "hc1",
                 feed_forward_streams_prefix: str = "hc2", learned: bool = True):
        self.hidden_size, self.streams, self.learned = int(hidden_size), int(streams), bool(learned)
        if not 1 <= self.streams <= 8:
            raise ValueError(f"{streams} residual streams (one to eight)")
        if not self.learned and self.streams != 1:
            raise ValueError("streams without learned weights: one stream only")
        self.mixer, self.feed_forward = mixer, feed_forward
        self.mixer_norm, self.feed_forward_norm = mixer_norm, feed_forward_norm
        for n in (mixer_norm, feed_forward_norm):
            # the read forms the norm itself: an RMS norm over the whole row with a plain weight
            if getattr(n, "groups", 1) != 1 or not hasattr(n, "eps") or n.hidden_size != self.hidden_size:
                raise ValueError("a block over residual streams takes RMS norms over the whole row")
        self._names = (mixer_prefix, feed_forward_prefix, mixer_norm_prefix, feed_forward_norm_prefix,
                       mixer_streams_prefix, feed_forward_streams_prefix)
        self.hc = {}

    def _children(self, prefix):
        m, f, n1, n2, _, _ = self._names
        out = [(self.mixer_norm, f"{prefix}.{n1}"), (self.mixer, f"{prefix}.{m}" if m else prefix)]
        if self.feed_forward is not None:
            out += [(self.feed_forward_norm, f"{prefix}.{n2}"), (self.feed_forward, f"{prefix}.{f}")]
        return out

    def _stream_prefixes(self, prefix):
        out = [f"{prefix}.{self._names[4]}"]
        if self.feed_forward is not None:
            out.append(f"{prefix}.{self._names[5]}")
        return out

    def tensor_specs(self, prefix):
        S = self.streams
        out = []
        for part, p in self._children(prefix):
            out += part.tensor_specs(p)
        for p in self._stream_prefixes(prefix) if self.learned else ():
            out += [TensorSpec(f"{p}.in", (S,), "vector"), TensorSpec(f"{p}.out", (S,), "vector"),
                    TensorSpec(f"{p}.mix", (S, S), "vector")]
        return out

    def bind(self, tensors, prefix):
        for part, p in self._children(prefix):
            part.bind(tensors, p)
        if self.learned:
            self.hc = [tuple(tensors[f"{p}.{n}"] for n in ("in", "out", "mix")) for p in self._stream_prefixes(prefix)]
        else:
            one = torch.ones(1, dtype=torch.float32, device=self.mixer_norm.weight.device)
            self.hc = [(one, one, one)] * len(self._stream_prefixes(prefix))

    def cache_need(self):
        return self.mixer.cache_need()

    @property
    def graph_safe(self):
        return bool(getattr(self.mixer, "graph_safe", False)
                    and (self.feed_forward is None or getattr(self.feed_forward, "graph_safe", False)))

    def forward(self, h, ctx, cache, owns_cache):
        T, S, H = h.shape[0], self.streams, self.hidden_size
        x = ctx.workspace.get("block_normed", (T, H), ctx.act_dtype)
        y = ctx.workspace.get("streams_sublayer_out", (T, H), torch.float32)
        in1, out1, mix1 = self.hc[0]
        # the write that the layer before left undone rides in this layer's first pass over the streams
        pending = ctx.shared.pop(PENDING_WRITE, None)
        # a mixer that reads its input shifted by a token lets the read do that where every request brings one token
        ask = getattr(self.mixer, "shift_in_read", None)
        shift = ask(ctx, cache, owns_cache) if ask is not None else None
        ops.streams_step(h, S, write=pending, read=(in1, self.mixer_norm.weight, self.mixer_norm.eps, x),
                         shift=None if shift is None else (shift[0], shift[1], ctx))
        extra = {} if shift is None else {"shifted": True}
        if getattr(self.mixer, "can_overwrite", False):
            self.mixer.forward(x, y, ctx, cache, owns_cache, accumulate=False, **extra)
        else:  # a mixer that only adds: into zeroed rows
            y.zero_()
            self.mixer.forward(x, y, ctx, cache, owns_cache, **extra)
        if self.feed_forward is None:
            ctx.shared[PENDING_WRITE] = (y, mix1, out1)
            return
        in2, out2, mix2 = self.hc[1]
        ops.streams_step(h, S, write=(y, mix1, out1),
                         read=(in2, self.feed_forward_norm.weight, self.feed_forward_norm.eps, x))
        if getattr(self.feed_forward, "can_overwrite", False):
            self.feed_forward.forward(x, y, ctx, accumulate=False)
        else:
            y.zero_()
            self.feed_forward.forward(x, y, ctx)
        ctx.shared[PENDING_WRITE] = (y, mix2, out2)


register_part("block", "residual_streams", ResidualStreamsBlock)
