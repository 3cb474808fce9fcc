"""A short causal convolution in front of a mixer, as a mixer that wraps another.

  u_t = y_t + sum_j c[:, j] * y_(t - taps + 1 + j)       per channel, y before the sequence's start = 0
and the wrapped mixer reads u instead of y.  The last ``taps - 1`` inputs of a request are its state (a slot of
[taps - 1, H], fp32, zero at admission), beside whatever the wrapped mixer keeps: the need is a CombinedNeed of
the two.  The convolution's tensor is named ``weight_name`` under the part's prefix and the wrapped mixer's
tensors live under ``inner_prefix`` there.
"""

from __future__ import annotations

import torch

from ..kernels import ops
from .base import CombinedNeed, FixedState, LayerCache, Mixer, TensorSpec
from .plan import PartSpec, build_part, register_part


class ShortConvInput(Mixer):
    accepts_lazy_norm = False

    def __init__(self, hidden_size: int, taps: int, inner, weight_name: str = "conv", inner_prefix: str = "mix"):
        self.hidden_size, self.taps = int(hidden_size), int(taps)
        if self.taps < 1:
            raise ValueError(f"a convolution of {taps} taps")
        self.inner = build_part("mixer", inner) if isinstance(inner, PartSpec) else inner
        self.weight_name, self.inner_prefix = weight_name, inner_prefix
        self.weight = None

    @property
    def graph_safe(self):
        return bool(getattr(self.inner, "graph_safe", False))

    def tensor_specs(self, prefix):
        return [TensorSpec(f"{prefix}.{self.weight_name}", (self.hidden_size, self.taps), "vector")] + \
            self.inner.tensor_specs(f"{prefix}.{self.inner_prefix}")

    def bind(self, tensors, prefix):
        self.weight = tensors[f"{prefix}.{self.weight_name}"]
        self.inner.bind(tensors, f"{prefix}.{self.inner_prefix}")

    def cache_need(self):
        history = FixedState((self.taps - 1, self.hidden_size), torch.float32) if self.taps > 1 else None
        return CombinedNeed((history, self.inner.cache_need()))

    def forward(self, x, h, ctx, cache: LayerCache, owns_cache: bool):
        history, inner_cache = cache.parts
        u = ctx.workspace.get("short_conv_out", (x.shape[0], self.hidden_size), x.dtype)
        ops.short_conv(x, u, self.weight, None if history is None else history.state, ctx, advance=owns_cache)
        self.inner.forward(u, h, ctx, inner_cache, owns_cache)


register_part("mixer", "short_conv_input", ShortConvInput)
