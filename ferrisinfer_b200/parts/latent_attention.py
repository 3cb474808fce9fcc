"""Attention over a latent that all heads share, as a part.

  q = y Wq^T, per head [dim plain | rot rotated];  y Wdkv^T = [c': rank | k_r: rot]
  c = rmsnorm(c') * n;  k_r and each head's q_r are rotated (rotate-half over the first ``rotary_dims`` of the part)
  per head: k = Wuk c (dim), v = Wuv c (vdim);  s = (q . k + q_r . k_r) * scale;  causal softmax;  o = sum w v
  o_h <- o_h * sigmoid(y Wg^T)_h;  h += concat(o) Wo^T

Only [c | k_r] is cached: one row of rank + rot per token, whatever the number of heads.  The step never forms k and v
of the cached tokens.  Since q . (Wuk c) = (Wuk^T q) . c, each head's plain query is taken through Wuk^T once
(``ops.head_gemm``), the attention then runs with ONE shared key head of rank + rot whose first rank elements are
also the value (``values_in_keys``), and each head's weighted sum of latents is taken through Wuv afterwards, where
the head's output gate multiplies.  Scores, weights and sums are fp32.
"""

from __future__ import annotations

import torch

from ..kernels import ops
from .base import LayerCache, Mixer, PagedKV, TensorSpec
from .plan import register_part
from .recurrent import _fused_rows


class LatentAttention(Mixer):
    accepts_lazy_norm = True
    graph_safe = True
    can_overwrite = True

    def __init__(self, hidden_size: int, num_heads: int, head_dim: int, rotary_head_dim: int, v_head_dim: int,
                 latent_rank: int, scale: float, rotary_base: float, rotary_dims: int, norm_eps: float,
                 output_gate: bool = True):
        if rotary_dims % 2 or rotary_dims > rotary_head_dim:
            raise ValueError(f"{rotary_dims} of {rotary_head_dim} dimensions cannot rotate in pairs")
        self.hidden_size, self.num_heads = int(hidden_size), int(num_heads)
        self.head_dim, self.rot, self.v_head_dim = int(head_dim), int(rotary_head_dim), int(v_head_dim)
        self.rank, self.scale = int(latent_rank), float(scale)
        self.rotary_base, self.rotary_dims = float(rotary_base), int(rotary_dims)
        self.norm_eps, self.output_gate = float(norm_eps), bool(output_gate)
        self.q_size = self.num_heads * (self.head_dim + self.rot)
        self.row = self.rank + self.rot  # a token's cache row, and the size of a head's query in the attention
        if self.row > 512:
            raise ValueError(f"cache rows of {self.row} are larger than the attention kernel takes (512)")
        self._freq = {}

    def tensor_specs(self, prefix):
        H, nh = self.hidden_size, self.num_heads
        specs = [
            TensorSpec(f"{prefix}.q", (self.q_size, H), "matrix"),
            TensorSpec(f"{prefix}.dkv", (self.row, H), "matrix"),
            TensorSpec(f"{prefix}.dkv.norm", (self.rank,), "norm"),
            TensorSpec(f"{prefix}.uk", (nh * self.head_dim, self.rank), "matrix"),
            TensorSpec(f"{prefix}.uv", (nh * self.v_head_dim, self.rank), "matrix"),
        ]
        if self.output_gate:
            specs.append(TensorSpec(f"{prefix}.g", (nh, H), "matrix"))
        return specs + [TensorSpec(f"{prefix}.o", (H, nh * self.v_head_dim), "matrix")]

    def bind(self, tensors, prefix):
        nh = self.num_heads
        parts = [tensors.pop(f"{prefix}.q"), tensors.pop(f"{prefix}.dkv")]
        if self.output_gate:
            parts.append(tensors.pop(f"{prefix}.g"))
        self.in_weight = _fused_rows(parts)  # [q | dkv | gate]
        self.latent_norm = tensors[f"{prefix}.dkv.norm"]
        # per head [K, N]: the key up-projection as stored ([dim, rank]); the value one transposed ([rank, vdim])
        self.uk = tensors.pop(f"{prefix}.uk").reshape(nh, self.head_dim, self.rank).contiguous()
        self.uv = tensors.pop(f"{prefix}.uv").reshape(nh, self.v_head_dim, self.rank).transpose(1, 2).contiguous()
        self.o_weight = tensors[f"{prefix}.o"]

    def cache_need(self):
        # one shared key head; the value is the key's first ``rank`` elements, so no value rows are kept
        return PagedKV(1, self.row, None, 0)

    def _frequencies(self, device):
        key = str(device)
        if key not in self._freq and self.rotary_dims:
            n = self.rotary_dims
            f = [self.rotary_base ** (-2.0 * i / n) for i in range(n // 2)]
            self._freq[key] = torch.tensor(f, dtype=torch.float64).to(torch.float32).to(device)
        return self._freq.get(key)

    def forward(self, x, h, ctx, cache: LayerCache, owns_cache: bool, accumulate: bool = True):
        T = x.shape[0]
        nh, d, r, dv, rank, row = self.num_heads, self.head_dim, self.rot, self.v_head_dim, self.rank, self.row
        ws = ctx.workspace
        meta = ctx.paged[cache.group]
        proj = ws.get("latent_in", (T, self.in_weight.shape[0]), ctx.act_dtype)
        ops.gemm(x, self.in_weight, None, proj)
        q_att = ws.get("latent_queries", (T, nh * row), ctx.act_dtype)
        ops.latent_prepare(proj, 0, self.q_size, self.latent_norm, self.norm_eps, ctx.positions,
                           self._frequencies(proj.device), self.rotary_dims, meta.slot_mapping, cache.k, q_att, nh, d, r,
                           rank, write_kv=owns_cache)
        ops.head_gemm(proj, d + r, self.uk, q_att, row)  # the plain queries through the key up-projection
        mixed = ws.get("latent_mixed", (T, nh * rank), ctx.act_dtype)
        ops.paged_attention(q_att, mixed, cache.k, None, meta.block_tables, ctx, nh, 1, row, 0, self.scale,
                            v_head_dim=rank, values_in_keys=True)
        out = ws.get("latent_out", (T, nh * dv), ctx.act_dtype)
        gate = proj[:, self.q_size + row:self.q_size + row + nh] if self.output_gate else None
        ops.head_gemm(mixed, rank, self.uv, out, dv, gate=gate)
        ops.gemm(out, self.o_weight, None, h, accumulate=accumulate)


register_part("mixer", "latent_attention", LatentAttention)
