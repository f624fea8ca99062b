"""Sequence mixers for ragged, paged inference batches.

``LatentAttention``: attention whose keys and values are linear images of one cached low-rank latent per token plus a
single rotated key part shared by all heads.  Queries go through their own normed latent.  Only ``[c | kr]`` is cached
(``R + dr`` numbers per token and layer instead of ``2 H d``); a layer may also read the cache of an earlier layer
(``kv_from``) and then has no key/value down-projection at all.  Per step:

    d        = h Wd^T                (one packed GEMM: query latent | key/value latent | key rope part)
    cq, cache= norm / rotate / append        (ops.latent_attention.latent_kv_write)
    q        = cq Wuq^T              [T, H, dn + dr]
    ql       = qn Uk_h               [T, H, R]   absorbed queries, fp32
    ol       = attention over the cache rows (ops.latent_attention.latent_attention)   [T, H, R]
    out      = (ol Uv_h^T) Wo^T

Reference: none — the reference has no model code (reference llmctl/runtime/engine.py:119-140)."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, Optional

import torch
import torch.nn as nn

from ..ops import functional as ops
from ..ops import latent_attention as lops
from ..ops.elementwise import rope_frequencies


@dataclass
class LatentAttentionSpec:
    heads: int
    dim: int            # unrotated query/key size per head (dn)
    rot_dim: int        # rotated query/key size per head (dr)
    vdim: int
    kv_rank: int
    q_rank: int
    scale: float
    rot_base: float
    rot_scaling: Optional[Dict[str, Any]] = None
    kv_from: Optional[int] = None       # index of the layer whose cache this layer reads

    @property
    def cache_width(self) -> int:
        return self.kv_rank + self.rot_dim


class LatentAttention(nn.Module):
    def __init__(self, width: int, spec: LatentAttentionSpec, eps: float, dtype, device):
        super().__init__()
        s = self.spec = spec
        self.eps = eps
        own = s.kv_from is None
        kw = dict(dtype=dtype, device=device)
        rows = s.q_rank + (s.kv_rank + s.rot_dim if own else 0)
        self.w_down = nn.Parameter(torch.empty(rows, width, **kw))                      # [dq ; dkv]
        self.q_norm = nn.Parameter(torch.ones(s.q_rank, **kw))
        self.kv_norm = nn.Parameter(torch.ones(s.kv_rank, **kw)) if own else None
        self.w_uq = nn.Parameter(torch.empty(s.heads * (s.dim + s.rot_dim), s.q_rank, **kw))
        self.w_uk = nn.Parameter(torch.empty(s.heads, s.dim, s.kv_rank, **kw))          # per head [dn, R]
        self.w_uv = nn.Parameter(torch.empty(s.heads, s.vdim, s.kv_rank, **kw))         # per head [dv, R]
        self.w_o = nn.Parameter(torch.empty(width, s.heads * s.vdim, **kw))
        f, self.rot_mult = rope_frequencies(s.rot_dim, s.rot_base, s.rot_scaling)
        self.register_buffer("rot_freq", f.to(device), persistent=False)

    def load(self, get, prefix: str) -> None:
        s = self.spec
        with torch.no_grad():
            parts = [get(prefix + "dq")] + ([get(prefix + "dkv")] if s.kv_from is None else [])
            self.w_down.copy_(torch.cat(parts, dim=0))
            self.q_norm.copy_(get(prefix + "dq.norm"))
            if s.kv_from is None:
                self.kv_norm.copy_(get(prefix + "dkv.norm"))
            self.w_uq.copy_(get(prefix + "uq"))
            self.w_uk.copy_(get(prefix + "uk").view(s.heads, s.dim, s.kv_rank))
            self.w_uv.copy_(get(prefix + "uv").view(s.heads, s.vdim, s.kv_rank))
            self.w_o.copy_(get(prefix + "o"))

    def forward(self, h: torch.Tensor, batch, cache: torch.Tensor) -> torch.Tensor:
        """h: [T, W] in the activation type; ``cache``: this layer's (or its source layer's) [blocks, bs, R + dr]."""
        s = self.spec
        T = h.shape[0]
        own = s.kv_from is None
        d = ops.linear(h, self.w_down)
        cq = lops.latent_kv_write(d, s.q_rank, s.kv_rank if own else 0, s.rot_dim if own else 0, self.q_norm, self.kv_norm,
                                  cache if own else None, batch.slots, batch.positions, self.rot_freq, self.rot_mult, self.eps)
        q = ops.linear(cq, self.w_uq)                                                   # [T, H * (dn + dr)]
        qn = q.view(T, s.heads, s.dim + s.rot_dim)[:, :, :s.dim].transpose(0, 1)        # [H, T, dn], a view
        # absorbed queries ql[t, h] = Uk_h^T qn[t, h]: fp32, except that the tensor-core attention kernel takes them
        # in bf16 (it multiplies in bf16 anyway); the kernel reads the [H, T, R] product through its strides
        if q.is_cuda and q.dtype == torch.bfloat16:
            if lops.uses_tensor_cores(q.dtype, s.kv_rank, s.rot_dim):
                ql = torch.bmm(qn, self.w_uk)
            else:
                ql = torch.bmm(qn, self.w_uk, out_dtype=torch.float32)
        else:
            ql = torch.bmm(qn.float(), self.w_uk.float())
        ql = ql.transpose(0, 1)
        # batches with prompt portions fill the tcgen05 kernel's 128-row tiles; a decoding token has only its heads to
        # offer, and the 16 / 32-row kernel reads the cache once for them
        if not batch.decode_only and lops.uses_tcgen05(q.dtype, s.kv_rank, s.rot_dim, cache.shape[1], q.is_cuda):
            rows = lops.ROWS_PER_TILE_TCGEN05
        else:
            rows = lops.rows_per_tile(q.dtype, s.kv_rank, s.rot_dim, q.is_cuda, s.heads if batch.decode_only else lops.ROWS_PER_TILE_WIDE)
        ol = lops.latent_attention(ql, q, s.dim, cache, batch.block_tables, batch.tiles(rows), batch.positions,
                                   self.rot_freq, self.rot_mult, s.scale, batch.heads_per_tile(s.heads, rows), batch.max_context,
                                   batch.attention_splits(s.heads, rows), rows=rows)
        o = torch.bmm(ol.transpose(0, 1), self.w_uv.transpose(1, 2)).transpose(0, 1).reshape(T, s.heads * s.vdim)
        return ops.linear(o, self.w_o)
