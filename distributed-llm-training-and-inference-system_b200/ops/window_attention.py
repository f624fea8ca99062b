"""Sliding-window attention with pooled far context over a paged cache — csrc/attention/pooled_window_attention.cu.

A query at position i sees the tokens j with ``0 <= i - j < S`` and one pooled key/value (the mean of the cached keys /
values) per block of P tokens that lies wholly before its window.  A layer's cache is ``[pages, bs + PS, G (d + e)]``:
``bs`` token rows ``[keys | values]`` per page, then the ``PS = ceil(bs / P)`` pooled rows of the blocks that start in
the page.  ``window_qkv_write`` post-processes the packed projection (bias, whole-projection RMS norm of q and k,
partial interleaved rotation, value mixing with an earlier layer's values) and appends to the cache;
``window_pool_update`` writes the pooled rows of the blocks a step completes; ``pooled_window_attention`` is the
attention itself, with per-head score temperatures and mixing of the normalised weights across heads.  CPU tensors run
the PyTorch restatement below (CPU tests); on a GPU a missing kernel raises.

Reference: none — the reference has no attention code (reference llmctl/serve/server.py:199-204)."""
from __future__ import annotations

import os
from typing import Optional

import torch

from . import native
from .elementwise import _is32, rotate_interleaved

c_void_p, c_int, c_ll, c_float = native.c_void_p, native.c_int, native.c_ll, native.c_float
native.register_signature("llmctl_window_qkv_write", [c_void_p, c_ll, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int,
                                                       c_void_p, c_float, c_float, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int,
                                                       c_void_p, c_int, c_void_p, c_int, c_int, c_void_p])
native.register_signature("llmctl_window_pool_update", [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int,
                                                         c_int, c_int, c_int, c_void_p])
native.register_signature("llmctl_pooled_window_attention_rows", [c_int, c_int, c_int, c_int])
native.register_signature("llmctl_pooled_window_attention_mma_ok", [c_int, c_int, c_int, c_int, c_int])
native.register_signature("llmctl_pooled_window_attention_mma", [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_void_p,
                                                                  c_void_p, c_void_p, c_float, c_int, c_int, c_int, c_int, c_int, c_int,
                                                                  c_int, c_int, c_void_p, c_int, c_int, c_void_p, c_void_p, c_void_p])
native._KERNELS_PER_CALL["llmctl_pooled_window_attention_mma"] = 1
native.register_signature("llmctl_pooled_window_attention", [c_void_p, c_void_p, c_void_p, c_int, c_void_p, c_int, c_int, c_void_p,
                                                              c_void_p, c_void_p, c_float, c_int, c_int, c_int, c_int, c_int, c_int,
                                                              c_int, c_int, c_void_p, c_int, c_void_p])


def pooled_rows_per_page(block_size: int, pool: int) -> int:
    """Pooled rows a page needs: the blocks of ``pool`` tokens whose first token lies in it (0 without pooling)."""
    return (block_size + pool - 1) // pool if pool else 0


def _pooled_row(table, b: int, P: int, bs: int, PS: int) -> int:
    page = (b * P) // bs
    first_b = (page * bs + P - 1) // P
    return int(table[page]) * (bs + PS) + bs + (b - first_b)


def _token_row(table, j: int, bs: int, PS: int) -> int:
    return int(table[j // bs]) * (bs + PS) + j % bs


def window_qkv_write(qkv: torch.Tensor, bias: Optional[torch.Tensor], qn_w: Optional[torch.Tensor], kn_w: Optional[torch.Tensor],
                     H: int, G: int, d: int, e: int, rot: int, freq: torch.Tensor, mult: float, eps: float,
                     positions: torch.Tensor, slots: torch.Tensor, cache: torch.Tensor, block_size: int,
                     v_first: Optional[torch.Tensor] = None, v_mode: int = 0, lam: Optional[torch.Tensor] = None) -> torch.Tensor:
    """qkv: [T, H d + G d + G e] packed projection WITHOUT bias; bias: same width or None; qn_w / kn_w: fp32 weights of
    the RMS norm over the whole q / k projection (None = no norm); rot: rotated numbers per head.  ``v_mode`` 1 stores
    this layer's values in ``v_first`` [T, G e]; 2 caches ``(1 - lam) v + lam v_first``.  Returns q: fp32 [T, H d];
    writes ``[k | v]`` into ``cache`` ([pages, bs + PS, G (d + e)]) at ``slots`` (int64, page * bs + offset; negative =
    skip)."""
    T = qkv.shape[0]
    bs, PS = block_size, cache.shape[1] - block_size
    Nq, Nk, Nv = H * d, G * d, G * e
    if qkv.is_cuda:
        assert qkv.stride(1) == 1 and cache.is_contiguous() and cache.dtype == qkv.dtype
        q = torch.empty(T, Nq, dtype=torch.float32, device=qkv.device)
        native.call("llmctl_window_qkv_write", qkv.data_ptr(), qkv.stride(0), native.ptr(bias), native.ptr(qn_w), native.ptr(kn_w),
                    H, G, d, e, rot, native.ptr(freq), float(mult), float(eps), positions.data_ptr(), slots.data_ptr(), q.data_ptr(),
                    cache.data_ptr(), bs, PS, native.ptr(v_first), int(v_mode), native.ptr(lam), T, _is32(qkv), native.stream_ptr())
        return q
    f = qkv.float()
    if bias is not None:
        f = f + bias.float()

    def norm(v, w):
        return v if w is None else v / torch.sqrt(v.pow(2).mean(-1, keepdim=True) + eps) * w.float()
    q = norm(f[:, :Nq], qn_w).reshape(T, H, d).clone()
    k = norm(f[:, Nq:Nq + Nk], kn_w).reshape(T, G, d).clone()
    if rot:
        q[..., :rot] = rotate_interleaved(q[..., :rot], positions, freq, mult)
        k[..., :rot] = rotate_interleaved(k[..., :rot], positions, freq, mult)
    v = f[:, Nq + Nk:].to(qkv.dtype)
    if v_mode == 1:
        v_first.copy_(v)
    v = v.float()
    if v_mode == 2:
        l = lam.float().reshape(())
        v = (1.0 - l) * v + l * v_first.float()
    ok = slots >= 0
    rows = (slots // bs) * (bs + PS) + slots % bs
    cache.view(-1, Nk + Nv)[rows[ok]] = torch.cat([k.reshape(T, Nk), v], dim=-1)[ok].to(cache.dtype)
    return q.reshape(T, Nq)


def window_pool_update(cache: torch.Tensor, positions: torch.Tensor, slots: torch.Tensor, seq_rows: torch.Tensor,
                       block_tables: torch.Tensor, block_size: int, pool: int) -> None:
    """For every token of the step that ends a block of ``pool`` positions (and has a cache slot): the mean of the block's
    cached rows goes to the block's pooled row.  seq_rows: int32 [T], row of ``block_tables`` of each token."""
    if not pool:
        return
    T = positions.numel()
    bs, PS, Wc = block_size, cache.shape[1] - block_size, cache.shape[2]
    assert PS == pooled_rows_per_page(bs, pool)
    if cache.is_cuda:
        native.call("llmctl_window_pool_update", cache.data_ptr(), positions.data_ptr(), slots.data_ptr(), seq_rows.data_ptr(),
                    block_tables.data_ptr(), block_tables.shape[1], bs, PS, pool, Wc, T, _is32(cache), native.stream_ptr())
        return
    flat = cache.view(-1, Wc)
    for t in range(T):
        p = int(positions[t])
        if int(slots[t]) < 0 or (p + 1) % pool:
            continue
        table = block_tables[int(seq_rows[t])]
        b = p // pool
        rows = [_token_row(table, j, bs, PS) for j in range(b * pool, p + 1)]
        flat[_pooled_row(table, b, pool, bs, PS)] = (flat[rows].float().sum(0) / pool).to(cache.dtype)


def attention_rows(H: int, d: int, e: int, tile_tokens: int) -> int:
    """Tokens a CTA of the attention kernel takes at these sizes (same rule as llmctl_pooled_window_attention_rows)."""
    return int(native.lib().llmctl_pooled_window_attention_rows(H, d, e, tile_tokens))


def uses_tensor_cores(dtype: torch.dtype, H: int, G: int, d: int, e: int, tile_tokens: int) -> bool:
    """bf16 caches whose sizes fit the mma.sync kernel (d a multiple of 16, e of 8, H e <= 2048, shared memory) run on
    it; fp32 and other sizes run the FMA kernel.  Same rule as llmctl_pooled_window_attention_mma_ok."""
    if dtype != torch.bfloat16 or not native.has_symbol("llmctl_pooled_window_attention_mma"):
        return False
    if os.environ.get("LLMCTL_WINDOW_ATTENTION", "") == "fma":         # ablation switch: the FMA kernel for bf16 too
        return False
    return bool(native.lib().llmctl_pooled_window_attention_mma_ok(H, G, d, e, tile_tokens))


def key_splits(ntiles: int, max_context: int, window: int, pool: int, sms: int = 148) -> int:
    """Slices to cut every tile's keys into on the tensor-core kernel: with few tiles (a decoding batch) and long
    contexts the keys are spread over about two CTAs per SM, at least 64 keys per slice."""
    if not max_context:
        return 1
    keys = min(max_context, window) + (max(max_context - window, 0) // pool if pool else 0) if window else max_context
    return int(max(1, min(2 * sms // max(ntiles, 1), keys // 64, 32)))


def pooled_window_attention(q: torch.Tensor, cache: torch.Tensor, block_tables: torch.Tensor, tiles: torch.Tensor,
                            tile_tokens: int, positions: torch.Tensor, temp: Optional[torch.Tensor], talk: Optional[torch.Tensor],
                            scale: float, H: int, G: int, d: int, e: int, window: int, pool: int, block_size: int,
                            out_dtype: torch.dtype, tensor_cores: bool = True, max_context: int = 0, splits: int = 0) -> torch.Tensor:
    """q: fp32 [T, H d] (normed, rotated); tiles: int32 [n, 4] = (first token row, tokens <= tile_tokens, block-table
    row, 0), the tokens of a tile being consecutive positions of one sequence; temp: fp32 [H] or None; talk: fp32 [H, H]
    or None; window 0 = every earlier token and no pooled blocks.  ``tensor_cores`` False forces the FMA kernel;
    ``max_context`` (longest context in the batch) lets the tensor-core kernel split the keys when tiles are few.
    Returns [T, H e] in ``out_dtype``."""
    T = q.shape[0]
    bs, PS = block_size, cache.shape[1] - block_size
    window = min(int(window), 1 << 30)            # position + window stays inside int32 in the kernels
    if q.is_cuda:
        assert q.dtype == torch.float32 and q.is_contiguous() and cache.is_contiguous() and cache.dtype == out_dtype
        out = torch.empty(T, H * e, dtype=out_dtype, device=q.device)
        if tensor_cores and uses_tensor_cores(cache.dtype, H, G, d, e, tile_tokens):
            n = tiles.shape[0]
            if not splits:
                splits = key_splits(n, max_context, window, pool)
            part_ml = torch.empty(n * splits * H * 32, dtype=torch.float32, device=q.device) if splits > 1 else None
            part_o = torch.empty(splits * T * H * e, dtype=torch.float32, device=q.device) if splits > 1 else None
            native.call("llmctl_pooled_window_attention_mma", q.data_ptr(), cache.data_ptr(), block_tables.data_ptr(),
                        block_tables.shape[1], tiles.data_ptr(), n, int(tile_tokens), positions.data_ptr(), native.ptr(temp),
                        native.ptr(talk), float(scale), H, G, d, e, int(window), int(pool), bs, PS, out.data_ptr(), int(splits), T,
                        native.ptr(part_ml), native.ptr(part_o), native.stream_ptr())
            return out
        native.call("llmctl_pooled_window_attention", q.data_ptr(), cache.data_ptr(), block_tables.data_ptr(), block_tables.shape[1],
                    tiles.data_ptr(), tiles.shape[0], int(tile_tokens), positions.data_ptr(), native.ptr(temp), native.ptr(talk),
                    float(scale), H, G, d, e, int(window), int(pool), bs, PS, out.data_ptr(), _is32(cache), native.stream_ptr())
        return out
    out = torch.zeros(T, H * e, dtype=torch.float32)
    flat = cache.view(-1, cache.shape[2]).float()
    rep = H // G
    qh = q.view(T, H, d)
    for t0, n, seq, _ in tiles.tolist():
        table = block_tables[seq]
        for t in range(t0, t0 + n):
            i = int(positions[t])
            rows = []
            if window:
                rows += [_pooled_row(table, b, pool, bs, PS) for b in range(max(i - window + 1, 0) // pool)]
            rows += [_token_row(table, j, bs, PS) for j in range(max(i - window + 1, 0) if window else 0, i + 1)]
            kv = flat[rows]
            k = kv[:, :G * d].reshape(-1, G, d).repeat_interleave(rep, dim=1)
            v = kv[:, G * d:].reshape(-1, G, e).repeat_interleave(rep, dim=1)
            s = torch.einsum("hd,nhd->hn", qh[t], k) * scale
            if temp is not None:
                s = s * temp.float()[:, None]
            w = torch.softmax(s, -1)
            if talk is not None:
                w = talk.float() @ w
            out[t] = torch.einsum("hn,nhe->he", w, v).reshape(-1)
    return out.to(out_dtype)
