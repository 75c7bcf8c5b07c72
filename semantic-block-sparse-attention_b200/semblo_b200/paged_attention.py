"""Attention over a vLLM-style paged KV cache through a block table, and the exact merge of two
attention states: the live half of semblo/vllm_plugin/paged_attention.py
(PostingTiles 37-41, PagedSparseAttentionResult 44-47, merge_paged_attention_results 50-78,
paged_posting_attention 961-1128).  The decode path without an arena reads the generated
suffix this way and merges it with the sparse attention over the prompt."""
from __future__ import annotations

from dataclasses import dataclass

import torch

from . import _lib
from ._lib import check, lib, ptr, require_cuda, stream_ptr


@dataclass(frozen=True)
class PostingTiles:
    starts: torch.Tensor            # [Q, Hkv, T] offsets into posting_positions[Hkv]
    lengths: torch.Tensor           # [Q, Hkv, T]
    counts: torch.Tensor            # [Q, Hkv]
    selected_tokens: torch.Tensor   # [Q, Hkv]


@dataclass(frozen=True)
class PagedSparseAttentionResult:
    output: torch.Tensor            # [Q, Hq, D]
    logsumexp: torch.Tensor | None  # [Q, Hq]


def merge_paged_attention_results(left: PagedSparseAttentionResult,
                                  right: PagedSparseAttentionResult) -> PagedSparseAttentionResult:
    """Exactly merge attention computed over two disjoint key sets (both need their log-sum-exp)."""
    if left.logsumexp is None or right.logsumexp is None:
        raise ValueError("attention-state merge requires logsumexp from both inputs")
    if left.output.shape != right.output.shape:
        raise ValueError("attention outputs must have identical shapes")
    if left.logsumexp.shape != right.logsumexp.shape:
        raise ValueError("attention logsumexp tensors must have identical shapes")
    require_cuda(left.output, right.output)
    if left.output.dtype != torch.bfloat16 or right.output.dtype != torch.bfloat16:
        raise ValueError("attention outputs are bf16")
    a, b = left.output.contiguous(), right.output.contiguous()
    la, lb = left.logsumexp.float().contiguous(), right.logsumexp.float().contiguous()
    out = torch.empty_like(a)
    lse = torch.empty_like(la)
    rows = la.numel()
    check(lib().semblo_merge_attention_states(ptr(a), ptr(la), ptr(b), ptr(lb), rows, int(a.shape[-1]), ptr(out), ptr(lse),
                                              stream_ptr()))
    return PagedSparseAttentionResult(output=out, logsumexp=lse)


_WORKSPACES: dict = {}


def _workspace(device, hq: int, hkv: int, dim: int, splits: int) -> torch.Tensor:
    key = (torch.device(device).index, hq, hkv, dim, splits)
    ws = _WORKSPACES.get(key)
    if ws is None:
        ws = torch.zeros(int(lib().semblo_paged_attention_workspace_bytes(hq, hkv, dim, splits)), dtype=torch.uint8,
                         device=device)
        _WORKSPACES[key] = ws
    return ws


def paged_posting_attention(q: torch.Tensor, kv_cache: torch.Tensor, posting_positions: torch.Tensor,
                            tiles: PostingTiles, query_positions: torch.Tensor, query_request_ids: torch.Tensor,
                            block_table: torch.Tensor, *, block_size: int, sm_scale: float,
                            softcap: float | None = None, token_tile: int = 16, num_splits: int = 1,
                            return_logsumexp: bool = False) -> PagedSparseAttentionResult:
    """Attention of each query over the positions its posting tiles list, kept where the position is at
    or before the query's own, read from ``kv_cache`` [2, blocks, block, Hkv, D] through the block table.
    One request (a batch-1 block table), as the reference's integration; no logit soft cap."""
    require_cuda(q, kv_cache, posting_positions, block_table)
    if q.ndim != 3:
        raise ValueError("q must have shape [Q,Hq,D]")
    if kv_cache.ndim != 5 or kv_cache.shape[0] != 2:
        raise ValueError("vLLM KV cache must have shape [2,num_blocks,block,Hkv,D]")
    if posting_positions.ndim != 2:
        raise ValueError("posting_positions must have shape [Hkv,L]")
    q_count, num_q_heads, head_dim = map(int, q.shape)
    num_kv_heads = int(kv_cache.shape[3])
    if posting_positions.shape[0] != num_kv_heads:
        raise ValueError("posting KV-head count differs from the cache")
    if num_q_heads % num_kv_heads:
        raise ValueError("query heads must be divisible by KV heads")
    if query_positions.shape != (q_count,) or query_request_ids.shape != (q_count,):
        raise ValueError("query metadata must have shape [Q]")
    if block_table.ndim != 2 or block_table.shape[0] != 1:
        raise ValueError("one request at a time: the block table must have shape [1, blocks]")
    if int(kv_cache.shape[2]) != int(block_size):
        raise ValueError("block_size does not match the vLLM cache")
    if int(kv_cache.shape[-1]) != head_dim:
        raise ValueError("KV-cache head dimension differs from q")
    if token_tile not in {8, 16, 32}:
        raise ValueError("token_tile must be 8, 16, or 32")
    if softcap:
        raise RuntimeError("paged posting attention has no logit soft cap here")
    if q.dtype != torch.bfloat16 or kv_cache.dtype != torch.bfloat16 or not kv_cache.is_contiguous():
        raise ValueError("q and a contiguous KV cache in bf16 are required")
    q = q.contiguous()
    post = posting_positions if posting_positions.stride(1) == 1 else posting_positions.contiguous()
    post = post.to(torch.int32) if post.dtype != torch.int32 else post
    table = block_table.to(torch.int32) if block_table.dtype != torch.int32 else block_table
    table = table.contiguous()
    starts, lengths, counts = (t.to(torch.int32).contiguous() for t in (tiles.starts, tiles.lengths, tiles.counts))
    positions = query_positions if query_positions.dtype in (torch.int32, torch.int64) else query_positions.to(torch.int32)
    output = torch.empty_like(q)
    lse = torch.empty(q_count, num_q_heads, dtype=torch.float32, device=q.device)
    splits = max(1, int(num_splits))
    ws = _workspace(q.device, num_q_heads, num_kv_heads, head_dim, splits)
    status = _lib.status_for(q.device)
    item = positions.element_size()
    for i in range(q_count):
        check(lib().semblo_paged_posting_attention(
            ptr(q[i]), positions.data_ptr() + i * item, 1 if positions.dtype == torch.int64 else 0, ptr(kv_cache),
            int(kv_cache.shape[1]), int(block_size), ptr(table), int(table.shape[1]), ptr(post), int(post.stride(0)),
            ptr(starts[i]), ptr(lengths[i]), ptr(counts[i]), int(starts.shape[2]), int(token_tile), num_q_heads,
            num_kv_heads, head_dim, float(sm_scale), splits, ptr(ws), ws.numel(), ptr(output[i]), ptr(lse[i]),
            ptr(status.word), stream_ptr()))
    return PagedSparseAttentionResult(output, lse if return_logsumexp else None)
