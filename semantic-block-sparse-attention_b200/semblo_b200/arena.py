"""Fixed-address decode state of one layer (mirror of semblo/vllm_plugin/arena.py:66-253):
capacity-shaped index buffers, the suffix store addressed by absolute position through a
block table, and the adoption of a request's freshly built index."""
from __future__ import annotations

import os

import torch

from .flat_index import flat_cluster_count
from .state import _PACK_ALIGN, ProductPostingIndex


def arena_cluster_count(capacity: int, unit_tokens: int, min_clusters_log2: int) -> int:
    """arena.py:42-47."""
    raw_c = flat_cluster_count(int(capacity), int(unit_tokens))
    num_clusters = 1 << max(int(min_clusters_log2), (max(raw_c, 1) - 1).bit_length())
    return int(min(num_clusters, 1 << (int(capacity).bit_length() - 1)))


def full_graph_decode_enabled() -> bool:
    """arena.py:38-39."""
    return os.environ.get("SEMBLO_FULL_GRAPH_DECODE") == "1"


def suffix_reserve(room: int | None = None) -> int:
    """arena.py:50-63: positions reserved for the generated suffix."""
    env = os.environ.get("SEMBLO_SUFFIX_RESERVE")
    if env is not None:
        return int(env)
    if room is not None:
        return max(1, min(65536, int(room)))
    return 65536


class DecodeArena:
    """Capacity-shaped buffers for one source layer and an index object over them
    (arena.py:66-140).  ``state`` (a SembloRuntimeState, or None) supplies engine-lifetime
    buffers through ``pooled_buffer`` so that every request of a layer sees the same
    addresses; without it the arena owns its tensors."""

    def __init__(self, state=None, layer: int = 0, *, capacity: int, num_kv_heads: int, head_dim: int,
                 index_dim: int | None = None, num_clusters: int, page_align: int,
                 kv_dtype: torch.dtype = torch.bfloat16, desc_dtype: torch.dtype | None = None, device,
                 suffix_block: int = 256, packed_capacity: int | None = None,
                 table_positions: int | None = None, keep_kpre: bool = False,
                 reserve: int | None = None) -> None:
        self.state = state
        self.layer = int(layer)
        self.capacity = int(capacity)
        self.num_clusters = int(num_clusters)
        self.reserve = int(reserve) if reserve is not None else suffix_reserve()
        self.suffix_block = int(suffix_block)
        self.packed_capacity = int(packed_capacity if packed_capacity is not None else capacity)
        self.page_align = max(int(page_align), 1)
        index_dim = int(head_dim if index_dim is None else index_dim)
        desc_dtype = kv_dtype if desc_dtype is None else desc_dtype
        if kv_dtype != torch.bfloat16 or desc_dtype != torch.bfloat16:
            raise ValueError("the decode arena holds bf16 K/V and bf16 descriptors")
        width = self.packed_capacity + self.num_clusters * self.page_align
        self.width = width + (-width) % _PACK_ALIGN
        device = torch.device(device)
        fresh = [True]

        def buf(name, shape, dtype, shared=False):
            if state is None:
                return torch.zeros(*shape, dtype=dtype, device=device)
            key = f"arena:{name}" if shared else f"arena:{self.layer}:{name}"
            known = key in state.index_buffers
            t = state.pooled_buffer(key, shape, dtype, device)
            if not known:
                t.zero_()
            else:
                fresh[0] = False
            return t

        i32 = torch.int32
        self.posting = buf("posting_positions", (num_kv_heads, self.width), i32)
        self.sizes = buf("bucket_sizes", (num_kv_heads, self.num_clusters), i32)
        self.indptr = buf("bucket_indptr", (num_kv_heads, self.num_clusters + 1), i32)
        self.codebooks = buf("codebooks", (num_kv_heads, 2, self.num_clusters, index_dim // 2), desc_dtype)
        self.packed_kv = buf("packed_kv", (2, self.width, num_kv_heads, head_dim), kv_dtype)
        self.prompt_length_t = buf("prompt_length", (1,), i32)
        self.suffix_blocks = self.reserve // self.suffix_block + 1
        self.suffix_kv = buf("suffix_kv", (2, self.suffix_blocks, self.suffix_block, num_kv_heads, head_dim), kv_dtype)
        span = int(table_positions if table_positions is not None else self.capacity + self.reserve)
        self.suffix_table = buf("suffix_block_table", (1, -(-span // self.suffix_block) + 1), i32, shared=True)
        self.suffix_kpre = (buf("suffix_kpre", (self.suffix_blocks, self.suffix_block, num_kv_heads, head_dim), kv_dtype)
                            if keep_kpre else None)
        if fresh[0]:
            # the one-token warm-up index (arena.py:102-113): cluster 0 of every head holds position 0
            self.sizes[:, 0] = 1
            self.indptr[:, 1:] = 1
            self.prompt_length_t.fill_(self.capacity)
        self.suffix_base = -1
        self.table_filled = 0
        self.adopted_epoch = None
        self.fused_decode_ws = None
        self.index = ProductPostingIndex(codebooks=self.codebooks, posting_positions=self.posting,
                                         bucket_indptr=self.indptr, bucket_sizes=self.sizes,
                                         prompt_length=self.capacity, max_position=self.capacity,
                                         flat_clusters=self.num_clusters)
        self.index.packed_kv = self.packed_kv
        self.install_suffix_store(self.capacity)

    def install_suffix_store(self, length: int) -> None:
        """arena.py:165-184."""
        base = int(length) // self.suffix_block
        if self.suffix_base != base:
            table = self.suffix_table
            table.zero_()
            n = max(0, min(self.suffix_blocks, int(table.shape[1]) - base))
            table[0, base:base + n] = torch.arange(n, dtype=torch.int32, device=table.device)
            self.suffix_base = base
            self.table_filled = base + n

    def extend_suffix_table(self, upto_position: int) -> None:
        """arena.py:186-203: ring mapping (block - base) mod NBLK."""
        last = int(upto_position) // self.suffix_block
        table = self.suffix_table
        if last >= int(table.shape[1]):
            raise RuntimeError(f"position {upto_position} is beyond the suffix block table ({int(table.shape[1])} blocks)")
        if last >= self.table_filled:
            blocks = torch.arange(self.table_filled, last + 1, device=table.device)
            table[0, self.table_filled:last + 1] = ((blocks - self.suffix_base) % self.suffix_blocks).to(torch.int32)
            self.table_filled = last + 1

    def adopt(self, index: ProductPostingIndex, epoch: int | None = None) -> ProductPostingIndex:
        """arena.py:216-253: copy a request's index into the fixed-address buffers (once per
        ``epoch`` when one is given)."""
        if epoch is not None and self.adopted_epoch == epoch:
            return self.index
        length = int(index.prompt_length)
        clusters = int(index.num_buckets)
        width = int(index.posting_positions.shape[1])
        if length > self.capacity or clusters > self.num_clusters or width > self.width:
            raise RuntimeError(f"decode arena holds {self.capacity} tokens ({self.width} posting slots) and "
                               f"{self.num_clusters} clusters; the request has {length} tokens ({width} slots) "
                               f"and {clusters}")
        self.posting[:, :width].copy_(index.posting_positions)
        self.sizes.zero_()
        self.sizes[:, :clusters].copy_(index.bucket_sizes)
        self.indptr[:, :clusters + 1].copy_(index.bucket_indptr)
        if clusters < self.num_clusters:
            self.indptr[:, clusters + 1:].copy_(index.bucket_indptr[:, -1:].expand(-1, self.num_clusters - clusters))
        self.codebooks.zero_()
        self.codebooks[:, :, :clusters].copy_(index.codebooks)
        if index.packed_kv is None:
            raise RuntimeError("the decode arena needs the cluster-ordered K/V copy (pack_prompt_kv)")
        packed_len = int(index.packed_kv.shape[1])
        if packed_len > self.width:
            raise RuntimeError(f"packed K/V of {packed_len} rows does not fit the arena's {self.width}")
        if index.packed_kv.data_ptr() != self.packed_kv.data_ptr():
            self.packed_kv[:, :packed_len].copy_(index.packed_kv)
        self.index.prompt_length = length
        self.index.max_position = length
        self.prompt_length_t.fill_(length)
        self.install_suffix_store(length)
        self.adopted_epoch = epoch
        return self.index


def arena_for(state, layer: int, *, capacity: int, unit_tokens: int, min_clusters_log2: int,
              num_kv_heads: int, head_dim: int, index_dim: int, page_align: int,
              kv_dtype: torch.dtype, desc_dtype: torch.dtype, device,
              packed_capacity: int | None = None, table_positions: int | None = None,
              keep_kpre: bool = False, reserve: int | None = None) -> DecodeArena:
    """The layer's arena, made on first use (arena.py:256-274)."""
    key = ("arena", int(layer))
    arena = state.index_buffers.get(key)
    if arena is None:
        arena = DecodeArena(state, layer, capacity=capacity, num_kv_heads=num_kv_heads, head_dim=head_dim,
                            index_dim=index_dim,
                            num_clusters=arena_cluster_count(capacity, unit_tokens, min_clusters_log2),
                            page_align=page_align, kv_dtype=kv_dtype, desc_dtype=desc_dtype, device=device,
                            suffix_block=int(getattr(state, "suffix_block_size", 256)),
                            packed_capacity=packed_capacity, table_positions=table_positions,
                            keep_kpre=keep_kpre, reserve=reserve)
        state.index_buffers[key] = arena
    return arena
