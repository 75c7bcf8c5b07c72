"""Fixed-address decode state of one layer (mirror of semblo/vllm_plugin/arena.py:66-253):
capacity-shaped index buffers, the suffix store addressed by absolute position through a
block table, and the adoption of a request's freshly built index."""
from __future__ import annotations

import torch

from .flat_index import flat_cluster_count
from .state import _PACK_ALIGN, ProductPostingIndex


def arena_cluster_count(capacity: int, unit_tokens: int, min_clusters_log2: int) -> int:
    """arena.py:42-47."""
    raw_c = flat_cluster_count(int(capacity), int(unit_tokens))
    num_clusters = 1 << max(int(min_clusters_log2), (max(raw_c, 1) - 1).bit_length())
    return int(min(num_clusters, 1 << (int(capacity).bit_length() - 1)))


class DecodeArena:
    def __init__(self, *, capacity: int, num_kv_heads: int, head_dim: int, num_clusters: int, page_align: int,
                 device, reserve: int, suffix_block: int = 256, packed_capacity: int | None = None,
                 table_positions: int | None = None, keep_kpre: bool = False,
                 kv_dtype=torch.bfloat16) -> None:
        self.capacity = int(capacity)
        self.num_clusters = int(num_clusters)
        self.reserve = int(reserve)
        self.suffix_block = int(suffix_block)
        self.packed_capacity = int(packed_capacity if packed_capacity is not None else capacity)
        self.page_align = max(int(page_align), 1)
        width = self.packed_capacity + self.num_clusters * self.page_align
        self.width = width + (-width) % _PACK_ALIGN
        i32 = dict(dtype=torch.int32, device=device)
        self.posting = torch.zeros(num_kv_heads, self.width, **i32)
        self.sizes = torch.zeros(num_kv_heads, self.num_clusters, **i32)
        self.indptr = torch.zeros(num_kv_heads, self.num_clusters + 1, **i32)
        self.codebooks = torch.zeros(num_kv_heads, 2, self.num_clusters, head_dim // 2, dtype=kv_dtype, device=device)
        self.packed_kv = torch.zeros(2, self.width, num_kv_heads, head_dim, dtype=kv_dtype, device=device)
        # the one-token warm-up index (arena.py:102-113)
        self.sizes[:, 0] = 1
        self.indptr[:, 1:] = 1
        self.prompt_length_t = torch.full((1,), self.capacity, **i32)
        self.suffix_blocks = self.reserve // self.suffix_block + 1
        self.suffix_kv = torch.zeros(2, self.suffix_blocks, self.suffix_block, num_kv_heads, head_dim,
                                     dtype=kv_dtype, device=device)
        span = int(table_positions if table_positions is not None else self.capacity + self.reserve)
        self.suffix_table = torch.zeros(1, -(-span // self.suffix_block) + 1, **i32)
        self.suffix_kpre = (torch.zeros(self.suffix_blocks, self.suffix_block, num_kv_heads, head_dim,
                                        dtype=kv_dtype, device=device) if keep_kpre else None)
        self.suffix_base = -1
        self.table_filled = 0
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

    def adopt(self, index: ProductPostingIndex) -> ProductPostingIndex:
        """arena.py:216-253: copy a request's index into the fixed-address buffers."""
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
        return self.index
