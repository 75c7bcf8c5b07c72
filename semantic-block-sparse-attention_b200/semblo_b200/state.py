"""The request-local index: cluster descriptors, posting lists and the cluster-ordered
K/V copy.  Mirrors the flat-partition half of semblo/vllm_plugin/state.py
(ProductPostingIndex 400-452, build 476-542, _build_flat 544-948, pack_prompt_kv
950-997, inverse_positions 999-1012)."""
from __future__ import annotations

import os
from dataclasses import dataclass
from typing import Any

import torch

from . import flat_index
from ._lib import check, lib, ptr, require_cuda, stream_ptr

_PACK_ALIGN = 256          # state.py:17
HEAD_SEED_STRIDE = 1000003


def _sink_tokens() -> int:
    return int(os.environ.get("SEMBLO_SINK_TOKENS", "0") or "0")


_UNSUPPORTED_ENV = ("SEMBLO_BLOCK_TOKENS", "SEMBLO_FIXED_CODEBOOK",
                    "SEMBLO_FLAT_MIN_TOKENS", "SEMBLO_FLAT_MAX_TOKENS", "SEMBLO_HIER_SPAN",
                    "SEMBLO_PAGE_CLUSTERS", "SEMBLO_FIT_PREFIX_TOKENS")


def _refuse_ablation_flags() -> None:
    """Ablation switches of the reference that this build does not implement raise
    instead of being silently ignored."""
    for name in _UNSUPPORTED_ENV:
        if os.environ.get(name, "0") not in ("", "0"):
            raise RuntimeError(f"{name} is an ablation switch of the reference that this build does not implement")
    if (os.environ.get("SEMBLO_FLAT_INIT", "random") or "random") != "random":
        raise RuntimeError("only SEMBLO_FLAT_INIT=random is implemented")
    if (os.environ.get("SEMBLO_FLAT_METRIC", "cosine") or "cosine") != "cosine":
        raise RuntimeError("only SEMBLO_FLAT_METRIC=cosine is implemented")
    if os.environ.get("SEMBLO_FLAT_DETERMINISTIC", "1") != "1":
        raise RuntimeError("the centroid sums are always deterministic here")


def flat_num_clusters(length: int, target_size: int, min_clusters_log2: int) -> int:
    """state.py:586-602."""
    min_c_log2 = max(3, int(os.environ.get("SEMBLO_FLAT_MIN_CLUSTERS_LOG2", min_clusters_log2)))
    raw_c = flat_index.flat_cluster_count(length, target_size)
    num_clusters = 1 << max(min_c_log2, (max(raw_c, 1) - 1).bit_length())
    num_clusters = min(num_clusters, 1 << (int(length).bit_length() - 1))
    forced = int(os.environ.get("SEMBLO_FLAT_CLUSTERS", "0"))
    return forced if forced > 0 else num_clusters


@dataclass
class ProductPostingIndex:
    codebooks: torch.Tensor            # [Hkv, 2, C, D/2] key dtype
    posting_positions: torch.Tensor    # [Hkv, W'] int32, cluster-major
    bucket_indptr: torch.Tensor        # [Hkv, C+1] int32 (page-aligned starts)
    bucket_sizes: torch.Tensor         # [Hkv, C] int32 (true sizes)
    prompt_length: int
    max_position: int
    packed_kv: torch.Tensor | None = None
    _inverse_positions: torch.Tensor | None = None
    page_align: int = 0
    flat_clusters: int = 0
    orig_bucket: torch.Tensor | None = None      # [Hkv, L] int32 cluster of each position
    original_kv: Any = None
    kv_page_table: torch.Tensor | None = None    # packed row / 16 -> physical page (paged pool)

    @property
    def num_kv_heads(self) -> int:
        return int(self.codebooks.shape[0])

    @property
    def num_buckets(self) -> int:
        return int(self.flat_clusters)

    @property
    def is_flat(self) -> bool:
        return True

    @classmethod
    def build(cls, product_keys: torch.Tensor, positions: torch.Tensor, *, num_centroids: int = 0,
              kmeans_iters: int = 4, kmeans_sample_size: int = 8192, codebook_seed: int | None = None,
              flat_unit_tokens: int = 0, flat_min_clusters_log2: int = 9, page_align: int = 0,
              layer_idx: int | None = None, centroids: list | None = None, num_clusters: int = 0,
              per_head_seed: bool = False, head_offset: int = 0, **unused) -> "ProductPostingIndex":
        """Fit the per-prompt partition and lay out the posting lists (state.py:476-948).

        ``product_keys`` [L, Hkv, I] is the key router's output.  ``centroids`` (one
        fp32 [C or C-1, I] tensor per head) skips the fit: assignment and layout only.
        ``num_clusters`` > 0 fixes the cluster count (as SEMBLO_FLAT_CLUSTERS does).
        ``per_head_seed`` (not a reference mode: the reference draws all heads from one generator in
        order, state.py:520-523, 648) re-seeds the generator for head h with ``codebook_seed +
        HEAD_SEED_STRIDE (head_offset + h)``, so the partition of a head does not depend on which other
        heads this process holds: a KV-head shard then equals the same heads of an unsharded build."""
        require_cuda(product_keys)
        if product_keys.ndim != 3:
            raise ValueError("product_keys must have shape [L,Hkv,I]")
        length, num_kv_heads, index_dim = product_keys.shape
        if positions.shape != (length,):
            raise ValueError("positions must have shape [L]")
        if length == 0:
            raise ValueError("cannot build an index for an empty prompt")
        _refuse_ablation_flags()
        flat_target = int(os.environ.get("SEMBLO_FLAT_UNIT_TOKENS", flat_unit_tokens))
        if flat_target <= 0:
            raise ValueError("the index needs the flat partition: set SEMBLO_FLAT_UNIT_TOKENS or "
                             "semblo_flat_unit_tokens to the mean block size")
        device = product_keys.device
        generator = None
        if codebook_seed is not None:
            generator = torch.Generator(device=device)
            generator.manual_seed(int(codebook_seed))
        num_clusters = int(num_clusters) if num_clusters > 0 else flat_num_clusters(length, flat_target,
                                                                                    flat_min_clusters_log2)
        per_centroid = int(os.environ.get("SEMBLO_FLAT_FIT_PER_C", "32"))
        fit_sample = min(length, max(int(kmeans_sample_size), per_centroid * num_clusters))
        fit_iters = int(os.environ.get("SEMBLO_FLAT_FIT_ITERS", "8"))
        page_align = int(os.environ.get("SEMBLO_FA3_ALIGN", page_align))
        sink = _sink_tokens()
        if sink:
            if sink % 16:
                raise RuntimeError(f"SEMBLO_SINK_TOKENS={sink}: a multiple of 16 keeps the sink cluster page-aligned")
            if length <= sink or length - sink < 2 * num_clusters:
                raise RuntimeError(f"SEMBLO_SINK_TOKENS={sink} leaves too few keys for {num_clusters - 1} clusters")
        half = index_dim // 2
        codebooks = torch.empty(num_kv_heads, 2, num_clusters, half, dtype=torch.bfloat16, device=device)
        assign = torch.empty(num_kv_heads, length, dtype=torch.int32, device=device)
        if per_head_seed and codebook_seed is None:
            raise ValueError("per_head_seed needs a codebook_seed")
        center = os.environ.get("SEMBLO_ROUTING_CENTER") == "1"
        if center and centroids is not None:
            raise RuntimeError("SEMBLO_ROUTING_CENTER re-centres the keys per prompt; given centroids were fitted "
                               "without it")
        for h in range(num_kv_heads):
            if per_head_seed:
                generator.manual_seed(int(codebook_seed) + HEAD_SEED_STRIDE * (int(head_offset) + h))
            keys = product_keys[:, h]
            if center:
                # state.py:649-670 of the reference: keys without a rotary embedding share one dominant
                # direction, and after normalisation k-means would put the prompt in one cluster; taking
                # the prompt's mean key out changes no token's rank under any query
                keys = (keys.float() - keys.float().mean(dim=0, keepdim=True)).to(keys.dtype)
            _, space_f32, space_bf16 = flat_index._normalize_space(keys)
            if sink:
                if centroids is None:
                    rest = flat_index.fit_flat_codebook(
                        space_f32[sink:], space_bf16[sink:], num_clusters - 1, num_iters=fit_iters,
                        sample_size=min(fit_sample, length - sink), generator=generator)
                else:
                    rest = centroids[h].float().contiguous()
                assign[h, :sink].zero_()
                flat_index.assign_flat_buckets(space_bf16[sink:], rest, out=assign[h, sink:], id_offset=1)
                check(lib().semblo_split_descriptor(ptr(rest), num_clusters - 1, 1, num_clusters, index_dim,
                                                    ptr(codebooks[h]), stream_ptr()))
            else:
                if centroids is None:
                    cents = flat_index.fit_flat_codebook(space_f32, space_bf16, num_clusters, num_iters=fit_iters,
                                                         sample_size=fit_sample, generator=generator)
                else:
                    cents = centroids[h].float().contiguous()
                flat_index.assign_flat_buckets(space_bf16, cents, out=assign[h])
                check(lib().semblo_split_descriptor(ptr(cents), num_clusters, 0, num_clusters, index_dim,
                                                    ptr(codebooks[h]), stream_ptr()))
        align = page_align if page_align > 1 else 1
        cap = length + num_clusters * (align - 1)
        cap += (-cap) % _PACK_ALIGN
        posting = torch.empty(num_kv_heads, cap, dtype=torch.int32, device=device)
        indptr = torch.empty(num_kv_heads, num_clusters + 1, dtype=torch.int32, device=device)
        sizes = torch.empty(num_kv_heads, num_clusters, dtype=torch.int32, device=device)
        inverse = torch.empty(num_kv_heads, length, dtype=torch.int32, device=device)
        ws_bytes = int(lib().semblo_layout_workspace_bytes(length, num_kv_heads)) + num_kv_heads * (num_clusters + 1) * 4
        ws = torch.empty(ws_bytes, dtype=torch.uint8, device=device)
        check(lib().semblo_build_layout(ptr(assign), length, num_kv_heads, num_clusters, align, ptr(posting), cap,
                                        ptr(indptr), ptr(sizes), ptr(inverse), ptr(ws), ws_bytes, stream_ptr()))
        # one host read, as the reference's int(ip_pad[-1]): the common posting width
        width = int(indptr[:, -1].max().item())
        index = cls(codebooks=codebooks if product_keys.dtype == torch.bfloat16 else codebooks.to(product_keys.dtype),
                    posting_positions=posting[:, :width], bucket_indptr=indptr, bucket_sizes=sizes,
                    prompt_length=length, max_position=length - 1, page_align=page_align if page_align > 1 else 0,
                    flat_clusters=num_clusters, _inverse_positions=inverse, orig_bucket=assign)
        return index

    def pack_prompt_kv(self, key: torch.Tensor, value: torch.Tensor, *, pool=None,
                       page_table: torch.Tensor | None = None) -> torch.Tensor:
        """state.py:950-997.  With ``page_table`` ([W / 16] int32) the cluster-ordered rows are
        written into 16-row pages of a paged pool in that order (vLLM block-table layout)."""
        require_cuda(key, value)
        if key.shape != value.shape:
            raise ValueError("key and value must have the same shape")
        if key.ndim != 3 or key.shape[0] != self.prompt_length:
            raise ValueError("key and value must have shape [L,Hkv,D]")
        if key.shape[1] != self.num_kv_heads:
            raise ValueError("key and value KV-head count differs from the index")
        if key.dtype != torch.bfloat16:
            raise ValueError("the cluster-ordered copy is bf16")
        width = int(self.posting_positions.shape[1])
        pad = (-width) % _PACK_ALIGN
        shape = (2, width + pad, self.num_kv_heads, key.shape[-1])
        packed = torch.empty(*shape, dtype=key.dtype, device=key.device) if pool is None else pool(shape, key.dtype, key.device)
        k = key if key.is_contiguous() else key.contiguous()
        v = value if value.is_contiguous() else value.contiguous()
        check(lib().semblo_pack_kv(ptr(k), ptr(v), ptr(self.posting_positions), self.posting_positions.stride(0),
                                   width, width + pad, self.num_kv_heads, key.shape[-1], ptr(packed),
                                   packed.stride(0), ptr(page_table), stream_ptr()))
        self.packed_kv = packed
        self.kv_page_table = page_table
        return packed

    def inverse_positions(self) -> torch.Tensor:
        return self._inverse_positions

    # ---- generated suffix (state.py:1000-1128 of the reference) --------------------------------
    def record_generated_positions(self, first_position: int, count: int = 1) -> None:
        """The next ``count`` generated positions, which must continue the sequence.  Tracked on the
        host from the step's first position: no device value is read."""
        expected = int(self.max_position) + 1
        if int(first_position) != expected:
            raise ValueError(f"generated suffix must be contiguous: expected {expected}, got {int(first_position)}")
        self.max_position = expected + int(count) - 1

    def _suffix_position_buffer(self, length: int) -> torch.Tensor:
        """Absolute positions prompt_length, prompt_length + 1, ... over a reservation of the next
        power of two at or above ``length`` (at least 64): made once per size, never rewritten."""
        capacity = 64
        while capacity < int(length):
            capacity *= 2
        buf = getattr(self, "_suffix_positions", None)
        if buf is None or int(buf.numel()) != capacity:
            buf = torch.arange(int(self.prompt_length), int(self.prompt_length) + capacity, dtype=torch.int32,
                               device=self.codebooks.device)
            self._suffix_positions = buf
            self.suffix_tiles = None
        return buf

    def generated_positions(self, device=None) -> torch.Tensor:
        length = int(self.max_position) + 1 - int(self.prompt_length)
        return self._suffix_position_buffer(max(length, 1))[:max(length, 0)]

    def generated_suffix_tiles(self, *, num_kv_heads: int, tile_size: int):
        """Tiles over the whole reservation of the generated suffix: (posting [Hkv, cap], starts,
        lengths [1, Hkv, slots], counts, selected [1, Hkv]).  Nothing in them changes while the suffix
        grows inside its reservation, because the attention kernel keeps a listed position only when
        it is at or before the query's own; the step therefore has no host value that varies."""
        length = int(self.max_position) + 1 - int(self.prompt_length)
        if length <= 0:
            raise ValueError("there is no generated suffix yet")
        buf = self._suffix_position_buffer(length)
        capacity = int(buf.numel())
        slots = -(-capacity // int(tile_size))
        cached = getattr(self, "suffix_tiles", None)
        if (cached is None or int(cached[0].shape[-1]) != slots or int(cached[4]) != int(tile_size)
                or int(cached[0].shape[1]) != int(num_kv_heads)):
            dev = buf.device
            starts = (torch.arange(slots, device=dev, dtype=torch.int32) * int(tile_size)).view(1, 1, -1) \
                .expand(1, num_kv_heads, -1).contiguous()
            lengths = torch.full((1, num_kv_heads, slots), int(tile_size), dtype=torch.int32, device=dev)
            counts = torch.full((1, num_kv_heads), slots, dtype=torch.int32, device=dev)
            selected = torch.full_like(counts, capacity)
            posting = buf.unsqueeze(0).expand(num_kv_heads, -1)          # every KV head reads the same positions
            cached = (starts, lengths, counts, selected, int(tile_size), posting)
            self.suffix_tiles = cached
        starts, lengths, counts, selected, _, posting = cached
        return posting, starts, lengths, counts, selected


class SembloRuntimeState:
    """Request-local state shared by the sparse layers of one model: the prompt's indexes by
    source layer, engine-lifetime buffers, and the position bookkeeping of
    semblo/vllm_plugin/state.py (SembloRuntimeState: pooled_buffer 1286-1300, reset 1322-1329,
    maybe_begin_prompt 1417-1477, put/get 1479-1494).  One request at a time."""

    def __init__(self, max_model_len: int, reset_layer_idx: int | None = None) -> None:
        self.max_model_len = int(max_model_len)
        self.reset_layer_idx = reset_layer_idx
        self.source_indexes: dict = {}
        self.index_buffers: dict = {}
        self.source_modules: dict = {}
        self.step_first_position = 0
        self.expected_next_position = 0
        self.prompt_epoch = 0
        self.dense_request = False
        self.suffix_block_size = 256
        self.suffix_kv: dict = {}
        self.suffix_block_table = None
        self.suffix_base_block = -1
        self.step_suffix_key = None
        self.step_suffix_tiles = None
        self.step_recorded_key = None

    # ---- the layers' own store of generated K/V (state.py:1239-1284 of the reference) ----------
    def ensure_suffix_store(self, layer_idx, *, prompt_length, max_model_len, num_kv_heads, head_dim, dtype,
                            device) -> torch.Tensor:
        """[2, blocks, 256, Hkv, D] for what this request can still generate, addressed by absolute
        position through ``suffix_block_table`` [1, blocks of the whole sequence] like a paged cache."""
        block = int(self.suffix_block_size)
        base = int(prompt_length) // block
        n_blocks = max(1, (int(max_model_len) + block - 1) // block - base)
        if self.suffix_block_table is None or self.suffix_base_block != base \
                or self.suffix_block_table.device != torch.device(device):
            table = torch.zeros(1, base + n_blocks, dtype=torch.int32, device=device)
            table[0, base:] = torch.arange(n_blocks, dtype=torch.int32, device=device)
            self.suffix_block_table = table
            self.suffix_base_block = base
            self.suffix_kv.clear()
        buf = self.suffix_kv.get(int(layer_idx))
        if buf is None:
            buf = torch.zeros(2, n_blocks, block, num_kv_heads, head_dim, dtype=dtype, device=device)
            self.suffix_kv[int(layer_idx)] = buf
        return buf

    def write_suffix_kv(self, layer_idx, positions, key, value) -> None:
        """One step's K/V at its own absolute position."""
        buf = self.suffix_kv[int(layer_idx)]
        block = int(self.suffix_block_size)
        rel = positions.to(torch.int64) - self.suffix_base_block * block
        b, off = rel // block, rel % block
        buf[0, b, off] = key.to(buf.dtype)
        buf[1, b, off] = value.to(buf.dtype)

    def pooled_like(self, key: str, like: torch.Tensor) -> torch.Tensor:
        return self.pooled_buffer(key, tuple(like.shape), like.dtype, like.device)

    def record_decode_positions(self, index: "ProductPostingIndex", count: int) -> None:
        """Once per step (the sparse layers of a step share the index bookkeeping per source layer)."""
        key = (self.prompt_epoch, self.step_first_position, id(index))
        if self.step_recorded_key != key:
            index.record_generated_positions(self.step_first_position, count)
            self.step_recorded_key = key

    def suffix_tiles_for_step(self, index: "ProductPostingIndex", *, num_kv_heads: int, tile_size: int,
                              pool: bool = False):
        """The generated-suffix tiles of the current step, built once for all sparse layers;
        ``pool`` copies them into engine-lifetime buffers so that a recorded decode step of the
        previous request still finds them at the same addresses."""
        key = (self.prompt_epoch, self.step_first_position, num_kv_heads, tile_size)
        if self.step_suffix_key != key:
            tiles = index.generated_suffix_tiles(num_kv_heads=num_kv_heads, tile_size=tile_size)
            if pool:
                names = ("suffix_posting", "suffix_starts", "suffix_lengths", "suffix_counts", "suffix_selected")
                moved = []
                for name, tensor in zip(names, tiles):
                    buffer = self.pooled_like(name, tensor)
                    if buffer.data_ptr() != tensor.data_ptr():
                        buffer.copy_(tensor)
                    moved.append(buffer)
                tiles = tuple(moved)
            self.step_suffix_tiles = tiles
            self.step_suffix_key = key
        return self.step_suffix_tiles

    def register_source_module(self, layer_idx: int, module) -> None:
        self.source_modules[int(layer_idx)] = module
        if self.reset_layer_idx is None or int(layer_idx) < int(self.reset_layer_idx):
            self.reset_layer_idx = int(layer_idx)          # the earliest sparse layer begins a prompt

    def get_source_module(self, layer_idx: int):
        return self.source_modules[int(layer_idx)]

    def pooled_buffer(self, key, shape, dtype, device) -> torch.Tensor:
        signature = (tuple(shape), dtype, torch.device(device))
        buffer = self.index_buffers.get(key)
        if buffer is None or self.index_buffers.get((key, "sig")) != signature:
            buffer = torch.empty(*shape, dtype=dtype, device=device)
            self.index_buffers[key] = buffer
            self.index_buffers[(key, "sig")] = signature
        return buffer

    def reset(self) -> None:
        self.dense_request = False
        self.source_indexes.clear()
        self.prompt_epoch += 1

    def maybe_begin_prompt(self, layer_idx: int, positions: torch.Tensor, engage_above_tokens: int = 0) -> None:
        """Reset the request-local indexes exactly once at a new prompt.  A decode step that follows
        the previous call by one position is tracked on the host; anything else reads
        ``positions[0]`` (one synchronisation, as in the reference)."""
        if self.reset_layer_idx is None or int(layer_idx) != int(self.reset_layer_idx):
            return
        if positions.ndim != 1 or positions.numel() == 0:
            raise ValueError("positions must be a non-empty one-dimensional tensor")
        if positions.numel() == 1 and self.expected_next_position > 0:
            self.step_first_position = self.expected_next_position
        else:
            self.step_first_position = int(positions[0].item())
        self.expected_next_position = self.step_first_position + positions.numel()
        if self.step_first_position == 0:
            expected = torch.arange(positions.numel(), device=positions.device, dtype=positions.dtype)
            if not torch.equal(positions, expected):
                raise RuntimeError("the full prompt must arrive in one contiguous prefill call")
            self.reset()
            self.dense_request = 0 < engage_above_tokens and positions.numel() <= engage_above_tokens

    def put(self, source_layer_idx: int, index: ProductPostingIndex) -> None:
        if int(source_layer_idx) in self.source_indexes:
            raise RuntimeError(f"semblo prompt index for source layer {source_layer_idx} was built more than once")
        self.source_indexes[int(source_layer_idx)] = index

    def get(self, source_layer_idx: int) -> ProductPostingIndex:
        try:
            return self.source_indexes[int(source_layer_idx)]
        except KeyError as exc:
            raise RuntimeError(f"semblo index for source layer {source_layer_idx} is unavailable") from exc
