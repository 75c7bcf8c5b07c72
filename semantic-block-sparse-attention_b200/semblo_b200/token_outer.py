"""Token-order streamed prefill of one sparse layer.

Mirrors semblo/vllm_plugin/token_outer_prefill.py: reserved_layout (39-63), append_rows
(66-87), TokenOuterSnapshot (90-124) and TokenOuterPrefillSession (127-400) without the
model hooks: the session takes the projected tensors of a slice and returns the attention
output.  The prompt arrives in slices of at most one query chunk.  Until ``fit_at`` the
slices are staged and attended densely; at ``fit_at`` the index is fitted on the staged
keys with the cluster count of the whole prompt and the store is laid out with per-cluster
reservations; every later slice is assigned to its nearest centroid, appended to the
reserved runs and attended with the cluster sizes as they were before the slice plus the
exact causal window over the slice itself."""
from __future__ import annotations

import os
from types import SimpleNamespace

import torch

from . import _lib
from ._lib import check, lib, ptr, require_cuda, stream_ptr
from .flat_index import routing_normalize
from .fused_prefill import CausalSnapshot, _attend_part, fused_chunk_attention, window_attention
from .state import ProductPostingIndex, flat_num_clusters
from .trivial_router import trivial_router_vectors


def token_outer_fit_at(total: int, chunk: int, target_tokens: int, dense_prefix_x: int = 4) -> int:
    """token_outer_prefill.py:148-161."""
    cap = int(os.environ.get("SEMBLO_FA3_DENSE_PREFIX_X", str(dense_prefix_x))) * int(target_tokens)
    fit_tokens = int(os.environ.get("SEMBLO_TOKEN_OUTER_FIT_TOKENS", "65536"))
    fit_tokens = min(fit_tokens, cap) if fit_tokens > 0 else cap
    return min(int(total), ((fit_tokens // int(chunk)) + 1) * int(chunk))


def reserved_layout(sizes_ref: torch.Tensor, n_ref: int, total_tokens: int, width: int, align: int) -> torch.Tensor:
    """Rows reserved per cluster [Hkv, C] int64 (token_outer_prefill.py:39-63): in proportion to
    the observed sizes, at least one page, multiples of ``align``, the spare spread in proportion.
    Small tensors, float64 as in the reference; one host read per head for the spare."""
    align = max(int(align), 1)
    sizes = sizes_ref.to(torch.float64)
    hkv, _ = sizes.shape
    want = sizes * (float(total_tokens) / float(max(int(n_ref), 1)))
    base = torch.ceil(want / align).to(torch.int64).clamp_min(1) * align
    for h in range(hkv):
        spare = int(width) - int(base[h].sum())
        if spare < 0:
            raise RuntimeError("the reserved layout does not fit the store")
        if spare >= align:
            share = want[h] / max(float(want[h].sum()), 1.0)
            extra = torch.floor(share * (spare // align)).to(torch.int64) * align
            base[h] += extra
    return base


def nearest_cluster(product_keys: torch.Tensor, codebooks: torch.Tensor) -> torch.Tensor:
    """_nearest_cluster for every head (suffix_flush.py:154-169): product_keys [n, Hkv, D] bf16
    unit routing keys, codebooks [Hkv, 2, C, D/2] -> ids [Hkv, n] int32."""
    require_cuda(product_keys, codebooks)
    n, hkv, d = product_keys.shape
    c = int(codebooks.shape[2])
    if product_keys.dtype != torch.bfloat16 or codebooks.dtype != torch.bfloat16:
        raise ValueError("nearest_cluster takes bf16 keys and descriptors")
    keys = product_keys if product_keys.is_contiguous() else product_keys.contiguous()
    ids = torch.empty(hkv, n, dtype=torch.int32, device=keys.device)
    dead = torch.empty(hkv, c // 32, dtype=torch.int32, device=keys.device)
    status = _lib.status_for(keys.device)
    check(lib().semblo_nearest_cluster(ptr(keys), n, hkv, d, ptr(codebooks), c, ptr(ids), ptr(dead),
                                       ptr(status.word), stream_ptr()))
    return ids


def append_rows(ids: torch.Tensor, indptr: torch.Tensor, sizes: torch.Tensor):
    """token_outer_prefill.py:66-87: destination rows [Hkv, n] int32 and per-cluster counts [Hkv, C]."""
    require_cuda(ids, indptr, sizes)
    hkv, n = ids.shape
    c = int(sizes.shape[1])
    rows = torch.empty(hkv, n, dtype=torch.int32, device=ids.device)
    counts = torch.empty(hkv, c, dtype=torch.int32, device=ids.device)
    ws_bytes = int(lib().semblo_layout_workspace_bytes(n, hkv)) + hkv * (c + 1) * 4
    ws = torch.empty(ws_bytes, dtype=torch.uint8, device=ids.device)
    check(lib().semblo_append_rows(ptr(ids.contiguous()), n, hkv, c, ptr(indptr), ptr(sizes), ptr(rows), ptr(counts),
                                   ptr(ws), ws_bytes, stream_ptr()))
    return rows, counts


def scatter_kv(k: torch.Tensor, v: torch.Tensor, positions: torch.Tensor | None, rows: torch.Tensor,
               packed: torch.Tensor, posting: torch.Tensor | None, inverse: torch.Tensor | None,
               inverse_offset: int = 0, page_table: torch.Tensor | None = None) -> None:
    """K/V rows of consecutive tokens into the packed store (the index_copy_ calls of
    token_outer_prefill.py:296-309, 354-358)."""
    n, hkv, d = k.shape
    status = _lib.status_for(k.device)
    check(lib().semblo_scatter_kv(ptr(k.contiguous()), ptr(v.contiguous()), ptr(positions), n, hkv, d, ptr(rows),
                                  rows.stride(0), ptr(packed), int(packed.shape[1]), packed.stride(0), ptr(posting),
                                  posting.stride(0) if posting is not None else 0, ptr(inverse),
                                  inverse.stride(0) if inverse is not None else 0, int(inverse_offset),
                                  ptr(page_table), ptr(status.word), stream_ptr()))


def gather_kv(packed: torch.Tensor, rows: torch.Tensor, page_table: torch.Tensor | None = None):
    """(k, v) [n, Hkv, D] = the packed rows ``rows`` [Hkv, n] (reads through the inverse map)."""
    hkv, n = rows.shape
    d = int(packed.shape[-1])
    out_k = torch.empty(n, hkv, d, dtype=packed.dtype, device=packed.device)
    out_v = torch.empty_like(out_k)
    check(lib().semblo_gather_kv(ptr(packed), packed.stride(0), ptr(rows), rows.stride(0), n, hkv, d, ptr(out_k),
                                 ptr(out_v), ptr(page_table), stream_ptr()))
    return out_k, out_v


def relayout_rows(rows_old: torch.Tensor, bucket: torch.Tensor, old_indptr: torch.Tensor,
                  new_indptr: torch.Tensor) -> torch.Tensor:
    """token_outer_prefill.py:282-287, 375-379: every key keeps its offset inside its cluster's run."""
    hkv, n = rows_old.shape
    if rows_old.stride(0) != bucket.stride(0):
        raise ValueError("rows and cluster ids must share their row stride")
    out = torch.empty_like(rows_old)
    if out.stride(0) != rows_old.stride(0):
        raise ValueError("rows must be dense")
    check(lib().semblo_relayout_rows(ptr(rows_old), ptr(bucket), n, rows_old.stride(0), hkv, ptr(old_indptr),
                                     ptr(new_indptr), int(old_indptr.shape[1]) - 1, ptr(out), stream_ptr()))
    return out


class TokenOuterSnapshot(CausalSnapshot):
    """The counts before the slice being attended (token_outer_prefill.py:90-124); the scratch
    buffers of the chunk driver live here as they do in CausalSnapshot."""

    def __init__(self, index) -> None:
        super().__init__(index)
        self.chunk_start = 0

    def advance(self, last_pos: int) -> torch.Tensor:
        if int(last_pos) + 1 != self.chunk_start:
            raise RuntimeError(f"the token-outer snapshot holds the counts before position {self.chunk_start}; "
                               f"the body asked for position {last_pos}")
        return self.sizes


class TokenOuterPrefillSession:
    """One sparse layer's share of a token-order prefill (token_outer_prefill.py:127-400)."""

    def __init__(self, *, total_tokens: int, chunk: int, num_q_heads: int, num_kv_heads: int, head_dim: int,
                 target_tokens: int, temperature: float, beta: float, sm_scale: float, flat_unit_tokens: int,
                 flat_min_clusters_log2: int, page_align: int, device, kmeans_sample_size: int = 8192,
                 codebook_seed: int | None = 0, query_chunk_size: int = 8192) -> None:
        if int(chunk) > int(query_chunk_size):
            raise RuntimeError(f"SEMBLO_PREFILL_CHUNK={chunk} must not exceed the query chunk "
                               f"({query_chunk_size}): a slice's keys are appended once, before its queries")
        if os.environ.get("SEMBLO_ROUTING_CENTER") == "1":
            raise RuntimeError("the token-outer prefill does not centre keys")
        if (os.environ.get("SEMBLO_ROUTING_NORMALIZE", "whole") or "whole") != "whole":
            raise RuntimeError("the token-outer prefill assigns in the whole-vector routing space")
        if int(os.environ.get("SEMBLO_FA3_LOCAL", "0") or "0") != 0:
            raise RuntimeError("the token-outer prefill attends a slice's own keys through the exact window only "
                               "(SEMBLO_FA3_LOCAL must be 0)")
        self.tokens, self.chunk = int(total_tokens), int(chunk)
        self.hq, self.hkv, self.dim = int(num_q_heads), int(num_kv_heads), int(head_dim)
        self.target, self.temperature, self.beta, self.sm_scale = int(target_tokens), temperature, beta, sm_scale
        self.unit, self.min_log2, self.align = int(flat_unit_tokens), int(flat_min_clusters_log2), int(page_align)
        self.sample, self.seed = int(kmeans_sample_size), codebook_seed
        self.device = torch.device(device)
        self.fit_at = token_outer_fit_at(self.tokens, self.chunk, self.target)
        self.cap = int(os.environ.get("SEMBLO_FA3_DENSE_PREFIX_X", "4")) * self.target
        self.stage_k = self.stage_v = self.stage_kpre = None
        self.index = None
        self.snapshot = None
        self.reserve = None
        self.repacks = 0
        self.positions = torch.arange(self.tokens, device=self.device)
        self.positions32 = self.positions.to(torch.int32)

    # -- per slice ------------------------------------------------------------------------
    def slice(self, q_post: torch.Tensor, q_pre: torch.Tensor, k_post: torch.Tensor, v_states: torch.Tensor,
              k_pre: torch.Tensor, start: int, stop: int, out: torch.Tensor | None = None) -> torch.Tensor:
        """q_post, q_pre [n, Hq, D]; k_post, v_states, k_pre [n, Hkv, D]; positions [start, stop)."""
        require_cuda(q_post, q_pre, k_post, v_states, k_pre)
        if stop - start != q_post.shape[0] or stop - start > self.chunk:
            raise ValueError("a slice holds at most one chunk of consecutive positions")
        # labelled with the operator's name, as the reference's slice is (token_outer_prefill.py:186)
        with torch.profiler.record_function("semblo::attention"):
            return self._slice(q_post, q_pre, k_post, v_states, k_pre, start, stop, out)

    def _slice(self, q_post, q_pre, k_post, v_states, k_pre, start, stop, out):
        if self.index is None and start >= self.fit_at:
            self._fit_and_pack()
        if out is None:
            out = torch.empty_like(q_post)
        if self.index is None:
            self._stage(k_post, v_states, k_pre, start, stop)
            return window_attention(q_post, self.positions32[start:stop], ordered_k=self.stage_k[:stop],
                                    ordered_v=self.stage_v[:stop], ordered_pos0=0, local_start=0,
                                    sm_scale=self.sm_scale, out=out)
        self._append(k_post, v_states, k_pre, start, stop)
        qv = trivial_router_vectors(q_pre)
        state = SimpleNamespace(vectors=qv.view(1, stop - start, self.hq, 1, self.dim))
        if start <= self.cap:
            # read densely through the inverse permutation
            rows = self.index._inverse_positions[:, :stop]
            with _attend_part("semblo::gather_kv"):
                local = gather_kv(self.index.packed_kv, rows) + (0,)
        else:
            local = (k_post, v_states, start)
        return fused_chunk_attention(q_post, state, self.index, self.positions32[start:stop], self.snapshot, start,
                                     stop - 1, temperature=self.temperature, beta=self.beta,
                                     target_tokens=self.target, sm_scale=self.sm_scale, out=out, local_kv=local)

    def finish(self) -> None:
        if self.index is None:
            self.fit_at = self.tokens              # the prompt ended before the fit point: fit on all of it
            self._fit_and_pack()
        # the store kernels refuse to run after a device-side condition: the end of the prompt reads the word
        _lib.status_for(self.device).raise_if_set()

    # -- dense start ---------------------------------------------------------------------
    def _stage(self, k3, v3, kp3, start, stop) -> None:
        if self.stage_k is None:
            n = self.fit_at
            self.stage_k = k3.new_empty((n,) + tuple(k3.shape[1:]))
            self.stage_v = v3.new_empty((n,) + tuple(v3.shape[1:]))
            self.stage_kpre = kp3.new_empty((n,) + tuple(kp3.shape[1:]))
        self.stage_k[start:stop] = k3
        self.stage_v[start:stop] = v3
        self.stage_kpre[start:stop] = kp3

    # -- fit -----------------------------------------------------------------------------
    def _fit_and_pack(self) -> None:
        p = self.fit_at
        clusters = flat_num_clusters(self.tokens, self.unit, self.min_log2)
        product = routing_normalize(self.stage_kpre[:p])
        # the count the whole prompt would get (the reference passes it through SEMBLO_FLAT_CLUSTERS)
        index = ProductPostingIndex.build(product, self.positions[:p], kmeans_sample_size=self.sample,
                                          codebook_seed=self.seed, flat_unit_tokens=self.unit,
                                          flat_min_clusters_log2=self.min_log2, page_align=self.align,
                                          num_clusters=clusters)
        del product
        align = max(int(index.page_align), 1)
        width = self.tokens + int(index.num_buckets) * align
        width += (-width) % 256
        reserve = reserved_layout(index.bucket_sizes, p, self.tokens, width, align)
        dev = self.device
        indptr = torch.zeros(self.hkv, int(index.num_buckets) + 1, dtype=torch.int32, device=dev)
        indptr[:, 1:] = torch.cumsum(reserve, 1).to(torch.int32)
        # every fitted key moves from its cluster's packed run to the reserved one
        assign = torch.zeros(self.hkv, self.tokens, dtype=torch.int32, device=dev)
        assign[:, :p] = index.orig_bucket
        inverse = torch.zeros(self.hkv, self.tokens, dtype=torch.int32, device=dev)
        inv_old = torch.zeros_like(inverse)
        inv_old[:, :p] = index.inverse_positions()
        check(lib().semblo_relayout_rows(ptr(inv_old), ptr(assign), p, inv_old.stride(0), self.hkv,
                                         ptr(index.bucket_indptr), ptr(indptr), int(index.num_buckets), ptr(inverse),
                                         stream_ptr()))
        packed = torch.zeros(2, width, self.hkv, self.dim, dtype=self.stage_k.dtype, device=dev)
        posting = torch.zeros(self.hkv, width, dtype=torch.int32, device=dev)
        scatter_kv(self.stage_k[:p], self.stage_v[:p], self.positions32[:p], inverse, packed, posting, None)
        index.packed_kv = packed
        index.posting_positions = posting
        index.bucket_indptr = indptr
        index._inverse_positions = inverse
        index.orig_bucket = assign
        index.prompt_length = self.tokens
        index.max_position = self.tokens - 1
        index.kv_page_table = None
        self.reserve = reserve
        self.index = index
        self.snapshot = TokenOuterSnapshot(index)
        self.stage_k = self.stage_v = self.stage_kpre = None

    # -- append --------------------------------------------------------------------------
    def _append(self, k3, v3, kp3, start, stop) -> None:
        index = self.index
        product = routing_normalize(kp3)                                      # [n, Hkv, D]
        ids = nearest_cluster(product, index.codebooks)                       # [Hkv, n]
        del product
        sizes = index.bucket_sizes
        rows, counts = append_rows(ids, index.bucket_indptr, sizes)
        if bool((sizes.to(torch.int64) + counts > self.reserve).any()):       # one host read, as the reference
            self._repack(start)
            rows, counts = append_rows(ids, index.bucket_indptr, sizes)
            if bool((sizes.to(torch.int64) + counts > self.reserve).any()):
                # The reference stops here (token_outer_prefill.py:350-352) and a cluster that the
                # slice pushes past its fresh reservation would run into its neighbour's rows.  Lay
                # the store out once more from the sizes that include the slice: every run then
                # holds its cluster by construction.
                self._repack(start, incoming=counts, n_incoming=stop - start)
                rows, counts = append_rows(ids, index.bucket_indptr, sizes)
        scatter_kv(k3, v3, self.positions32[start:stop], rows, index.packed_kv, index.posting_positions,
                   index._inverse_positions, inverse_offset=start)
        index.orig_bucket[:, start:stop] = ids
        # the body sees the counts before this slice; the slice's own keys go through the exact window
        self.snapshot.sizes = sizes.clone()
        self.snapshot.chunk_start = start
        sizes += counts

    def _repack(self, n_so_far: int, incoming: torch.Tensor | None = None, n_incoming: int = 0) -> None:
        """Lay the runs out again from the current proportions, in place (token_outer_prefill.py:366-392).
        ``incoming`` [Hkv, C] adds a slice's counts to the proportions (see _append)."""
        index = self.index
        align = max(int(index.page_align), 1)
        width = int(index.packed_kv.shape[1])
        basis = index.bucket_sizes if incoming is None else index.bucket_sizes + incoming
        reserve = reserved_layout(basis, n_so_far + n_incoming, self.tokens, width, align)
        new_ip = torch.zeros_like(index.bucket_indptr)
        new_ip[:, 1:] = torch.cumsum(reserve, 1).to(torch.int32)
        rows_old = index._inverse_positions
        rows_new = rows_old.clone()
        check(lib().semblo_relayout_rows(ptr(rows_old), ptr(index.orig_bucket), n_so_far, rows_old.stride(0), self.hkv,
                                         ptr(index.bucket_indptr), ptr(new_ip), int(index.num_buckets), ptr(rows_new),
                                         stream_ptr()))
        k_all, v_all = gather_kv(index.packed_kv, rows_old[:, :n_so_far])     # the clone of the old rows
        scatter_kv(k_all, v_all, self.positions32[:n_so_far], rows_new[:, :n_so_far], index.packed_kv,
                   index.posting_positions, None)
        index._inverse_positions = rows_new
        index.bucket_indptr = new_ip
        self.reserve = reserve
        self.repacks += 1
