"""Flat key partition: spherical k-means over the prompt's routing keys.

Mirrors semblo/inference/flat_index.py (fit_flat_codebook 193-289,
assign_flat_buckets 376-382, routing_space 144-166, flat_cluster_count 81-84).
The arithmetic runs in CUDA (tcgen05 similarity GEMM with the bf16-round +
first-arg-max epilogue, ordered segment sums); the three random draws stay
``torch.randperm`` calls on the caller's generator, as in the reference."""
from __future__ import annotations

import os

import torch

from . import _lib
from ._lib import check, lib, ptr, require_cuda, stream_ptr


def flat_cluster_count(length: int, target_size: int, *, min_clusters: int = 64,
                       max_clusters: int = 16384) -> int:
    return int(min(max(length // max(target_size, 1), min_clusters), max_clusters, length))


def routing_mode() -> str:
    mode = os.environ.get("SEMBLO_ROUTING_NORMALIZE", "whole") or "whole"
    if mode != "whole":
        raise RuntimeError(f"SEMBLO_ROUTING_NORMALIZE={mode!r}: this build implements the default "
                           "whole-vector routing space only")
    return mode


def _normalize(x: torch.Tensor, *, want_out: bool, want_f32: bool, want_bf16: bool, query_mode: bool):
    require_cuda(x)
    routing_mode()
    if x.dtype not in (torch.bfloat16, torch.float32):
        raise ValueError(f"routing vectors must be bf16 or fp32, got {x.dtype}")
    dim = x.shape[-1]
    rows = x.reshape(-1, dim)
    if rows.stride(1) != 1:
        rows = rows.contiguous()
    n = rows.shape[0]
    out = torch.empty(n, dim, dtype=x.dtype, device=x.device) if want_out else None
    f32 = torch.empty(n, dim, dtype=torch.float32, device=x.device) if want_f32 else None
    b16 = torch.empty(n, dim, dtype=torch.bfloat16, device=x.device) if want_bf16 else None
    check(lib().semblo_routing_normalize(ptr(rows), 0 if x.dtype == torch.bfloat16 else 1, n, dim,
                                         rows.stride(0), ptr(out), ptr(f32), ptr(b16),
                                         1 if query_mode else 0, stream_ptr()))
    return out, f32, b16


def routing_normalize(x: torch.Tensor) -> torch.Tensor:
    """routing_map.py:35-64: unit vectors in the input dtype."""
    out, _, _ = _normalize(x, want_out=True, want_f32=False, want_bf16=False, query_mode=False)
    return out.view(x.shape)


def routing_space(x: torch.Tensor) -> torch.Tensor:
    """flat_index.py:144-166: fp32 unit vectors."""
    _, f32, _ = _normalize_space(x)
    return f32.view(x.shape)


def _normalize_space(x: torch.Tensor):
    """(None, fp32 space, bf16 space) of already routed keys: one normalisation."""
    require_cuda(x)
    dim = x.shape[-1]
    rows = x.reshape(-1, dim)
    if rows.stride(1) != 1:
        rows = rows.contiguous()
    n = rows.shape[0]
    f32 = torch.empty(n, dim, dtype=torch.float32, device=x.device)
    b16 = torch.empty(n, dim, dtype=torch.bfloat16, device=x.device)
    # stage 1 of the kernel is the identity on unit input up to rounding; to normalise
    # exactly once the routed keys go through the fp32 path of stage 2 only
    check(lib().semblo_routing_normalize(ptr(rows), 0 if x.dtype == torch.bfloat16 else 1, n, dim,
                                         rows.stride(0), None, ptr(f32), ptr(b16), 2, stream_ptr()))
    return None, f32, b16


class _FitWorkspace:
    def __init__(self, n: int, num_clusters: int, dim: int, device) -> None:
        i32 = dict(dtype=torch.int32, device=device)
        self.assign = torch.empty(n, **i32)
        self.counts = torch.empty(num_clusters, **i32)
        self.ip = torch.empty(num_clusters + 1, **i32)
        self.empty_rank = torch.empty(num_clusters, **i32)
        self.n_empty = torch.empty(1, **i32)
        self.cent_f32 = torch.empty(num_clusters, dim, dtype=torch.float32, device=device)
        self.cent_bf16 = torch.empty(num_clusters, dim, dtype=torch.bfloat16, device=device)
        self.ws_bytes = int(lib().semblo_layout_workspace_bytes(n, 1))
        self.ws = torch.empty(self.ws_bytes, dtype=torch.uint8, device=device)
        # the host reads n_empty through a pinned word, copied on a stream of its own behind the counts, so
        # that the sort of the member lists (which needs no restart draws) runs while the read is on its way
        self.n_empty_host = torch.zeros(1, dtype=torch.int32).pin_memory()
        self.read_stream = torch.cuda.Stream(device=device)
        self.counted = torch.cuda.Event()
        self.read_done = torch.cuda.Event()


def _assign(x_bf16: torch.Tensor, cent_bf16: torch.Tensor, out: torch.Tensor, id_offset: int = 0) -> None:
    status = _lib.status_for(x_bf16.device)
    check(lib().semblo_assign_argmax(ptr(x_bf16), x_bf16.shape[0], ptr(cent_bf16), cent_bf16.shape[0],
                                     x_bf16.shape[1], ptr(out), id_offset, ptr(status.word), stream_ptr()))


def fit_flat_codebook(space_f32: torch.Tensor, space_bf16: torch.Tensor, num_clusters: int, *,
                      num_iters: int, sample_size: int, generator: torch.Generator | None) -> torch.Tensor:
    """flat_index.py:229-289 (cosine, random init) on already normalised keys.

    ``space_f32`` / ``space_bf16`` [n, I] are the fp32 routing space and its bf16
    rounding.  Returns fp32 centroids [C, I].  One host read per iteration decides
    whether the empty-cluster restart draws from the generator, exactly as the
    reference's ``bool(empty.any())``."""
    require_cuda(space_f32, space_bf16)
    n, dim = space_f32.shape
    fit_n = min(n, int(sample_size))
    if fit_n < num_clusters:
        raise ValueError("sample must be at least as large as num_clusters")
    device = space_f32.device
    perm = torch.randperm(n, device=device, generator=generator)
    idx = perm[:fit_n].contiguous()
    sample_f32 = torch.empty(fit_n, dim, dtype=torch.float32, device=device)
    sample_bf16 = torch.empty(fit_n, dim, dtype=torch.bfloat16, device=device)
    check(lib().semblo_gather_rows(ptr(space_f32), ptr(idx), fit_n, dim, ptr(sample_f32), ptr(sample_bf16), stream_ptr()))
    init = torch.randperm(fit_n, device=device, generator=generator)[:num_clusters].contiguous()
    w = _FitWorkspace(fit_n, num_clusters, dim, device)
    check(lib().semblo_gather_rows(ptr(sample_f32), ptr(init), num_clusters, dim, ptr(w.cent_f32), ptr(w.cent_bf16), stream_ptr()))
    for _ in range(num_iters):
        _assign(sample_bf16, w.cent_bf16, w.assign)
        check(lib().semblo_cluster_counts(ptr(w.assign), fit_n, fit_n, 1, num_clusters, 1, ptr(w.counts),
                                          ptr(w.ip), None, ptr(w.empty_rank), ptr(w.n_empty), stream_ptr()))
        w.counted.record()
        w.read_stream.wait_event(w.counted)
        with torch.cuda.stream(w.read_stream):
            w.n_empty_host.copy_(w.n_empty, non_blocking=True)
            w.read_done.record()
        check(lib().semblo_kmeans_sort_members(ptr(w.assign), fit_n, num_clusters, ptr(w.ws), w.ws_bytes, stream_ptr()))
        w.read_done.synchronize()
        repl = None
        if int(w.n_empty_host[0]) > 0:
            repl = torch.randperm(fit_n, device=device, generator=generator).contiguous()
        check(lib().semblo_kmeans_update_sorted(ptr(sample_f32), fit_n, num_clusters, dim, ptr(w.ip),
                                                ptr(w.empty_rank), ptr(repl), ptr(w.cent_f32), ptr(w.cent_bf16),
                                                ptr(w.ws), w.ws_bytes, stream_ptr()))
    return w.cent_f32


def assign_flat_buckets(space_bf16: torch.Tensor, centroids: torch.Tensor, *, out: torch.Tensor | None = None,
                        id_offset: int = 0) -> torch.Tensor:
    """flat_index.py:376-382: [n] int32 cluster ids (bf16-rounded similarity, lowest id on ties)."""
    require_cuda(space_bf16, centroids)
    cent = centroids if centroids.dtype == torch.bfloat16 else centroids.to(torch.bfloat16)
    if out is None:
        out = torch.empty(space_bf16.shape[0], dtype=torch.int32, device=space_bf16.device)
    _assign(space_bf16, cent.contiguous(), out, id_offset)
    return out
