"""Prefill chunk driver: causal snapshot, dense-prefix rule, selection, attention body.

Mirrors semblo/vllm_plugin/fused_prefill.py (CausalSnapshot 44-135,
fused_chunk_attention 219-550 on its default path: SEMBLO_FA3_BODY=16,
SEMBLO_KV_OUTER=1, sink rule 192-216) and the scoring/selection entry point
theta_select_bitmask_flat (fused_select.py:806-863).  No host synchronisation in
the chunk loop."""
from __future__ import annotations

import contextlib
import os

import torch

from . import _lib
from ._lib import check, lib, ptr, require_cuda, stream_ptr


# Profiler labels of the attention launches, with the reference's names and switch
# (kv_outer.py:243-252, fused_prefill.py:183); off by default: a label costs a little per call.
_ATTEND_PARTS = os.environ.get("SEMBLO_PROFILE_ATTEND_PARTS") == "1"


def _attend_part(name: str):
    if not _ATTEND_PARTS:
        return contextlib.nullcontext()
    return torch.profiler.record_function(name)


def _fitted_sink_tokens() -> int:
    sink = int(os.environ.get("SEMBLO_SINK_TOKENS", "0") or "0")
    return sink if sink > 0 else 0


class CausalSnapshot:
    """Running per-cluster count of keys with position <= p (fused_prefill.py:44-135)."""

    def __init__(self, index) -> None:
        self.index = index
        self.sizes = torch.zeros_like(index.bucket_sizes)
        self.next_pos = 0
        self.length = int(index.prompt_length)
        self.b_dim = int(index.num_buckets)
        self.qmask = None
        self.score = None
        self.select_sizes = None
        self.top1 = self.order = self.lse = self.sort_ws = self.partial = None

    def advance(self, last_pos: int) -> torch.Tensor:
        hi = min(int(last_pos) + 1, self.length)
        if hi > self.next_pos:
            ob = self.index.orig_bucket
            check(lib().semblo_snapshot_advance(ptr(ob), ob.stride(0), ob.shape[0], self.next_pos, hi,
                                                self.b_dim, ptr(self.sizes), stream_ptr()))
            self.next_pos = hi
        return self.sizes


def theta_select_bitmask_flat(vectors: torch.Tensor, codebooks: torch.Tensor, select_sizes: torch.Tensor, *,
                              temperature: float, beta: float, target_tokens: int, iters: int = 16,
                              qmask: torch.Tensor | None = None, score: torch.Tensor | None = None,
                              force_sink: bool = False, counts: torch.Tensor | None = None,
                              tokens: torch.Tensor | None = None, top1: torch.Tensor | None = None,
                              tile_key_beta: float = 0.0):
    """Scores + bisected threshold -> per-query packed bitmask [Q, Hkv, C/32].

    vectors [Q, Hq, D] bf16 routing vectors; select_sizes [Hkv, C] int32 (one snapshot for
    the whole chunk, the sink cluster already held out).  ``top1`` [Hkv, Q] receives the tile-order
    key: arg max of score + tile_key_beta log(1 + n).  Returns (qmask, score)."""
    require_cuda(vectors, codebooks, select_sizes)
    q_count, num_q_heads, dim = vectors.shape
    num_kv_heads, _, num_clusters, _ = codebooks.shape
    device = vectors.device
    if score is None:
        score = torch.empty(q_count, num_kv_heads, num_clusters, dtype=torch.float32, device=device)
    if qmask is None:
        qmask = torch.empty(q_count, num_kv_heads, num_clusters // 32, dtype=torch.int32, device=device)
    status = _lib.status_for(device)
    check(lib().semblo_score_clusters(ptr(vectors), q_count, num_q_heads, dim, ptr(codebooks), num_kv_heads,
                                      num_clusters, ptr(select_sizes), float(temperature), float(beta),
                                      ptr(score), ptr(status.word), stream_ptr()))
    check(lib().semblo_select_clusters(ptr(score), ptr(select_sizes), q_count, num_kv_heads, num_clusters,
                                       int(target_tokens), int(iters), 1 if force_sink else 0, ptr(qmask),
                                       ptr(counts), ptr(tokens), ptr(top1), float(tile_key_beta), stream_ptr()))
    return qmask, score


def window_attention(q: torch.Tensor, q_positions: torch.Tensor, *, ordered_k: torch.Tensor,
                     ordered_v: torch.Tensor, ordered_pos0: int = 0, local_start: int = 0, sm_scale: float,
                     out=None, lse=None, attended=None, partial=None) -> torch.Tensor:
    """Exact causal attention of consecutive queries over positions [local_start, q_position]
    of the position-ordered K/V (semblo_window_prefill)."""
    require_cuda(q, ordered_k, ordered_v)
    q_count, num_q_heads, head_dim = q.shape
    if q.dtype != torch.bfloat16:
        raise ValueError("prefill attention takes bf16 queries")
    q = q if q.is_contiguous() else q.contiguous()
    if out is None:
        out = torch.empty_like(q)
    ordered_k = ordered_k if ordered_k.is_contiguous() else ordered_k.contiguous()
    ordered_v = ordered_v if ordered_v.is_contiguous() else ordered_v.contiguous()
    status = _lib.status_for(q.device)
    check(lib().semblo_window_prefill(
        ptr(q), q_count, num_q_heads, int(ordered_k.shape[1]), head_dim, ptr(q_positions), ptr(ordered_k),
        ptr(ordered_v), int(ordered_k.shape[0]), int(ordered_pos0), int(local_start), float(sm_scale), ptr(out),
        ptr(partial), ptr(lse), ptr(attended), ptr(status.word), stream_ptr()))
    return out


def argsort_keys(keys: torch.Tensor, max_key: int, *, out: torch.Tensor | None = None,
                 workspace: torch.Tensor | None = None) -> torch.Tensor:
    """Stable arg-sort of int32 keys [heads, n] in [0, max_key)."""
    require_cuda(keys)
    heads, n = keys.shape
    if out is None:
        out = torch.empty_like(keys)
    need = int(lib().semblo_layout_workspace_bytes(n, heads))
    if workspace is None or workspace.numel() < need:
        workspace = torch.empty(need, dtype=torch.uint8, device=keys.device)
    check(lib().semblo_argsort_keys(ptr(keys), n, heads, int(max_key), ptr(out), ptr(workspace),
                                    workspace.numel(), stream_ptr()))
    return out


def sparse_gather_attention(q: torch.Tensor, *, packed_kv: torch.Tensor, qmask: torch.Tensor,
                            causal_sizes: torch.Tensor, indptr: torch.Tensor, sm_scale: float,
                            out: torch.Tensor, lse: torch.Tensor | None, merge: bool, page_table=None,
                            q_order=None, attended=None, partial=None, cta_order=None) -> torch.Tensor:
    """One launch of the row-gather sparse kernel (semblo_sparse_prefill_gather)."""
    require_cuda(q, packed_kv, qmask)
    q_count, num_q_heads, head_dim = q.shape
    q = q if q.is_contiguous() else q.contiguous()
    status = _lib.status_for(q.device)
    check(lib().semblo_sparse_prefill_gather(
        ptr(q), q_count, num_q_heads, int(packed_kv.shape[2]), head_dim, ptr(q_order), ptr(cta_order),
        ptr(packed_kv[0]),
        ptr(packed_kv[1]), int(packed_kv.shape[1]), ptr(page_table), ptr(qmask), ptr(causal_sizes), ptr(indptr),
        int(causal_sizes.shape[1]), float(sm_scale), 1 if merge else 0, ptr(partial), ptr(out), ptr(lse),
        ptr(attended),
        ptr(status.word), stream_ptr()))
    return out


def gather_launch_order(q_order, qmask: torch.Tensor, causal_sizes: torch.Tensor, num_q_heads: int, *,
                        work: torch.Tensor | None = None, out: torch.Tensor | None = None) -> torch.Tensor:
    """(tile, head) pairs of a sparse launch by descending gathered rows (semblo_gather_launch_order)."""
    require_cuda(qmask, causal_sizes)
    q_count, hkv = int(qmask.shape[0]), int(qmask.shape[1])
    qt = 128 // (num_q_heads // hkv)
    n = ((q_count + qt - 1) // qt) * hkv
    if work is None:
        work = torch.empty(n, dtype=torch.int32, device=qmask.device)
    if out is None:
        out = torch.empty(n, dtype=torch.int32, device=qmask.device)
    check(lib().semblo_gather_launch_order(ptr(q_order), ptr(qmask), ptr(causal_sizes), q_count, num_q_heads, hkv,
                                           int(causal_sizes.shape[1]), ptr(work), ptr(out), stream_ptr()))
    return out[:n]


def chunk_window_start(chunk_start: int, target_tokens: int, dense_prefix_x: int = 4) -> int:
    """First position of a chunk's exact window: 0 for a dense-prefix chunk (fused_prefill.py:250-279)."""
    cap = int(os.environ.get("SEMBLO_FA3_DENSE_PREFIX_X", str(dense_prefix_x))) * int(target_tokens)
    local = int(os.environ.get("SEMBLO_FA3_LOCAL", "0"))
    return 0 if chunk_start <= cap else max(0, chunk_start - local)


class WindowAhead:
    """The part of a prompt's attention that needs no index, issued ahead on a stream of its own.

    A dense-prefix chunk and the exact local window of every later chunk read only the
    position-ordered K/V, so they can run while the index is still being built and fill the
    multiprocessors that the build's many short kernels and host round trips leave idle.  ``ahead``
    chunks are in flight at most (one fp32 partial [chunk, Hq, D] and one LSE each); ``take`` makes
    the calling stream wait for a chunk's launch and hands over its partial, ``release`` lets the
    buffer be used again.  No reference counterpart: the reference runs the three launches of a
    chunk in order on one stream (kv_outer.py:632-805)."""

    def __init__(self, q: torch.Tensor, q_positions: torch.Tensor, ordered_k: torch.Tensor, ordered_v: torch.Tensor, *,
                 chunk: int, target_tokens: int, sm_scale: float, out: torch.Tensor, dense_prefix_x: int = 4,
                 attended=None, ahead: int = 16, before_launch=None, router_input: torch.Tensor | None = None) -> None:
        self.q, self.pos, self.k, self.v, self.out = q, q_positions, ordered_k, ordered_v, out
        self.chunk, self.target, self.sm_scale, self.x = int(chunk), int(target_tokens), float(sm_scale), dense_prefix_x
        self.attended, self.before_launch = attended, before_launch
        self.starts = list(range(0, int(q.shape[0]), self.chunk))
        self.stream = torch.cuda.Stream(device=q.device)
        self.depth = max(1, min(int(ahead), len(self.starts)))
        n_sparse = sum(1 for cs in self.starts if chunk_window_start(cs, self.target, self.x) > 0)
        slots = max(1, min(self.depth, n_sparse))
        hq, d = int(q.shape[1]), int(q.shape[2])
        self.partial = torch.empty(slots, self.chunk, hq, d, dtype=torch.float32, device=q.device)
        self.lse = torch.empty(slots, self.chunk, hq, dtype=torch.float32, device=q.device)
        # the routing vectors of a sparse chunk need no index either: with ``router_input`` ([n, Hq, D]
        # pre-RoPE queries) they are made ahead too, in front of the chunk's window launch
        self.router_input = router_input
        self.vectors = None if router_input is None else torch.empty(slots, self.chunk, hq, router_input.shape[2],
                                                                     dtype=router_input.dtype, device=q.device)
        self.routed: dict = {}          # chunk start -> event recorded behind its routing vectors
        self.done: dict = {}            # chunk start -> event recorded behind its launch
        self.slot_of: dict = {}
        self.free = [(s, None) for s in range(slots)]     # (slot, event after which it may be rewritten)
        self.issued = 0
        self.stream.wait_stream(torch.cuda.current_stream(q.device))
        self._issue(self.depth)

    def _issue(self, upto: int) -> None:
        from contextlib import nullcontext
        while self.issued < min(upto, len(self.starts)):
            cs = self.starts[self.issued]
            ce = min(int(self.q.shape[0]), cs + self.chunk) - 1
            wstart = chunk_window_start(cs, self.target, self.x)
            if wstart > 0 and not self.free:
                return                                     # every partial is still waiting for its sparse launch
            with torch.cuda.stream(self.stream):
                if self.before_launch is not None:
                    self.before_launch(cs, ce)
                k_w, v_w = self.k[wstart:ce + 1], self.v[wstart:ce + 1]
                if wstart == 0:
                    with _attend_part("semblo::attend_dense_prefix"):
                        window_attention(self.q[cs:ce + 1], self.pos[cs:ce + 1], ordered_k=k_w, ordered_v=v_w,
                                         ordered_pos0=0, local_start=0, sm_scale=self.sm_scale, out=self.out[cs:ce + 1],
                                         attended=self.attended)
                else:
                    slot, reusable = self.free.pop(0)
                    if reusable is not None:
                        self.stream.wait_event(reusable)
                    n = ce - cs + 1
                    if self.vectors is not None:
                        from .trivial_router import trivial_router_vectors
                        trivial_router_vectors(self.router_input[cs:ce + 1], out=self.vectors[slot, :n])
                        ev = torch.cuda.Event()
                        ev.record(self.stream)
                        self.routed[cs] = ev
                    with _attend_part("semblo::attend_current_chunk"):
                        window_attention(self.q[cs:ce + 1], self.pos[cs:ce + 1], ordered_k=k_w, ordered_v=v_w,
                                         ordered_pos0=wstart, local_start=wstart, sm_scale=self.sm_scale,
                                         out=self.out[cs:ce + 1], lse=self.lse[slot, :n], attended=self.attended,
                                         partial=self.partial[slot, :n])
                    self.slot_of[cs] = slot
                ev = torch.cuda.Event()
                ev.record(self.stream)
                self.done[cs] = ev
            self.issued += 1

    def is_dense(self, chunk_start: int) -> bool:
        return chunk_window_start(chunk_start, self.target, self.x) == 0

    def vectors_for(self, chunk_start: int):
        """Routing vectors [1, n, Hq, 1, D] of a sparse chunk made ahead (the calling stream waits for
        them), or None for a dense-prefix chunk."""
        if self.vectors is None:
            raise RuntimeError("no router input was given")
        if self.is_dense(chunk_start):
            return None
        if chunk_start not in self.routed:
            self._issue(self.starts.index(chunk_start) + 1)
        torch.cuda.current_stream(self.q.device).wait_event(self.routed.pop(chunk_start))
        n = min(int(self.q.shape[0]), chunk_start + self.chunk) - chunk_start
        v = self.vectors[self.slot_of[chunk_start], :n]
        return v.view(1, n, v.shape[1], 1, v.shape[2])

    def take(self, chunk_start: int):
        """The calling stream waits for the chunk's launch; returns (partial, lse) or None (dense prefix)."""
        if chunk_start not in self.done:
            self._issue(self.starts.index(chunk_start) + 1)
        torch.cuda.current_stream(self.q.device).wait_event(self.done.pop(chunk_start))
        slot = self.slot_of.get(chunk_start)
        if slot is None:
            return None
        n = min(int(self.q.shape[0]), chunk_start + self.chunk) - chunk_start
        return self.partial[slot, :n], self.lse[slot, :n]

    def release(self, chunk_start: int) -> None:
        """The chunk's sparse launch has been issued on the calling stream: its partial may be reused
        once that launch is over, and the next chunks' windows are issued."""
        slot = self.slot_of.pop(chunk_start, None)
        if slot is not None:
            ev = torch.cuda.Event()
            ev.record(torch.cuda.current_stream(self.q.device))
            self.free.append((slot, ev))
        self._issue(self.starts.index(chunk_start) + 1 + self.depth)

    def finish(self) -> None:
        torch.cuda.current_stream(self.q.device).wait_stream(self.stream)


def fused_chunk_attention(q_chunk: torch.Tensor, query_state, index, q_positions: torch.Tensor,
                          snapshot_state: CausalSnapshot, chunk_start: int, chunk_end: int, *,
                          temperature: float, beta: float, target_tokens: int, queries_per_block: int = 32,
                          sm_scale: float, iters: int = 16, dense_prefix_x: int = 4, out=None,
                          attended=None, local_kv=None, window: "WindowAhead | None" = None, _timer=None,
                          **unused) -> torch.Tensor:
    """Attention of one query chunk (fused_prefill.py:219-482, default path).

    ``query_state.vectors`` [1, Q, Hq, 1, D] routing vectors; ``index.original_kv`` must hold
    the position-ordered (k_post, v) of the prompt: the exact window is read from it.
    ``local_kv`` = (k, v, first_position) replaces it for this call (the streamed mode, which
    keeps no prompt-order copy, hands over the rows of the window it has gathered).
    ``attended`` (int64, optional) accumulates the attended (query, key) pairs of the dense / window
    launch in [0]; with four or more elements the sparse launch counts its pairs in [2] and the rows
    it gathered in [3], otherwise in [0] and [1].  ``window`` (a WindowAhead over the same prompt) has
    issued the dense / window launch already: this call waits for it and merges."""
    import semblo_b200
    semblo_b200.SPARSE_ATTENTION_CALLS += 1
    wstart = chunk_window_start(chunk_start, target_tokens, dense_prefix_x)
    if window is not None:
        if local_kv is not None:
            raise RuntimeError("windows issued ahead read the prompt-order K/V, not rows handed over per call")
        if window.is_dense(chunk_start) != (wstart == 0):
            raise RuntimeError("the windows issued ahead were planned with another budget or window")
        if out is not None and out.data_ptr() != window.out[chunk_start:chunk_end + 1].data_ptr():
            raise RuntimeError("the windows issued ahead write into their own output buffer: pass its rows as out")
        if wstart == 0:
            window.take(chunk_start)
            return window.out[chunk_start:chunk_end + 1]
        k_loc = v_loc = None
        pos0 = 0
    elif local_kv is not None:
        k_loc, v_loc, pos0 = local_kv
        if pos0 > wstart or pos0 + k_loc.shape[0] <= chunk_end:
            raise RuntimeError(f"the window [{wstart}, {chunk_end}] is not inside the rows handed over "
                               f"([{pos0}, {pos0 + k_loc.shape[0] - 1}])")
    else:
        original_kv = getattr(index, "original_kv", None)
        if original_kv is None:
            raise RuntimeError("the prefill body reads the chunk's exact window from the position-ordered K/V "
                               "(index.original_kv)")
        k_loc, v_loc = original_kv
        pos0 = 0

    def window_rows(first):
        return k_loc[first - pos0:chunk_end + 1 - pos0], v_loc[first - pos0:chunk_end + 1 - pos0]

    if wstart == 0:                                        # (not reached with windows issued ahead)
        if _timer:
            _timer("start")
        k_w, v_w = window_rows(0)
        with _attend_part("semblo::attend_dense_prefix"):
            res = window_attention(q_chunk, q_positions, ordered_k=k_w, ordered_v=v_w, ordered_pos0=0,
                                   local_start=0, sm_scale=sm_scale, out=out, attended=attended)
        if _timer:
            _timer("stop")
        return res
    base = snapshot_state.advance(wstart - 1)
    status = _lib.status_for(q_chunk.device)
    sink = _fitted_sink_tokens()
    if sink:
        if snapshot_state.select_sizes is None:
            snapshot_state.select_sizes = torch.empty_like(base)
        select_sizes = snapshot_state.select_sizes
        select_sizes.copy_(base)
        select_sizes[:, 0] = 0                         # _hold_out_sink
        select_target = max(0, int(target_tokens) - sink)
    else:
        select_sizes, select_target = base, int(target_tokens)
    vectors = query_state.vectors[0]
    vectors = vectors.reshape(vectors.shape[0], vectors.shape[1], -1)
    q_count, num_q_heads = q_chunk.shape[0], q_chunk.shape[1]
    snap = snapshot_state
    dev = q_chunk.device
    if snap.qmask is None or snap.qmask.shape[0] < q_count:
        hkv, c = index.num_kv_heads, index.num_buckets
        snap.qmask = torch.empty(q_count, hkv, c // 32, dtype=torch.int32, device=dev)
        snap.score = torch.empty(q_count, hkv, c, dtype=torch.float32, device=dev)
        snap.top1 = torch.empty(hkv, q_count, dtype=torch.int32, device=dev)
        snap.order = torch.empty(hkv, q_count, dtype=torch.int32, device=dev)
        snap.lse = torch.empty(q_count, num_q_heads, dtype=torch.float32, device=dev)
        snap.partial = torch.empty(q_count, num_q_heads, q_chunk.shape[2], dtype=torch.float32, device=dev)
        snap.sort_ws = torch.empty(int(lib().semblo_layout_workspace_bytes(q_count, hkv)), dtype=torch.uint8,
                                   device=dev)
    full = q_count == snap.qmask.shape[0]
    top1 = snap.top1 if full else torch.empty(index.num_kv_heads, q_count, dtype=torch.int32, device=dev)
    order = snap.order if full else torch.empty_like(top1)
    qmask, _ = theta_select_bitmask_flat(vectors, index.codebooks, select_sizes, temperature=temperature,
                                         beta=beta, target_tokens=select_target, iters=iters,
                                         qmask=snap.qmask[:q_count], score=snap.score[:q_count],
                                         force_sink=bool(sink), top1=top1, tile_key_beta=beta)
    # queries whose largest mixture probability falls on the same cluster select nearly the same
    # clusters: tiles are formed in that order so a tile's union of selections stays small
    argsort_keys(top1, index.num_buckets, out=order, workspace=snap.sort_ws)
    # the CTAs with the most rows to gather start first
    n_cta = ((q_count + 128 // (num_q_heads // index.num_kv_heads) - 1) // (128 // (num_q_heads // index.num_kv_heads))) * index.num_kv_heads
    if getattr(snap, "cta_work", None) is None or snap.cta_work.numel() < n_cta:
        snap.cta_work = torch.empty(n_cta, dtype=torch.int32, device=dev)
        snap.cta_order = torch.empty(n_cta, dtype=torch.int32, device=dev)
    cta_order = gather_launch_order(order, qmask, base, num_q_heads, work=snap.cta_work[:n_cta],
                                    out=snap.cta_order[:n_cta])
    if out is None:
        out = torch.empty_like(q_chunk)
    if _timer:
        _timer("start")
    if window is not None:
        partial, lse = window.take(chunk_start)            # waited for only now: scoring and selection need no window
    else:
        lse = snap.lse[:q_count]
        partial = snap.partial[:q_count]
        # the exact window [wstart, q] in position order, then the selected clusters merged into it
        k_w, v_w = window_rows(wstart)
        with _attend_part("semblo::attend_current_chunk"):
            window_attention(q_chunk, q_positions, ordered_k=k_w, ordered_v=v_w, ordered_pos0=wstart,
                             local_start=wstart, sm_scale=sm_scale, out=out, lse=lse, attended=attended,
                             partial=partial)
    if _timer:
        _timer("mid")
    # the kernel gathers the selected rows itself: the reference's gather_kv label has no launch of its own here
    with _attend_part("semblo::attend_selected_clusters"):
        sparse_gather_attention(q_chunk, packed_kv=index.packed_kv, qmask=qmask, causal_sizes=base,
                                indptr=index.bucket_indptr, sm_scale=sm_scale, out=out, lse=lse, merge=True,
                                page_table=getattr(index, "kv_page_table", None), q_order=order,
                                attended=attended[2:] if attended is not None and attended.numel() >= 4 else attended,
                                partial=partial, cta_order=cta_order)
    if _timer:
        _timer("stop")
    if window is not None:
        window.release(chunk_start)
    status.poll()
    return out


def fused_decode_attention(q_chunk: torch.Tensor, query_state, index, q_positions: torch.Tensor, *,
                           temperature: float, beta: float, target_tokens: int, sm_scale: float, iters: int = 16,
                           num_splits: int = 16):
    """Decode over the packed prompt of a request's own index (fused_prefill.py:625-718): select the single
    query's clusters over the full sizes with the sink rule, attend their rows, and return the output with
    its log-sum-exp; the caller merges the generated suffix (paged_attention.paged_posting_attention,
    merge_paged_attention_results).  Served by the kernels of the fused decode step run over the index's
    own buffers, with the routing vectors taken from ``query_state`` as they are."""
    from .fused_decode import FusedDecodeWorkspace
    from .paged_attention import PagedSparseAttentionResult
    require_cuda(q_chunk, index.codebooks, index.packed_kv)
    if q_chunk.ndim != 3 or q_chunk.shape[0] != 1:
        raise ValueError("the decode body takes one query: q_chunk [1, Hq, D]")
    _, hq, d = q_chunk.shape
    hkv, c = int(index.num_kv_heads), int(index.num_buckets)
    vectors = query_state.vectors[0].reshape(1, hq, -1).contiguous()
    if vectors.shape[-1] != d or vectors.dtype != torch.bfloat16:
        raise RuntimeError("the decode body routes with one whole bf16 vector per head (index_dim == head_dim)")
    width = int(index.packed_kv.shape[1])
    posting = index.posting_positions
    if int(posting.shape[1]) != width or not posting.is_contiguous():
        # the kernel reads posting and packed rows with one stride: a padded copy, made once per index
        padded = getattr(index, "_decode_posting", None)
        if padded is None or int(padded.shape[1]) != width:
            padded = torch.zeros(hkv, width, dtype=torch.int32, device=posting.device)
            padded[:, :posting.shape[1]] = posting
            index._decode_posting = padded
        posting = padded
    splits = max(1, int(num_splits))
    ws = getattr(index, "_decode_ws", None)
    key = (hq, hkv, d, c, width, splits)
    if ws is None or ws.shape_key != key:
        ws = FusedDecodeWorkspace(num_q_heads=hq, num_kv_heads=hkv, head_dim=d, num_clusters=c, packed_width=width,
                                  num_splits=splits, device=q_chunk.device)
        index._decode_ws = ws
        index._no_suffix = torch.full((1,), 2 ** 30, dtype=torch.int32, device=q_chunk.device)
    out = torch.empty(1, hq, d, dtype=torch.bfloat16, device=q_chunk.device)
    lse = torch.empty(1, hq, dtype=torch.float32, device=q_chunk.device)
    sink = _fitted_sink_tokens()
    status = _lib.status_for(q_chunk.device)
    positions = q_positions if q_positions.dtype in (torch.int32, torch.int64) else q_positions.to(torch.int32)
    check(lib().semblo_decode_step(
        ptr(q_chunk.contiguous()), ptr(vectors), None, None, None, ptr(positions),
        1 if positions.dtype == torch.int64 else 0, ptr(index.codebooks), ptr(index.bucket_sizes),
        ptr(index.bucket_indptr), ptr(posting), ptr(index.packed_kv), width, None, None, None, 0, 1, 0,
        ptr(index._no_suffix), hq, hkv, d, c, float(temperature), float(beta), int(target_tokens), sink, int(iters),
        float(sm_scale), splits, ptr(ws.buffer), ws.bytes, ptr(out), ptr(status.word), 7, ptr(lse), 1, stream_ptr()))
    status.poll()
    return PagedSparseAttentionResult(output=out, logsumexp=lse)
