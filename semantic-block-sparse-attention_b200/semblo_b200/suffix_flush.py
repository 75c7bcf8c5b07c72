"""Suffix flush: move the older part of the exact generated suffix into the clusters.

Mirrors semblo/vllm_plugin/suffix_flush.py (flush_range 140-151, flush_layer 172-208, repack_apply
97-133) on a DecodeArena.  It runs between decode steps,
eagerly, on the arena's own buffers."""
from __future__ import annotations

import os

import torch

from . import _lib
from ._lib import check, lib, ptr, stream_ptr
from .flat_index import routing_normalize
from .token_outer import nearest_cluster


def flush_every() -> int:
    """suffix_flush.py:29-30."""
    return int(os.environ.get("SEMBLO_SUFFIX_FLUSH_EVERY", "0") or 0)


def keep_exact() -> int:
    """suffix_flush.py:33-34."""
    return int(os.environ.get("SEMBLO_SUFFIX_KEEP_EXACT", "1024") or 1024)


def enabled() -> bool:
    return flush_every() > 0


def flush_range(prompt_len: int, written: int, plen_cur: int, keep: int, every: int):
    """suffix_flush.py:140-151: the positions [frm, to) to move now, or None."""
    live = prompt_len + written - plen_cur
    if live >= keep + every:
        return plen_cur, prompt_len + written - keep
    return None


def flush_arena(arena, frm: int, to: int, align: int | None = None, router=None) -> int:
    """Move suffix positions [frm, to) into their nearest clusters (suffix_flush.py:172-208).

    Reads the rows from the suffix store, assigns each to a cluster per KV head in the routing space
    the prefill used (``router``: the layer's SembloKeyRouter, none or the identity for routing on the
    keys themselves; then the whole-vector normalisation), re-packs the arena's store in place,
    advances the prompt length and extends the ring table.  Returns the widest packed length after
    the flush (one host read, as the reference's own return value)."""
    n = int(to) - int(frm)
    if n <= 0:
        return 0
    if arena.suffix_kpre is None:
        raise RuntimeError("the flush assigns by the pre-RoPE keys: build the arena with keep_kpre=True")
    dev = arena.packed_kv.device
    align = arena.page_align if align is None else max(int(align), 1)
    pos = torch.arange(frm, to, device=dev)
    blk = pos // arena.suffix_block
    phys = arena.suffix_table[0, blk].long()
    off = pos - blk * arena.suffix_block
    kpre = arena.suffix_kpre[phys, off].contiguous()                    # [n, Hkv, D]
    k = arena.suffix_kv[0, phys, off].contiguous()
    v = arena.suffix_kv[1, phys, off].contiguous()
    if router is None or router.is_identity():
        product = routing_normalize(kpre)
    else:
        product = router(kpre[None])[0]                                  # the map, zero padding, normalisation
    assign = nearest_cluster(product, arena.codebooks)                   # [Hkv, n]
    hkv, c = int(arena.sizes.shape[0]), int(arena.sizes.shape[1])
    d = int(arena.packed_kv.shape[-1])
    width = int(arena.packed_kv.shape[1])
    ws_bytes = int(lib().semblo_flush_workspace_bytes(n, hkv, c))
    # the copy of the old store and the workspace live with the arena: a flush between two decode
    # steps allocates nothing of the store's size and the arena's addresses stay what they were
    scratch = getattr(arena, "_flush_scratch", None)
    if scratch is None or scratch[0].shape != arena.packed_kv.shape or scratch[0].device != dev:
        scratch = (torch.empty_like(arena.packed_kv), torch.empty_like(arena.posting))
        arena._flush_scratch = scratch
    old_packed, old_posting = scratch
    ws = getattr(arena, "_flush_ws", None)
    if ws is None or ws.numel() < ws_bytes or ws.device != dev:
        ws = torch.empty(ws_bytes, dtype=torch.uint8, device=dev)
        arena._flush_ws = ws
    # the flush has a status word of its own: a stale code of another call cannot gate it, and the
    # host-side state below is committed only after the device has accepted the new layout
    status = _lib.DeviceStatus(dev)
    check(lib().semblo_flush_repack(ptr(arena.packed_kv), arena.packed_kv.stride(0), width, ptr(arena.posting),
                                    arena.posting.stride(0), ptr(arena.sizes), ptr(arena.indptr), c, hkv, d, align,
                                    ptr(k), ptr(v), ptr(pos.to(torch.int32)), ptr(assign), n, ptr(old_packed),
                                    ptr(old_posting), ptr(ws), ws.numel(), ptr(status.word), stream_ptr()))
    status.raise_if_set()        # refused (the result would not fit): the store is unchanged, as after the
                                 # reference's repack_apply, which raises before it moves anything
    arena.index.prompt_length = int(to)
    arena.index.max_position = int(to)
    arena.prompt_length_t.fill_(int(to))
    arena.extend_suffix_table(int(to) + arena.reserve - 1)
    return int(arena.indptr[:, -1].max().item())


def flush_layer(arena, module, frm: int, to: int, tmp=None) -> int:
    """``flush_arena`` for a layer (suffix_flush.py:172-208 of the reference, which is handed the
    module for its key router; ``tmp`` is the reference's scratch tensor and is not needed here: the
    scratch lives with the arena)."""
    return flush_arena(arena, frm, to, router=getattr(module, "semblo_key_router", None))


class SuffixFlusher:
    """When to flush, across decode steps (suffix_flush.py:211-283 of the reference): one instance per
    process, called on the host before every engine step -- a recorded decode step runs no Python, so
    this is where the flush happens, before the step is replayed on the same buffers.

    ``before_step(runner, scheduler_output)`` reads ``total_num_scheduled_tokens`` and
    ``num_scheduled_tokens`` of the scheduler's output: a step that is not one token of one request
    (a prefill chunk, several requests, nothing) only marks that the next single-token step starts a
    fresh count.  On a single-token step the tokens written since the prompt are counted, and when the
    exact suffix has grown to ``keep + every`` positions all but the newest ``keep`` are moved into
    the clusters of every layer's arena (``flush_layer``).  The runtime state is found on the runner's
    model (``runtime_state`` / ``semblo_runtime_state`` of any module) or handed to the constructor."""

    def __init__(self, state=None) -> None:
        self.keep, self.every = keep_exact(), flush_every()
        self.state = state
        self.epoch = None
        self.prompt_len = self.written = self.flushes = 0
        self.pending_reset = True
        self.log = os.environ.get("SEMBLO_SUFFIX_FLUSH_LOG", "0") == "1"

    def _find_state(self, runner):
        if self.state is None:
            model = getattr(runner, "model", None)
            for _ in range(4):                      # an engine may wrap the model (a graph wrapper, say)
                if model is None or hasattr(model, "modules"):
                    break
                model = getattr(model, "model", getattr(model, "runnable", None))
            if model is not None and hasattr(model, "modules"):
                for module in model.modules():
                    found = getattr(module, "semblo_runtime_state", None) or getattr(module, "runtime_state", None)
                    if found is not None:
                        self.state = found
                        break
        return self.state

    def _arenas(self) -> list:
        return sorted(((int(key[1]), value) for key, value in self.state.index_buffers.items()
                       if isinstance(key, tuple) and len(key) == 2 and key[0] == "arena"), key=lambda kv: kv[0])

    def before_step(self, runner, scheduler_output) -> None:
        total = int(getattr(scheduler_output, "total_num_scheduled_tokens", 0))
        per_request = getattr(scheduler_output, "num_scheduled_tokens", None) or {}
        if total != 1 or len(per_request) != 1:
            self.pending_reset = True
            return
        state = self._find_state(runner)
        if state is None:
            return
        arenas = self._arenas()
        if not arenas or any(getattr(arena, "suffix_kpre", None) is None for _, arena in arenas):
            return
        first = arenas[0][1]
        if self.pending_reset or self.epoch != state.prompt_epoch:
            self.pending_reset, self.epoch = False, state.prompt_epoch
            self.prompt_len, self.written = int(first.index.prompt_length), 0
        due = flush_range(self.prompt_len, self.written, int(first.index.prompt_length), self.keep, self.every)
        if due is not None:
            frm, to = due
            for layer, arena in arenas:
                module = state.source_modules.get(layer)
                if module is None:
                    raise RuntimeError(f"no source module registered for layer {layer}")
                flush_layer(arena, module, frm, to)
            self.flushes += 1
            if self.log:
                print(f"[semblo] suffix flush {self.flushes}: positions [{frm}, {to}) of {len(arenas)} layers moved "
                      f"into the clusters; exact suffix now {self.prompt_len + self.written - to} tokens", flush=True)
        self.written += 1

