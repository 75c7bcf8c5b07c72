"""The decode step of one sparse layer (mirror of semblo/vllm_plugin/fused_decode.py:393-521).

Three launches on the current stream (score + suffix write, select + CSR, attend +
merge; the last two start while their predecessor drains), no host reads and no
allocation after the workspace exists, so a CUDA graph can capture the step."""
from __future__ import annotations

import ctypes
import os

import torch

from . import _lib
from ._lib import check, lib, ptr, require_cuda, stream_ptr


def _pow2_at_least(n: int, floor: int = 16) -> int:
    return max(floor, 1 << (int(n) - 1).bit_length())


class FusedDecodeWorkspace:
    """Fixed-address scratch of the step (fused_decode.py:365-385)."""

    NAMES = ("tickets", "logit", "ml", "split", "rstart", "rlen", "rcum", "rcount", "rtokens",
             "pacc", "pml", "vectors")

    def __init__(self, *, num_q_heads: int, num_kv_heads: int, head_dim: int, num_clusters: int,
                 packed_width: int, num_splits: int, device) -> None:
        self.shape_key = (num_q_heads, num_kv_heads, head_dim, num_clusters, packed_width, num_splits)
        self.num_splits = num_splits
        self.bytes = int(lib().semblo_decode_workspace_bytes(num_q_heads, num_kv_heads, head_dim, num_clusters,
                                                             packed_width, num_splits))
        self.buffer = torch.zeros(self.bytes, dtype=torch.uint8, device=device)
        offs = (ctypes.c_int64 * len(self.NAMES))()
        check(lib().semblo_decode_workspace_offsets(num_q_heads, num_kv_heads, head_dim, num_clusters,
                                                    packed_width, num_splits, ctypes.cast(offs, ctypes.c_void_p)))
        self.offsets = dict(zip(self.NAMES, [int(o) for o in offs]))
        g = num_q_heads // num_kv_heads
        c = num_clusters

        def view(name, dtype, shape):
            n = 1
            for s in shape:
                n *= s
            item = torch.empty(0, dtype=dtype).element_size()
            o = self.offsets[name]
            return self.buffer[o:o + n * item].view(dtype).view(*shape)

        self.logit = view("logit", torch.float32, (num_kv_heads, g, c))
        self.split = view("split", torch.int32, (num_kv_heads, num_splits, 4))
        self.rstart = view("rstart", torch.int32, (num_kv_heads, c))
        self.rlen = view("rlen", torch.int32, (num_kv_heads, c))
        self.rcum = view("rcum", torch.int32, (num_kv_heads, c))
        self.rcount = view("rcount", torch.int32, (num_kv_heads,))
        self.rtokens = view("rtokens", torch.int32, (num_kv_heads,))
        self.vectors = view("vectors", torch.bfloat16, (num_q_heads, head_dim))


def fused_decode_step(layer, arena, *, q_post: torch.Tensor, q_pre: torch.Tensor, positions: torch.Tensor,
                      k_post: torch.Tensor | None, v_states: torch.Tensor | None,
                      k_pre: torch.Tensor | None = None, output: torch.Tensor, temperature: float,
                      beta: float, target_tokens: int, sm_scale: float, num_splits: int, iters: int = 16,
                      stage_mask: int = 7, lse_out: torch.Tensor | None = None, vectors_given: bool = False) -> None:
    """The whole decode step of one layer over ``arena`` into ``output`` [1, Hq * D].

    ``layer`` needs ``num_heads``, ``num_kv_heads`` and ``head_dim``.  The sink rule follows
    SEMBLO_SINK_TOKENS as in the reference (fused_prefill._fitted_sink_tokens).  ``stage_mask``:
    1 score, 2 select, 4 attend (7 = the whole step); adding 8 launches the stages strictly one
    after the other instead of overlapping each with the end of its predecessor.  ``lse_out`` [Hq]
    fp32 receives the natural-log log-sum-exp of the result; ``vectors_given`` says that ``q_pre``
    already holds routing vectors (the step then skips its router)."""
    require_cuda(q_post, q_pre, output)
    hq, hkv, d = int(layer.num_heads), int(layer.num_kv_heads), int(layer.head_dim)
    sink = int(os.environ.get("SEMBLO_SINK_TOKENS", "0") or "0")
    c = int(arena.num_clusters)
    if int(arena.codebooks.shape[-1]) * 2 != d:
        raise RuntimeError(f"the fused decode step routes with the query itself (index_dim must equal head_dim {d})")
    splits = max(1, int(num_splits))
    ws = arena.fused_decode_ws
    key = (hq, hkv, d, c, int(arena.width), splits)
    if ws is None or ws.shape_key != key:
        ws = FusedDecodeWorkspace(num_q_heads=hq, num_kv_heads=hkv, head_dim=d, num_clusters=c,
                                  packed_width=int(arena.width), num_splits=splits, device=q_pre.device)
        arena.fused_decode_ws = ws
    for t in (q_post, q_pre, k_post, v_states, k_pre):
        if t is not None and (t.dtype != torch.bfloat16 or not t.is_contiguous()):
            raise ValueError("the decode step takes contiguous bf16 tensors")
    if positions.dtype not in (torch.int64, torch.int32):
        raise ValueError("positions must be int64 or int32")
    status = _lib.status_for(q_pre.device)
    check(lib().semblo_decode_step(
        ptr(q_post), ptr(q_pre), ptr(k_post), ptr(v_states), ptr(k_pre), ptr(positions),
        1 if positions.dtype == torch.int64 else 0,
        ptr(arena.codebooks), ptr(arena.sizes), ptr(arena.indptr), ptr(arena.posting), ptr(arena.packed_kv),
        int(arena.width), ptr(arena.suffix_kv), ptr(arena.suffix_kpre), ptr(arena.suffix_table),
        int(arena.suffix_blocks), int(arena.suffix_block), int(arena.suffix_table.shape[1]),
        ptr(arena.prompt_length_t), hq, hkv, d, c, float(temperature), float(beta), int(target_tokens), sink,
        int(iters), float(sm_scale), splits, ptr(ws.buffer), ws.bytes, ptr(output), ptr(status.word),
        int(stage_mask), ptr(lse_out), 1 if vectors_given else 0, stream_ptr()))
    status.poll()          # non-blocking; a step learns of the previous step's device-side condition
