"""ctypes binding of libsemblo_b200.so (the C ABI declared in include/semblo_b200.h).

The library is the product: there is no Python or CPU fallback.  Importing this
module does not load it; the first call of :func:`lib` does, and raises if the
shared object has not been built."""
from __future__ import annotations

import ctypes
from ctypes import c_char_p, c_float, c_int, c_int32, c_int64, c_void_p
from pathlib import Path

import torch

_LIB_PATH = Path(__file__).resolve().parent.parent / "libsemblo_b200.so"
_lib = None
CALLS: dict = {}          # entry point -> number of calls (the benchmark's launch accounting)


class _Counting:
    """The loaded library with a per-entry-point call counter."""

    def __init__(self, handle) -> None:
        self._handle = handle
        self._wrapped: dict = {}

    def __getattr__(self, name):
        fn = self._wrapped.get(name)
        if fn is None:
            raw = getattr(self._handle, name)

            def fn(*args, _raw=raw, _name=name):
                CALLS[_name] = CALLS.get(_name, 0) + 1
                return _raw(*args)

            self._wrapped[name] = fn
        return fn

I32P = c_void_p
_SIGNATURES = {
    "semblo_version": (c_int, []),
    "semblo_last_error": (c_char_p, []),
    "semblo_routing_normalize": (c_int, [c_void_p, c_int, c_int64, c_int, c_int64, c_void_p, c_void_p, c_void_p, c_int, c_void_p]),
    "semblo_gather_rows": (c_int, [c_void_p, c_void_p, c_int64, c_int, c_void_p, c_void_p, c_void_p]),
    "semblo_assign_argmax": (c_int, [c_void_p, c_int64, c_void_p, c_int, c_int, c_void_p, c_int, c_void_p, c_void_p]),
    "semblo_cluster_counts": (c_int, [c_void_p, c_int64, c_int64, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p]),
    "semblo_kmeans_update": (c_int, [c_void_p, c_void_p, c_int64, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_void_p]),
    "semblo_kmeans_sort_members": (c_int, [c_void_p, c_int64, c_int, c_void_p, c_int64, c_void_p]),
    "semblo_kmeans_update_sorted": (c_int, [c_void_p, c_int64, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_void_p]),
    "semblo_split_descriptor": (c_int, [c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_void_p]),
    "semblo_layout_workspace_bytes": (c_int64, [c_int64, c_int]),
    "semblo_build_layout": (c_int, [c_void_p, c_int64, c_int, c_int, c_int, c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_void_p]),
    "semblo_pack_kv": (c_int, [c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64, c_int, c_int, c_void_p, c_int64, c_void_p, c_void_p]),
    "semblo_snapshot_advance": (c_int, [c_void_p, c_int64, c_int, c_int64, c_int64, c_int, c_void_p, c_void_p]),
    "semblo_score_clusters": (c_int, [c_void_p, c_int, c_int, c_int, c_void_p, c_int, c_int, c_void_p, c_float, c_float, c_void_p, c_void_p, c_void_p]),
    "semblo_select_clusters": (c_int, [c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_float, c_void_p]),
    "semblo_argsort_keys": (c_int, [c_void_p, c_int64, c_int, c_int, c_void_p, c_void_p, c_int64, c_void_p]),
    "semblo_nearest_cluster": (c_int, [c_void_p, c_int64, c_int, c_int, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p]),
    "semblo_append_rows": (c_int, [c_void_p, c_int64, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_void_p]),
    "semblo_scatter_kv": (c_int, [c_void_p, c_void_p, c_void_p, c_int64, c_int, c_int, c_void_p, c_int64, c_void_p, c_int64, c_int64, c_void_p, c_int64, c_void_p, c_int64, c_int64, c_void_p, c_void_p, c_void_p]),
    "semblo_gather_kv": (c_int, [c_void_p, c_int64, c_void_p, c_int64, c_int64, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p]),
    "semblo_relayout_rows": (c_int, [c_void_p, c_void_p, c_int64, c_int64, c_int, c_void_p, c_void_p, c_int, c_void_p, c_void_p]),
    "semblo_flush_workspace_bytes": (c_int64, [c_int64, c_int, c_int]),
    "semblo_flush_repack": (c_int, [c_void_p, c_int64, c_int64, c_void_p, c_int64, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_int64, c_void_p, c_void_p]),
    "semblo_argsort_keys_static_max_keys": (c_int64, []),
    "semblo_argsort_keys_static": (c_int, [c_void_p, c_int64, c_int, c_int, c_void_p, c_void_p]),
    "semblo_gather_launch_order": (c_int, [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p]),
    "semblo_sparse_prefill_gather": (c_int, [c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_float, c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p]),
    "semblo_window_prefill": (c_int, [c_void_p, c_int, c_int, c_int, c_int, c_void_p, c_void_p, c_void_p, c_int64, c_int, c_int, c_float, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p]),
    "semblo_decode_workspace_bytes": (c_int64, [c_int, c_int, c_int, c_int, c_int64, c_int]),
    "semblo_decode_workspace_offsets": (c_int, [c_int, c_int, c_int, c_int, c_int64, c_int, c_void_p]),
    "semblo_decode_step": (c_int, [c_void_p] * 6 + [c_int] + [c_void_p] * 5 + [c_int64] + [c_void_p] * 3 + [c_int] * 3 + [c_void_p] + [c_int] * 4 + [c_float, c_float, c_int, c_int, c_int, c_float, c_int, c_void_p, c_int64, c_void_p, c_void_p, c_int, c_void_p, c_int, c_void_p]),
    "semblo_paged_attention_workspace_bytes": (c_int64, [c_int, c_int, c_int, c_int]),
    "semblo_paged_posting_attention": (c_int, [c_void_p, c_void_p, c_int, c_void_p, c_int64, c_int, c_void_p, c_int, c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_void_p]),
    "semblo_merge_attention_states": (c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int, c_void_p, c_void_p, c_void_p]),
}


def library_path() -> Path:
    return _LIB_PATH


def exported_symbols() -> list[str]:
    return list(_SIGNATURES)


def lib():
    """The loaded library.  Raises RuntimeError if it has not been built."""
    global _lib
    if _lib is None:
        if not _LIB_PATH.exists():
            raise RuntimeError(
                f"{_LIB_PATH} is missing: build the CUDA extension first "
                "(python semantic-block-sparse-attention_b200/build.py); there is no fallback path")
        handle = ctypes.CDLL(str(_LIB_PATH))
        for name, (res, args) in _SIGNATURES.items():
            fn = getattr(handle, name)
            fn.restype = res
            fn.argtypes = args
        _lib = _Counting(handle)
    return _lib


def ptr(t: torch.Tensor | None):
    """Device pointer of a tensor (None -> NULL)."""
    return None if t is None else c_void_p(t.data_ptr())


def stream_ptr():
    return c_void_p(torch.cuda.current_stream().cuda_stream)


def check(code: int) -> None:
    if code != 0:
        msg = lib().semblo_last_error().decode("utf-8", "replace")
        if code == -1:
            raise ValueError(msg)
        raise RuntimeError(f"semblo_b200 call failed ({code}): {msg}")


def require_cuda(*tensors: torch.Tensor | None) -> None:
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise RuntimeError("semblo_b200 runs on CUDA tensors only; there is no CPU path")


STATUS_TEXT = {0: "ok", 101: "load wait timed out", 102: "mma wait timed out", 103: "softmax wait timed out",
               104: "epilogue wait timed out", 201: "a sized buffer would overflow"}


class DeviceStatus:
    """The int32 status word kernels report device-side conditions into.

    Kernels that change a store refuse to run while the word is non-zero, so the word has to be
    looked at: :meth:`raise_if_set` reads it now (one host synchronisation); :meth:`poll` never
    blocks - it raises what an earlier poll's copy has brought back and queues the next copy, so
    a loop that polls once per chunk or per step learns of a device-side condition one call late."""

    def __init__(self, device) -> None:
        self.word = torch.zeros(1, dtype=torch.int32, device=device)
        self._host = None
        self._event = None

    def _raise(self, code: int) -> None:
        self.word.zero_()
        raise RuntimeError(f"semblo_b200 kernel status {code}: {STATUS_TEXT.get(code, 'unknown')}")

    def raise_if_set(self) -> None:
        self._event = None
        code = int(self.word.item())
        if code:
            self._raise(code)

    def poll(self) -> None:
        if torch.cuda.is_current_stream_capturing():
            return
        if self._event is not None:
            if not self._event.query():
                return
            self._event = None
            code = int(self._host[0])
            if code:
                self._raise(code)
        if self._host is None:
            self._host = torch.zeros(1, dtype=torch.int32).pin_memory()
        self._host.copy_(self.word, non_blocking=True)
        self._event = torch.cuda.Event()
        self._event.record()


_STATUS: dict = {}


def status_for(device) -> DeviceStatus:
    """The status word shared by the calls on ``device`` (a device given without an index means the
    current one)."""
    index = torch.device(device).index
    key = torch.cuda.current_device() if index is None else index
    if key not in _STATUS:
        _STATUS[key] = DeviceStatus(torch.device("cuda", key))
    return _STATUS[key]
