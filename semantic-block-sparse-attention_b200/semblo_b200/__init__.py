"""B200-native (sm_100a) implementation of the semblo sparse-attention hot path.

Host side: Python/PyTorch mirrors of the reference's hot-path entry points (same
names and argument meaning) that forward raw device pointers to the hand-written
CUDA kernels in libsemblo_b200.so.  No Triton, no CPU fallback."""
from ._lib import lib, library_path, status_for  # noqa: F401

SPARSE_ATTENTION_CALLS = 0


def sparse_attention_calls() -> int:
    """How many times the sparse attention body ran (reference: model.py:61-71)."""
    return SPARSE_ATTENTION_CALLS
