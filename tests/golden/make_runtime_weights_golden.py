"""Writes tests/golden/runtime_weights/: a small routing-map side-car made by the reference's own writer
(scripts/prepare_nemotron_checkpoint.py:81-100) and verified by its own reader
(semblo/vllm_plugin/runtime_weights.py:158-182).  The reference is not available where the tests run, so the
two files are committed; run from the repository root of a checkout that has the reference beside it:

    python tests/golden/make_runtime_weights_golden.py <path to the reference checkout>

Two layers with a key router each: layer 3 a square map [4, 8, 8], layer 7 a map into fewer dimensions
[4, 6, 8]; seeded, bf16 and fp32.
"""
import json
import pathlib
import sys

import torch


def tensors():
    g = torch.Generator().manual_seed(20240607)
    return {
        "layers.3.self_attn.semblo_key_router.weight": torch.randn(4, 8, 8, generator=g).to(torch.bfloat16),
        "layers.7.self_attn.semblo_key_router.weight": torch.randn(4, 6, 8, generator=g),
    }


CONFIG = {"architectures": ["SembloNemotronHForCausalLM"], "head_dim": 8, "num_key_value_heads": 4,
          "semblo_index_dim": 8, "semblo_layer_indices": [3, 7], "semblo_target_tokens": 4096}


def main() -> None:
    ref = pathlib.Path(sys.argv[1]).resolve()
    sys.path.insert(0, str(ref))
    sys.path.insert(0, str(ref / "scripts"))
    from prepare_nemotron_checkpoint import write_runtime_weights
    from semblo.vllm_plugin.runtime_weights import verify_runtime_weights
    out = pathlib.Path(__file__).resolve().parent / "runtime_weights"
    out.mkdir(exist_ok=True)
    write_runtime_weights(out, tensors(), CONFIG, pathlib.Path("synthetic-snapshot"), script="tests/golden/make_runtime_weights_golden.py")
    manifest = verify_runtime_weights(out)
    print(json.dumps(manifest.to_dict(), indent=1)[:400])


if __name__ == "__main__":
    main()
