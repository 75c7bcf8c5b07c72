"""The runtime configuration fields the sparse-attention hot path reads.

A subset of semblo/vllm_plugin/config.py:92-200 (SembloVllmConfig) with the same names and
meanings; the fields that configure other parts of the plugin (weights files, profiling,
ablations) are not here.  ``validate`` refuses what this build does not implement."""
from __future__ import annotations

import os
from dataclasses import dataclass, field
from typing import Any


def _get(config: Any, name: str, default: Any) -> Any:
    """A key of a checkpoint config given as a dict or as an object with attributes."""
    return config.get(name, default) if isinstance(config, dict) else getattr(config, name, default)


def _as_bool(config: Any, name: str, default: bool) -> bool:
    """Command-line overrides arrive as text, and bool("False") is True (config.py:45-60)."""
    raw = _get(config, name, default)
    if not isinstance(raw, str):
        return bool(raw)
    word = raw.strip().lower()
    if word in ("true", "1", "yes", "on"):
        return True
    if word in ("false", "0", "no", "off", ""):
        return False
    raise ValueError(f"{name}: cannot read {raw!r} as a boolean")


# slice sizes of an earlier streamed prefill: refused rather than ignored (config.py:15-43)
_STALE_CHUNK_VARIABLES = ("SEMBLO_ATTN_CHUNK", "SEMBLO_MLP_CHUNK", "SEMBLO_GDN_CHUNK", "SEMBLO_MLP_SPLIT_GRAPH")


@dataclass(frozen=True)
class SembloVllmConfig:
    token_capacity: int                       # longest prompt a layer's decode arena is shaped for
    target_tokens: int                        # selection budget per query and KV head
    flat_unit_tokens: int                     # mean tokens per block: C = L / flat_unit_tokens
    index_dim: int                            # routing dimension (head_dim: identity or square map; less: a narrowing map)
    mode: str = "sparse"
    num_factors: int = 1
    num_centroids: int = 0
    kmeans_iters: int = 8
    kmeans_sample_size: int = 8192
    kmeans_init: str = "random"
    kmeans_preprocess: str = "none"
    codebook_seed: int = 0
    pack_prompt_kv: bool = True
    fused_select_block_queries: int = 32
    selection_temperature: float = 0.1
    bucket_size_penalty: float = 0.25
    layer_target_tokens: dict = field(default_factory=dict)
    decode_target_tokens: int = 0
    flat_min_clusters_log2: int = 9
    own_prompt_cache: bool = True
    engage_above_tokens: int = 0
    fa3_page_size: int = 16
    fa3_page_align: int = 16
    kv_outer: bool = True
    query_chunk_size: int = 8192
    decode_num_splits: int = 8                # splits of the generated-suffix attention
    packed_decode_num_splits: int = 32        # splits of the selected-cluster attention (doubled by the layer)
    triton_token_tile: int = 16
    runtime_checks: bool = True
    layer_indices: tuple = ()                 # the sparse layers
    prefill_chunk: int = 0                    # slice size of a streamed prefill (0: whole)
    dense_tail_tokens: int = 0
    runtime_weights_file: str | None = None   # the routing maps' side-car (runtime_weights.py)
    runtime_manifest_file: str | None = None
    runtime_allow_unused_layers: bool = False

    @classmethod
    def from_hf_config(cls, config: Any, *, identity_router: bool = False) -> "SembloVllmConfig":
        """The ``semblo_*`` keys of a checkpoint config (dict or object; its ``text_config`` when it has
        one), as config.py:205-335 of the reference reads them: same keys, same defaults, and the same
        environment overrides -- SEMBLO_TARGET_TOKENS, SEMBLO_DECODE_TARGET_TOKENS, SEMBLO_DENSE_TAIL_TOKENS,
        SEMBLO_PREFILL_CHUNK, SEMBLO_RUNTIME_CHECKS win over the config (budgets stay out of the engine's
        compile-cache key that way), and SEMBLO_ENGAGE_ABOVE_TOKENS does unless SEMBLO_FULL_GRAPH_DECODE=1,
        under which every request engages the index (the recorded step is the sparse one).  Only the
        fields this package reads are kept.  ``identity_router``: the maps are identities built in
        memory, so no side-car file may be named."""
        text = _get(config, "text_config", None)
        text = config if text is None else text
        env = os.environ
        enabled = bool(_get(text, "semblo_enabled", False))
        mode = str(_get(text, "semblo_vllm_mode", "sparse" if enabled else "dense_passthrough"))
        layers = _get(text, "semblo_layer_indices", None)
        if layers is None:
            layers = [i for i, kind in enumerate(_get(text, "layer_types", ())) if kind == "full_attention"]
        per_layer = _get(text, "semblo_target_tokens_per_layer", None)
        if per_layer is not None and not isinstance(per_layer, dict):
            raise ValueError("semblo_target_tokens_per_layer must be a mapping of layer index to token budget")
        for stale in _STALE_CHUNK_VARIABLES:
            if stale in env:
                raise ValueError(f"{stale} is gone: a long prefill streams in slices of SEMBLO_PREFILL_CHUNK tokens")
        checks = env.get("SEMBLO_RUNTIME_CHECKS")
        weights_file = str(_get(text, "semblo_runtime_weights_file", "")) or None
        if identity_router and weights_file:
            raise ValueError("identity routing maps are built in memory: the config must not name a weights file")
        cfg = cls(
            token_capacity=int(_get(text, "semblo_vllm_token_capacity", 8192)),
            target_tokens=int(env.get("SEMBLO_TARGET_TOKENS", _get(text, "semblo_target_tokens", 4096))),
            flat_unit_tokens=int(_get(text, "semblo_flat_unit_tokens", 0)),
            index_dim=int(_get(text, "semblo_index_dim", 128)),
            mode=mode,
            num_factors=1,       # the flat partition; ``semblo_num_factors`` only says how descriptors are stored (two halves)
            num_centroids=int(_get(text, "semblo_num_centroids", 64)),
            kmeans_iters=int(_get(text, "semblo_kmeans_iters", 4)),
            kmeans_sample_size=int(_get(text, "semblo_kmeans_sample_size", 8192)),
            kmeans_init=str(_get(text, "semblo_kmeans_init", "random")),
            kmeans_preprocess=str(_get(text, "semblo_kmeans_preprocess", "none")),
            codebook_seed=int(_get(text, "semblo_vllm_codebook_seed", 0)),
            pack_prompt_kv=bool(_get(text, "semblo_vllm_pack_prompt_kv", False)),
            fused_select_block_queries=int(_get(text, "semblo_fused_select_block_queries", 0)),
            selection_temperature=float(_get(text, "semblo_selection_temperature", 0.05)),
            bucket_size_penalty=float(_get(text, "semblo_bucket_size_penalty", 0.0)),
            layer_target_tokens={int(k): int(v) for k, v in (per_layer or {}).items()},
            decode_target_tokens=int(env.get("SEMBLO_DECODE_TARGET_TOKENS", _get(text, "semblo_decode_target_tokens", 0))),
            flat_min_clusters_log2=int(_get(text, "semblo_flat_min_clusters_log2", 9)),
            own_prompt_cache=_as_bool(text, "semblo_vllm_own_prompt_cache", False),
            engage_above_tokens=0 if env.get("SEMBLO_FULL_GRAPH_DECODE") == "1" else int(
                env.get("SEMBLO_ENGAGE_ABOVE_TOKENS", _get(text, "semblo_vllm_engage_above_tokens", 131072))),
            fa3_page_size=int(_get(text, "semblo_fa3_page_size", 16)),
            fa3_page_align=int(_get(text, "semblo_fa3_page_align", 16)),
            kv_outer=bool(_get(text, "semblo_kv_outer", True)),
            query_chunk_size=int(_get(text, "semblo_vllm_query_chunk_size", 256)),
            decode_num_splits=int(_get(text, "semblo_vllm_decode_num_splits", 8)),
            packed_decode_num_splits=int(_get(text, "semblo_vllm_packed_decode_num_splits", 32)),
            triton_token_tile=int(_get(text, "semblo_vllm_token_tile", 16)),
            runtime_checks=(checks.strip().lower() not in ("0", "false", "off", "")) if checks is not None
            else bool(_get(text, "semblo_vllm_runtime_checks", True)),
            layer_indices=tuple(int(i) for i in layers),
            prefill_chunk=int(env.get("SEMBLO_PREFILL_CHUNK", _get(text, "semblo_vllm_prefill_chunk", 0))),
            dense_tail_tokens=int(env.get("SEMBLO_DENSE_TAIL_TOKENS", _get(text, "semblo_dense_tail_tokens", 0))),
            runtime_weights_file=weights_file,
            runtime_manifest_file=str(_get(text, "semblo_runtime_manifest_file", "")) or None,
            runtime_allow_unused_layers=bool(_get(text, "semblo_runtime_allow_unused_layers", False)),
        )
        cfg.validate()
        return cfg

    def validate(self) -> None:
        if self.mode != "sparse":
            raise ValueError("only mode='sparse' is implemented")
        if not self.pack_prompt_kv or self.fused_select_block_queries <= 0:
            raise ValueError("the sparse path needs the packed prompt K/V and the fused selection")
        if not self.own_prompt_cache:
            raise ValueError("the prompt is served from the layer's own cluster-ordered copy (own_prompt_cache)")
        if self.num_factors != 1 or self.kmeans_init != "random" or self.kmeans_preprocess != "none":
            raise ValueError("only the flat partition with random initialisation is implemented")
        if self.flat_unit_tokens <= 0:
            raise ValueError("flat_unit_tokens must be positive")
        if self.dense_tail_tokens:
            raise ValueError("a dense tail (SEMBLO_DENSE_TAIL_TOKENS / semblo_dense_tail_tokens) is not implemented")
        if self.target_tokens <= 0 or self.decode_target_tokens < 0:
            raise ValueError("token budgets must be positive")
        if self.target_tokens > self.token_capacity:
            raise ValueError(f"token_capacity ({self.token_capacity}) must be at least target_tokens "
                             f"({self.target_tokens})")
        for layer, budget in self.layer_target_tokens.items():
            if not 0 < budget <= self.token_capacity:
                raise ValueError(f"the target_tokens of layer {layer} ({budget}) must lie in (0, token_capacity "
                                 f"{self.token_capacity}]")
        if self.selection_temperature <= 0 or self.query_chunk_size <= 0 or self.prefill_chunk < 0:
            raise ValueError("selection_temperature and query_chunk_size must be positive, prefill_chunk not negative")
