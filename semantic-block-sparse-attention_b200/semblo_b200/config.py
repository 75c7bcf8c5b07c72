"""The runtime configuration fields the sparse-attention hot path reads.

A subset of semblo/vllm_plugin/config.py:92-200 (SembloVllmConfig) with the same names and
meanings; the fields that configure other parts of the plugin (weights files, profiling,
ablations) are not here.  ``validate`` refuses what this build does not implement."""
from __future__ import annotations

from dataclasses import dataclass, field


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
