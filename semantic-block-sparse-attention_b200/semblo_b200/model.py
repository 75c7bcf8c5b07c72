"""The sparse-attention layer body behind the ``semblo::attention`` operator.

Mirror of the hot-path half of semblo/vllm_plugin/model.py (SembloAttention):
``_init_semblo_runtime`` 302-354, ``_fit_index`` / ``_build_or_append_index`` 378-430,
``_query_state`` 432-489, ``_decode_buffers`` / ``_decode_body`` 556-616, ``_arena`` 618-661,
``_adopt_into_arena`` 663-676, ``_full_graph_decode_step`` 708-747, ``_captured_decode_step`` 788-854,
``_run_product_attention`` 856-1008, ``_ensure_own_suffix_store`` / ``_write_own_suffix`` 1384-1429,
``_sparse_layer_forward`` 1130-1167, ``attention_forward`` 1169-1269,
``begin_streamed_prefill`` / ``begin_token_outer_prefill`` 1271-1287, ``_ingest_prompt_kv`` 1301-1382
and ``StreamedPrefillSession`` 1431-1529, for the configuration the kernels serve: flat partition,
identity routing map with whole-vector normalisation, the layer's own cluster-ordered prompt
copy (own_prompt_cache); generated tokens go through the fused decode step over the decode arena
(SEMBLO_FULL_GRAPH_DECODE=1) or, without an arena, through the decode kernels over the request's own
index plus the layer's store of generated K/V, recorded once per request as a CUDA graph
(decode_graph.DecodeStepGraph).  The model-specific
subclass sets ``num_heads / num_kv_heads / head_dim / scaling / is_kv_shared_layer`` and
``attn.layer_name``, implements ``_project_qkv`` and ``_finish_output``, and calls
``_init_semblo_runtime``; everything that differs from the served configuration raises."""
from __future__ import annotations

import os
from types import SimpleNamespace

import torch
from torch import nn

import semblo_b200

from . import _lib
from . import arena as _arena
from . import fused_decode as _fused_decode
from . import fused_prefill as _fused_prefill
from .attention_op import register_layer, sparse_attention_op
from .config import SembloVllmConfig
from .decode_graph import DecodeStepGraph, tensor_signature
from .paged_attention import PostingTiles, merge_paged_attention_results, paged_posting_attention
from .routing_map import SembloKeyRouter
from .flat_index import routing_normalize
from .state import ProductPostingIndex, SembloRuntimeState
from .trivial_router import trivial_router_vectors


class SembloAttention(nn.Module):
    """Sparse attention for one full-attention layer."""

    def _init_semblo_runtime(self, *, runtime_config: SembloVllmConfig, runtime_state: SembloRuntimeState,
                             layer_idx: int, source_layer_idx: int, uses_sparse_attention: bool = True,
                             builds_product_index: bool = True,
                             attention_logits_soft_cap: float | None = None) -> None:
        """Requires ``num_heads / num_kv_heads / head_dim / scaling`` to be set already."""
        runtime_config.validate()
        if attention_logits_soft_cap:
            raise RuntimeError("the fused sparse path has no logit soft cap")
        if int(runtime_config.index_dim) > int(self.head_dim):
            raise RuntimeError("the kernels route in a space of the head dimension: index_dim must not exceed "
                               "head_dim (the identity map, a loaded square map, or a map into fewer dimensions, "
                               "which is padded with zeros)")
        self.layer_idx = int(layer_idx)
        self.source_layer_idx = int(source_layer_idx)
        self.uses_sparse_attention = bool(uses_sparse_attention)
        self.builds_product_index = bool(builds_product_index)
        self.runtime_config = runtime_config
        self.runtime_state = runtime_state
        self.attention_logits_soft_cap = attention_logits_soft_cap
        self.layer_target_tokens = runtime_config.layer_target_tokens.get(self.layer_idx, runtime_config.target_tokens)
        self.layer_decode_target_tokens = (
            self.layer_target_tokens
            if self.layer_idx in runtime_config.layer_target_tokens or not runtime_config.decode_target_tokens
            else runtime_config.decode_target_tokens)
        self._effective_target = self.layer_target_tokens
        self._decode_graph = DecodeStepGraph(f"layer {self.layer_idx}")
        self._decode_buffers_cache = None
        if not hasattr(self, "is_kv_shared_layer"):
            self.is_kv_shared_layer = False
        if self.builds_product_index:
            # the routing map of this layer's keys and of the queries of every layer that reads its index:
            # the identity until a map is loaded into ``semblo_key_router.weight``
            self.semblo_key_router = SembloKeyRouter(self.num_kv_heads, self.head_dim, int(runtime_config.index_dim))
            runtime_state.register_source_module(self.layer_idx, self)
        layer_name = getattr(getattr(self, "attn", None), "layer_name", None)
        if layer_name is not None:
            register_layer(layer_name, self)

    # ---- the traced side -----------------------------------------------------------------
    def _positions_for_runtime(self, positions: torch.Tensor):
        return positions, positions

    def _sparse_layer_forward(self, positions: torch.Tensor, hidden_states: torch.Tensor) -> torch.Tensor:
        rope_positions, positions = self._positions_for_runtime(positions)
        q_post, k_post, v_states, q_pre, k_pre, gate = self._project_qkv(rope_positions, hidden_states)
        attn_output = torch.empty_like(q_post)
        sparse_attention_op(positions, hidden_states, q_post, k_post, v_states, q_pre, k_pre, attn_output,
                            self.attn.layer_name)
        return self._finish_output(attn_output, gate)

    # ---- index ---------------------------------------------------------------------------
    def _source_module(self) -> "SembloAttention":
        return self.runtime_state.get_source_module(self.source_layer_idx)

    def _fit_index(self, product, positions) -> ProductPostingIndex:
        if positions.numel() < 128:
            raise ValueError("sparse prefill requires at least 128 prompt tokens after chat formatting")
        cfg = self.runtime_config
        return ProductPostingIndex.build(
            product, positions, num_centroids=cfg.num_centroids, kmeans_iters=cfg.kmeans_iters,
            kmeans_sample_size=cfg.kmeans_sample_size, codebook_seed=cfg.codebook_seed + self.source_layer_idx,
            layer_idx=self.source_layer_idx, flat_unit_tokens=cfg.flat_unit_tokens,
            flat_min_clusters_log2=cfg.flat_min_clusters_log2, page_align=cfg.fa3_page_align)

    def _build_or_append_index(self, k_pre_rope: torch.Tensor, positions: torch.Tensor) -> ProductPostingIndex:
        if not self.builds_product_index:
            raise RuntimeError("only layers with their own K/V can build an index")
        if self.runtime_state.step_first_position != 0:
            return self.runtime_state.get(self.source_layer_idx)
        # SembloKeyRouter (routing_map.py:35-94): the map, then unit-normalise the whole vector
        router = self._router(k_pre_rope.device)
        keys = k_pre_rope.view(-1, self.num_kv_heads, self.head_dim)
        product = routing_normalize(keys) if router.is_identity() else router(keys[None])[0]
        index = self._fit_index(product, positions)
        self.runtime_state.put(self.source_layer_idx, index)
        return index

    def _router(self, device) -> SembloKeyRouter:
        router = self.semblo_key_router
        if router.weight.device != torch.device(device):
            router.to(device)
        return router

    def _query_state(self, q_pre_rope: torch.Tensor, source: "SembloAttention"):
        """Routing vectors of [Q, Hq, D] pre-RoPE queries: a query goes through the map of its KV head
        in the source layer and is normalised like the keys; one per head, uniform mixture."""
        if (os.environ.get("SEMBLO_ROUTING_NORMALIZE", "whole") or "whole") != "whole":
            raise RuntimeError("only SEMBLO_ROUTING_NORMALIZE=whole is implemented")
        queries, heads, dim = q_pre_rope.shape
        router = source._router(q_pre_rope.device)
        projected = q_pre_rope if router.is_identity() else router.widen(router.project_queries(q_pre_rope)).contiguous()
        vectors = trivial_router_vectors(projected).view(1, queries, heads, 1, dim)
        return SimpleNamespace(vectors=vectors, mixture_weights=None)

    # ---- one generated token without an arena ------------------------------------------------
    def _decode_buffers(self, q: torch.Tensor) -> tuple:
        """Output, query position and request id of the recorded step: made once per shape and
        rewritten in place, since a recording replays the addresses it was taken with."""
        cached = self._decode_buffers_cache
        if cached is None or cached[0] != tuple(q.shape) or cached[1].device != q.device:
            cached = (tuple(q.shape), torch.empty_like(q),
                      torch.empty(q.shape[0], dtype=torch.int32, device=q.device),
                      torch.zeros(q.shape[0], dtype=torch.int32, device=q.device))
            self._decode_buffers_cache = cached
            self._decode_graph.reset()
        return cached[1], cached[2], cached[3]

    def _paged_context(self):
        """Where the generated K/V of this layer's source live: the runtime state's suffix store,
        addressed by absolute position through its block table like a paged cache."""
        state = self.runtime_state
        buf = state.suffix_kv.get(self.source_layer_idx)
        if buf is None or state.suffix_block_table is None:
            raise RuntimeError("own_prompt_cache: the suffix store is read before any generated token was "
                               "written to it")
        return SimpleNamespace(kv_cache=buf, block_table=state.suffix_block_table,
                               block_size=int(state.suffix_block_size))

    def _decode_body(self, q, q_pre_rope, positions, index, context, source, out, q_positions, request_ids,
                     posting, suffix_tiles) -> None:
        """One generated token into ``out``: selected clusters of the prompt, the generated suffix,
        merged by their log-sum-exp.  Straight-line, no host read: this is what gets recorded."""
        q_positions.copy_(positions)
        query_state = self._query_state(q_pre_rope, source)
        cfg = self.runtime_config
        prompt_result = _fused_prefill.fused_decode_attention(
            q, query_state, index, q_positions, temperature=cfg.selection_temperature,
            beta=cfg.bucket_size_penalty, target_tokens=int(self._effective_target), sm_scale=self.scaling,
            num_splits=cfg.packed_decode_num_splits * 2)
        suffix_result = paged_posting_attention(
            q, context.kv_cache, posting, suffix_tiles, q_positions, request_ids, context.block_table,
            block_size=context.block_size, sm_scale=self.scaling, softcap=self.attention_logits_soft_cap,
            token_tile=cfg.triton_token_tile, num_splits=cfg.decode_num_splits, return_logsumexp=True)
        out.copy_(merge_paged_attention_results(prompt_result, suffix_result).output)

    def _captured_decode_step(self, q, q_pre_rope, positions, index, context, source) -> torch.Tensor:
        """The chunk loop's decode branch without the loop: one query, no allocation that varies and
        no host-side value that changes from step to step, recorded once and replayed."""
        out, q_positions, request_ids = self._decode_buffers(q)
        posting, starts, lengths, counts, selected = self.runtime_state.suffix_tiles_for_step(
            index, num_kv_heads=self.num_kv_heads, tile_size=self.runtime_config.triton_token_tile)
        suffix_tiles = PostingTiles(starts, lengths, counts, selected)

        def body() -> None:
            self._decode_body(q, q_pre_rope, positions, index, context, source, out, q_positions, request_ids,
                              posting, suffix_tiles)

        self._decode_graph.run(
            (("num_buckets", int(index.num_buckets)), ("target", int(self._effective_target)),
             tensor_signature(q=q, q_pre=q_pre_rope, positions=positions, out=out, q_positions=q_positions,
                              request_ids=request_ids, packed_kv=index.packed_kv,
                              posting_positions=index.posting_positions, codebooks=index.codebooks,
                              bucket_sizes=index.bucket_sizes, bucket_indptr=index.bucket_indptr,
                              kv_cache=context.kv_cache, block_table=context.block_table, suffix_posting=posting,
                              suffix_starts=starts, suffix_lengths=lengths, suffix_counts=counts)),
            body)
        return out

    def _ensure_own_suffix_store(self, index, like) -> None:
        """The layer's store of generated K/V, sized by what the request can still generate."""
        prompt_length = int(index.prompt_length)
        limit = int(self.runtime_state.max_model_len)
        if limit <= prompt_length:
            raise RuntimeError(f"own_prompt_cache: max_model_len {limit} leaves no room for a suffix after a "
                               f"{prompt_length}-token prompt")
        previous = self.runtime_state.suffix_kv.get(self.source_layer_idx)
        buf = self.runtime_state.ensure_suffix_store(
            self.source_layer_idx, prompt_length=prompt_length, max_model_len=limit, num_kv_heads=self.num_kv_heads,
            head_dim=self.head_dim, dtype=like.dtype, device=like.device)
        if previous is not buf:
            self._decode_graph.reset()            # the recording would read the previous request's store

    def _write_own_suffix(self, k_post, v_states, positions) -> None:
        """One generated token's K/V into the layer's store (prompt positions live in the
        cluster-ordered copy only)."""
        index = self.runtime_state.source_indexes.get(self.source_layer_idx)
        if index is None or int(self.runtime_state.step_first_position) < int(index.prompt_length):
            return
        self.runtime_state.write_suffix_kv(
            self.source_layer_idx, positions, k_post.view(-1, self.num_kv_heads, self.head_dim),
            v_states.view(-1, self.num_kv_heads, self.head_dim))

    # ---- arena ---------------------------------------------------------------------------
    def _arena(self, like: torch.Tensor):
        cfg = self.runtime_config
        unit_tokens = int(os.environ.get("SEMBLO_FLAT_UNIT_TOKENS", cfg.flat_unit_tokens))
        if unit_tokens <= 0:
            raise RuntimeError("the decode arena needs the flat index (flat_unit_tokens > 0)")
        from . import suffix_flush as _flush
        room = int(self.runtime_state.max_model_len) - int(cfg.token_capacity)
        reserve = _arena.suffix_reserve(room)
        extra = dict(reserve=reserve)
        if _flush.enabled():
            if os.environ.get("SEMBLO_ROUTING_CENTER") == "1":
                raise RuntimeError("the suffix flush does not re-centre keys (SEMBLO_ROUTING_CENTER=1)")
            if _flush.keep_exact() + _flush.flush_every() > reserve:
                raise RuntimeError("SEMBLO_SUFFIX_KEEP_EXACT + SEMBLO_SUFFIX_FLUSH_EVERY must not exceed the "
                                   f"suffix reserve ({reserve})")
            extra.update(packed_capacity=int(self.runtime_state.max_model_len),
                         table_positions=int(self.runtime_state.max_model_len) + reserve, keep_kpre=True)
        elif room > reserve:
            raise RuntimeError(f"the arena reserves {reserve} generated positions but max_model_len "
                               f"{self.runtime_state.max_model_len} minus the token capacity "
                               f"{cfg.token_capacity} allows {room}")
        return _arena.arena_for(
            self.runtime_state, self.source_layer_idx, capacity=int(cfg.token_capacity), unit_tokens=unit_tokens,
            min_clusters_log2=max(3, int(os.environ.get("SEMBLO_FLAT_MIN_CLUSTERS_LOG2", cfg.flat_min_clusters_log2))),
            num_kv_heads=self.num_kv_heads, head_dim=self.head_dim, index_dim=self.head_dim,   # the routed width
            page_align=int(os.environ.get("SEMBLO_FA3_ALIGN", cfg.fa3_page_align)), kv_dtype=like.dtype,
            desc_dtype=like.dtype, device=like.device, **extra)

    def _adopt_into_arena(self) -> None:
        """After a request's prefill: its index moves into the layer's arena."""
        index = self.runtime_state.source_indexes.get(self.source_layer_idx)
        if index is None or index.packed_kv is None:
            return
        self._arena(index.packed_kv).adopt(index, self.runtime_state.prompt_epoch)

    def _target_for_step(self, is_decode: bool) -> int:
        return self.layer_decode_target_tokens if is_decode else self.layer_target_tokens

    def _full_graph_decode_step(self, positions, q_post, k_post, v_states, q_pre, output, k_pre=None) -> None:
        """One generated token: the fused step over the layer's fixed-address arena.  No host
        state, so the caller may be capturing a CUDA graph."""
        arena = self._source_module()._arena(q_post)
        if not self.is_kv_shared_layer and (k_post is None or v_states is None):
            raise RuntimeError("physical sparse layers must produce K/V")
        self._effective_target = self._target_for_step(True)
        shared = self.is_kv_shared_layer
        source = self._source_module()
        given = not source._router(q_post.device).is_identity()
        if given:                                     # a loaded map: the step is handed the routing vectors
            q_pre = self._query_state(q_pre.view(-1, self.num_heads, self.head_dim), source).vectors \
                .view(-1, self.num_heads, self.head_dim).contiguous()
        _fused_decode.fused_decode_step(
            self, arena, q_post=q_post, q_pre=q_pre, positions=positions,
            k_post=None if shared else k_post.view(-1, self.num_kv_heads, self.head_dim),
            v_states=None if shared else v_states.view(-1, self.num_kv_heads, self.head_dim),
            k_pre=None if shared or k_pre is None else k_pre.view(-1, self.num_kv_heads, self.head_dim),
            output=output, temperature=self.runtime_config.selection_temperature,
            beta=self.runtime_config.bucket_size_penalty, target_tokens=int(self._effective_target),
            sm_scale=self.scaling, num_splits=self.runtime_config.packed_decode_num_splits * 2, vectors_given=given)

    # ---- prompt --------------------------------------------------------------------------
    def _ingest_prompt_kv(self, k_post, v_states, k_pre, positions, *, prompt_order_views: bool = True) -> None:
        """Build the index from the pre-RoPE keys and pack the prompt's post-RoPE K/V in cluster
        order.  ``prompt_order_views`` leaves views of this call's K/V on the index: the chunk loop
        reads each chunk's exact local window from them."""
        if self.is_kv_shared_layer:
            return
        if k_post is None or v_states is None:
            raise RuntimeError("physical sparse layers must produce K/V")
        if not self.builds_product_index:
            return
        if k_pre is None:
            raise RuntimeError("a product-index source must produce pre-RoPE keys")
        index = self._build_or_append_index(k_pre, positions)
        if index.packed_kv is not None and self.runtime_state.step_first_position >= int(index.prompt_length):
            self._write_own_suffix(k_post, v_states, positions)
            return
        if index.packed_kv is None:
            k3 = k_post.view(-1, self.num_kv_heads, self.head_dim)
            v3 = v_states.view(-1, self.num_kv_heads, self.head_dim)
            index.pack_prompt_kv(k3, v3)
            if prompt_order_views:
                index.original_kv = (k3, v3)
            if _arena.full_graph_decode_enabled():
                self._arena(k_post).install_suffix_store(int(index.prompt_length))
            else:
                self._ensure_own_suffix_store(index, k_post)

    def _run_product_attention(self, q_post_rope, q_pre_rope, positions, out=None, query_offset: int = 0,
                               window=None):
        """Sparse attention for the given prompt queries, written into ``out`` if given.
        ``query_offset`` is where these queries start in the prompt; ``window`` (a
        fused_prefill.WindowAhead over these queries and ``out``) has issued the index-free launches."""
        semblo_b200.SPARSE_ATTENTION_CALLS += 1
        source = self._source_module()
        index = self.runtime_state.get(self.source_layer_idx)
        q = q_post_rope.view(-1, self.num_heads, self.head_dim)
        q_pre = q_pre_rope.view(-1, self.num_heads, self.head_dim)
        output = out.view(-1, self.num_heads, self.head_dim) if out is not None else torch.empty_like(q)
        if self.runtime_state.step_first_position >= int(index.prompt_length):
            if positions.numel() != 1:
                raise RuntimeError("one generated token per step")
            self.runtime_state.record_decode_positions(index, 1)
            self._effective_target = self._target_for_step(True)
            step_out = self._captured_decode_step(q.contiguous(), q_pre.contiguous(), positions, index,
                                                  source._paged_context(), source)
            output.copy_(step_out)
            return output.flatten(-2, -1)
        self._effective_target = self._target_for_step(False)
        step = self.runtime_config.query_chunk_size
        n_queries = positions.numel()
        fused_snapshot = None
        for start in range(0, n_queries, step):
            end = min(n_queries, start + step)
            q_positions = positions[start:end].to(torch.int32)
            if window is not None and window.vectors is not None:
                query_state = SimpleNamespace(vectors=window.vectors_for(start), mixture_weights=None)
            else:
                query_state = self._query_state(q_pre[start:end], source)
            if fused_snapshot is None:
                fused_snapshot = getattr(index, "_token_outer_snapshot", None) or _fused_prefill.CausalSnapshot(index)
            _fused_prefill.fused_chunk_attention(
                q[start:end], query_state, index, q_positions, fused_snapshot, start + query_offset,
                end - 1 + query_offset, temperature=self.runtime_config.selection_temperature,
                beta=self.runtime_config.bucket_size_penalty, target_tokens=int(self._effective_target),
                queries_per_block=self.runtime_config.fused_select_block_queries, sm_scale=self.scaling,
                dense_prefix_x=4, out=output[start:end], window=window)
        if window is not None:
            window.finish()
        if getattr(index, "original_kv", None) is not None:
            index.original_kv = None                  # the views are dropped once the prompt has been attended
        _lib.status_for(q.device).poll()
        return output.flatten(-2, -1)

    def attention_forward(self, positions, hidden_states, q_post, k_post, v_states, q_pre, k_pre, output) -> None:
        """The attention core, reached only through the operator; the result goes into ``output``."""
        if _arena.full_graph_decode_enabled() and positions.numel() == 1:
            self._full_graph_decode_step(positions, q_post, k_post, v_states, q_pre, output, k_pre=k_pre)
            return
        self.runtime_state.maybe_begin_prompt(self.layer_idx, positions,
                                              engage_above_tokens=self.runtime_config.engage_above_tokens)
        if self.runtime_state.dense_request or not self.uses_sparse_attention:
            raise RuntimeError("this layer serves the sparse path only: the stock attention of a dense request "
                               "stays with the model's own attention layer")
        if positions.numel() > 1 and self._windows_ahead_enabled(k_post, v_states):
            self._prompt_with_windows_ahead(positions, q_post, k_post, v_states, q_pre, k_pre, output)
        else:
            self._ingest_prompt_kv(k_post, v_states, k_pre, positions)
            sparse_output = self._run_product_attention(q_post, q_pre, positions, out=output)
            if sparse_output.data_ptr() != output.data_ptr():
                output.copy_(sparse_output.view(output.shape))
        if _arena.full_graph_decode_enabled() and positions.numel() > 1:
            self._adopt_into_arena()

    def _windows_ahead_enabled(self, k_post, v_states) -> bool:
        """``SEMBLO_WINDOWS_AHEAD=0`` keeps the three launches of a chunk in order on the caller's stream."""
        return (os.environ.get("SEMBLO_WINDOWS_AHEAD", "1") == "1" and not self.is_kv_shared_layer
                and k_post is not None and v_states is not None and self.runtime_state.step_first_position == 0)

    def _prompt_with_windows_ahead(self, positions, q_post, k_post, v_states, q_pre, k_pre, output) -> None:
        """A whole prompt in one call: the dense-prefix chunks and every chunk's exact window need no
        index, so they are issued first, on a stream of normal priority, while the index build and the
        chunk loop run on a high-priority stream (joined with the caller's stream at both ends).  The
        multiprocessors that the build's short kernels and host round trips leave idle are then busy
        with window tiles.  Same launches on the same data as the in-order path: identical bytes."""
        dev = q_post.device
        caller = torch.cuda.current_stream(dev)
        if getattr(self, "_prompt_stream", None) is None or self._prompt_stream.device != dev:
            self._prompt_stream = torch.cuda.Stream(device=dev, priority=-1)
        chain = self._prompt_stream
        chain.wait_stream(caller)
        with torch.cuda.stream(chain):
            q3 = q_post.view(-1, self.num_heads, self.head_dim)
            out3 = output.view(-1, self.num_heads, self.head_dim)
            window = _fused_prefill.WindowAhead(
                q3, positions.to(torch.int32), k_post.view(-1, self.num_kv_heads, self.head_dim),
                v_states.view(-1, self.num_kv_heads, self.head_dim), chunk=self.runtime_config.query_chunk_size,
                target_tokens=int(self._target_for_step(False)), sm_scale=self.scaling, out=out3, dense_prefix_x=4,
                router_input=q_pre.view(-1, self.num_heads, self.head_dim)
                if self._source_module()._router(dev).is_identity() else None)
            self._ingest_prompt_kv(k_post, v_states, k_pre, positions)
            self._run_product_attention(q_post, q_pre, positions, out=output, window=window)
        caller.wait_stream(chain)

    # ---- prefill outside the traced model: the prompt arrives in slices -------------------------
    def begin_streamed_prefill(self, positions: torch.Tensor) -> "StreamedPrefillSession":
        """Layer-major streaming: ``keys`` for every slice, ``ingest`` once, ``queries`` for every slice."""
        return StreamedPrefillSession(self, positions)

    def begin_token_outer_prefill(self, positions: torch.Tensor, chunk: int) -> "LayerTokenOuterSession":
        """Token-order streaming: every slice passes once, with the index fitted on the prompt's head."""
        return LayerTokenOuterSession(self, positions, chunk)

    @staticmethod
    def _slice_positions(rope_positions: torch.Tensor, start: int, stop: int):
        """Rows [start, stop) of a plain [T] position row or of an [n, T] rotary grid."""
        if rope_positions.ndim == 2:
            return rope_positions[:, start:stop]
        return rope_positions[start:stop]


class StreamedPrefillSession:
    """One sparse layer's share of a layer-major streamed prefill (model.py:1431-1529 of the reference).

    The streamer hands the layer the prompt twice, a slice at a time: ``keys`` projects a slice and
    keeps only its K, V and pre-RoPE K until the whole prompt is staged; ``ingest`` fits the index on
    every key, packs the cluster-ordered copy and drops the staging; ``queries`` projects a slice
    again, keeps Q and the gate, selects, attends and finishes the slice's rows of the layer output.
    The index is fitted on the whole prompt, so the clusters are those of the one-call prefill."""

    def __init__(self, layer: SembloAttention, positions: torch.Tensor) -> None:
        self.layer = layer
        self.positions = positions
        self.tokens = int(positions.numel())
        self.k_post = self.v = self.k_pre = None
        layer.runtime_state.maybe_begin_prompt(layer.layer_idx, positions,
                                               engage_above_tokens=layer.runtime_config.engage_above_tokens)
        if layer.runtime_state.dense_request:
            raise RuntimeError("a dense request is not streamed through the sparse layer")

    def keys(self, rope_positions, hidden_states, start: int, stop: int) -> None:
        layer = self.layer
        if hasattr(layer, "_project_kv"):
            k_post, v_states, k_pre = layer._project_kv(rope_positions, hidden_states)
        else:
            _q, k_post, v_states, _qp, k_pre, _g = layer._project_qkv(rope_positions, hidden_states)
        if k_post is None or v_states is None or k_pre is None:
            raise RuntimeError("the streamed prefill needs a layer with its own K/V")
        if self.k_post is None:
            self.k_post = k_post.new_empty((self.tokens,) + tuple(k_post.shape[1:]))
            self.v = v_states.new_empty((self.tokens,) + tuple(v_states.shape[1:]))
            self.k_pre = k_pre.new_empty((self.tokens,) + tuple(k_pre.shape[1:]))
        self.k_post[start:stop] = k_post
        self.v[start:stop] = v_states
        self.k_pre[start:stop] = k_pre

    def ingest(self) -> None:
        if self.k_post is None:
            raise RuntimeError("no slice was projected before the index was asked for")
        with torch.profiler.record_function("semblo::attention"):
            # the staging is the prompt-order copy the chunks read their exact window from; it is
            # dropped with the session (the reference's FlashAttention body gathers the window from
            # the packed copy instead and frees the staging here)
            self.layer._ingest_prompt_kv(self.k_post, self.v, self.k_pre, self.positions, prompt_order_views=True)
        self.k_pre = None
        # one running snapshot for all the slices (they arrive in order)
        index = self.layer.runtime_state.get(self.layer.source_layer_idx)
        index._token_outer_snapshot = _fused_prefill.CausalSnapshot(index)

    def queries(self, rope_positions, positions, hidden_states, start: int) -> torch.Tensor:
        layer = self.layer
        q_post, _k, _v, q_pre, _kp, gate = layer._project_qkv(rope_positions, hidden_states)
        index = layer.runtime_state.get(layer.source_layer_idx)
        if getattr(index, "original_kv", None) is None and self.k_post is not None:
            index.original_kv = (self.k_post.view(-1, layer.num_kv_heads, layer.head_dim),
                                 self.v.view(-1, layer.num_kv_heads, layer.head_dim))
        with torch.profiler.record_function("semblo::attention"):
            attn = layer._run_product_attention(q_post, q_pre, positions, query_offset=start)
        return layer._finish_output(attn.view(hidden_states.shape[0], -1), gate)

    def finish(self) -> None:
        index = self.layer.runtime_state.source_indexes.get(self.layer.source_layer_idx)
        if index is not None:
            index.original_kv = None
            index._token_outer_snapshot = None
        self.k_post = self.v = None
        if _arena.full_graph_decode_enabled():
            self.layer._adopt_into_arena()


class LayerTokenOuterSession:
    """The layer's side of a token-order prefill (token_outer_prefill.py:127-212 of the reference):
    projects each slice and hands it to the streamed store (token_outer.TokenOuterPrefillSession);
    at the end the index becomes the request's index and, with an arena, moves into it."""

    def __init__(self, layer: SembloAttention, positions: torch.Tensor, chunk: int) -> None:
        from .token_outer import TokenOuterPrefillSession
        self.layer = layer
        cfg = layer.runtime_config
        # a loaded routing map: the streamed store is handed the projected pre-RoPE tensors (it uses them
        # for routing only), which is the identity map's path on those tensors
        self.router = layer._router(positions.device)
        self.rope_positions, self.flat = layer._positions_for_runtime(positions)
        layer.runtime_state.maybe_begin_prompt(layer.layer_idx, self.flat)
        self.inner = TokenOuterPrefillSession(
            total_tokens=int(self.flat.numel()), chunk=int(chunk), num_q_heads=layer.num_heads,
            num_kv_heads=layer.num_kv_heads, head_dim=layer.head_dim, target_tokens=int(layer._target_for_step(False)),
            temperature=cfg.selection_temperature, beta=cfg.bucket_size_penalty, sm_scale=layer.scaling,
            flat_unit_tokens=int(os.environ.get("SEMBLO_FLAT_UNIT_TOKENS", cfg.flat_unit_tokens)),
            flat_min_clusters_log2=max(3, int(os.environ.get("SEMBLO_FLAT_MIN_CLUSTERS_LOG2",
                                                             cfg.flat_min_clusters_log2))),
            page_align=int(os.environ.get("SEMBLO_FA3_ALIGN", cfg.fa3_page_align)), device=self.flat.device,
            kmeans_sample_size=cfg.kmeans_sample_size, codebook_seed=cfg.codebook_seed + layer.source_layer_idx,
            query_chunk_size=cfg.query_chunk_size)

    def slice(self, hidden_states: torch.Tensor, start: int, stop: int) -> torch.Tensor:
        layer = self.layer
        rope = layer._slice_positions(self.rope_positions, start, stop)
        q_post, k_post, v_states, q_pre, k_pre, gate = layer._project_qkv(rope, hidden_states)
        if k_post is None or v_states is None or k_pre is None:
            raise RuntimeError("the token-outer prefill needs a layer with its own K/V")
        hq, hkv, d = layer.num_heads, layer.num_kv_heads, layer.head_dim
        q_pre, k_pre = q_pre.view(-1, hq, d), k_pre.view(-1, hkv, d)
        if not self.router.is_identity():
            q_pre = self.router.widen(self.router.project_queries(q_pre)).contiguous()
            k_pre = self.router.widen(self.router.project(k_pre)).contiguous()
        attn = self.inner.slice(q_post.view(-1, hq, d), q_pre, k_post.view(-1, hkv, d),
                                v_states.view(-1, hkv, d), k_pre, start, stop)
        return layer._finish_output(attn.view(hidden_states.shape[0], -1), gate)

    def finish(self) -> None:
        self.inner.finish()
        layer = self.layer
        layer.runtime_state.put(layer.source_layer_idx, self.inner.index)
        if _arena.full_graph_decode_enabled():
            layer._arena(self.inner.index.packed_kv).install_suffix_store(int(self.inner.index.prompt_length))
            layer._adopt_into_arena()
        else:
            layer._ensure_own_suffix_store(self.inner.index, self.inner.index.packed_kv)
