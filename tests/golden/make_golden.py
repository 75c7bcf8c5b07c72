"""Generate the golden fixtures from the reference's own CPU code.

Run once in a container that has the reference checkout (it cannot travel to the
GPU box, so the outputs are committed):

    python tests/golden/make_golden.py /path/to/reference

Inputs are seeded; outputs are what the reference's functions return on the CPU.
bf16 tensors are stored as float32 (exact).  The fixtures pin the CPU
restatement under ``oracle/``; the CUDA kernels are then checked against that
restatement on the same inputs.
"""
from __future__ import annotations

import os
import sys
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent


def f32(t: torch.Tensor) -> np.ndarray:
    return t.detach().float().cpu().numpy() if t.is_floating_point() else t.detach().cpu().numpy()


def mixture_keys(length, hkv, dim, centres, seed, dtype):
    g = torch.Generator().manual_seed(seed)
    cent = torch.randn(hkv, centres, dim, generator=g)
    z = torch.randint(0, centres, (length,), generator=g)
    k = cent[:, z].permute(1, 0, 2) + 0.3 * torch.randn(length, hkv, dim, generator=g)
    return k.to(dtype)


def main(ref_root: str) -> None:
    sys.path.insert(0, ref_root)
    os.environ["SEMBLO_FLAT_UNIT_TOKENS"] = "16"
    os.environ["SEMBLO_FA3_ALIGN"] = "16"
    from semblo.inference import flat_index
    from semblo.vllm_plugin import arena as arena_mod
    from semblo.vllm_plugin import suffix_flush, token_outer_prefill, torch_select
    from semblo.vllm_plugin.fused_prefill import CausalSnapshot, _hold_out_sink
    from semblo.vllm_plugin.fused_select import theta_select_reference
    from semblo.vllm_plugin.paged_attention import (PagedSparseAttentionResult,
                                                    merge_paged_attention_results)
    from semblo.vllm_plugin.routing_map import SembloKeyRouter, routing_normalize
    from semblo.vllm_plugin.state import ProductPostingIndex, SembloRuntimeState
    from semblo.vllm_plugin.trivial_router import trivial_router_vectors

    out: dict[str, np.ndarray] = {}
    g = torch.Generator().manual_seed(1234)

    # ---- routing normalisation / query vectors ---------------------------------
    x = torch.randn(96, 4, 32, generator=g).to(torch.bfloat16)
    out["norm_in"] = f32(x)
    out["norm_out"] = f32(routing_normalize(x))
    out["router_out"] = f32(SembloKeyRouter(4, 32, 32)(x.unsqueeze(0))[0])
    out["space_out"] = f32(flat_index.routing_space(x))
    xq = torch.randn(40, 8, 32, generator=g).to(torch.bfloat16)
    out["qvec_in"] = f32(xq)
    out["qvec_out"] = f32(trivial_router_vectors(xq, 1))

    # ---- cluster count table -----------------------------------------------------
    rows = []
    for length in (128, 1000, 2048, 8192, 131072, 262144, 524288, 1048576, 3000000):
        for unit in (16, 64, 2048):
            for ml in (3, 7, 9):
                rows.append((length, unit, ml, arena_mod.arena_cluster_count(length, unit, ml)))
    out["cluster_count_table"] = np.array(rows, dtype=np.int64)

    # ---- k-means fit + assignment + layout (with and without a sink) ----------
    for tag, sink, length, hkv, dim, dtype in (
            ("b0", 0, 1024, 2, 32, torch.bfloat16),
            ("b1", 32, 1536, 2, 32, torch.bfloat16),
            ("b2", 0, 768, 1, 16, torch.float32)):
        keys = mixture_keys(length, hkv, dim, 24, 77 + sink, dtype)
        product = SembloKeyRouter(hkv, dim, dim)(keys.unsqueeze(0))[0]
        if sink:
            os.environ["SEMBLO_SINK_TOKENS"] = str(sink)
        else:
            os.environ.pop("SEMBLO_SINK_TOKENS", None)
        positions = torch.arange(length)
        index = ProductPostingIndex.build(
            product, positions, num_centroids=0, kmeans_iters=4, kmeans_sample_size=512,
            codebook_seed=5, flat_unit_tokens=16, flat_min_clusters_log2=5, page_align=16)
        out[f"{tag}_keys"] = f32(keys)
        out[f"{tag}_meta"] = np.array([sink, length, hkv, dim, index.flat_clusters,
                                       1 if dtype == torch.bfloat16 else 0], dtype=np.int64)
        out[f"{tag}_codebooks"] = f32(index.codebooks)
        out[f"{tag}_posting"] = f32(index.posting_positions)
        out[f"{tag}_indptr"] = f32(index.bucket_indptr)
        out[f"{tag}_sizes"] = f32(index.bucket_sizes)
        out[f"{tag}_inverse"] = f32(index.inverse_positions())
        gk = torch.Generator().manual_seed(9)
        kk = torch.randn(length, hkv, 8, generator=gk).to(dtype)
        vv = torch.randn(length, hkv, 8, generator=gk).to(dtype)
        packed = index.pack_prompt_kv(kk, vv)
        out[f"{tag}_pack_k"] = f32(kk)
        out[f"{tag}_pack_v"] = f32(vv)
        out[f"{tag}_packed"] = f32(packed)
        snap = CausalSnapshot(index)
        pts = [0, 17, length // 3, length // 2 + 5, length - 1]
        out[f"{tag}_snap_pos"] = np.array(pts, dtype=np.int64)
        out[f"{tag}_snap_sizes"] = np.stack([f32(snap.advance(p).clone()) for p in pts])

        # scores + the torch selector on this index
        nq, hq = 24, hkv * 4
        qv = trivial_router_vectors(
            (mixture_keys(nq, hkv, dim, 24, 77 + sink, dtype)[:, :, None, :]
             .expand(nq, hkv, 4, dim).reshape(nq, hq, dim)
             + 0.3 * torch.randn(nq, hq, dim, generator=gk)).to(torch.bfloat16), 1)
        vec4 = qv.view(nq, hq, 1, dim)
        cb = index.codebooks.to(torch.bfloat16)
        logs = torch_select.mixture_log_scores(vec4, None, cb, temperature=0.1, fused=False)
        out[f"{tag}_sel_q"] = f32(qv)
        out[f"{tag}_sel_logscore"] = f32(logs)
        sizes = snap.advance(length - 1).clone()
        nwords = index.flat_clusters // 32
        bitmask = torch.zeros(1, hkv, nwords, dtype=torch.int32)
        qmask = torch.zeros(nq, hkv, nwords, dtype=torch.int32)
        logmix = torch.zeros(nq, hq, 1)
        counts, tokens = torch_select.budget_select_bitmask(
            vec4, logmix, cb, sizes[None].contiguous(), bitmask, temperature=0.1, beta=0.25,
            target_tokens=256, g_union=nq, qmask=qmask)
        out[f"{tag}_sel_qmask"] = f32(qmask)
        out[f"{tag}_sel_counts"] = f32(counts)
        out[f"{tag}_sel_tokens"] = f32(tokens)
        # the sort-walk twin in fused_select
        pen = logs - 0.25 * torch.log1p(sizes.float())[None]
        out[f"{tag}_sortwalk"] = f32(theta_select_reference(pen, sizes, 256).to(torch.int32))
    os.environ.pop("SEMBLO_SINK_TOKENS", None)

    # ---- the same build with the prompt's mean key taken out (SEMBLO_ROUTING_CENTER=1): keys that
    # share one dominant direction, as those of a model without a rotary embedding do
    length, hkv, dim = 1024, 2, 32
    gd = torch.Generator().manual_seed(123)
    keys = (mixture_keys(length, hkv, dim, 24, 91, torch.float32)
            + 6.0 * torch.randn(1, hkv, dim, generator=gd)).to(torch.bfloat16)
    product = SembloKeyRouter(hkv, dim, dim)(keys.unsqueeze(0))[0]
    os.environ["SEMBLO_ROUTING_CENTER"] = "1"
    try:
        index = ProductPostingIndex.build(
            product, torch.arange(length), num_centroids=0, kmeans_iters=4, kmeans_sample_size=512,
            codebook_seed=5, flat_unit_tokens=16, flat_min_clusters_log2=5, page_align=16)
    finally:
        os.environ.pop("SEMBLO_ROUTING_CENTER", None)
    out["c0_keys"] = f32(keys)
    out["c0_meta"] = np.array([0, length, hkv, dim, index.flat_clusters, 1], dtype=np.int64)
    out["c0_codebooks"] = f32(index.codebooks)
    out["c0_posting"] = f32(index.posting_positions)
    out["c0_indptr"] = f32(index.bucket_indptr)
    out["c0_sizes"] = f32(index.bucket_sizes)
    out["c0_inverse"] = f32(index.inverse_positions())

    # ---- k-means pieces -----------------------------------------------------------
    xs = torch.nn.functional.normalize(torch.randn(700, 48, generator=g), dim=-1)
    cs = torch.nn.functional.normalize(torch.randn(40, 48, generator=g), dim=-1)
    asg = flat_index._argmax_sim_chunked(xs, cs, 256)
    out["km_x"], out["km_c"], out["km_assign"] = f32(xs), f32(cs), f32(asg)
    out["km_sums"] = f32(flat_index._segment_sum_matmul(xs, asg, 40, torch.bincount(asg, minlength=40)))
    gg = torch.Generator().manual_seed(3)
    out["km_fit"] = f32(flat_index.fit_flat_codebook(xs, 40, num_iters=6, sample_size=500, generator=gg))

    # ---- sink hold-out, LSE merge ----------------------------------------------------
    held, tgt = _hold_out_sink(torch.tensor([[5, 3, 0, 9]], dtype=torch.int32), 100, 32)
    out["holdout"] = np.array(held.tolist()[0] + [tgt], dtype=np.int64)
    o1, o2 = torch.randn(5, 4, 16, generator=g), torch.randn(5, 4, 16, generator=g)
    l1, l2 = torch.randn(5, 4, generator=g), torch.randn(5, 4, generator=g)
    l2[0, 0] = float("-inf")
    m = merge_paged_attention_results(PagedSparseAttentionResult(o1, l1),
                                      PagedSparseAttentionResult(o2, l2))
    out["merge_o1"], out["merge_o2"], out["merge_l1"], out["merge_l2"] = map(f32, (o1, o2, l1, l2))
    out["merge_out"], out["merge_lse"] = f32(m.output), f32(m.logsumexp)

    # ---- arena suffix table -------------------------------------------------------
    os.environ["SEMBLO_SUFFIX_RESERVE"] = "512"
    state = SembloRuntimeState()
    state.suffix_block_size = 256
    arena = arena_mod.arena_for(
        state, 3, capacity=4096, unit_tokens=2048, min_clusters_log2=3, num_kv_heads=2, head_dim=8,
        index_dim=8, page_align=16, kv_dtype=torch.float32, desc_dtype=torch.float32,
        device=torch.device("cpu"), table_positions=4096 + 4096)
    out["arena_shape"] = np.array([arena.width, arena.num_clusters, arena.suffix_blocks,
                                   arena.suffix_table.shape[1]], dtype=np.int64)
    out["arena_table0"] = f32(arena.suffix_table.clone())
    arena.install_suffix_store(1000)
    out["arena_table1"] = f32(arena.suffix_table.clone())
    arena.extend_suffix_table(1000 + 1500)
    out["arena_table2"] = f32(arena.suffix_table.clone())
    os.environ.pop("SEMBLO_SUFFIX_RESERVE", None)

    # ---- suffix flush --------------------------------------------------------------
    plan = suffix_flush.repack_plan(torch.tensor([3, 0, 2]), torch.tensor([0, 16, 16, 32]),
                                    torch.tensor([2, 0, 2, 1]), 16)
    out["plan_kat"] = np.concatenate([f32(plan.new_sizes), f32(plan.new_indptr), f32(plan.kind).astype(np.int64),
                                      f32(plan.old_src), f32(plan.new_src)]).astype(np.int64)
    L, C, hkv, dim, align, N = 300, 6, 2, 8, 16, 75
    assign = torch.randint(0, C, (hkv, L), generator=g)
    kv_by_pos = torch.randn(2, L, hkv, dim, generator=g)
    sizes = torch.stack([torch.bincount(assign[h], minlength=C) for h in range(hkv)]).to(torch.int32)
    padded = ((sizes + align - 1) // align) * align
    indptr = torch.zeros(hkv, C + 1, dtype=torch.int32)
    indptr[:, 1:] = padded.cumsum(1)
    width = int(indptr[:, -1].max()) + 20 * align
    width += (-width) % 256
    packed = torch.zeros(2, width, hkv, dim)
    posting = torch.zeros(hkv, width, dtype=torch.int32)
    for h in range(hkv):
        order = torch.argsort(assign[h], stable=True)
        start = 0
        for c in range(C):
            n = int(sizes[h, c])
            rows = order[start:start + n]
            packed[:, int(indptr[h, c]):int(indptr[h, c]) + n, h] = kv_by_pos[:, rows, h]
            posting[h, int(indptr[h, c]):int(indptr[h, c]) + n] = rows.to(torch.int32)
            start += n
    out["fl_packed0"], out["fl_posting0"], out["fl_sizes0"], out["fl_indptr0"] = map(
        f32, (packed.clone(), posting.clone(), sizes.clone(), indptr.clone()))
    new_assign = torch.randint(0, C, (hkv, N), generator=g)
    flushed_kv = torch.randn(2, N, hkv, dim, generator=g)
    flushed_pos = torch.arange(L, L + N, dtype=torch.int32)
    tmp = torch.zeros(2, width, dim)
    widest = suffix_flush.repack_apply(packed, posting, sizes, indptr, flushed_kv, flushed_pos,
                                       new_assign, align, tmp)
    out["fl_new_assign"], out["fl_new_kv"] = f32(new_assign), f32(flushed_kv)
    out["fl_packed1"], out["fl_posting1"], out["fl_sizes1"], out["fl_indptr1"] = map(
        f32, (packed, posting, sizes, indptr))
    out["fl_widest"] = np.array([widest, align, L, N], dtype=np.int64)
    sched = []
    plen = 1000
    for written in range(0, 400):
        r = suffix_flush.flush_range(1000, written, plen, 100, 50)
        if r is not None:
            sched.append((written, r[0], r[1]))
            plen = r[1]
    out["fl_schedule"] = np.array(sched, dtype=np.int64)
    keys_n = torch.randn(50, 16, generator=g)
    cbh = torch.nn.functional.normalize(torch.randn(12, 16, generator=g), dim=-1)
    cbh[0] = 0
    cb2 = torch.stack(list(cbh.chunk(2, dim=-1)))
    out["nc_keys"], out["nc_cb"] = f32(keys_n), f32(cb2)
    out["nc_ids"] = f32(suffix_flush._nearest_cluster(flat_index.routing_space(keys_n), cb2))

    # ---- token-outer bookkeeping ---------------------------------------------------
    sz = torch.randint(0, 40, (2, 32), generator=g)
    sz[0, 3] = 0
    n_ref = int(sz[0].sum())
    sz[1] = sz[1] * 0 + sz[0].flip(0)
    res = token_outer_prefill.reserved_layout(sz, n_ref, 4 * n_ref, 4 * n_ref + 32 * 16 + 100, 16)
    out["ro_sizes"], out["ro_args"], out["ro_reserve"] = f32(sz), np.array(
        [n_ref, 4 * n_ref, 4 * n_ref + 32 * 16 + 100, 16], dtype=np.int64), f32(res)
    ids = torch.randint(0, 32, (2, 64), generator=g)
    ip = torch.zeros(2, 33, dtype=torch.int32)
    ip[:, 1:] = res.cumsum(1).to(torch.int32)
    rows, counts = token_outer_prefill.append_rows(ids, ip, sz)
    out["ar_ids"], out["ar_indptr"], out["ar_rows"], out["ar_counts"] = map(f32, (ids, ip, rows, counts))

    np.savez_compressed(HERE / "reference_golden.npz", **out)
    print("wrote", HERE / "reference_golden.npz", sum(v.nbytes for v in out.values()) // 1024, "KiB raw")


if __name__ == "__main__":
    if len(sys.argv) < 2:
        raise SystemExit("usage: make_golden.py <path of the reference checkout>")
    main(sys.argv[1])
