"""The CPU restatement against the outputs of the reference's own CPU code
(tests/golden/reference_golden.npz, produced by tests/golden/make_golden.py) and
against the hand-written known-answer cases of the reference's tests."""
from __future__ import annotations

import math

import numpy as np
import pytest
import torch

from oracle import semblo_oracle as O


def T(a, dtype=None):
    t = torch.from_numpy(np.asarray(a))
    return t.to(dtype) if dtype is not None else t


def test_routing_normalisation_matches_reference(golden):
    x = T(golden["norm_in"], torch.bfloat16)
    assert torch.equal(O.routing_normalize(x).float(), T(golden["norm_out"]))
    assert torch.equal(O.routing_normalize(x).float(), T(golden["router_out"]))
    assert torch.equal(O.routing_space(x), T(golden["space_out"]))


def test_query_routing_vectors_match_reference(golden):
    x = T(golden["qvec_in"], torch.bfloat16)
    assert torch.equal(O.trivial_router_vectors(x).float(), T(golden["qvec_out"]))


def test_cluster_count_table(golden):
    for length, unit, ml, want in golden["cluster_count_table"].tolist():
        assert O.cluster_count(length, unit, ml) == want, (length, unit, ml)
    # the benchmark configurations (unit 64, floor 2^7)
    assert [O.cluster_count(n, 64, 7) for n in (8192, 131072, 524288, 1048576)] == [128, 2048, 8192, 16384]


@pytest.mark.parametrize("tag", ["b0", "b1", "b2"])
def test_index_build_is_bit_identical(golden, tag):
    sink, length, hkv, dim, clusters, is_bf16 = golden[f"{tag}_meta"].tolist()
    dtype = torch.bfloat16 if is_bf16 else torch.float32
    keys = T(golden[f"{tag}_keys"], dtype)
    product = O.routing_normalize(keys)
    index = O.build_flat(product, unit_tokens=16, min_clusters_log2=5, kmeans_sample_size=512,
                         seed=5, sink=sink, page_align=16)
    assert index.codebooks.shape[2] == clusters
    assert torch.equal(index.codebooks.float(), T(golden[f"{tag}_codebooks"]))
    assert torch.equal(index.bucket_sizes, T(golden[f"{tag}_sizes"]).int())
    assert torch.equal(index.bucket_indptr, T(golden[f"{tag}_indptr"]).int())
    assert torch.equal(index.posting_positions, T(golden[f"{tag}_posting"]).int())
    assert torch.equal(index.inverse_positions, T(golden[f"{tag}_inverse"]).int())
    # packing
    packed = O.pack_prompt_kv(index, T(golden[f"{tag}_pack_k"], dtype), T(golden[f"{tag}_pack_v"], dtype))
    assert torch.equal(packed.float(), T(golden[f"{tag}_packed"]))
    # causal snapshot
    for p, want in zip(golden[f"{tag}_snap_pos"].tolist(), golden[f"{tag}_snap_sizes"]):
        assert torch.equal(O.causal_sizes_at(index, p), T(want).int())


def test_centred_index_build_is_bit_identical(golden):
    """SEMBLO_ROUTING_CENTER=1 (state.py:649-670): the prompt's mean key is taken out per head."""
    sink, length, hkv, dim, clusters, _ = golden["c0_meta"].tolist()
    keys = T(golden["c0_keys"], torch.bfloat16)
    product = O.routing_normalize(keys)
    index = O.build_flat(product, unit_tokens=16, min_clusters_log2=5, kmeans_sample_size=512, seed=5,
                         sink=sink, page_align=16, center=True)
    assert torch.equal(index.codebooks.float(), T(golden["c0_codebooks"]))
    assert torch.equal(index.bucket_sizes, T(golden["c0_sizes"]).int())
    assert torch.equal(index.bucket_indptr, T(golden["c0_indptr"]).int())
    assert torch.equal(index.posting_positions, T(golden["c0_posting"]).int())
    assert torch.equal(index.inverse_positions, T(golden["c0_inverse"]).int())
    # without centring the same keys crowd into fewer clusters and leave the others empty
    plain = O.build_flat(product, unit_tokens=16, min_clusters_log2=5, kmeans_sample_size=512, seed=5,
                         sink=sink, page_align=16)
    assert int((plain.bucket_sizes > 0).sum()) < int((index.bucket_sizes > 0).sum())


@pytest.mark.parametrize("tag", ["b0", "b1", "b2"])
def test_scores_and_sort_walk_selector(golden, tag):
    sink, length, hkv, dim, clusters, _ = golden[f"{tag}_meta"].tolist()
    qv = T(golden[f"{tag}_sel_q"], torch.bfloat16)
    cb = T(golden[f"{tag}_codebooks"], torch.bfloat16)
    prob = O.mixture_prob(qv, cb, 0.1)
    logs = prob.clamp_min(1e-30).log()
    torch.testing.assert_close(logs, T(golden[f"{tag}_sel_logscore"]), atol=2e-5, rtol=0)
    sizes = T(golden[f"{tag}_snap_sizes"][-1]).int()
    # fused_select.theta_select_reference on the reference's own scores
    ref_logs = T(golden[f"{tag}_sel_logscore"])
    pen = ref_logs - 0.25 * torch.log1p(sizes.float())[None]
    pen = pen.masked_fill(sizes[None] <= 0, float("-inf"))
    walk = O.budget_walk(pen, sizes.float()[None].expand_as(pen), 256)
    assert torch.equal(walk.int(), T(golden[f"{tag}_sortwalk"]).int())
    # torch_select.budget_select_bitmask (sink taken first inside the budget)
    score = pen.clone()
    if sink:
        score[..., 0] = float("inf")
        score = score.masked_fill(sizes[None] <= 0, float("-inf"))
    sel = O.budget_walk(score, sizes.float()[None].expand_as(score), 256)
    assert torch.equal(O.pack_bits(sel), T(golden[f"{tag}_sel_qmask"]).int())
    assert torch.equal(sel.sum(-1).int(), T(golden[f"{tag}_sel_counts"]).int())
    assert torch.equal((sel * sizes[None]).sum(-1).int(), T(golden[f"{tag}_sel_tokens"]).int())
    assert torch.equal(O.unpack_bits(O.pack_bits(sel)), sel)


def test_theta_rule_is_a_superset_of_the_sort_walk_and_reaches_the_budget(golden):
    # the property the reference states for its bisected threshold (fused_select.py:8-11)
    for tag in ("b0", "b1"):
        sizes = T(golden[f"{tag}_snap_sizes"][-1]).int()
        logs = T(golden[f"{tag}_sel_logscore"])
        score = O.penalized_scores(logs.exp(), sizes[None], 0.25)
        sel, margin = O.theta_select(score, sizes[None], 256, 16, return_margin=True)
        walk = O.budget_walk(score.masked_fill(sizes[None] <= 0, float("-inf")),
                             sizes.float()[None].expand_as(score), 256)
        assert bool((sel | ~walk).all())
        tokens = (sel * sizes[None]).sum(-1)
        assert bool((tokens >= min(256, int(sizes.sum(-1).min()))).all())
        assert bool((margin >= 0).all())


def test_theta_rule_against_a_scalar_float32_loop():
    g = torch.Generator().manual_seed(0)
    score = torch.randn(7, 3, 64, generator=g) * 3
    sizes = torch.randint(0, 50, (3, 64), generator=g).int()
    sizes[1, :] = 1                    # everything fits -> all live selected
    score = torch.where(sizes[None] > 0, score, torch.full_like(score, O.NEG_BIG))
    sel = O.theta_select(score, sizes[None], 200, 16)
    f = np.float32
    for q in range(7):
        for h in range(3):
            s = score[q, h].numpy().astype(np.float32)
            z = sizes[h].numpy().astype(np.float32)
            live = z > 0
            hi = f(s.max() + f(1e-6))
            lo = f(min(f(np.where(live, s, f(3.4e38)).min() - f(1e-6)), f(hi - f(1e-5))))
            all_fit = z[live].sum() < 200
            for _ in range(16):
                mid = f((lo + hi) * f(0.5))
                above = z[s >= mid].sum()
                if above >= 200:
                    lo = mid
                else:
                    hi = mid
            theta = f(-3.4e38) if all_fit else lo
            want = live & (s >= theta)
            assert np.array_equal(sel[q, h].numpy(), want), (q, h)


def test_kmeans_pieces(golden):
    xs, cs = T(golden["km_x"]), T(golden["km_c"])
    assign = O.argmax_sim(xs, cs, 256)
    assert torch.equal(assign, T(golden["km_assign"]).long())
    assert torch.equal(O.segment_sum(xs, assign, 40), T(golden["km_sums"]))
    gen = torch.Generator().manual_seed(3)
    fit = O.fit_flat_codebook(xs, 40, num_iters=6, sample_size=500, generator=gen)
    assert torch.equal(fit, T(golden["km_fit"]))


def test_hold_out_sink_kat(golden):
    held, tgt = O.hold_out_sink(torch.tensor([[5, 3, 0, 9]], dtype=torch.int32), 100, 32)
    assert held.tolist()[0] + [tgt] == golden["holdout"].tolist() == [0, 3, 0, 9, 68]


def test_lse_merge(golden):
    out, lse = O.merge_states(T(golden["merge_o1"]), T(golden["merge_l1"]),
                              T(golden["merge_o2"]), T(golden["merge_l2"]))
    torch.testing.assert_close(out, T(golden["merge_out"]), atol=1e-6, rtol=1e-6)
    torch.testing.assert_close(lse, T(golden["merge_lse"]), atol=1e-6, rtol=1e-6)
    # the reference's hand-written case: two unit states -> halves, lse ln 2
    o, l = O.merge_states(torch.tensor([[[1.0, 0.0]]]), torch.tensor([[0.0]]),
                          torch.tensor([[[0.0, 1.0]]]), torch.tensor([[0.0]]))
    torch.testing.assert_close(o, torch.tensor([[[0.5, 0.5]]]))
    assert abs(float(l) - math.log(2.0)) < 1e-6


def test_arena_suffix_table(golden):
    width, clusters, nblk, tlen = golden["arena_shape"].tolist()
    a = O.make_arena(capacity=4096, num_clusters=O.cluster_count(4096, 2048, 3), num_kv_heads=2,
                     head_dim=8, page_align=16, reserve=512, kv_dtype=torch.float32,
                     desc_dtype=torch.float32, table_positions=8192)
    assert (a.posting.shape[1], a.sizes.shape[1], a.suffix_kv.shape[1], a.suffix_table.shape[1]) == \
        (width, clusters, nblk, tlen)
    assert torch.equal(a.suffix_table, T(golden["arena_table0"]).int())
    O.arena_install_suffix_store(a, 1000)
    assert torch.equal(a.suffix_table, T(golden["arena_table1"]).int())
    O.arena_extend_suffix_table(a, 2500)
    assert torch.equal(a.suffix_table, T(golden["arena_table2"]).int())
    # the reference's hand-written expectations (test_decode_arena_suffix_store.py:30-43)
    b = O.make_arena(capacity=4096, num_clusters=8, num_kv_heads=2, head_dim=8, page_align=16,
                     reserve=512, kv_dtype=torch.float32, desc_dtype=torch.float32)
    assert b.suffix_kv.shape == (2, 3, 256, 2, 8)
    assert b.suffix_table[0, 16:19].tolist() == [0, 1, 2] and int(b.suffix_table[0, :16].abs().sum()) == 0


def test_repack_plan_and_apply(golden):
    plan = O.repack_plan(torch.tensor([3, 0, 2]), torch.tensor([0, 16, 16, 32]),
                         torch.tensor([2, 0, 2, 1]), 16)
    got = torch.cat([plan.new_sizes, plan.new_indptr.long(), plan.kind.long(), plan.old_src, plan.new_src])
    assert got.tolist() == golden["plan_kat"].tolist()
    assert plan.new_sizes.tolist() == [4, 1, 4] and plan.new_indptr.tolist() == [0, 16, 32, 48]
    widest, align, L, N = golden["fl_widest"].tolist()
    packed = T(golden["fl_packed0"]).clone()
    posting = T(golden["fl_posting0"]).int().clone()
    sizes = T(golden["fl_sizes0"]).int().clone()
    indptr = T(golden["fl_indptr0"]).int().clone()
    w = O.repack_apply(packed, posting, sizes, indptr, T(golden["fl_new_kv"]),
                       torch.arange(L, L + N, dtype=torch.int32), T(golden["fl_new_assign"]).long(), align)
    assert w == widest
    assert torch.equal(packed, T(golden["fl_packed1"]))
    assert torch.equal(posting, T(golden["fl_posting1"]).int())
    assert torch.equal(sizes, T(golden["fl_sizes1"]).int())
    assert torch.equal(indptr, T(golden["fl_indptr1"]).int())


def test_flush_schedule_and_nearest_cluster(golden):
    sched, plen = [], 1000
    for written in range(400):
        r = O.flush_range(1000, written, plen, 100, 50)
        if r is not None:
            sched.append((written, r[0], r[1]))
            plen = r[1]
    assert sched == [tuple(r) for r in golden["fl_schedule"].tolist()]
    ids = O.nearest_cluster(O.routing_space(T(golden["nc_keys"])), T(golden["nc_cb"]))
    assert torch.equal(ids, T(golden["nc_ids"]).long())
    assert 0 not in ids.tolist()           # the zero descriptor is never chosen


def test_token_outer_bookkeeping(golden):
    n_ref, total, width, align = golden["ro_args"].tolist()
    res = O.reserved_layout(T(golden["ro_sizes"]), n_ref, total, width, align)
    assert torch.equal(res, T(golden["ro_reserve"]).long())
    assert bool((res % align == 0).all()) and bool((res >= align).all()) and int(res.sum(1).max()) <= width
    rows, counts = O.append_rows(T(golden["ar_ids"]), T(golden["ar_indptr"]).int(), T(golden["ro_sizes"]))
    assert torch.equal(rows, T(golden["ar_rows"]).long())
    assert torch.equal(counts, T(golden["ar_counts"]).long())
    assert O.token_outer_fit_at(262144, 8192, 4096) == 24576
    assert O.token_outer_fit_at(262144, 8192, 32768) == 73728
