"""Keys that arrive after the fit: token-order streamed prefill and suffix flush on the GPU,
through the C ABI, against the CPU oracle (integer stages bit-exact; nearest-centroid ids equal
except fp32 near-ties; attention within the reference's bf16 tolerance on the kernel's own
selection)."""
from __future__ import annotations

import os

import pytest
import torch

from oracle import semblo_oracle as O

pytestmark = pytest.mark.gpu

MAX_ABS = 2e-2
MEAN_ABS = 1e-3


@pytest.fixture(scope="module")
def dev():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from semblo_b200 import _lib
    _lib.lib()
    return torch.device("cuda:0")


def _status_ok(dev):
    from semblo_b200 import _lib
    _lib.status_for(dev).raise_if_set()


def _close(got, want, what):
    diff = (got.double().cpu() - want.double().cpu()).abs()
    assert float(diff.max()) <= MAX_ABS, f"{what}: max-abs {float(diff.max()):.4g}"
    assert float(diff.mean()) <= MEAN_ABS, f"{what}: mean-abs {float(diff.mean()):.4g}"


def _ids_match(ids_gpu, product, codebooks, what):
    """Kernel ids equal the oracle's, or the chosen centroid's fp32 cosine is within 2e-6 of the best."""
    hkv = codebooks.shape[0]
    differ = 0
    for h in range(hkv):
        want = O.nearest_cluster(O.routing_space(product[:, h]), codebooks[h])
        got = ids_gpu[h].long().cpu()
        bad = torch.nonzero(got != want).flatten()
        differ += int(bad.numel())
        if bad.numel():
            cents = torch.cat([codebooks[h][0], codebooks[h][1]], dim=-1).float()
            space = torch.nn.functional.normalize(product[bad, h].float(), dim=-1)
            sim = space @ cents.T
            gap = sim.gather(1, want[bad][:, None]) - sim.gather(1, got[bad][:, None])
            assert float(gap.max()) < 2e-6, f"{what}: a chosen centroid is {float(gap.max()):.3g} below the best"
            dead = cents.norm(dim=-1) == 0
            assert not bool(dead[got[bad]].any()), f"{what}: a zero descriptor was chosen"
    assert differ <= 0.005 * ids_gpu.numel(), f"{what}: {differ} ids differ"


@pytest.mark.parametrize("dim,sink", [(128, 64), (256, 0)])
def test_nearest_cluster_and_append_rows(dev, dim, sink):
    from semblo_b200 import token_outer as T
    hq, hkv, length, n_new = 8, 2, 4096, 777
    data = O.mixture_inputs(length=length + n_new, num_q_heads=hq, num_kv_heads=hkv, head_dim=dim, centres=16, seed=31)
    product = O.routing_normalize(data["k_pre"])
    index = O.build_flat(product[:length], unit_tokens=32, min_clusters_log2=7, kmeans_sample_size=1024, fit_iters=4,
                         seed=0, sink=sink, page_align=16)
    new = product[length:]
    ids = T.nearest_cluster(new.to(dev), index.codebooks.to(dev))
    _status_ok(dev)
    _ids_match(ids, new, index.codebooks, "nearest cluster")
    # rows and counts for the kernel's own ids: bit-exact
    rows, counts = T.append_rows(ids, index.bucket_indptr.to(dev), index.bucket_sizes.to(dev))
    rows_want, counts_want = O.append_rows(ids.cpu(), index.bucket_indptr, index.bucket_sizes)
    assert torch.equal(rows.cpu().long(), rows_want)
    assert torch.equal(counts.cpu().long(), counts_want)
    # an empty slice
    rows0, counts0 = T.append_rows(ids[:, :0].contiguous(), index.bucket_indptr.to(dev), index.bucket_sizes.to(dev))
    assert rows0.shape == (hkv, 0) and int(counts0.sum()) == 0


def test_scatter_gather_relayout(dev):
    from semblo_b200 import token_outer as T
    hkv, dim, n, width, c = 2, 128, 500, 2048, 64
    g = torch.Generator().manual_seed(5)
    k = torch.randn(n, hkv, dim, generator=g).bfloat16()
    v = torch.randn(n, hkv, dim, generator=g).bfloat16()
    rows = torch.stack([torch.randperm(width, generator=g)[:n] for _ in range(hkv)]).int()
    pos = (torch.arange(n) + 1000).int()
    packed = torch.zeros(2, width, hkv, dim, dtype=torch.bfloat16, device=dev)
    posting = torch.full((hkv, width), -1, dtype=torch.int32, device=dev)
    inverse = torch.zeros(hkv, 4000, dtype=torch.int32, device=dev)
    T.scatter_kv(k.to(dev), v.to(dev), pos.to(dev), rows.to(dev), packed, posting, inverse, inverse_offset=1000)
    _status_ok(dev)
    want = torch.zeros(2, width, hkv, dim, dtype=torch.bfloat16)
    want_post = torch.full((hkv, width), -1, dtype=torch.int32)
    for h in range(hkv):
        want[0][:, h].index_copy_(0, rows[h].long(), k[:, h])
        want[1][:, h].index_copy_(0, rows[h].long(), v[:, h])
        want_post[h].index_copy_(0, rows[h].long(), pos)
    assert torch.equal(packed.cpu(), want)
    assert torch.equal(posting.cpu(), want_post)
    assert torch.equal(inverse[:, 1000:1000 + n].cpu(), rows)
    k2, v2 = T.gather_kv(packed, rows.to(dev))
    assert torch.equal(k2.cpu(), k) and torch.equal(v2.cpu(), v)
    # a row outside the store is refused through the status word, nothing is written there
    from semblo_b200 import _lib
    bad = rows.clone()
    bad[0, 0] = width + 5
    T.scatter_kv(k.to(dev), v.to(dev), pos.to(dev), bad.to(dev), packed, posting, None)
    torch.cuda.synchronize()
    st = _lib.status_for(dev)
    assert int(st.word.item()) == 201
    st.word.zero_()
    # relayout: offsets inside a cluster's run are kept
    sizes = torch.randint(1, 20, (hkv, c), generator=g)
    old_ip = torch.zeros(hkv, c + 1, dtype=torch.int32)
    old_ip[:, 1:] = ((sizes + 15) // 16 * 16).cumsum(1).int()
    new_ip = torch.zeros(hkv, c + 1, dtype=torch.int32)
    new_ip[:, 1:] = ((sizes + 40) // 16 * 16).cumsum(1).int()
    bucket = torch.randint(0, c, (hkv, 300), generator=g).int()
    off = (torch.rand(hkv, 300, generator=g) * sizes.gather(1, bucket.long())).long()
    inv_old = (old_ip.long().gather(1, bucket.long()) + off).int()
    got = T.relayout_rows(inv_old.to(dev), bucket.to(dev), old_ip.to(dev), new_ip.to(dev))
    assert torch.equal(got.cpu().long(), O.relayout_rows(inv_old, old_ip, new_ip))


def test_token_outer_session_against_the_oracle(dev):
    """Dense start, fit with reservations, appended slices (one forced repack), slice by slice."""
    from semblo_b200 import token_outer as T
    dim, hq, hkv, sink, total, chunk, target = 128, 8, 2, 64, 6144, 1024, 256
    unit, min_log2, align = 32, 7, 16
    data = O.mixture_inputs(length=total, num_q_heads=hq, num_kv_heads=hkv, head_dim=dim, centres=24, seed=77)
    product = O.routing_normalize(data["k_pre"])
    sm_scale = dim ** -0.5
    os.environ["SEMBLO_SINK_TOKENS"] = str(sink)
    try:
        sess = T.TokenOuterPrefillSession(total_tokens=total, chunk=chunk, num_q_heads=hq, num_kv_heads=hkv,
                                          head_dim=dim, target_tokens=target, temperature=0.1, beta=0.25,
                                          sm_scale=sm_scale, flat_unit_tokens=unit, flat_min_clusters_log2=min_log2,
                                          page_align=align, device=dev, kmeans_sample_size=1024)
        assert sess.fit_at == O.token_outer_fit_at(total, chunk, target) == 2048
        ref = None          # the oracle's copy of the store once the index exists
        sparse_slices = 0
        for start in range(0, total, chunk):
            stop = start + chunk
            sl = slice(start, stop)
            if sess.index is None and start >= sess.fit_at:
                sess._fit_and_pack()
                ix = sess.index
                p = sess.fit_at
                sizes_fit = ix.bucket_sizes.cpu().clone()
                width = int(ix.packed_kv.shape[1])
                reserve = O.reserved_layout(sizes_fit, p, total, width, align)
                want_ip = torch.zeros(hkv, sizes_fit.shape[1] + 1, dtype=torch.int32)
                want_ip[:, 1:] = reserve.cumsum(1).int()
                assert torch.equal(ix.bucket_indptr.cpu(), want_ip)
                assert sizes_fit.shape[1] == O.cluster_count(total, unit, min_log2)
                inv = ix._inverse_positions[:, :p].cpu().long()
                assign = ix.orig_bucket[:, :p].cpu().long()
                lo = want_ip.long().gather(1, assign)
                assert bool(((inv >= lo) & (inv < lo + sizes_fit.long().gather(1, assign))).all())
                for h in range(hkv):
                    assert torch.equal(ix.packed_kv[0, :, h].cpu()[inv[h]], data["k_post"][:p, h])
                    assert torch.equal(ix.packed_kv[1, :, h].cpu()[inv[h]], data["v"][:p, h])
                    assert torch.equal(ix.posting_positions[h].cpu()[inv[h]].long(), torch.arange(p))
                    # position order inside every cluster: rows ascend with positions
                    key = assign[h] * (10 * width) + inv[h]
                    assert bool((key.argsort(stable=True) == (assign[h] * total + torch.arange(p)).argsort(stable=True)).all())
                ref = dict(packed=ix.packed_kv.cpu().clone(), posting=ix.posting_positions.cpu().clone(),
                           indptr=want_ip.clone(), sizes=sizes_fit.clone(), inverse=ix._inverse_positions.cpu().clone(),
                           codebooks=ix.codebooks.cpu().clone(), reserve=reserve.clone(), repacks=0)
            def oracle_repack(n_so_far, incoming=None, n_incoming=0):
                """token_outer_prefill.py:366-392 on the oracle's copy of the store."""
                old_ip = ref["indptr"].clone()
                basis = ref["sizes"] if incoming is None else (ref["sizes"].long() + incoming).int()
                new_res = O.reserved_layout(basis, n_so_far + n_incoming, total, int(ref["packed"].shape[1]), align)
                new_ip = torch.zeros_like(old_ip)
                new_ip[:, 1:] = new_res.cumsum(1).int()
                rows_new = O.relayout_rows(ref["inverse"][:, :n_so_far], old_ip, new_ip)
                packed_new, posting_new = ref["packed"].clone(), ref["posting"].clone()
                for h in range(hkv):
                    rows_old = ref["inverse"][h, :n_so_far].long()
                    packed_new[:, rows_new[h], h] = ref["packed"][:, rows_old, h]
                    posting_new[h, rows_new[h]] = ref["posting"][h, rows_old]
                ref["packed"], ref["posting"], ref["indptr"], ref["reserve"] = packed_new, posting_new, new_ip, new_res
                ref["inverse"][:, :n_so_far] = rows_new.int()
                ref["repacks"] += 1

            if sess.index is not None and start == 4096:
                # force the repack path once more: same proportions, the store laid out again
                sess._repack(start)
                oracle_repack(start)
                assert torch.equal(sess.index.bucket_indptr.cpu(), ref["indptr"])
                assert torch.equal(sess.index._inverse_positions[:, :start].cpu(), ref["inverse"][:, :start])
            out = sess.slice(data["q_post"][sl].to(dev), data["q_pre"][sl].to(dev), data["k_post"][sl].to(dev),
                             data["v"][sl].to(dev), data["k_pre"][sl].to(dev), start, stop)
            _status_ok(dev)
            qpos = torch.arange(start, stop)
            if ref is None:
                want, _ = O.dense_causal_attention(data["q_post"][sl], data["k_post"][:stop], data["v"][:stop], qpos,
                                                   sm_scale)
                _close(out, want, f"dense start, slice at {start}")
                continue
            # the slice's keys: ids, rows, store contents
            ids = sess.index.orig_bucket[:, sl].cpu()
            _ids_match(ids, product[sl], ref["codebooks"], f"slice at {start}")
            rows_want, counts = O.append_rows(ids, ref["indptr"], ref["sizes"])
            if bool((ref["sizes"].long() + counts > ref["reserve"]).any()):     # a cluster outgrew its reservation
                oracle_repack(start)
                rows_want, counts = O.append_rows(ids, ref["indptr"], ref["sizes"])
                if bool((ref["sizes"].long() + counts > ref["reserve"]).any()):  # still too small: include the slice
                    oracle_repack(start, counts, chunk)
                    rows_want, counts = O.append_rows(ids, ref["indptr"], ref["sizes"])
            assert torch.equal(sess.index.bucket_indptr.cpu(), ref["indptr"])
            assert torch.equal(sess.index._inverse_positions[:, sl].cpu().long(), rows_want)
            sizes_before = ref["sizes"].clone()
            for h in range(hkv):
                ref["packed"][0][:, h].index_copy_(0, rows_want[h], data["k_post"][sl, h])
                ref["packed"][1][:, h].index_copy_(0, rows_want[h], data["v"][sl, h])
                ref["posting"][h].index_copy_(0, rows_want[h], qpos.int())
            ref["inverse"][:, sl] = rows_want.int()
            ref["sizes"] = (ref["sizes"].long() + counts).int()
            assert torch.equal(sess.index.bucket_sizes.cpu(), ref["sizes"])
            assert torch.equal(sess.snapshot.sizes.cpu(), sizes_before)
            used = int(ref["indptr"][:, -1].max())
            assert torch.equal(sess.index.packed_kv.cpu()[:, :used], ref["packed"][:, :used])
            # attention: dense through the inverse map up to the cap, the sparse body afterwards
            if start <= 4 * target:
                want, _ = O.dense_causal_attention(data["q_post"][sl], data["k_post"][:stop], data["v"][:stop], qpos,
                                                   sm_scale)
                _close(out, want, f"dense through the inverse map, slice at {start}")
                continue
            sparse_slices += 1
            sel = O.unpack_bits(sess.snapshot.qmask[:chunk].cpu())
            oidx = O.FlatIndex(codebooks=ref["codebooks"], posting_positions=ref["posting"][:, :used],
                               bucket_indptr=ref["indptr"], bucket_sizes=sizes_before, inverse_positions=ref["inverse"],
                               assign=sess.index.orig_bucket.cpu().long(), prompt_length=total, page_align=align,
                               packed_kv=ref["packed"])
            want, _ = O.sparse_chunk_attention(data["q_post"][sl], oidx, sel, sizes_before, qpos, data["k_post"][sl],
                                               data["v"][sl], start, sm_scale)
            _close(out, want, f"sparse slice at {start}")
            vectors = O.trivial_router_vectors(data["q_pre"][sl])
            own = O.select_clusters(vectors, ref["codebooks"], sizes_before, temperature=0.1, beta=0.25,
                                    target_tokens=target, sink=sink, iters=16)
            assert int((sel != own).any(-1).sum()) <= 0.02 * chunk * hkv
        assert sparse_slices == 4 and sess.repacks == ref["repacks"] >= 1
    finally:
        os.environ.pop("SEMBLO_SINK_TOKENS", None)


@pytest.mark.parametrize("dim,sink", [(256, 64), (128, 0)])
def test_suffix_flush_repacks_the_arena(dev, dim, sink):
    from types import SimpleNamespace
    from semblo_b200.arena import DecodeArena
    from semblo_b200.fused_decode import fused_decode_step
    from semblo_b200 import suffix_flush as F
    hq, hkv, length, steps, keep = 8, 2, 3000, 40, 8
    data = O.mixture_inputs(length=length + steps, num_q_heads=hq, num_kv_heads=hkv, head_dim=dim, centres=16, seed=13)
    product = O.routing_normalize(data["k_pre"][:length])
    index = O.build_flat(product, unit_tokens=32, min_clusters_log2=7, kmeans_sample_size=1024, fit_iters=4, seed=0,
                         sink=sink, page_align=16)
    O.pack_prompt_kv(index, data["k_post"][:length], data["v"][:length])
    ref = O.make_arena(capacity=4096, num_clusters=128, num_kv_heads=hkv, head_dim=dim, page_align=16, reserve=256,
                       kv_dtype=torch.bfloat16, desc_dtype=torch.bfloat16, keep_kpre=True)
    O.arena_adopt(ref, index)
    arena = DecodeArena(capacity=4096, num_kv_heads=hkv, head_dim=dim, num_clusters=128, page_align=16, device=dev,
                        reserve=256, keep_kpre=True)
    from test_gpu_parity import _gpu_index
    arena.adopt(_gpu_index(index, dev))
    layer = SimpleNamespace(num_heads=hq, num_kv_heads=hkv, head_dim=dim)
    out = torch.empty(1, hq * dim, dtype=torch.bfloat16, device=dev)
    os.environ["SEMBLO_SINK_TOKENS"] = str(sink)
    try:
        for s in range(steps):
            pos = length + s
            O.suffix_write(ref, pos, data["k_post"][pos], data["v"][pos], data["k_pre"][pos])
            fused_decode_step(layer, arena, q_post=data["q_post"][pos:pos + 1].to(dev),
                              q_pre=data["q_pre"][pos:pos + 1].to(dev),
                              positions=torch.tensor([pos], device=dev), k_post=data["k_post"][pos:pos + 1].to(dev),
                              v_states=data["v"][pos:pos + 1].to(dev), k_pre=data["k_pre"][pos:pos + 1].to(dev),
                              output=out, temperature=0.1, beta=0.25, target_tokens=256, sm_scale=dim ** -0.5,
                              num_splits=4)
        rng = F.flush_range(length, steps, length, keep, 16)
        assert rng == O.flush_range(length, steps, length, keep, 16) == (length, length + steps - keep)
        frm, to = rng
        # the oracle's flush with the kernel's own assignment (ids are checked separately)
        pos = torch.arange(frm, to)
        blk = pos // ref.suffix_block
        phys = ref.suffix_table[0, blk].long()
        off = pos - blk * ref.suffix_block
        kpre = ref.suffix_kpre[phys, off]
        from semblo_b200.token_outer import nearest_cluster
        ids = nearest_cluster(O.routing_normalize(kpre).to(dev), arena.codebooks)
        _ids_match(ids, O.routing_normalize(kpre), ref.codebooks, "flush assignment")
        widest_want = O.repack_apply(ref.packed_kv, ref.posting, ref.sizes, ref.indptr, ref.suffix_kv[:, phys, off],
                                     pos.to(torch.int32), ids.cpu().long(), 16)
        ref.prompt_length_t.fill_(to)
        O.arena_extend_suffix_table(ref, to + ref.reserve - 1)
        widest = F.flush_arena(arena, frm, to)
        _status_ok(dev)
        assert widest == widest_want
        assert torch.equal(arena.sizes.cpu(), ref.sizes)
        assert torch.equal(arena.indptr.cpu(), ref.indptr)
        assert torch.equal(arena.posting.cpu()[:, :widest], ref.posting[:, :widest])
        assert torch.equal(arena.packed_kv.cpu()[:, :widest], ref.packed_kv[:, :widest])
        assert int(arena.prompt_length_t.item()) == to
        assert torch.equal(arena.suffix_table.cpu(), ref.suffix_table)
        # decode goes on over the flushed store
        pos_next = length + steps - 1
        fused_decode_step(layer, arena, q_post=data["q_post"][pos_next:pos_next + 1].to(dev),
                          q_pre=data["q_pre"][pos_next:pos_next + 1].to(dev),
                          positions=torch.tensor([pos_next], device=dev), k_post=None, v_states=None, k_pre=None,
                          output=out, temperature=0.1, beta=0.25, target_tokens=256, sm_scale=dim ** -0.5, num_splits=4)
        _status_ok(dev)
        ws = arena.fused_decode_ws
        sel = torch.zeros(hkv, 128, dtype=torch.bool)       # the kernel's selection, recovered from its CSR
        for h in range(hkv):
            n = int(ws.rcount[h])
            starts = ws.rstart[h, :n].cpu()
            sel[h, torch.searchsorted(ref.indptr[h].contiguous(), starts, right=True) - 1] = True
        want, _, _ = O.decode_step(ref, q_post=data["q_post"][pos_next], q_pre=data["q_pre"][pos_next], pos=pos_next,
                                   k_post=None, v=None, temperature=0.1, beta=0.25, target_tokens=256, sink=sink,
                                   sm_scale=dim ** -0.5, sel=sel)
        _close(out.view(hq, dim), want, "decode after the flush")
    finally:
        os.environ.pop("SEMBLO_SINK_TOKENS", None)
