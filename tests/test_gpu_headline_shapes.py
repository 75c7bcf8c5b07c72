"""Parity at the benchmarked shapes themselves: the decode step on a 524288-token arena with 8192
clusters and 37 splits, selection exactness at 8192 and 16384 clusters, and one sparse chunk and
a few decode steps of the 1048576-token, 8-KV-head, head_dim-128, 16384-cluster configuration.

The index is built by the CUDA path; the same integer index is handed to the oracle, so what is
compared is the selection rule and the attention body at these template instantiations."""
from __future__ import annotations

import os
from types import SimpleNamespace

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


def _set_env(unit, sink, local=None):
    os.environ["SEMBLO_FLAT_UNIT_TOKENS"] = str(unit)
    os.environ["SEMBLO_FA3_ALIGN"] = "16"
    os.environ["SEMBLO_SINK_TOKENS"] = str(sink)
    if local is not None:
        os.environ["SEMBLO_FA3_LOCAL"] = str(local)


def _clear_env():
    for k in ("SEMBLO_FLAT_UNIT_TOKENS", "SEMBLO_FA3_ALIGN", "SEMBLO_SINK_TOKENS", "SEMBLO_FA3_LOCAL"):
        os.environ.pop(k, None)


def _mixture_keys(length, hkv, dim, centres, seed, dev):
    """Gaussian-mixture keys and N(0,1) values on the device (sigma 0.3 around N(0,1) centres);
    no RoPE: decode and the sparse body are indifferent to it."""
    g = torch.Generator(device=dev)
    g.manual_seed(seed)
    cent = torch.randn(hkv, centres, dim, generator=g, device=dev)
    z = torch.randint(0, centres, (length,), generator=g, device=dev)
    k = torch.empty(length, hkv, dim, dtype=torch.bfloat16, device=dev)
    step = 131072
    for lo in range(0, length, step):
        hi = min(length, lo + step)
        k[lo:hi] = (cent[:, z[lo:hi]].permute(1, 0, 2)
                    + 0.3 * torch.randn(hi - lo, hkv, dim, generator=g, device=dev)).to(torch.bfloat16)
    v = torch.randn(length, hkv, dim, generator=g, device=dev).to(torch.bfloat16)
    return cent, z, k, v


def _queries_for(cent, z_rows, group, seed, dev):
    g = torch.Generator(device=dev)
    g.manual_seed(seed)
    hkv, _, dim = cent.shape
    base = cent[:, z_rows].permute(1, 0, 2)[:, :, None, :]
    q = base + 0.3 * torch.randn(z_rows.numel(), hkv, group, dim, generator=g, device=dev)
    return q.reshape(z_rows.numel(), hkv * group, dim).to(torch.bfloat16)


def _oracle_index(index, length):
    return O.FlatIndex(codebooks=index.codebooks.cpu(), posting_positions=index.posting_positions.cpu(),
                       bucket_indptr=index.bucket_indptr.cpu(), bucket_sizes=index.bucket_sizes.cpu(),
                       inverse_positions=index.inverse_positions().cpu(), assign=index.orig_bucket.cpu().long(),
                       prompt_length=length, page_align=16, packed_kv=index.packed_kv.cpu())


def _decode_steps_against_oracle(dev, *, length, hq, hkv, dim, centres, clusters, target, sink, reserve, splits,
                                 steps, seed):
    """Build on the GPU, adopt into both arenas, run ``steps`` decode steps; CSR bit-equal to
    the oracle's selection outside its 1e-4 margin, output within the bf16 tolerance of the oracle
    evaluated on the kernel's own selection, suffix store bytes equal at the end."""
    from semblo_b200 import _lib
    from semblo_b200.arena import DecodeArena
    from semblo_b200.flat_index import routing_normalize
    from semblo_b200.fused_decode import fused_decode_step
    from semblo_b200.state import ProductPostingIndex
    group = hq // hkv
    cent, z, k, v = _mixture_keys(length + steps, hkv, dim, centres, seed, dev)
    q = _queries_for(cent, z[length:], group, seed + 1, dev)
    index = ProductPostingIndex.build(routing_normalize(k[:length]), torch.arange(length, device=dev),
                                      kmeans_sample_size=8192, codebook_seed=0, flat_unit_tokens=64,
                                      flat_min_clusters_log2=7, page_align=16)
    assert int(index.num_buckets) == clusters
    index.pack_prompt_kv(k[:length].contiguous(), v[:length].contiguous())
    capacity = 1 << (length - 1).bit_length()
    arena = DecodeArena(capacity=capacity, num_kv_heads=hkv, head_dim=dim, num_clusters=clusters, page_align=16,
                        device=dev, reserve=reserve, keep_kpre=True)
    arena.adopt(index)
    ref = O.make_arena(capacity=capacity, num_clusters=clusters, num_kv_heads=hkv, head_dim=dim, page_align=16,
                       reserve=reserve, kv_dtype=torch.bfloat16, desc_dtype=torch.bfloat16, keep_kpre=True)
    O.arena_adopt(ref, _oracle_index(index, length))
    del index
    assert torch.equal(arena.suffix_table.cpu(), ref.suffix_table)
    layer = SimpleNamespace(num_heads=hq, num_kv_heads=hkv, head_dim=dim)
    sm_scale = dim ** -0.5
    out = torch.empty(1, hq * dim, dtype=torch.bfloat16, device=dev)
    kc, vc, qc = k[length:].cpu(), v[length:].cpu(), q.cpu()
    marginal = 0
    for s in range(steps):
        pos = length + s
        vectors = O.trivial_router_vectors(qc[s])
        sel_ref, _, margin = O.decode_select(vectors, ref, temperature=0.1, beta=0.25, target_tokens=target,
                                             sink=sink, return_margin=True)
        fused_decode_step(layer, arena, q_post=q[s:s + 1].contiguous(), q_pre=q[s:s + 1].contiguous(),
                          positions=torch.tensor([pos], device=dev), k_post=k[pos:pos + 1].contiguous(),
                          v_states=v[pos:pos + 1].contiguous(), k_pre=k[pos:pos + 1].contiguous(), output=out,
                          temperature=0.1, beta=0.25, target_tokens=target, sm_scale=sm_scale, num_splits=splits)
        _lib.status_for(dev).raise_if_set()
        ws = arena.fused_decode_ws
        sel = torch.zeros(hkv, clusters, dtype=torch.bool)
        for h in range(hkv):
            n = int(ws.rcount[h])
            starts = ws.rstart[h, :n].cpu()
            ids = torch.searchsorted(ref.indptr[h].contiguous(), starts, right=True) - 1
            sel[h, ids] = True
            lens = ws.rlen[h, :n].cpu()
            assert torch.equal(lens, ref.sizes[h][ids])
            assert torch.equal(ws.rcum[h, :n].cpu(), (lens.cumsum(0) - lens).int())
            assert int(ws.rtokens[h]) == int(lens.sum())
            # the budget is reached without the sink cluster, and not by more than the last cluster taken
            held = sel[h].clone()
            if sink:
                assert bool(sel[h, 0])
                held[0] = False
            assert int((held * ref.sizes[h]).sum()) >= min(target - sink, int(ref.sizes[h][1:].sum()))
        differ = (sel != sel_ref).any(-1)
        assert bool((margin[differ] < 1e-4).all()), (s, margin[differ])
        marginal += int(differ.sum())
        want, _, _ = O.decode_step(ref, q_post=qc[s], q_pre=qc[s], pos=pos, k_post=kc[s], v=vc[s], k_pre=kc[s],
                                   temperature=0.1, beta=0.25, target_tokens=target, sink=sink, sm_scale=sm_scale,
                                   sel=sel)
        diff = (out.view(hq, dim).double().cpu() - want).abs()
        assert float(diff.max()) <= MAX_ABS, f"step {s}: max-abs {float(diff.max()):.4g}"
        assert float(diff.mean()) <= MEAN_ABS, f"step {s}: mean-abs {float(diff.mean()):.4g}"
    assert marginal <= max(1, steps * hkv // 4)
    assert torch.equal(arena.suffix_kv.cpu().float(), ref.suffix_kv.float())
    assert torch.equal(arena.suffix_kpre.cpu().float(), ref.suffix_kpre.float())


def test_decode_at_524288_tokens_8192_clusters_37_splits(dev):
    """The benchmark's decode instantiation (16 query / 4 KV heads, head_dim 256).  The prompt ends three
    positions before a 256-row suffix block boundary, so the steps cross it."""
    _set_env(64, 128)
    try:
        _decode_steps_against_oracle(dev, length=524288 - 3, hq=16, hkv=4, dim=256, centres=512, clusters=8192,
                                     target=4096, sink=128, reserve=1024, splits=37, steps=8, seed=31)
    finally:
        _clear_env()


def test_decode_at_1048576_tokens_16384_clusters_head_dim_128(dev):
    """The head-sharded configuration's decode shape: 32 query / 8 KV heads, head_dim 128, budget 8192."""
    _set_env(64, 128)
    try:
        _decode_steps_against_oracle(dev, length=1048576 - 2, hq=32, hkv=8, dim=128, centres=1024, clusters=16384,
                                     target=8192, sink=128, reserve=1024, splits=18, steps=4, seed=57)
    finally:
        _clear_env()


@pytest.mark.parametrize("clusters", [8192, 16384])
def test_threshold_selection_exact_at_large_cluster_counts(dev, clusters):
    """The selector used above 4096 clusters against the oracle's float32 rule on identical scores."""
    from semblo_b200._lib import lib, ptr, check, stream_ptr
    g = torch.Generator().manual_seed(clusters)
    nq, hkv, target = 41, 3, 8192 - 128
    sizes = torch.randint(0, 130, (hkv, clusters), generator=g).int()
    sizes[:, ::7] = 0
    sizes[2] = (sizes[2] > 126).int()                     # everything fits for head 2
    score = torch.randn(nq, hkv, clusters, generator=g) * 2
    score = torch.where(sizes[None] > 0, score, torch.full_like(score, O.NEG_BIG))
    want = O.theta_select(score, sizes[None], target, 16)
    qmask = torch.empty(nq, hkv, clusters // 32, dtype=torch.int32, device=dev)
    counts = torch.empty(nq, hkv, dtype=torch.int32, device=dev)
    tokens = torch.empty(nq, hkv, dtype=torch.int32, device=dev)
    top1 = torch.empty(hkv, nq, dtype=torch.int32, device=dev)
    score_d, sizes_d = score.to(dev), sizes.to(dev)
    check(lib().semblo_select_clusters(ptr(score_d), ptr(sizes_d), nq, hkv, clusters, target, 16, 0,
                                       ptr(qmask), ptr(counts), ptr(tokens), ptr(top1), 0.0, stream_ptr()))
    assert torch.equal(O.unpack_bits(qmask.cpu()), want)
    assert torch.equal(counts.cpu(), want.sum(-1).int())
    assert torch.equal(tokens.cpu(), (want * sizes[None]).sum(-1).int())
    assert torch.equal(top1.cpu().long().t(), score.argmax(-1))


def test_sparse_chunk_of_the_1048576_token_configuration(dev):
    """One sparse chunk of the head-sharded configuration at its own shape (32 query / 8 KV heads,
    head_dim 128, 16384 clusters, budget 8192, sink 128, window 512): the selection is the rule applied
    to the kernel's own scores, sampled queries match the oracle's per-query gather."""
    from semblo_b200 import _lib
    from semblo_b200.flat_index import routing_normalize
    from semblo_b200.fused_prefill import CausalSnapshot, fused_chunk_attention
    from semblo_b200.state import ProductPostingIndex
    from semblo_b200.trivial_router import trivial_router_vectors
    length, hq, hkv, dim, target, sink, local, chunk = 1048576, 32, 8, 128, 8192, 128, 512, 8192
    _set_env(64, sink, local)
    try:
        cent, z, k, v = _mixture_keys(length, hkv, dim, 1024, 77, dev)
        index = ProductPostingIndex.build(routing_normalize(k), torch.arange(length, device=dev),
                                          kmeans_sample_size=8192, codebook_seed=0, flat_unit_tokens=64,
                                          flat_min_clusters_log2=7, page_align=16)
        assert int(index.num_buckets) == 16384
        index.pack_prompt_kv(k, v)
        index.original_kv = (k, v)
        cs = 90 * chunk
        ce = cs + chunk - 1
        q = _queries_for(cent, z[cs:ce + 1], hq // hkv, 78, dev)
        snap = CausalSnapshot(index)
        qv = trivial_router_vectors(q)
        out = torch.empty(chunk, hq, dim, dtype=torch.bfloat16, device=dev)
        fused_chunk_attention(q, SimpleNamespace(vectors=qv.view(1, chunk, hq, 1, dim)), index,
                              torch.arange(cs, ce + 1, dtype=torch.int32, device=dev), snap, cs, ce,
                              temperature=0.1, beta=0.25, target_tokens=target, sm_scale=dim ** -0.5, out=out)
        torch.cuda.synchronize()
        _lib.status_for(dev).raise_if_set()
        assert bool(torch.isfinite(out.float()).all())
        ws = cs - local
        sizes = snap.advance(ws - 1).cpu()
        pick = torch.randperm(chunk, generator=torch.Generator().manual_seed(5))[:12].sort().values
        sel = O.unpack_bits(snap.qmask[:chunk][pick.to(dev)].cpu())
        # the selection is exactly the rule on the kernel's own scores
        held_sizes, held_target = O.hold_out_sink(sizes, target, sink)
        own = O.theta_select(snap.score[:chunk][pick.to(dev)].cpu(), held_sizes[None], held_target, 16)
        own[..., 0] = True
        assert torch.equal(sel, own)
        tokens = ((sel & (torch.arange(16384) > 0)) * sizes[None]).sum(-1)
        assert bool((tokens >= target - sink).all())
        oidx = _oracle_index(index, length)
        want = O.sparse_chunk_attention_gather(q.cpu()[pick], oidx, sel, sizes, cs + pick, k[ws:ce + 1].cpu(),
                                               v[ws:ce + 1].cpu(), ws, dim ** -0.5, dtype=torch.float32)
        diff = (out.cpu()[pick].float() - want).abs()
        assert float(diff.max()) <= MAX_ABS, f"sampled queries: max-abs {float(diff.max()):.4g}"
        assert float(diff.mean()) <= MEAN_ABS
    finally:
        _clear_env()
