"""Benchmark of the semblo sparse-attention hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

One step = one full sparse prefill of one full-attention layer over one synthetic prompt:
routing normalisation, k-means fit (8 iterations) and assignment of the keys, page-aligned
cluster layout, the cluster-ordered paged K/V copy, then the query-chunk loop (query routing
vectors, causal snapshot, centroid scoring, budgeted selection, block-sparse attention with
the exact local window; exact dense attention while the prefix is below four budgets).

Workload at N = 1: 131072-token prompt, 16 query / 4 KV heads, head_dim 256, bf16, partial
RoPE on 25 % of the dims, keys from a 256-centre Gaussian mixture per head, 64-token blocks,
budget 4096 tokens + 128-token sink + 512-token local window, 16-token pages behind a seeded
random page permutation.  At N > 1 every rank runs that step for its own 4-KV-head shard of a
layer with 4 N KV heads and the per-head outputs are all-gathered with NCCL, chunk by chunk on a
communication stream while the next chunk computes (head-parallel, weak scaling); the value
then counts token-shards per second.

The JSON line also carries
  * ``decode``: microseconds per step at 524288 tokens and the roofline of its kernels;
  * ``head_sharded``: the head-sharded configuration as written - one 1048576-token layer with
    32 query / 8 KV heads of head_dim 128, 16384 clusters, budget 8192, its KV heads split
    8 / 4 / 2 / 1 per GPU on 1 / 2 / 4 / 8 GPUs (strong scaling), then 128 decode steps, every
    output gathered over NVLink;
  * ``roofline``: the sparse kernel's own fraction first, then every attention launch kind.
``--impl reference`` times the reference path on the host cores (the reference's own torch
functions where they run on a CPU and are present, the CPU restatement for the rest) on a
bounded sample of the same workload.
"""
from __future__ import annotations

import argparse
import gc
import json
import os
import subprocess
import sys
import threading
import time
from pathlib import Path
from types import SimpleNamespace

ROOT = Path(__file__).resolve().parent
for _p in (str(ROOT), str(ROOT / "semantic-block-sparse-attention_b200")):
    if _p not in sys.path:
        sys.path.insert(0, _p)

import torch  # noqa: E402

PREFILL = dict(length=131072, hq=16, hkv=4, dim=256, centres=256, unit=64, min_log2=7, target=4096,
               sink=128, local=512, chunk=8192, temperature=0.1, beta=0.25, page=16)
# dram__bytes_read.sum + dram__bytes_write.sum per launch, from one-pass ncu captures of this file's own
# command, keyed by (kernel, prompt length): a record of a past capture, not something a run produces
DRAM_TRAFFIC_PER_LAUNCH = {("sparse_gather_prefill_kernel<256,4>", 131072): 1.094e9,
                           ("decode_attend_kernel<256,4>", 524288): 17.78e6,
                           ("decode_score_kernel<256,4>", 524288): 16.85e6,
                           ("decode_select_kernel", 524288): 0.84e6}

HEAD_SHARDED = dict(length=1048576, hq=32, hkv=8, dim=128, centres=1024, unit=64, min_log2=7, target=8192,
                    sink=128, local=512, chunk=8192, temperature=0.1, beta=0.25, page=16, reserve=1024,
                    decode_steps=128)

DECODE = dict(length=524288, hq=16, hkv=4, dim=256, centres=512, unit=64, min_log2=7, target=4096,
              sink=128, reserve=1024, steps=256, temperature=0.1, beta=0.25, splits=37)


def peaks():
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        p = json.loads(path.read_text())
        return dict(hbm=float(p["hbm_gbs"]), tensor=float(p.get("bf16_tflops_sustained", p["bf16_tflops"])),
                    tensor_burst=float(p["bf16_tflops"]), source="measured")
    return dict(hbm=6650.0, tensor=1400.0, tensor_burst=1590.0, source="fallback")


# ------------------------------------------------------------------------- synthetic inputs
def mixture_inputs_device(cfg, seed, device, length=None, heads=None):
    """Seeded Gaussian-mixture keys/queries (sigma 0.3 around N(0,1) centres), N(0,1) values,
    partial RoPE (theta 1e7) on the first quarter of the dims: the recipe of the oracle's
    ``mixture_inputs``, generated on the device.  Every KV head has a generator of its own
    (seed + 7919 * global head id; the cluster label of a token is shared), so a rank that holds
    the heads ``heads`` of a layer gets exactly those heads of the unsharded tensors."""
    length = length or cfg["length"]
    hq, hkv, dim = cfg["hq"], cfg["hkv"], cfg["dim"]
    group = hq // hkv
    heads = range(hkv) if heads is None else heads
    nh = len(heads)
    g = torch.Generator(device=device)
    g.manual_seed(seed)
    z = torch.randint(0, cfg["centres"], (length,), generator=g, device=device)
    pos = torch.arange(length, device=device)
    r = dim // 4
    half = r // 2
    inv = 1e7 ** (-torch.arange(half, device=device, dtype=torch.float64) / half)
    k_pre = torch.empty(length, nh, dim, dtype=torch.bfloat16, device=device)
    k_post = torch.empty_like(k_pre)
    v = torch.empty_like(k_pre)
    q_pre = torch.empty(length, nh * group, dim, dtype=torch.bfloat16, device=device)
    q_post = torch.empty_like(q_pre)

    def rope(x, lo, hi):
        ang = pos[lo:hi].double()[:, None] * inv[None]
        shape = [hi - lo] + [1] * (x.ndim - 2) + [half]
        cos, sin = ang.cos().float().view(shape), ang.sin().float().view(shape)
        out = x.clone()
        out[..., :half] = x[..., :half] * cos - x[..., half:r] * sin
        out[..., half:r] = x[..., half:r] * cos + x[..., :half] * sin
        return out

    step = 65536
    for j, h in enumerate(heads):
        g.manual_seed(seed + 7919 * (h + 1))
        cent = torch.randn(cfg["centres"], dim, generator=g, device=device)
        for lo in range(0, length, step):
            hi = min(length, lo + step)
            base = cent[z[lo:hi]]                                            # [n, D]
            kf = base + 0.3 * torch.randn(hi - lo, dim, generator=g, device=device)
            k_pre[lo:hi, j] = kf.to(torch.bfloat16)
            k_post[lo:hi, j] = rope(kf, lo, hi).to(torch.bfloat16)
            v[lo:hi, j] = torch.randn(hi - lo, dim, generator=g, device=device).to(torch.bfloat16)
            qf = base[:, None, :] + 0.3 * torch.randn(hi - lo, group, dim, generator=g, device=device)
            q_pre[lo:hi, j * group:(j + 1) * group] = qf.to(torch.bfloat16)
            q_post[lo:hi, j * group:(j + 1) * group] = rope(qf, lo, hi).to(torch.bfloat16)
    return dict(q_pre=q_pre, q_post=q_post, k_pre=k_pre, k_post=k_post, v=v)


# ------------------------------------------------------------------------- the prefill step
class PrefillStep:
    """The reference's prompt forward of one sparse layer (model.py:1169-1269: ingest, then the
    query-chunk loop of _run_product_attention 856-1008) on the mirrored entry points, for the KV
    heads this rank holds (``hkv_local`` of them, starting at global head ``head_offset``)."""

    def __init__(self, cfg, device, world=1, hkv_local=None, head_offset=0, per_head_seed=False):
        from semblo_b200 import _lib
        self.cfg, self.device, self.world = cfg, device, world
        self.hkv = cfg["hkv"] if hkv_local is None else hkv_local
        self.hq = self.hkv * (cfg["hq"] // cfg["hkv"])
        self.head_offset, self.per_head_seed = head_offset, per_head_seed
        self.page_table = None
        self.attended = torch.zeros(4, dtype=torch.int64, device=device)    # window pairs, -, sparse pairs, gathered rows
        self.attn_events = []
        self.time_attention = False
        self.gather = None
        self.windows_ahead = True           # the index-free launches run on a stream of their own, ahead
        self._lib = _lib

    def run(self, x, out, before_chunk=None, after_chunk=None):
        """One prefill step.  before_chunk / after_chunk (chunk_start, chunk_end) run on the host around
        every query chunk (before_chunk also in front of a chunk's window launch, on whatever stream is
        current then): the end-to-end measurement hangs its copies on them."""
        from semblo_b200.flat_index import routing_normalize
        from semblo_b200.fused_prefill import CausalSnapshot, WindowAhead, fused_chunk_attention
        from semblo_b200.state import ProductPostingIndex
        from semblo_b200.trivial_router import trivial_router_vectors
        cfg, dev = self.cfg, self.device
        length, hq, dim, chunk = cfg["length"], self.hq, cfg["dim"], cfg["chunk"]
        sm_scale = dim ** -0.5
        window = None
        if self.windows_ahead and not self.time_attention:
            window = WindowAhead(x["q_post"], self.positions32, x["k_post"], x["v"], chunk=chunk,
                                 target_tokens=cfg["target"], sm_scale=sm_scale, out=out, attended=self.attended,
                                 ahead=16, before_launch=before_chunk, router_input=x["q_pre"])
        product = routing_normalize(x["k_pre"])
        index = ProductPostingIndex.build(product, self.positions, kmeans_sample_size=8192, codebook_seed=0,
                                          flat_unit_tokens=cfg["unit"], flat_min_clusters_log2=cfg["min_log2"],
                                          page_align=cfg["page"], per_head_seed=self.per_head_seed,
                                          head_offset=self.head_offset)
        del product
        width = int(index.posting_positions.shape[1])
        n_pages = (width + (-width) % 256) // 16
        if self.page_table is None or self.page_table.numel() != n_pages:
            g = torch.Generator(device=dev)
            g.manual_seed(1234)
            self.page_table = torch.randperm(n_pages, generator=g, device=dev).to(torch.int32)
        index.pack_prompt_kv(x["k_post"], x["v"], page_table=self.page_table)
        index.original_kv = (x["k_post"], x["v"])
        snap = CausalSnapshot(index)
        for cs in range(0, length, chunk):
            ce = min(length, cs + chunk) - 1
            n = ce - cs + 1
            if before_chunk is not None:
                before_chunk(cs, ce)
            if window is not None:
                state = SimpleNamespace(vectors=window.vectors_for(cs))        # made ahead; None for a dense chunk
            else:
                qv = trivial_router_vectors(x["q_pre"][cs:ce + 1])
                state = SimpleNamespace(vectors=qv.view(1, n, hq, 1, dim))
            fused_chunk_attention(x["q_post"][cs:ce + 1], state, index, self.positions32[cs:ce + 1], snap, cs, ce,
                                  temperature=cfg["temperature"], beta=cfg["beta"], target_tokens=cfg["target"],
                                  sm_scale=sm_scale, out=out[cs:ce + 1], attended=self.attended, window=window,
                                  _timer=self._timer if self.time_attention else None)
            if self.world > 1:
                # The one collective of the path: the chunk's per-head outputs to every rank.  It runs on a
                # communication stream behind this chunk's kernels while the next chunk computes; two
                # receive buffers alternate, and the step ends when the last gather has landed.
                if self.gather is None:
                    from semblo_b200.head_parallel import HeadGather
                    self.gather = HeadGather()
                    self.full_out = torch.empty(2, self.world, chunk, hq, dim, dtype=torch.bfloat16, device=dev)
                if n != chunk:
                    raise RuntimeError("the prompt length must be a multiple of the query chunk")
                self.gather.issue(out[cs:ce + 1], self.full_out[(cs // chunk) % 2])
            if after_chunk is not None:
                after_chunk(cs, ce)
        if window is not None:
            window.finish()
        if self.gather is not None:
            self.gather.wait()
        return index

    def _timer(self, phase):
        ev = torch.cuda.Event(enable_timing=True)
        ev.record()
        self.attn_events.append((phase, ev))

    def prepare(self):
        L = self.cfg["length"]
        self.positions = torch.arange(L, device=self.device)
        self.positions32 = self.positions.to(torch.int32)


def set_env(cfg):
    os.environ["SEMBLO_FLAT_UNIT_TOKENS"] = str(cfg["unit"])
    os.environ["SEMBLO_FA3_ALIGN"] = "16"
    os.environ["SEMBLO_SINK_TOKENS"] = str(cfg["sink"])
    if "local" in cfg:
        os.environ["SEMBLO_FA3_LOCAL"] = str(cfg["local"])


class ClockSampler:
    """nvidia-smi SM clock and throttle reasons during the timed region."""

    def __init__(self, index):
        self.index, self.samples, self.reasons, self.max_mhz = index, [], set(), None
        self.busy = []                      # clocks of the samples taken while the GPU reported work
        self.proc = None

    def start(self):
        q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap,utilization.gpu")
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.index}", f"--query-gpu={q}",
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.proc.stdout:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 6:
                continue
            try:
                self.samples.append(float(parts[0]))
                self.max_mhz = float(parts[1])
            except ValueError:
                continue
            for n, v in zip(names, parts[2:6]):
                if v.lower().startswith("active"):
                    self.reasons.add(n)
            try:
                if len(parts) > 6 and float(parts[6]) >= 30.0:
                    self.busy.append(float(parts[0]))
            except ValueError:
                pass

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": []}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        # the median over the samples taken under load (reported utilisation of at least 30 %; an idle
        # GPU with a context sits at its maximum clock, so the idle readings are the high ones); all
        # samples if none qualified (a run shorter than the tool's update period)
        s = sorted(self.busy) if self.busy else sorted(self.samples)
        med = s[len(s) // 2] if s else None
        return {"sm_mhz": med, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons),
                "samples_under_load": len(self.busy), "samples": len(self.samples)}


# ------------------------------------------------------------------------- launch accounting
def kernel_launches(calls: dict, clusters: int, chunk: int) -> int:
    passes = 1 if clusters <= 256 else 2
    order_sort = 1 if chunk <= 8192 and clusters <= 2048 else 3 * passes   # short key lists sort in one launch
    counts = 1                                      # histogram and scans in one launch up to 131072 keys
    per_call = {"semblo_routing_normalize": 1, "semblo_gather_rows": 1, "semblo_assign_argmax": 1,
                "semblo_cluster_counts": counts, "semblo_kmeans_update": 3 * passes + 1, "semblo_kmeans_sort_members": 3 * passes,
                "semblo_kmeans_update_sorted": 1, "semblo_split_descriptor": 1,
                "semblo_build_layout": counts + 3 * passes + 1, "semblo_pack_kv": 1, "semblo_snapshot_advance": 1,
                "semblo_score_clusters": 1, "semblo_select_clusters": 1, "semblo_window_prefill": 1, "semblo_sparse_prefill_gather": 1, "semblo_gather_launch_order": 2,
                "semblo_argsort_keys": order_sort,
                "semblo_decode_step": 3}
    return sum(per_call.get(k, 0) * v for k, v in calls.items())


# ------------------------------------------------------------------------- selection alone
def select_measure(device, clusters=2048, queries=8192, heads=4, target=4096, reps=4):
    """One chunk's selection launch on seeded scores (a small case for profiling the kernel)."""
    from semblo_b200._lib import lib, ptr, check, stream_ptr
    g = torch.Generator(device=device).manual_seed(1)
    score = (torch.randn(queries, heads, clusters, device=device, generator=g) * 8 - 20).float()
    sizes = torch.randint(0, 130, (heads, clusters), device=device, generator=g, dtype=torch.int32)
    qmask = torch.empty(queries, heads, clusters // 32, dtype=torch.int32, device=device)
    top1 = torch.empty(heads, queries, dtype=torch.int32, device=device)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    us = []
    for _ in range(reps):
        e0.record()
        check(lib().semblo_select_clusters(ptr(score), ptr(sizes), queries, heads, clusters, target, 16, 0, ptr(qmask),
                                           None, None, ptr(top1), 0.25, stream_ptr()))
        e1.record()
        torch.cuda.synchronize()
        us.append(round(e0.elapsed_time(e1) * 1e3, 1))
    return {"metric": "select_us_per_chunk", "clusters": clusters, "queries": queries, "kv_heads": heads,
            "launch_us": us, "score_bytes": score.numel() * 4}


# ------------------------------------------------------------------------- decode measurement
def decode_measure(device, pk):
    """Decode at 524288 tokens: build the index once, adopt it into the arena, then time decode
    steps appended through the suffix store (eager launches and a captured CUDA graph)."""
    from semblo_b200 import _lib
    from semblo_b200.arena import DecodeArena
    from semblo_b200.fused_decode import fused_decode_step
    from semblo_b200.flat_index import routing_normalize
    from semblo_b200.state import ProductPostingIndex, flat_num_clusters
    cfg = DECODE
    set_env(cfg)
    L, hq, hkv, dim = cfg["length"], cfg["hq"], cfg["hkv"], cfg["dim"]
    steps = cfg["steps"]
    x = mixture_inputs_device(cfg, 3000, device, length=L + steps)
    positions = torch.arange(L, device=device)
    product = routing_normalize(x["k_pre"][:L])
    index = ProductPostingIndex.build(product, positions, kmeans_sample_size=8192, codebook_seed=0,
                                      flat_unit_tokens=cfg["unit"], flat_min_clusters_log2=cfg["min_log2"], page_align=16)
    index.pack_prompt_kv(x["k_post"][:L].contiguous(), x["v"][:L].contiguous())
    clusters = flat_num_clusters(L, cfg["unit"], cfg["min_log2"])
    arena = DecodeArena(capacity=L, num_kv_heads=hkv, head_dim=dim, num_clusters=clusters, page_align=16,
                        device=device, reserve=cfg["reserve"], keep_kpre=True)
    arena.adopt(index)
    del index, product
    layer = SimpleNamespace(num_heads=hq, num_kv_heads=hkv, head_dim=dim)
    out = torch.empty(1, hq * dim, dtype=torch.bfloat16, device=device)
    pos_t = torch.zeros(1, dtype=torch.int64, device=device)
    bufs = {k: torch.empty(1, *x[k].shape[1:], dtype=torch.bfloat16, device=device) for k in x}
    sm_scale = dim ** -0.5

    def step():
        fused_decode_step(layer, arena, q_post=bufs["q_post"], q_pre=bufs["q_pre"], positions=pos_t,
                          k_post=bufs["k_post"], v_states=bufs["v"], k_pre=bufs["k_pre"], output=out,
                          temperature=cfg["temperature"], beta=cfg["beta"], target_tokens=cfg["target"],
                          sm_scale=sm_scale, num_splits=cfg["splits"])

    def load(s):
        for k in bufs:
            bufs[k].copy_(x[k][L + s:L + s + 1])
        pos_t.fill_(L + s)

    flush = torch.empty(256 << 20, dtype=torch.uint8, device=device)
    for s in range(4):
        load(s)
        step()
    torch.cuda.synchronize()
    _lib.status_for(device).raise_if_set()
    # eager, L2 flushed before every step
    ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(steps)]
    for s in range(steps):
        load(s)
        flush.zero_()
        ev[s][0].record()
        step()
        ev[s][1].record()
    torch.cuda.synchronize()
    eager_us = sorted(a.elapsed_time(b) * 1e3 for a, b in ev)
    ws = arena.fused_decode_ws
    n_rows = int(ws.rtokens.sum().item())
    n_suffix = hkv * steps                      # at the last step
    # graph replay
    graph = torch.cuda.CUDAGraph()
    load(steps - 1)
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        step()
    torch.cuda.current_stream().wait_stream(side)
    with torch.cuda.graph(graph):
        step()
    gev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(steps)]
    for s in range(steps):
        load(s)
        flush.zero_()
        gev[s][0].record()
        graph.replay()
        gev[s][1].record()
    torch.cuda.synchronize()
    _lib.status_for(device).raise_if_set()
    graph_us = sorted(a.elapsed_time(b) * 1e3 for a, b in gev)
    # sixteen steps back to back in one graph (same query, so the codebook and the rows stay in L2):
    # what a step costs without the launch of a graph around it
    g16 = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g16):
        for _ in range(16):
            step()
    b2b = []
    for _ in range(16):
        a_ev, b_ev = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a_ev.record()
        g16.replay()
        b_ev.record()
        b2b.append((a_ev, b_ev))
    torch.cuda.synchronize()
    back_to_back_us = sorted(a.elapsed_time(b) * 1e3 / 16 for a, b in b2b)
    # Each kernel alone (stage masks 1, 2, 4).  A graph of one small kernel between two events already
    # measures about 6 us on this part, so a stage is timed as the difference of two graphs: L2 flush +
    # stage, and the L2 flush alone - what the kernel adds to a stream that is already running.
    def graph_of(fn):
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            fn()
        return g

    def timed(g, n=48):
        evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(n)]
        for a, b in evs:
            a.record()
            g.replay()
            b.record()
        torch.cuda.synchronize()
        return sorted(a.elapsed_time(b) * 1e3 for a, b in evs)

    def stage(mask):
        fused_decode_step(layer, arena, q_post=bufs["q_post"], q_pre=bufs["q_pre"], positions=pos_t, k_post=None,
                          v_states=None, k_pre=None, output=out, temperature=cfg["temperature"],
                          beta=cfg["beta"], target_tokens=cfg["target"], sm_scale=sm_scale,
                          num_splits=cfg["splits"], stage_mask=mask)

    med = lambda v: v[len(v) // 2]
    flush_only = med(timed(graph_of(lambda: flush.zero_())))
    stage_us = {}
    for name, mask in (("score", 1), ("select", 2), ("attend", 4)):
        g = graph_of(lambda mask=mask: (flush.zero_(), stage(mask)))
        stage_us[name] = [max(0.0, v - flush_only) for v in timed(g)]
    attend_us = stage_us["attend"]
    gathered = (n_rows + n_suffix) * dim * 2 * 2 + n_rows * 4
    codebook = hkv * clusters * dim * 2 + hkv * clusters * 8
    return {
        "metric": "decode_us_per_step", "context": L, "clusters": clusters, "steps": steps,
        "eager_us": med(eager_us), "graph_us": med(graph_us), "graph_back_to_back_warm_us": med(back_to_back_us),
        "stage_timing": "graph(L2 flush + stage) - graph(L2 flush)", "attend_kernel_us": med(attend_us),
        "score_kernel_us": med(stage_us["score"]), "select_kernel_us": med(stage_us["select"]),
        "selected_rows": n_rows, "gathered_bytes": gathered, "codebook_bytes": codebook,
        "roofline_attend": {"bound": "hbm", "achieved": gathered / (med(attend_us) * 1e-6) / 1e9, "peak": pk["hbm"],
                            "unit": "GB/s", "frac": gathered / (med(attend_us) * 1e-6) / 1e9 / pk["hbm"],
                            "traffic": DRAM_TRAFFIC_PER_LAUNCH.get(("decode_attend_kernel<256,4>", L))},
        "roofline_step": {"bound": "hbm", "achieved": (gathered + codebook) / (med(graph_us) * 1e-6) / 1e9,
                          "peak": pk["hbm"], "unit": "GB/s",
                          "frac": (gathered + codebook) / (med(graph_us) * 1e-6) / 1e9 / pk["hbm"],
                          "traffic": sum(DRAM_TRAFFIC_PER_LAUNCH.get((k, L), 0.0) for k in (
                              "decode_score_kernel<256,4>", "decode_select_kernel", "decode_attend_kernel<256,4>")) or None},
    }


# ------------------------------------------------------------------------- head-sharded configuration
def head_sharded_measure(device, rank, world, pk, steps=2, warmup=1, length=None):
    """The head-sharded configuration as written: one layer of HEAD_SHARDED['length'] tokens with 8 KV heads,
    this rank holding 8 / world of them (reference rule: num_kv_heads % tp == 0, no KV-head replication,
    semblo/vllm_plugin/config.py:464-479), strong scaling.  Prefill steps with every chunk's output
    all-gathered behind the next chunk's compute, then decode steps whose outputs are gathered too.
    Times are device times, the maximum over the ranks.  Every KV head draws its k-means randomness
    from a generator of its own, so a shard equals the same heads of the unsharded layer; that is
    checked here on a small prompt (the gathered output against the whole layer computed locally)."""
    import torch.distributed as dist
    from semblo_b200 import _lib
    from semblo_b200.arena import DecodeArena
    from semblo_b200.fused_decode import fused_decode_step
    from semblo_b200.head_parallel import HeadGather, kv_head_shard
    from semblo_b200.state import flat_num_clusters
    cfg = dict(HEAD_SHARDED)
    if length:
        cfg["length"] = length
    set_env(cfg)
    heads = kv_head_shard(cfg["hkv"], rank, world)
    hkv_l = len(heads)
    group = cfg["hq"] // cfg["hkv"]
    hq_l, dim, L = hkv_l * group, cfg["dim"], cfg["length"]

    def reduce_max(v):
        if world == 1:
            return v
        t = torch.tensor([v], dtype=torch.float64, device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    # ---- shard check on a small prompt: sharded + gathered == unsharded, bit for bit
    small = dict(cfg, length=16384, centres=64, target=1024)      # budget 1024: the second chunk is sparse
    xs_all = mixture_inputs_device(small, 4100, device)
    full = PrefillStep(small, device, 1, per_head_seed=True)
    full.prepare()
    want = torch.empty(small["length"], small["hq"], dim, dtype=torch.bfloat16, device=device)
    full.run(xs_all, want)
    xs = mixture_inputs_device(small, 4100, device, heads=heads)
    part = PrefillStep(small, device, 1, hkv_local=hkv_l, head_offset=heads.start, per_head_seed=True)
    part.prepare()
    mine = torch.empty(small["length"], hq_l, dim, dtype=torch.bfloat16, device=device)
    part.run(xs, mine)
    gathered = torch.empty(world, small["length"], hq_l, dim, dtype=torch.bfloat16, device=device)
    hg = HeadGather()
    hg.issue(mine, gathered)
    hg.wait()
    torch.cuda.synchronize()
    same = bool(torch.equal(HeadGather.as_heads(gathered), want))
    if world > 1:
        t = torch.tensor([1 if same else 0], device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MIN)
        same = bool(t.item())
    del xs_all, xs, full, part, want, mine, gathered
    torch.cuda.empty_cache()

    # ---- prefill, strong scaling
    x = mixture_inputs_device(cfg, 5000, device, length=L + cfg["decode_steps"], heads=heads)
    xp = {k: v[:L] for k, v in x.items()}
    step = PrefillStep(cfg, device, world, hkv_local=hkv_l, head_offset=heads.start, per_head_seed=True)
    step.prepare()
    out = torch.empty(L, hq_l, dim, dtype=torch.bfloat16, device=device)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(warmup):
        step.run(xp, out)
    barrier()
    _lib.status_for(device).raise_if_set()
    step.attended.zero_()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    index = None
    for _ in range(steps):
        index = None                 # the previous step's index is dropped before the next one is built
        index = step.run(xp, out)
    e1.record()
    barrier()
    _lib.status_for(device).raise_if_set()
    prefill_ms = reduce_max(e0.elapsed_time(e1) / steps)
    counts = [int(v) // steps for v in step.attended.tolist()]

    # ---- decode: the request's index moves into the arena, then one token per step
    clusters = flat_num_clusters(L, cfg["unit"], cfg["min_log2"])
    arena = DecodeArena(capacity=L, num_kv_heads=hkv_l, head_dim=dim, num_clusters=clusters, page_align=16,
                        device=device, reserve=cfg["reserve"], keep_kpre=True)
    if index.kv_page_table is not None:
        # the arena reads the cluster-ordered copy in logical order: pack once more without the page table
        index.pack_prompt_kv(xp["k_post"], xp["v"])
    arena.adopt(index)
    del index, out
    layer = SimpleNamespace(num_heads=hq_l, num_kv_heads=hkv_l, head_dim=dim)
    o_local = torch.empty(1, hq_l * dim, dtype=torch.bfloat16, device=device)
    o_full = torch.empty(world, 1, hq_l * dim, dtype=torch.bfloat16, device=device)
    pos_t = torch.zeros(1, dtype=torch.int64, device=device)
    bufs = {k: torch.empty(1, *x[k].shape[1:], dtype=torch.bfloat16, device=device) for k in x}
    splits = max(1, 148 // hkv_l)
    dsteps = cfg["decode_steps"]

    def decode_step():
        fused_decode_step(layer, arena, q_post=bufs["q_post"], q_pre=bufs["q_pre"], positions=pos_t,
                          k_post=bufs["k_post"], v_states=bufs["v"], k_pre=bufs["k_pre"], output=o_local,
                          temperature=cfg["temperature"], beta=cfg["beta"], target_tokens=cfg["target"],
                          sm_scale=dim ** -0.5, num_splits=splits)
        if world > 1:
            dist.all_gather_into_tensor(o_full.flatten(0, 1), o_local)     # 8 KiB per rank, on the compute stream

    def load(s_):
        for k in bufs:
            bufs[k].copy_(x[k][L + s_:L + s_ + 1])
        pos_t.fill_(L + s_)

    flush = torch.empty(256 << 20, dtype=torch.uint8, device=device)
    for s_ in range(3):
        load(s_)
        decode_step()
    barrier()
    _lib.status_for(device).raise_if_set()
    ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(dsteps)]
    for s_ in range(dsteps):
        load(s_)
        flush.zero_()
        ev[s_][0].record()
        decode_step()
        ev[s_][1].record()
    barrier()
    _lib.status_for(device).raise_if_set()
    us = sorted(a.elapsed_time(b) * 1e3 for a, b in ev)
    decode_us = reduce_max(us[len(us) // 2])
    per_pair = 4.0 * dim * group
    return {
        "workload": f"{L}-token layer, GQA {cfg['hq']}q/{cfg['hkv']}kv, head_dim {dim}, {clusters} clusters, budget "
                    f"{cfg['target']} + sink {cfg['sink']} + local window {cfg['local']}, KV heads {cfg['hkv']} split "
                    f"{hkv_l} per GPU, outputs all-gathered with NCCL; then {dsteps} decode steps",
        "scaling": "strong", "n_gpus": world, "kv_heads_per_gpu": hkv_l,
        "prefill_tok_per_s": L / (prefill_ms * 1e-3), "prefill_ms_per_step": prefill_ms, "prefill_steps": steps,
        "attended_pairs_per_step_this_rank": counts[0] + counts[2],
        "prefill_tflops_this_rank": per_pair * (counts[0] + counts[2]) / (prefill_ms * 1e-3) / 1e12,
        "decode_us_per_step": decode_us, "decode_steps": dsteps, "decode_timing": "eager launches incl. the all-gather, "
        "L2 flushed before every step, median, max over ranks",
        "gather_bytes_per_chunk_per_rank": cfg["chunk"] * hq_l * dim * 2,
        "shards_equal_unsharded_layer": same,
    }


# ------------------------------------------------------------------------- CPU baseline
CPU_CONFIG1 = dict(length=8192, hq=8, hkv=2, dim=128, centres=64, unit=64, min_log2=7, target=1024, sink=128,
                   local=512, chunk=1024, decode_steps=32, temperature=0.1, beta=0.25)


def _reference_cpu_functions():
    """The reference's own torch functions that run on a CPU (index build, packing, causal snapshot, query
    router), from an install of the reference under baseline/_ref when one travelled with the tree; None
    otherwise (the CPU restatement then stands in for them too)."""
    ref = ROOT / "baseline" / "_ref"
    if not (ref / "semblo").is_dir():
        return None
    if str(ref) not in sys.path:
        sys.path.append(str(ref))
    try:
        from semblo.vllm_plugin.fused_prefill import CausalSnapshot
        from semblo.vllm_plugin.routing_map import SembloKeyRouter
        from semblo.vllm_plugin.state import ProductPostingIndex
        from semblo.vllm_plugin.trivial_router import trivial_router_vectors
    except Exception:
        return None
    return SimpleNamespace(CausalSnapshot=CausalSnapshot, SembloKeyRouter=SembloKeyRouter,
                           ProductPostingIndex=ProductPostingIndex, trivial_router_vectors=trivial_router_vectors)


def cpu_config1_full(threads=None):
    """The CPU-runnable configuration in full, nothing extrapolated: 8192-token prompt, 8 query / 2 KV heads,
    head_dim 128, fp32, 64-token blocks, budget 1024 + sink 128 + window 512, query chunks of 1024 (so the
    chunks past four budgets take the sparse path), then 32 decode steps.  Index build, packing, snapshot
    and router through the reference's own functions when they are present; the threshold selection and the
    attention bodies (Triton / FlashAttention-only in the reference) through the CPU restatement."""
    from oracle import semblo_oracle as O
    if threads:
        torch.set_num_threads(threads)
    c = CPU_CONFIG1
    L, hq, hkv, dim, chunk = c["length"], c["hq"], c["hkv"], c["dim"], c["chunk"]
    set_env(c)
    data = O.mixture_inputs(length=L + c["decode_steps"], num_q_heads=hq, num_kv_heads=hkv, head_dim=dim,
                            centres=c["centres"], seed=101, dtype=torch.float32)
    ref = _reference_cpu_functions()
    sm = dim ** -0.5
    t0 = time.perf_counter()
    if ref is not None:
        product = ref.SembloKeyRouter(hkv, dim, dim)(data["k_pre"][:L].unsqueeze(0))[0]
        index_r = ref.ProductPostingIndex.build(product, torch.arange(L), num_centroids=0, kmeans_iters=8,
                                                kmeans_sample_size=8192, codebook_seed=0, flat_unit_tokens=c["unit"],
                                                flat_min_clusters_log2=c["min_log2"], page_align=16)
        index_r.pack_prompt_kv(data["k_post"][:L], data["v"][:L])
        index = O.FlatIndex(codebooks=index_r.codebooks, posting_positions=index_r.posting_positions,
                            bucket_indptr=index_r.bucket_indptr, bucket_sizes=index_r.bucket_sizes,
                            inverse_positions=index_r.inverse_positions(), assign=None, prompt_length=L,
                            page_align=16, packed_kv=index_r.packed_kv)
        snap = ref.CausalSnapshot(index_r)
        sizes_at = lambda p: snap.advance(p).clone()
        router = lambda q: ref.trivial_router_vectors(q, 1)
    else:
        index = O.build_flat(O.routing_normalize(data["k_pre"][:L]), unit_tokens=c["unit"],
                             min_clusters_log2=c["min_log2"], kmeans_sample_size=8192, fit_iters=8, seed=0,
                             sink=c["sink"], page_align=16)
        O.pack_prompt_kv(index, data["k_post"][:L], data["v"][:L])
        sizes_at = lambda p: O.causal_sizes_at(index, p)
        router = O.trivial_router_vectors
    t_build = time.perf_counter() - t0
    t0 = time.perf_counter()
    for cs in range(0, L, chunk):
        ce = cs + chunk - 1
        qpos = torch.arange(cs, ce + 1)
        ws = O.chunk_plan(cs, c["target"], c["local"])
        if ws == 0:
            O.dense_causal_attention(data["q_post"][cs:ce + 1], data["k_post"][:ce + 1], data["v"][:ce + 1], qpos, sm,
                                     dtype=torch.float32)
            continue
        sizes = sizes_at(ws - 1)
        vectors = router(data["q_pre"][cs:ce + 1])
        sel = O.select_clusters(vectors, index.codebooks, sizes, temperature=c["temperature"], beta=c["beta"],
                                target_tokens=c["target"], sink=c["sink"])
        O.sparse_chunk_attention_gather(data["q_post"][cs:ce + 1], index, sel, sizes, qpos, data["k_post"][ws:ce + 1],
                                        data["v"][ws:ce + 1], ws, sm, dtype=torch.float32)
    t_attend = time.perf_counter() - t0
    arena = O.make_arena(capacity=L, num_clusters=int(index.bucket_sizes.shape[1]), num_kv_heads=hkv, head_dim=dim,
                         page_align=16, reserve=256, kv_dtype=torch.float32, desc_dtype=index.codebooks.dtype)
    O.arena_adopt(arena, index)
    t0 = time.perf_counter()
    for s_ in range(c["decode_steps"]):
        pos = L + s_
        O.decode_step(arena, q_post=data["q_post"][pos], q_pre=data["q_pre"][pos], pos=pos, k_post=data["k_post"][pos],
                      v=data["v"][pos], temperature=c["temperature"], beta=c["beta"], target_tokens=c["target"],
                      sink=c["sink"], sm_scale=sm)
    t_decode = time.perf_counter() - t0
    return {"workload": "8192-token prompt, GQA 8q/2kv, head_dim 128, fp32, 64-centre mixture, 64-token blocks, budget "
                        "1024 + sink 128 + window 512, query chunk 1024, then 32 decode steps; measured in full",
            "prefill_tok_per_s": L / (t_build + t_attend), "index_build_s": t_build, "attention_s": t_attend,
            "decode_us_per_step": t_decode / c["decode_steps"] * 1e6,
            "index_build_by": "the reference's own torch functions" if ref is not None else "the CPU restatement",
            "cores": threads or torch.get_num_threads()}


def cpu_reference_sample(cfg, threads=None):
    """The reference path on the host cores on a bounded sample of the prefill workload (about 10-20 s of
    CPU work), scaled to tokens per second of the whole 131072-token step: for one of the KV heads the
    normalisation, all eight k-means iterations on the full sample, assignment, layout and packing; 2048
    queries of a dense chunk and 4096 of a sparse chunk, spread over the chunk so the window lengths
    average as in the whole chunk.  Returns (tok/s, text)."""
    from oracle import semblo_oracle as O
    if threads:
        torch.set_num_threads(threads)
    L, hq, hkv, dim = cfg["length"], cfg["hq"], cfg["hkv"], cfg["dim"]
    set_env(cfg)
    t_all = time.perf_counter()
    data = O.mixture_inputs(length=L, num_q_heads=hq // hkv, num_kv_heads=1, head_dim=dim, centres=cfg["centres"], seed=7)
    t0 = time.perf_counter()
    index = O.build_flat(O.routing_normalize(data["k_pre"][:, :1]), unit_tokens=cfg["unit"],
                         min_clusters_log2=cfg["min_log2"], kmeans_sample_size=8192, fit_iters=8, seed=0,
                         sink=cfg["sink"], page_align=16)
    O.pack_prompt_kv(index, data["k_post"][:, :1], data["v"][:, :1])
    t_build = time.perf_counter() - t0
    build_s = hkv * t_build
    g = hq // hkv
    sm = dim ** -0.5
    chunk = cfg["chunk"]
    # a dense chunk: 256 queries spread over the second chunk
    nq_d = 4096
    cs_d = chunk
    pick = torch.arange(0, chunk, chunk // nq_d) + cs_d
    t0 = time.perf_counter()
    O.dense_causal_attention(data["q_post"][pick, :g], data["k_post"][:cs_d + chunk, :1], data["v"][:cs_d + chunk, :1],
                             pick, sm, dtype=torch.float32)
    t_dense = time.perf_counter() - t0
    dense_pairs_sample = float((pick + 1).sum())
    dense_chunks = [c for c in range(0, L, chunk) if O.chunk_plan(c, cfg["target"], cfg["local"]) == 0]
    dense_pairs = sum(float((torch.arange(c, c + chunk) + 1).sum()) for c in dense_chunks)
    dense_s = hkv * t_dense * dense_pairs / dense_pairs_sample
    # two sparse chunks (an early and a late one), every query of each
    nq_s = chunk
    sparse_at = (5 * chunk, 13 * chunk)
    t_sparse = 0.0
    for cs in sparse_at:
        ws = cs - cfg["local"]
        picks = torch.arange(0, chunk, chunk // nq_s) + cs
        t0 = time.perf_counter()
        sizes = O.causal_sizes_at(index, ws - 1)
        vectors = O.trivial_router_vectors(data["q_pre"][picks, :g])
        sel = O.select_clusters(vectors, index.codebooks, sizes, temperature=cfg["temperature"], beta=cfg["beta"],
                                target_tokens=cfg["target"], sink=cfg["sink"])
        O.sparse_chunk_attention_gather(data["q_post"][picks, :g], index, sel, sizes, picks,
                                        data["k_post"][ws:cs + chunk, :1], data["v"][ws:cs + chunk, :1], ws, sm)
        t_sparse += time.perf_counter() - t0
    t_sparse /= len(sparse_at)
    n_sparse = (L // chunk) - len(dense_chunks)
    sparse_s = hkv * n_sparse * (chunk / nq_s) * t_sparse
    total = build_s + dense_s + sparse_s
    text = (f"1 of {hkv} KV heads in full for the index (normalise, 8 k-means iterations, assignment, layout, pack: "
            f"{t_build:.1f}s), {nq_d} queries spread over a dense chunk ({t_dense:.1f}s) and all {nq_s} queries of two "
            f"sparse chunks ({t_sparse:.1f}s each); scaled to the whole step (build {build_s:.1f}s + dense {dense_s:.1f}s + sparse "
            f"{sparse_s:.1f}s); sample wall {time.perf_counter() - t_all:.1f}s")
    return L / total, text


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    cfg = PREFILL
    threads = os.cpu_count() or 1
    values = []
    text = ""
    budget_s = 240.0                                  # the whole run stays within a few minutes
    t_start = time.perf_counter()
    for i in range(args.warmup + args.steps):
        if i > 0 and time.perf_counter() - t_start > budget_s * i / (i + 1):
            break
        v, text = cpu_reference_sample(cfg, threads)
        if i >= min(args.warmup, 1) or not values:
            values.append(v)
    value = sum(values) / len(values)
    config1 = cpu_config1_full(threads)
    line = {"impl": "reference", "metric": "sparse_prefill_tok_per_s", "value": value, "unit": "tok/s",
            "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": cfg["length"] / value * 1e3, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "bf16 values, fp32 math", "data": "synthetic",
            "config": workload_config(1),
            "cpu_baseline": {"value": value, "unit": "tok/s", "cores": threads, "kind": "port",
                             "sample": text + f"; {len(values)} sample(s) averaged", "config1_full": config1},
            "e2e": {"value": value, "unit": "tok/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line))


def workload_config(world):
    c = PREFILL
    return {"workload": "single-layer block-sparse prefill, 131072-token prompt, GQA 16q/4kv, head_dim 256, bf16, "
                        "partial RoPE 25%, 256-centre mixture keys, 64-token blocks (2048 clusters), budget 4096 + "
                        "sink 128 + local window 512, query chunk 8192, 16-token pages in a random permutation",
            "tokens": c["length"], "kv_heads_per_gpu": c["hkv"], "parallelism": f"head-parallel x{world}",
            "l2": "inputs larger than L2 (K/V 0.8 GB, Q 2.1 GB per step)",
            "streams": "index build and chunk loop on a high-priority stream; dense-prefix and window launches "
                       "issued ahead on a second stream (they need no index)"}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=8)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200")
    ap.add_argument("--no-decode", action="store_true")
    ap.add_argument("--no-cpu", action="store_true")
    ap.add_argument("--no-head-sharded", action="store_true")
    ap.add_argument("--head-sharded-only", action="store_true",
                    help="run only the head-sharded configuration (optionally with --length) and print its record")
    ap.add_argument("--length", type=int, default=0, help="override the prompt length (profiling on a small case)")
    ap.add_argument("--decode-only", action="store_true",
                    help="run only the decode measurement and print its record (profiling the decode kernels)")
    ap.add_argument("--select-only", type=int, default=0, metavar="CLUSTERS",
                    help="run only one chunk's selection launch at this cluster count (profiling the kernel)")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
        return
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=device)
    from semblo_b200 import _lib
    _lib.lib()
    pk = peaks()
    if args.decode_only:
        print(json.dumps(decode_measure(device, pk)))
        return
    if args.select_only:
        print(json.dumps(select_measure(device, clusters=args.select_only, heads=8 if args.select_only >= 16384 else 4)))
        return
    if args.head_sharded_only:
        rec = head_sharded_measure(device, rank, world, pk, length=args.length or None)
        if rank == 0:
            print(json.dumps(rec))
        if world > 1:
            import torch.distributed as dist
            dist.barrier()
            dist.destroy_process_group()
        return
    cfg = dict(PREFILL)
    if args.length:
        cfg["length"] = args.length
    set_env(cfg)
    x = mixture_inputs_device(cfg, 2000, device, heads=range(rank * cfg["hkv"], (rank + 1) * cfg["hkv"]))
    torch.cuda.synchronize()
    # The step's dependent chain (index build, then the chunk loop) runs on a high-priority stream; the
    # launches that need no index run ahead on a stream of normal priority, so their CTAs take the
    # multiprocessors only where the chain leaves them idle.
    torch.cuda.set_stream(torch.cuda.Stream(device=device, priority=-1))
    step = PrefillStep(cfg, device, world)
    step.prepare()
    out = torch.empty(cfg["length"], cfg["hq"], cfg["dim"], dtype=torch.bfloat16, device=device)

    def barrier():
        if world > 1:
            import torch.distributed as dist
            dist.barrier()
        torch.cuda.synchronize()

    # the clock sampler starts before the warm-up: the start-up of its nvidia-smi process (a second
    # client of the driver) then falls into the untimed steps; it samples until the timed region ends
    sampler = ClockSampler(local_rank)
    sampler.start()
    for _ in range(args.warmup):
        step.run(x, out)
    barrier()
    _lib.status_for(device).raise_if_set()
    # ---- device-resident timing
    _lib.CALLS.clear()
    step.attended.zero_()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    gc.collect()
    gc.disable()                     # no collector pause inside the timed region
    barrier()
    e0.record()
    marks = [e0]
    index = None
    for _ in range(args.steps):
        index = None                 # the previous step's index is dropped before the next one is built
        index = step.run(x, out)
        marks.append(torch.cuda.Event(enable_timing=True))
        marks[-1].record()
    e1.record()
    barrier()
    gc.enable()
    ms = e0.elapsed_time(e1) / args.steps
    step_ms = [round(marks[i].elapsed_time(marks[i + 1]), 2) for i in range(args.steps)]
    _lib.status_for(device).raise_if_set()
    calls = dict(_lib.CALLS)
    clusters = int(index.num_buckets)
    launches = kernel_launches(calls, clusters, int(cfg["chunk"])) // args.steps
    counts = [int(v) // args.steps for v in step.attended.tolist()]
    attended = counts[0] + counts[2]                       # dense prefix + windows, selected clusters
    sparse_pairs, gathered_rows = counts[2], counts[3]
    # ---- the attention launches one after the other on one stream, for the per-kernel rooflines: in the
    # timed steps above the index-free launches overlap the index build and CUDA events around a single
    # launch would time its neighbours too
    split_steps = 2
    step.time_attention = True
    step.attn_events = []
    e2, e3 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    e2.record()
    for _ in range(split_steps):
        step.run(x, out)
    e3.record()
    barrier()
    serial_ms = e2.elapsed_time(e3) / split_steps
    evs = step.attn_events
    attn_ms = window_ms = gather_ms = dense_ms = 0.0
    for i, (phase, ev) in enumerate(evs):
        if phase == "start":
            nxt = evs[i + 1]
            if nxt[0] == "stop":
                dense_ms += ev.elapsed_time(nxt[1])
            else:
                window_ms += ev.elapsed_time(nxt[1])
                gather_ms += nxt[1].elapsed_time(evs[i + 2][1])
    dense_ms, window_ms, gather_ms = dense_ms / split_steps, window_ms / split_steps, gather_ms / split_steps
    attn_ms = dense_ms + window_ms + gather_ms
    step.time_attention = False
    g = cfg["hq"] // cfg["hkv"]
    flops = 4.0 * cfg["dim"] * g * attended
    if world > 1:
        import torch.distributed as dist
        t = torch.tensor([ms], device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    # ---- end to end: host buffers in, host result out, through the same public entry points
    host = {k: v.cpu().pin_memory() for k, v in x.items()}
    out_host = torch.empty(out.shape, dtype=out.dtype).pin_memory()
    dev_in = {k: torch.empty_like(v) for k, v in x.items()}

    # Host buffers in, host result out, every step.  Keys and values go first (the index build needs
    # all of them); the queries follow chunk by chunk on a copy stream while earlier chunks compute, and
    # every chunk's output leaves on a third stream as soon as it is written.  Two sets of device input
    # buffers alternate, so the upload of the next step's inputs runs behind the current step's compute.
    copy_s, d2h_s = torch.cuda.Stream(), torch.cuda.Stream()
    L_, chunk_ = cfg["length"], cfg["chunk"]
    dev_sets = [dev_in, {k: torch.empty_like(v) for k, v in dev_in.items()}]

    def upload(buf):
        """Enqueue one step's host-to-device copies on the copy stream; returns its events."""
        q_ready = {}
        with torch.cuda.stream(copy_s):
            for k in ("k_pre", "k_post", "v"):
                buf[k].copy_(host[k], non_blocking=True)
            kv_ready = torch.cuda.Event()
            kv_ready.record(copy_s)
            for cs in range(0, L_, chunk_):
                for k in ("q_pre", "q_post"):
                    buf[k][cs:cs + chunk_].copy_(host[k][cs:cs + chunk_], non_blocking=True)
                q_ready[cs] = torch.cuda.Event()
                q_ready[cs].record(copy_s)
        return kv_ready, q_ready

    def e2e_steps(n):
        cur = torch.cuda.current_stream()
        copy_s.wait_stream(cur)
        pending = upload(dev_sets[0])
        compute_done = [None, None]
        for i in range(n):
            buf = dev_sets[i % 2]
            kv_ready, q_ready = pending
            if i + 1 < n:
                if compute_done[(i + 1) % 2] is not None:
                    copy_s.wait_event(compute_done[(i + 1) % 2])     # the step that last read that set is over
                pending = upload(dev_sets[(i + 1) % 2])
            cur.wait_event(kv_ready)

            def before(cs, ce, q_ready=q_ready):
                torch.cuda.current_stream().wait_event(q_ready[cs])     # the chunk loop's stream or the windows'

            def after(cs, ce):
                done = torch.cuda.Event()
                done.record(cur)
                d2h_s.wait_event(done)
                with torch.cuda.stream(d2h_s):
                    out_host[cs:ce + 1].copy_(out[cs:ce + 1], non_blocking=True)

            step.run(buf, out, before_chunk=before, after_chunk=after)
            compute_done[i % 2] = torch.cuda.Event()
            compute_done[i % 2].record(cur)
            cur.wait_stream(d2h_s)                   # a step ends when its result is on the host
        return None

    step.time_attention = False
    e2e_steps(1)
    barrier()
    gc.collect()
    gc.disable()
    e0.record()
    e2e_steps(args.steps)
    e1.record()
    barrier()
    gc.enable()
    e2e_ms = e0.elapsed_time(e1) / args.steps
    clocks = sampler.stop()          # sampled through both timed regions (device-resident and end to end)
    if world > 1:
        import torch.distributed as dist
        t = torch.tensor([e2e_ms], device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_ms = float(t.item())
    h2d = sum(v.numel() * v.element_size() for v in host.values())
    d2h = out_host.numel() * out_host.element_size()
    del host, dev_in, dev_sets, out_host
    head_sharded = None
    if not args.length and not args.no_head_sharded:
        del x, out
        x = out = None
        torch.cuda.empty_cache()
        try:
            head_sharded = head_sharded_measure(device, rank, world, pk)
        except Exception as exc:                      # keep the headline if the second workload fails
            head_sharded = {"error": repr(exc)}
        set_env(cfg)
    if rank != 0:
        import torch.distributed as dist
        dist.barrier()                                # rank 0 joins it after printing the line
        dist.destroy_process_group()
        return
    tokens = cfg["length"] * world
    # attended pairs by launch kind: dense-prefix chunks count their full causal triangle, the window
    # launches of the sparse chunks the rest of counter 0, the sparse launches their own counter
    cap = 4 * cfg["target"]
    dense_pairs = sum((cs + min(cfg["length"], cs + cfg["chunk"]) + 1) * (min(cfg["length"], cs + cfg["chunk"]) - cs) // 2
                      for cs in range(0, cfg["length"], cfg["chunk"]) if cs <= cap) * cfg["hkv"]
    window_pairs = counts[0] - dense_pairs
    per_pair = 4.0 * cfg["dim"] * g
    dims = f"<{cfg['dim']},{g}>"

    def kern(name, pairs, ms):
        tf = per_pair * pairs / (ms * 1e-3) / 1e12 if ms > 0 else 0.0
        return {"kernel": name, "attended_pairs_per_step": pairs, "flops_per_step": per_pair * pairs,
                "ms_per_step": ms, "achieved": tf, "frac": tf / pk["tensor"]}

    sparse = kern("sparse_gather_prefill_kernel" + dims, sparse_pairs, gather_ms)
    roofline = {
        "bound": "tensor", "kernel": sparse["kernel"], "achieved": sparse["achieved"], "peak": pk["tensor"],
        "unit": "TFLOP/s", "frac": sparse["frac"],
        "traffic": DRAM_TRAFFIC_PER_LAUNCH.get((sparse["kernel"], cfg["length"])),
        "peak_source": pk["source"] + " (sustained bf16 GEMM)",
        "what": "selected-cluster pairs x 4 D G flop / summed CUDA-event time of the sparse launches",
        "gathered_rows_per_step": gathered_rows,
        "executed_flops_per_step": 4.0 * cfg["dim"] * 128 * gathered_rows,
        "launches": {"dense_prefix": kern("window_prefill_kernel" + dims, dense_pairs, dense_ms),
                     "window": kern("window_prefill_kernel" + dims, window_pairs, window_ms),
                     "sparse": sparse},
        "all_attention": {"attended_pairs_per_step": attended, "flops_per_step": flops, "ms_per_step": attn_ms,
                          "achieved": flops / (attn_ms * 1e-3) / 1e12,
                          "frac": flops / (attn_ms * 1e-3) / 1e12 / pk["tensor"]},
        "step": {"flops_per_step": flops, "ms_per_step": ms, "frac": flops / (ms * 1e-3) / 1e12 / pk["tensor"]},
        "launch_timing": f"{split_steps} extra steps with every launch in order on one stream ({serial_ms:.2f} ms per "
                         "step): in the timed steps the dense-prefix and window launches run ahead on a stream of "
                         "their own and overlap the index build",
    }
    line = {
        "metric": "sparse_prefill_tok_per_s", "value": tokens / (ms * 1e-3), "unit": "tok/s", "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "step_ms": step_ms,
        "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "config": workload_config(world),
        "clocks": clocks, "gpu_launches": launches,
        "e2e": {"value": tokens / (e2e_ms * 1e-3), "unit": "tok/s", "h2d_bytes_per_step": h2d,
                "d2h_bytes_per_step": d2h, "ms_per_step": e2e_ms},
        "roofline": roofline,
    }
    if head_sharded is not None:
        line["head_sharded"] = head_sharded
    if world == 1 and not args.no_decode and not args.length:
        del x, out, step, index
        torch.cuda.empty_cache()
        try:
            line["decode"] = decode_measure(device, pk)
        except Exception as exc:                      # keep the headline if the second workload fails
            line["decode"] = {"error": repr(exc)}
    if world == 1 and not args.no_cpu:
        v, text = cpu_reference_sample(PREFILL, os.cpu_count() or 1)
        line["cpu_baseline"] = {"value": v, "unit": "tok/s", "cores": os.cpu_count() or 1, "kind": "port", "sample": text,
                                "config1_full": cpu_config1_full(os.cpu_count() or 1)}
    if rank == 0:
        print(json.dumps(line))
    if world > 1:
        import torch.distributed as dist
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
