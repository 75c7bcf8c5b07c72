// Block-sparse decode step over the decode arena: suffix write, query routing,
// centroid scoring, threshold selection with CSR emission, split-KV gather attention
// over the selected cluster rows plus the exact generated suffix, and the LSE merge.
//
// The step is HBM-bound (codebook read + gathered K/V rows), so the kernels are
// plain coalesced 16-byte loads spread over the whole GPU:
//   decode_score_kernel   grid [Hkv, blocks]: suffix write (block 0,0), router, logits of a
//                         slice of the codebook and the slice's (max, sum-exp) per head
//   decode_penalise_kernel grid [Hkv, C / 256]: log-sum-exp, cluster probabilities, penalised score
//   decode_select_kernel  grid [Hkv]: bisection, CSR (start, len, cum) and the flat list of
//                         selected rows
//   decode_attend_kernel  grid [Hkv, splits]: each half-warp streams whole K/V rows
//                         (16 lanes x 16 B = one 256-B request per row and tensor); the last
//                         CTA of a head merges the splits and writes the output
// No host reads, no allocations, fixed addresses: the step can be captured in a CUDA graph.
//
// Reference behaviour restated here:
//   semblo/vllm_plugin/fused_decode.py:38-78     suffix write through the block table
//   semblo/vllm_plugin/trivial_router.py:23-45   query routing vector
//   semblo/vllm_plugin/fused_decode.py:80-199    selection with the sink rule, CSR in cluster order
//   semblo/vllm_plugin/fused_decode.py:201-358   attention over CSR rows + suffix, merge
#include <algorithm>
#include <climits>

#include "../../include/semblo_b200.h"
#include "host_common.h"
#include "sm100.cuh"

using semblo::ceil_div;

namespace {

constexpr float NEG_BIG = -3.4e38f;
constexpr float LOG2E = 1.4426950408889634f;
constexpr float LN2 = 0.6931471805599453f;
constexpr int MAX_G = 8;
constexpr int SCORE_BLOCKS_TARGET = 296;     // 2 CTAs per SM

struct DecodeArgs {
  int num_q_heads, num_kv_heads, head_dim, num_clusters, group;
  // inputs of the step
  const __nv_bfloat16 *q_post, *q_pre, *k_post, *v_new, *k_pre;
  const void* positions;
  int pos_is_int64;
  // arena
  const __nv_bfloat16* codebooks;
  const int32_t *sizes, *indptr, *posting;
  const __nv_bfloat16* packed_kv;
  int64_t packed_width;
  __nv_bfloat16* suffix_kv;
  __nv_bfloat16* suffix_kpre;
  const int32_t* suffix_table;
  int suffix_blocks, suffix_block, table_len;
  const int32_t* prompt_length;
  // parameters
  float scale_log2_router, beta, sm_scale_log2;
  int target_tokens, sink_tokens, iters, num_splits, score_blocks;
  // workspace
  float* ws_logit;      // [Hkv, G, C]
  float* ws_ml;         // [Hkv, score_blocks, G, 2]
  float* ws_score;      // [Hkv, C]
  int32_t *rstart, *rlen, *rcum;   // [Hkv, C]
  int32_t *rcount, *rtokens;       // [Hkv]
  int32_t* rows;        // [Hkv, packed_width]
  float* pacc;          // [Hq, splits, D]
  float* pml;           // [Hq, splits, 2]
  int32_t* tickets;     // [Hkv]
  __nv_bfloat16* vectors;   // [Hq, D] routing vectors (kept for inspection)
  __nv_bfloat16* out;
  int* status;
};

__device__ __forceinline__ long long load_pos(const DecodeArgs& a) {
  return a.pos_is_int64 ? *reinterpret_cast<const long long*>(a.positions)
                        : (long long)*reinterpret_cast<const int*>(a.positions);
}

__device__ __forceinline__ double warp_sumd(double v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// ------------------------------------------------------------------ score
// Sum of G per-lane values over the LPR lanes that share a codebook row, as a reduce-scatter:
// while more than one value is left, each exchange step halves the values a lane carries, so
// G = 4 over 32 lanes costs 6 shuffles instead of 20.  On return v[0] of lane l is the total
// of head head_of_lane(l).
template <int G, int LPR>
__device__ __forceinline__ void reduce_heads(float (&v)[G], int lane_in_row) {
  int n = G;
#pragma unroll
  for (int o = LPR / 2; o > 0; o >>= 1) {
    if (n > 1) {
      const bool upper = (lane_in_row & o) != 0;
      const int hn = n / 2;
#pragma unroll
      for (int i = 0; i < G / 2; ++i) {
        if (i < hn) {
          const float send = upper ? v[i] : v[i + hn];          // the half this lane gives away
          const float keep = upper ? v[i + hn] : v[i];
          v[i] = keep + __shfl_xor_sync(0xffffffffu, send, o);
        }
      }
      n = hn;
    } else {
      v[0] += __shfl_xor_sync(0xffffffffu, v[0], o);
    }
  }
}
// The head whose total reduce_heads leaves in a lane: one bit per halving step, highest first.
template <int G, int LPR>
__device__ __forceinline__ int head_of_lane(int lane_in_row) {
  int t = 0, n = G;
#pragma unroll
  for (int o = LPR / 2; o > 0 && n > 1; o >>= 1) {
    n /= 2;
    if (lane_in_row & o) t += n;
  }
  return t;
}

template <int D, int G>
__global__ void __launch_bounds__(256, 2)
decode_score_kernel(const DecodeArgs a) {
  __shared__ float qv[G * D];                        // routing vectors as fp32
  __shared__ float red[8][G][2];
  const int h = blockIdx.x, blk = blockIdx.y;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int C = a.num_clusters;

  if (h == 0 && blk == 0 && a.k_post != nullptr) {
    // the token's K/V (and pre-RoPE key) into the suffix store
    const long long pos = load_pos(a);
    const long long block = pos / a.suffix_block;
    if (block >= 0 && block < a.table_len) {
      const long long phys = a.suffix_table[block];
      const long long off = pos - block * a.suffix_block;
      const int64_t plane = (int64_t)a.suffix_blocks * a.suffix_block * a.num_kv_heads * D;
      const int64_t dst = (phys * a.suffix_block + off) * a.num_kv_heads * D;
      for (int i = threadIdx.x; i < a.num_kv_heads * D; i += blockDim.x) {
        a.suffix_kv[dst + i] = a.k_post[i];
        a.suffix_kv[plane + dst + i] = a.v_new[i];
        if (a.suffix_kpre && a.k_pre) a.suffix_kpre[dst + i] = a.k_pre[i];
      }
    } else if (threadIdx.x == 0) {
      atomicCAS(a.status, 0, sm100::STATUS_OVERFLOW);
    }
  }
  // A row (both halves of the codebook) is read by LPR lanes, 16 bytes each: lanes [0, LPR/2)
  // take half 0, the rest half 1.  The first SU rows of every lane group are requested before
  // anything else, so the codebook is on its way while the router runs.
  constexpr int HALF = D / 2;
  constexpr int LPR = D / 8;                          // 32 (D = 256) or 16 (D = 128)
  constexpr int RPW = 32 / LPR;                       // rows per warp and step
  constexpr int SU = 16;
  const int sub = lane / LPR, l_in = lane % LPR;
  const int f = l_in / (LPR / 2), chunk = l_in % (LPR / 2);
  const int per_block = (int)ceil_div(C, gridDim.y);
  const int c_lo = blk * per_block, c_hi = min(C, c_lo + per_block);
  const __nv_bfloat16* cb = a.codebooks + ((int64_t)(h * 2 + f) * C) * HALF + chunk * 8;
  uint4 raw[SU];
  auto fetch = [&](int cw) {
#pragma unroll
    for (int u = 0; u < SU; ++u) {
      const int c = cw + u * 8 * RPW + sub;
      raw[u] = make_uint4(0, 0, 0, 0);
      if (c < c_hi) raw[u] = __ldg(reinterpret_cast<const uint4*>(cb + (int64_t)c * HALF));
    }
  };
  fetch(c_lo + warp * RPW);

  // router: normalise in fp32, round to bf16, normalise again, round again
  for (int t = warp; t < G; t += 8) {
    const __nv_bfloat16* src = a.q_pre + (int64_t)(h * G + t) * D;
    float v[D / 32];
    double ss = 0.0;
#pragma unroll
    for (int i = 0; i < D / 32; ++i) {
      v[i] = __bfloat162float(src[lane + 32 * i]);
      ss += (double)v[i] * v[i];
    }
    const float n1 = fmaxf((float)sqrt(warp_sumd(ss)), 1e-12f);
    double ss2 = 0.0;
#pragma unroll
    for (int i = 0; i < D / 32; ++i) {
      v[i] = __bfloat162float(__float2bfloat16_rn(v[i] / n1));
      ss2 += (double)v[i] * v[i];
    }
    const float n2 = fmaxf((float)sqrt(warp_sumd(ss2)), 1e-12f);
#pragma unroll
    for (int i = 0; i < D / 32; ++i) {
      const int d = lane + 32 * i;
      const __nv_bfloat16 r = __float2bfloat16_rn(v[i] / n2);
      qv[t * D + d] = __bfloat162float(r);
      if (blk == 0) a.vectors[(int64_t)(h * G + t) * D + d] = r;
    }
  }
  __syncthreads();

  const int d0 = f * HALF + chunk * 8;
  float qreg[G][8];
#pragma unroll
  for (int t = 0; t < G; ++t)
#pragma unroll
    for (int e = 0; e < 8; ++e) qreg[t][e] = qv[t * D + d0 + e];
  // after the reduction a lane keeps the logits of one head only
  const int my_t = head_of_lane<G, LPR>(l_in);
  const bool writer = (l_in & (LPR / G - 1)) == 0;    // one lane per (row, head)
  float m_run = -INFINITY, l_run = 0.f;
  float* logit_out = a.ws_logit + ((int64_t)h * G + my_t) * C;
  for (int cw = c_lo + warp * RPW; cw < c_hi; cw += 8 * RPW * SU) {
    if (cw != c_lo + warp * RPW) fetch(cw);
#pragma unroll
    for (int u = 0; u < SU; ++u) {
      const int c = cw + u * 8 * RPW + sub;
      if (cw + u * 8 * RPW >= c_hi) break;           // warp-uniform
      const __nv_bfloat162* p2 = reinterpret_cast<const __nv_bfloat162*>(&raw[u]);
      float x[8];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 f2 = __bfloat1622float2(p2[e]);
        x[2 * e] = f2.x;
        x[2 * e + 1] = f2.y;
      }
      float dot[G];
#pragma unroll
      for (int t = 0; t < G; ++t) {
        dot[t] = 0.f;
#pragma unroll
        for (int e = 0; e < 8; ++e) dot[t] = fmaf(qreg[t][e], x[e], dot[t]);
      }
      reduce_heads<G, LPR>(dot, l_in);
      if (c < c_hi) {
        const float s2 = dot[0] * a.scale_log2_router;
        if (writer) logit_out[c] = s2;
        const float mx = fmaxf(m_run, s2);
        l_run = l_run * sm100::fast_exp2(m_run - mx) + sm100::fast_exp2(s2 - mx);
        m_run = mx;
      }
    }
  }
  // combine the (max, sum) of the block: the writer lanes of every sub-row hold a head's pair
  auto merge = [](float& m, float& l, float m_o, float l_o) {
    const float mx = fmaxf(m, m_o);
    l = (m == -INFINITY ? 0.f : l * sm100::fast_exp2(m - mx)) + (m_o == -INFINITY ? 0.f : l_o * sm100::fast_exp2(m_o - mx));
    m = mx;
  };
  if (RPW == 2) merge(m_run, l_run, __shfl_xor_sync(0xffffffffu, m_run, 16), __shfl_xor_sync(0xffffffffu, l_run, 16));
  if (sub == 0 && writer) { red[warp][my_t][0] = m_run; red[warp][my_t][1] = l_run; }
  __syncthreads();
  if (threadIdx.x < G) {
    const int t = threadIdx.x;
    float m = -INFINITY, l = 0.f;
    for (int w = 0; w < 8; ++w) merge(m, l, red[w][t][0], red[w][t][1]);
    float* dst = a.ws_ml + (((int64_t)h * gridDim.y + blk) * G + t) * 2;
    dst[0] = m;
    dst[1] = l;
  }
}

// ------------------------------------------------------------------ select
constexpr int SEL_THREADS = 1024;
constexpr int SEL_MAX_PER = 16;        // clusters per thread: C <= 16384
constexpr int SEL_CSR_SMEM = 2048;     // selected clusters whose (start, cum) are searched in shared memory
constexpr int PEN_THREADS = 256;

// Penalised score of every cluster: grid [Hkv, C / 256], one cluster per thread.  The head's
// log-sum-exp is rebuilt from the score kernel's block partials by one warp per query head
// (the partials of a head are read in parallel and merged with shuffles).
__global__ void __launch_bounds__(PEN_THREADS)
decode_penalise_kernel(const DecodeArgs a) {
  __shared__ float lse2[MAX_G];
  const int h = blockIdx.x;
  const int C = a.num_clusters, G = a.group;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (warp < G) {
    const int t = warp;
    float m = -INFINITY, l = 0.f;
    for (int b = lane; b < a.score_blocks; b += 32) {
      const float2 ml = __ldcg(reinterpret_cast<const float2*>(a.ws_ml + (((int64_t)h * a.score_blocks + b) * G + t) * 2));
      const float mx = fmaxf(m, ml.x);
      l = (m == -INFINITY ? 0.f : l * exp2f(m - mx)) + (ml.x == -INFINITY ? 0.f : ml.y * exp2f(ml.x - mx));
      m = mx;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float m_o = __shfl_xor_sync(0xffffffffu, m, o), l_o = __shfl_xor_sync(0xffffffffu, l, o);
      const float mx = fmaxf(m, m_o);
      l = (m == -INFINITY ? 0.f : l * exp2f(m - mx)) + (m_o == -INFINITY ? 0.f : l_o * exp2f(m_o - mx));
      m = mx;
    }
    if (lane == 0) lse2[t] = m + log2f(l);
  }
  __syncthreads();
  const int c = blockIdx.y * PEN_THREADS + threadIdx.x;
  if (c >= C) return;
  float lg[MAX_G];
#pragma unroll
  for (int t = 0; t < MAX_G; ++t)
    if (t < G) lg[t] = __ldcg(a.ws_logit + ((int64_t)h * G + t) * C + c);
  const int size = __ldg(a.sizes + (int64_t)h * C + c);
  float prob = 0.f;
#pragma unroll
  for (int t = 0; t < MAX_G; ++t)
    if (t < G) prob += exp2f(lg[t] - lse2[t]);
  const float n = (a.sink_tokens > 0 && c == 0) ? 0.f : (float)size;
  float sc = log2f(fmaxf(prob, 1e-38f)) * LN2;
  if (a.beta != 0.f) sc -= a.beta * logf(1.0f + n);
  a.ws_score[(int64_t)h * C + c] = n > 0.f ? sc : NEG_BIG;
}

// Threshold bisection, selection, CSR in cluster order and the flat row list: grid [Hkv].
// A thread owns PER consecutive clusters (PER * T >= C, C a multiple of 4).  Few threads with
// many clusters each: the per-warp cost of the 16 block-wide sums dominates otherwise.
template <int PER, int T>
__global__ void __launch_bounds__(T)
decode_select_kernel(const DecodeArgs a) {
  constexpr int NW = T / 32;
  __shared__ float fred[2][32];
  __shared__ int isum[2][32];
  __shared__ int wsum_a[32], wsum_b[32];
  __shared__ int csr_start[SEL_CSR_SMEM], csr_cum[SEL_CSR_SMEM];
  const int h = blockIdx.x;
  const int C = a.num_clusters;
  const int lane_s = threadIdx.x & 31, warp_s = threadIdx.x >> 5;
  const int c0 = threadIdx.x * PER;
  const bool has_sink = a.sink_tokens > 0;
  float score[PER];
  int real[PER], seen[PER];          // cluster size, and the size the budget sees (0 for the sink cluster)
#pragma unroll
  for (int i4 = 0; i4 < PER; i4 += 4) {
    float4 sc = make_float4(NEG_BIG, NEG_BIG, NEG_BIG, NEG_BIG);
    int4 sz = make_int4(0, 0, 0, 0);
    if (c0 + i4 < C) {
      sc = __ldcg(reinterpret_cast<const float4*>(a.ws_score + (int64_t)h * C + c0 + i4));
      sz = __ldg(reinterpret_cast<const int4*>(a.sizes + (int64_t)h * C + c0 + i4));
    }
    score[i4] = sc.x; score[i4 + 1] = sc.y; score[i4 + 2] = sc.z; score[i4 + 3] = sc.w;
    real[i4] = sz.x; real[i4 + 1] = sz.y; real[i4 + 2] = sz.z; real[i4 + 3] = sz.w;
  }
  float mx = -INFINITY, mn = 3.4e38f;
  int tot = 0;
#pragma unroll
  for (int i = 0; i < PER; ++i) {
    seen[i] = (has_sink && c0 + i == 0) ? 0 : real[i];
    if (c0 + i < C) mx = fmaxf(mx, score[i]);
    if (seen[i] > 0) { mn = fminf(mn, score[i]); tot += seen[i]; }
  }
  // block reductions with one barrier each: warp results go to one of two buffers (alternating,
  // so a fast warp's next write cannot overtake a slow warp's read), then every warp folds the 32
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    mn = fminf(mn, __shfl_xor_sync(0xffffffffu, mn, o));
  }
  tot = __reduce_add_sync(0xffffffffu, tot);
  if (lane_s == 0) { fred[0][warp_s] = mx; fred[1][warp_s] = mn; isum[1][warp_s] = tot; }
  __syncthreads();
  mx = lane_s < NW ? fred[0][lane_s] : -INFINITY;
  mn = lane_s < NW ? fred[1][lane_s] : 3.4e38f;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    mn = fminf(mn, __shfl_xor_sync(0xffffffffu, mn, o));
  }
  const int budget = max(a.target_tokens - a.sink_tokens, 0);
  const bool all_fit = __reduce_add_sync(0xffffffffu, lane_s < NW ? isum[1][lane_s] : 0) < budget;
  float hi = mx + 1e-6f;
  float lo = fminf(mn - 1e-6f, hi - 1e-5f);
  for (int it = 0; it < a.iters; ++it) {
    const float mid = (lo + hi) * 0.5f;
    int above = 0;
#pragma unroll
    for (int i = 0; i < PER; ++i) above += score[i] >= mid ? seen[i] : 0;
    above = __reduce_add_sync(0xffffffffu, above);
    if (lane_s == 0) isum[it & 1][warp_s] = above;
    __syncthreads();
    above = __reduce_add_sync(0xffffffffu, lane_s < NW ? isum[it & 1][lane_s] : 0);
    const bool reach = above >= budget;
    lo = reach ? mid : lo;
    hi = reach ? hi : mid;
  }
  const float theta = all_fit ? NEG_BIG : lo;
  // selection flags, CSR positions (block scan over threads; clusters of a thread are consecutive)
  int n_sel = 0, n_tok = 0;
  unsigned sel_bits = 0;
#pragma unroll
  for (int i = 0; i < PER; ++i) {
    const int c = c0 + i;
    const bool is_sink = has_sink && c == 0;
    const bool s = c < C && ((seen[i] > 0 && score[i] >= theta) || (is_sink && real[i] > 0));
    sel_bits |= s ? (1u << i) : 0u;
    n_sel += s;
    n_tok += s ? real[i] : 0;
  }
  // block-wide exclusive scan of (clusters, tokens): warp scans, then a scan of the warp totals
  int inc_a = n_sel, inc_b = n_tok;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const int va = __shfl_up_sync(0xffffffffu, inc_a, o), vb = __shfl_up_sync(0xffffffffu, inc_b, o);
    if (lane_s >= o) { inc_a += va; inc_b += vb; }
  }
  if (lane_s == 31) { wsum_a[warp_s] = inc_a; wsum_b[warp_s] = inc_b; }
  __syncthreads();
  int wa = lane_s < NW ? wsum_a[lane_s] : 0, wb = lane_s < NW ? wsum_b[lane_s] : 0;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const int va = __shfl_up_sync(0xffffffffu, wa, o), vb = __shfl_up_sync(0xffffffffu, wb, o);
    if (lane_s >= o) { wa += va; wb += vb; }
  }
  const int total_sel = __shfl_sync(0xffffffffu, wa, NW - 1), total_tok = __shfl_sync(0xffffffffu, wb, NW - 1);
  const int base_a = __shfl_sync(0xffffffffu, wa, warp_s) - wsum_a[warp_s];
  const int base_b = __shfl_sync(0xffffffffu, wb, warp_s) - wsum_b[warp_s];
  int pos = base_a + inc_a - n_sel, cum = base_b + inc_b - n_tok;
  int32_t* rs = a.rstart + (int64_t)h * C;
  int32_t* rl = a.rlen + (int64_t)h * C;
  int32_t* rc = a.rcum + (int64_t)h * C;
  int starts[PER];
#pragma unroll
  for (int i = 0; i < PER; ++i)
    starts[i] = ((sel_bits >> i) & 1) ? __ldg(a.indptr + (int64_t)h * (C + 1) + c0 + i) : 0;
#pragma unroll
  for (int i = 0; i < PER; ++i) {
    if ((sel_bits >> i) & 1) {
      rs[pos] = starts[i];
      rl[pos] = real[i];
      rc[pos] = cum;
      if (pos < SEL_CSR_SMEM) { csr_start[pos] = starts[i]; csr_cum[pos] = cum; }
      ++pos;
      cum += real[i];
    }
  }
  if (threadIdx.x == 0) {
    a.rcount[h] = total_sel;
    a.rtokens[h] = total_tok;
    if (total_tok > a.packed_width) atomicCAS(a.status, 0, sm100::STATUS_OVERFLOW);
  }
  __threadfence_block();
  __syncthreads();
  // flat list of selected packed rows: slot -> cluster by binary search over the cumulative sizes
  const int limit = min(total_tok, (int)a.packed_width);
  int32_t* rows = a.rows + (int64_t)h * a.packed_width;
  if (total_sel <= SEL_CSR_SMEM) {
    for (int o = threadIdx.x; o < limit; o += T) {
      int lo_r = 0, hi_r = total_sel;                 // last r with cum[r] <= o
      while (hi_r - lo_r > 1) {
        const int mid = (lo_r + hi_r) >> 1;
        if (csr_cum[mid] <= o) lo_r = mid; else hi_r = mid;
      }
      rows[o] = csr_start[lo_r] + (o - csr_cum[lo_r]);
    }
  } else {
    for (int o = threadIdx.x; o < limit; o += T) {
      int lo_r = 0, hi_r = total_sel;
      while (hi_r - lo_r > 1) {
        const int mid = (lo_r + hi_r) >> 1;
        if (rc[mid] <= o) lo_r = mid; else hi_r = mid;
      }
      rows[o] = rs[lo_r] + (o - rc[lo_r]);
    }
  }
}

// ------------------------------------------------------------------ attend + merge
template <int D, int G>
__global__ void __launch_bounds__(256)
decode_attend_kernel(const DecodeArgs a) {
  constexpr int DPL = D / 16;                  // dims per lane (a half-warp covers a row)
  constexpr int CH = DPL / 8;                  // 16-byte chunks per lane
  __shared__ float s_acc[8][G][D];             // per-warp partial outputs
  __shared__ float s_ml[8][G][2];
  __shared__ int s_last;
  const int h = blockIdx.x, split = blockIdx.y, nsplit = gridDim.y;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int hw = lane >> 4, l16 = lane & 15;
  const long long q_pos = load_pos(a);
  const int plen = *a.prompt_length;
  const int n_prompt = min(a.rtokens[h], (int)a.packed_width);
  const int n_suffix = (int)max(0LL, min(q_pos - plen + 1, (long long)a.suffix_blocks * a.suffix_block));
  const int total = n_prompt + n_suffix;
  const int per_split = (int)ceil_div(total, nsplit);
  const int lo = split * per_split, hi = min(total, lo + per_split);

  // q fragment: lane owns dims {ch * 128 + l16 * 8 + e}
  float q[G][DPL];
#pragma unroll
  for (int t = 0; t < G; ++t)
#pragma unroll
    for (int ch = 0; ch < CH; ++ch) {
      const uint4 raw = *reinterpret_cast<const uint4*>(a.q_post + (int64_t)(h * G + t) * D + ch * 128 + l16 * 8);
      const __nv_bfloat162* p2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float2 f2 = __bfloat1622float2(p2[e]);
        q[t][ch * 8 + 2 * e] = f2.x * a.sm_scale_log2;
        q[t][ch * 8 + 2 * e + 1] = f2.y * a.sm_scale_log2;
      }
    }
  float acc[G][DPL], m_run[G], l_run[G];
#pragma unroll
  for (int t = 0; t < G; ++t) {
    m_run[t] = -INFINITY;
    l_run[t] = 0.f;
#pragma unroll
    for (int d = 0; d < DPL; ++d) acc[t][d] = 0.f;
  }
  const int32_t* rows = a.rows + (int64_t)h * a.packed_width;
  const int32_t* posting = a.posting + (int64_t)h * a.packed_width;
  const int64_t pk_plane = a.packed_width * (int64_t)a.num_kv_heads * D;
  const int64_t sf_plane = (int64_t)a.suffix_blocks * a.suffix_block * a.num_kv_heads * D;

  // Each half-warp takes U rows per step.  The row indices of the next step, then all K / V
  // rows of this step, are in flight before any arithmetic, so a half-warp keeps U kilobyte-
  // sized requests outstanding instead of one.
  constexpr int U = 4;
  auto row_source = [&](int o, const __nv_bfloat16*& kp, int64_t& voff, int& post_row, bool& in_range) {
    // o: slot in [lo, hi); prompt slots come from the selected-row list, the rest from the suffix store
    kp = a.packed_kv;
    voff = pk_plane;
    post_row = -1;
    in_range = false;
    if (o >= hi) return;
    if (o < n_prompt) {
      const int r = rows[o];
      kp = a.packed_kv + ((int64_t)r * a.num_kv_heads + h) * D;
      post_row = r;
      in_range = true;
    } else {
      const long long pos = (long long)plen + (o - n_prompt);
      const long long block = pos / a.suffix_block;
      if (pos <= q_pos && block < a.table_len) {
        const long long phys = a.suffix_table[block];
        kp = a.suffix_kv + (((phys * a.suffix_block + (pos - block * a.suffix_block)) * a.num_kv_heads) + h) * D;
        voff = sf_plane;
        in_range = true;
      }
    }
  };
  for (int base = lo + warp * 2; base < hi; base += 16 * U) {
    const __nv_bfloat16* kp[U];
    int64_t voff[U];
    int post_row[U];
    bool keep[U];
#pragma unroll
    for (int u = 0; u < U; ++u) row_source(base + 16 * u + hw, kp[u], voff[u], post_row[u], keep[u]);
    uint4 kraw[U][CH], vraw[U][CH];
    int post[U];
#pragma unroll
    for (int u = 0; u < U; ++u) {
      post[u] = INT_MIN;
      if (keep[u] && post_row[u] >= 0) post[u] = __ldg(posting + post_row[u]);
#pragma unroll
      for (int ch = 0; ch < CH; ++ch) {
        kraw[u][ch] = make_uint4(0, 0, 0, 0);
        vraw[u][ch] = make_uint4(0, 0, 0, 0);
        if (keep[u]) {
          kraw[u][ch] = __ldg(reinterpret_cast<const uint4*>(kp[u] + ch * 128 + l16 * 8));
          vraw[u][ch] = __ldg(reinterpret_cast<const uint4*>(kp[u] + voff[u] + ch * 128 + l16 * 8));
        }
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      float s2[G];
#pragma unroll
      for (int t = 0; t < G; ++t) s2[t] = 0.f;
#pragma unroll
      for (int ch = 0; ch < CH; ++ch) {
        const __nv_bfloat162* p2 = reinterpret_cast<const __nv_bfloat162*>(&kraw[u][ch]);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float2 f2 = __bfloat1622float2(p2[e]);
#pragma unroll
          for (int t = 0; t < G; ++t) {
            s2[t] = fmaf(q[t][ch * 8 + 2 * e], f2.x, s2[t]);
            s2[t] = fmaf(q[t][ch * 8 + 2 * e + 1], f2.y, s2[t]);
          }
        }
      }
#pragma unroll
      for (int t = 0; t < G; ++t) {
#pragma unroll
        for (int off = 8; off > 0; off >>= 1) s2[t] += __shfl_xor_sync(0xffffffffu, s2[t], off);
      }
      // a prompt row counts only if its token is at or before the query's position
      if (keep[u] && (long long)post[u] <= q_pos) {
        float p[G];
#pragma unroll
        for (int t = 0; t < G; ++t) {
          const float mx = fmaxf(m_run[t], s2[t]);
          const float alpha = exp2f(m_run[t] - mx);       // 0 on the first row (m_run = -inf)
          p[t] = exp2f(s2[t] - mx);
          l_run[t] = l_run[t] * alpha + p[t];
          m_run[t] = mx;
          if (alpha != 1.f) {
#pragma unroll
            for (int d = 0; d < DPL; ++d) acc[t][d] *= alpha;
          }
        }
#pragma unroll
        for (int ch = 0; ch < CH; ++ch) {
          const __nv_bfloat162* p2 = reinterpret_cast<const __nv_bfloat162*>(&vraw[u][ch]);
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const float2 f2 = __bfloat1622float2(p2[e]);
#pragma unroll
            for (int t = 0; t < G; ++t) {
              acc[t][ch * 8 + 2 * e] = fmaf(p[t], f2.x, acc[t][ch * 8 + 2 * e]);
              acc[t][ch * 8 + 2 * e + 1] = fmaf(p[t], f2.y, acc[t][ch * 8 + 2 * e + 1]);
            }
          }
        }
      }
    }
  }
  // merge the two half-warps, then the 8 warps, into the split's partial
#pragma unroll
  for (int t = 0; t < G; ++t) {
    const float m_o = __shfl_xor_sync(0xffffffffu, m_run[t], 16);
    const float l_o = __shfl_xor_sync(0xffffffffu, l_run[t], 16);
    const float mx = fmaxf(m_run[t], m_o);
    const float w_s = m_run[t] == -INFINITY ? 0.f : exp2f(m_run[t] - mx);
    const float w_o = m_o == -INFINITY ? 0.f : exp2f(m_o - mx);
#pragma unroll
    for (int d = 0; d < DPL; ++d) {
      const float other = __shfl_xor_sync(0xffffffffu, acc[t][d], 16);
      acc[t][d] = acc[t][d] * w_s + other * w_o;
    }
    l_run[t] = l_run[t] * w_s + l_o * w_o;
    m_run[t] = mx;
    if (hw == 0) {
#pragma unroll
      for (int ch = 0; ch < CH; ++ch)
#pragma unroll
        for (int e = 0; e < 8; ++e) s_acc[warp][t][ch * 128 + l16 * 8 + e] = acc[t][ch * 8 + e];
      if (l16 == 0) { s_ml[warp][t][0] = m_run[t]; s_ml[warp][t][1] = l_run[t]; }
    }
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < G * D; idx += blockDim.x) {
    const int t = idx / D, d = idx % D;
    float mx = -INFINITY;
#pragma unroll
    for (int w = 0; w < 8; ++w) mx = fmaxf(mx, s_ml[w][t][0]);
    float num = 0.f, den = 0.f;
#pragma unroll
    for (int w = 0; w < 8; ++w) {
      const float m_w = s_ml[w][t][0];
      const float sc = m_w == -INFINITY ? 0.f : exp2f(m_w - mx);
      num += s_acc[w][t][d] * sc;
      den += s_ml[w][t][1] * sc;
    }
    a.pacc[((int64_t)(h * G + t) * nsplit + split) * D + d] = num;
    if (d == 0) {
      a.pml[((int64_t)(h * G + t) * nsplit + split) * 2] = mx;
      a.pml[((int64_t)(h * G + t) * nsplit + split) * 2 + 1] = den;
    }
  }
  // the last CTA of the head merges every split (no waiting: a ticket counter)
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) {
    const int ticket = atomicAdd(&a.tickets[h], 1);
    s_last = ticket == nsplit - 1;
    if (s_last) a.tickets[h] = 0;                   // ready for the next step / graph replay
  }
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  // Final merge by the head's last CTA.  The split weights are computed once into shared
  // memory; then every thread owns four consecutive output columns and reads one float4 per
  // split, all independent, so the loads overlap instead of queueing behind one another.
  float* s_w = &s_acc[0][0][0];                       // [G][nsplit] weights, then [G] denominators
  for (int t = warp; t < G; t += 8) {
    const float* ml = a.pml + (int64_t)(h * G + t) * nsplit * 2;
    float mx = -INFINITY;
    for (int s = lane; s < nsplit; s += 32) mx = fmaxf(mx, __ldcg(ml + 2 * s));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    float den = 0.f;
    for (int s = lane; s < nsplit; s += 32) {
      const float m_s = __ldcg(ml + 2 * s);
      const float sc = m_s == -INFINITY ? 0.f : exp2f(m_s - mx);
      s_w[t * nsplit + s] = sc;
      den += __ldcg(ml + 2 * s + 1) * sc;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) den += __shfl_xor_sync(0xffffffffu, den, o);
    if (lane == 0) s_w[G * nsplit + t] = den;
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < G * D / 4; idx += blockDim.x) {
    const int t = idx / (D / 4), d = (idx % (D / 4)) * 4;
    const float4* src = reinterpret_cast<const float4*>(a.pacc + (int64_t)(h * G + t) * nsplit * D + d);
    float4 num = make_float4(0.f, 0.f, 0.f, 0.f);
    constexpr int MB = 16;                              // splits whose partials are in flight together
    for (int s0 = 0; s0 < nsplit; s0 += MB) {
      float4 v[MB];
#pragma unroll
      for (int i = 0; i < MB; ++i)
        v[i] = s0 + i < nsplit ? __ldcg(src + (int64_t)(s0 + i) * (D / 4)) : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
      for (int i = 0; i < MB; ++i) {
        const float sc = s0 + i < nsplit ? s_w[t * nsplit + s0 + i] : 0.f;
        num.x += v[i].x * sc; num.y += v[i].y * sc; num.z += v[i].z * sc; num.w += v[i].w * sc;
      }
    }
    const float den = s_w[G * nsplit + t];
    const float inv = den == 0.f ? 0.f : 1.f / den;
    __nv_bfloat162 o01 = __floats2bfloat162_rn(num.x * inv, num.y * inv);
    __nv_bfloat162 o23 = __floats2bfloat162_rn(num.z * inv, num.w * inv);
    uint2 packed;
    packed.x = *reinterpret_cast<uint32_t*>(&o01);
    packed.y = *reinterpret_cast<uint32_t*>(&o23);
    *reinterpret_cast<uint2*>(a.out + (int64_t)(h * G + t) * D + d) = packed;
  }
}

int64_t align_up(int64_t x, int64_t a) { return (x + a - 1) / a * a; }

struct WsLayout {
  int64_t logit, ml, score, rstart, rlen, rcum, rcount, rtokens, rows, pacc, pml, tickets, vectors, total;
};

WsLayout ws_layout(int hq, int hkv, int d, int c, int64_t width, int splits, int score_blocks) {
  const int g = hq / hkv;
  WsLayout w;
  int64_t off = 0;
  auto take = [&](int64_t bytes) { int64_t o = off; off = align_up(off + bytes, 256); return o; };
  w.tickets = take((int64_t)hkv * 4);
  w.logit = take((int64_t)hkv * g * c * 4);
  w.ml = take((int64_t)hkv * score_blocks * g * 2 * 4);
  w.score = take((int64_t)hkv * c * 4);
  w.rstart = take((int64_t)hkv * c * 4);
  w.rlen = take((int64_t)hkv * c * 4);
  w.rcum = take((int64_t)hkv * c * 4);
  w.rcount = take((int64_t)hkv * 4);
  w.rtokens = take((int64_t)hkv * 4);
  w.rows = take((int64_t)hkv * width * 4);
  w.pacc = take((int64_t)hq * splits * d * 4);
  w.pml = take((int64_t)hq * splits * 2 * 4);
  w.vectors = take((int64_t)hq * d * 2);
  w.total = off;
  return w;
}

int score_blocks_for(int hkv, int c) {
  int b = std::max(1, SCORE_BLOCKS_TARGET / std::max(hkv, 1));
  b = std::min(b, std::max(1, c / 32));
  return b;
}

}  // namespace

extern "C" int64_t semblo_decode_workspace_bytes(int num_q_heads, int num_kv_heads, int head_dim,
                                                 int num_clusters, int64_t packed_width,
                                                 int num_splits) {
  return ws_layout(num_q_heads, num_kv_heads, head_dim, num_clusters, packed_width, num_splits,
                   score_blocks_for(num_kv_heads, num_clusters)).total;
}

extern "C" int semblo_decode_workspace_offsets(int num_q_heads, int num_kv_heads, int head_dim,
                                               int num_clusters, int64_t packed_width,
                                               int num_splits, int64_t* offsets /* [13] */) {
  const WsLayout w = ws_layout(num_q_heads, num_kv_heads, head_dim, num_clusters, packed_width,
                               num_splits, score_blocks_for(num_kv_heads, num_clusters));
  const int64_t v[13] = {w.tickets, w.logit, w.ml, w.score, w.rstart, w.rlen, w.rcum,
                         w.rcount, w.rtokens, w.rows, w.pacc, w.pml, w.vectors};
  for (int i = 0; i < 13; ++i) offsets[i] = v[i];
  return 0;
}

extern "C" int semblo_decode_step(
    const void* q_post, const void* q_pre, const void* k_post, const void* v_new, const void* k_pre,
    const void* positions, int pos_is_int64,
    const void* codebooks, const int32_t* sizes, const int32_t* indptr, const int32_t* posting,
    const void* packed_kv, int64_t packed_width,
    void* suffix_kv, void* suffix_kpre, const int32_t* suffix_table, int suffix_blocks,
    int suffix_block, int table_len, const int32_t* prompt_length,
    int num_q_heads, int num_kv_heads, int head_dim, int num_clusters,
    float temperature, float beta, int target_tokens, int sink_tokens, int iters, float sm_scale,
    int num_splits, void* workspace, int64_t workspace_bytes, void* output, int32_t* status,
    int stage_mask, void* stream) {
  SEMBLO_REQUIRE(num_kv_heads > 0 && num_q_heads % num_kv_heads == 0, "query heads must be a multiple of the KV heads");
  const int g = num_q_heads / num_kv_heads;
  SEMBLO_REQUIRE(g <= MAX_G, "at most %d query heads per KV head", MAX_G);
  SEMBLO_REQUIRE(head_dim == 128 || head_dim == 256, "head_dim %d must be 128 or 256", head_dim);
  SEMBLO_REQUIRE(num_clusters >= 32 && num_clusters <= SEL_THREADS * SEL_MAX_PER,
                 "cluster count %d outside [32, %d]", num_clusters, SEL_THREADS * SEL_MAX_PER);
  SEMBLO_REQUIRE(temperature > 0.f && num_splits > 0, "temperature and split count must be positive");
  SEMBLO_REQUIRE((k_post == nullptr) == (v_new == nullptr), "key and value of the new token go together");
  SEMBLO_REQUIRE(status != nullptr, "status word is required");
  const int sblocks = score_blocks_for(num_kv_heads, num_clusters);
  const WsLayout w = ws_layout(num_q_heads, num_kv_heads, head_dim, num_clusters, packed_width, num_splits, sblocks);
  SEMBLO_REQUIRE(workspace_bytes >= w.total, "decode workspace has %lld bytes, %lld needed",
                 (long long)workspace_bytes, (long long)w.total);
  uint8_t* ws = (uint8_t*)workspace;
  DecodeArgs a;
  a.num_q_heads = num_q_heads; a.num_kv_heads = num_kv_heads; a.head_dim = head_dim;
  a.num_clusters = num_clusters; a.group = g;
  a.q_post = (const __nv_bfloat16*)q_post; a.q_pre = (const __nv_bfloat16*)q_pre;
  a.k_post = (const __nv_bfloat16*)k_post; a.v_new = (const __nv_bfloat16*)v_new;
  a.k_pre = (const __nv_bfloat16*)k_pre;
  a.positions = positions; a.pos_is_int64 = pos_is_int64;
  a.codebooks = (const __nv_bfloat16*)codebooks; a.sizes = sizes; a.indptr = indptr; a.posting = posting;
  a.packed_kv = (const __nv_bfloat16*)packed_kv; a.packed_width = packed_width;
  a.suffix_kv = (__nv_bfloat16*)suffix_kv; a.suffix_kpre = (__nv_bfloat16*)suffix_kpre;
  a.suffix_table = suffix_table; a.suffix_blocks = suffix_blocks; a.suffix_block = suffix_block;
  a.table_len = table_len; a.prompt_length = prompt_length;
  a.scale_log2_router = LOG2E / temperature; a.beta = beta; a.sm_scale_log2 = sm_scale * LOG2E;
  a.target_tokens = target_tokens; a.sink_tokens = sink_tokens; a.iters = iters;
  a.num_splits = num_splits; a.score_blocks = sblocks;
  a.ws_logit = (float*)(ws + w.logit); a.ws_ml = (float*)(ws + w.ml); a.ws_score = (float*)(ws + w.score);
  a.rstart = (int32_t*)(ws + w.rstart); a.rlen = (int32_t*)(ws + w.rlen); a.rcum = (int32_t*)(ws + w.rcum);
  a.rcount = (int32_t*)(ws + w.rcount); a.rtokens = (int32_t*)(ws + w.rtokens);
  a.rows = (int32_t*)(ws + w.rows); a.pacc = (float*)(ws + w.pacc); a.pml = (float*)(ws + w.pml);
  a.tickets = (int32_t*)(ws + w.tickets); a.vectors = (__nv_bfloat16*)(ws + w.vectors);
  a.out = (__nv_bfloat16*)output; a.status = status;
  cudaStream_t st = (cudaStream_t)stream;
  if (stage_mask & 1) {
    const dim3 sgrid(num_kv_heads, sblocks);
    if (head_dim == 256 && g == 4) decode_score_kernel<256, 4><<<sgrid, 256, 0, st>>>(a);
    else if (head_dim == 128 && g == 4) decode_score_kernel<128, 4><<<sgrid, 256, 0, st>>>(a);
    else if (head_dim == 128 && g == 8) decode_score_kernel<128, 8><<<sgrid, 256, 0, st>>>(a);
    else return semblo::fail(semblo::SEMBLO_EINVAL, "decode scoring supports head_dim 256 with 4, or 128 with 4 or 8, query heads per KV head (got %d, %d)", head_dim, g);
  }
  if (stage_mask & 2) {
    decode_penalise_kernel<<<dim3(num_kv_heads, (unsigned)ceil_div(num_clusters, PEN_THREADS)), PEN_THREADS, 0, st>>>(a);
    if (num_clusters <= 2048) decode_select_kernel<4, 512><<<num_kv_heads, 512, 0, st>>>(a);
    else if (num_clusters <= 8192) decode_select_kernel<16, 512><<<num_kv_heads, 512, 0, st>>>(a);
    else decode_select_kernel<16, 1024><<<num_kv_heads, 1024, 0, st>>>(a);
  }
  if (stage_mask & 4) {
    dim3 grid(num_kv_heads, num_splits);
#define SEMBLO_DECODE_CASE(DD, GG) \
  if (head_dim == DD && g == GG) decode_attend_kernel<DD, GG><<<grid, 256, 0, st>>>(a); else
    SEMBLO_DECODE_CASE(256, 4)
    SEMBLO_DECODE_CASE(128, 4)
    SEMBLO_DECODE_CASE(128, 8)
#undef SEMBLO_DECODE_CASE
    return semblo::fail(semblo::SEMBLO_EINVAL, "decode attention supports 4 or 8 query heads per KV head (got %d)", g);
  }
  SEMBLO_LAUNCH_CHECK();
  return 0;
}
