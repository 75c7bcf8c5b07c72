// Block-sparse decode step over the decode arena: suffix write, query routing,
// centroid scoring, threshold selection with CSR emission, split-KV gather attention
// over the selected cluster rows plus the exact generated suffix, and the LSE merge.
//
// The step is HBM-bound (codebook read + gathered K/V rows), so the kernels are
// plain coalesced 16-byte loads spread over the whole GPU:
//   decode_score_kernel   grid [Hkv, blocks + 1]: router, logits of a slice of the codebook and the
//                         slice's (max, sum-exp) per head; the extra block row writes the
//                         token's K/V into the suffix store
//   decode_select_kernel  grid [8, Hkv], one thread-block cluster per head: log-sum-exp,
//                         penalised scores, the bisected threshold as a radix select over the
//                         clusters' paths through the tree of midpoints (histograms summed
//                         through distributed shared memory), CSR (start, len, cum) in cluster
//                         order and the CSR position where every attention split starts
//   decode_attend_kernel  grid [Hkv, splits]: expands its own slice of the CSR, brings all its
//                         K/V rows into shared memory with 16-byte asynchronous copies in one
//                         go, then one warp per row; the last CTA of a head merges the splits
//                         and writes the output
// The select and attend kernels are launched as programmatic dependents: they start while the
// kernel before them drains and wait (griddepcontrol.wait) before they touch its results.
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

#include <cooperative_groups.h>

namespace cg = cooperative_groups;
using semblo::ceil_div;
using sm100::pdl_launch_dependents;
using sm100::pdl_wait;

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
  int32_t *rstart, *rlen, *rcum;   // [Hkv, C]
  int32_t *rcount, *rtokens;       // [Hkv]
  int32_t* split_start; // [Hkv, splits, 4] per split: CSR entry and offset inside it where its rows begin, selected rows, selected clusters
  float* pacc;          // [Hq, splits, D]
  float* pml;           // [Hq, splits, 2]
  int32_t* tickets;     // [Hkv]
  __nv_bfloat16* vectors;   // [Hq, D] routing vectors (kept for inspection)
  __nv_bfloat16* out;
  float* lse_out;           // [Hq] natural-log log-sum-exp of the result, or null
  int vectors_given;        // q_pre already holds the routing vectors (no router pass)
  // paged_posting_attention: when tile_starts is set the attend kernel reads, instead of the selected
  // rows and the suffix store, the positions listed by posting tiles through a block table
  const int32_t *tile_starts, *tile_lengths, *tile_counts;   // [Hkv, T], [Hkv, T], [Hkv] of this query
  int tile_stride, token_tile;
  const int32_t* tile_posting;                               // [Hkv, Lp] positions
  int64_t tile_posting_stride;
  const __nv_bfloat16* cache;                                // [2, blocks, block_size, Hkv, D]
  int64_t cache_plane;
  const int32_t* block_table;
  int block_size, block_table_len;
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
  pdl_launch_dependents();            // the select kernel may take its seats; it waits for this grid to finish

  if (blk == gridDim.y - 1) {
    // The extra block row: head 0's CTA writes the token's K/V (and pre-RoPE key) into the suffix
    // store and does nothing else, so no scoring CTA carries that chain of dependent loads.
    if (h != 0 || a.k_post == nullptr) return;
    const long long pos = load_pos(a);
    const long long block = pos / a.suffix_block;
    if (block >= 0 && block < a.table_len) {
      const long long phys = a.suffix_table[block];
      const long long off = pos - block * a.suffix_block;
      const int64_t plane = (int64_t)a.suffix_blocks * a.suffix_block * a.num_kv_heads * D;
      const int64_t dst = (phys * a.suffix_block + off) * a.num_kv_heads * D;
      for (int i = threadIdx.x * 8; i < a.num_kv_heads * D; i += blockDim.x * 8) {
        *reinterpret_cast<uint4*>(a.suffix_kv + dst + i) = *reinterpret_cast<const uint4*>(a.k_post + i);
        *reinterpret_cast<uint4*>(a.suffix_kv + plane + dst + i) = *reinterpret_cast<const uint4*>(a.v_new + i);
        if (a.suffix_kpre && a.k_pre)
          *reinterpret_cast<uint4*>(a.suffix_kpre + dst + i) = *reinterpret_cast<const uint4*>(a.k_pre + i);
      }
    } else if (threadIdx.x == 0) {
      atomicCAS(a.status, 0, sm100::STATUS_OVERFLOW);
    }
    return;
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
  const int nblk = gridDim.y - 1;                     // scoring blocks (the last block row is the suffix write)
  const int per_block = (int)ceil_div(C, nblk);
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
    if (a.vectors_given) {                             // the caller ran the router: take the vectors as they are
#pragma unroll
      for (int i = 0; i < D / 32; ++i) {
        const int d = lane + 32 * i;
        qv[t * D + d] = __bfloat162float(src[d]);
        if (blk == 0) a.vectors[(int64_t)(h * G + t) * D + d] = src[d];
      }
      continue;
    }
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
    float* dst = a.ws_ml + (((int64_t)h * nblk + blk) * G + t) * 2;
    dst[0] = m;
    dst[1] = l;
  }
}

// ------------------------------------------------------------------ select
// One thread-block cluster of SEL_CL CTAs per KV head.  A thread owns SEL_PER consecutive
// clusters; CTA r of the head owns clusters [r C / SEL_CL, (r + 1) C / SEL_CL).
constexpr int SEL_CL = 8;
constexpr int SEL_THREADS = 512;
constexpr int SEL_PER = 4;
constexpr int SEL_MAX_CLUSTERS = SEL_CL * SEL_THREADS * SEL_PER;     // 16384
constexpr int SEL_WARPS = SEL_THREADS / 32;

// What the CTAs of a head exchange through distributed shared memory.
struct SelectShared {
  float lse2[MAX_G];
  float w_mx[SEL_WARPS], w_mn[SEL_WARPS];
  int w_tot[SEL_WARPS], w_sel[SEL_WARPS], w_tok[SEL_WARPS];
  float cta_mx, cta_mn;          // read by the other CTAs of the head
  int cta_tot, cta_sel, cta_tok;
  int hist1[256], hist2[256];    // read by the other CTAs of the head
  int total[256];
  float all_mx, all_mn;
  int all_tot, byte_found, byte_above, base_sel, base_tok, sum_sel, sum_tok;
};

// Largest bin b whose suffix sum total[b] + total[b + 1] + ... reaches `budget` (255 when the
// budget is not positive, 0 when nothing reaches it), and the sum of the bins above it.  Warp 0.
__device__ __forceinline__ void find_threshold_bin(const int* total, int budget, int lane, int* found, int* above) {
  int mine[8], s = 0;
#pragma unroll
  for (int k = 0; k < 8; ++k) { mine[k] = total[lane * 8 + k]; s += mine[k]; }
  int suf = s;                                         // sum over lanes >= this one
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const int v = __shfl_down_sync(0xffffffffu, suf, o);
    if (lane + o < 32) suf += v;
  }
  const unsigned reach = __ballot_sync(0xffffffffu, suf >= budget);
  if (reach == 0u) {
    if (lane == 0) { *found = 0; *above = 0; }
    return;
  }
  const int top = 31 - __clz(reach);
  if (lane == top) {
    int run = suf - s;                                 // the bins of the lanes above
    int b = 0, ab = 0;
#pragma unroll
    for (int k = 7; k >= 0; --k) {
      if (run + mine[k] >= budget) { b = lane * 8 + k; ab = run; break; }
      run += mine[k];
    }
    *found = b;
    *above = ab;
  }
}

// Selection of one decode query: penalised scores, the bisected threshold, CSR of the selected
// clusters in cluster order, and where every attention split starts in it.
//
// The 16-step bisection of fused_decode.py:159-187 is evaluated without its 16 dependent sweeps.
// The midpoints it can visit form a fixed binary tree over [lo0, hi0].  Every cluster walks that
// tree with its own score (bit k = score >= midpoint at depth k, then lo / hi move exactly as in
// the reference, in fp32), which gives it a 16-bit code; codes order the clusters as the midpoints
// do.  On the bisection's own path the step at depth k asks whether the sizes of the clusters
// with score >= m_k reach the budget; a cluster that left the path earlier sits wholly above or
// below every later midpoint of the path, so that sum is the sum over codes >= (path so far, 1,
// 0 ...).  The path is therefore the largest 16-bit value T whose suffix sum reaches the budget,
// found with two 256-bin histograms, and `score >= theta` is `code >= T`, bit for bit.
__global__ void __cluster_dims__(SEL_CL, 1, 1) __launch_bounds__(SEL_THREADS)
decode_select_kernel(const DecodeArgs a) {
  __shared__ SelectShared sh;
  cg::cluster_group cluster = cg::this_cluster();
  const int rank = (int)cluster.block_rank();
  const int h = blockIdx.y;
  const int C = a.num_clusters, G = a.group;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  pdl_launch_dependents();
  if (tid < 256) { sh.hist1[tid] = 0; sh.hist2[tid] = 0; }
  pdl_wait();                                          // the score kernel's logits and partials are complete
  // this thread's logits, sizes and cluster starts are requested before the log-sum-exp is built
  const int per_cta = C / SEL_CL;                      // C is a multiple of 32
  const int c0 = rank * per_cta + tid * SEL_PER;
  const bool active = tid * SEL_PER < per_cta;
  float4 lg[MAX_G];
  int4 sz = make_int4(0, 0, 0, 0);
  int starts[SEL_PER] = {0, 0, 0, 0};
  if (active) {
#pragma unroll
    for (int t = 0; t < MAX_G; ++t)
      if (t < G) lg[t] = __ldcg(reinterpret_cast<const float4*>(a.ws_logit + ((int64_t)h * G + t) * C + c0));
    sz = __ldg(reinterpret_cast<const int4*>(a.sizes + (int64_t)h * C + c0));
#pragma unroll
    for (int i = 0; i < SEL_PER; ++i) starts[i] = __ldg(a.indptr + (int64_t)h * (C + 1) + c0 + i);
  }
  if (warp < G) {
    // log-sum-exp of a query head from the score kernel's block partials: the maximum first, then
    // one pass of weighted sums
    const int t = warp;
    float2 part[4];
    float m = -INFINITY;
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const int b = lane + 32 * k;
      part[k] = b < a.score_blocks
                    ? __ldcg(reinterpret_cast<const float2*>(a.ws_ml + (((int64_t)h * a.score_blocks + b) * G + t) * 2))
                    : make_float2(-INFINITY, 0.f);
      m = fmaxf(m, part[k].x);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    float l = 0.f;
#pragma unroll
    for (int k = 0; k < 4; ++k) l += part[k].x == -INFINITY ? 0.f : part[k].y * exp2f(part[k].x - m);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) l += __shfl_xor_sync(0xffffffffu, l, o);
    if (lane == 0) sh.lse2[t] = m + log2f(l);
  }
  __syncthreads();

  // penalised scores of this thread's clusters
  const bool has_sink = a.sink_tokens > 0;
  float score[SEL_PER];
  int real[SEL_PER], seen[SEL_PER];
#pragma unroll
  for (int i = 0; i < SEL_PER; ++i) { score[i] = NEG_BIG; real[i] = 0; seen[i] = 0; }
  if (active) {
    float prob[SEL_PER] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int t = 0; t < MAX_G; ++t) {
      if (t < G) {
        const float ls = sh.lse2[t];
        prob[0] += exp2f(lg[t].x - ls); prob[1] += exp2f(lg[t].y - ls);
        prob[2] += exp2f(lg[t].z - ls); prob[3] += exp2f(lg[t].w - ls);
      }
    }
    real[0] = sz.x; real[1] = sz.y; real[2] = sz.z; real[3] = sz.w;
#pragma unroll
    for (int i = 0; i < SEL_PER; ++i) {
      seen[i] = (has_sink && c0 + i == 0) ? 0 : real[i];      // the budget does not see the sink cluster
      const float n = (float)seen[i];
      float sc = log2f(fmaxf(prob[i], 1e-38f)) * LN2;
      if (a.beta != 0.f) sc -= a.beta * logf(1.0f + n);
      score[i] = n > 0.f ? sc : NEG_BIG;
    }
  }
  // maximum over all clusters, minimum over the live ones, live tokens: warp, CTA, head
  float mx = -INFINITY, mn = 3.4e38f;
  int tot = 0;
  if (active) {
#pragma unroll
    for (int i = 0; i < SEL_PER; ++i) {
      mx = fmaxf(mx, score[i]);
      if (seen[i] > 0) { mn = fminf(mn, score[i]); tot += seen[i]; }
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    mn = fminf(mn, __shfl_xor_sync(0xffffffffu, mn, o));
  }
  tot = __reduce_add_sync(0xffffffffu, tot);
  if (lane == 0) { sh.w_mx[warp] = mx; sh.w_mn[warp] = mn; sh.w_tot[warp] = tot; }
  __syncthreads();
  if (warp == 0) {
    mx = lane < SEL_WARPS ? sh.w_mx[lane] : -INFINITY;
    mn = lane < SEL_WARPS ? sh.w_mn[lane] : 3.4e38f;
    tot = lane < SEL_WARPS ? sh.w_tot[lane] : 0;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
      mn = fminf(mn, __shfl_xor_sync(0xffffffffu, mn, o));
    }
    tot = __reduce_add_sync(0xffffffffu, tot);
    if (lane == 0) { sh.cta_mx = mx; sh.cta_mn = mn; sh.cta_tot = tot; }
  }
  cluster.sync();
  if (warp == 0) {
    mx = -INFINITY; mn = 3.4e38f; tot = 0;
    if (lane < SEL_CL) {
      const SelectShared* peer = cluster.map_shared_rank(&sh, lane);
      mx = peer->cta_mx; mn = peer->cta_mn; tot = peer->cta_tot;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
      mn = fminf(mn, __shfl_xor_sync(0xffffffffu, mn, o));
    }
    tot = __reduce_add_sync(0xffffffffu, tot);
    if (lane == 0) { sh.all_mx = mx; sh.all_mn = mn; sh.all_tot = tot; }
  }
  __syncthreads();
  const int budget = max(a.target_tokens - a.sink_tokens, 0);
  const bool all_fit = sh.all_tot < budget;
  const float hi0 = sh.all_mx + 1e-6f;
  const float lo0 = fminf(sh.all_mn - 1e-6f, hi0 - 1e-5f);

  // every cluster's path through the tree of midpoints
  unsigned code[SEL_PER];
#pragma unroll
  for (int i = 0; i < SEL_PER; ++i) {
    float lo = lo0, hi = hi0;
    unsigned cd = 0;
    for (int it = 0; it < a.iters; ++it) {
      const float mid = (lo + hi) * 0.5f;
      const bool up = score[i] >= mid;
      cd = (cd << 1) | (up ? 1u : 0u);
      lo = up ? mid : lo;
      hi = up ? hi : mid;
    }
    code[i] = cd << (16 - a.iters);
    if (seen[i] > 0) atomicAdd(&sh.hist1[code[i] >> 8], seen[i]);
  }
  cluster.sync();
  if (tid < 256) {
    int s = 0;
#pragma unroll
    for (int r = 0; r < SEL_CL; ++r) s += cluster.map_shared_rank(&sh, r)->hist1[tid];
    sh.total[tid] = s;
  }
  __syncthreads();
  if (warp == 0) find_threshold_bin(sh.total, budget, lane, &sh.byte_found, &sh.byte_above);
  __syncthreads();
  const unsigned top_byte = (unsigned)sh.byte_found;
  const int budget2 = budget - sh.byte_above;
#pragma unroll
  for (int i = 0; i < SEL_PER; ++i)
    if (seen[i] > 0 && (code[i] >> 8) == top_byte) atomicAdd(&sh.hist2[code[i] & 255u], seen[i]);
  cluster.sync();
  if (tid < 256) {
    int s = 0;
#pragma unroll
    for (int r = 0; r < SEL_CL; ++r) s += cluster.map_shared_rank(&sh, r)->hist2[tid];
    sh.total[tid] = s;
  }
  __syncthreads();
  if (warp == 0) find_threshold_bin(sh.total, budget2, lane, &sh.byte_found, &sh.byte_above);
  __syncthreads();
  const unsigned threshold = (top_byte << 8) | (unsigned)sh.byte_found;

  // selection flags; CSR positions by a scan over the threads of the head in cluster order
  int n_sel = 0, n_tok = 0;
  unsigned sel_bits = 0;
#pragma unroll
  for (int i = 0; i < SEL_PER; ++i) {
    const bool is_sink = has_sink && c0 + i == 0;
    const bool s = active && ((seen[i] > 0 && (all_fit || code[i] >= threshold)) || (is_sink && real[i] > 0));
    sel_bits |= s ? (1u << i) : 0u;
    n_sel += s;
    n_tok += s ? real[i] : 0;
  }
  int inc_a = n_sel, inc_b = n_tok;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const int va = __shfl_up_sync(0xffffffffu, inc_a, o), vb = __shfl_up_sync(0xffffffffu, inc_b, o);
    if (lane >= o) { inc_a += va; inc_b += vb; }
  }
  if (lane == 31) { sh.w_sel[warp] = inc_a; sh.w_tok[warp] = inc_b; }
  __syncthreads();
  int wa = lane < SEL_WARPS ? sh.w_sel[lane] : 0, wb = lane < SEL_WARPS ? sh.w_tok[lane] : 0;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const int va = __shfl_up_sync(0xffffffffu, wa, o), vb = __shfl_up_sync(0xffffffffu, wb, o);
    if (lane >= o) { wa += va; wb += vb; }
  }
  const int cta_sel = __shfl_sync(0xffffffffu, wa, SEL_WARPS - 1), cta_tok = __shfl_sync(0xffffffffu, wb, SEL_WARPS - 1);
  const int warp_base_a = __shfl_sync(0xffffffffu, wa, warp) - sh.w_sel[warp];
  const int warp_base_b = __shfl_sync(0xffffffffu, wb, warp) - sh.w_tok[warp];
  if (tid == 0) { sh.cta_sel = cta_sel; sh.cta_tok = cta_tok; }
  cluster.sync();
  if (warp == 0) {
    int ps = 0, pt = 0;
    if (lane < SEL_CL) {
      const SelectShared* peer = cluster.map_shared_rank(&sh, lane);
      ps = peer->cta_sel; pt = peer->cta_tok;
    }
    const int before_s = __reduce_add_sync(0xffffffffu, lane < rank ? ps : 0);
    const int before_t = __reduce_add_sync(0xffffffffu, lane < rank ? pt : 0);
    const int all_s = __reduce_add_sync(0xffffffffu, ps), all_t = __reduce_add_sync(0xffffffffu, pt);
    if (lane == 0) { sh.base_sel = before_s; sh.base_tok = before_t; sh.sum_sel = all_s; sh.sum_tok = all_t; }
  }
  __syncthreads();
  const int total_sel = sh.sum_sel, total_tok = sh.sum_tok;
  int pos = sh.base_sel + warp_base_a + inc_a - n_sel;
  int cum = sh.base_tok + warp_base_b + inc_b - n_tok;
  // the attention splits divide the selected rows and the live suffix evenly (the attend kernel
  // computes the same numbers); a CSR entry records every split that starts inside it
  const long long q_pos = load_pos(a);
  const int plen = *a.prompt_length;
  const int n_prompt = min(total_tok, (int)a.packed_width);
  const int n_suffix = (int)max(0LL, min(q_pos - plen + 1, (long long)a.suffix_blocks * a.suffix_block));
  const int per_split = max(1, (int)ceil_div(n_prompt + n_suffix, a.num_splits));
  int32_t* rs = a.rstart + (int64_t)h * C;
  int32_t* rl = a.rlen + (int64_t)h * C;
  int32_t* rc = a.rcum + (int64_t)h * C;
  // per split {CSR entry, offset inside it, selected rows, selected clusters}: the first two by the
  // thread whose entry holds the split's first row, the totals by the head's first CTA
  int4* split = reinterpret_cast<int4*>(a.split_start) + (int64_t)h * a.num_splits;
  if (sel_bits) {
#pragma unroll
    for (int i = 0; i < SEL_PER; ++i) {
      if ((sel_bits >> i) & 1) {
        const int len = real[i];
        rs[pos] = starts[i];
        rl[pos] = len;
        rc[pos] = cum;
        for (int s = (int)ceil_div(cum, per_split); s < a.num_splits && s * per_split < cum + len; ++s)
          *reinterpret_cast<int2*>(&split[s]) = make_int2(pos, s * per_split - cum);
        ++pos;
        cum += len;
      }
    }
  }
  if (rank == 0) {
    for (int s = tid; s < a.num_splits; s += SEL_THREADS)
      *(reinterpret_cast<int2*>(&split[s]) + 1) = make_int2(total_tok, total_sel);
    if (tid == 0) {
      a.rcount[h] = total_sel;
      a.rtokens[h] = total_tok;
      if (total_tok > a.packed_width) atomicCAS(a.status, 0, sm100::STATUS_OVERFLOW);
    }
  }
  cluster.sync();                 // no CTA of the head leaves while a peer may still read its shared memory
}

// ------------------------------------------------------------------ attend + merge
// A CTA takes the slots [lo, hi) of its head's rows (selected prompt rows in CSR order, then the
// live suffix positions).  All of its rows are brought into shared memory at once with 16-byte
// asynchronous copies, so the bytes in flight cost no registers.  The arithmetic runs on the
// tensor cores with the G query heads of the KV head as one operand dimension (warp-level
// mma.sync m16n8k16; a single query has no 64-row tile to offer tcgen05): warp w takes rows
// [16 w, 16 w + 16) of the chunk,
//   S^T [heads x rows] = Q [heads (padded to 16) x D] K^T,   O^T [D x heads] += V^T [D x rows] P [rows x heads],
// and the accumulator layout of S^T is the operand layout P needs, so P never leaves registers.
constexpr int ATT_CHUNK = 128;           // rows resident at a time (one 16-row tile per warp)
constexpr int ATT_ENTRIES = 256;         // CSR entries looked at per chunk (each holds at least one row)

template <int D, int G>
struct AttendSmem {
  static constexpr int K_OFF = 0;                                    // [CHUNK][D] bf16, 16-byte chunks swizzled by row
  static constexpr int V_OFF = K_OFF + ATT_CHUNK * D * 2;
  static constexpr int ACC_OFF = V_OFF + ATT_CHUNK * D * 2;          // float [8][G][D]
  static constexpr int ML_OFF = ACC_OFF + 8 * G * D * 4;             // float [8][G][2]
  static constexpr int KP_OFF = ML_OFF + 8 * G * 2 * 4;              // const bf16* [CHUNK]
  static constexpr int VP_OFF = KP_OFF + ATT_CHUNK * 8;
  static constexpr int OK_OFF = VP_OFF + ATT_CHUNK * 8;              // int [CHUNK]
  static constexpr int ES_OFF = OK_OFF + ATT_CHUNK * 4;              // int [ENTRIES]
  static constexpr int EC_OFF = ES_OFF + ATT_ENTRIES * 4;            // int [ENTRIES + 1]
  static constexpr int WS_OFF = EC_OFF + (ATT_ENTRIES + 1) * 4 + 12; // int [8] warp sums (16-byte aligned)
  static constexpr int MISC_OFF = WS_OFF + 32;                       // int [4]
  static constexpr int TOTAL = MISC_OFF + 16;
};

__device__ __forceinline__ void cp_async16(void* dst_smem, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(sm100::smem_u32(dst_smem)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_wait_all() {
  asm volatile("cp.async.commit_group;\n\tcp.async.wait_group 0;" ::: "memory");
}
__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const void* smem_row) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(sm100::smem_u32(smem_row)));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], const void* smem_row) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(sm100::smem_u32(smem_row)));
}
// D (16 x 8, fp32) += A (16 x 16, bf16, row-major) B (16 x 8, bf16, column-major)
__device__ __forceinline__ void mma_bf16_16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                               uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

template <int D, int G>
__global__ void __launch_bounds__(256)
decode_attend_kernel(const DecodeArgs a) {
  using S = AttendSmem<D, G>;
  constexpr int LPR = D / 8;                   // 16-byte chunks per row
  constexpr int RPW = 32 / LPR;                // rows a warp copies per instruction
  constexpr int KSTEPS = D / 16;
  extern __shared__ __align__(128) uint8_t smem[];
  __nv_bfloat16* s_k = reinterpret_cast<__nv_bfloat16*>(smem + S::K_OFF);
  __nv_bfloat16* s_v = reinterpret_cast<__nv_bfloat16*>(smem + S::V_OFF);
  float* s_acc = reinterpret_cast<float*>(smem + S::ACC_OFF);
  float* s_ml = reinterpret_cast<float*>(smem + S::ML_OFF);
  const __nv_bfloat16** s_kp = reinterpret_cast<const __nv_bfloat16**>(smem + S::KP_OFF);
  const __nv_bfloat16** s_vp = reinterpret_cast<const __nv_bfloat16**>(smem + S::VP_OFF);
  int* s_ok = reinterpret_cast<int*>(smem + S::OK_OFF);
  int* e_start = reinterpret_cast<int*>(smem + S::ES_OFF);
  int* e_cum = reinterpret_cast<int*>(smem + S::EC_OFF);
  int* s_wsum = reinterpret_cast<int*>(smem + S::WS_OFF);
  int* s_misc = reinterpret_cast<int*>(smem + S::MISC_OFF);        // [0] last-CTA flag, [1] entry cursor, [2] offset in it
  const int h = blockIdx.x, split = blockIdx.y, nsplit = gridDim.y;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int sub = lane / LPR, l_in = lane % LPR;
  const int g = lane >> 2, t4 = lane & 3;      // fragment coordinates of the lane

  // everything that does not depend on the selection comes before the wait
  const long long q_pos = load_pos(a);
  const int plen = a.prompt_length ? *a.prompt_length : 0;
  // Q as the 16 x 16 row-major operand of every 16-dim step: rows = query heads (rows >= G are zero)
  uint32_t qa[KSTEPS][2];
#pragma unroll
  for (int kk = 0; kk < KSTEPS; ++kk) {
    qa[kk][0] = 0u;
    qa[kk][1] = 0u;
    if (g < G) {
      const __nv_bfloat16* qrow = a.q_post + (int64_t)(h * G + g) * D + kk * 16 + t4 * 2;
      qa[kk][0] = *reinterpret_cast<const uint32_t*>(qrow);
      qa[kk][1] = *reinterpret_cast<const uint32_t*>(qrow + 8);
    }
  }
  float o[KSTEPS][4];                          // O^T: tile nn holds dims 16 nn + g (+ 8), heads 2 t4 (+ 1)
#pragma unroll
  for (int nn = 0; nn < KSTEPS; ++nn)
#pragma unroll
    for (int e = 0; e < 4; ++e) o[nn][e] = 0.f;
  float m_run = -INFINITY, l_part = 0.f;       // of head g (lanes with g < G); l_part: this lane's share of the row sum
  const int64_t pk_plane = a.packed_width * (int64_t)a.num_kv_heads * D;
  const int64_t sf_plane = (int64_t)a.suffix_blocks * a.suffix_block * a.num_kv_heads * D;
  const int32_t* posting = a.posting + (int64_t)h * a.packed_width;
  pdl_wait();                                          // the selection is complete

  const bool tile_mode = a.tile_starts != nullptr;
  int4 rec = make_int4(0, 0, 0, 0);
  if (!tile_mode) rec = __ldcg(reinterpret_cast<const int4*>(a.split_start) + (int64_t)h * nsplit + split);
  const int n_prompt = min(rec.z, (int)a.packed_width);
  const int n_entries = rec.w;
  // the slots after the selected rows: the live suffix positions, or every slot of the posting tiles
  const int n_suffix = tile_mode ? __ldg(a.tile_counts + h) * a.token_tile
                                 : (int)max(0LL, min(q_pos - plen + 1, (long long)a.suffix_blocks * a.suffix_block));
  const int total = n_prompt + n_suffix;
  const int per_split = max(1, (int)ceil_div(total, nsplit));
  const int lo = split * per_split, hi = min(total, lo + per_split);
  const int32_t* rs = a.rstart + (int64_t)h * a.num_clusters;
  const int32_t* rl = a.rlen + (int64_t)h * a.num_clusters;
  if (tid == 0) {
    const bool has_prompt = lo < min(hi, n_prompt);
    s_misc[1] = has_prompt ? rec.x : 0;
    s_misc[2] = has_prompt ? rec.y : 0;
  }
  __syncthreads();

  for (int base = lo; base < hi; base += ATT_CHUNK) {
    const int n = min(ATT_CHUNK, hi - base);
    const int n16 = (n + 15) & ~15;
    const int np = max(0, min(n, n_prompt - base));     // prompt slots of this chunk, the rest is suffix
    const int e_first = s_misc[1], e_off = s_misc[2];
    if (np > 0) {
      // ATT_ENTRIES entries from the cursor on: starts, and the running count of their rows
      const int e = e_first + tid;
      int st = 0, ln = 0;
      if (e < n_entries) {
        st = __ldcg(rs + e);
        ln = __ldcg(rl + e);
        if (tid == 0) { st += e_off; ln -= e_off; }
      }
      int inc = ln;
#pragma unroll
      for (int o2 = 1; o2 < 32; o2 <<= 1) {
        const int v = __shfl_up_sync(0xffffffffu, inc, o2);
        if (lane >= o2) inc += v;
      }
      if (lane == 31) s_wsum[warp] = inc;
      __syncthreads();
      int wpre = 0;
#pragma unroll
      for (int w = 0; w < 8; ++w) wpre += w < warp ? s_wsum[w] : 0;
      e_start[tid] = st;
      e_cum[tid + 1] = wpre + inc;
      if (tid == 0) e_cum[0] = 0;
    }
    __syncthreads();
    int post = INT_MIN;
    bool is_prompt = false;
    if (tid < n16) {
      const __nv_bfloat16* kp = nullptr;
      const __nv_bfloat16* vp = nullptr;
      if (tid < np) {
        int lo_e = 0, hi_e = ATT_ENTRIES;               // last entry whose first row is at or before this slot
        while (hi_e - lo_e > 1) {
          const int mid = (lo_e + hi_e) >> 1;
          if (e_cum[mid] <= tid) lo_e = mid; else hi_e = mid;
        }
        const int row = e_start[lo_e] + (tid - e_cum[lo_e]);
        kp = a.packed_kv + ((int64_t)row * a.num_kv_heads + h) * D;
        vp = kp + pk_plane;
        post = __ldg(posting + row);
        is_prompt = true;
      } else if (tid < n && tile_mode) {
        // slot -> (tile, offset) -> logical position -> block table -> cache row (paged_attention.py:445-815)
        const int slot = base + tid, k = slot / a.token_tile, o = slot - k * a.token_tile;
        if (o < __ldg(a.tile_lengths + (int64_t)h * a.tile_stride + k)) {
          const long long pos = __ldg(a.tile_posting + (int64_t)h * a.tile_posting_stride +
                                      __ldg(a.tile_starts + (int64_t)h * a.tile_stride + k) + o);
          const long long block = pos / a.block_size;
          if (pos >= 0 && pos <= q_pos && block < a.block_table_len) {
            const long long phys = a.block_table[block];
            kp = a.cache + (((phys * a.block_size + (pos - block * a.block_size)) * a.num_kv_heads) + h) * D;
            vp = kp + a.cache_plane;
          }
        }
      } else if (tid < n) {
        const long long pos = (long long)plen + (base + tid - n_prompt);
        const long long block = pos / a.suffix_block;
        if (pos <= q_pos && block < a.table_len) {
          const long long phys = a.suffix_table[block];
          kp = a.suffix_kv + (((phys * a.suffix_block + (pos - block * a.suffix_block)) * a.num_kv_heads) + h) * D;
          vp = kp + sf_plane;
        }
      }
      s_kp[tid] = kp;
      s_vp[tid] = vp;
    }
    if (tid == 0 && base + ATT_CHUNK < hi && np == n) {
      // the cursor for the next chunk: the entry that holds slot `n` of this one
      int lo_e = 0, hi_e = ATT_ENTRIES;
      while (hi_e - lo_e > 1) {
        const int mid = (lo_e + hi_e) >> 1;
        if (e_cum[mid] <= n) lo_e = mid; else hi_e = mid;
      }
      s_misc[1] = e_first + lo_e;
      s_misc[2] = (lo_e == 0 ? e_off : 0) + (n - e_cum[lo_e]);
    }
    __syncthreads();
    // all rows of the chunk in one go; rows without a source (masked, or padding up to the 16-row
    // tile) are zeroed so that a zero weight times stale shared memory cannot make a NaN
    for (int i = warp * RPW + sub; i < n16; i += 8 * RPW) {
      const __nv_bfloat16* kp = s_kp[i];
      const int off = i * D + ((l_in ^ (i & 7)) << 3);
      if (kp) {
        cp_async16(s_k + off, kp + l_in * 8);
        cp_async16(s_v + off, s_vp[i] + l_in * 8);
      } else {
        *reinterpret_cast<uint4*>(s_k + off) = make_uint4(0, 0, 0, 0);
        *reinterpret_cast<uint4*>(s_v + off) = make_uint4(0, 0, 0, 0);
      }
    }
    cp_async_wait_all();
    // a prompt row counts only if its token is at or before the query's position (the position's
    // load has been in flight beside the row copies)
    if (tid < n16) s_ok[tid] = s_kp[tid] != nullptr && (!is_prompt || (long long)post <= q_pos);
    __syncthreads();
    for (int r0 = warp * 16; r0 < n16; r0 += 8 * 16) {
      // S^T = Q K^T for the tile's two 8-row groups
      float sc[2][4];
#pragma unroll
      for (int j = 0; j < 2; ++j) {
#pragma unroll
        for (int e = 0; e < 4; ++e) sc[j][e] = 0.f;
        const int row = r0 + 8 * j + (lane & 7);
        const __nv_bfloat16* krow = s_k + row * D;
#pragma unroll
        for (int kk = 0; kk < KSTEPS; kk += 2) {
          uint32_t b[4];
          ldmatrix_x4(b, krow + (((2 * kk + (lane >> 3)) ^ (row & 7)) << 3));
          mma_bf16_16816(sc[j], qa[kk][0], 0u, qa[kk][1], 0u, b[0], b[1]);
          mma_bf16_16816(sc[j], qa[kk + 1][0], 0u, qa[kk + 1][1], 0u, b[2], b[3]);
        }
      }
      // lane (g, t4) holds head g, rows r0 + 8 j + 2 t4 (+ 1)
      float tmax = -INFINITY;
#pragma unroll
      for (int j = 0; j < 2; ++j)
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          const bool ok = s_ok[r0 + 8 * j + 2 * t4 + e] != 0;
          sc[j][e] = ok ? sc[j][e] * a.sm_scale_log2 : -INFINITY;
          tmax = fmaxf(tmax, sc[j][e]);
        }
      tmax = fmaxf(tmax, __shfl_xor_sync(0xffffffffu, tmax, 1));
      tmax = fmaxf(tmax, __shfl_xor_sync(0xffffffffu, tmax, 2));
      const float m_new = fmaxf(m_run, tmax);
      const float alpha = (m_new == -INFINITY || m_run == m_new) ? 1.f
                          : (m_run == -INFINITY ? 0.f : sm100::fast_exp2(m_run - m_new));
      float p[2][2], psum = 0.f;
#pragma unroll
      for (int j = 0; j < 2; ++j)
#pragma unroll
        for (int e = 0; e < 2; ++e) {
          p[j][e] = m_new == -INFINITY ? 0.f : sm100::fast_exp2(sc[j][e] - m_new);
          psum += p[j][e];
        }
      l_part = l_part * alpha + psum;
      m_run = m_new;
      __nv_bfloat162 pb0 = __floats2bfloat162_rn(p[0][0], p[0][1]);
      __nv_bfloat162 pb1 = __floats2bfloat162_rn(p[1][0], p[1][1]);
      const uint32_t b0 = *reinterpret_cast<uint32_t*>(&pb0), b1 = *reinterpret_cast<uint32_t*>(&pb1);
      // the accumulator holds heads 2 t4 and 2 t4 + 1: their factors live in lanes 8 t4 and 8 t4 + 4
      const float al0 = __shfl_sync(0xffffffffu, alpha, 8 * t4), al1 = __shfl_sync(0xffffffffu, alpha, 8 * t4 + 4);
      if (__any_sync(0xffffffffu, alpha != 1.f)) {
#pragma unroll
        for (int nn = 0; nn < KSTEPS; ++nn) {
          o[nn][0] *= al0; o[nn][1] *= al1; o[nn][2] *= al0; o[nn][3] *= al1;
        }
      }
      // O^T += V^T P: V^T tiles come out of the row-major rows through the transposing load
      const int vrow = r0 + ((lane >> 4) << 3) + (lane & 7);
      const __nv_bfloat16* vbase = s_v + vrow * D;
#pragma unroll
      for (int nn = 0; nn < KSTEPS; ++nn) {
        uint32_t av[4];
        ldmatrix_x4_trans(av, vbase + (((2 * nn + ((lane >> 3) & 1)) ^ (vrow & 7)) << 3));
        mma_bf16_16816(o[nn], av[0], av[1], av[2], av[3], b0, b1);
      }
    }
    __syncthreads();                                    // the rows are consumed before the next chunk overwrites them
  }
  // this warp's partial: row sums over the four lanes of a head, then O^T into shared memory
  l_part += __shfl_xor_sync(0xffffffffu, l_part, 1);
  l_part += __shfl_xor_sync(0xffffffffu, l_part, 2);
  if (g < G && t4 == 0) { s_ml[(warp * G + g) * 2] = m_run; s_ml[(warp * G + g) * 2 + 1] = l_part; }
#pragma unroll
  for (int nn = 0; nn < KSTEPS; ++nn)
#pragma unroll
    for (int e = 0; e < 2; ++e) {
      const int head = 2 * t4 + e;
      if (head < G) {
        s_acc[(warp * G + head) * D + 16 * nn + g] = o[nn][e];
        s_acc[(warp * G + head) * D + 16 * nn + g + 8] = o[nn][2 + e];
      }
    }
  __syncthreads();
  for (int idx = tid; idx < G * D; idx += blockDim.x) {
    const int t = idx / D, d = idx % D;
    float mx = -INFINITY;
#pragma unroll
    for (int w = 0; w < 8; ++w) mx = fmaxf(mx, s_ml[(w * G + t) * 2]);
    float num = 0.f, den = 0.f;
#pragma unroll
    for (int w = 0; w < 8; ++w) {
      const float m_w = s_ml[(w * G + t) * 2];
      const float sc = m_w == -INFINITY ? 0.f : exp2f(m_w - mx);
      num += s_acc[(w * G + t) * D + d] * sc;
      den += s_ml[(w * G + t) * 2 + 1] * sc;
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
  if (tid == 0) {
    const int ticket = atomicAdd(&a.tickets[h], 1);
    s_misc[0] = ticket == nsplit - 1;
    if (s_misc[0]) a.tickets[h] = 0;                  // ready for the next step / graph replay
  }
  __syncthreads();
  if (!s_misc[0]) return;
  __threadfence();
  // Final merge by the head's last CTA.  Every thread owns four consecutive output columns of one
  // query head and has that column group of up to MERGE_SPLITS splits in flight at once; while those
  // loads travel, the splits' (max, sum) pairs are turned into weights in shared memory.
  constexpr int MERGE_SPLITS = 40;
  float* s_w = s_acc;                                  // [G][nsplit] weights, then [G] denominators
  float* s_mx = s_ml;                                  // [G] maxima
  for (int idx0 = 0; idx0 < G * D / 4; idx0 += blockDim.x) {
    const int idx = idx0 + tid;
    const bool live = idx < G * D / 4;
    const int t = live ? idx / (D / 4) : 0, d = live ? (idx % (D / 4)) * 4 : 0;
    const float4* src = reinterpret_cast<const float4*>(a.pacc + (int64_t)(h * G + t) * nsplit * D + d);
    float4 num = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int s0 = 0; s0 < nsplit; s0 += MERGE_SPLITS) {
      float4 v[MERGE_SPLITS];
#pragma unroll
      for (int i = 0; i < MERGE_SPLITS; ++i)
        v[i] = (live && s0 + i < nsplit) ? __ldcg(src + (int64_t)(s0 + i) * (D / 4)) : make_float4(0.f, 0.f, 0.f, 0.f);
      if (idx0 == 0 && s0 == 0) {
        // weights of every (head, split), once
        for (int i = tid; i < G * nsplit; i += blockDim.x) s_w[i] = __ldcg(a.pml + ((int64_t)h * G * nsplit + i) * 2);
        __syncthreads();
        if (tid < G) {
          float mx = -INFINITY;
          for (int s2 = 0; s2 < nsplit; ++s2) mx = fmaxf(mx, s_w[tid * nsplit + s2]);
          s_mx[tid] = mx;
        }
        __syncthreads();
        for (int i = tid; i < G * nsplit; i += blockDim.x) {
          const float m_s = s_w[i], mx = s_mx[i / nsplit];
          s_w[i] = m_s == -INFINITY ? 0.f : exp2f(m_s - mx);
        }
        __syncthreads();
        if (tid < G) {
          float den = 0.f;
          for (int s2 = 0; s2 < nsplit; ++s2)
            den += __ldcg(a.pml + ((int64_t)(h * G + tid) * nsplit + s2) * 2 + 1) * s_w[tid * nsplit + s2];
          s_w[G * nsplit + tid] = den;
        }
        __syncthreads();
      }
#pragma unroll
      for (int i = 0; i < MERGE_SPLITS; ++i) {
        const float sc = s0 + i < nsplit ? s_w[t * nsplit + s0 + i] : 0.f;
        num.x += v[i].x * sc; num.y += v[i].y * sc; num.z += v[i].z * sc; num.w += v[i].w * sc;
      }
    }
    if (live) {
      const float den = s_w[G * nsplit + t];
      const float inv = den == 0.f ? 0.f : 1.f / den;
      __nv_bfloat162 o01 = __floats2bfloat162_rn(num.x * inv, num.y * inv);
      __nv_bfloat162 o23 = __floats2bfloat162_rn(num.z * inv, num.w * inv);
      uint2 packed;
      packed.x = *reinterpret_cast<uint32_t*>(&o01);
      packed.y = *reinterpret_cast<uint32_t*>(&o23);
      *reinterpret_cast<uint2*>(a.out + (int64_t)(h * G + t) * D + d) = packed;
      if (a.lse_out && d == 0) a.lse_out[h * G + t] = den > 0.f ? (s_mx[t] + log2f(den)) * LN2 : -INFINITY;
    }
  }
}

int64_t align_up(int64_t x, int64_t a) { return (x + a - 1) / a * a; }

struct WsLayout {
  int64_t logit, ml, split, rstart, rlen, rcum, rcount, rtokens, pacc, pml, tickets, vectors, total;
};

WsLayout ws_layout(int hq, int hkv, int d, int c, int splits, int score_blocks) {
  const int g = hq / hkv;
  WsLayout w;
  int64_t off = 0;
  auto take = [&](int64_t bytes) { int64_t o = off; off = align_up(off + bytes, 256); return o; };
  w.tickets = take((int64_t)hkv * 4);
  w.logit = take((int64_t)hkv * g * c * 4);
  w.ml = take((int64_t)hkv * score_blocks * g * 2 * 4);
  w.split = take((int64_t)hkv * splits * 4 * 4);
  w.rstart = take((int64_t)hkv * c * 4);
  w.rlen = take((int64_t)hkv * c * 4);
  w.rcum = take((int64_t)hkv * c * 4);
  w.rcount = take((int64_t)hkv * 4);
  w.rtokens = take((int64_t)hkv * 4);
  w.pacc = take((int64_t)hq * splits * d * 4);
  w.pml = take((int64_t)hq * splits * 2 * 4);
  w.vectors = take((int64_t)hq * d * 2);
  w.total = off;
  return w;
}

int score_blocks_for(int hkv, int c) {
  int b = std::max(1, SCORE_BLOCKS_TARGET / std::max(hkv, 1));
  b = std::min(b, 128);                       // the select kernel folds the block partials four per lane
  b = std::min(b, std::max(1, c / 32));
  return b;
}

// Launch with the programmatic-dependent-launch attribute: the kernel may start while its
// predecessor in the stream is still running, and its griddepcontrol.wait holds it until the
// predecessor has completed.  `overlap` = 0 gives the plain stream-ordered launch.
template <typename Kernel>
int launch_decode_kernel(Kernel kern, dim3 grid, int threads, size_t smem, cudaStream_t st, int overlap,
                         const DecodeArgs& a) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = dim3(threads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = overlap ? 1 : 0;
  SEMBLO_CUDA(cudaLaunchKernelEx(&cfg, kern, a));
  return 0;
}

template <int D, int G>
int launch_attend(const DecodeArgs& a, dim3 grid, cudaStream_t st, int overlap) {
  auto kern = decode_attend_kernel<D, G>;
  SEMBLO_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, AttendSmem<D, G>::TOTAL));
  return launch_decode_kernel(kern, grid, 256, AttendSmem<D, G>::TOTAL, st, overlap, a);
}

}  // namespace

extern "C" int64_t semblo_decode_workspace_bytes(int num_q_heads, int num_kv_heads, int head_dim,
                                                 int num_clusters, int64_t packed_width,
                                                 int num_splits) {
  (void)packed_width;
  return ws_layout(num_q_heads, num_kv_heads, head_dim, num_clusters, num_splits,
                   score_blocks_for(num_kv_heads, num_clusters)).total;
}

extern "C" int semblo_decode_workspace_offsets(int num_q_heads, int num_kv_heads, int head_dim,
                                               int num_clusters, int64_t packed_width,
                                               int num_splits, int64_t* offsets /* [12] */) {
  (void)packed_width;
  const WsLayout w = ws_layout(num_q_heads, num_kv_heads, head_dim, num_clusters, num_splits,
                               score_blocks_for(num_kv_heads, num_clusters));
  const int64_t v[12] = {w.tickets, w.logit, w.ml, w.split, w.rstart, w.rlen, w.rcum,
                         w.rcount, w.rtokens, w.pacc, w.pml, w.vectors};
  for (int i = 0; i < 12; ++i) offsets[i] = v[i];
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
    int stage_mask, float* lse_out, int flags, void* stream) {
  SEMBLO_REQUIRE(num_kv_heads > 0 && num_q_heads % num_kv_heads == 0, "query heads must be a multiple of the KV heads");
  const int g = num_q_heads / num_kv_heads;
  SEMBLO_REQUIRE(g <= MAX_G, "at most %d query heads per KV head", MAX_G);
  SEMBLO_REQUIRE(prompt_length != nullptr, "the prompt length scalar is required");
  SEMBLO_REQUIRE(head_dim == 128 || head_dim == 256, "head_dim %d must be 128 or 256", head_dim);
  SEMBLO_REQUIRE(num_clusters >= 32 && num_clusters % 32 == 0 && num_clusters <= SEL_MAX_CLUSTERS,
                 "cluster count %d must be a multiple of 32 in [32, %d]", num_clusters, SEL_MAX_CLUSTERS);
  SEMBLO_REQUIRE(iters >= 1 && iters <= 16, "bisection steps %d outside [1, 16]", iters);
  SEMBLO_REQUIRE(temperature > 0.f && num_splits > 0, "temperature and split count must be positive");
  SEMBLO_REQUIRE((k_post == nullptr) == (v_new == nullptr), "key and value of the new token go together");
  SEMBLO_REQUIRE(((reinterpret_cast<uintptr_t>(k_post) | reinterpret_cast<uintptr_t>(v_new) |
                   reinterpret_cast<uintptr_t>(k_pre) | reinterpret_cast<uintptr_t>(q_post) |
                   reinterpret_cast<uintptr_t>(suffix_kv) | reinterpret_cast<uintptr_t>(suffix_kpre) |
                   reinterpret_cast<uintptr_t>(packed_kv)) & 15) == 0,
                 "the step's tensors and the stores must be 16-byte aligned");
  SEMBLO_REQUIRE(status != nullptr, "status word is required");
  const int sblocks = score_blocks_for(num_kv_heads, num_clusters);
  const WsLayout w = ws_layout(num_q_heads, num_kv_heads, head_dim, num_clusters, num_splits, sblocks);
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
  a.ws_logit = (float*)(ws + w.logit); a.ws_ml = (float*)(ws + w.ml);
  a.split_start = (int32_t*)(ws + w.split);
  a.rstart = (int32_t*)(ws + w.rstart); a.rlen = (int32_t*)(ws + w.rlen); a.rcum = (int32_t*)(ws + w.rcum);
  a.rcount = (int32_t*)(ws + w.rcount); a.rtokens = (int32_t*)(ws + w.rtokens);
  a.pacc = (float*)(ws + w.pacc); a.pml = (float*)(ws + w.pml);
  a.tickets = (int32_t*)(ws + w.tickets); a.vectors = (__nv_bfloat16*)(ws + w.vectors);
  a.out = (__nv_bfloat16*)output; a.status = status;
  a.lse_out = lse_out; a.vectors_given = flags & 1;
  a.tile_starts = a.tile_lengths = a.tile_counts = a.tile_posting = nullptr;
  a.tile_stride = a.token_tile = 0; a.tile_posting_stride = 0;
  a.cache = nullptr; a.cache_plane = 0; a.block_table = nullptr; a.block_size = 1; a.block_table_len = 0;
  cudaStream_t st = (cudaStream_t)stream;
  // bit 3 of the stage mask turns the overlapped (programmatic dependent) launches off; a stage
  // launched alone has no predecessor of this step to overlap with
  const int overlap = (stage_mask & 8) ? 0 : 1;
  if (stage_mask & 1) {
    const dim3 sgrid(num_kv_heads, sblocks + 1);
    if (head_dim == 256 && g == 4) decode_score_kernel<256, 4><<<sgrid, 256, 0, st>>>(a);
    else if (head_dim == 128 && g == 4) decode_score_kernel<128, 4><<<sgrid, 256, 0, st>>>(a);
    else if (head_dim == 128 && g == 8) decode_score_kernel<128, 8><<<sgrid, 256, 0, st>>>(a);
    else return semblo::fail(semblo::SEMBLO_EINVAL, "decode scoring supports head_dim 256 with 4, or 128 with 4 or 8, query heads per KV head (got %d, %d)", head_dim, g);
    SEMBLO_LAUNCH_CHECK();
  }
  if (stage_mask & 2) {
    int rc = launch_decode_kernel(decode_select_kernel, dim3(SEL_CL, num_kv_heads), SEL_THREADS, 0, st,
                                  overlap && (stage_mask & 1), a);
    if (rc) return rc;
  }
  if (stage_mask & 4) {
    const dim3 grid(num_kv_heads, num_splits);
    const int ov = overlap && (stage_mask & 2);
    int rc;
    if (head_dim == 256 && g == 4) rc = launch_attend<256, 4>(a, grid, st, ov);
    else if (head_dim == 128 && g == 4) rc = launch_attend<128, 4>(a, grid, st, ov);
    else if (head_dim == 128 && g == 8) rc = launch_attend<128, 8>(a, grid, st, ov);
    else return semblo::fail(semblo::SEMBLO_EINVAL, "decode attention supports head_dim 256 with 4, or 128 with 4 or 8, query heads per KV head (got %d, %d)", head_dim, g);
    if (rc) return rc;
  }
  SEMBLO_LAUNCH_CHECK();
  return 0;
}

// ---------------------------------------------------------------------- paged posting attention
namespace {

// Exact merge of two attention states over disjoint key sets (paged_attention.py:50-78): one thread
// per output element pair.
__global__ void merge_states_kernel(const __nv_bfloat16* __restrict__ out_a, const float* __restrict__ lse_a,
                                    const __nv_bfloat16* __restrict__ out_b, const float* __restrict__ lse_b,
                                    int64_t rows, int dim, __nv_bfloat16* __restrict__ out, float* __restrict__ lse) {
  const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  const int half = dim / 2;
  if (idx >= rows * half) return;
  const int64_t r = idx / half;
  const int c = (int)(idx % half) * 2;
  const float la = lse_a[r], lb = lse_b[r];
  const float m = fmaxf(la, lb);
  float wa = 0.f, wb = 0.f, merged = -INFINITY;
  if (m != -INFINITY) {
    const float ea = expf(la - m), eb = expf(lb - m);
    merged = m + logf(ea + eb);
    wa = ea / (ea + eb);
    wb = eb / (ea + eb);
  }
  const float2 a2 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(out_a + r * dim + c));
  const float2 b2 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(out_b + r * dim + c));
  *reinterpret_cast<__nv_bfloat162*>(out + r * dim + c) = __floats2bfloat162_rn(a2.x * wa + b2.x * wb, a2.y * wa + b2.y * wb);
  if (c == 0) lse[r] = merged;
}

}  // namespace

extern "C" int semblo_merge_attention_states(const void* out_a, const float* lse_a, const void* out_b,
                                             const float* lse_b, int64_t rows, int head_dim, void* out,
                                             float* lse, void* stream) {
  SEMBLO_REQUIRE(out_a && out_b && lse_a && lse_b && out && lse, "both states and the two outputs are required");
  SEMBLO_REQUIRE(head_dim > 0 && head_dim % 2 == 0, "head_dim %d must be even", head_dim);
  if (rows == 0) return 0;
  const int64_t n = rows * (head_dim / 2);
  merge_states_kernel<<<(unsigned)ceil_div(n, 256), 256, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)out_a, lse_a, (const __nv_bfloat16*)out_b, lse_b, rows, head_dim, (__nv_bfloat16*)out, lse);
  SEMBLO_LAUNCH_CHECK();
  return 0;
}

extern "C" int64_t semblo_paged_attention_workspace_bytes(int num_q_heads, int num_kv_heads, int head_dim, int num_splits) {
  return ws_layout(num_q_heads, num_kv_heads, head_dim, 32, num_splits, 1).total;
}

extern "C" int semblo_paged_posting_attention(
    const void* q, const void* q_position, int pos_is_int64, const void* kv_cache, int64_t cache_blocks,
    int block_size, const int32_t* block_table, int block_table_len, const int32_t* posting_positions,
    int64_t posting_stride, const int32_t* tile_starts, const int32_t* tile_lengths, const int32_t* tile_counts,
    int tile_stride, int token_tile, int num_q_heads, int num_kv_heads, int head_dim, float sm_scale,
    int num_splits, void* workspace, int64_t workspace_bytes, void* output, float* lse_out, int32_t* status,
    void* stream) {
  SEMBLO_REQUIRE(num_kv_heads > 0 && num_q_heads % num_kv_heads == 0, "query heads must be a multiple of the KV heads");
  const int g = num_q_heads / num_kv_heads;
  SEMBLO_REQUIRE(q && q_position && kv_cache && block_table && posting_positions && tile_starts && tile_lengths &&
                     tile_counts && output && status,
                 "query, position, cache, block table, posting tiles, output and status word are required");
  SEMBLO_REQUIRE(block_size > 0 && token_tile > 0 && num_splits > 0 && tile_stride >= 0, "bad block, tile or split size");
  SEMBLO_REQUIRE(((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(kv_cache)) & 15) == 0,
                 "the query and the cache must be 16-byte aligned");
  const WsLayout w = ws_layout(num_q_heads, num_kv_heads, head_dim, 32, num_splits, 1);
  SEMBLO_REQUIRE(workspace_bytes >= w.total, "workspace has %lld bytes, %lld needed", (long long)workspace_bytes,
                 (long long)w.total);
  uint8_t* ws = (uint8_t*)workspace;
  DecodeArgs a = {};
  a.num_q_heads = num_q_heads; a.num_kv_heads = num_kv_heads; a.head_dim = head_dim; a.num_clusters = 32; a.group = g;
  a.q_post = (const __nv_bfloat16*)q;
  a.positions = q_position; a.pos_is_int64 = pos_is_int64;
  a.packed_width = 0; a.suffix_blocks = 0; a.suffix_block = 1; a.table_len = 0; a.prompt_length = nullptr;
  a.sm_scale_log2 = sm_scale * LOG2E; a.num_splits = num_splits;
  a.split_start = (int32_t*)(ws + w.split); a.rstart = (int32_t*)(ws + w.rstart); a.rlen = (int32_t*)(ws + w.rlen);
  a.pacc = (float*)(ws + w.pacc); a.pml = (float*)(ws + w.pml); a.tickets = (int32_t*)(ws + w.tickets);
  a.out = (__nv_bfloat16*)output; a.lse_out = lse_out; a.status = status;
  a.tile_starts = tile_starts; a.tile_lengths = tile_lengths; a.tile_counts = tile_counts;
  a.tile_stride = tile_stride; a.token_tile = token_tile;
  a.tile_posting = posting_positions; a.tile_posting_stride = posting_stride;
  a.cache = (const __nv_bfloat16*)kv_cache;
  a.cache_plane = cache_blocks * (int64_t)block_size * num_kv_heads * head_dim;
  a.block_table = block_table; a.block_size = block_size; a.block_table_len = block_table_len;
  const dim3 grid(num_kv_heads, num_splits);
  cudaStream_t st = (cudaStream_t)stream;
  int rc;
  if (head_dim == 256 && g == 4) rc = launch_attend<256, 4>(a, grid, st, 0);
  else if (head_dim == 128 && g == 4) rc = launch_attend<128, 4>(a, grid, st, 0);
  else if (head_dim == 128 && g == 8) rc = launch_attend<128, 8>(a, grid, st, 0);
  else return semblo::fail(semblo::SEMBLO_EINVAL, "paged posting attention supports head_dim 256 with 4, or 128 with 4 or 8, query heads per KV head (got %d, %d)", head_dim, g);
  if (rc) return rc;
  SEMBLO_LAUNCH_CHECK();
  return 0;
}
