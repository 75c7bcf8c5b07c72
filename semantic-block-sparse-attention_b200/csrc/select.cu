// Query . centroid scoring and budgeted cluster selection for prefill chunks.
//
//   score kernel : [QT queries x G heads = 128 rows, D] x [D, C] on tcgen05 (TMA-fed,
//                  TMEM accumulators), two passes over the codebook: pass 0 gives each
//                  row's log-sum-exp over the clusters, pass 1 turns the logits into
//                  softmax probabilities, sums them over the G heads of the KV head
//                  (lane butterfly) and writes the penalised log score
//                  log(max(P, 1e-38)) - beta log(1 + n_c)   (-3.4e38 where n_c = 0).
//   select kernel: one warp per (query, KV head): the 16-step bisection for the score
//                  threshold and the packed bitmask of the clusters at or above it.
//
// Reference behaviour restated here:
//   semblo/vllm_plugin/fused_select.py:1061-1247  _flat_scores_qtiled_kernel
//   semblo/vllm_plugin/fused_select.py:604-647    _streaming_select_kernel (resident branch)
//   semblo/vllm_plugin/fused_prefill.py:202-216   sink hold-out and forced bit
#include <algorithm>

#include "../../include/semblo_b200.h"
#include "host_common.h"
#include "attn_common.cuh"
#include <cstdlib>
#include "sm100.cuh"

using namespace sm100;
using semblo::ceil_div;
using semblo::sm_count;

namespace {

constexpr int SC_BN = 64;                 // centroids per accumulator: two CTAs share an SM (tensor memory 2 x 256 columns)
constexpr int SC_STAGES = 2;
constexpr float NEG_BIG = -3.4e38f;
constexpr float LOG2E = 1.4426950408889634f;
constexpr float LN2 = 0.6931471805599453f;

template <int D>
struct ScoreSmem {
  static constexpr int B_BYTES = SC_BN * D * 2;
  static constexpr int BAR_OFF = SC_STAGES * B_BYTES;
  static constexpr int Q_COL = 2 * SC_BN;            // TMEM: two accumulators, then the routing vectors (D / 2 columns)
  static constexpr int TMEM_COLS = Q_COL + D / 2 <= 256 ? 256 : 512;   // allocation: a power of two
  static_assert(Q_COL + D / 2 <= TMEM_COLS, "tensor memory budget");
  static constexpr int XCHG_OFF = BAR_OFF + 256;               // float [2][128][2]: (max, sum) of a half-row
  static constexpr int TOTAL = XCHG_OFF + 2048 + 1024;
};

// Sum v[] over the G adjacent lanes that hold the G heads of one query; afterwards
// v[0 .. 32/G) are complete sums and the returned value is the column offset of v[0].
template <int G>
__device__ __forceinline__ int head_butterfly(float (&v)[32], int lane) {
  int col = 0;
  int width = 32;
#pragma unroll
  for (int bit = 1; bit < G; bit <<= 1) {
    const int half = width >> 1;
    const bool up = (lane & bit) != 0;
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      if (i < half) {
        const float send = up ? v[i] : v[i + half];
        const float keep = up ? v[i + half] : v[i];
        v[i] = keep + __shfl_xor_sync(0xffffffffu, send, bit);
      }
    }
    col += up ? half : 0;
    width = half;
  }
  return col;
}

template <int D, int G>
__global__ void __launch_bounds__(320, SC_BN <= 64 ? 2 : 1)
score_kernel(const __nv_bfloat16* __restrict__ vectors,      // [Q, Hq, D] bf16
             const __grid_constant__ CUtensorMap tmap_cb,   // codebooks [Hkv*2, C, D/2] bf16, box (64, 128, 1)
             int num_queries, int num_clusters, const int32_t* __restrict__ sizes,   // [Hkv, C]
             float scale_log2,                     // log2(e) / temperature
             float beta, float* __restrict__ score,          // [Q, Hkv, C]
             int num_kv_heads, int* __restrict__ status) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  using L = ScoreSmem<D>;
  constexpr int SLABS = D / 64;
  constexpr int SLABS_PER_HALF = SLABS / 2;
  constexpr int QT = 128 / G;
  uint8_t* b_smem = smem;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::BAR_OFF);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 16);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  float* xchg = reinterpret_cast<float*>(smem + L::XCHG_OFF);
  // bars: 0 a_full (the routing vectors are in tensor memory), 1..2 b_full, 3..4 b_empty, 5..6 acc_full, 7..8 acc_empty, 9 epilogue rendezvous

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int h = blockIdx.y;
  const int q0 = blockIdx.x * QT;
  const int chunks = (num_clusters + SC_BN - 1) / SC_BN;
  const int total = 2 * chunks;                    // two passes over the codebook

  if (threadIdx.x == 0) {
    mbar_init(smem_u32(&bars[0]), 256);
    for (int s = 0; s < SC_STAGES; ++s) {
      mbar_init(smem_u32(&bars[1 + s]), 1);
      mbar_init(smem_u32(&bars[3 + s]), 1);
      mbar_init(smem_u32(&bars[5 + s]), 1);
      mbar_init(smem_u32(&bars[7 + s]), 8);        // the epilogue warps (one arrival each, by lane 0)
    }
    mbar_init(smem_u32(&bars[9]), 256);
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 0) {
    tmem_alloc(smem_u32(tmem_slot), L::TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 8) {
    if (elect_one()) {
      tma_prefetch_desc(&tmap_cb);
      for (int j = 0; j < total; ++j) {
        const int s = j % SC_STAGES;
        if (!mbar_wait(smem_u32(&bars[3 + s]), ((j / SC_STAGES) & 1) ^ 1, abort_flag, status, STATUS_TIMEOUT_LOAD))
          break;
        mbar_arrive_expect_tx(smem_u32(&bars[1 + s]), L::B_BYTES);
        const int c0 = (j % chunks) * SC_BN;
        for (int sl = 0; sl < SLABS; ++sl)
          tma_load_3d(smem_u32(b_smem + s * L::B_BYTES + sl * SC_BN * 128), &tmap_cb,
                      smem_u32(&bars[1 + s]), (sl % SLABS_PER_HALF) * 64, c0, h * 2 + sl / SLABS_PER_HALF);
      }
    }
  } else if (warp == 9) {
    if (elect_one()) {
      constexpr uint32_t idesc = make_idesc_bf16(128, SC_BN, false, false);
      bool ok = mbar_wait(smem_u32(&bars[0]), 0, abort_flag, status, STATUS_TIMEOUT_MMA);
      for (int j = 0; ok && j < total; ++j) {
        const int s = j % SC_STAGES, b = j & 1;
        if (!mbar_wait(smem_u32(&bars[1 + s]), (j / SC_STAGES) & 1, abort_flag, status, STATUS_TIMEOUT_MMA)) break;
        if (!mbar_wait(smem_u32(&bars[7 + b]), ((j >> 1) & 1) ^ 1, abort_flag, status, STATUS_TIMEOUT_MMA)) break;
        tc_fence_after();
        const uint32_t b_base = smem_u32(b_smem + s * L::B_BYTES);
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint32_t sl = kk >> 2, ko = (kk & 3) * 32;
          umma_ts(tmem_base + b * SC_BN, tmem_base + L::Q_COL + kk * 8,
                  make_smem_desc(b_base + sl * SC_BN * 128 + ko, 16, 1024), idesc, kk > 0 ? 1u : 0u);
        }
        umma_commit(smem_u32(&bars[3 + s]));
        umma_commit(smem_u32(&bars[5 + b]));
      }
    }
  } else {
    // epilogue warps 0-7: thread = (half, row); query i = row / G, head t = row % G.  The two
    // warps that share 32 rows split every chunk of SC_BN clusters: half 0 takes its first columns.
    constexpr int CC = SC_BN / 64;                 // 32-column groups per thread and chunk
    const int hf = warp >> 2;
    const int row = threadIdx.x & 127;
    const int qi = q0 + row / G;
    // the routing vectors go to tensor memory once: each of the two threads of a row copies half
    // of its dims (rows past the last query are zero)
    attn::stage_q_half<D, L::Q_COL>(
        qi < num_queries ? vectors + ((int64_t)qi * (num_kv_heads * G) + h * G + row % G) * D + hf * (D / 2) : nullptr, hf,
        (uint32_t)((warp & 3) * 32) << 16, tmem_base, smem_u32(&bars[0]));
    // Routing vectors and descriptors are unit vectors (up to bf16 rounding), so every logit is
    // bounded by 1.01 * scale: with a moderate scale the log-sum-exp needs no running maximum.
    const bool fixed_max = scale_log2 <= 60.f;
    const float m_fixed = 1.01f * scale_log2;
    float m_run = fixed_max ? m_fixed : -INFINITY, l_run = 0.f, lse2 = 0.f;
    const int32_t* sz = sizes + (int64_t)h * num_clusters;
    // column offset of this lane's share after the head butterfly (depends on the lane only)
    int col_off = 0;
    {
      int width = 32;
#pragma unroll
      for (int bit = 1; bit < G; bit <<= 1) {
        width >>= 1;
        col_off += (lane & bit) ? width : 0;
      }
    }
    constexpr int OUT = 32 / G;                    // outputs per thread per 32 columns
    bool ok = true;
    for (int j = 0; j < total && ok; ++j) {
      const int b = j & 1;
      const int pass = j / chunks;
      const int c0 = (j % chunks) * SC_BN;
      const bool full_chunk = c0 + SC_BN <= num_clusters;
      // sizes of this thread's output clusters, fetched before the accumulator is awaited
      int nsz[CC][OUT];
      if (pass == 1) {
#pragma unroll
        for (int cc = 0; cc < CC; ++cc)
#pragma unroll
          for (int i = 0; i < OUT; ++i) {
            const int c = c0 + (CC * hf + cc) * 32 + col_off + i;
            nsz[cc][i] = c < num_clusters ? sz[c] : 0;
          }
      }
      ok = mbar_wait_warp(smem_u32(&bars[5 + b]), (j >> 1) & 1, abort_flag, status, STATUS_TIMEOUT_EPILOGUE);
      if (!ok) break;
      tc_fence_after();
      if (j == chunks) {
        // both halves of a row combine their (max, sum) before the second pass
        xchg[(hf * 128 + row) * 2] = m_run;
        xchg[(hf * 128 + row) * 2 + 1] = l_run;
        mbar_arrive(smem_u32(&bars[9]));
        ok = mbar_wait_warp(smem_u32(&bars[9]), 0, abort_flag, status, STATUS_TIMEOUT_EPILOGUE);
        if (!ok) break;
        const float m_o = xchg[((hf ^ 1) * 128 + row) * 2], l_o = xchg[((hf ^ 1) * 128 + row) * 2 + 1];
        const float mx = fmaxf(m_run, m_o);
        const float l_all = (m_run == -INFINITY ? 0.f : l_run * fast_exp2(m_run - mx)) +
                            (m_o == -INFINITY ? 0.f : l_o * fast_exp2(m_o - mx));
        lse2 = mx + __log2f(l_all);
      }
      const float neg_ref = pass == 0 ? -m_run : -lse2;
#pragma unroll
      for (int cc = 0; cc < CC; ++cc) {
        const int c4 = CC * hf + cc;
        uint32_t r[32];
        tmem_ld32(tmem_base + ((uint32_t)((warp & 3) * 32) << 16) + b * SC_BN + c4 * 32, r);
        tmem_ld_wait();
        const int cbase = c0 + c4 * 32;
        if (pass == 0) {
          if (fixed_max) {
            float add = 0.f;
#pragma unroll
            for (int i = 0; i < 32; ++i) {
              const float e = fast_exp2(fmaf(__uint_as_float(r[i]), scale_log2, neg_ref));
              add += (full_chunk || cbase + i < num_clusters) ? e : 0.f;
            }
            l_run += add;
          } else {
            float mx = m_run;
#pragma unroll
            for (int i = 0; i < 32; ++i) {
              float s2 = __uint_as_float(r[i]) * scale_log2;
              s2 = (full_chunk || cbase + i < num_clusters) ? s2 : -INFINITY;
              r[i] = __float_as_uint(s2);
              mx = fmaxf(mx, s2);
            }
            float add = 0.f;
#pragma unroll
            for (int i = 0; i < 32; ++i) add += fast_exp2(__uint_as_float(r[i]) - mx);
            l_run = l_run * fast_exp2(m_run - mx) + add;
            m_run = mx;
          }
        } else {
          float v[32];
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] = fast_exp2(fmaf(__uint_as_float(r[i]), scale_log2, neg_ref));
          head_butterfly<G>(v, lane);
          if (qi < num_queries) {
            float* dst = score + ((int64_t)qi * num_kv_heads + h) * num_clusters + cbase + col_off;
            float o[OUT];
#pragma unroll
            for (int i = 0; i < OUT; ++i) {
              const float n = (float)nsz[cc][i];
              float sc = __log2f(fmaxf(v[i], 1e-38f)) * LN2;
              if (beta != 0.f) sc -= beta * (__log2f(1.0f + n) * LN2);
              o[i] = n > 0.f ? sc : NEG_BIG;
            }
            if (full_chunk && OUT % 4 == 0) {
#pragma unroll
              for (int i = 0; i < OUT; i += 4)
                *reinterpret_cast<float4*>(dst + i) = make_float4(o[i], o[i + 1], o[i + 2], o[i + 3]);
            } else {
#pragma unroll
              for (int i = 0; i < OUT; ++i)
                if (cbase + col_off + i < num_clusters) dst[i] = o[i];
            }
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if ((threadIdx.x & 31) == 0) mbar_arrive(smem_u32(&bars[7 + b]));
    }
  }
  __syncthreads();
  if (*abort_flag) __nanosleep(50000);
  if (warp == 0) tmem_dealloc(tmem_base, L::TMEM_COLS);
}

// ---------------------------------------------------------------- threshold selection
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ float warp_min(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fminf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ float warp_sumf(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// The key whose arg-max orders the attention tiles: the score with `key_beta` log(1 + n) added back.
// With key_beta = the penalty's beta that is the cluster of the largest mixture probability, which
// groups queries by where they point and not by which small cluster the size penalty favours;
// key_beta = 0 is the arg-max of the score itself.
__device__ __forceinline__ float tile_key(float score, float n, float key_beta) {
  return key_beta != 0.f && n > 0.f ? score + key_beta * __logf(1.0f + n) : score;
}

// One warp per (query, KV head).  Dynamic smem: sizes of the head [C] floats, then one
// [C] float score row per warp.
__global__ void select_kernel(const float* __restrict__ score,      // [Q, Hkv, C]
                              const int32_t* __restrict__ sizes,    // [Hkv, C] (sink held out)
                              int num_queries, int num_kv_heads, int num_clusters,
                              float target_tokens, int iters, int force_sink, float key_beta,
                              int32_t* __restrict__ qmask,          // [Q, Hkv, C/32]
                              int32_t* __restrict__ counts,         // [Q, Hkv] or null
                              int32_t* __restrict__ tokens,         // [Q, Hkv] or null
                              int32_t* __restrict__ top1) {         // [Hkv, Q] or null: the tile-order key
  extern __shared__ float sm[];
  const int warps = blockDim.x >> 5, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int h = blockIdx.y;
  float* s_size = sm;
  float* s_score = sm + num_clusters + (int64_t)warp * num_clusters;
  for (int c = threadIdx.x; c < num_clusters; c += blockDim.x)
    s_size[c] = (float)sizes[(int64_t)h * num_clusters + c];
  __syncthreads();
  const int q = blockIdx.x * warps + warp;
  if (q >= num_queries) return;
  const float* row = score + ((int64_t)q * num_kv_heads + h) * num_clusters;
  float mx = -INFINITY, mn = 3.4e38f, tot = 0.f, kmx = -INFINITY;
  int arg = 0;
  for (int c = lane; c < num_clusters; c += 32) {
    const float s = row[c], n = s_size[c];
    s_score[c] = s;
    const float key = tile_key(s, n, key_beta);
    if (key > kmx) { kmx = key; arg = c; }
    mx = fmaxf(mx, s);
    mn = fminf(mn, n > 0.f ? s : 3.4e38f);
    tot += n > 0.f ? n : 0.f;
  }
  __syncwarp();
  if (top1) {
    // lowest cluster id among the maxima of the key: a grouping key for the attention tiles
    const float best = warp_max(kmx);
    int cand = kmx == best ? arg : 0x7fffffff;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) cand = min(cand, __shfl_xor_sync(0xffffffffu, cand, o));
    if (lane == 0) top1[(int64_t)h * num_queries + q] = cand;
  }
  float hi = warp_max(mx) + 1e-6f;
  float lo = warp_min(mn) - 1e-6f;
  lo = fminf(lo, hi - 1e-5f);
  const bool all_fit = warp_sumf(tot) < target_tokens;
  for (int it = 0; it < iters; ++it) {
    const float mid = (lo + hi) * 0.5f;
    float above = 0.f;
    for (int c = lane; c < num_clusters; c += 32) above += s_score[c] >= mid ? s_size[c] : 0.f;
    above = warp_sumf(above);
    const bool reach = above >= target_tokens;
    lo = reach ? mid : lo;
    hi = reach ? hi : mid;
  }
  const float theta = all_fit ? NEG_BIG : lo;
  int32_t* qm = qmask + ((int64_t)q * num_kv_heads + h) * (num_clusters >> 5);
  int n_sel = 0;
  float n_tok = 0.f;
  for (int w = 0; w < (num_clusters >> 5); ++w) {
    const int c = w * 32 + lane;
    const bool sel = s_size[c] > 0.f && s_score[c] >= theta;
    unsigned bits = __ballot_sync(0xffffffffu, sel);
    n_sel += __popc(bits);
    n_tok += sel ? s_size[c] : 0.f;
    if (w == 0 && force_sink) bits |= 1u;
    if (lane == 0) qm[w] = (int32_t)bits;
  }
  n_tok = warp_sumf(n_tok);
  if (lane == 0) {
    if (counts) counts[(int64_t)q * num_kv_heads + h] = n_sel;
    if (tokens) tokens[(int64_t)q * num_kv_heads + h] = (int)n_tok;
  }
}

// acc += n where s >= mid: one compare (integer pipe) and one predicated fp32 add (FMA pipe).
__device__ __forceinline__ void add_if_ge(float& acc, float s, float mid, float n) {
  asm("{\n\t.reg .pred p;\n\tsetp.ge.f32 p, %1, %2;\n\t@p add.f32 %0, %0, %3;\n\t}" : "+f"(acc) : "f"(s), "f"(mid), "f"(n));
}

constexpr int SELECT_REG_WARPS = 4;

// Register-resident form for C = 32 * PER <= 2048: a warp keeps a whole score row and the sizes in
// registers, so a bisection step is a compare and a predicated add per cluster.  The kernel is bound
// by the integer pipe (compares, selects, votes), so everything that is the same for all rows of a
// head is tabulated once per block in shared memory — the size term of the tile-order key, the sizes
// as fp32 and a 0 / -inf mask of the empty clusters that is added to the scores once — and a block
// walks over many rows.
template <int PER>
__global__ void __launch_bounds__(SELECT_REG_WARPS * 32, PER >= 64 ? 3 : 4)
select_kernel_reg(const float* __restrict__ score, const int32_t* __restrict__ sizes, int num_queries,
                  int num_kv_heads, float target_tokens, int iters, int force_sink, float key_beta,
                  int32_t* __restrict__ qmask, int32_t* __restrict__ counts,
                  int32_t* __restrict__ tokens, int32_t* __restrict__ top1) {
  constexpr int C = PER * 32;
  __shared__ float s_pen[C], s_ninf[C], s_size[C];
  __shared__ unsigned s_bits[SELECT_REG_WARPS][PER];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int h = blockIdx.y;
  const int32_t* sz = sizes + (int64_t)h * C;
  for (int c = threadIdx.x; c < C; c += blockDim.x) {
    const float n = (float)sz[c];
    s_size[c] = n;
    s_ninf[c] = n > 0.f ? 0.f : -INFINITY;
    s_pen[c] = key_beta != 0.f && n > 0.f ? key_beta * __logf(1.0f + n) : 0.f;
  }
  __syncthreads();
  const int target_i = (int)target_tokens;
  for (int q = blockIdx.x * SELECT_REG_WARPS + warp; q < num_queries; q += gridDim.x * SELECT_REG_WARPS) {
    const float* row = score + ((int64_t)q * num_kv_heads + h) * C;
    float sc[PER], nn[PER];
#pragma unroll
    for (int i = 0; i < PER; ++i) sc[i] = __ldcs(row + i * 32 + lane);       // read once
    float mx = -INFINITY, mn = INFINITY, tot = 0.f, kmx = -INFINITY;
    int arg = 0;
#pragma unroll
    for (int i = 0; i < PER; ++i) {
      const int c = i * 32 + lane;
      const float s = sc[i], ninf = s_ninf[c];
      nn[i] = s_size[c];
      const float key = s + s_pen[c];
      if (key > kmx) { kmx = key; arg = i; }        // ascending ids: the first maximum stays
      mx = fmaxf(mx, s);
      mn = fminf(mn, s - ninf);                     // +inf for an empty cluster
      tot += nn[i];
      sc[i] = s + ninf;                             // -inf for an empty cluster: never above a threshold
    }
    const float best = warp_max(mx);
    if (top1) {
      const float kbest = warp_max(kmx);
      int cand = kmx == kbest ? arg * 32 + lane : 0x7fffffff;
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) cand = min(cand, __shfl_xor_sync(0xffffffffu, cand, o));
      if (lane == 0) top1[(int64_t)h * num_queries + q] = cand;
    }
    float hi = best + 1e-6f;
    float lo = warp_min(mn) - 1e-6f;
    lo = fminf(lo, hi - 1e-5f);
    const float row_total = warp_sumf(tot);
    const bool all_fit = row_total < target_tokens;
    // The sums of sizes are sums of small integers: exact in any order, and exact in fp32 while the
    // row's total stays below 2^24; longer rows take the same loop on integers.
    if (row_total < 16777216.f) {
      for (int it = 0; it < iters; ++it) {
        const float mid = (lo + hi) * 0.5f;
        float ab[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int i = 0; i < PER; ++i) add_if_ge(ab[i & 3], sc[i], mid, nn[i]);
        const int above = __reduce_add_sync(0xffffffffu, (int)((ab[0] + ab[1]) + (ab[2] + ab[3])));
        const bool reach = above >= target_i;
        lo = reach ? mid : lo;
        hi = reach ? hi : mid;
      }
    } else {
      for (int it = 0; it < iters; ++it) {
        const float mid = (lo + hi) * 0.5f;
        int ab[4] = {0, 0, 0, 0};
#pragma unroll
        for (int i = 0; i < PER; ++i) ab[i & 3] += sc[i] >= mid ? __ldg(sz + i * 32 + lane) : 0;
        const int above = __reduce_add_sync(0xffffffffu, (ab[0] + ab[1]) + (ab[2] + ab[3]));
        const bool reach = above >= target_i;
        lo = reach ? mid : lo;
        hi = reach ? hi : mid;
      }
    }
    const float theta = all_fit ? NEG_BIG : lo;
    float n_tok = 0.f;
    __syncwarp();                                   // the previous row's words have been read
#pragma unroll
    for (int i = 0; i < PER; ++i) {
      const unsigned bits = __ballot_sync(0xffffffffu, sc[i] >= theta);
      add_if_ge(n_tok, sc[i], theta, nn[i]);
      if (lane == 0) s_bits[warp][i] = bits;
    }
    __syncwarp();
    int32_t* qm = qmask + ((int64_t)q * num_kv_heads + h) * PER;
    int n_sel = 0;
    for (int w = lane; w < PER; w += 32) {
      unsigned bits = s_bits[warp][w];
      n_sel += __popc(bits);
      if (w == 0 && force_sink) bits |= 1u;
      qm[w] = (int32_t)bits;
    }
    if (counts || tokens) {
      n_sel = __reduce_add_sync(0xffffffffu, n_sel);
      n_tok = warp_sumf(n_tok);
      if (lane == 0) {
        if (counts) counts[(int64_t)q * num_kv_heads + h] = n_sel;
        if (tokens) tokens[(int64_t)q * num_kv_heads + h] = (int)n_tok;
      }
    }
  }
}

// Wide form for C = 512 * PER (4096, 8192, 16384 clusters): the 512 threads of a CTA hold ROWS
// (query, head) score rows at once (PER scores of each per thread, four consecutive clusters per
// 16-byte load) and the head's sizes once, all in registers; a bisection step is one compare and one
// predicated fp32 add per cluster and row, and the block-wide sums of all ROWS rows share one barrier.
// The per-head tables (the 0 / -inf mask of the empty clusters, the size term of the tile key) are made
// once per CTA, which then walks groups of rows.  Same arithmetic as select_kernel_reg: sums of
// integers below 2^24 in fp32 are exact in any order (heads with a larger total take integer sums).
constexpr int SELECT_WIDE_THREADS = 512;
constexpr int SELECT_WIDE_WARPS = SELECT_WIDE_THREADS / 32;
template <int PER, int ROWS>
__global__ void __launch_bounds__(SELECT_WIDE_THREADS, 1)
select_kernel_wide(const float* __restrict__ score, const int32_t* __restrict__ sizes, int num_queries,
                   int num_kv_heads, float target_tokens, int iters, int force_sink, float key_beta,
                   int32_t* __restrict__ qmask, int32_t* __restrict__ counts, int32_t* __restrict__ tokens,
                   int32_t* __restrict__ top1) {
  constexpr int T = SELECT_WIDE_THREADS;
  constexpr int C = PER * T;
  constexpr int W = SELECT_WIDE_WARPS;
  extern __shared__ float s_tab[];                         // [2][C]: size term of the key, empty-cluster mask
  float* s_pen = s_tab;
  float* s_ninf = s_tab + C;
  __shared__ float red_f[2][ROWS][3][W];                   // [flip][row][max, min, key][warp]
  __shared__ int red_i[2][ROWS][W];                        // [flip][row][warp]
  __shared__ float s_total;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int h = blockIdx.y;
  const int32_t* sz = sizes + (int64_t)h * C;
  float nn[PER];
  float tot = 0.f;
#pragma unroll
  for (int j = 0; j < PER / 4; ++j) {
    const int4 n4 = *reinterpret_cast<const int4*>(sz + j * 4 * T + tid * 4);
    const int ni[4] = {n4.x, n4.y, n4.z, n4.w};
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int c = j * 4 * T + tid * 4 + e;
      const float n = (float)ni[e];
      nn[4 * j + e] = n;
      tot += n;
      s_ninf[c] = n > 0.f ? 0.f : -INFINITY;
      s_pen[c] = key_beta != 0.f && n > 0.f ? key_beta * __logf(1.0f + n) : 0.f;
    }
  }
  tot = warp_sumf(tot);
  if (lane == 0) red_f[0][0][0][warp] = tot;
  __syncthreads();
  if (warp == 0) {
    const float t = warp_sumf(lane < W ? red_f[0][0][0][lane] : 0.f);
    if (lane == 0) s_total = t;
  }
  __syncthreads();
  const float row_total = s_total;
  const bool all_fit = row_total < target_tokens;
  const bool float_sums = row_total < 16777216.f;
  const int target_i = (int)target_tokens;
  int flip = 1;
  for (int q0 = blockIdx.x * ROWS; q0 < num_queries; q0 += gridDim.x * ROWS) {
    const int live = min(ROWS, num_queries - q0);          // uniform over the CTA
    float sc[ROWS][PER];
#pragma unroll
    for (int r = 0; r < ROWS; ++r) {
      const int q = r < live ? q0 + r : q0;                // rows past the end repeat the first, unwritten
      const float4* row = reinterpret_cast<const float4*>(score + ((int64_t)q * num_kv_heads + h) * C);
#pragma unroll
      for (int j = 0; j < PER / 4; ++j) {
        const float4 v = __ldcs(row + j * T + tid);
        sc[r][4 * j] = v.x; sc[r][4 * j + 1] = v.y; sc[r][4 * j + 2] = v.z; sc[r][4 * j + 3] = v.w;
      }
    }
    float mx[ROWS], mn[ROWS], kmx[ROWS];
    int arg[ROWS];
#pragma unroll
    for (int r = 0; r < ROWS; ++r) { mx[r] = -INFINITY; mn[r] = INFINITY; kmx[r] = -INFINITY; arg[r] = 0; }
#pragma unroll
    for (int j = 0; j < PER / 4; ++j) {
      const float4 p4 = *reinterpret_cast<const float4*>(s_pen + j * 4 * T + tid * 4);
      const float4 m4 = *reinterpret_cast<const float4*>(s_ninf + j * 4 * T + tid * 4);
      const float pen[4] = {p4.x, p4.y, p4.z, p4.w}, ninf[4] = {m4.x, m4.y, m4.z, m4.w};
#pragma unroll
      for (int r = 0; r < ROWS; ++r)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float s = sc[r][4 * j + e];
          const float key = s + pen[e];
          if (key > kmx[r]) { kmx[r] = key; arg[r] = j * 4 * T + tid * 4 + e; }   // ascending ids
          mx[r] = fmaxf(mx[r], s);
          mn[r] = fminf(mn[r], s - ninf[e]);               // +inf for an empty cluster
          sc[r][4 * j + e] = s + ninf[e];                  // -inf for an empty cluster
        }
    }
    // block statistics of all rows behind one barrier
#pragma unroll
    for (int r = 0; r < ROWS; ++r) {
      const float wmx = warp_max(mx[r]), wmn = warp_min(mn[r]), wk = warp_max(kmx[r]);
      int cand = kmx[r] == wk ? arg[r] : 0x7fffffff;
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) cand = min(cand, __shfl_xor_sync(0xffffffffu, cand, o));
      if (lane == 0) {
        red_f[flip][r][0][warp] = wmx; red_f[flip][r][1][warp] = wmn; red_f[flip][r][2][warp] = wk;
        red_i[flip][r][warp] = cand;
      }
    }
    __syncthreads();
    float lo[ROWS], hi[ROWS];
#pragma unroll
    for (int r = 0; r < ROWS; ++r) {
      const float bmx = warp_max(lane < W ? red_f[flip][r][0][lane] : -INFINITY);
      const float bmn = warp_min(lane < W ? red_f[flip][r][1][lane] : INFINITY);
      hi[r] = bmx + 1e-6f;
      lo[r] = fminf(bmn - 1e-6f, hi[r] - 1e-5f);
      if (top1 && warp == r && r < live) {
        const float kb = lane < W ? red_f[flip][r][2][lane] : -INFINITY;
        const float kbest = warp_max(kb);
        int cand = (lane < W && kb == kbest) ? red_i[flip][r][lane] : 0x7fffffff;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) cand = min(cand, __shfl_xor_sync(0xffffffffu, cand, o));
        if (lane == 0) top1[(int64_t)h * num_queries + q0 + r] = cand;
      }
    }
    flip ^= 1;
    for (int it = 0; it < iters; ++it) {
      float mid[ROWS];
      int part[ROWS];
#pragma unroll
      for (int r = 0; r < ROWS; ++r) mid[r] = (lo[r] + hi[r]) * 0.5f;
      if (float_sums) {
        float acc[ROWS][2];
#pragma unroll
        for (int r = 0; r < ROWS; ++r) acc[r][0] = acc[r][1] = 0.f;
#pragma unroll
        for (int i = 0; i < PER; ++i)
#pragma unroll
          for (int r = 0; r < ROWS; ++r) add_if_ge(acc[r][i & 1], sc[r][i], mid[r], nn[i]);
#pragma unroll
        for (int r = 0; r < ROWS; ++r) part[r] = (int)(acc[r][0] + acc[r][1]);
      } else {
#pragma unroll
        for (int r = 0; r < ROWS; ++r) {
          part[r] = 0;
#pragma unroll
          for (int i = 0; i < PER; ++i) part[r] += sc[r][i] >= mid[r] ? (int)nn[i] : 0;
        }
      }
#pragma unroll
      for (int r = 0; r < ROWS; ++r) {
        part[r] = __reduce_add_sync(0xffffffffu, part[r]);
        if (lane == 0) red_i[flip][r][warp] = part[r];
      }
      __syncthreads();
#pragma unroll
      for (int r = 0; r < ROWS; ++r) {
        const int above = __reduce_add_sync(0xffffffffu, lane < W ? red_i[flip][r][lane] : 0);
        const bool reach = above >= target_i;
        lo[r] = reach ? mid[r] : lo[r];
        hi[r] = reach ? hi[r] : mid[r];
      }
      flip ^= 1;
    }
#pragma unroll
    for (int r = 0; r < ROWS; ++r) {
      if (r >= live) break;
      const int q = q0 + r;
      const float theta = all_fit ? NEG_BIG : lo[r];
      int32_t* qm = qmask + ((int64_t)q * num_kv_heads + h) * (C / 32);
      int n_sel = 0;
      float n_tok = 0.f;
#pragma unroll
      for (int j = 0; j < PER / 4; ++j) {
        unsigned nib = 0;
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const bool sel = sc[r][4 * j + e] >= theta;
          nib |= sel ? (1u << e) : 0u;
          n_sel += sel;
          n_tok += sel ? nn[4 * j + e] : 0.f;
        }
        // a 32-bit word holds the nibbles of eight consecutive threads
        unsigned word = nib << (4 * (lane & 7));
        word |= __shfl_xor_sync(0xffffffffu, word, 1);
        word |= __shfl_xor_sync(0xffffffffu, word, 2);
        word |= __shfl_xor_sync(0xffffffffu, word, 4);
        if (j == 0 && tid == 0 && force_sink) word |= 1u;
        if ((lane & 7) == 0) qm[j * (T / 8) + (tid >> 3)] = (int32_t)word;
      }
      if (counts || tokens) {
        n_sel = __reduce_add_sync(0xffffffffu, n_sel);
        n_tok = warp_sumf(n_tok);
        if (lane == 0) { red_i[flip][0][warp] = n_sel; red_f[flip][0][0][warp] = n_tok; }
        __syncthreads();
        if (warp == 0) {
          const int ns = __reduce_add_sync(0xffffffffu, lane < W ? red_i[flip][0][lane] : 0);
          const float nt = warp_sumf(lane < W ? red_f[flip][0][0][lane] : 0.f);
          if (lane == 0) {
            if (counts) counts[(int64_t)q * num_kv_heads + h] = ns;
            if (tokens) tokens[(int64_t)q * num_kv_heads + h] = (int)nt;
          }
        }
        flip ^= 1;
      }
    }
  }
}

template <int D, int G>
int launch_score(const void* vectors, int num_queries, int num_q_heads, const void* codebooks,
                 int num_kv_heads, int num_clusters, const int32_t* sizes, float temperature,
                 float beta, float* score, int* status, cudaStream_t st) {
  constexpr int QT = 128 / G;
  CUtensorMap mc;
  if (reinterpret_cast<uintptr_t>(vectors) & 15)
    return semblo::fail(semblo::SEMBLO_EINVAL, "routing vectors %p are not 16-byte aligned", vectors);
  int rc;
  uint64_t dc[3] = {(uint64_t)D / 2, (uint64_t)num_clusters, (uint64_t)num_kv_heads * 2};
  uint64_t sc[2] = {(uint64_t)D, (uint64_t)num_clusters * D};
  uint32_t bc[3] = {64, (uint32_t)SC_BN, 1};
  rc = semblo::make_tensor_map_bf16(&mc, codebooks, 3, dc, sc, bc);
  if (rc) return rc;
  auto kern = score_kernel<D, G>;
  SEMBLO_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, ScoreSmem<D>::TOTAL));
  dim3 grid((unsigned)ceil_div(num_queries, QT), num_kv_heads);
  kern<<<grid, 320, ScoreSmem<D>::TOTAL, st>>>((const __nv_bfloat16*)vectors, mc, num_queries, num_clusters, sizes,
                                               LOG2E / temperature, beta, score, num_kv_heads, status);
  SEMBLO_LAUNCH_CHECK();
  return 0;
}

}  // namespace

extern "C" int semblo_score_clusters(const void* vectors_bf16, int num_queries, int num_q_heads,
                                     int head_dim, const void* codebooks_bf16, int num_kv_heads,
                                     int num_clusters, const int32_t* select_sizes,
                                     float temperature, float beta, float* score, int32_t* status,
                                     void* stream) {
  SEMBLO_REQUIRE(num_q_heads % num_kv_heads == 0, "query heads must be a multiple of the KV heads");
  SEMBLO_REQUIRE(temperature > 0.f, "temperature must be positive");
  SEMBLO_REQUIRE(status != nullptr, "status word is required");
  if (num_queries == 0) return 0;
  const int g = num_q_heads / num_kv_heads;
  cudaStream_t st = (cudaStream_t)stream;
#define SEMBLO_SCORE_CASE(DD, GG)                                                                  \
  if (head_dim == DD && g == GG)                                                                   \
    return launch_score<DD, GG>(vectors_bf16, num_queries, num_q_heads, codebooks_bf16, num_kv_heads, \
                                num_clusters, select_sizes, temperature, beta, score, status, st);
  SEMBLO_SCORE_CASE(256, 4)
  SEMBLO_SCORE_CASE(128, 4)
  SEMBLO_SCORE_CASE(256, 8)
  SEMBLO_SCORE_CASE(128, 8)
  SEMBLO_SCORE_CASE(256, 16)
  SEMBLO_SCORE_CASE(128, 16)
#undef SEMBLO_SCORE_CASE
  return semblo::fail(semblo::SEMBLO_EINVAL,
                      "scoring supports head_dim 128/256 with 4, 8 or 16 query heads per KV head "
                      "(got head_dim %d, group %d)", head_dim, g);
}

extern "C" int semblo_select_clusters(const float* score, const int32_t* select_sizes,
                                      int num_queries, int num_kv_heads, int num_clusters,
                                      int target_tokens, int iters, int force_sink, int32_t* qmask,
                                      int32_t* counts, int32_t* tokens, int32_t* top1, float tile_key_beta,
                                      void* stream) {
  SEMBLO_REQUIRE(num_clusters % 32 == 0, "cluster count %d must be a multiple of 32", num_clusters);
  if (num_queries == 0) return 0;
  cudaStream_t st_sel = (cudaStream_t)stream;
#define SEMBLO_SELECT_REG(PER)                                                                      \
  if (num_clusters == PER * 32) {                                                                   \
    const int per_head = std::max(1, sm_count() * (PER >= 64 ? 3 : 4) / num_kv_heads);              \
    dim3 grid_r((unsigned)std::min<int64_t>(ceil_div(num_queries, SELECT_REG_WARPS), per_head), num_kv_heads); \
    select_kernel_reg<PER><<<grid_r, SELECT_REG_WARPS * 32, 0, st_sel>>>(                           \
        score, select_sizes, num_queries, num_kv_heads, (float)target_tokens, iters, force_sink,    \
        tile_key_beta, qmask, counts, tokens, top1);                                                \
    SEMBLO_LAUNCH_CHECK();                                                                          \
    return 0;                                                                                       \
  }
  SEMBLO_SELECT_REG(4)
  SEMBLO_SELECT_REG(8)
  SEMBLO_SELECT_REG(16)
  SEMBLO_SELECT_REG(32)
  SEMBLO_SELECT_REG(64)
#undef SEMBLO_SELECT_REG
#define SEMBLO_SELECT_WIDE(PER, ROWS)                                                               \
  if (num_clusters == PER * SELECT_WIDE_THREADS) {                                                  \
    const size_t smem_w = (size_t)2 * PER * SELECT_WIDE_THREADS * 4;                                \
    SEMBLO_CUDA(cudaFuncSetAttribute(select_kernel_wide<PER, ROWS>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_w)); \
    const int per_head = std::max(1, sm_count() / num_kv_heads);                                    \
    dim3 grid_w((unsigned)std::min<int64_t>(ceil_div(num_queries, ROWS), per_head), num_kv_heads);  \
    select_kernel_wide<PER, ROWS><<<grid_w, SELECT_WIDE_THREADS, smem_w, st_sel>>>(                 \
        score, select_sizes, num_queries, num_kv_heads, (float)target_tokens, iters, force_sink,    \
        tile_key_beta, qmask, counts, tokens, top1);                                                \
    SEMBLO_LAUNCH_CHECK();                                                                          \
    return 0;                                                                                       \
  }
  SEMBLO_SELECT_WIDE(8, 4)
  SEMBLO_SELECT_WIDE(16, 4)
  SEMBLO_SELECT_WIDE(32, 2)
#undef SEMBLO_SELECT_WIDE
  int warps = 8;
  while (warps > 1 && (size_t)(warps + 1) * num_clusters * 4 > 200 * 1024) warps >>= 1;
  const size_t smem = (size_t)(warps + 1) * num_clusters * 4;
  SEMBLO_REQUIRE(smem <= 220 * 1024, "cluster count %d too large for the selection kernel", num_clusters);
  SEMBLO_CUDA(cudaFuncSetAttribute(select_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  dim3 grid((unsigned)ceil_div(num_queries, warps), num_kv_heads);
  select_kernel<<<grid, warps * 32, smem, (cudaStream_t)stream>>>(
      score, select_sizes, num_queries, num_kv_heads, num_clusters, (float)target_tokens, iters,
      force_sink, tile_key_beta, qmask, counts, tokens, top1);
  SEMBLO_LAUNCH_CHECK();
  return 0;
}
