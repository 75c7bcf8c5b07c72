// Softmax / epilogue code shared by the two prefill attention kernels.
//
// A tile is 128 rows x 64 keys.  Two warpgroups of 128 threads split the 64 columns of
// S: thread (half, row) owns columns [32 half, 32 half + 32) of its row.  The row maximum
// is exchanged through shared memory, the running reference maximum m_ref is kept
// identical in both threads of a row, each thread keeps the partial sum of its own
// columns, and each half rescales / finalises its own D/2 columns of O.
//
// Both A operands live in tensor memory, so shared memory holds K / V stages only:
//   Q  [128 x D]  bf16, two elements per 32-bit column, written once per CTA (stage_q_half);
//   P  [128 x 64] bf16 in the first 32 columns of the S buffer it was computed from (the
//      S values are in registers by then), read by O += P V as a TMEM operand.
// An S buffer therefore becomes free when the P V product of its tile has completed.
#pragma once
#include "sm100.cuh"

namespace attn {

using namespace sm100;

constexpr float LN2F = 0.6931471805599453f;
constexpr float LOG2EF = 1.4426950408889634f;
// true: O is normalised by the sum of the bf16-rounded weights the tensor core multiplies
// (two more integer operations per pair of keys); false: by the exact sum, as the LSE is.
constexpr bool ROUNDED_NORMALISER = false;
constexpr float RESCALE_GAP = 8.0f;              // log2 units: rescale O only when the max moved by > 2^8

// Rendezvous of softmax threads on an mbarrier (count = the threads that meet).  Unlike bar.sync the wait
// is bounded and observes the abort flag, so a role that gave up cannot strand its partners.
__device__ __forceinline__ bool softmax_group_sync(uint32_t bar, uint32_t parity, volatile int* abort_flag,
                                                   int* status) {
  mbar_arrive(bar);
  return mbar_wait(bar, parity, abort_flag, status, STATUS_TIMEOUT_SOFTMAX);
}

// Copies this thread's half of its query row (D/2 bf16 from qrow_half, or zeros when null) into
// the Q operand columns and arrives on bar_qfull (count: all softmax threads).
template <int D, int Q_COL>
__device__ __forceinline__ void stage_q_half(const __nv_bfloat16* qrow_half, int hf, uint32_t lane_addr,
                                             uint32_t tmem_base, uint32_t bar_qfull) {
#pragma unroll 1
  for (int c = 0; c < D / 128; ++c) {
    uint32_t w[32];
    if (qrow_half) {
      const uint4* src = reinterpret_cast<const uint4*>(qrow_half + c * 64);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const uint4 v = __ldg(src + i);
        w[4 * i] = v.x; w[4 * i + 1] = v.y; w[4 * i + 2] = v.z; w[4 * i + 3] = v.w;
      }
    } else {
#pragma unroll
      for (int i = 0; i < 32; ++i) w[i] = 0u;
    }
    tmem_st32(tmem_base + lane_addr + Q_COL + hf * (D / 4) + c * 32, w);
  }
  tmem_st_wait();
  tc_fence_before();
  mbar_arrive(bar_qfull);
}

// One half-row of one tile.  r[] holds the 32 raw logits of this half with masked entries
// already set to -inf; tmax_raw is their maximum.  my_pages = how many 16-column groups of
// this half exist in the tile (0, 1 or 2).  s_col = first TMEM column of the tile's S buffer,
// which receives P.  Returns false after a wait timed out.
template <int D, int O_COL>
__device__ __forceinline__ bool softmax_half_tile(
    uint32_t (&r)[32], float tmax_raw, int my_pages, int j, int hf, int row, uint32_t lane_addr,
    uint32_t tmem_base, uint32_t s_col, float* xchg /* [2][2][128] */, uint32_t bar_xchg0,
    uint32_t bar_pvdone_prev, uint32_t bar_pfull_b, float scale_log2, float& m_ref, float& l_part,
    float& l_rnd, volatile int* abort_flag, int* status) {
  // Both threads of a row exchange their maxima and take the larger, so they agree on the
  // reference exactly.  The two warps that share 32 rows meet on a barrier of their own (count
  // 64; double-buffered by tile parity), so the four warp pairs do not wait for one another.
  // Past this barrier both threads hold their S values in registers, so P may overwrite S.
  float* xc = xchg + (j & 1) * 256;
  xc[hf * 128 + row] = tmax_raw;
  if (!softmax_group_sync(bar_xchg0 + 8 * ((j & 1) * 4 + (row >> 5)), (j >> 1) & 1, abort_flag, status)) return false;
  tc_fence_after();
  const float tmax = fmaxf(tmax_raw, xc[(hf ^ 1) * 128 + row]) * scale_log2;
  // lazy rescale: only when the running reference falls more than 2^8 behind
  const bool need = j > 0 && m_ref != -INFINITY && tmax > m_ref + RESCALE_GAP;
  float alpha = 1.f;
  if (need) {
    alpha = fast_exp2(m_ref - tmax);
    m_ref = tmax;
    l_part *= alpha;
    l_rnd *= alpha;
  } else if (m_ref == -INFINITY) {
    m_ref = tmax;
  }
  if (__any_sync(0xffffffffu, need)) {
    // O must be quiescent: the previous tile's P V has to be complete
    if (!mbar_wait(bar_pvdone_prev, ((j - 1) >> 1) & 1, abort_flag, status, STATUS_TIMEOUT_SOFTMAX)) return false;
    tc_fence_after();
#pragma unroll 1
    for (int c = 0; c < D / 64; ++c) {
      uint32_t o[32];
      const uint32_t addr = tmem_base + lane_addr + O_COL + hf * (D / 2) + c * 32;
      tmem_ld32(addr, o);
      tmem_ld_wait();
#pragma unroll
      for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
      tmem_st32(addr, o);
    }
  }
  const float neg_m = m_ref == -INFINITY ? 0.f : -m_ref;
  float add = 0.f, add2 = 0.f, add_rnd = 0.f;
  if (my_pages > 0) {
    uint32_t packed[16];
#pragma unroll
    for (int p = 0; p < 2; ++p) {
      if (p < my_pages) {
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const float e0 = fast_exp2(fmaf(__uint_as_float(r[p * 16 + 2 * i]), scale_log2, neg_m));
          const float e1 = fast_exp2(fmaf(__uint_as_float(r[p * 16 + 2 * i + 1]), scale_log2, neg_m));
          __nv_bfloat162 pr = __floats2bfloat162_rn(e0, e1);
          const uint32_t w = *reinterpret_cast<uint32_t*>(&pr);
          packed[p * 8 + i] = w;
          if (i & 1) add2 += e0 + e1; else add += e0 + e1;
          if constexpr (ROUNDED_NORMALISER)
            add_rnd += __uint_as_float(w << 16) + __uint_as_float(w & 0xffff0000u);
        }
      } else {
#pragma unroll
        for (int i = 0; i < 8; ++i) packed[p * 8 + i] = 0u;
      }
    }
    // keys 32 hf + 2 i, 32 hf + 2 i + 1 of the row share column 16 hf + i of the P operand
    tmem_st16(tmem_base + lane_addr + s_col + hf * 16, packed);
  }
  l_part += add + add2;
  l_rnd += add_rnd;
  tmem_st_wait();
  tc_fence_before();
  mbar_arrive(bar_pfull_b);
  return true;
}

// Final write of this half's D/2 output columns.  merge != 0: another partial (normalised
// output in prev_f32, or in `dst` as bf16 when prev_f32 is null; natural-log LSE in lse_ptr) is
// LSE-merged with this one.  out_f32 != null: the result is written there in fp32 instead of
// `dst` (a partial that a later launch merges without an intermediate bf16 rounding).
template <int D, int O_COL>
__device__ __forceinline__ void epilogue_half(bool have_tiles, int hf, int row, uint32_t lane_addr,
                                              uint32_t tmem_base, float* xchg, uint32_t bar_epi, float m_ref,
                                              float l_part, float l_rnd, bool qvalid, int merge,
                                              __nv_bfloat16* dst /* row base */, const float* prev_f32,
                                              float* out_f32, float* lse_ptr /* this row's slot or null */,
                                              volatile int* abort_flag, int* status) {
  xchg[hf * 128 + row] = l_part;
  xchg[256 + hf * 128 + row] = l_rnd;
  if (!softmax_group_sync(bar_epi, 0, abort_flag, status)) return;
  const float l_run = l_part + xchg[(hf ^ 1) * 128 + row];
  const float l_rnd_run = l_rnd + xchg[256 + (hf ^ 1) * 128 + row];
  // O / l_rnd_run is the normalised partial when the rounded sum is kept
  const float own = !ROUNDED_NORMALISER ? 1.f : (l_rnd_run > 0.f ? l_run / l_rnd_run : 0.f);
  float wa = 0.f, wb = 1.f, denom = l_run, m_new = m_ref;
  if (merge && qvalid) {
    const float l2 = *lse_ptr * LOG2EF;                 // the other partial's LSE in log2 units
    m_new = fmaxf(l2, m_ref);
    if (m_new == -INFINITY) {
      wa = 0.f; wb = 0.f; denom = 0.f;
    } else {
      wa = fast_exp2(l2 - m_new);
      wb = m_ref == -INFINITY ? 0.f : fast_exp2(m_ref - m_new);
      denom = wa + l_run * wb;
    }
  }
  if (!softmax_group_sync(bar_epi, 1, abort_flag, status)) return;   // both halves have read the old LSE
  const float inv = denom > 0.f ? 1.f / denom : 0.f;
#pragma unroll 1
  for (int c = 0; c < D / 64; ++c) {
    uint32_t o[32];
    const int col0 = hf * (D / 2) + c * 32;
    if (have_tiles) {
      tmem_ld32(tmem_base + lane_addr + O_COL + col0, o);
      tmem_ld_wait();
    } else {
#pragma unroll
      for (int i = 0; i < 32; ++i) o[i] = 0u;
    }
    if (qvalid) {
      uint4* d4 = reinterpret_cast<uint4*>(dst + col0);
      float prev[32];
      if (merge) {
        if (prev_f32) {
          const float4* p4 = reinterpret_cast<const float4*>(prev_f32 + col0);
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const float4 v = p4[i];
            prev[4 * i] = v.x; prev[4 * i + 1] = v.y; prev[4 * i + 2] = v.z; prev[4 * i + 3] = v.w;
          }
        } else {
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const uint4 v = d4[i];
            const uint32_t u[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const float2 pv = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u[e]));
              prev[8 * i + 2 * e] = pv.x;
              prev[8 * i + 2 * e + 1] = pv.y;
            }
          }
        }
      }
      float x[32];
#pragma unroll
      for (int i = 0; i < 32; ++i) {
        float v = __uint_as_float(o[i]) * (wb * own);
        if (merge) v += prev[i] * wa;
        x[i] = v * inv;
      }
      if (out_f32) {
        float4* o4 = reinterpret_cast<float4*>(out_f32 + col0);
#pragma unroll
        for (int i = 0; i < 8; ++i) o4[i] = make_float4(x[4 * i], x[4 * i + 1], x[4 * i + 2], x[4 * i + 3]);
      } else {
        uint32_t w[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          __nv_bfloat162 pr = __floats2bfloat162_rn(x[2 * i], x[2 * i + 1]);
          w[i] = *reinterpret_cast<uint32_t*>(&pr);
        }
        d4[0] = make_uint4(w[0], w[1], w[2], w[3]);
        d4[1] = make_uint4(w[4], w[5], w[6], w[7]);
        d4[2] = make_uint4(w[8], w[9], w[10], w[11]);
        d4[3] = make_uint4(w[12], w[13], w[14], w[15]);
      }
    }
  }
  if (qvalid && lse_ptr && hf == 0) *lse_ptr = denom > 0.f ? (m_new + __log2f(denom)) * LN2F : -INFINITY;
}

}  // namespace attn
