// Softmax / epilogue code shared by the two prefill attention kernels.
//
// A tile is 128 rows x 64 keys.  Its softmax is one stage run by eight warps, two threads per
// row: one for columns [0, 32) and one for columns [32, 64) (half 0 / half 1).  Each thread
// reads its 32 logits from tensor memory once; the two half maxima of a row meet in shared
// memory at a barrier of the two warps involved.  Each thread keeps the lazily rescaled running
// maximum (identical in the two) and its half of the row sum, and writes P = exp2(scale * s - m)
// as bf16 over the first 16 columns of its own half (softmax_tile below).
//
// Both A operands live in tensor memory, so shared memory holds K / V stages only:
//   Q  [128 x D]  bf16, two elements per 32-bit column, written once per CTA (stage_q_half);
//   P  [128 x 64] bf16 in the first 16 columns of each half of the S buffer it was computed
//      from, read by O += P V as a TMEM operand.
// An S buffer therefore becomes free when the P V product of its tile has completed.
#pragma once
#include "sm100.cuh"

namespace attn {

using namespace sm100;

constexpr float LN2F = 0.6931471805599453f;
constexpr float LOG2EF = 1.4426950408889634f;
constexpr float RESCALE_GAP = 8.0f;              // log2 units: rescale O only when the max moved by > 2^8

// Rendezvous of softmax threads on an mbarrier (count = the threads that meet).  Unlike bar.sync the wait
// is bounded and observes the abort flag, so a role that gave up cannot strand its partners.
__device__ __forceinline__ bool softmax_group_sync(uint32_t bar, uint32_t parity, volatile int* abort_flag,
                                                   int* status) {
  mbar_arrive(bar);
  return mbar_wait(bar, parity, abort_flag, status, STATUS_TIMEOUT_SOFTMAX);
}

// Copies this thread's half of the first D dims of its query row (D/2 bf16 from qrow_half, or
// zeros when null) into the Q operand columns and arrives on bar_qfull (count: the softmax threads).
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

// The softmax of one tile for one half-row (hf: columns [32 hf, 32 hf + 32) of the tile, and
// columns [hf D/2, (hf + 1) D/2) of O when the accumulator has to be rescaled).  The raw logits
// are in TMEM columns [s_col, s_col + 64); `lim` is the number of leading columns this row may
// attend to (64: all; columns from `lim` on, which include those of pages the product did not
// write, count as -inf).  `pages` is the tile's count of 16-key groups.  The two threads of a row
// exchange their half maxima through mx (float [2][2][128]: tile parity, half, row) and
// bar_pair, the barrier of the two warps that share these 32 rows (count 2: a warp arrives once, by
// lane 0 after a __syncwarp -- 32 arrivals of a warp on one barrier are taken one after the other),
// in phase j.  Arrives on bar_pfull_b (count: the softmax warps) when P is stored.  Returns false
// after a wait timed out.
template <int D, int O_COL>
__device__ __forceinline__ bool softmax_tile(int pages, int lim, int j, int hf, int row, uint32_t lane_addr,
                                             uint32_t tmem_base, uint32_t s_col, float* mx, uint32_t bar_pair,
                                             uint32_t bar_pvdone_prev, uint32_t pvdone_prev_parity,
                                             uint32_t bar_pfull_b, float scale_log2, float& m_ref, float& l_part,
                                             volatile int* abort_flag, int* status) {
  const uint32_t s_addr = tmem_base + lane_addr + s_col + hf * 32;
  const bool active = pages > 2 * hf;                  // the product wrote at least one page of this half
  uint32_t x[32];
  float hm = -INFINITY;
  if (active) {
    tmem_ld32(s_addr, x);
    tmem_ld_wait();
    const int lx = lim - 32 * hf;
    if (!__all_sync(0xffffffffu, lx >= 32)) {
#pragma unroll
      for (int i = 0; i < 32; ++i)
        if (i >= lx) x[i] = 0xff800000u;
    }
    float tm[2] = {-INFINITY, -INFINITY};              // two short chains
#pragma unroll
    for (int i = 0; i < 32; i += 4) {
      tm[0] = fmax3(tm[0], __uint_as_float(x[i]), __uint_as_float(x[i + 1]));
      tm[1] = fmax3(tm[1], __uint_as_float(x[i + 2]), __uint_as_float(x[i + 3]));
    }
    hm = fmaxf(tm[0], tm[1]);
  }
  float* slot = mx + (j & 1) * 256;
  slot[hf * 128 + row] = hm;
  __syncwarp();                                        // one arrival per warp: the barrier counts warps
  if ((threadIdx.x & 31) == 0) mbar_arrive(bar_pair);
  if (!mbar_wait_warp(bar_pair, (uint32_t)(j & 1), abort_flag, status, STATUS_TIMEOUT_SOFTMAX)) return false;
  float tmax = fmaxf(hm, slot[(hf ^ 1) * 128 + row]);
  if (tmax < -1e29f) tmax = -INFINITY;               // only keys rejected through the selection operand
  tmax *= scale_log2;
  // lazy rescale: only when the running reference falls more than 2^8 behind
  const bool need = j > 0 && m_ref != -INFINITY && tmax > m_ref + RESCALE_GAP;
  float alpha = 1.f;
  if (need) {
    alpha = fast_exp2(m_ref - tmax);
    m_ref = tmax;
    l_part *= alpha;
  } else if (m_ref == -INFINITY) {
    m_ref = tmax;
  }
  if (__any_sync(0xffffffffu, need)) {
    // O must be quiescent: the previous tile's P V has to be complete
    if (!mbar_wait_warp(bar_pvdone_prev, pvdone_prev_parity, abort_flag, status, STATUS_TIMEOUT_SOFTMAX)) return false;
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
  if (active) {
    const float neg_m = m_ref == -INFINITY ? 0.f : -m_ref;
    uint32_t packed[16];
    float add0 = 0.f, add1 = 0.f;
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      const float e0 = fast_exp2(fmaf(__uint_as_float(x[2 * i]), scale_log2, neg_m));
      const float e1 = fast_exp2(fmaf(__uint_as_float(x[2 * i + 1]), scale_log2, neg_m));
      __nv_bfloat162 pr = __floats2bfloat162_rn(e0, e1);
      packed[i] = *reinterpret_cast<uint32_t*>(&pr);
      if (i & 1) add1 += e0 + e1; else add0 += e0 + e1;
    }
    l_part += add0 + add1;
    // keys 32 hf + 2 i, 32 hf + 2 i + 1 of the row share column 32 hf + i: P lies over this
    // half's own logits only (nobody else reads them).  The P V product takes its 16-key operand
    // slices from columns 0, 8, 32 and 40 of the buffer.
    tmem_st16(s_addr, packed);
  }
  tmem_st_wait();
  tc_fence_before();
  __syncwarp();                                        // every lane's P is stored: one arrival per warp
  if ((threadIdx.x & 31) == 0) mbar_arrive(bar_pfull_b);
  return true;
}

// Final write of D/2 output columns by each of the two softmax threads of a row (they hold the same
// running maximum and one half of the row sum each, exchanged through xchg).  merge != 0: another
// partial (normalised output in prev_f32, or in `dst` as bf16 when prev_f32 is null; natural-log
// LSE in lse_ptr) is LSE-merged with this one.  out_f32 != null: the result is written there in
// fp32 instead of `dst` (a partial that a later launch merges without an intermediate bf16 rounding).
template <int D, int O_COL>
__device__ __forceinline__ void epilogue_half(bool have_tiles, int hf, int row, uint32_t lane_addr,
                                              uint32_t tmem_base, float* xchg /* [2][128] */, uint32_t bar_epi,
                                              float m_ref, float l_part, bool qvalid, int merge,
                                              __nv_bfloat16* dst /* row base */, const float* prev_f32,
                                              float* out_f32, float* lse_ptr /* this row's slot or null */,
                                              volatile int* abort_flag, int* status) {
  xchg[hf * 128 + row] = l_part;
  if (!softmax_group_sync(bar_epi, 0, abort_flag, status)) return;
  const float l_run = l_part + xchg[(hf ^ 1) * 128 + row];
  constexpr float own = 1.f;
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
