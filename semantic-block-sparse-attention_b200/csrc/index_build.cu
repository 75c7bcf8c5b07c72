// Index build: routing-space normalisation, nearest-centroid assignment (tcgen05 GEMM
// with a bf16-round + first-arg-max epilogue), deterministic centroid update, the
// cluster-major page-aligned layout (stable radix sort by cluster id), and the
// cluster-ordered K/V copy.
//
// Reference behaviour restated here:
//   semblo/vllm_plugin/routing_map.py:35-64      routing_normalize (whole vector)
//   semblo/inference/flat_index.py:144-166       routing_space
//   semblo/inference/flat_index.py:356-373       _argmax_sim_chunked
//   semblo/inference/flat_index.py:268-288       k-means centroid update
//   semblo/vllm_plugin/state.py:44-84, 850-914   posting order, page alignment, inverse map
//   semblo/vllm_plugin/state.py:950-997          pack_prompt_kv
#include <cuda_bf16.h>
#include <mutex>

#include "../../include/semblo_b200.h"
#include "host_common.h"
#include "attn_common.cuh"
#include "sm100.cuh"

using namespace sm100;
using semblo::ceil_div;

namespace {

// ------------------------------------------------------------------ normalise
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ double warp_sum_d(double v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// One warp per row.  stage 1: u = x / max(|x|, 1e-12), rounded to the input dtype
// (written to `out`).  stage 2: space = u / max(|u|, 1e-12) in fp32 (written to
// space_f32 / space_bf16).  The sums of squares are accumulated in double so the
// norm is the correctly rounded one.
template <typename T, int MAXD>
__global__ void normalize_rows_kernel(const T* __restrict__ x, int64_t n_rows, int dim,
                                      int64_t row_stride, T* __restrict__ out,
                                      float* __restrict__ space_f32,
                                      __nv_bfloat16* __restrict__ space_bf16, int second_round) {
  const int lane = threadIdx.x & 31;
  const int64_t row = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= n_rows) return;
  constexpr int PER = MAXD / 32;
  float v[PER];
  double ss = 0.0;
#pragma unroll
  for (int i = 0; i < PER; ++i) {
    int d = lane + 32 * i;
    v[i] = d < dim ? (float)x[row * row_stride + d] : 0.f;
    ss += (double)v[i] * (double)v[i];
  }
  ss = warp_sum_d(ss);
  float nrm = fmaxf((float)sqrt(ss), 1e-12f);
  double ss2 = 0.0;
  if (second_round == 2) {
    // the input is already the routed (stage-1) vector: one normalisation only
    ss2 = ss;
  } else {
#pragma unroll
    for (int i = 0; i < PER; ++i) {
      T r = (T)(v[i] / nrm);
      v[i] = (float)r;
      int d = lane + 32 * i;
      if (out && d < dim) out[row * (int64_t)dim + d] = r;
      ss2 += (double)v[i] * (double)v[i];
    }
  }
  if (!space_f32 && !space_bf16) return;
  if (second_round != 2) ss2 = warp_sum_d(ss2);
  float nrm2 = fmaxf((float)sqrt(ss2), 1e-12f);
#pragma unroll
  for (int i = 0; i < PER; ++i) {
    int d = lane + 32 * i;
    if (d >= dim) continue;
    float s = v[i] / nrm2;
    if (second_round == 1) {
      // query router: the second normalisation is rounded to the storage dtype too
      T r = (T)s;
      if (space_bf16) space_bf16[row * (int64_t)dim + d] = __float2bfloat16_rn((float)r);
      if (space_f32) space_f32[row * (int64_t)dim + d] = (float)r;
    } else {
      if (space_f32) space_f32[row * (int64_t)dim + d] = s;
      if (space_bf16) space_bf16[row * (int64_t)dim + d] = __float2bfloat16_rn(s);
    }
  }
}

// The same computation for bf16 rows with 16-byte accesses: lane l holds elements [8 l, 8 l + 8)
// of the row (dim a multiple of 8, at most 256; rows and outputs 16-byte aligned).
__global__ void normalize_rows_bf16x8_kernel(const __nv_bfloat16* __restrict__ x, int64_t n_rows, int dim,
                                             int64_t row_stride, __nv_bfloat16* __restrict__ out,
                                             float* __restrict__ space_f32,
                                             __nv_bfloat16* __restrict__ space_bf16, int second_round) {
  const int lane = threadIdx.x & 31;
  const int64_t row = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= n_rows) return;
  const bool have = lane * 8 < dim;
  float v[8];
  double ss = 0.0;
  {
    uint4 raw = make_uint4(0u, 0u, 0u, 0u);
    if (have) raw = __ldg(reinterpret_cast<const uint4*>(x + row * row_stride) + lane);
    const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&w[i]));
      v[2 * i] = f.x; v[2 * i + 1] = f.y;
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) ss += (double)v[i] * (double)v[i];
  }
  ss = warp_sum_d(ss);
  const float nrm = fmaxf((float)sqrt(ss), 1e-12f);
  double ss2 = 0.0;
  if (second_round == 2) {
    ss2 = ss;                                        // the input is already the routed (stage-1) vector
  } else {
    uint32_t packed[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const __nv_bfloat16 r0 = __float2bfloat16_rn(v[2 * i] / nrm), r1 = __float2bfloat16_rn(v[2 * i + 1] / nrm);
      v[2 * i] = __bfloat162float(r0); v[2 * i + 1] = __bfloat162float(r1);
      packed[i] = (uint32_t)__bfloat16_as_ushort(r0) | ((uint32_t)__bfloat16_as_ushort(r1) << 16);
      ss2 += (double)v[2 * i] * (double)v[2 * i] + (double)v[2 * i + 1] * (double)v[2 * i + 1];
    }
    if (out && have)
      reinterpret_cast<uint4*>(out + row * (int64_t)dim)[lane] = make_uint4(packed[0], packed[1], packed[2], packed[3]);
  }
  if (!space_f32 && !space_bf16) return;
  if (second_round != 2) ss2 = warp_sum_d(ss2);
  const float nrm2 = fmaxf((float)sqrt(ss2), 1e-12f);
  float sv[8];
  uint32_t sp[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float s0 = v[2 * i] / nrm2, s1 = v[2 * i + 1] / nrm2;
    const __nv_bfloat16 b0 = __float2bfloat16_rn(s0), b1 = __float2bfloat16_rn(s1);
    sp[i] = (uint32_t)__bfloat16_as_ushort(b0) | ((uint32_t)__bfloat16_as_ushort(b1) << 16);
    // query router (second_round == 1): the second normalisation is rounded to the storage dtype too
    sv[2 * i] = second_round == 1 ? __bfloat162float(b0) : s0;
    sv[2 * i + 1] = second_round == 1 ? __bfloat162float(b1) : s1;
  }
  if (!have) return;
  if (space_bf16) reinterpret_cast<uint4*>(space_bf16 + row * (int64_t)dim)[lane] = make_uint4(sp[0], sp[1], sp[2], sp[3]);
  if (space_f32) {
    float4* o = reinterpret_cast<float4*>(space_f32 + row * (int64_t)dim) + 2 * lane;
    o[0] = make_float4(sv[0], sv[1], sv[2], sv[3]);
    o[1] = make_float4(sv[4], sv[5], sv[6], sv[7]);
  }
}

__global__ void gather_rows_kernel(const float* __restrict__ src, const int64_t* __restrict__ idx,
                                   int64_t m, int dim, float* __restrict__ dst_f32,
                                   __nv_bfloat16* __restrict__ dst_bf16) {
  const int lane = threadIdx.x & 31;
  const int64_t row = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= m) return;
  const float* s = src + idx[row] * dim;
  for (int d = lane; d < dim; d += 32) {
    float v = s[d];
    if (dst_f32) dst_f32[row * dim + d] = v;
    if (dst_bf16) dst_bf16[row * dim + d] = __float2bfloat16_rn(v);
  }
}

// ------------------------------------------------------------------ assignment GEMM
// One CTA owns 128 rows of x and streams the codebook in chunks of 64 centroids: two accumulators
// and the key tile then take 256 columns of tensor memory, so two CTAs share a multiprocessor and
// one's epilogue runs under the other's products.
// warp 4: TMA producer, warp 5: UMMA issuer, warps 0-3 and 6-9: epilogue (two threads per row).
constexpr int ASG_BN = 64;         // centroids per chunk
constexpr int ASG_STAGES = 2;

template <int D>
struct AssignSmem {
  static constexpr bool A_TMEM = D >= 128;           // the key tile is a tensor-memory operand (D / 2 columns)
  static constexpr int A_BYTES = A_TMEM ? 0 : 128 * D * 2;
  static constexpr int B_BYTES = ASG_BN * D * 2;
  static constexpr int BAR_OFF = A_BYTES + ASG_STAGES * B_BYTES;
  static constexpr int X_COL = 2 * ASG_BN;           // TMEM: two accumulators, then the keys
  static constexpr int TMEM_COLS = (A_TMEM && X_COL + D / 2 > 256) ? 512 : 256;
  static constexpr int XCHG_OFF = BAR_OFF + 256;       // (value, id) of the upper-half epilogue threads: [128] float + [128] int
  static constexpr int TOTAL = XCHG_OFF + 1024 + 1024; // + alignment slack
};

// SPLIT: the centroids are a descriptor pair [2][C][D/2] (3-D map: column in the half, row,
// half) instead of [C][D], the similarity is compared in fp32 as it comes out of the tensor
// core (no bf16 rounding), and centroids whose bit is set in dead_bits are never chosen.
template <int D, bool SPLIT>
__global__ void __launch_bounds__(320, 2)
assign_argmax_kernel(const __grid_constant__ CUtensorMap tmap_x, const __nv_bfloat16* __restrict__ x,
                     int64_t x_stride,
                     const __grid_constant__ CUtensorMap tmap_c, int64_t n, int num_centroids,
                     int32_t* __restrict__ assign_out, int id_offset,
                     const uint32_t* __restrict__ dead_bits, int* __restrict__ status) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  using L = AssignSmem<D>;
  constexpr int SLABS = D / 64;
  constexpr int HALF_SLABS = SLABS >= 2 ? SLABS / 2 : 1;
  uint8_t* a_smem = smem;
  uint8_t* b_smem = smem + L::A_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::BAR_OFF);
  // bars: 0 a_full, 1..2 b_full, 3..4 b_empty, 5..6 acc_full, 7..8 acc_empty
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 16);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int num_chunks = (num_centroids + ASG_BN - 1) / ASG_BN;
  const int64_t row0 = (int64_t)blockIdx.x * 128;

  if (threadIdx.x == 0) {
    mbar_init(smem_u32(&bars[0]), L::A_TMEM ? 256 : 1);
    for (int s = 0; s < ASG_STAGES; ++s) {
      mbar_init(smem_u32(&bars[1 + s]), 1);
      mbar_init(smem_u32(&bars[3 + s]), 1);
      mbar_init(smem_u32(&bars[5 + s]), 1);
      mbar_init(smem_u32(&bars[7 + s]), 8);        // the epilogue warps (one arrival each, by lane 0)
    }
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

  float epi_best = 0.f;
  int epi_id = 0, epi_row = 0, epi_hf = -1;      // set by the epilogue threads
  bool epi_ok = false;
  if (warp == 4) {
    if (elect_one()) {
      tma_prefetch_desc(&tmap_c);
      if (!L::A_TMEM) {
        tma_prefetch_desc(&tmap_x);
        mbar_arrive_expect_tx(smem_u32(&bars[0]), L::A_BYTES);
        for (int sl = 0; sl < SLABS; ++sl)
          tma_load_2d(smem_u32(a_smem + sl * 128 * 128), &tmap_x, smem_u32(&bars[0]), sl * 64, (int)row0);
      }
      for (int j = 0; j < num_chunks; ++j) {
        const int s = j % ASG_STAGES;
        if (!mbar_wait(smem_u32(&bars[3 + s]), ((j / ASG_STAGES) & 1) ^ 1, abort_flag, status,
                       STATUS_TIMEOUT_LOAD))
          break;
        mbar_arrive_expect_tx(smem_u32(&bars[1 + s]), L::B_BYTES);
        for (int sl = 0; sl < SLABS; ++sl) {
          const uint32_t dst = smem_u32(b_smem + s * L::B_BYTES + sl * ASG_BN * 128);
          if (SPLIT)
            tma_load_3d(dst, &tmap_c, smem_u32(&bars[1 + s]), (sl % HALF_SLABS) * 64, j * ASG_BN, sl / HALF_SLABS);
          else
            tma_load_2d(dst, &tmap_c, smem_u32(&bars[1 + s]), sl * 64, j * ASG_BN);
        }
      }
    }
  } else if (warp == 5) {
    if (elect_one()) {
      constexpr uint32_t idesc = make_idesc_bf16(128, ASG_BN, false, false);
      bool ok = mbar_wait(smem_u32(&bars[0]), 0, abort_flag, status, STATUS_TIMEOUT_MMA);
      for (int j = 0; ok && j < num_chunks; ++j) {
        const int s = j % ASG_STAGES;
        const int b = j & 1;
        if (!mbar_wait(smem_u32(&bars[1 + s]), (j / ASG_STAGES) & 1, abort_flag, status, STATUS_TIMEOUT_MMA)) break;
        if (!mbar_wait(smem_u32(&bars[7 + b]), ((j >> 1) & 1) ^ 1, abort_flag, status, STATUS_TIMEOUT_MMA)) break;
        tc_fence_after();
        const uint32_t a_base = smem_u32(a_smem);
        const uint32_t b_base = smem_u32(b_smem + s * L::B_BYTES);
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint32_t sl = kk >> 2, ko = (kk & 3) * 32;
          uint64_t bd = make_smem_desc(b_base + sl * ASG_BN * 128 + ko, 16, 1024);
          if (L::A_TMEM)
            umma_ts(tmem_base + b * ASG_BN, tmem_base + L::X_COL + kk * 8, bd, idesc, kk > 0 ? 1u : 0u);
          else
            umma_ss(tmem_base + b * ASG_BN, make_smem_desc(a_base + sl * 128 * 128 + ko, 16, 1024), bd, idesc,
                    kk > 0 ? 1u : 0u);
        }
        umma_commit(smem_u32(&bars[3 + s]));
        umma_commit(smem_u32(&bars[5 + b]));
      }
    }
  } else {
    // epilogue: eight warps, two threads per row (TMEM lane).  Warps 0-3 scan columns [0, 64) of
    // every 128-centroid chunk, warps 6-9 columns [64, 128), each in ascending order; the two
    // partial results of a row are combined after the loop (larger value, then smaller id).
    const int hf = warp >= 6 ? 1 : 0;
    const int row = (warp & 3) * 32 + (threadIdx.x & 31);
    const uint32_t lane_addr = (uint32_t)((warp & 3) * 32) << 16;
    if constexpr (L::A_TMEM) {
      // the key tile goes to tensor memory once: each of the two threads of a row copies half of it
      // (rows past the last key are zero)
      attn::stage_q_half<D, L::X_COL>(row0 + row < n ? x + (row0 + row) * x_stride + hf * (D / 2) : nullptr, hf,
                                      lane_addr, tmem_base, smem_u32(&bars[0]));
    }
    float best = -INFINITY;
    int best_id = 0;
    bool ok = true;
    const bool full = (num_centroids % ASG_BN) == 0;
    for (int j = 0; j < num_chunks && ok; ++j) {
      const int b = j & 1;
      ok = mbar_wait_warp(smem_u32(&bars[5 + b]), (j >> 1) & 1, abort_flag, status, STATUS_TIMEOUT_EPILOGUE);
      if (!ok) break;
      tc_fence_after();
#pragma unroll 1
      for (int c4 = 0; c4 < ASG_BN / 64; ++c4) {   // each of a row's two threads takes half of the chunk
        uint32_t r[32];
        tmem_ld32(tmem_base + lane_addr + b * ASG_BN + hf * (ASG_BN / 2) + c4 * 32, r);
        tmem_ld_wait();
        const int cbase = j * ASG_BN + hf * (ASG_BN / 2) + c4 * 32;
        uint32_t dead = 0u;
        if (SPLIT && dead_bits != nullptr && cbase < num_centroids) dead = __ldg(dead_bits + (cbase >> 5));
        if (full && dead == 0u) {
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            // the reference's bf16 matmul output: fp32 accumulate, round to nearest even
            float v = SPLIT ? __uint_as_float(r[i]) : __bfloat162float(__float2bfloat16_rn(__uint_as_float(r[i])));
            const bool take = v > best;
            best = take ? v : best;
            best_id = take ? cbase + i : best_id;
          }
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            float v = SPLIT ? __uint_as_float(r[i]) : __bfloat162float(__float2bfloat16_rn(__uint_as_float(r[i])));
            const bool take = (cbase + i < num_centroids) && !((dead >> i) & 1u) && (v > best);
            best = take ? v : best;
            best_id = take ? cbase + i : best_id;
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if ((threadIdx.x & 31) == 0) mbar_arrive(smem_u32(&bars[7 + b]));
    }
    float* xv = reinterpret_cast<float*>(smem + L::XCHG_OFF);
    int* xi = reinterpret_cast<int*>(smem + L::XCHG_OFF + 512);
    if (hf == 1) { xv[row] = ok ? best : NAN; xi[row] = best_id; }
    epi_best = best; epi_id = best_id; epi_ok = ok; epi_row = row; epi_hf = hf;
  }
  __syncthreads();
  if (epi_hf == 0) {
    const float ov = reinterpret_cast<const float*>(smem + L::XCHG_OFF)[epi_row];
    const int oi = reinterpret_cast<const int*>(smem + L::XCHG_OFF + 512)[epi_row];
    if (epi_ok && ov == ov && row0 + epi_row < n) {
      const bool take = ov > epi_best || (ov == epi_best && oi < epi_id);
      assign_out[row0 + epi_row] = (take ? oi : epi_id) + id_offset;
    }
  }
  __syncthreads();
  if (*abort_flag) __nanosleep(50000);
  if (warp == 0) tmem_dealloc(tmem_base, L::TMEM_COLS);
}

// ------------------------------------------------------------------ counts
// Exclusive prefix of one int per thread over the block (up to 1024 threads); `total` receives the
// block's sum.  warp_tot: 32 ints of shared memory.
__device__ __forceinline__ int block_exclusive_scan(int v, int* warp_tot, int& total) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  int incl = v;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const int up = __shfl_up_sync(0xffffffffu, incl, o);
    if (lane >= o) incl += up;
  }
  if (lane == 31) warp_tot[warp] = incl;
  __syncthreads();
  if (warp == 0) {
    const int nw = (blockDim.x + 31) >> 5;
    const int t = lane < nw ? warp_tot[lane] : 0;
    int ti = t;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int up = __shfl_up_sync(0xffffffffu, ti, o);
      if (lane >= o) ti += up;
    }
    warp_tot[lane] = ti - t;                       // exclusive prefix of the warp totals
    if (lane == 31) warp_tot[32] = ti;             // the block's sum
  }
  __syncthreads();
  total = warp_tot[32];
  const int r = warp_tot[warp] + incl - v;
  __syncthreads();                                 // warp_tot may be reused by the caller's next scan
  return r;
}

__global__ void count_kernel(const int32_t* __restrict__ assign, int64_t n, int64_t head_stride,
                             int num_clusters, int32_t* __restrict__ counts) {
  const int h = blockIdx.y;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n;
       i += (int64_t)gridDim.x * blockDim.x) {
    int c = assign[h * head_stride + i];
    if ((unsigned)c < (unsigned)num_clusters) atomicAdd(&counts[h * num_clusters + c], 1);
  }
}

// One block per head: exclusive scans of the true and the page-padded sizes, the
// number of empty clusters and (for the k-means restart) the rank of each empty one.
__global__ void scan_counts_kernel(const int32_t* __restrict__ counts, int num_clusters, int align,
                                   int32_t* __restrict__ ip_orig,     // [H, C+1]
                                   int32_t* __restrict__ ip_pad,      // [H, C+1] or null
                                   int32_t* __restrict__ empty_rank,  // [H, C] or null
                                   int32_t* __restrict__ n_empty) {   // [H] or null
  __shared__ int warp_tot[33];
  const int h = blockIdx.x;
  const int* cnt = counts + (int64_t)h * num_clusters;
  const int per = (num_clusters + blockDim.x - 1) / blockDim.x;
  const int lo = min(num_clusters, (int)threadIdx.x * per), hi = min(num_clusters, lo + per);
  int a = 0, b = 0, e = 0;
  for (int c = lo; c < hi; ++c) {
    int v = cnt[c];
    a += v;
    b += align > 1 ? ((v + align - 1) / align) * align : v;
    e += v == 0;
  }
  int ra, rb, rc;
  a = block_exclusive_scan(a, warp_tot, ra);
  b = block_exclusive_scan(b, warp_tot, rb);
  e = block_exclusive_scan(e, warp_tot, rc);
  if (threadIdx.x == 0) {
    ip_orig[(int64_t)h * (num_clusters + 1) + num_clusters] = ra;
    if (ip_pad) ip_pad[(int64_t)h * (num_clusters + 1) + num_clusters] = rb;
    if (n_empty) n_empty[h] = rc;
  }
  for (int c = lo; c < hi; ++c) {
    int v = cnt[c];
    ip_orig[(int64_t)h * (num_clusters + 1) + c] = a;
    if (ip_pad) ip_pad[(int64_t)h * (num_clusters + 1) + c] = b;
    if (empty_rank) empty_rank[(int64_t)h * num_clusters + c] = v == 0 ? e : -1;
    a += v;
    b += align > 1 ? ((v + align - 1) / align) * align : v;
    e += v == 0;
  }
}

// The two kernels above in one block per head, for short inputs (a k-means sample): the histogram is
// taken in shared memory (num_clusters ints, dynamic) and scanned in place.
__global__ void count_scan_small_kernel(const int32_t* __restrict__ assign, int64_t n, int64_t head_stride,
                                        int num_clusters, int align, int32_t* __restrict__ counts,
                                        int32_t* __restrict__ ip_orig, int32_t* __restrict__ ip_pad,
                                        int32_t* __restrict__ empty_rank, int32_t* __restrict__ n_empty) {
  extern __shared__ int s_hist[];
  __shared__ int warp_tot[33];
  const int h = blockIdx.x;
  for (int c = threadIdx.x; c < num_clusters; c += blockDim.x) s_hist[c] = 0;
  __syncthreads();
  for (int64_t i = threadIdx.x; i < n; i += blockDim.x) {
    const int c = assign[h * head_stride + i];
    if ((unsigned)c < (unsigned)num_clusters) atomicAdd(&s_hist[c], 1);
  }
  __syncthreads();
  const int per = (num_clusters + blockDim.x - 1) / blockDim.x;
  const int lo = min(num_clusters, (int)threadIdx.x * per), hi = min(num_clusters, lo + per);
  int a = 0, b = 0, e = 0;
  for (int c = lo; c < hi; ++c) {
    const int v = s_hist[c];
    a += v;
    b += align > 1 ? ((v + align - 1) / align) * align : v;
    e += v == 0;
  }
  int ra, rb, rc;
  a = block_exclusive_scan(a, warp_tot, ra);
  b = block_exclusive_scan(b, warp_tot, rb);
  e = block_exclusive_scan(e, warp_tot, rc);
  if (threadIdx.x == 0) {
    ip_orig[(int64_t)h * (num_clusters + 1) + num_clusters] = ra;
    if (ip_pad) ip_pad[(int64_t)h * (num_clusters + 1) + num_clusters] = rb;
    if (n_empty) n_empty[h] = rc;
  }
  for (int c = lo; c < hi; ++c) {
    const int v = s_hist[c];
    counts[(int64_t)h * num_clusters + c] = v;
    ip_orig[(int64_t)h * (num_clusters + 1) + c] = a;
    if (ip_pad) ip_pad[(int64_t)h * (num_clusters + 1) + c] = b;
    if (empty_rank) empty_rank[(int64_t)h * num_clusters + c] = v == 0 ? e : -1;
    a += v;
    b += align > 1 ? ((v + align - 1) / align) * align : v;
    e += v == 0;
  }
}

// ------------------------------------------------------------------ stable radix sort by cluster id
constexpr int SORT_THREADS = 256;
constexpr int SORT_ITEMS = 8;
constexpr int SORT_TILE = SORT_THREADS * SORT_ITEMS;     // 2048 keys per block

__global__ void sort_hist_kernel(const int32_t* __restrict__ keys, int64_t n, int64_t head_stride,
                                 int shift, int ntiles, int32_t* __restrict__ tile_hist) {
  __shared__ int hist[256];
  const int h = blockIdx.y, tile = blockIdx.x;
  hist[threadIdx.x] = 0;
  __syncthreads();
  const int64_t base = (int64_t)tile * SORT_TILE;
  for (int i = threadIdx.x; i < SORT_TILE; i += SORT_THREADS) {
    int64_t p = base + i;
    if (p < n) atomicAdd(&hist[(keys[h * head_stride + p] >> shift) & 255], 1);
  }
  __syncthreads();
  tile_hist[((int64_t)h * 256 + threadIdx.x) * ntiles + tile] = hist[threadIdx.x];
}

// exclusive scan of [256 * ntiles] ints per head, in place (digit-major order)
__global__ void sort_scan_kernel(int32_t* __restrict__ tile_hist, int total) {
  __shared__ int warp_tot[33];
  int32_t* a = tile_hist + (int64_t)blockIdx.x * total;
  const int per = (total + blockDim.x - 1) / blockDim.x;
  const int lo = min(total, (int)threadIdx.x * per), hi = min(total, lo + per);
  int s = 0;
  for (int i = lo; i < hi; ++i) s += a[i];
  int sum;
  s = block_exclusive_scan(s, warp_tot, sum);
  for (int i = lo; i < hi; ++i) { int v = a[i]; a[i] = s; s += v; }
}

// Stable scatter of one tile.  Warp w owns keys [256 w, 256 w + 256) of the tile and
// ranks them in 8 rounds of 32 consecutive keys.
__global__ void sort_scatter_kernel(const int32_t* __restrict__ keys_in,
                                    const int32_t* __restrict__ vals_in,   // null: identity
                                    int64_t n, int64_t head_stride, int shift, int ntiles,
                                    const int32_t* __restrict__ tile_hist,
                                    int32_t* __restrict__ keys_out, int32_t* __restrict__ vals_out) {
  __shared__ int cnt[8][256];
  const int h = blockIdx.y, tile = blockIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int i = threadIdx.x; i < 8 * 256; i += SORT_THREADS) (&cnt[0][0])[i] = 0;
  __syncthreads();
  const int64_t base = (int64_t)tile * SORT_TILE + warp * 256;
  int key[SORT_ITEMS], val[SORT_ITEMS], rank[SORT_ITEMS];
#pragma unroll
  for (int r = 0; r < SORT_ITEMS; ++r) {
    const int64_t p = base + r * 32 + lane;
    const bool live = p < n;
    key[r] = live ? keys_in[h * head_stride + p] : 0;
    val[r] = live ? (vals_in ? vals_in[h * head_stride + p] : (int)p) : 0;
    const int d = live ? ((key[r] >> shift) & 255) : 256 + lane;   // dead lanes match nobody
    const unsigned m = __match_any_sync(0xffffffffu, d);
    const int leader = __ffs(m) - 1;
    int old = 0;
    if (live && lane == leader) { old = cnt[warp][d]; cnt[warp][d] = old + __popc(m); }
    old = __shfl_sync(0xffffffffu, old, leader);
    rank[r] = old + __popc(m & ((1u << lane) - 1));
    __syncwarp();
  }
  __syncthreads();
  {
    // per-digit exclusive prefix over the 8 warps, plus the tile's global base
    const int d = threadIdx.x;
    int run = tile_hist[((int64_t)h * 256 + d) * ntiles + tile];
#pragma unroll
    for (int w = 0; w < 8; ++w) { int v = cnt[w][d]; cnt[w][d] = run; run += v; }
  }
  __syncthreads();
#pragma unroll
  for (int r = 0; r < SORT_ITEMS; ++r) {
    const int64_t p = base + r * 32 + lane;
    if (p < n) {
      const int d = (key[r] >> shift) & 255;
      const int64_t dst = h * head_stride + cnt[warp][d] + rank[r];
      keys_out[dst] = key[r];
      vals_out[dst] = val[r];
    }
  }
}

// Stable arg-sort of up to 8192 keys below `bins` (a power of two up to 2048) per head in one block:
// warp w owns keys [1024 w, 1024 w + 1024) and ranks them in 32 rounds of 32 consecutive keys against
// its own counters; the counters are then turned into start offsets (over the keys, then over the warps).
constexpr int SMALL_SORT_MAX_N = 8192;
__global__ void __launch_bounds__(256)
small_argsort_kernel(const int32_t* __restrict__ keys, int n, int64_t head_stride, int bins,
                     int32_t* __restrict__ order) {
  extern __shared__ int cnt[];                     // [8 warps][bins], then [bins] totals
  __shared__ int warp_tot[33];
  int* tot = cnt + 8 * bins;
  const int h = blockIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int32_t* k = keys + (int64_t)h * head_stride;
  for (int i = threadIdx.x; i < 8 * bins; i += 256) cnt[i] = 0;
  __syncthreads();
  int key[32], rank[32];
#pragma unroll
  for (int r = 0; r < 32; ++r) {
    const int p = warp * 1024 + r * 32 + lane;
    const bool live = p < n;
    key[r] = live ? k[p] : 0;
    const int d = live ? (key[r] & (bins - 1)) : bins + lane;      // dead lanes match nobody
    const unsigned m = __match_any_sync(0xffffffffu, d);
    const int leader = __ffs(m) - 1;
    int old = 0;
    if (live && lane == leader) { old = cnt[warp * bins + d]; cnt[warp * bins + d] = old + __popc(m); }
    old = __shfl_sync(0xffffffffu, old, leader);
    rank[r] = old + __popc(m & ((1u << lane) - 1));
    __syncwarp();
  }
  __syncthreads();
  // totals per key, their exclusive scan over the keys, then per key the prefix over the warps
  const int per = bins / 256 > 0 ? bins / 256 : 1;
  int mine = 0;
  for (int j = 0; j < per; ++j) {
    const int d = threadIdx.x * per + j;
    int t = 0;
    if (d < bins) {
#pragma unroll
      for (int w = 0; w < 8; ++w) t += cnt[w * bins + d];
      tot[d] = t;
    }
    mine += t;
  }
  int all;
  int run = block_exclusive_scan(mine, warp_tot, all);
  for (int j = 0; j < per; ++j) {
    const int d = threadIdx.x * per + j;
    if (d < bins) {
      int start = run;
      run += tot[d];
#pragma unroll
      for (int w = 0; w < 8; ++w) { const int v = cnt[w * bins + d]; cnt[w * bins + d] = start; start += v; }
    }
  }
  __syncthreads();
  int32_t* o = order + (int64_t)h * head_stride;
#pragma unroll
  for (int r = 0; r < 32; ++r) {
    const int p = warp * 1024 + r * 32 + lane;
    if (p < n) o[cnt[warp * bins + (key[r] & (bins - 1))] + rank[r]] = p;
  }
}

// posting[h][row] for every padded row, and the position -> row map.
__global__ void fill_layout_kernel(const int32_t* __restrict__ order, int64_t n, int64_t head_stride,
                                   const int32_t* __restrict__ counts,
                                   const int32_t* __restrict__ ip_orig,
                                   const int32_t* __restrict__ ip_pad, int num_clusters,
                                   int32_t* __restrict__ posting, int64_t posting_stride,
                                   int32_t* __restrict__ inverse) {
  const int h = blockIdx.y;
  const int32_t* ipp = ip_pad + (int64_t)h * (num_clusters + 1);
  const int32_t* ipo = ip_orig + (int64_t)h * (num_clusters + 1);
  const int32_t* ord = order + h * head_stride;
  const int total = ipp[num_clusters];
  const int first = ord[0];
  for (int64_t r = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; r < posting_stride;
       r += (int64_t)gridDim.x * blockDim.x) {
    int value = first;
    if (r < total) {
      int lo = 0, hi = num_clusters;          // last c with ipp[c] <= r
      while (hi - lo > 1) {
        int mid = (lo + hi) >> 1;
        if (ipp[mid] <= r) lo = mid; else hi = mid;
      }
      const int off = (int)r - ipp[lo];
      if (off < counts[(int64_t)h * num_clusters + lo]) {
        value = ord[ipo[lo] + off];
        inverse[h * n + value] = (int)r;
      }
    }
    posting[h * posting_stride + r] = value;
  }
}

// ------------------------------------------------------------------ centroid update
// One block per cluster, thread = dimension; members are summed in index order
// (`order` is the stable sort of the sample by cluster), so the result does not
// depend on scheduling.  Empty clusters restart on sample[repl[rank]] with count 1.
__global__ void centroid_update_kernel(const float* __restrict__ sample, const int32_t* __restrict__ order,
                                       const int32_t* __restrict__ ip, const int32_t* __restrict__ empty_rank,
                                       const int64_t* __restrict__ repl, int dim,
                                       float* __restrict__ cent_f32, __nv_bfloat16* __restrict__ cent_bf16) {
  __shared__ double red[32];
  const int c = blockIdx.x;
  const int lo = ip[c], hi = ip[c + 1];
  const int d = threadIdx.x;
  float acc = 0.f;
  if (hi > lo) {
    // member ids through shared memory, eight rows in flight; the additions stay in index order
    __shared__ int32_t ids[256];
    for (int base = lo; base < hi; base += 256) {
      const int n = min(256, hi - base);
      __syncthreads();
      for (int t = threadIdx.x; t < n; t += blockDim.x) ids[t] = order[base + t];
      __syncthreads();
      if (d < dim) {
        int i = 0;
        for (; i + 8 <= n; i += 8) {
          float v[8];
#pragma unroll
          for (int u = 0; u < 8; ++u) v[u] = __ldg(sample + (int64_t)ids[i + u] * dim + d);
#pragma unroll
          for (int u = 0; u < 8; ++u) acc += v[u];
        }
        for (; i < n; ++i) acc += __ldg(sample + (int64_t)ids[i] * dim + d);
      }
    }
    acc = acc / (float)(hi - lo);
  } else if (repl != nullptr && d < dim) {
    acc = sample[repl[empty_rank[c]] * dim + d];
  }
  // normalise (F.normalize: x / max(|x|, 1e-12))
  double sq = (d < dim) ? (double)acc * (double)acc : 0.0;
  sq = warp_sum_d(sq);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = sq;
  __syncthreads();
  if (threadIdx.x < 32) {
    double v = threadIdx.x < (blockDim.x >> 5) ? red[threadIdx.x] : 0.0;
    v = warp_sum_d(v);
    if (threadIdx.x == 0) red[0] = v;
  }
  __syncthreads();
  const float nrm = fmaxf((float)sqrt(red[0]), 1e-12f);
  if (d < dim) {
    const float v = acc / nrm;
    cent_f32[(int64_t)c * dim + d] = v;
    if (cent_bf16) cent_bf16[(int64_t)c * dim + d] = __float2bfloat16_rn(v);
  }
}

// codebooks[2][C][D/2] (storage dtype bf16) = the two halves of normalize(cents)
__global__ void split_descriptor_kernel(const float* __restrict__ cents, int num_rows, int row_offset,
                                        int num_clusters, int dim, __nv_bfloat16* __restrict__ out) {
  const int lane = threadIdx.x & 31;
  const int c = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (c >= num_clusters) return;
  const int src = c - row_offset;
  double ss = 0.0;
  if (src >= 0 && src < num_rows)
    for (int d = lane; d < dim; d += 32) { float v = cents[(int64_t)src * dim + d]; ss += (double)v * v; }
  ss = warp_sum_d(ss);
  const float nrm = fmaxf((float)sqrt(ss), 1e-12f);
  const int half = dim / 2;
  for (int d = lane; d < dim; d += 32) {
    float v = (src >= 0 && src < num_rows) ? cents[(int64_t)src * dim + d] / nrm : 0.f;
    const int f = d >= half;
    out[((int64_t)f * num_clusters + c) * half + (d - f * half)] = __float2bfloat16_rn(v);
  }
}

// ------------------------------------------------------------------ pack
// packed[kv][row][h][:] = src_kv[posting[h][row]][h][:]; rows >= width are zero.
// One warp moves one (row, head) K and V vector with 16-byte accesses.
__global__ void pack_kv_kernel(const __nv_bfloat16* __restrict__ k, const __nv_bfloat16* __restrict__ v,
                               const int32_t* __restrict__ posting, int64_t posting_stride, int64_t width,
                               int64_t packed_rows, int num_kv_heads, int head_dim,
                               __nv_bfloat16* __restrict__ packed, int64_t kv_stride,
                               const int32_t* __restrict__ page_table) {
  const int lane = threadIdx.x & 31;
  const int64_t item = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (item >= packed_rows * num_kv_heads) return;
  const int64_t row = item / num_kv_heads;
  const int h = (int)(item % num_kv_heads);
  int64_t drow = row;
  if (page_table) drow = (int64_t)page_table[row >> 4] * 16 + (row & 15);
  const int chunks = head_dim / 8;      // 16-byte chunks per vector
  uint4* dk = reinterpret_cast<uint4*>(packed + (drow * num_kv_heads + h) * head_dim);
  uint4* dv = reinterpret_cast<uint4*>(packed + kv_stride + (drow * num_kv_heads + h) * head_dim);
  if (row < width) {
    const int64_t src = posting[h * posting_stride + row];
    const uint4* sk = reinterpret_cast<const uint4*>(k + (src * num_kv_heads + h) * head_dim);
    const uint4* sv = reinterpret_cast<const uint4*>(v + (src * num_kv_heads + h) * head_dim);
    for (int i = lane; i < chunks; i += 32) { dk[i] = sk[i]; dv[i] = sv[i]; }
  } else {
    for (int i = lane; i < chunks; i += 32) { dk[i] = make_uint4(0, 0, 0, 0); dv[i] = make_uint4(0, 0, 0, 0); }
  }
}

// sizes[h][c] += |{p in [lo, hi): assign[h][p] == c}|
__global__ void snapshot_advance_kernel(const int32_t* __restrict__ assign, int64_t head_stride,
                                        int64_t lo, int64_t hi, int num_clusters,
                                        int32_t* __restrict__ sizes) {
  const int h = blockIdx.y;
  for (int64_t p = lo + (int64_t)blockIdx.x * blockDim.x + threadIdx.x; p < hi;
       p += (int64_t)gridDim.x * blockDim.x) {
    int c = assign[h * head_stride + p];
    if ((unsigned)c < (unsigned)num_clusters) atomicAdd(&sizes[(int64_t)h * num_clusters + c], 1);
  }
}

int sort_by_cluster(const int32_t* keys, int64_t n, int64_t head_stride, int heads, int num_clusters,
                    int32_t* order_out, int32_t* tmp_keys, int32_t* tmp_vals, int32_t* tmp_keys2,
                    int32_t* tile_hist, cudaStream_t st) {
  const int ntiles = (int)ceil_div(n, SORT_TILE);
  const int passes = num_clusters <= 256 ? 1 : 2;
  const int32_t* kin = keys;
  const int32_t* vin = nullptr;
  for (int p = 0; p < passes; ++p) {
    int32_t* kout = (p == passes - 1) ? tmp_keys2 : tmp_keys;
    int32_t* vout = (p == passes - 1) ? order_out : tmp_vals;
    dim3 grid(ntiles, heads);
    sort_hist_kernel<<<grid, SORT_THREADS, 0, st>>>(kin, n, head_stride, 8 * p, ntiles, tile_hist);
    sort_scan_kernel<<<heads, 1024, 0, st>>>(tile_hist, 256 * ntiles);
    sort_scatter_kernel<<<grid, SORT_THREADS, 0, st>>>(kin, vin, n, head_stride, 8 * p, ntiles, tile_hist, kout, vout);
    kin = kout;
    vin = vout;
  }
  SEMBLO_LAUNCH_CHECK();
  return 0;
}

template <int D, bool SPLIT>
int launch_assign(const void* x, int64_t n, int64_t x_stride_elems, const void* cent, int num_centroids, int32_t* out,
                  int id_offset, const uint32_t* dead_bits, int* status, cudaStream_t st) {
  CUtensorMap mx, mc;
  uint64_t dx[2] = {(uint64_t)D, (uint64_t)n}, sx[1] = {(uint64_t)x_stride_elems * 2};
  uint32_t box[2] = {64, 128};
  int rc = semblo::make_tensor_map_bf16(&mx, x, 2, dx, sx, box);
  if (rc) return rc;
  if (SPLIT) {
    uint64_t dc[3] = {(uint64_t)D / 2, (uint64_t)num_centroids, 2};
    uint64_t sc[2] = {(uint64_t)D, (uint64_t)num_centroids * D};          // bytes: row, half
    uint32_t bc[3] = {64, (uint32_t)ASG_BN, 1};
    rc = semblo::make_tensor_map_bf16(&mc, cent, 3, dc, sc, bc);
  } else {
    uint64_t dc[2] = {(uint64_t)D, (uint64_t)num_centroids}, sc[1] = {(uint64_t)D * 2};
    uint32_t bc2[2] = {64, (uint32_t)ASG_BN};
    rc = semblo::make_tensor_map_bf16(&mc, cent, 2, dc, sc, bc2);
  }
  if (rc) return rc;
  auto kern = assign_argmax_kernel<D, SPLIT>;
  SEMBLO_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, AssignSmem<D>::TOTAL));
  kern<<<(unsigned)ceil_div(n, 128), 320, AssignSmem<D>::TOTAL, st>>>(mx, (const __nv_bfloat16*)x, x_stride_elems, mc, n,
                                                                    num_centroids, out, id_offset,
                                                                    dead_bits, status);
  SEMBLO_LAUNCH_CHECK();
  return 0;
}

// one warp per centroid of a descriptor pair [2][C][half]: bit set when every element is zero
__global__ void dead_descriptor_kernel(const __nv_bfloat16* __restrict__ cb, int num_centroids, int half,
                                       uint32_t* __restrict__ dead_bits) {
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  const int c = warp;
  bool nonzero = false;
  if (c < num_centroids) {
    for (int f = 0; f < 2; ++f)
      for (int d = lane; d < half; d += 32)
        nonzero |= (__bfloat16_as_ushort(cb[((int64_t)f * num_centroids + c) * half + d]) & 0x7fffu) != 0;
  }
  const bool any = __any_sync(0xffffffffu, nonzero);
  // clusters are consecutive per warp, 32 warps of 32 centroids share a word: set bits atomically
  if (lane == 0 && c < num_centroids && !any) atomicOr(dead_bits + (c >> 5), 1u << (c & 31));
}

}  // namespace

// ====================================================================== C ABI

extern "C" int semblo_routing_normalize(const void* x, int dtype, int64_t n_rows, int dim,
                                        int64_t row_stride, void* out, float* space_f32,
                                        void* space_bf16, int query_mode, void* stream) {
  SEMBLO_REQUIRE(dim > 0 && dim <= 256, "dim %d must be in (0, 256]", dim);
  SEMBLO_REQUIRE(dtype == SEMBLO_BF16 || dtype == SEMBLO_F32, "dtype %d is not bf16 or f32", dtype);
  if (n_rows == 0) return 0;
  cudaStream_t st = (cudaStream_t)stream;
  const int wpb = 8;
  dim3 grid((unsigned)ceil_div(n_rows, wpb));
  const bool vec = dtype == SEMBLO_BF16 && dim % 8 == 0 && dim <= 256 && row_stride % 8 == 0 &&
                   (reinterpret_cast<uintptr_t>(x) & 15) == 0 && (reinterpret_cast<uintptr_t>(out) & 15) == 0 &&
                   (reinterpret_cast<uintptr_t>(space_f32) & 15) == 0 &&
                   (reinterpret_cast<uintptr_t>(space_bf16) & 15) == 0;
  if (vec)
    normalize_rows_bf16x8_kernel<<<grid, wpb * 32, 0, st>>>((const __nv_bfloat16*)x, n_rows, dim, row_stride,
                                                          (__nv_bfloat16*)out, space_f32,
                                                          (__nv_bfloat16*)space_bf16, query_mode);
  else if (dtype == SEMBLO_BF16)
    normalize_rows_kernel<__nv_bfloat16, 256><<<grid, wpb * 32, 0, st>>>(
        (const __nv_bfloat16*)x, n_rows, dim, row_stride, (__nv_bfloat16*)out, space_f32,
        (__nv_bfloat16*)space_bf16, query_mode);
  else
    normalize_rows_kernel<float, 256><<<grid, wpb * 32, 0, st>>>(
        (const float*)x, n_rows, dim, row_stride, (float*)out, space_f32, (__nv_bfloat16*)space_bf16,
        query_mode);
  SEMBLO_LAUNCH_CHECK();
  return 0;
}

extern "C" int semblo_gather_rows(const float* src, const int64_t* idx, int64_t m, int dim,
                                  float* dst_f32, void* dst_bf16, void* stream) {
  if (m == 0) return 0;
  gather_rows_kernel<<<(unsigned)ceil_div(m, 8), 256, 0, (cudaStream_t)stream>>>(
      src, idx, m, dim, dst_f32, (__nv_bfloat16*)dst_bf16);
  SEMBLO_LAUNCH_CHECK();
  return 0;
}

extern "C" int semblo_assign_argmax(const void* x_bf16, int64_t n, const void* cent_bf16,
                                    int num_centroids, int dim, int32_t* assign_out, int id_offset,
                                    int32_t* status, void* stream) {
  SEMBLO_REQUIRE(num_centroids > 0, "no centroids");
  SEMBLO_REQUIRE(status != nullptr, "status word is required");
  if (n == 0) return 0;
  cudaStream_t st = (cudaStream_t)stream;
  switch (dim) {
    case 64: return launch_assign<64, false>(x_bf16, n, 64, cent_bf16, num_centroids, assign_out, id_offset, nullptr, status, st);
    case 128: return launch_assign<128, false>(x_bf16, n, 128, cent_bf16, num_centroids, assign_out, id_offset, nullptr, status, st);
    case 256: return launch_assign<256, false>(x_bf16, n, 256, cent_bf16, num_centroids, assign_out, id_offset, nullptr, status, st);
    default: return semblo::fail(semblo::SEMBLO_EINVAL, "routing dim %d is not 64, 128 or 256", dim);
  }
}

extern "C" int semblo_nearest_cluster(const void* keys_bf16, int64_t n, int num_kv_heads, int head_dim,
                                      const void* codebooks, int num_clusters, int32_t* ids_out,
                                      uint32_t* dead_bits_scratch, int32_t* status, void* stream) {
  SEMBLO_REQUIRE(num_clusters > 0 && num_clusters % 32 == 0, "cluster count %d must be a positive multiple of 32", num_clusters);
  SEMBLO_REQUIRE(status != nullptr && dead_bits_scratch != nullptr, "status word and scratch are required");
  SEMBLO_REQUIRE(head_dim == 128 || head_dim == 256, "head_dim %d must be 128 or 256", head_dim);
  if (n == 0) return 0;
  cudaStream_t st = (cudaStream_t)stream;
  const int words = num_clusters / 32;
  SEMBLO_CUDA(cudaMemsetAsync(dead_bits_scratch, 0, sizeof(uint32_t) * (size_t)num_kv_heads * words, st));
  for (int h = 0; h < num_kv_heads; ++h) {
    const __nv_bfloat16* cb = (const __nv_bfloat16*)codebooks + (int64_t)h * 2 * num_clusters * (head_dim / 2);
    uint32_t* dead = dead_bits_scratch + (int64_t)h * words;
    dead_descriptor_kernel<<<(unsigned)ceil_div(num_clusters, 8), 256, 0, st>>>(cb, num_clusters, head_dim / 2, dead);
    const __nv_bfloat16* x = (const __nv_bfloat16*)keys_bf16 + (int64_t)h * head_dim;
    int rc;
    if (head_dim == 256)
      rc = launch_assign<256, true>(x, n, (int64_t)num_kv_heads * 256, cb, num_clusters, ids_out + (int64_t)h * n, 0, dead, status, st);
    else
      rc = launch_assign<128, true>(x, n, (int64_t)num_kv_heads * 128, cb, num_clusters, ids_out + (int64_t)h * n, 0, dead, status, st);
    if (rc) return rc;
  }
  SEMBLO_LAUNCH_CHECK();
  return 0;
}

extern "C" int64_t semblo_layout_workspace_bytes(int64_t n, int heads) {
  const int64_t ntiles = ceil_div(n, SORT_TILE);
  // order, tmp keys, tmp vals, tmp keys2 (n each per head), tile hist, ip_orig is caller's
  return heads * (4 * n + 256 * ntiles) * (int64_t)sizeof(int32_t) + 1024;
}

extern "C" int semblo_cluster_counts(const int32_t* assign, int64_t n, int64_t head_stride, int heads,
                                     int num_clusters, int align, int32_t* counts, int32_t* ip_orig,
                                     int32_t* ip_pad, int32_t* empty_rank, int32_t* n_empty,
                                     void* stream) {
  cudaStream_t st = (cudaStream_t)stream;
  if (n > 0 && n <= 131072 && num_clusters <= 12288) {       // one launch: histogram and scans in shared memory
    count_scan_small_kernel<<<heads, 1024, (size_t)num_clusters * sizeof(int), st>>>(
        assign, n, head_stride, num_clusters, align, counts, ip_orig, ip_pad, empty_rank, n_empty);
    SEMBLO_LAUNCH_CHECK();
    return 0;
  }
  SEMBLO_CUDA(cudaMemsetAsync(counts, 0, sizeof(int32_t) * (size_t)heads * num_clusters, st));
  if (n > 0) {
    dim3 grid((unsigned)std::min<int64_t>(ceil_div(n, 256), 1184), heads);
    count_kernel<<<grid, 256, 0, st>>>(assign, n, head_stride, num_clusters, counts);
  }
  scan_counts_kernel<<<heads, 1024, 0, st>>>(counts, num_clusters, align, ip_orig, ip_pad, empty_rank, n_empty);
  SEMBLO_LAUNCH_CHECK();
  return 0;
}

extern "C" int semblo_kmeans_update(const float* sample, const int32_t* assign, int64_t n,
                                    int num_clusters, int dim, const int32_t* ip_orig,
                                    const int32_t* empty_rank, const int64_t* repl, float* cent_f32,
                                    void* cent_bf16, void* workspace, int64_t workspace_bytes,
                                    void* stream) {
  SEMBLO_REQUIRE(dim <= 256 && dim % 32 == 0, "dim %d must be a multiple of 32 up to 256", dim);
  SEMBLO_REQUIRE(workspace_bytes >= semblo_layout_workspace_bytes(n, 1), "workspace too small");
  cudaStream_t st = (cudaStream_t)stream;
  int32_t* ws = (int32_t*)workspace;
  int32_t *order = ws, *tk = ws + n, *tv = ws + 2 * n, *tk2 = ws + 3 * n, *th = ws + 4 * n;
  int rc = sort_by_cluster(assign, n, n, 1, num_clusters, order, tk, tv, tk2, th, st);
  if (rc) return rc;
  centroid_update_kernel<<<num_clusters, dim, 0, st>>>(sample, order, ip_orig, empty_rank, repl, dim,
                                                      cent_f32, (__nv_bfloat16*)cent_bf16);
  SEMBLO_LAUNCH_CHECK();
  return 0;
}

extern "C" int semblo_kmeans_sort_members(const int32_t* assign, int64_t n, int num_clusters, void* workspace,
                                          int64_t workspace_bytes, void* stream) {
  SEMBLO_REQUIRE(workspace_bytes >= semblo_layout_workspace_bytes(n, 1), "workspace too small");
  int32_t* ws = (int32_t*)workspace;
  return sort_by_cluster(assign, n, n, 1, num_clusters, ws, ws + n, ws + 2 * n, ws + 3 * n, ws + 4 * n,
                         (cudaStream_t)stream);
}

extern "C" int semblo_kmeans_update_sorted(const float* sample, int64_t n, int num_clusters, int dim,
                                           const int32_t* ip_orig, const int32_t* empty_rank,
                                           const int64_t* repl, float* cent_f32, void* cent_bf16,
                                           const void* workspace, int64_t workspace_bytes, void* stream) {
  SEMBLO_REQUIRE(dim <= 256 && dim % 32 == 0, "dim %d must be a multiple of 32 up to 256", dim);
  SEMBLO_REQUIRE(workspace_bytes >= semblo_layout_workspace_bytes(n, 1), "workspace too small");
  centroid_update_kernel<<<num_clusters, dim, 0, (cudaStream_t)stream>>>(
      sample, (const int32_t*)workspace, ip_orig, empty_rank, repl, dim, cent_f32, (__nv_bfloat16*)cent_bf16);
  SEMBLO_LAUNCH_CHECK();
  return 0;
}

extern "C" int semblo_split_descriptor(const float* cents, int num_rows, int row_offset,
                                       int num_clusters, int dim, void* codebook_bf16, void* stream) {
  split_descriptor_kernel<<<(unsigned)ceil_div(num_clusters, 8), 256, 0, (cudaStream_t)stream>>>(
      cents, num_rows, row_offset, num_clusters, dim, (__nv_bfloat16*)codebook_bf16);
  SEMBLO_LAUNCH_CHECK();
  return 0;
}

extern "C" int semblo_build_layout(const int32_t* assign, int64_t n, int heads, int num_clusters,
                                   int align, int32_t* posting, int64_t posting_stride,
                                   int32_t* indptr, int32_t* sizes, int32_t* inverse,
                                   void* workspace, int64_t workspace_bytes, void* stream) {
  SEMBLO_REQUIRE(n > 0 && heads > 0 && num_clusters > 0, "empty layout");
  SEMBLO_REQUIRE(num_clusters <= 65536, "at most 65536 clusters");
  SEMBLO_REQUIRE(workspace_bytes >= semblo_layout_workspace_bytes(n, heads) +
                                        (int64_t)heads * (num_clusters + 1) * 4,
                 "workspace too small");
  SEMBLO_REQUIRE(posting_stride >= n + (int64_t)num_clusters * (align > 1 ? align - 1 : 0),
                 "posting stride %lld cannot hold the padded layout", (long long)posting_stride);
  cudaStream_t st = (cudaStream_t)stream;
  int32_t* ws = (int32_t*)workspace;
  const int64_t hn = (int64_t)heads * n;
  int32_t *order = ws, *tk = ws + hn, *tv = ws + 2 * hn, *tk2 = ws + 3 * hn, *th = ws + 4 * hn;
  int32_t* ip_orig = th + (int64_t)heads * 256 * ceil_div(n, SORT_TILE);
  int rc = semblo_cluster_counts(assign, n, n, heads, num_clusters, align, sizes, ip_orig, indptr,
                                 nullptr, nullptr, stream);
  if (rc) return rc;
  rc = sort_by_cluster(assign, n, n, heads, num_clusters, order, tk, tv, tk2, th, st);
  if (rc) return rc;
  dim3 grid((unsigned)std::min<int64_t>(ceil_div(posting_stride, 256), 2368), heads);
  fill_layout_kernel<<<grid, 256, 0, st>>>(order, n, n, sizes, ip_orig, indptr, num_clusters, posting,
                                           posting_stride, inverse);
  SEMBLO_LAUNCH_CHECK();
  return 0;
}

extern "C" int semblo_pack_kv(const void* k, const void* v, const int32_t* posting,
                              int64_t posting_stride, int64_t width, int64_t packed_rows,
                              int num_kv_heads, int head_dim, void* packed, int64_t kv_stride_elems,
                              const int32_t* page_table, void* stream) {
  SEMBLO_REQUIRE(head_dim % 8 == 0, "head_dim %d must be a multiple of 8", head_dim);
  SEMBLO_REQUIRE(width <= packed_rows, "packed buffer has %lld rows, the posting list %lld",
                 (long long)packed_rows, (long long)width);
  const int64_t items = packed_rows * num_kv_heads;
  if (items == 0) return 0;
  pack_kv_kernel<<<(unsigned)ceil_div(items, 8), 256, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)k, (const __nv_bfloat16*)v, posting, posting_stride, width, packed_rows,
      num_kv_heads, head_dim, (__nv_bfloat16*)packed, kv_stride_elems, page_table);
  SEMBLO_LAUNCH_CHECK();
  return 0;
}

extern "C" int semblo_snapshot_advance(const int32_t* assign, int64_t head_stride, int heads,
                                       int64_t lo, int64_t hi, int num_clusters, int32_t* sizes,
                                       void* stream) {
  if (hi <= lo) return 0;
  dim3 grid((unsigned)std::min<int64_t>(ceil_div(hi - lo, 256), 1184), heads);
  snapshot_advance_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>(assign, head_stride, lo, hi,
                                                                  num_clusters, sizes);
  SEMBLO_LAUNCH_CHECK();
  return 0;
}

extern "C" int semblo_argsort_keys(const int32_t* keys, int64_t n, int heads, int max_key,
                                   int32_t* order, void* workspace, int64_t workspace_bytes,
                                   void* stream) {
  SEMBLO_REQUIRE(max_key > 0 && max_key <= 65536, "keys must be below 65536");
  SEMBLO_REQUIRE(workspace_bytes >= semblo_layout_workspace_bytes(n, heads), "workspace too small");
  if (n == 0) return 0;
  if (n <= SMALL_SORT_MAX_N && max_key <= 2048) {           // one launch: a block per head
    int bins = 32;
    while (bins < max_key) bins <<= 1;
    const size_t smem = (size_t)9 * bins * sizeof(int);
    if (smem > 48 * 1024)
      SEMBLO_CUDA(cudaFuncSetAttribute(small_argsort_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    small_argsort_kernel<<<heads, 256, smem, (cudaStream_t)stream>>>(keys, (int)n, n, bins, order);
    SEMBLO_LAUNCH_CHECK();
    return 0;
  }
  int32_t* ws = (int32_t*)workspace;
  const int64_t hn = (int64_t)heads * n;
  return sort_by_cluster(keys, n, n, heads, max_key, order, ws, ws + hn, ws + 2 * hn, ws + 3 * hn,
                         (cudaStream_t)stream);
}

// ====================================================================== streamed updates
// Keys that arrive after the index was fitted (token-order streamed prefill, suffix flush):
// nearest-centroid ids come from semblo_nearest_cluster; the kernels below turn them into packed
// rows and move K/V rows.  Reference behaviour restated here:
//   semblo/vllm_plugin/token_outer_prefill.py:66-87    append_rows (destination rows, counts)
//   semblo/vllm_plugin/token_outer_prefill.py:339-392  _append, _repack (row moves)
//   semblo/vllm_plugin/suffix_flush.py:56-133          repack_plan / repack_apply
namespace {

// sorted slot j of head h -> destination row of the key it holds
__global__ void append_rank_kernel(const int32_t* __restrict__ ids, const int32_t* __restrict__ order,
                                   const int32_t* __restrict__ starts /* [H, C+1] */,
                                   const int32_t* __restrict__ indptr, const int32_t* __restrict__ sizes,
                                   int64_t n, int num_clusters, int32_t* __restrict__ rows) {
  const int h = blockIdx.y;
  for (int64_t j = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; j < n; j += (int64_t)gridDim.x * blockDim.x) {
    const int t = order[h * n + j];
    const int c = ids[h * n + t];
    const int rank = (int)j - starts[(int64_t)h * (num_clusters + 1) + c];
    rows[h * n + t] = indptr[(int64_t)h * (num_clusters + 1) + c] + sizes[(int64_t)h * num_clusters + c] + rank;
  }
}

// one warp per (token, head): K/V row into the packed store, position and inverse entry
__global__ void scatter_kv_kernel(const __nv_bfloat16* __restrict__ k, const __nv_bfloat16* __restrict__ v,
                                  const int32_t* __restrict__ positions, int64_t n, int num_kv_heads, int head_dim,
                                  const int32_t* __restrict__ rows, int64_t rows_stride,
                                  __nv_bfloat16* __restrict__ packed, int64_t kv_stride_elems,
                                  int32_t* __restrict__ posting, int64_t posting_stride,
                                  int32_t* __restrict__ inverse, int64_t inverse_stride, int64_t inverse_offset,
                                  const int32_t* __restrict__ page_table, int64_t packed_rows,
                                  int32_t* __restrict__ status) {
  const int64_t item = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (item >= n * num_kv_heads) return;
  const int64_t i = item / num_kv_heads;
  const int h = (int)(item % num_kv_heads);
  if (*reinterpret_cast<const volatile int32_t*>(status) != 0) return;   // an earlier stage refused
  const int row = rows[h * rows_stride + i];
  if (row < 0 || row >= packed_rows) {               // the store is full: refuse, never write outside it
    if (lane == 0) atomicCAS(status, 0, STATUS_OVERFLOW);
    return;
  }
  const int64_t phys = page_table ? (int64_t)page_table[row >> 4] * 16 + (row & 15) : row;
  const uint4* ks = reinterpret_cast<const uint4*>(k + (i * num_kv_heads + h) * head_dim);
  const uint4* vs = reinterpret_cast<const uint4*>(v + (i * num_kv_heads + h) * head_dim);
  uint4* kd = reinterpret_cast<uint4*>(packed + (phys * num_kv_heads + h) * head_dim);
  uint4* vd = reinterpret_cast<uint4*>(packed + kv_stride_elems + (phys * num_kv_heads + h) * head_dim);
  for (int c = lane; c < head_dim / 8; c += 32) {
    kd[c] = ks[c];
    vd[c] = vs[c];
  }
  if (lane == 0) {
    if (posting) posting[h * posting_stride + row] = positions[i];
    if (inverse) inverse[h * inverse_stride + inverse_offset + i] = row;
  }
}

// one warp per (token, head): packed rows back into [n, Hkv, D]
__global__ void gather_kv_kernel(const __nv_bfloat16* __restrict__ packed, int64_t kv_stride_elems,
                                 const int32_t* __restrict__ rows, int64_t rows_stride, int64_t n, int num_kv_heads,
                                 int head_dim, __nv_bfloat16* __restrict__ out_k, __nv_bfloat16* __restrict__ out_v,
                                 const int32_t* __restrict__ page_table) {
  const int64_t item = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (item >= n * num_kv_heads) return;
  const int64_t i = item / num_kv_heads;
  const int h = (int)(item % num_kv_heads);
  const int row = rows[h * rows_stride + i];
  const int64_t phys = page_table ? (int64_t)page_table[row >> 4] * 16 + (row & 15) : row;
  const uint4* ks = reinterpret_cast<const uint4*>(packed + (phys * num_kv_heads + h) * head_dim);
  const uint4* vs = reinterpret_cast<const uint4*>(packed + kv_stride_elems + (phys * num_kv_heads + h) * head_dim);
  uint4* kd = reinterpret_cast<uint4*>(out_k + (i * num_kv_heads + h) * head_dim);
  uint4* vd = reinterpret_cast<uint4*>(out_v + (i * num_kv_heads + h) * head_dim);
  for (int c = lane; c < head_dim / 8; c += 32) {
    kd[c] = ks[c];
    vd[c] = vs[c];
  }
}

__global__ void relayout_rows_kernel(const int32_t* __restrict__ rows_old, const int32_t* __restrict__ bucket,
                                     int64_t n, int64_t stride, const int32_t* __restrict__ old_indptr,
                                     const int32_t* __restrict__ new_indptr, int num_clusters,
                                     int32_t* __restrict__ rows_new) {
  const int h = blockIdx.y;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
    const int b = bucket[h * stride + i];
    rows_new[h * stride + i] = rows_old[h * stride + i] - old_indptr[(int64_t)h * (num_clusters + 1) + b] +
                               new_indptr[(int64_t)h * (num_clusters + 1) + b];
  }
}

// Suffix flush: new sizes and 16-aligned starts of every cluster
__global__ void flush_layout_kernel(const int32_t* __restrict__ old_sizes, const int32_t* __restrict__ added,
                                    int num_clusters, int align, int32_t* __restrict__ new_sizes,
                                    int32_t* __restrict__ new_indptr /* [H, C+1] */, int64_t packed_rows,
                                    int32_t* __restrict__ status) {
  __shared__ int s_part[1024];
  const int h = blockIdx.x;
  const int per = (num_clusters + blockDim.x - 1) / blockDim.x;
  const int lo = min(num_clusters, (int)threadIdx.x * per), hi = min(num_clusters, lo + per);
  int sum = 0;
  for (int c = lo; c < hi; ++c) {
    const int v = old_sizes[(int64_t)h * num_clusters + c] + added[(int64_t)h * num_clusters + c];
    sum += ((v + align - 1) / align) * align;
  }
  s_part[threadIdx.x] = sum;
  __syncthreads();
  if (threadIdx.x == 0) {
    int run = 0;
    for (int t = 0; t < (int)blockDim.x; ++t) { const int v = s_part[t]; s_part[t] = run; run += v; }
    new_indptr[(int64_t)h * (num_clusters + 1) + num_clusters] = run;
    if (run > packed_rows) atomicCAS(status, 0, STATUS_OVERFLOW);   // the re-packed store does not fit: nothing moves
  }
  __syncthreads();
  int run = s_part[threadIdx.x];
  for (int c = lo; c < hi; ++c) {
    const int v = old_sizes[(int64_t)h * num_clusters + c] + added[(int64_t)h * num_clusters + c];
    new_sizes[(int64_t)h * num_clusters + c] = v;
    new_indptr[(int64_t)h * (num_clusters + 1) + c] = run;
    run += ((v + align - 1) / align) * align;
  }
}

// Suffix flush: the new sizes and starts replace the old ones unless the flush was refused.
__global__ void flush_commit_kernel(const int32_t* __restrict__ new_sizes, const int32_t* __restrict__ new_indptr,
                                    int64_t n_sizes, int64_t n_indptr, int32_t* __restrict__ sizes,
                                    int32_t* __restrict__ indptr, const int32_t* __restrict__ status) {
  if (*reinterpret_cast<const volatile int32_t*>(status) != 0) return;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n_indptr; i += (int64_t)gridDim.x * blockDim.x) {
    if (i < n_sizes) sizes[i] = new_sizes[i];
    indptr[i] = new_indptr[i];
  }
}

// Suffix flush: one warp per (new row, head).  Old rows move from the copy of the old store,
// padding rows repeat the old row 0 (K/V and position); rows of flushed tokens are left to
// the scatter that follows.
__global__ void flush_move_kernel(const __nv_bfloat16* __restrict__ old_packed, const int32_t* __restrict__ old_posting,
                                  int64_t old_kv_stride_elems, int64_t posting_stride,
                                  const int32_t* __restrict__ old_sizes, const int32_t* __restrict__ old_indptr,
                                  const int32_t* __restrict__ new_sizes, const int32_t* __restrict__ new_indptr,
                                  int num_clusters, int num_kv_heads, int head_dim, int64_t max_rows,
                                  __nv_bfloat16* __restrict__ packed, int64_t kv_stride_elems,
                                  int32_t* __restrict__ posting, const int32_t* __restrict__ status) {
  const int64_t item = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (item >= max_rows * num_kv_heads) return;
  if (*reinterpret_cast<const volatile int32_t*>(status) != 0) return;
  const int64_t r = item / num_kv_heads;
  const int h = (int)(item % num_kv_heads);
  const int32_t* nip = new_indptr + (int64_t)h * (num_clusters + 1);
  if (r >= nip[num_clusters]) return;
  int lo = 0, hi = num_clusters;                      // last c with nip[c] <= r
  while (hi - lo > 1) {
    const int mid = (lo + hi) >> 1;
    if (nip[mid] <= r) lo = mid; else hi = mid;
  }
  const int c = lo;
  const int off = (int)r - nip[c];
  const int osz = old_sizes[(int64_t)h * num_clusters + c];
  int64_t src;
  if (off < osz) src = old_indptr[(int64_t)h * (num_clusters + 1) + c] + off;
  else if (off < new_sizes[(int64_t)h * num_clusters + c]) return;      // a flushed token's row
  else src = 0;
  const uint4* ks = reinterpret_cast<const uint4*>(old_packed + (src * num_kv_heads + h) * head_dim);
  const uint4* vs = reinterpret_cast<const uint4*>(old_packed + old_kv_stride_elems + (src * num_kv_heads + h) * head_dim);
  uint4* kd = reinterpret_cast<uint4*>(packed + (r * num_kv_heads + h) * head_dim);
  uint4* vd = reinterpret_cast<uint4*>(packed + kv_stride_elems + (r * num_kv_heads + h) * head_dim);
  for (int ch = lane; ch < head_dim / 8; ch += 32) {
    kd[ch] = ks[ch];
    vd[ch] = vs[ch];
  }
  if (lane == 0) posting[h * posting_stride + r] = old_posting[h * posting_stride + src];
}

}  // namespace

extern "C" int semblo_append_rows(const int32_t* ids, int64_t n, int heads, int num_clusters,
                                  const int32_t* indptr, const int32_t* sizes, int32_t* rows, int32_t* counts,
                                  void* workspace, int64_t workspace_bytes, void* stream) {
  SEMBLO_REQUIRE(num_clusters > 0 && num_clusters <= 65536 && heads > 0, "bad cluster or head count");
  SEMBLO_REQUIRE(workspace_bytes >= semblo_layout_workspace_bytes(n, heads) + (int64_t)heads * (num_clusters + 1) * 4,
                 "workspace too small");
  cudaStream_t st = (cudaStream_t)stream;
  if (n == 0) {
    SEMBLO_CUDA(cudaMemsetAsync(counts, 0, sizeof(int32_t) * (size_t)heads * num_clusters, st));
    return 0;
  }
  int32_t* ws = (int32_t*)workspace;
  const int64_t hn = (int64_t)heads * n;
  int32_t *order = ws, *tk = ws + hn, *tv = ws + 2 * hn, *tk2 = ws + 3 * hn, *th = ws + 4 * hn;
  int32_t* starts = th + (int64_t)heads * 256 * ceil_div(n, SORT_TILE);
  int rc = semblo_cluster_counts(ids, n, n, heads, num_clusters, 1, counts, starts, nullptr, nullptr, nullptr, stream);
  if (rc) return rc;
  rc = sort_by_cluster(ids, n, n, heads, num_clusters, order, tk, tv, tk2, th, st);
  if (rc) return rc;
  dim3 grid((unsigned)std::min<int64_t>(ceil_div(n, 256), 1184), heads);
  append_rank_kernel<<<grid, 256, 0, st>>>(ids, order, starts, indptr, sizes, n, num_clusters, rows);
  SEMBLO_LAUNCH_CHECK();
  return 0;
}

extern "C" int semblo_scatter_kv(const void* k, const void* v, const int32_t* positions, int64_t n,
                                 int num_kv_heads, int head_dim, const int32_t* rows, int64_t rows_stride,
                                 void* packed, int64_t packed_rows, int64_t kv_stride_elems, int32_t* posting,
                                 int64_t posting_stride, int32_t* inverse, int64_t inverse_stride,
                                 int64_t inverse_offset, const int32_t* page_table, int32_t* status, void* stream) {
  SEMBLO_REQUIRE(head_dim % 8 == 0, "head_dim %d must be a multiple of 8", head_dim);
  SEMBLO_REQUIRE(status != nullptr, "status word is required");
  SEMBLO_REQUIRE(posting == nullptr || positions != nullptr, "positions are needed to fill the posting list");
  const int64_t items = n * num_kv_heads;
  if (items == 0) return 0;
  scatter_kv_kernel<<<(unsigned)ceil_div(items, 8), 256, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)k, (const __nv_bfloat16*)v, positions, n, num_kv_heads, head_dim, rows, rows_stride,
      (__nv_bfloat16*)packed, kv_stride_elems, posting, posting_stride, inverse, inverse_stride, inverse_offset,
      page_table, packed_rows, status);
  SEMBLO_LAUNCH_CHECK();
  return 0;
}

extern "C" int semblo_gather_kv(const void* packed, int64_t kv_stride_elems, const int32_t* rows,
                                int64_t rows_stride, int64_t n, int num_kv_heads, int head_dim, void* out_k,
                                void* out_v, const int32_t* page_table, void* stream) {
  SEMBLO_REQUIRE(head_dim % 8 == 0, "head_dim %d must be a multiple of 8", head_dim);
  const int64_t items = n * num_kv_heads;
  if (items == 0) return 0;
  gather_kv_kernel<<<(unsigned)ceil_div(items, 8), 256, 0, (cudaStream_t)stream>>>(
      (const __nv_bfloat16*)packed, kv_stride_elems, rows, rows_stride, n, num_kv_heads, head_dim,
      (__nv_bfloat16*)out_k, (__nv_bfloat16*)out_v, page_table);
  SEMBLO_LAUNCH_CHECK();
  return 0;
}

extern "C" int semblo_relayout_rows(const int32_t* rows_old, const int32_t* bucket, int64_t n, int64_t stride,
                                    int heads, const int32_t* old_indptr, const int32_t* new_indptr,
                                    int num_clusters, int32_t* rows_new, void* stream) {
  if (n == 0) return 0;
  dim3 grid((unsigned)std::min<int64_t>(ceil_div(n, 256), 1184), heads);
  relayout_rows_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>(rows_old, bucket, n, stride, old_indptr, new_indptr,
                                                              num_clusters, rows_new);
  SEMBLO_LAUNCH_CHECK();
  return 0;
}

extern "C" int64_t semblo_flush_workspace_bytes(int64_t n, int heads, int num_clusters) {
  // append_rows workspace, then added [H, C], new_sizes [H, C], new_indptr [H, C+1], rows [H, n]
  return semblo_layout_workspace_bytes(n, heads) + (int64_t)heads * (num_clusters + 1) * 4 +
         ((int64_t)heads * (3 * (int64_t)num_clusters + 1) + (int64_t)heads * n) * 4 + 1024;
}

extern "C" int semblo_flush_repack(void* packed, int64_t kv_stride_elems, int64_t packed_rows, int32_t* posting,
                                   int64_t posting_stride, int32_t* sizes, int32_t* indptr, int num_clusters,
                                   int num_kv_heads, int head_dim, int align, const void* flushed_k,
                                   const void* flushed_v, const int32_t* flushed_pos, const int32_t* assign,
                                   int64_t n, void* old_packed_copy, int32_t* old_posting_copy, void* workspace,
                                   int64_t workspace_bytes, int32_t* status, void* stream) {
  SEMBLO_REQUIRE(align >= 1 && head_dim % 8 == 0, "bad alignment or head_dim");
  SEMBLO_REQUIRE(workspace_bytes >= semblo_flush_workspace_bytes(n, num_kv_heads, num_clusters), "workspace too small");
  SEMBLO_REQUIRE(old_packed_copy != nullptr && old_posting_copy != nullptr, "a copy of the old store is required");
  SEMBLO_REQUIRE(status != nullptr, "status word is required");
  // old_posting_copy rows are packed_rows apart and the move kernel indexes both postings with one stride
  SEMBLO_REQUIRE(posting_stride == packed_rows, "the posting list and the packed store must have the same row count");
  if (n == 0) return 0;
  cudaStream_t st = (cudaStream_t)stream;
  const int H = num_kv_heads, C = num_clusters;
  uint8_t* wsb = (uint8_t*)workspace;
  const int64_t append_bytes = semblo_layout_workspace_bytes(n, H) + (int64_t)H * (C + 1) * 4;
  int32_t* added = (int32_t*)(wsb + ((append_bytes + 255) / 256) * 256);
  int32_t* new_sizes = added + (int64_t)H * C;
  int32_t* new_indptr = new_sizes + (int64_t)H * C;
  int32_t* rows = new_indptr + (int64_t)H * (C + 1);
  // the old store, to read from while the live one is rewritten
  const size_t plane_bytes = (size_t)packed_rows * H * head_dim * 2;
  SEMBLO_CUDA(cudaMemcpyAsync(old_packed_copy, packed, plane_bytes, cudaMemcpyDeviceToDevice, st));
  SEMBLO_CUDA(cudaMemcpyAsync((__nv_bfloat16*)old_packed_copy + (int64_t)packed_rows * H * head_dim,
                              (const __nv_bfloat16*)packed + kv_stride_elems, plane_bytes, cudaMemcpyDeviceToDevice, st));
  SEMBLO_CUDA(cudaMemcpy2DAsync(old_posting_copy, (size_t)packed_rows * 4, posting, (size_t)posting_stride * 4,
                                (size_t)packed_rows * 4, H, cudaMemcpyDeviceToDevice, st));
  // counts of the flushed tokens, the new layout, then the flushed tokens' rows in it
  int rc = semblo_cluster_counts(assign, n, n, H, C, 1, added, new_indptr /* scratch, rewritten below */, nullptr,
                                 nullptr, nullptr, stream);
  if (rc) return rc;
  flush_layout_kernel<<<H, 1024, 0, st>>>(sizes, added, C, align, new_sizes, new_indptr, packed_rows, status);
  rc = semblo_append_rows(assign, n, H, C, new_indptr, sizes, rows, added, workspace, append_bytes, stream);
  if (rc) return rc;
  flush_move_kernel<<<(unsigned)ceil_div(packed_rows * H, 8), 256, 0, st>>>(
      (const __nv_bfloat16*)old_packed_copy, old_posting_copy, (int64_t)packed_rows * H * head_dim, posting_stride,
      sizes, indptr, new_sizes, new_indptr, C, H, head_dim, packed_rows, (__nv_bfloat16*)packed, kv_stride_elems,
      posting, status);
  rc = semblo_scatter_kv(flushed_k, flushed_v, flushed_pos, n, H, head_dim, rows, n, packed, packed_rows,
                         kv_stride_elems, posting, posting_stride, nullptr, 0, 0, nullptr, status, stream);
  if (rc) return rc;
  flush_commit_kernel<<<32, 256, 0, st>>>(new_sizes, new_indptr, (int64_t)H * C, (int64_t)H * (C + 1), sizes, indptr, status);
  SEMBLO_LAUNCH_CHECK();
  return 0;
}

// ====================================================================== no-allocation arg-sort
//
// semblo_argsort_keys with its scratch in a fixed array inside the library image instead of a
// caller-provided workspace.  Every scratch word is written by the sort before it is read, so
// nothing has to start at zero; all calls on a device share the one array.
namespace {

constexpr int64_t STATIC_SORT_MAX_KEYS = 65536;     // heads * n
constexpr int STATIC_SORT_MAX_HEADS = 64;
constexpr int64_t STATIC_SORT_HIST_WORDS = 256 * (STATIC_SORT_MAX_KEYS / SORT_TILE + STATIC_SORT_MAX_HEADS);
constexpr int64_t STATIC_SORT_WORDS = 4 * STATIC_SORT_MAX_KEYS + STATIC_SORT_HIST_WORDS;

static __device__ __align__(256) int32_t g_static_sort_scratch[STATIC_SORT_WORDS];

constexpr int STATIC_MAX_DEVICES = 64;
int32_t* g_static_sort_ptr[STATIC_MAX_DEVICES] = {};
std::mutex g_static_sort_mutex;

// Address of the scratch array on the current device, looked up once per device.
int static_sort_scratch(int32_t** out) {
  int dev = -1;
  SEMBLO_CUDA(cudaGetDevice(&dev));
  SEMBLO_REQUIRE(dev >= 0 && dev < STATIC_MAX_DEVICES, "device ordinal %d out of range", dev);
  std::lock_guard<std::mutex> lock(g_static_sort_mutex);
  if (!g_static_sort_ptr[dev]) {
    int32_t* p = nullptr;
    SEMBLO_CUDA(cudaGetSymbolAddress((void**)&p, g_static_sort_scratch));
    SEMBLO_REQUIRE(p != nullptr, "the scratch array has no address on device %d", dev);
    g_static_sort_ptr[dev] = p;
  }
  *out = g_static_sort_ptr[dev];
  return 0;
}

}  // namespace

extern "C" int64_t semblo_argsort_keys_static_max_keys(void) { return STATIC_SORT_MAX_KEYS; }

extern "C" int semblo_argsort_keys_static(const int32_t* keys, int64_t n, int heads, int max_key,
                                          int32_t* order, void* stream) {
  SEMBLO_REQUIRE(max_key > 0 && max_key <= 65536, "keys must be below 65536");
  SEMBLO_REQUIRE(n >= 0 && heads > 0 && heads <= STATIC_SORT_MAX_HEADS,
                 "heads %d outside [1, %d] of the fixed scratch", heads, STATIC_SORT_MAX_HEADS);
  SEMBLO_REQUIRE((int64_t)heads * n <= STATIC_SORT_MAX_KEYS,
                 "heads * n = %lld keys exceed the fixed scratch of %lld keys; use semblo_argsort_keys "
                 "with a workspace", (long long)((int64_t)heads * n), (long long)STATIC_SORT_MAX_KEYS);
  int32_t* ws = nullptr;
  int rc = static_sort_scratch(&ws);
  if (rc) return rc;
  if (n == 0) return 0;
  const int64_t hn = (int64_t)heads * n;
  return sort_by_cluster(keys, n, n, heads, max_key, order, ws, ws + hn, ws + 2 * hn, ws + 3 * hn,
                         (cudaStream_t)stream);
}
