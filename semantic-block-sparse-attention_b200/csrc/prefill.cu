// Exact causal window attention on tcgen05 / TMEM: the dense-prefix chunks and the
// local window of every sparse chunk.
//
// One CTA owns a tile of QT = 128 / G consecutive queries of one KV head (128 rows:
// query-major, the G heads of a query adjacent).  The output accumulator O [128, D], the
// query operand Q [128, D] and the probabilities P all live in TMEM, so shared memory is
// K / V stages only.  The producer streams positions [local_start, max q_pos of the
// tile] of the position-ordered K/V through TMA in 64-row tiles; S = Q K^T (UMMA, Q read
// from TMEM, fp32 result in TMEM), the softmax warps (two threads per row) apply the causal
// mask, keep a lazily rescaled running max and store P as bf16 over S, and O += P V is a
// second UMMA with P read from TMEM and V as an MN-major operand.  The kernel writes the
// normalised output and its log-sum-exp, which the sparse launch merges into.
//
// Reference behaviour restated here:
//   semblo/vllm_plugin/fused_prefill.py:155-189  exact dense attention for short prefixes
//   semblo/vllm_plugin/kv_outer.py:661-676       the chunk's own causal window
//   semblo/vllm_plugin/fused_prefill.py:250-279  window start / dense-prefix rule (caller)
#include <algorithm>
#include <climits>

#include "../../include/semblo_b200.h"
#include "host_common.h"
#include "attn_common.cuh"
#include "sm100.cuh"

using namespace sm100;
using semblo::ceil_div;

namespace {

constexpr int PAGE = 16;
constexpr int PAGES_PER_TILE = 4;
constexpr int BLOCK_N = PAGE * PAGES_PER_TILE;     // 64 keys per tile

struct TileInfo {
  int npages;          // 16-row groups in the tile, 0 = end of stream
  int rows;            // valid rows
  int kpos0;           // position of row 0
  int pad;
};

template <int D>
struct AttnCfg {
  static constexpr int STAGES = D >= 256 ? 3 : 6;
  static constexpr int KV_BYTES = BLOCK_N * D * 2;
  static constexpr int K_OFF = 0;
  static constexpr int V_OFF = K_OFF + STAGES * KV_BYTES;
  static constexpr int EPI_OFF = V_OFF + STAGES * KV_BYTES;   // float [2][128]
  static constexpr int MX_OFF = EPI_OFF + 2048;               // float [2][2][128]: half-row maxima
  static constexpr int BAR_OFF = MX_OFF + 2048;
  static constexpr int INFO_OFF = BAR_OFF + 256;
  static constexpr int TOTAL = INFO_OFF + STAGES * (int)sizeof(TileInfo) + 64;   // 1024-byte aligned base
  static constexpr int TMEM_COLS = 512;
  static constexpr int O_COL = 2 * BLOCK_N;                    // S/P buffers, then O, then Q
  static constexpr int Q_COL = O_COL + D;
  static_assert(Q_COL + D / 2 <= TMEM_COLS, "tensor memory budget");
};

struct PrefillArgs {
  int num_queries;
  int num_q_heads;
  int num_kv_heads;
  int num_clusters;
  const __nv_bfloat16* q;         // [Q, Hq, D]
  const int32_t* q_positions;     // [Q]
  int local_start;                // first position of the window (do_local)
  int local_pos0;                 // position held by row 0 of the position-ordered K/V
  int local_rows;                 // rows in the position-ordered K/V
  float scale_log2;               // sm_scale * log2(e)
  __nv_bfloat16* out;             // [Q, Hq, D]
  float* lse;                     // [Q, Hq] or null
  float* partial;                 // [Q, Hq, D] fp32: written instead of `out` when not null
  unsigned long long* attended;   // sum over (query, KV head) of attended keys, or null
  int* status;
};

// barrier slots
enum { B_QFULL = 0, B_OREADY = 1, B_SFULL = 2, B_PFULL = 4, B_PVDONE = 6, B_EPI = 8, B_PAIR = 9, B_KVFULL = 13 };

template <int D, int G>
__global__ void __launch_bounds__(320, 1)
window_prefill_kernel(const __grid_constant__ CUtensorMap tmap_ok,
                      const __grid_constant__ CUtensorMap tmap_ov, const PrefillArgs a) {
  using C = AttnCfg<D>;
  constexpr int QT = 128 / G;
  constexpr int STAGES = C::STAGES;
  constexpr int B_KVEMPTY = B_KVFULL + STAGES;
  static_assert(8 * (B_KVEMPTY + STAGES) <= 256, "barrier area");
  extern __shared__ __align__(1024) uint8_t smem[];
  if (smem_u32(smem) & 1023u) {                    // the swizzled tiles need 1024-byte alignment
    if (threadIdx.x == 0) atomicCAS(a.status, 0, STATUS_SMEM_ALIGN);
    return;
  }
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + C::BAR_OFF);
  TileInfo* info = reinterpret_cast<TileInfo*>(smem + C::INFO_OFF);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + C::INFO_OFF + STAGES * sizeof(TileInfo));
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  auto bar = [&](int i) { return smem_u32(&bars[i]); };

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int h = blockIdx.y;
  // later queries see more keys: the longest tiles start first, so the launch ends evenly
  const int q_tile0 = (int)(gridDim.x - 1 - blockIdx.x) * QT;

  if (threadIdx.x == 0) {
    mbar_init(bar(B_QFULL), 256);
    mbar_init(bar(B_OREADY), 1);
    mbar_init(bar(B_EPI), 256);
    for (int i = 0; i < 4; ++i) mbar_init(bar(B_PAIR + i), 2);    // the two warps that share 32 rows
    for (int b = 0; b < 2; ++b) {
      mbar_init(bar(B_SFULL + b), 1);
      mbar_init(bar(B_PFULL + b), 8);         // the softmax warps
      mbar_init(bar(B_PVDONE + b), 1);
    }
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(bar(B_KVFULL + s), 1);
      mbar_init(bar(B_KVEMPTY + s), 9);     // eight softmax warps + the UMMA commit
    }
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 0) {
    tmem_alloc(smem_u32(tmem_slot), C::TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 8) {
    // ------------------------------------------------------------ producer
    const int slot = q_tile0 + lane;
    const bool qvalid = lane < QT && slot < a.num_queries;
    const int qpos = qvalid ? a.q_positions[slot] : -1;
    int max_qpos = qpos;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) max_qpos = max(max_qpos, __shfl_xor_sync(0xffffffffu, max_qpos, o));
    if (lane == 0) {
      tma_prefetch_desc(&tmap_ok);
      tma_prefetch_desc(&tmap_ov);
      const int last = min(max_qpos, a.local_pos0 + a.local_rows - 1);
      int tile = 0;
      bool ok = true;
      for (int p = a.local_start; p <= last && ok; p += BLOCK_N, ++tile) {
        const int s = tile % STAGES;
        ok = mbar_wait(bar(B_KVEMPTY + s), ((tile / STAGES) & 1) ^ 1, abort_flag, a.status, STATUS_TIMEOUT_LOAD);
        if (!ok) break;
        const int rows = min(BLOCK_N, last - p + 1);
        info[s].npages = (rows + PAGE - 1) / PAGE;
        info[s].rows = rows;
        info[s].kpos0 = p;
        mbar_arrive_expect_tx(bar(B_KVFULL + s), (uint32_t)BLOCK_N * D * 2 * 2);
        for (int sl = 0; sl < D / 64; ++sl) {
          tma_load_2d(smem_u32(smem + C::K_OFF + s * C::KV_BYTES + sl * BLOCK_N * 128), &tmap_ok,
                      bar(B_KVFULL + s), h * D + sl * 64, p - a.local_pos0);
          tma_load_2d(smem_u32(smem + C::V_OFF + s * C::KV_BYTES + sl * BLOCK_N * 128), &tmap_ov,
                      bar(B_KVFULL + s), h * D + sl * 64, p - a.local_pos0);
        }
      }
      if (ok) {
        const int s = tile % STAGES;
        ok = mbar_wait(bar(B_KVEMPTY + s), ((tile / STAGES) & 1) ^ 1, abort_flag, a.status, STATUS_TIMEOUT_LOAD);
        if (ok) {
          info[s].npages = 0;
          mbar_arrive(bar(B_KVFULL + s));
        }
      }
    }
  } else if (warp == 9) {
    // ------------------------------------------------------------ UMMA issuer
    // One thread issues S(j) = Q K(j)^T and O += P(t) V(t) in the fixed order S(0), S(1), then
    // P V(t), S(t + 2) for t = 0, 1, ...  UMMAs of one thread execute in issue order, so S(t + 2)
    // may follow P V(t), which reads P from the same buffer, without waiting for it to complete.
    if (elect_one()) {
      constexpr uint32_t idesc_pv = make_idesc_bf16(128, D, false, true);
      bool ok = mbar_wait(bar(B_QFULL), 0, abort_flag, a.status, STATUS_TIMEOUT_MMA);
      tc_fence_after();
      int end_tile = INT_MAX;
      int qs = 0;                                      // stage of the next S product
      uint32_t q_par = 0;
      auto issue_s = [&](int j) {
        ok = mbar_wait(bar(B_KVFULL + qs), q_par, abort_flag, a.status, STATUS_TIMEOUT_MMA);
        if (!ok) return;
        const int np = info[qs].npages;
        if (np == 0) { end_tile = j; return; }
        tc_fence_after();
        const int b = j & 1;
        const uint32_t k_base = smem_u32(smem + C::K_OFF + qs * C::KV_BYTES);
        const uint32_t idesc_qk = make_idesc_bf16(128, np * PAGE, false, false);
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint32_t sl = kk >> 2, ko = (kk & 3) * 32;
          umma_ts(tmem_base + b * BLOCK_N, tmem_base + C::Q_COL + kk * 8,
                  make_smem_desc(k_base + sl * BLOCK_N * 128 + ko, 16, 1024), idesc_qk, kk > 0 ? 1u : 0u);
        }
        umma_commit(bar(B_SFULL + b));
        if (++qs == STAGES) { qs = 0; q_par ^= 1; }
      };
      for (int j = 0; j < 2 && ok && end_tile == INT_MAX; ++j) issue_s(j);
      int vs = 0;
      for (int t = 0; ok && t < end_tile; ++t) {
        const int b = t & 1;
        ok = mbar_wait(bar(B_PFULL + b), (uint32_t)((t >> 1) & 1), abort_flag, a.status, STATUS_TIMEOUT_MMA);
        if (!ok) break;
        tc_fence_after();
        const int np = info[vs].npages;                // the stage is held until this product's commit
        const uint32_t v_base = smem_u32(smem + C::V_OFF + vs * C::KV_BYTES);
        for (int kk = 0; kk < np; ++kk)
          umma_ts(tmem_base + C::O_COL, tmem_base + b * BLOCK_N + (kk >> 1) * 32 + (kk & 1) * 8,
                  make_smem_desc(v_base + kk * PAGE * 128, BLOCK_N * 128, 1024), idesc_pv,
                  (t > 0 || kk > 0) ? 1u : 0u);
        umma_commit(bar(B_KVEMPTY + vs));
        umma_commit(bar(B_PVDONE + b));
        if (++vs == STAGES) vs = 0;
        if (end_tile == INT_MAX) issue_s(t + 2);
      }
      if (ok) umma_commit(bar(B_OREADY));
    }
  } else {
    // ------------------------------------------------------------ softmax + epilogue
    // warps 0-3 take columns [0, 32) of every tile and warps 4-7 columns [32, 64); thread = row
    const int hf = (warp >> 2) & 1;
    const int row = threadIdx.x & 127;
    const int qslot = row / G, t = row % G;
    const int slot = q_tile0 + qslot;
    const bool qvalid = slot < a.num_queries;
    const int qi = qvalid ? slot : 0;
    const int qpos = qvalid ? a.q_positions[qi] : -1;
    const uint32_t lane_addr = (uint32_t)((warp & 3) * 32) << 16;
    const int64_t hidx = (int64_t)qi * a.num_q_heads + h * G + t;
    float m_ref = -INFINITY, l_part = 0.f;
    unsigned long long att = 0;
    bool ok = true;
    int j = 0, s = 0;
    uint32_t kv_par = 0;
    attn::stage_q_half<D, C::Q_COL>(qvalid ? a.q + hidx * D + hf * (D / 2) : nullptr, hf, lane_addr, tmem_base,
                                    bar(B_QFULL));
    for (;; ++j) {
      const int b = j & 1;
      ok = mbar_wait_warp(bar(B_KVFULL + s), kv_par, abort_flag, a.status, STATUS_TIMEOUT_SOFTMAX);
      if (!ok) break;
      const int np = info[s].npages;
      const int rows = info[s].rows, kpos0 = info[s].kpos0;
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(B_KVEMPTY + s));
      if (np == 0) break;                              // end of the stream
      ok = mbar_wait_warp(bar(B_SFULL + b), (uint32_t)((j >> 1) & 1), abort_flag, a.status, STATUS_TIMEOUT_SOFTMAX);
      if (!ok) break;
      tc_fence_after();
      // keys at or before the row's position; a tile wholly below the diagonal for every row of
      // the warp needs no mask
      const int lim = min(rows, qpos - kpos0 + 1);
      if (t == 0 && hf == 0) att += max(lim, 0);
      ok = attn::softmax_tile<D, C::O_COL>(np, lim, j, hf, row, lane_addr, tmem_base, b * BLOCK_N,
                                           reinterpret_cast<float*>(smem + C::MX_OFF), bar(B_PAIR + (warp & 3)),
                                           bar(B_PVDONE + ((j - 1) & 1)), (uint32_t)(((j - 1) >> 1) & 1),
                                           bar(B_PFULL + b), a.scale_log2, m_ref, l_part, abort_flag, a.status);
      if (!ok) break;
      if (++s == STAGES) { s = 0; kv_par ^= 1; }
    }
    if (ok) ok = mbar_wait(bar(B_OREADY), 0, abort_flag, a.status, STATUS_TIMEOUT_EPILOGUE);
    tc_fence_after();
    attn::epilogue_half<D, C::O_COL>(ok && j > 0, hf, row, lane_addr, tmem_base,
                                     reinterpret_cast<float*>(smem + C::EPI_OFF), bar(B_EPI), m_ref, l_part,
                                     ok && qvalid, 0, a.out + hidx * D, nullptr,
                                     a.partial ? a.partial + hidx * D : nullptr, a.lse ? a.lse + hidx : nullptr,
                                     abort_flag, a.status);
    if (ok && a.attended) {
      if (!qvalid) att = 0;
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) att += __shfl_xor_sync(0xffffffffu, att, o);
      if (lane == 0 && att) atomicAdd(a.attended, att);
    }
    tc_fence_before();
  }
  __syncthreads();
  if (*abort_flag) __nanosleep(50000);
  if (warp == 0) tmem_dealloc(tmem_base, C::TMEM_COLS);
}

template <int D, int G>
int launch_prefill(const void* ordered_k, const void* ordered_v, int64_t ordered_rows,
                   const PrefillArgs& a, cudaStream_t st) {
  using C = AttnCfg<D>;
  constexpr int QT = 128 / G;
  CUtensorMap mok, mov;
  const uint64_t row_bytes = (uint64_t)a.num_kv_heads * D * 2;
  uint32_t box[2] = {64, BLOCK_N};
  uint64_t d[2] = {(uint64_t)a.num_kv_heads * D, (uint64_t)ordered_rows};
  int rc = semblo::make_tensor_map_bf16(&mok, ordered_k, 2, d, &row_bytes, box);
  if (rc) return rc;
  rc = semblo::make_tensor_map_bf16(&mov, ordered_v, 2, d, &row_bytes, box);
  if (rc) return rc;
  auto kern = window_prefill_kernel<D, G>;
  SEMBLO_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::TOTAL));
  dim3 grid((unsigned)ceil_div(a.num_queries, QT), a.num_kv_heads);
  kern<<<grid, 320, C::TOTAL, st>>>(mok, mov, a);
  SEMBLO_LAUNCH_CHECK();
  return 0;
}

}  // namespace

extern "C" int semblo_window_prefill(const void* q, int num_queries, int num_q_heads, int num_kv_heads,
                                     int head_dim, const int32_t* q_positions, const void* ordered_k,
                                     const void* ordered_v, int64_t ordered_rows, int ordered_pos0,
                                     int local_start, float sm_scale, void* out, float* partial_out,
                                     float* lse, unsigned long long* attended, int32_t* status,
                                     void* stream) {
  SEMBLO_REQUIRE(num_kv_heads > 0 && num_q_heads % num_kv_heads == 0, "query heads must be a multiple of the KV heads");
  SEMBLO_REQUIRE(status != nullptr, "status word is required");
  SEMBLO_REQUIRE(ordered_k != nullptr && ordered_v != nullptr && q_positions != nullptr, "K, V and positions are required");
  SEMBLO_REQUIRE(local_start >= ordered_pos0, "the window starts before the first row of K/V");
  SEMBLO_REQUIRE(q != nullptr && (reinterpret_cast<uintptr_t>(q) & 15) == 0, "q must be 16-byte aligned");
  if (num_queries == 0) return 0;
  PrefillArgs a;
  a.num_queries = num_queries;
  a.num_q_heads = num_q_heads;
  a.num_kv_heads = num_kv_heads;
  a.num_clusters = 0;
  a.q = (const __nv_bfloat16*)q;
  a.q_positions = q_positions;
  a.local_start = local_start;
  a.local_pos0 = ordered_pos0;
  a.local_rows = (int)ordered_rows;
  a.scale_log2 = sm_scale * 1.4426950408889634f;
  a.out = (__nv_bfloat16*)out;
  a.lse = lse;
  a.partial = partial_out;
  a.attended = attended;
  a.status = status;
  const int g = num_q_heads / num_kv_heads;
  cudaStream_t st = (cudaStream_t)stream;
#define SEMBLO_PREFILL_CASE(DD, GG) \
  if (head_dim == DD && g == GG) return launch_prefill<DD, GG>(ordered_k, ordered_v, ordered_rows, a, st);
  SEMBLO_PREFILL_CASE(256, 4)
  SEMBLO_PREFILL_CASE(128, 4)
  SEMBLO_PREFILL_CASE(256, 8)
  SEMBLO_PREFILL_CASE(128, 8)
  SEMBLO_PREFILL_CASE(256, 16)
  SEMBLO_PREFILL_CASE(128, 16)
#undef SEMBLO_PREFILL_CASE
  return semblo::fail(semblo::SEMBLO_EINVAL,
                      "prefill attention supports head_dim 128/256 with 4, 8 or 16 query heads per "
                      "KV head (got head_dim %d, group %d)", head_dim, g);
}
