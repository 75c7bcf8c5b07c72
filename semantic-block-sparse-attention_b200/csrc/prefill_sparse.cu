// Block-sparse prefill attention, sparse part: row-granular gather of the selected
// clusters' visible rows, tcgen05 / TMEM attention, LSE merge with the window partial.
//
// One CTA owns QT = 128 / G queries of one KV head, taken in the caller's tile order
// (queries with similar selections are placed in the same tile).  Warp roles:
//   warps 0-3  softmax + epilogue, one thread per row (TMEM lane)
//   warp  4    planner: walks the tile's cluster bitmasks 32 clusters at a time (sizes and
//              starts fetched by 32 lanes in parallel), and expands the union of selected
//              clusters into a stream of packed rows, each tagged with the 32-bit set of
//              queries that selected its cluster; 64 rows make a tile
//   warps 5-8  gather: K rows of even / odd tiles, V rows of even / odd tiles; 16-byte
//              cp.async into the 128-byte-swizzled UMMA layout (only visible rows are
//              read: no page padding), then published to the async proxy
//   warp  9    UMMA issuer: S = Q K^T and O += P V, accumulators in TMEM, issued in
//              whichever order their operands become ready
// The epilogue merges the sparse partial with the window partial already stored in
// `out` / `lse` by the dense launch, so each query sees one softmax over the union.
//
// Reference behaviour restated here:
//   semblo/vllm_plugin/kv_outer.py:482-816   attended set, per-query selection, LSE merge order
#include <algorithm>
#include <climits>

#include "../../include/semblo_b200.h"
#include "host_common.h"
#include "sm100.cuh"

using namespace sm100;
using semblo::ceil_div;

namespace {

constexpr int BLOCK_N = 64;
constexpr int PLAN_STAGES = 3;
constexpr float LN2F = 0.6931471805599453f;
constexpr float LOG2EF = 1.4426950408889634f;
constexpr float RESCALE_GAP = 8.0f;

struct Plan {
  int count;             // rows in the tile (0 = end of stream)
  int pad[3];
  int row[BLOCK_N];      // physical packed row, -1 = zero fill
  uint32_t mask[BLOCK_N];
};

template <int D>
struct GatherCfg {
  static constexpr int STAGES = D >= 256 ? 2 : 4;
  static constexpr int SLABS = D / 64;
  static constexpr int Q_BYTES = 128 * D * 2;
  static constexpr int KV_BYTES = BLOCK_N * D * 2;
  static constexpr int P_BYTES = 128 * BLOCK_N * 2;
  static constexpr int Q_OFF = 0;
  static constexpr int K_OFF = Q_OFF + Q_BYTES;
  static constexpr int V_OFF = K_OFF + STAGES * KV_BYTES;
  static constexpr int P_OFF = V_OFF + STAGES * KV_BYTES;
  static constexpr int PLAN_OFF = P_OFF + 2 * P_BYTES;
  static constexpr int BAR_OFF = PLAN_OFF + PLAN_STAGES * (int)sizeof(Plan);
  static constexpr int MISC_OFF = BAR_OFF + 8 * (10 + 4 * STAGES + 2 * PLAN_STAGES);
  static constexpr int TOTAL = MISC_OFF + 16 + 1024;
  static constexpr int TMEM_COLS = D >= 256 ? 512 : 256;
  static constexpr int O_COL = 2 * BLOCK_N;
};

struct GatherArgs {
  int num_queries, num_q_heads, num_kv_heads, num_clusters;
  const int32_t* q_order;       // [Hkv, Q] tile order, or null
  const int32_t* qmask;         // [Q, Hkv, C/32]
  const int32_t* causal_sizes;  // [Hkv, C]
  const int32_t* indptr;        // [Hkv, C+1]
  const int32_t* page_table;    // or null
  const __nv_bfloat16* packed_k;
  const __nv_bfloat16* packed_v;
  float scale_log2;
  __nv_bfloat16* out;           // [Q, Hq, D] in: window partial, out: merged
  float* lse;                   // [Q, Hq]    in: window lse,     out: merged (natural log)
  int merge;                    // 0: no window partial, write the sparse result alone
  unsigned long long* attended;
  int* status;
};

enum { B_QFULL = 0, B_OREADY = 1, B_SFULL = 2, B_SEMPTY = 4, B_PFULL = 6, B_PEMPTY = 8, B_KFULL = 10 };

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src, uint32_t bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void cp_async_wait_all() {
  asm volatile("cp.async.commit_group;\n\tcp.async.wait_group 0;" ::: "memory");
}

template <int D, int G>
__global__ void __launch_bounds__(320, 1)
sparse_gather_prefill_kernel(const __grid_constant__ CUtensorMap tmap_q, const GatherArgs a) {
  using C = GatherCfg<D>;
  constexpr int QT = 128 / G;
  constexpr int STAGES = C::STAGES;
  constexpr int B_KEMPTY = B_KFULL + STAGES;
  constexpr int B_VFULL = B_KEMPTY + STAGES;
  constexpr int B_VEMPTY = B_VFULL + STAGES;
  constexpr int B_PLANFULL = B_VEMPTY + STAGES;
  constexpr int B_PLANEMPTY = B_PLANFULL + PLAN_STAGES;
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + C::BAR_OFF);
  Plan* plan = reinterpret_cast<Plan*>(smem + C::PLAN_OFF);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + C::MISC_OFF);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  auto bar = [&](int i) { return smem_u32(&bars[i]); };

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int h = blockIdx.y;
  const int q_tile0 = blockIdx.x * QT;

  if (threadIdx.x == 0) {
    mbar_init(bar(B_QFULL), 1);
    mbar_init(bar(B_OREADY), 1);
    for (int b = 0; b < 2; ++b) {
      mbar_init(bar(B_SFULL + b), 1);
      mbar_init(bar(B_SEMPTY + b), 128);
      mbar_init(bar(B_PFULL + b), 128);
      mbar_init(bar(B_PEMPTY + b), 1);
    }
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(bar(B_KFULL + s), 1);
      mbar_init(bar(B_KEMPTY + s), 1);
      mbar_init(bar(B_VFULL + s), 1);
      mbar_init(bar(B_VEMPTY + s), 1);
    }
    for (int s = 0; s < PLAN_STAGES; ++s) {
      mbar_init(bar(B_PLANFULL + s), 1);
      mbar_init(bar(B_PLANEMPTY + s), 7);     // a K and a V gather warp, the UMMA thread, four softmax warps
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

  if (warp == 4) {
    // ------------------------------------------------------------ planner (+ Q load)
    const int slot = q_tile0 + lane;
    const bool qvalid = lane < QT && slot < a.num_queries;
    const int qi = qvalid ? (a.q_order ? a.q_order[(int64_t)h * a.num_queries + slot] : slot) : 0;
    const unsigned vmask = __ballot_sync(0xffffffffu, qvalid);
    if (lane == 0) {
      tma_prefetch_desc(&tmap_q);
      mbar_arrive_expect_tx(bar(B_QFULL), (uint32_t)__popc(vmask) * G * D * 2);
    }
    for (int i = 0; i < QT; ++i) {
      const int qsrc = __shfl_sync(0xffffffffu, qi, i);
      if (lane == 0 && ((vmask >> i) & 1))
        for (int sl = 0; sl < C::SLABS; ++sl)
          tma_load_3d(smem_u32(smem + C::Q_OFF + sl * 128 * 128 + i * G * 128), &tmap_q, bar(B_QFULL),
                      sl * 64, h * G, qsrc);
    }
    const int nwords = a.num_clusters >> 5;
    const int32_t* qm = a.qmask + ((int64_t)qi * a.num_kv_heads + h) * nwords;
    const int32_t* csz = a.causal_sizes + (int64_t)h * a.num_clusters;
    const int32_t* ipt = a.indptr + (int64_t)h * (a.num_clusters + 1);
    int tile = 0, fill = 0;
    long long gathered = 0;
    bool ok = true;
    auto acquire = [&]() {          // make plan stage of `tile` writable
      const int ps = tile % PLAN_STAGES;
      if (lane == 0)
        ok = mbar_wait(bar(B_PLANEMPTY + ps), ((tile / PLAN_STAGES) & 1) ^ 1, abort_flag, a.status, STATUS_TIMEOUT_LOAD);
      ok = __shfl_sync(0xffffffffu, (int)ok, 0) != 0;
    };
    auto publish = [&](int count) {
      const int ps = tile % PLAN_STAGES;
      __syncwarp();
      if (lane == 0) {
        plan[ps].count = count;
        mbar_arrive(bar(B_PLANFULL + ps));
      }
      gathered += count;
      ++tile;
      fill = 0;
    };
    acquire();
    // software pipeline over the bitmask words: word w+2 and the sizes / starts of the clusters
    // of word w+1 are in flight while word w is expanded
    auto load_word = [&](int w) -> unsigned { return (qvalid && w < nwords) ? (unsigned)qm[w] : 0u; };
    unsigned word1 = load_word(0), word2 = load_word(1);
    unsigned any1 = __reduce_or_sync(0xffffffffu, word1);
    int n1 = ((any1 >> lane) & 1) ? csz[lane] : 0;
    int start1 = ((any1 >> lane) & 1) ? ipt[lane] : 0;
    int pt1 = (a.page_table && ((any1 >> lane) & 1)) ? a.page_table[start1 >> 4] : 0;
    for (int w = 0; w < nwords && ok; ++w) {
      const unsigned word = word1, any = any1;
      int n_b = max(n1, 0);
      const int start_b = start1, pt_b = pt1;
      // prefetch for the following words
      word1 = word2;
      word2 = load_word(w + 2);
      any1 = __reduce_or_sync(0xffffffffu, word1);
      {
        const bool has1 = (w + 1 < nwords) && ((any1 >> lane) & 1);
        const int c1 = (w + 1) * 32 + lane;
        n1 = has1 ? csz[c1] : 0;
        start1 = has1 ? ipt[c1] : 0;
      }
      if (any != 0) {
        // mask_b: the queries of the tile that selected cluster (w, lane)
        unsigned mask_b = 0;
        for (unsigned tmp = any; tmp; tmp &= tmp - 1) {
          const int b = __ffs(tmp) - 1;
          const unsigned m = __ballot_sync(0xffffffffu, (word >> b) & 1u);
          if (lane == b) mask_b = m;
        }
        int pre = n_b;                               // inclusive scan over lanes
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
          const int v = __shfl_up_sync(0xffffffffu, pre, o);
          if (lane >= o) pre += v;
        }
        const int total = __shfl_sync(0xffffffffu, pre, 31);
        const int excl = pre - n_b;
        for (int j0 = 0; j0 < total && ok;) {
          const int cnt = min(min(32, total - j0), BLOCK_N - fill);
          const int j = j0 + lane;
          // first lane whose inclusive prefix exceeds j
          int lo = 0;
#pragma unroll
          for (int step = 16; step > 0; step >>= 1) {
            const int v = __shfl_sync(0xffffffffu, pre, lo + step - 1);
            if (v <= j) lo += step;
          }
          lo = min(lo, 31);
          const int sb = __shfl_sync(0xffffffffu, start_b, lo);
          const int eb = __shfl_sync(0xffffffffu, excl, lo);
          const int pb = __shfl_sync(0xffffffffu, pt_b, lo);
          const unsigned mb = __shfl_sync(0xffffffffu, mask_b, lo);
          if (lane < cnt) {
            const int off = j - eb;
            int row = sb + off;
            if (a.page_table) row = (off < 16 ? pb : a.page_table[row >> 4]) * 16 + (row & 15);
            const int ps = tile % PLAN_STAGES;
            plan[ps].row[fill + lane] = row;
            plan[ps].mask[fill + lane] = mb;
          }
          fill += cnt;
          j0 += cnt;
          if (fill == BLOCK_N) {
            publish(BLOCK_N);
            acquire();
          }
        }
      }
      // the first page of every cluster of the next word (its start has arrived by now)
      pt1 = (a.page_table && ((any1 >> lane) & 1) && w + 1 < nwords) ? a.page_table[start1 >> 4] : 0;
    }
    if (ok && fill > 0) {
      const int ps = tile % PLAN_STAGES;
      const int padded = (fill + 15) & ~15;
      for (int i = fill + lane; i < padded; i += 32) {
        plan[ps].row[i] = -1;
        plan[ps].mask[i] = 0u;
      }
      publish(fill);
      acquire();
    }
    if (a.attended && lane == 0 && gathered) atomicAdd(a.attended + 1, (unsigned long long)gathered);
    if (ok) {
      // end of stream, once per gather warp (they alternate tiles)
      publish(0);
      acquire();
      if (ok) publish(0);
    }
  } else if (warp >= 5 && warp <= 8) {
    // ------------------------------------------------------------ gather warps
    // warps 5/6 copy the K rows of even/odd tiles, warps 7/8 the V rows: consecutive tiles
    // are in flight in different warps, so a tile's latency hides behind its neighbours'.
    const bool is_v = warp >= 7;
    const int par = (warp - 5) & 1;
    const __nv_bfloat16* src_base = is_v ? a.packed_v : a.packed_k;
    const int b_full = is_v ? B_VFULL : B_KFULL, b_empty = is_v ? B_VEMPTY : B_KEMPTY;
    const int64_t row_elems = (int64_t)a.num_kv_heads * D;
    constexpr int LANES_PER_ROW = D / 8;           // 16-byte chunks per row: 32 (D=256) or 16 (D=128)
    constexpr int ROWS_PER_ITER = 32 / LANES_PER_ROW;
    const int sub = lane / LANES_PER_ROW, l_in = lane % LANES_PER_ROW;
    const int slab = l_in >> 3, chunk = l_in & 7;
    const int64_t lane_off = (int64_t)h * D + l_in * 8;
    for (int t = par;; t += 2) {
      const int ps = t % PLAN_STAGES, s = t % STAGES;
      if (!mbar_wait(bar(B_PLANFULL + ps), (t / PLAN_STAGES) & 1, abort_flag, a.status, STATUS_TIMEOUT_LOAD)) break;
      const int cnt = plan[ps].count;
      if (cnt == 0) break;
      const int r_lo = plan[ps].row[lane], r_hi = plan[ps].row[lane + 32];
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(B_PLANEMPTY + ps));
      if (!mbar_wait(bar(b_empty + s), ((t / STAGES) & 1) ^ 1, abort_flag, a.status, STATUS_TIMEOUT_LOAD)) break;
      const int n16 = (cnt + 15) & ~15;
      const uint32_t base = smem_u32(smem + (is_v ? C::V_OFF : C::K_OFF) + s * C::KV_BYTES) + slab * (BLOCK_N * 128);
#pragma unroll 4
      for (int j0 = 0; j0 < n16; j0 += ROWS_PER_ITER) {
        const int j = j0 + sub;
        const int row = __shfl_sync(0xffffffffu, j0 < 32 ? r_lo : r_hi, j & 31);
        const int64_t off = (int64_t)max(row, 0) * row_elems + lane_off;
        cp_async16(base + swz128(j, chunk), src_base + off, row >= 0 ? 16u : 0u);
      }
      cp_async_wait_all();
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(b_full + s));
    }
  } else if (warp == 9) {
    // ------------------------------------------------------------ UMMA issuer
    // S(j) = Q K(j)^T is issued as soon as K(j) has landed and the S buffer is free;
    // O += P(j) V(j) as soon as the softmax warps have written P(j): whichever is ready first.
    if (elect_one()) {
      const uint32_t q_base = smem_u32(smem + C::Q_OFF);
      constexpr uint32_t idesc_pv = make_idesc_bf16(128, D, false, true);
      bool ok = mbar_wait(bar(B_QFULL), 0, abort_flag, a.status, STATUS_TIMEOUT_MMA);
      int next_qk = 0, next_pv = 0, end_tile = INT_MAX, plan_seen = -1, cnt_cur = 0;
      int np_of[4] = {0, 0, 0, 0};                    // pages of the tiles in flight (index tile & 3)
      unsigned long long t0 = globaltimer();
      uint32_t idle = 0;
      while (ok) {
        bool progress = false;
        if (next_qk < end_tile && next_qk - next_pv < 2) {
          const int j = next_qk, ps = j % PLAN_STAGES, s = j % STAGES, b = j & 1;
          if (plan_seen < j && mbar_try_wait(bar(B_PLANFULL + ps), (j / PLAN_STAGES) & 1)) {
            cnt_cur = plan[ps].count;
            mbar_arrive(bar(B_PLANEMPTY + ps));
            plan_seen = j;
            if (cnt_cur == 0) end_tile = j;
            progress = true;
          }
          if (plan_seen == j && cnt_cur > 0 && mbar_try_wait(bar(B_KFULL + s), (j / STAGES) & 1) &&
              mbar_try_wait(bar(B_SEMPTY + b), ((j >> 1) & 1) ^ 1)) {
            tc_fence_after();
            const int np = (cnt_cur + 15) >> 4;
            np_of[j & 3] = np;
            const uint32_t k_base = smem_u32(smem + C::K_OFF + s * C::KV_BYTES);
            const uint32_t idesc_qk = make_idesc_bf16(128, np * 16, false, false);
#pragma unroll
            for (int kk = 0; kk < D / 16; ++kk) {
              const uint32_t sl = kk >> 2, ko = (kk & 3) * 32;
              umma_ss(tmem_base + b * BLOCK_N, make_smem_desc(q_base + sl * 128 * 128 + ko, 16, 1024),
                      make_smem_desc(k_base + sl * BLOCK_N * 128 + ko, 16, 1024), idesc_qk, kk > 0 ? 1u : 0u);
            }
            umma_commit(bar(B_KEMPTY + s));
            umma_commit(bar(B_SFULL + b));
            ++next_qk;
            progress = true;
          }
        }
        if (next_pv < next_qk) {
          const int t = next_pv, b = t & 1, s = t % STAGES;
          if (mbar_try_wait(bar(B_PFULL + b), (t >> 1) & 1) && mbar_try_wait(bar(B_VFULL + s), (t / STAGES) & 1)) {
            tc_fence_after();
            const int np = np_of[t & 3];
            const uint32_t p_base = smem_u32(smem + C::P_OFF + b * C::P_BYTES);
            const uint32_t v_base = smem_u32(smem + C::V_OFF + s * C::KV_BYTES);
            for (int kk = 0; kk < np; ++kk)
              umma_ss(tmem_base + C::O_COL, make_smem_desc(p_base + kk * 32, 16, 1024),
                      make_smem_desc(v_base + kk * 16 * 128, BLOCK_N * 128, 1024), idesc_pv,
                      (t > 0 || kk > 0) ? 1u : 0u);
            umma_commit(bar(B_VEMPTY + s));
            umma_commit(bar(B_PEMPTY + b));
            ++next_pv;
            progress = true;
          }
        }
        if (next_pv == end_tile) break;
        if (progress) {
          idle = 0;
        } else if ((++idle & 0x3ff) == 0) {
          if (idle == 0x400) t0 = globaltimer();
          if (*abort_flag || *reinterpret_cast<volatile int*>(a.status) != 0) { *abort_flag = 1; ok = false; }
          else if (globaltimer() - t0 > WAIT_LIMIT_NS) { *abort_flag = 1; atomicCAS(a.status, 0, STATUS_TIMEOUT_MMA); ok = false; }
        }
      }
      if (ok) umma_commit(bar(B_OREADY));
    }
  } else {
    // ------------------------------------------------------------ softmax + epilogue (thread = row)
    const int row = threadIdx.x;
    const int qslot = row / G, t = row % G;
    const int slot = q_tile0 + qslot;
    const bool qvalid = slot < a.num_queries;
    const int qi = qvalid ? (a.q_order ? a.q_order[(int64_t)h * a.num_queries + slot] : slot) : 0;
    const uint32_t lane_addr = (uint32_t)(warp * 32) << 16;
    float m_ref = -INFINITY, l_run = 0.f;
    unsigned long long att = 0;
    bool ok = true;
    int j = 0;
    for (;; ++j) {
      const int ps = j % PLAN_STAGES, b = j & 1;
      ok = mbar_wait(bar(B_PLANFULL + ps), (j / PLAN_STAGES) & 1, abort_flag, a.status, STATUS_TIMEOUT_SOFTMAX);
      if (!ok) break;
      const int cnt = plan[ps].count;
      if (cnt == 0) {
        __syncwarp();
        if (lane == 0) mbar_arrive(bar(B_PLANEMPTY + ps));
        break;
      }
      const int np = (cnt + 15) >> 4;
      ok = mbar_wait(bar(B_SFULL + b), (j >> 1) & 1, abort_flag, a.status, STATUS_TIMEOUT_SOFTMAX);
      if (!ok) break;
      tc_fence_after();
      uint32_t r0[32], r1[32];
      tmem_ld32(tmem_base + lane_addr + b * BLOCK_N, r0);
      if (np > 2) tmem_ld32(tmem_base + lane_addr + b * BLOCK_N + 32, r1);
      tmem_ld_wait();
      tc_fence_before();
      mbar_arrive(bar(B_SEMPTY + b));
      // masked raw logits (scaling is folded into the exponent below)
      float tmax = -INFINITY;
      int n_on = 0;
      const uint32_t qbit = 1u << qslot;
      const uint4* mk = reinterpret_cast<const uint4*>(plan[ps].mask);
#pragma unroll
      for (int g4 = 0; g4 < BLOCK_N / 4; ++g4) {
        if (g4 * 4 < np * 16) {
          const uint4 m4 = mk[g4];
          const uint32_t mm[4] = {m4.x, m4.y, m4.z, m4.w};
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const int col = g4 * 4 + e;
            uint32_t& slot_r = col < 32 ? r0[col] : r1[col - 32];
            const bool allowed = (mm[e] & qbit) != 0u;
            const float sraw = allowed ? __uint_as_float(slot_r) : -INFINITY;
            slot_r = __float_as_uint(sraw);
            tmax = fmaxf(tmax, sraw);
            n_on += allowed;
          }
        }
      }
      tmax *= a.scale_log2;                      // scale > 0: the max commutes with it
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(B_PLANEMPTY + ps));
      if (t == 0) att += n_on;
      bool need = j > 0 && m_ref != -INFINITY && tmax > m_ref + RESCALE_GAP;
      float alpha = 1.f;
      if (need) {
        alpha = exp2f(m_ref - tmax);
        m_ref = tmax;
        l_run *= alpha;
      } else if (m_ref == -INFINITY) {
        m_ref = tmax;
      }
      ok = mbar_wait(bar(B_PEMPTY + b), ((j >> 1) & 1) ^ 1, abort_flag, a.status, STATUS_TIMEOUT_SOFTMAX);
      if (!ok) break;
      if (__any_sync(0xffffffffu, need)) {
        ok = mbar_wait(bar(B_PEMPTY + ((j - 1) & 1)), ((j - 1) >> 1) & 1, abort_flag, a.status, STATUS_TIMEOUT_SOFTMAX);
        if (!ok) break;
        tc_fence_after();
#pragma unroll 1
        for (int c = 0; c < D / 32; ++c) {
          uint32_t o[32];
          tmem_ld32(tmem_base + lane_addr + C::O_COL + c * 32, o);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
          tmem_st32(tmem_base + lane_addr + C::O_COL + c * 32, o);
        }
        tmem_st_wait();
        tc_fence_before();
      }
      const float m_use = m_ref == -INFINITY ? 0.f : m_ref;
      const float neg_m = -m_use, sc = a.scale_log2;
      uint8_t* p_row = smem + C::P_OFF + b * C::P_BYTES;
      float add = 0.f;
#pragma unroll
      for (int p = 0; p < 4; ++p) {
        if (p < np) {
          uint32_t packed[8];
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const uint32_t u0 = p < 2 ? r0[p * 16 + 2 * i] : r1[(p - 2) * 16 + 2 * i];
            const uint32_t u1 = p < 2 ? r0[p * 16 + 2 * i + 1] : r1[(p - 2) * 16 + 2 * i + 1];
            const float e0 = fast_exp2(fmaf(__uint_as_float(u0), sc, neg_m));
            const float e1 = fast_exp2(fmaf(__uint_as_float(u1), sc, neg_m));
            add += e0 + e1;
            __nv_bfloat162 pr = __floats2bfloat162_rn(e0, e1);
            packed[i] = *reinterpret_cast<uint32_t*>(&pr);
          }
          *reinterpret_cast<uint4*>(p_row + swz128(row, 2 * p)) = make_uint4(packed[0], packed[1], packed[2], packed[3]);
          *reinterpret_cast<uint4*>(p_row + swz128(row, 2 * p + 1)) = make_uint4(packed[4], packed[5], packed[6], packed[7]);
        }
      }
      l_run += add;
      fence_proxy_async_smem();
      mbar_arrive(bar(B_PFULL + b));
    }
    if (ok) ok = mbar_wait(bar(B_OREADY), 0, abort_flag, a.status, STATUS_TIMEOUT_EPILOGUE);
    if (ok) {
      tc_fence_after();
      // merge with the window partial (out holds its normalised output, lse its natural-log LSE)
      const int64_t hidx = (int64_t)qi * a.num_q_heads + h * G + t;
      float wa = 0.f, wb = 1.f, denom = l_run, m_new = m_ref;
      if (a.merge && qvalid) {
        const float l2 = a.lse[hidx] * LOG2EF;                 // window LSE in log2 units
        m_new = fmaxf(l2, m_ref);
        if (m_new == -INFINITY) {
          wa = 0.f; wb = 0.f; denom = 0.f;
        } else {
          wa = exp2f(l2 - m_new);
          wb = m_ref == -INFINITY ? 0.f : exp2f(m_ref - m_new);
          denom = wa + l_run * wb;
        }
      }
      const float inv = denom > 0.f ? 1.f / denom : 0.f;
      __nv_bfloat16* dst = a.out + hidx * D;
#pragma unroll 1
      for (int c = 0; c < D / 32; ++c) {
        uint32_t o[32];
        if (j > 0) {
          tmem_ld32(tmem_base + lane_addr + C::O_COL + c * 32, o);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) o[i] = 0u;
        }
        if (qvalid) {
          uint4* d4 = reinterpret_cast<uint4*>(dst + c * 32);
          uint32_t prev[16];
          if (a.merge) {
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              const uint4 v = d4[i];
              prev[4 * i] = v.x; prev[4 * i + 1] = v.y; prev[4 * i + 2] = v.z; prev[4 * i + 3] = v.w;
            }
          }
          uint32_t w[16];
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            float x0 = __uint_as_float(o[2 * i]) * wb, x1 = __uint_as_float(o[2 * i + 1]) * wb;
            if (a.merge) {
              const float2 pv = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&prev[i]));
              x0 += pv.x * wa;
              x1 += pv.y * wa;
            }
            __nv_bfloat162 pr = __floats2bfloat162_rn(x0 * inv, x1 * inv);
            w[i] = *reinterpret_cast<uint32_t*>(&pr);
          }
          d4[0] = make_uint4(w[0], w[1], w[2], w[3]);
          d4[1] = make_uint4(w[4], w[5], w[6], w[7]);
          d4[2] = make_uint4(w[8], w[9], w[10], w[11]);
          d4[3] = make_uint4(w[12], w[13], w[14], w[15]);
        }
      }
      if (qvalid && a.lse) a.lse[hidx] = denom > 0.f ? (m_new + log2f(denom)) * LN2F : -INFINITY;
      if (a.attended) {
        if (!qvalid) att = 0;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) att += __shfl_xor_sync(0xffffffffu, att, o);
        if (lane == 0 && att) atomicAdd(a.attended, att);
      }
    }
    tc_fence_before();
  }
  __syncthreads();
  if (*abort_flag) __nanosleep(50000);
  if (warp == 0) tmem_dealloc(tmem_base, C::TMEM_COLS);
}

template <int D, int G>
int launch_gather(const void* q, const GatherArgs& a, cudaStream_t st) {
  using C = GatherCfg<D>;
  constexpr int QT = 128 / G;
  CUtensorMap mq;
  uint64_t d[3] = {(uint64_t)D, (uint64_t)a.num_q_heads, (uint64_t)a.num_queries};
  uint64_t s[2] = {(uint64_t)D * 2, (uint64_t)a.num_q_heads * D * 2};
  uint32_t b[3] = {64, (uint32_t)G, 1};
  int rc = semblo::make_tensor_map_bf16(&mq, q, 3, d, s, b);
  if (rc) return rc;
  auto kern = sparse_gather_prefill_kernel<D, G>;
  SEMBLO_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::TOTAL));
  dim3 grid((unsigned)ceil_div(a.num_queries, QT), a.num_kv_heads);
  kern<<<grid, 320, C::TOTAL, st>>>(mq, a);
  SEMBLO_LAUNCH_CHECK();
  return 0;
}

}  // namespace

extern "C" int semblo_sparse_prefill_gather(
    const void* q, int num_queries, int num_q_heads, int num_kv_heads, int head_dim,
    const int32_t* q_order, const void* packed_k, const void* packed_v, const int32_t* page_table,
    const int32_t* qmask, const int32_t* causal_sizes, const int32_t* indptr, int num_clusters,
    float sm_scale, int merge, void* out, float* lse, unsigned long long* attended,
    int32_t* status, void* stream) {
  SEMBLO_REQUIRE(num_kv_heads > 0 && num_q_heads % num_kv_heads == 0, "query heads must be a multiple of the KV heads");
  SEMBLO_REQUIRE(status != nullptr, "status word is required");
  SEMBLO_REQUIRE(qmask && packed_k && packed_v && causal_sizes && indptr, "selection, packed K/V, sizes and indptr are required");
  SEMBLO_REQUIRE(num_clusters % 32 == 0, "cluster count %d must be a multiple of 32", num_clusters);
  SEMBLO_REQUIRE(!merge || lse != nullptr, "merging needs the window's log-sum-exp");
  SEMBLO_REQUIRE((reinterpret_cast<uintptr_t>(packed_k) & 15) == 0 && (reinterpret_cast<uintptr_t>(packed_v) & 15) == 0,
                 "packed K/V must be 16-byte aligned");
  if (num_queries == 0) return 0;
  GatherArgs a;
  a.num_queries = num_queries; a.num_q_heads = num_q_heads; a.num_kv_heads = num_kv_heads;
  a.num_clusters = num_clusters; a.q_order = q_order; a.qmask = qmask; a.causal_sizes = causal_sizes;
  a.indptr = indptr; a.page_table = page_table;
  a.packed_k = (const __nv_bfloat16*)packed_k; a.packed_v = (const __nv_bfloat16*)packed_v;
  a.scale_log2 = sm_scale * LOG2EF; a.out = (__nv_bfloat16*)out; a.lse = lse; a.merge = merge;
  a.attended = attended; a.status = status;
  const int g = num_q_heads / num_kv_heads;
  cudaStream_t st = (cudaStream_t)stream;
#define SEMBLO_GATHER_CASE(DD, GG) \
  if (head_dim == DD && g == GG) return launch_gather<DD, GG>(q, a, st);
  SEMBLO_GATHER_CASE(256, 4)
  SEMBLO_GATHER_CASE(128, 4)
  SEMBLO_GATHER_CASE(256, 8)
  SEMBLO_GATHER_CASE(128, 8)
  SEMBLO_GATHER_CASE(256, 16)
  SEMBLO_GATHER_CASE(128, 16)
#undef SEMBLO_GATHER_CASE
  return semblo::fail(semblo::SEMBLO_EINVAL,
                      "sparse prefill supports head_dim 128/256 with 4, 8 or 16 query heads per KV head "
                      "(got head_dim %d, group %d)", head_dim, g);
}
