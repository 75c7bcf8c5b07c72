// Block-sparse prefill attention, sparse part: row-granular gather of the selected
// clusters' visible rows, tcgen05 / TMEM attention, LSE merge with the window partial.
//
// One CTA owns QT = 128 / G queries of one KV head, taken in the caller's tile order
// (queries with similar selections are placed in the same tile).  Warp roles:
//   warps 0-7  mask stage of the softmax (two threads per row, 32 columns each): keep the
//              logits of the keys whose cluster the row's query selected, take the maximum
//   warps 8-15 exp stage of the softmax (two threads per row): running maximum and sum, P as
//              bf16 into TMEM; they also write the output in the epilogue
//   warp  16   planner: walks the tile's cluster bitmasks 32 clusters at a time (sizes and
//              starts fetched by 32 lanes in parallel), and expands the union of selected
//              clusters into a stream of packed rows, each tagged with the 32-bit set of
//              queries that selected its cluster; 64 rows make a tile
//   warps 17-20 gather: K rows of even / odd tiles, V rows of even / odd tiles; 16-byte
//              cp.async into the 128-byte-swizzled UMMA layout (only visible rows are
//              read: no page padding), then published to the async proxy
//   warp  21   UMMA issuer: S = Q K^T and O += P V, accumulators in TMEM, issued in
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
#include "attn_common.cuh"
#include "sm100.cuh"

using namespace sm100;
using semblo::ceil_div;

namespace {

constexpr int BLOCK_N = 64;
constexpr uint32_t POLL_NS = 50;      // how long the UMMA thread sleeps on one barrier before it looks at the other
constexpr int PLAN_STAGES = 8;
constexpr float LOG2EF = 1.4426950408889634f;

// The plan ring: stream position p lives at entry p % (PLAN_STAGES * BLOCK_N); tile T is slot
// T % PLAN_STAGES, i.e. entries [64 slot, 64 slot + 64).
struct Plan {
  int row[PLAN_STAGES * BLOCK_N];        // logical packed row (before the page table); padding rows have mask 0
  uint32_t mask[PLAN_STAGES * BLOCK_N];  // the queries of the tile that attend to the row
  int count[PLAN_STAGES];                // rows in the tile (0 = end of stream)
};
static_assert((PLAN_STAGES & (PLAN_STAGES - 1)) == 0, "the ring index is a mask");

template <int D>
struct GatherCfg {
  static constexpr int STAGES = D >= 256 ? 3 : 6;
  static constexpr int SLABS = D / 64;
  static constexpr int KV_BYTES = BLOCK_N * D * 2;
  static constexpr int K_OFF = 0;
  static constexpr int V_OFF = K_OFF + STAGES * KV_BYTES;
  static constexpr int EPI_OFF = V_OFF + STAGES * KV_BYTES;     // float [2][128]
  static constexpr int PLAN_OFF = EPI_OFF + 2048;
  static constexpr int NOTE_OFF = PLAN_OFF + (int)sizeof(Plan);   // attn::TileNote [2]
  static constexpr int BAR_OFF = NOTE_OFF + 2 * (int)sizeof(attn::TileNote);
  static constexpr int MISC_OFF = BAR_OFF + 8 * (11 + 4 * STAGES + 2 * PLAN_STAGES);
  static constexpr int TOTAL = MISC_OFF + 16;      // the dynamic segment must start 1024-byte aligned
  static constexpr int TMEM_COLS = 512;
  static constexpr int O_COL = 2 * BLOCK_N;        // S/P buffers, then O, then Q
  static constexpr int Q_COL = O_COL + D;
  static_assert(Q_COL + D / 2 <= TMEM_COLS, "tensor memory budget");
  static_assert(TOTAL <= 232448, "shared memory budget");
};

struct GatherArgs {
  int num_queries, num_q_heads, num_kv_heads, num_clusters;
  const __nv_bfloat16* q;       // [Q, Hq, D]
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
  const float* partial;         // [Q, Hq, D] fp32 window partial, or null: it is in `out` as bf16
  int merge;                    // 0: no window partial, write the sparse result alone
  unsigned long long* attended;
  int* status;
};

// Optional wait accounting (build with -DSEMBLO_TRACE): every role adds the cycles it spends
// in each phase to attended[8 + 8 * role + phase]; the buffer must then hold 48 counters.
#ifdef SEMBLO_TRACE
#define TR_DECL long long tr_last = clock64(); long long tr[8] = {0, 0, 0, 0, 0, 0, 0, 0};
#define TR(i) { const long long tr_now = clock64(); tr[i] += tr_now - tr_last; tr_last = tr_now; }
#define TR_FLUSH(role) if (a.attended && lane == 0) { for (int i_ = 0; i_ < 8; ++i_) if (tr[i_]) atomicAdd(a.attended + 8 + 8 * (role) + i_, (unsigned long long)tr[i_]); }
// timeline of one CTA: event e of tile T at attended[64 + 256 e + T]
#define EV(e, T) if (a.attended && blockIdx.x == 5 && blockIdx.y == 0 && (T) < 256) a.attended[64 + 256 * (e) + (T)] = (unsigned long long)clock64();
#else
#define TR_DECL
#define TR(i)
#define TR_FLUSH(role)
#define EV(e, T)
#endif

enum { B_QFULL = 0, B_OREADY = 1, B_SFULL = 2, B_PFULL = 4, B_PVDONE = 6, B_XFULL = 8, B_EPI = 10, B_KFULL = 11 };

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_wait_all() {
  asm volatile("cp.async.commit_group;\n\tcp.async.wait_group 0;" ::: "memory");
}

template <int D, int G>
__global__ void __launch_bounds__(704, 1)
sparse_gather_prefill_kernel(const GatherArgs a) {
  using C = GatherCfg<D>;
  constexpr int QT = 128 / G;
  constexpr int STAGES = C::STAGES;
  constexpr int B_KEMPTY = B_KFULL + STAGES;
  constexpr int B_VFULL = B_KEMPTY + STAGES;
  constexpr int B_VEMPTY = B_VFULL + STAGES;
  constexpr int B_PLANFULL = B_VEMPTY + STAGES;
  constexpr int B_PLANEMPTY = B_PLANFULL + PLAN_STAGES;
  extern __shared__ __align__(1024) uint8_t smem[];
  if (smem_u32(smem) & 1023u) {                    // the swizzled tiles need 1024-byte alignment
    if (threadIdx.x == 0) atomicCAS(a.status, 0, STATUS_SMEM_ALIGN);
    return;
  }
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + C::BAR_OFF);
  attn::TileNote* note = reinterpret_cast<attn::TileNote*>(smem + C::NOTE_OFF);
  Plan* plan = reinterpret_cast<Plan*>(smem + C::PLAN_OFF);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + C::MISC_OFF);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  auto bar = [&](int i) { return smem_u32(&bars[i]); };

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int h = blockIdx.y;
  const int q_tile0 = blockIdx.x * QT;

  if (threadIdx.x == 0) {
    mbar_init(bar(B_QFULL), 256);
    mbar_init(bar(B_OREADY), 1);
    mbar_init(bar(B_EPI), 256);
    for (int b = 0; b < 2; ++b) {
      mbar_init(bar(B_SFULL + b), 1);
      mbar_init(bar(B_XFULL + b), 256);
      mbar_init(bar(B_PFULL + b), 256);
      mbar_init(bar(B_PVDONE + b), 1);
    }
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(bar(B_KFULL + s), 1);
      mbar_init(bar(B_KEMPTY + s), 1);
      mbar_init(bar(B_VFULL + s), 1);
      mbar_init(bar(B_VEMPTY + s), 1);
    }
    for (int s = 0; s < PLAN_STAGES; ++s) {
      mbar_init(bar(B_PLANFULL + s), 1);
      mbar_init(bar(B_PLANEMPTY + s), 11);    // a K and a V gather warp, the UMMA thread, eight mask warps
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

  if (warp == 16) {
    // ------------------------------------------------------------ planner
    const int slot = q_tile0 + lane;
    const bool qvalid = lane < QT && slot < a.num_queries;
    const int qi = qvalid ? (a.q_order ? a.q_order[(int64_t)h * a.num_queries + slot] : slot) : 0;
    const int nwords = a.num_clusters >> 5;
    const int32_t* qm = a.qmask + ((int64_t)qi * a.num_kv_heads + h) * nwords;
    const int32_t* csz = a.causal_sizes + (int64_t)h * a.num_clusters;
    const int32_t* ipt = a.indptr + (int64_t)h * (a.num_clusters + 1);
    // The selected clusters' visible rows form one stream; 64 consecutive stream positions
    // are a tile, and tile T lives in plan slot T % PLAN_STAGES.
    int pos = 0;                 // stream position of the next row
    int acq = 0, pub = 0;        // tiles made writable / published so far
    long long pairs = 0;
    bool ok = true;
    TR_DECL
    auto acquire_to = [&](int upto) {          // make tiles [acq, upto) writable
      TR(1)
      while (ok && acq < upto) {
        if (lane == 0)
          ok = mbar_wait(bar(B_PLANEMPTY + acq % PLAN_STAGES), ((acq / PLAN_STAGES) & 1) ^ 1, abort_flag, a.status,
                         STATUS_TIMEOUT_LOAD);
        ok = __shfl_sync(0xffffffffu, (int)ok, 0) != 0;
        ++acq;
      }
      TR(0)
    };
    auto publish_to = [&](int upto, int last_count) {   // publish tiles [pub, upto), the last with last_count rows
      __syncwarp();
      if (lane == 0)
        for (int t = pub; t < upto; ++t) {
          plan->count[t % PLAN_STAGES] = t == upto - 1 ? last_count : BLOCK_N;
          mbar_arrive(bar(B_PLANFULL + t % PLAN_STAGES));
          EV(0, t)
        }
      pub = max(pub, upto);
    };
    auto put = [&](int p, int row, unsigned mask) {
      const int e = p & (PLAN_STAGES * BLOCK_N - 1);
      plan->row[e] = row;
      plan->mask[e] = mask;
    };
    // software pipeline over the bitmask words: word w+2 and the sizes / starts of the clusters
    // of word w+1 are in flight while word w is expanded
    auto load_word = [&](int w) -> unsigned { return (qvalid && w < nwords) ? (unsigned)qm[w] : 0u; };
    unsigned word1 = load_word(0), word2 = load_word(1);
    unsigned any1 = __reduce_or_sync(0xffffffffu, word1);
    int n1 = ((any1 >> lane) & 1) ? csz[lane] : 0;
    int start1 = ((any1 >> lane) & 1) ? ipt[lane] : 0;
    constexpr int SELF_MAX = 16;     // longer runs are written by the whole warp
    for (int w = 0; w < nwords && ok; ++w) {
      const unsigned word = word1, any = any1;
      const int n_b = max(n1, 0);
      const int start_b = start1;
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
      if (any == 0) continue;
      TR(1)
      // mask_b: the queries of the tile that selected cluster (w, lane) -- the 32 x 32 bit
      // matrix (query lane, cluster bit) transposed across the warp in five exchange steps
      unsigned mask_b = word;
#pragma unroll
      for (int d = 16; d > 0; d >>= 1) {
        const unsigned m = d == 16 ? 0x0000ffffu : d == 8 ? 0x00ff00ffu : d == 4 ? 0x0f0f0f0fu
                         : d == 2 ? 0x33333333u : 0x55555555u;             // columns whose bit d is clear
        const unsigned y = __shfl_xor_sync(0xffffffffu, mask_b, d);
        mask_b = (lane & d) ? (((y & ~m) >> d) | (mask_b & ~m)) : ((mask_b & m) | ((y & m) << d));
      }
      TR(2)
      pairs += (long long)n_b * __popc(mask_b);      // (query, key) pairs this cluster contributes
      int pre = n_b;                                 // inclusive scan over lanes
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int v = __shfl_up_sync(0xffffffffu, pre, o);
        if (lane >= o) pre += v;
      }
      const int total = __shfl_sync(0xffffffffu, pre, 31);
      if (total == 0) continue;
      // lane b owns stream positions [a_b, e_b): its cluster's rows start_b, start_b + 1, ...
      const int a_b = pos + pre - n_b, e_b = pos + pre, end = pos + total;
      const int row_minus_pos = start_b - a_b;
      int wlo = pos;
      TR(3)
      while (wlo < end && ok) {
        // a wave: as far as the plan ring reaches beyond the oldest unpublished tile
        const int whi = min(end, (pub + PLAN_STAGES) * BLOCK_N);
        acquire_to((whi + BLOCK_N - 1) / BLOCK_N);
        if (!ok) break;
        const int lo = max(a_b, wlo), hi = min(e_b, whi);
        const bool big = hi - lo > SELF_MAX;
        if (!big)
          for (int p = lo; p < hi; ++p) put(p, row_minus_pos + p, mask_b);
        TR(4)
        for (unsigned bigs = __ballot_sync(0xffffffffu, big); bigs; bigs &= bigs - 1) {
          const int bb = __ffs(bigs) - 1;
          const int blo = __shfl_sync(0xffffffffu, lo, bb), bhi = __shfl_sync(0xffffffffu, hi, bb);
          const int brow = __shfl_sync(0xffffffffu, row_minus_pos, bb);
          const unsigned bmask = __shfl_sync(0xffffffffu, mask_b, bb);
          for (int p = blo + lane; p < bhi; p += 32) put(p, brow + p, bmask);
        }
        TR(5)
        publish_to(whi / BLOCK_N, BLOCK_N);
        wlo = whi;
        TR(6)
      }
      pos = end;
    }
    const int fill = pos % BLOCK_N;
    if (ok && fill > 0) {
      // the open tile: the rest of it is a valid row that no query attends to (the copies stop
      // at the next 16-row group, the masks are cleared to the end of the tile)
      for (int i = fill + lane; i < BLOCK_N; i += 32) put(pos - fill + i, 0, 0u);
      publish_to(pub + 1, fill);
    }
    if (a.attended) {
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) pairs += __shfl_xor_sync(0xffffffffu, pairs, o);
      if (lane == 0 && pairs) atomicAdd(a.attended, (unsigned long long)pairs);
      if (lane == 0 && pos) atomicAdd(a.attended + 1, (unsigned long long)pos);
    }
    TR(1)
    TR_FLUSH(0)
    // end of stream, once per gather warp (they alternate tiles)
    for (int e = 0; e < 2 && ok; ++e) {
      acquire_to(pub + 1);
      if (ok) publish_to(pub + 1, 0);
    }
  } else if (warp >= 17 && warp <= 20) {
    // ------------------------------------------------------------ gather warps
    // warps 9/10 copy the K rows of even/odd tiles, warps 11/12 the V rows: consecutive tiles
    // are in flight in different warps, so a tile's latency hides behind its neighbours'.
    const bool is_v = warp >= 19;
    const int par = (warp - 17) & 1;
    const __nv_bfloat16* src_base = is_v ? a.packed_v : a.packed_k;
    const int b_full = is_v ? B_VFULL : B_KFULL, b_empty = is_v ? B_VEMPTY : B_KEMPTY;
    const int64_t row_elems = (int64_t)a.num_kv_heads * D;
    constexpr int LANES_PER_ROW = D / 8;           // 16-byte chunks per row: 32 (D=256) or 16 (D=128)
    constexpr int ROWS_PER_ITER = 32 / LANES_PER_ROW;
    const int sub = lane / LANES_PER_ROW, l_in = lane % LANES_PER_ROW;
    const int slab = l_in >> 3, chunk = l_in & 7;
    const __nv_bfloat16* src_lane = src_base + (int64_t)h * D + l_in * 8;
    // destination of copy u of a group, relative to the group's first row (128-byte swizzle)
    constexpr int GROUP = 8;
    uint32_t dst_off[GROUP];
#pragma unroll
    for (int u = 0; u < GROUP; ++u) dst_off[u] = swz128(u * ROWS_PER_ITER + sub, chunk);
    TR_DECL
    for (int t = par;; t += 2) {
      const int ps = t % PLAN_STAGES, s = t % STAGES;
      if (!mbar_wait(bar(B_PLANFULL + ps), (t / PLAN_STAGES) & 1, abort_flag, a.status, STATUS_TIMEOUT_LOAD)) break;
      TR(0)
      if (lane == 0) { EV(is_v ? 9 : 1, t) }
      const int cnt = plan->count[ps];
      if (cnt == 0) break;
      int r_lo = plan->row[ps * BLOCK_N + lane], r_hi = plan->row[ps * BLOCK_N + lane + 32];
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(B_PLANEMPTY + ps));
      const int n16 = (cnt + 15) & ~15;
      if (a.page_table) {
        // logical row -> physical row of the paged pool: 64 independent lookups in flight
        if (lane < n16) r_lo = a.page_table[r_lo >> 4] * 16 + (r_lo & 15);
        if (lane + 32 < n16) r_hi = a.page_table[r_hi >> 4] * 16 + (r_hi & 15);
      }
      if (!mbar_wait(bar(b_empty + s), ((t / STAGES) & 1) ^ 1, abort_flag, a.status, STATUS_TIMEOUT_LOAD)) break;
      TR(1)
      if (lane == 0) { EV(is_v ? 10 : 2, t) }
      const uint32_t base = smem_u32(smem + (is_v ? C::V_OFF : C::K_OFF) + s * C::KV_BYTES) + slab * (BLOCK_N * 128);
      // 8 copies per step: the row indices are fetched first so the shuffles overlap
#ifdef SEMBLO_SKIP_COPY
      if (false)
#endif
      for (int j0 = 0; j0 < n16; j0 += GROUP * ROWS_PER_ITER) {
        int rows[GROUP];
#pragma unroll
        for (int u = 0; u < GROUP; ++u)
          rows[u] = __shfl_sync(0xffffffffu, j0 < 32 ? r_lo : r_hi, (j0 + u * ROWS_PER_ITER + sub) & 31);
#pragma unroll
        for (int u = 0; u < GROUP; ++u)
          cp_async16(base + j0 * 128 + dst_off[u], src_lane + (int64_t)rows[u] * row_elems);
      }
      TR(2)
      cp_async_wait_all();
      TR(3)
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(b_full + s));
      if (lane == 0) { EV(is_v ? 4 : 3, t) }
      TR(4)
    }
    TR_FLUSH(is_v ? 2 : 1)
  } else if (warp == 21) {
    // ------------------------------------------------------------ UMMA issuer
    // S(j) = Q K(j)^T is issued as soon as K(j) has landed and P V(j-2), which reads the same
    // S/P buffer, has been issued (UMMAs of one thread execute in issue order); O += P(j) V(j)
    // as soon as the softmax warps have stored P(j): whichever is ready first.
    if (elect_one()) {
      constexpr uint32_t idesc_pv = make_idesc_bf16(128, D, false, true);
      bool ok = mbar_wait(bar(B_QFULL), 0, abort_flag, a.status, STATUS_TIMEOUT_MMA);
      tc_fence_after();
      int next_qk = 0, next_pv = 0, end_tile = INT_MAX, plan_seen = -1, cnt_cur = 0;
      int np_of[4] = {0, 0, 0, 0};                    // pages of the tiles in flight (index tile & 3)
      unsigned long long t0 = globaltimer();
      uint32_t idle = 0;
      TR_DECL
      while (ok) {
        bool progress = false;
        if (next_qk < end_tile && next_qk - next_pv < 2) {
          const int j = next_qk, ps = j % PLAN_STAGES, s = j % STAGES, b = j & 1;
          if (plan_seen < j && mbar_try_wait_for(bar(B_PLANFULL + ps), (j / PLAN_STAGES) & 1, POLL_NS)) {
            cnt_cur = plan->count[ps];
            mbar_arrive(bar(B_PLANEMPTY + ps));
            plan_seen = j;
            if (cnt_cur == 0) end_tile = j;
            progress = true;
          }
          if (plan_seen == j && cnt_cur > 0 && mbar_try_wait_for(bar(B_KFULL + s), (j / STAGES) & 1, POLL_NS)) {
            tc_fence_after();
            TR(1)
            const int np = (cnt_cur + 15) >> 4;
            np_of[j & 3] = np;
            const uint32_t k_base = smem_u32(smem + C::K_OFF + s * C::KV_BYTES);
            const uint32_t idesc_qk = make_idesc_bf16(128, np * 16, false, false);
#pragma unroll
            for (int kk = 0; kk < D / 16; ++kk) {
              const uint32_t sl = kk >> 2, ko = (kk & 3) * 32;
              umma_ts(tmem_base + b * BLOCK_N, tmem_base + C::Q_COL + kk * 8,
                      make_smem_desc(k_base + sl * BLOCK_N * 128 + ko, 16, 1024), idesc_qk, kk > 0 ? 1u : 0u);
            }
            umma_commit(bar(B_KEMPTY + s));
            umma_commit(bar(B_SFULL + b));
            TR(2)
            EV(5, j)
            ++next_qk;
            progress = true;
          }
        }
        if (next_pv < next_qk) {
          const int t = next_pv, b = t & 1, s = t % STAGES;
          if (mbar_try_wait_for(bar(B_PFULL + b), (t >> 1) & 1, POLL_NS) && mbar_try_wait_for(bar(B_VFULL + s), (t / STAGES) & 1, POLL_NS)) {
            tc_fence_after();
            TR(1)
            const int np = np_of[t & 3];
            const uint32_t v_base = smem_u32(smem + C::V_OFF + s * C::KV_BYTES);
            for (int kk = 0; kk < np; ++kk)
              umma_ts(tmem_base + C::O_COL, tmem_base + b * BLOCK_N + (kk >> 1) * 32 + (kk & 1) * 8,
                      make_smem_desc(v_base + kk * 16 * 128, BLOCK_N * 128, 1024), idesc_pv,
                      (t > 0 || kk > 0) ? 1u : 0u);
            umma_commit(bar(B_VEMPTY + s));
            umma_commit(bar(B_PVDONE + b));
            TR(3)
            EV(6, t)
            ++next_pv;
            progress = true;
          }
        }
        if (next_pv == end_tile) break;
        if (progress) { TR(1) } else { TR(0) }
        if (progress) {
          idle = 0;
        } else if ((++idle & 0x3ff) == 0) {
          if (idle == 0x400) t0 = globaltimer();
          if (*abort_flag || *reinterpret_cast<volatile int*>(a.status) != 0) { *abort_flag = 1; ok = false; }
          else if (globaltimer() - t0 > WAIT_LIMIT_NS) { *abort_flag = 1; atomicCAS(a.status, 0, STATUS_TIMEOUT_MMA); ok = false; }
        }
      }
      if (ok) umma_commit(bar(B_OREADY));
      { const int lane = 0; (void)lane; TR_FLUSH(3) }
    }
  } else {
    // ------------------------------------------------------------ softmax + epilogue
    // warps 0-7: mask stage, warps 8-15: exp stage; in both, warps 0-3 of the stage take columns
    // [0, 32) of every tile and warps 4-7 columns [32, 64); thread = row
    const int stage = warp >> 3;
    const int hf = (warp >> 2) & 1;
    const int row = threadIdx.x & 127;
    const int qslot = row / G, t = row % G;
    const int slot = q_tile0 + qslot;
    const bool qvalid = slot < a.num_queries;
    const int qi = qvalid ? (a.q_order ? a.q_order[(int64_t)h * a.num_queries + slot] : slot) : 0;
    const uint32_t lane_addr = (uint32_t)((warp & 3) * 32) << 16;
    const uint32_t qbit = 1u << qslot;
    const int64_t hidx = (int64_t)qi * a.num_q_heads + h * G + t;
    float m_ref = -INFINITY, l_part = 0.f;
    bool ok = true;
    int j = 0;
    TR_DECL
    if (stage == 0) {
      attn::stage_q_half<D, C::Q_COL>(qvalid ? a.q + hidx * D + hf * (D / 2) : nullptr, hf, lane_addr, tmem_base,
                                      bar(B_QFULL));
      for (;; ++j) {
        const int ps = j % PLAN_STAGES, b = j & 1;
        TR(5)
        ok = mbar_wait(bar(B_PLANFULL + ps), (j / PLAN_STAGES) & 1, abort_flag, a.status, STATUS_TIMEOUT_SOFTMAX);
        if (!ok) break;
        TR(0)
        const int cnt = plan->count[ps];
        if (cnt == 0) {
          __syncwarp();
          if (lane == 0) mbar_arrive(bar(B_PLANEMPTY + ps));
          // end of the stream: the note slot is free once P V of tile j - 2 has been issued
          if (j >= 2) ok = mbar_wait(bar(B_PVDONE + b), ((j - 2) >> 1) & 1, abort_flag, a.status, STATUS_TIMEOUT_SOFTMAX);
          if (threadIdx.x == 0) note[b].pages = 0;
          mbar_arrive(bar(B_XFULL + b));
          break;
        }
        const int np = (cnt + 15) >> 4;
        // the masks of this half are fetched while the accumulator is awaited
        const uint4* mk = reinterpret_cast<const uint4*>(plan->mask + ps * BLOCK_N + hf * 32);
        uint4 m4[8];
#pragma unroll
        for (int g4 = 0; g4 < 8; ++g4) m4[g4] = mk[g4];
        ok = mbar_wait(bar(B_SFULL + b), (j >> 1) & 1, abort_flag, a.status, STATUS_TIMEOUT_SOFTMAX);
        if (!ok) break;
        TR(1)
        if (threadIdx.x == 0) { EV(7, j) }
        tc_fence_after();
        // a key counts for this row only if the row's query selected the key's cluster
        // (keys past the tile's last row carry an empty mask: the planner clears them)
        float tm[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};      // four short chains
        if (2 * hf < np) {
          uint32_t r[32];
          const uint32_t addr = tmem_base + lane_addr + b * BLOCK_N + hf * 32;
          tmem_ld32(addr, r);
          tmem_ld_wait();
#pragma unroll
          for (int g4 = 0; g4 < 8; ++g4) {
            const uint32_t mm[4] = {m4[g4].x, m4[g4].y, m4[g4].z, m4[g4].w};
            float sv[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              sv[e] = (mm[e] & qbit) != 0u ? __uint_as_float(r[g4 * 4 + e]) : -INFINITY;
              r[g4 * 4 + e] = __float_as_uint(sv[e]);
            }
            tm[g4 & 1] = fmax3(tm[g4 & 1], sv[0], sv[1]);
            tm[2 + (g4 & 1)] = fmax3(tm[2 + (g4 & 1)], sv[2], sv[3]);
          }
          tmem_st32(addr, r);
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(bar(B_PLANEMPTY + ps));
        note[b].row_max[hf * 128 + row] = fmaxf(fmaxf(tm[0], tm[1]), fmaxf(tm[2], tm[3]));
        if (threadIdx.x == 0) note[b].pages = np;
        tmem_st_wait();
        tc_fence_before();
        mbar_arrive(bar(B_XFULL + b));
        if (threadIdx.x == 0) { EV(11, j) }
        TR(2)
      }
    } else {
      for (;; ++j) {
        const int b = j & 1;
        TR(5)
        ok = mbar_wait(bar(B_XFULL + b), (j >> 1) & 1, abort_flag, a.status, STATUS_TIMEOUT_SOFTMAX);
        if (!ok) break;
        TR(1)
        const int np = note[b].pages;
        if (np == 0) break;
        tc_fence_after();
        ok = attn::exp_tile<D, C::O_COL>(np, fmaxf(note[b].row_max[row], note[b].row_max[128 + row]), j, hf, lane_addr,
                                         tmem_base, b * BLOCK_N, bar(B_PVDONE + ((j - 1) & 1)), bar(B_PFULL + b),
                                         a.scale_log2, m_ref, l_part, abort_flag, a.status);
        if (!ok) break;
        if (lane == 0) { EV(warp == 8 ? 8 : 8 + (warp & 3), j) }
        TR(4)
      }
    }
#ifndef SEMBLO_TRACE_WARP
#define SEMBLO_TRACE_WARP 0
#endif
    if (warp == SEMBLO_TRACE_WARP) { TR_FLUSH(4) }
    if (warp == SEMBLO_TRACE_WARP + 8) { TR_FLUSH(5) }

    if (stage == 1) {
      if (ok) ok = mbar_wait(bar(B_OREADY), 0, abort_flag, a.status, STATUS_TIMEOUT_EPILOGUE);
      tc_fence_after();
      attn::epilogue_half<D, C::O_COL>(ok && j > 0, hf, row, lane_addr, tmem_base,
                                       reinterpret_cast<float*>(smem + C::EPI_OFF), bar(B_EPI), m_ref, l_part,
                                       ok && qvalid, a.merge, a.out + hidx * D,
                                       a.partial ? a.partial + hidx * D : nullptr, nullptr, a.lse ? a.lse + hidx : nullptr,
                                       abort_flag, a.status);
    }
    tc_fence_before();
  }
  __syncthreads();
  if (*abort_flag) __nanosleep(50000);
  if (warp == 0) tmem_dealloc(tmem_base, C::TMEM_COLS);
}

template <int D, int G>
int launch_gather(const GatherArgs& a, cudaStream_t st) {
  using C = GatherCfg<D>;
  constexpr int QT = 128 / G;
  auto kern = sparse_gather_prefill_kernel<D, G>;
  SEMBLO_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::TOTAL));
  dim3 grid((unsigned)ceil_div(a.num_queries, QT), a.num_kv_heads);
  kern<<<grid, 704, C::TOTAL, st>>>(a);
  SEMBLO_LAUNCH_CHECK();
  return 0;
}

}  // namespace

extern "C" int semblo_sparse_prefill_gather(
    const void* q, int num_queries, int num_q_heads, int num_kv_heads, int head_dim,
    const int32_t* q_order, const void* packed_k, const void* packed_v, const int32_t* page_table,
    const int32_t* qmask, const int32_t* causal_sizes, const int32_t* indptr, int num_clusters,
    float sm_scale, int merge, const float* partial_in, void* out, float* lse,
    unsigned long long* attended, int32_t* status, void* stream) {
  SEMBLO_REQUIRE(num_kv_heads > 0 && num_q_heads % num_kv_heads == 0, "query heads must be a multiple of the KV heads");
  SEMBLO_REQUIRE(status != nullptr, "status word is required");
  SEMBLO_REQUIRE(qmask && packed_k && packed_v && causal_sizes && indptr, "selection, packed K/V, sizes and indptr are required");
  SEMBLO_REQUIRE(num_clusters % 32 == 0, "cluster count %d must be a multiple of 32", num_clusters);
  SEMBLO_REQUIRE(!merge || lse != nullptr, "merging needs the window's log-sum-exp");
  SEMBLO_REQUIRE((reinterpret_cast<uintptr_t>(packed_k) & 15) == 0 && (reinterpret_cast<uintptr_t>(packed_v) & 15) == 0,
                 "packed K/V must be 16-byte aligned");
  SEMBLO_REQUIRE(q != nullptr && (reinterpret_cast<uintptr_t>(q) & 15) == 0, "q must be 16-byte aligned");
  if (num_queries == 0) return 0;
  GatherArgs a;
  a.num_queries = num_queries; a.num_q_heads = num_q_heads; a.num_kv_heads = num_kv_heads;
  a.num_clusters = num_clusters; a.q = (const __nv_bfloat16*)q; a.q_order = q_order; a.qmask = qmask; a.causal_sizes = causal_sizes;
  a.indptr = indptr; a.page_table = page_table;
  a.packed_k = (const __nv_bfloat16*)packed_k; a.packed_v = (const __nv_bfloat16*)packed_v;
  a.scale_log2 = sm_scale * LOG2EF; a.out = (__nv_bfloat16*)out; a.lse = lse; a.merge = merge; a.partial = partial_in;
  a.attended = attended; a.status = status;
  const int g = num_q_heads / num_kv_heads;
  cudaStream_t st = (cudaStream_t)stream;
#define SEMBLO_GATHER_CASE(DD, GG) \
  if (head_dim == DD && g == GG) return launch_gather<DD, GG>(a, st);
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
