// Block-sparse prefill attention, sparse part: row-granular gather of the selected
// clusters' visible rows, tcgen05 / TMEM attention, LSE merge with the window partial.
//
// One CTA owns QT = 128 / G queries of one KV head, taken in the caller's tile order
// (queries with similar selections are placed in the same tile).  Warp roles (GW = 3):
//   warps 0-7  softmax, two threads per row with 32 columns each (attn::softmax_tile): running
//              maximum and sum, P as bf16 into TMEM; they also write the output in the epilogue
//   warp  8    planner: walks the tile's cluster bitmasks 32 clusters at a time (sizes and
//              starts fetched by 32 lanes in parallel), and expands the union of selected
//              clusters into a stream of packed rows, each tagged with the 32-bit set of
//              query slots that selected its cluster; 64 rows make a tile
//   warps 9 .. 8 + 2 GW  gather: GW warps for the K rows and GW for the V rows, tile t in warp
//              t mod GW; 16-byte cp.async into the 128-byte-swizzled UMMA layout (only visible
//              rows are read: no page padding), then published to the async proxy
//   next warp  UMMA issuer: S = [Q | E] [K | B]^T and O += P V, accumulators in TMEM, in the
//              fixed order P V(t), S(t + 2)
//   last warp  selection operand B of every tile from the planner's slot masks
// The selection itself is applied by the S product (see the comment above GatherCfg): the
// softmax warps never look at a mask.
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

constexpr int GW = 3;     // gather warps per operand; warp w of them takes tiles t = w (mod GW)
constexpr int W_GATHER = 9, W_MMA = W_GATHER + 2 * GW, W_BIAS = W_MMA + 1;
constexpr int GATHER_THREADS = 32 * (W_BIAS + 1);
constexpr int NSB = 2;       // S buffers: tiles between Q K^T and the end of their softmax
constexpr int BIAS_BYTES = BLOCK_N * 64;     // per tile: 64 keys x 32 query slots, bf16
constexpr uint32_t BIAS_OFF_BITS = 0xF180u;  // bf16 -2^100: the logit of a key the row's query did not select

// The selection enters the logits through the tensor cores: S = [Q | E] [K | B]^T, where row
// r of E is the one-hot vector of the row's query slot (32 slots) and B[key][slot] is 0 if
// the slot's query selected the key's cluster and -2^100 otherwise.  Adding 0 leaves a
// selected logit bit-exact; a rejected one becomes about -2^100, whose exponential is 0.
//
// Tensor memory (512 columns) holds NSB S buffers of 64 columns, O (D columns) and Q (D / 2).
// With two S buffers everything fits at D = 256; a third one (NSB = 3) moves the last
// 128 dims of Q into shared memory and leaves room for two V stages only.
template <int D>
struct GatherCfg {
  static constexpr int K_STAGES = D >= 256 ? 3 : 5;
  static constexpr int V_STAGES = D >= 256 ? (NSB >= 3 ? 2 : 3) : 5;
  static constexpr int Q_TMEM_DIMS = (D >= 256 && NSB >= 3) ? 128 : D;
  static constexpr int Q_SMEM_DIMS = D - Q_TMEM_DIMS;
  static constexpr int SLABS = D / 64;
  static constexpr int KV_BYTES = BLOCK_N * D * 2;
  static constexpr int QHI_BYTES = 128 * Q_SMEM_DIMS * 2;
  static constexpr int QHI_OFF = 0;
  static constexpr int K_OFF = QHI_OFF + QHI_BYTES;
  static constexpr int V_OFF = K_OFF + K_STAGES * KV_BYTES;
  static constexpr int ONEHOT_OFF = V_OFF + V_STAGES * KV_BYTES;   // E: 128 rows x 64 bytes, 64-byte swizzle
  static constexpr int BIAS_OFF = ONEHOT_OFF + 128 * 64;           // B: one tile per K stage
  static constexpr int LUT_OFF = BIAS_OFF + K_STAGES * BIAS_BYTES; // uint4 [256]: 8 selection bits -> 8 bf16
  static constexpr int MX_OFF = LUT_OFF + 4096;                    // float [2][2][128]: half-row maxima
  static constexpr int EPI_OFF = MX_OFF + 2048;                    // float [2][128]
  static constexpr int PLAN_OFF = EPI_OFF + 2048;
  static constexpr int BAR_OFF = PLAN_OFF + (int)sizeof(Plan);
  static constexpr int NUM_BARS = 8 + 3 * NSB + 2 * K_STAGES + 2 * V_STAGES + 2 * PLAN_STAGES;
  static constexpr int MISC_OFF = BAR_OFF + 8 * NUM_BARS;          // tmem slot, abort flag, pages [NSB]
  static constexpr int TOTAL = MISC_OFF + 32;      // the dynamic segment must start 1024-byte aligned
  static constexpr int TMEM_COLS = 512;
  static constexpr int O_COL = NSB * BLOCK_N;      // S/P buffers, then O, then Q
  static constexpr int Q_COL = O_COL + D;
  static_assert(Q_COL + Q_TMEM_DIMS / 2 <= TMEM_COLS, "tensor memory budget");
  static_assert(TOTAL <= 232448, "shared memory budget");
  // a gather warp waits on a stage by phase parity, which only tells neighbouring phases apart:
  // no warp may run a whole ring ahead of another
  static_assert(GW <= K_STAGES && GW <= V_STAGES, "more gather warps than stages");
  static_assert(ONEHOT_OFF % 1024 == 0, "swizzled operands start on the swizzle period");
};

struct GatherArgs {
  int num_queries, num_q_heads, num_kv_heads, num_clusters;
  const __nv_bfloat16* q;       // [Q, Hq, D]
  const int32_t* q_order;       // [Hkv, Q] tile order, or null
  const int32_t* cta_order;     // [tiles * Hkv] (tile * Hkv + head) in launch order, or null
  const int32_t* qmask;         // [Q, Hkv, C/32]
  const int32_t* causal_sizes;  // [Hkv, C]
  const int32_t* indptr;        // [Hkv, C+1]
  const int32_t* page_table;    // or null
  const __nv_bfloat16* packed_k;
  const __nv_bfloat16* packed_v;
  int64_t packed_rows;          // rows of the pools
  float scale_log2;
  __nv_bfloat16* out;           // [Q, Hq, D] in: window partial, out: merged
  float* lse;                   // [Q, Hq]    in: window lse,     out: merged (natural log)
  const float* partial;         // [Q, Hq, D] fp32 window partial, or null: it is in `out` as bf16
  int merge;                    // 0: no window partial, write the sparse result alone
  unsigned long long* attended;
  int* status;
};

enum { B_QFULL = 0, B_OREADY = 1, B_EPI = 2, B_QHI = 3, B_PAIR = 4, B_SFULL = 8, B_PFULL = 8 + NSB,
       B_PVDONE = 8 + 2 * NSB, B_KFULL = 8 + 3 * NSB };

// Shared-memory descriptor of a K-major operand whose rows are 64 bytes (64-byte swizzle,
// eight-row groups 512 bytes apart).
__device__ __forceinline__ uint64_t make_smem_desc_sw64(uint32_t addr) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((addr & 0x3ffff) >> 4);
  d |= static_cast<uint64_t>(1) << 16;
  d |= static_cast<uint64_t>(512 >> 4) << 32;
  d |= 1ull << 46;            // descriptor version (Blackwell)
  d |= 4ull << 61;            // SWIZZLE_64B
  return d;
}
// Byte offset of 16-byte chunk c of row r in such an operand.
__device__ __forceinline__ uint32_t sw64_off(int r, int c) {
  return (uint32_t)((r >> 3) * 512 + (r & 7) * 64 + ((c ^ ((r >> 1) & 3)) << 4));
}

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_wait_all() {
  asm volatile("cp.async.commit_group;\n\tcp.async.wait_group 0;" ::: "memory");
}

template <int D, int G>
__global__ void __launch_bounds__(GATHER_THREADS, 1)
sparse_gather_prefill_kernel(const __grid_constant__ CUtensorMap tmap_q, const GatherArgs a) {
  using C = GatherCfg<D>;
  constexpr int QT = 128 / G;
  constexpr int K_STAGES = C::K_STAGES, V_STAGES = C::V_STAGES;
  constexpr int B_KEMPTY = B_KFULL + K_STAGES;
  constexpr int B_VFULL = B_KEMPTY + K_STAGES;
  constexpr int B_VEMPTY = B_VFULL + V_STAGES;
  constexpr int B_PLANFULL = B_VEMPTY + V_STAGES;
  constexpr int B_PLANEMPTY = B_PLANFULL + PLAN_STAGES;
  extern __shared__ __align__(1024) uint8_t smem[];
  if (smem_u32(smem) & 1023u) {                    // the swizzled tiles need 1024-byte alignment
    if (threadIdx.x == 0) atomicCAS(a.status, 0, STATUS_SMEM_ALIGN);
    return;
  }
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + C::BAR_OFF);
  Plan* plan = reinterpret_cast<Plan*>(smem + C::PLAN_OFF);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + C::MISC_OFF);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  volatile int* tile_pages = reinterpret_cast<volatile int*>(tmem_slot + 2);   // [NSB]; 0 ends the stream
  auto bar = [&](int i) { return smem_u32(&bars[i]); };

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // with a launch order the grid is one-dimensional and entry i names the (tile, head) of CTA i
  const int cta_id = a.cta_order ? a.cta_order[blockIdx.x] : -1;
  const int h = cta_id >= 0 ? cta_id % a.num_kv_heads : (int)blockIdx.y;
  const int q_tile0 = (cta_id >= 0 ? cta_id / a.num_kv_heads : (int)blockIdx.x) * QT;

  if (threadIdx.x == 0) {
    mbar_init(bar(B_QFULL), 256);
    mbar_init(bar(B_OREADY), 1);
    mbar_init(bar(B_EPI), 256);
    mbar_init(bar(B_QHI), 1);
    for (int i = 0; i < 4; ++i) mbar_init(bar(B_PAIR + i), 2);    // the two warps that share 32 rows
    for (int b = 0; b < NSB; ++b) {
      mbar_init(bar(B_SFULL + b), 2);          // the issuer's own arrival (after the page count) + its commit
      mbar_init(bar(B_PFULL + b), 8);          // the softmax warps
      mbar_init(bar(B_PVDONE + b), 1);
    }
    for (int s = 0; s < K_STAGES; ++s) {
      mbar_init(bar(B_KFULL + s), 2);          // the K rows and the tile's selection operand
      mbar_init(bar(B_KEMPTY + s), 1);
    }
    for (int s = 0; s < V_STAGES; ++s) {
      mbar_init(bar(B_VFULL + s), 1);
      mbar_init(bar(B_VEMPTY + s), 1);
    }
    for (int s = 0; s < PLAN_STAGES; ++s) {
      mbar_init(bar(B_PLANFULL + s), 1);
      mbar_init(bar(B_PLANEMPTY + s), 4);     // a K and a V gather warp, the UMMA issuer, the selection warp
    }
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 0) {
    tmem_alloc(smem_u32(tmem_slot), C::TMEM_COLS);
    tmem_relinquish();
  }
  {
    // table: 8 selection bits -> 8 bf16 (0 where the bit is set); E: one-hot query slot of every row
    uint4* lut = reinterpret_cast<uint4*>(smem + C::LUT_OFF);
    for (int i = threadIdx.x; i < 256; i += blockDim.x) {
      const uint32_t n = ~(uint32_t)i;
      uint32_t w[4];
#pragma unroll
      for (int k = 0; k < 4; ++k)
        w[k] = (((n >> (2 * k)) & 1u) | (((n >> (2 * k + 1)) & 1u) << 16)) * BIAS_OFF_BITS;
      lut[i] = make_uint4(w[0], w[1], w[2], w[3]);
    }
    for (int i = threadIdx.x; i < 128 * 4; i += blockDim.x) {
      const int r = i >> 2, c = i & 3, qs = r / G;
      uint32_t w[4] = {0u, 0u, 0u, 0u};
      if ((qs >> 3) == c) w[(qs & 7) >> 1] = 0x3F80u << (16 * (qs & 1));
      *reinterpret_cast<uint4*>(smem + C::ONEHOT_OFF + sw64_off(r, c)) = make_uint4(w[0], w[1], w[2], w[3]);
    }
    fence_proxy_async_smem();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 8) {
    // ------------------------------------------------------------ planner
    const int slot = q_tile0 + lane;
    const bool qvalid = lane < QT && slot < a.num_queries;
    const int qi = qvalid ? (a.q_order ? a.q_order[(int64_t)h * a.num_queries + slot] : slot) : 0;
    if (C::Q_SMEM_DIMS > 0) {
      // the dims of Q that stay in shared memory: one box (64 dims, G heads) per query and slab
      const unsigned vmask = __ballot_sync(0xffffffffu, qvalid);
      if (lane == 0) {
        tma_prefetch_desc(&tmap_q);
        mbar_arrive_expect_tx(bar(B_QHI), (uint32_t)__popc(vmask) * G * C::Q_SMEM_DIMS * 2);
      }
      for (int i = 0; i < QT; ++i) {
        const int qsrc = __shfl_sync(0xffffffffu, qi, i);
        if (lane == 0 && ((vmask >> i) & 1))
          for (int sl = 0; sl < C::Q_SMEM_DIMS / 64; ++sl)
            tma_load_3d(smem_u32(smem + C::QHI_OFF + sl * 128 * 128 + i * G * 128), &tmap_q, bar(B_QHI),
                        C::Q_TMEM_DIMS + sl * 64, h * G, qsrc);
      }
    }
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
    auto acquire_to = [&](int upto) {          // make tiles [acq, upto) writable
      while (ok && acq < upto) {
        if (lane == 0)
          ok = mbar_wait(bar(B_PLANEMPTY + acq % PLAN_STAGES), ((acq / PLAN_STAGES) & 1) ^ 1, abort_flag, a.status,
                         STATUS_TIMEOUT_LOAD);
        ok = __shfl_sync(0xffffffffu, (int)ok, 0) != 0;
        ++acq;
      }
    };
    auto publish_to = [&](int upto, int last_count) {   // publish tiles [pub, upto), the last with last_count rows
      __syncwarp();
      if (lane == 0)
        for (int t = pub; t < upto; ++t) {
          plan->count[t % PLAN_STAGES] = t == upto - 1 ? last_count : BLOCK_N;
          mbar_arrive(bar(B_PLANFULL + t % PLAN_STAGES));
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
      while (wlo < end && ok) {
        // a wave: as far as the plan ring reaches beyond the oldest unpublished tile
        const int whi = min(end, (pub + PLAN_STAGES) * BLOCK_N);
        acquire_to((whi + BLOCK_N - 1) / BLOCK_N);
        if (!ok) break;
        const int lo = max(a_b, wlo), hi = min(e_b, whi);
        const bool big = hi - lo > SELF_MAX;
        if (!big)
          for (int p = lo; p < hi; ++p) put(p, row_minus_pos + p, mask_b);
        for (unsigned bigs = __ballot_sync(0xffffffffu, big); bigs; bigs &= bigs - 1) {
          const int bb = __ffs(bigs) - 1;
          const int blo = __shfl_sync(0xffffffffu, lo, bb), bhi = __shfl_sync(0xffffffffu, hi, bb);
          const int brow = __shfl_sync(0xffffffffu, row_minus_pos, bb);
          const unsigned bmask = __shfl_sync(0xffffffffu, mask_b, bb);
          for (int p = blo + lane; p < bhi; p += 32) put(p, brow + p, bmask);
        }
        publish_to(whi / BLOCK_N, BLOCK_N);
        wlo = whi;
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
    // end of stream, once per gather warp of an operand (they take tiles in turn)
    for (int e = 0; e < GW && ok; ++e) {
      acquire_to(pub + 1);
      if (ok) publish_to(pub + 1, 0);
    }
  } else if (warp >= W_GATHER && warp < W_MMA) {
    // ------------------------------------------------------------ gather warps
    // GW warps copy the K rows and GW warps the V rows, tile t in warp t mod GW of its operand:
    // consecutive tiles are in flight in different warps, so a tile's latency hides behind its
    // neighbours'.
    const bool is_v = warp >= W_GATHER + GW;
    const int par = (warp - W_GATHER) % GW;
    const __nv_bfloat16* src_base = is_v ? a.packed_v : a.packed_k;
    const int b_full = is_v ? B_VFULL : B_KFULL, b_empty = is_v ? B_VEMPTY : B_KEMPTY;
    const int stages = is_v ? V_STAGES : K_STAGES;
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
    for (int t = par;; t += GW) {
      const int ps = t % PLAN_STAGES, s = t % stages;
      if (!mbar_wait(bar(B_PLANFULL + ps), (t / PLAN_STAGES) & 1, abort_flag, a.status, STATUS_TIMEOUT_LOAD)) break;
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
      if (!mbar_wait(bar(b_empty + s), ((t / stages) & 1) ^ 1, abort_flag, a.status, STATUS_TIMEOUT_LOAD)) break;
      const uint32_t base = smem_u32(smem + (is_v ? C::V_OFF : C::K_OFF) + s * C::KV_BYTES) + slab * (BLOCK_N * 128);
      // 8 copies per step: the row indices are fetched first so the shuffles overlap
      for (int j0 = 0; j0 < n16; j0 += GROUP * ROWS_PER_ITER) {
        int rows[GROUP];
#pragma unroll
        for (int u = 0; u < GROUP; ++u)
          rows[u] = __shfl_sync(0xffffffffu, j0 < 32 ? r_lo : r_hi, (j0 + u * ROWS_PER_ITER + sub) & 31);
#pragma unroll
        for (int u = 0; u < GROUP; ++u)
          cp_async16(base + j0 * 128 + dst_off[u], src_lane + (int64_t)rows[u] * row_elems);
      }
      cp_async_wait_all();
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(b_full + s));
    }
  } else if (warp == W_MMA) {
    // ------------------------------------------------------------ UMMA issuer
    // One thread issues S(j) = [Q | E] [K(j) | B(j)]^T and O += P(t) V(t) in the fixed order
    // S(0) .. S(NSB-1), then P V(t), S(t + NSB) for t = 0, 1, ...  UMMAs of one thread execute in
    // issue order, so S(t + NSB) may follow P V(t), which reads P from the same buffer, without
    // waiting for it to complete.  The tile's page count travels with the buffer: it is stored
    // before this thread's own arrival on the buffer's barrier (0 ends the stream).
    if (elect_one()) {
      constexpr uint32_t idesc_pv = make_idesc_bf16(128, D, false, true);
      bool ok = mbar_wait(bar(B_QFULL), 0, abort_flag, a.status, STATUS_TIMEOUT_MMA);
      if (ok && C::Q_SMEM_DIMS > 0) ok = mbar_wait(bar(B_QHI), 0, abort_flag, a.status, STATUS_TIMEOUT_MMA);
      tc_fence_after();
      const uint32_t qhi_base = smem_u32(smem + C::QHI_OFF);
      const uint32_t onehot_base = smem_u32(smem + C::ONEHOT_OFF);
      int ps = 0, ks = 0, qb = 0;                     // ring slots of the next S product
      uint32_t plan_par = 0, k_par = 0;
      bool ended = false;
      auto issue_s = [&](int j) {
        ok = mbar_wait(bar(B_PLANFULL + ps), plan_par, abort_flag, a.status, STATUS_TIMEOUT_MMA);
        if (!ok) return;
        const int cnt = plan->count[ps];
        mbar_arrive(bar(B_PLANEMPTY + ps));
        if (cnt == 0) {                               // end of the stream
          tile_pages[qb] = 0;
          mbar_arrive(bar(B_SFULL + qb));
          mbar_arrive(bar(B_SFULL + qb));
          ended = true;
          return;
        }
        const int np = (cnt + 15) >> 4;
        tile_pages[qb] = np;
        mbar_arrive(bar(B_SFULL + qb));
        ok = mbar_wait(bar(B_KFULL + ks), k_par, abort_flag, a.status, STATUS_TIMEOUT_MMA);
        if (!ok) return;
        tc_fence_after();
        const uint32_t k_base = smem_u32(smem + C::K_OFF + ks * C::KV_BYTES);
        const uint32_t bias_base = smem_u32(smem + C::BIAS_OFF + ks * BIAS_BYTES);
        const uint32_t idesc_qk = make_idesc_bf16(128, np * 16, false, false);
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint32_t sl = kk >> 2, ko = (kk & 3) * 32;
          const uint64_t kd = make_smem_desc(k_base + sl * BLOCK_N * 128 + ko, 16, 1024);
          if (kk < C::Q_TMEM_DIMS / 16)
            umma_ts(tmem_base + qb * BLOCK_N, tmem_base + C::Q_COL + kk * 8, kd, idesc_qk, kk > 0 ? 1u : 0u);
          else                        // the dims of Q that live in shared memory
            umma_ss(tmem_base + qb * BLOCK_N,
                    make_smem_desc(qhi_base + (sl - C::Q_TMEM_DIMS / 64) * 128 * 128 + ko, 16, 1024), kd, idesc_qk, 1u);
        }
#pragma unroll
        for (int kk = 0; kk < 2; ++kk)  // the selection: 32 query slots
          umma_ss(tmem_base + qb * BLOCK_N, make_smem_desc_sw64(onehot_base + kk * 32),
                  make_smem_desc_sw64(bias_base + kk * 32), idesc_qk, 1u);
        umma_commit(bar(B_KEMPTY + ks));
        umma_commit(bar(B_SFULL + qb));
        if (++ps == PLAN_STAGES) { ps = 0; plan_par ^= 1; }
        if (++ks == K_STAGES) { ks = 0; k_par ^= 1; }
        if (++qb == NSB) qb = 0;
      };
      int next_s = 0;
      for (; next_s < NSB && ok && !ended; ++next_s) issue_s(next_s);
      int vs = 0, pb = 0;
      uint32_t v_par = 0, p_par = 0;
      for (int t = 0; ok; ++t) {
        ok = mbar_wait(bar(B_PFULL + pb), p_par, abort_flag, a.status, STATUS_TIMEOUT_MMA);
        if (!ok) break;
        const int np = tile_pages[pb];
        if (np == 0) break;
        ok = mbar_wait(bar(B_VFULL + vs), v_par, abort_flag, a.status, STATUS_TIMEOUT_MMA);
        if (!ok) break;
        tc_fence_after();
        const uint32_t v_base = smem_u32(smem + C::V_OFF + vs * C::KV_BYTES);
        for (int kk = 0; kk < np; ++kk)
          umma_ts(tmem_base + C::O_COL, tmem_base + pb * BLOCK_N + (kk >> 1) * 32 + (kk & 1) * 8,
                  make_smem_desc(v_base + kk * 16 * 128, BLOCK_N * 128, 1024), idesc_pv,
                  (t > 0 || kk > 0) ? 1u : 0u);
        umma_commit(bar(B_VEMPTY + vs));
        umma_commit(bar(B_PVDONE + pb));
        if (++vs == V_STAGES) { vs = 0; v_par ^= 1; }
        if (++pb == NSB) { pb = 0; p_par ^= 1; }
        if (!ended) { issue_s(next_s); ++next_s; }
      }
      if (ok) umma_commit(bar(B_OREADY));
    }
  } else if (warp == W_BIAS) {
    // ------------------------------------------------------------ selection operand B
    // B[key][slot] of a tile from the planner's per-key slot masks: lane = (key & 7, 8-slot
    // group), eight keys per pass; one table lookup turns 8 mask bits into 8 bf16.
    const uint4* lut = reinterpret_cast<const uint4*>(smem + C::LUT_OFF);
    const int r0 = lane >> 2, c = lane & 3;
    int ps = 0, s = 0;
    uint32_t plan_par = 0, empty_par = 1;
    for (int t = 0;; ++t) {
      if (!mbar_wait(bar(B_PLANFULL + ps), plan_par, abort_flag, a.status, STATUS_TIMEOUT_LOAD)) break;
      if (plan->count[ps] == 0) break;
      uint32_t m[8];
#pragma unroll
      for (int it = 0; it < 8; ++it) m[it] = plan->mask[ps * BLOCK_N + it * 8 + r0];
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(B_PLANEMPTY + ps));
      if (!mbar_wait(bar(B_KEMPTY + s), empty_par, abort_flag, a.status, STATUS_TIMEOUT_LOAD)) break;
      uint8_t* dst = smem + C::BIAS_OFF + s * BIAS_BYTES;
#pragma unroll
      for (int it = 0; it < 8; ++it)
        *reinterpret_cast<uint4*>(dst + sw64_off(it * 8 + r0, c)) = lut[(m[it] >> (8 * c)) & 0xFFu];
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(B_KFULL + s));
      if (++ps == PLAN_STAGES) { ps = 0; plan_par ^= 1; }
      if (++s == K_STAGES) { s = 0; empty_par ^= 1; }
    }
  } else if (warp < 8) {
    // ------------------------------------------------------------ softmax + epilogue
    // Two threads per row: warps 0-3 take columns [0, 32) of every tile, warps 4-7 columns
    // [32, 64).  Both read all 64 logits for the row maximum, so they agree on it without
    // talking to each other; each turns its own half into P.
    const int hf = (warp >> 2) & 1;
    const int row = threadIdx.x & 127;
    const int qslot = row / G, t = row % G;
    const int slot = q_tile0 + qslot;
    const bool qvalid = slot < a.num_queries;
    const int qi = qvalid ? (a.q_order ? a.q_order[(int64_t)h * a.num_queries + slot] : slot) : 0;
    const uint32_t lane_addr = (uint32_t)((warp & 3) * 32) << 16;
    const int64_t hidx = (int64_t)qi * a.num_q_heads + h * G + t;
    float m_ref = -INFINITY, l_part = 0.f;
    bool ok = true;
    int j = 0, b = 0;
    uint32_t s_par = 0, pv_prev_par = 0;             // pv_prev_par: parity of P V(j - 1) on its buffer
    attn::stage_q_half<C::Q_TMEM_DIMS, C::Q_COL>(qvalid ? a.q + hidx * D + hf * (C::Q_TMEM_DIMS / 2) : nullptr, hf,
                                                 lane_addr, tmem_base, bar(B_QFULL));
    for (;; ++j) {
      ok = mbar_wait_warp(bar(B_SFULL + b), s_par, abort_flag, a.status, STATUS_TIMEOUT_SOFTMAX);
      if (!ok) break;
      const int np = tile_pages[b];
      if (np == 0) {                        // end of the stream: tell the P V issuer
        if (lane == 0) mbar_arrive(bar(B_PFULL + b));
        break;
      }
      tc_fence_after();
      // columns past the tile's pages were not written by this tile's product: lim = 16 np
      ok = attn::softmax_tile<D, C::O_COL>(np, np * 16, j, hf, row, lane_addr, tmem_base, b * BLOCK_N,
                                           reinterpret_cast<float*>(smem + C::MX_OFF), bar(B_PAIR + (warp & 3)), bar(B_PVDONE + (b == 0 ? NSB - 1 : b - 1)),
                                           pv_prev_par, bar(B_PFULL + b), a.scale_log2, m_ref, l_part, abort_flag,
                                           a.status);
      if (!ok) break;
      if (++b == NSB) { b = 0; s_par ^= 1; }
      // P V(j) of the tile just finished lives on buffer (j % NSB) with parity (j / NSB) & 1
      pv_prev_par = (uint32_t)((j / NSB) & 1);
    }
    if (ok) ok = mbar_wait(bar(B_OREADY), 0, abort_flag, a.status, STATUS_TIMEOUT_EPILOGUE);
    tc_fence_after();
    attn::epilogue_half<D, C::O_COL>(ok && j > 0, hf, row, lane_addr, tmem_base,
                                     reinterpret_cast<float*>(smem + C::EPI_OFF), bar(B_EPI), m_ref, l_part,
                                     ok && qvalid, a.merge, a.out + hidx * D,
                                     a.partial ? a.partial + hidx * D : nullptr, nullptr, a.lse ? a.lse + hidx : nullptr,
                                     abort_flag, a.status);
    tc_fence_before();
  }
  __syncthreads();
  if (*abort_flag) __nanosleep(50000);
  if (warp == 0) tmem_dealloc(tmem_base, C::TMEM_COLS);
}

// ------------------------------------------------------------------ launch order
// work[tile * Hkv + h] = rows in the union of the tile's selections (what the tile's CTA gathers).
// One warp per (tile, head): lanes take the bitmask words in turn.
__global__ void tile_work_kernel(const int32_t* __restrict__ q_order, const int32_t* __restrict__ qmask,
                                 const int32_t* __restrict__ causal_sizes, int num_queries, int num_kv_heads,
                                 int num_clusters, int qt, int num_tiles, int32_t* __restrict__ work) {
  const int lane = threadIdx.x & 31;
  const int item = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (item >= num_tiles * num_kv_heads) return;
  const int tile = item / num_kv_heads, h = item % num_kv_heads;
  const int nwords = num_clusters >> 5;
  const int32_t* csz = causal_sizes + (int64_t)h * num_clusters;
  // lane i holds the query of slot i (qt <= 32); -1 past the end
  const int my_slot = tile * qt + lane;
  const int my_q = (lane < qt && my_slot < num_queries)
                       ? (q_order ? q_order[(int64_t)h * num_queries + my_slot] : my_slot) : -1;
  int total = 0;
  for (int w0 = 0; w0 < nwords; w0 += 32) {
    const int w = w0 + lane;
    uint32_t u = 0u;
#pragma unroll 8
    for (int i = 0; i < qt; ++i) {
      const int qi = __shfl_sync(0xffffffffu, my_q, i);
      if (qi >= 0 && w < nwords) u |= (uint32_t)__ldg(qmask + ((int64_t)qi * num_kv_heads + h) * nwords + w);
    }
    if (u) {
      // the word's 32 sizes in eight independent 16-byte loads
      const int4* c4 = reinterpret_cast<const int4*>(csz + w * 32);
#pragma unroll
      for (int k = 0; k < 8; ++k) {
        const int4 v = __ldg(c4 + k);
        const uint32_t nib = (u >> (4 * k)) & 0xFu;
        total += ((nib & 1u) ? v.x : 0) + ((nib & 2u) ? v.y : 0) + ((nib & 4u) ? v.z : 0) + ((nib & 8u) ? v.w : 0);
      }
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) total += __shfl_xor_sync(0xffffffffu, total, o);
  if (lane == 0) work[item] = total;
}

// order[] = the items (tile * heads + head) head by head, each head's by descending work in
// `classes` classes of equal width (one block; heads * classes <= 1024).  CTAs that run at the same
// time then gather from one head's rows, a working set the L2 can hold.  heads = 1: one global order.
__global__ void tile_order_kernel(const int32_t* __restrict__ work, int n, int heads, int classes,
                                  int32_t* __restrict__ order) {
  __shared__ int s_max;
  __shared__ int s_hist[1024];
  if (threadIdx.x == 0) s_max = 0;
  s_hist[threadIdx.x] = 0;
  __syncthreads();
  int m = 0;
  for (int i = threadIdx.x; i < n; i += blockDim.x) m = max(m, work[i]);
  atomicMax(&s_max, m);
  __syncthreads();
  const long long top = (long long)s_max + 1;
  const int bins = heads * classes;
  for (int i = threadIdx.x; i < n; i += blockDim.x)
    atomicAdd(&s_hist[(i % heads) * classes + classes - 1 - (int)((long long)work[i] * classes / top)], 1);
  __syncthreads();
  if (threadIdx.x < 32) {                 // exclusive scan of up to 1024 bins: 32 per lane
    const int lane = threadIdx.x;
    int sum = 0;
    for (int k = 0; k < 32; ++k) sum += lane * 32 + k < bins ? s_hist[lane * 32 + k] : 0;
    int incl = sum;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int up = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += up;
    }
    int run = incl - sum;
    for (int k = 0; k < 32; ++k) {
      if (lane * 32 + k < bins) { const int c = s_hist[lane * 32 + k]; s_hist[lane * 32 + k] = run; run += c; }
    }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < n; i += blockDim.x)
    order[atomicAdd(&s_hist[(i % heads) * classes + classes - 1 - (int)((long long)work[i] * classes / top)], 1)] = i;
}

template <int D, int G>
int launch_gather(const GatherArgs& a, cudaStream_t st) {
  using C = GatherCfg<D>;
  constexpr int QT = 128 / G;
  CUtensorMap mq;
  {
    uint64_t d[3] = {(uint64_t)D, (uint64_t)a.num_q_heads, (uint64_t)a.num_queries};
    uint64_t st2[2] = {(uint64_t)D * 2, (uint64_t)a.num_q_heads * D * 2};
    uint32_t bx[3] = {64, (uint32_t)G, 1};
    int rc = semblo::make_tensor_map_bf16(&mq, a.q, 3, d, st2, bx);
    if (rc) return rc;
  }
  auto kern = sparse_gather_prefill_kernel<D, G>;
  SEMBLO_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::TOTAL));
  dim3 grid((unsigned)ceil_div(a.num_queries, QT), a.num_kv_heads);
  if (a.cta_order) grid = dim3(grid.x * grid.y, 1);
  kern<<<grid, GATHER_THREADS, C::TOTAL, st>>>(mq, a);
  SEMBLO_LAUNCH_CHECK();
  return 0;
}

}  // namespace

extern "C" int semblo_sparse_prefill_gather(
    const void* q, int num_queries, int num_q_heads, int num_kv_heads, int head_dim,
    const int32_t* q_order, const int32_t* cta_order, const void* packed_k, const void* packed_v,
    int64_t packed_rows, const int32_t* page_table,
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
  SEMBLO_REQUIRE(packed_rows > 0 && packed_rows < (int64_t)1 << 31, "packed_rows %lld is out of range", (long long)packed_rows);
  if (num_queries == 0) return 0;
  GatherArgs a;
  a.num_queries = num_queries; a.num_q_heads = num_q_heads; a.num_kv_heads = num_kv_heads;
  a.num_clusters = num_clusters; a.q = (const __nv_bfloat16*)q; a.q_order = q_order; a.cta_order = cta_order; a.qmask = qmask; a.causal_sizes = causal_sizes;
  a.indptr = indptr; a.page_table = page_table;
  a.packed_k = (const __nv_bfloat16*)packed_k; a.packed_v = (const __nv_bfloat16*)packed_v;
  a.packed_rows = packed_rows;
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

extern "C" int semblo_gather_launch_order(const int32_t* q_order, const int32_t* qmask, const int32_t* causal_sizes,
                                          int num_queries, int num_q_heads, int num_kv_heads, int num_clusters,
                                          int32_t* work, int32_t* order_out, void* stream) {
  SEMBLO_REQUIRE(num_kv_heads > 0 && num_q_heads % num_kv_heads == 0, "query heads must be a multiple of the KV heads");
  SEMBLO_REQUIRE(qmask && causal_sizes && work && order_out, "selection, sizes and the two outputs are required");
  SEMBLO_REQUIRE(num_clusters % 32 == 0, "cluster count %d must be a multiple of 32", num_clusters);
  const int g = num_q_heads / num_kv_heads;
  SEMBLO_REQUIRE(g == 4 || g == 8 || g == 16, "4, 8 or 16 query heads per KV head (got %d)", g);
  if (num_queries == 0) return 0;
  const int qt = 128 / g;
  const int tiles = (num_queries + qt - 1) / qt;
  const int n = tiles * num_kv_heads;
  cudaStream_t st = (cudaStream_t)stream;
  tile_work_kernel<<<(unsigned)ceil_div(n, 8), 256, 0, st>>>(q_order, qmask, causal_sizes, num_queries, num_kv_heads,
                                                             num_clusters, qt, tiles, work);
  SEMBLO_REQUIRE(num_kv_heads <= 128, "at most 128 KV heads");
  const int classes = std::min(64, 1024 / num_kv_heads);
  tile_order_kernel<<<1, 1024, 0, st>>>(work, n, num_kv_heads, classes, order_out);
  SEMBLO_LAUNCH_CHECK();
  return 0;
}
