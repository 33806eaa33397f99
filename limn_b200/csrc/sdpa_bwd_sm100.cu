// "sdpa_bwd_q" and "sdpa_bwd_kv" for f16/bf16 with hd and hd_v multiples of 8 up to 128 (kernels for 64 and 128; a
// narrower head runs in the next of the two, its missing columns read as zeros by TMA and never stored): TMA-staged
// tiles, tcgen05 MMAs accumulating in tensor memory, probabilities rebuilt from the saved
// log-sum-exp. Two separate passes, as in the kernels these replace (limn/cuda_emit.py:968-1083):
// every dQ row and every dK/dV row has one owning CTA and is accumulated in a fixed order,
// so there are no atomics and two runs give the same bits.
//
// sdpa_bwd_q: a work item owns 128 query rows (Q and dO tiles stay in shared memory) and streams
// key tiles j of 128 keys:
//     S  = Q K_j^T            (both K-major)            -> tensor memory, fp32
//     dP = dO V_j^T           (both K-major)            -> tensor memory, fp32
//     dS = exp2(S*c - L) * (dP - delta)  by 256 threads -> tensor memory, 16-bit, in columns of its own
//     dQ += dS K_j            (A from tensor memory, B = the same K_j tile read MN-major)
// sdpa_bwd_kv: a work item owns 128 keys (K and V tiles stay) and streams query tiles i:
//     S^T  = K Q_i^T, dP^T = V dO_i^T                   -> tensor memory (keys on the lanes)
//     P^T, dS^T as above, per-query L and delta read from shared memory
//     dV += P^T dO_i, dK += dS^T Q_i   (A from tensor memory, B = the streamed tiles MN-major)
// Two schedules (templates kEarly / kSeq, see the kernel): where tensor memory has room for S, dP and the
// 16-bit operands side by side (the dQ pass, and the dK/dV pass at head dim 64) the next tile's scores are
// issued as soon as this tile's are in registers; in the dK/dV pass at head dim 128 S^T and dP^T take turns in
// one region instead. Every MMA is full width (N = 128 or D). A key mask (hidden key = -inf score) is served by both.
// The scale is applied once to dQ and dK when they are written (oracle: limn/sdpa.py:157-170,
// :190-203, where ds carries the scale per element; the products are the same up to rounding).
//
// The grid is one CTA per SM; a CTA fetches work items (one owned tile each, longest streams first) from a
// counter until none is left, so the next item's tiles are loading, and its first scores computed, while the
// current item's accumulators are written out.
//
// Warp roles (10 working warps): 0-3 and 4-7 are two groups of 128 threads, thread r of each owning
// lane r (a query row, or a key row) and each group taking 64 of a tile's 128 columns;
// warp 8 is the TMA producer, warp 9 issues MMAs and owns tensor memory.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <cstdlib>

#include "common.h"
#include "sm100_ptx.cuh"
#include "tensor_map.h"

namespace limn_b200 {
namespace {

using namespace ptx;

constexpr int kTile = 128;
// Ten warps work; the CTA is launched with twelve because the compiler spills less in the elementwise loop at
// this block size (measured: 1 to 2 % faster). Warps 10 and 11 go straight to the final barrier.
constexpr int kThreads = 384;
#ifndef LIMN_BWD_KV_THREADS
#define LIMN_BWD_KV_THREADS 352
#endif
// The dK/dV pass never uses warps 10 and 11 (the dQ pass does, when it computes the row statistics itself), and
// its elementwise loop comes out of the compiler a little better with one spare warp than with two (1 % at head dim
// 64, nothing at 128; the dQ pass is 2 to 4 % slower that way and keeps its twelve).
template <bool kKV>
constexpr int bwd_threads() {
  return kKV ? LIMN_BWD_KV_THREADS : kThreads;
}
constexpr int kProducerWarp = 8;
constexpr int kMmaWarp = 9;
constexpr uint32_t kTmemCols = 512;
constexpr float kLog2e = 1.4426950408889634f;
// Early schedule: of every 8 pairs of scores, how many take exp2 as a cubic on the FMA pipe instead of on the
// special-function unit. Measured on B200 with the work-fetching kernels: 1 or 2 of 8 lose 3 to 5 % in the dQ
// pass and 7 % or more in the dK/dV pass at head dim 64, so the default is none.
#ifndef LIMN_BWD_POLY_PAIRS
#define LIMN_BWD_POLY_PAIRS 0
#endif
constexpr int kPolyPairsOf8 = LIMN_BWD_POLY_PAIRS;

template <int D, bool kKV, bool kMask>
struct BwdLayout {
  static constexpr int kTileBytes = kTile * D * 2;
  static constexpr int kAtomBytes = kTile * 128;
  // ring depths of the two streamed tiles. In the dQ pass at head dim 128 the V tile is only read by the
  // scores and leaves early, so two slots do for it and K gets the third that shared memory has room for.
  static constexpr int kStagesA = D == 128 ? (kKV ? 2 : 3) : 3;
  static constexpr int kStagesB = D == 128 ? 2 : 3;
  static constexpr int kHeldOff = 0;                               // two resident tiles
  static constexpr int kStreamAOff = 2 * kTileBytes;               // ring of the first streamed tile (K, or Q)
  static constexpr int kStreamBOff = kStreamAOff + kStagesA * kTileBytes;  // ring of the second (V, or dO)
  // The dK/dV pass at head dim 64 (where shared memory has the room): the epilogue leaves dV and dK here as blocks of
  // 128 rows x 128 B in the swizzled layout and TMA stores them, instead of every thread storing its own row in
  // 16-byte pieces (32 transactions per instruction for the load/store unit: 2 000 clocks per work item). Measured:
  // 13 % off the pass at S = 256, 2 % at S = 2048. In the dQ pass, where a thread stores half a row, the hand-overs
  // cost as much as they save (+2 % at S = 2048), so it keeps storing from registers.
  static constexpr bool kTileStore = D == 64 && kKV;
  static constexpr int kStoreOff = kStreamBOff + kStagesB * kTileBytes;
  static constexpr int kStatOff = kStoreOff + (kTileStore ? (kKV ? 2 : 1) * kAtomBytes : 0);
  static constexpr int kBarOff = kStatOff + (kKV ? 8 * 2 * 2 * 64 * 4 : 0);  // dK/dV pass, per warp [2 buffers][128 floats]: statistics of the streamed queries
  static constexpr int kBytes = kBarOff + 512 + 1024;
  static_assert(kBytes <= 227 * 1024, "shared memory per CTA");
  // tensor-memory columns
  static constexpr int kSCol = 0;      // S (or S^T); P^T overlays it as 16-bit
  static constexpr int kPCol = 128;    // dP (or dP^T); dS overlays it as 16-bit
  static constexpr int kAcc0 = 256;    // dQ, or dV
  static constexpr int kAcc1 = 256 + D;  // dK
  static constexpr int kDsCol = 448;     // early schedule: dS (or dS^T) as 16-bit, 64 columns
  static constexpr int kPtCol = 384;     // early schedule, dK/dV pass at head dim 64: P^T as 16-bit, 64 columns
  static constexpr int kSeqPtCol = 128;  // sequential schedule: P^T, 64 columns (S^T and dP^T share columns 0-127)
  static constexpr int kSeqDsCol = 192;  // sequential schedule: dS^T, 64 columns
};

template <int D, bool kKV, bool kMask>
struct BwdBars {
  static constexpr int kSA = BwdLayout<D, kKV, kMask>::kStagesA, kSB = BwdLayout<D, kKV, kMask>::kStagesB;
  static constexpr int held_full = 0;
  static constexpr int a_full = 1;                // + slot
  static constexpr int a_empty = a_full + kSA;
  static constexpr int b_full = a_empty + kSA;
  static constexpr int b_empty = b_full + kSB;
  static constexpr int s_full = b_empty + kSB;    // + half: that half's columns of S and dP are ready
  static constexpr int ds_full = s_full + 2;      // + half: its 16-bit operands are written (128 arrivals)
  static constexpr int extra = ds_full + 2;       // + 0/1, sequential schedule: S^T / dP^T are in registers (256 arrivals)
  static constexpr int acc_full = extra + 2;
  static constexpr int acc_free = acc_full + 1;     // the epilogue has read the accumulators (256 arrivals)
  static constexpr int held_empty = acc_free + 1;   // the item's last scores are computed: the resident tiles may be replaced
  static constexpr int work_full = held_empty + 1;  // + slot: the producer has fetched a work item
  static constexpr int work_empty = work_full + 2;  // + slot: every consumer has read it
  static constexpr int delta_full = work_empty + 2;   // + slot, fused dQ pass: the item's row statistics are in shared memory (64 arrivals)
  static constexpr int delta_empty = delta_full + 2;  // + slot: the elementwise threads have taken them (256 arrivals)
  static constexpr int store_full = delta_empty + 2;  // tile-store epilogue: every row of the staging blocks is written (256 arrivals)
  static constexpr int store_free = store_full + 1;   // the tile stores before have read the blocks
  static constexpr int count = store_free + 1;
};

// Build-time diagnostic (-DLIMN_TRACE): one CTA records clock64() at each step of its pipeline into a
// buffer named by the LIMN_TRACE_PTR environment variable. Compiled out of the shipped library.
#ifdef LIMN_TRACE
#define TRACE_EVENT(code) do { if (blockIdx.x == 7 && lane == 0 && trace_n < 250) { prm.trace[warp * 512 + 2 * trace_n] = clock64(); prm.trace[warp * 512 + 2 * trace_n + 1] = (code); ++trace_n; } } while (0)
#else
#define TRACE_EVENT(code) do {} while (0)
#endif

struct BwdParams {
  long long bh;
#ifdef LIMN_TRACE
  long long* trace;
#endif
  const unsigned short* mask;  // (bh, t_k) key flags in the storage dtype, 0 hides a key; null without a mask
  const float* lse;
  const float* delta;
  // dQ pass with the row statistic computed on the way (fused entry point): the forward's O and dO as plain
  // pointers, and where to leave delta for the dK/dV pass. Null otherwise: delta is then an input.
  const void* o_rows;
  const void* do_rows;
  float* delta_out;
  void* out0;   // dQ, or dK
  void* out1;   // dV
  unsigned* status;
  unsigned* schedule;  // [0] next work item, [1] CTAs that have finished; both zero between launches
  int group;           // problems per scheduling group (see cta_work)
  int heads;           // problem p is (batch p / heads, head p % heads) in the tensor maps and in the outputs
  Strides out_strides; // of dQ (dQ pass) or of dK (dK/dV pass), in elements
  Strides out1_strides;  // of dV
  Strides o_strides, do_strides;  // fused dQ pass: of the rows of O and dO the row statistic is computed from
  unsigned items;      // work items: bh * (tiles of 128 rows a problem's owner side has)
  int t_q, t_k;
  int width;           // columns of Q, K, dQ, dK as they lie in memory (<= D): TMA zero-fills the rest, stores skip it
  int width_v;         // the same of V, dO, O, dV
  int q_tiles, kv_tiles;
  float scale;
};

// barrier among the 128 threads of one group (ids 1 and 2; 0 is __syncthreads)
__device__ __forceinline__ void group_barrier(int group) { asm volatile("bar.sync %0, 128;" ::"r"(group + 1) : "memory"); }

// One accumulator row slice (32 fp32 columns) scaled, rounded and written as 64 bytes, or as many 16-byte pieces
// of them as the row has columns left.
template <bool kFp16>
__device__ __forceinline__ void store_row32(void* base, long long elem_offset, const uint32_t (&acc)[32], float mul, int cols_left) {
  uint4* dst = reinterpret_cast<uint4*>(static_cast<unsigned char*>(base) + elem_offset * 2);
#pragma unroll
  for (int v4 = 0; v4 < 4; ++v4) {
    uint32_t w[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float a = __uint_as_float(acc[v4 * 8 + 2 * i]) * mul;
      const float b = __uint_as_float(acc[v4 * 8 + 2 * i + 1]) * mul;
      w[i] = kFp16 ? pack_f16(a, b) : pack_bf16(a, b);
    }
    if (8 * v4 < cols_left) dst[v4] = make_uint4(w[0], w[1], w[2], w[3]);
  }
}

// sum_d a[d] * b[d] over one row of `pieces` * 8 <= D 16-bit elements each, in fp32 (four partial sums): the delta
// of one query row from its O and dO rows (limn/tensor.py:705-706).
template <int D, bool kFp16>
__device__ __forceinline__ float row_dot(const void* a_row, const void* b_row, int pieces) {
  const uint4* a = static_cast<const uint4*>(a_row);
  const uint4* b = static_cast<const uint4*>(b_row);
  // every load is issued before the first sum (a loop that may leave early would take them one at a time, and the
  // statistics would come late: 10 to 16 % on the whole pass): a row narrower than D reads its last piece again
  // and drops the product
  uint4 xv[D / 8], yv[D / 8];
#pragma unroll
  for (int i = 0; i < D / 8; ++i) {
    const int at = i < pieces ? i : pieces - 1;
    xv[i] = a[at], yv[i] = b[at];
  }
  float acc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
  for (int i = 0; i < D / 8; ++i) {
    const bool real = i < pieces;
    const uint4 x = xv[i], y = yv[i];
    const uint32_t xs[4] = {x.x, x.y, x.z, x.w}, ys[4] = {real ? y.x : 0u, real ? y.y : 0u, real ? y.z : 0u, real ? y.w : 0u};
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      float x0, x1, y0, y1;
      if (kFp16) {
        const float2 fx = __half22float2(*reinterpret_cast<const __half2*>(&xs[w])), fy = __half22float2(*reinterpret_cast<const __half2*>(&ys[w]));
        x0 = fx.x, x1 = fx.y, y0 = fy.x, y1 = fy.y;
      } else {
        x0 = __uint_as_float(xs[w] << 16), x1 = __uint_as_float(xs[w] & 0xffff0000u);
        y0 = __uint_as_float(ys[w] << 16), y1 = __uint_as_float(ys[w] & 0xffff0000u);
      }
      acc[w] = fmaf(x0, y0, acc[w]);
      acc[w] = fmaf(x1, y1, acc[w]);
    }
  }
  return (acc[0] + acc[1]) + (acc[2] + acc[3]);
}

// kKV = false: sdpa_bwd_q (CTA owns query rows, streams K/V). kKV = true: sdpa_bwd_kv.
// Exactly one of kEarly and kSeq is set; they pick the schedule. kEarly: S and dP have their own 128 columns
// each and the 16-bit operands columns of their own too, so the next tile's scores are issued as soon as this
// tile's have been read into registers and run beside the elementwise stage; it needs 64 (dQ pass) or 128
// (dK/dV pass) columns beyond scores and accumulators, which the dK/dV pass has only at head dim 64. kSeq (the dK/dV pass at head dim 128, where all 512 columns are spoken for):
// S^T and dP^T take turns in one 128-column region, S^T first, dP^T as soon as S^T is in registers, so that
// 128 columns are left for the operands and every MMA is full width.
template <int D, bool kCausal, bool kFp16, bool kKV, bool kEarly, bool kSeq, bool kMask>
__global__ void __launch_bounds__((bwd_threads<kKV>()), 1)
sdpa_bwd_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                const __grid_constant__ CUtensorMap map_v, const __grid_constant__ CUtensorMap map_do,
                const __grid_constant__ CUtensorMap map_out0, const __grid_constant__ CUtensorMap map_out1, const BwdParams prm) {
  using L = BwdLayout<D, kKV, kMask>;
  using B = BwdBars<D, kKV, kMask>;
  extern __shared__ unsigned char smem_unaligned[];
  __shared__ uint32_t tmem_slot;
  __shared__ uint32_t abort_flag;
  __shared__ unsigned work_ring[2];
  // dK/dV pass: the ring's items as the producer decoded them, so that the divisions are done once and off the
  // consumers' path (650 clocks per item there; measured 6 % off the pass at S = 2048). The dQ pass decodes in every
  // role: with the fields coming from shared memory it measured 2 to 4 % slower.
  __shared__ int work_items[2][8];
  __shared__ float delta_ring[2][kTile];  // fused dQ pass: delta of the item's 128 query rows, two items deep

  const uint32_t base = (smem_addr(smem_unaligned) + 1023u) & ~1023u;
  unsigned char* base_ptr = smem_unaligned + (base - smem_addr(smem_unaligned));
  float* stat = reinterpret_cast<float*>(base_ptr + L::kStatOff);
  const uint32_t bars = base + L::kBarOff;
  auto bar = [&](int i) { return bars + 8u * i; };

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  // ---- a work item: the tile of 128 rows it owns and the range of tiles streamed past it ----
  const int own_tiles = kKV ? prm.kv_tiles : prm.q_tiles;
  struct Item {
    int problem;
    int head, batch;  // the problem's coordinates in the operands
    int own0;    // first owned row
    int first;   // first streamed tile
    int count;   // streamed tiles
  };
  auto decode = [&](unsigned index) {
    Item item;
    int slot;
    cta_work(static_cast<int>(index), own_tiles, prm.bh, prm.group, item.problem, slot);
    item.batch = item.problem / prm.heads;
    item.head = item.problem - item.batch * prm.heads;
    // longest streams first: under causal the last query tile sees every key tile, the first key tile every query tile
    const int own = (kCausal && !kKV) ? own_tiles - 1 - slot : slot;
    item.own0 = own * kTile;
    if (kKV) {
      item.first = kCausal ? own : 0;
      item.count = prm.q_tiles - item.first;
    } else {
      item.first = 0;
      item.count = kCausal ? min(prm.kv_tiles, own + 1) : prm.kv_tiles;
    }
    return item;
  };

  if (threadIdx.x == 0) {
    for (int i = 0; i < B::count; ++i) {
      uint32_t arrivals = 1u;
      if (kSeq) {
        // s_full + 0/1: S^T / dP^T ready; extra + 0/1: read into registers; ds_full: operands stored;
        // ds_full + 1: products done (one commit)
        if (i == B::extra || i == B::extra + 1 || i == B::ds_full) arrivals = 256u;
      } else if (kEarly) {
        // s_full + 1 doubles as "scores read into registers", ds_full + 1 as "products done" (one commit)
        if (i == B::s_full + 1 || i == B::ds_full) arrivals = 256u;
      }
      if (i == B::acc_free || i == B::store_full) arrivals = 256u;
      // the MMA warp and the eight elementwise warps, and in the fused dQ pass the two warps that compute delta
      if (i == B::work_empty || i == B::work_empty + 1) arrivals = (!kKV && prm.o_rows != nullptr) ? 11u : 9u;
      if (i == B::delta_full || i == B::delta_full + 1) arrivals = 64u;    // every thread of the two warps that wrote them
      if (i == B::delta_empty || i == B::delta_empty + 1) arrivals = 256u;  // every elementwise thread, having read its own
      mbar_init(bar(i), arrivals);
    }
    mbar_init_fence();
  }
  // up to here nothing has touched global memory, so all of it may run under the tail of the kernel before this one
  grid_dependency_wait();
  grid_launch_dependents();
  if (threadIdx.x == 0) abort_flag = *reinterpret_cast<volatile unsigned*>(prm.status) != kStatusOk;
  __syncthreads();
  if (warp == kMmaWarp && !abort_flag) {
    tmem_alloc(smem_addr(&tmem_slot), kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem = tmem_slot;

  // resident tiles: (Q, dO) for the dQ pass, (K, V) for the dK/dV pass; streamed: the other pair
  const CUtensorMap* held_a = kKV ? &map_k : &map_q;
  const CUtensorMap* held_b = kKV ? &map_v : &map_do;
  const CUtensorMap* stream_a = kKV ? &map_q : &map_k;
  const CUtensorMap* stream_b = kKV ? &map_do : &map_v;
  const uint32_t held_a_smem = base + L::kHeldOff, held_b_smem = held_a_smem + L::kTileBytes;
  // everything about the rings is keyed by the streamed tile's ordinal `it`
  auto stream_a_smem = [&](int it) { return base + L::kStreamAOff + (it % L::kStagesA) * L::kTileBytes; };
  auto stream_b_smem = [&](int it) { return base + L::kStreamBOff + (it % L::kStagesB) * L::kTileBytes; };
  auto a_full = [&](int it) { return bar(B::a_full + it % L::kStagesA); };
  auto a_empty = [&](int it) { return bar(B::a_empty + it % L::kStagesA); };
  auto b_full = [&](int it) { return bar(B::b_full + it % L::kStagesB); };
  auto b_empty = [&](int it) { return bar(B::b_empty + it % L::kStagesB); };
  auto a_wrap = [&](int it) { return static_cast<uint32_t>((it / L::kStagesA) & 1); };
  auto b_wrap = [&](int it) { return static_cast<uint32_t>((it / L::kStagesB) & 1); };

  bool ok = !abort_flag;  // an earlier kernel on this device gave up: take no work, only leave the counters as found
#ifdef LIMN_TRACE
  int trace_n = 0;
#endif
  TRACE_EVENT(0);

  // The grid is one CTA per SM. The producer fetches work items from a counter and passes them to the other
  // warps through a two-entry ring, so the next item's tiles are on their way while the current item is still
  // being computed. Every role walks the same items in the same order; `done` counts the streamed tiles of
  // the items before the current one, and rings and per-tile barrier phases are keyed by done + it.
  auto next_item = [&](unsigned n_item, unsigned& index) {
    const unsigned ring = n_item & 1u;
    if (!mbar_wait(bar(B::work_full + ring), (n_item >> 1) & 1u, prm.status, 0x1400u | ring)) return false;
    index = *reinterpret_cast<volatile unsigned*>(&work_ring[ring]);
    return true;
  };
  // dK/dV pass: the same, with the item as the producer decoded it (read before the caller arrives on work_empty:
  // the slot is the producer's again after that)
  auto next_decoded = [&](unsigned n_item, unsigned& index, Item& item) {
    const unsigned ring = n_item & 1u;
    if (!mbar_wait(bar(B::work_full + ring), (n_item >> 1) & 1u, prm.status, 0x1400u | ring)) return false;
    index = *reinterpret_cast<volatile unsigned*>(&work_ring[ring]);
    const volatile int* f = work_items[ring];
    item.problem = f[0], item.head = f[1], item.batch = f[2], item.own0 = f[3], item.first = f[4], item.count = f[5];
    return true;
  };

  if (warp == kProducerWarp) {
    // ================= TMA producer, work fetcher =================
    if (lane == 0 && ok) {
      tma_prefetch_descriptor(held_a);
      tma_prefetch_descriptor(held_b);
      tma_prefetch_descriptor(stream_a);
      tma_prefetch_descriptor(stream_b);
      int done = 0;
      for (unsigned n_item = 0; ok; ++n_item) {
        const unsigned ring = n_item & 1u;
        ok = mbar_wait(bar(B::work_empty + ring), ((n_item >> 1) & 1u) ^ 1u, prm.status, 0x1120u | ring);
        if (!ok) break;
        // a CTA's first item is its own number (no round trip to the counter on the way to the first load); the
        // counter hands out what lies beyond the grid
        const unsigned index = n_item == 0 ? blockIdx.x : gridDim.x + atomicAdd(prm.schedule, 1u);
        Item item = {0, 0, 0, 0, 0, 0};
        if (index < prm.items) item = decode(index);
        if constexpr (kKV) {
          volatile int* f = work_items[ring];
          f[0] = item.problem, f[1] = item.head, f[2] = item.batch, f[3] = item.own0, f[4] = item.first, f[5] = item.count;
        }
        *reinterpret_cast<volatile unsigned*>(&work_ring[ring]) = index;
        mbar_arrive(bar(B::work_full + ring));
        if (index >= prm.items) break;
        ok = mbar_wait(bar(B::held_empty), (n_item & 1u) ^ 1u, prm.status, 0x1130u);
        if (!ok) break;
        mbar_expect_tx(bar(B::held_full), 2 * L::kTileBytes);
#pragma unroll
        for (int a = 0; a < D / 64; ++a) {
          tma_load_4d(held_a_smem + a * L::kAtomBytes, held_a, bar(B::held_full), a * 64, item.own0, item.head, item.batch);
          tma_load_4d(held_b_smem + a * L::kAtomBytes, held_b, bar(B::held_full), a * 64, item.own0, item.head, item.batch);
        }
        for (int it = 0; it < item.count; ++it) {
          const int g = done + it;
          const int row0 = (item.first + it) * kTile;
          ok = mbar_wait(a_empty(g), a_wrap(g) ^ 1u, prm.status, 0x1100u);
          if (!ok) break;
          mbar_expect_tx(a_full(g), L::kTileBytes);
#pragma unroll
          for (int a = 0; a < D / 64; ++a)
            tma_load_4d(stream_a_smem(g) + a * L::kAtomBytes, stream_a, a_full(g), a * 64, row0, item.head, item.batch);
          ok = mbar_wait(b_empty(g), b_wrap(g) ^ 1u, prm.status, 0x1110u);
          if (!ok) break;
          mbar_expect_tx(b_full(g), L::kTileBytes);
#pragma unroll
          for (int a = 0; a < D / 64; ++a)
            tma_load_4d(stream_b_smem(g) + a * L::kAtomBytes, stream_b, b_full(g), a * 64, row0, item.head, item.batch);
        }
        done += item.count;
      }
    }
  } else if (warp == kMmaWarp) {
    // ================= MMA issuer =================
    if (lane == 0 && ok) {
      constexpr uint32_t idesc_acc = mma_idesc(kTile, D, kFp16, false, true);
      int done = 0;
      if constexpr (kSeq) {
        constexpr uint32_t idesc_full = mma_idesc(kTile, kTile, kFp16, false, false);
        constexpr uint32_t kAtom16 = L::kAtomBytes >> 4;
        // C[128 x 128] = A B^T over the head dim into the shared score columns
        auto issue_score = [&](uint32_t a_tile, uint32_t b_tile, int which) {
          const uint32_t a0 = desc_lo(a_tile, 0), b0 = desc_lo(b_tile, 0);
          mma_ss_lo<false>(tmem + L::kSCol, a0, b0, idesc_full);
#pragma unroll
          for (int kk = 1; kk < D / 16; ++kk) {
            const uint32_t off = (kk / 4) * kAtom16 + (kk % 4) * 2;
            mma_ss_lo<true>(tmem + L::kSCol, a0 + off, b0 + off, idesc_full);
          }
          mma_commit(bar(B::s_full + which));
        };
        auto issue_acc_full = [&](uint32_t c_col, uint32_t a_col, uint32_t b_tile, bool fresh) {
          const uint32_t b_lo = desc_lo(b_tile, L::kAtomBytes);
#pragma unroll
          for (int kk = 0; kk < kTile / 16; ++kk)
            mma_ts_lo(tmem + c_col, tmem + a_col + kk * 8, b_lo + kk * (16 * 128 / 16), idesc_acc, (kk > 0 || !fresh) ? 1u : 0u);
        };
        auto wait_tile = [&](int it) {
          bool got = mbar_wait(a_full(it), a_wrap(it), prm.status, 0x1210u);
          if (got) got = mbar_wait(b_full(it), b_wrap(it), prm.status, 0x1211u);
          return got;
        };
        for (unsigned n_item = 0; ok; ++n_item) {
          unsigned index;
          int count = 0;
          if constexpr (kKV) {
            Item taken;
            ok = next_decoded(n_item, index, taken);
            count = taken.count;
          } else {
            ok = next_item(n_item, index);
          }
          if (!ok) break;
          mbar_arrive(bar(B::work_empty + (n_item & 1u)));
          if (index >= prm.items) break;
          if constexpr (!kKV) count = decode(index).count;
          ok = mbar_wait(bar(B::held_full), n_item & 1u, prm.status, 0x1200u);
          if (ok) ok = wait_tile(done);
          if (!ok) break;
          tc_fence_after_sync();
          issue_score(held_a_smem, stream_a_smem(done), 0);  // S^T = K Q_0^T (the previous item's last dP^T has been read)
          for (int it = 0; it < count && ok; ++it) {
            const int g = done + it;
            // dP^T takes the score columns as soon as S^T has been read out of them
            ok = mbar_wait(bar(B::extra + 0), g & 1, prm.status, 0x1260u);
            if (!ok) break;
            tc_fence_after_sync();
            issue_score(held_b_smem, stream_b_smem(g), 1);  // dP^T = V dO_i^T
            if (it + 1 == count) mma_commit(bar(B::held_empty));  // K and V have been read for the last time
            // and the next tile's S^T as soon as dP^T has been read
            ok = mbar_wait(bar(B::extra + 1), g & 1, prm.status, 0x1261u);
            if (!ok) break;
            if (it + 1 < count) {
              ok = wait_tile(g + 1);
              if (!ok) break;
              tc_fence_after_sync();
              issue_score(held_a_smem, stream_a_smem(g + 1), 0);
            }
            ok = mbar_wait(bar(B::ds_full), g & 1, prm.status, 0x1220u);
            // the item's first products overwrite the accumulators: the previous item's epilogue must have read them
            if (ok && it == 0) ok = mbar_wait(bar(B::acc_free), (n_item & 1u) ^ 1u, prm.status, 0x1270u);
            if (!ok) break;
            tc_fence_after_sync();
            issue_acc_full(L::kAcc0, L::kSeqPtCol, stream_b_smem(g), it == 0);  // dV += P^T dO_i
            issue_acc_full(L::kAcc1, L::kSeqDsCol, stream_a_smem(g), it == 0);  // dK += dS^T Q_i
            mma_commit(bar(B::ds_full + 1));  // products done: the operand columns may be rewritten
            mma_commit(a_empty(g));
            mma_commit(b_empty(g));
          }
          if (!ok) break;
          mma_commit(bar(B::acc_full));
          done += count;
        }
      } else if constexpr (kEarly) {
        constexpr uint32_t idesc_full = mma_idesc(kTile, kTile, kFp16, false, false);
        constexpr uint32_t kAtom16 = L::kAtomBytes >> 4;
        // S and dP of the whole streamed tile: C[128 x 128] = A B^T over the head dim
        auto issue_scores_full = [&](int stage) {
          const uint32_t a0 = desc_lo(held_a_smem, 0), b0 = desc_lo(stream_a_smem(stage), 0);
          const uint32_t a1 = desc_lo(held_b_smem, 0), b1 = desc_lo(stream_b_smem(stage), 0);
          mma_ss_lo<false>(tmem + L::kSCol, a0, b0, idesc_full);
#pragma unroll
          for (int kk = 1; kk < D / 16; ++kk) {
            const uint32_t off = (kk / 4) * kAtom16 + (kk % 4) * 2;
            mma_ss_lo<true>(tmem + L::kSCol, a0 + off, b0 + off, idesc_full);
          }
          mma_ss_lo<false>(tmem + L::kPCol, a1, b1, idesc_full);
#pragma unroll
          for (int kk = 1; kk < D / 16; ++kk) {
            const uint32_t off = (kk / 4) * kAtom16 + (kk % 4) * 2;
            mma_ss_lo<true>(tmem + L::kPCol, a1 + off, b1 + off, idesc_full);
          }
          mma_commit(bar(B::s_full));
        };
        // C[128 x D] += A B over all 128 rows of a streamed tile, A 16-bit in its own 64 columns
        auto issue_acc_full = [&](uint32_t c_col, uint32_t a_col, uint32_t b_tile, bool fresh) {
          const uint32_t b_lo = desc_lo(b_tile, L::kAtomBytes);
#pragma unroll
          for (int kk = 0; kk < kTile / 16; ++kk)
            mma_ts_lo(tmem + c_col, tmem + a_col + kk * 8, b_lo + kk * (16 * 128 / 16), idesc_acc, (kk > 0 || !fresh) ? 1u : 0u);
        };
        auto wait_tile = [&](int it) {
          bool got = mbar_wait(a_full(it), a_wrap(it), prm.status, 0x1210u);
          if (got) got = mbar_wait(b_full(it), b_wrap(it), prm.status, 0x1211u);
          return got;
        };
        for (unsigned n_item = 0; ok; ++n_item) {
          unsigned index;
          int count = 0;
          if constexpr (kKV) {
            Item taken;
            ok = next_decoded(n_item, index, taken);
            count = taken.count;
          } else {
            ok = next_item(n_item, index);
          }
          if (!ok) break;
          mbar_arrive(bar(B::work_empty + (n_item & 1u)));
          if (index >= prm.items) break;
          if constexpr (!kKV) count = decode(index).count;
          ok = mbar_wait(bar(B::held_full), n_item & 1u, prm.status, 0x1200u);
          // the previous item's last scores must be in registers before this item's first overwrite them
          if (ok && done > 0) ok = mbar_wait(bar(B::s_full + 1), (done - 1) & 1, prm.status, 0x1241u);
          if (ok) ok = wait_tile(done);
          if (!ok) break;
          tc_fence_after_sync();
          issue_scores_full(done);
          if (!kKV) mma_commit(b_empty(done));  // dQ pass: V is read by the scores only
          if (count == 1) mma_commit(bar(B::held_empty));
          for (int it = 0; it < count && ok; ++it) {
            const int g = done + it;
            if (it + 1 < count) {
              // the next tile's scores may overwrite this tile's once every thread holds them in registers
              ok = mbar_wait(bar(B::s_full + 1), g & 1, prm.status, 0x1240u);
              if (ok) ok = wait_tile(g + 1);
              if (!ok) break;
              tc_fence_after_sync();
              issue_scores_full(g + 1);
              if (!kKV) mma_commit(b_empty(g + 1));
              if (it + 2 == count) mma_commit(bar(B::held_empty));  // the resident tiles have been read for the last time
            }
            ok = mbar_wait(bar(B::ds_full), g & 1, prm.status, 0x1220u);
            // the item's first products overwrite the accumulators: the previous item's epilogue must have read them
            if (ok && it == 0) ok = mbar_wait(bar(B::acc_free), (n_item & 1u) ^ 1u, prm.status, 0x1270u);
            if (!ok) break;
            tc_fence_after_sync();
            if (kKV) {
              issue_acc_full(L::kAcc0, L::kPtCol, stream_b_smem(g), it == 0);  // dV += P^T dO_i
              issue_acc_full(L::kAcc1, L::kDsCol, stream_a_smem(g), it == 0);  // dK += dS^T Q_i
            } else {
              issue_acc_full(L::kAcc0, L::kDsCol, stream_a_smem(g), it == 0);  // dQ += dS K_j
            }
            mma_commit(bar(B::ds_full + 1));            // products done: the operand columns may be rewritten
            mma_commit(a_empty(g));
            if (kKV) mma_commit(b_empty(g));
          }
          if (!ok) break;
          mma_commit(bar(B::acc_full));
          done += count;
        }
      }
    }
  } else if (warp < kProducerWarp) {
    // ================= elementwise stage + epilogue: 2 groups x 128 threads =================
    const int group = warp >> 2;             // which 64 of a tile's 128 columns
    const int r = threadIdx.x & 127;         // lane of tensor memory: query row (dQ pass) or key row (dK/dV pass)
    const uint32_t lane_base = static_cast<uint32_t>((warp & 3) * 32) << 16;
    const uint32_t t_s = tmem + lane_base + L::kSCol;
    const uint32_t t_p = tmem + lane_base + L::kPCol;
    const float sl2 = prm.scale * kLog2e;
    const uint64_t sl2_2 = f2_pack(sl2, sl2);
    int done = 0;
    // The statistics an item needs before its first tile, raw as loaded: the own row's L and delta (dQ pass), or
    // L and delta of this lane's two columns of the first streamed tile (dK/dV pass). They are fetched when
    // the item becomes known, which is before the previous item's epilogue, so the loads' latency is hidden
    // behind it; nothing reads them until the item starts.
    struct Fetched { float l0, l1, d0, d1; };
    auto fetch_head = [&](const Item& of) {
      const long long sb = static_cast<long long>(of.problem) * prm.t_q;
      Fetched f = {0.f, 0.f, 0.f, 0.f};
      if (kKV) {
        const int q0 = min(of.first * kTile + group * 64 + lane, prm.t_q - 1), q1 = min(of.first * kTile + group * 64 + lane + 32, prm.t_q - 1);
        f.l0 = prm.lse[sb + q0], f.l1 = prm.lse[sb + q1];
        f.d0 = prm.delta[sb + q0], f.d1 = prm.delta[sb + q1];
      } else {
        const int row = min(of.own0 + r, prm.t_q - 1);
        f.l0 = prm.lse[sb + row];
        if (prm.o_rows == nullptr) f.d0 = prm.delta[sb + row];  // (the fused pass takes delta from shared memory when the item starts)
      }
      return f;
    };
    // the next item, if the producer has one: its index, and its first statistics on their way
    auto take_item = [&](unsigned n_item, unsigned& index, Item& item, Fetched& head) {
      index = prm.items;
      Item taken = {0, 0, 0, 0, 0, 0};
      if constexpr (kKV) {
        if (!__all_sync(0xffffffffu, next_decoded(n_item, index, taken))) return false;
      } else {
        if (!__all_sync(0xffffffffu, next_item(n_item, index))) return false;
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(B::work_empty + (n_item & 1u)));
      if (index < prm.items) {
        if constexpr (kKV) item = taken; else item = decode(index);
        head = fetch_head(item);
      }
      return true;
    };
    unsigned index = prm.items;
    Item item = {0, 0, 0, 0};
    Fetched head = {0.f, 0.f, 0.f, 0.f};
    if (ok) ok = take_item(0, index, item, head);
    for (unsigned n_item = 0; ok && index < prm.items; ++n_item) {
    const int problem = item.problem, own0 = item.own0, first = item.first, count = item.count;
    const long long stat_base = static_cast<long long>(problem) * prm.t_q;
    // statistics enter negated: x = s * c + (-L log2e), t = dP + (-delta). A row or column past t_q
    // gets -L = -inf, which makes its probability exactly 0.
    uint64_t row_neg_l2 = 0, row_neg_delta = 0;
    if (!kKV) {
      const bool in = own0 + r < prm.t_q;
      if (prm.o_rows != nullptr) {
        // the fused entry point: warps 10 and 11 computed the item's row statistics when the item was published
        const unsigned slot = n_item & 1u;
        ok = __all_sync(0xffffffffu, mbar_wait(bar(B::delta_full + slot), (n_item >> 1) & 1u, prm.status, 0x1340u | slot));
        if (!ok) break;
        head.d0 = *reinterpret_cast<volatile float*>(&delta_ring[slot][r]);
        mbar_arrive(bar(B::delta_empty + slot));
      }
      const float nl = in ? -head.l0 * kLog2e : -INFINITY;
      const float nd = in ? -head.d0 : 0.f;
      row_neg_l2 = f2_pack(nl, nl);
      row_neg_delta = f2_pack(nd, nd);
    }
    // dK/dV pass: the statistics of the streamed tile's queries. Every warp keeps its own copy of its group's
    // 64 columns in shared memory (-L log2e then -delta), each lane fetching two columns of each from global
    // memory one tile ahead of their use, so no warp ever waits for another here.
    // A warp issues in order, so nothing may depend on these loads until the next tile: the raw values are
    // parked in registers and negated, scaled and range-checked only when they are staged.
    auto fetch_stat = [&](int tile0) {
      Fetched f;
      const int q0 = min(tile0 + group * 64 + lane, prm.t_q - 1), q1 = min(tile0 + group * 64 + lane + 32, prm.t_q - 1);
      f.l0 = prm.lse[stat_base + q0], f.l1 = prm.lse[stat_base + q1];
      f.d0 = prm.delta[stat_base + q0], f.d1 = prm.delta[stat_base + q1];
      return f;
    };
    Fetched fetched = head;
    // Key mask: a hidden key's probabilities are exactly 0, which an additive -inf on its scores gives. In the
    // dK/dV pass the key is this thread's own row, one flag for the whole pass; in the dQ pass keys are the
    // columns, and each warp stages its group's 64 flags per streamed tile, fetched one tile ahead.
    auto key_bias = [&](int key) {
      const bool live = key < prm.t_k && (prm.mask[static_cast<long long>(problem) * prm.t_k + key] & 0x7fffu) != 0;
      return live ? 0.f : -INFINITY;
    };
    // (dQ pass: the flags stay as loaded until the next tile needs them. A warp issues in order, so turning them
    // into anything right after the load would stall it for the load's latency, every tile.)
    auto key_flag = [&](int key) -> unsigned {
      return key < prm.t_k ? prm.mask[static_cast<long long>(problem) * prm.t_k + key] : 0u;  // past the end: hidden
    };
    uint64_t row_bias2 = 0;
    unsigned col_flag0 = 1u, col_flag1 = 1u;
    if (kMask) {
      if (kKV) {
        const float b = key_bias(own0 + r);
        row_bias2 = f2_pack(b, b);
      } else {
        col_flag0 = key_flag(first * kTile + group * 64 + lane);
        col_flag1 = key_flag(first * kTile + group * 64 + lane + 32);
      }
    }
    for (int it = 0; it < count; ++it) {
      const int g = done + it;                  // the tile's ordinal over all items: rings and barrier phases go by it
      const int other0 = (first + it) * kTile;  // first key (dQ pass) or first query (dK/dV pass) of the streamed tile
      // per warp: [2 buffers][-L log2e, -delta][64 columns]
      float* st = stat + (warp * 2 + (g & 1)) * (2 * 64);
      // dQ pass under a key mask: which of the group's 64 keys of this tile are hidden, as two words in registers
      // (a ballot over the flags each lane fetched a tile ahead); most tiles of a padded batch have none
      unsigned hidden_lo = 0u, hidden_hi = 0u;
      if (kMask && !kKV) {
        hidden_lo = __ballot_sync(0xffffffffu, (col_flag0 & 0x7fffu) == 0u);
        hidden_hi = __ballot_sync(0xffffffffu, (col_flag1 & 0x7fffu) == 0u);
        if (it + 1 < count) {
          col_flag0 = key_flag(other0 + kTile + group * 64 + lane);
          col_flag1 = key_flag(other0 + kTile + group * 64 + lane + 32);
        }
      }
      if (kKV) {
        const bool in0 = other0 + group * 64 + lane < prm.t_q, in1 = other0 + group * 64 + lane + 32 < prm.t_q;
        st[lane] = in0 ? -fetched.l0 * kLog2e : -INFINITY, st[lane + 32] = in1 ? -fetched.l1 * kLog2e : -INFINITY;
        TRACE_EVENT(8);
        st[64 + lane] = in0 ? -fetched.d0 : 0.f, st[96 + lane] = in1 ? -fetched.d1 : 0.f;
        __syncwarp();
        TRACE_EVENT(9);
        if (it + 1 < count) fetched = fetch_stat(other0 + kTile);
      }
      if constexpr (kSeq) {
        // S^T and dP^T arrive one after the other in the same columns; the probabilities wait in registers
        TRACE_EVENT(1);
        if (ok) ok = __all_sync(0xffffffffu, mbar_wait(bar(B::s_full + 0), g & 1, prm.status, 0x1300u | group));
        if (!ok) continue;
        TRACE_EVENT(2);
        tc_fence_after_sync();
        uint32_t s[2][32];
        tmem_ld32(t_s + group * 64, s[0]);
        tmem_ld32(t_s + group * 64 + 32, s[1]);
        tmem_ld_wait();
        tc_fence_before_sync();
        mbar_arrive(bar(B::extra + 0));  // dP^T may overwrite S^T
        TRACE_EVENT(3);
        if (kCausal && other0 == own0) {
#pragma unroll
          for (int c = 0; c < 2; ++c)
#pragma unroll
            for (int e = 0; e < 32; ++e)
              if (group * 64 + c * 32 + e < r) s[c][e] = 0xff800000u;  // query before key: probability exactly 0
        }
        uint32_t p_packed[32];
#pragma unroll
        for (int c = 0; c < 2; ++c)
#pragma unroll
          for (int e = 0; e < 32; e += 2) {
            const float2 a = *reinterpret_cast<const float2*>(st + c * 32 + e);
            uint64_t neg_l2 = f2_pack(a.x, a.y);
            if (kMask) neg_l2 = f2_add(neg_l2, row_bias2);
            float p0, p1;
            f2_unpack(f2_fma(f2_pack_bits(s[c][e], s[c][e + 1]), sl2_2, neg_l2), p0, p1);
            p0 = exp2_approx(p0), p1 = exp2_approx(p1);
            s[c][e] = __float_as_uint(p0), s[c][e + 1] = __float_as_uint(p1);  // kept for dS
            p_packed[c * 16 + (e >> 1)] = kFp16 ? pack_f16(p0, p1) : pack_bf16(p0, p1);
          }
        TRACE_EVENT(4);
        // the previous tile's products must have consumed the operand columns before they are rewritten
        if (g > 0) {
          ok = __all_sync(0xffffffffu, mbar_wait(bar(B::ds_full + 1), (g - 1) & 1, prm.status, 0x1320u | group));
          if (!ok) continue;
          tc_fence_after_sync();
        }
        tmem_st32(tmem + lane_base + L::kSeqPtCol + group * 32, p_packed);
        ok = __all_sync(0xffffffffu, mbar_wait(bar(B::s_full + 1), g & 1, prm.status, 0x1330u | group));
        if (!ok) continue;
        tc_fence_after_sync();
        uint32_t dp[2][32];
        tmem_ld32(t_s + group * 64, dp[0]);
        tmem_ld32(t_s + group * 64 + 32, dp[1]);
        tmem_ld_wait();
        tc_fence_before_sync();
        mbar_arrive(bar(B::extra + 1));  // the next tile's S^T may overwrite dP^T
        uint32_t ds_packed[32];
#pragma unroll
        for (int c = 0; c < 2; ++c)
#pragma unroll
          for (int e = 0; e < 32; e += 2) {
            const float2 b = *reinterpret_cast<const float2*>(st + 64 + c * 32 + e);
            float d0, d1;
            f2_unpack(f2_mul(f2_pack_bits(s[c][e], s[c][e + 1]), f2_add(f2_pack_bits(dp[c][e], dp[c][e + 1]), f2_pack(b.x, b.y))), d0, d1);
            ds_packed[c * 16 + (e >> 1)] = kFp16 ? pack_f16(d0, d1) : pack_bf16(d0, d1);
          }
        tmem_st32(tmem + lane_base + L::kSeqDsCol + group * 32, ds_packed);
        tmem_st_wait();
        TRACE_EVENT(5);
        tc_fence_before_sync();
        mbar_arrive(bar(B::ds_full));
        TRACE_EVENT(7);
      } else if constexpr (kEarly) {
        TRACE_EVENT(1);
        if (ok) ok = __all_sync(0xffffffffu, mbar_wait(bar(B::s_full), g & 1, prm.status, 0x1300u | group));
        if (!ok) continue;
        TRACE_EVENT(2);
        tc_fence_after_sync();
        // this group's 64 columns of S and dP, all into registers, so the tile's tensor memory can be reused
        uint32_t s[2][32], dp[2][32];
        tmem_ld32(t_s + group * 64, s[0]);
        tmem_ld32(t_s + group * 64 + 32, s[1]);
        tmem_ld32(t_p + group * 64, dp[0]);
        tmem_ld32(t_p + group * 64 + 32, dp[1]);
        tmem_ld_wait();
        tc_fence_before_sync();
        mbar_arrive(bar(B::s_full + 1));
        TRACE_EVENT(3);
        const bool diagonal = kCausal && other0 == own0;
        const bool ragged = !kKV && other0 + kTile > prm.t_k;
        const bool masked = kMask && !kKV && (hidden_lo | hidden_hi) != 0u;
        if (diagonal || ragged || masked) {
#pragma unroll
          for (int c = 0; c < 2; ++c)
#pragma unroll
            for (int e = 0; e < 32; ++e) {
              const int col = group * 64 + c * 32 + e;
              bool hidden = false;
              if (diagonal) hidden = kKV ? (col < r) : (col > r);   // a key index must not exceed the query index
              if (ragged) hidden = hidden || (other0 + col >= prm.t_k);
              if (kMask && !kKV) hidden = hidden || (((c == 0 ? hidden_lo : hidden_hi) >> e) & 1u) != 0u;
              if (hidden) s[c][e] = 0xff800000u;  // -inf: the probability becomes exactly 0
            }
        }
        uint32_t p_packed[32], ds_packed[32];
#pragma unroll
        for (int c = 0; c < 2; ++c) {
#pragma unroll
          for (int e = 0; e < 32; e += 2) {
            uint64_t neg_l2, neg_delta;
            if (kKV) {
              const float2 a = *reinterpret_cast<const float2*>(st + c * 32 + e);
              const float2 b = *reinterpret_cast<const float2*>(st + 64 + c * 32 + e);
              neg_l2 = f2_pack(a.x, a.y);
              neg_delta = f2_pack(b.x, b.y);
            } else {
              neg_l2 = row_neg_l2;
              neg_delta = row_neg_delta;
            }
            if (kMask) {
              if (kKV) neg_l2 = f2_add(neg_l2, row_bias2);  // (the dQ pass has rewritten its hidden keys' scores above)
            }
            const uint64_t x2 = f2_fma(f2_pack_bits(s[c][e], s[c][e + 1]), sl2_2, neg_l2);
            float p0, p1;
            if (((e >> 1) & 7) < kPolyPairsOf8) {
              exp2_poly2(x2, p0, p1);  // on the FMA pipe, beside the special-function unit
            } else {
              f2_unpack(x2, p0, p1);
              p0 = exp2_approx(p0), p1 = exp2_approx(p1);
            }
            float d0, d1;
            f2_unpack(f2_mul(f2_pack(p0, p1), f2_add(f2_pack_bits(dp[c][e], dp[c][e + 1]), neg_delta)), d0, d1);
            if (kKV) p_packed[c * 16 + (e >> 1)] = kFp16 ? pack_f16(p0, p1) : pack_bf16(p0, p1);
            ds_packed[c * 16 + (e >> 1)] = kFp16 ? pack_f16(d0, d1) : pack_bf16(d0, d1);
          }
        }
        TRACE_EVENT(4);
        // the previous tile's products must have consumed the operand columns before they are rewritten
        if (g > 0) {
          ok = __all_sync(0xffffffffu, mbar_wait(bar(B::ds_full + 1), (g - 1) & 1, prm.status, 0x1320u | group));
          if (!ok) continue;
          tc_fence_after_sync();
        }
        if (kKV) tmem_st32(tmem + lane_base + L::kPtCol + group * 32, p_packed);
        tmem_st32(tmem + lane_base + L::kDsCol + group * 32, ds_packed);
        tmem_st_wait();
        TRACE_EVENT(5);
        tc_fence_before_sync();
        mbar_arrive(bar(B::ds_full));
      }
    }
    // learn the next item (the producer fetched it several tiles ago) and start its first loads before the epilogue
    unsigned upcoming = prm.items;
    Item upcoming_item = item;
    Fetched upcoming_head = head;
    if (ok) ok = take_item(n_item + 1, upcoming, upcoming_item, upcoming_head);
    if (ok) ok = __all_sync(0xffffffffu, mbar_wait(bar(B::acc_full), n_item & 1u, prm.status, 0x1310u));
    if (ok && L::kTileStore) {
      tc_fence_after_sync();
      // the stores of the item before have read the staging blocks: the thread that issued them says so
      const bool leader = threadIdx.x == 0;
      if (leader) {
        tma_store_wait_read();
        mbar_arrive(bar(B::store_free));
      }
      ok = __all_sync(0xffffffffu, mbar_wait(bar(B::store_free), n_item & 1u, prm.status, 0x1350u));
      if (ok) {
        // dK/dV pass: group 0 stages this key's dV row, group 1 its dK row, a block each; dQ pass: each group half
        // of this query's dQ row, in the one block
        const uint32_t block = base + L::kStoreOff + (kKV ? group * L::kAtomBytes : 0);
        const float mul = (kKV && group == 0) ? 1.f : prm.scale;
#pragma unroll
        for (int c = 0; c < (kKV ? 2 : 1); ++c) {
          const int col = kKV ? 32 * c : group * 32;
          uint32_t acc[32];
          tmem_ld32(tmem + lane_base + ((kKV && group == 1) ? L::kAcc1 : L::kAcc0) + col, acc);
          tmem_ld_wait();
#pragma unroll
          for (int v4 = 0; v4 < 4; ++v4) {
            uint32_t w[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              const float a = __uint_as_float(acc[v4 * 8 + 2 * i]) * mul;
              const float b = __uint_as_float(acc[v4 * 8 + 2 * i + 1]) * mul;
              w[i] = kFp16 ? pack_f16(a, b) : pack_bf16(a, b);
            }
            st_shared_v4(swizzled_piece(block, r, (col >> 3) + v4), w[0], w[1], w[2], w[3]);
          }
        }
        // the accumulators are in registers or staged: the next item's first products may overwrite them
        tc_fence_before_sync();
        mbar_arrive(bar(B::acc_free));
        fence_async_shared();
        mbar_arrive(bar(B::store_full));
        if (leader && mbar_wait(bar(B::store_full), n_item & 1u, prm.status, 0x1360u)) {
          tma_store_4d(&map_out0, base + L::kStoreOff + (kKV ? L::kAtomBytes : 0), 0, own0, item.head, item.batch);  // dQ, or dK
          if (kKV) tma_store_4d(&map_out1, base + L::kStoreOff, 0, own0, item.head, item.batch);                      // dV
          tma_store_commit();
        }
      }
    } else if (ok) {
      tc_fence_after_sync();
      const int row = own0 + r;
      if (kKV) {
        // group 0 writes this key's dV row, group 1 its dK row
        const bool in = row < prm.t_k;
        const Strides& mine = group == 0 ? prm.out1_strides : prm.out_strides;
        const long long out_at = item.batch * mine.batch + item.head * mine.head + row * mine.row;
        const uint32_t t_acc = tmem + lane_base + (group == 0 ? L::kAcc0 : L::kAcc1);
        void* dst = group == 0 ? prm.out1 : prm.out0;
        const float mul = group == 0 ? 1.f : prm.scale;
#pragma unroll
        for (int c = 0; c < D / 32; ++c) {
          uint32_t acc[32];
          tmem_ld32(t_acc + 32 * c, acc);
          tmem_ld_wait();
          if (in) store_row32<kFp16>(dst, out_at + 32 * c, acc, mul, (group == 0 ? prm.width_v : prm.width) - 32 * c);
        }
      } else {
        // each group writes half of this query's dQ row
        const bool in = row < prm.t_q;
        const long long out_at = item.batch * prm.out_strides.batch + item.head * prm.out_strides.head + row * prm.out_strides.row;
#pragma unroll
        for (int c = 0; c < D / 64; ++c) {
          const int col = group * (D / 2) + 32 * c;
          uint32_t acc[32];
          tmem_ld32(tmem + lane_base + L::kAcc0 + col, acc);
          tmem_ld_wait();
          if (in) store_row32<kFp16>(prm.out0, out_at + col, acc, prm.scale, prm.width - col);
        }
      }
      // the accumulators are in registers or stored: the next item's first products may overwrite them
      tc_fence_before_sync();
      mbar_arrive(bar(B::acc_free));
    }
    done += count;
    index = upcoming, item = upcoming_item, head = upcoming_head;
    }  // items
    // the last tile stores must have read their staging blocks before the CTA gives its shared memory back
    if (L::kTileStore && threadIdx.x == 0) tma_store_wait_read();
  }

  else if (!kKV && prm.o_rows != nullptr) {
    // ================= fused dQ pass: the row statistic delta = sum_d dO * O, by the two spare warps =================
    // They follow the producer's work ring like every other consumer and so learn of an item while the item
    // before it is still being computed: by the time the elementwise warps start on it, its 128 statistics lie in
    // shared memory (and in the caller's delta buffer, for the dK/dV pass). Thread j of the 64 takes rows j and j + 64.
    const int j = threadIdx.x - (kMmaWarp + 1) * 32;
    for (unsigned n_item = 0; ok; ++n_item) {
      unsigned index;
      ok = __all_sync(0xffffffffu, next_item(n_item, index));
      if (!ok) break;
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(B::work_empty + (n_item & 1u)));
      if (index >= prm.items) break;
      const Item item = decode(index);
      const unsigned slot = n_item & 1u;
      ok = __all_sync(0xffffffffu, mbar_wait(bar(B::delta_empty + slot), ((n_item >> 1) & 1u) ^ 1u, prm.status, 0x1500u | slot));
      if (!ok) break;
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        const int local = j + 64 * half;
        const int row = min(item.own0 + local, prm.t_q - 1);
        const long long o_at = (item.batch * prm.o_strides.batch + item.head * prm.o_strides.head + row * prm.o_strides.row) * 2;
        const long long do_at = (item.batch * prm.do_strides.batch + item.head * prm.do_strides.head + row * prm.do_strides.row) * 2;
        const float d = row_dot<D, kFp16>(static_cast<const unsigned char*>(prm.o_rows) + o_at, static_cast<const unsigned char*>(prm.do_rows) + do_at, prm.width_v >> 3);
        delta_ring[slot][local] = d;
        if (item.own0 + local < prm.t_q) prm.delta_out[static_cast<long long>(item.problem) * prm.t_q + row] = d;
      }
      mbar_arrive(bar(B::delta_full + slot));  // every writer arrives for itself: the arrival orders its writes before it
    }
  }

  // ---- teardown ----
  tc_fence_before_sync();
  __syncthreads();
  if (warp == kMmaWarp && !abort_flag) {
    if (*reinterpret_cast<volatile unsigned*>(prm.status) != kStatusOk) {
      for (int i = 0; i < 2000; ++i) __nanosleep(1000);  // let copies and MMAs still in flight land
    }
    tc_fence_after_sync();
    tmem_free(tmem, kTmemCols);
  }
  // the last CTA to leave puts the work counters back to zero for the next launch that is handed this pair
  if (threadIdx.x == 0 && atomicAdd(prm.schedule + 1, 1u) == gridDim.x - 1) {
    prm.schedule[0] = 0u;
    prm.schedule[1] = 0u;
    __threadfence();
  }
}

template <int D, bool kCausal, bool kFp16, bool kKV, bool kMask>
int launch_bwd(const Problem& p) {
  constexpr bool kEarly = !kKV || D == 64;  // the dK/dV pass at head dim 128 has no spare tensor-memory columns ...
  constexpr bool kSeq = !kEarly;            // ... so there S^T and dP^T share one region, one after the other
  using L = BwdLayout<D, kKV, kMask>;
  CUtensorMap map_q, map_k, map_v, map_do;
  const int heads = p.heads > 0 ? p.heads : static_cast<int>(p.bh), batch = static_cast<int>(p.bh / heads);
  if (int rc = make_tile_map(&map_q, p.q, kFp16, batch, heads, p.t_q, p.hd, kTile, operand_strides(p, kOpQ, heads, p.t_q, p.hd))) return rc;
  if (int rc = make_tile_map(&map_k, p.k, kFp16, batch, heads, p.t_k, p.hd, kTile, operand_strides(p, kOpK, heads, p.t_k, p.hd))) return rc;
  if (int rc = make_tile_map(&map_v, p.v, kFp16, batch, heads, p.t_k, p.hd_v, kTile, operand_strides(p, kOpV, heads, p.t_k, p.hd_v))) return rc;
  if (int rc = make_tile_map(&map_do, p.dout, kFp16, batch, heads, p.t_q, p.hd_v, kTile, operand_strides(p, kOpDout, heads, p.t_q, p.hd_v))) return rc;
  CUtensorMap map_out0 = map_q, map_out1 = map_q;  // only read by the kernels that store tiles
  if (L::kTileStore) {
    if (kKV) {
      if (int rc = make_tile_map(&map_out0, p.dk, kFp16, batch, heads, p.t_k, p.hd, kTile, operand_strides(p, kOpDk, heads, p.t_k, p.hd))) return rc;
      if (int rc = make_tile_map(&map_out1, p.dv, kFp16, batch, heads, p.t_k, p.hd_v, kTile, operand_strides(p, kOpDv, heads, p.t_k, p.hd_v))) return rc;
    } else {
      if (int rc = make_tile_map(&map_out0, p.dq, kFp16, batch, heads, p.t_q, p.hd, kTile, operand_strides(p, kOpDq, heads, p.t_q, p.hd))) return rc;
    }
  }
  BwdParams prm;
  prm.mask = static_cast<const unsigned short*>(p.mask);
  prm.lse = static_cast<const float*>(p.lse_in);
  prm.delta = static_cast<const float*>(p.delta);
  prm.o_rows = (!kKV && p.fuse_delta) ? p.out : nullptr;
  prm.do_rows = (!kKV && p.fuse_delta) ? p.dout : nullptr;
  prm.delta_out = (!kKV && p.fuse_delta) ? static_cast<float*>(const_cast<void*>(p.delta)) : nullptr;
  prm.out0 = kKV ? p.dk : p.dq;
  prm.out1 = kKV ? p.dv : nullptr;
  prm.heads = heads;
  prm.out_strides = kKV ? operand_strides(p, kOpDk, heads, p.t_k, p.hd) : operand_strides(p, kOpDq, heads, p.t_q, p.hd);
  prm.out1_strides = operand_strides(p, kOpDv, heads, p.t_k, p.hd_v);
  prm.o_strides = operand_strides(p, kOpOut, heads, p.t_q, p.hd_v);
  prm.do_strides = operand_strides(p, kOpDout, heads, p.t_q, p.hd_v);
  {
    const long long all = prm.out_strides.batch | prm.out_strides.head | prm.out_strides.row | prm.out1_strides.batch |
                          prm.out1_strides.head | prm.out1_strides.row | prm.o_strides.batch | prm.o_strides.head | prm.o_strides.row;
    if (all & 7) return fail(LIMN_B200_BAD_ARGUMENT, "sdpa backward: operand strides must be multiples of 8 elements");
    const uintptr_t bases = reinterpret_cast<uintptr_t>(prm.out0) | reinterpret_cast<uintptr_t>(prm.out1) | reinterpret_cast<uintptr_t>(prm.o_rows);
    if (bases & 15u) return fail(LIMN_B200_BAD_ARGUMENT, "sdpa backward: an output (or O) is not 16-byte aligned");
  }
  prm.status = p.status;
  if (prm.status == nullptr)
    if (int rc = status_word(&prm.status)) return rc;
  prm.bh = p.bh;
  prm.t_q = p.t_q, prm.t_k = p.t_k;
  prm.width = p.hd;
  prm.width_v = p.hd_v;
  prm.q_tiles = (p.t_q + kTile - 1) / kTile;
  prm.kv_tiles = (p.t_k + kTile - 1) / kTile;
#ifdef LIMN_TRACE
  const char* trace_ptr = getenv("LIMN_TRACE_PTR");
  if (trace_ptr == nullptr) return fail(LIMN_B200_BAD_ARGUMENT, "this is a -DLIMN_TRACE build: set LIMN_TRACE_PTR to the trace buffer's device address");
  prm.trace = reinterpret_cast<long long*>(strtoull(trace_ptr, nullptr, 16));
#endif
  prm.scale = static_cast<float>(p.scale);
  const long long items = p.bh * (kKV ? prm.kv_tiles : prm.q_tiles);
  if (items > 0x7fffffffLL) return fail(LIMN_B200_UNSUPPORTED, "sdpa backward: %lld work items exceed the counter", items);
  prm.items = static_cast<unsigned>(items);
  prm.schedule = p.schedule;
  if (prm.schedule == nullptr)
    if (int rc = schedule_words(&prm.schedule)) return rc;
  int sms = 0;
  if (int rc = sm_count(&sms)) return rc;
  prm.group = work_group(p, items, sms);
  const long long ctas = items < sms ? items : sms;  // one CTA per SM, each fetching items until none is left
  auto kernel = sdpa_bwd_kernel<D, kCausal, kFp16, kKV, kEarly, kSeq, kMask>;
  // the attribute is per device and per kernel instantiation; set it on first use there
  static bool sized[64] = {};
  int device = 0;
  LIMN_CUDA(cudaGetDevice(&device), "asking for the current device");
  if (device >= 0 && device < 64 && !sized[device]) {
    LIMN_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kBytes),
              "sizing shared memory for an sdpa backward kernel");
    sized[device] = true;
  }
  LIMN_CUDA(launch_overlapped(kernel, dim3(static_cast<unsigned>(ctas)), dim3(bwd_threads<kKV>()), L::kBytes, p.stream, map_q, map_k, map_v, map_do, map_out0, map_out1, prm),
            "launching an sdpa backward kernel");
  note_launches(1);
  return LIMN_B200_OK;
}

template <int D, bool kKV, bool kMask>
int launch_bwd_m(const Problem& p) {
  const bool fp16 = p.dtype == LIMN_B200_F16;
  if (p.causal) return fp16 ? launch_bwd<D, true, true, kKV, kMask>(p) : launch_bwd<D, true, false, kKV, kMask>(p);
  return fp16 ? launch_bwd<D, false, true, kKV, kMask>(p) : launch_bwd<D, false, false, kKV, kMask>(p);
}

template <int D, bool kKV>
int launch_bwd_d(const Problem& p) {
  return p.mask ? launch_bwd_m<D, kKV, true>(p) : launch_bwd_m<D, kKV, false>(p);
}

}  // namespace

int tcgen05_bwd_q(const Problem& p) { return (p.hd > 64 || p.hd_v > 64) ? launch_bwd_d<128, false>(p) : launch_bwd_d<64, false>(p); }
int tcgen05_bwd_kv(const Problem& p) { return (p.hd > 64 || p.hd_v > 64) ? launch_bwd_d<128, true>(p) : launch_bwd_d<64, true>(p); }

}  // namespace limn_b200
