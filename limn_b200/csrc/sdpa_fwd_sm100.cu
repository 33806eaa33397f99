// "sdpa" forward for f16/bf16 with hd and hd_v multiples of 8 up to 128, with or without a key mask: TMA-staged tiles,
// tcgen05 MMAs accumulating in tensor memory, online softmax with one thread per query row. The kernels are built for
// head dims 64 and 128; a narrower head runs in the next of the two: TMA fills the columns a row does not have with
// zeros, which add nothing to a score and give zero output columns that are not stored. hd and hd_v may differ for
// the same reason: Q and K are read with hd columns, V with hd_v, and O is stored hd_v wide.
//
// A work item is two consecutive tiles of 128 query rows of one (batch, head) problem; the problem's keys
// and values stream past them in tiles of 128 keys:
//   S_t = Q_t K_j^T          tcgen05.mma, both operands K-major in shared memory, S_t in tensor memory
//   P_t = exp2(S_t - m_t)    128 softmax threads per Q tile, one row each; P_t overwrites S_t as 16-bit
//   O_t += P_t V_j           tcgen05.mma, A = P_t from tensor memory, B = V_j (MN-major) from shared memory
// Two Q tiles per item keep the tensor pipe busy on one while the other is in its softmax.
// Each output row has exactly one owner and is accumulated in a fixed key order, so two
// runs give the same bits, as the kernel this replaces promises (limn/cuda_emit.py:748-752).
//
// The grid is one CTA per SM. A CTA fetches items from a counter (longest first) until none is left, so
// barriers, tensor memory and descriptors are set up once, and the next item's Q, K and V are on their way
// (and its first scores computed) while the current item's last tile and epilogue are still running.
//
// Warp roles (10 warps): 0-3 softmax/epilogue of Q tile 0, 4-7 of Q tile 1, 8 TMA producer and work
// fetcher, 9 MMA issuer and tensor-memory owner.
//
// Semantics follow the oracle (limn/sdpa.py:91-137): causal keeps key j for row i when
// j <= i; O is rounded once from the fp32 accumulator; L = m + log(l) in natural log.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <cstdlib>

#include "common.h"
#include "sm100_ptx.cuh"
#include "tensor_map.h"

namespace limn_b200 {
namespace {

using namespace ptx;

constexpr int kTileRows = 128;   // query rows per Q tile, keys per K/V tile
constexpr int kQTiles = 2;       // Q tiles per CTA
// Ten warps work, but the block size decides how the compiler allocates registers in the softmax loop (all sizes
// end at 168 registers; what differs is what is spilled where), and the best size differs by instantiation.
// Measured on B200: head dim 128 under a causal mask, 11 warps (0.7 % over 12, 8 % over 10); without a key mask
// otherwise, 10 warps (head dim 64: 1 to 5 % over 12; head dim 128 without a causal mask: 1 %); the key-mask kernels
// stay at the 12 they were tuned with. The spare warps go straight to the final barrier.
template <int D, bool kCausal, bool kMask>
constexpr int fwd_threads() {
  return kMask ? 384 : (D == 128 && kCausal) ? 352 : 320;
}
constexpr int kProducerWarp = 8;
constexpr int kMmaWarp = 9;
constexpr uint32_t kTmemCols = 512;
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kRescaleSlack = 8.f;   // log2 units a row maximum may outgrow its reference before O is rescaled
// Of every 8 pairs of scores, how many take exp2 as a cubic on the FMA pipe instead of on the special-function
// unit. Measured on B200: one pair is best at head dim 64 and without a causal mask (1 to 2.5 % over none or two),
// none under a causal mask at head dim 128 (1 to 2 % over one or two); three or more are slower everywhere.
// LIMN_POLY_PAIRS overrides the choice for experiments.
template <int D, bool kCausal>
constexpr int poly_pairs_of_8() {
#ifdef LIMN_POLY_PAIRS
  return LIMN_POLY_PAIRS;
#else
  return (D == 128 && kCausal) ? 0 : 1;
#endif
}

template <int D, bool kCausal, bool kMask>
struct FwdLayout {
  static constexpr int kTileBytes = kTileRows * D * 2;
  static constexpr int kAtomBytes = kTileRows * 128;        // one 64-element-wide column block of a tile
  // K and V rings, each this deep. Shared memory would hold more at head dim 64, but deeper rings are slower there
  // (measured 3: +1.5 %, 5: +4 %): two tiles in flight cover the load latency, more only put TMA's writes in the MMAs' way.
  static constexpr int kStages = 2;
  static constexpr int kQOff = 0;
  static constexpr int kKOff = kQOff + kQTiles * kTileBytes;
  static constexpr int kVOff = kKOff + kStages * kTileBytes;
  // Where the epilogue leaves O for the tile store: one 64-column block (128 rows x 128 B) per softmax group, which a
  // group's two blocks take turns in. Used at head dim 128 under a causal mask, where it is worth 2 to 3 %: the two
  // Q tiles of an item end at different times there and each group's stores are on its own critical path. Without
  // a causal mask both groups reach the epilogue together and the hand-overs cost more than the stores did (-1 %
  // at head dim 128, -6 % at 64, measured).
  static constexpr bool kTileStore = D == 128 && kCausal;
  static constexpr int kStageOff = kVOff + kStages * kTileBytes;
  static constexpr int kBarOff = kStageOff + (kTileStore ? kQTiles * kAtomBytes : 0);
  static constexpr int kBytes = kBarOff + 512 + 1024;       // room for 64 barriers + slack to align the base to 1024
  // tensor-memory columns
  static constexpr int kSCol = 0;                           // S_t at kSCol + 128 t (P_t overlays its first 64)
  static constexpr int kOCol = 256;                         // O_t at kOCol + D t
};

// barrier indices inside the barrier block
template <int D>
struct FwdBars {
  static constexpr int kS = FwdLayout<D, false, false>::kStages;
  static constexpr int q_full = 0;               // + t
  static constexpr int k_full = 2;               // + stage
  static constexpr int k_empty = k_full + kS;
  static constexpr int v_full = k_empty + kS;
  static constexpr int v_empty = v_full + kS;
  static constexpr int s_full = v_empty + kS;    // + t
  static constexpr int p_full = s_full + 2;      // + t
  static constexpr int o_full = p_full + 2;      // + t
  static constexpr int p_half = o_full + 2;      // + t: the first 64 keys' worth of P_t is in place (and O_t rescaled)
  static constexpr int q_empty = p_half + 2;     // + t: the item's last S_t has been computed, Q_t may be replaced
  static constexpr int o_free = q_empty + 2;     // + t: the epilogue has read O_t, the next item may overwrite it
  static constexpr int work_full = o_free + 2;   // + slot: the producer has fetched a work item
  static constexpr int work_empty = work_full + 2;  // + slot: every consumer has read it
  static constexpr int stage_full = work_empty + 2;   // + t: every row of a staging block is written (128 arrivals)
  static constexpr int stage_free = stage_full + 2;   // + t: the tile store has read the block
  static constexpr int count = stage_free + 2;
};

// Build-time diagnostic (-DLIMN_TRACE): one CTA records clock64() at each step of its pipeline into a
// buffer named by the LIMN_TRACE_PTR environment variable. Compiled out of the shipped library.
#ifdef LIMN_TRACE
#define TRACE_EVENT(code) do { if (blockIdx.x == 7 && lane == 0 && trace_n < 250) { prm.trace[warp * 512 + 2 * trace_n] = clock64(); prm.trace[warp * 512 + 2 * trace_n + 1] = (code); ++trace_n; } } while (0)
#else
#define TRACE_EVENT(code) do {} while (0)
#endif

struct FwdParams {
  long long bh;
#ifdef LIMN_TRACE
  long long* trace;
#endif
  const unsigned short* mask;  // (bh, t_k) key flags in the storage dtype, 0 hides a key; null without a mask
  void* out;
  float* lse;
  unsigned* status;
  unsigned* schedule;  // [0] next work item, [1] CTAs that have finished; both zero between launches
  int group;           // problems per scheduling group (see cta_work)
  int heads;           // problem p is (batch p / heads, head p % heads) in the tensor maps and in `out`
  Strides out_strides; // of O, in elements
  unsigned items;      // work items: bh * q_pairs
  int t_q, t_k;
  int width;        // columns of V and O as they lie in memory (<= D)
  int q_pairs;      // work items per problem
  int kv_tiles;     // ceil(t_k / 128)
  float scale;
};

template <int D, bool kCausal, bool kFp16, bool kMask>
__global__ void __launch_bounds__((fwd_threads<D, kCausal, kMask>()), 1)
sdpa_fwd_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                const __grid_constant__ CUtensorMap map_v, const __grid_constant__ CUtensorMap map_o, const FwdParams prm) {
  using L = FwdLayout<D, kCausal, kMask>;
  using B = FwdBars<D>;
  extern __shared__ unsigned char smem_unaligned[];
  __shared__ uint32_t tmem_slot;
  __shared__ uint32_t abort_flag;
  __shared__ unsigned work_ring[2];

  const uint32_t raw = smem_addr(smem_unaligned);
  const uint32_t base = (raw + 1023u) & ~1023u;
  const uint32_t bars = base + L::kBarOff;
  auto bar = [&](int i) { return bars + 8u * i; };

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  // ---- which rows a work item covers ----
  struct Item {
    int problem;
    int head, batch;    // the problem's coordinates in the operands
    int q0[kQTiles];    // first query row of each Q tile
    int n_kv[kQTiles];  // key tiles each Q tile consumes
    int n_max;
  };
  auto decode = [&](unsigned index) {
    Item it;
    int slot;
    cta_work(static_cast<int>(index), prm.q_pairs, prm.bh, prm.group, it.problem, slot);
    it.batch = it.problem / prm.heads;
    it.head = it.problem - it.batch * prm.heads;
    const int pair = prm.q_pairs - 1 - slot;  // longest causal rows first
#pragma unroll
    for (int t = 0; t < kQTiles; ++t) {
      it.q0[t] = (pair * kQTiles + t) * kTileRows;
      int n = prm.kv_tiles;
      if (kCausal) n = min(n, pair * kQTiles + t + 1);
      it.n_kv[t] = it.q0[t] < prm.t_q ? n : 0;
    }
    it.n_max = max(it.n_kv[0], it.n_kv[1]);
    return it;
  };

  // ---- set-up: barriers, tensor memory ----
  if (threadIdx.x == 0) {
    for (int i = 0; i < B::count; ++i) {
      unsigned arrivals = 1u;
      if ((i >= B::p_full && i < B::p_full + 2) || (i >= B::p_half && i < B::p_half + 2) || (i >= B::o_free && i < B::o_free + 2) ||
          (i >= B::stage_full && i < B::stage_full + 2))
        arrivals = 128u;                                           // every thread of a softmax group
      if (i >= B::work_empty && i < B::work_empty + 2) arrivals = 9u;  // the MMA warp and the eight softmax warps
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

  bool ok = !abort_flag;  // an earlier kernel on this device gave up: take no work, only leave the counters as found
#ifdef LIMN_TRACE
  int trace_n = 0;
#endif
  TRACE_EVENT(0);

  // Work items are fetched by the producer and passed to the other warps through a two-entry ring, so
  // the producer can load the next item's Q, K and V while the current item is still being computed.
  // Every role walks the same items in the same order and counts its own barrier phases as it goes.
  auto next_item = [&](unsigned n_item, unsigned& index) {
    const unsigned slot = n_item & 1u;
    if (!mbar_wait(bar(B::work_full + slot), (n_item >> 1) & 1u, prm.status, 0x0400u | slot)) return false;
    index = *reinterpret_cast<volatile unsigned*>(&work_ring[slot]);
    return true;
  };

  if (warp == kProducerWarp) {
    // ================= TMA producer, work fetcher =================
    if (lane == 0 && ok) {
      tma_prefetch_descriptor(&map_q);
      tma_prefetch_descriptor(&map_k);
      tma_prefetch_descriptor(&map_v);
      unsigned q_uses[kQTiles] = {0u, 0u};  // items so far in which Q tile t had rows
      unsigned step = 0;                    // key tiles loaded so far, over all items
      for (unsigned n_item = 0; ok; ++n_item) {
        const unsigned slot = n_item & 1u;
        ok = mbar_wait(bar(B::work_empty + slot), ((n_item >> 1) & 1u) ^ 1u, prm.status, 0x0120u | slot);
        if (!ok) break;
        // a CTA's first item is its own number (no round trip to the counter on the way to the first load); the
        // counter hands out what lies beyond the grid
        const unsigned index = n_item == 0 ? blockIdx.x : gridDim.x + atomicAdd(prm.schedule, 1u);
        *reinterpret_cast<volatile unsigned*>(&work_ring[slot]) = index;
        mbar_arrive(bar(B::work_full + slot));
        if (index >= prm.items) break;
        const Item item = decode(index);
#pragma unroll
        for (int t = 0; t < kQTiles; ++t) {
          if (item.n_kv[t] == 0 || !ok) continue;
          ok = mbar_wait(bar(B::q_empty + t), (q_uses[t] & 1u) ^ 1u, prm.status, 0x0130u | t);
          if (!ok) break;
          ++q_uses[t];
          mbar_expect_tx(bar(B::q_full + t), L::kTileBytes);
#pragma unroll
          for (int a = 0; a < D / 64; ++a)
            tma_load_4d(base + L::kQOff + t * L::kTileBytes + a * L::kAtomBytes, &map_q, bar(B::q_full + t), a * 64,
                        item.q0[t], item.head, item.batch);
        }
        for (int j = 0; j < item.n_max && ok; ++j, ++step) {
          const int stage = step % L::kStages;
          const uint32_t wrap = (step / L::kStages) & 1;
          ok = mbar_wait(bar(B::k_empty + stage), wrap ^ 1u, prm.status, 0x0100u | stage);
          if (!ok) break;
          mbar_expect_tx(bar(B::k_full + stage), L::kTileBytes);
#pragma unroll
          for (int a = 0; a < D / 64; ++a)
            tma_load_4d(base + L::kKOff + stage * L::kTileBytes + a * L::kAtomBytes, &map_k, bar(B::k_full + stage), a * 64,
                        j * kTileRows, item.head, item.batch);
          ok = mbar_wait(bar(B::v_empty + stage), wrap ^ 1u, prm.status, 0x0110u | stage);
          if (!ok) break;
          mbar_expect_tx(bar(B::v_full + stage), L::kTileBytes);
#pragma unroll
          for (int a = 0; a < D / 64; ++a)
            tma_load_4d(base + L::kVOff + stage * L::kTileBytes + a * L::kAtomBytes, &map_v, bar(B::v_full + stage), a * 64,
                        j * kTileRows, item.head, item.batch);
        }
      }
    }
  } else if (warp == kMmaWarp) {
    // ================= MMA issuer =================
    if (lane == 0 && ok) {
      constexpr uint32_t idesc_s = mma_idesc(kTileRows, kTileRows, kFp16, false, false);
      constexpr uint32_t idesc_pv = mma_idesc(kTileRows, D, kFp16, false, true);
      // S_t = Q_t K^T over the head dim, 16 elements per instruction
      auto issue_s = [&](int t, int stage) {
        const uint32_t q_lo = desc_lo(base + L::kQOff + t * L::kTileBytes, 0);
        const uint32_t k_lo = desc_lo(base + L::kKOff + stage * L::kTileBytes, 0);
        const uint32_t c = tmem + L::kSCol + t * 128;
        mma_ss_lo<false>(c, q_lo, k_lo, idesc_s);
#pragma unroll
        for (int kk = 1; kk < D / 16; ++kk) {
          constexpr uint32_t kAtom16 = L::kAtomBytes >> 4;
          const uint32_t off = (kk / 4) * kAtom16 + (kk % 4) * 2;  // in 16-byte units
          mma_ss_lo<true>(c, q_lo + off, k_lo + off, idesc_s);
        }
      };
      // O_t += P_t V over the 128 keys of the tile, 16 keys per instruction
      auto issue_pv = [&](int t, int stage, int part, bool first) {
        const uint32_t v_lo = desc_lo(base + L::kVOff + stage * L::kTileBytes, L::kAtomBytes);
        const uint32_t c = tmem + L::kOCol + t * D;
        const uint32_t a = tmem + L::kSCol + t * 128;
#pragma unroll
        for (int kk = 4 * part; kk < 4 * part + 4; ++kk)
          mma_ts_lo(c, a + kk * 8, v_lo + kk * (16 * 128 / 16), idesc_pv, (kk > 0 || !first) ? 1u : 0u);
      };
      unsigned q_uses[kQTiles] = {0u, 0u};  // items finished in which Q tile t had rows
      unsigned tiles[kQTiles] = {0u, 0u};   // key tiles Q tile t has been through, over all items
      unsigned step = 0;                    // key tiles consumed so far, over all items
      for (unsigned n_item = 0; ok; ++n_item) {
        unsigned index;
        ok = next_item(n_item, index);
        if (!ok) break;
        mbar_arrive(bar(B::work_empty + (n_item & 1u)));
        if (index >= prm.items) break;
        const Item item = decode(index);
#pragma unroll
        for (int t = 0; t < kQTiles; ++t)
          if (item.n_kv[t] > 0 && ok) ok = mbar_wait(bar(B::q_full + t), q_uses[t] & 1u, prm.status, 0x0200u | t);
        if (!ok) break;
        if (item.n_max > 0) {
          const int stage = step % L::kStages;
          ok = mbar_wait(bar(B::k_full + stage), (step / L::kStages) & 1, prm.status, 0x0210u);
          if (!ok) break;
          tc_fence_after_sync();
#pragma unroll
          for (int t = 0; t < kQTiles; ++t)
            if (item.n_kv[t] > 0) {
              // (the S_t region is free: the MMAs run in issue order, and the last one issued for this tile was
              // the product that consumed the P_t stored there)
              issue_s(t, stage);
              mma_commit(bar(B::s_full + t));
              if (item.n_kv[t] == 1) mma_commit(bar(B::q_empty + t));
            }
          mma_commit(bar(B::k_empty + stage));
        }
        for (int j = 0; j < item.n_max && ok; ++j, ++step) {
          const int stage = step % L::kStages;
          const uint32_t wrap = (step / L::kStages) & 1;
          const int next = (step + 1) % L::kStages;
          const uint32_t next_wrap = ((step + 1) / L::kStages) & 1;
          ok = mbar_wait(bar(B::v_full + stage), wrap, prm.status, 0x0220u | stage);
          bool issued_next = false;
#pragma unroll
          for (int t = 0; t < kQTiles; ++t) {
            if (!ok || j >= item.n_kv[t]) continue;
            TRACE_EVENT(100 + t);
            const uint32_t phase = tiles[t] & 1u;
            // the product starts on the first 64 keys while the softmax is still on the last 64
            ok = mbar_wait(bar(B::p_half + t), phase, prm.status, 0x0260u | t);
            if (!ok) break;
            // the item's first product overwrites O_t: the previous item's epilogue must have read it
            if (j == 0) ok = mbar_wait(bar(B::o_free + t), (q_uses[t] & 1u) ^ 1u, prm.status, 0x0270u | t);
            if (!ok) break;
            tc_fence_after_sync();
            issue_pv(t, stage, 0, j == 0);
            ok = mbar_wait(bar(B::p_full + t), phase, prm.status, 0x0230u | t);
            if (!ok) break;
            TRACE_EVENT(110 + t);
            tc_fence_after_sync();
            issue_pv(t, stage, 1, j == 0);
            TRACE_EVENT(120 + t);
            ++tiles[t];
            if (j + 1 < item.n_kv[t]) {
              // the scores can only follow the product that consumed the P_t lying over them; s_full then also
              // tells the softmax that O_t is settled
              ok = mbar_wait(bar(B::k_full + next), next_wrap, prm.status, 0x0240u | next);
              if (!ok) break;
              tc_fence_after_sync();
              issue_s(t, next);
              mma_commit(bar(B::s_full + t));
              if (j + 2 == item.n_kv[t]) mma_commit(bar(B::q_empty + t));
              TRACE_EVENT(130 + t);
              issued_next = true;
            } else {
              mma_commit(bar(B::o_full + t));
            }
          }
          if (!ok) break;
          mma_commit(bar(B::v_empty + stage));
          if (issued_next) mma_commit(bar(B::k_empty + next));
        }
#pragma unroll
        for (int t = 0; t < kQTiles; ++t)
          if (item.n_kv[t] > 0) ++q_uses[t];
      }
    }
  } else if (warp < kProducerWarp) {
    // ================= softmax + epilogue, one thread per query row =================
    const int t = warp >> 2;
    const int row_in_tile = threadIdx.x & 127;
    const uint32_t lane_base = static_cast<uint32_t>((warp & 3) * 32) << 16;
    const uint32_t t_s = tmem + lane_base + L::kSCol + t * 128;
    const uint32_t t_o = tmem + lane_base + L::kOCol + t * D;
    const float sl2 = prm.scale * kLog2e;
    // m is the score (in raw units) the exponentials are measured against. It only moves when the
    // row maximum has outgrown it by more than kRescaleSlack (in log2 units), so most tiles need no
    // rescaling of O_t; until then probabilities may reach 2^kRescaleSlack, which fp32 sums and
    // 16-bit P carry without loss. The result is the same softmax: L = m * scale + log(l).
    const uint64_t sl2_2 = f2_pack(sl2, sl2);
    unsigned tiles = 0;   // key tiles this group has been through, over all items
    unsigned o_uses = 0;  // items this group has finished
    unsigned stores = 0;  // staging blocks this group has handed to TMA
    // Key mask: a hidden key is a score of -inf for every row. Each lane fetches four of a tile's 128 flags one tile
    // ahead of their use; a ballot per 32 keys then gives every thread all of them.
    // (the flags stay as loaded until the next tile needs them: a warp issues in order, so turning them into anything
    // right after the load would stall it for the load's latency, every tile)
    auto fetch_flags = [&](int problem, int kv0, unsigned (&out4)[4]) {
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const int key = kv0 + 32 * c + lane;
        out4[c] = key < prm.t_k ? prm.mask[static_cast<long long>(problem) * prm.t_k + key] : 0u;  // past the end: hidden
      }
    };
    for (unsigned n_item = 0; ok; ++n_item) {
    unsigned index;
    ok = __all_sync(0xffffffffu, next_item(n_item, index));
    if (!ok) break;
    __syncwarp();
    if (lane == 0) mbar_arrive(bar(B::work_empty + (n_item & 1u)));
    if (index >= prm.items) break;
    const Item item = decode(index);
    const int problem = item.problem;
    const int n = item.n_kv[t];
    if (n == 0) continue;
    const int row = item.q0[t] + row_in_tile;
    float m = -INFINITY, l = 0.f;
    unsigned flags[4] = {1u, 1u, 1u, 1u};
    if (kMask) fetch_flags(problem, 0, flags);
    for (int j = 0; j < n; ++j, ++tiles) {
      // Key mask: which of the tile's 128 keys are hidden, as four ballot words in registers (each lane fetched four
      // of the flags a tile ahead). A tile none of whose keys is hidden (every tile but the last few of a padded
      // batch) is handled like an unmasked one.
      unsigned hid[4] = {0u, 0u, 0u, 0u};
      bool any_hidden = false;
      if (kMask) {
#pragma unroll
        for (int c = 0; c < 4; ++c) hid[c] = __ballot_sync(0xffffffffu, (flags[c] & 0x7fffu) == 0u);
        any_hidden = ((hid[0] | hid[1]) | (hid[2] | hid[3])) != 0u;
        if (j + 1 < n) fetch_flags(problem, (j + 1) * kTileRows, flags);
      }
      ok = __all_sync(0xffffffffu, mbar_wait(bar(B::s_full + t), tiles & 1u, prm.status, 0x0300u | t));  // warp-uniform: the tensor-memory ops below are warp-wide
      if (!ok) break;
      TRACE_EVENT(2);
      tc_fence_after_sync();
      uint32_t s[4][32];
#pragma unroll
      for (int c = 0; c < 4; ++c) tmem_ld32(t_s + 32 * c, s[c]);
      tmem_ld_wait();
      TRACE_EVENT(3);
      const int kv0 = j * kTileRows;
      const bool diagonal = kCausal && kv0 + kTileRows > item.q0[t];     // some key of this tile is right of some row
      const bool ragged = kv0 + kTileRows > prm.t_k;                // some key of this tile does not exist
      if (diagonal || ragged || (kMask && any_hidden)) {
        int limit = prm.t_k - kv0;                                  // keys [0, limit) of the tile are visible
        if (kCausal) limit = min(limit, row - kv0 + 1);
#pragma unroll
        for (int c = 0; c < 4; ++c)
#pragma unroll
          for (int i = 0; i < 32; ++i)
            if (c * 32 + i >= limit || (kMask && ((hid[c] >> i) & 1u) != 0u)) s[c][i] = 0xff800000u;  // -inf
      }
      float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
      for (int c = 0; c < 4; ++c)
#pragma unroll
        for (int i = 0; i < 32; i += 2) mx4[(i >> 1) & 3] = max3(mx4[(i >> 1) & 3], __uint_as_float(s[c][i]), __uint_as_float(s[c][i + 1]));
      const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3]));
      // Without a key mask the first tile always has a visible key (key 0), so mx is finite from the start.
      // With one, a row may have met no visible key yet: then mx and m are both -inf, nothing moves, and the
      // exponentials are measured against 0 so that they come out exp2(-inf) = 0 instead of NaN.
      const bool moves = (mx - m) * sl2 > kRescaleSlack;  // true at the first visible key, where m is -inf
      float alpha = 1.f;
      if (moves) {
        alpha = exp2_approx((m - mx) * sl2);
        m = mx;
      }
      TRACE_EVENT(4);
      const float shift = (kMask && m == -INFINITY) ? 0.f : -m * sl2;
      const uint64_t shift2 = f2_pack(shift, shift);
      uint64_t sum2[2] = {0ull, 0ull};
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        if (h == 1) {
          // O_t was last written by the PV of tile j-1, which s_full also covers. It is rescaled before any of
          // this tile's P_t is handed over (the product on the first half starts early), at the point where
          // the first half's scores are no longer held in registers.
          if (j > 0 && __any_sync(0xffffffffu, moves)) {
#pragma unroll
            for (int c = 0; c < D / 32; ++c) {
              uint32_t o[32];
              tmem_ld32(t_o + 32 * c, o);
              tmem_ld_wait();
#pragma unroll
              for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
              tmem_st32(t_o + 32 * c, o);
            }
          }
        }
        uint32_t packed[32];
#pragma unroll
        for (int cc = 0; cc < 2; ++cc) {
          const int c = 2 * h + cc;
#pragma unroll
          for (int i = 0; i < 32; i += 2) {
            const uint64_t x2 = f2_fma(f2_pack_bits(s[c][i], s[c][i + 1]), sl2_2, shift2);
            float p0, p1;
            // (not under a key mask: the cubic turns a hidden key's -inf into 2^-125 rather than 0, which a row
            // with no visible key at all would then mistake for a denominator)
            if (!kMask && ((i >> 1) & 7) < poly_pairs_of_8<D, kCausal>()) {
              exp2_poly2(x2, p0, p1);
            } else {
              f2_unpack(x2, p0, p1);
              p0 = exp2_approx(p0);
              p1 = exp2_approx(p1);
            }
            sum2[(i >> 1) & 1] = f2_add(sum2[(i >> 1) & 1], f2_pack(p0, p1));
            packed[cc * 16 + (i >> 1)] = kFp16 ? pack_f16(p0, p1) : pack_bf16(p0, p1);
          }
          if (h == 1 && cc == 0) {
            // the first half's store was issued a chunk of exponentials ago; hand it over
            tmem_st_wait();
            tc_fence_before_sync();
            mbar_arrive(bar(B::p_half + t));
          }
        }
        tmem_st32(t_s + 32 * h, packed);
      }
      TRACE_EVENT(5);
      float sum_a, sum_b, sum_c, sum_d;
      f2_unpack(sum2[0], sum_a, sum_b);
      f2_unpack(sum2[1], sum_c, sum_d);
      l = l * alpha + ((sum_a + sum_b) + (sum_c + sum_d));
      tmem_st_wait();
      TRACE_EVENT(6);
      tc_fence_before_sync();
      mbar_arrive(bar(B::p_full + t));
    }
    if (ok) ok = __all_sync(0xffffffffu, mbar_wait(bar(B::o_full + t), o_uses & 1u, prm.status, 0x0310u | t));
    if (ok) {
      tc_fence_after_sync();
      const float inv = 1.f / l;
      const long long out_row = static_cast<long long>(problem) * prm.t_q + row;  // in L, which is always dense
      if constexpr (L::kTileStore) {
        // O goes out as tile stores: every thread leaves its row, rounded, in the group's staging block (in the
        // swizzled layout, so the 32 rows of a warp fall on distinct banks), and one thread hands the block to TMA,
        // which writes whole 128-byte rows and leaves out the rows and columns the tensor does not have. (A thread
        // storing its own row in 16-byte pieces costs the load/store unit 32 transactions per instruction.)
        const uint32_t stage = base + L::kStageOff + t * L::kAtomBytes;
        const bool leader = (warp & 3) == 0 && lane == 0;
#pragma unroll
        for (int blk = 0; blk < D / 64 && ok; ++blk, ++stores) {
          // the store before this one has read the block: the thread that issued it says so (waits are bounded,
          // like every wait here: a group whose warps disagree about going on must not hang on one another)
          if (leader) {
            tma_store_wait_read();
            mbar_arrive(bar(B::stage_free + t));
          }
          ok = __all_sync(0xffffffffu, mbar_wait(bar(B::stage_free + t), stores & 1u, prm.status, 0x0320u | t));
          if (!ok) break;
#pragma unroll
          for (int cc = 0; cc < 2; ++cc) {
            uint32_t o[32];
            tmem_ld32(t_o + 64 * blk + 32 * cc, o);
            tmem_ld_wait();
#pragma unroll
            for (int v4 = 0; v4 < 4; ++v4) {
              uint32_t w[4];
#pragma unroll
              for (int i = 0; i < 4; ++i) {
                const float a = __uint_as_float(o[v4 * 8 + 2 * i]) * inv;
                const float b = __uint_as_float(o[v4 * 8 + 2 * i + 1]) * inv;
                w[i] = kFp16 ? pack_f16(a, b) : pack_bf16(a, b);
              }
              st_shared_v4(swizzled_piece(stage, row_in_tile, cc * 4 + v4), w[0], w[1], w[2], w[3]);
            }
          }
          if (blk == D / 64 - 1) {
            // O_t is in registers or staged: the next item's first product may overwrite it
            tc_fence_before_sync();
            mbar_arrive(bar(B::o_free + t));
          }
          fence_async_shared();
          mbar_arrive(bar(B::stage_full + t));
          if (leader) {
            if (mbar_wait(bar(B::stage_full + t), stores & 1u, prm.status, 0x0330u | t)) {
              tma_store_4d(&map_o, stage, 64 * blk, item.q0[t], item.head, item.batch);
              tma_store_commit();
            }
          }
        }
        if (row < prm.t_q) prm.lse[out_row] = m * prm.scale + logf(l);
      } else {
      const long long out_at = item.batch * prm.out_strides.batch + item.head * prm.out_strides.head + row * prm.out_strides.row;
#pragma unroll
      for (int c = 0; c < D / 32; ++c) {
        uint32_t o[32];
        tmem_ld32(t_o + 32 * c, o);
        tmem_ld_wait();
        if (row < prm.t_q) {
          uint4* dst = reinterpret_cast<uint4*>(static_cast<unsigned char*>(prm.out) + (out_at + 32 * c) * 2);
#pragma unroll
          for (int v4 = 0; v4 < 4; ++v4) {
            uint32_t w[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              const float a = __uint_as_float(o[v4 * 8 + 2 * i]) * inv;
              const float b = __uint_as_float(o[v4 * 8 + 2 * i + 1]) * inv;
              w[i] = kFp16 ? pack_f16(a, b) : pack_bf16(a, b);
            }
            if (32 * c + 8 * v4 < prm.width) dst[v4] = make_uint4(w[0], w[1], w[2], w[3]);
          }
        }
      }
      if (row < prm.t_q) prm.lse[out_row] = m * prm.scale + logf(l);
      // O_t is in registers or stored: the next item's first product may overwrite it
      tc_fence_before_sync();
      mbar_arrive(bar(B::o_free + t));
      }
      ++o_uses;
    }
    }  // items
    // the last tile store must have read its staging block before the CTA gives its shared memory back
    if (L::kTileStore && (warp & 3) == 0 && lane == 0) tma_store_wait_read();
  }

  // ---- teardown ----
  tc_fence_before_sync();
  __syncthreads();
  if (warp == kMmaWarp && !abort_flag) {
    if (*reinterpret_cast<volatile unsigned*>(prm.status) != kStatusOk) {
      // a wait gave up somewhere: give copies and MMAs still in flight time to land before the
      // tensor memory and shared memory they target are released
      for (int i = 0; i < 2000; ++i) __nanosleep(1000);
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

template <int D, bool kCausal, bool kFp16, bool kMask>
int launch_fwd(const Problem& p) {
  using L = FwdLayout<D, kCausal, kMask>;
  CUtensorMap map_q, map_k, map_v, map_o;
  const int heads = p.heads > 0 ? p.heads : static_cast<int>(p.bh), batch = static_cast<int>(p.bh / heads);
  if (int rc = make_tile_map(&map_q, p.q, kFp16, batch, heads, p.t_q, p.hd, kTileRows, operand_strides(p, kOpQ, heads, p.t_q, p.hd))) return rc;
  if (int rc = make_tile_map(&map_k, p.k, kFp16, batch, heads, p.t_k, p.hd, kTileRows, operand_strides(p, kOpK, heads, p.t_k, p.hd))) return rc;
  if (int rc = make_tile_map(&map_v, p.v, kFp16, batch, heads, p.t_k, p.hd_v, kTileRows, operand_strides(p, kOpV, heads, p.t_k, p.hd_v))) return rc;
  if (int rc = make_tile_map(&map_o, p.out, kFp16, batch, heads, p.t_q, p.hd_v, kTileRows, operand_strides(p, kOpOut, heads, p.t_q, p.hd_v))) return rc;
  FwdParams prm;
  prm.out = p.out;
  prm.heads = heads;
  prm.out_strides = operand_strides(p, kOpOut, heads, p.t_q, p.hd_v);
  prm.width = p.hd_v;
  if ((prm.out_strides.batch | prm.out_strides.head | prm.out_strides.row) & 7)
    return fail(LIMN_B200_BAD_ARGUMENT, "sdpa: operand strides must be multiples of 8 elements");
  if (reinterpret_cast<uintptr_t>(p.out) & 15u) return fail(LIMN_B200_BAD_ARGUMENT, "sdpa: the output is not 16-byte aligned");
  prm.mask = static_cast<const unsigned short*>(p.mask);
  prm.lse = static_cast<float*>(p.lse_out);
  prm.status = p.status;
  if (prm.status == nullptr)
    if (int rc = status_word(&prm.status)) return rc;
  prm.bh = p.bh;
  prm.t_q = p.t_q, prm.t_k = p.t_k;
  prm.q_pairs = (p.t_q + kQTiles * kTileRows - 1) / (kQTiles * kTileRows);
  prm.kv_tiles = (p.t_k + kTileRows - 1) / kTileRows;
#ifdef LIMN_TRACE
  const char* trace_ptr = getenv("LIMN_TRACE_PTR");
  if (trace_ptr == nullptr) return fail(LIMN_B200_BAD_ARGUMENT, "this is a -DLIMN_TRACE build: set LIMN_TRACE_PTR to the trace buffer's device address");
  prm.trace = reinterpret_cast<long long*>(strtoull(trace_ptr, nullptr, 16));
#endif
  prm.scale = static_cast<float>(p.scale);
  const long long items = p.bh * prm.q_pairs;
  if (items > 0x7fffffffLL) return fail(LIMN_B200_UNSUPPORTED, "sdpa: %lld work items exceed the counter", items);
  prm.items = static_cast<unsigned>(items);
  if (int rc = schedule_words(&prm.schedule)) return rc;
  int sms = 0;
  if (int rc = sm_count(&sms)) return rc;
  prm.group = work_group(p, items, sms);
  const long long ctas = items < sms ? items : sms;  // one CTA per SM (shared and tensor memory allow no more), each fetching items until none is left
  auto kernel = sdpa_fwd_kernel<D, kCausal, kFp16, kMask>;
  // the attribute is per device and per kernel instantiation; set it on first use there
  static bool sized[64] = {};
  int device = 0;
  LIMN_CUDA(cudaGetDevice(&device), "asking for the current device");
  if (device >= 0 && device < 64 && !sized[device]) {
    LIMN_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kBytes),
              "sizing shared memory for the sdpa kernel");
    sized[device] = true;
  }
  LIMN_CUDA(launch_overlapped(kernel, dim3(static_cast<unsigned>(ctas)), dim3(fwd_threads<D, kCausal, kMask>()), L::kBytes, p.stream, map_q, map_k, map_v, map_o, prm),
            "launching the sdpa kernel");
  note_launches(1);
  return LIMN_B200_OK;
}

template <int D, bool kMask>
int launch_fwd_m(const Problem& p) {
  const bool fp16 = p.dtype == LIMN_B200_F16;
  if (p.causal) return fp16 ? launch_fwd<D, true, true, kMask>(p) : launch_fwd<D, true, false, kMask>(p);
  return fp16 ? launch_fwd<D, false, true, kMask>(p) : launch_fwd<D, false, false, kMask>(p);
}

template <int D>
int launch_fwd_d(const Problem& p) {
  return p.mask ? launch_fwd_m<D, true>(p) : launch_fwd_m<D, false>(p);
}

}  // namespace

int tcgen05_fwd(const Problem& p) { return (p.hd > 64 || p.hd_v > 64) ? launch_fwd_d<128>(p) : launch_fwd_d<64>(p); }

}  // namespace limn_b200
