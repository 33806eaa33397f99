// "sdpa" forward for decode shapes: a handful of query rows (t_q <= 4) against a long run of keys, f16/bf16 with
// hd == hd_v in {64, 128}, no causal mask (causal needs t_q == t_k), with or without a key mask. This is the step of a
// kv cache: one new token reads every slot filled so far (the reference tests the shape at
// tests/test_attention.py:385-396 and serves it with the same one-thread-per-query-row kernel as everything else,
// limn/cuda_emit.py:921-965, which leaves all but t_q threads of a block idle).
//
// The work is reading K and V once; the arithmetic is a few flops per byte, so tensor cores have nothing to add and
// the 128-row MMA tile of the prefill kernel would spend 127 of its 128 rows on nothing. Here one CTA of 16 warps
// owns one (batch, head) problem. D / 8 lanes share a key (each holds 8 of its elements as one 16-byte load), so a
// warp instruction fetches 2 or 4 consecutive keys, 512 contiguous bytes; every group of lanes walks its own
// subsequence of the keys, four at a time with all eight loads (K and V) issued before the first is used, and keeps an
// online softmax of its own per query row: a running maximum, a denominator and 8 accumulator elements per lane. The
// groups of a warp are merged with shuffles, the 16 warps through shared memory, always in the same order, so two runs
// give the same bits. A batch too small to fill the GPU with one CTA per problem gets a thread-block cluster of up
// to 8 CTAs per problem instead: the CTAs of a cluster deal the problem's keys out among themselves, and CTA 0 folds
// the others' results out of their shared memory (distributed shared memory, no scratch in global memory) in rank
// order. Semantics as the oracle's (limn/sdpa.py:91-137): a hidden key contributes exactly 0, a row with
// no visible key is NaN with L = -inf, O is rounded once from fp32, L = m + log(l) in natural log.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "common.h"
#include "tensor_map.h"

namespace limn_b200 {
namespace {

constexpr int kWarps = 16;
constexpr int kThreads = kWarps * 32;
constexpr int kUnroll = 4;  // keys a group of lanes has in flight
constexpr int kMaxRows = 4;
constexpr float kLog2e = 1.4426950408889634f;

struct DecodeParams {
  const void* q;
  const void* k;
  const void* v;
  const unsigned short* mask;  // (bh, t_k) flags in the storage dtype, 0 hides a key; null without a mask
  void* out;
  float* lse;
  int heads;  // problem p is (batch p / heads, head p % heads)
  Strides q_strides, k_strides, v_strides, o_strides;  // in elements
  int t_q, t_k;
  float scale;
  int split;  // CTAs per problem (the cluster size): 1, 2, 4 or 8
};

// ---- thread-block cluster: rank, barrier, a peer CTA's shared memory ----
__device__ __forceinline__ unsigned cluster_rank() {
  unsigned r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ float peer_shared(const float* mine, unsigned rank) {
  unsigned local = static_cast<unsigned>(__cvta_generic_to_shared(mine)), remote;
  float v;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local), "r"(rank));
  asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(remote) : "memory");
  return v;
}

template <bool kFp16>
__device__ __forceinline__ void widen8(const uint4& raw, float (&f)[8]) {
  const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    if (kFp16) {
      const float2 pair = __half22float2(*reinterpret_cast<const __half2*>(&w[i]));
      f[2 * i] = pair.x, f[2 * i + 1] = pair.y;
    } else {
      f[2 * i] = __uint_as_float(w[i] << 16), f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
    }
  }
}

// Fold the running softmax (m_b, l_b, acc_b) into (m_a, l_a, acc_a). Scores are in raw units; sl2 = scale * log2 e.
__device__ __forceinline__ void merge(float& m_a, float& l_a, float (&acc_a)[8], float m_b, float l_b, const float (&acc_b)[8], float sl2) {
  const float m = fmaxf(m_a, m_b);
  // a side that has seen no visible key has m = -inf and l = 0: its factor must be 0, not exp2(-inf + inf)
  const float fa = m_a == -INFINITY ? 0.f : exp2f((m_a - m) * sl2);
  const float fb = m_b == -INFINITY ? 0.f : exp2f((m_b - m) * sl2);
  l_a = l_a * fa + l_b * fb;
#pragma unroll
  for (int i = 0; i < 8; ++i) acc_a[i] = acc_a[i] * fa + acc_b[i] * fb;
  m_a = m;
}

// Two CTAs per SM where the registers allow it (one or two query rows), so that every problem of a batch of a few
// hundred is resident at once and the problems share HBM instead of queueing for SMs.
template <int D, bool kFp16, bool kMask, int R>
__global__ void __launch_bounds__(kThreads, R <= 2 ? 2 : 1) sdpa_decode_kernel(const DecodeParams prm) {
  constexpr int kLanesPerKey = D / 8;           // 16 or 8
  constexpr int kGroups = 32 / kLanesPerKey;    // keys per warp instruction: 2 or 4
  __shared__ float part_m[kWarps][R], part_l[kWarps][R];
  __shared__ float part_acc[kWarps][R][D];
  __shared__ float cta_m[R], cta_l[R], cta_o[R][D];  // this CTA's share of the problem, for the cluster's CTA 0

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int group = lane / kLanesPerKey, gl = lane % kLanesPerKey;
  const int split = prm.split;
  const unsigned rank = split > 1 ? cluster_rank() : 0u;
  const int problem = blockIdx.x / split;
  const int batch = problem / prm.heads, head = problem - batch * prm.heads;
  const float sl2 = prm.scale * kLog2e;

  const unsigned char* q_base = static_cast<const unsigned char*>(prm.q) + (batch * prm.q_strides.batch + head * prm.q_strides.head) * 2;
  const unsigned char* k_base = static_cast<const unsigned char*>(prm.k) + (batch * prm.k_strides.batch + head * prm.k_strides.head) * 2;
  const unsigned char* v_base = static_cast<const unsigned char*>(prm.v) + (batch * prm.v_strides.batch + head * prm.v_strides.head) * 2;
  const long long k_row = prm.k_strides.row * 2, v_row = prm.v_strides.row * 2;  // bytes between keys
  const unsigned short* flags = kMask ? prm.mask + static_cast<long long>(problem) * prm.t_k : nullptr;

  // this lane's 8 elements of every query row
  float q[R][8];
#pragma unroll
  for (int r = 0; r < R; ++r) {
    const uint4 raw = *reinterpret_cast<const uint4*>(q_base + (static_cast<long long>(r) * prm.q_strides.row + gl * 8) * 2);
    widen8<kFp16>(raw, q[r]);
  }

  float m[R], l[R], acc[R][8];
#pragma unroll
  for (int r = 0; r < R; ++r) {
    m[r] = -INFINITY, l[r] = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[r][i] = 0.f;
  }

  // keys are dealt out so that the groups of a warp, and the warps of the CTA, read consecutive keys together
  constexpr int kPerPass = kWarps * kUnroll * kGroups;
  for (int first = rank * kPerPass; first < prm.t_k; first += split * kPerPass) {
    uint4 k_raw[kUnroll], v_raw[kUnroll];
    int key[kUnroll];
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      key[u] = first + (u * kWarps + warp) * kGroups + group;
      const int at = min(key[u], prm.t_k - 1);  // past the end: read the last key again, its score is discarded below
      k_raw[u] = *reinterpret_cast<const uint4*>(k_base + at * k_row + gl * 16);
    }
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      const int at = min(key[u], prm.t_k - 1);
      v_raw[u] = *reinterpret_cast<const uint4*>(v_base + at * v_row + gl * 16);
    }
    float s[R][kUnroll];
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      float kf[8];
      widen8<kFp16>(k_raw[u], kf);
      bool visible = key[u] < prm.t_k;
      if (kMask && visible) visible = (flags[key[u]] & 0x7fffu) != 0;
#pragma unroll
      for (int r = 0; r < R; ++r) {
        float dot = 0.f;
#pragma unroll
        for (int i = 0; i < 8; ++i) dot = fmaf(q[r][i], kf[i], dot);
#pragma unroll
        for (int step = kLanesPerKey / 2; step > 0; step >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, step);
        s[r][u] = visible ? dot : -INFINITY;
      }
    }
#pragma unroll
    for (int r = 0; r < R; ++r) {
      float mx = s[r][0];
#pragma unroll
      for (int u = 1; u < kUnroll; ++u) mx = fmaxf(mx, s[r][u]);
      const float m_new = fmaxf(m[r], mx);
      if (m_new == -INFINITY) continue;  // nothing visible yet: p would be exp2(-inf + inf)
      const float alpha = exp2f((m[r] - m_new) * sl2);  // 0 at the first visible key, where m is -inf
      m[r] = m_new;
      float p[kUnroll], sum = 0.f;
#pragma unroll
      for (int u = 0; u < kUnroll; ++u) {
        p[u] = exp2f((s[r][u] - m_new) * sl2);
        sum += p[u];
      }
      l[r] = l[r] * alpha + sum;
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[r][i] *= alpha;
#pragma unroll
      for (int u = 0; u < kUnroll; ++u) {
        float vf[8];
        widen8<kFp16>(v_raw[u], vf);
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[r][i] = fmaf(p[u], vf[i], acc[r][i]);
      }
    }
  }

  // ---- the groups of a warp (lanes gl, gl + kLanesPerKey, ... hold the same 8 elements) ----
#pragma unroll
  for (int r = 0; r < R; ++r) {
#pragma unroll
    for (int step = kLanesPerKey; step < 32; step <<= 1) {
      const float m_b = __shfl_xor_sync(0xffffffffu, m[r], step), l_b = __shfl_xor_sync(0xffffffffu, l[r], step);
      float acc_b[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) acc_b[i] = __shfl_xor_sync(0xffffffffu, acc[r][i], step);
      // both partners compute the same sum in the same order: the lower one keeps (a, b), the upper one (b, a),
      // and addition commutes, so every lane ends with identical values
      if (lane & step) {
        float m_a = m_b, l_a = l_b;
        merge(m_a, l_a, acc_b, m[r], l[r], acc[r], sl2);
        m[r] = m_a, l[r] = l_a;
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[r][i] = acc_b[i];
      } else {
        merge(m[r], l[r], acc[r], m_b, l_b, acc_b, sl2);
      }
    }
    if (group == 0) {
      if (gl == 0) part_m[warp][r] = m[r], part_l[warp][r] = l[r];
#pragma unroll
      for (int i = 0; i < 8; ++i) part_acc[warp][r][gl * 8 + i] = acc[r][i];
    }
  }
  __syncthreads();

  // ---- the 16 warps: thread (r, d) folds them in warp order ----
  for (int at = threadIdx.x; at < R * D; at += kThreads) {
    const int r = at / D, d = at - r * D;
    float m_tot = -INFINITY;
#pragma unroll
    for (int w = 0; w < kWarps; ++w) m_tot = fmaxf(m_tot, part_m[w][r]);
    float l_tot = 0.f, o = 0.f;
#pragma unroll
    for (int w = 0; w < kWarps; ++w) {
      const float f = part_m[w][r] == -INFINITY ? 0.f : exp2f((part_m[w][r] - m_tot) * sl2);
      l_tot = fmaf(part_l[w][r], f, l_tot);
      o = fmaf(part_acc[w][r][d], f, o);
    }
    cta_o[r][d] = o;
    if (d == 0) cta_m[r] = m_tot, cta_l[r] = l_tot;
  }
  if (split > 1) cluster_sync();  // every CTA of the cluster has its share in shared memory
  else __syncthreads();

  // ---- the CTAs of the cluster, folded by CTA 0 in rank order; one element per thread, rounded once ----
  if (rank == 0) {
    for (int at = threadIdx.x; at < R * D; at += kThreads) {
      const int r = at / D, d = at - r * D;
      float m_tot = cta_m[r], l_tot = cta_l[r], o = cta_o[r][d];
      for (int c = 1; c < split; ++c) {
        const float m_c = peer_shared(&cta_m[r], c), l_c = peer_shared(&cta_l[r], c), o_c = peer_shared(&cta_o[r][d], c);
        const float m_new = fmaxf(m_tot, m_c);
        const float fa = m_tot == -INFINITY ? 0.f : exp2f((m_tot - m_new) * sl2);
        const float fc = m_c == -INFINITY ? 0.f : exp2f((m_c - m_new) * sl2);
        l_tot = l_tot * fa + l_c * fc;
        o = o * fa + o_c * fc;
        m_tot = m_new;
      }
      const float value = o / l_tot;  // 0 / 0 = NaN for a row with no visible key, as the oracle gives
      unsigned char* dst = static_cast<unsigned char*>(prm.out) +
                           (batch * prm.o_strides.batch + head * prm.o_strides.head + static_cast<long long>(r) * prm.o_strides.row + d) * 2;
      if (kFp16) *reinterpret_cast<__half*>(dst) = __float2half_rn(value);
      else *reinterpret_cast<__nv_bfloat16*>(dst) = __float2bfloat16_rn(value);
      if (d == 0) prm.lse[static_cast<long long>(problem) * prm.t_q + r] = m_tot * prm.scale + logf(l_tot);
    }
  }
  if (split > 1) cluster_sync();  // no CTA leaves while CTA 0 may still be reading its shared memory
}

template <int D, bool kFp16, bool kMask, int R>
int launch_one(const Problem& p, const DecodeParams& prm) {
  cudaLaunchConfig_t config = {};
  config.gridDim = dim3(static_cast<unsigned>(p.bh * prm.split));
  config.blockDim = dim3(kThreads);
  config.stream = p.stream;
  cudaLaunchAttribute attribute[1];
  attribute[0].id = cudaLaunchAttributeClusterDimension;
  attribute[0].val.clusterDim.x = static_cast<unsigned>(prm.split);
  attribute[0].val.clusterDim.y = 1;
  attribute[0].val.clusterDim.z = 1;
  config.attrs = attribute;
  config.numAttrs = 1;
  LIMN_CUDA(cudaLaunchKernelEx(&config, sdpa_decode_kernel<D, kFp16, kMask, R>, prm), "launching the sdpa decode kernel");
  note_launches(1);
  return LIMN_B200_OK;
}

template <int D, bool kFp16, bool kMask>
int launch_rows(const Problem& p, const DecodeParams& prm) {
  switch (p.t_q) {
    case 1: return launch_one<D, kFp16, kMask, 1>(p, prm);
    case 2: return launch_one<D, kFp16, kMask, 2>(p, prm);
    case 3: return launch_one<D, kFp16, kMask, 3>(p, prm);
    default: return launch_one<D, kFp16, kMask, 4>(p, prm);
  }
}

template <int D>
int launch_d(const Problem& p, const DecodeParams& prm) {
  const bool fp16 = p.dtype == LIMN_B200_F16;
  if (p.mask) return fp16 ? launch_rows<D, true, true>(p, prm) : launch_rows<D, false, true>(p, prm);
  return fp16 ? launch_rows<D, true, false>(p, prm) : launch_rows<D, false, false>(p, prm);
}

}  // namespace

bool decode_serves(Op op, const Problem& p) {
  if (op != Op::Fwd) return false;
  if (p.dtype != LIMN_B200_BF16 && p.dtype != LIMN_B200_F16) return false;
  if (p.hd != p.hd_v || (p.hd != 64 && p.hd != 128)) return false;
  if (p.t_q > kMaxRows || p.causal) return false;  // (causal needs t_q == t_k: a prefill shape, however short)
  if (!(p.scale > 0.0) || p.bh > 0x7fffffffLL) return false;
  // 16-byte loads: aligned bases (a null pointer is refused before this is asked in earnest)
  const uintptr_t bases = reinterpret_cast<uintptr_t>(p.q) | reinterpret_cast<uintptr_t>(p.k) | reinterpret_cast<uintptr_t>(p.v);
  return (bases & 15u) == 0;
}

int decode_launch(const Problem& p) {
  DecodeParams prm;
  prm.q = p.q, prm.k = p.k, prm.v = p.v;
  prm.mask = static_cast<const unsigned short*>(p.mask);
  prm.out = p.out, prm.lse = static_cast<float*>(p.lse_out);
  prm.heads = p.heads > 0 ? p.heads : static_cast<int>(p.bh);
  prm.q_strides = operand_strides(p, kOpQ, prm.heads, p.t_q, p.hd);
  prm.k_strides = operand_strides(p, kOpK, prm.heads, p.t_k, p.hd);
  prm.v_strides = operand_strides(p, kOpV, prm.heads, p.t_k, p.hd);
  prm.o_strides = operand_strides(p, kOpOut, prm.heads, p.t_q, p.hd);
  {
    const long long all = prm.q_strides.batch | prm.q_strides.head | prm.q_strides.row | prm.k_strides.batch | prm.k_strides.head |
                          prm.k_strides.row | prm.v_strides.batch | prm.v_strides.head | prm.v_strides.row;
    if (all & 7) return fail(LIMN_B200_BAD_ARGUMENT, "sdpa: operand strides must be multiples of 8 elements");
  }
  prm.t_q = p.t_q, prm.t_k = p.t_k;
  prm.scale = static_cast<float>(p.scale);
  // One CTA per problem fills the GPU from a few hundred problems on (two CTAs fit an SM). Below that, 2, 4 or 8
  // CTAs share a problem, as long as each still has a full pass of keys (16 warps x 4 in flight x keys per warp load).
  int sms = 0;
  if (int rc = sm_count(&sms)) return rc;
  const int per_pass = kWarps * kUnroll * (32 / (p.hd / 8));
  int split = 1;
  while (split < 8 && p.bh * split * 2 <= 2LL * sms && (p.t_k + per_pass - 1) / per_pass >= split * 2) split *= 2;
  prm.split = split;
  return p.hd == 128 ? launch_d<128>(p, prm) : launch_d<64>(p, prm);
}

}  // namespace limn_b200
