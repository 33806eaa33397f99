// General fused-attention kernels: any float storage type, any head dims, optional key mask,
// rectangular t_q x t_k. These serve every problem the tcgen05 kernels do not take
// (float32 and float64 in particular, which have to be computed at their own width to meet
// the reference's 1e-5 / 1e-12 checks: tests/test_attention.py:250-255, limn/sdpa.py:279-291);
// the tiled kernels of sdpa_general_tiled.cu take over where a problem fills their tiles, and
// what stays here is float64, head dims above 256 and sides shorter than 16 rows.
//
// Shape of the work: one warp owns one row for the whole pass (a query row in the forward
// and the dQ pass, a key row in the dK/dV pass), so every total has exactly one owner, no
// float is ever added atomically and two runs give the same bits, as the reference's kernels
// promise (limn/cuda_emit.py:748-752). Inside a warp the 32 lanes each take one streamed row
// (a key, or a query in the dK/dV pass) for the dot products, and then share the head
// dimension (lane, lane + 32, ...) when the row's totals are updated.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <cmath>
#include <cstdint>
#include <type_traits>

#include "common.h"

namespace limn_b200 {
namespace {

constexpr int kWarps = 8;  // rows per block, one per warp
constexpr unsigned kFull = 0xffffffffu;

template <typename T>
__device__ __forceinline__ float widen(T x);
template <>
__device__ __forceinline__ float widen<float>(float x) { return x; }
template <>
__device__ __forceinline__ float widen<__half>(__half x) { return __half2float(x); }
template <>
__device__ __forceinline__ float widen<__nv_bfloat16>(__nv_bfloat16 x) { return __bfloat162float(x); }

template <typename T, typename C>
__device__ __forceinline__ C load(const T* p) {
  if constexpr (sizeof(T) == 8) {
    return *p;
  } else {
    return static_cast<C>(widen<T>(*p));
  }
}

template <typename T, typename C>
__device__ __forceinline__ void store(T* p, C x) {
  if constexpr (sizeof(T) == 8) {
    *p = x;
  } else if constexpr (sizeof(T) == 4) {
    *p = x;
  } else if constexpr (std::is_same<T, __half>::value) {
    *p = __float2half_rn(x);
  } else {
    *p = __float2bfloat16_rn(x);
  }
}

__device__ __forceinline__ float gexp(float x) { return expf(x); }
__device__ __forceinline__ double gexp(double x) { return exp(x); }
__device__ __forceinline__ float glog(float x) { return logf(x); }
__device__ __forceinline__ double glog(double x) { return log(x); }

template <typename C>
__device__ __forceinline__ C warp_max(C x) {
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) {
    C other = __shfl_xor_sync(kFull, x, off);
    x = other > x ? other : x;
  }
  return x;
}

template <typename C>
__device__ __forceinline__ C warp_sum(C x) {
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) x += __shfl_xor_sync(kFull, x, off);
  return x;
}

template <typename C>
__device__ __forceinline__ C neg_inf() {
  return -static_cast<C>(INFINITY);
}

// dot of a row held in shared memory (compute width) with a row in global memory
template <typename T, typename C>
__device__ __forceinline__ C dot_row(const C* held, const T* row, int n) {
  C acc = 0;
  for (int d = 0; d < n; ++d) acc += held[d] * load<T, C>(row + d);
  return acc;
}

// ---- forward: O and L for one query row per warp (oracle: limn/sdpa.py:114-137) ----
template <typename T, typename C, int ND>
__global__ void __launch_bounds__(kWarps * 32)
general_fwd_kernel(const T* __restrict__ q, const T* __restrict__ k, const T* __restrict__ v,
                   const T* __restrict__ mask, T* __restrict__ out, C* __restrict__ lse, long long rows,
                   int t_q, int t_k, int hd, int hd_v, int causal, C scale) {
  extern __shared__ __align__(16) unsigned char shared_raw[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long row = static_cast<long long>(blockIdx.x) * kWarps + warp;
  if (row >= rows) return;  // whole warp leaves together; there is no block-wide barrier below
  const long long b = row / t_q;
  const int i = static_cast<int>(row - b * t_q);
  C* q_held = reinterpret_cast<C*>(shared_raw) + static_cast<size_t>(warp) * hd;
  for (int d = lane; d < hd; d += 32) q_held[d] = load<T, C>(q + row * hd + d);
  __syncwarp();

  const T* k_base = k + b * t_k * hd;
  const T* v_base = v + b * t_k * hd_v;
  const T* m_base = mask ? mask + b * t_k : nullptr;
  C acc[ND];
#pragma unroll
  for (int c = 0; c < ND; ++c) acc[c] = 0;
  C top = neg_inf<C>(), denom = 0;
  const int keys_end = causal ? i + 1 : t_k;
  for (int j0 = 0; j0 < keys_end; j0 += 32) {
    const int j = j0 + lane;
    bool seen = j < keys_end;
    if (seen && m_base) seen = load<T, C>(m_base + j) != C(0);
    C s = seen ? dot_row<T, C>(q_held, k_base + static_cast<long long>(j) * hd, hd) * scale : neg_inf<C>();
    const C span_top = warp_max(s);
    if (span_top == neg_inf<C>()) continue;  // every key of this span is hidden; uniform across the warp
    const C raised = span_top > top ? span_top : top;
    const C shrink = gexp(top - raised);  // exp(-inf) = 0 on the first visible span
    const C w = seen ? gexp(s - raised) : C(0);
    denom = denom * shrink + warp_sum(w);
#pragma unroll
    for (int c = 0; c < ND; ++c) acc[c] *= shrink;
    const int span = min(32, keys_end - j0);
    for (int jj = 0; jj < span; ++jj) {
      const C wj = __shfl_sync(kFull, w, jj);
      if (wj == C(0)) continue;  // uniform: a hidden key adds nothing
      const T* v_row = v_base + static_cast<long long>(j0 + jj) * hd_v;
#pragma unroll
      for (int c = 0; c < ND; ++c) {
        const int d = lane + 32 * c;
        if (d < hd_v) acc[c] += wj * load<T, C>(v_row + d);
      }
    }
    top = raised;
  }
#pragma unroll
  for (int c = 0; c < ND; ++c) {
    const int d = lane + 32 * c;
    if (d < hd_v) store<T, C>(out + row * hd_v + d, acc[c] / denom);  // 0/0 = NaN for a row with no key
  }
  if (lane == 0) lse[row] = top + glog(denom);
}

// ---- dQ for one query row per warp (oracle: limn/sdpa.py:157-170) ----
template <typename T, typename C, int ND>
__global__ void __launch_bounds__(kWarps * 32)
general_bwd_q_kernel(const T* __restrict__ q, const T* __restrict__ k, const T* __restrict__ v,
                     const T* __restrict__ dout, const C* __restrict__ lse, const C* __restrict__ delta,
                     const T* __restrict__ mask, T* __restrict__ dq, long long rows, int t_q, int t_k, int hd,
                     int hd_v, int causal, C scale) {
  extern __shared__ __align__(16) unsigned char shared_raw[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long row = static_cast<long long>(blockIdx.x) * kWarps + warp;
  if (row >= rows) return;
  const long long b = row / t_q;
  const int i = static_cast<int>(row - b * t_q);
  C* q_held = reinterpret_cast<C*>(shared_raw) + static_cast<size_t>(warp) * (hd + hd_v);
  C* do_held = q_held + hd;
  for (int d = lane; d < hd; d += 32) q_held[d] = load<T, C>(q + row * hd + d);
  for (int d = lane; d < hd_v; d += 32) do_held[d] = load<T, C>(dout + row * hd_v + d);
  __syncwarp();
  const C row_lse = lse[row], row_delta = delta[row];

  const T* k_base = k + b * t_k * hd;
  const T* v_base = v + b * t_k * hd_v;
  const T* m_base = mask ? mask + b * t_k : nullptr;
  C acc[ND];
#pragma unroll
  for (int c = 0; c < ND; ++c) acc[c] = 0;
  const int keys_end = causal ? i + 1 : t_k;
  for (int j0 = 0; j0 < keys_end; j0 += 32) {
    const int j = j0 + lane;
    bool seen = j < keys_end;
    if (seen && m_base) seen = load<T, C>(m_base + j) != C(0);
    C ds = 0;
    if (seen) {
      const C s = dot_row<T, C>(q_held, k_base + static_cast<long long>(j) * hd, hd);
      const C dp = dot_row<T, C>(do_held, v_base + static_cast<long long>(j) * hd_v, hd_v);
      const C p = gexp(s * scale - row_lse);
      ds = p * (dp - row_delta) * scale;
    }
    if (!__any_sync(kFull, seen)) continue;
    const int span = min(32, keys_end - j0);
    for (int jj = 0; jj < span; ++jj) {
      const C dsj = __shfl_sync(kFull, ds, jj);
      const T* k_row = k_base + static_cast<long long>(j0 + jj) * hd;
#pragma unroll
      for (int c = 0; c < ND; ++c) {
        const int d = lane + 32 * c;
        if (d < hd) acc[c] += dsj * load<T, C>(k_row + d);
      }
    }
  }
#pragma unroll
  for (int c = 0; c < ND; ++c) {
    const int d = lane + 32 * c;
    if (d < hd) store<T, C>(dq + row * hd + d, acc[c]);
  }
}

// ---- dK and dV for one key row per warp (oracle: limn/sdpa.py:190-203) ----
template <typename T, typename C, int ND>
__global__ void __launch_bounds__(kWarps * 32)
general_bwd_kv_kernel(const T* __restrict__ q, const T* __restrict__ k, const T* __restrict__ v,
                      const T* __restrict__ dout, const C* __restrict__ lse, const C* __restrict__ delta,
                      const T* __restrict__ mask, T* __restrict__ dk, T* __restrict__ dv, long long rows, int t_q,
                      int t_k, int hd, int hd_v, int causal, C scale) {
  extern __shared__ __align__(16) unsigned char shared_raw[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long row = static_cast<long long>(blockIdx.x) * kWarps + warp;  // over bh * t_k
  if (row >= rows) return;
  const long long b = row / t_k;
  const int j = static_cast<int>(row - b * t_k);
  C* k_held = reinterpret_cast<C*>(shared_raw) + static_cast<size_t>(warp) * (hd + hd_v);
  C* v_held = k_held + hd;
  for (int d = lane; d < hd; d += 32) k_held[d] = load<T, C>(k + row * hd + d);
  for (int d = lane; d < hd_v; d += 32) v_held[d] = load<T, C>(v + row * hd_v + d);
  __syncwarp();
  const bool live = mask ? load<T, C>(mask + row) != C(0) : true;

  const T* q_base = q + b * t_q * hd;
  const T* do_base = dout + b * t_q * hd_v;
  const C* lse_base = lse + b * t_q;
  const C* delta_base = delta + b * t_q;
  C acc_k[ND], acc_v[ND];
#pragma unroll
  for (int c = 0; c < ND; ++c) acc_k[c] = 0, acc_v[c] = 0;
  const int first = causal ? j : 0;  // the first query that sees this key
  if (live) {
    for (int i0 = first; i0 < t_q; i0 += 32) {
      const int i = i0 + lane;
      C p = 0, ds = 0;
      if (i < t_q) {
        const C s = dot_row<T, C>(k_held, q_base + static_cast<long long>(i) * hd, hd);
        const C dp = dot_row<T, C>(v_held, do_base + static_cast<long long>(i) * hd_v, hd_v);
        p = gexp(s * scale - lse_base[i]);
        ds = p * (dp - delta_base[i]) * scale;
      }
      const int span = min(32, t_q - i0);
      for (int ii = 0; ii < span; ++ii) {
        const C pi = __shfl_sync(kFull, p, ii);
        const C dsi = __shfl_sync(kFull, ds, ii);
        const T* do_row = do_base + static_cast<long long>(i0 + ii) * hd_v;
        const T* q_row = q_base + static_cast<long long>(i0 + ii) * hd;
#pragma unroll
        for (int c = 0; c < ND; ++c) {
          const int d = lane + 32 * c;
          if (d < hd_v) acc_v[c] += pi * load<T, C>(do_row + d);
          if (d < hd) acc_k[c] += dsi * load<T, C>(q_row + d);
        }
      }
    }
  }
#pragma unroll
  for (int c = 0; c < ND; ++c) {
    const int d = lane + 32 * c;
    if (d < hd) store<T, C>(dk + row * hd + d, acc_k[c]);
    if (d < hd_v) store<T, C>(dv + row * hd_v + d, acc_v[c]);
  }
}

// ---- delta = sum_d dO * O, one row per warp (limn/tensor.py:705-706) ----
template <typename T, typename C>
__global__ void __launch_bounds__(kWarps * 32)
row_dot_kernel(const T* __restrict__ out, const T* __restrict__ dout, C* __restrict__ delta, long long rows,
               int hd_v) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long row = static_cast<long long>(blockIdx.x) * kWarps + warp;
  if (row >= rows) return;
  C acc = 0;
  for (int d = lane; d < hd_v; d += 32) acc += load<T, C>(dout + row * hd_v + d) * load<T, C>(out + row * hd_v + d);
  acc = warp_sum(acc);
  if (lane == 0) delta[row] = acc;
}


// The same row dot for 2-byte storage when a row is a whole number of 16-byte pieces: each
// thread takes 8 elements of one row with one 16-byte load from each tensor, and the
// threads of a row (kLanes of them, the power of two that holds the row's hd_v / 8 pieces, consecutive
// lanes; those beyond the row's pieces idle) fold their partial sums with shuffles. Both tensors are read
// exactly once at full sector width, so the kernel runs at memory speed; the generic kernel above serves
// every other shape.
template <bool kFp16, int kLanes>
__global__ void __launch_bounds__(256)
row_dot16_kernel(const uint4* __restrict__ out, const uint4* __restrict__ dout, float* __restrict__ delta,
                 long long rows, int pieces, int heads, int t) {
  const long long slot = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  const long long row = slot / kLanes;
  const int within = static_cast<int>(slot - row * kLanes);
  float acc = 0.f;
  if (row < rows && within < pieces) {
    const long long piece = row * pieces + within;  // 16-byte piece index
    const uint4 a = out[piece], b = dout[piece];
    const uint32_t aw[4] = {a.x, a.y, a.z, a.w}, bw[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      float a0, a1, b0, b1;
      if (kFp16) {
        const float2 fa = __half22float2(*reinterpret_cast<const __half2*>(&aw[i]));
        const float2 fb = __half22float2(*reinterpret_cast<const __half2*>(&bw[i]));
        a0 = fa.x, a1 = fa.y, b0 = fb.x, b1 = fb.y;
      } else {
        a0 = __uint_as_float(aw[i] << 16), a1 = __uint_as_float(aw[i] & 0xffff0000u);
        b0 = __uint_as_float(bw[i] << 16), b1 = __uint_as_float(bw[i] & 0xffff0000u);
      }
      acc = fmaf(a0, b0, acc);
      acc = fmaf(a1, b1, acc);
    }
  }
#pragma unroll
  for (int off = kLanes / 2; off > 0; off >>= 1) acc += __shfl_xor_sync(kFull, acc, off);
  if (row < rows && within == 0) {
    long long to = row;
    if (heads > 0) {
      // rows lie in memory as (batch, t, head); delta is (batch, head, t)
      const long long bt = row / heads;
      const int h = static_cast<int>(row - bt * heads);
      const long long b = bt / t;
      to = (b * heads + h) * t + (bt - b * t);
    }
    delta[to] = acc;
  }
}

template <bool kFp16>
bool launch_row_dot16(const void* out, const void* dout, void* delta, long long rows, int hd_v, cudaStream_t stream,
                      int heads = 0, int t = 0) {
  const int pieces = hd_v / 8;
  if (hd_v % 8 != 0 || pieces > 32) return false;
  if ((reinterpret_cast<uintptr_t>(out) | reinterpret_cast<uintptr_t>(dout)) & 15u) return false;
  int lanes = 1;
  while (lanes < pieces) lanes *= 2;
  const long long slots = rows * lanes;
  const long long blocks = (slots + 255) / 256;
  if (blocks > 0x7fffffffLL) return false;
  const dim3 grid(static_cast<unsigned>(blocks)), block(256);
  auto a = static_cast<const uint4*>(out), b = static_cast<const uint4*>(dout);
  auto d = static_cast<float*>(delta);
  switch (lanes) {
    case 1: row_dot16_kernel<kFp16, 1><<<grid, block, 0, stream>>>(a, b, d, rows, pieces, heads, t); break;
    case 2: row_dot16_kernel<kFp16, 2><<<grid, block, 0, stream>>>(a, b, d, rows, pieces, heads, t); break;
    case 4: row_dot16_kernel<kFp16, 4><<<grid, block, 0, stream>>>(a, b, d, rows, pieces, heads, t); break;
    case 8: row_dot16_kernel<kFp16, 8><<<grid, block, 0, stream>>>(a, b, d, rows, pieces, heads, t); break;
    case 16: row_dot16_kernel<kFp16, 16><<<grid, block, 0, stream>>>(a, b, d, rows, pieces, heads, t); break;
    default: row_dot16_kernel<kFp16, 32><<<grid, block, 0, stream>>>(a, b, d, rows, pieces, heads, t); break;
  }
  return true;
}

template <typename T, typename C, int ND>
int launch_typed(Op op, const Problem& p) {
  const long long rows = p.bh * (op == Op::BwdKV ? p.t_k : p.t_q);
  const long long blocks = (rows + kWarps - 1) / kWarps;
  if (blocks > 0x7fffffffLL) return fail(LIMN_B200_UNSUPPORTED, "sdpa: %lld rows need more blocks than one grid holds", rows);
  const size_t shared = static_cast<size_t>(kWarps) * sizeof(C) * (op == Op::Fwd ? p.hd : p.hd + p.hd_v);
  const dim3 grid(static_cast<unsigned>(blocks)), block(kWarps * 32);
  const C scale = static_cast<C>(p.scale);
  auto as = [](const void* x) { return static_cast<const T*>(x); };
  cudaError_t attr = cudaSuccess;
  switch (op) {
    case Op::Fwd:
      if (shared > 48 * 1024)
        attr = cudaFuncSetAttribute(general_fwd_kernel<T, C, ND>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)shared);
      LIMN_CUDA(attr, "sizing shared memory for the general sdpa kernel");
      general_fwd_kernel<T, C, ND><<<grid, block, shared, p.stream>>>(
          as(p.q), as(p.k), as(p.v), as(p.mask), static_cast<T*>(p.out), static_cast<C*>(p.lse_out), rows, p.t_q,
          p.t_k, p.hd, p.hd_v, p.causal, scale);
      break;
    case Op::BwdQ:
      if (shared > 48 * 1024)
        attr = cudaFuncSetAttribute(general_bwd_q_kernel<T, C, ND>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)shared);
      LIMN_CUDA(attr, "sizing shared memory for the general sdpa_bwd_q kernel");
      general_bwd_q_kernel<T, C, ND><<<grid, block, shared, p.stream>>>(
          as(p.q), as(p.k), as(p.v), as(p.dout), static_cast<const C*>(p.lse_in), static_cast<const C*>(p.delta),
          as(p.mask), static_cast<T*>(p.dq), rows, p.t_q, p.t_k, p.hd, p.hd_v, p.causal, scale);
      break;
    case Op::BwdKV:
      if (shared > 48 * 1024)
        attr = cudaFuncSetAttribute(general_bwd_kv_kernel<T, C, ND>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)shared);
      LIMN_CUDA(attr, "sizing shared memory for the general sdpa_bwd_kv kernel");
      general_bwd_kv_kernel<T, C, ND><<<grid, block, shared, p.stream>>>(
          as(p.q), as(p.k), as(p.v), as(p.dout), static_cast<const C*>(p.lse_in), static_cast<const C*>(p.delta),
          as(p.mask), static_cast<T*>(p.dk), static_cast<T*>(p.dv), rows, p.t_q, p.t_k, p.hd, p.hd_v, p.causal,
          scale);
      break;
  }
  LIMN_CUDA(cudaGetLastError(), "launching a general sdpa kernel");
  note_launches(1);
  return LIMN_B200_OK;
}

template <typename T, typename C>
int launch_width(Op op, const Problem& p) {
  const int widest = p.hd > p.hd_v ? p.hd : p.hd_v;
  if (widest <= 32) return launch_typed<T, C, 1>(op, p);
  if (widest <= 64) return launch_typed<T, C, 2>(op, p);
  if (widest <= 128) return launch_typed<T, C, 4>(op, p);
  if (widest <= 256) return launch_typed<T, C, 8>(op, p);
  if (widest <= 512) return launch_typed<T, C, 16>(op, p);
  if (widest <= 1024) return launch_typed<T, C, 32>(op, p);
  return fail(LIMN_B200_UNSUPPORTED, "sdpa: head dims up to 1024 are served, got hd=%d hd_v=%d", p.hd, p.hd_v);
}

}  // namespace

int general_launch(Op op, const Problem& p) {
  if (general_tiled_serves(op, p)) return general_tiled_launch(op, p);
  switch (p.dtype) {
    case LIMN_B200_F32: return launch_width<float, float>(op, p);
    case LIMN_B200_F16: return launch_width<__half, float>(op, p);
    case LIMN_B200_BF16: return launch_width<__nv_bfloat16, float>(op, p);
    case LIMN_B200_F64: return launch_width<double, double>(op, p);
  }
  return fail(LIMN_B200_BAD_ARGUMENT, "sdpa: unknown dtype code %d", p.dtype);
}

int general_delta(const void* out, const void* dout, void* delta, int dtype, long long rows, int hd_v,
                  cudaStream_t stream) {
  const long long blocks = (rows + kWarps - 1) / kWarps;
  if (blocks > 0x7fffffffLL) return fail(LIMN_B200_UNSUPPORTED, "sdpa_delta: %lld rows need more blocks than one grid holds", rows);
  const dim3 grid(static_cast<unsigned>(blocks)), block(kWarps * 32);
  if ((dtype == LIMN_B200_F16 && launch_row_dot16<true>(out, dout, delta, rows, hd_v, stream)) ||
      (dtype == LIMN_B200_BF16 && launch_row_dot16<false>(out, dout, delta, rows, hd_v, stream))) {
    LIMN_CUDA(cudaGetLastError(), "launching the row-dot kernel");
    note_launches(1);
    return LIMN_B200_OK;
  }
  switch (dtype) {
    case LIMN_B200_F32:
      row_dot_kernel<float, float><<<grid, block, 0, stream>>>((const float*)out, (const float*)dout, (float*)delta, rows, hd_v);
      break;
    case LIMN_B200_F16:
      row_dot_kernel<__half, float><<<grid, block, 0, stream>>>((const __half*)out, (const __half*)dout, (float*)delta, rows, hd_v);
      break;
    case LIMN_B200_BF16:
      row_dot_kernel<__nv_bfloat16, float><<<grid, block, 0, stream>>>((const __nv_bfloat16*)out, (const __nv_bfloat16*)dout, (float*)delta, rows, hd_v);
      break;
    case LIMN_B200_F64:
      row_dot_kernel<double, double><<<grid, block, 0, stream>>>((const double*)out, (const double*)dout, (double*)delta, rows, hd_v);
      break;
    default:
      return fail(LIMN_B200_BAD_ARGUMENT, "sdpa_delta: unknown dtype code %d", dtype);
  }
  LIMN_CUDA(cudaGetLastError(), "launching the row-dot kernel");
  note_launches(1);
  return LIMN_B200_OK;
}

int general_delta_bthd(const void* out, const void* dout, void* delta, int dtype, int batch, int heads, int t, int hd_v,
                       cudaStream_t stream) {
  const long long rows = static_cast<long long>(batch) * heads * t;
  if ((dtype == LIMN_B200_F16 && launch_row_dot16<true>(out, dout, delta, rows, hd_v, stream, heads, t)) ||
      (dtype == LIMN_B200_BF16 && launch_row_dot16<false>(out, dout, delta, rows, hd_v, stream, heads, t))) {
    LIMN_CUDA(cudaGetLastError(), "launching the row-dot kernel");
    note_launches(1);
    return LIMN_B200_OK;
  }
  return fail(LIMN_B200_UNSUPPORTED, "sdpa_delta: the (batch, t, heads, hd) layout is served for f16/bf16 with hd_v a multiple of 8 up to 256");
}

}  // namespace limn_b200
