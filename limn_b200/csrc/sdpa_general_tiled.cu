// Tiled SIMT fused-attention kernels: float32, float16 and bfloat16 storage computed in float32 on the
// CUDA cores, head dims up to 256, optional key mask, rectangular t_q x t_k. They serve what the tcgen05
// kernels leave (float32 above all, which has to be computed at its own width to meet the reference's 1e-5
// check: tests/test_attention.py:250-255) whenever the problem is large enough to fill a tile; the one-row-
// per-warp kernels in sdpa_general.cu keep float64, wider heads and short sequences.
//
// Shape of the work: a block of 256 threads owns 64 rows (query rows in the forward and the dQ pass, key rows
// in the dK/dV pass) and streams the other side through shared memory in tiles of BN rows (64, 32 or 16 of them
// for head dims up to 64, 128 or 256). Every tile is two small matrix products on a 16 x 16 thread grid: scores
// (rows x streamed rows, contraction over the head dim, a 4 x BN/16 micro-tile per thread read from shared memory
// as float4), then, after the scores went through shared memory, the update of the rows' totals (contraction
// over the streamed rows, 4 x HD/16 per thread). Each total has one owner and a fixed summation order, no float
// is added atomically: two runs give the same bits, as the reference's kernels promise
// (limn/cuda_emit.py:748-752).
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include <cmath>
#include <cstdint>

#include "common.h"

namespace limn_b200 {
namespace {

constexpr int kThreads = 256;
constexpr int kBM = 64;   // rows a block owns
constexpr int kPad = 4;   // floats of padding per shared-memory row: keeps float4 reads of 16 rows on distinct banks
constexpr unsigned kFull = 0xffffffffu;

template <typename T>
__device__ __forceinline__ float widen(T x);
template <>
__device__ __forceinline__ float widen<float>(float x) { return x; }
template <>
__device__ __forceinline__ float widen<__half>(__half x) { return __half2float(x); }
template <>
__device__ __forceinline__ float widen<__nv_bfloat16>(__nv_bfloat16 x) { return __bfloat162float(x); }

template <typename T>
__device__ __forceinline__ T narrow(float x);
template <>
__device__ __forceinline__ float narrow<float>(float x) { return x; }
template <>
__device__ __forceinline__ __half narrow<__half>(float x) { return __float2half_rn(x); }
template <>
__device__ __forceinline__ __nv_bfloat16 narrow<__nv_bfloat16>(float x) { return __float2bfloat16_rn(x); }

// Rows [first, first + R) of a (rows, width) matrix into dst[R][HD + kPad] as float; rows past the matrix and
// columns past `width` become zero, so the products below may run over whole tiles.
template <typename T, int HD, int R>
__device__ __forceinline__ void stage(float* dst, const T* src, int first, int rows, int width, bool wide) {
  constexpr int LD = HD + kPad;
  constexpr int V = 16 / sizeof(T);  // elements per 16-byte piece
  if (wide) {                        // width is a whole number of pieces and the base is 16-byte aligned
    constexpr int per_row = HD / V;
    for (int e = threadIdx.x; e < R * per_row; e += kThreads) {
      const int r = e / per_row, c = (e - r * per_row) * V;
      float x[V];
      if (first + r < rows && c < width) {
        const uint4 raw = *reinterpret_cast<const uint4*>(src + static_cast<long long>(first + r) * width + c);
        const T* t = reinterpret_cast<const T*>(&raw);
#pragma unroll
        for (int i = 0; i < V; ++i) x[i] = widen<T>(t[i]);
      } else {
#pragma unroll
        for (int i = 0; i < V; ++i) x[i] = 0.f;
      }
#pragma unroll
      for (int i = 0; i < V; i += 4)
        *reinterpret_cast<float4*>(dst + r * LD + c + i) = make_float4(x[i], x[i + 1], x[i + 2], x[i + 3]);
    }
  } else {
    for (int e = threadIdx.x; e < R * HD; e += kThreads) {
      const int r = e / HD, c = e - r * HD;
      dst[r * LD + c] = (first + r < rows && c < width) ? widen<T>(src[static_cast<long long>(first + r) * width + c]) : 0.f;
    }
  }
}

// acc[a][b] += sum_d A[row0 + a][d] * B[col0 + 16 b][d] for d < depth (a multiple of 4)
template <int LD, int NB>
__device__ __forceinline__ void dot_tiles(float (&acc)[4][NB], const float* a_rows, const float* b_rows, int depth) {
  for (int d = 0; d < depth; d += 4) {
    float4 av[4], bv[NB];
#pragma unroll
    for (int a = 0; a < 4; ++a) av[a] = *reinterpret_cast<const float4*>(a_rows + a * LD + d);
#pragma unroll
    for (int b = 0; b < NB; ++b) bv[b] = *reinterpret_cast<const float4*>(b_rows + b * 16 * LD + d);
#pragma unroll
    for (int a = 0; a < 4; ++a)
#pragma unroll
      for (int b = 0; b < NB; ++b) {
        acc[a][b] = fmaf(av[a].x, bv[b].x, acc[a][b]);
        acc[a][b] = fmaf(av[a].y, bv[b].y, acc[a][b]);
        acc[a][b] = fmaf(av[a].z, bv[b].z, acc[a][b]);
        acc[a][b] = fmaf(av[a].w, bv[b].w, acc[a][b]);
      }
  }
}

// Columns of the head dim one thread owns in the second product: NV = HD / 16 of them, as NV / VW vectors of VW
// consecutive floats, vector c of thread tx starting at column c * 16 * VW + tx * VW.
template <int HD>
struct Cols {
  static constexpr int NV = HD / 16;
  static constexpr int VW = NV < 4 ? NV : 4;
  static constexpr int NC = NV / VW;
  __device__ static __forceinline__ int at(int tx, int i) { return (i / VW) * 16 * VW + tx * VW + (i % VW); }
};

// acc[a][i] += sum_j W[row0 + a][j] * X[j][col(i)] for j < BN
template <int HD, int BN>
__device__ __forceinline__ void weigh_rows(float (&acc)[4][HD / 16], const float* w_rows, const float* x, int tx) {
  using C = Cols<HD>;
  constexpr int LD = HD + kPad, LP = BN + kPad;
#pragma unroll 2
  for (int j = 0; j < BN; j += 4) {
    float4 w4[4];
#pragma unroll
    for (int a = 0; a < 4; ++a) w4[a] = *reinterpret_cast<const float4*>(w_rows + a * LP + j);
#pragma unroll
    for (int jj = 0; jj < 4; ++jj) {
      float xv[C::NV];
#pragma unroll
      for (int c = 0; c < C::NC; ++c) {
        const float* from = x + (j + jj) * LD + c * 16 * C::VW + tx * C::VW;
        if constexpr (C::VW == 4) {
          const float4 t = *reinterpret_cast<const float4*>(from);
          xv[c * 4] = t.x, xv[c * 4 + 1] = t.y, xv[c * 4 + 2] = t.z, xv[c * 4 + 3] = t.w;
        } else if constexpr (C::VW == 2) {
          const float2 t = *reinterpret_cast<const float2*>(from);
          xv[c * 2] = t.x, xv[c * 2 + 1] = t.y;
        } else {
          xv[c] = *from;
        }
      }
#pragma unroll
      for (int a = 0; a < 4; ++a) {
        const float w = jj == 0 ? w4[a].x : jj == 1 ? w4[a].y : jj == 2 ? w4[a].z : w4[a].w;
#pragma unroll
        for (int i = 0; i < C::NV; ++i) acc[a][i] = fmaf(w, xv[i], acc[a][i]);
      }
    }
  }
}

// the rows this thread owns of a block's result, written where they are real
template <typename T, int HD>
__device__ __forceinline__ void store_rows(T* dst, const float (&acc)[4][HD / 16], long long first_row, int rows_here,
                                           int width, int ty, int tx) {
  using C = Cols<HD>;
#pragma unroll
  for (int a = 0; a < 4; ++a) {
    const int r = ty * 4 + a;
    if (r >= rows_here) continue;
#pragma unroll
    for (int i = 0; i < C::NV; ++i) {
      const int col = C::at(tx, i);
      if (col < width) dst[(first_row + r) * width + col] = narrow<T>(acc[a][i]);
    }
  }
}

__device__ __forceinline__ float group_max(float x) {  // over the 16 threads that share a row
#pragma unroll
  for (int off = 8; off > 0; off >>= 1) x = fmaxf(x, __shfl_xor_sync(kFull, x, off));
  return x;
}
__device__ __forceinline__ float group_sum(float x) {
#pragma unroll
  for (int off = 8; off > 0; off >>= 1) x += __shfl_xor_sync(kFull, x, off);
  return x;
}

struct Args {
  const void *q, *k, *v, *mask, *dout;
  const float *lse_in, *delta;
  void *out, *dq, *dk, *dv;
  float* lse_out;
  int tiles;  // blocks per problem
  int t_q, t_k, hd, hd_v, causal;
  float scale;
  bool wide_qk, wide_v;  // 16-byte loads are safe for (q, k) and for (v, dO)
};

// ---- forward: O and L for 64 query rows (oracle: limn/sdpa.py:114-137) ----
template <typename T, int HD, int BN>
__global__ void __launch_bounds__(kThreads) tiled_fwd_kernel(const Args g) {
  constexpr int LD = HD + kPad, LP = BN + kPad, NB = BN / 16, NV = HD / 16;
  extern __shared__ __align__(16) float shared[];
  float* qs = shared;
  float* ks = qs + kBM * LD;
  float* vs = ks + BN * LD;
  float* ps = vs + BN * LD;
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  const long long b = blockIdx.x / g.tiles;
  const int i0 = (g.tiles - 1 - static_cast<int>(blockIdx.x - b * g.tiles)) * kBM;  // long causal rows first
  const T* q = static_cast<const T*>(g.q) + b * g.t_q * g.hd;
  const T* k = static_cast<const T*>(g.k) + b * g.t_k * g.hd;
  const T* v = static_cast<const T*>(g.v) + b * g.t_k * g.hd_v;
  const T* mask = g.mask ? static_cast<const T*>(g.mask) + b * g.t_k : nullptr;
  const int depth = (g.hd + 3) & ~3;

  stage<T, HD, kBM>(qs, q, i0, g.t_q, g.hd, g.wide_qk);
  float top[4], denom[4], acc[4][NV];
#pragma unroll
  for (int a = 0; a < 4; ++a) {
    top[a] = -INFINITY, denom[a] = 0.f;
#pragma unroll
    for (int i = 0; i < NV; ++i) acc[a][i] = 0.f;
  }
  const int keys_end = g.causal ? min(g.t_k, i0 + kBM) : g.t_k;
  for (int j0 = 0; j0 < keys_end; j0 += BN) {
    __syncthreads();  // the tile before this one has been read by everyone
    stage<T, HD, BN>(ks, k, j0, g.t_k, g.hd, g.wide_qk);
    stage<T, HD, BN>(vs, v, j0, g.t_k, g.hd_v, g.wide_v);
    bool open[NB];
#pragma unroll
    for (int c = 0; c < NB; ++c) {
      const int j = j0 + tx + 16 * c;
      open[c] = j < g.t_k && (!mask || widen<T>(mask[j]) != 0.f);
    }
    __syncthreads();
    float s[4][NB];
#pragma unroll
    for (int a = 0; a < 4; ++a)
#pragma unroll
      for (int c = 0; c < NB; ++c) s[a][c] = 0.f;
    dot_tiles<LD, NB>(s, qs + ty * 4 * LD, ks + tx * LD, depth);
#pragma unroll
    for (int a = 0; a < 4; ++a) {
      const int i = i0 + ty * 4 + a;
      float tile_top = -INFINITY;
#pragma unroll
      for (int c = 0; c < NB; ++c) {
        const bool seen = open[c] && (!g.causal || j0 + tx + 16 * c <= i);
        s[a][c] = seen ? s[a][c] * g.scale : -INFINITY;
        tile_top = fmaxf(tile_top, s[a][c]);
      }
      const float raised = fmaxf(top[a], group_max(tile_top));
      float shrink = 1.f;
      if (raised == -INFINITY) {  // no key of this row seen so far: nothing to add, nothing to rescale
#pragma unroll
        for (int c = 0; c < NB; ++c) s[a][c] = 0.f;
      } else {
        shrink = expf(top[a] - raised);  // exp(-inf) = 0 on the first visible tile
#pragma unroll
        for (int c = 0; c < NB; ++c) s[a][c] = expf(s[a][c] - raised);
      }
      float added = 0.f;
#pragma unroll
      for (int c = 0; c < NB; ++c) {
        added += s[a][c];
        ps[(ty * 4 + a) * LP + tx + 16 * c] = s[a][c];
      }
      denom[a] = denom[a] * shrink + added;  // this thread's share; the shares meet after the last tile
#pragma unroll
      for (int i2 = 0; i2 < NV; ++i2) acc[a][i2] *= shrink;
      top[a] = raised;
    }
    __syncthreads();
    weigh_rows<HD, BN>(acc, ps + ty * 4 * LP, vs, tx);
  }
  const int rows_here = min(kBM, g.t_q - i0);
#pragma unroll
  for (int a = 0; a < 4; ++a) {
    const float total = group_sum(denom[a]);
#pragma unroll
    for (int i = 0; i < NV; ++i) acc[a][i] = acc[a][i] / total;  // 0/0 = NaN for a row with no key, as the oracle has it
    const int r = ty * 4 + a;
    if (tx == 0 && r < rows_here) g.lse_out[b * g.t_q + i0 + r] = top[a] + logf(total);
  }
  store_rows<T, HD>(static_cast<T*>(g.out), acc, b * g.t_q + i0, rows_here, g.hd_v, ty, tx);
}

// ---- dQ for 64 query rows (oracle: limn/sdpa.py:157-170) ----
template <typename T, int HD, int BN>
__global__ void __launch_bounds__(kThreads) tiled_bwd_q_kernel(const Args g) {
  constexpr int LD = HD + kPad, LP = BN + kPad, NB = BN / 16, NV = HD / 16;
  extern __shared__ __align__(16) float shared[];
  float* qs = shared;
  float* dos = qs + kBM * LD;
  float* ks = dos + kBM * LD;
  float* vs = ks + BN * LD;
  float* ss = vs + BN * LD;
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  const long long b = blockIdx.x / g.tiles;
  const int i0 = (g.tiles - 1 - static_cast<int>(blockIdx.x - b * g.tiles)) * kBM;
  const T* q = static_cast<const T*>(g.q) + b * g.t_q * g.hd;
  const T* k = static_cast<const T*>(g.k) + b * g.t_k * g.hd;
  const T* v = static_cast<const T*>(g.v) + b * g.t_k * g.hd_v;
  const T* dout = static_cast<const T*>(g.dout) + b * g.t_q * g.hd_v;
  const T* mask = g.mask ? static_cast<const T*>(g.mask) + b * g.t_k : nullptr;
  const int depth = (g.hd + 3) & ~3, depth_v = (g.hd_v + 3) & ~3;

  stage<T, HD, kBM>(qs, q, i0, g.t_q, g.hd, g.wide_qk);
  stage<T, HD, kBM>(dos, dout, i0, g.t_q, g.hd_v, g.wide_v);
  float row_lse[4], row_delta[4], acc[4][NV];
#pragma unroll
  for (int a = 0; a < 4; ++a) {
    const int i = i0 + ty * 4 + a;
    row_lse[a] = i < g.t_q ? g.lse_in[b * g.t_q + i] : 0.f;
    row_delta[a] = i < g.t_q ? g.delta[b * g.t_q + i] : 0.f;
#pragma unroll
    for (int c = 0; c < NV; ++c) acc[a][c] = 0.f;
  }
  const int keys_end = g.causal ? min(g.t_k, i0 + kBM) : g.t_k;
  for (int j0 = 0; j0 < keys_end; j0 += BN) {
    __syncthreads();
    stage<T, HD, BN>(ks, k, j0, g.t_k, g.hd, g.wide_qk);
    stage<T, HD, BN>(vs, v, j0, g.t_k, g.hd_v, g.wide_v);
    bool open[NB];
#pragma unroll
    for (int c = 0; c < NB; ++c) {
      const int j = j0 + tx + 16 * c;
      open[c] = j < g.t_k && (!mask || widen<T>(mask[j]) != 0.f);
    }
    __syncthreads();
    float s[4][NB], dp[4][NB];
#pragma unroll
    for (int a = 0; a < 4; ++a)
#pragma unroll
      for (int c = 0; c < NB; ++c) s[a][c] = 0.f, dp[a][c] = 0.f;
    dot_tiles<LD, NB>(s, qs + ty * 4 * LD, ks + tx * LD, depth);
    dot_tiles<LD, NB>(dp, dos + ty * 4 * LD, vs + tx * LD, depth_v);
#pragma unroll
    for (int a = 0; a < 4; ++a) {
      const int i = i0 + ty * 4 + a;
#pragma unroll
      for (int c = 0; c < NB; ++c) {
        const bool seen = open[c] && i < g.t_q && (!g.causal || j0 + tx + 16 * c <= i);
        const float p = seen ? expf(s[a][c] * g.scale - row_lse[a]) : 0.f;
        ss[(ty * 4 + a) * LP + tx + 16 * c] = seen ? p * (dp[a][c] - row_delta[a]) * g.scale : 0.f;
      }
    }
    __syncthreads();
    weigh_rows<HD, BN>(acc, ss + ty * 4 * LP, ks, tx);
  }
  store_rows<T, HD>(static_cast<T*>(g.dq), acc, b * g.t_q + i0, min(kBM, g.t_q - i0), g.hd, ty, tx);
}

// ---- dK and dV for 64 key rows (oracle: limn/sdpa.py:190-203) ----
template <typename T, int HD, int BN>
__global__ void __launch_bounds__(kThreads) tiled_bwd_kv_kernel(const Args g) {
  constexpr int LD = HD + kPad, LP = BN + kPad, NB = BN / 16, NV = HD / 16;
  extern __shared__ __align__(16) float shared[];
  float* ks = shared;
  float* vs = ks + kBM * LD;
  float* qs = vs + kBM * LD;
  float* dos = qs + BN * LD;
  float* pt = dos + BN * LD;
  float* dst = pt + kBM * LP;
  float* lse_s = dst + kBM * LP;
  float* delta_s = lse_s + BN;
  const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
  const long long b = blockIdx.x / g.tiles;
  const int j0 = static_cast<int>(blockIdx.x - b * g.tiles) * kBM;  // early causal keys (the long ones) first
  const T* q = static_cast<const T*>(g.q) + b * g.t_q * g.hd;
  const T* k = static_cast<const T*>(g.k) + b * g.t_k * g.hd;
  const T* v = static_cast<const T*>(g.v) + b * g.t_k * g.hd_v;
  const T* dout = static_cast<const T*>(g.dout) + b * g.t_q * g.hd_v;
  const T* mask = g.mask ? static_cast<const T*>(g.mask) + b * g.t_k : nullptr;
  const int depth = (g.hd + 3) & ~3, depth_v = (g.hd_v + 3) & ~3;

  stage<T, HD, kBM>(ks, k, j0, g.t_k, g.hd, g.wide_qk);
  stage<T, HD, kBM>(vs, v, j0, g.t_k, g.hd_v, g.wide_v);
  bool live[4];
  float acc_k[4][NV], acc_v[4][NV];
#pragma unroll
  for (int a = 0; a < 4; ++a) {
    const int j = j0 + ty * 4 + a;
    live[a] = j < g.t_k && (!mask || widen<T>(mask[j]) != 0.f);
#pragma unroll
    for (int c = 0; c < NV; ++c) acc_k[a][c] = 0.f, acc_v[a][c] = 0.f;
  }
  const int first = g.causal ? (j0 / BN) * BN : 0;  // the first query tile that sees one of these keys
  for (int i0 = first; i0 < g.t_q; i0 += BN) {
    __syncthreads();
    stage<T, HD, BN>(qs, q, i0, g.t_q, g.hd, g.wide_qk);
    stage<T, HD, BN>(dos, dout, i0, g.t_q, g.hd_v, g.wide_v);
    if (threadIdx.x < BN) {
      const int i = i0 + threadIdx.x;
      lse_s[threadIdx.x] = i < g.t_q ? g.lse_in[b * g.t_q + i] : 0.f;
      delta_s[threadIdx.x] = i < g.t_q ? g.delta[b * g.t_q + i] : 0.f;
    }
    __syncthreads();
    float s[4][NB], dp[4][NB];
#pragma unroll
    for (int a = 0; a < 4; ++a)
#pragma unroll
      for (int c = 0; c < NB; ++c) s[a][c] = 0.f, dp[a][c] = 0.f;
    dot_tiles<LD, NB>(s, ks + ty * 4 * LD, qs + tx * LD, depth);
    dot_tiles<LD, NB>(dp, vs + ty * 4 * LD, dos + tx * LD, depth_v);
#pragma unroll
    for (int a = 0; a < 4; ++a) {
      const int j = j0 + ty * 4 + a;
#pragma unroll
      for (int c = 0; c < NB; ++c) {
        const int ii = tx + 16 * c, i = i0 + ii;
        const bool seen = live[a] && i < g.t_q && (!g.causal || j <= i);
        const float p = seen ? expf(s[a][c] * g.scale - lse_s[ii]) : 0.f;
        pt[(ty * 4 + a) * LP + ii] = p;
        dst[(ty * 4 + a) * LP + ii] = seen ? p * (dp[a][c] - delta_s[ii]) * g.scale : 0.f;
      }
    }
    __syncthreads();
    weigh_rows<HD, BN>(acc_v, pt + ty * 4 * LP, dos, tx);
    weigh_rows<HD, BN>(acc_k, dst + ty * 4 * LP, qs, tx);
  }
  const int rows_here = min(kBM, g.t_k - j0);
  store_rows<T, HD>(static_cast<T*>(g.dk), acc_k, b * g.t_k + j0, rows_here, g.hd, ty, tx);
  store_rows<T, HD>(static_cast<T*>(g.dv), acc_v, b * g.t_k + j0, rows_here, g.hd_v, ty, tx);
}

template <int HD, int BN>
constexpr size_t shared_bytes(Op op) {
  constexpr size_t LD = HD + kPad, LP = BN + kPad;
  switch (op) {
    case Op::Fwd: return sizeof(float) * ((kBM + 2 * BN) * LD + kBM * LP);
    case Op::BwdQ: return sizeof(float) * ((2 * kBM + 2 * BN) * LD + kBM * LP);
    case Op::BwdKV: return sizeof(float) * ((2 * kBM + 2 * BN) * LD + 2 * kBM * LP + 2 * BN);
  }
  return 0;
}

template <typename T, int HD, int BN>
int launch_sized(Op op, const Problem& p) {
  const int owned = op == Op::BwdKV ? p.t_k : p.t_q;
  Args g = {};
  g.q = p.q, g.k = p.k, g.v = p.v, g.mask = p.mask, g.dout = p.dout;
  g.lse_in = static_cast<const float*>(p.lse_in), g.delta = static_cast<const float*>(p.delta);
  g.out = p.out, g.dq = p.dq, g.dk = p.dk, g.dv = p.dv, g.lse_out = static_cast<float*>(p.lse_out);
  g.tiles = (owned + kBM - 1) / kBM;
  g.t_q = p.t_q, g.t_k = p.t_k, g.hd = p.hd, g.hd_v = p.hd_v, g.causal = p.causal ? 1 : 0;
  g.scale = static_cast<float>(p.scale);
  constexpr int piece = 16 / sizeof(T);
  auto aligned = [](const void* x) { return x == nullptr || (reinterpret_cast<uintptr_t>(x) & 15u) == 0; };
  g.wide_qk = p.hd % piece == 0 && aligned(p.q) && aligned(p.k);
  g.wide_v = p.hd_v % piece == 0 && aligned(p.v) && aligned(p.dout);
  const long long blocks = p.bh * g.tiles;
  if (blocks > 0x7fffffffLL) return fail(LIMN_B200_UNSUPPORTED, "sdpa: %lld row tiles need more blocks than one grid holds", blocks);
  const size_t shared = shared_bytes<HD, BN>(op);
  void (*kernel)(const Args) = op == Op::Fwd    ? tiled_fwd_kernel<T, HD, BN>
                               : op == Op::BwdQ ? tiled_bwd_q_kernel<T, HD, BN>
                                                : tiled_bwd_kv_kernel<T, HD, BN>;
  if (shared > 48 * 1024)
    LIMN_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(shared)),
              "sizing shared memory for a tiled sdpa kernel");
  kernel<<<dim3(static_cast<unsigned>(blocks)), dim3(kThreads), shared, p.stream>>>(g);
  LIMN_CUDA(cudaGetLastError(), "launching a tiled sdpa kernel");
  note_launches(1);
  return LIMN_B200_OK;
}

template <typename T>
int launch_typed(Op op, const Problem& p) {
  const int widest = p.hd > p.hd_v ? p.hd : p.hd_v;
  if (widest <= 32) return launch_sized<T, 32, 64>(op, p);
  if (widest <= 64) return launch_sized<T, 64, 64>(op, p);
  if (widest <= 128) return launch_sized<T, 128, 32>(op, p);
  return launch_sized<T, 256, 16>(op, p);
}

}  // namespace

bool general_tiled_serves(Op, const Problem& p) {
  if (p.dtype == LIMN_B200_F64 || p.hd > 256 || p.hd_v > 256) return false;
  if (p.layout != LIMN_B200_BHTD || p.strided) return false;
  return p.t_q >= 16 && p.t_k >= 16;  // shorter sides leave most of a 64-row tile idle: one row per warp is better
}

int general_tiled_launch(Op op, const Problem& p) {
  switch (p.dtype) {
    case LIMN_B200_F32: return launch_typed<float>(op, p);
    case LIMN_B200_F16: return launch_typed<__half>(op, p);
    case LIMN_B200_BF16: return launch_typed<__nv_bfloat16>(op, p);
  }
  return fail(LIMN_B200_BAD_ARGUMENT, "sdpa: dtype code %d is not served by the tiled kernels", p.dtype);
}

}  // namespace limn_b200
