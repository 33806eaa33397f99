// The C ABI (include/limn_b200.h): argument checks, dispatch between the two kernel
// families, error text, the per-device status word, and the small CUDA plumbing set that
// hosts without their own binding use.
#include <cuda.h>
#include <cuda_runtime.h>

#include <cstdlib>
#include <cstring>
#include <mutex>

#include "common.h"
#include "tensor_map.h"

namespace limn_b200 {
namespace {

thread_local char g_error[512] = "";
thread_local int g_launches = 0;

constexpr int kMaxDevices = 64;
std::mutex g_status_mutex;
unsigned int* g_status_words[kMaxDevices] = {};

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn g_encode_tiled = nullptr;
std::once_flag g_encode_once;

}  // namespace

int fail(int code, const char* fmt, ...) {
  va_list args;
  va_start(args, fmt);
  vsnprintf(g_error, sizeof(g_error), fmt, args);
  va_end(args);
  return code;
}

void clear_error() { g_error[0] = '\0'; }
void note_launches(int n) { g_launches += n; }
void reset_launches() { g_launches = 0; }

int cuda_fail(cudaError_t err, const char* doing) {
  return fail(LIMN_B200_CUDA_ERROR, "cuda: %s: %s", doing, cudaGetErrorString(err));
}

int status_word(unsigned int** word) {
  int device = 0;
  LIMN_CUDA(cudaGetDevice(&device), "asking for the current device");
  if (device < 0 || device >= kMaxDevices) return fail(LIMN_B200_UNSUPPORTED, "device ordinal %d out of range", device);
  std::lock_guard<std::mutex> lock(g_status_mutex);
  if (g_status_words[device] == nullptr) {
    unsigned int* fresh = nullptr;
    LIMN_CUDA(cudaMalloc(&fresh, 256), "allocating the device status word");
    LIMN_CUDA(cudaMemset(fresh, 0, 256), "clearing the device status word");
    g_status_words[device] = fresh;
  }
  *word = g_status_words[device];
  return LIMN_B200_OK;
}

int schedule_words(unsigned int** pair) {
  static unsigned int* rings[kMaxDevices] = {};
  static unsigned next[kMaxDevices] = {};
  int device = 0;
  LIMN_CUDA(cudaGetDevice(&device), "asking for the current device");
  if (device < 0 || device >= kMaxDevices) return fail(LIMN_B200_UNSUPPORTED, "device ordinal %d out of range", device);
  std::lock_guard<std::mutex> lock(g_status_mutex);
  if (rings[device] == nullptr) {
    unsigned int* fresh = nullptr;
    LIMN_CUDA(cudaMalloc(&fresh, kScheduleRing * 2 * sizeof(unsigned)), "allocating the work counters");
    LIMN_CUDA(cudaMemset(fresh, 0, kScheduleRing * 2 * sizeof(unsigned)), "clearing the work counters");
    rings[device] = fresh;
  }
  *pair = rings[device] + 2 * (next[device]++ % kScheduleRing);
  return LIMN_B200_OK;
}

int work_group(const Problem& p, long long items, int sms) {
  const long long all = p.bh > 0 ? p.bh : 1;
  // A GPU with only a few items per SM is decided by balance: one group, every problem's longest items first
  // (measured on B200, 20 problems of S = 3000 causal: 0.056 ms against 0.079 ms in groups of 8).
  if (items <= 4LL * sms) return static_cast<int>(all);
  // Otherwise by locality: the items running side by side should share few enough K and V tiles for L2
  // (256 problems of S = 4096, D = 128: groups of 8 to 16 are 1.5 % faster than 32, 10 % faster than one group).
  constexpr long long kL2Share = 32LL << 20;  // of B200's 126 MB
  const long long streamed = static_cast<long long>(p.t_k) * (p.hd + p.hd_v) * 2;  // K and V of one problem, 16-bit
  long long group = streamed > 0 ? kL2Share / streamed : 1;
  if (group < 1) group = 1;
  if (group > all) group = all;
  return static_cast<int>(group);
}

int sm_count(int* count) {
  static int cached[kMaxDevices] = {};
  int device = 0;
  LIMN_CUDA(cudaGetDevice(&device), "asking for the current device");
  if (device < 0 || device >= kMaxDevices) return fail(LIMN_B200_UNSUPPORTED, "device ordinal %d out of range", device);
  if (cached[device] == 0) {
    int n = 0;
    LIMN_CUDA(cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, device), "asking for the SM count");
    cached[device] = n;
  }
  *count = cached[device];
  return LIMN_B200_OK;
}

Strides strides_of(int layout, int heads, int rows, int width) {
  if (layout == LIMN_B200_BTHD)
    return Strides{static_cast<long long>(rows) * heads * width, width, static_cast<long long>(heads) * width};
  return Strides{static_cast<long long>(heads) * rows * width, static_cast<long long>(rows) * width, width};
}

int make_tile_map(CUtensorMap* map, const void* base, bool fp16, int batch, int heads, int rows, int width, int box_rows,
                  const Strides& strides) {
  std::call_once(g_encode_once, [] {
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult found;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &found) == cudaSuccess &&
        found == cudaDriverEntryPointSuccess)
      g_encode_tiled = reinterpret_cast<EncodeTiledFn>(fn);
  });
  if (g_encode_tiled == nullptr)
    return fail(LIMN_B200_CUDA_ERROR, "cuda: the driver does not export cuTensorMapEncodeTiled");
  if ((reinterpret_cast<uintptr_t>(base) & 15u) != 0)
    return fail(LIMN_B200_BAD_ARGUMENT, "sdpa: tensor base %p is not 16-byte aligned", base);
  if ((strides.batch | strides.head | strides.row) & 7)
    return fail(LIMN_B200_BAD_ARGUMENT, "sdpa: operand strides must be multiples of 8 elements");
  // A map depends only on the base address, the extents and the strides, and a host that pools its buffers
  // (limn does, limn/backend_cuda.py:297-307) hands the same ones back step after step, so the last few
  // encodings are kept per thread. At the smallest shapes the encoding costs as much host time as the kernel
  // takes to run.
  struct Entry {
    const void* base;
    int batch, heads, rows, width, box_rows, fp16;
    Strides strides;
    CUtensorMap map;
  };
  constexpr int kEntries = 16;
  thread_local Entry cache[kEntries];
  thread_local int used = 0, next_slot = 0;
  for (int i = 0; i < used; ++i) {
    const Entry& e = cache[i];
    if (e.base == base && e.batch == batch && e.heads == heads && e.rows == rows && e.width == width &&
        e.box_rows == box_rows && e.fp16 == (fp16 ? 1 : 0) && e.strides.batch == strides.batch &&
        e.strides.head == strides.head && e.strides.row == strides.row) {
      *map = e.map;
      return LIMN_B200_OK;
    }
  }
  const cuuint64_t dims[4] = {static_cast<cuuint64_t>(width), static_cast<cuuint64_t>(rows), static_cast<cuuint64_t>(heads),
                              static_cast<cuuint64_t>(batch)};
  const cuuint64_t byte_strides[3] = {static_cast<cuuint64_t>(strides.row) * 2, static_cast<cuuint64_t>(strides.head) * 2,
                                      static_cast<cuuint64_t>(strides.batch) * 2};
  const cuuint32_t box[4] = {64, static_cast<cuuint32_t>(box_rows), 1, 1};
  const cuuint32_t elem[4] = {1, 1, 1, 1};
  const CUresult res = g_encode_tiled(
      map, fp16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(base), dims,
      byte_strides, box, elem, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
      CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (res != CUDA_SUCCESS) return fail(LIMN_B200_CUDA_ERROR, "cuda: encoding a tensor map failed with CUresult %d", (int)res);
  Entry& slot = cache[next_slot];
  slot = Entry{base, batch, heads, rows, width, box_rows, fp16 ? 1 : 0, strides, *map};
  next_slot = (next_slot + 1) % kEntries;
  if (used < kEntries) ++used;
  return LIMN_B200_OK;
}

namespace {

int check_problem(const char* name, const Problem& p) {
  if (p.dtype < LIMN_B200_F32 || p.dtype > LIMN_B200_F64)
    return fail(LIMN_B200_BAD_ARGUMENT, "%s: unknown dtype code %d", name, p.dtype);
  if (p.bh < 0 || p.t_q <= 0 || p.t_k <= 0 || p.hd <= 0 || p.hd_v <= 0)
    return fail(LIMN_B200_BAD_ARGUMENT, "%s: extents must be positive, got bh=%lld t_q=%d t_k=%d hd=%d hd_v=%d", name,
                p.bh, p.t_q, p.t_k, p.hd, p.hd_v);
  if (p.causal && p.t_q != p.t_k)
    return fail(LIMN_B200_BAD_ARGUMENT, "%s: causal sdpa needs square keys, got %d queries and %d keys", name, p.t_q,
                p.t_k);
  return LIMN_B200_OK;
}

Problem problem(const void* q, const void* k, const void* v, const void* mask, int dtype, long long bh, int t_q,
                int t_k, int hd, int hd_v, int causal, double scale, void* stream) {
  Problem p;
  p.q = q, p.k = k, p.v = v, p.mask = mask;
  p.dtype = dtype, p.bh = bh, p.t_q = t_q, p.t_k = t_k, p.hd = hd, p.hd_v = hd_v;
  p.causal = causal != 0, p.scale = scale, p.stream = static_cast<cudaStream_t>(stream);
  return p;
}

}  // namespace

int validate_op(Op op, const char* name, const Problem& p) {
  if (int rc = check_problem(name, p)) return rc;
  const bool have_inputs = p.q && p.k && p.v;
  bool have_rest = true;
  switch (op) {
    case Op::Fwd: have_rest = p.out && p.lse_out; break;
    case Op::BwdQ: have_rest = p.dout && p.lse_in && p.delta && p.dq && (!p.fuse_delta || p.out); break;
    case Op::BwdKV: have_rest = p.dout && p.lse_in && p.delta && p.dk && p.dv; break;
  }
  if (!have_inputs || !have_rest) return fail(LIMN_B200_BAD_ARGUMENT, "%s: a required pointer is null", name);
  if (p.bh > 0 && !tcgen05_serves(op, p) && p.layout != LIMN_B200_BHTD)
    return fail(LIMN_B200_UNSUPPORTED,
                "%s: the (batch, t, heads, hd) layout is served for f16/bf16 with hd and hd_v multiples of 8 up to 128; make the "
                "operands contiguous as (batch, heads, t, hd) for anything else",
                name);
  return LIMN_B200_OK;
}

int dispatch_op(Op op, const char* name, const Problem& p) {
  clear_error();
  g_launches = 0;
  if (int rc = validate_op(op, name, p)) return rc;
  if (p.bh == 0) return LIMN_B200_OK;
  if (decode_serves(op, p)) return decode_launch(p);
  if (tcgen05_serves(op, p)) {
    // The dQ kernel can compute the row statistic on its spare warps, which saves a launch and a pass over O and dO:
    // 7 % at S = 256. From a few key tiles per work item on, the separate row-dot kernel in front of it is the faster
    // way to the same delta and dQ (2.5 to 3 % at S = 2048 and 3000), so dense operands of that size take it.
    if (op == Op::BwdQ && p.fuse_delta && !p.strided && p.layout == LIMN_B200_BHTD && p.t_k > 512) {
      if (int rc = general_delta(p.out, p.dout, const_cast<void*>(p.delta), p.dtype, p.bh * p.t_q, p.hd_v, p.stream)) return rc;
      Problem unfused = p;
      unfused.fuse_delta = false;
      return tcgen05_launch(op, unfused);
    }
    return tcgen05_launch(op, p);
  }
  if (op == Op::BwdQ && p.fuse_delta) {
    // the general kernels read delta: fill it first, as the unfused sequence would
    if (int rc = general_delta(p.out, p.dout, const_cast<void*>(p.delta), p.dtype, p.bh * p.t_q, p.hd_v, p.stream)) return rc;
  }
  return general_launch(op, p);
}

}  // namespace limn_b200

using namespace limn_b200;

extern "C" {

int limn_b200_sdpa_fwd(const void* q, const void* k, const void* v, const void* key_mask, void* out, void* lse,
                       int dtype, long long bh, int t_q, int t_k, int hd, int hd_v, int causal, double scale,
                       void* stream) {
  Problem p = problem(q, k, v, key_mask, dtype, bh, t_q, t_k, hd, hd_v, causal, scale, stream);
  p.out = out, p.lse_out = lse;
  return dispatch_op(Op::Fwd, "sdpa", p);
}

int limn_b200_sdpa_bwd_q(const void* q, const void* k, const void* v, const void* dout, const void* lse,
                         const void* delta, const void* key_mask, void* dq, int dtype, long long bh, int t_q, int t_k,
                         int hd, int hd_v, int causal, double scale, void* stream) {
  Problem p = problem(q, k, v, key_mask, dtype, bh, t_q, t_k, hd, hd_v, causal, scale, stream);
  p.dout = dout, p.lse_in = lse, p.delta = delta, p.dq = dq;
  return dispatch_op(Op::BwdQ, "sdpa_bwd_q", p);
}

int limn_b200_sdpa_bwd_q_fused(const void* q, const void* k, const void* v, const void* out, const void* dout,
                               const void* lse, const void* key_mask, void* dq, void* delta, int dtype, long long bh,
                               int t_q, int t_k, int hd, int hd_v, int causal, double scale, void* stream) {
  Problem p = problem(q, k, v, key_mask, dtype, bh, t_q, t_k, hd, hd_v, causal, scale, stream);
  p.out = const_cast<void*>(out), p.dout = dout, p.lse_in = lse, p.delta = delta, p.dq = dq;
  p.fuse_delta = true;
  return dispatch_op(Op::BwdQ, "sdpa_bwd_q_fused", p);
}

int limn_b200_sdpa_bwd_kv(const void* q, const void* k, const void* v, const void* dout, const void* lse,
                          const void* delta, const void* key_mask, void* dk, void* dv, int dtype, long long bh, int t_q,
                          int t_k, int hd, int hd_v, int causal, double scale, void* stream) {
  Problem p = problem(q, k, v, key_mask, dtype, bh, t_q, t_k, hd, hd_v, causal, scale, stream);
  p.dout = dout, p.lse_in = lse, p.delta = delta, p.dk = dk, p.dv = dv;
  return dispatch_op(Op::BwdKV, "sdpa_bwd_kv", p);
}

namespace {

// The layout entry points' shared argument handling: bh = batch * heads, heads kept for the strides.
int with_layout(const char* name, Problem& p, int layout, int batch, int heads) {
  if (layout != LIMN_B200_BHTD && layout != LIMN_B200_BTHD)
    return fail(LIMN_B200_BAD_ARGUMENT, "%s: unknown layout code %d", name, layout);
  if (batch < 0 || heads <= 0) return fail(LIMN_B200_BAD_ARGUMENT, "%s: batch must be >= 0 and heads > 0", name);
  p.bh = static_cast<long long>(batch) * heads;
  p.layout = layout;
  p.heads = layout == LIMN_B200_BHTD ? 0 : heads;  // dense operands are bh problems of one "batch"
  return LIMN_B200_OK;
}

}  // namespace

int limn_b200_sdpa_fwd_layout(const void* q, const void* k, const void* v, const void* key_mask, void* out, void* lse,
                              int layout, int dtype, int batch, int heads, int t_q, int t_k, int hd, int hd_v,
                              int causal, double scale, void* stream) {
  clear_error();
  Problem p = problem(q, k, v, key_mask, dtype, 0, t_q, t_k, hd, hd_v, causal, scale, stream);
  if (int rc = with_layout("sdpa", p, layout, batch, heads)) return rc;
  p.out = out, p.lse_out = lse;
  return dispatch_op(Op::Fwd, "sdpa", p);
}

int limn_b200_sdpa_bwd_q_layout(const void* q, const void* k, const void* v, const void* dout, const void* lse,
                                const void* delta, const void* key_mask, void* dq, int layout, int dtype, int batch,
                                int heads, int t_q, int t_k, int hd, int hd_v, int causal, double scale, void* stream) {
  clear_error();
  Problem p = problem(q, k, v, key_mask, dtype, 0, t_q, t_k, hd, hd_v, causal, scale, stream);
  if (int rc = with_layout("sdpa_bwd_q", p, layout, batch, heads)) return rc;
  p.dout = dout, p.lse_in = lse, p.delta = delta, p.dq = dq;
  return dispatch_op(Op::BwdQ, "sdpa_bwd_q", p);
}

int limn_b200_sdpa_bwd_q_fused_layout(const void* q, const void* k, const void* v, const void* out, const void* dout,
                                      const void* lse, const void* key_mask, void* dq, void* delta, int layout, int dtype,
                                      int batch, int heads, int t_q, int t_k, int hd, int hd_v, int causal, double scale,
                                      void* stream) {
  clear_error();
  Problem p = problem(q, k, v, key_mask, dtype, 0, t_q, t_k, hd, hd_v, causal, scale, stream);
  if (int rc = with_layout("sdpa_bwd_q_fused", p, layout, batch, heads)) return rc;
  p.out = const_cast<void*>(out), p.dout = dout, p.lse_in = lse, p.delta = delta, p.dq = dq;
  p.fuse_delta = true;
  return dispatch_op(Op::BwdQ, "sdpa_bwd_q_fused", p);
}

int limn_b200_sdpa_bwd_kv_layout(const void* q, const void* k, const void* v, const void* dout, const void* lse,
                                 const void* delta, const void* key_mask, void* dk, void* dv, int layout, int dtype,
                                 int batch, int heads, int t_q, int t_k, int hd, int hd_v, int causal, double scale,
                                 void* stream) {
  clear_error();
  Problem p = problem(q, k, v, key_mask, dtype, 0, t_q, t_k, hd, hd_v, causal, scale, stream);
  if (int rc = with_layout("sdpa_bwd_kv", p, layout, batch, heads)) return rc;
  p.dout = dout, p.lse_in = lse, p.delta = delta, p.dk = dk, p.dv = dv;
  return dispatch_op(Op::BwdKV, "sdpa_bwd_kv", p);
}

namespace {

// The strided entry points' shared argument handling: bh = batch * heads and one (batch, head, row) stride triple
// per operand, in elements, in the order the entry point documents.
int with_strides(const char* name, Problem& p, int batch, int heads, const long long* strides, const Operand* order, int count) {
  if (strides == nullptr) return fail(LIMN_B200_BAD_ARGUMENT, "%s: null strides", name);
  if (batch < 0 || heads <= 0) return fail(LIMN_B200_BAD_ARGUMENT, "%s: batch must be >= 0 and heads > 0", name);
  p.bh = static_cast<long long>(batch) * heads;
  p.heads = heads;
  p.strided = true;
  for (int i = 0; i < count; ++i) {
    const Strides given{strides[3 * i], strides[3 * i + 1], strides[3 * i + 2]};
    if (given.batch < 0 || given.head < 0 || given.row <= 0 || ((given.batch | given.head | given.row) & 7))
      return fail(LIMN_B200_BAD_ARGUMENT, "%s: strides must be non-negative multiples of 8 elements (rows: positive), got (%lld, %lld, %lld) for operand %d",
                  name, given.batch, given.head, given.row, i);
    p.strides[order[i]] = given;
  }
  return LIMN_B200_OK;
}

int strided_dispatch(Op op, const char* name, const Problem& p) {
  if (int rc = validate_op(op, name, p)) return rc;
  if (p.bh > 0 && !tcgen05_serves(op, p))
    return fail(LIMN_B200_UNSUPPORTED, "%s: strided operands are served for f16/bf16 with hd and hd_v multiples of 8 up to 128; make the operands contiguous for anything else", name);
  return dispatch_op(op, name, p);
}

}  // namespace

int limn_b200_sdpa_fwd_strided(const void* q, const void* k, const void* v, const void* key_mask, void* out, void* lse,
                               const long long* strides, int dtype, int batch, int heads, int t_q, int t_k, int hd, int hd_v,
                               int causal, double scale, void* stream) {
  clear_error();
  Problem p = problem(q, k, v, key_mask, dtype, 0, t_q, t_k, hd, hd_v, causal, scale, stream);
  static const Operand order[] = {kOpQ, kOpK, kOpV, kOpOut};
  if (int rc = with_strides("sdpa_strided", p, batch, heads, strides, order, 4)) return rc;
  p.out = out, p.lse_out = lse;
  return strided_dispatch(Op::Fwd, "sdpa_strided", p);
}

int limn_b200_sdpa_bwd_q_fused_strided(const void* q, const void* k, const void* v, const void* out, const void* dout,
                                       const void* lse, const void* key_mask, void* dq, void* delta, const long long* strides,
                                       int dtype, int batch, int heads, int t_q, int t_k, int hd, int hd_v, int causal,
                                       double scale, void* stream) {
  clear_error();
  Problem p = problem(q, k, v, key_mask, dtype, 0, t_q, t_k, hd, hd_v, causal, scale, stream);
  static const Operand order[] = {kOpQ, kOpK, kOpV, kOpOut, kOpDout, kOpDq};
  if (int rc = with_strides("sdpa_bwd_q_fused_strided", p, batch, heads, strides, order, 6)) return rc;
  p.out = const_cast<void*>(out), p.dout = dout, p.lse_in = lse, p.delta = delta, p.dq = dq;
  p.fuse_delta = true;
  return strided_dispatch(Op::BwdQ, "sdpa_bwd_q_fused_strided", p);
}

int limn_b200_sdpa_bwd_kv_strided(const void* q, const void* k, const void* v, const void* dout, const void* lse,
                                  const void* delta, const void* key_mask, void* dk, void* dv, const long long* strides,
                                  int dtype, int batch, int heads, int t_q, int t_k, int hd, int hd_v, int causal, double scale,
                                  void* stream) {
  clear_error();
  Problem p = problem(q, k, v, key_mask, dtype, 0, t_q, t_k, hd, hd_v, causal, scale, stream);
  static const Operand order[] = {kOpQ, kOpK, kOpV, kOpDout, kOpDk, kOpDv};
  if (int rc = with_strides("sdpa_bwd_kv_strided", p, batch, heads, strides, order, 6)) return rc;
  p.dout = dout, p.lse_in = lse, p.delta = delta, p.dk = dk, p.dv = dv;
  return strided_dispatch(Op::BwdKV, "sdpa_bwd_kv_strided", p);
}

int limn_b200_sdpa_delta_layout(const void* out, const void* dout, void* delta, int layout, int dtype, int batch,
                                int heads, int t_q, int hd_v, void* stream) {
  clear_error();
  g_launches = 0;
  if (!out || !dout || !delta) return fail(LIMN_B200_BAD_ARGUMENT, "sdpa_delta: a required pointer is null");
  if (layout != LIMN_B200_BHTD && layout != LIMN_B200_BTHD)
    return fail(LIMN_B200_BAD_ARGUMENT, "sdpa_delta: unknown layout code %d", layout);
  if (batch < 0 || heads <= 0 || t_q <= 0 || hd_v <= 0)
    return fail(LIMN_B200_BAD_ARGUMENT, "sdpa_delta: extents must be positive");
  if (batch == 0) return LIMN_B200_OK;
  if (layout == LIMN_B200_BHTD)
    return general_delta(out, dout, delta, dtype, static_cast<long long>(batch) * heads * t_q, hd_v,
                         static_cast<cudaStream_t>(stream));
  return general_delta_bthd(out, dout, delta, dtype, batch, heads, t_q, hd_v, static_cast<cudaStream_t>(stream));
}

int limn_b200_sdpa_delta(const void* out, const void* dout, void* delta, int dtype, long long rows, int hd_v,
                         void* stream) {
  clear_error();
  g_launches = 0;
  if (!out || !dout || !delta) return fail(LIMN_B200_BAD_ARGUMENT, "sdpa_delta: a required pointer is null");
  if (rows < 0 || hd_v <= 0) return fail(LIMN_B200_BAD_ARGUMENT, "sdpa_delta: extents must be positive");
  if (rows == 0) return LIMN_B200_OK;
  return general_delta(out, dout, delta, dtype, rows, hd_v, static_cast<cudaStream_t>(stream));
}

int limn_b200_sdpa_path(int dtype, long long bh, int t_q, int t_k, int hd, int hd_v, int causal, int has_mask,
                        double scale) {
  clear_error();
  alignas(16) static const int placeholder[4] = {0, 0, 0, 0};
  Problem p = problem(placeholder, placeholder, placeholder, has_mask ? placeholder : nullptr, dtype, bh, t_q, t_k,
                      hd, hd_v, causal, scale, nullptr);
  if (check_problem("sdpa", p) != LIMN_B200_OK) return -1;
  if (decode_serves(Op::Fwd, p)) return LIMN_B200_PATH_DECODE;
  return tcgen05_serves(Op::Fwd, p) ? LIMN_B200_PATH_TCGEN05 : LIMN_B200_PATH_GENERAL;
}

int limn_b200_last_launch_count(void) { return g_launches; }
const char* limn_b200_last_error(void) { return g_error; }
int limn_b200_version(void) { return 100; }

int limn_b200_device_status(unsigned int* status) {
  clear_error();
  if (!status) return fail(LIMN_B200_BAD_ARGUMENT, "device_status: null result pointer");
  unsigned int* word = nullptr;
  if (int rc = status_word(&word)) return rc;
  LIMN_CUDA(cudaDeviceSynchronize(), "waiting for the device before reading its status word");
  LIMN_CUDA(cudaMemcpy(status, word, sizeof(unsigned int), cudaMemcpyDeviceToHost), "reading the device status word");
  if (*status == 0) return LIMN_B200_OK;
  LIMN_CUDA(cudaMemset(word, 0, sizeof(unsigned int)), "clearing the device status word");
  return fail(LIMN_B200_DEVICE_TIMEOUT,
              "a kernel gave up on a bounded wait (status 0x%08x: role %u, barrier %u); kernels launched after it on this "
              "device wrote nothing until now",
              *status, (*status >> 8) & 0xffu, *status & 0xffu);
}

/* ---- plumbing ---- */
int limn_b200_device_count(int* count) {
  clear_error();
  LIMN_CUDA(cudaGetDeviceCount(count), "counting devices");
  return LIMN_B200_OK;
}
int limn_b200_set_device(int ordinal) {
  clear_error();
  LIMN_CUDA(cudaSetDevice(ordinal), "selecting a device");
  return LIMN_B200_OK;
}
int limn_b200_mem_alloc(void** device_ptr, unsigned long long nbytes) {
  clear_error();
  LIMN_CUDA(cudaMalloc(device_ptr, nbytes ? nbytes : 1), "allocating device memory");
  return LIMN_B200_OK;
}
int limn_b200_mem_free(void* device_ptr) {
  clear_error();
  LIMN_CUDA(cudaFree(device_ptr), "freeing device memory");
  return LIMN_B200_OK;
}
int limn_b200_mem_set(void* device_ptr, int byte, unsigned long long nbytes, void* stream) {
  clear_error();
  LIMN_CUDA(cudaMemsetAsync(device_ptr, byte, nbytes, static_cast<cudaStream_t>(stream)), "filling device memory");
  return LIMN_B200_OK;
}
int limn_b200_host_alloc(void** pinned_ptr, unsigned long long nbytes) {
  clear_error();
  LIMN_CUDA(cudaMallocHost(pinned_ptr, nbytes ? nbytes : 1), "allocating pinned host memory");
  return LIMN_B200_OK;
}
int limn_b200_host_free(void* pinned_ptr) {
  clear_error();
  LIMN_CUDA(cudaFreeHost(pinned_ptr), "freeing pinned host memory");
  return LIMN_B200_OK;
}
int limn_b200_copy_h2d(void* device_dst, const void* host_src, unsigned long long nbytes, void* stream) {
  clear_error();
  LIMN_CUDA(cudaMemcpyAsync(device_dst, host_src, nbytes, cudaMemcpyHostToDevice, static_cast<cudaStream_t>(stream)),
            "uploading bytes");
  return LIMN_B200_OK;
}
int limn_b200_copy_d2h(void* host_dst, const void* device_src, unsigned long long nbytes, void* stream) {
  clear_error();
  LIMN_CUDA(cudaMemcpyAsync(host_dst, device_src, nbytes, cudaMemcpyDeviceToHost, static_cast<cudaStream_t>(stream)),
            "downloading bytes");
  return LIMN_B200_OK;
}
int limn_b200_copy_d2d(void* device_dst, const void* device_src, unsigned long long nbytes, void* stream) {
  clear_error();
  LIMN_CUDA(cudaMemcpyAsync(device_dst, device_src, nbytes, cudaMemcpyDeviceToDevice, static_cast<cudaStream_t>(stream)),
            "copying bytes on the device");
  return LIMN_B200_OK;
}
int limn_b200_stream_create(void** stream) {
  clear_error();
  cudaStream_t s;
  LIMN_CUDA(cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking), "creating a stream");
  *stream = s;
  return LIMN_B200_OK;
}
int limn_b200_stream_destroy(void* stream) {
  clear_error();
  LIMN_CUDA(cudaStreamDestroy(static_cast<cudaStream_t>(stream)), "destroying a stream");
  return LIMN_B200_OK;
}
int limn_b200_stream_wait_event(void* stream, void* event) {
  clear_error();
  LIMN_CUDA(cudaStreamWaitEvent(static_cast<cudaStream_t>(stream), static_cast<cudaEvent_t>(event), 0),
            "making a stream wait for an event");
  return LIMN_B200_OK;
}
int limn_b200_stream_sync(void* stream) {
  clear_error();
  LIMN_CUDA(cudaStreamSynchronize(static_cast<cudaStream_t>(stream)), "waiting for a stream");
  return LIMN_B200_OK;
}
int limn_b200_device_sync(void) {
  clear_error();
  LIMN_CUDA(cudaDeviceSynchronize(), "waiting for the device");
  return LIMN_B200_OK;
}
int limn_b200_event_create(void** event) {
  clear_error();
  cudaEvent_t e;
  LIMN_CUDA(cudaEventCreate(&e), "creating an event");
  *event = e;
  return LIMN_B200_OK;
}
int limn_b200_event_destroy(void* event) {
  clear_error();
  LIMN_CUDA(cudaEventDestroy(static_cast<cudaEvent_t>(event)), "destroying an event");
  return LIMN_B200_OK;
}
int limn_b200_event_record(void* event, void* stream) {
  clear_error();
  LIMN_CUDA(cudaEventRecord(static_cast<cudaEvent_t>(event), static_cast<cudaStream_t>(stream)), "recording an event");
  return LIMN_B200_OK;
}
int limn_b200_event_elapsed_ms(void* start, void* stop, float* ms) {
  clear_error();
  LIMN_CUDA(cudaEventElapsedTime(ms, static_cast<cudaEvent_t>(start), static_cast<cudaEvent_t>(stop)),
            "reading an event interval");
  return LIMN_B200_OK;
}

}  // extern "C"
