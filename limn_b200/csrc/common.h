// Shared host-side declarations for the limn_b200 library: the problem description every
// kernel family takes, error reporting, and the per-device status word.
#pragma once

#include <cuda_runtime.h>

#include <cstdarg>
#include <cstdio>

#include "../../include/limn_b200.h"

namespace limn_b200 {

// Where element (batch b, head h, row t, column 0) of an operand lives: base + b * batch + h * head + t * row
// elements. Columns are always contiguous.
struct Strides {
  long long batch = 0, head = 0, row = 0;
};
// The operands of the three ops, for per-operand strides.
enum Operand { kOpQ = 0, kOpK, kOpV, kOpDout, kOpOut, kOpDq, kOpDk, kOpDv, kOperands };

// One attention problem, as the C ABI received it. Pointers the op does not use are null.
struct Problem {
  const void* q = nullptr;
  const void* k = nullptr;
  const void* v = nullptr;
  const void* dout = nullptr;
  const void* lse_in = nullptr;  // backward: the forward's L
  const void* delta = nullptr;   // backward: row dot of dO and O
  const void* mask = nullptr;    // (bh, t_k) in the storage dtype, 0 hides a key; may be null
  void* out = nullptr;           // forward: O
  void* lse_out = nullptr;       // forward: L
  void* dq = nullptr;
  void* dk = nullptr;
  void* dv = nullptr;
  int dtype = 0;
  long long bh = 0;
  int t_q = 0, t_k = 0, hd = 0, hd_v = 0;
  int causal = 0;
  double scale = 0.0;
  cudaStream_t stream = nullptr;
  // Operand layout (a limn_b200_layout value). Dense (BHTD) problems leave heads at 0: bh problems, one "batch".
  // With heads > 0, bh = batch * heads and problem p is (batch p / heads, head p % heads).
  int layout = 0;
  int heads = 0;
  // The strided entry points give every operand its own strides (a q, k, v that are slices of one projection's
  // output do not share the layout of the output they produce); otherwise the strides follow from `layout`.
  bool strided = false;
  Strides strides[kOperands];
  // dQ pass only: compute delta from `out` (the forward's O) and dO on the way and write it to `delta`, instead of
  // reading it. Served by the tensor-core kernels; the general family runs the row-dot kernel first.
  bool fuse_delta = false;
  // Where kernels that wait record giving up. Null means the per-device word status_word() allocates.
  unsigned int* status = nullptr;
  // Two zeroed words for the kernels' work counters. Null means a pair from schedule_words().
  unsigned int* schedule = nullptr;
};

enum class Op { Fwd, BwdQ, BwdKV };

// Error text for the calling thread; returns `code` so call sites can `return fail(...)`.
int fail(int code, const char* fmt, ...);
void clear_error();
void note_launches(int n);
void reset_launches();

// cudaError_t -> status code with a message naming what was being done.
int cuda_fail(cudaError_t err, const char* doing);
#define LIMN_CUDA(expr, doing)                                   \
  do {                                                           \
    cudaError_t err__ = (expr);                                  \
    if (err__ != cudaSuccess) return ::limn_b200::cuda_fail(err__, doing); \
  } while (0)

// Device address of the current device's status word (allocated on first use, one per
// device, zero-initialised). Kernels that wait write a non-zero code there when they give up.
int status_word(unsigned int** word);
// Two zeroed words (next work item, CTAs finished) for one launch of a kernel whose CTAs fetch their
// work items themselves. A kernel leaves its pair zeroed again, so the pairs are handed out in turn from
// a fixed per-device ring; a pair is only met twice by launches kScheduleRing apart.
constexpr int kScheduleRing = 128;
int schedule_words(unsigned int** pair);
// How many problems the tensor-core kernels schedule as one group (see cta_work): all of them when the GPU
// has only a few work items per SM, else as many as keep their K and V inside a share of L2.
int work_group(const Problem& p, long long items, int sms);
// Streaming multiprocessors of the current device.
int sm_count(int* count);

// Argument checks and dispatch shared by every entry point for the three ops. validate_op only checks
// (extents, dtype, required pointers, layout support) and launches nothing; dispatch_op checks, then launches.
int validate_op(Op op, const char* name, const Problem& p);
int dispatch_op(Op op, const char* name, const Problem& p);

// Strides of a (batch, heads, rows, width) operand in the given limn_b200_layout, and of operand `which` of a
// problem: the ones the caller gave, else the layout's.
Strides strides_of(int layout, int heads, int rows, int width);
inline Strides operand_strides(const Problem& p, Operand which, int heads, int rows, int width) {
  return p.strided ? p.strides[which] : strides_of(p.layout, heads, rows, width);
}

// Launch with programmatic stream serialization: the kernel may be scheduled while the last CTAs of the kernel
// before it in the stream are still running, and waits for that kernel itself (ptx::grid_dependency_wait) before
// it touches global memory. Hides the launch latency and set-up of back-to-back kernels.
template <typename... Params, typename... Args>
cudaError_t launch_overlapped(void (*kernel)(Params...), dim3 grid, dim3 block, size_t shared_bytes, cudaStream_t stream,
                              Args&&... args) {
  cudaLaunchConfig_t config = {};
  config.gridDim = grid;
  config.blockDim = block;
  config.dynamicSmemBytes = shared_bytes;
  config.stream = stream;
  cudaLaunchAttribute attribute[1];
  attribute[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attribute[0].val.programmaticStreamSerializationAllowed = 1;
  config.attrs = attribute;
  config.numAttrs = 1;
  return cudaLaunchKernelEx(&config, kernel, static_cast<Params>(args)...);
}

// Kernel families. Each returns a status code and enqueues on p.stream.
int general_launch(Op op, const Problem& p);
// The tiled members of the general family (float32/float16/bfloat16, head dims up to 256, sides of 16 rows and
// more); general_launch hands them what they serve and keeps the rest for the one-row-per-warp kernels.
bool general_tiled_serves(Op op, const Problem& p);
int general_tiled_launch(Op op, const Problem& p);
int general_delta(const void* out, const void* dout, void* delta, int dtype, long long rows, int hd_v,
                  cudaStream_t stream);
int general_delta_bthd(const void* out, const void* dout, void* delta, int dtype, int batch, int heads, int t, int hd_v,
                       cudaStream_t stream);
bool tcgen05_serves(Op op, const Problem& p);
int tcgen05_launch(Op op, const Problem& p);
// The forward for decode shapes (a few query rows against many keys): bandwidth-bound, no tensor cores.
bool decode_serves(Op op, const Problem& p);
int decode_launch(const Problem& p);

}  // namespace limn_b200
