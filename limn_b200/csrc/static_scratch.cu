// limn_b200_sdpa_bwd_q_static: the dQ pass for hosts that must not allocate.
//
// The ordinary route to dQ needs two pieces of device memory besides its inputs and outputs:
// the row statistic delta = sum_d dO * O (one number per query row, which the caller has to
// hold in a buffer of its own and fill with a reduce kernel), and the word in which a kernel
// that waits records that it gave up (which the library allocates with cudaMalloc the first
// time a device is used). Some hosts can do neither. A host that has handed all of device
// memory to its own pool has nowhere to take a new buffer from, and a cudaMalloc behind its
// back either fails or takes memory the pool believes it owns. Code that runs where CUDA's
// allocation calls are not permitted at all, because they synchronise the device or may not be
// issued from that context, cannot call them either. For those hosts this entry point keeps
// both pieces in one array that is part of the library's device image: no call allocates or
// frees, the array simply comes with the code. (CUDA places a library's device image, this
// array included, on a GPU when the library is first used there, see below.)
//
// The price is a fixed capacity and shared state:
//   * the array holds delta for at most LIMN_B200_STATIC_MAX_ROWS = 2^20 query rows
//     (bh * t_q), 8 bytes each so that float64 fits, 8 MiB + 256 bytes per GPU that loads the
//     library; a larger problem is refused with LIMN_B200_UNSUPPORTED and nothing is launched;
//   * every call on a device uses the same array. Calls that run one after the other on one
//     stream are ordered by the stream; calls that can overlap on the GPU (different streams,
//     different host threads) race on it and must be serialised by the caller;
//   * the array keeps whatever the last call left. delta is overwritten in full for the rows
//     of the current call before it is read, so nothing stale is ever used; the status word
//     has to start at zero, so each call clears it on the stream before its kernels.
//
// The first call on each device looks the array's device address up. That is a host-side
// query, done once per device with that device current; it should happen before any stream
// capture is begun on that device. With CUDA's default lazy module loading it is also the
// moment the driver places this file's device image (the 8 MiB array) and, at their first
// launch, the images of the row-dot and dQ kernels on that GPU. A host whose pool is about to
// take every free byte should therefore make one small call on each device first (or run with
// CUDA_MODULE_LOADING=EAGER, which places everything when the library is loaded): otherwise that
// first call can fail with an out-of-memory error from the driver, which is reported as
// LIMN_B200_CUDA_ERROR.
#include <cuda_runtime.h>

#include <mutex>

#include "common.h"

namespace limn_b200 {
namespace {

constexpr long long kMaxRows = 1LL << 20;
constexpr size_t kStatusBytes = 256;  // the status word, padded so delta starts 256-byte aligned

// [0, 4): status word. [64, 72): the dQ kernel's two work counters. [256, 256 + 8 * kMaxRows): delta, float or
// double per row.
// In host code this name is only a handle for cudaGetSymbolAddress; it is not a device address.
static __device__ __align__(256) unsigned char g_static_scratch[kStatusBytes + 8 * kMaxRows];

constexpr int kMaxDevices = 64;
std::mutex g_setup_mutex;
unsigned char* g_scratch_address[kMaxDevices] = {};

// Device address of the array on the current device, looked up on first use.
int scratch_address(unsigned char** address) {
  int device = 0;
  LIMN_CUDA(cudaGetDevice(&device), "asking for the current device");
  if (device < 0 || device >= kMaxDevices) return fail(LIMN_B200_UNSUPPORTED, "device ordinal %d out of range", device);
  std::lock_guard<std::mutex> lock(g_setup_mutex);
  if (g_scratch_address[device] == nullptr) {
    void* ptr = nullptr;
    LIMN_CUDA(cudaGetSymbolAddress(&ptr, g_static_scratch), "looking up the static scratch array");
    if (ptr == nullptr) return fail(LIMN_B200_CUDA_ERROR, "cuda: the static scratch array has no device address");
    g_scratch_address[device] = static_cast<unsigned char*>(ptr);
  }
  *address = g_scratch_address[device];
  return LIMN_B200_OK;
}

}  // namespace
}  // namespace limn_b200

using namespace limn_b200;

extern "C" int limn_b200_sdpa_bwd_q_static(const void* q, const void* k, const void* v, const void* out,
                                           const void* dout, const void* lse, const void* key_mask, void* dq,
                                           unsigned int* status_out, int dtype, long long bh, int t_q, int t_k,
                                           int hd, int hd_v, int causal, double scale, void* stream) {
  clear_error();
  reset_launches();
  // Every check comes before the first thing put on the stream: a refused call enqueues nothing and leaves
  // the shared array as it was.
  if (!out || !dout) return fail(LIMN_B200_BAD_ARGUMENT, "sdpa_bwd_q_static: a required pointer is null");
  if (bh < 0 || t_q <= 0) return fail(LIMN_B200_BAD_ARGUMENT, "sdpa_bwd_q_static: extents must be positive");
  const long long rows = bh * t_q;
  if (rows > kMaxRows)
    return fail(LIMN_B200_UNSUPPORTED,
                "sdpa_bwd_q_static: %lld query rows (bh * t_q) exceed the %lld the static scratch holds; "
                "use limn_b200_sdpa_bwd_q with a delta buffer of your own",
                rows, kMaxRows);
  Problem p;
  p.q = q, p.k = k, p.v = v, p.mask = key_mask;
  p.dout = dout, p.lse_in = lse, p.dq = dq;
  p.dtype = dtype, p.bh = bh, p.t_q = t_q, p.t_k = t_k, p.hd = hd, p.hd_v = hd_v;
  p.causal = causal != 0, p.scale = scale, p.stream = static_cast<cudaStream_t>(stream);
  p.delta = out;  // any non-null value for the pointer checks; the real address is filled in below
  if (int rc = validate_op(Op::BwdQ, "sdpa_bwd_q_static", p)) return rc;
  unsigned char* scratch = nullptr;
  if (int rc = scratch_address(&scratch)) return rc;
  cudaStream_t s = p.stream;
  unsigned int* status = reinterpret_cast<unsigned int*>(scratch);
  p.delta = scratch + kStatusBytes;
  p.status = status;
  p.schedule = reinterpret_cast<unsigned int*>(scratch + 64);
  if (rows == 0) return LIMN_B200_OK;
  LIMN_CUDA(cudaMemsetAsync(scratch, 0, 128, s), "clearing the static status word and work counters");
  if (int rc = general_delta(out, dout, scratch + kStatusBytes, dtype, rows, hd_v, s)) return rc;
  if (int rc = dispatch_op(Op::BwdQ, "sdpa_bwd_q_static", p)) return rc;
  note_launches(1);  // the row dot, beside what dispatch_op counted
  if (status_out)
    LIMN_CUDA(cudaMemcpyAsync(status_out, status, sizeof(unsigned int), cudaMemcpyDeviceToDevice, s),
              "handing the status word to the caller");
  return LIMN_B200_OK;
}
