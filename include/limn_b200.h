/* limn_b200: fused scaled-dot-product attention for NVIDIA B200 (sm_100a), C ABI.
 *
 * These are the entry points a host binds in place of the three CUSTOM kernels limn's cuda
 * device compiles with NVRTC (limn/backend_cuda.py:352-361 builds them from the emitters at
 * limn/cuda_emit.py:921-1083). Every tensor is dense row-major with its leading dims
 * flattened into `bh` independent problems, exactly as the reference's block decoding does
 * (limn/cuda_emit.py:765-775, :853-862). All pointers are device pointers unless a function
 * says otherwise; nothing here allocates per call, synchronises, or keeps a pointer after
 * it returns. Kernels are enqueued on `stream` (NULL = the legacy default stream, which is
 * where limn launches: limn/backend_cuda.py:413).
 *
 * Every function returns 0 on success and a non-zero code otherwise; the message for the
 * calling thread's last failure is limn_b200_last_error(). The host binding turns that
 * into the RuntimeError the reference raises from check() (limn/backend_cuda.py:154-162).
 */
#ifndef LIMN_B200_H
#define LIMN_B200_H

#ifdef __cplusplus
extern "C" {
#endif

/* Storage dtypes of q, k, v, dO and the outputs (limn/ops.py:24-27). The row statistics
 * L and delta are float32 for F32/F16/BF16 and float64 for F64 (limn/ops.py:53-62). */
enum limn_b200_dtype {
  LIMN_B200_F32 = 0,
  LIMN_B200_F16 = 1,
  LIMN_B200_BF16 = 2,
  LIMN_B200_F64 = 3
};

enum limn_b200_status {
  LIMN_B200_OK = 0,
  LIMN_B200_BAD_ARGUMENT = 1,   /* null pointer, non-positive extent, causal with t_q != t_k, unknown dtype */
  LIMN_B200_UNSUPPORTED = 2,    /* extents beyond what any kernel here serves */
  LIMN_B200_CUDA_ERROR = 3,     /* a CUDA runtime/driver call failed; the message names it */
  LIMN_B200_DEVICE_TIMEOUT = 4  /* a kernel gave up on a bounded wait; see limn_b200_device_status */
};

/* Which kernel family served (or would serve) a problem. */
enum limn_b200_path {
  LIMN_B200_PATH_GENERAL = 0,  /* SIMT kernels: any float dtype, any hd/hd_v */
  LIMN_B200_PATH_TCGEN05 = 1,  /* TMA + tcgen05 kernels: f16/bf16, hd and hd_v multiples of 8 up to 128 (run as 64 or 128), any t_q/t_k, with or without key mask */
  LIMN_B200_PATH_DECODE = 2    /* forward only: f16/bf16, hd == hd_v in {64, 128}, t_q <= 4 without a causal mask (the step of a
                                  kv cache): one CTA streams a problem's keys and values once, bound by HBM, no tensor cores */
};

/* "sdpa": replaces emit_sdpa (limn/cuda_emit.py:921-965); oracle limn/sdpa.py:91-137.
 *   q (bh, t_q, hd), k (bh, t_k, hd), v (bh, t_k, hd_v), key_mask (bh, t_k) in the same dtype
 *   or NULL (0 hides a key), out (bh, t_q, hd_v) in the same dtype, lse (bh, t_q) float32
 *   (float64 for F64). A query row with no visible key gets NaN and lse = -inf. */
int limn_b200_sdpa_fwd(const void* q, const void* k, const void* v, const void* key_mask,
                       void* out, void* lse,
                       int dtype, long long bh, int t_q, int t_k, int hd, int hd_v,
                       int causal, double scale, void* stream);

/* "sdpa_bwd_q": replaces emit_sdpa_bwd_q (limn/cuda_emit.py:968-1005); oracle limn/sdpa.py:140-170.
 *   dout (bh, t_q, hd_v); lse and delta (bh, t_q) in the statistics dtype; dq (bh, t_q, hd). */
int limn_b200_sdpa_bwd_q(const void* q, const void* k, const void* v, const void* dout,
                         const void* lse, const void* delta, const void* key_mask,
                         void* dq,
                         int dtype, long long bh, int t_q, int t_k, int hd, int hd_v,
                         int causal, double scale, void* stream);

/* "sdpa_bwd_q" with the row dot folded in: the same dQ as limn_b200_sdpa_delta followed by limn_b200_sdpa_bwd_q,
 * one launch and one pass over O and dO fewer where that is the faster way (short sequences); for dense operands
 * with more than 512 keys the call runs the row-dot kernel and the dQ kernel itself, which is faster there. Either
 * way one call. Replaces the pair limn's frontend schedules between the forward and
 * the backward ops (the reduce of limn/tensor.py:705-706 and emit_sdpa_bwd_q, limn/cuda_emit.py:968-1005).
 *   out is the forward's O (bh, t_q, hd_v), an input here; delta (bh, t_q) in the statistics dtype is an OUTPUT:
 *   every CTA computes the statistic of the query rows it owns from their rows of O and dO and leaves it there for
 *   limn_b200_sdpa_bwd_kv, which needs it for every query it streams and therefore has to run after this call. */
int limn_b200_sdpa_bwd_q_fused(const void* q, const void* k, const void* v, const void* out, const void* dout,
                               const void* lse, const void* key_mask,
                               void* dq, void* delta,
                               int dtype, long long bh, int t_q, int t_k, int hd, int hd_v,
                               int causal, double scale, void* stream);

/* "sdpa_bwd_kv": replaces emit_sdpa_bwd_kv (limn/cuda_emit.py:1008-1083); oracle limn/sdpa.py:173-203.
 *   dk (bh, t_k, hd), dv (bh, t_k, hd_v). Rows of a hidden key are written as exact zeros. */
int limn_b200_sdpa_bwd_kv(const void* q, const void* k, const void* v, const void* dout,
                          const void* lse, const void* delta, const void* key_mask,
                          void* dk, void* dv,
                          int dtype, long long bh, int t_q, int t_k, int hd, int hd_v,
                          int causal, double scale, void* stream);

/* dQ for hosts that must not allocate. No counterpart in the reference: limn's frontend always
 * brings delta in a buffer of its own (limn/tensor.py:705-707) and its cuda device allocates freely.
 *   Same result as limn_b200_sdpa_delta followed by limn_b200_sdpa_bwd_q, but delta and the kernels'
 *   status word live in a fixed array inside the library image instead of in memory somebody has to
 *   allocate: a host whose own pool holds all device memory, or code that runs where CUDA allocation
 *   calls are not allowed, passes only inputs and outputs. `out` is the forward's O (bh, t_q, hd_v);
 *   `status_out` is an optional device word that receives the kernels' status (0 = no wait gave up).
 *   Limits: bh * t_q <= LIMN_B200_STATIC_MAX_ROWS, else LIMN_B200_UNSUPPORTED and nothing is launched.
 *   All calls on a device share the array: calls that can overlap on the GPU race and must be
 *   serialised by the caller. The first call on a device looks the array's address up (and, with CUDA's lazy
 *   module loading, is when the driver places the array and the kernels on that GPU): make it before any
 *   stream capture on that device and while the device still has ~10 MiB free, or set CUDA_MODULE_LOADING=EAGER.
 *   Every argument check happens before anything is enqueued: a refused call launches nothing and leaves the
 *   array untouched. */
#define LIMN_B200_STATIC_MAX_ROWS (1LL << 20)
int limn_b200_sdpa_bwd_q_static(const void* q, const void* k, const void* v, const void* out,
                                const void* dout, const void* lse, const void* key_mask,
                                void* dq, unsigned int* status_out,
                                int dtype, long long bh, int t_q, int t_k, int hd, int hd_v,
                                int causal, double scale, void* stream);

/* delta = sum_d dout * out per query row, in the statistics dtype: the row dot the frontend
 * computes between the forward and the two backward ops (limn/tensor.py:705-706). Offered so
 * a host that drives the three ops directly need not bring its own reduce kernel. */
int limn_b200_sdpa_delta(const void* out, const void* dout, void* delta,
                         int dtype, long long rows, int hd_v, void* stream);

/* ---- operands as the model holds them: (batch, t, heads, hd) ----
 * limn's frontend permutes (batch, t, heads, hd) activations to (batch, heads, t, hd) and wraps each operand in
 * CONTIGUOUS before the CUSTOM node (limn/tensor.py:561-562; the gradient of that permute copies again on the way
 * back, limn/tensor.py:736-746), so every attention call is surrounded by full-tensor copies. These entry points
 * read and write the token-major layout in place through the tensor maps' strides, so a frontend that skips the
 * permute can skip the copies too. They have no counterpart in the reference.
 *   layout LIMN_B200_BHTD: q, k, v, dout, out, dq, dk, dv are (batch, heads, t, hd) dense: the same as the entry
 *     points above with bh = batch * heads.
 *   layout LIMN_B200_BTHD: they are (batch, t, heads, hd) dense.
 *   Either way lse and delta are (batch * heads, t_q) and key_mask (batch * heads, t_k), as above.
 *   LIMN_B200_BTHD is served for f16/bf16 with hd and hd_v multiples of 8 up to 128 (the tensor-core kernels); anything else
 *   returns LIMN_B200_UNSUPPORTED and launches nothing. */
enum limn_b200_layout {
  LIMN_B200_BHTD = 0,
  LIMN_B200_BTHD = 1
};
int limn_b200_sdpa_fwd_layout(const void* q, const void* k, const void* v, const void* key_mask,
                              void* out, void* lse,
                              int layout, int dtype, int batch, int heads, int t_q, int t_k, int hd, int hd_v,
                              int causal, double scale, void* stream);
int limn_b200_sdpa_bwd_q_layout(const void* q, const void* k, const void* v, const void* dout,
                                const void* lse, const void* delta, const void* key_mask,
                                void* dq,
                                int layout, int dtype, int batch, int heads, int t_q, int t_k, int hd, int hd_v,
                                int causal, double scale, void* stream);
int limn_b200_sdpa_bwd_q_fused_layout(const void* q, const void* k, const void* v, const void* out, const void* dout,
                                      const void* lse, const void* key_mask,
                                      void* dq, void* delta,
                                      int layout, int dtype, int batch, int heads, int t_q, int t_k, int hd, int hd_v,
                                      int causal, double scale, void* stream);
int limn_b200_sdpa_bwd_kv_layout(const void* q, const void* k, const void* v, const void* dout,
                                 const void* lse, const void* delta, const void* key_mask,
                                 void* dk, void* dv,
                                 int layout, int dtype, int batch, int heads, int t_q, int t_k, int hd, int hd_v,
                                 int causal, double scale, void* stream);
int limn_b200_sdpa_delta_layout(const void* out, const void* dout, void* delta,
                                int layout, int dtype, int batch, int heads, int t_q, int hd_v, void* stream);

/* ---- operands with strides of their own ----
 * q, k and v of an attention layer are usually slices of one projection's output, (batch, t, 3, heads, hd), and the
 * layer's result is wanted as (batch, t, heads * hd): no single layout describes both. These entry points take one
 * (batch, head, row) stride triple per operand, in elements (columns are contiguous; every stride a multiple of 8,
 * every pointer 16-byte aligned and already offset to the operand's first element), so a frontend can hand over its
 * views as they are instead of copying them (limn/tensor.py:561-562, :736-746 make those copies). lse and delta stay
 * (batch * heads, t_q), key_mask (batch * heads, t_k). No counterpart in the reference. f16/bf16 with hd and hd_v
 * multiples of 8 up to 128 only; anything else returns LIMN_B200_UNSUPPORTED and launches nothing.
 *   limn_b200_sdpa_fwd_strided:          strides of q, k, v, out                 (4 triples)
 *   limn_b200_sdpa_bwd_q_fused_strided:  strides of q, k, v, out, dout, dq        (6 triples); delta is written
 *   limn_b200_sdpa_bwd_kv_strided:       strides of q, k, v, dout, dk, dv         (6 triples) */
int limn_b200_sdpa_fwd_strided(const void* q, const void* k, const void* v, const void* key_mask,
                               void* out, void* lse, const long long* strides,
                               int dtype, int batch, int heads, int t_q, int t_k, int hd, int hd_v,
                               int causal, double scale, void* stream);
int limn_b200_sdpa_bwd_q_fused_strided(const void* q, const void* k, const void* v, const void* out, const void* dout,
                                       const void* lse, const void* key_mask,
                                       void* dq, void* delta, const long long* strides,
                                       int dtype, int batch, int heads, int t_q, int t_k, int hd, int hd_v,
                                       int causal, double scale, void* stream);
int limn_b200_sdpa_bwd_kv_strided(const void* q, const void* k, const void* v, const void* dout,
                                  const void* lse, const void* delta, const void* key_mask,
                                  void* dk, void* dv, const long long* strides,
                                  int dtype, int batch, int heads, int t_q, int t_k, int hd, int hd_v,
                                  int causal, double scale, void* stream);

/* Which path the dispatcher picks for a problem (a limn_b200_path value), or -1 with an
 * error message if the arguments are invalid. Launches nothing. */
int limn_b200_sdpa_path(int dtype, long long bh, int t_q, int t_k, int hd, int hd_v,
                        int causal, int has_mask, double scale);

/* How many kernels the last successful limn_b200_sdpa_* call on this thread enqueued. */
int limn_b200_last_launch_count(void);

/* Message for the calling thread's most recent failure ("" if none). Stands where the
 * driver's error string stands in limn/backend_cuda.py:154-162. */
const char* limn_b200_last_error(void);

/* Library version, major * 10000 + minor * 100 + patch. */
int limn_b200_version(void);

/* Kernels that wait (on TMA or tensor-core completion) give up after a bounded time and
 * record a code in a per-device status word instead of hanging; kernels launched on that device
 * afterwards return at once, writing nothing, until the word has been read. This synchronises the
 * current device, reads its word into *status and clears it. Returns LIMN_B200_OK with *status == 0
 * when no kernel gave up, LIMN_B200_DEVICE_TIMEOUT with *status = 0x5741rrbb (role rr, barrier bb)
 * when one did. The reference reports a failed kernel from its batch barrier
 * (limn/backend_cuda.py:349 through check(), :154-162); limn_b200.install() makes finish() call this. */
int limn_b200_device_status(unsigned int* status);

/* Diagnostic, no counterpart in the reference: one warp waits on a barrier nobody arrives at, with the
 * production kernels' bounded wait but a budget of `budget_ticks` clock ticks (at most 1e8), so that the wait
 * runs out, the status word of the current device receives 0x57417e57 and the kernel returns normally.
 * `gave_up` is an optional device word that receives 1 (the wait ran out) or 0. It lets a test walk the
 * give-up path (status code, later launches standing down, counters left clean, read-and-clear) without
 * making any production kernel misbehave and without hanging or faulting anything. */
int limn_b200_wait_probe(long long budget_ticks, unsigned int* gave_up, void* stream);

/* ---- the gather of (batch, head) shards over NCCL, for sharded hosts without a communication library of their own ----
 * No counterpart in the reference, which is single-GPU (limn/backend_cuda.py:283 takes device 0). The problems of a
 * batch are independent: rank r of N computes problems [r BH/N, (r+1) BH/N) with the entry points above and no
 * communication, and the outputs are then gathered into one tensor on every GPU. One process per GPU, one
 * communicator per process; NCCL (libnccl.so.2, or the file LIMN_B200_NCCL_LIBRARY names) is loaded when the first of
 * these is called, so a single-GPU host never needs it. Failures come back as status codes with a message, never as
 * an abort: LIMN_B200_UNSUPPORTED when NCCL cannot be loaded, LIMN_B200_BAD_ARGUMENT for a misuse,
 * LIMN_B200_CUDA_ERROR with NCCL's own error string otherwise.
 *   limn_b200_nccl_unique_id: rank 0 fills LIMN_B200_NCCL_ID_BYTES bytes (host memory); the host carries them to the
 *     other ranks by whatever means it has (a file, a socket, its launcher).
 *   limn_b200_nccl_init: every rank, with its own device current, the same id and world size.
 *   limn_b200_nccl_all_gather: recv (world * bytes_per_rank bytes) receives every rank's send (bytes_per_rank bytes) in
 *     rank order, enqueued on `stream`; send may be the rank's own slice of recv.
 *   limn_b200_nccl_destroy: releases the communicator. */
#define LIMN_B200_NCCL_ID_BYTES 128
int limn_b200_nccl_unique_id(void* id_out);
int limn_b200_nccl_init(int rank, int world, const void* id);
int limn_b200_nccl_all_gather(const void* send, void* recv, unsigned long long bytes_per_rank, void* stream);
int limn_b200_nccl_destroy(void);

/* ---- plumbing for hosts without a CUDA binding of their own (tests, benchmark) ----
 * limn itself allocates and copies through the driver API (limn/backend_cuda.py:297-326)
 * and never calls these. */
int limn_b200_device_count(int* count);
int limn_b200_set_device(int ordinal);
int limn_b200_mem_alloc(void** device_ptr, unsigned long long nbytes);
int limn_b200_mem_free(void* device_ptr);
int limn_b200_mem_set(void* device_ptr, int byte, unsigned long long nbytes, void* stream);
int limn_b200_host_alloc(void** pinned_ptr, unsigned long long nbytes);
int limn_b200_host_free(void* pinned_ptr);
int limn_b200_copy_h2d(void* device_dst, const void* host_src, unsigned long long nbytes, void* stream);
int limn_b200_copy_d2h(void* host_dst, const void* device_src, unsigned long long nbytes, void* stream);
int limn_b200_copy_d2d(void* device_dst, const void* device_src, unsigned long long nbytes, void* stream);
int limn_b200_stream_create(void** stream);
int limn_b200_stream_destroy(void* stream);
int limn_b200_stream_wait_event(void* stream, void* event);
int limn_b200_stream_sync(void* stream);
int limn_b200_device_sync(void);
int limn_b200_event_create(void** event);
int limn_b200_event_destroy(void* event);
int limn_b200_event_record(void* event, void* stream);
int limn_b200_event_elapsed_ms(void* start, void* stop, float* ms);

#ifdef __cplusplus
}
#endif
#endif /* LIMN_B200_H */
