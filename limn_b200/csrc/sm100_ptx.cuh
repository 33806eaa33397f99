// Thin wrappers over the sm_100a PTX the attention kernels are built from: mbarriers with
// bounded waits, TMA tile loads, tensor-memory allocation, tcgen05 MMAs and their
// descriptors, and tensor-memory loads/stores. Nothing here is a library dependency; each
// wrapper is one or two instructions of inline PTX.
#pragma once

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace limn_b200 {
namespace ptx {

// ---- status codes a kernel leaves in the device status word when a bounded wait runs out ----
constexpr unsigned kStatusOk = 0u;
constexpr unsigned kStatusWaitTimeout = 0x57410000u;  // low 16 bits: which wait (role << 8 | barrier id)

// A wait gives up after this many clock64() ticks (a few seconds at B200 clocks): far beyond
// any legitimate wait, short enough that a mis-armed barrier ends the kernel, not the GPU.
constexpr long long kWaitBudgetTicks = 4000000000LL;

__device__ __forceinline__ uint32_t smem_addr(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ uint32_t lane_id() {
  uint32_t x;
  asm volatile("mov.u32 %0, %%laneid;" : "=r"(x));
  return x;
}

// One lane of a converged warp, chosen by the hardware.
__device__ __forceinline__ bool elect_one() {
  uint32_t pred = 0;
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "elect.sync _|p, 0xffffffff;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t"
      "}\n"
      : "=r"(pred));
  return pred != 0;
}

// ---- mbarrier ----
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_init_fence() {
  // make the initialised barriers visible to the async proxy (TMA, tcgen05.commit)
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t done;
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t"
      "}\n"
      : "=r"(done)
      : "r"(bar), "r"(parity)
      : "memory");
  return done != 0;
}

// Wait for the phase with the given parity to complete, or give up: returns false after `budget` clock64()
// ticks, having recorded `tag` in the status word. Callers leave their loops on false.
__device__ __forceinline__ bool mbar_wait_for(uint32_t bar, uint32_t parity, unsigned* status, unsigned tag, long long budget) {
  if (mbar_try_wait(bar, parity)) return true;
  const long long start = clock64();
  for (;;) {
#pragma unroll 1
    for (int spin = 0; spin < 256; ++spin)
      if (mbar_try_wait(bar, parity)) return true;
    if (clock64() - start > budget) {
      atomicCAS(status, kStatusOk, kStatusWaitTimeout | (tag & 0xffffu));
      return false;
    }
    if (*reinterpret_cast<volatile unsigned*>(status) != kStatusOk) return false;  // someone else already gave up
  }
}
// The wait every kernel uses: the budget is kWaitBudgetTicks.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, unsigned* status, unsigned tag) {
  return mbar_wait_for(bar, parity, status, tag, kWaitBudgetTicks);
}

// ---- programmatic dependent launch ----
// A kernel launched with the programmatic-serialization attribute may start while the kernel before it in the
// stream is still running its last CTAs; grid_dependency_wait() is where it then waits until that kernel has
// finished and its writes are visible (a no-op when the kernel was launched the ordinary way). Nothing that
// reads or writes global memory may come before it. grid_launch_dependents() tells the scheduler that the
// kernel after this one may begin the same way as soon as this one's CTAs make room.
__device__ __forceinline__ void grid_dependency_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void grid_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// ---- fences ----
__device__ __forceinline__ void fence_async_shared() {
  // generic-proxy writes to shared memory -> visible to the async proxy (TMA store, MMA operands)
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_before_sync() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after_sync() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}

// ---- TMA: 4-D tiled load (element, row, head, batch) global -> shared, completion on an mbarrier; every CTA fetches its own tiles ----
__device__ __forceinline__ void tma_prefetch_descriptor(const CUtensorMap* map) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(map)) : "memory");
}
// c0 is the innermost coordinate (elements); it must be a multiple of 16 bytes worth of elements.
__device__ __forceinline__ void tma_load_4d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int c0, int c1,
                                            int c2, int c3) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
      : "memory");
}

// ---- tensor memory ----
// Allocate `cols` columns (power of two, 32..512); the base address lands in *slot (shared).
// Executed by one whole warp; the same warp frees it.
// A tile store from shared memory (in the tensor map's box layout) to global memory, asynchronous: rows and columns
// of the box that lie outside the tensor are not written. Stores issued by a thread form groups (tma_store_commit);
// tma_store_wait_read returns once all of that thread's groups have finished reading shared memory.
__device__ __forceinline__ void tma_store_4d(const CUtensorMap* map, uint32_t src, int c0, int c1, int c2, int c3) {
  asm volatile("cp.async.bulk.tensor.4d.global.shared::cta.tile.bulk_group [%0, {%2, %3, %4, %5}], [%1];" ::"l"(
                   reinterpret_cast<uint64_t>(map)),
               "r"(src), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
               : "memory");
}
__device__ __forceinline__ void tma_store_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
__device__ __forceinline__ void tma_store_wait_read() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
// Where the 16-byte piece `piece` (0..7) of row `row` lies in a 128-byte-swizzled tile of 128-byte rows at `tile`
// (1024-byte aligned): the layout TMA reads and writes with CU_TENSOR_MAP_SWIZZLE_128B.
__device__ __forceinline__ uint32_t swizzled_piece(uint32_t tile, int row, int piece) {
  return tile + static_cast<uint32_t>(row) * 128u + (static_cast<uint32_t>(piece ^ (row & 7)) << 4);
}
__device__ __forceinline__ void st_shared_v4(uint32_t addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
  asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}

__device__ __forceinline__ void tmem_alloc(uint32_t slot, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(slot), "r"(cols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_free(uint32_t base, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(base), "r"(cols) : "memory");
}

// ---- descriptors ----
// Shared-memory matrix descriptor for a 128-byte-swizzled operand tile whose rows are 128
// bytes (64 two-byte elements) apart, as TMA writes it with CU_TENSOR_MAP_SWIZZLE_128B.
//   K-major operand (the contraction dim is the contiguous one): stride_bytes = 1024, the
//     distance between 8-row groups; leading_bytes is not used by the hardware.
//   MN-major operand (the M or N dim is contiguous): leading_bytes = distance between
//     64-element column blocks along M/N, stride_bytes = 1024 = distance between groups of
//     8 rows along K.
__device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t addr, uint32_t leading_bytes, uint32_t stride_bytes) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((addr & 0x3ffffu) >> 4);               // bits 0-13: start address
  d |= static_cast<uint64_t>((leading_bytes >> 4) & 0x3fffu) << 16;  // bits 16-29
  d |= static_cast<uint64_t>((stride_bytes >> 4) & 0x3fffu) << 32;   // bits 32-45
  d |= 1ull << 46;                                                   // bits 46-47: descriptor version (sm_100)
  d |= 2ull << 61;                                                   // bits 61-63: 128-byte swizzle
  return d;
}

// Instruction descriptor for tcgen05.mma.kind::f16: fp32 accumulate, A and B both bf16 or
// both fp16. a_mn / b_mn say the operand is MN-major (0 = K-major).
__host__ __device__ constexpr uint32_t mma_idesc(int m, int n, bool fp16, bool a_mn, bool b_mn) {
  return (1u << 4)                      // D format: f32
         | ((fp16 ? 0u : 1u) << 7)      // A format: f16 = 0, bf16 = 1
         | ((fp16 ? 0u : 1u) << 10)     // B format
         | ((a_mn ? 1u : 0u) << 15)     // A major
         | ((b_mn ? 1u : 0u) << 16)     // B major
         | (static_cast<uint32_t>(n >> 3) << 17)
         | (static_cast<uint32_t>(m >> 4) << 24);
}

// D[tmem] (+)= A[smem] * B[smem]; one thread issues for the CTA.
__device__ __forceinline__ void mma_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                       uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t"
      "}\n" ::"r"(d_tmem),
      "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// D[tmem] (+)= A[tmem] * B[smem]: A's rows sit on the 128 lanes, two 16-bit elements per column.
__device__ __forceinline__ void mma_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc,
                                       uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t"
      "}\n" ::"r"(d_tmem),
      "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// The same descriptor split into words, so an issue loop adds a constant to the low word
// instead of rebuilding 64 bits per instruction (one thread issues every MMA of a CTA, and
// its instruction count is on the critical path). The high word is the same for every
// 128-byte-swizzled tile with 1024-byte groups; the low word holds the address and the
// leading offset, and advancing the address by `bytes` adds bytes >> 4 to it.
constexpr uint32_t kDescHiSw128 = (1024u >> 4) | (1u << 14) | (2u << 29);
__device__ __forceinline__ uint32_t desc_lo(uint32_t addr, uint32_t leading_bytes) {
  return ((addr & 0x3ffffu) >> 4) | (((leading_bytes >> 4) & 0x3fffu) << 16);
}
template <bool kAccumulate>
__device__ __forceinline__ void mma_ss_lo(uint32_t d_tmem, uint32_t a_lo, uint32_t b_lo, uint32_t idesc) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      ".reg .b64 da, db;\n\t"
      "mov.b64 da, {%1, %4};\n\t"
      "mov.b64 db, {%2, %4};\n\t"
      "setp.ne.b32 p, %5, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %3, p;\n\t"
      "}\n" ::"r"(d_tmem),
      "r"(a_lo), "r"(b_lo), "r"(idesc), "r"(kDescHiSw128), "n"(kAccumulate ? 1 : 0)
      : "memory");
}
__device__ __forceinline__ void mma_ts_lo(uint32_t d_tmem, uint32_t a_tmem, uint32_t b_lo, uint32_t idesc,
                                          uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      ".reg .b64 db;\n\t"
      "mov.b64 db, {%2, %4};\n\t"
      "setp.ne.b32 p, %5, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], db, %3, p;\n\t"
      "}\n" ::"r"(d_tmem),
      "r"(a_tmem), "r"(b_lo), "r"(idesc), "r"(kDescHiSw128), "r"(accumulate)
      : "memory");
}

// The barrier gets one arrival when every MMA this thread issued before now has finished.
__device__ __forceinline__ void mma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

// ---- tensor memory <-> registers. A warp reaches the 32 lanes starting at 32 * (warp % 4);
// with the 32x32b shape thread t gets lane base+t and `N` consecutive 32-bit columns. ----
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};" ::"r"(taddr),
      "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
      "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]),
      "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]),
      "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};" ::"r"(taddr),
      "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
      "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
      : "memory");
}

// ---- small numeric helpers ----
__device__ __forceinline__ float exp2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
// Two floats rounded to nearest-even and packed, `lo` in the low half-word.
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  uint32_t r;
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
  return r;
}
__device__ __forceinline__ uint32_t pack_f16(float lo, float hi) {
  uint32_t r;
  asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
  return r;
}

// ---- packed fp32 pairs (one instruction, two lanes of math) ----
__device__ __forceinline__ uint64_t f2_pack(float lo, float hi) {
  uint64_t r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
  return r;
}
__device__ __forceinline__ uint64_t f2_pack_bits(uint32_t lo, uint32_t hi) {
  uint64_t r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "r"(lo), "r"(hi));
  return r;
}
__device__ __forceinline__ void f2_unpack(uint64_t v, float& lo, float& hi) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ uint64_t f2_fma(uint64_t a, uint64_t b, uint64_t c) {
  uint64_t r;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
  return r;
}
__device__ __forceinline__ uint64_t f2_add(uint64_t a, uint64_t b) {
  uint64_t r;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
  return r;
}
__device__ __forceinline__ uint64_t f2_mul(uint64_t a, uint64_t b) {
  uint64_t r;
  asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
  return r;
}
__device__ __forceinline__ float max3(float a, float b, float c) {
  float r;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(b), "f"(c));
  return r;
}

// 2^x for two values on the FMA pipe instead of the special-function unit: round x to the
// nearest integer n with the 1.5 * 2^23 trick, evaluate a cubic for 2^(x - n) on [-0.5, 0.5]
// (max relative error 7.5e-5), and add n into the exponent field. x is clamped at -125 so the
// exponent stays in the normal range; values that small stand for 0.
__device__ __forceinline__ void exp2_poly2(uint64_t x2, float& lo, float& hi) {
  float x0, x1;
  f2_unpack(x2, x0, x1);
  x2 = f2_pack(fmaxf(x0, -125.f), fmaxf(x1, -125.f));
  const uint64_t magic = f2_pack(12582912.f, 12582912.f);
  const uint64_t t2 = f2_add(x2, magic);
  const uint64_t n2 = f2_add(t2, f2_pack(-12582912.f, -12582912.f));
  const uint64_t r2 = f2_fma(n2, f2_pack(-1.f, -1.f), x2);
  uint64_t p2 = f2_fma(f2_pack(0.0551716685f, 0.0551716685f), r2, f2_pack(0.2426111400f, 0.2426111400f));
  p2 = f2_fma(p2, r2, f2_pack(0.6932609677f, 0.6932609677f));
  p2 = f2_fma(p2, r2, f2_pack(0.9999280572f, 0.9999280572f));
  float t0, t1, p0, p1;
  f2_unpack(t2, t0, t1);
  f2_unpack(p2, p0, p1);
  lo = __int_as_float(__float_as_int(p0) + (__float_as_int(t0) << 23));
  hi = __int_as_float(__float_as_int(p1) + (__float_as_int(t1) << 23));
}

// Which (problem, slot) work item `index` is. Items are fetched in index order, so the order is the schedule:
// problems go in groups of `group` whose K and V stay in L2 together, and inside a group the slots are walked
// outermost, all of the group's problems per slot. With `slot 0 = the longest stream` (causal) that is
// longest-first within a group, and a group ends with its shortest items, which keeps the tail short. The
// host picks the group as large as L2 allows (work_group below): a GPU that holds only a few dozen
// problems then runs them as one group, longest items of all problems first.
__device__ __forceinline__ void cta_work(int index, int slots, long long bh, int group_size, int& problem, int& slot) {
  const int per_group = group_size * slots;
  const int group = index / per_group;
  const int first = group * group_size;
  const int members = static_cast<int>(bh - first < group_size ? bh - first : group_size);
  const int within = index - group * per_group;
  slot = within / members;
  problem = first + within - slot * members;
}

}  // namespace ptx
}  // namespace limn_b200
