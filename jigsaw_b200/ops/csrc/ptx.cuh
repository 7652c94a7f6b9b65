// Thin inline-PTX wrappers for the Blackwell (sm_100a) execution model:
// mbarrier, TMA (cp.async.bulk.tensor, never with a cluster multicast qualifier),
// tcgen05 (TMEM allocation, UMMA issue, commit, TMEM loads) and the shared-memory /
// instruction descriptors they consume.  Every wait in this file is bounded: after
// a time limit it records an error code in a status word and returns false, so a
// kernel can drain and exit instead of hanging the GPU.
#pragma once

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace jb {

// Error codes written to the status word by bounded waits.
enum : int {
  JB_OK = 0,
  JB_ERR_MBAR_TIMEOUT = 1,   // an mbarrier phase never completed
  JB_ERR_FLAG_TIMEOUT = 2,   // a cross-GPU flag never reached the expected epoch
  JB_ERR_BAD_ARG = 3,
};

// Upper bound of any single wait, in nanoseconds of %globaltimer.
#ifndef JB_WAIT_LIMIT_NS
#define JB_WAIT_LIMIT_NS 2000000000ull
#endif

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ uint64_t globaltimer_ns() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}

__device__ __forceinline__ bool elect_one() {
  uint32_t pred;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "elect.sync _|p, 0xffffffff;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(pred));
  return pred != 0;
}

// ---------------------------------------------------------------- mbarrier
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void fence_mbar_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}

// Bounded wait on an mbarrier phase.  `abort_flag` lives in shared memory and is
// set by whichever wait of the CTA gives up first; once set, every later wait
// returns false at once.  Callers do NOT branch on the result: the role loops keep their
// uniform trip counts (which lets the compiler hold descriptors and loop state in uniform
// registers) and simply run to the end without waiting, on whatever data is there; the
// host sees the error code in the status word and discards the result.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag,
                                          int* status, int where = 0) {
  if (mbar_try_wait(bar, parity)) return true;
  if (*abort_flag) return false;   // an earlier wait of this CTA gave up: drain without waiting
  const uint64_t t0 = globaltimer_ns();
  uint32_t spins = 0;
  while (true) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((++spins & 63u) == 0u) {
      if (*abort_flag) return false;
      if (globaltimer_ns() - t0 > JB_WAIT_LIMIT_NS) {
        *abort_flag = 1;
        if (status && atomicCAS(status, JB_OK, JB_ERR_MBAR_TIMEOUT) == JB_OK) {
          status[1] = where;                 // which wait gave up (kernel-specific code)
          status[2] = static_cast<int>(blockIdx.x);
          status[3] = static_cast<int>(threadIdx.x);
        }
        return false;
      }
    }
  }
}

// ---------------------------------------------------------------- proxies / fences
__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_before_sync() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after_sync() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}

// ---------------------------------------------------------------- TMA (local memory only)
__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap* m) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(m) : "memory");
}
__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* m, uint64_t* bar, int c0, int c1) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(dst)), "l"(m), "r"(smem_u32(bar)), "r"(c0), "r"(c1)
      : "memory");
}
__device__ __forceinline__ void tma_load_3d(void* dst, const CUtensorMap* m, uint64_t* bar, int c0, int c1,
                                            int c2) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(smem_u32(dst)), "l"(m), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2)
      : "memory");
}
__device__ __forceinline__ void tma_load_4d(void* dst, const CUtensorMap* m, uint64_t* bar, int c0, int c1,
                                            int c2, int c3) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
      ::"r"(smem_u32(dst)), "l"(m), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
      : "memory");
}

// TMA store of a shared-memory tile (bulk async-group completion).  Coordinates beyond the
// tensor's extents are clipped, never written.
__device__ __forceinline__ void tma_store_4d(const CUtensorMap* m, const void* src, int c0, int c1, int c2, int c3) {
  asm volatile("cp.async.bulk.tensor.4d.global.shared::cta.tile.bulk_group [%0, {%2, %3, %4, %5}], [%1];"
               ::"l"(m), "r"(smem_u32(src)), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
               : "memory");
}
__device__ __forceinline__ void bulk_commit_group() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// All committed bulk stores have finished READING their shared-memory source.
__device__ __forceinline__ void bulk_wait_read_all() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
// All committed bulk stores have completed.
__device__ __forceinline__ void bulk_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
// Barrier among `count` threads (a multiple of 32) of the CTA; id 1..15 (0 is __syncthreads).
__device__ __forceinline__ void named_barrier(int id, int count) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(count) : "memory");
}

// ---------------------------------------------------------------- TMEM
// Allocation is done by one full warp; ncols is a power of two in [32, 512].
__device__ __forceinline__ void tmem_alloc(uint32_t* smem_dst, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_dst)),
               "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}

// D[tmem] (+)= A[smem desc] * B[smem desc]; issued by ONE thread.
__device__ __forceinline__ void umma_f16(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                         uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Arrive on an mbarrier once every UMMA issued so far by this thread has finished.
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
               : "memory");
}

// Warp-convergent issue: the whole warp runs the (uniform) address arithmetic so that the
// compiler can keep descriptors in uniform registers; one elected lane issues the instruction.
__device__ __forceinline__ void umma_f16_elect(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                               uint32_t accumulate) {
  if (elect_one()) umma_f16(d_tmem, adesc, bdesc, idesc, accumulate);
}
__device__ __forceinline__ void umma_commit_elect(uint64_t* bar) {
  if (elect_one()) umma_commit(bar);
}

// 32 lanes x 32 columns of fp32 accumulators -> 32 registers per thread.  The warp
// reads the TMEM lane quadrant (warp_idx % 4); taddr = (lane << 16) | column.
__device__ __forceinline__ void tmem_ld_32x32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
        "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]),
        "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]),
        "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_32x16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
// 32 registers per thread -> 32 lanes x 32 columns of TMEM (the inverse of tmem_ld_32x32).
__device__ __forceinline__ void tmem_st_32x32(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
        "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]),
        "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]),
        "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// ---------------------------------------------------------------- descriptors
// Shared-memory matrix descriptor, 128-byte swizzle.  The tile is made of rows of
// 128 bytes (64 bf16); eight consecutive rows form one 1024-byte swizzle block and
// blocks follow one another every `sbo_bytes`.
//  * K-major operand: a row is one M/N index, its 128 bytes are 64 K values.
//  * MN-major operand: a row is one K index, its 128 bytes are 64 M/N values;
//    `lbo_bytes` is then the distance between consecutive 64-wide M/N blocks.
// The start address may be shifted by whole 128-byte rows (a view of the tile that starts
// a few rows later): the hardware takes the swizzle XOR from the absolute shared-memory
// address bits, exactly as TMA did when it wrote the tile, so the base-offset field stays
// zero.  The convolution numerics tests pin this behaviour.
__device__ __forceinline__ uint64_t make_smem_desc_sw128(uint32_t saddr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((saddr & 0x3FFFFu) >> 4);
  d |= static_cast<uint64_t>((lbo_bytes >> 4) & 0x3FFFu) << 16;
  d |= static_cast<uint64_t>((sbo_bytes >> 4) & 0x3FFFu) << 32;
  d |= static_cast<uint64_t>(1) << 46;                          // descriptor version (Blackwell)
  d |= static_cast<uint64_t>(2) << 61;                          // SWIZZLE_128B
  return d;
}

// Advance the start address of a descriptor by `bytes` (a multiple of 16; no carry out of the
// 14-bit address field as long as the operand stays inside the CTA's shared memory window).
__device__ __forceinline__ uint64_t desc_advance(uint64_t desc, uint32_t bytes) {
  return desc + static_cast<uint64_t>(bytes >> 4);
}

// Instruction descriptor: bf16 x bf16 -> fp32, dense, M in {64,128}, N % 8 == 0 (N % 16 for M=128).
// a_mn / b_mn: 0 = K-major operand, 1 = MN-major operand.
__host__ __device__ constexpr uint32_t make_idesc_bf16(uint32_t M, uint32_t N, uint32_t a_mn, uint32_t b_mn) {
  return (1u << 4)            // D format: F32
         | (1u << 7)          // A format: BF16
         | (1u << 10)         // B format: BF16
         | (a_mn << 15) | (b_mn << 16) | ((N >> 3) << 17) | ((M >> 4) << 24);
}

// ---------------------------------------------------------------- small math helpers
// GELU (erf form) through Phi(x) ~= sigmoid(2 x P(x^2)) with a cubic P fitted to
// atanh(erf(x / sqrt 2)) / x on |x| <= 5 (saturated beyond).  Maximum absolute error against
// the exact erf form: 1.5e-5 for GELU, 5.3e-5 for its derivative, both far below the
// resolution of the bf16 values they are rounded to.  One ex2 and one rcp per element.
#define JB_GELU_C0 0.79775657106f
#define JB_GELU_C1 0.036653938199f
#define JB_GELU_C2 -0.00023358518874f
#define JB_GELU_C3 -1.0182393111e-05f

__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float rcp_approx(float x) {
  float y;
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
// Phi(x) of the standard normal; `t` returns min(|x|, 5)^2 for the derivative.
__device__ __forceinline__ float normal_cdf_fast(float x, float& t) {
  const float ax = fminf(fabsf(x), 5.0f);
  t = ax * ax;
  const float p = fmaf(t, fmaf(t, fmaf(t, JB_GELU_C3, JB_GELU_C2), JB_GELU_C1), JB_GELU_C0);
  const float u = copysignf(ax * p, x);
  // sigmoid(2u) = 1 / (1 + 2^(-2 u log2 e)).  (0.5 + 0.5 tanh.approx(u), one special-function
  // instruction instead of two, measured slower in the convolution epilogue: 0.99 ms against 0.91 ms.)
  return rcp_approx(1.0f + ex2_approx(u * -2.885390081777927f));
}
__device__ __forceinline__ float gelu_erf(float x) {
  float t;
  return x * normal_cdf_fast(x, t);
}
__device__ __forceinline__ float gelu_erf_grad(float x) {
  float t;
  const float P = normal_cdf_fast(x, t);
  // d/dx [x P] = P + x P' with P' = 2 u'(x) P (1 - P), u' = c0 + 3 c1 t + 5 c2 t^2 + 7 c3 t^3
  float du = fmaf(t, fmaf(t, fmaf(t, 7.0f * JB_GELU_C3, 5.0f * JB_GELU_C2), 3.0f * JB_GELU_C1), JB_GELU_C0);
  du = (t < 25.0f) ? du : 0.0f;
  return fmaf(x * (2.0f * du), P * (1.0f - P), P);
}
// GELU(x) and GELU'(x) together (they share Phi): the forward epilogue stores the derivative
// so that the backward pass only multiplies.
__device__ __forceinline__ void gelu_erf_with_grad(float x, float& y, float& dy) {
  float t;
  const float P = normal_cdf_fast(x, t);
  float du = fmaf(t, fmaf(t, fmaf(t, 7.0f * JB_GELU_C3, 5.0f * JB_GELU_C2), 3.0f * JB_GELU_C1), JB_GELU_C0);
  du = (t < 25.0f) ? du : 0.0f;
  y = x * P;
  dy = fmaf(x * (2.0f * du), P * (1.0f - P), P);
}
// Two elements per instruction: the same approximation evaluated in f16x2 arithmetic with one
// tanh.approx.f16x2 for the pair (sigmoid(2u) = 0.5 + 0.5 tanh(u)).  The convolution epilogues are bound by
// instruction issue (about 25 fp32 instructions per element in the scalar form above); this form needs
// about 12.  Error against the exact erf form: below 1.3e-3 absolute for GELU and 1.9e-3 for its
// derivative (emulated over [-8, 8]), the size of the bf16 rounding the results go through anyway.  The
// products with x are formed in fp32 from the unrounded accumulator value.
__device__ __forceinline__ __half2 tanh_approx_h2(__half2 u) {
  uint32_t in = *reinterpret_cast<uint32_t*>(&u), out;
  asm("tanh.approx.f16x2 %0, %1;" : "=r"(out) : "r"(in));
  return *reinterpret_cast<__half2*>(&out);
}
__device__ __forceinline__ __half2 normal_cdf_h2(float x0, float x1, __half2& xc, __half2& t, __half2& th) {
  const __half2 x = __floats2half2_rn(x0, x1);
  xc = __hmin2(__hmax2(x, __float2half2_rn(-5.0f)), __float2half2_rn(5.0f));
  t = __hmul2(xc, xc);
  __half2 p = __hfma2(t, __float2half2_rn(JB_GELU_C3), __float2half2_rn(JB_GELU_C2));
  p = __hfma2(p, t, __float2half2_rn(JB_GELU_C1));
  p = __hfma2(p, t, __float2half2_rn(JB_GELU_C0));
  th = tanh_approx_h2(__hmul2(xc, p));
  return __hfma2(__float2half2_rn(0.5f), th, __float2half2_rn(0.5f));
}
__device__ __forceinline__ void gelu_erf_x2(float x0, float x1, float& y0, float& y1) {
  __half2 xc, t, th;
  const float2 P = __half22float2(normal_cdf_h2(x0, x1, xc, t, th));
  y0 = x0 * P.x;
  y1 = x1 * P.y;
}
__device__ __forceinline__ void gelu_erf_with_grad_x2(float x0, float x1, float& y0, float& y1, float& d0, float& d1) {
  __half2 xc, t, th;
  const __half2 Ph = normal_cdf_h2(x0, x1, xc, t, th);
  // Phi' = 0.5 (1 - tanh^2 u) u'(x), u' = c0 + 3 c1 t + 5 c2 t^2 + 7 c3 t^3 (the 0.5 folded into the coefficients)
  __half2 du = __hfma2(t, __float2half2_rn(3.5f * JB_GELU_C3), __float2half2_rn(2.5f * JB_GELU_C2));
  du = __hfma2(du, t, __float2half2_rn(1.5f * JB_GELU_C1));
  du = __hfma2(du, t, __float2half2_rn(0.5f * JB_GELU_C0));
  const __half2 om = __hfma2(__hneg2(th), th, __float2half2_rn(1.0f));
  const float2 D = __half22float2(__hfma2(xc, __hmul2(om, du), Ph));
  const float2 P = __half22float2(Ph);
  y0 = x0 * P.x;
  y1 = x1 * P.y;
  d0 = D.x;
  d1 = D.y;
}
__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

// The launch arguments of a kernel inside a CUDA graph are frozen, but every replay must publish and
// await a later epoch.  The graph bumps a device counter once per replay; the epoch of this launch is
// its captured value plus (replays * productions of the slot per replay).
__device__ __forceinline__ uint32_t live_epoch(uint32_t epoch, uint32_t stride, const uint32_t* replay) {
  return replay == nullptr ? epoch : epoch + stride * __ldg(replay);
}

}  // namespace jb
