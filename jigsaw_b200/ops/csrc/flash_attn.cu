// Attention forward for head dimension 64 on tcgen05: O = softmax(scale * Q K^T) V and the row-wise
// log-sum-exp (what the chunk merge of ring attention needs), no mask, bf16 in / bf16 + fp32 out.
//
// One CTA owns 128 query rows of one (batch, head) and walks over the keys in blocks of 128:
//   warp 0     TMA producer: Q once, then K and V blocks through a ring of FA_STAGES stages
//   warp 1     UMMA issuer:  S_j = Q K_j^T (M 128, N 128, K 64) into one of two TMEM buffers, then
//              PV_j = P_j V_j (M 128, N 64, K 128) into one of two TMEM buffers; S_{j+1} is issued
//              before PV_j so that the tensor cores work while block j's softmax runs
//   warps 2-5  softmax: thread = query row (TMEM lane).  Pass 1 reads S_j for the row maximum, pass 2
//              reads it again, exponentiates, writes P_j as bf16 into shared memory in the 128-byte
//              swizzled K-major layout the UMMA descriptor expects; the previous block's PV is then
//              folded into the fp32 output registers with the rescale factor of its own block.
// Every mbarrier wait is bounded (mbar_wait); a wait that gives up records itself in the status
// word and the CTA runs to its end without waiting.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "ptx.cuh"
#include "tmap.cuh"

namespace jb {

constexpr int FA_D = 64;          // head dimension
constexpr int FA_BM = 128;        // query rows per CTA
constexpr int FA_BN = 128;        // keys per block
constexpr int FA_STAGES = 3;
constexpr int FA_THREADS = 32 * 6;
constexpr int FA_TILE = 128 * 128;                 // bytes of a [128 x 64] bf16 tile
constexpr int FA_P_BYTES = 2 * FA_TILE;            // [128 x 128] bf16 as two K atoms of 64
constexpr int FA_SMEM = FA_TILE + FA_STAGES * 2 * FA_TILE + 2 * FA_P_BYTES + 256 + 1024;
static_assert(FA_SMEM <= 227 * 1024, "shared memory of one CTA");

__global__ void __launch_bounds__(FA_THREADS, 1)
flash_attn_fwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                      const __grid_constant__ CUtensorMap tmV, __nv_bfloat16* __restrict__ o, float* __restrict__ lse,
                      int sq, int sk, long long o_stride_s, long long o_stride_bh, float scale_log2, int* status) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* q_s = smem;
  uint8_t* kv_s = smem + FA_TILE;                                   // stage s: K at 2 s, V at 2 s + 1
  uint8_t* p_s = kv_s + FA_STAGES * 2 * FA_TILE;                     // two P buffers
  uint64_t* bars = reinterpret_cast<uint64_t*>(p_s + 2 * FA_P_BYTES);
  uint64_t* q_full = bars;                       // [1]
  uint64_t* k_full = bars + 1;                   // [STAGES]
  uint64_t* v_full = k_full + FA_STAGES;         // [STAGES]
  uint64_t* kv_empty = v_full + FA_STAGES;       // [STAGES]
  uint64_t* s_full = kv_empty + FA_STAGES;       // [2]
  uint64_t* s_empty = s_full + 2;                // [2]
  uint64_t* p_full = s_empty + 2;                // [2]
  uint64_t* p_empty = p_full + 2;                // [2]
  uint64_t* pv_full = p_empty + 2;               // [2]
  uint64_t* pv_empty = pv_full + 2;              // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(pv_empty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int q0 = blockIdx.x * FA_BM;
  const int bh = blockIdx.y;
  const int nblk = (sk + FA_BN - 1) / FA_BN;
  constexpr uint32_t TMEM_COLS = 512;            // S: 2 x 128 columns, PV: 2 x 64 columns

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int s = 0; s < FA_STAGES; ++s) {
      mbar_init(&k_full[s], 1);
      mbar_init(&v_full[s], 1);
      mbar_init(&kv_empty[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(&s_full[b], 1);
      mbar_init(&s_empty[b], 4);
      mbar_init(&p_full[b], 4);
      mbar_init(&p_empty[b], 1);
      mbar_init(&pv_full[b], 1);
      mbar_init(&pv_empty[b], 4);
    }
    *abort_flag = 0;
    fence_mbar_init();
    tma_prefetch_desc(&tmQ);
    tma_prefetch_desc(&tmK);
    tma_prefetch_desc(&tmV);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      mbar_expect_tx(q_full, FA_TILE);
      tma_load_3d(q_s, &tmQ, q_full, 0, q0, bh);
      for (int j = 0; j < nblk; ++j) {
        const int st = j % FA_STAGES;
        const uint32_t ph = static_cast<uint32_t>(j / FA_STAGES) & 1u;
        mbar_wait(&kv_empty[st], ph ^ 1u, abort_flag, status, 1);
        mbar_expect_tx(&k_full[st], FA_TILE);
        tma_load_3d(kv_s + (2 * st) * FA_TILE, &tmK, &k_full[st], 0, j * FA_BN, bh);
        mbar_expect_tx(&v_full[st], FA_TILE);
        tma_load_3d(kv_s + (2 * st + 1) * FA_TILE, &tmV, &v_full[st], 0, j * FA_BN, bh);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ UMMA issuer
    constexpr uint32_t idesc_s = make_idesc_bf16(FA_BM, FA_BN, 0, 0);      // Q (K-major) x K (K-major)
    constexpr uint32_t idesc_pv = make_idesc_bf16(FA_BM, FA_D, 0, 1);      // P (K-major) x V (rows = keys)
    const uint64_t q_desc = make_smem_desc_sw128(smem_u32(q_s), 16, 1024);
    const uint64_t kv_desc0 = make_smem_desc_sw128(smem_u32(kv_s), 16, 1024);
    const uint64_t v_desc0 = make_smem_desc_sw128(smem_u32(kv_s), 8192, 1024);
    const uint64_t p_desc0 = make_smem_desc_sw128(smem_u32(p_s), 16, 1024);
    mbar_wait(q_full, 0, abort_flag, status, 2);
    // PV of block i: waits for V_i, P_i and a free PV buffer, then releases the stage and the P buffer
    auto issue_pv = [&](int i) {
      const int b = i & 1;
      const int st = i % FA_STAGES;
      const uint32_t ph2 = static_cast<uint32_t>(i >> 1) & 1u;
      mbar_wait(&v_full[st], static_cast<uint32_t>(i / FA_STAGES) & 1u, abort_flag, status, 3);
      mbar_wait(&p_full[b], ph2, abort_flag, status, 4);
      mbar_wait(&pv_empty[b], ph2 ^ 1u, abort_flag, status, 5);
      tc_fence_after_sync();
      const uint64_t vd = desc_advance(v_desc0, static_cast<uint32_t>((2 * st + 1) * FA_TILE));
      const uint64_t pd = desc_advance(p_desc0, static_cast<uint32_t>(b * FA_P_BYTES));
      const uint32_t d_tmem = tmem_base + 256u + static_cast<uint32_t>(b * FA_D);
#pragma unroll
      for (int k = 0; k < FA_BN / 16; ++k) {
        // P: 16 keys = 32 bytes inside the swizzle row, second atom of 64 keys one tile further;
        // V: 16 keys = 16 rows of 128 bytes
        umma_f16_elect(d_tmem, desc_advance(pd, static_cast<uint32_t>((k >> 2) * FA_TILE + (k & 3) * 32)),
                       desc_advance(vd, static_cast<uint32_t>(k * 2048)), idesc_pv, k != 0 ? 1u : 0u);
      }
      umma_commit_elect(&kv_empty[st]);
      umma_commit_elect(&p_empty[b]);
      umma_commit_elect(&pv_full[b]);
    };
    for (int j = 0; j < nblk; ++j) {
      const int b = j & 1;
      const int st = j % FA_STAGES;
      mbar_wait(&k_full[st], static_cast<uint32_t>(j / FA_STAGES) & 1u, abort_flag, status, 6);
      mbar_wait(&s_empty[b], (static_cast<uint32_t>(j >> 1) & 1u) ^ 1u, abort_flag, status, 7);
      tc_fence_after_sync();
      const uint64_t kd = desc_advance(kv_desc0, static_cast<uint32_t>((2 * st) * FA_TILE));
      const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(b * FA_BN);
#pragma unroll
      for (int k = 0; k < FA_D / 16; ++k)
        umma_f16_elect(d_tmem, desc_advance(q_desc, static_cast<uint32_t>(k * 32)),
                       desc_advance(kd, static_cast<uint32_t>(k * 32)), idesc_s, k != 0 ? 1u : 0u);
      umma_commit_elect(&s_full[b]);
      if (j > 0) issue_pv(j - 1);
    }
    issue_pv(nblk - 1);
  } else {
    // ------------------------------------------------------------ softmax / output (4 warps, thread = row)
    const int quad = warp & 3;
    const int row = quad * 32 + lane;
    const uint32_t lane_addr = tmem_base + (static_cast<uint32_t>(quad * 32) << 16);
    float acc[FA_D];
#pragma unroll
    for (int i = 0; i < FA_D; ++i) acc[i] = 0.f;
    float m = -INFINITY, l = 0.f, alpha_prev = 0.f;
    // fold PV of block i into the output registers: acc = acc * alpha_i + PV_i
    auto fold_pv = [&](int i, float alpha) {
      const int b = i & 1;
      mbar_wait(&pv_full[b], static_cast<uint32_t>(i >> 1) & 1u, abort_flag, status, 8);
      tc_fence_after_sync();
#pragma unroll
      for (int c0 = 0; c0 < FA_D; c0 += 32) {
        uint32_t r[32];
        tmem_ld_32x32(lane_addr + 256u + static_cast<uint32_t>(b * FA_D + c0), r);
        tmem_ld_wait();
#pragma unroll
        for (int e = 0; e < 32; ++e) acc[c0 + e] = fmaf(acc[c0 + e], alpha, __uint_as_float(r[e]));
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&pv_empty[b]);
    };
    for (int j = 0; j < nblk; ++j) {
      const int b = j & 1;
      const uint32_t ph2 = static_cast<uint32_t>(j >> 1) & 1u;
      const int valid = sk - j * FA_BN;                  // columns of this block that are real keys
      mbar_wait(&s_full[b], ph2, abort_flag, status, 9);
      tc_fence_after_sync();
      const uint32_t s_addr = lane_addr + static_cast<uint32_t>(b * FA_BN);
      float mx = -INFINITY;
#pragma unroll 1
      for (int c0 = 0; c0 < FA_BN; c0 += 32) {
        uint32_t r[32];
        tmem_ld_32x32(s_addr + c0, r);
        tmem_ld_wait();
#pragma unroll
        for (int e = 0; e < 32; ++e)
          if (c0 + e < valid) mx = fmaxf(mx, __uint_as_float(r[e]));
      }
      const float m_new = fmaxf(m, mx * scale_log2);
      const float alpha = ex2_approx(m - m_new);          // 0 for the first block (m = -inf)
      mbar_wait(&p_empty[b], ph2 ^ 1u, abort_flag, status, 10);
      uint8_t* p_row = p_s + b * FA_P_BYTES + row * 128;
      float sum = 0.f;
#pragma unroll 1
      for (int c0 = 0; c0 < FA_BN; c0 += 32) {
        uint32_t r[32];
        tmem_ld_32x32(s_addr + c0, r);
        tmem_ld_wait();
        float p[32];
#pragma unroll
        for (int e = 0; e < 32; ++e) {
          const float x = (c0 + e < valid) ? ex2_approx(fmaf(__uint_as_float(r[e]), scale_log2, -m_new)) : 0.f;
          p[e] = x;
          sum += x;
        }
        uint8_t* atom = p_row + (c0 >> 6) * FA_TILE;       // K atom of 64 keys
#pragma unroll
        for (int e = 0; e < 32; e += 8) {
          uint4 v;
          v.x = pack_bf16x2(p[e], p[e + 1]);
          v.y = pack_bf16x2(p[e + 2], p[e + 3]);
          v.z = pack_bf16x2(p[e + 4], p[e + 5]);
          v.w = pack_bf16x2(p[e + 6], p[e + 7]);
          const int chunk = ((c0 & 63) + e) >> 3;          // 16-byte chunk of the 128-byte row
          *reinterpret_cast<uint4*>(atom + ((chunk ^ (row & 7)) << 4)) = v;
        }
      }
      tc_fence_before_sync();
      fence_proxy_async_smem();                            // P must be visible to the tensor core's reads
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(&s_empty[b]);
        mbar_arrive(&p_full[b]);
      }
      l = fmaf(l, alpha, sum);
      m = m_new;
      if (j > 0) fold_pv(j - 1, alpha_prev);
      alpha_prev = alpha;
    }
    fold_pv(nblk - 1, alpha_prev);
    if (q0 + row < sq) {
      const float inv = 1.f / l;
      __nv_bfloat16* dst = o + static_cast<long long>(bh) * o_stride_bh + static_cast<long long>(q0 + row) * o_stride_s;
#pragma unroll
      for (int e = 0; e < FA_D; e += 8) {
        uint4 v;
        v.x = pack_bf16x2(acc[e] * inv, acc[e + 1] * inv);
        v.y = pack_bf16x2(acc[e + 2] * inv, acc[e + 3] * inv);
        v.z = pack_bf16x2(acc[e + 4] * inv, acc[e + 5] * inv);
        v.w = pack_bf16x2(acc[e + 6] * inv, acc[e + 7] * inv);
        *reinterpret_cast<uint4*>(dst + e) = v;
      }
      lse[static_cast<long long>(bh) * sq + q0 + row] = (m + log2f(l)) * 0.6931471805599453f;
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

}  // namespace jb

// C ABI.  q, k, v: bf16, head dimension 64 contiguous, addressed as [bh][s][64] through element strides
// (`*_stride_s` between rows, `*_stride_bh` between (batch, head) slices; multiples of 8 elements, 16-byte
// aligned bases).  o likewise; lse is fp32 [bh][sq].  scale multiplies q k^T (natural-log softmax).
// Returns 0 on success, a negative code if the launch could not be set up.
extern "C" int jb_flash_attn_fwd(const void* q, const void* k, const void* v, void* o, float* lse, int bh, int sq,
                                 int sk, long long q_stride_s, long long q_stride_bh, long long k_stride_s,
                                 long long k_stride_bh, long long v_stride_s, long long v_stride_bh,
                                 long long o_stride_s, long long o_stride_bh, float scale, int* status, void* stream) {
  using namespace jb;
  if (bh < 1 || bh > 65535 || sq < 1 || sk < 1) return -1;
  const long long strides[] = {q_stride_s, q_stride_bh, k_stride_s, k_stride_bh, v_stride_s, v_stride_bh, o_stride_s, o_stride_bh};
  for (long long s : strides)
    if (s & 7) return -1;
  const void* ptrs[] = {q, k, v, o};
  for (const void* p : ptrs)
    if (reinterpret_cast<uintptr_t>(p) & 15) return -1;
  CUtensorMap tmQ, tmK, tmV;
  const uint32_t box[3] = {FA_D, FA_BM, 1};
  {
    const uint64_t dims[3] = {FA_D, static_cast<uint64_t>(sq), static_cast<uint64_t>(bh)};
    const uint64_t st[2] = {static_cast<uint64_t>(q_stride_s) * 2, static_cast<uint64_t>(q_stride_bh) * 2};
    if (make_tmap_bf16(&tmQ, q, 3, dims, st, box) != 0) return -2;
  }
  {
    const uint64_t dims[3] = {FA_D, static_cast<uint64_t>(sk), static_cast<uint64_t>(bh)};
    const uint64_t stk[2] = {static_cast<uint64_t>(k_stride_s) * 2, static_cast<uint64_t>(k_stride_bh) * 2};
    const uint64_t stv[2] = {static_cast<uint64_t>(v_stride_s) * 2, static_cast<uint64_t>(v_stride_bh) * 2};
    if (make_tmap_bf16(&tmK, k, 3, dims, stk, box) != 0) return -2;
    if (make_tmap_bf16(&tmV, v, 3, dims, stv, box) != 0) return -2;
  }
  static bool attr_set = false;
  if (!attr_set) {
    if (cudaFuncSetAttribute(flash_attn_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, FA_SMEM) != cudaSuccess)
      return -3;
    attr_set = true;
  }
  const dim3 grid((sq + FA_BM - 1) / FA_BM, bh);
  flash_attn_fwd_kernel<<<grid, FA_THREADS, FA_SMEM, static_cast<cudaStream_t>(stream)>>>(
      tmQ, tmK, tmV, static_cast<__nv_bfloat16*>(o), lse, sq, sk, o_stride_s, o_stride_bh,
      scale * 1.4426950408889634f, status);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}
