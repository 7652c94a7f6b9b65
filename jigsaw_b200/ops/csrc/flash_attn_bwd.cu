// Attention backward for head dimension 64 on tcgen05, companion of flash_attn.cu.  Three kernels:
//   fa_delta_kernel     D[row] = sum_d dO[row][d] * O[row][d]                       (memory-bound)
//   fa_bwd_kernel<0>    one CTA per block of 128 keys, loop over query blocks:
//                         S = Q K^T, dP = dO V^T, P = exp(scale S - LSE), dS = scale P (dP - D),
//                         dV += P^T dO, dK += dS^T Q      (accumulators stay in TMEM over the loop)
//   fa_bwd_kernel<1>    one CTA per block of 128 queries, loop over key blocks:
//                         S, dP, dS as above, dQ += dS K
// S and dP are recomputed in both kernels so that no gradient needs atomics or a reduction: every
// gradient block is produced completely by the one CTA that owns it.  That also carries ring attention:
// the STREAMED operand pair (queries and output gradients for <0>, keys and values for <1>) may come in
// up to eight parts that belong to different GPUs; the kernel waits (bounded) for a part's arrival flag and
// loads its blocks by TMA (no multicast) through the part's own tensor map (the callers have the copy engines
// push every rank's part into a local staging slot), so the owner of a key block computes its complete
// dK / dV from every rank's queries, and no gradient is sent back.
//
// Roles: warp 0 TMA producer, warp 1 UMMA issuer, warps 2-9 row warps (thread = one query row and one
// half of the 128 key columns; no reduction along a row is needed in the backward pass).  P and dS go
// to the tensor cores through shared memory as [query][key] tiles in the 128-byte swizzled layout; the
// same bytes serve as a K-major operand (dS K) and, transposed, as an MN-major operand (P^T dO, dS^T Q).
// The issuer starts S and dP of the next block before the accumulating products of the current one, so
// that the row warps' exponentials overlap them.  Every wait is bounded.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "ptx.cuh"
#include "tmap.cuh"

namespace jb {

constexpr int FB_D = 64;
constexpr int FB_B = 128;                       // rows of a query block and of a key block
constexpr int FB_ROW_WARPS = 8;
constexpr int FB_THREADS = 32 * (2 + FB_ROW_WARPS);
constexpr int FB_TILE = 128 * 128;              // bytes of a [128 x 64] bf16 tile
constexpr int FB_PT = 2 * FB_TILE;              // bytes of a [128 x 128] bf16 tile (two 64-wide blocks)
constexpr int FB_STAGES = 2;
// resident pair (K, V or Q, dO) + ring of streamed pairs + P + dS + barriers + alignment slack
constexpr int FB_SMEM = 2 * FB_TILE + FB_STAGES * 2 * FB_TILE + 2 * FB_PT + 256 + 1024;
static_assert(FB_SMEM <= 227 * 1024, "shared memory of one CTA");
constexpr int FB_MAX_PARTS = 8;

struct FbParts {
  CUtensorMap c[FB_MAX_PARTS];          // streamed pair, first operand  (<0>: Q,  <1>: K) of each part
  CUtensorMap d[FB_MAX_PARTS];          // streamed pair, second operand (<0>: dO, <1>: V)
  const float* lse[FB_MAX_PARTS];       // <0>: log-sum-exp and D of the part's query rows ([bh][rows_part]);
  const float* delta[FB_MAX_PARTS];     //      <1>: entry 0 holds the local ones ([bh][rows of the resident block's tensor])
  const uint32_t* flag[FB_MAX_PARTS];   // local flag word raised by the part's owner, or null
  uint32_t epoch, stride;
  const uint32_t* replay;
  int parts, first;
  int rows_part;                        // rows of the streamed operands per part
};

__global__ void fa_delta_kernel(const __nv_bfloat16* __restrict__ o, const __nv_bfloat16* __restrict__ d_o,
                                float* __restrict__ delta, long long rows) {
  // eight lanes per row of 64 values (16 bytes each)
  const long long row = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 3;
  const int part = threadIdx.x & 7;
  float s = 0.f;
  if (row < rows) {
    const uint4 a = *reinterpret_cast<const uint4*>(o + row * FB_D + part * 8);
    const uint4 b = *reinterpret_cast<const uint4*>(d_o + row * FB_D + part * 8);
    const __nv_bfloat162* pa = reinterpret_cast<const __nv_bfloat162*>(&a);
    const __nv_bfloat162* pb = reinterpret_cast<const __nv_bfloat162*>(&b);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 x = __bfloat1622float2(pa[i]);
      const float2 y = __bfloat1622float2(pb[i]);
      s = fmaf(x.x, y.x, fmaf(x.y, y.y, s));
    }
  }
  s += __shfl_xor_sync(0xffffffffu, s, 1);
  s += __shfl_xor_sync(0xffffffffu, s, 2);
  s += __shfl_xor_sync(0xffffffffu, s, 4);
  if (row < rows && part == 0) delta[row] = s;
}

// 32 values of one thread's row as bf16 into a [128 x 128] tile made of two [128 rows x 128 bytes]
// blocks with the 128-byte swizzle: 16-byte chunk c of row r sits at chunk c ^ (r & 7).
__device__ __forceinline__ void store_row_chunk(uint8_t* tile, int row, int c0, const float (&p)[32]) {
  uint8_t* blk = tile + (c0 >> 6) * FB_TILE + row * 128;
#pragma unroll
  for (int e = 0; e < 32; e += 8) {
    uint4 v;
    v.x = pack_bf16x2(p[e], p[e + 1]);
    v.y = pack_bf16x2(p[e + 2], p[e + 3]);
    v.z = pack_bf16x2(p[e + 4], p[e + 5]);
    v.w = pack_bf16x2(p[e + 6], p[e + 7]);
    const int chunk = ((c0 & 63) + e) >> 3;
    *reinterpret_cast<uint4*>(blk + ((chunk ^ (row & 7)) << 4)) = v;
  }
}

__device__ __forceinline__ void fb_wait_flag(const uint32_t* f, uint32_t want, volatile int* abort_flag, int* status) {
  if (f == nullptr) return;
  const uint64_t t0 = globaltimer_ns();
  while (true) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(f) : "memory");
    if (static_cast<int32_t>(v - want) >= 0) break;
    if (*abort_flag || globaltimer_ns() - t0 > JB_WAIT_LIMIT_NS) {
      *abort_flag = 1;
      if (status) atomicCAS(status, JB_OK, JB_ERR_FLAG_TIMEOUT);
      return;
    }
    __nanosleep(64);
  }
  asm volatile("fence.proxy.async;" ::: "memory");
}

// MODE 0: dK / dV (the CTA's block is a key block, the loop runs over query blocks of all parts).
// MODE 1: dQ      (the CTA's block is a query block, the loop runs over key blocks of all parts).
// tmA / tmB: the resident pair (MODE 0: K, V; MODE 1: Q, dO); sp: the streamed pair
// (MODE 0: Q, dO; MODE 1: K, V).  rows_res: rows of the resident tensors.
template <int MODE>
__global__ void __launch_bounds__(FB_THREADS, 1)
fa_bwd_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
              const __grid_constant__ FbParts sp, __nv_bfloat16* __restrict__ out0, __nv_bfloat16* __restrict__ out1,
              int rows_res, float scale, int* status) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* res_s = smem;                                         // resident pair: [0] and [1]
  uint8_t* ring_s = smem + 2 * FB_TILE;                          // stage s: first at 2 s, second at 2 s + 1
  uint8_t* p_s = ring_s + FB_STAGES * 2 * FB_TILE;               // P   [query][key]
  uint8_t* ds_s = p_s + FB_PT;                                   // dS  [query][key]
  uint64_t* bars = reinterpret_cast<uint64_t*>(ds_s + FB_PT);
  uint64_t* res_full = bars;                     // [1]
  uint64_t* ring_full = bars + 1;                // [STAGES]
  uint64_t* ring_empty = ring_full + FB_STAGES;  // [STAGES]
  uint64_t* s_full = ring_empty + FB_STAGES;     // S and dP are in TMEM
  uint64_t* pds_full = s_full + 1;               // P and dS are in shared memory; S and dP have been read
  uint64_t* pds_free = pds_full + 1;             // the UMMAs that read P and dS are done
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(pds_free + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int own0 = blockIdx.x * FB_B;            // first row of this CTA's block
  const int bh = blockIdx.y;
  const int nbp = (sp.rows_part + FB_B - 1) / FB_B;
  const int n_loop = sp.parts * nbp;
  constexpr uint32_t TMEM_COLS = 512;            // S 0..127, dP 128..255, accumulators 256.. (64 columns each)

  if (threadIdx.x == 0) {
    mbar_init(res_full, 1);
    for (int s = 0; s < FB_STAGES; ++s) {
      mbar_init(&ring_full[s], 1);
      mbar_init(&ring_empty[s], 1);
    }
    mbar_init(s_full, 1);
    mbar_init(pds_full, FB_ROW_WARPS);
    mbar_init(pds_free, 1);
    *abort_flag = 0;
    fence_mbar_init();
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
    tma_prefetch_desc(&sp.c[sp.first]);
    tma_prefetch_desc(&sp.d[sp.first]);
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
      mbar_expect_tx(res_full, 2 * FB_TILE);
      tma_load_3d(res_s, &tmA, res_full, 0, own0, bh);
      tma_load_3d(res_s + FB_TILE, &tmB, res_full, 0, own0, bh);
      const uint32_t want = live_epoch(sp.epoch, sp.stride, sp.replay);
      int part = sp.first, ib = 0;
      for (int i = 0; i < n_loop; ++i) {
        if (ib == 0) fb_wait_flag(sp.flag[part], want, abort_flag, status);
        const int st = i % FB_STAGES;
        mbar_wait(&ring_empty[st], (static_cast<uint32_t>(i / FB_STAGES) & 1u) ^ 1u, abort_flag, status, 1);
        mbar_expect_tx(&ring_full[st], 2 * FB_TILE);
        tma_load_3d(ring_s + (2 * st) * FB_TILE, &sp.c[part], &ring_full[st], 0, ib * FB_B, bh);
        tma_load_3d(ring_s + (2 * st + 1) * FB_TILE, &sp.d[part], &ring_full[st], 0, ib * FB_B, bh);
        if (++ib == nbp) {
          ib = 0;
          if (++part == sp.parts) part = 0;
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ UMMA issuer
    constexpr uint32_t idesc_s = make_idesc_bf16(FB_B, FB_B, 0, 0);        // [128 x 64] x [128 x 64]^T
    constexpr uint32_t idesc_t = make_idesc_bf16(FB_B, FB_D, 1, 1);        // transposed tile x streamed rows
    constexpr uint32_t idesc_q = make_idesc_bf16(FB_B, FB_D, 0, 1);        // dS (K-major) x K rows
    const uint32_t res_a = smem_u32(res_s);
    const uint32_t ring_a = smem_u32(ring_s);
    // query-side tiles (Q, dO) and key-side tiles (K, V) of iteration i
    auto q_addr = [&](int i) { return MODE == 0 ? ring_a + (2 * (i % FB_STAGES)) * FB_TILE : res_a; };
    auto k_addr = [&](int i) { return MODE == 0 ? res_a : ring_a + (2 * (i % FB_STAGES)) * FB_TILE; };
    auto issue_s_dp = [&](int i) {
      const uint32_t q_a = q_addr(i), k_a = k_addr(i);
      const uint64_t qd = make_smem_desc_sw128(q_a, 16, 1024), kd = make_smem_desc_sw128(k_a, 16, 1024);
      const uint64_t dod = make_smem_desc_sw128(q_a + FB_TILE, 16, 1024), vd = make_smem_desc_sw128(k_a + FB_TILE, 16, 1024);
#pragma unroll
      for (int k = 0; k < FB_D / 16; ++k)                                   // S = Q K^T
        umma_f16_elect(tmem_base, desc_advance(qd, k * 32), desc_advance(kd, k * 32), idesc_s, k != 0 ? 1u : 0u);
#pragma unroll
      for (int k = 0; k < FB_D / 16; ++k)                                   // dP = dO V^T
        umma_f16_elect(tmem_base + 128u, desc_advance(dod, k * 32), desc_advance(vd, k * 32), idesc_s, k != 0 ? 1u : 0u);
      umma_commit_elect(s_full);
    };
    mbar_wait(res_full, 0, abort_flag, status, 2);
    mbar_wait(&ring_full[0], 0, abort_flag, status, 3);
    tc_fence_after_sync();
    issue_s_dp(0);
    for (int i = 0; i < n_loop; ++i) {
      const int st = i % FB_STAGES;
      const uint32_t ph = static_cast<uint32_t>(i) & 1u;
      const bool more = i + 1 < n_loop;
      if (more)
        mbar_wait(&ring_full[(i + 1) % FB_STAGES], static_cast<uint32_t>((i + 1) / FB_STAGES) & 1u, abort_flag, status, 4);
      mbar_wait(pds_full, ph, abort_flag, status, 5);
      tc_fence_after_sync();
      if (more) issue_s_dp(i + 1);                  // S and dP of block i have been read by every row warp
      const uint32_t q_a = q_addr(i), k_a = k_addr(i);
      if (MODE == 0) {
        // dV += P^T dO and dK += dS^T Q: A is the [query][key] tile read transposed (rows = reduction index,
        // two 64-key blocks one tile apart), B the streamed [query][64] tile (rows = reduction index)
        const uint64_t pt = make_smem_desc_sw128(smem_u32(p_s), FB_TILE, 1024);
        const uint64_t dst = make_smem_desc_sw128(smem_u32(ds_s), FB_TILE, 1024);
        const uint64_t dob = make_smem_desc_sw128(q_a + FB_TILE, 8192, 1024), qb = make_smem_desc_sw128(q_a, 8192, 1024);
#pragma unroll
        for (int k = 0; k < FB_B / 16; ++k)
          umma_f16_elect(tmem_base + 256u, desc_advance(pt, k * 2048), desc_advance(dob, k * 2048), idesc_t,
                         (i | k) != 0 ? 1u : 0u);
#pragma unroll
        for (int k = 0; k < FB_B / 16; ++k)
          umma_f16_elect(tmem_base + 320u, desc_advance(dst, k * 2048), desc_advance(qb, k * 2048), idesc_t,
                         (i | k) != 0 ? 1u : 0u);
      } else {
        // dQ += dS K: A = dS K-major (two blocks of 64 keys), B = K rows (rows = reduction index)
        const uint64_t dsk = make_smem_desc_sw128(smem_u32(ds_s), 16, 1024);
        const uint64_t kb = make_smem_desc_sw128(k_a, 8192, 1024);
#pragma unroll
        for (int k = 0; k < FB_B / 16; ++k)
          umma_f16_elect(tmem_base + 256u, desc_advance(dsk, static_cast<uint32_t>((k >> 2) * FB_TILE + (k & 3) * 32)),
                         desc_advance(kb, k * 2048), idesc_q, (i | k) != 0 ? 1u : 0u);
      }
      umma_commit_elect(&ring_empty[st]);
      umma_commit_elect(pds_free);
    }
  } else {
    // ------------------------------------------------------------ row warps (thread = query row, half of the keys)
    const int quad = warp & 3;
    const int half = (warp - 2) >> 2;                              // key columns [64 half, 64 half + 64)
    const int row = quad * 32 + lane;
    const uint32_t lane_addr = tmem_base + (static_cast<uint32_t>(quad * 32) << 16);
    const float scale_log2 = scale * 1.4426950408889634f;
    int part = sp.first, ib = 0;
    for (int i = 0; i < n_loop; ++i) {
      const uint32_t ph = static_cast<uint32_t>(i) & 1u;
      // global query row of this thread, and where its LSE / D live
      const int qrow = MODE == 0 ? ib * FB_B + row : own0 + row;
      const int qrows = MODE == 0 ? sp.rows_part : rows_res;
      const float* lse_p = MODE == 0 ? sp.lse[part] : sp.lse[0];
      const float* del_p = MODE == 0 ? sp.delta[part] : sp.delta[0];
      if (++ib == nbp) {
        ib = 0;
        if (++part == sp.parts) part = 0;
      }
      mbar_wait(s_full, ph, abort_flag, status, 7);
      tc_fence_after_sync();
      // rows past the end get P = 0 (LSE = +inf) and D = 0.  (The flag of the part has been seen by the
      // producer before S could complete, so a peer's LSE / D are final here.)
      const float l2 = qrow < qrows ? __ldg(lse_p + static_cast<long long>(bh) * qrows + qrow) * 1.4426950408889634f : INFINITY;
      const float dl = qrow < qrows ? __ldg(del_p + static_cast<long long>(bh) * qrows + qrow) : 0.f;
#pragma unroll 1
      for (int cc = 0; cc < 64; cc += 32) {
        const int c0 = half * 64 + cc;
        uint32_t r[32], g[32];
        tmem_ld_32x32(lane_addr + c0, r);
        tmem_ld_32x32(lane_addr + 128u + c0, g);
        tmem_ld_wait();
        float p[32], d[32];
#pragma unroll
        for (int e = 0; e < 32; ++e) {
          p[e] = ex2_approx(fmaf(__uint_as_float(r[e]), scale_log2, -l2));
          d[e] = p[e] * (__uint_as_float(g[e]) - dl) * scale;
        }
        if (cc == 0) mbar_wait(pds_free, ph ^ 1u, abort_flag, status, 8);      // the previous block's products have read P / dS
        if (MODE == 0) store_row_chunk(p_s, row, c0, p);
        store_row_chunk(ds_s, row, c0, d);
      }
      tc_fence_before_sync();
      fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) mbar_arrive(pds_full);
    }
    // ---- accumulators -> global (thread = row of this CTA's block; the two halves split the 64 columns)
    mbar_wait(pds_free, static_cast<uint32_t>(n_loop - 1) & 1u, abort_flag, status, 9);
    tc_fence_after_sync();
    const long long base = (static_cast<long long>(bh) * rows_res + own0 + row) * FB_D;
#pragma unroll 1
    for (int a = 0; a < (MODE == 0 ? 2 : 1); ++a) {
      // MODE 0: accumulator 0 = dV (out1), accumulator 1 = dK (out0); MODE 1: dQ (out0)
      __nv_bfloat16* dst = (MODE == 0 && a == 0) ? out1 : out0;
      const int c0 = half * 32;
      uint32_t r[32];
      tmem_ld_32x32(lane_addr + 256u + static_cast<uint32_t>(a * 64 + c0), r);
      tmem_ld_wait();
      if (own0 + row < rows_res) {
#pragma unroll
        for (int e = 0; e < 32; e += 8) {
          uint4 v;
          v.x = pack_bf16x2(__uint_as_float(r[e]), __uint_as_float(r[e + 1]));
          v.y = pack_bf16x2(__uint_as_float(r[e + 2]), __uint_as_float(r[e + 3]));
          v.z = pack_bf16x2(__uint_as_float(r[e + 4]), __uint_as_float(r[e + 5]));
          v.w = pack_bf16x2(__uint_as_float(r[e + 6]), __uint_as_float(r[e + 7]));
          *reinterpret_cast<uint4*>(dst + base + c0 + e) = v;
        }
      }
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

static int fb_operand_map(CUtensorMap* m, const void* base, int rows, int bh) {
  const uint32_t box[3] = {jb::FB_D, jb::FB_B, 1};
  const uint64_t dims[3] = {jb::FB_D, static_cast<uint64_t>(rows), static_cast<uint64_t>(bh)};
  const uint64_t st[2] = {jb::FB_D * 2, static_cast<uint64_t>(rows) * jb::FB_D * 2};
  return jb::make_tmap_bf16(m, base, 3, dims, st, box);
}

static int fb_set_attributes() {
  using namespace jb;
  static bool attr_set = false;
  if (!attr_set) {
    if (cudaFuncSetAttribute(fa_bwd_kernel<0>, cudaFuncAttributeMaxDynamicSharedMemorySize, FB_SMEM) != cudaSuccess ||
        cudaFuncSetAttribute(fa_bwd_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, FB_SMEM) != cudaSuccess)
      return -3;
    attr_set = true;
  }
  return 0;
}

// D[row] = sum_d dO[row][d] O[row][d] for contiguous [rows][64] bf16 tensors.
extern "C" int jb_flash_attn_delta(const void* o, const void* d_o, float* delta, long long rows, void* stream) {
  if (rows < 1) return -1;
  jb::fa_delta_kernel<<<static_cast<unsigned>((rows * 8 + 255) / 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(o), static_cast<const __nv_bfloat16*>(d_o), delta, rows);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

// Gradients with the sequence split into `parts` equal parts over GPUs (ring attention); all tensors are
// contiguous bf16 [bh][s_part][64] (LSE, D: fp32 [bh][s_part]), 16-byte aligned.
//   q, d_o, k, v        this rank's own part (local memory)
//   q_parts, do_parts, lse_parts, delta_parts, k_parts, v_parts
//                       the same tensors of every part (entry `me` = the local ones; the others are
//                       pointers into the peers' memory), visited in the order me, me + 1, ... cyclically
//   flags[p]            local flag word that must reach `epoch` before part p is read, or null
//   dq, dk, dv          gradients of this rank's own part
// With parts = 1 this is plain attention backward.  Returns 0 on success, a negative code otherwise.
extern "C" int jb_flash_attn_bwd_parts(const void* q, const void* k, const void* v, const void* d_o,
                                       const void* const* q_parts, const void* const* do_parts,
                                       const float* const* lse_parts, const float* const* delta_parts,
                                       const void* const* k_parts, const void* const* v_parts, const void* const* flags,
                                       unsigned int epoch, unsigned int stride, const unsigned int* replay, int parts,
                                       int me, void* dq, void* dk, void* dv, int bh, int s_part, float scale, int* status,
                                       void* stream) {
  using namespace jb;
  if (bh < 1 || bh > 65535 || s_part < 1 || parts < 1 || parts > FB_MAX_PARTS || me < 0 || me >= parts) return -1;
  const void* ptrs[] = {q, k, v, d_o, dq, dk, dv};
  for (const void* p : ptrs)
    if (reinterpret_cast<uintptr_t>(p) & 15) return -1;
  CUtensorMap tmQ, tmK, tmV, tmDO;
  if (fb_operand_map(&tmQ, q, s_part, bh) != 0 || fb_operand_map(&tmDO, d_o, s_part, bh) != 0 ||
      fb_operand_map(&tmK, k, s_part, bh) != 0 || fb_operand_map(&tmV, v, s_part, bh) != 0)
    return -2;
  FbParts sq{}, sk{};
  for (int p = 0; p < parts; ++p) {
    const void* four[] = {q_parts[p], do_parts[p], k_parts[p], v_parts[p]};
    for (const void* x : four)
      if (reinterpret_cast<uintptr_t>(x) & 15) return -1;
    if (fb_operand_map(&sq.c[p], q_parts[p], s_part, bh) != 0 || fb_operand_map(&sq.d[p], do_parts[p], s_part, bh) != 0 ||
        fb_operand_map(&sk.c[p], k_parts[p], s_part, bh) != 0 || fb_operand_map(&sk.d[p], v_parts[p], s_part, bh) != 0)
      return -2;
    sq.lse[p] = lse_parts[p];
    sq.delta[p] = delta_parts[p];
    sq.flag[p] = sk.flag[p] = flags == nullptr ? nullptr : static_cast<const uint32_t*>(flags[p]);
  }
  sk.lse[0] = lse_parts[me];
  sk.delta[0] = delta_parts[me];
  sq.epoch = sk.epoch = epoch;
  sq.stride = sk.stride = stride;
  sq.replay = sk.replay = replay;
  sq.parts = sk.parts = parts;
  sq.first = sk.first = me;
  sq.rows_part = sk.rows_part = s_part;
  if (fb_set_attributes() != 0) return -3;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const dim3 grid((s_part + FB_B - 1) / FB_B, bh);
  fa_bwd_kernel<0><<<grid, FB_THREADS, FB_SMEM, st>>>(tmK, tmV, sq, static_cast<__nv_bfloat16*>(dk),
                                                     static_cast<__nv_bfloat16*>(dv), s_part, scale, status);
  fa_bwd_kernel<1><<<grid, FB_THREADS, FB_SMEM, st>>>(tmQ, tmDO, sk, static_cast<__nv_bfloat16*>(dq), nullptr, s_part,
                                                     scale, status);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

// C ABI of plain attention backward.  q, o, d_o, dq: [bh][sq][64]; k, v, dk, dv: [bh][sk][64]; all bf16,
// contiguous, 16-byte aligned.  lse: [bh][sq] fp32 as returned by jb_flash_attn_fwd (natural logarithm, of
// the scaled scores); delta: [bh][sq] fp32 scratch.  Returns 0 on success, a negative code otherwise.
extern "C" int jb_flash_attn_bwd(const void* q, const void* k, const void* v, const void* o, const void* d_o,
                                 const float* lse, float* delta, void* dq, void* dk, void* dv, int bh, int sq, int sk,
                                 float scale, int* status, void* stream) {
  using namespace jb;
  if (bh < 1 || bh > 65535 || sq < 1 || sk < 1) return -1;
  const void* ptrs[] = {q, k, v, o, d_o, dq, dk, dv};
  for (const void* p : ptrs)
    if (reinterpret_cast<uintptr_t>(p) & 15) return -1;
  CUtensorMap tmQ, tmK, tmV, tmDO;
  if (fb_operand_map(&tmQ, q, sq, bh) != 0 || fb_operand_map(&tmDO, d_o, sq, bh) != 0 ||
      fb_operand_map(&tmK, k, sk, bh) != 0 || fb_operand_map(&tmV, v, sk, bh) != 0)
    return -2;
  FbParts pq{}, pk{};
  pq.c[0] = tmQ; pq.d[0] = tmDO; pq.lse[0] = lse; pq.delta[0] = delta; pq.parts = 1; pq.rows_part = sq;
  pk.c[0] = tmK; pk.d[0] = tmV; pk.lse[0] = lse; pk.delta[0] = delta; pk.parts = 1; pk.rows_part = sk;
  if (fb_set_attributes() != 0) return -3;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int rc = jb_flash_attn_delta(o, d_o, delta, static_cast<long long>(bh) * sq, stream);
  if (rc != 0) return rc;
  fa_bwd_kernel<0><<<dim3((sk + FB_B - 1) / FB_B, bh), FB_THREADS, FB_SMEM, st>>>(
      tmK, tmV, pq, static_cast<__nv_bfloat16*>(dk), static_cast<__nv_bfloat16*>(dv), sk, scale, status);
  fa_bwd_kernel<1><<<dim3((sq + FB_B - 1) / FB_B, bh), FB_THREADS, FB_SMEM, st>>>(
      tmQ, tmDO, pk, static_cast<__nv_bfloat16*>(dq), nullptr, sq, scale, status);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}
