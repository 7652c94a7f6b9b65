// Attention forward for head dimension 64 on tcgen05: O = softmax(scale * Q K^T) V and the row-wise
// log-sum-exp, no mask, bf16 in / bf16 + fp32 out.  The keys and values may come in up to eight PARTS
// that belong to different GPUs (ring / sequence-parallel attention): the kernel walks over the parts
// starting with its own, waits (bounded) for the arrival flag of a part before the first block of that
// part, and loads its blocks by TMA (no multicast) through the part's own tensor map.  The callers let the
// copy engines push every rank's part into a local staging slot, so each byte crosses NVLink once per
// destination and the loads hit local memory; a map over a peer's memory works as well.  The running
// maximum and sum stay in registers and the output accumulator stays in TMEM across all parts, so a
// ring of P chunks is ONE launch and needs no merge step.
//
// One CTA owns two tiles of 128 query rows of one (batch, head) and walks over the keys in blocks of 128:
//   warp 0      TMA producer: both Q tiles once, then K and V blocks through a ring of FA_STAGES stages
//   warp 1      UMMA issuer: S_t = Q_t K_j^T (M 128, N 128, K 64) into the tile's TMEM columns and
//               O_t += P_t V_j (M 128, N 64, K 128) into the tile's accumulator columns; S_t of block
//               j + 1 is issued before P_t V_j so that it is ready when the softmax of block j ends
//   warps 2-5   softmax of tile 0, warps 6-9 softmax of tile 1: thread = query row (TMEM lane).  Pass 1
//               reads S for the row maximum, pass 2 reads it again, exponentiates and writes P as bf16
//               into shared memory in the 128-byte swizzled K-major layout of the UMMA descriptor.
//               While one tile's warps exponentiate, the tensor core works for the other tile.
// The accumulator is only rescaled when the running maximum grew by more than 8 (in log2 units) since
// the last rescale; until then the stale maximum is used for P, the row sum and the final
// log-sum-exp alike, which is exact and keeps the rescale (a TMEM round trip) off the common path.
// Every wait is bounded (mbar_wait); a wait that gives up records itself in the status word and the CTA
// runs to its end without waiting.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "ptx.cuh"
#include "tmap.cuh"

namespace jb {

constexpr int FA_D = 64;          // head dimension
constexpr int FA_BM = 128;        // query rows per tile
constexpr int FA_QT = 2;          // query tiles per CTA
constexpr int FA_BN = 128;        // keys per block
constexpr int FA_STAGES = 3;
constexpr int FA_THREADS = 32 * (2 + 4 * FA_QT);
constexpr int FA_TILE = 128 * 128;                 // bytes of a [128 x 64] bf16 tile
constexpr int FA_P_BYTES = 2 * FA_TILE;            // [128 x 128] bf16 as two K atoms of 64
constexpr int FA_SMEM = FA_QT * FA_TILE + FA_STAGES * 2 * FA_TILE + FA_QT * FA_P_BYTES + 256 + 1024;
constexpr float FA_RESCALE_STEP = 8.0f;            // log2 units
static_assert(FA_SMEM <= 227 * 1024, "shared memory of one CTA");

constexpr int FA_MAX_PARTS = 8;

struct FaParts {
  CUtensorMap k[FA_MAX_PARTS];     // [bh][sk_part][64] of each part (a peer's memory for a remote part)
  CUtensorMap v[FA_MAX_PARTS];
  const uint32_t* flag[FA_MAX_PARTS];   // local flag word raised by the part's owner once K / V are staged; null: no wait
  uint32_t epoch;                  // value the flags must reach (plus stride * *replay inside a replayed graph)
  uint32_t stride;
  const uint32_t* replay;
  int parts;                       // number of parts
  int first;                       // part visited first, then first + 1, ... cyclically
  int sk_part;                     // keys per part
};

// Bounded wait for a cross-GPU flag by one thread (the TMA producer).
__device__ __forceinline__ void fa_wait_flag(const uint32_t* f, uint32_t want, volatile int* abort_flag, int* status) {
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
  // the owner's data was written through the generic proxy; TMA reads through the async proxy
  asm volatile("fence.proxy.async;" ::: "memory");
}

__global__ void __launch_bounds__(FA_THREADS, 1)
flash_attn_fwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ FaParts kv,
                      __nv_bfloat16* __restrict__ o, float* __restrict__ lse, int sq, long long o_stride_s,
                      long long o_stride_bh, float scale_log2, int* status) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* q_s = smem;                                              // tile t at t * FA_TILE
  uint8_t* kv_s = q_s + FA_QT * FA_TILE;                            // stage s: K at 2 s, V at 2 s + 1
  uint8_t* p_s = kv_s + FA_STAGES * 2 * FA_TILE;                     // tile t at t * FA_P_BYTES
  uint64_t* bars = reinterpret_cast<uint64_t*>(p_s + FA_QT * FA_P_BYTES);
  uint64_t* q_full = bars;                       // [1]
  uint64_t* kv_full = bars + 1;                  // [STAGES]
  uint64_t* kv_empty = kv_full + FA_STAGES;      // [STAGES]
  uint64_t* s_full = kv_empty + FA_STAGES;       // [QT]  S_t of the current block is in TMEM
  uint64_t* p_full = s_full + FA_QT;             // [QT]  P_t is in shared memory, S_t has been read, O_t is rescaled
  uint64_t* pv_done = p_full + FA_QT;            // [QT]  O_t += P_t V has completed (P_t may be overwritten)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(pv_done + FA_QT);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int q0 = blockIdx.x * (FA_QT * FA_BM);
  const int bh = blockIdx.y;
  const int nbp = (kv.sk_part + FA_BN - 1) / FA_BN;        // blocks per part
  const int nblk = kv.parts * nbp;
  constexpr uint32_t TMEM_COLS = 512;            // S: QT x 128 columns, O: QT x 64 columns from column 256

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int s = 0; s < FA_STAGES; ++s) {
      mbar_init(&kv_full[s], 1);
      mbar_init(&kv_empty[s], 1);
    }
    for (int t = 0; t < FA_QT; ++t) {
      mbar_init(&s_full[t], 1);
      mbar_init(&p_full[t], 4);
      mbar_init(&pv_done[t], 1);
    }
    *abort_flag = 0;
    fence_mbar_init();
    tma_prefetch_desc(&tmQ);
    tma_prefetch_desc(&kv.k[kv.first]);
    tma_prefetch_desc(&kv.v[kv.first]);
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
      mbar_expect_tx(q_full, FA_QT * FA_TILE);
#pragma unroll
      for (int t = 0; t < FA_QT; ++t) tma_load_3d(q_s + t * FA_TILE, &tmQ, q_full, 0, q0 + t * FA_BM, bh);
      const uint32_t want = live_epoch(kv.epoch, kv.stride, kv.replay);
      int part = kv.first, jb = 0;
      for (int j = 0; j < nblk; ++j) {
        if (jb == 0) fa_wait_flag(kv.flag[part], want, abort_flag, status);
        const int st = j % FA_STAGES;
        mbar_wait(&kv_empty[st], (static_cast<uint32_t>(j / FA_STAGES) & 1u) ^ 1u, abort_flag, status, 1);
        mbar_expect_tx(&kv_full[st], 2 * FA_TILE);
        tma_load_3d(kv_s + (2 * st) * FA_TILE, &kv.k[part], &kv_full[st], 0, jb * FA_BN, bh);
        tma_load_3d(kv_s + (2 * st + 1) * FA_TILE, &kv.v[part], &kv_full[st], 0, jb * FA_BN, bh);
        if (++jb == nbp) {
          jb = 0;
          if (++part == kv.parts) part = 0;
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ UMMA issuer
    constexpr uint32_t idesc_s = make_idesc_bf16(FA_BM, FA_BN, 0, 0);      // Q (K-major) x K (K-major)
    constexpr uint32_t idesc_pv = make_idesc_bf16(FA_BM, FA_D, 0, 1);      // P (K-major) x V (rows = keys)
    const uint64_t q_desc0 = make_smem_desc_sw128(smem_u32(q_s), 16, 1024);
    const uint64_t k_desc0 = make_smem_desc_sw128(smem_u32(kv_s), 16, 1024);
    const uint64_t v_desc0 = make_smem_desc_sw128(smem_u32(kv_s), 8192, 1024);
    const uint64_t p_desc0 = make_smem_desc_sw128(smem_u32(p_s), 16, 1024);
    auto issue_s = [&](int t, int j) {
      const int st = j % FA_STAGES;
      const uint64_t qd = desc_advance(q_desc0, static_cast<uint32_t>(t * FA_TILE));
      const uint64_t kd = desc_advance(k_desc0, static_cast<uint32_t>((2 * st) * FA_TILE));
      const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(t * FA_BN);
#pragma unroll
      for (int k = 0; k < FA_D / 16; ++k)
        umma_f16_elect(d_tmem, desc_advance(qd, static_cast<uint32_t>(k * 32)),
                       desc_advance(kd, static_cast<uint32_t>(k * 32)), idesc_s, k != 0 ? 1u : 0u);
      umma_commit_elect(&s_full[t]);
    };
    auto issue_pv = [&](int t, int j) {
      const int st = j % FA_STAGES;
      const uint64_t vd = desc_advance(v_desc0, static_cast<uint32_t>((2 * st + 1) * FA_TILE));
      const uint64_t pd = desc_advance(p_desc0, static_cast<uint32_t>(t * FA_P_BYTES));
      const uint32_t d_tmem = tmem_base + 256u + static_cast<uint32_t>(t * FA_D);
#pragma unroll
      for (int k = 0; k < FA_BN / 16; ++k) {
        // P: 16 keys = 32 bytes inside the swizzle row, second atom of 64 keys one tile further;
        // V: 16 keys = 16 rows of 128 bytes
        umma_f16_elect(d_tmem, desc_advance(pd, static_cast<uint32_t>((k >> 2) * FA_TILE + (k & 3) * 32)),
                       desc_advance(vd, static_cast<uint32_t>(k * 2048)), idesc_pv, (j | k) != 0 ? 1u : 0u);
      }
      umma_commit_elect(&pv_done[t]);
    };
    mbar_wait(q_full, 0, abort_flag, status, 2);
    mbar_wait(&kv_full[0], 0, abort_flag, status, 3);
    tc_fence_after_sync();
#pragma unroll
    for (int t = 0; t < FA_QT; ++t) issue_s(t, 0);
    for (int j = 0; j < nblk; ++j) {
      const bool more = j + 1 < nblk;
      if (more)
        mbar_wait(&kv_full[(j + 1) % FA_STAGES], static_cast<uint32_t>((j + 1) / FA_STAGES) & 1u, abort_flag, status, 4);
#pragma unroll
      for (int t = 0; t < FA_QT; ++t) {
        mbar_wait(&p_full[t], static_cast<uint32_t>(j) & 1u, abort_flag, status, 5);
        tc_fence_after_sync();
        if (more) issue_s(t, j + 1);
        issue_pv(t, j);
      }
      umma_commit_elect(&kv_empty[j % FA_STAGES]);
    }
  } else {
    // ------------------------------------------------------------ softmax / output (thread = row of its tile)
    const int tile = (warp - 2) >> 2;
    const int quad = warp & 3;                                       // TMEM lane quadrant of this warp
    const int row = quad * 32 + lane;
    const uint32_t lane_addr = tmem_base + (static_cast<uint32_t>(quad * 32) << 16);
    const uint32_t s_addr = lane_addr + static_cast<uint32_t>(tile * FA_BN);
    const uint32_t o_addr = lane_addr + 256u + static_cast<uint32_t>(tile * FA_D);
    uint8_t* p_row = p_s + tile * FA_P_BYTES + row * 128;
    float m = -INFINITY, l = 0.f;
    int jb = 0;
    for (int j = 0; j < nblk; ++j) {
      const uint32_t ph = static_cast<uint32_t>(j) & 1u;
      const int valid = kv.sk_part - jb * FA_BN;          // columns of this block that are real keys
      if (++jb == nbp) jb = 0;
      mbar_wait(&s_full[tile], ph, abort_flag, status, 6);
      tc_fence_after_sync();
      float mx = -INFINITY;
#pragma unroll 1
      for (int c0 = 0; c0 < FA_BN; c0 += 32) {
        uint32_t r[32];
        tmem_ld_32x32(s_addr + c0, r);
        tmem_ld_wait();
        if (valid >= FA_BN) {
#pragma unroll
          for (int e = 0; e < 32; ++e) mx = fmaxf(mx, __uint_as_float(r[e]));
        } else {
#pragma unroll
          for (int e = 0; e < 32; ++e)
            if (c0 + e < valid) mx = fmaxf(mx, __uint_as_float(r[e]));
        }
      }
      const float m_new = fmaxf(m, mx * scale_log2);
      const bool grow = m_new > m + FA_RESCALE_STEP;       // true for the first block (m = -inf)
      if (j > 0) {
        // P_t of the previous block has been consumed and O_t is at rest
        mbar_wait(&pv_done[tile], ph ^ 1u, abort_flag, status, 7);
        tc_fence_after_sync();
      }
      if (__any_sync(0xffffffffu, grow)) {
        const float alpha = grow ? ex2_approx(m - m_new) : 1.0f;     // 0 for the first block
        if (grow) m = m_new;
        l *= alpha;
        if (j > 0) {
#pragma unroll
          for (int c0 = 0; c0 < FA_D; c0 += 32) {
            uint32_t r[32];
            tmem_ld_32x32(o_addr + c0, r);
            tmem_ld_wait();
#pragma unroll
            for (int e = 0; e < 32; ++e) r[e] = __float_as_uint(__uint_as_float(r[e]) * alpha);
            tmem_st_32x32(o_addr + c0, r);
          }
          tmem_st_wait();
        }
      }
      float sum = 0.f;
#pragma unroll 1
      for (int c0 = 0; c0 < FA_BN; c0 += 32) {
        uint32_t r[32];
        tmem_ld_32x32(s_addr + c0, r);
        tmem_ld_wait();
        float p[32];
        if (valid >= FA_BN) {
#pragma unroll
          for (int e = 0; e < 32; ++e) p[e] = ex2_approx(fmaf(__uint_as_float(r[e]), scale_log2, -m));
        } else {
#pragma unroll
          for (int e = 0; e < 32; ++e)
            p[e] = (c0 + e < valid) ? ex2_approx(fmaf(__uint_as_float(r[e]), scale_log2, -m)) : 0.f;
        }
#pragma unroll
        for (int e = 0; e < 32; ++e) sum += p[e];
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
      l += sum;
      tc_fence_before_sync();
      fence_proxy_async_smem();                            // P must be visible to the tensor core's reads
      __syncwarp();
      if (lane == 0) mbar_arrive(&p_full[tile]);
    }
    mbar_wait(&pv_done[tile], static_cast<uint32_t>(nblk - 1) & 1u, abort_flag, status, 8);
    tc_fence_after_sync();
    const int qrow = q0 + tile * FA_BM + row;
    const float inv = 1.f / l;
    __nv_bfloat16* dst = o + static_cast<long long>(bh) * o_stride_bh + static_cast<long long>(qrow) * o_stride_s;
#pragma unroll
    for (int c0 = 0; c0 < FA_D; c0 += 32) {
      uint32_t r[32];
      tmem_ld_32x32(o_addr + c0, r);
      tmem_ld_wait();
      if (qrow < sq) {
#pragma unroll
        for (int e = 0; e < 32; e += 8) {
          uint4 v;
          v.x = pack_bf16x2(__uint_as_float(r[e]) * inv, __uint_as_float(r[e + 1]) * inv);
          v.y = pack_bf16x2(__uint_as_float(r[e + 2]) * inv, __uint_as_float(r[e + 3]) * inv);
          v.z = pack_bf16x2(__uint_as_float(r[e + 4]) * inv, __uint_as_float(r[e + 5]) * inv);
          v.w = pack_bf16x2(__uint_as_float(r[e + 6]) * inv, __uint_as_float(r[e + 7]) * inv);
          *reinterpret_cast<uint4*>(dst + c0 + e) = v;
        }
      }
    }
    if (qrow < sq) lse[static_cast<long long>(bh) * sq + qrow] = (m + log2f(l)) * 0.6931471805599453f;
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

}  // namespace jb

// Shared set-up of the launchers: the tensor map of one [bh][rows][64] bf16 operand.
static int fa_operand_map(CUtensorMap* m, const void* base, int rows, int bh, long long stride_s, long long stride_bh) {
  const uint32_t box[3] = {jb::FA_D, jb::FA_BM, 1};
  const uint64_t dims[3] = {jb::FA_D, static_cast<uint64_t>(rows), static_cast<uint64_t>(bh)};
  const uint64_t st[2] = {static_cast<uint64_t>(stride_s) * 2, static_cast<uint64_t>(stride_bh) * 2};
  return jb::make_tmap_bf16(m, base, 3, dims, st, box);
}

// C ABI.  q: bf16 [bh][sq][64]; the keys / values come in `parts` parts of `sk_part` rows each,
// k_parts[p] / v_parts[p]: bf16 [bh][sk_part][64] (pointers into this GPU's memory or a peer's); all
// addressed through element strides (`*_stride_s` between rows, `*_stride_bh` between (batch, head)
// slices; multiples of 8 elements, 16-byte aligned bases; K and V parts share one layout).  flags[p]: local
// flag word that must reach `epoch` before part p is read, or null.  The parts are visited in the order
// first, first + 1, ... (cyclically).  o likewise strided; lse is fp32 [bh][sq].  scale multiplies q k^T
// (natural-log softmax).  Returns 0 on success, a negative code if the launch could not be set up.
extern "C" int jb_flash_attn_fwd_parts(const void* q, const void* const* k_parts, const void* const* v_parts,
                                       const void* const* flags, unsigned int epoch, unsigned int stride,
                                       const unsigned int* replay, int parts, int first, void* o, float* lse, int bh,
                                       int sq, int sk_part, long long q_stride_s, long long q_stride_bh,
                                       long long kv_stride_s, long long kv_stride_bh, long long o_stride_s,
                                       long long o_stride_bh, float scale, int* status, void* stream) {
  using namespace jb;
  if (bh < 1 || bh > 65535 || sq < 1 || sk_part < 1 || parts < 1 || parts > FA_MAX_PARTS || first < 0 || first >= parts)
    return -1;
  const long long strides[] = {q_stride_s, q_stride_bh, kv_stride_s, kv_stride_bh, o_stride_s, o_stride_bh};
  for (long long s : strides)
    if (s & 7) return -1;
  if ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(o)) & 15) return -1;
  CUtensorMap tmQ;
  if (fa_operand_map(&tmQ, q, sq, bh, q_stride_s, q_stride_bh) != 0) return -2;
  FaParts kv{};
  for (int p = 0; p < parts; ++p) {
    if ((reinterpret_cast<uintptr_t>(k_parts[p]) | reinterpret_cast<uintptr_t>(v_parts[p])) & 15) return -1;
    if (fa_operand_map(&kv.k[p], k_parts[p], sk_part, bh, kv_stride_s, kv_stride_bh) != 0) return -2;
    if (fa_operand_map(&kv.v[p], v_parts[p], sk_part, bh, kv_stride_s, kv_stride_bh) != 0) return -2;
    kv.flag[p] = flags == nullptr ? nullptr : static_cast<const uint32_t*>(flags[p]);
  }
  kv.epoch = epoch;
  kv.stride = stride;
  kv.replay = replay;
  kv.parts = parts;
  kv.first = first;
  kv.sk_part = sk_part;
  static bool attr_set = false;
  if (!attr_set) {
    if (cudaFuncSetAttribute(flash_attn_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, FA_SMEM) != cudaSuccess)
      return -3;
    attr_set = true;
  }
  const dim3 grid((sq + FA_QT * FA_BM - 1) / (FA_QT * FA_BM), bh);
  flash_attn_fwd_kernel<<<grid, FA_THREADS, FA_SMEM, static_cast<cudaStream_t>(stream)>>>(
      tmQ, kv, static_cast<__nv_bfloat16*>(o), lse, sq, o_stride_s, o_stride_bh, scale * 1.4426950408889634f, status);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

// One local part: q [bh][sq][64], k / v [bh][sk][64] with separate strides for K and V.
extern "C" int jb_flash_attn_fwd(const void* q, const void* k, const void* v, void* o, float* lse, int bh, int sq,
                                 int sk, long long q_stride_s, long long q_stride_bh, long long k_stride_s,
                                 long long k_stride_bh, long long v_stride_s, long long v_stride_bh,
                                 long long o_stride_s, long long o_stride_bh, float scale, int* status, void* stream) {
  if (k_stride_s != v_stride_s || k_stride_bh != v_stride_bh) return -1;
  const void* kp[1] = {k};
  const void* vp[1] = {v};
  return jb_flash_attn_fwd_parts(q, kp, vp, nullptr, 0, 0, nullptr, 1, 0, o, lse, bh, sq, sk, q_stride_s, q_stride_bh,
                                 k_stride_s, k_stride_bh, o_stride_s, o_stride_bh, scale, status, stream);
}
