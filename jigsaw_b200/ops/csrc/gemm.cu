// bf16 GEMM on the 5th-generation tensor cores (tcgen05 + TMEM), fed by TMA.
//
//   C[M,N] = act(A * B + bias)        A, B bf16; accumulation fp32 in TMEM
//
// Both operands may be stored K-major (reduction index contiguous) or MN-major
// (output index contiguous), so the three products a linear layer needs
//   Y  = X  * W^T   (A K-major,  B K-major)
//   dX = dY * W     (A K-major,  B MN-major)
//   dW = dY^T * X   (A MN-major, B MN-major)
// run from the stored tensors without a transpose pass.  A CTA is persistent over
// 128 x BN output tiles; warp 0 issues TMA loads into a multi-stage shared-memory
// ring, warp 1 issues tcgen05.mma into a double-buffered TMEM accumulator, warps
// 2..9 drain finished accumulators (tcgen05.ld), apply bias / GELU and store.
//
// Capability parity: replaces the cuBLAS `torch.matmul` calls of the reference
// (jigsaw/modules/linear/_distributed_matmul.py:100-110, 159-177).

#include "ptx.cuh"
#include "tmap.cuh"

namespace jb {

constexpr int GEMM_BM = 128;
constexpr int GEMM_BK = 64;   // 64 bf16 = one 128-byte swizzle row
constexpr int GEMM_EPI_WARPS = 8;     // two per TMEM lane quadrant, each draining half of the columns
constexpr int GEMM_THREADS = 32 * (2 + GEMM_EPI_WARPS);

struct GemmEpilogue {
  void* c;            // output, row-major [M, ldc]
  long long ldc;      // elements
  const float* bias;  // [N] or nullptr
  int act;            // 0 none, 1 GELU(erf)
  int out_fp32;       // 0 -> bf16 output, 1 -> fp32 output
  int accumulate;     // 1 -> C += result (fp32 output only)
  // Reduce-scatter fused into the epilogue: the N dimension is cut into parts of `part_cols` columns,
  // part p belongs to GPU p, and a tile of part p is stored into c_part[p] (row stride part_cols) --
  // this GPU's slab in GPU p's inbox (a peer pointer) -- instead of into c.  part_cols = 0: off.
  void* c_part[8];
  int part_cols;
};

// All-gather fused into the GEMM: the reduction dimension of A is split over `parts` GPUs, each part is
// a [M, k_part] matrix in that GPU's memory (same symmetric offset everywhere).  The TMA producer reads
// the k-blocks of part p straight from GPU p (plain TMA loads from peer memory, no cluster qualifier)
// once p's epoch flag says its part is complete.
constexpr int GEMM_MAX_PARTS = 8;
struct GemmGather {
  CUtensorMap map[GEMM_MAX_PARTS];
  const uint32_t* flag[GEMM_MAX_PARTS];   // local flag words, one per source rank (null: no wait)
  uint32_t epoch, stride;
  const uint32_t* replay;
  int parts;                               // <= 1: plain GEMM, `map` unused
  int kblocks_per_part;
};

template <int BN>
struct GemmSmem {
  static constexpr int A_BYTES = GEMM_BM * 128;
  static constexpr int B_BYTES = BN * 128;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int STAGES = (BN >= 256) ? 4 : (BN >= 128 ? 6 : 8);
  static constexpr int BAR_BYTES = 256;
  static constexpr int TOTAL = STAGES * STAGE_BYTES + BAR_BYTES + 1024;  // + alignment slack
  // staged epilogue: 32 rows x 128 bytes per epilogue warp behind the barriers
  static constexpr int EPI_STAGE_BYTES = 32 * 128;
  static constexpr int TOTAL_STAGED = TOTAL + GEMM_EPI_WARPS * EPI_STAGE_BYTES;
};

// STAGED = 1: bf16 tiles leave through a per-warp shared-memory buffer so that eight lanes write 128
// contiguous bytes of one output row (a full line per request, which is what stores into a peer's memory
// across NVLink need); STAGED = 0: every thread stores its own row, 16 bytes per instruction.
template <int BN, int A_MN, int B_MN, int STAGED = 0>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                 const __grid_constant__ GemmGather gather, GemmEpilogue ep, int M, int N, int K, int* status) {
  using S = GemmSmem<BN>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + S::STAGES * S::STAGE_BYTES);
  uint64_t* full = bars;                    // [STAGES]
  uint64_t* empty = bars + S::STAGES;       // [STAGES]
  uint64_t* acc_full = bars + 2 * S::STAGES;      // [2]
  uint64_t* acc_empty = bars + 2 * S::STAGES + 2; // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * S::STAGES + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int tiles_m = (M + GEMM_BM - 1) / GEMM_BM;
  const int tiles_n = (N + BN - 1) / BN;
  const int num_tiles = tiles_m * tiles_n;
  const int kblocks = (K + GEMM_BK - 1) / GEMM_BK;
  constexpr uint32_t TMEM_COLS = (2 * BN <= 32) ? 32 : (2 * BN <= 64 ? 64 : (2 * BN <= 128 ? 128 : (2 * BN <= 256 ? 256 : 512)));

  if (threadIdx.x == 0) {
    for (int s = 0; s < S::STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(&acc_full[s], 1);
      mbar_init(&acc_empty[s], GEMM_EPI_WARPS);
    }
    *abort_flag = 0;
    fence_mbar_init();
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
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
      int s = 0;
      uint32_t ph = 0;
      int ready_parts = 0;     // parts [0, ready_parts) have been waited for
      const uint32_t want = live_epoch(gather.epoch, gather.stride, gather.replay);
      for (int t = blockIdx.x; t < num_tiles; t += gridDim.x) {
        const int m0 = (t / tiles_n) * GEMM_BM;
        const int n0 = (t % tiles_n) * BN;
        bool ok = true;
        for (int kb = 0; kb < kblocks && ok; ++kb) {
          ok = mbar_wait(&empty[s], ph ^ 1u, abort_flag, status);
          if (!ok) break;
          const int k0 = kb * GEMM_BK;
          int part = 0;
          if (A_MN == 0 && gather.parts > 1) {
            part = kb / gather.kblocks_per_part;
            while (ready_parts <= part && ok) {          // first use of a part: its owner must have published it
              const uint32_t* f = gather.flag[ready_parts];
              if (f != nullptr) {
                const uint64_t t0 = globaltimer_ns();
                while (true) {
                  uint32_t v;
                  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(f) : "memory");
                  if (static_cast<int32_t>(v - want) >= 0) break;
                  if (*abort_flag || globaltimer_ns() - t0 > JB_WAIT_LIMIT_NS) {
                    *abort_flag = 1;      // every bounded wait of this CTA now returns at once
                    if (status) atomicCAS(status, JB_OK, JB_ERR_FLAG_TIMEOUT);
                    ok = false;
                    break;
                  }
                  __nanosleep(64);
                }
                asm volatile("fence.proxy.async;" ::: "memory");
              }
              ++ready_parts;
            }
            if (!ok) break;
          }
          uint8_t* a_dst = smem + s * S::STAGE_BYTES;
          uint8_t* b_dst = a_dst + S::A_BYTES;
          mbar_expect_tx(&full[s], S::STAGE_BYTES);
          if (A_MN == 0 && gather.parts > 1) {
            tma_load_2d(a_dst, &gather.map[part], &full[s], k0 - part * gather.kblocks_per_part * GEMM_BK, m0);
          } else if (A_MN == 0) {
            tma_load_2d(a_dst, &tmA, &full[s], k0, m0);
          } else {
#pragma unroll
            for (int j = 0; j < GEMM_BM / 64; ++j) tma_load_2d(a_dst + j * 8192, &tmA, &full[s], m0 + 64 * j, k0);
          }
          if (B_MN == 0) {
            tma_load_2d(b_dst, &tmB, &full[s], k0, n0);
          } else {
#pragma unroll
            for (int j = 0; j < BN / 64; ++j) tma_load_2d(b_dst + j * 8192, &tmB, &full[s], n0 + 64 * j, k0);
          }
          if (++s == S::STAGES) {
            s = 0;
            ph ^= 1u;
          }
        }
        if (!ok) break;
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ UMMA issuer
    {
      constexpr uint32_t idesc = make_idesc_bf16(GEMM_BM, BN, A_MN, B_MN);
      int s = 0;
      uint32_t ph = 0;
      int it = 0;
      const uint32_t a_addr0 = smem_u32(smem);
      const uint64_t a_desc0 = A_MN ? make_smem_desc_sw128(a_addr0, 8192, 1024) : make_smem_desc_sw128(a_addr0, 16, 1024);
      const uint64_t b_desc0 = B_MN ? make_smem_desc_sw128(a_addr0 + S::A_BYTES, 8192, 1024)
                                    : make_smem_desc_sw128(a_addr0 + S::A_BYTES, 16, 1024);
      for (int t = blockIdx.x; t < num_tiles; t += gridDim.x, ++it) {
        const int as = it & 1;
        const uint32_t aph = (it >> 1) & 1u;
        mbar_wait(&acc_empty[as], aph ^ 1u, abort_flag, status);
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(as * BN);
        for (int kb = 0; kb < kblocks; ++kb) {
          mbar_wait(&full[s], ph, abort_flag, status);
          tc_fence_after_sync();
          const uint64_t ad0 = desc_advance(a_desc0, static_cast<uint32_t>(s * S::STAGE_BYTES));
          const uint64_t bd0 = desc_advance(b_desc0, static_cast<uint32_t>(s * S::STAGE_BYTES));
#pragma unroll
          for (int k = 0; k < GEMM_BK / 16; ++k) {
            // K-major: 16 K values = 32 bytes inside the swizzle row.
            // MN-major: 16 K values = 16 rows of 128 bytes.
            umma_f16_elect(d_tmem, desc_advance(ad0, k * (A_MN ? 2048 : 32)), desc_advance(bd0, k * (B_MN ? 2048 : 32)), idesc,
                     (kb | k) != 0 ? 1u : 0u);
          }
          umma_commit_elect(&empty[s]);
          if (++s == S::STAGES) {
            s = 0;
            ph ^= 1u;
          }
        }
        umma_commit_elect(&acc_full[as]);
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue (8 warps)
    const int quad = warp & 3;                 // TMEM lanes 32 * quad .. + 31 are the ones this warp may read
    const int chalf = (warp - 2) >> 2;         // which half of the tile's columns
    int it = 0;
    for (int t = blockIdx.x; t < num_tiles; t += gridDim.x, ++it) {
      const int as = it & 1;
      const uint32_t aph = (it >> 1) & 1u;
      const int m0 = (t / tiles_n) * GEMM_BM;
      const int n0 = (t % tiles_n) * BN;
      if (!mbar_wait(&acc_full[as], aph, abort_flag, status)) break;
      tc_fence_after_sync();
      const int row = m0 + quad * 32 + lane;
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + static_cast<uint32_t>(as * BN);
      // destination of this tile: the plain output, or the slab of the GPU that owns these columns
      void* c_base = ep.c;
      long long ldc = ep.ldc;
      int col_shift = 0;
      if (ep.part_cols > 0) {
        const int part = n0 / ep.part_cols;
        c_base = ep.c_part[part];
        ldc = ep.part_cols;
        col_shift = part * ep.part_cols;
      }
      bool staged_done = false;
      if constexpr (STAGED != 0 && BN >= 128) {
        if (!ep.out_fp32 && n0 + BN <= N && (ldc & 7) == 0) {
          uint8_t* stage = smem + S::STAGES * S::STAGE_BYTES + S::BAR_BYTES + (warp - 2) * S::EPI_STAGE_BYTES;
          __nv_bfloat16* cb = reinterpret_cast<__nv_bfloat16*>(c_base);
#pragma unroll 1
          for (int c0 = chalf * (BN / 2); c0 < (chalf + 1) * (BN / 2); c0 += 64) {
#pragma unroll
            for (int h = 0; h < 2; ++h) {
              uint32_t r[32];
              tmem_ld_32x32(taddr + c0 + 32 * h, r);
              tmem_ld_wait();
              const int col0 = n0 + c0 + 32 * h;
#pragma unroll
              for (int j = 0; j < 32; j += 8) {
                float v[8];
#pragma unroll
                for (int e = 0; e < 8; ++e) {
                  float x = __uint_as_float(r[j + e]);
                  if (ep.bias != nullptr) x += __ldg(ep.bias + col0 + j + e);
                  if (ep.act == 1) x = gelu_erf(x);
                  v[e] = x;
                }
                uint4 o;
                o.x = pack_bf16x2(v[0], v[1]);
                o.y = pack_bf16x2(v[2], v[3]);
                o.z = pack_bf16x2(v[4], v[5]);
                o.w = pack_bf16x2(v[6], v[7]);
                const int chunk = h * 4 + (j >> 3);                  // 16-byte chunk of the 128-byte staged row
                *reinterpret_cast<uint4*>(stage + lane * 128 + ((chunk ^ (lane & 7)) << 4)) = o;
              }
            }
            __syncwarp();
#pragma unroll
            for (int i = 0; i < 8; ++i) {                            // four rows per instruction, 128 bytes each
              const int rl = i * 4 + (lane >> 3);
              const int chunk = lane & 7;
              const int grow = m0 + quad * 32 + rl;
              const uint4 o = *reinterpret_cast<const uint4*>(stage + rl * 128 + ((chunk ^ (rl & 7)) << 4));
              if (grow < M)
                *reinterpret_cast<uint4*>(cb + static_cast<long long>(grow) * ldc + (n0 + c0 - col_shift) + chunk * 8) = o;
            }
            __syncwarp();
          }
          staged_done = true;
        }
      }
#pragma unroll 1
      for (int c0 = chalf * (BN / 2); c0 < (chalf + 1) * (BN / 2) && !staged_done; c0 += 32) {
        uint32_t r[32];
        tmem_ld_32x32(taddr + c0, r);
        tmem_ld_wait();
        if (row < M) {
          const int col0 = n0 + c0;
          float v[32];
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            float x = __uint_as_float(r[j]);
            if (ep.bias != nullptr && col0 + j < N) x += __ldg(ep.bias + col0 + j);
            if (ep.act == 1) x = gelu_erf(x);
            v[j] = x;
          }
          if (ep.out_fp32) {
            float* dst = reinterpret_cast<float*>(c_base) + static_cast<long long>(row) * ldc + (col0 - col_shift);
            if (col0 + 32 <= N && (ldc & 3) == 0) {
#pragma unroll
              for (int j = 0; j < 32; j += 4) {
                float4 o = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
                if (ep.accumulate) {
                  const float4 old = *reinterpret_cast<float4*>(dst + j);
                  o.x += old.x; o.y += old.y; o.z += old.z; o.w += old.w;
                }
                *reinterpret_cast<float4*>(dst + j) = o;
              }
            } else {
              for (int j = 0; j < 32 && col0 + j < N; ++j) dst[j] = ep.accumulate ? dst[j] + v[j] : v[j];
            }
          } else {
            __nv_bfloat16* dst =
                reinterpret_cast<__nv_bfloat16*>(c_base) + static_cast<long long>(row) * ldc + (col0 - col_shift);
            if (col0 + 32 <= N && (ldc & 7) == 0) {
#pragma unroll
              for (int j = 0; j < 32; j += 8) {
                uint4 o;
                o.x = pack_bf16x2(v[j], v[j + 1]);
                o.y = pack_bf16x2(v[j + 2], v[j + 3]);
                o.z = pack_bf16x2(v[j + 4], v[j + 5]);
                o.w = pack_bf16x2(v[j + 6], v[j + 7]);
                *reinterpret_cast<uint4*>(dst + j) = o;
              }
            } else {
              for (int j = 0; j < 32 && col0 + j < N; ++j) dst[j] = __float2bfloat16(v[j]);
            }
          }
        }
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&acc_empty[as]);
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

struct GatherSpec {                      // host-side description of a gathered A operand
  const void* part[GEMM_MAX_PARTS];
  const uint32_t* flag[GEMM_MAX_PARTS];
  uint32_t epoch, stride;
  const uint32_t* replay;
  int parts, k_part;
};

template <int BN, int A_MN, int B_MN, int STAGED = 0>
static int launch_gemm(const void* A, const void* B, const GemmEpilogue& ep, int M, int N, int K, long long lda,
                       long long ldb, int sm_count, int* status, cudaStream_t stream,
                       const GatherSpec* gs = nullptr) {
  using S = GemmSmem<BN>;
  CUtensorMap tmA, tmB;
  {
    // K-major: memory [rows = M][K contiguous]; MN-major: memory [rows = K][M contiguous].
    uint64_t dims[2], strides[1];
    uint32_t box[2];
    if (A_MN == 0) {
      // with a gathered A operand this map only describes part 0 (the kernel uses the per-part maps)
      dims[0] = (gs != nullptr && gs->parts > 1) ? gs->k_part : K; dims[1] = M; box[0] = 64; box[1] = GEMM_BM;
    } else {
      dims[0] = M; dims[1] = K; box[0] = 64; box[1] = GEMM_BK;
    }
    strides[0] = static_cast<uint64_t>(lda) * 2;
    if (make_tmap_bf16(&tmA, A, 2, dims, strides, box) != 0) return -2;
    if (B_MN == 0) {
      dims[0] = K; dims[1] = N; box[0] = 64; box[1] = BN;
    } else {
      dims[0] = N; dims[1] = K; box[0] = 64; box[1] = GEMM_BK;
    }
    strides[0] = static_cast<uint64_t>(ldb) * 2;
    if (make_tmap_bf16(&tmB, B, 2, dims, strides, box) != 0) return -2;
  }
  GemmGather gather{};
  if (gs != nullptr && gs->parts > 1) {
    if (A_MN != 0 || gs->parts > GEMM_MAX_PARTS || gs->k_part % GEMM_BK != 0) return -1;
    for (int p = 0; p < gs->parts; ++p) {
      uint64_t dims[2] = {static_cast<uint64_t>(gs->k_part), static_cast<uint64_t>(M)};
      uint64_t strides[1] = {static_cast<uint64_t>(lda) * 2};
      uint32_t box[2] = {64, GEMM_BM};
      if (make_tmap_bf16(&gather.map[p], gs->part[p], 2, dims, strides, box) != 0) return -2;
      gather.flag[p] = gs->flag[p];
    }
    gather.epoch = gs->epoch; gather.stride = gs->stride; gather.replay = gs->replay;
    gather.parts = gs->parts;
    gather.kblocks_per_part = gs->k_part / GEMM_BK;
  }
  auto kern = gemm_bf16_kernel<BN, A_MN, B_MN, STAGED>;
  constexpr int smem_bytes = STAGED != 0 ? S::TOTAL_STAGED : S::TOTAL;
  static_assert(smem_bytes <= 227 * 1024, "shared memory of one CTA");
  static bool attr_set = false;
  if (!attr_set) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes) != cudaSuccess) return -3;
    attr_set = true;
  }
  const int tiles = ((M + GEMM_BM - 1) / GEMM_BM) * ((N + BN - 1) / BN);
  const int grid = tiles < sm_count ? tiles : sm_count;
  kern<<<grid, GEMM_THREADS, smem_bytes, stream>>>(tmA, tmB, gather, ep, M, N, K, status);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

}  // namespace jb

// Process-wide switch: bf16 outputs of jb_gemm_bf16 leave through the staged epilogue (128-byte row
// pieces written by eight lanes) instead of one row per thread.  Off unless the host turns it on.
static int g_staged_epilogue = 1;   // measured faster on every shape (0.77 / 0.69 / 0.70 against 0.73 / 0.44 / 0.62 of the cuBLAS peak)
extern "C" void jb_set_staged_epilogue(int on) { g_staged_epilogue = on; }

// C ABI.  a_mn / b_mn select the stored layout of each operand:
//   a_mn = 0: A is [M, K] row-major (lda = row stride);  a_mn = 1: A is [K, M] row-major.
//   b_mn = 0: B is [N, K] row-major (ldb = row stride);  b_mn = 1: B is [K, N] row-major.
// Leading dimensions must be multiples of 8 elements and base pointers 16-byte aligned.
// Returns 0 on success, a negative code if the launch could not be set up.
extern "C" int jb_gemm_bf16(const void* A, const void* B, void* C, const float* bias, int M, int N, int K,
                            long long lda, long long ldb, long long ldc, int a_mn, int b_mn, int act,
                            int out_fp32, int accumulate, int sm_count, int* status, void* stream) {
  using namespace jb;
  if ((lda & 7) || (ldb & 7) || (reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(B) & 15))
    return -1;
  GemmEpilogue ep{C, ldc, bias, act, out_fp32, accumulate};
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int key = (a_mn ? 2 : 0) | (b_mn ? 1 : 0);
  // Tile width: wide tiles when N is large, narrower ones to fill the SMs otherwise.
  const int tiles128 = ((M + 127) / 128) * ((N + 127) / 128);
  const bool wide = (N >= 256) && (((M + 127) / 128) * ((N + 255) / 256) >= sm_count);
  const bool narrow = (N <= 64) || (tiles128 < sm_count / 2 && N % 64 == 0);
#define JB_GEMM_DISPATCH(BN)                                                                                   \
  switch (key) {                                                                                                \
    case 0: return launch_gemm<BN, 0, 0>(A, B, ep, M, N, K, lda, ldb, sm_count, status, st);                    \
    case 1: return launch_gemm<BN, 0, 1>(A, B, ep, M, N, K, lda, ldb, sm_count, status, st);                    \
    case 2: return launch_gemm<BN, 1, 0>(A, B, ep, M, N, K, lda, ldb, sm_count, status, st);                    \
    default: return launch_gemm<BN, 1, 1>(A, B, ep, M, N, K, lda, ldb, sm_count, status, st);                   \
  }
#define JB_GEMM_DISPATCH_STAGED(BN)                                                                            \
  switch (key) {                                                                                                \
    case 0: return launch_gemm<BN, 0, 0, 1>(A, B, ep, M, N, K, lda, ldb, sm_count, status, st);                 \
    case 1: return launch_gemm<BN, 0, 1, 1>(A, B, ep, M, N, K, lda, ldb, sm_count, status, st);                 \
    case 2: return launch_gemm<BN, 1, 0, 1>(A, B, ep, M, N, K, lda, ldb, sm_count, status, st);                 \
    default: return launch_gemm<BN, 1, 1, 1>(A, B, ep, M, N, K, lda, ldb, sm_count, status, st);                \
  }
  const bool staged = g_staged_epilogue != 0 && out_fp32 == 0 && !narrow;
  if (wide) {
    if (staged) { JB_GEMM_DISPATCH_STAGED(256) }
    JB_GEMM_DISPATCH(256)
  } else if (narrow) {
    JB_GEMM_DISPATCH(64)
  } else {
    if (staged) { JB_GEMM_DISPATCH_STAGED(128) }
    JB_GEMM_DISPATCH(128)
  }
#undef JB_GEMM_DISPATCH
#undef JB_GEMM_DISPATCH_STAGED
}

// C = act(A * B^T + bias) where the reduction dimension of A is split over `parts` GPUs: part p is a
// row-major [M, k_part] bf16 matrix (row stride lda_part) at a_part[p] (peer pointers allowed).  Before
// the first k-block of part p is requested the kernel waits (bounded) until flag[p] (a local word, null
// = ready) reaches epoch (+ stride * *replay inside a CUDA graph).  B is [N, parts * k_part] row-major.
struct JbGather {
  const void* a_part[8];
  const void* flag[8];
  unsigned int epoch, stride;
  const unsigned int* replay;
  int parts, k_part;
  long long lda_part;
};

extern "C" int jb_gemm_bf16_gather(const JbGather* g, const void* B, void* C, const float* bias, int M, int N,
                                   long long ldb, long long ldc, int act, int out_fp32, int sm_count, int* status,
                                   void* stream) {
  using namespace jb;
  if (g == nullptr || g->parts < 2 || g->parts > GEMM_MAX_PARTS || (g->lda_part & 7) || (ldb & 7)) return -1;
  GatherSpec gs{};
  for (int p = 0; p < g->parts; ++p) {
    if (reinterpret_cast<uintptr_t>(g->a_part[p]) & 15) return -1;
    gs.part[p] = g->a_part[p];
    gs.flag[p] = static_cast<const uint32_t*>(g->flag[p]);
  }
  gs.epoch = g->epoch; gs.stride = g->stride; gs.replay = g->replay; gs.parts = g->parts; gs.k_part = g->k_part;
  const int K = g->parts * g->k_part;
  GemmEpilogue ep{C, ldc, bias, act, out_fp32, 0};
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const bool wide = (N >= 256) && (((M + 127) / 128) * ((N + 255) / 256) >= sm_count);
  const bool narrow = (N <= 64) || ((((M + 127) / 128) * ((N + 127) / 128)) < sm_count / 2 && N % 64 == 0);
  const void* A0 = g->a_part[0];
  if (wide) return launch_gemm<256, 0, 0>(A0, B, ep, M, N, K, g->lda_part, ldb, sm_count, status, st, &gs);
  if (narrow) return launch_gemm<64, 0, 0>(A0, B, ep, M, N, K, g->lda_part, ldb, sm_count, status, st, &gs);
  return launch_gemm<128, 0, 0>(A0, B, ep, M, N, K, g->lda_part, ldb, sm_count, status, st, &gs);
}

namespace jb {
__global__ void publish_kernel(uint32_t* f0, uint32_t* f1, uint32_t* f2, uint32_t* f3, uint32_t* f4, uint32_t* f5,
                               uint32_t* f6, uint32_t* f7, uint32_t epoch, uint32_t stride, const uint32_t* replay) {
  uint32_t* f[8] = {f0, f1, f2, f3, f4, f5, f6, f7};
  const uint32_t e = live_epoch(epoch, stride, replay);
  __threadfence_system();
  if (threadIdx.x < 8 && f[threadIdx.x] != nullptr)
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(f[threadIdx.x]), "r"(e) : "memory");
}
}  // namespace jb

// Publish `epoch` into up to eight flag words (peer pointers allowed) once all earlier work of the stream
// is complete: the hand-off from a producer of symmetric memory to kernels on other GPUs that read it.
extern "C" int jb_publish(void* const* flags, int n, unsigned int epoch, unsigned int stride,
                          const unsigned int* replay, void* stream) {
  if (n < 0 || n > 8) return -1;
  uint32_t* f[8] = {};
  for (int i = 0; i < n; ++i) f[i] = static_cast<uint32_t*>(flags[i]);
  jb::publish_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(f[0], f[1], f[2], f[3], f[4], f[5], f[6], f[7],
                                                                      epoch, stride, replay);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

// C = A * B with the reduce-scatter of C's column parts fused into the epilogue: column part p
// (part_cols columns, part_cols a multiple of 64) of this GPU's partial product is stored as a bf16
// [M, part_cols] slab at c_part[p] (for p != this GPU a pointer into GPU p's inbox).  The caller
// publishes a flag afterwards (jb_publish) and the owners sum their slabs (jb_sum_slabs).
static int gemm_scatter(const void* A, const void* B, void* const* c_part, int parts, int part_cols, int M, int K,
                        long long lda, long long ldb, int a_mn, int b_mn, int staged, int sm_count, int* status,
                        void* stream) {
  using namespace jb;
  if (parts < 2 || parts > 8 || part_cols % 64 != 0 || (lda & 7) || (ldb & 7)) return -1;
  const int N = parts * part_cols;
  GemmEpilogue ep{};
  ep.out_fp32 = 0;
  ep.part_cols = part_cols;
  for (int p = 0; p < parts; ++p) ep.c_part[p] = c_part[p];
  ep.c = c_part[0];
  ep.ldc = part_cols;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int key = (a_mn ? 2 : 0) | (b_mn ? 1 : 0);
  // tiles must not straddle two parts: the tile width divides part_cols
  const int bn = (part_cols % 256 == 0 && ((M + 127) / 128) * (N / 256) >= sm_count) ? 256 : (part_cols % 128 == 0 ? 128 : 64);
#define JB_GEMM_SC(BN)                                                                              \
  switch (key) {                                                                                     \
    case 0: return launch_gemm<BN, 0, 0>(A, B, ep, M, N, K, lda, ldb, sm_count, status, st);        \
    case 1: return launch_gemm<BN, 0, 1>(A, B, ep, M, N, K, lda, ldb, sm_count, status, st);        \
    case 2: return launch_gemm<BN, 1, 0>(A, B, ep, M, N, K, lda, ldb, sm_count, status, st);        \
    default: return launch_gemm<BN, 1, 1>(A, B, ep, M, N, K, lda, ldb, sm_count, status, st);       \
  }
#define JB_GEMM_SC_STAGED(BN)                                                                       \
  switch (key) {                                                                                     \
    case 0: return launch_gemm<BN, 0, 0, 1>(A, B, ep, M, N, K, lda, ldb, sm_count, status, st);     \
    case 1: return launch_gemm<BN, 0, 1, 1>(A, B, ep, M, N, K, lda, ldb, sm_count, status, st);     \
    case 2: return launch_gemm<BN, 1, 0, 1>(A, B, ep, M, N, K, lda, ldb, sm_count, status, st);     \
    default: return launch_gemm<BN, 1, 1, 1>(A, B, ep, M, N, K, lda, ldb, sm_count, status, st);    \
  }
  if (staged != 0 && bn == 256) { JB_GEMM_SC_STAGED(256) }
  if (staged != 0 && bn == 128) { JB_GEMM_SC_STAGED(128) }
  if (bn == 256) { JB_GEMM_SC(256) } else if (bn == 128) { JB_GEMM_SC(128) } else { JB_GEMM_SC(64) }
#undef JB_GEMM_SC
#undef JB_GEMM_SC_STAGED
}

extern "C" int jb_gemm_bf16_scatter(const void* A, const void* B, void* const* c_part, int parts, int part_cols, int M,
                                    int K, long long lda, long long ldb, int a_mn, int b_mn, int sm_count, int* status,
                                    void* stream) {
  return gemm_scatter(A, B, c_part, parts, part_cols, M, K, lda, ldb, a_mn, b_mn, 0, sm_count, status, stream);
}

// The same product with the staged epilogue (tiles leave through shared memory as 128-byte row pieces).
extern "C" int jb_gemm_bf16_scatter_staged(const void* A, const void* B, void* const* c_part, int parts, int part_cols,
                                           int M, int K, long long lda, long long ldb, int a_mn, int b_mn, int sm_count,
                                           int* status, void* stream) {
  return gemm_scatter(A, B, c_part, parts, part_cols, M, K, lda, ldb, a_mn, b_mn, 1, sm_count, status, stream);
}

namespace jb {
// out = sum over the slabs [parts][n] (bf16) of this GPU's inbox, after every source rank's flag has
// reached the epoch (bounded wait by one thread per CTA; null flag = this GPU's own slab).
struct SumSlabArgs {
  const __nv_bfloat16* slabs;
  long long n;                 // elements per slab
  int parts;
  const uint32_t* flag[8];
  uint32_t epoch, stride;
  const uint32_t* replay;
  void* out; int out_bf16;
  int* status;
};

__global__ void __launch_bounds__(256) sum_slabs_kernel(const SumSlabArgs a) {
  __shared__ int ok;
  if (threadIdx.x == 0) {
    ok = 1;
    const uint32_t want = live_epoch(a.epoch, a.stride, a.replay);
    const uint64_t t0 = globaltimer_ns();
    for (int p = 0; p < a.parts && ok; ++p) {
      const uint32_t* f = a.flag[p];
      if (f == nullptr) continue;
      while (true) {
        uint32_t v;
        asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(f) : "memory");
        if (static_cast<int32_t>(v - want) >= 0) break;
        if (globaltimer_ns() - t0 > JB_WAIT_LIMIT_NS) {
          if (a.status) atomicCAS(a.status, JB_OK, JB_ERR_FLAG_TIMEOUT);
          ok = 0;
          break;
        }
        __nanosleep(64);
      }
    }
  }
  __syncthreads();
  for (long long i = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) * 8; i < a.n;
       i += static_cast<long long>(gridDim.x) * blockDim.x * 8) {
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int p = 0; p < a.parts; ++p) {
      const uint4 v = __ldcg(reinterpret_cast<const uint4*>(a.slabs + static_cast<long long>(p) * a.n + i));
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        acc[2 * j] += __low2float(h[j]);
        acc[2 * j + 1] += __high2float(h[j]);
      }
    }
    if (a.out_bf16) {
      uint4 o;
      o.x = pack_bf16x2(acc[0], acc[1]); o.y = pack_bf16x2(acc[2], acc[3]);
      o.z = pack_bf16x2(acc[4], acc[5]); o.w = pack_bf16x2(acc[6], acc[7]);
      *reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(a.out) + i) = o;
    } else {
      float* o = static_cast<float*>(a.out) + i;
      *reinterpret_cast<float4*>(o) = make_float4(acc[0], acc[1], acc[2], acc[3]);
      *reinterpret_cast<float4*>(o + 4) = make_float4(acc[4], acc[5], acc[6], acc[7]);
    }
  }
}
}  // namespace jb

// out[n] = sum_p slabs[p][n] (bf16 slabs, n a multiple of 8) once flag[p] >= epoch for every p.
extern "C" int jb_sum_slabs(const void* slabs, long long n, int parts, const void* const* flags, unsigned int epoch,
                            unsigned int stride, const unsigned int* replay, void* out, int out_bf16, int* status,
                            int sm_count, void* stream) {
  using namespace jb;
  if (n <= 0 || (n & 7) || parts < 1 || parts > 8) return -1;
  SumSlabArgs a{};
  a.slabs = static_cast<const __nv_bfloat16*>(slabs); a.n = n; a.parts = parts;
  for (int p = 0; p < parts; ++p) a.flag[p] = static_cast<const uint32_t*>(flags[p]);
  a.epoch = epoch; a.stride = stride; a.replay = replay; a.out = out; a.out_bf16 = out_bf16; a.status = status;
  long long grid = (n / 8 + 255) / 256;
  if (grid > static_cast<long long>(sm_count) * 4) grid = static_cast<long long>(sm_count) * 4;
  sum_slabs_kernel<<<static_cast<unsigned int>(grid), 256, 0, static_cast<cudaStream_t>(stream)>>>(a);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}
