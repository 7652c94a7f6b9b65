// Halo-fused 3x3 convolution (stride 1, padding 1) for 64-channel NHWC bf16 tiles on
// tcgen05 tensor cores: forward, data gradient and weight gradient.
//
// Data layout.  Every activation / gradient tile lives in a PADDED buffer
//   [NB][H+2][W+2][64] bf16
// whose one-pixel border is the halo.  The producer of a tile (the epilogue of the
// previous convolution, or the pack kernel) writes the interior locally and stores
// its edge rows / columns / corner pixels straight into the borders of the up to
// eight neighbouring ranks' buffers over NVLink (plain peer stores), then publishes
// an epoch in the neighbours' flag words.  A border on the edge of the global domain
// is never written and stays zero, which is the convolution's zero padding.  The
// consumer waits (bounded) for the flags and afterwards reads LOCAL memory only, so
// every operand tile is fetched by TMA (no cluster multicast anywhere).
//
// Implicit GEMM.  An output tile is 128 consecutive pixels of one row: M = 128,
// N = output channels, K = 9 taps x 64 input channels.  A CTA walks down a column
// strip; input rows are kept in an 8-slot shared-memory window (130 pixels x 128 B,
// 128-byte swizzle) so each input row is fetched from L2 about once, and the nine
// taps are nine shifted views of three slots: the shift is applied to the start
// address of the UMMA shared-memory descriptor.  The 9 x 64 x N weights stay resident
// in shared memory for the life of the CTA.  Accumulators are double-buffered in TMEM
// so the epilogue of row h overlaps the MMAs of row h+1.
//
// Capability parity: replaces halo_gather + F.conv2d, conv2d_input + halo_scatter_add
// and conv2d_weight of the reference (jigsaw/modules/convolution/_conv/halo.py:66-251,
// jigsaw/modules/convolution/_conv/distributed.py:212-396).

#include "ptx.cuh"
#include "tmap.cuh"

namespace jb {

constexpr int CV_TW = 128;                        // output pixels per tile
constexpr int CV_BOXW = 130;                      // input pixels per slot (tile + 2)
constexpr int CV_SLOT_BYTES = 136 * 128;          // 17 KiB, keeps slots 1024-byte aligned
constexpr int CV_SLOTS = 7;                       // window slots of the forward / data-gradient kernel
constexpr int CV_CHUNK = 5;                       // output rows per window refill (slots - 2)
constexpr int WG_SLOTS = 8;                       // window of the weight-gradient kernel
constexpr int WG_CHUNK = 6;
constexpr int CV_STAGE_BYTES = 128 * 128;         // one 128-pixel x 64-channel bf16 tile
constexpr int CV_MMA_WARPS = 4;                   // MMA-issuing warps = accumulator buffers in TMEM
#ifndef JB_CV_EPI_WARPS
#define JB_CV_EPI_WARPS 16
#endif
constexpr int CV_EPI_WARPS = JB_CV_EPI_WARPS;      // two or four per TMEM lane quadrant
constexpr int CV_THREADS = 32 * (1 + CV_MMA_WARPS + CV_EPI_WARPS);  // + one TMA producer warp

struct HaloPush {
  // Index (sy + 1) * 3 + (sx + 1); entry 4 (self) unused.  Null = no neighbour there.
  void* buf[9];         // base of that neighbour's padded buffer (same shape as ours)
  uint32_t* flag[9];    // flag word on that neighbour to set once all our stores are out
  uint32_t epoch;       // value to publish (plus stride * *replay when the launch sits in a replayed CUDA graph)
  uint32_t enabled;     // 0: no neighbour at all (single rank)
  uint32_t stride;      // productions of this flag slot per replay of the graph
  const uint32_t* replay;  // device counter of graph replays, or null outside a graph
};

struct HaloWait {
  const uint32_t* flag[9];  // local flag words to wait for (null = none)
  uint32_t epoch;
  uint32_t enabled;
  uint32_t stride;          // as in HaloPush
  const uint32_t* replay;
};

struct ConvArgs {
  int NB, H, W;            // local tile
  int tiles_w;             // ceil(W / 128)
  int rows_per_strip;
  int nstrips;
  int cout_real;           // channels actually stored by the dense outputs
  // epilogue
  const float* bias;               // [N] fp32 or null
  const __nv_bfloat16* gelu_src;   // dense [NB][H][W][64]: multiply the result by it (data gradient: the saved
                                   // derivative of the activation that follows the previous layer)
  __nv_bfloat16* dense_pre;        // dense [NB][H][W][64]: act'(value before the activation), saved for backward
  int act;                         // 1: GELU after bias
  __nv_bfloat16* padded_out;       // padded [NB][H+2][W+2][64] output (interior) + halo push
  __nv_bfloat16* dense_out;        // dense [NB][H][W][cout_real] output
  HaloPush push;
  HaloWait wait;
  unsigned int* done_counter;      // local scratch word, zero before the first launch
  int* status;
};

__device__ __forceinline__ void halo_wait_all(const HaloWait& w, volatile int* abort_flag, int* status) {
  if (!w.enabled) return;
  const uint64_t t0 = globaltimer_ns();
  const uint32_t want = live_epoch(w.epoch, w.stride, w.replay);
  for (int d = 0; d < 9; ++d) {
    const uint32_t* f = w.flag[d];
    if (f == nullptr) continue;
    while (true) {
      uint32_t v;
      asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(f) : "memory");
      if (static_cast<int32_t>(v - want) >= 0) break;
      if (*abort_flag) return;
      if (globaltimer_ns() - t0 > JB_WAIT_LIMIT_NS) {
        *abort_flag = 1;
        if (status) atomicCAS(status, JB_OK, JB_ERR_FLAG_TIMEOUT);
        return;
      }
      __nanosleep(100);
    }
  }
  // Peer data arrived through the generic proxy; the TMA engine reads through the async proxy.
  asm volatile("fence.proxy.async;" ::: "memory");
}

// Called by every thread after the role loops.  The last CTA of the grid publishes the epoch.
__device__ __forceinline__ void halo_publish(const HaloPush& p, unsigned int* done_counter) {
  if (!p.enabled) return;
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence_system();
    const unsigned int prev = atomicAdd(done_counter, 1u);
    if (prev == gridDim.x - 1) {
      *done_counter = 0u;
      __threadfence_system();
      const uint32_t epoch = live_epoch(p.epoch, p.stride, p.replay);
      for (int d = 0; d < 9; ++d) {
        if (p.flag[d] != nullptr) {
          asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p.flag[d]), "r"(epoch) : "memory");
        }
      }
    }
  }
}

// Store 32 (or fewer) consecutive channels of one pixel into the interior of the local padded
// buffer and, for pixels on the tile edge, into the matching border of the neighbours.
template <int NV, bool LOCAL = true>  // NV = number of uint4 (8 channels each); LOCAL: also store the interior
__device__ __forceinline__ void store_padded_with_halo(const ConvArgs& a, const uint4 (&v)[NV], int n, int h, int w,
                                                       int c0) {
  const long long prow = static_cast<long long>(a.W + 2) * 64;
  const long long pimg = static_cast<long long>(a.H + 2) * prow;
  if (LOCAL) {
    __nv_bfloat16* dst = a.padded_out + n * pimg + (h + 1) * prow + static_cast<long long>(w + 1) * 64 + c0;
#pragma unroll
    for (int j = 0; j < NV; ++j) reinterpret_cast<uint4*>(dst)[j] = v[j];
  }
  if (!a.push.enabled) return;
  const bool top = (h == 0), bot = (h == a.H - 1), lef = (w == 0), rig = (w == a.W - 1);
  if (!(top || bot || lef || rig)) return;
#pragma unroll
  for (int sy = -1; sy <= 1; ++sy) {
#pragma unroll
    for (int sx = -1; sx <= 1; ++sx) {
      if (sy == 0 && sx == 0) continue;
      const int d = (sy + 1) * 3 + (sx + 1);
      if (a.push.buf[d] == nullptr) continue;
      const bool hit_y = (sy == -1) ? top : (sy == 1 ? bot : true);
      const bool hit_x = (sx == -1) ? lef : (sx == 1 ? rig : true);
      if (!(hit_y && hit_x)) continue;
      // Our top row is the neighbour-above's bottom border, and so on.
      const int dr = (sy == -1) ? (a.H + 1) : (sy == 1 ? 0 : h + 1);
      const int dc = (sx == -1) ? (a.W + 1) : (sx == 1 ? 0 : w + 1);
      __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(a.push.buf[d]) + n * pimg + dr * prow +
                           static_cast<long long>(dc) * 64 + c0;
#pragma unroll
      for (int j = 0; j < NV; ++j) reinterpret_cast<uint4*>(dst)[j] = v[j];
    }
  }
}


// Shared epilogue of the convolution kernels: CPW consecutive output channels (starting at
// c0) of pixel (n, h, w) held in fp32 registers.
// Bias values of the CPW channels a thread owns; they are the same for every tile, so the
// kernels load them once into registers.
template <int CPW>
__device__ __forceinline__ void load_bias_regs(const ConvArgs& a, int c0, float (&b)[CPW]) {
#pragma unroll
  for (int j = 0; j < CPW; ++j) b[j] = (a.bias != nullptr) ? __ldg(a.bias + c0 + j) : 0.f;
}

// The GELU'(src) operand of a pixel, fetched early (before waiting for the accumulator) so
// that its latency hides behind the wait.
template <int CPW>
__device__ __forceinline__ void prefetch_gelu_src(const ConvArgs& a, int n, int h, int w, int c0, uint4 (&g)[CPW / 8]) {
  if (a.gelu_src == nullptr || w >= a.W) return;
  const long long pix = (static_cast<long long>(n) * a.H + h) * static_cast<long long>(a.W) + w;
  const uint4* src = reinterpret_cast<const uint4*>(a.gelu_src + pix * 64 + c0);
#pragma unroll
  for (int q = 0; q < CPW / 8; ++q) g[q] = __ldg(src + q);
}

template <int CPW>
__device__ __forceinline__ void conv_epilogue(const ConvArgs& a, float (&v)[CPW], const float (&bias)[CPW],
                                              const uint4 (&gsrc)[CPW / 8], int n, int h, int w, int c0) {
  const long long pix = (static_cast<long long>(n) * a.H + h) * static_cast<long long>(a.W) + w;
#pragma unroll
  for (int j = 0; j < CPW; ++j) v[j] += bias[j];
  if (a.gelu_src != nullptr) {
#pragma unroll
    for (int q = 0; q < CPW / 8; ++q) {
      const uint4 u = gsrc[q];
      const uint32_t uu[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
      for (int p = 0; p < 4; ++p) {
        const __nv_bfloat162 b2 = *reinterpret_cast<const __nv_bfloat162*>(&uu[p]);
        v[q * 8 + 2 * p] *= __low2float(b2);
        v[q * 8 + 2 * p + 1] *= __high2float(b2);
      }
    }
  }
  if (a.act == 1) {
    float d[CPW];
#pragma unroll
    for (int j = 0; j < CPW; j += 2) gelu_erf_with_grad_x2(v[j], v[j + 1], v[j], v[j + 1], d[j], d[j + 1]);
    if (a.dense_pre != nullptr) {
      uint4* dst = reinterpret_cast<uint4*>(a.dense_pre + pix * 64 + c0);
#pragma unroll
      for (int q = 0; q < CPW / 8; ++q) {
        uint4 o;
        o.x = pack_bf16x2(d[q * 8 + 0], d[q * 8 + 1]);
        o.y = pack_bf16x2(d[q * 8 + 2], d[q * 8 + 3]);
        o.z = pack_bf16x2(d[q * 8 + 4], d[q * 8 + 5]);
        o.w = pack_bf16x2(d[q * 8 + 6], d[q * 8 + 7]);
        dst[q] = o;
      }
    }
  }
  if (a.padded_out != nullptr) {
    uint4 o[CPW / 8];
#pragma unroll
    for (int q = 0; q < CPW / 8; ++q) {
      o[q].x = pack_bf16x2(v[q * 8 + 0], v[q * 8 + 1]);
      o[q].y = pack_bf16x2(v[q * 8 + 2], v[q * 8 + 3]);
      o[q].z = pack_bf16x2(v[q * 8 + 4], v[q * 8 + 5]);
      o[q].w = pack_bf16x2(v[q * 8 + 6], v[q * 8 + 7]);
    }
    store_padded_with_halo<CPW / 8>(a, o, n, h, w, c0);
  }
  if (a.dense_out != nullptr) {
    __nv_bfloat16* dst = a.dense_out + pix * a.cout_real + c0;
    if ((a.cout_real & 7) == 0 && c0 + CPW <= a.cout_real) {
#pragma unroll
      for (int q = 0; q < CPW / 8; ++q) {
        uint4 o;
        o.x = pack_bf16x2(v[q * 8 + 0], v[q * 8 + 1]);
        o.y = pack_bf16x2(v[q * 8 + 2], v[q * 8 + 3]);
        o.z = pack_bf16x2(v[q * 8 + 4], v[q * 8 + 5]);
        o.w = pack_bf16x2(v[q * 8 + 6], v[q * 8 + 7]);
        reinterpret_cast<uint4*>(dst)[q] = o;
      }
    } else {
#pragma unroll
      for (int j = 0; j < CPW; ++j)
        if (c0 + j < a.cout_real) dst[j] = __float2bfloat16(v[j]);
    }
  }
}

// ------------------------------------------------------------------------------------------
// Forward (B_MN = 0, weights [9][NOUT][64] = tap, cout, cin) and data gradient
// (B_MN = 1, same weight tensor read as tap, K = cout, N = cin, taps mirrored).
//
// THIN = 1: the input has at most four channels and lives in a padded buffer [NB][H+2][W+2][4].
// Nine taps x four channels are only 36 values per output pixel, so the issuing warp first gathers
// them into one K-major operand row per pixel (an im2col tile of 128 pixels x 64 values, the last
// 28 zero, 128-byte swizzled) and then issues ONE product of K = 48 instead of nine of K = 64;
// the weights are a single [64][64] tile (row = output channel, column = tap * 4 + input channel).
// Everything after the accumulator (bias, GELU, saved derivative, padded output, halo push) is shared.
// ------------------------------------------------------------------------------------------
constexpr int CV_THIN_SLOT_BYTES = 1280;           // 130 pixels x 8 bytes, rounded up
constexpr int CV_THIN_ROW_BYTES = CV_BOXW * 8;

template <int NOUT, int B_MN, int THIN = 0>
__global__ void __launch_bounds__(CV_THREADS, 1)
conv3x3_tc_kernel(const __grid_constant__ CUtensorMap tmIn, const __grid_constant__ CUtensorMap tmW,
                  const __grid_constant__ CUtensorMap tmOut, const __grid_constant__ CUtensorMap tmAux,
                  const ConvArgs a) {
  static_assert(THIN == 0 || (NOUT == 64 && B_MN == 0), "the thin-input variant writes 64 channels");
  constexpr int WTAP_BYTES = (B_MN ? 64 : NOUT) * 128;
  constexpr int W_BYTES = (THIN ? 1 : 9) * WTAP_BYTES;
  constexpr int SLOT_BYTES = THIN ? CV_THIN_SLOT_BYTES : CV_SLOT_BYTES;
  constexpr int ROW_TX_BYTES = THIN ? CV_THIN_ROW_BYTES : CV_BOXW * 128;
  constexpr uint32_t ACC_COLS = CV_MMA_WARPS * NOUT;
  constexpr uint32_t TMEM_COLS = ACC_COLS <= 32 ? 32 : (ACC_COLS <= 64 ? 64 : (ACC_COLS <= 128 ? 128 : 256));
  // Wide layers stage their output tiles in shared memory and write them with TMA stores
  // (full lines, one request per tile); they also fetch the GELU'-source tile with TMA.
  constexpr bool STAGED = (NOUT == 64);
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* w_smem = smem;
  uint8_t* slots = smem + ((W_BYTES + 1023) & ~1023);
  uint8_t* a_tiles = slots + ((CV_SLOTS * SLOT_BYTES + 1023) & ~1023);   // THIN: one im2col tile per issuing warp
  uint8_t* stage_out = a_tiles + (THIN ? CV_MMA_WARPS * CV_STAGE_BYTES : 0);   // [128 px][64 ch] padded-output tile
  uint8_t* stage_aux = stage_out + (STAGED ? CV_STAGE_BYTES : 0);  // dense output tile, or GELU'-source tile
  uint64_t* bars = reinterpret_cast<uint64_t*>(stage_aux + (STAGED ? CV_STAGE_BYTES : 0));
  uint64_t* full = bars;                  // [8]   TMA landed in window slot j
  uint64_t* empty = bars + 8;             // [8]   the (up to) three rows reading slot j are done
  uint64_t* acc_full = bars + 16;         // [CV_MMA_WARPS]
  uint64_t* acc_empty = bars + 20;        // [CV_MMA_WARPS]
  uint64_t* wbar = bars + 24;             // [1]
  uint64_t* src_full = bars + 25;         // [1]   GELU'-source tile landed
  uint64_t* src_empty = bars + 26;        // [1]   ... and has been read by every epilogue warp
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 27);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int items = a.NB * a.tiles_w * a.nstrips;
  const bool has_src = STAGED && a.gelu_src != nullptr;
  const bool aux_out = STAGED && (a.dense_pre != nullptr || a.dense_out != nullptr);

  if (threadIdx.x == 0) {
    for (int s = 0; s < 8; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 3);
    }
    for (int s = 0; s < CV_MMA_WARPS; ++s) {
      mbar_init(&acc_full[s], 1);
      mbar_init(&acc_empty[s], CV_EPI_WARPS);
    }
    mbar_init(wbar, 1);
    mbar_init(src_full, 1);
    mbar_init(src_empty, CV_EPI_WARPS);
    *abort_flag = 0;
    fence_mbar_init();
    tma_prefetch_desc(&tmIn);
    tma_prefetch_desc(&tmW);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, TMEM_COLS);
    tmem_relinquish();
  }
  if constexpr (THIN != 0) {
    // columns 36..63 of the im2col tiles are never written again: zero the tiles once
    for (int i = threadIdx.x; i < CV_MMA_WARPS * CV_STAGE_BYTES / 16; i += CV_THREADS)
      reinterpret_cast<uint4*>(a_tiles)[i] = make_uint4(0u, 0u, 0u, 0u);
    fence_proxy_async_smem();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ---------------------------------------------------------------- TMA producer
    if (lane == 0) {
      mbar_expect_tx(wbar, W_BYTES);
      for (int t = 0; t < (THIN ? 1 : 9); ++t) tma_load_2d(w_smem + t * WTAP_BYTES, &tmW, wbar, 0, t * (B_MN ? 64 : NOUT));
      halo_wait_all(a.wait, abort_flag, a.status);
      uint32_t eph = 0;   // per-slot phase bits of the empty barriers
      uint32_t sph = 0;   // phase of src_empty
      for (int item = blockIdx.x; item < items; item += gridDim.x) {
        const int s = item % a.nstrips;
        const int tw = (item / a.nstrips) % a.tiles_w;
        const int n = item / (a.nstrips * a.tiles_w);
        const int h0 = s * a.rows_per_strip;
        const int h1 = min(a.H, h0 + a.rows_per_strip);
        for (int hc = h0; hc < h1; hc += CV_CHUNK) {
          const int n_out = min(CV_CHUNK, h1 - hc);
          for (int i = 0; i < n_out; ++i) {
            if (*abort_flag) break;          // after a timeout: issue nothing more
            for (int j = (i == 0 ? 0 : i + 2); j <= i + 2; ++j) {
              mbar_wait(&empty[j], ((eph >> j) & 1u) ^ 1u, abort_flag, a.status, 10 + j);
              eph ^= (1u << j);
              mbar_expect_tx(&full[j], ROW_TX_BYTES);
              // THIN: the tensor map counts pixel PAIRS (16 bytes) along its second dimension
              tma_load_4d(slots + j * SLOT_BYTES, &tmIn, &full[j], 0, THIN ? tw * (CV_TW / 2) : tw * CV_TW, hc + j, n);
            }
            if (has_src) {
              mbar_wait(src_empty, sph ^ 1u, abort_flag, a.status, 20);
              if (*abort_flag) break;
              sph ^= 1u;
              mbar_expect_tx(src_full, CV_STAGE_BYTES);
              tma_load_4d(stage_aux, &tmAux, src_full, 0, tw * CV_TW, hc + i, n);
            }
          }
        }
      }
    }
  } else if (warp <= CV_MMA_WARPS) {
    // ---------------------------------------------------------------- UMMA issuers
    // Issuing one tcgen05.mma costs a warp on the order of a hundred cycles, three times the
    // 32 cycles a 128x64x16 MMA occupies the tensor core.  Four warps therefore issue in
    // parallel: warp m owns accumulator buffer m and every fourth output row, so no two warps
    // ever touch the same accumulator.  The whole warp runs the loop (uniform trip counts,
    // descriptors in uniform registers); one elected lane issues.
    const int mi = warp - 1;
    constexpr uint32_t idesc = make_idesc_bf16(128, NOUT, 0, B_MN);
    mbar_wait(wbar, 0, abort_flag, a.status, 1);
    uint32_t fph = 0;  // per-slot phase bits of the full barriers
    int it = 0;
    const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(mi * NOUT);
    // Descriptors of slot 0 / tap 0; every other operand is a constant byte offset away.
    const uint64_t a_desc0 = make_smem_desc_sw128(smem_u32(slots), 16, 1024);
    const uint64_t b_desc0 = B_MN ? make_smem_desc_sw128(smem_u32(w_smem), 8192, 1024)
                                  : make_smem_desc_sw128(smem_u32(w_smem), 16, 1024);
    for (int item = blockIdx.x; item < items; item += gridDim.x) {
      const int s = item % a.nstrips;
      const int h0 = s * a.rows_per_strip;
      const int h1 = min(a.H, h0 + a.rows_per_strip);
      for (int hc = h0; hc < h1; hc += CV_CHUNK) {
        const int n_out = min(CV_CHUNK, h1 - hc);
        for (int i = 0; i < n_out; ++i, ++it) {
          // Every issuing warp follows every refill of every slot, also for rows it does not
          // own: a parity wait can only tell the current phase from the previous one, so a warp
          // that skipped a refill could mistake a stale phase for the one it needs.
          for (int j = (i == 0 ? 0 : i + 2); j <= i + 2; ++j)
            mbar_wait(&full[j], (fph >> j) & 1u, abort_flag, a.status, 40 + j);
          if ((it % CV_MMA_WARPS) != mi) continue;
          const uint32_t aph = (it / CV_MMA_WARPS) & 1u;
          mbar_wait(&acc_empty[mi], aph ^ 1u, abort_flag, a.status, 30 + mi);
          if (*abort_flag) continue;         // after a timeout: issue nothing more
          tc_fence_after_sync();
          if constexpr (THIN != 0) {
            // gather the 3 x 3 x 4 inputs of 128 pixels into this warp's im2col tile (the previous product
            // that read it has completed: its accumulator has been drained), then one product of K = 48
            uint8_t* tile = a_tiles + mi * CV_STAGE_BYTES;
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              const int m = q * 32 + lane;
              uint8_t* row = tile + m * 128;
#pragma unroll
              for (int dy = 0; dy < 3; ++dy) {
                const uint8_t* src = slots + (i + dy) * SLOT_BYTES + m * 8;
#pragma unroll
                for (int dx = 0; dx < 3; ++dx) {
                  const int t = dy * 3 + dx;
                  const uint2 v = *reinterpret_cast<const uint2*>(src + dx * 8);
                  *reinterpret_cast<uint2*>(row + (((t >> 1) ^ (m & 7)) << 4) + (t & 1) * 8) = v;
                }
              }
            }
            fence_proxy_async_smem();
            __syncwarp();
            const uint64_t ad0 = make_smem_desc_sw128(smem_u32(tile), 16, 1024);
#pragma unroll
            for (int k = 0; k < 3; ++k)
              umma_f16_elect(d_tmem, desc_advance(ad0, k * 32), desc_advance(b_desc0, k * 32), idesc, k != 0 ? 1u : 0u);
            umma_commit_elect(&acc_full[mi]);
            // the window slots were read by ordinary loads: release them with plain arrivals
#pragma unroll
            for (int d = 0; d < 3; ++d) {
              const int j = i + d;
              const int lo = max(0, j - 2), hi = min(n_out - 1, j);
              if (lane == 0) {
                mbar_arrive(&empty[j]);
                if (i == lo)
                  for (int e = hi - lo + 1; e < 3; ++e) mbar_arrive(&empty[j]);
              }
            }
          } else {
          const uint64_t a_row = desc_advance(a_desc0, static_cast<uint32_t>(i * CV_SLOT_BYTES));
#pragma unroll
          for (int dy = 0; dy < 3; ++dy) {
#pragma unroll
            for (int dx = 0; dx < 3; ++dx) {
              const int wt = B_MN ? ((2 - dy) * 3 + (2 - dx)) : (dy * 3 + dx);
#pragma unroll
              for (int k = 0; k < 4; ++k) {
                const uint64_t ad = desc_advance(a_row, dy * CV_SLOT_BYTES + dx * 128 + k * 32);
                const uint64_t bd = desc_advance(b_desc0, wt * WTAP_BYTES + k * (B_MN ? 2048 : 32));
                umma_f16_elect(d_tmem, ad, bd, idesc, (dy | dx | k) != 0 ? 1u : 0u);
              }
            }
          }
          umma_commit_elect(&acc_full[mi]);
          // Release the three window slots this row read.  A slot needs three arrivals per
          // refill; near the ends of a chunk fewer rows read it, and the first reader supplies
          // the missing ones.
#pragma unroll
          for (int d = 0; d < 3; ++d) {
            const int j = i + d;
            const int lo = max(0, j - 2), hi = min(n_out - 1, j);
            umma_commit_elect(&empty[j]);
            if (i == lo && lane == 0) {
              for (int e = hi - lo + 1; e < 3; ++e) mbar_arrive(&empty[j]);
            }
          }
          }
        }
        fph ^= (1u << (n_out + 2)) - 1u;
      }
    }
  } else {
    // ---------------------------------------------------------------- epilogue (8 warps)
    // Warp e drains TMEM lane quadrant (warp % 4) and one half of the accumulator columns:
    // thread = (pixel quad * 32 + lane, CPW consecutive channels).
    const int e = warp - (1 + CV_MMA_WARPS);
    const int quad = warp & 3;
    const int half = e >> 2;
    constexpr int CPW = (NOUT >= 64) ? (NOUT * 4 / CV_EPI_WARPS) : NOUT;   // columns handled per warp
    constexpr int EPI_THREADS = 32 * CV_EPI_WARPS;
    const bool active = (half * CPW) < NOUT;
    const int c0 = half * CPW;
    const bool leader = (e == 0 && lane == 0);
    const int m = quad * 32 + lane;                     // pixel of the tile = row of the staging tiles
    int it = 0;
    uint32_t sfph = 0;                                  // phase of src_full
    float bias_r[CPW];
    load_bias_regs<CPW>(a, c0, bias_r);
    for (int item = blockIdx.x; item < items; item += gridDim.x) {
      const int s = item % a.nstrips;
      const int tw = (item / a.nstrips) % a.tiles_w;
      const int n = item / (a.nstrips * a.tiles_w);
      const int h0 = s * a.rows_per_strip;
      const int h1 = min(a.H, h0 + a.rows_per_strip);
      const int w = tw * CV_TW + m;
      for (int h = h0; h < h1; ++h, ++it) {
        const int as = it % CV_MMA_WARPS;
        const uint32_t aph = (it / CV_MMA_WARPS) & 1u;
        uint4 gsrc[CPW / 8];
        if constexpr (STAGED) {
          if (has_src) {
            // the tile of pre-activations whose GELU' multiplies this gradient tile
            mbar_wait(src_full, sfph, abort_flag, a.status, 50);
            sfph ^= 1u;
#pragma unroll
            for (int q = 0; q < CPW / 8; ++q) {
              const int chunk = (c0 / 8 + q) ^ (m & 7);
              gsrc[q] = *reinterpret_cast<const uint4*>(stage_aux + m * 128 + chunk * 16);
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(src_empty);
          }
        } else {
          if (active) prefetch_gelu_src<CPW>(a, n, h, w, c0, gsrc);
        }
        mbar_wait(&acc_full[as], aph, abort_flag, a.status, 60 + as);
        tc_fence_after_sync();
        uint32_t r[CPW];
        if (active) {
          const uint32_t taddr =
              tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + static_cast<uint32_t>(as * NOUT + c0);
          if constexpr (CPW == 32) {
            tmem_ld_32x32(taddr, r);
          } else {
            tmem_ld_32x16(taddr, r);
          }
          tmem_ld_wait();
        }
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(&acc_empty[as]);
        float v[CPW];
#pragma unroll
        for (int j = 0; j < CPW; ++j) v[j] = __uint_as_float(r[j]);
        if constexpr (!STAGED) {
          if (!active || w >= a.W) continue;
          conv_epilogue<CPW>(a, v, bias_r, gsrc, n, h, w, c0);
        } else {
          // ---- math in registers
#pragma unroll
          for (int j = 0; j < CPW; ++j) v[j] += bias_r[j];
          if (has_src) {
#pragma unroll
            for (int q = 0; q < CPW / 8; ++q) {
              const uint32_t uu[4] = {gsrc[q].x, gsrc[q].y, gsrc[q].z, gsrc[q].w};
#pragma unroll
              for (int p = 0; p < 4; ++p) {
                const __nv_bfloat162 b2 = *reinterpret_cast<const __nv_bfloat162*>(&uu[p]);
                v[q * 8 + 2 * p] *= __low2float(b2);
                v[q * 8 + 2 * p + 1] *= __high2float(b2);
              }
            }
          }
          uint4 aux_v[CPW / 8], out_v[CPW / 8];
          const bool aux_is_pre = a.dense_pre != nullptr;
          if (a.act == 1 && !aux_is_pre) {
#pragma unroll
            for (int j = 0; j < CPW; j += 2) gelu_erf_x2(v[j], v[j + 1], v[j], v[j + 1]);
          } else if (a.act == 1) {
            float d[CPW];
#pragma unroll
            for (int j = 0; j < CPW; j += 2) gelu_erf_with_grad_x2(v[j], v[j + 1], v[j], v[j + 1], d[j], d[j + 1]);
#pragma unroll
            for (int q = 0; q < CPW / 8; ++q) {
              aux_v[q].x = pack_bf16x2(d[q * 8 + 0], d[q * 8 + 1]);
              aux_v[q].y = pack_bf16x2(d[q * 8 + 2], d[q * 8 + 3]);
              aux_v[q].z = pack_bf16x2(d[q * 8 + 4], d[q * 8 + 5]);
              aux_v[q].w = pack_bf16x2(d[q * 8 + 6], d[q * 8 + 7]);
            }
          }
#pragma unroll
          for (int q = 0; q < CPW / 8; ++q) {
            out_v[q].x = pack_bf16x2(v[q * 8 + 0], v[q * 8 + 1]);
            out_v[q].y = pack_bf16x2(v[q * 8 + 2], v[q * 8 + 3]);
            out_v[q].z = pack_bf16x2(v[q * 8 + 4], v[q * 8 + 5]);
            out_v[q].w = pack_bf16x2(v[q * 8 + 6], v[q * 8 + 7]);
          }
          // ---- staging tiles: wait until the previous tile's TMA stores have read them
          if (leader) bulk_wait_read_all();
          named_barrier(1, EPI_THREADS);
#pragma unroll
          for (int q = 0; q < CPW / 8; ++q) {
            const int chunk = (c0 / 8 + q) ^ (m & 7);
            if (a.padded_out != nullptr) *reinterpret_cast<uint4*>(stage_out + m * 128 + chunk * 16) = out_v[q];
            if (aux_out) *reinterpret_cast<uint4*>(stage_aux + m * 128 + chunk * 16) = aux_is_pre ? aux_v[q] : out_v[q];
          }
          // edge pixels go straight to the neighbours' borders
          if (a.padded_out != nullptr && w < a.W) store_padded_with_halo<CPW / 8, false>(a, out_v, n, h, w, c0);
          fence_proxy_async_smem();
          named_barrier(2, EPI_THREADS);
          if (leader) {
            if (a.padded_out != nullptr) tma_store_4d(&tmOut, stage_out, 0, tw * CV_TW + 1, h + 1, n);
            if (aux_out) tma_store_4d(&tmAux, stage_aux, 0, tw * CV_TW, h, n);
            bulk_commit_group();
          }
        }
      }
    }
    if (STAGED && leader) bulk_wait_all();
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
  halo_publish(a.push, a.done_counter);
}

// ------------------------------------------------------------------------------------------
// Weight gradient:  gW[tap][ci][co] = sum over pixels of  x[p + tap][ci] * gy[p][co]
// M = 128 = two taps x 64 ci (two shifted views of the input window, MN-major),
// N = 64 co (the gy tile, MN-major), K = pixels.  Nine taps make four full pairs plus one
// tap paired with a tile of ones, whose 64 result rows are sum_p gy[p][co]: the bias
// gradient falls out of the same accumulation.  Accumulators stay in TMEM (5 x 64 columns)
// for the life of the CTA; one partial per CTA is written at the end and a second small
// kernel sums the partials in a fixed order (deterministic).
// ------------------------------------------------------------------------------------------
constexpr int WG_GSTAGES = 3;
constexpr int WG_MMA_WARPS = 5;                    // one per accumulator chain
constexpr int WG_THREADS = 32 * (1 + WG_MMA_WARPS + 4);
constexpr int WG_PARTIAL_FLOATS = 5 * 128 * 64;

struct WgradArgs {
  int NB, H, W, tiles_w, rows_per_strip, nstrips;
  float* partials;   // [gridDim.x][5][128][64] fp32 scratch
  HaloWait wait;     // the input window reads halo pixels
  int* status;
};

__global__ void __launch_bounds__(WG_THREADS, 1)
conv3x3_wgrad_kernel(const __grid_constant__ CUtensorMap tmX, const __grid_constant__ CUtensorMap tmG,
                     const WgradArgs a) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* slots = smem;
  uint8_t* gtiles = slots + WG_SLOTS * CV_SLOT_BYTES;
  uint8_t* ones = gtiles + WG_GSTAGES * 16384;
  uint64_t* bars = reinterpret_cast<uint64_t*>(ones + 2048);
  uint64_t* full = bars;              // [8]
  uint64_t* empty = bars + 8;         // [8]  3 rows x 5 issuing warps arrive per refill
  uint64_t* gfull = bars + 16;        // [3]
  uint64_t* gempty = bars + 19;       // [3]  5 issuing warps arrive
  uint64_t* acc_full = bars + 22;     // [1]  5 issuing warps arrive
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 23);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  constexpr uint32_t TMEM_COLS = 512;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int items = a.NB * a.tiles_w * a.nstrips;

  // Tile of bf16 ones (16 rows x 128 bytes); invariant under the swizzle.
  for (int i = threadIdx.x; i < 2048 / 4; i += WG_THREADS) reinterpret_cast<uint32_t*>(ones)[i] = 0x3F803F80u;
  fence_proxy_async_smem();
  if (threadIdx.x == 0) {
    for (int s = 0; s < 8; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 3 * WG_MMA_WARPS);
    }
    for (int s = 0; s < WG_GSTAGES; ++s) {
      mbar_init(&gfull[s], 1);
      mbar_init(&gempty[s], WG_MMA_WARPS);
    }
    mbar_init(acc_full, WG_MMA_WARPS);
    *abort_flag = 0;
    fence_mbar_init();
    tma_prefetch_desc(&tmX);
    tma_prefetch_desc(&tmG);
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
    // ---------------------------------------------------------------- TMA producer
    if (lane == 0) {
      halo_wait_all(a.wait, abort_flag, a.status);
      uint32_t eph = 0;
      int gs = 0;
      uint32_t gph = 0;
      for (int item = blockIdx.x; item < items; item += gridDim.x) {
        const int s = item % a.nstrips;
        const int tw = (item / a.nstrips) % a.tiles_w;
        const int n = item / (a.nstrips * a.tiles_w);
        const int h0 = s * a.rows_per_strip;
        const int h1 = min(a.H, h0 + a.rows_per_strip);
        for (int hc = h0; hc < h1; hc += WG_CHUNK) {
          const int n_out = min(WG_CHUNK, h1 - hc);
          for (int i = 0; i < n_out; ++i) {
            if (*abort_flag) break;
            for (int j = (i == 0 ? 0 : i + 2); j <= i + 2; ++j) {
              mbar_wait(&empty[j], ((eph >> j) & 1u) ^ 1u, abort_flag, a.status, 110 + j);
              eph ^= (1u << j);
              mbar_expect_tx(&full[j], CV_BOXW * 128);
              tma_load_4d(slots + j * CV_SLOT_BYTES, &tmX, &full[j], 0, tw * CV_TW, hc + j, n);
            }
            mbar_wait(&gempty[gs], gph ^ 1u, abort_flag, a.status, 120 + gs);
            if (*abort_flag) break;
            mbar_expect_tx(&gfull[gs], 16384);
            // gy lives in a padded buffer too: interior pixel (h, w) is at (h + 1, w + 1).
            tma_load_4d(gtiles + gs * 16384, &tmG, &gfull[gs], 0, tw * CV_TW + 1, hc + i + 1, n);
            if (++gs == WG_GSTAGES) {
              gs = 0;
              gph ^= 1u;
            }
          }
        }
      }
    }
  } else if (warp <= WG_MMA_WARPS) {
    // ---------------------------------------------------------------- UMMA issuers
    // One warp per accumulator chain (issue cost, not the tensor core, bounds a single
    // issuing warp).  Chain c accumulates into TMEM columns [64 c, 64 c + 64):
    //   c = 0,1,2 : taps (c,0) + (c,1)   (second 64 rows of M = the view one pixel to the right)
    //   c = 3     : taps (0,2) + (1,2)   (second half = the same view one slot further)
    //   c = 4     : tap  (2,2) + ones    (bias gradient)
    const int c = warp - 1;
    constexpr uint32_t idesc = make_idesc_bf16(128, 64, 1, 1);
    uint32_t fph = 0;
    int gs = 0;
    uint32_t gph = 0;
    bool first = true;
    const uint32_t s_addr = smem_u32(slots);
    const uint32_t ones_addr = smem_u32(ones);
    const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(64 * c);
    const uint64_t g_desc0 = make_smem_desc_sw128(smem_u32(gtiles), 8192, 1024);
    // A-operand view of this chain relative to the first slot of the row
    const uint32_t view_off = (c < 3) ? static_cast<uint32_t>(c * CV_SLOT_BYTES)
                                      : (c == 3 ? 256u : static_cast<uint32_t>(2 * CV_SLOT_BYTES + 256));
    const uint32_t pair_lbo = (c < 3) ? 128u : static_cast<uint32_t>(CV_SLOT_BYTES);
    const uint64_t a_desc0 = make_smem_desc_sw128(s_addr + view_off, pair_lbo, 1024);
    for (int item = blockIdx.x; item < items; item += gridDim.x) {
      const int s = item % a.nstrips;
      const int h0 = s * a.rows_per_strip;
      const int h1 = min(a.H, h0 + a.rows_per_strip);
      for (int hc = h0; hc < h1; hc += WG_CHUNK) {
        const int n_out = min(WG_CHUNK, h1 - hc);
        for (int i = 0; i < n_out; ++i) {
          for (int j = (i == 0 ? 0 : i + 2); j <= i + 2; ++j)
            mbar_wait(&full[j], (fph >> j) & 1u, abort_flag, a.status, 140 + j);
          mbar_wait(&gfull[gs], gph, abort_flag, a.status, 150 + gs);
          if (!*abort_flag) {
            tc_fence_after_sync();
            const uint64_t bd0 = desc_advance(g_desc0, static_cast<uint32_t>(gs * 16384));
            const uint64_t ad0 = desc_advance(a_desc0, static_cast<uint32_t>(i * CV_SLOT_BYTES));
            const uint32_t v22 = s_addr + (i + 2) * CV_SLOT_BYTES + 256;
#pragma unroll
            for (int k = 0; k < 8; ++k) {
              const uint32_t acc = (first && k == 0) ? 0u : 1u;
              const uint32_t ko = k * 2048;  // 16 pixels x 128 bytes
              const uint64_t bd = desc_advance(bd0, ko);
              // chain 4 pairs its tap with the tile of ones: the distance shrinks as k advances
              const uint64_t ad = (c == 4) ? make_smem_desc_sw128(v22 + ko, ones_addr - (v22 + ko), 1024)
                                           : desc_advance(ad0, ko);
              umma_f16_elect(d_tmem, ad, bd, idesc, acc);
            }
            first = false;
            umma_commit_elect(&gempty[gs]);
#pragma unroll
            for (int d = 0; d < 3; ++d) {
              const int j = i + d;
              const int lo = max(0, j - 2), hi = min(n_out - 1, j);
              umma_commit_elect(&empty[j]);
              if (i == lo && lane == 0) {
                for (int e = hi - lo + 1; e < 3; ++e) mbar_arrive(&empty[j]);
              }
            }
          }
          if (++gs == WG_GSTAGES) {
            gs = 0;
            gph ^= 1u;
          }
        }
        fph ^= (1u << (n_out + 2)) - 1u;
      }
    }
    umma_commit_elect(acc_full);
  } else {
    // ---------------------------------------------------------------- epilogue: one pass at the end
    const int quad = warp & 3;
    mbar_wait(acc_full, 0, abort_flag, a.status, 160);
    tc_fence_after_sync();
    float* dst = a.partials + static_cast<long long>(blockIdx.x) * WG_PARTIAL_FLOATS;
    const int m = quad * 32 + lane;
    for (int chain = 0; chain < 5; ++chain) {
      for (int c0 = 0; c0 < 64; c0 += 32) {
        uint32_t r[32];
        const uint32_t taddr =
            tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + static_cast<uint32_t>(chain * 64 + c0);
        tmem_ld_32x32(taddr, r);
        tmem_ld_wait();
        float4* o = reinterpret_cast<float4*>(dst + (chain * 128 + m) * 64 + c0);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          o[j] = make_float4(__uint_as_float(r[4 * j]), __uint_as_float(r[4 * j + 1]), __uint_as_float(r[4 * j + 2]),
                             __uint_as_float(r[4 * j + 3]));
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

// Sum the per-CTA partials in CTA order and emit the torch layouts:
//   gw[co][ci][ty][tx] (fp32) and gb[co] (fp32).
__global__ void conv3x3_wgrad_reduce_kernel(const float* __restrict__ partials, int nparts, float* __restrict__ gw,
                                            float* __restrict__ gb) {
  const int idx = blockIdx.x * blockDim.x + threadIdx.x;  // over 9*64*64 + 64
  if (idx < 9 * 64 * 64) {
    const int co = idx & 63;
    const int ci = (idx >> 6) & 63;
    const int tap = idx >> 12;
    const int dy = tap / 3, dx = tap % 3;
    int chain, halfm;
    if (dx < 2) {
      chain = dy;
      halfm = dx;
    } else if (dy < 2) {
      chain = 3;
      halfm = dy;
    } else {
      chain = 4;
      halfm = 0;
    }
    const long long off = (static_cast<long long>(chain) * 128 + halfm * 64 + ci) * 64 + co;
    float s = 0.f;
    for (int p = 0; p < nparts; ++p) s += partials[static_cast<long long>(p) * WG_PARTIAL_FLOATS + off];
    gw[((co * 64 + ci) * 3 + dy) * 3 + dx] = s;
  } else if (idx < 9 * 64 * 64 + 64) {
    const int co = idx - 9 * 64 * 64;
    const long long off = (static_cast<long long>(4) * 128 + 64) * 64 + co;
    float s = 0.f;
    for (int p = 0; p < nparts; ++p) s += partials[static_cast<long long>(p) * WG_PARTIAL_FLOATS + off];
    if (gb != nullptr) gb[co] = s;
  }
}

// ------------------------------------------------------------------------------------------
// Weight gradient of a layer with at most four channels on one side (first / last layer of a network).
//   R[m][tap * 4 + c] = sum over this rank's pixels q of  big[q][m] * small[q + (ty - 1, tx - 1)][c]
// big:   padded [NB][H+2][W+2][64] buffer, interior pixels only (no halo needed);
// small: padded [NB][H+2][W+2][4] buffer read with its halo (a three-row window per output row).
// The issuing warp gathers the 36 shifted values of 128 pixels into an im2col tile (column 36 = 1, so
// that R[m][36] = sum_q big[q][m]) and multiplies: A = the big tile read MN-major (M = 64 channels, the
// upper 64 rows of M = a tile of ones, so that R[64][n] = sum_q im2col[q][n]), B = the im2col tile read
// MN-major (N = 64), K = 128 pixels per tile.  Each of the four issuing warps owns every fourth tile and
// its own accumulator; the epilogue adds the four and writes one partial per CTA, summed in CTA order by
// conv3x3_wgrad_thin_reduce_kernel into the torch layouts:
//   side 0 (thin input,  big = gradient of the output, small = input):   gw[m][c][ty][tx] = R[m][t * 4 + c],       gb[m] = R[m][36]
//   side 1 (thin output, big = input, small = gradient of the output):   gw[c][m][ty][tx] = R[m][(8 - t) * 4 + c], gb[c] = R[64][16 + c]
// (side 1 sums over the pixels of the INPUT this rank owns, pairing each with output-gradient pixels that may
// belong to a neighbour: over all ranks every pair is counted once, which is what the summed gradient needs).
// ------------------------------------------------------------------------------------------
constexpr int WT_WARPS = CV_MMA_WARPS;             // issuing warps = big-tile stages = im2col tiles
constexpr int WT_THREADS = 32 * (1 + WT_WARPS + 4);
constexpr int WT_PARTIAL_FLOATS = 128 * 64;

struct WgradThinArgs {
  int NB, H, W, tiles_w, rows_per_strip, nstrips;
  float* partials;   // [gridDim.x][128][64]
  HaloWait wait;     // the small buffer is read with its halo
  int* status;
};

__global__ void __launch_bounds__(WT_THREADS, 1)
conv3x3_wgrad_thin_kernel(const __grid_constant__ CUtensorMap tmBig, const __grid_constant__ CUtensorMap tmSmall,
                          const WgradThinArgs a) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* big = smem;                                            // WT_WARPS stages of [128 px][64 ch]
  uint8_t* im2col = big + WT_WARPS * CV_STAGE_BYTES;              // WT_WARPS tiles of [128 px][64 values]
  uint8_t* ones = im2col + WT_WARPS * CV_STAGE_BYTES;             // 2 KB
  uint8_t* slots = ones + 2048;                                   // CV_SLOTS rows of the small buffer
  uint64_t* bars = reinterpret_cast<uint64_t*>(slots + ((CV_SLOTS * CV_THIN_SLOT_BYTES + 1023) & ~1023));
  uint64_t* full = bars;              // [8]
  uint64_t* empty = bars + 8;         // [8]
  uint64_t* gfull = bars + 16;        // [WT_WARPS]
  uint64_t* gempty = bars + 20;       // [WT_WARPS]
  uint64_t* acc_full = bars + 24;     // [1]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 25);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  constexpr uint32_t TMEM_COLS = 256;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int items = a.NB * a.tiles_w * a.nstrips;

  for (int i = threadIdx.x; i < 2048 / 4; i += WT_THREADS) reinterpret_cast<uint32_t*>(ones)[i] = 0x3F803F80u;
  // im2col tiles: zero, then the constant column 36 = 1.0 (16-byte chunk 4, second half, first value)
  for (int i = threadIdx.x; i < WT_WARPS * CV_STAGE_BYTES / 16; i += WT_THREADS)
    reinterpret_cast<uint4*>(im2col)[i] = make_uint4(0u, 0u, 0u, 0u);
  __syncthreads();
  for (int r = threadIdx.x; r < WT_WARPS * 128; r += WT_THREADS) {
    const int m = r & 127;
    uint8_t* row = im2col + (r >> 7) * CV_STAGE_BYTES + m * 128;
    *reinterpret_cast<uint16_t*>(row + ((4 ^ (m & 7)) << 4) + 8) = 0x3F80;
  }
  fence_proxy_async_smem();
  if (threadIdx.x == 0) {
    for (int s = 0; s < 8; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 3);
    }
    for (int s = 0; s < WT_WARPS; ++s) {
      mbar_init(&gfull[s], 1);
      mbar_init(&gempty[s], 1);
    }
    mbar_init(acc_full, WT_WARPS);
    *abort_flag = 0;
    fence_mbar_init();
    tma_prefetch_desc(&tmBig);
    tma_prefetch_desc(&tmSmall);
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
    // ---------------------------------------------------------------- TMA producer
    if (lane == 0) {
      halo_wait_all(a.wait, abort_flag, a.status);
      uint32_t eph = 0;
      int it = 0;
      for (int item = blockIdx.x; item < items; item += gridDim.x) {
        const int s = item % a.nstrips;
        const int tw = (item / a.nstrips) % a.tiles_w;
        const int n = item / (a.nstrips * a.tiles_w);
        const int h0 = s * a.rows_per_strip;
        const int h1 = min(a.H, h0 + a.rows_per_strip);
        for (int hc = h0; hc < h1; hc += CV_CHUNK) {
          const int n_out = min(CV_CHUNK, h1 - hc);
          for (int i = 0; i < n_out; ++i, ++it) {
            if (*abort_flag) break;
            for (int j = (i == 0 ? 0 : i + 2); j <= i + 2; ++j) {
              mbar_wait(&empty[j], ((eph >> j) & 1u) ^ 1u, abort_flag, a.status, 210 + j);
              eph ^= (1u << j);
              mbar_expect_tx(&full[j], CV_THIN_ROW_BYTES);
              tma_load_4d(slots + j * CV_THIN_SLOT_BYTES, &tmSmall, &full[j], 0, tw * (CV_TW / 2), hc + j, n);
            }
            const int gs = it % WT_WARPS;
            mbar_wait(&gempty[gs], (static_cast<uint32_t>(it / WT_WARPS) & 1u) ^ 1u, abort_flag, a.status, 220 + gs);
            if (*abort_flag) break;
            mbar_expect_tx(&gfull[gs], CV_STAGE_BYTES);
            // interior pixel (h, w) of the big buffer sits at (h + 1, w + 1)
            tma_load_4d(big + gs * CV_STAGE_BYTES, &tmBig, &gfull[gs], 0, tw * CV_TW + 1, hc + i + 1, n);
          }
        }
      }
    }
  } else if (warp <= WT_WARPS) {
    // ---------------------------------------------------------------- gather + UMMA issue (warp mi owns tile it % 4 == mi)
    const int mi = warp - 1;
    constexpr uint32_t idesc = make_idesc_bf16(128, 64, 1, 1);
    uint32_t fph = 0;
    int it = 0;
    bool first = true;
    const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(64 * mi);
    uint8_t* tile = im2col + mi * CV_STAGE_BYTES;
    const uint32_t big_addr = smem_u32(big + mi * CV_STAGE_BYTES);
    const uint32_t ones_addr = smem_u32(ones);
    const uint64_t b_desc0 = make_smem_desc_sw128(smem_u32(tile), 8192, 1024);
    for (int item = blockIdx.x; item < items; item += gridDim.x) {
      const int s = item % a.nstrips;
      const int h0 = s * a.rows_per_strip;
      const int h1 = min(a.H, h0 + a.rows_per_strip);
      for (int hc = h0; hc < h1; hc += CV_CHUNK) {
        const int n_out = min(CV_CHUNK, h1 - hc);
        for (int i = 0; i < n_out; ++i, ++it) {
          for (int j = (i == 0 ? 0 : i + 2); j <= i + 2; ++j)
            mbar_wait(&full[j], (fph >> j) & 1u, abort_flag, a.status, 240 + j);
          if ((it % WT_WARPS) != mi) continue;
          const uint32_t gph = static_cast<uint32_t>(it / WT_WARPS) & 1u;
          // the previous product of this warp (which read this im2col tile) has completed when its stage was
          // released: the producer refilled the stage only after that commit
          mbar_wait(&gfull[mi], gph, abort_flag, a.status, 250 + mi);
          if (*abort_flag) continue;
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            const int m = q * 32 + lane;
            uint8_t* row = tile + m * 128;
#pragma unroll
            for (int dy = 0; dy < 3; ++dy) {
              const uint8_t* src = slots + (i + dy) * CV_THIN_SLOT_BYTES + m * 8;
#pragma unroll
              for (int dx = 0; dx < 3; ++dx) {
                const int t = dy * 3 + dx;
                const uint2 v = *reinterpret_cast<const uint2*>(src + dx * 8);
                *reinterpret_cast<uint2*>(row + (((t >> 1) ^ (m & 7)) << 4) + (t & 1) * 8) = v;
              }
            }
          }
          fence_proxy_async_smem();
          __syncwarp();
          tc_fence_after_sync();
#pragma unroll
          for (int k = 0; k < 8; ++k) {
            const uint32_t ko = k * 2048;  // 16 pixels x 128 bytes
            const uint64_t ad = make_smem_desc_sw128(big_addr + ko, ones_addr - (big_addr + ko), 1024);
            umma_f16_elect(d_tmem, ad, desc_advance(b_desc0, ko), idesc, (first && k == 0) ? 0u : 1u);
          }
          first = false;
          umma_commit_elect(&gempty[mi]);
#pragma unroll
          for (int d = 0; d < 3; ++d) {
            const int j = i + d;
            const int lo = max(0, j - 2), hi = min(n_out - 1, j);
            if (lane == 0) {
              mbar_arrive(&empty[j]);
              if (i == lo)
                for (int e = hi - lo + 1; e < 3; ++e) mbar_arrive(&empty[j]);
            }
          }
        }
        fph ^= (1u << (n_out + 2)) - 1u;
      }
    }
    umma_commit_elect(acc_full);
  } else {
    // ---------------------------------------------------------------- epilogue: add the four accumulators, one partial per CTA
    const int quad = warp & 3;
    mbar_wait(acc_full, 0, abort_flag, a.status, 260);
    tc_fence_after_sync();
    float* dst = a.partials + static_cast<long long>(blockIdx.x) * WT_PARTIAL_FLOATS;
    const int m = quad * 32 + lane;
    // which issuing warps produced anything (a grid with fewer tiles than warps leaves some accumulators unwritten)
    int used = 0;
    {
      int total = 0;
      for (int item = blockIdx.x; item < items; item += gridDim.x) {
        const int s = item % a.nstrips;
        const int h0 = s * a.rows_per_strip;
        total += min(a.H, h0 + a.rows_per_strip) - h0;
      }
      used = total < WT_WARPS ? total : WT_WARPS;
    }
    for (int c0 = 0; c0 < 64; c0 += 32) {
      float acc[32];
#pragma unroll
      for (int j = 0; j < 32; ++j) acc[j] = 0.f;
      for (int w = 0; w < used; ++w) {
        uint32_t r[32];
        tmem_ld_32x32(tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + static_cast<uint32_t>(w * 64 + c0), r);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 32; ++j) acc[j] += __uint_as_float(r[j]);
      }
      float4* o = reinterpret_cast<float4*>(dst + m * 64 + c0);
#pragma unroll
      for (int j = 0; j < 8; ++j) o[j] = make_float4(acc[4 * j], acc[4 * j + 1], acc[4 * j + 2], acc[4 * j + 3]);
    }
  }

  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// Sum the per-CTA partials of conv3x3_wgrad_thin_kernel in CTA order and emit the torch layouts
// (see the kernel's comment): side 0: gw [64][cs][3][3], gb [64]; side 1: gw [cs][64][3][3], gb [cs].
__global__ void conv3x3_wgrad_thin_reduce_kernel(const float* __restrict__ partials, int nparts, int side, int cs,
                                                 float* __restrict__ gw, float* __restrict__ gb) {
  const int idx = blockIdx.x * blockDim.x + threadIdx.x;
  const int nw = 64 * cs * 9;
  const int nb = side == 0 ? 64 : cs;
  int row, col;
  float* out;
  if (idx < nw) {
    int m, c, t;
    if (side == 0) {          // idx = ((m * cs + c) * 9 + t)
      t = idx % 9; c = (idx / 9) % cs; m = idx / (9 * cs);
      col = t * 4 + c;
    } else {                  // idx = ((c * 64 + m) * 9 + t)
      t = idx % 9; m = (idx / 9) % 64; c = idx / (9 * 64);
      col = (8 - t) * 4 + c;
    }
    row = m;
    out = gw + idx;
  } else if (idx < nw + nb) {
    const int j = idx - nw;
    if (gb == nullptr) return;
    if (side == 0) { row = j; col = 36; } else { row = 64; col = 16 + j; }
    out = gb + j;
  } else {
    return;
  }
  float s = 0.f;
  for (int p = 0; p < nparts; ++p) s += partials[static_cast<long long>(p) * WT_PARTIAL_FLOATS + row * 64 + col];
  *out = s;
}

static int padded_tmap(CUtensorMap* tm, const void* base, int NB, int H, int W, int boxw, int shrink_w) {
  // dims (C, W + 2 - shrink_w, H + 2, NB); strides of the full padded buffer.
  uint64_t dims[4] = {64, static_cast<uint64_t>(W + 2 - shrink_w), static_cast<uint64_t>(H + 2),
                      static_cast<uint64_t>(NB)};
  uint64_t strides[3] = {128, static_cast<uint64_t>(W + 2) * 128, static_cast<uint64_t>(H + 2) * (W + 2) * 128};
  uint32_t box[4] = {64, static_cast<uint32_t>(boxw), 1, 1};
  return make_tmap_bf16(tm, base, 4, dims, strides, box);
}

static void choose_strips(int H, int NB, int tiles_w, int sm_count, int chunk, int* rows_per_strip, int* nstrips) {
  // Strips of a multiple of `chunk` rows; aim for >= 8 work items per CTA when the tile allows it.
  int rps = 8 * chunk;
  while (rps > chunk && static_cast<long long>(NB) * tiles_w * ((H + rps - 1) / rps) < 8LL * sm_count) rps -= chunk;
  if (rps > H) rps = ((H + chunk - 1) / chunk) * chunk;
  *rows_per_strip = rps;
  *nstrips = (H + rps - 1) / rps;
}

}  // namespace jb

using namespace jb;

struct JbHalo {          // C mirror passed from Python (ctypes)
  void* push_buf[9];
  void* push_flag[9];
  void* wait_flag[9];
  unsigned int push_epoch;
  unsigned int wait_epoch;
  unsigned int push_enabled;
  unsigned int wait_enabled;
  unsigned int push_stride;      // CUDA-graph replays: see live_epoch()
  unsigned int wait_stride;
  const unsigned int* replay;    // null outside a graph
};

// Forward / data-gradient launcher.
//  in_padded : [NB][H+2][W+2][64] bf16 (halo filled)        weights : [9][nout_pad][64] bf16
//  mode 0 = forward (weights tap,cout,cin; nout_pad in {16, 64}); mode 1 = data gradient (nout_pad = 64).
extern "C" int jb_conv3x3_c64(const void* in_padded, const void* weights, const float* bias, const void* gelu_src,
                              void* dense_pre, void* padded_out, void* dense_out, int NB, int H, int W,
                              int nout_pad, int cout_real, int act, int mode, const JbHalo* halo,
                              unsigned int* done_counter, int* status, int sm_count, void* stream) {
  if (nout_pad != 64 && nout_pad != 16) return -1;
  if (mode == 1 && nout_pad != 64) return -1;
  if (dense_pre != nullptr && act != 1) return -1;   // the saved tensor is the activation's derivative
  CUtensorMap tmIn, tmW;
  if (padded_tmap(&tmIn, in_padded, NB, H, W, CV_BOXW, 0) != 0) return -2;
  {
    uint64_t dims[2] = {64, static_cast<uint64_t>(9 * nout_pad)};
    uint64_t strides[1] = {128};
    uint32_t box[2] = {64, static_cast<uint32_t>(mode == 1 ? 64 : nout_pad)};
    if (make_tmap_bf16(&tmW, weights, 2, dims, strides, box) != 0) return -2;
  }
  ConvArgs a{};
  a.NB = NB; a.H = H; a.W = W;
  a.tiles_w = (W + CV_TW - 1) / CV_TW;
  choose_strips(H, NB, a.tiles_w, sm_count, CV_CHUNK, &a.rows_per_strip, &a.nstrips);
  a.cout_real = cout_real;
  a.bias = bias;
  a.gelu_src = static_cast<const __nv_bfloat16*>(gelu_src);
  a.dense_pre = static_cast<__nv_bfloat16*>(dense_pre);
  a.act = act;
  a.padded_out = static_cast<__nv_bfloat16*>(padded_out);
  a.dense_out = static_cast<__nv_bfloat16*>(dense_out);
  a.done_counter = done_counter;
  a.status = status;
  if (halo != nullptr) {
    for (int d = 0; d < 9; ++d) {
      a.push.buf[d] = halo->push_buf[d];
      a.push.flag[d] = static_cast<uint32_t*>(halo->push_flag[d]);
      a.wait.flag[d] = static_cast<const uint32_t*>(halo->wait_flag[d]);
    }
    a.push.epoch = halo->push_epoch;
    a.push.enabled = halo->push_enabled;
    a.push.stride = halo->push_stride;
    a.push.replay = halo->replay;
    a.wait.epoch = halo->wait_epoch;
    a.wait.enabled = halo->wait_enabled;
    a.wait.stride = halo->wait_stride;
    a.wait.replay = halo->replay;
  }
  // Output / auxiliary tensor maps of the staged (64-column) kernels.
  CUtensorMap tmOut = tmIn, tmAux = tmIn;
  if (nout_pad == 64) {
    const void* aux = gelu_src ? gelu_src : (dense_pre ? static_cast<const void*>(dense_pre) : static_cast<const void*>(dense_out));
    const int n_aux = (gelu_src != nullptr) + (dense_pre != nullptr) + (dense_out != nullptr);
    if (n_aux > 1 || (dense_out != nullptr && cout_real != 64)) return -1;
    // hide the right border column so that a partial last tile never writes into the halo
    if (padded_out != nullptr && padded_tmap(&tmOut, padded_out, NB, H, W, CV_TW, 1) != 0) return -2;
    if (aux != nullptr) {
      uint64_t dims[4] = {64, static_cast<uint64_t>(W), static_cast<uint64_t>(H), static_cast<uint64_t>(NB)};
      uint64_t strides[3] = {128, static_cast<uint64_t>(W) * 128, static_cast<uint64_t>(H) * W * 128};
      uint32_t box[4] = {64, CV_TW, 1, 1};
      if (make_tmap_bf16(&tmAux, aux, 4, dims, strides, box) != 0) return -2;
    }
  }
  const int items = NB * a.tiles_w * a.nstrips;
  const int grid = items < sm_count ? items : sm_count;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  constexpr int SMEM64 = 9 * 8192 + CV_SLOTS * CV_SLOT_BYTES + 2 * CV_STAGE_BYTES + 512 + 1024;
  constexpr int SMEM16 = ((9 * 2048 + 1023) & ~1023) + CV_SLOTS * CV_SLOT_BYTES + 512 + 1024;
  cudaError_t e;
  if (mode == 1) {
    auto k = conv3x3_tc_kernel<64, 1>;
    e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM64);
    if (e != cudaSuccess) return -3;
    k<<<grid, CV_THREADS, SMEM64, st>>>(tmIn, tmW, tmOut, tmAux, a);
  } else if (nout_pad == 64) {
    auto k = conv3x3_tc_kernel<64, 0>;
    e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM64);
    if (e != cudaSuccess) return -3;
    k<<<grid, CV_THREADS, SMEM64, st>>>(tmIn, tmW, tmOut, tmAux, a);
  } else {
    auto k = conv3x3_tc_kernel<16, 0>;
    e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM16);
    if (e != cudaSuccess) return -3;
    k<<<grid, CV_THREADS, SMEM16, st>>>(tmIn, tmW, tmOut, tmAux, a);
  }
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

// Thin-input convolution: in_padded4 is [NB][H+2][W+2][4] bf16 (halo filled; W even), weights a single
// [64][64] bf16 tile whose row n holds output channel n and whose column tap * 4 + c the weight of input
// channel c at tap (ty, tx) = (tap / 3, tap % 3), i.e. out[p][n] = sum in[p + (ty - 1, tx - 1)][c] w[n][tap * 4 + c];
// columns 36..63 are ignored.  Used for the first layer of a network (forward) and, with mirrored taps, for
// the data gradient of a last layer with at most four output channels.  The epilogue arguments are those of
// jb_conv3x3_c64 with 64 output channels.
extern "C" int jb_conv3x3_thin_in(const void* in_padded4, const void* weights, const float* bias, const void* gelu_src,
                                  void* dense_pre, void* padded_out, void* dense_out, int NB, int H, int W, int act,
                                  const JbHalo* halo, unsigned int* done_counter, int* status, int sm_count, void* stream) {
  if (W & 1) return -1;
  if (dense_pre != nullptr && act != 1) return -1;
  CUtensorMap tmIn, tmW;
  {
    // pixel pairs as the innermost 16-byte unit: (8 values, (W + 2) / 2 pairs, H + 2 rows, NB images)
    uint64_t dims[4] = {8, static_cast<uint64_t>((W + 2) / 2), static_cast<uint64_t>(H + 2), static_cast<uint64_t>(NB)};
    uint64_t strides[3] = {16, static_cast<uint64_t>(W + 2) * 8, static_cast<uint64_t>(H + 2) * (W + 2) * 8};
    uint32_t box[4] = {8, CV_BOXW / 2, 1, 1};
    if (make_tmap_bf16(&tmIn, in_padded4, 4, dims, strides, box, false) != 0) return -2;
  }
  {
    uint64_t dims[2] = {64, 64};
    uint64_t strides[1] = {128};
    uint32_t box[2] = {64, 64};
    if (make_tmap_bf16(&tmW, weights, 2, dims, strides, box) != 0) return -2;
  }
  ConvArgs a{};
  a.NB = NB; a.H = H; a.W = W;
  a.tiles_w = (W + CV_TW - 1) / CV_TW;
  choose_strips(H, NB, a.tiles_w, sm_count, CV_CHUNK, &a.rows_per_strip, &a.nstrips);
  a.cout_real = 64;
  a.bias = bias;
  a.gelu_src = static_cast<const __nv_bfloat16*>(gelu_src);
  a.dense_pre = static_cast<__nv_bfloat16*>(dense_pre);
  a.act = act;
  a.padded_out = static_cast<__nv_bfloat16*>(padded_out);
  a.dense_out = static_cast<__nv_bfloat16*>(dense_out);
  a.done_counter = done_counter;
  a.status = status;
  if (halo != nullptr) {
    for (int d = 0; d < 9; ++d) {
      a.push.buf[d] = halo->push_buf[d];
      a.push.flag[d] = static_cast<uint32_t*>(halo->push_flag[d]);
      a.wait.flag[d] = static_cast<const uint32_t*>(halo->wait_flag[d]);
    }
    a.push.epoch = halo->push_epoch;
    a.push.enabled = halo->push_enabled;
    a.push.stride = halo->push_stride;
    a.push.replay = halo->replay;
    a.wait.epoch = halo->wait_epoch;
    a.wait.enabled = halo->wait_enabled;
    a.wait.stride = halo->wait_stride;
    a.wait.replay = halo->replay;
  }
  CUtensorMap tmOut = tmW, tmAux = tmW;
  const void* aux = gelu_src ? gelu_src : (dense_pre ? static_cast<const void*>(dense_pre) : static_cast<const void*>(dense_out));
  const int n_aux = (gelu_src != nullptr) + (dense_pre != nullptr) + (dense_out != nullptr);
  if (n_aux > 1) return -1;
  if (padded_out != nullptr && padded_tmap(&tmOut, padded_out, NB, H, W, CV_TW, 1) != 0) return -2;
  if (aux != nullptr) {
    uint64_t dims[4] = {64, static_cast<uint64_t>(W), static_cast<uint64_t>(H), static_cast<uint64_t>(NB)};
    uint64_t strides[3] = {128, static_cast<uint64_t>(W) * 128, static_cast<uint64_t>(H) * W * 128};
    uint32_t box[4] = {64, CV_TW, 1, 1};
    if (make_tmap_bf16(&tmAux, aux, 4, dims, strides, box) != 0) return -2;
  }
  const int items = NB * a.tiles_w * a.nstrips;
  const int grid = items < sm_count ? items : sm_count;
  constexpr int SMEM = 8192 + ((CV_SLOTS * CV_THIN_SLOT_BYTES + 1023) & ~1023) + CV_MMA_WARPS * CV_STAGE_BYTES +
                       2 * CV_STAGE_BYTES + 512 + 1024;
  auto k = conv3x3_tc_kernel<64, 0, 1>;
  if (cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM) != cudaSuccess) return -3;
  k<<<grid, CV_THREADS, SMEM, static_cast<cudaStream_t>(stream)>>>(tmIn, tmW, tmOut, tmAux, a);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

// Number of fp32 scratch elements jb_conv3x3_wgrad_thin needs for a given SM count.
extern "C" long long jb_conv3x3_wgrad_thin_scratch_floats(int sm_count) {
  return static_cast<long long>(sm_count) * WT_PARTIAL_FLOATS;
}

// Weight (and bias) gradient of a layer with at most four channels on one side.
//  big_padded  : [NB][H+2][W+2][64] bf16; its interior pixels are read
//  small_padded: [NB][H+2][W+2][4] bf16 (halo filled; W even)
//  side 0: the layer has `cs` input channels (small = layer input, big = gradient of its output):
//          gw [64][cs][3][3], gb [64]
//  side 1: the layer has `cs` output channels (small = gradient of its output, big = layer input):
//          gw [cs][64][3][3], gb [cs]
//  scratch: jb_conv3x3_wgrad_thin_scratch_floats(sm_count) floats.  gb may be null.
extern "C" int jb_conv3x3_wgrad_thin(const void* big_padded, const void* small_padded, float* gw, float* gb,
                                     float* scratch, int NB, int H, int W, int side, int cs, const JbHalo* halo,
                                     int* status, int sm_count, void* stream) {
  if ((W & 1) || cs < 1 || cs > 4 || (side != 0 && side != 1)) return -1;
  CUtensorMap tmBig, tmSmall;
  // hide the right border column of the big buffer so that pixels beyond W read as zero
  if (padded_tmap(&tmBig, big_padded, NB, H, W, CV_TW, 1) != 0) return -2;
  {
    uint64_t dims[4] = {8, static_cast<uint64_t>((W + 2) / 2), static_cast<uint64_t>(H + 2), static_cast<uint64_t>(NB)};
    uint64_t strides[3] = {16, static_cast<uint64_t>(W + 2) * 8, static_cast<uint64_t>(H + 2) * (W + 2) * 8};
    uint32_t box[4] = {8, CV_BOXW / 2, 1, 1};
    if (make_tmap_bf16(&tmSmall, small_padded, 4, dims, strides, box, false) != 0) return -2;
  }
  WgradThinArgs a{};
  a.NB = NB; a.H = H; a.W = W;
  a.tiles_w = (W + CV_TW - 1) / CV_TW;
  choose_strips(H, NB, a.tiles_w, sm_count, CV_CHUNK, &a.rows_per_strip, &a.nstrips);
  a.partials = scratch;
  a.status = status;
  if (halo != nullptr) {
    for (int d = 0; d < 9; ++d) a.wait.flag[d] = static_cast<const uint32_t*>(halo->wait_flag[d]);
    a.wait.epoch = halo->wait_epoch;
    a.wait.enabled = halo->wait_enabled;
    a.wait.stride = halo->wait_stride;
    a.wait.replay = halo->replay;
  }
  const int items = NB * a.tiles_w * a.nstrips;
  const int grid = items < sm_count ? items : sm_count;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  constexpr int SMEM = 2 * WT_WARPS * CV_STAGE_BYTES + 2048 + ((CV_SLOTS * CV_THIN_SLOT_BYTES + 1023) & ~1023) + 512 + 1024;
  if (cudaFuncSetAttribute(conv3x3_wgrad_thin_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM) != cudaSuccess)
    return -3;
  conv3x3_wgrad_thin_kernel<<<grid, WT_THREADS, SMEM, st>>>(tmBig, tmSmall, a);
  if (cudaGetLastError() != cudaSuccess) return -4;
  const int n = 64 * cs * 9 + (side == 0 ? 64 : cs);
  conv3x3_wgrad_thin_reduce_kernel<<<(n + 255) / 256, 256, 0, st>>>(scratch, grid, side, cs, gw, gb);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

// Number of fp32 scratch elements jb_conv3x3_c64_wgrad needs for a given SM count.
extern "C" long long jb_conv3x3_wgrad_scratch_floats(int sm_count) {
  return static_cast<long long>(sm_count) * WG_PARTIAL_FLOATS;
}

// Weight (and bias) gradient.  x_padded: [NB][H+2][W+2][64] input of the layer (halo filled),
// gy_padded: [NB][H+2][W+2][64] gradient of the layer output (interior used), gw: [64][64][3][3] fp32,
// gb: [64] fp32 or null, scratch: jb_conv3x3_wgrad_scratch_floats(sm_count) floats.
extern "C" int jb_conv3x3_c64_wgrad(const void* x_padded, const void* gy_padded, float* gw, float* gb,
                                    float* scratch, int NB, int H, int W, const JbHalo* halo, int* status,
                                    int sm_count, void* stream) {
  CUtensorMap tmX, tmG;
  if (padded_tmap(&tmX, x_padded, NB, H, W, CV_BOXW, 0) != 0) return -2;
  // Hide the right border column of gy so that pixels beyond W read as zero.
  if (padded_tmap(&tmG, gy_padded, NB, H, W, CV_TW, 1) != 0) return -2;
  WgradArgs a{};
  a.NB = NB; a.H = H; a.W = W;
  a.tiles_w = (W + CV_TW - 1) / CV_TW;
  choose_strips(H, NB, a.tiles_w, sm_count, WG_CHUNK, &a.rows_per_strip, &a.nstrips);
  a.partials = scratch;
  a.status = status;
  if (halo != nullptr) {
    for (int d = 0; d < 9; ++d) a.wait.flag[d] = static_cast<const uint32_t*>(halo->wait_flag[d]);
    a.wait.epoch = halo->wait_epoch;
    a.wait.enabled = halo->wait_enabled;
    a.wait.stride = halo->wait_stride;
    a.wait.replay = halo->replay;
  }
  const int items = NB * a.tiles_w * a.nstrips;
  const int grid = items < sm_count ? items : sm_count;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  constexpr int SMEM = WG_SLOTS * CV_SLOT_BYTES + WG_GSTAGES * 16384 + 2048 + 256 + 1024;
  if (cudaFuncSetAttribute(conv3x3_wgrad_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM) != cudaSuccess)
    return -3;
  conv3x3_wgrad_kernel<<<grid, WG_THREADS, SMEM, st>>>(tmX, tmG, a);
  if (cudaGetLastError() != cudaSuccess) return -4;
  const int n = 9 * 64 * 64 + 64;
  conv3x3_wgrad_reduce_kernel<<<(n + 255) / 256, 256, 0, st>>>(scratch, grid, gw, gb);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}
