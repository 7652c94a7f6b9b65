// Getting data into the padded halo layout:
//   halo_pack : any strided (N, C, H, W) fp32 / bf16 tensor -> padded NHWC bf16 buffer [NB][H+2][W+2][CP]
//               (channels zero-filled up to CW <= CP) with the edge pixels stored straight into the
//               neighbours' borders over NVLink.  CP = 64 feeds the 64-channel kernels, CP = 4 the
//               thin-channel kernels of conv3x3.cu (first / last layer of a network).
//
// Capability parity: the first / last layers of the reference CNN run through the same
// F.conv2d + halo exchange as every other layer (jigsaw/modules/convolution/_conv/base.py:628-688).

#include "ptx.cuh"

namespace jb {

struct PackArgs {
  const void* src;
  int src_is_fp32;
  long long sn, sc, sh, sw;   // element strides of the source
  int NB, C, H, W;            // logical shape
  int CP;                     // channels (pixel stride) of the padded buffer, multiple of 4
  int CW;                     // channels actually written (>= C, multiple of 4, <= CP); the rest of a
                              // pixel is left as it is (callers keep such buffers zero there)
  __nv_bfloat16* dst;         // [NB][H+2][W+2][CP]
  HaloPush push;
  unsigned int* done_counter;
};

// One thread per pixel, PACK_PIX pixels of one row per thread, channels in groups of four.  For a
// pixel-contiguous source (NCHW) the reads of a warp are coalesced per channel; for a
// channel-contiguous source (NHWC) each thread reads its pixel's channels from one short run.
// Only blocks that stored into a neighbour's memory pay for a system-scope fence.
constexpr int PACK_THREADS = 256;
constexpr int PACK_PIX = 4;

__global__ void __launch_bounds__(PACK_THREADS) halo_pack_kernel(const PackArgs a) {
  const int h = blockIdx.y, n = blockIdx.z;
  const int tid = threadIdx.x;
  const long long prow = static_cast<long long>(a.W + 2) * a.CP;
  const long long pimg = static_cast<long long>(a.H + 2) * prow;
  const int groups = a.CW / 4;  // 4 channels = 8 bytes per store
  const bool top = (h == 0), bot = (h == a.H - 1);
  bool pushed = false;
  const long long src_row = n * a.sn + h * a.sh;
#pragma unroll
  for (int k = 0; k < PACK_PIX; ++k) {
    const int w = (blockIdx.x * PACK_PIX + k) * PACK_THREADS + tid;
    if (w >= a.W) continue;
    const long long src_pix = src_row + static_cast<long long>(w) * a.sw;
    __nv_bfloat16* out_pix = a.dst + n * pimg + (h + 1) * prow + static_cast<long long>(w + 1) * a.CP;
    const bool lef = (w == 0), rig = (w == a.W - 1);
    const bool edge = a.push.enabled && (top || bot || lef || rig);
    for (int g = 0; g < groups; ++g) {
      float v[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int c = g * 4 + j;
        v[j] = 0.f;
        if (c < a.C) {
          const long long off = src_pix + c * a.sc;
          v[j] = a.src_is_fp32 ? static_cast<const float*>(a.src)[off]
                               : __bfloat162float(static_cast<const __nv_bfloat16*>(a.src)[off]);
        }
      }
      uint2 o;
      o.x = pack_bf16x2(v[0], v[1]);
      o.y = pack_bf16x2(v[2], v[3]);
      *reinterpret_cast<uint2*>(out_pix + g * 4) = o;
      if (!edge) continue;
      for (int sy = -1; sy <= 1; ++sy) {
        for (int sx = -1; sx <= 1; ++sx) {
          if (sy == 0 && sx == 0) continue;
          const int d = (sy + 1) * 3 + (sx + 1);
          if (a.push.buf[d] == nullptr) continue;
          const bool hit_y = (sy == -1) ? top : (sy == 1 ? bot : true);
          const bool hit_x = (sx == -1) ? lef : (sx == 1 ? rig : true);
          if (!(hit_y && hit_x)) continue;
          const int dr = (sy == -1) ? (a.H + 1) : (sy == 1 ? 0 : h + 1);
          const int dc = (sx == -1) ? (a.W + 1) : (sx == 1 ? 0 : w + 1);
          *reinterpret_cast<uint2*>(reinterpret_cast<__nv_bfloat16*>(a.push.buf[d]) + n * pimg + dr * prow +
                                    static_cast<long long>(dc) * a.CP + g * 4) = o;
          pushed = true;
        }
      }
    }
  }
  // publish: same protocol as the convolution kernels (last block of the grid sets the flags)
  if (a.push.enabled) {
    if (pushed) __threadfence_system();      // this thread's peer stores are visible before the count
    __syncthreads();
    if (tid == 0) {
      const unsigned int total = gridDim.x * gridDim.y * gridDim.z;
      __threadfence();
      const unsigned int prev = atomicAdd(a.done_counter, 1u);
      if (prev == total - 1) {
        *a.done_counter = 0u;
        __threadfence_system();
        const uint32_t epoch = live_epoch(a.push.epoch, a.push.stride, a.push.replay);
        for (int d = 0; d < 9; ++d)
          if (a.push.flag[d] != nullptr)
            asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(a.push.flag[d]), "r"(epoch) : "memory");
      }
    }
  }
}

}  // namespace jb

using namespace jb;

static void fill_halo(HaloPush* push, HaloWait* wait, const JbHalo* halo) {
  if (halo == nullptr) return;
  for (int d = 0; d < 9; ++d) {
    if (push) {
      push->buf[d] = halo->push_buf[d];
      push->flag[d] = static_cast<uint32_t*>(halo->push_flag[d]);
    }
    if (wait) wait->flag[d] = static_cast<const uint32_t*>(halo->wait_flag[d]);
  }
  if (push) {
    push->epoch = halo->push_epoch;
    push->enabled = halo->push_enabled;
    push->stride = halo->push_stride;
    push->replay = halo->replay;
  }
  if (wait) {
    wait->epoch = halo->wait_epoch;
    wait->enabled = halo->wait_enabled;
    wait->stride = halo->wait_stride;
    wait->replay = halo->replay;
  }
}

// Copy a strided (NB, C, H, W) tensor into a padded NHWC bf16 buffer [NB][H+2][W+2][CP] and push
// the edge pixels to the neighbours.  Strides are in elements.  Only the first CW channels of a pixel
// are written.
extern "C" int jb_halo_pack(const void* src, int src_is_fp32, long long sn, long long sc, long long sh,
                            long long sw, int NB, int C, int H, int W, int CP, int CW, void* dst, const JbHalo* halo,
                            unsigned int* done_counter, void* stream) {
  if (CP % 4 != 0 || CW % 4 != 0 || C > CW || CW > CP || CP > 256) return -1;
  PackArgs a{};
  a.src = src; a.src_is_fp32 = src_is_fp32;
  a.sn = sn; a.sc = sc; a.sh = sh; a.sw = sw;
  a.NB = NB; a.C = C; a.H = H; a.W = W; a.CP = CP; a.CW = CW;
  a.dst = static_cast<__nv_bfloat16*>(dst);
  a.done_counter = done_counter;
  fill_halo(&a.push, nullptr, halo);
  dim3 grid((W + PACK_THREADS * PACK_PIX - 1) / (PACK_THREADS * PACK_PIX), H, NB);
  if (grid.y > 65535 || grid.z > 65535) return -1;
  halo_pack_kernel<<<grid, PACK_THREADS, 0, static_cast<cudaStream_t>(stream)>>>(a);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}
