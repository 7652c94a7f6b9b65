// Companions of the tcgen05 convolution for the layers it does not cover and for getting
// data into the padded halo layout:
//   * halo_pack      : any strided (N, C, H, W) fp32/bf16 tensor -> padded NHWC bf16 buffer
//                      (channels zero-filled up to CP) with the edge pixels stored straight
//                      into the neighbours' borders over NVLink;
//   * conv3x3_thin   : 3x3 convolution from a few channels (CP = 4, e.g. RGB, or the gradient
//                      of a 3-channel output) to 64 channels on CUDA cores, with the same
//                      epilogue (bias, GELU, GELU' multiply, padded output + halo push);
//   * wgrad_thin     : the matching weight gradient, out[tap][cs][c] = sum_p big[p][c] *
//                      small[p + sign * (tap - 1)][cs] plus a row of sum_p big[p][c].
// These layers are bound by the 64-channel tensor they read or write, not by arithmetic.
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

// ------------------------------------------------------------------------------------------
// 3x3 convolution, CP = 4 input channels -> 64 output channels, CUDA cores.
//   in : padded [NB][H+2][W+2][4] bf16 (halo filled)
//   w  : fp32 [9][4][64] (tap, cin, cout); taps already mirrored by the caller for a data gradient
// Thread = (pixel of a 128-pixel row segment, half of the output channels).
// ------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) conv3x3_thin_kernel(const __nv_bfloat16* __restrict__ in,
                                                            const float* __restrict__ w, const ConvArgs a) {
  __shared__ __align__(16) float ws[9 * 4 * 64];
  __shared__ int abort_flag;
  for (int i = threadIdx.x; i < 9 * 4 * 64; i += 256) ws[i] = w[i];
  if (threadIdx.x == 0) {
    abort_flag = 0;
    halo_wait_all(a.wait, &abort_flag, a.status);
  }
  __syncthreads();
  const int half = threadIdx.x >> 7;
  const int m = threadIdx.x & 127;
  const int c0 = half * 32;
  const long long prow = static_cast<long long>(a.W + 2) * 4;
  const long long pimg = static_cast<long long>(a.H + 2) * prow;
  float bias_r[32];
  load_bias_regs<32>(a, c0, bias_r);
  const int segs = a.tiles_w;
  const long long total = static_cast<long long>(a.NB) * a.H * segs;
  for (long long item = blockIdx.x; item < total; item += gridDim.x) {
    const int seg = static_cast<int>(item % segs);
    const int h = static_cast<int>((item / segs) % a.H);
    const int n = static_cast<int>(item / (static_cast<long long>(segs) * a.H));
    const int wpix = seg * 128 + m;
    if (wpix >= a.W) continue;
    float x[9][4];
#pragma unroll
    for (int dy = 0; dy < 3; ++dy) {
#pragma unroll
      for (int dx = 0; dx < 3; ++dx) {
        const uint2 u = __ldg(reinterpret_cast<const uint2*>(in + n * pimg + (h + dy) * prow +
                                                             static_cast<long long>(wpix + dx) * 4));
        const __nv_bfloat162 lo = *reinterpret_cast<const __nv_bfloat162*>(&u.x);
        const __nv_bfloat162 hi = *reinterpret_cast<const __nv_bfloat162*>(&u.y);
        x[dy * 3 + dx][0] = __low2float(lo);
        x[dy * 3 + dx][1] = __high2float(lo);
        x[dy * 3 + dx][2] = __low2float(hi);
        x[dy * 3 + dx][3] = __high2float(hi);
      }
    }
    float v[32];
#pragma unroll
    for (int j = 0; j < 32; ++j) v[j] = 0.f;
#pragma unroll
    for (int t = 0; t < 9; ++t) {
#pragma unroll
      for (int ci = 0; ci < 3; ++ci) {
        const float xv = x[t][ci];
        const float4* wr = reinterpret_cast<const float4*>(ws + (t * 4 + ci) * 64 + c0);
#pragma unroll
        for (int q = 0; q < 8; ++q) {
          const float4 ww = wr[q];
          v[4 * q + 0] = fmaf(xv, ww.x, v[4 * q + 0]);
          v[4 * q + 1] = fmaf(xv, ww.y, v[4 * q + 1]);
          v[4 * q + 2] = fmaf(xv, ww.z, v[4 * q + 2]);
          v[4 * q + 3] = fmaf(xv, ww.w, v[4 * q + 3]);
        }
      }
    }
    uint4 gsrc[4];
    prefetch_gelu_src<32>(a, n, h, wpix, c0, gsrc);
    conv_epilogue<32>(a, v, bias_r, gsrc, n, h, wpix, c0);
  }
  halo_publish(a.push, a.done_counter);
}

// ------------------------------------------------------------------------------------------
// Thin weight gradient.  big: padded [NB][H+2][W+2][64] (interior read), small: padded
// [NB][H+2][W+2][4].  out (fp32, pre-zeroed, atomically accumulated): [28][64] with
//   out[t * 3 + cs][c] = sum_p big[p][c] * small[p + sign * (t - centre)][cs],  t < 9, cs < 3
//   out[27][c]         = sum_p big[p][c]
// Thread = (channel c, one of four groups of seven rows of `out`).
// ------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) wgrad_thin_kernel(const __nv_bfloat16* __restrict__ big,
                                                          const __nv_bfloat16* __restrict__ small, float* out, int NB,
                                                          int H, int W, int sign, HaloWait wait, int* status) {
  __shared__ float sm[64][28];   // 64 pixels x 28 coefficients (27 shifted small values and a one)
  __shared__ int abort_flag;
  if (threadIdx.x == 0) {
    abort_flag = 0;
    halo_wait_all(wait, &abort_flag, status);
  }
  __syncthreads();
  const int c = threadIdx.x & 63;
  const int g = threadIdx.x >> 6;
  float acc[7];
#pragma unroll
  for (int k = 0; k < 7; ++k) acc[k] = 0.f;
  const long long brow = static_cast<long long>(W + 2) * 64, bimg = static_cast<long long>(H + 2) * brow;
  const long long srow = static_cast<long long>(W + 2) * 4, simg = static_cast<long long>(H + 2) * srow;
  const int segs = (W + 63) / 64;
  const long long total = static_cast<long long>(NB) * H * segs;
  for (long long item = blockIdx.x; item < total; item += gridDim.x) {
    const int seg = static_cast<int>(item % segs);
    const int h = static_cast<int>((item / segs) % H);
    const int n = static_cast<int>(item / (static_cast<long long>(segs) * H));
    const int w0 = seg * 64;
    __syncthreads();
    for (int i = threadIdx.x; i < 64 * 28; i += 256) {
      const int p = i / 28, k = i % 28;
      float v = 0.f;
      if (w0 + p < W) {
        if (k == 27) {
          v = 1.f;
        } else {
          const int t = k / 3, cs = k % 3;
          const int dy = sign * (t / 3 - 1), dx = sign * (t % 3 - 1);
          v = __bfloat162float(small[n * simg + (h + 1 + dy) * srow + static_cast<long long>(w0 + p + 1 + dx) * 4 + cs]);
        }
      }
      sm[p][k] = v;
    }
    __syncthreads();
    const __nv_bfloat16* bp = big + n * bimg + (h + 1) * brow + static_cast<long long>(w0 + 1) * 64 + c;
    const int np = min(64, W - w0);
    for (int p = 0; p < np; ++p) {
      const float b = __bfloat162float(bp[static_cast<long long>(p) * 64]);
#pragma unroll
      for (int k = 0; k < 7; ++k) acc[k] = fmaf(b, sm[p][g * 7 + k], acc[k]);
    }
  }
#pragma unroll
  for (int k = 0; k < 7; ++k) atomicAdd(out + (g * 7 + k) * 64 + c, acc[k]);
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

// 3x3 convolution from a 4-channel padded buffer to 64 channels (see conv3x3_thin_kernel).
extern "C" int jb_conv3x3_thin(const void* in_padded4, const float* w_tap_cin_cout, const float* bias,
                               const void* gelu_src, void* dense_pre, void* padded_out, void* dense_out, int NB,
                               int H, int W, int act, const JbHalo* halo, unsigned int* done_counter, int* status,
                               int sm_count, void* stream) {
  ConvArgs a{};
  a.NB = NB; a.H = H; a.W = W;
  a.tiles_w = (W + 127) / 128;
  a.cout_real = 64;
  a.bias = bias;
  a.gelu_src = static_cast<const __nv_bfloat16*>(gelu_src);
  a.dense_pre = static_cast<__nv_bfloat16*>(dense_pre);
  a.act = act;
  a.padded_out = static_cast<__nv_bfloat16*>(padded_out);
  a.dense_out = static_cast<__nv_bfloat16*>(dense_out);
  a.done_counter = done_counter;
  a.status = status;
  fill_halo(&a.push, &a.wait, halo);
  const long long items = static_cast<long long>(NB) * H * a.tiles_w;
  const long long want = static_cast<long long>(sm_count) * 8;
  const int grid = static_cast<int>(items < want ? items : want);
  conv3x3_thin_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(in_padded4), w_tap_cin_cout, a);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

// Thin weight gradient; `out` ([28][64] fp32) is zeroed here and accumulated atomically.
extern "C" int jb_wgrad_thin(const void* big_padded64, const void* small_padded4, float* out, int NB, int H, int W,
                             int sign, const JbHalo* halo, int* status, int sm_count, void* stream) {
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (cudaMemsetAsync(out, 0, 28 * 64 * sizeof(float), st) != cudaSuccess) return -3;
  HaloWait wait{};
  fill_halo(nullptr, &wait, halo);
  const long long items = static_cast<long long>(NB) * H * ((W + 63) / 64);
  const long long want = static_cast<long long>(sm_count) * 8;
  const int grid = static_cast<int>(items < want ? items : want);
  wgrad_thin_kernel<<<grid, 256, 0, st>>>(static_cast<const __nv_bfloat16*>(big_padded64),
                                          static_cast<const __nv_bfloat16*>(small_padded4), out, NB, H, W, sign, wait,
                                          status);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}
