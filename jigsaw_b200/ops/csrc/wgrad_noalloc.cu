// Allocation-free variant of the weight-gradient entry point: see jb_noalloc.h.
#include "jb_noalloc.h"

#include <mutex>

static_assert(JB_NOALLOC_WGRAD_SCRATCH_BYTES == JB_NOALLOC_WGRAD_MAX_CTAS * jb::WG_PARTIAL_FLOATS * 4,
              "the static scratch must hold one block of partial sums per thread block");

namespace {

// Scratch of the allocation-free path: per-CTA partial sums and the status word of the
// kernel's bounded waits.  In host code these names are only handles for
// cudaGetSymbolAddress; they are not device addresses.
static __device__ __align__(256) float g_noalloc_partials[JB_NOALLOC_WGRAD_SCRATCH_BYTES / 4];
static __device__ __align__(256) int g_noalloc_status[4];

struct NoallocDevice {
  bool ready = false;
  float* partials = nullptr;
  int* status = nullptr;
  int sm_count = 0;
};
static NoallocDevice g_noalloc_dev[64];
static std::mutex g_noalloc_lock;      // first calls from several host threads fill the table one at a time

// Device addresses of the scratch, looked up once per device with that device current.
static int noalloc_setup(NoallocDevice** out) {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return -6;
  NoallocDevice& d = g_noalloc_dev[dev];
  std::lock_guard<std::mutex> guard(g_noalloc_lock);
  if (!d.ready) {
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_noalloc_partials) != cudaSuccess || p == nullptr) return -7;
    d.partials = static_cast<float*>(p);
    if (cudaGetSymbolAddress(&p, g_noalloc_status) != cudaSuccess || p == nullptr) return -7;
    d.status = static_cast<int*>(p);
    if (cudaDeviceGetAttribute(&d.sm_count, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return -7;
    d.ready = true;
  }
  *out = &d;
  return 0;
}

}  // namespace

extern "C" int jb_conv3x3_c64_wgrad_noalloc(const void* x_padded, const void* gy_padded, float* gw, float* gb,
                                            int NB, int H, int W, int check_status, void* stream) {
  using namespace jb;
  if (NB < 1 || H < 1 || W < 1) return -1;
  if (static_cast<long long>(NB) * H * W > JB_NOALLOC_WGRAD_MAX_PIXELS || W > 65534) {
    fprintf(stderr,
            "jigsaw_b200: jb_conv3x3_c64_wgrad_noalloc refuses NB=%d H=%d W=%d: the allocation-free path is limited "
            "to %lld pixels per call (static scratch of %d bytes); use jb_conv3x3_c64_wgrad with caller-provided "
            "scratch for larger tiles\n",
            NB, H, W, static_cast<long long>(JB_NOALLOC_WGRAD_MAX_PIXELS), JB_NOALLOC_WGRAD_SCRATCH_BYTES);
    return -5;
  }
  NoallocDevice* d = nullptr;
  const int rc = noalloc_setup(&d);
  if (rc != 0) return rc;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (check_status) {
    // reading the status back synchronises the stream, which a capturing stream cannot do:
    // refuse before anything is enqueued
    cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
    if (cudaStreamIsCapturing(st, &cap) != cudaSuccess) return -3;
    if (cap != cudaStreamCaptureStatusNone) return -8;
  }
  // The status word is the only part of the scratch that must start at zero.
  if (cudaMemsetAsync(d->status, 0, 4 * sizeof(int), st) != cudaSuccess) return -3;

  CUtensorMap tmX, tmG;
  if (padded_tmap(&tmX, x_padded, NB, H, W, CV_BOXW, 0) != 0) return -2;
  if (padded_tmap(&tmG, gy_padded, NB, H, W, CV_TW, 1) != 0) return -2;
  WgradArgs a{};
  a.NB = NB; a.H = H; a.W = W;
  a.tiles_w = (W + CV_TW - 1) / CV_TW;
  const int ctas = d->sm_count < JB_NOALLOC_WGRAD_MAX_CTAS ? d->sm_count : JB_NOALLOC_WGRAD_MAX_CTAS;
  choose_strips(H, NB, a.tiles_w, ctas, WG_CHUNK, &a.rows_per_strip, &a.nstrips);
  a.partials = d->partials;
  a.status = d->status;
  const int items = NB * a.tiles_w * a.nstrips;
  const int grid = items < ctas ? items : ctas;
  constexpr int SMEM = WG_SLOTS * CV_SLOT_BYTES + WG_GSTAGES * 16384 + 2048 + 256 + 1024;
  if (cudaFuncSetAttribute(conv3x3_wgrad_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM) != cudaSuccess)
    return -3;
  conv3x3_wgrad_kernel<<<grid, WG_THREADS, SMEM, st>>>(tmX, tmG, a);
  if (cudaGetLastError() != cudaSuccess) return -4;
  const int n = 9 * 64 * 64 + 64;
  conv3x3_wgrad_reduce_kernel<<<(n + 255) / 256, 256, 0, st>>>(d->partials, grid, gw, gb);
  if (cudaGetLastError() != cudaSuccess) return -4;
  if (check_status) {
    int host_status[4] = {0, 0, 0, 0};
    if (cudaMemcpyAsync(host_status, d->status, sizeof(host_status), cudaMemcpyDeviceToHost, st) != cudaSuccess) return -3;
    if (cudaStreamSynchronize(st) != cudaSuccess) return -3;
    if (host_status[0] != 0) return 1;
  }
  return 0;
}
