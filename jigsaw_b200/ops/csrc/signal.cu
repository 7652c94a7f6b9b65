// Write-after-read protection of recycled halo buffers.
//
// A padded buffer is written by its owner (interior) and by the owner's neighbours (border).  The
// arrival flags tell a consumer when the border of the CURRENT content is complete; they say nothing
// about when a neighbour has finished READING the previous content of the same buffer, so a rank that
// runs ahead could push the next border into memory its neighbour still reads.  Two tiny kernels close
// that gap without any host synchronisation:
//   slot_release_kernel  runs in stream order after the last consumer of a buffer's content and tells
//                        every neighbour "I am done with epoch e of this buffer" (a max, so a late
//                        duplicate can never lower it);
//   slot_acquire_kernel  runs in stream order before the producer of the next content: it waits
//                        (bounded) until every neighbour has released the previous epoch, which it
//                        reads from a device word kept per buffer slot, and records the new epoch there.
// Keeping "the previous epoch" in device memory makes the pair correct inside a replayed CUDA graph,
// where the first production of a step follows the last production of the previous replay.
#include <cuda_runtime.h>
#include <stdint.h>

#include "ptx.cuh"

namespace jb {

__global__ void slot_acquire_kernel(const uint32_t* a0, const uint32_t* a1, const uint32_t* a2, const uint32_t* a3,
                                    const uint32_t* a4, const uint32_t* a5, const uint32_t* a6, const uint32_t* a7,
                                    uint32_t* last_epoch, uint32_t new_epoch, uint32_t stride, const uint32_t* replay,
                                    int* status) {
  const uint32_t* acks[8] = {a0, a1, a2, a3, a4, a5, a6, a7};
  const uint32_t prev = *last_epoch;                 // every lane reads before lane 0 overwrites
  __syncwarp();
  if (threadIdx.x == 0) *last_epoch = live_epoch(new_epoch, stride, replay);
  const uint32_t* mine = threadIdx.x < 8 ? acks[threadIdx.x] : nullptr;
  if (mine == nullptr || prev == 0u) return;         // nothing was ever produced into this slot
  const uint64_t t0 = globaltimer_ns();
  while (true) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(mine) : "memory");
    if (static_cast<int32_t>(v - prev) >= 0) break;
    if (globaltimer_ns() - t0 > JB_WAIT_LIMIT_NS) {
      if (status && atomicCAS(status, JB_OK, JB_ERR_FLAG_TIMEOUT) == JB_OK) {
        status[1] = 900;                             // the wait for a neighbour's release gave up
        status[2] = static_cast<int>(threadIdx.x);
        status[3] = static_cast<int>(prev);
      }
      break;
    }
    __nanosleep(64);
  }
}

__global__ void slot_release_kernel(uint32_t* r0, uint32_t* r1, uint32_t* r2, uint32_t* r3, uint32_t* r4, uint32_t* r5,
                                    uint32_t* r6, uint32_t* r7, uint32_t epoch, uint32_t stride, const uint32_t* replay) {
  uint32_t* rel[8] = {r0, r1, r2, r3, r4, r5, r6, r7};
  const uint32_t e = live_epoch(epoch, stride, replay);
  if (threadIdx.x < 8 && rel[threadIdx.x] != nullptr)
    asm volatile("red.release.sys.global.max.u32 [%0], %1;" ::"l"(rel[threadIdx.x]), "r"(e) : "memory");
}

}  // namespace jb

// Copy `bytes` from `src` to `dst` (either may be a peer's memory mapped into this process) with the copy
// engines, in stream order: no SM is involved, so the copy runs beside whatever kernels occupy the GPU.
extern "C" int jb_memcpy_async(void* dst, const void* src, long long bytes, void* stream) {
  if (bytes <= 0) return -1;
  return cudaMemcpyAsync(dst, src, static_cast<size_t>(bytes), cudaMemcpyDefault, static_cast<cudaStream_t>(stream)) ==
                 cudaSuccess
             ? 0
             : -4;
}

// The same for `rows` rows of `width` bytes each, `dpitch` / `spitch` bytes apart (a column block of a matrix).
extern "C" int jb_memcpy2d_async(void* dst, long long dpitch, const void* src, long long spitch, long long width,
                                 long long rows, void* stream) {
  if (width <= 0 || rows <= 0) return -1;
  return cudaMemcpy2DAsync(dst, static_cast<size_t>(dpitch), src, static_cast<size_t>(spitch), static_cast<size_t>(width),
                           static_cast<size_t>(rows), cudaMemcpyDefault, static_cast<cudaStream_t>(stream)) == cudaSuccess
             ? 0
             : -4;
}

// Before producing content `new_epoch` into a buffer slot: wait until the (up to eight) local
// acknowledgement words have reached the epoch of the slot's previous content, then record the new
// epoch in `last_epoch` (a device word owned by the slot).
extern "C" int jb_slot_acquire(const void* const* acks, int n, void* last_epoch, unsigned int new_epoch,
                               unsigned int stride, const unsigned int* replay, int* status, void* stream) {
  if (n < 0 || n > 8 || last_epoch == nullptr) return -1;
  const uint32_t* a[8] = {};
  for (int i = 0; i < n; ++i) a[i] = static_cast<const uint32_t*>(acks[i]);
  jb::slot_acquire_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(
      a[0], a[1], a[2], a[3], a[4], a[5], a[6], a[7], static_cast<uint32_t*>(last_epoch), new_epoch, stride, replay, status);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

// After the last consumer of content `epoch`: raise the (up to eight) acknowledgement words on the
// neighbours (peer pointers) to that epoch.
extern "C" int jb_slot_release(void* const* rel, int n, unsigned int epoch, unsigned int stride,
                               const unsigned int* replay, void* stream) {
  if (n < 0 || n > 8) return -1;
  uint32_t* r[8] = {};
  for (int i = 0; i < n; ++i) r[i] = static_cast<uint32_t*>(rel[i]);
  jb::slot_release_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(r[0], r[1], r[2], r[3], r[4], r[5], r[6], r[7],
                                                                           epoch, stride, replay);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}
