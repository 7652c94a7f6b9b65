// Cyclic roll of a tensor along one or two dimensions that are tiled over GPUs, as ONE kernel: every
// element is stored straight at its destination, in this GPU's output or in a neighbour's (plain
// stores over NVLink); the last CTA then publishes an epoch flag to the destination ranks and waits
// (bounded) for the flags of the source ranks, so the output is complete when the kernel ends.
//
// The tensor is viewed as [A][H][M][W][I]: H and W are the rolled dimensions (W = 1 when only one is
// rolled), I the contiguous tail, moved in 16-byte vectors.  With n rows per rank and a shift
// s = q n + rem (0 <= rem < n), rows [0, n - rem) go to rank r + q and rows [n - rem, n) to rank
// r + q + 1 (mod G), which covers any shift; a dimension that is not split has G = 1.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include "ptx.cuh"

namespace jb {

struct RollArgs {
  const uint4* x;
  long long A, M, I;            // I in 16-byte vectors
  int H, W;                     // local extents of the rolled dimensions
  int rem_h, rem_w;             // shift modulo the local extent
  uint4* out[4];                // destination output for (ah, aw): index ah * 2 + aw (may be this GPU's)
  uint32_t* flag_out[4];        // flag word on that destination (null: this GPU or unused)
  const uint32_t* flag_in[4];   // local flag words to wait for (null: none)
  uint32_t epoch, stride;
  const uint32_t* replay;
  unsigned int* done_counter;
  int* status;
};

__global__ void __launch_bounds__(256) roll_kernel(const RollArgs a) {
  const long long rowI = a.I;
  const long long total = a.A * a.H * a.M * a.W * rowI;
  bool remote = false;
  for (long long idx = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; idx < total;
       idx += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long i = idx % rowI;
    long long r = idx / rowI;
    const int w = static_cast<int>(r % a.W); r /= a.W;
    const long long m = r % a.M; r /= a.M;
    const int h = static_cast<int>(r % a.H);
    const long long b = r / a.H;
    int dh = h + a.rem_h, ah = 0;
    if (dh >= a.H) { dh -= a.H; ah = 1; }
    int dw = w + a.rem_w, aw = 0;
    if (dw >= a.W) { dw -= a.W; aw = 1; }
    const int k = ah * 2 + aw;
    const long long dst = (((b * a.H + dh) * a.M + m) * a.W + dw) * rowI + i;
    a.out[k][dst] = a.x[idx];
    remote |= a.flag_out[k] != nullptr;
  }
  if (remote) __threadfence_system();
  __syncthreads();
  if (threadIdx.x != 0) return;
  __threadfence();
  if (atomicAdd(a.done_counter, 1u) != gridDim.x - 1) return;
  *a.done_counter = 0u;
  __threadfence_system();
  const uint32_t epoch = live_epoch(a.epoch, a.stride, a.replay);
  for (int k = 0; k < 4; ++k)
    if (a.flag_out[k] != nullptr)
      asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(a.flag_out[k]), "r"(epoch) : "memory");
  const uint64_t t0 = globaltimer_ns();
  for (int k = 0; k < 4; ++k) {
    const uint32_t* f = a.flag_in[k];
    if (f == nullptr) continue;
    while (true) {
      uint32_t v;
      asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(f) : "memory");
      if (static_cast<int32_t>(v - epoch) >= 0) break;
      if (globaltimer_ns() - t0 > JB_WAIT_LIMIT_NS) {
        if (a.status) atomicCAS(a.status, JB_OK, JB_ERR_FLAG_TIMEOUT);
        return;
      }
      __nanosleep(64);
    }
  }
}

}  // namespace jb

struct JbRoll {
  const void* x;
  long long A, M, I16;
  int H, W, rem_h, rem_w;
  void* out[4];
  void* flag_out[4];
  const void* flag_in[4];
  unsigned int epoch, stride;
  const unsigned int* replay;
};

extern "C" int jb_roll(const JbRoll* r, unsigned int* done_counter, int* status, int sm_count, void* stream) {
  using namespace jb;
  if (r->A <= 0 || r->H <= 0 || r->M <= 0 || r->W <= 0 || r->I16 <= 0) return -1;
  if (r->rem_h < 0 || r->rem_h >= r->H || r->rem_w < 0 || r->rem_w >= r->W) return -1;
  RollArgs a{};
  a.x = static_cast<const uint4*>(r->x);
  a.A = r->A; a.M = r->M; a.I = r->I16; a.H = r->H; a.W = r->W; a.rem_h = r->rem_h; a.rem_w = r->rem_w;
  for (int k = 0; k < 4; ++k) {
    a.out[k] = static_cast<uint4*>(r->out[k]);
    a.flag_out[k] = static_cast<uint32_t*>(r->flag_out[k]);
    a.flag_in[k] = static_cast<const uint32_t*>(r->flag_in[k]);
    if (a.out[k] == nullptr) return -1;
  }
  a.epoch = r->epoch; a.stride = r->stride; a.replay = r->replay;
  a.done_counter = done_counter; a.status = status;
  const long long total = a.A * a.H * a.M * a.W * a.I;
  long long grid = (total + 255) / 256;
  const long long cap = static_cast<long long>(sm_count) * 8;
  if (grid > cap) grid = cap;
  roll_kernel<<<static_cast<unsigned int>(grid), 256, 0, static_cast<cudaStream_t>(stream)>>>(a);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}
