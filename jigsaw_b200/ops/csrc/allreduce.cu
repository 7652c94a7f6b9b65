// Sum all-reduce of an fp32 buffer over up to eight GPUs through peer memory, one launch per rank.
//
// Every rank has staged its contribution in its own copy of a symmetric buffer (same offset on every
// GPU).  The kernel then
//   1. tells the peers that this rank's buffer is staged, and waits (bounded) for theirs;
//   2. reduce-scatter by pulling: rank r owns slice r of the buffer, reads that slice from every rank's
//      copy (plain peer loads, 16 bytes per lane) and adds the P values in rank order, so the result does
//      not depend on timing and is bit-identical on all ranks;
//   3. all-gather by pushing: the owner stores the reduced (and scaled) slice into every rank's copy;
//   4. the last block of the grid tells the peers that this rank's stores are out and waits (bounded) for
//      the peers' notices, so that the buffer is complete on this GPU when the kernel ends.
// Small buffers (gradients of replicated parameters, a few MiB at most per bucket) are bound by the
// latency of those two notices, a few microseconds; the launch is meant to sit on a side stream under
// the remaining backward kernels.
#include <cuda_runtime.h>
#include <stdint.h>

#include "ptx.cuh"

namespace jb {

constexpr int AR_MAX_RANKS = 8;

struct AllReduceArgs {
  float* buf[AR_MAX_RANKS];                // every rank's copy of the buffer (entry `me`: local)
  uint32_t* notice_out[AR_MAX_RANKS];      // word on rank i that this rank raises (null for i == me)
  const uint32_t* notice_in[AR_MAX_RANKS]; // local word that rank i raises (null for i == me)
  uint32_t epoch;                          // call number of this buffer; the notices carry 2 e - 1 (staged) and 2 e (done)
  uint32_t stride;
  const uint32_t* replay;
  int ranks, me;
  long long n;                             // floats, a multiple of 4
  float scale;
  unsigned int* done_counter;              // local word, zero before the launch, left zero
  int* status;
};

__device__ __forceinline__ bool ar_wait(const uint32_t* f, uint32_t want, int* status, int where) {
  const uint64_t t0 = globaltimer_ns();
  while (true) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(f) : "memory");
    if (static_cast<int32_t>(v - want) >= 0) return true;
    if (globaltimer_ns() - t0 > JB_WAIT_LIMIT_NS) {
      if (status && atomicCAS(status, JB_OK, JB_ERR_FLAG_TIMEOUT) == JB_OK) {
        status[1] = where;
        status[2] = static_cast<int>(blockIdx.x);
        status[3] = static_cast<int>(want);
      }
      return false;
    }
    __nanosleep(64);
  }
}

__global__ void __launch_bounds__(256) allreduce_kernel(const AllReduceArgs a) {
  const uint32_t e = live_epoch(a.epoch, a.stride, a.replay);
  const uint32_t staged = 2u * e - 1u, done = 2u * e;
  // 1. notice "staged" (the staging copies precede this launch in stream order), then wait for the peers
  if (blockIdx.x == 0 && threadIdx.x < a.ranks && a.notice_out[threadIdx.x] != nullptr) {
    __threadfence_system();
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(a.notice_out[threadIdx.x]), "r"(staged) : "memory");
  }
  __shared__ int ok;
  if (threadIdx.x == 0) ok = 1;
  __syncthreads();
  if (threadIdx.x < a.ranks && a.notice_in[threadIdx.x] != nullptr) {
    if (!ar_wait(a.notice_in[threadIdx.x], staged, a.status, 950)) ok = 0;
  }
  __syncthreads();
  // 2 + 3. this rank's slice: pull, add in rank order, scale, push
  const long long vecs = a.n / 4;
  const long long per = (vecs + a.ranks - 1) / a.ranks;
  const long long lo = per * a.me;
  const long long hi = lo + per < vecs ? lo + per : vecs;
  if (ok) {
    for (long long i = lo + static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < hi;
         i += static_cast<long long>(gridDim.x) * blockDim.x) {
      float4 s = reinterpret_cast<const float4*>(a.buf[0])[i];
      for (int r = 1; r < a.ranks; ++r) {
        const float4 v = reinterpret_cast<const float4*>(a.buf[r])[i];
        s.x += v.x; s.y += v.y; s.z += v.z; s.w += v.w;
      }
      s.x *= a.scale; s.y *= a.scale; s.z *= a.scale; s.w *= a.scale;
      for (int r = 0; r < a.ranks; ++r) reinterpret_cast<float4*>(a.buf[r])[i] = s;
    }
  }
  // 4. last block: notice "done" to the peers, wait for theirs
  __threadfence_system();
  __syncthreads();
  __shared__ bool last;
  if (threadIdx.x == 0) {
    __threadfence_system();
    last = atomicAdd(a.done_counter, 1u) == gridDim.x - 1;
  }
  __syncthreads();
  if (!last) return;
  if (threadIdx.x == 0) *a.done_counter = 0u;
  if (threadIdx.x < a.ranks && a.notice_out[threadIdx.x] != nullptr) {
    __threadfence_system();
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(a.notice_out[threadIdx.x]), "r"(done) : "memory");
  }
  if (threadIdx.x < a.ranks && a.notice_in[threadIdx.x] != nullptr) ar_wait(a.notice_in[threadIdx.x], done, a.status, 951);
}

}  // namespace jb

struct JbAllReduce {      // C mirror passed from Python (ctypes)
  void* buf[8];
  void* notice_out[8];
  void* notice_in[8];
  unsigned int epoch, stride;
  const unsigned int* replay;
  int ranks, me;
  long long n;
  float scale;
};

// In-place sum (times `scale`) of `n` floats (a multiple of 4; 16-byte aligned buffers) over `ranks` GPUs.
// done_counter: a zeroed local word (left zero).  Returns 0 on success, a negative code otherwise.
extern "C" int jb_all_reduce_sum(const JbAllReduce* r, unsigned int* done_counter, int* status, int max_blocks,
                                 void* stream) {
  using namespace jb;
  if (r->ranks < 1 || r->ranks > AR_MAX_RANKS || r->me < 0 || r->me >= r->ranks || r->n < 4 || (r->n & 3)) return -1;
  AllReduceArgs a{};
  for (int i = 0; i < r->ranks; ++i) {
    if (reinterpret_cast<uintptr_t>(r->buf[i]) & 15) return -1;
    a.buf[i] = static_cast<float*>(r->buf[i]);
    a.notice_out[i] = static_cast<uint32_t*>(r->notice_out[i]);
    a.notice_in[i] = static_cast<const uint32_t*>(r->notice_in[i]);
  }
  a.epoch = r->epoch; a.stride = r->stride; a.replay = r->replay;
  a.ranks = r->ranks; a.me = r->me; a.n = r->n; a.scale = r->scale;
  a.done_counter = done_counter;
  a.status = status;
  const long long per = (r->n / 4 + r->ranks - 1) / r->ranks;
  long long blocks = (per + 255) / 256;
  if (blocks < 1) blocks = 1;
  if (blocks > max_blocks) blocks = max_blocks;
  allreduce_kernel<<<static_cast<unsigned>(blocks), 256, 0, static_cast<cudaStream_t>(stream)>>>(a);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}
