// All-to-all that re-shards a tensor (split one dimension over the ranks, concatenate what arrives
// along another) as ONE kernel over peer memory: every 16-byte vector is stored straight at its final
// position in the destination rank's output (plain stores over NVLink), the last CTA publishes an epoch
// flag to every peer and waits (bounded) for theirs.  This is the sequence <-> head exchange of Ulysses
// attention.
//
// The tensor is viewed as [D0][D1][D2][D3][V] (V = 16-byte vectors of the contiguous tail); dimension
// `split` is cut into P chunks, chunk p goes to rank p and lands at block `me` of dimension `cat`.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include "ptx.cuh"

namespace jb {

struct A2aArgs {
  const uint4* x;
  long long dim[5];            // input extents, dim[4] in vectors
  int split, cat;              // dimensions 0..3
  int parts, me;
  uint4* out[8];               // output base on every rank
  uint32_t* flag_out[8];       // flag word on rank p for source `me` (null for p == me)
  const uint32_t* flag_in[8];  // local flag words, one per source (null for me)
  uint32_t epoch, stride;
  const uint32_t* replay;
  unsigned int* done_counter;
  int* status;
};

__global__ void __launch_bounds__(256) a2a_kernel(const A2aArgs a) {
  const long long total = a.dim[0] * a.dim[1] * a.dim[2] * a.dim[3] * a.dim[4];
  const long long chunk = a.dim[a.split] / a.parts;
  long long od[5];             // output extents
  for (int i = 0; i < 5; ++i) od[i] = a.dim[i];
  od[a.split] = chunk;
  od[a.cat] = a.dim[a.cat] * a.parts;
  for (long long idx = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; idx < total;
       idx += static_cast<long long>(gridDim.x) * blockDim.x) {
    long long r = idx, ix[5];
    for (int i = 4; i >= 0; --i) {
      ix[i] = r % a.dim[i];
      r /= a.dim[i];
    }
    const int dest = static_cast<int>(ix[a.split] / chunk);
    ix[a.split] -= dest * chunk;
    ix[a.cat] += static_cast<long long>(a.me) * a.dim[a.cat];
    const long long o = (((ix[0] * od[1] + ix[1]) * od[2] + ix[2]) * od[3] + ix[3]) * od[4] + ix[4];
    a.out[dest][o] = a.x[idx];
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x != 0) return;
  __threadfence();
  if (atomicAdd(a.done_counter, 1u) != gridDim.x - 1) return;
  *a.done_counter = 0u;
  __threadfence_system();
  const uint32_t epoch = live_epoch(a.epoch, a.stride, a.replay);
  for (int p = 0; p < a.parts; ++p)
    if (a.flag_out[p] != nullptr)
      asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(a.flag_out[p]), "r"(epoch) : "memory");
  const uint64_t t0 = globaltimer_ns();
  for (int p = 0; p < a.parts; ++p) {
    const uint32_t* f = a.flag_in[p];
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

struct JbA2a {
  const void* x;
  long long dim[5];
  int split, cat, parts, me;
  void* out[8];
  void* flag_out[8];
  const void* flag_in[8];
  unsigned int epoch, stride;
  const unsigned int* replay;
};

extern "C" int jb_all_to_all(const JbA2a* r, unsigned int* done_counter, int* status, int sm_count, void* stream) {
  using namespace jb;
  if (r->parts < 2 || r->parts > 8 || r->split < 0 || r->split > 3 || r->cat < 0 || r->cat > 3 || r->split == r->cat)
    return -1;
  A2aArgs a{};
  a.x = static_cast<const uint4*>(r->x);
  long long total = 1;
  for (int i = 0; i < 5; ++i) {
    if (r->dim[i] <= 0) return -1;
    a.dim[i] = r->dim[i];
    total *= r->dim[i];
  }
  if (a.dim[r->split] % r->parts != 0) return -1;
  a.split = r->split; a.cat = r->cat; a.parts = r->parts; a.me = r->me;
  for (int p = 0; p < r->parts; ++p) {
    a.out[p] = static_cast<uint4*>(r->out[p]);
    a.flag_out[p] = static_cast<uint32_t*>(r->flag_out[p]);
    a.flag_in[p] = static_cast<const uint32_t*>(r->flag_in[p]);
    if (a.out[p] == nullptr) return -1;
  }
  a.epoch = r->epoch; a.stride = r->stride; a.replay = r->replay;
  a.done_counter = done_counter; a.status = status;
  long long grid = (total + 255) / 256;
  const long long cap = static_cast<long long>(sm_count) * 8;
  if (grid > cap) grid = cap;
  a2a_kernel<<<static_cast<unsigned int>(grid), 256, 0, static_cast<cudaStream_t>(stream)>>>(a);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

// ------------------------------------------------------------------------------------------
// Fetch a contiguous block from another GPU's memory with plain 16-byte loads over NVLink, after
// its owner's epoch flag says the block is complete (bounded wait).  Ring attention uses this to
// pull the key / value chunk of a step straight from the chunk's owner while the previous chunk
// is being attended to on another stream.
// ------------------------------------------------------------------------------------------
namespace jb {
__global__ void __launch_bounds__(256) peer_fetch_kernel(const uint4* __restrict__ src, uint4* __restrict__ dst,
                                                         long long n16, const uint32_t* flag, uint32_t epoch,
                                                         uint32_t stride, const uint32_t* replay, int* status) {
  __shared__ int ok;
  if (threadIdx.x == 0) {
    ok = 1;
    if (flag != nullptr) {
      const uint32_t want = live_epoch(epoch, stride, replay);
      const uint64_t t0 = globaltimer_ns();
      while (true) {
        uint32_t v;
        asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(flag) : "memory");
        if (static_cast<int32_t>(v - want) >= 0) break;
        if (globaltimer_ns() - t0 > JB_WAIT_LIMIT_NS) {
          if (status) atomicCAS(status, JB_OK, JB_ERR_FLAG_TIMEOUT);
          ok = 0;
          break;
        }
        __nanosleep(64);
      }
    }
  }
  __syncthreads();
  if (!ok) return;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n16;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    uint4 v;
    asm volatile("ld.global.relaxed.sys.v4.u32 {%0, %1, %2, %3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(src + i) : "memory");
    dst[i] = v;
  }
}
}  // namespace jb

// dst[0 .. nbytes) = src[0 .. nbytes) where src may be a peer pointer; waits for *flag >= epoch first
// (flag is a local word, null = no wait).  nbytes must be a multiple of 16.
extern "C" int jb_peer_fetch(const void* src, void* dst, long long nbytes, const void* flag, unsigned int epoch,
                             unsigned int stride, const unsigned int* replay, int* status, int ctas, void* stream) {
  if (nbytes <= 0 || (nbytes & 15)) return -1;
  const long long n16 = nbytes / 16;
  long long grid = (n16 + 255) / 256;
  if (grid > ctas) grid = ctas;
  jb::peer_fetch_kernel<<<static_cast<unsigned int>(grid), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint4*>(src), static_cast<uint4*>(dst), n16, static_cast<const uint32_t*>(flag), epoch, stride,
      replay, status);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

// Wait (bounded) until every given local flag word has reached the epoch: the consumer side of a push
// whose data is then read by ordinary kernels of the same stream.
namespace jb {
__global__ void wait_flags_kernel(const uint32_t* f0, const uint32_t* f1, const uint32_t* f2, const uint32_t* f3,
                                  const uint32_t* f4, const uint32_t* f5, const uint32_t* f6, const uint32_t* f7,
                                  uint32_t epoch, uint32_t stride, const uint32_t* replay, int* status) {
  const uint32_t* f[8] = {f0, f1, f2, f3, f4, f5, f6, f7};
  const uint32_t* mine = f[threadIdx.x & 7];
  if (threadIdx.x >= 8 || mine == nullptr) return;
  const uint32_t want = live_epoch(epoch, stride, replay);
  const uint64_t t0 = globaltimer_ns();
  while (true) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(mine) : "memory");
    if (static_cast<int32_t>(v - want) >= 0) break;
    if (globaltimer_ns() - t0 > JB_WAIT_LIMIT_NS) {
      if (status) atomicCAS(status, JB_OK, JB_ERR_FLAG_TIMEOUT);
      break;
    }
    __nanosleep(64);
  }
}
}  // namespace jb

extern "C" int jb_wait_flags(const void* const* flags, int n, unsigned int epoch, unsigned int stride,
                             const unsigned int* replay, int* status, void* stream) {
  if (n < 0 || n > 8) return -1;
  const uint32_t* f[8] = {};
  for (int i = 0; i < n; ++i) f[i] = static_cast<const uint32_t*>(flags[i]);
  jb::wait_flags_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(f[0], f[1], f[2], f[3], f[4], f[5], f[6], f[7],
                                                                         epoch, stride, replay, status);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}
