// Host-side construction of TMA tensor maps (bf16, 128-byte swizzle) without linking
// libcuda: the driver entry point is looked up through the runtime.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

namespace jb {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn get_encode_tiled() {
  static EncodeTiledFn fn = nullptr;
  if (fn == nullptr) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q);
    if (e != cudaSuccess || q != cudaDriverEntryPointSuccess || p == nullptr) return nullptr;
    fn = reinterpret_cast<EncodeTiledFn>(p);
  }
  return fn;
}

// The encoder is a driver-API call and needs a current context on the calling thread.  A thread
// that has only used cached allocations so far (an autograd worker, for instance) may not have one;
// creating and destroying an event through the runtime binds the device's primary context and is
// legal while another stream is being captured.
inline void ensure_current_context() {
  typedef CUresult (*GetCurrentFn)(CUcontext*);
  static GetCurrentFn get_current = nullptr;
  if (get_current == nullptr) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuCtxGetCurrent", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      get_current = reinterpret_cast<GetCurrentFn>(p);
  }
  CUcontext ctx = nullptr;
  if (get_current != nullptr && get_current(&ctx) == CUDA_SUCCESS && ctx != nullptr) return;
  cudaEvent_t ev;
  if (cudaEventCreateWithFlags(&ev, cudaEventDisableTiming) == cudaSuccess) cudaEventDestroy(ev);
}

// rank <= 5.  dims[0] is the innermost (contiguous) extent in elements; strides_bytes[i]
// is the byte stride of dims[i+1] (rank-1 entries, each a multiple of 16); box[] is the
// tile copied per request (box[0]*2 bytes == 128 for the 128-byte swizzle used here).
// Out-of-range elements read as zero.  Returns 0 on success.
inline int make_tmap_bf16(CUtensorMap* out, const void* base, int rank, const uint64_t* dims,
                          const uint64_t* strides_bytes, const uint32_t* box, bool swizzle128 = true) {
  EncodeTiledFn fn = get_encode_tiled();
  if (fn == nullptr) return -1;
  ensure_current_context();
  cuuint64_t gdim[5];
  cuuint64_t gstr[4];
  cuuint32_t bx[5];
  cuuint32_t es[5];
  for (int i = 0; i < rank; ++i) {
    gdim[i] = dims[i];
    bx[i] = box[i];
    es[i] = 1;
  }
  for (int i = 0; i + 1 < rank; ++i) gstr[i] = strides_bytes[i];
  CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, static_cast<cuuint32_t>(rank), const_cast<void*>(base),
                  gdim, gstr, bx, es, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    fprintf(stderr, "jigsaw_b200: cuTensorMapEncodeTiled failed with code %d\n", static_cast<int>(r));
    return static_cast<int>(r);
  }
  return 0;
}

}  // namespace jb
