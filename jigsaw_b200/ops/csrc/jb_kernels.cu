// Single translation unit of the sm_100a kernel library (C ABI, loaded with ctypes).
// Build:  nvcc -gencode arch=compute_100a,code=sm_100a -lineinfo -O3 -std=c++17 \
//              -shared -Xcompiler -fPIC -o libjb_kernels.so jb_kernels.cu
#include "gemm.cu"
#include "conv3x3.cu"
#include "conv_thin.cu"
#include "wgrad_noalloc.cu"
#include "norm.cu"
#include "elementwise.cu"
#include "roll.cu"
#include "alltoall.cu"
#include "signal.cu"
#include "allreduce.cu"
#include "flash_attn.cu"
#include "flash_attn_bwd.cu"

extern "C" int jb_abi_version() { return 1; }
