// Memory-bound helper kernels: online-softmax merge of attention chunks, fused squared-error loss
// (forward sum and backward gradient on strided tensors), multi-tensor Adam / AdamW.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "ptx.cuh"

namespace jb {

// ------------------------------------------------------------------------------------------
// Merge the result (o2, l2) of a new key/value chunk into the running state (o1 fp32, l1):
//   w = sigmoid(l2 - l1);  o1 += w (o2 - o1);  l1 = max(l1, l2) + log1p(exp(-|l1 - l2|))
// rows = b * h * s (a query of one head).
// ------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) merge_kernel(float* __restrict__ o1, float* __restrict__ l1,
                                                    const void* __restrict__ o2, int o2_bf16,
                                                    const float* __restrict__ l2, long long rows, int d) {
  // One thread per four consecutive features; the thread of a row's first vector also updates the
  // row's log-sum-exp.  All threads of a row sit in one warp (the launcher only picks this variant when
  // d / 4 divides 32), so every reader of l1[row] has passed the warp barrier before the writer stores.
  const int vec_per_row = d >> 2;
  const long long idx = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  const long long row = idx / vec_per_row;
  const int v = static_cast<int>(idx % vec_per_row);
  float a = 0.f, b = 0.f;
  const bool live = row < rows;
  if (live) {
    a = l1[row];
    b = l2[row];
  }
  __syncwarp();
  if (!live) return;
  // a = -inf (nothing merged yet) gives w = 1; b = -inf keeps the state
  const float diff = b - a;
  const float w = (b == -INFINITY) ? 0.f : 1.f / (1.f + __expf(-diff));
  float4* po = reinterpret_cast<float4*>(o1 + row * d) + v;
  float4 cur = *po;
  float4 nw;
  if (o2_bf16) {
    const uint2 raw = *(reinterpret_cast<const uint2*>(static_cast<const __nv_bfloat16*>(o2) + row * d) + v);
    const __nv_bfloat162 p0 = *reinterpret_cast<const __nv_bfloat162*>(&raw.x);
    const __nv_bfloat162 p1 = *reinterpret_cast<const __nv_bfloat162*>(&raw.y);
    nw = make_float4(__low2float(p0), __high2float(p0), __low2float(p1), __high2float(p1));
  } else {
    nw = *(reinterpret_cast<const float4*>(static_cast<const float*>(o2) + row * d) + v);
  }
  cur.x += w * (nw.x - cur.x); cur.y += w * (nw.y - cur.y); cur.z += w * (nw.z - cur.z); cur.w += w * (nw.w - cur.w);
  *po = cur;
  if (v == 0) {
    const float m = fmaxf(a, b);
    l1[row] = (m == -INFINITY) ? m : m + log1pf(__expf(-fabsf(diff)));
  }
}

// scalar variant: one warp per row, any d
__global__ void __launch_bounds__(256) merge_rows_kernel(float* __restrict__ o1, float* __restrict__ l1,
                                                         const void* __restrict__ o2, int o2_bf16,
                                                         const float* __restrict__ l2, long long rows, int d) {
  const long long row = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (row >= rows) return;
  const float a = l1[row], b = l2[row];
  __syncwarp();
  const float diff = b - a;
  const float w = (b == -INFINITY) ? 0.f : 1.f / (1.f + __expf(-diff));
  float* po = o1 + row * d;
  for (int i = lane; i < d; i += 32) {
    const float nw = o2_bf16 ? __bfloat162float(static_cast<const __nv_bfloat16*>(o2)[row * d + i])
                             : static_cast<const float*>(o2)[row * d + i];
    const float cur = po[i];
    po[i] = cur + w * (nw - cur);
  }
  if (lane == 0) {
    const float m = fmaxf(a, b);
    l1[row] = (m == -INFINITY) ? m : m + log1pf(__expf(-fabsf(diff)));
  }
}

// ------------------------------------------------------------------------------------------
// Element-wise losses f(a, b) on tensors of up to four dimensions with arbitrary strides:
//   forward : out[0] = sum f(a, b)            (deterministic two-level reduction)
//   backward: ga = scale[0] * df/da, written with the strides of a
// f is chosen by `op`: squared error, absolute error, smooth L1 (beta), binary cross-entropy of
// probabilities (logarithms clamped at -100, as PyTorch does) and of logits.
// ------------------------------------------------------------------------------------------
enum : int { PAIR_SQ = 0, PAIR_L1 = 1, PAIR_SMOOTH_L1 = 2, PAIR_BCE = 3, PAIR_BCE_LOGITS = 4 };

__device__ __forceinline__ float pair_value(int op, float a, float b, float beta) {
  const float d = a - b;
  switch (op) {
    case PAIR_SQ: return d * d;
    case PAIR_L1: return fabsf(d);
    case PAIR_SMOOTH_L1: {
      const float ad = fabsf(d);
      return ad < beta ? 0.5f * d * d / beta : ad - 0.5f * beta;
    }
    case PAIR_BCE: return -(b * fmaxf(logf(a), -100.f) + (1.f - b) * fmaxf(logf(1.f - a), -100.f));
    default: return fmaxf(a, 0.f) - a * b + log1pf(expf(-fabsf(a)));           // PAIR_BCE_LOGITS
  }
}

__device__ __forceinline__ float pair_grad(int op, float a, float b, float beta) {
  const float d = a - b;
  switch (op) {
    case PAIR_SQ: return 2.f * d;
    case PAIR_L1: return d > 0.f ? 1.f : (d < 0.f ? -1.f : 0.f);
    case PAIR_SMOOTH_L1: return fabsf(d) < beta ? d / beta : (d > 0.f ? 1.f : -1.f);
    case PAIR_BCE: return d / fmaxf((1.f - a) * a, 1e-12f);
    default: return 1.f / (1.f + expf(-a)) - b;                                 // PAIR_BCE_LOGITS
  }
}

struct Strided4 {
  const void* ptr;
  int is_bf16;
  long long stride[4];
};

struct MseArgs {
  Strided4 a, b;
  int size[4];          // logical shape (leading dimensions padded with 1)
  long long numel;
  float* partial;       // [grid]
  float* out;           // scalar
  unsigned int* counter;
  const float* scale;   // backward: upstream gradient (device scalar)
  void* ga;             // backward: gradient of a (strides of a)
  int ga_bf16;
  int a_dense;          // a's offset equals the linear index in the given dimension order
  int op;               // PAIR_*
  float beta;           // smooth L1
};

__device__ __forceinline__ float load_strided(const Strided4& t, long long off) {
  return t.is_bf16 ? __bfloat162float(static_cast<const __nv_bfloat16*>(t.ptr)[off])
                   : static_cast<const float*>(t.ptr)[off];
}

// The caller orders the dimensions so that `a` is walked in memory order (its offset is then the linear
// index when it is dense); only `b` needs its index taken apart, in 32-bit arithmetic when it fits.
__device__ __forceinline__ void mse_offsets(const MseArgs& p, long long i, long long* oa, long long* ob) {
  const int s3 = p.size[3], s2 = p.size[2], s1 = p.size[1];
  long long i0;
  int i1, i2, i3;
  if (p.numel < 0x7fffffffll) {
    unsigned int r = static_cast<unsigned int>(i);
    i3 = r % s3; r /= s3;
    i2 = r % s2; r /= s2;
    i1 = r % s1;
    i0 = r / s1;
  } else {
    long long r = i;
    i3 = static_cast<int>(r % s3); r /= s3;
    i2 = static_cast<int>(r % s2); r /= s2;
    i1 = static_cast<int>(r % s1);
    i0 = r / s1;
  }
  *oa = p.a_dense ? i : i0 * p.a.stride[0] + i1 * p.a.stride[1] + i2 * p.a.stride[2] + i3 * p.a.stride[3];
  *ob = i0 * p.b.stride[0] + i1 * p.b.stride[1] + i2 * p.b.stride[2] + i3 * p.b.stride[3];
}

__global__ void __launch_bounds__(256) mse_fwd_kernel(const MseArgs p) {
  float s = 0.f;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < p.numel;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    long long oa, ob;
    mse_offsets(p, i, &oa, &ob);
    s += pair_value(p.op, load_strided(p.a, oa), load_strided(p.b, ob), p.beta);
  }
  __shared__ float red[8];
  __shared__ bool last;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = s;
  __syncthreads();
  if (threadIdx.x == 0) {
    float t = 0.f;
    for (int w = 0; w < 8; ++w) t += red[w];
    p.partial[blockIdx.x] = t;
    __threadfence();
    last = atomicAdd(p.counter, 1u) == gridDim.x - 1;
  }
  __syncthreads();
  if (last && threadIdx.x < 32) {          // the last block adds the partials in a fixed order
    __threadfence();
    float t = 0.f;
    for (unsigned int g = threadIdx.x; g < gridDim.x; g += 32) t += __ldcg(p.partial + g);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
    if (threadIdx.x == 0) {
      *p.out = t;
      *p.counter = 0u;
    }
  }
}

// Few innermost entries (the channels of a channels-last prediction): one thread per pixel.  The
// prediction is read and its gradient written as one short run per thread, consecutive threads take
// consecutive pixels, so each of the target's channel planes is read coalesced; the index is taken
// apart once per pixel.
template <bool BWD>
__global__ void __launch_bounds__(256) mse_pix_kernel(const MseArgs p) {
  const int C = p.size[3];
  const unsigned int s2 = p.size[2], s1 = p.size[1];
  const long long pixels = p.numel / C;
  const float k = BWD ? __ldg(p.scale) : 0.f;
  float s = 0.f;
  for (long long j = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; j < pixels;
       j += static_cast<long long>(gridDim.x) * blockDim.x) {
    long long r = j;
    const long long i2 = r % s2; r /= s2;
    const long long i1 = r % s1;
    const long long i0 = r / s1;
    const long long ob = i0 * p.b.stride[0] + i1 * p.b.stride[1] + i2 * p.b.stride[2];
    const long long oa = j * C;
    for (int c = 0; c < C; ++c) {
      const float av = load_strided(p.a, oa + c), bv = load_strided(p.b, ob + c * p.b.stride[3]);
      if (BWD) {
        const float gv = k * pair_grad(p.op, av, bv, p.beta);
        if (p.ga_bf16) static_cast<__nv_bfloat16*>(p.ga)[oa + c] = __float2bfloat16(gv);
        else static_cast<float*>(p.ga)[oa + c] = gv;
      } else {
        s += pair_value(p.op, av, bv, p.beta);
      }
    }
  }
  if (BWD) return;
  __shared__ float red[8];
  __shared__ bool last;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = s;
  __syncthreads();
  if (threadIdx.x == 0) {
    float t = 0.f;
    for (int w = 0; w < 8; ++w) t += red[w];
    p.partial[blockIdx.x] = t;
    __threadfence();
    last = atomicAdd(p.counter, 1u) == gridDim.x - 1;
  }
  __syncthreads();
  if (last && threadIdx.x < 32) {
    __threadfence();
    float t = 0.f;
    for (unsigned int g = threadIdx.x; g < gridDim.x; g += 32) t += __ldcg(p.partial + g);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
    if (threadIdx.x == 0) {
      *p.out = t;
      *p.counter = 0u;
    }
  }
}

__global__ void __launch_bounds__(256) mse_bwd_kernel(const MseArgs p) {
  const float k = __ldg(p.scale);
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < p.numel;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    long long oa, ob;
    mse_offsets(p, i, &oa, &ob);
    const float g = k * pair_grad(p.op, load_strided(p.a, oa), load_strided(p.b, ob), p.beta);
    if (p.ga_bf16) static_cast<__nv_bfloat16*>(p.ga)[oa] = __float2bfloat16(g);
    else static_cast<float*>(p.ga)[oa] = g;
  }
}

// ------------------------------------------------------------------------------------------
// Multi-tensor Adam / AdamW: one launch updates up to ADAM_MAX_TENSORS fp32 parameters.
// `step` is a device scalar holding the number of the step being taken (already incremented),
// so the launch can sit in a CUDA graph.
// ------------------------------------------------------------------------------------------
constexpr int ADAM_MAX_TENSORS = 48;
constexpr int ADAM_CHUNK = 4096;   // elements per block

struct AdamTable {
  float* p[ADAM_MAX_TENSORS];
  const float* g[ADAM_MAX_TENSORS];
  float* m[ADAM_MAX_TENSORS];
  float* v[ADAM_MAX_TENSORS];
  int first_chunk[ADAM_MAX_TENSORS + 1];   // prefix sums of chunks per tensor
  long long numel[ADAM_MAX_TENSORS];
  int count;
};

struct AdamHyper {
  float lr, beta1, beta2, eps, weight_decay;
  int decoupled;          // 1: AdamW
  int maximize;
  const float* step;      // device scalar
  const float* grad_scale;  // optional device scalar multiplied into every gradient (clipping), may be null
};

__device__ __forceinline__ void adam_update(const AdamTable& t, const AdamHyper& h, const float lr) {
  // which tensor does this block's chunk belong to (few tensors: linear scan)
  int ti = 0;
  while (ti + 1 < t.count && static_cast<int>(blockIdx.x) >= t.first_chunk[ti + 1]) ++ti;
  const long long base = static_cast<long long>(blockIdx.x - t.first_chunk[ti]) * ADAM_CHUNK;
  const long long n = t.numel[ti];
  const float step = __ldg(h.step);
  const float c1 = 1.f - __powf(h.beta1, step);
  const float c2 = 1.f - __powf(h.beta2, step);
  const float step_size = lr / c1;
  const float inv_sqrt_c2 = rsqrtf(c2);
  const float gs = h.grad_scale != nullptr ? __ldg(h.grad_scale) : 1.f;
  float* p = t.p[ti];
  const float* g = t.g[ti];
  float* m = t.m[ti];
  float* v = t.v[ti];
  for (long long i = base + threadIdx.x; i < n && i < base + ADAM_CHUNK; i += 256) {
    float grad = g[i] * gs;
    if (h.maximize) grad = -grad;
    float w = p[i];
    if (h.weight_decay != 0.f) {
      if (h.decoupled) w *= 1.f - lr * h.weight_decay;
      else grad += h.weight_decay * w;
    }
    const float mi = h.beta1 * m[i] + (1.f - h.beta1) * grad;
    const float vi = h.beta2 * v[i] + (1.f - h.beta2) * grad * grad;
    m[i] = mi;
    v[i] = vi;
    p[i] = w - step_size * mi / (sqrtf(vi) * inv_sqrt_c2 + h.eps);
  }
}

__global__ void __launch_bounds__(256) adam_kernel(const __grid_constant__ AdamTable t, const AdamHyper h) {
  adam_update(t, h, h.lr);
}

// The same update with the learning rate read from device memory, so that a schedule can change it between
// replays of a CUDA graph that captured the launch.
__global__ void __launch_bounds__(256) adam_lr_kernel(const __grid_constant__ AdamTable t, const AdamHyper h,
                                                      const float* __restrict__ lr) {
  adam_update(t, h, __ldg(lr));
}

// Sum of squares of up to ADAM_MAX_TENSORS tensors (gradient norm): per-block partials, then the
// last block reduces them in a fixed order and accumulates into out[0].
__global__ void __launch_bounds__(256) sumsq_kernel(const __grid_constant__ AdamTable t, float* partial,
                                                    unsigned int* counter, float* out) {
  int ti = 0;
  while (ti + 1 < t.count && static_cast<int>(blockIdx.x) >= t.first_chunk[ti + 1]) ++ti;
  const long long base = static_cast<long long>(blockIdx.x - t.first_chunk[ti]) * ADAM_CHUNK;
  const long long n = t.numel[ti];
  const float* g = t.g[ti];
  float s = 0.f;
  for (long long i = base + threadIdx.x; i < n && i < base + ADAM_CHUNK; i += 256) s += g[i] * g[i];
  __shared__ float red[8];
  __shared__ bool last;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = s;
  __syncthreads();
  if (threadIdx.x == 0) {
    float r = 0.f;
    for (int w = 0; w < 8; ++w) r += red[w];
    partial[blockIdx.x] = r;
    __threadfence();
    last = atomicAdd(counter, 1u) == gridDim.x - 1;
  }
  __syncthreads();
  if (last && threadIdx.x < 32) {
    __threadfence();
    float r = 0.f;
    for (unsigned int b = threadIdx.x; b < gridDim.x; b += 32) r += __ldcg(partial + b);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) r += __shfl_xor_sync(0xffffffffu, r, o);
    if (threadIdx.x == 0) {
      *out += r;
      *counter = 0u;
    }
  }
}

__global__ void incr_kernel(float* x) { *x += 1.f; }

}  // namespace jb

using namespace jb;

extern "C" int jb_merge_chunks(float* o1, float* l1, const void* o2, int o2_bf16, const float* l2, long long rows,
                               int d, void* stream) {
  if (rows <= 0 || d <= 0) return -1;
  // vector variant: rows must not straddle warps (32 % (d / 4) == 0), so that all readers of a row's
  // log-sum-exp pass the warp barrier before its writer stores the new value
  const bool vec = (d % 4 == 0) && (d / 4 <= 32) && (32 % (d / 4) == 0);
  if (vec) {
    const long long threads = rows * (d / 4);
    const unsigned int grid = static_cast<unsigned int>((threads + 255) / 256);
    merge_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(o1, l1, o2, o2_bf16, l2, rows, d);
  } else {
    const long long threads = rows * 32;
    const unsigned int grid = static_cast<unsigned int>((threads + 255) / 256);
    merge_rows_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(o1, l1, o2, o2_bf16, l2, rows, d);
  }
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

struct JbStrided4 {
  const void* ptr;
  int is_bf16;
  long long stride[4];
};

static void mse_fill(MseArgs* p, const JbStrided4* a, const JbStrided4* b, const int* size) {
  p->a.ptr = a->ptr; p->a.is_bf16 = a->is_bf16;
  p->b.ptr = b->ptr; p->b.is_bf16 = b->is_bf16;
  p->numel = 1;
  for (int i = 0; i < 4; ++i) {
    p->a.stride[i] = a->stride[i];
    p->b.stride[i] = b->stride[i];
    p->size[i] = size[i];
    p->numel *= size[i];
  }
  long long expect = 1;
  p->a_dense = 1;
  for (int i = 3; i >= 0; --i) {
    if (size[i] != 1 && a->stride[i] != expect) p->a_dense = 0;
    expect *= size[i];
  }
}

extern "C" int jb_mse_grid(long long numel, int sm_count) {
  const long long want = (numel + 256 * 8 - 1) / (256 * 8);
  const long long cap = static_cast<long long>(sm_count) * 8;
  return static_cast<int>(want < 1 ? 1 : (want < cap ? want : cap));
}

// out[0] = sum f(a, b), f chosen by op (0 squared error, 1 absolute error, 2 smooth L1 with `beta`, 3 binary
// cross-entropy of probabilities, 4 of logits).  partial: jb_mse_grid() floats; counter: zeroed word (left zero).
extern "C" int jb_pair_loss_sum(const JbStrided4* a, const JbStrided4* b, const int* size, int op, float beta,
                                float* partial, unsigned int* counter, float* out, int sm_count, void* stream) {
  MseArgs p{};
  mse_fill(&p, a, b, size);
  if (p.numel <= 0 || op < 0 || op > 4 || (op == PAIR_SMOOTH_L1 && !(beta > 0.f))) return -1;
  p.op = op; p.beta = beta;
  p.partial = partial; p.counter = counter; p.out = out;
  if (p.a_dense && p.size[3] <= 4)
    mse_pix_kernel<false><<<jb_mse_grid(p.numel, sm_count), 256, 0, static_cast<cudaStream_t>(stream)>>>(p);
  else
    mse_fwd_kernel<<<jb_mse_grid(p.numel, sm_count), 256, 0, static_cast<cudaStream_t>(stream)>>>(p);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

// ga = scale[0] * df/da, written with the strides of a.
extern "C" int jb_pair_loss_grad(const JbStrided4* a, const JbStrided4* b, const int* size, int op, float beta,
                                 const float* scale, void* ga, int ga_bf16, int sm_count, void* stream) {
  MseArgs p{};
  mse_fill(&p, a, b, size);
  if (p.numel <= 0 || op < 0 || op > 4 || (op == PAIR_SMOOTH_L1 && !(beta > 0.f))) return -1;
  p.op = op; p.beta = beta;
  p.scale = scale; p.ga = ga; p.ga_bf16 = ga_bf16;
  if (p.a_dense && p.size[3] <= 4)
    mse_pix_kernel<true><<<jb_mse_grid(p.numel, sm_count), 256, 0, static_cast<cudaStream_t>(stream)>>>(p);
  else
    mse_bwd_kernel<<<jb_mse_grid(p.numel, sm_count), 256, 0, static_cast<cudaStream_t>(stream)>>>(p);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

struct JbAdamTensors {
  void* p[48];
  const void* g[48];
  void* m[48];
  void* v[48];
  long long numel[48];
  int count;
};

static int adam_table(AdamTable* t, const JbAdamTensors* in) {
  if (in->count <= 0 || in->count > ADAM_MAX_TENSORS) return -1;
  t->count = in->count;
  int chunks = 0;
  for (int i = 0; i < in->count; ++i) {
    t->p[i] = static_cast<float*>(in->p[i]);
    t->g[i] = static_cast<const float*>(in->g[i]);
    t->m[i] = static_cast<float*>(in->m[i]);
    t->v[i] = static_cast<float*>(in->v[i]);
    t->numel[i] = in->numel[i];
    t->first_chunk[i] = chunks;
    chunks += static_cast<int>((in->numel[i] + ADAM_CHUNK - 1) / ADAM_CHUNK);
  }
  t->first_chunk[in->count] = chunks;
  return chunks;
}

extern "C" int jb_increment(float* x, void* stream) {
  incr_kernel<<<1, 1, 0, static_cast<cudaStream_t>(stream)>>>(x);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

// One Adam / AdamW step for up to 48 fp32 tensors; `step` holds the (already incremented) step number.
extern "C" int jb_adam_multi(const JbAdamTensors* tensors, float lr, float beta1, float beta2, float eps,
                             float weight_decay, int decoupled, int maximize, const float* step,
                             const float* grad_scale, void* stream) {
  AdamTable t{};
  const int chunks = adam_table(&t, tensors);
  if (chunks <= 0) return -1;
  AdamHyper h{lr, beta1, beta2, eps, weight_decay, decoupled, maximize, step, grad_scale};
  adam_kernel<<<chunks, 256, 0, static_cast<cudaStream_t>(stream)>>>(t, h);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

// The same step with the learning rate in device memory (`lr`: one float).
extern "C" int jb_adam_multi_lr(const JbAdamTensors* tensors, const float* lr, float beta1, float beta2, float eps,
                                float weight_decay, int decoupled, int maximize, const float* step,
                                const float* grad_scale, void* stream) {
  AdamTable t{};
  const int chunks = adam_table(&t, tensors);
  if (chunks <= 0 || lr == nullptr) return -1;
  AdamHyper h{0.f, beta1, beta2, eps, weight_decay, decoupled, maximize, step, grad_scale};
  adam_lr_kernel<<<chunks, 256, 0, static_cast<cudaStream_t>(stream)>>>(t, h, lr);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

// out[0] += sum over the tensors' g of g^2.  partial: one float per chunk (jb_chunks()); counter zeroed.
extern "C" int jb_sumsq_multi(const JbAdamTensors* tensors, float* partial, unsigned int* counter, float* out,
                              void* stream) {
  AdamTable t{};
  const int chunks = adam_table(&t, tensors);
  if (chunks <= 0) return -1;
  sumsq_kernel<<<chunks, 256, 0, static_cast<cudaStream_t>(stream)>>>(t, partial, counter, out);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

extern "C" int jb_chunks(long long numel) { return static_cast<int>((numel + ADAM_CHUNK - 1) / ADAM_CHUNK); }
