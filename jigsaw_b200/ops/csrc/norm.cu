// LayerNorm over a feature dimension that is split across GPUs, forward and backward, each as ONE
// kernel: local row statistics -> exchange with the other column ranks through peer memory ->
// normalisation.  The exchange is a push: every rank stores its per-row partials straight into the
// inboxes of its peers (plain stores over NVLink), publishes an epoch flag per CTA, and waits
// (bounded) for the flags of the same CTA index on the peers, which by construction handles the same
// rows.  Grids never exceed the number of co-resident CTAs, so a waiting CTA cannot starve the CTA
// it waits for.  Rows are re-read from L2 for the second phase.
//
// Statistics are combined with the parallel-variance formula (equal counts per rank):
//   mean = sum_p mean_p / P,   M2 = sum_p M2_p + n * sum_p (mean_p - mean)^2,   var = M2 / (n P)
// which matches the two-pass (mean, then centred second moment) definition.
//
// Backward: dx = rstd * (g w - S1 / N - xhat * S2 / N) with S1 = sum g w, S2 = sum g w xhat over the
// global feature dimension (exchanged the same way); dw = sum_rows g xhat and db = sum_rows g are
// accumulated per CTA in shared memory and reduced by a second small kernel.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "ptx.cuh"

namespace jb {

constexpr int LN_THREADS = 256;
constexpr int LN_WARPS = LN_THREADS / 32;
constexpr int LN_MAX_PARTS = 8;
constexpr int LN_REG_CHUNKS = 8;     // columns per lane kept in registers by the backward kernel (n <= 1024)

struct LnExchange {
  float* inbox_local;               // [2][P][R][2] this rank's inbox (parity, source rank, row, value)
  float* inbox_peer[LN_MAX_PARTS];  // the same buffer on every column rank (entry of this rank unused)
  uint32_t* flag_local;             // [P][grid]
  uint32_t* flag_peer[LN_MAX_PARTS];
  uint32_t epoch;                   // value to publish; its parity selects the inbox half
  uint32_t stride;                  // CUDA-graph replays: see live_epoch()
  const uint32_t* replay;
  int parts, me;
};

struct LnArgs {
  const void* x; int x_bf16;
  const void* g; int g_bf16;        // backward only: upstream gradient
  void* out; int out_bf16;          // forward: y; backward: dx
  const float* w; const float* b;   // local slices, may be null
  float* mean; float* rstd;         // [R]: written by forward, read by backward
  float* dw_part; float* db_part;   // backward: [grid][n]
  int R, n;
  float eps;
  LnExchange ex;
  int* status;
};

__device__ __forceinline__ float4 ln_load4(const void* base, int is_bf16, long long idx) {
  if (is_bf16) {
    const uint2 v = *reinterpret_cast<const uint2*>(static_cast<const __nv_bfloat16*>(base) + idx);
    const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&v.x);
    const __nv_bfloat162 b = *reinterpret_cast<const __nv_bfloat162*>(&v.y);
    return make_float4(__low2float(a), __high2float(a), __low2float(b), __high2float(b));
  }
  return *reinterpret_cast<const float4*>(static_cast<const float*>(base) + idx);
}

__device__ __forceinline__ void ln_store4(void* base, int is_bf16, long long idx, float4 v) {
  if (is_bf16) {
    uint2 o;
    o.x = pack_bf16x2(v.x, v.y);
    o.y = pack_bf16x2(v.z, v.w);
    *reinterpret_cast<uint2*>(static_cast<__nv_bfloat16*>(base) + idx) = o;
  } else {
    *reinterpret_cast<float4*>(static_cast<float*>(base) + idx) = v;
  }
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// Publish this CTA's partials and wait for the same CTA of every peer.  Returns false after a
// timeout (status is set; the caller still finishes with whatever is in the inbox).
__device__ __forceinline__ bool ln_exchange(const LnExchange& ex, uint32_t epoch, int* status) {
  __threadfence_system();          // this thread's peer stores first
  __syncthreads();
  __shared__ int ok;
  if (threadIdx.x == 0) ok = 1;
  __syncthreads();
  if (threadIdx.x < ex.parts && static_cast<int>(threadIdx.x) != ex.me) {
    const int p = threadIdx.x;
    uint32_t* out = ex.flag_peer[p] + static_cast<size_t>(ex.me) * gridDim.x + blockIdx.x;
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(out), "r"(epoch) : "memory");
    const uint32_t* in = ex.flag_local + static_cast<size_t>(p) * gridDim.x + blockIdx.x;
    const uint64_t t0 = globaltimer_ns();
    while (true) {
      uint32_t v;
      asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(in) : "memory");
      if (static_cast<int32_t>(v - epoch) >= 0) break;
      if (globaltimer_ns() - t0 > JB_WAIT_LIMIT_NS) {
        if (status) atomicCAS(status, JB_OK, JB_ERR_FLAG_TIMEOUT);
        ok = 0;
        break;
      }
      __nanosleep(64);
    }
  }
  __syncthreads();
  return ok != 0;
}

// rows of this CTA: a contiguous chunk
__device__ __forceinline__ void ln_rows(int R, int* r0, int* r1) {
  const int per = (R + gridDim.x - 1) / gridDim.x;
  *r0 = min(R, static_cast<int>(blockIdx.x) * per);
  *r1 = min(R, *r0 + per);
}

__global__ void __launch_bounds__(LN_THREADS) ln_fwd_kernel(const LnArgs a) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  int r0, r1;
  ln_rows(a.R, &r0, &r1);
  const LnExchange& ex = a.ex;
  const int P = ex.parts;
  const uint32_t epoch = live_epoch(ex.epoch, ex.stride, ex.replay);
  const size_t half = static_cast<size_t>(epoch & 1u) * P * a.R * 2;
  const float inv_n = 1.f / static_cast<float>(a.n);
  if (P == 1 && a.n <= LN_REG_CHUNKS * 128) {
    // unsplit feature dimension: the row stays in registers between the statistics and the normalisation
    const int chunks = (a.n + 127) / 128;
    for (int r = r0 + warp; r < r1; r += LN_WARPS) {
      const long long base = static_cast<long long>(r) * a.n;
      float4 v[LN_REG_CHUNKS];
      float s = 0.f;
#pragma unroll
      for (int k = 0; k < LN_REG_CHUNKS; ++k) {
        const int i = lane * 4 + k * 128;
        v[k] = (k < chunks && i < a.n) ? ln_load4(a.x, a.x_bf16, base + i) : make_float4(0.f, 0.f, 0.f, 0.f);
        s += (v[k].x + v[k].y) + (v[k].z + v[k].w);
      }
      const float mean = warp_sum(s) * inv_n;
      float q = 0.f;
#pragma unroll
      for (int k = 0; k < LN_REG_CHUNKS; ++k) {
        const int i = lane * 4 + k * 128;
        if (k < chunks && i < a.n) {
          const float d0 = v[k].x - mean, d1 = v[k].y - mean, d2 = v[k].z - mean, d3 = v[k].w - mean;
          q += (d0 * d0 + d1 * d1) + (d2 * d2 + d3 * d3);
        }
      }
      const float rstd = rsqrtf(warp_sum(q) * inv_n + a.eps);
      if (lane == 0) {
        a.mean[r] = mean;
        a.rstd[r] = rstd;
      }
#pragma unroll
      for (int k = 0; k < LN_REG_CHUNKS; ++k) {
        const int i = lane * 4 + k * 128;
        if (k < chunks && i < a.n) {
          float4 o = v[k];
          o.x = (o.x - mean) * rstd; o.y = (o.y - mean) * rstd; o.z = (o.z - mean) * rstd; o.w = (o.w - mean) * rstd;
          if (a.w != nullptr) {
            const float4 w = *reinterpret_cast<const float4*>(a.w + i);
            o.x *= w.x; o.y *= w.y; o.z *= w.z; o.w *= w.w;
          }
          if (a.b != nullptr) {
            const float4 b = *reinterpret_cast<const float4*>(a.b + i);
            o.x += b.x; o.y += b.y; o.z += b.z; o.w += b.w;
          }
          ln_store4(a.out, a.out_bf16, base + i, o);
        }
      }
    }
    return;
  }
  // ---- phase 1: local mean and centred second moment of every row
  for (int r = r0 + warp; r < r1; r += LN_WARPS) {
    const long long base = static_cast<long long>(r) * a.n;
    float s = 0.f;
    for (int i = lane * 4; i < a.n; i += 128) {
      const float4 v = ln_load4(a.x, a.x_bf16, base + i);
      s += (v.x + v.y) + (v.z + v.w);
    }
    const float mean_l = warp_sum(s) * inv_n;
    float q = 0.f;
    for (int i = lane * 4; i < a.n; i += 128) {
      const float4 v = ln_load4(a.x, a.x_bf16, base + i);
      const float d0 = v.x - mean_l, d1 = v.y - mean_l, d2 = v.z - mean_l, d3 = v.w - mean_l;
      q += (d0 * d0 + d1 * d1) + (d2 * d2 + d3 * d3);
    }
    const float m2_l = warp_sum(q);
    if (P == 1) {
      if (lane == 0) {
        a.mean[r] = mean_l;
        a.rstd[r] = rsqrtf(m2_l * inv_n + a.eps);
      }
    } else if (lane < P) {
      const size_t slot = half + (static_cast<size_t>(ex.me) * a.R + r) * 2;
      float* dst = (lane == ex.me) ? ex.inbox_local : ex.inbox_peer[lane];
      *reinterpret_cast<float2*>(dst + slot) = make_float2(mean_l, m2_l);
    }
  }
  if (P > 1) {
    ln_exchange(ex, epoch, a.status);
    for (int r = r0 + warp; r < r1; r += LN_WARPS) {
      float mp = 0.f, m2p = 0.f;
      if (lane < P) {
        const float2 v = __ldcg(reinterpret_cast<const float2*>(
            ex.inbox_local + half + (static_cast<size_t>(lane) * a.R + r) * 2));
        mp = v.x;
        m2p = v.y;
      }
      const float mean = warp_sum(mp) / static_cast<float>(P);
      const float d = (lane < P) ? (mp - mean) : 0.f;
      const float m2 = warp_sum(m2p + static_cast<float>(a.n) * d * d);
      if (lane == 0) {
        a.mean[r] = mean;
        a.rstd[r] = rsqrtf(m2 * inv_n / static_cast<float>(P) + a.eps);
      }
    }
  }
  __syncwarp();
  // ---- phase 2: normalise (each warp re-reads the statistics it wrote itself)
  for (int r = r0 + warp; r < r1; r += LN_WARPS) {
    const long long base = static_cast<long long>(r) * a.n;
    const float mean = a.mean[r], rstd = a.rstd[r];
    for (int i = lane * 4; i < a.n; i += 128) {
      float4 v = ln_load4(a.x, a.x_bf16, base + i);
      v.x = (v.x - mean) * rstd; v.y = (v.y - mean) * rstd; v.z = (v.z - mean) * rstd; v.w = (v.w - mean) * rstd;
      if (a.w != nullptr) {
        const float4 w = *reinterpret_cast<const float4*>(a.w + i);
        v.x *= w.x; v.y *= w.y; v.z *= w.z; v.w *= w.w;
      }
      if (a.b != nullptr) {
        const float4 b = *reinterpret_cast<const float4*>(a.b + i);
        v.x += b.x; v.y += b.y; v.z += b.z; v.w += b.w;
      }
      ln_store4(a.out, a.out_bf16, base + i, v);
    }
  }
}

template <bool WANT_DW>
__global__ void __launch_bounds__(LN_THREADS, WANT_DW ? 1 : 3) ln_bwd_kernel(const LnArgs a) {
  extern __shared__ float acc[];   // [2][n]: dw, db partials of this CTA
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  int r0, r1;
  ln_rows(a.R, &r0, &r1);
  const LnExchange& ex = a.ex;
  const int P = ex.parts;
  const uint32_t epoch = live_epoch(ex.epoch, ex.stride, ex.replay);
  const size_t half = static_cast<size_t>(epoch & 1u) * P * a.R * 2;
  constexpr bool want_dw = WANT_DW;
  if (want_dw)
    for (int i = threadIdx.x; i < 2 * a.n; i += LN_THREADS) acc[i] = 0.f;
  __syncthreads();
  float4 rdw[WANT_DW ? LN_REG_CHUNKS : 1], rdb[WANT_DW ? LN_REG_CHUNKS : 1];
#pragma unroll
  for (int k = 0; k < (WANT_DW ? LN_REG_CHUNKS : 1); ++k) rdw[k] = rdb[k] = make_float4(0.f, 0.f, 0.f, 0.f);
  const float inv_N = 1.f / (static_cast<float>(a.n) * static_cast<float>(P));
  if (P == 1 && a.n <= LN_REG_CHUNKS * 128) {
    // unsplit feature dimension: x and g of a row stay in registers between the two reductions and dx
    const int chunks = (a.n + 127) / 128;
    for (int r = r0 + warp; r < r1; r += LN_WARPS) {
      const long long base = static_cast<long long>(r) * a.n;
      const float mean = a.mean[r], rstd = a.rstd[r];
      float4 hx[LN_REG_CHUNKS], gw[LN_REG_CHUNKS];
      float s1 = 0.f, s2 = 0.f;
#pragma unroll
      for (int k = 0; k < LN_REG_CHUNKS; ++k) {
        const int i = lane * 4 + k * 128;
        hx[k] = gw[k] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (k < chunks && i < a.n) {
          const float4 x = ln_load4(a.x, a.x_bf16, base + i);
          const float4 g = ln_load4(a.g, a.g_bf16, base + i);
          float4 w = make_float4(1.f, 1.f, 1.f, 1.f);
          if (a.w != nullptr) w = *reinterpret_cast<const float4*>(a.w + i);
          hx[k] = make_float4((x.x - mean) * rstd, (x.y - mean) * rstd, (x.z - mean) * rstd, (x.w - mean) * rstd);
          if constexpr (WANT_DW) {
            rdw[k].x += g.x * hx[k].x; rdw[k].y += g.y * hx[k].y; rdw[k].z += g.z * hx[k].z; rdw[k].w += g.w * hx[k].w;
            rdb[k].x += g.x; rdb[k].y += g.y; rdb[k].z += g.z; rdb[k].w += g.w;
          }
          gw[k] = make_float4(g.x * w.x, g.y * w.y, g.z * w.z, g.w * w.w);
          s1 += (gw[k].x + gw[k].y) + (gw[k].z + gw[k].w);
          s2 += (gw[k].x * hx[k].x + gw[k].y * hx[k].y) + (gw[k].z * hx[k].z + gw[k].w * hx[k].w);
        }
      }
      const float S1 = warp_sum(s1) * inv_N, S2 = warp_sum(s2) * inv_N;
#pragma unroll
      for (int k = 0; k < LN_REG_CHUNKS; ++k) {
        const int i = lane * 4 + k * 128;
        if (k < chunks && i < a.n) {
          float4 d;
          d.x = rstd * (gw[k].x - S1 - hx[k].x * S2);
          d.y = rstd * (gw[k].y - S1 - hx[k].y * S2);
          d.z = rstd * (gw[k].z - S1 - hx[k].z * S2);
          d.w = rstd * (gw[k].w - S1 - hx[k].w * S2);
          ln_store4(a.out, a.out_bf16, base + i, d);
        }
      }
    }
  } else {
  // ---- phase 1: S1 = sum g w, S2 = sum g w xhat per row (local part); dw / db partials
  for (int r = r0 + warp; r < r1; r += LN_WARPS) {
    const long long base = static_cast<long long>(r) * a.n;
    const float mean = a.mean[r], rstd = a.rstd[r];
    float s1 = 0.f, s2 = 0.f;
    // columns [0, LN_REG_CHUNKS * 128): sums for dw / db in registers (constant trip count, so the
    // accumulators are never indexed dynamically); columns beyond: shared-memory adds
#pragma unroll
    for (int k = 0; k < LN_REG_CHUNKS; ++k) {
      const int i = lane * 4 + k * 128;
      if (i < a.n) {
        const float4 x = ln_load4(a.x, a.x_bf16, base + i);
        const float4 g = ln_load4(a.g, a.g_bf16, base + i);
        float4 w = make_float4(1.f, 1.f, 1.f, 1.f);
        if (a.w != nullptr) w = *reinterpret_cast<const float4*>(a.w + i);
        const float h0 = (x.x - mean) * rstd, h1 = (x.y - mean) * rstd, h2 = (x.z - mean) * rstd, h3 = (x.w - mean) * rstd;
        const float gw0 = g.x * w.x, gw1 = g.y * w.y, gw2 = g.z * w.z, gw3 = g.w * w.w;
        s1 += (gw0 + gw1) + (gw2 + gw3);
        s2 += (gw0 * h0 + gw1 * h1) + (gw2 * h2 + gw3 * h3);
        if constexpr (WANT_DW) {
          rdw[k].x += g.x * h0; rdw[k].y += g.y * h1; rdw[k].z += g.z * h2; rdw[k].w += g.w * h3;
          rdb[k].x += g.x; rdb[k].y += g.y; rdb[k].z += g.z; rdb[k].w += g.w;
        }
      }
    }
    for (int i = lane * 4 + LN_REG_CHUNKS * 128; i < a.n; i += 128) {
      const float4 x = ln_load4(a.x, a.x_bf16, base + i);
      const float4 g = ln_load4(a.g, a.g_bf16, base + i);
      float4 w = make_float4(1.f, 1.f, 1.f, 1.f);
      if (a.w != nullptr) w = *reinterpret_cast<const float4*>(a.w + i);
      const float h0 = (x.x - mean) * rstd, h1 = (x.y - mean) * rstd, h2 = (x.z - mean) * rstd, h3 = (x.w - mean) * rstd;
      const float gw0 = g.x * w.x, gw1 = g.y * w.y, gw2 = g.z * w.z, gw3 = g.w * w.w;
      s1 += (gw0 + gw1) + (gw2 + gw3);
      s2 += (gw0 * h0 + gw1 * h1) + (gw2 * h2 + gw3 * h3);
      if (want_dw) {
        atomicAdd(acc + i + 0, g.x * h0); atomicAdd(acc + i + 1, g.y * h1);
        atomicAdd(acc + i + 2, g.z * h2); atomicAdd(acc + i + 3, g.w * h3);
        atomicAdd(acc + a.n + i + 0, g.x); atomicAdd(acc + a.n + i + 1, g.y);
        atomicAdd(acc + a.n + i + 2, g.z); atomicAdd(acc + a.n + i + 3, g.w);
      }
    }
    s1 = warp_sum(s1);
    s2 = warp_sum(s2);
    if (lane < P) {
      const size_t slot = half + (static_cast<size_t>(ex.me) * a.R + r) * 2;
      float* dst = (P == 1 || lane == ex.me) ? ex.inbox_local : ex.inbox_peer[lane];
      *reinterpret_cast<float2*>(dst + slot) = make_float2(s1, s2);
    }
  }
  if (P > 1) ln_exchange(ex, epoch, a.status);
  else __syncwarp();
  // ---- phase 2: dx
  for (int r = r0 + warp; r < r1; r += LN_WARPS) {
    const long long base = static_cast<long long>(r) * a.n;
    const float mean = a.mean[r], rstd = a.rstd[r];
    float p1 = 0.f, p2 = 0.f;
    if (lane < P) {
      const float2 v = __ldcg(reinterpret_cast<const float2*>(
          ex.inbox_local + half + (static_cast<size_t>(lane) * a.R + r) * 2));
      p1 = v.x;
      p2 = v.y;
    }
    const float S1 = warp_sum(p1) * inv_N, S2 = warp_sum(p2) * inv_N;
    for (int i = lane * 4; i < a.n; i += 128) {
      const float4 x = ln_load4(a.x, a.x_bf16, base + i);
      const float4 g = ln_load4(a.g, a.g_bf16, base + i);
      float4 w = make_float4(1.f, 1.f, 1.f, 1.f);
      if (a.w != nullptr) w = *reinterpret_cast<const float4*>(a.w + i);
      float4 d;
      d.x = rstd * (g.x * w.x - S1 - (x.x - mean) * rstd * S2);
      d.y = rstd * (g.y * w.y - S1 - (x.y - mean) * rstd * S2);
      d.z = rstd * (g.z * w.z - S1 - (x.z - mean) * rstd * S2);
      d.w = rstd * (g.w * w.w - S1 - (x.w - mean) * rstd * S2);
      ln_store4(a.out, a.out_bf16, base + i, d);
    }
  }
  }   // split feature dimension
  if constexpr (WANT_DW) {
#pragma unroll
    for (int k = 0; k < LN_REG_CHUNKS; ++k) {        // one shared-memory add per warp and column
      const int i = lane * 4 + k * 128;
      if (i < a.n) {
        atomicAdd(acc + i + 0, rdw[k].x); atomicAdd(acc + i + 1, rdw[k].y);
        atomicAdd(acc + i + 2, rdw[k].z); atomicAdd(acc + i + 3, rdw[k].w);
        atomicAdd(acc + a.n + i + 0, rdb[k].x); atomicAdd(acc + a.n + i + 1, rdb[k].y);
        atomicAdd(acc + a.n + i + 2, rdb[k].z); atomicAdd(acc + a.n + i + 3, rdb[k].w);
      }
    }
    __syncthreads();
    for (int i = threadIdx.x; i < a.n; i += LN_THREADS) {
      a.dw_part[static_cast<size_t>(blockIdx.x) * a.n + i] = acc[i];
      a.db_part[static_cast<size_t>(blockIdx.x) * a.n + i] = acc[a.n + i];
    }
  }
}

// dw / db partial sums of LayerNorm: a CTA owns 128 columns and a slab of rows; 32 column lanes (four
// columns each, so a warp reads 256 or 512 consecutive bytes of a row) times 8 row lanes.
constexpr int LN_COL_ROWS = 512;   // rows per slab
__global__ void __launch_bounds__(256) ln_dwdb_kernel(const LnArgs a) {
  __shared__ float4 red[2][8][32];
  const int cl = threadIdx.x & 31, rl = threadIdx.x >> 5;
  const int i = blockIdx.x * 128 + cl * 4;
  const int r0 = blockIdx.y * LN_COL_ROWS;
  const int r1 = min(a.R, r0 + LN_COL_ROWS);
  float4 dw = make_float4(0.f, 0.f, 0.f, 0.f), db = dw;
  if (i < a.n) {
#pragma unroll 4
    for (int r = r0 + rl; r < r1; r += 8) {
      const long long base = static_cast<long long>(r) * a.n + i;
      const float4 x = ln_load4(a.x, a.x_bf16, base);
      const float4 g = ln_load4(a.g, a.g_bf16, base);
      const float mean = __ldg(a.mean + r), rstd = __ldg(a.rstd + r);
      dw.x += g.x * (x.x - mean) * rstd; dw.y += g.y * (x.y - mean) * rstd;
      dw.z += g.z * (x.z - mean) * rstd; dw.w += g.w * (x.w - mean) * rstd;
      db.x += g.x; db.y += g.y; db.z += g.z; db.w += g.w;
    }
  }
  red[0][rl][cl] = dw;
  red[1][rl][cl] = db;
  __syncthreads();
  if (rl == 0 && i < a.n) {
    float4 sw = red[0][0][cl], sb = red[1][0][cl];
#pragma unroll
    for (int k = 1; k < 8; ++k) {
      const float4 u = red[0][k][cl], v = red[1][k][cl];
      sw.x += u.x; sw.y += u.y; sw.z += u.z; sw.w += u.w;
      sb.x += v.x; sb.y += v.y; sb.z += v.z; sb.w += v.w;
    }
    *reinterpret_cast<float4*>(a.dw_part + static_cast<size_t>(blockIdx.y) * a.n + i) = sw;
    *reinterpret_cast<float4*>(a.db_part + static_cast<size_t>(blockIdx.y) * a.n + i) = sb;
  }
}

// out[i] = sum_g part[g][i]   (deterministic order)
__global__ void ln_colsum_kernel(const float* __restrict__ p0, const float* __restrict__ p1, int G, int n,
                                 float* __restrict__ o0, float* __restrict__ o1) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  float s0 = 0.f, s1 = 0.f;
  for (int g = 0; g < G; ++g) {
    s0 += p0[static_cast<size_t>(g) * n + i];
    s1 += p1[static_cast<size_t>(g) * n + i];
  }
  if (o0) o0[i] = s0;
  if (o1) o1[i] = s1;
}


// ------------------------------------------------------------------------------------------
// Softmax cross-entropy over a class dimension that is split across GPUs (index targets).
// logits are viewed as [B][C_local][S] (S = 1 for a trailing class dimension); a "row" is one
// (b, s) pair.  Each rank computes (max, sum exp, true-class logit if it owns the class) per row,
// the partials are exchanged like the LayerNorm statistics, and every rank ends with
//   lse = M + log sum_p s_p exp(m_p - M),   loss = lse - logit[target]   (0 for ignored rows).
// Backward needs no communication: d logits = g_row (exp(x - lse) - onehot).
// ------------------------------------------------------------------------------------------
struct CeArgs {
  const void* x; int x_bf16;
  const long long* target;      // [R] global class index
  long long ignore_index;
  int B, C, S;                  // C = local classes
  int class_lo;                 // first global class of this rank
  float* loss;                  // [R]
  float* lse;                   // [R]
  const float* grow;            // backward: upstream gradient per row [R]
  void* dx; int dx_bf16;        // backward: gradient of the logits
  LnExchange ex;                // inbox slots are float4 here: [2][P][R][4]
  int* status;
};

__device__ __forceinline__ float ce_load(const CeArgs& a, long long off) {
  return a.x_bf16 ? __bfloat162float(static_cast<const __nv_bfloat16*>(a.x)[off]) : static_cast<const float*>(a.x)[off];
}

__device__ __forceinline__ void ce_row_partials(const CeArgs& a, long long r, int lane, int nl, float* m, float* s,
                                                float* t) {
  // nl = number of lanes cooperating on this row (1 or 32)
  const long long b = r / a.S, sp = r % a.S;
  const long long base = b * a.C * static_cast<long long>(a.S) + sp;
  float mx = -INFINITY;
  for (int c = lane; c < a.C; c += nl) mx = fmaxf(mx, ce_load(a, base + static_cast<long long>(c) * a.S));
  if (nl == 32) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
  }
  float sum = 0.f;
  if (mx != -INFINITY)
    for (int c = lane; c < a.C; c += nl) sum += __expf(ce_load(a, base + static_cast<long long>(c) * a.S) - mx);
  if (nl == 32) sum = warp_sum(sum);
  float tv = 0.f;
  if (a.target != nullptr) {                    // null: only the log-sum-exp is wanted (softmax / log-softmax)
    const long long tg = a.target[r] - a.class_lo;
    if (a.target[r] != a.ignore_index && tg >= 0 && tg < a.C) tv = ce_load(a, base + tg * a.S);
  }
  *m = mx; *s = sum; *t = tv;
}

template <bool WARP_PER_ROW>
__global__ void __launch_bounds__(LN_THREADS) ce_fwd_kernel(const CeArgs a) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int R = a.B * a.S;
  int r0, r1;
  ln_rows(R, &r0, &r1);
  const LnExchange& ex = a.ex;
  const int P = ex.parts;
  const uint32_t epoch = live_epoch(ex.epoch, ex.stride, ex.replay);
  const size_t half = static_cast<size_t>(epoch & 1u) * P * R * 4;
  const int first = WARP_PER_ROW ? warp : static_cast<int>(threadIdx.x);
  const int step = WARP_PER_ROW ? LN_WARPS : LN_THREADS;
  for (int r = r0 + first; r < r1; r += step) {
    float m, s, t;
    ce_row_partials(a, r, WARP_PER_ROW ? lane : 0, WARP_PER_ROW ? 32 : 1, &m, &s, &t);
    if (P == 1) {
      if (!WARP_PER_ROW || lane == 0) {
        const float lse = m + __logf(s);
        a.lse[r] = lse;
        if (a.loss != nullptr) a.loss[r] = (a.target != nullptr && a.target[r] != a.ignore_index) ? lse - t : 0.f;
      }
    } else {
      const float4 v = make_float4(m, s, t, 0.f);
      const size_t slot = half + (static_cast<size_t>(ex.me) * R + r) * 4;
      if (WARP_PER_ROW) {
        if (lane < P) {
          float* dst = (lane == ex.me) ? ex.inbox_local : ex.inbox_peer[lane];
          *reinterpret_cast<float4*>(dst + slot) = v;
        }
      } else {
        for (int p = 0; p < P; ++p) {
          float* dst = (p == ex.me) ? ex.inbox_local : ex.inbox_peer[p];
          *reinterpret_cast<float4*>(dst + slot) = v;
        }
      }
    }
  }
  if (P == 1) return;
  ln_exchange(ex, epoch, a.status);
  for (int r = r0 + static_cast<int>(threadIdx.x); r < r1; r += LN_THREADS) {
    float M = -INFINITY;
    for (int p = 0; p < P; ++p)
      M = fmaxf(M, __ldcg(ex.inbox_local + half + (static_cast<size_t>(p) * R + r) * 4));
    float S = 0.f, T = 0.f;
    for (int p = 0; p < P; ++p) {
      const float4 v = __ldcg(reinterpret_cast<const float4*>(ex.inbox_local + half + (static_cast<size_t>(p) * R + r) * 4));
      S += v.y * __expf(v.x - M);
      T += v.z;
    }
    const float lse = M + __logf(S);
    a.lse[r] = lse;
    if (a.loss != nullptr) a.loss[r] = (a.target != nullptr && a.target[r] != a.ignore_index) ? lse - T : 0.f;
  }
}

// ------------------------------------------------------------------------------------------
// Softmax / log-softmax over a class dimension that may be split across GPUs.  The row-wise
// log-sum-exp comes from ce_fwd_kernel above (null targets: local partials, in-kernel exchange,
// finish); these kernels are the element-wise rest.  x, y, g: [B][C][S]; rows are (b, s) pairs.
//   apply   : y = x - lse (log) or exp(x - lse)
//   rowdot  : d[row] = sum_c g (log) or sum_c g y   (local classes; the caller sums d over the ranks)
//   backward: dx = g - exp(y) d (log) or y (g - d)
// ------------------------------------------------------------------------------------------
struct SmArgs {
  const void* x; int x_bf16;        // apply: logits; rowdot / backward: the saved output y
  const void* g; int g_bf16;
  const float* row;                 // apply: lse; backward: d
  void* out; int out_bf16;
  float* rowout;                    // rowdot
  int B, C, S;
  int log_mode;
};

__device__ __forceinline__ float sm_load(const void* p, int bf16, long long off) {
  return bf16 ? __bfloat162float(static_cast<const __nv_bfloat16*>(p)[off]) : static_cast<const float*>(p)[off];
}
__device__ __forceinline__ void sm_store(void* p, int bf16, long long off, float v) {
  if (bf16) static_cast<__nv_bfloat16*>(p)[off] = __float2bfloat16(v);
  else static_cast<float*>(p)[off] = v;
}

template <bool BWD>
__global__ void __launch_bounds__(256) softmax_elementwise_kernel(const SmArgs a) {
  const long long cs = static_cast<long long>(a.C) * a.S;
  const long long n = cs * a.B;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long b = i / cs;
    const long long r = b * a.S + (i - b * cs) % a.S;
    const float v = sm_load(a.x, a.x_bf16, i);
    const float rv = __ldg(a.row + r);
    float o;
    if (!BWD) {
      o = a.log_mode ? v - rv : __expf(v - rv);
    } else {
      const float gv = sm_load(a.g, a.g_bf16, i);
      o = a.log_mode ? gv - __expf(v) * rv : v * (gv - rv);
    }
    sm_store(a.out, a.out_bf16, i, o);
  }
}

template <bool WARP_PER_ROW>
__global__ void __launch_bounds__(256) softmax_rowdot_kernel(const SmArgs a) {
  const long long R = static_cast<long long>(a.B) * a.S;
  const int lane = WARP_PER_ROW ? (threadIdx.x & 31) : 0;
  const int nl = WARP_PER_ROW ? 32 : 1;
  const long long t = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  const long long first = WARP_PER_ROW ? (t >> 5) : t;
  const long long step = (static_cast<long long>(gridDim.x) * blockDim.x) / nl;
  for (long long r = first; r < R; r += step) {
    const long long b = r / a.S, sp = r % a.S;
    const long long base = b * a.C * static_cast<long long>(a.S) + sp;
    float d = 0.f;
    for (int c = lane; c < a.C; c += nl) {
      const long long off = base + static_cast<long long>(c) * a.S;
      const float gv = sm_load(a.g, a.g_bf16, off);
      d += a.log_mode ? gv : gv * sm_load(a.x, a.x_bf16, off);
    }
    if (WARP_PER_ROW) d = warp_sum(d);
    if (lane == 0) a.rowout[r] = d;
  }
}

// One thread per row walks the classes (no index arithmetic per element; with a strided class
// dimension the threads of a warp touch consecutive addresses); a trailing class dimension takes one
// warp per row.
template <bool WARP_PER_ROW>
__global__ void __launch_bounds__(256) ce_bwd_kernel(const CeArgs a) {
  const long long R = static_cast<long long>(a.B) * a.S;
  const int lane = WARP_PER_ROW ? (threadIdx.x & 31) : 0;
  const int nl = WARP_PER_ROW ? 32 : 1;
  const long long t = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  const long long first = WARP_PER_ROW ? (t >> 5) : t;
  const long long step = (static_cast<long long>(gridDim.x) * blockDim.x) / nl;
  for (long long r = first; r < R; r += step) {
    const long long b = r / a.S, sp = r % a.S;
    const long long base = b * a.C * static_cast<long long>(a.S) + sp;
    const long long tg = a.target[r];
    const bool live = tg != a.ignore_index;
    const float lse = a.lse[r];
    const float gr = live ? a.grow[r] : 0.f;
    const long long hot = tg - a.class_lo;
    for (int c = lane; c < a.C; c += nl) {
      const long long off = base + static_cast<long long>(c) * a.S;
      float g = 0.f;
      if (live) g = gr * (__expf(ce_load(a, off) - lse) - (hot == c ? 1.f : 0.f));
      if (a.dx_bf16) static_cast<__nv_bfloat16*>(a.dx)[off] = __float2bfloat16(g);
      else static_cast<float*>(a.dx)[off] = g;
    }
  }
}

// ------------------------------------------------------------------------------------------
// GroupNorm whose spatial extent is tiled over GPUs.  x is [N][C][S] (S = local voxels); a
// normalisation group (n, g) is a contiguous run of L = cg * S elements.  Every group is split over
// `splits` CTAs (grid = groups * splits <= number of SMs, all CTAs co-resident):
//   phase 1  each CTA: (count, mean, M2) of its chunk                       -> partials in global memory
//   barrier  grid-wide (atomic counter, bounded spin)
//   leaders  the first CTA of a group merges the chunk partials, exchanges the group's partial with
//            the other tile ranks through peer memory (as the LayerNorm rows above) and writes
//            (mean, rstd) of the group
//   barrier  grid-wide
//   phase 2  each CTA normalises its chunk (per-channel affine).
// Backward has the same shape with (sum g w, sum g w xhat) as the exchanged pair; the per-channel
// sums for dw / db are accumulated per CTA in shared memory and written as partials.
// ------------------------------------------------------------------------------------------
constexpr int GN_MAX_CG = 256;   // channels per group

struct GnArgs {
  const void* x; int x_bf16;
  const void* g; int g_bf16;        // backward
  void* out; int out_bf16;
  const float* w; const float* b;   // [C] local, may be null
  float* stats;                     // [groups][2] mean, rstd (forward writes, backward reads)
  float* partial;                   // [grid][4]
  float* dw_part; float* db_part;   // backward: [grid][cg]
  unsigned int* counters;           // 3 zeroed words (left zero)
  int groups;                       // N * local groups
  int groups_per_sample;            // local groups
  int splits;
  int cg;                           // channels per group
  long long S;                      // local voxels per channel
  float eps;
  LnExchange ex;                    // inbox [2][P][groups][4]; flags [P][groups]
  int* status;
};

__device__ __forceinline__ bool gn_grid_barrier(unsigned int* counter, unsigned int target, int* status) {
  __shared__ int ok;
  __syncthreads();
  if (threadIdx.x == 0) {
    ok = 1;
    __threadfence();
    atomicAdd(counter, 1u);
    const uint64_t t0 = globaltimer_ns();
    while (atomicAdd(counter, 0u) < target) {
      if (globaltimer_ns() - t0 > JB_WAIT_LIMIT_NS) {
        if (status) atomicCAS(status, JB_OK, JB_ERR_MBAR_TIMEOUT);
        ok = 0;
        break;
      }
      __nanosleep(32);
    }
    __threadfence();
  }
  __syncthreads();
  return ok != 0;
}

__device__ __forceinline__ float gn_block_sum(float v) {
  __shared__ float red[LN_WARPS];
  v = warp_sum(v);
  __syncthreads();
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
  __syncthreads();
  float t = 0.f;
#pragma unroll
  for (int i = 0; i < LN_WARPS; ++i) t += red[i];
  return t;
}

// Leader of a group: push (a, b, c) to the peers' inboxes, wait for theirs.  One warp.
__device__ __forceinline__ void gn_exchange(const LnExchange& ex, uint32_t epoch, int gi, int groups, float4 mine,
                                            int* status) {
  const int lane = threadIdx.x & 31;
  const size_t half = static_cast<size_t>(epoch & 1u) * ex.parts * groups * 4;
  if (lane < ex.parts) {
    float* dst = (lane == ex.me) ? ex.inbox_local : ex.inbox_peer[lane];
    *reinterpret_cast<float4*>(dst + half + (static_cast<size_t>(ex.me) * groups + gi) * 4) = mine;
    __threadfence_system();
    if (lane != ex.me) {
      uint32_t* out = ex.flag_peer[lane] + static_cast<size_t>(ex.me) * groups + gi;
      asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(out), "r"(epoch) : "memory");
      const uint32_t* in = ex.flag_local + static_cast<size_t>(lane) * groups + gi;
      const uint64_t t0 = globaltimer_ns();
      while (true) {
        uint32_t v;
        asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(in) : "memory");
        if (static_cast<int32_t>(v - epoch) >= 0) break;
        if (globaltimer_ns() - t0 > JB_WAIT_LIMIT_NS) {
          if (status) atomicCAS(status, JB_OK, JB_ERR_FLAG_TIMEOUT);
          break;
        }
        __nanosleep(64);
      }
    }
  }
  __syncwarp();
}

template <bool BWD>
__global__ void __launch_bounds__(LN_THREADS) gn_kernel(const GnArgs a) {
  extern __shared__ float ch_acc[];   // backward: [2][cg]
  const int gi = blockIdx.x / a.splits, j = blockIdx.x % a.splits;
  const long long L = static_cast<long long>(a.cg) * a.S;
  long long Lc = (L + a.splits - 1) / a.splits;
  Lc = (Lc + 3) & ~3ll;
  const long long e0 = min(L, j * Lc), e1 = min(L, e0 + Lc);
  const long long base = static_cast<long long>(gi) * L;
  const int c0 = (gi % a.groups_per_sample) * a.cg;     // first local channel of the group
  const LnExchange& ex = a.ex;
  const int P = ex.parts;
  const uint32_t epoch = live_epoch(ex.epoch, ex.stride, ex.replay);
  float mean_g = 0.f, rstd_g = 0.f;
  if (BWD) {
    mean_g = a.stats[gi * 2];
    rstd_g = a.stats[gi * 2 + 1];
    for (int i = threadIdx.x; i < 2 * a.cg; i += LN_THREADS) ch_acc[i] = 0.f;
    __syncthreads();
  }
  // ---- phase 1
  float p0 = 0.f, p1 = 0.f;
  if (!BWD) {
    float s = 0.f;
    for (long long e = e0 + threadIdx.x * 4; e < e1; e += LN_THREADS * 4) {
      const float4 v = ln_load4(a.x, a.x_bf16, base + e);
      s += (v.x + v.y) + (v.z + v.w);
    }
    const float cnt = static_cast<float>(e1 - e0);
    const float mean_c = cnt > 0.f ? gn_block_sum(s) / cnt : 0.f;
    float q = 0.f;
    for (long long e = e0 + threadIdx.x * 4; e < e1; e += LN_THREADS * 4) {
      const float4 v = ln_load4(a.x, a.x_bf16, base + e);
      const float d0 = v.x - mean_c, d1 = v.y - mean_c, d2 = v.z - mean_c, d3 = v.w - mean_c;
      q += (d0 * d0 + d1 * d1) + (d2 * d2 + d3 * d3);
    }
    p0 = mean_c;
    p1 = gn_block_sum(q);
    if (threadIdx.x == 0)
      *reinterpret_cast<float4*>(a.partial + static_cast<size_t>(blockIdx.x) * 4) = make_float4(cnt, p0, p1, 0.f);
  } else {
    float s1 = 0.f, s2 = 0.f;
    int cur = -1;                 // channel whose sums are held in registers
    float cgh = 0.f, cgs = 0.f;
    for (long long e = e0 + threadIdx.x * 4; e < e1; e += LN_THREADS * 4) {
      const float4 x = ln_load4(a.x, a.x_bf16, base + e);
      const float4 g = ln_load4(a.g, a.g_bf16, base + e);
      const int c = static_cast<int>(e / a.S);
      if (c != cur) {
        if (cur >= 0) {
          atomicAdd(ch_acc + cur, cgh);
          atomicAdd(ch_acc + a.cg + cur, cgs);
        }
        cur = c;
        cgh = cgs = 0.f;
      }
      const float w = a.w != nullptr ? a.w[c0 + c] : 1.f;
      const float h0 = (x.x - mean_g) * rstd_g, h1 = (x.y - mean_g) * rstd_g, h2 = (x.z - mean_g) * rstd_g,
                  h3 = (x.w - mean_g) * rstd_g;
      const float gh = (g.x * h0 + g.y * h1) + (g.z * h2 + g.w * h3);
      const float gs = (g.x + g.y) + (g.z + g.w);
      s1 += w * gs;
      s2 += w * gh;
      cgh += gh;
      cgs += gs;
    }
    if (cur >= 0) {
      atomicAdd(ch_acc + cur, cgh);
      atomicAdd(ch_acc + a.cg + cur, cgs);
    }
    p0 = gn_block_sum(s1);
    p1 = gn_block_sum(s2);
    if (threadIdx.x == 0)
      *reinterpret_cast<float4*>(a.partial + static_cast<size_t>(blockIdx.x) * 4) = make_float4(p0, p1, 0.f, 0.f);
    __syncthreads();
    for (int i = threadIdx.x; i < a.cg; i += LN_THREADS) {
      a.dw_part[static_cast<size_t>(blockIdx.x) * a.cg + i] = ch_acc[i];
      a.db_part[static_cast<size_t>(blockIdx.x) * a.cg + i] = ch_acc[a.cg + i];
    }
  }
  gn_grid_barrier(a.counters + 0, gridDim.x, a.status);
  // ---- leaders: merge chunks, exchange across tile ranks
  if (j == 0 && threadIdx.x < 32) {
    const int lane = threadIdx.x;
    float4 mine;
    if (!BWD) {
      // merge (count, mean, M2) of the chunks: sequential Chan updates in lane 0 (splits is small)
      float n = 0.f, mu = 0.f, m2 = 0.f;
      if (lane == 0) {
        for (int k = 0; k < a.splits; ++k) {
          const float4 v = __ldcg(reinterpret_cast<const float4*>(a.partial + static_cast<size_t>(gi * a.splits + k) * 4));
          if (v.x <= 0.f) continue;
          const float tot = n + v.x, d = v.y - mu;
          mu += d * v.x / tot;
          m2 += v.z + d * d * n * v.x / tot;
          n = tot;
        }
      }
      mine = make_float4(n, mu, m2, 0.f);
    } else {
      float s1 = 0.f, s2 = 0.f;
      if (lane == 0) {
        for (int k = 0; k < a.splits; ++k) {
          const float4 v = __ldcg(reinterpret_cast<const float4*>(a.partial + static_cast<size_t>(gi * a.splits + k) * 4));
          s1 += v.x;
          s2 += v.y;
        }
      }
      mine = make_float4(s1, s2, 0.f, 0.f);
    }
    mine.x = __shfl_sync(0xffffffffu, mine.x, 0);
    mine.y = __shfl_sync(0xffffffffu, mine.y, 0);
    mine.z = __shfl_sync(0xffffffffu, mine.z, 0);
    if (P > 1) {
      gn_exchange(ex, epoch, gi, a.groups, mine, a.status);
      if (lane == 0) {
        const size_t half = static_cast<size_t>(epoch & 1u) * P * a.groups * 4;
        float n = 0.f, mu = 0.f, m2 = 0.f, s1 = 0.f, s2 = 0.f;
        for (int p = 0; p < P; ++p) {
          const float4 v = __ldcg(reinterpret_cast<const float4*>(ex.inbox_local + half + (static_cast<size_t>(p) * a.groups + gi) * 4));
          if (!BWD) {
            if (v.x <= 0.f) continue;
            const float tot = n + v.x, d = v.y - mu;
            mu += d * v.x / tot;
            m2 += v.z + d * d * n * v.x / tot;
            n = tot;
          } else {
            s1 += v.x;
            s2 += v.y;
          }
        }
        mine = BWD ? make_float4(s1, s2, 0.f, 0.f) : make_float4(n, mu, m2, 0.f);
      }
    }
    if (lane == 0) {
      if (!BWD) {
        a.stats[gi * 2] = mine.y;
        a.stats[gi * 2 + 1] = rsqrtf(mine.z / mine.x + a.eps);
      } else {
        const float inv = 1.f / (static_cast<float>(L) * static_cast<float>(P));
        a.partial[static_cast<size_t>(gi * a.splits) * 4 + 2] = mine.x * inv;    // S1 / N
        a.partial[static_cast<size_t>(gi * a.splits) * 4 + 3] = mine.y * inv;    // S2 / N
      }
      __threadfence();
    }
  }
  gn_grid_barrier(a.counters + 1, gridDim.x, a.status);
  // ---- phase 2
  if (!BWD) {
    const float mean = __ldcg(a.stats + gi * 2), rstd = __ldcg(a.stats + gi * 2 + 1);
    for (long long e = e0 + threadIdx.x * 4; e < e1; e += LN_THREADS * 4) {
      float4 v = ln_load4(a.x, a.x_bf16, base + e);
      const int c = c0 + static_cast<int>(e / a.S);
      const float w = (a.w != nullptr ? a.w[c] : 1.f) * rstd;
      const float b = a.b != nullptr ? a.b[c] : 0.f;
      v.x = (v.x - mean) * w + b; v.y = (v.y - mean) * w + b; v.z = (v.z - mean) * w + b; v.w = (v.w - mean) * w + b;
      ln_store4(a.out, a.out_bf16, base + e, v);
    }
  } else {
    const float S1 = __ldcg(a.partial + static_cast<size_t>(gi * a.splits) * 4 + 2);
    const float S2 = __ldcg(a.partial + static_cast<size_t>(gi * a.splits) * 4 + 3);
    for (long long e = e0 + threadIdx.x * 4; e < e1; e += LN_THREADS * 4) {
      const float4 x = ln_load4(a.x, a.x_bf16, base + e);
      const float4 g = ln_load4(a.g, a.g_bf16, base + e);
      const int c = c0 + static_cast<int>(e / a.S);
      const float w = a.w != nullptr ? a.w[c] : 1.f;
      float4 d;
      d.x = rstd_g * (g.x * w - S1 - (x.x - mean_g) * rstd_g * S2);
      d.y = rstd_g * (g.y * w - S1 - (x.y - mean_g) * rstd_g * S2);
      d.z = rstd_g * (g.z * w - S1 - (x.z - mean_g) * rstd_g * S2);
      d.w = rstd_g * (g.w * w - S1 - (x.w - mean_g) * rstd_g * S2);
      ln_store4(a.out, a.out_bf16, base + e, d);
    }
  }
  // ---- leave the counters zero for the next launch
  __syncthreads();
  if (threadIdx.x == 0) {
    if (atomicAdd(a.counters + 2, 1u) == gridDim.x - 1) {
      a.counters[0] = 0u;
      a.counters[1] = 0u;
      a.counters[2] = 0u;
      __threadfence();
    }
  }
}

}  // namespace jb

using namespace jb;

struct JbLnExchange {          // C mirror passed from Python (ctypes)
  void* inbox_local;
  void* inbox_peer[8];
  void* flag_local;
  void* flag_peer[8];
  unsigned int epoch;
  unsigned int stride;
  const unsigned int* replay;
  int parts, me;
};

static int ln_fill(LnArgs* a, const JbLnExchange* ex) {
  a->ex.parts = 1;
  if (ex == nullptr || ex->parts <= 1) {
    if (ex != nullptr) a->ex.inbox_local = static_cast<float*>(ex->inbox_local);
    return 0;
  }
  if (ex->parts > LN_MAX_PARTS) return -1;
  a->ex.inbox_local = static_cast<float*>(ex->inbox_local);
  a->ex.flag_local = static_cast<uint32_t*>(ex->flag_local);
  for (int p = 0; p < ex->parts; ++p) {
    a->ex.inbox_peer[p] = static_cast<float*>(ex->inbox_peer[p]);
    a->ex.flag_peer[p] = static_cast<uint32_t*>(ex->flag_peer[p]);
  }
  a->ex.epoch = ex->epoch;
  a->ex.stride = ex->stride;
  a->ex.replay = ex->replay;
  a->ex.parts = ex->parts;
  a->ex.me = ex->me;
  return 0;
}

// CTAs of `kernel` that can be resident at once (the kernels here wait on one another across GPUs or
// across the grid, so a grid never exceeds this).
template <typename K>
static int resident_ctas(K kernel, int threads, size_t smem, int sm_count) {
  int per_sm = 0;
  if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, threads, smem) != cudaSuccess || per_sm < 1) per_sm = 1;
  return per_sm * sm_count;
}

// Number of CTAs a LayerNorm launch uses for R rows of n features (the caller sizes flags and partials
// with it); `backward` selects the kernel whose residency bounds the grid.
extern "C" int jb_layer_norm_grid2(int R, int n, int backward, int sm_count) {
  const int want = (R + LN_WARPS - 1) / LN_WARPS;
  const int cap = backward ? resident_ctas(ln_bwd_kernel<false>, LN_THREADS, 0, sm_count)
                           : resident_ctas(ln_fwd_kernel, LN_THREADS, 0, sm_count);
  return want < cap ? (want < 1 ? 1 : want) : cap;
}
extern "C" long long jb_layer_norm_scratch_floats(int R, int n) {
  return 2ll * ((R + LN_COL_ROWS - 1) / LN_COL_ROWS) * n;
}
extern "C" int jb_layer_norm_grid(int R, int sm_count) { return jb_layer_norm_grid2(R, 1024, 1, sm_count); }

// y = LayerNorm(x) over the last dimension of x [R][n] (n = local slice, n % 4 == 0); saves mean / rstd.
extern "C" int jb_layer_norm_fwd(const void* x, int x_bf16, void* y, int y_bf16, const float* w, const float* b,
                                 float* mean, float* rstd, int R, int n, float eps, const JbLnExchange* ex,
                                 int* status, int sm_count, void* stream) {
  if (n % 4 != 0 || R <= 0) return -1;
  LnArgs a{};
  a.x = x; a.x_bf16 = x_bf16; a.out = y; a.out_bf16 = y_bf16; a.w = w; a.b = b;
  a.mean = mean; a.rstd = rstd; a.R = R; a.n = n; a.eps = eps; a.status = status;
  if (ln_fill(&a, ex) != 0) return -1;
  const int grid = jb_layer_norm_grid2(R, n, 0, sm_count);
  ln_fwd_kernel<<<grid, LN_THREADS, 0, static_cast<cudaStream_t>(stream)>>>(a);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

// dx, dw, db of the same.  scratch: 2 * ceil(R / 512) * n floats (jb_layer_norm_scratch_floats).  The exchange needs an inbox even with one part.
extern "C" int jb_layer_norm_bwd(const void* x, int x_bf16, const void* g, int g_bf16, void* dx, int dx_bf16,
                                 const float* w, const float* mean, const float* rstd, float* dw, float* db,
                                 float* scratch, int R, int n, const JbLnExchange* ex, int* status, int sm_count,
                                 void* stream) {
  if (n % 4 != 0 || R <= 0 || n > 12000 || ex == nullptr || ex->inbox_local == nullptr) return -1;
  LnArgs a{};
  a.x = x; a.x_bf16 = x_bf16; a.g = g; a.g_bf16 = g_bf16; a.out = dx; a.out_bf16 = dx_bf16; a.w = w;
  a.mean = const_cast<float*>(mean); a.rstd = const_cast<float*>(rstd); a.R = R; a.n = n; a.status = status;
  if (ln_fill(&a, ex) != 0) return -1;
  const int grid = jb_layer_norm_grid2(R, n, 1, sm_count);
  const bool want = dw != nullptr || db != nullptr;
  const int slabs = (R + LN_COL_ROWS - 1) / LN_COL_ROWS;
  if (want) {
    a.dw_part = scratch;
    a.db_part = scratch + static_cast<size_t>(slabs) * n;
  }
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  ln_bwd_kernel<false><<<grid, LN_THREADS, 0, st>>>(a);
  if (cudaGetLastError() != cudaSuccess) return -4;
  if (want) {
    // the row statistics are already final (forward): the column sums need no exchange
    ln_dwdb_kernel<<<dim3((n + 127) / 128, slabs), 256, 0, st>>>(a);
    if (cudaGetLastError() != cudaSuccess) return -4;
    ln_colsum_kernel<<<(n + 255) / 256, 256, 0, st>>>(a.dw_part, a.db_part, slabs, n, dw, db);
    if (cudaGetLastError() != cudaSuccess) return -4;
  }
  return 0;
}

extern "C" int jb_cross_entropy_grid(int B, int C, int S, int sm_count);

// Per-row cross-entropy of logits [B][C][S] (C = local class shard starting at class_lo) against global
// class indices target[B*S]; writes loss[R] and lse[R].  Exchange inbox slots are 4 floats per row.
extern "C" int jb_cross_entropy_fwd(const void* x, int x_bf16, const long long* target, long long ignore_index, int B,
                                    int C, int S, int class_lo, float* loss, float* lse, const JbLnExchange* ex,
                                    int* status, int sm_count, void* stream) {
  if (B <= 0 || C <= 0 || S <= 0) return -1;
  CeArgs a{};
  a.x = x; a.x_bf16 = x_bf16; a.target = target; a.ignore_index = ignore_index;
  a.B = B; a.C = C; a.S = S; a.class_lo = class_lo; a.loss = loss; a.lse = lse; a.status = status;
  LnArgs tmp{};
  if (ln_fill(&tmp, ex) != 0) return -1;
  a.ex = tmp.ex;
  const int R = B * S;
  const bool warp_rows = (S == 1 && C >= 64);
  const int grid = jb_cross_entropy_grid(B, C, S, sm_count);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (warp_rows) ce_fwd_kernel<true><<<grid, LN_THREADS, 0, st>>>(a);
  else ce_fwd_kernel<false><<<grid, LN_THREADS, 0, st>>>(a);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

static unsigned int sm_grid(long long threads, int sm_count) {
  long long grid = (threads + 255) / 256;
  const long long cap = static_cast<long long>(sm_count) * 16;
  return static_cast<unsigned int>(grid < 1 ? 1 : (grid > cap ? cap : grid));
}

// y = x - lse[row] (log_mode) or exp(x - lse[row]) for x [B][C][S], rows = (b, s).
extern "C" int jb_softmax_apply(const void* x, int x_bf16, const float* lse, void* y, int y_bf16, int B, int C, int S,
                                int log_mode, int sm_count, void* stream) {
  if (B <= 0 || C <= 0 || S <= 0) return -1;
  SmArgs a{};
  a.x = x; a.x_bf16 = x_bf16; a.row = lse; a.out = y; a.out_bf16 = y_bf16; a.B = B; a.C = C; a.S = S; a.log_mode = log_mode;
  softmax_elementwise_kernel<false><<<sm_grid(static_cast<long long>(B) * C * S, sm_count), 256, 0,
                                     static_cast<cudaStream_t>(stream)>>>(a);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

// d[row] = sum over the local classes of g (log_mode) or of g * y.
extern "C" int jb_softmax_rowdot(const void* y, int y_bf16, const void* g, int g_bf16, float* d, int B, int C, int S,
                                 int log_mode, int sm_count, void* stream) {
  if (B <= 0 || C <= 0 || S <= 0) return -1;
  SmArgs a{};
  a.x = y; a.x_bf16 = y_bf16; a.g = g; a.g_bf16 = g_bf16; a.rowout = d; a.B = B; a.C = C; a.S = S; a.log_mode = log_mode;
  const bool warp_rows = (S == 1 && C >= 64);
  const long long threads = static_cast<long long>(B) * S * (warp_rows ? 32 : 1);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (warp_rows) softmax_rowdot_kernel<true><<<sm_grid(threads, sm_count), 256, 0, st>>>(a);
  else softmax_rowdot_kernel<false><<<sm_grid(threads, sm_count), 256, 0, st>>>(a);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

// dx = g - exp(y) d[row] (log_mode) or y (g - d[row]).
extern "C" int jb_softmax_bwd(const void* y, int y_bf16, const void* g, int g_bf16, const float* d, void* dx, int dx_bf16,
                              int B, int C, int S, int log_mode, int sm_count, void* stream) {
  if (B <= 0 || C <= 0 || S <= 0) return -1;
  SmArgs a{};
  a.x = y; a.x_bf16 = y_bf16; a.g = g; a.g_bf16 = g_bf16; a.row = d; a.out = dx; a.out_bf16 = dx_bf16;
  a.B = B; a.C = C; a.S = S; a.log_mode = log_mode;
  softmax_elementwise_kernel<true><<<sm_grid(static_cast<long long>(B) * C * S, sm_count), 256, 0,
                                    static_cast<cudaStream_t>(stream)>>>(a);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

extern "C" int jb_cross_entropy_grid(int B, int C, int S, int sm_count) {
  const int R = B * S;
  const bool warp_rows = (S == 1 && C >= 64);
  const int per_cta = warp_rows ? LN_WARPS : LN_THREADS;
  const int grid = (R + per_cta - 1) / per_cta;
  const int cap = warp_rows ? resident_ctas(ce_fwd_kernel<true>, LN_THREADS, 0, sm_count)
                            : resident_ctas(ce_fwd_kernel<false>, LN_THREADS, 0, sm_count);
  return grid > cap ? cap : grid;
}

// dx = grow[row] * (softmax - onehot) from the saved lse; rows with ignore_index get zero.
extern "C" int jb_cross_entropy_bwd(const void* x, int x_bf16, const long long* target, long long ignore_index, int B,
                                    int C, int S, int class_lo, const float* lse, const float* grow, void* dx,
                                    int dx_bf16, int sm_count, void* stream) {
  if (B <= 0 || C <= 0 || S <= 0) return -1;
  CeArgs a{};
  a.x = x; a.x_bf16 = x_bf16; a.target = target; a.ignore_index = ignore_index;
  a.B = B; a.C = C; a.S = S; a.class_lo = class_lo; a.lse = const_cast<float*>(lse); a.grow = grow;
  a.dx = dx; a.dx_bf16 = dx_bf16;
  const bool warp_rows = (S == 1 && C >= 64);
  const long long threads = static_cast<long long>(B) * S * (warp_rows ? 32 : 1);
  long long grid = (threads + 255) / 256;
  if (grid > static_cast<long long>(sm_count) * 32) grid = static_cast<long long>(sm_count) * 32;
  if (warp_rows) ce_bwd_kernel<true><<<static_cast<unsigned int>(grid), 256, 0, static_cast<cudaStream_t>(stream)>>>(a);
  else ce_bwd_kernel<false><<<static_cast<unsigned int>(grid), 256, 0, static_cast<cudaStream_t>(stream)>>>(a);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

// Number of CTAs per normalisation group so that groups * splits fits the SMs (0: too many groups).
extern "C" int jb_group_norm_splits(int groups, int sm_count) {
  const int a = resident_ctas(gn_kernel<false>, LN_THREADS, 0, sm_count);
  const int b = resident_ctas(gn_kernel<true>, LN_THREADS, 2 * GN_MAX_CG * sizeof(float), sm_count);
  const int cap = a < b ? a : b;
  return groups > cap ? 0 : cap / groups;
}

static int gn_fill(GnArgs* a, const JbLnExchange* ex, int groups, int groups_per_sample, int cg, long long S,
                   int sm_count) {
  if (groups <= 0 || cg <= 0 || cg > GN_MAX_CG || S <= 0 || (S & 3)) return -1;
  a->groups = groups; a->groups_per_sample = groups_per_sample; a->cg = cg; a->S = S;
  a->splits = jb_group_norm_splits(groups, sm_count);
  if (a->splits <= 0) return -1;
  LnArgs tmp{};
  if (ln_fill(&tmp, ex) != 0) return -1;
  a->ex = tmp.ex;
  return 0;
}

// y = GroupNorm(x) for x [N][C][S] with `groups_per_sample` local groups of cg channels; stats [groups][2]
// receives (mean, rstd).  partial: 4 * groups * splits floats; counters: 3 zeroed words (left zero).
extern "C" int jb_group_norm_fwd(const void* x, int x_bf16, void* y, int y_bf16, const float* w, const float* b,
                                 float* stats, float* partial, unsigned int* counters, int groups,
                                 int groups_per_sample, int cg, long long S, float eps, const JbLnExchange* ex,
                                 int* status, int sm_count, void* stream) {
  GnArgs a{};
  if (gn_fill(&a, ex, groups, groups_per_sample, cg, S, sm_count) != 0) return -1;
  a.x = x; a.x_bf16 = x_bf16; a.out = y; a.out_bf16 = y_bf16; a.w = w; a.b = b; a.stats = stats;
  a.partial = partial; a.counters = counters; a.eps = eps; a.status = status;
  gn_kernel<false><<<groups * a.splits, LN_THREADS, 0, static_cast<cudaStream_t>(stream)>>>(a);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

// dx and per-CTA channel partials dw_part / db_part ([groups * splits][cg]) of the same.
extern "C" int jb_group_norm_bwd(const void* x, int x_bf16, const void* g, int g_bf16, void* dx, int dx_bf16,
                                 const float* w, const float* stats, float* partial, float* dw_part, float* db_part,
                                 unsigned int* counters, int groups, int groups_per_sample, int cg, long long S,
                                 const JbLnExchange* ex, int* status, int sm_count, void* stream) {
  GnArgs a{};
  if (gn_fill(&a, ex, groups, groups_per_sample, cg, S, sm_count) != 0) return -1;
  a.x = x; a.x_bf16 = x_bf16; a.g = g; a.g_bf16 = g_bf16; a.out = dx; a.out_bf16 = dx_bf16; a.w = w;
  a.stats = const_cast<float*>(stats); a.partial = partial; a.dw_part = dw_part; a.db_part = db_part;
  a.counters = counters; a.status = status;
  gn_kernel<true><<<groups * a.splits, LN_THREADS, 2 * cg * sizeof(float), static_cast<cudaStream_t>(stream)>>>(a);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}
