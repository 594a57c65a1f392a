// Memory-bound kernels of the MoE layer for sm_100a: identity copy, RMSNorm, T-Route select,
// the permutation plan (stable counting sort), row scatter, deterministic gate-weighted
// combine (+ backward), SwiGLU backward, and the K1 arrival / K2 pack index kernels.
//
// All reductions that decide numerics run in a fixed order (no float atomics), so results are
// bit-reproducible and follow the canonical tree "groups ascending, experts ascending inside a
// group, fp32 accumulation, one rounding per level".
//
// Reference behaviour: terrace/model.py:46-47 (rmsnorm), terrace/routing.py:45-96 (t_route
// mode "full"), terrace/layer.py:101-112 (permute / un-permute around the grouped matmul),
// terrace/ops/__init__.py:255-300 (K1), terrace/ops/k2_ref.py:70-134 (K2).
#include "host_util.h"
#include "launch.h"
#include "ptx_sm100.cuh"
#include "symm_layout.h"

#include <cuda_bf16.h>

namespace tb200 {

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// Warp-cooperative copy of `bytes` bytes (any size); widest vector the alignment allows.
__device__ __forceinline__ void warp_copy_bytes(void* dst, const void* src, int bytes, int lane) {
  const uintptr_t both = reinterpret_cast<uintptr_t>(dst) | reinterpret_cast<uintptr_t>(src) |
                         static_cast<uintptr_t>(bytes);
  if ((both & 15) == 0) {
    const uint4* s = static_cast<const uint4*>(src);
    uint4* d = static_cast<uint4*>(dst);
    for (int i = lane; i < bytes / 16; i += 32) d[i] = s[i];
  } else if ((both & 3) == 0) {
    const uint32_t* s = static_cast<const uint32_t*>(src);
    uint32_t* d = static_cast<uint32_t*>(dst);
    for (int i = lane; i < bytes / 4; i += 32) d[i] = s[i];
  } else {
    const uint8_t* s = static_cast<const uint8_t*>(src);
    uint8_t* d = static_cast<uint8_t*>(dst);
    for (int i = lane; i < bytes; i += 32) d[i] = s[i];
  }
}

// ---------------------------------------------------------------------------------------------
// identity copy
// ---------------------------------------------------------------------------------------------
__global__ void passthrough_kernel(const uint8_t* __restrict__ src, uint8_t* __restrict__ dst,
                                   size_t bytes) {
  const size_t n16 = bytes / 16;
  const size_t stride = static_cast<size_t>(gridDim.x) * blockDim.x;
  const size_t tid = static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (((reinterpret_cast<uintptr_t>(src) | reinterpret_cast<uintptr_t>(dst)) & 15) == 0) {
    const uint4* s = reinterpret_cast<const uint4*>(src);
    uint4* d = reinterpret_cast<uint4*>(dst);
    for (size_t i = tid; i < n16; i += stride) d[i] = s[i];
    for (size_t i = n16 * 16 + tid; i < bytes; i += stride) dst[i] = src[i];
  } else {
    for (size_t i = tid; i < bytes; i += stride) dst[i] = src[i];
  }
}

// ---------------------------------------------------------------------------------------------
// RMSNorm: one warp per row, fp32 math
// ---------------------------------------------------------------------------------------------
template <typename T> __device__ __forceinline__ float to_f(T v);
template <> __device__ __forceinline__ float to_f<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f<__nv_bfloat16>(__nv_bfloat16 v) {
  return __bfloat162float(v);
}
template <typename T> __device__ __forceinline__ T from_f(float v);
template <> __device__ __forceinline__ float from_f<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f<__nv_bfloat16>(float v) {
  return __float2bfloat16_rn(v);
}

template <typename T>
__global__ void rmsnorm_fwd_kernel(const T* __restrict__ x, const T* __restrict__ w,
                                   T* __restrict__ y, float* __restrict__ rstd, long long rows,
                                   int dim, float eps) {
  const int lane = threadIdx.x & 31;
  const long long row = static_cast<long long>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= rows) return;
  const T* xr = x + row * dim;
  T* yr = y + row * dim;
  float ss = 0.f;
  if (sizeof(T) == 2 && dim % 8 == 0) {
    // 16-byte path: 8 bf16 per lane per step
    const uint4* x4 = reinterpret_cast<const uint4*>(xr);
    for (int i = lane; i < dim / 8; i += 32) {
      const uint4 v = x4[i];
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = __bfloat1622float2(h[j]);
        ss += f.x * f.x + f.y * f.y;
      }
    }
    ss = warp_sum(ss);
    const float r = rsqrtf(ss / dim + eps);
    if (lane == 0 && rstd != nullptr) rstd[row] = r;
    const uint4* w4 = reinterpret_cast<const uint4*>(w);
    uint4* y4 = reinterpret_cast<uint4*>(yr);
    for (int i = lane; i < dim / 8; i += 32) {
      const uint4 v = x4[i], g = w4[i];
      const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
      const __nv_bfloat162* gh = reinterpret_cast<const __nv_bfloat162*>(&g);
      uint4 o;
      __nv_bfloat162* oh = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float2 f = __bfloat1622float2(h[j]), gw = __bfloat1622float2(gh[j]);
        // same rounding points as the eager expression x * rsqrt(.) * w in bf16
        const float2 n = __bfloat1622float2(__floats2bfloat162_rn(f.x * r, f.y * r));
        oh[j] = __floats2bfloat162_rn(n.x * gw.x, n.y * gw.y);
      }
      y4[i] = o;
    }
    return;
  }
  for (int i = lane; i < dim; i += 32) {
    const float v = to_f(xr[i]);
    ss += v * v;
  }
  ss = warp_sum(ss);
  const float r = rsqrtf(ss / dim + eps);
  if (lane == 0 && rstd != nullptr) rstd[row] = r;
  for (int i = lane; i < dim; i += 32) {
    // same rounding points as the eager expression x * rsqrt(.) * w in the tensor dtype
    const T xn = from_f<T>(to_f(xr[i]) * r);
    yr[i] = from_f<T>(to_f(xn) * to_f(w[i]));
  }
}

// dx = r * (dy*w) - x * r^3 * mean(dy*w*x);  dw partial sums per block-row group (fixed order)
template <typename T>
__global__ void rmsnorm_bwd_kernel(const T* __restrict__ x, const T* __restrict__ w,
                                   const T* __restrict__ dy, const float* __restrict__ rstd,
                                   T* __restrict__ dx, float* __restrict__ dw_partial,
                                   long long rows, int dim) {
  // blockDim = (32 lanes, W warps); every block owns a contiguous slab of rows and writes one
  // partial dw vector; the host sums the partials in a fixed order.
  const int lane = threadIdx.x;
  const int warp = threadIdx.y;
  const int nwarps = blockDim.y;
  extern __shared__ float sdw[];      // [nwarps][dim]
  float* mydw = sdw + static_cast<size_t>(warp) * dim;
  for (int i = lane; i < dim; i += 32) mydw[i] = 0.f;
  const long long per_block = (rows + gridDim.x - 1) / gridDim.x;
  const long long r0 = static_cast<long long>(blockIdx.x) * per_block;
  const long long r1 = min(rows, r0 + per_block);
  for (long long row = r0 + warp; row < r1; row += nwarps) {
    const T* xr = x + row * dim;
    const T* dyr = dy + row * dim;
    const float r = rstd[row];
    float dot = 0.f;
    for (int i = lane; i < dim; i += 32) dot += to_f(dyr[i]) * to_f(w[i]) * to_f(xr[i]);
    dot = warp_sum(dot);
    const float c = dot * r * r * r / dim;
    T* dxr = dx + row * dim;
    for (int i = lane; i < dim; i += 32) {
      const float xv = to_f(xr[i]), g = to_f(dyr[i]);
      dxr[i] = from_f<T>(g * to_f(w[i]) * r - xv * c);
      mydw[i] += g * xv * r;
    }
  }
  __syncthreads();
  for (int i = threadIdx.y * 32 + lane; i < dim; i += 32 * nwarps) {
    float acc = 0.f;
    for (int wv = 0; wv < nwarps; ++wv) acc += sdw[static_cast<size_t>(wv) * dim + i];
    dw_partial[static_cast<size_t>(blockIdx.x) * dim + i] = acc;
  }
}

// bf16 rows whose width is a multiple of 256: every lane owns 8 consecutive columns per step and
// moves them with 16-byte accesses; one warp per row, 4 warps per block, several blocks per SM.
// Same arithmetic and the same fixed summation order per block as the generic kernel above.
__global__ void rmsnorm_bwd_vec_kernel(const __nv_bfloat16* __restrict__ x,
                                       const __nv_bfloat16* __restrict__ w,
                                       const __nv_bfloat16* __restrict__ dy,
                                       const float* __restrict__ rstd,
                                       __nv_bfloat16* __restrict__ dx,
                                       float* __restrict__ dw_partial, long long rows, int dim) {
  const int lane = threadIdx.x, warp = threadIdx.y, nwarps = blockDim.y;
  extern __shared__ float sdw[];      // [nwarps][dim]
  float* mydw = sdw + static_cast<size_t>(warp) * dim;
  for (int i = lane; i < dim; i += 32) mydw[i] = 0.f;
  const int steps = dim >> 8;
  const long long per_block = (rows + gridDim.x - 1) / gridDim.x;
  const long long r0 = static_cast<long long>(blockIdx.x) * per_block;
  const long long r1 = min(rows, r0 + per_block);
  for (long long row = r0 + warp; row < r1; row += nwarps) {
    const uint4* xr = reinterpret_cast<const uint4*>(x + row * dim);
    const uint4* dyr = reinterpret_cast<const uint4*>(dy + row * dim);
    const uint4* wr = reinterpret_cast<const uint4*>(w);
    float dot = 0.f;
    for (int j = 0; j < steps; ++j) {
      const int c = j * 32 + lane;
      const uint4 xv = xr[c], gv = dyr[c], wv = wr[c];
      const __nv_bfloat162* xb = reinterpret_cast<const __nv_bfloat162*>(&xv);
      const __nv_bfloat162* gb = reinterpret_cast<const __nv_bfloat162*>(&gv);
      const __nv_bfloat162* wb = reinterpret_cast<const __nv_bfloat162*>(&wv);
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const float2 xf = __bfloat1622float2(xb[u]), gf = __bfloat1622float2(gb[u]),
                     wf = __bfloat1622float2(wb[u]);
        dot += gf.x * wf.x * xf.x;
        dot += gf.y * wf.y * xf.y;
      }
    }
    dot = warp_sum(dot);
    const float r = rstd[row];
    const float cfac = dot * r * r * r / dim;
    uint4* dxr = reinterpret_cast<uint4*>(dx + row * dim);
    for (int j = 0; j < steps; ++j) {
      const int c = j * 32 + lane;
      const uint4 xv = xr[c], gv = dyr[c], wv = wr[c];      // second read: L1 / L2
      const __nv_bfloat162* xb = reinterpret_cast<const __nv_bfloat162*>(&xv);
      const __nv_bfloat162* gb = reinterpret_cast<const __nv_bfloat162*>(&gv);
      const __nv_bfloat162* wb = reinterpret_cast<const __nv_bfloat162*>(&wv);
      uint4 out;
      __nv_bfloat162* ob = reinterpret_cast<__nv_bfloat162*>(&out);
      float4* acc = reinterpret_cast<float4*>(mydw + c * 8);
      float4 a0 = acc[0], a1 = acc[1];
      float* af[2] = {reinterpret_cast<float*>(&a0), reinterpret_cast<float*>(&a1)};
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const float2 xf = __bfloat1622float2(xb[u]), gf = __bfloat1622float2(gb[u]),
                     wf = __bfloat1622float2(wb[u]);
        ob[u] = __floats2bfloat162_rn(gf.x * wf.x * r - xf.x * cfac, gf.y * wf.y * r - xf.y * cfac);
        af[u >> 1][(u & 1) * 2] += gf.x * xf.x * r;
        af[u >> 1][(u & 1) * 2 + 1] += gf.y * xf.y * r;
      }
      acc[0] = a0;
      acc[1] = a1;
      dxr[c] = out;
    }
  }
  __syncthreads();
  for (int i = threadIdx.y * 32 + lane; i < dim; i += 32 * nwarps) {
    float acc = 0.f;
    for (int wv = 0; wv < nwarps; ++wv) acc += sdw[static_cast<size_t>(wv) * dim + i];
    dw_partial[static_cast<size_t>(blockIdx.x) * dim + i] = acc;
  }
}

// bf16 rows whose width is (4..8 warps) x 256 x (1..4): the block's warps split the columns, so a lane
// owns STEPS groups of 8 columns for the whole kernel and keeps their weight-gradient sums in
// registers (no shared-memory accumulators, occupancy is bounded by registers only).  x and dy
// are read once and held between the row dot product and the dx / dw pass; the dot product
// crosses warps through a double-buffered shared array, one barrier per batch of RB rows.
// Summation order is fixed: lane partial, warp butterfly, warps in index order.
template <int STEPS, int RB>
__global__ void __launch_bounds__(256)
rmsnorm_bwd_cols_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w,
                        const __nv_bfloat16* __restrict__ dy, const float* __restrict__ rstd,
                        __nv_bfloat16* __restrict__ dx, float* __restrict__ dw_partial,
                        long long rows, int dim) {
  const int lane = threadIdx.x, warp = threadIdx.y, nwarps = blockDim.y;
  __shared__ float s_dot[2][RB][8];
  // column group (of 8) owned by this lane in step j: (j * nwarps + warp) * 32 + lane
  float wf[STEPS][8], dwacc[STEPS][8];
#pragma unroll
  for (int j = 0; j < STEPS; ++j) {
    const uint4 wv = reinterpret_cast<const uint4*>(w)[(j * nwarps + warp) * 32 + lane];
    const __nv_bfloat162* wb = reinterpret_cast<const __nv_bfloat162*>(&wv);
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const float2 f = __bfloat1622float2(wb[u]);
      wf[j][2 * u] = f.x;
      wf[j][2 * u + 1] = f.y;
      dwacc[j][2 * u] = 0.f;
      dwacc[j][2 * u + 1] = 0.f;
    }
  }
  const long long per_block = (rows + gridDim.x - 1) / gridDim.x;
  const long long r0 = static_cast<long long>(blockIdx.x) * per_block;
  const long long r1 = min(rows, r0 + per_block);
  const int groups_per_row = dim >> 3;
  int buf = 0;
  for (long long base = r0; base < r1; base += RB, buf ^= 1) {
    uint4 xv[RB][STEPS], gv[RB][STEPS];
    float part[RB];
#pragma unroll
    for (int b = 0; b < RB; ++b) {
      const long long row = base + b;
      part[b] = 0.f;
      if (row < r1) {
        const uint4* xr = reinterpret_cast<const uint4*>(x) + row * groups_per_row;
        const uint4* gr = reinterpret_cast<const uint4*>(dy) + row * groups_per_row;
#pragma unroll
        for (int j = 0; j < STEPS; ++j) {
          xv[b][j] = xr[(j * nwarps + warp) * 32 + lane];
          gv[b][j] = gr[(j * nwarps + warp) * 32 + lane];
        }
#pragma unroll
        for (int j = 0; j < STEPS; ++j) {
          const __nv_bfloat162* xb = reinterpret_cast<const __nv_bfloat162*>(&xv[b][j]);
          const __nv_bfloat162* gb = reinterpret_cast<const __nv_bfloat162*>(&gv[b][j]);
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            const float2 xf = __bfloat1622float2(xb[u]), gf = __bfloat1622float2(gb[u]);
            part[b] += gf.x * wf[j][2 * u] * xf.x;
            part[b] += gf.y * wf[j][2 * u + 1] * xf.y;
          }
        }
      }
      part[b] = warp_sum(part[b]);
      if (lane == 0) s_dot[buf][b][warp] = part[b];
    }
    __syncthreads();
#pragma unroll
    for (int b = 0; b < RB; ++b) {
      const long long row = base + b;
      if (row >= r1) break;
      float dot = 0.f;
      for (int wi = 0; wi < nwarps; ++wi) dot += s_dot[buf][b][wi];
      const float r = rstd[row];
      const float cfac = dot * r * r * r / dim;
      uint4* dxr = reinterpret_cast<uint4*>(dx) + row * groups_per_row;
#pragma unroll
      for (int j = 0; j < STEPS; ++j) {
        const __nv_bfloat162* xb = reinterpret_cast<const __nv_bfloat162*>(&xv[b][j]);
        const __nv_bfloat162* gb = reinterpret_cast<const __nv_bfloat162*>(&gv[b][j]);
        uint4 out;
        __nv_bfloat162* ob = reinterpret_cast<__nv_bfloat162*>(&out);
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const float2 xf = __bfloat1622float2(xb[u]), gf = __bfloat1622float2(gb[u]);
          ob[u] = __floats2bfloat162_rn(gf.x * wf[j][2 * u] * r - xf.x * cfac,
                                        gf.y * wf[j][2 * u + 1] * r - xf.y * cfac);
          dwacc[j][2 * u] += gf.x * xf.x * r;
          dwacc[j][2 * u + 1] += gf.y * xf.y * r;
        }
        dxr[(j * nwarps + warp) * 32 + lane] = out;
      }
    }
  }
  float* out_row = dw_partial + static_cast<size_t>(blockIdx.x) * dim;
#pragma unroll
  for (int j = 0; j < STEPS; ++j) {
    float4* o = reinterpret_cast<float4*>(out_row + ((j * nwarps + warp) * 32 + lane) * 8);
    o[0] = make_float4(dwacc[j][0], dwacc[j][1], dwacc[j][2], dwacc[j][3]);
    o[1] = make_float4(dwacc[j][4], dwacc[j][5], dwacc[j][6], dwacc[j][7]);
  }
}

template <int STEPS, int RB>
static void launch_rmsnorm_bwd_cols(int warps, const void* x, const void* w, const void* dy,
                                    const float* rstd, void* dx, float* dw_partial, int n_partial,
                                    long long rows, int dim, cudaStream_t stream) {
  rmsnorm_bwd_cols_kernel<STEPS, RB><<<n_partial, dim3(32, warps), 0, stream>>>(
      static_cast<const __nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(w),
      static_cast<const __nv_bfloat16*>(dy), rstd, static_cast<__nv_bfloat16*>(dx), dw_partial,
      rows, dim);
}

// ---------------------------------------------------------------------------------------------
// T-Route select, mode "full": one warp per token
// ---------------------------------------------------------------------------------------------
constexpr int ROUTE_MAX_E = 512;
constexpr int ROUTE_MAX_G = 64;
constexpr int ROUTE_WARPS = 4;

// Advance (prev, prev_i) to the next element of v[0..n) in the order "value descending, index
// ascending" and add its value to `sum`.  Call with prev = +inf, prev_i = -1 to start.
__device__ __forceinline__ void next_best(const float* v, int n, float& prev, int& prev_i,
                                          float& sum) {
  float best = -INFINITY;
  int bi = -1;
  for (int j = 0; j < n; ++j) {
    const float x = v[j];
    const bool after_prev = x < prev || (x == prev && j > prev_i);
    if (after_prev && (bi < 0 || x > best)) { best = x; bi = j; }
  }
  if (bi < 0) { bi = prev_i < 0 ? 0 : prev_i; best = v[bi]; }   // only with NaNs in v
  prev = best;
  prev_i = bi;
  sum += best;
}

__global__ void route_select_kernel(const float* __restrict__ logits,
                                    const float* __restrict__ bias, long long* __restrict__ idx,
                                    float* __restrict__ gates, long long* __restrict__ group_idx,
                                    float* __restrict__ load, float* __restrict__ aff_sel, int T,
                                    int E, int n_groups, int top_k, int top_groups, int pool) {
  __shared__ float s_aff[ROUTE_WARPS][ROUTE_MAX_E];
  __shared__ float s_sel[ROUTE_WARPS][ROUTE_MAX_E];
  __shared__ float s_gsc[ROUTE_WARPS][ROUTE_MAX_G];
  __shared__ int s_grp[ROUTE_WARPS][ROUTE_MAX_G];
  __shared__ int s_pick[ROUTE_WARPS][64];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x * ROUTE_WARPS + warp;
  if (t >= T) return;
  const int g = E / n_groups;
  const int q = top_k / top_groups;
  float* aff = s_aff[warp];
  float* sel = s_sel[warp];
  for (int e = lane; e < E; e += 32) {
    const float a = 1.0f / (1.0f + expf(-logits[static_cast<size_t>(t) * E + e]));
    aff[e] = a;
    sel[e] = a + bias[e];
  }
  __syncwarp();
  // group score = mean of the `pool` best selection scores of the group
  const int width = pool < g ? pool : g;
  for (int gi = lane; gi < n_groups; gi += 32) {
    const float* sg = sel + gi * g;
    float sum = 0.f, prev = INFINITY;
    int prev_i = -1;
    for (int r = 0; r < width; ++r) next_best(sg, g, prev, prev_i, sum);
    s_gsc[warp][gi] = sum / width;
  }
  __syncwarp();
  // top-M groups, descending score, lowest index wins ties
  if (lane == 0) {
    float prev = INFINITY, dummy = 0.f;
    int prev_i = -1;
    for (int m = 0; m < top_groups; ++m) {
      next_best(s_gsc[warp], n_groups, prev, prev_i, dummy);
      s_grp[warp][m] = prev_i;
    }
  }
  __syncwarp();
  // per-group top-q, descending biased affinity
  for (int m = lane; m < top_groups; m += 32) {
    const int gi = s_grp[warp][m];
    const float* sg = sel + gi * g;
    float prev = INFINITY, dummy = 0.f;
    int prev_i = -1;
    for (int r = 0; r < q; ++r) {
      next_best(sg, g, prev, prev_i, dummy);
      s_pick[warp][m * q + r] = gi * g + prev_i;
    }
  }
  __syncwarp();
  float a = 0.f;
  int e = 0;
  if (lane < top_k) {
    e = s_pick[warp][lane];
    a = aff[e];
  }
  // gates = raw affinity renormalised over the k picks (sequential sum: fixed order)
  float total = 0.f;
  for (int j = 0; j < top_k; ++j) total += __shfl_sync(0xffffffffu, a, j);
  if (lane < top_k) {
    idx[static_cast<size_t>(t) * top_k + lane] = e;
    gates[static_cast<size_t>(t) * top_k + lane] = a / total;
    aff_sel[static_cast<size_t>(t) * top_k + lane] = a;
    atomicAdd(&load[e], 1.0f);                      // integer-valued: order independent
  }
  if (lane < top_groups) group_idx[static_cast<size_t>(t) * top_groups + lane] = s_grp[warp][lane];
}

__global__ void route_select_bwd_kernel(const float* __restrict__ dgates,
                                        const float* __restrict__ gates,
                                        const float* __restrict__ aff_sel,
                                        const long long* __restrict__ idx,
                                        float* __restrict__ dlogits, int T, int E, int top_k) {
  const int t = blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= T) return;
  float total = 0.f, dot = 0.f;
  for (int j = 0; j < top_k; ++j) {
    total += aff_sel[static_cast<size_t>(t) * top_k + j];
    dot += dgates[static_cast<size_t>(t) * top_k + j] * gates[static_cast<size_t>(t) * top_k + j];
  }
  for (int j = 0; j < top_k; ++j) {
    const size_t o = static_cast<size_t>(t) * top_k + j;
    const float a = aff_sel[o];
    const float da = (dgates[o] - dot) / total;
    dlogits[static_cast<size_t>(t) * E + idx[o]] = da * a * (1.0f - a);
  }
}

// ---------------------------------------------------------------------------------------------
// Permutation plan: stable counting sort of the (token, pick) pairs by expert.
//   pass 1: each warp owns a contiguous token chunk; per token insertion-sorts its k picks,
//           assigns the local rank of each pick inside (chunk, expert) and builds a chunk histogram
//   pass 2: one block turns [chunk][E] histograms into bases (expert-major, chunk-minor)
//   pass 3: pos = base + local rank
// ---------------------------------------------------------------------------------------------
constexpr int PLAN_MAX_K = 32;
constexpr int PLAN_CHUNKS = TB200_PLAN_CHUNKS;

__global__ void plan_pass1_kernel(const long long* __restrict__ expert_idx,
                                  const float* __restrict__ gates, int* __restrict__ es,
                                  float* __restrict__ gs, int* __restrict__ cols,
                                  int* __restrict__ rank_local, int* __restrict__ chunk_hist, int T,
                                  int k, int E) {
  extern __shared__ int s_cnt[];        // [E] picks so far, then [E] lane masks of the group
  unsigned* s_mask = reinterpret_cast<unsigned*>(s_cnt + E);
  const int chunk = blockIdx.x;
  const int per = (T + PLAN_CHUNKS - 1) / PLAN_CHUNKS;
  const int t0 = chunk * per, t1 = min(T, t0 + per);
  const int lane = threadIdx.x;
  for (int e = lane; e < E; e += 32) {
    s_cnt[e] = 0;
    s_mask[e] = 0u;
  }
  __syncwarp();
  for (int tb = t0; tb < t1; tb += 32) {
    const int t = tb + lane;
    const bool live = t < t1;
    int e_loc[PLAN_MAX_K];
    if (live) {
      float g_loc[PLAN_MAX_K];
      int c_loc[PLAN_MAX_K];
      for (int j = 0; j < k; ++j) {
        e_loc[j] = static_cast<int>(expert_idx[static_cast<size_t>(t) * k + j]);
        g_loc[j] = gates ? gates[static_cast<size_t>(t) * k + j] : 1.0f;
        c_loc[j] = j;
      }
      for (int i = 1; i < k; ++i) {         // stable insertion sort, ascending expert id
        const int ev = e_loc[i], cv = c_loc[i];
        const float gv = g_loc[i];
        int j = i - 1;
        while (j >= 0 && e_loc[j] > ev) {
          e_loc[j + 1] = e_loc[j]; g_loc[j + 1] = g_loc[j]; c_loc[j + 1] = c_loc[j];
          --j;
        }
        e_loc[j + 1] = ev; g_loc[j + 1] = gv; c_loc[j + 1] = cv;
      }
      for (int j = 0; j < k; ++j) {
        es[static_cast<size_t>(t) * k + j] = e_loc[j];
        gs[static_cast<size_t>(t) * k + j] = g_loc[j];
        cols[static_cast<size_t>(t) * k + j] = c_loc[j];
      }
    }
    // Rank of every pick inside its expert, in TOKEN order (the canonical order the capacity
    // rule and the host model use).  Routing gives a token distinct experts, so "lower lanes that
    // picked e" is a bit count over a per-expert lane mask.  A group that holds a token with a
    // repeated expert (not a top-k routing) falls back to column-major ranking, which still
    // gives every pick a distinct in-range rank.
    bool dup = false;
    if (live)
      for (int j = 1; j < k; ++j) dup |= e_loc[j] == e_loc[j - 1];
    if (!__any_sync(0xffffffffu, dup)) {
      if (live)
        for (int j = 0; j < k; ++j)
          if (e_loc[j] >= 0 && e_loc[j] < E) atomicOr(&s_mask[e_loc[j]], 1u << lane);
      __syncwarp();
      if (live)
        for (int j = 0; j < k; ++j) {
          const int e = e_loc[j];
          rank_local[static_cast<size_t>(t) * k + j] =
              (e >= 0 && e < E) ? s_cnt[e] + __popc(s_mask[e] & ((1u << lane) - 1u)) : -1;
        }
      __syncwarp();
      if (live)
        for (int j = 0; j < k; ++j) {
          const int e = e_loc[j];
          if (e >= 0 && e < E && (s_mask[e] >> lane) == 1u) s_cnt[e] += __popc(s_mask[e]);
        }
      __syncwarp();
      if (live)
        for (int j = 0; j < k; ++j)
          if (e_loc[j] >= 0 && e_loc[j] < E) s_mask[e_loc[j]] = 0u;
      __syncwarp();
    } else {
      for (int j = 0; j < k; ++j) {
        const int e = live ? e_loc[j] : -1 - lane;            // dead lanes match nobody
        const unsigned peers = __match_any_sync(0xffffffffu, e);
        if (live && e >= 0 && e < E) {
          const int before = __popc(peers & ((1u << lane) - 1u));
          rank_local[static_cast<size_t>(t) * k + j] = s_cnt[e] + before;
        } else if (live) {
          rank_local[static_cast<size_t>(t) * k + j] = -1;     // out-of-range id: skipped later
        }
        __syncwarp();
        if (live && e >= 0 && e < E && (peers >> lane) == 1u) s_cnt[e] += __popc(peers);
        __syncwarp();
      }
    }
  }
  for (int e = lane; e < E; e += 32) chunk_hist[static_cast<size_t>(chunk) * E + e] = s_cnt[e];
}

// prior[E] (may be null): rows of lower-ranked sources that precede ours inside every expert
// Exclusive prefix over the `n_chunks` (multiple of 32) rows of hist[chunk][stride] for column
// `col`, done by one warp; returns the column total (valid in every lane).
__device__ __forceinline__ int warp_chunk_prefix(int* hist, int n_chunks, int stride, int col,
                                                 int lane) {
  const int per = n_chunks / 32;
  int local[8];
  int sum = 0;
  for (int i = 0; i < per; ++i) {
    local[i] = hist[static_cast<size_t>(lane * per + i) * stride + col];
    sum += local[i];
  }
  int incl = sum;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const int v = __shfl_up_sync(0xffffffffu, incl, o);
    if (lane >= o) incl += v;
  }
  int run = incl - sum;
  for (int i = 0; i < per; ++i) {
    hist[static_cast<size_t>(lane * per + i) * stride + col] = run;
    run += local[i];
  }
  return __shfl_sync(0xffffffffu, incl, 31);
}

__global__ void plan_pass2_kernel(int* __restrict__ chunk_hist, int* __restrict__ seg_start,
                                  int* __restrict__ seg_count, int E, int seg_align) {
  // single block; one warp per expert column at a time
  extern __shared__ int s_tot[];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  for (int e = warp; e < E; e += nwarps) {
    const int total = warp_chunk_prefix(chunk_hist, PLAN_CHUNKS, E, e, lane);
    if (lane == 0) {
      s_tot[e] = total;
      seg_count[e] = total;
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int off = 0;
    for (int e = 0; e < E; ++e) {
      seg_start[e] = off;
      off += (s_tot[e] + seg_align - 1) / seg_align * seg_align;
    }
  }
}

__global__ void plan_pass3_kernel(const int* __restrict__ es, const int* __restrict__ rank_local,
                                  const int* __restrict__ chunk_base,
                                  const int* __restrict__ seg_start, int* __restrict__ pos, int T,
                                  int k, int E) {
  const int p = blockIdx.x * blockDim.x + threadIdx.x;
  if (p >= T * k) return;
  const int t = p / k;
  const int per = (T + PLAN_CHUNKS - 1) / PLAN_CHUNKS;
  const int chunk = t / per;
  const int e = es[p];
  const int r = rank_local[p];
  pos[p] = (r < 0 || e < 0 || e >= E)
               ? -1
               : seg_start[e] + chunk_base[static_cast<size_t>(chunk) * E + e] + r;
}

// xs[pos[t, j]] = x[t]: one warp per (token, pick)
__global__ void scatter_rows_kernel(const uint8_t* __restrict__ x, uint8_t* __restrict__ xs,
                                    const int* __restrict__ pos, int n_pairs, int k, int row_bytes,
                                    long long xs_rows, int* __restrict__ status) {
  const int lane = threadIdx.x & 31;
  const int p = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (p >= n_pairs) return;
  const int dst = pos[p];
  if (dst < 0 || dst >= xs_rows) {
    if (lane == 0 && status) atomicCAS(status, 0, ST_BAD_INDEX);
    return;
  }
  warp_copy_bytes(xs + static_cast<size_t>(dst) * row_bytes,
                  x + static_cast<size_t>(p / k) * row_bytes, row_bytes, lane);
}

// y[t] = sum_groups ( round_bf16( sum_picks gs * out[pos] ) ), one block per token; every thread
// owns 8 consecutive columns (one 16-byte load per pick)
__global__ void combine_kernel(const __nv_bfloat16* __restrict__ out, const int* __restrict__ pos,
                               const int* __restrict__ es, const float* __restrict__ gs,
                               __nv_bfloat16* __restrict__ y, int T, int k, int dim,
                               int group_size, long long out_rows, int* __restrict__ status) {
  __shared__ int s_row[PLAN_MAX_K];
  __shared__ int s_grp[PLAN_MAX_K];
  __shared__ float s_w[PLAN_MAX_K];
  for (int t = blockIdx.x; t < T; t += gridDim.x) {
    __syncthreads();
    if (static_cast<int>(threadIdx.x) < k) {
      const int o = t * k + threadIdx.x;
      int row = pos[o];
      if (row < 0 || row >= out_rows) {
        row = -1;
        if (status) atomicCAS(status, 0, ST_BAD_INDEX);
      }
      s_row[threadIdx.x] = row;
      s_grp[threadIdx.x] = es[o] / group_size;
      s_w[threadIdx.x] = gs ? gs[o] : 1.0f;
    }
    __syncthreads();
    for (int c = threadIdx.x; c < dim / 8; c += blockDim.x) {
      float tot[8], par[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) tot[i] = par[i] = 0.f;
      for (int j = 0; j < k; ++j) {
        if (j > 0 && s_grp[j] != s_grp[j - 1]) {
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            tot[i] += __bfloat162float(__float2bfloat16_rn(par[i]));
            par[i] = 0.f;
          }
        }
        const int row = s_row[j];
        if (row < 0) continue;
        const float w = s_w[j];
        const uint4 v = *(reinterpret_cast<const uint4*>(out + static_cast<size_t>(row) * dim) + c);
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float2 f = __bfloat1622float2(h[i]);
          par[2 * i] += w * f.x;
          par[2 * i + 1] += w * f.y;
        }
      }
      uint4 o4;
      __nv_bfloat162* oh = reinterpret_cast<__nv_bfloat162*>(&o4);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float a0 = tot[2 * i] + __bfloat162float(__float2bfloat16_rn(par[2 * i]));
        const float a1 = tot[2 * i + 1] + __bfloat162float(__float2bfloat16_rn(par[2 * i + 1]));
        oh[i] = __floats2bfloat162_rn(a0, a1);
      }
      *(reinterpret_cast<uint4*>(y + static_cast<size_t>(t) * dim) + c) = o4;
    }
  }
}

// dout[pos] = gs * dy[t];  dgs[t, j] = <out[pos], dy[t]>   one warp per (token, pick)
__global__ void combine_bwd_kernel(const __nv_bfloat16* __restrict__ dy,
                                   const __nv_bfloat16* __restrict__ out,
                                   const int* __restrict__ pos, const float* __restrict__ gs,
                                   __nv_bfloat16* __restrict__ dout, float* __restrict__ dgs,
                                   int n_pairs, int k, int dim, long long out_rows,
                                   int* __restrict__ status) {
  const int lane = threadIdx.x & 31;
  const int p = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (p >= n_pairs) return;
  const int row = pos[p];
  if (row < 0 || row >= out_rows) {
    if (lane == 0) {
      if (status) atomicCAS(status, 0, ST_BAD_INDEX);
      if (dgs) dgs[p] = 0.f;
    }
    return;
  }
  const float w = gs ? gs[p] : 1.0f;
  const __nv_bfloat162* d2 =
      reinterpret_cast<const __nv_bfloat162*>(dy + static_cast<size_t>(p / k) * dim);
  const __nv_bfloat162* o2 = reinterpret_cast<const __nv_bfloat162*>(out + static_cast<size_t>(row) * dim);
  __nv_bfloat162* r2 = reinterpret_cast<__nv_bfloat162*>(dout + static_cast<size_t>(row) * dim);
  float dot = 0.f;
  for (int i = lane; i < dim / 2; i += 32) {
    const float2 g = __bfloat1622float2(d2[i]);
    if (dgs) {
      const float2 o = __bfloat1622float2(o2[i]);
      dot += g.x * o.x + g.y * o.y;
    }
    r2[i] = __floats2bfloat162_rn(w * g.x, w * g.y);
  }
  if (dgs) {
    dot = warp_sum(dot);
    if (lane == 0) dgs[p] = dot;
  }
}

// Zero the padding rows [count, align_up(count)) of every group of a row buffer.
__global__ void zero_pad_rows_kernel(uint8_t* __restrict__ buf, const int* __restrict__ seg_start,
                                     const int* __restrict__ seg_count, int align, int row_bytes,
                                     long long buf_rows) {
  const int e = blockIdx.x, j = blockIdx.y;
  const int cnt = seg_count[e];
  const int pad = (cnt + align - 1) / align * align - cnt;
  if (j >= pad) return;
  const long long row = static_cast<long long>(seg_start[e]) + cnt + j;
  if (row < 0 || row >= buf_rows) return;
  uint4* dst = reinterpret_cast<uint4*>(buf + static_cast<size_t>(row) * row_bytes);
  for (int i = threadIdx.x; i < row_bytes / 16; i += blockDim.x) dst[i] = make_uint4(0, 0, 0, 0);
}

__global__ void swiglu_bwd_kernel(const __nv_bfloat16* __restrict__ h13,
                                  const __nv_bfloat16* __restrict__ dact,
                                  __nv_bfloat16* __restrict__ dh13, long long rows, int d) {
  const long long n = rows * (d / 2);
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long row = i / (d / 2);
    const int c = static_cast<int>(i - row * (d / 2)) * 2;
    const float2 g = __bfloat1622float2(
        *reinterpret_cast<const __nv_bfloat162*>(h13 + row * 2 * d + c));
    const float2 u = __bfloat1622float2(
        *reinterpret_cast<const __nv_bfloat162*>(h13 + row * 2 * d + d + c));
    const float2 da = __bfloat1622float2(
        *reinterpret_cast<const __nv_bfloat162*>(dact + row * d + c));
    const float s0 = 1.f / (1.f + __expf(-g.x)), s1 = 1.f / (1.f + __expf(-g.y));
    const float dg0 = da.x * u.x * s0 * (1.f + g.x * (1.f - s0));
    const float dg1 = da.y * u.y * s1 * (1.f + g.y * (1.f - s1));
    *reinterpret_cast<__nv_bfloat162*>(dh13 + row * 2 * d + c) = __floats2bfloat162_rn(dg0, dg1);
    *reinterpret_cast<__nv_bfloat162*>(dh13 + row * 2 * d + d + c) =
        __floats2bfloat162_rn(da.x * g.x * s0, da.y * g.y * s1);
  }
}

// ---------------------------------------------------------------------------------------------
// RoPE fused with the head split of the attention input.
//   split:  qkv[B, T, 3 * nh * hd]  ->  q, k (rotated), v   each [B, nh, T, hd]
//   merge:  dq, dk (rotated back), dv [B, nh, T, hd]  ->  dqkv[B, T, 3 * nh * hd]
// Interleaved pairs (even, odd) of the head dimension rotate by the angle of (position, pair):
//   e' = e cos - o sin,  o' = e sin + o cos      (fp32, rounded once; the adjoint rotates back)
// One thread moves 8 elements = 4 pairs.  Replaces the slice / multiply / stack / flatten / cast /
// transpose-copy chain of the reference's `_rope` (terrace/model.py:56-71) with one pass.
// ---------------------------------------------------------------------------------------------
__global__ void rope_split_merge_kernel(__nv_bfloat16* __restrict__ qkv,
                                        __nv_bfloat16* __restrict__ q, __nv_bfloat16* __restrict__ k,
                                        __nv_bfloat16* __restrict__ v, const float* __restrict__ cs,
                                        const float* __restrict__ sn, int B, int T, int nh, int hd,
                                        int merge) {
  const int D = nh * hd;
  const int chunks = 3 * D / 8;                      // 16-byte chunks per token
  const long long total = static_cast<long long>(B) * T * chunks;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const long long bt = i / chunks;
    const int c = static_cast<int>(i - bt * chunks) * 8;       // column inside [0, 3D)
    const int b = static_cast<int>(bt / T), t = static_cast<int>(bt - static_cast<long long>(b) * T);
    const int which = c / D, col = c - which * D;               // 0 q, 1 k, 2 v
    const int h = col / hd, e0 = col - h * hd;
    __nv_bfloat16* flat = qkv + bt * 3 * D + c;
    __nv_bfloat16* head = (which == 0 ? q : which == 1 ? k : v) +
                          ((static_cast<long long>(b) * nh + h) * T + t) * hd + e0;
    uint4 val = *reinterpret_cast<const uint4*>(merge ? head : flat);
    if (which < 2) {
      __nv_bfloat162* pr = reinterpret_cast<__nv_bfloat162*>(&val);
      const float sign = merge ? -1.0f : 1.0f;                 // the adjoint rotates by -angle
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int pair = (e0 >> 1) + j;
        const float co = cs[static_cast<long long>(t) * (hd / 2) + pair];
        const float si = sign * sn[static_cast<long long>(t) * (hd / 2) + pair];
        const float2 eo = __bfloat1622float2(pr[j]);
        // separate roundings (no FMA contraction): the bits of the eager fp32 expression
        pr[j] = __floats2bfloat162_rn(__fsub_rn(__fmul_rn(eo.x, co), __fmul_rn(eo.y, si)),
                                      __fadd_rn(__fmul_rn(eo.x, si), __fmul_rn(eo.y, co)));
      }
    }
    *reinterpret_cast<uint4*>(merge ? flat : head) = val;
  }
}

// ---------------------------------------------------------------------------------------------
// Generic stable counting sort of N items by a small key, in two kernels (used by K1 and K2).
//   pass 1: chunk c (one warp) counts keys of its items and records each item's local rank
//   pass 2 (one block): bucket bases (bucket-major, chunk-minor) -> base[c][b]; totals[b]
// ---------------------------------------------------------------------------------------------
constexpr int SORT_CHUNKS = 64;
constexpr int SORT_MAX_BUCKETS = 1024;

// K1: item p = (row r = p / quota, i = p % quota); key = rslot[p] / epr
__global__ void k1_pass1_kernel(const long long* __restrict__ rslot, int* __restrict__ rank_local,
                                int* __restrict__ chunk_hist, int P, int epr, int rpn) {
  __shared__ int s_cnt[SORT_MAX_BUCKETS];
  const int lane = threadIdx.x;
  const int per = (P + SORT_CHUNKS - 1) / SORT_CHUNKS;
  const int p0 = blockIdx.x * per, p1 = min(P, p0 + per);
  for (int b = lane; b < rpn; b += 32) s_cnt[b] = 0;
  __syncwarp();
  for (int pb = p0; pb < p1; pb += 32) {
    const int p = pb + lane;
    const bool live = p < p1;
    long long slot = live ? rslot[p] : -1;
    int key = live ? static_cast<int>(slot / epr) : -1 - lane;
    const bool ok = live && slot >= 0 && key < rpn;
    if (!ok) key = -1 - lane;
    const unsigned peers = __match_any_sync(0xffffffffu, key);
    if (ok) rank_local[p] = s_cnt[key] + __popc(peers & ((1u << lane) - 1u));
    else if (live) rank_local[p] = -1;
    __syncwarp();
    if (ok && (peers >> lane) == 1u) s_cnt[key] += __popc(peers);
    __syncwarp();
  }
  for (int b = lane; b < rpn; b += 32) chunk_hist[blockIdx.x * rpn + b] = s_cnt[b];
}

__global__ void sort_pass2_kernel(int* __restrict__ chunk_hist, long long* __restrict__ totals,
                                  int n_buckets) {
  __shared__ int s_tot[SORT_MAX_BUCKETS];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  for (int b = warp; b < n_buckets; b += nwarps) {
    const int total = warp_chunk_prefix(chunk_hist, SORT_CHUNKS, n_buckets, b, lane);
    if (lane == 0) {
      s_tot[b] = total;
      totals[b] = total;
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int off = 0;
    for (int b = 0; b < n_buckets; ++b) {
      const int t = s_tot[b];
      s_tot[b] = off;
      off += t;
    }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < SORT_CHUNKS * n_buckets; i += blockDim.x)
    chunk_hist[i] += s_tot[i % n_buckets];
}

// one warp per pair: place index planes, gate bits and the row
__global__ void k1_pass3_kernel(const uint8_t* __restrict__ rx, const long long* __restrict__ rslot,
                                const uint8_t* __restrict__ rgate, uint8_t* __restrict__ send_buf,
                                uint8_t* __restrict__ gate_pairs, long long* __restrict__ r_idx,
                                long long* __restrict__ slot_idx, const int* __restrict__ rank_local,
                                const int* __restrict__ chunk_base, int P, int quota, int epr,
                                int rpn, int row_bytes, int gate_bytes, int* __restrict__ status) {
  const int lane = threadIdx.x & 31;
  const int p = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (p >= P) return;
  const int r = rank_local[p];
  if (r < 0) return;                                   // out-of-range slot: skipped (contained)
  const int per = (P + SORT_CHUNKS - 1) / SORT_CHUNKS;
  const long long slot = rslot[p];
  const int key = static_cast<int>(slot / epr);
  const int dst = chunk_base[(p / per) * rpn + key] + r;
  if (dst < 0 || dst >= P) {
    if (lane == 0 && status) atomicCAS(status, 0, ST_BAD_INDEX);
    return;
  }
  if (lane == 0) {
    r_idx[dst] = p / quota;
    slot_idx[dst] = slot;
  }
  if (lane < gate_bytes)
    gate_pairs[static_cast<size_t>(dst) * gate_bytes + lane] =
        rgate[static_cast<size_t>(p) * gate_bytes + lane];
  warp_copy_bytes(send_buf + static_cast<size_t>(dst) * row_bytes,
                  rx + static_cast<size_t>(p / quota) * row_bytes, row_bytes, lane);
}

// K2 pass 1: item = (token t, run j) with run = j-th group of the token's ascending picks;
// key = destination group.  Also sorts the picks and stores them for pass 3.
__global__ void k2_pass1_kernel(const long long* __restrict__ expert_idx, int* __restrict__ es,
                                int* __restrict__ cols, int* __restrict__ rank_local,
                                int* __restrict__ chunk_hist, int T, int k, int groups_m, int slots,
                                int n_nodes) {
  __shared__ int s_cnt[SORT_MAX_BUCKETS];
  const int lane = threadIdx.x;
  const int per = (T + SORT_CHUNKS - 1) / SORT_CHUNKS;
  const int t0 = blockIdx.x * per, t1 = min(T, t0 + per);
  const int q = k / groups_m;
  for (int b = lane; b < n_nodes; b += 32) s_cnt[b] = 0;
  __syncwarp();
  for (int tb = t0; tb < t1; tb += 32) {
    const int t = tb + lane;
    const bool live = t < t1;
    int e_loc[PLAN_MAX_K];
    if (live) {
      int c_loc[PLAN_MAX_K];
      for (int j = 0; j < k; ++j) {
        e_loc[j] = static_cast<int>(expert_idx[static_cast<size_t>(t) * k + j]);
        c_loc[j] = j;
      }
      for (int i = 1; i < k; ++i) {
        const int ev = e_loc[i], cv = c_loc[i];
        int j = i - 1;
        while (j >= 0 && e_loc[j] > ev) { e_loc[j + 1] = e_loc[j]; c_loc[j + 1] = c_loc[j]; --j; }
        e_loc[j + 1] = ev; c_loc[j + 1] = cv;
      }
      for (int j = 0; j < k; ++j) {
        es[static_cast<size_t>(t) * k + j] = e_loc[j];
        cols[static_cast<size_t>(t) * k + j] = c_loc[j];
      }
    }
    for (int m = 0; m < groups_m; ++m) {
      int key = live ? e_loc[m * q] / slots : -1 - lane;
      const bool ok = live && e_loc[m * q] >= 0 && key < n_nodes;
      if (!ok) key = -1 - lane;
      const unsigned peers = __match_any_sync(0xffffffffu, key);
      if (ok) rank_local[static_cast<size_t>(t) * groups_m + m] =
                  s_cnt[key] + __popc(peers & ((1u << lane) - 1u));
      else if (live) rank_local[static_cast<size_t>(t) * groups_m + m] = -1;
      __syncwarp();
      if (ok && (peers >> lane) == 1u) s_cnt[key] += __popc(peers);
      __syncwarp();
    }
  }
  for (int b = lane; b < n_nodes; b += 32) chunk_hist[blockIdx.x * n_nodes + b] = s_cnt[b];
}

__global__ void k2_pass3_kernel(const uint8_t* __restrict__ hidden, const uint8_t* __restrict__ gates,
                                const int* __restrict__ es, const int* __restrict__ cols,
                                const int* __restrict__ rank_local,
                                const int* __restrict__ chunk_base, uint8_t* __restrict__ payload,
                                long long* __restrict__ mask, uint8_t* __restrict__ gate_rows,
                                long long* __restrict__ u_src, int T, int k, int groups_m, int slots,
                                int n_nodes, int row_bytes, int gate_bytes,
                                int* __restrict__ status) {
  const int lane = threadIdx.x & 31;
  const int item = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  const int P = T * groups_m;
  if (item >= P) return;
  const int r = rank_local[item];
  if (r < 0) return;
  const int t = item / groups_m, m = item - t * groups_m;
  const int q = k / groups_m;
  const int per = (T + SORT_CHUNKS - 1) / SORT_CHUNKS;
  const int key = es[static_cast<size_t>(t) * k + m * q] / slots;
  const int dst = chunk_base[(t / per) * n_nodes + key] + r;
  if (dst < 0 || dst >= P) {
    if (lane == 0 && status) atomicCAS(status, 0, ST_BAD_INDEX);
    return;
  }
  if (lane == 0) u_src[dst] = t;
  if (lane < q) {
    const int e = es[static_cast<size_t>(t) * k + m * q + lane];
    mask[static_cast<size_t>(dst) * q + lane] = e % slots;
  }
  for (int b = lane; b < q * gate_bytes; b += 32) {
    const int i = b / gate_bytes, o = b - i * gate_bytes;
    const int col = cols[static_cast<size_t>(t) * k + m * q + i];
    gate_rows[(static_cast<size_t>(dst) * q + i) * gate_bytes + o] =
        gates[(static_cast<size_t>(t) * k + col) * gate_bytes + o];
  }
  warp_copy_bytes(payload + static_cast<size_t>(dst) * row_bytes,
                  hidden + static_cast<size_t>(t) * row_bytes, row_bytes, lane);
}

}  // namespace tb200

using namespace tb200;

#define LAUNCH_OK() (cudaGetLastError() == cudaSuccess ? TB200_OK : TB200_ERR_LAUNCH)

extern "C" int tb200_passthrough(const void* src, void* dst, size_t bytes, cudaStream_t stream) {
  if (bytes == 0) return TB200_OK;
  const int threads = 256;
  size_t blocks = (bytes / 16 + threads - 1) / threads;
  if (blocks < 1) blocks = 1;
  if (blocks > sm_count() * 8) blocks = sm_count() * 8;
  passthrough_kernel<<<static_cast<unsigned>(blocks), threads, 0, stream>>>(
      static_cast<const uint8_t*>(src), static_cast<uint8_t*>(dst), bytes);
  return LAUNCH_OK();
}

extern "C" int tb200_rmsnorm_fwd(const void* x, const void* w, void* y, float* rstd,
                                 long long rows, int dim, float eps, int is_bf16,
                                 cudaStream_t stream) {
  if (rows == 0) return TB200_OK;
  const int warps = 8;
  const unsigned blocks = static_cast<unsigned>((rows + warps - 1) / warps);
  if (is_bf16)
    rmsnorm_fwd_kernel<__nv_bfloat16><<<blocks, warps * 32, 0, stream>>>(
        static_cast<const __nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(w),
        static_cast<__nv_bfloat16*>(y), rstd, rows, dim, eps);
  else
    rmsnorm_fwd_kernel<float><<<blocks, warps * 32, 0, stream>>>(
        static_cast<const float*>(x), static_cast<const float*>(w), static_cast<float*>(y), rstd,
        rows, dim, eps);
  return LAUNCH_OK();
}

extern "C" int tb200_rmsnorm_bwd(const void* x, const void* w, const void* dy, const float* rstd,
                                 void* dx, float* dw_partial, int n_partial, long long rows,
                                 int dim, int is_bf16, cudaStream_t stream) {
  if (rows == 0 || n_partial <= 0) return TB200_ERR_ARG;
  // column-split kernel: 4 to 8 warps, each lane owning 1 to 4 groups of 8 columns
  int cols_warps = 0;
  if (is_bf16 && dim % 256 == 0)
    for (int wn = 8; wn >= 4 && cols_warps == 0; --wn)
      if (dim % (wn * 256) == 0 && dim / (wn * 256) <= 4) cols_warps = wn;
  if (cols_warps != 0) {
    const int warps = cols_warps;
    switch (dim / (warps * 256)) {
      case 1: launch_rmsnorm_bwd_cols<1, 4>(warps, x, w, dy, rstd, dx, dw_partial, n_partial, rows, dim, stream); break;
      case 2: launch_rmsnorm_bwd_cols<2, 2>(warps, x, w, dy, rstd, dx, dw_partial, n_partial, rows, dim, stream); break;
      case 3: launch_rmsnorm_bwd_cols<3, 2>(warps, x, w, dy, rstd, dx, dw_partial, n_partial, rows, dim, stream); break;
      default: launch_rmsnorm_bwd_cols<4, 1>(warps, x, w, dy, rstd, dx, dw_partial, n_partial, rows, dim, stream); break;
    }
    return LAUNCH_OK();
  }
  if (is_bf16 && dim % 256 == 0 && dim <= 8192) {
    // 4 warps per block keep the per-block accumulators small enough for several blocks per SM
    const size_t smem_vec = 4 * static_cast<size_t>(dim) * sizeof(float);
    static OncePerDevice configured;
    if (configured.need()) {
      cudaFuncSetAttribute(rmsnorm_bwd_vec_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                           4 * 8192 * static_cast<int>(sizeof(float)));
      configured.done();
    }
    rmsnorm_bwd_vec_kernel<<<n_partial, dim3(32, 4), smem_vec, stream>>>(
        static_cast<const __nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(w),
        static_cast<const __nv_bfloat16*>(dy), rstd, static_cast<__nv_bfloat16*>(dx), dw_partial,
        rows, dim);
    return LAUNCH_OK();
  }
  int warps = 8;
  while (warps > 1 && static_cast<size_t>(warps) * dim * sizeof(float) > 160 * 1024) warps >>= 1;
  const size_t smem = static_cast<size_t>(warps) * dim * sizeof(float);
  if (smem > 200 * 1024) return TB200_ERR_SIZE;
  dim3 block(32, warps);
  if (is_bf16) {
    auto kern = rmsnorm_bwd_kernel<__nv_bfloat16>;
    cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    kern<<<n_partial, block, smem, stream>>>(
        static_cast<const __nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(w),
        static_cast<const __nv_bfloat16*>(dy), rstd, static_cast<__nv_bfloat16*>(dx), dw_partial,
        rows, dim);
  } else {
    auto kern = rmsnorm_bwd_kernel<float>;
    cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    kern<<<n_partial, block, smem, stream>>>(static_cast<const float*>(x),
                                             static_cast<const float*>(w),
                                             static_cast<const float*>(dy), rstd,
                                             static_cast<float*>(dx), dw_partial, rows, dim);
  }
  return LAUNCH_OK();
}

extern "C" int tb200_route_select(const float* logits, const float* bias, long long* idx,
                                  float* gates, long long* group_idx, float* load,
                                  float* affinity_sel, int T, int E, int n_groups, int top_k,
                                  int top_groups, int pool, cudaStream_t stream) {
  if (T == 0) return TB200_OK;
  if (E > ROUTE_MAX_E || n_groups > ROUTE_MAX_G || E % n_groups || top_k > 32 ||
      top_k % top_groups || top_groups > n_groups || top_k / top_groups > E / n_groups)
    return TB200_ERR_SIZE;
  route_select_kernel<<<(T + ROUTE_WARPS - 1) / ROUTE_WARPS, ROUTE_WARPS * 32, 0, stream>>>(
      logits, bias, idx, gates, group_idx, load, affinity_sel, T, E, n_groups, top_k, top_groups,
      pool);
  return LAUNCH_OK();
}

extern "C" int tb200_route_select_bwd(const float* dgates, const float* gates,
                                      const float* affinity_sel, const long long* idx,
                                      float* dlogits, int T, int E, int top_k,
                                      cudaStream_t stream) {
  if (T == 0) return TB200_OK;
  route_select_bwd_kernel<<<(T + 127) / 128, 128, 0, stream>>>(dgates, gates, affinity_sel, idx,
                                                             dlogits, T, E, top_k);
  return LAUNCH_OK();
}

extern "C" size_t tb200_plan_scratch_ints(int T, int k, int E) {
  return static_cast<size_t>(T) * k + static_cast<size_t>(PLAN_CHUNKS) * E;
}

// One warp per token chunk; shared memory: [E] counters + [E] lane masks (64 KiB at E = 8192, which
// needs the opt-in limit).
static void launch_plan_pass1(const long long* expert_idx, const float* gates, int* es, float* gs,
                              int* cols, int* rank_local, int* chunk_hist, int T, int k, int E,
                              cudaStream_t stream) {
  static OncePerDevice configured;
  if (configured.need()) {
    cudaFuncSetAttribute(plan_pass1_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                         2 * 8192 * static_cast<int>(sizeof(int)));
    configured.done();
  }
  plan_pass1_kernel<<<PLAN_CHUNKS, 32, 2 * E * sizeof(int), stream>>>(expert_idx, gates, es, gs, cols,
                                                                    rank_local, chunk_hist, T, k, E);
}

extern "C" int tb200_plan_pass1(const long long* expert_idx, const float* gates, int* es,
                                float* gs, int* cols, int* rank_local, int* chunk_hist, int T,
                                int k, int E, cudaStream_t stream) {
  if (k > PLAN_MAX_K || E > 8192) return TB200_ERR_SIZE;
  launch_plan_pass1(expert_idx, gates, es, gs, cols, rank_local, chunk_hist, T, k, E, stream);
  return LAUNCH_OK();
}

extern "C" int tb200_moe_plan(const long long* expert_idx, const float* gates, int* es, float* gs,
                              int* cols, int* pos, int* seg_start, int* seg_count, int* scratch,
                              int T, int k, int E, int seg_align, cudaStream_t stream) {
  if (k > PLAN_MAX_K || E > 8192 || seg_align < 1) return TB200_ERR_SIZE;
  int* rank_local = scratch;
  int* chunk_hist = scratch + static_cast<size_t>(T) * k;
  launch_plan_pass1(expert_idx, gates, es, gs, cols, rank_local, chunk_hist, T, k, E, stream);
  plan_pass2_kernel<<<1, 256, E * sizeof(int), stream>>>(chunk_hist, seg_start, seg_count, E,
                                                         seg_align);
  if (T * k > 0)
    plan_pass3_kernel<<<(T * k + 255) / 256, 256, 0, stream>>>(es, rank_local, chunk_hist,
                                                               seg_start, pos, T, k, E);
  return LAUNCH_OK();
}

extern "C" int tb200_moe_scatter_rows(const void* x, void* xs, const int* pos, int T, int k,
                                      int dim, long long xs_rows, int* status,
                                      cudaStream_t stream) {
  const int n = T * k;
  if (n == 0) return TB200_OK;
  scatter_rows_kernel<<<(n + 7) / 8, 256, 0, stream>>>(static_cast<const uint8_t*>(x),
                                                       static_cast<uint8_t*>(xs), pos, n, k,
                                                       dim * 2, xs_rows, status);
  return LAUNCH_OK();
}

extern "C" int tb200_moe_combine(const void* out, const int* pos, const int* es, const float* gs,
                                 void* y, int T, int k, int dim, int group_size,
                                 long long out_rows, int* status, cudaStream_t stream) {
  if (T == 0) return TB200_OK;
  if (dim % 8 || group_size < 1 || k > PLAN_MAX_K) return TB200_ERR_ARG;
  int threads = dim / 8 >= 256 ? 256 : (dim / 8 >= 128 ? 128 : 64);
  combine_kernel<<<T, threads, 0, stream>>>(static_cast<const __nv_bfloat16*>(out), pos, es, gs,
                                            static_cast<__nv_bfloat16*>(y), T, k, dim, group_size,
                                            out_rows, status);
  return LAUNCH_OK();
}

extern "C" int tb200_moe_combine_bwd(const void* dy, const void* out, const int* pos,
                                     const float* gs, void* dout, float* dgs, int T, int k,
                                     int dim, long long out_rows, int* status,
                                     cudaStream_t stream) {
  const int n = T * k;
  if (n == 0) return TB200_OK;
  if (dim % 2) return TB200_ERR_ARG;
  combine_bwd_kernel<<<(n + 7) / 8, 256, 0, stream>>>(
      static_cast<const __nv_bfloat16*>(dy), static_cast<const __nv_bfloat16*>(out), pos, gs,
      static_cast<__nv_bfloat16*>(dout), dgs, n, k, dim, out_rows, status);
  return LAUNCH_OK();
}

extern "C" int tb200_zero_pad_rows(void* buf, const int* seg_start, const int* seg_count,
                                   int n_groups, int align, int row_bytes, long long buf_rows,
                                   cudaStream_t stream) {
  if (align <= 1 || n_groups <= 0) return TB200_OK;
  if (row_bytes % 16 || align > 1024) return TB200_ERR_ARG;
  dim3 grid(n_groups, align - 1);
  zero_pad_rows_kernel<<<grid, 128, 0, stream>>>(static_cast<uint8_t*>(buf), seg_start, seg_count,
                                                 align, row_bytes, buf_rows);
  return LAUNCH_OK();
}

extern "C" int tb200_swiglu_bwd(const void* h13, const void* dact, void* dh13, long long rows,
                                int d, cudaStream_t stream) {
  if (rows == 0) return TB200_OK;
  if (d % 2) return TB200_ERR_ARG;
  swiglu_bwd_kernel<<<sm_count() * 8, 256, 0, stream>>>(static_cast<const __nv_bfloat16*>(h13),
                                                 static_cast<const __nv_bfloat16*>(dact),
                                                 static_cast<__nv_bfloat16*>(dh13), rows, d);
  return LAUNCH_OK();
}

extern "C" int tb200_rope_split_merge(void* qkv, void* q, void* k, void* v, const float* cos_t,
                                      const float* sin_t, int B, int T, int n_heads, int head_dim,
                                      int merge, cudaStream_t stream) {
  if (B <= 0 || T <= 0) return TB200_OK;
  if (head_dim % 8 || n_heads < 1) return TB200_ERR_ARG;
  const long long total = static_cast<long long>(B) * T * (3 * n_heads * head_dim / 8);
  long long blocks = (total + 255) / 256;
  const long long cap = static_cast<long long>(sm_count()) * 16;
  if (blocks > cap) blocks = cap;
  rope_split_merge_kernel<<<static_cast<int>(blocks), 256, 0, stream>>>(
      static_cast<__nv_bfloat16*>(qkv), static_cast<__nv_bfloat16*>(q),
      static_cast<__nv_bfloat16*>(k), static_cast<__nv_bfloat16*>(v), cos_t, sin_t, B, T, n_heads,
      head_dim, merge);
  return LAUNCH_OK();
}

extern "C" size_t tb200_k1_scratch_ints(int R, int quota, int rpn) {
  return static_cast<size_t>(R) * quota + static_cast<size_t>(SORT_CHUNKS) * rpn;
}

extern "C" int tb200_k1_arrival(const void* rx, const long long* rslot, const void* rgate,
                                void* send_buf, void* gate_pairs, long long* r_idx,
                                long long* slot_idx, long long* i_send, int* scratch, int R,
                                int quota, int epr, int rpn, int row_bytes, int gate_bytes,
                                int* status, cudaStream_t stream) {
  if (rpn > SORT_MAX_BUCKETS || rpn < 1 || epr < 1 || quota < 1 || gate_bytes > 32)
    return TB200_ERR_SIZE;
  const int P = R * quota;
  int* rank_local = scratch;
  int* chunk_hist = scratch + P;
  k1_pass1_kernel<<<SORT_CHUNKS, 32, 0, stream>>>(rslot, rank_local, chunk_hist, P, epr, rpn);
  sort_pass2_kernel<<<1, 256, 0, stream>>>(chunk_hist, i_send, rpn);
  if (P > 0)
    k1_pass3_kernel<<<(P + 7) / 8, 256, 0, stream>>>(
        static_cast<const uint8_t*>(rx), rslot, static_cast<const uint8_t*>(rgate),
        static_cast<uint8_t*>(send_buf), static_cast<uint8_t*>(gate_pairs), r_idx, slot_idx,
        rank_local, chunk_hist, P, quota, epr, rpn, row_bytes, gate_bytes, status);
  return LAUNCH_OK();
}

extern "C" size_t tb200_k2_scratch_ints(int T, int k, int groups_m, int n_nodes) {
  return 2 * static_cast<size_t>(T) * k + static_cast<size_t>(T) * groups_m +
         static_cast<size_t>(SORT_CHUNKS) * n_nodes;
}

extern "C" int tb200_k2_pack(const void* hidden, const long long* expert_idx, const void* gates,
                             void* payload, long long* mask, void* gate_rows, long long* u_src,
                             long long* node_counts, int* scratch, int T, int k, int groups_m,
                             int slots, int n_nodes, int row_bytes, int gate_bytes, int* status,
                             cudaStream_t stream) {
  if (k > PLAN_MAX_K || n_nodes > SORT_MAX_BUCKETS || k % groups_m || k / groups_m > 32 ||
      gate_bytes > 8)
    return TB200_ERR_SIZE;
  // scratch layout: es[T*k] | cols[T*k] | rank_local[T*M] | chunk_hist[SORT_CHUNKS*n_nodes]
  int* es = scratch;
  int* cols = es + static_cast<size_t>(T) * k;
  int* rank_local = cols + static_cast<size_t>(T) * k;
  int* chunk_hist = rank_local + static_cast<size_t>(T) * groups_m;
  k2_pass1_kernel<<<SORT_CHUNKS, 32, 0, stream>>>(expert_idx, es, cols, rank_local, chunk_hist, T,
                                                  k, groups_m, slots, n_nodes);
  sort_pass2_kernel<<<1, 256, 0, stream>>>(chunk_hist, node_counts, n_nodes);
  const int P = T * groups_m;
  if (P > 0)
    k2_pass3_kernel<<<(P + 7) / 8, 256, 0, stream>>>(
        static_cast<const uint8_t*>(hidden), static_cast<const uint8_t*>(gates), es, cols,
        rank_local, chunk_hist, static_cast<uint8_t*>(payload), mask,
        static_cast<uint8_t*>(gate_rows), u_src, T, k, groups_m, slots, n_nodes, row_bytes,
        gate_bytes, status);
  return LAUNCH_OK();
}

// ---------------------------------------------------------------------------------------------
// Allocation-free plan (see no_alloc.h): same three kernels as tb200_moe_plan, scratch in a
// fixed device array owned by this library instead of a caller-provided buffer.
// ---------------------------------------------------------------------------------------------
#include "no_alloc.h"

#include <cstdio>
#include <mutex>

static __device__ __align__(256) int g_plan_static_scratch[TB200_PLAN_STATIC_MAX_INTS];

namespace {
constexpr int kMaxDevices = 64;
int* g_plan_static_ptr[kMaxDevices] = {nullptr};   // device address of the array, per device
std::mutex g_plan_static_mu;

// The array's name is only a host-side handle here; kernels need its device address, which has
// to be asked for once per device with that device current.
int* plan_static_scratch_ptr() {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return nullptr;
  std::lock_guard<std::mutex> lock(g_plan_static_mu);
  if (g_plan_static_ptr[dev] == nullptr) {
    void* p = nullptr;
    const cudaError_t rc = cudaGetSymbolAddress(&p, g_plan_static_scratch);
    if (rc != cudaSuccess || p == nullptr) {
      std::fprintf(stderr, "tb200_moe_plan_static: cudaGetSymbolAddress failed on device %d: %s\n",
                   dev, cudaGetErrorString(rc));
      return nullptr;
    }
    g_plan_static_ptr[dev] = static_cast<int*>(p);
  }
  return g_plan_static_ptr[dev];
}
}  // namespace

extern "C" int tb200_moe_plan_static(const long long* expert_idx, const float* gates, int* es,
                                     float* gs, int* cols, int* pos, int* seg_start,
                                     int* seg_count, int T, int k, int E, int seg_align,
                                     cudaStream_t stream) {
  if (T < 0 || k < 1 || E < 1 || seg_align < 1) return TB200_ERR_ARG;
  if (static_cast<long long>(T) * k > TB200_PLAN_STATIC_MAX_PAIRS ||
      E > TB200_PLAN_STATIC_MAX_EXPERTS || k > PLAN_MAX_K) {
    std::fprintf(stderr,
                 "tb200_moe_plan_static: T*k = %lld, E = %d, k = %d exceed the built-in scratch "
                 "(T*k <= %d, E <= %d, k <= %d); use tb200_moe_plan with your own scratch\n",
                 static_cast<long long>(T) * k, E, k, TB200_PLAN_STATIC_MAX_PAIRS,
                 TB200_PLAN_STATIC_MAX_EXPERTS, PLAN_MAX_K);
    return TB200_ERR_SIZE;
  }
  int* scratch = plan_static_scratch_ptr();
  if (scratch == nullptr) return TB200_ERR_DRIVER;
  // same layout as tb200_moe_plan: rank_local [T*k] | chunk_hist [PLAN_CHUNKS * E]; pass 1 writes
  // every word pass 2 and pass 3 read, so stale contents of an earlier call are harmless
  int* rank_local = scratch;
  int* chunk_hist = scratch + static_cast<size_t>(T) * k;
  launch_plan_pass1(expert_idx, gates, es, gs, cols, rank_local, chunk_hist, T, k, E, stream);
  plan_pass2_kernel<<<1, 256, E * sizeof(int), stream>>>(chunk_hist, seg_start, seg_count, E,
                                                         seg_align);
  if (T * k > 0)
    plan_pass3_kernel<<<(T * k + 255) / 256, 256, 0, stream>>>(es, rank_local, chunk_hist,
                                                               seg_start, pos, T, k, E);
  return LAUNCH_OK();
}
