// T-Route router in ONE kernel for sm_100a: router GEMM on the tensor cores with the whole
// selection in its epilogue, so the logits never touch HBM.
//
//   logits[128 tokens, E] = x[128, H] * W[E, H]^T     tcgen05.mma, 128 x E x 16 per instruction,
//                                                     operands staged by TMA (128-byte swizzle),
//                                                     fp32 accumulator in TMEM
//   epilogue, one thread per token (the token's row of the accumulator is read with tcgen05.ld):
//     affinity = sigmoid(logit); selection score = affinity + bias
//     group score = mean of the `pool` best selection scores of a group
//     top-M groups (descending score, lowest index wins ties)
//     per picked group the top-q experts (descending selection score)
//     gates = raw affinity renormalised over the k picks; expert histogram per CTA
//
// A token's E affinities live in one padded row of shared memory that only its own thread reads
// and writes (dynamic indexing without register spills, conflict-free by the +1 padding).
// Replaces the chain sigmoid(x @ W^T) -> t_route(mode "full") of the reference
// (terrace/routing.py:70-96, 132-134), which the earlier path of this package ran as a GEMM
// launch, a cast and a select launch.  E up to 128 (a multiple of 16); larger routers keep the
// two-launch path.
#include "host_util.h"
#include "launch.h"
#include "ptx_sm100.cuh"
#include "tmap.h"

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <math.h>

namespace tb200 {

constexpr int RT_BM = 128;                 // tokens per CTA
constexpr int RT_BK = 64;                  // 64 bf16 = one 128-byte swizzle line
constexpr int RT_A_BYTES = RT_BM * RT_BK * 2;
constexpr int RT_MAX_STAGES = 8;           // as many as fit beside the affinity rows (host decides)
constexpr int RT_THREADS = 192;            // warp 0 TMA, warp 1 MMA, warps 2..5 epilogue
constexpr int RT_MAX_E = 128;
constexpr int RT_MAX_G = 64;

struct RouterParams {
  const float* bias;        // [E]
  long long* idx;           // [T, k]
  float* gates;             // [T, k]
  long long* group_idx;     // [T, M]
  float* load;              // [E], accumulated
  float* aff_sel;           // [T, k] raw affinity of every pick (for the backward pass)
  int T, E, H, n_groups, top_k, top_groups, pool;
  int stages;               // TMA stages in flight: the kernel streams x once and is bound by them
  int* status;
};

struct RouterCtl {
  uint64_t full[RT_MAX_STAGES];
  uint64_t empty[RT_MAX_STAGES];
  uint64_t acc_full;
  uint32_t tmem_base;
  volatile int abort_flag;
};

// Next element of score(j) = v[j] + b[j], j in [0, n), in the order "value descending, index
// ascending" after (prev, prev_i); start with prev = +inf, prev_i = -1.
__device__ __forceinline__ void rt_next_best(const float* v, const float* b, int n, float& prev,
                                             int& prev_i) {
  float best = -INFINITY;
  int bi = -1;
  for (int j = 0; j < n; ++j) {
    const float x = v[j] + b[j];
    const bool after_prev = x < prev || (x == prev && j > prev_i);
    if (after_prev && (bi < 0 || x > best)) {
      best = x;
      bi = j;
    }
  }
  if (bi < 0) {                    // only with NaNs among the scores
    bi = prev_i < 0 ? 0 : prev_i;
    best = v[bi] + b[bi];
  }
  prev = best;
  prev_i = bi;
}

__global__ void __launch_bounds__(RT_THREADS, 1)
route_fused_kernel(const __grid_constant__ CUtensorMap tmap_x,
                   const __grid_constant__ CUtensorMap tmap_w, const RouterParams p) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* stage_base = reinterpret_cast<uint8_t*>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  const int E = p.E;
  const int b_bytes = E * RT_BK * 2;
  const int stage_bytes = RT_A_BYTES + b_bytes;
  const int STAGES = p.stages;
  float* s_aff = reinterpret_cast<float*>(stage_base + STAGES * stage_bytes);      // [128][E + 1]
  float* s_gsc = s_aff + RT_BM * (E + 1);                                          // [128][G + 1]
  float* s_bias = s_gsc + RT_BM * (p.n_groups + 1);                                // [E]
  int* s_hist = reinterpret_cast<int*>(s_bias + E);                                // [E]
  RouterCtl* ctl = reinterpret_cast<RouterCtl*>(
      (reinterpret_cast<uintptr_t>(s_hist + E) + 15) & ~static_cast<uintptr_t>(15));

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int kblocks = (p.H + RT_BK - 1) / RT_BK;
  const int row0 = blockIdx.x * RT_BM;
  uint32_t tmem_cols = 32;
  while (tmem_cols < static_cast<uint32_t>(E)) tmem_cols <<= 1;

  if (warp == 0 && lane == 0) {
    ctl->abort_flag = 0;
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&ctl->full[s], 1);
      mbar_init(&ctl->empty[s], 1);
    }
    mbar_init(&ctl->acc_full, 1);
    fence_barrier_init();
    prefetch_tmap(&tmap_x);
    prefetch_tmap(&tmap_w);
  }
  if (warp == 1) {
    tmem_alloc(&ctl->tmem_base, tmem_cols);
    tmem_relinquish();
  }
  for (int e = threadIdx.x; e < E; e += RT_THREADS) {
    s_bias[e] = p.bias[e];
    s_hist[e] = 0;
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = ctl->tmem_base;

  if (warp == 0) {
    // =========================== TMA producer =================================================
    if (lane == 0) {
      for (int kb = 0; kb < kblocks; ++kb) {
        const int s = kb % STAGES;
        const uint32_t round = kb / STAGES;
        if (round > 0 && !mbar_wait(&ctl->empty[s], (round - 1) & 1, &ctl->abort_flag)) {
          ctl->abort_flag = ST_TIMEOUT_EMPTY;
          if (p.status) atomicCAS(p.status, 0, ST_TIMEOUT_EMPTY);
          break;
        }
        uint8_t* sa = stage_base + s * stage_bytes;
        mbar_expect_tx(&ctl->full[s], stage_bytes);
        tma_load_2d(sa, &tmap_x, &ctl->full[s], kb * RT_BK, row0);
        tma_load_2d(sa + RT_A_BYTES, &tmap_w, &ctl->full[s], kb * RT_BK, 0);
      }
    }
  } else if (warp == 1) {
    // =========================== MMA issuer ===================================================
    const uint32_t idesc = make_idesc_bf16(RT_BM, E, false, false);
    const uint64_t a_desc0 = make_smem_desc(smem_u32(stage_base), 16, 1024);
    const uint64_t b_desc0 = make_smem_desc(smem_u32(stage_base) + RT_A_BYTES, 16, 1024);
    bool ok = true;
    for (int kb = 0; kb < kblocks && ok; ++kb) {
      const int s = kb % STAGES;
      const uint32_t round = kb / STAGES;
      const bool got = mbar_wait(&ctl->full[s], round & 1, &ctl->abort_flag);
      if (!__all_sync(0xffffffffu, got)) {
        if (lane == 0) {
          ctl->abort_flag = ST_TIMEOUT_FULL;
          if (p.status) atomicCAS(p.status, 0, ST_TIMEOUT_FULL);
        }
        ok = false;
        break;
      }
      tc_fence_after();
      if (lane == 0) {
        const uint64_t stage_off = static_cast<uint64_t>((s * stage_bytes) >> 4);
#pragma unroll
        for (int k4 = 0; k4 < RT_BK / 16; ++k4) {
          const uint64_t off = stage_off + ((k4 * 32) >> 4);     // 16 K elements = 32 bytes
          umma_bf16(tmem_base, a_desc0 + off, b_desc0 + off, idesc, (kb | k4) != 0 ? 1u : 0u);
        }
        umma_commit(&ctl->empty[s]);
      }
      __syncwarp();
    }
    if (ok && lane == 0) umma_commit(&ctl->acc_full);
    __syncwarp();
  } else {
    // =========================== epilogue: one thread per token ================================
    const int quad = warp & 3;                   // TMEM lane quadrant this warp may read
    const int row = quad * 32 + lane;
    const int t = row0 + row;
    const bool got = mbar_wait(&ctl->acc_full, 0, &ctl->abort_flag);
    const bool ok = __all_sync(0xffffffffu, got);
    if (!ok && lane == 0) {
      ctl->abort_flag = ST_TIMEOUT_ACC;
      if (p.status) atomicCAS(p.status, 0, ST_TIMEOUT_ACC);
    }
    if (ok) {
      tc_fence_after();
      float* aff = s_aff + row * (E + 1);
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quad * 32) << 16);
      for (int c = 0; c < E; c += 32) {          // E % 16 == 0: the last chunk may be half full
        uint32_t r[32];
        tmem_ld_32x32(taddr + c, r);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 32; ++j)
          if (c + j < E) aff[c + j] = 1.0f / (1.0f + expf(-__uint_as_float(r[j])));
      }
      if (t < p.T) {
        const int G = p.n_groups, g = E / G, k = p.top_k, M = p.top_groups, q = k / M;
        float* gsc = s_gsc + row * (G + 1);
        // group score = mean of the `pool` best selection scores of the group
        const int width = p.pool < g ? p.pool : g;
        for (int gi = 0; gi < G; ++gi) {
          float prev = INFINITY, sum = 0.f;
          int prev_i = -1;
          for (int r = 0; r < width; ++r) {
            rt_next_best(aff + gi * g, s_bias + gi * g, g, prev, prev_i);
            sum += prev;
          }
          gsc[gi] = sum / width;
        }
        // top-M groups, then per group the top-q experts
        float gprev = INFINITY, total = 0.f;
        int gprev_i = -1;
        const size_t o = static_cast<size_t>(t) * k;
        for (int m = 0; m < M; ++m) {
          {   // next group in descending score order (no bias term on group scores)
            float best = -INFINITY;
            int bi = -1;
            for (int j = 0; j < G; ++j) {
              const float x = gsc[j];
              const bool after_prev = x < gprev || (x == gprev && j > gprev_i);
              if (after_prev && (bi < 0 || x > best)) {
                best = x;
                bi = j;
              }
            }
            if (bi < 0) {
              bi = gprev_i < 0 ? 0 : gprev_i;
              best = gsc[bi];
            }
            gprev = best;
            gprev_i = bi;
          }
          p.group_idx[static_cast<size_t>(t) * M + m] = gprev_i;
          float prev = INFINITY;
          int prev_i = -1;
          for (int r = 0; r < q; ++r) {
            rt_next_best(aff + gprev_i * g, s_bias + gprev_i * g, g, prev, prev_i);
            const int e = gprev_i * g + prev_i;
            const float a = aff[e];
            p.idx[o + m * q + r] = e;
            p.aff_sel[o + m * q + r] = a;
            total += a;                         // sequential sum over the picks: fixed order
            atomicAdd(&s_hist[e], 1);
          }
        }
        for (int j = 0; j < k; ++j) p.gates[o + j] = p.aff_sel[o + j] / total;
      }
    }
    // the four epilogue warps meet, then flush the CTA's expert histogram
    asm volatile("bar.sync 1, 128;" ::: "memory");
    for (int e = threadIdx.x - 64; e < E; e += 128) {
      const int n = s_hist[e];
      if (n > 0) atomicAdd(&p.load[e], static_cast<float>(n));   // integer-valued: order free
    }
  }

  if (ctl->abort_flag != 0) {
    // give copies that may still be in flight time to land before shared memory is released
    const unsigned long long t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 1000000ull) __nanosleep(256);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, tmem_cols);
  }
}

}  // namespace tb200

using namespace tb200;

extern "C" int tb200_route_fused_supported(int E, int H, int n_groups, int top_k, int top_groups) {
  return E >= 16 && E <= RT_MAX_E && E % 16 == 0 && H % 8 == 0 && H >= RT_BK &&
         n_groups >= 1 && n_groups <= RT_MAX_G && E % n_groups == 0 && top_k >= 1 &&
         top_k <= 32 && top_groups >= 1 && top_k % top_groups == 0 && top_groups <= n_groups &&
         top_k / top_groups <= E / n_groups;
}

extern "C" int tb200_route_fused(const void* x, const void* w, const float* bias, long long* idx,
                                 float* gates, long long* group_idx, float* load,
                                 float* affinity_sel, int T, int E, int H, int n_groups,
                                 int top_k, int top_groups, int pool, int* status,
                                 cudaStream_t stream) {
  if (T == 0) return TB200_OK;
  if (!tb200_route_fused_supported(E, H, n_groups, top_k, top_groups) || pool < 1)
    return TB200_ERR_SIZE;
  CUtensorMap tx, tw;
  {
    uint64_t dims[2] = {static_cast<uint64_t>(H), static_cast<uint64_t>(T)};
    uint64_t str[1] = {static_cast<uint64_t>(H) * 2};
    uint32_t box[2] = {RT_BK, RT_BM};
    const int rc = make_tmap(&tx, x, 2, dims, str, box);
    if (rc != TB200_OK) return rc;
  }
  {
    uint64_t dims[2] = {static_cast<uint64_t>(H), static_cast<uint64_t>(E)};
    uint64_t str[1] = {static_cast<uint64_t>(H) * 2};
    uint32_t box[2] = {RT_BK, static_cast<uint32_t>(E)};
    const int rc = make_tmap(&tw, w, 2, dims, str, box);
    if (rc != TB200_OK) return rc;
  }
  // everything but the stages, then as many stages as the 220 KiB opt-in leaves room for
  const size_t fixed = 1024 + sizeof(float) * (static_cast<size_t>(RT_BM) * (E + 1) +
                                               static_cast<size_t>(RT_BM) * (n_groups + 1) + 2 * E) +
                       sizeof(RouterCtl) + 64;
  const size_t stage_bytes = RT_A_BYTES + static_cast<size_t>(E) * RT_BK * 2;
  int stages = static_cast<int>((220 * 1024 - fixed) / stage_bytes);
  if (stages > RT_MAX_STAGES) stages = RT_MAX_STAGES;
  if (stages < 2) return TB200_ERR_SIZE;
  RouterParams p{bias, idx, gates, group_idx, load, affinity_sel, T, E, H, n_groups, top_k,
                 top_groups, pool, stages, status};
  const size_t smem = fixed + stages * stage_bytes;
  static OncePerDevice configured;
  if (configured.need()) {
    if (cudaFuncSetAttribute(route_fused_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             220 * 1024) != cudaSuccess)
      return TB200_ERR_LAUNCH;
    configured.done();
  }
  if (smem > 220 * 1024) return TB200_ERR_SIZE;
  route_fused_kernel<<<(T + RT_BM - 1) / RT_BM, RT_THREADS, smem, stream>>>(tx, tw, p);
  return cudaGetLastError() == cudaSuccess ? TB200_OK : TB200_ERR_LAUNCH;
}
