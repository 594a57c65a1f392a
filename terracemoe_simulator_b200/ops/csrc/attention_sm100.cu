// Causal / full self-attention for sm_100a on the 5th-generation tensor cores: forward (O, LSE)
// and backward (dQ, dK, dV), bf16 in / out, fp32 softmax and accumulation, head width 64 or 128.
//
// Every matmul is a tcgen05.mma (cta_group::1, 128 rows) with operands in shared memory
// (128-byte swizzle) and the result in TMEM; Q / K / V / dO tiles arrive by TMA; one thread per
// query (or key) row reads its row of S or dP from TMEM with tcgen05.ld, so row maxima and sums
// need no shuffles.  P and dS go back to shared memory as bf16 in the same swizzled image that
// TMA produces, which one descriptor reads as a K-major operand (P V, dS K) and another as an
// M-major operand (P^T dO, dS^T Q) without moving a byte.
//
//   forward    one CTA per (head, 128 queries): S_j = Q K_j^T (two TMEM buffers, so S_{j+1} is
//              computed while the softmax of block j runs), online softmax, P_j V_j into TMEM,
//              O accumulated in registers with the running-max correction, K / V double-buffered.
//   dK, dV     one CTA per (head, 128 keys), loop over query blocks: S and dP in TMEM, P and dS
//              to shared memory, dV += P^T dO and dK += dS^T Q accumulate in TMEM.
//   dQ         one CTA per (head, 128 queries), loop over key blocks: dQ += dS K in TMEM.
// No float atomics anywhere: results are deterministic.
//
// The reference computes attention with torch's scaled_dot_product_attention
// (terrace/model.py:55-71); this file replaces that library call on B200.
#include "host_util.h"
#include "launch.h"
#include "ptx_sm100.cuh"

#include <cuda.h>
#include <cuda_runtime.h>
#include <math.h>
#include <stdio.h>

namespace tb200 {

constexpr int AT_ROWS = 128;          // rows per block (queries or keys)
constexpr int AT_THREADS = 320;       // warp 0 TMA, warp 1 MMA, warps 2..9: two threads per row
                                      // (columns 0-63 and 64-127 of a 128-wide block), i.e. two
                                      // row warps per scheduler so that their latencies overlap
constexpr int AT_ROW_THREADS = 256;    // (10 warps = 3 on the fullest scheduler: 168 registers each)
constexpr int AT_BOX = AT_ROWS * 128; // one TMA box: 128 rows x 64 bf16 = 16 KiB
constexpr int AT_TMEM_COLS = 512;

struct AttnParams {
  int S;                 // sequence length (multiple of 128)
  int BH;                // batch * heads
  int causal;
  float scale;           // 1 / sqrt(D)
  float scale_log2;      // scale * log2(e)
  __nv_bfloat16* O;      // fwd out            [BH, S, D]
  float* LSE;            // fwd out / bwd in   [BH, S]  natural log-sum-exp of the scaled scores
  const float* DELTA;    // bwd in             [BH, S]  rowsum(dO * O)
  __nv_bfloat16* dQ;
  __nv_bfloat16* dK;
  __nv_bfloat16* dV;
  int* status;
};

struct __align__(8) AttnCtl {
  uint64_t bar[16];
  uint32_t tmem_base;
  volatile int abort_flag;
  float xch[2][2][AT_ROWS];   // [block parity][column half][row]: row maxima / sums exchanged
};

// barrier among the 256 row threads only (the TMA and MMA warps never join it)
__device__ __forceinline__ void at_row_sync() {
  asm volatile("bar.sync 1, %0;" ::"n"(AT_ROW_THREADS) : "memory");
}

__device__ __forceinline__ void at_abort(AttnCtl* ctl, int* status, int code) {
  ctl->abort_flag = code;
  if (status != nullptr) atomicCAS(status, 0, code);
}
__device__ __forceinline__ bool at_wait(AttnCtl* ctl, int b, uint32_t parity) {
  const bool got = mbar_wait(&ctl->bar[b], parity, &ctl->abort_flag);
  return __all_sync(0xffffffffu, got);
}
__device__ __forceinline__ uint32_t at_pack(float a, float b) {
  __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&v);
}

// A tile of 128 rows x D bf16 is D / 64 boxes of 128 rows x 128 bytes, 128-byte swizzled.
// K-major view (row = M or N index, the 64 contiguous elements run along K):
__device__ __forceinline__ uint64_t at_desc_k(uint32_t tile_addr, int k16) {
  return make_smem_desc(tile_addr + (k16 >> 2) * AT_BOX + (k16 & 3) * 32, 16, 1024);
}
// MN-major view (row = K index, the 64 contiguous elements run along M or N; 16 rows per step):
__device__ __forceinline__ uint64_t at_desc_mn(uint32_t tile_addr, int k16) {
  return make_smem_desc(tile_addr + k16 * 2048, AT_BOX, 1024);
}

// 32 consecutive columns [c0, c0 + 32) of row `row`, as 16 packed bf16 pairs, into a swizzled
// 128-row tile whose rows hold 128 columns (two boxes).
__device__ __forceinline__ void at_store_chunk32(uint8_t* tile, int row, int c0,
                                                 const uint32_t (&w)[16]) {
  uint8_t* base = tile + (c0 >> 6) * AT_BOX + row * 128;
  const int chunk0 = (c0 & 63) >> 3;
#pragma unroll
  for (int q = 0; q < 4; ++q) {
    uint4 v = make_uint4(w[q * 4], w[q * 4 + 1], w[q * 4 + 2], w[q * 4 + 3]);
    *reinterpret_cast<uint4*>(base + (((chunk0 + q) ^ (row & 7)) << 4)) = v;
  }
}

template <int D>
__device__ __forceinline__ void at_load_tile(uint8_t* dst, const CUtensorMap* tm, uint64_t* bar,
                                             int row0) {
#pragma unroll
  for (int c = 0; c < D / 64; ++c) tma_load_2d(dst + c * AT_BOX, tm, bar, c * 64, row0);
}

__device__ __forceinline__ void at_setup(AttnCtl* ctl, int n_bars, const int* counts, int warp,
                                         int lane) {
  if (threadIdx.x == 0) {
    ctl->abort_flag = 0;
    for (int i = 0; i < n_bars; ++i) mbar_init(&ctl->bar[i], counts[i]);
    fence_barrier_init();
  }
  if (warp == 1) {
    tmem_alloc(&ctl->tmem_base, AT_TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  (void)lane;
}

__device__ __forceinline__ void at_teardown(AttnCtl* ctl, int warp, uint32_t tmem_base) {
  if (ctl->abort_flag != 0) {
    const unsigned long long t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 1000000ull) __nanosleep(256);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, AT_TMEM_COLS);
  }
}

// Row maximum of 64 scores held in registers; with MASK only columns [0, n_valid) count.
// Four independent chains, so consecutive instructions do not wait on one another.
template <bool MASK>
__device__ __forceinline__ float at_row_max64(const uint32_t (&sv)[2][32], int n_valid) {
  float m0 = -INFINITY, m1 = -INFINITY, m2 = -INFINITY, m3 = -INFINITY;
#pragma unroll
  for (int c = 0; c < 2; ++c) {
#pragma unroll
    for (int i = 0; i < 32; i += 4) {
      float x0 = __uint_as_float(sv[c][i]), x1 = __uint_as_float(sv[c][i + 1]);
      float x2 = __uint_as_float(sv[c][i + 2]), x3 = __uint_as_float(sv[c][i + 3]);
      if (MASK) {
        if (c * 32 + i >= n_valid) x0 = -INFINITY;
        if (c * 32 + i + 1 >= n_valid) x1 = -INFINITY;
        if (c * 32 + i + 2 >= n_valid) x2 = -INFINITY;
        if (c * 32 + i + 3 >= n_valid) x3 = -INFINITY;
      }
      m0 = fmaxf(m0, x0);
      m1 = fmaxf(m1, x1);
      m2 = fmaxf(m2, x2);
      m3 = fmaxf(m3, x3);
    }
  }
  return fmaxf(fmaxf(m0, m1), fmaxf(m2, m3));
}

// exp2(s * scale_log2 - mxs) of 32 scores -> bf16 into columns [c0, c0 + 32) of row `row` of the
// swizzled P tile (one 16-byte store per 8 values); returns their sum.
template <bool MASK>
__device__ __forceinline__ float at_exp_store32(const uint32_t (&sv)[32], uint8_t* tile, int row,
                                                int c0, int col0, int n_valid, float scale_log2,
                                                float mxs) {
  float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;
  uint8_t* base = tile + (c0 >> 6) * AT_BOX + row * 128;
  const int chunk0 = (c0 & 63) >> 3;
#pragma unroll
  for (int q = 0; q < 4; ++q) {
    uint32_t w[4];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int i = q * 8 + h * 4;
      float a = exp2f(__uint_as_float(sv[i]) * scale_log2 - mxs);
      float b = exp2f(__uint_as_float(sv[i + 1]) * scale_log2 - mxs);
      float c = exp2f(__uint_as_float(sv[i + 2]) * scale_log2 - mxs);
      float d = exp2f(__uint_as_float(sv[i + 3]) * scale_log2 - mxs);
      if (MASK) {
        if (col0 + i >= n_valid) a = 0.f;
        if (col0 + i + 1 >= n_valid) b = 0.f;
        if (col0 + i + 2 >= n_valid) c = 0.f;
        if (col0 + i + 3 >= n_valid) d = 0.f;
      }
      s0 += a;
      s1 += b;
      s2 += c;
      s3 += d;
      w[h * 2] = at_pack(a, b);
      w[h * 2 + 1] = at_pack(c, d);
    }
    *reinterpret_cast<uint4*>(base + (((chunk0 + q) ^ (row & 7)) << 4)) =
        make_uint4(w[0], w[1], w[2], w[3]);
  }
  return (s0 + s1) + (s2 + s3);
}

// =============================================================================================
// forward
// =============================================================================================
enum { FB_Q = 0, FB_KF = 1, FB_KE = 3, FB_VF = 5, FB_VE = 7, FB_SF = 9, FB_SE = 11, FB_PF = 13,
       FB_PV = 14, FB_N = 15 };

template <int D>
__global__ void __launch_bounds__(AT_THREADS, 1)
attn_fwd_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                const __grid_constant__ CUtensorMap tm_v, const AttnParams p) {
  constexpr int TILE = AT_ROWS * D * 2;
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* base = reinterpret_cast<uint8_t*>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  uint8_t* sQ = base;
  uint8_t* sK = sQ + TILE;            // two stages
  uint8_t* sV = sK + 2 * TILE;        // two stages
  uint8_t* sP = sV + 2 * TILE;        // 128 x 128 bf16
  AttnCtl* ctl = reinterpret_cast<AttnCtl*>(sP + 2 * AT_BOX);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nqb = p.S / AT_ROWS;
  const int qb = nqb - 1 - static_cast<int>(blockIdx.x) / p.BH;   // long rows first
  const int bh = static_cast<int>(blockIdx.x) % p.BH;
  const int n_kv = p.causal ? qb + 1 : nqb;
  const int row_base = bh * p.S;

  {
    const int counts[FB_N] = {1, 1, 1, 1, 1, 1, 1, 1, 1, 1, 1, 8, 8, 8, 1};
    at_setup(ctl, FB_N, counts, warp, lane);
  }
  const uint32_t tmem = ctl->tmem_base;

  if (warp == 0) {
    if (lane == 0) {
      prefetch_tmap(&tm_q);
      prefetch_tmap(&tm_k);
      prefetch_tmap(&tm_v);
      mbar_expect_tx(&ctl->bar[FB_Q], TILE);
      at_load_tile<D>(sQ, &tm_q, &ctl->bar[FB_Q], row_base + qb * AT_ROWS);
      for (int j = 0; j < n_kv; ++j) {
        const int s = j & 1, r = j >> 1;
        if (r > 0 && !mbar_wait(&ctl->bar[FB_KE + s], (r - 1) & 1, &ctl->abort_flag)) {
          at_abort(ctl, p.status, ST_TIMEOUT_EMPTY);
          break;
        }
        mbar_expect_tx(&ctl->bar[FB_KF + s], TILE);
        at_load_tile<D>(sK + s * TILE, &tm_k, &ctl->bar[FB_KF + s], row_base + j * AT_ROWS);
        if (r > 0 && !mbar_wait(&ctl->bar[FB_VE + s], (r - 1) & 1, &ctl->abort_flag)) {
          at_abort(ctl, p.status, ST_TIMEOUT_EMPTY);
          break;
        }
        mbar_expect_tx(&ctl->bar[FB_VF + s], TILE);
        at_load_tile<D>(sV + s * TILE, &tm_v, &ctl->bar[FB_VF + s], row_base + j * AT_ROWS);
      }
    }
  } else if (warp == 1) {
    constexpr uint32_t idesc_qk = make_idesc_bf16(128, 128, false, false);
    constexpr uint32_t idesc_pv = make_idesc_bf16(128, D, false, true);
    const uint32_t q_addr = smem_u32(sQ), p_addr = smem_u32(sP);
    bool ok = at_wait(ctl, FB_Q, 0);
    if (!ok && lane == 0) at_abort(ctl, p.status, ST_TIMEOUT_FULL);
    auto issue_qk = [&](int j) -> bool {
      const int s = j & 1, r = j >> 1;
      if (!at_wait(ctl, FB_KF + s, r & 1)) return false;
      if (r > 0 && !at_wait(ctl, FB_SE + s, (r - 1) & 1)) return false;
      tc_fence_after();
      if (lane == 0) {
        const uint32_t k_addr = smem_u32(sK + s * TILE);
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk)
          umma_bf16(tmem + s * 128, at_desc_k(q_addr, kk), at_desc_k(k_addr, kk), idesc_qk,
                    kk != 0 ? 1u : 0u);
        umma_commit(&ctl->bar[FB_SF + s]);
        umma_commit(&ctl->bar[FB_KE + s]);
      }
      __syncwarp();
      return true;
    };
    if (ok) ok = issue_qk(0);
    for (int j = 0; j < n_kv && ok; ++j) {
      if (j + 1 < n_kv) ok = issue_qk(j + 1);
      if (!ok) break;
      const int s = j & 1, r = j >> 1;
      if (!at_wait(ctl, FB_PF, j & 1) || !at_wait(ctl, FB_VF + s, r & 1)) {
        ok = false;
        break;
      }
      tc_fence_after();
      if (lane == 0) {
        const uint32_t v_addr = smem_u32(sV + s * TILE);
#pragma unroll
        for (int kk = 0; kk < AT_ROWS / 16; ++kk)
          umma_bf16(tmem + 256, at_desc_k(p_addr, kk), at_desc_mn(v_addr, kk), idesc_pv,
                    kk != 0 ? 1u : 0u);
        umma_commit(&ctl->bar[FB_PV]);
        umma_commit(&ctl->bar[FB_VE + s]);
      }
      __syncwarp();
    }
    if (!ok && lane == 0) at_abort(ctl, p.status, ST_TIMEOUT_ACC);
  } else {
    const int quad = warp & 3;
    const int half = (warp - 2) >> 2;          // which 64 columns of a block this thread owns
    const int row = quad * 32 + lane;
    const uint32_t lane_addr = tmem + (static_cast<uint32_t>(quad * 32) << 16);
    const int q_glob = qb * AT_ROWS + row;
    constexpr int DH = D / 2;                  // output columns per thread
    float m = -INFINITY, l = 0.f, alpha_pending = 0.f;
    float o[DH];
#pragma unroll
    for (int i = 0; i < DH; ++i) o[i] = 0.f;
    bool ok = true;
    for (int j = 0; j < n_kv; ++j) {
      const int s = j & 1, r = j >> 1;
      ok = ok && at_wait(ctl, FB_SF + s, r & 1);
      tc_fence_after();
      // on the diagonal block of a causal mask this thread sees columns [0, n_valid) of its half
      const bool diag = p.causal && j == qb;
      const int n_valid = min(max(row - half * 64 + 1, 0), 64);
      // pass 1: row maximum over this thread's 64 columns (both loads in flight), then over both
      // halves of the row.  The scores are read again in pass 2: keeping them in registers next
      // to the 64 output accumulators spilled and ran slower.
      float mx = -INFINITY;
      if (ok) {
        uint32_t sv[2][32];
        tmem_ld_32x32(lane_addr + s * 128 + half * 64, sv[0]);
        tmem_ld_32x32(lane_addr + s * 128 + half * 64 + 32, sv[1]);
        tmem_ld_wait();
        mx = diag ? at_row_max64<true>(sv, n_valid) : at_row_max64<false>(sv, 64);
      }
      ctl->xch[s][half][row] = mx;
      at_row_sync();                          // every row thread reaches this, also after a timeout
      mx = fmaxf(fmaxf(mx, ctl->xch[s][half ^ 1][row]), m);
      if (!ok) continue;
      const float alpha = (m == -INFINITY) ? 0.f : exp2f((m - mx) * p.scale_log2);
      if (j > 0) {
        if (!at_wait(ctl, FB_PV, (j - 1) & 1)) {
          ok = false;
          continue;
        }
        tc_fence_after();
      }
      // pass 2: probabilities to shared memory; the previous block's P V (computed against the
      // previous maximum) is loaded alongside each score chunk and folded into O
      const float mxs = mx * p.scale_log2;
      float rowsum = 0.f;
      static_assert(DH / 32 <= 2, "one P V chunk per score chunk");
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        uint32_t sv[32], pv[32];
        const bool fold = j > 0 && c < DH / 32;
        tmem_ld_32x32(lane_addr + s * 128 + half * 64 + c * 32, sv);
        if (fold) tmem_ld_32x32(lane_addr + 256 + half * DH + c * 32, pv);
        tmem_ld_wait();
        rowsum += diag ? at_exp_store32<true>(sv, sP, row, half * 64 + c * 32, c * 32, n_valid,
                                              p.scale_log2, mxs)
                       : at_exp_store32<false>(sv, sP, row, half * 64 + c * 32, c * 32, 64,
                                               p.scale_log2, mxs);
        if (c < DH / 32) {
          if (fold) {
#pragma unroll
            for (int i = 0; i < 32; ++i)
              o[(c < DH / 32 ? c : 0) * 32 + i] =
                  o[(c < DH / 32 ? c : 0) * 32 + i] * alpha_pending + __uint_as_float(pv[i]);
          }
        }
      }
      alpha_pending = alpha;
      l = l * alpha + rowsum;                 // this half's share of the row sum
      m = mx;
      fence_proxy_async_smem();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) {
        mbar_arrive(&ctl->bar[FB_PF]);
        mbar_arrive(&ctl->bar[FB_SE + s]);
      }
    }
    if (ok && !at_wait(ctl, FB_PV, (n_kv - 1) & 1)) ok = false;
    // both halves of a row add their sums (buffer of the parity the last block did not use)
    ctl->xch[n_kv & 1][half][row] = l;
    at_row_sync();
    l += ctl->xch[n_kv & 1][half ^ 1][row];
    if (ok) {
      tc_fence_after();
      const float inv = 1.f / l;
      __nv_bfloat16* orow = p.O + (static_cast<size_t>(row_base) + q_glob) * D + half * DH;
#pragma unroll
      for (int c = 0; c < DH / 32; ++c) {
        uint32_t v[32];
        tmem_ld_32x32(lane_addr + 256 + half * DH + c * 32, v);
        tmem_ld_wait();
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          uint4 out;
          uint32_t* po = reinterpret_cast<uint32_t*>(&out);
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const int e = q * 8 + 2 * i;
            const float a = (o[c * 32 + e] * alpha_pending + __uint_as_float(v[e])) * inv;
            const float b = (o[c * 32 + e + 1] * alpha_pending + __uint_as_float(v[e + 1])) * inv;
            po[i] = at_pack(a, b);
          }
          *reinterpret_cast<uint4*>(orow + c * 32 + q * 8) = out;
        }
      }
      if (half == 0) p.LSE[static_cast<size_t>(row_base) + q_glob] = m * p.scale + logf(l);
    } else if (lane == 0) {
      at_abort(ctl, p.status, ST_TIMEOUT_ACC);
    }
  }
  at_teardown(ctl, warp, tmem);
}

// =============================================================================================
// backward: delta = rowsum(dO * O)
// =============================================================================================
__global__ void attn_delta_kernel(const __nv_bfloat16* __restrict__ O,
                                  const __nv_bfloat16* __restrict__ dO, float* __restrict__ delta,
                                  long long rows, int D) {
  const long long row = static_cast<long long>(blockIdx.x) * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= rows) return;
  const int lane = threadIdx.x & 31;
  const uint2* a = reinterpret_cast<const uint2*>(O + row * D);
  const uint2* b = reinterpret_cast<const uint2*>(dO + row * D);
  float acc = 0.f;
  for (int i = lane; i < D / 4; i += 32) {
    const uint2 x = a[i], y = b[i];
    const float2 x0 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&x.x));
    const float2 x1 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&x.y));
    const float2 y0 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&y.x));
    const float2 y1 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&y.y));
    acc += x0.x * y0.x + x0.y * y0.y + x1.x * y1.x + x1.y * y1.y;
  }
#pragma unroll
  for (int d = 16; d > 0; d >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, d);
  if (lane == 0) delta[row] = acc;
}

template <bool WRITE_P, bool MASK>
__device__ __forceinline__ void at_p_ds_cols(uint32_t lane_addr, uint8_t* sP, uint8_t* sdS,
                                             int row, int half, float lse_l2, float delta,
                                             float scale, float scale_log2, int limit) {
  // this thread's 64 columns of S and of dP: four TMEM loads in flight, one wait
  uint32_t sv[2][32], dv[2][32];
#pragma unroll
  for (int c = 0; c < 2; ++c) {
    tmem_ld_32x32(lane_addr + half * 64 + c * 32, sv[c]);
    tmem_ld_32x32(lane_addr + 128 + half * 64 + c * 32, dv[c]);
  }
  tmem_ld_wait();
  const float dsc = delta * scale;
#pragma unroll
  for (int c = 0; c < 2; ++c) {
    const int col0 = half * 64 + c * 32;
    const int off = (col0 >> 6) * AT_BOX + row * 128;
    const int chunk0 = (col0 & 63) >> 3;
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      uint32_t wp[4], wd[4];
#pragma unroll
      for (int h = 0; h < 4; ++h) {
        const int i = q * 8 + h * 2;
        float p0 = exp2f(__uint_as_float(sv[c][i]) * scale_log2 - lse_l2);
        float p1 = exp2f(__uint_as_float(sv[c][i + 1]) * scale_log2 - lse_l2);
        if (MASK) {
          if (col0 + i > limit) p0 = 0.f;
          if (col0 + i + 1 > limit) p1 = 0.f;
        }
        const float d0 = p0 * (__uint_as_float(dv[c][i]) * scale - dsc);
        const float d1 = p1 * (__uint_as_float(dv[c][i + 1]) * scale - dsc);
        wp[h] = at_pack(p0, p1);
        wd[h] = at_pack(d0, d1);
      }
      const int sw = ((chunk0 + q) ^ (row & 7)) << 4;
      if (WRITE_P)
        *reinterpret_cast<uint4*>(sP + off + sw) = make_uint4(wp[0], wp[1], wp[2], wp[3]);
      *reinterpret_cast<uint4*>(sdS + off + sw) = make_uint4(wd[0], wd[1], wd[2], wd[3]);
    }
  }
}

// One thread's 64 columns of S and dP (TMEM) -> P and dS in shared memory.
//   p  = exp2(s * scale_log2 - lse * log2e),  ds = p * (dp - delta) * scale
// Columns (keys) > limit are masked; limit >= 127 means no mask.
template <bool WRITE_P>
__device__ __forceinline__ void at_p_ds_row(uint32_t lane_addr, uint8_t* sP, uint8_t* sdS, int row,
                                            int half, float lse_l2, float delta, float scale,
                                            float scale_log2, int limit, bool masked) {
  if (masked)
    at_p_ds_cols<WRITE_P, true>(lane_addr, sP, sdS, row, half, lse_l2, delta, scale, scale_log2,
                                limit);
  else
    at_p_ds_cols<WRITE_P, false>(lane_addr, sP, sdS, row, half, lse_l2, delta, scale, scale_log2,
                                 limit);
}

// =============================================================================================
// backward: dK, dV  (one CTA per key block, loop over query blocks)
// =============================================================================================
enum { KB_KV = 0, KB_QF = 1, KB_QE = 2, KB_SF = 3, KB_PF = 4, KB_DONE = 5, KB_N = 6 };

template <int D>
__global__ void __launch_bounds__(AT_THREADS, 1)
attn_bwd_dkdv_kernel(const __grid_constant__ CUtensorMap tm_q,
                     const __grid_constant__ CUtensorMap tm_k,
                     const __grid_constant__ CUtensorMap tm_v,
                     const __grid_constant__ CUtensorMap tm_do, const AttnParams p) {
  constexpr int TILE = AT_ROWS * D * 2;
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* base = reinterpret_cast<uint8_t*>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  uint8_t* sK = base;
  uint8_t* sV = sK + TILE;
  uint8_t* sQ = sV + TILE;
  uint8_t* sdO = sQ + TILE;
  uint8_t* sP = sdO + TILE;
  uint8_t* sdS = sP + 2 * AT_BOX;
  AttnCtl* ctl = reinterpret_cast<AttnCtl*>(sdS + 2 * AT_BOX);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nb = p.S / AT_ROWS;
  const int jb = static_cast<int>(blockIdx.x) / p.BH;              // key block: long loops first
  const int bh = static_cast<int>(blockIdx.x) % p.BH;
  const int i0 = p.causal ? jb : 0;
  const int n_it = nb - i0;
  const int row_base = bh * p.S;
  {
    const int counts[KB_N] = {1, 1, 1, 1, 8, 1};
    at_setup(ctl, KB_N, counts, warp, lane);
  }
  const uint32_t tmem = ctl->tmem_base;
  // TMEM columns: S [0,128)  dP [128,256)  dV [256,256+D)  dK [256+D,256+2D)

  if (warp == 0) {
    if (lane == 0) {
      prefetch_tmap(&tm_q);
      prefetch_tmap(&tm_do);
      mbar_expect_tx(&ctl->bar[KB_KV], 2 * TILE);
      at_load_tile<D>(sK, &tm_k, &ctl->bar[KB_KV], row_base + jb * AT_ROWS);
      at_load_tile<D>(sV, &tm_v, &ctl->bar[KB_KV], row_base + jb * AT_ROWS);
      for (int it = 0; it < n_it; ++it) {
        if (it > 0 && !mbar_wait(&ctl->bar[KB_QE], (it - 1) & 1, &ctl->abort_flag)) {
          at_abort(ctl, p.status, ST_TIMEOUT_EMPTY);
          break;
        }
        mbar_expect_tx(&ctl->bar[KB_QF], 2 * TILE);
        at_load_tile<D>(sQ, &tm_q, &ctl->bar[KB_QF], row_base + (i0 + it) * AT_ROWS);
        at_load_tile<D>(sdO, &tm_do, &ctl->bar[KB_QF], row_base + (i0 + it) * AT_ROWS);
      }
    }
  } else if (warp == 1) {
    constexpr uint32_t idesc_s = make_idesc_bf16(128, 128, false, false);
    constexpr uint32_t idesc_g = make_idesc_bf16(128, D, true, true);
    const uint32_t k_addr = smem_u32(sK), v_addr = smem_u32(sV), q_addr = smem_u32(sQ),
                   do_addr = smem_u32(sdO), p_addr = smem_u32(sP), ds_addr = smem_u32(sdS);
    bool ok = at_wait(ctl, KB_KV, 0);
    for (int it = 0; it < n_it && ok; ++it) {
      if (!at_wait(ctl, KB_QF, it & 1)) {
        ok = false;
        break;
      }
      tc_fence_after();
      if (lane == 0) {
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk)
          umma_bf16(tmem, at_desc_k(q_addr, kk), at_desc_k(k_addr, kk), idesc_s, kk != 0);
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk)
          umma_bf16(tmem + 128, at_desc_k(do_addr, kk), at_desc_k(v_addr, kk), idesc_s, kk != 0);
        umma_commit(&ctl->bar[KB_SF]);
      }
      __syncwarp();
      if (!at_wait(ctl, KB_PF, it & 1)) {
        ok = false;
        break;
      }
      tc_fence_after();
      if (lane == 0) {
#pragma unroll
        for (int kk = 0; kk < AT_ROWS / 16; ++kk)
          umma_bf16(tmem + 256, at_desc_mn(p_addr, kk), at_desc_mn(do_addr, kk), idesc_g,
                    (it | kk) != 0);
#pragma unroll
        for (int kk = 0; kk < AT_ROWS / 16; ++kk)
          umma_bf16(tmem + 256 + D, at_desc_mn(ds_addr, kk), at_desc_mn(q_addr, kk), idesc_g,
                    (it | kk) != 0);
        umma_commit(&ctl->bar[KB_QE]);     // Q / dO may be overwritten
        umma_commit(&ctl->bar[KB_DONE]);   // P / dS may be overwritten; accumulators current
      }
      __syncwarp();
    }
    if (!ok && lane == 0) at_abort(ctl, p.status, ST_TIMEOUT_ACC);
  } else {
    const int quad = warp & 3;
    const int half = (warp - 2) >> 2;
    const int row = quad * 32 + lane;
    const uint32_t lane_addr = tmem + (static_cast<uint32_t>(quad * 32) << 16);
    bool ok = true;
    for (int it = 0; it < n_it && ok; ++it) {
      const int ib = i0 + it;
      const size_t g = static_cast<size_t>(row_base) + ib * AT_ROWS + row;   // this thread's query
      const float lse_l2 = p.LSE[g] * 1.4426950408889634f;
      const float delta = p.DELTA[g];
      if (!at_wait(ctl, KB_SF, it & 1)) {
        ok = false;
        break;
      }
      if (it > 0 && !at_wait(ctl, KB_DONE, (it - 1) & 1)) {
        ok = false;
        break;
      }
      tc_fence_after();
      // keys of this block visible to query `row` of the diagonal block: key <= query
      const int limit = (p.causal && ib == jb) ? row : 1 << 30;
      at_p_ds_row<true>(lane_addr, sP, sdS, row, half, lse_l2, delta, p.scale, p.scale_log2, limit,
                        p.causal && ib == jb);
      fence_proxy_async_smem();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&ctl->bar[KB_PF]);
    }
    if (ok && !at_wait(ctl, KB_DONE, (n_it - 1) & 1)) ok = false;
    if (ok) {
      tc_fence_after();
      const size_t g = (static_cast<size_t>(row_base) + jb * AT_ROWS + row) * D;   // this key row
      // half 0 writes dV, half 1 writes dK
      {
        const int which = half;
        __nv_bfloat16* dst = (which == 0 ? p.dV : p.dK) + g;
#pragma unroll
        for (int c = 0; c < D / 32; ++c) {
          uint32_t v[32];
          tmem_ld_32x32(lane_addr + 256 + which * D + c * 32, v);
          tmem_ld_wait();
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            uint4 out;
            out.x = at_pack(__uint_as_float(v[q * 8 + 0]), __uint_as_float(v[q * 8 + 1]));
            out.y = at_pack(__uint_as_float(v[q * 8 + 2]), __uint_as_float(v[q * 8 + 3]));
            out.z = at_pack(__uint_as_float(v[q * 8 + 4]), __uint_as_float(v[q * 8 + 5]));
            out.w = at_pack(__uint_as_float(v[q * 8 + 6]), __uint_as_float(v[q * 8 + 7]));
            *reinterpret_cast<uint4*>(dst + c * 32 + q * 8) = out;
          }
        }
      }
    } else if (lane == 0) {
      at_abort(ctl, p.status, ST_TIMEOUT_ACC);
    }
  }
  at_teardown(ctl, warp, tmem);
}

// =============================================================================================
// backward: dQ  (one CTA per query block, loop over key blocks)
// =============================================================================================
enum { QB_QF = 0, QB_KF = 1, QB_KE = 2, QB_SF = 3, QB_PF = 4, QB_DONE = 5, QB_N = 6 };

template <int D>
__global__ void __launch_bounds__(AT_THREADS, 1)
attn_bwd_dq_kernel(const __grid_constant__ CUtensorMap tm_q,
                   const __grid_constant__ CUtensorMap tm_k,
                   const __grid_constant__ CUtensorMap tm_v,
                   const __grid_constant__ CUtensorMap tm_do, const AttnParams p) {
  constexpr int TILE = AT_ROWS * D * 2;
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* base = reinterpret_cast<uint8_t*>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  uint8_t* sQ = base;
  uint8_t* sdO = sQ + TILE;
  uint8_t* sK = sdO + TILE;
  uint8_t* sV = sK + TILE;
  uint8_t* sdS = sV + TILE;
  AttnCtl* ctl = reinterpret_cast<AttnCtl*>(sdS + 2 * AT_BOX);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nb = p.S / AT_ROWS;
  const int ib = nb - 1 - static_cast<int>(blockIdx.x) / p.BH;     // long loops first
  const int bh = static_cast<int>(blockIdx.x) % p.BH;
  const int n_it = p.causal ? ib + 1 : nb;
  const int row_base = bh * p.S;
  {
    const int counts[QB_N] = {1, 1, 1, 1, 8, 1};
    at_setup(ctl, QB_N, counts, warp, lane);
  }
  const uint32_t tmem = ctl->tmem_base;
  // TMEM columns: S [0,128)  dP [128,256)  dQ [256,256+D)

  if (warp == 0) {
    if (lane == 0) {
      prefetch_tmap(&tm_k);
      prefetch_tmap(&tm_v);
      mbar_expect_tx(&ctl->bar[QB_QF], 2 * TILE);
      at_load_tile<D>(sQ, &tm_q, &ctl->bar[QB_QF], row_base + ib * AT_ROWS);
      at_load_tile<D>(sdO, &tm_do, &ctl->bar[QB_QF], row_base + ib * AT_ROWS);
      for (int j = 0; j < n_it; ++j) {
        if (j > 0 && !mbar_wait(&ctl->bar[QB_KE], (j - 1) & 1, &ctl->abort_flag)) {
          at_abort(ctl, p.status, ST_TIMEOUT_EMPTY);
          break;
        }
        mbar_expect_tx(&ctl->bar[QB_KF], 2 * TILE);
        at_load_tile<D>(sK, &tm_k, &ctl->bar[QB_KF], row_base + j * AT_ROWS);
        at_load_tile<D>(sV, &tm_v, &ctl->bar[QB_KF], row_base + j * AT_ROWS);
      }
    }
  } else if (warp == 1) {
    constexpr uint32_t idesc_s = make_idesc_bf16(128, 128, false, false);
    constexpr uint32_t idesc_q = make_idesc_bf16(128, D, false, true);
    const uint32_t k_addr = smem_u32(sK), v_addr = smem_u32(sV), q_addr = smem_u32(sQ),
                   do_addr = smem_u32(sdO), ds_addr = smem_u32(sdS);
    bool ok = at_wait(ctl, QB_QF, 0);
    for (int j = 0; j < n_it && ok; ++j) {
      if (!at_wait(ctl, QB_KF, j & 1)) {
        ok = false;
        break;
      }
      tc_fence_after();
      if (lane == 0) {
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk)
          umma_bf16(tmem, at_desc_k(q_addr, kk), at_desc_k(k_addr, kk), idesc_s, kk != 0);
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk)
          umma_bf16(tmem + 128, at_desc_k(do_addr, kk), at_desc_k(v_addr, kk), idesc_s, kk != 0);
        umma_commit(&ctl->bar[QB_SF]);
      }
      __syncwarp();
      if (!at_wait(ctl, QB_PF, j & 1)) {
        ok = false;
        break;
      }
      tc_fence_after();
      if (lane == 0) {
#pragma unroll
        for (int kk = 0; kk < AT_ROWS / 16; ++kk)
          umma_bf16(tmem + 256, at_desc_k(ds_addr, kk), at_desc_mn(k_addr, kk), idesc_q,
                    (j | kk) != 0);
        umma_commit(&ctl->bar[QB_KE]);
        umma_commit(&ctl->bar[QB_DONE]);
      }
      __syncwarp();
    }
    if (!ok && lane == 0) at_abort(ctl, p.status, ST_TIMEOUT_ACC);
  } else {
    const int quad = warp & 3;
    const int half = (warp - 2) >> 2;
    const int row = quad * 32 + lane;
    const uint32_t lane_addr = tmem + (static_cast<uint32_t>(quad * 32) << 16);
    const size_t g = static_cast<size_t>(row_base) + ib * AT_ROWS + row;
    const float lse_l2 = p.LSE[g] * 1.4426950408889634f;
    const float delta = p.DELTA[g];
    bool ok = true;
    for (int j = 0; j < n_it && ok; ++j) {
      if (!at_wait(ctl, QB_SF, j & 1)) {
        ok = false;
        break;
      }
      if (j > 0 && !at_wait(ctl, QB_DONE, (j - 1) & 1)) {
        ok = false;
        break;
      }
      tc_fence_after();
      const int limit = (p.causal && j == ib) ? row : 1 << 30;
      at_p_ds_row<false>(lane_addr, nullptr, sdS, row, half, lse_l2, delta, p.scale, p.scale_log2, limit,
                         p.causal && j == ib);
      fence_proxy_async_smem();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&ctl->bar[QB_PF]);
    }
    if (ok && !at_wait(ctl, QB_DONE, (n_it - 1) & 1)) ok = false;
    if (ok) {
      tc_fence_after();
      __nv_bfloat16* dst = p.dQ + g * D;
#pragma unroll
      for (int c = half * (D / 64); c < (half + 1) * (D / 64); ++c) {
        uint32_t v[32];
        tmem_ld_32x32(lane_addr + 256 + c * 32, v);
        tmem_ld_wait();
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          uint4 out;
          out.x = at_pack(__uint_as_float(v[q * 8 + 0]), __uint_as_float(v[q * 8 + 1]));
          out.y = at_pack(__uint_as_float(v[q * 8 + 2]), __uint_as_float(v[q * 8 + 3]));
          out.z = at_pack(__uint_as_float(v[q * 8 + 4]), __uint_as_float(v[q * 8 + 5]));
          out.w = at_pack(__uint_as_float(v[q * 8 + 6]), __uint_as_float(v[q * 8 + 7]));
          *reinterpret_cast<uint4*>(dst + c * 32 + q * 8) = out;
        }
      }
    } else if (lane == 0) {
      at_abort(ctl, p.status, ST_TIMEOUT_ACC);
    }
  }
  at_teardown(ctl, warp, tmem);
}

// ---------------------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------------------
typedef CUresult (*AtEncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                               const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                               const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                               CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static int at_make_tmap(CUtensorMap* out, const void* ptr, long long rows, int D) {
  static AtEncodeFn fn = nullptr;
  if (fn == nullptr) {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q) !=
            cudaSuccess || q != cudaDriverEntryPointSuccess)
      return TB200_ERR_DRIVER;
    fn = reinterpret_cast<AtEncodeFn>(sym);
  }
  static thread_local bool context_bound = false;   // the encode needs a current context
  if (!context_bound) {
    cudaFree(nullptr);
    context_bound = true;
  }
  cuuint64_t gdim[2] = {static_cast<cuuint64_t>(D), static_cast<cuuint64_t>(rows)};
  cuuint64_t gstr[1] = {static_cast<cuuint64_t>(D) * 2};
  cuuint32_t box[2] = {64, AT_ROWS};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), gdim, gstr,
                  box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    fprintf(stderr, "terrace_b200: attention tensor-map encode failed (CUresult %d)\n",
            static_cast<int>(r));
    return TB200_ERR_TMAP;
  }
  return TB200_OK;
}

template <typename K>
static int at_configure(K kern, size_t smem) {
  return cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                              static_cast<int>(smem)) == cudaSuccess
             ? TB200_OK
             : TB200_ERR_LAUNCH;
}

template <int D>
static int at_fwd(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv,
                  const AttnParams& p, cudaStream_t stream) {
  constexpr size_t smem = 5 * AT_ROWS * D * 2 + 2 * AT_BOX + sizeof(AttnCtl) + 1024;
  static OncePerDevice done;
  if (done.need()) {
    if (at_configure(attn_fwd_kernel<D>, smem) != TB200_OK) return TB200_ERR_LAUNCH;
    done.done();
  }
  attn_fwd_kernel<D><<<p.BH * (p.S / AT_ROWS), AT_THREADS, smem, stream>>>(tq, tk, tv, p);
  return cudaGetLastError() == cudaSuccess ? TB200_OK : TB200_ERR_LAUNCH;
}

template <int D>
static int at_bwd(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv,
                  const CUtensorMap& tdo, const AttnParams& p, cudaStream_t stream) {
  constexpr size_t smem_kv = 4 * AT_ROWS * D * 2 + 4 * AT_BOX + sizeof(AttnCtl) + 1024;
  constexpr size_t smem_q = 4 * AT_ROWS * D * 2 + 2 * AT_BOX + sizeof(AttnCtl) + 1024;
  static OncePerDevice done;
  if (done.need()) {
    if (at_configure(attn_bwd_dkdv_kernel<D>, smem_kv) != TB200_OK) return TB200_ERR_LAUNCH;
    if (at_configure(attn_bwd_dq_kernel<D>, smem_q) != TB200_OK) return TB200_ERR_LAUNCH;
    done.done();
  }
  const int grid = p.BH * (p.S / AT_ROWS);
  attn_bwd_dkdv_kernel<D><<<grid, AT_THREADS, smem_kv, stream>>>(tq, tk, tv, tdo, p);
  if (cudaGetLastError() != cudaSuccess) return TB200_ERR_LAUNCH;
  attn_bwd_dq_kernel<D><<<grid, AT_THREADS, smem_q, stream>>>(tq, tk, tv, tdo, p);
  return cudaGetLastError() == cudaSuccess ? TB200_OK : TB200_ERR_LAUNCH;
}

static bool at_shape_ok(int BH, int S, int D) {
  return BH > 0 && S > 0 && S % AT_ROWS == 0 && (D == 64 || D == 128) &&
         static_cast<long long>(BH) * (S / AT_ROWS) < (1ll << 31);
}

}  // namespace tb200

using namespace tb200;

extern "C" int tb200_attn_fwd(const void* q, const void* k, const void* v, void* o, float* lse,
                              int BH, int S, int D, int causal, float scale, int* status,
                              cudaStream_t stream) {
  if (!at_shape_ok(BH, S, D)) return TB200_ERR_ARG;
  CUtensorMap tq, tk, tv;
  const long long rows = static_cast<long long>(BH) * S;
  int rc = at_make_tmap(&tq, q, rows, D);
  if (rc == TB200_OK) rc = at_make_tmap(&tk, k, rows, D);
  if (rc == TB200_OK) rc = at_make_tmap(&tv, v, rows, D);
  if (rc != TB200_OK) return rc;
  AttnParams p{};
  p.S = S;
  p.BH = BH;
  p.causal = causal;
  p.scale = scale;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.O = static_cast<__nv_bfloat16*>(o);
  p.LSE = lse;
  p.status = status;
  return D == 128 ? at_fwd<128>(tq, tk, tv, p, stream) : at_fwd<64>(tq, tk, tv, p, stream);
}

extern "C" int tb200_attn_bwd(const void* q, const void* k, const void* v, const void* o,
                              const void* d_o, const float* lse, float* delta, void* dq, void* dk,
                              void* dv, int BH, int S, int D, int causal, float scale, int* status,
                              cudaStream_t stream) {
  if (!at_shape_ok(BH, S, D)) return TB200_ERR_ARG;
  CUtensorMap tq, tk, tv, tdo;
  const long long rows = static_cast<long long>(BH) * S;
  int rc = at_make_tmap(&tq, q, rows, D);
  if (rc == TB200_OK) rc = at_make_tmap(&tk, k, rows, D);
  if (rc == TB200_OK) rc = at_make_tmap(&tv, v, rows, D);
  if (rc == TB200_OK) rc = at_make_tmap(&tdo, d_o, rows, D);
  if (rc != TB200_OK) return rc;
  attn_delta_kernel<<<static_cast<unsigned>((rows + 7) / 8), 256, 0, stream>>>(
      static_cast<const __nv_bfloat16*>(o), static_cast<const __nv_bfloat16*>(d_o), delta, rows, D);
  if (cudaGetLastError() != cudaSuccess) return TB200_ERR_LAUNCH;
  AttnParams p{};
  p.S = S;
  p.BH = BH;
  p.causal = causal;
  p.scale = scale;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.LSE = const_cast<float*>(lse);
  p.DELTA = delta;
  p.dQ = static_cast<__nv_bfloat16*>(dq);
  p.dK = static_cast<__nv_bfloat16*>(dk);
  p.dV = static_cast<__nv_bfloat16*>(dv);
  p.status = status;
  return D == 128 ? at_bwd<128>(tq, tk, tv, tdo, p, stream) : at_bwd<64>(tq, tk, tv, tdo, p, stream);
}
