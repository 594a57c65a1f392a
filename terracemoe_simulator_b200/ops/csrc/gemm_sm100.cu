// Grouped / dense bf16 GEMMs for sm_100a on the 5th-generation tensor cores.
//
//   tcgen05.mma (cta_group::1, kind::f16, 128 x 256 x 16 per instruction) issued by one elected
//   thread, operands staged in shared memory by TMA (cp.async.bulk.tensor, 128-byte swizzle),
//   fp32 accumulators in TMEM (two 256-column stages, so the epilogue of tile i overlaps the main
//   loop of tile i+1), epilogue through tcgen05.ld.  Persistent CTAs (one per SM) walk a tile
//   list that every CTA derives on the device from the per-expert row counts, so no host sync
//   is needed between routing and the expert GEMMs.
//
// Long groups (1024+ rows on average) run on CTA pairs (cta_group::2, 256 x 256 tiles, six 32 KiB
// stages per CTA): measured +3-5 % over single CTAs; short groups stay on 128-row tiles, where
// the second CTA of a pair would often have no rows.  The loop is bound by bytes in flight:
// with loads or MMAs removed the same kernel runs at 1680-1730 TFLOPS-equivalent, together at
// 1260-1320, i.e. 192 KiB of staging per SM over a 1.4-1.8 us loaded L2 latency.  An L2
// prefetch of later K slices made it 10-20 % slower (more L2 requests), so there is none.
//
// Three operand-layout variants cover every GEMM of the MoE layer and of the dense layers:
//   * fwd   : C[rows, N]  = A[rows, K] * W[e][K, N]      (A K-major, B N-major)   x @ w13, h @ w2
//   * dgrad : C[rows, N]  = A[rows, K] * W[e][N, K]^T    (A K-major, B K-major)   dy @ w^T, nn.Linear
//   * wgrad : W'[e][M, N] = A[rows, M]^T * B[rows, N]    (A M-major, B N-major)   x^T @ dy
// The fwd variant has an optional fused SwiGLU epilogue: the B tile holds 128 gate columns and
// the matching 128 up columns, and the epilogue writes silu(gate) * up (and, for training, the
// two pre-activations).
//
// Computes what the reference does with a Python loop of per-expert matmuls
// (terrace/layer.py:30-68 `_grouped_mm_fwd` / `_GroupedMM`).
#include "host_util.h"
#include "launch.h"
#include "ptx_sm100.cuh"
#include "tmap.h"

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include <mutex>

namespace tb200 {

constexpr int BM = 128;               // accumulator rows per CTA
constexpr int BN = 256;               // accumulator columns per tile
constexpr int BK = 64;                // 64 bf16 = 128 bytes = one swizzle line
constexpr int A_BYTES = BM * BK * 2;  // 16 KiB
constexpr int BOX_BYTES = 64 * BK * 2; // one 64 x 64 box = 8 KiB
constexpr int GEMM_THREADS = 192;     // warp 0 TMA, warp 1 MMA, warps 2..5 epilogue
constexpr int MAX_GROUPS = 1024;
constexpr int TMEM_COLS = 512;
constexpr int MAX_STAGES = 6;
constexpr int OUT_STAGE_BYTES = 4 * 32 * 128;   // per epilogue warp: 32 rows x 64 bf16

// CTAS = 1: one CTA per 128 x 256 tile (cta_group::1), 4 stages of 48 KiB.
// CTAS = 2: a cluster of two CTAs per 256 x 256 tile (cta_group::2): each CTA stages its 128
//           rows of A and its 128 columns of B (32 KiB per stage, 6 stages) and holds the
//           accumulator rows of its half; per CTA the tensor core reads a third less shared
//           memory per flop and L2 -> SM traffic for B halves.
template <int CTAS>
struct Cfg {
  static constexpr int BN_LOCAL = BN / CTAS;
  static constexpr int B_BYTES = BN_LOCAL * BK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int STAGES = CTAS == 1 ? 4 : 6;
  static constexpr int BM_TILE = BM * CTAS;
  static constexpr int B_BOXES = BN_LOCAL / 64;
};

struct GemmParams {
  const int* seg_start;   // [E] first row of every group in A / C
  const int* seg_count;   // [E] rows of every group
  int n_groups;
  int N;                  // output columns per group (for SwiGLU: the activation width d)
  int K;                  // reduction length (wgrad: unused, rows come from seg_count)
  int M;                  // wgrad only: rows of the weight gradient (input features)
  int ldc;                // row stride of C in elements
  int ldc2;               // row stride of C2 in elements
  int up_offset;          // SwiGLU: column of the first up-projection weight (= d)
  __nv_bfloat16* C;
  __nv_bfloat16* C2;      // SwiGLU: optional [rows, 2d] pre-activations (may be null)
  int* status;
  const int* wait_flags;  // optional: arrival flags that must reach wait_epoch before A is read
  int wait_n;
  int wait_epoch;
  int pad_align;          // > 0: every group's rows are padded to this multiple; fwd / dgrad write
                          // zeros into the padding rows, wgrad (multiple of BK) relies on them
  // EPI_SCATTER only: output row r goes to scatter_base[m / scatter_slots] + (m % scatter_slots)
  // rows of ldc elements, m = row_map[r]; the bases may be peer GPUs' buffers (plain peer stores)
  const int* row_map;
  const unsigned long long* scatter_base;
  int scatter_slots;
  int scatter_world;
};

struct __align__(8) PipeBarriers {
  uint64_t full[MAX_STAGES];
  uint64_t empty[MAX_STAGES];
  uint64_t acc_full[2];
  uint64_t acc_empty[2];
};

struct SharedCtl {
  PipeBarriers bars;
  uint32_t tmem_base;
  volatile int abort_flag;
  int total_tiles;
  int tile_start[MAX_GROUPS + 1];
};

__device__ __forceinline__ void raise_abort(SharedCtl* ctl, int* status, int code) {
  ctl->abort_flag = code;
  if (status != nullptr) atomicCAS(status, 0, code);
}

// Whole-warp bounded wait with a warp-uniform verdict (lanes must not disagree, the callers
// use warp-synchronous instructions afterwards).
template <int CTAS>
__device__ __forceinline__ bool warp_wait(uint64_t* bar, uint32_t parity,
                                          volatile int* abort_flag) {
  // plain (CTA-scope) polling also for barriers that the other CTA of a pair signals: the data
  // they guard moves through the async proxy (TMA -> UMMA -> TMEM), and a cluster-scope acquire
  // on every poll costs more than the four MMAs it gates
  const bool got = mbar_wait(bar, parity, abort_flag);
  return __all_sync(0xffffffffu, got);
}

__device__ __forceinline__ uint32_t pack_bf16(float a, float b) {
  __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&v);
}

__device__ __forceinline__ float silu_f(float x) { return x / (1.0f + __expf(-x)); }

// One warp's 32 rows x 64 columns (lane = row, fp32 in r0 | r1) -> bf16 -> this warp's staging
// area in shared memory (16-byte chunks XOR-swizzled by row, conflict-free both ways) -> global
// memory with four complete 128-byte rows per store instruction.  Rows [0, rows_live) are
// written; rows [rows_real, rows_live) and, with all_zero, every row are written as zeros.
__device__ __forceinline__ void stage_and_store64(uint8_t* stg, int lane, const uint32_t (&r0)[32],
                                                  const uint32_t (&r1)[32], __nv_bfloat16* cbase,
                                                  size_t ld, int n0, int n_limit, int rows_live,
                                                  int rows_real, bool all_zero) {
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    uint4 v;
    if (j < 4) {
      v.x = pack_bf16(__uint_as_float(r0[j * 8 + 0]), __uint_as_float(r0[j * 8 + 1]));
      v.y = pack_bf16(__uint_as_float(r0[j * 8 + 2]), __uint_as_float(r0[j * 8 + 3]));
      v.z = pack_bf16(__uint_as_float(r0[j * 8 + 4]), __uint_as_float(r0[j * 8 + 5]));
      v.w = pack_bf16(__uint_as_float(r0[j * 8 + 6]), __uint_as_float(r0[j * 8 + 7]));
    } else {
      v.x = pack_bf16(__uint_as_float(r1[j * 8 - 32]), __uint_as_float(r1[j * 8 - 31]));
      v.y = pack_bf16(__uint_as_float(r1[j * 8 - 30]), __uint_as_float(r1[j * 8 - 29]));
      v.z = pack_bf16(__uint_as_float(r1[j * 8 - 28]), __uint_as_float(r1[j * 8 - 27]));
      v.w = pack_bf16(__uint_as_float(r1[j * 8 - 26]), __uint_as_float(r1[j * 8 - 25]));
    }
    *reinterpret_cast<uint4*>(stg + lane * 128 + ((j ^ (lane & 7)) << 4)) = v;
  }
  __syncwarp();
  const int ch = lane & 7;
  const bool col_ok = n0 + ch * 8 < n_limit;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int rr = i * 4 + (lane >> 3);
    uint4 v = *reinterpret_cast<const uint4*>(stg + rr * 128 + ((ch ^ (rr & 7)) << 4));
    if (all_zero || rr >= rows_real) v = make_uint4(0, 0, 0, 0);
    if (col_ok && rr < rows_live)
      *reinterpret_cast<uint4*>(cbase + static_cast<size_t>(rr) * ld + ch * 8) = v;
  }
  __syncwarp();
}

// Same staging as stage_and_store64, but every row goes to its own destination: lane r holds the
// address of row r (0 = skip the row); the store loop fetches it with two shuffles.  The
// destinations may live in peer GPUs' memory.
__device__ __forceinline__ void stage_and_scatter64(uint8_t* stg, int lane, const uint32_t (&r0)[32],
                                                    const uint32_t (&r1)[32],
                                                    unsigned long long row_addr, int n0,
                                                    int n_limit) {
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    uint4 v;
    if (j < 4) {
      v.x = pack_bf16(__uint_as_float(r0[j * 8 + 0]), __uint_as_float(r0[j * 8 + 1]));
      v.y = pack_bf16(__uint_as_float(r0[j * 8 + 2]), __uint_as_float(r0[j * 8 + 3]));
      v.z = pack_bf16(__uint_as_float(r0[j * 8 + 4]), __uint_as_float(r0[j * 8 + 5]));
      v.w = pack_bf16(__uint_as_float(r0[j * 8 + 6]), __uint_as_float(r0[j * 8 + 7]));
    } else {
      v.x = pack_bf16(__uint_as_float(r1[j * 8 - 32]), __uint_as_float(r1[j * 8 - 31]));
      v.y = pack_bf16(__uint_as_float(r1[j * 8 - 30]), __uint_as_float(r1[j * 8 - 29]));
      v.z = pack_bf16(__uint_as_float(r1[j * 8 - 28]), __uint_as_float(r1[j * 8 - 27]));
      v.w = pack_bf16(__uint_as_float(r1[j * 8 - 26]), __uint_as_float(r1[j * 8 - 25]));
    }
    *reinterpret_cast<uint4*>(stg + lane * 128 + ((j ^ (lane & 7)) << 4)) = v;
  }
  __syncwarp();
  const int ch = lane & 7;
  const bool col_ok = n0 + ch * 8 < n_limit;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int rr = i * 4 + (lane >> 3);
    const uint4 v = *reinterpret_cast<const uint4*>(stg + rr * 128 + ((ch ^ (rr & 7)) << 4));
    const unsigned long long dst = __shfl_sync(0xffffffffu, row_addr, rr);
    if (col_ok && dst != 0ull)
      *reinterpret_cast<uint4*>(dst + static_cast<unsigned long long>(n0 + ch * 8) * 2ull) = v;
  }
  __syncwarp();
}

// Locate the group of global tile index t (tile_start is a prefix array); `e` is a cursor that
// only moves forward because every role visits tiles in increasing order.
__device__ __forceinline__ void locate_tile(const SharedCtl* ctl, int n_groups, int t, int& e) {
  while (e + 1 < n_groups && t >= ctl->tile_start[e + 1]) ++e;
}

__device__ __forceinline__ int clamp32(int v) { return v < 0 ? 0 : (v > 32 ? 32 : v); }

enum { MODE_FWD = 0, MODE_DGRAD = 1, MODE_WGRAD = 2 };
// EPI_SCATTER: plain epilogue whose rows go to per-row destinations (the combine leg of expert
// parallelism folded into the GEMM: the tile is stored straight into the token owner's buffer)
// EPI_SWIGLU_BWD: the tile is d(act); the epilogue reads the saved pre-activations
// [gate | up] of its rows (C2) and writes d[gate | up] (C, 2N wide) -- the SwiGLU backward
// without the d(act) round trip through memory
enum { EPI_PLAIN = 0, EPI_SWIGLU = 1, EPI_SCATTER = 2, EPI_SWIGLU_BWD = 3 };

template <int MODE, int EPI, int CTAS>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
            const GemmParams p) {
  using C = Cfg<CTAS>;
  constexpr int STAGES = C::STAGES;
  constexpr int STAGE_BYTES = C::STAGE_BYTES;
  constexpr int BM_TILE = C::BM_TILE;
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  // stage buffers need 1024-byte alignment for the 128-byte swizzle
  uint8_t* stage_base = reinterpret_cast<uint8_t*>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  uint8_t* out_stage = stage_base + STAGES * STAGE_BYTES;
  SharedCtl* ctl = reinterpret_cast<SharedCtl*>(out_stage + OUT_STAGE_BYTES);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int crank = CTAS == 1 ? 0 : static_cast<int>(cluster_ctarank());
  const bool leader = crank == 0;
  const int unit = blockIdx.x / CTAS;            // index of this CTA (pair) among the workers
  const int n_units = gridDim.x / CTAS;
  const int n_tiles_n = (MODE == MODE_WGRAD) ? (p.N + BN - 1) / BN
                        : (EPI == EPI_SWIGLU) ? (p.N + 127) / 128
                                              : (p.N + BN - 1) / BN;
  const int n_tiles_m_w = (p.M + BM_TILE - 1) / BM_TILE;   // wgrad only

  // ---- one-time setup ---------------------------------------------------------------------
  if (warp == 0) {
    // tile table: exclusive prefix of tiles per group, 32 groups per warp step
    int carry = 0;
    for (int base = 0; base < p.n_groups; base += 32) {
      const int e = base + lane;
      int tiles = 0;
      if (e < p.n_groups) {
        tiles = (MODE == MODE_WGRAD)
                    ? n_tiles_m_w * n_tiles_n
                    : ((p.seg_count[e] + BM_TILE - 1) / BM_TILE) * n_tiles_n;
      }
      int incl = tiles;
#pragma unroll
      for (int d = 1; d < 32; d <<= 1) {
        const int v = __shfl_up_sync(0xffffffffu, incl, d);
        if (lane >= d) incl += v;
      }
      if (e < p.n_groups) ctl->tile_start[e] = carry + incl - tiles;
      carry += __shfl_sync(0xffffffffu, incl, 31);
    }
    if (lane == 0) {
      ctl->tile_start[p.n_groups] = carry;
      ctl->total_tiles = carry;
      ctl->abort_flag = 0;
      for (int s = 0; s < STAGES; ++s) {
        mbar_init(&ctl->bars.full[s], 1);
        mbar_init(&ctl->bars.empty[s], 1);
      }
      for (int a = 0; a < 2; ++a) {
        mbar_init(&ctl->bars.acc_full[a], 1);
        mbar_init(&ctl->bars.acc_empty[a], 4 * CTAS);
      }
      fence_barrier_init();
    }
  }
  if (warp == 1) {
    if (CTAS == 1) {
      tmem_alloc(&ctl->tmem_base, TMEM_COLS);
      tmem_relinquish();
    } else {
      tmem_alloc_pair(&ctl->tmem_base, TMEM_COLS);
      tmem_relinquish_pair();
    }
  }
  if (warp == 0 && lane == 0) {
    prefetch_tmap(&tmap_a);
    prefetch_tmap(&tmap_b);
  }
  tc_fence_before();
  if (CTAS == 1) {
    __syncthreads();
  } else {
    __syncthreads();
    cluster_sync_all();       // the other CTA's barriers are initialised before anyone signals them
  }
  tc_fence_after();
  const uint32_t tmem_base = ctl->tmem_base;
  const int total_tiles = ctl->total_tiles;

  if (warp == 0) {
    // =========================== TMA producer =============================================
    if (lane == 0) {
      int e = 0;
      uint32_t it = 0;
      bool ok = true;
      const uint32_t full0_leader = CTAS == 1 ? smem_u32(&ctl->bars.full[0])
                                              : mapa_u32(smem_u32(&ctl->bars.full[0]), 0);
      if (p.wait_flags != nullptr) {
        // rows of A are stored by peer GPUs: wait for their arrival flags, then order the
        // generic-proxy writes before this thread's TMA (async-proxy) reads
        for (int i = 0; i < p.wait_n && ok; ++i) {
          if (!wait_flag_ge(p.wait_flags + i, p.wait_epoch)) {
            raise_abort(ctl, p.status, ST_TIMEOUT_FLAG);
            ok = false;
          }
        }
        fence_proxy_async_all();
      }
      for (int t = unit; t < total_tiles && ok; t += n_units) {
        locate_tile(ctl, p.n_groups, t, e);
        const int local = t - ctl->tile_start[e];
        const int mt = local / n_tiles_n;
        const int nt = local - mt * n_tiles_n;
        const int seg0 = p.seg_start[e];
        const int cnt = p.seg_count[e];
        const int kblocks = (MODE == MODE_WGRAD) ? (cnt + BK - 1) / BK : (p.K + BK - 1) / BK;
        const int m_off = mt * BM_TILE + crank * BM;          // this CTA's accumulator rows
        const int n_off = crank * C::BN_LOCAL;                // this CTA's columns of the B tile
        for (int kb = 0; kb < kblocks; ++kb, ++it) {
          const int s = it % STAGES;
          const uint32_t round = it / STAGES;
          if (round > 0) {
            if (!mbar_wait(&ctl->bars.empty[s], (round - 1) & 1, &ctl->abort_flag)) {
              raise_abort(ctl, p.status, ST_TIMEOUT_EMPTY);
              ok = false;
              break;
            }
          }
          uint8_t* sa = stage_base + s * STAGE_BYTES;
          uint8_t* sb = sa + A_BYTES;
          uint64_t* bar = &ctl->bars.full[s];
          // pair: both CTAs' bytes are counted on the leader's barrier, armed by the leader
          const uint32_t bar_addr = full0_leader + s * 8;
          if (leader) mbar_expect_tx(bar, STAGE_BYTES * CTAS);
          auto load2 = [&](void* dst, const CUtensorMap* tm, int x, int y) {
            if (CTAS == 1) tma_load_2d(dst, tm, bar, x, y);
            else tma_load_2d_pair(dst, tm, bar_addr, x, y);
          };
          auto load3 = [&](void* dst, const CUtensorMap* tm, int x, int y, int z) {
            if (CTAS == 1) tma_load_3d(dst, tm, bar, x, y, z);
            else tma_load_3d_pair(dst, tm, bar_addr, x, y, z);
          };
          if (MODE == MODE_WGRAD) {
            const int row0 = seg0 + kb * BK;
            for (int j = 0; j < 2; ++j)
              load2(sa + j * BOX_BYTES, &tmap_a, m_off + j * 64, row0);
            for (int j = 0; j < C::B_BOXES; ++j)
              load2(sb + j * BOX_BYTES, &tmap_b, nt * BN + n_off + j * 64, row0);
          } else {
            load2(sa, &tmap_a, kb * BK, seg0 + m_off);
            if (MODE == MODE_DGRAD && EPI == EPI_SWIGLU) {
              // weight rows [gate | up]: 128 gate rows, then the matching 128 up rows
              if (CTAS == 1) {
                load3(sb, &tmap_b, kb * BK, nt * 128, e);
                load3(sb + C::B_BYTES / 2, &tmap_b, kb * BK, p.up_offset + nt * 128, e);
              } else {
                load3(sb, &tmap_b, kb * BK, (crank ? p.up_offset : 0) + nt * 128, e);
              }
            } else if (MODE == MODE_DGRAD) {
              load3(sb, &tmap_b, kb * BK, nt * BN + n_off, e);
            } else if (EPI == EPI_SWIGLU) {
              if (CTAS == 1) {
                for (int j = 0; j < 2; ++j)
                  load3(sb + j * BOX_BYTES, &tmap_b, nt * 128 + j * 64, kb * BK, e);
                for (int j = 0; j < 2; ++j)
                  load3(sb + (2 + j) * BOX_BYTES, &tmap_b, p.up_offset + nt * 128 + j * 64,
                        kb * BK, e);
              } else {
                for (int j = 0; j < 2; ++j)
                  load3(sb + j * BOX_BYTES, &tmap_b,
                        (crank ? p.up_offset : 0) + nt * 128 + j * 64, kb * BK, e);
              }
            } else {
              for (int j = 0; j < C::B_BOXES; ++j)
                load3(sb + j * BOX_BYTES, &tmap_b, nt * BN + n_off + j * 64, kb * BK, e);
            }
          }
        }
      }
    }
  } else if (warp == 1) {
    // =========================== MMA issuer (pair: the leader CTA only) ====================
    constexpr uint32_t idesc =
        make_idesc_bf16(BM_TILE, BN, MODE == MODE_WGRAD, MODE != MODE_DGRAD);
    // advance per 16 K elements inside a stage: 32 bytes along a K-major line, two 8-line atoms
    // (2048 bytes) in an MN-major box; operand A of a stage sits A_BYTES before operand B
    constexpr int A_KSTEP = MODE == MODE_WGRAD ? 2048 : 32;
    constexpr int B_KSTEP = MODE == MODE_DGRAD ? 32 : 2048;
    const uint64_t a_desc0 = MODE == MODE_WGRAD
                                 ? make_smem_desc(smem_u32(stage_base), BOX_BYTES, 1024)
                                 : make_smem_desc(smem_u32(stage_base), 16, 1024);
    const uint64_t b_desc0 = MODE == MODE_DGRAD
                                 ? make_smem_desc(smem_u32(stage_base) + A_BYTES, 16, 1024)
                                 : make_smem_desc(smem_u32(stage_base) + A_BYTES, BOX_BYTES, 1024);
    const uint32_t empty0_cta0 = CTAS == 1 ? 0u : mapa_u32(smem_u32(&ctl->bars.empty[0]), 0);
    const uint32_t empty0_cta1 = CTAS == 1 ? 0u : mapa_u32(smem_u32(&ctl->bars.empty[0]), 1);
    int e = 0;
    uint32_t it = 0;
    uint32_t tile_iter = 0;
    bool ok = leader;
    for (int t = unit; t < total_tiles && ok; t += n_units, ++tile_iter) {
      locate_tile(ctl, p.n_groups, t, e);
      const int cnt = p.seg_count[e];
      const int kblocks = (MODE == MODE_WGRAD) ? (cnt + BK - 1) / BK : (p.K + BK - 1) / BK;
      const int a = tile_iter & 1;
      const uint32_t around = tile_iter >> 1;
      if (around > 0 &&
          !warp_wait<CTAS>(&ctl->bars.acc_empty[a], (around - 1) & 1, &ctl->abort_flag)) {
        if (lane == 0) raise_abort(ctl, p.status, ST_TIMEOUT_ACC);
        ok = false;
        break;
      }
      tc_fence_after();
      const uint32_t d_tmem = tmem_base + a * BN;
      for (int kb = 0; kb < kblocks; ++kb, ++it) {
        const int s = it % STAGES;
        const uint32_t round = it / STAGES;
        if (!warp_wait<CTAS>(&ctl->bars.full[s], round & 1, &ctl->abort_flag)) {
          if (lane == 0) raise_abort(ctl, p.status, ST_TIMEOUT_FULL);
          ok = false;
          break;
        }
        uint8_t* sa = stage_base + s * STAGE_BYTES;
        uint8_t* sb = sa + A_BYTES;
        if (MODE == MODE_WGRAD && CTAS == 1) {
          // rows past the end of the group belong to the next group: zero their lines
          // (the pair variant is only launched with groups padded to a multiple of BK)
          const int valid = cnt - kb * BK;
          if (valid < BK && (p.pad_align <= 0 || p.pad_align % BK != 0)) {
            const int lines = BK - valid;
            for (int i = lane; i < lines * 8 * 6; i += 32) {
              const int box = i / (lines * 8);
              const int r = i - box * lines * 8;
              const int line = valid + (r >> 3);
              uint8_t* base = (box < 2 ? sa + box * BOX_BYTES : sb + (box - 2) * BOX_BYTES);
              *reinterpret_cast<uint4*>(base + line * 128 + (r & 7) * 16) = make_uint4(0, 0, 0, 0);
            }
            fence_proxy_async_smem();
          }
          __syncwarp();
        }
        tc_fence_after();
        if (lane == 0) {
          // descriptors differ from the stage-0 ones only in the 16-byte address field
          const uint64_t stage_off = static_cast<uint64_t>((s * STAGE_BYTES) >> 4);
#pragma unroll
          for (int k4 = 0; k4 < BK / 16; ++k4) {
            const uint64_t da = a_desc0 + stage_off + ((k4 * A_KSTEP) >> 4);
            const uint64_t db = b_desc0 + stage_off + ((k4 * B_KSTEP) >> 4);
            if (CTAS == 1) umma_bf16(d_tmem, da, db, idesc, (kb | k4) != 0 ? 1u : 0u);
            else umma_bf16_pair(d_tmem, da, db, idesc, (kb | k4) != 0 ? 1u : 0u);
          }
          // frees the stage (in both CTAs of a pair) when these MMAs retire
          if (CTAS == 1) {
            umma_commit(&ctl->bars.empty[s]);
          } else {
            umma_commit_pair(empty0_cta0 + s * 8);
            umma_commit_pair(empty0_cta1 + s * 8);
          }
        }
        __syncwarp();
      }
      if (ok && lane == 0) {
        if (CTAS == 1) {
          umma_commit(&ctl->bars.acc_full[a]);
        } else {
          const uint32_t fb = smem_u32(&ctl->bars.acc_full[a]);
          umma_commit_pair(mapa_u32(fb, 0));
          umma_commit_pair(mapa_u32(fb, 1));
        }
      }
      __syncwarp();
    }
  } else {
    // =========================== epilogue (4 warps) =======================================
    const int quad = warp & 3;                 // TMEM lane quadrant this warp may read
    const int row_in_tile = quad * 32 + lane;
    uint8_t* stg = out_stage + quad * (32 * 128);
    int e = 0;
    uint32_t tile_iter = 0;
    bool ok = true;
    for (int t = unit; t < total_tiles && ok; t += n_units, ++tile_iter) {
      locate_tile(ctl, p.n_groups, t, e);
      const int local = t - ctl->tile_start[e];
      const int mt = local / n_tiles_n;
      const int nt = local - mt * n_tiles_n;
      const int cnt = p.seg_count[e];
      const int seg0 = p.seg_start[e];
      const int m_off = mt * BM_TILE + crank * BM;
      const int a = tile_iter & 1;
      const uint32_t around = tile_iter >> 1;
      if (!warp_wait<CTAS>(&ctl->bars.acc_full[a], around & 1, &ctl->abort_flag)) {
        if (lane == 0) raise_abort(ctl, p.status, ST_TIMEOUT_ACC);
        ok = false;
        break;
      }
      tc_fence_after();
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quad * 32) << 16) + a * BN;
      if (MODE == MODE_WGRAD) {
        const int m0 = m_off + quad * 32;      // first weight-gradient row of this warp
        const int rows_live = clamp32(p.M - m0);
        const bool empty_group = cnt == 0;     // no MMA ran: the accumulator is undefined
        __nv_bfloat16* cbase = p.C + (static_cast<size_t>(e) * p.M + m0) * p.ldc;
#pragma unroll 1
        for (int c = 0; c < BN / 32; c += 2) {
          // two TMEM loads in flight before the wait: their latencies overlap
          uint32_t r0[32], r1[32];
          tmem_ld_32x32(taddr + c * 32, r0);
          tmem_ld_32x32(taddr + (c + 1) * 32, r1);
          tmem_ld_wait();
          const int n0 = nt * BN + c * 32;
          stage_and_store64(stg, lane, r0, r1, cbase + n0, p.ldc, n0, p.N, rows_live, rows_live,
                            empty_group);
        }
      } else if (EPI == EPI_SWIGLU) {
        const int row = m_off + row_in_tile;
        const int padded = p.pad_align > 0 ? (cnt + p.pad_align - 1) / p.pad_align * p.pad_align
                                           : cnt;
        const bool real = row < cnt;
        const bool live = row < padded;            // padding rows are written as zeros
        __nv_bfloat16* crow = p.C + static_cast<size_t>(seg0 + row) * p.ldc;
        __nv_bfloat16* c2row =
            p.C2 ? p.C2 + static_cast<size_t>(seg0 + row) * p.ldc2 : nullptr;
#pragma unroll 1
        for (int c = 0; c < 4; ++c) {
          uint32_t g[32], u[32];
          tmem_ld_32x32(taddr + c * 32, g);
          tmem_ld_32x32(taddr + 128 + c * 32, u);
          tmem_ld_wait();
          const int n0 = nt * 128 + c * 32;
          if (live) {
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              if (n0 + j * 8 < p.N) {
                uint4 v, vg, vu;
                uint32_t* pv = reinterpret_cast<uint32_t*>(&v);
                uint32_t* pg = reinterpret_cast<uint32_t*>(&vg);
                uint32_t* pu = reinterpret_cast<uint32_t*>(&vu);
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                  const float g0 = __uint_as_float(g[j * 8 + 2 * i]);
                  const float g1 = __uint_as_float(g[j * 8 + 2 * i + 1]);
                  const float u0 = __uint_as_float(u[j * 8 + 2 * i]);
                  const float u1 = __uint_as_float(u[j * 8 + 2 * i + 1]);
                  pg[i] = pack_bf16(g0, g1);
                  pu[i] = pack_bf16(u0, u1);
                  // activation from the bf16-rounded pre-activations, so that a backward pass
                  // that re-reads them sees exactly the forward's inputs
                  __nv_bfloat162 gb = *reinterpret_cast<__nv_bfloat162*>(&pg[i]);
                  __nv_bfloat162 ub = *reinterpret_cast<__nv_bfloat162*>(&pu[i]);
                  const float2 gf = __bfloat1622float2(gb);
                  const float2 uf = __bfloat1622float2(ub);
                  pv[i] = pack_bf16(silu_f(gf.x) * uf.x, silu_f(gf.y) * uf.y);
                }
                if (!real) v = vg = vu = make_uint4(0, 0, 0, 0);
                *reinterpret_cast<uint4*>(crow + n0 + j * 8) = v;
                if (c2row) {
                  *reinterpret_cast<uint4*>(c2row + n0 + j * 8) = vg;
                  *reinterpret_cast<uint4*>(c2row + p.up_offset + n0 + j * 8) = vu;
                }
              }
            }
          }
        }
      } else if (EPI == EPI_SWIGLU_BWD) {
        const int row = m_off + row_in_tile;
        const int padded = p.pad_align > 0 ? (cnt + p.pad_align - 1) / p.pad_align * p.pad_align
                                           : cnt;
        const bool real = row < cnt;
        const bool live = row < padded;            // padding rows are written as zeros
        const __nv_bfloat16* hrow = p.C2 + static_cast<size_t>(seg0 + row) * p.ldc2;
        __nv_bfloat16* orow = p.C + static_cast<size_t>(seg0 + row) * p.ldc;
#pragma unroll 1
        for (int c = 0; c < BN / 32; ++c) {
          uint32_t da[32];
          tmem_ld_32x32(taddr + c * 32, da);
          tmem_ld_wait();
          const int n0 = nt * BN + c * 32;
          if (live) {
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              if (n0 + j * 8 < p.N) {
                uint4 vg = make_uint4(0, 0, 0, 0), vu = make_uint4(0, 0, 0, 0);
                if (real) {
                  const uint4 g8 = *reinterpret_cast<const uint4*>(hrow + n0 + j * 8);
                  const uint4 u8 = *reinterpret_cast<const uint4*>(hrow + p.up_offset + n0 + j * 8);
                  const __nv_bfloat162* gb = reinterpret_cast<const __nv_bfloat162*>(&g8);
                  const __nv_bfloat162* ub = reinterpret_cast<const __nv_bfloat162*>(&u8);
                  uint32_t* pg = reinterpret_cast<uint32_t*>(&vg);
                  uint32_t* pu = reinterpret_cast<uint32_t*>(&vu);
#pragma unroll
                  for (int i = 0; i < 4; ++i) {
                    // d(act) rounded to bf16 first: the value a separate kernel would read back
                    uint32_t dpk = pack_bf16(__uint_as_float(da[j * 8 + 2 * i]),
                                             __uint_as_float(da[j * 8 + 2 * i + 1]));
                    const float2 d2 = __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&dpk));
                    const float2 g2 = __bfloat1622float2(gb[i]);
                    const float2 u2 = __bfloat1622float2(ub[i]);
                    const float s0 = 1.f / (1.f + __expf(-g2.x)), s1 = 1.f / (1.f + __expf(-g2.y));
                    pg[i] = pack_bf16(d2.x * u2.x * s0 * (1.f + g2.x * (1.f - s0)),
                                      d2.y * u2.y * s1 * (1.f + g2.y * (1.f - s1)));
                    pu[i] = pack_bf16(d2.x * g2.x * s0, d2.y * g2.y * s1);
                  }
                }
                *reinterpret_cast<uint4*>(orow + n0 + j * 8) = vg;
                *reinterpret_cast<uint4*>(orow + p.up_offset + n0 + j * 8) = vu;
              }
            }
          }
        }
      } else if (EPI == EPI_SCATTER) {
        const int row = m_off + row_in_tile;       // this lane's row inside the group
        unsigned long long row_addr = 0ull;
        if (row < cnt) {
          const int m = __ldcg(p.row_map + seg0 + row);
          const int src = m >= 0 ? m / p.scatter_slots : -1;
          if (src >= 0 && src < p.scatter_world) {
            const int slot = m - src * p.scatter_slots;
            row_addr = __ldg(p.scatter_base + src) +
                       static_cast<unsigned long long>(slot) *
                           static_cast<unsigned long long>(p.ldc) * 2ull;
          } else if (p.status != nullptr) {
            atomicCAS(p.status, 0, ST_BAD_INDEX);  // recorded, the row is skipped
          }
        }
#pragma unroll 1
        for (int c = 0; c < BN / 32; c += 2) {
          uint32_t r0[32], r1[32];
          tmem_ld_32x32(taddr + c * 32, r0);
          tmem_ld_32x32(taddr + (c + 1) * 32, r1);
          tmem_ld_wait();
          stage_and_scatter64(stg, lane, r0, r1, row_addr, nt * BN + c * 32, p.N);
        }
      } else {
        const int padded = p.pad_align > 0 ? (cnt + p.pad_align - 1) / p.pad_align * p.pad_align
                                           : cnt;
        const int r0w = m_off + quad * 32;         // first row (inside the group) of this warp
        const int rows_live = clamp32(padded - r0w);   // padding rows are written as zeros
        const int rows_real = clamp32(cnt - r0w);
        __nv_bfloat16* cbase = p.C + static_cast<size_t>(seg0 + r0w) * p.ldc;
#pragma unroll 1
        for (int c = 0; c < BN / 32; c += 2) {
          uint32_t r0[32], r1[32];
          tmem_ld_32x32(taddr + c * 32, r0);
          tmem_ld_32x32(taddr + (c + 1) * 32, r1);
          tmem_ld_wait();
          const int n0 = nt * BN + c * 32;
          stage_and_store64(stg, lane, r0, r1, cbase + n0, p.ldc, n0, p.N, rows_live, rows_real,
                            false);
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) {
        if (CTAS == 1 || leader) mbar_arrive(&ctl->bars.acc_empty[a]);
        else mbar_arrive_cluster(mapa_u32(smem_u32(&ctl->bars.acc_empty[a]), 0));
      }
    }
    // rows stored into other GPUs' memory: publish them before the kernel (and the flag that a
    // later launch raises) can complete
    if (EPI == EPI_SCATTER) __threadfence_system();
  }

  // ---- teardown: everybody meets, then the allocating warp frees TMEM ------------------------
  if (ctl->abort_flag != 0) {
    // give copies that may still be in flight time to land before shared memory is released
    const unsigned long long t0 = globaltimer_ns();
    while (globaltimer_ns() - t0 < 1000000ull) __nanosleep(256);
  }
  tc_fence_before();
  __syncthreads();
  if (CTAS == 2) cluster_sync_all();   // neither CTA leaves while the other may still signal it
  if (warp == 1) {
    tc_fence_after();
    if (CTAS == 1) tmem_dealloc(tmem_base, TMEM_COLS);
    else tmem_dealloc_pair(tmem_base, TMEM_COLS);
  }
}

// ---------------------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (fn == nullptr) {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) ==
            cudaSuccess &&
        q == cudaDriverEntryPointSuccess) {
      fn = reinterpret_cast<EncodeTiledFn>(ptr);
    }
  }
  return fn;
}

// bf16 tensor map with 128-byte swizzle; dims/strides innermost first, strides in bytes for
// dims 1.. (rank - 1).
static int encode_tmap(CUtensorMap* out, const void* base, int rank, const uint64_t* dims,
                       const uint64_t* strides_bytes, const uint32_t* box) {
  EncodeTiledFn fn = encode_fn();
  if (fn == nullptr) return TB200_ERR_DRIVER;
  // the encode is a driver call and needs a current context; a thread that has only switched
  // devices (an autograd worker) may not have bound the primary context yet
  static thread_local bool context_bound = false;
  if (!context_bound) {
    cudaFree(nullptr);
    context_bound = true;
  }
  cuuint64_t gdim[3];
  cuuint64_t gstr[2];
  cuuint32_t bdim[3];
  cuuint32_t estr[3] = {1, 1, 1};
  for (int i = 0; i < rank; ++i) {
    gdim[i] = dims[i];
    bdim[i] = box[i];
  }
  for (int i = 0; i + 1 < rank; ++i) gstr[i] = strides_bytes[i];
  CUresult r = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, static_cast<cuuint32_t>(rank),
                  const_cast<void*>(base), gdim, gstr, bdim, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    fprintf(stderr, "terrace_b200: tensor-map encode failed (CUresult %d): base %p rank %d dims"
            " [%llu %llu %llu] strides [%llu %llu] box [%u %u %u]\n", static_cast<int>(r), base,
            rank, (unsigned long long)gdim[0], (unsigned long long)(rank > 1 ? gdim[1] : 0),
            (unsigned long long)(rank > 2 ? gdim[2] : 0), (unsigned long long)gstr[0],
            (unsigned long long)(rank > 2 ? gstr[1] : 0), bdim[0], rank > 1 ? bdim[1] : 0,
            rank > 2 ? bdim[2] : 0);
    return TB200_ERR_TMAP;
  }
  return TB200_OK;
}

// The descriptor depends only on (base, dims, strides, box), and a training loop presents the
// same few operands every step (weights, arena sections, cached activations), so encoded maps are
// kept in a small table and the driver call leaves the launch path after the first step.
struct TmapKey {
  const void* base;
  int rank;
  uint64_t dims[3];
  uint64_t strides[2];
  uint32_t box[3];
  bool operator==(const TmapKey& o) const { return memcmp(this, &o, sizeof(TmapKey)) == 0; }
};
struct TmapSlot {
  TmapKey key;
  CUtensorMap map;
  bool used;
};
constexpr int TMAP_SLOTS = 512;          // direct-mapped; a collision just re-encodes

int make_tmap(CUtensorMap* out, const void* base, int rank, const uint64_t* dims,
              const uint64_t* strides_bytes, const uint32_t* box) {
  static TmapSlot table[TMAP_SLOTS];
  static std::mutex mu;
  TmapKey key;
  memset(&key, 0, sizeof(key));
  key.base = base;
  key.rank = rank;
  for (int i = 0; i < rank; ++i) {
    key.dims[i] = dims[i];
    key.box[i] = box[i];
  }
  for (int i = 0; i + 1 < rank; ++i) key.strides[i] = strides_bytes[i];
  uint64_t h = 1469598103934665603ull;
  const unsigned char* kb = reinterpret_cast<const unsigned char*>(&key);
  for (size_t i = 0; i < sizeof(key); ++i) h = (h ^ kb[i]) * 1099511628211ull;
  TmapSlot& slot = table[h % TMAP_SLOTS];
  std::lock_guard<std::mutex> lock(mu);
  if (slot.used && slot.key == key) {
    *out = slot.map;
    return TB200_OK;
  }
  const int rc = encode_tmap(out, base, rank, dims, strides_bytes, box);
  if (rc == TB200_OK) {
    slot.key = key;
    slot.map = *out;
    slot.used = true;
  }
  return rc;
}

template <int CTAS>
constexpr size_t gemm_smem() {
  return Cfg<CTAS>::STAGES * Cfg<CTAS>::STAGE_BYTES + OUT_STAGE_BYTES + sizeof(SharedCtl) + 1024;
}

// Pair (cta_group::2) policy: TERRACE_GEMM_PAIR = 0 (never), 1 (whenever the shapes allow) or
// auto (default: when the 256-row tiles do not waste work).  Read once.
static int pair_policy() {
  static int policy = -2;
  if (policy == -2) {
    const char* v = getenv("TERRACE_GEMM_PAIR");
    if (v == nullptr || v[0] == 'a') policy = -1;
    else policy = (v[0] == '1') ? 1 : 0;
  }
  return policy;
}

template <int MODE, int EPI, int CTAS>
static int launch_gemm(const CUtensorMap& ta, const CUtensorMap& tb, const GemmParams& p,
                       int max_ctas, cudaStream_t stream) {
  // the shared-memory opt-in is an attribute of the function ON ONE DEVICE
  static OncePerDevice configured;
  auto kern = gemm_kernel<MODE, EPI, CTAS>;
  constexpr size_t smem = gemm_smem<CTAS>();
  if (configured.need()) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             static_cast<int>(smem)) != cudaSuccess)
      return TB200_ERR_LAUNCH;
    configured.done();
  }
  int grid = sm_count();
  if (max_ctas > 0 && max_ctas < grid) grid = max_ctas;
  grid -= grid % CTAS;
  if (grid < CTAS) grid = CTAS;
  if (CTAS == 1) {
    kern<<<grid, GEMM_THREADS, smem, stream>>>(ta, tb, p);
  } else {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(static_cast<unsigned>(grid), 1, 1);
    cfg.blockDim = dim3(GEMM_THREADS, 1, 1);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = CTAS;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    if (cudaLaunchKernelEx(&cfg, kern, ta, tb, p) != cudaSuccess) {
      cudaGetLastError();
      return TB200_ERR_LAUNCH;
    }
  }
  return cudaGetLastError() == cudaSuccess ? TB200_OK : TB200_ERR_LAUNCH;
}

}  // namespace tb200

using namespace tb200;

static int grouped_gemm_impl(const void* A, const void* B, void* C, void* C2,
                             const int* seg_start, const int* seg_count, int n_groups,
                             long long a_rows, int N, int K, int ldc, int ldc2, int b_rows,
                             int b_cols, int mode, int epilogue, int* status, int max_ctas,
                             const int* wait_flags, int wait_n, int wait_epoch, int pad_align,
                             const int* row_map, const unsigned long long* scatter_base,
                             int scatter_slots, int scatter_world, cudaStream_t stream) {
  if (n_groups <= 0 || n_groups > MAX_GROUPS) return TB200_ERR_ARG;
  const bool scatter = epilogue == EPI_SCATTER;
  if (scatter && (row_map == nullptr || scatter_base == nullptr || scatter_slots < 1 ||
                  scatter_world < 1))
    return TB200_ERR_ARG;
  if ((K % 8) || (N % 8) || (ldc % 8) || (b_cols % 8)) return TB200_ERR_ARG;
  if (mode != MODE_FWD && mode != MODE_DGRAD) return TB200_ERR_ARG;
  // 256-row tiles of a CTA pair pay off when groups are long: with short groups the second
  // CTA of the last pair of a group often has no rows
  const int policy = pair_policy();
  const bool pair = policy == 1 || (policy == -1 && a_rows / n_groups >= 1024);
  CUtensorMap ta, tb;
  {
    uint64_t dims[2] = {static_cast<uint64_t>(K), static_cast<uint64_t>(a_rows)};
    uint64_t str[1] = {static_cast<uint64_t>(K) * 2};
    uint32_t box[2] = {BK, BM};
    int rc = make_tmap(&ta, A, 2, dims, str, box);
    if (rc != TB200_OK) return rc;
  }
  {
    // B is [n_groups, b_rows, b_cols] row-major.  fwd: b_rows = K, b_cols = N(+up half).
    // dgrad: b_rows = N, b_cols = K.
    uint64_t dims[3] = {static_cast<uint64_t>(b_cols), static_cast<uint64_t>(b_rows),
                        static_cast<uint64_t>(n_groups)};
    uint64_t str[2] = {static_cast<uint64_t>(b_cols) * 2,
                       static_cast<uint64_t>(b_cols) * static_cast<uint64_t>(b_rows) * 2};
    uint32_t box[3] = {64, static_cast<uint32_t>(mode == MODE_DGRAD
                                                     ? ((epilogue == EPI_SWIGLU || pair) ? 128 : BN)
                                                     : BK), 1};
    int rc = make_tmap(&tb, B, 3, dims, str, box);
    if (rc != TB200_OK) return rc;
  }
  GemmParams p{};
  p.seg_start = seg_start;
  p.seg_count = seg_count;
  p.n_groups = n_groups;
  p.N = N;
  p.K = K;
  p.M = 0;
  p.ldc = ldc;
  p.ldc2 = ldc2;
  p.up_offset = N;
  p.C = static_cast<__nv_bfloat16*>(C);
  p.C2 = static_cast<__nv_bfloat16*>(C2);
  p.status = status;
  p.wait_flags = wait_flags;
  p.wait_n = wait_n;
  p.wait_epoch = wait_epoch;
  p.pad_align = pad_align;
  p.row_map = row_map;
  p.scatter_base = scatter_base;
  p.scatter_slots = scatter_slots;
  p.scatter_world = scatter_world;
  if (epilogue == EPI_SWIGLU_BWD) {
    if (C2 == nullptr) return TB200_ERR_ARG;
    if (mode == MODE_DGRAD) {
      if (pair) return launch_gemm<MODE_DGRAD, EPI_SWIGLU_BWD, 2>(ta, tb, p, max_ctas, stream);
      return launch_gemm<MODE_DGRAD, EPI_SWIGLU_BWD, 1>(ta, tb, p, max_ctas, stream);
    }
    if (pair) return launch_gemm<MODE_FWD, EPI_SWIGLU_BWD, 2>(ta, tb, p, max_ctas, stream);
    return launch_gemm<MODE_FWD, EPI_SWIGLU_BWD, 1>(ta, tb, p, max_ctas, stream);
  }
  if (scatter) {
    if (pair) {
      if (mode == MODE_DGRAD)
        return launch_gemm<MODE_DGRAD, EPI_SCATTER, 2>(ta, tb, p, max_ctas, stream);
      return launch_gemm<MODE_FWD, EPI_SCATTER, 2>(ta, tb, p, max_ctas, stream);
    }
    if (mode == MODE_DGRAD)
      return launch_gemm<MODE_DGRAD, EPI_SCATTER, 1>(ta, tb, p, max_ctas, stream);
    return launch_gemm<MODE_FWD, EPI_SCATTER, 1>(ta, tb, p, max_ctas, stream);
  }
  if (pair) {
    if (mode == MODE_DGRAD && epilogue == EPI_SWIGLU)
      return launch_gemm<MODE_DGRAD, EPI_SWIGLU, 2>(ta, tb, p, max_ctas, stream);
    if (mode == MODE_DGRAD)
      return launch_gemm<MODE_DGRAD, EPI_PLAIN, 2>(ta, tb, p, max_ctas, stream);
    if (epilogue == EPI_SWIGLU)
      return launch_gemm<MODE_FWD, EPI_SWIGLU, 2>(ta, tb, p, max_ctas, stream);
    return launch_gemm<MODE_FWD, EPI_PLAIN, 2>(ta, tb, p, max_ctas, stream);
  }
  if (mode == MODE_DGRAD && epilogue == EPI_SWIGLU)
    return launch_gemm<MODE_DGRAD, EPI_SWIGLU, 1>(ta, tb, p, max_ctas, stream);
  if (mode == MODE_DGRAD)
    return launch_gemm<MODE_DGRAD, EPI_PLAIN, 1>(ta, tb, p, max_ctas, stream);
  if (epilogue == EPI_SWIGLU)
    return launch_gemm<MODE_FWD, EPI_SWIGLU, 1>(ta, tb, p, max_ctas, stream);
  return launch_gemm<MODE_FWD, EPI_PLAIN, 1>(ta, tb, p, max_ctas, stream);
}

extern "C" int tb200_grouped_gemm(const void* A, const void* B, void* C, void* C2,
                                  const int* seg_start, const int* seg_count, int n_groups,
                                  long long a_rows, int N, int K, int ldc, int ldc2, int b_rows,
                                  int b_cols, int mode, int epilogue, int* status, int max_ctas,
                                  const int* wait_flags, int wait_n, int wait_epoch,
                                  int pad_align, cudaStream_t stream) {
  if (epilogue != EPI_PLAIN && epilogue != EPI_SWIGLU && epilogue != EPI_SWIGLU_BWD)
    return TB200_ERR_ARG;
  return grouped_gemm_impl(A, B, C, C2, seg_start, seg_count, n_groups, a_rows, N, K, ldc, ldc2,
                           b_rows, b_cols, mode, epilogue, status, max_ctas, wait_flags, wait_n,
                           wait_epoch, pad_align, nullptr, nullptr, 0, 0, stream);
}

extern "C" int tb200_grouped_gemm_scatter(const void* A, const void* B, const int* seg_start,
                                          const int* seg_count, int n_groups, long long a_rows,
                                          int N, int K, int ld_dst, int b_rows, int b_cols,
                                          int mode, const int* row_map,
                                          const unsigned long long* scatter_base,
                                          int scatter_slots, int scatter_world, int* status,
                                          int max_ctas, cudaStream_t stream) {
  return grouped_gemm_impl(A, B, nullptr, nullptr, seg_start, seg_count, n_groups, a_rows, N, K,
                           ld_dst, 0, b_rows, b_cols, mode, EPI_SCATTER, status, max_ctas, nullptr,
                           0, 0, 0, row_map, scatter_base, scatter_slots, scatter_world, stream);
}

extern "C" int tb200_grouped_wgrad(const void* X, const void* dY, void* dW, const int* seg_start,
                                   const int* seg_count, int n_groups, long long rows, int M,
                                   int N, int* status, int max_ctas, int pad_align,
                                   cudaStream_t stream) {
  if (n_groups <= 0 || n_groups > MAX_GROUPS) return TB200_ERR_ARG;
  if ((M % 8) || (N % 8)) return TB200_ERR_ARG;
  CUtensorMap ta, tb;
  {
    uint64_t dims[2] = {static_cast<uint64_t>(M), static_cast<uint64_t>(rows)};
    uint64_t str[1] = {static_cast<uint64_t>(M) * 2};
    uint32_t box[2] = {64, BK};
    int rc = make_tmap(&ta, X, 2, dims, str, box);
    if (rc != TB200_OK) return rc;
  }
  {
    uint64_t dims[2] = {static_cast<uint64_t>(N), static_cast<uint64_t>(rows)};
    uint64_t str[1] = {static_cast<uint64_t>(N) * 2};
    uint32_t box[2] = {64, BK};
    int rc = make_tmap(&tb, dY, 2, dims, str, box);
    if (rc != TB200_OK) return rc;
  }
  GemmParams p{};
  p.seg_start = seg_start;
  p.seg_count = seg_count;
  p.n_groups = n_groups;
  p.N = N;
  p.K = 0;
  p.M = M;
  p.ldc = N;
  p.ldc2 = 0;
  p.up_offset = 0;
  p.C = static_cast<__nv_bfloat16*>(dW);
  p.C2 = nullptr;
  p.status = status;
  p.wait_flags = nullptr;
  p.wait_n = 0;
  p.wait_epoch = 0;
  p.pad_align = pad_align;
  // the pair variant has no K-tail masking: groups must be padded to whole K slices
  const int policy = pair_policy();
  const bool aligned = pad_align > 0 && pad_align % BK == 0;
  const bool long_groups = rows / n_groups >= 1024;
  if (aligned && M >= 256 && (policy == 1 || (policy == -1 && long_groups)))
    return launch_gemm<MODE_WGRAD, EPI_PLAIN, 2>(ta, tb, p, max_ctas, stream);
  return launch_gemm<MODE_WGRAD, EPI_PLAIN, 1>(ta, tb, p, max_ctas, stream);
}
