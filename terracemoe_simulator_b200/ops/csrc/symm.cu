// Fused expert-parallel dispatch / combine over NVSwitch peer memory (sm_100a).
//
// One-hop:  every (token, pick) row is stored straight into the OWNER GPU's expert-sorted GEMM
//           input at its final position; the combine pulls the expert outputs back from the
//           owners and reduces them in the canonical order.
// Two-hop (T-A2A): Hop A stores ONE row per (token, group) plus a small header (final positions,
//           expert ids, gates) into the group representative; the representative forwards each
//           arrived row to the owners inside its group (Hop B) -- again to the final position in
//           the owner's GEMM input --; on the way back the representative applies the gates
//           while it reduces the q pairs of a row (gate-at-arrival) and the origin adds its M
//           group rows.
// All positions are computed by the ORIGIN from an all-gathered [W][E] histogram, so there is
// no host round trip, no second counts exchange and the expert input has the same
// (expert, source rank, token) order on both paths: one-hop and two-hop are bit-identical.
//
// Transport: plain st.global / ld.global.cg on peer addresses + st.release.sys / ld.acquire.sys
// epoch flags.  Every wait is bounded and reports through the status word.
//
// Replaces the all_to_all_single sequences of terrace/ep_dist.py:98-122 (one-hop) and
// terrace/ta2a_fwd.py:522-670 (two-hop), the arrival chain (terrace/ops/__init__.py:255-300)
// and the pack chain (terrace/ops/k2_ref.py) of the reference.
#include "host_util.h"
#include "launch.h"
#include "ptx_sm100.cuh"
#include "symm_layout.h"

#include <cuda_bf16.h>

namespace tb200 {

__device__ __forceinline__ int* flag_ptr(const Tb200Arena& a, int rank, int kind, int idx) {
  return reinterpret_cast<int*>(a.peer[rank] + a.off_flags) + kind * TB200_MAX_WORLD + idx;
}
template <typename T>
__device__ __forceinline__ T* sect(const Tb200Arena& a, int rank, long long off) {
  return reinterpret_cast<T*>(a.peer[rank] + off);
}
__device__ __forceinline__ float warp_sum_f(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// One warp copies a row of n 16-byte chunks; four loads are issued before the four stores so that
// every lane keeps 64 bytes in flight (a peer store retires only after its NVLink round trip).
__device__ __forceinline__ void warp_copy_row(uint4* __restrict__ dst, const uint4* __restrict__ src,
                                              int n, int lane) {
  int i = lane;
  for (; i + 96 < n; i += 128) {
    const uint4 v0 = __ldcg(src + i), v1 = __ldcg(src + i + 32), v2 = __ldcg(src + i + 64),
                v3 = __ldcg(src + i + 96);
    dst[i] = v0;
    dst[i + 32] = v1;
    dst[i + 64] = v2;
    dst[i + 96] = v3;
  }
  for (; i < n; i += 32) dst[i] = __ldcg(src + i);
}

// Does local expert `le` (or an invalid pick, which the first chunk reports) belong to the
// launch that covers local experts [le_lo, le_hi)?
__device__ __forceinline__ bool in_chunk(int e, int n_experts, int epr, int le_lo, int le_hi) {
  if (e < 0 || e >= n_experts) return le_lo == 0;
  const int le = e % epr;
  return le >= le_lo && le < le_hi;
}

// Last-block-done: after this block's peer stores, publish them system-wide and count the block;
// the block that completes the count returns true (it then raises the flags).
__device__ __forceinline__ bool block_done_is_last(int* counter) {
  __shared__ int s_last;
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) {
    const int prev = atomicAdd(counter, 1);
    __threadfence_system();           // acquire side: order the other blocks' stores before ours
    s_last = (prev == static_cast<int>(gridDim.x) - 1);
    if (s_last) *counter = 0;
  }
  __syncthreads();
  return s_last != 0;
}

// Block-wide bounded wait on `n` local flags (flags[first .. first + n) >= epoch).
__device__ __forceinline__ bool block_wait_flags(const Tb200Arena& a, int kind, int first, int n,
                                                 int epoch, int* status, int code) {
  __shared__ int s_ok;
  if (threadIdx.x == 0) s_ok = 1;
  __syncthreads();
  if (static_cast<int>(threadIdx.x) < n) {
    if (!wait_flag_ge(flag_ptr(a, a.rank, kind, first + threadIdx.x), epoch)) {
      s_ok = 0;
      if (status) atomicCAS(status, 0, code);
    }
  }
  __syncthreads();
  return s_ok != 0;
}

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

// ---------------------------------------------------------------------------------------------
// Plan: all-gather the expert histogram, derive every offset table.  One block.
// ---------------------------------------------------------------------------------------------
struct PlanTables {
  int* chunk_hist;    // [CHUNKS][E]   in: per-chunk counts, out: exclusive prefix over chunks
  int* chunka_hist;   // [CHUNKS][N_g] same for Hop A rows (two-hop), may be null
  int* my_base;       // [E]  first row of MY block inside the owner's segment of expert e
  int* seg_start;     // [epr] local GEMM segments
  int* seg_count;     // [epr]
  int* rows_a;        // [W][N_g] Hop A rows rank s sends to group g
  int* my_prefix;     // [E]  rows of lower source ranks in expert e (my first row's rank in e)
};

// cap > 0: every expert accepts at most `cap` rows, in canonical order (source rank, token);
// segments shrink to min(total, cap) and the push kernels drop the picks beyond it.
__global__ void ep_plan_kernel(Tb200Arena a, PlanTables t, int epoch, int seg_align, int cap,
                               int* status) {
  extern __shared__ int sm[];
  const int E = a.n_experts, W = a.world;
  int* tot_mine = sm;             // [E]
  int* tot_all = sm + E;          // [E]
  int* seg_g = sm + 2 * E;        // [E]
  int* src_prefix = sm + 3 * E;   // [E]
  {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    for (int e = warp; e < E; e += nwarps) {
      const int total = warp_chunk_prefix(t.chunk_hist, TB200_PLAN_CHUNKS, E, e, lane);
      if (lane == 0) tot_mine[e] = total;
    }
    if (t.chunka_hist != nullptr) {
      for (int g = warp; g < a.n_nodes; g += nwarps)
        warp_chunk_prefix(t.chunka_hist, TB200_PLAN_CHUNKS, a.n_nodes, g, lane);
    }
  }
  __syncthreads();
  // publish my histogram into every rank's counts_all[me]
  for (int i = threadIdx.x; i < W * E; i += blockDim.x) {
    const int r = i / E, e = i - r * E;
    sect<int>(a, r, a.off_counts_all)[a.rank * E + e] = tot_mine[e];
  }
  __threadfence_system();
  __syncthreads();
  if (static_cast<int>(threadIdx.x) < W)
    st_release_sys(flag_ptr(a, threadIdx.x, FK_COUNTS, a.rank), epoch);
  block_wait_flags(a, FK_COUNTS, 0, W, epoch, status, ST_TIMEOUT_COUNTS);
  const int* call = sect<int>(a, a.rank, a.off_counts_all);
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    int before = 0, total = 0;
    for (int s = 0; s < W; ++s) {
      const int v = __ldcg(call + s * E + e);
      if (s < a.rank) before += v;
      total += v;
    }
    src_prefix[e] = before;
    tot_all[e] = (cap > 0 && total > cap) ? cap : total;
  }
  __syncthreads();
  if (static_cast<int>(threadIdx.x) < W) {          // thread o lays out owner o's segments
    int off = 0;
    for (int le = 0; le < a.epr; ++le) {
      const int e = threadIdx.x * a.epr + le;
      seg_g[e] = off;
      off += (tot_all[e] + seg_align - 1) / seg_align * seg_align;
    }
    if (off > a.cap_rows && status) atomicCAS(status, 0, ST_BAD_INDEX);
  }
  __syncthreads();
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    t.my_base[e] = seg_g[e] + src_prefix[e];
    t.my_prefix[e] = src_prefix[e];
    if (e / a.epr == a.rank) {
      t.seg_start[e - a.rank * a.epr] = seg_g[e];
      t.seg_count[e - a.rank * a.epr] = tot_all[e];
    }
  }
  if (t.rows_a != nullptr) {
    const int slots = a.epr * a.rpn;
    for (int i = threadIdx.x; i < W * a.n_nodes; i += blockDim.x) {
      const int s = i / a.n_nodes, g = i - s * a.n_nodes;
      int picks = 0;
      for (int j = 0; j < slots; ++j) picks += __ldcg(call + s * E + g * slots + j);
      t.rows_a[i] = picks / a.q;
    }
  }
}

// ---------------------------------------------------------------------------------------------
// One-hop push: one warp per (token, sorted pick).
//   dst[owner][pos] = scale * x[t]      (scale = gate when `gs` != null, the backward push)
//   dgs[p] = <src2[owner][pos], x[t]>   (when `dgs` != null: gate gradient, reads the owner's
//                                        saved expert output)
// A launch covers the picks whose LOCAL expert index lies in [le_lo, le_hi) and then raises the
// arrival flags to `flag_value`: the owners' GEMMs over that expert range can start while the
// next launch is still sending (the flag values of one step grow from launch to launch).
// ---------------------------------------------------------------------------------------------
__global__ void ep_push_kernel(Tb200Arena a, const __nv_bfloat16* __restrict__ x,
                               const int* __restrict__ es, const int* __restrict__ rank_local,
                               const int* __restrict__ chunk_base, const int* __restrict__ my_base,
                               int* __restrict__ pos_out, const float* __restrict__ gs,
                               float* __restrict__ dgs, long long off_dst, long long off_dot,
                               int T, int flag_kind, int flag_value, int le_lo, int le_hi,
                               int* done_counter, int* status, long long off_rowmap, int ret_slots,
                               int dot_local, const int* __restrict__ my_prefix, int cap) {
  const int lane = threadIdx.x & 31;
  const int k = a.top_k, H = a.hidden;
  const int n_pairs = T * k;
  const int per = (T + TB200_PLAN_CHUNKS - 1) / TB200_PLAN_CHUNKS;
  for (int p = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); p < n_pairs;
       p += gridDim.x * (blockDim.x >> 5)) {
    const int t = p / k;
    const int e = es[p];
    if (!in_chunk(e, a.n_experts, a.epr, le_lo, le_hi)) continue;
    const int r = rank_local[p];
    int pos = -1;
    bool dropped = false;        // beyond the expert's capacity: not an error, just not sent
    if (r >= 0 && e >= 0 && e < a.n_experts) {
      const int in_chunks = chunk_base[(t / per) * a.n_experts + e] + r;
      dropped = cap > 0 && my_prefix[e] + in_chunks >= cap;
      if (!dropped) pos = my_base[e] + in_chunks;
    }
    if (pos_out && lane == 0) pos_out[p] = pos;
    if (pos < 0 || pos >= a.cap_rows) {
      if (lane == 0) {
        if (status && !dropped) atomicCAS(status, 0, ST_BAD_INDEX);
        if (dgs) dgs[p] = 0.f;
      }
      continue;
    }
    const int owner = e / a.epr;
    const uint4* src = reinterpret_cast<const uint4*>(x + static_cast<size_t>(t) * H);
    uint4* dst = reinterpret_cast<uint4*>(sect<__nv_bfloat16>(a, owner, off_dst) +
                                          static_cast<size_t>(pos) * H);
    // return address of this row for a GEMM epilogue that scatters its output: (me, slot p)
    if (off_rowmap >= 0 && lane == 0) sect<int>(a, owner, off_rowmap)[pos] = a.rank * ret_slots + p;
    if (gs == nullptr && dgs == nullptr) {
      warp_copy_row(dst, src, H / 8, lane);
    } else {
      const float w = gs ? gs[p] : 1.0f;
      // the saved expert output of this pick: at the owner's row, or (when the forward GEMM
      // scattered its rows to the origins) in my own return slot p
      const uint4* oth = !dgs ? nullptr
                         : dot_local ? reinterpret_cast<const uint4*>(
                                           sect<__nv_bfloat16>(a, a.rank, off_dot) +
                                           static_cast<size_t>(p) * H)
                                     : reinterpret_cast<const uint4*>(
                                           sect<__nv_bfloat16>(a, owner, off_dot) +
                                           static_cast<size_t>(pos) * H);
      float dot = 0.f;
#pragma unroll 2
      for (int i = lane; i < H / 8; i += 32) {
        uint4 v = __ldcg(src + i);
        __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&v);
        if (oth) {
          uint4 o = __ldcg(oth + i);
          const __nv_bfloat162* oh = reinterpret_cast<const __nv_bfloat162*>(&o);
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const float2 g2 = __bfloat1622float2(h[j]), o2 = __bfloat1622float2(oh[j]);
            dot += g2.x * o2.x + g2.y * o2.y;
          }
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 g2 = __bfloat1622float2(h[j]);
          h[j] = __floats2bfloat162_rn(w * g2.x, w * g2.y);
        }
        dst[i] = v;
      }
      if (dgs) {
        dot = warp_sum_f(dot);
        if (lane == 0) dgs[p] = dot;
      }
    }
  }
  if (block_done_is_last(done_counter)) {
    if (static_cast<int>(threadIdx.x) < a.world)
      st_release_sys(flag_ptr(a, threadIdx.x, flag_kind, a.rank), flag_value);
  }
}

// Raise flag[kind][me] = epoch on the ranks [first, first + n), optionally after waiting for local
// flags to reach `wait_value` (the echo path of the dispatch/combine microbenchmark).
__global__ void signal_kernel(Tb200Arena a, int kind, int first, int n, int stride, int epoch,
                              int wait_kind, int wait_first, int wait_n, int wait_value, int idx,
                              int* status) {
  if (wait_kind >= 0)
    block_wait_flags(a, wait_kind, wait_first, wait_n, wait_value, status, ST_TIMEOUT_FLAG);
  __threadfence_system();
  __syncthreads();
  if (static_cast<int>(threadIdx.x) < n)
    st_release_sys(flag_ptr(a, first + threadIdx.x * stride, kind, idx), epoch);
}

// ---------------------------------------------------------------------------------------------
// One-hop pull combine: y[t] = sum_groups round( sum_picks gs * src[owner][pos] ), one block per
// token.  gs == null -> weight 1 (backward of the dispatch).
// ---------------------------------------------------------------------------------------------
__global__ void ep_pull_combine_kernel(Tb200Arena a, const int* __restrict__ pos,
                                       const int* __restrict__ es, const float* __restrict__ gs,
                                       __nv_bfloat16* __restrict__ y, long long off_src, int T,
                                       int group_size, int wait_kind, int epoch, int* status,
                                       int local_slots) {
  // local_slots > 0: the rows already sit in MY section at slot t * k + j (the owners' GEMM
  // epilogues stored them there); otherwise they are read from the owners' sections at pos
  block_wait_flags(a, wait_kind, 0, a.world, epoch, status, ST_TIMEOUT_FLAG);
  const int k = a.top_k, H = a.hidden;
  for (int t = blockIdx.x; t < T; t += gridDim.x) {
    for (int c = threadIdx.x; c < H / 8; c += blockDim.x) {
      float tot[8], par[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) tot[j] = par[j] = 0.f;
      int prev_group = -1;
      for (int j = 0; j < k; ++j) {
        const int o = t * k + j;
        const int e = es[o];
        const int grp = e / group_size;
        if (j > 0 && grp != prev_group) {
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            tot[i] += __bfloat162float(__float2bfloat16_rn(par[i]));
            par[i] = 0.f;
          }
        }
        prev_group = grp;
        const int row = local_slots > 0 ? o : pos[o];
        const int row_cap = local_slots > 0 ? local_slots : a.cap_rows;
        if (row < 0 || row >= row_cap || e < 0 || e >= a.n_experts) continue;
        if (local_slots > 0 && pos[o] < 0) continue;     // the push skipped this pick
        const float w = gs ? gs[o] : 1.0f;
        const uint4 v = __ldcg(reinterpret_cast<const uint4*>(
                                   sect<__nv_bfloat16>(a, local_slots > 0 ? a.rank : e / a.epr,
                                                       off_src) +
                                   static_cast<size_t>(row) * H) + c);
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float2 f = __bfloat1622float2(h[i]);
          par[2 * i] += w * f.x;
          par[2 * i + 1] += w * f.y;
        }
      }
      uint4 out;
      __nv_bfloat162* oh = reinterpret_cast<__nv_bfloat162*>(&out);
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const float a0 = tot[2 * i] + __bfloat162float(__float2bfloat16_rn(par[2 * i]));
        const float a1 = tot[2 * i + 1] + __bfloat162float(__float2bfloat16_rn(par[2 * i + 1]));
        oh[i] = __floats2bfloat162_rn(a0, a1);
      }
      *(reinterpret_cast<uint4*>(y + static_cast<size_t>(t) * H) + c) = out;
    }
  }
}

// ---------------------------------------------------------------------------------------------
// Two-hop, origin side.
// ---------------------------------------------------------------------------------------------
// Counting-sort ranks of the (token, run) items by destination group; one warp per token chunk.
__global__ void hopa_rank_kernel(const int* __restrict__ es, int* __restrict__ ranka_local,
                                 int* __restrict__ chunka_hist, int T, int k, int groups_m,
                                 int slots, int n_nodes) {
  __shared__ int s_cnt[TB200_MAX_WORLD * 4];
  __shared__ unsigned s_mask[TB200_MAX_WORLD * 4];
  const int lane = threadIdx.x;
  const int per = (T + TB200_PLAN_CHUNKS - 1) / TB200_PLAN_CHUNKS;
  const int t0 = blockIdx.x * per, t1 = min(T, t0 + per);
  const int q = k / groups_m;
  for (int g = lane; g < n_nodes; g += 32) {
    s_cnt[g] = 0;
    s_mask[g] = 0u;
  }
  __syncwarp();
  // Rank of every (token, run) among the rows bound for its group, in TOKEN order: a token
  // sends at most one run to a group, so the lower tokens of a 32-token batch that address
  // group g are a bit count over a per-group lane mask.
  for (int tb = t0; tb < t1; tb += 32) {
    const int t = tb + lane;
    const bool live = t < t1;
    auto group_of = [&](int m) {
      const int e = es[t * k + m * q];
      const int g = e >= 0 ? e / slots : -1;
      return (g >= 0 && g < n_nodes) ? g : -1;
    };
    if (live)
      for (int m = 0; m < groups_m; ++m) {
        const int g = group_of(m);
        if (g >= 0) atomicOr(&s_mask[g], 1u << lane);
      }
    __syncwarp();
    if (live)
      for (int m = 0; m < groups_m; ++m) {
        const int g = group_of(m);
        ranka_local[t * groups_m + m] =
            g >= 0 ? s_cnt[g] + __popc(s_mask[g] & ((1u << lane) - 1u)) : -1;
      }
    __syncwarp();
    if (live)
      for (int m = 0; m < groups_m; ++m) {
        const int g = group_of(m);
        if (g >= 0 && (s_mask[g] >> lane) == 1u) s_cnt[g] += __popc(s_mask[g]);
      }
    __syncwarp();
    if (live)
      for (int m = 0; m < groups_m; ++m) {
        const int g = group_of(m);
        if (g >= 0) s_mask[g] = 0u;
      }
    __syncwarp();
  }
  for (int g = lane; g < n_nodes; g += 32) chunka_hist[blockIdx.x * n_nodes + g] = s_cnt[g];
}

// Hop A push: one warp per (token, run): row (+ header) into the representative of the run's
// group.  `with_header` = forward (writes pos / expert / gate per pick and computes pos).
__global__ void hopa_push_kernel(Tb200Arena a, const __nv_bfloat16* __restrict__ x,
                                 const int* __restrict__ es, const float* __restrict__ gs,
                                 const int* __restrict__ rank_local,
                                 const int* __restrict__ chunk_base,
                                 const int* __restrict__ my_base,
                                 const int* __restrict__ ranka_local,
                                 const int* __restrict__ chunka_base, int* __restrict__ pos_out,
                                 int* __restrict__ rowa_out, long long off_rows, int with_header,
                                 int T, int flag_kind, int epoch, int* done_counter, int* status,
                                 const int* __restrict__ my_prefix, int cap) {
  const int lane = threadIdx.x & 31;
  const int k = a.top_k, H = a.hidden, M = a.groups_m, q = a.q;
  const int slots = a.epr * a.rpn;
  const int my_local = a.rank % a.rpn, my_group = a.rank / a.rpn;
  const int per = (T + TB200_PLAN_CHUNKS - 1) / TB200_PLAN_CHUNKS;
  for (int item = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); item < T * M;
       item += gridDim.x * (blockDim.x >> 5)) {
    const int t = item / M, m = item - t * M;
    const int e0 = es[t * k + m * q];
    const int ra = ranka_local[item];
    const int g = (e0 >= 0) ? e0 / slots : -1;
    int dst_row = -1;
    if (ra >= 0 && g >= 0 && g < a.n_nodes)
      dst_row = my_group * a.tokens_cap + chunka_base[(t / per) * a.n_nodes + g] + ra;
    if (with_header) {
      if (lane == 0) rowa_out[item] = dst_row;
    } else {
      dst_row = rowa_out[item];
    }
    if (dst_row < 0 || dst_row >= a.n_nodes * a.tokens_cap || g < 0 || g >= a.n_nodes) {
      if (lane == 0 && status) atomicCAS(status, 0, ST_BAD_INDEX);
      continue;
    }
    const int rep = g * a.rpn + my_local;
    if (with_header && lane < q) {
      const int p = t * k + m * q + lane;
      const int e = es[p];
      const int r = rank_local[p];
      int pos = -1;            // also what a pick beyond the expert's capacity carries
      if (r >= 0 && e >= 0 && e < a.n_experts) {
        const int in_chunks = chunk_base[(t / per) * a.n_experts + e] + r;
        if (!(cap > 0 && my_prefix[e] + in_chunks >= cap)) pos = my_base[e] + in_chunks;
      }
      pos_out[p] = pos;
      int* hdr = sect<int>(a, rep, a.off_ha_hdr) + static_cast<size_t>(dst_row) * 3 * q;
      hdr[lane] = pos;
      hdr[q + lane] = e;
      hdr[2 * q + lane] = __float_as_int(gs[p]);
    }
    const uint4* src = reinterpret_cast<const uint4*>(x + static_cast<size_t>(t) * H);
    uint4* dst = reinterpret_cast<uint4*>(sect<__nv_bfloat16>(a, rep, off_rows) +
                                          static_cast<size_t>(dst_row) * H);
    warp_copy_row(dst, src, H / 8, lane);
  }
  if (block_done_is_last(done_counter)) {
    if (static_cast<int>(threadIdx.x) < a.n_nodes)
      st_release_sys(flag_ptr(a, threadIdx.x * a.rpn + my_local, flag_kind, my_group), epoch);
  }
}

// ---------------------------------------------------------------------------------------------
// Two-hop, representative (arrival) side.
// ---------------------------------------------------------------------------------------------
// Hop B push: one warp per (arrived row, pick): forward the row to the pick's owner at its final
// position.  scale_gate: multiply by the pick's gate (backward); want_dgate: also write
// dgate[row][c] = <saved expert output of the pick, row>.  Like the one-hop push, a launch covers
// the picks of local experts [le_lo, le_hi) and raises the owners' data flags to `flag_value`.
// off_rowmap >= 0: the return address of every forwarded row (me, slot row * q + c) is left in
// the owner's row map for a GEMM epilogue that scatters its output back to this representative;
// dot_local: the saved expert output is read from MY return section (off_dot) at that slot
// instead of the owner's row.
__global__ void arrival_push_kernel(Tb200Arena a, const int* __restrict__ rows_a,
                                    long long off_rows, long long off_dst, long long off_dot,
                                    int scale_gate, int want_dgate, int wait_kind, int data_kind,
                                    int dg_kind, int epoch, int flag_value, int le_lo, int le_hi,
                                    int* done_counter, int* status, long long off_rowmap,
                                    int dot_local) {
  const int lane = threadIdx.x & 31;
  const int H = a.hidden, q = a.q, Tc = a.tokens_cap;
  const int my_local = a.rank % a.rpn, my_group = a.rank / a.rpn;
  block_wait_flags(a, wait_kind, 0, a.n_nodes, epoch, status, ST_TIMEOUT_FLAG);
  const int total = a.n_nodes * Tc * q;
  const __nv_bfloat16* rows = sect<__nv_bfloat16>(a, a.rank, off_rows);
  const int* hdrs = sect<int>(a, a.rank, a.off_ha_hdr);
  float* dgate = sect<float>(a, a.rank, a.off_dgate);
  for (int item = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); item < total;
       item += gridDim.x * (blockDim.x >> 5)) {
    const int row = item / q, c = item - row * q;
    const int sg = row / Tc, i = row - sg * Tc;
    const int n_rows = rows_a[(sg * a.rpn + my_local) * a.n_nodes + my_group];
    if (i >= n_rows) continue;
    const int* hdr = hdrs + static_cast<size_t>(row) * 3 * q;
    const int pos = __ldcg(hdr + c);
    const int e = __ldcg(hdr + q + c);
    if (!in_chunk(e, a.n_experts, a.epr, le_lo, le_hi)) continue;
    if (pos < 0 || pos >= a.cap_rows || e < 0 || e >= a.n_experts ||
        e / (a.epr * a.rpn) != my_group) {
      if (lane == 0) {
        // pos == -1 with a valid expert: the origin dropped the pick (capacity), no error
        const bool dropped = pos == -1 && e >= 0 && e < a.n_experts;
        if (status && !dropped) atomicCAS(status, 0, ST_BAD_INDEX);
        if (want_dgate) dgate[static_cast<size_t>(row) * q + c] = 0.f;
      }
      continue;
    }
    const int owner = e / a.epr;
    const float w = scale_gate ? __int_as_float(__ldcg(hdr + 2 * q + c)) : 1.0f;
    const uint4* src = reinterpret_cast<const uint4*>(rows + static_cast<size_t>(row) * H);
    uint4* dst = reinterpret_cast<uint4*>(sect<__nv_bfloat16>(a, owner, off_dst) +
                                          static_cast<size_t>(pos) * H);
    if (off_rowmap >= 0 && lane == 0)
      sect<int>(a, owner, off_rowmap)[pos] = a.rank * (a.n_nodes * Tc * q) + item;
    if (!scale_gate && !want_dgate) {
      warp_copy_row(dst, src, H / 8, lane);
      continue;
    }
    const uint4* oth = !want_dgate ? nullptr
                       : dot_local ? reinterpret_cast<const uint4*>(
                                         sect<__nv_bfloat16>(a, a.rank, off_dot) +
                                         static_cast<size_t>(item) * H)
                                   : reinterpret_cast<const uint4*>(
                                         sect<__nv_bfloat16>(a, owner, off_dot) +
                                         static_cast<size_t>(pos) * H);
    float dot = 0.f;
#pragma unroll 2
    for (int j = lane; j < H / 8; j += 32) {
      uint4 v = __ldcg(src + j);
      __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&v);
      uint4 o = make_uint4(0, 0, 0, 0);
      if (oth) o = __ldcg(oth + j);
      const __nv_bfloat162* oh = reinterpret_cast<const __nv_bfloat162*>(&o);
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const float2 g2 = __bfloat1622float2(h[u]), o2 = __bfloat1622float2(oh[u]);
        dot += g2.x * o2.x + g2.y * o2.y;
        h[u] = __floats2bfloat162_rn(w * g2.x, w * g2.y);
      }
      dst[j] = v;
    }
    if (want_dgate) {
      dot = warp_sum_f(dot);
      if (lane == 0) dgate[static_cast<size_t>(row) * q + c] = dot;
    }
  }
  if (block_done_is_last(done_counter)) {
    if (static_cast<int>(threadIdx.x) < a.rpn)
      st_release_sys(flag_ptr(a, my_group * a.rpn + threadIdx.x, data_kind, a.rank), flag_value);
    if (dg_kind >= 0 && static_cast<int>(threadIdx.x) < a.n_nodes)
      st_release_sys(flag_ptr(a, threadIdx.x * a.rpn + my_local, dg_kind, my_group), epoch);
  }
}

// Arrival combine: one block per arrived row: red[row] = sum_c gate_c * src[owner_c][pos_c]
// (picks ascending), fp32, rounded once.
__global__ void arrival_combine_kernel(Tb200Arena a, const int* __restrict__ rows_a,
                                       long long off_src, long long off_red, int use_gate,
                                       int wait_kind, int red_kind, int epoch, int* done_counter,
                                       int* status, int push_back, int local_slots) {
  // push_back: the reduced row goes straight into the ORIGIN's section (block of my group, row
  // i) instead of my own (block of the source group); the origin then combines from local memory
  // local_slots: the owners' GEMM epilogues stored the expert output of (row, c) into MY section
  // off_src at slot row * q + c; otherwise it is read from the owner's section at pos
  const int H = a.hidden, q = a.q, Tc = a.tokens_cap;
  const int my_local = a.rank % a.rpn, my_group = a.rank / a.rpn;
  block_wait_flags(a, wait_kind, my_group * a.rpn, a.rpn, epoch, status, ST_TIMEOUT_FLAG);
  const int* hdrs = sect<int>(a, a.rank, a.off_ha_hdr);
  __nv_bfloat16* red_local = sect<__nv_bfloat16>(a, a.rank, off_red);
  for (int row = blockIdx.x; row < a.n_nodes * Tc; row += gridDim.x) {
    const int sg = row / Tc, i = row - sg * Tc;
    const int n_rows = rows_a[(sg * a.rpn + my_local) * a.n_nodes + my_group];
    if (i >= n_rows) continue;
    const int* hdr = hdrs + static_cast<size_t>(row) * 3 * q;
    __nv_bfloat16* red_row =
        push_back ? sect<__nv_bfloat16>(a, sg * a.rpn + my_local, off_red) +
                        (static_cast<size_t>(my_group) * Tc + i) * H
                  : red_local + static_cast<size_t>(row) * H;
    for (int cix = threadIdx.x; cix < H / 8; cix += blockDim.x) {
      float acc[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] = 0.f;
      for (int c = 0; c < q; ++c) {
        const int pos = __ldcg(hdr + c);
        const int e = __ldcg(hdr + q + c);
        if (pos < 0 || pos >= a.cap_rows || e < 0 || e >= a.n_experts) continue;
        const float w = use_gate ? __int_as_float(__ldcg(hdr + 2 * q + c)) : 1.0f;
        const __nv_bfloat16* srow =
            local_slots ? sect<__nv_bfloat16>(a, a.rank, off_src) +
                              (static_cast<size_t>(row) * q + c) * H
                        : sect<__nv_bfloat16>(a, e / a.epr, off_src) + static_cast<size_t>(pos) * H;
        const uint4 v = __ldcg(reinterpret_cast<const uint4*>(srow) + cix);
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const float2 f = __bfloat1622float2(h[u]);
          acc[2 * u] += w * f.x;
          acc[2 * u + 1] += w * f.y;
        }
      }
      uint4 out;
      __nv_bfloat162* oh = reinterpret_cast<__nv_bfloat162*>(&out);
#pragma unroll
      for (int u = 0; u < 4; ++u) oh[u] = __floats2bfloat162_rn(acc[2 * u], acc[2 * u + 1]);
      *(reinterpret_cast<uint4*>(red_row) + cix) = out;
    }
  }
  if (block_done_is_last(done_counter)) {
    if (static_cast<int>(threadIdx.x) < a.n_nodes)
      st_release_sys(flag_ptr(a, threadIdx.x * a.rpn + my_local, red_kind, my_group), epoch);
  }
}

// Origin combine: y[t] = sum over the token's M group rows (groups ascending), one block per token.
__global__ void origin_combine_kernel(Tb200Arena a, const int* __restrict__ es,
                                      const int* __restrict__ rowa, __nv_bfloat16* __restrict__ y,
                                      long long off_red, int T, int wait_kind, int epoch,
                                      int* status, int local_rows) {
  // local_rows: the representatives pushed the reduced rows into MY section (block of their
  // group, same row inside the block); otherwise they are read from the representatives
  block_wait_flags(a, wait_kind, 0, a.n_nodes, epoch, status, ST_TIMEOUT_FLAG);
  const int H = a.hidden, M = a.groups_m, q = a.q, k = a.top_k;
  const int slots = a.epr * a.rpn, my_local = a.rank % a.rpn, my_group = a.rank / a.rpn;
  for (int t = blockIdx.x; t < T; t += gridDim.x) {
    for (int cix = threadIdx.x; cix < H / 8; cix += blockDim.x) {
      float acc[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] = 0.f;
      for (int m = 0; m < M; ++m) {
        const int e0 = es[t * k + m * q];
        const int row = rowa[t * M + m];
        if (e0 < 0 || e0 >= a.n_experts || row < 0 || row >= a.n_nodes * a.tokens_cap) continue;
        const int g = e0 / slots;
        int rep = g * a.rpn + my_local, src_row = row;
        if (local_rows) {
          const int i = row - my_group * a.tokens_cap;      // my rank among the rows sent to g
          if (i < 0 || i >= a.tokens_cap || g >= a.n_nodes) continue;
          rep = a.rank;
          src_row = g * a.tokens_cap + i;
        }
        const uint4 v = __ldcg(reinterpret_cast<const uint4*>(
                                   sect<__nv_bfloat16>(a, rep, off_red) +
                                   static_cast<size_t>(src_row) * H) + cix);
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const float2 f = __bfloat1622float2(h[u]);
          acc[2 * u] += f.x;
          acc[2 * u + 1] += f.y;
        }
      }
      uint4 out;
      __nv_bfloat162* oh = reinterpret_cast<__nv_bfloat162*>(&out);
#pragma unroll
      for (int u = 0; u < 4; ++u) oh[u] = __floats2bfloat162_rn(acc[2 * u], acc[2 * u + 1]);
      *(reinterpret_cast<uint4*>(y + static_cast<size_t>(t) * H) + cix) = out;
    }
  }
}

// dgs[t, m*q + c] = dgate[rep_m][rowa[t, m]][c]
__global__ void origin_pull_dgate_kernel(Tb200Arena a, const int* __restrict__ es,
                                         const int* __restrict__ rowa, float* __restrict__ dgs,
                                         int T, int wait_kind, int epoch, int* status) {
  block_wait_flags(a, wait_kind, 0, a.n_nodes, epoch, status, ST_TIMEOUT_FLAG);
  const int M = a.groups_m, q = a.q, k = a.top_k;
  const int slots = a.epr * a.rpn, my_local = a.rank % a.rpn;
  for (int p = blockIdx.x * blockDim.x + threadIdx.x; p < T * k; p += gridDim.x * blockDim.x) {
    const int t = p / k, j = p - t * k;
    const int m = j / q, c = j - m * q;
    const int e0 = es[t * k + m * q];
    const int row = rowa[t * M + m];
    float v = 0.f;
    if (e0 >= 0 && e0 < a.n_experts && row >= 0 && row < a.n_nodes * a.tokens_cap) {
      const int rep = (e0 / slots) * a.rpn + my_local;
      v = __ldcg(sect<float>(a, rep, a.off_dgate) + static_cast<size_t>(row) * q + c);
    }
    dgs[p] = v;
  }
}

}  // namespace tb200

using namespace tb200;

#define LAUNCH_OK() (cudaGetLastError() == cudaSuccess ? TB200_OK : TB200_ERR_LAUNCH)

static bool arena_ok(const Tb200Arena* a) {
  return a && a->world >= 1 && a->world <= TB200_MAX_WORLD && a->hidden % 8 == 0 &&
         a->n_experts == a->epr * a->world && a->world % a->rpn == 0 &&
         a->n_nodes == a->world / a->rpn && a->n_nodes <= TB200_MAX_WORLD &&
         a->top_k == a->q * a->groups_m && a->q <= 32 && a->n_experts <= 1024;
}

extern "C" int tb200_ep_plan(const Tb200Arena* a, int* chunk_hist, int* chunka_hist, int* my_base,
                             int* seg_start, int* seg_count, int* rows_a, int* my_prefix,
                             int epoch, int seg_align, int cap, int* status, cudaStream_t stream) {
  if (!arena_ok(a) || seg_align < 1 || my_prefix == nullptr) return TB200_ERR_ARG;
  PlanTables t{chunk_hist, chunka_hist, my_base, seg_start, seg_count, rows_a, my_prefix};
  ep_plan_kernel<<<1, 256, 4 * a->n_experts * sizeof(int), stream>>>(*a, t, epoch, seg_align,
                                                                     cap, status);
  return LAUNCH_OK();
}

// Grid of a warp-per-item kernel: enough blocks of 8 warps for `items`, at most 8 per SM.
static int warp_item_grid(long long items) {
  long long blocks = (items + 7) / 8;
  const long long cap = static_cast<long long>(sm_count()) * 8;
  if (blocks < 1) blocks = 1;
  return static_cast<int>(blocks > cap ? cap : blocks);
}

extern "C" int tb200_ep_push(const Tb200Arena* a, const void* x, const int* es,
                             const int* rank_local, const int* chunk_base, const int* my_base,
                             int* pos_out, const float* gs, float* dgs, long long off_dst,
                             long long off_dot, int T, int flag_kind, int flag_value, int le_lo,
                             int le_hi, int* done_counter, int* status, long long off_rowmap,
                             int ret_slots, int dot_local, const int* my_prefix, int cap,
                             cudaStream_t stream) {
  if (!arena_ok(a) || le_lo < 0 || le_hi > a->epr || le_lo >= le_hi) return TB200_ERR_ARG;
  if (cap > 0 && my_prefix == nullptr) return TB200_ERR_ARG;
  if ((off_rowmap >= 0 || dot_local) && ret_slots < T * a->top_k) return TB200_ERR_ARG;
  // a launch that covers a part of the experts touches about that share of the picks
  const long long items = static_cast<long long>(T) * a->top_k;
  const int blocks = warp_item_grid(le_hi - le_lo == a->epr ? items
                                                            : items * (le_hi - le_lo) / a->epr * 2);
  ep_push_kernel<<<blocks, 256, 0, stream>>>(*a, static_cast<const __nv_bfloat16*>(x), es,
                                             rank_local, chunk_base, my_base, pos_out, gs, dgs,
                                             off_dst, off_dot, T, flag_kind, flag_value, le_lo,
                                             le_hi, done_counter, status, off_rowmap, ret_slots,
                                             dot_local, my_prefix, cap);
  return LAUNCH_OK();
}

extern "C" int tb200_signal(const Tb200Arena* a, int kind, int first, int n, int stride, int idx,
                            int epoch, int wait_kind, int wait_first, int wait_n, int wait_value,
                            int* status, cudaStream_t stream) {
  if (!arena_ok(a) || n > 32 || wait_n > 32) return TB200_ERR_ARG;
  signal_kernel<<<1, 32, 0, stream>>>(*a, kind, first, n, stride, epoch, wait_kind, wait_first,
                                      wait_n, wait_value, idx, status);
  return LAUNCH_OK();
}

extern "C" int tb200_ep_pull_combine(const Tb200Arena* a, const int* pos, const int* es,
                                     const float* gs, void* y, long long off_src, int T,
                                     int group_size, int wait_kind, int epoch, int* status,
                                     int local_slots, cudaStream_t stream) {
  if (!arena_ok(a) || group_size < 1) return TB200_ERR_ARG;
  if (local_slots > 0 && local_slots < T * a->top_k) return TB200_ERR_ARG;
  const int cap = sm_count() * 8;
  const int blocks = T < 1 ? 1 : (T > cap ? cap : T);
  ep_pull_combine_kernel<<<blocks, 256, 0, stream>>>(*a, pos, es, gs,
                                                     static_cast<__nv_bfloat16*>(y), off_src, T,
                                                     group_size, wait_kind, epoch, status,
                                                     local_slots);
  return LAUNCH_OK();
}

extern "C" int tb200_hopa_rank(const Tb200Arena* a, const int* es, int* ranka_local,
                               int* chunka_hist, int T, cudaStream_t stream) {
  if (!arena_ok(a)) return TB200_ERR_ARG;
  hopa_rank_kernel<<<TB200_PLAN_CHUNKS, 32, 0, stream>>>(es, ranka_local, chunka_hist, T,
                                                         a->top_k, a->groups_m,
                                                         a->epr * a->rpn, a->n_nodes);
  return LAUNCH_OK();
}

extern "C" int tb200_hopa_push(const Tb200Arena* a, const void* x, const int* es, const float* gs,
                               const int* rank_local, const int* chunk_base, const int* my_base,
                               const int* ranka_local, const int* chunka_base, int* pos_out,
                               int* rowa, long long off_rows, int with_header, int T,
                               int flag_kind, int epoch, int* done_counter, int* status,
                               const int* my_prefix, int cap, cudaStream_t stream) {
  if (!arena_ok(a) || T > a->tokens_cap) return TB200_ERR_ARG;
  if (cap > 0 && my_prefix == nullptr) return TB200_ERR_ARG;
  const int blocks = warp_item_grid(static_cast<long long>(T) * a->groups_m);
  hopa_push_kernel<<<blocks, 256, 0, stream>>>(
      *a, static_cast<const __nv_bfloat16*>(x), es, gs, rank_local, chunk_base, my_base,
      ranka_local, chunka_base, pos_out, rowa, off_rows, with_header, T, flag_kind, epoch,
      done_counter, status, my_prefix, cap);
  return LAUNCH_OK();
}

extern "C" int tb200_arrival_push(const Tb200Arena* a, const int* rows_a, long long off_rows,
                                  long long off_dst, long long off_dot, int scale_gate,
                                  int want_dgate, int wait_kind, int data_kind, int dg_kind,
                                  int epoch, int flag_value, int le_lo, int le_hi,
                                  int* done_counter, int* status, long long off_rowmap,
                                  int dot_local, cudaStream_t stream) {
  if (!arena_ok(a) || le_lo < 0 || le_hi > a->epr || le_lo >= le_hi) return TB200_ERR_ARG;
  arrival_push_kernel<<<sm_count() * 8, 256, 0, stream>>>(
      *a, rows_a, off_rows, off_dst, off_dot, scale_gate, want_dgate, wait_kind, data_kind,
      dg_kind, epoch, flag_value, le_lo, le_hi, done_counter, status, off_rowmap, dot_local);
  return LAUNCH_OK();
}

extern "C" int tb200_arrival_combine(const Tb200Arena* a, const int* rows_a, long long off_src,
                                     long long off_red, int use_gate, int wait_kind, int red_kind,
                                     int epoch, int* done_counter, int* status, int push_back,
                                     int local_slots, cudaStream_t stream) {
  if (!arena_ok(a)) return TB200_ERR_ARG;
  arrival_combine_kernel<<<sm_count() * 8, 256, 0, stream>>>(*a, rows_a, off_src, off_red,
                                                             use_gate, wait_kind, red_kind, epoch,
                                                             done_counter, status, push_back,
                                                             local_slots);
  return LAUNCH_OK();
}

extern "C" int tb200_origin_combine(const Tb200Arena* a, const int* es, const int* rowa, void* y,
                                    long long off_red, int T, int wait_kind, int epoch, int* status,
                                    int local_rows, cudaStream_t stream) {
  if (!arena_ok(a)) return TB200_ERR_ARG;
  const int cap = sm_count() * 8;
  const int blocks = T < 1 ? 1 : (T > cap ? cap : T);
  origin_combine_kernel<<<blocks, 256, 0, stream>>>(*a, es, rowa, static_cast<__nv_bfloat16*>(y),
                                                    off_red, T, wait_kind, epoch, status,
                                                    local_rows);
  return LAUNCH_OK();
}

extern "C" int tb200_origin_pull_dgate(const Tb200Arena* a, const int* es, const int* rowa,
                                       float* dgs, int T, int wait_kind, int epoch, int* status,
                                       cudaStream_t stream) {
  if (!arena_ok(a)) return TB200_ERR_ARG;
  origin_pull_dgate_kernel<<<64, 256, 0, stream>>>(*a, es, rowa, dgs, T, wait_kind, epoch, status);
  return LAUNCH_OK();
}
