// C launch interface of the sm_100a kernels.  Plain pointers and a stream: no allocation, no
// torch types, so the kernels can be driven from the torch bindings (bindings.cpp) or from any
// other host runtime.  Every function returns TB200_OK or an error code and never throws.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum {
  TB200_OK = 0,
  TB200_ERR_ARG = 1,      // unsupported shape / alignment
  TB200_ERR_DRIVER = 2,   // driver entry point unavailable
  TB200_ERR_TMAP = 3,     // tensor-map encode failed
  TB200_ERR_LAUNCH = 4,   // kernel launch failed
  TB200_ERR_SIZE = 5,     // problem exceeds a stated maximum
};

// ---- gemm_sm100.cu ---------------------------------------------------------------------------
// mode 0 (fwd):   C[rows, N] = A[rows, K] * B[g][K, N]   (B row-major [b_rows=K, b_cols])
// mode 1 (dgrad): C[rows, N] = A[rows, K] * B[g][N, K]^T (B row-major [b_rows=N, b_cols=K])
// epilogue 1: B holds [gate | up] halves (fwd: b_cols = 2N; dgrad: b_rows = 2N);
// C = silu(gate) * up, and when C2 != null the bf16 pre-activations go to C2[rows, 2N].
// epilogue 3: SwiGLU backward fused behind the GEMM that produces d(act): the product is d(act)
// [rows, N]; C2 (input) holds the saved pre-activations [rows, 2N] = [gate | up] and C (output,
// ldc = 2N) receives d[gate | up].
// Rows of group g are A[seg_start[g] .. seg_start[g] + seg_count[g]).
int tb200_grouped_gemm(const void* A, const void* B, void* C, void* C2, const int* seg_start,
                       const int* seg_count, int n_groups, long long a_rows, int N, int K, int ldc,
                       int ldc2, int b_rows, int b_cols, int mode, int epilogue, int* status,
                       int max_ctas, const int* wait_flags, int wait_n, int wait_epoch,
                       int pad_align, cudaStream_t stream);
// Plain fwd / dgrad GEMM whose output rows are scattered: row r (inside the segments) goes to
// scatter_base[m / scatter_slots] + (m % scatter_slots) * ld_dst elements with m = row_map[r];
// scatter_base[] are device addresses that may belong to peer GPUs (plain stores, published
// system-wide before the kernel ends).  Rows with a map value outside [0, world * slots) are
// skipped and ST_BAD_INDEX is recorded.  Padding rows are not written anywhere.
int tb200_grouped_gemm_scatter(const void* A, const void* B, const int* seg_start,
                               const int* seg_count, int n_groups, long long a_rows, int N, int K,
                               int ld_dst, int b_rows, int b_cols, int mode, const int* row_map,
                               const unsigned long long* scatter_base, int scatter_slots,
                               int scatter_world, int* status, int max_ctas, cudaStream_t stream);
// dW[g][M, N] = X[rows of g, M]^T * dY[rows of g, N]; groups with no rows get zeros.
// (dW may be a slice of a larger gradient tensor: a chunk of the groups at a time)
int tb200_grouped_wgrad(const void* X, const void* dY, void* dW, const int* seg_start,
                        const int* seg_count, int n_groups, long long rows, int M, int N,
                        int* status, int max_ctas, int pad_align, cudaStream_t stream);
// pad_align > 0 declares that every group's rows are padded to that multiple: the fwd / dgrad
// kernels then write zeros into the padding rows of C (and C2), and the wgrad kernel, when the
// multiple is a multiple of 64, reads them as zero contributions instead of masking the K tail in
// shared memory.  Zero the padding of buffers no GEMM writes with tb200_zero_pad_rows.
int tb200_zero_pad_rows(void* buf, const int* seg_start, const int* seg_count, int n_groups,
                        int align, int row_bytes, long long buf_rows, cudaStream_t stream);

// ---- attention_sm100.cu ----------------------------------------------------------------------
// Self-attention over q, k, v [BH, S, D] bf16 contiguous (S a multiple of 128, D 64 or 128):
// o = softmax(scale * q k^T (+ causal mask)) v, lse[BH, S] = log-sum-exp of the scaled scores.
int tb200_attn_fwd(const void* q, const void* k, const void* v, void* o, float* lse, int BH,
                   int S, int D, int causal, float scale, int* status, cudaStream_t stream);
// Gradients dq, dk, dv [BH, S, D] from d_o; `delta` is [BH, S] fp32 scratch (rowsum(d_o * o)).
int tb200_attn_bwd(const void* q, const void* k, const void* v, const void* o, const void* d_o,
                   const float* lse, float* delta, void* dq, void* dk, void* dv, int BH, int S,
                   int D, int causal, float scale, int* status, cudaStream_t stream);

// ---- moe_kernels.cu --------------------------------------------------------------------------
int tb200_passthrough(const void* src, void* dst, size_t bytes, cudaStream_t stream);

int tb200_rmsnorm_fwd(const void* x, const void* w, void* y, float* rstd, long long rows, int dim,
                      float eps, int is_bf16, cudaStream_t stream);
int tb200_rmsnorm_bwd(const void* x, const void* w, const void* dy, const float* rstd, void* dx,
                      float* dw_partial, int n_partial, long long rows, int dim, int is_bf16,
                      cudaStream_t stream);

// Router select (mode "full"): logits[T, E] fp32 -> idx[T, k] int64, gates[T, k] fp32,
// group_idx[T, M] int64, load[E] fp32 (accumulated; caller zeroes).
int tb200_route_select(const float* logits, const float* bias, long long* idx, float* gates,
                       long long* group_idx, float* load, float* affinity_sel, int T, int E,
                       int n_groups, int top_k, int top_groups, int pool, cudaStream_t stream);
// The same selection fused behind the router GEMM (router_sm100.cu): x[T, H] and w[E, H] bf16,
// logits accumulate in TMEM and never reach memory.  E <= 128 and a multiple of 16.
int tb200_route_fused_supported(int E, int H, int n_groups, int top_k, int top_groups);
int tb200_route_fused(const void* x, const void* w, const float* bias, long long* idx,
                      float* gates, long long* group_idx, float* load, float* affinity_sel, int T,
                      int E, int H, int n_groups, int top_k, int top_groups, int pool, int* status,
                      cudaStream_t stream);
// dlogits[T, E] (pre-zeroed) from dgates[T, k]: through the renormalisation and the sigmoid.
int tb200_route_select_bwd(const float* dgates, const float* gates, const float* affinity_sel,
                           const long long* idx, float* dlogits, int T, int E, int top_k,
                           cudaStream_t stream);

// Local permutation plan: counting sort of the T*k picks by expert, stable in (token, expert).
//   es/gs/cols [T, k]: per-token ascending expert ids, their gates, their original columns
//   pos [T, k]: row of every (sorted) pick in the expert-sorted buffer
//   seg_start/seg_count [E]
// `scratch` needs tb200_plan_scratch_ints(T, k, E) ints.
size_t tb200_plan_scratch_ints(int T, int k, int E);
// first pass only (sorted picks, local ranks, per-chunk histogram [TB200_PLAN_CHUNKS][E])
int tb200_plan_pass1(const long long* expert_idx, const float* gates, int* es, float* gs, int* cols,
                     int* rank_local, int* chunk_hist, int T, int k, int E, cudaStream_t stream);
int tb200_moe_plan(const long long* expert_idx, const float* gates, int* es, float* gs, int* cols,
                   int* pos, int* seg_start, int* seg_count, int* scratch, int T, int k, int E,
                   int seg_align, cudaStream_t stream);
// xs[pos[t, j]] = x[t]   (bf16 rows of `dim` elements)
int tb200_moe_scatter_rows(const void* x, void* xs, const int* pos, int T, int k, int dim,
                           long long xs_rows, int* status, cudaStream_t stream);
// y[t] = sum over groups asc ( sum over picks asc in group  gs * out[pos] ), fp32 accumulation,
// group partial and total each rounded once to bf16.  gs == null means weight 1.
int tb200_moe_combine(const void* out, const int* pos, const int* es, const float* gs, void* y,
                      int T, int k, int dim, int group_size, long long out_rows, int* status,
                      cudaStream_t stream);
// dout[pos] = gs * dy[t];  dgs[t, j] = <out[pos], dy[t]>
int tb200_moe_combine_bwd(const void* dy, const void* out, const int* pos, const float* gs,
                          void* dout, float* dgs, int T, int k, int dim, long long out_rows,
                          int* status, cudaStream_t stream);
// RoPE fused with the head split: merge == 0 reads qkv[B, T, 3 * nh * hd] and writes q, k
// (rotated) and v, each [B, nh, T, hd]; merge == 1 is the adjoint (gradients back into qkv
// layout, q and k parts rotated by the opposite angle).  cos / sin: fp32 [T, hd / 2].
int tb200_rope_split_merge(void* qkv, void* q, void* k, void* v, const float* cos_t,
                           const float* sin_t, int B, int T, int n_heads, int head_dim, int merge,
                           cudaStream_t stream);
// SwiGLU backward: h13[rows, 2d] = [gate | up], dact[rows, d] -> dh13[rows, 2d]
int tb200_swiglu_bwd(const void* h13, const void* dact, void* dh13, long long rows, int d,
                     cudaStream_t stream);

// K1 arrival chain and K2 send-side pack (element types moved as raw bytes).
int tb200_k1_arrival(const void* rx, const long long* rslot, const void* rgate, void* send_buf,
                     void* gate_pairs, long long* r_idx, long long* slot_idx, long long* i_send,
                     int* scratch, int R, int quota, int epr, int rpn, int row_bytes,
                     int gate_bytes, int* status, cudaStream_t stream);
size_t tb200_k1_scratch_ints(int R, int quota, int rpn);
int tb200_k2_pack(const void* hidden, const long long* expert_idx, const void* gates,
                  void* payload, long long* mask, void* gate_rows, long long* u_src,
                  long long* node_counts, int* scratch, int T, int k, int groups_m, int slots,
                  int n_nodes, int row_bytes, int gate_bytes, int* status, cudaStream_t stream);
size_t tb200_k2_scratch_ints(int T, int k, int groups_m, int n_nodes);

// ---- symm.cu -----------------------------------------------------------------------------------
struct Tb200Arena;
// cap > 0: capacity per expert (rows accepted in canonical order: source rank, then token);
// my_prefix[E] receives the rows of lower source ranks per expert, which the push kernels need
// to decide, without any further exchange, which of their picks fall beyond the capacity.
int tb200_ep_plan(const struct Tb200Arena* a, int* chunk_hist, int* chunka_hist, int* my_base,
                  int* seg_start, int* seg_count, int* rows_a, int* my_prefix, int epoch,
                  int seg_align, int cap, int* status, cudaStream_t stream);
// The push kernels cover the picks of LOCAL experts [le_lo, le_hi) (0 .. epr = all) and raise the
// owners' arrival flags to `flag_value` when their rows have landed; a step that sends in several
// launches passes growing values, and each owner GEMM waits for the value of its expert range.
int tb200_ep_push(const struct Tb200Arena* a, const void* x, const int* es, const int* rank_local,
                  const int* chunk_base, const int* my_base, int* pos_out, const float* gs,
                  float* dgs, long long off_dst, long long off_dot, int T, int flag_kind,
                  int flag_value, int le_lo, int le_hi, int* done_counter, int* status,
                  long long off_rowmap, int ret_slots, int dot_local, const int* my_prefix,
                  int cap, cudaStream_t stream);
int tb200_signal(const struct Tb200Arena* a, int kind, int first, int n, int stride, int idx,
                 int epoch, int wait_kind, int wait_first, int wait_n, int wait_value, int* status,
                 cudaStream_t stream);
int tb200_ep_pull_combine(const struct Tb200Arena* a, const int* pos, const int* es,
                          const float* gs, void* y, long long off_src, int T, int group_size,
                          int wait_kind, int epoch, int* status, int local_slots,
                          cudaStream_t stream);
int tb200_hopa_rank(const struct Tb200Arena* a, const int* es, int* ranka_local, int* chunka_hist,
                    int T, cudaStream_t stream);
int tb200_hopa_push(const struct Tb200Arena* a, const void* x, const int* es, const float* gs,
                    const int* rank_local, const int* chunk_base, const int* my_base,
                    const int* ranka_local, const int* chunka_base, int* pos_out, int* rowa,
                    long long off_rows, int with_header, int T, int flag_kind, int epoch,
                    int* done_counter, int* status, const int* my_prefix, int cap,
                    cudaStream_t stream);
int tb200_arrival_push(const struct Tb200Arena* a, const int* rows_a, long long off_rows,
                       long long off_dst, long long off_dot, int scale_gate, int want_dgate,
                       int wait_kind, int data_kind, int dg_kind, int epoch, int flag_value,
                       int le_lo, int le_hi, int* done_counter, int* status, long long off_rowmap,
                       int dot_local, cudaStream_t stream);
int tb200_arrival_combine(const struct Tb200Arena* a, const int* rows_a, long long off_src,
                          long long off_red, int use_gate, int wait_kind, int red_kind, int epoch,
                          int* done_counter, int* status, int push_back, int local_slots,
                          cudaStream_t stream);
int tb200_origin_combine(const struct Tb200Arena* a, const int* es, const int* rowa, void* y,
                         long long off_red, int T, int wait_kind, int epoch, int* status,
                         int local_rows, cudaStream_t stream);
int tb200_origin_pull_dgate(const struct Tb200Arena* a, const int* es, const int* rowa, float* dgs,
                            int T, int wait_kind, int epoch, int* status, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
