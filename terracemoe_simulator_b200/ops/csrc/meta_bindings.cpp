// Shape-only (Meta) implementations of the compute and transport ops: every op that returns a
// tensor says here what it returns (sizes, dtypes, device) without touching data, so that
// fake-tensor tracing, torch.export and shape inference can walk through a model that uses the
// native kernels.  In-place ops return nothing and therefore need no entry beyond an empty body.
//
// The reference registers a Meta kernel beside each of its device kernels
// (terrace/ops/csrc/terrace_ops.cpp:209-245, terrace_k2_pack.cpp:185-197); the three ops it
// shares with this library (passthrough, k1_arrival, k2_pack) have theirs in bindings.cpp.
#include <ATen/ATen.h>
#include <torch/library.h>

#include <tuple>

#include "meta.h"
#include "symm_layout.h"

namespace {

using at::Tensor;
using OptTensor = c10::optional<Tensor>;

Tensor like(const Tensor& t, at::IntArrayRef sizes, at::ScalarType dtype) {
  return at::empty(sizes, t.options().dtype(dtype));
}
Tensor none_like(const Tensor& t) { return at::empty({0}, t.options()); }

std::tuple<Tensor, Tensor> rmsnorm_fwd(const Tensor& x, const Tensor&, double) {
  auto lead = x.sizes().vec();
  lead.pop_back();
  return {at::empty_like(x), like(x, lead, at::kFloat)};
}

std::tuple<Tensor, Tensor> rmsnorm_bwd(const Tensor& x, const Tensor& w, const Tensor&,
                                       const Tensor&) {
  // per-block partial sums of the weight gradient; the wrapper reduces over dim 0, so only the
  // second extent matters to callers (the first is the block count of a 148-SM device)
  return {at::empty_like(x), like(x, {4 * 148, w.numel()}, at::kFloat)};
}

std::tuple<Tensor, Tensor, Tensor, Tensor, Tensor> route_out(const Tensor& ref, int64_t T,
                                                             int64_t E, int64_t k, int64_t M) {
  return {like(ref, {T, k}, at::kLong), like(ref, {T, k}, at::kFloat), like(ref, {T, M}, at::kLong),
          like(ref, {E}, at::kFloat), like(ref, {T, k}, at::kFloat)};
}

std::tuple<Tensor, Tensor, Tensor, Tensor, Tensor> route_select(const Tensor& logits,
                                                                const Tensor&, int64_t,
                                                                int64_t top_k, int64_t top_groups,
                                                                int64_t) {
  return route_out(logits, logits.size(0), logits.size(1), top_k, top_groups);
}

std::tuple<Tensor, Tensor, Tensor, Tensor, Tensor> route_fused(const Tensor& hidden,
                                                               const Tensor& weight, const Tensor&,
                                                               int64_t, int64_t top_k,
                                                               int64_t top_groups, int64_t) {
  return route_out(hidden, hidden.size(0), weight.size(0), top_k, top_groups);
}

Tensor route_select_bwd(const Tensor&, const Tensor& gates, const Tensor&, const Tensor& idx,
                        int64_t E) {
  return like(gates, {idx.size(0), E}, at::kFloat);
}

std::tuple<Tensor, Tensor, Tensor, Tensor, Tensor, Tensor> moe_plan(const Tensor& expert_idx,
                                                                    const OptTensor&, int64_t E,
                                                                    int64_t) {
  const int64_t T = expert_idx.size(0), k = expert_idx.size(1);
  auto i = [&](at::IntArrayRef s) { return like(expert_idx, s, at::kInt); };
  return {i({T, k}), like(expert_idx, {T, k}, at::kFloat), i({T, k}), i({T, k}), i({E}), i({E})};
}

Tensor moe_scatter_rows(const Tensor& x, const Tensor&, int64_t rows_out) {
  return like(x, {rows_out, x.size(1)}, x.scalar_type());
}

Tensor moe_combine(const Tensor& out, const Tensor& pos, const Tensor&, const OptTensor&,
                   int64_t) {
  return like(out, {pos.size(0), out.size(1)}, out.scalar_type());
}

std::tuple<Tensor, Tensor> moe_combine_bwd(const Tensor& dy, const Tensor& out, const Tensor& pos,
                                           const OptTensor&, bool need_dgs) {
  return {at::empty_like(out), need_dgs ? like(dy, pos.sizes(), at::kFloat)
                                        : like(dy, {0}, at::kFloat)};
}

Tensor swiglu_bwd(const Tensor& h13, const Tensor&) { return at::empty_like(h13); }

int64_t gemm_n(const Tensor& B, int64_t mode, int64_t epilogue) {
  const int64_t n = mode == 0 ? B.size(2) : B.size(1);
  return epilogue == 1 ? n / 2 : n;
}

std::tuple<Tensor, Tensor> grouped_gemm(const Tensor& A, const Tensor& B, const Tensor&,
                                        const Tensor&, int64_t mode, int64_t epilogue,
                                        bool save_pre, int64_t, int64_t) {
  const int64_t N = gemm_n(B, mode, epilogue);
  Tensor C = like(A, {A.size(0), N}, A.scalar_type());
  return {C, (epilogue == 1 && save_pre) ? like(A, {A.size(0), 2 * N}, A.scalar_type())
                                         : none_like(A)};
}

Tensor grouped_wgrad(const Tensor& X, const Tensor& dY, const Tensor& seg_start, const Tensor&,
                     int64_t, int64_t) {
  return like(X, {seg_start.numel(), X.size(1), dY.size(1)}, X.scalar_type());
}

void grouped_wgrad_out(const Tensor&, const Tensor&, Tensor, int64_t, const Tensor&, const Tensor&,
                       int64_t, int64_t) {}

void zero_pad_rows(Tensor, const Tensor&, const Tensor&, int64_t) {}

std::tuple<Tensor, Tensor, Tensor> rope_split(const Tensor& qkv, const Tensor&, const Tensor&,
                                              int64_t n_heads) {
  const int64_t hd = qkv.size(2) / (3 * n_heads);
  auto one = [&]() { return like(qkv, {qkv.size(0), n_heads, qkv.size(1), hd}, qkv.scalar_type()); };
  return {one(), one(), one()};
}

Tensor rope_merge(const Tensor& dq, const Tensor&, const Tensor&, const Tensor&, const Tensor&) {
  return like(dq, {dq.size(0), dq.size(2), 3 * dq.size(1) * dq.size(3)}, dq.scalar_type());
}

std::tuple<Tensor, Tensor> attn_fwd(const Tensor& q, const Tensor&, const Tensor&, bool, double) {
  auto lead = q.sizes().vec();
  lead.pop_back();
  return {at::empty_like(q), like(q, lead, at::kFloat)};
}

std::tuple<Tensor, Tensor, Tensor> attn_bwd(const Tensor& q, const Tensor&, const Tensor&,
                                            const Tensor&, const Tensor&, const Tensor&, bool,
                                            double) {
  return {at::empty_like(q), at::empty_like(q), at::empty_like(q)};
}

// ---- transport ops: geometry comes from the arena descriptor (a CPU byte blob) ----------------
const Tb200Arena* arena_of(const Tensor& blob) {
  TORCH_CHECK(blob.device().is_cpu() && blob.numel() == static_cast<int64_t>(sizeof(Tb200Arena)),
              "arena descriptor must come from symm_make_arena");
  return reinterpret_cast<const Tb200Arena*>(blob.data_ptr<uint8_t>());
}

std::tuple<Tensor, Tensor, Tensor, Tensor, Tensor> ep_plan_pass1(const Tensor& expert_idx,
                                                                 const Tensor& gates, int64_t E) {
  const int64_t T = expert_idx.size(0), k = expert_idx.size(1);
  auto i = [&](at::IntArrayRef s) { return like(expert_idx, s, at::kInt); };
  return {i({T, k}), at::empty_like(gates), i({T, k}), i({T, k}), i({TB200_PLAN_CHUNKS, E})};
}

std::tuple<Tensor, Tensor, Tensor, Tensor, Tensor> ep_plan(const Tensor& arena, Tensor chunk_hist,
                                                           const OptTensor&, int64_t, int64_t,
                                                           int64_t) {
  const Tb200Arena* a = arena_of(arena);
  auto i = [&](at::IntArrayRef s) { return like(chunk_hist, s, at::kInt); };
  return {i({a->n_experts}), i({a->epr}), i({a->epr}), i({a->world, a->n_nodes}),
          i({a->n_experts})};
}

void ep_push(const Tensor&, const Tensor&, const Tensor&, const Tensor&, const Tensor&,
             const Tensor&, const OptTensor&, Tensor, const OptTensor&, int64_t, int64_t, bool,
             int64_t, int64_t, int64_t, int64_t, Tensor, int64_t, int64_t, const OptTensor&,
             int64_t) {}

void ep_signal(const Tensor&, int64_t, int64_t, int64_t, int64_t, int64_t, int64_t, int64_t,
               int64_t, int64_t, int64_t, const Tensor&) {}

Tensor ep_pull_combine(const Tensor& arena, const Tensor& pos, const Tensor&, const OptTensor&,
                       int64_t, int64_t, int64_t, int64_t, int64_t) {
  return like(pos, {pos.size(0), arena_of(arena)->hidden}, at::kBFloat16);
}

void grouped_gemm_scatter(const Tensor&, const Tensor&, const Tensor&, const Tensor&, int64_t,
                          const Tensor&, const Tensor&, int64_t) {}

std::tuple<Tensor, Tensor> hopa_rank(const Tensor& arena, const Tensor& es) {
  const Tb200Arena* a = arena_of(arena);
  return {like(es, {es.size(0), a->groups_m}, at::kInt),
          like(es, {TB200_PLAN_CHUNKS, a->n_nodes}, at::kInt)};
}

std::tuple<Tensor, Tensor> hopa_push(const Tensor& arena, const Tensor& x, const Tensor& es,
                                     const Tensor&, const Tensor&, const Tensor&, const Tensor&,
                                     const Tensor&, const Tensor&, const OptTensor& rowa_in,
                                     int64_t, bool with_header, int64_t, int64_t, Tensor,
                                     const OptTensor&, int64_t) {
  const Tb200Arena* a = arena_of(arena);
  const int64_t T = x.size(0);
  if (!with_header) return {like(es, {0}, at::kInt), *rowa_in};
  return {like(es, {T, a->top_k}, at::kInt), like(es, {T, a->groups_m}, at::kInt)};
}

void arrival_push(const Tensor&, const Tensor&, int64_t, int64_t, int64_t, bool, bool, bool,
                  int64_t, int64_t, int64_t, int64_t, int64_t, int64_t, int64_t, Tensor, int64_t) {}

void arrival_combine(const Tensor&, const Tensor&, int64_t, int64_t, bool, int64_t, int64_t,
                     int64_t, Tensor, bool, bool) {}

Tensor origin_combine(const Tensor& arena, const Tensor& es, const Tensor&, int64_t, int64_t,
                      int64_t, bool) {
  return like(es, {es.size(0), arena_of(arena)->hidden}, at::kBFloat16);
}

Tensor origin_pull_dgate(const Tensor& arena, const Tensor& es, const Tensor&, int64_t, int64_t) {
  return like(es, {es.size(0), arena_of(arena)->top_k}, at::kFloat);
}

void grouped_gemm_ex(const Tensor&, const Tensor&, Tensor, const OptTensor&, const Tensor&,
                     const Tensor&, int64_t, int64_t, const OptTensor&, int64_t, int64_t, int64_t,
                     int64_t, int64_t) {}

}  // namespace

#define TB_META(name) m.impl(#name, &name)

void terrace_b200_register_meta(torch::Library& m) {
  TB_META(rmsnorm_fwd);
  TB_META(rmsnorm_bwd);
  TB_META(route_select);
  TB_META(route_fused);
  TB_META(route_select_bwd);
  TB_META(moe_plan);
  TB_META(moe_scatter_rows);
  TB_META(moe_combine);
  TB_META(moe_combine_bwd);
  TB_META(swiglu_bwd);
  TB_META(grouped_gemm);
  TB_META(grouped_wgrad);
  TB_META(grouped_wgrad_out);
  TB_META(zero_pad_rows);
  TB_META(rope_split);
  TB_META(rope_merge);
  TB_META(attn_fwd);
  TB_META(attn_bwd);
  TB_META(ep_plan_pass1);
  TB_META(ep_plan);
  TB_META(ep_push);
  TB_META(ep_signal);
  TB_META(ep_pull_combine);
  TB_META(grouped_gemm_scatter);
  TB_META(hopa_rank);
  TB_META(hopa_push);
  TB_META(arrival_push);
  TB_META(arrival_combine);
  TB_META(origin_combine);
  TB_META(origin_pull_dgate);
  TB_META(grouped_gemm_ex);
}
