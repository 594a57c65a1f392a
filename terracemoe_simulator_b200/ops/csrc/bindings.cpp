// torch bindings: TORCH_LIBRARY(terrace) with CUDA and Meta implementations.
//
// Same op schemas as the reference's library for the three ops it defines
// (terrace/ops/csrc/terrace_ops.cpp:228-233, terrace_k2_pack.cpp:207-212):
//   terrace::passthrough(Tensor x) -> Tensor
//   terrace::k1_arrival(Tensor rx, Tensor rslot, Tensor rgate, int quota, int epr, int rpn,
//                       int my_local) -> (Tensor, Tensor, Tensor, Tensor, Tensor)
//   terrace::k2_pack(Tensor hidden, Tensor expert_idx, Tensor gates, int world, int n_experts,
//                    int rpn, int groups_m) -> (Tensor, Tensor, Tensor, Tensor, Tensor)
// plus the compute ops of the MoE layer (norm, route, plan, scatter, combine, grouped GEMMs).
// Host-side validation fails loudly (TORCH_CHECK) before anything is launched; device-side
// containment problems are reported through a per-device status word (terrace::take_status).
#include <ATen/ATen.h>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/library.h>

#include <mutex>
#include <tuple>
#include <vector>

#include "launch.h"
#include "meta.h"
#include "symm.h"

namespace {

using at::Tensor;

long long* i64(const Tensor& t) { return reinterpret_cast<long long*>(t.data_ptr<int64_t>()); }

cudaStream_t cur_stream() { return at::cuda::getCurrentCUDAStream().stream(); }

void check_rc(int rc, const char* what) {
  TORCH_CHECK(rc == TB200_OK, what, " failed with terrace_b200 error code ", rc);
}

// One int32 status word per device; kernels CAS their first problem code into it.
Tensor& status_word(int device) {
  static std::mutex mu;
  static std::vector<Tensor> words(64);
  std::lock_guard<std::mutex> lock(mu);
  TORCH_CHECK(device >= 0 && device < 64, "device index out of range");
  if (!words[device].defined()) {
    words[device] = at::zeros({1}, at::TensorOptions().dtype(at::kInt).device(at::kCUDA, device));
  }
  return words[device];
}
int* status_ptr(const Tensor& like) { return status_word(like.get_device()).data_ptr<int>(); }

int64_t take_status(int64_t device) {
  Tensor& w = status_word(static_cast<int>(device));
  const int v = w.item<int>();
  if (v != 0) w.zero_();
  return v;
}

#define CHECK_CUDA_CONTIG(t) \
  TORCH_CHECK((t).is_cuda() && (t).is_contiguous(), #t " must be a contiguous CUDA tensor")

// ---------------------------------------------------------------------------------------------
Tensor passthrough_cuda(const Tensor& x) {
  c10::cuda::CUDAGuard guard(x.device());
  Tensor src = x.contiguous();
  Tensor out = at::empty_like(src);
  check_rc(tb200_passthrough(src.data_ptr(), out.data_ptr(), src.nbytes(), cur_stream()),
           "passthrough");
  return out;
}
Tensor passthrough_meta(const Tensor& x) { return at::empty_like(x); }

// ---------------------------------------------------------------------------------------------
using Tup5 = std::tuple<Tensor, Tensor, Tensor, Tensor, Tensor>;

void k1_checks(const Tensor& rx, const Tensor& rslot, const Tensor& rgate, int64_t quota,
               int64_t epr, int64_t rpn, int64_t my_local) {
  TORCH_CHECK(rx.dim() == 2 && rslot.dim() == 2 && rgate.dim() == 2, "k1_arrival: 2-D inputs");
  TORCH_CHECK(rslot.scalar_type() == at::kLong, "k1_arrival: rslot must be int64");
  TORCH_CHECK(rgate.scalar_type() == rx.scalar_type(),
              "k1_arrival: rgate dtype must equal rx dtype");
  TORCH_CHECK(rslot.size(0) == rx.size(0) && rgate.sizes() == rslot.sizes(),
              "k1_arrival: rslot/rgate must be [R, quota]");
  TORCH_CHECK(rslot.size(1) == quota, "k1_arrival: rslot has ", rslot.size(1),
              " columns but quota is ", quota);
  TORCH_CHECK(epr >= 1 && rpn >= 1 && rpn <= 1024, "k1_arrival: bad epr/rpn");
  TORCH_CHECK(my_local >= 0 && my_local < rpn, "k1_arrival: my_local outside [0, rpn)");
}

Tup5 k1_arrival_cuda(const Tensor& rx_, const Tensor& rslot_, const Tensor& rgate_, int64_t quota,
                     int64_t epr, int64_t rpn, int64_t my_local) {
  k1_checks(rx_, rslot_, rgate_, quota, epr, rpn, my_local);
  c10::cuda::CUDAGuard guard(rx_.device());
  Tensor rx = rx_.contiguous(), rslot = rslot_.contiguous(), rgate = rgate_.contiguous();
  const int64_t R = rx.size(0), H = rx.size(1), P = R * quota;
  auto lopt = rx.options().dtype(at::kLong);
  Tensor send_buf = at::empty({P, H}, rx.options());
  Tensor gate_pairs = at::empty({P}, rx.options());
  Tensor r_idx = at::zeros({P}, lopt), slot_idx = at::zeros({P}, lopt);
  Tensor i_send = at::zeros({rpn}, lopt);
  if (P == 0) return {send_buf, gate_pairs, r_idx, slot_idx, i_send};
  Tensor scratch = at::empty({static_cast<int64_t>(tb200_k1_scratch_ints(R, quota, rpn))},
                             rx.options().dtype(at::kInt));
  check_rc(tb200_k1_arrival(rx.data_ptr(), i64(rslot), rgate.data_ptr(),
                            send_buf.data_ptr(), gate_pairs.data_ptr(), i64(r_idx),
                            i64(slot_idx), i64(i_send),
                            scratch.data_ptr<int>(), R, quota, epr, rpn,
                            static_cast<int>(H * rx.element_size()),
                            static_cast<int>(rx.element_size()), status_ptr(rx), cur_stream()),
           "k1_arrival");
  return {send_buf, gate_pairs, r_idx, slot_idx, i_send};
}

Tup5 k1_arrival_meta(const Tensor& rx, const Tensor& rslot, const Tensor& rgate, int64_t quota,
                     int64_t epr, int64_t rpn, int64_t my_local) {
  const int64_t P = rx.size(0) * quota;
  auto lopt = rx.options().dtype(at::kLong);
  return {at::empty({P, rx.size(1)}, rx.options()), at::empty({P}, rx.options()),
          at::empty({P}, lopt), at::empty({P}, lopt), at::empty({rpn}, lopt)};
}

void k2_checks(const Tensor& hidden, const Tensor& expert_idx, const Tensor& gates, int64_t world,
               int64_t n_experts, int64_t rpn, int64_t groups_m) {
  TORCH_CHECK(hidden.dim() == 2 && expert_idx.dim() == 2 && gates.dim() == 2, "k2_pack: 2-D inputs");
  TORCH_CHECK(expert_idx.scalar_type() == at::kLong, "k2_pack: expert_idx must be int64");
  TORCH_CHECK(gates.scalar_type() == hidden.scalar_type(),
              "k2_pack: gates dtype must equal hidden dtype");
  TORCH_CHECK(hidden.size(0) == expert_idx.size(0) && gates.sizes() == expert_idx.sizes(),
              "k2_pack: geometry mismatch");
  TORCH_CHECK(world > 0 && rpn > 0 && groups_m > 0 && n_experts > 0, "k2_pack: bad scalars");
  TORCH_CHECK(world % rpn == 0 && n_experts % world == 0 && expert_idx.size(1) % groups_m == 0,
              "k2_pack: world/rpn/n_experts/k/groups_m do not divide");
  TORCH_CHECK(world / rpn <= 1024 && expert_idx.size(1) <= 32, "k2_pack: N_g <= 1024, k <= 32");
  TORCH_CHECK(n_experts < (1LL << 31) && expert_idx.numel() < (1LL << 31), "k2_pack: id range");
}

Tup5 k2_pack_cuda(const Tensor& hidden_, const Tensor& expert_idx_, const Tensor& gates_,
                  int64_t world, int64_t n_experts, int64_t rpn, int64_t groups_m) {
  k2_checks(hidden_, expert_idx_, gates_, world, n_experts, rpn, groups_m);
  c10::cuda::CUDAGuard guard(hidden_.device());
  Tensor hidden = hidden_.contiguous(), eidx = expert_idx_.contiguous(), gates = gates_.contiguous();
  const int64_t T = eidx.size(0), k = eidx.size(1), H = hidden.size(1);
  const int64_t q = k / groups_m, P = T * groups_m, n_nodes = world / rpn;
  const int64_t slots = (n_experts / world) * rpn;
  auto lopt = hidden.options().dtype(at::kLong);
  Tensor payload = at::empty({P, H}, hidden.options());
  Tensor mask = at::zeros({P, q}, lopt);
  Tensor gate_rows = at::zeros({P, q}, hidden.options());
  Tensor u_src = at::zeros({P}, lopt);
  Tensor node_counts = at::zeros({n_nodes}, lopt);
  if (P == 0) return {payload, mask, gate_rows, u_src, node_counts};
  Tensor scratch = at::empty(
      {static_cast<int64_t>(tb200_k2_scratch_ints(T, k, groups_m, n_nodes))},
      hidden.options().dtype(at::kInt));
  check_rc(tb200_k2_pack(hidden.data_ptr(), i64(eidx), gates.data_ptr(),
                         payload.data_ptr(), i64(mask), gate_rows.data_ptr(),
                         i64(u_src), i64(node_counts),
                         scratch.data_ptr<int>(), T, k, groups_m, slots, n_nodes,
                         static_cast<int>(H * hidden.element_size()),
                         static_cast<int>(hidden.element_size()), status_ptr(hidden), cur_stream()),
           "k2_pack");
  return {payload, mask, gate_rows, u_src, node_counts};
}

Tup5 k2_pack_meta(const Tensor& hidden, const Tensor& expert_idx, const Tensor& gates,
                  int64_t world, int64_t n_experts, int64_t rpn, int64_t groups_m) {
  const int64_t T = expert_idx.size(0), k = expert_idx.size(1);
  const int64_t q = k / groups_m, P = T * groups_m;
  auto lopt = hidden.options().dtype(at::kLong);
  return {at::empty({P, hidden.size(1)}, hidden.options()), at::empty({P, q}, lopt),
          at::empty({P, q}, hidden.options()), at::empty({P}, lopt),
          at::empty({world / rpn}, lopt)};
}

// ---------------------------------------------------------------------------------------------
std::tuple<Tensor, Tensor> rmsnorm_fwd(const Tensor& x, const Tensor& w, double eps) {
  CHECK_CUDA_CONTIG(x);
  CHECK_CUDA_CONTIG(w);
  TORCH_CHECK(x.scalar_type() == w.scalar_type(), "rmsnorm: x and w dtypes differ");
  TORCH_CHECK(x.scalar_type() == at::kBFloat16 || x.scalar_type() == at::kFloat,
              "rmsnorm: bf16 or fp32");
  c10::cuda::CUDAGuard guard(x.device());
  const int64_t dim = x.size(-1), rows = x.numel() / dim;
  TORCH_CHECK(w.numel() == dim, "rmsnorm: weight length");
  Tensor y = at::empty_like(x);
  Tensor rstd = at::empty({rows}, x.options().dtype(at::kFloat));
  check_rc(tb200_rmsnorm_fwd(x.data_ptr(), w.data_ptr(), y.data_ptr(), rstd.data_ptr<float>(), rows,
                             static_cast<int>(dim), static_cast<float>(eps),
                             x.scalar_type() == at::kBFloat16, cur_stream()),
           "rmsnorm_fwd");
  return {y, rstd};
}

std::tuple<Tensor, Tensor> rmsnorm_bwd(const Tensor& x, const Tensor& w, const Tensor& dy,
                                       const Tensor& rstd) {
  CHECK_CUDA_CONTIG(x);
  CHECK_CUDA_CONTIG(dy);
  CHECK_CUDA_CONTIG(w);
  CHECK_CUDA_CONTIG(rstd);
  TORCH_CHECK(dy.sizes() == x.sizes() && dy.scalar_type() == x.scalar_type() &&
                  w.scalar_type() == x.scalar_type() && w.numel() == x.size(-1) &&
                  rstd.scalar_type() == at::kFloat && rstd.numel() * x.size(-1) == x.numel(),
              "rmsnorm_bwd: inconsistent shapes or dtypes");
  c10::cuda::CUDAGuard guard(x.device());
  const int64_t dim = x.size(-1), rows = x.numel() / dim;
  Tensor dx = at::empty_like(x);
  // one partial weight-gradient row per block, four blocks per SM
  const int n_partial = 4 * at::cuda::getCurrentDeviceProperties()->multiProcessorCount;
  Tensor part = at::empty({n_partial, dim}, x.options().dtype(at::kFloat));
  check_rc(tb200_rmsnorm_bwd(x.data_ptr(), w.data_ptr(), dy.data_ptr(), rstd.data_ptr<float>(),
                             dx.data_ptr(), part.data_ptr<float>(), n_partial, rows,
                             static_cast<int>(dim), x.scalar_type() == at::kBFloat16, cur_stream()),
           "rmsnorm_bwd");
  return {dx, part};
}

// ---------------------------------------------------------------------------------------------
Tup5 route_select(const Tensor& logits, const Tensor& bias, int64_t n_groups, int64_t top_k,
                  int64_t top_groups, int64_t pool) {
  CHECK_CUDA_CONTIG(logits);
  CHECK_CUDA_CONTIG(bias);
  TORCH_CHECK(logits.scalar_type() == at::kFloat && bias.scalar_type() == at::kFloat,
              "route_select: fp32 logits and bias");
  c10::cuda::CUDAGuard guard(logits.device());
  const int64_t T = logits.size(0), E = logits.size(1);
  auto lopt = logits.options().dtype(at::kLong);
  Tensor idx = at::empty({T, top_k}, lopt);
  Tensor gates = at::empty({T, top_k}, logits.options());
  Tensor aff = at::empty({T, top_k}, logits.options());
  Tensor gidx = at::empty({T, top_groups}, lopt);
  Tensor load = at::zeros({E}, logits.options());
  check_rc(tb200_route_select(logits.data_ptr<float>(), bias.data_ptr<float>(),
                              i64(idx), gates.data_ptr<float>(),
                              i64(gidx), load.data_ptr<float>(),
                              aff.data_ptr<float>(), T, E, n_groups, top_k, top_groups, pool,
                              cur_stream()),
           "route_select");
  return {idx, gates, gidx, load, aff};
}

// Router GEMM + T-Route selection in one launch: hidden [T, H] bf16, weight [E, H] bf16.
std::tuple<Tensor, Tensor, Tensor, Tensor, Tensor> route_fused(
    const Tensor& hidden, const Tensor& weight, const Tensor& bias, int64_t n_groups,
    int64_t top_k, int64_t top_groups, int64_t pool) {
  CHECK_CUDA_CONTIG(hidden);
  CHECK_CUDA_CONTIG(weight);
  CHECK_CUDA_CONTIG(bias);
  TORCH_CHECK(hidden.dim() == 2 && weight.dim() == 2 && hidden.size(1) == weight.size(1) &&
                  hidden.scalar_type() == at::kBFloat16 && weight.scalar_type() == at::kBFloat16,
              "route_fused: bf16 hidden [T, H] and weight [E, H]");
  TORCH_CHECK(bias.scalar_type() == at::kFloat && bias.numel() == weight.size(0),
              "route_fused: fp32 bias [E]");
  const int T = static_cast<int>(hidden.size(0)), H = static_cast<int>(hidden.size(1));
  const int E = static_cast<int>(weight.size(0));
  TORCH_CHECK(tb200_route_fused_supported(E, H, n_groups, top_k, top_groups),
              "route_fused: unsupported router geometry (E <= 128 and E % 16 == 0 required)");
  c10::cuda::CUDAGuard guard(hidden.device());
  auto fopt = hidden.options().dtype(at::kFloat);
  auto lopt = hidden.options().dtype(at::kLong);
  Tensor idx = at::empty({T, top_k}, lopt), gidx = at::empty({T, top_groups}, lopt);
  Tensor gates = at::empty({T, top_k}, fopt), aff = at::empty({T, top_k}, fopt);
  Tensor load = at::zeros({E}, fopt);
  check_rc(tb200_route_fused(hidden.data_ptr(), weight.data_ptr(), bias.data_ptr<float>(),
                             i64(idx), gates.data_ptr<float>(), i64(gidx), load.data_ptr<float>(),
                             aff.data_ptr<float>(), T, E, H, n_groups, top_k, top_groups, pool,
                             status_ptr(hidden), cur_stream()),
           "route_fused");
  return {idx, gates, gidx, load, aff};
}

bool route_fused_supported(int64_t E, int64_t H, int64_t n_groups, int64_t top_k,
                           int64_t top_groups) {
  return tb200_route_fused_supported(E, H, n_groups, top_k, top_groups) != 0;
}

Tensor route_select_bwd(const Tensor& dgates, const Tensor& gates, const Tensor& aff,
                        const Tensor& idx, int64_t E) {
  CHECK_CUDA_CONTIG(dgates);
  CHECK_CUDA_CONTIG(gates);
  CHECK_CUDA_CONTIG(aff);
  CHECK_CUDA_CONTIG(idx);
  TORCH_CHECK(idx.dim() == 2 && idx.scalar_type() == at::kLong && gates.sizes() == idx.sizes() &&
                  aff.sizes() == idx.sizes() && dgates.sizes() == idx.sizes() &&
                  gates.scalar_type() == at::kFloat && aff.scalar_type() == at::kFloat,
              "route_select_bwd: inconsistent shapes or dtypes");
  c10::cuda::CUDAGuard guard(dgates.device());
  const int64_t T = idx.size(0), k = idx.size(1);
  Tensor dlogits = at::zeros({T, E}, gates.options());
  Tensor dg = dgates.to(at::kFloat).contiguous();
  check_rc(tb200_route_select_bwd(dg.data_ptr<float>(), gates.data_ptr<float>(),
                                  aff.data_ptr<float>(), i64(idx),
                                  dlogits.data_ptr<float>(), T, E, k, cur_stream()),
           "route_select_bwd");
  return dlogits;
}

// ---------------------------------------------------------------------------------------------
std::tuple<Tensor, Tensor, Tensor, Tensor, Tensor, Tensor> moe_plan(
    const Tensor& expert_idx, const c10::optional<Tensor>& gates, int64_t E, int64_t seg_align) {
  CHECK_CUDA_CONTIG(expert_idx);
  TORCH_CHECK(expert_idx.scalar_type() == at::kLong && expert_idx.dim() == 2, "moe_plan: idx");
  c10::cuda::CUDAGuard guard(expert_idx.device());
  const int64_t T = expert_idx.size(0), k = expert_idx.size(1);
  auto iopt = expert_idx.options().dtype(at::kInt);
  auto fopt = expert_idx.options().dtype(at::kFloat);
  Tensor es = at::empty({T, k}, iopt), cols = at::empty({T, k}, iopt), pos = at::empty({T, k}, iopt);
  Tensor gs = at::empty({T, k}, fopt);
  Tensor seg_start = at::empty({E}, iopt), seg_count = at::empty({E}, iopt);
  Tensor scratch = at::empty({static_cast<int64_t>(tb200_plan_scratch_ints(T, k, E))}, iopt);
  const float* gp = nullptr;
  Tensor g32;
  if (gates.has_value()) {
    g32 = gates->to(at::kFloat).contiguous();
    gp = g32.data_ptr<float>();
  }
  check_rc(tb200_moe_plan(i64(expert_idx), gp, es.data_ptr<int>(),
                          gs.data_ptr<float>(), cols.data_ptr<int>(), pos.data_ptr<int>(),
                          seg_start.data_ptr<int>(), seg_count.data_ptr<int>(),
                          scratch.data_ptr<int>(), T, k, E, seg_align, cur_stream()),
           "moe_plan");
  return {es, gs, cols, pos, seg_start, seg_count};
}

Tensor moe_scatter_rows(const Tensor& x, const Tensor& pos, int64_t rows_out) {
  CHECK_CUDA_CONTIG(x);
  CHECK_CUDA_CONTIG(pos);
  TORCH_CHECK(x.scalar_type() == at::kBFloat16 && x.dim() == 2, "moe_scatter_rows: bf16 [T, H]");
  TORCH_CHECK(pos.dim() == 2 && pos.scalar_type() == at::kInt && pos.size(0) == x.size(0),
              "moe_scatter_rows: pos must be int32 [T, k]");
  c10::cuda::CUDAGuard guard(x.device());
  const int64_t T = pos.size(0), k = pos.size(1);
  Tensor xs = at::empty({rows_out, x.size(1)}, x.options());
  check_rc(tb200_moe_scatter_rows(x.data_ptr(), xs.data_ptr(), pos.data_ptr<int>(), T, k,
                                  x.size(1), rows_out, status_ptr(x), cur_stream()),
           "moe_scatter_rows");
  return xs;
}

Tensor moe_combine(const Tensor& out, const Tensor& pos, const Tensor& es,
                   const c10::optional<Tensor>& gs, int64_t group_size) {
  CHECK_CUDA_CONTIG(out);
  CHECK_CUDA_CONTIG(pos);
  CHECK_CUDA_CONTIG(es);
  TORCH_CHECK(out.scalar_type() == at::kBFloat16 && out.dim() == 2, "moe_combine: bf16 rows");
  TORCH_CHECK(pos.dim() == 2 && pos.scalar_type() == at::kInt && es.sizes() == pos.sizes() &&
                  es.scalar_type() == at::kInt,
              "moe_combine: pos and es must be int32 [T, k]");
  TORCH_CHECK(!gs.has_value() || (gs->sizes() == pos.sizes() && gs->scalar_type() == at::kFloat &&
                                  gs->is_contiguous()),
              "moe_combine: gs must be fp32 [T, k]");
  c10::cuda::CUDAGuard guard(out.device());
  const int64_t T = pos.size(0), k = pos.size(1);
  Tensor y = at::empty({T, out.size(1)}, out.options());
  check_rc(tb200_moe_combine(out.data_ptr(), pos.data_ptr<int>(), es.data_ptr<int>(),
                             gs.has_value() ? gs->data_ptr<float>() : nullptr, y.data_ptr(), T, k,
                             out.size(1), group_size, out.size(0), status_ptr(out), cur_stream()),
           "moe_combine");
  return y;
}

std::tuple<Tensor, Tensor> moe_combine_bwd(const Tensor& dy, const Tensor& out, const Tensor& pos,
                                           const c10::optional<Tensor>& gs, bool need_dgs) {
  CHECK_CUDA_CONTIG(dy);
  CHECK_CUDA_CONTIG(out);
  CHECK_CUDA_CONTIG(pos);
  TORCH_CHECK(dy.scalar_type() == at::kBFloat16 && out.scalar_type() == at::kBFloat16 &&
                  dy.dim() == 2 && out.dim() == 2 && dy.size(1) == out.size(1),
              "moe_combine_bwd: bf16 dy [T, H] and out [rows, H]");
  TORCH_CHECK(pos.dim() == 2 && pos.scalar_type() == at::kInt && pos.size(0) == dy.size(0),
              "moe_combine_bwd: pos must be int32 [T, k]");
  TORCH_CHECK(!gs.has_value() || (gs->sizes() == pos.sizes() && gs->scalar_type() == at::kFloat &&
                                  gs->is_contiguous()),
              "moe_combine_bwd: gs must be fp32 [T, k]");
  c10::cuda::CUDAGuard guard(dy.device());
  const int64_t T = pos.size(0), k = pos.size(1);
  Tensor dout = at::empty_like(out);      // every row of a valid pick is written
  Tensor dgs = need_dgs ? at::empty({T, k}, dy.options().dtype(at::kFloat)) : Tensor();
  check_rc(tb200_moe_combine_bwd(dy.data_ptr(), out.data_ptr(), pos.data_ptr<int>(),
                                 gs.has_value() ? gs->data_ptr<float>() : nullptr, dout.data_ptr(),
                                 need_dgs ? dgs.data_ptr<float>() : nullptr, T, k, dy.size(1),
                                 out.size(0), status_ptr(dy), cur_stream()),
           "moe_combine_bwd");
  return {dout, need_dgs ? dgs : at::empty({0}, dy.options().dtype(at::kFloat))};
}

Tensor swiglu_bwd(const Tensor& h13, const Tensor& dact) {
  CHECK_CUDA_CONTIG(h13);
  CHECK_CUDA_CONTIG(dact);
  TORCH_CHECK(h13.dim() == 2 && dact.dim() == 2 && h13.size(0) == dact.size(0) &&
                  h13.size(1) == 2 * dact.size(1),
              "swiglu_bwd: h13 must be [rows, 2d] and dact [rows, d]");
  TORCH_CHECK(h13.scalar_type() == at::kBFloat16 && dact.scalar_type() == at::kBFloat16,
              "swiglu_bwd: bf16 tensors");
  c10::cuda::CUDAGuard guard(h13.device());
  Tensor dh = at::empty_like(h13);
  check_rc(tb200_swiglu_bwd(h13.data_ptr(), dact.data_ptr(), dh.data_ptr(), dact.size(0),
                            dact.size(1), cur_stream()),
           "swiglu_bwd");
  return dh;
}

// qkv [B, T, 3 * nh * hd] bf16 -> (q, k, v) [B, nh, T, hd]; q and k rotated (interleaved RoPE)
std::tuple<Tensor, Tensor, Tensor> rope_split(const Tensor& qkv, const Tensor& cos_t,
                                              const Tensor& sin_t, int64_t n_heads) {
  CHECK_CUDA_CONTIG(qkv);
  CHECK_CUDA_CONTIG(cos_t);
  CHECK_CUDA_CONTIG(sin_t);
  TORCH_CHECK(qkv.dim() == 3 && qkv.scalar_type() == at::kBFloat16 && qkv.size(2) % (3 * n_heads) == 0,
              "rope_split: bf16 qkv [B, T, 3 * heads * head_dim]");
  const int64_t B = qkv.size(0), T = qkv.size(1), hd = qkv.size(2) / (3 * n_heads);
  TORCH_CHECK(hd % 8 == 0 && cos_t.scalar_type() == at::kFloat && sin_t.scalar_type() == at::kFloat &&
                  cos_t.numel() == T * hd / 2 && sin_t.numel() == T * hd / 2,
              "rope_split: head_dim % 8 == 0 and fp32 cos / sin tables [T, head_dim / 2]");
  c10::cuda::CUDAGuard guard(qkv.device());
  Tensor q = at::empty({B, n_heads, T, hd}, qkv.options());
  Tensor k = at::empty_like(q), v = at::empty_like(q);
  check_rc(tb200_rope_split_merge(qkv.data_ptr(), q.data_ptr(), k.data_ptr(), v.data_ptr(),
                                  cos_t.data_ptr<float>(), sin_t.data_ptr<float>(), B, T, n_heads,
                                  hd, 0, cur_stream()),
           "rope_split");
  return {q, k, v};
}

// the adjoint: (dq, dk, dv) [B, nh, T, hd] -> dqkv [B, T, 3 * nh * hd]
Tensor rope_merge(const Tensor& dq, const Tensor& dk, const Tensor& dv, const Tensor& cos_t,
                  const Tensor& sin_t) {
  CHECK_CUDA_CONTIG(dq);
  CHECK_CUDA_CONTIG(dk);
  CHECK_CUDA_CONTIG(dv);
  CHECK_CUDA_CONTIG(cos_t);
  CHECK_CUDA_CONTIG(sin_t);
  TORCH_CHECK(dq.dim() == 4 && dq.scalar_type() == at::kBFloat16 && dq.sizes() == dk.sizes() &&
                  dq.sizes() == dv.sizes() && dk.scalar_type() == at::kBFloat16 &&
                  dv.scalar_type() == at::kBFloat16,
              "rope_merge: three bf16 tensors [B, heads, T, head_dim]");
  const int64_t B = dq.size(0), nh = dq.size(1), T = dq.size(2), hd = dq.size(3);
  TORCH_CHECK(hd % 8 == 0 && cos_t.numel() == T * hd / 2 && sin_t.numel() == T * hd / 2,
              "rope_merge: fp32 cos / sin tables [T, head_dim / 2]");
  c10::cuda::CUDAGuard guard(dq.device());
  Tensor dqkv = at::empty({B, T, 3 * nh * hd}, dq.options());
  check_rc(tb200_rope_split_merge(dqkv.data_ptr(), dq.data_ptr(), dk.data_ptr(), dv.data_ptr(),
                                  cos_t.data_ptr<float>(), sin_t.data_ptr<float>(), B, T, nh, hd, 1,
                                  cur_stream()),
           "rope_merge");
  return dqkv;
}

void zero_pad_rows(Tensor buf, const Tensor& seg_start, const Tensor& seg_count, int64_t align) {
  TORCH_CHECK(buf.is_cuda() && buf.is_contiguous() && buf.dim() == 2, "zero_pad_rows: [rows, cols]");
  TORCH_CHECK(seg_start.scalar_type() == at::kInt && seg_count.scalar_type() == at::kInt &&
                  seg_start.numel() == seg_count.numel(),
              "zero_pad_rows: int32 segment tables");
  c10::cuda::CUDAGuard guard(buf.device());
  check_rc(tb200_zero_pad_rows(buf.data_ptr(), seg_start.data_ptr<int>(),
                               seg_count.data_ptr<int>(), seg_start.numel(), align,
                               static_cast<int>(buf.size(1) * buf.element_size()), buf.size(0),
                               cur_stream()),
           "zero_pad_rows");
}

// ---------------------------------------------------------------------------------------------
// grouped GEMMs.  mode 0: B[g] is [K, N(*2 for SwiGLU)];  mode 1: B[g] is [N, K].
std::tuple<Tensor, Tensor> grouped_gemm(const Tensor& A, const Tensor& B, const Tensor& seg_start,
                                        const Tensor& seg_count, int64_t mode, int64_t epilogue,
                                        bool save_pre, int64_t max_ctas, int64_t pad_align) {
  CHECK_CUDA_CONTIG(A);
  CHECK_CUDA_CONTIG(B);
  TORCH_CHECK(A.scalar_type() == at::kBFloat16 && B.scalar_type() == at::kBFloat16,
              "grouped_gemm: bf16 operands");
  TORCH_CHECK(A.dim() == 2 && B.dim() == 3, "grouped_gemm: A [rows, K], B [G, r, c]");
  TORCH_CHECK(seg_start.scalar_type() == at::kInt && seg_count.scalar_type() == at::kInt,
              "grouped_gemm: int32 segment tables");
  c10::cuda::CUDAGuard guard(A.device());
  const int64_t rows = A.size(0), K = A.size(1), G = B.size(0);
  const int64_t b_rows = B.size(1), b_cols = B.size(2);
  int64_t N;
  if (mode == 0) {
    TORCH_CHECK(b_rows == K, "grouped_gemm fwd: B rows must equal K");
    N = epilogue == 1 ? b_cols / 2 : b_cols;
  } else {
    TORCH_CHECK(b_cols == K, "grouped_gemm dgrad: B cols must equal K");
    N = epilogue == 1 ? b_rows / 2 : b_rows;
  }
  TORCH_CHECK(seg_start.numel() == G && seg_count.numel() == G, "grouped_gemm: segment tables");
  Tensor C = at::empty({rows, N}, A.options());
  Tensor C2 = (epilogue == 1 && save_pre) ? at::empty({rows, 2 * N}, A.options()) : Tensor();
  if (rows > 0)
    check_rc(tb200_grouped_gemm(A.data_ptr(), B.data_ptr(), C.data_ptr(),
                                C2.defined() ? C2.data_ptr() : nullptr, seg_start.data_ptr<int>(),
                                seg_count.data_ptr<int>(), G, rows, N, K, N, 2 * N, b_rows, b_cols,
                                mode, epilogue, status_ptr(A), max_ctas, nullptr, 0, 0,
                                static_cast<int>(pad_align), cur_stream()),
             "grouped_gemm");
  return {C, C2.defined() ? C2 : at::empty({0}, A.options())};
}

Tensor grouped_wgrad(const Tensor& X, const Tensor& dY, const Tensor& seg_start,
                     const Tensor& seg_count, int64_t max_ctas, int64_t pad_align) {
  CHECK_CUDA_CONTIG(X);
  CHECK_CUDA_CONTIG(dY);
  TORCH_CHECK(X.scalar_type() == at::kBFloat16 && dY.scalar_type() == at::kBFloat16,
              "grouped_wgrad: bf16 operands");
  TORCH_CHECK(X.dim() == 2 && dY.dim() == 2 && X.size(0) == dY.size(0), "grouped_wgrad: row mismatch");
  TORCH_CHECK(seg_start.scalar_type() == at::kInt && seg_count.scalar_type() == at::kInt &&
                  seg_start.numel() == seg_count.numel() && seg_start.is_cuda() &&
                  seg_count.is_cuda(),
              "grouped_wgrad: int32 CUDA segment tables");
  c10::cuda::CUDAGuard guard(X.device());
  const int64_t G = seg_start.numel();
  Tensor dW = at::empty({G, X.size(1), dY.size(1)}, X.options());
  check_rc(tb200_grouped_wgrad(X.data_ptr(), dY.data_ptr(), dW.data_ptr(),
                               seg_start.data_ptr<int>(), seg_count.data_ptr<int>(), G, X.size(0),
                               X.size(1), dY.size(1), status_ptr(X), max_ctas,
                               static_cast<int>(pad_align), cur_stream()),
           "grouped_wgrad");
  return dW;
}

// Weight gradient of the groups [g0, g0 + G) written into dW[g0 : g0 + G] of a gradient tensor
// that covers all groups (G = seg_start.numel()): one launch per chunk of experts.
void grouped_wgrad_out(const Tensor& X, const Tensor& dY, Tensor dW, int64_t g0,
                       const Tensor& seg_start, const Tensor& seg_count, int64_t max_ctas,
                       int64_t pad_align) {
  CHECK_CUDA_CONTIG(X);
  CHECK_CUDA_CONTIG(dY);
  CHECK_CUDA_CONTIG(dW);
  TORCH_CHECK(X.scalar_type() == at::kBFloat16 && dY.scalar_type() == at::kBFloat16 &&
                  dW.scalar_type() == at::kBFloat16,
              "grouped_wgrad_out: bf16 operands");
  TORCH_CHECK(X.dim() == 2 && dY.dim() == 2 && X.size(0) == dY.size(0) && dW.dim() == 3 &&
                  dW.size(1) == X.size(1) && dW.size(2) == dY.size(1),
              "grouped_wgrad_out: X [rows, M], dY [rows, N], dW [groups, M, N]");
  const int64_t G = seg_start.numel();
  TORCH_CHECK(seg_start.scalar_type() == at::kInt && seg_count.scalar_type() == at::kInt &&
                  seg_count.numel() == G && seg_start.is_cuda() && seg_count.is_cuda() &&
                  seg_start.is_contiguous() && seg_count.is_contiguous(),
              "grouped_wgrad_out: int32 CUDA segment tables");
  TORCH_CHECK(g0 >= 0 && G >= 1 && g0 + G <= dW.size(0), "grouped_wgrad_out: group range");
  c10::cuda::CUDAGuard guard(X.device());
  auto* out = static_cast<char*>(dW.data_ptr()) + g0 * dW.size(1) * dW.size(2) * 2;
  check_rc(tb200_grouped_wgrad(X.data_ptr(), dY.data_ptr(), out, seg_start.data_ptr<int>(),
                               seg_count.data_ptr<int>(), G, X.size(0), X.size(1), dY.size(1),
                               status_ptr(X), max_ctas, static_cast<int>(pad_align), cur_stream()),
           "grouped_wgrad_out");
}

}  // namespace

// ---------------------------------------------------------------------------------------------
// attention: q, k, v [B, H, S, D] (or [BH, S, D]) bf16 contiguous
std::tuple<Tensor, Tensor> attn_fwd(const Tensor& q, const Tensor& k, const Tensor& v, bool causal,
                                    double scale) {
  CHECK_CUDA_CONTIG(q);
  CHECK_CUDA_CONTIG(k);
  CHECK_CUDA_CONTIG(v);
  TORCH_CHECK(q.scalar_type() == at::kBFloat16 && k.scalar_type() == at::kBFloat16 &&
                  v.scalar_type() == at::kBFloat16, "attn_fwd: bf16 operands");
  TORCH_CHECK(q.dim() >= 3 && q.sizes() == k.sizes() && q.sizes() == v.sizes(),
              "attn_fwd: q, k, v of one shape [..., S, D]");
  c10::cuda::CUDAGuard guard(q.device());
  const int64_t D = q.size(-1), S = q.size(-2), BH = q.numel() / (S * D);
  TORCH_CHECK(S % 128 == 0 && (D == 64 || D == 128), "attn_fwd: S % 128 == 0 and D in {64, 128}");
  Tensor o = at::empty_like(q);
  auto lse_shape = q.sizes().vec();
  lse_shape.pop_back();
  Tensor lse = at::empty(lse_shape, q.options().dtype(at::kFloat));
  check_rc(tb200_attn_fwd(q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(),
                          lse.data_ptr<float>(), static_cast<int>(BH), static_cast<int>(S),
                          static_cast<int>(D), causal ? 1 : 0, static_cast<float>(scale),
                          status_ptr(q), cur_stream()),
           "attn_fwd");
  return {o, lse};
}

std::tuple<Tensor, Tensor, Tensor> attn_bwd(const Tensor& q, const Tensor& k, const Tensor& v,
                                            const Tensor& o, const Tensor& d_o, const Tensor& lse,
                                            bool causal, double scale) {
  CHECK_CUDA_CONTIG(q);
  CHECK_CUDA_CONTIG(k);
  CHECK_CUDA_CONTIG(v);
  CHECK_CUDA_CONTIG(o);
  CHECK_CUDA_CONTIG(d_o);
  CHECK_CUDA_CONTIG(lse);
  TORCH_CHECK(q.scalar_type() == at::kBFloat16 && d_o.scalar_type() == at::kBFloat16 &&
                  o.scalar_type() == at::kBFloat16 && lse.scalar_type() == at::kFloat,
              "attn_bwd: bf16 tensors and an fp32 lse");
  TORCH_CHECK(q.sizes() == k.sizes() && q.sizes() == v.sizes() && q.sizes() == o.sizes() &&
                  q.sizes() == d_o.sizes(), "attn_bwd: shape mismatch");
  c10::cuda::CUDAGuard guard(q.device());
  const int64_t D = q.size(-1), S = q.size(-2), BH = q.numel() / (S * D);
  TORCH_CHECK(lse.numel() == BH * S, "attn_bwd: lse must be [..., S]");
  TORCH_CHECK(S % 128 == 0 && (D == 64 || D == 128), "attn_bwd: S % 128 == 0 and D in {64, 128}");
  Tensor dq = at::empty_like(q), dk = at::empty_like(q), dv = at::empty_like(q);
  Tensor delta = at::empty_like(lse);
  check_rc(tb200_attn_bwd(q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), d_o.data_ptr(),
                          lse.data_ptr<float>(), delta.data_ptr<float>(), dq.data_ptr(),
                          dk.data_ptr(), dv.data_ptr(), static_cast<int>(BH), static_cast<int>(S),
                          static_cast<int>(D), causal ? 1 : 0, static_cast<float>(scale),
                          status_ptr(q), cur_stream()),
           "attn_bwd");
  return {dq, dk, dv};
}

TORCH_LIBRARY(terrace, m) {
  m.def("passthrough(Tensor x) -> Tensor");
  m.def("k1_arrival(Tensor rx, Tensor rslot, Tensor rgate, int quota, int epr, int rpn, "
        "int my_local) -> (Tensor, Tensor, Tensor, Tensor, Tensor)");
  m.def("k2_pack(Tensor hidden, Tensor expert_idx, Tensor gates, int world, int n_experts, "
        "int rpn, int groups_m) -> (Tensor, Tensor, Tensor, Tensor, Tensor)");
  m.def("take_status(int device) -> int", &take_status);
  m.def("rmsnorm_fwd(Tensor x, Tensor w, float eps) -> (Tensor, Tensor)");
  m.def("rmsnorm_bwd(Tensor x, Tensor w, Tensor dy, Tensor rstd) -> (Tensor, Tensor)");
  m.def("route_select(Tensor logits, Tensor bias, int n_groups, int top_k, int top_groups, "
        "int pool) -> (Tensor, Tensor, Tensor, Tensor, Tensor)");
  m.def("route_fused(Tensor hidden, Tensor weight, Tensor bias, int n_groups, int top_k, "
        "int top_groups, int pool) -> (Tensor, Tensor, Tensor, Tensor, Tensor)");
  m.def("route_fused_supported(int E, int H, int n_groups, int top_k, int top_groups) -> bool",
        &route_fused_supported);
  m.def("route_select_bwd(Tensor dgates, Tensor gates, Tensor aff, Tensor idx, int E) -> Tensor");
  m.def("moe_plan(Tensor expert_idx, Tensor? gates, int E, int seg_align) -> "
        "(Tensor, Tensor, Tensor, Tensor, Tensor, Tensor)");
  m.def("moe_scatter_rows(Tensor x, Tensor pos, int rows_out) -> Tensor");
  m.def("moe_combine(Tensor out, Tensor pos, Tensor es, Tensor? gs, int group_size) -> Tensor");
  m.def("moe_combine_bwd(Tensor dy, Tensor out, Tensor pos, Tensor? gs, bool need_dgs) -> "
        "(Tensor, Tensor)");
  m.def("swiglu_bwd(Tensor h13, Tensor dact) -> Tensor");
  m.def("grouped_gemm(Tensor A, Tensor B, Tensor seg_start, Tensor seg_count, int mode, "
        "int epilogue, bool save_pre, int max_ctas, int pad_align=0) -> (Tensor, Tensor)");
  m.def("grouped_wgrad(Tensor X, Tensor dY, Tensor seg_start, Tensor seg_count, int max_ctas, "
        "int pad_align=0) -> Tensor");
  m.def("grouped_wgrad_out(Tensor X, Tensor dY, Tensor(a!) dW, int g0, Tensor seg_start, "
        "Tensor seg_count, int max_ctas, int pad_align=0) -> ()");
  m.def("rope_split(Tensor qkv, Tensor cos, Tensor sin, int n_heads) -> (Tensor, Tensor, Tensor)");
  m.def("rope_merge(Tensor dq, Tensor dk, Tensor dv, Tensor cos, Tensor sin) -> Tensor");
  m.def("zero_pad_rows(Tensor(a!) buf, Tensor seg_start, Tensor seg_count, int align) -> ()");
  m.def("attn_fwd(Tensor q, Tensor k, Tensor v, bool causal, float scale) -> (Tensor, Tensor)");
  m.def("attn_bwd(Tensor q, Tensor k, Tensor v, Tensor o, Tensor d_o, Tensor lse, bool causal, "
        "float scale) -> (Tensor, Tensor, Tensor)");
  terrace_b200_register_symm(m);
}

TORCH_LIBRARY_IMPL(terrace, CUDA, m) {
  m.impl("passthrough", &passthrough_cuda);
  m.impl("k1_arrival", &k1_arrival_cuda);
  m.impl("k2_pack", &k2_pack_cuda);
  m.impl("rmsnorm_fwd", &rmsnorm_fwd);
  m.impl("rmsnorm_bwd", &rmsnorm_bwd);
  m.impl("route_select", &route_select);
  m.impl("route_fused", &route_fused);
  m.impl("route_select_bwd", &route_select_bwd);
  m.impl("moe_plan", &moe_plan);
  m.impl("moe_scatter_rows", &moe_scatter_rows);
  m.impl("moe_combine", &moe_combine);
  m.impl("moe_combine_bwd", &moe_combine_bwd);
  m.impl("swiglu_bwd", &swiglu_bwd);
  m.impl("grouped_gemm", &grouped_gemm);
  m.impl("grouped_wgrad", &grouped_wgrad);
  m.impl("grouped_wgrad_out", &grouped_wgrad_out);
  m.impl("rope_split", &rope_split);
  m.impl("rope_merge", &rope_merge);
  m.impl("zero_pad_rows", &zero_pad_rows);
  m.impl("attn_fwd", &attn_fwd);
  m.impl("attn_bwd", &attn_bwd);
  terrace_b200_register_symm_cuda(m);
}

TORCH_LIBRARY_IMPL(terrace, Meta, m) {
  m.impl("passthrough", &passthrough_meta);
  m.impl("k1_arrival", &k1_arrival_meta);
  m.impl("k2_pack", &k2_pack_meta);
  terrace_b200_register_meta(m);
}
