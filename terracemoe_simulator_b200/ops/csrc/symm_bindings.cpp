// Host runtime of the symmetric arena + torch ops around the fused dispatch / combine kernels.
//
// Arena memory is a plain cudaMalloc allocation (not the caching allocator) so that it can be
// exported with cudaIpcGetMemHandle and opened by the other ranks of the node; the Python side
// exchanges the 64-byte handles through torch.distributed and hands the resulting peer pointers
// to symm_make_arena, which packs the Tb200Arena descriptor the kernels take by value.
#include <ATen/ATen.h>
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/library.h>

#include <cstring>
#include <mutex>
#include <vector>

#include "launch.h"
#include "symm.h"
#include "symm_layout.h"

namespace {

using at::Tensor;

cudaStream_t cur_stream() { return at::cuda::getCurrentCUDAStream().stream(); }

void check_rc(int rc, const char* what) {
  TORCH_CHECK(rc == TB200_OK, what, " failed with terrace_b200 error code ", rc);
}
void check_cuda(cudaError_t e, const char* what) {
  TORCH_CHECK(e == cudaSuccess, what, ": ", cudaGetErrorString(e));
}

const Tb200Arena* arena_of(const Tensor& blob) {
  TORCH_CHECK(blob.device().is_cpu() && blob.scalar_type() == at::kByte && blob.is_contiguous() &&
                  blob.numel() == static_cast<int64_t>(sizeof(Tb200Arena)),
              "arena descriptor must come from symm_make_arena");
  return reinterpret_cast<const Tb200Arena*>(blob.data_ptr<uint8_t>());
}

long long section_offset(const Tb200Arena* a, int64_t sel) {
  switch (sel) {
    case 0: return a->off_xin;
    case 1: return a->off_yout;
    case 2: return a->off_dout;
    case 3: return a->off_dxs;
    case 4: return a->off_ha_rows;
    case 5: return a->off_red;
    case 6: return a->off_hb_rows;
    case 7: return a->off_dred;
    default: TORCH_CHECK(false, "unknown arena section ", sel);
  }
  return 0;
}

// status word shared with bindings.cpp through the take_status op: keep one per device here too
Tensor& symm_status(int device) {
  static std::mutex mu;
  static std::vector<Tensor> words(64);
  std::lock_guard<std::mutex> lock(mu);
  if (!words[device].defined())
    words[device] = at::zeros({1}, at::TensorOptions().dtype(at::kInt).device(at::kCUDA, device));
  return words[device];
}
int* st_ptr(const Tensor& like) { return symm_status(like.get_device()).data_ptr<int>(); }

// The device status word itself (no copy, no synchronisation): a training loop can read it a few
// steps late through a deferred device-to-host copy instead of stalling on take_status.
Tensor symm_status_tensor(int64_t device) { return symm_status(static_cast<int>(device)); }

int64_t symm_take_status(int64_t device) {
  Tensor& w = symm_status(static_cast<int>(device));
  const int v = w.item<int>();
  if (v != 0) w.zero_();
  return v;
}

Tensor symm_alloc(int64_t nbytes, int64_t device) {
  TORCH_CHECK(nbytes > 0, "symm_alloc: size must be positive");
  c10::cuda::CUDAGuard guard(static_cast<c10::DeviceIndex>(device));
  void* ptr = nullptr;
  check_cuda(cudaMalloc(&ptr, static_cast<size_t>(nbytes)), "symm_alloc cudaMalloc");
  check_cuda(cudaMemset(ptr, 0, static_cast<size_t>(nbytes)), "symm_alloc cudaMemset");
  check_cuda(cudaDeviceSynchronize(), "symm_alloc sync");
  auto opts = at::TensorOptions().dtype(at::kByte).device(at::kCUDA, device);
  return at::from_blob(ptr, {nbytes}, [](void* p) { cudaFree(p); }, opts);
}

Tensor symm_ipc_handle(const Tensor& buf) {
  TORCH_CHECK(buf.is_cuda(), "symm_ipc_handle: CUDA buffer");
  c10::cuda::CUDAGuard guard(buf.device());
  cudaIpcMemHandle_t h;
  check_cuda(cudaIpcGetMemHandle(&h, buf.data_ptr()), "cudaIpcGetMemHandle");
  Tensor out = at::empty({static_cast<int64_t>(sizeof(h))}, at::kByte);
  std::memcpy(out.data_ptr<uint8_t>(), &h, sizeof(h));
  return out;
}

int64_t symm_ipc_open(const Tensor& handle, int64_t device) {
  TORCH_CHECK(handle.device().is_cpu() && handle.numel() == sizeof(cudaIpcMemHandle_t),
              "symm_ipc_open: 64-byte CPU handle");
  c10::cuda::CUDAGuard guard(static_cast<c10::DeviceIndex>(device));
  cudaIpcMemHandle_t h;
  std::memcpy(&h, handle.data_ptr<uint8_t>(), sizeof(h));
  void* ptr = nullptr;
  check_cuda(cudaIpcOpenMemHandle(&ptr, h, cudaIpcMemLazyEnablePeerAccess), "cudaIpcOpenMemHandle");
  return reinterpret_cast<int64_t>(ptr);
}

void symm_ipc_close(int64_t ptr, int64_t device) {
  c10::cuda::CUDAGuard guard(static_cast<c10::DeviceIndex>(device));
  cudaIpcCloseMemHandle(reinterpret_cast<void*>(ptr));
}

// geom = {world, rank, n_experts, epr, rpn, n_nodes, tokens_cap, top_k, groups_m, q, hidden,
//         cap_rows};  offsets = the 12 section offsets in struct order
Tensor symm_make_arena(std::vector<int64_t> peers, std::vector<int64_t> offsets,
                       std::vector<int64_t> geom) {
  TORCH_CHECK(peers.size() >= 1 && peers.size() <= TB200_MAX_WORLD, "symm_make_arena: world");
  TORCH_CHECK(offsets.size() == 12 && geom.size() == 12, "symm_make_arena: table sizes");
  Tb200Arena a;
  std::memset(&a, 0, sizeof(a));
  for (size_t i = 0; i < peers.size(); ++i) a.peer[i] = static_cast<unsigned long long>(peers[i]);
  a.off_counts_all = offsets[0];
  a.off_flags = offsets[1];
  a.off_xin = offsets[2];
  a.off_yout = offsets[3];
  a.off_dout = offsets[4];
  a.off_dxs = offsets[5];
  a.off_ha_rows = offsets[6];
  a.off_ha_hdr = offsets[7];
  a.off_red = offsets[8];
  a.off_hb_rows = offsets[9];
  a.off_dred = offsets[10];
  a.off_dgate = offsets[11];
  a.world = geom[0]; a.rank = geom[1]; a.n_experts = geom[2]; a.epr = geom[3]; a.rpn = geom[4];
  a.n_nodes = geom[5]; a.tokens_cap = geom[6]; a.top_k = geom[7]; a.groups_m = geom[8];
  a.q = geom[9]; a.hidden = geom[10]; a.cap_rows = geom[11];
  TORCH_CHECK(a.world == static_cast<int>(peers.size()), "symm_make_arena: world != #peers");
  for (auto off : offsets) TORCH_CHECK(off % 16 == 0, "symm_make_arena: 16-byte aligned sections");
  Tensor out = at::empty({static_cast<int64_t>(sizeof(a))}, at::kByte);
  std::memcpy(out.data_ptr<uint8_t>(), &a, sizeof(a));
  return out;
}

// ---------------------------------------------------------------------------------------------
std::tuple<Tensor, Tensor, Tensor, Tensor, Tensor> ep_plan_pass1(const Tensor& expert_idx,
                                                                 const Tensor& gates, int64_t E) {
  TORCH_CHECK(expert_idx.is_cuda() && expert_idx.is_contiguous() &&
                  expert_idx.scalar_type() == at::kLong && expert_idx.dim() == 2,
              "ep_plan_pass1: int64 [T, k] CUDA indices");
  TORCH_CHECK(gates.is_cuda() && gates.is_contiguous() && gates.scalar_type() == at::kFloat &&
                  gates.sizes() == expert_idx.sizes(),
              "ep_plan_pass1: fp32 gates [T, k]");
  c10::cuda::CUDAGuard guard(expert_idx.device());
  const int64_t T = expert_idx.size(0), k = expert_idx.size(1);
  auto iopt = expert_idx.options().dtype(at::kInt);
  Tensor es = at::empty({T, k}, iopt), cols = at::empty({T, k}, iopt);
  Tensor rank_local = at::empty({T, k}, iopt);
  Tensor gs = at::empty({T, k}, gates.options());
  Tensor chunk_hist = at::empty({TB200_PLAN_CHUNKS, E}, iopt);
  check_rc(tb200_plan_pass1(reinterpret_cast<const long long*>(expert_idx.data_ptr<int64_t>()),
                            gates.data_ptr<float>(), es.data_ptr<int>(), gs.data_ptr<float>(),
                            cols.data_ptr<int>(), rank_local.data_ptr<int>(),
                            chunk_hist.data_ptr<int>(), T, k, E, cur_stream()),
           "ep_plan_pass1");
  return {es, gs, cols, rank_local, chunk_hist};
}

// Returns (my_base, seg_start, seg_count, rows_a, my_prefix).  cap > 0 bounds the rows every
// expert accepts (canonical order: source rank, then token).
std::tuple<Tensor, Tensor, Tensor, Tensor, Tensor> ep_plan(
    const Tensor& arena, Tensor chunk_hist, const c10::optional<Tensor>& chunka_hist,
    int64_t epoch, int64_t seg_align, int64_t cap) {
  const Tb200Arena* a = arena_of(arena);
  c10::cuda::CUDAGuard guard(chunk_hist.device());
  auto iopt = chunk_hist.options();
  Tensor my_base = at::empty({a->n_experts}, iopt);
  Tensor seg_start = at::empty({a->epr}, iopt), seg_count = at::empty({a->epr}, iopt);
  Tensor rows_a = at::zeros({a->world, a->n_nodes}, iopt);
  Tensor my_prefix = at::empty({a->n_experts}, iopt);
  check_rc(tb200_ep_plan(a, chunk_hist.data_ptr<int>(),
                         chunka_hist.has_value() ? chunka_hist->data_ptr<int>() : nullptr,
                         my_base.data_ptr<int>(), seg_start.data_ptr<int>(),
                         seg_count.data_ptr<int>(), rows_a.data_ptr<int>(),
                         my_prefix.data_ptr<int>(), epoch, static_cast<int>(seg_align),
                         static_cast<int>(cap), st_ptr(chunk_hist), cur_stream()),
           "ep_plan");
  return {my_base, seg_start, seg_count, rows_a, my_prefix};
}

// One-hop push of the picks whose local expert index lies in [le_lo, le_hi) into the owners'
// sections at byte offset `dst_off`; `pos` ([T, k], written for the covered picks) and `dgs`
// (gate gradients, optional) are shared by the launches of one step.  rowmap_off >= 0: the
// return address (source rank, slot) of every row is left in the owner's row map for a GEMM
// whose epilogue scatters its rows back (grouped_gemm_scatter).  dot_local: the gate gradient
// reads the saved expert output from MY return section (`dot_off`) at slot p instead of the
// owner's row at `dot_off`.
void ep_push(const Tensor& arena, const Tensor& x, const Tensor& es, const Tensor& rank_local,
             const Tensor& chunk_base, const Tensor& my_base, const c10::optional<Tensor>& gs,
             Tensor pos, const c10::optional<Tensor>& dgs, int64_t dst_off, int64_t dot_off,
             bool dot_local, int64_t flag_kind, int64_t flag_value, int64_t le_lo, int64_t le_hi,
             Tensor done, int64_t rowmap_off, int64_t ret_slots,
             const c10::optional<Tensor>& my_prefix, int64_t cap) {
  const Tb200Arena* a = arena_of(arena);
  TORCH_CHECK(rowmap_off < 0 || rowmap_off % 16 == 0, "ep_push: row map offset alignment");
  TORCH_CHECK(dst_off >= 0 && dst_off % 16 == 0 && dot_off % 16 == 0,
              "ep_push: section offsets must be 16-byte aligned");
  TORCH_CHECK(x.is_cuda() && x.is_contiguous() && x.scalar_type() == at::kBFloat16 &&
                  x.dim() == 2 && x.size(1) == a->hidden,
              "ep_push: bf16 [T, H] rows");
  TORCH_CHECK(es.sizes() == rank_local.sizes() && es.size(0) == x.size(0) &&
                  es.size(1) == a->top_k && es.scalar_type() == at::kInt,
              "ep_push: index planes must be int32 [T, k]");
  TORCH_CHECK(pos.is_cuda() && pos.is_contiguous() && pos.scalar_type() == at::kInt &&
                  pos.sizes() == es.sizes(),
              "ep_push: pos must be int32 [T, k]");
  const bool want_dgs = dgs.has_value();
  if (want_dgs)
    TORCH_CHECK(dgs->is_cuda() && dgs->is_contiguous() && dgs->scalar_type() == at::kFloat &&
                    dgs->sizes() == es.sizes(),
                "ep_push: dgs must be fp32 [T, k]");
  c10::cuda::CUDAGuard guard(x.device());
  const int64_t T = x.size(0);
  check_rc(tb200_ep_push(a, x.data_ptr(), es.data_ptr<int>(), rank_local.data_ptr<int>(),
                         chunk_base.data_ptr<int>(), my_base.data_ptr<int>(), pos.data_ptr<int>(),
                         gs.has_value() ? gs->data_ptr<float>() : nullptr,
                         want_dgs ? dgs->data_ptr<float>() : nullptr, dst_off,
                         want_dgs ? dot_off : 0, T, flag_kind, flag_value, le_lo, le_hi,
                         done.data_ptr<int>(), st_ptr(x), rowmap_off, static_cast<int>(ret_slots),
                         dot_local ? 1 : 0,
                         my_prefix.has_value() ? my_prefix->data_ptr<int>() : nullptr,
                         my_prefix.has_value() ? static_cast<int>(cap) : 0, cur_stream()),
           "ep_push");
}

void ep_signal(const Tensor& arena, int64_t kind, int64_t first, int64_t n, int64_t stride,
               int64_t idx, int64_t epoch, int64_t wait_kind, int64_t wait_first, int64_t wait_n,
               int64_t wait_value, const Tensor& like) {
  const Tb200Arena* a = arena_of(arena);
  c10::cuda::CUDAGuard guard(like.device());
  check_rc(tb200_signal(a, kind, first, n, stride, idx, epoch, wait_kind, wait_first, wait_n,
                        wait_value, st_ptr(like), cur_stream()),
           "ep_signal");
}

// y[t] = canonical gate-weighted reduction of the token's k expert-output rows, read from the
// owners' sections at byte offset `src_off` (row pos) or, with local_slots > 0, from MY section
// at `src_off`, slot t * k + j (the owners' GEMM epilogues stored them there).
Tensor ep_pull_combine(const Tensor& arena, const Tensor& pos, const Tensor& es,
                       const c10::optional<Tensor>& gs, int64_t src_off, int64_t group_size,
                       int64_t wait_kind, int64_t epoch, int64_t local_slots) {
  const Tb200Arena* a = arena_of(arena);
  TORCH_CHECK(src_off >= 0 && src_off % 16 == 0, "ep_pull_combine: section offset");
  TORCH_CHECK(pos.is_cuda() && pos.is_contiguous() && pos.sizes() == es.sizes() &&
                  pos.size(1) == a->top_k,
              "ep_pull_combine: [T, k] index planes");
  c10::cuda::CUDAGuard guard(pos.device());
  const int64_t T = pos.size(0);
  Tensor y = at::empty({T, a->hidden}, pos.options().dtype(at::kBFloat16));
  check_rc(tb200_ep_pull_combine(a, pos.data_ptr<int>(), es.data_ptr<int>(),
                                 gs.has_value() ? gs->data_ptr<float>() : nullptr, y.data_ptr(),
                                 src_off, T, group_size, wait_kind, epoch, st_ptr(pos),
                                 static_cast<int>(local_slots), cur_stream()),
           "ep_pull_combine");
  return y;
}

std::tuple<Tensor, Tensor> hopa_rank(const Tensor& arena, const Tensor& es) {
  const Tb200Arena* a = arena_of(arena);
  c10::cuda::CUDAGuard guard(es.device());
  const int64_t T = es.size(0);
  Tensor ranka = at::empty({T, a->groups_m}, es.options());
  Tensor chunka = at::empty({TB200_PLAN_CHUNKS, a->n_nodes}, es.options());
  check_rc(tb200_hopa_rank(a, es.data_ptr<int>(), ranka.data_ptr<int>(), chunka.data_ptr<int>(), T,
                           cur_stream()),
           "hopa_rank");
  return {ranka, chunka};
}

std::tuple<Tensor, Tensor> hopa_push(const Tensor& arena, const Tensor& x, const Tensor& es,
                                     const Tensor& gs, const Tensor& rank_local,
                                     const Tensor& chunk_base, const Tensor& my_base,
                                     const Tensor& ranka_local, const Tensor& chunka_base,
                                     const c10::optional<Tensor>& rowa_in, int64_t rows_sel,
                                     bool with_header, int64_t flag_kind, int64_t epoch,
                                     Tensor done, const c10::optional<Tensor>& my_prefix,
                                     int64_t cap) {
  const Tb200Arena* a = arena_of(arena);
  TORCH_CHECK(x.is_cuda() && x.is_contiguous() && x.scalar_type() == at::kBFloat16 &&
                  x.dim() == 2 && x.size(1) == a->hidden && x.size(0) <= a->tokens_cap,
              "hopa_push: bf16 [T <= tokens_cap, H] rows");
  TORCH_CHECK(with_header || rowa_in.has_value(), "hopa_push: backward needs the forward rows");
  c10::cuda::CUDAGuard guard(x.device());
  const int64_t T = x.size(0);
  Tensor pos = with_header ? at::empty({T, a->top_k}, es.options()) : at::empty({0}, es.options());
  Tensor rowa = with_header ? at::empty({T, a->groups_m}, es.options()) : *rowa_in;
  check_rc(tb200_hopa_push(a, x.data_ptr(), es.data_ptr<int>(), gs.data_ptr<float>(),
                           rank_local.data_ptr<int>(), chunk_base.data_ptr<int>(),
                           my_base.data_ptr<int>(), ranka_local.data_ptr<int>(),
                           chunka_base.data_ptr<int>(), with_header ? pos.data_ptr<int>() : nullptr,
                           rowa.data_ptr<int>(), section_offset(a, rows_sel), with_header ? 1 : 0,
                           T, flag_kind, epoch, done.data_ptr<int>(), st_ptr(x),
                           my_prefix.has_value() ? my_prefix->data_ptr<int>() : nullptr,
                           my_prefix.has_value() ? static_cast<int>(cap) : 0, cur_stream()),
           "hopa_push");
  return {pos, rowa};
}

void arrival_push(const Tensor& arena, const Tensor& rows_a, int64_t rows_sel, int64_t dst_off,
                  int64_t dot_off, bool dot_local, bool scale_gate, bool want_dgate,
                  int64_t wait_kind, int64_t data_kind, int64_t dg_kind, int64_t epoch,
                  int64_t flag_value, int64_t le_lo, int64_t le_hi, Tensor done,
                  int64_t rowmap_off) {
  const Tb200Arena* a = arena_of(arena);
  TORCH_CHECK(dst_off >= 0 && dst_off % 16 == 0 && dot_off % 16 == 0 &&
                  (rowmap_off < 0 || rowmap_off % 16 == 0),
              "arrival_push: section offsets must be 16-byte aligned");
  c10::cuda::CUDAGuard guard(rows_a.device());
  check_rc(tb200_arrival_push(a, rows_a.data_ptr<int>(), section_offset(a, rows_sel), dst_off,
                              want_dgate ? dot_off : 0, scale_gate, want_dgate, wait_kind,
                              data_kind, dg_kind, epoch, flag_value, le_lo, le_hi,
                              done.data_ptr<int>(), st_ptr(rows_a), rowmap_off, dot_local ? 1 : 0,
                              cur_stream()),
           "arrival_push");
}

void arrival_combine(const Tensor& arena, const Tensor& rows_a, int64_t src_off, int64_t red_sel,
                     bool use_gate, int64_t wait_kind, int64_t red_kind, int64_t epoch,
                     Tensor done, bool push_back, bool local_slots) {
  const Tb200Arena* a = arena_of(arena);
  TORCH_CHECK(src_off >= 0 && src_off % 16 == 0, "arrival_combine: section offset");
  c10::cuda::CUDAGuard guard(rows_a.device());
  check_rc(tb200_arrival_combine(a, rows_a.data_ptr<int>(), src_off, section_offset(a, red_sel),
                                 use_gate, wait_kind, red_kind, epoch, done.data_ptr<int>(),
                                 st_ptr(rows_a), push_back ? 1 : 0, local_slots ? 1 : 0,
                                 cur_stream()),
           "arrival_combine");
}

Tensor origin_combine(const Tensor& arena, const Tensor& es, const Tensor& rowa, int64_t red_sel,
                      int64_t wait_kind, int64_t epoch, bool local_rows) {
  const Tb200Arena* a = arena_of(arena);
  c10::cuda::CUDAGuard guard(es.device());
  const int64_t T = es.size(0);
  Tensor y = at::empty({T, a->hidden}, es.options().dtype(at::kBFloat16));
  check_rc(tb200_origin_combine(a, es.data_ptr<int>(), rowa.data_ptr<int>(), y.data_ptr(),
                                section_offset(a, red_sel), T, wait_kind, epoch, st_ptr(es),
                                local_rows ? 1 : 0, cur_stream()),
           "origin_combine");
  return y;
}

Tensor origin_pull_dgate(const Tensor& arena, const Tensor& es, const Tensor& rowa,
                         int64_t wait_kind, int64_t epoch) {
  const Tb200Arena* a = arena_of(arena);
  c10::cuda::CUDAGuard guard(es.device());
  const int64_t T = es.size(0);
  Tensor dgs = at::empty({T, a->top_k}, es.options().dtype(at::kFloat));
  check_rc(tb200_origin_pull_dgate(a, es.data_ptr<int>(), rowa.data_ptr<int>(),
                                   dgs.data_ptr<float>(), T, wait_kind, epoch, st_ptr(es),
                                   cur_stream()),
           "origin_pull_dgate");
  return dgs;
}

// Grouped GEMM with caller-provided output (an arena section or a plain tensor) and optional
// arrival-flag gating of the A operand.
void grouped_gemm_ex(const Tensor& A, const Tensor& B, Tensor C, const c10::optional<Tensor>& C2,
                     const Tensor& seg_start, const Tensor& seg_count, int64_t mode,
                     int64_t epilogue, const c10::optional<Tensor>& arena, int64_t wait_kind,
                     int64_t wait_first, int64_t wait_n, int64_t epoch, int64_t pad_align) {
  TORCH_CHECK(A.is_cuda() && A.is_contiguous() && B.is_cuda() && B.is_contiguous() &&
                  C.is_cuda() && C.is_contiguous(),
              "grouped_gemm_ex: contiguous CUDA tensors");
  TORCH_CHECK(A.scalar_type() == at::kBFloat16 && B.scalar_type() == at::kBFloat16 &&
                  C.scalar_type() == at::kBFloat16 && A.dim() == 2 && B.dim() == 3 && C.dim() == 2,
              "grouped_gemm_ex: bf16 A [rows, K], B [G, r, c], C [rows, N]");
  TORCH_CHECK(seg_start.scalar_type() == at::kInt && seg_count.scalar_type() == at::kInt &&
                  seg_start.numel() == B.size(0) && seg_count.numel() == B.size(0),
              "grouped_gemm_ex: int32 segment tables of length G");
  c10::cuda::CUDAGuard guard(A.device());
  const int64_t rows = A.size(0), K = A.size(1), G = B.size(0);
  const int64_t b_rows = B.size(1), b_cols = B.size(2);
  int64_t N;
  if (mode == 0) {
    TORCH_CHECK(b_rows == K, "grouped_gemm_ex fwd: B rows must equal K");
    N = epilogue == 1 ? b_cols / 2 : b_cols;
  } else {
    TORCH_CHECK(b_cols == K, "grouped_gemm_ex dgrad: B cols must equal K");
    N = epilogue == 1 ? b_rows / 2 : b_rows;
  }
  if (epilogue == 3) {   // SwiGLU backward behind the dgrad GEMM: C = d[gate | up], C2 = [gate | up]
    TORCH_CHECK(C2.has_value() && C.size(0) >= rows && C.size(1) == 2 * N,
                "grouped_gemm_ex: epilogue 3 needs C [>= rows, 2N] and the saved "
                "pre-activations in C2");
  } else {
    TORCH_CHECK(C.size(0) >= rows && C.size(1) == N, "grouped_gemm_ex: C must be [>= rows, N]");
  }
  if (C2.has_value())
    TORCH_CHECK(C2->is_contiguous() && C2->size(0) >= rows && C2->size(1) == 2 * N &&
                    C2->scalar_type() == at::kBFloat16,
                "grouped_gemm_ex: C2 must be bf16 [>= rows, 2N]");
  const int* wait_flags = nullptr;
  if (arena.has_value() && wait_n > 0) {
    const Tb200Arena* a = arena_of(*arena);
    wait_flags = reinterpret_cast<const int*>(a->peer[a->rank] + a->off_flags) +
                 wait_kind * TB200_MAX_WORLD + wait_first;
  }
  check_rc(tb200_grouped_gemm(A.data_ptr(), B.data_ptr(), C.data_ptr(),
                              C2.has_value() ? C2->data_ptr() : nullptr, seg_start.data_ptr<int>(),
                              seg_count.data_ptr<int>(), G, rows, N, K, epilogue == 3 ? 2 * N : N,
                              2 * N, b_rows, b_cols, mode, epilogue, st_ptr(A), 0, wait_flags,
                              wait_n, epoch,
                              static_cast<int>(pad_align), cur_stream()),
           "grouped_gemm_ex");
}

// Grouped fwd / dgrad GEMM whose output rows go straight to their return slots, possibly in
// peer GPUs' arenas: row r -> scatter_base[m / slots] + (m % slots) * N elements, m = row_map[r].
void grouped_gemm_scatter(const Tensor& A, const Tensor& B, const Tensor& seg_start,
                          const Tensor& seg_count, int64_t mode, const Tensor& row_map,
                          const Tensor& scatter_base, int64_t slots) {
  TORCH_CHECK(A.is_cuda() && A.is_contiguous() && B.is_cuda() && B.is_contiguous() &&
                  A.scalar_type() == at::kBFloat16 && B.scalar_type() == at::kBFloat16 &&
                  A.dim() == 2 && B.dim() == 3,
              "grouped_gemm_scatter: bf16 A [rows, K], B [G, r, c]");
  TORCH_CHECK(seg_start.scalar_type() == at::kInt && seg_count.scalar_type() == at::kInt &&
                  seg_start.numel() == B.size(0) && seg_count.numel() == B.size(0),
              "grouped_gemm_scatter: int32 segment tables of length G");
  TORCH_CHECK(row_map.is_cuda() && row_map.scalar_type() == at::kInt && row_map.is_contiguous() &&
                  row_map.numel() >= A.size(0),
              "grouped_gemm_scatter: int32 row map covering the rows of A");
  TORCH_CHECK(scatter_base.is_cuda() && scatter_base.scalar_type() == at::kLong &&
                  scatter_base.is_contiguous() && scatter_base.numel() >= 1 &&
                  scatter_base.numel() <= TB200_MAX_WORLD && slots > 0,
              "grouped_gemm_scatter: int64 base address per rank");
  c10::cuda::CUDAGuard guard(A.device());
  const int64_t rows = A.size(0), K = A.size(1), G = B.size(0);
  const int64_t b_rows = B.size(1), b_cols = B.size(2);
  int64_t N;
  if (mode == 0) {
    TORCH_CHECK(b_rows == K, "grouped_gemm_scatter fwd: B rows must equal K");
    N = b_cols;
  } else {
    TORCH_CHECK(mode == 1 && b_cols == K, "grouped_gemm_scatter dgrad: B cols must equal K");
    N = b_rows;
  }
  check_rc(tb200_grouped_gemm_scatter(
               A.data_ptr(), B.data_ptr(), seg_start.data_ptr<int>(), seg_count.data_ptr<int>(),
               G, rows, N, K, N, b_rows, b_cols, mode, row_map.data_ptr<int>(),
               reinterpret_cast<const unsigned long long*>(scatter_base.data_ptr<int64_t>()),
               static_cast<int>(slots), static_cast<int>(scatter_base.numel()), st_ptr(A), 0,
               cur_stream()),
           "grouped_gemm_scatter");
}

}  // namespace

void terrace_b200_register_symm(torch::Library& m) {
  m.def("symm_take_status(int device) -> int", &symm_take_status);
  m.def("symm_status_tensor(int device) -> Tensor", &symm_status_tensor);
  m.def("symm_alloc(int nbytes, int device) -> Tensor", &symm_alloc);
  m.def("symm_ipc_handle(Tensor buf) -> Tensor", &symm_ipc_handle);
  m.def("symm_ipc_open(Tensor handle, int device) -> int", &symm_ipc_open);
  m.def("symm_ipc_close(int ptr, int device) -> ()", &symm_ipc_close);
  m.def("symm_make_arena(int[] peers, int[] offsets, int[] geom) -> Tensor", &symm_make_arena);
  m.def("ep_plan_pass1(Tensor expert_idx, Tensor gates, int E) -> "
        "(Tensor, Tensor, Tensor, Tensor, Tensor)");
  m.def("ep_plan(Tensor arena, Tensor(a!) chunk_hist, Tensor(b!)? chunka_hist, int epoch, "
        "int seg_align=1, int cap=0) -> (Tensor, Tensor, Tensor, Tensor, Tensor)");
  m.def("ep_push(Tensor arena, Tensor x, Tensor es, Tensor rank_local, Tensor chunk_base, "
        "Tensor my_base, Tensor? gs, Tensor(a!) pos, Tensor(b!)? dgs, int dst_off, int dot_off, "
        "bool dot_local, int flag_kind, int flag_value, int le_lo, int le_hi, Tensor(c!) done, "
        "int rowmap_off, int ret_slots, Tensor? my_prefix=None, int cap=0) -> ()");
  m.def("ep_signal(Tensor arena, int kind, int first, int n, int stride, int idx, int epoch, "
        "int wait_kind, int wait_first, int wait_n, int wait_value, Tensor like) -> ()");
  m.def("ep_pull_combine(Tensor arena, Tensor pos, Tensor es, Tensor? gs, int src_off, "
        "int group_size, int wait_kind, int epoch, int local_slots=0) -> Tensor");
  m.def("grouped_gemm_scatter(Tensor A, Tensor B, Tensor seg_start, Tensor seg_count, int mode, "
        "Tensor row_map, Tensor scatter_base, int slots) -> ()");
  m.def("hopa_rank(Tensor arena, Tensor es) -> (Tensor, Tensor)");
  m.def("hopa_push(Tensor arena, Tensor x, Tensor es, Tensor gs, Tensor rank_local, "
        "Tensor chunk_base, Tensor my_base, Tensor ranka_local, Tensor chunka_base, "
        "Tensor? rowa_in, int rows_sel, bool with_header, int flag_kind, int epoch, "
        "Tensor(a!) done, Tensor? my_prefix=None, int cap=0) -> (Tensor, Tensor)");
  m.def("arrival_push(Tensor arena, Tensor rows_a, int rows_sel, int dst_off, int dot_off, "
        "bool dot_local, bool scale_gate, bool want_dgate, int wait_kind, int data_kind, "
        "int dg_kind, int epoch, int flag_value, int le_lo, int le_hi, Tensor(a!) done, "
        "int rowmap_off) -> ()");
  m.def("arrival_combine(Tensor arena, Tensor rows_a, int src_off, int red_sel, bool use_gate, "
        "int wait_kind, int red_kind, int epoch, Tensor(a!) done, bool push_back=False, "
        "bool local_slots=False) -> ()");
  m.def("origin_combine(Tensor arena, Tensor es, Tensor rowa, int red_sel, int wait_kind, "
        "int epoch, bool local_rows=False) -> Tensor");
  m.def("origin_pull_dgate(Tensor arena, Tensor es, Tensor rowa, int wait_kind, int epoch) -> "
        "Tensor");
  m.def("grouped_gemm_ex(Tensor A, Tensor B, Tensor(a!) C, Tensor(b!)? C2, Tensor seg_start, "
        "Tensor seg_count, int mode, int epilogue, Tensor? arena, int wait_kind, int wait_first, "
        "int wait_n, int epoch, int pad_align=0) -> ()");
}

// The device implementations of the ops declared above (every op that takes a CUDA tensor);
// the host-only ops (allocation, IPC, status) stay catch-all functions.
void terrace_b200_register_symm_cuda(torch::Library& m) {
  m.impl("ep_plan_pass1", &ep_plan_pass1);
  m.impl("ep_plan", &ep_plan);
  m.impl("ep_push", &ep_push);
  m.impl("ep_signal", &ep_signal);
  m.impl("ep_pull_combine", &ep_pull_combine);
  m.impl("grouped_gemm_scatter", &grouped_gemm_scatter);
  m.impl("hopa_rank", &hopa_rank);
  m.impl("hopa_push", &hopa_push);
  m.impl("arrival_push", &arrival_push);
  m.impl("arrival_combine", &arrival_combine);
  m.impl("origin_combine", &origin_combine);
  m.impl("origin_pull_dgate", &origin_pull_dgate);
  m.impl("grouped_gemm_ex", &grouped_gemm_ex);
}
