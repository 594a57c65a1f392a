// Allocation-free variant of the MoE permutation plan.
//
// This entry point has no counterpart in the reference.  It exists for callers that are not
// allowed to allocate device memory at the moment they need a plan: code running inside a
// memory-pool-managed region or under a runtime that forbids cudaMalloc/cudaFree on the hot path
// (they synchronise the device), embedders that drive the library from plain C without a tensor
// allocator, and replay loops whose buffers must all be fixed up front.  The regular entry point
// (tb200_moe_plan in launch.h) makes its caller provide a scratch buffer; this one keeps the
// scratch in a fixed array inside the library.
//
// Contract
//   * Inputs and outputs are caller-owned device buffers, exactly as for tb200_moe_plan:
//       expert_idx [T, k] int64, gates [T, k] fp32 (may be null: all gates 1)
//       es, cols, pos [T, k] int32, gs [T, k] fp32, seg_start, seg_count [E] int32
//   * Scratch lives in a file-scope device array of TB200_PLAN_STATIC_MAX_INTS 32-bit words
//     (1.5 MiB) that every GPU loading the library holds until the process exits.
//   * Limits: T * k <= TB200_PLAN_STATIC_MAX_PAIRS (262144), E <= TB200_PLAN_STATIC_MAX_EXPERTS
//     (1024), k <= 32.  Larger problems are rejected with TB200_ERR_SIZE (5) and a message on
//     stderr; nothing is launched.
//   * The function calls no cudaMalloc, cudaFree or other allocating routine.  Its first call on
//     a device resolves the array's device address (cudaGetSymbolAddress) and remembers it; make
//     that first call with the device current and before starting any stream capture.
//   * All calls on one device share the one array and it keeps the previous call's contents.  The
//     kernels overwrite every word they later read, so nothing has to be cleared between calls,
//     but two calls that overlap on the GPU (different streams, no ordering between them) race on
//     it: order them on one stream or with events.
//   * Results are identical to tb200_moe_plan for the same inputs.
#pragma once
#include <cuda_runtime.h>

#define TB200_PLAN_STATIC_MAX_PAIRS 262144
#define TB200_PLAN_STATIC_MAX_EXPERTS 1024
#define TB200_PLAN_STATIC_MAX_INTS (TB200_PLAN_STATIC_MAX_PAIRS + 128 * TB200_PLAN_STATIC_MAX_EXPERTS)

#ifdef __cplusplus
extern "C" {
#endif

int tb200_moe_plan_static(const long long* expert_idx, const float* gates, int* es, float* gs,
                          int* cols, int* pos, int* seg_start, int* seg_count, int T, int k, int E,
                          int seg_align, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
