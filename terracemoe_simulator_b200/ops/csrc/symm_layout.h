// Layout of the symmetric arena shared by the ranks of one expert-parallel group.
//
// Every rank allocates one device buffer with the SAME section offsets and maps every peer's
// buffer (CUDA IPC over NVLink / NVSwitch).  Kernels address a peer's section as
// `peer[r] + offset`.  Data moves with plain peer stores and loads issued inside the kernels;
// completion is signalled with epoch-valued flag words (st.release.sys / ld.acquire.sys),
// which only ever grow, so no flag is reset between steps.
//
// Has no counterpart in the reference, whose transport is torch.distributed all_to_all_single;
// its closest relative is the one-sided put benchmark (tools/onesided/bench_onesided.py).
#pragma once

#define TB200_MAX_WORLD 16
#define TB200_PLAN_CHUNKS 128

enum Tb200FlagKind {
  FK_COUNTS = 0,   // [src]    src's expert histogram has landed in counts_all[src]
  FK_HOPA,         // [group]  forward Hop A rows of the source in that group have landed
  FK_DATA,         // [rank]   all rows that rank pushes into my expert input have landed
  FK_OUT,          // [rank]   that owner's expert output buffer is complete
  FK_RED,          // [group]  that group's representative finished its reduced rows
  FK_B_HOPA,       // backward twins
  FK_B_DATA,
  FK_B_DG,
  FK_B_OUT,
  FK_B_RED,
  FK_NUM
};

struct Tb200Arena {
  unsigned long long peer[TB200_MAX_WORLD];  // arena base address of every rank (own included)
  long long off_counts_all;  // int   [W][E]
  long long off_flags;       // int   [FK_NUM][TB200_MAX_WORLD]
  long long off_xin;         // bf16  [cap_rows][H]   expert-sorted GEMM input (dispatch target)
  long long off_yout;        // bf16  [cap_rows][H]   expert output (combine source)
  long long off_dout;        // bf16  [cap_rows][H]   backward: gradient of yout
  long long off_dxs;         // bf16  [cap_rows][H]   backward: gradient of xin
  long long off_ha_rows;     // bf16  [N_g * T][H]    forward Hop A arrival rows
  long long off_ha_hdr;      // int   [N_g * T][3q]   per arrival row: pos[q], expert[q], gate[q]
  long long off_red;         // bf16  [N_g * T][H]    gate-weighted per-(token, group) sums
  long long off_hb_rows;     // bf16  [N_g * T][H]    backward Hop A arrival rows (dy)
  long long off_dred;        // bf16  [N_g * T][H]    backward reduced rows
  long long off_dgate;       // float [N_g * T][q]    backward gate gradients at the arrival rank
  int world, rank, n_experts, epr, rpn, n_nodes;
  int tokens_cap, top_k, groups_m, q, hidden, cap_rows;
};
