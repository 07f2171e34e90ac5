// Forward publish fused into its first consumer:  Y = X W^T  where W is pulled
// from its owner's GPU by the same kernel that multiplies with it.
#pragma once
#include <stdint.h>

extern "C" {

struct DmuonPullLinearArgs {
  const void* X;          // [M, K] bf16, row pitch ldx (multiple of 8)
  void* Y;                // [M, N] bf16, row pitch ldy (multiple of 8)
  void* W_local;          // [N, K] bf16 contiguous (pitch K): this GPU's slot of the publish arena
  const void* W_remote;   // the owner's slot through its peer mapping, or null when W_local is already current
  int M, N, K;
  long long ldx, ldy;
  int* tile_ready;        // [ceil(N / 256)] ints, zeroed by the caller before the launch (scratch)
  const int* pub_flag;    // local flag word the owner sets when its slot is published (may be null)
  int pub_want;
  long long budget_cycles;   // budget of the wait on pub_flag
  int* status;
  int max_ctas;           // 0 = one CTA per SM
};

// Returns 0 or an error code (negative: bad argument; positive: cudaError_t).
int dmuon_pull_linear_sm100(const DmuonPullLinearArgs* args, void* stream);
}
