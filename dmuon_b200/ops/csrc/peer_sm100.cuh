// Kernels that move dedicated-parameter data between GPUs with plain peer
// loads and stores on NVSwitch-mapped symmetric buffers, or with multimem
// reduce-loads / stores on their multicast mapping (no library collective, no
// TMA), fused with the adjacent elementwise work.
#pragma once
#include <stdint.h>

#include "multi_tensor.cuh"

extern "C" {

enum { DMUON_MAX_PEERS = 8 };

// flags[peer][slot] = value on every listed peer (release, system scope).
struct DmuonSignalArgs {
  int* peer_flags[DMUON_MAX_PEERS];   // base of every peer's flag array (peer-mapped)
  int world;
  int slot;
  int value;
};

// Wait until local_flags[first + i] >= want for i in [0, count).
struct DmuonWaitArgs {
  const int* local_flags;
  int first, count, want;
  long long budget_cycles;
  int* status;                        // set to 4 when the budget ran out
};

// Reduce-to-owner fused with the Muon prologue.  For tensor t the gradient is
//   g = scale * sum_r  peer_base[r][offset[t] + i]       (fixed rank order, fp32)
// followed by   mom = mu*mom + g ; u = nesterov ? g + mu*mom : mom
// (or u = g when mom[t] is null), x = cast(u), sumsq[slot] += sum(u^2).
// Every block first waits (bounded) until ready_flags[r] >= ready_want for all
// ranks, i.e. until every rank has finished writing its gradient arena.
struct DmuonPeerPrologueArgs {
  const void* peer_base[DMUON_MAX_PEERS];
  int world;
  float scale;
  long long offset[DMUON_MAX_TENSORS];   // elements into the arena
  void* mom[DMUON_MAX_TENSORS];
  void* x[DMUON_MAX_TENSORS];
  long long numel[DMUON_MAX_TENSORS];
  int slot[DMUON_MAX_TENSORS];
  int n;
  int grad_dtype, mom_dtype, x_dtype;
  float mu;
  int nesterov;
  const float* gscale;
  float* sumsq;
  const int* ready_flags;
  int ready_want;
  long long budget_cycles;
  int* status;
  int max_blocks_per_tensor;             // 0 = default
  const float* xscale;                   // optional per-slot multiplier of the stored x (see DmuonPrologueArgs)
};

// Pull: dst[t] (local) = src[t] (on the owner, peer-mapped) after the owner's
// flag reached `want`.  Sizes in bytes, multiples of 16, 16-byte aligned.
struct DmuonPullArgs {
  const void* src[DMUON_MAX_TENSORS];
  void* dst[DMUON_MAX_TENSORS];
  long long nbytes[DMUON_MAX_TENSORS];
  int flag_slot[DMUON_MAX_TENSORS];      // local flag to wait on for this copy
  int n;
  const int* local_flags;
  int want;
  long long budget_cycles;
  int* status;
  int blocks_per_tensor;                 // 0 = default
};

int dmuon_signal_peers(const DmuonSignalArgs* a, void* stream);
int dmuon_wait_flags(const DmuonWaitArgs* a, void* stream);
int dmuon_peer_prologue(const DmuonPeerPrologueArgs* a, void* stream);
int dmuon_peer_pull(const DmuonPullArgs* a, void* stream);

// Sum of a few scalars over all ranks inside one tiny kernel (gradient-clip norms):
// every rank writes its values into its own symmetric scratch row, raises its flag
// on every peer, waits (bounded) for all peers' flags and adds up the rows in rank
// order, so every rank gets bit-identical sums.  Optionally turns the sums into clip
// coefficients min(1, max_norm / (sqrt(sum) + 1e-6)).
// Scratch per rank: vals float[2][DMUON_SCALAR_MAX], flags int[2][DMUON_MAX_PEERS];
// the slot parity is epoch & 1 and epochs must increase by one per call on every rank.
enum { DMUON_SCALAR_MAX = 8 };
struct DmuonScalarAllreduceArgs {
  float* peer_vals[DMUON_MAX_PEERS];
  int* peer_flags[DMUON_MAX_PEERS];
  int world, rank, n, epoch;
  const float* local;     // n partial sums on this rank
  float* out;             // n global sums
  float* coef;            // optional: n clip coefficients
  float max_norm;
  long long budget_cycles;
  int* status;
};
int dmuon_scalar_allreduce(const DmuonScalarAllreduceArgs* a, void* stream);

// NVSwitch multicast transfers (NVLS).  `mc` addresses lie in the multicast
// mapping of a symmetric buffer: the same offset of every rank's buffer.
//   mode 0  reduce:     dst[t] (local)       = sum over ranks of mc_src[t], formed in the switch
//                       (element type `dtype`; 16-bit types accumulate in fp32 and round once)
//   mode 1  broadcast:  every rank's mc_dst[t] = src[t] (local)
// Sizes in bytes, multiples of 16; all addresses 16-byte aligned.  The caller
// orders these against the other ranks with the flag kernels above.
struct DmuonMulticastArgs {
  const void* src[DMUON_MAX_TENSORS];
  void* dst[DMUON_MAX_TENSORS];
  long long nbytes[DMUON_MAX_TENSORS];
  int n;
  int mode;
  int dtype;                             // DMUON_FP32 / DMUON_BF16 / DMUON_FP16 (mode 0 only)
  int blocks_per_tensor;                 // 0 = default
};
int dmuon_multicast_copy(const DmuonMulticastArgs* a, void* stream);

// Copy-engine transfer (cudaMemcpyAsync, cudaMemcpyDefault); dst / src may be peer mappings.
int dmuon_copy_async(void* dst, const void* src, long long nbytes, void* stream);
}
