// Tensor-parallel gather and scatter of the Muon path over peer memory.
//
// A matrix that is sharded over T tensor-parallel ranks is orthogonalised as a
// whole by ONE of them (its TP owner).  These two kernels move the shards
// without a collective and without an intermediate concatenated copy:
//
//   gather + prologue   the owner reads every rank's reduced gradient shard
//                       (plain loads through the peer mapping of that rank's
//                       symmetric buffer) and writes momentum, Nesterov mix,
//                       cast operand and sum of squares straight into the
//                       rows / columns the shard occupies in the FULL matrix
//   pull + apply        every rank reads its slice of the owner's pre-scaled
//                       update (again through the peer mapping) and applies
//                       w = w * decay + slice to its master shard
//
// The shard side of each job is contiguous (rows x cols); the full-matrix side
// is a 2-D slice with a row pitch.  Ordering against the other ranks is done by
// the flag kernels of peer_sm100.cuh, launched around these.
//
// Replaces the reference's NCCL gather + torch.cat and NCCL scatter + mul_/add_
// (dmuon/_backends/fsdp2/group.py:1376-1521, :1536-1655).
#pragma once
#include <stdint.h>

#include "multi_tensor.cuh"

extern "C" {

// For job t:  g = src[t][r * cols + c]                      (shard, contiguous)
//   buf = mu * buf + g * gscale ; u = nesterov ? g * gscale + mu * buf : buf      (buf = mom slice, may be null)
//   x[r * pitch + c] = cast(u * xscale[slot]) ; sumsq[slot] += sum(u^2)
struct DmuonTpGatherArgs {
  const void* src[DMUON_MAX_TENSORS];
  void* mom[DMUON_MAX_TENSORS];       // first element of the slice inside the full momentum, or null
  void* x[DMUON_MAX_TENSORS];         // first element of the slice inside the full operand
  int rows[DMUON_MAX_TENSORS];
  int cols[DMUON_MAX_TENSORS];
  long long pitch[DMUON_MAX_TENSORS]; // row pitch of the mom / x slices, elements
  int slot[DMUON_MAX_TENSORS];
  int n;
  int src_dtype, mom_dtype, x_dtype;
  float mu;
  int nesterov;
  const float* gscale;
  float* sumsq;                       // may be null
  const float* xscale;                // may be null
};

// For job t:  dst[t][r * cols + c] = dst * decay[t] + src[t][r * pitch + c]
// dst: master shard (contiguous, dst_dtype); src: fp32 slice of the owner's full update.
struct DmuonTpApplyArgs {
  const float* src[DMUON_MAX_TENSORS];
  void* dst[DMUON_MAX_TENSORS];
  int rows[DMUON_MAX_TENSORS];
  int cols[DMUON_MAX_TENSORS];
  long long pitch[DMUON_MAX_TENSORS];
  float decay[DMUON_MAX_TENSORS];
  int n;
  int dst_dtype;
};

int dmuon_tp_gather_prologue(const DmuonTpGatherArgs* a, void* stream);
int dmuon_tp_apply_delta(const DmuonTpApplyArgs* a, void* stream);
}
