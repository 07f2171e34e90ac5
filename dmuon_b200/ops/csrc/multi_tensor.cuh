// Argument blocks for the multi-tensor elementwise kernels.  Pointers travel in
// the kernel parameter space (no device-side tables to upload): one launch
// covers up to kMaxTensors tensors, blockIdx.y selects the tensor and the
// blocks of a row walk it with a grid-stride loop of 128-bit accesses.
#pragma once
#include <stdint.h>

extern "C" {

enum { DMUON_MAX_TENSORS = 48 };

// dtype codes shared with the Python side
enum { DMUON_BF16 = 0, DMUON_FP16 = 1, DMUON_FP32 = 2 };

// Muon prologue: momentum update, Nesterov mix, cast, sum of squares.
//   buf = mu * buf + g * gscale ;  u = nesterov ? g * gscale + mu * buf : buf
//   x = cast(u) ;  sumsq[slot] += sum(u^2)
struct DmuonPrologueArgs {
  const void* grad[DMUON_MAX_TENSORS];
  void* mom[DMUON_MAX_TENSORS];
  void* x[DMUON_MAX_TENSORS];
  long long numel[DMUON_MAX_TENSORS];
  int slot[DMUON_MAX_TENSORS];   // index into sumsq
  int n;
  int grad_dtype, mom_dtype, x_dtype;
  float mu;
  int nesterov;
  const float* gscale;           // optional device scalar (clip coefficient)
  float* sumsq;                  // zeroed by the caller
  // optional per-slot multiplier applied to the STORED x only (x = cast(u * xscale[slot]); sumsq stays
  // the sum of u^2): lets a 16-bit operand be written in the same pass with a scale known beforehand
  const float* xscale;
};

// scale[i] = 1 / (sqrt(sumsq[i]) + eps), scale2[i] = scale[i]^2
struct DmuonNormArgs {
  const float* sumsq;
  float* scale;
  float* scale2;
  int n;
  float eps;
};

// AdamW, decoupled weight decay, per-tensor step counts:
//   p *= 1 - lr*wd ; m = b1 m + (1-b1) g ; v = b2 v + (1-b2) g^2
//   p -= (lr / bc1) * m / (sqrt(v) / sqrt(bc2) + eps)
struct DmuonAdamWArgs {
  void* param[DMUON_MAX_TENSORS];
  const void* grad[DMUON_MAX_TENSORS];
  void* exp_avg[DMUON_MAX_TENSORS];
  void* exp_avg_sq[DMUON_MAX_TENSORS];
  void* publish[DMUON_MAX_TENSORS];   // optional bf16 copy of the new param
  long long numel[DMUON_MAX_TENSORS];
  float step_size[DMUON_MAX_TENSORS];     // lr / bc1
  float inv_sqrt_bc2[DMUON_MAX_TENSORS];  // 1 / sqrt(bc2)
  int n;
  int param_dtype, grad_dtype, state_dtype;
  float lr, beta1, beta2, eps, weight_decay;
  const float* gscale;                // optional device scalar (clip coefficient)
};

// Segmented sum of squares and in-place scaling for gradient clipping.
struct DmuonClipArgs {
  void* tensor[DMUON_MAX_TENSORS];
  long long numel[DMUON_MAX_TENSORS];
  int segment[DMUON_MAX_TENSORS];
  int dtype[DMUON_MAX_TENSORS];
  int n;
  float* seg_sumsq;                   // [num_segments], accumulated with atomics
  const float* seg_coef;              // [num_segments], used by the scale kernel
};

// dst = cast(src * scale[slot]) ; generic multi-tensor cast/copy.
struct DmuonCastArgs {
  const void* src[DMUON_MAX_TENSORS];
  void* dst[DMUON_MAX_TENSORS];
  long long numel[DMUON_MAX_TENSORS];
  int slot[DMUON_MAX_TENSORS];
  int n;
  int src_dtype, dst_dtype;
  const float* scale;                 // optional per-slot device scales
};

int dmuon_muon_prologue(const DmuonPrologueArgs* a, void* stream);
int dmuon_norm_scales(const DmuonNormArgs* a, void* stream);
int dmuon_adamw(const DmuonAdamWArgs* a, void* stream);
int dmuon_clip_sumsq(const DmuonClipArgs* a, void* stream);
int dmuon_clip_scale(const DmuonClipArgs* a, void* stream);
int dmuon_cast(const DmuonCastArgs* a, void* stream);
}
