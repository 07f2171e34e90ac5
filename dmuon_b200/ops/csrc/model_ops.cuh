// Fused activation-side kernels of the decoder models (SwiGLU, rotary
// embedding, softmax cross-entropy with its gradient).  The reference ships no
// model code, so these have no counterpart there; they exist because the
// training step that carries the optimizer is otherwise bound by chains of
// single-op elementwise kernels over 8192 x 14336 activations.
//
// dtype codes are the ones of multi_tensor.cuh (0 bf16, 1 fp16, 2 fp32).
#pragma once
#include <stdint.h>

extern "C" {

// Gated MLP activation, act = 0: silu (SwiGLU), act = 1: gelu with the tanh approximation (GeGLU).
// out = act(gate) * up                                   (n elements each)
int dmuon_swiglu_fwd(const void* gate, const void* up, void* out, long long n, int act, int dtype, void* stream);

// d_gate = d_out * up * act'(gate) ;  d_up = d_out * act(gate)
// d_gate / d_up may alias gate / up (every element is read before it is written).
int dmuon_swiglu_bwd(const void* gate, const void* up, const void* d_out, void* d_gate, void* d_up,
                     long long n, int act, int dtype, void* stream);

// Rotary embedding in place on q [rows, q_heads, head_dim] and k [rows,
// k_heads, head_dim] (row = batch * seq + position; row strides in elements),
// rotate-half pairing (i, i + head_dim/2), tables cos/sin [seq, head_dim/2]
// fp32.  inverse != 0 applies the transposed rotation (the backward pass).
// head_dim must be a multiple of 16; k may be null.
int dmuon_rope_inplace(void* q, void* k, const float* cos_t, const float* sin_t,
                       long long rows, int seq, int q_heads, int k_heads, int head_dim,
                       long long q_row_stride, long long k_row_stride, int inverse, int dtype, void* stream);

// Softmax cross-entropy over rows of logits [rows, vocab] (row stride ld).
//   row_loss[r] = logsumexp(logits[r]) - logits[r, label[r]]        (0 where label[r] < 0)
//   logits[r, :] <- (softmax(logits[r]) - onehot(label[r])) * grad_scale   (in place; 0 where label[r] < 0)
// One pass for the statistics, one for the gradient; the second read of a row
// comes from L2.
int dmuon_softmax_xent_inplace(void* logits, const long long* labels, float* row_loss,
                               long long rows, int vocab, long long ld, float grad_scale, int dtype, void* stream);

}  // extern "C"
