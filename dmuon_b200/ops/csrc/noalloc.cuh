// Allocation-free entry point of the symmetric (Gram / SYRK) product.
//
// This entry point has no counterpart in the reference implementation.
//
// Who it is for: code that wants  D = alpha * X X^T + diag * I  (or X^T X) from
// the tcgen05 kernel but is not in a position to obtain device memory for the
// kernel's bookkeeping -- for example a plugin that lives inside another
// runtime's memory pool and must not call cudaMalloc behind its back, a
// real-time control loop where an allocation (an implicit device
// synchronisation and an unbounded latency) is not acceptable, or a C host
// without PyTorch's caching allocator.  The regular entry point
// (dmuon_gemm_sm100) expects the caller to supply a tile table and a status
// word in device memory; here both live in a fixed array inside the library.
//
// The scratch is one file-scope `static __device__` array of
// DMUON_NOALLOC_SCRATCH_BYTES (about 257 KiB).  Every GPU on which the library
// runs a kernel holds that array from module load until the process exits.
//
// Limits and rules
//   * at most DMUON_NOALLOC_MAX_TILES (16384) output tiles per matrix; with
//     128 x 256 tiles that is any M up to 32640 (255 rows of tiles, exactly
//     16384 tiles).  Larger problems are rejected with
//     DMUON_NOALLOC_E_TOO_LARGE and nothing is launched.
//   * with batch > 1 both batch strides must be non-zero (every matrix needs
//     its own output); otherwise DMUON_NOALLOC_E_BAD_ARGUMENT.
//   * the first call on a device looks up the array's device address
//     (cudaGetSymbolAddress with that device current) and sets the kernel's
//     shared-memory attribute.  Make that first call outside any stream
//     capture; later calls only enqueue two kernels and a 256-byte memset.
//   * every call reuses the same array: the tile table is rewritten and the
//     status word cleared at the start of each call, in stream order.  Two calls
//     whose kernels can overlap on the GPU (different streams, no dependency)
//     race on it -- serialise them.
//   * no cudaMalloc / cudaFree / library allocation is made by these functions.
#pragma once

#ifdef __cplusplus
extern "C" {
#endif

enum {
  DMUON_NOALLOC_MAX_TILES = 16384,
  DMUON_NOALLOC_HEADER_BYTES = 256,
  DMUON_NOALLOC_SCRATCH_BYTES = 256 + 16384 * 16,
};

enum {
  DMUON_NOALLOC_OK = 0,
  DMUON_NOALLOC_E_BAD_ARGUMENT = -1,   // null pointer, misaligned pointer, pitch not a multiple of 8 elements
  DMUON_NOALLOC_E_TOO_LARGE = -22,     // more than DMUON_NOALLOC_MAX_TILES tiles per matrix
  DMUON_NOALLOC_E_SYMBOL = -30,        // cudaGetSymbolAddress failed on this device
};

// D[b] = alpha * X[b] X[b]^T + diag * I      (x_mn_major == 0, X stored [M, K], K contiguous)
// D[b] = alpha * X[b]^T X[b] + diag * I      (x_mn_major == 1, X stored [K, M], M contiguous)
// X and D are bf16 (is_fp16 == 0) or fp16 (is_fp16 == 1); ldx / ldd are row
// pitches in elements (multiples of 8), strides are per-matrix distances in
// elements.  Only tiles touching the lower triangle are computed; the result
// is stored as a full symmetric matrix.  Returns 0, one of the negative codes
// above, or a positive value: the cudaError_t of a failed launch or memset
// (dmuon_syrk_noalloc_strerror gives CUDA's text for those).
int dmuon_syrk_noalloc(const void* X, void* D, int M, int K, int batch, long long ldx, long long ldd,
                       long long strideX, long long strideD, int is_fp16, int x_mn_major, float alpha,
                       float diag, void* stream);

// Synchronises `stream` and returns the status word of the last call on the
// current device: 0, or the code of the bounded wait that ran out.
int dmuon_syrk_noalloc_status(void* stream);

// Text for a return code of dmuon_syrk_noalloc.
const char* dmuon_syrk_noalloc_strerror(int code);

#ifdef __cplusplus
}
#endif
