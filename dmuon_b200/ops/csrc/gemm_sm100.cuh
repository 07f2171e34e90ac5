// Argument block shared by the host launcher and the tcgen05 GEMM kernel.
#pragma once
#include <stdint.h>

extern "C" {

// One batched product  D[b] = alpha * A[b] * B[b]^T + beta * C[b] + diag * I.
//
// A supplies M x K, B supplies N x K.  "K-major" means the operand is stored
// with K contiguous (row-major [M, K] / [N, K]); "MN-major" means it is stored
// with M (or N) contiguous (row-major [K, M] / [K, N]).  lda / ldb are the row
// pitches of the stored matrices in elements and must be multiples of 8.
struct DmuonGemmArgs {
  const void* A;
  const void* B;
  long long lda, ldb;          // row pitch of the stored operand, elements
  long long strideA, strideB;  // batch stride, elements (multiple of 8)
  int a_mn_major, b_mn_major;
  int ab_fp16;                 // operands are fp16 (1) or bf16 (0)

  int M, N, K, batch;

  // Tile list: tiles_per_batch entries of (row_tile, col_tile, flags, 0) with
  // row_tile in units of 128 rows and col_tile in units of BN columns.
  // flags bit 0: also store the transposed tile (symmetric output).
  const int* tile_tab;
  int tiles_per_batch;
  int bn;                      // 128 or 256

  float alpha, beta, diag;
  const float* alpha_vec;      // optional per-batch device multiplier of alpha
  // Either flat base pointers with a batch stride, or per-batch pointer tables
  // (device arrays of `batch` pointers) when *_tab is not null.
  const void* C;
  void* D;
  void* D2;                    // optional bf16 copy of D
  const void* const* C_tab;
  void* const* D_tab;
  void* const* D2_tab;
  long long ldc, ldd, ldd2;
  long long strideC, strideD, strideD2;
  int out_kind;                // C and D element type: 0 bf16, 1 fp16, 2 fp32

  // Optional readiness flags for B column tiles (used when another part of the
  // same kernel is still copying B into local memory): the producer waits
  // until b_ready[col_tile] >= b_ready_epoch before it loads that tile.
  const int* b_ready;
  int b_ready_epoch;

  int* status;                 // device int; set non-zero when a wait ran out
  int max_ctas;                // 0 = one CTA per SM
  // 1: run on CTA pairs (tcgen05 cta_group::2).  The tile list is then in units
  // of 256 rows x 256 columns and bn must be 256.
  // 2: run on clusters of two CTA pairs that share their A rows.  Each entry of
  // the tile list then names two 256 x 256 tiles: x = m0 | m1 << 16,
  // y = n0 | n1 << 16, z bit 0 / 1 = store tile 0 / 1 transposed as well,
  // bit 2 = both tiles cover the same rows (m0 == m1; A is then loaded once per
  // cluster), bit 3 = tile 1 is a filler whose result is not stored.
  int two_cta;
  // 1: D2 / D2_tab hold addresses in the NVSwitch MULTICAST mapping of a symmetric
  // buffer: the bf16 copy is written with multimem.st and lands at the same offset
  // of every rank's buffer (the owner's publish becomes part of the product that
  // computes the new weights).  Needs N, ldd2 and strideD2 multiples of 8, 16-byte
  // aligned bases (every table entry too), and a tile list without mirror flags.
  int d2_multimem;
};

// Returns 0 on success, a cudaError_t / negative code otherwise.
int dmuon_gemm_sm100(const DmuonGemmArgs* args, void* stream);

// Clusters of four CTAs that the quad kernel can keep resident on the current
// device (0 when the query fails; the quad path is then unavailable).
int dmuon_gemm_quad_max_clusters(void);

// Number of launches of kernels from this library since load (host counter).
long long dmuon_launch_count(void);
}
