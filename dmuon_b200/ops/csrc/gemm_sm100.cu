// Batched tcgen05 GEMM for sm_100a:  D = alpha * A * B^T + beta * C + diag * I.
//
// One persistent CTA per SM, 192 threads in three roles:
//   warp 0      TMA producer: streams 128 x 64 (A) and BN x 64 (B) bf16/fp16
//               tiles into a ring of 128-byte-swizzled shared-memory stages
//   warp 1      MMA issuer: one thread issues tcgen05.mma (128 x BN x 16) into
//               one of two TMEM accumulators and commits mbarriers
//   warps 2-5   epilogue: tcgen05.ld the finished accumulator, apply
//               alpha/beta/diag, cast, store (and store the transposed tile
//               for symmetric outputs) while the next tile's MMAs already run
//
// The tile list is data (a table built by the host), so the same kernel runs
// dense products, lower-triangle-only symmetric products (Gram / SYRK) and any
// batch of them.  Operands may be K-major or MN-major, so X X^T, X^T X, Q X and
// X Q all run without a transposed copy of X.
//
// Covers the roles of the reference's symmetric-rank-k kernel
// (dmuon/kernels/syrk_sm80.py:183-399, mma.sync + cp.async) and of the
// library GEMMs its Newton-Schulz calls (dmuon/optim/newton_schulz.py:381-444).
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <atomic>
#include <mutex>

#include "gemm_sm100.cuh"
#include "ptx_sm100.cuh"

namespace dmuon {

constexpr int BM = 128;
constexpr int BK = 64;       // 64 two-byte elements = one 128-byte swizzle row
constexpr int UMMA_K = 16;
constexpr int kThreads = 192;
constexpr int kBlockBytes = 64 * 128;  // one 64 x 64 swizzled block (MN-major staging)

template <int BN>
struct Cfg {
  static constexpr int kStages = (BN == 256) ? 4 : 6;
  static constexpr int kABytes = BM * BK * 2;
  static constexpr int kBBytes = BN * BK * 2;
  static constexpr int kStageBytes = kABytes + kBBytes;
  static constexpr int kTmemCols = 2 * BN;
  static constexpr int kBarBytes = 256;
  static constexpr int kSmemBytes = kStages * kStageBytes + kBarBytes + 1024;
};

struct KParams {
  int M, N, K, batch;
  const int4* tile_tab;
  int tiles_per_batch;
  int a_mn_major, b_mn_major, ab_fp16;
  float alpha, beta, diag;
  const float* alpha_vec;
  const void* C;
  void* D;
  void* D2;
  const void* const* C_tab;
  void* const* D_tab;
  void* const* D2_tab;
  long long ldc, ldd, ldd2;
  long long strideC, strideD, strideD2;
  int out_kind;
  const int* b_ready;
  int b_ready_epoch;
  int* status;
  int d2_multimem;
};

// ---- epilogue helpers -------------------------------------------------------

template <typename T>
__device__ __forceinline__ float to_f32(T x);
template <>
__device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 x) { return __bfloat162float(x); }
template <>
__device__ __forceinline__ float to_f32<__half>(__half x) { return __half2float(x); }
template <>
__device__ __forceinline__ float to_f32<float>(float x) { return x; }

template <typename T>
__device__ __forceinline__ T from_f32(float x);
template <>
__device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float x) { return __float2bfloat16_rn(x); }
template <>
__device__ __forceinline__ __half from_f32<__half>(float x) { return __float2half_rn(x); }
template <>
__device__ __forceinline__ float from_f32<float>(float x) { return x; }

template <typename T>
__device__ __forceinline__ void load_row32(const T* src, float (&c)[32], int nvalid, bool vec) {
  if (vec && nvalid == 32) {
    constexpr int kPerVec = 16 / sizeof(T);
    const uint4* s4 = reinterpret_cast<const uint4*>(src);
#pragma unroll
    for (int i = 0; i < 32 / kPerVec; ++i) {
      uint4 raw = s4[i];
      const T* e = reinterpret_cast<const T*>(&raw);
#pragma unroll
      for (int j = 0; j < kPerVec; ++j) c[i * kPerVec + j] = to_f32<T>(e[j]);
    }
  } else {
#pragma unroll
    for (int j = 0; j < 32; ++j) c[j] = (j < nvalid) ? to_f32<T>(src[j]) : 0.f;
  }
}

template <typename T>
__device__ __forceinline__ void store_row32(T* dst, const float (&v)[32], int nvalid, bool vec) {
  if (vec && nvalid == 32) {
    constexpr int kPerVec = 16 / sizeof(T);
    uint4* d4 = reinterpret_cast<uint4*>(dst);
#pragma unroll
    for (int i = 0; i < 32 / kPerVec; ++i) {
      uint4 raw;
      T* e = reinterpret_cast<T*>(&raw);
#pragma unroll
      for (int j = 0; j < kPerVec; ++j) e[j] = from_f32<T>(v[i * kPerVec + j]);
      d4[i] = raw;
    }
  } else {
#pragma unroll
    for (int j = 0; j < 32; ++j)
      if (j < nvalid) dst[j] = from_f32<T>(v[j]);
  }
}

// bf16 row chunk to a multicast address: every rank's copy of the buffer
// receives it (multimem.st through the switch).  The host only selects this
// path when every row start is 16-byte aligned and N is a multiple of 8.
__device__ __forceinline__ void store_row32_multicast(__nv_bfloat16* mc_dst, const float (&v)[32], int nvalid) {
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    if (i * 8 < nvalid) {
      uint4 raw;
      __nv_bfloat16* e = reinterpret_cast<__nv_bfloat16*>(&raw);
#pragma unroll
      for (int j = 0; j < 8; ++j) e[j] = __float2bfloat16_rn(v[i * 8 + j]);
      multimem_st_16B(mc_dst + i * 8, raw);
    }
  }
}

template <typename T>
__device__ __forceinline__ void store_col32(T* dst, long long ld, const float (&v)[32], int nvalid) {
  // dst points at element (col0, row) of the transposed tile; consecutive
  // lanes hold consecutive rows, so each store instruction is contiguous
  // across the warp.
#pragma unroll
  for (int j = 0; j < 32; ++j)
    if (j < nvalid) dst[static_cast<long long>(j) * ld] = from_f32<T>(v[j]);
}

template <typename T>
__device__ __forceinline__ void epilogue_chunk(const KParams& p, const T* Cb, T* Db,
                                               __nv_bfloat16* D2b, float (&v)[32], int row, int col0,
                                               bool mirror) {
  const int nvalid = min(32, p.N - col0);
  const bool row_ok = row < p.M;
  if (p.beta != 0.f && row_ok) {
    float c[32];
    const T* src = Cb + static_cast<long long>(row) * p.ldc + col0;
    const bool vec = ((p.ldc * sizeof(T)) % 16 == 0) && ((reinterpret_cast<uintptr_t>(Cb) & 15) == 0);
    load_row32<T>(src, c, nvalid, vec);
#pragma unroll
    for (int j = 0; j < 32; ++j) v[j] = fmaf(p.beta, c[j], v[j]);
  }
  if (p.diag != 0.f) {
#pragma unroll
    for (int j = 0; j < 32; ++j)
      if (col0 + j == row) v[j] += p.diag;
  }
  if (!row_ok) return;
  {
    T* dst = Db + static_cast<long long>(row) * p.ldd + col0;
    const bool vec = ((p.ldd * sizeof(T)) % 16 == 0) && ((reinterpret_cast<uintptr_t>(Db) & 15) == 0);
    store_row32<T>(dst, v, nvalid, vec);
    if (mirror) store_col32<T>(Db + static_cast<long long>(col0) * p.ldd + row, p.ldd, v, nvalid);
  }
  if (D2b != nullptr && p.d2_multimem) {
    store_row32_multicast(D2b + static_cast<long long>(row) * p.ldd2 + col0, v, nvalid);
  } else if (D2b != nullptr) {
    __nv_bfloat16* dst = D2b + static_cast<long long>(row) * p.ldd2 + col0;
    const bool vec = ((p.ldd2 * 2) % 16 == 0) && ((reinterpret_cast<uintptr_t>(D2b) & 15) == 0);
    store_row32<__nv_bfloat16>(dst, v, nvalid, vec);
    if (mirror)
      store_col32<__nv_bfloat16>(D2b + static_cast<long long>(col0) * p.ldd2 + row, p.ldd2, v, nvalid);
  }
}

// ---- kernel -------------------------------------------------------------------

template <int BN>
__global__ void __launch_bounds__(kThreads, 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                    const KParams p) {
  using C = Cfg<BN>;
  constexpr int S = C::kStages;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* sA = smem;
  uint8_t* sB = smem + S * C::kABytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + S * C::kStageBytes);
  const uint32_t full0 = smem_u32(bars);
  const uint32_t empty0 = smem_u32(bars + S);
  const uint32_t tfull0 = smem_u32(bars + 2 * S);
  const uint32_t tempty0 = smem_u32(bars + 2 * S + 2);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * S + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < S; ++s) {
      mbar_init(full0 + 8 * s, 1);
      mbar_init(empty0 + 8 * s, 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(tfull0 + 8 * a, 1);
      mbar_init(tempty0 + 8 * a, 4);
    }
    *abort_flag = 0;
    fence_barrier_init();
    fence_proxy_async_smem();
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(tmem_slot), C::kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  const int total_tiles = p.tiles_per_batch * p.batch;
  const int num_kb = (p.K + BK - 1) / BK;
  int fail_code = 0;

  if (warp == 0) {
    if (lane == 0) {
      // ---------------- TMA producer ----------------
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int t = blockIdx.x; ok && t < total_tiles; t += gridDim.x) {
        const int b = t / p.tiles_per_batch;
        const int4 e = p.tile_tab[t - b * p.tiles_per_batch];
        const int m0 = e.x * BM;
        const int n0 = e.y * BN;
        if (p.b_ready != nullptr) {
          if (!wait_flag_ge_gpu(p.b_ready + e.y, p.b_ready_epoch, kWaitBudgetCycles)) {
            *abort_flag = 1;
            fail_code = kStatusTimeoutPeerFlag;
            break;
          }
        }
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait_bounded(empty0 + 8 * stage, phase ^ 1u, abort_flag)) {
            ok = false;
            fail_code = kStatusTimeoutProducer;
            break;
          }
          const uint32_t fb = full0 + 8 * stage;
          mbar_arrive_expect_tx(fb, C::kStageBytes);
          const uint32_t a_dst = smem_u32(sA + stage * C::kABytes);
          const uint32_t b_dst = smem_u32(sB + stage * C::kBBytes);
          if (!p.a_mn_major) {
            tma_load_3d(a_dst, &tmA, fb, kb * BK, m0, b);
          } else {
#pragma unroll
            for (int mb = 0; mb < BM / 64; ++mb)
              tma_load_3d(a_dst + mb * kBlockBytes, &tmA, fb, m0 + 64 * mb, kb * BK, b);
          }
          if (!p.b_mn_major) {
            tma_load_3d(b_dst, &tmB, fb, kb * BK, n0, b);
          } else {
#pragma unroll
            for (int nb = 0; nb < BN / 64; ++nb)
              tma_load_3d(b_dst + nb * kBlockBytes, &tmB, fb, n0 + 64 * nb, kb * BK, b);
          }
          if (++stage == S) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      // ---------------- MMA issuer ----------------
      const uint32_t idesc =
          make_idesc_f16(BM, BN, p.ab_fp16 != 0, p.a_mn_major != 0, p.b_mn_major != 0);
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      for (int t = blockIdx.x; ok && t < total_tiles; t += gridDim.x) {
        if (!mbar_wait_bounded(tempty0 + 8 * acc, acc_phase ^ 1u, abort_flag)) {
          fail_code = kStatusTimeoutMma;
          break;
        }
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(acc * BN);
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait_bounded(full0 + 8 * stage, phase, abort_flag)) {
            ok = false;
            fail_code = kStatusTimeoutMma;
            break;
          }
          tc_fence_after_sync();
          const uint32_t a_base = smem_u32(sA + stage * C::kABytes);
          const uint32_t b_base = smem_u32(sB + stage * C::kBBytes);
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            // K-major: 8-row groups are 1024 B apart, a K step of 16 elements is
            // 32 B inside the swizzle row.  MN-major: 64-wide blocks are 8192 B
            // apart, 8 K-rows are 1024 B apart, a K step of 16 rows is 2048 B.
            const uint64_t adesc = p.a_mn_major
                                       ? make_smem_desc_sw128(a_base + k * 2048, kBlockBytes, 1024)
                                       : make_smem_desc_sw128(a_base + k * 32, 16, 1024);
            const uint64_t bdesc = p.b_mn_major
                                       ? make_smem_desc_sw128(b_base + k * 2048, kBlockBytes, 1024)
                                       : make_smem_desc_sw128(b_base + k * 32, 16, 1024);
            umma_f16_ss(d_tmem, adesc, bdesc, idesc, (kb | k) != 0 ? 1u : 0u);
          }
          umma_commit(empty0 + 8 * stage);
          if (++stage == S) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (!ok) break;
        umma_commit(tfull0 + 8 * acc);
        acc ^= 1;
        if (acc == 0) acc_phase ^= 1u;
      }
    }
  } else {
    // ---------------- epilogue (warps 2..5) ----------------
    const int q = warp & 3;  // TMEM lane quarter this warp may read
    int acc = 0;
    uint32_t acc_phase = 0;
    for (int t = blockIdx.x; t < total_tiles; t += gridDim.x) {
      const int b = t / p.tiles_per_batch;
      const int4 e = p.tile_tab[t - b * p.tiles_per_batch];
      const int m0 = e.x * BM;
      const int n0 = e.y * BN;
      const bool mirror = (e.z & 1) != 0;
      if (!mbar_wait_bounded(tfull0 + 8 * acc, acc_phase, abort_flag)) {
        fail_code = kStatusTimeoutEpilogue;
        break;
      }
      tc_fence_after_sync();
      const int row = m0 + q * 32 + lane;
      const char* Cb = reinterpret_cast<const char*>(p.C_tab ? p.C_tab[b] : p.C);
      char* Db = reinterpret_cast<char*>(p.D_tab ? p.D_tab[b] : p.D);
      __nv_bfloat16* D2b = reinterpret_cast<__nv_bfloat16*>(p.D2_tab ? p.D2_tab[b] : p.D2);
      const int esz = (p.out_kind == 2) ? 4 : 2;
      if (!p.C_tab && Cb) Cb += static_cast<long long>(b) * p.strideC * esz;
      if (!p.D_tab) Db += static_cast<long long>(b) * p.strideD * esz;
      if (!p.D2_tab && D2b) D2b += static_cast<long long>(b) * p.strideD2;
      const float alpha = p.alpha_vec ? p.alpha * p.alpha_vec[b] : p.alpha;
      for (int c = 0; c < BN; c += 32) {
        const int col0 = n0 + c;
        if (col0 >= p.N) break;  // uniform across the warp
        uint32_t r[32];
        tmem_ld_32x32(tmem_base + (static_cast<uint32_t>(q * 32) << 16) +
                          static_cast<uint32_t>(acc * BN + c),
                      r);
        tmem_ld_wait();
        float v[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] = alpha * __uint_as_float(r[j]);
        if (p.out_kind == 0) {
          epilogue_chunk<__nv_bfloat16>(p, reinterpret_cast<const __nv_bfloat16*>(Cb),
                                        reinterpret_cast<__nv_bfloat16*>(Db), D2b, v, row, col0, mirror);
        } else if (p.out_kind == 1) {
          epilogue_chunk<__half>(p, reinterpret_cast<const __half*>(Cb), reinterpret_cast<__half*>(Db),
                                 D2b, v, row, col0, mirror);
        } else {
          epilogue_chunk<float>(p, reinterpret_cast<const float*>(Cb), reinterpret_cast<float*>(Db), D2b,
                                v, row, col0, mirror);
        }
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(tempty0 + 8 * acc);
      acc ^= 1;
      if (acc == 0) acc_phase ^= 1u;
    }
  }

  // ---------------- teardown ----------------
  tc_fence_before_sync();
  __syncthreads();
  if (*abort_flag) {
    if (fail_code != 0 && p.status != nullptr) atomicCAS(p.status, 0, fail_code);
    // Give bulk copies that may still be in flight time to land before the
    // shared memory of this CTA is handed to another one.
    for (int i = 0; i < 64; ++i) __nanosleep(2000);
    __syncthreads();
  }
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, C::kTmemCols);
  }
}

// ---- CTA-pair kernel (tcgen05 cta_group::2) -------------------------------------
//
// Two CTAs of a cluster share one 256 x 256 output tile.  Each CTA stages its
// own 128 rows of A and its own 128 of the 256 B columns, the leader (even
// rank) issues 256 x 256 x 16 MMAs that read both CTAs' shared memory, and each
// CTA ends up with its 128 rows of the accumulator in its own TMEM.  Per
// k-block a CTA now pulls 32 KB from L2 for the work that took 48 KB with the
// single-CTA kernel -- the L2 feed is what limits that kernel (ncu: tensor pipe
// 75 % busy, 16 TB/s from L2).  No multicast: every load is issued by the CTA
// that consumes it; only barrier signals cross the pair.
constexpr int kPairStages = 6;
constexpr int kPairABytes = BM * BK * 2;            // 128 rows per CTA
constexpr int kPairBBytes = 128 * BK * 2;           // 128 of the 256 columns per CTA
constexpr int kPairStageBytes = kPairABytes + kPairBBytes;
constexpr int kPairBN = 256;
constexpr int kPairSmemBytes = kPairStages * kPairStageBytes + 256 + 1024;

__global__ void __launch_bounds__(kThreads, 1)
gemm_tcgen05_pair_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                         const KParams p) {
  constexpr int S = kPairStages;
  constexpr int BNp = kPairBN;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* sA = smem;
  uint8_t* sB = smem + S * kPairABytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + S * kPairStageBytes);
  const uint32_t full0 = smem_u32(bars);
  const uint32_t empty0 = smem_u32(bars + S);
  const uint32_t tfull0 = smem_u32(bars + 2 * S);
  const uint32_t tempty0 = smem_u32(bars + 2 * S + 2);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * S + 4);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();          // 0 = leader
  const bool leader = rank == 0;
  const int pair_id = blockIdx.x >> 1;
  const int num_pairs = gridDim.x >> 1;

  if (threadIdx.x == 0) {
    for (int s = 0; s < S; ++s) {
      mbar_init(full0 + 8 * s, 1);      // used on the leader: its own arrive + both CTAs' bytes
      mbar_init(empty0 + 8 * s, 1);     // one commit from the leader's MMA thread, in each CTA
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(tfull0 + 8 * a, 1);     // one commit from the leader, in each CTA
      mbar_init(tempty0 + 8 * a, 8);    // used on the leader: 4 epilogue warps of each CTA
    }
    *abort_flag = 0;
    fence_barrier_init();
    fence_proxy_async_smem();
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
  }
  if (warp == 1) {
    tmem_alloc_pair(smem_u32(tmem_slot), 2 * BNp);
    tmem_relinquish_pair();
  }
  tc_fence_before_sync();
  __syncthreads();
  cluster_sync_all();                    // both CTAs' barriers exist before anything crosses the pair
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  const int total_tiles = p.tiles_per_batch * p.batch;
  const int num_kb = (p.K + BK - 1) / BK;
  int fail_code = 0;

  if (warp == 0) {
    if (lane == 0) {
      // ---------------- TMA producer (both CTAs) ----------------
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int t = pair_id; ok && t < total_tiles; t += num_pairs) {
        const int b = t / p.tiles_per_batch;
        const int4 e = p.tile_tab[t - b * p.tiles_per_batch];
        const int m0 = e.x * 256 + 128 * static_cast<int>(rank);
        const int n0 = e.y * BNp + 128 * static_cast<int>(rank);
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait_bounded(empty0 + 8 * stage, phase ^ 1u, abort_flag)) {
            ok = false;
            fail_code = kStatusTimeoutProducer;
            break;
          }
          if (leader) mbar_arrive_expect_tx(full0 + 8 * stage, 2 * kPairStageBytes);
          const uint32_t fb = (full0 + 8 * stage) & 0xFEFFFFFFu;     // the leader's barrier
          const uint32_t a_dst = smem_u32(sA + stage * kPairABytes);
          const uint32_t b_dst = smem_u32(sB + stage * kPairBBytes);
          if (!p.a_mn_major) {
            tma_load_3d_pair(a_dst, &tmA, fb, kb * BK, m0, b);
          } else {
#pragma unroll
            for (int mb = 0; mb < 2; ++mb)
              tma_load_3d_pair(a_dst + mb * kBlockBytes, &tmA, fb, m0 + 64 * mb, kb * BK, b);
          }
          if (!p.b_mn_major) {
            tma_load_3d_pair(b_dst, &tmB, fb, kb * BK, n0, b);
          } else {
#pragma unroll
            for (int nb = 0; nb < 2; ++nb)
              tma_load_3d_pair(b_dst + nb * kBlockBytes, &tmB, fb, n0 + 64 * nb, kb * BK, b);
          }
          if (++stage == S) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && leader) {
      // ---------------- MMA issuer (leader only) ----------------
      const uint32_t idesc =
          make_idesc_f16(256, BNp, p.ab_fp16 != 0, p.a_mn_major != 0, p.b_mn_major != 0);
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      for (int t = pair_id; ok && t < total_tiles; t += num_pairs) {
        if (!mbar_wait_bounded(tempty0 + 8 * acc, acc_phase ^ 1u, abort_flag)) {
          fail_code = kStatusTimeoutMma;
          break;
        }
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(acc * BNp);
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait_bounded(full0 + 8 * stage, phase, abort_flag)) {
            ok = false;
            fail_code = kStatusTimeoutMma;
            break;
          }
          tc_fence_after_sync();
          const uint32_t a_base = smem_u32(sA + stage * kPairABytes);
          const uint32_t b_base = smem_u32(sB + stage * kPairBBytes);
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            const uint64_t adesc = p.a_mn_major
                                       ? make_smem_desc_sw128(a_base + k * 2048, kBlockBytes, 1024)
                                       : make_smem_desc_sw128(a_base + k * 32, 16, 1024);
            const uint64_t bdesc = p.b_mn_major
                                       ? make_smem_desc_sw128(b_base + k * 2048, kBlockBytes, 1024)
                                       : make_smem_desc_sw128(b_base + k * 32, 16, 1024);
            umma_f16_ss_pair(d_tmem, adesc, bdesc, idesc, (kb | k) != 0 ? 1u : 0u);
          }
          // free the stage in both CTAs
          umma_commit_pair(mapa_shared(empty0 + 8 * stage, 0));
          umma_commit_pair(mapa_shared(empty0 + 8 * stage, 1));
          if (++stage == S) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (!ok) break;
        umma_commit_pair(mapa_shared(tfull0 + 8 * acc, 0));
        umma_commit_pair(mapa_shared(tfull0 + 8 * acc, 1));
        acc ^= 1;
        if (acc == 0) acc_phase ^= 1u;
      }
    }
  } else {
    // ---------------- epilogue (warps 2..5 of both CTAs) ----------------
    const int q = warp & 3;
    int acc = 0;
    uint32_t acc_phase = 0;
    for (int t = pair_id; t < total_tiles; t += num_pairs) {
      const int b = t / p.tiles_per_batch;
      const int4 e = p.tile_tab[t - b * p.tiles_per_batch];
      const int m0 = e.x * 256 + 128 * static_cast<int>(rank);
      const int n0 = e.y * BNp;
      const bool mirror = (e.z & 1) != 0;
      if (!mbar_wait_bounded(tfull0 + 8 * acc, acc_phase, abort_flag)) {
        fail_code = kStatusTimeoutEpilogue;
        break;
      }
      tc_fence_after_sync();
      const int row = m0 + q * 32 + lane;
      const char* Cb = reinterpret_cast<const char*>(p.C_tab ? p.C_tab[b] : p.C);
      char* Db = reinterpret_cast<char*>(p.D_tab ? p.D_tab[b] : p.D);
      __nv_bfloat16* D2b = reinterpret_cast<__nv_bfloat16*>(p.D2_tab ? p.D2_tab[b] : p.D2);
      const int esz = (p.out_kind == 2) ? 4 : 2;
      if (!p.C_tab && Cb) Cb += static_cast<long long>(b) * p.strideC * esz;
      if (!p.D_tab) Db += static_cast<long long>(b) * p.strideD * esz;
      if (!p.D2_tab && D2b) D2b += static_cast<long long>(b) * p.strideD2;
      const float alpha = p.alpha_vec ? p.alpha * p.alpha_vec[b] : p.alpha;
      for (int c = 0; c < BNp; c += 32) {
        const int col0 = n0 + c;
        if (col0 >= p.N) break;
        uint32_t r[32];
        tmem_ld_32x32(tmem_base + (static_cast<uint32_t>(q * 32) << 16) + static_cast<uint32_t>(acc * BNp + c), r);
        tmem_ld_wait();
        float v[32];
#pragma unroll
        for (int j = 0; j < 32; ++j) v[j] = alpha * __uint_as_float(r[j]);
        if (p.out_kind == 0) {
          epilogue_chunk<__nv_bfloat16>(p, reinterpret_cast<const __nv_bfloat16*>(Cb),
                                        reinterpret_cast<__nv_bfloat16*>(Db), D2b, v, row, col0, mirror);
        } else if (p.out_kind == 1) {
          epilogue_chunk<__half>(p, reinterpret_cast<const __half*>(Cb), reinterpret_cast<__half*>(Db), D2b, v,
                                 row, col0, mirror);
        } else {
          epilogue_chunk<float>(p, reinterpret_cast<const float*>(Cb), reinterpret_cast<float*>(Db), D2b, v, row,
                                col0, mirror);
        }
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(mapa_shared(tempty0 + 8 * acc, 0));   // the leader's barrier
      acc ^= 1;
      if (acc == 0) acc_phase ^= 1u;
    }
  }

  // ---------------- teardown ----------------
  tc_fence_before_sync();
  __syncthreads();
  if (*abort_flag) {
    if (fail_code != 0 && p.status != nullptr) atomicCAS(p.status, 0, fail_code);
    for (int i = 0; i < 64; ++i) __nanosleep(2000);
    __syncthreads();
  }
  cluster_sync_all();                    // the peer may still read this CTA's shared memory until here
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc_pair(tmem_base, 2 * BNp);
  }
}

// ---- CTA-quad kernel: two CTA pairs of one cluster share their A rows ---------------
//
// The pair kernel above is bound by the L2 -> SM stream (32 KB per CTA per
// k-block at 64 B/clk/SM).  Here a cluster of four CTAs holds two pairs that
// work on two column tiles of the SAME 256 output rows.  CTA r and its sibling
// r^2 need the same 128 rows of A, so each loads only 64 of them from L2
// (its "own quarter") and forwards that quarter to the sibling with a
// shared-memory -> distributed-shared-memory bulk copy that completes on the
// sibling's mbarrier.  Per k-block a CTA now reads 8 KB of A + 16 KB of B from
// L2 (0.75 x) and 8 KB arrives over the SM-to-SM network.  No load is
// multicast: every TMA load is issued by the CTA whose shared memory it fills.
//
// Tile list entries describe two tiles: x = m0 | m1 << 16, y = n0 | n1 << 16
// (units of 256), z bit 0/1 = mirror flag of tile 0/1, bit 2 = the tiles share
// their rows (m0 == m1), bit 3 = tile 1 is a filler that stores nothing.
// Without bit 2 each CTA loads both of its quarters itself and nothing is
// forwarded; every barrier still cycles once per k-block, so both modes run
// through one protocol.
//
// Per stage and CTA: `own_a` (the quarter this CTA loads), `fwd_in` (the other
// quarter: forwarded by the sibling, or loaded locally), `empty` (MMA commit).
// The pair leader also has `full` (B of both CTAs) and `peer_ready` (its
// partner's two A barriers, relayed by the partner's otherwise idle MMA warp).
// Before a producer refills a stage it tells the sibling "my stage is free for
// round n" through a counter in the sibling's shared memory and waits for the
// sibling's counter: the sibling's forward may only land in a free stage, and
// a stage may only be refilled once the sibling has consumed what was
// forwarded out of it.
constexpr int kQuadStages = 7;
constexpr int kQuadThreads = 224;                     // the pair kernel's six warps + one forwarding warp
constexpr int kQuarterBytes = 64 * BK * 2;            // 64 A rows of one k-block (8 KB)
constexpr int kQuadABytes = 2 * kQuarterBytes;        // 128 rows per CTA
constexpr int kQuadBBytes = 128 * BK * 2;             // 128 of the pair's 256 columns per CTA
constexpr int kQuadStageBytes = kQuadABytes + kQuadBBytes;
constexpr int kQuadBarBytes = 512;
constexpr int kQuadSmemBytes = kQuadStages * kQuadStageBytes + kQuadBarBytes + 1024;

__device__ __forceinline__ bool poll_ge_bounded(volatile uint32_t* ctr, uint32_t want, volatile int* abort_flag) {
  if (*ctr >= want) return true;
  const long long t0 = clock64();
  uint32_t spins = 0;
  while (true) {
    if (*ctr >= want) return true;
    if ((++spins & 63u) == 0u) {
      if (*abort_flag) return false;
      if (clock64() - t0 > kWaitBudgetCycles) {
        *abort_flag = 1;
        return false;
      }
    }
  }
}

// One warp's share (32 accumulator rows) of a 256-column output tile.
__device__ __forceinline__ void epilogue_rows32(const KParams& p, uint32_t tmem_addr, int row, int n0, int b,
                                                bool mirror) {
  const char* Cb = reinterpret_cast<const char*>(p.C_tab ? p.C_tab[b] : p.C);
  char* Db = reinterpret_cast<char*>(p.D_tab ? p.D_tab[b] : p.D);
  __nv_bfloat16* D2b = reinterpret_cast<__nv_bfloat16*>(p.D2_tab ? p.D2_tab[b] : p.D2);
  const int esz = (p.out_kind == 2) ? 4 : 2;
  if (!p.C_tab && Cb) Cb += static_cast<long long>(b) * p.strideC * esz;
  if (!p.D_tab) Db += static_cast<long long>(b) * p.strideD * esz;
  if (!p.D2_tab && D2b) D2b += static_cast<long long>(b) * p.strideD2;
  const float alpha = p.alpha_vec ? p.alpha * p.alpha_vec[b] : p.alpha;
  for (int c = 0; c < 256; c += 32) {
    const int col0 = n0 + c;
    if (col0 >= p.N) break;  // uniform across the warp
    uint32_t r[32];
    tmem_ld_32x32(tmem_addr + static_cast<uint32_t>(c), r);
    tmem_ld_wait();
    float v[32];
#pragma unroll
    for (int j = 0; j < 32; ++j) v[j] = alpha * __uint_as_float(r[j]);
    if (p.out_kind == 0) {
      epilogue_chunk<__nv_bfloat16>(p, reinterpret_cast<const __nv_bfloat16*>(Cb),
                                    reinterpret_cast<__nv_bfloat16*>(Db), D2b, v, row, col0, mirror);
    } else if (p.out_kind == 1) {
      epilogue_chunk<__half>(p, reinterpret_cast<const __half*>(Cb), reinterpret_cast<__half*>(Db), D2b, v, row,
                             col0, mirror);
    } else {
      epilogue_chunk<float>(p, reinterpret_cast<const float*>(Cb), reinterpret_cast<float*>(Db), D2b, v, row,
                            col0, mirror);
    }
  }
}

__global__ void __launch_bounds__(kQuadThreads, 1)
gemm_tcgen05_quad_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                         const KParams p) {
  constexpr int S = kQuadStages;
  constexpr int BNp = kPairBN;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* sA = smem;
  uint8_t* sB = smem + S * kQuadABytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + S * kQuadStageBytes);
  const uint32_t full0 = smem_u32(bars);
  const uint32_t empty0 = smem_u32(bars + S);
  const uint32_t owna0 = smem_u32(bars + 2 * S);
  const uint32_t fwdin0 = smem_u32(bars + 3 * S);
  const uint32_t pready0 = smem_u32(bars + 4 * S);
  const uint32_t tfull0 = smem_u32(bars + 5 * S);
  const uint32_t tempty0 = smem_u32(bars + 5 * S + 2);
  uint32_t* words = reinterpret_cast<uint32_t*>(bars + 5 * S + 4);
  const uint32_t sibfree0 = smem_u32(words);            // S counters written by the sibling CTA
  uint32_t* tmem_slot = words + S;
  volatile int* abort_flag = reinterpret_cast<volatile int*>(words + S + 1);
  volatile uint32_t* fwd_cnt = words + S + 2;           // k-blocks the forwarding thread has handled

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();              // 0..3
  const uint32_t half = rank & 1u;                      // which 128 rows / columns of the pair's tile
  const uint32_t pair = rank >> 1;                      // which of the two tiles
  const uint32_t lead = rank & ~1u;                     // rank of this pair's MMA-issuing CTA
  const uint32_t sib = rank ^ 2u;                       // same half of the other pair
  const bool leader = half == 0;
  const int quad_id = blockIdx.x >> 2;
  const int num_quads = gridDim.x >> 2;

  if (threadIdx.x == 0) {
    for (int s = 0; s < S; ++s) {
      mbar_init(full0 + 8 * s, 1);      // leader: its own arrive + the B bytes of both CTAs
      mbar_init(empty0 + 8 * s, 1);     // one commit from the pair's MMA thread, in each CTA
      mbar_init(owna0 + 8 * s, 1);      // own arrive + the bytes of the quarter this CTA loads
      mbar_init(fwdin0 + 8 * s, 1);     // own arrive + the bytes of the other quarter
      mbar_init(pready0 + 8 * s, 1);    // leader: the partner's relay
      words[s] = 0;
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(tfull0 + 8 * a, 1);
      mbar_init(tempty0 + 8 * a, 8);
    }
    *abort_flag = 0;
    *fwd_cnt = 0;
    fence_barrier_init();
    fence_proxy_async_smem();
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
  }
  if (warp == 1) {
    tmem_alloc_pair(smem_u32(tmem_slot), 2 * BNp);
    tmem_relinquish_pair();
  }
  tc_fence_before_sync();
  __syncthreads();
  cluster_sync_all();                    // every CTA's barriers and counters exist before anything crosses
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  const int total_tiles = p.tiles_per_batch * p.batch;
  const int num_kb = (p.K + BK - 1) / BK;
  int fail_code = 0;

  // both tiles of an entry, selected by `pair`
#define DMUON_QUAD_DECODE(e)                                                             \
  const int m_blk = pair ? ((e).x >> 16) : ((e).x & 0xffff);                             \
  const int n_blk = pair ? ((e).y >> 16) : ((e).y & 0xffff);                             \
  const bool share = ((e).z & 4) != 0;

  if (warp == 0) {
    if (lane == 0) {
      // ---------------- TMA producer (every CTA) ----------------
      uint32_t cnt = 0;
      bool ok = true;
      for (int t = quad_id; ok && t < total_tiles; t += num_quads) {
        const int b = t / p.tiles_per_batch;
        const int4 e = p.tile_tab[t - b * p.tiles_per_batch];
        DMUON_QUAD_DECODE(e)
        const int m0 = m_blk * 256 + 128 * static_cast<int>(half);
        const int n0 = n_blk * BNp + 128 * static_cast<int>(half);
        for (int kb = 0; kb < num_kb; ++kb, ++cnt) {
          const uint32_t stage = cnt % S;
          const uint32_t round = cnt / S;
          const uint32_t phase = round & 1u;
          // this pair is done with the stage, the forwarding thread has dealt with its last
          // contents, and the sibling is done with ITS stage (so what this CTA forwarded out
          // of the stage has been consumed and what it forwards next lands in free memory)
          if (!mbar_wait_bounded(empty0 + 8 * stage, phase ^ 1u, abort_flag) ||
              (cnt >= S && !poll_ge_bounded(fwd_cnt, cnt - S + 1, abort_flag))) {
            ok = false;
            fail_code = kStatusTimeoutProducer;
            break;
          }
          st_release_cluster_u32(mapa_shared(sibfree0 + 4 * stage, sib), round + 1);
          if (!counter_wait_bounded(sibfree0 + 4 * stage, round + 1, abort_flag)) {
            ok = false;
            fail_code = kStatusTimeoutProducer;
            break;
          }
          if (leader) mbar_arrive_expect_tx(full0 + 8 * stage, 2 * kQuadBBytes);
          mbar_arrive_expect_tx(owna0 + 8 * stage, kQuarterBytes);
          mbar_arrive_expect_tx(fwdin0 + 8 * stage, kQuarterBytes);
          const uint32_t a_dst = smem_u32(sA + stage * kQuadABytes);
          const uint32_t b_dst = smem_u32(sB + stage * kQuadBBytes);
          const int q = static_cast<int>(pair);
          if (!p.a_mn_major) {
            tma_load_3d(a_dst + q * kQuarterBytes, &tmA, owna0 + 8 * stage, kb * BK, m0 + 64 * q, b);
            if (!share)
              tma_load_3d(a_dst + (1 - q) * kQuarterBytes, &tmA, fwdin0 + 8 * stage, kb * BK, m0 + 64 * (1 - q), b);
          } else {
            tma_load_3d(a_dst + q * kQuarterBytes, &tmA, owna0 + 8 * stage, m0 + 64 * q, kb * BK, b);
            if (!share)
              tma_load_3d(a_dst + (1 - q) * kQuarterBytes, &tmA, fwdin0 + 8 * stage, m0 + 64 * (1 - q), kb * BK, b);
          }
          const uint32_t fb = mapa_shared(full0 + 8 * stage, lead);
          if (!p.b_mn_major) {
            tma_load_3d_pair(b_dst, &tmB, fb, kb * BK, n0, b);
          } else {
#pragma unroll
            for (int nb = 0; nb < 2; ++nb)
              tma_load_3d_pair(b_dst + nb * kBlockBytes, &tmB, fb, n0 + 64 * nb, kb * BK, b);
          }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0 && leader) {
      // ---------------- MMA issuer (pair leaders) ----------------
      const uint32_t idesc =
          make_idesc_f16(256, BNp, p.ab_fp16 != 0, p.a_mn_major != 0, p.b_mn_major != 0);
      uint32_t cnt = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      for (int t = quad_id; ok && t < total_tiles; t += num_quads) {
        if (!mbar_wait_bounded(tempty0 + 8 * acc, acc_phase ^ 1u, abort_flag)) {
          fail_code = kStatusTimeoutMma;
          break;
        }
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(acc * BNp);
        for (int kb = 0; kb < num_kb; ++kb, ++cnt) {
          const uint32_t stage = cnt % S;
          const uint32_t phase = (cnt / S) & 1u;
          if (!mbar_wait_bounded(full0 + 8 * stage, phase, abort_flag) ||
              !mbar_wait_bounded(owna0 + 8 * stage, phase, abort_flag) ||
              !mbar_wait_bounded(fwdin0 + 8 * stage, phase, abort_flag) ||
              !mbar_wait_bounded(pready0 + 8 * stage, phase, abort_flag)) {
            ok = false;
            fail_code = kStatusTimeoutMma;
            break;
          }
          tc_fence_after_sync();
          const uint32_t a_base = smem_u32(sA + stage * kQuadABytes);
          const uint32_t b_base = smem_u32(sB + stage * kQuadBBytes);
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            const uint64_t adesc = p.a_mn_major
                                       ? make_smem_desc_sw128(a_base + k * 2048, kBlockBytes, 1024)
                                       : make_smem_desc_sw128(a_base + k * 32, 16, 1024);
            const uint64_t bdesc = p.b_mn_major
                                       ? make_smem_desc_sw128(b_base + k * 2048, kBlockBytes, 1024)
                                       : make_smem_desc_sw128(b_base + k * 32, 16, 1024);
            umma_f16_ss_pair(d_tmem, adesc, bdesc, idesc, (kb | k) != 0 ? 1u : 0u);
          }
          umma_commit_pair(mapa_shared(empty0 + 8 * stage, lead));
          umma_commit_pair(mapa_shared(empty0 + 8 * stage, lead + 1));
        }
        if (!ok) break;
        umma_commit_pair(mapa_shared(tfull0 + 8 * acc, lead));
        umma_commit_pair(mapa_shared(tfull0 + 8 * acc, lead + 1));
        acc ^= 1;
        if (acc == 0) acc_phase ^= 1u;
      }
    } else if (lane == 0) {
      // ---------------- relay (the leader cannot wait on this CTA's barriers) ----------------
      uint32_t cnt = 0;
      bool ok = true;
      for (int t = quad_id; ok && t < total_tiles; t += num_quads) {
        for (int kb = 0; kb < num_kb; ++kb, ++cnt) {
          const uint32_t stage = cnt % S;
          const uint32_t phase = (cnt / S) & 1u;
          if (!mbar_wait_bounded(owna0 + 8 * stage, phase, abort_flag) ||
              !mbar_wait_bounded(fwdin0 + 8 * stage, phase, abort_flag)) {
            ok = false;
            fail_code = kStatusTimeoutMma;
            break;
          }
          mbar_arrive_cluster(mapa_shared(pready0 + 8 * stage, lead));
        }
      }
    }
  } else if (warp == 6) {
    if (lane == 0) {
      // ---------------- forwarder: own quarter -> the sibling's shared memory ----------------
      uint32_t cnt = 0;
      bool ok = true;
      for (int t = quad_id; ok && t < total_tiles; t += num_quads) {
        const int b = t / p.tiles_per_batch;
        const int4 e = p.tile_tab[t - b * p.tiles_per_batch];
        const bool share = (e.z & 4) != 0;
        for (int kb = 0; kb < num_kb; ++kb, ++cnt) {
          const uint32_t stage = cnt % S;
          const uint32_t phase = (cnt / S) & 1u;
          if (!mbar_wait_bounded(owna0 + 8 * stage, phase, abort_flag)) {
            ok = false;
            fail_code = kStatusTimeoutProducer;
            break;
          }
          if (share) {
            const uint32_t src = smem_u32(sA + stage * kQuadABytes) + pair * kQuarterBytes;
            bulk_copy_s2cluster(mapa_shared(src, sib), src, kQuarterBytes, mapa_shared(fwdin0 + 8 * stage, sib));
          }
          *fwd_cnt = cnt + 1;
        }
      }
    }
  } else {
    // ---------------- epilogue (warps 2..5 of every CTA) ----------------
    const int q = warp & 3;
    int acc = 0;
    uint32_t acc_phase = 0;
    for (int t = quad_id; t < total_tiles; t += num_quads) {
      const int b = t / p.tiles_per_batch;
      const int4 e = p.tile_tab[t - b * p.tiles_per_batch];
      DMUON_QUAD_DECODE(e)
      (void)share;
      const bool mirror = ((e.z >> pair) & 1) != 0;
      const bool filler = pair != 0 && (e.z & 8) != 0;
      if (!mbar_wait_bounded(tfull0 + 8 * acc, acc_phase, abort_flag)) {
        fail_code = kStatusTimeoutEpilogue;
        break;
      }
      tc_fence_after_sync();
      if (!filler) {
        const int row = m_blk * 256 + 128 * static_cast<int>(half) + q * 32 + lane;
        epilogue_rows32(p, tmem_base + (static_cast<uint32_t>(q * 32) << 16) + static_cast<uint32_t>(acc * BNp), row,
                        n_blk * BNp, b, mirror);
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(mapa_shared(tempty0 + 8 * acc, lead));
      acc ^= 1;
      if (acc == 0) acc_phase ^= 1u;
    }
  }
#undef DMUON_QUAD_DECODE

  // ---------------- teardown ----------------
  tc_fence_before_sync();
  __syncthreads();
  if (*abort_flag) {
    if (fail_code != 0 && p.status != nullptr) atomicCAS(p.status, 0, fail_code);
    for (int i = 0; i < 64; ++i) __nanosleep(2000);
    __syncthreads();
  }
  cluster_sync_all();                    // peers may still read or write this CTA's shared memory until here
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc_pair(tmem_base, 2 * BNp);
  }
}

// ---- host side ------------------------------------------------------------------

using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                              const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                              CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                              CUtensorMapFloatOOBfill);

static EncodeFn get_encode_fn() {
  static EncodeFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeFn>(sym);
  });
  return fn;
}

// Tensor map over a batched row-major matrix [batch][rows][cols] of 2-byte
// elements; the box is box_cols x box_rows x 1 with 128-byte swizzle.
static int make_map(CUtensorMap* map, const void* base, bool fp16, long long cols, long long rows,
                    long long batch, long long ld, long long batch_stride, int box_cols, int box_rows) {
  EncodeFn enc = get_encode_fn();
  if (enc == nullptr) return -2;
  cuuint64_t dims[3] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(rows),
                        static_cast<cuuint64_t>(batch)};
  long long bs = (batch > 1 && batch_stride > 0) ? batch_stride : rows * ld;
  cuuint64_t strides[2] = {static_cast<cuuint64_t>(ld) * 2, static_cast<cuuint64_t>(bs) * 2};
  cuuint32_t box[3] = {static_cast<cuuint32_t>(box_cols), static_cast<cuuint32_t>(box_rows), 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = enc(map, fp16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3,
                   const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : -3;
}

static std::atomic<long long> g_launches{0};

// Raise a kernel's dynamic shared-memory limit once per device (kernel slot k).
static std::mutex g_attr_mu;
static bool g_attr_set[4][16] = {};

template <typename Kern>
static cudaError_t ensure_smem_attr(int slot, Kern kern, int bytes) {
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 16) return cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
  std::lock_guard<std::mutex> lock(g_attr_mu);
  if (!g_attr_set[slot][dev]) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
    if (e != cudaSuccess) return e;
    g_attr_set[slot][dev] = true;
  }
  return cudaSuccess;
}

static KParams make_params(const DmuonGemmArgs& a) {
  KParams p;
  p.M = a.M; p.N = a.N; p.K = a.K; p.batch = a.batch;
  p.tile_tab = reinterpret_cast<const int4*>(a.tile_tab);
  p.tiles_per_batch = a.tiles_per_batch;
  p.a_mn_major = a.a_mn_major; p.b_mn_major = a.b_mn_major; p.ab_fp16 = a.ab_fp16;
  p.alpha = a.alpha; p.beta = a.beta; p.diag = a.diag;
  p.alpha_vec = a.alpha_vec;
  p.C = a.C; p.D = a.D; p.D2 = a.D2;
  p.C_tab = a.C_tab; p.D_tab = a.D_tab; p.D2_tab = a.D2_tab;
  p.ldc = a.ldc; p.ldd = a.ldd; p.ldd2 = a.ldd2;
  p.strideC = a.strideC; p.strideD = a.strideD; p.strideD2 = a.strideD2;
  p.out_kind = a.out_kind;
  p.b_ready = a.b_ready; p.b_ready_epoch = a.b_ready_epoch;
  p.status = a.status;
  p.d2_multimem = a.d2_multimem;
  if (p.C == nullptr && p.C_tab == nullptr) p.beta = 0.f;
  return p;
}

template <int BN>
static int launch(const DmuonGemmArgs& a, const CUtensorMap& tmA, const CUtensorMap& tmB,
                  cudaStream_t stream, int num_sms) {
  auto kern = gemm_tcgen05_kernel<BN>;
  {
    cudaError_t e = ensure_smem_attr(BN == 256 ? 0 : 1, kern, Cfg<BN>::kSmemBytes);
    if (e != cudaSuccess) return static_cast<int>(e);
  }
  KParams p = make_params(a);
  const long long total = static_cast<long long>(a.tiles_per_batch) * a.batch;
  int cap = (a.max_ctas > 0 && a.max_ctas < num_sms) ? a.max_ctas : num_sms;
  int grid = static_cast<int>(total < cap ? total : cap);
  if (grid <= 0) return 0;
  kern<<<grid, kThreads, Cfg<BN>::kSmemBytes, stream>>>(tmA, tmB, p);
  g_launches.fetch_add(1, std::memory_order_relaxed);
  return static_cast<int>(cudaGetLastError());
}

static int launch_pair(const DmuonGemmArgs& a, const CUtensorMap& tmA, const CUtensorMap& tmB,
                       cudaStream_t stream, int num_sms) {
  {
    cudaError_t e = ensure_smem_attr(2, gemm_tcgen05_pair_kernel, kPairSmemBytes);
    if (e != cudaSuccess) return static_cast<int>(e);
  }
  KParams p = make_params(a);
  p.b_ready = nullptr; p.b_ready_epoch = 0;
  const long long total = static_cast<long long>(a.tiles_per_batch) * a.batch;
  int pairs = num_sms / 2;
  if (a.max_ctas > 0 && a.max_ctas / 2 < pairs) pairs = a.max_ctas / 2;
  if (total < pairs) pairs = static_cast<int>(total);
  if (pairs <= 0) return 0;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(2 * pairs, 1, 1);
  cfg.blockDim = dim3(kThreads, 1, 1);
  cfg.dynamicSmemBytes = kPairSmemBytes;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  cudaError_t e = cudaLaunchKernelEx(&cfg, gemm_tcgen05_pair_kernel, tmA, tmB, p);
  g_launches.fetch_add(1, std::memory_order_relaxed);
  return static_cast<int>(e != cudaSuccess ? e : cudaGetLastError());
}

static void quad_launch_config(cudaLaunchConfig_t* cfg, cudaLaunchAttribute* attr, int quads, cudaStream_t stream) {
  *cfg = cudaLaunchConfig_t{};
  cfg->gridDim = dim3(4 * quads, 1, 1);
  cfg->blockDim = dim3(kQuadThreads, 1, 1);
  cfg->dynamicSmemBytes = kQuadSmemBytes;
  cfg->stream = stream;
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 4;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg->attrs = attr;
  cfg->numAttrs = 1;
}

// How many clusters of four CTAs of the quad kernel can be resident at once on
// the current device (SMs of a GPC that do not fill a cluster stay idle).  The
// kernel is persistent, so the grid never exceeds this.  0 if the query fails.
static int quad_max_clusters() {
  static int cached[16] = {};
  static std::mutex mu;
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 16) return 0;
  std::lock_guard<std::mutex> lock(mu);
  if (cached[dev] == 0) {
    if (ensure_smem_attr(3, gemm_tcgen05_quad_kernel, kQuadSmemBytes) != cudaSuccess) return 0;
    cudaLaunchConfig_t cfg;
    cudaLaunchAttribute attr[1];
    quad_launch_config(&cfg, attr, 37, nullptr);
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, gemm_tcgen05_quad_kernel, &cfg) != cudaSuccess || n <= 0) {
      cudaGetLastError();
      cached[dev] = -1;
    } else {
      cached[dev] = n;
    }
  }
  return cached[dev] > 0 ? cached[dev] : 0;
}

static int launch_quad(const DmuonGemmArgs& a, const CUtensorMap& tmA, const CUtensorMap& tmB,
                       cudaStream_t stream) {
  int quads = quad_max_clusters();
  if (quads <= 0) return -4;
  KParams p = make_params(a);
  p.b_ready = nullptr; p.b_ready_epoch = 0;
  const long long total = static_cast<long long>(a.tiles_per_batch) * a.batch;
  if (a.max_ctas > 0 && a.max_ctas / 4 < quads) quads = a.max_ctas / 4;
  if (total < quads) quads = static_cast<int>(total);
  if (quads <= 0) return 0;
  cudaLaunchConfig_t cfg;
  cudaLaunchAttribute attr[1];
  quad_launch_config(&cfg, attr, quads, stream);
  cudaError_t e = cudaLaunchKernelEx(&cfg, gemm_tcgen05_quad_kernel, tmA, tmB, p);
  g_launches.fetch_add(1, std::memory_order_relaxed);
  return static_cast<int>(e != cudaSuccess ? e : cudaGetLastError());
}

}  // namespace dmuon

extern "C" int dmuon_gemm_quad_max_clusters(void) { return dmuon::quad_max_clusters(); }

extern "C" long long dmuon_launch_count(void) {
  return dmuon::g_launches.load(std::memory_order_relaxed);
}

namespace dmuon {
void count_launch() { g_launches.fetch_add(1, std::memory_order_relaxed); }
}

extern "C" int dmuon_gemm_sm100(const DmuonGemmArgs* args, void* stream_v) {
  using namespace dmuon;
  const DmuonGemmArgs& a = *args;
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_v);
  if (a.M <= 0 || a.N <= 0 || a.K <= 0 || a.batch <= 0) return 0;
  if ((a.bn != 128 && a.bn != 256) || a.tile_tab == nullptr || a.tiles_per_batch <= 0) return -1;
  if ((a.lda % 8) != 0 || (a.ldb % 8) != 0 || (a.strideA % 8) != 0 || (a.strideB % 8) != 0) return -1;
  if ((reinterpret_cast<uintptr_t>(a.A) & 15) || (reinterpret_cast<uintptr_t>(a.B) & 15)) return -1;
  // the multicast form of the second output writes whole 16-byte groups of a row and has no transposed store
  if (a.d2_multimem && ((a.N % 8) != 0 || (a.ldd2 % 8) != 0 || (a.strideD2 % 8) != 0 ||
                        (reinterpret_cast<uintptr_t>(a.D2) & 15)))
    return -1;
  static int num_sms[16] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 16 && num_sms[dev] == 0)
    cudaDeviceGetAttribute(&num_sms[dev], cudaDevAttrMultiProcessorCount, dev);
  const int sms = (dev < 16) ? num_sms[dev] : 148;

  CUtensorMap tmA, tmB;
  int rc;
  if (!a.a_mn_major)
    rc = make_map(&tmA, a.A, a.ab_fp16 != 0, a.K, a.M, a.batch, a.lda, a.strideA, BK, BM);
  else
    rc = make_map(&tmA, a.A, a.ab_fp16 != 0, a.M, a.K, a.batch, a.lda, a.strideA, 64, BK);
  if (rc != 0) return rc;
  if (a.two_cta == 2) {
    // CTA quads: A is loaded in quarters of 64 rows, B as for pairs
    if (a.bn != 256) return -1;
    if (!a.a_mn_major) rc = make_map(&tmA, a.A, a.ab_fp16 != 0, a.K, a.M, a.batch, a.lda, a.strideA, BK, 64);
    if (rc != 0) return rc;
    if (!a.b_mn_major)
      rc = make_map(&tmB, a.B, a.ab_fp16 != 0, a.K, a.N, a.batch, a.ldb, a.strideB, BK, 128);
    else
      rc = make_map(&tmB, a.B, a.ab_fp16 != 0, a.N, a.K, a.batch, a.ldb, a.strideB, 64, BK);
    if (rc != 0) return rc;
    return launch_quad(a, tmA, tmB, stream);
  }
  if (a.two_cta) {
    if (a.bn != 256) return -1;
    // each CTA of a pair loads 128 of the 256 B columns
    if (!a.b_mn_major)
      rc = make_map(&tmB, a.B, a.ab_fp16 != 0, a.K, a.N, a.batch, a.ldb, a.strideB, BK, 128);
    else
      rc = make_map(&tmB, a.B, a.ab_fp16 != 0, a.N, a.K, a.batch, a.ldb, a.strideB, 64, BK);
    if (rc != 0) return rc;
    return launch_pair(a, tmA, tmB, stream, sms);
  }
  if (!a.b_mn_major)
    rc = make_map(&tmB, a.B, a.ab_fp16 != 0, a.K, a.N, a.batch, a.ldb, a.strideB, BK, a.bn);
  else
    rc = make_map(&tmB, a.B, a.ab_fp16 != 0, a.N, a.K, a.batch, a.ldb, a.strideB, 64, BK);
  if (rc != 0) return rc;
  if (a.bn == 256) return launch<256>(a, tmA, tmB, stream, sms);
  return launch<128>(a, tmA, tmB, stream, sms);
}

// ---------------------------------------------------------------------------
// Allocation-free symmetric product (see noalloc.cuh).  Same kernel as above;
// its tile table and status word live in a static device array instead of
// caller-provided memory.
// ---------------------------------------------------------------------------
#include "noalloc.cuh"

namespace dmuon {

// [0, 256): header, word 0 = status.  [256, ...): tile table (int4 per tile).
static __device__ __align__(256) unsigned char g_noalloc_scratch[DMUON_NOALLOC_SCRATCH_BYTES];

// Device code may name the array directly.  One thread per row of tiles: it
// counts the tiles of its row that touch the lower triangle, finds where its
// row starts in the table by summing the counts of the rows before it, and
// writes its entries.  (At most 256 rows: a matrix with more has more tiles
// than the table holds and was refused by the host.)
constexpr int kNoallocMaxRowTiles = 256;

__global__ void __launch_bounds__(kNoallocMaxRowTiles, 1) noalloc_fill_tiles_kernel(int M, int bn) {
  __shared__ int counts[kNoallocMaxRowTiles];
  int4* tab = reinterpret_cast<int4*>(g_noalloc_scratch + DMUON_NOALLOC_HEADER_BYTES);
  const int mt = (M + BM - 1) / BM;
  const int i = threadIdx.x;
  int mine = 0;
  if (i < mt) mine = (min(M, (i + 1) * BM) - 1) / bn + 1;
  counts[i] = mine;
  __syncthreads();
  if (i >= mt) return;
  int n = 0;
  for (int r = 0; r < i; ++r) n += counts[r];
  for (int j = 0; j < mine; ++j) {
    const int mirror = ((j + 1) * bn <= i * BM) ? 1 : 0;
    tab[n + j] = make_int4(i, j, mirror, 0);
  }
}

static int noalloc_tile_count(int M, int bn) {
  const int mt = (M + BM - 1) / BM;
  long long n = 0;
  for (int i = 0; i < mt; ++i) {
    const int last_row = (M < (i + 1) * BM ? M : (i + 1) * BM) - 1;
    n += last_row / bn + 1;
  }
  return n > 0x7fffffff ? 0x7fffffff : static_cast<int>(n);
}

// Host code must not pass `g_noalloc_scratch` itself to a kernel: in host code
// that name is only a stand-in.  The device address is looked up once per
// device, with that device current.
static unsigned char* noalloc_scratch_ptr(int* err) {
  static unsigned char* ptrs[16] = {};
  static std::mutex mu;
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 16) {
    *err = DMUON_NOALLOC_E_SYMBOL;
    return nullptr;
  }
  std::lock_guard<std::mutex> lock(mu);
  if (ptrs[dev] == nullptr) {
    void* p = nullptr;
    const cudaError_t e = cudaGetSymbolAddress(&p, g_noalloc_scratch);
    if (e != cudaSuccess || p == nullptr) {
      *err = DMUON_NOALLOC_E_SYMBOL;
      return nullptr;
    }
    ptrs[dev] = static_cast<unsigned char*>(p);
  }
  return ptrs[dev];
}

}  // namespace dmuon

extern "C" int dmuon_syrk_noalloc(const void* X, void* D, int M, int K, int batch, long long ldx, long long ldd,
                                  long long strideX, long long strideD, int is_fp16, int x_mn_major, float alpha,
                                  float diag, void* stream_v) {
  using namespace dmuon;
  if (X == nullptr || D == nullptr || M <= 0 || K <= 0 || batch <= 0) return DMUON_NOALLOC_E_BAD_ARGUMENT;
  if ((ldx % 8) != 0 || (ldd % 8) != 0 || (strideX % 8) != 0 || (strideD % 8) != 0)
    return DMUON_NOALLOC_E_BAD_ARGUMENT;
  if ((reinterpret_cast<uintptr_t>(X) & 15) || (reinterpret_cast<uintptr_t>(D) & 15))
    return DMUON_NOALLOC_E_BAD_ARGUMENT;
  // every matrix of a batch needs its own output: a zero stride would make them overwrite each other
  if (batch > 1 && (strideD == 0 || strideX == 0)) return DMUON_NOALLOC_E_BAD_ARGUMENT;
  const int bn = (M <= 128) ? 128 : 256;
  if ((M + BM - 1) / BM > kNoallocMaxRowTiles) return DMUON_NOALLOC_E_TOO_LARGE;
  const int ntiles = noalloc_tile_count(M, bn);
  if (ntiles > DMUON_NOALLOC_MAX_TILES) return DMUON_NOALLOC_E_TOO_LARGE;
  int err = 0;
  unsigned char* scratch = noalloc_scratch_ptr(&err);
  if (scratch == nullptr) return err;
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_v);

  // the array keeps the previous call's contents: clear the header, rewrite the table
  cudaError_t ce = cudaMemsetAsync(scratch, 0, DMUON_NOALLOC_HEADER_BYTES, stream);
  if (ce != cudaSuccess) return static_cast<int>(ce);
  noalloc_fill_tiles_kernel<<<1, kNoallocMaxRowTiles, 0, stream>>>(M, bn);
  count_launch();
  ce = cudaGetLastError();
  if (ce != cudaSuccess) return static_cast<int>(ce);

  DmuonGemmArgs a = {};
  a.A = X;
  a.B = X;
  a.lda = a.ldb = ldx;
  a.strideA = a.strideB = strideX;
  a.a_mn_major = a.b_mn_major = x_mn_major ? 1 : 0;
  a.ab_fp16 = is_fp16 ? 1 : 0;
  a.M = a.N = M;
  a.K = K;
  a.batch = batch;
  a.tile_tab = reinterpret_cast<const int*>(scratch + DMUON_NOALLOC_HEADER_BYTES);
  a.tiles_per_batch = ntiles;
  a.bn = bn;
  a.alpha = alpha;
  a.beta = 0.f;
  a.diag = diag;
  a.D = D;
  a.ldd = ldd;
  a.strideD = strideD;
  a.out_kind = is_fp16 ? 1 : 0;
  a.status = reinterpret_cast<int*>(scratch);

  int dev = 0;
  cudaGetDevice(&dev);
  int sms = 148;
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  CUtensorMap tmA, tmB;
  int rc;
  if (!a.a_mn_major) {
    rc = make_map(&tmA, a.A, a.ab_fp16 != 0, a.K, a.M, a.batch, a.lda, a.strideA, BK, BM);
    if (rc == 0) rc = make_map(&tmB, a.B, a.ab_fp16 != 0, a.K, a.N, a.batch, a.ldb, a.strideB, BK, bn);
  } else {
    rc = make_map(&tmA, a.A, a.ab_fp16 != 0, a.M, a.K, a.batch, a.lda, a.strideA, 64, BK);
    if (rc == 0) rc = make_map(&tmB, a.B, a.ab_fp16 != 0, a.N, a.K, a.batch, a.ldb, a.strideB, 64, BK);
  }
  if (rc != 0) return DMUON_NOALLOC_E_BAD_ARGUMENT;
  return bn == 256 ? launch<256>(a, tmA, tmB, stream, sms) : launch<128>(a, tmA, tmB, stream, sms);
}

extern "C" int dmuon_syrk_noalloc_status(void* stream_v) {
  using namespace dmuon;
  int err = 0;
  unsigned char* scratch = noalloc_scratch_ptr(&err);
  if (scratch == nullptr) return err;
  int status = 0;
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_v);
  if (cudaMemcpyAsync(&status, scratch, sizeof(int), cudaMemcpyDeviceToHost, stream) != cudaSuccess) return -1;
  if (cudaStreamSynchronize(stream) != cudaSuccess) return -1;
  return status;
}

extern "C" const char* dmuon_syrk_noalloc_strerror(int code) {
  switch (code) {
    case DMUON_NOALLOC_OK: return "ok";
    case DMUON_NOALLOC_E_BAD_ARGUMENT:
      return "bad argument: null or misaligned pointer, non-positive size, a pitch/stride that is not a multiple of 8 "
             "elements, or a zero batch stride with more than one matrix";
    case DMUON_NOALLOC_E_TOO_LARGE:
      return "problem too large for the built-in scratch array: more than 16384 output tiles per matrix (M above 32640)";
    case DMUON_NOALLOC_E_SYMBOL: return "cudaGetSymbolAddress failed for the built-in scratch array on this device";
    default:
      // positive values are cudaError_t codes passed through from a launch or memset
      return code > 0 ? cudaGetErrorString(static_cast<cudaError_t>(code)) : "unknown code";
  }
}
