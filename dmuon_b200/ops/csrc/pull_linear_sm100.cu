// Owner-broadcast fused into the consuming GEMM (sm_100a).
//
//   Y[M, N] = X[M, K] * W[N, K]^T      bf16 in, fp32 accumulate in TMEM, bf16 out
//
// W lives on another GPU (its owner).  One persistent kernel does both jobs:
//
//   warp 6  (every CTA)  pulls W over NVLink: 16 KB chunks, owner -> this CTA's
//           shared memory with a bulk copy (no multicast), then shared memory ->
//           this GPU's copy of W with a bulk store.  Chunks are dealt round-robin
//           to the CTAs in address order, so column tile 0 of W completes first;
//           each finished chunk bumps its tile's counter (release, GPU scope).
//   warp 0  TMA producer: before it loads tiles of W column tile j from LOCAL
//           memory it waits (bounded) until that tile's counter says all chunks
//           have landed; X tiles stream as usual.
//   warp 1  tcgen05.mma issuer, warps 2-5 epilogue -- as in gemm_sm100.cu.
//
// Tiles are ordered column-tile-major, so the multiplication with column tile j
// runs while tiles j+1, j+2, ... are still in flight: W crosses NVLink exactly
// once, lands in the local publish arena (where backward and any other reader
// find it), and the transfer hides under the tensor work.  With about 2 x 16 KB
// in flight per CTA, 148 CTAs keep ~4.7 MB outstanding, enough to cover the
// NVLink bandwidth-delay product.
//
// Replaces `dist.broadcast` of the packed buffer followed by cuBLAS `F.linear`
// (reference: dmuon/_backends/fsdp2/group.py:791-807 and the user's forward).
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <mutex>

#include "ptx_sm100.cuh"
#include "pull_linear_sm100.cuh"

namespace dmuon {
void count_launch();

namespace pl {

constexpr int BM = 128, BN = 256, BK = 64, UMMA_K = 16;
constexpr int kStages = 4;
constexpr int kABytes = BM * BK * 2;
constexpr int kBBytes = BN * BK * 2;
constexpr int kStageBytes = kABytes + kBBytes;
constexpr int kThreads = 224;
constexpr int kChunk = 16384;
constexpr int kFetchBufs = 2;
constexpr int kBarBytes = 256;
constexpr int kSmemBytes = kStages * kStageBytes + kBarBytes + kFetchBufs * kChunk + 1024;

struct Params {
  __nv_bfloat16* Y;
  unsigned char* W_local;
  const unsigned char* W_remote;
  int M, N, K;
  long long ldy;
  int* tile_ready;
  const int* pub_flag;
  int pub_want;
  long long budget_cycles;
  int* status;
};

__global__ void __launch_bounds__(kThreads, 1)
pull_linear_kernel(const __grid_constant__ CUtensorMap tmX, const __grid_constant__ CUtensorMap tmW,
                   const Params p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* sA = smem;
  uint8_t* sB = smem + kStages * kABytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kStages * kStageBytes);
  uint8_t* sF = smem + kStages * kStageBytes + kBarBytes;
  const uint32_t full0 = smem_u32(bars);
  const uint32_t empty0 = smem_u32(bars + kStages);
  const uint32_t tfull0 = smem_u32(bars + 2 * kStages);
  const uint32_t tempty0 = smem_u32(bars + 2 * kStages + 2);
  const uint32_t fbar0 = smem_u32(bars + 2 * kStages + 4);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * kStages + 4 + kFetchBufs);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(full0 + 8 * s, 1);
      mbar_init(empty0 + 8 * s, 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(tfull0 + 8 * a, 1);
      mbar_init(tempty0 + 8 * a, 4);
    }
    for (int b = 0; b < kFetchBufs; ++b) mbar_init(fbar0 + 8 * b, 1);
    *abort_flag = 0;
    fence_barrier_init();
    fence_proxy_async_smem();
    tma_prefetch_desc(&tmX);
    tma_prefetch_desc(&tmW);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(tmem_slot), 2 * BN);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  const int mt = (p.M + BM - 1) / BM;
  const int nt = (p.N + BN - 1) / BN;
  const int total_tiles = mt * nt;
  const int num_kb = (p.K + BK - 1) / BK;
  const long long tile_bytes = static_cast<long long>(BN) * p.K * 2;   // multiple of kChunk (K % 32 == 0)
  const long long w_bytes = static_cast<long long>(p.N) * p.K * 2;
  const bool pulling = p.W_remote != nullptr;
  // every role may have to wait for the owner's publish: same budget everywhere
  const long long wait_budget = p.budget_cycles + kWaitBudgetCycles;
  int fail_code = 0;

  if (warp == 0) {
    if (lane == 0) {
      // ---------------- TMA producer ----------------
      int stage = 0;
      uint32_t phase = 0;
      int ready_tile = -1;
      bool ok = true;
      for (int t = blockIdx.x; ok && t < total_tiles; t += gridDim.x) {
        const int j = t / mt;
        const int i = t - j * mt;
        if (pulling && j != ready_tile) {
          long long bytes_j = w_bytes - static_cast<long long>(j) * tile_bytes;
          if (bytes_j > tile_bytes) bytes_j = tile_bytes;
          const int want = static_cast<int>((bytes_j + kChunk - 1) / kChunk);
          if (!wait_flag_ge_gpu(p.tile_ready + j, want, wait_budget)) {
            *abort_flag = 1;
            fail_code = kStatusTimeoutPeerFlag;
            break;
          }
          fence_proxy_async_all();    // the tile was written by bulk stores of other CTAs
          ready_tile = j;
        }
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait_long(empty0 + 8 * stage, phase ^ 1u, abort_flag, wait_budget)) {
            ok = false;
            fail_code = kStatusTimeoutProducer;
            break;
          }
          const uint32_t fb = full0 + 8 * stage;
          mbar_arrive_expect_tx(fb, kStageBytes);
          tma_load_3d(smem_u32(sA + stage * kABytes), &tmX, fb, kb * BK, i * BM, 0);
          tma_load_3d(smem_u32(sB + stage * kBBytes), &tmW, fb, kb * BK, j * BN, 0);
          if (++stage == kStages) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      // ---------------- MMA issuer ----------------
      const uint32_t idesc = make_idesc_f16(BM, BN, false, false, false);
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      for (int t = blockIdx.x; ok && t < total_tiles; t += gridDim.x) {
        if (!mbar_wait_long(tempty0 + 8 * acc, acc_phase ^ 1u, abort_flag, wait_budget)) {
          fail_code = kStatusTimeoutMma;
          break;
        }
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + static_cast<uint32_t>(acc * BN);
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait_long(full0 + 8 * stage, phase, abort_flag, wait_budget)) {
            ok = false;
            fail_code = kStatusTimeoutMma;
            break;
          }
          tc_fence_after_sync();
          const uint32_t a_base = smem_u32(sA + stage * kABytes);
          const uint32_t b_base = smem_u32(sB + stage * kBBytes);
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            umma_f16_ss(d_tmem, make_smem_desc_sw128(a_base + k * 32, 16, 1024),
                        make_smem_desc_sw128(b_base + k * 32, 16, 1024), idesc, (kb | k) != 0 ? 1u : 0u);
          }
          umma_commit(empty0 + 8 * stage);
          if (++stage == kStages) {
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
  } else if (warp < 6) {
    // ---------------- epilogue (warps 2..5) ----------------
    const int q = warp & 3;
    int acc = 0;
    uint32_t acc_phase = 0;
    const bool vec = ((p.ldy * 2) % 16 == 0) && ((reinterpret_cast<uintptr_t>(p.Y) & 15) == 0);
    for (int t = blockIdx.x; t < total_tiles; t += gridDim.x) {
      const int j = t / mt;
      const int i = t - j * mt;
      if (!mbar_wait_long(tfull0 + 8 * acc, acc_phase, abort_flag, wait_budget)) {
        fail_code = kStatusTimeoutEpilogue;
        break;
      }
      tc_fence_after_sync();
      const int row = i * BM + q * 32 + lane;
      for (int c = 0; c < BN; c += 32) {
        const int col0 = j * BN + c;
        if (col0 >= p.N) break;
        uint32_t r[32];
        tmem_ld_32x32(tmem_base + (static_cast<uint32_t>(q * 32) << 16) + static_cast<uint32_t>(acc * BN + c), r);
        tmem_ld_wait();
        if (row < p.M) {
          __nv_bfloat16* dst = p.Y + static_cast<long long>(row) * p.ldy + col0;
          const int nvalid = min(32, p.N - col0);
          if (vec && nvalid == 32) {
            uint4* d4 = reinterpret_cast<uint4*>(dst);
#pragma unroll
            for (int v = 0; v < 4; ++v) {
              uint4 raw;
              __nv_bfloat16* e = reinterpret_cast<__nv_bfloat16*>(&raw);
#pragma unroll
              for (int x = 0; x < 8; ++x) e[x] = __float2bfloat16_rn(__uint_as_float(r[v * 8 + x]));
              d4[v] = raw;
            }
          } else {
#pragma unroll
            for (int x = 0; x < 32; ++x)
              if (x < nvalid) dst[x] = __float2bfloat16_rn(__uint_as_float(r[x]));
          }
        }
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(tempty0 + 8 * acc);
      acc ^= 1;
      if (acc == 0) acc_phase ^= 1u;
    }
  } else {
    // ---------------- fetch warp (warp 6): owner -> smem -> local W ----------------
    if (lane == 0 && pulling) {
      bool ok = true;
      if (p.pub_flag != nullptr && !wait_flag_ge_sys(p.pub_flag, p.pub_want, p.budget_cycles)) {
        *abort_flag = 1;
        fail_code = kStatusTimeoutPeerFlag;
        ok = false;
      }
      const long long total_chunks = (w_bytes + kChunk - 1) / kChunk;
      const long long first = blockIdx.x;
      const long long stride = gridDim.x;
      auto chunk_bytes = [&](long long c) -> uint32_t {
        const long long left = w_bytes - c * kChunk;
        return static_cast<uint32_t>(left < kChunk ? left : kChunk);
      };
      auto issue = [&](long long k) {
        const long long c = first + k * stride;
        const int b = static_cast<int>(k & 1);
        const uint32_t n = chunk_bytes(c);
        mbar_arrive_expect_tx(fbar0 + 8 * b, n);
        bulk_load_g2s(smem_u32(sF + b * kChunk), p.W_remote + c * kChunk, n, fbar0 + 8 * b);
      };
      const long long n_my = (total_chunks > first) ? (total_chunks - first + stride - 1) / stride : 0;
      if (ok && n_my > 0) issue(0);
      for (long long k = 0; ok && k < n_my; ++k) {
        // every earlier store has completed (wait_group 0 below), so the other buffer is free
        if (k + 1 < n_my) issue(k + 1);
        const int b = static_cast<int>(k & 1);
        if (!mbar_wait_long(fbar0 + 8 * b, static_cast<uint32_t>((k >> 1) & 1), abort_flag, wait_budget)) {
          fail_code = kStatusTimeoutPeerFlag;
          break;
        }
        const long long c = first + k * stride;
        const uint32_t n = chunk_bytes(c);
        fence_proxy_async_smem();
        bulk_store_s2g(p.W_local + c * kChunk, smem_u32(sF + b * kChunk), n);
        bulk_commit_group();
        bulk_wait_group<0>();          // the chunk is in local memory
        fence_proxy_async_all();
        __threadfence();
        red_add_release_gpu(p.tile_ready + static_cast<int>((c * kChunk) / tile_bytes), 1);
      }
    }
  }

  // ---------------- teardown ----------------
  tc_fence_before_sync();
  __syncthreads();
  if (*abort_flag) {
    if (fail_code != 0 && p.status != nullptr) atomicCAS(p.status, 0, fail_code);
    for (int i = 0; i < 64; ++i) __nanosleep(2000);   // let bulk copies still in flight land
    __syncthreads();
  }
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, 2 * BN);
  }
}

using EncodeFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                              const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                              CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                              CUtensorMapFloatOOBfill);

static EncodeFn encode_fn() {
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

static int make_map(CUtensorMap* map, const void* base, long long cols, long long rows, long long ld,
                    int box_rows) {
  EncodeFn enc = encode_fn();
  if (enc == nullptr) return -2;
  cuuint64_t dims[3] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(rows), 1};
  cuuint64_t strides[2] = {static_cast<cuuint64_t>(ld) * 2, static_cast<cuuint64_t>(rows) * ld * 2};
  cuuint32_t box[3] = {BK, static_cast<cuuint32_t>(box_rows), 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : -3;
}

}  // namespace pl
}  // namespace dmuon

extern "C" int dmuon_pull_linear_sm100(const DmuonPullLinearArgs* args, void* stream_v) {
  using namespace dmuon;
  using namespace dmuon::pl;
  const DmuonPullLinearArgs& a = *args;
  if (a.M <= 0 || a.N <= 0 || a.K <= 0) return 0;
  if (a.X == nullptr || a.Y == nullptr || a.W_local == nullptr) return -1;
  if ((a.K % 32) != 0 || (a.ldx % 8) != 0 || (a.ldy % 8) != 0) return -1;
  if ((reinterpret_cast<uintptr_t>(a.X) & 15) || (reinterpret_cast<uintptr_t>(a.W_local) & 15) ||
      (reinterpret_cast<uintptr_t>(a.W_remote) & 15))
    return -1;
  if (a.W_remote != nullptr && a.tile_ready == nullptr) return -1;
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_v);
  static bool attr_set[16] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 16 && !attr_set[dev]) {
    cudaError_t e = cudaFuncSetAttribute(pull_linear_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
    if (e != cudaSuccess) return static_cast<int>(e);
    attr_set[dev] = true;
  }
  int sms = 148;
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  CUtensorMap tmX, tmW;
  int rc = make_map(&tmX, a.X, a.K, a.M, a.ldx, BM);
  if (rc != 0) return rc;
  rc = make_map(&tmW, a.W_local, a.K, a.N, a.K, BN);
  if (rc != 0) return rc;
  Params p;
  p.Y = reinterpret_cast<__nv_bfloat16*>(a.Y);
  p.W_local = reinterpret_cast<unsigned char*>(a.W_local);
  p.W_remote = reinterpret_cast<const unsigned char*>(a.W_remote);
  p.M = a.M; p.N = a.N; p.K = a.K;
  p.ldy = a.ldy;
  p.tile_ready = a.tile_ready;
  p.pub_flag = a.pub_flag;
  p.pub_want = a.pub_want;
  p.budget_cycles = a.budget_cycles > 0 ? a.budget_cycles : 4000000000LL;
  p.status = a.status;
  const long long total = static_cast<long long>((a.M + BM - 1) / BM) * ((a.N + BN - 1) / BN);
  // when pulling, every SM takes part in the transfer even if it has no tile
  int grid = (a.max_ctas > 0 && a.max_ctas < sms) ? a.max_ctas : sms;
  if (a.W_remote == nullptr && total < grid) grid = static_cast<int>(total);
  pull_linear_kernel<<<grid, kThreads, kSmemBytes, stream>>>(tmX, tmW, p);
  count_launch();
  return static_cast<int>(cudaGetLastError());
}
