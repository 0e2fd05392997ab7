// 8-bit operand GEMMs for sm_100a (tcgen05, TMEM accumulators, TMA-fed):
//
//   fp8 e4m3 x fp8 e4m3, per-token x per-channel scales  (w8a8 "fp8" linear layers)
//   fp8 e4m3 x fp8 e4m3, 1x128 activation x 128x128 weight block scales (DeepSeek-V3)
//   int8 x int8 with int32 accumulation, per-token x per-channel scales (w8a8 int8)
//
//   C[M,N] (bf16) = (A[M,K] * B[N,K]^T) scaled (+ bias)
//
// Same structure as the bf16 kernel (gemm_bf16.cu): persistent CTAs, warp 0 TMA producer,
// warp 1 MMA issuer, warps 2..5 epilogue, 128-byte-swizzled K-major tiles (here 128
// elements of K per tile row), double-buffered accumulators.  The block-scaled variant
// uses two-level accumulation: every 128-wide K block is multiplied into a fresh TMEM
// accumulator and promoted into fp32 registers with its scale pair, because the checkpoint's
// scales are arbitrary fp32 values.
//
// Reference ops: csrc/src/linear_quant.cpp:23 (block scaled), csrc/src/dot_bias_quant.cpp:22,
// csrc/src/cutlass_scaled_mm.cpp:34 (per-token x per-channel, fp8 and int8).
#include "common.cuh"

namespace b200 {
namespace gemm8 {

constexpr unsigned int kKernelId = 11;
constexpr int BM = 128;
constexpr int BN = 128;
constexpr int BK = 128;      // elements = bytes
constexpr int UMMA_K = 32;
constexpr int STAGES = 6;
constexpr int kThreads = 192;
constexpr int kABytes = BM * BK;
constexpr int kBBytes = BN * BK;
constexpr int kStageBytes = kABytes + kBBytes;
constexpr int kBarOffset = STAGES * kStageBytes;
constexpr int kSmemTotal = kBarOffset + 256 + 1024;

enum Mode : int { kRowCol = 0, kBlock128 = 1 };

struct Args {
  __nv_bfloat16* C;
  long long ldc;
  const float* a_scale;   // kRowCol: [M]; kBlock128: [M, K/128] (row pitch lds_a)
  const float* b_scale;   // kRowCol: [N]; kBlock128: [ceil(N/128), K/128] (row pitch lds_b)
  const __nv_bfloat16* bias;
  long long lds_a, lds_b;
  int M, N, K;
  int tiles_m, tiles_n;
  // grouped (mixture-of-experts) mode: A rows are sorted by expert in tiles of BM rows,
  // expert_ids[tile_m] names the weight matrix of a row tile (-1 or a tile at / past
  // *num_post_pad: nothing to do), B holds the experts' [N, K] matrices one after the other,
  // b_scale their scale tables, row_scale an optional per-row factor (routing weight)
  const int* expert_ids;
  const int* num_post_pad;
  const float* row_scale;
  unsigned int* status;
};

// Expert of a row tile, or -1 when the tile has no work.  Every role of the CTA evaluates it
// on the same data, so they skip the same tiles.
__device__ __forceinline__ int tile_expert(const Args& p, int m0) {
  if (p.expert_ids == nullptr) return 0;
  if (m0 >= *p.num_post_pad) return -1;
  return p.expert_ids[m0 / BM];
}

template <bool INT8>
__device__ __forceinline__ void mma8(uint32_t tmem_d, uint64_t da, uint64_t db, uint32_t idesc,
                                     uint32_t acc) {
  if constexpr (INT8) umma_i8(tmem_d, da, db, idesc, acc);
  else umma_f8(tmem_d, da, db, idesc, acc);
}

template <bool INT8, int MODE>
__global__ void __launch_bounds__(kThreads, 1)
    gemm_q8_kernel(const __grid_constant__ CUtensorMap tmA,
                   const __grid_constant__ CUtensorMap tmB, const Args p) {
  constexpr uint32_t kTmemCols = 2 * BN;
  // int8: formats = signed 8-bit (1), accumulator S32 (2); fp8: e4m3 (0), accumulator F32 (1)
  constexpr uint32_t kIdesc = INT8 ? make_idesc(BM, BN, 1, 1, 2) : make_idesc(BM, BN, 0, 0, 1);

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + kBarOffset);
  uint64_t* empty_bar = full_bar + STAGES;
  uint64_t* tfull_bar = empty_bar + STAGES;
  uint64_t* tempty_bar = tfull_bar + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty_bar + 2);
  volatile uint32_t* abort_flag = tmem_slot + 1;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(&tfull_bar[a], 1);
      mbar_init(&tempty_bar[a], 4);
    }
    *abort_flag = 0u;
    mbar_fence_init();
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const int num_kb = (p.K + BK - 1) / BK;
  const int num_tiles = p.tiles_m * p.tiles_n;

  if (warp == 0) {
    if (elect_one()) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; ok && tile < num_tiles; tile += gridDim.x) {
        const int m0 = (tile % p.tiles_m) * BM, n0 = (tile / p.tiles_m) * BN;
        const int expert = tile_expert(p, m0);
        if (expert < 0) continue;
        const int b_row = expert * p.N + n0;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1u, p.status, kKernelId, 0x100u + stage,
                         abort_flag)) {
            ok = false;
            break;
          }
          uint8_t* sa = smem + stage * kStageBytes;
          mbar_expect_tx(&full_bar[stage], kStageBytes);
          tma_load_2d(sa, &tmA, &full_bar[stage], kb * BK, m0);
          tma_load_2d(sa + kABytes, &tmB, &full_bar[stage], kb * BK, b_row);
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
      }
    }
  } else if (warp == 1) {
    if (elect_one()) {
      int stage = 0;
      uint32_t phase = 0;
      // accumulator hand-off granularity: per tile (kRowCol) or per K block (kBlock128)
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; ok && tile < num_tiles; tile += gridDim.x) {
        if (tile_expert(p, (tile % p.tiles_m) * BM) < 0) continue;
        if constexpr (MODE == kRowCol) {
          if (!mbar_wait(&tempty_bar[acc], acc_phase ^ 1u, p.status, kKernelId, 0x200u + acc,
                         abort_flag))
            break;
          tc_fence_after();
        }
        for (int kb = 0; kb < num_kb; ++kb) {
          if constexpr (MODE == kBlock128) {
            if (!mbar_wait(&tempty_bar[acc], acc_phase ^ 1u, p.status, kKernelId, 0x200u + acc,
                           abort_flag)) {
              ok = false;
              break;
            }
            tc_fence_after();
          }
          if (!mbar_wait(&full_bar[stage], phase, p.status, kKernelId, 0x300u + stage,
                         abort_flag)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t tmem_d = tmem_base + static_cast<uint32_t>(acc * BN);
          const uint32_t a_addr = smem_u32(smem + stage * kStageBytes);
          const uint64_t adesc = make_desc_k_sw128(a_addr);
          const uint64_t bdesc = make_desc_k_sw128(a_addr + kABytes);
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            const uint32_t accumulate =
                (MODE == kBlock128) ? (k != 0 ? 1u : 0u) : ((kb | k) != 0 ? 1u : 0u);
            mma8<INT8>(tmem_d, adesc + static_cast<uint64_t>(k * 2),
                       bdesc + static_cast<uint64_t>(k * 2), kIdesc, accumulate);
          }
          umma_commit(&empty_bar[stage]);
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
          if constexpr (MODE == kBlock128) {
            umma_commit(&tfull_bar[acc]);
            acc ^= 1;
            if (acc == 0) acc_phase ^= 1u;
          }
        }
        if (!ok) break;
        if constexpr (MODE == kRowCol) {
          umma_commit(&tfull_bar[acc]);
          acc ^= 1;
          if (acc == 0) acc_phase ^= 1u;
        }
      }
    }
  } else {
    const int q = warp & 3;
    int acc = 0;
    uint32_t acc_phase = 0;
    bool ok = true;
    for (int tile = blockIdx.x; ok && tile < num_tiles; tile += gridDim.x) {
      const int m0 = (tile % p.tiles_m) * BM, n0 = (tile / p.tiles_m) * BN;
      const int expert = tile_expert(p, m0);
      if (expert < 0) continue;
      const int row = m0 + q * 32 + lane;
      const bool row_ok = row < p.M;
      const float rs = (p.row_scale != nullptr && row_ok) ? p.row_scale[row] : 1.0f;
      const uint32_t lane_addr = tmem_base + (static_cast<uint32_t>(q * 32) << 16);
      __nv_bfloat16* crow = p.C + static_cast<long long>(row) * p.ldc;

      if constexpr (MODE == kRowCol) {
        if (!mbar_wait(&tfull_bar[acc], acc_phase, p.status, kKernelId, 0x400u + acc, abort_flag))
          break;
        tc_fence_after();
        const float sa = row_ok ? p.a_scale[row] * rs : 0.0f;
        const float* b_scale = p.b_scale + static_cast<long long>(expert) * p.N;
#pragma unroll 1
        for (int c = 0; c < BN / 32; ++c) {
          uint32_t r[32];
          tmem_ld_32x32(lane_addr + acc * BN + c * 32, r);
          tmem_ld_wait();
          const int col = n0 + c * 32;
          if (!row_ok || col >= p.N) continue;
          const int ncols = min(32, p.N - col);
          float v[32];
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const float a = INT8 ? static_cast<float>(static_cast<int32_t>(r[i]))
                                 : __uint_as_float(r[i]);
            v[i] = a * sa;
          }
          for (int i = 0; i < ncols; ++i) {
            v[i] *= b_scale[col + i];
            if (p.bias != nullptr) v[i] += __bfloat162float(p.bias[col + i]);
          }
          if (ncols == 32) {
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              uint4 u;
              u.x = pack_bf16x2(v[i * 8 + 0], v[i * 8 + 1]);
              u.y = pack_bf16x2(v[i * 8 + 2], v[i * 8 + 3]);
              u.z = pack_bf16x2(v[i * 8 + 4], v[i * 8 + 5]);
              u.w = pack_bf16x2(v[i * 8 + 6], v[i * 8 + 7]);
              reinterpret_cast<uint4*>(crow + col)[i] = u;
            }
          } else {
            for (int i = 0; i < ncols; ++i) crow[col + i] = __float2bfloat16(v[i]);
          }
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&tempty_bar[acc]);
        acc ^= 1;
        if (acc == 0) acc_phase ^= 1u;
      } else {
        // two-level accumulation: promote every K block with its scale pair
        float accum[BN];
#pragma unroll
        for (int i = 0; i < BN; ++i) accum[i] = 0.0f;
        const float* sa_row = p.a_scale + static_cast<long long>(row_ok ? row : 0) * p.lds_a;
        const float* sb_row =
            p.b_scale + (static_cast<long long>(expert) * ((p.N + 127) / 128) + n0 / 128) * p.lds_b;
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(&tfull_bar[acc], acc_phase, p.status, kKernelId, 0x400u + acc,
                         abort_flag)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const float s = sa_row[kb] * sb_row[kb];
#pragma unroll
          for (int c = 0; c < BN / 32; ++c) {
            uint32_t r[32];
            tmem_ld_32x32(lane_addr + acc * BN + c * 32, r);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) accum[c * 32 + i] += __uint_as_float(r[i]) * s;
          }
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(&tempty_bar[acc]);
          acc ^= 1;
          if (acc == 0) acc_phase ^= 1u;
        }
        if (!ok) break;
        if (row_ok) {
#pragma unroll
          for (int c = 0; c < BN / 8; ++c) {
            const int col = n0 + c * 8;
            if (col >= p.N) break;
            float v[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              v[i] = accum[c * 8 + i] * rs;
              if (p.bias != nullptr && col + i < p.N) v[i] += __bfloat162float(p.bias[col + i]);
            }
            if (col + 8 <= p.N) {
              uint4 u;
              u.x = pack_bf16x2(v[0], v[1]);
              u.y = pack_bf16x2(v[2], v[3]);
              u.z = pack_bf16x2(v[4], v[5]);
              u.w = pack_bf16x2(v[6], v[7]);
              *reinterpret_cast<uint4*>(crow + col) = u;
            } else {
              for (int i = 0; col + i < p.N; ++i) crow[col + i] = __float2bfloat16(v[i]);
            }
          }
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_base, kTmemCols);
}

template <bool INT8, int MODE>
int launch(const CUtensorMap& tmA, const CUtensorMap& tmB, const Args& a, cudaStream_t stream) {
  auto kern = gemm_q8_kernel<INT8, MODE>;
  static bool configured[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !configured[dev]) {
    cudaError_t e =
        cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemTotal);
    if (e != cudaSuccess) return static_cast<int>(e);
    configured[dev] = true;
  }
  const int tiles = a.tiles_m * a.tiles_n;
  const int grid = tiles < sm_count() ? tiles : sm_count();
  kern<<<grid, kThreads, kSmemTotal, stream>>>(tmA, tmB, a);
  return static_cast<int>(cudaGetLastError());
}

}  // namespace gemm8
}  // namespace b200

// kind: 0 fp8 e4m3 row x col scales, 1 fp8 e4m3 block scales (1x128 / 128x128),
//       2 int8 row x col scales.
// A [M,K], B [N,K] one byte per element, row pitches lda / ldb in bytes (multiples of 16);
// C bf16 [M,N]; K a multiple of 16 (128 for kind 1).
B200_API int b200_gemm_q8(const void* A, long long lda, const void* B, long long ldb, void* C,
                          long long ldc, int M, int N, int K, const float* a_scale,
                          long long lds_a, const float* b_scale, long long lds_b,
                          const void* bias, int kind, void* stream) {
  using namespace b200;
  using namespace b200::gemm8;
  if (M <= 0 || N <= 0) return 0;
  if (K <= 0 || (K % 16) != 0 || (lda % 16) != 0 || (ldb % 16) != 0 || (N % 8) != 0 ||
      (ldc % 8) != 0 || a_scale == nullptr || b_scale == nullptr)
    return -2;
  if (kind == 1 && (K % 128) != 0) return -2;
  CUtensorMap tmA, tmB;
  int r = encode_tmap_2d(&tmA, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, A, static_cast<uint64_t>(M),
                         static_cast<uint64_t>(K), static_cast<uint64_t>(lda), BM, BK,
                         CU_TENSOR_MAP_SWIZZLE_128B);
  if (r != 0) return r < 0 ? -6 : r;
  r = encode_tmap_2d(&tmB, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, B, static_cast<uint64_t>(N),
                     static_cast<uint64_t>(K), static_cast<uint64_t>(ldb), BN, BK,
                     CU_TENSOR_MAP_SWIZZLE_128B);
  if (r != 0) return r < 0 ? -6 : r;
  Args a;
  a.C = static_cast<__nv_bfloat16*>(C);
  a.ldc = ldc;
  a.a_scale = a_scale;
  a.b_scale = b_scale;
  a.bias = static_cast<const __nv_bfloat16*>(bias);
  a.lds_a = lds_a;
  a.lds_b = lds_b;
  a.M = M; a.N = N; a.K = K;
  a.tiles_m = (M + BM - 1) / BM;
  a.tiles_n = (N + BN - 1) / BN;
  a.expert_ids = nullptr; a.num_post_pad = nullptr; a.row_scale = nullptr;
  a.status = status_ptr();
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (kind == 0) return launch<false, kRowCol>(tmA, tmB, a, s);
  if (kind == 1) return launch<false, kBlock128>(tmA, tmB, a, s);
  if (kind == 2) return launch<true, kRowCol>(tmA, tmB, a, s);
  return -7;
}

// Grouped (mixture-of-experts) form of b200_gemm_q8: A [M_cap, K] holds the token rows sorted
// by expert in tiles of 128 rows (b200_moe_align), B [E * N, K] the experts' weights, b_scale
// [E, N] (kind 0 / 2) or [E, ceil(N / 128), K / 128] (kind 1), row_scale an optional
// per-row factor applied to the output.  Tiles whose expert id is negative or that start at
// or past *num_post_pad are skipped.  Replaces the quantised branches of the reference's
// fused_moe_kernel / fused_moe_quant_kernel (csrc/torch_bindings.cpp:118-178).
B200_API int b200_gemm_q8_grouped(const void* A, long long lda, const void* B, long long ldb,
                                  void* C, long long ldc, int M_cap, int N, int K, int E,
                                  const float* a_scale, long long lds_a, const float* b_scale,
                                  long long lds_b, const int* expert_ids,
                                  const int* num_post_pad, const float* row_scale, int kind,
                                  void* stream) {
  using namespace b200;
  using namespace b200::gemm8;
  if (M_cap <= 0 || N <= 0 || E <= 0) return 0;
  if (K <= 0 || (K % 16) != 0 || (lda % 16) != 0 || (ldb % 16) != 0 || (N % 8) != 0 ||
      (ldc % 8) != 0 || (M_cap % BM) != 0 || a_scale == nullptr || b_scale == nullptr ||
      expert_ids == nullptr || num_post_pad == nullptr)
    return -2;
  if (kind == 1 && (K % 128) != 0) return -2;
  CUtensorMap tmA, tmB;
  int r = encode_tmap_2d(&tmA, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, A, static_cast<uint64_t>(M_cap),
                         static_cast<uint64_t>(K), static_cast<uint64_t>(lda), BM, BK,
                         CU_TENSOR_MAP_SWIZZLE_128B);
  if (r != 0) return r < 0 ? -6 : r;
  r = encode_tmap_2d(&tmB, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, B,
                     static_cast<uint64_t>(E) * static_cast<uint64_t>(N), static_cast<uint64_t>(K),
                     static_cast<uint64_t>(ldb), BN, BK, CU_TENSOR_MAP_SWIZZLE_128B);
  if (r != 0) return r < 0 ? -6 : r;
  Args a;
  a.C = static_cast<__nv_bfloat16*>(C);
  a.ldc = ldc;
  a.a_scale = a_scale;
  a.b_scale = b_scale;
  a.bias = nullptr;
  a.lds_a = lds_a;
  a.lds_b = lds_b;
  a.M = M_cap; a.N = N; a.K = K;
  a.tiles_m = M_cap / BM;
  a.tiles_n = (N + BN - 1) / BN;
  a.expert_ids = expert_ids; a.num_post_pad = num_post_pad; a.row_scale = row_scale;
  a.status = status_ptr();
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (kind == 0) return launch<false, kRowCol>(tmA, tmB, a, s);
  if (kind == 1) return launch<false, kBlock128>(tmA, tmB, a, s);
  if (kind == 2) return launch<true, kRowCol>(tmA, tmB, a, s);
  return -7;
}
