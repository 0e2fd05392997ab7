// bf16 GEMM for decode-sized activations:  C[M,N] = A[M,K] * B[N,K]^T,  M <= 256.
//
// With M <= 256 every weight byte is used once, so the kernel is bound by how fast the weight
// matrix streams through the machine.  The persistent 128-row-tile kernel (gemm_bf16.cu) reads
// each weight tile through L2 once per 128-row tile and re-reads the activation tile for
// every column tile; at M = 256 that moves 3-6 bytes from L2 into shared memory per weight
// byte and the L2 -> SM path, not HBM, is the limit.  This kernel instead gives one CTA the whole M
// extent of a column tile:
//
//   * one work unit = (column tile of BN weights rows) x (K slice); one unit per CTA, all
//     units of a problem resident at once (units <= SM count) unless there is no K split;
//   * per pipeline stage TMA brings one BN x 64 weight tile and one or two 128 x 64
//     activation tiles; the MMA warp issues two tcgen05.mma (rows 0-127 and 128-255) against
//     the same weight tile in shared memory, accumulating into two TMEM regions;
//   * K is split so that about one unit exists per SM even when N / BN is small
//     (o_proj, down_proj).  The CTAs of a column tile write fp32 partial sums to an L2-resident
//     workspace, meet at a counter (bounded wait), and each reduces a row slice of the tile
//     in a fixed order (bitwise reproducible), applying the epilogue;
//   * epilogues: none, + bias, SiLU(gate) * up (gate / up interleaved in blocks of 32 rows).
//
// Replaces the vendor matmul behind the decode path of every unquantised linear layer of the
// reference (vllm_gcu/kernels/linear.py; SiluAndMul of vllm_gcu/kernels/activation.py:20-32
// folded into the gate-up projection).
#include "common.cuh"

#include <cstdlib>

namespace b200 {
namespace skinny {

constexpr unsigned int kKernelId = 11;
constexpr int BM = 128;
constexpr int BK = 64;
constexpr int UMMA_K = 16;
constexpr int kThreads = 192;

enum Epi : int { kNone = 0, kBias = 1, kSiluMul = 2 };

struct Args {
  __nv_bfloat16* C;
  long long ldc;
  const __nv_bfloat16* bias;
  int M, N, K;
  int tiles_n, splits, num_kb;
  float* ws;            // [units][MT * 128][BN] fp32 partial sums (splits > 1)
  unsigned int* ctr;    // [tiles_n][2] arrive / depart counters, zero between launches
  unsigned int* status;
};

template <int BN, int MT, int STAGES>
struct Smem {
  static constexpr int kABytes = BM * BK * 2;
  static constexpr int kBBytes = BN * BK * 2;
  static constexpr int kStageBytes = MT * kABytes + kBBytes;
  static constexpr int kBarOffset = STAGES * kStageBytes;
  static constexpr int kTotal = kBarOffset + 256 + 1024;
  static_assert(kTotal <= 232448, "exceeds the shared memory of one CTA");
};

__device__ __forceinline__ void store8_bf16(__nv_bfloat16* dst, const float* v) {
  uint4 u;
  u.x = pack_bf16x2(v[0], v[1]);
  u.y = pack_bf16x2(v[2], v[3]);
  u.z = pack_bf16x2(v[4], v[5]);
  u.w = pack_bf16x2(v[6], v[7]);
  *reinterpret_cast<uint4*>(dst) = u;
}

template <int BN, int MT, int STAGES, int EPI>
__global__ void __launch_bounds__(kThreads, 1)
    gemm_skinny_kernel(const __grid_constant__ CUtensorMap tmA,
                       const __grid_constant__ CUtensorMap tmB, const Args p) {
  using L = Smem<BN, MT, STAGES>;
  constexpr uint32_t kAccCols = MT * BN;
  constexpr uint32_t kTmemCols = kAccCols <= 32 ? 32 : (kAccCols <= 64 ? 64 : (kAccCols <= 128 ? 128 : (kAccCols <= 256 ? 256 : 512)));
  constexpr uint32_t kIdesc = make_idesc(BM, BN, 1, 1);
  static_assert(EPI != kSiluMul || BN == 256, "SiLU-mul epilogue needs BN = 256");

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + L::kBarOffset);
  uint64_t* empty_bar = full_bar + STAGES;
  uint64_t* tfull_bar = empty_bar + STAGES;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tfull_bar + 1);
  volatile uint32_t* abort_flag = tmem_slot + 1;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    mbar_init(tfull_bar, 1);
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

  const int unit = blockIdx.x;
  const int tile = unit / p.splits;
  const int split = unit - tile * p.splits;
  const int n0 = tile * BN;
  const int kb0 = static_cast<int>(static_cast<long long>(split) * p.num_kb / p.splits);
  const int kb1 = static_cast<int>(static_cast<long long>(split + 1) * p.num_kb / p.splits);

  if (warp == 0) {
    if (elect_one()) {
      int stage = 0;
      uint32_t phase = 0;
      for (int kb = kb0; kb < kb1; ++kb) {
        if (!mbar_wait(&empty_bar[stage], phase ^ 1u, p.status, kKernelId, 0x100u + stage,
                       abort_flag))
          break;
        uint8_t* sa = smem + stage * L::kStageBytes;
        uint8_t* sb = sa + MT * L::kABytes;
        mbar_expect_tx(&full_bar[stage], L::kStageBytes);
        tma_load_2d(sb, &tmB, &full_bar[stage], kb * BK, n0);
#pragma unroll
        for (int mt = 0; mt < MT; ++mt)
          tma_load_2d(sa + mt * L::kABytes, &tmA, &full_bar[stage], kb * BK, mt * BM);
        if (++stage == STAGES) {
          stage = 0;
          phase ^= 1u;
        }
      }
    }
  } else if (warp == 1) {
    if (elect_one()) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int kb = kb0; kb < kb1; ++kb) {
        if (!mbar_wait(&full_bar[stage], phase, p.status, kKernelId, 0x300u + stage, abort_flag)) {
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t a_addr = smem_u32(smem + stage * L::kStageBytes);
        const uint32_t b_addr = a_addr + MT * L::kABytes;
        const uint64_t bdesc = make_desc_k_sw128(b_addr);
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) {
          const uint64_t adesc = make_desc_k_sw128(a_addr + mt * L::kABytes);
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k)
            umma_f16(tmem_base + static_cast<uint32_t>(mt * BN),
                     adesc + static_cast<uint64_t>(k * 2), bdesc + static_cast<uint64_t>(k * 2),
                     kIdesc, (kb > kb0 || k > 0) ? 1u : 0u);
        }
        umma_commit(&empty_bar[stage]);
        if (++stage == STAGES) {
          stage = 0;
          phase ^= 1u;
        }
      }
      if (ok) umma_commit(tfull_bar);
    }
  } else {
    // ---------------- epilogue (warps 2..5) ----------------
    const int q = warp & 3;
    const int te = threadIdx.x - 64;
    mbar_wait(tfull_bar, 0u, p.status, kKernelId, 0x400u, abort_flag);   // sets abort on timeout
    asm volatile("bar.sync 1, 128;" ::: "memory");
    const bool have = *abort_flag == 0u;     // the same answer in all epilogue threads
    tc_fence_after();
    if (have && p.splits == 1) {
#pragma unroll 1
      for (int mt = 0; mt < MT; ++mt) {
        const int row = mt * BM + q * 32 + lane;
        const bool row_ok = row < p.M;
        const uint32_t taddr =
            tmem_base + (static_cast<uint32_t>(q * 32) << 16) + static_cast<uint32_t>(mt * BN);
        if constexpr (EPI == kSiluMul) {
          __nv_bfloat16* crow = p.C + static_cast<long long>(row) * p.ldc + (n0 >> 1);
          const int out_n = p.N >> 1;
#pragma unroll 1
          for (int c = 0; c < 4; ++c) {
            // 64-column group c of the tile: 32 gate columns, then the 32 matching up columns
            uint32_t g[32], u[32];
            tmem_ld_32x32(taddr + c * 64, g);
            tmem_ld_32x32(taddr + c * 64 + 32, u);
            tmem_ld_wait();
            float v[32];
#pragma unroll
            for (int i = 0; i < 32; ++i)
              v[i] = silu_f(__uint_as_float(g[i])) * __uint_as_float(u[i]);
            if (row_ok && (n0 >> 1) + c * 32 < out_n) {
#pragma unroll
              for (int i = 0; i < 4; ++i) store8_bf16(crow + c * 32 + i * 8, v + i * 8);
            }
          }
        } else {
#pragma unroll 1
          for (int c = 0; c < BN / 32; ++c) {
            uint32_t r[32];
            tmem_ld_32x32(taddr + c * 32, r);
            tmem_ld_wait();
            const int col = n0 + c * 32;
            if (!row_ok || col >= p.N) continue;
            float v[32];
#pragma unroll
            for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
            __nv_bfloat16* crow = p.C + static_cast<long long>(row) * p.ldc + col;
            if (col + 32 <= p.N) {
              if constexpr (EPI == kBias) {
#pragma unroll
                for (int i = 0; i < 32; ++i) v[i] += __bfloat162float(p.bias[col + i]);
              }
#pragma unroll
              for (int i = 0; i < 4; ++i) store8_bf16(crow + i * 8, v + i * 8);
            } else {
              for (int i = 0; i < p.N - col; ++i) {
                float x = v[i];
                if constexpr (EPI == kBias) x += __bfloat162float(p.bias[col + i]);
                crow[i] = __float2bfloat16(x);
              }
            }
          }
        }
      }
    } else if (have) {
      // ---- split K: park the fp32 partial, meet the other K slices, reduce a row slice ----
      constexpr int R = MT * BM;
      float* mine = p.ws + static_cast<long long>(unit) * (R * BN);
#pragma unroll 1
      for (int mt = 0; mt < MT; ++mt) {
        const int row = mt * BM + q * 32 + lane;
        const uint32_t taddr =
            tmem_base + (static_cast<uint32_t>(q * 32) << 16) + static_cast<uint32_t>(mt * BN);
#pragma unroll 1
        for (int c = 0; c < BN / 32; ++c) {
          uint32_t r[32];
          tmem_ld_32x32(taddr + c * 32, r);
          tmem_ld_wait();
          if (row >= p.M) continue;
          float4* dst = reinterpret_cast<float4*>(mine + static_cast<long long>(row) * BN + c * 32);
#pragma unroll
          for (int i = 0; i < 8; ++i)
            dst[i] = make_float4(__uint_as_float(r[i * 4]), __uint_as_float(r[i * 4 + 1]),
                                 __uint_as_float(r[i * 4 + 2]), __uint_as_float(r[i * 4 + 3]));
        }
      }
      // ctr == nullptr: a second kernel adds the partial sums (no CTA waits for another)
      if (p.ctr != nullptr) {
      __threadfence();
      asm volatile("bar.sync 1, 128;" ::: "memory");
      unsigned int* arrive = p.ctr + 2 * tile;
      unsigned int* depart = arrive + 1;
      if (te == 0) {
        atomicAdd(arrive, 1u);
        bool ok = false;
        for (uint32_t it = 0; it < (1u << 22); ++it) {
          unsigned int v;
          asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(arrive) : "memory");
          if (v >= static_cast<unsigned int>(p.splits)) { ok = true; break; }
          if (it > 32) __nanosleep(64);
        }
        if (!ok) {
          report_status(p.status, kStatusFlagTimeout, kKernelId, 0x500u);
          *abort_flag = 1u;
        }
      }
      asm volatile("bar.sync 1, 128;" ::: "memory");
      if (*abort_flag == 0u) {
        const int rows_used = min(p.M, R);
        const int r0 = static_cast<int>(static_cast<long long>(split) * rows_used / p.splits);
        const int r1 = static_cast<int>(static_cast<long long>(split + 1) * rows_used / p.splits);
        const float* base = p.ws + static_cast<long long>(tile) * p.splits * (R * BN);
        if constexpr (EPI == kSiluMul) {
          constexpr int kV = 128 / 4;   // float4 groups of the gate half
          const int out_n = p.N >> 1;
          for (int e = te; e < (r1 - r0) * kV; e += 128) {
            const int row = r0 + e / kV, c4 = (e % kV) * 4;
            // output column c4 of the tile: gate at (c4 / 32) * 64 + c4 % 32, up 32 further
            const int gcol = (c4 >> 5) * 64 + (c4 & 31);
            float4 g = make_float4(0.f, 0.f, 0.f, 0.f), u = g;
            for (int s = 0; s < p.splits; ++s) {
              const float* src = base + static_cast<long long>(s) * (R * BN) +
                                 static_cast<long long>(row) * BN + gcol;
              const float4 a = __ldcg(reinterpret_cast<const float4*>(src));
              const float4 b = __ldcg(reinterpret_cast<const float4*>(src + 32));
              g.x += a.x; g.y += a.y; g.z += a.z; g.w += a.w;
              u.x += b.x; u.y += b.y; u.z += b.z; u.w += b.w;
            }
            const int col = (n0 >> 1) + c4;
            if (col < out_n) {
              uint2 o;
              o.x = pack_bf16x2(silu_f(g.x) * u.x, silu_f(g.y) * u.y);
              o.y = pack_bf16x2(silu_f(g.z) * u.z, silu_f(g.w) * u.w);
              *reinterpret_cast<uint2*>(p.C + static_cast<long long>(row) * p.ldc + col) = o;
            }
          }
        } else {
          constexpr int kV = BN / 4;
          for (int e = te; e < (r1 - r0) * kV; e += 128) {
            const int row = r0 + e / kV, c4 = (e % kV) * 4;
            float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
            for (int s = 0; s < p.splits; ++s) {
              const float4 a = __ldcg(reinterpret_cast<const float4*>(
                  base + static_cast<long long>(s) * (R * BN) + static_cast<long long>(row) * BN + c4));
              acc.x += a.x; acc.y += a.y; acc.z += a.z; acc.w += a.w;
            }
            const int col = n0 + c4;
            if (col >= p.N) continue;
            if constexpr (EPI == kBias) {
              acc.x += __bfloat162float(p.bias[col]);
              acc.y += __bfloat162float(p.bias[col + 1]);
              acc.z += __bfloat162float(p.bias[col + 2]);
              acc.w += __bfloat162float(p.bias[col + 3]);
            }
            uint2 o;
            o.x = pack_bf16x2(acc.x, acc.y);
            o.y = pack_bf16x2(acc.z, acc.w);
            *reinterpret_cast<uint2*>(p.C + static_cast<long long>(row) * p.ldc + col) = o;
          }
        }
      }
      // the last CTA of the tile to leave clears both counters for the next launch
      asm volatile("bar.sync 1, 128;" ::: "memory");
      if (te == 0 && *abort_flag == 0u) {
        if (atomicAdd(depart, 1u) == static_cast<unsigned int>(p.splits) - 1u) {
          *arrive = 0u;
          *depart = 0u;
        }
      }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_base, kTmemCols);
}

template <int BN, int MT, int STAGES, int EPI>
int launch(const CUtensorMap& tmA, const CUtensorMap& tmB, const Args& a, int units,
           cudaStream_t stream) {
  using L = Smem<BN, MT, STAGES>;
  auto kern = gemm_skinny_kernel<BN, MT, STAGES, EPI>;
  static bool configured[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !configured[dev]) {
    cudaError_t e =
        cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kTotal);
    if (e != cudaSuccess) return static_cast<int>(e);
    configured[dev] = true;
  }
  kern<<<units, kThreads, L::kTotal, stream>>>(tmA, tmB, a);
  return static_cast<int>(cudaGetLastError());
}

// ---------------------------------------------------------------------------
// Persistent 256 x 256 tiles for large M: same shared-memory stage as above (two 128-row
// activation tiles + one 256-row weight tile per 64 of K), so a CTA moves 64 KB from L2 per
// 2 x 512 tensor-core cycles - two thirds of what the 128 x 256 tiles of gemm_bf16.cu move -
// at the price of a single accumulator set (all 512 TMEM columns): the MMA of the next tile
// starts when the epilogue warps have read the accumulators of this one.
// ---------------------------------------------------------------------------
struct WideArgs {
  __nv_bfloat16* C;
  long long ldc;
  const __nv_bfloat16* bias;
  int M, N, K;
  int tiles_m, tiles_n, num_kb;
  int group_m;          // M tiles per raster group (see wide_tile)
  unsigned int* status;
};

// Tile order of the persistent CTAs: groups of `group_m` row panels, and inside a group the
// row index runs fastest.  The ~148 tiles that are in flight at one time then cover about
// group_m row panels x 148 / group_m column panels instead of all row panels x a few column
// panels, which is the smallest set of A and B panels (the square) for that many tiles: fewer
// bytes per wave from L2 and DRAM.
__device__ __forceinline__ void wide_tile(const WideArgs& p, int tile, int& tm, int& tn) {
  const int group = p.group_m * p.tiles_n;
  const int g = tile / group;
  const int first = g * p.group_m;
  const int gm = min(p.tiles_m - first, p.group_m);
  const int r = tile - g * group;
  tm = first + r % gm;
  tn = r / gm;
}

template <int EPI>
__global__ void __launch_bounds__(kThreads, 1)
    gemm_wide2_kernel(const __grid_constant__ CUtensorMap tmA,
                      const __grid_constant__ CUtensorMap tmB, const WideArgs p) {
  constexpr int BN = 256, MT = 2, STAGES = 3;
  using L = Smem<BN, MT, STAGES>;
  constexpr uint32_t kTmemCols = 512;
  constexpr uint32_t kIdesc = make_idesc(BM, BN, 1, 1);

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + L::kBarOffset);
  uint64_t* empty_bar = full_bar + STAGES;
  uint64_t* tfull_bar = empty_bar + STAGES;
  uint64_t* tempty_bar = tfull_bar + 1;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty_bar + 1);
  volatile uint32_t* abort_flag = tmem_slot + 1;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 1);
    }
    mbar_init(tfull_bar, 1);
    mbar_init(tempty_bar, 4);
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
  const int num_tiles = p.tiles_m * p.tiles_n;

  if (warp == 0) {
    if (elect_one()) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; ok && tile < num_tiles; tile += gridDim.x) {
        int tm, tn;
        wide_tile(p, tile, tm, tn);
        const int m0 = tm * (MT * BM), n0 = tn * BN;
        for (int kb = 0; kb < p.num_kb; ++kb) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1u, p.status, kKernelId, 0x900u + stage,
                         abort_flag)) {
            ok = false;
            break;
          }
          uint8_t* sa = smem + stage * L::kStageBytes;
          uint8_t* sb = sa + MT * L::kABytes;
          mbar_expect_tx(&full_bar[stage], L::kStageBytes);
          tma_load_2d(sb, &tmB, &full_bar[stage], kb * BK, n0);
          tma_load_2d(sa, &tmA, &full_bar[stage], kb * BK, m0);
          tma_load_2d(sa + L::kABytes, &tmA, &full_bar[stage], kb * BK, m0 + BM);
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
    }
  } else if (warp == 1) {
    if (elect_one()) {
      int stage = 0;
      uint32_t phase = 0, tphase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; ok && tile < num_tiles; tile += gridDim.x) {
        if (!mbar_wait(tempty_bar, tphase ^ 1u, p.status, kKernelId, 0x910u, abort_flag)) break;
        tc_fence_after();
        for (int kb = 0; kb < p.num_kb; ++kb) {
          if (!mbar_wait(&full_bar[stage], phase, p.status, kKernelId, 0x920u + stage,
                         abort_flag)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t a_addr = smem_u32(smem + stage * L::kStageBytes);
          const uint32_t b_addr = a_addr + MT * L::kABytes;
          const uint64_t bdesc = make_desc_k_sw128(b_addr);
#pragma unroll
          for (int mt = 0; mt < MT; ++mt) {
            const uint64_t adesc = make_desc_k_sw128(a_addr + mt * L::kABytes);
#pragma unroll
            for (int k = 0; k < BK / UMMA_K; ++k)
              umma_f16(tmem_base + static_cast<uint32_t>(mt * BN),
                       adesc + static_cast<uint64_t>(k * 2), bdesc + static_cast<uint64_t>(k * 2),
                       kIdesc, (kb | k) != 0 ? 1u : 0u);
          }
          umma_commit(&empty_bar[stage]);
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (!ok) break;
        umma_commit(tfull_bar);
        tphase ^= 1u;
      }
    }
  } else {
    const int q = warp & 3;
    uint32_t tphase = 0;
    for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x) {
      int tm, tn;
      wide_tile(p, tile, tm, tn);
      const int m0 = tm * (MT * BM), n0 = tn * BN;
      if (!mbar_wait(tfull_bar, tphase, p.status, kKernelId, 0x930u, abort_flag)) break;
      tc_fence_after();
#pragma unroll 1
      for (int mt = 0; mt < MT; ++mt) {
        const int row = m0 + mt * BM + q * 32 + lane;
        const bool row_ok = row < p.M;
        const uint32_t taddr =
            tmem_base + (static_cast<uint32_t>(q * 32) << 16) + static_cast<uint32_t>(mt * BN);
        if constexpr (EPI == kSiluMul) {
          __nv_bfloat16* crow = p.C + static_cast<long long>(row) * p.ldc + (n0 >> 1);
          const int out_n = p.N >> 1;
#pragma unroll 1
          for (int c = 0; c < 4; ++c) {
            // 64-column group c of the tile: 32 gate columns, then the 32 matching up columns
            uint32_t g[32], u[32];
            tmem_ld_32x32(taddr + c * 64, g);
            tmem_ld_32x32(taddr + c * 64 + 32, u);
            tmem_ld_wait();
            float v[32];
#pragma unroll
            for (int i = 0; i < 32; ++i)
              v[i] = silu_f(__uint_as_float(g[i])) * __uint_as_float(u[i]);
            if (row_ok && (n0 >> 1) + c * 32 < out_n) {
#pragma unroll
              for (int i = 0; i < 4; ++i) store8_bf16(crow + c * 32 + i * 8, v + i * 8);
            }
          }
        } else {
#pragma unroll 1
          for (int c = 0; c < BN / 32; ++c) {
            uint32_t r[32];
            tmem_ld_32x32(taddr + c * 32, r);
            tmem_ld_wait();
            const int col = n0 + c * 32;
            if (!row_ok || col >= p.N) continue;
            float v[32];
#pragma unroll
            for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
            if constexpr (EPI == kBias) {
#pragma unroll
              for (int i = 0; i < 32; ++i) v[i] += __bfloat162float(p.bias[col + i]);
            }
            __nv_bfloat16* crow = p.C + static_cast<long long>(row) * p.ldc + col;
#pragma unroll
            for (int i = 0; i < 4; ++i) store8_bf16(crow + i * 8, v + i * 8);
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(tempty_bar);
      tphase ^= 1u;
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_base, kTmemCols);
}

template <int EPI>
int launch_wide2(const CUtensorMap& tmA, const CUtensorMap& tmB, const WideArgs& a,
                 cudaStream_t stream) {
  using L = Smem<256, 2, 3>;
  auto kern = gemm_wide2_kernel<EPI>;
  static bool configured[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !configured[dev]) {
    cudaError_t e =
        cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kTotal);
    if (e != cudaSuccess) return static_cast<int>(e);
    configured[dev] = true;
  }
  const int tiles = a.tiles_m * a.tiles_n;
  const int grid = tiles < sm_count() ? tiles : sm_count();
  kern<<<grid, kThreads, L::kTotal, stream>>>(tmA, tmB, a);
  return static_cast<int>(cudaGetLastError());
}

struct Plan {
  int bn, splits;
};

// Picks the column-tile width and the K split.  The estimate is the larger of the total bytes
// that move from L2 into shared memory (over an aggregate L2 -> SM rate) and the bytes of one
// unit (over what one SM can ingest); units never exceed the SM count when K is split.
// C = sum over K slices of the partial sums a split launch left in ws (+ bias): the slices of
// a column tile lie one after the other, [tile][slice][R x bn]; fixed summation order.
__global__ void __launch_bounds__(256)
    skinny_reduce_kernel(const float* ws, __nv_bfloat16* C, long long ldc,
                         const __nv_bfloat16* bias, int M, int N, int bn, int R, int splits) {
  const long long idx = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  const int n4 = N >> 2;
  if (idx >= static_cast<long long>(M) * n4) return;
  const int row = static_cast<int>(idx / n4), col = static_cast<int>(idx % n4) * 4;
  const int tile = col / bn, c_in = col - tile * bn;
  const float* src = ws + (static_cast<long long>(tile) * splits) * (static_cast<long long>(R) * bn) +
                     static_cast<long long>(row) * bn + c_in;
  float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
  for (int sl = 0; sl < splits; ++sl) {
    const float4 a = __ldcg(reinterpret_cast<const float4*>(src + static_cast<long long>(sl) * R * bn));
    acc.x += a.x; acc.y += a.y; acc.z += a.z; acc.w += a.w;
  }
  if (bias != nullptr) {
    acc.x += __bfloat162float(bias[col]);
    acc.y += __bfloat162float(bias[col + 1]);
    acc.z += __bfloat162float(bias[col + 2]);
    acc.w += __bfloat162float(bias[col + 3]);
  }
  uint2 o;
  o.x = pack_bf16x2(acc.x, acc.y);
  o.y = pack_bf16x2(acc.z, acc.w);
  *reinterpret_cast<uint2*>(C + static_cast<long long>(row) * ldc + col) = o;
}

// Plan for the two-kernel K split.  A CTA takes in at most about 64 bytes per clock from L2
// (120 GB/s), and with M <= 256 that port, not HBM, bounds the kernel: every CTA reads the
// whole activation slice of its K range again.  Wide column tiles with a deep K split move the
// fewest bytes through it; the price is the fp32 partial sums (written and read once, L2
// resident) and a second launch.
inline Plan make_plan2(int M, int N, int K, int epi, int sms) {
  const int mt = M > BM ? 2 : 1;
  const int num_kb = (K + BK - 1) / BK;
  Plan best{256, 1};
  double best_t = 1e30;
  const int cands[3] = {256, 128, 64};
  for (int ci = 0; ci < 3; ++ci) {
    const int bn = cands[ci];
    if (epi == kSiluMul && bn != 256) continue;
    if (N % bn != 0) continue;
    const int tiles = N / bn;
    for (int sl = 1; sl <= 16; ++sl) {
      if (sl > 1 && (epi == kSiluMul || tiles * sl > sms || num_kb / sl < 8)) break;
      const double units = static_cast<double>(tiles) * sl;
      const double waves = units <= sms ? 1.0 : units / sms;
      const double unit_bytes = (mt * 128.0 + bn) * (static_cast<double>(K) / sl) * 2.0;
      double t = unit_bytes * waves / 1.2e11 + 3.0e-6;
      // measured: parking the accumulators as fp32 and the second launch cost about 6 us
      if (sl > 1) t += 2.0 * sl * M * static_cast<double>(N) * 4.0 / 4.0e12 + 6.0e-6;
      if (t < best_t) {
        best_t = t;
        best = Plan{bn, sl};
      }
    }
  }
  return best;
}

inline Plan make_plan(int M, int N, int K, int epi, int sms) {
  const int mt = M > BM ? 2 : 1;
  const int num_kb = (K + BK - 1) / BK;
  Plan best{256, 1};
  double best_t = 1e30;
  const int cands[3] = {256, 128, 64};
  for (int ci = 0; ci < 3; ++ci) {
    const int bn = cands[ci];
    if (epi == kSiluMul && bn != 256) continue;
    if (bn > 64 && N < bn) continue;
    const int tiles = (N + bn - 1) / bn;
    for (int s = 1; s <= 16; ++s) {
      if (s > 1 && (tiles * s > sms || num_kb / s < 4)) break;
      const double kc = static_cast<double>(K) / s;
      const double unit_bytes = (mt * 128.0 + bn) * kc * 2.0 + (s > 1 ? 2.0 * mt * 128.0 * bn * 4.0 : 0.0);
      const double units = static_cast<double>(tiles) * s;
      const double waves = units <= sms ? 1.0 : (units / sms);
      const double t = fmax(unit_bytes * units / 9.0e12, unit_bytes * waves / 9.0e10) + (s > 1 ? 2.0e-6 : 0.0);
      if (t < best_t) {
        best_t = t;
        best = Plan{bn, s};
      }
    }
  }
  return best;
}

}  // namespace skinny
}  // namespace b200

// Workspace the caller must provide for b200_gemm_skinny: *ws_bytes of fp32 partial sums and
// *ctr_words zero-initialised 32-bit counters (both upper bounds for any M <= 256, N).
B200_API int b200_gemm_skinny_workspace(int N, long long* ws_bytes, int* ctr_words) {
  using namespace b200;
  *ws_bytes = static_cast<long long>(sm_count()) * 256 * 256 * 4;
  *ctr_words = 2 * ((N + 63) / 64) + 2;
  return 0;
}

// C[M,N] (bf16) = A[M,K] * B[N,K]^T for M <= 256 with epilogue epi: 0 none, 1 + bias[N],
// 2 SiLU(gate)*up (B rows interleaved gate/up in blocks of 32; C is [M, N/2]).
// Row pitches in elements; K, lda, ldb, N, ldc multiples of 8; 16-byte aligned pointers.
// ws / ctr: see b200_gemm_skinny_workspace (ctr must be zero before the first call; the kernel
// leaves it zero).  Launches on one stream may share the workspace; concurrent streams need
// their own.  allow_split = 0 restricts the kernel to plans without a K split.  Returns 0, a
// CUDA error code, a negative argument error, or -20 when the shape is outside what this
// kernel covers (the caller uses b200_gemm_bf16).
B200_API int b200_gemm_skinny(const void* A, long long lda, const void* B, long long ldb, void* C,
                              long long ldc, int M, int N, int K, const void* bias, int epi,
                              void* ws, void* ctr, int allow_split, void* stream) {
  using namespace b200;
  using namespace b200::skinny;
  if (M <= 0 || N <= 0) return 0;
  if (M > 2 * BM) return -20;
  if (K <= 0 || (K % 8) != 0 || (lda % 8) != 0 || (ldb % 8) != 0 || (N % 8) != 0 ||
      (ldc % 8) != 0)
    return -2;
  if ((reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(B) |
       reinterpret_cast<uintptr_t>(C)) & 15)
    return -3;
  if (epi == kSiluMul && (N % 256) != 0) return -4;
  if (epi == kBias && bias == nullptr) return -5;
  if (epi < 0 || epi > 2) return -20;
  const int sms = sm_count();
  Plan pl = allow_split == 2 ? make_plan2(M, N, K, epi, sms) : make_plan(M, N, K, epi, sms);
  if (allow_split == 2 && pl.splits == 1) {
    // without a split this kernel only takes what it took before: one wave of 256-wide tiles
    const int tiles = (N + 255) / 256;
    if (pl.bn != 256 || N < 256 || tiles > sms || tiles * 2 < sms) return -20;
  }
  if (pl.splits > 1 && !allow_split) {
    // Measured on B200: at M = 256 the fp32 partial sums of a K split cost as much L2 traffic
    // as the split saves, and the persistent-tile kernel is faster.  Without the split this
    // kernel is used when one wave of 256-wide column tiles covers the problem.
    pl = Plan{256, 1};
    const int tiles = (N + 255) / 256;
    if (N < 256 || tiles > sms || tiles * 2 < sms) return -20;
  }
  if (pl.splits > 1 && (ws == nullptr || (ctr == nullptr && allow_split != 2))) return -5;
  const int mt = M > BM ? 2 : 1;

  CUtensorMap tmA, tmB;
  int r = encode_tmap_2d(&tmA, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, A, static_cast<uint64_t>(M),
                         static_cast<uint64_t>(K), static_cast<uint64_t>(lda) * 2, BM, BK,
                         CU_TENSOR_MAP_SWIZZLE_128B);
  if (r != 0) return r < 0 ? -6 : r;
  r = encode_tmap_2d(&tmB, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, B, static_cast<uint64_t>(N),
                     static_cast<uint64_t>(K), static_cast<uint64_t>(ldb) * 2, pl.bn, BK,
                     CU_TENSOR_MAP_SWIZZLE_128B);
  if (r != 0) return r < 0 ? -6 : r;

  Args a;
  a.C = static_cast<__nv_bfloat16*>(C);
  a.ldc = ldc;
  a.bias = static_cast<const __nv_bfloat16*>(bias);
  a.M = M; a.N = N; a.K = K;
  a.tiles_n = (N + pl.bn - 1) / pl.bn;
  a.splits = pl.splits;
  a.num_kb = (K + BK - 1) / BK;
  a.ws = static_cast<float*>(ws);
  a.ctr = allow_split == 2 ? nullptr : static_cast<unsigned int*>(ctr);
  a.status = status_ptr();
  const int units = a.tiles_n * a.splits;
  cudaStream_t s = static_cast<cudaStream_t>(stream);

  int rc = -20;
#define B200_SK(BN_, MT_, ST_)                                                      \
  switch (epi) {                                                                    \
    case kNone: rc = launch<BN_, MT_, ST_, kNone>(tmA, tmB, a, units, s); break;    \
    case kBias: rc = launch<BN_, MT_, ST_, kBias>(tmA, tmB, a, units, s); break;    \
    default: break;                                                                 \
  }
  if (epi == kSiluMul) {
    if (mt == 2) return launch<256, 2, 3, kSiluMul>(tmA, tmB, a, units, s);
    return launch<256, 1, 4, kSiluMul>(tmA, tmB, a, units, s);
  }
  if (pl.bn == 256) {
    if (mt == 2) { B200_SK(256, 2, 3) } else { B200_SK(256, 1, 4) }
  } else if (pl.bn == 128) {
    if (mt == 2) { B200_SK(128, 2, 4) } else { B200_SK(128, 1, 6) }
  } else {
    if (mt == 2) { B200_SK(64, 2, 5) } else { B200_SK(64, 1, 8) }
  }
#undef B200_SK
  if (rc != 0 || a.splits == 1 || a.ctr != nullptr) return rc;
  // two-kernel K split: add the partial sums
  const long long work = static_cast<long long>(M) * (N / 4);
  skinny_reduce_kernel<<<static_cast<unsigned>((work + 255) / 256), 256, 0, s>>>(
      a.ws, a.C, a.ldc, epi == kBias ? a.bias : nullptr, M, N, pl.bn, mt * BM, a.splits);
  return static_cast<int>(cudaGetLastError());
}

// The plan b200_gemm_skinny would use (for tests and benchmarks): bn and splits.
B200_API int b200_gemm_skinny_plan(int M, int N, int K, int epi, int* bn, int* splits) {
  using namespace b200;
  const skinny::Plan pl = skinny::make_plan(M, N, K, epi, sm_count());
  *bn = pl.bn;
  *splits = pl.splits;
  return 0;
}

// C[M,N] = A[M,K] * B[N,K]^T with persistent 256 x 256 tiles (large M).  N must be a multiple
// of 256 (epi 2: gate / up interleaved in blocks of 32, C is [M, N/2]); other constraints as
// b200_gemm_bf16.  Returns -20 when the shape does not qualify.
B200_API int b200_gemm_wide2(const void* A, long long lda, const void* B, long long ldb, void* C,
                             long long ldc, int M, int N, int K, const void* bias, int epi,
                             void* stream) {
  using namespace b200;
  using namespace b200::skinny;
  if (M <= 0 || N <= 0) return 0;
  if ((N % 256) != 0 || M < 512 || epi < 0 || epi > 2) return -20;
  if (K <= 0 || (K % 8) != 0 || (lda % 8) != 0 || (ldb % 8) != 0 || (ldc % 8) != 0) return -2;
  if ((reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(B) |
       reinterpret_cast<uintptr_t>(C)) & 15)
    return -3;
  if (epi == kBias && bias == nullptr) return -5;
  CUtensorMap tmA, tmB;
  int r = encode_tmap_2d(&tmA, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, A, static_cast<uint64_t>(M),
                         static_cast<uint64_t>(K), static_cast<uint64_t>(lda) * 2, BM, BK,
                         CU_TENSOR_MAP_SWIZZLE_128B);
  if (r != 0) return r < 0 ? -6 : r;
  r = encode_tmap_2d(&tmB, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, B, static_cast<uint64_t>(N),
                     static_cast<uint64_t>(K), static_cast<uint64_t>(ldb) * 2, 256, BK,
                     CU_TENSOR_MAP_SWIZZLE_128B);
  if (r != 0) return r < 0 ? -6 : r;
  WideArgs a;
  a.C = static_cast<__nv_bfloat16*>(C);
  a.ldc = ldc;
  a.bias = static_cast<const __nv_bfloat16*>(bias);
  a.M = M; a.N = N; a.K = K;
  a.tiles_m = (M + 255) / 256;
  a.tiles_n = N / 256;
  a.num_kb = (K + BK - 1) / BK;
  a.status = status_ptr();
  {
    int gm = 1;
    while (gm * gm < sm_count()) ++gm;      // ~ sqrt(number of tiles in flight)
    const char* env = getenv("VLLM_B200_GEMM_GROUP_M");
    if (env != nullptr && atoi(env) > 0) gm = atoi(env);
    a.group_m = gm < a.tiles_m ? gm : a.tiles_m;
  }
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (epi == kSiluMul) return launch_wide2<kSiluMul>(tmA, tmB, a, s);
  if (epi == kBias) return launch_wide2<kBias>(tmA, tmB, a, s);
  return launch_wide2<kNone>(tmA, tmB, a, s);
}
