// Weight-only quantised GEMM for decode-sized activations:
//   C[M, N] = A[M, K] * dequant(W)[N, K]^T,   M <= 256, W stored as 4-bit or 8-bit integers
// with per-group scales:  w = q * scale - zs  (zs = zero point * scale), groups of g along K.
//
// Replaces the reference's `gptq_gemm` / `awq_gemm` ops for AWQ and GPTQ checkpoints
// (vllm_gcu/kernels/quantization/awq.py:70-118, gptq.py:95-164) on the decode path.  With
// M <= 256 the layer is bound by the weight bytes it reads; de-quantising into a bf16 scratch
// first and running the bf16 GEMM moves 4.5 bytes per weight (read 0.5, write 2, read 2), this
// kernel moves 0.5: four producer warps read the packed integers straight from global memory,
// de-quantise in registers (4 bit: bf16 pair arithmetic with a single rounding; 8 bit: fp32
// multiply-add rounded to bf16, as the stand-alone de-quantisation kernel does) and write the
// bf16 tile into shared memory in the K-major 128-byte
// swizzled layout that tcgen05.mma reads; the activation tiles arrive by TMA; accumulators
// live in tensor memory.  Packed weights are prefetched eight K blocks ahead into registers.
//
// Warp roles: warp 0 TMA (activations), warp 1 MMA issuer + TMEM owner, warps 2..5 weight
// producers during the main loop and epilogue afterwards.  Bounded waits, status word.
#include "common.cuh"

namespace b200 {
namespace wna16 {

constexpr unsigned int kKernelId = 23;
constexpr int BM = 128;
constexpr int BN = 64;
constexpr int BK = 64;
constexpr int UMMA_K = 16;
constexpr int kThreads = 192;
constexpr int kStages = 4;
constexpr int kPrefetch = 8;

struct Args {
  const uint8_t* qw;              // [N, K / 2] (low nibble = even k) or [N, K] for 8 bit
  const __nv_bfloat16* scales;    // [N, K / g]
  const __nv_bfloat16* zs;        // [N, K / g]
  const __nv_bfloat16* bias;      // optional [N]
  __nv_bfloat16* C;
  long long ldc;
  int M, N, K, g;
  unsigned int* status;
};

template <int MT>
struct Smem {
  static constexpr int kABytes = BM * BK * 2;
  static constexpr int kBBytes = BN * BK * 2;
  static constexpr int kStageBytes = MT * kABytes + kBBytes;
  static constexpr int kBarOffset = kStages * kStageBytes;
  static constexpr int kTotal = kBarOffset + 256 + 1024;
};

template <int BITS, int MT>
__global__ void __launch_bounds__(kThreads)
    gemm_wna16_kernel(const __grid_constant__ CUtensorMap tmA, const Args p) {
  using L = Smem<MT>;
  constexpr uint32_t kTmemCols = MT * BN <= 64 ? 64 : 128;
  constexpr uint32_t kIdesc = make_idesc(BM, BN, 1, 1);
  constexpr int kBytesPer = BITS == 4 ? 16 : 32;      // packed bytes of 32 weights

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + L::kBarOffset);
  uint64_t* empty_bar = full_bar + kStages;
  uint64_t* tfull_bar = empty_bar + kStages;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tfull_bar + 1);
  volatile uint32_t* abort_flag = tmem_slot + 1;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&full_bar[s], 1 + 4);       // TMA thread (with the byte count) + 4 producer warps
      mbar_init(&empty_bar[s], 1);
    }
    mbar_init(tfull_bar, 1);
    *abort_flag = 0u;
    mbar_fence_init();
    tma_prefetch_desc(&tmA);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  const int n0 = blockIdx.x * BN;
  const int num_kb = p.K / BK;

  if (warp == 0) {
    if (elect_one()) {
      int stage = 0;
      uint32_t phase = 0;
      for (int kb = 0; kb < num_kb; ++kb) {
        if (!mbar_wait(&empty_bar[stage], phase ^ 1u, p.status, kKernelId, 0x100u + stage,
                       abort_flag))
          break;
        uint8_t* sa = smem + stage * L::kStageBytes;
        mbar_expect_tx(&full_bar[stage], MT * L::kABytes);
#pragma unroll
        for (int mt = 0; mt < MT; ++mt)
          tma_load_2d(sa + mt * L::kABytes, &tmA, &full_bar[stage], kb * BK, mt * BM);
        if (++stage == kStages) {
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
      for (int kb = 0; kb < num_kb; ++kb) {
        if (!mbar_wait(&full_bar[stage], phase, p.status, kKernelId, 0x300u + stage, abort_flag)) {
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t a_addr = smem_u32(smem + stage * L::kStageBytes);
        const uint64_t bdesc = make_desc_k_sw128(a_addr + MT * L::kABytes);
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) {
          const uint64_t adesc = make_desc_k_sw128(a_addr + mt * L::kABytes);
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k)
            umma_f16(tmem_base + static_cast<uint32_t>(mt * BN),
                     adesc + static_cast<uint64_t>(k * 2), bdesc + static_cast<uint64_t>(k * 2),
                     kIdesc, (kb > 0 || k > 0) ? 1u : 0u);
        }
        umma_commit(&empty_bar[stage]);
        if (++stage == kStages) {
          stage = 0;
          phase ^= 1u;
        }
      }
      if (ok) umma_commit(tfull_bar);
    }
  } else {
    // ---------------- weight producers (warps 2..5), then epilogue ----------------
    const int t = threadIdx.x - 64;          // 0..127
    const int row = t >> 1;                  // weight row inside the tile
    const int kh = t & 1;                    // which 32 of the 64 k of a block
    const int n = n0 + row;
    const bool n_ok = n < p.N;
    const int groups = p.K / p.g;
    const uint8_t* qrow =
        p.qw + static_cast<long long>(n_ok ? n : 0) * (BITS == 4 ? p.K / 2 : p.K) + kh * kBytesPer;
    const __nv_bfloat16* srow = p.scales + static_cast<long long>(n_ok ? n : 0) * groups;
    const __nv_bfloat16* zrow = p.zs + static_cast<long long>(n_ok ? n : 0) * groups;
    // register ring of packed weights, kPrefetch K blocks ahead
    // (scale and zero point travel with them: a dependent load per K block would put a
    // memory latency on every step)
    uint4 ring[kPrefetch][BITS == 4 ? 1 : 2];
    __nv_bfloat16 ring_s[kPrefetch], ring_z[kPrefetch];
#pragma unroll
    for (int i = 0; i < kPrefetch; ++i) {
      if (i < num_kb) {
        const uint4* src = reinterpret_cast<const uint4*>(qrow + static_cast<long long>(i) * (2 * kBytesPer));
        ring[i][0] = src[0];
        if constexpr (BITS == 8) ring[i][1] = src[1];
        const int grp = (i * BK + kh * 32) / p.g;
        ring_s[i] = srow[grp];
        ring_z[i] = zrow[grp];
      }
    }
    int stage = 0;
    uint32_t phase = 0;
    bool ok = true;
    for (int kb0 = 0; kb0 < num_kb && ok; kb0 += kPrefetch) {
#pragma unroll
      for (int i = 0; i < kPrefetch; ++i) {
        const int kb = kb0 + i;
        if (kb >= num_kb || !ok) break;
        uint4 cur[BITS == 4 ? 1 : 2];
        cur[0] = ring[i][0];
        if constexpr (BITS == 8) cur[1] = ring[i][1];
        const float s = __bfloat162float(ring_s[i]);
        const float z = __bfloat162float(ring_z[i]);
        if (kb + kPrefetch < num_kb) {
          const uint4* src = reinterpret_cast<const uint4*>(
              qrow + static_cast<long long>(kb + kPrefetch) * (2 * kBytesPer));
          ring[i][0] = src[0];
          if constexpr (BITS == 8) ring[i][1] = src[1];
          const int grp = ((kb + kPrefetch) * BK + kh * 32) / p.g;
          ring_s[i] = srow[grp];
          ring_z[i] = zrow[grp];
        }
        uint32_t w[16];
        if constexpr (BITS == 4) {
          // Two nibbles at a time as a bf16 pair: 0x4300 | q is the bf16 number 128 + q, the
          // subtraction of 128 is exact, and one bf16 fused multiply-add gives q * s - zs with
          // a single rounding (the stand-alone kernel rounds an fp32 result: equal except
          // for double-rounding ties).  Nibble i of a word is element i, so the pairs come
          // out as (0, 4), (1, 5), (2, 6), (3, 7) and two byte permutes per four restore
          // the order.
          const uint32_t pw[4] = {cur[0].x, cur[0].y, cur[0].z, cur[0].w};
          const __nv_bfloat162 s2 = __float2bfloat162_rn(s);
          const __nv_bfloat162 nz2 = __float2bfloat162_rn(-z);
          const __nv_bfloat162 k128 = __float2bfloat162_rn(128.0f);
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            uint32_t tt[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const uint32_t bits = ((pw[j] >> (4 * e)) & 0x000F000Fu) | 0x43004300u;
              __nv_bfloat162 q2 = *reinterpret_cast<const __nv_bfloat162*>(&bits);
              q2 = __hfma2(__hsub2(q2, k128), s2, nz2);
              tt[e] = *reinterpret_cast<const uint32_t*>(&q2);
            }
            w[j * 4 + 0] = __byte_perm(tt[0], tt[1], 0x5410);
            w[j * 4 + 1] = __byte_perm(tt[2], tt[3], 0x5410);
            w[j * 4 + 2] = __byte_perm(tt[0], tt[1], 0x7632);
            w[j * 4 + 3] = __byte_perm(tt[2], tt[3], 0x7632);
          }
        } else {
          const uint8_t* pb = reinterpret_cast<const uint8_t*>(&cur[0]);
#pragma unroll
          for (int e = 0; e < 16; ++e) {
            const float f0 = static_cast<float>(pb[2 * e]) * s - z;
            const float f1 = static_cast<float>(pb[2 * e + 1]) * s - z;
            w[e] = pack_bf16x2(f0, f1);
          }
        }
        if (!n_ok) {
#pragma unroll
          for (int e = 0; e < 16; ++e) w[e] = 0u;
        }
        if (!mbar_wait(&empty_bar[stage], phase ^ 1u, p.status, kKernelId, 0x200u + stage,
                       abort_flag)) {
          ok = false;
          break;
        }
        uint8_t* sb = smem + stage * L::kStageBytes + MT * L::kABytes + row * 128;
#pragma unroll
        for (int c = 0; c < 4; ++c)
          *reinterpret_cast<uint4*>(sb + (((kh * 4 + c) ^ (row & 7)) << 4)) =
              make_uint4(w[c * 4], w[c * 4 + 1], w[c * 4 + 2], w[c * 4 + 3]);
        fence_async_smem();
        __syncwarp();
        if (lane == 0) mbar_arrive(&full_bar[stage]);
        if (++stage == kStages) {
          stage = 0;
          phase ^= 1u;
        }
      }
    }
    // ---------------- epilogue ----------------
    const int q = warp & 3;
    mbar_wait(tfull_bar, 0u, p.status, kKernelId, 0x400u, abort_flag);   // sets abort on timeout
    asm volatile("bar.sync 1, 128;" ::: "memory");
    const bool have = *abort_flag == 0u;
    tc_fence_after();
    if (have) {
#pragma unroll 1
      for (int mt = 0; mt < MT; ++mt) {
        const int r = mt * BM + q * 32 + lane;
        const uint32_t taddr =
            tmem_base + (static_cast<uint32_t>(q * 32) << 16) + static_cast<uint32_t>(mt * BN);
#pragma unroll 1
        for (int c = 0; c < BN / 32; ++c) {
          uint32_t acc[32];
          tmem_ld_32x32(taddr + c * 32, acc);
          tmem_ld_wait();
          const int col = n0 + c * 32;
          if (r >= p.M || col >= p.N) continue;
          __nv_bfloat16* crow = p.C + static_cast<long long>(r) * p.ldc + col;
          if (col + 32 <= p.N && (p.ldc & 7) == 0) {
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              float v[8];
#pragma unroll
              for (int e = 0; e < 8; ++e) {
                v[e] = __uint_as_float(acc[i * 8 + e]);
                if (p.bias != nullptr) v[e] += __bfloat162float(p.bias[col + i * 8 + e]);
              }
              uint4 u;
              u.x = pack_bf16x2(v[0], v[1]);
              u.y = pack_bf16x2(v[2], v[3]);
              u.z = pack_bf16x2(v[4], v[5]);
              u.w = pack_bf16x2(v[6], v[7]);
              *reinterpret_cast<uint4*>(crow + i * 8) = u;
            }
          } else {
#pragma unroll
            for (int e = 0; e < 32; ++e) {
              if (col + e < p.N) {
                float v = __uint_as_float(acc[e]);
                if (p.bias != nullptr) v += __bfloat162float(p.bias[col + e]);
                crow[e] = __float2bfloat16(v);
              }
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

template <int BITS, int MT>
static int launch(const CUtensorMap& tmA, const Args& a, cudaStream_t s) {
  using L = Smem<MT>;
  auto kern = gemm_wna16_kernel<BITS, MT>;
  static bool configured[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !configured[dev]) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kTotal);
    if (e != cudaSuccess) return static_cast<int>(e);
    configured[dev] = true;
  }
  kern<<<(a.N + BN - 1) / BN, kThreads, L::kTotal, s>>>(tmA, a);
  return static_cast<int>(cudaGetLastError());
}

}  // namespace wna16
}  // namespace b200

// A [M, K] bf16 (row pitch lda), qw / scales / zs as described above, C [M, N] bf16.
// Returns -20 when the shape is outside what the kernel covers (M > 256, K % 64, group size
// not a multiple of 32, misaligned pointers): callers de-quantise and use the bf16 GEMM.
B200_API int b200_gemm_wna16(const void* A, long long lda, const void* qw, const void* scales,
                             const void* zs, const void* bias, void* C, long long ldc, int M,
                             int N, int K, int g, int bits, void* stream) {
  using namespace b200;
  using namespace b200::wna16;
  if (M <= 0 || N <= 0) return 0;
  if (M > 2 * BM || K <= 0 || (K % BK) != 0 || g <= 0 || (g % 32) != 0 || (K % g) != 0 ||
      (bits != 4 && bits != 8) || (lda % 8) != 0 ||
      ((reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(qw)) & 15))
    return -20;
  CUtensorMap tmA;
  int r = encode_tmap_2d(&tmA, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, A, static_cast<uint64_t>(M),
                         static_cast<uint64_t>(K), static_cast<uint64_t>(lda) * 2, BM, BK,
                         CU_TENSOR_MAP_SWIZZLE_128B);
  if (r != 0) return r < 0 ? -6 : r;
  Args a;
  a.qw = static_cast<const uint8_t*>(qw);
  a.scales = static_cast<const __nv_bfloat16*>(scales);
  a.zs = static_cast<const __nv_bfloat16*>(zs);
  a.bias = static_cast<const __nv_bfloat16*>(bias);
  a.C = static_cast<__nv_bfloat16*>(C);
  a.ldc = ldc; a.M = M; a.N = N; a.K = K; a.g = g;
  a.status = status_ptr();
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const bool two = M > BM;
  if (bits == 4) return two ? launch<4, 2>(tmA, a, s) : launch<4, 1>(tmA, a, s);
  return two ? launch<8, 2>(tmA, a, s) : launch<8, 1>(tmA, a, s);
}
