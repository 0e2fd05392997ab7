// Weight-only quantised GEMM for decode-sized activations:
//   C[M, N] = A[M, K] * dequant(W)[N, K]^T,   M <= 256, W stored as 4-bit or 8-bit integers
// with per-group scales:  w = q * scale - zs  (zs = zero point * scale), groups of g along K.
//
// Replaces the reference's `gptq_gemm` / `awq_gemm` ops for AWQ and GPTQ checkpoints
// (vllm_gcu/kernels/quantization/awq.py:70-118, gptq.py:95-164) on the decode path.  With
// M <= 256 the layer is bound by the weight bytes it reads; de-quantising into a bf16 scratch
// first and running the bf16 GEMM moves 4.5 bytes per weight (read 0.5, write 2, read 2), this
// kernel moves 0.5: producer warps read the packed integers straight from global memory,
// de-quantise in registers (4 bit: bf16 pair arithmetic with a single rounding; 8 bit: fp32
// multiply-add rounded to bf16, as the stand-alone de-quantisation kernel does) and write the
// bf16 tile into shared memory in the K-major 128-byte swizzled layout that tcgen05.mma
// reads; the activation tiles arrive by TMA; accumulators live in tensor memory.  Packed
// weights and their scales are prefetched sixteen K blocks ahead into registers; each producer
// warp builds whole K blocks on its own (every eighth one).
//
// Warp roles: warp 0 TMA (activations), warp 1 MMA issuer + TMEM owner, warps 2..9 weight
// producers (two per scheduler, so one covers the other's stalls); warps 2..5 run the epilogue.
// When N / 64 column tiles would leave most SMs idle, K is split over blockIdx.y: fp32 partial
// sums go to a workspace and a second kernel adds them (fixed order) and applies the bias.
// Bounded waits, status word.
#include "common.cuh"

namespace b200 {
namespace wna16 {

constexpr unsigned int kKernelId = 23;
constexpr int BM = 128;
constexpr int BN = 64;
constexpr int BK = 64;
constexpr int UMMA_K = 16;
constexpr int kMaxProdWarps = 8;
constexpr int kThreads = 64 + 32 * kMaxProdWarps;

struct Args {
  const uint8_t* qw;              // [N, K / 2] (low nibble = even k) or [N, K] for 8 bit
  const __nv_bfloat16* scales;    // [N, K / g]
  const __nv_bfloat16* zs;        // [N, K / g]
  const __nv_bfloat16* bias;      // optional [N]
  __nv_bfloat16* C;
  long long ldc;
  int M, N, K, g;
  int splits;                     // K split over blockIdx.y; > 1: fp32 partial sums to ws
  float* ws;                      // [splits, M, N]
  unsigned int* status;
  // grouped mode (mixture-of-experts): A holds expert-sorted rows in tiles of 128, tile t
  // (= blockIdx.z) multiplies the weights of expert expert_ids[t]; qw / scales / zs carry a
  // leading expert dimension.  Null expert_ids: one dense weight matrix.
  const int* expert_ids;          // [M / 128]
  const int* num_post_pad;        // device scalar: rows in use (a multiple of 128)
  const float* row_scale;         // optional [M]: factor applied to every output row
  long long w_stride;             // bytes between experts in qw
  long long s_stride;             // elements between experts in scales / zs
};

// The loop empty -> TMA load -> full -> MMA -> empty takes about 2 us; with S stages a K block
// completes every 2 / S us, so the stages fill the shared memory (4 stages: 0.5 us per block).
// Every stage belongs to exactly one producer warp (stages == producer warps, warp w builds
// the K blocks w, w + stages, ...): a warp meets its stage's barrier phases in order, so the
// parity waits cannot be overtaken.  (With stages shared between warps a fast warp could pass
// a wait meant for a later phase and arrive twice on one barrier phase.)  Two activation
// tiles per stage leave room for four stages, so only four warps produce then.  With one
// activation tile there are two shapes: eight stages / eight producer warps (one CTA per SM),
// and four / four (96 KB, 192 threads: two CTAs per SM) for grids of more than 1.5 CTAs per
// SM, where a second resident CTA is worth more than a deeper pipeline.
template <int MT, int STAGES>
struct Smem {
  static constexpr int kStages = STAGES;
  static constexpr int kProdWarps = kStages;
  static constexpr int kABytes = BM * BK * 2;
  static constexpr int kBBytes = BN * BK * 2;
  static constexpr int kStageBytes = MT * kABytes + kBBytes;
  static constexpr int kBarOffset = kStages * kStageBytes;
  static constexpr int kTotal = kBarOffset + 256 + 1024;
};

template <int BITS, int MT, int STAGES>
__global__ void __launch_bounds__(kThreads)
    gemm_wna16_kernel(const __grid_constant__ CUtensorMap tmA, const Args p) {
  using L = Smem<MT, STAGES>;
  constexpr int kStages = L::kStages;
  constexpr uint32_t kTmemCols = MT * BN <= 64 ? 64 : 128;
  constexpr uint32_t kIdesc = make_idesc(BM, BN, 1, 1);
  constexpr int kBytesPer = BITS == 4 ? 16 : 32;      // packed bytes of 32 weights

  // grouped mode: this CTA's row tile and expert (the whole CTA leaves before any barrier,
  // tensor-memory allocation or copy when the tile is past the rows in use)
  const int tile_m = p.expert_ids != nullptr ? static_cast<int>(blockIdx.z) : 0;
  long long w_off = 0, s_off = 0;
  if (p.expert_ids != nullptr) {
    if (tile_m * BM >= *p.num_post_pad) return;
    const int expert = p.expert_ids[tile_m];
    if (expert < 0) return;
    w_off = static_cast<long long>(expert) * p.w_stride;
    s_off = static_cast<long long>(expert) * p.s_stride;
  }

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
      mbar_init(&full_bar[s], 1 + 1);       // TMA thread (with the byte count) + one producer warp
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
  // this CTA's K blocks: [kb_lo, kb_lo + num_kb)
  const int total_kb = p.K / BK;
  const int kb_lo = static_cast<int>(static_cast<long long>(blockIdx.y) * total_kb / p.splits);
  const int num_kb =
      static_cast<int>(static_cast<long long>(blockIdx.y + 1) * total_kb / p.splits) - kb_lo;

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
          tma_load_2d(sa + mt * L::kABytes, &tmA, &full_bar[stage], (kb_lo + kb) * BK,
                      (tile_m + mt) * BM);
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
    // ---------------- weight producers (warps 2..9), then epilogue (warps 2..5) -----------
    // Producer warp w owns the K blocks kb = w (mod 8) and builds the whole 64 x 64 tile of
    // each: the proxy fence that has to follow the shared-memory stores costs a few hundred
    // nanoseconds per thread, and with one warp per block the fences of consecutive
    // blocks overlap instead of adding up.  Lane l holds rows l and l + 32.
    constexpr int kProdWarps = L::kProdWarps;
    const int pw = warp - 2;
    const int groups = p.K / p.g;
    const int g_shift = 31 - __clz(p.g);             // the group size is a power of two
    constexpr int kVec = BITS == 4 ? 2 : 4;          // uint4 per row and K block
    constexpr int kDepth = 2;                        // own blocks prefetched ahead (= 16 K blocks)
    const uint8_t* qrow[2];
    const __nv_bfloat16* srow[2];
    const __nv_bfloat16* zrow[2];
    bool n_ok[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      const int n = n0 + lane + 32 * r;
      n_ok[r] = n < p.N;
      const long long nn = n_ok[r] ? n : 0;
      qrow[r] = p.qw + w_off + nn * (BITS == 4 ? p.K / 2 : p.K);
      srow[r] = p.scales + s_off + nn * groups;
      zrow[r] = p.zs + s_off + nn * groups;
    }
    uint4 ring[kDepth][2][kVec];
    __nv_bfloat16 ring_s[kDepth][2][2], ring_z[kDepth][2][2];
    auto fetch = [&](int slot, int kb) {
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        const uint4* src =
            reinterpret_cast<const uint4*>(qrow[r]) + static_cast<long long>(kb_lo + kb) * kVec;
#pragma unroll
        for (int v = 0; v < kVec; ++v)
          ring[slot][r][v] = src[v];
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          const int grp = ((kb_lo + kb) * BK + h * 32) >> g_shift;
          ring_s[slot][r][h] = srow[r][grp];
          ring_z[slot][r][h] = zrow[r][grp];
        }
      }
    };
#pragma unroll
    for (int d = 0; d < kDepth; ++d)
      if (pw < kProdWarps && pw + kProdWarps * d < num_kb) fetch(d, pw + kProdWarps * d);
    bool ok = true;
    for (int kb0 = pw; pw < kProdWarps && kb0 < num_kb && ok; kb0 += kProdWarps * kDepth) {
#pragma unroll
      for (int d = 0; d < kDepth; ++d) {
        const int kb = kb0 + kProdWarps * d;
        if (kb >= num_kb || !ok) break;
        const int stage = kb % kStages;
        const uint32_t phase = static_cast<uint32_t>(kb / kStages) & 1u;
        uint32_t w[2][2][16];                      // [row][half of the block][16 bf16 pairs]
#pragma unroll
        for (int r = 0; r < 2; ++r) {
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            const float sc = __bfloat162float(ring_s[d][r][h]);
            const float zz = __bfloat162float(ring_z[d][r][h]);
            if constexpr (BITS == 4) {
              // Two nibbles at a time as a bf16 pair: 0x4300 | q is the bf16 number 128 + q,
              // the subtraction of 128 is exact, and one bf16 fused multiply-add gives
              // q * s - zs with a single rounding (the stand-alone kernel rounds an fp32
              // result: equal except for double-rounding ties).  Nibble i of a word is
              // element i, so the pairs come out as (0, 4), (1, 5), (2, 6), (3, 7) and two
              // byte permutes per four restore the order.
              const uint4 c = ring[d][r][h];
              const uint32_t pq[4] = {c.x, c.y, c.z, c.w};
              const __nv_bfloat162 s2 = __float2bfloat162_rn(sc);
              const __nv_bfloat162 nz2 = __float2bfloat162_rn(-zz);
              const __nv_bfloat162 k128 = __float2bfloat162_rn(128.0f);
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                uint32_t tt[4];
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                  const uint32_t bits = ((pq[j] >> (4 * e)) & 0x000F000Fu) | 0x43004300u;
                  __nv_bfloat162 q2 = *reinterpret_cast<const __nv_bfloat162*>(&bits);
                  q2 = __hfma2(__hsub2(q2, k128), s2, nz2);
                  tt[e] = *reinterpret_cast<const uint32_t*>(&q2);
                }
                w[r][h][j * 4 + 0] = __byte_perm(tt[0], tt[1], 0x5410);
                w[r][h][j * 4 + 1] = __byte_perm(tt[2], tt[3], 0x5410);
                w[r][h][j * 4 + 2] = __byte_perm(tt[0], tt[1], 0x7632);
                w[r][h][j * 4 + 3] = __byte_perm(tt[2], tt[3], 0x7632);
              }
            } else {
#pragma unroll
              for (int v = 0; v < 2; ++v) {
                const uint4 c = ring[d][r][h * 2 + v];
                const uint32_t pq[4] = {c.x, c.y, c.z, c.w};
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                  const float f0 = static_cast<float>(pq[j] & 0xFFu) * sc - zz;
                  const float f1 = static_cast<float>((pq[j] >> 8) & 0xFFu) * sc - zz;
                  const float f2 = static_cast<float>((pq[j] >> 16) & 0xFFu) * sc - zz;
                  const float f3 = static_cast<float>(pq[j] >> 24) * sc - zz;
                  w[r][h][v * 8 + j * 2] = pack_bf16x2(f0, f1);
                  w[r][h][v * 8 + j * 2 + 1] = pack_bf16x2(f2, f3);
                }
              }
            }
            if (!n_ok[r]) {
#pragma unroll
              for (int e = 0; e < 16; ++e) w[r][h][e] = 0u;
            }
          }
        }
        if (kb + kProdWarps * kDepth < num_kb) fetch(d, kb + kProdWarps * kDepth);
        if (!mbar_wait(&empty_bar[stage], phase ^ 1u, p.status, kKernelId, 0x200u + stage,
                       abort_flag)) {
          ok = false;
          break;
        }
        uint8_t* sb = smem + stage * L::kStageBytes + MT * L::kABytes;
#pragma unroll
        for (int r = 0; r < 2; ++r) {
          const int row = lane + 32 * r;
#pragma unroll
          for (int c = 0; c < 8; ++c)
            *reinterpret_cast<uint4*>(sb + row * 128 + ((c ^ (row & 7)) << 4)) =
                make_uint4(w[r][c >> 2][(c & 3) * 4], w[r][c >> 2][(c & 3) * 4 + 1],
                           w[r][c >> 2][(c & 3) * 4 + 2], w[r][c >> 2][(c & 3) * 4 + 3]);
        }
        fence_async_smem();
        __syncwarp();
        if (lane == 0) mbar_arrive(&full_bar[stage]);
      }
    }
    // ---------------- epilogue ----------------
    const int q = warp & 3;
    bool have = false;
    if (warp < 6) {
      mbar_wait(tfull_bar, 0u, p.status, kKernelId, 0x400u, abort_flag);   // sets abort on timeout
      asm volatile("bar.sync 1, 128;" ::: "memory");
      have = *abort_flag == 0u;
      tc_fence_after();
    }
    if (have) {
#pragma unroll 1
      for (int mt = 0; mt < MT; ++mt) {
        const int r = (tile_m + mt) * BM + q * 32 + lane;
        const uint32_t taddr =
            tmem_base + (static_cast<uint32_t>(q * 32) << 16) + static_cast<uint32_t>(mt * BN);
#pragma unroll 1
        for (int c = 0; c < BN / 32; ++c) {
          uint32_t acc[32];
          tmem_ld_32x32(taddr + c * 32, acc);
          tmem_ld_wait();
          const int col = n0 + c * 32;
          if (r >= p.M || col >= p.N) continue;
          if (p.splits > 1) {
            float* wrow = p.ws + (static_cast<long long>(blockIdx.y) * p.M + r) * p.N + col;
#pragma unroll
            for (int e = 0; e < 32; ++e)
              if (col + e < p.N) wrow[e] = __uint_as_float(acc[e]);
            continue;
          }
          __nv_bfloat16* crow = p.C + static_cast<long long>(r) * p.ldc + col;
          const float rs = p.row_scale != nullptr ? p.row_scale[r] : 1.0f;
          if (col + 32 <= p.N && (p.ldc & 7) == 0) {
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              float v[8];
#pragma unroll
              for (int e = 0; e < 8; ++e) {
                v[e] = __uint_as_float(acc[i * 8 + e]) * rs;
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
                float v = __uint_as_float(acc[e]) * rs;
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

// C[r, c] = sum over splits of ws[s, r, c] (+ bias[c]), summed in split order.
__global__ void __launch_bounds__(256)
    wna16_reduce_kernel(const float* ws, const __nv_bfloat16* bias, __nv_bfloat16* C, long long ldc,
                        int M, int N, int splits) {
  const long long idx = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (idx >= static_cast<long long>(M) * N) return;
  const int r = static_cast<int>(idx / N), c = static_cast<int>(idx % N);
  float acc = 0.0f;
  for (int s = 0; s < splits; ++s) acc += ws[(static_cast<long long>(s) * M + r) * N + c];
  if (bias != nullptr) acc += __bfloat162float(bias[c]);
  C[static_cast<long long>(r) * ldc + c] = __float2bfloat16(acc);
}

// K splits that bring the grid to about one CTA per SM (every split keeps >= 16 K blocks).
static int plan_splits(int N, int K) {
  const int tiles = (N + BN - 1) / BN;
  const int sms = sm_count() > 0 ? sm_count() : 148;
  int splits = sms / tiles;
  const int cap = (K / BK) / 16;
  if (splits > cap) splits = cap;
  if (splits > 8) splits = 8;
  return splits < 1 ? 1 : splits;
}

template <int BITS, int MT, int STAGES>
static int launch(const CUtensorMap& tmA, const Args& a, cudaStream_t s) {
  using L = Smem<MT, STAGES>;
  auto kern = gemm_wna16_kernel<BITS, MT, STAGES>;
  static bool configured[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !configured[dev]) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kTotal);
    if (e != cudaSuccess) return static_cast<int>(e);
    configured[dev] = true;
  }
  dim3 grid((a.N + BN - 1) / BN, a.splits, a.expert_ids != nullptr ? (a.M + BM - 1) / BM : 1);
  kern<<<grid, 64 + 32 * STAGES, L::kTotal, s>>>(tmA, a);
  int e = static_cast<int>(cudaGetLastError());
  if (e != 0 || a.splits == 1) return e;
  const long long total = static_cast<long long>(a.M) * a.N;
  wna16_reduce_kernel<<<static_cast<unsigned>((total + 255) / 256), 256, 0, s>>>(
      a.ws, a.bias, a.C, a.ldc, a.M, a.N, a.splits);
  return static_cast<int>(cudaGetLastError());
}

}  // namespace wna16
}  // namespace b200

// A [M, K] bf16 (row pitch lda), qw / scales / zs as described above, C [M, N] bf16.
// Returns -20 when the shape is outside what the kernel covers (M > 256, K % 64, group size
// not a power of two >= 32, misaligned pointers): callers de-quantise and use the bf16 GEMM.
// Floats of workspace b200_gemm_wna16 wants for this shape (0: no K split).
B200_API long long b200_gemm_wna16_workspace(int M, int N, int K) {
  if (M <= 0 || N <= 0 || K <= 0 || (K % b200::wna16::BK) != 0) return 0;
  const int splits = b200::wna16::plan_splits(N, K);
  return splits > 1 ? static_cast<long long>(splits) * M * N : 0;
}

// `ws` may be null: then K is not split.
B200_API int b200_gemm_wna16(const void* A, long long lda, const void* qw, const void* scales,
                             const void* zs, const void* bias, void* C, long long ldc, int M,
                             int N, int K, int g, int bits, float* ws, void* stream) {
  using namespace b200;
  using namespace b200::wna16;
  if (M <= 0 || N <= 0) return 0;
  if (M > 2 * BM || K <= 0 || (K % BK) != 0 || g < 32 || (g & (g - 1)) != 0 || (K % g) != 0 ||
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
  a.splits = ws != nullptr ? plan_splits(N, K) : 1;
  a.ws = ws;
  a.expert_ids = nullptr; a.num_post_pad = nullptr; a.row_scale = nullptr;
  a.w_stride = 0; a.s_stride = 0;

  a.status = status_ptr();
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const bool two = M > BM;
  const int ctas = ((N + BN - 1) / BN) * a.splits;
  const int sms = sm_count() > 0 ? sm_count() : 148;
  const bool wide = !two && 2 * ctas > 3 * sms;
  if (bits == 4)
    return two ? launch<4, 2, 4>(tmA, a, s)
               : (wide ? launch<4, 1, 4>(tmA, a, s) : launch<4, 1, 8>(tmA, a, s));
  return two ? launch<8, 2, 4>(tmA, a, s)
             : (wide ? launch<8, 1, 4>(tmA, a, s) : launch<8, 1, 8>(tmA, a, s));
}

// Grouped form for mixture-of-experts layers whose experts stay packed (the reference's
// moe_wna16 path, vllm_gcu/kernels/quantization/moe_wna16.py:487-572): A [M_cap, K] bf16 holds
// the expert-sorted rows in tiles of 128 (`b200_moe_align` / `b200_moe_permute`), tile t uses
// expert expert_ids[t]; qw [E, N, K/2] (or [E, N, K] for 8 bit), scales / zs [E, N, K/g];
// num_post_pad is the device scalar with the rows in use; row_scale (optional, [M_cap])
// multiplies every output row (the routing weight, second GEMM).  C [M_cap, N] bf16; rows of
// tiles past num_post_pad are not written.  Returns -20 for shapes the kernel does not cover.
B200_API int b200_gemm_wna16_grouped(const void* A, long long lda, const void* qw,
                                     const void* scales, const void* zs, void* C, long long ldc,
                                     int M_cap, int N, int K, int E, int g, int bits,
                                     const int* expert_ids, const int* num_post_pad,
                                     const float* row_scale, void* stream) {
  using namespace b200;
  using namespace b200::wna16;
  if (M_cap <= 0 || N <= 0 || E <= 0) return 0;
  if ((M_cap % BM) != 0 || K <= 0 || (K % BK) != 0 || g < 32 || (g & (g - 1)) != 0 ||
      (K % g) != 0 || (bits != 4 && bits != 8) || (lda % 8) != 0 ||
      expert_ids == nullptr || num_post_pad == nullptr ||
      ((reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(qw)) & 15))
    return -20;
  const long long w_stride = static_cast<long long>(N) * (bits == 4 ? K / 2 : K);
  if ((w_stride & 15) != 0) return -20;
  CUtensorMap tmA;
  int r = encode_tmap_2d(&tmA, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, A,
                         static_cast<uint64_t>(M_cap), static_cast<uint64_t>(K),
                         static_cast<uint64_t>(lda) * 2, BM, BK, CU_TENSOR_MAP_SWIZZLE_128B);
  if (r != 0) return r < 0 ? -6 : r;
  Args a;
  a.qw = static_cast<const uint8_t*>(qw);
  a.scales = static_cast<const __nv_bfloat16*>(scales);
  a.zs = static_cast<const __nv_bfloat16*>(zs);
  a.bias = nullptr;
  a.C = static_cast<__nv_bfloat16*>(C);
  a.ldc = ldc; a.M = M_cap; a.N = N; a.K = K; a.g = g;
  a.splits = 1;
  a.ws = nullptr;
  a.status = status_ptr();
  a.expert_ids = expert_ids; a.num_post_pad = num_post_pad; a.row_scale = row_scale;
  a.w_stride = w_stride;
  a.s_stride = static_cast<long long>(N) * (K / g);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const long long ctas = static_cast<long long>((N + BN - 1) / BN) * (M_cap / BM);
  const int sms = sm_count() > 0 ? sm_count() : 148;
  const bool wide = 2 * ctas > 3 * sms;
  if (bits == 4) return wide ? launch<4, 1, 4>(tmA, a, s) : launch<4, 1, 8>(tmA, a, s);
  return wide ? launch<8, 1, 4>(tmA, a, s) : launch<8, 1, 8>(tmA, a, s);
}
