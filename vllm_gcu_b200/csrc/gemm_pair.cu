// bf16 GEMM for large M on CTA pairs:  C[M,N] = A[M,K] * B[N,K]^T  with one 256 x 256 output
// tile per pair of CTAs (a cluster of two), `tcgen05.mma.cta_group::2`.
//
// Why pairs.  A single CTA that computes a 256 x 256 tile with M = 128 instructions reads the
// weight tile twice from shared memory (once per 128-row half) while TMA writes 64 KB per K
// block into the same shared memory, and its accumulators fill all of tensor memory, so the
// epilogue of a tile cannot run under the MMAs of the next.  With the tile spread over two SMs
// each CTA stages its 128 rows of A and 128 of the 256 weight rows (32 KB per K block); the
// pair instruction (M = 256 over both SMs) reads every operand byte from shared memory once
// and hands each SM the other SM's weight half; each CTA keeps a 128 x 256 accumulator half
// (256 TMEM columns), so two accumulator sets fit and the epilogue overlaps the next tile.
// Measured on the Llama-3-8B prefill shapes (8192 rows): 1.49 - 1.63 PFLOP/s, the level of
// the vendor library, against 1.07 - 1.39 for the single-CTA 256 x 256 kernel.
//
// A second shape (VLLM_B200_PAIR_MT=2) gives each CTA two 128-row blocks of A per stage: a
// 512 x 256 pair tile, 48 KB per K block for twice the work, one accumulator set.  It moves a
// quarter fewer bytes from L2 per flop but loses the epilogue overlap and measured slower.
//
// Tile rows [m0, m0 + 256 MT): instruction t computes rows m0 + 256 t + [0, 256) (CTA 0 the
// first 128, CTA 1 the second) into 256 TMEM columns of each CTA; CTA r stages weight rows
// n0 + [128 r, 128 r + 128).
//
// Roles (192 threads per CTA): warp 0 = TMA producer (this CTA's blocks; plain loads, no
// multicast; every load completes on the leader's barrier), warp 1 = MMA issuer in the leader
// CTA (cluster rank 0) and TMEM owner; warps 2..5 = epilogue of the CTA's own rows.
// Barriers: `full` (leader: TMA bytes of both CTAs), `empty` and `tfull` (both CTAs, arrived
// by `tcgen05.commit` with cluster multicast), `tempty` (leader: both epilogues have drained
// an accumulator set).  Arrivals and waits use CTA-scope semantics: what they order is read
// and written by the tensor-core proxy behind tcgen05 fences; cluster-scope release / acquire
// on every stage measured about 2 us per hop and halved the throughput.  Every wait is
// bounded; a wait that runs out sets the status word and the CTA falls through to the closing
// cluster barrier, so neither CTA of a pair leaves while the other may still touch its shared
// memory.
//
// Replaces the vendor matmul behind the prefill path of the unquantised linear layers
// (vllm_gcu/kernels/linear.py), like the single-CTA kernels of gemm_bf16.cu / gemm_skinny.cu.
#include "common.cuh"

#include <cstdlib>

namespace b200 {
namespace pair {

constexpr unsigned int kKernelId = 12;
constexpr int BMH = 128;          // rows per CTA (half of the pair's 256)
constexpr int BN = 256;           // columns of the pair tile
constexpr int BNH = 128;          // weight rows staged per CTA
constexpr int BK = 64;
constexpr int UMMA_K = 16;
constexpr int kThreads = 192;

enum Epi : int { kNone = 0, kBias = 1, kSiluMul = 2 };

struct Args {
  __nv_bfloat16* C;
  long long ldc;
  const __nv_bfloat16* bias;
  int M, N, K;
  int tiles_m, tiles_n, num_kb;
  int group_m;
  unsigned int* status;
  // K split (decode-sized inputs with few tiles): one (tile, K slice) per pair
  int splits;
  float* ws;            // [tiles * splits][256][256] fp32 partial sums
  unsigned int* ctr;    // [tiles][2] arrive / depart counters, zero between launches
};

// MT = 128-row blocks of A per CTA and stage: 2 gives the 512 x 256 pair tile (one accumulator
// set, all of tensor memory), 1 a 256 x 256 pair tile with two accumulator sets, so that the
// epilogue of a tile runs under the MMAs of the next.
template <int MT>
struct Smem {
  static constexpr int kStages = MT == 1 ? 6 : 4;
  static constexpr int kAcc = MT == 1 ? 2 : 1;
  static constexpr int kABytes = BMH * BK * 2;
  static constexpr int kBBytes = BNH * BK * 2;
  static constexpr int kStageBytes = MT * kABytes + kBBytes;
  static constexpr int kBarOffset = kStages * kStageBytes;
  static constexpr int kTotal = kBarOffset + 512 + 1024;
  static_assert(kTotal <= 232448, "exceeds the shared memory of one CTA");
};

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// Address of `local` (a shared-memory location of this CTA) in CTA `rank` of the cluster.
__device__ __forceinline__ uint32_t map_to_cta(const void* local, uint32_t rank) {
  uint32_t out;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(out) : "r"(smem_u32(local)), "r"(rank));
  return out;
}
__device__ __forceinline__ void mbar_arrive_remote(uint32_t cluster_addr) {
  // (default semantics, release at CTA scope: what the waiting side hands on goes through the
  // tensor-core proxy behind tcgen05 fences, not through generic loads; a cluster-scope release
  // here and cluster-scope acquires in the waits cost several microseconds per stage)
  asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx_remote(uint32_t cluster_addr, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cluster.b64 _, [%0], %1;" ::"r"(
                   cluster_addr),
               "r"(bytes)
               : "memory");
}
// Tile load into this CTA's shared memory whose completion is counted on a barrier of either
// CTA of the pair (`bar_cluster_addr` from map_to_cta).  No multicast.
__device__ __forceinline__ void tma_load_2d_pair(void* smem_dst, const CUtensorMap* m,
                                                 uint32_t bar_cluster_addr, int32_t x,
                                                 int32_t y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4}], [%2];"
      :
      : "r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(m)), "r"(bar_cluster_addr),
        "r"(x), "r"(y)
      : "memory");
}
// D[tmem] (+)= A[smem] * B[smem]^T over both CTAs of the pair: 256 x N x 16 per instruction,
// rows 0-127 from / into the leader, rows 128-255 the other CTA; each CTA holds N / 2 rows of B.
__device__ __forceinline__ void umma_f16_pair(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b,
                                              uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t"
      "}\n"
      :
      : "r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Arrives on the barrier at this shared-memory offset in both CTAs of the pair once every MMA
// issued so far by this thread has completed.
__device__ __forceinline__ void umma_commit_pair(uint64_t* bar) {
  const uint16_t mask = 3;
  asm volatile(
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 "
      "[%0], %1;" ::"r"(smem_u32(bar)),
      "h"(mask)
      : "memory");
}

__device__ __forceinline__ void store8_bf16(__nv_bfloat16* dst, const float* v) {
  uint4 u;
  u.x = pack_bf16x2(v[0], v[1]);
  u.y = pack_bf16x2(v[2], v[3]);
  u.z = pack_bf16x2(v[4], v[5]);
  u.w = pack_bf16x2(v[6], v[7]);
  *reinterpret_cast<uint4*>(dst) = u;
}

// Tile order: groups of `group_m` row panels, the row index running fastest inside a group
// (the tiles in flight at one time then cover a near-square set of A and B panels).
__device__ __forceinline__ void tile_coords(const Args& p, int tile, int& tm, int& tn) {
  const int group = p.group_m * p.tiles_n;
  const int g = tile / group;
  const int first = g * p.group_m;
  const int gm = min(p.tiles_m - first, p.group_m);
  const int r = tile - g * group;
  tm = first + r % gm;
  tn = r / gm;
}

template <int EPI, int MT>
__global__ void __launch_bounds__(kThreads, 1)
    gemm_pair_kernel(const __grid_constant__ CUtensorMap tmA,
                     const __grid_constant__ CUtensorMap tmB, const Args p) {
  using L = Smem<MT>;
  constexpr int STAGES = L::kStages;
  constexpr int NACC = L::kAcc;
  constexpr uint32_t kTmemCols = 512;       // MT 2: rows +0 / +256; MT 1: two accumulator sets
  constexpr uint32_t kIdesc = make_idesc(2 * BMH, BN, 1, 1);

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + L::kBarOffset);   // used in the leader
  uint64_t* empty_bar = full_bar + STAGES;
  uint64_t* tfull_bar = empty_bar + STAGES;                 // [NACC]
  uint64_t* tempty_bar = tfull_bar + NACC;                  // [NACC], used in the leader
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty_bar + NACC);
  volatile uint32_t* abort_flag = tmem_slot + 1;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();                  // 0 = leader
  const int pair_id = blockIdx.x >> 1;
  const int num_pairs = gridDim.x >> 1;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 2);                           // one producer per CTA
      mbar_init(&empty_bar[s], 1);
    }
    for (int b = 0; b < NACC; ++b) {
      mbar_init(&tfull_bar[b], 1);
      mbar_init(&tempty_bar[b], 8);                         // four epilogue warps of each CTA
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
  cluster_sync_all();            // the other CTA's barriers exist before anything arrives there
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const int num_tiles = p.tiles_m * p.tiles_n;

  if (warp == 0) {
    // ---------------- TMA producer: this CTA's 128 rows of A and 128 weight rows -----------
    if (elect_one()) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = pair_id; ok && tile < num_tiles; tile += num_pairs) {
        int tm, tn;
        tile_coords(p, tile, tm, tn);
        const int m0 = tm * (2 * MT * BMH) + static_cast<int>(rank) * BMH;
        const int n0 = tn * BN + static_cast<int>(rank) * BNH;
        for (int kb = 0; kb < p.num_kb; ++kb) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1u, p.status, kKernelId, 0x100u + stage,
                         abort_flag)) {
            ok = false;
            break;
          }
          uint8_t* sa = smem + stage * L::kStageBytes;
          uint8_t* sb = sa + MT * L::kABytes;
          const uint32_t full_leader = map_to_cta(&full_bar[stage], 0);
          mbar_expect_tx_remote(full_leader, L::kStageBytes);
          tma_load_2d_pair(sb, &tmB, full_leader, kb * BK, n0);
#pragma unroll
          for (int mt = 0; mt < MT; ++mt)
            tma_load_2d_pair(sa + mt * L::kABytes, &tmA, full_leader, kb * BK,
                             m0 + mt * 2 * BMH);
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
    }
  } else if (warp == 1) {
    if (rank == 0 && elect_one()) {
      // ---------------- MMA issuer (leader) ----------------
      int stage = 0;
      uint32_t phase = 0;
      uint32_t tphase[2] = {0u, 0u};
      bool ok = true;
      int it = 0;
      for (int tile = pair_id; ok && tile < num_tiles; tile += num_pairs, ++it) {
        const int b = NACC == 2 ? (it & 1) : 0;
        if (!mbar_wait(&tempty_bar[b], tphase[b] ^ 1u, p.status, kKernelId, 0x300u + b,
                       abort_flag))
          break;
        tphase[b] ^= 1u;
        tc_fence_after();
        const uint32_t acc_base = tmem_base + static_cast<uint32_t>(b * BN);
        for (int kb = 0; kb < p.num_kb; ++kb) {
          if (!mbar_wait(&full_bar[stage], phase, p.status, kKernelId, 0x310u + stage,
                         abort_flag)) {
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
              umma_f16_pair(acc_base + static_cast<uint32_t>(mt * BN),
                            adesc + static_cast<uint64_t>(k * 2),
                            bdesc + static_cast<uint64_t>(k * 2), kIdesc,
                            (kb | k) != 0 ? 1u : 0u);
          }
          umma_commit_pair(&empty_bar[stage]);              // frees the stage in both CTAs
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (!ok) break;
        umma_commit_pair(&tfull_bar[b]);                    // accumulators ready in both CTAs
      }
    }
  } else {
    // ---------------- epilogue: this CTA's 2 x 128 rows of the tile ----------------
    const int q = warp & 3;
    uint32_t tphase[2] = {0u, 0u};
    const uint32_t tempty_leader[2] = {map_to_cta(&tempty_bar[0], 0),
                                       map_to_cta(&tempty_bar[NACC - 1], 0)};
    int it = 0;
    for (int tile = pair_id; tile < num_tiles; tile += num_pairs, ++it) {
      const int b = NACC == 2 ? (it & 1) : 0;
      int tm, tn;
      tile_coords(p, tile, tm, tn);
      const int m0 = tm * (2 * MT * BMH) + static_cast<int>(rank) * BMH, n0 = tn * BN;
      if (!mbar_wait(&tfull_bar[b], tphase[b], p.status, kKernelId, 0x400u + b, abort_flag))
        break;
      tphase[b] ^= 1u;
      tc_fence_after();
#pragma unroll 1
      for (int mt = 0; mt < MT; ++mt) {
        const int row = m0 + mt * 2 * BMH + q * 32 + lane;
        const bool row_ok = row < p.M;
        const uint32_t taddr =
            tmem_base + (static_cast<uint32_t>(q * 32) << 16) +
            static_cast<uint32_t>((mt + b) * BN);
        if constexpr (EPI == kSiluMul) {
          __nv_bfloat16* crow = p.C + static_cast<long long>(row) * p.ldc + (n0 >> 1);
#pragma unroll 1
          for (int c = 0; c < BN / 64; ++c) {
            // 64-column group c: 32 gate columns, then the 32 matching up columns
            uint32_t g[32], u[32];
            tmem_ld_32x32(taddr + c * 64, g);
            tmem_ld_32x32(taddr + c * 64 + 32, u);
            tmem_ld_wait();
            float v[32];
#pragma unroll
            for (int i = 0; i < 32; ++i)
              v[i] = silu_f(__uint_as_float(g[i])) * __uint_as_float(u[i]);
            if (row_ok) {
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
            if (!row_ok) continue;
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
      if (lane == 0) mbar_arrive_remote(tempty_leader[b]);  // (the leader's own address too)
    }
  }
  // Nobody leaves before both CTAs are past their last MMA, commit and remote arrive.
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();
  if (warp == 1) tmem_dealloc(tmem_base, kTmemCols);
}

// ---------------------------------------------------------------------------
// K split for inputs of a few hundred rows whose 256 x 256 tiles are too few to occupy the
// SM pairs (qkv, o_proj, down_proj at decode batch sizes): every pair takes one (tile, K slice),
// parks its fp32 partial sums in an L2-resident workspace, the 2 x splits CTAs of a tile meet
// at a counter (bounded wait; all units are resident at once: units <= pairs the device can
// co-schedule) and each reduces a row slice of the tile in a fixed order and applies the
// epilogue.  Same pair pipeline as above with one accumulator set.
// ---------------------------------------------------------------------------
template <int EPI>
__global__ void __launch_bounds__(kThreads, 1)
    gemm_pair_split_kernel(const __grid_constant__ CUtensorMap tmA,
                           const __grid_constant__ CUtensorMap tmB, const Args p) {
  using L = Smem<1>;
  constexpr int STAGES = L::kStages;
  constexpr uint32_t kTmemCols = 256;
  constexpr uint32_t kIdesc = make_idesc(2 * BMH, BN, 1, 1);
  constexpr int R = 2 * BMH;                                // rows of a tile

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + L::kBarOffset);   // used in the leader
  uint64_t* empty_bar = full_bar + STAGES;
  uint64_t* tfull_bar = empty_bar + STAGES;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tfull_bar + 1);
  volatile uint32_t* abort_flag = tmem_slot + 1;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();                  // 0 = leader
  const int unit = blockIdx.x >> 1;
  const int tile = unit / p.splits, split = unit - tile * p.splits;
  const int tm = tile / p.tiles_n, tn = tile - tm * p.tiles_n;
  const int kb_lo = static_cast<int>(static_cast<long long>(split) * p.num_kb / p.splits);
  const int nkb = static_cast<int>(static_cast<long long>(split + 1) * p.num_kb / p.splits) - kb_lo;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(&full_bar[s], 2);
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
  cluster_sync_all();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    if (elect_one()) {
      int stage = 0;
      uint32_t phase = 0;
      const int m0 = tm * R + static_cast<int>(rank) * BMH;
      const int n0 = tn * BN + static_cast<int>(rank) * BNH;
      for (int kb = 0; kb < nkb; ++kb) {
        if (!mbar_wait(&empty_bar[stage], phase ^ 1u, p.status, kKernelId, 0x500u + stage,
                       abort_flag))
          break;
        uint8_t* sa = smem + stage * L::kStageBytes;
        uint8_t* sb = sa + L::kABytes;
        const uint32_t full_leader = map_to_cta(&full_bar[stage], 0);
        mbar_expect_tx_remote(full_leader, L::kStageBytes);
        tma_load_2d_pair(sb, &tmB, full_leader, (kb_lo + kb) * BK, n0);
        tma_load_2d_pair(sa, &tmA, full_leader, (kb_lo + kb) * BK, m0);
        if (++stage == STAGES) {
          stage = 0;
          phase ^= 1u;
        }
      }
    }
  } else if (warp == 1) {
    if (rank == 0 && elect_one()) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int kb = 0; kb < nkb; ++kb) {
        if (!mbar_wait(&full_bar[stage], phase, p.status, kKernelId, 0x510u + stage,
                       abort_flag)) {
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t a_addr = smem_u32(smem + stage * L::kStageBytes);
        const uint64_t adesc = make_desc_k_sw128(a_addr);
        const uint64_t bdesc = make_desc_k_sw128(a_addr + L::kABytes);
#pragma unroll
        for (int k = 0; k < BK / UMMA_K; ++k)
          umma_f16_pair(tmem_base, adesc + static_cast<uint64_t>(k * 2),
                        bdesc + static_cast<uint64_t>(k * 2), kIdesc, (kb | k) != 0 ? 1u : 0u);
        umma_commit_pair(&empty_bar[stage]);
        if (++stage == STAGES) {
          stage = 0;
          phase ^= 1u;
        }
      }
      if (ok) umma_commit_pair(tfull_bar);
    }
  } else {
    // ---------------- epilogue warps: park, meet, reduce a row slice ----------------
    const int q = warp & 3;
    const int te = static_cast<int>(threadIdx.x) - 64;      // 0 .. 127
    const int m0 = tm * R, n0 = tn * BN;
    const int rows_used = min(p.M - m0, R);
    bool have = mbar_wait(tfull_bar, 0u, p.status, kKernelId, 0x520u, abort_flag);
    asm volatile("bar.sync 1, 128;" ::: "memory");
    have = have && *abort_flag == 0u;
    tc_fence_after();
    if (have) {
      float* mine = p.ws + static_cast<long long>(unit) * (R * BN);
      const int row = static_cast<int>(rank) * BMH + q * 32 + lane;       // row of the tile
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(q * 32) << 16);
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t r[32];
        tmem_ld_32x32(taddr + c * 32, r);
        tmem_ld_wait();
        if (row >= rows_used) continue;
        float4* dst = reinterpret_cast<float4*>(mine + static_cast<long long>(row) * BN + c * 32);
#pragma unroll
        for (int i = 0; i < 8; ++i)
          dst[i] = make_float4(__uint_as_float(r[i * 4]), __uint_as_float(r[i * 4 + 1]),
                               __uint_as_float(r[i * 4 + 2]), __uint_as_float(r[i * 4 + 3]));
      }
      __threadfence();
      asm volatile("bar.sync 1, 128;" ::: "memory");
      unsigned int* arrive = p.ctr + 2 * tile;
      unsigned int* depart = arrive + 1;
      const unsigned int members = 2u * static_cast<unsigned int>(p.splits);
      if (te == 0) {
        atomicAdd(arrive, 1u);
        bool ok = false;
        for (uint32_t it = 0; it < (1u << 22); ++it) {
          unsigned int v;
          asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(arrive) : "memory");
          if (v >= members) { ok = true; break; }
          if (it > 32) __nanosleep(64);
        }
        if (!ok) {
          report_status(p.status, kStatusFlagTimeout, kKernelId, 0x530u);
          *abort_flag = 1u;
        }
      }
      asm volatile("bar.sync 1, 128;" ::: "memory");
      if (*abort_flag == 0u) {
        const int idx = split * 2 + static_cast<int>(rank);
        const int r0 = static_cast<int>(static_cast<long long>(idx) * rows_used / members);
        const int r1 = static_cast<int>(static_cast<long long>(idx + 1) * rows_used / members);
        const float* base = p.ws + static_cast<long long>(tile) * p.splits * (R * BN);
        if constexpr (EPI == kSiluMul) {
          constexpr int kV = 128 / 4;                       // float4 groups of the gate half
          for (int e = te; e < (r1 - r0) * kV; e += 128) {
            const int rw = r0 + e / kV, c4 = (e % kV) * 4;
            // output column c4 of the tile: gate at (c4 / 32) * 64 + c4 % 32, up 32 further
            const int gcol = (c4 >> 5) * 64 + (c4 & 31);
            float4 g = make_float4(0.f, 0.f, 0.f, 0.f), u = g;
            for (int s = 0; s < p.splits; ++s) {
              const float* src = base + static_cast<long long>(s) * (R * BN) +
                                 static_cast<long long>(rw) * BN + gcol;
              const float4 a = __ldcg(reinterpret_cast<const float4*>(src));
              const float4 b = __ldcg(reinterpret_cast<const float4*>(src + 32));
              g.x += a.x; g.y += a.y; g.z += a.z; g.w += a.w;
              u.x += b.x; u.y += b.y; u.z += b.z; u.w += b.w;
            }
            uint2 o;
            o.x = pack_bf16x2(silu_f(g.x) * u.x, silu_f(g.y) * u.y);
            o.y = pack_bf16x2(silu_f(g.z) * u.z, silu_f(g.w) * u.w);
            *reinterpret_cast<uint2*>(p.C + static_cast<long long>(m0 + rw) * p.ldc + (n0 >> 1) +
                                      c4) = o;
          }
        } else {
          constexpr int kV = BN / 4;
          for (int e = te; e < (r1 - r0) * kV; e += 128) {
            const int rw = r0 + e / kV, c4 = (e % kV) * 4;
            float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
            for (int s = 0; s < p.splits; ++s) {
              const float4 a = __ldcg(reinterpret_cast<const float4*>(
                  base + static_cast<long long>(s) * (R * BN) + static_cast<long long>(rw) * BN +
                  c4));
              acc.x += a.x; acc.y += a.y; acc.z += a.z; acc.w += a.w;
            }
            const int col = n0 + c4;
            if constexpr (EPI == kBias) {
              acc.x += __bfloat162float(p.bias[col]);
              acc.y += __bfloat162float(p.bias[col + 1]);
              acc.z += __bfloat162float(p.bias[col + 2]);
              acc.w += __bfloat162float(p.bias[col + 3]);
            }
            uint2 o;
            o.x = pack_bf16x2(acc.x, acc.y);
            o.y = pack_bf16x2(acc.z, acc.w);
            *reinterpret_cast<uint2*>(p.C + static_cast<long long>(m0 + rw) * p.ldc + col) = o;
          }
        }
      }
      // the last CTA of the tile to leave clears both counters for the next launch
      asm volatile("bar.sync 1, 128;" ::: "memory");
      if (te == 0 && *abort_flag == 0u) {
        if (atomicAdd(depart, 1u) == members - 1u) {
          *arrive = 0u;
          *depart = 0u;
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();
  if (warp == 1) tmem_dealloc(tmem_base, kTmemCols);
}

template <int MT>
static int max_pairs(const void* kern, int smem_bytes) {
  // pairs of SMs that can hold a cluster at the same time (per device, cached)
  static int cached[64] = {0};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) return 0;
  if (cached[dev] == 0) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(2 * 74);
    cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = static_cast<size_t>(smem_bytes);
    cudaLaunchAttribute attr;
    attr.id = cudaLaunchAttributeClusterDimension;
    attr.val.clusterDim.x = 2;
    attr.val.clusterDim.y = 1;
    attr.val.clusterDim.z = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, kern, &cfg) != cudaSuccess || n <= 0) {
      cudaGetLastError();
      n = -1;
    }
    cached[dev] = n;
  }
  return cached[dev];
}

template <int EPI, int MT>
int launch(const CUtensorMap& tmA, const CUtensorMap& tmB, const Args& a, cudaStream_t stream) {
  using Smem = b200::pair::Smem<MT>;
  auto kern = gemm_pair_kernel<EPI, MT>;
  static bool configured[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !configured[dev]) {
    cudaError_t e =
        cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Smem::kTotal);
    if (e != cudaSuccess) return static_cast<int>(e);
    configured[dev] = true;
  }
  const int cap = max_pairs<MT>(reinterpret_cast<const void*>(kern), Smem::kTotal);
  if (cap <= 0) return -20;                                 // no room for a cluster of two
  const int tiles = a.tiles_m * a.tiles_n;
  const int pairs = tiles < cap ? tiles : cap;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(2 * pairs);
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = Smem::kTotal;
  cfg.stream = stream;
  cudaLaunchAttribute attr;
  attr.id = cudaLaunchAttributeClusterDimension;
  attr.val.clusterDim.x = 2;
  attr.val.clusterDim.y = 1;
  attr.val.clusterDim.z = 1;
  cfg.attrs = &attr;
  cfg.numAttrs = 1;
  return static_cast<int>(cudaLaunchKernelEx(&cfg, kern, tmA, tmB, a));
}

template <int EPI>
int launch_split(const CUtensorMap& tmA, const CUtensorMap& tmB, const Args& a, int units,
                 cudaStream_t stream) {
  using Smem = b200::pair::Smem<1>;
  auto kern = gemm_pair_split_kernel<EPI>;
  static bool configured[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !configured[dev]) {
    cudaError_t e =
        cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Smem::kTotal);
    if (e != cudaSuccess) return static_cast<int>(e);
    configured[dev] = true;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(2 * units);
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = Smem::kTotal;
  cfg.stream = stream;
  cudaLaunchAttribute attr;
  attr.id = cudaLaunchAttributeClusterDimension;
  attr.val.clusterDim.x = 2;
  attr.val.clusterDim.y = 1;
  attr.val.clusterDim.z = 1;
  cfg.attrs = &attr;
  cfg.numAttrs = 1;
  return static_cast<int>(cudaLaunchKernelEx(&cfg, kern, tmA, tmB, a));
}

// Pairs the device can co-schedule for the split kernel (its resource use equals that of
// the 256 x 256 pair kernel).
static int split_capacity() {
  auto kern = gemm_pair_kernel<kNone, 1>;
  static bool configured[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !configured[dev]) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             Smem<1>::kTotal) != cudaSuccess)
      return -1;
    configured[dev] = true;
  }
  return max_pairs<1>(reinterpret_cast<const void*>(kern), Smem<1>::kTotal);
}

}  // namespace pair
}  // namespace b200

// C[M,N] = A[M,K] * B[N,K]^T on CTA pairs (256 x 256 tile per pair).  N must be a multiple of
// 256 and K of 64 (epi 2: gate / up interleaved in blocks of 32, C is [M, N/2]); other
// constraints as b200_gemm_bf16.  Returns -20 when the shape does not qualify or the device
// cannot co-schedule a cluster of two.
B200_API int b200_gemm_pair(const void* A, long long lda, const void* B, long long ldb, void* C,
                            long long ldc, int M, int N, int K, const void* bias, int epi,
                            void* stream) {
  using namespace b200;
  using namespace b200::pair;
  if (M <= 0 || N <= 0) return 0;
  if ((N % 256) != 0 || (K % BK) != 0 || K <= 0 || epi < 0 || epi > 2) return -20;
  if ((lda % 8) != 0 || (ldb % 8) != 0 || (ldc % 8) != 0) return -2;
  if ((reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(B) |
       reinterpret_cast<uintptr_t>(C)) & 15)
    return -3;
  if (epi == kBias && bias == nullptr) return -5;
  CUtensorMap tmA, tmB;
  int r = encode_tmap_2d(&tmA, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, A, static_cast<uint64_t>(M),
                         static_cast<uint64_t>(K), static_cast<uint64_t>(lda) * 2, BMH, BK,
                         CU_TENSOR_MAP_SWIZZLE_128B);
  if (r != 0) return r < 0 ? -6 : r;
  r = encode_tmap_2d(&tmB, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, B, static_cast<uint64_t>(N),
                     static_cast<uint64_t>(K), static_cast<uint64_t>(ldb) * 2, BNH, BK,
                     CU_TENSOR_MAP_SWIZZLE_128B);
  if (r != 0) return r < 0 ? -6 : r;
  Args a;
  a.C = static_cast<__nv_bfloat16*>(C);
  a.ldc = ldc;
  a.bias = static_cast<const __nv_bfloat16*>(bias);
  a.M = M; a.N = N; a.K = K;
  const int mt = getenv("VLLM_B200_PAIR_MT") != nullptr && atoi(getenv("VLLM_B200_PAIR_MT")) == 2
                     ? 2 : 1;
  a.tiles_m = (M + 256 * mt - 1) / (256 * mt);
  a.tiles_n = N / 256;
  a.num_kb = K / BK;
  a.status = status_ptr();
  a.splits = 1; a.ws = nullptr; a.ctr = nullptr;
  {
    int gm = 1;
    while (gm * gm < sm_count() / 2) ++gm;    // ~ sqrt(number of tiles in flight)
    const char* env = getenv("VLLM_B200_GEMM_GROUP_M");
    if (env != nullptr && atoi(env) > 0) gm = atoi(env);
    a.group_m = gm < a.tiles_m ? gm : a.tiles_m;
  }
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (mt == 1) {
    if (epi == kSiluMul) return launch<kSiluMul, 1>(tmA, tmB, a, s);
    if (epi == kBias) return launch<kBias, 1>(tmA, tmB, a, s);
    return launch<kNone, 1>(tmA, tmB, a, s);
  }
  if (epi == kSiluMul) return launch<kSiluMul, 2>(tmA, tmB, a, s);
  if (epi == kBias) return launch<kBias, 2>(tmA, tmB, a, s);
  return launch<kNone, 2>(tmA, tmB, a, s);
}

// Workspace the K-split entry wants: *ws_floats fp32 and *ctr_words zeroed 32-bit counters
// (both upper bounds for every shape it takes).  Returns 0, or -20 without cluster support.
B200_API int b200_gemm_pair_split_workspace(long long* ws_floats, int* ctr_words) {
  const int cap = b200::pair::split_capacity();
  if (cap <= 0) return -20;
  *ws_floats = static_cast<long long>(cap) * 256 * 256;
  *ctr_words = 2 * cap;
  return 0;
}

// C[M,N] = A[M,K] * B[N,K]^T on CTA pairs with a K split, for inputs whose 256 x 256 tiles are
// too few to occupy the SM pairs (M <= 512).  Constraints as b200_gemm_pair; `ws` / `ctr` from
// b200_gemm_pair_split_workspace (`ctr` zero on the first call; the kernel leaves it zero).
// Returns -20 when a split does not apply (enough tiles, K too short, no cluster support).
B200_API int b200_gemm_pair_split(const void* A, long long lda, const void* B, long long ldb,
                                  void* C, long long ldc, int M, int N, int K, const void* bias,
                                  int epi, float* ws, unsigned int* ctr, void* stream) {
  using namespace b200;
  using namespace b200::pair;
  if (M <= 0 || N <= 0) return 0;
  if ((N % 256) != 0 || (K % BK) != 0 || K <= 0 || epi < 0 || epi > 2 || M > 512 ||
      ws == nullptr || ctr == nullptr)
    return -20;
  if ((lda % 8) != 0 || (ldb % 8) != 0 || (ldc % 8) != 0) return -2;
  if ((reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(B) |
       reinterpret_cast<uintptr_t>(C)) & 15)
    return -3;
  if (epi == kBias && bias == nullptr) return -5;
  const int cap = split_capacity();
  if (cap <= 0) return -20;
  Args a;
  a.tiles_m = (M + 255) / 256;
  a.tiles_n = N / 256;
  a.num_kb = K / BK;
  const int tiles = a.tiles_m * a.tiles_n;
  int splits = cap / tiles;
  if (splits > a.num_kb / 8) splits = a.num_kb / 8;       // every slice keeps >= 8 K blocks
  if (splits > 8) splits = 8;
  if (splits < 2) return -20;
  CUtensorMap tmA, tmB;
  int r = encode_tmap_2d(&tmA, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, A, static_cast<uint64_t>(M),
                         static_cast<uint64_t>(K), static_cast<uint64_t>(lda) * 2, BMH, BK,
                         CU_TENSOR_MAP_SWIZZLE_128B);
  if (r != 0) return r < 0 ? -6 : r;
  r = encode_tmap_2d(&tmB, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, B, static_cast<uint64_t>(N),
                     static_cast<uint64_t>(K), static_cast<uint64_t>(ldb) * 2, BNH, BK,
                     CU_TENSOR_MAP_SWIZZLE_128B);
  if (r != 0) return r < 0 ? -6 : r;
  a.C = static_cast<__nv_bfloat16*>(C);
  a.ldc = ldc;
  a.bias = static_cast<const __nv_bfloat16*>(bias);
  a.M = M; a.N = N; a.K = K;
  a.group_m = 1;
  a.status = status_ptr();
  a.splits = splits;
  a.ws = ws;
  a.ctr = ctr;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int units = tiles * splits;
  if (epi == kSiluMul) return launch_split<kSiluMul>(tmA, tmB, a, units, s);
  if (epi == kBias) return launch_split<kBias>(tmA, tmB, a, units, s);
  return launch_split<kNone>(tmA, tmB, a, units, s);
}
