// Prefill / chunked-prefill / prefix attention on the 5th-generation tensor cores.
//
// One CTA = 128 query rows of one head.  Per tile of 128 keys:
//   S = Q K^T      tcgen05.mma, Q and K tiles K-major in shared memory (TMA, 128-byte swizzle),
//                  fp32 scores in tensor memory (two buffers);
//   softmax        eight warps, two threads per query row (64 keys each): two passes over the
//                  scores in TMEM (row maximum, then exp2 and row sum), probabilities written
//                  to shared memory as bf16 in the K-major swizzled layout the next MMA reads;
//   O += P V       tcgen05.mma with V as an MN-major operand (keys x head_dim rows exactly as
//                  they lie in the paged cache), output accumulated in tensor memory.
// The running maximum is only raised when the new maximum exceeds it by more than 8 (log2
// domain); otherwise probabilities up to 2^8 are used, which fp32 sums and bf16 P hold, and
// the accumulator in TMEM needs no rescale.  When it is raised, the softmax warps rescale
// the accumulator in place (tcgen05.ld / tcgen05.st) between two P V products.
// Warp roles: warp 0 TMA producer (K and V pages through the block table, 16 tokens per
// copy), warp 1 MMA issuer and TMEM owner, warps 2..9 softmax and epilogue.  S of tile j + 1
// is issued before P V of tile j, so the tensor cores compute the next scores while the
// softmax warps work on the current ones.
//
// Semantics of context_attention_forward / flash_attn_varlen with a block table
// (csrc/src/context_attention_forward.cpp:49, vllm_gcu/v1/attention/flash_attn.py:26-177):
// causal over absolute positions, optional sliding window, GQA, natural-log LSE output.
#include <mutex>
#include <unordered_map>

#include "common.cuh"

namespace b200 {
namespace fmha {

constexpr unsigned int kKernelId = 21;
constexpr int BQ = 128;      // query rows per CTA
constexpr int BKV = 128;     // keys per tile
constexpr int HD = 128;      // head dimension
constexpr int kPage = 16;    // tokens per TMA copy (divides the cache block size)
constexpr int kThreads = 320;   // TMA warp, MMA warp, 2 x 4 softmax warps
constexpr int kSub = BQ * 64 * 2;          // one [128 x 64] bf16 sub-tile: 16 KB
constexpr int kTile = 2 * kSub;            // a [128 x 128] bf16 tile: 32 KB
constexpr int kStages = 2;

// shared memory map (bytes, tile bases 1024-aligned)
constexpr int kOffQ = 0;
constexpr int kOffK = kOffQ + kTile;
constexpr int kOffV = kOffK + kStages * kTile;
constexpr int kOffP = kOffV + kStages * kTile;
constexpr int kOffBar = kOffP + kTile;
constexpr int kOffX = kOffBar + 256;       // row maxima / sums exchanged between the warp groups
constexpr int kSmemBytes = kOffX + 2 * BQ * 4 + 1024;

// tensor memory columns
constexpr uint32_t kColS = 0;      // two score buffers of 128 columns
constexpr uint32_t kColO = 256;    // output accumulator, 128 columns
constexpr uint32_t kTmemCols = 512;

__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

struct Args {
  __nv_bfloat16* out;      // [T, Hq * 128], row pitch ldo
  float* lse;              // optional [Hq, T]
  const int* cu_q;         // [B + 1]
  const int* seq_lens;     // [B]
  const int* block_tables; // [B, max_blocks]
  long long ldo;
  int B, T, Hq, Hkv, max_blocks, block_size, causal, window;
  float scale;
  unsigned int* status;
};

__global__ void __launch_bounds__(kThreads, 1)
    fmha_prefill_kernel(const __grid_constant__ CUtensorMap tmQ,
                        const __grid_constant__ CUtensorMap tmK,
                        const __grid_constant__ CUtensorMap tmV, const Args a) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kOffBar);
  uint64_t* q_full = bars;             // 1
  uint64_t* k_full = bars + 1;         // 2
  uint64_t* k_empty = bars + 3;        // 2
  uint64_t* v_full = bars + 5;         // 2
  uint64_t* v_empty = bars + 7;        // 2
  uint64_t* s_full = bars + 9;         // 2
  uint64_t* s_empty = bars + 11;       // 2
  uint64_t* p_full = bars + 13;        // 1
  uint64_t* o_done = bars + 14;        // 1
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 15);
  volatile uint32_t* abort_flag = tmem_slot + 1;
  int* s_info = reinterpret_cast<int*>(tmem_slot + 2);   // [0] sequence, [1] q tile in sequence

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int head = blockIdx.y;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&k_full[i], 1);
      mbar_init(&k_empty[i], 1);
      mbar_init(&v_full[i], 1);
      mbar_init(&v_empty[i], 1);
      mbar_init(&s_full[i], 1);
      mbar_init(&s_empty[i], 8);
    }
    mbar_init(p_full, 8);
    mbar_init(o_done, 1);
    *abort_flag = 0u;
    mbar_fence_init();
    tma_prefetch_desc(&tmQ);
    tma_prefetch_desc(&tmK);
    tma_prefetch_desc(&tmV);
  }
  if (warp == 2) {
    // which sequence and query tile this CTA works on: 32 sequences per step, all lanes load
    // in parallel, prefix sum of the tile counts inside the warp
    int found = -1, qt = 0, base = 0;
    for (int b0 = 0; b0 < a.B && found < 0; b0 += 32) {
      const int b = b0 + lane;
      int nt_b = 0;
      if (b < a.B) nt_b = (a.cu_q[b + 1] - a.cu_q[b] + BQ - 1) / BQ;
      int inc = nt_b;
#pragma unroll
      for (int d = 1; d < 32; d <<= 1) {
        const int n = __shfl_up_sync(0xffffffffu, inc, d);
        if (lane >= d) inc += n;
      }
      const int start = base + inc - nt_b;
      const bool mine = nt_b > 0 && static_cast<int>(blockIdx.x) >= start &&
                        static_cast<int>(blockIdx.x) < start + nt_b;
      const unsigned int vote = __ballot_sync(0xffffffffu, mine);
      if (vote != 0u) {
        const int src = __ffs(vote) - 1;
        found = b0 + src;
        qt = static_cast<int>(blockIdx.x) - __shfl_sync(0xffffffffu, start, src);
      }
      base += __shfl_sync(0xffffffffu, inc, 31);
    }
    if (lane == 0) {
      s_info[0] = found;
      s_info[1] = qt;
    }
  }
  __syncthreads();
  const int seq = s_info[0];
  if (seq < 0) return;                       // surplus CTA (grid is an upper bound)
  if (warp == 1) {
    tmem_alloc(tmem_slot, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  const int q_start = a.cu_q[seq];
  const int q_len = a.cu_q[seq + 1] - q_start;
  const int seq_len = a.seq_lens[seq];
  const int q0 = s_info[1] * BQ;                        // first query of the tile, in the sequence
  const int rows = min(BQ, q_len - q0);
  const int pos0 = seq_len - q_len + q0;                // absolute position of the tile's first row
  // keys the tile can see: [kv_lo, kv_hi)
  const int kv_hi = a.causal ? min(seq_len, pos0 + rows) : seq_len;
  int kv_lo = 0;
  if (a.window > 0) kv_lo = max(0, pos0 - a.window + 1);
  const int t0 = kv_lo / BKV;
  const int nt = (kv_hi + BKV - 1) / BKV - t0;          // >= 1
  const int kvh = head / (a.Hq / a.Hkv);

  if (warp == 0) {
    // ---------------- TMA producer ----------------
    if (elect_one()) {
      mbar_expect_tx(q_full, kTile);
      tma_load_2d(smem + kOffQ, &tmQ, q_full, head * HD, q_start + q0);
      tma_load_2d(smem + kOffQ + kSub, &tmQ, q_full, head * HD + 64, q_start + q0);
      const int* bt = a.block_tables + static_cast<long long>(seq) * a.max_blocks;
      const int last_tok = seq_len - 1;
      bool ok = true;
      for (int j = 0; ok && j < nt; ++j) {
        const int st = j & 1;
        const uint32_t par = ((j >> 1) & 1) ^ 1u;
        const int key0 = (t0 + j) * BKV;
        for (int kv = 0; kv < 2 && ok; ++kv) {
          uint64_t* empty = kv == 0 ? &k_empty[st] : &v_empty[st];
          uint64_t* full = kv == 0 ? &k_full[st] : &v_full[st];
          const CUtensorMap* tm = kv == 0 ? &tmK : &tmV;
          uint8_t* dst = smem + (kv == 0 ? kOffK : kOffV) + st * kTile;
          if (!mbar_wait(empty, par, a.status, kKernelId, 0x100u + kv * 16 + st, abort_flag)) {
            ok = false;
            break;
          }
          mbar_expect_tx(full, kTile);
          for (int c = 0; c < BKV / kPage; ++c) {
            const int tok = min(key0 + c * kPage, last_tok);   // pages past the end: any valid page
            const int blk = bt[tok / a.block_size];
            const int y = blk * a.block_size + ((key0 + c * kPage) % a.block_size);
            const int x = kvh * HD;
            tma_load_2d(dst + c * (kPage * 128), tm, full, x, y);
            tma_load_2d(dst + kSub + c * (kPage * 128), tm, full, x + 64, y);
          }
        }
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    if (elect_one()) {
      constexpr uint32_t kIdescS = make_idesc(BQ, BKV, 1, 1);
      constexpr uint32_t kIdescO = make_idesc(BQ, HD, 1, 1) | kIdescBMajorMN;
      const uint32_t q_addr = smem_u32(smem + kOffQ);
      const uint32_t p_addr = smem_u32(smem + kOffP);
      auto issue_s = [&](int j) -> bool {
        const int st = j & 1;
        if (!mbar_wait(&k_full[st], (j >> 1) & 1, a.status, kKernelId, 0x200u + st, abort_flag))
          return false;
        if (j >= 2 &&
            !mbar_wait(&s_empty[st], ((j >> 1) - 1) & 1, a.status, kKernelId, 0x210u + st, abort_flag))
          return false;
        tc_fence_after();
        const uint32_t k_addr = smem_u32(smem + kOffK + st * kTile);
#pragma unroll
        for (int ks = 0; ks < HD / 16; ++ks) {
          const uint32_t sub = (ks >> 2) * kSub;
          umma_f16(tmem_base + kColS + st * BKV,
                   make_desc_k_sw128(q_addr + sub) + static_cast<uint64_t>((ks & 3) * 2),
                   make_desc_k_sw128(k_addr + sub) + static_cast<uint64_t>((ks & 3) * 2), kIdescS,
                   ks > 0 ? 1u : 0u);
        }
        umma_commit(&k_empty[st]);
        umma_commit(&s_full[st]);
        return true;
      };
      bool ok = mbar_wait(q_full, 0, a.status, kKernelId, 0x220u, abort_flag);
      ok = ok && issue_s(0);
      for (int j = 0; ok && j < nt; ++j) {
        if (j + 1 < nt) ok = issue_s(j + 1);
        if (!ok) break;
        const int st = j & 1;
        if (!mbar_wait(&v_full[st], (j >> 1) & 1, a.status, kKernelId, 0x230u + st, abort_flag) ||
            !mbar_wait(p_full, j & 1, a.status, kKernelId, 0x240u, abort_flag)) {
          ok = false;
          break;
        }
        tc_fence_after();
        const uint32_t v_addr = smem_u32(smem + kOffV + st * kTile);
        const uint64_t vdesc = make_desc_mn_sw128(v_addr, kSub);
#pragma unroll
        for (int ks = 0; ks < BKV / 16; ++ks) {
          umma_f16(tmem_base + kColO,
                   make_desc_k_sw128(p_addr + (ks >> 2) * kSub) + static_cast<uint64_t>((ks & 3) * 2),
                   vdesc + static_cast<uint64_t>(ks) * (2048 >> 4), kIdescO,
                   (j > 0 || ks > 0) ? 1u : 0u);
        }
        umma_commit(&v_empty[st]);
        umma_commit(o_done);
      }
    }
  } else {
    // ---------------- softmax + epilogue (warps 2..9) ----------------
    // Two groups of four warps: group g handles keys / output columns [64 g, 64 g + 64) of
    // every row, so each scheduler holds two softmax warps and one covers the other's TMEM
    // and arithmetic latency.  The two threads of a row exchange their partial row maximum
    // through shared memory once per tile; row sums stay per thread until the end.
    const int g = (warp - 2) >> 2;
    const int qd = warp & 3;                    // TMEM lane quarter
    const int r = qd * 32 + lane;               // query row in the tile
    const uint32_t lane_addr = tmem_base + (static_cast<uint32_t>(qd * 32) << 16);
    const int pos = pos0 + r;
    const int hi = a.causal ? min(pos, seq_len - 1) : seq_len - 1;      // last visible key
    const int lo = a.window > 0 ? max(0, pos - a.window + 1) : 0;       // first visible key
    const float sl2 = a.scale * 1.4426950408889634f;
    float m_used = -INFINITY, l = 0.0f;
    uint8_t* sp = smem + kOffP + g * kSub;      // this group's 64-key sub-tile of P
    float* xch = reinterpret_cast<float*>(smem + kOffX);   // [2][128]
    bool ok = true;
    for (int j = 0; j < nt; ++j) {
      const int b = j & 1;
      if (ok && !mbar_wait(&s_full[b], (j >> 1) & 1, a.status, kKernelId, 0x300u + b, abort_flag))
        ok = false;
      tc_fence_after();
      const uint32_t s_addr = lane_addr + kColS + b * BKV + g * 64;
      const int key0 = (t0 + j) * BKV + g * 64;
      // Only tiles that touch the causal diagonal, the window start or the end of the
      // sequence need per-element masks; the test is uniform over the CTA.
      const int tile_key0 = (t0 + j) * BKV;
      const bool need_mask =
          (tile_key0 + BKV - 1 > (a.causal ? min(pos0, seq_len - 1) : seq_len - 1)) ||
          (a.window > 0 && tile_key0 < pos0 + BQ - a.window);
      // pass 1: maximum over this thread's 64 keys
      float mt = -INFINITY;
      if (ok) {
#pragma unroll 1
        for (int c = 0; c < 2; ++c) {
          uint32_t v[32];
          tmem_ld_32x32(s_addr + c * 32, v);
          tmem_ld_wait();
          if (need_mask) {
#pragma unroll
            for (int i = 0; i < 32; ++i) {
              const int key = key0 + c * 32 + i;
              if (key <= hi && key >= lo) mt = fmaxf(mt, __uint_as_float(v[i]));
            }
          } else {
            float m0 = mt, m1 = -INFINITY, m2 = -INFINITY, m3 = -INFINITY;
#pragma unroll
            for (int i = 0; i < 32; i += 4) {
              m0 = fmaxf(m0, __uint_as_float(v[i]));
              m1 = fmaxf(m1, __uint_as_float(v[i + 1]));
              m2 = fmaxf(m2, __uint_as_float(v[i + 2]));
              m3 = fmaxf(m3, __uint_as_float(v[i + 3]));
            }
            mt = fmaxf(fmaxf(m0, m1), fmaxf(m2, m3));
          }
        }
      }
      xch[g * BQ + r] = mt;
      asm volatile("bar.sync 2, 256;" ::: "memory");       // every softmax thread, every tile
      mt = fmaxf(mt, xch[(g ^ 1) * BQ + r]);
      asm volatile("bar.sync 3, 256;" ::: "memory");       // the slot may be rewritten next tile
      float alpha = 1.0f;
      float m_new = m_used;
      if (mt > m_used && (m_used == -INFINITY || (mt - m_used) * sl2 > 8.0f)) {
        m_new = mt;
        alpha = m_used == -INFINITY ? 0.0f : ex2_approx((m_used - m_new) * sl2);
      }
      const float mb = (m_new == -INFINITY ? 0.0f : m_new) * sl2;
      // pass 2: probabilities (bf16, kept in registers until the P buffer is free) and row sum
      uint32_t pk[32];
      float rs0 = 0.0f, rs1 = 0.0f;
      if (ok) {
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          uint32_t v[32];
          tmem_ld_32x32(s_addr + c * 32, v);
          tmem_ld_wait();
          if (need_mask) {
#pragma unroll
            for (int i = 0; i < 32; i += 2) {
              const int key = key0 + c * 32 + i;
              float p0 = ex2_approx(fmaf(__uint_as_float(v[i]), sl2, -mb));
              float p1 = ex2_approx(fmaf(__uint_as_float(v[i + 1]), sl2, -mb));
              if (key > hi || key < lo) p0 = 0.0f;
              if (key + 1 > hi || key + 1 < lo) p1 = 0.0f;
              rs0 += p0;
              rs1 += p1;
              pk[c * 16 + (i >> 1)] = pack_bf16x2(p0, p1);
            }
          } else {
#pragma unroll
            for (int i = 0; i < 32; i += 2) {
              const float p0 = ex2_approx(fmaf(__uint_as_float(v[i]), sl2, -mb));
              const float p1 = ex2_approx(fmaf(__uint_as_float(v[i + 1]), sl2, -mb));
              rs0 += p0;
              rs1 += p1;
              pk[c * 16 + (i >> 1)] = pack_bf16x2(p0, p1);
            }
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (ok && lane == 0) mbar_arrive(&s_empty[b]);
      l = l * alpha + rs0 + rs1;
      m_used = m_new;
      // the previous P V product must be complete before P is overwritten / O is rescaled
      if (ok && j > 0) {
        if (!mbar_wait(o_done, (j - 1) & 1, a.status, kKernelId, 0x310u, abort_flag)) ok = false;
        tc_fence_after();
        if (ok && __any_sync(0xffffffffu, alpha != 1.0f)) {
#pragma unroll 1
          for (int c = 0; c < 2; ++c) {
            uint32_t v[32];
            tmem_ld_32x32(lane_addr + kColO + g * 64 + c * 32, v);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) v[i] = __float_as_uint(__uint_as_float(v[i]) * alpha);
            tmem_st_32x32(lane_addr + kColO + g * 64 + c * 32, v);
          }
          tmem_st_wait();
        }
      }
      if (ok) {
        // P -> shared memory, K-major rows of 128 bytes, 16-byte chunks XOR-swizzled by row % 8
#pragma unroll
        for (int cc = 0; cc < 8; ++cc) {
          uint4 u = make_uint4(pk[cc * 4], pk[cc * 4 + 1], pk[cc * 4 + 2], pk[cc * 4 + 3]);
          *reinterpret_cast<uint4*>(sp + r * 128 + ((cc ^ (r & 7)) << 4)) = u;
        }
        fence_async_smem();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(p_full);
      }
    }
    // epilogue: total row sum = both halves
    xch[g * BQ + r] = l;
    asm volatile("bar.sync 2, 256;" ::: "memory");
    l += xch[(g ^ 1) * BQ + r];
    if (ok && mbar_wait(o_done, (nt - 1) & 1, a.status, kKernelId, 0x320u, abort_flag)) {
      tc_fence_after();
      const float inv = l > 0.0f ? 1.0f / l : 0.0f;
      const bool row_ok = r < rows;
      __nv_bfloat16* orow =
          a.out + static_cast<long long>(q_start + q0 + r) * a.ldo + head * HD + g * 64;
#pragma unroll 1
      for (int c = 0; c < 2; ++c) {
        uint32_t v[32];
        tmem_ld_32x32(lane_addr + kColO + g * 64 + c * 32, v);
        tmem_ld_wait();
        if (row_ok) {
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            uint4 u;
            u.x = pack_bf16x2(__uint_as_float(v[i * 8 + 0]) * inv, __uint_as_float(v[i * 8 + 1]) * inv);
            u.y = pack_bf16x2(__uint_as_float(v[i * 8 + 2]) * inv, __uint_as_float(v[i * 8 + 3]) * inv);
            u.z = pack_bf16x2(__uint_as_float(v[i * 8 + 4]) * inv, __uint_as_float(v[i * 8 + 5]) * inv);
            u.w = pack_bf16x2(__uint_as_float(v[i * 8 + 6]) * inv, __uint_as_float(v[i * 8 + 7]) * inv);
            *reinterpret_cast<uint4*>(orow + c * 32 + i * 8) = u;
          }
        }
      }
      if (g == 0 && row_ok && a.lse != nullptr)
        a.lse[static_cast<long long>(head) * a.T + q_start + q0 + r] =
            l > 0.0f ? m_used * a.scale + logf(l) : -INFINITY;
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_base, kTmemCols);
}

// Tensor maps are cached per (base, rows, cols, box rows): the KV caches of a model never move.
struct MapKey {
  const void* base;
  unsigned long long rows, cols;
  int box_rows;
  bool operator==(const MapKey& o) const {
    return base == o.base && rows == o.rows && cols == o.cols && box_rows == o.box_rows;
  }
};
struct MapKeyHash {
  size_t operator()(const MapKey& k) const {
    return std::hash<const void*>()(k.base) ^ (k.rows * 1315423911ull) ^ (k.cols << 7) ^ k.box_rows;
  }
};

static int get_map(const void* base, unsigned long long rows, unsigned long long cols,
                   unsigned long long ld_bytes, int box_rows, bool cache_it, CUtensorMap* out) {
  static std::unordered_map<MapKey, CUtensorMap, MapKeyHash> cache;
  static std::mutex mu;
  MapKey key{base, rows, cols, box_rows};
  std::lock_guard<std::mutex> lock(mu);
  if (cache_it) {
    auto it = cache.find(key);
    if (it != cache.end()) {
      *out = it->second;
      return 0;
    }
  }
  CUtensorMap m;
  int r = encode_tmap_2d(&m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, base, rows, cols, ld_bytes,
                         box_rows, 64, CU_TENSOR_MAP_SWIZZLE_128B);
  if (r != 0) return r;
  if (cache_it) {
    if (cache.size() > 4096) cache.clear();
    cache.emplace(key, m);
  }
  *out = m;
  return 0;
}

}  // namespace fmha
}  // namespace b200

// Same contract as b200_varlen_prefill for bf16, head_dim 128, caches laid out as
// [num_slots, Hkv * 128] rows and a block size that is a multiple of 16; num_q_tiles must be
// >= sum_b ceil(q_len_b / 128).  Returns -20 when the layout does not qualify (callers use
// b200_varlen_prefill).
B200_API int b200_fmha_prefill(const void* q, long long ldq, void* out, long long ldo, float* lse,
                               const int* cu_q, const int* seq_lens, const void* k_cache,
                               const void* v_cache, long long slot_stride, long long head_stride,
                               long long num_slots, const int* block_tables, int max_blocks,
                               int block_size, int B, int T, int num_q_tiles, int Hq, int Hkv,
                               int HD, float scale, int causal, int window, int dtype,
                               void* stream) {
  using namespace b200;
  using namespace b200::fmha;
  if (B <= 0 || T <= 0 || num_q_tiles <= 0) return 0;
  if (dtype != 0 || HD != fmha::HD || (block_size % kPage) != 0 || head_stride != fmha::HD ||
      slot_stride != static_cast<long long>(Hkv) * fmha::HD || Hkv <= 0 || Hq % Hkv != 0 ||
      (ldq % 8) != 0 || (ldo % 8) != 0 ||
      ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(out) |
        reinterpret_cast<uintptr_t>(k_cache) | reinterpret_cast<uintptr_t>(v_cache)) & 15))
    return -20;
  CUtensorMap tmQ, tmK, tmV;
  const unsigned long long cols = static_cast<unsigned long long>(Hkv) * fmha::HD;
  int r = get_map(q, static_cast<unsigned long long>(T), static_cast<unsigned long long>(Hq) * fmha::HD,
                  static_cast<unsigned long long>(ldq) * 2, BQ, false, &tmQ);
  if (r != 0) return r < 0 ? -6 : r;
  r = get_map(k_cache, static_cast<unsigned long long>(num_slots), cols, cols * 2, kPage, true, &tmK);
  if (r != 0) return r < 0 ? -6 : r;
  r = get_map(v_cache, static_cast<unsigned long long>(num_slots), cols, cols * 2, kPage, true, &tmV);
  if (r != 0) return r < 0 ? -6 : r;
  Args a;
  a.out = static_cast<__nv_bfloat16*>(out);
  a.lse = lse; a.cu_q = cu_q; a.seq_lens = seq_lens; a.block_tables = block_tables;
  a.ldo = ldo; a.B = B; a.T = T; a.Hq = Hq; a.Hkv = Hkv; a.max_blocks = max_blocks;
  a.block_size = block_size; a.causal = causal; a.window = window; a.scale = scale;
  a.status = status_ptr();
  static bool configured[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !configured[dev]) {
    cudaError_t e = cudaFuncSetAttribute(fmha_prefill_kernel,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
    if (e != cudaSuccess) return static_cast<int>(e);
    configured[dev] = true;
  }
  dim3 grid(num_q_tiles, Hq);
  fmha_prefill_kernel<<<grid, kThreads, kSmemBytes, static_cast<cudaStream_t>(stream)>>>(
      tmQ, tmK, tmV, a);
  return static_cast<int>(cudaGetLastError());
}
