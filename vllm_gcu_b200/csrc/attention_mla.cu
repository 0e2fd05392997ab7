// Multi-head latent attention over the paged latent cache, on the 5th-generation tensor cores.
//
// Latent-absorbed form (vllm_gcu/attention/backends/mla_v1_fusion.py:60-180 calls the vendor's
// paged attention in "MLA mode" for it): every head of a token attends with a 576-wide query
// (512 latent + 64 rotary) to the same cache row of 576 values, and the value is the first 512
// of those.  One kernel covers decode (one token per request), multi-token verification and
// prefill chunks: query rows are (token, head) pairs, 128 rows per tile, a tile holds
// 128 / num_heads consecutive tokens of one request and each row sees the keys up to its own
// token's position.
//
//   S = Q K^T    tcgen05.mma over nine 64-wide chunks of the 576 columns; Q (nine chunks, loaded
//                once) and the key tile (64 keys x 576) are K-major in shared memory (TMA, 128-byte
//                swizzle); fp32 scores in tensor memory;
//   softmax      eight warps, two threads per row (32 keys each), lazily raised running maximum;
//                probabilities go to shared memory as bf16 in the K-major swizzled layout;
//   O += P V     V is the key tile itself read as an MN-major operand (keys x latent columns).
//
// The 128 x 512 fp32 output does not fit tensor memory next to the scores, so a tile is worked
// on by two CTAs (neighbours in blockIdx.x): both compute the scores, each accumulates 256 of the 512 output
// columns.  Two shapes of the kernel:
//   QROWS = 128  Q takes 144 KB, so there is room for one key tile (72 KB) only; the
//                probabilities reuse the chunks of the key tile that this CTA's half of V does
//                not need, which are free once the score MMAs have completed;
//   QROWS = 32   tiles with at most 32 valid rows (decode with up to 32 heads per rank): only
//                those rows of Q are loaded (the MMA still spans 128 rows and reads whatever
//                follows in shared memory for the others; rows are independent and the
//                surplus ones are never stored), which leaves room for two key tiles and a
//                separate P buffer: loads, score MMAs of tile j + 1 and softmax of tile j overlap.
// Long contexts are split over blockIdx.y; the partial results (normalised output +
// log-sum-exp per row) are merged by mla_combine_kernel.
//
// Warp roles: warp 0 TMA producer, warp 1 MMA issuer and TMEM owner, warps 2..9 softmax and
// epilogue.  Every wait is bounded and reports through the status word.
#include <mutex>
#include <unordered_map>

#include "common.cuh"

namespace b200 {
namespace mla {

constexpr unsigned int kKernelId = 22;
constexpr int BQ = 128;        // query rows (token, head) per tile
constexpr int BKV = 64;        // keys per tile
constexpr int kL = 512;        // latent width = value width
constexpr int kW = 576;        // latent + rotary
constexpr int kChunks = kW / 64;          // 9
constexpr int kPage = 16;      // tokens per TMA copy
constexpr int kThreads = 320;
constexpr int kKChunk = BKV * 128;        // [64 x 64] bf16: 8 KB
constexpr int kKTile = kChunks * kKChunk; // 72 KB
constexpr uint32_t kColS = 0;      // one or two score buffers of 64 columns
constexpr uint32_t kColO = 256;    // 256 columns of output
constexpr uint32_t kTmemCols = 512;

template <int QROWS>
struct Lay {
  static constexpr int kStages = QROWS == BQ ? 1 : 2;
  static constexpr int kQChunk = QROWS * 128;               // bytes of one 64-column chunk of Q
  static constexpr int kOffBar = 0;                          // barriers first: Q may be read past its end
  static constexpr int kOffX = 128;
  static constexpr int kOffQ = 2048;
  static constexpr int kOffK = kOffQ + kChunks * kQChunk;
  static constexpr int kOffP = kOffK + kStages * kKTile;     // separate P buffer (two stages only)
  static constexpr int kEnd = kOffP + (kStages == 2 ? BQ * 128 : 0);
  // the 128-row MMA reads 16 KB from the start of every Q chunk: keep that inside the allocation
  static constexpr int kReadEnd = kOffQ + (kChunks - 1) * kQChunk + BQ * 128;
  static constexpr int kSmemBytes = (kEnd > kReadEnd ? kEnd : kReadEnd) + 1024;
};

__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

struct Args {
  __nv_bfloat16* out;      // [T * N, 512]
  float* ws_o;             // splits > 1: [splits, T * N, 512] normalised partial outputs
  float* ws_lse;           // splits > 1: [splits, T * N] natural-log LSE (-inf: nothing seen)
  const int* cu_q;         // [B + 1], or null: one query token per request
  const int* seq_lens;     // [B]
  const int* block_tables; // [B, max_blocks]
  int B, T, N, log2N, max_blocks, block_size, splits;
  float scale;
  unsigned int* status;
};

template <int QROWS>
__global__ void __launch_bounds__(kThreads, 1)
    mla_attn_kernel(const __grid_constant__ CUtensorMap tmQ,
                    const __grid_constant__ CUtensorMap tmK, const Args a) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  using L = Lay<QROWS>;
  constexpr int kStages = L::kStages;
  constexpr int kOffQ = L::kOffQ, kOffK = L::kOffK, kQChunk = L::kQChunk;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::kOffBar);
  uint64_t* q_full = bars;
  uint64_t* k_full = bars + 1;      // [2]
  uint64_t* k_empty = bars + 3;     // [2]
  uint64_t* s_full = bars + 5;      // [2]
  uint64_t* s_empty = bars + 7;     // [2]
  uint64_t* p_full = bars + 9;
  uint64_t* o_done = bars + 10;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 11);
  volatile uint32_t* abort_flag = tmem_slot + 1;
  int* s_info = reinterpret_cast<int*>(tmem_slot + 2);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  // The two CTAs of a tile are neighbours in the grid, so they run at the same time and the
  // second one finds the key tiles in L2 (as separate grid rows they ran waves apart and
  // every tile was read from DRAM twice).
  const int half = blockIdx.x & 1;             // output columns [256 half, 256 half + 256)
  const int tile_id = blockIdx.x >> 1;
  const int split = blockIdx.y;
  const int tq = BQ >> a.log2N;                // tokens per tile

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&k_full[i], 1);
      mbar_init(&k_empty[i], 1);
      mbar_init(&s_full[i], 1);
      mbar_init(&s_empty[i], 8);
    }
    mbar_init(p_full, 8);
    mbar_init(o_done, 1);
    *abort_flag = 0u;
    mbar_fence_init();
    tma_prefetch_desc(&tmQ);
    tma_prefetch_desc(&tmK);
  }
  if (warp == 2) {
    // sequence and tile-in-sequence of this CTA: prefix sum of the tile counts, 32 requests
    // per step
    int found = -1, qt = 0, base = 0;
    for (int b0 = 0; b0 < a.B && found < 0; b0 += 32) {
      const int b = b0 + lane;
      int nt_b = 0;
      if (b < a.B) {
        const int ql = a.cu_q ? a.cu_q[b + 1] - a.cu_q[b] : 1;
        nt_b = (ql + tq - 1) / tq;
      }
      int inc = nt_b;
#pragma unroll
      for (int d = 1; d < 32; d <<= 1) {
        const int n = __shfl_up_sync(0xffffffffu, inc, d);
        if (lane >= d) inc += n;
      }
      const int start = base + inc - nt_b;
      const bool mine = nt_b > 0 && tile_id >= start && tile_id < start + nt_b;
      const unsigned int vote = __ballot_sync(0xffffffffu, mine);
      if (vote != 0u) {
        const int src = __ffs(vote) - 1;
        found = b0 + src;
        qt = tile_id - __shfl_sync(0xffffffffu, start, src);
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
  if (seq < 0) return;                          // surplus CTA (the grid is an upper bound)

  const int q_start = a.cu_q ? a.cu_q[seq] : seq;
  const int q_len = a.cu_q ? a.cu_q[seq + 1] - q_start : 1;
  const int seq_len = a.seq_lens[seq];
  const int tok0 = s_info[1] * tq;                        // first token of the tile, in the request
  const int ntok = min(tq, q_len - tok0);                 // valid tokens of the tile
  const int pos0 = seq_len - q_len + tok0;                // absolute position of the first token
  const int kv_hi = max(0, min(seq_len, pos0 + ntok));    // keys any row of the tile can see
  const int nt_all = (kv_hi + BKV - 1) / BKV;
  const int per = (nt_all + a.splits - 1) / a.splits;
  const int t0 = split * per;
  const int nt = max(0, min(nt_all, t0 + per) - t0);
  const long long row0 = (static_cast<long long>(q_start) + tok0) << a.log2N;   // first (token, head) row
  const long long rows_total = static_cast<long long>(a.T) << a.log2N;
  const int valid_rows = ntok << a.log2N;

  if (nt == 0) {
    // nothing to attend to in this split (or an empty request): neutral partial / zero output
    for (int i = threadIdx.x; i < valid_rows * 32; i += kThreads) {
      const int r = i >> 5, c8 = (i & 31) * 8;
      if (a.splits > 1) {
        float* dst = a.ws_o + (static_cast<long long>(split) * rows_total + row0 + r) * kL +
                     half * 256 + c8;
        *reinterpret_cast<float4*>(dst) = make_float4(0.f, 0.f, 0.f, 0.f);
        *reinterpret_cast<float4*>(dst + 4) = make_float4(0.f, 0.f, 0.f, 0.f);
      } else {
        *reinterpret_cast<uint4*>(a.out + (row0 + r) * kL + half * 256 + c8) =
            make_uint4(0u, 0u, 0u, 0u);
      }
    }
    if (a.splits > 1 && half == 0)
      for (int r = threadIdx.x; r < valid_rows; r += kThreads)
        a.ws_lse[static_cast<long long>(split) * rows_total + row0 + r] = -INFINITY;
    return;
  }

  if (warp == 1) {
    tmem_alloc(tmem_slot, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  // one stage: the probabilities live in two chunks of the key tile that this CTA's V half
  // does not use; two stages: in their own buffer
  const int p_chunk = half == 0 ? 4 : 0;
  uint8_t* p_smem = kStages == 1 ? smem + kOffK + p_chunk * kKChunk : smem + L::kOffP;

  if (warp == 0) {
    // ---------------- TMA producer ----------------
    // (One thread issues the 36 copies of a key tile; issuing them from all lanes of the warp
    // measured 25 % slower.)
    if (elect_one()) {
      mbar_expect_tx(q_full, kChunks * kQChunk);
      for (int c = 0; c < kChunks; ++c)
        tma_load_2d(smem + kOffQ + c * kQChunk, &tmQ, q_full, c * 64, static_cast<int>(row0));
      const int* bt = a.block_tables + static_cast<long long>(seq) * a.max_blocks;
      const int last_tok = seq_len - 1;
      for (int j = 0; j < nt; ++j) {
        const int st = j % kStages;
        const uint32_t use = static_cast<uint32_t>(j / kStages);
        if (!mbar_wait(&k_empty[st], (use & 1u) ^ 1u, a.status, kKernelId, 0x100u + st, abort_flag))
          break;
        mbar_expect_tx(&k_full[st], kKTile);
        const int key0 = (t0 + j) * BKV;
        for (int pg = 0; pg < BKV / kPage; ++pg) {
          const int tok = min(key0 + pg * kPage, last_tok);     // pages past the end: any valid page
          const int blk = bt[tok / a.block_size];
          const int y = blk * a.block_size + ((key0 + pg * kPage) % a.block_size);
          for (int c = 0; c < kChunks; ++c)
            tma_load_2d(smem + kOffK + st * kKTile + c * kKChunk + pg * (kPage * 128), &tmK,
                        &k_full[st], c * 64, y);
        }
        // While this tile is worked on, pull the next one into L2: its load then pays an L2
        // latency instead of an HBM latency (with one stage that load is on the critical path).
        if (j + 1 < nt) {
          const int nkey0 = (t0 + j + 1) * BKV;
          for (int pg = 0; pg < BKV / kPage; ++pg) {
            if (nkey0 + pg * kPage > last_tok) break;
            const int blk = bt[(nkey0 + pg * kPage) / a.block_size];
            const int y = blk * a.block_size + ((nkey0 + pg * kPage) % a.block_size);
            for (int c = 0; c < kChunks; ++c) tma_prefetch_2d(&tmK, c * 64, y);
          }
        }
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    if (elect_one()) {
      constexpr uint32_t kIdescS = make_idesc(BQ, BKV, 1, 1);
      constexpr uint32_t kIdescO = make_idesc(BQ, 256, 1, 1) | kIdescBMajorMN;
      const uint32_t q_addr = smem_u32(smem + kOffQ);
      const uint32_t p_addr = smem_u32(p_smem);
      auto issue_s = [&](int j) -> bool {
        const int st = j % kStages;
        const uint32_t use = static_cast<uint32_t>(j / kStages);
        if (!mbar_wait(&k_full[st], use & 1u, a.status, kKernelId, 0x210u + st, abort_flag))
          return false;
        if (kStages == 2 && j >= 2 &&
            !mbar_wait(&s_empty[st], (use - 1u) & 1u, a.status, kKernelId, 0x230u + st, abort_flag))
          return false;
        tc_fence_after();
        const uint32_t k_addr = smem_u32(smem + kOffK + st * kKTile);
#pragma unroll 1
        for (int c = 0; c < kChunks; ++c) {
#pragma unroll
          for (int ks = 0; ks < 4; ++ks)
            umma_f16(tmem_base + kColS + st * BKV,
                     make_desc_k_sw128(q_addr + c * kQChunk) + static_cast<uint64_t>(ks * 2),
                     make_desc_k_sw128(k_addr + c * kKChunk) + static_cast<uint64_t>(ks * 2),
                     kIdescS, (c > 0 || ks > 0) ? 1u : 0u);
        }
        umma_commit(&s_full[st]);
        return true;
      };
      bool ok = mbar_wait(q_full, 0, a.status, kKernelId, 0x200u, abort_flag);
      ok = ok && issue_s(0);
      for (int j = 0; ok && j < nt; ++j) {
        // Two stages: the scores of tile j + 1 and P V of tile j are issued in whichever order
        // their inputs arrive.  (The key tile j + 1 could only be requested after P V of tile
        // j - 1 had finished; waiting for it first would hold back P V of tile j.)
        bool s_pending = kStages == 2 && j + 1 < nt;
        const int st = j % kStages;
        if (s_pending) {
          const int st1 = (j + 1) % kStages;
          const uint32_t use1 = static_cast<uint32_t>((j + 1) / kStages);
          for (uint32_t it = 0; it < kMbarSpinLimit; ++it) {
            if (mbar_test(&k_full[st1], use1 & 1u) &&
                (j + 1 < 2 || mbar_test(&s_empty[st1], (use1 - 1u) & 1u))) {
              ok = issue_s(j + 1);            // its waits return at once
              s_pending = false;
              break;
            }
            if (mbar_test(p_full, j & 1)) break;
            if ((it & 1023u) == 1023u && *abort_flag != 0u) { ok = false; break; }
          }
        }
        if (!ok) break;
        if (!mbar_wait(p_full, j & 1, a.status, kKernelId, 0x220u, abort_flag)) break;
        tc_fence_after();
        const uint32_t k_addr = smem_u32(smem + kOffK + st * kKTile);
        const uint64_t vdesc = make_desc_mn_sw128(k_addr + half * 4 * kKChunk, kKChunk);
#pragma unroll
        for (int ks = 0; ks < BKV / 16; ++ks)
          umma_f16(tmem_base + kColO, make_desc_k_sw128(p_addr) + static_cast<uint64_t>(ks * 2),
                   vdesc + static_cast<uint64_t>(ks) * (2048 >> 4), kIdescO,
                   (j > 0 || ks > 0) ? 1u : 0u);
        umma_commit(&k_empty[st]);
        umma_commit(o_done);
        if ((kStages == 1 || s_pending) && j + 1 < nt) ok = issue_s(j + 1);
      }
    }
  } else {
    // ---------------- softmax + epilogue (warps 2..9) ----------------
    // group g: keys [32 g, 32 g + 32) of the tile and output columns [128 g, 128 g + 128) of
    // this CTA's half
    const int g = (warp - 2) >> 2;
    const int qd = warp & 3;                     // TMEM lane quarter
    const int r = qd * 32 + lane;                // row in the tile
    const uint32_t lane_addr = tmem_base + (static_cast<uint32_t>(qd * 32) << 16);
    const bool row_ok = r < valid_rows;
    const int hi = row_ok ? min(pos0 + (r >> a.log2N), seq_len - 1) : -1;   // last visible key
    const int hi_first = min(pos0, seq_len - 1);
    const float sl2 = a.scale * 1.4426950408889634f;
    float m_used = -INFINITY, l = 0.0f;
    float* xch = reinterpret_cast<float*>(smem + L::kOffX);    // [2][128]
    bool ok = true;
    for (int j = 0; j < nt; ++j) {
      const int st = j % kStages;
      if (ok && !mbar_wait(&s_full[st], static_cast<uint32_t>(j / kStages) & 1u, a.status,
                           kKernelId, 0x300u + st, abort_flag))
        ok = false;
      tc_fence_after();
      const int tile_key0 = (t0 + j) * BKV;
      const int key0 = tile_key0 + g * 32;
      const bool need_mask = valid_rows < BQ || tile_key0 + BKV - 1 > hi_first;
      uint32_t v[32];
      float mt = -INFINITY;
      if (ok) {
        tmem_ld_32x32(lane_addr + kColS + st * BKV + g * 32, v);
        tmem_ld_wait();
        if (need_mask) {
#pragma unroll
          for (int i = 0; i < 32; ++i)
            if (key0 + i <= hi) mt = fmaxf(mt, __uint_as_float(v[i]));
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) mt = fmaxf(mt, __uint_as_float(v[i]));
        }
      }
      xch[g * BQ + r] = mt;
      asm volatile("bar.sync 2, 256;" ::: "memory");
      mt = fmaxf(mt, xch[(g ^ 1) * BQ + r]);
      asm volatile("bar.sync 3, 256;" ::: "memory");
      float alpha = 1.0f;
      float m_new = m_used;
      if (mt > m_used && (m_used == -INFINITY || (mt - m_used) * sl2 > 8.0f)) {
        m_new = mt;
        alpha = m_used == -INFINITY ? 0.0f : ex2_approx((m_used - m_new) * sl2);
      }
      const float mb = (m_new == -INFINITY ? 0.0f : m_new) * sl2;
      uint32_t pk[16];
      float rs = 0.0f;
      if (ok) {
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          float p0 = ex2_approx(fmaf(__uint_as_float(v[i]), sl2, -mb));
          float p1 = ex2_approx(fmaf(__uint_as_float(v[i + 1]), sl2, -mb));
          if (need_mask) {
            if (key0 + i > hi) p0 = 0.0f;
            if (key0 + i + 1 > hi) p1 = 0.0f;
          }
          rs += p0 + p1;
          pk[i >> 1] = pack_bf16x2(p0, p1);
        }
      }
      l = l * alpha + rs;
      m_used = m_new;
      if (kStages == 2) {
        tc_fence_before();
        __syncwarp();
        if (ok && lane == 0) mbar_arrive(&s_empty[st]);
        // the previous P V product must be complete before P is overwritten / O is rescaled
        if (ok && j > 0 &&
            !mbar_wait(o_done, (j - 1) & 1, a.status, kKernelId, 0x310u, abort_flag))
          ok = false;
        tc_fence_after();
      }
      // (One stage: the previous P V product is complete already, the key tile of this
      // iteration was loaded only after it.)  Rescale the accumulator when the maximum rose.
      if (ok && j > 0 && __any_sync(0xffffffffu, alpha != 1.0f)) {
#pragma unroll 1
        for (int c = 0; c < 4; ++c) {
          uint32_t o[32];
          tmem_ld_32x32(lane_addr + kColO + g * 128 + c * 32, o);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
          tmem_st_32x32(lane_addr + kColO + g * 128 + c * 32, o);
        }
        tmem_st_wait();
      }
      if (ok) {
        // P row = 64 keys = 128 bytes; this thread owns 16-byte chunks 4 g .. 4 g + 3,
        // XOR-swizzled by row % 8
#pragma unroll
        for (int cc = 0; cc < 4; ++cc) {
          uint4 u = make_uint4(pk[cc * 4], pk[cc * 4 + 1], pk[cc * 4 + 2], pk[cc * 4 + 3]);
          *reinterpret_cast<uint4*>(p_smem + r * 128 + (((g * 4 + cc) ^ (r & 7)) << 4)) = u;
        }
        fence_async_smem();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(p_full);
      }
    }
    xch[g * BQ + r] = l;
    asm volatile("bar.sync 2, 256;" ::: "memory");
    l += xch[(g ^ 1) * BQ + r];
    if (ok && mbar_wait(o_done, (nt - 1) & 1, a.status, kKernelId, 0x320u, abort_flag)) {
      tc_fence_after();
      const float inv = l > 0.0f ? 1.0f / l : 0.0f;
      const long long grow = row0 + r;
      const int col0 = half * 256 + g * 128;
#pragma unroll 1
      for (int c = 0; c < 4; ++c) {
        uint32_t o[32];
        tmem_ld_32x32(lane_addr + kColO + g * 128 + c * 32, o);
        tmem_ld_wait();
        if (!row_ok) continue;
        if (a.splits > 1) {
          float* dst = a.ws_o + (static_cast<long long>(split) * rows_total + grow) * kL + col0 + c * 32;
#pragma unroll
          for (int i = 0; i < 8; ++i)
            *reinterpret_cast<float4*>(dst + i * 4) =
                make_float4(__uint_as_float(o[i * 4]) * inv, __uint_as_float(o[i * 4 + 1]) * inv,
                            __uint_as_float(o[i * 4 + 2]) * inv, __uint_as_float(o[i * 4 + 3]) * inv);
        } else {
          __nv_bfloat16* dst = a.out + grow * kL + col0 + c * 32;
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            uint4 u;
            u.x = pack_bf16x2(__uint_as_float(o[i * 8 + 0]) * inv, __uint_as_float(o[i * 8 + 1]) * inv);
            u.y = pack_bf16x2(__uint_as_float(o[i * 8 + 2]) * inv, __uint_as_float(o[i * 8 + 3]) * inv);
            u.z = pack_bf16x2(__uint_as_float(o[i * 8 + 4]) * inv, __uint_as_float(o[i * 8 + 5]) * inv);
            u.w = pack_bf16x2(__uint_as_float(o[i * 8 + 6]) * inv, __uint_as_float(o[i * 8 + 7]) * inv);
            *reinterpret_cast<uint4*>(dst + i * 8) = u;
          }
        }
      }
      if (a.splits > 1 && half == 0 && g == 0 && row_ok)
        a.ws_lse[static_cast<long long>(split) * rows_total + grow] =
            l > 0.0f ? m_used * a.scale + logf(l) : -INFINITY;
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_base, kTmemCols);
}

// out[row] = sum_z w_z * ws_o[z][row],  w_z = exp(lse_z - max) / sum exp(lse - max)
__global__ void __launch_bounds__(128)
    mla_combine_kernel(const float* ws_o, const float* ws_lse, __nv_bfloat16* out,
                       long long rows_total, int splits) {
  const long long row = blockIdx.x;
  float mx = -INFINITY;
  for (int z = 0; z < splits; ++z) mx = fmaxf(mx, ws_lse[z * rows_total + row]);
  float den = 0.0f;
  for (int z = 0; z < splits; ++z) {
    const float v = ws_lse[z * rows_total + row];
    den += v == -INFINITY ? 0.0f : __expf(v - mx);
  }
  const int c = threadIdx.x * 4;
  float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
  if (den > 0.0f) {
    for (int z = 0; z < splits; ++z) {
      const float v = ws_lse[z * rows_total + row];
      if (v == -INFINITY) continue;
      const float w = __expf(v - mx) / den;
      const float4 o = *reinterpret_cast<const float4*>(ws_o + (z * rows_total + row) * kL + c);
      acc.x += w * o.x; acc.y += w * o.y; acc.z += w * o.z; acc.w += w * o.w;
    }
  }
  uint2 u;
  u.x = pack_bf16x2(acc.x, acc.y);
  u.y = pack_bf16x2(acc.z, acc.w);
  *reinterpret_cast<uint2*>(out + row * kL + c) = u;
}

struct MapKey {
  const void* base;
  unsigned long long rows;
  int box_rows;
  bool operator==(const MapKey& o) const {
    return base == o.base && rows == o.rows && box_rows == o.box_rows;
  }
};
struct MapKeyHash {
  size_t operator()(const MapKey& k) const {
    return std::hash<const void*>()(k.base) ^ (k.rows * 1315423911ull) ^ k.box_rows;
  }
};

static int get_map(const void* base, unsigned long long rows, int box_rows, bool cache_it,
                   CUtensorMap* out) {
  static std::unordered_map<MapKey, CUtensorMap, MapKeyHash> cache;
  static std::mutex mu;
  MapKey key{base, rows, box_rows};
  std::lock_guard<std::mutex> lock(mu);
  if (cache_it) {
    auto it = cache.find(key);
    if (it != cache.end()) {
      *out = it->second;
      return 0;
    }
  }
  CUtensorMap m;
  int r = encode_tmap_2d(&m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, base, rows, kW,
                         static_cast<unsigned long long>(kW) * 2, box_rows, 64,
                         CU_TENSOR_MAP_SWIZZLE_128B);
  if (r != 0) return r;
  if (cache_it) {
    if (cache.size() > 4096) cache.clear();
    cache.emplace(key, m);
  }
  *out = m;
  return 0;
}

}  // namespace mla
}  // namespace b200

// Floats of workspace b200_mla_attention needs for `splits` > 1 (0 for one split).
B200_API long long b200_mla_workspace_floats(int T, int N, int splits) {
  if (splits <= 1) return 0;
  return static_cast<long long>(splits) * T * N * (b200::mla::kL + 1);
}

// q:    [T, N, 576] bf16 contiguous (latent-absorbed query | rotated rope part)
// cache:[num_slots, 576] bf16 (block b, offset o -> row b * block_size + o)
// out:  [T, N, 512] bf16.  cu_q null = one query token per request (decode, T == B).
// num_tiles >= sum_b ceil(q_len_b / (128 / N)).  N must be a power of two <= 128 and the block
// size a multiple of 16; otherwise -20 (callers fall back).
B200_API int b200_mla_attention(const void* q, void* out, const void* cache, long long num_slots,
                                const int* cu_q, const int* seq_lens, const int* block_tables,
                                int max_blocks, int block_size, int B, int T, int N,
                                int num_tiles, int splits, float* workspace, float scale,
                                void* stream) {
  using namespace b200;
  using namespace b200::mla;
  if (B <= 0 || T <= 0 || num_tiles <= 0) return 0;
  if (N <= 0 || N > BQ || (N & (N - 1)) != 0 || (block_size % kPage) != 0 ||
      ((reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(out) |
        reinterpret_cast<uintptr_t>(cache)) & 15))
    return -20;
  if (splits < 1) splits = 1;
  if (splits > 1 && workspace == nullptr) return -12;
  int log2N = 0;
  while ((1 << log2N) < N) ++log2N;
  // tiles with at most 32 valid rows (decode, up to 32 heads): the variant that loads only
  // those rows of Q and double-buffers the key tiles
  const bool small = cu_q == nullptr && N <= 32;
  CUtensorMap tmQ, tmK;
  int r = get_map(q, static_cast<unsigned long long>(T) * N, small ? 32 : BQ, false, &tmQ);
  if (r != 0) return r < 0 ? -6 : r;
  r = get_map(cache, static_cast<unsigned long long>(num_slots), kPage, true, &tmK);
  if (r != 0) return r < 0 ? -6 : r;
  Args a;
  a.out = static_cast<__nv_bfloat16*>(out);
  const long long rows_total = static_cast<long long>(T) * N;
  a.ws_o = workspace;
  a.ws_lse = workspace ? workspace + static_cast<long long>(splits) * rows_total * kL : nullptr;
  a.cu_q = cu_q; a.seq_lens = seq_lens; a.block_tables = block_tables;
  a.B = B; a.T = T; a.N = N; a.log2N = log2N; a.max_blocks = max_blocks;
  a.block_size = block_size; a.splits = splits; a.scale = scale;
  a.status = status_ptr();
  static bool configured[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !configured[dev]) {
    cudaError_t e = cudaFuncSetAttribute(mla_attn_kernel<BQ>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         Lay<BQ>::kSmemBytes);
    if (e == cudaSuccess)
      e = cudaFuncSetAttribute(mla_attn_kernel<32>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                               Lay<32>::kSmemBytes);
    if (e != cudaSuccess) return static_cast<int>(e);
    configured[dev] = true;
  }
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  dim3 grid(num_tiles * 2, splits);
  if (small)
    mla_attn_kernel<32><<<grid, kThreads, Lay<32>::kSmemBytes, s>>>(tmQ, tmK, a);
  else
    mla_attn_kernel<BQ><<<grid, kThreads, Lay<BQ>::kSmemBytes, s>>>(tmQ, tmK, a);
  int e = static_cast<int>(cudaGetLastError());
  if (e != 0 || splits == 1) return e;
  mla_combine_kernel<<<static_cast<unsigned>(rows_total), 128, 0, s>>>(a.ws_o, a.ws_lse, a.out,
                                                                      rows_total, splits);
  return static_cast<int>(cudaGetLastError());
}
