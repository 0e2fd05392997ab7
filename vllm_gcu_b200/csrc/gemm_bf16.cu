// Dense bf16 GEMM for sm_100a:  C[M,N] = A[M,K] * B[N,K]^T  (+ epilogue).
//
// Design
//   * persistent kernel, one CTA per SM, static round-robin tile schedule with
//     the M index fastest so CTAs that run at the same time share a weight tile
//     in L2;
//   * warp 0 = TMA producer, warp 1 = tcgen05.mma issuer and TMEM owner,
//     warps 2..5 = epilogue (one TMEM lane quarter each);
//   * operands are staged by TMA into 128-byte-swizzled K-major tiles
//     (BM x 64 and BN x 64 bf16) through a STAGES-deep mbarrier ring;
//   * accumulators live in tensor memory, double buffered (2 x BN fp32 columns)
//     so the epilogue of tile i overlaps the main loop of tile i+1;
//   * epilogues: plain, +bias, SiLU(gate)*up for a gate/up weight interleaved in
//     blocks of 32 rows, +residual, fp32 output.
//
// Replaces the vendor matmul behind every unquantised linear layer of the
// reference (vllm_gcu/kernels/linear.py, upstream UnquantizedLinearMethod) and
// folds vllm_gcu/kernels/activation.py:20-32 (SiluAndMul) into the gate-up GEMM.
#include "common.cuh"

namespace b200 {
namespace gemm {

constexpr unsigned int kKernelId = 10;
constexpr int BM = 128;
constexpr int BK = 64;
constexpr int UMMA_K = 16;
constexpr int kThreads = 192;

enum Epilogue : int {
  kEpiNone = 0,
  kEpiBias = 1,
  kEpiSiluMul = 2,
  kEpiResidual = 3,
  kEpiFp32 = 4,
  kEpiAllReduce = 5,  // row-parallel partial product -> tile-wise two-shot all-reduce over peers
  kEpiAllGather = 6,  // column-parallel shard -> every peer's full-width output (peer stores)
  kEpiGatherA = 7,    // A rows are gathered from the peers' shards by extra warps of this kernel
  kEpiReduceNorm = 8, // row-parallel partial -> row owners reduce (+ residual, RMSNorm) and broadcast
};

template <int EPI>
constexpr int kThreadsFor =
    (EPI == kEpiGatherA || EPI == kEpiAllReduce || EPI == kEpiReduceNorm) ? 320 : 192;
template <int EPI>
constexpr bool kPeerEpi = (EPI == kEpiAllReduce || EPI == kEpiAllGather || EPI == kEpiGatherA ||
                           EPI == kEpiReduceNorm);

constexpr int kMaxPeers = 8;

// Peer-visible addresses of the symmetric buffers used by the fused all-reduce epilogue.
// Index r is rank r's copy; [rank] is this GPU's own memory.
struct ArArgs {
  __nv_bfloat16* partial[kMaxPeers];  // [tiles][BM*BN] bf16 partial products of rank r
  __nv_bfloat16* out[kMaxPeers];      // [M, ldc] reduced result on rank r
  uint32_t* ready[kMaxPeers];         // [tiles][p]: partial of (tile, src) is complete (epoch value)
  uint32_t* done[kMaxPeers];          // [tiles]: reduced tile has been written to rank r (epoch)
  uint32_t* epoch_ptr;                // local: epoch of the previous launch
  uint32_t* done_ctr;                 // local: CTAs of this launch that have finished
  int rank, p;
  int oneshot;                        // 1: push partials to every peer, reduce locally
  long long slot_elems;               // one-shot: elements per (parity, source rank) slot
  long long col_off;                  // all-gather epilogue: first output column of this rank
  // row-owner reduce (kEpiReduceNorm): rank r reduces rows [128 r / p, 128 (r + 1) / p) of every
  // 128-row tile, adds the residual, normalises and stores the rows into every rank
  __nv_bfloat16* res_out[kMaxPeers];  // [M, N] new residual on rank r (symmetric)
  const __nv_bfloat16* res_in;        // local [M, ld_res_in] residual (null: none)
  long long ld_res_in;
  const __nv_bfloat16* norm_weight;   // [N] (null: plain all-reduce, out = sum + residual)
  float eps;
  int bcast_res;                      // 1: the new residual goes to every rank, 0: owner only
  // how the partial rows reach their reducer:
  //   0 pull      every rank parks its partial matrix locally, owners read the rows from the peers
  //   1 push      the epilogue stores each row into the slot (parity, source rank) of its owner
  //   2 push-all  every rank receives all rows and reduces all of them (one hop, no broadcast)
  int rn_mode;
  long long slot_rows;                // push: rows per (parity, source) slot on a receiver
  // kEpiReduceNorm counts arrivals instead of keeping a flag per tile: ready[r][tm] is a counter
  // on rank r that every rank bumps once per finished column tile of M tile tm; ready_base[tm]
  // (local) is its value before this launch, advanced by the last CTA of the launch
  uint32_t* ready_base;
  // mode 3 ("data carries its own arrival"): no flags and no fences.  The transport buffers
  // hold a sentinel word until real data lands in them; partial[r] / out[r] then point to
  // three rotating buffers of ll_cap elements each on rank r (rows pushed to their owner /
  // finished rows pushed to everyone), the finished rows are copied into ll_out_local, and
  // ll_used[2 * b], ll_used[2 * b + 1] remember how much of buffer b a launch has dirtied
  __nv_bfloat16* ll_out_local;        // [M, ldc] result on this rank
  long long ll_cap;
  long long* ll_used;
  // multicast (NVLS) views of the same symmetric buffers; null = plain peer loads / stores
  const __nv_bfloat16* mc_partial;
  __nv_bfloat16* mc_out;
  __nv_bfloat16* mc_res;
};

// All-gather of the A operand inside the GEMM (sequence-parallel input of a column-parallel
// layer).  Rank r owns rows [row_off[r], row_off[r + 1]) of A; its shard lives in symmetric
// memory.  Four extra warps copy the shards with plain peer loads into the local buffer
// `a_full` (the only memory the TMA descriptor covers) one 128-row chunk at a time and publish
// chunk_ready[chunk]; the TMA warp waits for the chunk before loading it.
struct AgArgs {
  const __nv_bfloat16* shard[kMaxPeers];  // rows of rank r, pitch lds
  __nv_bfloat16* a_full;                  // local [M, lda]
  long long lds, lda;
  uint32_t* in_ready[kMaxPeers];          // [p] on rank r: in_ready[r][src] = src's shard is valid
  uint32_t* rd_done[kMaxPeers];           // [p] on rank r: rd_done[r][reader] = reader is done with r's shard
  uint32_t* chunk_ready;                  // local [tiles_m]
  uint32_t* gather_ctr;                   // local
  int row_off[kMaxPeers + 1];             // first row of every rank's shard; [p] = M
  int enabled;
};

__device__ __forceinline__ int ag_owner(const AgArgs& g, int np, int row) {
  int o = 0;
  while (o + 1 < np && row >= g.row_off[o + 1]) ++o;
  return o;
}

struct Args {
  void* C;
  long long ldc;
  const __nv_bfloat16* bias;
  const __nv_bfloat16* residual;
  long long ldr;
  int M, N, K;
  int tiles_m, tiles_n;
  unsigned int* status;
  // grouped (mixture-of-experts) mode: A rows are sorted by expert in tiles of BM rows
  const int* expert_ids;      // [tiles_m] expert of each M tile (-1: skip), null = dense GEMM
  const int* num_valid_rows;  // device scalar: rows of A that are in use (multiple of BM)
  const float* row_scale;     // optional [M] factor applied to each output row
  int m_rot;                  // M tiles are visited starting at this tile (gathered-A mode)
  int n_fastest;              // 1: consecutive tiles walk along N (tile = tm * tiles_n + tn)
  ArArgs ar;
  AgArgs ag;
};

// Resolves tile -> (m0, n0, first B row).  Returns false for tiles that carry no work.
template <int BN_>
__device__ __forceinline__ bool tile_coords(const Args& p, int tile, int& m0, int& n0,
                                            int& b_row) {
  if (p.n_fastest) {
    // whole rows of the output complete early, in the order their owners reduce them
    m0 = (tile / p.tiles_n) * BM;
    n0 = (tile % p.tiles_n) * BN_;
    b_row = n0;
    return true;
  }
  int tm = tile % p.tiles_m + p.m_rot;
  if (tm >= p.tiles_m) tm -= p.tiles_m;
  m0 = tm * BM;
  n0 = (tile / p.tiles_m) * BN_;
  b_row = n0;
  if (p.expert_ids != nullptr) {
    if (m0 >= *p.num_valid_rows) return false;
    const int e = p.expert_ids[tm];
    if (e < 0) return false;
    b_row = e * p.N + n0;
  }
  return true;
}

// Bounded acquire-wait until *flag reaches `want` (a peer that is one launch ahead may
// already have written want + 1).  Returns false on timeout.
__device__ __forceinline__ bool wait_flag_sys(const uint32_t* flag, uint32_t want,
                                              uint32_t limit = kFlagSpinLimit) {
  for (uint32_t it = 0; it < limit; ++it) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(flag) : "memory");
    if (static_cast<int32_t>(v - want) >= 0) return true;  // epochs only grow
    if (it > 64) __nanosleep(100);
  }
  return false;
}
// Release store at system scope.  The release orders the writes that precede it in this thread
// and, through the barrier that every caller places before it, those of the threads that met
// there (cumulativity); a separate full fence in front of it only doubles the drain.
__device__ __forceinline__ void signal_flag_sys(uint32_t* flag, uint32_t val) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(flag), "r"(val) : "memory");
}
__device__ __forceinline__ uint4 ld_volatile_v4(const void* p) {
  uint4 v;
  asm volatile("ld.volatile.global.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p)
               : "memory");
  return v;
}
__device__ __forceinline__ void epi_bar_sync() { asm volatile("bar.sync 1, 128;" ::: "memory"); }
__device__ __forceinline__ void gather_bar_sync() { asm volatile("bar.sync 2, 128;" ::: "memory"); }
// Bounded acquire-wait at GPU scope on a flag written by another CTA of this kernel.
__device__ __forceinline__ bool wait_flag_gpu(const uint32_t* flag, uint32_t want) {
  for (uint32_t it = 0; it < (1u << 22); ++it) {
    uint32_t v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(flag) : "memory");
    if (static_cast<int32_t>(v - want) >= 0) return true;
    if (it > 64) __nanosleep(100);
  }
  return false;
}

// Sums `np` bf16 tiles (slot r at base + r * stride) into out rows; 8 vectors in flight per
// thread and source so the loads overlap.
template <int BN_>
__device__ __forceinline__ void reduce_tile(const __nv_bfloat16* const* srcs, int np,
                                            long long tile_off, int te, int m0, int n0, int M,
                                            int N, const __nv_bfloat16* residual, long long ldr,
                                            __nv_bfloat16* const* outs, int nout, long long ldc) {
  constexpr int kVecPerRow = BN_ / 8;
  constexpr int kU = 8;
  for (int v0 = te; v0 < BM * kVecPerRow; v0 += 128 * kU) {
    float acc[kU][8];
#pragma unroll
    for (int k = 0; k < kU; ++k)
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[k][i] = 0.0f;
    for (int r = 0; r < np; ++r) {
      uint4 u[kU];
#pragma unroll
      for (int k = 0; k < kU; ++k) {
        const int v = v0 + k * 128;
        u[k] = (v < BM * kVecPerRow) ? ld_volatile_v4(srcs[r] + tile_off + v * 8)
                                     : make_uint4(0, 0, 0, 0);
      }
#pragma unroll
      for (int k = 0; k < kU; ++k) {
        const float2 a = unpack_bf16x2(u[k].x), b = unpack_bf16x2(u[k].y),
                     c2 = unpack_bf16x2(u[k].z), d = unpack_bf16x2(u[k].w);
        acc[k][0] += a.x; acc[k][1] += a.y; acc[k][2] += b.x; acc[k][3] += b.y;
        acc[k][4] += c2.x; acc[k][5] += c2.y; acc[k][6] += d.x; acc[k][7] += d.y;
      }
    }
#pragma unroll
    for (int k = 0; k < kU; ++k) {
      const int v = v0 + k * 128;
      if (v >= BM * kVecPerRow) continue;
      const int row = v / kVecPerRow, cv = v % kVecPerRow;
      const int grow = m0 + row, gcol = n0 + cv * 8;
      if (grow >= M || gcol >= N) continue;
      if (residual != nullptr) {
        const uint4 u = *reinterpret_cast<const uint4*>(residual + static_cast<long long>(grow) * ldr + gcol);
        const float2 a = unpack_bf16x2(u.x), b = unpack_bf16x2(u.y), c2 = unpack_bf16x2(u.z),
                     d = unpack_bf16x2(u.w);
        acc[k][0] += a.x; acc[k][1] += a.y; acc[k][2] += b.x; acc[k][3] += b.y;
        acc[k][4] += c2.x; acc[k][5] += c2.y; acc[k][6] += d.x; acc[k][7] += d.y;
      }
      uint4 o;
      o.x = pack_bf16x2(acc[k][0], acc[k][1]);
      o.y = pack_bf16x2(acc[k][2], acc[k][3]);
      o.z = pack_bf16x2(acc[k][4], acc[k][5]);
      o.w = pack_bf16x2(acc[k][6], acc[k][7]);
      const long long ooff = static_cast<long long>(grow) * ldc + gcol;
      for (int r = 0; r < nout; ++r) *reinterpret_cast<uint4*>(outs[r] + ooff) = o;
    }
  }
}


// ---------------------------------------------------------------------------
// Row-owner reduction (kEpiReduceNorm)
// ---------------------------------------------------------------------------
// In-switch reduction / broadcast through the NVLink multicast view of a symmetric buffer.
__device__ __forceinline__ uint4 mc_ld_reduce_bf16(const void* mc) {
  uint4 v;
  asm volatile(
      "multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0,%1,%2,%3}, [%4];"
      : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
      : "l"(mc)
      : "memory");
  return v;
}
__device__ __forceinline__ void mc_st_v4(void* mc, const uint4& v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1,%2,%3,%4};" ::"l"(mc), "r"(v.x),
               "r"(v.y), "r"(v.z), "r"(v.w)
               : "memory");
}
__device__ __forceinline__ uint32_t ld_relaxed_sys_u32(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.relaxed.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
// Barrier among the 128 threads of warps 6..9 that also ANDs a predicate.
__device__ __forceinline__ bool aux_bar_and(bool pred) {
  uint32_t r;
  asm volatile(
      "{\n\t"
      ".reg .pred P, Q;\n\t"
      "setp.ne.u32 P, %1, 0;\n\t"
      "bar.red.and.pred Q, 2, 128, P;\n\t"
      "selp.b32 %0, 1, 0, Q;\n\t"
      "}\n"
      : "=r"(r)
      : "r"(static_cast<uint32_t>(pred))
      : "memory");
  return r != 0;
}
__device__ __forceinline__ void add8(float (&a)[8], const uint4& u) {
  const float2 x = unpack_bf16x2(u.x), y = unpack_bf16x2(u.y), z = unpack_bf16x2(u.z),
               w = unpack_bf16x2(u.w);
  a[0] += x.x; a[1] += x.y; a[2] += y.x; a[3] += y.y;
  a[4] += z.x; a[5] += z.y; a[6] += w.x; a[7] += w.y;
}
__device__ __forceinline__ uint4 pack8(const float (&a)[8]) {
  uint4 o;
  o.x = pack_bf16x2(a[0], a[1]);
  o.y = pack_bf16x2(a[2], a[3]);
  o.z = pack_bf16x2(a[4], a[5]);
  o.w = pack_bf16x2(a[6], a[7]);
  return o;
}

constexpr int kRnKeep = 8;   // 16-byte chunks of a row one reducer thread holds: N <= 8 * 128 * 8

__device__ __forceinline__ uint32_t ld_acquire_sys_u32(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
// Release store alone: it orders the writes that precede it in this thread and, through a
// barrier before it, those of the threads that met there; no separate full fence.
__device__ __forceinline__ void st_release_sys(uint32_t* flag, uint32_t val) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(flag), "r"(val) : "memory");
}
__device__ __forceinline__ void red_release_sys_add(uint32_t* ctr, uint32_t val) {
  asm volatile("red.release.sys.global.add.u32 [%0], %1;" ::"l"(ctr), "r"(val) : "memory");
}
// Bounded wait until the arrival counter has advanced by `need` beyond `base` (one polling
// thread; peers that are a launch ahead only push it further).
__device__ __forceinline__ bool wait_count_sys(const uint32_t* ctr, uint32_t base, uint32_t need,
                                               uint32_t limit) {
  for (uint32_t it = 0; it < limit; ++it) {
    if (static_cast<int32_t>(ld_acquire_sys_u32(ctr) - base - need) >= 0) return true;
    if (it > 32) __nanosleep(40);
  }
  return false;
}

// One output row, handled by TPR reducer threads (thread `t` of them owns the chunks t,
// t + TPR, ... of the row): all 128 reducer threads of the CTA for decode-sized problems (one
// round trip per row), one warp per row when a rank owns many rows (four rows in flight per
// CTA, no CTA-wide barrier).  Sums the p partial rows (plain peer loads, U chunks x 16 / U
// ranks in flight, or one multimem.ld_reduce per chunk), adds the residual, rounds to bf16
// (the new residual) and - with a norm weight - scales by the RMS statistics of the rounded
// row.  With TPR = 128 the rounded row stays in registers between the two passes (`red`: a
// 4-float shared scratch for the statistics); with TPR = 32 it is read back from the residual
// buffer this thread has just written.
template <int U, int TPR>
__device__ __noinline__ void reduce_norm_row(const ArArgs& ar, int row, int N, long long ldc,
                                                int t, float* red, long long push_off) {
  constexpr bool kKeep = TPR == 128;
  constexpr int kIters = kKeep ? kRnKeep : (kRnKeep * 128 / TPR);
  const int nvec = N >> 3;
  const int np = ar.p, rank = ar.rank;
  const long long roff = static_cast<long long>(row) * N;      // partial / res_out rows: pitch N
  const bool push = ar.rn_mode != 0;
  const int ndst = ar.rn_mode == 2 ? 1 : np;                   // push-all: results stay local
  // source s of this row: pull = rank s's parked matrix, push = slot s of the local buffer
  const long long slot_pitch = ar.slot_rows * static_cast<long long>(N);
  uint4 z[kKeep ? kRnKeep : 1];
  float sumsq = 0.0f;
  const bool have_norm = ar.norm_weight != nullptr;
#pragma unroll
  for (int j0 = 0; j0 < kIters; j0 += U) {
    if (t + j0 * TPR >= nvec) break;
    float acc[U][8];
#pragma unroll
    for (int u = 0; u < U; ++u)
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[u][i] = 0.0f;
    if (ar.mc_partial != nullptr && !push) {
      uint4 v[U];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const int c = t + (j0 + u) * TPR;
        v[u] = c < nvec ? mc_ld_reduce_bf16(ar.mc_partial + roff + c * 8) : make_uint4(0, 0, 0, 0);
      }
#pragma unroll
      for (int u = 0; u < U; ++u) add8(acc[u], v[u]);
    } else {
      constexpr int kR = 8 / U;                  // ranks per batch of loads (8 loads in flight)
      for (int r0 = 0; r0 < np; r0 += kR) {
        uint4 v[kR][U];
#pragma unroll
        for (int r = 0; r < kR; ++r)
#pragma unroll
          for (int u = 0; u < U; ++u) {
            const int c = t + (j0 + u) * TPR;
            const __nv_bfloat16* src =
                push ? ar.partial[rank] + push_off + (r0 + r) * slot_pitch
                     : ar.partial[(r0 + r) < np ? (r0 + r) : 0] + roff;
            v[r][u] = (r0 + r < np && c < nvec) ? ld_volatile_v4(src + c * 8)
                                                : make_uint4(0, 0, 0, 0);
          }
#pragma unroll
        for (int r = 0; r < kR; ++r)
#pragma unroll
          for (int u = 0; u < U; ++u) add8(acc[u], v[r][u]);
      }
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int c = t + (j0 + u) * TPR;
      if (c >= nvec) continue;
      if (ar.res_in != nullptr) {
        const uint4 rv = *reinterpret_cast<const uint4*>(
            ar.res_in + static_cast<long long>(row) * ar.ld_res_in + c * 8);
        add8(acc[u], rv);
      }
      const uint4 o = pack8(acc[u]);
      if constexpr (kKeep) z[j0 + u] = o;
      if (have_norm) {
        // statistics of the rounded values, as an unfused add + RMSNorm would see them
        float f[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        add8(f, o);
#pragma unroll
        for (int i = 0; i < 8; ++i) sumsq += f[i] * f[i];
        // the new residual: every rank, or the owner only
        if (ar.bcast_res && ndst > 1) {
          if (ar.mc_res != nullptr) {
            mc_st_v4(ar.mc_res + roff + c * 8, o);
            if constexpr (!kKeep) *reinterpret_cast<uint4*>(ar.res_out[rank] + roff + c * 8) = o;
          } else {
            for (int r = 0; r < np; ++r)
              *reinterpret_cast<uint4*>(ar.res_out[r] + roff + c * 8) = o;
          }
        } else {
          *reinterpret_cast<uint4*>(ar.res_out[rank] + roff + c * 8) = o;
        }
      } else {
        const long long ooff = static_cast<long long>(row) * ldc + c * 8;
        if (ndst == 1) {
          *reinterpret_cast<uint4*>(ar.out[rank] + ooff) = o;
        } else if (ar.mc_out != nullptr) {
          mc_st_v4(ar.mc_out + ooff, o);
        } else {
          for (int r = 0; r < np; ++r) *reinterpret_cast<uint4*>(ar.out[r] + ooff) = o;
        }
      }
    }
  }
  if (!have_norm) return;
  sumsq = warp_sum(sumsq);
  if constexpr (TPR == 128) {
    if ((t & 31) == 0) red[t >> 5] = sumsq;
    gather_bar_sync();
    sumsq = red[0] + red[1] + red[2] + red[3];
    gather_bar_sync();                           // `red` is reused by the next row
  }
  const float rstd = rsqrtf(sumsq / static_cast<float>(N) + ar.eps);
  constexpr int kB = 4;                          // chunks per batch of the second pass
#pragma unroll
  for (int j0 = 0; j0 < kIters; j0 += kB) {
    if (t + j0 * TPR >= nvec) break;
    uint4 zz[kB], ww[kB];
#pragma unroll
    for (int u = 0; u < kB; ++u) {
      const int c = t + (j0 + u) * TPR;
      if (c >= nvec) continue;
      if constexpr (kKeep) {
        zz[u] = z[j0 + u];
      } else {
        zz[u] = ld_volatile_v4(ar.res_out[rank] + roff + c * 8);   // written by this thread
      }
      ww[u] = *reinterpret_cast<const uint4*>(ar.norm_weight + c * 8);
    }
#pragma unroll
    for (int u = 0; u < kB; ++u) {
      const int c = t + (j0 + u) * TPR;
      if (c >= nvec) continue;
      float f[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      float w[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      add8(f, zz[u]);
      add8(w, ww[u]);
#pragma unroll
      for (int i = 0; i < 8; ++i) f[i] = f[i] * rstd * w[i];
      const uint4 o = pack8(f);
      const long long ooff = static_cast<long long>(row) * ldc + c * 8;
      if (ndst == 1) {
        *reinterpret_cast<uint4*>(ar.out[rank] + ooff) = o;
      } else if (ar.mc_out != nullptr) {
        mc_st_v4(ar.mc_out + ooff, o);
      } else {
        for (int r = 0; r < np; ++r) *reinterpret_cast<uint4*>(ar.out[r] + ooff) = o;
      }
    }
  }
}


// ---- mode 3: sentinel-tagged transport -----------------------------------------------------
// A 32-bit word of two bf16 negative zeros marks "not written yet"; writers turn that one bit
// pattern into two positive zeros, so real data never looks like the sentinel.  Every 32-bit
// word is checked on the receiving side: stores of aligned 32-bit words are never torn.
constexpr uint32_t kLLSentinel = 0x80008000u;
__device__ __forceinline__ uint4 ll_sanitize(uint4 v) {
  v.x = v.x == kLLSentinel ? 0u : v.x;
  v.y = v.y == kLLSentinel ? 0u : v.y;
  v.z = v.z == kLLSentinel ? 0u : v.z;
  v.w = v.w == kLLSentinel ? 0u : v.w;
  return v;
}
__device__ __forceinline__ bool ll_valid(const uint4& v) {
  return v.x != kLLSentinel && v.y != kLLSentinel && v.z != kLLSentinel && v.w != kLLSentinel;
}
__device__ __forceinline__ void st_volatile_v4(void* p, const uint4& v) {
  asm volatile("st.volatile.global.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x), "r"(v.y),
               "r"(v.z), "r"(v.w)
               : "memory");
}

// One owned row in mode 3, all 128 reducer threads on it.  `src` = first source slot of the
// row in the local receive buffer (slot s at src + s * slot_pitch), `dst_off` = offset of the
// row in every rank's result transport buffer.  Returns false if a wait ran out.
template <int U>
__device__ __noinline__ bool ll_reduce_row(const ArArgs& ar, const __nv_bfloat16* src,
                                           long long slot_pitch, long long buf_off, int row,
                                           int N, int te, float* red, uint32_t spin) {
  const int nvec = N >> 3;
  const int np = ar.p, rank = ar.rank;
  const long long roff = static_cast<long long>(row) * N;
  uint4 z[kRnKeep];
  float sumsq = 0.0f;
  bool alive = true;
  const bool have_norm = ar.norm_weight != nullptr;
  constexpr int kR = 8 / U;
  // what does not depend on the peers is fetched before the wait: the residual and the norm
  // weights of this thread's first chunks
  constexpr int kPf = 4;
  uint4 res_pf[kPf], w_pf[kPf];
#pragma unroll
  for (int j = 0; j < kPf; ++j) {
    const int c = te + j * 128;
    res_pf[j] = (ar.res_in != nullptr && c < nvec)
                    ? *reinterpret_cast<const uint4*>(
                          ar.res_in + static_cast<long long>(row) * ar.ld_res_in + c * 8)
                    : make_uint4(0, 0, 0, 0);
    w_pf[j] = (have_norm && c < nvec) ? *reinterpret_cast<const uint4*>(ar.norm_weight + c * 8)
                                      : make_uint4(0, 0, 0, 0);
  }
#pragma unroll
  for (int j0 = 0; j0 < kRnKeep; j0 += U) {
    if (te + j0 * 128 >= nvec) break;
    float acc[U][8];
#pragma unroll
    for (int u = 0; u < U; ++u)
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[u][i] = 0.0f;
    for (int r0 = 0; r0 < np; r0 += kR) {
      uint4 v[kR][U];
      bool ok = false;
      for (uint32_t it = 0; it < spin && !ok; ++it) {
        ok = true;
#pragma unroll
        for (int r = 0; r < kR; ++r)
#pragma unroll
          for (int u = 0; u < U; ++u) {
            const int c = te + (j0 + u) * 128;
            const bool in = r0 + r < np && c < nvec;
            v[r][u] = in ? ld_volatile_v4(src + (r0 + r) * slot_pitch + c * 8)
                         : make_uint4(0, 0, 0, 0);
          }
#pragma unroll
        for (int r = 0; r < kR; ++r)
#pragma unroll
          for (int u = 0; u < U; ++u) ok = ok && ll_valid(v[r][u]);
        if (!ok && it > 8) __nanosleep(20);
      }
      alive = alive && ok;
#pragma unroll
      for (int r = 0; r < kR; ++r)
#pragma unroll
        for (int u = 0; u < U; ++u) add8(acc[u], v[r][u]);
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int c = te + (j0 + u) * 128;
      if (c >= nvec) continue;
      if (j0 + u < kPf) {
        add8(acc[u], res_pf[j0 + u]);            // zeros when there is no residual
      } else if (ar.res_in != nullptr) {
        add8(acc[u], *reinterpret_cast<const uint4*>(
                         ar.res_in + static_cast<long long>(row) * ar.ld_res_in + c * 8));
      }
      const uint4 o = pack8(acc[u]);
      z[j0 + u] = o;
      if (have_norm) {
        float f[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        add8(f, o);
#pragma unroll
        for (int i = 0; i < 8; ++i) sumsq += f[i] * f[i];
        *reinterpret_cast<uint4*>(ar.res_out[rank] + roff + c * 8) = o;   // owner keeps the residual
      }
    }
  }
  float rstd = 1.0f;
  if (have_norm) {
    sumsq = warp_sum(sumsq);
    if ((te & 31) == 0) red[te >> 5] = sumsq;
    gather_bar_sync();
    sumsq = red[0] + red[1] + red[2] + red[3];
    gather_bar_sync();
    rstd = rsqrtf(sumsq / static_cast<float>(N) + ar.eps);
  }
#pragma unroll
  for (int j = 0; j < kRnKeep; ++j) {
    const int c = te + j * 128;
    if (c >= nvec) break;
    uint4 o = z[j];
    if (have_norm) {
      float f[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      float w[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      add8(f, o);
      add8(w, j < kPf ? w_pf[j] : *reinterpret_cast<const uint4*>(ar.norm_weight + c * 8));
#pragma unroll
      for (int i = 0; i < 8; ++i) f[i] = f[i] * rstd * w[i];
      o = pack8(f);
    }
    o = ll_sanitize(o);
    for (int r = 0; r < np; ++r) st_volatile_v4(ar.out[r] + buf_off + roff + c * 8, o);
  }
  return alive;
}

template <int BN, int STAGES, int EPI = kEpiNone>
struct Smem {
  static constexpr int kABytes = BM * BK * 2;
  static constexpr int kBBytes = BN * BK * 2;
  static constexpr int kStageBytes = kABytes + kBBytes;
  // epilogues that store into peer memory stage the bf16 tile here so that the peer stores
  // are full, contiguous 128-byte lines instead of one 16-byte piece per row
  static constexpr int kOutOffset = STAGES * kStageBytes;
  static constexpr int kOutCols = BN < 128 ? BN : 128;   // columns staged per pass
  static constexpr int kOutBytes =
      (EPI == kEpiAllReduce || EPI == kEpiAllGather || EPI == kEpiReduceNorm)
          ? BM * kOutCols * 2
          : 0;
  static constexpr int kBarOffset = kOutOffset + kOutBytes;
  static constexpr int kArBytes = EPI == kEpiReduceNorm ? 640 : 0;   // shared copy of ArArgs
  static constexpr int kTotal = kBarOffset + 256 + kArBytes + 1024;  // barriers + alignment slack
  static_assert(kTotal <= 232448, "exceeds the shared memory of one CTA");
};

// Shared staging tile [BM][BN] bf16; the 16-byte chunk index of a row is XORed with the low
// three bits of the row, so row-per-lane writes and flat reads are both conflict free.
template <int BN_>
__device__ __forceinline__ uint32_t stage_off(int row, int chunk) {
  return static_cast<uint32_t>(row * (BN_ * 2) + ((chunk ^ (row & 7)) << 4));
}
// Moves BN_ columns of this thread's accumulator row (32 TMEM columns per step, starting at
// taddr) into the staging tile.
template <int BN_>
__device__ __forceinline__ void stage_tile(uint8_t* stage, uint32_t taddr, int row) {
#pragma unroll 1
  for (int c = 0; c < BN_ / 32; ++c) {
    uint32_t r[32];
    tmem_ld_32x32(taddr + c * 32, r);
    tmem_ld_wait();
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      uint4 u;
      u.x = pack_bf16x2(__uint_as_float(r[i * 8 + 0]), __uint_as_float(r[i * 8 + 1]));
      u.y = pack_bf16x2(__uint_as_float(r[i * 8 + 2]), __uint_as_float(r[i * 8 + 3]));
      u.z = pack_bf16x2(__uint_as_float(r[i * 8 + 4]), __uint_as_float(r[i * 8 + 5]));
      u.w = pack_bf16x2(__uint_as_float(r[i * 8 + 6]), __uint_as_float(r[i * 8 + 7]));
      *reinterpret_cast<uint4*>(stage + stage_off<BN_>(row, c * 4 + i)) = u;
    }
  }
}

// Stores 32 consecutive output columns of one row (values in v[0..31]).
__device__ __forceinline__ void store_row_bf16(__nv_bfloat16* dst, const float* v, int ncols) {
  if (ncols >= 32) {
    uint4* d4 = reinterpret_cast<uint4*>(dst);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      uint4 u;
      u.x = pack_bf16x2(v[i * 8 + 0], v[i * 8 + 1]);
      u.y = pack_bf16x2(v[i * 8 + 2], v[i * 8 + 3]);
      u.z = pack_bf16x2(v[i * 8 + 4], v[i * 8 + 5]);
      u.w = pack_bf16x2(v[i * 8 + 6], v[i * 8 + 7]);
      d4[i] = u;
    }
  } else {
    for (int i = 0; i < ncols; ++i) dst[i] = __float2bfloat16(v[i]);
  }
}

template <int BN, int STAGES, int EPI>
__global__ void __launch_bounds__(kThreadsFor<EPI>, 1)
    gemm_bf16_kernel(const __grid_constant__ CUtensorMap tmA,
                     const __grid_constant__ CUtensorMap tmB, const Args p) {
  using L = Smem<BN, STAGES, EPI>;
  constexpr uint32_t kTmemCols = 2 * BN <= 128 ? 128 : (2 * BN <= 256 ? 256 : 512);
  constexpr uint32_t kIdesc = make_idesc(BM, BN, 1, 1);

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + L::kBarOffset);
  uint64_t* empty_bar = full_bar + STAGES;
  uint64_t* tfull_bar = empty_bar + STAGES;
  uint64_t* tempty_bar = tfull_bar + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty_bar + 2);
  volatile uint32_t* abort_flag = tmem_slot + 1;
  // written by warps 6..9 only (before their named barrier) and read after it, so that all of
  // them leave their loops in the same iteration
  volatile uint32_t* aux_abort = tmem_slot + 2;
  float* aux_red = reinterpret_cast<float*>(tmem_slot + 4);   // 4 floats of the reducer warps
  // copy of the peer-address block for the out-of-line row functions of the reducer warps
  // (taking the address of the kernel parameter itself would move all of it to local memory)
  ArArgs* ar_s = reinterpret_cast<ArArgs*>(smem + L::kBarOffset + 256);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

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
    *aux_abort = 0u;
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
  uint32_t epoch = 0;
  if constexpr (kPeerEpi<EPI>)
    epoch = *reinterpret_cast<volatile uint32_t*>(p.ar.epoch_ptr) + 1u;

  if (warp == 0) {
    // ---------------- TMA producer ----------------
    if (elect_one()) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; ok && tile < num_tiles; tile += gridDim.x) {
        int m0, n0, b_row;
        if (!tile_coords<BN>(p, tile, m0, n0, b_row)) continue;
        if constexpr (EPI == kEpiGatherA) {
          // rows of this M tile must have been copied into the local buffer (generic-proxy
          // stores by the gather warps of some CTA) before the async proxy reads them
          if (!wait_flag_gpu(p.ag.chunk_ready + m0 / BM, epoch)) {
            report_status(p.status, kStatusFlagTimeout, kKernelId, 0x700u);
            *abort_flag = 1u;
            break;
          }
          asm volatile("fence.proxy.async;" ::: "memory");
        }
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(&empty_bar[stage], phase ^ 1u, p.status, kKernelId, 0x100u + stage,
                         abort_flag)) {
            ok = false;
            break;
          }
          uint8_t* sa = smem + stage * L::kStageBytes;
          uint8_t* sb = sa + L::kABytes;
          mbar_expect_tx(&full_bar[stage], L::kStageBytes);
          tma_load_2d(sa, &tmA, &full_bar[stage], kb * BK, m0);
          tma_load_2d(sb, &tmB, &full_bar[stage], kb * BK, b_row);
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    if (elect_one()) {
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; ok && tile < num_tiles; tile += gridDim.x) {
        {
          int m0s, n0s, brs;
          if (!tile_coords<BN>(p, tile, m0s, n0s, brs)) continue;
        }
        if (!mbar_wait(&tempty_bar[acc], acc_phase ^ 1u, p.status, kKernelId, 0x200u + acc,
                       abort_flag))
          break;
        tc_fence_after();
        const uint32_t tmem_d = tmem_base + static_cast<uint32_t>(acc * BN);
        for (int kb = 0; kb < num_kb; ++kb) {
          if (!mbar_wait(&full_bar[stage], phase, p.status, kKernelId, 0x300u + stage,
                         abort_flag)) {
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t a_addr = smem_u32(smem + stage * L::kStageBytes);
          const uint32_t b_addr = a_addr + L::kABytes;
          const uint64_t adesc = make_desc_k_sw128(a_addr);
          const uint64_t bdesc = make_desc_k_sw128(b_addr);
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            // 16 bf16 along K = 32 bytes = 2 descriptor address units
            umma_f16(tmem_d, adesc + static_cast<uint64_t>(k * 2),
                     bdesc + static_cast<uint64_t>(k * 2), kIdesc, (kb | k) != 0 ? 1u : 0u);
          }
          umma_commit(&empty_bar[stage]);
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (!ok) break;
        umma_commit(&tfull_bar[acc]);
        acc ^= 1;
        if (acc == 0) acc_phase ^= 1u;
      }
    }
  } else if (warp >= 6) {
    if constexpr (EPI == kEpiAllReduce) {
      // ---------------- reducers (warps 6..9): run while the tensor cores work on later tiles

      const int te = threadIdx.x - 192;  // 0..127 among the reducer warps
      const int np = p.ar.p, rank = p.ar.rank;
      const uint32_t spin = flag_spin_limit(p.status);
      if (p.ar.oneshot) {
        // phase 2 (one-shot): every rank reduces every tile from its own slots
        const __nv_bfloat16* srcs[kMaxPeers];
        for (int r = 0; r < kMaxPeers; ++r)
          srcs[r] = p.ar.partial[rank] +
                    (static_cast<long long>(epoch & 1u) * np + (r < np ? r : 0)) * p.ar.slot_elems;
        __nv_bfloat16* outs[1] = {p.ar.out[rank]};
        for (int t = blockIdx.x; t < num_tiles; t += gridDim.x) {
          bool ok = true;
          if (te < np)
            ok = wait_flag_sys(p.ar.ready[rank] + static_cast<long long>(t) * np + te, epoch, spin);
          if (!ok) {
            report_status(p.status, kStatusFlagTimeout, kKernelId, 0x500u + te);
            *aux_abort = 1u;
          }
          gather_bar_sync();
          if (*aux_abort != 0u) break;
          reduce_tile<BN>(srcs, np, static_cast<long long>(t) * (BM * BN), te,
                          (t % p.tiles_m) * BM, (t / p.tiles_m) * BN, p.M, p.N, p.residual, p.ldr,
                          outs, 1, p.ldc);
        }
      } else {
        // phase 2 (two-shot): reduce the tiles this rank owns (tile % p == rank), broadcast
        for (int t = rank + static_cast<int>(blockIdx.x) * np; t < num_tiles;
             t += gridDim.x * np) {
          bool ok = true;
          if (te < np)
            ok = wait_flag_sys(p.ar.ready[rank] + static_cast<long long>(t) * np + te, epoch, spin);
          if (!ok) {
            report_status(p.status, kStatusFlagTimeout, kKernelId, 0x500u + te);
            *aux_abort = 1u;
          }
          gather_bar_sync();
          if (*aux_abort != 0u) break;
          reduce_tile<BN>(p.ar.partial, np, static_cast<long long>(t) * (BM * BN), te,
                          (t % p.tiles_m) * BM, (t / p.tiles_m) * BN, p.M, p.N, p.residual, p.ldr,
                          p.ar.out, np, p.ldc);
          gather_bar_sync();
          if (te < np) signal_flag_sys(p.ar.done[te] + t, epoch);
        }
        // phase 3: the result is complete on this rank once every tile reports done
        for (int t = te; t < num_tiles && *aux_abort == 0u; t += 128) {
          if (!wait_flag_sys(p.ar.done[rank] + t, epoch, spin)) {
            report_status(p.status, kStatusFlagTimeout, kKernelId, 0x600u);
            *aux_abort = 1u;
          }
        }
      }
    }
    if constexpr (EPI == kEpiReduceNorm) {
      // ---------------- row owners (warps 6..9) ----------------
      // Rank r owns rows [lo, hi) of every 128-row tile (push-all mode: every rank owns all
      // rows).  A row is reduced once every rank has delivered all column tiles of its M tile;
      // the finished row is stored into every rank and marked done there.  Few rows per rank
      // (decode): one row at a time per CTA, all 128 threads on it.  Many rows: one row per
      // warp, four rows in flight per CTA; the done flags of a group of rows go out with one
      // release, so the drain of the remote stores is paid once per group.
      const int te = threadIdx.x - 192;
      const int wq = te >> 5, ln = te & 31;
      const int np = p.ar.p, rank = p.ar.rank;
      const uint32_t spin = flag_spin_limit(p.status);
      static_assert(sizeof(ArArgs) <= 640 && sizeof(ArArgs) % 4 == 0, "shared copy of ArArgs");
      for (int w = te; w < static_cast<int>(sizeof(ArArgs) / 4); w += 128)
        reinterpret_cast<uint32_t*>(ar_s)[w] = reinterpret_cast<const uint32_t*>(&p.ar)[w];
      gather_bar_sync();
      const ArArgs& ars = *ar_s;
      const bool all_own = p.ar.rn_mode == 2;
      const int lo = all_own ? 0 : BM * rank / np, hi = all_own ? BM : BM * (rank + 1) / np;
      const int rpt = hi - lo;
      const int nflags = p.tiles_n * np;
      const int my_rows = p.tiles_m * rpt;
      const long long par_off =
          static_cast<long long>(epoch & 1u) * np * p.ar.slot_rows * static_cast<long long>(p.N);
      int tm_ready = -1;                               // last M tile whose flags were seen
      bool dead = false;
      if (p.ar.rn_mode == 3) {
        // sentinel-tagged transport: no flag, no fence; every thread waits for its own data
        const long long buf_off = static_cast<long long>(epoch % 3u) * p.ar.ll_cap;
        const long long slot_pitch = p.ar.slot_rows * static_cast<long long>(p.N);
        for (int i = blockIdx.x; i < my_rows; i += gridDim.x) {
          const int tm = i / rpt;
          const int row = tm * BM + lo + (i - tm * rpt);
          if (row >= p.M) continue;
          const __nv_bfloat16* src =
              p.ar.partial[rank] + buf_off + static_cast<long long>(i) * p.N;
          const bool ok = np > 4 ? ll_reduce_row<2>(ars, src, slot_pitch, buf_off, row, p.N, te,
                                                    aux_red, spin)
                                 : ll_reduce_row<4>(ars, src, slot_pitch, buf_off, row, p.N, te,
                                                    aux_red, spin);
          if (!aux_bar_and(ok)) {
            if (te == 0) report_status(p.status, kStatusFlagTimeout, kKernelId, 0x920u);
            dead = true;
            break;
          }
        }
        // collect the finished rows (from every owner) out of the transport buffer
        const int nvec = p.N >> 3;
        for (int r = blockIdx.x; !dead && r < p.M; r += gridDim.x) {
          const __nv_bfloat16* srow = p.ar.out[rank] + buf_off + static_cast<long long>(r) * p.N;
          bool ok_all = true;
          for (int c0 = te; c0 < nvec; c0 += 128 * 4) {
            uint4 v[4];
            bool ok = false;
            for (uint32_t it = 0; it < spin && !ok; ++it) {
              ok = true;
#pragma unroll
              for (int u = 0; u < 4; ++u) {
                const int c = c0 + u * 128;
                v[u] = c < nvec ? ld_volatile_v4(srow + c * 8) : make_uint4(0, 0, 0, 0);
                ok = ok && ll_valid(v[u]);
              }
              if (!ok && it > 8) __nanosleep(20);
            }
            ok_all = ok_all && ok;
#pragma unroll
            for (int u = 0; u < 4; ++u) {
              const int c = c0 + u * 128;
              if (c < nvec)
                *reinterpret_cast<uint4*>(p.ar.ll_out_local +
                                          static_cast<long long>(r) * p.ldc + c * 8) = v[u];
            }
          }
          if (!ok_all) {
            report_status(p.status, kStatusFlagTimeout, kKernelId, 0x921u);
            break;
          }
        }
      } else if (min(my_rows, p.M) <= static_cast<int>(gridDim.x) * 2) {
        int done_rows[2] = {-1, -1};
        int nd = 0;
        auto flush_cta = [&]() {
          gather_bar_sync();                           // every thread's stores precede the release
          if (!all_own && te < nd * np)
            st_release_sys(p.ar.done[te % np] + done_rows[te / np], epoch);
          nd = 0;
        };
        for (int i = blockIdx.x; i < my_rows; i += gridDim.x) {
          const int tm = i / rpt;
          const int row = tm * BM + lo + (i - tm * rpt);
          if (row >= p.M) continue;
          if (tm != tm_ready) {
            // one thread polls the arrival counter of this M tile; the barrier hands its
            // verdict (and, by cumulativity, its acquire) to the other 127
            bool ok = true;
            if (te == 0)
              ok = wait_count_sys(p.ar.ready[rank] + tm, p.ar.ready_base[tm], nflags, spin);
            const bool all = aux_bar_and(ok);
            if (!all) {
              if (te == 0) report_status(p.status, kStatusFlagTimeout, kKernelId, 0x900u);
              dead = true;
              break;                                   // the same decision in all 128 threads
            }
            tm_ready = tm;
          }
          const long long push_off = par_off + static_cast<long long>(i) * p.N;
          if (np > 4)
            reduce_norm_row<2, 128>(ars, row, p.N, p.ldc, te, aux_red, push_off);
          else
            reduce_norm_row<4, 128>(ars, row, p.N, p.ldc, te, aux_red, push_off);
          if (nd == 0) done_rows[0] = row; else done_rows[1] = row;
          if (++nd == 2) flush_cta();
        }
        if (!dead && nd > 0) flush_cta();
      } else {
        const int group = 32 / np;                     // rows whose flags one release covers
        int grow_[16];
        int ng = 0;
        auto flush = [&]() {
          __syncwarp();
          if (!all_own && ln < ng * np) st_release_sys(p.ar.done[ln % np] + grow_[ln / np], epoch);
          __syncwarp();
          ng = 0;
        };
        for (int i = static_cast<int>(blockIdx.x) * 4 + wq; i < my_rows; i += gridDim.x * 4) {
          const int tm = i / rpt;
          const int row = tm * BM + lo + (i - tm * rpt);
          if (row >= p.M) continue;
          if (tm != tm_ready) {
            bool ok = true;
            if (ln == 0)
              ok = wait_count_sys(p.ar.ready[rank] + tm, p.ar.ready_base[tm], nflags, spin);
            const bool all = __all_sync(0xffffffffu, ok);
            if (!all) {
              if (ln == 0) report_status(p.status, kStatusFlagTimeout, kKernelId, 0x901u);
              dead = true;
              break;
            }
            tm_ready = tm;
          }
          const long long push_off = par_off + static_cast<long long>(i) * p.N;
          if (np > 4)
            reduce_norm_row<2, 32>(ars, row, p.N, p.ldc, ln, aux_red, push_off);
          else
            reduce_norm_row<4, 32>(ars, row, p.N, p.ldc, ln, aux_red, push_off);
          // grow_ is indexed with a loop-carried count: keep it in registers by unrolling
#pragma unroll
          for (int k = 0; k < 16; ++k)
            if (k == ng) grow_[k] = row;
          if (++ng == group) flush();
        }
        if (!dead && ng > 0) flush();
      }
      // the output is complete here once the owner of every row has marked it
      for (int r = static_cast<int>(blockIdx.x) * 128 + te;
           p.ar.rn_mode != 3 && !all_own && !dead && r < p.M; r += gridDim.x * 128) {
        if (!wait_flag_sys(p.ar.done[rank] + r, epoch, spin)) {
          report_status(p.status, kStatusFlagTimeout, kKernelId, 0x910u);
          break;
        }
      }
    }
    // ---------------- A gather (warps 6..9, gathered-A variant only) ----------------
    if constexpr (EPI == kEpiGatherA) {
      const int tg = threadIdx.x - 192;  // 0..127
      const int np = p.ar.p, rank = p.ar.rank;
      if (blockIdx.x == 0 && tg < np)    // this rank's shard was written before the launch
        signal_flag_sys(p.ag.in_ready[tg] + rank, epoch);
      const int kvec = p.K / 8;
      bool ok = true;
      for (int c = blockIdx.x; ok && c < p.tiles_m; c += gridDim.x) {
        int tm = c + p.m_rot;
        if (tm >= p.tiles_m) tm -= p.tiles_m;
        const int r0 = tm * BM, r1 = min(p.M, r0 + BM);
        const int o0 = ag_owner(p.ag, np, r0), o1 = ag_owner(p.ag, np, r1 - 1);
        if (tg >= o0 && tg <= o1 && tg != rank) {
          if (!wait_flag_sys(p.ag.in_ready[rank] + tg, epoch)) {
            report_status(p.status, kStatusFlagTimeout, kKernelId, 0x710u + tg);
            *aux_abort = 1u;
          }
        }
        gather_bar_sync();
        if (*aux_abort != 0u) break;
        const int nvec = (r1 - r0) * kvec;
        constexpr int kU = 8;
        for (int v0 = tg; v0 < nvec; v0 += 128 * kU) {
          uint4 u[kU];
#pragma unroll
          for (int k = 0; k < kU; ++k) {
            const int v = v0 + k * 128;
            if (v < nvec) {
              const int row = r0 + v / kvec, cv = v % kvec;
              const int owner = ag_owner(p.ag, np, row);
              u[k] = ld_volatile_v4(p.ag.shard[owner] +
                                    static_cast<long long>(row - p.ag.row_off[owner]) * p.ag.lds +
                                    cv * 8);
            }
          }
#pragma unroll
          for (int k = 0; k < kU; ++k) {
            const int v = v0 + k * 128;
            if (v < nvec) {
              const int row = r0 + v / kvec, cv = v % kvec;
              *reinterpret_cast<uint4*>(p.ag.a_full + static_cast<long long>(row) * p.ag.lda +
                                        cv * 8) = u[k];
            }
          }
        }
        asm volatile("fence.proxy.async;" ::: "memory");
        __threadfence();
        gather_bar_sync();
        if (tg == 0)
          asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(p.ag.chunk_ready + tm),
                       "r"(epoch)
                       : "memory");
      }
      gather_bar_sync();
      if (tg == 0) {
        // the last CTA to finish its chunks tells every owner that this rank is done reading
        __threadfence();
        if (atomicAdd(p.ag.gather_ctr, 1u) == gridDim.x - 1) {
          *p.ag.gather_ctr = 0u;
          for (int r = 0; r < np; ++r) signal_flag_sys(p.ag.rd_done[r] + rank, epoch);
        }
      }
      // the shard may be overwritten after this kernel: wait until every reader is done
      if (blockIdx.x == 0 && tg < np && *aux_abort == 0u) {
        if (!wait_flag_sys(p.ag.rd_done[rank] + tg, epoch))
          report_status(p.status, kStatusFlagTimeout, kKernelId, 0x720u + tg);
      }
    }
  } else {
    // ---------------- epilogue (warps 2..5) ----------------
    const int q = warp & 3;  // TMEM lane quarter this warp may read
    int acc = 0;
    uint32_t acc_phase = 0;
    if constexpr (EPI == kEpiReduceNorm) {
      if (p.ar.rn_mode == 3) {
        // While the tensor cores work on the first tile: put the sentinel back into the
        // transport buffers that the launch after the next one will use.  They were last
        // written two launches ago, and every word written then has been read since.
        const int te0 = threadIdx.x - 64;
        const uint32_t b = epoch % 3u, c = (epoch + 2u) % 3u;
        const uint4 sent = make_uint4(kLLSentinel, kLLSentinel, kLLSentinel, kLLSentinel);
        const long long n0 = p.ar.ll_used[2 * c] >> 3, n1 = p.ar.ll_used[2 * c + 1] >> 3;
        uint4* s0 = reinterpret_cast<uint4*>(p.ar.partial[p.ar.rank] + c * p.ar.ll_cap);
        uint4* s1 = reinterpret_cast<uint4*>(p.ar.out[p.ar.rank] + c * p.ar.ll_cap);
        const long long stride = static_cast<long long>(gridDim.x) * 128;
        for (long long v = static_cast<long long>(blockIdx.x) * 128 + te0; v < n0; v += stride)
          s0[v] = sent;
        for (long long v = static_cast<long long>(blockIdx.x) * 128 + te0; v < n1; v += stride)
          s1[v] = sent;
        if (blockIdx.x == 0 && te0 == 0) {
          p.ar.ll_used[2 * b] = static_cast<long long>(p.ar.p) * p.ar.slot_rows * p.N;
          p.ar.ll_used[2 * b + 1] = static_cast<long long>(p.M) * p.N;
        }
      }
    }
    if constexpr (EPI == kEpiAllGather) {
      // A peer's output buffer may be overwritten once that peer has started this launch
      // (its stream is then past the consumers of the previous result).
      const int te0 = threadIdx.x - 64;
      if (blockIdx.x == 0 && te0 < p.ar.p) signal_flag_sys(p.ar.done[te0] + p.ar.rank, epoch);
      if (te0 < p.ar.p && !wait_flag_sys(p.ar.done[p.ar.rank] + te0, epoch)) {
        report_status(p.status, kStatusFlagTimeout, kKernelId, 0x810u + te0);
        *abort_flag = 1u;
      }
      epi_bar_sync();
    }
    for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x) {
      int m0, n0, b_row_unused;
      if (!tile_coords<BN>(p, tile, m0, n0, b_row_unused)) continue;
      if (!mbar_wait(&tfull_bar[acc], acc_phase, p.status, kKernelId, 0x400u + acc, abort_flag))
        break;
      tc_fence_after();
      const int row = m0 + q * 32 + lane;
      const bool row_ok = row < p.M;
      const uint32_t taddr =
          tmem_base + (static_cast<uint32_t>(q * 32) << 16) + static_cast<uint32_t>(acc * BN);

      if constexpr (EPI == kEpiSiluMul) {
        // every 64-column group of the tile = 32 gate columns, then the 32 matching up columns
        static_assert(EPI != kEpiSiluMul || BN % 64 == 0, "SiLU-mul epilogue: 64-column groups");
        const int out_n0 = (n0 >> 1);
        const int out_n = p.N >> 1;
        __nv_bfloat16* crow =
            reinterpret_cast<__nv_bfloat16*>(p.C) + static_cast<long long>(row) * p.ldc;
#pragma unroll 1
        for (int c = 0; c < BN / 64; ++c) {
          uint32_t g[32], u[32];
          tmem_ld_32x32(taddr + c * 64, g);
          tmem_ld_32x32(taddr + c * 64 + 32, u);
          tmem_ld_wait();
          float v[32];
#pragma unroll
          for (int i = 0; i < 32; ++i)
            v[i] = silu_f(__uint_as_float(g[i])) * __uint_as_float(u[i]);
          const int col = out_n0 + c * 32;
          if (row_ok && col < out_n) store_row_bf16(crow + col, v, min(32, out_n - col));
        }
      } else if constexpr (EPI == kEpiAllReduce) {
        // phase 1: publish the bf16 partial tile.  Two-shot: park it in this GPU's own
        // symmetric buffer and tell the tile's owner.  One-shot: push it into the slot
        // (epoch parity, this rank) of every peer and tell every peer.  The tile goes
        // through the staging buffer so that every store instruction of a warp covers 512
        // contiguous bytes of the (contiguous) tile in the destination.
        uint8_t* stage = smem + L::kOutOffset;
        constexpr int SC = L::kOutCols;            // staged columns per pass
        constexpr int kChunksPerRow = SC / 8;
        const int te1 = threadIdx.x - 64;
        const long long tile_elems = static_cast<long long>(tile) * (BM * BN);
        const long long slot_off =
            p.ar.oneshot ? (static_cast<long long>(epoch & 1u) * p.ar.p + p.ar.rank) * p.ar.slot_elems
                         : 0;
#pragma unroll 1
        for (int h = 0; h < BN / SC; ++h) {
          stage_tile<SC>(stage, taddr + h * SC, q * 32 + lane);
          if (h == BN / SC - 1) {
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&tempty_bar[acc]);   // the accumulator is free again
          }
          epi_bar_sync();
#pragma unroll 2
          for (int v = te1; v < BM * kChunksPerRow; v += 128) {
            const int rr = v / kChunksPerRow, cc = v % kChunksPerRow;
            const uint4 u = *reinterpret_cast<const uint4*>(stage + stage_off<SC>(rr, cc));
            const long long off = tile_elems + rr * BN + h * SC + cc * 8;
            if (p.ar.oneshot) {
              for (int pr = 0; pr < p.ar.p; ++pr)
                *reinterpret_cast<uint4*>(p.ar.partial[pr] + slot_off + off) = u;
            } else {
              *reinterpret_cast<uint4*>(p.ar.partial[p.ar.rank] + off) = u;
            }
          }
          epi_bar_sync();
        }
        if (p.ar.oneshot) {
          if (te1 < p.ar.p)
            signal_flag_sys(p.ar.ready[te1] + static_cast<long long>(tile) * p.ar.p + p.ar.rank,
                            epoch);
        } else if (te1 == 0) {
          const int owner = tile % p.ar.p;
          signal_flag_sys(p.ar.ready[owner] + static_cast<long long>(tile) * p.ar.p + p.ar.rank,
                          epoch);
        }
      } else if constexpr (EPI == kEpiReduceNorm) {
        // deliver the bf16 partial tile as rows of the [M, N] matrix (the owners read whole
        // rows): pull mode parks it in this GPU's own symmetric buffer; the push modes store
        // every row into the slot (epoch parity, this rank) of its owner / of every rank.
        // Then tell every rank: each of them owns rows of this M tile.
        uint8_t* stage = smem + L::kOutOffset;
        constexpr int SC = L::kOutCols;
        constexpr int kChunksPerRow = SC / 8;
        const int te1 = threadIdx.x - 64;
        const int np = p.ar.p, rank = p.ar.rank;
        const int mode = p.ar.rn_mode;
        const int tm = m0 / BM;
        const int rpt = mode == 2 ? BM : BM / np;          // push modes need 128 % p == 0
        const long long slot_base =
            mode == 3 ? static_cast<long long>(rank) * p.ar.slot_rows
                      : (static_cast<long long>(epoch & 1u) * np + rank) * p.ar.slot_rows;
        const long long ll_off = static_cast<long long>(epoch % 3u) * p.ar.ll_cap;
#pragma unroll 1
        for (int h = 0; h < BN / SC; ++h) {
          stage_tile<SC>(stage, taddr + h * SC, q * 32 + lane);
          if (h == BN / SC - 1) {
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&tempty_bar[acc]);
          }
          epi_bar_sync();
#pragma unroll 2
          for (int v = te1; v < BM * kChunksPerRow; v += 128) {
            const int rr = v / kChunksPerRow, cc = v % kChunksPerRow;
            const int grow = m0 + rr, gcol = n0 + h * SC + cc * 8;
            if (grow >= p.M || gcol >= p.N) continue;
            const uint4 u = *reinterpret_cast<const uint4*>(stage + stage_off<SC>(rr, cc));
            if (mode == 0) {
              *reinterpret_cast<uint4*>(p.ar.partial[rank] +
                                        static_cast<long long>(grow) * p.N + gcol) = u;
            } else if (mode == 1) {
              const int o = rr / rpt;
              const long long ro = slot_base + static_cast<long long>(tm) * rpt + (rr - o * rpt);
              *reinterpret_cast<uint4*>(p.ar.partial[o] + ro * p.N + gcol) = u;
            } else if (mode == 3) {
              const int o = rr / rpt;
              const long long ro = slot_base + static_cast<long long>(tm) * rpt + (rr - o * rpt);
              st_volatile_v4(p.ar.partial[o] + ll_off + ro * p.N + gcol, ll_sanitize(u));
            } else {
              const long long ro = slot_base + static_cast<long long>(tm) * BM + rr;
              for (int r = 0; r < np; ++r)
                *reinterpret_cast<uint4*>(p.ar.partial[r] + ro * p.N + gcol) = u;
            }
          }
          epi_bar_sync();
        }
        if (mode != 3 && te1 < np) red_release_sys_add(p.ar.ready[te1] + tm, 1u);
      } else if constexpr (EPI == kEpiAllGather) {
        // store this rank's column block of the tile into every peer's full-width output;
        // staged so that a warp writes whole row segments (BN * 2 contiguous bytes per row)
        uint8_t* stage = smem + L::kOutOffset;
        constexpr int SC = L::kOutCols;
        constexpr int kChunksPerRow = SC / 8;
        const int te1 = threadIdx.x - 64;
#pragma unroll 1
        for (int h = 0; h < BN / SC; ++h) {
          stage_tile<SC>(stage, taddr + h * SC, q * 32 + lane);
          if (h == BN / SC - 1) {
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&tempty_bar[acc]);
          }
          epi_bar_sync();
          for (int v = te1; v < BM * kChunksPerRow; v += 128) {
            const int rr = v / kChunksPerRow, cc = v % kChunksPerRow;
            const int grow = m0 + rr, gcol = n0 + h * SC + cc * 8;
            if (grow >= p.M || gcol >= p.N) continue;
            const uint4 u = *reinterpret_cast<const uint4*>(stage + stage_off<SC>(rr, cc));
            const long long off = static_cast<long long>(grow) * p.ldc + p.ar.col_off + gcol;
            for (int pr = 0; pr < p.ar.p; ++pr) *reinterpret_cast<uint4*>(p.ar.out[pr] + off) = u;
          }
          epi_bar_sync();
        }
        if (te1 < p.ar.p)
          signal_flag_sys(p.ar.ready[te1] + static_cast<long long>(tile) * p.ar.p + p.ar.rank,
                          epoch);
      } else {
#pragma unroll 1
        for (int c = 0; c < BN / 32; ++c) {
          uint32_t r[32];
          tmem_ld_32x32(taddr + c * 32, r);
          tmem_ld_wait();
          const int col = n0 + c * 32;
          if (!row_ok || col >= p.N) continue;
          const int ncols = min(32, p.N - col);
          float v[32];
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
          if (p.row_scale != nullptr) {
            const float rs = p.row_scale[row];
#pragma unroll
            for (int i = 0; i < 32; ++i) v[i] *= rs;
          }
          if constexpr (EPI == kEpiBias) {
            for (int i = 0; i < ncols; ++i) v[i] += __bfloat162float(p.bias[col + i]);
          }
          if constexpr (EPI == kEpiResidual) {
            const __nv_bfloat16* rr = p.residual + static_cast<long long>(row) * p.ldr + col;
            for (int i = 0; i < ncols; ++i) v[i] += __bfloat162float(rr[i]);
          }
          if constexpr (EPI == kEpiFp32) {
            float* crow = reinterpret_cast<float*>(p.C) + static_cast<long long>(row) * p.ldc + col;
            if (ncols == 32) {
#pragma unroll
              for (int i = 0; i < 8; ++i)
                reinterpret_cast<float4*>(crow)[i] =
                    make_float4(v[i * 4], v[i * 4 + 1], v[i * 4 + 2], v[i * 4 + 3]);
            } else {
              for (int i = 0; i < ncols; ++i) crow[i] = v[i];
            }
          } else {
            __nv_bfloat16* crow =
                reinterpret_cast<__nv_bfloat16*>(p.C) + static_cast<long long>(row) * p.ldc + col;
            store_row_bf16(crow, v, ncols);
          }
        }
      }
      if constexpr (EPI != kEpiAllReduce && EPI != kEpiAllGather && EPI != kEpiReduceNorm) {
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&tempty_bar[acc]);
      }
      acc ^= 1;
      if (acc == 0) acc_phase ^= 1u;
    }

    if constexpr (EPI == kEpiAllGather) {
      // the output is complete on this rank once every peer's column block of every tile
      // has landed; each CTA checks the tiles it produced itself
      const int te = threadIdx.x - 64;
      const int np = p.ar.p, rank = p.ar.rank;
      for (int t = blockIdx.x; t < num_tiles && *abort_flag == 0u; t += gridDim.x) {
        if (te < np &&
            !wait_flag_sys(p.ar.ready[rank] + static_cast<long long>(t) * np + te, epoch)) {
          report_status(p.status, kStatusFlagTimeout, kKernelId, 0x800u + te);
          *abort_flag = 1u;
        }
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tmem_base, kTmemCols);
  if constexpr (kPeerEpi<EPI>) {
    // the last CTA to finish publishes the new epoch for the next launch
    if (threadIdx.x == 0) {
      __threadfence();
      if (atomicAdd(p.ar.done_ctr, 1u) == gridDim.x - 1) {
        *p.ar.done_ctr = 0u;
        if (EPI == kEpiReduceNorm && p.ar.rn_mode != 3) {
          // every CTA of this launch has read its bases: move them past this launch's arrivals
          for (int tm = 0; tm < p.tiles_m; ++tm)
            p.ar.ready_base[tm] += static_cast<uint32_t>(p.tiles_n * p.ar.p);
        }
        __threadfence();
        *reinterpret_cast<volatile uint32_t*>(p.ar.epoch_ptr) = epoch;
      }
    }
  }
}

template <int BN, int STAGES, int EPI>
int launch(const CUtensorMap& tmA, const CUtensorMap& tmB, const Args& a, cudaStream_t stream) {
  using L = Smem<BN, STAGES, EPI>;
  auto kern = gemm_bf16_kernel<BN, STAGES, EPI>;
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
  kern<<<grid, kThreadsFor<EPI>, L::kTotal, stream>>>(tmA, tmB, a);
  return static_cast<int>(cudaGetLastError());
}

}  // namespace gemm
}  // namespace b200

// C[M,N] (bf16, or fp32 when epi == 4) = A[M,K] * B[N,K]^T with epilogue `epi`:
//   0 none, 1 + bias[N], 2 SiLU(gate)*up (B rows interleaved gate/up in blocks
//   of 32, N a multiple of 64; C is [M, N/2]), 3 + residual[M,N], 4 fp32 output.
// lda / ldb / ldc / ldr are row pitches in elements.  K, lda, ldb must be
// multiples of 8; N, ldc multiples of 8; all base pointers 16-byte aligned.
// Returns 0 on success, a CUDA error code, or a negative argument error.
B200_API int b200_gemm_bf16(const void* A, long long lda, const void* B, long long ldb, void* C,
                            long long ldc, int M, int N, int K, const void* bias,
                            const void* residual, long long ldr, int epi, void* stream) {
  using namespace b200;
  using namespace b200::gemm;
  if (M <= 0 || N <= 0) return 0;
  if (K <= 0 || (K % 8) != 0 || (lda % 8) != 0 || (ldb % 8) != 0 || (N % 8) != 0 ||
      (ldc % 8) != 0)
    return -2;
  if ((reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(B) |
       reinterpret_cast<uintptr_t>(C)) & 15)
    return -3;
  if (epi == kEpiSiluMul && (N % 64) != 0) return -4;
  if (epi == kEpiBias && bias == nullptr) return -5;
  if (epi == kEpiResidual && residual == nullptr) return -5;

  // Tile width: the candidate with the smallest (waves over the SMs) x (tile width + the
  // activation tile's share of the shared-memory fill).  Wide tiles win when there is enough
  // work; for decode-sized M a width that yields one full wave wins (6144 columns: 96).
  const int tiles_m = (M + BM - 1) / BM;
  int bn = 256;
  {
    const int cands[4] = {256, 128, 96, 64};
    long long best = -1;
    for (int i = 0; i < 4; ++i) {
      const int c = cands[i];
      if (c == 256 && (N % 256) != 0) continue;
      // the SiLU-mul epilogue pairs 32 + 32 columns: whole 64-column groups per tile
      if (epi == kEpiSiluMul && ((c % 64) != 0 || (N % c) != 0)) continue;
      const long long tiles = static_cast<long long>(tiles_m) * ((N + c - 1) / c);
      const long long waves = (tiles + sm_count() - 1) / sm_count();
      const long long cost = waves * (c + 32);
      if (best < 0 || cost < best) {
        best = cost;
        bn = c;
      }
    }
  }
  const bool wide = bn == 256;

  CUtensorMap tmA, tmB;
  int r = encode_tmap_2d(&tmA, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, A, static_cast<uint64_t>(M),
                         static_cast<uint64_t>(K), static_cast<uint64_t>(lda) * 2, BM, BK,
                         CU_TENSOR_MAP_SWIZZLE_128B);
  if (r != 0) return r < 0 ? -6 : r;
  r = encode_tmap_2d(&tmB, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, B, static_cast<uint64_t>(N),
                     static_cast<uint64_t>(K), static_cast<uint64_t>(ldb) * 2, bn, BK,
                     CU_TENSOR_MAP_SWIZZLE_128B);
  if (r != 0) return r < 0 ? -6 : r;

  Args a;
  a.C = C;
  a.ldc = ldc;
  a.bias = static_cast<const __nv_bfloat16*>(bias);
  a.residual = static_cast<const __nv_bfloat16*>(residual);
  a.ldr = ldr;
  a.M = M;
  a.N = N;
  a.K = K;
  a.tiles_m = tiles_m;
  a.tiles_n = (N + bn - 1) / bn;
  a.status = status_ptr();
  a.expert_ids = nullptr;
  a.num_valid_rows = nullptr;
  a.row_scale = nullptr;
  a.m_rot = 0;
  a.n_fastest = 0;
  a.ag = AgArgs{};
  a.ar = ArArgs{};
  cudaStream_t s = static_cast<cudaStream_t>(stream);

#define B200_GEMM_CASE(E)                                                       \
  case E:                                                                       \
    if (wide) return launch<256, 4, E>(tmA, tmB, a, s);                         \
    if (bn == 64) return launch<64, 8, E>(tmA, tmB, a, s);                      \
    if (bn == 96) return launch<96, 6, E>(tmA, tmB, a, s);                      \
    return launch<128, 6, E>(tmA, tmB, a, s);
  switch (epi) {
    B200_GEMM_CASE(kEpiNone)
    B200_GEMM_CASE(kEpiBias)
    B200_GEMM_CASE(kEpiResidual)
    B200_GEMM_CASE(kEpiFp32)
    case kEpiSiluMul:
      if (bn == 64) return launch<64, 8, kEpiSiluMul>(tmA, tmB, a, s);
      if (bn == 128) return launch<128, 6, kEpiSiluMul>(tmA, tmB, a, s);
      return launch<256, 4, kEpiSiluMul>(tmA, tmB, a, s);
    default:
      return -7;
  }
#undef B200_GEMM_CASE
}

// Row-parallel GEMM fused with the all-reduce over the tensor-parallel peers:
//   out_r[M,N] = sum over ranks ( A_rank[M,K] * B_rank[N,K]^T ) (+ residual), on every rank r.
// Every rank launches this with the same M, N, K.  `partial`, `out`, `ready`, `done` are
// arrays of `p` peer-visible device addresses (symmetric memory, index = rank);
// `epoch_ptr` / `done_ctr` are local zero-initialised words.  Tile t is reduced by rank
// t % p, which pulls the p partial tiles with plain peer loads and pushes the sum to all
// ranks with peer stores; flags use release/acquire at system scope with bounded waits.
// With oneshot != 0 every rank instead pushes its partial tiles into slot
// (epoch parity, rank) of every peer's partial buffer and reduces all tiles locally
// (one flag hop; best for small M or p == 2); slot_elems is the slot pitch in elements.
// Capacity needed: partial >= tiles * 128 * BN bf16 (two-shot) or 2 * p * slot_elems
// (one-shot), ready >= tiles * p, done >= tiles words, where
// tiles = ceil(M/128) * ceil(N/BN) and BN is what b200_gemm_ar_tile_n(M, N) returns.
B200_API int b200_gemm_ar_tile_n(int M, int N) {
  using namespace b200;
  const int tiles_m = (M + b200::gemm::BM - 1) / b200::gemm::BM;
  if ((N % 256) == 0 && static_cast<long long>(tiles_m) * (N / 256) >= sm_count()) return 256;
  return (static_cast<long long>(tiles_m) * ((N + 127) / 128) < sm_count()) ? 64 : 128;
}

B200_API int b200_gemm_bf16_allreduce(const void* A, long long lda, const void* B, long long ldb,
                                      long long ldc, int M, int N, int K, void* const* partial,
                                      void* const* out, void* const* ready, void* const* done,
                                      void* epoch_ptr, void* done_ctr, int rank, int p,
                                      const void* residual, long long ldr, int oneshot,
                                      long long slot_elems, void* stream) {
  using namespace b200;
  using namespace b200::gemm;
  if (M <= 0 || N <= 0) return 0;
  if (p < 1 || p > kMaxPeers || rank < 0 || rank >= p) return -2;
  if (K <= 0 || (K % 8) != 0 || (lda % 8) != 0 || (ldb % 8) != 0 || (N % 8) != 0 ||
      (ldc % 8) != 0)
    return -2;
  const int bn = b200_gemm_ar_tile_n(M, N);
  CUtensorMap tmA, tmB;
  int r = encode_tmap_2d(&tmA, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, A, static_cast<uint64_t>(M),
                         static_cast<uint64_t>(K), static_cast<uint64_t>(lda) * 2, BM, BK,
                         CU_TENSOR_MAP_SWIZZLE_128B);
  if (r != 0) return r < 0 ? -6 : r;
  r = encode_tmap_2d(&tmB, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, B, static_cast<uint64_t>(N),
                     static_cast<uint64_t>(K), static_cast<uint64_t>(ldb) * 2, bn, BK,
                     CU_TENSOR_MAP_SWIZZLE_128B);
  if (r != 0) return r < 0 ? -6 : r;
  Args a;
  a.C = nullptr;
  a.ldc = ldc;
  a.bias = nullptr;
  a.residual = static_cast<const __nv_bfloat16*>(residual);
  a.ldr = ldr;
  a.M = M; a.N = N; a.K = K;
  a.tiles_m = (M + BM - 1) / BM;
  a.tiles_n = (N + bn - 1) / bn;
  a.status = status_ptr();
  a.expert_ids = nullptr;
  a.num_valid_rows = nullptr;
  a.row_scale = nullptr;
  a.m_rot = 0;
  a.n_fastest = 0;
  a.ag = AgArgs{};
  for (int i = 0; i < kMaxPeers; ++i) {
    a.ar.partial[i] = i < p ? static_cast<__nv_bfloat16*>(partial[i]) : nullptr;
    a.ar.out[i] = i < p ? static_cast<__nv_bfloat16*>(out[i]) : nullptr;
    a.ar.ready[i] = i < p ? static_cast<uint32_t*>(ready[i]) : nullptr;
    a.ar.done[i] = i < p ? static_cast<uint32_t*>(done[i]) : nullptr;
  }
  a.ar.epoch_ptr = static_cast<uint32_t*>(epoch_ptr);
  a.ar.done_ctr = static_cast<uint32_t*>(done_ctr);
  a.ar.rank = rank;
  a.ar.p = p;
  a.ar.oneshot = oneshot;
  a.ar.slot_elems = slot_elems;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (bn == 64) return launch<64, 8, kEpiAllReduce>(tmA, tmB, a, s);
  if (bn == 256) return launch<256, 4, kEpiAllReduce>(tmA, tmB, a, s);
  return launch<128, 6, kEpiAllReduce>(tmA, tmB, a, s);
}

// Row-parallel GEMM fused with the all-reduce, the residual add and the RMSNorm that follow it
// in a transformer layer:
//   z      = sum over ranks ( A_rank[M,K] * B_rank[N,K]^T ) + residual      (rounded to bf16)
//   out_r  = z * rsqrt(mean(z^2) + eps) * norm_weight    on every rank r    (norm_weight given)
//   out_r  = z                                           on every rank r    (norm_weight null)
// Every rank parks its bf16 partial product in its own symmetric buffer; inside every 128-row
// tile rank r owns rows [128 r / p, 128 (r + 1) / p): reducer warps of the same kernel wait
// for all column tiles of those rows from all ranks, pull them with plain peer loads (or one
// in-switch multimem.ld_reduce when the multicast views mc_* are given), and store the
// finished rows into every rank (peer stores or multimem.st).  The new residual z goes to
// res_out of the owner only (bcast_res = 0: enough when the next consumer of the residual is
// again this entry point) or of every rank (bcast_res = 1).  Without a norm weight res_out is
// not written.
// rn_mode selects how the partial rows travel: 0 = every rank parks its partial matrix in its
// own buffer and the owners pull their rows (the mode for many rows; the only one that can use
// mc_partial); 1 = the epilogue pushes every row into the owner's buffer, slot
// (launch parity, source rank), and the owner reduces from local memory (decode-sized
// problems: one NVLink round trip less on the critical path); 2 = every row is pushed to
// every rank and every rank reduces all rows (one hop, nothing is broadcast afterwards; done
// is not used).  Modes 1 and 2 need 128 % p == 0 and a partial buffer of
// 2 * p * ceil(M/128) * (128 / p) * N elements (mode 2: 2 * p * ceil(M/128) * 128 * N).
// 3 = like 1, but nothing is flagged or fenced: the transport buffers hold a sentinel word
// (two bf16 negative zeros) wherever no data has landed yet and every receiver polls the data
// itself, which takes the release / acquire round trips off the critical path of a decode
// step.  partial[r] and out[r] then name three rotating transport buffers of ll_cap elements
// each on rank r (all filled with 0x80008000 words before the first call; the kernel restores
// the sentinel itself afterwards), the result lands in ll_out_local [M, ldc] (local),
// ll_used is 6 local zero-initialised 64-bit words; bcast_res must be 0 and
// ceil(M/128) * 128 * N <= ll_cap.
// partial / out / res_out / ready / done: arrays of p peer-visible addresses (index = rank):
// partial [M, N] bf16, out [M, ldc], res_out [M, N], ready ceil(M/128) words (arrival
// counters), done M words; ready_base: local ceil(M/128) words; epoch_ptr / done_ctr: local
// words; all zero before the first call and private to this entry point.  residual: local [M, ldr] or null.  N <= 8192.  All ranks pass the
// same shapes.  A launch returns when every row of `out` has arrived on this rank.
B200_API int b200_gemm_bf16_ar_norm(const void* A, long long lda, const void* B, long long ldb,
                                    long long ldc, int M, int N, int K, void* const* partial,
                                    void* const* out, void* const* res_out, void* const* ready,
                                    void* const* done, void* ready_base, void* epoch_ptr,
                                    void* done_ctr, int rank, int p, const void* residual,
                                    long long ldr, const void* norm_weight, float eps,
                                    int bcast_res, int rn_mode, const void* mc_partial, void* mc_out,
                                    void* mc_res, void* ll_out_local, long long ll_cap,
                                    void* ll_used, void* stream) {
  using namespace b200;
  using namespace b200::gemm;
  if (M <= 0 || N <= 0) return 0;
  if (p < 1 || p > kMaxPeers || rank < 0 || rank >= p) return -2;
  if (K <= 0 || (K % 8) != 0 || (lda % 8) != 0 || (ldb % 8) != 0 || (N % 8) != 0 ||
      (ldc % 8) != 0 || (ldr % 8) != 0 || N > kRnKeep * 128 * 8)
    return -2;
  if (rn_mode < 0 || rn_mode > 3 || (rn_mode != 0 && (BM % p) != 0)) return -2;
  if (rn_mode == 3) {
    const long long tiles_m = (M + BM - 1) / BM;
    if (ll_out_local == nullptr || ll_used == nullptr || bcast_res != 0 ||
        tiles_m * BM * static_cast<long long>(N) > ll_cap || (ll_cap % 8) != 0)
      return -2;
  }
  const int bn = b200_gemm_ar_tile_n(M, N);
  CUtensorMap tmA, tmB;
  int r = encode_tmap_2d(&tmA, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, A, static_cast<uint64_t>(M),
                         static_cast<uint64_t>(K), static_cast<uint64_t>(lda) * 2, BM, BK,
                         CU_TENSOR_MAP_SWIZZLE_128B);
  if (r != 0) return r < 0 ? -6 : r;
  r = encode_tmap_2d(&tmB, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, B, static_cast<uint64_t>(N),
                     static_cast<uint64_t>(K), static_cast<uint64_t>(ldb) * 2, bn, BK,
                     CU_TENSOR_MAP_SWIZZLE_128B);
  if (r != 0) return r < 0 ? -6 : r;
  Args a{};
  a.ldc = ldc;
  a.M = M; a.N = N; a.K = K;
  a.tiles_m = (M + BM - 1) / BM;
  a.tiles_n = (N + bn - 1) / bn;
  a.status = status_ptr();
  a.n_fastest = 1;
  for (int i = 0; i < p; ++i) {
    a.ar.partial[i] = static_cast<__nv_bfloat16*>(partial[i]);
    a.ar.out[i] = static_cast<__nv_bfloat16*>(out[i]);
    a.ar.res_out[i] = res_out ? static_cast<__nv_bfloat16*>(res_out[i]) : nullptr;
    a.ar.ready[i] = static_cast<uint32_t*>(ready[i]);
    a.ar.done[i] = static_cast<uint32_t*>(done[i]);
  }
  a.ar.epoch_ptr = static_cast<uint32_t*>(epoch_ptr);
  a.ar.done_ctr = static_cast<uint32_t*>(done_ctr);
  a.ar.rank = rank;
  a.ar.p = p;
  a.ar.res_in = static_cast<const __nv_bfloat16*>(residual);
  a.ar.ld_res_in = ldr;
  a.ar.norm_weight = static_cast<const __nv_bfloat16*>(norm_weight);
  a.ar.eps = eps;
  a.ar.bcast_res = bcast_res;
  a.ar.rn_mode = rn_mode;
  a.ar.ready_base = static_cast<uint32_t*>(ready_base);
  a.ar.ll_out_local = static_cast<__nv_bfloat16*>(ll_out_local);
  a.ar.ll_cap = ll_cap;
  a.ar.ll_used = static_cast<long long*>(ll_used);
  a.ar.slot_rows = static_cast<long long>(a.tiles_m) * (rn_mode == 2 ? BM : BM / p);
  a.ar.mc_partial = static_cast<const __nv_bfloat16*>(mc_partial);
  a.ar.mc_out = static_cast<__nv_bfloat16*>(mc_out);
  a.ar.mc_res = static_cast<__nv_bfloat16*>(mc_res);
  if (norm_weight != nullptr && res_out == nullptr) return -5;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (bn == 64) return launch<64, 8, kEpiReduceNorm>(tmA, tmB, a, s);
  if (bn == 256) return launch<256, 4, kEpiReduceNorm>(tmA, tmB, a, s);
  return launch<128, 6, kEpiReduceNorm>(tmA, tmB, a, s);
}

namespace {
int fill_peer_args(b200::gemm::Args& a, void* const* out, void* const* ready,
                   void* const* started, void* epoch_ptr,
                   void* done_ctr, int rank, int p) {
  using namespace b200::gemm;
  if (p < 1 || p > kMaxPeers || rank < 0 || rank >= p) return -2;
  a.ar = ArArgs{};
  for (int i = 0; i < p; ++i) {
    a.ar.out[i] = out ? static_cast<__nv_bfloat16*>(out[i]) : nullptr;
    a.ar.ready[i] = ready ? static_cast<uint32_t*>(ready[i]) : nullptr;
    a.ar.done[i] = started ? static_cast<uint32_t*>(started[i]) : nullptr;
  }
  a.ar.epoch_ptr = static_cast<uint32_t*>(epoch_ptr);
  a.ar.done_ctr = static_cast<uint32_t*>(done_ctr);
  a.ar.rank = rank;
  a.ar.p = p;
  return 0;
}
}  // namespace

// Column-parallel GEMM fused with the all-gather of its output over the peers (the
// vocabulary-parallel LM head): rank r computes C_r[M, N] = A[M,K] * B_r[N,K]^T and its
// epilogue stores the tile into columns [col_off, col_off + N) of the [M, ldc] output of
// EVERY rank with peer stores, then raises ready[peer][tile * p + rank]; a launch returns
// once all peers' blocks of the tiles it produced have landed locally.  A rank stores into a
// peer only after that peer has entered the same launch (started[peer][rank] flag), so one
// output buffer per rank is enough even when the launches are replayed from a CUDA graph.
// `out` / `ready` / `started` are arrays of p peer-visible addresses; ready needs tiles * p
// words with tiles = ceil(M/128) * ceil(N/BN), BN = b200_gemm_ar_tile_n(M, N); started needs
// p words.  All ranks pass the same M, N, K.
B200_API int b200_gemm_bf16_allgather(const void* A, long long lda, const void* B, long long ldb,
                                      long long ldc, long long col_off, int M, int N, int K,
                                      void* const* out, void* const* ready,
                                      void* const* started, void* epoch_ptr, void* done_ctr,
                                      int rank, int p, void* stream) {
  using namespace b200;
  using namespace b200::gemm;
  if (M <= 0 || N <= 0) return 0;
  if (K <= 0 || (K % 8) != 0 || (lda % 8) != 0 || (ldb % 8) != 0 || (N % 8) != 0 ||
      (ldc % 8) != 0 || (col_off % 8) != 0)
    return -2;
  const int bn = b200_gemm_ar_tile_n(M, N);
  CUtensorMap tmA, tmB;
  int r = encode_tmap_2d(&tmA, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, A, static_cast<uint64_t>(M),
                         static_cast<uint64_t>(K), static_cast<uint64_t>(lda) * 2, BM, BK,
                         CU_TENSOR_MAP_SWIZZLE_128B);
  if (r != 0) return r < 0 ? -6 : r;
  r = encode_tmap_2d(&tmB, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, B, static_cast<uint64_t>(N),
                     static_cast<uint64_t>(K), static_cast<uint64_t>(ldb) * 2, bn, BK,
                     CU_TENSOR_MAP_SWIZZLE_128B);
  if (r != 0) return r < 0 ? -6 : r;
  Args a{};
  a.ldc = ldc;
  a.M = M; a.N = N; a.K = K;
  a.tiles_m = (M + BM - 1) / BM;
  a.tiles_n = (N + bn - 1) / bn;
  a.status = status_ptr();
  a.ag = AgArgs{};
  r = fill_peer_args(a, out, ready, started, epoch_ptr, done_ctr, rank, p);
  if (r != 0) return r;
  a.ar.col_off = col_off;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (bn == 64) return launch<64, 8, kEpiAllGather>(tmA, tmB, a, s);
  if (bn == 256) return launch<256, 4, kEpiAllGather>(tmA, tmB, a, s);
  return launch<128, 6, kEpiAllGather>(tmA, tmB, a, s);
}

// All-gather of the input fused into a column-parallel GEMM (sequence-parallel activations):
//   C[M, N] = gather_r(A_r)[M, K] * B[N, K]^T,   rank r owning rows
//   [row_off[r], row_off[r+1]) with row_off[0] = 0 and row_off[p] = M (host array, p + 1 ints).
// `shard` holds p peer-visible addresses of the row shards (pitch lds); a_full is a
// LOCAL [M, lda] staging buffer that the gather warps of the kernel fill chunk by chunk with
// peer loads while the tensor cores already work on the chunks that have arrived (own rows
// first, then the peers in ring order).  in_ready / rd_done: p words per rank in symmetric
// memory; chunk_ready: ceil(M/128) local words; gather_ctr, epoch_ptr, done_ctr: local words,
// all zero-initialised once.  The caller may overwrite its shard as soon as the launch has
// finished (the kernel waits until every peer is done reading it).
B200_API int b200_gemm_bf16_gather_a(void* const* shard, long long lds, const int* row_off,
                                     void* a_full,
                                     long long lda, const void* B, long long ldb, void* C,
                                     long long ldc, int M, int N, int K, void* const* in_ready,
                                     void* const* rd_done, void* chunk_ready, void* gather_ctr,
                                     void* epoch_ptr, void* done_ctr, int rank, int p,
                                     void* stream) {
  using namespace b200;
  using namespace b200::gemm;
  if (M <= 0 || N <= 0) return 0;
  if (K <= 0 || (K % 8) != 0 || (lda % 8) != 0 || (ldb % 8) != 0 || (N % 8) != 0 ||
      (ldc % 8) != 0 || (lds % 8) != 0 || row_off == nullptr || p < 1 || p > kMaxPeers ||
      row_off[0] != 0 || row_off[p] != M)
    return -2;
  for (int i = 0; i < p; ++i)
    if (row_off[i + 1] < row_off[i]) return -2;
  const int tiles_m = (M + BM - 1) / BM;
  const bool narrow = static_cast<long long>(tiles_m) * ((N + 127) / 128) < sm_count();
  const int bn = narrow ? 64 : 128;
  CUtensorMap tmA, tmB;
  int r = encode_tmap_2d(&tmA, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, a_full,
                         static_cast<uint64_t>(M), static_cast<uint64_t>(K),
                         static_cast<uint64_t>(lda) * 2, BM, BK, CU_TENSOR_MAP_SWIZZLE_128B);
  if (r != 0) return r < 0 ? -6 : r;
  r = encode_tmap_2d(&tmB, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, B, static_cast<uint64_t>(N),
                     static_cast<uint64_t>(K), static_cast<uint64_t>(ldb) * 2, bn, BK,
                     CU_TENSOR_MAP_SWIZZLE_128B);
  if (r != 0) return r < 0 ? -6 : r;
  Args a{};
  a.C = C;
  a.ldc = ldc;
  a.M = M; a.N = N; a.K = K;
  a.tiles_m = tiles_m;
  a.tiles_n = (N + bn - 1) / bn;
  a.status = status_ptr();
  r = fill_peer_args(a, nullptr, nullptr, nullptr, epoch_ptr, done_ctr, rank, p);
  if (r != 0) return r;
  a.ag = AgArgs{};
  for (int i = 0; i < p; ++i) {
    a.ag.shard[i] = static_cast<const __nv_bfloat16*>(shard[i]);
    a.ag.in_ready[i] = static_cast<uint32_t*>(in_ready[i]);
    a.ag.rd_done[i] = static_cast<uint32_t*>(rd_done[i]);
  }
  a.ag.a_full = static_cast<__nv_bfloat16*>(a_full);
  a.ag.lds = lds;
  a.ag.lda = lda;
  a.ag.chunk_ready = static_cast<uint32_t*>(chunk_ready);
  a.ag.gather_ctr = static_cast<uint32_t*>(gather_ctr);
  for (int i = 0; i <= p; ++i) a.ag.row_off[i] = row_off[i];
  for (int i = p + 1; i <= kMaxPeers; ++i) a.ag.row_off[i] = M;
  a.ag.enabled = 1;
  a.m_rot = (row_off[rank] / BM) % tiles_m;   // start with the tiles of this rank's own rows
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (bn == 64) return launch<64, 8, kEpiGatherA>(tmA, tmB, a, s);
  return launch<128, 6, kEpiGatherA>(tmA, tmB, a, s);
}

// Grouped GEMM for mixture-of-experts layers.  A [M_cap, K] holds token rows sorted by
// expert, every expert segment padded to a multiple of 128 rows (b200_moe_align);
// B [E * N, K] stacks the expert weights; tile i of A uses expert expert_ids[i] (-1 and
// tiles at or past *num_valid_rows are skipped, so M_cap may be a static upper bound).
// epi 0: C[M_cap, N] = A * B_e^T (optionally scaled per row by row_scale);
// epi 2: SiLU(gate) * up with the gate / up rows of every expert interleaved in blocks of
// 32 (C is [M_cap, N / 2]).  N must be a multiple of the tile width (256 for epi 2,
// else 128 or 64).
B200_API int b200_gemm_bf16_grouped(const void* A, long long lda, const void* B, long long ldb,
                                    void* C, long long ldc, int M_cap, int N, int K, int E,
                                    const int* expert_ids, const int* num_valid_rows,
                                    const float* row_scale, int epi, void* stream) {
  using namespace b200;
  using namespace b200::gemm;
  if (M_cap <= 0 || N <= 0 || E <= 0) return 0;
  if ((M_cap % BM) != 0 || K <= 0 || (K % 8) != 0 || (lda % 8) != 0 || (ldb % 8) != 0 ||
      (ldc % 8) != 0 || expert_ids == nullptr || num_valid_rows == nullptr)
    return -2;
  int bn;
  if (epi == kEpiSiluMul) {
    if ((N % 256) != 0) return -4;
    bn = 256;
  } else if (epi == kEpiNone) {
    bn = (N % 128) == 0 ? 128 : 64;
    if ((N % bn) != 0) return -4;
  } else {
    return -7;
  }
  CUtensorMap tmA, tmB;
  int r = encode_tmap_2d(&tmA, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, A,
                         static_cast<uint64_t>(M_cap), static_cast<uint64_t>(K),
                         static_cast<uint64_t>(lda) * 2, BM, BK, CU_TENSOR_MAP_SWIZZLE_128B);
  if (r != 0) return r < 0 ? -6 : r;
  r = encode_tmap_2d(&tmB, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, B,
                     static_cast<uint64_t>(E) * N, static_cast<uint64_t>(K),
                     static_cast<uint64_t>(ldb) * 2, bn, BK, CU_TENSOR_MAP_SWIZZLE_128B);
  if (r != 0) return r < 0 ? -6 : r;
  Args a;
  a.C = C;
  a.ldc = ldc;
  a.bias = nullptr;
  a.residual = nullptr;
  a.ldr = 0;
  a.M = M_cap; a.N = N; a.K = K;
  a.tiles_m = M_cap / BM;
  a.tiles_n = N / bn;
  a.status = status_ptr();
  a.expert_ids = expert_ids;
  a.num_valid_rows = num_valid_rows;
  a.row_scale = row_scale;
  a.m_rot = 0;
  a.n_fastest = 0;
  a.ag = AgArgs{};
  a.ar = ArArgs{};
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (epi == kEpiSiluMul) return launch<256, 4, kEpiSiluMul>(tmA, tmB, a, s);
  if (bn == 128) return launch<128, 6, kEpiNone>(tmA, tmB, a, s);
  return launch<64, 8, kEpiNone>(tmA, tmB, a, s);
}
