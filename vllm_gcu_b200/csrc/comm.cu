// Stand-alone collectives over symmetric memory (NVLink 5 / NVSwitch peer access).
//
//   all_reduce   two-shot: rank r pulls slice r of every peer's staging buffer with plain
//                peer loads, sums in fp32 and pushes the result to every peer's output
//   all_gather   each rank pushes its shard into every peer's output
//
// Synchronisation: 32-bit flags holding the launch epoch, written with st.release.sys
// and polled with ld.acquire.sys; every wait is bounded and reports a timeout through the
// status word instead of spinning forever.  The epoch lives in device memory and is advanced
// by the last CTA of each launch, so the kernels can be replayed from CUDA graphs.
//
// These are the small-message fast paths next to NCCL (which stays the baseline and the
// fallback); the reference reaches the same collectives through
// vllm_gcu/distributed/gcu_communicator.py:88-126 and parallel_state.py:107-203.
#include "common.cuh"

namespace b200 {
namespace comm {

constexpr unsigned int kKernelId = 50;
constexpr int kMaxPeers = 8;

struct Peers {
  void* src[kMaxPeers];
  void* out[kMaxPeers];
  uint32_t* flag[kMaxPeers];  // per rank: [0..p) arrive flags, [p..2p) done flags
};

__device__ __forceinline__ bool wait_flag(const uint32_t* flag, uint32_t want, uint32_t limit) {
  for (uint32_t it = 0; it < limit; ++it) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(flag) : "memory");
    if (static_cast<int32_t>(v - want) >= 0) return true;  // epochs only grow
    if (it > 64) __nanosleep(100);
  }
  return false;
}
__device__ __forceinline__ void signal_flag(uint32_t* flag, uint32_t val) {
  __threadfence_system();
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(flag), "r"(val) : "memory");
}
__device__ __forceinline__ uint4 ld_v4(const void* p) {
  uint4 v;
  asm volatile("ld.volatile.global.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p)
               : "memory");
  return v;
}

// mode 0: all-reduce (sum) of n bf16 elements; mode 1: all-gather of n elements per rank.
__global__ void __launch_bounds__(512)
    collective_kernel(const Peers pr, uint32_t* epoch_ptr, uint32_t* ctr, long long n, int rank,
                      int p, int mode, unsigned int* status) {
  __shared__ int s_abort;
  const uint32_t epoch = *reinterpret_cast<volatile uint32_t*>(epoch_ptr) + 1u;
  const uint32_t spin = flag_spin_limit(status);
  if (threadIdx.x == 0) s_abort = 0;
  __syncthreads();
  // announce that this rank's staging buffer is ready (it was filled before the launch)
  if (blockIdx.x == 0 && threadIdx.x < p) signal_flag(pr.flag[threadIdx.x] + rank, epoch);
  if (threadIdx.x < p) {
    if (!wait_flag(pr.flag[rank] + threadIdx.x, epoch, spin)) {
      report_status(status, kStatusFlagTimeout, kKernelId, 0x100u + threadIdx.x);
      s_abort = 1;
    }
  }
  __syncthreads();
  if (s_abort == 0) {
    const long long nvec = n >> 3;
    const long long tid = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
    const long long nthreads = static_cast<long long>(gridDim.x) * blockDim.x;
    if (mode == 0) {
      const long long lo = nvec * rank / p, hi = nvec * (rank + 1) / p;
      for (long long v = lo + tid; v < hi; v += nthreads) {
        float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        for (int r = 0; r < p; ++r) {
          const uint4 u = ld_v4(static_cast<const uint4*>(pr.src[r]) + v);
          const float2 a = unpack_bf16x2(u.x), b = unpack_bf16x2(u.y), c = unpack_bf16x2(u.z),
                       d = unpack_bf16x2(u.w);
          acc[0] += a.x; acc[1] += a.y; acc[2] += b.x; acc[3] += b.y;
          acc[4] += c.x; acc[5] += c.y; acc[6] += d.x; acc[7] += d.y;
        }
        uint4 o;
        o.x = pack_bf16x2(acc[0], acc[1]);
        o.y = pack_bf16x2(acc[2], acc[3]);
        o.z = pack_bf16x2(acc[4], acc[5]);
        o.w = pack_bf16x2(acc[6], acc[7]);
        for (int r = 0; r < p; ++r) static_cast<uint4*>(pr.out[r])[v] = o;
      }
    } else {
      const uint4* mine = static_cast<const uint4*>(pr.src[rank]);
      for (long long v = tid; v < nvec; v += nthreads) {
        const uint4 u = mine[v];
        for (int r = 0; r < p; ++r) static_cast<uint4*>(pr.out[r])[nvec * rank + v] = u;
      }
    }
  }
  // last CTA of this rank: tell everyone that this rank's pushes are complete
  __shared__ int s_last;
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence_system();
    s_last = (atomicAdd(ctr, 1u) == gridDim.x - 1) ? 1 : 0;
  }
  __syncthreads();
  if (s_last) {
    if (threadIdx.x < p) signal_flag(pr.flag[threadIdx.x] + p + rank, epoch);
  }
  // nobody leaves before every peer's pushes have landed here
  if (threadIdx.x < p && s_abort == 0) {
    if (!wait_flag(pr.flag[rank] + p + threadIdx.x, epoch, spin))
      report_status(status, kStatusFlagTimeout, kKernelId, 0x200u + threadIdx.x);
  }
  __syncthreads();
  if (s_last && threadIdx.x == 0) {
    // every CTA of this launch has passed its atomicAdd; publish the epoch for the next one
    // once they have all left the wait above is not required: the epoch word is only read
    // at kernel start and the next launch starts after this one completes.
    *ctr = 0u;
    __threadfence();
    *reinterpret_cast<volatile uint32_t*>(epoch_ptr) = epoch;
  }
}

// Greedy sampling over a vocabulary-parallel LM head: every rank holds logits[B, V_local] of
// its vocabulary block.  One CTA per row finds the local (max, argmax), stores the 16-byte
// record {value bits, global token id, epoch, 0} into slot (epoch parity, this rank, row) of
// every rank with one vector store, then polls its own p slots of that row until they carry
// this launch's epoch (bounded), and writes the winning token id.  One kernel and one hop
// instead of gathering B x V logits: 16 bytes per row and rank cross NVLink.
struct SlotPtrs {
  uint4* s[kMaxPeers];
};

__global__ void __launch_bounds__(256)
    argmax_allgather_kernel(const __nv_bfloat16* logits, long long ld, int B, int v_local,
                            int v_offset, const SlotPtrs slots, int max_rows, uint32_t* epoch_ptr,
                            uint32_t* ctr, int rank, int p, long long* out_ids,
                            unsigned int* status) {
  __shared__ float s_val[8];
  __shared__ int s_idx[8];
  const uint32_t epoch = *reinterpret_cast<volatile uint32_t*>(epoch_ptr) + 1u;
  const uint32_t spin = flag_spin_limit(status);
  const int row = blockIdx.x;
  const __nv_bfloat16* x = logits + static_cast<long long>(row) * ld;
  float best = -INFINITY;
  int bi = 0x7fffffff;
  const int nvec = v_local >> 3;
  for (int v = threadIdx.x; v < nvec; v += blockDim.x) {
    const uint4 u = *reinterpret_cast<const uint4*>(x + v * 8);
    const float2 a = unpack_bf16x2(u.x), b = unpack_bf16x2(u.y), c = unpack_bf16x2(u.z),
                 d = unpack_bf16x2(u.w);
    const float f[8] = {a.x, a.y, b.x, b.y, c.x, c.y, d.x, d.y};
#pragma unroll
    for (int i = 0; i < 8; ++i)
      if (f[i] > best) { best = f[i]; bi = v * 8 + i; }       // ascending ids: first maximum
  }
  for (int i = nvec * 8 + threadIdx.x; i < v_local; i += blockDim.x) {
    const float f = __bfloat162float(x[i]);
    if (f > best || (f == best && i < bi)) { best = f; bi = i; }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
  }
  if ((threadIdx.x & 31) == 0) { s_val[threadIdx.x >> 5] = best; s_idx[threadIdx.x >> 5] = bi; }
  __syncthreads();
  if (threadIdx.x < 32) {
    const int lane = threadIdx.x;
    best = lane < (blockDim.x >> 5) ? s_val[lane] : -INFINITY;
    bi = lane < (blockDim.x >> 5) ? s_idx[lane] : 0x7fffffff;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
    }
    const long long slot_base = static_cast<long long>(epoch & 1u) * p * max_rows;
    if (lane < p) {
      uint4 rec;
      rec.x = __float_as_uint(best);
      rec.y = static_cast<uint32_t>(bi == 0x7fffffff ? 0 : bi + v_offset);
      rec.z = epoch;
      rec.w = 0u;
      uint4* dst = slots.s[lane] + slot_base + static_cast<long long>(rank) * max_rows + row;
      asm volatile("st.volatile.global.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(dst), "r"(rec.x),
                   "r"(rec.y), "r"(rec.z), "r"(rec.w)
                   : "memory");
    }
    // collect the p records of this row
    float rv = -INFINITY;
    uint32_t ri = 0xffffffffu;
    bool ok = true;
    if (lane < p) {
      const uint4* src = slots.s[rank] + slot_base + static_cast<long long>(lane) * max_rows + row;
      ok = false;
      for (uint32_t it = 0; it < spin; ++it) {
        const uint4 u = ld_v4(src);
        if (u.z == epoch) {
          rv = __uint_as_float(u.x);
          ri = u.y;
          ok = true;
          break;
        }
        if (it > 64) __nanosleep(100);
      }
      if (!ok) report_status(status, kStatusFlagTimeout, kKernelId, 0x300u + lane);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, rv, o);
      const uint32_t oi = __shfl_xor_sync(0xffffffffu, ri, o);
      if (ov > rv || (ov == rv && oi < ri)) { rv = ov; ri = oi; }
    }
    if (lane == 0) out_ids[row] = static_cast<long long>(ri == 0xffffffffu ? 0u : ri);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    if (atomicAdd(ctr, 1u) == gridDim.x - 1) {
      *ctr = 0u;
      __threadfence();
      *reinterpret_cast<volatile uint32_t*>(epoch_ptr) = epoch;
    }
  }
}

}  // namespace comm
}  // namespace b200

// src / out / flag: arrays of p peer-visible addresses (index = rank).  flag regions hold
// 2 * p zero-initialised words per rank.  epoch_ptr / ctr: local zero-initialised words.
// mode 0: out_r[0..n) = sum_r src_r[0..n) (bf16, n % 8 == 0);
// mode 1: out_r[rank * n .. (rank + 1) * n) = src_rank[0..n).
B200_API int b200_allreduce(void* const* src, void* const* out, void* const* flag,
                            void* epoch_ptr, void* ctr, void* /*reserved*/, long long n, int rank,
                            int p, int mode, void* stream) {
  using namespace b200;
  using namespace b200::comm;
  if (n <= 0) return 0;
  if (p < 1 || p > kMaxPeers || rank < 0 || rank >= p || (n % 8) != 0) return -2;
  Peers pr;
  for (int i = 0; i < kMaxPeers; ++i) {
    pr.src[i] = i < p ? src[i] : nullptr;
    pr.out[i] = i < p ? out[i] : nullptr;
    pr.flag[i] = i < p ? static_cast<uint32_t*>(flag[i]) : nullptr;
  }
  const long long nvec = n / 8;
  const long long work = mode == 0 ? (nvec + p - 1) / p : nvec;
  long long blocks = (work + 511) / 512;
  const int cap = sm_count();
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  collective_kernel<<<static_cast<int>(blocks), 512, 0, static_cast<cudaStream_t>(stream)>>>(
      pr, static_cast<uint32_t*>(epoch_ptr), static_cast<uint32_t*>(ctr), n, rank, p, mode,
      status_ptr());
  return static_cast<int>(cudaGetLastError());
}

// Token ids of the row-wise maximum over a vocabulary-parallel logits matrix:
// out_ids[b] = argmax over all ranks' blocks of logits_r[b, 0..v_local) + v_offset_r (ties go
// to the smaller id).  logits: local bf16 [B, ld]; slots: p peer-visible addresses of
// 2 * p * max_rows 16-byte records each (zero before the first call); epoch_ptr / ctr: local
// zero words.  B <= max_rows; all ranks pass the same B.
B200_API int b200_argmax_allgather(const void* logits, long long ld, int B, int v_local,
                                   int v_offset, void* const* slots, int max_rows,
                                   void* epoch_ptr, void* ctr, int rank, int p, void* out_ids,
                                   void* stream) {
  using namespace b200;
  using namespace b200::comm;
  if (B <= 0) return 0;
  if (p < 1 || p > kMaxPeers || rank < 0 || rank >= p || B > max_rows || v_local < 0 ||
      (ld % 8) != 0)
    return -2;
  SlotPtrs sp;
  for (int i = 0; i < kMaxPeers; ++i) sp.s[i] = i < p ? static_cast<uint4*>(slots[i]) : nullptr;
  argmax_allgather_kernel<<<B, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(logits), ld, B, v_local, v_offset, sp, max_rows,
      static_cast<uint32_t*>(epoch_ptr), static_cast<uint32_t*>(ctr), rank, p,
      static_cast<long long*>(out_ids), status_ptr());
  return static_cast<int>(cudaGetLastError());
}
