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

__device__ __forceinline__ bool wait_flag(const uint32_t* flag, uint32_t want) {
  for (uint32_t it = 0; it < (1u << 22); ++it) {
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
  if (threadIdx.x == 0) s_abort = 0;
  __syncthreads();
  // announce that this rank's staging buffer is ready (it was filled before the launch)
  if (blockIdx.x == 0 && threadIdx.x < p) signal_flag(pr.flag[threadIdx.x] + rank, epoch);
  if (threadIdx.x < p) {
    if (!wait_flag(pr.flag[rank] + threadIdx.x, epoch)) {
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
    if (!wait_flag(pr.flag[rank] + p + threadIdx.x, epoch))
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
