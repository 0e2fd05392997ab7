// Expert-parallel token dispatch and combine over peer memory (NVLink / NVSwitch).
//
// Every rank holds different tokens (data-parallel attention); a token must visit each
// rank that owns one of its top-k experts.  Three kernels, no host synchronisation, every
// row count stays on the device:
//
//   ep_route     one CTA.  Per destination rank, the tokens that have an expert there, in
//                token order (a token is sent once per destination rank, not once per
//                expert), the position of every token in each destination's list, and the
//                push of this rank's count vector into the count matrix of every peer.
//   ep_dispatch  waits for the count matrix (ep x ep words, the only hop before data
//                moves), derives all offsets from it, then packs and stores each row
//                [hidden | top-k ids | top-k weights] straight into the destination's
//                receive buffer at a compact, source-major position with plain peer
//                stores; the last CTA raises a flag on every destination; CTA 0 returns
//                only when all sources' flags have arrived, so the receive buffers are
//                complete when the kernel ends.  The receive count is a device scalar that
//                the expert kernels take as their valid-row bound.
//   ep_combine   pushes the expert output row of every received row back into the
//                source's return buffer (same layout as its send list), flags, waits for
//                all destinations, then reduces per token in fp32, rank-major order:
//                out[t] = add[t] + alpha * sum_r ret[send_off[r] + pos(t, r)].
//
// Reuse of the symmetric buffers needs no extra barrier: a rank can only enter dispatch
// n + 1 after every peer has pushed its counts for n + 1, which each peer does after its
// own combine n.  The count matrix is double buffered by epoch parity.  Epochs live on the
// device and are advanced by the last CTA, so the launches can be replayed from a CUDA graph.
// All waits are bounded and report through the status word.
//
// Reference behaviour: vllm_gcu/kernels/prepare_finalize.py:126-394 (get_ep_indices, pack,
// all_to_all_vd both ways, index_add_ combine), csrc/src/get_ep_indices.cpp:36.
#include "common.cuh"

namespace b200 {
namespace ep {

constexpr unsigned int kKernelId = 70;
constexpr int kMaxRanks = 8;
constexpr int kWarps = 8;

// Layout of the local meta block (ints) written by ep_dispatch and read by ep_combine and
// the host wrappers.
constexpr int kMetaRecvTotal = 0;
constexpr int kMetaSendTotal = 1;
constexpr int kMetaRecvOff = 8;    // [ep + 1]
constexpr int kMetaSendOff = 24;   // [ep + 1]
constexpr int kMetaCounts = 40;    // [ep][8]
constexpr int kMetaInts = 40 + kMaxRanks * kMaxRanks;

__device__ __forceinline__ bool wait_flag_sys(const uint32_t* flag, uint32_t want) {
  for (uint32_t it = 0; it < (1u << 22); ++it) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(flag) : "memory");
    if (static_cast<int32_t>(v - want) >= 0) return true;
    if (it > 64) __nanosleep(100);
  }
  return false;
}
__device__ __forceinline__ uint4 ld_volatile_v4(const void* p) {
  uint4 v;
  asm volatile("ld.volatile.global.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p)
               : "memory");
  return v;
}
__device__ __forceinline__ void signal_flag_sys(uint32_t* flag, uint32_t val) {
  __threadfence_system();
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(flag), "r"(val) : "memory");
}
// Count-matrix entry: (epoch << 32) | count, written with one 64-bit store.
__device__ __forceinline__ bool wait_count(const unsigned long long* p, uint32_t epoch,
                                           int* count) {
  for (uint32_t it = 0; it < (1u << 22); ++it) {
    unsigned long long v;
    asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    if (static_cast<uint32_t>(v >> 32) == epoch) {
      *count = static_cast<int>(v & 0xffffffffull);
      return true;
    }
    if (it > 64) __nanosleep(100);
  }
  return false;
}

__device__ __forceinline__ unsigned int dest_mask(const int* ids, int k, int epr, int ep) {
  unsigned int m = 0;
  for (int s = 0; s < k; ++s) {
    const int e = ids[s];
    if (e >= 0) {
      const int r = e / epr;
      if (r < ep) m |= 1u << r;
    }
  }
  return m;
}

struct RouteArgs {
  const int* topk_ids;  // [T, k]
  int T, k, epr, ep, rank;
  int* tok_idx;         // [T * min(k, ep)] token of every send row, destination-major
  int* tok_pos;         // [T, ep] position of the token in destination r's list, or -1
  const uint32_t* epoch_ptr;
  unsigned long long* cmat[kMaxRanks];  // peer r's [2][ep][ep] count matrix
};

__global__ void __launch_bounds__(1024) ep_route_kernel(const RouteArgs a) {
  __shared__ int cnts[kMaxRanks][1024];
  __shared__ int tot[kMaxRanks];
  __shared__ int off[kMaxRanks + 1];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int chunk = (a.T + 1023) / 1024;
  const int t0 = min(a.T, tid * chunk), t1 = min(a.T, t0 + chunk);
  int c[kMaxRanks];
#pragma unroll
  for (int r = 0; r < kMaxRanks; ++r) c[r] = 0;
  for (int t = t0; t < t1; ++t) {
    const unsigned int m = dest_mask(a.topk_ids + static_cast<long long>(t) * a.k, a.k, a.epr, a.ep);
#pragma unroll
    for (int r = 0; r < kMaxRanks; ++r) c[r] += (m >> r) & 1u;
  }
#pragma unroll
  for (int r = 0; r < kMaxRanks; ++r) cnts[r][tid] = c[r];
  __syncthreads();
  if (warp < a.ep) {   // exclusive scan of one destination's 1024 per-thread counts
    int run = 0;
    for (int i = lane; i < 1024; i += 32) {
      const int v = cnts[warp][i];
      int inc = v;
#pragma unroll
      for (int d = 1; d < 32; d <<= 1) {
        const int n = __shfl_up_sync(0xffffffffu, inc, d);
        if (lane >= d) inc += n;
      }
      cnts[warp][i] = run + inc - v;
      run += __shfl_sync(0xffffffffu, inc, 31);
    }
    if (lane == 0) tot[warp] = run;
  }
  __syncthreads();
  if (tid == 0) {
    int o = 0;
    for (int r = 0; r < a.ep; ++r) { off[r] = o; o += tot[r]; }
    off[a.ep] = o;
  }
  __syncthreads();
  for (int t = t0; t < t1; ++t) {
    const unsigned int m = dest_mask(a.topk_ids + static_cast<long long>(t) * a.k, a.k, a.epr, a.ep);
    for (int r = 0; r < a.ep; ++r) {
      int pos = -1;
      if ((m >> r) & 1u) {
        pos = cnts[r][tid]++;
        a.tok_idx[off[r] + pos] = t;
      }
      a.tok_pos[static_cast<long long>(t) * a.ep + r] = pos;
    }
  }
  // this rank's count vector goes into row `rank` of every peer's matrix
  if (tid < a.ep * a.ep) {
    const uint32_t epoch = *a.epoch_ptr + 1u;
    const int peer = tid / a.ep, r = tid % a.ep;
    unsigned long long* dst =
        a.cmat[peer] + (static_cast<long long>(epoch & 1u) * a.ep + a.rank) * a.ep + r;
    const unsigned long long v =
        (static_cast<unsigned long long>(epoch) << 32) | static_cast<unsigned int>(tot[r]);
    asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(dst), "l"(v) : "memory");
  }
}

__device__ __forceinline__ void copy_row(const __nv_bfloat16* src, __nv_bfloat16* dst, int nvec,
                                         int lane) {
  const uint4* s4 = reinterpret_cast<const uint4*>(src);
  uint4* d4 = reinterpret_cast<uint4*>(dst);
  constexpr int kU = 4;
  for (int v0 = lane; v0 < nvec; v0 += 32 * kU) {
    uint4 u[kU];
#pragma unroll
    for (int i = 0; i < kU; ++i)
      if (v0 + i * 32 < nvec) u[i] = s4[v0 + i * 32];
#pragma unroll
    for (int i = 0; i < kU; ++i)
      if (v0 + i * 32 < nvec) d4[v0 + i * 32] = u[i];
  }
}

struct DispatchArgs {
  const __nv_bfloat16* x;  // [T, H]
  long long ldx;
  const int* topk_ids;     // [T, k]
  const float* topk_w;     // [T, k]
  const int* tok_idx;
  int H, k, ep, rank;
  int recv_cap;            // rows of a receive buffer
  const unsigned long long* cmat_local;
  __nv_bfloat16* recv_x[kMaxRanks];
  int* recv_ids[kMaxRanks];
  float* recv_w[kMaxRanks];
  uint32_t* data_flag[kMaxRanks];  // [ep] on rank r: data_flag[r][src]
  uint32_t* epoch_ptr;
  uint32_t* done_ctr;
  int* meta;
  unsigned int* status;
};

__global__ void __launch_bounds__(kWarps * 32) ep_dispatch_kernel(const DispatchArgs a) {
  __shared__ int C[kMaxRanks][kMaxRanks];
  __shared__ int send_off[kMaxRanks + 1], recv_off[kMaxRanks + 1], dst_base[kMaxRanks];
  __shared__ unsigned int abort_flag;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int ep = a.ep, rank = a.rank;
  const uint32_t epoch = *reinterpret_cast<volatile uint32_t*>(a.epoch_ptr) + 1u;
  if (tid == 0) abort_flag = 0u;
  __syncthreads();
  if (tid < ep * ep) {
    int cnt = 0;
    if (!wait_count(a.cmat_local + static_cast<long long>(epoch & 1u) * ep * ep + tid, epoch,
                    &cnt)) {
      report_status(a.status, kStatusFlagTimeout, kKernelId, 0x100u + tid);
      abort_flag = 1u;
    }
    C[tid / ep][tid % ep] = cnt;
  }
  __syncthreads();
  if (abort_flag != 0u) return;
  if (tid == 0) {
    int so = 0, ro = 0;
    for (int r = 0; r < ep; ++r) {
      send_off[r] = so; so += C[rank][r];
      recv_off[r] = ro; ro += C[r][rank];
      int b = 0;
      for (int s = 0; s < rank; ++s) b += C[s][r];
      dst_base[r] = b;
    }
    send_off[ep] = so;
    recv_off[ep] = ro;
    if (ro > a.recv_cap) {   // cannot happen when recv_cap >= ep * max tokens per rank
      report_status(a.status, kStatusBounds, kKernelId, 0x110u);
      abort_flag = 1u;
    }
    if (blockIdx.x == 0) {
      a.meta[kMetaRecvTotal] = ro;
      a.meta[kMetaSendTotal] = so;
      for (int r = 0; r <= ep; ++r) {
        a.meta[kMetaRecvOff + r] = recv_off[r];
        a.meta[kMetaSendOff + r] = send_off[r];
      }
      for (int s = 0; s < ep; ++s)
        for (int d = 0; d < ep; ++d) a.meta[kMetaCounts + s * kMaxRanks + d] = C[s][d];
    }
  }
  __syncthreads();
  if (abort_flag != 0u) return;

  const int S = send_off[ep];
  const int nvec = a.H / 8;
  for (int i = blockIdx.x * kWarps + warp; i < S; i += gridDim.x * kWarps) {
    int r = 0;
    while (r + 1 < ep && i >= send_off[r + 1]) ++r;
    const int t = a.tok_idx[i];
    const long long row = dst_base[r] + (i - send_off[r]);
    copy_row(a.x + static_cast<long long>(t) * a.ldx, a.recv_x[r] + row * a.H, nvec, lane);
    if (lane < a.k) {
      a.recv_ids[r][row * a.k + lane] = a.topk_ids[static_cast<long long>(t) * a.k + lane];
      a.recv_w[r][row * a.k + lane] = a.topk_w[static_cast<long long>(t) * a.k + lane];
    }
  }
  __syncthreads();
  if (tid == 0) {
    __threadfence_system();
    if (atomicAdd(a.done_ctr, 1u) == gridDim.x - 1) {
      *a.done_ctr = 0u;
      __threadfence();
      for (int r = 0; r < ep; ++r) signal_flag_sys(a.data_flag[r] + rank, epoch);
      *reinterpret_cast<volatile uint32_t*>(a.epoch_ptr) = epoch;
    }
  }
  if (blockIdx.x == 0 && tid < ep) {
    if (!wait_flag_sys(a.data_flag[rank] + tid, epoch))
      report_status(a.status, kStatusFlagTimeout, kKernelId, 0x120u + tid);
  }
}

struct CombineArgs {
  const __nv_bfloat16* y;   // [>= recv_total, H] expert output per received row
  long long ldy;
  const int* tok_pos;       // [T, ep]
  const __nv_bfloat16* add; // optional [T, H] (shared-expert output)
  long long ld_add;
  __nv_bfloat16* out;       // [T, H]
  long long ldo;
  float alpha;
  int T, H, ep, rank;
  const int* meta;
  __nv_bfloat16* ret[kMaxRanks];
  uint32_t* ret_flag[kMaxRanks];
  uint32_t* epoch_ptr;
  uint32_t* done_ctr;
  unsigned int* status;
};

__global__ void __launch_bounds__(kWarps * 32) ep_combine_kernel(const CombineArgs a) {
  __shared__ int send_off[kMaxRanks + 1], recv_off[kMaxRanks + 1], ret_base[kMaxRanks];
  __shared__ unsigned int abort_flag;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int ep = a.ep, rank = a.rank;
  const uint32_t epoch = *reinterpret_cast<volatile uint32_t*>(a.epoch_ptr) + 1u;
  if (tid == 0) {
    abort_flag = 0u;
    for (int r = 0; r <= ep; ++r) {
      send_off[r] = a.meta[kMetaSendOff + r];
      recv_off[r] = a.meta[kMetaRecvOff + r];
    }
    for (int s = 0; s < ep; ++s) {   // where this rank's block starts in source s's send list
      int b = 0;
      for (int r = 0; r < rank; ++r) b += a.meta[kMetaCounts + s * kMaxRanks + r];
      ret_base[s] = b;
    }
  }
  __syncthreads();
  const int R = recv_off[ep];
  const int nvec = a.H / 8;
  for (int i = blockIdx.x * kWarps + warp; i < R; i += gridDim.x * kWarps) {
    int s = 0;
    while (s + 1 < ep && i >= recv_off[s + 1]) ++s;
    const long long row = ret_base[s] + (i - recv_off[s]);
    copy_row(a.y + static_cast<long long>(i) * a.ldy, a.ret[s] + row * a.H, nvec, lane);
  }
  __syncthreads();
  if (tid == 0) {
    __threadfence_system();
    if (atomicAdd(a.done_ctr, 1u) == gridDim.x - 1) {
      *a.done_ctr = 0u;
      __threadfence();
      for (int s = 0; s < ep; ++s) signal_flag_sys(a.ret_flag[s] + rank, epoch);
      *reinterpret_cast<volatile uint32_t*>(a.epoch_ptr) = epoch;
    }
  }
  // every destination's rows must have landed before any token is reduced
  if (tid < ep && !wait_flag_sys(a.ret_flag[rank] + tid, epoch)) {
    report_status(a.status, kStatusFlagTimeout, kKernelId, 0x200u + tid);
    abort_flag = 1u;
  }
  __syncthreads();
  if (abort_flag != 0u) return;

  const __nv_bfloat16* ret_local = a.ret[rank];
  for (int t = blockIdx.x * kWarps + warp; t < a.T; t += gridDim.x * kWarps) {
    int my_pos = -1;
    if (lane < ep) my_pos = a.tok_pos[static_cast<long long>(t) * ep + lane];
    for (int v = lane; v < nvec; v += 32) {
      float acc[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[i] = 0.0f;
      for (int r = 0; r < ep; ++r) {
        const int pos = __shfl_sync(0xffffffffu, my_pos, r);
        if (pos < 0) continue;
        const uint4 u = ld_volatile_v4(ret_local + (static_cast<long long>(send_off[r]) + pos) * a.H +
                                       v * 8);
        const float2 f0 = unpack_bf16x2(u.x), f1 = unpack_bf16x2(u.y), f2 = unpack_bf16x2(u.z),
                     f3 = unpack_bf16x2(u.w);
        acc[0] += f0.x; acc[1] += f0.y; acc[2] += f1.x; acc[3] += f1.y;
        acc[4] += f2.x; acc[5] += f2.y; acc[6] += f3.x; acc[7] += f3.y;
      }
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[i] *= a.alpha;
      if (a.add != nullptr) {
        const uint4 u = *reinterpret_cast<const uint4*>(a.add + static_cast<long long>(t) * a.ld_add + v * 8);
        const float2 f0 = unpack_bf16x2(u.x), f1 = unpack_bf16x2(u.y), f2 = unpack_bf16x2(u.z),
                     f3 = unpack_bf16x2(u.w);
        acc[0] += f0.x; acc[1] += f0.y; acc[2] += f1.x; acc[3] += f1.y;
        acc[4] += f2.x; acc[5] += f2.y; acc[6] += f3.x; acc[7] += f3.y;
      }
      uint4 o;
      o.x = pack_bf16x2(acc[0], acc[1]);
      o.y = pack_bf16x2(acc[2], acc[3]);
      o.z = pack_bf16x2(acc[4], acc[5]);
      o.w = pack_bf16x2(acc[6], acc[7]);
      *reinterpret_cast<uint4*>(a.out + static_cast<long long>(t) * a.ldo + v * 8) = o;
    }
  }
}

}  // namespace ep
}  // namespace b200

using namespace b200;
using namespace b200::ep;

B200_API int b200_ep_meta_ints() { return kMetaInts; }

// Routing for the fused dispatch.  tok_idx needs T * min(k, ep) ints, tok_pos T * ep ints.
// cmat: ep peer-visible addresses of the [2][ep][ep] 64-bit count matrices; epoch_ptr is the
// local epoch word that b200_ep_dispatch advances.  ep <= 8, k <= 32.
B200_API int b200_ep_route(const int* topk_ids, int T, int k, int experts_per_rank, int ep,
                           int rank, int* tok_idx, int* tok_pos, void* const* cmat,
                           const void* epoch_ptr, void* stream) {
  if (ep < 1 || ep > kMaxRanks || k < 1 || k > 32 || experts_per_rank < 1 || rank < 0 ||
      rank >= ep || T < 0)
    return -2;
  RouteArgs a;
  a.topk_ids = topk_ids; a.T = T; a.k = k; a.epr = experts_per_rank; a.ep = ep; a.rank = rank;
  a.tok_idx = tok_idx; a.tok_pos = tok_pos;
  a.epoch_ptr = static_cast<const uint32_t*>(epoch_ptr);
  for (int i = 0; i < kMaxRanks; ++i)
    a.cmat[i] = i < ep ? static_cast<unsigned long long*>(cmat[i]) : nullptr;
  ep_route_kernel<<<1, 1024, 0, static_cast<cudaStream_t>(stream)>>>(a);
  return static_cast<int>(cudaGetLastError());
}

// Dispatch (must follow b200_ep_route on the same stream).  Receive buffers on every rank:
// recv_x [recv_cap, H] bf16, recv_ids [recv_cap, k] int32, recv_w [recv_cap, k] fp32,
// data_flag [ep] words; recv_cap >= the largest number of rows a rank can receive
// (ep * max tokens per rank).  meta: b200_ep_meta_ints() local ints; meta[0] is the number
// of received rows (device scalar for the expert kernels).  H must be a multiple of 8.
B200_API int b200_ep_dispatch(const void* x, long long ldx, const int* topk_ids,
                              const float* topk_w, const int* tok_idx, int T, int H, int k, int ep,
                              int rank, int recv_cap, const void* cmat_local,
                              void* const* recv_x, void* const* recv_ids, void* const* recv_w,
                              void* const* data_flag, void* epoch_ptr, void* done_ctr, int* meta,
                              void* stream) {
  if (ep < 1 || ep > kMaxRanks || k < 1 || k > 32 || (H % 8) != 0 || (ldx % 8) != 0 || rank < 0 ||
      rank >= ep)
    return -2;
  DispatchArgs a;
  a.x = static_cast<const __nv_bfloat16*>(x); a.ldx = ldx; a.topk_ids = topk_ids;
  a.topk_w = topk_w; a.tok_idx = tok_idx; a.H = H; a.k = k; a.ep = ep; a.rank = rank;
  a.recv_cap = recv_cap;
  a.cmat_local = static_cast<const unsigned long long*>(cmat_local);
  for (int i = 0; i < kMaxRanks; ++i) {
    a.recv_x[i] = i < ep ? static_cast<__nv_bfloat16*>(recv_x[i]) : nullptr;
    a.recv_ids[i] = i < ep ? static_cast<int*>(recv_ids[i]) : nullptr;
    a.recv_w[i] = i < ep ? static_cast<float*>(recv_w[i]) : nullptr;
    a.data_flag[i] = i < ep ? static_cast<uint32_t*>(data_flag[i]) : nullptr;
  }
  a.epoch_ptr = static_cast<uint32_t*>(epoch_ptr);
  a.done_ctr = static_cast<uint32_t*>(done_ctr);
  a.meta = meta;
  a.status = status_ptr();
  const long long rows = static_cast<long long>(T) * (k < ep ? k : ep);
  long long grid = (rows + kWarps - 1) / kWarps;
  if (grid < 1) grid = 1;
  if (grid > sm_count()) grid = sm_count();
  ep_dispatch_kernel<<<static_cast<int>(grid), kWarps * 32, 0, static_cast<cudaStream_t>(stream)>>>(a);
  return static_cast<int>(cudaGetLastError());
}

// Combine.  y [rows, H]: one expert-output row per received row (rows >= meta[0]);
// ret: ep peer-visible [T_cap * min(k, ep), H] return buffers; ret_flag: [ep] words per rank.
// out[t] = add[t] + alpha * sum over the destinations of token t, accumulated in fp32 in rank
// order.  max_rows bounds the rows this rank may have received (sizes the grid only).
B200_API int b200_ep_combine(const void* y, long long ldy, int max_rows, const int* tok_pos,
                             const void* add, long long ld_add, void* out, long long ldo,
                             float alpha, int T, int H, int ep, int rank, const int* meta,
                             void* const* ret, void* const* ret_flag, void* epoch_ptr,
                             void* done_ctr, void* stream) {
  if (ep < 1 || ep > kMaxRanks || (H % 8) != 0 || (ldy % 8) != 0 || (ldo % 8) != 0 ||
      (ld_add % 8) != 0 || rank < 0 || rank >= ep)
    return -2;
  CombineArgs a;
  a.y = static_cast<const __nv_bfloat16*>(y); a.ldy = ldy; a.tok_pos = tok_pos;
  a.add = static_cast<const __nv_bfloat16*>(add); a.ld_add = ld_add;
  a.out = static_cast<__nv_bfloat16*>(out); a.ldo = ldo; a.alpha = alpha;
  a.T = T; a.H = H; a.ep = ep; a.rank = rank; a.meta = meta;
  for (int i = 0; i < kMaxRanks; ++i) {
    a.ret[i] = i < ep ? static_cast<__nv_bfloat16*>(ret[i]) : nullptr;
    a.ret_flag[i] = i < ep ? static_cast<uint32_t*>(ret_flag[i]) : nullptr;
  }
  a.epoch_ptr = static_cast<uint32_t*>(epoch_ptr);
  a.done_ctr = static_cast<uint32_t*>(done_ctr);
  a.status = status_ptr();
  // All CTAs wait for the peers after pushing, so the grid must be resident at once.
  long long work = max_rows > T ? max_rows : T;
  long long grid = (work + kWarps - 1) / kWarps;
  if (grid < 1) grid = 1;
  if (grid > sm_count()) grid = sm_count();
  ep_combine_kernel<<<static_cast<int>(grid), kWarps * 32, 0, static_cast<cudaStream_t>(stream)>>>(a);
  return static_cast<int>(cudaGetLastError());
}
