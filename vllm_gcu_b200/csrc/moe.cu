// Mixture-of-experts routing and data movement kernels for sm_100a.
//
//   moe_topk          softmax / sigmoid scoring, optional grouped selection with bias
//                     correction (DeepSeek), top-k, renormalisation, scaling; one warp per
//                     token, scores staged in shared memory
//   moe_align         counting sort of (token, slot) pairs by (local) expert, each expert
//                     segment padded to the 128-row GEMM tile; produces the sorted pair ids,
//                     the expert of every tile, the padded row count and the inverse map
//   moe_permute       gathers activation rows into expert-sorted order (the A operand of
//                     the grouped tcgen05 GEMM in gemm_bf16.cu)
//   moe_unpermute_sum out[t] = sum_slots y[pos(t, slot)] (+ shared-expert output); the top-k
//                     weights were already applied by the second GEMM's epilogue
//   get_ep_indices    per destination rank, the tokens that have an expert there
//
// All row counts that depend on routing stay on the device, so the whole MoE layer can be
// captured in a CUDA graph with static buffer sizes (the reference threads a device scalar
// `expert_num_tokens` through its kernels for the same reason,
// vllm_gcu/kernels/modular_experts.py:81-288).
//
// Reference ops: csrc/src/topk_softmax.cpp:32, fused_grouped_topk.cpp:35,
// moe_align_block_size.cpp:37 (+ _pad / exts_ variants), moe_sum.cpp:75,
// get_ep_indices.cpp:36, eplb_map_to_physical_and_record.cpp:36.
#include "common.cuh"

namespace b200 {
namespace moe {

constexpr unsigned int kKernelId = 60;
constexpr int kTileM = 128;

struct TopkArgs {
  const void* gating;     // [T, E]
  const float* bias;      // [E] or null
  float* weights;         // [T, k]
  int* ids;               // [T, k]
  const int* log2phy;     // optional [E, R] logical -> physical replicas
  const int* replica_cnt; // optional [E]
  int* load;              // optional [E_phys] load histogram
  long long ldg;
  int T, E, k, n_group, topk_group, R;
  int sigmoid, renorm;
  float scale;
  int dtype;              // 0 bf16, 1 fp16, 2 fp32
};

__device__ __forceinline__ float load_gate(const void* p, long long i, int dtype) {
  if (dtype == 0) return __bfloat162float(static_cast<const __nv_bfloat16*>(p)[i]);
  if (dtype == 1) return __half2float(static_cast<const __half*>(p)[i]);
  return static_cast<const float*>(p)[i];
}

// 4 warps per CTA, one token per warp.  Shared: per warp 2 * E floats.
__global__ void __launch_bounds__(128) moe_topk_kernel(const TopkArgs a) {
  extern __shared__ float sm[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x * 4 + warp;
  if (t >= a.T) return;
  float* sc = sm + warp * 2 * a.E;   // unbiased scores
  float* sel = sc + a.E;             // selection scores
  const long long base = static_cast<long long>(t) * a.ldg;

  float mx = -INFINITY;
  for (int e = lane; e < a.E; e += 32) {
    const float g = load_gate(a.gating, base + e, a.dtype);
    sc[e] = g;
    mx = fmaxf(mx, g);
  }
  mx = warp_max(mx);
  if (a.sigmoid) {
    for (int e = lane; e < a.E; e += 32) sc[e] = 1.0f / (1.0f + __expf(-sc[e]));
  } else {
    float sum = 0.0f;
    for (int e = lane; e < a.E; e += 32) {
      const float p = __expf(sc[e] - mx);
      sc[e] = p;
      sum += p;
    }
    sum = warp_sum(sum);
    const float inv = 1.0f / sum;
    for (int e = lane; e < a.E; e += 32) sc[e] *= inv;
  }
  for (int e = lane; e < a.E; e += 32) sel[e] = sc[e] + (a.bias ? a.bias[e] : 0.0f);
  __syncwarp();

  if (a.n_group > 1) {
    const int gs = a.E / a.n_group;
    // group score: sum of top-2 (with bias) or max (without)
    float gscore = -INFINITY;
    if (lane < a.n_group) {
      float m1 = -INFINITY, m2 = -INFINITY;
      for (int j = 0; j < gs; ++j) {
        const float v = sel[lane * gs + j];
        if (v > m1) { m2 = m1; m1 = v; } else if (v > m2) { m2 = v; }
      }
      gscore = a.bias ? m1 + m2 : m1;
    }
    // keep the topk_group best groups (ties: lower index first)
    unsigned keep = 0;
    for (int r = 0; r < a.topk_group; ++r) {
      float best = (keep >> lane) & 1u ? -INFINITY : gscore;
      int bi = lane;
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const float ob = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (ob > best || (ob == best && oi < bi)) { best = ob; bi = oi; }
      }
      keep |= 1u << bi;
    }
    for (int e = lane; e < a.E; e += 32)
      if (!((keep >> (e / gs)) & 1u)) sel[e] = -INFINITY;
    __syncwarp();
  }

  float wsum = 0.0f;
  float my_w = 0.0f;
  int my_id = 0;
  for (int r = 0; r < a.k; ++r) {
    float best = -INFINITY;
    int bi = 0x7fffffff;
    for (int e = lane; e < a.E; e += 32) {
      const float v = sel[e];
      if (v > best) { best = v; bi = e; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ob > best || (ob == best && oi < bi)) { best = ob; bi = oi; }
    }
    if (bi >= a.E) bi = 0;  // fewer than k selectable experts
    const float w = sc[bi];
    wsum += w;
    if (lane == r) { my_w = w; my_id = bi; }
    __syncwarp();
    if (lane == 0) sel[bi] = -INFINITY;
    __syncwarp();
  }
  if (lane < a.k) {
    float w = my_w;
    if (a.renorm) w = w / (wsum + 1e-20f);
    w *= a.scale;
    int id = my_id;
    if (a.log2phy != nullptr) {
      const int pos = t * a.k + lane;
      const int rc = a.replica_cnt ? max(1, a.replica_cnt[id]) : 1;
      id = a.log2phy[static_cast<long long>(id) * a.R + pos % rc];
      if (a.load != nullptr) atomicAdd(&a.load[id], 1);
    }
    a.weights[static_cast<long long>(t) * a.k + lane] = w;
    a.ids[static_cast<long long>(t) * a.k + lane] = id;
  }
}

// ---------------------------------------------------------------------------
struct AlignArgs {
  const int* topk_ids;      // [T, k]
  const int* expert_map;    // optional [E_global] -> local id or -1
  const int* valid_tokens;  // optional device scalar: only the first n tokens count
  int* sorted_ids;          // [cap] pair index (token * k + slot) or sentinel numel
  int* expert_ids;          // [cap / 128] expert of every tile, -1 beyond the valid tiles
  int* num_post_pad;        // [1]
  int* pos_of;              // [T * k] position of each pair, -1 if dropped
  int numel, k, num_local_experts, cap;
  unsigned int* status;
};

__global__ void __launch_bounds__(1024) moe_align_kernel(const AlignArgs a) {
  extern __shared__ int smi[];
  int* count = smi;                              // [E]
  int* offset = smi + a.num_local_experts;       // [E + 1] padded exclusive offsets
  int* cursor = offset + a.num_local_experts + 1;
  const int E = a.num_local_experts;
  const int n = a.valid_tokens ? min(a.numel, *a.valid_tokens * a.k) : a.numel;
  for (int e = threadIdx.x; e < E; e += blockDim.x) { count[e] = 0; cursor[e] = 0; }
  __syncthreads();
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    int e = a.topk_ids[i];
    if (a.expert_map != nullptr) e = (e >= 0) ? a.expert_map[e] : -1;
    if (e >= 0 && e < E) atomicAdd(&count[e], 1);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int off = 0;
    for (int e = 0; e < E; ++e) {
      offset[e] = off;
      off += (count[e] + kTileM - 1) / kTileM * kTileM;
    }
    offset[E] = off;
    if (off > a.cap) {
      report_status(a.status, kStatusBounds, kKernelId, static_cast<unsigned>(off));
      off = 0;  // nothing valid: consumers skip every tile
      for (int e = 0; e <= E; ++e) offset[e] = 0;
    }
    *a.num_post_pad = off;
  }
  __syncthreads();
  const int total = offset[E];
  for (int i = threadIdx.x; i < a.cap; i += blockDim.x) a.sorted_ids[i] = a.numel;
  for (int b = threadIdx.x; b < a.cap / kTileM; b += blockDim.x) {
    const int row = b * kTileM;
    int e = -1;
    if (row < total) {
      int lo = 0, hi = E;  // last e with offset[e] <= row
      while (hi - lo > 1) {
        const int mid = (lo + hi) >> 1;
        if (offset[mid] <= row) lo = mid; else hi = mid;
      }
      e = lo;
    }
    a.expert_ids[b] = e;
  }
  __syncthreads();
  for (int i = threadIdx.x; i < a.numel; i += blockDim.x) {
    int pos = -1;
    if (i < n && total > 0) {
      int e = a.topk_ids[i];
      if (a.expert_map != nullptr) e = (e >= 0) ? a.expert_map[e] : -1;
      if (e >= 0 && e < E) {
        pos = offset[e] + atomicAdd(&cursor[e], 1);
        a.sorted_ids[pos] = i;
      }
    }
    a.pos_of[i] = pos;
  }
}

// A_sorted[pos] = x[sorted_ids[pos] / k]; padding rows are zeroed.  One CTA per row.
template <typename T>
__global__ void __launch_bounds__(256)
    moe_permute_kernel(const T* x, long long ldx, T* out, long long ldo, const int* sorted_ids,
                       const int* num_post_pad, int numel, int k, int H) {
  const int pos = blockIdx.x;
  if (pos >= *num_post_pad) return;
  const int pair = sorted_ids[pos];
  uint4* dst = reinterpret_cast<uint4*>(out + static_cast<long long>(pos) * ldo);
  const int nvec = H >> 3;
  if (pair >= numel) {
    for (int v = threadIdx.x; v < nvec; v += blockDim.x) dst[v] = make_uint4(0, 0, 0, 0);
    return;
  }
  const uint4* src = reinterpret_cast<const uint4*>(x + static_cast<long long>(pair / k) * ldx);
  for (int v = threadIdx.x; v < nvec; v += blockDim.x) dst[v] = src[v];
}

// out[t] = (add ? add[t] : 0) + alpha * sum_s y[pos_of[t * k + s]]   (fp32 accumulation)
template <typename T>
__global__ void __launch_bounds__(256)
    moe_unpermute_sum_kernel(const T* y, long long ldy, const int* pos_of, const T* add,
                             long long lda, T* out, long long ldo, const int* valid_tokens, int k,
                             int H, float alpha) {
  const int t = blockIdx.x;
  if (valid_tokens != nullptr && t >= *valid_tokens) return;
  const int nvec = H >> 3;
  for (int v = threadIdx.x; v < nvec; v += blockDim.x) {
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int s = 0; s < k; ++s) {
      const int pos = pos_of[static_cast<long long>(t) * k + s];
      if (pos < 0) continue;
      float f[8];
      vec8_load<T>(y + static_cast<long long>(pos) * ldy + v * 8, f);
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[i] += f[i];
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] *= alpha;
    if (add != nullptr) {
      float f[8];
      vec8_load<T>(add + static_cast<long long>(t) * lda + v * 8, f);
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[i] += f[i];
    }
    vec8_store<T>(out + static_cast<long long>(t) * ldo + v * 8, acc);
  }
}

// Per sorted row: the routing weight of its (token, slot) pair (0 for padding rows).
__global__ void moe_row_weights_kernel(const int* sorted_ids, const float* topk_w,
                                       const int* num_post_pad, float* row_w, int numel, int cap) {
  const int pos = blockIdx.x * blockDim.x + threadIdx.x;
  if (pos >= cap) return;
  float w = 0.0f;
  if (pos < *num_post_pad) {
    const int pair = sorted_ids[pos];
    if (pair < numel) w = topk_w[pair];
  }
  row_w[pos] = w;
}

// get_ep_indices: one CTA; count[r] = #tokens with an expert on rank r, indices rank-major.
__global__ void __launch_bounds__(1024)
    ep_indices_kernel(const int* topk_ids, int T, int k, int experts_per_rank, int ep,
                      int* ep_count, int* ep_token_indices, int* total) {
  __shared__ int cnt[64];
  __shared__ int off[65];
  __shared__ int cur[64];
  for (int r = threadIdx.x; r < ep; r += blockDim.x) { cnt[r] = 0; cur[r] = 0; }
  __syncthreads();
  for (int t = threadIdx.x; t < T; t += blockDim.x) {
    unsigned long long mask = 0;
    for (int s = 0; s < k; ++s) {
      const int e = topk_ids[t * k + s];
      if (e >= 0) mask |= 1ull << min(63, e / experts_per_rank);
    }
    for (int r = 0; r < ep; ++r)
      if ((mask >> r) & 1ull) atomicAdd(&cnt[r], 1);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int o = 0;
    for (int r = 0; r < ep; ++r) { off[r] = o; o += cnt[r]; ep_count[r] = cnt[r]; }
    off[ep] = o;
    *total = o;
  }
  __syncthreads();
  for (int t = threadIdx.x; t < T; t += blockDim.x) {
    unsigned long long mask = 0;
    for (int s = 0; s < k; ++s) {
      const int e = topk_ids[t * k + s];
      if (e >= 0) mask |= 1ull << min(63, e / experts_per_rank);
    }
    for (int r = 0; r < ep; ++r)
      if ((mask >> r) & 1ull) ep_token_indices[off[r] + atomicAdd(&cur[r], 1)] = t;
  }
}

}  // namespace moe
}  // namespace b200

using namespace b200;
using namespace b200::moe;

// Routing.  n_group <= 1 gives plain top-k; bias != null enables the DeepSeek bias-corrected
// grouped selection.  log2phy / replica_cnt / load (all optional) apply the EPLB
// logical -> physical mapping and record the load histogram.  E <= 1024, k <= 32,
// n_group <= 32.
B200_API int b200_moe_topk(const void* gating, long long ldg, const float* bias, float* weights,
                           int* ids, int T, int E, int k, int n_group, int topk_group,
                           int sigmoid, int renorm, float scale, const int* log2phy, int R,
                           const int* replica_cnt, int* load, int dtype, void* stream) {
  if (T <= 0) return 0;
  if (E <= 0 || E > 1024 || k <= 0 || k > 32 || n_group > 32) return -2;
  if (n_group > 1 && (E % n_group) != 0) return -2;
  TopkArgs a;
  a.gating = gating; a.bias = bias; a.weights = weights; a.ids = ids; a.log2phy = log2phy;
  a.replica_cnt = replica_cnt; a.load = load; a.ldg = ldg; a.T = T; a.E = E; a.k = k;
  a.n_group = n_group; a.topk_group = topk_group; a.R = R; a.sigmoid = sigmoid;
  a.renorm = renorm; a.scale = scale; a.dtype = dtype;
  const size_t smem = static_cast<size_t>(4) * 2 * E * sizeof(float);
  moe_topk_kernel<<<(T + 3) / 4, 128, smem, static_cast<cudaStream_t>(stream)>>>(a);
  return static_cast<int>(cudaGetLastError());
}

// cap must be a multiple of 128 and >= numel + num_local_experts * 127 rounded up.
B200_API int b200_moe_align(const int* topk_ids, const int* expert_map, const int* valid_tokens,
                            int* sorted_ids, int* expert_ids, int* num_post_pad, int* pos_of,
                            int numel, int k, int num_local_experts, int cap, void* stream) {
  if (cap <= 0 || (cap % kTileM) != 0 || num_local_experts <= 0 || num_local_experts > 2048)
    return -2;
  AlignArgs a;
  a.topk_ids = topk_ids; a.expert_map = expert_map; a.valid_tokens = valid_tokens;
  a.sorted_ids = sorted_ids; a.expert_ids = expert_ids; a.num_post_pad = num_post_pad;
  a.pos_of = pos_of; a.numel = numel; a.k = k; a.num_local_experts = num_local_experts;
  a.cap = cap; a.status = status_ptr();
  const size_t smem = static_cast<size_t>(3 * num_local_experts + 1) * sizeof(int);
  moe_align_kernel<<<1, 1024, smem, static_cast<cudaStream_t>(stream)>>>(a);
  return static_cast<int>(cudaGetLastError());
}

B200_API int b200_moe_permute(const void* x, long long ldx, void* out, long long ldo,
                              const int* sorted_ids, const int* num_post_pad, int numel, int k,
                              int H, int cap, int dtype, void* stream) {
  if (cap <= 0) return 0;
  if ((H % 8) != 0) return -2;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (dtype == 0)
    moe_permute_kernel<__nv_bfloat16><<<cap, 256, 0, s>>>(
        static_cast<const __nv_bfloat16*>(x), ldx, static_cast<__nv_bfloat16*>(out), ldo,
        sorted_ids, num_post_pad, numel, k, H);
  else if (dtype == 1)
    moe_permute_kernel<__half><<<cap, 256, 0, s>>>(static_cast<const __half*>(x), ldx,
                                                   static_cast<__half*>(out), ldo, sorted_ids,
                                                   num_post_pad, numel, k, H);
  else
    return -8;
  return static_cast<int>(cudaGetLastError());
}

B200_API int b200_moe_row_weights(const int* sorted_ids, const float* topk_w,
                                  const int* num_post_pad, float* row_w, int numel, int cap,
                                  void* stream) {
  if (cap <= 0) return 0;
  moe_row_weights_kernel<<<(cap + 255) / 256, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      sorted_ids, topk_w, num_post_pad, row_w, numel, cap);
  return static_cast<int>(cudaGetLastError());
}

B200_API int b200_moe_unpermute_sum(const void* y, long long ldy, const int* pos_of,
                                    const void* add, long long lda, void* out, long long ldo,
                                    const int* valid_tokens, int T, int k, int H, float alpha,
                                    int dtype, void* stream) {
  if (T <= 0) return 0;
  if ((H % 8) != 0) return -2;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (dtype == 0)
    moe_unpermute_sum_kernel<__nv_bfloat16><<<T, 256, 0, s>>>(
        static_cast<const __nv_bfloat16*>(y), ldy, pos_of, static_cast<const __nv_bfloat16*>(add),
        lda, static_cast<__nv_bfloat16*>(out), ldo, valid_tokens, k, H, alpha);
  else if (dtype == 1)
    moe_unpermute_sum_kernel<__half><<<T, 256, 0, s>>>(
        static_cast<const __half*>(y), ldy, pos_of, static_cast<const __half*>(add), lda,
        static_cast<__half*>(out), ldo, valid_tokens, k, H, alpha);
  else
    return -8;
  return static_cast<int>(cudaGetLastError());
}

B200_API int b200_get_ep_indices(const int* topk_ids, int T, int k, int experts_per_rank, int ep,
                                 int* ep_count, int* ep_token_indices, int* total, void* stream) {
  if (ep <= 0 || ep > 64) return -2;
  ep_indices_kernel<<<1, 1024, 0, static_cast<cudaStream_t>(stream)>>>(
      topk_ids, T, k, experts_per_rank, ep, ep_count, ep_token_indices, total);
  return static_cast<int>(cudaGetLastError());
}
