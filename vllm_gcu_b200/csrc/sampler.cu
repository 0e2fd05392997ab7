// Token sampling for sm_100a: greedy argmax and a fused
// temperature / top-k / top-p / Gumbel-max sampler that never sorts the
// vocabulary (radix selection on order-preserving keys), plus the in-place
// top-k/top-p mask.  One CTA per row; the row stays in L2 between passes.
//
// Reference ops: csrc/src/top_k_top_p.cpp:16,
// csrc/src/topk_topp_random_sampler_from_logits.cpp:29 (argmax(probs / q) with
// q ~ Exp(1), vllm_gcu/kernels/sampler.py:102-134).
#include "common.cuh"

namespace b200 {
namespace sampler {

constexpr int kThreads = 1024;

template <typename T>
__device__ __forceinline__ float ldf(const void* p, long long i) {
  return to_f32<T>(static_cast<const T*>(p)[i]);
}

__device__ __forceinline__ uint32_t order_key(float f) {
  const uint32_t u = __float_as_uint(f);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

__device__ __forceinline__ uint64_t mix64(uint64_t z) {
  z += 0x9E3779B97F4A7C15ull;
  z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
  z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
  return z ^ (z >> 31);
}
// Exp(1) variate for (seed, counter).
__device__ __forceinline__ float exp_noise(uint64_t seed, uint64_t ctr) {
  const uint64_t r = mix64(seed ^ mix64(ctr));
  const float u = (static_cast<float>(r >> 40) + 0.5f) * (1.0f / 16777216.0f);  // (0, 1)
  return -__logf(u);
}

// Calls f(index, value) for every element of a row; 16-byte vector loads when the row start is
// 16-byte aligned (8 bf16 / fp16 or 4 fp32 per load), scalar loads otherwise.  Every thread of
// the block must call it; the order of the calls within a thread is ascending in index.
template <typename T, typename F>
__device__ __forceinline__ void for_each_elem(const void* row, int V, F f) {
  constexpr int kVec = 16 / sizeof(T);
  const T* p = static_cast<const T*>(row);
  if ((reinterpret_cast<uintptr_t>(p) & 15) == 0) {
    const int nv = V / kVec;
    for (int v = threadIdx.x; v < nv; v += blockDim.x) {
      const uint4 u = *reinterpret_cast<const uint4*>(p + v * kVec);
      const T* e = reinterpret_cast<const T*>(&u);
#pragma unroll
      for (int j = 0; j < kVec; ++j) f(v * kVec + j, to_f32<T>(e[j]));
    }
    for (int i = nv * kVec + threadIdx.x; i < V; i += blockDim.x) f(i, to_f32<T>(p[i]));
  } else {
    for (int i = threadIdx.x; i < V; i += blockDim.x) f(i, to_f32<T>(p[i]));
  }
}

struct ArgMax {
  float v;
  int i;
};
__device__ __forceinline__ ArgMax amax_combine(ArgMax a, ArgMax b) {
  if (b.v > a.v || (b.v == a.v && b.i < a.i)) return b;
  return a;
}
__device__ __forceinline__ ArgMax block_argmax(ArgMax x, ArgMax* red) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    ArgMax y;
    y.v = __shfl_xor_sync(0xffffffffu, x.v, o);
    y.i = __shfl_xor_sync(0xffffffffu, x.i, o);
    x = amax_combine(x, y);
  }
  __syncthreads();
  if (lane == 0) red[warp] = x;
  __syncthreads();
  const int nw = (blockDim.x + 31) >> 5;
  ArgMax t = lane < nw ? red[lane] : ArgMax{-INFINITY, 0x7fffffff};
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    ArgMax y;
    y.v = __shfl_xor_sync(0xffffffffu, t.v, o);
    y.i = __shfl_xor_sync(0xffffffffu, t.i, o);
    t = amax_combine(t, y);
  }
  return t;
}

// Largest key c such that sum over {key >= c, key >= floor_key} of w >= target.
// w = 1 (COUNT) or exp(x - row_max) (weights).  All threads get the result.
//   iter(f)  calls f(index, x) for the elements this thread owns (x already divided by T).
//   frac > 0 the target is frac * (total weight of the elements >= floor_key), taken from the
//            first histogram, so no separate pass computes the total.
//   REP      the first pass (sign + exponent byte, where almost every logit of a row falls
//            into a handful of bins) adds into 16 copies of the histogram, one per lane group,
//            laid out so that the copies of a bin sit in 16 different banks: 32 lanes hitting
//            one bin serialise two deep instead of 32 deep.  rep = 4096 floats.
template <bool COUNT, bool REP, typename Iter>
__device__ uint32_t radix_select(Iter iter, float row_max, uint32_t floor_key, float target,
                                 float frac, float* hist, float* rep, uint32_t* sh_u,
                                 float* sh_f) {
  uint32_t prefix = 0, mask = 0;
  float above = 0.0f;
  for (int byte = 3; byte >= 0; --byte) {
    for (int i = threadIdx.x; i < 256; i += blockDim.x) hist[i] = 0.0f;
    if (REP && byte == 3)
      for (int i = threadIdx.x; i < 4096; i += blockDim.x) rep[i] = 0.0f;
    __syncthreads();
    if (REP && byte == 3) {
      const int copy = threadIdx.x & 15;
      iter([&](int, float x) {
        const uint32_t key = order_key(x);
        if (key < floor_key) return;
        const float w = COUNT ? 1.0f : __expf(x - row_max);
        atomicAdd(&rep[(key >> 24) * 16 + copy], w);
      });
      __syncthreads();
      if (threadIdx.x < 256) {
        float sum = 0.0f;
#pragma unroll
        for (int j = 0; j < 16; ++j) sum += rep[threadIdx.x * 16 + ((j + threadIdx.x) & 15)];
        hist[threadIdx.x] = sum;
      }
    } else {
      iter([&](int, float x) {
        const uint32_t key = order_key(x);
        if (key < floor_key || (key & mask) != prefix) return;
        const float w = COUNT ? 1.0f : __expf(x - row_max);
        atomicAdd(&hist[(key >> (8 * byte)) & 255u], w);
      });
    }
    __syncthreads();
    if (threadIdx.x < 32) {
      // Scan from bin 255 down for the first bin where the running sum reaches the target:
      // lane l owns bins [8l, 8l + 8).
      const int lane = threadIdx.x;
      float h[8], mine = 0.0f;
#pragma unroll
      for (int j = 0; j < 8; ++j) { h[j] = hist[lane * 8 + j]; mine += h[j]; }
      float incl = mine;                     // sum over lanes >= lane
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const float y = __shfl_down_sync(0xffffffffu, incl, o);
        if (lane + o < 32) incl += y;
      }
      if (byte == 3 && frac > 0.0f) target = frac * __shfl_sync(0xffffffffu, incl, 0);
      const float higher = incl - mine;
      const unsigned hit = __ballot_sync(0xffffffffu, above + higher + mine >= target);
      const int owner = hit ? 31 - __clz(hit) : 0;
      if (lane == owner) {
        float acc = above + higher;
        int j = 7;
        for (; j > 0; --j) {
          if (acc + h[j] >= target) break;
          acc += h[j];
        }
        if (!hit) {                           // never reached: bin 0, everything above it
          j = 0;
        }
        *sh_u = prefix | (static_cast<uint32_t>(lane * 8 + j) << (8 * byte));
        *sh_f = acc;
      }
    }
    __syncthreads();
    prefix = *sh_u;
    above = *sh_f;
    mask |= 0xFFu << (8 * byte);
    __syncthreads();
  }
  return prefix;
}

struct Args {
  const void* logits;       // [B, V]
  void* masked_out;         // optional: in-place mask target (same dtype), for top_k_top_p
  const float* temperature; // [B] (null or 0 -> greedy)
  const int* top_k;         // [B] (null or <= 0 -> off)
  const float* top_p;       // [B] (null or >= 1 -> off)
  const float* noise;       // optional [B, V] Exp(1) variates (q); null -> built-in generator
  const long long* seeds;   // [B] when noise == null
  long long* out_ids;       // [B]
  long long ld;
  long long step;           // mixed into the counter so every step draws new noise
  int B, V;
  int mask_only;
};

template <typename T>
__global__ void __launch_bounds__(kThreads) sample_kernel(const Args a) {
  // 32 KB shared by the replicated histogram of a full-row select (first 16 KB) and the
  // candidate list that replaces the row once top-k has cut it down.
  constexpr int kCap = 4096;
  __shared__ __align__(16) unsigned char big[kCap * 8];
  __shared__ float hist[256];
  __shared__ ArgMax red[32];
  __shared__ uint32_t sh_u;
  __shared__ float sh_f;
  __shared__ int cand_n;
  float* rep = reinterpret_cast<float*>(big);
  float* cand_v = reinterpret_cast<float*>(big);
  int* cand_i = reinterpret_cast<int*>(big) + kCap;
  const int row = blockIdx.x;
  const T* lg = static_cast<const T*>(a.logits) + static_cast<long long>(row) * a.ld;
  const float temp = a.temperature ? a.temperature[row] : 0.0f;
  const int k = a.top_k ? a.top_k[row] : 0;
  const float p = a.top_p ? a.top_p[row] : 1.0f;
  const bool greedy = !a.mask_only && temp <= 0.0f;
  const float inv_temp = (a.mask_only || greedy) ? 1.0f : 1.0f / temp;
  auto row_iter = [&](auto f) {
    for_each_elem<T>(lg, a.V, [&](int i, float raw) { f(i, raw * inv_temp); });
  };

  // pass 0: max (and greedy argmax)
  ArgMax best{-INFINITY, 0x7fffffff};
  row_iter([&](int i, float x) {
    if (x > best.v) best = ArgMax{x, i};
  });
  best = block_argmax(best, red);
  if (greedy) {
    if (threadIdx.x == 0) a.out_ids[row] = best.i;
    return;
  }
  const float row_max = best.v;

  uint32_t floor_key = 0;
  int n_cand = -1;                    // >= 0: the kept set sits in cand_v / cand_i
  if (k > 0 && k < a.V) {
    floor_key = radix_select<true, true>(row_iter, row_max, 0u, static_cast<float>(k), 0.0f, hist,
                                         rep, &sh_u, &sh_f);
    if (k <= kCap && (p < 1.0f || !a.mask_only)) {
      // One more pass over the row collects the survivors; everything after it (top-p,
      // the draw) reads them from shared memory.  Ties at the k-th value can overflow the
      // list: then the row is read again instead.
      if (threadIdx.x == 0) cand_n = 0;
      __syncthreads();
      row_iter([&](int i, float x) {
        if (order_key(x) < floor_key) return;
        const int slot = atomicAdd(&cand_n, 1);
        if (slot < kCap) { cand_v[slot] = x; cand_i[slot] = i; }
      });
      __syncthreads();
      if (cand_n <= kCap) n_cand = cand_n;
    }
  }
  auto cand_iter = [&](auto f) {
    for (int j = threadIdx.x; j < n_cand; j += blockDim.x) f(cand_i[j], cand_v[j]);
  };
  if (p < 1.0f) {
    const uint32_t pkey =
        n_cand >= 0 ? radix_select<false, false>(cand_iter, row_max, floor_key, 0.0f, p, hist,
                                                 nullptr, &sh_u, &sh_f)
                    : radix_select<false, true>(row_iter, row_max, floor_key, 0.0f, p, hist, rep,
                                                &sh_u, &sh_f);
    floor_key = max(floor_key, pkey);
  }

  if (a.mask_only) {
    T* out = static_cast<T*>(a.masked_out) + static_cast<long long>(row) * a.ld;
    for (int i = threadIdx.x; i < a.V; i += blockDim.x) {
      const float x = ldf<T>(lg, i);
      out[i] = order_key(x) >= floor_key ? lg[i] : from_f32<T>(-INFINITY);
    }
    return;
  }

  // Gumbel-max over the kept set: argmax(x / T - log q), q ~ Exp(1)
  const uint64_t seed = a.seeds ? static_cast<uint64_t>(a.seeds[row]) : 0x1234567ull + row;
  ArgMax pick{-INFINITY, 0x7fffffff};
  auto draw = [&](int i, float x) {
    if (order_key(x) < floor_key) return;
    const float q = a.noise ? a.noise[static_cast<long long>(row) * a.V + i]
                            : exp_noise(seed, static_cast<uint64_t>(a.step) * 0x100000000ull + i);
    const float sc = x - __logf(fmaxf(q, 1e-30f));
    if (sc > pick.v || (sc == pick.v && i < pick.i)) pick = ArgMax{sc, i};
  };
  if (n_cand >= 0) cand_iter(draw);
  else row_iter(draw);
  pick = block_argmax(pick, red);
  if (threadIdx.x == 0) a.out_ids[row] = pick.i;
}

}  // namespace sampler
}  // namespace b200

// Fused sampler.  dtype: 0 bf16, 1 fp16, 2 fp32 logits.  temperature == null or
// a row value <= 0 selects greedy argmax for that row.
B200_API int b200_sample(const void* logits, long long ld, int B, int V, int dtype,
                         const float* temperature, const int* top_k, const float* top_p,
                         const float* noise, const long long* seeds, long long step,
                         long long* out_ids, void* stream) {
  using namespace b200::sampler;
  if (B <= 0) return 0;
  Args a;
  a.logits = logits; a.masked_out = nullptr; a.temperature = temperature; a.top_k = top_k;
  a.top_p = top_p; a.noise = noise; a.seeds = seeds; a.out_ids = out_ids; a.ld = ld;
  a.step = step; a.B = B; a.V = V; a.mask_only = 0;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (dtype == 0) sample_kernel<__nv_bfloat16><<<B, kThreads, 0, s>>>(a);
  else if (dtype == 1) sample_kernel<__half><<<B, kThreads, 0, s>>>(a);
  else if (dtype == 2) sample_kernel<float><<<B, kThreads, 0, s>>>(a);
  else return -8;
  return static_cast<int>(cudaGetLastError());
}

// In-place top-k / top-p mask: entries outside the kept set become -inf.
B200_API int b200_top_k_top_p(void* logits, long long ld, int B, int V, int dtype,
                              const int* top_k, const float* top_p, void* stream) {
  using namespace b200::sampler;
  if (B <= 0) return 0;
  Args a;
  a.logits = logits; a.masked_out = logits; a.temperature = nullptr; a.top_k = top_k;
  a.top_p = top_p; a.noise = nullptr; a.seeds = nullptr; a.out_ids = nullptr; a.ld = ld;
  a.step = 0; a.B = B; a.V = V; a.mask_only = 1;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (dtype == 0) sample_kernel<__nv_bfloat16><<<B, kThreads, 0, s>>>(a);
  else if (dtype == 1) sample_kernel<__half><<<B, kThreads, 0, s>>>(a);
  else if (dtype == 2) sample_kernel<float><<<B, kThreads, 0, s>>>(a);
  else return -8;
  return static_cast<int>(cudaGetLastError());
}
