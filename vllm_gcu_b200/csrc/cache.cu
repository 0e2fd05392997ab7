// Rotary embedding and KV-cache maintenance kernels for sm_100a.
//
//   rope_cache_flash    RoPE on q and k in place + write of k, v into the paged
//                       cache [blocks, block_size, kv_heads, head] in one pass
//                       (either half can be switched off, which gives the
//                       stand-alone rotary_embedding / reshape_and_cache_flash)
//   reshape_and_cache   write into the x-packed layout
//                       K [blocks, kv_heads, head/x, block_size, x],
//                       V [blocks, kv_heads, head, block_size], optional
//                       int8 (scale + zero point) or fp8 quantisation
//   mla_rope_cache      split latent -> RMSNorm(kv_c) -> RoPE(q_pe, k_pe) ->
//                       optional fp8 -> paged write of [kv_c | k_pe]
//   concat_and_cache_mla, gather_cache, copy_blocks, swap_blocks
//
// Reference ops: csrc/src/rotary_embedding.cpp:38, reshape_and_cache.cpp:34,
// reshape_and_cache_flash.cpp:23, concat_and_cache_mla.cpp:35,
// rotary_embedding_with_kv_cache.cpp:42 (native fallback in
// vllm_gcu/attention/backends/mla_fusion.py:73-106), gather_cache.cpp:18,
// cache_kernels.cpp:10-58.
#include "common.cuh"

namespace b200 {
namespace cache {

constexpr unsigned int kKernelId = 20;

struct RopeCacheArgs {
  void* q;                 // [T, Hq, D] (row pitch ldq) rotated in place; may be null
  void* k;                 // [T, Hkv, D] (row pitch ldk) rotated in place; may be null
  const void* v;           // [T, Hkv, D] (row pitch ldv); may be null
  const long long* positions;  // [T]; null = no rotation
  const void* cos_sin;     // [max_pos, rot_dim] = [cos | sin]
  const long long* slot_mapping;  // [T]; null = no cache write
  void* k_cache;
  void* v_cache;
  const float* k_scale;    // fp8 cache only
  const float* v_scale;
  long long ldq, ldk, ldv;
  long long cache_slot_stride;  // elements between consecutive slots
  long long cache_head_stride;  // elements between heads inside a slot
  long long num_slots;
  int T, Hq, Hkv, D, rot_dim;
  int is_neox;
  int cos_sin_fp32;
  int cache_fp8;   // 0: cache holds T, 1: fp8 e4m3, 2: int8 (symmetric)
  unsigned int* status;
};

template <typename T>
__device__ __forceinline__ float cs_at(const void* base, long long idx, int fp32) {
  return fp32 ? static_cast<const float*>(base)[idx] : to_f32<T>(static_cast<const T*>(base)[idx]);
}

// Rotates one head vector in place.  NeoX: pairs (i, i + rot/2); GPT-J: (2i, 2i+1).
template <typename T>
__device__ __forceinline__ void rotate_head(T* x, const void* cs, long long cs_row, int rot_dim,
                                            int is_neox, int fp32, int lane, int nlanes) {
  const int half = rot_dim >> 1;
  for (int i = lane; i < half; i += nlanes) {
    const float c = cs_at<T>(cs, cs_row + i, fp32);
    const float s = cs_at<T>(cs, cs_row + half + i, fp32);
    const int i0 = is_neox ? i : 2 * i;
    const int i1 = is_neox ? i + half : 2 * i + 1;
    const float a = to_f32<T>(x[i0]);
    const float b = to_f32<T>(x[i1]);
    x[i0] = from_f32<T>(a * c - b * s);
    x[i1] = from_f32<T>(b * c + a * s);
  }
}

template <typename T>
__global__ void __launch_bounds__(256) rope_cache_flash_kernel(const RopeCacheArgs a) {
  const int t = blockIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
  T* q = a.q ? static_cast<T*>(a.q) + static_cast<long long>(t) * a.ldq : nullptr;
  T* k = a.k ? static_cast<T*>(a.k) + static_cast<long long>(t) * a.ldk : nullptr;
  const T* v = a.v ? static_cast<const T*>(a.v) + static_cast<long long>(t) * a.ldv : nullptr;

  if (a.positions != nullptr) {
    const long long cs_row = a.positions[t] * a.rot_dim;
    const int heads = (q ? a.Hq : 0) + (k ? a.Hkv : 0);
    const int half = a.rot_dim >> 1;
    const bool vec_ok = a.is_neox && (half & 7) == 0 && (a.D & 7) == 0 && (a.ldq & 7) == 0 &&
                        (a.ldk & 7) == 0 &&
                        ((reinterpret_cast<uintptr_t>(a.q) | reinterpret_cast<uintptr_t>(a.k)) & 15) == 0;
    if (vec_ok) {
      // NeoX pairs (i, i + half): one thread rotates 8 pairs with 16-byte loads and stores.
      const int vph = half >> 3;
      for (int it = threadIdx.x; it < heads * vph; it += blockDim.x) {
        const int h = it / vph, i = (it % vph) * 8;
        T* x = (q && h < a.Hq) ? q + static_cast<long long>(h) * a.D
                               : k + static_cast<long long>(h - (q ? a.Hq : 0)) * a.D;
        float lo[8], hi[8], c[8], sn[8];
        vec8_load<T>(x + i, lo);
        vec8_load<T>(x + half + i, hi);
        if (a.cos_sin_fp32 && (reinterpret_cast<uintptr_t>(a.cos_sin) & 15) == 0) {
          const float4* cp = reinterpret_cast<const float4*>(
              static_cast<const float*>(a.cos_sin) + cs_row + i);
          const float4* sp = reinterpret_cast<const float4*>(
              static_cast<const float*>(a.cos_sin) + cs_row + half + i);
          const float4 c0 = cp[0], c1 = cp[1], s0 = sp[0], s1 = sp[1];
          c[0] = c0.x; c[1] = c0.y; c[2] = c0.z; c[3] = c0.w;
          c[4] = c1.x; c[5] = c1.y; c[6] = c1.z; c[7] = c1.w;
          sn[0] = s0.x; sn[1] = s0.y; sn[2] = s0.z; sn[3] = s0.w;
          sn[4] = s1.x; sn[5] = s1.y; sn[6] = s1.z; sn[7] = s1.w;
        } else {
#pragma unroll
          for (int u = 0; u < 8; ++u) {
            c[u] = cs_at<T>(a.cos_sin, cs_row + i + u, a.cos_sin_fp32);
            sn[u] = cs_at<T>(a.cos_sin, cs_row + half + i + u, a.cos_sin_fp32);
          }
        }
        float r0[8], r1[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          r0[u] = lo[u] * c[u] - hi[u] * sn[u];
          r1[u] = hi[u] * c[u] + lo[u] * sn[u];
        }
        vec8_store<T>(x + i, r0);
        vec8_store<T>(x + half + i, r1);
      }
    } else
    for (int h = warp; h < heads; h += nwarps) {
      T* x = (q && h < a.Hq) ? q + static_cast<long long>(h) * a.D
                             : k + static_cast<long long>(h - (q ? a.Hq : 0)) * a.D;
      rotate_head<T>(x, a.cos_sin, cs_row, a.rot_dim, a.is_neox, a.cos_sin_fp32, lane, 32);
    }
  }
  if (a.slot_mapping == nullptr) return;
  const long long slot = a.slot_mapping[t];
  if (slot < 0) return;  // padding token
  if (slot >= a.num_slots) {
    if (threadIdx.x == 0) report_status(a.status, kStatusBounds, kKernelId, static_cast<unsigned>(t));
    return;
  }
  __syncthreads();  // rotated k visible to all threads of the CTA
  const int nvec = (a.Hkv * a.D) >> 3;
  const int vec_per_head = a.D >> 3;
  for (int i = threadIdx.x; i < 2 * nvec; i += blockDim.x) {
    const bool is_v = i >= nvec;
    const int j = is_v ? i - nvec : i;
    const T* src = is_v ? v : k;
    if (src == nullptr) continue;
    const int h = j / vec_per_head, e = (j % vec_per_head) * 8;
    const long long dst_off = slot * a.cache_slot_stride + h * a.cache_head_stride + e;
    if (a.cache_fp8) {
      float f[8];
      vec8_load<T>(src + static_cast<long long>(h) * a.D + e, f);
      const float inv = 1.0f / (is_v ? *a.v_scale : *a.k_scale);
      uint2 pk;
      uint8_t* b = reinterpret_cast<uint8_t*>(&pk);
      if (a.cache_fp8 == 2) {          // int8, symmetric (zero point 0)
#pragma unroll
        for (int u = 0; u < 8; ++u)
          b[u] = static_cast<uint8_t>(static_cast<int8_t>(
              fminf(fmaxf(rintf(f[u] * inv), -128.0f), 127.0f)));
      } else {
#pragma unroll
        for (int u = 0; u < 8; ++u) b[u] = f32_to_e4m3(f[u] * inv);
      }
      uint8_t* dst = static_cast<uint8_t*>(is_v ? a.v_cache : a.k_cache);
      *reinterpret_cast<uint2*>(dst + dst_off) = pk;
    } else {
      T* dst = static_cast<T*>(is_v ? a.v_cache : a.k_cache);
      *reinterpret_cast<uint4*>(dst + dst_off) =
          *reinterpret_cast<const uint4*>(src + static_cast<long long>(h) * a.D + e);
    }
  }
}

// ---------------------------------------------------------------------------
// x-packed layout (paged attention v1/v2 style caches)
// ---------------------------------------------------------------------------
struct ReshapeArgs {
  const void* key;     // [T, Hkv, D], row pitch ldk
  const void* value;   // [T, Hkv, D], row pitch ldv
  void* k_cache;       // [blocks, Hkv, D/x, bs, x]
  void* v_cache;       // [blocks, Hkv, D, bs]
  const long long* slot_mapping;
  long long ldk, ldv;
  long long num_slots;
  int T, Hkv, D, block_size, x;
  int qmode;  // 0 none, 1 int8 (scale, zero point), 2 fp8 e4m3 (scale)
  float k_scale, v_scale, k_zp, v_zp;
  unsigned int* status;
};

template <typename T>
__global__ void __launch_bounds__(256) reshape_and_cache_kernel(const ReshapeArgs a) {
  const int t = blockIdx.x;
  const long long slot = a.slot_mapping[t];
  if (slot < 0) return;
  if (slot >= a.num_slots) {
    if (threadIdx.x == 0) report_status(a.status, kStatusBounds, kKernelId + 1, static_cast<unsigned>(t));
    return;
  }
  const long long blk = slot / a.block_size;
  const int off = static_cast<int>(slot % a.block_size);
  const T* key = static_cast<const T*>(a.key) + static_cast<long long>(t) * a.ldk;
  const T* val = static_cast<const T*>(a.value) + static_cast<long long>(t) * a.ldv;
  const int n = a.Hkv * a.D;
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    const int h = i / a.D, d = i % a.D;
    const long long kidx =
        (((blk * a.Hkv + h) * (a.D / a.x) + d / a.x) * a.block_size + off) * a.x + d % a.x;
    const long long vidx = ((blk * a.Hkv + h) * a.D + d) * a.block_size + off;
    const float kf = to_f32<T>(key[i]), vf = to_f32<T>(val[i]);
    if (a.qmode == 0) {
      static_cast<T*>(a.k_cache)[kidx] = key[i];
      static_cast<T*>(a.v_cache)[vidx] = val[i];
    } else if (a.qmode == 1) {
      float kq = fminf(fmaxf(rintf(kf / a.k_scale) + a.k_zp, -128.0f), 127.0f);
      float vq = fminf(fmaxf(rintf(vf / a.v_scale) + a.v_zp, -128.0f), 127.0f);
      static_cast<int8_t*>(a.k_cache)[kidx] = static_cast<int8_t>(kq);
      static_cast<int8_t*>(a.v_cache)[vidx] = static_cast<int8_t>(vq);
    } else {
      static_cast<uint8_t*>(a.k_cache)[kidx] = f32_to_e4m3(kf / a.k_scale);
      static_cast<uint8_t*>(a.v_cache)[vidx] = f32_to_e4m3(vf / a.v_scale);
    }
  }
}

// ---------------------------------------------------------------------------
// MLA: fused split + RMSNorm + RoPE + (fp8) + paged write
// ---------------------------------------------------------------------------
struct MlaArgs {
  void* q_pe;              // [T, H, R] rotated in place when q_out == null
  void* q_out;             // optional [T, H, *] destination, row pitch ldqo, head pitch hsqo
  const void* kv;          // [T, L + R] raw latent, row pitch ldkv (null for concat-only)
  const void* kv_c_in;     // concat-only mode: already normed [T, L]
  const void* k_pe_in;     // concat-only mode: already rotated [T, R]
  void* kv_cache;          // [num_slots, L + R] (T or fp8 bytes)
  void* k_pe_out;          // optional [T, R]
  void* k_c_normed_out;    // optional [T, L]
  const long long* positions;
  const float* cos_sin;    // fp32 [max_pos, R] = [cos | sin]
  const void* weight;      // [L]
  const long long* slot_mapping;
  const float* scale;      // fp8 cache scale (scalar)
  long long ldq, hsq, ldqo, hsqo, ldkv, cache_slot_stride, num_slots;
  int T, H, L, R;
  float eps;
  int is_neox;
  int cache_fp8;
  unsigned int* status;
};

template <typename T>
__global__ void __launch_bounds__(256) mla_rope_cache_kernel(const MlaArgs a) {
  extern __shared__ float sm[];  // L + R floats
  __shared__ float red[32];
  const int t = blockIdx.x;
  float* s_c = sm;
  float* s_pe = sm + a.L;
  const int half = a.R >> 1;

  if (a.kv != nullptr) {
    const T* kv = static_cast<const T*>(a.kv) + static_cast<long long>(t) * a.ldkv;
    const T* w = static_cast<const T*>(a.weight);
    float ss = 0.0f;
    for (int i = threadIdx.x; i < a.L; i += blockDim.x) {
      const float x = to_f32<T>(kv[i]);
      s_c[i] = x;
      ss += x * x;
    }
    ss = block_sum(ss, red);
    const float rstd = rsqrtf(ss / a.L + a.eps);
    for (int i = threadIdx.x; i < a.L; i += blockDim.x)
      s_c[i] = round_like<T>(s_c[i] * rstd * to_f32<T>(w[i]));
    const long long cs_row = a.positions[t] * a.R;
    for (int i = threadIdx.x; i < half; i += blockDim.x) {
      const float c = a.cos_sin[cs_row + i], s = a.cos_sin[cs_row + half + i];
      const int i0 = a.is_neox ? i : 2 * i, i1 = a.is_neox ? i + half : 2 * i + 1;
      const float x0 = to_f32<T>(kv[a.L + i0]), x1 = to_f32<T>(kv[a.L + i1]);
      s_pe[i0] = round_like<T>(x0 * c - x1 * s);
      s_pe[i1] = round_like<T>(x1 * c + x0 * s);
    }
    // query rope
    if (a.q_pe != nullptr) {
      const T* qin = static_cast<const T*>(a.q_pe) + static_cast<long long>(t) * a.ldq;
      T* qout = a.q_out ? static_cast<T*>(a.q_out) + static_cast<long long>(t) * a.ldqo
                        : static_cast<T*>(a.q_pe) + static_cast<long long>(t) * a.ldq;
      const long long hso = a.q_out ? a.hsqo : a.hsq;
      for (int i = threadIdx.x; i < a.H * half; i += blockDim.x) {
        const int h = i / half, j = i % half;
        const float c = a.cos_sin[cs_row + j], s = a.cos_sin[cs_row + half + j];
        const int i0 = a.is_neox ? j : 2 * j, i1 = a.is_neox ? j + half : 2 * j + 1;
        const float x0 = to_f32<T>(qin[h * a.hsq + i0]), x1 = to_f32<T>(qin[h * a.hsq + i1]);
        qout[h * hso + i0] = from_f32<T>(x0 * c - x1 * s);
        qout[h * hso + i1] = from_f32<T>(x1 * c + x0 * s);
      }
    }
  } else {
    const T* c_in = static_cast<const T*>(a.kv_c_in) + static_cast<long long>(t) * a.L;
    const T* p_in = static_cast<const T*>(a.k_pe_in) + static_cast<long long>(t) * a.R;
    for (int i = threadIdx.x; i < a.L; i += blockDim.x) s_c[i] = to_f32<T>(c_in[i]);
    for (int i = threadIdx.x; i < a.R; i += blockDim.x) s_pe[i] = to_f32<T>(p_in[i]);
  }
  __syncthreads();

  if (a.k_pe_out != nullptr) {
    T* o = static_cast<T*>(a.k_pe_out) + static_cast<long long>(t) * a.R;
    for (int i = threadIdx.x; i < a.R; i += blockDim.x) o[i] = from_f32<T>(s_pe[i]);
  }
  if (a.k_c_normed_out != nullptr) {
    T* o = static_cast<T*>(a.k_c_normed_out) + static_cast<long long>(t) * a.L;
    for (int i = threadIdx.x; i < a.L; i += blockDim.x) o[i] = from_f32<T>(s_c[i]);
  }
  if (a.slot_mapping == nullptr) return;
  const long long slot = a.slot_mapping[t];
  if (slot < 0) return;
  if (slot >= a.num_slots) {
    if (threadIdx.x == 0) report_status(a.status, kStatusBounds, kKernelId + 2, static_cast<unsigned>(t));
    return;
  }
  const int W = a.L + a.R;
  if (a.cache_fp8) {
    const float inv = 1.0f / *a.scale;
    uint8_t* dst = static_cast<uint8_t*>(a.kv_cache) + slot * a.cache_slot_stride;
    for (int i = threadIdx.x; i < W; i += blockDim.x) dst[i] = f32_to_e4m3(sm[i] * inv);
  } else {
    T* dst = static_cast<T*>(a.kv_cache) + slot * a.cache_slot_stride;
    for (int i = threadIdx.x; i < W; i += blockDim.x) dst[i] = from_f32<T>(sm[i]);
  }
}

// ---------------------------------------------------------------------------
// gather_cache: pages -> contiguous rows
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(128)
    gather_cache_kernel(const uint8_t* src, uint8_t* dst, const int* block_table,
                        const int* cu_seq_lens, const int* seq_starts, int batch,
                        int max_blocks, int block_size, long long row_bytes,
                        long long src_slot_stride_bytes, long long num_slots, unsigned int* status) {
  const int tok = blockIdx.x;
  // locate the sequence of this output row
  int lo = 0, hi = batch;
  while (lo < hi) {
    const int mid = (lo + hi) >> 1;
    if (cu_seq_lens[mid + 1] <= tok) lo = mid + 1; else hi = mid;
  }
  if (lo >= batch) return;
  const int b = lo;
  const int pos = tok - cu_seq_lens[b] + (seq_starts ? seq_starts[b] : 0);
  const int blk = block_table[static_cast<long long>(b) * max_blocks + pos / block_size];
  const long long slot = static_cast<long long>(blk) * block_size + pos % block_size;
  if (slot < 0 || slot >= num_slots) {
    if (threadIdx.x == 0) report_status(status, kStatusBounds, kKernelId + 3, static_cast<unsigned>(tok));
    return;
  }
  const uint4* s4 = reinterpret_cast<const uint4*>(src + slot * src_slot_stride_bytes);
  uint4* d4 = reinterpret_cast<uint4*>(dst + static_cast<long long>(tok) * row_bytes);
  for (int i = threadIdx.x; i < row_bytes / 16; i += blockDim.x) d4[i] = s4[i];
}

// copy_blocks: every cache tensor gets the same (src, dst) block pairs.
__global__ void __launch_bounds__(256)
    copy_blocks_kernel(const long long* cache_ptrs, const long long* mapping, long long block_bytes) {
  uint8_t* base = reinterpret_cast<uint8_t*>(cache_ptrs[blockIdx.y]);
  const long long src = mapping[2 * blockIdx.x], dst = mapping[2 * blockIdx.x + 1];
  const uint4* s4 = reinterpret_cast<const uint4*>(base + src * block_bytes);
  uint4* d4 = reinterpret_cast<uint4*>(base + dst * block_bytes);
  for (long long i = threadIdx.x; i < block_bytes / 16; i += blockDim.x) d4[i] = s4[i];
}

}  // namespace cache
}  // namespace b200

using namespace b200;
using namespace b200::cache;

// RoPE (+ cache write).  dtype 0 bf16 / 1 fp16.  Any of q / k / v / positions /
// slot_mapping may be null to skip that part.  D must be a multiple of 8.
B200_API int b200_rope_cache_flash(void* q, long long ldq, void* k, long long ldk, const void* v,
                                   long long ldv, const long long* positions, const void* cos_sin,
                                   int cos_sin_fp32, int rot_dim, int is_neox,
                                   const long long* slot_mapping, void* k_cache, void* v_cache,
                                   long long cache_slot_stride, long long cache_head_stride,
                                   long long num_slots, int cache_fp8, const float* k_scale,
                                   const float* v_scale, int T, int Hq, int Hkv, int D, int dtype,
                                   void* stream) {
  if (T <= 0) return 0;
  if ((D % 8) != 0 || (rot_dim % 2) != 0 || rot_dim > D) return -2;
  RopeCacheArgs a;
  a.q = q; a.k = k; a.v = v; a.positions = positions; a.cos_sin = cos_sin;
  a.slot_mapping = slot_mapping; a.k_cache = k_cache; a.v_cache = v_cache;
  a.k_scale = k_scale; a.v_scale = v_scale; a.ldq = ldq; a.ldk = ldk; a.ldv = ldv;
  a.cache_slot_stride = cache_slot_stride; a.cache_head_stride = cache_head_stride;
  a.num_slots = num_slots; a.T = T; a.Hq = Hq; a.Hkv = Hkv; a.D = D; a.rot_dim = rot_dim;
  a.is_neox = is_neox; a.cos_sin_fp32 = cos_sin_fp32; a.cache_fp8 = cache_fp8;
  a.status = status_ptr();
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (dtype == 0) rope_cache_flash_kernel<__nv_bfloat16><<<T, 256, 0, s>>>(a);
  else if (dtype == 1) rope_cache_flash_kernel<__half><<<T, 256, 0, s>>>(a);
  else return -8;
  return static_cast<int>(cudaGetLastError());
}

B200_API int b200_reshape_and_cache(const void* key, long long ldk, const void* value,
                                    long long ldv, void* k_cache, void* v_cache,
                                    const long long* slot_mapping, long long num_slots, int T,
                                    int Hkv, int D, int block_size, int x, int qmode,
                                    float k_scale, float v_scale, float k_zp, float v_zp,
                                    int dtype, void* stream) {
  if (T <= 0) return 0;
  if (x <= 0 || (D % x) != 0) return -2;
  ReshapeArgs a;
  a.key = key; a.value = value; a.k_cache = k_cache; a.v_cache = v_cache;
  a.slot_mapping = slot_mapping; a.ldk = ldk; a.ldv = ldv; a.num_slots = num_slots; a.T = T;
  a.Hkv = Hkv; a.D = D; a.block_size = block_size; a.x = x; a.qmode = qmode;
  a.k_scale = k_scale; a.v_scale = v_scale; a.k_zp = k_zp; a.v_zp = v_zp;
  a.status = status_ptr();
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (dtype == 0) reshape_and_cache_kernel<__nv_bfloat16><<<T, 256, 0, s>>>(a);
  else if (dtype == 1) reshape_and_cache_kernel<__half><<<T, 256, 0, s>>>(a);
  else return -8;
  return static_cast<int>(cudaGetLastError());
}

// Fused MLA cache update (kv != null) or plain concat-and-cache (kv == null,
// kv_c_in / k_pe_in given).
B200_API int b200_mla_rope_cache(void* q_pe, long long ldq, long long hsq, void* q_out,
                                 long long ldqo, long long hsqo, const void* kv, long long ldkv,
                                 const void* kv_c_in, const void* k_pe_in, void* kv_cache,
                                 long long cache_slot_stride, long long num_slots,
                                 void* k_pe_out, void* k_c_normed_out,
                                 const long long* positions, const float* cos_sin,
                                 const void* weight, const long long* slot_mapping,
                                 const float* scale, int T, int H, int L, int R, float eps,
                                 int is_neox, int cache_fp8, int dtype, void* stream) {
  if (T <= 0) return 0;
  MlaArgs a;
  a.q_pe = q_pe; a.q_out = q_out; a.kv = kv; a.kv_c_in = kv_c_in; a.k_pe_in = k_pe_in;
  a.kv_cache = kv_cache; a.k_pe_out = k_pe_out; a.k_c_normed_out = k_c_normed_out;
  a.positions = positions; a.cos_sin = cos_sin; a.weight = weight; a.slot_mapping = slot_mapping;
  a.scale = scale; a.ldq = ldq; a.hsq = hsq; a.ldqo = ldqo; a.hsqo = hsqo; a.ldkv = ldkv;
  a.cache_slot_stride = cache_slot_stride; a.num_slots = num_slots; a.T = T; a.H = H; a.L = L;
  a.R = R; a.eps = eps; a.is_neox = is_neox; a.cache_fp8 = cache_fp8;
  a.status = status_ptr();
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const size_t smem = static_cast<size_t>(L + R) * sizeof(float);
  if (dtype == 0) mla_rope_cache_kernel<__nv_bfloat16><<<T, 256, smem, s>>>(a);
  else if (dtype == 1) mla_rope_cache_kernel<__half><<<T, 256, smem, s>>>(a);
  else return -8;
  return static_cast<int>(cudaGetLastError());
}

B200_API int b200_gather_cache(const void* src, void* dst, const int* block_table,
                               const int* cu_seq_lens, const int* seq_starts, int batch,
                               int max_blocks, int block_size, long long row_bytes,
                               long long src_slot_stride_bytes, long long num_slots,
                               int total_tokens, void* stream) {
  if (total_tokens <= 0) return 0;
  if ((row_bytes % 16) != 0 || (src_slot_stride_bytes % 16) != 0) return -2;
  gather_cache_kernel<<<total_tokens, 128, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint8_t*>(src), static_cast<uint8_t*>(dst), block_table, cu_seq_lens,
      seq_starts, batch, max_blocks, block_size, row_bytes, src_slot_stride_bytes, num_slots,
      status_ptr());
  return static_cast<int>(cudaGetLastError());
}

// cache_ptrs: device array of `num_caches` base addresses; mapping: device
// int64 [num_pairs, 2] of (src block, dst block).
B200_API int b200_copy_blocks(const long long* cache_ptrs, int num_caches,
                              const long long* mapping, int num_pairs, long long block_bytes,
                              void* stream) {
  if (num_pairs <= 0 || num_caches <= 0) return 0;
  if ((block_bytes % 16) != 0) return -2;
  dim3 grid(num_pairs, num_caches);
  copy_blocks_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(cache_ptrs, mapping,
                                                                         block_bytes);
  return static_cast<int>(cudaGetLastError());
}

// Host-driven block swap between two caches (either may be pinned host
// memory).  mapping_host: int64 [num_pairs, 2] in host memory.  Runs of
// consecutive block ids are merged into one asynchronous copy each; there is
// no host synchronisation.
B200_API int b200_swap_blocks(const void* src, void* dst, const long long* mapping_host,
                              int num_pairs, long long block_bytes, void* stream) {
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  int i = 0;
  while (i < num_pairs) {
    int j = i + 1;
    while (j < num_pairs && mapping_host[2 * j] == mapping_host[2 * (j - 1)] + 1 &&
           mapping_host[2 * j + 1] == mapping_host[2 * (j - 1) + 1] + 1)
      ++j;
    cudaError_t e = cudaMemcpyAsync(
        static_cast<uint8_t*>(dst) + mapping_host[2 * i + 1] * block_bytes,
        static_cast<const uint8_t*>(src) + mapping_host[2 * i] * block_bytes,
        static_cast<size_t>(j - i) * block_bytes, cudaMemcpyDefault, s);
    if (e != cudaSuccess) return static_cast<int>(e);
    i = j;
  }
  return 0;
}
