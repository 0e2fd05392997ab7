// KV-cache offload kernels for the LMCache connector (sm_100a) and pinned host buffers.
//
//   multi_layer_kv_transfer   tokens (by slot mapping) <-> one contiguous buffer
//                             [2, L, T, W] (or [L, T, W] for MLA) across all layers, whose
//                             paged buffers are given as a device table of base pointers
//   single_layer_kv_transfer  the same for one layer, token-major or kv-major buffer
//   rotary_embedding_k        re-rotates cached keys from their old to new positions
//                             (cache blending re-uses KV computed at other offsets)
//   cachegen_cdf              per (layer, channel) cumulative histogram of quantised KV bins
//   pinned host allocation    cudaHostAlloc / NUMA-bound + cudaHostRegister
//
// A paged layer buffer is [2, num_slots, W] (K then V, each `page_buffer_size` slots) or
// [num_slots, W] for MLA.  direction != 0: paged -> buffer; 0: buffer -> paged.
// Reference: lmcache/csrc/multi_layer_kv_transfer.cpp:33, single_layer_kv_transfer.cpp:31,
// load_and_reshape_flash.cpp:29, reshape_and_cache_back_flash.cpp:29,
// rotary_embedding_k_fused.cpp:30, calculate_cdf.cpp:40, mem_alloc.cpp:28-116.
#include "common.cuh"

#include <cstdlib>
#include <cstring>

namespace b200 {
namespace lmc {

__global__ void __launch_bounds__(256)
    multi_layer_kernel(uint8_t* buf, const long long* layer_ptrs, const long long* slot_mapping,
                       int num_layers, int num_tokens, long long row_bytes,
                       long long page_buffer_slots, int direction, int use_mla,
                       unsigned int* status) {
  const int t = blockIdx.x, layer = blockIdx.y, kv = blockIdx.z;
  const long long slot = slot_mapping[t];
  if (slot < 0) return;
  if (slot >= page_buffer_slots) {
    if (threadIdx.x == 0) report_status(status, kStatusBounds, 70u, static_cast<unsigned>(t));
    return;
  }
  uint8_t* paged = reinterpret_cast<uint8_t*>(layer_ptrs[layer]) +
                   (static_cast<long long>(kv) * page_buffer_slots + slot) * row_bytes;
  // buffer index: [kv][layer][token] (MLA: kv extent is 1)
  uint8_t* b = buf + ((static_cast<long long>(kv) * num_layers + layer) * num_tokens + t) * row_bytes;
  (void)use_mla;
  uint4* d4 = reinterpret_cast<uint4*>(direction ? b : paged);
  const uint4* s4 = reinterpret_cast<const uint4*>(direction ? paged : b);
  for (long long i = threadIdx.x; i < row_bytes / 16; i += blockDim.x) d4[i] = s4[i];
}

__global__ void __launch_bounds__(256)
    single_layer_kernel(uint8_t* buf, uint8_t* k_cache, uint8_t* v_cache,
                        const long long* slot_mapping, int num_tokens, long long row_bytes,
                        long long num_slots, int direction, int token_major,
                        unsigned int* status) {
  const int t = blockIdx.x, kv = blockIdx.y;
  const long long slot = slot_mapping[t];
  if (slot < 0) return;
  if (slot >= num_slots) {
    if (threadIdx.x == 0) report_status(status, kStatusBounds, 71u, static_cast<unsigned>(t));
    return;
  }
  uint8_t* paged = (kv ? v_cache : k_cache) + slot * row_bytes;
  const long long bi = token_major ? (static_cast<long long>(t) * 2 + kv)
                                   : (static_cast<long long>(kv) * num_tokens + t);
  uint8_t* b = buf + bi * row_bytes;
  uint4* d4 = reinterpret_cast<uint4*>(direction ? b : paged);
  const uint4* s4 = reinterpret_cast<const uint4*>(direction ? paged : b);
  for (long long i = threadIdx.x; i < row_bytes / 16; i += blockDim.x) d4[i] = s4[i];
}

// key[t, h, :] is rotated by (new_pos - old_pos): un-rotate with the old angle, rotate with
// the new one, fused into one complex multiplication per pair.
template <typename T>
__global__ void __launch_bounds__(256)
    rerotate_k_kernel(T* key, long long ldk, const long long* old_pos, const long long* new_pos,
                      const T* cos_sin, int num_heads, int head_size, int rot_dim, int is_neox) {
  const int t = blockIdx.x;
  const int half = rot_dim >> 1;
  const long long ro = old_pos[t] * rot_dim, rn = new_pos[t] * rot_dim;
  for (int i = threadIdx.x; i < num_heads * half; i += blockDim.x) {
    const int h = i / half, j = i % half;
    const float co = to_f32<T>(cos_sin[ro + j]), so = to_f32<T>(cos_sin[ro + half + j]);
    const float cn = to_f32<T>(cos_sin[rn + j]), sn = to_f32<T>(cos_sin[rn + half + j]);
    // e^{i(new - old)} = (cn + i sn)(co - i so)
    const float c = cn * co + sn * so, s = sn * co - cn * so;
    T* x = key + static_cast<long long>(t) * ldk + static_cast<long long>(h) * head_size;
    const int i0 = is_neox ? j : 2 * j, i1 = is_neox ? j + half : 2 * j + 1;
    const float a = to_f32<T>(x[i0]), b = to_f32<T>(x[i1]);
    x[i0] = from_f32<T>(a * c - b * s);
    x[i1] = from_f32<T>(b * c + a * s);
  }
}

// input int8 [L, T, C] with values in [0, max_bins); output int16 [L, C, max_bins + 1]:
// cdf[l, c, b] = floor(count(values < b) * scale) with the last entry pinned to 2^16 - 1 ... the
// codec consumes monotone 16-bit cumulative frequencies.
__global__ void __launch_bounds__(256)
    cachegen_cdf_kernel(const int8_t* input, short* out, int L, int T, int C, int max_bins) {
  const int l = blockIdx.y, c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= C) return;
  int hist[64];
  for (int b = 0; b < max_bins; ++b) hist[b] = 0;
  for (int t = 0; t < T; ++t) {
    const int v = input[(static_cast<long long>(l) * T + t) * C + c];
    if (v >= 0 && v < max_bins) ++hist[v];
  }
  short* o = out + (static_cast<long long>(l) * C + c) * (max_bins + 1);
  long long run = 0;
  o[0] = 0;
  for (int b = 0; b < max_bins; ++b) {
    run += hist[b];
    const long long q = T > 0 ? (run * 65535LL) / T : 0;
    o[b + 1] = static_cast<short>(static_cast<unsigned short>(q > 65535 ? 65535 : q));
  }
}

}  // namespace lmc
}  // namespace b200

using namespace b200;

B200_API int b200_lmc_multi_layer_kv_transfer(void* buf, const long long* layer_ptrs,
                                              const long long* slot_mapping, int num_layers,
                                              int num_tokens, long long row_bytes,
                                              long long page_buffer_slots, int direction,
                                              int use_mla, void* stream) {
  if (num_tokens <= 0 || num_layers <= 0) return 0;
  if ((row_bytes % 16) != 0) return -2;
  dim3 grid(num_tokens, num_layers, use_mla ? 1 : 2);
  lmc::multi_layer_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<uint8_t*>(buf), layer_ptrs, slot_mapping, num_layers, num_tokens, row_bytes,
      page_buffer_slots, direction, use_mla, status_ptr());
  return static_cast<int>(cudaGetLastError());
}

B200_API int b200_lmc_single_layer_kv_transfer(void* buf, void* k_cache, void* v_cache,
                                               const long long* slot_mapping, int num_tokens,
                                               long long row_bytes, long long num_slots,
                                               int direction, int token_major, void* stream) {
  if (num_tokens <= 0) return 0;
  if ((row_bytes % 16) != 0) return -2;
  dim3 grid(num_tokens, 2);
  lmc::single_layer_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<uint8_t*>(buf), static_cast<uint8_t*>(k_cache), static_cast<uint8_t*>(v_cache),
      slot_mapping, num_tokens, row_bytes, num_slots, direction, token_major, status_ptr());
  return static_cast<int>(cudaGetLastError());
}

B200_API int b200_lmc_rerotate_k(void* key, long long ldk, const long long* old_pos,
                                 const long long* new_pos, const void* cos_sin, int T,
                                 int num_heads, int head_size, int rot_dim, int is_neox, int dtype,
                                 void* stream) {
  if (T <= 0) return 0;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (dtype == 0)
    lmc::rerotate_k_kernel<__nv_bfloat16><<<T, 256, 0, s>>>(
        static_cast<__nv_bfloat16*>(key), ldk, old_pos, new_pos,
        static_cast<const __nv_bfloat16*>(cos_sin), num_heads, head_size, rot_dim, is_neox);
  else if (dtype == 1)
    lmc::rerotate_k_kernel<__half><<<T, 256, 0, s>>>(
        static_cast<__half*>(key), ldk, old_pos, new_pos, static_cast<const __half*>(cos_sin),
        num_heads, head_size, rot_dim, is_neox);
  else
    return -8;
  return static_cast<int>(cudaGetLastError());
}

B200_API int b200_lmc_calculate_cdf(const void* input, void* out, int L, int T, int C,
                                    int max_bins, void* stream) {
  if (L <= 0 || C <= 0) return 0;
  if (max_bins <= 0 || max_bins >= 64) return -2;
  dim3 grid((C + 255) / 256, L);
  lmc::cachegen_cdf_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const int8_t*>(input), static_cast<short*>(out), L, T, C, max_bins);
  return static_cast<int>(cudaGetLastError());
}

// Pinned host memory.  numa_node < 0: plain cudaHostAlloc; otherwise page-aligned memory is
// first-touched by the calling thread (run it on a CPU of the wanted node) and registered.
B200_API void* b200_alloc_pinned(unsigned long long size, int numa_node) {
  void* p = nullptr;
  if (numa_node < 0) {
    if (cudaHostAlloc(&p, size, cudaHostAllocDefault) != cudaSuccess) return nullptr;
    return p;
  }
  if (posix_memalign(&p, 4096, size) != 0) return nullptr;
  std::memset(p, 0, size);
  if (cudaHostRegister(p, size, cudaHostRegisterDefault) != cudaSuccess) {
    std::free(p);
    return nullptr;
  }
  return p;
}

B200_API int b200_free_pinned(void* p, int numa_node) {
  if (p == nullptr) return 0;
  if (numa_node < 0) return static_cast<int>(cudaFreeHost(p));
  cudaError_t e = cudaHostUnregister(p);
  std::free(p);
  return static_cast<int>(e);
}

B200_API int b200_gpu_pci_bus_id(int device, char* out, int len) {
  return static_cast<int>(cudaDeviceGetPCIBusId(out, len, device));
}

// ---------------------------------------------------------------------------
// CacheGen arithmetic codec (lmcache/csrc/encode_cuda_new.cpp:29, decode_cuda_new.cpp:28,
// decode_cuda_prefsum.cpp:27): one stream per (layer, token); the C channel symbols of a
// token are coded in order with the per-(layer, channel) cumulative table of
// b200_lmc_calculate_cdf.  Binary arithmetic coder with 32-bit low / high registers and
// carry-less renormalisation (pending underflow bits).  Table entry i is used as
// cdf[i] + i so that every symbol keeps a non-empty interval even when the histogram never
// saw it; encoder and decoder apply the same rule, so any table decodes what it encoded.
// ---------------------------------------------------------------------------
namespace b200 {
namespace lmc {

struct BitWriter {
  uint8_t* dst;
  int cap;
  int nbytes;
  uint32_t acc;
  int nbits;
  bool overflow;
  __device__ void put(uint32_t bit) {
    acc = (acc << 1) | (bit & 1u);
    if (++nbits == 8) {
      if (nbytes < cap) dst[nbytes] = static_cast<uint8_t>(acc);
      else overflow = true;
      ++nbytes;
      acc = 0;
      nbits = 0;
    }
  }
  __device__ void put_with_pending(uint32_t bit, int& pending) {
    put(bit);
    for (; pending > 0; --pending) put(bit ^ 1u);
  }
  __device__ void flush() {
    while (nbits != 0) put(0u);
  }
};

__device__ __forceinline__ uint32_t cdf_at(const unsigned short* row, int i, int bins) {
  return (i >= bins ? 65536u : static_cast<uint32_t>(row[i])) + static_cast<uint32_t>(i);
}

__global__ void cachegen_encode_kernel(const unsigned short* cdf, const int8_t* sym,
                                       uint8_t* out, int* out_len, int L, int T, int C,
                                       int bins, int max_bytes) {
  const int s = blockIdx.x * blockDim.x + threadIdx.x;
  if (s >= L * T) return;
  const int l = s / T;
  const uint32_t total = 65536u + static_cast<uint32_t>(bins);
  BitWriter w{out + static_cast<long long>(s) * max_bytes, max_bytes, 0, 0u, 0, false};
  uint32_t low = 0u, high = 0xFFFFFFFFu;
  int pending = 0;
  const int8_t* src = sym + static_cast<long long>(s) * C;
  for (int c = 0; c < C; ++c) {
    int v = src[c];
    v = v < 0 ? 0 : (v >= bins ? bins - 1 : v);
    const unsigned short* row = cdf + (static_cast<long long>(l) * C + c) * (bins + 1);
    const unsigned long long span = static_cast<unsigned long long>(high) - low + 1ull;
    const uint32_t c_lo = cdf_at(row, v, bins), c_hi = cdf_at(row, v + 1, bins);
    high = low + static_cast<uint32_t>(span * c_hi / total) - 1u;
    low = low + static_cast<uint32_t>(span * c_lo / total);
    for (;;) {
      if (high < 0x80000000u) {
        w.put_with_pending(0u, pending);
      } else if (low >= 0x80000000u) {
        w.put_with_pending(1u, pending);
      } else if (low >= 0x40000000u && high < 0xC0000000u) {
        ++pending;
        low -= 0x40000000u;
        high -= 0x40000000u;
      } else {
        break;
      }
      low <<= 1;
      high = (high << 1) | 1u;
    }
  }
  ++pending;
  w.put_with_pending(low < 0x40000000u ? 0u : 1u, pending);
  w.flush();
  out_len[s] = w.overflow ? -1 : w.nbytes;
}

struct BitReader {
  const uint8_t* src;
  int nbytes;
  int pos;
  __device__ uint32_t get() {
    const int byte = pos >> 3;
    const uint32_t b = byte < nbytes ? (src[byte] >> (7 - (pos & 7))) & 1u : 0u;
    ++pos;
    return b;
  }
};

// offsets != null: packed streams (stream s occupies bytes [offsets[s], offsets[s + 1]));
// otherwise stream s starts at s * max_bytes and lens[s] gives its length.
__global__ void cachegen_decode_kernel(const unsigned short* cdf, const uint8_t* bytes,
                                       const int* lens, const long long* offsets, int8_t* out,
                                       int L, int T, int C, int bins, int max_bytes) {
  const int s = blockIdx.x * blockDim.x + threadIdx.x;
  if (s >= L * T) return;
  const int l = s / T;
  const uint32_t total = 65536u + static_cast<uint32_t>(bins);
  BitReader r;
  if (offsets != nullptr) {
    r.src = bytes + offsets[s];
    r.nbytes = static_cast<int>(offsets[s + 1] - offsets[s]);
  } else {
    r.src = bytes + static_cast<long long>(s) * max_bytes;
    r.nbytes = lens[s] < 0 ? 0 : lens[s];
  }
  r.pos = 0;
  uint32_t low = 0u, high = 0xFFFFFFFFu, code = 0u;
  for (int i = 0; i < 32; ++i) code = (code << 1) | r.get();
  int8_t* dst = out + static_cast<long long>(s) * C;
  for (int c = 0; c < C; ++c) {
    const unsigned short* row = cdf + (static_cast<long long>(l) * C + c) * (bins + 1);
    const unsigned long long span = static_cast<unsigned long long>(high) - low + 1ull;
    const uint32_t target = static_cast<uint32_t>(
        ((static_cast<unsigned long long>(code - low) + 1ull) * total - 1ull) / span);
    int v = 0;
    {   // largest v with cdf'(v) <= target (tables are short: linear scan)
      while (v + 1 < bins && cdf_at(row, v + 1, bins) <= target) ++v;
    }
    dst[c] = static_cast<int8_t>(v);
    const uint32_t c_lo = cdf_at(row, v, bins), c_hi = cdf_at(row, v + 1, bins);
    high = low + static_cast<uint32_t>(span * c_hi / total) - 1u;
    low = low + static_cast<uint32_t>(span * c_lo / total);
    for (;;) {
      if (high < 0x80000000u) {
      } else if (low >= 0x80000000u) {
        low -= 0x80000000u;
        high -= 0x80000000u;
        code -= 0x80000000u;
      } else if (low >= 0x40000000u && high < 0xC0000000u) {
        low -= 0x40000000u;
        high -= 0x40000000u;
        code -= 0x40000000u;
      } else {
        break;
      }
      low <<= 1;
      high = (high << 1) | 1u;
      code = (code << 1) | r.get();
    }
  }
}

}  // namespace lmc
}  // namespace b200

// cdf int16 [L, C, bins + 1] (as produced by b200_lmc_calculate_cdf), sym int8 [L, T, C];
// out uint8 [L * T, max_bytes], out_len int32 [L * T] (bytes used; -1: max_bytes too small).
B200_API int b200_lmc_encode(const void* cdf, const void* sym, void* out, int* out_len, int L,
                             int T, int C, int bins, int max_bytes, void* stream) {
  if (L <= 0 || T <= 0) return 0;
  if (bins <= 0 || bins >= 64 || C <= 0 || max_bytes < 8) return -2;
  const int n = L * T;
  b200::lmc::cachegen_encode_kernel<<<(n + 127) / 128, 128, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const unsigned short*>(cdf), static_cast<const int8_t*>(sym),
      static_cast<uint8_t*>(out), out_len, L, T, C, bins, max_bytes);
  return static_cast<int>(cudaGetLastError());
}

// Inverse of b200_lmc_encode.  Either lens (fixed max_bytes slots) or offsets (int64
// [L * T + 1] prefix sums over packed streams) describes where each stream lies.
B200_API int b200_lmc_decode(const void* cdf, const void* bytes, const int* lens,
                             const long long* offsets, void* out, int L, int T, int C, int bins,
                             int max_bytes, void* stream) {
  if (L <= 0 || T <= 0) return 0;
  if (bins <= 0 || bins >= 64 || C <= 0 || (lens == nullptr && offsets == nullptr)) return -2;
  const int n = L * T;
  b200::lmc::cachegen_decode_kernel<<<(n + 127) / 128, 128, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const unsigned short*>(cdf), static_cast<const uint8_t*>(bytes), lens, offsets,
      static_cast<int8_t*>(out), L, T, C, bins, max_bytes);
  return static_cast<int>(cudaGetLastError());
}
