// Paged decode attention with TMA-fed KV pages (sm_100a), head_dim 128, bf16 / fp16.
//
// Same math and split-KV contract as paged_decode_kernel in attention.cu; what changes is the
// data path.  One producer warp walks the block table and issues one TMA tile copy per
// (16-token page chunk, 64-wide half of the head) straight from the paged cache
// [num_slots, kv_heads * 128] into 128-byte-swizzled shared memory, through a ring of
// mbarrier-guarded stages; four consumer warps (16 tokens each per 64-token tile) read
// their MMA fragments conflict-free from the swizzled tiles.  No thread spends issue slots
// on address generation or cp.async bookkeeping, and several tiles are in flight per CTA,
// which is what a decode step at large batch needs to approach HBM bandwidth.
//
// Every mbarrier wait is bounded (common.cuh); a timeout is reported through the status word
// and the CTA leaves through its normal exit.
#include "common.cuh"

#include <unordered_map>
#include <mutex>

namespace b200 {
namespace attn_tma {

constexpr unsigned int kKernelId = 31;
constexpr int HD = 128;
constexpr int kTile = 64;          // tokens per stage
constexpr int kChunk = 16;         // tokens per TMA box (rows)
constexpr int kHalf = 64;          // elements per TMA box (128 bytes)
constexpr int kStages = 3;
constexpr int kBoxBytes = kChunk * kHalf * 2;               // 2048
constexpr int kStageBytes = 2 * (kTile / kChunk) * 2 * kBoxBytes;  // K + V, 4 chunks, 2 halves = 32768
constexpr int kConsumers = 128;
constexpr int kThreads = kConsumers + 32;
constexpr float kLog2e = 1.4426950408889634f;

template <typename T>
__device__ __forceinline__ void mma16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0,
                                         uint32_t b1) {
  if constexpr (std::is_same<T, __nv_bfloat16>::value) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, "
        "{%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
  } else {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, "
        "{%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
  }
}
template <typename T>
__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
  if constexpr (std::is_same<T, __nv_bfloat16>::value) {
    return pack_bf16x2(lo, hi);
  } else {
    __half2 h = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&h);
  }
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t smem_addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(smem_addr));
}
__device__ __forceinline__ uint32_t lds32(uint32_t smem_addr) {
  uint32_t v;
  asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(smem_addr));
  return v;
}
__device__ __forceinline__ void consumer_bar() { asm volatile("bar.sync 1, 128;" ::: "memory"); }

struct Args {
  const void* q;
  void* out;
  float* tmp_out;
  float* tmp_lse;
  const int* seq_lens;
  const int* block_tables;
  long long ldq, ldo;
  int B, Hq, Hkv, num_splits, max_blocks, block_size;
  float scale;
  unsigned int* status;
};

template <typename T>
__global__ void __launch_bounds__(kThreads)
    paged_decode_tma_kernel(const __grid_constant__ CUtensorMap tmK,
                            const __grid_constant__ CUtensorMap tmV, const Args a) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + kStages * kStageBytes);
  uint64_t* empty_bar = full_bar + kStages;
  volatile uint32_t* abort_flag = reinterpret_cast<uint32_t*>(empty_bar + kStages);

  const int b = blockIdx.x, kvh = blockIdx.y, split = blockIdx.z;
  const int G = a.Hq / a.Hkv;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int seq_len = a.seq_lens[b];
  const int per_split = (seq_len + a.num_splits - 1) / a.num_splits;
  const int chunk = ((per_split + kTile - 1) / kTile) * kTile;
  const int start = split * chunk;
  const int end = min(seq_len, start + chunk);

  if (start >= end) {
    for (int r = 0; r < G; ++r) {
      const int head = kvh * G + r;
      if (a.num_splits > 1) {
        if (threadIdx.x == 0)
          a.tmp_lse[(static_cast<long long>(b) * a.Hq + head) * a.num_splits + split] = -INFINITY;
      } else {
        T* o = static_cast<T*>(a.out) + static_cast<long long>(b) * a.ldo + head * HD;
        for (int d = threadIdx.x; d < HD; d += kThreads) o[d] = from_f32<T>(0.0f);
      }
    }
    return;
  }
  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&full_bar[s], 1);
      mbar_init(&empty_bar[s], 4);
    }
    *abort_flag = 0u;
    mbar_fence_init();
    tma_prefetch_desc(&tmK);
    tma_prefetch_desc(&tmV);
  }
  __syncthreads();
  const int ntiles = (end - start + kTile - 1) / kTile;

  if (warp == 4) {
    // ---------------- producer ----------------
    if (elect_one()) {
      const int* bt = a.block_tables + static_cast<long long>(b) * a.max_blocks;
      int stage = 0;
      uint32_t phase = 0;
      for (int it = 0; it < ntiles; ++it) {
        if (!mbar_wait(&empty_bar[stage], phase ^ 1u, a.status, kKernelId, 0x100u + stage,
                       abort_flag))
          break;
        const int t0 = start + it * kTile;
        int nchunks = (min(end, t0 + kTile) - t0 + kChunk - 1) / kChunk;
        mbar_expect_tx(&full_bar[stage], static_cast<uint32_t>(nchunks) * 4u * kBoxBytes);
        uint8_t* sk = smem + stage * kStageBytes;
        uint8_t* sv = sk + kStageBytes / 2;
        for (int c = 0; c < nchunks; ++c) {
          const int tok = t0 + c * kChunk;
          const int blk = bt[tok / a.block_size];
          const int y = blk * a.block_size + tok % a.block_size;
          const int x = kvh * HD;
          tma_load_2d(sk + (c * 2 + 0) * kBoxBytes, &tmK, &full_bar[stage], x, y);
          tma_load_2d(sk + (c * 2 + 1) * kBoxBytes, &tmK, &full_bar[stage], x + kHalf, y);
          tma_load_2d(sv + (c * 2 + 0) * kBoxBytes, &tmV, &full_bar[stage], x, y);
          tma_load_2d(sv + (c * 2 + 1) * kBoxBytes, &tmV, &full_bar[stage], x + kHalf, y);
        }
        if (++stage == kStages) { stage = 0; phase ^= 1u; }
      }
    }
    return;   // the producer warp takes no part in the merge
  }

  // ---------------- consumers (warps 0..3) ----------------
  constexpr int kKC = HD / 16, kNT = HD / 8;
  const int g = lane >> 2, tig = lane & 3;
  uint32_t qf[kKC][4];
  {
    const T* qb = static_cast<const T*>(a.q) + static_cast<long long>(b) * a.ldq +
                  static_cast<long long>(kvh) * G * HD;
#pragma unroll
    for (int kc = 0; kc < kKC; ++kc) {
      const int c0 = kc * 16 + 2 * tig;
      qf[kc][0] = (g < G) ? *reinterpret_cast<const uint32_t*>(qb + g * HD + c0) : 0u;
      qf[kc][1] = (g + 8 < G) ? *reinterpret_cast<const uint32_t*>(qb + (g + 8) * HD + c0) : 0u;
      qf[kc][2] = (g < G) ? *reinterpret_cast<const uint32_t*>(qb + g * HD + c0 + 8) : 0u;
      qf[kc][3] = (g + 8 < G) ? *reinterpret_cast<const uint32_t*>(qb + (g + 8) * HD + c0 + 8) : 0u;
    }
  }
  float o_acc[kNT][4];
#pragma unroll
  for (int i = 0; i < kNT; ++i) o_acc[i][0] = o_acc[i][1] = o_acc[i][2] = o_acc[i][3] = 0.0f;
  float m_run[2] = {-INFINITY, -INFINITY};
  float l_run[2] = {0.0f, 0.0f};
  const float sl2 = a.scale * kLog2e;
  const uint32_t smem_base = smem_u32(smem);

  int stage = 0;
  uint32_t phase = 0;
  bool ok = true;
  for (int it = 0; it < ntiles && ok; ++it) {
    if (!mbar_wait(&full_bar[stage], phase, a.status, kKernelId, 0x200u + stage, abort_flag)) {
      ok = false;
      break;
    }
    const int tok0 = start + it * kTile + warp * kChunk;
    if (tok0 < end) {
      const uint32_t sk = smem_base + stage * kStageBytes + warp * 2 * kBoxBytes;
      const uint32_t sv = sk + kStageBytes / 2;
      float s[2][4];
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.0f;
        const int row = j * 8 + g;
#pragma unroll
        for (int kc = 0; kc < kKC; ++kc) {
          const int half = kc >> 2;                // (kc * 16) / 64
          const int ch = (kc & 3) * 2;             // 16-byte chunk of the 128-byte row
          const uint32_t rbase = sk + half * kBoxBytes + row * 128 + 4 * tig;
          const uint32_t b0 = lds32(rbase + (((ch) ^ g) << 4));
          const uint32_t b1 = lds32(rbase + (((ch + 1) ^ g) << 4));
          mma16816<T>(s[j], qf[kc], b0, b1);
        }
      }
      float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
      for (int j = 0; j < 2; ++j) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int tok = tok0 + j * 8 + 2 * tig + (e & 1);
          const float v = (tok < end) ? s[j][e] * sl2 : -INFINITY;
          s[j][e] = v;
          mx[e >> 1] = fmaxf(mx[e >> 1], v);
        }
      }
      float corr[2];
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
        mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
        const float m_new = fmaxf(m_run[r], mx[r]);
        corr[r] = exp2f(m_run[r] - m_new);
        m_run[r] = m_new;
        l_run[r] *= corr[r];
      }
#pragma unroll
      for (int j = 0; j < 2; ++j) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float p = exp2f(s[j][e] - m_run[e >> 1]);
          s[j][e] = p;
          l_run[e >> 1] += p;
        }
      }
      uint32_t pf[4];
      pf[0] = pack2<T>(s[0][0], s[0][1]);
      pf[1] = pack2<T>(s[0][2], s[0][3]);
      pf[2] = pack2<T>(s[1][0], s[1][1]);
      pf[3] = pack2<T>(s[1][2], s[1][3]);
      const int mi = lane >> 3, r8 = lane & 7;
      const int vrow = (mi & 1) * 8 + r8;
#pragma unroll
      for (int np = 0; np < kNT / 2; ++np) {
        o_acc[2 * np][0] *= corr[0]; o_acc[2 * np][1] *= corr[0];
        o_acc[2 * np][2] *= corr[1]; o_acc[2 * np][3] *= corr[1];
        o_acc[2 * np + 1][0] *= corr[0]; o_acc[2 * np + 1][1] *= corr[0];
        o_acc[2 * np + 1][2] *= corr[1]; o_acc[2 * np + 1][3] *= corr[1];
        const int d = np * 16 + (mi >> 1) * 8;
        const int half = d >> 6;
        const int ch = (d & 63) >> 3;
        uint32_t vb[4];
        ldmatrix_x4_trans(vb, sv + half * kBoxBytes + vrow * 128 + (((ch) ^ r8) << 4));
        mma16816<T>(o_acc[2 * np], pf, vb[0], vb[1]);
        mma16816<T>(o_acc[2 * np + 1], pf, vb[2], vb[3]);
      }
    }
    __syncwarp();
    if (lane == 0) mbar_arrive(&empty_bar[stage]);
    if (++stage == kStages) { stage = 0; phase ^= 1u; }
  }

#pragma unroll
  for (int r = 0; r < 2; ++r) {
    l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 1);
    l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 2);
  }
  // merge the four consumer warps; the stage memory is free once all of them are here
  consumer_bar();
  float* sm_m = reinterpret_cast<float*>(smem);
  float* sm_l = sm_m + 64;
  float* sm_o = sm_l + 64;
  if (tig == 0) {
    sm_m[warp * 16 + g] = m_run[0];
    sm_m[warp * 16 + g + 8] = m_run[1];
    sm_l[warp * 16 + g] = l_run[0];
    sm_l[warp * 16 + g + 8] = l_run[1];
  }
#pragma unroll
  for (int nt = 0; nt < kNT; ++nt) {
    float* o0 = sm_o + (warp * 16 + g) * HD + nt * 8 + 2 * tig;
    float* o1 = sm_o + (warp * 16 + g + 8) * HD + nt * 8 + 2 * tig;
    o0[0] = o_acc[nt][0]; o0[1] = o_acc[nt][1];
    o1[0] = o_acc[nt][2]; o1[1] = o_acc[nt][3];
  }
  consumer_bar();
  for (int idx = threadIdx.x; idx < G * HD; idx += kConsumers) {
    const int r = idx / HD, d = idx % HD;
    float M = -INFINITY;
#pragma unroll
    for (int w = 0; w < 4; ++w) M = fmaxf(M, sm_m[w * 16 + r]);
    float L = 0.0f, o = 0.0f;
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      const float mw = sm_m[w * 16 + r];
      const float f = (mw == -INFINITY) ? 0.0f : exp2f(mw - M);
      L += sm_l[w * 16 + r] * f;
      o += sm_o[(w * 16 + r) * HD + d] * f;
    }
    const float val = (ok && L > 0.0f) ? o / L : 0.0f;
    const int head = kvh * G + r;
    if (a.num_splits > 1) {
      const long long base = (static_cast<long long>(b) * a.Hq + head) * a.num_splits + split;
      a.tmp_out[base * HD + d] = val;
      if (d == 0) a.tmp_lse[base] = (ok && L > 0.0f) ? M + log2f(L) : -INFINITY;
    } else {
      static_cast<T*>(a.out)[static_cast<long long>(b) * a.ldo + head * HD + d] = from_f32<T>(val);
    }
  }
}

// Tensor maps are cached per (cache base, rows, row elements, dtype): encoding costs a few
// microseconds and the KV caches of a model never move.
struct MapKey {
  const void* base;
  unsigned long long rows, cols;
  int dtype;
  bool operator==(const MapKey& o) const {
    return base == o.base && rows == o.rows && cols == o.cols && dtype == o.dtype;
  }
};
struct MapKeyHash {
  size_t operator()(const MapKey& k) const {
    return std::hash<const void*>()(k.base) ^ (k.rows * 1315423911ull) ^ (k.cols << 7) ^ k.dtype;
  }
};

static int get_map(const void* base, unsigned long long rows, unsigned long long cols,
                   unsigned long long ld_bytes, int dtype, CUtensorMap* out) {
  static std::unordered_map<MapKey, CUtensorMap, MapKeyHash> cache;
  static std::mutex mu;
  MapKey key{base, rows, cols, dtype};
  std::lock_guard<std::mutex> lock(mu);
  auto it = cache.find(key);
  if (it != cache.end()) {
    *out = it->second;
    return 0;
  }
  CUtensorMap m;
  int r = encode_tmap_2d(&m, dtype == 0 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                                        : CU_TENSOR_MAP_DATA_TYPE_FLOAT16,
                         2, base, rows, cols, ld_bytes, kChunk, kHalf, CU_TENSOR_MAP_SWIZZLE_128B);
  if (r != 0) return r;
  if (cache.size() > 4096) cache.clear();
  cache.emplace(key, m);
  *out = m;
  return 0;
}

}  // namespace attn_tma
}  // namespace b200

B200_API int b200_decode_reduce(void* out, long long ldo, float* tmp_out, float* tmp_lse,
                                int num_splits, int B, int Hq, int HD, int dtype, void* stream);

// Same contract as b200_paged_decode for head_dim 128 with the caches laid out as
// [num_slots, Hkv * 128] rows (slot_stride == Hkv * 128, head_stride == 128) and a block size
// that is a multiple of 16.  Returns -20 when the layout does not qualify (callers fall back
// to b200_paged_decode).
B200_API int b200_paged_decode_tma(const void* q, long long ldq, void* out, long long ldo,
                                   const void* k_cache, const void* v_cache,
                                   long long slot_stride, long long head_stride,
                                   long long num_slots, const int* block_tables, int max_blocks,
                                   int block_size, const int* seq_lens, float* tmp_out,
                                   float* tmp_lse, int num_splits, int B, int Hq, int Hkv, int HD,
                                   float scale, int dtype, void* stream) {
  using namespace b200;
  using namespace b200::attn_tma;
  if (B <= 0) return 0;
  if (HD != 128 || (block_size % kChunk) != 0 || head_stride != 128 ||
      slot_stride != static_cast<long long>(Hkv) * 128 || (dtype != 0 && dtype != 1) ||
      Hkv <= 0 || Hq % Hkv != 0 || Hq / Hkv > 16 ||
      (reinterpret_cast<uintptr_t>(k_cache) & 15) || (reinterpret_cast<uintptr_t>(v_cache) & 15))
    return -20;
  if (num_splits < 1) return -2;
  if (num_splits > 1 && (tmp_out == nullptr || tmp_lse == nullptr)) return -5;
  CUtensorMap tmK, tmV;
  const unsigned long long cols = static_cast<unsigned long long>(Hkv) * 128;
  int r = get_map(k_cache, static_cast<unsigned long long>(num_slots), cols, cols * 2, dtype, &tmK);
  if (r != 0) return r < 0 ? -6 : r;
  r = get_map(v_cache, static_cast<unsigned long long>(num_slots), cols, cols * 2, dtype, &tmV);
  if (r != 0) return r < 0 ? -6 : r;
  Args a;
  a.q = q; a.out = out; a.tmp_out = tmp_out; a.tmp_lse = tmp_lse; a.seq_lens = seq_lens;
  a.block_tables = block_tables; a.ldq = ldq; a.ldo = ldo; a.B = B; a.Hq = Hq; a.Hkv = Hkv;
  a.num_splits = num_splits; a.max_blocks = max_blocks; a.block_size = block_size;
  a.scale = scale; a.status = status_ptr();
  constexpr int smem = kStages * kStageBytes + 256 + 1024;
  static_assert(kStages * kStageBytes >= (128 + 4 * 16 * b200::attn_tma::HD) * 4,
                "merge buffer must fit");
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  dim3 grid(B, Hkv, num_splits);
  static bool done0[64] = {false}, done1[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dtype == 0) {
    auto kern = paged_decode_tma_kernel<__nv_bfloat16>;
    if (dev >= 0 && dev < 64 && !done0[dev]) {
      cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
      if (e != cudaSuccess) return static_cast<int>(e);
      done0[dev] = true;
    }
    kern<<<grid, kThreads, smem, s>>>(tmK, tmV, a);
  } else {
    auto kern = paged_decode_tma_kernel<__half>;
    if (dev >= 0 && dev < 64 && !done1[dev]) {
      cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
      if (e != cudaSuccess) return static_cast<int>(e);
      done1[dev] = true;
    }
    kern<<<grid, kThreads, smem, s>>>(tmK, tmV, a);
  }
  int e = static_cast<int>(cudaGetLastError());
  if (e != 0 || num_splits <= 1) return e;
  return b200_decode_reduce(out, ldo, tmp_out, tmp_lse, num_splits, B, Hq, HD, dtype, stream);
}
