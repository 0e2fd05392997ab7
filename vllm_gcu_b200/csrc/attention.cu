// Paged attention for sm_100a over the "flash" cache layout
// [num_blocks, block_size, kv_heads, head_dim]:
//
//   paged_decode     one query token per sequence, GQA heads of one KV head
//                    packed as the M dimension of the tensor-core tile, split-KV
//                    with an LSE-weighted reduction (flash-decoding);
//   varlen_prefill   causal attention of new tokens over cached prefix + themselves
//                    (chunked prefill, prefix-cache hits and plain prefill are the
//                    same code path: the keys always come from the paged cache);
//   merge_attn_states  LSE-weighted merge of two partial results.
//
// Both attention kernels stage K/V pages into shared memory with cp.async,
// double buffered, and use bf16/fp16 mma.m16n8k16 with fp32 online softmax.
// Decode is bound by HBM traffic of the KV cache; the MMA shape is chosen so the
// issue rate never limits the stream.
//
// Reference ops: csrc/src/paged_attention_v1.cpp:68, paged_attention_v2.cpp:65,
// context_attention_forward.cpp:49, merge_attn_states.cpp:20; selection logic
// vllm_gcu/attention/ops/paged_attn.py:100-211.
#include "common.cuh"

namespace b200 {
namespace attn {

constexpr int kTile = 64;     // KV tokens per shared-memory tile
constexpr int kThreads = 128;
constexpr int kPad = 8;       // elements of row padding (bank-conflict-free fragments)
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

__device__ __forceinline__ void cp_async16(void* smem_dst, const void* gsrc) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(smem_dst)), "l"(gsrc)
               : "memory");
}
__device__ __forceinline__ void cp_async_commit() {
  asm volatile("cp.async.commit_group;" ::: "memory");
}
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], const void* smem_row) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(smem_u32(smem_row)));
}

struct KvView {
  const void* k_cache;
  const void* v_cache;
  const int* block_tables;   // [B, max_blocks]
  long long slot_stride;     // elements between consecutive slots
  long long head_stride;     // elements between kv heads inside a slot
  long long num_slots;
  int max_blocks;
  int block_size;
  // 8-bit caches: 0 = cache holds T, 1 = fp8 e4m3 (value = q * scale),
  // 2 = int8 (value = (q - zero_point) * scale).  Strides are then in bytes.
  int qmode = 0;
  float k_scale = 1.0f, v_scale = 1.0f, k_zp = 0.0f, v_zp = 0.0f;
};

// Eight cached 8-bit values -> eight T in shared memory.
template <typename T>
__device__ __forceinline__ void dequant8(T* dst, const uint8_t* src, int qmode, float scale,
                                         float zp) {
  const uint2 raw = *reinterpret_cast<const uint2*>(src);
  const uint8_t* b = reinterpret_cast<const uint8_t*>(&raw);
  float f[8];
#pragma unroll
  for (int i = 0; i < 8; ++i)
    f[i] = qmode == 1 ? e4m3_to_f32(b[i]) * scale
                      : (static_cast<float>(static_cast<int8_t>(b[i])) - zp) * scale;
  vec8_store<T>(dst, f);
}

// Stages KV tokens [t0, t0 + kTile) of sequence `b`, kv head `kvh` into shared
// memory rows of HD + kPad elements.  Rows at or past kv_end are zero filled.
template <typename T, int HD>
__device__ __forceinline__ void load_kv_tile(T* sK, T* sV, const KvView& kv, int b, int kvh,
                                             int t0, int kv_end) {
  constexpr int kStride = HD + kPad;
  constexpr int kChunks = HD / 8;
  const int* bt = kv.block_tables + static_cast<long long>(b) * kv.max_blocks;
  const T* kc = static_cast<const T*>(kv.k_cache);
  const T* vc = static_cast<const T*>(kv.v_cache);
  for (int c = threadIdx.x; c < kTile * kChunks; c += kThreads) {
    const int row = c / kChunks, ch = c % kChunks;
    const int tok = t0 + row;
    T* dk = sK + row * kStride + ch * 8;
    T* dv = sV + row * kStride + ch * 8;
    // a sequence longer than its block-table row reads zeros past the row, never the next row
    bool ok = tok < kv_end && tok / kv.block_size < kv.max_blocks;
    long long slot = 0;
    if (ok) {
      const int blk = bt[tok / kv.block_size];
      slot = static_cast<long long>(blk) * kv.block_size + tok % kv.block_size;
      ok = slot >= 0 && slot < kv.num_slots;  // a bad table entry reads zeros, never memory
    }
    if (ok && kv.qmode != 0) {
      // 8-bit cache: plain loads, dequantised on the way into shared memory
      const long long off = slot * kv.slot_stride + kvh * kv.head_stride + ch * 8;
      dequant8<T>(dk, static_cast<const uint8_t*>(kv.k_cache) + off, kv.qmode, kv.k_scale, kv.k_zp);
      dequant8<T>(dv, static_cast<const uint8_t*>(kv.v_cache) + off, kv.qmode, kv.v_scale, kv.v_zp);
    } else if (ok) {
      const long long off = slot * kv.slot_stride + kvh * kv.head_stride + ch * 8;
      cp_async16(dk, kc + off);
      cp_async16(dv, vc + off);
    } else {
      *reinterpret_cast<uint4*>(dk) = make_uint4(0, 0, 0, 0);
      *reinterpret_cast<uint4*>(dv) = make_uint4(0, 0, 0, 0);
    }
  }
}

// ---------------------------------------------------------------------------
// decode
// ---------------------------------------------------------------------------
struct DecodeArgs {
  const void* q;        // [B, Hq, HD], row pitch ldq
  void* out;            // [B, Hq, HD], row pitch ldo
  float* tmp_out;       // [B, Hq, splits, HD] when splits > 1
  float* tmp_lse;       // [B, Hq, splits] (log2 domain)
  const int* seq_lens;  // [B]
  KvView kv;
  long long ldq, ldo;
  int B, Hq, Hkv, num_splits;
  float scale;
  const float* alibi;   // optional [Hq] slopes: score += slope * (key position - query position)
};

template <typename T, int HD>
__global__ void __launch_bounds__(kThreads) paged_decode_kernel(const DecodeArgs a) {
  constexpr int kStride = HD + kPad;
  constexpr int kKC = HD / 16;  // k-chunks of the QK product
  constexpr int kNT = HD / 8;   // n-tiles of the PV product
  extern __shared__ __align__(16) uint8_t smem_raw[];
  T* stage[2];
  stage[0] = reinterpret_cast<T*>(smem_raw);
  stage[1] = stage[0] + 2 * kTile * kStride;

  const int b = blockIdx.x, kvh = blockIdx.y, split = blockIdx.z;
  const int G = a.Hq / a.Hkv;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, tig = lane & 3;
  const int seq_len = a.seq_lens[b];
  const int per_split = (seq_len + a.num_splits - 1) / a.num_splits;
  const int chunk = ((per_split + kTile - 1) / kTile) * kTile;
  const int start = split * chunk;
  const int end = min(seq_len, start + chunk);

  if (start >= end) {  // nothing in this split (or empty sequence)
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

  // Q fragments: rows = the G query heads that share this KV head (G <= 16)
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
  // ALiBi: the query sits at position seq_len - 1 (log2 domain like the scores)
  float al[2] = {0.0f, 0.0f};
  if (a.alibi != nullptr) {
    if (g < G) al[0] = a.alibi[kvh * G + g] * kLog2e;
    if (g + 8 < G) al[1] = a.alibi[kvh * G + g + 8] * kLog2e;
  }

  const int ntiles = (end - start + kTile - 1) / kTile;
  load_kv_tile<T, HD>(stage[0], stage[0] + kTile * kStride, a.kv, b, kvh, start, end);
  cp_async_commit();

  for (int it = 0; it < ntiles; ++it) {
    const int cur = it & 1;
    if (it + 1 < ntiles) {
      T* nk = stage[cur ^ 1];
      load_kv_tile<T, HD>(nk, nk + kTile * kStride, a.kv, b, kvh, start + (it + 1) * kTile, end);
    }
    cp_async_commit();
    cp_async_wait<1>();
    __syncthreads();

    const T* sK = stage[cur] + warp * 16 * kStride;  // this warp's 16 tokens
    const T* sV = stage[cur] + kTile * kStride + warp * 16 * kStride;
    const int tok0 = start + it * kTile + warp * 16;

    if (tok0 < end) {
      float s[2][4];
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.0f;
#pragma unroll
        for (int kc = 0; kc < kKC; ++kc) {
          const T* kr = sK + (j * 8 + g) * kStride + kc * 16 + 2 * tig;
          const uint32_t b0 = *reinterpret_cast<const uint32_t*>(kr);
          const uint32_t b1 = *reinterpret_cast<const uint32_t*>(kr + 8);
          mma16816<T>(s[j], qf[kc], b0, b1);
        }
      }
      // scale, mask, row max
      float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
      for (int j = 0; j < 2; ++j) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int tok = tok0 + j * 8 + 2 * tig + (e & 1);
          const float v = (tok < end)
                              ? s[j][e] * sl2 + al[e >> 1] * static_cast<float>(tok - (seq_len - 1))
                              : -INFINITY;
          s[j][e] = v;
          mx[e >> 1] = fmaxf(mx[e >> 1], v);
        }
      }
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
        mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
      }
      float corr[2];
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        const float m_new = fmaxf(m_run[r], mx[r]);  // finite: tok0 < end
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
#pragma unroll
      for (int np = 0; np < kNT / 2; ++np) {
        o_acc[2 * np][0] *= corr[0]; o_acc[2 * np][1] *= corr[0];
        o_acc[2 * np][2] *= corr[1]; o_acc[2 * np][3] *= corr[1];
        o_acc[2 * np + 1][0] *= corr[0]; o_acc[2 * np + 1][1] *= corr[0];
        o_acc[2 * np + 1][2] *= corr[1]; o_acc[2 * np + 1][3] *= corr[1];
        uint32_t vb[4];
        const int mi = lane >> 3, r = lane & 7;
        ldmatrix_x4_trans(vb, sV + ((mi & 1) * 8 + r) * kStride + np * 16 + (mi >> 1) * 8);
        mma16816<T>(o_acc[2 * np], pf, vb[0], vb[1]);
        mma16816<T>(o_acc[2 * np + 1], pf, vb[2], vb[3]);
      }
    }
    __syncthreads();  // everyone is done with stage[cur] before it is refilled
  }
  cp_async_wait<0>();

  // quad-reduce the row sums
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 1);
    l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 2);
  }

  // merge the four warps through shared memory (stage memory is free now)
  float* sm_m = reinterpret_cast<float*>(smem_raw);  // [4][16]
  float* sm_l = sm_m + 64;                           // [4][16]
  float* sm_o = sm_l + 64;                           // [4][16][HD]
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
  __syncthreads();
  for (int idx = threadIdx.x; idx < G * HD; idx += kThreads) {
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
    const float val = L > 0.0f ? o / L : 0.0f;
    const int head = kvh * G + r;
    if (a.num_splits > 1) {
      const long long base = (static_cast<long long>(b) * a.Hq + head) * a.num_splits + split;
      a.tmp_out[base * HD + d] = val;
      if (d == 0) a.tmp_lse[base] = L > 0.0f ? M + log2f(L) : -INFINITY;
    } else {
      static_cast<T*>(a.out)[static_cast<long long>(b) * a.ldo + head * HD + d] = from_f32<T>(val);
    }
  }
}

template <typename T, int HD>
__global__ void __launch_bounds__(128) decode_reduce_kernel(const DecodeArgs a) {
  const int b = blockIdx.x, head = blockIdx.y;
  const long long base = (static_cast<long long>(b) * a.Hq + head) * a.num_splits;
  float M = -INFINITY;
  for (int s = 0; s < a.num_splits; ++s) M = fmaxf(M, a.tmp_lse[base + s]);
  for (int d = threadIdx.x; d < HD; d += blockDim.x) {
    float acc = 0.0f, wsum = 0.0f;
    for (int s = 0; s < a.num_splits; ++s) {
      const float l = a.tmp_lse[base + s];
      if (l == -INFINITY) continue;  // empty split: its tmp_out was never written
      const float w = exp2f(l - M);
      wsum += w;
      acc += w * a.tmp_out[(base + s) * HD + d];
    }
    static_cast<T*>(a.out)[static_cast<long long>(b) * a.ldo + head * HD + d] =
        from_f32<T>(wsum > 0.0f ? acc / wsum : 0.0f);
  }
}

// ---------------------------------------------------------------------------
// varlen prefill over the paged cache
// ---------------------------------------------------------------------------
struct PrefillArgs {
  const void* q;          // [T, Hq, HD], row pitch ldq
  void* out;              // [T, Hq, HD], row pitch ldo
  float* lse;             // optional [Hq, T] natural-log LSE
  const int* cu_q;        // [B + 1] query offsets
  const int* seq_lens;    // [B] total kv length (prefix + new tokens)
  KvView kv;
  long long ldq, ldo;
  int B, T, Hq, Hkv;
  int causal;
  int window;             // sliding window (<= 0: none)
  float scale;
  const float* alibi;     // optional [Hq] slopes, see DecodeArgs
};

template <typename T, int HD>
__global__ void __launch_bounds__(kThreads) varlen_prefill_kernel(const PrefillArgs a) {
  constexpr int kStride = HD + kPad;
  constexpr int kKC = HD / 16;
  constexpr int kNT = HD / 8;
  constexpr int kQTile = 64;
  extern __shared__ __align__(16) uint8_t smem_raw[];
  __shared__ int s_b, s_qt;
  T* stage[2];
  stage[0] = reinterpret_cast<T*>(smem_raw);
  stage[1] = stage[0] + 2 * kTile * kStride;

  if (threadIdx.x == 0) {
    int acc = 0, found = -1, qt = 0;
    for (int b = 0; b < a.B; ++b) {
      const int nt = (a.cu_q[b + 1] - a.cu_q[b] + kQTile - 1) / kQTile;
      if (static_cast<int>(blockIdx.x) < acc + nt) {
        found = b;
        qt = blockIdx.x - acc;
        break;
      }
      acc += nt;
    }
    s_b = found;
    s_qt = qt;
  }
  __syncthreads();
  const int b = s_b;
  if (b < 0) return;
  const int head = blockIdx.y;
  const int kvh = head / (a.Hq / a.Hkv);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, tig = lane & 3;
  const int q0 = a.cu_q[b];
  const int q_len = a.cu_q[b + 1] - q0;
  const int kv_len = a.seq_lens[b];
  const int ctx = kv_len - q_len;  // cached tokens before this chunk
  const int row_base = s_qt * kQTile + warp * 16;
  const int rows[2] = {row_base + g, row_base + g + 8};

  uint32_t qf[kKC][4];
  {
    const T* qb = static_cast<const T*>(a.q) + static_cast<long long>(head) * HD;
#pragma unroll
    for (int kc = 0; kc < kKC; ++kc) {
      const int c0 = kc * 16 + 2 * tig;
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        const bool ok = rows[r] < q_len;
        const T* p = qb + static_cast<long long>(q0 + rows[r]) * a.ldq + c0;
        qf[kc][r] = ok ? *reinterpret_cast<const uint32_t*>(p) : 0u;
        qf[kc][r + 2] = ok ? *reinterpret_cast<const uint32_t*>(p + 8) : 0u;
      }
    }
  }
  float o_acc[kNT][4];
#pragma unroll
  for (int i = 0; i < kNT; ++i) o_acc[i][0] = o_acc[i][1] = o_acc[i][2] = o_acc[i][3] = 0.0f;
  float m_run[2] = {-INFINITY, -INFINITY};
  float l_run[2] = {0.0f, 0.0f};
  const float sl2 = a.scale * kLog2e;
  const float al = a.alibi != nullptr ? a.alibi[head] * kLog2e : 0.0f;

  // keys this CTA can see
  const int last_row = min(q_len, s_qt * kQTile + kQTile) - 1;
  int kv_end = a.causal ? min(kv_len, ctx + last_row + 1) : kv_len;
  int kv_begin = 0;
  if (a.window > 0) kv_begin = max(0, ctx + s_qt * kQTile - a.window + 1) / kTile * kTile;
  const int ntiles = (kv_end - kv_begin + kTile - 1) / kTile;

  if (ntiles > 0) {
    load_kv_tile<T, HD>(stage[0], stage[0] + kTile * kStride, a.kv, b, kvh, kv_begin, kv_end);
  }
  cp_async_commit();
  for (int it = 0; it < ntiles; ++it) {
    const int cur = it & 1;
    const int t0 = kv_begin + it * kTile;
    if (it + 1 < ntiles) {
      T* nk = stage[cur ^ 1];
      load_kv_tile<T, HD>(nk, nk + kTile * kStride, a.kv, b, kvh, t0 + kTile, kv_end);
    }
    cp_async_commit();
    cp_async_wait<1>();
    __syncthreads();
    const T* sK = stage[cur];
    const T* sV = stage[cur] + kTile * kStride;

    // the warp can skip tiles that lie entirely above its causal diagonal
    const bool warp_active = !a.causal || t0 <= ctx + row_base + 15;
    if (warp_active) {
      float s[kTile / 8][4];
#pragma unroll
      for (int j = 0; j < kTile / 8; ++j) {
        s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.0f;
#pragma unroll
        for (int kc = 0; kc < kKC; ++kc) {
          const T* kr = sK + (j * 8 + g) * kStride + kc * 16 + 2 * tig;
          mma16816<T>(s[j], qf[kc], *reinterpret_cast<const uint32_t*>(kr),
                      *reinterpret_cast<const uint32_t*>(kr + 8));
        }
      }
      float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
      for (int j = 0; j < kTile / 8; ++j) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int tok = t0 + j * 8 + 2 * tig + (e & 1);
          const int pos = ctx + rows[e >> 1];
          bool ok = tok < kv_end;
          if (a.causal) ok = ok && tok <= pos;
          if (a.window > 0) ok = ok && tok > pos - a.window;
          const float v = ok ? s[j][e] * sl2 + al * static_cast<float>(tok - pos) : -INFINITY;
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
        corr[r] = (m_new == -INFINITY) ? 1.0f : exp2f(m_run[r] - m_new);
        m_run[r] = m_new;
        l_run[r] *= corr[r];
      }
#pragma unroll
      for (int j = 0; j < kTile / 8; ++j) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float mr = m_run[e >> 1];
          const float p = (mr == -INFINITY) ? 0.0f : exp2f(s[j][e] - mr);
          s[j][e] = p;
          l_run[e >> 1] += p;
        }
      }
#pragma unroll
      for (int nt = 0; nt < kNT; ++nt) {
        o_acc[nt][0] *= corr[0]; o_acc[nt][1] *= corr[0];
        o_acc[nt][2] *= corr[1]; o_acc[nt][3] *= corr[1];
      }
#pragma unroll
      for (int kk = 0; kk < kTile / 16; ++kk) {
        uint32_t pf[4];
        pf[0] = pack2<T>(s[2 * kk][0], s[2 * kk][1]);
        pf[1] = pack2<T>(s[2 * kk][2], s[2 * kk][3]);
        pf[2] = pack2<T>(s[2 * kk + 1][0], s[2 * kk + 1][1]);
        pf[3] = pack2<T>(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
        for (int np = 0; np < kNT / 2; ++np) {
          uint32_t vb[4];
          const int mi = lane >> 3, r = lane & 7;
          ldmatrix_x4_trans(
              vb, sV + (kk * 16 + (mi & 1) * 8 + r) * kStride + np * 16 + (mi >> 1) * 8);
          mma16816<T>(o_acc[2 * np], pf, vb[0], vb[1]);
          mma16816<T>(o_acc[2 * np + 1], pf, vb[2], vb[3]);
        }
      }
    }
    __syncthreads();
  }
  cp_async_wait<0>();

#pragma unroll
  for (int r = 0; r < 2; ++r) {
    l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 1);
    l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 2);
  }
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    if (rows[r] >= q_len) continue;
    const float inv = l_run[r] > 0.0f ? 1.0f / l_run[r] : 0.0f;
    T* o = static_cast<T*>(a.out) + static_cast<long long>(q0 + rows[r]) * a.ldo +
           static_cast<long long>(head) * HD;
#pragma unroll
    for (int nt = 0; nt < kNT; ++nt) {
      *reinterpret_cast<uint32_t*>(o + nt * 8 + 2 * tig) =
          pack2<T>(o_acc[nt][2 * r] * inv, o_acc[nt][2 * r + 1] * inv);
    }
    if (a.lse != nullptr && tig == 0) {
      a.lse[static_cast<long long>(head) * a.T + q0 + rows[r]] =
          l_run[r] > 0.0f ? (m_run[r] + log2f(l_run[r])) / kLog2e : -INFINITY;
    }
  }
}

// out = merge(prefix, suffix) with LSE weights; lse tensors are [H, T] (natural log).
template <typename T>
__global__ void __launch_bounds__(128)
    merge_attn_states_kernel(T* out, float* out_lse, const T* p_out, const float* p_lse,
                             const T* s_out, const float* s_lse, int Tn, int H, int Dv) {
  const int t = blockIdx.x, h = blockIdx.y;
  const float pl = p_lse[static_cast<long long>(h) * Tn + t];
  const float sl = s_lse[static_cast<long long>(h) * Tn + t];
  const float pl2 = isinf(pl) && pl > 0 ? -INFINITY : pl;
  const float sl2 = isinf(sl) && sl > 0 ? -INFINITY : sl;
  const float m = fmaxf(pl2, sl2);
  float wp, ws;
  if (m == -INFINITY) {
    wp = ws = 0.0f;
  } else {
    const float ep = __expf(pl2 - m), es = __expf(sl2 - m);
    wp = ep / (ep + es);
    ws = es / (ep + es);
    if (out_lse != nullptr && threadIdx.x == 0)
      out_lse[static_cast<long long>(h) * Tn + t] = m + __logf(ep + es);
  }
  if (m == -INFINITY && out_lse != nullptr && threadIdx.x == 0)
    out_lse[static_cast<long long>(h) * Tn + t] = -INFINITY;
  const long long base = (static_cast<long long>(t) * H + h) * Dv;
  for (int d = threadIdx.x; d < Dv; d += blockDim.x)
    out[base + d] = from_f32<T>(to_f32<T>(p_out[base + d]) * wp + to_f32<T>(s_out[base + d]) * ws);
}

// Opts the kernel into `bytes` of dynamic shared memory, once per device.
template <typename KernelT>
int set_smem(KernelT kern, int bytes, bool (&done)[64]) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return -9;
  if (done[dev]) return 0;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
  if (e != cudaSuccess) return static_cast<int>(e);
  done[dev] = true;
  return 0;
}

template <typename T, int HD>
int launch_decode(const DecodeArgs& a, cudaStream_t s) {
  constexpr int smem = 2 * 2 * kTile * (HD + kPad) * static_cast<int>(sizeof(T));
  static_assert(smem >= (128 + 4 * 16 * HD) * 4, "merge buffer must fit in the stage memory");
  auto kern = paged_decode_kernel<T, HD>;
  static bool done[64] = {false};
  int e = set_smem(kern, smem, done);
  if (e != 0) return e;
  dim3 grid(a.B, a.Hkv, a.num_splits);
  kern<<<grid, kThreads, smem, s>>>(a);
  e = static_cast<int>(cudaGetLastError());
  if (e != 0 || a.num_splits <= 1) return e;
  decode_reduce_kernel<T, HD><<<dim3(a.B, a.Hq), 128, 0, s>>>(a);
  return static_cast<int>(cudaGetLastError());
}

template <typename T, int HD>
int launch_prefill(const PrefillArgs& a, int num_q_tiles, cudaStream_t s) {
  constexpr int smem = 2 * 2 * kTile * (HD + kPad) * static_cast<int>(sizeof(T));
  auto kern = varlen_prefill_kernel<T, HD>;
  static bool done[64] = {false};
  int e = set_smem(kern, smem, done);
  if (e != 0) return e;
  dim3 grid(num_q_tiles, a.Hq);
  kern<<<grid, kThreads, smem, s>>>(a);
  return static_cast<int>(cudaGetLastError());
}

}  // namespace attn
}  // namespace b200

using namespace b200;
using namespace b200::attn;

// Number of KV splits the decode kernel wants for this problem (host helper,
// deterministic: callers size the workspace with it).
B200_API int b200_decode_num_splits(int B, int Hkv, int max_seq_len) {
  const long long ctas = static_cast<long long>(B) * Hkv;
  const int target = 2 * sm_count();
  if (ctas >= target || max_seq_len <= 512) return 1;
  long long s = (target + ctas - 1) / ctas;
  const long long by_len = (max_seq_len + 255) / 256;
  if (s > by_len) s = by_len;
  if (s > 32) s = 32;
  return s < 1 ? 1 : static_cast<int>(s);
}

// Decode attention.  Workspace (only read when num_splits > 1):
//   tmp_out fp32 [B, Hq, num_splits, HD], tmp_lse fp32 [B, Hq, num_splits].
// dtype 0 bf16 / 1 fp16; HD in {64, 128, 256}; Hq / Hkv <= 16.
static int paged_decode_impl(const void* q, long long ldq, void* out, long long ldo,
                             const void* k_cache, const void* v_cache, long long slot_stride,
                             long long head_stride, long long num_slots,
                             const int* block_tables, int max_blocks, int block_size,
                             const int* seq_lens, float* tmp_out, float* tmp_lse,
                             int num_splits, int B, int Hq, int Hkv, int HD, float scale,
                             int dtype, int qmode, float k_scale, float v_scale, float k_zp,
                             float v_zp, void* stream, const float* alibi = nullptr) {
  if (B <= 0) return 0;
  if (Hkv <= 0 || Hq % Hkv != 0 || Hq / Hkv > 16) return -2;
  if (num_splits < 1) return -2;
  if (num_splits > 1 && (tmp_out == nullptr || tmp_lse == nullptr)) return -5;
  DecodeArgs a;
  a.q = q; a.out = out; a.tmp_out = tmp_out; a.tmp_lse = tmp_lse; a.seq_lens = seq_lens;
  a.kv.k_cache = k_cache; a.kv.v_cache = v_cache; a.kv.block_tables = block_tables;
  a.kv.slot_stride = slot_stride; a.kv.head_stride = head_stride; a.kv.num_slots = num_slots;
  a.kv.max_blocks = max_blocks; a.kv.block_size = block_size;
  a.kv.qmode = qmode; a.kv.k_scale = k_scale; a.kv.v_scale = v_scale;
  a.kv.k_zp = k_zp; a.kv.v_zp = v_zp;
  a.ldq = ldq; a.ldo = ldo; a.B = B; a.Hq = Hq; a.Hkv = Hkv; a.num_splits = num_splits;
  a.scale = scale;
  a.alibi = alibi;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
#define B200_DEC(TT, H) return launch_decode<TT, H>(a, s)
  if (dtype == 0) {
    if (HD == 128) B200_DEC(__nv_bfloat16, 128);
    if (HD == 64) B200_DEC(__nv_bfloat16, 64);
    if (HD == 256) B200_DEC(__nv_bfloat16, 256);
  } else if (dtype == 1) {
    if (HD == 128) B200_DEC(__half, 128);
    if (HD == 64) B200_DEC(__half, 64);
    if (HD == 256) B200_DEC(__half, 256);
  }
#undef B200_DEC
  return -8;
}

B200_API int b200_paged_decode(const void* q, long long ldq, void* out, long long ldo,
                               const void* k_cache, const void* v_cache, long long slot_stride,
                               long long head_stride, long long num_slots,
                               const int* block_tables, int max_blocks, int block_size,
                               const int* seq_lens, float* tmp_out, float* tmp_lse,
                               int num_splits, int B, int Hq, int Hkv, int HD, float scale,
                               int dtype, void* stream) {
  return paged_decode_impl(q, ldq, out, ldo, k_cache, v_cache, slot_stride, head_stride, num_slots,
                           block_tables, max_blocks, block_size, seq_lens, tmp_out, tmp_lse,
                           num_splits, B, Hq, Hkv, HD, scale, dtype, 0, 1.0f, 1.0f, 0.0f, 0.0f,
                           stream);
}

// Decode attention with ALiBi position biases: `alibi` holds one fp32 slope per query head and
// slope * (key position - query position) is added to every score before the softmax (the
// `alibi_slopes` operand of the reference's paged_attention_v1,
// vllm_gcu/attention/ops/paged_attn.py:78-162).  A null `alibi` is plain attention.
B200_API int b200_paged_decode_alibi(const void* q, long long ldq, void* out, long long ldo,
                                     const void* k_cache, const void* v_cache,
                                     long long slot_stride, long long head_stride,
                                     long long num_slots, const int* block_tables, int max_blocks,
                                     int block_size, const int* seq_lens, float* tmp_out,
                                     float* tmp_lse, int num_splits, int B, int Hq, int Hkv,
                                     int HD, float scale, int dtype, const float* alibi,
                                     void* stream) {
  return paged_decode_impl(q, ldq, out, ldo, k_cache, v_cache, slot_stride, head_stride, num_slots,
                           block_tables, max_blocks, block_size, seq_lens, tmp_out, tmp_lse,
                           num_splits, B, Hq, Hkv, HD, scale, dtype, 0, 1.0f, 1.0f, 0.0f, 0.0f,
                           stream, alibi);
}

// Decode attention over an 8-bit KV cache (same layout, one byte per element; slot_stride and
// head_stride in bytes).  qmode 1: fp8 e4m3 with per-tensor scales; qmode 2: int8 with scales
// and zero points (the reference's int8 KV cache, vllm_gcu/kernels/quantization/kv_cache.py:12-61).
// Queries and output stay bf16 / fp16 (dtype).
B200_API int b200_paged_decode_q8kv(const void* q, long long ldq, void* out, long long ldo,
                                    const void* k_cache, const void* v_cache,
                                    long long slot_stride, long long head_stride,
                                    long long num_slots, const int* block_tables, int max_blocks,
                                    int block_size, const int* seq_lens, float* tmp_out,
                                    float* tmp_lse, int num_splits, int B, int Hq, int Hkv, int HD,
                                    float scale, int dtype, int qmode, float k_scale,
                                    float v_scale, float k_zp, float v_zp, void* stream) {
  if (qmode != 1 && qmode != 2) return -2;
  return paged_decode_impl(q, ldq, out, ldo, k_cache, v_cache, slot_stride, head_stride, num_slots,
                           block_tables, max_blocks, block_size, seq_lens, tmp_out, tmp_lse,
                           num_splits, B, Hq, Hkv, HD, scale, dtype, qmode, k_scale, v_scale,
                           k_zp, v_zp, stream);
}

// Second pass of split-KV decode: LSE-weighted sum of the per-split partial outputs
// (tmp_out fp32 [B, Hq, num_splits, HD], tmp_lse fp32 [B, Hq, num_splits], log2 domain).
B200_API int b200_decode_reduce(void* out, long long ldo, float* tmp_out, float* tmp_lse,
                                int num_splits, int B, int Hq, int HD, int dtype, void* stream) {
  if (B <= 0 || num_splits <= 1) return 0;
  DecodeArgs a{};
  a.out = out; a.tmp_out = tmp_out; a.tmp_lse = tmp_lse; a.ldo = ldo; a.B = B; a.Hq = Hq;
  a.num_splits = num_splits;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  dim3 grid(B, Hq);
#define B200_RED(TT, H) decode_reduce_kernel<TT, H><<<grid, 128, 0, s>>>(a)
  if (dtype == 0 && HD == 128) B200_RED(__nv_bfloat16, 128);
  else if (dtype == 0 && HD == 64) B200_RED(__nv_bfloat16, 64);
  else if (dtype == 0 && HD == 256) B200_RED(__nv_bfloat16, 256);
  else if (dtype == 1 && HD == 128) B200_RED(__half, 128);
  else if (dtype == 1 && HD == 64) B200_RED(__half, 64);
  else if (dtype == 1 && HD == 256) B200_RED(__half, 256);
  else return -8;
#undef B200_RED
  return static_cast<int>(cudaGetLastError());
}

// Prefill / chunked-prefill / prefix attention.  num_q_tiles must be
// sum_b ceil(q_len_b / 64) (an upper bound is fine: extra CTAs exit).
static int varlen_prefill_impl(const void* q, long long ldq, void* out, long long ldo,
                               float* lse, const int* cu_q, const int* seq_lens,
                               const void* k_cache, const void* v_cache, long long slot_stride,
                               long long head_stride, long long num_slots,
                               const int* block_tables, int max_blocks, int block_size, int B,
                               int T, int num_q_tiles, int Hq, int Hkv, int HD, float scale,
                               int causal, int window, int dtype, int qmode, float k_scale,
                               float v_scale, float k_zp, float v_zp, void* stream,
                               const float* alibi = nullptr) {
  if (B <= 0 || T <= 0 || num_q_tiles <= 0) return 0;
  if (Hkv <= 0 || Hq % Hkv != 0) return -2;
  PrefillArgs a;
  a.q = q; a.out = out; a.lse = lse; a.cu_q = cu_q; a.seq_lens = seq_lens;
  a.kv.k_cache = k_cache; a.kv.v_cache = v_cache; a.kv.block_tables = block_tables;
  a.kv.slot_stride = slot_stride; a.kv.head_stride = head_stride; a.kv.num_slots = num_slots;
  a.kv.max_blocks = max_blocks; a.kv.block_size = block_size;
  a.kv.qmode = qmode; a.kv.k_scale = k_scale; a.kv.v_scale = v_scale;
  a.kv.k_zp = k_zp; a.kv.v_zp = v_zp;
  a.ldq = ldq; a.ldo = ldo; a.B = B; a.T = T; a.Hq = Hq; a.Hkv = Hkv; a.causal = causal;
  a.window = window; a.scale = scale;
  a.alibi = alibi;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
#define B200_PRE(TT, H) return launch_prefill<TT, H>(a, num_q_tiles, s)
  if (dtype == 0) {
    if (HD == 128) B200_PRE(__nv_bfloat16, 128);
    if (HD == 64) B200_PRE(__nv_bfloat16, 64);
  } else if (dtype == 1) {
    if (HD == 128) B200_PRE(__half, 128);
    if (HD == 64) B200_PRE(__half, 64);
  }
#undef B200_PRE
  return -8;
}

B200_API int b200_varlen_prefill(const void* q, long long ldq, void* out, long long ldo,
                                 float* lse, const int* cu_q, const int* seq_lens,
                                 const void* k_cache, const void* v_cache, long long slot_stride,
                                 long long head_stride, long long num_slots,
                                 const int* block_tables, int max_blocks, int block_size, int B,
                                 int T, int num_q_tiles, int Hq, int Hkv, int HD, float scale,
                                 int causal, int window, int dtype, void* stream) {
  return varlen_prefill_impl(q, ldq, out, ldo, lse, cu_q, seq_lens, k_cache, v_cache, slot_stride,
                             head_stride, num_slots, block_tables, max_blocks, block_size, B, T,
                             num_q_tiles, Hq, Hkv, HD, scale, causal, window, dtype, 0, 1.0f, 1.0f,
                             0.0f, 0.0f, stream);
}

// Prefill attention with ALiBi position biases (context_attention_forward with alibi slopes
// and memory_efficient_attention_alibi of the reference, vllm_gcu/attention/ops/paged_attn.py:
// 195-210); see b200_paged_decode_alibi.
B200_API int b200_varlen_prefill_alibi(const void* q, long long ldq, void* out, long long ldo,
                                       float* lse, const int* cu_q, const int* seq_lens,
                                       const void* k_cache, const void* v_cache,
                                       long long slot_stride, long long head_stride,
                                       long long num_slots, const int* block_tables,
                                       int max_blocks, int block_size, int B, int T,
                                       int num_q_tiles, int Hq, int Hkv, int HD, float scale,
                                       int causal, int window, int dtype, const float* alibi,
                                       void* stream) {
  return varlen_prefill_impl(q, ldq, out, ldo, lse, cu_q, seq_lens, k_cache, v_cache, slot_stride,
                             head_stride, num_slots, block_tables, max_blocks, block_size, B, T,
                             num_q_tiles, Hq, Hkv, HD, scale, causal, window, dtype, 0, 1.0f, 1.0f,
                             0.0f, 0.0f, stream, alibi);
}

// Prefill attention over an 8-bit KV cache; see b200_paged_decode_q8kv for qmode and scales.
B200_API int b200_varlen_prefill_q8kv(const void* q, long long ldq, void* out, long long ldo,
                                      float* lse, const int* cu_q, const int* seq_lens,
                                      const void* k_cache, const void* v_cache,
                                      long long slot_stride, long long head_stride,
                                      long long num_slots, const int* block_tables,
                                      int max_blocks, int block_size, int B, int T,
                                      int num_q_tiles, int Hq, int Hkv, int HD, float scale,
                                      int causal, int window, int dtype, int qmode, float k_scale,
                                      float v_scale, float k_zp, float v_zp, void* stream) {
  if (qmode != 1 && qmode != 2) return -2;
  return varlen_prefill_impl(q, ldq, out, ldo, lse, cu_q, seq_lens, k_cache, v_cache, slot_stride,
                             head_stride, num_slots, block_tables, max_blocks, block_size, B, T,
                             num_q_tiles, Hq, Hkv, HD, scale, causal, window, dtype, qmode, k_scale,
                             v_scale, k_zp, v_zp, stream);
}

B200_API int b200_merge_attn_states(void* out, float* out_lse, const void* p_out,
                                    const float* p_lse, const void* s_out, const float* s_lse,
                                    int T, int H, int Dv, int dtype, void* stream) {
  if (T <= 0) return 0;
  dim3 grid(T, H);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (dtype == 0)
    merge_attn_states_kernel<__nv_bfloat16><<<grid, 128, 0, s>>>(
        static_cast<__nv_bfloat16*>(out), out_lse, static_cast<const __nv_bfloat16*>(p_out), p_lse,
        static_cast<const __nv_bfloat16*>(s_out), s_lse, T, H, Dv);
  else if (dtype == 1)
    merge_attn_states_kernel<__half><<<grid, 128, 0, s>>>(
        static_cast<__half*>(out), out_lse, static_cast<const __half*>(p_out), p_lse,
        static_cast<const __half*>(s_out), s_lse, T, H, Dv);
  else
    return -8;
  return static_cast<int>(cudaGetLastError());
}

// ---------------------------------------------------------------------------
// Allocation-free variant of the decode entry point (declared in no_alloc.h)
// ---------------------------------------------------------------------------
#include "no_alloc.h"

#include <cstdio>
#include <mutex>

namespace {

// Split-KV workspace inside the library image.  In host code these names are only
// stand-ins for the symbols; the device addresses come from cudaGetSymbolAddress.
static __device__ __align__(256) float g_noalloc_out[B200_NOALLOC_MAX_OUT_FLOATS];
static __device__ __align__(256) float g_noalloc_lse[B200_NOALLOC_MAX_LSE_FLOATS];

thread_local char t_noalloc_err[256] = "";

struct NoAllocPtrs {
  float* out = nullptr;
  float* lse = nullptr;
};

// Resolved once per device, with that device current.  std::call_once orders the stores to
// the cache entry before every later reader on any host thread.
int noalloc_ptrs(NoAllocPtrs* res) {
  constexpr int kMaxDevices = 64;
  static NoAllocPtrs cache[kMaxDevices];
  static cudaError_t setup_err[kMaxDevices];
  static std::once_flag once[kMaxDevices];
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) {
    snprintf(t_noalloc_err, sizeof(t_noalloc_err), "cudaGetDevice failed: %s",
             cudaGetErrorString(e));
    return B200_NOALLOC_SETUP_FAILED;
  }
  if (dev < 0 || dev >= kMaxDevices) {
    snprintf(t_noalloc_err, sizeof(t_noalloc_err),
             "device ordinal %d is outside the %d devices this entry point keeps a workspace "
             "address for", dev, kMaxDevices);
    return B200_NOALLOC_SETUP_FAILED;
  }
  std::call_once(once[dev], [dev]() {
    void* po = nullptr;
    void* pl = nullptr;
    cudaError_t e2 = cudaGetSymbolAddress(&po, g_noalloc_out);
    if (e2 == cudaSuccess) e2 = cudaGetSymbolAddress(&pl, g_noalloc_lse);
    if (e2 == cudaSuccess && (po == nullptr || pl == nullptr)) e2 = cudaErrorInvalidSymbol;
    setup_err[dev] = e2;
    cache[dev].lse = static_cast<float*>(pl);
    cache[dev].out = static_cast<float*>(po);
  });
  if (setup_err[dev] != cudaSuccess) {
    snprintf(t_noalloc_err, sizeof(t_noalloc_err),
             "cudaGetSymbolAddress for the built-in workspace failed: %s",
             cudaGetErrorString(setup_err[dev]));
    return B200_NOALLOC_SETUP_FAILED;
  }
  *res = cache[dev];
  return 0;
}

}  // namespace

B200_API const char* b200_noalloc_last_error(void) { return t_noalloc_err; }

B200_API int b200_paged_decode_noalloc(const void* q, long long ldq, void* out, long long ldo,
                                       const void* k_cache, const void* v_cache,
                                       long long slot_stride, long long head_stride,
                                       long long num_slots, const int* block_tables,
                                       int max_blocks, int block_size, const int* seq_lens,
                                       int num_splits, int B, int Hq, int Hkv, int HD, float scale,
                                       int dtype, void* stream) {
  t_noalloc_err[0] = 0;
  if (B <= 0) return 0;
  if (num_splits < 1) {
    snprintf(t_noalloc_err, sizeof(t_noalloc_err), "num_splits must be at least 1 (got %d)",
             num_splits);
    return -2;   // the code b200_paged_decode returns for the same argument
  }
  const long long need_out = static_cast<long long>(B) * Hq * num_splits * HD;
  const long long need_lse = static_cast<long long>(B) * Hq * num_splits;
  if (num_splits > 1 &&
      (need_out > B200_NOALLOC_MAX_OUT_FLOATS || need_lse > B200_NOALLOC_MAX_LSE_FLOATS)) {
    snprintf(t_noalloc_err, sizeof(t_noalloc_err),
             "problem needs %lld + %lld workspace floats, the built-in workspace holds %d + %d "
             "(reduce B * Hq * num_splits * HD or use b200_paged_decode with your own workspace)",
             need_out, need_lse, B200_NOALLOC_MAX_OUT_FLOATS, B200_NOALLOC_MAX_LSE_FLOATS);
    return B200_NOALLOC_TOO_LARGE;
  }
  NoAllocPtrs ws;
  const int rc = noalloc_ptrs(&ws);
  if (rc != 0) return rc;
  const int r = b200_paged_decode(q, ldq, out, ldo, k_cache, v_cache, slot_stride, head_stride,
                                  num_slots, block_tables, max_blocks, block_size, seq_lens,
                                  ws.out, ws.lse, num_splits, B, Hq, Hkv, HD, scale, dtype, stream);
  if (r != 0)
    snprintf(t_noalloc_err, sizeof(t_noalloc_err), "b200_paged_decode returned %d", r);
  return r;
}
