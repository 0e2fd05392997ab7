// Shared device-side building blocks for the sm_100a kernels of this library:
// mbarrier / TMA / tcgen05 PTX wrappers, bounded waits and the status word.
//
// Every wait in this library is bounded.  A wait that runs out records a code
// in the status word (read by b200_status_take() on the host) and makes the
// kernel leave through its normal exit path, so TMEM is released and the
// context stays usable.
#pragma once

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <type_traits>

#define B200_API extern "C" __attribute__((visibility("default")))

namespace b200 {

// ---------------------------------------------------------------------------
// status word (one per loaded library image and device)
// ---------------------------------------------------------------------------
enum StatusCode : unsigned int {
  kStatusOk = 0,
  kStatusMbarTimeout = 1,    // an mbarrier wait ran out
  kStatusFlagTimeout = 2,    // a wait on a peer / host flag ran out
  kStatusBounds = 3,         // an index guard caught an out-of-range value
};

// Layout of the status word (device global memory, one per device; kernels get
// its address as a parameter): [0] first non-zero code, [1] kernel id,
// [2] detail (barrier index / peer), [3] number of reports.
__device__ __forceinline__ void report_status(unsigned int* st, unsigned int code,
                                              unsigned int kernel_id, unsigned int detail) {
  if (st == nullptr) return;
  if (atomicCAS(&st[0], 0u, code) == 0u) {
    st[1] = kernel_id;
    st[2] = detail;
  }
  atomicAdd(&st[3], 1u);
}

// Spin budget of waits on flags that another GPU (or the host) writes.  Word [4] of the status
// block overrides it at run time (0 = this default), see b200_set_flag_wait_limit: a short
// budget lets a test watch a wait run out without waiting for a second.
constexpr uint32_t kFlagSpinLimit = 1u << 22;
__device__ __forceinline__ uint32_t flag_spin_limit(const unsigned int* st) {
  if (st == nullptr) return kFlagSpinLimit;
  const uint32_t v = *reinterpret_cast<const volatile unsigned int*>(st + 4);
  return v != 0u ? v : kFlagSpinLimit;
}

// Spin budget for mbarrier waits.  try_wait suspends for a hardware-chosen
// interval each call, so this many polls is on the order of a second.
constexpr uint32_t kMbarSpinLimit = 1u << 24;

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ bool elect_one() {
  uint32_t pred;
  asm volatile(
      "{\n\t"
      ".reg .pred P;\n\t"
      "elect.sync _|P, 0xffffffff;\n\t"
      "selp.b32 %0, 1, 0, P;\n\t"
      "}\n"
      : "=r"(pred));
  return pred != 0;
}

// ---------------------------------------------------------------------------
// mbarrier
// ---------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}

__device__ __forceinline__ void mbar_fence_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)),
               "r"(bytes)
               : "memory");
}

__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

__device__ __forceinline__ bool mbar_test(uint64_t* bar, uint32_t parity) {
  uint32_t done;
  asm volatile(
      "{\n\t"
      ".reg .pred P;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 P, [%1], %2;\n\t"
      "selp.b32 %0, 1, 0, P;\n\t"
      "}\n"
      : "=r"(done)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return done != 0;
}

// Bounded wait.  Returns false when the budget ran out (status recorded).
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, unsigned int* st,
                                          unsigned int kernel_id, unsigned int detail,
                                          volatile uint32_t* abort_flag = nullptr) {
  for (uint32_t it = 0; it < kMbarSpinLimit; ++it) {
    if (mbar_test(bar, parity)) return true;
    if (abort_flag != nullptr && (it & 1023u) == 1023u && *abort_flag != 0u) return false;
  }
  report_status(st, kStatusMbarTimeout, kernel_id, detail);
  if (abort_flag != nullptr) *abort_flag = 1u;
  return false;
}

// ---------------------------------------------------------------------------
// TMA (tiled bulk tensor copies, never with cluster multicast)
// ---------------------------------------------------------------------------
__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap* m) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(m)) : "memory");
}

// 2-D tile load global -> shared, completion on an mbarrier of this CTA.
// x is the innermost coordinate; x * element size must be a multiple of 16 B.
__device__ __forceinline__ void tma_load_2d(void* smem_dst, const CUtensorMap* m, uint64_t* bar,
                                            int32_t x, int32_t y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cta.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4}], [%2];"
      :
      : "r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(m)), "r"(smem_u32(bar)), "r"(x),
        "r"(y)
      : "memory");
}

// Brings a 2-D tile into L2 only (no shared-memory destination, no completion to wait for).
__device__ __forceinline__ void tma_prefetch_2d(const CUtensorMap* m, int32_t x, int32_t y) {
  asm volatile("cp.async.bulk.prefetch.tensor.2d.L2.global [%0, {%1, %2}];"
               :
               : "l"(reinterpret_cast<uint64_t>(m)), "r"(x), "r"(y)
               : "memory");
}

__device__ __forceinline__ void tma_load_3d(void* smem_dst, const CUtensorMap* m, uint64_t* bar,
                                            int32_t x, int32_t y, int32_t z) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cta.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4, %5}], [%2];"
      :
      : "r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(m)), "r"(smem_u32(bar)), "r"(x),
        "r"(y), "r"(z)
      : "memory");
}

// 2-D tile store shared -> global (bulk async group).
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* m, const void* smem_src, int32_t x,
                                             int32_t y) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];"
               :
               : "l"(reinterpret_cast<uint64_t>(m)), "r"(smem_u32(smem_src)), "r"(x), "r"(y)
               : "memory");
}
__device__ __forceinline__ void tma_store_commit() {
  asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}
template <int N>
__device__ __forceinline__ void tma_store_wait_read() {
  asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
template <int N>
__device__ __forceinline__ void tma_store_wait() {
  asm volatile("cp.async.bulk.wait_group %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

// ---------------------------------------------------------------------------
// tcgen05 (5th generation tensor cores, accumulators in tensor memory)
// ---------------------------------------------------------------------------
__device__ __forceinline__ void tmem_alloc(uint32_t* smem_result, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                   smem_u32(smem_result)),
               "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tc_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}

// D[tmem] (+)= A[smem] * B[smem], issued by one thread.  kind::f16 covers
// fp16 and bf16 operands with fp32 accumulation.
__device__ __forceinline__ void umma_f16(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b,
                                         uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t"
      "}\n"
      :
      : "r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}
// fp8 (e4m3 / e5m2) operands, fp32 accumulation, K = 32 per instruction.
__device__ __forceinline__ void umma_f8(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b,
                                        uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t"
      "}\n"
      :
      : "r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}
// int8 operands, int32 accumulation, K = 32 per instruction.
__device__ __forceinline__ void umma_i8(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b,
                                        uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t"
      "}\n"
      :
      : "r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate)
      : "memory");
}

// Make an mbarrier of this CTA track completion of all tcgen05 ops issued so
// far by this thread (implies tcgen05.fence::before_thread_sync).
__device__ __forceinline__ void umma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                   smem_u32(bar))
               : "memory");
}

// 32 lanes x 32 columns of 32-bit accumulators -> 32 registers per thread
// (thread i of the warp reads TMEM lane base+i, columns col .. col+31).
__device__ __forceinline__ void tmem_ld_32x32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]),
        "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
        "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() {
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
// Stores 32 consecutive fp32 columns of this thread's TMEM lane (counterpart of
// tmem_ld_32x32); complete after tmem_st_wait().
__device__ __forceinline__ void tmem_st_32x32(uint32_t taddr, const uint32_t* r) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
      :
      : "r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]),
        "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]),
        "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]),
        "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]),
        "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
      : "memory");
}
__device__ __forceinline__ void tmem_st_wait() {
  asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}
// Makes generic-proxy writes to shared memory visible to the async proxy (TMA, tcgen05.mma).
__device__ __forceinline__ void fence_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

// Shared-memory matrix descriptor for a K-major operand tile stored as rows of
// 128 bytes with the 128-byte swizzle that TMA SWIZZLE_128B produces.  Eight
// rows form one 1024-byte swizzle atom; atoms follow each other along M/N
// (stride byte offset 1024).  The tile base must be 1024-byte aligned; a K
// step inside the atom is a plain byte advance of the start address.
__device__ __forceinline__ uint64_t make_desc_k_sw128(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr & 0x3FFFFu) >> 4);  // start address
  d |= static_cast<uint64_t>(1) << 16;                       // leading byte offset (unused)
  d |= static_cast<uint64_t>(1024 >> 4) << 32;               // stride byte offset
  d |= static_cast<uint64_t>(1) << 46;                       // descriptor version (sm_100)
  d |= static_cast<uint64_t>(2) << 61;                       // SWIZZLE_128B
  return d;
}

// Descriptor of an MN-major operand tile (the contraction index runs over rows of 128 bytes,
// 64 elements of the M/N extent are contiguous in a row; this is how a [keys, head_dim] value
// tile lands in shared memory under TMA SWIZZLE_128B).  Eight rows form a 1024-byte atom and
// atoms follow each other along K (stride byte offset 1024); the next 64 elements of the M/N
// extent start `mn_chunk_bytes` further (leading byte offset).  A step of 16 along K advances
// the start address by 2048 bytes.  Needs the MN-major bit of the instruction descriptor.
__device__ __forceinline__ uint64_t make_desc_mn_sw128(uint32_t smem_addr, uint32_t mn_chunk_bytes) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr & 0x3FFFFu) >> 4);
  d |= static_cast<uint64_t>((mn_chunk_bytes >> 4) & 0x3FFFu) << 16;
  d |= static_cast<uint64_t>(1024 >> 4) << 32;
  d |= static_cast<uint64_t>(1) << 46;
  d |= static_cast<uint64_t>(2) << 61;
  return d;
}
constexpr uint32_t kIdescBMajorMN = 1u << 16;   // instruction descriptor: B operand is MN-major

// Instruction descriptor, dense, fp32 accumulate, both operands K-major.
// fmt: 0 = f16, 1 = bf16 for kind::f16; 0 = e4m3, 1 = e5m2 for kind::f8f6f4.
__host__ __device__ constexpr uint32_t make_idesc(uint32_t m, uint32_t n, uint32_t a_fmt,
                                                  uint32_t b_fmt, uint32_t c_fmt = 1) {
  return (c_fmt << 4) | (a_fmt << 7) | (b_fmt << 10) | ((n >> 3) << 17) | ((m >> 4) << 24);
}

// ---------------------------------------------------------------------------
// small math / packing helpers
// ---------------------------------------------------------------------------
__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}
__device__ __forceinline__ float2 unpack_bf16x2(uint32_t u) {
  __nv_bfloat162 v = *reinterpret_cast<__nv_bfloat162*>(&u);
  return __bfloat1622float2(v);
}
__device__ __forceinline__ float silu_f(float x) { return x / (1.0f + __expf(-x)); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Block-wide sum for up to 1024 threads; `red` is 32 floats of shared memory.
__device__ __forceinline__ float block_sum(float v, float* red) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  const int nw = (blockDim.x + 31) >> 5;
  float t = (lane < nw) ? red[lane] : 0.0f;
  t = warp_sum(t);
  return t;
}
__device__ __forceinline__ float block_max(float v, float* red) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  v = warp_max(v);
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  const int nw = (blockDim.x + 31) >> 5;
  float t = (lane < nw) ? red[lane] : -INFINITY;
  t = warp_max(t);
  return t;
}

// 8 x 16-bit elements <-> 8 floats through one 16-byte access.
template <typename T>
__device__ __forceinline__ void vec8_load(const T* p, float (&f)[8]) {
  static_assert(sizeof(T) == 2, "16-bit element types only");
  const uint4 u = *reinterpret_cast<const uint4*>(p);
  const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float2 x;
    if constexpr (std::is_same<T, __nv_bfloat16>::value) {
      x = unpack_bf16x2(w[i]);
    } else {
      __half2 h = *reinterpret_cast<const __half2*>(&w[i]);
      x = __half22float2(h);
    }
    f[2 * i] = x.x;
    f[2 * i + 1] = x.y;
  }
}
template <typename T>
__device__ __forceinline__ void vec8_store(T* p, const float (&f)[8]) {
  static_assert(sizeof(T) == 2, "16-bit element types only");
  uint32_t w[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    if constexpr (std::is_same<T, __nv_bfloat16>::value) {
      w[i] = pack_bf16x2(f[2 * i], f[2 * i + 1]);
    } else {
      __half2 h = __floats2half2_rn(f[2 * i], f[2 * i + 1]);
      w[i] = *reinterpret_cast<uint32_t*>(&h);
    }
  }
  *reinterpret_cast<uint4*>(p) = make_uint4(w[0], w[1], w[2], w[3]);
}
template <typename T>
__device__ __forceinline__ float to_f32(T v) {
  if constexpr (std::is_same<T, __nv_bfloat16>::value) return __bfloat162float(v);
  else if constexpr (std::is_same<T, __half>::value) return __half2float(v);
  else return static_cast<float>(v);
}
template <typename T>
__device__ __forceinline__ T from_f32(float v) {
  if constexpr (std::is_same<T, __nv_bfloat16>::value) return __float2bfloat16(v);
  else if constexpr (std::is_same<T, __half>::value) return __float2half(v);
  else return static_cast<T>(v);
}
template <typename T>
__device__ __forceinline__ float round_like(float v) {
  return to_f32<T>(from_f32<T>(v));
}
__device__ __forceinline__ uint8_t f32_to_e4m3(float v) {
  return static_cast<uint8_t>(__nv_cvt_float_to_fp8(v, __NV_SATFINITE, __NV_E4M3));
}
__device__ __forceinline__ float e4m3_to_f32(uint8_t v) {
  __half_raw h = __nv_cvt_fp8_to_halfraw(static_cast<__nv_fp8_storage_t>(v), __NV_E4M3);
  return __half2float(*reinterpret_cast<__half*>(&h));
}

}  // namespace b200

// ---------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------
namespace b200 {

// Encodes a 2-D row-major tensor map: `rows` x `cols` elements, row pitch
// `ld_bytes`, box = box_rows x box_cols, given swizzle.  Returns 0 on success.
int encode_tmap_2d(CUtensorMap* out, CUtensorMapDataType dt, int elt_bytes, const void* base,
                   uint64_t rows, uint64_t cols, uint64_t ld_bytes, uint32_t box_rows,
                   uint32_t box_cols, CUtensorMapSwizzle swz);

int encode_tmap_3d(CUtensorMap* out, CUtensorMapDataType dt, int elt_bytes, const void* base,
                   uint64_t d2, uint64_t d1, uint64_t d0, uint64_t stride2_bytes,
                   uint64_t stride1_bytes, uint32_t box2, uint32_t box1, uint32_t box0,
                   CUtensorMapSwizzle swz);

int sm_count();

// Device address of the status word of the current device (null on failure).
unsigned int* status_ptr();

}  // namespace b200
