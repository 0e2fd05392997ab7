// RMSNorm family for sm_100a: plain / fused residual-add, optionally followed
// by quantisation in the same pass (static fp8, dynamic per-token fp8, dynamic
// 1x128-group fp8, static int8, dynamic per-token int8), plus LayerNorm with
// static int8 output.
//
// One CTA per row, 16-byte vector accesses, fp32 statistics.  The row is read
// from HBM once; the later passes hit L1/L2.
//
// Semantics follow the reference ops rms_norm / fused_add_rms_norm
// (csrc/src/rms_norm.cpp:38, csrc/src/fused_add_rms_norm.cpp:40,
// vllm_gcu/kernels/layernorm.py:10-41) and the norm+quant family
// (csrc/src/rms_norm_per_token_group_quant_fp8.cpp:24,
// csrc/src/fused_add_rms_norm_static_fp8_quant.cpp, ..._int8_quant.cpp:27,
// csrc/src/layer_norm_static_int8_quant.cpp:39).
#include "common.cuh"

namespace b200 {
namespace norm {

enum QMode : int {
  kQNone = 0,
  kQFp8Static = 1,
  kQFp8Token = 2,
  kQFp8Group128 = 3,
  kQInt8Static = 4,
  kQInt8Token = 5,
};

constexpr float kFp8Max = 448.0f;

template <typename T>
struct Vec8 {
  uint4 raw;
};

template <typename T>
__device__ __forceinline__ void load8(const T* p, float (&f)[8]);
template <>
__device__ __forceinline__ void load8<__nv_bfloat16>(const __nv_bfloat16* p, float (&f)[8]) {
  uint4 u = *reinterpret_cast<const uint4*>(p);
  float2 a = unpack_bf16x2(u.x), b = unpack_bf16x2(u.y), c = unpack_bf16x2(u.z),
         d = unpack_bf16x2(u.w);
  f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y; f[4] = c.x; f[5] = c.y; f[6] = d.x; f[7] = d.y;
}
template <>
__device__ __forceinline__ void load8<__half>(const __half* p, float (&f)[8]) {
  uint4 u = *reinterpret_cast<const uint4*>(p);
  const __half2* h = reinterpret_cast<const __half2*>(&u);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float2 x = __half22float2(h[i]);
    f[2 * i] = x.x;
    f[2 * i + 1] = x.y;
  }
}
template <typename T>
__device__ __forceinline__ void store8(T* p, const float (&f)[8]);
template <>
__device__ __forceinline__ void store8<__nv_bfloat16>(__nv_bfloat16* p, const float (&f)[8]) {
  uint4 u;
  u.x = pack_bf16x2(f[0], f[1]);
  u.y = pack_bf16x2(f[2], f[3]);
  u.z = pack_bf16x2(f[4], f[5]);
  u.w = pack_bf16x2(f[6], f[7]);
  *reinterpret_cast<uint4*>(p) = u;
}
template <>
__device__ __forceinline__ void store8<__half>(__half* p, const float (&f)[8]) {
  uint4 u;
  __half2* h = reinterpret_cast<__half2*>(&u);
#pragma unroll
  for (int i = 0; i < 4; ++i) h[i] = __floats2half2_rn(f[2 * i], f[2 * i + 1]);
  *reinterpret_cast<uint4*>(p) = u;
}

// Rounds the value the way the output type will (so quantisation sees what an
// unfused norm followed by a quant op would see).
template <typename T>
__device__ __forceinline__ float round_to(float v);
template <>
__device__ __forceinline__ float round_to<__nv_bfloat16>(float v) {
  return __bfloat162float(__float2bfloat16(v));
}
template <>
__device__ __forceinline__ float round_to<__half>(float v) {
  return __half2float(__float2half(v));
}

__device__ __forceinline__ uint8_t to_fp8(float v) {
  return static_cast<uint8_t>(__nv_cvt_float_to_fp8(v, __NV_SATFINITE, __NV_E4M3));
}
__device__ __forceinline__ int8_t to_int8(float v) {
  float r = rintf(v);
  r = fminf(fmaxf(r, -128.0f), 127.0f);
  return static_cast<int8_t>(r);
}

struct Args {
  const void* x;         // [T, H] input (also normed output when out == nullptr and no quant)
  void* residual;        // [T, H] in/out when ADD
  const void* weight;    // [H]
  const void* bias;      // [H] LayerNorm only
  void* out;             // [T, H] T or quantised bytes
  float* scale_out;      // dynamic modes: [T] or [T, H/128]
  const float* scale_in; // static modes: scalar
  const int* valid_rows; // optional device count of valid rows
  long long ldx, ldr, ldo;
  int T, H;
  float eps;
  int layer_norm;
};

template <typename T, int QMODE, bool ADD>
__global__ void __launch_bounds__(1024) rms_norm_kernel(const Args a) {
  __shared__ float red[32];
  const int row = blockIdx.x;
  if (a.valid_rows != nullptr && row >= *a.valid_rows) return;
  const T* x = static_cast<const T*>(a.x) + static_cast<long long>(row) * a.ldx;
  T* res = ADD ? static_cast<T*>(a.residual) + static_cast<long long>(row) * a.ldr : nullptr;
  const T* w = static_cast<const T*>(a.weight);
  const int nvec = a.H >> 3;

  // pass 1: (residual add) + statistics
  float sumsq = 0.0f, sum = 0.0f;
  for (int v = threadIdx.x; v < nvec; v += blockDim.x) {
    float f[8];
    load8<T>(x + v * 8, f);
    if constexpr (ADD) {
      float r[8];
      load8<T>(res + v * 8, r);
#pragma unroll
      for (int i = 0; i < 8; ++i) f[i] = round_to<T>(f[i] + r[i]);
      store8<T>(res + v * 8, f);
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      sumsq += f[i] * f[i];
      sum += f[i];
    }
  }
  sumsq = block_sum(sumsq, red);
  float mean = 0.0f, rstd;
  if (a.layer_norm) {
    sum = block_sum(sum, red);
    mean = sum / a.H;
    rstd = rsqrtf(fmaxf(sumsq / a.H - mean * mean, 0.0f) + a.eps);
  } else {
    rstd = rsqrtf(sumsq / a.H + a.eps);
  }
  const T* src = ADD ? res : x;
  const T* bias = static_cast<const T*>(a.bias);

  auto normed = [&](int v, float (&f)[8]) {
    float wv[8];
    load8<T>(src + v * 8, f);
    load8<T>(w + v * 8, wv);
#pragma unroll
    for (int i = 0; i < 8; ++i) f[i] = round_to<T>((f[i] - mean) * rstd * wv[i]);
    if (bias != nullptr) {
      float bv[8];
      load8<T>(bias + v * 8, bv);
#pragma unroll
      for (int i = 0; i < 8; ++i) f[i] = round_to<T>(f[i] + bv[i]);
    }
  };

  if constexpr (QMODE == kQNone) {
    T* out = static_cast<T*>(a.out) + static_cast<long long>(row) * a.ldo;
    for (int v = threadIdx.x; v < nvec; v += blockDim.x) {
      float f[8];
      normed(v, f);
      store8<T>(out + v * 8, f);
    }
  } else if constexpr (QMODE == kQFp8Group128) {
    // 16 consecutive threads own one group of 128 elements
    uint8_t* out = static_cast<uint8_t*>(a.out) + static_cast<long long>(row) * a.ldo;
    float* sc = a.scale_out + static_cast<long long>(row) * (a.H >> 7);
    const int nvec_pad = (nvec + 31) & ~31;  // whole warps stay in the loop
    for (int v = threadIdx.x; v < nvec_pad; v += blockDim.x) {
      float f[8];
      float amax = 0.0f;
      const bool ok = v < nvec;
      if (ok) {
        normed(v, f);
#pragma unroll
        for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(f[i]));
      }
#pragma unroll
      for (int o = 8; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
      const float s = fmaxf(amax, 1e-10f) / kFp8Max;
      if (ok) {
        const float inv = 1.0f / s;
        uint2 pk;
        uint8_t* b = reinterpret_cast<uint8_t*>(&pk);
#pragma unroll
        for (int i = 0; i < 8; ++i) b[i] = to_fp8(f[i] * inv);
        *reinterpret_cast<uint2*>(out + v * 8) = pk;
        if ((v & 15) == 0) sc[v >> 4] = s;
      }
    }
  } else {
    float scale;
    if constexpr (QMODE == kQFp8Token || QMODE == kQInt8Token) {
      float amax = 0.0f;
      for (int v = threadIdx.x; v < nvec; v += blockDim.x) {
        float f[8];
        normed(v, f);
#pragma unroll
        for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(f[i]));
      }
      amax = block_max(amax, red);
      scale = fmaxf(amax, 1e-10f) / (QMODE == kQFp8Token ? kFp8Max : 127.0f);
      if (threadIdx.x == 0) a.scale_out[row] = scale;
    } else {
      scale = *a.scale_in;
    }
    const float inv = 1.0f / scale;
    uint8_t* out = static_cast<uint8_t*>(a.out) + static_cast<long long>(row) * a.ldo;
    for (int v = threadIdx.x; v < nvec; v += blockDim.x) {
      float f[8];
      normed(v, f);
      uint2 pk;
      uint8_t* b = reinterpret_cast<uint8_t*>(&pk);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        if constexpr (QMODE == kQFp8Static || QMODE == kQFp8Token)
          b[i] = to_fp8(f[i] * inv);
        else
          b[i] = static_cast<uint8_t>(to_int8(f[i] * inv));
      }
      *reinterpret_cast<uint2*>(out + v * 8) = pk;
    }
  }
}

template <typename T, int QMODE>
int launch2(const Args& a, bool add, cudaStream_t s) {
  int threads = ((a.H >> 3) + 31) & ~31;
  if (threads > 1024) threads = 1024;
  if (threads < 32) threads = 32;
  if (add)
    rms_norm_kernel<T, QMODE, true><<<a.T, threads, 0, s>>>(a);
  else
    rms_norm_kernel<T, QMODE, false><<<a.T, threads, 0, s>>>(a);
  return static_cast<int>(cudaGetLastError());
}

template <typename T>
int launch1(const Args& a, int qmode, bool add, cudaStream_t s) {
  switch (qmode) {
    case kQNone: return launch2<T, kQNone>(a, add, s);
    case kQFp8Static: return launch2<T, kQFp8Static>(a, add, s);
    case kQFp8Token: return launch2<T, kQFp8Token>(a, add, s);
    case kQFp8Group128: return launch2<T, kQFp8Group128>(a, add, s);
    case kQInt8Static: return launch2<T, kQInt8Static>(a, add, s);
    case kQInt8Token: return launch2<T, kQInt8Token>(a, add, s);
    default: return -7;
  }
}

}  // namespace norm
}  // namespace b200

// Generic entry point of the norm family.
//   dtype: 0 bf16, 1 fp16.  qmode: see QMode.  residual != null selects the
//   fused-add variant (residual <- x + residual; out <- norm(residual)).
//   layer_norm != 0 subtracts the mean and adds `bias` (may be null).
//   H must be a multiple of 8 (128 for the group-quant mode); pitches are in
//   elements of their tensor.
B200_API int b200_norm(const void* x, long long ldx, void* residual, long long ldr,
                       const void* weight, const void* bias, void* out, long long ldo,
                       float* scale_out, const float* scale_in, const int* valid_rows, int T,
                       int H, float eps, int dtype, int qmode, int layer_norm, void* stream) {
  using namespace b200::norm;
  if (T <= 0 || H <= 0) return 0;
  if ((H % 8) != 0 || (ldx % 8) != 0 || (ldo % 8) != 0) return -2;
  if (qmode == kQFp8Group128 && (H % 128) != 0) return -2;
  Args a;
  a.x = x; a.residual = residual; a.weight = weight; a.bias = bias; a.out = out;
  a.scale_out = scale_out; a.scale_in = scale_in; a.valid_rows = valid_rows;
  a.ldx = ldx; a.ldr = ldr; a.ldo = ldo; a.T = T; a.H = H; a.eps = eps;
  a.layer_norm = layer_norm;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const bool add = residual != nullptr;
  if (dtype == 0) return launch1<__nv_bfloat16>(a, qmode, add, s);
  if (dtype == 1) return launch1<__half>(a, qmode, add, s);
  return -8;
}
