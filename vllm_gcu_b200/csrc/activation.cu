// Gated and plain activations for sm_100a, optionally fused with quantisation.
//
//   out[t, j] = act(x[t, j]) * x[t, d + j]           (act_and_mul family)
//   out[t, j] = x[t, j] * act(x[t, d + j])           (mul_and_silu)
//   out[t, j] = act(x[t, j])                         (element-wise family)
//
// Quantising epilogues: dynamic 1x128-group fp8 (scale per row and group),
// static per-tensor fp8, static symmetric int8, static asymmetric int8.  An
// optional device-side row count limits the work to the valid prefix of a
// padded buffer (MoE static buffers under CUDA graphs).
//
// Reference ops: csrc/src/silu_and_mul.cpp:44, silu_and_mul_pad.cpp:33,
// mul_and_silu.cpp, gelu_and_mul.cpp:33, gelu_tanh_and_mul.cpp:33,
// fatrelu_and_mul.cpp, gelu_new.cpp:38, gelu_fast.cpp:31, gelu_quick.cpp:20,
// silu_mul_per_token_group_quant(_with_size).cpp, silu_mul_static_fp8_quant.cpp:21,
// silu_mul_static_int8_quant.cpp:26, silu_asym_quant.cpp:17 and the gelu_* quant
// variants; Python side vllm_gcu/kernels/activation.py:16-80.
#include "common.cuh"

namespace b200 {
namespace act {

enum Act : int {
  kSilu = 0,
  kGelu = 1,
  kGeluTanh = 2,
  kFatRelu = 3,
  kGeluNew = 4,
  kGeluFast = 5,
  kGeluQuick = 6,
  kIdentity = 7,
};
enum Mode : int { kActMul = 0, kMulAct = 1, kPlain = 2 };
enum Quant : int { kQNone = 0, kQFp8Group128 = 1, kQFp8Static = 2, kQInt8Static = 3, kQInt8Asym = 4 };

template <int ACT>
__device__ __forceinline__ float apply(float x, float thr) {
  if constexpr (ACT == kSilu) return x / (1.0f + __expf(-x));
  if constexpr (ACT == kGelu) return 0.5f * x * (1.0f + erff(x * 0.70710678118654752f));
  if constexpr (ACT == kGeluTanh || ACT == kGeluNew) {
    const float k = 0.7978845608028654f;
    return 0.5f * x * (1.0f + tanhf(k * (x + 0.044715f * x * x * x)));
  }
  if constexpr (ACT == kFatRelu) return x > thr ? x : 0.0f;
  if constexpr (ACT == kGeluFast)
    return 0.5f * x * (1.0f + tanhf(x * 0.79788456f * (1.0f + 0.044715f * x * x)));
  if constexpr (ACT == kGeluQuick) return x / (1.0f + __expf(-1.702f * x));
  return x;
}

template <typename T>
__device__ __forceinline__ void ld8(const T* p, float (&f)[8]) {
  uint4 u = *reinterpret_cast<const uint4*>(p);
  if constexpr (sizeof(T) == 2 && std::is_same<T, __nv_bfloat16>::value) {
    float2 a = unpack_bf16x2(u.x), b = unpack_bf16x2(u.y), c = unpack_bf16x2(u.z),
           d = unpack_bf16x2(u.w);
    f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y; f[4] = c.x; f[5] = c.y; f[6] = d.x; f[7] = d.y;
  } else {
    const __half2* h = reinterpret_cast<const __half2*>(&u);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      float2 x = __half22float2(h[i]);
      f[2 * i] = x.x;
      f[2 * i + 1] = x.y;
    }
  }
}
template <typename T>
__device__ __forceinline__ void st8(T* p, const float (&f)[8]) {
  uint4 u;
  if constexpr (std::is_same<T, __nv_bfloat16>::value) {
    u.x = pack_bf16x2(f[0], f[1]);
    u.y = pack_bf16x2(f[2], f[3]);
    u.z = pack_bf16x2(f[4], f[5]);
    u.w = pack_bf16x2(f[6], f[7]);
  } else {
    __half2* h = reinterpret_cast<__half2*>(&u);
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __floats2half2_rn(f[2 * i], f[2 * i + 1]);
  }
  *reinterpret_cast<uint4*>(p) = u;
}
template <typename T>
__device__ __forceinline__ float rnd(float v) {
  if constexpr (std::is_same<T, __nv_bfloat16>::value)
    return __bfloat162float(__float2bfloat16(v));
  else
    return __half2float(__float2half(v));
}

struct Args {
  const void* x;
  void* out;
  float* scale_out;        // [T, d/128] for group quant
  const float* scale_in;   // scalar for static modes
  const int* azp;          // scalar zero point (asymmetric int8)
  const int* valid_rows;
  long long ldx, ldo;
  int T, d;
  float threshold;
};

template <typename T, int ACT, int MODE, int QUANT>
__global__ void __launch_bounds__(512) act_kernel(const Args a) {
  const int row = blockIdx.x;
  if (a.valid_rows != nullptr && row >= *a.valid_rows) return;
  const T* x = static_cast<const T*>(a.x) + static_cast<long long>(row) * a.ldx;
  const int nvec = a.d >> 3;
  const int nvec_pad = (QUANT == kQFp8Group128) ? ((nvec + 31) & ~31) : nvec;
  float inv_static = 1.0f;
  int zp = 0;
  if constexpr (QUANT == kQFp8Static || QUANT == kQInt8Static || QUANT == kQInt8Asym)
    inv_static = 1.0f / *a.scale_in;
  if constexpr (QUANT == kQInt8Asym) zp = *a.azp;

  for (int v = threadIdx.x; v < nvec_pad; v += blockDim.x) {
    const bool ok = v < nvec;
    float f[8];
    if (ok) {
      float g[8];
      ld8<T>(x + v * 8, g);
      if constexpr (MODE == kPlain) {
#pragma unroll
        for (int i = 0; i < 8; ++i) f[i] = rnd<T>(apply<ACT>(g[i], a.threshold));
      } else {
        float u[8];
        ld8<T>(x + a.d + v * 8, u);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          if constexpr (MODE == kActMul)
            f[i] = rnd<T>(apply<ACT>(g[i], a.threshold) * u[i]);
          else
            f[i] = rnd<T>(g[i] * apply<ACT>(u[i], a.threshold));
        }
      }
    }
    if constexpr (QUANT == kQNone) {
      if (ok) st8<T>(static_cast<T*>(a.out) + static_cast<long long>(row) * a.ldo + v * 8, f);
    } else if constexpr (QUANT == kQFp8Group128) {
      float amax = 0.0f;
      if (ok) {
#pragma unroll
        for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(f[i]));
      }
#pragma unroll
      for (int o = 8; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
      const float s = fmaxf(amax, 1e-10f) / 448.0f;
      if (ok) {
        const float inv = 1.0f / s;
        uint2 pk;
        uint8_t* b = reinterpret_cast<uint8_t*>(&pk);
#pragma unroll
        for (int i = 0; i < 8; ++i)
          b[i] = static_cast<uint8_t>(__nv_cvt_float_to_fp8(f[i] * inv, __NV_SATFINITE, __NV_E4M3));
        *reinterpret_cast<uint2*>(static_cast<uint8_t*>(a.out) +
                                  static_cast<long long>(row) * a.ldo + v * 8) = pk;
        if ((v & 15) == 0) a.scale_out[static_cast<long long>(row) * (a.d >> 7) + (v >> 4)] = s;
      }
    } else {
      if (ok) {
        uint2 pk;
        uint8_t* b = reinterpret_cast<uint8_t*>(&pk);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          if constexpr (QUANT == kQFp8Static) {
            b[i] = static_cast<uint8_t>(
                __nv_cvt_float_to_fp8(f[i] * inv_static, __NV_SATFINITE, __NV_E4M3));
          } else {
            float r = rintf(f[i] * inv_static) + static_cast<float>(zp);
            r = fminf(fmaxf(r, -128.0f), 127.0f);
            b[i] = static_cast<uint8_t>(static_cast<int8_t>(r));
          }
        }
        *reinterpret_cast<uint2*>(static_cast<uint8_t*>(a.out) +
                                  static_cast<long long>(row) * a.ldo + v * 8) = pk;
      }
    }
  }
}

template <typename T, int ACT, int MODE>
int launch_q(const Args& a, int quant, cudaStream_t s) {
  int threads = ((a.d >> 3) + 31) & ~31;
  threads = threads > 512 ? 512 : (threads < 32 ? 32 : threads);
  switch (quant) {
    case kQNone: act_kernel<T, ACT, MODE, kQNone><<<a.T, threads, 0, s>>>(a); break;
    case kQFp8Group128: act_kernel<T, ACT, MODE, kQFp8Group128><<<a.T, threads, 0, s>>>(a); break;
    case kQFp8Static: act_kernel<T, ACT, MODE, kQFp8Static><<<a.T, threads, 0, s>>>(a); break;
    case kQInt8Static: act_kernel<T, ACT, MODE, kQInt8Static><<<a.T, threads, 0, s>>>(a); break;
    case kQInt8Asym: act_kernel<T, ACT, MODE, kQInt8Asym><<<a.T, threads, 0, s>>>(a); break;
    default: return -7;
  }
  return static_cast<int>(cudaGetLastError());
}

template <typename T>
int launch_t(const Args& a, int act, int mode, int quant, cudaStream_t s) {
#define B200_ACT_CASE(A)                                              \
  case A:                                                             \
    if (mode == kActMul) return launch_q<T, A, kActMul>(a, quant, s); \
    if (mode == kPlain) return launch_q<T, A, kPlain>(a, quant, s);   \
    break;
  switch (act) {
    case kSilu:
      if (mode == kActMul) return launch_q<T, kSilu, kActMul>(a, quant, s);
      if (mode == kMulAct) return launch_q<T, kSilu, kMulAct>(a, quant, s);
      if (mode == kPlain) return launch_q<T, kSilu, kPlain>(a, quant, s);
      break;
    B200_ACT_CASE(kGelu)
    B200_ACT_CASE(kGeluTanh)
    B200_ACT_CASE(kFatRelu)
    B200_ACT_CASE(kGeluNew)
    B200_ACT_CASE(kGeluFast)
    B200_ACT_CASE(kGeluQuick)
    case kIdentity:
      if (mode == kActMul) return launch_q<T, kIdentity, kActMul>(a, quant, s);
      if (mode == kPlain) return launch_q<T, kIdentity, kPlain>(a, quant, s);  // pure quantisation
      break;
    default:
      break;
  }
#undef B200_ACT_CASE
  return -7;
}

}  // namespace act
}  // namespace b200

// x is [T, 2d] for the gated modes and [T, d] for mode 2; out is [T, d].
// dtype 0 bf16 / 1 fp16.  d must be a multiple of 8 (128 for group quant).
B200_API int b200_activation(const void* x, long long ldx, void* out, long long ldo,
                             float* scale_out, const float* scale_in, const int* azp,
                             const int* valid_rows, int T, int d, int act, int mode, int quant,
                             float threshold, int dtype, void* stream) {
  using namespace b200::act;
  if (T <= 0 || d <= 0) return 0;
  if ((d % 8) != 0 || (ldx % 8) != 0 || (ldo % 8) != 0) return -2;
  if (quant == kQFp8Group128 && (d % 128) != 0) return -2;
  Args a;
  a.x = x; a.out = out; a.scale_out = scale_out; a.scale_in = scale_in; a.azp = azp;
  a.valid_rows = valid_rows; a.ldx = ldx; a.ldo = ldo; a.T = T; a.d = d; a.threshold = threshold;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (dtype == 0) return launch_t<__nv_bfloat16>(a, act, mode, quant, s);
  if (dtype == 1) return launch_t<__half>(a, act, mode, quant, s);
  return -8;
}
