// Stand-alone quantisation kernels for sm_100a.
//
//   dynamic per-token quantisation to fp8 e4m3 / int8 (row scale = amax / 448 or / 127)
//   dynamic per-tensor fp8 quantisation (two kernels: amax reduction, then quantise)
//   static int8 de-quantisation (symmetric and with zero point)
//   weight-only de-quantisation: 4-bit / 8-bit group-quantised weights in this library's
//   K-major packed layout -> bf16 [N, K] (A operand B of the tcgen05 GEMM)
//
// Static and 1x128-group quantisation of activations is handled by activation.cu
// (identity activation, plain mode) and norm.cu (fused with the norm).
//
// Reference ops: csrc/src/dynamic_per_token_scaled_fp8_quant.cpp:33,
// dynamic_scaled_fp8_quant.cpp, dynamic_scaled_int8_quant.cpp:17,
// static_scaled_int8_dequant.cpp:18, static_scaled_int8_asym_dequant.cpp:20,
// awq_gemm_gcu.cpp:43 / gptq_gemm_gcu.cpp:44 / weight_only_quant.cpp:35 (weight formats,
// rearranged at load time as in vllm_gcu/kernels/quantization/rearrange.py:6-133).
#include "common.cuh"

namespace b200 {
namespace quant {

template <typename T, bool INT8>
__global__ void __launch_bounds__(1024)
    per_token_quant_kernel(const T* x, long long ldx, uint8_t* out, long long ldo, float* scales,
                           const int* valid_rows, int H) {
  __shared__ float red[32];
  const int row = blockIdx.x;
  if (valid_rows != nullptr && row >= *valid_rows) return;
  const T* xr = x + static_cast<long long>(row) * ldx;
  const int nvec = H >> 3;
  float amax = 0.0f;
  for (int v = threadIdx.x; v < nvec; v += blockDim.x) {
    float f[8];
    vec8_load<T>(xr + v * 8, f);
#pragma unroll
    for (int i = 0; i < 8; ++i) amax = fmaxf(amax, fabsf(f[i]));
  }
  amax = block_max(amax, red);
  const float s = fmaxf(amax, 1e-10f) / (INT8 ? 127.0f : 448.0f);
  if (threadIdx.x == 0) scales[row] = s;
  const float inv = 1.0f / s;
  for (int v = threadIdx.x; v < nvec; v += blockDim.x) {
    float f[8];
    vec8_load<T>(xr + v * 8, f);
    uint2 pk;
    uint8_t* b = reinterpret_cast<uint8_t*>(&pk);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      if constexpr (INT8) {
        const float r = fminf(fmaxf(rintf(f[i] * inv), -128.0f), 127.0f);
        b[i] = static_cast<uint8_t>(static_cast<int8_t>(r));
      } else {
        b[i] = f32_to_e4m3(f[i] * inv);
      }
    }
    *reinterpret_cast<uint2*>(out + static_cast<long long>(row) * ldo + v * 8) = pk;
  }
}

template <typename T>
__global__ void __launch_bounds__(1024)
    tensor_amax_kernel(const T* x, long long n, float* amax_out) {
  __shared__ float red[32];
  float amax = 0.0f;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x)
    amax = fmaxf(amax, fabsf(to_f32<T>(x[i])));
  amax = block_max(amax, red);
  if (threadIdx.x == 0) atomicMax(reinterpret_cast<int*>(amax_out), __float_as_int(amax));
}

template <typename T>
__global__ void tensor_quant_kernel(const T* x, uint8_t* out, long long n, const float* amax,
                                    float* scale_out) {
  const float s = fmaxf(*amax, 1e-10f) / 448.0f;
  if (blockIdx.x == 0 && threadIdx.x == 0) *scale_out = s;
  const float inv = 1.0f / s;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x)
    out[i] = f32_to_e4m3(to_f32<T>(x[i]) * inv);
}

template <typename T>
__global__ void int8_dequant_kernel(const int8_t* q, T* out, long long n, const float* scale,
                                    const int* azp) {
  const float s = *scale;
  const float z = azp ? static_cast<float>(*azp) : 0.0f;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < n;
       i += static_cast<long long>(gridDim.x) * blockDim.x)
    out[i] = from_f32<T>((static_cast<float>(q[i]) - z) * s);
}

// Weight-only de-quantisation.  Packed layout (built at load time):
//   qw      uint8 [N, K/2] for 4 bit (low nibble = even k) or [N, K] for 8 bit
//   scales  T [N, K/g],  zs  T [N, K/g] = zero_point * scale
//   w[n, k] = q * scale - zs
template <typename T, int BITS>
__global__ void __launch_bounds__(256)
    weight_dequant_kernel(const uint8_t* qw, const T* scales, const T* zs, T* out, int N, int K,
                          int g) {
  const long long idx = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  const int kv = K >> 3;  // 8 outputs per thread
  if (idx >= static_cast<long long>(N) * kv) return;
  const int n = static_cast<int>(idx / kv), k0 = static_cast<int>(idx % kv) * 8;
  const int grp = k0 / g;
  const float s = to_f32<T>(scales[static_cast<long long>(n) * (K / g) + grp]);
  const float z = to_f32<T>(zs[static_cast<long long>(n) * (K / g) + grp]);
  float f[8];
  if constexpr (BITS == 4) {
    const uint32_t p = *reinterpret_cast<const uint32_t*>(qw + static_cast<long long>(n) * (K / 2) + k0 / 2);
#pragma unroll
    for (int i = 0; i < 8; ++i) f[i] = static_cast<float>((p >> (4 * i)) & 0xFu) * s - z;
  } else {
    const uint2 p = *reinterpret_cast<const uint2*>(qw + static_cast<long long>(n) * K + k0);
    const uint8_t* b = reinterpret_cast<const uint8_t*>(&p);
#pragma unroll
    for (int i = 0; i < 8; ++i) f[i] = static_cast<float>(b[i]) * s - z;
  }
  vec8_store<T>(out + static_cast<long long>(n) * K + k0, f);
}

}  // namespace quant
}  // namespace b200

using namespace b200;
using namespace b200::quant;

// kind 0: fp8 e4m3, 1: int8.  dtype 0 bf16 / 1 fp16.  H % 8 == 0.
B200_API int b200_per_token_quant(const void* x, long long ldx, void* out, long long ldo,
                                  float* scales, const int* valid_rows, int T, int H, int kind,
                                  int dtype, void* stream) {
  if (T <= 0) return 0;
  if ((H % 8) != 0 || (ldx % 8) != 0 || (ldo % 8) != 0) return -2;
  int threads = ((H >> 3) + 31) & ~31;
  threads = threads > 1024 ? 1024 : (threads < 32 ? 32 : threads);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  uint8_t* o = static_cast<uint8_t*>(out);
#define B200_PTQ(TT, I8) \
  per_token_quant_kernel<TT, I8><<<T, threads, 0, s>>>(static_cast<const TT*>(x), ldx, o, ldo, scales, valid_rows, H)
  if (dtype == 0 && kind == 0) B200_PTQ(__nv_bfloat16, false);
  else if (dtype == 0 && kind == 1) B200_PTQ(__nv_bfloat16, true);
  else if (dtype == 1 && kind == 0) B200_PTQ(__half, false);
  else if (dtype == 1 && kind == 1) B200_PTQ(__half, true);
  else return -8;
#undef B200_PTQ
  return static_cast<int>(cudaGetLastError());
}

// Dynamic per-tensor fp8: scale_out[0] = amax / 448.  `amax_ws` is one float of workspace.
B200_API int b200_per_tensor_fp8_quant(const void* x, void* out, long long n, float* amax_ws,
                                       float* scale_out, int dtype, void* stream) {
  if (n <= 0) return 0;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  cudaError_t e = cudaMemsetAsync(amax_ws, 0, sizeof(float), s);
  if (e != cudaSuccess) return static_cast<int>(e);
  const int blocks = static_cast<int>(n / 4096 + 1 > 592 ? 592 : n / 4096 + 1);
  if (dtype == 0) {
    tensor_amax_kernel<__nv_bfloat16><<<blocks, 1024, 0, s>>>(static_cast<const __nv_bfloat16*>(x), n, amax_ws);
    tensor_quant_kernel<__nv_bfloat16><<<blocks, 1024, 0, s>>>(static_cast<const __nv_bfloat16*>(x), static_cast<uint8_t*>(out), n, amax_ws, scale_out);
  } else if (dtype == 1) {
    tensor_amax_kernel<__half><<<blocks, 1024, 0, s>>>(static_cast<const __half*>(x), n, amax_ws);
    tensor_quant_kernel<__half><<<blocks, 1024, 0, s>>>(static_cast<const __half*>(x), static_cast<uint8_t*>(out), n, amax_ws, scale_out);
  } else {
    return -8;
  }
  return static_cast<int>(cudaGetLastError());
}

B200_API int b200_int8_dequant(const void* q, void* out, long long n, const float* scale,
                               const int* azp, int dtype, void* stream) {
  if (n <= 0) return 0;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const int blocks = static_cast<int>(n / 1024 + 1 > 1184 ? 1184 : n / 1024 + 1);
  if (dtype == 0)
    int8_dequant_kernel<__nv_bfloat16><<<blocks, 256, 0, s>>>(static_cast<const int8_t*>(q), static_cast<__nv_bfloat16*>(out), n, scale, azp);
  else if (dtype == 1)
    int8_dequant_kernel<__half><<<blocks, 256, 0, s>>>(static_cast<const int8_t*>(q), static_cast<__half*>(out), n, scale, azp);
  else if (dtype == 2)
    int8_dequant_kernel<float><<<blocks, 256, 0, s>>>(static_cast<const int8_t*>(q), static_cast<float*>(out), n, scale, azp);
  else
    return -8;
  return static_cast<int>(cudaGetLastError());
}

// bits 4 or 8; K % 8 == 0, g divides K and g % 8 == 0.
B200_API int b200_weight_dequant(const void* qw, const void* scales, const void* zs, void* out,
                                 int N, int K, int g, int bits, int dtype, void* stream) {
  if (N <= 0 || K <= 0) return 0;
  if ((K % 8) != 0 || g <= 0 || (g % 8) != 0 || (K % g) != 0) return -2;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const long long work = static_cast<long long>(N) * (K / 8);
  const int blocks = static_cast<int>((work + 255) / 256);
  const uint8_t* q = static_cast<const uint8_t*>(qw);
#define B200_WDQ(TT, BB) \
  weight_dequant_kernel<TT, BB><<<blocks, 256, 0, s>>>(q, static_cast<const TT*>(scales), static_cast<const TT*>(zs), static_cast<TT*>(out), N, K, g)
  if (dtype == 0 && bits == 4) B200_WDQ(__nv_bfloat16, 4);
  else if (dtype == 0 && bits == 8) B200_WDQ(__nv_bfloat16, 8);
  else if (dtype == 1 && bits == 4) B200_WDQ(__half, 4);
  else if (dtype == 1 && bits == 8) B200_WDQ(__half, 8);
  else return -8;
#undef B200_WDQ
  return static_cast<int>(cudaGetLastError());
}
