// Multi-LoRA batched gather matrix-vector product for sm_100a:
//
//   y[t, y_off : y_off + h_out] += scale * W[idx[t]] (h_out x h_in) . x[t]      (idx[t] < 0: skip)
//
// One CTA per token.  "Shrink" shapes (long h_in, short h_out = rank): one warp per output
// row, 16-byte loads along h_in, warp reduction.  "Expand" shapes (h_in = rank <= 256): one
// thread per output row with the input vector staged in shared memory.  Prefill-sized
// batches go through the grouped tcgen05 GEMM instead (adapters play the role of experts),
// see vllm_gcu_b200/lora/ops.py.
//
// Reference: csrc/src/dispatch_bgmv.cpp:19, dispatch_bgmv_low_level.cpp:21,
// vllm_gcu/lora/lora_ops.py:10-139.
#include "common.cuh"

namespace b200 {
namespace lora {

template <typename T, typename TY>
__global__ void __launch_bounds__(256)
    bgmv_kernel(TY* y, long long ldy, const T* x, long long ldx, const T* w, const int* idx,
                int h_in, int h_out, int y_off, float scale, int add) {
  extern __shared__ float sx[];
  const int t = blockIdx.x;
  const int l = idx[t];
  if (l < 0) return;
  const T* xr = x + static_cast<long long>(t) * ldx;
  const T* wl = w + static_cast<long long>(l) * h_out * h_in;
  TY* yr = y + static_cast<long long>(t) * ldy + y_off;
  if (h_in <= 256) {
    for (int i = threadIdx.x; i < h_in; i += blockDim.x) sx[i] = to_f32<T>(xr[i]);
    __syncthreads();
    for (int o = threadIdx.x; o < h_out; o += blockDim.x) {
      const T* wr = wl + static_cast<long long>(o) * h_in;
      float acc = 0.0f;
      for (int i = 0; i < h_in; ++i) acc += to_f32<T>(wr[i]) * sx[i];
      const float prev = add ? to_f32<TY>(yr[o]) : 0.0f;
      yr[o] = from_f32<TY>(prev + acc * scale);
    }
  } else {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
    const int nvec = h_in >> 3;
    for (int o = warp; o < h_out; o += nw) {
      const T* wr = wl + static_cast<long long>(o) * h_in;
      float acc = 0.0f;
      for (int v = lane; v < nvec; v += 32) {
        float a[8], b[8];
        vec8_load<T>(wr + v * 8, a);
        vec8_load<T>(xr + v * 8, b);
#pragma unroll
        for (int i = 0; i < 8; ++i) acc += a[i] * b[i];
      }
      acc = warp_sum(acc);
      if (lane == 0) {
        const float prev = add ? to_f32<TY>(yr[o]) : 0.0f;
        yr[o] = from_f32<TY>(prev + acc * scale);
      }
    }
  }
}

}  // namespace lora
}  // namespace b200

// dtype: element type of x and w (0 bf16, 1 fp16); ydtype: element type of y (0, 1 or 2 = fp32,
// the shrink output is kept in fp32).  h_in % 8 == 0 when h_in > 256.
B200_API int b200_bgmv(void* y, long long ldy, const void* x, long long ldx, const void* w,
                       const int* idx, int T, int h_in, int h_out, int y_off, float scale, int add,
                       int dtype, int ydtype, void* stream) {
  using namespace b200::lora;
  if (T <= 0 || h_out <= 0) return 0;
  if (h_in > 256 && (h_in % 8) != 0) return -2;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const size_t smem = h_in <= 256 ? static_cast<size_t>(h_in) * sizeof(float) : 0;
#define B200_BGMV(TT, TY) \
  bgmv_kernel<TT, TY><<<T, 256, smem, s>>>(static_cast<TY*>(y), ldy, static_cast<const TT*>(x), ldx, static_cast<const TT*>(w), idx, h_in, h_out, y_off, scale, add)
  if (dtype == 0 && ydtype == 0) B200_BGMV(__nv_bfloat16, __nv_bfloat16);
  else if (dtype == 0 && ydtype == 2) B200_BGMV(__nv_bfloat16, float);
  else if (dtype == 1 && ydtype == 1) B200_BGMV(__half, __half);
  else if (dtype == 1 && ydtype == 2) B200_BGMV(__half, float);
  else return -8;
#undef B200_BGMV
  return static_cast<int>(cudaGetLastError());
}
