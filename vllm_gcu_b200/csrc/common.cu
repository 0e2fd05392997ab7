// Host-side helpers shared by all kernel families: tensor-map encoding through
// the driver entry point (no link-time dependency on libcuda), the status word
// and device queries.
#include "common.cuh"

#include <mutex>

namespace b200 {

// [0..3] first error (code, kernel, detail, count); [4] run-time flag-wait budget (0: default)
__device__ unsigned int g_status[8] = {0u, 0u, 0u, 0u, 0u, 0u, 0u, 0u};

unsigned int* status_ptr() {
  static unsigned int* cached[64] = {nullptr};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  if (cached[dev] == nullptr) {
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_status) != cudaSuccess) return nullptr;
    cached[dev] = static_cast<unsigned int*>(p);
  }
  return cached[dev];
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, []() {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) ==
            cudaSuccess &&
        q == cudaDriverEntryPointSuccess) {
      fn = reinterpret_cast<EncodeTiledFn>(p);
    }
  });
  return fn;
}

int encode_tmap_2d(CUtensorMap* out, CUtensorMapDataType dt, int elt_bytes, const void* base,
                   uint64_t rows, uint64_t cols, uint64_t ld_bytes, uint32_t box_rows,
                   uint32_t box_cols, CUtensorMapSwizzle swz) {
  EncodeTiledFn fn = get_encode_fn();
  if (fn == nullptr) return -1;
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {ld_bytes};
  cuuint32_t box[2] = {box_cols, box_rows};
  cuuint32_t estr[2] = {1, 1};
  (void)elt_bytes;
  CUresult r = fn(out, dt, 2, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, swz, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : static_cast<int>(r);
}

int encode_tmap_3d(CUtensorMap* out, CUtensorMapDataType dt, int elt_bytes, const void* base,
                   uint64_t d2, uint64_t d1, uint64_t d0, uint64_t stride2_bytes,
                   uint64_t stride1_bytes, uint32_t box2, uint32_t box1, uint32_t box0,
                   CUtensorMapSwizzle swz) {
  EncodeTiledFn fn = get_encode_fn();
  if (fn == nullptr) return -1;
  cuuint64_t dims[3] = {d0, d1, d2};
  cuuint64_t strides[2] = {stride1_bytes, stride2_bytes};
  cuuint32_t box[3] = {box0, box1, box2};
  cuuint32_t estr[3] = {1, 1, 1};
  (void)elt_bytes;
  CUresult r = fn(out, dt, 3, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, swz, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : static_cast<int>(r);
}

int sm_count() {
  static int cached[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  if (cached[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0)
      n = 148;
    cached[dev] = n;
  }
  return cached[dev];
}

}  // namespace b200

// Reads the status word of the current device into out[4] and clears it.
// Synchronises the given stream first.  Returns the CUDA error code.
B200_API int b200_status_take(unsigned int* out, void* stream) {
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  cudaError_t e = cudaStreamSynchronize(s);
  if (e != cudaSuccess) return static_cast<int>(e);
  e = cudaMemcpyFromSymbol(out, b200::g_status, sizeof(unsigned int) * 4);
  if (e != cudaSuccess) return static_cast<int>(e);
  unsigned int zero[4] = {0u, 0u, 0u, 0u};
  e = cudaMemcpyToSymbol(b200::g_status, zero, sizeof(zero));
  return static_cast<int>(e);
}

// Sets the iteration budget of every wait on a peer- or host-written flag on the current
// device (0 restores the built-in default of about a second).  Takes effect for kernels
// launched after the call on the same stream order as a synchronous copy.
B200_API int b200_set_flag_wait_limit(unsigned int iterations) {
  return static_cast<int>(
      cudaMemcpyToSymbol(b200::g_status, &iterations, sizeof(unsigned int), 4 * sizeof(unsigned int)));
}

B200_API int b200_sm_count() { return b200::sm_count(); }

B200_API int b200_abi_version() { return 1; }
