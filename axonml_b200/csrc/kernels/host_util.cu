// Host helpers shared by the kernel launchers: tensor-map encoding through the driver entry
// point, SM count, a library version probe.
#include <cudaTypedefs.h>
#include <mutex>

#include "common.cuh"

namespace axh {

static PFN_cuTensorMapEncodeTiled_v12000 g_encode = nullptr;
static std::once_flag g_encode_once;

static void resolve_encode() {
  void* fn = nullptr;
  cudaDriverEntryPointQueryResult qres;
  cudaError_t e = cudaGetDriverEntryPointByVersion("cuTensorMapEncodeTiled", &fn, 12000,
                                                   cudaEnableDefault, &qres);
  if (e == cudaSuccess && qres == cudaDriverEntryPointSuccess)
    g_encode = (PFN_cuTensorMapEncodeTiled_v12000)fn;
}

int encode_tensor_map(CUtensorMap* map, CUtensorMapDataType dtype, int rank, const void* base,
                      const uint64_t* dims, const uint64_t* strides_bytes, const uint32_t* box,
                      CUtensorMapSwizzle swizzle) {
  std::call_once(g_encode_once, resolve_encode);
  if (!g_encode) return 999;
  cuuint64_t gdims[5];
  cuuint64_t gstrides[4];
  cuuint32_t gbox[5];
  cuuint32_t estr[5];
  for (int i = 0; i < rank; ++i) {
    gdims[i] = dims[i];
    gbox[i] = box[i];
    estr[i] = 1;
  }
  for (int i = 0; i + 1 < rank; ++i) gstrides[i] = strides_bytes[i];
  CUresult r = g_encode(map, dtype, (cuuint32_t)rank, const_cast<void*>(base), gdims, gstrides,
                        gbox, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle,
                        CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return (int)r;
}

int sm_count() {
  static int cached[64] = {0};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) dev = 0;
  if (cached[dev] == 0) {
    int n = 0;
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    cached[dev] = n > 0 ? n : 1;
  }
  return cached[dev];
}

}  // namespace axh

AX_API int ax_version() { return 1; }
AX_API int ax_sm_count() { return axh::sm_count(); }

// ---------------------------------------------------------------- bounds-checked debug build
#ifdef AX_BOUNDS
namespace ax { __device__ int g_bounds_word[6] = {0, 0, 0, 0, 0, 0}; }
namespace {
// Walks one element past an n-element extent on purpose, through the checked accessor: in this
// build the access is skipped and reported, which is what the self-test looks for.
__global__ void bounds_selftest_kernel(float* p, long n) {
  const long i = (long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i <= n && AX_INB(i, 1, n, 9000)) p[i] += 1.f;
}
}  // namespace
#endif

// 1 when this library was compiled with the index checks.
AX_API int ax_bounds_enabled() {
#ifdef AX_BOUNDS
  return 1;
#else
  return 0;
#endif
}

// Copies the first recorded violation {code, where, index lo, index hi, extent lo, extent hi} into
// out[6] (all zero: none) and clears it.  Synchronises the device.
AX_API int ax_bounds_read(int* out) {
  for (int i = 0; i < 6; ++i) out[i] = 0;
#ifdef AX_BOUNDS
  cudaError_t e = cudaDeviceSynchronize();
  if (e != cudaSuccess) return (int)e;
  e = cudaMemcpyFromSymbol(out, ax::g_bounds_word, sizeof(int) * 6);
  if (e != cudaSuccess) return (int)e;
  const int zero[6] = {0, 0, 0, 0, 0, 0};
  e = cudaMemcpyToSymbol(ax::g_bounds_word, zero, sizeof(zero));
  return (int)e;
#else
  return 0;
#endif
}

// Debug build only: increments p[0..n) through the checked accessor with one thread too many.
AX_API int ax_bounds_selftest(float* p, long n, cudaStream_t stream) {
#ifdef AX_BOUNDS
  bounds_selftest_kernel<<<(unsigned)((n + 1 + 255) / 256), 256, 0, stream>>>(p, n);
  return (int)cudaGetLastError();
#else
  (void)p; (void)n; (void)stream;
  return -1;
#endif
}
