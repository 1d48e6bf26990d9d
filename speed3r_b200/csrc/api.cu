// Host-side plumbing shared by every entry point: error messages, the per-device status word,
// tensor-map (TMA descriptor) creation through the driver entry point.
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <mutex>

#include "common.cuh"

namespace s3r {

static thread_local char g_err[512] = "";

int set_error(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
  return code;
}

int check_cuda(cudaError_t e, const char* what) {
  if (e == cudaSuccess) return 0;
  set_error(static_cast<int>(e), "%s: %s", what, cudaGetErrorString(e));
  return static_cast<int>(e);
}

__device__ uint32_t g_status_word = 0;

uint32_t* device_status_ptr() {
  // The address of a __device__ variable differs per device; cache one per device ordinal.
  static uint32_t* cache[64] = {};
  static std::mutex mu;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  std::lock_guard<std::mutex> lock(mu);
  if (!cache[dev]) {
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, g_status_word) != cudaSuccess) return nullptr;
    cache[dev] = static_cast<uint32_t*>(p);
  }
  return cache[dev];
}

int sm_count() {
  static int cache[64] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  if (!cache[dev]) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    cache[dev] = n;
  }
  return cache[dev];
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  });
  return fn;
}

int make_tensor_map(CUtensorMap* out, const void* base, int rank, const uint64_t* dims,
                    const uint64_t* strides_bytes, const uint32_t* box, CUtensorMapSwizzle swizzle,
                    CUtensorMapDataType dtype) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return set_error(S3R_ERR_DRIVER, "cuTensorMapEncodeTiled entry point not available");
  cuuint64_t gdim[5];
  cuuint64_t gstr[4];
  cuuint32_t bx[5], es[5];
  for (int i = 0; i < rank; ++i) {
    gdim[i] = dims[i];
    bx[i] = box[i];
    es[i] = 1;
    if (i > 0) gstr[i - 1] = strides_bytes[i - 1];
  }
  CUresult r = fn(out, dtype, static_cast<cuuint32_t>(rank), const_cast<void*>(base), gdim, gstr, bx, es,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS)
    return set_error(S3R_ERR_DRIVER, "cuTensorMapEncodeTiled failed with CUresult %d (rank %d, dims %llu/%llu)",
                     static_cast<int>(r), rank, (unsigned long long)dims[0], (unsigned long long)(rank > 1 ? dims[1] : 0));
  return 0;
}

}  // namespace s3r

extern "C" {

int s3r_version(void) { return 100; }

int s3r_last_error(char* buf, int n) {
  if (!buf || n <= 0) return static_cast<int>(strlen(s3r::g_err));
  strncpy(buf, s3r::g_err, static_cast<size_t>(n) - 1);
  buf[n - 1] = 0;
  return static_cast<int>(strlen(buf));
}

int s3r_device_status(uint32_t* status_host, int clear) {
  S3R_REQUIRE(status_host != nullptr, S3R_ERR_NULL, "status_host is NULL");
  uint32_t* p = s3r::device_status_ptr();
  S3R_REQUIRE(p != nullptr, S3R_ERR_DRIVER, "could not resolve the device status word");
  S3R_CUDA(cudaDeviceSynchronize());
  S3R_CUDA(cudaMemcpy(status_host, p, sizeof(uint32_t), cudaMemcpyDeviceToHost));
  if (clear) S3R_CUDA(cudaMemset(p, 0, sizeof(uint32_t)));
  return 0;
}

int s3r_copy2d_async(void* dst, size_t dst_pitch, const void* src, size_t src_pitch, size_t width_bytes,
                     size_t rows, void* stream) {
  S3R_REQUIRE(dst && src, S3R_ERR_NULL, "s3r_copy2d_async: NULL pointer");
  S3R_REQUIRE(width_bytes > 0 && rows > 0 && dst_pitch >= width_bytes && src_pitch >= width_bytes, S3R_ERR_SHAPE,
              "s3r_copy2d_async: need 0 < width <= both pitches and rows > 0");
  S3R_CUDA(cudaMemcpy2DAsync(dst, dst_pitch, src, src_pitch, width_bytes, rows, cudaMemcpyDefault,
                             static_cast<cudaStream_t>(stream)));
  return 0;
}

}  // extern "C"
