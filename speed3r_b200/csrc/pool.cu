// Block pooling of q/k/v (the compression step) and its backward.  Both are pure streaming
// kernels bounded by HBM bandwidth: every thread moves 16-byte vectors (8 bf16 channels), a
// token row of one head is 128 contiguous bytes, and neighbouring threads walk neighbouring heads so
// that the packed qkv projection is read in 2 KB contiguous runs.
#include "common.cuh"

namespace s3r {

struct alignas(16) Bf16x8 {
  uint32_t w[4];
};

__global__ void __launch_bounds__(256)
pool_fwd_kernel(const __nv_bfloat16* __restrict__ in, int64_t sb, int64_t sh, int64_t st,
                __nv_bfloat16* __restrict__ out, int B, int H, int T, int d, int Nc, int kernel, int stride) {
  const int vec_per_row = d >> 3;
  const int64_t total = static_cast<int64_t>(B) * Nc * H * vec_per_row;
  const float inv = 1.0f / static_cast<float>(kernel);
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    // fastest -> slowest: channel vector, head, pooled row, batch
    int c8 = static_cast<int>(i % vec_per_row);
    int64_t r = i / vec_per_row;
    int h = static_cast<int>(r % H);
    r /= H;
    int j = static_cast<int>(r % Nc);
    int b = static_cast<int>(r / Nc);
    const __nv_bfloat16* src = in + b * sb + h * sh + static_cast<int64_t>(j) * stride * st + c8 * 8;
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int t = 0; t < kernel; ++t) {
      Bf16x8 v = *reinterpret_cast<const Bf16x8*>(src + t * st);
#pragma unroll
      for (int w = 0; w < 4; ++w) {
        acc[2 * w] += bf16_lo(v.w[w]);
        acc[2 * w + 1] += bf16_hi(v.w[w]);
      }
    }
    Bf16x8 o;
#pragma unroll
    for (int w = 0; w < 4; ++w) o.w[w] = pack_bf16(acc[2 * w] * inv, acc[2 * w + 1] * inv);
    __nv_bfloat16* dst = out + ((static_cast<int64_t>(b) * H + h) * Nc + j) * d + c8 * 8;
    *reinterpret_cast<Bf16x8*>(dst) = o;
  }
}

__global__ void __launch_bounds__(256)
pool_bwd_kernel(const __nv_bfloat16* __restrict__ d_out, __nv_bfloat16* __restrict__ d_in, int64_t sb, int64_t sh,
                int64_t st, int B, int H, int T, int d, int Nc, int kernel, int stride, int accumulate) {
  const int vec_per_row = d >> 3;
  const int64_t total = static_cast<int64_t>(B) * T * H * vec_per_row;
  const float inv = 1.0f / static_cast<float>(kernel);
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    int c8 = static_cast<int>(i % vec_per_row);
    int64_t r = i / vec_per_row;
    int h = static_cast<int>(r % H);
    r /= H;
    int t = static_cast<int>(r % T);
    int b = static_cast<int>(r / T);
    // windows j with j*stride <= t < j*stride + kernel
    int j_hi = min(Nc - 1, t / stride);
    int j_lo = (t - kernel + 1 <= 0) ? 0 : (t - kernel + stride) / stride;   // ceil((t-kernel+1)/stride)
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    const __nv_bfloat16* src = d_out + (static_cast<int64_t>(b) * H + h) * Nc * d + c8 * 8;
    for (int j = j_lo; j <= j_hi; ++j) {
      Bf16x8 v = *reinterpret_cast<const Bf16x8*>(src + static_cast<int64_t>(j) * d);
#pragma unroll
      for (int w = 0; w < 4; ++w) {
        acc[2 * w] += bf16_lo(v.w[w]);
        acc[2 * w + 1] += bf16_hi(v.w[w]);
      }
    }
    __nv_bfloat16* dst = d_in + b * sb + h * sh + t * st + c8 * 8;
    Bf16x8 o;
    if (accumulate) {
      Bf16x8 old = *reinterpret_cast<const Bf16x8*>(dst);
#pragma unroll
      for (int w = 0; w < 4; ++w)
        o.w[w] = pack_bf16(bf16_lo(old.w[w]) + acc[2 * w] * inv, bf16_hi(old.w[w]) + acc[2 * w + 1] * inv);
    } else {
#pragma unroll
      for (int w = 0; w < 4; ++w) o.w[w] = pack_bf16(acc[2 * w] * inv, acc[2 * w + 1] * inv);
    }
    *reinterpret_cast<Bf16x8*>(dst) = o;
  }
}

static int pool_grid(int64_t total_threads) {
  int64_t blocks = (total_threads + 255) / 256;
  int64_t cap = static_cast<int64_t>(sm_count()) * 16;   // 16 resident CTAs of 256 threads fill an SM's 2048 threads... x2 waves
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  return static_cast<int>(blocks);
}

}  // namespace s3r

using namespace s3r;

extern "C" int s3r_pool_fwd(const void* in, int64_t stride_b, int64_t stride_h, int64_t stride_t, void* out, int B,
                            int H, int T, int d, int kernel, int stride, void* stream) {
  S3R_REQUIRE(in && out, S3R_ERR_NULL, "s3r_pool_fwd: NULL pointer");
  S3R_REQUIRE(B > 0 && H > 0 && T > 0 && d > 0 && kernel > 0 && stride > 0, S3R_ERR_SHAPE,
              "s3r_pool_fwd: sizes must be positive (B=%d H=%d T=%d d=%d kernel=%d stride=%d)", B, H, T, d, kernel, stride);
  S3R_REQUIRE(d % 8 == 0, S3R_ERR_UNSUPPORTED, "s3r_pool_fwd: head_dim %d is not a multiple of 8", d);
  S3R_REQUIRE(T >= kernel, S3R_ERR_SHAPE, "s3r_pool_fwd: T=%d shorter than the pooling kernel %d", T, kernel);
  S3R_REQUIRE((reinterpret_cast<uintptr_t>(in) & 15) == 0 && (reinterpret_cast<uintptr_t>(out) & 15) == 0 &&
                  stride_b % 8 == 0 && stride_h % 8 == 0 && stride_t % 8 == 0,
              S3R_ERR_ALIGNMENT, "s3r_pool_fwd: pointers and strides must keep 16-byte alignment");
  int Nc = (T - kernel) / stride + 1;
  int64_t total = static_cast<int64_t>(B) * Nc * H * (d / 8);
  pool_fwd_kernel<<<pool_grid(total), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(in), stride_b, stride_h, stride_t, static_cast<__nv_bfloat16*>(out), B, H, T,
      d, Nc, kernel, stride);
  S3R_CUDA(cudaGetLastError());
  return 0;
}

extern "C" int s3r_pool_bwd(const void* d_out, void* d_in, int64_t stride_b, int64_t stride_h, int64_t stride_t,
                            int B, int H, int T, int d, int kernel, int stride, int accumulate, void* stream) {
  S3R_REQUIRE(d_out && d_in, S3R_ERR_NULL, "s3r_pool_bwd: NULL pointer");
  S3R_REQUIRE(B > 0 && H > 0 && T > 0 && d > 0 && kernel > 0 && stride > 0 && T >= kernel, S3R_ERR_SHAPE,
              "s3r_pool_bwd: bad sizes (B=%d H=%d T=%d d=%d kernel=%d stride=%d)", B, H, T, d, kernel, stride);
  S3R_REQUIRE(d % 8 == 0, S3R_ERR_UNSUPPORTED, "s3r_pool_bwd: head_dim %d is not a multiple of 8", d);
  S3R_REQUIRE((reinterpret_cast<uintptr_t>(d_out) & 15) == 0 && (reinterpret_cast<uintptr_t>(d_in) & 15) == 0 &&
                  stride_b % 8 == 0 && stride_h % 8 == 0 && stride_t % 8 == 0,
              S3R_ERR_ALIGNMENT, "s3r_pool_bwd: pointers and strides must keep 16-byte alignment");
  int Nc = (T - kernel) / stride + 1;
  int64_t total = static_cast<int64_t>(B) * T * H * (d / 8);
  pool_bwd_kernel<<<pool_grid(total), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(d_out), static_cast<__nv_bfloat16*>(d_in), stride_b, stride_h, stride_t, B, H,
      T, d, Nc, kernel, stride, accumulate);
  S3R_CUDA(cudaGetLastError());
  return 0;
}
