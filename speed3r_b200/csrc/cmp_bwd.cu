// Compression branch, backward: dense flash-attention backward over the pooled tensors.
//   delta = sum_d o*do ; dQ kernel: CTA = 128 query rows x all key tiles of 64 ;
//   dK/dV kernel: CTA = 128 key rows x all query tiles of 64.
// Tiles are shared by the CTA's 8 warps through a two-stage cp.async ring; the arithmetic is the
// mma.sync building blocks of bwd_common.cuh (P and dS are rounded to bf16 before the second
// products, like the reference kernels).
#include "bwd_common.cuh"

namespace s3r {

constexpr int kCbWarps = 8;
constexpr int kCbRows = kCbWarps * 16;        // rows owned by a CTA
constexpr int kCbTile = 64;                   // rows per streamed tile
constexpr int kCbTileBytes = kCbTile * kPitch;
constexpr int kCbStageBytes = 2 * kCbTileBytes;

struct CmpBwdParams {
  const __nv_bfloat16 *q, *k, *v, *d_o;
  const float *lse, *delta;
  __nv_bfloat16 *dq, *dk, *dv;
  int Nq, Nc;
  float cs, scale;
};

// `rows` rows x 128 B -> padded tile, all 256 threads; rows >= nrows zero-filled
__device__ __forceinline__ void cta_load_tile(uint32_t dst, const __nv_bfloat16* src, int rows, int nrows, int tid) {
  for (int ch = tid; ch < rows * 8; ch += kCbWarps * 32) {
    const int r = ch >> 3, c16 = ch & 7;
    cp_async16(dst + r * kPitch + c16 * 16, src + static_cast<int64_t>(r) * 64 + c16 * 8, r < nrows);
  }
}

__global__ void __launch_bounds__(kCbWarps * 32) cmp_bwd_dq_kernel(const CmpBwdParams p) {
  __shared__ __align__(16) uint8_t smem[2][kCbStageBytes];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2;
  const int ctas = (p.Nq + kCbRows - 1) / kCbRows;
  const int bh = blockIdx.x / ctas;
  const int row0 = (blockIdx.x % ctas) * kCbRows;
  const uint32_t sm[2] = {smem_u32(&smem[0][0]), smem_u32(&smem[1][0])};

  // Q (stage 0) and dO (stage 1): 128 rows each
  cta_load_tile(sm[0], p.q + (static_cast<int64_t>(bh) * p.Nq + row0) * 64, kCbRows, p.Nq - row0, threadIdx.x);
  cta_load_tile(sm[1], p.d_o + (static_cast<int64_t>(bh) * p.Nq + row0) * 64, kCbRows, p.Nq - row0, threadIdx.x);
  cp_async_commit();
  cp_async_wait<0>();
  __syncthreads();
  uint32_t qf[4][4], dof[4][4];
  load_a_frags(qf, sm[0] + warp * 16 * kPitch, lane);
  load_a_frags(dof, sm[1] + warp * 16 * kPitch, lane);
  __syncthreads();
  float lse2[2], delta[2];
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const int t = row0 + warp * 16 + g + 8 * r;
    lse2[r] = (t < p.Nq) ? p.lse[static_cast<int64_t>(bh) * p.Nq + t] * 1.4426950408889634f : INFINITY;
    delta[r] = (t < p.Nq) ? p.delta[static_cast<int64_t>(bh) * p.Nq + t] : 0.f;
  }
  float dq[8][4] = {};
  const __nv_bfloat16* Kb = p.k + static_cast<int64_t>(bh) * p.Nc * 64;
  const __nv_bfloat16* Vb = p.v + static_cast<int64_t>(bh) * p.Nc * 64;
  const int ntiles = (p.Nc + kCbTile - 1) / kCbTile;
  auto prefetch = [&](int it) {
    const int k0 = it * kCbTile;
    cta_load_tile(sm[it & 1], Kb + static_cast<int64_t>(k0) * 64, kCbTile, p.Nc - k0, threadIdx.x);
    cta_load_tile(sm[it & 1] + kCbTileBytes, Vb + static_cast<int64_t>(k0) * 64, kCbTile, p.Nc - k0, threadIdx.x);
    cp_async_commit();
  };
  prefetch(0);
  for (int it = 0; it < ntiles; ++it) {
    if (it + 1 < ntiles) { prefetch(it + 1); cp_async_wait<1>(); } else { cp_async_wait<0>(); }
    __syncthreads();
    const uint32_t cur = sm[it & 1];
#pragma unroll
    for (int sb = 0; sb < kCbTile / 16; ++sb) {
      const int kv = p.Nc - (it * kCbTile + sb * 16);
      if (kv > 0)
        pair_dq(qf, dof, lse2, delta, cur + sb * 16 * kPitch, cur + kCbTileBytes + sb * 16 * kPitch, min(16, kv), p.cs,
                p.scale, dq, lane);
    }
    __syncthreads();
  }
  const int wrow0 = row0 + warp * 16;
  __nv_bfloat16* out = p.dq + (static_cast<int64_t>(bh) * p.Nq + wrow0) * 64;
  store_acc_bf16(dq, [&](int r) { return (wrow0 + r < p.Nq) ? out + r * 64 : nullptr; }, lane);
}

__global__ void __launch_bounds__(kCbWarps * 32, 2) cmp_bwd_dkdv_kernel(const CmpBwdParams p) {
  __shared__ __align__(16) uint8_t smem[2][kCbStageBytes];
  __shared__ float stats[2][2 * kCbTile];      // [stage][lse2 x64 | delta x64]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int ctas = (p.Nc + kCbRows - 1) / kCbRows;
  const int bh = blockIdx.x / ctas;
  const int row0 = (blockIdx.x % ctas) * kCbRows;
  const uint32_t sm[2] = {smem_u32(&smem[0][0]), smem_u32(&smem[1][0])};

  cta_load_tile(sm[0], p.k + (static_cast<int64_t>(bh) * p.Nc + row0) * 64, kCbRows, p.Nc - row0, threadIdx.x);
  cta_load_tile(sm[1], p.v + (static_cast<int64_t>(bh) * p.Nc + row0) * 64, kCbRows, p.Nc - row0, threadIdx.x);
  cp_async_commit();
  cp_async_wait<0>();
  __syncthreads();
  uint32_t kf[4][4], vf[4][4];
  load_a_frags(kf, sm[0] + warp * 16 * kPitch, lane);
  load_a_frags(vf, sm[1] + warp * 16 * kPitch, lane);
  __syncthreads();

  float dk[8][4] = {}, dv[8][4] = {};
  const __nv_bfloat16* Qb = p.q + static_cast<int64_t>(bh) * p.Nq * 64;
  const __nv_bfloat16* Db = p.d_o + static_cast<int64_t>(bh) * p.Nq * 64;
  const float* Lb = p.lse + static_cast<int64_t>(bh) * p.Nq;
  const float* Eb = p.delta + static_cast<int64_t>(bh) * p.Nq;
  const int ntiles = (p.Nq + kCbTile - 1) / kCbTile;
  auto prefetch = [&](int it) {
    const int q0 = it * kCbTile;
    cta_load_tile(sm[it & 1], Qb + static_cast<int64_t>(q0) * 64, kCbTile, p.Nq - q0, threadIdx.x);
    cta_load_tile(sm[it & 1] + kCbTileBytes, Db + static_cast<int64_t>(q0) * 64, kCbTile, p.Nq - q0, threadIdx.x);
    cp_async_commit();
    if (threadIdx.x < 2 * kCbTile) {
      const int t = q0 + (threadIdx.x & (kCbTile - 1));
      float val;
      if (threadIdx.x < kCbTile) val = (t < p.Nq) ? Lb[t] * 1.4426950408889634f : INFINITY;
      else val = (t < p.Nq) ? Eb[t] : 0.f;
      stats[it & 1][threadIdx.x] = val;
    }
  };
  prefetch(0);
  for (int it = 0; it < ntiles; ++it) {
    if (it + 1 < ntiles) { prefetch(it + 1); cp_async_wait<1>(); } else { cp_async_wait<0>(); }
    __syncthreads();
    const uint32_t cur = sm[it & 1];
#pragma unroll
    for (int sb = 0; sb < kCbTile / 16; ++sb) {
      if (it * kCbTile + sb * 16 < p.Nq)
        pair_dkdv(kf, vf, cur + sb * 16 * kPitch, cur + kCbTileBytes + sb * 16 * kPitch, &stats[it & 1][sb * 16],
                  &stats[it & 1][kCbTile + sb * 16], p.cs, p.scale, dk, dv, lane);
    }
    __syncthreads();
  }
  const int wrow0 = row0 + warp * 16;
  __nv_bfloat16* okp = p.dk + (static_cast<int64_t>(bh) * p.Nc + wrow0) * 64;
  __nv_bfloat16* ovp = p.dv + (static_cast<int64_t>(bh) * p.Nc + wrow0) * 64;
  store_acc_bf16(dk, [&](int r) { return (wrow0 + r < p.Nc) ? okp + r * 64 : nullptr; }, lane);
  store_acc_bf16(dv, [&](int r) { return (wrow0 + r < p.Nc) ? ovp + r * 64 : nullptr; }, lane);
}

}  // namespace s3r

using namespace s3r;

extern "C" int s3r_cmp_attn_bwd(const void* q_c, const void* k_c, const void* v_c, const void* o_c, const float* lse,
                                const void* do_c, float* delta, void* dq_c, void* dk_c, void* dv_c, int B, int H,
                                int Nq, int Nc, int d, float scale, void* stream) {
  S3R_REQUIRE(q_c && k_c && v_c && o_c && lse && do_c && delta && dq_c && dk_c && dv_c, S3R_ERR_NULL,
              "s3r_cmp_attn_bwd: NULL pointer");
  S3R_REQUIRE(B > 0 && H > 0 && Nq > 0 && Nc > 0, S3R_ERR_SHAPE, "s3r_cmp_attn_bwd: bad sizes");
  S3R_REQUIRE(d == 64, S3R_ERR_UNSUPPORTED, "s3r_cmp_attn_bwd: head_dim %d not supported (64 only)", d);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  int rc = s3r_delta(o_c, do_c, delta, static_cast<int64_t>(B) * H * Nq, d, stream);
  if (rc) return rc;
  CmpBwdParams p;
  p.q = static_cast<const __nv_bfloat16*>(q_c);
  p.k = static_cast<const __nv_bfloat16*>(k_c);
  p.v = static_cast<const __nv_bfloat16*>(v_c);
  p.d_o = static_cast<const __nv_bfloat16*>(do_c);
  p.lse = lse; p.delta = delta;
  p.dq = static_cast<__nv_bfloat16*>(dq_c);
  p.dk = static_cast<__nv_bfloat16*>(dk_c);
  p.dv = static_cast<__nv_bfloat16*>(dv_c);
  p.Nq = Nq; p.Nc = Nc;
  p.cs = scale * 1.4426950408889634f;
  p.scale = scale;
  const int BH = B * H;
  cmp_bwd_dkdv_kernel<<<BH * ((Nc + kCbRows - 1) / kCbRows), kCbWarps * 32, 0, st>>>(p);
  cmp_bwd_dq_kernel<<<BH * ((Nq + kCbRows - 1) / kCbRows), kCbWarps * 32, 0, st>>>(p);
  S3R_CUDA(cudaGetLastError());
  return 0;
}
