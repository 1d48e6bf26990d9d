// Warp-level building blocks shared by the backward kernels of both branches (mma.sync m16n8k16,
// operands in shared memory with a 144-byte row pitch so that ldmatrix is bank-conflict free).
//
// Notation: one warp owns 16 "row" items (queries in the dQ kernels, keys in the dK/dV kernels)
// and meets 16 "column" items (keys, resp. queries) at a time.
#pragma once
#include "common.cuh"

namespace s3r {

constexpr int kPitch = 144;   // bytes per 64-element bf16 row in shared memory (128 + 16 padding)

__device__ __forceinline__ void cp_async16(uint32_t dst_smem, const void* src, bool valid) {
  // src-size 0 zero-fills the destination without touching global memory
  const int sz = valid ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst_smem), "l"(src), "r"(sz) : "memory");
}
// one 32-bit word; src-size 0 zero-fills
__device__ __forceinline__ void cp_async4(uint32_t dst_smem, const void* src, bool valid) {
  const int sz = valid ? 4 : 0;
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;" ::"r"(dst_smem), "l"(src), "r"(sz) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

// A-operand fragments (16 rows x 64) of the tile whose first row is at `base` (shared address).
__device__ __forceinline__ void load_a_frags(uint32_t (&f)[4][4], uint32_t base, int lane) {
  const uint32_t row = (lane & 7) + ((lane >> 3) & 1) * 8;
#pragma unroll
  for (int ks = 0; ks < 4; ++ks)
    ldsm_x4(f[ks][0], f[ks][1], f[ks][2], f[ks][3], base + row * kPitch + (2 * ks + (lane >> 4)) * 16);
}
// B operand "rows are n, columns are k" (X^T products): 16 n-rows starting at `base`, k-step ks.
__device__ __forceinline__ void load_b_nk(uint32_t (&b)[4], uint32_t base, int ks, int lane) {
  const uint32_t row = (lane & 7) + (lane >> 4) * 8;
  ldsm_x4(b[0], b[1], b[2], b[3], base + row * kPitch + (2 * ks + ((lane >> 3) & 1)) * 16);
}
// B operand "rows are k, columns are n" (X products): 16 k-rows starting at `base`, n columns 16*dp..
__device__ __forceinline__ void load_b_kn(uint32_t (&b)[4], uint32_t base, int dp, int lane) {
  const uint32_t row = (lane & 7) + ((lane >> 3) & 1) * 8;
  ldsm_x4_t(b[0], b[1], b[2], b[3], base + row * kPitch + (2 * dp + (lane >> 4)) * 16);
}

// dQ contribution of 16 keys to this warp's 16 queries.
//   qf, dof : A fragments of Q and dO (16 x 64)
//   lse2[2], delta[2] : log2-domain lse and delta of rows g and g+8
//   ksm, vsm : shared addresses of the 16 key rows / value rows
//   kvalid   : number of real keys among the 16 (the rest are zero-filled padding)
__device__ __forceinline__ void pair_dq(const uint32_t (&qf)[4][4], const uint32_t (&dof)[4][4], const float (&lse2)[2],
                                        const float (&delta)[2], uint32_t ksm, uint32_t vsm, int kvalid, float cs,
                                        float scale, float (&dq)[8][4], int lane) {
  float s[2][4] = {}, dp[2][4] = {};
#pragma unroll
  for (int ks = 0; ks < 4; ++ks) {
    uint32_t b[4];
    load_b_nk(b, ksm, ks, lane);
    mma_bf16(s[0], qf[ks], b[0], b[1]);
    mma_bf16(s[1], qf[ks], b[2], b[3]);
    load_b_nk(b, vsm, ks, lane);
    mma_bf16(dp[0], dof[ks], b[0], b[1]);
    mma_bf16(dp[1], dof[ks], b[2], b[3]);
  }
  const int c = lane & 3;
  float ds[2][4];
#pragma unroll
  for (int nt = 0; nt < 2; ++nt)
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int r = e >> 1;
      const int key = nt * 8 + 2 * c + (e & 1);
      float pr = fast_exp2(fmaf(s[nt][e], cs, -lse2[r]));
      if (key >= kvalid) pr = 0.f;
      ds[nt][e] = pr * (dp[nt][e] - delta[r]) * scale;
    }
  uint32_t a[4] = {pack_bf16(ds[0][0], ds[0][1]), pack_bf16(ds[0][2], ds[0][3]), pack_bf16(ds[1][0], ds[1][1]),
                   pack_bf16(ds[1][2], ds[1][3])};
#pragma unroll
  for (int d4 = 0; d4 < 4; ++d4) {
    uint32_t b[4];
    load_b_kn(b, ksm, d4, lane);
    mma_bf16(dq[2 * d4], a, b[0], b[1]);
    mma_bf16(dq[2 * d4 + 1], a, b[2], b[3]);
  }
}

// dK / dV contribution of 16 queries to this warp's 16 keys.
//   kf, vf : A fragments of K and V (16 keys x 64)
//   qsm, dosm : shared addresses of the 16 query rows of Q and dO
//   lse2s, deltas : shared arrays (16 floats) for those queries; lse2 = +inf marks a padding query
__device__ __forceinline__ void pair_dkdv(const uint32_t (&kf)[4][4], const uint32_t (&vf)[4][4], uint32_t qsm,
                                          uint32_t dosm, const float* lse2s, const float* deltas, float cs,
                                          float scale, float (&dk)[8][4], float (&dv)[8][4], int lane) {
  float st[2][4] = {}, dpt[2][4] = {};
#pragma unroll
  for (int ks = 0; ks < 4; ++ks) {
    uint32_t b[4];
    load_b_nk(b, qsm, ks, lane);
    mma_bf16(st[0], kf[ks], b[0], b[1]);
    mma_bf16(st[1], kf[ks], b[2], b[3]);
    load_b_nk(b, dosm, ks, lane);
    mma_bf16(dpt[0], vf[ks], b[0], b[1]);
    mma_bf16(dpt[1], vf[ks], b[2], b[3]);
  }
  const int c = lane & 3;
  float pt[2][4], ds[2][4];
#pragma unroll
  for (int nt = 0; nt < 2; ++nt)
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const int qc = nt * 8 + 2 * c + (e & 1);
      const float pr = fast_exp2(fmaf(st[nt][e], cs, -lse2s[qc]));
      pt[nt][e] = pr;
      ds[nt][e] = pr * (dpt[nt][e] - deltas[qc]) * scale;
    }
  uint32_t pa[4] = {pack_bf16(pt[0][0], pt[0][1]), pack_bf16(pt[0][2], pt[0][3]), pack_bf16(pt[1][0], pt[1][1]),
                    pack_bf16(pt[1][2], pt[1][3])};
  uint32_t da[4] = {pack_bf16(ds[0][0], ds[0][1]), pack_bf16(ds[0][2], ds[0][3]), pack_bf16(ds[1][0], ds[1][1]),
                    pack_bf16(ds[1][2], ds[1][3])};
#pragma unroll
  for (int d4 = 0; d4 < 4; ++d4) {
    uint32_t b[4];
    load_b_kn(b, dosm, d4, lane);
    mma_bf16(dv[2 * d4], pa, b[0], b[1]);
    mma_bf16(dv[2 * d4 + 1], pa, b[2], b[3]);
    load_b_kn(b, qsm, d4, lane);
    mma_bf16(dk[2 * d4], da, b[0], b[1]);
    mma_bf16(dk[2 * d4 + 1], da, b[2], b[3]);
  }
}

// Store a 16 x 64 fp32 accumulator tile (mma C layout) as bf16 rows of 128 bytes.
// row_ptr(r) must give the global address of row r (0..15) or nullptr to skip it.
template <typename RowPtr>
__device__ __forceinline__ void store_acc_bf16(const float (&acc)[8][4], RowPtr row_ptr, int lane) {
  const int g = lane >> 2, c = lane & 3;
  __nv_bfloat16* r0 = row_ptr(g);
  __nv_bfloat16* r1 = row_ptr(g + 8);
#pragma unroll
  for (int dt = 0; dt < 8; ++dt) {
    if (r0) *reinterpret_cast<uint32_t*>(r0 + dt * 8 + 2 * c) = pack_bf16(acc[dt][0], acc[dt][1]);
    if (r1) *reinterpret_cast<uint32_t*>(r1 + dt * 8 + 2 * c) = pack_bf16(acc[dt][2], acc[dt][3]);
  }
}

}  // namespace s3r
