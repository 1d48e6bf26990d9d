// Plain one-thread-per-query-row restatements of the two forward attentions (fp32 arithmetic on
// the bf16 inputs, exact expf/logf).  They are slow and exist only so that tests can cross-check
// the tensor-core kernels on the device at sizes a CPU check cannot reach.  No product path
// calls them.  The file also holds the probe of the bounded wait (a wait that is made to run out).
#include "../common.cuh"

namespace s3r {

constexpr int kChkThreads = 128;
constexpr int kChkTile = 32;
constexpr int kChkMaxTopk = 64;

__global__ void __launch_bounds__(kChkThreads)
check_cmp_kernel(const __nv_bfloat16* __restrict__ Q, const __nv_bfloat16* __restrict__ K,
                 const __nv_bfloat16* __restrict__ V, __nv_bfloat16* __restrict__ O, float* __restrict__ LSE,
                 int32_t* __restrict__ IDX, int Nq, int Nc, int topk, float scale) {
  __shared__ float ks[kChkTile][64];
  __shared__ float vs[kChkTile][64];
  const int bh = blockIdx.y;
  const int row = blockIdx.x * kChkThreads + threadIdx.x;
  const bool live = row < Nq;
  float q[64], acc[64];
  uint64_t best[kChkMaxTopk];   // descending; starts as zeros like the reference's running set
  for (int i = 0; i < kChkMaxTopk; ++i) best[i] = 0ull;
  for (int c = 0; c < 64; ++c) {
    q[c] = live ? __bfloat162float(Q[(static_cast<int64_t>(bh) * Nq + row) * 64 + c]) : 0.f;
    acc[c] = 0.f;
  }
  float m = -INFINITY, l = 0.f;
  for (int n0 = 0; n0 < Nc; n0 += kChkTile) {
    __syncthreads();
    for (int i = threadIdx.x; i < kChkTile * 64; i += kChkThreads) {
      int r = i >> 6, c = i & 63;
      bool in = n0 + r < Nc;
      int64_t off = (static_cast<int64_t>(bh) * Nc + n0 + r) * 64 + c;
      ks[r][c] = in ? __bfloat162float(K[off]) : 0.f;
      vs[r][c] = in ? __bfloat162float(V[off]) : 0.f;
    }
    __syncthreads();
    if (!live) continue;
    const int nk = min(kChkTile, Nc - n0);
    for (int r = 0; r < nk; ++r) {
      float s = 0.f;
#pragma unroll
      for (int c = 0; c < 64; ++c) s = fmaf(q[c], ks[r][c], s);
      // top-k on the raw logit
      const uint64_t comp = (static_cast<uint64_t>(sortable_key(s)) << 32) | static_cast<uint32_t>(Nc - 1 - (n0 + r));
      if (comp > best[topk - 1]) {
        int pos = topk - 1;
        while (pos > 0 && best[pos - 1] < comp) { best[pos] = best[pos - 1]; --pos; }
        best[pos] = comp;
      }
      // online softmax
      const float ss = s * scale;
      const float mn = fmaxf(m, ss);
      const float a = expf(m - mn), pr = expf(ss - mn);
      l = l * a + pr;
#pragma unroll
      for (int c = 0; c < 64; ++c) acc[c] = acc[c] * a + pr * vs[r][c];
      m = mn;
    }
  }
  if (!live) return;
  const float inv = 1.f / l;
  for (int c = 0; c < 64; ++c) O[(static_cast<int64_t>(bh) * Nq + row) * 64 + c] = __float2bfloat16(acc[c] * inv);
  LSE[static_cast<int64_t>(bh) * Nq + row] = m + logf(l);
  for (int i = 0; i < topk; ++i)
    IDX[(static_cast<int64_t>(bh) * Nq + row) * topk + i] = Nc - 1 - static_cast<int32_t>(best[i] & 0xffffffffull);
}

__global__ void __launch_bounds__(kChkThreads)
check_sel_kernel(const __nv_bfloat16* __restrict__ Q, const __nv_bfloat16* __restrict__ K,
                 const __nv_bfloat16* __restrict__ V, const int32_t* __restrict__ IDX, __nv_bfloat16* __restrict__ O,
                 float* __restrict__ LSE, int Tq, int Tk, int block, int topk, float scale) {
  const int bh = blockIdx.y;
  const int row = blockIdx.x * kChkThreads + threadIdx.x;
  if (row >= Tq) return;
  const int nqb = (Tq + block - 1) / block;
  const int32_t* list = IDX + (static_cast<int64_t>(bh) * nqb + row / block) * topk;
  float q[64], acc[64];
  for (int c = 0; c < 64; ++c) {
    q[c] = __bfloat162float(Q[(static_cast<int64_t>(bh) * Tq + row) * 64 + c]);
    acc[c] = 0.f;
  }
  float m = -INFINITY, l = 0.f;
  for (int i = 0; i < topk; ++i) {
    const int n = list[i];
    if (n < 0 || static_cast<int64_t>(n) * block >= Tk) continue;
    for (int r = 0; r < block; ++r) {
      const int tok = n * block + r;
      if (tok >= Tk) break;
      const __nv_bfloat16* kr = K + (static_cast<int64_t>(bh) * Tk + tok) * 64;
      const __nv_bfloat16* vr = V + (static_cast<int64_t>(bh) * Tk + tok) * 64;
      float s = 0.f;
      for (int c = 0; c < 64; ++c) s = fmaf(q[c], __bfloat162float(kr[c]), s);
      const float ss = s * scale;
      const float mn = fmaxf(m, ss);
      const float a = expf(m - mn), pr = expf(ss - mn);
      l = l * a + pr;
      for (int c = 0; c < 64; ++c) acc[c] = acc[c] * a + pr * __bfloat162float(vr[c]);
      m = mn;
    }
  }
  const float inv = l > 0.f ? 1.f / l : 0.f;
  for (int c = 0; c < 64; ++c) O[(static_cast<int64_t>(bh) * Tq + row) * 64 + c] = __float2bfloat16(acc[c] * inv);
  LSE[static_cast<int64_t>(bh) * Tq + row] = l > 0.f ? m + logf(l) : -INFINITY;
}

// One warp waits on a barrier nobody arrives on; the bounded wait has to give up after limit_ns.
__global__ void wait_probe_kernel(uint64_t limit_ns, uint64_t* waited_ns, uint32_t* status) {
  __shared__ uint64_t bar;
  __shared__ uint32_t abort_flag;
  if (threadIdx.x == 0) {
    abort_flag = 0;
    mbar_init(&bar, 1);
    mbar_fence_init();
  }
  __syncwarp();
  const uint64_t t0 = globaltimer_ns();
  const bool ok = mbar_wait_warp(&bar, 0, &abort_flag, limit_ns);
  const uint64_t dt = globaltimer_ns() - t0;
  if (threadIdx.x == 0) {
    *waited_ns = dt;
    if (!ok) atomicOr(status, kStatusWaitTimeout);
  }
}

}  // namespace s3r

using namespace s3r;

extern "C" int s3r_check_wait_gives_up(uint64_t limit_ns, uint64_t* waited_ns, void* stream) {
  S3R_REQUIRE(waited_ns != nullptr, S3R_ERR_NULL, "s3r_check_wait_gives_up: NULL pointer");
  S3R_REQUIRE(limit_ns > 0 && limit_ns <= 100000000ull, S3R_ERR_UNSUPPORTED,
              "s3r_check_wait_gives_up: the limit must be within (0, 100 ms]");
  uint32_t* status = device_status_ptr();
  S3R_REQUIRE(status != nullptr, S3R_ERR_DRIVER, "s3r_check_wait_gives_up: could not resolve the device status word");
  wait_probe_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(limit_ns, waited_ns, status);
  S3R_CUDA(cudaGetLastError());
  return 0;
}

extern "C" int s3r_check_cmp_attn_topk_fwd(const void* q_c, const void* k_c, const void* v_c, void* o_c, float* lse,
                                           int32_t* idx, int B, int H, int Nq, int Nc, int d, int topk, float scale,
                                           void* stream) {
  S3R_REQUIRE(q_c && k_c && v_c && o_c && lse && idx, S3R_ERR_NULL, "s3r_check_cmp_attn_topk_fwd: NULL pointer");
  S3R_REQUIRE(B > 0 && H > 0 && Nq > 0 && Nc > 0, S3R_ERR_SHAPE, "s3r_check_cmp_attn_topk_fwd: bad sizes");
  S3R_REQUIRE(d == 64 && topk > 0 && topk <= kChkMaxTopk, S3R_ERR_UNSUPPORTED,
              "s3r_check_cmp_attn_topk_fwd: d must be 64 and topk in [1,64]");
  dim3 grid((Nq + kChkThreads - 1) / kChkThreads, B * H);
  check_cmp_kernel<<<grid, kChkThreads, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(q_c), static_cast<const __nv_bfloat16*>(k_c),
      static_cast<const __nv_bfloat16*>(v_c), static_cast<__nv_bfloat16*>(o_c), lse, idx, Nq, Nc, topk, scale);
  S3R_CUDA(cudaGetLastError());
  return 0;
}

extern "C" int s3r_check_sel_attn_fwd(const void* q, const void* k, const void* v, const int32_t* idx, void* o_s,
                                      float* lse_s, int B, int H, int Tq, int Tk, int d, int block, int topk,
                                      float scale, void* stream) {
  S3R_REQUIRE(q && k && v && idx && o_s && lse_s, S3R_ERR_NULL, "s3r_check_sel_attn_fwd: NULL pointer");
  S3R_REQUIRE(B > 0 && H > 0 && Tq > 0 && Tk > 0 && block > 0 && topk > 0, S3R_ERR_SHAPE,
              "s3r_check_sel_attn_fwd: bad sizes");
  S3R_REQUIRE(d == 64, S3R_ERR_UNSUPPORTED, "s3r_check_sel_attn_fwd: d must be 64");
  dim3 grid((Tq + kChkThreads - 1) / kChkThreads, B * H);
  check_sel_kernel<<<grid, kChkThreads, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(q), static_cast<const __nv_bfloat16*>(k), static_cast<const __nv_bfloat16*>(v),
      idx, static_cast<__nv_bfloat16*>(o_s), lse_s, Tq, Tk, block, topk, scale);
  S3R_CUDA(cudaGetLastError());
  return 0;
}
