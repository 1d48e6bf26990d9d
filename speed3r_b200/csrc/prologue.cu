// Prologue of the sparse global attention, one pass over the packed projection: everything the reference
// does between `qkv = self.qkv(x)` and its two attention calls
// (pi3/models/layers/sparse_attention.py:95-123): split into q, k, v in [B,H,N,d], per-head LayerNorm of q
// and k, 2-D rotary embedding at the token positions, and for the compression branch the block means of
// the RAW q, k, v followed by the same LayerNorm and the rotary embedding at the block's mean position.
// In PyTorch that is about fifteen elementwise passes over [B,H,N,d]; here the projection is read once
// (6 KB per token, contiguous) and each output written once, so the kernel is bounded by HBM:
// 2 * 3*N*H*d*2 bytes plus the pooled tensors.
//
// One CTA owns one block of `block` tokens of one batch element; eight lanes own one (q|k|v, head) row
// of 64 channels (16 bytes per lane) and walk the block's tokens, so a block's mean never leaves
// registers.  Rounding points follow the reference under bf16 autocast: LayerNorm in fp32 from bf16
// input, rounded to bf16; the rotary products and their sum each rounded to bf16; the block mean
// accumulated in fp32 and rounded once.  cos/sin come from the caller's table (angles rounded to bf16
// before cos/sin, pi3/models/layers/pos_embed.py:112-159), so they are bit-identical to the reference's.
#include "common.cuh"

namespace s3r {

struct PrologueParams {
  const __nv_bfloat16* qkv;          // [B,N,3,H,64]
  const int64_t* pos;                // [B,N,2] (y,x) or null: no rotary embedding
  const __nv_bfloat16* cos_tab;      // [tab_rows,32]
  const __nv_bfloat16* sin_tab;
  int tab_rows;
  const float* qw; const float* qb;  // LayerNorm affine of q (null: no normalisation)
  const float* kw; const float* kb;
  float eps;
  __nv_bfloat16 *q, *k, *v, *q_c, *k_c, *v_c;
  int B, H, N, Nc, block;
  uint32_t* status;                  // device status word: a position outside the tables sets kStatusBadIndex
};

struct alignas(16) Vec8 {
  uint32_t w[4];
};

__device__ __forceinline__ float bf16r(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }

// LayerNorm over the 64 channels held by 8 lanes (8 each), fp32, two passes; the caller rounds to bf16.
// `gmask` names the 8 lanes of the row: rows of one warp may belong to different tensors (q, k or v) and
// take different paths, so every shuffle synchronises its own group only.
__device__ __forceinline__ void ln_row(float (&x)[8], const float (&w)[8], const float (&b)[8], float eps,
                                       uint32_t gmask) {
  float s = 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) s += x[i];
  s += __shfl_xor_sync(gmask, s, 1);
  s += __shfl_xor_sync(gmask, s, 2);
  s += __shfl_xor_sync(gmask, s, 4);
  const float mean = s * (1.f / 64.f);
  float v = 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) { const float dlt = x[i] - mean; v = fmaf(dlt, dlt, v); }
  v += __shfl_xor_sync(gmask, v, 1);
  v += __shfl_xor_sync(gmask, v, 2);
  v += __shfl_xor_sync(gmask, v, 4);
  const float rstd = rsqrtf(v * (1.f / 64.f) + eps);
#pragma unroll
  for (int i = 0; i < 8; ++i) x[i] = fmaf((x[i] - mean) * rstd, w[i], b[i]);   // rounded to bf16 when packed
}

// 2-D rotary embedding of a row held by 8 lanes, on packed bf16 pairs: lanes 0-3 hold the y half (32
// channels), lanes 4-7 the x half; inside a half channel j pairs with j+16, i.e. lane l with lane l^2.
// out = bf16(bf16(t*cos) + bf16(rot*sin)),  rot = -t[j+16] for j < 16 and t[j-16] otherwise: the packed
// bf16 multiply and add (the _rn forms, which the compiler may not contract into one FMA) round exactly
// where the reference's bf16 tensor ops do.
__device__ __forceinline__ uint32_t bf2_mul(uint32_t a, uint32_t b) {
  const __nv_bfloat162 r = __hmul2_rn(*reinterpret_cast<const __nv_bfloat162*>(&a), *reinterpret_cast<const __nv_bfloat162*>(&b));
  return *reinterpret_cast<const uint32_t*>(&r);
}
__device__ __forceinline__ uint32_t bf2_add(uint32_t a, uint32_t b) {
  const __nv_bfloat162 r = __hadd2_rn(*reinterpret_cast<const __nv_bfloat162*>(&a), *reinterpret_cast<const __nv_bfloat162*>(&b));
  return *reinterpret_cast<const uint32_t*>(&r);
}
__device__ __forceinline__ void rope_row(uint32_t (&xw)[4], const __nv_bfloat16* __restrict__ cos_tab,
                                         const __nv_bfloat16* __restrict__ sin_tab, int row, int l8,
                                         uint32_t gmask) {
  const Vec8 c = *reinterpret_cast<const Vec8*>(cos_tab + static_cast<int64_t>(row) * 32 + (l8 & 3) * 8);
  const Vec8 s = *reinterpret_cast<const Vec8*>(sin_tab + static_cast<int64_t>(row) * 32 + (l8 & 3) * 8);
  const uint32_t flip = (l8 & 2) == 0 ? 0x80008000u : 0u;
#pragma unroll
  for (int wd = 0; wd < 4; ++wd) {
    const uint32_t other = __shfl_xor_sync(gmask, xw[wd], 2) ^ flip;
    xw[wd] = bf2_add(bf2_mul(xw[wd], c.w[wd]), bf2_mul(other, s.w[wd]));
  }
}

// kMaxThreads = 384 covers up to 16 heads with 80 registers per thread at two CTAs per SM; more heads use
// the 1024-thread form (64 registers).
template <int kMaxThreads>
__global__ void __launch_bounds__(kMaxThreads, kMaxThreads <= 384 ? 2 : 1)
prologue_fwd_kernel(const PrologueParams p) {
  const int l8 = threadIdx.x & 7;
  const int g = threadIdx.x >> 3;                  // row of the token: (q|k|v, head)
  const uint32_t gmask = 0xffu << (threadIdx.x & 24);
  const int which = g / p.H, h = g - which * p.H;
  const int b = blockIdx.x / p.Nc, j = blockIdx.x - b * p.Nc;
  const float* lw = which == 0 ? p.qw : p.kw;
  const float* lb = which == 0 ? p.qb : p.kb;
  const bool norm = which < 2 && lw != nullptr;
  const bool rope = which < 2 && p.pos != nullptr;
  __nv_bfloat16* out = which == 0 ? p.q : (which == 1 ? p.k : p.v);
  __nv_bfloat16* out_c = which == 0 ? p.q_c : (which == 1 ? p.k_c : p.v_c);
  const int64_t bh = static_cast<int64_t>(b) * p.H + h;

  float wreg[8], breg[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    wreg[i] = norm ? __ldg(lw + l8 * 8 + i) : 1.f;
    breg[i] = norm ? __ldg(lb + l8 * 8 + i) : 0.f;
  }
  float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  float pos_sum = 0.f;                              // of this lane's coordinate (y for lanes 0-3, x for 4-7)
  const int n0 = j * p.block;
  const __nv_bfloat16* src0 = p.qkv + ((static_cast<int64_t>(b) * p.N + n0) * 3 * p.H + g) * 64 + l8 * 8;
  const int64_t tok_stride = static_cast<int64_t>(3) * p.H * 64;
  auto load = [&](int t) { return *reinterpret_cast<const Vec8*>(src0 + t * tok_stride); };
  // one token of this row: accumulate the raw block sum, normalise, rotate, store
  auto token = [&](int n, const Vec8& raw) {
    float x[8];
#pragma unroll
    for (int wd = 0; wd < 4; ++wd) { x[2 * wd] = bf16_lo(raw.w[wd]); x[2 * wd + 1] = bf16_hi(raw.w[wd]); }
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] += x[i];
    Vec8 o = raw;
    if (which < 2) {
      if (norm) {
        ln_row(x, wreg, breg, p.eps, gmask);
#pragma unroll
        for (int wd = 0; wd < 4; ++wd) o.w[wd] = pack_bf16(x[2 * wd], x[2 * wd + 1]);
      }
      if (rope) {
        const int64_t pv = p.pos[(static_cast<int64_t>(b) * p.N + n) * 2 + (l8 >> 2)];
        pos_sum += static_cast<float>(pv);
        const int row = min(max(static_cast<int>(pv), 0), p.tab_rows - 1);
        if (pv != row) atomicOr(p.status, kStatusBadIndex);      // clamped: the result for this token is wrong
        rope_row(o.w, p.cos_tab, p.sin_tab, row, l8, gmask);
      }
    }
    *reinterpret_cast<Vec8*>(out + (bh * p.N + n) * 64 + l8 * 8) = o;
  };
  // The kernel lives on bytes in flight: the loads of the next four tokens are issued before the current
  // four are processed (their shuffle and rounding chains are long, the loads are independent of them).
  Vec8 cur[4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
    if (i < p.block) cur[i] = load(i);
  for (int t0 = 0; t0 < p.block; t0 += 4) {
    Vec8 nxt[4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
      if (t0 + 4 + i < p.block) nxt[i] = load(t0 + 4 + i);
#pragma unroll
    for (int i = 0; i < 4; ++i)
      if (t0 + i < p.block) token(n0 + t0 + i, cur[i]);
#pragma unroll
    for (int i = 0; i < 4; ++i) cur[i] = nxt[i];
  }
  // compression branch: mean of the raw rows, then the same norm and the rotary embedding at the block's
  // mean position (float mean, truncated: xpos.view(..).float().mean(dim=2).int())
  const float inv = 1.f / static_cast<float>(p.block);
  float x[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) x[i] = bf16r(acc[i] * inv);
  if (norm) ln_row(x, wreg, breg, p.eps, gmask);
  Vec8 o;
#pragma unroll
  for (int wd = 0; wd < 4; ++wd) o.w[wd] = pack_bf16(x[2 * wd], x[2 * wd + 1]);
  if (rope) {
    const int pc = static_cast<int>(pos_sum / static_cast<float>(p.block));
    const int row = min(max(pc, 0), p.tab_rows - 1);
    if (pc != row) atomicOr(p.status, kStatusBadIndex);
    rope_row(o.w, p.cos_tab, p.sin_tab, row, l8, gmask);
  }
  *reinterpret_cast<Vec8*>(out_c + (bh * p.Nc + j) * 64 + l8 * 8) = o;
}

}  // namespace s3r

using namespace s3r;

extern "C" int s3r_qkv_prologue_fwd(const void* qkv, const int64_t* pos, const void* cos_tab, const void* sin_tab,
                                    int tab_rows, const float* q_weight, const float* q_bias, const float* k_weight,
                                    const float* k_bias, float eps, void* q, void* k, void* v, void* q_c, void* k_c,
                                    void* v_c, int B, int H, int N, int d, int block, void* stream) {
  S3R_REQUIRE(qkv && q && k && v && q_c && k_c && v_c, S3R_ERR_NULL, "s3r_qkv_prologue_fwd: NULL tensor");
  S3R_REQUIRE(B > 0 && H > 0 && N > 0 && block > 0, S3R_ERR_SHAPE,
              "s3r_qkv_prologue_fwd: sizes must be positive (B=%d H=%d N=%d block=%d)", B, H, N, block);
  S3R_REQUIRE(d == 64, S3R_ERR_UNSUPPORTED, "s3r_qkv_prologue_fwd: head_dim %d not supported (64 only)", d);
  S3R_REQUIRE(N % block == 0, S3R_ERR_SHAPE, "s3r_qkv_prologue_fwd: N=%d is not a multiple of the block %d", N, block);
  S3R_REQUIRE(3 * H * 8 <= 1024, S3R_ERR_UNSUPPORTED, "s3r_qkv_prologue_fwd: %d heads exceed one CTA (42 at most)", H);
  S3R_REQUIRE((q_weight != nullptr) == (q_bias != nullptr) && (k_weight != nullptr) == (k_bias != nullptr) &&
                  (q_weight != nullptr) == (k_weight != nullptr),
              S3R_ERR_NULL, "s3r_qkv_prologue_fwd: LayerNorm weights and biases of q and k come together or not at all");
  S3R_REQUIRE(pos == nullptr || (cos_tab && sin_tab && tab_rows > 0), S3R_ERR_NULL,
              "s3r_qkv_prologue_fwd: positions need the cos/sin tables");
  const uintptr_t al = reinterpret_cast<uintptr_t>(qkv) | reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k) |
                       reinterpret_cast<uintptr_t>(v) | reinterpret_cast<uintptr_t>(q_c) |
                       reinterpret_cast<uintptr_t>(k_c) | reinterpret_cast<uintptr_t>(v_c) |
                       reinterpret_cast<uintptr_t>(cos_tab) | reinterpret_cast<uintptr_t>(sin_tab);
  S3R_REQUIRE((al & 15) == 0, S3R_ERR_ALIGNMENT, "s3r_qkv_prologue_fwd: tensors must be 16-byte aligned");
  const int Nc = N / block;
  const int64_t grid = static_cast<int64_t>(B) * Nc;
  S3R_REQUIRE(grid < (1ll << 31), S3R_ERR_TOO_LARGE, "s3r_qkv_prologue_fwd: grid of %lld CTAs is too large",
              (long long)grid);
  PrologueParams p;
  p.qkv = static_cast<const __nv_bfloat16*>(qkv);
  p.pos = pos;
  p.cos_tab = static_cast<const __nv_bfloat16*>(cos_tab);
  p.sin_tab = static_cast<const __nv_bfloat16*>(sin_tab);
  p.tab_rows = tab_rows;
  p.qw = q_weight; p.qb = q_bias; p.kw = k_weight; p.kb = k_bias;
  p.eps = eps;
  p.q = static_cast<__nv_bfloat16*>(q); p.k = static_cast<__nv_bfloat16*>(k); p.v = static_cast<__nv_bfloat16*>(v);
  p.q_c = static_cast<__nv_bfloat16*>(q_c); p.k_c = static_cast<__nv_bfloat16*>(k_c);
  p.v_c = static_cast<__nv_bfloat16*>(v_c);
  p.B = B; p.H = H; p.N = N; p.Nc = Nc; p.block = block;
  p.status = device_status_ptr();
  S3R_REQUIRE(p.status != nullptr, S3R_ERR_DRIVER, "s3r_qkv_prologue_fwd: could not resolve the device status word");
  if (3 * H * 8 <= 384)
    prologue_fwd_kernel<384><<<static_cast<unsigned>(grid), 3 * H * 8, 0, static_cast<cudaStream_t>(stream)>>>(p);
  else
    prologue_fwd_kernel<1024><<<static_cast<unsigned>(grid), 3 * H * 8, 0, static_cast<cudaStream_t>(stream)>>>(p);
  S3R_CUDA(cudaGetLastError());
  return 0;
}
