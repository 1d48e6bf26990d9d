// Compression branch, backward: dense flash-attention backward over the pooled tensors on the
// tensor-memory MMA (tcgen05), operands staged by TMA.
//
//   delta = sum_d o*do                                  (s3r_delta)
//   dK/dV kernel: a CTA owns 256 key rows (two M=128 row tiles) and streams all query tiles of 64 rows
//        S^T = K Q^T, dP^T = V dO^T                     (M=128 keys, N=64 queries, K=64)
//        P^T = exp2(S^T*c - lse[q]),  dS^T = P^T * (dP^T - delta[q])        thread = key row
//        dV += P^T dO,  dK += dS^T Q                    (M=128, N=64, K=64 queries; A from tensor memory)
//   dQ kernel: a CTA owns 256 query rows and streams all key tiles of 64 rows
//        S = Q K^T, dP = dO V^T;  dS = exp2(S*c - lse[row]) * (dP - delta[row]);  dQ += dS K
// P and dS are rounded to bf16 before the second products, like the reference kernels
// (flash_attention_topk.py:246-512); the softmax scale of dS is applied once, to the dK / dQ accumulators.
//
// One template covers both: the CTA's own tiles X0, X1 (K,V or Q,dO) are the A operands of the first
// products, the streamed tiles Y0, Y1 (64 rows; Q,dO or K,V) their B operands (K-major) and, read with
// the other descriptor, the B operands of the second products (N contiguous).
// Every CTA reads the whole streamed tensors from L2: bytes per score = 256 / owned rows (254 GB for both
// kernels at 1000 views with 128 owned rows), so a CTA owns 256 rows - as many as tensor memory holds
// accumulators for (2 row tiles x (dK, dV) x 64 columns = 256 columns; the other 256 hold S and dP).
// Roles: warp 0 TMA producer, warp 1 tcgen05.mma issuer, warp 2 tensor-memory allocator, warp 3 loads the
// streamed rows' lse/delta (dK/dV kernel), warps 4-7 and 8-11 one compute warpgroup per row tile.  P and dS
// are written in place, over the low columns of S and dP (a thread's bf16 chunk c covers columns
// 8c..8c+7, all of which it has already read as part of fp32 chunk c/2).  A tile goes through two
// passes per warpgroup - P from S (kept in registers as fp32), then dS from dP - each with its own
// pair of barriers, so that the next S is being multiplied while dS is computed and the next dP while the
// next P is.  Measured at 1000 views (Nq = Nc = 63000, 16 heads): 60 ms for both kernels, against 41 ms
// for the same MMA sequence with the arithmetic left out and 160 ms for the mma.sync kernels they replace.
#include "common.cuh"

namespace s3r {

constexpr int kCbThreads = 384;
constexpr int kCbStages = 6;
constexpr int kCbOwnRows = 256;
constexpr int kCbOwnBytes = 128 * 128;        // 128 rows x 64 bf16
constexpr int kCbStrBytes = 64 * 128;         // 64 rows x 64 bf16
constexpr int kCbOffX = 0;                                    // row tile t: X0 at t*2*kCbOwnBytes, X1 behind it
constexpr int kCbOffY = 4 * kCbOwnBytes;                      // ring of (Y0, Y1)
constexpr int kCbOffStat = kCbOffY + kCbStages * 2 * kCbStrBytes;   // ring of 64 x (lse2, delta)
constexpr int kCbSmemBytes = kCbOffStat + kCbStages * 128 * 4 + 1024;
// tensor-memory columns: row tile t holds S at 128 t and dP at 128 t + 64 (P and dS in their first 32
// columns), its accumulators at 256 + 128 t (dV) and 256 + 128 t + 64 (dK | dQ)
constexpr uint32_t kCbColBuf = 128, kCbColDP = 64, kCbColAcc = 256, kCbColAcc1 = 64;

struct CbCtl {
  uint64_t x_full, o_full;
  uint64_t y_full[kCbStages], y_empty[kCbStages], st_full[kCbStages];
  uint64_t s_full[2], dp_full[2], p_full[2], ds_full[2];
  uint32_t tmem_base;
  uint32_t abort_flag;
};

struct CbParams {
  const float *lse, *delta;      // [BH, Nq]
  __nv_bfloat16 *out0, *out1;    // dK/dV kernel: dV, dK [BH, Nc, 64];  dQ kernel: unused, dQ [BH, Nq, 64]
  int n_own, n_str;              // rows of the owned and of the streamed tensors (Nc, Nq | Nq, Nc)
  int Nq;
  float cs, scale;               // softmax scale * log2(e), softmax scale
  uint32_t* status;
};

// MODE 0: dK/dV (own = K, V; streamed = Q, dO).  MODE 1: dQ (own = Q, dO; streamed = K, V).
template <int MODE>
__global__ void __launch_bounds__(kCbThreads, 1)
cmp_bwd_kernel(const __grid_constant__ CUtensorMap map_x0, const __grid_constant__ CUtensorMap map_x1,
               const __grid_constant__ CUtensorMap map_y0, const __grid_constant__ CUtensorMap map_y1, const CbParams p) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ CbCtl ctl;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int own_tiles = (p.n_own + kCbOwnRows - 1) / kCbOwnRows;
  const int bh = blockIdx.x / own_tiles;
  const int r0 = (blockIdx.x % own_tiles) * kCbOwnRows;
  const int ntiles = (p.n_str + 63) / 64;
  const uint32_t sbase = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* sptr = smem_raw + (sbase - smem_u32(smem_raw));
  float* stats = reinterpret_cast<float*>(sptr + kCbOffStat);        // [stage][lse2 x64 | delta x64]

  if (threadIdx.x == 0) {
    ctl.abort_flag = 0;
    mbar_init(&ctl.x_full, 1);
    mbar_init(&ctl.o_full, 1);
    for (int s = 0; s < kCbStages; ++s) {
      mbar_init(&ctl.y_full[s], 1);
      mbar_init(&ctl.y_empty[s], 1);
      mbar_init(&ctl.st_full[s], 1);
    }
    for (int t = 0; t < 2; ++t) {
      mbar_init(&ctl.s_full[t], 1);
      mbar_init(&ctl.dp_full[t], 1);
      mbar_init(&ctl.p_full[t], 128);
      mbar_init(&ctl.ds_full[t], 128);
    }
    mbar_fence_init();
  }
  if (warp == 2) {
    tmem_alloc(&ctl.tmem_base, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = ctl.tmem_base;
  volatile uint32_t* abort_flag = &ctl.abort_flag;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      mbar_expect_tx(&ctl.x_full, 4 * kCbOwnBytes);
#pragma unroll
      for (int t = 0; t < 2; ++t) {
        tma_load_3d(sbase + kCbOffX + t * 2 * kCbOwnBytes, &map_x0, &ctl.x_full, 0, r0 + t * 128, bh);
        tma_load_3d(sbase + kCbOffX + t * 2 * kCbOwnBytes + kCbOwnBytes, &map_x1, &ctl.x_full, 0, r0 + t * 128, bh);
      }
      int issued = 0;
      for (int i = 0; i < ntiles; ++i) {
        const int s = i % kCbStages;
        if (!mbar_wait(&ctl.y_empty[s], ((i / kCbStages) & 1) ^ 1, abort_flag)) break;
        mbar_expect_tx(&ctl.y_full[s], 2 * kCbStrBytes);
        tma_load_3d(sbase + kCbOffY + s * 2 * kCbStrBytes, &map_y0, &ctl.y_full[s], 0, i * 64, bh);
        tma_load_3d(sbase + kCbOffY + s * 2 * kCbStrBytes + kCbStrBytes, &map_y1, &ctl.y_full[s], 0, i * 64, bh);
        issued = i + 1;
      }
      if (*abort_flag) {
        // give copies already in flight a bounded chance to land before the CTA's memory is released
        for (int i = max(0, issued - kCbStages); i < issued; ++i) {
          volatile uint32_t dummy = 0;
          mbar_wait(&ctl.y_full[i % kCbStages], (i / kCbStages) & 1, &dummy);
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer (converged warp, one elected lane issues)
    {
      const bool leader = elect_one_sync();
      constexpr uint32_t idesc_1 = umma_idesc_bf16(128, 64, 0, 0);    // both operands K-major
      constexpr uint32_t idesc_2 = umma_idesc_bf16(128, 64, 0, 1);    // B = streamed tile read as [rows][64]: N contiguous
      // descriptors are built once; a tile's descriptor is the base plus its byte offset / 16
      const uint64_t desc_x = umma_desc_sw128(sbase + kCbOffX), desc_y = umma_desc_sw128(sbase + kCbOffY);
      bool ok = mbar_wait_warp(&ctl.x_full, 0, abort_flag);
      // Per row tile t the MMAs come in two groups per streamed tile i:
      //   A(t,i): [P of tile i-1 stored]  dV += P^T dO (tile i-1)   then   S = X0 Y0^T (tile i)   -> s_full[t]
      //   B(t,i): [dS of tile i-1 stored] dK += dS^T Q (tile i-1)   then   dP = X1 Y1^T (tile i)  -> dp_full[t]
      // S and dP are overwritten by MMAs issued right behind the MMAs that read P and dS from the same
      // columns; the tensor pipe runs them in issue order.  The two row tiles are issued half a period
      // apart -  A(0,i)  B(1,i-1)  B(0,i)  A(1,i)  - so that one warpgroup is in its exponentials while the
      // other is in the multiply-and-pack pass.  (Measured equal to the in-step order A(0) A(1) B(0) B(1) at
      // 1000 views, 60 ms for both kernels: a warpgroup's passes take as long alone as side by side.)
      int st0 = 0, st1 = 0, st2 = 0;              // ring stages of tiles i, i-1, i-2
      uint32_t ph0 = 0;
      auto ydesc = [&](int st) { return desc_y + static_cast<uint64_t>(st * (2 * kCbStrBytes >> 4)); };
      const uint64_t x_t0 = desc_x, x_t1 = desc_x + static_cast<uint64_t>(2 * kCbOwnBytes >> 4);
      const uint32_t d0 = tmem + kCbColAcc, d1 = tmem + kCbColAcc + 128;
      const uint32_t b0 = tmem, b1 = tmem + kCbColBuf;
#pragma unroll 1
      for (int i = 0; i <= ntiles && ok; ++i) {
        const bool more = i < ntiles;
        const uint64_t y0 = ydesc(st0), y1 = ydesc(st1), y2 = ydesc(st2);
        // A(0,i)
        if (more) ok = mbar_wait_warp(&ctl.y_full[st0], ph0, abort_flag);
        if (ok && i >= 1) ok = mbar_wait_warp(&ctl.p_full[0], (i - 1) & 1, abort_flag);
        if (!ok) break;
        tc_fence_after();
        if (leader) {
          if (MODE == 0 && i >= 1) umma_ts_k4<128>(d0, b0, y1 + (kCbStrBytes >> 4), idesc_2, i > 1 ? 1u : 0u);
          if (more) {
            umma_ss_k4<2, 2>(b0, x_t0, y0, idesc_1, 0u);
            umma_commit(&ctl.s_full[0]);
          }
        }
        __syncwarp();
        // B(1,i-1)
        if (i >= 1) {
          if (i >= 2) {
            ok = mbar_wait_warp(&ctl.ds_full[1], i & 1, abort_flag);
            if (!ok) break;
          }
          tc_fence_after();
          if (leader) {
            if (i >= 2) umma_ts_k4<128>(d1 + kCbColAcc1, b1 + kCbColDP, y2, idesc_2, i > 2 ? 1u : 0u);
            umma_ss_k4<2, 2>(b1 + kCbColDP, x_t1 + (kCbOwnBytes >> 4), y1 + (kCbStrBytes >> 4), idesc_1, 0u);
            umma_commit(&ctl.dp_full[1]);
            if (i >= 2) umma_commit(&ctl.y_empty[st2]);
          }
          __syncwarp();
        }
        // B(0,i)
        if (i >= 1) {
          ok = mbar_wait_warp(&ctl.ds_full[0], (i - 1) & 1, abort_flag);
          if (!ok) break;
        }
        tc_fence_after();
        if (leader) {
          if (i >= 1) umma_ts_k4<128>(d0 + kCbColAcc1, b0 + kCbColDP, y1, idesc_2, i > 1 ? 1u : 0u);
          if (more) {
            umma_ss_k4<2, 2>(b0 + kCbColDP, x_t0 + (kCbOwnBytes >> 4), y0 + (kCbStrBytes >> 4), idesc_1, 0u);
            umma_commit(&ctl.dp_full[0]);
          }
        }
        __syncwarp();
        // A(1,i)
        if (i >= 1) {
          ok = mbar_wait_warp(&ctl.p_full[1], (i - 1) & 1, abort_flag);
          if (!ok) break;
        }
        tc_fence_after();
        if (leader) {
          if (MODE == 0 && i >= 1) umma_ts_k4<128>(d1, b1, y1 + (kCbStrBytes >> 4), idesc_2, i > 1 ? 1u : 0u);
          if (more) {
            umma_ss_k4<2, 2>(b1, x_t1, y0, idesc_1, 0u);
            umma_commit(&ctl.s_full[1]);
          }
        }
        __syncwarp();
        st2 = st1;
        st1 = st0;
        if (++st0 == kCbStages) { st0 = 0; ph0 ^= 1u; }
      }
      // the last dK of row tile 1: B(1, ntiles) without a next tile (after the shift st2 is the last tile's stage)
      if (ok) {
        ok = mbar_wait_warp(&ctl.ds_full[1], (ntiles - 1) & 1, abort_flag);
        if (ok) {
          tc_fence_after();
          if (leader) umma_ts_k4<128>(d1 + kCbColAcc1, b1 + kCbColDP, ydesc(st2), idesc_2, ntiles > 1 ? 1u : 0u);
          __syncwarp();
        }
      }
      if (leader) umma_commit(&ctl.o_full);
      __syncwarp();
      if (!ok) {
        volatile uint32_t dummy = 0;
        mbar_wait(&ctl.o_full, 0, &dummy);        // let issued MMAs drain before tensor memory is freed
      }
    }
  } else if (warp == 3) {
    // ------------------------------------------------------------------ lse / delta of the streamed rows (dK/dV kernel)
    if (MODE == 0) {
      for (int i = 0; i < ntiles; ++i) {
        const int s = i % kCbStages;
        if (!mbar_wait_warp(&ctl.y_empty[s], ((i / kCbStages) & 1) ^ 1, abort_flag)) break;
        float* dst = stats + s * 128;
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          const int q = i * 64 + h * 32 + lane;
          const bool in = q < p.n_str;
          // rows past the end: lse = +inf makes P exactly 0
          dst[h * 32 + lane] = in ? p.lse[static_cast<int64_t>(bh) * p.Nq + q] * 1.4426950408889634f : INFINITY;
          dst[64 + h * 32 + lane] = in ? p.delta[static_cast<int64_t>(bh) * p.Nq + q] : 0.f;
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&ctl.st_full[s]);
      }
    }
  } else if (warp >= 4) {
    // ------------------------------------------------------------------ compute, thread = owned row
    const int t = (warp - 4) >> 2;                  // row tile of this warpgroup
    const int quarter = warp & 3;
    const int row = r0 + t * 128 + quarter * 32 + lane;
    const uint32_t lane_base = tmem + (static_cast<uint32_t>(quarter * 32) << 16);
    const uint32_t t_s = lane_base + t * kCbColBuf, t_dp = t_s + kCbColDP;
    const float cs = p.cs;
    float my_lse2 = INFINITY, my_delta = 0.f;       // dQ kernel: this row's statistics
    if (MODE == 1 && row < p.n_own) {
      my_lse2 = p.lse[static_cast<int64_t>(bh) * p.Nq + row] * 1.4426950408889634f;
      my_delta = p.delta[static_cast<int64_t>(bh) * p.Nq + row];
    }
    bool ok = true;
    float pf[64];                                   // P of this row against the tile's 64 streamed rows
    for (int i = 0; i < ntiles; ++i) {
      const int s = i % kCbStages;
      if (!mbar_wait_warp(&ctl.s_full[t], i & 1, abort_flag)) { ok = false; break; }
      if (MODE == 0 && !mbar_wait_warp(&ctl.st_full[s], (i / kCbStages) & 1, abort_flag)) { ok = false; break; }
      tc_fence_after();
      const float4* st4 = reinterpret_cast<const float4*>(stats + s * 128);
      // pass 1: P = exp2(S c - lse), kept in registers; dK/dV kernel: bf16 P written over the low columns of S
      // (columns 8c..8c+7 were read with chunk c/2).  Tensor-memory loads run one chunk ahead.
      auto pass1 = [&](const uint32_t (&xs)[16], int c) {
        uint32_t pk[8];
#pragma unroll
        for (int g4 = 0; g4 < 4; ++g4) {
          float l4[4];
          if (MODE == 0) {
            const float4 a = st4[c * 4 + g4];         // same address in every lane: broadcast
            l4[0] = a.x; l4[1] = a.y; l4[2] = a.z; l4[3] = a.w;
          } else {
            l4[0] = l4[1] = l4[2] = l4[3] = my_lse2;
          }
#pragma unroll
          for (int e = 0; e < 4; ++e) pf[16 * c + 4 * g4 + e] = fast_exp2(fmaf(__uint_as_float(xs[4 * g4 + e]), cs, -l4[e]));
          if (MODE == 0) {
            pk[2 * g4] = pack_bf16(pf[16 * c + 4 * g4], pf[16 * c + 4 * g4 + 1]);
            pk[2 * g4 + 1] = pack_bf16(pf[16 * c + 4 * g4 + 2], pf[16 * c + 4 * g4 + 3]);
          }
        }
        if (MODE == 0) tmem_st8(t_s + c * 8, pk);
      };
      // pass 2: dS = P (dP - delta), written over the low columns of dP
      auto pass2 = [&](const uint32_t (&xd)[16], int c) {
        uint32_t dk[8];
#pragma unroll
        for (int g4 = 0; g4 < 4; ++g4) {
          float d4[4];
          if (MODE == 0) {
            const float4 b = st4[16 + c * 4 + g4];
            d4[0] = b.x; d4[1] = b.y; d4[2] = b.z; d4[3] = b.w;
          } else {
            d4[0] = d4[1] = d4[2] = d4[3] = my_delta;
          }
          float dv[4];
#pragma unroll
          for (int e = 0; e < 4; ++e) dv[e] = pf[16 * c + 4 * g4 + e] * (__uint_as_float(xd[4 * g4 + e]) - d4[e]);
          dk[2 * g4] = pack_bf16(dv[0], dv[1]);
          dk[2 * g4 + 1] = pack_bf16(dv[2], dv[3]);
        }
        tmem_st8(t_dp + c * 8, dk);
      };
      uint32_t xa[16], xb[16];
      tmem_ld16(t_s, xa);
      tmem_ld_wait();
      tmem_ld16(t_s + 16, xb);
      pass1(xa, 0);
      tmem_ld_wait();
      tmem_ld16(t_s + 32, xa);
      pass1(xb, 1);
      tmem_ld_wait();
      tmem_ld16(t_s + 48, xb);
      pass1(xa, 2);
      tmem_ld_wait();
      if (MODE == 1) {                                // S is in registers: the next S may overwrite it
        tc_fence_before();
        mbar_arrive(&ctl.p_full[t]);
      }
      pass1(xb, 3);
      if (MODE == 0) {
        tmem_st_wait();
        tc_fence_before();
        mbar_arrive(&ctl.p_full[t]);
      }
      if (!mbar_wait_warp(&ctl.dp_full[t], i & 1, abort_flag)) { ok = false; break; }
      tc_fence_after();
      tmem_ld16(t_dp, xa);
      tmem_ld_wait();
      tmem_ld16(t_dp + 16, xb);
      pass2(xa, 0);
      tmem_ld_wait();
      tmem_ld16(t_dp + 32, xa);
      pass2(xb, 1);
      tmem_ld_wait();
      tmem_ld16(t_dp + 48, xb);
      pass2(xa, 2);
      tmem_ld_wait();
      pass2(xb, 3);
      tmem_st_wait();
      tc_fence_before();
      mbar_arrive(&ctl.ds_full[t]);
    }
    // epilogue: this row tile's accumulators -> bf16 (dK and dQ carry the softmax scale)
    if (ok) ok = mbar_wait_warp(&ctl.o_full, 0, abort_flag);
    if (ok) {
      tc_fence_after();
#pragma unroll 1
      for (int a = (MODE == 0 ? 0 : 1); a < 2; ++a) {
        const float f = (a == 0) ? 1.f : p.scale;
        __nv_bfloat16* out = (a == 0 ? p.out0 : p.out1) + (static_cast<int64_t>(bh) * p.n_own + row) * 64;
#pragma unroll 1
        for (int hf = 0; hf < 2; ++hf) {
          uint32_t o[32];
          tmem_ld32(lane_base + kCbColAcc + t * 128 + a * kCbColAcc1 + hf * 32, o);
          tmem_ld_wait();
          if (row < p.n_own) {
            uint4* dst = reinterpret_cast<uint4*>(out + hf * 32);
#pragma unroll
            for (int v = 0; v < 4; ++v)
              dst[v] = make_uint4(pack_bf16(__uint_as_float(o[8 * v]) * f, __uint_as_float(o[8 * v + 1]) * f),
                                  pack_bf16(__uint_as_float(o[8 * v + 2]) * f, __uint_as_float(o[8 * v + 3]) * f),
                                  pack_bf16(__uint_as_float(o[8 * v + 4]) * f, __uint_as_float(o[8 * v + 5]) * f),
                                  pack_bf16(__uint_as_float(o[8 * v + 6]) * f, __uint_as_float(o[8 * v + 7]) * f));
          }
        }
      }
    }
    if (!ok) {
      *abort_flag = 1u;
      if (lane == 0) atomicOr(p.status, kStatusWaitTimeout);
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 2) tmem_dealloc(tmem, 512);
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
  const uintptr_t al = reinterpret_cast<uintptr_t>(q_c) | reinterpret_cast<uintptr_t>(k_c) | reinterpret_cast<uintptr_t>(v_c) |
                       reinterpret_cast<uintptr_t>(do_c) | reinterpret_cast<uintptr_t>(dq_c) |
                       reinterpret_cast<uintptr_t>(dk_c) | reinterpret_cast<uintptr_t>(dv_c);
  S3R_REQUIRE((al & 15) == 0, S3R_ERR_ALIGNMENT, "s3r_cmp_attn_bwd: tensors must be 16-byte aligned");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  int rc = s3r_delta(o_c, do_c, delta, static_cast<int64_t>(B) * H * Nq, d, stream);
  if (rc) return rc;
  const int BH = B * H;
  CUtensorMap mq128, mdo128, mk128, mv128, mq64, mdo64, mk64, mv64;
  {
    uint32_t box128[3] = {64, 128, 1}, box64[3] = {64, 64, 1};
    uint64_t dq_[3] = {64, static_cast<uint64_t>(Nq), static_cast<uint64_t>(BH)};
    uint64_t sq_[2] = {128, static_cast<uint64_t>(Nq) * 128};
    uint64_t dk_[3] = {64, static_cast<uint64_t>(Nc), static_cast<uint64_t>(BH)};
    uint64_t sk_[2] = {128, static_cast<uint64_t>(Nc) * 128};
    struct { CUtensorMap* m; const void* ptr; uint64_t* dims; uint64_t* strides; uint32_t* box; } maps[8] = {
        {&mq128, q_c, dq_, sq_, box128}, {&mdo128, do_c, dq_, sq_, box128}, {&mk128, k_c, dk_, sk_, box128},
        {&mv128, v_c, dk_, sk_, box128}, {&mq64, q_c, dq_, sq_, box64},     {&mdo64, do_c, dq_, sq_, box64},
        {&mk64, k_c, dk_, sk_, box64},   {&mv64, v_c, dk_, sk_, box64}};
    for (auto& e : maps) {
      rc = make_tensor_map(e.m, e.ptr, 3, e.dims, e.strides, e.box, CU_TENSOR_MAP_SWIZZLE_128B);
      if (rc) return rc;
    }
  }
  CbParams p;
  p.lse = lse; p.delta = delta;
  p.Nq = Nq;
  p.cs = scale * 1.4426950408889634f;
  p.scale = scale;
  p.status = device_status_ptr();
  S3R_REQUIRE(p.status != nullptr, S3R_ERR_DRIVER, "s3r_cmp_attn_bwd: could not resolve the device status word");
  S3R_CUDA(cudaFuncSetAttribute(cmp_bwd_kernel<0>, cudaFuncAttributeMaxDynamicSharedMemorySize, kCbSmemBytes));
  S3R_CUDA(cudaFuncSetAttribute(cmp_bwd_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, kCbSmemBytes));
  // dK, dV: own = K, V (Nc rows), streamed = Q, dO (Nq rows)
  p.out0 = static_cast<__nv_bfloat16*>(dv_c);
  p.out1 = static_cast<__nv_bfloat16*>(dk_c);
  p.n_own = Nc; p.n_str = Nq;
  const int64_t g0 = static_cast<int64_t>(BH) * ((Nc + kCbOwnRows - 1) / kCbOwnRows),
                g1 = static_cast<int64_t>(BH) * ((Nq + kCbOwnRows - 1) / kCbOwnRows);
  S3R_REQUIRE(g0 < (1ll << 31) && g1 < (1ll << 31), S3R_ERR_TOO_LARGE, "s3r_cmp_attn_bwd: grid too large");
  cmp_bwd_kernel<0><<<static_cast<unsigned>(g0), kCbThreads, kCbSmemBytes, st>>>(mk128, mv128, mq64, mdo64, p);
  // dQ: own = Q, dO (Nq rows), streamed = K, V (Nc rows)
  p.out0 = nullptr;
  p.out1 = static_cast<__nv_bfloat16*>(dq_c);
  p.n_own = Nq; p.n_str = Nc;
  cmp_bwd_kernel<1><<<static_cast<unsigned>(g1), kCbThreads, kCbSmemBytes, st>>>(mq128, mdo128, mk64, mv64, p);
  S3R_CUDA(cudaGetLastError());
  return 0;
}
