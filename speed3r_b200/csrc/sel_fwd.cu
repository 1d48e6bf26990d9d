// Selection branch, forward: block-sparse flash attention over the K key blocks each query block
// selected, with the gated merge of the two branches fused into the epilogue.
//
// Bound: gather bandwidth.  A query block of BS rows reads topk*BS key rows and value rows
// (2*topk*BS*128 B) for 4*BS*topk*BS*64 flop, i.e. BS flop per byte (16 at the reference's block
// size) against a machine balance of ~250 flop/B, so the kernel is organised around keeping many
// independent TMA gathers in flight, not around tensor-core throughput:
//   * one "group" of BS/16 warps owns one query block; a CTA holds 8 warps = 8/(BS/16) groups;
//   * each group has its own ring of STAGES shared-memory stages; lane 0 of the group's first warp
//     issues one TMA tiled copy per selected key block (K and V, 128-byte swizzle) and the copies
//     complete on the stage's mbarrier;
//   * each warp multiplies its 16 query rows with the stage's keys with mma.sync m16n8k16 (a
//     16-row query block is exactly one MMA M tile), keeps the online softmax in registers and
//     accumulates P*V;
//   * the epilogue normalises, optionally applies  y = g0*o_c + g1*o_s  and writes 128-byte rows.
// CTAs are ordered head-major so that the CTAs resident at one time gather from one head's K/V.
#include "common.cuh"

namespace s3r {

// Block size 16 (the reference's): the loop of one warp is a chain of dependent instructions, so the
// kernel runs faster with more warps per SM than with deeper rings: 12 warps with 2 stages of 32 keys
// (216 KB of shared memory) beat 8 warps with 3 stages by 20 % on B200.
#ifndef S3R_SEL16_WARPS
#define S3R_SEL16_WARPS 12
#endif
#ifndef S3R_SEL16_STAGES
#define S3R_SEL16_STAGES 2
#endif
#ifndef S3R_SEL16_STAGE_KEYS
#define S3R_SEL16_STAGE_KEYS 32
#endif

// Larger blocks (32, 64 tokens: not the reference's setting): the same lesson - two CTAs of 8 warps per SM
// (128 registers, 2-stage rings) run the 64-token kernel in 15.5 ms at 1000 views where one CTA with a 6-stage
// ring (171 registers) took 22.5 ms.
#ifndef S3R_SELBIG_STAGES
#define S3R_SELBIG_STAGES 2
#endif
#ifndef S3R_SELBIG_MIN_CTAS
#define S3R_SELBIG_MIN_CTAS 2
#endif

template <int BS>
struct SelCfg {
  static constexpr int kWarps = (BS == 16) ? S3R_SEL16_WARPS : 8;
  static constexpr int kWpg = BS / 16;                    // warps per query block
  static constexpr int kGroups = kWarps / kWpg;           // query blocks per CTA
  static constexpr int kStageKeys = BS < 32 ? S3R_SEL16_STAGE_KEYS : BS;    // keys per pipeline stage
  static constexpr int kBlkPerStage = kStageKeys / BS;
  static constexpr int kStageBytes = kStageKeys * 128 * 2;  // K tile + V tile
  static constexpr int kStages = (BS == 16) ? S3R_SEL16_STAGES : S3R_SELBIG_STAGES;
  static constexpr int kMinCtas = (BS == 16) ? 1 : S3R_SELBIG_MIN_CTAS;
  static constexpr int kQBytes = BS * 128;
  static constexpr int kMaxTopk = 64;
  static constexpr int kSmemBytes = kGroups * (kStages * kStageBytes + kQBytes) + 1024 /*alignment slack*/;
};

struct SelSmemCtl {
  uint64_t full[16][6];    // [group][stage]
  uint64_t empty[16][6];
  uint64_t qbar[16];
  int32_t list[16][64];    // valid key blocks of each group's query block, table order
  int32_t nvalid[16];
  uint32_t abort_flag;
};

struct SelParams {
  const int32_t* idx;
  __nv_bfloat16* o_s;
  float* lse_s;
  const __nv_bfloat16* gate;
  int64_t gsb, gsh, gst;
  const __nv_bfloat16* o_c;
  __nv_bfloat16* y;
  int B, H, Tq, Tk, Tc /*tokens per kv chunk*/, nqb, topk;
  float scale_log2e;
  uint32_t* status;
};

template <int BS>
__global__ void __launch_bounds__(SelCfg<BS>::kWarps * 32, SelCfg<BS>::kMinCtas)
sel_fwd_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
               const __grid_constant__ CUtensorMap map_v, const SelParams p) {
  using C = SelCfg<BS>;
  extern __shared__ uint8_t smem_raw[];
  __shared__ SelSmemCtl ctl;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int group = warp / C::kWpg, wig = warp % C::kWpg;
  const int g = lane >> 2, c = lane & 3;

  const int cta_per_bh = (p.nqb + C::kGroups - 1) / C::kGroups;
  const int bh = blockIdx.x / cta_per_bh;
  const int qb = (blockIdx.x % cta_per_bh) * C::kGroups + group;   // this group's query block
  const bool active = qb < p.nqb;

  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t grp_base = smem_base + group * (C::kStages * C::kStageBytes + C::kQBytes);
  const uint32_t q_smem = grp_base + C::kStages * C::kStageBytes;
  uint8_t* grp_ptr = smem_raw + (grp_base - smem_u32(smem_raw));

  if (threadIdx.x == 0) {
    ctl.abort_flag = 0;
    for (int gi = 0; gi < C::kGroups; ++gi) {
      for (int s = 0; s < C::kStages; ++s) {
        mbar_init(&ctl.full[gi][s], 1);
        mbar_init(&ctl.empty[gi][s], C::kWpg);
      }
      mbar_init(&ctl.qbar[gi], 1);
    }
    mbar_fence_init();
  }
  __syncthreads();
  volatile uint32_t* abort_flag = &ctl.abort_flag;

  int nvalid = 0;
  if (active && wig == 0) {
    // Compact the valid entries of this query block's row of the table, keeping table order.
    const int32_t* row = p.idx + (static_cast<int64_t>(bh) * p.nqb + qb) * p.topk;
    int base = 0;
    for (int r0 = 0; r0 < p.topk; r0 += 32) {
      int i = r0 + lane;
      int n = (i < p.topk) ? row[i] : -1;
      bool ok = (n >= 0) && (static_cast<int64_t>(n) * BS < p.Tk);
      uint32_t m = __ballot_sync(0xffffffffu, ok);
      if (ok) ctl.list[group][base + __popc(m & ((1u << lane) - 1u))] = n;
      base += __popc(m);
    }
    if (lane == 0) ctl.nvalid[group] = base;
  }
  if (C::kWpg == 1) __syncwarp();
  else asm volatile("bar.sync %0, %1;" ::"r"(1 + group), "r"(C::kWpg * 32) : "memory");
  if (active) nvalid = ctl.nvalid[group];
  const int nstages = (nvalid + C::kBlkPerStage - 1) / C::kBlkPerStage;
  const bool producer = active && (wig == 0) && (lane == 0);

  const bool chunked = p.Tc != p.Tk;
  // Called by the whole first warp of the group: lane 0 arms the barrier, then lanes 0..2*nb-1 issue one TMA
  // tiled copy each (even lanes a key block, odd lanes its value block), so the copies of a stage cost the
  // warp one instruction stream instead of 2*nb in a row.
  auto issue = [&](int it) {
    const int s = it % C::kStages;
    const int blk0 = it * C::kBlkPerStage;
    const int nb = min(C::kBlkPerStage, nvalid - blk0);
    uint64_t* bar = &ctl.full[group][s];
    if (lane == 0) mbar_expect_tx(bar, static_cast<uint32_t>(nb * BS * 128 * 2));
    __syncwarp();
    if (lane < 2 * nb) {
      const int j = lane >> 1;
      const bool values = (lane & 1) != 0;
      const int t0 = ctl.list[group][blk0 + j] * BS;
      int ch = 0, tl = t0;
      if (chunked) { ch = t0 / p.Tc; tl = t0 - ch * p.Tc; }
      uint8_t* dst = grp_ptr + s * C::kStageBytes + (values ? C::kStageKeys * 128 : 0) + j * BS * 128;
      tma_load_4d(dst, values ? &map_v : &map_k, bar, 0, tl, bh, ch);
    }
  };

  if (producer) {
    mbar_expect_tx(&ctl.qbar[group], C::kQBytes);
    tma_load_4d(grp_ptr + C::kStages * C::kStageBytes, &map_q, &ctl.qbar[group], 0, qb * BS, bh, 0);
  }
  if (active && wig == 0)
    for (int it = 0; it < min(C::kStages, nstages); ++it) issue(it);

  // ---- per-warp state -----------------------------------------------------------------------
  constexpr int NT = C::kStageKeys / 8;          // S n-tiles per stage
  uint32_t qf[4][4];
  float o_acc[8][4];
  float m_run[2] = {-INFINITY, -INFINITY};       // running max (log2 domain), rows g and g+8
  float l_run[2] = {0.f, 0.f};                   // this thread's partial row sums
#pragma unroll
  for (int i = 0; i < 8; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) o_acc[i][j] = 0.f;

  const bool tail_partial = (p.Tk % BS) != 0;
  const int last_blk = (p.Tk - 1) / BS;
  bool ok = true;
  if (active) {
    ok = mbar_wait_warp(&ctl.qbar[group], 0, abort_flag);
    if (ok) {
      const uint32_t row = wig * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
#pragma unroll
      for (int ks = 0; ks < 4; ++ks)
        ldsm_x4(qf[ks][0], qf[ks][1], qf[ks][2], qf[ks][3], q_smem + swz128(row, 2 * ks + (lane >> 4)));
    }
  }

  if (active && ok) {
    for (int it = 0; it < nstages; ++it) {
      const int s = it % C::kStages;
      const uint32_t ph = (it / C::kStages) & 1;
      if (!mbar_wait_warp(&ctl.full[group][s], ph, abort_flag)) { ok = false; break; }
      const uint32_t k_smem = grp_base + s * C::kStageBytes;
      const uint32_t v_smem = k_smem + C::kStageKeys * 128;
      const int blk0 = it * C::kBlkPerStage;
      const int nb = min(C::kBlkPerStage, nvalid - blk0);
      const int nkeys = nb * BS;                      // multiple of 16

      // S = Q K^T for this warp's 16 rows
      float sacc[NT][4];
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) { sacc[nt][0] = sacc[nt][1] = sacc[nt][2] = sacc[nt][3] = 0.f; }
#pragma unroll
      for (int np = 0; np < NT / 2; ++np) {
        if (np * 16 < nkeys) {
          const uint32_t krow = np * 16 + (lane & 7) + (lane >> 4) * 8;
#pragma unroll
          for (int ks = 0; ks < 4; ++ks) {
            uint32_t b0, b1, b2, b3;
            ldsm_x4(b0, b1, b2, b3, k_smem + swz128(krow, 2 * ks + ((lane >> 3) & 1)));
            mma_bf16(sacc[2 * np], qf[ks], b0, b1);
            mma_bf16(sacc[2 * np + 1], qf[ks], b2, b3);
          }
        }
      }
      // mask keys past the end of the sequence (last, partial key block) and absent blocks
      bool need_mask = nb < C::kBlkPerStage;
      if (tail_partial) {
        for (int j = 0; j < nb; ++j) need_mask |= (ctl.list[group][blk0 + j] == last_blk);
      }
      if (need_mask) {
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
          const int key0 = nt * 8 + 2 * c;                     // key index inside the stage
          const int blk = key0 / BS;
          bool v0 = false, v1 = false;
          if (blk < nb) {
            const int tok = ctl.list[group][blk0 + blk] * BS + (key0 - blk * BS);
            v0 = tok < p.Tk;
            v1 = tok + 1 < p.Tk;
          }
          if (!v0) { sacc[nt][0] = -INFINITY; sacc[nt][2] = -INFINITY; }
          if (!v1) { sacc[nt][1] = -INFINITY; sacc[nt][3] = -INFINITY; }
        }
      }
      // online softmax in the log2 domain: p = exp2(s*scale*log2e - m)
      float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) {
        mx[0] = fmax3(mx[0], sacc[nt][0], sacc[nt][1]);
        mx[1] = fmax3(mx[1], sacc[nt][2], sacc[nt][3]);
      }
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
        mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
      }
      float alpha[2], msafe[2];
      bool grew = false;
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        const float mn = fmaxf(m_run[r], mx[r] * p.scale_log2e);   // scale > 0 keeps the order
        grew |= (mn != m_run[r]);
        msafe[r] = (mn == -INFINITY) ? 0.f : mn;
        alpha[r] = fast_exp2(m_run[r] - msafe[r]);           // exp2(-inf) = 0 on the first stage
        m_run[r] = mn;
      }
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) {
        sacc[nt][0] = fast_exp2(fmaf(sacc[nt][0], p.scale_log2e, -msafe[0]));
        sacc[nt][1] = fast_exp2(fmaf(sacc[nt][1], p.scale_log2e, -msafe[0]));
        sacc[nt][2] = fast_exp2(fmaf(sacc[nt][2], p.scale_log2e, -msafe[1]));
        sacc[nt][3] = fast_exp2(fmaf(sacc[nt][3], p.scale_log2e, -msafe[1]));
      }
      // the running maxima stop moving after the first stages: rescale only when some row's did
      if (__any_sync(0xffffffffu, grew)) {
        l_run[0] *= alpha[0]; l_run[1] *= alpha[1];
#pragma unroll
        for (int dt = 0; dt < 8; ++dt) {
          o_acc[dt][0] *= alpha[0]; o_acc[dt][1] *= alpha[0];
          o_acc[dt][2] *= alpha[1]; o_acc[dt][3] *= alpha[1];
        }
      }
      {   // row sums as a tree: no 16-deep chain of dependent adds
        float t0s = 0.f, t1s = 0.f;
#pragma unroll
        for (int nt = 0; nt < NT; nt += 2) {
          t0s += (sacc[nt][0] + sacc[nt][1]) + (sacc[nt + 1][0] + sacc[nt + 1][1]);
          t1s += (sacc[nt][2] + sacc[nt][3]) + (sacc[nt + 1][2] + sacc[nt + 1][3]);
        }
        l_run[0] += t0s; l_run[1] += t1s;
      }
      // O += P V
#pragma unroll
      for (int kk = 0; kk < NT / 2; ++kk) {
        if (kk * 16 < nkeys) {
          uint32_t a[4];
          a[0] = pack_bf16(sacc[2 * kk][0], sacc[2 * kk][1]);
          a[1] = pack_bf16(sacc[2 * kk][2], sacc[2 * kk][3]);
          a[2] = pack_bf16(sacc[2 * kk + 1][0], sacc[2 * kk + 1][1]);
          a[3] = pack_bf16(sacc[2 * kk + 1][2], sacc[2 * kk + 1][3]);
          const uint32_t vrow = kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
#pragma unroll
          for (int dp = 0; dp < 4; ++dp) {
            uint32_t b0, b1, b2, b3;
            ldsm_x4_t(b0, b1, b2, b3, v_smem + swz128(vrow, 2 * dp + (lane >> 4)));
            mma_bf16(o_acc[2 * dp], a, b0, b1);
            mma_bf16(o_acc[2 * dp + 1], a, b2, b3);
          }
        }
      }
      // release the stage; the group's producer refills it once every warp of the group is done
      __syncwarp();
      if (lane == 0) mbar_arrive(&ctl.empty[group][s]);
      if (wig == 0 && it + C::kStages < nstages) {
        if (!mbar_wait_warp(&ctl.empty[group][s], ph, abort_flag)) ok = false;
        else issue(it + C::kStages);
      }
      if (!ok) break;
    }
  }

  if (active && !ok && lane == 0) atomicOr(p.status, kStatusWaitTimeout);

  // ---- epilogue -----------------------------------------------------------------------------
  if (active && ok) {
    float lsum[2], inv[2], lse[2];
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      float l = l_run[r];
      l += __shfl_xor_sync(0xffffffffu, l, 1);
      l += __shfl_xor_sync(0xffffffffu, l, 2);
      lsum[r] = l;
      inv[r] = (l > 0.f) ? 1.0f / l : 0.f;               // no valid key: o = 0, lse = -inf
      lse[r] = (l > 0.f) ? (m_run[r] + log2f(l)) * 0.6931471805599453f : -INFINITY;
    }
    const int row_in_blk = wig * 16 + g;                  // rows g and g+8 of this warp's 16
    const int t0 = qb * BS + row_in_blk, t1 = t0 + 8;
    if (p.lse_s && c == 0) {
      float* L = p.lse_s + static_cast<int64_t>(bh) * p.Tq;
      if (t0 < p.Tq) L[t0] = lse[0];
      if (t1 < p.Tq) L[t1] = lse[1];
    }
    // stage normalised o_s (bf16) in this warp's slice of the Q tile, then write 128-byte rows
    const uint32_t stage_rows0 = wig * 16;
    uint8_t* qtile = grp_ptr + C::kStages * C::kStageBytes;
    __syncwarp();
    if (p.o_s) {
#pragma unroll
      for (int dt = 0; dt < 8; ++dt) {
        *reinterpret_cast<uint32_t*>(qtile + swz128(stage_rows0 + g, dt) + 4 * c) =
            pack_bf16(o_acc[dt][0] * inv[0], o_acc[dt][1] * inv[0]);
        *reinterpret_cast<uint32_t*>(qtile + swz128(stage_rows0 + g + 8, dt) + 4 * c) =
            pack_bf16(o_acc[dt][2] * inv[1], o_acc[dt][3] * inv[1]);
      }
      __syncwarp();
      __nv_bfloat16* O = p.o_s + (static_cast<int64_t>(bh) * p.Tq + static_cast<int64_t>(qb) * BS) * 64;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int r = stage_rows0 + (lane >> 3) + 4 * i;
        if (qb * BS + r < p.Tq)
          *reinterpret_cast<uint4*>(O + r * 64 + (lane & 7) * 8) =
              *reinterpret_cast<const uint4*>(qtile + swz128(r, lane & 7));
      }
      __syncwarp();
    }
    if (p.y) {
      const int b = bh / p.H, h = bh % p.H;
      float g0[2] = {0.f, 0.f}, g1[2] = {0.f, 0.f};
      const __nv_bfloat16* G = p.gate + b * p.gsb + h * p.gsh;
      if (t0 < p.Tq) {
        uint32_t w = *reinterpret_cast<const uint32_t*>(G + t0 * p.gst);
        g0[0] = bf16_lo(w); g1[0] = bf16_hi(w);
      }
      if (t1 < p.Tq) {
        uint32_t w = *reinterpret_cast<const uint32_t*>(G + t1 * p.gst);
        g0[1] = bf16_lo(w); g1[1] = bf16_hi(w);
      }
      const __nv_bfloat16* OC = p.o_c + (static_cast<int64_t>(bh) * p.nqb + qb) * 64;
#pragma unroll
      for (int dt = 0; dt < 8; ++dt) {
        const uint32_t ocw = *reinterpret_cast<const uint32_t*>(OC + dt * 8 + 2 * c);
        const float c0 = bf16_lo(ocw), c1 = bf16_hi(ocw);
        *reinterpret_cast<uint32_t*>(qtile + swz128(stage_rows0 + g, dt) + 4 * c) =
            pack_bf16(g0[0] * c0 + g1[0] * o_acc[dt][0] * inv[0], g0[0] * c1 + g1[0] * o_acc[dt][1] * inv[0]);
        *reinterpret_cast<uint32_t*>(qtile + swz128(stage_rows0 + g + 8, dt) + 4 * c) =
            pack_bf16(g0[1] * c0 + g1[1] * o_acc[dt][2] * inv[1], g0[1] * c1 + g1[1] * o_acc[dt][3] * inv[1]);
      }
      __syncwarp();
      __nv_bfloat16* Y = p.y + (static_cast<int64_t>(b) * p.Tq + static_cast<int64_t>(qb) * BS) * (p.H * 64) + h * 64;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int r = stage_rows0 + (lane >> 3) + 4 * i;
        if (qb * BS + r < p.Tq)
          *reinterpret_cast<uint4*>(Y + static_cast<int64_t>(r) * (p.H * 64) + (lane & 7) * 8) =
              *reinterpret_cast<const uint4*>(qtile + swz128(r, lane & 7));
      }
    }
    (void)lsum;
  }
}

template <int BS>
static int launch_sel_fwd(const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv, const SelParams& p,
                          int BH, cudaStream_t st) {
  using C = SelCfg<BS>;
  static bool attr_set[64] = {};
  int dev = 0;
  S3R_CUDA(cudaGetDevice(&dev));
  if (dev >= 0 && dev < 64 && !attr_set[dev]) {
    S3R_CUDA(cudaFuncSetAttribute(sel_fwd_kernel<BS>, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmemBytes));
    attr_set[dev] = true;
  }
  const int cta_per_bh = (p.nqb + C::kGroups - 1) / C::kGroups;
  const int64_t grid = static_cast<int64_t>(BH) * cta_per_bh;
  S3R_REQUIRE(grid < (1ll << 31), S3R_ERR_TOO_LARGE, "s3r_sel_attn_fwd: grid of %lld CTAs is too large", (long long)grid);
  sel_fwd_kernel<BS><<<static_cast<unsigned>(grid), C::kWarps * 32, C::kSmemBytes, st>>>(mq, mk, mv, p);
  S3R_CUDA(cudaGetLastError());
  return 0;
}

}  // namespace s3r

using namespace s3r;

extern "C" int s3r_sel_attn_fwd(const void* q, const void* k, const void* v, int kv_chunks, int64_t kv_chunk_stride,
                                const int32_t* idx, void* o_s, float* lse_s, const void* gate,
                                int64_t gate_stride_b, int64_t gate_stride_h, int64_t gate_stride_t, const void* o_c,
                                void* y, int B, int H, int Tq, int Tk, int d, int block, int topk, float scale,
                                void* stream) {
  S3R_REQUIRE(q && k && v && idx, S3R_ERR_NULL, "s3r_sel_attn_fwd: q, k, v and idx are required");
  S3R_REQUIRE(o_s || y, S3R_ERR_NULL, "s3r_sel_attn_fwd: at least one of o_s and y must be given");
  S3R_REQUIRE((gate != nullptr) == (y != nullptr) && (o_c != nullptr) == (y != nullptr), S3R_ERR_NULL,
              "s3r_sel_attn_fwd: gate, o_c and y must be given together");
  S3R_REQUIRE(B > 0 && H > 0 && Tq > 0 && Tk > 0 && topk > 0 && kv_chunks > 0, S3R_ERR_SHAPE,
              "s3r_sel_attn_fwd: sizes must be positive (B=%d H=%d Tq=%d Tk=%d topk=%d chunks=%d)", B, H, Tq, Tk, topk,
              kv_chunks);
  S3R_REQUIRE(d == 64, S3R_ERR_UNSUPPORTED, "s3r_sel_attn_fwd: head_dim %d not supported (64 only)", d);
  S3R_REQUIRE(block == 16 || block == 32 || block == 64, S3R_ERR_UNSUPPORTED,
              "s3r_sel_attn_fwd: block %d not supported (16, 32, 64)", block);
  S3R_REQUIRE(topk <= 64, S3R_ERR_UNSUPPORTED, "s3r_sel_attn_fwd: topk %d exceeds 64", topk);
  S3R_REQUIRE(scale > 0.f, S3R_ERR_UNSUPPORTED, "s3r_sel_attn_fwd: softmax scale must be positive");
  S3R_REQUIRE(Tk % kv_chunks == 0 && (kv_chunks == 1 || (Tk / kv_chunks) % block == 0), S3R_ERR_SHAPE,
              "s3r_sel_attn_fwd: Tk=%d must split into %d chunks of whole blocks", Tk, kv_chunks);
  const uintptr_t al = reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(k) | reinterpret_cast<uintptr_t>(v) |
                       reinterpret_cast<uintptr_t>(o_s) | reinterpret_cast<uintptr_t>(y) |
                       reinterpret_cast<uintptr_t>(o_c);
  S3R_REQUIRE((al & 15) == 0 && (kv_chunk_stride % 8) == 0, S3R_ERR_ALIGNMENT,
              "s3r_sel_attn_fwd: tensors must be 16-byte aligned");
  S3R_REQUIRE(!gate || ((reinterpret_cast<uintptr_t>(gate) & 3) == 0 && gate_stride_b % 2 == 0 &&
                        gate_stride_h % 2 == 0 && gate_stride_t % 2 == 0),
              S3R_ERR_ALIGNMENT, "s3r_sel_attn_fwd: gate pairs must be 4-byte aligned");

  const int BH = B * H;
  const int Tc = Tk / kv_chunks;
  CUtensorMap mq, mk, mv;
  {
    uint64_t dims[4] = {64, static_cast<uint64_t>(Tq), static_cast<uint64_t>(BH), 1};
    uint64_t strides[3] = {128, static_cast<uint64_t>(Tq) * 128, static_cast<uint64_t>(Tq) * 128 * BH};
    uint32_t box[4] = {64, static_cast<uint32_t>(block), 1, 1};
    int rc = make_tensor_map(&mq, q, 4, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc) return rc;
  }
  {
    uint64_t dims[4] = {64, static_cast<uint64_t>(Tc), static_cast<uint64_t>(BH), static_cast<uint64_t>(kv_chunks)};
    uint64_t cs = kv_chunks > 1 ? static_cast<uint64_t>(kv_chunk_stride) * 2 : static_cast<uint64_t>(Tc) * 128 * BH;
    uint64_t strides[3] = {128, static_cast<uint64_t>(Tc) * 128, cs};
    uint32_t box[4] = {64, static_cast<uint32_t>(block), 1, 1};
    int rc = make_tensor_map(&mk, k, 4, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc) return rc;
    rc = make_tensor_map(&mv, v, 4, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc) return rc;
  }
  SelParams p;
  p.idx = idx;
  p.o_s = static_cast<__nv_bfloat16*>(o_s);
  p.lse_s = lse_s;
  p.gate = static_cast<const __nv_bfloat16*>(gate);
  p.gsb = gate_stride_b; p.gsh = gate_stride_h; p.gst = gate_stride_t;
  p.o_c = static_cast<const __nv_bfloat16*>(o_c);
  p.y = static_cast<__nv_bfloat16*>(y);
  p.B = B; p.H = H; p.Tq = Tq; p.Tk = Tk; p.Tc = Tc;
  p.nqb = (Tq + block - 1) / block;
  p.topk = topk;
  p.scale_log2e = scale * 1.4426950408889634f;
  p.status = device_status_ptr();
  S3R_REQUIRE(p.status != nullptr, S3R_ERR_DRIVER, "s3r_sel_attn_fwd: could not resolve the device status word");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (block == 16) return launch_sel_fwd<16>(mq, mk, mv, p, BH, st);
  if (block == 32) return launch_sel_fwd<32>(mq, mk, mv, p, BH, st);
  return launch_sel_fwd<64>(mq, mk, mv, p, BH, st);
}
