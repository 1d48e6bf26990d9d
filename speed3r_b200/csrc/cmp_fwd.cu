// Compression branch, forward: dense attention of the pooled queries over the pooled keys with
// the per-row top-k of the RAW logits fused in (the row's top-k columns are the key blocks the
// selection branch will read).
//
// Bound: tensor cores in principle (4*Nq*Nc*64 flop per head), with the softmax exponentials and
// the top-k threshold tests as the practical co-limit, so the MMAs are taken off the issue path:
//   warp 0  (1 lane)  TMA producer: Q tile pair once, then K and V tiles of 128 keys into rings
//   warp 1  (1 lane)  tcgen05.mma issuer: S = Q K^T (M=128,N=128) and O += P V (M=128,N=64)
//   warp 2            tensor-memory allocator
//   warps 4-7, 8-11   two softmax warpgroups, one per 128-row query tile; thread = row
// A CTA owns 256 query rows (two tiles sharing every K/V tile).  Tensor memory: S_A, S_B (128
// fp32 columns each), O_A, O_B (64 each).  P (bf16) is written back over the S columns and fed to
// the second MMA straight from tensor memory.
//
// Online softmax with a lazily updated maximum: the exponent offset only moves when the running
// maximum grows by more than 2^8, and only then is O rescaled in tensor memory, by the softmax
// threads themselves (each owns one TMEM lane).
//
// Top-k.  Per row, shared memory holds the best 32 entries (key(score), column) SORTED across the
// lanes of the row's warp (slot l belongs to lane l), plus a small pending buffer.  A thread tests
// 16-column chunks of its row against the row's threshold (the topk-th kept score) and appends
// hits to the pending buffer on its own (no warp cooperation); when a buffer is full the warp
// merges it into the sorted list in one pass (merge ranks from one ballot per pending entry) and
// the threshold rises.  Ties on the score keep the smaller column first because columns arrive in
// ascending order.  Slots start empty (key 0), which decodes to column Nc-1, the reference's padding.
#include "common.cuh"

namespace s3r {

constexpr int kCmpThreads = 384;
constexpr int kTileBytes = 128 * 128;        // 128 rows x 64 bf16
constexpr int kListBytes = 256 * 32 * 8;     // 256 rows x 32 sorted entries x (key, column)
constexpr int kPend = 8;                     // pending entries per row
constexpr int kPendBytes = 256 * kPend * 8;
constexpr int kStages = 3;
constexpr int kOffQ = 0;
constexpr int kOffK = 2 * kTileBytes;
constexpr int kOffV = kOffK + kStages * kTileBytes;
constexpr int kOffL = kOffV + kStages * kTileBytes;
constexpr int kOffPend = kOffL + kListBytes;
constexpr int kCmpSmemBytes = kOffPend + kPendBytes + 1024;

struct CmpCtl {
  uint64_t q_full, o_full;
  uint64_t k_full[4], k_empty[4], v_full[4], v_empty[4];
  uint64_t s_full[2], p_full[2];
  uint32_t tmem_base;
  uint32_t abort_flag;
};

struct CmpParams {
  __nv_bfloat16* o;
  float* lse;
  int32_t* idx;
  int Nq, Nc, topk, flags;
  float c_scale;        // softmax scale * log2(e)
  uint32_t* status;
};

__device__ __forceinline__ float key_to_float(uint32_t key) {
  if (key == 0u) return -INFINITY;            // empty slot: everything qualifies
  const uint32_t b = (key & 0x80000000u) ? (key ^ 0x80000000u) : ~key;
  return __uint_as_float(b);
}

// Thread-local: append this thread's hits among x[e_start..15] (first column col0) to its row's
// pending buffer.  Stops at the first hit that does not fit and leaves e_start there; e_start = 16
// when the chunk is finished.
__device__ __forceinline__ void topk_append16(const uint32_t* x, int col0, int nvalid, float thr, uint2* my_pend,
                                              int& cnt, int& e_start) {
  bool full = false;
#pragma unroll
  for (int e = 0; e < 16; ++e) {
    const float v = __uint_as_float(x[e]);
    if (!full && e >= e_start && e < nvalid && v >= thr) {
      if (cnt < kPend) {
        my_pend[cnt] = make_uint2(sortable_key(v), static_cast<uint32_t>(col0 + e));
        ++cnt;
      } else {
        full = true;
        e_start = e;
      }
    }
  }
  if (!full) e_start = 16;
}

// Warp-cooperative merge of the m pending entries of one row into its sorted list.  Old entry l
// moves to l + (#pending better than it); pending j lands at (#old >= it) + (#pending better than
// it).  An old entry wins a tie on the key (its column is smaller); pending entries tie-break on
// the column.  Returns the key in slot topk-1 afterwards (0 while fewer than topk real entries).
__device__ __forceinline__ uint32_t topk_flush_row(uint2* list_row, const uint2* pend_row, int m, int lane, int topk) {
  __syncwarp();
  const uint2 old = list_row[lane];
  const uint2 mine = (lane < m) ? pend_row[lane] : make_uint2(0u, 0u);
  int shift = 0, myrank = 0;
#pragma unroll
  for (int j = 0; j < kPend; ++j) {
    if (j < m) {                                     // warp-uniform
      const uint2 pj = pend_row[j];
      const bool pb = pj.x > old.x;
      shift += pb ? 1 : 0;
      const int nge = __popc(__ballot_sync(0xffffffffu, !pb));
      const bool jb = (pj.x > mine.x) || (pj.x == mine.x && pj.y < mine.y);
      myrank += (jb ? 1 : 0) + (lane == j ? nge : 0);
    }
  }
  __syncwarp();
  if (lane + shift < 32) list_row[lane + shift] = old;
  if (lane < m && myrank < 32) list_row[myrank] = mine;
  __syncwarp();
  return list_row[topk - 1].x;
}

__global__ void __launch_bounds__(kCmpThreads, 1)
cmp_fwd_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
               const __grid_constant__ CUtensorMap map_v, const CmpParams p) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ CmpCtl ctl;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tiles_per_bh = (p.Nq + 255) / 256;
  const int bh = blockIdx.x / tiles_per_bh;
  const int q0 = (blockIdx.x % tiles_per_bh) * 256;
  const int ntiles = (p.Nc + 127) / 128;

  const uint32_t sbase = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* sptr = smem_raw + (sbase - smem_u32(smem_raw));
  uint2* lists = reinterpret_cast<uint2*>(sptr + kOffL);
  uint2* pends = reinterpret_cast<uint2*>(sptr + kOffPend);

  if (threadIdx.x == 0) {
    ctl.abort_flag = 0;
    mbar_init(&ctl.q_full, 1);
    mbar_init(&ctl.o_full, 1);
    for (int s = 0; s < 4; ++s) {
      mbar_init(&ctl.k_full[s], 1);
      mbar_init(&ctl.k_empty[s], 1);
      mbar_init(&ctl.v_full[s], 1);
      mbar_init(&ctl.v_empty[s], 1);
    }
    for (int t = 0; t < 2; ++t) {
      mbar_init(&ctl.s_full[t], 1);
      mbar_init(&ctl.p_full[t], 128);
    }
    mbar_fence_init();
  }
  if (warp == 2) {
    tmem_alloc(&ctl.tmem_base, 512);
    tmem_relinquish();
  }
  for (int i = threadIdx.x; i < 256 * 32; i += kCmpThreads) lists[i] = make_uint2(0u, 0u);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = ctl.tmem_base;
  volatile uint32_t* abort_flag = &ctl.abort_flag;

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      mbar_expect_tx(&ctl.q_full, 2 * kTileBytes);
      tma_load_3d(sbase + kOffQ, &map_q, &ctl.q_full, 0, q0, bh);
      tma_load_3d(sbase + kOffQ + kTileBytes, &map_q, &ctl.q_full, 0, q0 + 128, bh);
      int issued = 0;
      for (int j = 0; j < ntiles; ++j) {
        const int s = j % kStages;
        const uint32_t ph = (j / kStages) & 1;
        if (!mbar_wait(&ctl.k_empty[s], ph ^ 1, abort_flag)) break;
        mbar_expect_tx(&ctl.k_full[s], kTileBytes);
        tma_load_3d(sbase + kOffK + s * kTileBytes, &map_k, &ctl.k_full[s], 0, j * 128, bh);
        if (!mbar_wait(&ctl.v_empty[s], ph ^ 1, abort_flag)) { issued = j + 1; break; }   // K of tile j is in flight
        mbar_expect_tx(&ctl.v_full[s], kTileBytes);
        tma_load_3d(sbase + kOffV + s * kTileBytes, &map_v, &ctl.v_full[s], 0, j * 128, bh);
        issued = j + 1;
      }
      if (*abort_flag) {
        // give copies already in flight a bounded chance to land before the CTA's memory is released
        for (int j = max(0, issued - kStages); j < issued; ++j) {
          volatile uint32_t dummy = 0;
          mbar_wait(&ctl.k_full[j % kStages], (j / kStages) & 1, &dummy);
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc_qk = umma_idesc_bf16(128, 128, 0, 0);
      constexpr uint32_t idesc_pv = umma_idesc_bf16(128, 64, 0, 1);   // V tile is [keys][d]: N contiguous
      auto issue_qk = [&](int t, int s) {
#pragma unroll
        for (int ks = 0; ks < 4; ++ks)
          umma_ss(tmem + t * 128, umma_desc_sw128(sbase + kOffQ + t * kTileBytes + ks * 32),
                  umma_desc_sw128(sbase + kOffK + s * kTileBytes + ks * 32), idesc_qk, ks > 0);
      };
      auto issue_pv = [&](int t, int s, bool acc) {
#pragma unroll
        for (int ks = 0; ks < 8; ++ks)
          umma_ts(tmem + 256 + t * 64, tmem + t * 128 + ks * 8, umma_desc_sw128(sbase + kOffV + s * kTileBytes + ks * 2048),
                  idesc_pv, (acc || ks > 0) ? 1u : 0u);
      };
      bool ok = mbar_wait(&ctl.q_full, 0, abort_flag) && mbar_wait(&ctl.k_full[0], 0, abort_flag);
      if (ok) {
        tc_fence_after();
        issue_qk(0, 0);
        umma_commit(&ctl.s_full[0]);
        issue_qk(1, 0);
        umma_commit(&ctl.s_full[1]);
        umma_commit(&ctl.k_empty[0]);
        for (int j = 0; j < ntiles && ok; ++j) {
          const int s = j % kStages;
          const bool nxt = j + 1 < ntiles;
          const int sn = (j + 1) % kStages;
          ok = mbar_wait(&ctl.v_full[s], (j / kStages) & 1, abort_flag);
          if (ok && nxt) ok = mbar_wait(&ctl.k_full[sn], ((j + 1) / kStages) & 1, abort_flag);
          for (int t = 0; t < 2 && ok; ++t) {
            ok = mbar_wait(&ctl.p_full[t], j & 1, abort_flag);
            if (!ok) break;
            tc_fence_after();
            issue_pv(t, s, j > 0);
            if (t == 1) umma_commit(&ctl.v_empty[s]);
            if (nxt) {
              issue_qk(t, sn);
              umma_commit(&ctl.s_full[t]);
              if (t == 1) umma_commit(&ctl.k_empty[sn]);
            }
          }
        }
      }
      umma_commit(&ctl.o_full);
      if (!ok) {
        volatile uint32_t dummy = 0;
        mbar_wait(&ctl.o_full, 0, &dummy);     // let issued MMAs drain before tensor memory is freed
      }
    }
  } else if (warp >= 4) {
    // ------------------------------------------------------------------ softmax + top-k, thread = row
    const int t = (warp - 4) >> 2;
    const int quarter = warp & 3;
    const int row_local = t * 128 + quarter * 32 + lane;      // 0..255 inside the CTA
    const int grow = q0 + row_local;
    uint2* warp_lists = lists + (t * 128 + quarter * 32) * 32;
    uint2* warp_pend = pends + (t * 128 + quarter * 32) * kPend;
    uint2* my_pend = warp_pend + lane * kPend;
    const uint32_t t_s = tmem + (static_cast<uint32_t>(quarter * 32) << 16) + t * 128;
    const uint32_t t_o = tmem + (static_cast<uint32_t>(quarter * 32) << 16) + 256 + t * 64;
    const float cs = p.c_scale;
    float m_used = -INFINITY, l = 0.f, thr = -INFINITY;
    int cnt = 0;
    bool ok = true;

    // merge the pending buffers of the rows in `mask` into their sorted lists
    auto flush_rows = [&](uint32_t mask) {
      while (mask) {
        const int src = __ffs(mask) - 1;
        mask &= mask - 1;
        const int m = __shfl_sync(0xffffffffu, cnt, src);
        const uint32_t kth = topk_flush_row(warp_lists + src * 32, warp_pend + src * kPend, m, lane, p.topk);
        if (lane == src) {
          cnt = 0;
          thr = key_to_float(kth);
        }
      }
    };

    for (int j = 0; j < ntiles; ++j) {
      if (!mbar_wait_warp(&ctl.s_full[t], j & 1, abort_flag)) { ok = false; break; }
      tc_fence_after();
      const int col0 = j * 128;
      const bool tail = (col0 + 128 > p.Nc);

      // pass 1: row maximum of the raw logits + top-k candidates
      float rmax = -INFINITY;
#pragma unroll 1
      for (int c4 = 0; c4 < 4; ++c4) {
        uint32_t x[32];
        tmem_ld32(t_s + c4 * 32, x);
        tmem_ld_wait();
        int nvalid = 32;
        if (tail) {
          nvalid = min(32, max(0, p.Nc - (col0 + c4 * 32)));
#pragma unroll
          for (int i = 0; i < 32; ++i)
            if (i >= nvalid) x[i] = 0xff800000u;   // -inf
        }
#pragma unroll
        for (int hf = 0; hf < 2; ++hf) {
          float cm = __uint_as_float(x[hf * 16]);
#pragma unroll
          for (int i = 1; i < 16; ++i) cm = fmaxf(cm, __uint_as_float(x[hf * 16 + i]));
          rmax = fmaxf(rmax, cm);
          const bool hot = (cm >= thr);
          if (!(p.flags & 2) && __any_sync(0xffffffffu, hot)) {
            int e_start = hot ? 0 : 16;
            while (true) {
              topk_append16(x + hf * 16, col0 + c4 * 32 + hf * 16, nvalid - hf * 16, thr, my_pend, cnt, e_start);
              const uint32_t fullmask = __ballot_sync(0xffffffffu, e_start < 16);
              if (!fullmask) break;
              flush_rows(fullmask);
            }
          }
        }
      }

      // exponent offset; rescale O only when the maximum moved by more than 2^8
      const float mt = rmax * cs;
      float factor = 1.f;
      bool need = false;
      if (j == 0) {
        m_used = mt;
      } else if (mt > m_used + 8.f) {
        factor = fast_exp2(m_used - mt);
        m_used = mt;
        l *= factor;
        need = true;
      }
      if (j > 0 && __any_sync(0xffffffffu, need)) {
#pragma unroll 1
        for (int hf = 0; hf < 2; ++hf) {
          uint32_t o[32];
          tmem_ld32(t_o + hf * 32, o);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * factor);
          tmem_st32(t_o + hf * 32, o);
        }
        tmem_st_wait();
      }

      // pass 2: P = exp2(s*c - m), row sum, bf16 P back over the S columns
      float ls[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll 1
      for (int c4 = 0; c4 < 4; ++c4) {
        uint32_t x[32];
        tmem_ld32(t_s + c4 * 32, x);
        tmem_ld_wait();
        if (tail) {
          const int nvalid = min(32, max(0, p.Nc - (col0 + c4 * 32)));
#pragma unroll
          for (int i = 0; i < 32; ++i)
            if (i >= nvalid) x[i] = 0xff800000u;
        }
        uint32_t pk[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          const float p0 = fast_exp2(fmaf(__uint_as_float(x[2 * i]), cs, -m_used));
          const float p1 = fast_exp2(fmaf(__uint_as_float(x[2 * i + 1]), cs, -m_used));
          ls[i & 3] += p0 + p1;
          pk[i] = pack_bf16(p0, p1);
        }
        tmem_st16(t_s + c4 * 16, pk);
      }
      l += (ls[0] + ls[1]) + (ls[2] + ls[3]);
      tmem_st_wait();
      tc_fence_before();
      mbar_arrive(&ctl.p_full[t]);
    }

    // epilogue: O / l, lse, and the sorted index rows
    if (ok) ok = mbar_wait_warp(&ctl.o_full, 0, abort_flag);
    if (ok) {
      tc_fence_after();
      const float inv = 1.f / l;
      if (grow < p.Nq) p.lse[static_cast<int64_t>(bh) * p.Nq + grow] = (m_used + log2f(l)) * 0.6931471805599453f;
#pragma unroll 1
      for (int hf = 0; hf < 2; ++hf) {
        uint32_t o[32];
        tmem_ld32(t_o + hf * 32, o);
        tmem_ld_wait();
        if (grow < p.Nq) {
          uint4* dst = reinterpret_cast<uint4*>(p.o + (static_cast<int64_t>(bh) * p.Nq + grow) * 64 + hf * 32);
#pragma unroll
          for (int i = 0; i < 4; ++i)
            dst[i] = make_uint4(pack_bf16(__uint_as_float(o[8 * i]) * inv, __uint_as_float(o[8 * i + 1]) * inv),
                                pack_bf16(__uint_as_float(o[8 * i + 2]) * inv, __uint_as_float(o[8 * i + 3]) * inv),
                                pack_bf16(__uint_as_float(o[8 * i + 4]) * inv, __uint_as_float(o[8 * i + 5]) * inv),
                                pack_bf16(__uint_as_float(o[8 * i + 6]) * inv, __uint_as_float(o[8 * i + 7]) * inv));
        }
      }
      flush_rows(__ballot_sync(0xffffffffu, cnt > 0));
      __syncwarp();
      const int wrow0 = q0 + t * 128 + quarter * 32;
      // the lists are sorted: slot l is rank l; an empty slot decodes to column Nc-1
      for (int r = 0; r < 32 && wrow0 + r < p.Nq; ++r) {
        const uint2 ent = warp_lists[r * 32 + lane];
        if (lane < p.topk)
          p.idx[(static_cast<int64_t>(bh) * p.Nq + wrow0 + r) * p.topk + lane] =
              (ent.x == 0u) ? (p.Nc - 1) : static_cast<int32_t>(ent.y);
      }
    }
    if (!ok && lane == 0) atomicOr(p.status, kStatusWaitTimeout);
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 2) tmem_dealloc(tmem, 512);
}

}  // namespace s3r

using namespace s3r;

// Profiling switch: bit 1 set = skip the top-k scan (idx is then meaningless).  0 by default.
static int g_cmp_variant = 0;
extern "C" void s3r_debug_set_cmp_variant(int v) { g_cmp_variant = v; }

extern "C" int s3r_cmp_attn_topk_fwd(const void* q_c, const void* k_c, const void* v_c, void* o_c, float* lse,
                                     int32_t* idx, int B, int H, int Nq, int Nc, int d, int topk, float scale,
                                     void* stream) {
  S3R_REQUIRE(q_c && k_c && v_c && o_c && lse && idx, S3R_ERR_NULL, "s3r_cmp_attn_topk_fwd: NULL pointer");
  S3R_REQUIRE(B > 0 && H > 0 && Nq > 0 && Nc > 0, S3R_ERR_SHAPE,
              "s3r_cmp_attn_topk_fwd: sizes must be positive (B=%d H=%d Nq=%d Nc=%d)", B, H, Nq, Nc);
  S3R_REQUIRE(d == 64, S3R_ERR_UNSUPPORTED, "s3r_cmp_attn_topk_fwd: head_dim %d not supported (64 only)", d);
  S3R_REQUIRE(topk >= 1 && topk <= 32, S3R_ERR_UNSUPPORTED, "s3r_cmp_attn_topk_fwd: topk %d not in [1,32]", topk);
  S3R_REQUIRE(scale > 0.f, S3R_ERR_UNSUPPORTED, "s3r_cmp_attn_topk_fwd: softmax scale must be positive");
  const uintptr_t al = reinterpret_cast<uintptr_t>(q_c) | reinterpret_cast<uintptr_t>(k_c) |
                       reinterpret_cast<uintptr_t>(v_c) | reinterpret_cast<uintptr_t>(o_c);
  S3R_REQUIRE((al & 15) == 0, S3R_ERR_ALIGNMENT, "s3r_cmp_attn_topk_fwd: tensors must be 16-byte aligned");
  const int BH = B * H;
  CUtensorMap mq, mk, mv;
  uint32_t box[3] = {64, 128, 1};
  {
    uint64_t dims[3] = {64, static_cast<uint64_t>(Nq), static_cast<uint64_t>(BH)};
    uint64_t strides[2] = {128, static_cast<uint64_t>(Nq) * 128};
    int rc = make_tensor_map(&mq, q_c, 3, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc) return rc;
  }
  {
    uint64_t dims[3] = {64, static_cast<uint64_t>(Nc), static_cast<uint64_t>(BH)};
    uint64_t strides[2] = {128, static_cast<uint64_t>(Nc) * 128};
    int rc = make_tensor_map(&mk, k_c, 3, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc) return rc;
    rc = make_tensor_map(&mv, v_c, 3, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc) return rc;
  }
  CmpParams p;
  p.o = static_cast<__nv_bfloat16*>(o_c);
  p.lse = lse;
  p.idx = idx;
  p.Nq = Nq; p.Nc = Nc; p.topk = topk; p.flags = g_cmp_variant;
  p.c_scale = scale * 1.4426950408889634f;
  p.status = device_status_ptr();
  S3R_REQUIRE(p.status != nullptr, S3R_ERR_DRIVER, "s3r_cmp_attn_topk_fwd: could not resolve the device status word");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  static bool attr_set[64] = {};
  int dev = 0;
  S3R_CUDA(cudaGetDevice(&dev));
  if (dev >= 0 && dev < 64 && !attr_set[dev]) {
    S3R_CUDA(cudaFuncSetAttribute(cmp_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kCmpSmemBytes));
    attr_set[dev] = true;
  }
  const int64_t grid = static_cast<int64_t>(BH) * ((Nq + 255) / 256);
  S3R_REQUIRE(grid < (1ll << 31), S3R_ERR_TOO_LARGE, "s3r_cmp_attn_topk_fwd: grid too large");
  cmp_fwd_kernel<<<static_cast<unsigned>(grid), kCmpThreads, kCmpSmemBytes, st>>>(mq, mk, mv, p);
  S3R_CUDA(cudaGetLastError());
  return 0;
}
