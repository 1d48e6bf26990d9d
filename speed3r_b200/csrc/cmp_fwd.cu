// Compression branch, forward: dense attention of the pooled queries over the pooled keys with
// the per-row top-k of the RAW logits fused in (the row's top-k columns are the key blocks the
// selection branch will read).
//
// Bound: tensor cores in principle (4*Nq*Nc*64 flop per head), with the softmax exponentials and
// the top-k threshold tests as the practical co-limit.  The MMAs are taken off the issue path and
// the two per-element jobs run on different warps so that their latencies overlap:
//   warp 0  (1 lane)   TMA producer: Q tile pair once, then K and V tiles of 128 keys into rings
//   warp 1             tcgen05.mma issuer (converged warp, one elected lane issues): S = Q K^T (M=128,N=128)
//                      and O += P V (M=128,N=64)
//   warp 2             tensor-memory allocator
//   warps 4-7, 8-11    softmax warpgroups, one per 128-row query tile; thread = row
//   warps 12-15, 16-19 top-k warpgroups, one per query tile; thread = row, reading the same S
// A CTA owns 256 query rows (two tiles sharing every K/V tile).  Tensor memory (512 columns):
// S_A, S_B (128 fp32 columns each), O_A, O_B (64 each), P_A, P_B (bf16 pairs, 64 each).  P is fed
// to the second MMA straight from tensor memory.  S of a tile may be overwritten by the next
// Q K^T only after both its softmax and its top-k warpgroup have read it.
//
// Online softmax with a lazily updated offset: the exponent offset starts at the first tile's row
// maximum and only moves when a tile's sum of P shows that the scores have outgrown it by ~2^24; only
// then is O rescaled in tensor memory, by the softmax threads themselves (each owns one TMEM lane).
// No per-score maximum is tracked in between.
//
// Top-k.  Per row, shared memory holds the best 32 entries (key(score), ~column) as a binary min-heap
// whose root is the worst kept entry; the row's threshold is the root's score.  Everything is done by
// the row's own thread so that the 32 rows of a warp proceed side by side (a warp-cooperative insert
// is a long chain of dependent votes and shuffles that serves one row at a time):
//   * per 16 columns a thread builds a branch-free hit mask against its threshold and moves its
//     hits (key, column) into its row's small pending buffer;
//   * the tile is released to the MMA pipeline as soon as it has been read;
//   * every few tiles, or when a buffer fills, each thread merges its pending hits into its heap
//     (replace the root, sink at most five levels, in lockstep across the warp) and refreshes its
//     threshold.  Batching keeps most lanes busy in that step;
//   * at the end each thread heap-sorts its row in place: slot 0 is rank 0.
// Heaps and pending buffers are laid out [slot][lane] per warp, so thread-private accesses never
// conflict on shared-memory banks whatever slots the lanes touch.
// Ties on the score keep the smaller column first: the heap orders (score, ~column) as one 64-bit word.
// Slots start empty (key 0), which decodes to column Nc-1, the reference's padding.
#include "common.cuh"

namespace s3r {

constexpr int kCmpThreads = 640;             // 12 pipeline/softmax warps + 8 top-k warps
constexpr int kTileBytes = 128 * 128;        // 128 rows x 64 bf16
constexpr int kListBytes = 256 * 32 * 8;      // 8 warps x [32 slots][32 lanes] x (key, column)
#ifndef S3R_CMP_STAGES
#define S3R_CMP_STAGES 3
#endif
#ifndef S3R_CMP_PEND
#define S3R_CMP_PEND 8
#endif
#ifndef S3R_CMP_PEND_SLACK
#define S3R_CMP_PEND_SLACK 2
#endif
constexpr int kStages = S3R_CMP_STAGES;
#ifndef S3R_CMP_MERGE_EVERY
#define S3R_CMP_MERGE_EVERY 4
#endif
constexpr int kMergeEvery = S3R_CMP_MERGE_EVERY;   // tiles between merges of the pending hits
constexpr int kOffQ = 0;
constexpr int kOffK = 2 * kTileBytes;
constexpr int kOffV = kOffK + kStages * kTileBytes;
constexpr int kOffL = kOffV + kStages * kTileBytes;
constexpr int kScratchBytes = 8 * 16 * 32 * 4;          // per top-k warp: 16 logits x 32 rows
constexpr int kOffScr = kOffL + kListBytes;
constexpr int kPend = S3R_CMP_PEND;                                // pending hits per row between merges
constexpr int kPendBytes = 256 * kPend * 8;
constexpr int kOffPend = kOffScr + kScratchBytes;
constexpr int kCmpSmemBytes = kOffPend + kPendBytes + 1024;
// tensor-memory columns
constexpr uint32_t kColS = 0, kColO = 256, kColP = 384;

struct CmpCtl {
  uint64_t q_full, o_full;
  uint64_t k_full[4], k_empty[4], v_full[4], v_empty[4];
  uint64_t s_full[2], p_full[2], tk_done[2], pv_done[2];
  uint32_t tmem_base;
  uint32_t abort_flag;
};

struct CmpParams {
  __nv_bfloat16* o;
  float* lse;
  int32_t* idx;
  int Nq, Nc, topk;
  int n_rank, rank_take;   // block ranking (RANK = 1): number of ranked blocks, columns counted per group of 4
  float c_scale;        // softmax scale * log2(e)
  uint32_t* status;
};

// Index of the lowest set bit of a non-zero 16-bit mask, and the integer held exactly by a float in
// [1, 2^16), both on the integer pipes: find-first-set, population count and float-to-int conversion
// execute on the same 16-lane unit as the exponentials, which the softmax warps keep busy.
__device__ __forceinline__ int lowbit16_alu(uint32_t m) {
  const uint32_t b = m & (0u - m);
  return ((b & 0xff00u) ? 8 : 0) + ((b & 0xf0f0u) ? 4 : 0) + ((b & 0xccccu) ? 2 : 0) + ((b & 0xaaaau) ? 1 : 0);
}
__device__ __forceinline__ uint32_t small_int_of_float(float f) {
  const uint32_t b = __float_as_uint(f);
  return ((b & 0x7fffffu) | 0x800000u) >> (150u - (b >> 23));
}

// Threshold for the float pre-filter `score > thr`: a score can only enter a full list if its key
// is strictly greater than the key in slot topk-1 (an equal key loses to the older, smaller
// column), so rows full of equal scores stop producing hits once their list is full.  The one
// place where float order and key order disagree is -0.0 < +0.0: a kept -0.0 yields a threshold
// just below zero so that +0.0 still passes the pre-filter (the exact test is on the keys).
__device__ __forceinline__ float key_to_float(uint32_t key) {
  if (key == 0u) return -INFINITY;            // empty slot: every finite score qualifies
  if (key == 0x7fffffffu) return __uint_as_float(0x80000001u);   // -0.0 -> largest negative subnormal
  const uint32_t b = (key & 0x80000000u) ? (key ^ 0x80000000u) : ~key;
  return __uint_as_float(b);
}

// A row's best entries live in a binary MIN-heap of `size` 64-bit words (key(score) << 32 | ~column) in
// the row's own shared-memory column ([slot][lane] layout: whatever slots the 32 lanes touch, they never
// meet on a bank).  The root is the worst kept entry, i.e. the row's threshold.  A newcomer replaces the
// root and sinks: at most five levels for 32 entries, executed in lockstep by the 32 rows of a warp (a
// settled lane idles through the remaining levels), ~16 shared-memory accesses instead of the ~62 of a
// shift through a sorted list.  With ~column in the low half a larger word is a better entry under the
// reference's order (score descending, column ascending), so one 64-bit compare decides everything.
__device__ __forceinline__ uint64_t heap_ld(const uint2* p) {
  const uint2 v = *p;
  return (static_cast<uint64_t>(v.x) << 32) | v.y;
}
__device__ __forceinline__ void heap_st(uint2* p, uint64_t v) {
  *p = make_uint2(static_cast<uint32_t>(v >> 32), static_cast<uint32_t>(v));
}
// Puts `v` in the root's place and restores the heap property over h[0..size).
__device__ __forceinline__ void heap_sift_root(uint2* h, uint64_t v, int size, bool active) {
  int i = 0;
  bool go = active;
#pragma unroll
  for (int level = 0; level < 5; ++level) {
    const int l = 2 * i + 1, r = l + 1;
    uint64_t cl = ~0ull, cr = ~0ull;
    if (go && l < size) cl = heap_ld(h + l * 32);
    if (go && r < size) cr = heap_ld(h + r * 32);
    const bool right = cr < cl;
    const uint64_t c = right ? cr : cl;
    const bool mv = go && c < v;
    if (mv) heap_st(h + i * 32, c);
    i = mv ? (right ? r : l) : i;
    go = mv;
  }
  if (active) heap_st(h + i * 32, v);
}
// Heap sort in place: afterwards slot 0 holds the best entry, slot size-1 the worst.
__device__ __forceinline__ void heap_sort_desc(uint2* h, int size) {
  for (int end = size - 1; end >= 1; --end) {
    const uint64_t last = heap_ld(h + end * 32);
    const uint64_t root = heap_ld(h);
    heap_st(h + end * 32, root);          // the smallest of h[0..end] goes to the back
    heap_sift_root(h, last, end, true);
  }
}

// Merge this thread's pending hits (key, column; ascending columns) into its heap and refresh its threshold.
__device__ __noinline__ void topk_merge_own(uint2* my_list, const uint2* my_pend, int& cnt, float& thr, int topk) {
  for (int i = 0; i < cnt; ++i) {
    const uint2 h = my_pend[i * 32];
    const uint64_t ent = (static_cast<uint64_t>(h.x) << 32) | (~h.y);
    // strictly better than the worst kept entry (an equal score arrives with a larger column: it loses)
    const bool want = ent > heap_ld(my_list);
    heap_sift_root(my_list, ent, topk, want);
  }
  if (cnt > 0) thr = key_to_float(my_list[0].x);
  cnt = 0;
}

// RANK = 0: the table holds the top-k COLUMNS of each row by raw logit (the reference's setting, where a
// compressed key is a selection block).  RANK = 1: compressed keys are finer than selection blocks (windows of
// Lc tokens every Sc, blocks of Bs = 4*Sc); the table holds the top-k BLOCKS by the softmax mass of the
// block's own columns 4n .. 4n+take-1, ranked through log2 sum_j 2^(c*s_j), which needs no row normaliser.
template <int RANK>
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
      mbar_init(&ctl.tk_done[t], 128);
      mbar_init(&ctl.pv_done[t], 1);
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
    // ------------------------------------------------------------------ MMA issuer (converged warp, one elected lane issues)
    {
      const bool leader = elect_one_sync();
      constexpr uint32_t idesc_qk = umma_idesc_bf16(128, 128, 0, 0);
      constexpr uint32_t idesc_pv = umma_idesc_bf16(128, 64, 0, 1);   // V tile is [keys][d]: N contiguous
      // descriptors are built once; a tile's descriptor is the base plus its byte offset / 16
      const uint64_t desc_q = umma_desc_sw128(sbase + kOffQ), desc_k = umma_desc_sw128(sbase + kOffK),
                     desc_v = umma_desc_sw128(sbase + kOffV);
      auto issue_qk = [&](int t, int s) {
        umma_ss_k4<2, 2>(tmem + kColS + t * 128, desc_q + static_cast<uint64_t>(t * (kTileBytes >> 4)),
                         desc_k + static_cast<uint64_t>(s * (kTileBytes >> 4)), idesc_qk, 0u);
      };
      auto issue_pv = [&](int t, int s, uint32_t acc) {
        const uint64_t v = desc_v + static_cast<uint64_t>(s * (kTileBytes >> 4));
        umma_ts_k4<128>(tmem + kColO + t * 64, tmem + kColP + t * 64, v, idesc_pv, acc);
        umma_ts_k4<128>(tmem + kColO + t * 64, tmem + kColP + t * 64 + 32, v + 4 * 128, idesc_pv, 1u);
      };
      bool ok = mbar_wait_warp(&ctl.q_full, 0, abort_flag) && mbar_wait_warp(&ctl.k_full[0], 0, abort_flag);
      if (ok) {
        tc_fence_after();
        if (leader) {
          issue_qk(0, 0);
          umma_commit(&ctl.s_full[0]);
          issue_qk(1, 0);
          umma_commit(&ctl.s_full[1]);
          umma_commit(&ctl.k_empty[0]);
        }
        __syncwarp();
        int s = 0, sn = 1 % kStages;
        uint32_t ph = 0, phn = (1 / kStages) & 1;
#pragma unroll 1
        for (int j = 0; j < ntiles && ok; ++j) {
          const bool nxt = j + 1 < ntiles;
          ok = mbar_wait_warp(&ctl.v_full[s], ph, abort_flag);
          if (ok && nxt) ok = mbar_wait_warp(&ctl.k_full[sn], phn, abort_flag);
          if (!ok) break;
#pragma unroll
          for (int t = 0; t < 2; ++t) {
            ok = mbar_wait_warp(&ctl.p_full[t], j & 1, abort_flag);
            if (!ok) break;
            tc_fence_after();
            // The next scores are what the 256 waiting threads need; P V only has to finish before the next
            // P V of the tile.  So when the top-k warps have released S already, Q K^T goes first.
            const bool qk_first = nxt && __all_sync(0xffffffffu, mbar_test_wait(&ctl.tk_done[t], j & 1));
            if (qk_first) {
              tc_fence_after();
              if (leader) {
                issue_qk(t, sn);
                umma_commit(&ctl.s_full[t]);
              }
            }
            if (leader) {
              issue_pv(t, s, j > 0 ? 1u : 0u);
              umma_commit(&ctl.pv_done[t]);          // P of this tile may be overwritten, O is at rest
              if (t == 1) umma_commit(&ctl.v_empty[s]);
            }
            __syncwarp();
            if (nxt && !qk_first) {
              ok = mbar_wait_warp(&ctl.tk_done[t], j & 1, abort_flag);    // S of this tile has been read by top-k too
              if (!ok) break;
              tc_fence_after();
              if (leader) {
                issue_qk(t, sn);
                umma_commit(&ctl.s_full[t]);
              }
            }
            if (nxt && t == 1 && leader) umma_commit(&ctl.k_empty[sn]);
            __syncwarp();
          }
          s = sn; ph = phn;
          if (++sn == kStages) { sn = 0; phn ^= 1u; }
        }
      }
      if (leader) umma_commit(&ctl.o_full);
      __syncwarp();
      if (!ok) {
        volatile uint32_t dummy = 0;
        mbar_wait(&ctl.o_full, 0, &dummy);     // let issued MMAs drain before tensor memory is freed
      }
    }
  } else if (warp >= 4 && warp < 12) {
    // ------------------------------------------------------------------ softmax, thread = row
    const int t = (warp - 4) >> 2;
    const int quarter = warp & 3;
    const int grow = q0 + t * 128 + quarter * 32 + lane;
    const uint32_t lane_base = tmem + (static_cast<uint32_t>(quarter * 32) << 16);
    const uint32_t t_s = lane_base + kColS + t * 128;
    const uint32_t t_o = lane_base + kColO + t * 64;
    const uint32_t t_p = lane_base + kColP + t * 64;
    const float cs = p.c_scale;
    float m_used = -INFINITY, l = 0.f;
    bool ok = true;

    for (int j = 0; j < ntiles; ++j) {
      if (!mbar_wait_warp(&ctl.s_full[t], j & 1, abort_flag)) { ok = false; break; }
      tc_fence_after();
      const int col0 = j * 128;
      const bool tail = (col0 + 128 > p.Nc);

      // One pass with tensor-memory loads kept one chunk ahead of the arithmetic: P is computed
      // with the exponent offset carried over from earlier tiles.  Only if some row's scores have
      // outgrown its offset so far that P nears overflow is the tile redone with the row's exact
      // maximum as the new offset (O and l rescaled).  S stays valid until this warpgroup arrives
      // on p_full, so the redo re-reads it.  Tile 0 has no offset yet: its maximum is taken first.
      auto mask_tail = [&](uint32_t (&x)[16], int c8) {
        const int nvalid = min(16, max(0, p.Nc - (col0 + c8 * 16)));
#pragma unroll
        for (int i = 0; i < 16; ++i)
          if (i >= nvalid) x[i] = 0xff800000u;   // -inf
      };
      if (j == 0) {
        float rmax0 = -INFINITY;
#pragma unroll 1
        for (int c8 = 0; c8 < 8; ++c8) {
          uint32_t x[16];
          tmem_ld16(t_s + c8 * 16, x);
          tmem_ld_wait();
          if (tail) mask_tail(x, c8);
#pragma unroll
          for (int i = 0; i < 16; ++i) rmax0 = fmaxf(rmax0, __uint_as_float(x[i]));
        }
        m_used = rmax0 * cs;
      }
      // P of the previous tile must have been consumed by its P V before it is overwritten, and O must be
      // at rest before a rescale: when the issuer put the next Q K^T ahead of P V, s_full alone does not
      // say so.  The wait is normally satisfied already.
      if (j > 0) {
        if (!mbar_wait_warp(&ctl.pv_done[t], (j - 1) & 1, abort_flag)) { ok = false; break; }
        tc_fence_after();
      }
      float ls[4];
      bool redo, redone = false;
      do {
        ls[0] = ls[1] = ls[2] = ls[3] = 0.f;
        auto process = [&](uint32_t (&x)[16], int c8) {
          if (tail) mask_tail(x, c8);
          uint32_t pk[8];
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const float s0 = __uint_as_float(x[2 * i]), s1 = __uint_as_float(x[2 * i + 1]);
            const float p0 = fast_exp2(fmaf(s0, cs, -m_used));
            const float p1 = fast_exp2(fmaf(s1, cs, -m_used));
            ls[i & 3] += p0 + p1;
            pk[i] = pack_bf16(p0, p1);
          }
          tmem_st8(t_p + c8 * 8, pk);
        };
        uint32_t xa[16], xb[16];
        tmem_ld16(t_s, xa);
#pragma unroll 1
        for (int c8 = 0; c8 < 8; c8 += 2) {
          tmem_ld_wait();
          tmem_ld16(t_s + (c8 + 1) * 16, xb);
          process(xa, c8);
          tmem_ld_wait();
          if (c8 + 2 < 8) tmem_ld16(t_s + (c8 + 2) * 16, xa);
          process(xb, c8 + 1);
        }
        // The offset m_used may lag behind the row's true maximum: P is then large, which costs nothing
        // (bf16 and fp32 keep their relative precision, O and l are fp32) until it nears overflow.  The tile's
        // own sum of P tells: every P is positive, so max P <= sum <= 128 max P, and no per-score maximum has
        // to be tracked.  Past 2^24 (or on a non-finite sum) the tile is redone once with the exact maximum.
        const float tsum = (ls[0] + ls[1]) + (ls[2] + ls[3]);
        const bool need = !(tsum <= 16777216.f);
        redo = !redone && __any_sync(0xffffffffu, need);
        if (redo) {
          redone = true;
          float rmax = -INFINITY;
#pragma unroll 1
          for (int c8 = 0; c8 < 8; ++c8) {
            uint32_t x[16];
            tmem_ld16(t_s + c8 * 16, x);
            tmem_ld_wait();
            if (tail) mask_tail(x, c8);
#pragma unroll
            for (int i = 0; i < 16; i += 2) rmax = fmax3(rmax, __uint_as_float(x[i]), __uint_as_float(x[i + 1]));
          }
          const float mt = rmax * cs;
          const bool grow = need && mt > m_used;
          const float factor = grow ? fast_exp2(m_used - mt) : 1.f;
          if (grow) {
            m_used = mt;
            l *= factor;
          }
          tmem_st_wait();
          if (j > 0) {
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
        }
      } while (redo);
      l += (ls[0] + ls[1]) + (ls[2] + ls[3]);
      tmem_st_wait();
      tc_fence_before();
      mbar_arrive(&ctl.p_full[t]);
    }

    // epilogue: O / l and lse
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
    }
    if (!ok && lane == 0) atomicOr(p.status, kStatusWaitTimeout);
  } else if (warp >= 12) {
    // ------------------------------------------------------------------ top-k, thread = row
    const int t = (warp - 12) >> 2;
    const int quarter = warp & 3;
    const uint32_t t_s = tmem + (static_cast<uint32_t>(quarter * 32) << 16) + kColS + t * 128;
    uint2* warp_lists = lists + (warp - 12) * (32 * 32);            // [slot][lane]
    uint2* my_list = warp_lists + lane;
    uint32_t* scratch = reinterpret_cast<uint32_t*>(sptr + kOffScr) + (warp - 12) * (16 * 32);
    uint2* my_pend = reinterpret_cast<uint2*>(sptr + kOffPend) + (warp - 12) * (kPend * 32) + lane;   // [i][lane]
    int cnt = 0;
    const int topk = p.topk;
    float thr = -INFINITY;
    bool ok = true;

    for (int j = 0; j < ntiles; ++j) {
      if (!mbar_wait_warp(&ctl.s_full[t], j & 1, abort_flag)) { ok = false; break; }
      tc_fence_after();
      const int col0 = j * 128;
      const bool tail = (col0 + 128 > p.Nc);

      auto handle = [&](uint32_t (&x)[16], int c8) {
        const int cbase = col0 + c8 * 16;
        if (tail) {
          const int nvalid = min(16, max(0, p.Nc - cbase));
#pragma unroll
          for (int i = 0; i < 16; ++i)
            if (i >= nvalid) x[i] = 0xff7fffffu;   // -FLT_MAX: never a hit, and 0 * it stays finite
        }
        // Once the lists have filled, most chunks hold no hit for any of the warp's 32 rows: a
        // three-input max tree (8 instructions for 16 scores) and one vote skip the mask below for them.
        float cm;
        {
          const float m0 = fmax3(__uint_as_float(x[0]), __uint_as_float(x[1]), __uint_as_float(x[2]));
          const float m1 = fmax3(__uint_as_float(x[3]), __uint_as_float(x[4]), __uint_as_float(x[5]));
          const float m2 = fmax3(__uint_as_float(x[6]), __uint_as_float(x[7]), __uint_as_float(x[8]));
          const float m3 = fmax3(__uint_as_float(x[9]), __uint_as_float(x[10]), __uint_as_float(x[11]));
          const float m4 = fmax3(__uint_as_float(x[12]), __uint_as_float(x[13]), __uint_as_float(x[14]));
          cm = fmaxf(fmax3(fmax3(m0, m1, m2), m3, m4), __uint_as_float(x[15]));
          if (!__any_sync(0xffffffffu, cm > thr)) return;
        }
        // Hit mask on the FMA pipe (compares, selects and logic ops all share the half-rate ALU
        // pipe, which this kernel saturates first):  t = saturate((x - thr) * 2^60) is 1.0 for a
        // hit and 0.0 otherwise (the fused product is exact before rounding, so any x > thr gives
        // >= 1);  sum t * 2^i is the mask; when there is exactly one hit it is the chunk's maximum,
        // which the tree above has left in cm.  Chunks with several hits, or a full buffer, take the indexed path below, which
        // appends in ascending column order (that is what keeps equal scores in column order).
        // (2^90: exact for thresholds below 2^37 in magnitude and score gaps above 2^-90, i.e. for
        // every pair of distinct fp32 logits larger than 2^-66 in magnitude.)
        const float kHuge = 1.2379400392853803e27f;              // 2^90
        // while the list has free slots (thr = -inf) every real score is a hit, the -FLT_MAX fillers
        // of the tail are not: a large finite offset does both (an infinite one would not)
        const float nthr = (thr == -INFINITY) ? 3.0e38f : -thr * kHuge;
        float acc0 = 0.f, acc1 = 0.f;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const float a = __uint_as_float(x[i]), b = __uint_as_float(x[8 + i]);
          const float t0 = __saturatef(fmaf(a, kHuge, nthr));
          const float t1 = __saturatef(fmaf(b, kHuge, nthr));
          acc0 = fmaf(t0, static_cast<float>(1u << i), acc0);
          acc1 = fmaf(t1, static_cast<float>(256u << i), acc1);
        }
        // The mask is an exact integer below 2^16 held in a float: a single hit is a power of two (zero
        // mantissa) whose exponent is the column.  Read off the bits, this keeps the float-to-int
        // conversion and the find-first-set (both on the pipe the exponentials keep busy) out of the common case.
        const float accf = acc0 + acc1;
        const uint32_t ab = __float_as_uint(accf);
        bool left = accf != 0.f;
        // (a zero or non-finite maximum goes the indexed way: max cannot tell -0.0 from +0.0)
        if (left && (ab & 0x7fffffu) == 0u && cnt < kPend && cm != 0.f && fabsf(cm) < INFINITY) {
          my_pend[cnt * 32] = make_uint2(sortable_key(cm), static_cast<uint32_t>(cbase) + (ab >> 23) - 127u);
          ++cnt;
          left = false;
        }
        if (!__any_sync(0xffffffffu, left)) return;                // nothing left anywhere in the warp
        uint32_t m = left ? small_int_of_float(accf) : 0u;
        if (m) {
          // this thread's own copy of the chunk, so that a hit can be fetched by its (dynamic) index
          uint4* s4 = reinterpret_cast<uint4*>(scratch);
#pragma unroll
          for (int q = 0; q < 4; ++q) s4[q * 32 + lane] = make_uint4(x[4 * q], x[4 * q + 1], x[4 * q + 2], x[4 * q + 3]);
        }
        while (true) {
          while (m && cnt < kPend) {
            const int e = lowbit16_alu(m);
            m &= m - 1;
            const float v = __uint_as_float(scratch[(((e >> 2) * 32 + lane) << 2) + (e & 3)]);
            my_pend[cnt * 32] = make_uint2(sortable_key(v), static_cast<uint32_t>(cbase + e));
            ++cnt;
          }
          if (!__any_sync(0xffffffffu, m != 0u)) break;          // nobody ran out of room
          topk_merge_own(my_list, my_pend, cnt, thr, topk);      // every lane merges what it has
        }
      };

      // Block ranking: the 16 columns of a chunk are four groups of four; a group's score is
      // log2 sum 2^(c*s) over its first `rank_take` columns.  Hits are appended in ascending block order.
      auto handle_blocks = [&](uint32_t (&x)[16], int c8) {
        const int gbase = (col0 + c8 * 16) >> 2;
        const float cs = p.c_scale;
        float r[4];
        bool valid[4];
#pragma unroll
        for (int gi = 0; gi < 4; ++gi) {
          float a[4];
#pragma unroll
          for (int e = 0; e < 4; ++e) a[e] = (e < p.rank_take) ? __uint_as_float(x[4 * gi + e]) * cs : -INFINITY;
          const float m = fmaxf(fmax3(a[0], a[1], a[2]), a[3]);
          const float sum = (fast_exp2(a[0] - m) + fast_exp2(a[1] - m)) + (fast_exp2(a[2] - m) + fast_exp2(a[3] - m));
          valid[gi] = gbase + gi < p.n_rank;            // all of the group's counted columns exist
          r[gi] = valid[gi] ? m + fast_log2(sum) : -INFINITY;
        }
        const float cm = fmaxf(fmaxf(r[0], r[1]), fmaxf(r[2], r[3]));
        if (!__any_sync(0xffffffffu, cm > thr || (thr == -INFINITY && (valid[0] || valid[1] || valid[2] || valid[3])))) return;
#pragma unroll
        for (int gi = 0; gi < 4; ++gi) {
          // an empty slot (thr = -inf) takes any ranked block, whatever its score
          const bool hit = valid[gi] && (r[gi] > thr || thr == -INFINITY);
          while (__any_sync(0xffffffffu, hit && cnt >= kPend)) topk_merge_own(my_list, my_pend, cnt, thr, topk);
          if (hit) {
            my_pend[cnt * 32] = make_uint2(sortable_key(r[gi]), static_cast<uint32_t>(gbase + gi));
            ++cnt;
          }
        }
      };

      // tensor-memory loads run one chunk ahead of the handling
      uint32_t xa[16], xb[16];
      tmem_ld16(t_s, xa);
#pragma unroll 1
      for (int c8 = 0; c8 < 8; c8 += 2) {
        tmem_ld_wait();
        tmem_ld16(t_s + (c8 + 1) * 16, xb);
        if (RANK == 0) handle(xa, c8); else handle_blocks(xa, c8);
        tmem_ld_wait();
        if (c8 + 2 < 8) {
          tmem_ld16(t_s + (c8 + 2) * 16, xa);
        } else {                              // S has been read in full: the next Q K^T may overwrite it
          tc_fence_before();
          mbar_arrive(&ctl.tk_done[t]);
        }
        if (RANK == 0) handle(xb, c8 + 1); else handle_blocks(xb, c8 + 1);
      }
      // the tile is already released; merge the pending hits every few tiles, or early when some
      // buffer is nearly full
      if ((j % kMergeEvery) == kMergeEvery - 1 || j == ntiles - 1 ||
          __any_sync(0xffffffffu, cnt >= kPend - S3R_CMP_PEND_SLACK))
        topk_merge_own(my_list, my_pend, cnt, thr, topk);
      __syncwarp();
    }

    // sorted index rows: slot l is rank l; an empty slot decodes to column Nc-1
    if (ok) {
      heap_sort_desc(my_list, topk);
      __syncwarp();
      const int wrow0 = q0 + t * 128 + quarter * 32;
      for (int r = 0; r < 32 && wrow0 + r < p.Nq; ++r) {
        const uint2 ent = warp_lists[lane * 32 + r];
        if (lane < topk)
          p.idx[(static_cast<int64_t>(bh) * p.Nq + wrow0 + r) * topk + lane] =
              (ent.x == 0u) ? ((RANK == 0 ? p.Nc : p.n_rank) - 1) : static_cast<int32_t>(~ent.y);
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

static int launch_cmp_fwd(const char* who, const void* q_c, const void* k_c, const void* v_c, void* o_c, float* lse,
                          int32_t* idx, int B, int H, int Nq, int Nc, int d, int topk, float scale, int rank_take,
                          void* stream) {
  S3R_REQUIRE(q_c && k_c && v_c && o_c && lse && idx, S3R_ERR_NULL, "%s: NULL pointer", who);
  S3R_REQUIRE(B > 0 && H > 0 && Nq > 0 && Nc > 0, S3R_ERR_SHAPE, "%s: sizes must be positive (B=%d H=%d Nq=%d Nc=%d)", who,
              B, H, Nq, Nc);
  S3R_REQUIRE(d == 64, S3R_ERR_UNSUPPORTED, "%s: head_dim %d not supported (64 only)", who, d);
  S3R_REQUIRE(topk >= 1 && topk <= 32, S3R_ERR_UNSUPPORTED, "%s: topk %d not in [1,32]", who, topk);
  S3R_REQUIRE(scale > 0.f, S3R_ERR_UNSUPPORTED, "%s: softmax scale must be positive", who);
  const uintptr_t al = reinterpret_cast<uintptr_t>(q_c) | reinterpret_cast<uintptr_t>(k_c) |
                       reinterpret_cast<uintptr_t>(v_c) | reinterpret_cast<uintptr_t>(o_c);
  S3R_REQUIRE((al & 15) == 0, S3R_ERR_ALIGNMENT, "%s: tensors must be 16-byte aligned", who);
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
  p.Nq = Nq; p.Nc = Nc; p.topk = topk;
  p.rank_take = rank_take;
  p.n_rank = rank_take > 0 ? (Nc - rank_take) / 4 + 1 : 0;      // groups of four columns with all counted columns present
  p.c_scale = scale * 1.4426950408889634f;
  p.status = device_status_ptr();
  S3R_REQUIRE(p.status != nullptr, S3R_ERR_DRIVER, "%s: could not resolve the device status word", who);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int64_t grid = static_cast<int64_t>(BH) * ((Nq + 255) / 256);
  S3R_REQUIRE(grid < (1ll << 31), S3R_ERR_TOO_LARGE, "%s: grid too large", who);
  // per device and idempotent: setting it on every call keeps the entry points free of process-global state
  if (rank_take == 0) {
    S3R_CUDA(cudaFuncSetAttribute(cmp_fwd_kernel<0>, cudaFuncAttributeMaxDynamicSharedMemorySize, kCmpSmemBytes));
    cmp_fwd_kernel<0><<<static_cast<unsigned>(grid), kCmpThreads, kCmpSmemBytes, st>>>(mq, mk, mv, p);
  } else {
    S3R_CUDA(cudaFuncSetAttribute(cmp_fwd_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, kCmpSmemBytes));
    cmp_fwd_kernel<1><<<static_cast<unsigned>(grid), kCmpThreads, kCmpSmemBytes, st>>>(mq, mk, mv, p);
  }
  S3R_CUDA(cudaGetLastError());
  return 0;
}

extern "C" int s3r_cmp_attn_topk_fwd(const void* q_c, const void* k_c, const void* v_c, void* o_c, float* lse,
                                     int32_t* idx, int B, int H, int Nq, int Nc, int d, int topk, float scale,
                                     void* stream) {
  return launch_cmp_fwd("s3r_cmp_attn_topk_fwd", q_c, k_c, v_c, o_c, lse, idx, B, H, Nq, Nc, d, topk, scale, 0, stream);
}

extern "C" int s3r_cmp_attn_blocktopk_fwd(const void* q_c, const void* k_c, const void* v_c, void* o_c, float* lse,
                                          int32_t* idx, int B, int H, int Nq, int Nc, int d, int topk, float scale,
                                          int group, int take, void* stream) {
  S3R_REQUIRE(group == 4, S3R_ERR_UNSUPPORTED, "s3r_cmp_attn_blocktopk_fwd: %d compressed keys per block (4 only)", group);
  S3R_REQUIRE(take >= 1 && take <= 4 && Nc >= take, S3R_ERR_UNSUPPORTED,
              "s3r_cmp_attn_blocktopk_fwd: take=%d must be in [1,4] and <= Nc=%d", take, Nc);
  return launch_cmp_fwd("s3r_cmp_attn_blocktopk_fwd", q_c, k_c, v_c, o_c, lse, idx, B, H, Nq, Nc, d, topk, scale, take,
                        stream);
}
