// Selection branch, backward: key-centric index (CSR) of the selection table built on the device,
// the fused backward of the gated merge, and the two sparse gradient kernels.
//
//   dQ    : one warp per 16 query rows, looping over the key blocks its query block selected
//   dK/dV : one warp per 16 key rows, looping over the query blocks that selected its key block
//           (CSR lists, ascending query block => a fixed summation order, no atomics on floats)
// Both stream 16-row tiles through a cp.async ring private to the warp (two stages for dQ, whose list
// sits in shared memory; three for dK/dV, which also fetches its list and the rows' statistics ahead) and
// use the mma.sync building blocks of bwd_common.cuh.  Both gather ~130 GB of 128-byte rows out of L2 at
// 1000 views (16..64 flop per byte): dQ 16 ms, dK/dV 22 ms.
#include <mutex>

#include "bwd_common.cuh"

namespace s3r {

// ------------------------------------------------------------------------------------------------
// key-centric CSR
// ------------------------------------------------------------------------------------------------
__global__ void csr_count_kernel(const int32_t* __restrict__ idx, int32_t* __restrict__ counts, int64_t per_bh,
                                 int64_t total, int Nkb) {
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int n = idx[i];
    if (n >= 0 && n < Nkb) atomicAdd(&counts[(i / per_bh) * (Nkb + 1) + n], 1);
  }
}

// One CTA per (b,h): exclusive scan of counts[0..Nkb) in place -> offsets[0..Nkb]; cursor = offsets.
__global__ void __launch_bounds__(1024) csr_scan_kernel(int32_t* __restrict__ offsets, int32_t* __restrict__ cursor,
                                                        int Nkb) {
  __shared__ int32_t warp_sums[32];
  __shared__ int32_t carry_s;
  int32_t* off = offsets + static_cast<int64_t>(blockIdx.x) * (Nkb + 1);
  int32_t* cur = cursor + static_cast<int64_t>(blockIdx.x) * Nkb;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (threadIdx.x == 0) carry_s = 0;
  __syncthreads();
  for (int base = 0; base < Nkb; base += 1024) {
    const int i = base + threadIdx.x;
    const int32_t v = (i < Nkb) ? off[i] : 0;
    int32_t x = v;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int32_t y = __shfl_up_sync(0xffffffffu, x, o);
      if (lane >= o) x += y;
    }
    if (lane == 31) warp_sums[warp] = x;
    __syncthreads();
    if (warp == 0) {
      int32_t w = warp_sums[lane];
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int32_t y = __shfl_up_sync(0xffffffffu, w, o);
        if (lane >= o) w += y;
      }
      warp_sums[lane] = w;   // inclusive
    }
    __syncthreads();
    const int32_t carry = carry_s;
    const int32_t excl = carry + (warp > 0 ? warp_sums[warp - 1] : 0) + x - v;
    if (i < Nkb) {
      off[i] = excl;
      cur[i] = excl;
    }
    __syncthreads();
    if (threadIdx.x == 1023) carry_s = carry + warp_sums[31];
    __syncthreads();
  }
  if (threadIdx.x == 0) off[Nkb] = carry_s;
}

__global__ void csr_fill_kernel(const int32_t* __restrict__ idx, int32_t* __restrict__ cursor,
                                int32_t* __restrict__ tmp, int64_t per_bh, int64_t total, int Nkb, int topk) {
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int n = idx[i];
    if (n >= 0 && n < Nkb) {
      const int64_t bh = i / per_bh;
      const int32_t pos = atomicAdd(&cursor[bh * Nkb + n], 1);
      tmp[bh * per_bh + pos] = static_cast<int32_t>((i - bh * per_bh) / topk);   // query block
    }
  }
}

// The fill above leaves every segment complete but in arrival order; the gradient kernel needs ascending
// query blocks (a fixed summation order).  Segments are sorted by length class:
//   len <= 32      one warp ranks the segment with shuffles (the common case: the mean length is top-k)
//   len <= 4096    one CTA, bitonic network in shared memory
//   longer         ("sink" key blocks that most query blocks select) one CTA walks the (b,h) slice of the
//                  table in order and compacts the matching query blocks: O(Nq*topk), no comparison sort
// The first kernel handles the short class and queues every other segment for the second.
constexpr int kCsrSmemSort = 4096;

__global__ void __launch_bounds__(256) csr_sort_small_kernel(const int32_t* __restrict__ offsets,
                                                             const int32_t* __restrict__ tmp, int32_t* __restrict__ qids,
                                                             int64_t per_bh, int Nkb, int64_t nseg,
                                                             int32_t* __restrict__ queue) {
  const int lane = threadIdx.x & 31;
  const int64_t seg = (blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x) >> 5;
  if (seg >= nseg) return;
  const int64_t bh = seg / Nkb;
  const int n = static_cast<int>(seg - bh * Nkb);
  const int32_t* off = offsets + bh * (Nkb + 1);
  const int beg = off[n], len = off[n + 1] - beg;
  if (len > 32) {
    if (lane == 0) queue[1 + atomicAdd(&queue[0], 1)] = static_cast<int32_t>(seg);
    return;
  }
  const int32_t x = (lane < len) ? tmp[bh * per_bh + beg + lane] : 0x7fffffff;
  int rank = 0;
  for (int t = 0; t < len; ++t) {
    const int32_t yt = __shfl_sync(0xffffffffu, x, t);
    rank += (yt < x) || (yt == x && t < lane);
  }
  if (lane < len) qids[bh * per_bh + beg + rank] = x;
}

__global__ void __launch_bounds__(256) csr_sort_long_kernel(const int32_t* __restrict__ idx,
                                                            const int32_t* __restrict__ offsets,
                                                            const int32_t* __restrict__ tmp, int32_t* __restrict__ qids,
                                                            int64_t per_bh, int Nkb, int topk,
                                                            const int32_t* __restrict__ queue) {
  __shared__ int32_t buf[kCsrSmemSort];
  __shared__ int32_t warp_tot[8];
  __shared__ int32_t run_base;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int nqueued = queue[0];
  for (int w = blockIdx.x; w < nqueued; w += gridDim.x) {
    const int64_t seg = queue[1 + w];
    const int64_t bh = seg / Nkb;
    const int n = static_cast<int>(seg - bh * Nkb);
    const int32_t* off = offsets + bh * (Nkb + 1);
    const int beg = off[n], len = off[n + 1] - beg;
    int32_t* dst = qids + bh * per_bh + beg;
    if (len <= kCsrSmemSort) {
      int P = 64;
      while (P < len) P <<= 1;
      const int32_t* src = tmp + bh * per_bh + beg;
      for (int i = tid; i < P; i += 256) buf[i] = (i < len) ? src[i] : 0x7fffffff;
      __syncthreads();
      for (int k = 2; k <= P; k <<= 1) {
        for (int j = k >> 1; j > 0; j >>= 1) {
          for (int i = tid; i < P; i += 256) {
            const int l = i ^ j;
            if (l > i) {
              const int32_t a = buf[i], b = buf[l];
              const bool up = (i & k) == 0;
              if ((a > b) == up) { buf[i] = b; buf[l] = a; }
            }
          }
          __syncthreads();
        }
      }
      for (int i = tid; i < len; i += 256) dst[i] = buf[i];
      __syncthreads();
    } else {
      // ordered compaction over the (b,h) slice of the table: 8 consecutive entries per thread
      const int32_t* tab = idx + bh * per_bh;
      if (tid == 0) run_base = 0;
      __syncthreads();
      for (int64_t base = 0; base < per_bh; base += 256 * 8) {
        const int64_t i0 = base + static_cast<int64_t>(tid) * 8;
        int32_t e[8];
        int cnt = 0;
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          e[u] = (i0 + u < per_bh) ? tab[i0 + u] : -1;
          cnt += (e[u] == n);
        }
        int incl = cnt;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
          const int y = __shfl_up_sync(0xffffffffu, incl, o);
          if (lane >= o) incl += y;
        }
        if (lane == 31) warp_tot[warp] = incl;
        __syncthreads();
        int before = run_base + incl - cnt;
        int total = 0;
#pragma unroll
        for (int ww = 0; ww < 8; ++ww) {
          const int t = warp_tot[ww];
          before += (ww < warp) ? t : 0;
          total += t;
        }
#pragma unroll
        for (int u = 0; u < 8; ++u)
          if (e[u] == n) dst[before++] = static_cast<int32_t>((i0 + u) / topk);
        __syncthreads();
        if (tid == 0) run_base += total;
        __syncthreads();
      }
    }
  }
}

// ------------------------------------------------------------------------------------------------
// delta = sum_d o * do  (8 lanes per row, 16-byte loads)
// ------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) delta_kernel(const __nv_bfloat16* __restrict__ o,
                                                    const __nv_bfloat16* __restrict__ d_o, float* __restrict__ delta,
                                                    int64_t rows) {
  const int64_t gid = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x;
  const int64_t row = gid >> 3;
  const int c8 = threadIdx.x & 7;
  float s = 0.f;
  if (row < rows) {
    const uint4 a = *reinterpret_cast<const uint4*>(o + row * 64 + c8 * 8);
    const uint4 b = *reinterpret_cast<const uint4*>(d_o + row * 64 + c8 * 8);
    const uint32_t aw[4] = {a.x, a.y, a.z, a.w}, bw[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
    for (int w = 0; w < 4; ++w) s += bf16_lo(aw[w]) * bf16_lo(bw[w]) + bf16_hi(aw[w]) * bf16_hi(bw[w]);
  }
  s += __shfl_xor_sync(0xffffffffu, s, 1);
  s += __shfl_xor_sync(0xffffffffu, s, 2);
  s += __shfl_xor_sync(0xffffffffu, s, 4);
  if (row < rows && c8 == 0) delta[row] = s;
}

// ------------------------------------------------------------------------------------------------
// backward of the gated merge: one warp per (b,h,query block); 8 lanes per token, 4 tokens a pass
// ------------------------------------------------------------------------------------------------
struct MergeBwdParams {
  const __nv_bfloat16* dy;
  const __nv_bfloat16* gate;
  int64_t gsb, gsh, gst;
  const __nv_bfloat16* o_c;
  const __nv_bfloat16* o_s;
  __nv_bfloat16* do_s;
  float* dgate;
  __nv_bfloat16* do_c;
  float* delta_s;
  int B, H, Tq, block, nqb;
};

__global__ void __launch_bounds__(256) merge_bwd_kernel(const MergeBwdParams p) {
  const int lane = threadIdx.x & 31;
  const int64_t wid = (blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x) >> 5;
  if (wid >= static_cast<int64_t>(p.B) * p.H * p.nqb) return;
  const int m = static_cast<int>(wid % p.nqb);
  const int bh = static_cast<int>(wid / p.nqb);
  const int b = bh / p.H, h = bh % p.H;
  const int sub = lane >> 3, c8 = lane & 7;
  float oc[8], acc[8];
  {
    const uint4 v = *reinterpret_cast<const uint4*>(p.o_c + (static_cast<int64_t>(bh) * p.nqb + m) * 64 + c8 * 8);
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) { oc[2 * i] = bf16_lo(w[i]); oc[2 * i + 1] = bf16_hi(w[i]); acc[2 * i] = acc[2 * i + 1] = 0.f; }
  }
  for (int t0 = 0; t0 < p.block; t0 += 4) {
    const int t = m * p.block + t0 + sub;
    const bool live = (t0 + sub < p.block) && (t < p.Tq);
    float dyv[8] = {}, osv[8] = {}, g0 = 0.f, g1 = 0.f;
    if (live) {
      const uint4 a = *reinterpret_cast<const uint4*>(p.dy + ((static_cast<int64_t>(b) * p.Tq + t) * p.H + h) * 64 + c8 * 8);
      const uint4 s = *reinterpret_cast<const uint4*>(p.o_s + (static_cast<int64_t>(bh) * p.Tq + t) * 64 + c8 * 8);
      const uint32_t aw[4] = {a.x, a.y, a.z, a.w}, sw[4] = {s.x, s.y, s.z, s.w};
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        dyv[2 * i] = bf16_lo(aw[i]); dyv[2 * i + 1] = bf16_hi(aw[i]);
        osv[2 * i] = bf16_lo(sw[i]); osv[2 * i + 1] = bf16_hi(sw[i]);
      }
      const uint32_t gw = *reinterpret_cast<const uint32_t*>(p.gate + b * p.gsb + h * p.gsh + t * p.gst);
      g0 = bf16_lo(gw); g1 = bf16_hi(gw);
    }
    float d0 = 0.f, d1 = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      d0 += dyv[i] * oc[i];
      d1 += dyv[i] * osv[i];
      acc[i] += g0 * dyv[i];
    }
#pragma unroll
    for (int o = 1; o < 8; o <<= 1) {
      d0 += __shfl_xor_sync(0xffffffffu, d0, o);
      d1 += __shfl_xor_sync(0xffffffffu, d1, o);
    }
    if (live) {
      uint4 out;
      out.x = pack_bf16(g1 * dyv[0], g1 * dyv[1]); out.y = pack_bf16(g1 * dyv[2], g1 * dyv[3]);
      out.z = pack_bf16(g1 * dyv[4], g1 * dyv[5]); out.w = pack_bf16(g1 * dyv[6], g1 * dyv[7]);
      *reinterpret_cast<uint4*>(p.do_s + (static_cast<int64_t>(bh) * p.Tq + t) * 64 + c8 * 8) = out;
      if (c8 == 0) {
        *reinterpret_cast<float2*>(p.dgate + (static_cast<int64_t>(bh) * p.Tq + t) * 2) = make_float2(d0, d1);
        p.delta_s[static_cast<int64_t>(bh) * p.Tq + t] = g1 * d1;
      }
    }
  }
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    acc[i] += __shfl_xor_sync(0xffffffffu, acc[i], 8);
    acc[i] += __shfl_xor_sync(0xffffffffu, acc[i], 16);
  }
  if (sub == 0) {
    uint4 out;
    out.x = pack_bf16(acc[0], acc[1]); out.y = pack_bf16(acc[2], acc[3]);
    out.z = pack_bf16(acc[4], acc[5]); out.w = pack_bf16(acc[6], acc[7]);
    *reinterpret_cast<uint4*>(p.do_c + (static_cast<int64_t>(bh) * p.nqb + m) * 64 + c8 * 8) = out;
  }
}

// ------------------------------------------------------------------------------------------------
// sparse dQ and dK/dV
// ------------------------------------------------------------------------------------------------
constexpr int kBwdWarps = 4;
constexpr int kTile = 16 * kPitch;            // one 16-row tile in shared memory

struct SelBwdParams {
  const __nv_bfloat16 *q, *k, *v, *d_o;
  const int32_t *idx, *offsets, *qids;
  const float *lse, *delta;
  __nv_bfloat16 *dq, *dk, *dv;
  int B, H, Tq, Tk, block, topk, nqb, nkb;
  float cs, scale;
};

// 16 rows x 128 B from global (row stride 64 elements) into a padded tile; rows >= nrows zero-filled
__device__ __forceinline__ void load_tile16(uint32_t dst, const __nv_bfloat16* src, int nrows, int lane) {
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int ch = lane + 32 * i, r = ch >> 3, c16 = ch & 7;
    cp_async16(dst + r * kPitch + c16 * 16, src + static_cast<int64_t>(r) * 64 + c16 * 8, r < nrows);
  }
}

#ifndef S3R_DQ_MIN_CTAS
#define S3R_DQ_MIN_CTAS 1
#endif
__global__ void __launch_bounds__(kBwdWarps * 32, S3R_DQ_MIN_CTAS) sel_bwd_dq_kernel(const SelBwdParams p) {
  __shared__ __align__(16) uint8_t smem[kBwdWarps][2][2 * kTile];
  __shared__ int32_t lists[kBwdWarps][64];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2;
  const int nslices = (p.Tq + 15) / 16;
  const int64_t task = static_cast<int64_t>(blockIdx.x) * kBwdWarps + warp;
  if (task >= static_cast<int64_t>(p.B) * p.H * nslices) return;
  const int bh = static_cast<int>(task / nslices);
  const int row0 = static_cast<int>(task % nslices) * 16;
  const int m = row0 / p.block;
  const uint32_t sm0 = smem_u32(&smem[warp][0][0]), sm1 = smem_u32(&smem[warp][1][0]);

  // valid entries of the query block's row of the table, table order
  int nvalid = 0;
  {
    const int32_t* row = p.idx + (static_cast<int64_t>(bh) * p.nqb + m) * p.topk;
    for (int r0 = 0; r0 < p.topk; r0 += 32) {
      const int i = r0 + lane;
      const int n = (i < p.topk) ? row[i] : -1;
      const bool ok = (n >= 0) && (static_cast<int64_t>(n) * p.block < p.Tk);
      const uint32_t bal = __ballot_sync(0xffffffffu, ok);
      if (ok) lists[warp][nvalid + __popc(bal & ((1u << lane) - 1u))] = n;
      nvalid += __popc(bal);
    }
    __syncwarp();
  }
  const __nv_bfloat16* Kb = p.k + static_cast<int64_t>(bh) * p.Tk * 64;
  const __nv_bfloat16* Vb = p.v + static_cast<int64_t>(bh) * p.Tk * 64;

  // Q and dO fragments (through stage 0)
  uint32_t qf[4][4], dof[4][4];
  const int qrows = min(16, p.Tq - row0);
  load_tile16(sm0, p.q + (static_cast<int64_t>(bh) * p.Tq + row0) * 64, qrows, lane);
  load_tile16(sm0 + kTile, p.d_o + (static_cast<int64_t>(bh) * p.Tq + row0) * 64, qrows, lane);
  cp_async_commit();
  cp_async_wait<0>();
  __syncwarp();
  load_a_frags(qf, sm0, lane);
  load_a_frags(dof, sm0 + kTile, lane);
  __syncwarp();
  float lse2[2], delta[2];
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const int t = row0 + g + 8 * r;
    float l = (t < p.Tq) ? p.lse[static_cast<int64_t>(bh) * p.Tq + t] : INFINITY;
    if (l == -INFINITY) l = INFINITY;                 // row without any valid key: no gradient
    lse2[r] = l * 1.4426950408889634f;
    delta[r] = (t < p.Tq) ? p.delta[static_cast<int64_t>(bh) * p.Tq + t] : 0.f;
  }
  float dq[8][4] = {};

  const int spb = p.block / 16;                       // 16-key tiles per key block
  const int ntiles = nvalid * spb;
  auto prefetch = [&](int it) {
    const int tok0 = lists[warp][it / spb] * p.block + (it % spb) * 16;
    const uint32_t dst = (it & 1) ? sm1 : sm0;
    const int nrows = min(16, p.Tk - tok0);
    load_tile16(dst, Kb + static_cast<int64_t>(tok0) * 64, nrows, lane);
    load_tile16(dst + kTile, Vb + static_cast<int64_t>(tok0) * 64, nrows, lane);
    cp_async_commit();
  };
  if (ntiles > 0) prefetch(0);
  for (int it = 0; it < ntiles; ++it) {
    if (it + 1 < ntiles) { prefetch(it + 1); cp_async_wait<1>(); } else { cp_async_wait<0>(); }
    __syncwarp();
    const int tok0 = lists[warp][it / spb] * p.block + (it % spb) * 16;
    const uint32_t cur = (it & 1) ? sm1 : sm0;
    pair_dq(qf, dof, lse2, delta, cur, cur + kTile, min(16, p.Tk - tok0), p.cs, p.scale, dq, lane);
    __syncwarp();
  }
  __nv_bfloat16* out = p.dq + (static_cast<int64_t>(bh) * p.Tq + row0) * 64;
  store_acc_bf16(dq, [&](int r) { return (row0 + r < p.Tq) ? out + r * 64 : nullptr; }, lane);
}

// The loop over the query blocks that selected this key block is a chain of dependent accesses (list
// entry -> row addresses -> rows and their lse/delta), so everything is fetched ahead: the list 32 entries
// at a time into a register per lane (read back with a shuffle), rows and statistics by cp.async into a
// ring kDkdvStages deep.  Nothing in the loop waits for a load it has just issued.
// One warp per CTA: the loop length of a warp is the number of query blocks that selected its key block,
// which varies from warp to warp; warps sharing a CTA would hold its registers and shared memory until the
// longest of them is done.
#ifndef S3R_DKDV_WARPS
#define S3R_DKDV_WARPS 1
#endif
#ifndef S3R_DKDV_MIN_CTAS
#define S3R_DKDV_MIN_CTAS 16               // caps the kernel at 128 registers: 16 instead of 10 warps per SM
#endif
#ifndef S3R_DKDV_STAGES
#define S3R_DKDV_STAGES 3
#endif
constexpr int kDkdvWarps = S3R_DKDV_WARPS;
constexpr int kDkdvStages = S3R_DKDV_STAGES;
constexpr int kDkdvStageBytes = 2 * kTile + 128;          // Q tile, dO tile, 16 x lse | 16 x delta
constexpr int kDkdvSmemBytes = kDkdvWarps * kDkdvStages * kDkdvStageBytes;

__global__ void __launch_bounds__(kDkdvWarps * 32, S3R_DKDV_MIN_CTAS) sel_bwd_dkdv_kernel(const SelBwdParams p) {
  extern __shared__ __align__(16) uint8_t dkdv_smem[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nslices = (p.Tk + 15) / 16;
  const int64_t task = static_cast<int64_t>(blockIdx.x) * kDkdvWarps + warp;
  if (task >= static_cast<int64_t>(p.B) * p.H * nslices) return;
  const int bh = static_cast<int>(task / nslices);
  const int row0 = static_cast<int>(task % nslices) * 16;
  const int n = row0 / p.block;
  uint8_t* my = dkdv_smem + warp * kDkdvStages * kDkdvStageBytes;
  const uint32_t sm0 = smem_u32(my);

  uint32_t kf[4][4], vf[4][4];
  const int krows = min(16, p.Tk - row0);
  load_tile16(sm0, p.k + (static_cast<int64_t>(bh) * p.Tk + row0) * 64, krows, lane);
  load_tile16(sm0 + kTile, p.v + (static_cast<int64_t>(bh) * p.Tk + row0) * 64, krows, lane);
  cp_async_commit();
  cp_async_wait<0>();
  __syncwarp();
  load_a_frags(kf, sm0, lane);
  load_a_frags(vf, sm0 + kTile, lane);
  __syncwarp();

  const int32_t* off = p.offsets + static_cast<int64_t>(bh) * (p.nkb + 1);
  const int beg = off[n], cnt = off[n + 1] - beg;
  const int32_t* ql = p.qids + static_cast<int64_t>(bh) * p.nqb * p.topk + beg;
  const __nv_bfloat16* Qb = p.q + static_cast<int64_t>(bh) * p.Tq * 64;
  const __nv_bfloat16* Db = p.d_o + static_cast<int64_t>(bh) * p.Tq * 64;
  const float* Lb = p.lse + static_cast<int64_t>(bh) * p.Tq;
  const float* Eb = p.delta + static_cast<int64_t>(bh) * p.Tq;

  float dk[8][4] = {}, dv[8][4] = {};
  const int spb = p.block / 16;
  const int ntiles = cnt * spb;
  // list entries of chunk c (32 of them) live in `q_cur`, those of chunk c+1 in `q_nxt`
  int q_chunk = 0;
  int q_cur = (lane < cnt) ? ql[lane] : 0;
  int q_nxt = (32 + lane < cnt) ? ql[32 + lane] : 0;
  auto prefetch = [&](int it) {
    const int qb = it / spb;
    if ((qb >> 5) != q_chunk) {                       // warp-uniform
      q_chunk = qb >> 5;
      q_cur = q_nxt;
      const int j = (q_chunk + 1) * 32 + lane;
      q_nxt = (j < cnt) ? ql[j] : 0;
    }
    const int tok0 = __shfl_sync(0xffffffffu, q_cur, qb & 31) * p.block + (it % spb) * 16;
    const uint32_t dst = sm0 + (it % kDkdvStages) * kDkdvStageBytes;
    const int nrows = max(0, min(16, p.Tq - tok0));
    load_tile16(dst, Qb + static_cast<int64_t>(tok0) * 64, nrows, lane);
    load_tile16(dst + kTile, Db + static_cast<int64_t>(tok0) * 64, nrows, lane);
    // per-query statistics: lanes 0-15 lse, lanes 16-31 delta (a padding query gets 0 and 0: its Q and dO
    // rows are zero as well, so P = 1 meets dO = 0 and dP - delta = 0)
    const int t = tok0 + (lane & 15);
    cp_async4(dst + 2 * kTile + lane * 4, (lane < 16 ? Lb : Eb) + min(t, p.Tq - 1), t < p.Tq);
    cp_async_commit();
  };
#pragma unroll
  for (int a = 0; a < kDkdvStages - 1; ++a) {
    if (a < ntiles) prefetch(a); else cp_async_commit();
  }
  for (int it = 0; it < ntiles; ++it) {
    if (it + kDkdvStages - 1 < ntiles) prefetch(it + kDkdvStages - 1); else cp_async_commit();
    cp_async_wait<kDkdvStages - 1>();
    __syncwarp();
    uint8_t* st = my + (it % kDkdvStages) * kDkdvStageBytes;
    float* stats = reinterpret_cast<float*>(st + 2 * kTile);
    if (lane < 16) {                                  // lse -> lse * log2(e); a row without any valid key: no gradient
      const float l = stats[lane];
      stats[lane] = (l == -INFINITY) ? INFINITY : l * 1.4426950408889634f;
    }
    __syncwarp();
    const uint32_t cur = smem_u32(st);
    pair_dkdv(kf, vf, cur, cur + kTile, stats, stats + 16, p.cs, p.scale, dk, dv, lane);
    __syncwarp();
  }
  __nv_bfloat16* okp = p.dk + (static_cast<int64_t>(bh) * p.Tk + row0) * 64;
  __nv_bfloat16* ovp = p.dv + (static_cast<int64_t>(bh) * p.Tk + row0) * 64;
  store_acc_bf16(dk, [&](int r) { return (row0 + r < p.Tk) ? okp + r * 64 : nullptr; }, lane);
  store_acc_bf16(dv, [&](int r) { return (row0 + r < p.Tk) ? ovp + r * 64 : nullptr; }, lane);
}

static int grid_for(int64_t threads, int block) {
  int64_t b = (threads + block - 1) / block;
  const int64_t cap = static_cast<int64_t>(sm_count()) * 32;
  if (b > cap) b = cap;
  return static_cast<int>(b < 1 ? 1 : b);
}

}  // namespace s3r

using namespace s3r;

extern "C" size_t s3r_csr_workspace_bytes(int B, int H, int Nq, int topk, int Nkb) {
  if (B <= 0 || H <= 0 || Nq <= 0 || topk <= 0 || Nkb <= 0) return 0;
  const size_t bh = static_cast<size_t>(B) * H;
  size_t cursor = (bh * Nkb * sizeof(int32_t) + 255) & ~static_cast<size_t>(255);
  size_t tmp = (bh * Nq * topk * sizeof(int32_t) + 255) & ~static_cast<size_t>(255);
  // queue of the segments longer than a warp: at most one per 33 table entries, plus its counter
  size_t queue = ((bh * Nq * topk / 33 + 2) * sizeof(int32_t) + 255) & ~static_cast<size_t>(255);
  return cursor + tmp + queue;
}

extern "C" int s3r_build_key_csr(const int32_t* idx, int32_t* offsets, int32_t* qids, int B, int H, int Nq, int topk,
                                 int Nkb, void* workspace, size_t workspace_bytes, void* stream) {
  S3R_REQUIRE(idx && offsets && qids && workspace, S3R_ERR_NULL, "s3r_build_key_csr: NULL pointer");
  S3R_REQUIRE(B > 0 && H > 0 && Nq > 0 && topk > 0 && Nkb > 0, S3R_ERR_SHAPE, "s3r_build_key_csr: bad sizes");
  S3R_REQUIRE(workspace_bytes >= s3r_csr_workspace_bytes(B, H, Nq, topk, Nkb), S3R_ERR_TOO_LARGE,
              "s3r_build_key_csr: workspace of %zu bytes is smaller than the %zu needed", workspace_bytes,
              s3r_csr_workspace_bytes(B, H, Nq, topk, Nkb));
  S3R_REQUIRE((reinterpret_cast<uintptr_t>(workspace) & 255) == 0, S3R_ERR_ALIGNMENT,
              "s3r_build_key_csr: workspace must be 256-byte aligned");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int64_t bh = static_cast<int64_t>(B) * H;
  const int64_t per_bh = static_cast<int64_t>(Nq) * topk, total = bh * per_bh;
  int32_t* cursor = static_cast<int32_t*>(workspace);
  int32_t* tmp = reinterpret_cast<int32_t*>(static_cast<uint8_t*>(workspace) +
                                            ((bh * Nkb * sizeof(int32_t) + 255) & ~static_cast<size_t>(255)));
  const int64_t nseg = bh * Nkb;
  S3R_REQUIRE(nseg < (1ll << 31) && total < (1ll << 40), S3R_ERR_TOO_LARGE, "s3r_build_key_csr: table too large");
  int32_t* queue = reinterpret_cast<int32_t*>(reinterpret_cast<uint8_t*>(tmp) +
                                              ((bh * Nq * topk * sizeof(int32_t) + 255) & ~static_cast<size_t>(255)));
  S3R_CUDA(cudaMemsetAsync(offsets, 0, bh * (Nkb + 1) * sizeof(int32_t), st));
  S3R_CUDA(cudaMemsetAsync(queue, 0, sizeof(int32_t), st));
  csr_count_kernel<<<grid_for(total, 256), 256, 0, st>>>(idx, offsets, per_bh, total, Nkb);
  csr_scan_kernel<<<static_cast<unsigned>(bh), 1024, 0, st>>>(offsets, cursor, Nkb);
  csr_fill_kernel<<<grid_for(total, 256), 256, 0, st>>>(idx, cursor, tmp, per_bh, total, Nkb, topk);
  csr_sort_small_kernel<<<static_cast<unsigned>((nseg * 32 + 255) / 256), 256, 0, st>>>(offsets, tmp, qids, per_bh, Nkb,
                                                                                        nseg, queue);
  csr_sort_long_kernel<<<sm_count() * 4, 256, 0, st>>>(idx, offsets, tmp, qids, per_bh, Nkb, topk, queue);
  S3R_CUDA(cudaGetLastError());
  return 0;
}

// ------------------------------------------------------------------------------------------------
// The same index build for callers that cannot allocate device memory.
//
// Some hosts of this library have no allocator to ask: a plug-in running inside another runtime
// that handed out all device memory at start-up, or a latency-critical loop in which a
// cudaMalloc (which synchronises the device) is not acceptable.  For them the scratch of the
// index build lives in the library image itself: a fixed array that every GPU that loads the
// library keeps until the process exits.  Sizes whose scratch does not fit are refused.
//
// In host code the array's name is only a stand-in; its device address is obtained once per
// device with cudaGetSymbolAddress (with that device current) and handed to the kernels.
// ------------------------------------------------------------------------------------------------
static __device__ __align__(256) unsigned char g_csr_static_scratch[S3R_CSR_STATIC_SCRATCH_BYTES];

extern "C" int s3r_build_key_csr_static(const int32_t* idx, int32_t* offsets, int32_t* qids, int B, int H, int Nq,
                                        int topk, int Nkb, void* stream) {
  S3R_REQUIRE(idx && offsets && qids, S3R_ERR_NULL, "s3r_build_key_csr_static: NULL pointer");
  S3R_REQUIRE(B > 0 && H > 0 && Nq > 0 && topk > 0 && Nkb > 0, S3R_ERR_SHAPE, "s3r_build_key_csr_static: bad sizes");
  const size_t need = s3r_csr_workspace_bytes(B, H, Nq, topk, Nkb);
  S3R_REQUIRE(need <= static_cast<size_t>(S3R_CSR_STATIC_SCRATCH_BYTES), S3R_ERR_TOO_LARGE,
              "s3r_build_key_csr_static: this table needs %zu bytes of scratch, the built-in buffer holds %zu; "
              "use s3r_build_key_csr with a caller-provided workspace",
              need, static_cast<size_t>(S3R_CSR_STATIC_SCRATCH_BYTES));
  // set-up, once per device: resolve the device address of the built-in buffer
  static void* dev_ptr[64] = {};
  static std::mutex mu;
  int dev = -1;
  S3R_CUDA(cudaGetDevice(&dev));
  S3R_REQUIRE(dev >= 0 && dev < 64, S3R_ERR_UNSUPPORTED, "s3r_build_key_csr_static: device ordinal %d out of range", dev);
  void* scratch = nullptr;
  {
    std::lock_guard<std::mutex> lock(mu);
    if (!dev_ptr[dev]) {
      void* p = nullptr;
      S3R_CUDA(cudaGetSymbolAddress(&p, g_csr_static_scratch));
      dev_ptr[dev] = p;
    }
    scratch = dev_ptr[dev];
  }
  // What must start at zero (the counter of the long-segment queue) is cleared by the build itself; the scan
  // writes every cursor and the sorts only read slots the fill wrote, so nothing an earlier call left behind
  // is ever read.
  return s3r_build_key_csr(idx, offsets, qids, B, H, Nq, topk, Nkb, scratch, S3R_CSR_STATIC_SCRATCH_BYTES, stream);
}

extern "C" int s3r_delta(const void* o, const void* d_o, float* delta, int64_t rows, int d, void* stream) {
  S3R_REQUIRE(o && d_o && delta, S3R_ERR_NULL, "s3r_delta: NULL pointer");
  S3R_REQUIRE(rows > 0, S3R_ERR_SHAPE, "s3r_delta: rows must be positive");
  S3R_REQUIRE(d == 64, S3R_ERR_UNSUPPORTED, "s3r_delta: head_dim %d not supported (64 only)", d);
  const int64_t blocks = (rows * 8 + 255) / 256;
  delta_kernel<<<static_cast<unsigned>(blocks), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(o), static_cast<const __nv_bfloat16*>(d_o), delta, rows);
  S3R_CUDA(cudaGetLastError());
  return 0;
}

extern "C" int s3r_merge_bwd(const void* dy, const void* gate, int64_t gate_stride_b, int64_t gate_stride_h,
                             int64_t gate_stride_t, const void* o_c, const void* o_s, void* do_s, float* dgate,
                             void* do_c, float* delta_s, int B, int H, int Tq, int d, int block, void* stream) {
  S3R_REQUIRE(dy && gate && o_c && o_s && do_s && dgate && do_c && delta_s, S3R_ERR_NULL, "s3r_merge_bwd: NULL pointer");
  S3R_REQUIRE(B > 0 && H > 0 && Tq > 0 && block > 0, S3R_ERR_SHAPE, "s3r_merge_bwd: bad sizes");
  S3R_REQUIRE(d == 64, S3R_ERR_UNSUPPORTED, "s3r_merge_bwd: head_dim %d not supported (64 only)", d);
  MergeBwdParams p;
  p.dy = static_cast<const __nv_bfloat16*>(dy);
  p.gate = static_cast<const __nv_bfloat16*>(gate);
  p.gsb = gate_stride_b; p.gsh = gate_stride_h; p.gst = gate_stride_t;
  p.o_c = static_cast<const __nv_bfloat16*>(o_c);
  p.o_s = static_cast<const __nv_bfloat16*>(o_s);
  p.do_s = static_cast<__nv_bfloat16*>(do_s);
  p.dgate = dgate;
  p.do_c = static_cast<__nv_bfloat16*>(do_c);
  p.delta_s = delta_s;
  p.B = B; p.H = H; p.Tq = Tq; p.block = block;
  p.nqb = (Tq + block - 1) / block;
  const int64_t warps = static_cast<int64_t>(B) * H * p.nqb;
  merge_bwd_kernel<<<static_cast<unsigned>((warps * 32 + 255) / 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(p);
  S3R_CUDA(cudaGetLastError());
  return 0;
}

extern "C" int s3r_sel_attn_bwd(const void* q, const void* k, const void* v, const int32_t* idx,
                                const int32_t* offsets, const int32_t* qids, const float* lse_s, const float* delta_s,
                                const void* do_s, void* dq, void* dk, void* dv, int B, int H, int Tq, int Tk, int d,
                                int block, int topk, float scale, void* stream) {
  S3R_REQUIRE(q && k && v && idx && offsets && qids && lse_s && delta_s && do_s && dq && dk && dv, S3R_ERR_NULL,
              "s3r_sel_attn_bwd: NULL pointer");
  S3R_REQUIRE(B > 0 && H > 0 && Tq > 0 && Tk > 0 && topk > 0, S3R_ERR_SHAPE, "s3r_sel_attn_bwd: bad sizes");
  S3R_REQUIRE(d == 64, S3R_ERR_UNSUPPORTED, "s3r_sel_attn_bwd: head_dim %d not supported (64 only)", d);
  S3R_REQUIRE(block == 16 || block == 32 || block == 64, S3R_ERR_UNSUPPORTED,
              "s3r_sel_attn_bwd: block %d not supported (16, 32, 64)", block);
  S3R_REQUIRE(topk <= 64, S3R_ERR_UNSUPPORTED, "s3r_sel_attn_bwd: topk %d exceeds 64", topk);
  SelBwdParams p;
  p.q = static_cast<const __nv_bfloat16*>(q);
  p.k = static_cast<const __nv_bfloat16*>(k);
  p.v = static_cast<const __nv_bfloat16*>(v);
  p.d_o = static_cast<const __nv_bfloat16*>(do_s);
  p.idx = idx; p.offsets = offsets; p.qids = qids;
  p.lse = lse_s; p.delta = delta_s;
  p.dq = static_cast<__nv_bfloat16*>(dq);
  p.dk = static_cast<__nv_bfloat16*>(dk);
  p.dv = static_cast<__nv_bfloat16*>(dv);
  p.B = B; p.H = H; p.Tq = Tq; p.Tk = Tk; p.block = block; p.topk = topk;
  p.nqb = (Tq + block - 1) / block;
  p.nkb = (Tk + block - 1) / block;
  p.cs = scale * 1.4426950408889634f;
  p.scale = scale;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int64_t bh = static_cast<int64_t>(B) * H;
  const int64_t tq = bh * ((Tq + 15) / 16), tk = bh * ((Tk + 15) / 16);
  S3R_CUDA(cudaFuncSetAttribute(sel_bwd_dkdv_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kDkdvSmemBytes));
  S3R_REQUIRE((tk + kDkdvWarps - 1) / kDkdvWarps < (1ll << 31), S3R_ERR_TOO_LARGE, "s3r_sel_attn_bwd: grid too large");
  sel_bwd_dkdv_kernel<<<static_cast<unsigned>((tk + kDkdvWarps - 1) / kDkdvWarps), kDkdvWarps * 32, kDkdvSmemBytes, st>>>(p);
  sel_bwd_dq_kernel<<<static_cast<unsigned>((tq + kBwdWarps - 1) / kBwdWarps), kBwdWarps * 32, 0, st>>>(p);
  S3R_CUDA(cudaGetLastError());
  return 0;
}
