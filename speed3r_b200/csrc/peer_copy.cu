// Gather of peers' shards for the sequence-partitioned op: a copy kernel of FEW CTAs that pulls from
// peer memory (mapped through CUDA IPC) with plain 16-byte loads and stores locally.
//
// Why a kernel of its own: the exchange of token-level K/V (3.6 GB received per rank at 8 GPUs) should run
// beside the compression attention, which needs only pooled data.  The compression kernel fills every SM
// (all shared memory, nearly all registers), and both an NCCL all-gather and a driver peer copy of
// IPC-mapped memory are SM kernels whose CTAs then either wait for it or hold it back.  This kernel is
// launched first with a small, fixed number of CTAs: those SMs are busy pulling for a few milliseconds,
// all others run the attention from the start.  Bound: NVLink (about 0.74 TB/s into one GPU); a CTA keeps
// 16 loads of 16 bytes per thread in flight to cover the link latency.
// Peers' memory is only ever the source of plain loads.
#include <cstring>

#include "common.cuh"

namespace s3r {

constexpr int kPullMaxSeg = 16;
constexpr int kPullThreads = 512;
constexpr int kPullUnroll = 16;

struct PullParams {
  const uint4* src[kPullMaxSeg];
  uint4* dst[kPullMaxSeg];
  int64_t n16[kPullMaxSeg];       // 16-byte vectors per segment
  int nseg;
};

__global__ void __launch_bounds__(kPullThreads) peer_pull_kernel(const PullParams p) {
  // Segments are interleaved over the CTAs in blocks of kPullThreads*kPullUnroll vectors, so that every
  // CTA reads from every peer all the time (each peer's link carries the same share).
  const int64_t blk = static_cast<int64_t>(kPullThreads) * kPullUnroll;
  for (int s = 0; s < p.nseg; ++s) {
    const uint4* __restrict__ src = p.src[s];
    uint4* __restrict__ dst = p.dst[s];
    const int64_t n = p.n16[s];
    for (int64_t base = static_cast<int64_t>((blockIdx.x + s) % gridDim.x) * blk; base < n;
         base += static_cast<int64_t>(gridDim.x) * blk) {
      uint4 v[kPullUnroll];
#pragma unroll
      for (int u = 0; u < kPullUnroll; ++u) {
        const int64_t i = base + static_cast<int64_t>(u) * kPullThreads + threadIdx.x;
        if (i < n) v[u] = src[i];
      }
#pragma unroll
      for (int u = 0; u < kPullUnroll; ++u) {
        const int64_t i = base + static_cast<int64_t>(u) * kPullThreads + threadIdx.x;
        if (i < n) dst[i] = v[u];
      }
    }
  }
}

}  // namespace s3r

using namespace s3r;

// Export / import of a device buffer between the processes of one node (CUDA IPC).  The importing side
// opens the handle with ITS OWN device current and lazy peer access, so that the returned address can be
// dereferenced by kernels of that device (a mapping opened under the exporter's device could not).
typedef CUresult (*GetAddressRangeFn)(CUdeviceptr*, size_t*, CUdeviceptr);

extern "C" int s3r_ipc_export(const void* ptr, void* handle64, int64_t* offset) {
  S3R_REQUIRE(ptr && handle64 && offset, S3R_ERR_NULL, "s3r_ipc_export: NULL pointer");
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "handle size");
  void* fn = nullptr;
  cudaDriverEntryPointQueryResult q;
  S3R_CUDA(cudaGetDriverEntryPoint("cuMemGetAddressRange", &fn, cudaEnableDefault, &q));
  S3R_REQUIRE(fn != nullptr && q == cudaDriverEntryPointSuccess, S3R_ERR_DRIVER, "s3r_ipc_export: cuMemGetAddressRange not available");
  CUdeviceptr base = 0;
  size_t size = 0;
  const CUresult r = reinterpret_cast<GetAddressRangeFn>(fn)(&base, &size, reinterpret_cast<CUdeviceptr>(ptr));
  S3R_REQUIRE(r == CUDA_SUCCESS, S3R_ERR_DRIVER, "s3r_ipc_export: cuMemGetAddressRange failed (%d)", static_cast<int>(r));
  cudaIpcMemHandle_t h;
  S3R_CUDA(cudaIpcGetMemHandle(&h, reinterpret_cast<void*>(base)));
  memcpy(handle64, &h, sizeof(h));
  *offset = static_cast<int64_t>(reinterpret_cast<CUdeviceptr>(ptr) - base);
  return 0;
}

extern "C" int s3r_ipc_import(const void* handle64, int64_t offset, void** ptr) {
  S3R_REQUIRE(handle64 && ptr && offset >= 0, S3R_ERR_NULL, "s3r_ipc_import: bad arguments");
  cudaIpcMemHandle_t h;
  memcpy(&h, handle64, sizeof(h));
  void* base = nullptr;
  S3R_CUDA(cudaIpcOpenMemHandle(&base, h, cudaIpcMemLazyEnablePeerAccess));
  *ptr = static_cast<uint8_t*>(base) + offset;
  return 0;
}

extern "C" int s3r_peer_pull(const void* const* src, void* const* dst, const int64_t* bytes, int nseg, int ctas,
                             void* stream) {
  S3R_REQUIRE(src && dst && bytes, S3R_ERR_NULL, "s3r_peer_pull: NULL pointer");
  S3R_REQUIRE(nseg >= 1 && nseg <= kPullMaxSeg, S3R_ERR_SHAPE, "s3r_peer_pull: %d segments (1..%d)", nseg, kPullMaxSeg);
  S3R_REQUIRE(ctas >= 1 && ctas <= 1024, S3R_ERR_SHAPE, "s3r_peer_pull: %d CTAs (1..1024)", ctas);
  PullParams p;
  p.nseg = nseg;
  for (int s = 0; s < nseg; ++s) {
    S3R_REQUIRE(src[s] && dst[s], S3R_ERR_NULL, "s3r_peer_pull: NULL segment pointer");
    S3R_REQUIRE(bytes[s] > 0 && (bytes[s] & 15) == 0, S3R_ERR_SHAPE, "s3r_peer_pull: segment sizes must be positive multiples of 16 bytes");
    S3R_REQUIRE(((reinterpret_cast<uintptr_t>(src[s]) | reinterpret_cast<uintptr_t>(dst[s])) & 15) == 0, S3R_ERR_ALIGNMENT,
                "s3r_peer_pull: segments must be 16-byte aligned");
    p.src[s] = static_cast<const uint4*>(src[s]);
    p.dst[s] = static_cast<uint4*>(dst[s]);
    p.n16[s] = bytes[s] >> 4;
  }
  peer_pull_kernel<<<ctas, kPullThreads, 0, static_cast<cudaStream_t>(stream)>>>(p);
  S3R_CUDA(cudaGetLastError());
  return 0;
}
