// Peer-memory plumbing for the sequence-parallel exchange on one NVSwitch domain: buffers
// that other ranks' kernels write into directly (plain stores through CUDA IPC mappings),
// and a copy kernel that pushes row blocks to several peers in one launch.
//
// The five b2_peer_* entry points are the only ones in this library that allocate, map or
// free device memory; they are called when a sequence-parallel group is set up or torn
// down, never on the per-step path.  No kernel here waits on another GPU: ordering between
// ranks is the caller's (a collective on the same stream between the writes and the reads).
#include <cuda_runtime.h>

#include <cstring>

#include "b2_common.cuh"
#include "b2_launch.h"

namespace b2 {
namespace {

constexpr int kMaxSegments = 8;
constexpr int kCopyThreads = 256;
constexpr int kCopyUnroll = 4;

struct CopySegments {
  const uint4* src[kMaxSegments];
  uint4* dst[kMaxSegments];
  int64_t vecs[kMaxSegments];
  int n;
};

// Segment after segment, every CTA taking a grid-strided share of 16-byte vectors with four
// loads in flight per thread.  Sources and destinations may be local or peer memory.
__global__ void __launch_bounds__(kCopyThreads)
copy_segments_kernel(const CopySegments seg) {
  const int64_t stride = (int64_t)gridDim.x * kCopyThreads;
  for (int i = 0; i < seg.n; ++i) {
    const uint4* __restrict__ src = seg.src[i];
    uint4* __restrict__ dst = seg.dst[i];
    const int64_t n = seg.vecs[i];
    int64_t v = (int64_t)blockIdx.x * kCopyThreads + threadIdx.x;
    for (; v + (kCopyUnroll - 1) * stride < n; v += kCopyUnroll * stride) {
      uint4 t[kCopyUnroll];
#pragma unroll
      for (int u = 0; u < kCopyUnroll; ++u) t[u] = ldg_stream(src + v + u * stride);
#pragma unroll
      for (int u = 0; u < kCopyUnroll; ++u) dst[v + u * stride] = t[u];
    }
    for (; v < n; v += stride) dst[v] = ldg_stream(src + v);
  }
}

}  // namespace

int launch_copy_segments(const void* const* src, void* const* dst, const int64_t* bytes, int n,
                         cudaStream_t stream) {
  CopySegments seg;
  int64_t most = 0;
  seg.n = 0;
  for (int i = 0; i < n; ++i) {
    if (bytes[i] == 0) continue;
    seg.src[seg.n] = (const uint4*)src[i];
    seg.dst[seg.n] = (uint4*)dst[i];
    seg.vecs[seg.n] = bytes[i] / 16;
    if (seg.vecs[seg.n] > most) most = seg.vecs[seg.n];
    ++seg.n;
  }
  for (int i = seg.n; i < kMaxSegments; ++i) {
    seg.src[i] = nullptr;
    seg.dst[i] = nullptr;
    seg.vecs[i] = 0;
  }
  if (seg.n == 0) return B2_OK;
  const int64_t want = (most + kCopyThreads * kCopyUnroll - 1) / (kCopyThreads * kCopyUnroll);
  const int64_t cap = (int64_t)kNumSMsB200 * 8;
  const int blocks = (int)(want < cap ? (want < 1 ? 1 : want) : cap);
  copy_segments_kernel<<<blocks, kCopyThreads, 0, stream>>>(seg);
  return check_launch("copy_segments");
}

}  // namespace b2

using namespace b2;

extern "C" {

int b2_peer_alloc(int64_t bytes, void** ptr) {
  if (!ptr) return fail(B2_NULL_POINTER, "peer_alloc: ptr is null");
  *ptr = nullptr;
  if (bytes <= 0) return fail(B2_BAD_SHAPE, "peer_alloc: bytes=%lld", (long long)bytes);
  void* p = nullptr;
  cudaError_t e = cudaMalloc(&p, (size_t)bytes);
  if (e != cudaSuccess) {
    cudaGetLastError();
    return fail(B2_TOO_LARGE, "peer_alloc: cudaMalloc(%lld): %s", (long long)bytes, cudaGetErrorString(e));
  }
  e = cudaMemset(p, 0, (size_t)bytes);
  if (e != cudaSuccess) {
    cudaFree(p);
    return fail(B2_LAUNCH_FAILED, "peer_alloc: cudaMemset: %s", cudaGetErrorString(e));
  }
  *ptr = p;
  return B2_OK;
}

int b2_peer_free(void* ptr) {
  if (!ptr) return B2_OK;
  cudaError_t e = cudaFree(ptr);
  if (e != cudaSuccess) return fail(B2_LAUNCH_FAILED, "peer_free: %s", cudaGetErrorString(e));
  return B2_OK;
}

int b2_peer_export(void* ptr, void* handle, int32_t handle_bytes) {
  if (!ptr || !handle) return fail(B2_NULL_POINTER, "peer_export: null pointer");
  if (handle_bytes != (int32_t)sizeof(cudaIpcMemHandle_t))
    return fail(B2_BAD_SHAPE, "peer_export: handle buffer must be %d bytes", (int)sizeof(cudaIpcMemHandle_t));
  cudaIpcMemHandle_t h;
  cudaError_t e = cudaIpcGetMemHandle(&h, ptr);
  if (e != cudaSuccess) {
    cudaGetLastError();
    return fail(B2_LAUNCH_FAILED, "peer_export: cudaIpcGetMemHandle: %s", cudaGetErrorString(e));
  }
  memcpy(handle, &h, sizeof(h));
  return B2_OK;
}

int b2_peer_open(const void* handle, int32_t handle_bytes, void** ptr) {
  if (!handle || !ptr) return fail(B2_NULL_POINTER, "peer_open: null pointer");
  *ptr = nullptr;
  if (handle_bytes != (int32_t)sizeof(cudaIpcMemHandle_t))
    return fail(B2_BAD_SHAPE, "peer_open: handle must be %d bytes", (int)sizeof(cudaIpcMemHandle_t));
  cudaIpcMemHandle_t h;
  memcpy(&h, handle, sizeof(h));
  void* p = nullptr;
  cudaError_t e = cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess);
  if (e != cudaSuccess) {
    cudaGetLastError();
    return fail(B2_LAUNCH_FAILED, "peer_open: cudaIpcOpenMemHandle: %s", cudaGetErrorString(e));
  }
  *ptr = p;
  return B2_OK;
}

int b2_peer_close(void* ptr) {
  if (!ptr) return B2_OK;
  cudaError_t e = cudaIpcCloseMemHandle(ptr);
  if (e != cudaSuccess) {
    cudaGetLastError();
    return fail(B2_LAUNCH_FAILED, "peer_close: cudaIpcCloseMemHandle: %s", cudaGetErrorString(e));
  }
  return B2_OK;
}

int b2_copy_segments(const void* const* src, void* const* dst, const int64_t* bytes, int32_t n,
                     void* stream) {
  if (n < 0 || n > kMaxSegments) return fail(B2_BAD_SHAPE, "copy_segments: n=%d, at most %d segments", n, kMaxSegments);
  if (n == 0) return B2_OK;
  if (!src || !dst || !bytes) return fail(B2_NULL_POINTER, "copy_segments: null table");
  for (int i = 0; i < n; ++i) {
    if (bytes[i] < 0 || bytes[i] % 16) return fail(B2_BAD_SHAPE, "copy_segments: segment %d: %lld bytes (multiple of 16 wanted)", i, (long long)bytes[i]);
    if (bytes[i] == 0) continue;
    if (!src[i] || !dst[i]) return fail(B2_NULL_POINTER, "copy_segments: segment %d: null pointer", i);
    if (!aligned16(src[i]) || !aligned16(dst[i])) return fail(B2_BAD_STRIDE, "copy_segments: segment %d: pointers must be 16-byte aligned", i);
  }
  return launch_copy_segments(src, dst, bytes, n, (cudaStream_t)stream);
}

}  // extern "C"
