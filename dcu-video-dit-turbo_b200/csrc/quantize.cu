// Rowwise bf16 -> int8 quantizer and the fused SwiGLU + quantizer for sm_100a.
//
// Both are HBM-bound: every input byte is read from HBM exactly once with 128-bit
// streaming loads, the row stays in registers between the absmax reduction and
// the quantisation, and int8 output leaves as 64-bit stores.  A row is owned by
// TPR threads (one warp or a few), so the reduction is a handful of shuffles
// (plus one shared-memory hop when a row spans warps).
//
// Arithmetic contract (bit-exact):
//   kernels/exact-rowwise-int8/quantizer_kernel.hip:17-21,67-104 (reference)
//   kernels/swiglu-quant/swiglu_quant_kernel.hip:18-27,43-44     (reference)
#include "b2_common.cuh"

namespace b2 {
namespace {

constexpr int kThreads = 256;

// Reduce a NaN-propagating max over the TPR threads that own one row and return
// it to all of them.  TPR is a power of two in [32, 256].
template <int TPR>
__device__ __forceinline__ float row_allreduce_max(float v, float* smem) {
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) v = nanmax(v, __shfl_xor_sync(0xffffffffu, v, off));
  if constexpr (TPR > 32) {
    constexpr int WPR = TPR / 32;  // warps per row
    const int warp = threadIdx.x >> 5;
    if ((threadIdx.x & 31) == 0) smem[warp] = v;
    __syncthreads();
    const int first = (warp / WPR) * WPR;
    float m = smem[first];
#pragma unroll
    for (int i = 1; i < WPR; ++i) m = nanmax(m, smem[first + i]);
    v = m;
  }
  return v;
}

// Where a row's vectors come from.  Contiguous: x[row, :].  Gathered: the row is spread
// over world*chunks segments of seg_vec vectors in a buffer laid out
// [chunks][world][M][seg_vec] (what the reverse all-to-all of sequence-parallel attention
// delivers: segment (p, ch) holds heads p*H/world + ch*c .. +c of the row), so the
// quantizer reads the exchange buffer in place and no unpack copy is made.
struct RowGather {
  int seg_vec;   // 0: contiguous
  int chunks;
  int world;
};
// Offset of row 0's vector c, and the distance between consecutive rows: the segment
// arithmetic (two integer divisions) runs once per thread, outside the row loop.
__device__ __forceinline__ int64_t source_vec0(const RowGather& g, int64_t M, int c) {
  if (g.seg_vec == 0) return c;
  const int seg = c / g.seg_vec, w = c - seg * g.seg_vec;
  const int p = seg / g.chunks, ch = seg - p * g.chunks;
  return ((int64_t)ch * g.world + p) * M * g.seg_vec + w;
}

// One row per TPR threads, VPT 16-byte vectors (8 bf16) per thread, K % 8 == 0,
// K <= TPR*VPT*8.  Rows are assigned round-robin to row slots over a grid-stride
// loop so a fixed, SM-count-sized grid covers any M.
template <int TPR, int VPT>
__global__ void __launch_bounds__(kThreads)
quantize_rows_kernel(const uint4* __restrict__ x, uint2* __restrict__ q, float* __restrict__ scales,
                     int64_t M, int kvec, const RowGather gather) {
  __shared__ float red[kThreads / 32];
  constexpr int RPC = kThreads / TPR;  // rows per CTA per iteration
  const int slot = threadIdx.x / TPR;
  const int lane = threadIdx.x % TPR;
  const int64_t row_step = gather.seg_vec == 0 ? kvec : gather.seg_vec;
  int64_t src0[VPT];
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int c = lane + i * TPR;
    src0[i] = c < kvec ? source_vec0(gather, M, c) : 0;
  }
  for (int64_t row0 = (int64_t)blockIdx.x * RPC; row0 < M; row0 += (int64_t)gridDim.x * RPC) {
    const int64_t row = row0 + slot;
    const bool live = row < M;
    uint4 v[VPT];
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int c = lane + i * TPR;
      v[i] = (live && c < kvec) ? ldg_stream(x + src0[i] + row * row_step) : make_uint4(0, 0, 0, 0);
    }
    uint32_t acc = v[0].x;   // the chain starts from data (see absmax_bf16x2)
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      if (i != 0) acc = absmax_bf16x2(acc, v[i].x);
      acc = absmax_bf16x2(acc, v[i].y);
      acc = absmax_bf16x2(acc, v[i].z);
      acc = absmax_bf16x2(acc, v[i].w);
    }
    const float absmax = row_allreduce_max<TPR>(fold_absmax(acc), red);
    float r;
    bool zero_row;
    const float scale = row_scale_from_absmax(absmax, &r, &zero_row);
    if (live) {
      if (lane == 0) scales[row] = scale;
      uint2* qr = q + row * kvec;
#pragma unroll
      for (int i = 0; i < VPT; ++i) {
        const int c = lane + i * TPR;
        if (c < kvec) qr[c] = zero_row ? make_uint2(0, 0) : quant_vec8(v[i], r);
      }
    }
    if constexpr (TPR > 32) __syncthreads();  // `red` is reused next iteration
  }
}

// Fallback for any K (odd widths, huge rows): one CTA per row, scalar loads, the
// row is read twice (the second read comes from L2).
__global__ void __launch_bounds__(kThreads)
quantize_rows_generic_kernel(const __nv_bfloat16* __restrict__ x, int8_t* __restrict__ q,
                             float* __restrict__ scales, int64_t M, int64_t K) {
  __shared__ float red[kThreads / 32];
  for (int64_t row = blockIdx.x; row < M; row += gridDim.x) {
    const __nv_bfloat16* xr = x + row * K;
    float m = 0.0f;
    for (int64_t c = threadIdx.x; c < K; c += kThreads) m = nanmax(m, fabsf(__bfloat162float(xr[c])));
    const float absmax = row_allreduce_max<kThreads>(m, red);
    float r;
    bool zero_row;
    const float scale = row_scale_from_absmax(absmax, &r, &zero_row);
    if (threadIdx.x == 0) scales[row] = scale;
    for (int64_t c = threadIdx.x; c < K; c += kThreads) {
      const uint32_t w = (uint32_t)__bfloat16_as_ushort(xr[c]);
      q[row * K + c] = zero_row ? (int8_t)0 : (int8_t)(quant_pair(w, r) & 0xffu);
    }
    __syncthreads();
  }
}

__global__ void fill_f32_kernel(float* p, int64_t n, float v) {
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n;
       i += (int64_t)gridDim.x * blockDim.x)
    p[i] = v;
}

// ---- SwiGLU + quantizer ------------------------------------------------------

// bf16(silu(g)) depends on the 16 bits of the bf16 gate alone, so the whole function is a
// table of 65536 bf16 values (128 KB).  It is built once per device from the exact formula
// above and every CTA of the row kernel keeps a copy in shared memory: the first rounding of
// the operator then costs one shared-memory load per element instead of two trips through
// the transcendental unit (exp2, reciprocal) plus the bookkeeping that made their result
// bit-exact, and it is exact by construction for every gate, NaN and infinities included.
constexpr int kSiluEntries = 65536;
__device__ __align__(16) uint16_t g_silu_bf16[kSiluEntries];

__global__ void build_silu_table_kernel() {
  const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < (uint32_t)kSiluEntries)
    g_silu_bf16[i] = __bfloat16_as_ushort(__float2bfloat16_rn(silu_exact(__uint_as_float(i << 16))));
}

// swiglu_pair_exact (b2_common.cuh) is the same from the exact formula (generic kernel).
// The same through the table in shared memory.
__device__ __forceinline__ uint32_t swiglu_pair_lut(uint32_t g, uint32_t u, const uint16_t* lut) {
  const uint32_t s = (uint32_t)lut[g & 0xffffu] | ((uint32_t)lut[g >> 16] << 16);
  return bf16x2_mul_rn(s, u);
}

constexpr int kSwigluThreads = 512;
constexpr int kSwigluSmem = kSiluEntries * 2;   // dynamic shared memory: the table

// FULL: the row fills every vector of every thread (K == TPR*VPT*8): no per-vector range tests.
template <int TPR, int VPT, bool FULL>
__global__ void __launch_bounds__(kSwigluThreads, 1)
swiglu_quantize_rows_kernel(const uint4* __restrict__ x, uint2* __restrict__ q,
                            float* __restrict__ scales, int64_t M, int kvec) {
  extern __shared__ __align__(16) uint16_t lut[];
  __shared__ float red[3][kSwigluThreads / 32];   // three reduction buffers in rotation (slot_allreduce)
  {
    const uint4* src = reinterpret_cast<const uint4*>(g_silu_bf16);
    uint4* dst = reinterpret_cast<uint4*>(lut);
    for (int i = threadIdx.x; i < kSwigluSmem / 16; i += kSwigluThreads) dst[i] = src[i];
  }
  __syncthreads();
  constexpr int RPC = kSwigluThreads / TPR;
  const int slot = threadIdx.x / TPR;
  const int lane = threadIdx.x % TPR;
  // The next row's vectors are requested before the current row is processed, so the loads
  // of one row overlap the arithmetic and the stores of the previous one.
  auto load_row = [&](int64_t row, uint4 (&g)[VPT], uint4 (&u)[VPT]) {
    const bool live = row < M;
    const uint4* gr = x + row * (2 * (int64_t)kvec);  // gate half
    const uint4* ur = gr + kvec;                       // up half
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int c = lane + i * TPR;
      const bool ok = live && (FULL || c < kvec);
      g[i] = ok ? ldg_stream(gr + c) : make_uint4(0, 0, 0, 0);
      u[i] = ok ? ldg_stream(ur + c) : make_uint4(0, 0, 0, 0);
    }
  };
  const int64_t stride = (int64_t)gridDim.x * RPC;
  uint4 g[VPT], u[VPT];
  load_row((int64_t)blockIdx.x * RPC + slot, g, u);
  int phase = 0;
  for (int64_t row0 = (int64_t)blockIdx.x * RPC; row0 < M; row0 += stride) {
    const int64_t row = row0 + slot;
    const bool live = row < M;
    uint4 gn[VPT], un[VPT];
    load_row(row + stride, gn, un);
    uint4 a[VPT];
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      a[i].x = swiglu_pair_lut(g[i].x, u[i].x, lut);
      a[i].y = swiglu_pair_lut(g[i].y, u[i].y, lut);
      a[i].z = swiglu_pair_lut(g[i].z, u[i].z, lut);
      a[i].w = swiglu_pair_lut(g[i].w, u[i].w, lut);
    }
    uint32_t acc = a[0].x;   // the chain starts from data (see absmax_bf16x2)
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      if (i != 0) acc = absmax_bf16x2(acc, a[i].x);
      acc = absmax_bf16x2(acc, a[i].y);
      acc = absmax_bf16x2(acc, a[i].z);
      acc = absmax_bf16x2(acc, a[i].w);
    }
    const float absmax = slot_allreduce<kSwigluThreads, TPR>(fold_absmax(acc), red[phase], slot, NanMaxOp());
    phase = phase == 2 ? 0 : phase + 1;
    float r;
    bool zero_row;
    const float scale = row_scale_from_absmax(absmax, &r, &zero_row);
    if (live) {
      if (lane == 0) scales[row] = scale;
      uint2* qr = q + row * kvec;
#pragma unroll
      for (int i = 0; i < VPT; ++i) {
        const int c = lane + i * TPR;
        if (FULL || c < kvec) qr[c] = zero_row ? make_uint2(0, 0) : quant_vec8(a[i], r);
      }
    }
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      g[i] = gn[i];
      u[i] = un[i];
    }
  }
}

// Fallback for any K: one CTA per row, activated values recomputed in pass 2.
__global__ void __launch_bounds__(kThreads)
swiglu_quantize_rows_generic_kernel(const __nv_bfloat16* __restrict__ x, int8_t* __restrict__ q,
                                    float* __restrict__ scales, int64_t M, int64_t K) {
  __shared__ float red[kThreads / 32];
  for (int64_t row = blockIdx.x; row < M; row += gridDim.x) {
    const __nv_bfloat16* gr = x + row * 2 * K;
    const __nv_bfloat16* ur = gr + K;
    float m = 0.0f;
    for (int64_t c = threadIdx.x; c < K; c += kThreads) {
      const uint32_t a = swiglu_pair_exact(__bfloat16_as_ushort(gr[c]), __bfloat16_as_ushort(ur[c]));
      m = nanmax(m, fabsf(bf16lo_to_f32(a)));
    }
    const float absmax = row_allreduce_max<kThreads>(m, red);
    float r;
    bool zero_row;
    const float scale = row_scale_from_absmax(absmax, &r, &zero_row);
    if (threadIdx.x == 0) scales[row] = scale;
    for (int64_t c = threadIdx.x; c < K; c += kThreads) {
      const uint32_t a = swiglu_pair_exact(__bfloat16_as_ushort(gr[c]), __bfloat16_as_ushort(ur[c]));
      q[row * K + c] = zero_row ? (int8_t)0 : (int8_t)(quant_pair(a & 0xffffu, r) & 0xffu);
    }
    __syncthreads();
  }
}

int grid_for_rows(int64_t M, int rows_per_cta, int ctas_per_sm) {
  int64_t need = (M + rows_per_cta - 1) / rows_per_cta;
  int64_t cap = (int64_t)kNumSMsB200 * ctas_per_sm;
  return (int)(need < cap ? need : cap);
}

}  // namespace

// Picks the register-resident variant for K, or the generic kernel.  world > 0 selects the
// gathered source layout [chunks][world][M][K / (world*chunks)] (vector path only; the
// caller has checked the shape).
int launch_quantize_gathered(const void* x, int8_t* q, float* scale, int64_t M, int64_t K, int world,
                             int chunks, cudaStream_t stream) {
  const bool vec_ok = (K % 8 == 0) && aligned16(x) && ((reinterpret_cast<uintptr_t>(q) & 7u) == 0);
  const int kvec = (int)(K / 8);
  RowGather gather{0, 1, 1};
  if (world > 0) {
    if (!vec_ok || K > 16384) return fail(B2_BAD_SHAPE, "quantize_int8_rowwise_gathered: K must be a multiple of 8, at most 16384");
    gather = RowGather{kvec / (world * chunks), chunks, world};
  }
#define B2_Q(TPR, VPT)                                                                     \
  quantize_rows_kernel<TPR, VPT><<<grid_for_rows(M, kThreads / TPR, 8), kThreads, 0, stream>>>( \
      (const uint4*)x, (uint2*)q, scale, M, kvec, gather)
  if (vec_ok && K <= 1024) B2_Q(32, 4);
  else if (vec_ok && K <= 2048) B2_Q(32, 8);
  else if (vec_ok && K <= 3072) B2_Q(32, 12);
  else if (vec_ok && K <= 4096) B2_Q(64, 8);
  else if (vec_ok && K <= 6144) B2_Q(64, 12);
  else if (vec_ok && K <= 8192) B2_Q(128, 8);
  else if (vec_ok && K <= 16384) B2_Q(256, 8);
  else
    quantize_rows_generic_kernel<<<grid_for_rows(M, 1, 8), kThreads, 0, stream>>>(
        (const __nv_bfloat16*)x, q, scale, M, K);
#undef B2_Q
  return check_launch("quantize_int8_rowwise");
}

int launch_quantize(const void* x, int8_t* q, float* scale, int64_t M, int64_t K,
                    cudaStream_t stream) {
  return launch_quantize_gathered(x, q, scale, M, K, 0, 1, stream);
}

namespace {

// Once per device: build the SiLU table (and wait for it, so that a first call from another
// stream of the same device cannot run ahead of it).  The wait makes the very first call on a
// device unsuitable for a stream capture; every later call only enqueues.
int ensure_silu_table(cudaStream_t stream) {
  static PerDeviceSetup per_device;
  const DeviceSlot* slot = nullptr;
  return per_device.get("swiglu_quantize_int8_rowwise", [stream](int, DeviceSlot&) -> int {
    build_silu_table_kernel<<<kSiluEntries / 256, 256, 0, stream>>>();
    int st = check_launch("swiglu_quantize_int8_rowwise (table)");
    if (st != B2_OK) return st;
    const cudaError_t e = cudaStreamSynchronize(stream);
    if (e != cudaSuccess)
      return fail(B2_LAUNCH_FAILED, "swiglu_quantize_int8_rowwise: building the SiLU table: %s (the first "
                  "call on a device must come before any stream capture)", cudaGetErrorString(e));
    return B2_OK;
  }, &slot);
}

template <int TPR, int VPT>
int launch_swiglu_rows(const void* x, int8_t* q, float* scale, int64_t M, int kvec, cudaStream_t stream) {
  static PerDeviceSetup per_device;   // one per instantiation: the shared-memory opt-in is per kernel and device
  const DeviceSlot* slot = nullptr;
  const int st = per_device.get("swiglu_quantize_int8_rowwise", [](int dev, DeviceSlot& s) -> int {
    cudaError_t e = cudaFuncSetAttribute(swiglu_quantize_rows_kernel<TPR, VPT, true>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, kSwigluSmem);
    if (e == cudaSuccess)
      e = cudaFuncSetAttribute(swiglu_quantize_rows_kernel<TPR, VPT, false>,
                               cudaFuncAttributeMaxDynamicSharedMemorySize, kSwigluSmem);
    if (e != cudaSuccess) return fail(B2_LAUNCH_FAILED, "swiglu_quantize_int8_rowwise: smem attribute: %s", cudaGetErrorString(e));
    s.a = kNumSMsB200;
    cudaDeviceGetAttribute(&s.a, cudaDevAttrMultiProcessorCount, dev);
    return B2_OK;
  }, &slot);
  if (st != B2_OK) return st;
  constexpr int RPC = kSwigluThreads / TPR;
  const int64_t need = (M + RPC - 1) / RPC;
  const int grid = (int)(need < slot->a ? need : slot->a);   // one CTA per SM (its table fills the shared memory)
  if (kvec == TPR * VPT)
    swiglu_quantize_rows_kernel<TPR, VPT, true><<<grid, kSwigluThreads, kSwigluSmem, stream>>>(
        (const uint4*)x, (uint2*)q, scale, M, kvec);
  else
    swiglu_quantize_rows_kernel<TPR, VPT, false><<<grid, kSwigluThreads, kSwigluSmem, stream>>>(
        (const uint4*)x, (uint2*)q, scale, M, kvec);
  return check_launch("swiglu_quantize_int8_rowwise");
}

}  // namespace

// The device address of the table on the current device (built first if need be), for
// kernels of other translation units that look SiLU up in global memory.
int silu_table_device_pointer(cudaStream_t stream, const uint16_t** table) {
  const int st = ensure_silu_table(stream);
  if (st != B2_OK) return st;
  void* p = nullptr;
  const cudaError_t e = cudaGetSymbolAddress(&p, g_silu_bf16);
  if (e != cudaSuccess) return fail(B2_LAUNCH_FAILED, "SiLU table address: %s", cudaGetErrorString(e));
  *table = reinterpret_cast<const uint16_t*>(p);
  return B2_OK;
}


int launch_swiglu_quantize(const void* x, int8_t* q, float* scale, int64_t M, int64_t K,
                           cudaStream_t stream) {
  const bool vec_ok = (K % 8 == 0) && aligned16(x) && ((reinterpret_cast<uintptr_t>(q) & 7u) == 0);
  const int kvec = (int)(K / 8);
  if (vec_ok && K <= 16384) {
    const int st = ensure_silu_table(stream);
    if (st != B2_OK) return st;
    if (K <= 1024) return launch_swiglu_rows<32, 4>(x, q, scale, M, kvec, stream);
    if (K <= 2048) return launch_swiglu_rows<64, 4>(x, q, scale, M, kvec, stream);
    if (K <= 4096) return launch_swiglu_rows<128, 4>(x, q, scale, M, kvec, stream);
    if (K <= 8192) return launch_swiglu_rows<256, 4>(x, q, scale, M, kvec, stream);
    return launch_swiglu_rows<512, 4>(x, q, scale, M, kvec, stream);
  }
  swiglu_quantize_rows_generic_kernel<<<grid_for_rows(M, 1, 8), kThreads, 0, stream>>>(
      (const __nv_bfloat16*)x, q, scale, M, K);
  return check_launch("swiglu_quantize_int8_rowwise");
}

int launch_fill_f32(float* p, int64_t n, float v, cudaStream_t stream) {
  if (n <= 0) return B2_OK;
  int64_t blocks = (n + 255) / 256;
  if (blocks > 1024) blocks = 1024;
  fill_f32_kernel<<<(int)blocks, 256, 0, stream>>>(p, n, v);
  return check_launch("fill_f32");
}

}  // namespace b2
