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
    uint32_t acc = 0;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      acc = absmax_bf16x2(acc, v[i].x);
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

// SiLU in fp32 exactly as the eager op computes it: g / (1 + expf(-g)) with the accurate
// expf and an IEEE division.
__device__ __forceinline__ float silu_exact(float g) {
  return __fdiv_rn(g, __fadd_rn(1.0f, expf(-g)));
}
// Fast SiLU: ex2.approx and rcp.approx instead of expf and the division.  Only its
// ROUNDING TO BF16 has to equal the exact one's.  The exponent argument g*log2(e) is
// carried as a rounded product plus its exact residual (two FMAs on the otherwise idle FMA
// pipe), which keeps the relative error of the fast result within a few fp32 ulps for
// |g| <= 64; whenever the fast fp32 result lies more than 16 ulps away from a bf16 rounding
// midpoint (low 16 bits == 0x8000) both versions therefore round to the same bf16.
// Otherwise *sure is cleared and the caller recomputes exactly (0.05 % of the elements).
// tests/test_gpu_int8_path.py checks the result against the eager op for all 65536 gates.
__device__ __forceinline__ float silu_fast(float g, bool* sure) {
  constexpr float kNegLog2eHi = -1.4426950216293335f;   // fp32(log2 e), negated
  constexpr float kNegLog2eLo = -1.9259629911266175e-8f;  // log2 e - fp32(log2 e), negated
  const float t = g * kNegLog2eHi;
  float r = fmaf(g, kNegLog2eHi, -t);  // exact rounding residual of the product
  r = fmaf(g, kNegLog2eLo, r);
  float e, rc;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(t));
  e = fmaf(e, r * 0.6931471805599453f, e);  // 2^(t+r) = 2^t * (1 + r ln 2)
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(rc) : "f"(1.0f + e));
  const float s = g * rc;
  // |g| <= 64 keeps every intermediate finite and normal (beyond it: exact path)
  *sure = (fabsf(g) <= 64.0f) && (((__float_as_uint(s) & 0xffffu) - (0x8000u - 16u)) > 32u);
  return s;
}

// bf16( bf16(silu(g)) * u ) on a packed pair; two bf16 roundings.
__device__ __forceinline__ uint32_t swiglu_pair(uint32_t g, uint32_t u) {
  const float g0 = bf16lo_to_f32(g), g1 = bf16hi_to_f32(g);
  bool sure0, sure1;
  float s0 = silu_fast(g0, &sure0);
  float s1 = silu_fast(g1, &sure1);
  // A vote over the lanes that are converged here keeps the rare exact path a real branch
  // instead of predicated code.  The mask must be the ACTIVE mask: the scalar fallback
  // kernel calls this from loops whose trip count differs between lanes.
  if (__any_sync(__activemask(), !(sure0 && sure1))) {
    s0 = silu_exact(g0);
    s1 = silu_exact(g1);
  }
  // second rounding: the fp32 product of two bf16 values is exact, so rounding it to bf16 is
  // the packed bf16 multiply's single rounding (one FMA-pipe instruction instead of seven)
  return bf16x2_mul_rn(pack_bf16x2_rn(s0, s1), u);
}

template <int TPR, int VPT>
__global__ void __launch_bounds__(kThreads)
swiglu_quantize_rows_kernel(const uint4* __restrict__ x, uint2* __restrict__ q,
                            float* __restrict__ scales, int64_t M, int kvec) {
  __shared__ float red[kThreads / 32];
  constexpr int RPC = kThreads / TPR;
  const int slot = threadIdx.x / TPR;
  const int lane = threadIdx.x % TPR;
  for (int64_t row0 = (int64_t)blockIdx.x * RPC; row0 < M; row0 += (int64_t)gridDim.x * RPC) {
    const int64_t row = row0 + slot;
    const bool live = row < M;
    const uint4* gr = x + row * (2 * (int64_t)kvec);  // gate half
    const uint4* ur = gr + kvec;                       // up half
    uint4 a[VPT];
    {
      uint4 g[VPT], u[VPT];
#pragma unroll
      for (int i = 0; i < VPT; ++i) {
        const int c = lane + i * TPR;
        const bool ok = live && c < kvec;
        g[i] = ok ? ldg_stream(gr + c) : make_uint4(0, 0, 0, 0);
        u[i] = ok ? ldg_stream(ur + c) : make_uint4(0, 0, 0, 0);
      }
#pragma unroll
      for (int i = 0; i < VPT; ++i) {
        a[i].x = swiglu_pair(g[i].x, u[i].x);
        a[i].y = swiglu_pair(g[i].y, u[i].y);
        a[i].z = swiglu_pair(g[i].z, u[i].z);
        a[i].w = swiglu_pair(g[i].w, u[i].w);
      }
    }
    uint32_t acc = 0;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      acc = absmax_bf16x2(acc, a[i].x);
      acc = absmax_bf16x2(acc, a[i].y);
      acc = absmax_bf16x2(acc, a[i].z);
      acc = absmax_bf16x2(acc, a[i].w);
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
        if (c < kvec) qr[c] = zero_row ? make_uint2(0, 0) : quant_vec8(a[i], r);
      }
    }
    if constexpr (TPR > 32) __syncthreads();
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
      const uint32_t a = swiglu_pair(__bfloat16_as_ushort(gr[c]), __bfloat16_as_ushort(ur[c]));
      m = nanmax(m, fabsf(bf16lo_to_f32(a)));
    }
    const float absmax = row_allreduce_max<kThreads>(m, red);
    float r;
    bool zero_row;
    const float scale = row_scale_from_absmax(absmax, &r, &zero_row);
    if (threadIdx.x == 0) scales[row] = scale;
    for (int64_t c = threadIdx.x; c < K; c += kThreads) {
      const uint32_t a = swiglu_pair(__bfloat16_as_ushort(gr[c]), __bfloat16_as_ushort(ur[c]));
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

int launch_swiglu_quantize(const void* x, int8_t* q, float* scale, int64_t M, int64_t K,
                           cudaStream_t stream) {
  const bool vec_ok = (K % 8 == 0) && aligned16(x) && ((reinterpret_cast<uintptr_t>(q) & 7u) == 0);
  const int kvec = (int)(K / 8);
#define B2_S(TPR, VPT)                                                                   \
  swiglu_quantize_rows_kernel<TPR, VPT>                                                  \
      <<<grid_for_rows(M, kThreads / TPR, 8), kThreads, 0, stream>>>((const uint4*)x, (uint2*)q, \
                                                                     scale, M, kvec)
  if (vec_ok && K <= 1024) B2_S(32, 4);
  else if (vec_ok && K <= 2048) B2_S(64, 4);
  else if (vec_ok && K <= 4096) B2_S(128, 4);
  else if (vec_ok && K <= 8192) B2_S(256, 4);
  else if (vec_ok && K <= 16384) B2_S(256, 8);
  else
    swiglu_quantize_rows_generic_kernel<<<grid_for_rows(M, 1, 8), kThreads, 0, stream>>>(
        (const __nv_bfloat16*)x, q, scale, M, K);
#undef B2_S
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
