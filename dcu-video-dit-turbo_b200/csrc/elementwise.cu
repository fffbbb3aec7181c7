// Column-broadcast elementwise kernels: the standalone INT8 dequant epilogue
// (scalar and 4-wide contracts), mod-scale-shift and the gated residual.
//
// All are HBM-bound.  A thread owns a fixed group of columns, keeps that group's
// per-column operands (column scale, bias, 1+scale, shift, gate) in registers and
// walks down the rows with several independent 128-bit loads in flight, so there
// is no per-element index arithmetic (no `%`) and no row-count grid limit.
//
// Arithmetic contracts (bit-exact):
//   kernels/int8-epilogue/epilogue_kernel.hip:39-53      (reference)
//   kernels/int8-epilogue-vec4/epilogue_kernel.hip:17-30 (reference)
//   kernels/mod-scale-shift/mod_kernel.hip:16-21         (reference)
#include "b2_common.cuh"

namespace b2 {
namespace {

constexpr int kColThreads = 128;
constexpr int kRowUnroll = 4;

__device__ __forceinline__ float bias_as_bf16_f32(const void* bias, int kind, int64_t c) {
  if (kind == B2_BIAS_BF16) return __bfloat162float(((const __nv_bfloat16*)bias)[c]);
  return round_bf16_f32(((const float*)bias)[c]);
}

// out = bf16(float(acc) * (rs*cs)); with bias: bf16(float(out) + bf16(bias)).
__device__ __forceinline__ float dequant_one(int32_t a, float rs, float cs) {
  return __fmul_rn(__int2float_rn(a), __fmul_rn(rs, cs));
}

template <bool HAS_BIAS>
__global__ void __launch_bounds__(kColThreads)
epilogue_vec4_kernel(const int4* __restrict__ acc, const float* __restrict__ rs,
                     const float* __restrict__ cs, const void* __restrict__ bias, int bias_kind,
                     uint2* __restrict__ out, int64_t M, int64_t n4) {
  const int64_t c4 = (int64_t)blockIdx.x * kColThreads + threadIdx.x;
  if (c4 >= n4) return;
  const float4 s = *reinterpret_cast<const float4*>(cs + c4 * 4);
  float b0 = 0.f, b1 = 0.f, b2v = 0.f, b3 = 0.f;
  if (HAS_BIAS) {
    b0 = bias_as_bf16_f32(bias, bias_kind, c4 * 4 + 0);
    b1 = bias_as_bf16_f32(bias, bias_kind, c4 * 4 + 1);
    b2v = bias_as_bf16_f32(bias, bias_kind, c4 * 4 + 2);
    b3 = bias_as_bf16_f32(bias, bias_kind, c4 * 4 + 3);
  }
  const int64_t stride = gridDim.y;
  for (int64_t r0 = blockIdx.y; r0 < M; r0 += stride * kRowUnroll) {
    int4 a[kRowUnroll];
    float rsv[kRowUnroll];
#pragma unroll
    for (int u = 0; u < kRowUnroll; ++u) {
      const int64_t r = r0 + u * stride;
      if (r < M) {
        const uint4 t = ldg_stream(reinterpret_cast<const uint4*>(acc + r * n4 + c4));
        a[u] = make_int4((int)t.x, (int)t.y, (int)t.z, (int)t.w);
        rsv[u] = rs[r];
      }
    }
#pragma unroll
    for (int u = 0; u < kRowUnroll; ++u) {
      const int64_t r = r0 + u * stride;
      if (r < M) {
        float o0 = dequant_one(a[u].x, rsv[u], s.x), o1 = dequant_one(a[u].y, rsv[u], s.y);
        float o2 = dequant_one(a[u].z, rsv[u], s.z), o3 = dequant_one(a[u].w, rsv[u], s.w);
        uint32_t p0 = pack_bf16x2_rn(o0, o1), p1 = pack_bf16x2_rn(o2, o3);
        if (HAS_BIAS) {
          p0 = pack_bf16x2_rn(__fadd_rn(bf16lo_to_f32(p0), b0), __fadd_rn(bf16hi_to_f32(p0), b1));
          p1 = pack_bf16x2_rn(__fadd_rn(bf16lo_to_f32(p1), b2v), __fadd_rn(bf16hi_to_f32(p1), b3));
        }
        out[r * n4 + c4] = make_uint2(p0, p1);
      }
    }
  }
}

// Any N (N % 4 != 0): one column per thread.
template <bool HAS_BIAS>
__global__ void __launch_bounds__(kColThreads)
epilogue_scalar_kernel(const int32_t* __restrict__ acc, const float* __restrict__ rs,
                       const float* __restrict__ cs, const void* __restrict__ bias, int bias_kind,
                       __nv_bfloat16* __restrict__ out, int64_t M, int64_t N) {
  const int64_t c = (int64_t)blockIdx.x * kColThreads + threadIdx.x;
  if (c >= N) return;
  const float s = cs[c];
  const float b = HAS_BIAS ? bias_as_bf16_f32(bias, bias_kind, c) : 0.f;
  for (int64_t r = blockIdx.y; r < M; r += gridDim.y) {
    float o = round_bf16_f32(dequant_one(acc[r * N + c], rs[r], s));
    if (HAS_BIAS) o = __fadd_rn(o, b);
    out[r * N + c] = __float2bfloat16_rn(o);
  }
}

// 8 bf16 per thread: x = bf16(bf16(x*f) + sh), f = bf16(1+scale)
__global__ void __launch_bounds__(kColThreads)
mod_scale_shift_vec8_kernel(uint4* __restrict__ x, const uint4* __restrict__ scale,
                            const uint4* __restrict__ shift, int64_t M, int64_t c8) {
  const int64_t cv = (int64_t)blockIdx.x * kColThreads + threadIdx.x;
  if (cv >= c8) return;
  const uint4 sc = scale[cv], sh = shift[cv];
  float f[8], s[8];
  const uint32_t scw[4] = {sc.x, sc.y, sc.z, sc.w}, shw[4] = {sh.x, sh.y, sh.z, sh.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    f[2 * i] = round_bf16_f32(__fadd_rn(1.0f, bf16lo_to_f32(scw[i])));
    f[2 * i + 1] = round_bf16_f32(__fadd_rn(1.0f, bf16hi_to_f32(scw[i])));
    s[2 * i] = bf16lo_to_f32(shw[i]);
    s[2 * i + 1] = bf16hi_to_f32(shw[i]);
  }
  const int64_t stride = gridDim.y;
  for (int64_t r0 = blockIdx.y; r0 < M; r0 += stride * kRowUnroll) {
    uint4 v[kRowUnroll];
#pragma unroll
    for (int u = 0; u < kRowUnroll; ++u) {
      const int64_t r = r0 + u * stride;
      if (r < M) v[u] = x[r * c8 + cv];
    }
#pragma unroll
    for (int u = 0; u < kRowUnroll; ++u) {
      const int64_t r = r0 + u * stride;
      if (r < M) {
        uint32_t w[4] = {v[u].x, v[u].y, v[u].z, v[u].w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const uint32_t p = pack_bf16x2_rn(__fmul_rn(bf16lo_to_f32(w[i]), f[2 * i]),
                                            __fmul_rn(bf16hi_to_f32(w[i]), f[2 * i + 1]));
          w[i] = pack_bf16x2_rn(__fadd_rn(bf16lo_to_f32(p), s[2 * i]),
                                __fadd_rn(bf16hi_to_f32(p), s[2 * i + 1]));
        }
        x[r * c8 + cv] = make_uint4(w[0], w[1], w[2], w[3]);
      }
    }
  }
}

__global__ void __launch_bounds__(kColThreads)
mod_scale_shift_scalar_kernel(__nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ scale,
                              const __nv_bfloat16* __restrict__ shift, int64_t M, int64_t C) {
  const int64_t c = (int64_t)blockIdx.x * kColThreads + threadIdx.x;
  if (c >= C) return;
  const float f = round_bf16_f32(__fadd_rn(1.0f, __bfloat162float(scale[c])));
  const float s = __bfloat162float(shift[c]);
  for (int64_t r = blockIdx.y; r < M; r += gridDim.y) {
    const float p = round_bf16_f32(__fmul_rn(__bfloat162float(x[r * C + c]), f));
    x[r * C + c] = __float2bfloat16_rn(__fadd_rn(p, s));
  }
}

// x = bf16(x + bf16(g*y)), 8 bf16 per thread
__global__ void __launch_bounds__(kColThreads)
gate_residual_vec8_kernel(uint4* __restrict__ x, const uint4* __restrict__ y,
                          const uint4* __restrict__ gate, int64_t M, int64_t c8) {
  const int64_t cv = (int64_t)blockIdx.x * kColThreads + threadIdx.x;
  if (cv >= c8) return;
  const uint4 gv = gate[cv];
  const uint32_t gw[4] = {gv.x, gv.y, gv.z, gv.w};
  float g[8];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    g[2 * i] = bf16lo_to_f32(gw[i]);
    g[2 * i + 1] = bf16hi_to_f32(gw[i]);
  }
  const int64_t stride = gridDim.y;
  for (int64_t r0 = blockIdx.y; r0 < M; r0 += stride * kRowUnroll) {
    uint4 xv[kRowUnroll], yv[kRowUnroll];
#pragma unroll
    for (int u = 0; u < kRowUnroll; ++u) {
      const int64_t r = r0 + u * stride;
      if (r < M) {
        xv[u] = x[r * c8 + cv];
        yv[u] = ldg_stream(y + r * c8 + cv);
      }
    }
#pragma unroll
    for (int u = 0; u < kRowUnroll; ++u) {
      const int64_t r = r0 + u * stride;
      if (r < M) {
        uint32_t xw[4] = {xv[u].x, xv[u].y, xv[u].z, xv[u].w};
        const uint32_t yw[4] = {yv[u].x, yv[u].y, yv[u].z, yv[u].w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const uint32_t p = pack_bf16x2_rn(__fmul_rn(bf16lo_to_f32(yw[i]), g[2 * i]),
                                            __fmul_rn(bf16hi_to_f32(yw[i]), g[2 * i + 1]));
          xw[i] = pack_bf16x2_rn(__fadd_rn(bf16lo_to_f32(xw[i]), bf16lo_to_f32(p)),
                                 __fadd_rn(bf16hi_to_f32(xw[i]), bf16hi_to_f32(p)));
        }
        x[r * c8 + cv] = make_uint4(xw[0], xw[1], xw[2], xw[3]);
      }
    }
  }
}

__global__ void __launch_bounds__(kColThreads)
gate_residual_scalar_kernel(__nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ y,
                            const __nv_bfloat16* __restrict__ gate, int64_t M, int64_t C) {
  const int64_t c = (int64_t)blockIdx.x * kColThreads + threadIdx.x;
  if (c >= C) return;
  const float g = __bfloat162float(gate[c]);
  for (int64_t r = blockIdx.y; r < M; r += gridDim.y) {
    const float p = round_bf16_f32(__fmul_rn(__bfloat162float(y[r * C + c]), g));
    x[r * C + c] = __float2bfloat16_rn(__fadd_rn(__bfloat162float(x[r * C + c]), p));
  }
}

// 2-D grid: x covers the column groups, y splits the rows so that the whole grid
// is a few CTAs per SM.
dim3 col_grid(int64_t col_groups, int64_t M) {
  int64_t gx = (col_groups + kColThreads - 1) / kColThreads;
  int64_t want = (int64_t)kNumSMsB200 * 16;
  int64_t gy = (want + gx - 1) / gx;
  int64_t max_gy = (M + kRowUnroll - 1) / kRowUnroll;
  if (gy > max_gy) gy = max_gy;
  if (gy < 1) gy = 1;
  if (gy > 65535) gy = 65535;
  return dim3((unsigned)gx, (unsigned)gy, 1);
}

}  // namespace

int launch_epilogue(const int32_t* acc, const float* rs, const float* cs, const void* bias,
                    int bias_kind, void* out, int64_t M, int64_t N, cudaStream_t stream) {
  const bool vec = (N % 4 == 0) && aligned16(acc) && aligned16(cs) &&
                   ((reinterpret_cast<uintptr_t>(out) & 7u) == 0);
  const bool has_bias = bias_kind != B2_BIAS_NONE;
  if (vec) {
    const dim3 g = col_grid(N / 4, M);
    if (has_bias)
      epilogue_vec4_kernel<true><<<g, kColThreads, 0, stream>>>((const int4*)acc, rs, cs, bias,
                                                                bias_kind, (uint2*)out, M, N / 4);
    else
      epilogue_vec4_kernel<false><<<g, kColThreads, 0, stream>>>((const int4*)acc, rs, cs, bias,
                                                                 bias_kind, (uint2*)out, M, N / 4);
  } else {
    const dim3 g = col_grid(N, M);
    if (has_bias)
      epilogue_scalar_kernel<true><<<g, kColThreads, 0, stream>>>(
          acc, rs, cs, bias, bias_kind, (__nv_bfloat16*)out, M, N);
    else
      epilogue_scalar_kernel<false><<<g, kColThreads, 0, stream>>>(
          acc, rs, cs, bias, bias_kind, (__nv_bfloat16*)out, M, N);
  }
  return check_launch("epilogue");
}

int launch_mod_scale_shift(void* x, const void* scale, const void* shift, int64_t M, int64_t C,
                           cudaStream_t stream) {
  const bool vec = (C % 8 == 0) && aligned16(x) && aligned16(scale) && aligned16(shift);
  if (vec) {
    mod_scale_shift_vec8_kernel<<<col_grid(C / 8, M), kColThreads, 0, stream>>>(
        (uint4*)x, (const uint4*)scale, (const uint4*)shift, M, C / 8);
  } else {
    mod_scale_shift_scalar_kernel<<<col_grid(C, M), kColThreads, 0, stream>>>(
        (__nv_bfloat16*)x, (const __nv_bfloat16*)scale, (const __nv_bfloat16*)shift, M, C);
  }
  return check_launch("mod_scale_shift");
}

int launch_gate_residual(void* x, const void* y, const void* gate, int64_t M, int64_t C,
                         cudaStream_t stream) {
  const bool vec = (C % 8 == 0) && aligned16(x) && aligned16(y) && aligned16(gate);
  if (vec) {
    gate_residual_vec8_kernel<<<col_grid(C / 8, M), kColThreads, 0, stream>>>(
        (uint4*)x, (const uint4*)y, (const uint4*)gate, M, C / 8);
  } else {
    gate_residual_scalar_kernel<<<col_grid(C, M), kColThreads, 0, stream>>>(
        (__nv_bfloat16*)x, (const __nv_bfloat16*)y, (const __nv_bfloat16*)gate, M, C);
  }
  return check_launch("gate_residual");
}

}  // namespace b2
