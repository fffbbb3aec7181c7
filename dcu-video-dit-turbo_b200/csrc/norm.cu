// DiT-block glue that is row-local: LayerNorm (no affine) + adaLN modulation,
// optionally fused with the rowwise INT8 quantizer (the producer of a GEMM's A
// operand), and per-head QK RMSNorm + rotary embedding on a packed qkv buffer.
//
// The reference project has no source for these operators (they live in the host
// application's model file), so the conventions are this library's own:
//   LayerNorm: fp32 mean and biased variance over the row, (x-mean)*rsqrt(var+eps),
//     rounded once to bf16; then the mod-scale-shift contract (three roundings,
//     kernels/mod-scale-shift/mod_kernel.hip:16-21 in the reference); then, when
//     fused, the rowwise quantizer contract
//     (kernels/exact-rowwise-int8/quantizer_kernel.hip:17-21 in the reference).
//   QK norm + RoPE: y = x*rsqrt(mean(x^2)+eps)*w in fp32, rotation of adjacent
//     pairs (2i,2i+1) by (cos,sin)[row][i], rounded once to bf16.
#include "b2_common.cuh"

namespace b2 {
namespace {

constexpr int kThreads = 256;

template <int TPR>
__device__ __forceinline__ float row_allreduce_sum(float v, float* smem) {
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
  if constexpr (TPR > 32) {
    constexpr int WPR = TPR / 32;
    const int warp = threadIdx.x >> 5;
    __syncthreads();  // previous use of smem is complete
    if ((threadIdx.x & 31) == 0) smem[warp] = v;
    __syncthreads();
    const int first = (warp / WPR) * WPR;
    float s = smem[first];
#pragma unroll
    for (int i = 1; i < WPR; ++i) s += smem[first + i];
    v = s;
  }
  return v;
}

template <int TPR>
__device__ __forceinline__ float row_allreduce_nanmax(float v, float* smem) {
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) v = nanmax(v, __shfl_xor_sync(0xffffffffu, v, off));
  if constexpr (TPR > 32) {
    constexpr int WPR = TPR / 32;
    const int warp = threadIdx.x >> 5;
    __syncthreads();
    if ((threadIdx.x & 31) == 0) smem[warp] = v;
    __syncthreads();
    const int first = (warp / WPR) * WPR;
    float s = smem[first];
#pragma unroll
    for (int i = 1; i < WPR; ++i) s = nanmax(s, smem[first + i]);
    v = s;
  }
  return v;
}

// One row per TPR threads, VPT vectors of 8 bf16 per thread; C % 8 == 0,
// C <= TPR*VPT*8.  QUANT selects the fused quantizer output.
template <int TPR, int VPT, bool QUANT>
__global__ void __launch_bounds__(kThreads, 2)
layernorm_mod_kernel(const uint4* __restrict__ x, const uint4* __restrict__ scale,
                     const uint4* __restrict__ shift, uint4* __restrict__ out_bf16,
                     uint2* __restrict__ out_q, float* __restrict__ out_scale, int64_t M, int cvec,
                     float inv_c, float eps) {
  __shared__ float red[kThreads / 32];
  // per-column operands staged once per CTA: factor = bf16(1+scale) and shift, packed
  // like the data (8 bf16 per uint4)
  extern __shared__ uint4 colvec[];
  uint4* fac_s = colvec;
  uint4* shf_s = colvec + cvec;
  for (int c = threadIdx.x; c < cvec; c += kThreads) {
    const uint4 sc = scale[c];
    uint4 f;
    f.x = pack_bf16x2_rn(__fadd_rn(1.0f, bf16lo_to_f32(sc.x)), __fadd_rn(1.0f, bf16hi_to_f32(sc.x)));
    f.y = pack_bf16x2_rn(__fadd_rn(1.0f, bf16lo_to_f32(sc.y)), __fadd_rn(1.0f, bf16hi_to_f32(sc.y)));
    f.z = pack_bf16x2_rn(__fadd_rn(1.0f, bf16lo_to_f32(sc.z)), __fadd_rn(1.0f, bf16hi_to_f32(sc.z)));
    f.w = pack_bf16x2_rn(__fadd_rn(1.0f, bf16lo_to_f32(sc.w)), __fadd_rn(1.0f, bf16hi_to_f32(sc.w)));
    fac_s[c] = f;
    shf_s[c] = shift[c];
  }
  __syncthreads();
  constexpr int RPC = kThreads / TPR;
  const int slot = threadIdx.x / TPR;
  const int lane = threadIdx.x % TPR;
  for (int64_t row0 = (int64_t)blockIdx.x * RPC; row0 < M; row0 += (int64_t)gridDim.x * RPC) {
    const int64_t row = row0 + slot;
    const bool live = row < M;
    uint4 v[VPT];
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int c = lane + i * TPR;
      v[i] = (live && c < cvec) ? ldg_stream(x + row * cvec + c) : make_uint4(0, 0, 0, 0);
    }
    // the row this slot handles next is requested into L2 now: the three dependent reductions
    // below leave few loads in flight per SM otherwise
    {
      const int64_t next = row + (int64_t)gridDim.x * RPC;
      if (next < M) {
#pragma unroll
        for (int i = 0; i < VPT; ++i) {   // one 128-byte line per 8 lanes' vectors
          const int c = lane + i * TPR;
          if (c < cvec && (lane & 7) == 0)
            asm volatile("prefetch.global.L2 [%0];" ::"l"(x + next * cvec + c));
        }
      }
    }
    // the row is unpacked to fp32 once and stays in registers for all three passes
    float xf[VPT][8];
    float sum = 0.f;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const uint32_t w[4] = {v[i].x, v[i].y, v[i].z, v[i].w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        xf[i][2 * j] = bf16lo_to_f32(w[j]);
        xf[i][2 * j + 1] = bf16hi_to_f32(w[j]);
        sum += xf[i][2 * j] + xf[i][2 * j + 1];
      }
    }
    const float mean = row_allreduce_sum<TPR>(sum, red) * inv_c;
    float sq = 0.f;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int c = lane + i * TPR;
      if (c < cvec) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float a = xf[i][2 * j] - mean, b = xf[i][2 * j + 1] - mean;
          sq += a * a + b * b;
        }
      }
    }
    const float rstd = rsqrtf(row_allreduce_sum<TPR>(sq, red) * inv_c + eps);
    uint32_t acc = 0;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int c = lane + i * TPR;
      if (c < cvec) {
        const uint4 fc = fac_s[c], sh = shf_s[c];
        const uint32_t fcw[4] = {fc.x, fc.y, fc.z, fc.w}, shw[4] = {sh.x, sh.y, sh.z, sh.w};
        uint32_t w[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const uint32_t n = pack_bf16x2_rn((xf[i][2 * j] - mean) * rstd, (xf[i][2 * j + 1] - mean) * rstd);
          // The two modulation roundings as packed bf16 instructions on the FMA pipe.  Each is
          // the correctly rounded product / sum of two bf16 values, which is what the fp32
          // formulation computes too: the fp32 product of two bf16 is exact, and the fp32 sum
          // of two bf16 is exact unless their exponents lie more than 16 apart, where the small
          // term is far below half an ulp in either formulation.
          w[j] = bf16x2_add_rn(bf16x2_mul_rn(n, fcw[j]), shw[j]);
          if (QUANT) acc = absmax_bf16x2(acc, w[j]);
        }
        v[i] = make_uint4(w[0], w[1], w[2], w[3]);
        if (!QUANT && live) out_bf16[row * cvec + c] = v[i];
      }
    }
    if constexpr (QUANT) {
      const float absmax = row_allreduce_nanmax<TPR>(fold_absmax(acc), red);
      float r;
      bool zero_row;
      const float s = row_scale_from_absmax(absmax, &r, &zero_row);
      if (live) {
        if (lane == 0) out_scale[row] = s;
#pragma unroll
        for (int i = 0; i < VPT; ++i) {
          const int c = lane + i * TPR;
          if (c < cvec) out_q[row * cvec + c] = zero_row ? make_uint2(0, 0) : quant_vec8(v[i], r);
        }
      }
    }
  }
}

// qkv bf16 [S,3,H,128]; 16 threads per (row, part in {q,k}, head), 8 elements each.
__global__ void __launch_bounds__(kThreads)
qk_norm_rope_kernel(uint4* __restrict__ qkv, const uint4* __restrict__ qw,
                    const uint4* __restrict__ kw, const float4* __restrict__ cos_tab,
                    const float4* __restrict__ sin_tab, int64_t S, int H, float eps) {
  const int64_t total = S * 2 * H * 16;
  for (int64_t t = (int64_t)blockIdx.x * kThreads + threadIdx.x; (t & ~(int64_t)31) < total;
       t += (int64_t)gridDim.x * kThreads) {
    const bool live = t < total;
    const int64_t tt = live ? t : total - 1;
    const int l = (int)(tt & 15);
    const int64_t hv = tt >> 4;
    const int h = (int)(hv % H);
    const int part = (int)((hv / H) & 1);
    const int64_t s = hv / (2 * H);
    uint4* p = qkv + ((s * 3 + part) * H + h) * 16 + l;
    const uint4 v = *p;
    const uint4 wv = (part == 0 ? qw : kw)[l];
    const uint32_t w[4] = {v.x, v.y, v.z, v.w}, ww[4] = {wv.x, wv.y, wv.z, wv.w};
    float e[8];
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      e[2 * j] = bf16lo_to_f32(w[j]);
      e[2 * j + 1] = bf16hi_to_f32(w[j]);
      ss += e[2 * j] * e[2 * j] + e[2 * j + 1] * e[2 * j + 1];
    }
#pragma unroll
    for (int off = 8; off > 0; off >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, off);
    const float rms = rsqrtf(ss * (1.0f / 128.0f) + eps);
    const float4 c = cos_tab[s * 16 + l], sn = sin_tab[s * 16 + l];
    const float cc[4] = {c.x, c.y, c.z, c.w}, sv[4] = {sn.x, sn.y, sn.z, sn.w};
    uint32_t o[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float y0 = e[2 * j] * rms * bf16lo_to_f32(ww[j]);
      const float y1 = e[2 * j + 1] * rms * bf16hi_to_f32(ww[j]);
      o[j] = pack_bf16x2_rn(y0 * cc[j] - y1 * sv[j], y1 * cc[j] + y0 * sv[j]);
    }
    if (live) *p = make_uint4(o[0], o[1], o[2], o[3]);
  }
}

// The same normalisation and rotation, written straight into the send buffer of the
// sequence-parallel all-to-all instead of in place: qkv bf16 [L,3,H,128] -> send
// [chunks][world][L][c][3][128] with head h = (p*chunks + ch)*c + ci (rank p receives its
// heads of every chunk), V copied unchanged.  16 threads per (row, part in {q,k,v}, head).
__global__ void __launch_bounds__(kThreads)
qk_norm_rope_pack_kernel(const uint4* __restrict__ qkv, uint4* __restrict__ send,
                         const uint4* __restrict__ qw, const uint4* __restrict__ kw,
                         const float4* __restrict__ cos_tab, const float4* __restrict__ sin_tab,
                         int64_t L, int H, int world, int chunks, float eps) {
  const int64_t total = L * 3 * H * 16;
  const int c_heads = H / (world * chunks);
  for (int64_t t = (int64_t)blockIdx.x * kThreads + threadIdx.x; (t & ~(int64_t)31) < total;
       t += (int64_t)gridDim.x * kThreads) {
    const bool live = t < total;
    const int64_t tt = live ? t : total - 1;
    const int l = (int)(tt & 15);
    const int64_t hv = tt >> 4;
    const int h = (int)(hv % H);
    const int part = (int)((hv / H) % 3);
    const int64_t s = hv / (3 * H);
    const uint4 v = ldg_stream(qkv + ((s * 3 + part) * H + h) * 16 + l);
    const int seg = h / c_heads, ci = h - seg * c_heads;     // seg = p*chunks + ch
    const int p = seg / chunks, ch = seg - p * chunks;
    uint4* dst = send + (((((int64_t)ch * world + p) * L + s) * c_heads + ci) * 3 + part) * 16 + l;
    // V is a plain copy.  The 16 threads of a (row, part, head) group agree on `part`, and the
    // shuffles below stay inside such a group and name only its 16 lanes, so a V group can
    // leave while the other half of the warp (a Q or K group when H is odd) carries on.
    const uint32_t group_mask = 0xffffu << (threadIdx.x & 16);
    if (part == 2) {
      if (live) *dst = v;
      continue;
    }
    const uint4 wv = (part == 1 ? kw : qw)[l];
    const uint32_t w[4] = {v.x, v.y, v.z, v.w}, ww[4] = {wv.x, wv.y, wv.z, wv.w};
    float e[8];
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      e[2 * j] = bf16lo_to_f32(w[j]);
      e[2 * j + 1] = bf16hi_to_f32(w[j]);
      ss += e[2 * j] * e[2 * j] + e[2 * j + 1] * e[2 * j + 1];
    }
#pragma unroll
    for (int off = 8; off > 0; off >>= 1) ss += __shfl_xor_sync(group_mask, ss, off);
    const float rms = rsqrtf(ss * (1.0f / 128.0f) + eps);
    const float4 c = cos_tab[s * 16 + l], sn = sin_tab[s * 16 + l];
    const float cc[4] = {c.x, c.y, c.z, c.w}, sv[4] = {sn.x, sn.y, sn.z, sn.w};
    uint32_t o[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float y0 = e[2 * j] * rms * bf16lo_to_f32(ww[j]);
      const float y1 = e[2 * j + 1] * rms * bf16hi_to_f32(ww[j]);
      o[j] = pack_bf16x2_rn(y0 * cc[j] - y1 * sv[j], y1 * cc[j] + y0 * sv[j]);
    }
    if (live) *dst = make_uint4(o[0], o[1], o[2], o[3]);
  }
}

int grid_for_rows(int64_t M, int rows_per_cta, int ctas_per_sm) {
  int64_t need = (M + rows_per_cta - 1) / rows_per_cta;
  int64_t cap = (int64_t)kNumSMsB200 * ctas_per_sm;
  return (int)(need < cap ? need : cap);
}

}  // namespace

int launch_layernorm_mod(const void* x, const void* scale, const void* shift, void* out_bf16,
                         int8_t* out_q, float* out_scale, int64_t M, int64_t C, float eps,
                         bool quant, cudaStream_t stream) {
  const int cvec = (int)(C / 8);
  const float inv_c = 1.0f / (float)C;
  const size_t smem_bytes = (size_t)cvec * 2 * sizeof(uint4);  // <= 32 KB for C <= 8192
#define B2_LN(TPR, VPT)                                                                          \
  do {                                                                                           \
    const int g = grid_for_rows(M, kThreads / TPR, 8);                                           \
    if (quant)                                                                                   \
      layernorm_mod_kernel<TPR, VPT, true><<<g, kThreads, smem_bytes, stream>>>(                          \
          (const uint4*)x, (const uint4*)scale, (const uint4*)shift, nullptr, (uint2*)out_q,     \
          out_scale, M, cvec, inv_c, eps);                                                       \
    else                                                                                         \
      layernorm_mod_kernel<TPR, VPT, false><<<g, kThreads, smem_bytes, stream>>>(                         \
          (const uint4*)x, (const uint4*)scale, (const uint4*)shift, (uint4*)out_bf16, nullptr,  \
          nullptr, M, cvec, inv_c, eps);                                                         \
  } while (0)
  // at most 6 vectors (48 fp32 values) per thread, so the unpacked row fits in registers
  if (C <= 1024) B2_LN(32, 4);
  else if (C <= 2048) B2_LN(64, 4);
  else if (C <= 3072) B2_LN(64, 6);
  else if (C <= 4096) B2_LN(128, 4);
  else if (C <= 6144) B2_LN(128, 6);
  else if (C <= 8192) B2_LN(256, 4);
  else return fail(B2_NOT_WHITELISTED, "layernorm_mod: C=%lld exceeds 8192", (long long)C);
#undef B2_LN
  return check_launch("layernorm_mod");
}

int launch_qk_norm_rope(void* qkv, const void* qw, const void* kw, const float* cos_tab,
                        const float* sin_tab, int64_t S, int H, float eps, cudaStream_t stream) {
  const int64_t total = S * 2 * H * 16;
  int64_t blocks = (total + kThreads - 1) / kThreads;
  const int64_t cap = (int64_t)kNumSMsB200 * 32;
  if (blocks > cap) blocks = cap;
  qk_norm_rope_kernel<<<(int)blocks, kThreads, 0, stream>>>(
      (uint4*)qkv, (const uint4*)qw, (const uint4*)kw, (const float4*)cos_tab,
      (const float4*)sin_tab, S, H, eps);
  return check_launch("qk_norm_rope");
}

int launch_qk_norm_rope_pack(const void* qkv, void* send, const void* qw, const void* kw,
                             const float* cos_tab, const float* sin_tab, int64_t L, int H, int world,
                             int chunks, float eps, cudaStream_t stream) {
  const int64_t total = L * 3 * H * 16;
  int64_t blocks = (total + kThreads - 1) / kThreads;
  const int64_t cap = (int64_t)kNumSMsB200 * 32;
  if (blocks > cap) blocks = cap;
  qk_norm_rope_pack_kernel<<<(int)blocks, kThreads, 0, stream>>>(
      (const uint4*)qkv, (uint4*)send, (const uint4*)qw, (const uint4*)kw, (const float4*)cos_tab,
      (const float4*)sin_tab, L, H, world, chunks, eps);
  return check_launch("qk_norm_rope_pack");
}

}  // namespace b2
