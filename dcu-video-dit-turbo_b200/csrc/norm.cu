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

// One row per TPR threads, VPT vectors of 8 bf16 per thread; C % 8 == 0,
// C <= TPR*VPT*8.  QUANT selects the fused quantizer output; FULL says that the row fills
// every vector of every thread (C == TPR*VPT*8), which removes the per-vector range tests.
// The full-row form needs 78 registers and runs three CTAs per SM (measured 0.80 of the HBM
// peak against 0.71 at two); the ragged form keeps two (at three it would spill).
template <int TPR, int VPT, bool QUANT, bool FULL>
__global__ void __launch_bounds__(kThreads, FULL ? 3 : 2)
layernorm_mod_kernel(const uint4* __restrict__ x, const uint4* __restrict__ scale,
                     const uint4* __restrict__ shift, uint4* __restrict__ out_bf16,
                     uint2* __restrict__ out_q, float* __restrict__ out_scale, int64_t M, int cvec,
                     float inv_c, float eps) {
  __shared__ float red[3][kThreads / 32];   // one buffer per reduction of a row (slot_allreduce)
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
      v[i] = (live && (FULL || c < cvec)) ? ldg_stream(x + row * cvec + c) : make_uint4(0, 0, 0, 0);
    }
    // the row this slot handles next is requested into L2 now: the three dependent reductions
    // below leave few loads in flight per SM otherwise
    {
      const int64_t next = row + (int64_t)gridDim.x * RPC;
      if (next < M) {
#pragma unroll
        for (int i = 0; i < VPT; ++i) {   // one 128-byte line per 8 lanes' vectors
          const int c = lane + i * TPR;
          if ((FULL || c < cvec) && (lane & 7) == 0)
            asm volatile("prefetch.global.L2 [%0];" ::"l"(x + next * cvec + c));
        }
      }
    }
    // the row is unpacked once, to packed fp32 pairs, and stays in registers for all three
    // passes; sums, differences, squares and the scaling are packed f32x2 instructions
    uint64_t xf[VPT][4];
    uint64_t sum2[2] = {0ull, 0ull};
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const uint32_t w[4] = {v[i].x, v[i].y, v[i].z, v[i].w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        xf[i][j] = bf16x2_to_f32x2(w[j]);
        sum2[j & 1] = add2(sum2[j & 1], xf[i][j]);
      }
    }
    float sum;
    {
      float a0, a1, b0, b1;
      unpack2(sum2[0], a0, a1);
      unpack2(sum2[1], b0, b1);
      sum = (a0 + a1) + (b0 + b1);
    }
    const float mean = slot_allreduce<kThreads, TPR>(sum, red[0], slot, SumOp()) * inv_c;
    const uint64_t mean2 = pack2(mean, mean);
    uint64_t sq2[2] = {0ull, 0ull};
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int c = lane + i * TPR;
      if (FULL || c < cvec) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          xf[i][j] = sub2(xf[i][j], mean2);          // kept: the normalisation reuses x - mean
          sq2[j & 1] = fma2(xf[i][j], xf[i][j], sq2[j & 1]);
        }
      }
    }
    float sq;
    {
      float a0, a1, b0, b1;
      unpack2(sq2[0], a0, a1);
      unpack2(sq2[1], b0, b1);
      sq = (a0 + a1) + (b0 + b1);
    }
    const float rstd = rsqrtf(slot_allreduce<kThreads, TPR>(sq, red[1], slot, SumOp()) * inv_c + eps);
    const uint64_t rstd2 = pack2(rstd, rstd);
    uint32_t acc = 0;
#pragma unroll
    for (int i = 0; i < VPT; ++i) {
      const int c = lane + i * TPR;
      if (FULL || c < cvec) {
        const uint4 fc = fac_s[c], sh = shf_s[c];
        const uint32_t fcw[4] = {fc.x, fc.y, fc.z, fc.w}, shw[4] = {sh.x, sh.y, sh.z, sh.w};
        uint32_t w[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const uint32_t n = f32x2_to_bf16x2_rn(mul2(xf[i][j], rstd2));
          // The two modulation roundings as packed bf16 instructions on the FMA pipe.  Each is
          // the correctly rounded product / sum of two bf16 values, which is what the fp32
          // formulation computes too: the fp32 product of two bf16 is exact, and the fp32 sum
          // of two bf16 is exact unless their exponents lie more than 16 apart, where the small
          // term is far below half an ulp in either formulation.
          w[j] = bf16x2_add_rn(bf16x2_mul_rn(n, fcw[j]), shw[j]);
          // the chain starts from data: vector 0 is live in every thread that holds any
          if (QUANT) acc = (i == 0 && j == 0) ? w[j] : absmax_bf16x2(acc, w[j]);
        }
        v[i] = make_uint4(w[0], w[1], w[2], w[3]);
        if (!QUANT && live) out_bf16[row * cvec + c] = v[i];
      }
    }
    if constexpr (QUANT) {
      const float absmax = slot_allreduce<kThreads, TPR>(fold_absmax(acc), red[2], slot, NanMaxOp());
      float r;
      bool zero_row;
      const float s = row_scale_from_absmax(absmax, &r, &zero_row);
      if (live) {
        if (lane == 0) out_scale[row] = s;
#pragma unroll
        for (int i = 0; i < VPT; ++i) {
          const int c = lane + i * TPR;
          if (FULL || c < cvec) out_q[row * cvec + c] = zero_row ? make_uint2(0, 0) : quant_vec8(v[i], r);
        }
      }
    }
  }
}

// RMSNorm + rotary embedding for the 8 channels one thread holds of a 128-channel head; the
// 16 threads of the head (a half-warp: lanes `group_mask`) reduce the sum of squares.
// Shared by the in-place and the packing kernel, so both give the same bits.
__device__ __forceinline__ uint4 norm_rope_vec8(const uint4 v, const uint4 wv, const float4 c,
                                                const float4 sn, float eps, uint32_t group_mask) {
  const uint32_t w[4] = {v.x, v.y, v.z, v.w}, ww[4] = {wv.x, wv.y, wv.z, wv.w};
  uint64_t e2[4];
  uint64_t ss2 = 0ull;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    e2[j] = bf16x2_to_f32x2(w[j]);
    ss2 = fma2(e2[j], e2[j], ss2);
  }
  float s0, s1;
  unpack2(ss2, s0, s1);
  float ss = s0 + s1;
#pragma unroll
  for (int off = 8; off > 0; off >>= 1) ss += __shfl_xor_sync(group_mask, ss, off);
  const float rms = rsqrtf(ss * (1.0f / 128.0f) + eps);
  const uint64_t rms2 = pack2(rms, rms);
  const float cc[4] = {c.x, c.y, c.z, c.w}, sv[4] = {sn.x, sn.y, sn.z, sn.w};
  uint32_t o[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    float y0, y1;
    unpack2(mul2(mul2(e2[j], rms2), bf16x2_to_f32x2(ww[j])), y0, y1);   // (x * rms) * w
    o[j] = pack_bf16x2_rn(__fmaf_rn(y0, cc[j], -__fmul_rn(y1, sv[j])),
                          __fmaf_rn(y1, cc[j], __fmul_rn(y0, sv[j])));
  }
  return make_uint4(o[0], o[1], o[2], o[3]);
}

constexpr int kRopeMaxPeers = 8;  // ranks of one NVSwitch domain the scatter kernel addresses
constexpr int kRopeMaxIter = 6;   // 16-byte vectors of one row per thread (template ITER): heads <= 32

// qkv bf16 [S,3,H,128], q and k normed and rotated in place.  One CTA walks rows; a thread
// keeps the same vectors of every row (vector i of the row's 2*H*16 q/k vectors: channel
// group l = i & 15, part and head from i >> 4), so there is no index arithmetic per element.
template <int ITER>
__global__ void __launch_bounds__(kThreads)
qk_norm_rope_kernel(uint4* __restrict__ qkv, const uint4* __restrict__ qw,
                    const uint4* __restrict__ kw, const float4* __restrict__ cos_tab,
                    const float4* __restrict__ sin_tab, int64_t S, int H, float eps) {
  const int vec_qk = 2 * H * 16;            // q and k are adjacent in a row
  const int64_t row_vec = 3 * (int64_t)H * 16;
  const int l = threadIdx.x & 15;
  const uint32_t group_mask = 0xffffu << (threadIdx.x & 16);
  const uint4 wq = qw[l], wk = kw[l];
  for (int64_t s = blockIdx.x; s < S; s += gridDim.x) {
    uint4* row = qkv + s * row_vec;
    const float4 c = cos_tab[s * 16 + l], sn = sin_tab[s * 16 + l];
    uint4 v[ITER];
#pragma unroll
    for (int it = 0; it < ITER; ++it) {
      const int i = threadIdx.x + it * kThreads;
      // a 16-lane group is live or dead as a whole (vec_qk is a multiple of 16)
      if (i < vec_qk) v[it] = row[i];
    }
#pragma unroll
    for (int it = 0; it < ITER; ++it) {
      const int i = threadIdx.x + it * kThreads;
      if (i < vec_qk) row[i] = norm_rope_vec8(v[it], (i >> 4) >= H ? wk : wq, c, sn, eps, group_mask);
    }
  }
}

// The same normalisation and rotation, written straight into the send buffer of the
// sequence-parallel all-to-all instead of in place: qkv bf16 [L,3,H,128] -> send
// [chunks][world][L][c][3][128] with head h = (p*chunks + ch)*c + ci (rank p receives its
// heads of every chunk), V copied unchanged.  A thread keeps the same vectors of every row, so
// the destination arithmetic runs once per thread, outside the row loop.
template <int ITER>
__global__ void __launch_bounds__(kThreads)
qk_norm_rope_pack_kernel(const uint4* __restrict__ qkv, uint4* __restrict__ send,
                         const uint4* __restrict__ qw, const uint4* __restrict__ kw,
                         const float4* __restrict__ cos_tab, const float4* __restrict__ sin_tab,
                         int64_t L, int H, int world, int chunks, float eps) {
  const int row_vec = 3 * H * 16;
  const int c_heads = H / (world * chunks);
  const int l = threadIdx.x & 15;
  const uint32_t group_mask = 0xffffu << (threadIdx.x & 16);
  const uint4 wq = qw[l], wk = kw[l];
  // destination of vector i of row 0, and the distance between rows there
  int64_t dst0[ITER];
  int part_of[ITER];
#pragma unroll
  for (int it = 0; it < ITER; ++it) {
    const int i = threadIdx.x + it * kThreads;
    dst0[it] = 0;
    part_of[it] = 3;   // dead
    if (i < row_vec) {
      const int hp = i >> 4, part = hp / H, h = hp - part * H;
      const int seg = h / c_heads, ci = h - seg * c_heads;     // seg = p*chunks + ch
      const int p = seg / chunks, ch = seg - p * chunks;
      dst0[it] = (((((int64_t)ch * world + p) * L) * c_heads + ci) * 3 + part) * 16 + l;
      part_of[it] = part;
    }
  }
  const int64_t dst_row = (int64_t)c_heads * 3 * 16;
  for (int64_t s = blockIdx.x; s < L; s += gridDim.x) {
    const uint4* row = qkv + s * row_vec;
    const float4 c = cos_tab[s * 16 + l], sn = sin_tab[s * 16 + l];
    uint4 v[ITER];
#pragma unroll
    for (int it = 0; it < ITER; ++it)
      if (part_of[it] < 3) v[it] = ldg_stream(row + threadIdx.x + it * kThreads);
#pragma unroll
    for (int it = 0; it < ITER; ++it) {
      if (part_of[it] == 3) continue;
      // V is a plain copy.  The 16 lanes of a (part, head) group agree on `part`, and the
      // shuffles stay inside the group and name only its lanes.
      const uint4 o = part_of[it] == 2 ? v[it]
                                       : norm_rope_vec8(v[it], part_of[it] == 1 ? wk : wq, c, sn, eps, group_mask);
      send[dst0[it] + s * dst_row] = o;
    }
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
    const bool full = cvec == TPR * VPT;                                                         \
    if (quant && full)                                                                           \
      layernorm_mod_kernel<TPR, VPT, true, true><<<g, kThreads, smem_bytes, stream>>>(           \
          (const uint4*)x, (const uint4*)scale, (const uint4*)shift, nullptr, (uint2*)out_q,     \
          out_scale, M, cvec, inv_c, eps);                                                       \
    else if (quant)                                                                              \
      layernorm_mod_kernel<TPR, VPT, true, false><<<g, kThreads, smem_bytes, stream>>>(          \
          (const uint4*)x, (const uint4*)scale, (const uint4*)shift, nullptr, (uint2*)out_q,     \
          out_scale, M, cvec, inv_c, eps);                                                       \
    else                                                                                         \
      layernorm_mod_kernel<TPR, VPT, false, false><<<g, kThreads, smem_bytes, stream>>>(         \
          (const uint4*)x, (const uint4*)scale, (const uint4*)shift, (uint4*)out_bf16, nullptr,  \
          nullptr, M, cvec, inv_c, eps);                                                         \
  } while (0)
  // at most 6 vectors (48 fp32 values) per thread, so the unpacked row fits in registers
  if (C <= 1024) B2_LN(32, 4);
  else if (C <= 2048) B2_LN(64, 4);
  else if (C <= 3072) B2_LN(64, 6);   // (128, 3) at three CTAs per SM measured 7 % slower
  else if (C <= 4096) B2_LN(128, 4);
  else if (C <= 6144) B2_LN(128, 6);
  else if (C <= 8192) B2_LN(256, 4);
  else return fail(B2_NOT_WHITELISTED, "layernorm_mod: C=%lld exceeds 8192", (long long)C);
#undef B2_LN
  return check_launch("layernorm_mod");
}

// The packing kernel with the sequence-parallel exchange folded in: instead of a local send
// buffer that an all-to-all then moves, every vector goes straight to the rank that owns its
// head, into that rank's receive buffer [chunks, S, c, 3, 128] at row row0 + s (plain 16-byte
// stores through peer pointers; dst.base[rank] is this GPU's own buffer).  A (head, part) is
// 256 contiguous bytes at the destination.  Same arithmetic as the other two kernels.
struct RopePeerBases {
  uint4* base[kRopeMaxPeers];
};

template <int ITER>
__global__ void __launch_bounds__(kThreads)
qk_norm_rope_scatter_kernel(const uint4* __restrict__ qkv, const __grid_constant__ RopePeerBases dst,
                            const uint4* __restrict__ qw, const uint4* __restrict__ kw,
                            const float4* __restrict__ cos_tab, const float4* __restrict__ sin_tab,
                            int64_t L, int H, int world, int chunks, int64_t row0, int64_t S, float eps) {
  const int row_vec = 3 * H * 16;
  const int c_heads = H / (world * chunks);
  const int l = threadIdx.x & 15;
  const uint32_t group_mask = 0xffffu << (threadIdx.x & 16);
  const uint4 wq = qw[l], wk = kw[l];
  // where vector i of this rank's row 0 lands, and the distance between rows there
  uint4* dst0[ITER];
  int part_of[ITER];
#pragma unroll
  for (int it = 0; it < ITER; ++it) {
    const int i = threadIdx.x + it * kThreads;
    dst0[it] = nullptr;
    part_of[it] = 3;   // dead
    if (i < row_vec) {
      const int hp = i >> 4, part = hp / H, h = hp - part * H;
      const int seg = h / c_heads, ci = h - seg * c_heads;     // seg = p*chunks + ch
      const int p = seg / chunks, ch = seg - p * chunks;
      dst0[it] = dst.base[p] + ((((int64_t)ch * S + row0) * c_heads + ci) * 3 + part) * 16 + l;
      part_of[it] = part;
    }
  }
  const int64_t dst_row = (int64_t)c_heads * 3 * 16;
  for (int64_t s = blockIdx.x; s < L; s += gridDim.x) {
    const uint4* row = qkv + s * row_vec;
    const float4 c = cos_tab[s * 16 + l], sn = sin_tab[s * 16 + l];
    uint4 v[ITER];
#pragma unroll
    for (int it = 0; it < ITER; ++it)
      if (part_of[it] < 3) v[it] = ldg_stream(row + threadIdx.x + it * kThreads);
#pragma unroll
    for (int it = 0; it < ITER; ++it) {
      if (part_of[it] == 3) continue;
      const uint4 o = part_of[it] == 2 ? v[it]
                                       : norm_rope_vec8(v[it], part_of[it] == 1 ? wk : wq, c, sn, eps, group_mask);
      dst0[it][s * dst_row] = o;
    }
  }
}

int launch_qk_norm_rope(void* qkv, const void* qw, const void* kw, const float* cos_tab,
                        const float* sin_tab, int64_t S, int H, float eps, cudaStream_t stream) {
  if (3 * H * 16 > kRopeMaxIter * kThreads)
    return fail(B2_NOT_WHITELISTED, "qk_norm_rope: at most %d heads", kRopeMaxIter * kThreads / 48);
  const int64_t cap = (int64_t)kNumSMsB200 * 8;
  const int64_t blocks = S < cap ? S : cap;
#define B2_ROPE(ITER)                                                              \
  qk_norm_rope_kernel<ITER><<<(int)blocks, kThreads, 0, stream>>>(                 \
      (uint4*)qkv, (const uint4*)qw, (const uint4*)kw, (const float4*)cos_tab,     \
      (const float4*)sin_tab, S, H, eps)
  switch ((2 * H * 16 + kThreads - 1) / kThreads) {   // vectors of one row per thread
    case 1: B2_ROPE(1); break;
    case 2: B2_ROPE(2); break;
    case 3: B2_ROPE(3); break;
    default: B2_ROPE(4); break;
  }
#undef B2_ROPE
  return check_launch("qk_norm_rope");
}

int launch_qk_norm_rope_pack(const void* qkv, void* send, const void* qw, const void* kw,
                             const float* cos_tab, const float* sin_tab, int64_t L, int H, int world,
                             int chunks, float eps, cudaStream_t stream) {
  if (3 * H * 16 > kRopeMaxIter * kThreads)
    return fail(B2_NOT_WHITELISTED, "qk_norm_rope_pack: at most %d heads", kRopeMaxIter * kThreads / 48);
  const int64_t cap = (int64_t)kNumSMsB200 * 8;
  const int64_t blocks = L < cap ? L : cap;
#define B2_ROPE_PACK(ITER)                                                                       \
  qk_norm_rope_pack_kernel<ITER><<<(int)blocks, kThreads, 0, stream>>>(                          \
      (const uint4*)qkv, (uint4*)send, (const uint4*)qw, (const uint4*)kw, (const float4*)cos_tab, \
      (const float4*)sin_tab, L, H, world, chunks, eps)
  switch ((3 * H * 16 + kThreads - 1) / kThreads) {   // vectors of one row per thread
    case 1: B2_ROPE_PACK(1); break;
    case 2: B2_ROPE_PACK(2); break;
    case 3: B2_ROPE_PACK(3); break;
    case 4: B2_ROPE_PACK(4); break;
    case 5: B2_ROPE_PACK(5); break;
    default: B2_ROPE_PACK(6); break;
  }
#undef B2_ROPE_PACK
  return check_launch("qk_norm_rope_pack");
}

int launch_qk_norm_rope_scatter(const void* qkv, void* const* recv_bases, const void* qw, const void* kw,
                                const float* cos_tab, const float* sin_tab, int64_t L, int H, int world,
                                int chunks, int64_t row0, int64_t S, float eps, cudaStream_t stream) {
  if (3 * H * 16 > kRopeMaxIter * kThreads)
    return fail(B2_NOT_WHITELISTED, "qk_norm_rope_scatter: at most %d heads", kRopeMaxIter * kThreads / 48);
  if (world > kRopeMaxPeers)
    return fail(B2_NOT_WHITELISTED, "qk_norm_rope_scatter: at most %d ranks", kRopeMaxPeers);
  RopePeerBases dst;
  for (int p = 0; p < kRopeMaxPeers; ++p) dst.base[p] = (uint4*)(p < world ? recv_bases[p] : nullptr);
  const int64_t cap = (int64_t)kNumSMsB200 * 8;
  const int64_t blocks = L < cap ? L : cap;
#define B2_ROPE_SCATTER(ITER)                                                                     \
  qk_norm_rope_scatter_kernel<ITER><<<(int)blocks, kThreads, 0, stream>>>(                        \
      (const uint4*)qkv, dst, (const uint4*)qw, (const uint4*)kw, (const float4*)cos_tab,         \
      (const float4*)sin_tab, L, H, world, chunks, row0, S, eps)
  switch ((3 * H * 16 + kThreads - 1) / kThreads) {   // vectors of one row per thread
    case 1: B2_ROPE_SCATTER(1); break;
    case 2: B2_ROPE_SCATTER(2); break;
    case 3: B2_ROPE_SCATTER(3); break;
    case 4: B2_ROPE_SCATTER(4); break;
    case 5: B2_ROPE_SCATTER(5); break;
    default: B2_ROPE_SCATTER(6); break;
  }
#undef B2_ROPE_SCATTER
  return check_launch("qk_norm_rope_scatter");
}

}  // namespace b2
