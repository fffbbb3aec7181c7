// Epilogue shared by the single-CTA and the CTA-pair INT8 GEMM kernels: one thread owns
// one accumulator row and walks it in 32-column chunks read from tensor memory.
//
//   plain      out_i32[row, col] = acc
//   dequant    y = bf16( bf16(float(acc) * (rs[row]*cs[col])) + bf16(bias[col]) )
//              (kernels/int8-epilogue/epilogue_kernel.hip:39-53 in the reference, bit-exact)
//   residual   x[row, col] = bf16( x + bf16(gate[col] * y) ) in place: the gated residual
//              of the DiT block applied while the tile is still in registers, so y never
//              makes a round trip through memory
//   swiglu     the weight rows (with their scales and bias) arrive interleaved in groups of
//              64: accumulator columns [128k, 128k+64) are gate columns [64k, 64k+64) and
//              [128k+64, 128k+128) the matching up columns; out[row, 64k+j] =
//              bf16( bf16(silu(y_gate)) * y_up ), y as in dequant: the first half of
//              swiglu-quant (kernels/swiglu-quant/swiglu_quant_kernel.hip:18-27 in the
//              reference) applied while the tile is in registers, so the [M, 2F] projection
//              never reaches memory; out is bf16 [M, N/2]
#pragma once

#include "b2_common.cuh"

namespace b2 {

struct EpilogueArgs {
  int M, N;
  int32_t* out_i32;            // plain mode when non-null
  __nv_bfloat16* out_bf16;     // dequant mode
  const float* rs;
  const float* cs;
  const void* bias;
  int bias_kind;
  const __nv_bfloat16* gate;   // residual mode when non-null (with `residual`)
  __nv_bfloat16* residual;
  int swiglu;                  // swiglu mode (dequant mode's pointers; out_bf16 is [M, N/2])
  const uint16_t* silu_lut;    // swiglu mode: bf16(silu(g)) indexed by the gate's 16 bits (global memory)
};

constexpr int kEpiTileN = 256;
constexpr int kColVecFloats = 3 * kEpiTileN;   // scale | bias | gate, per accumulator buffer

// Stage the tile's per-column operands into shared memory (called by the 128 epilogue
// threads, `et` in [0,128)); the caller synchronises them afterwards.
__device__ __forceinline__ void epilogue_stage_columns(const EpilogueArgs& a, float* cvec, int col0,
                                                       int et) {
  for (int c = et; c < kEpiTileN; c += 128) {
    const int col = col0 + c;
    float s = 0.f, b = 0.f, g = 0.f;
    if (col < a.N) {
      s = a.cs[col];
      if (a.bias_kind == B2_BIAS_BF16)
        b = __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(a.bias)[col]);
      else if (a.bias_kind == B2_BIAS_FP32)
        b = round_bf16_f32(reinterpret_cast<const float*>(a.bias)[col]);
      if (a.gate != nullptr) g = __bfloat162float(a.gate[col]);
    }
    cvec[c] = s;
    cvec[kEpiTileN + c] = b;
    cvec[2 * kEpiTileN + c] = g;
  }
}

// Residual mode reads x[row, col0 .. col0+256) in 16-byte pieces, one row per thread: every
// piece would be a fresh trip to DRAM in the middle of the epilogue.  The row segment (four
// 128-byte lines) is requested into L2 while the tile's main loop is still running.
__device__ __forceinline__ void epilogue_prefetch_residual(const EpilogueArgs& a, int row, int col0) {
  if (a.gate == nullptr || row >= a.M) return;
  const char* p = reinterpret_cast<const char*>(a.residual + (int64_t)row * a.N + col0);
#pragma unroll
  for (int b = 0; b < kEpiTileN * 2; b += 128)
    if (col0 + b / 2 < a.N) asm volatile("prefetch.global.L2 [%0];" ::"l"(p + b));
}

// Residual mode: the 32 columns of x that one chunk of one row updates, as four 16-byte loads
// (8 columns each); groups at or beyond N, and rows at or beyond M, stay zero.  Issued one chunk
// AHEAD of the arithmetic that needs them, so that the trip to L2 overlaps the current chunk.
__device__ __forceinline__ void epilogue_load_residual(const EpilogueArgs& a, int row, int col, uint4 (&x)[4]) {
#pragma unroll
  for (int j4 = 0; j4 < 4; ++j4) x[j4] = make_uint4(0, 0, 0, 0);
  if (a.gate == nullptr || row >= a.M) return;
  const uint4* xsrc = reinterpret_cast<const uint4*>(a.residual + (int64_t)row * a.N + col);
#pragma unroll
  for (int j4 = 0; j4 < 4; ++j4)
    if (col + j4 * 8 < a.N) x[j4] = xsrc[j4];
}

// Dequant (+ bias, + gated residual) of one 32-column chunk of one row into 16 packed bf16
// words.  `c` is the chunk's offset inside the tile, `col` its global column (< N).  In
// residual mode `x` holds the chunk's residual columns (epilogue_load_residual); 8-column groups
// at or beyond N are left as zeros (they are never stored).
__device__ __forceinline__ void epilogue_compute_chunk(const EpilogueArgs& a, const uint32_t (&v)[32],
                                                       int col, int c, float rsv, const float* cvec,
                                                       const uint4 (&x)[4], uint32_t (&o)[16]) {
  const float* cscale = cvec + c;
  const float* cbias = cvec + kEpiTileN + c;
  const float* cgate = cvec + 2 * kEpiTileN + c;
  const bool has_bias = a.bias_kind != B2_BIAS_NONE;
  const bool residual = a.gate != nullptr;
#pragma unroll
  for (int j4 = 0; j4 < 4; ++j4) {  // N % 8 == 0: whole 8-column groups are in or out
    const bool in = col + j4 * 8 < a.N;
    const uint32_t xw[4] = {x[j4].x, x[j4].y, x[j4].z, x[j4].w};
#pragma unroll
    for (int jj = 0; jj < 4; ++jj) {
      const int j = j4 * 4 + jj;
      const float f0 = __fmul_rn(__int2float_rn((int)v[2 * j]), __fmul_rn(rsv, cscale[2 * j]));
      const float f1 = __fmul_rn(__int2float_rn((int)v[2 * j + 1]), __fmul_rn(rsv, cscale[2 * j + 1]));
      uint32_t p = pack_bf16x2_rn(f0, f1);
      if (has_bias)
        p = pack_bf16x2_rn(__fadd_rn(bf16lo_to_f32(p), cbias[2 * j]),
                           __fadd_rn(bf16hi_to_f32(p), cbias[2 * j + 1]));
      if (residual) {
        const uint32_t g = pack_bf16x2_rn(__fmul_rn(bf16lo_to_f32(p), cgate[2 * j]),
                                          __fmul_rn(bf16hi_to_f32(p), cgate[2 * j + 1]));
        p = pack_bf16x2_rn(__fadd_rn(bf16lo_to_f32(xw[jj]), bf16lo_to_f32(g)),
                           __fadd_rn(bf16hi_to_f32(xw[jj]), bf16hi_to_f32(g)));
      }
      o[j] = in ? p : 0u;
    }
  }
}

// Dequant + bias of a packed pair of accumulators (the dequant mode's arithmetic).
__device__ __forceinline__ uint32_t epilogue_dequant_pair(uint32_t v0, uint32_t v1, float rsv, float cs0,
                                                          float cs1, bool has_bias, float b0, float b1) {
  const float f0 = __fmul_rn(__int2float_rn((int)v0), __fmul_rn(rsv, cs0));
  const float f1 = __fmul_rn(__int2float_rn((int)v1), __fmul_rn(rsv, cs1));
  uint32_t p = pack_bf16x2_rn(f0, f1);
  if (has_bias) p = pack_bf16x2_rn(__fadd_rn(bf16lo_to_f32(p), b0), __fadd_rn(bf16hi_to_f32(p), b1));
  return p;
}

// swiglu mode: 32 gate accumulators (tile offset cg) and the 32 matching up accumulators
// (tile offset cu = cg + 64) of one row -> 16 packed bf16 outputs.
__device__ __forceinline__ void epilogue_swiglu_chunk(const EpilogueArgs& a, const uint32_t (&vg)[32],
                                                      const uint32_t (&vu)[32], int cg, int cu, float rsv,
                                                      const float* cvec, uint32_t (&o)[16]) {
  const bool has_bias = a.bias_kind != B2_BIAS_NONE;
  const float* gs = cvec + cg;
  const float* gb = cvec + kEpiTileN + cg;
  const float* us = cvec + cu;
  const float* ub = cvec + kEpiTileN + cu;
#pragma unroll
  for (int j = 0; j < 16; ++j) {
    const uint32_t g = epilogue_dequant_pair(vg[2 * j], vg[2 * j + 1], rsv, gs[2 * j], gs[2 * j + 1], has_bias,
                                             gb[2 * j], gb[2 * j + 1]);
    const uint32_t u = epilogue_dequant_pair(vu[2 * j], vu[2 * j + 1], rsv, us[2 * j], us[2 * j + 1], has_bias,
                                             ub[2 * j], ub[2 * j + 1]);
    // bf16(silu(g)) is a function of the gate's 16 bits: two cached table loads replace two
    // expf + two IEEE divisions per pair, which a single warp per scheduler cannot hide
    const uint32_t sl = (uint32_t)__ldg(a.silu_lut + (g & 0xffffu)) | ((uint32_t)__ldg(a.silu_lut + (g >> 16)) << 16);
    o[j] = bf16x2_mul_rn(sl, u);
  }
}

// Staging tile of one epilogue warp for the TMA-store path: 32 rows (one per lane) x 64 bf16
// columns = 32 x 128 bytes in the 128-byte-swizzle layout of a tensor-map box {64, 32}: the
// 16-byte chunk k of row r sits at r*128 + ((k ^ (r & 7)) * 16).  1024-byte aligned.
constexpr int kEpiStageBytes = 32 * 128;
// Lane `lane` writes its 16 packed words of 32-column half `half` (0 or 1) of the 64-column step.
__device__ __forceinline__ void epilogue_stage_write(uint32_t stage_smem, int lane, int half,
                                                     const uint32_t (&o)[16]) {
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    const uint32_t addr = stage_smem + lane * 128 + (((half * 4 + k) ^ (lane & 7)) << 4);
    asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(o[4 * k]), "r"(o[4 * k + 1]),
                 "r"(o[4 * k + 2]), "r"(o[4 * k + 3])
                 : "memory");
  }
}

// One 32-column chunk of one row, stored directly.  `c` is the chunk's offset inside the tile,
// `col` its global column; the row is valid and col < N (checked by the caller).
__device__ __forceinline__ void epilogue_store_chunk(const EpilogueArgs& a, const uint32_t (&v)[32],
                                                     int row, int col, int c, float rsv,
                                                     const float* cvec) {
  if (a.out_i32 != nullptr) {
    uint4* dst = reinterpret_cast<uint4*>(a.out_i32 + (int64_t)row * a.N + col);
#pragma unroll
    for (int j = 0; j < 8; ++j)  // N % 4 == 0
      if (col + j * 4 < a.N) dst[j] = make_uint4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
    return;
  }
  const float* cscale = cvec + c;
  const float* cbias = cvec + kEpiTileN + c;
  const float* cgate = cvec + 2 * kEpiTileN + c;
  const bool has_bias = a.bias_kind != B2_BIAS_NONE;
  const bool residual = a.gate != nullptr;
  __nv_bfloat16* base = (residual ? a.residual : a.out_bf16) + (int64_t)row * a.N + col;
  uint4* dst = reinterpret_cast<uint4*>(base);
#pragma unroll
  for (int j4 = 0; j4 < 4; ++j4) {  // N % 8 == 0: whole 8-column groups are in or out
    if (col + j4 * 8 >= a.N) break;
    uint32_t o[4];
    uint4 xv = make_uint4(0, 0, 0, 0);
    if (residual) xv = dst[j4];
    const uint32_t xw[4] = {xv.x, xv.y, xv.z, xv.w};
#pragma unroll
    for (int jj = 0; jj < 4; ++jj) {
      const int j = j4 * 4 + jj;
      const float f0 = __fmul_rn(__int2float_rn((int)v[2 * j]), __fmul_rn(rsv, cscale[2 * j]));
      const float f1 = __fmul_rn(__int2float_rn((int)v[2 * j + 1]), __fmul_rn(rsv, cscale[2 * j + 1]));
      uint32_t p = pack_bf16x2_rn(f0, f1);
      if (has_bias)
        p = pack_bf16x2_rn(__fadd_rn(bf16lo_to_f32(p), cbias[2 * j]),
                           __fadd_rn(bf16hi_to_f32(p), cbias[2 * j + 1]));
      if (residual) {
        const uint32_t g = pack_bf16x2_rn(__fmul_rn(bf16lo_to_f32(p), cgate[2 * j]),
                                          __fmul_rn(bf16hi_to_f32(p), cgate[2 * j + 1]));
        p = pack_bf16x2_rn(__fadd_rn(bf16lo_to_f32(xw[jj]), bf16lo_to_f32(g)),
                           __fadd_rn(bf16hi_to_f32(xw[jj]), bf16hi_to_f32(g)));
      }
      o[jj] = p;
    }
    dst[j4] = make_uint4(o[0], o[1], o[2], o[3]);
  }
}

}  // namespace b2
