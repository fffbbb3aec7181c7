// Pieces shared by the two bf16 FlashAttention forward kernels (one CTA per pair of query
// tiles, and the CTA-pair form): tile geometry, the softmax role (one thread per score row),
// the FMA-pipe exponential, and the tensor-map encoder.
#pragma once

#include <cmath>

#include "b2_common.cuh"
#include "b2_launch.h"
#include "sm100_ptx.cuh"

namespace b2 {
namespace flash {

constexpr int BLOCK_M = 128;   // query rows per tile
constexpr int BLOCK_N = 128;   // kv rows per step
constexpr int HEAD_DIM = 128;
constexpr int HALF_BYTES = 128 * 128;        // one [128 rows x 64 bf16] swizzled half tile
constexpr int TILE_BYTES = 2 * HALF_BYTES;   // 32 KB
constexpr int kSoftmaxWarps = 8, kMmaWarp = 8, kLoadWarp = 9;   // warps 10, 11 idle
constexpr int NUM_THREADS = (kSoftmaxWarps + 4) * 32;   // 384: two softmax warpgroups + one service warpgroup
#ifndef B2_FLASH_REGS_SOFTMAX
#define B2_FLASH_REGS_SOFTMAX 232
#endif
#ifndef B2_FLASH_REGS_SERVICE
#define B2_FLASH_REGS_SERVICE 32
#endif
// P is published to the MMA issuer in this many column groups per step (2 or 4)
#ifndef B2_FLASH_P_PARTS
#define B2_FLASH_P_PARTS 2
#endif
// Which of the 8 score pairs of a 16-column chunk take their exponential on the FMA pipe
// (bit i = pair i) instead of the exp2 unit.
#ifndef B2_FLASH_EMU_MASK
#define B2_FLASH_EMU_MASK 0x22
#endif
// setmaxnreg.inc waits, without a limit, until the registers it asks for are free in the
// CTA's own allocation, so the split must fit into what the kernel was launched with:
// per scheduler, two softmax warps and one service warp share three launch allocations.
// The launcher checks this against the compiled register count before every first launch.
constexpr int kLaunchRegs = 168;   // 65536 / 384 threads, rounded down to the allocation unit of 8
static_assert(2 * B2_FLASH_REGS_SOFTMAX + B2_FLASH_REGS_SERVICE <= 3 * kLaunchRegs,
              "register split exceeds the CTA's launch allocation");
constexpr int P_PARTS = B2_FLASH_P_PARTS;
static_assert(P_PARTS == 2 || P_PARTS == 4, "P is published in halves or quarters");
constexpr int TMEM_COLS = 512;
constexpr int COL_S0 = 0, COL_S1 = 128, COL_O0 = 256, COL_O1 = 384;


// mbarrier indices (two of each: ring stage or query tile); P_PART + 2*part + tile
enum { Q_FULL = 0, K_FULL = 2, K_EMPTY = 4, V_FULL = 6, V_EMPTY = 8, S_FULL = 10, O_FULL = 12,
       P_PART = 14 };
constexpr int NUM_BARS = 14 + 2 * P_PARTS;

struct FlashArgs {
  __nv_bfloat16* out;  // [B, S, H, 128]
  int B, H, S;
  int n_kv;           // ceil(S / 128)
  int q_swap, k_swap, v_swap;  // 1: tensor map dims are (D, H, S, B); 0: (D, S, H, B)
  float scale_log2;   // softmax_scale * log2(e)
};

__device__ __forceinline__ float fmax3(float a, float b, float c) {
  float m;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(m) : "f"(a), "f"(b), "f"(c));
  return m;
}
__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
// 2^x for a packed pair on the FMA pipe.  x <= 8 by construction of the running max (larger
// values never reach an exponential); x < -127 (and -inf of masked columns) gives exactly 0;
// NaN stays NaN.
__device__ __forceinline__ uint64_t ex2_poly2(uint64_t xx) {
  float x0, x1;
  unpack2(xx, x0, x1);
  asm("max.NaN.f32 %0, %0, 0fC2FE0000;" : "+f"(x0));   // max(x, -127), NaN kept
  asm("max.NaN.f32 %0, %0, 0fC2FE0000;" : "+f"(x1));
  const uint64_t xc = pack2(x0, x1);
  const uint64_t magic = pack2(12582912.0f, 12582912.0f);   // 1.5 * 2^23
  uint64_t j, jf, f;
  // round DOWN: the low mantissa bits of j hold floor(x) (two's complement)
  asm("add.rm.ftz.f32x2 %0, %1, %2;" : "=l"(j) : "l"(xc), "l"(magic));
  asm("sub.rn.ftz.f32x2 %0, %1, %2;" : "=l"(jf) : "l"(j), "l"(magic));
  asm("sub.rn.ftz.f32x2 %0, %1, %2;" : "=l"(f) : "l"(xc), "l"(jf));   // x - floor(x), in [0, 1)
  uint64_t q = fma2(pack2(0.07706984132528305f, 0.07706984132528305f), f,
                    pack2(0.22764800488948822f, 0.22764800488948822f));
  q = fma2(q, f, pack2(0.6951131224632263f, 0.6951131224632263f));
  q = fma2(q, f, pack2(1.0f, 1.0f));
  // 2^floor(x) built in the exponent field; floor(x) = -127 gives 0
  float j0, j1;
  unpack2(j, j0, j1);
  const uint32_t s0 = (__float_as_uint(j0) << 23) + 0x3f800000u;
  const uint32_t s1 = (__float_as_uint(j1) << 23) + 0x3f800000u;
  return mul2(q, pack2(__uint_as_float(s0), __uint_as_float(s1)));
}

// One pair of scores -> exponentials (added to a running packed sum) -> packed bf16.
template <bool POLY>
__device__ __forceinline__ uint32_t exp_pair(uint32_t sa, uint32_t sb, uint64_t sl2x2, uint64_t nmsx2,
                                             uint64_t& sum2) {
  const uint64_t xx = fma2(pack2(__uint_as_float(sa), __uint_as_float(sb)), sl2x2, nmsx2);
  float e0, e1;
  if constexpr (POLY) {
    const uint64_t ee = ex2_poly2(xx);
    sum2 = add2(sum2, ee);
    unpack2(ee, e0, e1);
  } else {
    float x0, x1;
    unpack2(xx, x0, x1);
    e0 = ex2_approx(x0);
    e1 = ex2_approx(x1);
    sum2 = add2(sum2, pack2(e0, e1));
  }
  return pack_bf16x2_rn(e0, e1);
}

// 16 scores of one thread (one chunk) -> 8 packed bf16 probabilities.
__device__ __forceinline__ void exp_chunk(const uint32_t* s, uint32_t (&p)[8], uint64_t sl2x2,
                                          uint64_t nmsx2, uint64_t (&sm2)[4]) {
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    if ((B2_FLASH_EMU_MASK >> i) & 1)
      p[i] = exp_pair<true>(s[2 * i], s[2 * i + 1], sl2x2, nmsx2, sm2[i & 3]);
    else
      p[i] = exp_pair<false>(s[2 * i], s[2 * i + 1], sl2x2, nmsx2, sm2[i & 3]);
  }
}


// The softmax + output role of warps 0-7 (warps 0-3: query tile 0, warps 4-7: tile 1), one
// thread per score row.  `bar0` is the shared-memory address of this CTA's mbarrier array;
// `arrive_p(part, tile)` publishes one column group of P to the MMA issuer (one call per warp,
// made by lane 0 after the stores are complete and fenced); `tile_row0(tile)` is the global
// query row of the tile's first row.
template <class ArriveP, class TileRow0>
__device__ __forceinline__ void softmax_role(const FlashArgs& args, uint32_t tmem_base, uint32_t bar0,
                                             volatile int* abort_flag, int warp, int lane, int n_kv, int h,
                                             int b, ArriveP arrive_p, TileRow0 tile_row0) {
  auto bar = [&](int idx) -> uint32_t { return bar0 + idx * 8; };
  // ---------------- softmax + output: one thread per row, all 128 columns ----------------
  const int t = warp >> 2;            // query tile
  const int quarter = warp & 3;       // tensor-memory lane quarter of this warp
  const int row_in_tile = quarter * 32 + lane;
  const uint32_t lane_sel = (uint32_t)(quarter * 32) << 16;
  const uint32_t s_tmem = tmem_base + (t ? COL_S1 : COL_S0) + lane_sel;
  const uint32_t p_tmem = s_tmem;     // P (64 columns of packed bf16) overwrites the first half of S
  const uint32_t o_tmem = tmem_base + (t ? COL_O1 : COL_O0) + lane_sel;
  bool ok = true;
  const float sl2 = args.scale_log2;
  const int tail_valid = args.S - (n_kv - 1) * BLOCK_N;  // valid columns of the last step
  float row_max = -INFINITY;  // raw-score domain
  float row_sum = 0.f;
  for (int j = 0; j < n_kv; ++j) {
    if (ok) ok = mbar_wait(bar(S_FULL + t), j & 1, abort_flag, kStatusFlashTimeout);
    tc_fence_after();
    // the row's 128 scores -> registers
    uint32_t s[128];
#pragma unroll
    for (int c = 0; c < 128; c += 32) tmem_ld_32x32b_x32(s_tmem + c, *reinterpret_cast<uint32_t(*)[32]>(&s[c]));
    tmem_wait_ld();
    if (j + 1 == n_kv && tail_valid < BLOCK_N) {
#pragma unroll
      for (int c = 0; c < 128; ++c)
        if (c >= tail_valid) s[c] = 0xff800000u;  // -inf
    }
    float mx[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
    for (int c = 0; c < 128; c += 2)
      mx[(c >> 1) & 3] = fmax3(mx[(c >> 1) & 3], __uint_as_float(s[c]), __uint_as_float(s[c + 1]));
    const float m_row = fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3]));
    // lazy raise (always on the first step)
    const bool raise = (m_row - row_max) * sl2 > 8.0f;
    float alpha = 1.0f;
    if (raise) {
      alpha = ex2_approx((row_max - m_row) * sl2);  // 0 on the first step
      row_max = m_row;
      row_sum *= alpha;
    }
    if (j != 0 && __any_sync(0xffffffffu, raise)) {
#pragma unroll 1
      for (int c = 0; c < 128; c += 16) {
        uint32_t o[16];
        tmem_ld_32x32b_x16(o_tmem + c, o);
        tmem_wait_ld();
#pragma unroll
        for (int i = 0; i < 16; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
        tmem_st_32x32b_x16(o_tmem + c, o);
      }
    }
    const float neg_ms = -row_max * sl2;
    // exponentials on packed pairs: one f32x2 FMA and one f32x2 add per two scores
    const uint64_t sl2x2 = pack2(sl2, sl2), nmsx2 = pack2(neg_ms, neg_ms);
    uint64_t sm2[4] = {0ull, 0ull, 0ull, 0ull};
    // eight chunks of 16 scores -> 8 columns of packed bf16 each; a column group is published
    // as soon as it is written
#pragma unroll
    for (int q = 0; q < 8; ++q) {
      uint32_t p[8];
      exp_chunk(&s[16 * q], p, sl2x2, nmsx2, sm2);
      tmem_st_32x32b_x8(p_tmem + 8 * q, p);
      if ((q + 1) % (8 / P_PARTS) == 0) {
        tmem_wait_st();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) arrive_p(q / (8 / P_PARTS), t);  // one arrival per warp
      }
    }
    {
      float a0, a1, b0, b1, c0, c1, d0, d1;
      unpack2(sm2[0], a0, a1);
      unpack2(sm2[1], b0, b1);
      unpack2(sm2[2], c0, c1);
      unpack2(sm2[3], d0, d1);
      row_sum += ((a0 + a1) + (b0 + b1)) + ((c0 + c1) + (d0 + d1));
    }
  }
  // ---- final: O / l -> bf16 -> global (BSHD) ----
  if (ok) ok = mbar_wait(bar(O_FULL + t), 0, abort_flag, kStatusFlashTimeout);
  if (ok) {
    tc_fence_after();
    const float l = row_sum;
    const int row = tile_row0(t) + row_in_tile;
    const float inv = (l == 0.f || l != l) ? 1.0f : 1.0f / l;
    __nv_bfloat16* dst = args.out + (((int64_t)b * args.S + row) * args.H + h) * (int64_t)HEAD_DIM;
#pragma unroll 1
    for (int c = 0; c < 128; c += 32) {
      uint32_t o[32];
      tmem_ld_32x32b_x32(o_tmem + c, o);
      tmem_wait_ld();
      if (row < args.S) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          uint4 w;
          w.x = pack_bf16x2_rn(__uint_as_float(o[8 * i + 0]) * inv, __uint_as_float(o[8 * i + 1]) * inv);
          w.y = pack_bf16x2_rn(__uint_as_float(o[8 * i + 2]) * inv, __uint_as_float(o[8 * i + 3]) * inv);
          w.z = pack_bf16x2_rn(__uint_as_float(o[8 * i + 4]) * inv, __uint_as_float(o[8 * i + 5]) * inv);
          w.w = pack_bf16x2_rn(__uint_as_float(o[8 * i + 6]) * inv, __uint_as_float(o[8 * i + 7]) * inv);
          reinterpret_cast<uint4*>(dst + c)[i] = w;
        }
      }
    }
  }
}

// 4-D bf16 map over a logical [B,H,S,128] tensor; the two middle dimensions are
// ordered by stride (ascending).  *swap = 1 when the order is (D, H, S, B).
inline int encode_qkv_map(CUtensorMap* map, const void* base, int B, int H, int S, const int64_t* st,
                          int* swap, int box_rows = BLOCK_M) {
  PFN_encodeTiled enc = get_encode_tiled();
  if (!enc) return fail(B2_LAUNCH_FAILED, "flash_fwd: cuTensorMapEncodeTiled is unavailable");
  int64_t sb = st[0], sh = st[1], ss = st[2];
  if (H == 1) sh = ss * (int64_t)S;  // any valid value: the dimension has extent 1
  *swap = sh < ss ? 1 : 0;
  cuuint64_t dims[4];
  cuuint64_t strides[3];
  cuuint32_t box[4];
  dims[0] = HEAD_DIM;
  box[0] = 64;
  if (*swap) {
    dims[1] = (cuuint64_t)H; strides[0] = (cuuint64_t)sh * 2; box[1] = 1;
    dims[2] = (cuuint64_t)S; strides[1] = (cuuint64_t)ss * 2; box[2] = (cuuint32_t)box_rows;
  } else {
    dims[1] = (cuuint64_t)S; strides[0] = (cuuint64_t)ss * 2; box[1] = (cuuint32_t)box_rows;
    dims[2] = (cuuint64_t)H; strides[1] = (cuuint64_t)sh * 2; box[2] = 1;
  }
  dims[3] = (cuuint64_t)B;
  box[3] = 1;
  if (B == 1) {
    const cuuint64_t a = strides[0] * dims[1], c = strides[1] * dims[2];
    sb = (int64_t)((a > c ? a : c) / 2);
  }
  strides[2] = (cuuint64_t)sb * 2;
  const cuuint32_t estr[4] = {1, 1, 1, 1};
  CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(base), dims, strides,
                   box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(B2_LAUNCH_FAILED, "flash_fwd: tensor map encode failed (%d)", (int)r);
  return B2_OK;
}


}  // namespace flash
}  // namespace b2
