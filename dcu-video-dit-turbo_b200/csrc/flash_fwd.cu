// bf16 FlashAttention forward for sm_100a (non-causal, head_dim 128, strided BHSD
// inputs, contiguous BSHD output).
//
// Replaces the reference's forward kernel chain
//   kernels/flash-attention-gfx936/csrc/flash_attn_hipc/h3_flash_api.cpp:30-130
//   kernels/flash-attention-gfx936/csrc/flash_attn_hipc/src/flash_fwd_b16_fa.h:13-360
// Same mathematics (fp32 scores and accumulators, exp2-domain online softmax with the
// row sum taken before P is rounded to bf16, conditional rescale, tail columns masked
// to -inf, final O/l, bf16 round-to-nearest-even store) on a Blackwell schedule:
//
//   One CTA owns TWO 128-row query tiles of one (batch, head) and walks the KV
//   sequence in 128-row steps.
//     warps 0-3   softmax for query tile 0: one thread per row, S row read from
//                 tensor memory into registers, online softmax, P written back to
//                 tensor memory as bf16 (aliasing the S columns)
//     warps 4-7   the same for query tile 1
//     warp 8      MMA issuer: S = Q.K^T (tcgen05.mma kind::f16, operands in shared
//                 memory) and O += P.V (P read from tensor memory, V from shared
//                 memory as an MN-major operand); accumulators S0,S1,O0,O1 fill
//                 the 512 tensor-memory columns
//     warp 9      TMA loader: Q once, K and V tiles through a two-stage ring
//                 (128-byte swizzle; plain per-CTA loads, no multicast)
//   The two tiles ping-pong: while the softmax warps of one tile run exp2 the
//   tensor core works on the other tile's MMAs.
//   The O rescale is lazy: a row's running max is only raised (and O, l rescaled)
//   when the new max exceeds it by more than 2^8 in the exp2 domain, so after the
//   first steps the rescale almost never runs; the final O/l is exact either way.
// Every mbarrier wait is bounded; on a timeout the kernel records a status word and
// returns through the common teardown.
#include <cmath>

#include "b2_common.cuh"
#include "b2_launch.h"
#include "sm100_ptx.cuh"

namespace b2 {

unsigned int read_clear_status_flash() { return read_and_clear_device_status(); }

namespace {

constexpr int BLOCK_M = 128;   // query rows per tile
constexpr int BLOCK_N = 128;   // kv rows per step
constexpr int HEAD_DIM = 128;
constexpr int HALF_BYTES = 128 * 128;        // one [128 rows x 64 bf16] swizzled half tile
constexpr int TILE_BYTES = 2 * HALF_BYTES;   // 32 KB
constexpr int KV_STAGES = 2;
constexpr int NUM_THREADS = 320;
constexpr int TMEM_COLS = 512;
constexpr int COL_S0 = 0, COL_S1 = 128, COL_O0 = 256, COL_O1 = 384;

constexpr int SMEM_Q = 0;                                   // 2 tiles
constexpr int SMEM_K = SMEM_Q + 2 * TILE_BYTES;             // KV_STAGES tiles
constexpr int SMEM_V = SMEM_K + KV_STAGES * TILE_BYTES;     // KV_STAGES tiles
constexpr int SMEM_BARS = SMEM_V + KV_STAGES * TILE_BYTES;  // 16 mbarriers
constexpr int SMEM_TOTAL = 1024 + SMEM_BARS + 16 * 8 + 16;

// mbarrier indices
enum { Q_FULL = 0, K_FULL = 2, K_EMPTY = 4, V_FULL = 6, V_EMPTY = 8, S_FULL = 10, P_FULL = 12,
       O_FULL = 14 };

struct FlashArgs {
  __nv_bfloat16* out;  // [B, S, H, 128]
  int B, H, S;
  int n_kv;           // ceil(S / 128)
  int q_swap, k_swap, v_swap;  // 1: tensor map dims are (D, H, S, B); 0: (D, S, H, B)
  float scale_log2;   // softmax_scale * log2(e)
};

__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// rows x 64-element half tiles of one [128 x 128] bf16 tile
__device__ __forceinline__ void load_tile(uint32_t dst, const CUtensorMap* map, uint32_t bar,
                                          int row0, int h, int b, int swap) {
  mbar_expect_tx(bar, TILE_BYTES);
  if (swap) {
    tma_load_4d(dst, map, bar, 0, h, row0, b);
    tma_load_4d(dst + HALF_BYTES, map, bar, 64, h, row0, b);
  } else {
    tma_load_4d(dst, map, bar, 0, row0, h, b);
    tma_load_4d(dst + HALF_BYTES, map, bar, 64, row0, h, b);
  }
}

// S[128x128] = A[128 x 128(d)] . B[128 x 128(d)]^T, both K-major half-tile pairs
__device__ __forceinline__ void issue_qk(uint32_t d_tmem, uint32_t q_addr, uint32_t k_addr) {
  constexpr uint32_t idesc = make_idesc(/*f32*/ 1, /*bf16*/ 1, /*bf16*/ 1, 0, 0, BLOCK_M, BLOCK_N);
#pragma unroll
  for (int i = 0; i < HEAD_DIM / 16; ++i) {
    const uint32_t off = (i >> 2) * HALF_BYTES + (i & 3) * 32;
    mma_f16_ss(d_tmem, make_smem_desc_sw128(q_addr + off, 16, 1024),
               make_smem_desc_sw128(k_addr + off, 16, 1024), idesc, i != 0);
  }
}

// O[128x128(d)] (+)= P[128 x 128(kv)] (tensor memory, bf16) . V[128(kv) x 128(d)]
// V is the MN-major B operand: 64-wide d blocks LBO = one half tile apart, 8-row kv
// groups SBO = 1024 bytes apart; 16 kv rows per MMA = 2048 bytes.
__device__ __forceinline__ void issue_pv(uint32_t o_tmem, uint32_t p_tmem, uint32_t v_addr,
                                         bool accumulate) {
  constexpr uint32_t idesc = make_idesc(1, 1, 1, 0, /*B MN-major*/ 1, BLOCK_M, HEAD_DIM);
#pragma unroll
  for (int i = 0; i < BLOCK_N / 16; ++i) {
    mma_f16_ts(o_tmem, p_tmem + i * 8, make_smem_desc_sw128(v_addr + i * 2048, HALF_BYTES, 1024),
               idesc, accumulate || i != 0);
  }
}

__global__ void __launch_bounds__(NUM_THREADS, 1)
flash_fwd_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                 const __grid_constant__ CUtensorMap tmap_v, const FlashArgs args) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + SMEM_BARS);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 16);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  const uint32_t sbase = smem_u32(smem);
  const uint32_t bar0 = smem_u32(bars);
  auto bar = [&](int idx) -> uint32_t { return bar0 + idx * 8; };

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int pair = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int n_kv = args.n_kv;

  if (threadIdx.x == 0) {
    for (int i = 0; i < 16; ++i) mbar_init(bar(i), (i == P_FULL || i == P_FULL + 1) ? 128 : 1);
    *abort_flag = 0;
    fence_barrier_init();
    tma_prefetch_desc(&tmap_q);
    tma_prefetch_desc(&tmap_k);
    tma_prefetch_desc(&tmap_v);
  }
  if (warp == 8) {
    tmem_alloc(smem_u32(tmem_slot), TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 9) {
    // ------------------------------- TMA loader -------------------------------
    if (lane == 0) {
      const int q_row0 = pair * 2 * BLOCK_M;
      load_tile(sbase + SMEM_Q, &tmap_q, bar(Q_FULL), q_row0, h, b, args.q_swap);
      load_tile(sbase + SMEM_K, &tmap_k, bar(K_FULL), 0, h, b, args.k_swap);
      load_tile(sbase + SMEM_Q + TILE_BYTES, &tmap_q, bar(Q_FULL + 1), q_row0 + BLOCK_M, h, b,
                args.q_swap);
      load_tile(sbase + SMEM_V, &tmap_v, bar(V_FULL), 0, h, b, args.v_swap);
      for (int j = 1; j < n_kv; ++j) {
        const int st = j & 1;
        const uint32_t par = ((j >> 1) & 1) ^ 1;
        if (!mbar_wait(bar(K_EMPTY + st), par, abort_flag, kStatusFlashTimeout)) break;
        load_tile(sbase + SMEM_K + st * TILE_BYTES, &tmap_k, bar(K_FULL + st), j * BLOCK_N, h, b,
                  args.k_swap);
        if (!mbar_wait(bar(V_EMPTY + st), par, abort_flag, kStatusFlashTimeout)) break;
        load_tile(sbase + SMEM_V + st * TILE_BYTES, &tmap_v, bar(V_FULL + st), j * BLOCK_N, h, b,
                  args.v_swap);
      }
    }
  } else if (warp == 8) {
    // ------------------------------- MMA issuer -------------------------------
    if (lane == 0) {
      const uint32_t q0 = sbase + SMEM_Q, q1 = q0 + TILE_BYTES;
      const uint32_t s0 = tmem_base + COL_S0, s1 = tmem_base + COL_S1;
      const uint32_t o0 = tmem_base + COL_O0, o1 = tmem_base + COL_O1;
      bool ok = mbar_wait(bar(Q_FULL), 0, abort_flag, kStatusFlashTimeout) &&
                mbar_wait(bar(K_FULL), 0, abort_flag, kStatusFlashTimeout);
      if (ok) {
        tc_fence_after();
        issue_qk(s0, q0, sbase + SMEM_K);
        tc_commit(bar(S_FULL));
        ok = mbar_wait(bar(Q_FULL + 1), 0, abort_flag, kStatusFlashTimeout);
      }
      if (ok) {
        tc_fence_after();
        issue_qk(s1, q1, sbase + SMEM_K);
        tc_commit(bar(S_FULL + 1));
        tc_commit(bar(K_EMPTY));
      }
      for (int j = 0; ok && j < n_kv; ++j) {
        const int st = j & 1;
        const uint32_t v_addr = sbase + SMEM_V + st * TILE_BYTES;
        const bool last = j + 1 == n_kv;
        const int st2 = (j + 1) & 1;
        const uint32_t k_next = sbase + SMEM_K + st2 * TILE_BYTES;
        if (!(ok = mbar_wait(bar(V_FULL + st), (j >> 1) & 1, abort_flag, kStatusFlashTimeout))) break;
        if (!(ok = mbar_wait(bar(P_FULL), j & 1, abort_flag, kStatusFlashTimeout))) break;
        tc_fence_after();
        issue_pv(o0, s0, v_addr, j != 0);
        if (last) {
          tc_commit(bar(O_FULL));
        } else {
          if (!(ok = mbar_wait(bar(K_FULL + st2), ((j + 1) >> 1) & 1, abort_flag, kStatusFlashTimeout))) break;
          tc_fence_after();
          issue_qk(s0, q0, k_next);
          tc_commit(bar(S_FULL));
        }
        if (!(ok = mbar_wait(bar(P_FULL + 1), j & 1, abort_flag, kStatusFlashTimeout))) break;
        tc_fence_after();
        issue_pv(o1, s1, v_addr, j != 0);
        tc_commit(bar(V_EMPTY + st));
        if (last) {
          tc_commit(bar(O_FULL + 1));
        } else {
          issue_qk(s1, q1, k_next);
          tc_commit(bar(S_FULL + 1));
          tc_commit(bar(K_EMPTY + st2));
        }
      }
    }
  } else {
    // ------------------------- softmax + output, one row per thread -------------------------
    const int t = warp >> 2;        // query tile of this warpgroup
    const int quarter = warp & 3;   // tensor-memory lane quarter
    const uint32_t lane_sel = (uint32_t)(quarter * 32) << 16;
    const uint32_t s_tmem = tmem_base + (t ? COL_S1 : COL_S0) + lane_sel;
    const uint32_t o_tmem = tmem_base + (t ? COL_O1 : COL_O0) + lane_sel;
    const float sl2 = args.scale_log2;
    const int tail_valid = args.S - (n_kv - 1) * BLOCK_N;  // valid columns of the last step
    float row_max = -INFINITY;  // raw-score domain, may lag the true max by < 2^8/sl2
    float row_sum = 0.f;
    bool ok = true;
    for (int j = 0; j < n_kv; ++j) {
      if (!(ok = mbar_wait(bar(S_FULL + t), j & 1, abort_flag, kStatusFlashTimeout))) break;
      tc_fence_after();
      uint32_t sraw[128];
      {
        uint32_t(&c0)[32] = *reinterpret_cast<uint32_t(*)[32]>(&sraw[0]);
        uint32_t(&c1)[32] = *reinterpret_cast<uint32_t(*)[32]>(&sraw[32]);
        uint32_t(&c2)[32] = *reinterpret_cast<uint32_t(*)[32]>(&sraw[64]);
        uint32_t(&c3)[32] = *reinterpret_cast<uint32_t(*)[32]>(&sraw[96]);
        tmem_ld_32x32b_x32(s_tmem + 0, c0);
        tmem_ld_32x32b_x32(s_tmem + 32, c1);
        tmem_ld_32x32b_x32(s_tmem + 64, c2);
        tmem_ld_32x32b_x32(s_tmem + 96, c3);
        tmem_wait_ld();
      }
      if (j + 1 == n_kv && tail_valid < BLOCK_N) {
#pragma unroll
        for (int c = 0; c < 128; ++c)
          if (c >= tail_valid) sraw[c] = 0xff800000u;  // -inf
      }
      float m = __uint_as_float(sraw[0]);
#pragma unroll
      for (int c = 1; c < 128; ++c) m = fmaxf(m, __uint_as_float(sraw[c]));
      // lazy rescale: raise the running max only when it lags by more than 2^8
      const bool raise = (m - row_max) * sl2 > 8.0f;  // true on the first step (row_max = -inf)
      if (__any_sync(0xffffffffu, raise)) {
        float alpha = 1.0f;
        if (raise) {
          alpha = ex2_approx((row_max - m) * sl2);  // 0 on the first step
          row_max = m;
          row_sum *= alpha;
        }
        if (j != 0) {
#pragma unroll 1
          for (int c = 0; c < HEAD_DIM; c += 32) {
            uint32_t o[32];
            tmem_ld_32x32b_x32(o_tmem + c, o);
            tmem_wait_ld();
#pragma unroll
            for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
            tmem_st_32x32b_x32(o_tmem + c, o);
          }
        }
      }
      const float neg_ms = -row_max * sl2;
      uint32_t p[64];
      float sum0 = 0.f, sum1 = 0.f;
#pragma unroll
      for (int c = 0; c < 64; ++c) {
        const float e0 = ex2_approx(fmaf(__uint_as_float(sraw[2 * c]), sl2, neg_ms));
        const float e1 = ex2_approx(fmaf(__uint_as_float(sraw[2 * c + 1]), sl2, neg_ms));
        sum0 += e0;
        sum1 += e1;
        p[c] = pack_bf16x2_rn(e0, e1);
      }
      row_sum += sum0 + sum1;
      {
        uint32_t(&p0)[32] = *reinterpret_cast<uint32_t(*)[32]>(&p[0]);
        uint32_t(&p1)[32] = *reinterpret_cast<uint32_t(*)[32]>(&p[32]);
        tmem_st_32x32b_x32(s_tmem + 0, p0);
        tmem_st_32x32b_x32(s_tmem + 32, p1);
      }
      tmem_wait_st();
      tc_fence_before();
      mbar_arrive(bar(P_FULL + t));
    }
    // ---- final: O / l -> bf16 -> global (BSHD) ----
    if (ok) ok = mbar_wait(bar(O_FULL + t), 0, abort_flag, kStatusFlashTimeout);
    if (ok) {
      tc_fence_after();
      const int row = (pair * 2 + t) * BLOCK_M + quarter * 32 + lane;
      const float inv = (row_sum == 0.f || row_sum != row_sum) ? 1.0f : 1.0f / row_sum;
      __nv_bfloat16* dst =
          args.out + (((int64_t)b * args.S + row) * args.H + h) * (int64_t)HEAD_DIM;
#pragma unroll 1
      for (int c = 0; c < HEAD_DIM; c += 32) {
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

  // ------------------------------- teardown -------------------------------
  __syncwarp();
  if (*abort_flag != 0) {
    const long long t0 = clock64();
    while (clock64() - t0 < 200000) {
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 8) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// 4-D bf16 map over a logical [B,H,S,128] tensor; the two middle dimensions are
// ordered by stride (ascending).  *swap = 1 when the order is (D, H, S, B).
int encode_qkv_map(CUtensorMap* map, const void* base, int B, int H, int S, const int64_t* st,
                   int* swap) {
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
    dims[2] = (cuuint64_t)S; strides[1] = (cuuint64_t)ss * 2; box[2] = BLOCK_M;
  } else {
    dims[1] = (cuuint64_t)S; strides[0] = (cuuint64_t)ss * 2; box[1] = BLOCK_M;
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

}  // namespace

int launch_flash_fwd(const void* q, const void* k, const void* v, void* out, int B, int H, int S,
                     const int64_t* qs, const int64_t* ks, const int64_t* vs, float scale,
                     cudaStream_t stream) {
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(flash_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         SMEM_TOTAL);
    if (e != cudaSuccess) return fail(B2_LAUNCH_FAILED, "flash_fwd: smem attribute: %s", cudaGetErrorString(e));
    attr_set = true;
  }
  if (H > 65535 || B > 65535) return fail(B2_TOO_LARGE, "flash_fwd: heads/batch exceed the launch grid");
  CUtensorMap tq, tk, tv;
  FlashArgs a;
  int st = encode_qkv_map(&tq, q, B, H, S, qs, &a.q_swap);
  if (st != B2_OK) return st;
  st = encode_qkv_map(&tk, k, B, H, S, ks, &a.k_swap);
  if (st != B2_OK) return st;
  st = encode_qkv_map(&tv, v, B, H, S, vs, &a.v_swap);
  if (st != B2_OK) return st;
  a.out = reinterpret_cast<__nv_bfloat16*>(out);
  a.B = B;
  a.H = H;
  a.S = S;
  a.n_kv = (S + BLOCK_N - 1) / BLOCK_N;
  a.scale_log2 = (float)((double)scale * 1.4426950408889634);
  const int pairs = (S + 2 * BLOCK_M - 1) / (2 * BLOCK_M);
  flash_fwd_kernel<<<dim3(pairs, H, B), NUM_THREADS, SMEM_TOTAL, stream>>>(tq, tk, tv, a);
  return check_launch("flash_fwd");
}

}  // namespace b2
