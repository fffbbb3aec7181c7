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
//     warps 0-3    softmax for query tile 0, ONE thread per row: warp w reads the 32
//                  tensor-memory lanes of its quarter and keeps all 128 scores of its row in
//                  registers, so the row maximum and the row sum need no exchange between
//                  threads
//     warps 4-7    the same for query tile 1
//     warp 8       MMA issuer: S = Q.K^T (tcgen05.mma kind::f16, operands in shared
//                  memory) and O += P.V (P read from tensor memory, V from shared
//                  memory as an MN-major operand); accumulators S0,S1,O0,O1 fill the
//                  512 tensor-memory columns
//     warp 9       TMA loader: Q once, K and V tiles through a two-stage ring
//                  (128-byte swizzle; plain per-CTA loads, no multicast)
//     warps 10-11  idle; they complete the service warpgroup, which hands most of its
//                  registers to the softmax warpgroups (setmaxnreg)
//   The two tiles ping-pong: while one tile's softmax runs, the tensor core works on
//   the other tile's MMAs.  P overwrites S in place as bf16.
//   The exp2 unit delivers 16 results per clock per SM: 1024 clocks for a 128x128 tile, which
//   is exactly the time of the tile's two MMAs, so with every exponential on that unit the
//   softmax can at best tie with the tensor core.  A fixed share of the score pairs therefore
//   takes its exponential on the FMA pipe (2^floor(x) times a cubic in the fraction, relative
//   error 8.7e-5, a twentieth of the bf16 rounding P gets next), and the two pipes work side
//   by side.  The running max is raised, rescaling O and l, only when it lags by more than
//   2^8 in the exp2 domain (rare after the first steps; the final O/l is exact either way).
//   The scale-and-subtract and the row sum run as packed f32x2 instructions.  P is published
//   in column groups, each with its own mbarrier, so the tensor core starts O += P.V on the
//   first group while the later ones are still being exponentiated.
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
#define B2_FLASH_EMU_MASK 0x88
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

constexpr int SMEM_Q = 0;                                   // 2 tiles
constexpr int SMEM_K = SMEM_Q + 2 * TILE_BYTES;             // KV_STAGES tiles
constexpr int SMEM_V = SMEM_K + KV_STAGES * TILE_BYTES;     // KV_STAGES tiles
constexpr int SMEM_BARS = SMEM_V + KV_STAGES * TILE_BYTES;  // mbarriers + tmem slot + abort
constexpr int NUM_BARS = 14 + 2 * P_PARTS;
constexpr int SMEM_TOTAL = 1024 + SMEM_BARS + NUM_BARS * 8 + 16;

// mbarrier indices (two of each: ring stage or query tile); P_PART + 2*part + tile
enum { Q_FULL = 0, K_FULL = 2, K_EMPTY = 4, V_FULL = 6, V_EMPTY = 8, S_FULL = 10, O_FULL = 12,
       P_PART = 14 };

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

constexpr uint32_t kIdescQK = make_idesc(/*f32*/ 1, /*bf16*/ 1, /*bf16*/ 1, 0, 0, BLOCK_M, BLOCK_N);
constexpr uint32_t kIdescPV = make_idesc(1, 1, 1, 0, /*B MN-major*/ 1, BLOCK_M, HEAD_DIM);

__global__ void __launch_bounds__(NUM_THREADS, 1)
flash_fwd_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                 const __grid_constant__ CUtensorMap tmap_v, const FlashArgs args) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + SMEM_BARS);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + NUM_BARS);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  const uint32_t sbase = smem_u32(smem);
  const uint32_t bar0 = smem_u32(bars);
  auto bar = [&](int idx) -> uint32_t { return bar0 + idx * 8; };

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int pair = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int n_kv = args.n_kv;

  if (threadIdx.x == 0) {
    for (int i = 0; i < NUM_BARS; ++i)
      mbar_init(bar(i), i >= P_PART ? 4 : 1);   // P groups: one arrival per softmax warp of the tile
    *abort_flag = 0;
    fence_barrier_init();
    tma_prefetch_desc(&tmap_q);
    tma_prefetch_desc(&tmap_k);
    tma_prefetch_desc(&tmap_v);
  }
  if (warp == kMmaWarp) {
    tmem_alloc(smem_u32(tmem_slot), TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  // Registers move from the service warpgroup (MMA issuer, loader, two idle warps) to the
  // softmax warpgroups: each scheduler holds two softmax warps and one service warp.
  if (warp >= kMmaWarp) {
  asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(B2_FLASH_REGS_SERVICE));
  if (warp == kLoadWarp) {
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
  } else if (warp == kMmaWarp) {
    // ------------------------------- MMA issuer -------------------------------
    // The whole warp walks the loop and one elected lane issues the MMAs and commits: with
    // no lane-divergent region around them, addresses and descriptors stay warp-uniform.
    const bool leader = elect_one() != 0;
    {
      const uint32_t s0 = tmem_base + COL_S0, s1 = tmem_base + COL_S1;
      const uint32_t o0 = tmem_base + COL_O0, o1 = tmem_base + COL_O1;
      // Descriptor low words are derived from six base words right where an MMA batch is
      // issued (a handful of integer adds per batch), so the issuer needs few registers.
      const uint32_t q0 = desc_lo(sbase + SMEM_Q, 16), q1 = desc_lo(sbase + SMEM_Q + TILE_BYTES, 16);
      const uint32_t kA = desc_lo(sbase + SMEM_K, 16), kB = desc_lo(sbase + SMEM_K + TILE_BYTES, 16);
      const uint32_t vA = desc_lo(sbase + SMEM_V, HALF_BYTES);
      const uint32_t vB = desc_lo(sbase + SMEM_V + TILE_BYTES, HALF_BYTES);
      // S = Q.K^T: K-major half-tile pairs, 32 bytes of head dim per MMA
      auto issue_qk = [&](uint32_t d, uint32_t q_lo, uint32_t k_lo) {
        if (leader) mma_f16_ss_kmajor_x8(d, q_lo, k_lo, kIdescQK);
      };
      // O += P.V for one published column group of P (kv rows [part*128/P_PARTS, ...)).  P: 8
      // tensor-memory columns (16 bf16 of kv) per MMA; V: MN-major, 16 kv rows = 2048 bytes
      // per MMA.
      auto issue_pv = [&](uint32_t d, uint32_t p_base, uint32_t v_lo, const int part, uint32_t acc) {
        if (leader) {
          if constexpr (P_PARTS == 2) {
            if (part == 0)
              mma_f16_ts_seq<0, 4>(d, p_base, v_lo, kIdescPV, acc);
            else
              mma_f16_ts_seq<4, 4>(d, p_base, v_lo, kIdescPV, acc);
          } else {
            if (part == 0)
              mma_f16_ts_seq<0, 2>(d, p_base, v_lo, kIdescPV, acc);
            else if (part == 1)
              mma_f16_ts_seq<2, 2>(d, p_base, v_lo, kIdescPV, acc);
            else if (part == 2)
              mma_f16_ts_seq<4, 2>(d, p_base, v_lo, kIdescPV, acc);
            else
              mma_f16_ts_seq<6, 2>(d, p_base, v_lo, kIdescPV, acc);
          }
        }
      };
      // all column groups of one tile's P, each as soon as it is published
      auto pv_tile = [&](const int t, uint32_t d, uint32_t p_base, uint32_t v_lo, const int j) -> bool {
#pragma unroll
        for (int part = 0; part < P_PARTS; ++part) {
          if (!mbar_wait(bar(P_PART + 2 * part + t), j & 1, abort_flag, kStatusFlashTimeout)) return false;
          tc_fence_after();
          issue_pv(d, p_base, v_lo, part, (part != 0 || j != 0) ? 1u : 0u);
        }
        return true;
      };
      bool ok = mbar_wait(bar(Q_FULL), 0, abort_flag, kStatusFlashTimeout) &&
                mbar_wait(bar(K_FULL), 0, abort_flag, kStatusFlashTimeout);
      if (ok) {
        tc_fence_after();
        issue_qk(s0, q0, kA);
        if (leader) tc_commit(bar(S_FULL));
        ok = mbar_wait(bar(Q_FULL + 1), 0, abort_flag, kStatusFlashTimeout);
      }
      if (ok) {
        tc_fence_after();
        issue_qk(s1, q1, kA);
        if (leader) tc_commit(bar(S_FULL + 1));
        if (leader) tc_commit(bar(K_EMPTY));
      }
      // One kv step; `st` is the ring stage of step j, the next step's K sits in the other.
      auto step = [&](const int j, const uint32_t vd, const uint32_t kd_next, const int st) -> bool {
        const bool last = j + 1 == n_kv;
        const int st2 = st ^ 1;
        if (!pv_tile(0, o0, s0, vd, j)) return false;
        if (last) {
          if (leader) tc_commit(bar(O_FULL));
        } else {
          if (!mbar_wait(bar(K_FULL + st2), ((j + 1) >> 1) & 1, abort_flag, kStatusFlashTimeout)) return false;
          tc_fence_after();
          issue_qk(s0, q0, kd_next);
          if (leader) tc_commit(bar(S_FULL));
        }
        if (!pv_tile(1, o1, s1, vd, j)) return false;
        if (leader) tc_commit(bar(V_EMPTY + st));
        if (last) {
          if (leader) tc_commit(bar(O_FULL + 1));
        } else {
          // next step's V: waited for here, while the tensor core still has this step's MMAs
          // queued, so the wait is off the path between this step's last and the next step's
          // first MMA
          if (!mbar_wait(bar(V_FULL + st2), ((j + 1) >> 1) & 1, abort_flag, kStatusFlashTimeout)) return false;
          issue_qk(s1, q1, kd_next);
          if (leader) tc_commit(bar(S_FULL + 1));
          if (leader) tc_commit(bar(K_EMPTY + st2));
        }
        return true;
      };
      if (ok) ok = mbar_wait(bar(V_FULL), 0, abort_flag, kStatusFlashTimeout);
      for (int j = 0; ok && j < n_kv; j += 2) {
        ok = step(j, vA, kB, 0);
        if (ok && j + 1 < n_kv) ok = step(j + 1, vB, kA, 1);
      }
    }
  }
  } else {
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(B2_FLASH_REGS_SOFTMAX));
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
          if (lane == 0) mbar_arrive(bar(P_PART + 2 * (q / (8 / P_PARTS)) + t));  // one arrival per warp
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
      const int row = (pair * 2 + t) * BLOCK_M + row_in_tile;
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

  // ------------------------------- teardown -------------------------------
  __syncwarp();
  if (*abort_flag != 0) {
    const long long t0 = clock64();
    while (clock64() - t0 < 200000) {
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == kMmaWarp) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// Self-test of the bounded-wait machinery: one CTA waits on an mbarrier that nobody ever
// arrives on, with a deliberately tiny poll budget.  The wait gives up, records the
// status word and the kernel returns normally; the GPU context stays usable.
__global__ void bounded_wait_selftest_kernel() {
  __shared__ uint64_t never;
  __shared__ int abort_flag;
  if (threadIdx.x == 0) {
    mbar_init(smem_u32(&never), 1);
    abort_flag = 0;
    fence_barrier_init();
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    bool done = false;
    for (uint32_t i = 0; i < 4096u && !done; ++i) done = mbar_try_wait(smem_u32(&never), 0) != 0;
    if (!done) mbar_give_up(&abort_flag, kStatusSelfTest);
  }
  __syncthreads();
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

int launch_bounded_wait_selftest(cudaStream_t stream) {
  bounded_wait_selftest_kernel<<<1, 32, 0, stream>>>();
  return check_launch("bounded_wait_selftest");
}

int launch_flash_fwd(const void* q, const void* k, const void* v, void* out, int B, int H, int S,
                     const int64_t* qs, const int64_t* ks, const int64_t* vs, float scale,
                     cudaStream_t stream) {
  static PerDeviceSetup per_device;
  const DeviceSlot* slot = nullptr;
  const int setup_status = per_device.get("flash_fwd", [](int, DeviceSlot&) -> int {
    cudaError_t e = cudaFuncSetAttribute(flash_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         SMEM_TOTAL);
    if (e != cudaSuccess) return fail(B2_LAUNCH_FAILED, "flash_fwd: smem attribute: %s", cudaGetErrorString(e));
    cudaFuncAttributes fa;
    e = cudaFuncGetAttributes(&fa, flash_fwd_kernel);
    if (e != cudaSuccess) return fail(B2_LAUNCH_FAILED, "flash_fwd: attributes: %s", cudaGetErrorString(e));
    if (2 * B2_FLASH_REGS_SOFTMAX + B2_FLASH_REGS_SERVICE > 3 * ((fa.numRegs + 7) / 8 * 8))
      return fail(B2_LAUNCH_FAILED, "flash_fwd: register split %d/%d does not fit %d launch registers",
                  B2_FLASH_REGS_SOFTMAX, B2_FLASH_REGS_SERVICE, fa.numRegs);
    return B2_OK;
  }, &slot);
  if (setup_status != B2_OK) return setup_status;
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
