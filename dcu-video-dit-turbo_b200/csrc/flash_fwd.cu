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
#include "flash_common.cuh"

namespace b2 {

unsigned int read_clear_status_flash() { return read_and_clear_device_status(); }

namespace {

using namespace flash;

constexpr int KV_STAGES = 2;
constexpr int SMEM_Q = 0;                                   // 2 tiles
constexpr int SMEM_K = SMEM_Q + 2 * TILE_BYTES;             // KV_STAGES tiles
constexpr int SMEM_V = SMEM_K + KV_STAGES * TILE_BYTES;     // KV_STAGES tiles
constexpr int SMEM_BARS = SMEM_V + KV_STAGES * TILE_BYTES;  // mbarriers + tmem slot + abort
constexpr int SMEM_TOTAL = 1024 + SMEM_BARS + NUM_BARS * 8 + 16;

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
    softmax_role(
        args, tmem_base, bar0, abort_flag, warp, lane, n_kv, h, b,
        [&](int part, int t) { mbar_arrive(bar(P_PART + 2 * part + t)); },
        [&](int t) { return (pair * 2 + t) * BLOCK_M; });
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

}  // namespace

int launch_bounded_wait_selftest(cudaStream_t stream) {
  bounded_wait_selftest_kernel<<<1, 32, 0, stream>>>();
  return check_launch("bounded_wait_selftest");
}

int launch_flash_fwd(const void* q, const void* k, const void* v, void* out, int B, int H, int S,
                     const int64_t* qs, const int64_t* ks, const int64_t* vs, float scale,
                     cudaStream_t stream) {
  // opt-in (B2_FLASH_PAIR=1): two CTAs per 512 query rows sharing K and V; measured slower
  const int pair_status = launch_flash_fwd_pair(q, k, v, out, B, H, S, qs, ks, vs, scale, stream);
  if (pair_status >= 0) return pair_status;
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
