// bf16 FlashAttention forward, CTA-pair form: two CTAs of a cluster (two SMs) run every
// MMA together with tcgen05.mma.cta_group::2.  Same mathematics, same softmax role and the
// same results as flash_fwd.cu; the pair changes only how the operands reach the tensor cores.
//
// OPT-IN (environment B2_FLASH_PAIR=1), not the default: it passes the same parity tests, but
// it measured 950 TFLOP/s against 1247 for the one-CTA kernel at 109099 tokens x 24 heads
// (905 against 1185-1191 at 23638).  The softmax -> MMA -> softmax hand-offs of a tile, which
// bound this kernel, now cross between two SMs three times per step (multicast commit out,
// remote mbarrier arrive back, and the pair's MMA waits for the slower of the two SMs), and with
// tensor memory full there is no third tile to hide the longer chain behind.
//
// Why: at long sequences the kernel runs against the power limit, so what counts is energy
// per FLOP.  With one CTA per SM every SM loads and reads a whole K tile and a whole V tile
// per step.  Paired, the two SMs share them: each CTA loads only ITS half of K (64 kv rows,
// the N half of Q.K^T's B operand) and ITS half of V (64 channels, the N half of P.V's B
// operand), and the pair's MMA reads one half from each SM's shared memory.  Shared-memory
// fills, shared-memory operand reads and L2 traffic for K/V per SM are halved; the MMA issue
// work is halved too (one issuer drives both SMs).  Every load is a plain per-CTA TMA load
// (cta_group::2 form so that its bytes are counted on the leader's mbarrier): no multicast.
//
//   A cluster owns 512 query rows of one (batch, head): tile t in {0,1} is 256 rows, of
//   which CTA rank r holds rows [128r, 128r+128) in its own tensor memory (S_t, O_t).
//   warps 0-7    softmax, one thread per score row (flash_common.cuh), in both CTAs; P column
//                groups are published on the LEADER's mbarriers (remote arrive for rank 1)
//   warp 8       MMA issuer, leader CTA only: 256x128x16 MMAs; tcgen05.commit multicasts
//                S / O "full" and K / V "empty" to both CTAs
//   warp 9       TMA loader, both CTAs: own Q rows, own K half, own V half; bytes complete on
//                the leader's "full" barriers
// Every mbarrier wait is bounded; both CTAs meet at a cluster barrier before either frees
// tensor memory or exits.
#include <cstdlib>

#include "flash_common.cuh"

namespace b2 {

unsigned int read_clear_status_flash2() { return read_and_clear_device_status(); }

namespace {

using namespace flash;

constexpr int KV_STAGES = 2;
constexpr int KHALF_BYTES = 64 * 128;            // one [64 kv rows x 64 channels] swizzled half of this CTA's K rows
constexpr int KTILE_BYTES = 2 * KHALF_BYTES;     // 16 KB: 64 kv rows x 128 channels
constexpr int VTILE_BYTES = 128 * 128;           // 16 KB: 128 kv rows x 64 channels
constexpr int SMEM_Q = 0;                                    // 2 tiles of this CTA's 128 rows
constexpr int SMEM_K = SMEM_Q + 2 * TILE_BYTES;              // KV_STAGES x 16 KB
constexpr int SMEM_V = SMEM_K + KV_STAGES * KTILE_BYTES;     // KV_STAGES x 16 KB
constexpr int SMEM_BARS = SMEM_V + KV_STAGES * VTILE_BYTES;  // mbarriers + tmem slot + abort
constexpr int SMEM_TOTAL = 1024 + SMEM_BARS + NUM_BARS * 8 + 16;

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// shared::cluster address of `addr` (a shared::cta address) in CTA `rank`
__device__ __forceinline__ uint32_t map_to_cta(uint32_t addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// per-CTA TMA load whose bytes are counted on a barrier given as a shared::cluster address
__device__ __forceinline__ void tma_load_4d_pair(uint32_t dst, const CUtensorMap* m, uint32_t bar_cluster,
                                                 int x, int y, int z, int w) {
  asm volatile(
      "cp.async.bulk.tensor.4d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4, %5, %6}], [%2];" ::"r"(dst),
      "l"(reinterpret_cast<uint64_t>(m)), "r"(bar_cluster), "r"(x), "r"(y), "r"(z), "r"(w)
      : "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t smem_dst, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_dst), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish_pair() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
// arrive on the same-offset barrier of both CTAs once all MMAs issued so far completed
__device__ __forceinline__ void tc_commit_pair(uint32_t bar) {
  asm volatile(
      "tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(bar),
      "h"((uint16_t)3)
      : "memory");
}

// Eight pair MMAs for S = Q.K^T.  A (Q): this CTA's 128 rows, K-major, two 64-channel half
// tiles 16384 bytes (1024 descriptor units) apart.  B (K): this CTA's 64 kv rows, K-major, two
// 64-channel half tiles 8192 bytes (512 units) apart.  32 bytes (2 units) of channels per MMA.
#define B2_SS_PAIR(aoff, boff, pred)                                                \
  "add.u32 ra, %1, " #aoff "; add.u32 rb, %2, " #boff ";\n\t"                       \
  "mov.b64 da, {ra, %3}; mov.b64 db, {rb, %3};\n\t"                                \
  "tcgen05.mma.cta_group::2.kind::f16 [%0], da, db, %4, " pred ";\n\t"
__device__ __forceinline__ void mma_f16_ss_kmajor_x8_pair(uint32_t d_tmem, uint32_t a_lo, uint32_t b_lo,
                                                          uint32_t idesc) {
  asm volatile(
      "{\n\t"
      ".reg .pred p0, p1;\n\t"
      ".reg .b64 da, db;\n\t"
      ".reg .b32 ra, rb;\n\t"
      "setp.ne.b32 p0, 0, 0;\n\t"
      "setp.eq.b32 p1, 0, 0;\n\t" B2_SS_PAIR(0, 0, "p0") B2_SS_PAIR(2, 2, "p1") B2_SS_PAIR(4, 4, "p1")
          B2_SS_PAIR(6, 6, "p1") B2_SS_PAIR(1024, 512, "p1") B2_SS_PAIR(1026, 514, "p1")
              B2_SS_PAIR(1028, 516, "p1") B2_SS_PAIR(1030, 518, "p1") "}" ::"r"(d_tmem),
      "r"(a_lo), "r"(b_lo), "r"(kDescHiSw128), "r"(idesc)
      : "memory");
}
#undef B2_SS_PAIR
// Four pair MMAs for O += P.V over consecutive 16-row kv slices M0..M0+3: A (P) at
// a_tmem + M*8 columns of each CTA's own tensor memory, B (V, MN-major, this CTA's 64
// channels) at b_lo + M*128 descriptor units (16 kv rows x 128 bytes).
template <int M0>
__device__ __forceinline__ void mma_f16_ts_x4_pair(uint32_t d_tmem, uint32_t a_tmem, uint32_t b_lo,
                                                   uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p0, p1;\n\t"
      ".reg .b64 db;\n\t"
      ".reg .b32 ra, rb;\n\t"
      "setp.ne.b32 p0, %5, 0;\n\t"
      "setp.eq.b32 p1, 0, 0;\n\t"
      "add.u32 ra, %1, %6; add.u32 rb, %2, %7; mov.b64 db, {rb, %3};\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], [ra], db, %4, p0;\n\t"
      "add.u32 ra, %1, %8; add.u32 rb, %2, %9; mov.b64 db, {rb, %3};\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], [ra], db, %4, p1;\n\t"
      "add.u32 ra, %1, %10; add.u32 rb, %2, %11; mov.b64 db, {rb, %3};\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], [ra], db, %4, p1;\n\t"
      "add.u32 ra, %1, %12; add.u32 rb, %2, %13; mov.b64 db, {rb, %3};\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], [ra], db, %4, p1;\n\t"
      "}" ::"r"(d_tmem),
      "r"(a_tmem), "r"(b_lo), "r"(kDescHiSw128), "r"(idesc), "r"(accumulate), "n"(M0 * 8),
      "n"(M0 * 128), "n"((M0 + 1) * 8), "n"((M0 + 1) * 128), "n"((M0 + 2) * 8), "n"((M0 + 2) * 128),
      "n"((M0 + 3) * 8), "n"((M0 + 3) * 128)
      : "memory");
}

static_assert(P_PARTS == 2, "the CTA-pair kernel publishes P in halves");

constexpr uint32_t kIdescQK2 = make_idesc(/*f32*/ 1, /*bf16*/ 1, /*bf16*/ 1, 0, 0, 2 * BLOCK_M, BLOCK_N);
constexpr uint32_t kIdescPV2 = make_idesc(1, 1, 1, 0, /*B MN-major*/ 1, 2 * BLOCK_M, HEAD_DIM);

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(NUM_THREADS, 1)
flash_fwd_2cta_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
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
  const uint32_t rank = cluster_ctarank();   // 0 = leader
  const int cluster = blockIdx.x >> 1, h = blockIdx.y, b = blockIdx.z;
  const int n_kv = args.n_kv;
  // global query row of this CTA's part of tile t
  auto tile_row0 = [&](int t) { return cluster * 4 * BLOCK_M + t * 2 * BLOCK_M + (int)rank * BLOCK_M; };

  if (threadIdx.x == 0) {
    for (int i = 0; i < NUM_BARS; ++i)
      mbar_init(bar(i), i >= P_PART ? 8 : 1);   // P groups (leader's): one arrival per softmax warp of the tile, both CTAs
    *abort_flag = 0;
    fence_barrier_init();
    tma_prefetch_desc(&tmap_q);
    tma_prefetch_desc(&tmap_k);
    tma_prefetch_desc(&tmap_v);
  }
  if (warp == kMmaWarp) {
    tmem_alloc_pair(smem_u32(tmem_slot), TMEM_COLS);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();   // both CTAs' barriers are initialised before any remote access
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp >= kMmaWarp) {
  asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(B2_FLASH_REGS_SERVICE));
  if (warp == kLoadWarp) {
    // ------------------------------- TMA loader (both CTAs) -------------------------------
    if (lane == 0) {
      // this CTA's rows / channels of every tile; bytes complete on the LEADER's barrier, which
      // the leader arms for both CTAs' bytes
      auto load_q = [&](int t) {
        const uint32_t full = map_to_cta(bar(Q_FULL + t), 0);
        if (rank == 0) mbar_expect_tx(bar(Q_FULL + t), 2 * TILE_BYTES);
        const uint32_t dst = sbase + SMEM_Q + t * TILE_BYTES;
        const int row0 = tile_row0(t);
        if (args.q_swap) {
          tma_load_4d_pair(dst, &tmap_q, full, 0, h, row0, b);
          tma_load_4d_pair(dst + HALF_BYTES, &tmap_q, full, 64, h, row0, b);
        } else {
          tma_load_4d_pair(dst, &tmap_q, full, 0, row0, h, b);
          tma_load_4d_pair(dst + HALF_BYTES, &tmap_q, full, 64, row0, h, b);
        }
      };
      auto load_k = [&](int j, int st) {   // kv rows [128j + 64r, +64), all 128 channels
        const uint32_t full = map_to_cta(bar(K_FULL + st), 0);
        if (rank == 0) mbar_expect_tx(bar(K_FULL + st), 2 * KTILE_BYTES);
        const uint32_t dst = sbase + SMEM_K + st * KTILE_BYTES;
        const int row0 = j * BLOCK_N + (int)rank * 64;
        if (args.k_swap) {
          tma_load_4d_pair(dst, &tmap_k, full, 0, h, row0, b);
          tma_load_4d_pair(dst + KHALF_BYTES, &tmap_k, full, 64, h, row0, b);
        } else {
          tma_load_4d_pair(dst, &tmap_k, full, 0, row0, h, b);
          tma_load_4d_pair(dst + KHALF_BYTES, &tmap_k, full, 64, row0, h, b);
        }
      };
      auto load_v = [&](int j, int st) {   // kv rows [128j, +128), channels [64r, +64)
        const uint32_t full = map_to_cta(bar(V_FULL + st), 0);
        if (rank == 0) mbar_expect_tx(bar(V_FULL + st), 2 * VTILE_BYTES);
        const uint32_t dst = sbase + SMEM_V + st * VTILE_BYTES;
        const int row0 = j * BLOCK_N, ch0 = (int)rank * 64;
        if (args.v_swap)
          tma_load_4d_pair(dst, &tmap_v, full, ch0, h, row0, b);
        else
          tma_load_4d_pair(dst, &tmap_v, full, ch0, row0, h, b);
      };
      load_q(0);
      load_k(0, 0);
      load_q(1);
      load_v(0, 0);
      for (int j = 1; j < n_kv; ++j) {
        const int st = j & 1;
        const uint32_t par = ((j >> 1) & 1) ^ 1;
        if (!mbar_wait(bar(K_EMPTY + st), par, abort_flag, kStatusFlashTimeout)) break;
        load_k(j, st);
        if (!mbar_wait(bar(V_EMPTY + st), par, abort_flag, kStatusFlashTimeout)) break;
        load_v(j, st);
      }
    }
  } else if (warp == kMmaWarp && rank == 0) {
    // ------------------------------- MMA issuer (leader only) -------------------------------
    const bool leader = elect_one() != 0;
    {
      const uint32_t s0 = tmem_base + COL_S0, s1 = tmem_base + COL_S1;
      const uint32_t o0 = tmem_base + COL_O0, o1 = tmem_base + COL_O1;
      const uint32_t q0 = desc_lo(sbase + SMEM_Q, 16), q1 = desc_lo(sbase + SMEM_Q + TILE_BYTES, 16);
      const uint32_t kA = desc_lo(sbase + SMEM_K, 16), kB = desc_lo(sbase + SMEM_K + KTILE_BYTES, 16);
      // V: MN-major, 64 channels per CTA = one 128-byte swizzle atom wide, so no second atom
      // along N exists and the leading byte offset is never used (any valid value)
      const uint32_t vA = desc_lo(sbase + SMEM_V, VTILE_BYTES);
      const uint32_t vB = desc_lo(sbase + SMEM_V + VTILE_BYTES, VTILE_BYTES);
      auto issue_qk = [&](uint32_t d, uint32_t q_lo, uint32_t k_lo) {
        if (leader) mma_f16_ss_kmajor_x8_pair(d, q_lo, k_lo, kIdescQK2);
      };
      auto pv_tile = [&](const int t, uint32_t d, uint32_t p_base, uint32_t v_lo, const int j) -> bool {
        if (!mbar_wait(bar(P_PART + t), j & 1, abort_flag, kStatusFlashTimeout)) return false;
        tc_fence_after();
        if (leader) mma_f16_ts_x4_pair<0>(d, p_base, v_lo, kIdescPV2, j != 0 ? 1u : 0u);
        if (!mbar_wait(bar(P_PART + 2 + t), j & 1, abort_flag, kStatusFlashTimeout)) return false;
        tc_fence_after();
        if (leader) mma_f16_ts_x4_pair<4>(d, p_base, v_lo, kIdescPV2, 1u);
        return true;
      };
      bool ok = mbar_wait(bar(Q_FULL), 0, abort_flag, kStatusFlashTimeout) &&
                mbar_wait(bar(K_FULL), 0, abort_flag, kStatusFlashTimeout);
      if (ok) {
        tc_fence_after();
        issue_qk(s0, q0, kA);
        if (leader) tc_commit_pair(bar(S_FULL));
        ok = mbar_wait(bar(Q_FULL + 1), 0, abort_flag, kStatusFlashTimeout);
      }
      if (ok) {
        tc_fence_after();
        issue_qk(s1, q1, kA);
        if (leader) tc_commit_pair(bar(S_FULL + 1));
        if (leader) tc_commit_pair(bar(K_EMPTY));
      }
      // One kv step; `st` is the ring stage of step j, the next step's K sits in the other.
      auto step = [&](const int j, const uint32_t vd, const uint32_t kd_next, const int st) -> bool {
        const bool last = j + 1 == n_kv;
        const int st2 = st ^ 1;
        if (!pv_tile(0, o0, s0, vd, j)) return false;
        if (last) {
          if (leader) tc_commit_pair(bar(O_FULL));
        } else {
          if (!mbar_wait(bar(K_FULL + st2), ((j + 1) >> 1) & 1, abort_flag, kStatusFlashTimeout)) return false;
          tc_fence_after();
          issue_qk(s0, q0, kd_next);
          if (leader) tc_commit_pair(bar(S_FULL));
        }
        if (!pv_tile(1, o1, s1, vd, j)) return false;
        if (leader) tc_commit_pair(bar(V_EMPTY + st));
        if (last) {
          if (leader) tc_commit_pair(bar(O_FULL + 1));
        } else {
          if (!mbar_wait(bar(V_FULL + st2), ((j + 1) >> 1) & 1, abort_flag, kStatusFlashTimeout)) return false;
          issue_qk(s1, q1, kd_next);
          if (leader) tc_commit_pair(bar(S_FULL + 1));
          if (leader) tc_commit_pair(bar(K_EMPTY + st2));
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
        [&](int part, int t) { mbar_arrive_cluster(map_to_cta(bar(P_PART + 2 * part + t), 0)); },
        tile_row0);
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
  cluster_sync_all();   // neither CTA retires (or frees tensor memory) before both are done
  if (warp == kMmaWarp) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, TMEM_COLS);
  }
}

}  // namespace

// Returns -1 when the pair kernel does not apply (not requested with B2_FLASH_PAIR=1, or no
// cluster support on the device); the caller then uses the one-CTA kernel.
int launch_flash_fwd_pair(const void* q, const void* k, const void* v, void* out, int B, int H, int S,
                          const int64_t* qs, const int64_t* ks, const int64_t* vs, float scale,
                          cudaStream_t stream) {
  static PerDeviceSetup per_device;   // slot.a = 1 when the pair kernel can run on this device
  const DeviceSlot* slot = nullptr;
  const int setup_status = per_device.get("flash_fwd (CTA pair)", [](int, DeviceSlot& s) -> int {
    const char* env = getenv("B2_FLASH_PAIR");
    s.a = (env && env[0] == '1') ? 1 : 0;
    if (!s.a) return B2_OK;
    cudaError_t e = cudaFuncSetAttribute(flash_fwd_2cta_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         SMEM_TOTAL);
    cudaFuncAttributes fa;
    if (e == cudaSuccess) e = cudaFuncGetAttributes(&fa, flash_fwd_2cta_kernel);
    if (e != cudaSuccess) {
      cudaGetLastError();
      s.a = 0;
      return B2_OK;
    }
    // the register hand-over must fit the launch allocation (see flash_common.cuh)
    if (2 * B2_FLASH_REGS_SOFTMAX + B2_FLASH_REGS_SERVICE > 3 * ((fa.numRegs + 7) / 8 * 8)) {
      s.a = 0;
      return B2_OK;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(2);
    cfg.blockDim = dim3(NUM_THREADS);
    cfg.dynamicSmemBytes = SMEM_TOTAL;
    cudaLaunchAttribute attr;
    attr.id = cudaLaunchAttributeClusterDimension;
    attr.val.clusterDim.x = 2;
    attr.val.clusterDim.y = 1;
    attr.val.clusterDim.z = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, flash_fwd_2cta_kernel, &cfg) != cudaSuccess || n < 1) {
      cudaGetLastError();
      s.a = 0;
    }
    return B2_OK;
  }, &slot);
  if (setup_status != B2_OK) return setup_status;
  if (!slot->a) return -1;
  if (H > 65535 || B > 65535) return fail(B2_TOO_LARGE, "flash_fwd: heads/batch exceed the launch grid");
  CUtensorMap tq, tk, tv;
  FlashArgs a;
  int st = encode_qkv_map(&tq, q, B, H, S, qs, &a.q_swap, BLOCK_M);
  if (st != B2_OK) return st;
  st = encode_qkv_map(&tk, k, B, H, S, ks, &a.k_swap, 64);
  if (st != B2_OK) return st;
  st = encode_qkv_map(&tv, v, B, H, S, vs, &a.v_swap, BLOCK_N);
  if (st != B2_OK) return st;
  a.out = reinterpret_cast<__nv_bfloat16*>(out);
  a.B = B;
  a.H = H;
  a.S = S;
  a.n_kv = (S + BLOCK_N - 1) / BLOCK_N;
  a.scale_log2 = (float)((double)scale * 1.4426950408889634);
  const int clusters = (S + 4 * BLOCK_M - 1) / (4 * BLOCK_M);
  flash_fwd_2cta_kernel<<<dim3(2 * clusters, H, B), NUM_THREADS, SMEM_TOTAL, stream>>>(tq, tk, tv, a);
  return check_launch("flash_fwd (CTA pair)");
}

}  // namespace b2
