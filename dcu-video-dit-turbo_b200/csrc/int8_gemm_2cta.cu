// INT8 GEMM, CTA-pair variant: two CTAs of a cluster (two SMs) compute one 256 x 256
// output tile with tcgen05.mma.cta_group::2.  Same contract and the same fused dequant
// epilogue as int8_gemm.cu (which stays the path for small M and the fallback).
//
// Why: a 128x256 tile per SM pulls 48 KB of operands through L2 per 128 bytes of K
// (170 int-ops per byte) and the profile shows the tensor pipe waiting on that delivery.
// Paired, each SM loads only ITS 128 rows of A and ITS 128 rows of W (32 KB per K step,
// 256 int-ops per byte); the pair's MMA reads both halves of W, one from each SM's shared
// memory.  Every load is a plain per-CTA TMA load (cta_group::2 form so that its bytes are
// counted on the leader's mbarrier); there is no multicast load anywhere.
//
//   CTA rank r in {0,1} of the pair owns tile rows [128r, 128r+128): its A rows, its half of
//   the W rows, its 128 x 256 int32 accumulator in its own tensor memory (double buffered).
//   warp 0  TMA producer (both CTAs): waits on its own `empty` barrier, loads into its own
//           shared memory, completes bytes on the LEADER's `full` barrier
//   warp 1  MMA issuer (leader only): 256x256x32 MMAs; tcgen05.commit multicasts to both
//           CTAs' `empty` / `tmem_full` barriers
//   warps 2-5 epilogue (both CTAs): own accumulator rows -> scales, bias, bf16; each warp stages
//           32 rows x 64 columns in shared memory (128-byte swizzle) and ONE lane hands the
//           tile to a TMA store, so the output leaves as whole 128-byte lines instead of 32
//           separate 16-byte pieces per instruction, and ragged edges are clipped by the
//           tensor map; arrive on the leader's `tmem_empty` barrier (remote for the peer)
// All mbarrier waits are bounded; both CTAs always meet at a final cluster barrier before
// either frees tensor memory or exits, so no CTA touches a retired peer.
#include <cstdlib>

#include "b2_common.cuh"
#include "b2_launch.h"
#include "gemm_epilogue.cuh"
#include "sm100_ptx.cuh"

namespace b2 {

unsigned int read_clear_status_gemm2() { return read_and_clear_device_status(); }

namespace {

constexpr int BM = 128;          // rows per CTA (256 per pair)
constexpr int BN = 256;          // columns per pair tile
constexpr int BNH = 128;         // W rows loaded per CTA
constexpr int BK = 128;          // bytes of K per stage
constexpr int UMMA_K = 32;
constexpr int STAGES = 6;
constexpr int A_BYTES = BM * BK;   // 16 KB
constexpr int B_BYTES = BNH * BK;  // 16 KB
constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int NUM_THREADS = 192;
constexpr int EPI_THREADS = 128;
constexpr int TMEM_COLS = 512;
constexpr int GROUP_M = 8;       // 256-row tiles swept per N pass

constexpr int SMEM_RING = STAGES * STAGE_BYTES;
constexpr int SMEM_OUT = (EPI_THREADS / 32) * kEpiStageBytes;  // one staging tile per epilogue warp
constexpr int SMEM_COLVEC = 2 * kColVecFloats * 4;  // [buf][scale|bias|gate][256] fp32
constexpr int NUM_BARS = 2 * STAGES + 4;
constexpr int SMEM_TOTAL = 1024 + SMEM_RING + SMEM_OUT + SMEM_COLVEC + NUM_BARS * 8 + 16;
static_assert(SMEM_TOTAL <= 227 * 1024, "shared memory budget");

struct Gemm2Args {
  int M, N, K;
  int tiles_m, tiles_n, num_tiles, k_blocks;  // tiles are 256 x 256
  EpilogueArgs epi;
};

__device__ __forceinline__ void decode_tile(int tile, const Gemm2Args& a, int& m_idx, int& n_idx) {
  const int per_group = GROUP_M * a.tiles_n;
  const int group = tile / per_group;
  const int first_m = group * GROUP_M;
  const int rows = min(GROUP_M, a.tiles_m - first_m);
  const int in_group = tile - group * per_group;
  m_idx = first_m + in_group % rows;
  n_idx = in_group / rows;
}

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
__device__ __forceinline__ void tma_load_2d_pair(uint32_t dst, const CUtensorMap* m, uint32_t bar_cluster,
                                                 int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4}], [%2];" ::"r"(dst),
      "l"(reinterpret_cast<uint64_t>(m)), "r"(bar_cluster), "r"(x), "r"(y)
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
__device__ __forceinline__ void mma_i8_ss_pair(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc,
                                               uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::i8 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(NUM_THREADS, 1)
int8_gemm_2cta_kernel(const __grid_constant__ CUtensorMap tmap_a,
                      const __grid_constant__ CUtensorMap tmap_b,
                      const __grid_constant__ CUtensorMap tmap_out, const Gemm2Args args) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  float* colvec = reinterpret_cast<float*>(smem + SMEM_RING + SMEM_OUT);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + SMEM_RING + SMEM_OUT + SMEM_COLVEC);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + NUM_BARS);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const uint32_t ring = smem_u32(smem);
  const uint32_t full0 = smem_u32(bars), empty0 = full0 + STAGES * 8;
  const uint32_t tfull0 = empty0 + STAGES * 8, tempty0 = tfull0 + 2 * 8;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();       // 0 = leader
  const int cluster_id = blockIdx.x >> 1;
  const int num_clusters = gridDim.x >> 1;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full0 + s * 8, 1);    // leader's: its producer's arrive.expect_tx
      mbar_init(empty0 + s * 8, 1);   // each CTA's: one multicast commit
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(tfull0 + b * 8, 1);                       // each CTA's: one multicast commit
      mbar_init(tempty0 + b * 8, 2 * (EPI_THREADS / 32)); // leader's: 4 warps of each CTA
    }
    *abort_flag = 0;
    fence_barrier_init();
    tma_prefetch_desc(&tmap_a);
    tma_prefetch_desc(&tmap_b);
    tma_prefetch_desc(&tmap_out);
  }
  if (warp == 1) {
    tmem_alloc_pair(smem_u32(tmem_slot), TMEM_COLS);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();   // both CTAs' barriers are initialised before any remote access
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------ TMA producer (both CTAs) ------------------------------
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = cluster_id; ok && tile < args.num_tiles; tile += num_clusters) {
        int m_idx, n_idx;
        decode_tile(tile, args, m_idx, n_idx);
        const int a_row = m_idx * 2 * BM + (int)rank * BM;
        const int b_row = n_idx * BN + (int)rank * BNH;
        for (int kb = 0; kb < args.k_blocks; ++kb) {
          if (!(ok = mbar_wait(empty0 + stage * 8, phase ^ 1, abort_flag, kStatusGemmTimeout))) break;
          const uint32_t full_leader = map_to_cta(full0 + stage * 8, 0);
          const uint32_t a_dst = ring + stage * STAGE_BYTES;
          if (rank == 0) mbar_expect_tx(full0 + stage * 8, 2 * STAGE_BYTES);  // both CTAs' bytes
          tma_load_2d_pair(a_dst, &tmap_a, full_leader, kb * BK, a_row);
          tma_load_2d_pair(a_dst + A_BYTES, &tmap_b, full_leader, kb * BK, b_row);
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------- MMA issuer (leader only) -------------------------------
    if (rank == 0 && lane == 0) {
      constexpr uint32_t idesc = make_idesc(/*s32*/ 2, /*s8*/ 1, /*s8*/ 1, 0, 0, 2 * BM, BN);
      int stage = 0;
      uint32_t phase = 0;
      int buf = 0;
      uint32_t buf_phase = 0;
      bool ok = true;
      for (int tile = cluster_id; ok && tile < args.num_tiles; tile += num_clusters) {
        if (!(ok = mbar_wait(tempty0 + buf * 8, buf_phase ^ 1, abort_flag, kStatusGemmTimeout))) break;
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + buf * BN;
        for (int kb = 0; kb < args.k_blocks; ++kb) {
          if (!(ok = mbar_wait(full0 + stage * 8, phase, abort_flag, kStatusGemmTimeout))) break;
          tc_fence_after();
          const uint32_t a_addr = ring + stage * STAGE_BYTES;
          const uint64_t adesc = make_smem_desc_sw128(a_addr, 16, 1024);
          const uint64_t bdesc = make_smem_desc_sw128(a_addr + A_BYTES, 16, 1024);
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k)
            mma_i8_ss_pair(d_tmem, adesc + 2 * k, bdesc + 2 * k, idesc, (kb | k) != 0);
          tc_commit_pair(empty0 + stage * 8);  // frees the stage in both CTAs
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
        if (!ok) break;
        tc_commit_pair(tfull0 + buf * 8);  // accumulators complete in both CTAs
        buf ^= 1;
        if (buf == 0) buf_phase ^= 1;
      }
    }
  } else {
    // --------------------------------- epilogue (both CTAs) ---------------------------------
    const int quarter = warp & 3;
    const int et = threadIdx.x - 64;
    int buf = 0;
    uint32_t buf_phase = 0;
    const EpilogueArgs& epi = args.epi;
    const bool fused = epi.out_i32 == nullptr;
    for (int tile = cluster_id; tile < args.num_tiles; tile += num_clusters) {
      int m_idx, n_idx;
      decode_tile(tile, args, m_idx, n_idx);
      const int col0 = n_idx * BN;
      float* cvec = colvec + buf * kColVecFloats;
      const int row = m_idx * 2 * BM + (int)rank * BM + quarter * 32 + lane;
      if (fused) {
        epilogue_prefetch_residual(epi, row, col0);
        epilogue_stage_columns(epi, cvec, col0, et);
        asm volatile("bar.sync 1, 128;" ::: "memory");
      }
      if (!mbar_wait(tfull0 + buf * 8, buf_phase, abort_flag, kStatusGemmTimeout)) break;
      tc_fence_after();
      const bool row_ok = row < epi.M;
      const float rsv = (fused && row_ok) ? epi.rs[row] : 0.f;
      const uint32_t taddr = tmem_base + buf * BN + ((uint32_t)(quarter * 32) << 16);
      if (fused && epi.swiglu) {
        // 128 accumulator columns (64 gate + 64 up) per step -> 64 output columns, staged and
        // stored like the dequant mode's 64-column step, at half the column offset
        const uint32_t stage = ring + SMEM_RING + quarter * kEpiStageBytes;
        const int row_warp = row - lane;   // global row of lane 0
#pragma unroll 1
        for (int c = 0; c < BN; c += 128) {
          if (col0 + c >= epi.N) break;
          if (lane == 0) bulk_wait_group_read<0>();   // the previous store has read the tile
          __syncwarp();
#pragma unroll 1
          for (int hh = 0; hh < 2; ++hh) {
            uint32_t vg[32], vu[32];
            uint32_t o[16];
            tmem_ld_32x32b_x32(taddr + c + 32 * hh, vg);
            tmem_ld_32x32b_x32(taddr + c + 64 + 32 * hh, vu);
            tmem_wait_ld();
            epilogue_swiglu_chunk(epi, vg, vu, c + 32 * hh, c + 64 + 32 * hh, rsv, cvec, o);
            epilogue_stage_write(stage, lane, hh, o);
          }
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0 && row_warp < epi.M) {
            tma_store_2d(&tmap_out, stage, (col0 + c) / 2, row_warp);
            bulk_commit_group();
          }
        }
      } else if (fused) {
        // 64 columns per step: two 32-column halves are computed into the warp's staging tile,
        // then one lane issues the TMA store of the 32 x 64 tile
        const uint32_t stage = ring + SMEM_RING + quarter * kEpiStageBytes;
        const int row_warp = row - lane;   // global row of lane 0
        uint4 x_next[4];   // residual mode: the next chunk's columns of x, loaded one chunk ahead
        epilogue_load_residual(epi, row, col0, x_next);
#pragma unroll 1
        for (int c = 0; c < BN; c += 64) {
          if (col0 + c >= epi.N) break;
          if (lane == 0) bulk_wait_group_read<0>();   // the previous store has read the tile
          __syncwarp();
#pragma unroll 1
          for (int hh = 0; hh < 2; ++hh) {
            uint32_t v[32];
            uint32_t o[16];
            uint4 x_now[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) x_now[i] = x_next[i];
            const int c_next = c + 32 * hh + 32;
            if (c_next < BN) epilogue_load_residual(epi, row, col0 + c_next, x_next);
            tmem_ld_32x32b_x32(taddr + c + 32 * hh, v);
            tmem_wait_ld();
#pragma unroll
            for (int i = 0; i < 16; ++i) o[i] = 0u;
            if (col0 + c + 32 * hh < epi.N)
              epilogue_compute_chunk(epi, v, col0 + c + 32 * hh, c + 32 * hh, rsv, cvec, x_now, o);
            epilogue_stage_write(stage, lane, hh, o);
          }
          fence_proxy_async_smem();
          __syncwarp();
          if (lane == 0 && row_warp < epi.M) {
            tma_store_2d(&tmap_out, stage, col0 + c, row_warp);
            bulk_commit_group();
          }
        }
      } else {
#pragma unroll 1
        for (int c = 0; c < BN; c += 32) {
          uint32_t v[32];
          tmem_ld_32x32b_x32(taddr + c, v);
          tmem_wait_ld();
          if (row_ok && col0 + c < epi.N) epilogue_store_chunk(epi, v, row, col0 + c, c, rsv, cvec);
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(map_to_cta(tempty0 + buf * 8, 0));
      buf ^= 1;
      if (buf == 0) buf_phase ^= 1;
    }
    if (lane == 0) bulk_wait_group<0>();   // this warp's stores are complete before the CTA may retire
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
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, TMEM_COLS);
  }
}

int encode_map(CUtensorMap* map, const void* base, int64_t rows, int64_t k, int box_rows) {
  PFN_encodeTiled enc = get_encode_tiled();
  if (!enc) return fail(B2_LAUNCH_FAILED, "int8_gemm: cuTensorMapEncodeTiled is unavailable");
  const cuuint64_t dims[2] = {(cuuint64_t)k, (cuuint64_t)rows};
  const cuuint64_t strides[1] = {(cuuint64_t)k};
  const cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)box_rows};
  const cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides,
                   box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(B2_LAUNCH_FAILED, "int8_gemm: tensor map encode failed (%d)", (int)r);
  return B2_OK;
}

// bf16 [M, N] output (or the in-place residual operand) as boxes of 64 columns x 32 rows,
// 128-byte swizzle: what one epilogue warp stages per step.
int encode_out_map(CUtensorMap* map, void* base, int64_t M, int64_t N) {
  PFN_encodeTiled enc = get_encode_tiled();
  if (!enc) return fail(B2_LAUNCH_FAILED, "int8_gemm: cuTensorMapEncodeTiled is unavailable");
  const cuuint64_t dims[2] = {(cuuint64_t)N, (cuuint64_t)M};
  const cuuint64_t strides[1] = {(cuuint64_t)N * 2};
  const cuuint32_t box[2] = {64, 32};
  const cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, base, dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                   CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(B2_LAUNCH_FAILED, "int8_gemm: output tensor map encode failed (%d)", (int)r);
  return B2_OK;
}

}  // namespace

// Returns -1 when the pair kernel does not apply (small M, no cluster support, or disabled
// with B2_GEMM_PAIR=0); the caller then uses the single-CTA kernel.
int launch_int8_gemm_pair(const int8_t* A, const int8_t* W, int32_t* out_i32, void* out_bf16,
                          const float* rs, const float* cs, const void* bias, int bias_kind,
                          const void* gate, void* residual, int64_t M, int64_t N, int64_t K,
                          cudaStream_t stream, int swiglu) {
  // slot.a = 1 when the pair kernel can run on this device, slot.b = resident clusters
  static PerDeviceSetup per_device;
  const DeviceSlot* slot = nullptr;
  const int setup_status = per_device.get("int8_gemm (CTA pair)", [](int dev, DeviceSlot& s) -> int {
    const char* env = getenv("B2_GEMM_PAIR");
    s.a = (env && env[0] == '0') ? 0 : 1;
    if (s.a && cudaFuncSetAttribute(int8_gemm_2cta_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                    SMEM_TOTAL) != cudaSuccess) {
      cudaGetLastError();
      s.a = 0;
    }
    if (s.a) {
      int sms = kNumSMsB200;
      cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
      cudaLaunchConfig_t cfg = {};
      cfg.gridDim = dim3((unsigned)(sms / 2 * 2));
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
      if (cudaOccupancyMaxActiveClusters(&n, int8_gemm_2cta_kernel, &cfg) != cudaSuccess || n < 1) {
        cudaGetLastError();
        s.a = 0;
      } else {
        s.b = n;
      }
    }
    return B2_OK;
  }, &slot);
  if (setup_status != B2_OK) return setup_status;
  const int enabled = slot->a, max_clusters = slot->b;
  if (!enabled || M < 2 * BM) return -1;
  const uint16_t* silu_lut = nullptr;
  if (swiglu) {
    const int lut_status = silu_table_device_pointer(stream, &silu_lut);
    if (lut_status != B2_OK) return lut_status;
  }

  CUtensorMap ta, tb, tout;
  int st = encode_map(&ta, A, M, K, BM);
  if (st != B2_OK) return st;
  st = encode_map(&tb, W, N, K, BNH);
  if (st != B2_OK) return st;
  // fused modes store through this map (the plain int32 mode stores directly and never uses it)
  void* bf16_dst = residual != nullptr ? residual : out_bf16;
  if (bf16_dst != nullptr) {
    st = encode_out_map(&tout, bf16_dst, M, swiglu ? N / 2 : N);
    if (st != B2_OK) return st;
  } else {
    tout = ta;
  }
  Gemm2Args a;
  a.M = (int)M;
  a.N = (int)N;
  a.K = (int)K;
  a.tiles_m = (int)((M + 2 * BM - 1) / (2 * BM));
  a.tiles_n = (int)((N + BN - 1) / BN);
  const int64_t tiles = (int64_t)a.tiles_m * a.tiles_n;
  if (tiles > 0x7fffffffLL) return fail(B2_TOO_LARGE, "int8_gemm: too many tiles");
  a.num_tiles = (int)tiles;
  a.k_blocks = (int)((K + BK - 1) / BK);
  a.epi.M = (int)M;
  a.epi.N = (int)N;
  a.epi.out_i32 = out_i32;
  a.epi.out_bf16 = reinterpret_cast<__nv_bfloat16*>(out_bf16);
  a.epi.rs = rs;
  a.epi.cs = cs;
  a.epi.bias = bias;
  a.epi.bias_kind = bias_kind;
  a.epi.gate = reinterpret_cast<const __nv_bfloat16*>(gate);
  a.epi.residual = reinterpret_cast<__nv_bfloat16*>(residual);
  a.epi.swiglu = swiglu;
  a.epi.silu_lut = silu_lut;
  const int clusters = a.num_tiles < max_clusters ? a.num_tiles : max_clusters;
  int8_gemm_2cta_kernel<<<clusters * 2, NUM_THREADS, SMEM_TOTAL, stream>>>(ta, tb, tout, a);
  return check_launch("int8_gemm (CTA pair)");
}

}  // namespace b2
