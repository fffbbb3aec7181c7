// INT8 GEMM for sm_100a: acc[M,N] = A[M,K] . W[N,K]^T on the 5th-generation tensor
// cores (tcgen05.mma kind::i8, int32 accumulators in tensor memory), with the
// dequant epilogue fused: out = bf16(bf16(float(acc)*(rs[m]*cs[n])) + bf16(bias[n])).
//
// Replaces, in one kernel, the reference's library GEMM call plus its separate
// epilogue kernel and the int32 [M,N] round trip through memory between them:
//   launcher/benchmark_launcher_v14_hires_int8_candidate.py:805-824 (GEMM call)
//   kernels/int8-epilogue/epilogue_kernel.hip:39-53 (epilogue arithmetic, bit-exact)
//
// Structure: persistent CTAs (one per SM), 128 x 256 output tiles, warp-specialised:
//   warp 0     TMA producer: A and W tiles (128-byte-swizzled, K-major) into a
//              4-stage shared-memory ring; plain per-CTA loads, no multicast
//   warp 1     MMA issuer: one thread issues tcgen05.mma 128x256x32 per 32 bytes
//              of K; tcgen05.commit releases ring stages and publishes accumulators
//   warps 2-5  epilogue: tcgen05.ld the accumulator (one row per thread), apply the
//              scales / bias, store bf16 (or raw int32).  The accumulator is double
//              buffered in tensor memory (2 x 256 columns) so the epilogue of tile i
//              overlaps the main loop of tile i+1.
// Ragged M, N and K edges rely on TMA zero fill for loads and on guards for stores.
// Every mbarrier wait is bounded; on a timeout the kernel records a status word,
// drains and returns.
#include "b2_common.cuh"
#include "b2_launch.h"
#include "gemm_epilogue.cuh"
#include "sm100_ptx.cuh"

namespace b2 {

PFN_encodeTiled get_encode_tiled() {
  static PFN_encodeTiled fn = nullptr;
  if (fn) return fn;
  void* p = nullptr;
  cudaDriverEntryPointQueryResult qres;
  if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) !=
          cudaSuccess ||
      qres != cudaDriverEntryPointSuccess)
    return nullptr;
  fn = reinterpret_cast<PFN_encodeTiled>(p);
  return fn;
}

unsigned int read_clear_status_gemm() { return read_and_clear_device_status(); }

namespace {

constexpr int BM = 128;
constexpr int BN = 256;
constexpr int BK = 128;  // bytes of K per stage = one 128-byte swizzle row
constexpr int UMMA_K = 32;
constexpr int STAGES = 4;
constexpr int A_BYTES = BM * BK;
constexpr int B_BYTES = BN * BK;
constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int NUM_THREADS = 192;
constexpr int EPI_THREADS = 128;
constexpr int TMEM_COLS = 512;
constexpr int GROUP_M = 16;  // M-tiles swept per N pass (keeps the A group in L2)

constexpr int SMEM_RING = STAGES * STAGE_BYTES;
constexpr int SMEM_COLVEC = 2 * kColVecFloats * 4;  // [buf][scale|bias|gate][256] fp32
constexpr int SMEM_BARS = 16 * 8;
constexpr int SMEM_TOTAL = 1024 /*align slack*/ + SMEM_RING + SMEM_COLVEC + SMEM_BARS + 16;

struct GemmArgs {
  int M, N, K;
  int tiles_m, tiles_n, num_tiles, k_blocks;
  EpilogueArgs epi;
};

__device__ __forceinline__ void decode_tile(int tile, const GemmArgs& a, int& m_idx, int& n_idx) {
  const int per_group = GROUP_M * a.tiles_n;
  const int group = tile / per_group;
  const int first_m = group * GROUP_M;
  const int rows = min(GROUP_M, a.tiles_m - first_m);
  const int in_group = tile - group * per_group;
  m_idx = first_m + in_group % rows;
  n_idx = in_group / rows;
}

__global__ void __launch_bounds__(NUM_THREADS, 1)
int8_gemm_kernel(const __grid_constant__ CUtensorMap tmap_a,
                 const __grid_constant__ CUtensorMap tmap_b, const GemmArgs args) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  float* colvec = reinterpret_cast<float*>(smem + SMEM_RING);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + SMEM_RING + SMEM_COLVEC);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 16);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const uint32_t ring = smem_u32(smem);
  const uint32_t full0 = smem_u32(bars), empty0 = full0 + STAGES * 8;
  const uint32_t tfull0 = empty0 + STAGES * 8, tempty0 = tfull0 + 2 * 8;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) {
      mbar_init(full0 + s * 8, 1);
      mbar_init(empty0 + s * 8, 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(tfull0 + b * 8, 1);
      mbar_init(tempty0 + b * 8, EPI_THREADS / 32);
    }
    *abort_flag = 0;
    fence_barrier_init();
    tma_prefetch_desc(&tmap_a);
    tma_prefetch_desc(&tmap_b);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(tmem_slot), TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; ok && tile < args.num_tiles; tile += gridDim.x) {
        int m_idx, n_idx;
        decode_tile(tile, args, m_idx, n_idx);
        for (int kb = 0; kb < args.k_blocks; ++kb) {
          if (!(ok = mbar_wait(empty0 + stage * 8, phase ^ 1, abort_flag, kStatusGemmTimeout))) break;
          const uint32_t full = full0 + stage * 8;
          const uint32_t a_dst = ring + stage * STAGE_BYTES;
          mbar_expect_tx(full, STAGE_BYTES);
          tma_load_2d(a_dst, &tmap_a, full, kb * BK, m_idx * BM);
          tma_load_2d(a_dst + A_BYTES, &tmap_b, full, kb * BK, n_idx * BN);
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------- MMA issuer -------------------------------
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc(/*s32*/ 2, /*s8*/ 1, /*s8*/ 1, 0, 0, BM, BN);
      int stage = 0;
      uint32_t phase = 0;
      int buf = 0;
      uint32_t buf_phase = 0;
      bool ok = true;
      for (int tile = blockIdx.x; ok && tile < args.num_tiles; tile += gridDim.x) {
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
          for (int k = 0; k < BK / UMMA_K; ++k) {
            // +2 per step: 32 bytes along K inside the swizzled 128-byte row
            mma_i8_ss(d_tmem, adesc + 2 * k, bdesc + 2 * k, idesc, (kb | k) != 0);
          }
          tc_commit(empty0 + stage * 8);  // stage reusable once these MMAs retire
          if (++stage == STAGES) {
            stage = 0;
            phase ^= 1;
          }
        }
        if (!ok) break;
        tc_commit(tfull0 + buf * 8);  // accumulator complete
        buf ^= 1;
        if (buf == 0) buf_phase ^= 1;
      }
    }
  } else {
    // --------------------------------- epilogue ---------------------------------
    const int quarter = warp & 3;  // tensor-memory lane quarter this warp may read
    const int et = threadIdx.x - 64;
    int buf = 0;
    uint32_t buf_phase = 0;
    const EpilogueArgs& epi = args.epi;
    const bool fused = epi.out_i32 == nullptr;
    for (int tile = blockIdx.x; tile < args.num_tiles; tile += gridDim.x) {
      int m_idx, n_idx;
      decode_tile(tile, args, m_idx, n_idx);
      const int col0 = n_idx * BN;
      float* cvec = colvec + buf * kColVecFloats;
      const int row = m_idx * BM + quarter * 32 + lane;
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
        // 64 gate + 64 up accumulator columns -> 64 outputs, stored directly
#pragma unroll 1
        for (int c = 0; c < BN; c += 128) {
#pragma unroll 1
          for (int hh = 0; hh < 2; ++hh) {
            uint32_t vg[32], vu[32];
            uint32_t o[16];
            tmem_ld_32x32b_x32(taddr + c + 32 * hh, vg);
            tmem_ld_32x32b_x32(taddr + c + 64 + 32 * hh, vu);
            tmem_wait_ld();
            if (row_ok && col0 + c < epi.N) {
              epilogue_swiglu_chunk(epi, vg, vu, c + 32 * hh, c + 64 + 32 * hh, rsv, cvec, o);
              uint4* dst = reinterpret_cast<uint4*>(epi.out_bf16 + (int64_t)row * (epi.N / 2) + (col0 + c) / 2 + 32 * hh);
#pragma unroll
              for (int j = 0; j < 4; ++j) dst[j] = make_uint4(o[4 * j], o[4 * j + 1], o[4 * j + 2], o[4 * j + 3]);
            }
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
      if (lane == 0) mbar_arrive(tempty0 + buf * 8);
      buf ^= 1;
      if (buf == 0) buf_phase ^= 1;
    }
  }

  // ------------------------------- teardown -------------------------------
  __syncwarp();
  if (*abort_flag != 0) {
    // give copies that may still be in flight time to land before the CTA retires
    const long long t0 = clock64();
    while (clock64() - t0 < 200000) {
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

int encode_k_major_map(CUtensorMap* map, const void* base, int64_t rows, int64_t k, int box_rows) {
  PFN_encodeTiled enc = get_encode_tiled();
  if (!enc) return fail(B2_LAUNCH_FAILED, "int8_gemm: cuTensorMapEncodeTiled is unavailable");
  const cuuint64_t dims[2] = {(cuuint64_t)k, (cuuint64_t)rows};
  const cuuint64_t strides[1] = {(cuuint64_t)k};  // bytes between rows
  const cuuint32_t box[2] = {(cuuint32_t)BK, (cuuint32_t)box_rows};
  const cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides,
                   box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(B2_LAUNCH_FAILED, "int8_gemm: tensor map encode failed (%d)", (int)r);
  return B2_OK;
}

}  // namespace

int launch_int8_gemm(const int8_t* A, const int8_t* W, int32_t* out_i32, void* out_bf16,
                     const float* rs, const float* cs, const void* bias, int bias_kind,
                     const void* gate, void* residual, int64_t M, int64_t N, int64_t K,
                     cudaStream_t stream, int swiglu) {
  // large M: two CTAs per 256x256 tile (less operand traffic per SM); else one CTA per tile
  const int pair_status = launch_int8_gemm_pair(A, W, out_i32, out_bf16, rs, cs, bias, bias_kind, gate, residual, M, N, K, stream, swiglu);
  if (pair_status >= 0) return pair_status;
  static PerDeviceSetup per_device;
  const DeviceSlot* slot = nullptr;
  const int setup_status = per_device.get("int8_gemm", [](int dev, DeviceSlot& s) -> int {
    cudaError_t e = cudaFuncSetAttribute(int8_gemm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         SMEM_TOTAL);
    if (e != cudaSuccess) return fail(B2_LAUNCH_FAILED, "int8_gemm: smem attribute: %s", cudaGetErrorString(e));
    s.a = kNumSMsB200;
    cudaDeviceGetAttribute(&s.a, cudaDevAttrMultiProcessorCount, dev);
    return B2_OK;
  }, &slot);
  if (setup_status != B2_OK) return setup_status;
  const uint16_t* silu_lut = nullptr;
  if (swiglu) {
    const int lut_status = silu_table_device_pointer(stream, &silu_lut);
    if (lut_status != B2_OK) return lut_status;
  }
  CUtensorMap ta, tb;
  int st = encode_k_major_map(&ta, A, M, K, BM);
  if (st != B2_OK) return st;
  st = encode_k_major_map(&tb, W, N, K, BN);
  if (st != B2_OK) return st;

  GemmArgs a;
  a.M = (int)M;
  a.N = (int)N;
  a.K = (int)K;
  a.tiles_m = (int)((M + BM - 1) / BM);
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

  const int sms = slot->a;
  const int grid = a.num_tiles < sms ? a.num_tiles : sms;
  int8_gemm_kernel<<<grid, NUM_THREADS, SMEM_TOTAL, stream>>>(ta, tb, a);
  return check_launch("int8_gemm");
}

}  // namespace b2
