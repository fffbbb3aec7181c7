// Thin inline-PTX wrappers for the Blackwell (sm_100a) execution model used by the
// tensor-core kernels: mbarriers with BOUNDED waits, TMA tiled loads, tcgen05
// tensor-memory allocation, MMA issue, commit and loads, and the shared-memory /
// instruction descriptor encodings.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace b2 {

// Device-side error word of the including translation unit: bounded waits that give
// up OR a code into it instead of hanging or trapping.  Each tensor-core translation
// unit exports a reader (see read_clear_status_*), which b2_check_device_status() polls.
static __device__ unsigned int g_device_status = 0;

static inline unsigned int read_and_clear_device_status() {
  unsigned int word = 0, zero = 0;
  if (cudaMemcpyFromSymbol(&word, g_device_status, sizeof(word)) != cudaSuccess) return 0xffffffffu;
  if (word != 0) cudaMemcpyToSymbol(g_device_status, &zero, sizeof(zero));
  return word;
}

// Codes OR-ed into g_device_status by waits that gave up.
constexpr unsigned int kStatusGemmTimeout = 0x1u;
constexpr unsigned int kStatusFlashTimeout = 0x2u;
constexpr unsigned int kStatusSelfTest = 0x100u;


__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return (uint32_t)__cvta_generic_to_shared(p);
}

__device__ __forceinline__ uint32_t elect_one() {
  uint32_t pred;
  asm volatile(
      "{\n\t.reg .pred p;\n\telect.sync _|p, 0xffffffff;\n\tselp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(pred));
  return pred;
}

// ---- mbarrier ------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void fence_barrier_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
               : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ uint32_t mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok;
}
// Bounded wait: returns false (after recording `code` and raising *abort_flag) when the
// phase did not complete within the poll budget or another role already aborted.  Callers
// leave their loops and fall through to the common teardown.  The bound is a poll COUNT,
// not a clock reading: special-register reads are slow when the SM's transcendental unit
// is saturated, and these waits sit on the tensor pipe's critical path.
// (Measured on the attention kernel: a tighter poll loop takes issue slots from the
// arithmetic warps, -15%; try_wait with an explicit suspend-time hint of 20 ns to 10 us
// costs 1.5-5%.)
constexpr uint32_t kWaitPollLimit = 1u << 26;   // suspending try_wait polls (>= ~1 s)

__device__ __forceinline__ bool mbar_give_up(volatile int* abort_flag, unsigned int code) {
  atomicOr(&g_device_status, code);
  *abort_flag = 1;
  return false;
}
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag,
                                          unsigned int code) {
#pragma unroll 1
  for (uint32_t i = 0; i < kWaitPollLimit; ++i) {
    if (mbar_try_wait(bar, parity)) return true;
    if ((i & 255u) == 255u && *abort_flag != 0) break;
  }
  return mbar_give_up(abort_flag, code);
}

// ---- TMA (tiled bulk tensor loads, no multicast) ----------------------------------
__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap* m) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(m)) : "memory");
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* m, uint32_t bar, int x,
                                            int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4}], [%2];" ::"r"(dst),
      "l"(reinterpret_cast<uint64_t>(m)), "r"(bar), "r"(x), "r"(y)
      : "memory");
}
__device__ __forceinline__ void tma_load_4d(uint32_t dst, const CUtensorMap* m, uint32_t bar, int x,
                                            int y, int z, int w) {
  asm volatile(
      "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4, %5, %6}], [%2];" ::"r"(dst),
      "l"(reinterpret_cast<uint64_t>(m)), "r"(bar), "r"(x), "r"(y), "r"(z), "r"(w)
      : "memory");
}

// ---- TMA tiled store (shared -> global), bulk-group completion ----------------------------
// The shared-memory tile was written with ordinary stores: every writing thread executes
// fence_proxy_async_smem() after its stores and the threads synchronise before ONE thread
// issues the copy.  The source may be overwritten once bulk_wait_group_read<0>() returns in the
// issuing thread; parts of the box outside the tensor are not written.  The innermost
// coordinate x times the element size must be a multiple of 16 bytes.
__device__ __forceinline__ void fence_proxy_async_smem() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* m, uint32_t src, int x, int y) {
  asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];" ::"l"(
                   reinterpret_cast<uint64_t>(m)),
               "r"(src), "r"(x), "r"(y)
               : "memory");
}
__device__ __forceinline__ void bulk_commit_group() {
  asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}
template <int N>
__device__ __forceinline__ void bulk_wait_group_read() {
  asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
template <int N>
__device__ __forceinline__ void bulk_wait_group() {
  asm volatile("cp.async.bulk.wait_group %0;" ::"n"(N) : "memory");
}

// ---- tcgen05: tensor memory and MMA ----------------------------------------------------
__device__ __forceinline__ void tmem_alloc(uint32_t smem_dst, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_dst),
               "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols)
               : "memory");
}
__device__ __forceinline__ void tc_fence_before() {
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
// Arrives on the mbarrier once every MMA issued so far by this thread completed.
__device__ __forceinline__ void tc_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                   bar)
               : "memory");
}
// D[tmem] (+)= A[smem desc] * B[smem desc]
__device__ __forceinline__ void mma_i8_ss(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc,
                                          uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t}" ::"r"(d_tmem),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}

// High word of a 128-byte-swizzle shared-memory descriptor with an 8-row-group stride of
// 1024 bytes: SBO >> 4 = 64 (bits 32-45), version 1 (bits 46-47), swizzle code 2 (61-63).
constexpr uint32_t kDescHiSw128 = 64u | (1u << 14) | (2u << 29);
// Low word: start address >> 4 (bits 0-13) and the leading byte offset >> 4 (bits 16-29).
__device__ __forceinline__ uint32_t desc_lo(uint32_t smem_addr, uint32_t lbo_bytes) {
  return ((smem_addr >> 4) & 0x3fffu) | ((lbo_bytes >> 4) << 16);
}

// Eight / four MMAs whose descriptor low words are `base + compile-time offset`: the adds
// sit inside the asm block, next to their MMA, so the compiler cannot hoist sixteen
// loop-invariant words per batch into registers (the issuing warp runs on a small
// register budget).
#define B2_SS_BASE(off, pred)                                                      \
  "add.u32 ra, %1, " #off "; add.u32 rb, %2, " #off ";\n\t"                        \
  "mov.b64 da, {ra, %3}; mov.b64 db, {rb, %3};\n\t"                               \
  "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %4, " pred ";\n\t"
// K-major 128-row operands in two 64-element half tiles 16384 bytes apart (1024 in
// descriptor units), 32 bytes (2 units) of K per MMA.
__device__ __forceinline__ void mma_f16_ss_kmajor_x8(uint32_t d_tmem, uint32_t a_lo, uint32_t b_lo,
                                                     uint32_t idesc) {
  asm volatile(
      "{\n\t"
      ".reg .pred p0, p1;\n\t"
      ".reg .b64 da, db;\n\t"
      ".reg .b32 ra, rb;\n\t"
      "setp.ne.b32 p0, 0, 0;\n\t"
      "setp.eq.b32 p1, 0, 0;\n\t" B2_SS_BASE(0, "p0") B2_SS_BASE(2, "p1") B2_SS_BASE(4, "p1")
          B2_SS_BASE(6, "p1") B2_SS_BASE(1024, "p1") B2_SS_BASE(1026, "p1") B2_SS_BASE(1028, "p1")
              B2_SS_BASE(1030, "p1") "}" ::"r"(d_tmem),
      "r"(a_lo), "r"(b_lo), "r"(kDescHiSw128), "r"(idesc)
      : "memory");
}
#undef B2_SS_BASE
// Four MMAs with A in tensor memory: MMA i reads A at a_tmem + M_i*8 columns and B at
// b_lo + M_i*128 descriptor units, M = {M0, M0+1, M0+4, M0+5}.
template <int M0>
__device__ __forceinline__ void mma_f16_ts_x4(uint32_t d_tmem, uint32_t a_tmem, uint32_t b_lo,
                                              uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p0, p1;\n\t"
      ".reg .b64 db;\n\t"
      ".reg .b32 ra, rb;\n\t"
      "setp.ne.b32 p0, %5, 0;\n\t"
      "setp.eq.b32 p1, 0, 0;\n\t"
      "add.u32 ra, %1, %6; add.u32 rb, %2, %7; mov.b64 db, {rb, %3};\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [ra], db, %4, p0;\n\t"
      "add.u32 ra, %1, %8; add.u32 rb, %2, %9; mov.b64 db, {rb, %3};\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [ra], db, %4, p1;\n\t"
      "add.u32 ra, %1, %10; add.u32 rb, %2, %11; mov.b64 db, {rb, %3};\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [ra], db, %4, p1;\n\t"
      "add.u32 ra, %1, %12; add.u32 rb, %2, %13; mov.b64 db, {rb, %3};\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [ra], db, %4, p1;\n\t"
      "}" ::"r"(d_tmem),
      "r"(a_tmem), "r"(b_lo), "r"(kDescHiSw128), "r"(idesc), "r"(accumulate),
      "n"(M0 * 8), "n"(M0 * 128), "n"((M0 + 1) * 8), "n"((M0 + 1) * 128), "n"((M0 + 4) * 8),
      "n"((M0 + 4) * 128), "n"((M0 + 5) * 8), "n"((M0 + 5) * 128)
      : "memory");
}

// COUNT (2 or 4) MMAs with A in tensor memory over CONSECUTIVE 16-element slices of K:
// MMA i reads A at a_tmem + (M0+i)*8 columns and B at b_lo + (M0+i)*128 descriptor units.
// `accumulate` applies to the first MMA; the others always accumulate.
template <int M0, int COUNT>
__device__ __forceinline__ void mma_f16_ts_seq(uint32_t d_tmem, uint32_t a_tmem, uint32_t b_lo,
                                               uint32_t idesc, uint32_t accumulate) {
  static_assert(COUNT == 2 || COUNT == 4, "two or four MMAs per batch");
  if constexpr (COUNT == 4) {
    asm volatile(
        "{\n\t"
        ".reg .pred p0, p1;\n\t"
        ".reg .b64 db;\n\t"
        ".reg .b32 ra, rb;\n\t"
        "setp.ne.b32 p0, %5, 0;\n\t"
        "setp.eq.b32 p1, 0, 0;\n\t"
        "add.u32 ra, %1, %6; add.u32 rb, %2, %7; mov.b64 db, {rb, %3};\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [ra], db, %4, p0;\n\t"
        "add.u32 ra, %1, %8; add.u32 rb, %2, %9; mov.b64 db, {rb, %3};\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [ra], db, %4, p1;\n\t"
        "add.u32 ra, %1, %10; add.u32 rb, %2, %11; mov.b64 db, {rb, %3};\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [ra], db, %4, p1;\n\t"
        "add.u32 ra, %1, %12; add.u32 rb, %2, %13; mov.b64 db, {rb, %3};\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [ra], db, %4, p1;\n\t"
        "}" ::"r"(d_tmem),
        "r"(a_tmem), "r"(b_lo), "r"(kDescHiSw128), "r"(idesc), "r"(accumulate), "n"(M0 * 8),
        "n"(M0 * 128), "n"((M0 + 1) * 8), "n"((M0 + 1) * 128), "n"((M0 + 2) * 8), "n"((M0 + 2) * 128),
        "n"((M0 + 3) * 8), "n"((M0 + 3) * 128)
        : "memory");
  } else {
    asm volatile(
        "{\n\t"
        ".reg .pred p0, p1;\n\t"
        ".reg .b64 db;\n\t"
        ".reg .b32 ra, rb;\n\t"
        "setp.ne.b32 p0, %5, 0;\n\t"
        "setp.eq.b32 p1, 0, 0;\n\t"
        "add.u32 ra, %1, %6; add.u32 rb, %2, %7; mov.b64 db, {rb, %3};\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [ra], db, %4, p0;\n\t"
        "add.u32 ra, %1, %8; add.u32 rb, %2, %9; mov.b64 db, {rb, %3};\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [ra], db, %4, p1;\n\t"
        "}" ::"r"(d_tmem),
        "r"(a_tmem), "r"(b_lo), "r"(kDescHiSw128), "r"(idesc), "r"(accumulate), "n"(M0 * 8),
        "n"(M0 * 128), "n"((M0 + 1) * 8), "n"((M0 + 1) * 128)
        : "memory");
  }
}

__device__ __forceinline__ void named_barrier_sync(uint32_t id, uint32_t threads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}

__device__ __forceinline__ void tmem_wait_ld() {
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_wait_st() {
  asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}

// 32 lanes x 32 consecutive 32-bit columns: thread i of the warp receives lane
// (base lane + i), columns [col, col+32).
__device__ __forceinline__ void tmem_ld_32x32b_x32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]),
        "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
        "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_32x32b_x16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
        "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
        "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_st_32x32b_x16(uint32_t taddr, const uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};" ::"r"(taddr),
      "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
      "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
      : "memory");
}

__device__ __forceinline__ void tmem_st_32x32b_x8(uint32_t taddr, const uint32_t (&r)[8]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"r"(taddr),
      "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7])
      : "memory");
}

// ---- descriptors ----------------------------------------------------------------------
// Shared-memory matrix descriptor (sm_100 format): start address >> 4 in bits 0-13,
// leading byte offset >> 4 in 16-29, stride byte offset >> 4 in 32-45, version 1 in
// 46-47, swizzle mode in 61-63 (2 = 128-byte swizzle).
__host__ __device__ constexpr uint64_t make_smem_desc_sw128(uint32_t smem_addr, uint32_t lbo_bytes,
                                                            uint32_t sbo_bytes) {
  return (uint64_t)((smem_addr >> 4) & 0x3fffu) | ((uint64_t)((lbo_bytes >> 4) & 0x3fffu) << 16) |
         ((uint64_t)((sbo_bytes >> 4) & 0x3fffu) << 32) | (1ull << 46) | (2ull << 61);
}

// Instruction descriptor: D format bits 4-5 (1 = f32, 2 = s32), A format 7-9, B format
// 10-12 (f16 kind: 1 = bf16; i8 kind: 1 = signed), A/B major bits 15/16 (0 = K-major,
// 1 = MN-major), N >> 3 in 17-22, M >> 4 in 24-28.
__host__ __device__ constexpr uint32_t make_idesc(uint32_t d_fmt, uint32_t a_fmt, uint32_t b_fmt,
                                                  uint32_t a_mn_major, uint32_t b_mn_major,
                                                  uint32_t m, uint32_t n) {
  return (d_fmt << 4) | (a_fmt << 7) | (b_fmt << 10) | (a_mn_major << 15) | (b_mn_major << 16) |
         ((n >> 3) << 17) | ((m >> 4) << 24);
}

// Host: cuTensorMapEncodeTiled resolved through the runtime (no libcuda link).
typedef CUresult (*PFN_encodeTiled)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                    const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                    const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                    CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
PFN_encodeTiled get_encode_tiled();

}  // namespace b2
