// Shared helpers for the libb2dit kernels: status plumbing, bf16 bit tricks and
// the row-scale arithmetic common to the quantizer family.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <mutex>

#include "../../include/b2dit.h"

namespace b2 {

// Thread-local error message behind b2_last_error().
void set_error(const char* fmt, ...);
int fail(int status, const char* fmt, ...);
int check_launch(const char* what);

constexpr int kNumSMsB200 = 148;

// One-time launch set-up that CUDA keeps PER DEVICE (cudaFuncSetAttribute, occupancy
// queries, the SM count): a process that drives several GPUs must repeat it on each, and
// two threads may make the first call at once.  get() runs `setup(device, slot)` once for
// the CURRENT device under a lock and afterwards hands back that device's slot.
struct DeviceSlot {
  bool ready = false;
  int a = 0, b = 0;   // kernel-specific values (e.g. enabled flag, cluster count, SM count)
};
class PerDeviceSetup {
 public:
  template <class Setup>
  int get(const char* what, Setup&& setup, const DeviceSlot** out) {
    int dev = -1;
    const cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return fail(B2_LAUNCH_FAILED, "%s: cudaGetDevice: %s", what, cudaGetErrorString(e));
    if (dev < 0 || dev >= kMaxDevices) return fail(B2_TOO_LARGE, "%s: device index %d not supported", what, dev);
    std::lock_guard<std::mutex> lock(mutex_);
    DeviceSlot& slot = slots_[dev];
    if (!slot.ready) {
      const int st = setup(dev, slot);
      if (st != B2_OK) return st;
      slot.ready = true;
    }
    *out = &slot;
    return B2_OK;
  }

 private:
  static constexpr int kMaxDevices = 64;
  std::mutex mutex_;
  DeviceSlot slots_[kMaxDevices];
};

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// ---- packed pairs of fp32 (sm_100: one f32x2 instruction does two lanes of work; every
// operation rounds to nearest even and keeps subnormals, exactly like its scalar form) ----
__device__ __forceinline__ uint64_t pack2(float lo, float hi) {
  uint64_t r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
  return r;
}
__device__ __forceinline__ void unpack2(uint64_t v, float& lo, float& hi) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ uint64_t fma2(uint64_t a, uint64_t b, uint64_t c) {
  uint64_t d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
  return d;
}
__device__ __forceinline__ uint64_t add2(uint64_t a, uint64_t b) {
  uint64_t d;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}
__device__ __forceinline__ uint64_t sub2(uint64_t a, uint64_t b) {
  uint64_t d;
  asm("sub.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}
__device__ __forceinline__ uint64_t mul2(uint64_t a, uint64_t b) {
  uint64_t d;
  asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}

// ---- bf16 <-> fp32 on packed pairs -----------------------------------------
__device__ __forceinline__ float bf16lo_to_f32(uint32_t w) { return __uint_as_float(w << 16); }
__device__ __forceinline__ float bf16hi_to_f32(uint32_t w) {
  return __uint_as_float(w & 0xffff0000u);
}
// Round two fp32 to bf16 (nearest even) and pack: lo in bits 0-15.
__device__ __forceinline__ uint32_t pack_bf16x2_rn(float lo, float hi) {
  __nv_bfloat162 p = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&p);
}
// The two bf16 of a packed word as a packed fp32 pair, and back (rounding to nearest even).
__device__ __forceinline__ uint64_t bf16x2_to_f32x2(uint32_t w) {
  return pack2(bf16lo_to_f32(w), bf16hi_to_f32(w));
}
__device__ __forceinline__ uint32_t f32x2_to_bf16x2_rn(uint64_t v) {
  float lo, hi;
  unpack2(v, lo, hi);
  return pack_bf16x2_rn(lo, hi);
}
// Packed bf16 product and sum, each rounded once to nearest even (subnormals kept).
__device__ __forceinline__ uint32_t bf16x2_mul_rn(uint32_t a, uint32_t b) {
  uint32_t d;
  asm("mul.rn.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
  return d;
}
__device__ __forceinline__ uint32_t bf16x2_add_rn(uint32_t a, uint32_t b) {
  uint32_t d;
  asm("add.rn.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
  return d;
}
// SiLU in fp32 exactly as the eager op computes it: g / (1 + expf(-g)) with the accurate
// expf and an IEEE division.
__device__ __forceinline__ float silu_exact(float g) {
  return __fdiv_rn(g, __fadd_rn(1.0f, expf(-g)));
}
// bf16( bf16(silu(g)) * u ) on a packed pair from the exact formula
// (kernels/swiglu-quant/swiglu_quant_kernel.hip:18-27 in the reference: two roundings).
__device__ __forceinline__ uint32_t swiglu_pair_exact(uint32_t g, uint32_t u) {
  const uint32_t s = pack_bf16x2_rn(silu_exact(bf16lo_to_f32(g)), silu_exact(bf16hi_to_f32(g)));
  // second rounding: the fp32 product of two bf16 values is exact, so rounding it to bf16 is
  // the packed bf16 multiply's single rounding
  return bf16x2_mul_rn(s, u);
}
__device__ __forceinline__ float round_bf16_f32(float v) {
  return __bfloat162float(__float2bfloat16_rn(v));
}

// Packed running max of magnitudes with NaN propagation (a NaN anywhere poisons the lane):
// ONE instruction per pair.  The magnitude of each half is max(|acc|, |w|); its sign bit is
// the xor of the operands' signs and carries no meaning (fold_absmax drops it).
// START THE CHAIN FROM A DATA WORD (acc = first word), never from a literal zero: with a
// constant-zero operand the instruction was observed to return max(0, w), i.e. to drop
// negative values (measured on sm_100a, CUDA 12.9; the plain form below is unaffected).
__device__ __forceinline__ uint32_t absmax_bf16x2(uint32_t acc, uint32_t w) {
  uint32_t d;
  asm("max.NaN.xorsign.abs.bf16x2 %0, %1, %2;" : "=r"(d) : "r"(acc), "r"(w));
  return d;
}
// Fold the two halves of a packed running max into one fp32 (NaN propagating).
__device__ __forceinline__ float fold_absmax(uint32_t acc) {
  acc &= 0x7fff7fffu;
  float lo = bf16lo_to_f32(acc), hi = bf16hi_to_f32(acc);
  return (lo != lo || hi != hi) ? __uint_as_float(0x7fc00000u) : fmaxf(lo, hi);
}
__device__ __forceinline__ float nanmax(float a, float b) {
  return (a != a || b != b) ? __uint_as_float(0x7fc00000u) : fmaxf(a, b);
}

// fp32(1/127): the reference multiplies by the reciprocal instead of dividing.
constexpr float kInv127 = 0.0078740157186985015869140625f;

// Row scale from the row's absmax (NaN if the row holds a NaN).  Returns the fp32
// scale that is stored, and through *recip the multiplier used for the elements:
// rn(1 / bf16(scale)).  For every normal bf16 divisor, x * rn(1/d) rounds to the
// same bf16 as the IEEE quotient x / d (checked exhaustively over all bf16 pairs),
// and the scale floor 1e-30 keeps the divisor normal.  A NaN or infinite divisor
// makes every quotient 0 or NaN, i.e. every output 0: *zero_row says so.
__device__ __forceinline__ float row_scale_from_absmax(float absmax, float* recip,
                                                       bool* zero_row) {
  float scale;
  if (absmax != absmax) {
    scale = __uint_as_float(0x7fc00000u);
  } else {
    scale = __fmul_rn(absmax, kInv127);
    if (scale < 1.0e-30f) scale = 1.0e-30f;
  }
  float sm = round_bf16_f32(scale);
  if (sm == 0.0f) sm = round_bf16_f32(1.1754943508222875e-38f);
  *zero_row = !(fabsf(sm) <= 3.4e38f);  // NaN or inf divisor
  *recip = __frcp_rn(sm);
  return scale;
}

// Quantise one packed pair with the row reciprocal: bf16(x*r) -> clamp -> round half even
// -> low byte.  Returns the two int8 in bits 0-7 and 8-15.
// Only the upper clamp can ever act: |x| <= absmax and the divisor is bf16(absmax/127)
// (or the 1e-30 floor), so |bf16(x*r)| <= 127.5, which rounds to +128 (clamped to 127) or
// to -128 (in range).  Rows with a NaN or infinite divisor never get here (zero_row).
__device__ __forceinline__ uint32_t quant_pair(uint32_t w, float r) {
  // the product and the integer rounding each run as one packed f32x2 instruction
  uint32_t p = f32x2_to_bf16x2_rn(mul2(bf16x2_to_f32x2(w), pack2(r, r)));
  asm("min.bf16x2 %0, %0, %1;" : "+r"(p) : "r"(0x42fe42feu));  // both halves: min(d, 127.0)
  // adding 1.5*2^23 rounds to nearest-even integer; the low mantissa byte is the
  // two's-complement int8
  float e0, e1;
  unpack2(add2(bf16x2_to_f32x2(p), pack2(12582912.0f, 12582912.0f)), e0, e1);
  return __byte_perm(__float_as_uint(e0), __float_as_uint(e1), 0x0040);  // byte0 = e0.byte0, byte1 = e1.byte0
}

// 8 bf16 (uint4) -> 8 int8 (uint2)
__device__ __forceinline__ uint2 quant_vec8(const uint4& v, float r) {
  uint32_t a = quant_pair(v.x, r), b = quant_pair(v.y, r);
  uint32_t c = quant_pair(v.z, r), d = quant_pair(v.w, r);
  uint2 o;
  o.x = __byte_perm(a, b, 0x5410);
  o.y = __byte_perm(c, d, 0x5410);
  return o;
}

// Named barrier among the TPR threads (a multiple of 32) that own row slot `slot` of NSLOTS:
// slots of a CTA do not wait for one another.  The barrier id is a compile-time constant per
// slot (ids 1..NSLOTS; 0 is __syncthreads), so the kernel declares only the barriers it uses.
template <int NSLOTS, int TPR, int K = 0>
__device__ __forceinline__ void slot_barrier(int slot) {
  static_assert(NSLOTS >= 1 && NSLOTS <= 15, "at most 15 named barriers besides __syncthreads");
  if constexpr (K < NSLOTS) {
    if (slot == K)   // slot is warp-uniform
      asm volatile("bar.sync %0, %1;" ::"n"(K + 1), "n"(TPR) : "memory");
    else
      slot_barrier<NSLOTS, TPR, K + 1>(slot);
  }
}

// Reduction over the TPR threads (TPR/32 warps, all in one row slot) that own a row; THREADS is
// the CTA size.  Each warp reduces with shuffles; across warps one value per warp goes through
// `buf` (one float per warp of the CTA) and ONE named barrier of the slot.  The caller passes a
// different `buf` to consecutive reductions (two in rotation are enough), so a buffer is
// rewritten only after a further barrier of the same slot, when every warp has read it.
template <int THREADS, int TPR, class Op>
__device__ __forceinline__ float slot_allreduce(float v, float* buf, int slot, Op op) {
#pragma unroll
  for (int off = 16; off > 0; off >>= 1) v = op(v, __shfl_xor_sync(0xffffffffu, v, off));
  if constexpr (TPR > 32) {
    constexpr int WPR = TPR / 32;
    const int warp = threadIdx.x >> 5;
    if ((threadIdx.x & 31) == 0) buf[warp] = v;
    slot_barrier<THREADS / TPR, TPR>(slot);
    const int first = (warp / WPR) * WPR;
    float m = buf[first];
#pragma unroll
    for (int i = 1; i < WPR; ++i) m = op(m, buf[first + i]);
    v = m;
  }
  return v;
}
struct NanMaxOp {
  __device__ __forceinline__ float operator()(float a, float b) const { return nanmax(a, b); }
};
struct SumOp {
  __device__ __forceinline__ float operator()(float a, float b) const { return a + b; }
};

__device__ __forceinline__ uint4 ldg_stream(const uint4* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}

}  // namespace b2
