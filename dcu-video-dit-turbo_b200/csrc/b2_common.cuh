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
__device__ __forceinline__ float round_bf16_f32(float v) {
  return __bfloat162float(__float2bfloat16_rn(v));
}

// |a|,|b| packed max with NaN propagation (a NaN anywhere poisons the lane).
__device__ __forceinline__ uint32_t absmax_bf16x2(uint32_t acc, uint32_t w) {
  __nv_bfloat162 a = *reinterpret_cast<__nv_bfloat162*>(&acc);
  __nv_bfloat162 b = __habs2(*reinterpret_cast<__nv_bfloat162*>(&w));
  __nv_bfloat162 m = __hmax2_nan(a, b);
  return *reinterpret_cast<uint32_t*>(&m);
}
// Fold the two halves of a packed running max into one fp32 (NaN propagating).
__device__ __forceinline__ float fold_absmax(uint32_t acc) {
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
  float d0 = __fmul_rn(bf16lo_to_f32(w), r);
  float d1 = __fmul_rn(bf16hi_to_f32(w), r);
  uint32_t p = pack_bf16x2_rn(d0, d1);
  asm("min.bf16x2 %0, %0, %1;" : "+r"(p) : "r"(0x42fe42feu));  // both halves: min(d, 127.0)
  float e0 = bf16lo_to_f32(p);
  float e1 = bf16hi_to_f32(p);
  // adding 1.5*2^23 rounds to nearest-even integer; the low mantissa byte is the
  // two's-complement int8
  uint32_t b0 = __float_as_uint(__fadd_rn(e0, 12582912.0f));
  uint32_t b1 = __float_as_uint(__fadd_rn(e1, 12582912.0f));
  return __byte_perm(b0, b1, 0x0040);  // byte0 = b0.byte0, byte1 = b1.byte0
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

__device__ __forceinline__ uint4 ldg_stream(const uint4* p) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}

}  // namespace b2
