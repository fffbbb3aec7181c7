// b2_int8_linear_noalloc: the whole INT8 linear (quantise -> GEMM -> dequant) for callers
// that cannot provide scratch memory.
//
// b2_int8_linear needs two caller-provided scratch buffers (the quantised activation and
// its row scales).  Some callers have no way to get them: a host runtime that has already
// handed every byte of device memory to its own pool, a plugin that is only given its input
// and output tensors, or a serving loop where a device allocation (which may synchronise
// the whole device) is not acceptable once traffic has started.  For them this variant keeps
// the scratch in a fixed array inside the library image.
//
// Cost and limits, stated plainly:
//   * the array is kScratchBytes (32 MiB + 256 KiB) and every GPU that loads the library
//     holds it until the process exits;
//   * M <= 65536 rows and M*K <= 32 MiB of quantised activation; larger calls are refused
//     with B2_TOO_LARGE (use b2_int8_linear with your own scratch instead);
//   * all calls share the one array per device.  Nothing in it has to start at zero (the
//     quantise step overwrites every byte the GEMM later reads), so it is not cleared; it
//     keeps the previous call's contents.  Two calls whose kernels can overlap on the same
//     GPU (different streams, different threads) race on it: serialise them;
//   * the first call on each device looks up the array's device address (set-up below).
//     Make that first call during start-up, before any stream capture is begun.
#include <mutex>

#include "b2_common.cuh"
#include "b2_launch.h"

namespace b2 {
namespace {

constexpr int64_t kMaxRows = 65536;
constexpr int64_t kScaleBytes = kMaxRows * 4;            // 256 KiB of fp32 row scales
constexpr int64_t kQuantBytes = 32ll * 1024 * 1024;      // 32 MiB of int8 activations
constexpr int64_t kScratchBytes = kScaleBytes + kQuantBytes;

// File-scope device array.  In host code this NAME is only a host-side handle, not a
// device address: the address a kernel can use comes from cudaGetSymbolAddress.
static __device__ __align__(256) unsigned char g_linear_scratch[kScratchBytes];

constexpr int kMaxDevices = 64;
std::mutex g_setup_mutex;
unsigned char* g_scratch_ptr[kMaxDevices] = {};

// Once per device, with that device current: resolve the array's device address.
int scratch_for_current_device(unsigned char** out) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return fail(B2_LAUNCH_FAILED, "int8_linear_noalloc: cudaGetDevice: %s", cudaGetErrorString(e));
  if (dev < 0 || dev >= kMaxDevices) return fail(B2_TOO_LARGE, "int8_linear_noalloc: device index %d not supported", dev);
  std::lock_guard<std::mutex> lock(g_setup_mutex);
  if (g_scratch_ptr[dev] == nullptr) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_linear_scratch);
    if (e != cudaSuccess || p == nullptr)
      return fail(B2_LAUNCH_FAILED, "int8_linear_noalloc: cudaGetSymbolAddress: %s", cudaGetErrorString(e));
    g_scratch_ptr[dev] = static_cast<unsigned char*>(p);
  }
  *out = g_scratch_ptr[dev];
  return B2_OK;
}

}  // namespace
}  // namespace b2

using namespace b2;

extern "C" int b2_int8_linear_noalloc(const void* x, int input_act, const int8_t* W,
                                      const float* col_scale, const void* bias, int bias_kind,
                                      void* out, int64_t M, int64_t N, int64_t K, void* stream) {
  if (input_act != B2_ACT_NONE && input_act != B2_ACT_SWIGLU)
    return fail(B2_BAD_DTYPE, "int8_linear_noalloc: unknown input activation %d", input_act);
  if (bias_kind < B2_BIAS_NONE || bias_kind > B2_BIAS_FP32)
    return fail(B2_BAD_DTYPE, "int8_linear_noalloc: bias must be none, bfloat16, or float32");
  if (M < 0 || N < 0 || K <= 0) return fail(B2_BAD_SHAPE, "int8_linear_noalloc: bad size");
  if (M == 0 || N == 0) return B2_OK;
  if (K % 16 != 0 || N % 8 != 0)
    return fail(B2_NOT_WHITELISTED, "int8_linear_noalloc: K must be a multiple of 16 and N of 8");
  if (M > kMaxRows || M * K > kQuantBytes)
    return fail(B2_TOO_LARGE,
                "int8_linear_noalloc: M=%lld K=%lld exceeds the built-in scratch (at most %lld rows and "
                "%lld bytes of int8 activation); use b2_int8_linear with caller-provided scratch",
                (long long)M, (long long)K, (long long)kMaxRows, (long long)kQuantBytes);
  if (N > 0x7fffffffLL || K > 0x7fffffffLL) return fail(B2_TOO_LARGE, "int8_linear_noalloc: dimension exceeds int32");
  if (!x || !W || !col_scale || !out) return fail(B2_NULL_POINTER, "int8_linear_noalloc: null pointer");
  if (bias_kind != B2_BIAS_NONE && !bias) return fail(B2_NULL_POINTER, "int8_linear_noalloc: bias kind %d with a null bias", bias_kind);
  if (!aligned16(x) || !aligned16(W) || !aligned16(out))
    return fail(B2_BAD_STRIDE, "int8_linear_noalloc: x, W and out must be 16-byte aligned");

  unsigned char* scratch = nullptr;
  int st = scratch_for_current_device(&scratch);
  if (st != B2_OK) return st;
  float* s_scratch = reinterpret_cast<float*>(scratch);
  int8_t* q_scratch = reinterpret_cast<int8_t*>(scratch + kScaleBytes);

  cudaStream_t cs = (cudaStream_t)stream;
  st = input_act == B2_ACT_SWIGLU ? launch_swiglu_quantize(x, q_scratch, s_scratch, M, K, cs)
                                  : launch_quantize(x, q_scratch, s_scratch, M, K, cs);
  if (st != B2_OK) return st;
  return launch_int8_gemm(q_scratch, W, nullptr, out, s_scratch, col_scale, bias, bias_kind, nullptr, nullptr, M, N, K, cs);
}
