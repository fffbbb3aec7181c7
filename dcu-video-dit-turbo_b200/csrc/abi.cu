// extern "C" surface of libb2dit.so: argument validation, status codes and the
// thread-local error string.  Nothing here allocates device memory; every check
// runs before the first launch.
#include <cmath>
#include <cstdarg>
#include <cstdio>

#include "b2_common.cuh"
#include "b2_launch.h"

namespace b2 {

static thread_local char t_error[512] = "";

void set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(t_error, sizeof(t_error), fmt, ap);
  va_end(ap);
}

int fail(int status, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(t_error, sizeof(t_error), fmt, ap);
  va_end(ap);
  return status;
}

int check_launch(const char* what) {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return fail(B2_LAUNCH_FAILED, "%s: launch failed: %s", what, cudaGetErrorString(e));
  return B2_OK;
}

}  // namespace b2

using namespace b2;

#define B2_REQUIRE_PTR(p)                                                  \
  do {                                                                     \
    if ((p) == nullptr) return fail(B2_NULL_POINTER, "%s: %s is null", __func__, #p); \
  } while (0)

extern "C" {

int b2_version(void) { return B2_ABI_VERSION; }

const char* b2_last_error(void) { return t_error; }

const char* b2_status_string(int s) {
  switch (s) {
    case B2_OK: return "OK";
    case B2_BAD_DTYPE: return "BAD_DTYPE";
    case B2_BAD_SHAPE: return "BAD_SHAPE";
    case B2_BAD_STRIDE: return "BAD_STRIDE";
    case B2_NOT_WHITELISTED: return "NOT_WHITELISTED";
    case B2_LAUNCH_FAILED: return "LAUNCH_FAILED";
    case B2_TIMEOUT: return "TIMEOUT";
    case B2_NULL_POINTER: return "NULL_POINTER";
    case B2_TOO_LARGE: return "TOO_LARGE";
  }
  return "UNKNOWN";
}

int b2_check_device_status(void* stream) {
  cudaError_t e = cudaStreamSynchronize((cudaStream_t)stream);
  if (e != cudaSuccess) return fail(B2_LAUNCH_FAILED, "stream synchronize: %s", cudaGetErrorString(e));
  const unsigned int word = read_clear_status_gemm() | read_clear_status_gemm2() | read_clear_status_flash() |
                            read_clear_status_flash2();
  if (word == 0xffffffffu) return fail(B2_LAUNCH_FAILED, "status word could not be read");
  if (word != 0) return fail(B2_TIMEOUT, "device-side bounded wait gave up (code 0x%x)", word);
  return B2_OK;
}

int b2_selftest_bounded_wait(void* stream) {
  return launch_bounded_wait_selftest((cudaStream_t)stream);
}

int b2_quantize_int8_rowwise(const void* x, int8_t* q, float* scale, int64_t M, int64_t K,
                             void* stream) {
  if (M < 0 || K < 0) return fail(B2_BAD_SHAPE, "quantize: negative size M=%lld K=%lld", (long long)M, (long long)K);
  if (M == 0) return B2_OK;
  B2_REQUIRE_PTR(scale);
  if (K == 0) return launch_fill_f32(scale, M, 1.0e-30f, (cudaStream_t)stream);
  B2_REQUIRE_PTR(x);
  B2_REQUIRE_PTR(q);
  if (reinterpret_cast<uintptr_t>(x) & 1u) return fail(B2_BAD_STRIDE, "quantize: x is not 2-byte aligned");
  if (reinterpret_cast<uintptr_t>(scale) & 3u) return fail(B2_BAD_STRIDE, "quantize: scale is not 4-byte aligned");
  return launch_quantize(x, q, scale, M, K, (cudaStream_t)stream);
}

int b2_swiglu_quantize_int8_rowwise(const void* x, int8_t* q, float* scale, int64_t M, int64_t K,
                                    void* stream) {
  if (M < 0 || K < 0) return fail(B2_BAD_SHAPE, "swiglu_quantize: negative size");
  if (M == 0 || K == 0) return B2_OK;
  B2_REQUIRE_PTR(x);
  B2_REQUIRE_PTR(q);
  B2_REQUIRE_PTR(scale);
  if (reinterpret_cast<uintptr_t>(x) & 1u) return fail(B2_BAD_STRIDE, "swiglu_quantize: x is not 2-byte aligned");
  if (reinterpret_cast<uintptr_t>(scale) & 3u) return fail(B2_BAD_STRIDE, "swiglu_quantize: scale is not 4-byte aligned");
  return launch_swiglu_quantize(x, q, scale, M, K, (cudaStream_t)stream);
}

static int check_epilogue_args(const char* who, const int32_t* acc, const float* rs, const float* cs,
                               const void* bias, int bias_kind, void* out, int64_t M, int64_t N) {
  if (M < 0 || N < 0) return fail(B2_BAD_SHAPE, "%s: negative size", who);
  if (bias_kind < B2_BIAS_NONE || bias_kind > B2_BIAS_FP32) return fail(B2_BAD_DTYPE, "%s: bias must be none, bfloat16, or float32 (kind=%d)", who, bias_kind);
  if (M == 0 || N == 0) return B2_OK;
  if (!acc || !rs || !cs || !out) return fail(B2_NULL_POINTER, "%s: null pointer", who);
  if (bias_kind != B2_BIAS_NONE && !bias) return fail(B2_NULL_POINTER, "%s: bias kind %d with a null bias", who, bias_kind);
  if ((reinterpret_cast<uintptr_t>(acc) & 3u) || (reinterpret_cast<uintptr_t>(rs) & 3u) ||
      (reinterpret_cast<uintptr_t>(cs) & 3u) || (reinterpret_cast<uintptr_t>(out) & 1u))
    return fail(B2_BAD_STRIDE, "%s: misaligned pointer", who);
  return -1;  // proceed
}

int b2_epilogue(const int32_t* acc, const float* rs, const float* cs, const void* bias,
                int bias_kind, void* out, int64_t M, int64_t N, void* stream) {
  int st = check_epilogue_args("epilogue", acc, rs, cs, bias, bias_kind, out, M, N);
  if (st >= 0) return st;
  return launch_epilogue(acc, rs, cs, bias, bias_kind, out, M, N, (cudaStream_t)stream);
}

int b2_epilogue_vec4(const int32_t* acc, const float* rs, const float* cs, void* out, int64_t M,
                     int64_t N, void* stream) {
  int st = check_epilogue_args("epilogue_vec4", acc, rs, cs, nullptr, B2_BIAS_NONE, out, M, N);
  if (st >= 0) return st;
  return launch_epilogue(acc, rs, cs, nullptr, B2_BIAS_NONE, out, M, N, (cudaStream_t)stream);
}

int b2_mod_scale_shift(void* x, const void* scale, const void* shift, int64_t M, int64_t C,
                       void* stream) {
  if (M < 0 || C < 0) return fail(B2_BAD_SHAPE, "mod_scale_shift: negative size");
  if (M == 0 || C == 0) return B2_OK;
  B2_REQUIRE_PTR(x);
  B2_REQUIRE_PTR(scale);
  B2_REQUIRE_PTR(shift);
  return launch_mod_scale_shift(x, scale, shift, M, C, (cudaStream_t)stream);
}

int b2_images_to_u8(const void* images, int32_t dtype, uint8_t* out, int64_t n, void* stream) {
  if (n < 0) return fail(B2_BAD_SHAPE, "images_to_u8: negative size");
  if (dtype < 0 || dtype > 2) return fail(B2_BAD_DTYPE, "images_to_u8: dtype must be 0 (float32), 1 (bfloat16) or 2 (float16)");
  if (n == 0) return B2_OK;
  if (!images || !out) return fail(B2_NULL_POINTER, "images_to_u8: null pointer");
  return launch_images_to_u8(images, dtype, out, n, (cudaStream_t)stream);
}

int b2_gate_residual(void* x, const void* y, const void* gate, int64_t M, int64_t C, void* stream) {
  if (M < 0 || C < 0) return fail(B2_BAD_SHAPE, "gate_residual: negative size");
  if (M == 0 || C == 0) return B2_OK;
  B2_REQUIRE_PTR(x);
  B2_REQUIRE_PTR(y);
  B2_REQUIRE_PTR(gate);
  return launch_gate_residual(x, y, gate, M, C, (cudaStream_t)stream);
}

static int check_ln(const char* who, const void* x, const void* scale, const void* shift, int64_t M,
                    int64_t C, float eps) {
  if (M < 0 || C <= 0) return fail(B2_BAD_SHAPE, "%s: bad size M=%lld C=%lld", who, (long long)M, (long long)C);
  if (C % 8 != 0) return fail(B2_NOT_WHITELISTED, "%s: C must be a multiple of 8", who);
  if (!(eps >= 0.0f)) return fail(B2_BAD_SHAPE, "%s: eps must be >= 0", who);
  if (M == 0) return B2_OK;
  if (!x || !scale || !shift) return fail(B2_NULL_POINTER, "%s: null pointer", who);
  if (!aligned16(x) || !aligned16(scale) || !aligned16(shift)) return fail(B2_BAD_STRIDE, "%s: pointers must be 16-byte aligned", who);
  return -1;
}

int b2_layernorm_mod(const void* x, const void* scale, const void* shift, void* out, int64_t M,
                     int64_t C, float eps, void* stream) {
  int st = check_ln("layernorm_mod", x, scale, shift, M, C, eps);
  if (st >= 0) return st;
  if (!out || !aligned16(out)) return fail(B2_BAD_STRIDE, "layernorm_mod: out null or misaligned");
  return launch_layernorm_mod(x, scale, shift, out, nullptr, nullptr, M, C, eps, false, (cudaStream_t)stream);
}

int b2_layernorm_mod_quant(const void* x, const void* scale, const void* shift, int8_t* q,
                           float* scale_out, int64_t M, int64_t C, float eps, void* stream) {
  int st = check_ln("layernorm_mod_quant", x, scale, shift, M, C, eps);
  if (st >= 0) return st;
  if (!q || !scale_out) return fail(B2_NULL_POINTER, "layernorm_mod_quant: null output");
  if (reinterpret_cast<uintptr_t>(q) & 7u) return fail(B2_BAD_STRIDE, "layernorm_mod_quant: q must be 8-byte aligned");
  return launch_layernorm_mod(x, scale, shift, nullptr, q, scale_out, M, C, eps, true, (cudaStream_t)stream);
}

int b2_qk_norm_rope(void* qkv, const void* qw, const void* kw, const float* cos_tab,
                    const float* sin_tab, int64_t S, int32_t H, float eps, void* stream) {
  if (S < 0 || H <= 0) return fail(B2_BAD_SHAPE, "qk_norm_rope: bad size");
  if (S == 0) return B2_OK;
  if (!qkv || !qw || !kw || !cos_tab || !sin_tab) return fail(B2_NULL_POINTER, "qk_norm_rope: null pointer");
  if (!aligned16(qkv) || !aligned16(qw) || !aligned16(kw) || !aligned16(cos_tab) || !aligned16(sin_tab))
    return fail(B2_BAD_STRIDE, "qk_norm_rope: pointers must be 16-byte aligned");
  return launch_qk_norm_rope(qkv, qw, kw, cos_tab, sin_tab, S, H, eps, (cudaStream_t)stream);
}

int b2_qk_norm_rope_pack(const void* qkv, void* send, const void* qw, const void* kw,
                         const float* cos_tab, const float* sin_tab, int64_t L, int32_t H,
                         int32_t world, int32_t chunks, float eps, void* stream) {
  if (L < 0 || H <= 0 || world <= 0 || chunks <= 0 || H % (world * chunks) != 0)
    return fail(B2_BAD_SHAPE, "qk_norm_rope_pack: world*chunks must divide the head count (L=%lld H=%d world=%d chunks=%d)",
                (long long)L, H, world, chunks);
  if (L == 0) return B2_OK;
  if (!qkv || !send || !qw || !kw || !cos_tab || !sin_tab) return fail(B2_NULL_POINTER, "qk_norm_rope_pack: null pointer");
  if (!aligned16(qkv) || !aligned16(send) || !aligned16(qw) || !aligned16(kw) || !aligned16(cos_tab) || !aligned16(sin_tab))
    return fail(B2_BAD_STRIDE, "qk_norm_rope_pack: pointers must be 16-byte aligned");
  if (qkv == send) return fail(B2_BAD_STRIDE, "qk_norm_rope_pack: the send buffer must not alias the input");
  if (!(eps >= 0.f)) return fail(B2_BAD_SHAPE, "qk_norm_rope_pack: eps must be non-negative");
  return launch_qk_norm_rope_pack(qkv, send, qw, kw, cos_tab, sin_tab, L, H, world, chunks, eps, (cudaStream_t)stream);
}

int b2_qk_norm_rope_scatter(const void* qkv, void* const* recv_bases, const void* qw, const void* kw,
                            const float* cos_tab, const float* sin_tab, int64_t L, int32_t H,
                            int32_t world, int32_t chunks, int64_t row0, int64_t S, float eps,
                            void* stream) {
  if (L < 0 || H <= 0 || world <= 0 || chunks <= 0 || H % (world * chunks) != 0)
    return fail(B2_BAD_SHAPE, "qk_norm_rope_scatter: world*chunks must divide the head count (L=%lld H=%d world=%d chunks=%d)",
                (long long)L, H, world, chunks);
  if (world > 8) return fail(B2_NOT_WHITELISTED, "qk_norm_rope_scatter: at most 8 ranks (world=%d)", world);
  if (row0 < 0 || S < 0 || row0 + L > S)
    return fail(B2_BAD_SHAPE, "qk_norm_rope_scatter: rows [%lld, %lld) do not fit a sequence of %lld",
                (long long)row0, (long long)(row0 + L), (long long)S);
  if (L == 0) return B2_OK;
  if (!qkv || !recv_bases || !qw || !kw || !cos_tab || !sin_tab) return fail(B2_NULL_POINTER, "qk_norm_rope_scatter: null pointer");
  if (!aligned16(qkv) || !aligned16(qw) || !aligned16(kw) || !aligned16(cos_tab) || !aligned16(sin_tab))
    return fail(B2_BAD_STRIDE, "qk_norm_rope_scatter: pointers must be 16-byte aligned");
  for (int p = 0; p < world; ++p) {
    if (!recv_bases[p]) return fail(B2_NULL_POINTER, "qk_norm_rope_scatter: receive buffer of rank %d is null", p);
    if (!aligned16(recv_bases[p])) return fail(B2_BAD_STRIDE, "qk_norm_rope_scatter: receive buffer of rank %d is not 16-byte aligned", p);
    if (recv_bases[p] == qkv) return fail(B2_BAD_STRIDE, "qk_norm_rope_scatter: a receive buffer must not alias the input");
  }
  if (!(eps >= 0.f)) return fail(B2_BAD_SHAPE, "qk_norm_rope_scatter: eps must be non-negative");
  return launch_qk_norm_rope_scatter(qkv, recv_bases, qw, kw, cos_tab, sin_tab, L, H, world, chunks, row0, S,
                                     eps, (cudaStream_t)stream);
}

int b2_quantize_int8_rowwise_gathered(const void* x, int8_t* q, float* scale, int64_t M, int64_t K,
                                      int32_t world, int32_t chunks, void* stream) {
  if (M < 0 || K <= 0 || world <= 0 || chunks <= 0 || K % ((int64_t)world * chunks * 8) != 0 || K > 16384)
    return fail(B2_BAD_SHAPE, "quantize_int8_rowwise_gathered: K=%lld must be a multiple of 8*world*chunks (world=%d chunks=%d), at most 16384",
                (long long)K, world, chunks);
  if (M == 0) return B2_OK;
  if (!x || !q || !scale) return fail(B2_NULL_POINTER, "quantize_int8_rowwise_gathered: null pointer");
  if (!aligned16(x) || (reinterpret_cast<uintptr_t>(q) & 7u))
    return fail(B2_BAD_STRIDE, "quantize_int8_rowwise_gathered: x must be 16-byte and q 8-byte aligned");
  return launch_quantize_gathered(x, q, scale, M, K, world, chunks, (cudaStream_t)stream);
}

static int check_gemm(const char* who, const int8_t* A, const int8_t* W, int64_t M, int64_t N,
                      int64_t K, int n_mult) {
  if (M < 0 || N < 0 || K < 0) return fail(B2_BAD_SHAPE, "%s: negative size", who);
  if (M == 0 || N == 0) return B2_OK;
  if (K == 0) return fail(B2_BAD_SHAPE, "%s: K must be positive", who);
  if (K % 16 != 0) return fail(B2_NOT_WHITELISTED, "%s: K=%lld must be a multiple of 16", who, (long long)K);
  if (N % n_mult != 0) return fail(B2_NOT_WHITELISTED, "%s: N=%lld must be a multiple of %d", who, (long long)N, n_mult);
  if (M > 0x7fffffffLL || N > 0x7fffffffLL || K > 0x7fffffffLL) return fail(B2_TOO_LARGE, "%s: dimension exceeds int32", who);
  if (!A || !W) return fail(B2_NULL_POINTER, "%s: null operand", who);
  if (!aligned16(A) || !aligned16(W)) return fail(B2_BAD_STRIDE, "%s: operands must be 16-byte aligned", who);
  return -1;
}

int b2_int8_gemm(const int8_t* A, const int8_t* W, int32_t* acc, int64_t M, int64_t N, int64_t K,
                 void* stream) {
  int st = check_gemm("int8_gemm", A, W, M, N, K, 4);
  if (st >= 0) return st;
  if (!acc || !aligned16(acc)) return fail(B2_BAD_STRIDE, "int8_gemm: acc null or not 16-byte aligned");
  return launch_int8_gemm(A, W, acc, nullptr, nullptr, nullptr, nullptr, B2_BIAS_NONE, nullptr, nullptr, M, N, K, (cudaStream_t)stream);
}

int b2_int8_gemm_dequant(const int8_t* A, const float* rs, const int8_t* W, const float* cs,
                         const void* bias, int bias_kind, void* out, int64_t M, int64_t N,
                         int64_t K, void* stream) {
  if (bias_kind < B2_BIAS_NONE || bias_kind > B2_BIAS_FP32) return fail(B2_BAD_DTYPE, "int8_gemm_dequant: bias must be none, bfloat16, or float32");
  int st = check_gemm("int8_gemm_dequant", A, W, M, N, K, 8);
  if (st >= 0) return st;
  if (!rs || !cs || !out) return fail(B2_NULL_POINTER, "int8_gemm_dequant: null pointer");
  if (bias_kind != B2_BIAS_NONE && !bias) return fail(B2_NULL_POINTER, "int8_gemm_dequant: bias kind %d with a null bias", bias_kind);
  if (!aligned16(out)) return fail(B2_BAD_STRIDE, "int8_gemm_dequant: out must be 16-byte aligned");
  return launch_int8_gemm(A, W, nullptr, out, rs, cs, bias, bias_kind, nullptr, nullptr, M, N, K, (cudaStream_t)stream);
}

int b2_int8_gemm_dequant_residual(const int8_t* A, const float* rs, const int8_t* W,
                                  const float* cs, const void* bias, int bias_kind,
                                  const void* gate, void* x_inout, int64_t M, int64_t N,
                                  int64_t K, void* stream) {
  if (bias_kind < B2_BIAS_NONE || bias_kind > B2_BIAS_FP32) return fail(B2_BAD_DTYPE, "int8_gemm_dequant_residual: bias must be none, bfloat16, or float32");
  int st = check_gemm("int8_gemm_dequant_residual", A, W, M, N, K, 8);
  if (st >= 0) return st;
  if (!rs || !cs || !gate || !x_inout) return fail(B2_NULL_POINTER, "int8_gemm_dequant_residual: null pointer");
  if (bias_kind != B2_BIAS_NONE && !bias) return fail(B2_NULL_POINTER, "int8_gemm_dequant_residual: bias kind %d with a null bias", bias_kind);
  if (!aligned16(x_inout)) return fail(B2_BAD_STRIDE, "int8_gemm_dequant_residual: x must be 16-byte aligned");
  return launch_int8_gemm(A, W, nullptr, nullptr, rs, cs, bias, bias_kind, gate, x_inout, M, N, K, (cudaStream_t)stream);
}

int b2_int8_gemm_dequant_swiglu(const int8_t* A, const float* rs, const int8_t* W, const float* cs,
                                const void* bias, int bias_kind, void* out, int64_t M, int64_t N,
                                int64_t K, void* stream) {
  if (bias_kind < B2_BIAS_NONE || bias_kind > B2_BIAS_FP32) return fail(B2_BAD_DTYPE, "int8_gemm_dequant_swiglu: bias must be none, bfloat16, or float32");
  int st = check_gemm("int8_gemm_dequant_swiglu", A, W, M, N, K, 8);
  if (st >= 0) return st;
  if (N % 128 != 0)
    return fail(B2_NOT_WHITELISTED, "int8_gemm_dequant_swiglu: N=%lld must be a multiple of 128 (gate and up rows interleaved in groups of 64)", (long long)N);
  if (!rs || !cs || !out) return fail(B2_NULL_POINTER, "int8_gemm_dequant_swiglu: null pointer");
  if (bias_kind != B2_BIAS_NONE && !bias) return fail(B2_NULL_POINTER, "int8_gemm_dequant_swiglu: bias kind %d with a null bias", bias_kind);
  if (!aligned16(out)) return fail(B2_BAD_STRIDE, "int8_gemm_dequant_swiglu: out must be 16-byte aligned");
  return launch_int8_gemm(A, W, nullptr, out, rs, cs, bias, bias_kind, nullptr, nullptr, M, N, K, (cudaStream_t)stream, 1);
}

int b2_int8_linear(const void* x, int input_act, const int8_t* W, const float* cs, const void* bias,
                   int bias_kind, void* out, int8_t* q_scratch, float* s_scratch, int64_t M,
                   int64_t N, int64_t K, void* stream) {
  if (input_act != B2_ACT_NONE && input_act != B2_ACT_SWIGLU) return fail(B2_BAD_DTYPE, "int8_linear: unknown input activation %d", input_act);
  if (bias_kind < B2_BIAS_NONE || bias_kind > B2_BIAS_FP32) return fail(B2_BAD_DTYPE, "int8_linear: bias must be none, bfloat16, or float32");
  int st = check_gemm("int8_linear", q_scratch, W, M, N, K, 8);
  if (st >= 0) return st;
  if (!x || !cs || !out || !s_scratch) return fail(B2_NULL_POINTER, "int8_linear: null pointer");
  if (bias_kind != B2_BIAS_NONE && !bias) return fail(B2_NULL_POINTER, "int8_linear: bias kind %d with a null bias", bias_kind);
  if (!aligned16(out) || !aligned16(x)) return fail(B2_BAD_STRIDE, "int8_linear: x/out must be 16-byte aligned");
  st = input_act == B2_ACT_SWIGLU
           ? launch_swiglu_quantize(x, q_scratch, s_scratch, M, K, (cudaStream_t)stream)
           : launch_quantize(x, q_scratch, s_scratch, M, K, (cudaStream_t)stream);
  if (st != B2_OK) return st;
  return launch_int8_gemm(q_scratch, W, nullptr, out, s_scratch, cs, bias, bias_kind, nullptr, nullptr, M, N, K, (cudaStream_t)stream);
}

int b2_flash_fwd(const void* q, const void* k, const void* v, void* out, int32_t B, int32_t H,
                 int32_t S, int64_t qsb, int64_t qsh, int64_t qss, int64_t ksb, int64_t ksh,
                 int64_t kss, int64_t vsb, int64_t vsh, int64_t vss, float scale, void* stream) {
  if (B <= 0 || H <= 0 || S <= 0) return fail(B2_BAD_SHAPE, "flash_fwd: batch, heads, and sequence length must be positive");
  if (!std::isfinite(scale) || !(scale > 0.0f)) return fail(B2_BAD_SHAPE, "flash_fwd: softmax_scale must be finite and positive");
  if (!q || !k || !v || !out) return fail(B2_NULL_POINTER, "flash_fwd: null pointer");
  if (!aligned16(q) || !aligned16(k) || !aligned16(v) || !aligned16(out)) return fail(B2_BAD_STRIDE, "flash_fwd: pointers must be 16-byte aligned");
  const int64_t qs[3] = {qsb, qsh, qss}, ks[3] = {ksb, ksh, kss}, vs[3] = {vsb, vsh, vss};
  const int64_t* all[3] = {qs, ks, vs};
  for (int t = 0; t < 3; ++t) {
    for (int d = 0; d < 3; ++d) {
      const int64_t s = all[t][d];
      if (s < 0) return fail(B2_BAD_STRIDE, "flash_fwd: negative stride");
      if (s % 8 != 0) return fail(B2_BAD_STRIDE, "flash_fwd: strides must be multiples of 8 elements (16 bytes)");
    }
    if (all[t][2] < 128) return fail(B2_BAD_STRIDE, "flash_fwd: row stride below the head dimension");
    // the reference keeps every offset int32-addressable (h3_flash_api.cpp:16-27);
    // TMA needs byte strides below 2^40
    if (all[t][0] >= (1LL << 38) || all[t][1] >= (1LL << 38) || all[t][2] >= (1LL << 38))
      return fail(B2_TOO_LARGE, "flash_fwd: stride too large");
  }
  return launch_flash_fwd(q, k, v, out, B, H, S, qs, ks, vs, scale, (cudaStream_t)stream);
}

}  // extern "C"
