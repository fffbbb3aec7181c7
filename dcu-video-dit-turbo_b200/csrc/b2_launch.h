// Internal launch functions behind the C ABI (one per kernel family).  Each
// assumes validated arguments, enqueues on `stream` and returns a b2_status.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace b2 {

int launch_quantize(const void* x, int8_t* q, float* scale, int64_t M, int64_t K,
                    cudaStream_t stream);
// world > 0: source rows gathered from [chunks][world][M][K / (world*chunks)]
int launch_quantize_gathered(const void* x, int8_t* q, float* scale, int64_t M, int64_t K, int world,
                             int chunks, cudaStream_t stream);
int launch_swiglu_quantize(const void* x, int8_t* q, float* scale, int64_t M, int64_t K,
                           cudaStream_t stream);
int launch_fill_f32(float* p, int64_t n, float v, cudaStream_t stream);
// bf16(silu(g)) for all 65536 bf16 gates, in global memory of the current device (built on first use)
int silu_table_device_pointer(cudaStream_t stream, const uint16_t** table);
int launch_epilogue(const int32_t* acc, const float* rs, const float* cs, const void* bias,
                    int bias_kind, void* out, int64_t M, int64_t N, cudaStream_t stream);
int launch_mod_scale_shift(void* x, const void* scale, const void* shift, int64_t M, int64_t C,
                           cudaStream_t stream);
int launch_images_to_u8(const void* x, int dtype, uint8_t* out, int64_t n, cudaStream_t stream);
int launch_gate_residual(void* x, const void* y, const void* gate, int64_t M, int64_t C,
                         cudaStream_t stream);
int launch_layernorm_mod(const void* x, const void* scale, const void* shift, void* out_bf16,
                         int8_t* out_q, float* out_scale, int64_t M, int64_t C, float eps,
                         bool quant, cudaStream_t stream);
int launch_qk_norm_rope(void* qkv, const void* qw, const void* kw, const float* cos_tab,
                        const float* sin_tab, int64_t S, int H, float eps, cudaStream_t stream);
int launch_qk_norm_rope_pack(const void* qkv, void* send, const void* qw, const void* kw,
                             const float* cos_tab, const float* sin_tab, int64_t L, int H, int world,
                             int chunks, float eps, cudaStream_t stream);
// recv_bases: host array of `world` device pointers (each rank's receive buffer as mapped here)
int launch_qk_norm_rope_scatter(const void* qkv, void* const* recv_bases, const void* qw, const void* kw,
                                const float* cos_tab, const float* sin_tab, int64_t L, int H, int world,
                                int chunks, int64_t row0, int64_t S, float eps, cudaStream_t stream);
int launch_copy_segments(const void* const* src, void* const* dst, const int64_t* bytes, int n,
                         cudaStream_t stream);
// out_i32 != nullptr: plain int32 result.  Otherwise the fused dequant epilogue writes
// bf16 to out_bf16, or, with gate/residual non-null, x = bf16(x + bf16(gate*y)) in place, or,
// with swiglu != 0 (W, cs, bias interleaved gate/up in groups of 64 rows), the SwiGLU product
// bf16 [M, N/2] to out_bf16.
int launch_int8_gemm(const int8_t* A, const int8_t* W, int32_t* out_i32, void* out_bf16,
                     const float* rs, const float* cs, const void* bias, int bias_kind,
                     const void* gate, void* residual, int64_t M, int64_t N, int64_t K,
                     cudaStream_t stream, int swiglu = 0);
// CTA-pair (cta_group::2) variant; returns -1 when it does not apply.
int launch_int8_gemm_pair(const int8_t* A, const int8_t* W, int32_t* out_i32, void* out_bf16,
                          const float* rs, const float* cs, const void* bias, int bias_kind,
                          const void* gate, void* residual, int64_t M, int64_t N, int64_t K,
                          cudaStream_t stream, int swiglu = 0);
int launch_flash_fwd(const void* q, const void* k, const void* v, void* out, int B, int H, int S,
                     const int64_t* qs, const int64_t* ks, const int64_t* vs, float scale,
                     cudaStream_t stream);

// CTA-pair (cta_group::2) variant; returns -1 when it does not apply.
int launch_flash_fwd_pair(const void* q, const void* k, const void* v, void* out, int B, int H, int S,
                          const int64_t* qs, const int64_t* ks, const int64_t* vs, float scale,
                          cudaStream_t stream);

int launch_bounded_wait_selftest(cudaStream_t stream);
// Read and clear the device-side status word of a tensor-core translation unit.
unsigned int read_clear_status_gemm();
unsigned int read_clear_status_gemm2();
unsigned int read_clear_status_flash();
unsigned int read_clear_status_flash2();

}  // namespace b2
