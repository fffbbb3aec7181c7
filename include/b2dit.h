/*
 * b2dit.h - C ABI of libb2dit.so, the sm_100a implementation of the DiT hot path.
 *
 * Plain C: raw device pointers, sizes, element strides, a CUDA stream handle
 * (cudaStream_t passed as void*).  No torch types.  Every entry point
 *   - validates its arguments BEFORE launching anything and returns a b2_status,
 *   - never allocates or frees device memory (the caller owns every buffer),
 *   - enqueues its kernels on `stream` and returns without synchronising.
 * On a non-zero status b2_last_error() holds a thread-local message.
 *
 * Each declaration cites the reference interface it replaces (path within the
 * reference project : line).
 */
#ifndef B2DIT_H_
#define B2DIT_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define B2_ABI_VERSION 1

typedef enum b2_status {
  B2_OK = 0,
  B2_BAD_DTYPE = 1,        /* bias_kind / activation code out of range            */
  B2_BAD_SHAPE = 2,        /* negative, zero where forbidden, or inconsistent size */
  B2_BAD_STRIDE = 3,       /* misaligned pointer or stride                         */
  B2_NOT_WHITELISTED = 4,  /* shape outside what the kernel family supports        */
  B2_LAUNCH_FAILED = 5,    /* cudaGetLastError() after the launch was non-zero     */
  B2_TIMEOUT = 6,          /* a bounded device-side wait gave up                   */
  B2_NULL_POINTER = 7,
  B2_TOO_LARGE = 8         /* size beyond a documented static limit                */
} b2_status;

/* bias_kind: kernels/int8-epilogue/epilogue_kernel.hip:13-17 (enum BiasKind) */
#define B2_BIAS_NONE 0
#define B2_BIAS_BF16 1
#define B2_BIAS_FP32 2

/* input activation applied before quantisation,
 * launcher/benchmark_launcher_v14_hires_int8_candidate.py:976 (`input_act`) */
#define B2_ACT_NONE 0
#define B2_ACT_SWIGLU 1

int b2_version(void);
const char* b2_last_error(void);
const char* b2_status_string(int status);

/* Reads the device-side error word (set by bounded waits that gave up) and
 * clears it.  Synchronises `stream`.  Returns B2_OK or B2_TIMEOUT. */
int b2_check_device_status(void* stream);

/* Failure-detection self-test: launches one CTA whose only wait can never be satisfied
 * and has a tiny poll budget.  The kernel gives up, records a status word and returns;
 * the next b2_check_device_status() reports B2_TIMEOUT and clears it.  Nothing traps,
 * faults or hangs.  (No counterpart in the reference, which has no device-side waits.) */
int b2_selftest_bounded_wait(void* stream);

/* Rowwise bf16 -> int8 quantizer.
 * Replaces h3_quantize_int8_rowwise_hip, kernels/exact-rowwise-int8/quantizer_kernel.hip:118-144
 * (Python: quantize_int8_rowwise(x) -> [q, scale], kernels/exact-rowwise-int8/quantizer.cpp:5-9).
 * x bf16 [M,K] contiguous; q int8 [M,K]; scale fp32 [M] (the reference's [M,1]).
 * M == 0 or K == 0 is legal: with M != 0 and K == 0 the scales are filled with 1e-30. */
int b2_quantize_int8_rowwise(const void* x, int8_t* q, float* scale, int64_t M, int64_t K,
                             void* stream);

/* INT8 dequant epilogue, scalar contract with optional bias.
 * Replaces h3_epilogue_hip, kernels/int8-epilogue/epilogue_kernel.hip:65-133
 * (Python: epilogue(acc,row_scale,col_scale,bias), kernels/int8-epilogue/epilogue.cpp:9-13).
 * The reference's M <= 65535 launch limit (:85-86) does not exist here. */
int b2_epilogue(const int32_t* acc, const float* row_scale, const float* col_scale,
                const void* bias, int bias_kind, void* out_bf16, int64_t M, int64_t N,
                void* stream);

/* INT8 dequant epilogue, bias-less 4-wide contract.
 * Replaces h3_epilogue_vec4_hip, kernels/int8-epilogue-vec4/epilogue_kernel.hip:33-48
 * (Python: epilogue(acc,row,col), kernels/int8-epilogue-vec4/epilogue.cpp:3-5). */
int b2_epilogue_vec4(const int32_t* acc, const float* row_scale, const float* col_scale,
                     void* out_bf16, int64_t M, int64_t N, void* stream);

/* In-place x = bf16(bf16(x*bf16(1+scale[c])) + shift[c]).
 * Replaces h3_mod_scale_shift_hip, kernels/mod-scale-shift/mod_kernel.hip:24-38
 * (Python: mod_scale_shift_(x,scale,shift), kernels/mod-scale-shift/mod.cpp:3-5). */
int b2_mod_scale_shift(void* x_bf16, const void* scale_bf16, const void* shift_bf16, int64_t M,
                       int64_t C, void* stream);

/* Fused SwiGLU + rowwise quantizer: x bf16 [M,2K] -> q int8 [M,K], scale fp32 [M].
 * Replaces h3_swiglu_quantize_int8_rowwise_hip, kernels/swiglu-quant/swiglu_quant_kernel.hip:111-137
 * (Python: swiglu_quantize_int8_rowwise(x), kernels/swiglu-quant/swiglu_quant.cpp:5-9).
 * bf16(silu(gate)) comes from a 65536-entry table held in a fixed array inside the library
 * (128 KB per GPU, no allocation).  The FIRST call on each device fills it with the exact
 * formula and waits for that kernel on `stream`; make that call before any stream capture.
 * The same holds for b2_int8_linear with B2_ACT_SWIGLU and for b2_int8_linear_noalloc. */
int b2_swiglu_quantize_int8_rowwise(const void* x, int8_t* q, float* scale, int64_t M, int64_t K,
                                    void* stream);

/* acc[M,N] (int32) = A[M,K] . W[N,K]^T, both int8 row-major (K contiguous).
 * Replaces the library GEMM call torch._int_mm(x_8, weight.T),
 * launcher/benchmark_launcher_v14_hires_int8_candidate.py:805-824.
 * Requires K % 16 == 0 and N % 4 == 0 (TMA 16-byte rules); any M >= 1. */
int b2_int8_gemm(const int8_t* A, const int8_t* W, int32_t* acc, int64_t M, int64_t N, int64_t K,
                 void* stream);

/* GEMM with the dequant epilogue fused: out bf16 [M,N] =
 *   bf16( bf16(float(acc)*(rs[m]*cs[n])) + bf16(bias[n]) ).
 * Replaces steps 5+6 of _int8_linear_nocopy,
 * launcher/benchmark_launcher_v14_hires_int8_candidate.py:1007-1052.
 * Requires K % 16 == 0 and N % 8 == 0. */
int b2_int8_gemm_dequant(const int8_t* A, const float* row_scale, const int8_t* W,
                         const float* col_scale, const void* bias, int bias_kind, void* out_bf16,
                         int64_t M, int64_t N, int64_t K, void* stream);

/* The same GEMM with the DiT block's gated residual applied in the epilogue:
 *   y = the dequantised, biased bf16 value above;  x[m,n] = bf16( x[m,n] + bf16(gate[n]*y) ).
 * x bf16 [M,N] is updated in place, gate bf16 [N]; y never goes through memory.  Bit-identical
 * to b2_int8_gemm_dequant followed by b2_gate_residual.  (Fusion of two steps of
 * _int8_linear_nocopy's caller; the reference has no source for the residual itself.) */
int b2_int8_gemm_dequant_residual(const int8_t* A, const float* row_scale, const int8_t* W,
                                  const float* col_scale, const void* bias, int bias_kind,
                                  const void* gate_bf16, void* x_inout_bf16, int64_t M, int64_t N,
                                  int64_t K, void* stream);

/* The same GEMM with the first half of swiglu-quant applied in the epilogue (for the FFN's
 * first projection).  W int8 [N,K], col_scale fp32 [N] and bias [N] hold the projection's gate
 * rows and up rows INTERLEAVED in groups of 64: rows [128k, 128k+64) are gate rows
 * [64k, 64k+64) and rows [128k+64, 128k+128) the matching up rows (N = 2F, N % 128 == 0).
 *   out bf16 [M, N/2]:  out[m, 64k+j] = bf16( bf16(silu(y_gate)) * y_up ),
 * y the dequantised, biased bf16 values above, silu(g) = g / (1 + expf(-g)) in fp32: exactly
 * what kernels/swiglu-quant/swiglu_quant_kernel.hip:18-27 computes from the [M,2F] projection
 * before it quantises, so b2_quantize_int8_rowwise(out) gives the bits of
 * b2_swiglu_quantize_int8_rowwise(b2_int8_gemm_dequant(...)) with the un-interleaved weight,
 * and the [M,2F] tensor never goes through memory.  bf16(silu(g)) comes from the same
 * 65536-entry table as b2_swiglu_quantize_int8_rowwise (built from that formula on the first
 * call on a device, which waits for it: make that call before any stream capture).  (A
 * fusion; the reference runs the projection and swiglu-quant as two operators.) */
int b2_int8_gemm_dequant_swiglu(const int8_t* A, const float* row_scale, const int8_t* W_interleaved,
                                const float* col_scale_interleaved, const void* bias_interleaved,
                                int bias_kind, void* out_bf16, int64_t M, int64_t N, int64_t K,
                                void* stream);

/* Whole INT8 linear: (activation) -> rowwise quantise -> GEMM -> dequant epilogue.
 * Replaces _int8_linear_nocopy, launcher/benchmark_launcher_v14_hires_int8_candidate.py:960-1067
 * (bf16 output, per-output-channel weight scale, no ConvRot).
 * x bf16 [M,K] (act none) or [M,2K] (act swiglu); W int8 [N,K]; col_scale fp32 [N].
 * q_scratch int8 [M,K] and s_scratch fp32 [M] are caller-provided scratch. */
int b2_int8_linear(const void* x_bf16, int input_act, const int8_t* W, const float* col_scale,
                   const void* bias, int bias_kind, void* out_bf16, int8_t* q_scratch,
                   float* s_scratch, int64_t M, int64_t N, int64_t K, void* stream);

/* The same linear for callers that cannot supply scratch memory: hosts whose own pool
 * already owns all device memory, plugins that only receive their input and output
 * buffers, serving loops that must not allocate once running.  The quantised activation and
 * its scales live in a fixed array inside the library (32 MiB + 256 KiB, held by every GPU
 * that loads the library until the process exits).  Limits: M <= 65536 and M*K <= 32 MiB,
 * otherwise B2_TOO_LARGE.  All calls on a GPU share that array and it keeps the previous
 * call's contents (nothing in it needs to start at zero): calls that can overlap on the GPU
 * race, so serialise them.  The first call on each device resolves the array's address;
 * make it during start-up, before any stream capture.  The array that is used belongs to
 * the CURRENT device (cudaGetDevice) at the time of the call: make the device that owns x,
 * W and out current first, as for every other entry point.  Allocates nothing.
 * This entry point has no counterpart in the reference project. */
int b2_int8_linear_noalloc(const void* x_bf16, int input_act, const int8_t* W,
                           const float* col_scale, const void* bias, int bias_kind, void* out_bf16,
                           int64_t M, int64_t N, int64_t K, void* stream);

/* bf16 FlashAttention forward, non-causal, head_dim 128.
 * Replaces h3_flash_fwd_bhsd, kernels/flash-attention-gfx936/csrc/flash_attn_hipc/h3_flash_api.cpp:30-130
 * (Python: fwd_bhsd(q,k,v,softmax_scale), :133-142).
 * q,k,v: logical [B,H,S,128] bf16 with element strides (batch, head, row) and a
 * contiguous last dimension; strides must be multiples of 8 elements and pointers
 * 16-byte aligned.  out: contiguous [B,S,H,128] bf16 (the reference's BSHD backing
 * storage, :65-69).  softmax_scale finite and > 0. */
int b2_flash_fwd(const void* q, const void* k, const void* v, void* out, int32_t B, int32_t H,
                 int32_t S, int64_t q_stride_b, int64_t q_stride_h, int64_t q_stride_s,
                 int64_t k_stride_b, int64_t k_stride_h, int64_t k_stride_s, int64_t v_stride_b,
                 int64_t v_stride_h, int64_t v_stride_s, float softmax_scale, void* stream);

/* ---- DiT-block glue.  The reference has no source for these (they live in the
 * host application's model file); conventions are this library's own. ---------- */

/* out = bf16(LayerNorm_noaffine_fp32(x)) then mod-scale-shift's three roundings;
 * x bf16 [M,C], out bf16 [M,C] (may alias x). */
int b2_layernorm_mod(const void* x_bf16, const void* scale_bf16, const void* shift_bf16,
                     void* out_bf16, int64_t M, int64_t C, float eps, void* stream);

/* Same, followed by the rowwise quantizer: writes q int8 [M,C] and scale fp32 [M]. */
int b2_layernorm_mod_quant(const void* x_bf16, const void* scale_bf16, const void* shift_bf16,
                           int8_t* q, float* scale_out, int64_t M, int64_t C, float eps,
                           void* stream);

/* Per-head RMSNorm (weight bf16 [128]) + rotary on adjacent pairs, in place on the
 * q and k parts of a packed qkv bf16 [S, 3, H, 128] buffer.  cos/sin fp32 [S,64]. */
int b2_qk_norm_rope(void* qkv_bf16, const void* q_weight_bf16, const void* k_weight_bf16,
                    const float* cos_tab, const float* sin_tab, int64_t S, int32_t H, float eps,
                    void* stream);

/* The two ends of the sequence-parallel (Ulysses) exchange without their pack / unpack
 * copies (the reference measures both as ceilings: communication/bench_fused_qkv_alltoall.py,
 * communication/bench_reverse_unpack_ceiling.py; its packed layout is
 * benchmarks/bench_sp_head_chunk_overlap.py:140-164).
 *
 * b2_qk_norm_rope_pack: b2_qk_norm_rope, but reading qkv bf16 [L,3,H,128] and writing the
 * all-to-all send buffer bf16 [chunks][world][L][c][3][128], c = H/(world*chunks), head
 * h = (p*chunks + ch)*c + ci; V is copied unchanged.  Slice [ch] is one all-to-all.
 *
 * b2_quantize_int8_rowwise_gathered: b2_quantize_int8_rowwise whose input row m is spread
 * over the reverse all-to-all's receive buffer bf16 [chunks][world][M][K/(world*chunks)]
 * (segment (p, ch) holds columns ((p*chunks + ch) * K/(world*chunks)) onward); q int8 [M,K]
 * and scale fp32 [M] come out exactly as if the row had been contiguous. */
int b2_qk_norm_rope_pack(const void* qkv_bf16, void* send_bf16, const void* q_weight_bf16,
                         const void* k_weight_bf16, const float* cos_tab, const float* sin_tab,
                         int64_t L, int32_t H, int32_t world, int32_t chunks, float eps,
                         void* stream);
int b2_quantize_int8_rowwise_gathered(const void* x_bf16, int8_t* q, float* scale, int64_t M,
                                      int64_t K, int32_t world, int32_t chunks, void* stream);

/* The same exchange carried by the kernels themselves over peer memory, for ranks of one
 * NVSwitch domain (at most 8).  These entry points have no counterpart in the reference, whose
 * sequence-parallel model moves the layouts above with torch.distributed all-to-all calls
 * (benchmarks/bench_sp_head_chunk_overlap.py:140-193); the bytes that arrive are the same.
 *
 * b2_peer_alloc / b2_peer_free: a zero-filled device buffer of the CURRENT device that other
 * processes may map (plain cudaMalloc, outside any caching allocator).  b2_peer_export fills
 * a 64-byte handle for it; b2_peer_open maps a handle exported by another process of the
 * same machine (peer access is enabled on first use) and b2_peer_close unmaps it.  Set-up
 * and tear-down only: these are the only entry points of the library that allocate, map or
 * free device memory, and they synchronise the device.
 *
 * b2_qk_norm_rope_scatter: b2_qk_norm_rope_pack writing every vector straight into the
 * receive buffer of the rank that owns its head: recv_bases is a HOST array of `world`
 * device pointers, entry p being rank p's buffer bf16 [chunks][S][c][3][128] as mapped in this
 * process (the caller's own buffer at its own index); this rank's row l lands at row row0 + l.
 * Plain 16-byte stores; nothing waits.  The caller orders the ranks: every rank's scatter
 * must have completed before any rank reads its buffer, and all reads before the next scatter
 * (e.g. a collective on the same stream in between).
 *
 * b2_copy_segments: n <= 8 contiguous copies (16-byte aligned, sizes multiples of 16) in one
 * launch; sources and destinations may be local or peer-mapped.  Used for the reverse
 * direction: rows [row0_p, row0_p + L_p) of the attention output go to slot [ch][me] of rank
 * p's buffer bf16 [chunks][world][L_p][c][128], which b2_quantize_int8_rowwise_gathered reads. */
int b2_peer_alloc(int64_t bytes, void** ptr);
int b2_peer_free(void* ptr);
int b2_peer_export(void* ptr, void* handle, int32_t handle_bytes);
int b2_peer_open(const void* handle, int32_t handle_bytes, void** ptr);
int b2_peer_close(void* ptr);
int b2_qk_norm_rope_scatter(const void* qkv_bf16, void* const* recv_bases, const void* q_weight_bf16,
                            const void* k_weight_bf16, const float* cos_tab, const float* sin_tab,
                            int64_t L, int32_t H, int32_t world, int32_t chunks, int64_t row0,
                            int64_t S, float eps, void* stream);
int b2_copy_segments(const void* const* src, void* const* dst, const int64_t* bytes, int32_t n,
                     void* stream);

/* Decoded frames -> RGB24 bytes for the video encoder, the whole clip in one launch:
 * out[i] = uint8(clamp(images[i] * 255, 0, 255)), product rounded to the input type, cast
 * truncating, NaN -> 0.  Replaces the per-frame `(image * 255).clamp(0, 255).byte()` + copy
 * that the reference batches in launcher/benchmark_launcher_v14_hires_int8_candidate.py:607-723
 * (H3_SAVE_BATCH_U8).  dtype: 0 float32, 1 bfloat16, 2 float16; n = element count. */
int b2_images_to_u8(const void* images, int32_t dtype, uint8_t* out, int64_t n, void* stream);

/* x = bf16(x + bf16(gate[c]*y)) in place on x; x,y bf16 [M,C], gate bf16 [C]. */
int b2_gate_residual(void* x_bf16, const void* y_bf16, const void* gate_bf16, int64_t M, int64_t C,
                     void* stream);

#ifdef __cplusplus
}
#endif
#endif /* B2DIT_H_ */
