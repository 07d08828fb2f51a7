/*
 * feather_b200.h - C ABI of libfeather_b200.so (sm_100a).
 *
 * The library is the native side of the FeatherOps mixed-precision linear:
 *     C[M,N] = cvt( (A[M,K] fp16 . up(W[K,N] fp8e5m2)) * scale ) + bias        fp32 accumulate
 * with W stored prepacked as (K/16, N, 16) bytes, plus the quantise-and-prepack that produces W.
 *
 * Conventions shared by every entry point
 *   - plain pointers and sizes only; every pointer is a DEVICE pointer unless its name ends in _host
 *   - pointers are borrowed: the caller keeps the memory alive until the stream work has finished
 *   - work is enqueued on `stream`; nothing here synchronises the device
 *   - no entry point allocates device memory (scratch is passed in by the caller); none throws
 *   - the return value is a feather_status (0 = ok).  Device-side failures (a bounded wait inside a
 *     kernel that ran out) are written to the optional `status_dev` word and are visible to the host
 *     after the stream has been synchronised.
 *
 * Each declaration cites the interface of the reference (woct0rdho/ComfyUI-FeatherOps) it stands in
 * for, as path:line inside that project.
 */
#ifndef FEATHER_B200_H_
#define FEATHER_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(__GNUC__)
#define FEATHER_API __attribute__((visibility("default")))
#else
#define FEATHER_API
#endif

/* CUDA stream handle (cudaStream_t) passed as an opaque pointer so this header needs no CUDA include. */
typedef void* feather_stream_t;

typedef enum feather_status {
    FEATHER_OK = 0,
    FEATHER_ERR_BAD_ARGUMENT = 1,    /* null pointer, negative size, K % 16 != 0, misaligned pointer ... */
    FEATHER_ERR_UNSUPPORTED = 2,     /* e.g. unknown kernel variant, streaming kernel asked for more than 32 tokens */
    FEATHER_ERR_WORKSPACE = 3,       /* variant needs more scratch than was passed */
    FEATHER_ERR_CUDA = 4,            /* a CUDA runtime / driver call failed; see feather_last_error_string */
    FEATHER_ERR_DEVICE_TIMEOUT = 5,  /* value found in *status_dev after a kernel gave up on a bounded wait */
    FEATHER_ERR_NO_DEVICE = 6        /* no sm_100 device / driver entry point unavailable */
} feather_status;

/* Weight / output dtype codes, same numbering as kernel/hip/hip_kernel.cu:579-580 */
enum { FEATHER_B_E4M3 = 0, FEATHER_B_E5M2 = 1 };
enum { FEATHER_OUT_FP16 = 0, FEATHER_OUT_BF16 = 1 };
/* Source dtype codes of the quantiser */
enum { FEATHER_SRC_FP32 = 0, FEATHER_SRC_BF16 = 1, FEATHER_SRC_FP16 = 2 };

/* Kernel variant selection for feather_scaled_mm_ex.  All fields 0 = let the library choose.
 *   tokens_tile : activation rows per MMA tile (the MMA N extent): 16, 32, 64, 128, 192 or 256
 *   cta_pair    : 1 = one CTA per tile (128 weight columns), 2 = two-CTA pairs (256 weight columns)
 *   split_k     : number of K slices reduced through the fp32 workspace (1 = none)
 *   transform_groups : groups of four warps that upcast e5m2 weight stages (1 or 2)
 *   max_ctas    : cap on the persistent grid (0 = number of SMs)
 *   kernel      : 0 = choose from the shape (streaming up to 16 tokens, up to 24 for weights of at most 32 MB); 1 = the tensor-memory (tcgen05) kernel; 2 = the
 *                 register-streaming kernel, at most 32 tokens (needs no workspace, ignores the other fields)
 *   staging     : output staging of 256-token pair tiles: 0 = choose (two buffers per epilogue group when blocks also go to
 *                 peer GPUs, one otherwise), 1 = one buffer, 2 = two buffers
 */
enum { FEATHER_KERNEL_AUTO = 0, FEATHER_KERNEL_TMEM = 1, FEATHER_KERNEL_STREAM = 2 };
typedef struct feather_mm_variant {
    int tokens_tile;
    int cta_pair;
    int split_k;
    int transform_groups;
    int max_ctas;
    int kernel;
    int staging;
} feather_mm_variant;

/* ---------------------------------------------------------------------------------------------
 * GEMM
 * ------------------------------------------------------------------------------------------- */

/* Drop-in for `extern "C" bool launch_scaled_mm(...)`, kernel/hip/hip_kernel.cu:564-582: same argument
 * order and meaning, cudaStream_t in place of hipStream_t.  The five tile integers are accepted and
 * ignored (the variant is chosen from the shape); b_dtype is 1 (e5m2) or 0 (e4m3fn, upcast exactly).  Returns 1 when the launch
 * was enqueued, 0 otherwise (the reference returns false for an unknown config).  This entry point
 * takes no workspace, so it never splits K through one: where the shape calls for it (up to 16 tokens, up to 24 for small
 * weights) it runs the register-streaming kernel (which splits K inside a CTA), else the tensor-memory kernel unsplit. */
FEATHER_API int launch_scaled_mm(const void* a, const uint8_t* b_prepacked, const float* scale, const uint16_t* bias, uint16_t* c,
                     int64_t M, int64_t N, int64_t K, int has_scale, int has_bias, int block_warps_m, int block_warps_n,
                     int unroll_k, int repeat_m, int repeat_n, int b_dtype, int output_dtype, feather_stream_t stream);

/* Full form used by the Python operator (kernel/hip/hip_kernel.py:12-39 `_configured_op` ->
 * `torch.ops.feather_ops.scaled_mm`, kernel/hip/hip_kernel.cu:635-744).
 *   a            fp16 [M,K] row-major, 16-byte aligned
 *   b_prepacked  e5m2 bytes [K/16, N, 16], 16-byte aligned
 *   scale        fp32[1] or NULL; bias  out-dtype [N] or NULL
 *   c            out-dtype [M, ldc] row-major; only columns [0,N) of each row are written.  ldc >= N
 *                lets a column shard write straight into its slice of a wider output.
 *   workspace    scratch for split-K variants (may be NULL), 16-byte aligned.  It must be zero-filled
 *                once after allocation (tile counters live in its first 64 KiB); every launch that completes
 *                leaves the counters at zero again, so the same buffer serves any later call.
 *                Two launches that may overlap on the device need separate workspaces.
 *   status_dev   int32 device word or NULL; left untouched on success
 */
FEATHER_API int feather_scaled_mm_ex(const void* a, const uint8_t* b_prepacked, const float* scale, const void* bias, void* c, int64_t M,
                         int64_t N, int64_t K, int64_t ldc, int output_dtype, const feather_mm_variant* variant,
                         void* workspace, size_t workspace_bytes, int* status_dev, feather_stream_t stream);

/* The GEMM with the operand and result types the hot path meets around the reference's fp16 x e5m2 -> out-dtype core:
 *   a_dtype      FEATHER_SRC_FP16 or FEATHER_SRC_BF16.  bf16 activations are multiplied as they are (the weights are upcast to
 *                bf16, which holds every fp8 value exactly), so the caller's `x.to(fp16)` pass (comfy_feather/ops.py:88,
 *                kernel/convert.py:24-34) disappears.  For every activation that fp16 represents exactly the result is bitwise
 *                what cast-first gives; outside that range (|x| > 65504, or below 2^-14 with more bits than fp16 subnormals
 *                keep) this path multiplies the unrounded value where cast-first would multiply inf or a rounded one.
 *   b_dtype      FEATHER_B_E5M2 or FEATHER_B_E4M3 (fp8e4m3fn bytes in the same (K/16, N, 16) layout; exact upcast including
 *                subnormals and the NaN codes - kernel/hip/hip_kernel.cu:83-99 of the reference approximates it).
 *   output_dtype dtype the scaled sum is rounded to and the bias is added in (bias has this dtype), as in feather_scaled_mm_ex
 *   final_dtype  dtype of c: -1 or output_dtype stores that value; the other 16-bit dtype applies one more rounding first,
 *                which is the caller's `y.to(dtype_orig)` (comfy_feather/ops.py:103) done in the epilogue.
 * Everything else as feather_scaled_mm_ex.  A handful of tokens of fp16 activations with e5m2 weights take the streaming kernel as
 * there; bf16 activations and e4m3 weights always take the tensor-memory kernel. */
FEATHER_API int feather_scaled_mm_typed(const void* a, int a_dtype, const uint8_t* b_prepacked, int b_dtype, const float* scale, const void* bias,
                                        void* c, int64_t M, int64_t N, int64_t K, int64_t ldc, int output_dtype, int final_dtype,
                                        const feather_mm_variant* variant, void* workspace, size_t workspace_bytes, int* status_dev,
                                        feather_stream_t stream);

/* The linear with an un-merged (low-VRAM) LoRA term folded into the GEMM's accumulator instead of added to the output afterwards
 * (comfy_feather/lora.py:4-35 of the reference computes y += ((x A^T) B^T) * strength with two GEMMs and a read-modify-write of
 * the whole [M, N] output per patch):
 *     c = cast( cvt( (a . up(W) + t . lb^T) * scale ) + bias )
 * after the weight's k-blocks every tile runs rank/64 more blocks whose operands are already 16-bit:
 *   t             [M, rank]  row-major, fp16 (also with bf16 activations: the low-rank blocks run as fp16 x fp16 MMAs into the same
 *                 accumulator): the down-projection x A^T of all patches side by side, times a power of two alpha
 *   lb_prepacked  [rank/8, N, 8] fp16: lb[j][n][i] = B'[n][8j + i] with B' = B * strength / (scale * alpha), so that
 *                 (t . lb^T) * scale is the LoRA term (alpha only moves both factors into fp16's range)
 *   rank          total rank of all patches, padded with zero columns to a multiple of 64
 * Everything else as feather_scaled_mm_typed with e5m2 weights; the variant must not split K.  The tensor-memory kernel is used
 * for any M.  The result differs from the reference's sequence by its roundings only (one rounding of the sum instead of one per
 * patch). */
FEATHER_API int feather_scaled_mm_lora(const void* a, int a_dtype, const uint8_t* b_prepacked, const float* scale, const void* bias, void* c,
                                       int64_t M, int64_t N, int64_t K, int64_t ldc, int output_dtype, int final_dtype, const void* t,
                                       const void* lb_prepacked, int64_t rank, const feather_mm_variant* variant, int* status_dev,
                                       feather_stream_t stream);

/* Column-sharded linear over the GPUs of one box, exchange fused into the GEMM: the same launch as feather_scaled_mm_ex,
 * but every finished output block is stored (TMA store) to each of the n_dst buffers in c_list_host - a HOST array of device
 * pointers: entry 0 the caller's own [M, ldc] buffer (already offset to this rank's first column), the others the same position
 * in the peer GPUs' buffers (peer-mapped addresses, e.g. from torch symmetric memory), reached over NVLink.  No load touches
 * peer memory.  Needs 16-byte aligned rows (ldc % 8 == 0, aligned pointers); K is never split, so all ranks produce bitwise
 * the single-GPU result.  The caller synchronises the ranks (a barrier after the launch) before anyone reads the outputs.
 * The reference has no multi-GPU path; this entry point has no counterpart in the reference. */
FEATHER_API int feather_scaled_mm_multi(const void* a, const uint8_t* b_prepacked, const float* scale, const void* bias,
                                        void* const* c_list_host, int n_dst, int64_t M, int64_t N, int64_t K, int64_t ldc, int output_dtype,
                                        const feather_mm_variant* variant, int* status_dev, feather_stream_t stream);

/* Row-parallel half of a tensor-parallel pair of linears (K sharded across the GPUs of one box, so every rank holds a
 * partial sum of the whole [M, N] output): the same launch as feather_scaled_mm_multi, but the destinations are sharded by
 * token rows.  c_list_host[d] (a HOST array of n_dst device pointers, peer-mapped for d != own rank) receives this rank's
 * partial of rows [d * rows_per_dst, (d + 1) * rows_per_dst) as a [rows_per_dst, ldc] row-major block, rounded to the output
 * dtype; each finished block is TMA-stored to the one buffer that owns its rows while the tensor cores run the next tile.
 * Every rank passes, for destination d, ITS OWN slot of rank d's buffer, so the owner ends up with one partial per rank and
 * sums them with feather_reduce_partials.  rows_per_dst must be a multiple of 32; only stores cross NVLink.  Pass
 * bias = NULL here and give the bias to feather_reduce_partials (it must be added once, not once per rank).
 * The reference has no multi-GPU path; this entry point has no counterpart in the reference. */
FEATHER_API int feather_scaled_mm_scatter(const void* a, const uint8_t* b_prepacked, const float* scale, const void* bias,
                                          void* const* c_list_host, int n_dst, int64_t rows_per_dst, int64_t M, int64_t N, int64_t K,
                                          int64_t ldc, int output_dtype, const feather_mm_variant* variant, int* status_dev,
                                          feather_stream_t stream);

/* Second step of the row-parallel linear: out[r][n] = cvt(sum_s fp32(partials[s][r][n])) + bias[n] (+ residual[r][n]), the sum
 * taken in slot order s = 0 .. n_src-1 in fp32 (deterministic), one rounding to the 16-bit dtype, the bias added in that dtype
 * as in the GEMM epilogue (kernel/naive.py:34-40 of the reference), then the optional residual (same dtype, [rows, ld_res]).
 *   partials      [n_src][rows][N] contiguous, 16-bit dtype per `dtype` (FEATHER_OUT_*), on this GPU
 *   dst_list_host HOST array of n_dst device pointers; the result rows are written to each (own buffer and peer-mapped
 *                 buffers of the other ranks, plain 16-byte stores over NVLink), row pitch ld_dst elements.  This is the
 *                 all-gather of the reduced rows: pass every rank's full output offset to this rank's first row.
 * N must be a multiple of 8 and all pointers 16-byte aligned.  No counterpart in the reference. */
FEATHER_API int feather_reduce_partials(const void* partials, int n_src, int64_t rows, int64_t N, const void* bias, const void* residual,
                                        int64_t ld_res, void* const* dst_list_host, int n_dst, int64_t ld_dst, int dtype,
                                        feather_stream_t stream);

/* Strided block copy by a copy engine (no SM time): `rows` rows of `width_bytes` bytes from src (row pitch src_pitch_bytes) to
 * dst (row pitch dst_pitch_bytes), device to device, asynchronous on `stream`.  dst may be peer-mapped memory of another GPU
 * of the box: this is how a column-sharded linear hands its finished [M, N/g] block to the other ranks' [M, N] outputs on a
 * second stream while the next linear's GEMM has the SMs (feather_scaled_mm_multi instead overlaps the transfer with the
 * same linear's tiles).  The copy is a store as seen from this GPU: nothing is loaded from peer memory.  The reference has no
 * multi-GPU path; this entry point has no counterpart in the reference. */
FEATHER_API int feather_copy_block(void* dst, int64_t dst_pitch_bytes, const void* src, int64_t src_pitch_bytes, int64_t width_bytes,
                                   int64_t rows, feather_stream_t stream);

/* Scratch bytes the variant chosen for (M,N,K) needs (0 when it does not split K; for the streaming kernel an upper bound of
 * what a K split across CTAs may use - with less, or none, it splits less, or not at all).  Pass the same
 * `variant` (or NULL) as to feather_scaled_mm_ex.  The reference's shipped kernel never splits K (README.md:31
 * names an unshipped split-k branch), so its launcher has no scratch argument (kernel/hip/hip_kernel.cu:564-582). */
FEATHER_API size_t feather_scaled_mm_workspace_bytes(int64_t M, int64_t N, int64_t K, const feather_mm_variant* variant);

/* For callers that cannot allocate device memory themselves - code running inside a CUDA-graph capture or a host
 * callback, plugins that are handed pointers by an allocator they do not own, or C programs that want to link the
 * library and call one function without managing a workspace.  Same arguments and results as feather_scaled_mm_ex called
 * with a workspace of feather_scaled_mm_static_scratch_bytes() bytes (8 MiB), minus the workspace argument: the split-K
 * scratch is a fixed array of that size inside the library's device image, so every GPU that loads the library holds
 * those bytes until the process exits.
 *   - A K split the library chooses itself (variant NULL or split_k 0) is shrunk to what the array holds, exactly as
 *     feather_scaled_mm_ex shrinks it to the caller's workspace.  Only a variant that pins a larger split_k is rejected,
 *     with FEATHER_ERR_WORKSPACE (the message says how much is needed): pass a smaller split_k, or use feather_scaled_mm_ex.
 *   - For a handful of tokens the library's own choice is the register-streaming kernel; it uses the array only for the counters
 *     and partial sums of a K split across CTAs, which it chooses when the weight's columns alone cannot fill the SMs.
 *   - The call allocates and frees nothing.  The first call on each device that needs the array looks its device address
 *     up (cudaGetSymbolAddress, with that device current) and keeps it; make that first call outside any stream capture.
 *   - All calls on a device share the one array and it keeps what the previous call left there; the call clears the tile
 *     counters it is about to use on `stream` before launching.  Two calls that can overlap on the GPU (different
 *     streams, no dependency) would race on it: serialise them or use feather_scaled_mm_ex with separate workspaces.
 * This entry point has no counterpart in the reference. */
FEATHER_API int feather_scaled_mm_static(const void* a, const uint8_t* b_prepacked, const float* scale, const void* bias, void* c,
                                         int64_t M, int64_t N, int64_t K, int64_t ldc, int output_dtype,
                                         const feather_mm_variant* variant, int* status_dev, feather_stream_t stream);

/* Size in bytes of the built-in scratch used by feather_scaled_mm_static.  No counterpart in the reference. */
FEATHER_API size_t feather_scaled_mm_static_scratch_bytes(void);

/* Writes the variant the library would choose for (M,N,K) on the current device into *out.
 * Stands in for the autotuner of kernel/hip/utils.py:192-223 (`old_autotune`). */
FEATHER_API int feather_scaled_mm_choose(int64_t M, int64_t N, int64_t K, size_t workspace_bytes, feather_mm_variant* out);

/* ---------------------------------------------------------------------------------------------
 * Weight format: quantise, prepack, inverse
 * ------------------------------------------------------------------------------------------- */

/* comfy_feather/quant.py:52-74 `quantize_fp8e5m2_scaled` followed by quant.py:11-13 `prepack_transpose`.
 *   src        [N,K] row-major, dtype per src_dtype (fp32 / bf16 / fp16), K % 16 == 0
 *   premul     fp32[1] or NULL: loader path `weight.float() * scale` (quant.py:128) applied to fp32 input
 *              before the amax (only valid with FEATHER_SRC_FP32)
 *   scale_io   fp32[1]: if recalc_scale != 0 it receives amax|x|/57344 (0 -> 1, fp16 clamp of quant.py:56-58);
 *              otherwise it is read as the given scale
 *   amax_scratch  uint32[2] scratch, any contents
 *   dst        [K/16, N, 16] e5m2 bytes
 * Round-to-nearest-even only (the seed = None / 0 branch, quant.py:72-73). */
FEATHER_API int feather_quantize_prepack(const void* src, int src_dtype, const float* premul, int64_t N, int64_t K, int recalc_scale,
                             float* scale_io, uint32_t* amax_scratch, uint8_t* dst, feather_stream_t stream);

/* quant.py:11-13 `prepack_transpose` on bytes: [N,K] -> [K/16,N,16]  (e5m2 checkpoints, quant.py:125-126);
 * also kernel/hip/hip_kernel.py:170-171 `prepack_b_for_scaled_mm` when src_is_kn != 0 (src is [K,N]). */
FEATHER_API int feather_prepack_bytes(const uint8_t* src, int64_t N, int64_t K, int src_is_kn, uint8_t* dst, feather_stream_t stream);

/* quant.py:17-19 `unprepack_transpose`: [K/16,N,16] -> [N,K] bytes (state_dict_tensors, quant.py:108-113). */
FEATHER_API int feather_unprepack_bytes(const uint8_t* src, int64_t N, int64_t K, uint8_t* dst, feather_stream_t stream);

/* quant.py:98-102 `FeatherFP8E5M2PackedLayout.dequantize`: unprepack -> fp32 * scale -> dst dtype
 * (FEATHER_SRC_* codes), dst [N,K] row-major. */
FEATHER_API int feather_dequantize(const uint8_t* src_prepacked, const float* scale, int64_t N, int64_t K, int dst_dtype, void* dst,
                       feather_stream_t stream);

/* kernel/convert.py:24-34 `bf16_to_fp16` (elementwise, round-to-nearest-even like `x.to(torch.float16)`). */
FEATHER_API int feather_bf16_to_fp16(const uint16_t* src, uint16_t* dst, int64_t n, feather_stream_t stream);

/* ---------------------------------------------------------------------------------------------
 * Library state
 * ------------------------------------------------------------------------------------------- */
FEATHER_API const char* feather_last_error_string(void);
/* Library version as major*10000 + minor*100 + patch. */
FEATHER_API int feather_version(void);

#ifdef __cplusplus
}
#endif
#endif /* FEATHER_B200_H_ */
