// Exchange steps of the sharded linears (the GPUs of one box).
//
// Row-parallel linear (K sharded):
// Every rank's GEMM has TMA-stored its partial of token rows [d*R, (d+1)*R) into slot `rank` of rank d's buffer
// (feather_scaled_mm_scatter), so this GPU holds n_src partials [n_src][R][N] of the rows it owns.  The kernel here adds
// them in fp32 in slot order (deterministic on every rank and every run), rounds once to the 16-bit output dtype, adds the
// bias in that dtype exactly as the GEMM epilogue does, optionally adds a residual, and writes the finished rows to every
// destination: its own [M, N] output and, with plain 16-byte stores over NVLink, the same rows of each peer's output.
// That last part is the all-gather of the reduced rows, so no separate collective follows.  Only stores cross NVLink.
//
// HBM-bound: reads n_src * R * N * 2 bytes (+ residual), writes R * N * 2 bytes per destination.
//
// Column-parallel linear (N sharded): feather_copy_block hands a finished [M, N/g] column block to a copy engine, which
// writes it into the same columns of a peer's [M, N] buffer without taking an SM - on a second stream, under the GEMM of
// the next linear.
// The reference has no multi-GPU path, so nothing here has a counterpart there; the rounding and bias rules are those of
// kernel/naive.py:34-40 (cast to the output dtype, then add the bias in that dtype).
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/feather_b200.h"
#include "host_util.h"

namespace feather {

constexpr int kMaxReduceDst = 8;
constexpr int kMaxReduceSrc = 8;

struct ReduceDst {
    uint16_t* p[kMaxReduceDst];
};

template <bool kBf16>
__device__ __forceinline__ float2 unpack2(uint32_t w) {
    if constexpr (kBf16)
        return make_float2(__uint_as_float(w << 16), __uint_as_float(w & 0xFFFF0000u));
    else
        return __half22float2(*reinterpret_cast<const __half2*>(&w));
}

// sum (fp32) -> out dtype (RTNE) -> + bias in the out dtype -> + residual in the out dtype
template <bool kBf16>
__device__ __forceinline__ uint32_t finish2(float s0, float s1, bool has_bias, uint32_t bias2, bool has_res, uint32_t res2) {
    if constexpr (kBf16) {
        __nv_bfloat162 v = __floats2bfloat162_rn(s0, s1);
        if (has_bias) v = __hadd2(v, *reinterpret_cast<const __nv_bfloat162*>(&bias2));
        if (has_res) v = __hadd2(v, *reinterpret_cast<const __nv_bfloat162*>(&res2));
        return *reinterpret_cast<const uint32_t*>(&v);
    } else {
        __half2 v = __floats2half2_rn(s0, s1);
        if (has_bias) v = __hadd2(v, *reinterpret_cast<const __half2*>(&bias2));
        if (has_res) v = __hadd2(v, *reinterpret_cast<const __half2*>(&res2));
        return *reinterpret_cast<const uint32_t*>(&v);
    }
}

template <bool kBf16>
__global__ void __launch_bounds__(256) reduce_partials_kernel(const uint16_t* __restrict__ partials, int n_src, long long rows, int N,
                                                              const uint16_t* __restrict__ bias, const uint16_t* __restrict__ residual,
                                                              long long ld_res, ReduceDst dst, int n_dst, long long ld_dst) {
    const int vec_per_row = N / 8;
    const long long nvec = rows * vec_per_row;
    const long long slot = rows * static_cast<long long>(N) / 8;          // uint4 per partial
    const uint4* const src = reinterpret_cast<const uint4*>(partials);
    for (long long i = blockIdx.x * 256LL + threadIdx.x; i < nvec; i += 256LL * gridDim.x) {
        const long long r = i / vec_per_row;
        const int cv = static_cast<int>(i - r * vec_per_row);
        float acc[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[j] = 0.0f;
        // all loads of a vector are independent; the additions stay in slot order
        uint4 v[kMaxReduceSrc];
#pragma unroll
        for (int s = 0; s < kMaxReduceSrc; ++s)
            if (s < n_src) v[s] = __ldcs(src + s * slot + i);
#pragma unroll
        for (int s = 0; s < kMaxReduceSrc; ++s) {
            if (s < n_src) {
                const uint32_t w[4] = {v[s].x, v[s].y, v[s].z, v[s].w};
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const float2 f = unpack2<kBf16>(w[j]);
                    acc[2 * j] += f.x;
                    acc[2 * j + 1] += f.y;
                }
            }
        }
        uint4 b = make_uint4(0u, 0u, 0u, 0u), rs = make_uint4(0u, 0u, 0u, 0u);
        if (bias != nullptr) b = __ldg(reinterpret_cast<const uint4*>(bias) + cv);
        if (residual != nullptr) rs = __ldcs(reinterpret_cast<const uint4*>(residual + r * ld_res) + cv);
        const uint32_t bw[4] = {b.x, b.y, b.z, b.w}, rw[4] = {rs.x, rs.y, rs.z, rs.w};
        uint32_t o[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) o[j] = finish2<kBf16>(acc[2 * j], acc[2 * j + 1], bias != nullptr, bw[j], residual != nullptr, rw[j]);
        const uint4 out = make_uint4(o[0], o[1], o[2], o[3]);
#pragma unroll
        for (int d = 0; d < kMaxReduceDst; ++d)
            if (d < n_dst) *(reinterpret_cast<uint4*>(dst.p[d] + r * ld_dst) + cv) = out;
    }
}

}  // namespace feather

using namespace feather;

extern "C" int feather_reduce_partials(const void* partials, int n_src, int64_t rows, int64_t N, const void* bias, const void* residual,
                                       int64_t ld_res, void* const* dst_list_host, int n_dst, int64_t ld_dst, int dtype,
                                       feather_stream_t stream_) {
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    auto aligned16 = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; };
    if (partials == nullptr || dst_list_host == nullptr) return set_error(FEATHER_ERR_BAD_ARGUMENT, "partials and dst_list_host must not be null");
    if (n_src < 1 || n_src > kMaxReduceSrc) return set_error(FEATHER_ERR_BAD_ARGUMENT, "n_src must be 1 .. %d", kMaxReduceSrc);
    if (n_dst < 1 || n_dst > kMaxReduceDst) return set_error(FEATHER_ERR_BAD_ARGUMENT, "n_dst must be 1 .. %d", kMaxReduceDst);
    if (rows < 0 || N <= 0 || N > 0x7FFFFFFF) return set_error(FEATHER_ERR_BAD_ARGUMENT, "rows and N must be positive");
    if (N % 8 != 0 || ld_dst % 8 != 0 || ld_dst < N) return set_error(FEATHER_ERR_BAD_ARGUMENT, "N and ld_dst must be multiples of 8, ld_dst >= N");
    if (residual != nullptr && (ld_res % 8 != 0 || ld_res < N || !aligned16(residual)))
        return set_error(FEATHER_ERR_BAD_ARGUMENT, "residual must be 16-byte aligned with ld_res a multiple of 8 and >= N");
    if (dtype != FEATHER_OUT_FP16 && dtype != FEATHER_OUT_BF16) return set_error(FEATHER_ERR_BAD_ARGUMENT, "dtype must be 0 (fp16) or 1 (bf16)");
    if (!aligned16(partials) || (bias != nullptr && !aligned16(bias))) return set_error(FEATHER_ERR_BAD_ARGUMENT, "partials and bias must be 16-byte aligned");
    ReduceDst dst{};
    for (int d = 0; d < n_dst; ++d) {
        if (dst_list_host[d] == nullptr || !aligned16(dst_list_host[d]))
            return set_error(FEATHER_ERR_BAD_ARGUMENT, "every destination must be non-null and 16-byte aligned");
        dst.p[d] = reinterpret_cast<uint16_t*>(dst_list_host[d]);
    }
    if (rows == 0) return FEATHER_OK;
    const long long nvec = rows * (N / 8);
    long long blocks = (nvec + 255) / 256;
    if (blocks > 148 * 8) blocks = 148 * 8;
    if (dtype == FEATHER_OUT_BF16)
        reduce_partials_kernel<true><<<static_cast<unsigned>(blocks), 256, 0, stream>>>(
            reinterpret_cast<const uint16_t*>(partials), n_src, rows, static_cast<int>(N), reinterpret_cast<const uint16_t*>(bias),
            reinterpret_cast<const uint16_t*>(residual), ld_res, dst, n_dst, ld_dst);
    else
        reduce_partials_kernel<false><<<static_cast<unsigned>(blocks), 256, 0, stream>>>(
            reinterpret_cast<const uint16_t*>(partials), n_src, rows, static_cast<int>(N), reinterpret_cast<const uint16_t*>(bias),
            reinterpret_cast<const uint16_t*>(residual), ld_res, dst, n_dst, ld_dst);
    const cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return set_error(FEATHER_ERR_CUDA, "reduce_partials launch failed: %s", cudaGetErrorString(e));
    return FEATHER_OK;
}

extern "C" int feather_copy_block(void* dst, int64_t dst_pitch_bytes, const void* src, int64_t src_pitch_bytes, int64_t width_bytes, int64_t rows,
                                  feather_stream_t stream_) {
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    if (dst == nullptr || src == nullptr) return set_error(FEATHER_ERR_BAD_ARGUMENT, "dst and src must not be null");
    if (width_bytes < 0 || rows < 0 || dst_pitch_bytes < width_bytes || src_pitch_bytes < width_bytes)
        return set_error(FEATHER_ERR_BAD_ARGUMENT, "width and rows must not be negative and no pitch smaller than the width");
    if (width_bytes == 0 || rows == 0) return FEATHER_OK;
    const cudaError_t e = cudaMemcpy2DAsync(dst, static_cast<size_t>(dst_pitch_bytes), src, static_cast<size_t>(src_pitch_bytes),
                                            static_cast<size_t>(width_bytes), static_cast<size_t>(rows), cudaMemcpyDeviceToDevice, stream);
    if (e != cudaSuccess) return set_error(FEATHER_ERR_CUDA, "cudaMemcpy2DAsync failed: %s", cudaGetErrorString(e));
    return FEATHER_OK;
}
