// Weight-format kernels: amax -> per-tensor scale -> e5m2 quantise -> prepack to (K/16, N, 16), the inverse
// (unprepack, dequantise), byte-only prepack, and bf16 -> fp16.
//
// Bit-exact targets (the reference computes these with torch elementwise ops on the weight's device):
//   comfy_feather/quant.py:52-74   quantize_fp8e5m2_scaled   (seed None/0 branch: round-to-nearest-even)
//   comfy_feather/quant.py:11-19   prepack_transpose / unprepack_transpose
//   comfy_feather/quant.py:98-102  FeatherFP8E5M2PackedLayout.dequantize
//   kernel/hip/hip_kernel.py:170   prepack_b_for_scaled_mm
//   kernel/convert.py:24-34        bf16_to_fp16
//
// All of them are HBM-bound byte movers: loads and stores are 16-byte vectors, coalesced on both sides by
// staging the (n, k16-block) permutation through shared memory.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/feather_b200.h"
#include "host_util.h"

namespace feather {

char* error_buffer() {
    static thread_local char buf[512] = "";
    return buf;
}

// fp32 -> e5m2 bits, round-to-nearest-even, overflow to inf (not saturating), NaN -> sign|0x7F.
// Same mapping as the fp32 -> Float8_e5m2 cast torch applies for `x.to(torch.float8_e5m2)`.
__device__ __forceinline__ uint32_t f32_to_e5m2_bits(float f) {
    const uint32_t u = __float_as_uint(f);
    const uint32_t sign = (u >> 24) & 0x80u;
    uint32_t a = u & 0x7FFFFFFFu;
    uint32_t r;
    if (a >= 0x47800000u) {                     // |f| >= 65536, inf or NaN
        r = a > 0x7F800000u ? 0x7Fu : 0x7Cu;
    } else if (a < 0x38800000u) {               // below 2^-14: subnormal e5m2, spacing 2^-16
        r = static_cast<uint32_t>(__float2int_rn(__uint_as_float(a) * 65536.0f));
    } else {
        a += 0x000FFFFFu + ((a >> 21) & 1u);    // RTNE on the 21 dropped mantissa bits
        r = (a >> 21) - (112u << 2);            // rebias exponent 127 -> 15; a carry may reach 0x7C = inf
    }
    return r | sign;
}

// Four fp32 -> four e5m2 bytes (element i in byte i).  The hardware conversion rounds to nearest even like torch but
// saturates, so it is used only where torch's result is finite: |x| < 61440 (61440 is the tie between 57344, the largest
// finite e5m2, and 65536, which torch rounds to inf).  A word holding anything at or above that, or a NaN, takes the
// software path; as unsigned integers, |x| bit patterns order like the values and every NaN is above inf.
__device__ __forceinline__ uint32_t f32x4_to_e5m2_word(float x0, float x1, float x2, float x3) {
    const uint32_t a0 = __float_as_uint(x0) & 0x7FFFFFFFu, a1 = __float_as_uint(x1) & 0x7FFFFFFFu;
    const uint32_t a2 = __float_as_uint(x2) & 0x7FFFFFFFu, a3 = __float_as_uint(x3) & 0x7FFFFFFFu;
    const uint32_t m = max(max(a0, a1), max(a2, a3));
    if (m >= 0x47700000u)
        return f32_to_e5m2_bits(x0) | (f32_to_e5m2_bits(x1) << 8) | (f32_to_e5m2_bits(x2) << 16) | (f32_to_e5m2_bits(x3) << 24);
    uint16_t lo, hi;
    // cvt...x2 d, a, b: a -> upper byte, b -> lower byte
    asm("cvt.rn.satfinite.e5m2x2.f32 %0, %1, %2;" : "=h"(lo) : "f"(x1), "f"(x0));
    asm("cvt.rn.satfinite.e5m2x2.f32 %0, %1, %2;" : "=h"(hi) : "f"(x3), "f"(x2));
    return static_cast<uint32_t>(lo) | (static_cast<uint32_t>(hi) << 16);
}

template <int kSrc>
struct Src;
template <>
struct Src<FEATHER_SRC_FP32> {
    static constexpr int kPerVec = 4;   // elements per 16-byte load
    __device__ static void load(const void* base, long long vec_index, float (&x)[4]) {
        const float4 v = __ldg(reinterpret_cast<const float4*>(base) + vec_index);
        x[0] = v.x; x[1] = v.y; x[2] = v.z; x[3] = v.w;
    }
    // x * inv in the source dtype
    __device__ static float mul(float x, float inv) { return __fmul_rn(x, inv); }
    __device__ static float round_scalar(float inv) { return inv; }
};
template <>
struct Src<FEATHER_SRC_BF16> {
    static constexpr int kPerVec = 8;
    __device__ static void load(const void* base, long long vec_index, float (&x)[8]) {
        const uint4 v = __ldg(reinterpret_cast<const uint4*>(base) + vec_index);
        const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            x[2 * i] = __uint_as_float(w[i] << 16);
            x[2 * i + 1] = __uint_as_float(w[i] & 0xFFFF0000u);
        }
    }
    __device__ static float mul(float x, float inv) { return __bfloat162float(__float2bfloat16_rn(__fmul_rn(x, inv))); }
    __device__ static float round_scalar(float inv) { return __bfloat162float(__float2bfloat16_rn(inv)); }
};
template <>
struct Src<FEATHER_SRC_FP16> {
    static constexpr int kPerVec = 8;
    __device__ static void load(const void* base, long long vec_index, float (&x)[8]) {
        const uint4 v = __ldg(reinterpret_cast<const uint4*>(base) + vec_index);
        const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            x[2 * i] = __half2float(__ushort_as_half(static_cast<uint16_t>(w[i] & 0xFFFFu)));
            x[2 * i + 1] = __half2float(__ushort_as_half(static_cast<uint16_t>(w[i] >> 16)));
        }
    }
    __device__ static float mul(float x, float inv) { return __half2float(__float2half_rn(__fmul_rn(x, inv))); }
    __device__ static float round_scalar(float inv) { return __half2float(__float2half_rn(inv)); }
};

// ------------------------------------------------------------------------------------------------
// amax over |x| (after the optional fp32 pre-multiply).  Non-negative floats order like their bit
// patterns and every NaN pattern is larger than inf's, so an unsigned max propagates NaN as torch.amax does.
// ------------------------------------------------------------------------------------------------
template <int kSrc>
__global__ void __launch_bounds__(256) amax_kernel(const void* __restrict__ src, const float* __restrict__ premul, long long nvec,
                                                   uint32_t* __restrict__ out_bits) {
    using S = Src<kSrc>;
    const float pm = (kSrc == FEATHER_SRC_FP32 && premul != nullptr) ? __ldg(premul) : 1.0f;
    const bool use_pm = (kSrc == FEATHER_SRC_FP32 && premul != nullptr);
    uint32_t m = 0;
    for (long long i = blockIdx.x * 256LL + threadIdx.x; i < nvec; i += 256LL * gridDim.x) {
        float x[S::kPerVec];
        S::load(src, i, x);
#pragma unroll
        for (int j = 0; j < S::kPerVec; ++j) {
            const float v = use_pm ? __fmul_rn(x[j], pm) : x[j];
            const uint32_t b = __float_as_uint(v) & 0x7FFFFFFFu;
            m = b > m ? b : m;
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const uint32_t other = __shfl_xor_sync(0xffffffffu, m, o);
        m = other > m ? other : m;
    }
    __shared__ uint32_t warp_max[8];
    if ((threadIdx.x & 31) == 0) warp_max[threadIdx.x >> 5] = m;
    __syncthreads();
    if (threadIdx.x == 0) {
        uint32_t b = warp_max[0];
#pragma unroll
        for (int i = 1; i < 8; ++i) b = warp_max[i] > b ? warp_max[i] : b;
        atomicMax(out_bits, b);
    }
}

// scale = f32(amax) / 57344; 0 -> 1; fp16 sources clamp 1/scale to the fp16 range (quant.py:54-58).
__global__ void scale_from_amax_kernel(const uint32_t* __restrict__ amax_bits, int src_is_fp16, float* __restrict__ scale_out) {
    const float amax = __uint_as_float(*amax_bits);
    float scale = __fdiv_rn(amax, 57344.0f);
    if (scale == 0.0f) scale = 1.0f;
    if (src_is_fp16) {
        float inv = __fdiv_rn(1.0f, scale);
        // torch.clamp propagates NaN; fminf/fmaxf would not
        if (inv == inv) inv = inv < -65504.0f ? -65504.0f : (inv > 65504.0f ? 65504.0f : inv);
        scale = __fdiv_rn(1.0f, inv);
    }
    *scale_out = scale;
}

// ------------------------------------------------------------------------------------------------
// quantise + prepack.  One block converts a tile of 32 weight rows (n) x 128 k (fp32 source) or 256 k (16-bit source) and
// writes 8 or 16 k16-block planes of 32 n x 16 bytes (512 contiguous bytes each).
// ------------------------------------------------------------------------------------------------
constexpr int kQRows = 32;
// k extent of a tile: 512 bytes of every source row, whatever the source type (shorter row segments cost DRAM efficiency)
template <int kSrc>
struct QTile {
    static constexpr int kK = (kSrc == FEATHER_SRC_FP32) ? 128 : 256;
};

template <int kSrc>
__global__ void __launch_bounds__(256)
quantize_prepack_kernel(const void* __restrict__ src, const float* __restrict__ premul, const float* __restrict__ scale,
                        uint8_t* __restrict__ dst, int N, int K) {
    using S = Src<kSrc>;
    constexpr int kPer = S::kPerVec;
    constexpr int kQK = QTile<kSrc>::kK;
    constexpr int kVecPerRow = kQK / kPer;                 // 32 16-byte vectors per row segment
    constexpr int kIters = kQRows * kVecPerRow / 256;      // 4
    __shared__ __align__(16) uint8_t tile[kQK / 16][kQRows + 1][16];   // +1 row: conflict-free 16-byte access both ways

    // Blocks walk the weight from its end to its start: the amax pass that ran just before read it start to end, so the
    // tail is what is still in L2 and the second read of that part costs no HBM traffic.
    const int n0 = (gridDim.y - 1 - blockIdx.y) * kQRows;
    const int k0 = (gridDim.x - 1 - blockIdx.x) * kQK;
    const bool use_pm = (kSrc == FEATHER_SRC_FP32 && premul != nullptr);
    const float pm = use_pm ? __ldg(premul) : 1.0f;
    // inv_scale = (1.0 / scale).to(x.dtype)
    const float inv = S::round_scalar(__fdiv_rn(1.0f, __ldg(scale)));

#pragma unroll
    for (int it = 0; it < kIters; ++it) {
        const int idx = it * 256 + threadIdx.x;
        const int row = idx / kVecPerRow;
        const int cv = idx % kVecPerRow;
        const int n = n0 + row;
        const int k = k0 + cv * kPer;
        if (n < N && k < K) {
            float x[kPer];
            S::load(src, (static_cast<long long>(n) * K + k) / kPer, x);
            uint32_t packed[kPer / 4];
#pragma unroll
            for (int w = 0; w < kPer / 4; ++w) {
                float y[4];
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    float v = x[4 * w + j];
                    if (use_pm) v = __fmul_rn(v, pm);
                    y[j] = S::mul(v, inv);
                }
                packed[w] = f32x4_to_e5m2_word(y[0], y[1], y[2], y[3]);
            }
            const int kk = cv * kPer;                       // k offset inside the tile
            uint8_t* const cell = &tile[kk / 16][row][kk % 16];
            if constexpr (kPer == 4) {
                *reinterpret_cast<uint32_t*>(cell) = packed[0];
            } else {
                *reinterpret_cast<uint2*>(cell) = make_uint2(packed[0], packed[1]);
            }
        }
    }
    __syncthreads();
#pragma unroll
    for (int it = 0; it < (kQK / 16) * kQRows / 256; ++it) {
        const int idx = it * 256 + threadIdx.x;
        const int kb = idx / kQRows;
        const int row = idx % kQRows;
        const int n = n0 + row;
        const int k = k0 + kb * 16;
        if (n < N && k < K) {
            const uint4 v = *reinterpret_cast<const uint4*>(&tile[kb][row][0]);
            *reinterpret_cast<uint4*>(dst + (static_cast<long long>(k / 16) * N + n) * 16) = v;
        }
    }
}

// ------------------------------------------------------------------------------------------------
// byte prepack / unprepack: tile of 32 n x 32 k16-blocks (512 bytes per row)
// ------------------------------------------------------------------------------------------------
constexpr int kPRows = 32;
constexpr int kPKb = 32;

template <bool kInverse>
__global__ void __launch_bounds__(256) prepack_bytes_kernel(const uint8_t* __restrict__ src, uint8_t* __restrict__ dst, int N, int K) {
    __shared__ uint4 tile[kPKb][kPRows + 1];
    const int n0 = blockIdx.y * kPRows;
    const int kb0 = blockIdx.x * kPKb;
    const int nkb = K / 16;
    // row-major side: consecutive threads walk k16-blocks of one row; plane side: consecutive threads walk rows of one plane
#pragma unroll
    for (int it = 0; it < 4; ++it) {
        const int idx = it * 256 + threadIdx.x;
        const int a = idx / 32, b = idx % 32;
        if (!kInverse) {
            const int n = n0 + a, kb = kb0 + b;
            if (n < N && kb < nkb) tile[b][a] = __ldg(reinterpret_cast<const uint4*>(src + static_cast<long long>(n) * K) + kb);
        } else {
            const int kb = kb0 + a, n = n0 + b;
            if (n < N && kb < nkb) tile[a][b] = __ldg(reinterpret_cast<const uint4*>(src) + static_cast<long long>(kb) * N + n);
        }
    }
    __syncthreads();
#pragma unroll
    for (int it = 0; it < 4; ++it) {
        const int idx = it * 256 + threadIdx.x;
        const int a = idx / 32, b = idx % 32;
        if (!kInverse) {
            const int kb = kb0 + a, n = n0 + b;
            if (n < N && kb < nkb) *(reinterpret_cast<uint4*>(dst) + static_cast<long long>(kb) * N + n) = tile[a][b];
        } else {
            const int n = n0 + a, kb = kb0 + b;
            if (n < N && kb < nkb) *(reinterpret_cast<uint4*>(dst + static_cast<long long>(n) * K) + kb) = tile[b][a];
        }
    }
}

// src [K,N] bytes -> dst[kb][n][j] = src[16 kb + j][n].  One thread per (kb, n); reads coalesced along n.
__global__ void __launch_bounds__(256) prepack_kn_kernel(const uint8_t* __restrict__ src, uint8_t* __restrict__ dst, int N, int K) {
    const int n = blockIdx.x * 256 + threadIdx.x;
    const int kb = blockIdx.y;
    if (n >= N) return;
    uint32_t w[4] = {0, 0, 0, 0};
#pragma unroll
    for (int j = 0; j < 16; ++j) w[j / 4] |= static_cast<uint32_t>(__ldg(src + (static_cast<long long>(kb) * 16 + j) * N + n)) << (8 * (j % 4));
    *(reinterpret_cast<uint4*>(dst) + static_cast<long long>(kb) * N + n) = make_uint4(w[0], w[1], w[2], w[3]);
}

// ------------------------------------------------------------------------------------------------
// dequantise: (K/16,N,16) e5m2 -> [N,K] in fp32 / bf16 / fp16: (float(w) * scale).to(dtype)
// ------------------------------------------------------------------------------------------------
template <int kDst>
__global__ void __launch_bounds__(256)
dequantize_kernel(const uint8_t* __restrict__ src, const float* __restrict__ scale, void* __restrict__ dst, int N, int K) {
    __shared__ uint4 tile[kPKb][kPRows + 1];
    const int n0 = blockIdx.y * kPRows;
    const int kb0 = blockIdx.x * kPKb;
    const int nkb = K / 16;
    const float s = __ldg(scale);
#pragma unroll
    for (int it = 0; it < 4; ++it) {
        const int idx = it * 256 + threadIdx.x;
        const int a = idx / 32, b = idx % 32;
        const int kb = kb0 + a, n = n0 + b;
        if (n < N && kb < nkb) tile[a][b] = __ldg(reinterpret_cast<const uint4*>(src) + static_cast<long long>(kb) * N + n);
    }
    __syncthreads();
#pragma unroll
    for (int it = 0; it < 4; ++it) {
        const int idx = it * 256 + threadIdx.x;
        const int a = idx / 32, b = idx % 32;
        const int n = n0 + a, kb = kb0 + b;
        if (n >= N || kb >= nkb) continue;
        const uint4 q = tile[b][a];
        const uint32_t w[4] = {q.x, q.y, q.z, q.w};
        float f[16];
#pragma unroll
        for (int j = 0; j < 16; ++j) {
            const uint32_t byte = (w[j / 4] >> (8 * (j % 4))) & 0xFFu;
            f[j] = __fmul_rn(__half2float(__ushort_as_half(static_cast<uint16_t>(byte << 8))), s);
        }
        const long long off = static_cast<long long>(n) * K + static_cast<long long>(kb) * 16;
        if constexpr (kDst == FEATHER_SRC_FP32) {
            float4* o = reinterpret_cast<float4*>(reinterpret_cast<float*>(dst) + off);
#pragma unroll
            for (int j = 0; j < 4; ++j) o[j] = make_float4(f[4 * j], f[4 * j + 1], f[4 * j + 2], f[4 * j + 3]);
        } else {
            uint32_t h[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                uint32_t lo, hi;
                if constexpr (kDst == FEATHER_SRC_BF16) {
                    lo = __bfloat16_as_ushort(__float2bfloat16_rn(f[2 * j]));
                    hi = __bfloat16_as_ushort(__float2bfloat16_rn(f[2 * j + 1]));
                } else {
                    lo = __half_as_ushort(__float2half_rn(f[2 * j]));
                    hi = __half_as_ushort(__float2half_rn(f[2 * j + 1]));
                }
                h[j] = lo | (hi << 16);
            }
            uint4* o = reinterpret_cast<uint4*>(reinterpret_cast<uint16_t*>(dst) + off);
            o[0] = make_uint4(h[0], h[1], h[2], h[3]);
            o[1] = make_uint4(h[4], h[5], h[6], h[7]);
        }
    }
}

// ------------------------------------------------------------------------------------------------
// bf16 -> fp16, round-to-nearest-even (overflow to inf), 8 elements per thread per step
// ------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256) bf16_to_fp16_kernel(const uint16_t* __restrict__ src, uint16_t* __restrict__ dst, long long n) {
    const long long nvec = n / 8;
    for (long long i = blockIdx.x * 256LL + threadIdx.x; i < nvec; i += 256LL * gridDim.x) {
        const uint4 v = __ldg(reinterpret_cast<const uint4*>(src) + i);
        const uint32_t w[4] = {v.x, v.y, v.z, v.w};
        uint32_t o[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const uint32_t lo = __half_as_ushort(__float2half_rn(__uint_as_float(w[j] << 16)));
            const uint32_t hi = __half_as_ushort(__float2half_rn(__uint_as_float(w[j] & 0xFFFF0000u)));
            o[j] = lo | (hi << 16);
        }
        *(reinterpret_cast<uint4*>(dst) + i) = make_uint4(o[0], o[1], o[2], o[3]);
    }
    // tail (n not a multiple of 8)
    if (blockIdx.x == 0) {
        for (long long i = nvec * 8 + threadIdx.x; i < n; i += 256)
            dst[i] = __half_as_ushort(__float2half_rn(__uint_as_float(static_cast<uint32_t>(src[i]) << 16)));
    }
}

static int check_launch(const char* what) {
    const cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return set_error(FEATHER_ERR_CUDA, "%s launch failed: %s", what, cudaGetErrorString(e));
    return FEATHER_OK;
}

static bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

static int check_nk(int64_t N, int64_t K) {
    if (N <= 0 || K <= 0) return set_error(FEATHER_ERR_BAD_ARGUMENT, "N and K must be positive");
    if (K % 16 != 0) return set_error(FEATHER_ERR_BAD_ARGUMENT, "Feather FP8 packed weights require K divisible by 16");
    if (N > 0x7FFFFFFF || K > 0x7FFFFFFF) return set_error(FEATHER_ERR_BAD_ARGUMENT, "N and K must fit in 31 bits");
    if ((N + kQRows - 1) / kQRows > 65535) return set_error(FEATHER_ERR_BAD_ARGUMENT, "N too large for one launch");
    return FEATHER_OK;
}

}  // namespace feather

using namespace feather;

extern "C" int feather_quantize_prepack(const void* src, int src_dtype, const float* premul, int64_t N, int64_t K, int recalc_scale,
                                        float* scale_io, uint32_t* amax_scratch, uint8_t* dst, feather_stream_t stream_) {
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    if (src == nullptr || dst == nullptr || scale_io == nullptr) return set_error(FEATHER_ERR_BAD_ARGUMENT, "src, dst and scale_io must not be null");
    if (int st = check_nk(N, K)) return st;
    if (src_dtype != FEATHER_SRC_FP32 && src_dtype != FEATHER_SRC_BF16 && src_dtype != FEATHER_SRC_FP16)
        return set_error(FEATHER_ERR_BAD_ARGUMENT, "src_dtype must be 0 (fp32), 1 (bf16) or 2 (fp16)");
    if (premul != nullptr && src_dtype != FEATHER_SRC_FP32) return set_error(FEATHER_ERR_BAD_ARGUMENT, "premul needs an fp32 source");
    if (!aligned16(src) || !aligned16(dst)) return set_error(FEATHER_ERR_BAD_ARGUMENT, "src and dst must be 16-byte aligned");
    if (recalc_scale && amax_scratch == nullptr) return set_error(FEATHER_ERR_BAD_ARGUMENT, "amax_scratch must not be null when the scale is recalculated");

    const long long total = static_cast<long long>(N) * K;
    if (recalc_scale) {
        cudaError_t e = cudaMemsetAsync(amax_scratch, 0, sizeof(uint32_t), stream);
        if (e != cudaSuccess) return set_error(FEATHER_ERR_CUDA, "memset failed: %s", cudaGetErrorString(e));
        const int per = src_dtype == FEATHER_SRC_FP32 ? 4 : 8;
        const long long nvec = total / per;
        long long blocks = (nvec + 255) / 256;
        if (blocks > 148 * 16) blocks = 148 * 16;
        if (blocks < 1) blocks = 1;
        switch (src_dtype) {
            case FEATHER_SRC_FP32: amax_kernel<FEATHER_SRC_FP32><<<static_cast<unsigned>(blocks), 256, 0, stream>>>(src, premul, nvec, amax_scratch); break;
            case FEATHER_SRC_BF16: amax_kernel<FEATHER_SRC_BF16><<<static_cast<unsigned>(blocks), 256, 0, stream>>>(src, premul, nvec, amax_scratch); break;
            default: amax_kernel<FEATHER_SRC_FP16><<<static_cast<unsigned>(blocks), 256, 0, stream>>>(src, premul, nvec, amax_scratch); break;
        }
        if (int st = check_launch("amax")) return st;
        scale_from_amax_kernel<<<1, 1, 0, stream>>>(amax_scratch, src_dtype == FEATHER_SRC_FP16 ? 1 : 0, scale_io);
        if (int st = check_launch("scale")) return st;
    }
    const int qk = src_dtype == FEATHER_SRC_FP32 ? QTile<FEATHER_SRC_FP32>::kK : QTile<FEATHER_SRC_BF16>::kK;
    const dim3 grid(static_cast<unsigned>((K + qk - 1) / qk), static_cast<unsigned>((N + kQRows - 1) / kQRows));
    switch (src_dtype) {
        case FEATHER_SRC_FP32:
            quantize_prepack_kernel<FEATHER_SRC_FP32><<<grid, 256, 0, stream>>>(src, premul, scale_io, dst, static_cast<int>(N), static_cast<int>(K));
            break;
        case FEATHER_SRC_BF16:
            quantize_prepack_kernel<FEATHER_SRC_BF16><<<grid, 256, 0, stream>>>(src, premul, scale_io, dst, static_cast<int>(N), static_cast<int>(K));
            break;
        default:
            quantize_prepack_kernel<FEATHER_SRC_FP16><<<grid, 256, 0, stream>>>(src, premul, scale_io, dst, static_cast<int>(N), static_cast<int>(K));
            break;
    }
    return check_launch("quantize_prepack");
}

extern "C" int feather_prepack_bytes(const uint8_t* src, int64_t N, int64_t K, int src_is_kn, uint8_t* dst, feather_stream_t stream_) {
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    if (src == nullptr || dst == nullptr) return set_error(FEATHER_ERR_BAD_ARGUMENT, "src and dst must not be null");
    if (int st = check_nk(N, K)) return st;
    if (!aligned16(dst)) return set_error(FEATHER_ERR_BAD_ARGUMENT, "dst must be 16-byte aligned");
    if (src_is_kn) {
        if (K / 16 > 65535) return set_error(FEATHER_ERR_BAD_ARGUMENT, "K too large for one launch");
        const dim3 grid(static_cast<unsigned>((N + 255) / 256), static_cast<unsigned>(K / 16));
        prepack_kn_kernel<<<grid, 256, 0, stream>>>(src, dst, static_cast<int>(N), static_cast<int>(K));
        return check_launch("prepack_kn");
    }
    if (!aligned16(src)) return set_error(FEATHER_ERR_BAD_ARGUMENT, "src must be 16-byte aligned");
    const dim3 grid(static_cast<unsigned>((K / 16 + kPKb - 1) / kPKb), static_cast<unsigned>((N + kPRows - 1) / kPRows));
    prepack_bytes_kernel<false><<<grid, 256, 0, stream>>>(src, dst, static_cast<int>(N), static_cast<int>(K));
    return check_launch("prepack_bytes");
}

extern "C" int feather_unprepack_bytes(const uint8_t* src, int64_t N, int64_t K, uint8_t* dst, feather_stream_t stream_) {
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    if (src == nullptr || dst == nullptr) return set_error(FEATHER_ERR_BAD_ARGUMENT, "src and dst must not be null");
    if (int st = check_nk(N, K)) return st;
    if (!aligned16(src) || !aligned16(dst)) return set_error(FEATHER_ERR_BAD_ARGUMENT, "src and dst must be 16-byte aligned");
    const dim3 grid(static_cast<unsigned>((K / 16 + kPKb - 1) / kPKb), static_cast<unsigned>((N + kPRows - 1) / kPRows));
    prepack_bytes_kernel<true><<<grid, 256, 0, stream>>>(src, dst, static_cast<int>(N), static_cast<int>(K));
    return check_launch("unprepack_bytes");
}

extern "C" int feather_dequantize(const uint8_t* src_prepacked, const float* scale, int64_t N, int64_t K, int dst_dtype, void* dst,
                                  feather_stream_t stream_) {
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    if (src_prepacked == nullptr || dst == nullptr || scale == nullptr) return set_error(FEATHER_ERR_BAD_ARGUMENT, "src, scale and dst must not be null");
    if (int st = check_nk(N, K)) return st;
    if (!aligned16(src_prepacked) || !aligned16(dst)) return set_error(FEATHER_ERR_BAD_ARGUMENT, "src and dst must be 16-byte aligned");
    const dim3 grid(static_cast<unsigned>((K / 16 + kPKb - 1) / kPKb), static_cast<unsigned>((N + kPRows - 1) / kPRows));
    const int n = static_cast<int>(N), k = static_cast<int>(K);
    switch (dst_dtype) {
        case FEATHER_SRC_FP32: dequantize_kernel<FEATHER_SRC_FP32><<<grid, 256, 0, stream>>>(src_prepacked, scale, dst, n, k); break;
        case FEATHER_SRC_BF16: dequantize_kernel<FEATHER_SRC_BF16><<<grid, 256, 0, stream>>>(src_prepacked, scale, dst, n, k); break;
        case FEATHER_SRC_FP16: dequantize_kernel<FEATHER_SRC_FP16><<<grid, 256, 0, stream>>>(src_prepacked, scale, dst, n, k); break;
        default: return set_error(FEATHER_ERR_BAD_ARGUMENT, "dst_dtype must be 0 (fp32), 1 (bf16) or 2 (fp16)");
    }
    return check_launch("dequantize");
}

extern "C" int feather_bf16_to_fp16(const uint16_t* src, uint16_t* dst, int64_t n, feather_stream_t stream_) {
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    if (n < 0) return set_error(FEATHER_ERR_BAD_ARGUMENT, "n must not be negative");
    if (n == 0) return FEATHER_OK;
    if (src == nullptr || dst == nullptr) return set_error(FEATHER_ERR_BAD_ARGUMENT, "src and dst must not be null");
    if (!aligned16(src) || !aligned16(dst)) return set_error(FEATHER_ERR_BAD_ARGUMENT, "src and dst must be 16-byte aligned");
    long long blocks = (n / 8 + 255) / 256;
    if (blocks > 148 * 16) blocks = 148 * 16;
    if (blocks < 1) blocks = 1;
    bf16_to_fp16_kernel<<<static_cast<unsigned>(blocks), 256, 0, stream>>>(src, dst, n);
    return check_launch("bf16_to_fp16");
}

extern "C" const char* feather_last_error_string(void) { return error_buffer(); }
extern "C" int feather_version(void) { return 100; }
