// Streaming kernel for the bandwidth-bound end of the mixed-precision linear: M <= 32 tokens.
//
// At a handful of tokens the job is to pull the prepacked e5m2 weight (K*N bytes) through the SMs once, at HBM speed; the
// arithmetic is tiny.  The tcgen05 kernel is the wrong tool there (one thread issues eight MMAs per 16 KB of weights and
// becomes the limit), so this kernel keeps everything in registers:
//
//   work item   P strips of 8 output columns n (P*8 n), all of K; P is picked so the items fill the SMs in as few, as full rounds as possible
//   CTA         16 warps; warp w takes the k16-blocks [w*KB/16, (w+1)*KB/16) of the item, so the K split needs no workspace
//   per k16-block and strip: one 32-bit load per lane straight from the prepacked layout (a warp load is the 128 contiguous bytes
//               of a strip), 2 x prmt (e5m2 -> fp16 is byte << 8), one mma.sync.m16n8k16 (tokens x n, fp32 accumulate)
//               per 16-token tile; token fragments come from global/L1 and are reused across the P strips
//   reduce      the 16 warps' fp32 partials go through shared memory and are added in warp order (deterministic), then
//               * scale -> RTNE -> + bias in the output dtype, as in the tensor-memory kernel
//
// Same math as kernel/hip/hip_kernel.cu:125-420 of the reference (which has no small-M path: its README.md:31 names an
// unshipped split-k branch).
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <mutex>

#include "../../include/feather_b200.h"
#include "host_util.h"

namespace feather {

constexpr int kSmWarps = 16;
constexpr int kSmThreads = kSmWarps * 32;

__device__ __forceinline__ void mma_m16n8k16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// out_mode bit 0: the scaled sum is rounded to bf16 (else fp16) and the bias is added in that dtype; bit 1: the value is then
// cast once more, to the other 16-bit dtype, and stored as that.
__device__ __forceinline__ uint16_t sm_finish(float acc, float scale, int out_mode, bool has_bias, uint16_t bias_bits) {
    const float r = acc * scale;
    if (out_mode & 1) {
        __nv_bfloat16 v = __float2bfloat16_rn(r);
        if (has_bias) v = __float2bfloat16_rn(__bfloat162float(v) + __bfloat162float(__ushort_as_bfloat16(bias_bits)));
        if (out_mode & 2) return __half_as_ushort(__float2half_rn(__bfloat162float(v)));
        return __bfloat16_as_ushort(v);
    }
    __half v = __float2half_rn(r);
    if (has_bias) v = __hadd(v, __ushort_as_half(bias_bits));
    if (out_mode & 2) return __bfloat16_as_ushort(__float2bfloat16_rn(__half2float(v)));
    return __half_as_ushort(v);
}

// MT: 16-token tiles (1 or 2); P: strips of 8 n per work item; U: k16-blocks whose loads are issued together.
//
// Inside a k16-block the MMA's k index is permuted (the sum over k does not care): MMA k = 2j, 2j+1 is physical
// k = 4j, 4j+1 and MMA k = 2j+8, 2j+9 is physical k = 4j+2, 4j+3.  Lane (g, j) then needs exactly the aligned 32-bit word j
// of chunk g - a warp load is 128 contiguous bytes - and one 64-bit token load per row.
template <int MT, int P, int U>
__global__ void __launch_bounds__(kSmThreads, 1)
small_m_kernel(const uint16_t* __restrict__ a, const uint8_t* __restrict__ w, const float* __restrict__ scale_ptr,
               const uint16_t* __restrict__ bias, uint16_t* __restrict__ c, int M, int N, int K, long long ldc, int out_bf16, int num_items) {
    constexpr int kTok = MT * 16;
    constexpr int kCols = P * 8;
    constexpr int kPitch = kCols + 1;
    extern __shared__ float red[];                          // [kSmWarps][kTok][kPitch]

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, j = lane & 3;
    const int nkb = K / 16;
    const int kb_begin = static_cast<int>(static_cast<long long>(warp) * nkb / kSmWarps);
    const int kb_end = static_cast<int>(static_cast<long long>(warp + 1) * nkb / kSmWarps);
    const float scale = scale_ptr != nullptr ? __ldg(scale_ptr) : 1.0f;
    const bool has_bias = bias != nullptr;

    for (int item = blockIdx.x; item < num_items; item += gridDim.x) {
        const int n_base = item * kCols;
        float acc[MT][P][4];
#pragma unroll
        for (int mt = 0; mt < MT; ++mt)
#pragma unroll
            for (int s = 0; s < P; ++s)
#pragma unroll
                for (int i = 0; i < 4; ++i) acc[mt][s][i] = 0.0f;

        // this lane's word in the first k16-block plane, strip 0; strips are 128 bytes apart, planes N*16 bytes apart
        const uint8_t* const w_lane = w + static_cast<long long>(n_base) * 16 + lane * 4;
        const long long plane = static_cast<long long>(N) * 16;

        // Two register buffers: the loads of the next U k16-blocks are issued before the current block is multiplied, so the
        // warp always has a block of loads in flight (a plain load-then-compute loop drains the memory pipeline every turn).
        auto load_block = [&](int kb0, uint32_t (&wv)[U][P], uint2 (&af)[U][MT][2]) {
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const int kb = kb0 + u;
                const bool kb_ok = kb < kb_end;
#pragma unroll
                for (int s = 0; s < P; ++s) {
                    wv[u][s] = 0u;
                    if (kb_ok && n_base + s * 8 + g < N) wv[u][s] = __ldg(reinterpret_cast<const uint32_t*>(w_lane + kb * plane + s * 128));
                }
#pragma unroll
                for (int mt = 0; mt < MT; ++mt) {
                    const int r0 = mt * 16 + g, r1 = r0 + 8;
                    const long long k = static_cast<long long>(kb) * 16 + 4 * j;
                    af[u][mt][0] = (kb_ok && r0 < M) ? __ldg(reinterpret_cast<const uint2*>(a + r0 * static_cast<long long>(K) + k)) : make_uint2(0u, 0u);
                    af[u][mt][1] = (kb_ok && r1 < M) ? __ldg(reinterpret_cast<const uint2*>(a + r1 * static_cast<long long>(K) + k)) : make_uint2(0u, 0u);
                }
            }
        };
        auto multiply_block = [&](const uint32_t (&wv)[U][P], const uint2 (&af)[U][MT][2]) {
#pragma unroll
            for (int u = 0; u < U; ++u)
#pragma unroll
                for (int s = 0; s < P; ++s) {
                    const uint32_t b0 = __byte_perm(wv[u][s], 0u, 0x1404);     // physical k = 4j, 4j+1   -> fp16 pair (byte << 8)
                    const uint32_t b1 = __byte_perm(wv[u][s], 0u, 0x3424);     // physical k = 4j+2, 4j+3
#pragma unroll
                    for (int mt = 0; mt < MT; ++mt) {
                        const uint32_t frag[4] = {af[u][mt][0].x, af[u][mt][1].x, af[u][mt][0].y, af[u][mt][1].y};
                        mma_m16n8k16(acc[mt][s], frag, b0, b1);
                    }
                }
        };
        uint32_t w0[U][P], w1[U][P];
        uint2 a0[U][MT][2], a1[U][MT][2];
        int kb0 = kb_begin;
        if (kb0 < kb_end) load_block(kb0, w0, a0);
        while (kb0 < kb_end) {
            const int kb1 = kb0 + U;
            if (kb1 < kb_end) load_block(kb1, w1, a1);
            multiply_block(w0, a0);
            if (kb1 >= kb_end) break;
            kb0 = kb1 + U;
            if (kb0 < kb_end) load_block(kb0, w0, a0);
            multiply_block(w1, a1);
        }

        // fragment layout of D: d0 (row g, col 2j), d1 (row g, col 2j+1), d2 (row g+8, col 2j), d3 (row g+8, col 2j+1)
        float* const mine = red + warp * (kTok * kPitch);
#pragma unroll
        for (int mt = 0; mt < MT; ++mt)
#pragma unroll
            for (int s = 0; s < P; ++s) {
                mine[(mt * 16 + g) * kPitch + s * 8 + 2 * j] = acc[mt][s][0];
                mine[(mt * 16 + g) * kPitch + s * 8 + 2 * j + 1] = acc[mt][s][1];
                mine[(mt * 16 + g + 8) * kPitch + s * 8 + 2 * j] = acc[mt][s][2];
                mine[(mt * 16 + g + 8) * kPitch + s * 8 + 2 * j + 1] = acc[mt][s][3];
            }
        __syncthreads();
        for (int o = threadIdx.x; o < kTok * kCols; o += kSmThreads) {
            const int tok = o / kCols, col = o % kCols;
            const int n = n_base + col;
            if (tok < M && n < N) {
                float sum = 0.0f;
#pragma unroll
                for (int wi = 0; wi < kSmWarps; ++wi) sum += red[wi * (kTok * kPitch) + tok * kPitch + col];   // warp order: deterministic
                const uint16_t bias_bits = has_bias ? __ldg(bias + n) : uint16_t(0);
                c[static_cast<long long>(tok) * ldc + n] = sm_finish(sum, scale, out_bf16, has_bias, bias_bits);
            }
        }
        __syncthreads();
    }
}

// Up to 8 tokens: the weights are the 16-row MMA operand (16 n x 16 k = 256 bytes of weights per MMA, half the MMAs of the
// kernel above, which is bound by the legacy MMA rate) and the tokens the 8-column operand.  P: strips of 16 n per item.
template <int P, int U>
__global__ void __launch_bounds__(kSmThreads, 1)
small_m8_kernel(const uint16_t* __restrict__ a, const uint8_t* __restrict__ w, const float* __restrict__ scale_ptr,
                const uint16_t* __restrict__ bias, uint16_t* __restrict__ c, int M, int N, int K, long long ldc, int out_bf16, int num_items) {
    constexpr int kCols = P * 16;
    constexpr int kPitch = kCols + 1;
    extern __shared__ float red[];                          // [kSmWarps][8 tokens][kPitch]

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, j = lane & 3;
    const int nkb = K / 16;
    const int kb_begin = static_cast<int>(static_cast<long long>(warp) * nkb / kSmWarps);
    const int kb_end = static_cast<int>(static_cast<long long>(warp + 1) * nkb / kSmWarps);
    const float scale = scale_ptr != nullptr ? __ldg(scale_ptr) : 1.0f;
    const bool has_bias = bias != nullptr;

    for (int item = blockIdx.x; item < num_items; item += gridDim.x) {
        const int n_base = item * kCols;
        float acc[P][4];
#pragma unroll
        for (int s = 0; s < P; ++s)
#pragma unroll
            for (int i = 0; i < 4; ++i) acc[s][i] = 0.0f;
        // lane (g, j): word j of chunk g (rows 0-7 of a strip) and of chunk g + 8; a strip is 256 contiguous bytes
        const uint8_t* const w_lane = w + static_cast<long long>(n_base) * 16 + lane * 4;
        const long long plane = static_cast<long long>(N) * 16;

        auto load_block = [&](int kb0, uint32_t (&wv)[U][P][2], uint2 (&tk)[U]) {
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const int kb = kb0 + u;
                const bool kb_ok = kb < kb_end;
#pragma unroll
                for (int s = 0; s < P; ++s) {
                    const int n0 = n_base + s * 16 + g;
                    wv[u][s][0] = (kb_ok && n0 < N) ? __ldg(reinterpret_cast<const uint32_t*>(w_lane + kb * plane + s * 256)) : 0u;
                    wv[u][s][1] = (kb_ok && n0 + 8 < N) ? __ldg(reinterpret_cast<const uint32_t*>(w_lane + kb * plane + s * 256 + 128)) : 0u;
                }
                tk[u] = (kb_ok && g < M) ? __ldg(reinterpret_cast<const uint2*>(a + g * static_cast<long long>(K) + static_cast<long long>(kb) * 16 + 4 * j))
                                         : make_uint2(0u, 0u);
            }
        };
        auto multiply_block = [&](const uint32_t (&wv)[U][P][2], const uint2 (&tk)[U]) {
#pragma unroll
            for (int u = 0; u < U; ++u)
#pragma unroll
                for (int s = 0; s < P; ++s) {
                    // same k permutation as above: bytes 0,1 of the word are MMA k = 2j, 2j+1; bytes 2,3 are MMA k = 2j+8, 2j+9
                    const uint32_t frag[4] = {__byte_perm(wv[u][s][0], 0u, 0x1404), __byte_perm(wv[u][s][1], 0u, 0x1404),
                                              __byte_perm(wv[u][s][0], 0u, 0x3424), __byte_perm(wv[u][s][1], 0u, 0x3424)};
                    mma_m16n8k16(acc[s], frag, tk[u].x, tk[u].y);
                }
        };
        uint32_t w0[U][P][2], w1[U][P][2];
        uint2 t0[U], t1[U];
        int kb0 = kb_begin;
        if (kb0 < kb_end) load_block(kb0, w0, t0);
        while (kb0 < kb_end) {
            const int kb1 = kb0 + U;
            if (kb1 < kb_end) load_block(kb1, w1, t1);
            multiply_block(w0, t0);
            if (kb1 >= kb_end) break;
            kb0 = kb1 + U;
            if (kb0 < kb_end) load_block(kb0, w0, t0);
            multiply_block(w1, t1);
        }
        // D: d0 (n g, token 2j), d1 (n g, token 2j+1), d2 (n g+8, token 2j), d3 (n g+8, token 2j+1)
        float* const mine = red + warp * (8 * kPitch);
#pragma unroll
        for (int s = 0; s < P; ++s) {
            mine[(2 * j) * kPitch + s * 16 + g] = acc[s][0];
            mine[(2 * j + 1) * kPitch + s * 16 + g] = acc[s][1];
            mine[(2 * j) * kPitch + s * 16 + g + 8] = acc[s][2];
            mine[(2 * j + 1) * kPitch + s * 16 + g + 8] = acc[s][3];
        }
        __syncthreads();
        for (int o = threadIdx.x; o < 8 * kCols; o += kSmThreads) {
            const int tok = o / kCols, col = o % kCols;
            const int n = n_base + col;
            if (tok < M && n < N) {
                float sum = 0.0f;
#pragma unroll
                for (int wi = 0; wi < kSmWarps; ++wi) sum += red[wi * (8 * kPitch) + tok * kPitch + col];
                const uint16_t bias_bits = has_bias ? __ldg(bias + n) : uint16_t(0);
                c[static_cast<long long>(tok) * ldc + n] = sm_finish(sum, scale, out_bf16, has_bias, bias_bits);
            }
        }
        __syncthreads();
    }
}

template <int P, int U>
static cudaError_t launch_small8(const void* a, const uint8_t* w, const float* scale, const void* bias, void* c, int M, int N, int K, long long ldc,
                                 int out_bf16, int sms, cudaStream_t stream) {
    auto kernel = small_m8_kernel<P, U>;
    constexpr int kSmem = kSmWarps * 8 * (P * 16 + 1) * static_cast<int>(sizeof(float));
    static std::mutex mu;
    static bool configured[64];
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    {
        std::lock_guard<std::mutex> lock(mu);
        if (dev >= 0 && dev < 64 && !configured[dev]) {
            e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmem);
            if (e != cudaSuccess) return e;
            configured[dev] = true;
        }
    }
    const int items = (N + P * 16 - 1) / (P * 16);
    const int grid = items < sms ? items : sms;
    kernel<<<grid, kSmThreads, kSmem, stream>>>(reinterpret_cast<const uint16_t*>(a), w, scale, reinterpret_cast<const uint16_t*>(bias),
                                                reinterpret_cast<uint16_t*>(c), M, N, K, ldc, out_bf16, items);
    return cudaGetLastError();
}

template <int MT, int P, int U>
static cudaError_t launch_small(const void* a, const uint8_t* w, const float* scale, const void* bias, void* c, int M, int N, int K, long long ldc,
                                int out_bf16, int sms, cudaStream_t stream) {
    auto kernel = small_m_kernel<MT, P, U>;
    constexpr int kSmem = kSmWarps * MT * 16 * (P * 8 + 1) * static_cast<int>(sizeof(float));
    static std::mutex mu;
    static bool configured[64];
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    {
        std::lock_guard<std::mutex> lock(mu);
        if (dev >= 0 && dev < 64 && !configured[dev]) {
            e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmem);
            if (e != cudaSuccess) return e;
            configured[dev] = true;
        }
    }
    const int items = (N + P * 8 - 1) / (P * 8);
    const int grid = items < sms ? items : sms;
    kernel<<<grid, kSmThreads, kSmem, stream>>>(reinterpret_cast<const uint16_t*>(a), w, scale, reinterpret_cast<const uint16_t*>(bias),
                                                reinterpret_cast<uint16_t*>(c), M, N, K, ldc, out_bf16, items);
    return cudaGetLastError();
}

// Strips of 8 columns per work item, from the instantiated set: the one that wastes the fewest SM-rounds; among equals the
// largest (token fragments are reused across the strips of an item).
static int pick_strips(int N, int sms, int max_p, int strip_cols = 8) {
    static const int kChoices[] = {16, 12, 10, 8, 6, 5, 4, 3, 2, 1};
    const int strips = (N + strip_cols - 1) / strip_cols;
    int best_p = 1;
    double best_eff = -1.0;
    for (int p : kChoices) {
        if (p > max_p) continue;
        const int items = (strips + p - 1) / p;
        const int rounds = (items + sms - 1) / sms;
        const double eff = static_cast<double>(strips) / (static_cast<double>(rounds) * sms * p);
        if (eff > best_eff + 0.02) {
            best_eff = eff;
            best_p = p;
        }
    }
    return best_p;
}

#define FEATHER_SMALL_CASE(MT_, P_, U_) \
    case P_: e = launch_small<MT_, P_, U_>(a, w, scale, bias, c, m, n, k, ldc, out_bf16, sms, stream); break;
#define FEATHER_SMALL8_CASE(P_, U_) \
    case P_: e = launch_small8<P_, U_>(a, w, scale, bias, c, m, n, k, ldc, out_bf16, sms, stream); break;

int small_m_launch(const void* a, const uint8_t* w, const float* scale, const void* bias, void* c, int64_t M, int64_t N, int64_t K, int64_t ldc,
                   int output_dtype, int flip_final, int sms, cudaStream_t stream) {
    // the kernels' `out_bf16` argument carries both bits of sm_finish's out_mode
    const int out_bf16 = (output_dtype == FEATHER_OUT_BF16 ? 1 : 0) | (flip_final ? 2 : 0);
    const int m = static_cast<int>(M), n = static_cast<int>(N), k = static_cast<int>(K);
    cudaError_t e = cudaErrorInvalidValue;
    if (M <= 8) {
        switch (pick_strips(n, sms, 8, 16)) {
            FEATHER_SMALL8_CASE(8, 1)
            FEATHER_SMALL8_CASE(6, 1)
            FEATHER_SMALL8_CASE(5, 2)
            FEATHER_SMALL8_CASE(4, 2)
            FEATHER_SMALL8_CASE(3, 2)
            FEATHER_SMALL8_CASE(2, 4)
            FEATHER_SMALL8_CASE(1, 8)
            default: break;
        }
    } else if (M <= 16) {
        switch (pick_strips(n, sms, 16)) {
            FEATHER_SMALL_CASE(1, 16, 1)
            FEATHER_SMALL_CASE(1, 12, 2)
            FEATHER_SMALL_CASE(1, 10, 2)
            FEATHER_SMALL_CASE(1, 8, 2)
            FEATHER_SMALL_CASE(1, 6, 4)
            FEATHER_SMALL_CASE(1, 5, 4)
            FEATHER_SMALL_CASE(1, 4, 4)
            FEATHER_SMALL_CASE(1, 3, 4)
            FEATHER_SMALL_CASE(1, 2, 8)
            FEATHER_SMALL_CASE(1, 1, 8)
            default: break;
        }
    } else {   // two token tiles: twice the accumulators, so at most 8 strips per item
        switch (pick_strips(n, sms, 8)) {
            FEATHER_SMALL_CASE(2, 8, 1)
            FEATHER_SMALL_CASE(2, 6, 1)
            FEATHER_SMALL_CASE(2, 5, 2)
            FEATHER_SMALL_CASE(2, 4, 2)
            FEATHER_SMALL_CASE(2, 3, 2)
            FEATHER_SMALL_CASE(2, 2, 4)
            FEATHER_SMALL_CASE(2, 1, 4)
            default: break;
        }
    }
    if (e != cudaSuccess) return set_error(FEATHER_ERR_CUDA, "small-M kernel launch failed: %s", cudaGetErrorString(e));
    return FEATHER_OK;
}

}  // namespace feather
