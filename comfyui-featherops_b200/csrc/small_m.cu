// Streaming kernel for the bandwidth-bound end of the mixed-precision linear: M <= 32 tokens.
//
// At a handful of tokens the job is to pull the prepacked e5m2 weight (K*N bytes) through the SMs once, at HBM speed; the
// arithmetic is tiny.  The tcgen05 kernel is the wrong tool there (one thread issues eight MMAs per 16 KB of weights and
// becomes the limit), so this kernel keeps everything in registers:
//
//   work item   P strips of output columns n, all of K; P is picked so the items fill the SMs in as few, as full rounds as possible
//   CTA         16 warps; warp w takes the k16-blocks [w*KB/16, (w+1)*KB/16) of the item, so the K split needs no workspace
//   per k16-block and strip of 16 columns: two 32-bit loads per lane straight from the prepacked layout (a warp load is 128
//               contiguous bytes), 4 x prmt (e5m2 -> fp16 is byte << 8) build the 16 n x 16 k MMA operand once, and one
//               mma.sync.m16n8k16 per group of eight tokens multiplies it (fp32 accumulate); token fragments come from
//               global/L1 and are reused across the P strips.  One to four token groups (up to 32 tokens).
//   reduce      the 16 warps' fp32 partials go through shared memory and are added in warp order (deterministic), then
//               * scale -> RTNE -> + bias in the output dtype, as in the tensor-memory kernel
//
//   K split     when the strips alone cannot fill the SMs in full rounds (N = 5120: 320 strips of 16 columns on 148 SMs), ks CTAs
//               share a work item, each over 1/ks of K; a CTA parks its fp32 partial in the caller's workspace and the last
//               of the ks to arrive (a counter per item) adds the partials in slice order - deterministic - and finishes
//   launch      with programmatic dependent launch: the CTAs may become resident and run their prologue while the previous
//               kernel on the stream drains; nothing touches global memory before griddepcontrol.wait
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
#include "ptx.cuh"

namespace feather {

constexpr int kSmWarps = 16;
constexpr int kSmThreads = kSmWarps * 32;
constexpr size_t kSmCounterBytes = 65536;     // tile counters at the start of the workspace (same layout as the tensor-memory kernel's)


struct SplitArgs {
    int ks;              // CTAs per work item (K slices); 1 = no split, the pointers are unused
    float* partials;     // [item][slice][tokens][columns] fp32
    int* counters;       // [item], zero on entry, left at zero
};

// Cross-CTA part of a K split, run by all threads of the CTA after its own 16 warps' partials are in shared memory (`red`,
// summed in warp order by `sum_of`).  Returns through `emit(tok, col, value)` for the elements this thread finishes, which
// happens in the last CTA of the item to arrive; the others only park their partial.
template <int kTok, int kCols, typename SumFn, typename EmitFn>
__device__ __forceinline__ void split_finish(const SplitArgs& sp, int group, int slice, int* flag_smem, SumFn sum_of, EmitFn emit) {
    float* const mine = sp.partials + (static_cast<long long>(group) * sp.ks + slice) * (kTok * kCols);
    for (int o = threadIdx.x; o < kTok * kCols; o += kSmThreads) __stcg(mine + o, sum_of(o / kCols, o % kCols));
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) *flag_smem = (atomicAdd(sp.counters + group, 1) == sp.ks - 1) ? 1 : 0;
    __syncthreads();
    if (*flag_smem != 0) {
        __threadfence();
        const float* const all = sp.partials + static_cast<long long>(group) * sp.ks * (kTok * kCols);
        for (int o = threadIdx.x; o < kTok * kCols; o += kSmThreads) {
            float sum = 0.0f;
            for (int sl = 0; sl < sp.ks; ++sl) sum += __ldcg(all + sl * (kTok * kCols) + o);     // slice order: deterministic
            emit(o / kCols, o % kCols, sum);
        }
        if (threadIdx.x == 0) sp.counters[group] = 0;     // ready for the next launch
    }
    __syncthreads();
}

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

// Inside a k16-block the MMA's k index is permuted (the sum over k does not care): MMA k = 2j, 2j+1 is physical
// k = 4j, 4j+1 and MMA k = 2j+8, 2j+9 is physical k = 4j+2, 4j+3.  Lane (g, j) then needs exactly the aligned 32-bit word j
// of a 16-byte chunk - a warp load is 128 contiguous bytes - and one 64-bit token load per row.
//
// Up to 8 * NT tokens (NT = 1 .. 4): the weights are the 16-row MMA operand (16 n x 16 k = 256 bytes of weights per MMA and
// token group) and each group of eight tokens the 8-column operand; the weight fragment of a strip is built once and
// multiplied with every token group.  P: strips of 16 n per item.
template <int P, int U, int NT>
__global__ void __launch_bounds__(kSmThreads, 1)
small_m8_kernel(const uint16_t* __restrict__ a, const uint8_t* __restrict__ w, const float* __restrict__ scale_ptr,
                const uint16_t* __restrict__ bias, uint16_t* __restrict__ c, int M, int N, int K, long long ldc, int out_bf16, int num_items,
                SplitArgs sp) {
    constexpr int kCols = P * 16;
    constexpr int kPitch = kCols + 1;
    constexpr int kTok = 8 * NT;
    extern __shared__ float red[];                          // [kSmWarps][kTok tokens][kPitch]
    __shared__ int last_flag;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, j = lane & 3;
    const int nkb = K / 16;
    pdl_launch_dependents();
    pdl_wait_for_previous_kernel();
    const float scale = scale_ptr != nullptr ? __ldg(scale_ptr) : 1.0f;
    const bool has_bias = bias != nullptr;

    for (int item = blockIdx.x; item < num_items; item += gridDim.x) {
        const int group = item / sp.ks, slice = item - group * sp.ks;
        const int sl_begin = static_cast<int>(static_cast<long long>(slice) * nkb / sp.ks);
        const int sl_end = static_cast<int>(static_cast<long long>(slice + 1) * nkb / sp.ks);
        const int kb_begin = sl_begin + static_cast<int>(static_cast<long long>(warp) * (sl_end - sl_begin) / kSmWarps);
        const int kb_end = sl_begin + static_cast<int>(static_cast<long long>(warp + 1) * (sl_end - sl_begin) / kSmWarps);
        const int n_base = group * kCols;
        float acc[NT][P][4];
#pragma unroll
        for (int t = 0; t < NT; ++t)
#pragma unroll
            for (int s = 0; s < P; ++s)
#pragma unroll
                for (int i = 0; i < 4; ++i) acc[t][s][i] = 0.0f;
        // lane (g, j): word j of chunk g (rows 0-7 of a strip) and of chunk g + 8; a strip is 256 contiguous bytes
        const uint8_t* const w_lane = w + static_cast<long long>(n_base) * 16 + lane * 4;
        const long long plane = static_cast<long long>(N) * 16;

        auto load_block = [&](int kb0, uint32_t (&wv)[U][P][2], uint2 (&tk)[U][NT]) {
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
#pragma unroll
                for (int t = 0; t < NT; ++t)
                    tk[u][t] = (kb_ok && g + 8 * t < M)
                                   ? __ldg(reinterpret_cast<const uint2*>(a + (g + 8 * t) * static_cast<long long>(K) + static_cast<long long>(kb) * 16 + 4 * j))
                                   : make_uint2(0u, 0u);
            }
        };
        auto multiply_block = [&](const uint32_t (&wv)[U][P][2], const uint2 (&tk)[U][NT]) {
#pragma unroll
            for (int u = 0; u < U; ++u)
#pragma unroll
                for (int s = 0; s < P; ++s) {
                    // same k permutation as above: bytes 0,1 of the word are MMA k = 2j, 2j+1; bytes 2,3 are MMA k = 2j+8, 2j+9
                    const uint32_t frag[4] = {__byte_perm(wv[u][s][0], 0u, 0x1404), __byte_perm(wv[u][s][1], 0u, 0x1404),
                                              __byte_perm(wv[u][s][0], 0u, 0x3424), __byte_perm(wv[u][s][1], 0u, 0x3424)};
#pragma unroll
                    for (int t = 0; t < NT; ++t) mma_m16n8k16(acc[t][s], frag, tk[u][t].x, tk[u][t].y);
                }
        };
        uint32_t w0[U][P][2], w1[U][P][2];
        uint2 t0[U][NT], t1[U][NT];
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
        // D of token group t: d0 (n g, token 8t + 2j), d1 (n g, token 8t + 2j+1), d2 (n g+8, token 8t + 2j), d3 (n g+8, token 8t + 2j+1)
        float* const mine = red + warp * (kTok * kPitch);
#pragma unroll
        for (int t = 0; t < NT; ++t)
#pragma unroll
            for (int s = 0; s < P; ++s) {
                mine[(8 * t + 2 * j) * kPitch + s * 16 + g] = acc[t][s][0];
                mine[(8 * t + 2 * j + 1) * kPitch + s * 16 + g] = acc[t][s][1];
                mine[(8 * t + 2 * j) * kPitch + s * 16 + g + 8] = acc[t][s][2];
                mine[(8 * t + 2 * j + 1) * kPitch + s * 16 + g + 8] = acc[t][s][3];
            }
        __syncthreads();
        auto sum_of = [&](int tok, int col) {
            float sum = 0.0f;
#pragma unroll
            for (int wi = 0; wi < kSmWarps; ++wi) sum += red[wi * (kTok * kPitch) + tok * kPitch + col];
            return sum;
        };
        auto emit = [&](int tok, int col, float sum) {
            const int n = n_base + col;
            if (tok < M && n < N) {
                const uint16_t bias_bits = has_bias ? __ldg(bias + n) : uint16_t(0);
                c[static_cast<long long>(tok) * ldc + n] = sm_finish(sum, scale, out_bf16, has_bias, bias_bits);
            }
        };
        if (sp.ks == 1) {
            for (int o = threadIdx.x; o < kTok * kCols; o += kSmThreads) emit(o / kCols, o % kCols, sum_of(o / kCols, o % kCols));
            __syncthreads();
        } else {
            split_finish<kTok, kCols>(sp, group, slice, &last_flag, sum_of, emit);
        }
    }
}

struct StreamLaunch {
    const void* a;
    const uint8_t* w;
    const float* scale;
    const void* bias;
    void* c;
    int M, N, K;
    long long ldc;
    int out_mode, sms, ks;
    void* workspace;
    cudaStream_t stream;
};

// One launch path for every instantiation: dynamic shared memory opt-in once per device, programmatic dependent launch
// allowed, `ks` CTAs per group of strips when the caller's workspace carries the cross-CTA reduction.
template <typename Kernel>
static cudaError_t launch_stream(Kernel kernel, int smem_bytes, int cols_per_item, int tokens_per_item, const StreamLaunch& L, bool* configured,
                                 std::mutex& mu) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    {
        std::lock_guard<std::mutex> lock(mu);
        if (dev >= 0 && dev < 64 && !configured[dev]) {
            e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes);
            if (e != cudaSuccess) return e;
            configured[dev] = true;
        }
    }
    const int groups = (L.N + cols_per_item - 1) / cols_per_item;
    const int items = groups * L.ks;
    SplitArgs sp{L.ks, nullptr, nullptr};
    if (L.ks > 1) {
        sp.counters = reinterpret_cast<int*>(L.workspace);
        sp.partials = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(L.workspace) + kSmCounterBytes);
    }
    (void)tokens_per_item;
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(static_cast<unsigned>(items < L.sms ? items : L.sms), 1, 1);
    cfg.blockDim = dim3(kSmThreads, 1, 1);
    cfg.dynamicSmemBytes = static_cast<size_t>(smem_bytes);
    cfg.stream = L.stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, reinterpret_cast<const uint16_t*>(L.a), L.w, L.scale, reinterpret_cast<const uint16_t*>(L.bias),
                              reinterpret_cast<uint16_t*>(L.c), L.M, L.N, L.K, L.ldc, L.out_mode, items, sp);
}

template <int P, int U, int NT = 1>
static cudaError_t launch_small8(const StreamLaunch& L) {
    static std::mutex mu;
    static bool configured[64];
    return launch_stream(small_m8_kernel<P, U, NT>, kSmWarps * 8 * NT * (P * 16 + 1) * static_cast<int>(sizeof(float)), P * 16, 8 * NT, L, configured, mu);
}

// How the weight is cut into CTA-sized pieces: P strips per work item (token fragments are reused across the strips of an
// item) and ks K slices per item.  Cost model: rounds of CTAs over the SMs x k16-block-strips per CTA, plus a fixed
// per-CTA cost (prologue, in-CTA reduction, and for a split the trip through the workspace) counted in the same unit.
// Without a workspace ks stays 1.
struct StreamPlan {
    int p, ks;
};
static StreamPlan plan_stream(int N, int K, int sms, const int* p_choices, int n_choices, int strip_cols, int tokens, size_t ws_bytes,
                              double split_cost = 40.0) {
    const int strips = (N + strip_cols - 1) / strip_cols;
    const int nkb = K / 16;
    StreamPlan best{1, 1};
    double best_cost = -1.0;
    for (int i = 0; i < n_choices; ++i) {
        const int p = p_choices[i];
        const int groups = (strips + p - 1) / p;
        for (int ks = 1; ks <= 8; ++ks) {
            if (ks > 1) {
                if (nkb / ks < 2 * kSmWarps) break;                                  // every warp keeps at least two k16-blocks
                const size_t need = kSmCounterBytes + static_cast<size_t>(groups) * ks * tokens * p * strip_cols * sizeof(float);
                if (need > ws_bytes || static_cast<size_t>(groups) * sizeof(int) > kSmCounterBytes) break;
            }
            const long long ctas = static_cast<long long>(groups) * ks;
            const long long rounds = (ctas + sms - 1) / sms;
            const double per_cta = static_cast<double>(p) * nkb / ks + 60.0 + (ks > 1 ? split_cost : 0.0);
            const double cost = rounds * per_cta;
            if (best_cost < 0 || cost < best_cost * 0.98) {
                best_cost = cost;
                best = StreamPlan{p, ks};
            }
        }
    }
    return best;
}

#define FEATHER_SMALL8_CASE(P_, U_) \
    case P_: e = launch_small8<P_, U_>(L); break;

size_t small_m_workspace_bytes(int64_t M, int64_t N, int64_t K, int sms) {
    // upper bound over the plans the launcher may pick: groups * ks * tokens * columns stays below 8 * tokens * N
    (void)K;
    (void)sms;
    const int tokens = M <= 8 ? 8 : M <= 16 ? 16 : 32;
    return kSmCounterBytes + static_cast<size_t>(8) * tokens * static_cast<size_t>(N + 256) * sizeof(float);
}

int small_m_launch(const void* a, const uint8_t* w, const float* scale, const void* bias, void* c, int64_t M, int64_t N, int64_t K, int64_t ldc,
                   int output_dtype, int flip_final, int sms, void* workspace, size_t workspace_bytes, cudaStream_t stream) {
    StreamLaunch L{a, w, scale, bias, c, static_cast<int>(M), static_cast<int>(N), static_cast<int>(K), ldc,
                   // the kernels' `out_bf16` argument carries both bits of sm_finish's out_mode
                   (output_dtype == FEATHER_OUT_BF16 ? 1 : 0) | (flip_final ? 2 : 0), sms, 1, workspace, stream};
    const size_t ws = (workspace != nullptr && (reinterpret_cast<uintptr_t>(workspace) & 15u) == 0) ? workspace_bytes : 0;
    cudaError_t e = cudaErrorInvalidValue;
    if (M <= 8) {
        static const int kP[] = {9, 8, 7, 6, 5, 4, 3, 2, 1};
        const StreamPlan pl = plan_stream(L.N, L.K, sms, kP, 9, 16, 8, ws);
        L.ks = pl.ks;
        switch (pl.p) {
            FEATHER_SMALL8_CASE(9, 1)
            FEATHER_SMALL8_CASE(8, 1)
            FEATHER_SMALL8_CASE(7, 1)
            FEATHER_SMALL8_CASE(6, 1)
            FEATHER_SMALL8_CASE(5, 2)
            FEATHER_SMALL8_CASE(4, 2)
            FEATHER_SMALL8_CASE(3, 2)
            FEATHER_SMALL8_CASE(2, 4)
            FEATHER_SMALL8_CASE(1, 8)
            default: break;
        }
    } else if (M <= 16) {
        // Two groups of eight tokens against the same weight fragments.  With 16 tokens the trip through the workspace (fence,
        // counter, the last CTA's reads) costs about as much as 700 k16-block-strips of streaming - measured 2.6 us against
        // 3.7 ns per strip - so K is split only where that buys many more busy SMs.
        static const int kP[] = {6, 5, 4, 3, 2, 1};
        const StreamPlan pl = plan_stream(L.N, L.K, sms, kP, 6, 16, 16, ws, 700.0);
        L.ks = pl.ks;
        switch (pl.p) {
            case 6: e = launch_small8<6, 1, 2>(L); break;
            case 5: e = launch_small8<5, 2, 2>(L); break;
            case 4: e = launch_small8<4, 2, 2>(L); break;
            case 3: e = launch_small8<3, 2, 2>(L); break;
            case 2: e = launch_small8<2, 4, 2>(L); break;
            case 1: e = launch_small8<1, 8, 2>(L); break;
            default: break;
        }
    } else if (M <= 24) {   // three groups of eight tokens
        static const int kP[] = {4, 3, 2, 1};
        const StreamPlan pl = plan_stream(L.N, L.K, sms, kP, 4, 16, 24, ws, 900.0);
        L.ks = pl.ks;
        switch (pl.p) {
            case 4: e = launch_small8<4, 1, 3>(L); break;
            case 3: e = launch_small8<3, 2, 3>(L); break;
            case 2: e = launch_small8<2, 2, 3>(L); break;
            case 1: e = launch_small8<1, 4, 3>(L); break;
            default: break;
        }
    } else {                // four groups
        static const int kP[] = {3, 2, 1};
        const StreamPlan pl = plan_stream(L.N, L.K, sms, kP, 3, 16, 32, ws, 1100.0);
        L.ks = pl.ks;
        switch (pl.p) {
            case 3: e = launch_small8<3, 1, 4>(L); break;
            case 2: e = launch_small8<2, 2, 4>(L); break;
            case 1: e = launch_small8<1, 4, 4>(L); break;
            default: break;
        }
    }
    if (e != cudaSuccess) return set_error(FEATHER_ERR_CUDA, "small-M kernel launch failed: %s", cudaGetErrorString(e));
    return FEATHER_OK;
}

}  // namespace feather
