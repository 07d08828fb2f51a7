// fp16 activations @ prepacked fp8e5m2 weights -> fp16/bf16, fp32 accumulate, for sm_100a.
//
// Stands in for the reference's scaled_mm_kernel / launch_scaled_mm (kernel/hip/hip_kernel.cu:125-632).
// The design is not the reference's: the weight tile is the MMA "A" operand and lives in tensor memory.
//
//   out^T tile [128 weight columns n  x  TN tokens]  +=  up(W)[128 n x 16 k]  *  A^T[16 k x TN tokens]
//
//   producer warp   TMA: W bytes  [4 k16-blocks][128 n][16 B] (the prepacked layout, verbatim)  -> smem ring
//                   TMA: A tokens [TN rows][64 k] fp16, 128-byte swizzle                         -> smem ring
//   transform warps ld.shared 16 B (one n, 16 k) -> 8 x prmt (e5m2 -> fp16 is `byte << 8`, exact)
//                   -> tcgen05.st into a TMEM ring (32 columns per 64-k stage); fp16 W never touches smem
//   MMA warp        tcgen05.mma kind::f16, A from TMEM, B (tokens) from smem descriptor, D fp32 in TMEM
//   epilogue warps  tcgen05.ld -> *scale -> RTNE to out dtype -> +bias in out dtype -> global stores
//                   (lane = n, so a warp writes 32 consecutive n of one token row); split-K slices park
//                   fp32 partials in a workspace and the last slice to arrive reduces them in slice order.
//
// CG = 2 pairs two CTAs on one 256-n tile (tcgen05 cta_group::2): each CTA loads/transforms its own
// 128 n and half of the tokens; barriers that the issuing CTA needs are signalled across the pair.
// No TMA multicast is used anywhere.
//
// Every wait is bounded (ptx.cuh); on expiry the CTA records a code in *status, drains and returns.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>
#include <string.h>

#include <mutex>

#include "../../include/feather_b200.h"
#include "host_util.h"
#include "ptx.cuh"

namespace feather {

constexpr int kBW = 128;                      // weight columns per CTA = MMA M per CTA = TMEM lanes
constexpr int kBK = 64;                       // k per pipeline stage
constexpr int kKSteps = kBK / 16;             // MMA k-steps per stage
constexpr int kWStageBytes = kBW * kBK;       // e5m2 bytes per stage
constexpr int kTStages = 4;                   // TMEM ring depth for upcast weights
constexpr int kTColsPerStage = kBK / 2;       // 32-bit TMEM columns per stage (two fp16 per column)
constexpr int kEpilogueWarps = 4;
constexpr int kMaxStages = 24;

__host__ __device__ constexpr int pow2_at_least(int x) {
    int p = 32;
    while (p < x) p <<= 1;
    return p;
}

template <int TN, int CG>
struct Cfg {
    static_assert(TN == 16 || TN == 32 || TN == 64 || TN == 128 || TN == 256, "tokens tile");
    static_assert(CG == 1 || CG == 2, "cta group");
    static constexpr int kTokLoad = TN / CG;              // token rows this CTA loads per stage
    static constexpr int kAStageBytes = kTokLoad * 128;   // 64 fp16 per row
    static constexpr int kStageBytes = kWStageBytes + kAStageBytes;
    static constexpr int kAccs = (TN <= 128) ? 2 : 1;     // accumulator buffers in TMEM
    static constexpr int kAccCols = kAccs * TN;
    static constexpr int kTmemCols = pow2_at_least(kAccCols + kTStages * kTColsPerStage);
    static constexpr int kBarrierBytes = 1024;
    static constexpr int kSmemBudget = 227 * 1024 - 1024 /*alignment slack*/ - kBarrierBytes;
    static constexpr int kStagesRaw = kSmemBudget / kStageBytes;
    static constexpr int kStages = kStagesRaw > kMaxStages ? kMaxStages : kStagesRaw;
    static constexpr int kSmemBytes = kStages * kStageBytes + kBarrierBytes + 1024;
    static_assert(kTmemCols <= 512, "TMEM columns");
    static_assert(kAStageBytes % 1024 == 0, "swizzle atom alignment of token stages");
    static_assert((3 * kMaxStages + 2 * kTStages + 2 * 2 + 1) * 8 + 16 <= kBarrierBytes, "barrier block");
};

struct MmParams {
    const float* scale;
    const void* bias;
    void* c;
    float* ws_partials;
    int* ws_counters;
    int* status;
    int M, N, K;
    long long ldc;
    int out_bf16;
    int splits;
    int tiles_n, tiles_t, num_units, total_kb;
};

struct Unit {
    int tile, split, n0, tok0, kb_begin, kb_count;
};

template <int TN, int CG>
__device__ __forceinline__ Unit decode_unit(const MmParams& p, int u) {
    Unit w;
    w.tile = u / p.splits;
    w.split = u - w.tile * p.splits;
    const int nt = w.tile % p.tiles_n;
    const int tt = w.tile / p.tiles_n;
    w.n0 = nt * kBW * CG;
    w.tok0 = tt * TN;
    const int base = p.total_kb / p.splits;
    const int rem = p.total_kb - base * p.splits;
    w.kb_begin = w.split * base + (w.split < rem ? w.split : rem);
    w.kb_count = base + (w.split < rem ? 1 : 0);
    return w;
}

// role ids recorded in the status word: bits 8..15
enum { kRoleProducer = 1, kRoleMma = 2, kRoleTransform = 3, kRoleEpilogue = 4 };

template <int CG>
__device__ __forceinline__ void give_up(const MmParams& p, volatile int* abort_flag, int role, int detail) {
    *abort_flag = 1;
    if constexpr (CG == 2) {
        const uint32_t peer = mapa_u32(smem_u32(const_cast<int*>(abort_flag)), cluster_ctarank() ^ 1u);
        asm volatile("st.shared::cluster.u32 [%0], %1;" ::"r"(peer), "r"(1) : "memory");
    }
    if (p.status != nullptr) atomicCAS(p.status, 0, FEATHER_ERR_DEVICE_TIMEOUT | (role << 8) | ((detail & 0xFFFF) << 16));
}

__device__ __forceinline__ uint16_t finish_value(float acc, float scale, bool out_bf16, bool has_bias, uint16_t bias_bits) {
    const float r = acc * scale;
    if (out_bf16) {
        __nv_bfloat16 v = __float2bfloat16_rn(r);
        if (has_bias) v = __float2bfloat16_rn(__bfloat162float(v) + __bfloat162float(__ushort_as_bfloat16(bias_bits)));
        return __bfloat16_as_ushort(v);
    }
    __half v = __float2half_rn(r);
    if (has_bias) v = __hadd(v, __ushort_as_half(bias_bits));
    return __half_as_ushort(v);
}

template <int TN, int CG, int TG>
__global__ void __launch_bounds__(32 * (kEpilogueWarps + 4 * TG + 2), 1)
scaled_mm_kernel(const __grid_constant__ CUtensorMap tmap_w, const __grid_constant__ CUtensorMap tmap_a, const MmParams p) {
    using C = Cfg<TN, CG>;
    constexpr int kStages = C::kStages;
    constexpr int kAccs = C::kAccs;
    constexpr int kFirstTransformWarp = kEpilogueWarps;
    constexpr int kProducerWarp = kEpilogueWarps + 4 * TG;
    constexpr int kMmaWarp = kProducerWarp + 1;
    constexpr bool kPair = (CG == 2);

    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* const smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));

    const uint32_t smem_a = smem_base;                                   // [kStages][kAStageBytes]
    const uint32_t smem_w = smem_base + kStages * C::kAStageBytes;       // [kStages][kWStageBytes]
    const uint32_t bar_base = smem_base + kStages * C::kStageBytes;      // barrier block
    uint8_t* const bar_gen = smem_gen + kStages * C::kStageBytes;

    const uint32_t bar_wfull = bar_base;                                 // [kStages]
    const uint32_t bar_afull = bar_wfull + 8 * kMaxStages;               // [kStages]
    const uint32_t bar_sempty = bar_afull + 8 * kMaxStages;              // [kStages]
    const uint32_t bar_tfull = bar_sempty + 8 * kMaxStages;              // [kTStages]
    const uint32_t bar_tempty = bar_tfull + 8 * kTStages;                // [kTStages]
    const uint32_t bar_accfull = bar_tempty + 8 * kTStages;              // [2]
    const uint32_t bar_accempty = bar_accfull + 8 * 2;                   // [2]
    const uint32_t bar_drain = bar_accempty + 8 * 2;                     // [1]
    constexpr int kWordsOff = (3 * kMaxStages + 2 * kTStages + 2 * 2 + 1) * 8;
    volatile uint32_t* const tmem_slot = reinterpret_cast<volatile uint32_t*>(bar_gen + kWordsOff);
    volatile int* const abort_flag = reinterpret_cast<volatile int*>(bar_gen + kWordsOff + 4);
    volatile int* const last_flag = reinterpret_cast<volatile int*>(bar_gen + kWordsOff + 8);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const uint32_t rank = kPair ? cluster_ctarank() : 0u;
    const int cluster_id = blockIdx.x / CG;
    const int num_clusters = gridDim.x / CG;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) {
            mbar_init(bar_wfull + 8 * s, 1);
            mbar_init(bar_afull + 8 * s, CG);
            mbar_init(bar_sempty + 8 * s, 4 + 1);
        }
        for (int t = 0; t < kTStages; ++t) {
            mbar_init(bar_tfull + 8 * t, 4 * CG);
            mbar_init(bar_tempty + 8 * t, 1);
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(bar_accfull + 8 * a, 1);
            mbar_init(bar_accempty + 8 * a, kEpilogueWarps * CG);
        }
        mbar_init(bar_drain, 1);
        *abort_flag = 0;
        *last_flag = 0;
        fence_mbar_init();
        fence_proxy_async_smem();
    }
    if (warp == kProducerWarp && lane == 0) {
        prefetch_tmap(&tmap_w);
        prefetch_tmap(&tmap_a);
    }
    if (warp == kMmaWarp) {
        tmem_alloc<CG>(smem_u32(const_cast<uint32_t*>(tmem_slot)), C::kTmemCols);
        tmem_relinquish<CG>();
    }
    tc_fence_before();
    if constexpr (kPair) {
        cluster_arrive_release();
        cluster_wait_acquire();
    } else {
        __syncthreads();
    }
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    const uint32_t tmem_wring = tmem_base + C::kAccCols;   // column offset of the upcast-weight ring

    if (warp == kProducerWarp) {
        // ------------------------------------------------------------------ TMA producer (one lane)
        if (lane == 0) {
            uint32_t it = 0;
            bool ok = true;
            for (int u = cluster_id; ok && u < p.num_units; u += num_clusters) {
                const Unit w = decode_unit<TN, CG>(p, u);
                for (int i = 0; i < w.kb_count; ++i, ++it) {
                    const uint32_t s = it % kStages;
                    const uint32_t ph = (it / kStages) & 1u;
                    if (!mbar_wait<kPair>(bar_sempty + 8 * s, ph ^ 1u, abort_flag)) {
                        give_up<CG>(p, abort_flag, kRoleProducer, s);
                        ok = false;
                        break;
                    }
                    const int kb = w.kb_begin + i;
                    mbar_arrive_expect_tx(bar_wfull + 8 * s, kWStageBytes);
                    tma_load_3d(smem_w + s * kWStageBytes, &tmap_w, bar_wfull + 8 * s, 0, w.n0 + static_cast<int>(rank) * kBW,
                                kb * kKSteps);
                    if constexpr (!kPair) {
                        mbar_arrive_expect_tx(bar_afull + 8 * s, C::kAStageBytes);
                        tma_load_2d(smem_a + s * C::kAStageBytes, &tmap_a, bar_afull + 8 * s, kb * kBK, w.tok0);
                    } else {
                        const uint32_t leader_bar = mapa_u32(bar_afull + 8 * s, 0);
                        mbar_arrive_expect_tx_cluster(leader_bar, C::kAStageBytes);
                        tma_load_2d_pair(smem_a + s * C::kAStageBytes, &tmap_a, leader_bar, kb * kBK,
                                         w.tok0 + static_cast<int>(rank) * C::kTokLoad);
                    }
                }
            }
            if (!ok) {
                // Let this CTA's own copies land before shared memory goes away: bounded wait on the
                // weight barriers armed most recently, then a short fixed pause for the token loads.
                const uint32_t back = it < static_cast<uint32_t>(kStages) ? it : static_cast<uint32_t>(kStages);
                for (uint32_t j = 1; j <= back; ++j) {
                    const uint32_t jt = it - j;
                    const uint64_t t0 = globaltimer_ns();
                    while (!mbar_try_wait(bar_wfull + 8 * (jt % kStages), (jt / kStages) & 1u) && globaltimer_ns() - t0 < 1000000ull) {
                    }
                }
                const uint64_t t1 = globaltimer_ns();
                while (globaltimer_ns() - t1 < 20000ull) {
                }
            }
        }
    } else if (warp == kMmaWarp) {
        // ------------------------------------------------------------------ MMA issuer (leader CTA, one lane)
        if (rank == 0 && lane == 0) {
            constexpr uint32_t idesc = umma_idesc_f16(kBW * CG, TN);
            uint32_t it = 0, ui = 0;
            bool ok = true;
            for (int u = cluster_id; ok && u < p.num_units; u += num_clusters, ++ui) {
                const Unit w = decode_unit<TN, CG>(p, u);
                const uint32_t a = ui % kAccs;
                const uint32_t aph = (ui / kAccs) & 1u;
                if (!mbar_wait<kPair>(bar_accempty + 8 * a, aph ^ 1u, abort_flag)) {
                    give_up<CG>(p, abort_flag, kRoleMma, 0x100);
                    break;
                }
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + a * TN;
                for (int i = 0; i < w.kb_count; ++i, ++it) {
                    const uint32_t s = it % kStages;
                    const uint32_t ph = (it / kStages) & 1u;
                    const uint32_t t = it % kTStages;
                    const uint32_t tph = (it / kTStages) & 1u;
                    if (!mbar_wait<kPair>(bar_afull + 8 * s, ph, abort_flag)) {
                        give_up<CG>(p, abort_flag, kRoleMma, 0x200 | s);
                        ok = false;
                        break;
                    }
                    if (!mbar_wait<kPair>(bar_tfull + 8 * t, tph, abort_flag)) {
                        give_up<CG>(p, abort_flag, kRoleMma, 0x300 | t);
                        ok = false;
                        break;
                    }
                    tc_fence_after();
                    const uint32_t a_tmem = tmem_wring + t * kTColsPerStage;
                    const uint64_t b_desc = umma_desc_kmajor_sw128(smem_a + s * C::kAStageBytes);
#pragma unroll
                    for (int ks = 0; ks < kKSteps; ++ks) {
                        // +32 bytes of K inside the 128-byte swizzle row = +2 in the descriptor's address field
                        umma_f16_ts<CG>(d_tmem, a_tmem + ks * 8, b_desc + static_cast<uint64_t>(ks * 2), idesc, (i | ks) != 0 ? 1u : 0u);
                    }
                    if constexpr (!kPair) {
                        umma_commit_1cta(bar_sempty + 8 * s);
                        umma_commit_1cta(bar_tempty + 8 * t);
                    } else {
                        umma_commit_pair(bar_sempty + 8 * s, 0x3);
                        umma_commit_pair(bar_tempty + 8 * t, 0x3);
                    }
                }
                if (!ok) break;
                if constexpr (!kPair)
                    umma_commit_1cta(bar_accfull + 8 * a);
                else
                    umma_commit_pair(bar_accfull + 8 * a, 0x3);
            }
            // Nothing of this CTA pair may be torn down while an MMA is still reading it.
            umma_commit_1cta(bar_drain);
            {
                const uint64_t t0 = globaltimer_ns();
                while (!mbar_try_wait(bar_drain, 0) && globaltimer_ns() - t0 < kWaitLimitNs) {
                }
            }
        }
    } else if (warp >= kFirstTransformWarp) {
        // ------------------------------------------------------------------ e5m2 -> fp16 into TMEM
        const int q = warp & 3;
        const int g = (warp - kFirstTransformWarp) >> 2;
        const uint32_t w_lane_off = static_cast<uint32_t>(q * 32 + lane) * 16u;
        const uint32_t t_lane = static_cast<uint32_t>(q * 32) << 16;
        uint32_t it = 0;
        bool ok = true;
        for (int u = cluster_id; ok && u < p.num_units; u += num_clusters) {
            const Unit w = decode_unit<TN, CG>(p, u);
            for (int i = 0; i < w.kb_count; ++i, ++it) {
                if (static_cast<int>(it % TG) != g) continue;
                const uint32_t s = it % kStages;
                const uint32_t ph = (it / kStages) & 1u;
                const uint32_t t = it % kTStages;
                const uint32_t tph = (it / kTStages) & 1u;
                bool got = mbar_wait<false>(bar_wfull + 8 * s, ph, abort_flag);
                got = got && mbar_wait<kPair>(bar_tempty + 8 * t, tph ^ 1u, abort_flag);
                if (!__all_sync(0xffffffffu, got)) {
                    if (lane == 0) give_up<CG>(p, abort_flag, kRoleTransform, (q << 8) | s);
                    ok = false;
                    break;
                }
                tc_fence_after();
                const uint32_t src = smem_w + s * kWStageBytes + w_lane_off;
                const uint32_t dst = tmem_wring + t_lane + t * kTColsPerStage;
#pragma unroll
                for (int j = 0; j < kKSteps; ++j) {
                    uint32_t x0, x1, x2, x3;
                    asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];"
                                 : "=r"(x0), "=r"(x1), "=r"(x2), "=r"(x3)
                                 : "r"(src + j * (kBW * 16)));
                    uint32_t v[8];
                    // bytes b0..b3 of a word are k, k+1, k+2, k+3; fp16(b) = b << 8
                    v[0] = __byte_perm(x0, 0u, 0x1404);
                    v[1] = __byte_perm(x0, 0u, 0x3424);
                    v[2] = __byte_perm(x1, 0u, 0x1404);
                    v[3] = __byte_perm(x1, 0u, 0x3424);
                    v[4] = __byte_perm(x2, 0u, 0x1404);
                    v[5] = __byte_perm(x2, 0u, 0x3424);
                    v[6] = __byte_perm(x3, 0u, 0x1404);
                    v[7] = __byte_perm(x3, 0u, 0x3424);
                    tmem_st_32x32b_x8(dst + j * 8, v);
                }
                tc_wait_st();
                tc_fence_before();
                __syncwarp();
                if (lane == 0) {
                    mbar_arrive(bar_sempty + 8 * s);
                    if constexpr (!kPair)
                        mbar_arrive(bar_tfull + 8 * t);
                    else
                        mbar_arrive_cluster(mapa_u32(bar_tfull + 8 * t, 0));
                }
            }
        }
    } else {
        // ------------------------------------------------------------------ epilogue (warps 0..3)
        const int q = warp;
        const uint32_t t_lane = static_cast<uint32_t>(q * 32) << 16;
        const float scale = p.scale != nullptr ? __ldg(p.scale) : 1.0f;
        const bool out_bf16 = p.out_bf16 != 0;
        const bool has_bias = p.bias != nullptr;
        uint16_t* const c16 = reinterpret_cast<uint16_t*>(p.c);
        constexpr int kTileCols = kBW * CG;
        uint32_t ui = 0;
        // A warp whose wait ran out stays in the loop as a bystander (alive = false): it touches no
        // tensor memory but still joins the named barriers of the split-K path, so the other
        // epilogue warps can never be left waiting for it.
        bool alive = true;
        for (int u = cluster_id; u < p.num_units; u += num_clusters, ++ui) {
            if (!alive && p.splits == 1) break;
            const Unit w = decode_unit<TN, CG>(p, u);
            const uint32_t a = ui % kAccs;
            const uint32_t aph = (ui / kAccs) & 1u;
            if (alive) {
                const bool got = mbar_wait<kPair>(bar_accfull + 8 * a, aph, abort_flag);
                if (!__all_sync(0xffffffffu, got)) {
                    if (lane == 0) give_up<CG>(p, abort_flag, kRoleEpilogue, q);
                    alive = false;
                    if (p.splits == 1) break;
                }
            }
            tc_fence_after();
            const int col = static_cast<int>(rank) * kBW + q * 32 + lane;  // column inside the tile
            const int n = w.n0 + col;
            const bool n_ok = n < p.N;
            const uint16_t bias_bits = (has_bias && n_ok) ? __ldg(reinterpret_cast<const uint16_t*>(p.bias) + n) : uint16_t(0);
            const uint32_t src = tmem_base + t_lane + a * TN;
            if (p.splits == 1) {
#pragma unroll 1
                for (int c0 = 0; c0 < TN; c0 += 16) {
                    if (w.tok0 + c0 >= p.M) break;
                    uint32_t v[16];
                    tmem_ld_32x32b_x16(src + c0, v);
                    tc_wait_ld();
                    if (n_ok) {
#pragma unroll
                        for (int j = 0; j < 16; ++j) {
                            const int tok = w.tok0 + c0 + j;
                            if (tok < p.M)
                                c16[static_cast<long long>(tok) * p.ldc + n] =
                                    finish_value(__uint_as_float(v[j]), scale, out_bf16, has_bias, bias_bits);
                        }
                    }
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0) {
                    if constexpr (!kPair)
                        mbar_arrive(bar_accempty + 8 * a);
                    else
                        mbar_arrive_cluster(mapa_u32(bar_accempty + 8 * a, 0));
                }
            } else {
                // split-K: park this slice's fp32 partial, then the last slice to arrive reduces in slice order
                float* const part = p.ws_partials + (static_cast<long long>(w.tile) * p.splits + w.split) * (TN * kTileCols);
                if (alive) {
#pragma unroll 1
                    for (int c0 = 0; c0 < TN; c0 += 16) {
                        if (w.tok0 + c0 >= p.M) break;
                        uint32_t v[16];
                        tmem_ld_32x32b_x16(src + c0, v);
                        tc_wait_ld();
#pragma unroll
                        for (int j = 0; j < 16; ++j) __stcg(part + (c0 + j) * kTileCols + col, __uint_as_float(v[j]));
                    }
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) {
                        if constexpr (!kPair)
                            mbar_arrive(bar_accempty + 8 * a);
                        else
                            mbar_arrive_cluster(mapa_u32(bar_accempty + 8 * a, 0));
                    }
                }
                __threadfence();
                asm volatile("bar.sync 1, 128;" ::: "memory");
                int* const counter = p.ws_counters + w.tile * CG + static_cast<int>(rank);
                if (threadIdx.x == 0) {
                    const int old = atomicAdd(counter, 1);
                    *last_flag = (old == p.splits - 1) ? 1 : 0;
                }
                asm volatile("bar.sync 1, 128;" ::: "memory");
                const bool is_last = *last_flag != 0;
                if (is_last) {
                    __threadfence();
                    const float* const tile_part = p.ws_partials + static_cast<long long>(w.tile) * p.splits * (TN * kTileCols);
                    if (n_ok && alive) {
#pragma unroll 1
                        for (int c = 0; c < TN; ++c) {
                            const int tok = w.tok0 + c;
                            if (tok >= p.M) break;
                            float acc = 0.0f;
                            for (int sp = 0; sp < p.splits; ++sp)
                                acc += __ldcg(tile_part + static_cast<long long>(sp) * (TN * kTileCols) + c * kTileCols + col);
                            c16[static_cast<long long>(tok) * p.ldc + n] = finish_value(acc, scale, out_bf16, has_bias, bias_bits);
                        }
                    }
                }
                asm volatile("bar.sync 1, 128;" ::: "memory");   // everyone has read last_flag / the partials
                if (is_last && threadIdx.x == 0) *counter = 0;    // ready for the next launch
            }
        }
    }

    // ---------------------------------------------------------------------- teardown
    tc_fence_before();
    if constexpr (kPair) {
        cluster_arrive_release();
        cluster_wait_acquire();
    } else {
        __syncthreads();
    }
    if (warp == kMmaWarp) {
        tc_fence_after();
        tmem_dealloc<CG>(tmem_base, C::kTmemCols);
    }
}

// ================================================================================================
// Host side
// ================================================================================================

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_tiled_fn() {
    static EncodeTiledFn fn = [] {
        void* f = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPointByVersion("cuTensorMapEncodeTiled", &f, 12000, cudaEnableDefault, &q) != cudaSuccess ||
            q != cudaDriverEntryPointSuccess)
            f = nullptr;
        return reinterpret_cast<EncodeTiledFn>(f);
    }();
    return fn;
}

static int sm_count_of_current_device() {
    static std::mutex mu;
    static int cached[64];
    static bool have[64];
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 0;
    std::lock_guard<std::mutex> lock(mu);
    if (!have[dev]) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return 0;
        cached[dev] = n;
        have[dev] = true;
    }
    return cached[dev];
}

struct Plan {
    int tn, cg, tg, splits, max_ctas;
    int tiles_n, tiles_t, total_kb, num_units;
    size_t ws_bytes, counter_bytes;
};

static bool valid_tn(int tn) { return tn == 16 || tn == 32 || tn == 64 || tn == 128 || tn == 256; }

// Shape heuristic.  Stands in for the reference's per-shape autotune over 28 tile configs
// (kernel/hip/utils.py:192-223): here the tile is fixed by the token count and the machine is filled by
// splitting K when the weight tiles alone cannot.
static bool make_plan(int64_t M, int64_t N, int64_t K, const feather_mm_variant* v, size_t ws_avail, bool ws_known, int sms, Plan* out) {
    Plan pl{};
    pl.total_kb = static_cast<int>((K + kBK - 1) / kBK);
    int tn = v ? v->tokens_tile : 0;
    if (tn == 0) tn = M <= 16 ? 16 : M <= 32 ? 32 : M <= 64 ? 64 : M <= 128 ? 128 : 256;
    if (!valid_tn(tn)) return false;
    int cg = v ? v->cta_pair : 0;
    if (cg == 0) cg = 1;
    if (cg != 1 && cg != 2) return false;
    if (cg == 2 && tn < 32) return false;   // each CTA of a pair loads tn/2 token rows, at least one 8-row swizzle group x2
    pl.tn = tn;
    pl.cg = cg;
    pl.tg = v ? v->transform_groups : 0;
    if (pl.tg == 0) pl.tg = 2;
    if (pl.tg != 1 && pl.tg != 2) return false;
    pl.tiles_n = static_cast<int>((N + kBW * cg - 1) / (kBW * cg));
    pl.tiles_t = static_cast<int>((M + tn - 1) / tn);
    const long long tiles = static_cast<long long>(pl.tiles_n) * pl.tiles_t;
    if (tiles <= 0 || tiles > 0x3FFFFFFF) return false;
    const int clusters = (sms > 0 ? sms : 148) / cg;
    int splits = v ? v->split_k : 0;
    if (splits == 0) {
        splits = 1;
        if (tiles < clusters && pl.total_kb >= 16) {
            // aim at >= 2 work units per cluster, keep at least 8 k-blocks (512 k) per slice
            int want = static_cast<int>((2LL * clusters + tiles - 1) / tiles);
            int cap = pl.total_kb / 8;
            splits = want < cap ? want : cap;
            if (splits < 1) splits = 1;
        }
        const size_t per_split = static_cast<size_t>(tiles) * tn * kBW * cg * sizeof(float);
        const size_t counters = ((static_cast<size_t>(tiles) * cg * sizeof(int) + 255) / 256) * 256;
        if (ws_known && splits > 1 && counters + per_split * splits > ws_avail) {
            // shrink to what the caller's scratch can hold
            size_t fit = ws_avail > counters ? (ws_avail - counters) / per_split : 0;
            splits = fit >= 2 ? static_cast<int>(fit) : 1;
        }
    }
    if (splits < 1 || splits > pl.total_kb) return false;
    pl.splits = splits;
    pl.num_units = static_cast<int>(tiles) * splits;
    pl.counter_bytes = splits > 1 ? ((static_cast<size_t>(tiles) * cg * sizeof(int) + 255) / 256) * 256 : 0;
    pl.ws_bytes = splits > 1 ? pl.counter_bytes + static_cast<size_t>(tiles) * splits * tn * kBW * cg * sizeof(float) : 0;
    pl.max_ctas = v ? v->max_ctas : 0;
    *out = pl;
    return true;
}

template <int TN, int CG, int TG>
static cudaError_t launch_variant(const CUtensorMap& tw, const CUtensorMap& ta, const MmParams& p, int grid, cudaStream_t stream) {
    using C = Cfg<TN, CG>;
    auto kernel = scaled_mm_kernel<TN, CG, TG>;
    static std::mutex mu;
    static bool configured[64];
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    {
        std::lock_guard<std::mutex> lock(mu);
        if (dev >= 0 && dev < 64 && !configured[dev]) {
            e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, C::kSmemBytes);
            if (e != cudaSuccess) return e;
            configured[dev] = true;
        }
    }
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(static_cast<unsigned>(grid), 1, 1);
    cfg.blockDim = dim3(32 * (kEpilogueWarps + 4 * TG + 2), 1, 1);
    cfg.dynamicSmemBytes = C::kSmemBytes;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = CG;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, tw, ta, p);
}

template <int TN>
static cudaError_t launch_tn(int cg, int tg, const CUtensorMap& tw, const CUtensorMap& ta, const MmParams& p, int grid, cudaStream_t s) {
    if (cg == 1) return tg == 1 ? launch_variant<TN, 1, 1>(tw, ta, p, grid, s) : launch_variant<TN, 1, 2>(tw, ta, p, grid, s);
    if constexpr (TN >= 32)
        return tg == 1 ? launch_variant<TN, 2, 1>(tw, ta, p, grid, s) : launch_variant<TN, 2, 2>(tw, ta, p, grid, s);
    return cudaErrorInvalidValue;
}

static int scaled_mm_impl(const void* a, const uint8_t* b, const float* scale, const void* bias, void* c, int64_t M, int64_t N,
                          int64_t K, int64_t ldc, int output_dtype, const feather_mm_variant* variant, void* workspace,
                          size_t workspace_bytes, int* status_dev, cudaStream_t stream) {
    if (a == nullptr || b == nullptr || c == nullptr) return set_error(FEATHER_ERR_BAD_ARGUMENT, "a, b_prepacked and c must not be null");
    if (M < 0 || N <= 0 || K <= 0) return set_error(FEATHER_ERR_BAD_ARGUMENT, "M, N, K must be positive");
    if (K % 16 != 0) return set_error(FEATHER_ERR_BAD_ARGUMENT, "K must be divisible by 16");
    if (ldc < N) return set_error(FEATHER_ERR_BAD_ARGUMENT, "ldc must be at least N");
    if (M > 0x7FFFFFFF || N > 0x7FFFFFFF || K > 0x7FFFFFFF) return set_error(FEATHER_ERR_BAD_ARGUMENT, "M, N, K must fit in 31 bits");
    if (output_dtype != FEATHER_OUT_FP16 && output_dtype != FEATHER_OUT_BF16)
        return set_error(FEATHER_ERR_BAD_ARGUMENT, "output_dtype must be 0 (fp16) or 1 (bf16)");
    if ((reinterpret_cast<uintptr_t>(a) & 15u) != 0) return set_error(FEATHER_ERR_BAD_ARGUMENT, "a data pointer must be 16-byte aligned");
    if ((reinterpret_cast<uintptr_t>(b) & 15u) != 0)
        return set_error(FEATHER_ERR_BAD_ARGUMENT, "b_prepacked data pointer must be 16-byte aligned");
    if ((reinterpret_cast<uintptr_t>(c) & 1u) != 0) return set_error(FEATHER_ERR_BAD_ARGUMENT, "c data pointer must be 2-byte aligned");
    if (M == 0) return FEATHER_OK;

    const int sms = sm_count_of_current_device();
    if (sms <= 0) return set_error(FEATHER_ERR_NO_DEVICE, "no CUDA device");
    Plan pl;
    if (!make_plan(M, N, K, variant, workspace ? workspace_bytes : 0, true, sms, &pl))
        return set_error(FEATHER_ERR_UNSUPPORTED, "unsupported kernel variant");
    if (pl.splits > 1) {
        if (workspace == nullptr || workspace_bytes < pl.ws_bytes)
            return set_error(FEATHER_ERR_WORKSPACE, "split-K variant needs a larger workspace");
        if ((reinterpret_cast<uintptr_t>(workspace) & 15u) != 0) return set_error(FEATHER_ERR_BAD_ARGUMENT, "workspace must be 16-byte aligned");
    }
    const int tg = pl.tg;

    EncodeTiledFn encode = encode_tiled_fn();
    if (encode == nullptr) return set_error(FEATHER_ERR_NO_DEVICE, "cuTensorMapEncodeTiled is not available from the driver");

    CUtensorMap tmap_w, tmap_a;
    {
        // W bytes as a rank-3 tensor (16, N, K/16); a box is 4 k16-blocks x 128 n x 16 B, laid down verbatim.
        const cuuint64_t dims[3] = {16, static_cast<cuuint64_t>(N), static_cast<cuuint64_t>(K / 16)};
        const cuuint64_t strides[2] = {16, static_cast<cuuint64_t>(N) * 16};
        const cuuint32_t box[3] = {16, kBW, kKSteps};
        const cuuint32_t estr[3] = {1, 1, 1};
        const CUresult r = encode(&tmap_w, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, const_cast<uint8_t*>(b), dims, strides, box, estr,
                                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) return set_error(FEATHER_ERR_CUDA, "cuTensorMapEncodeTiled(W) failed with CUresult %d", static_cast<int>(r));
    }
    {
        // A as (K, M) fp16; a box is 64 k x (tokens per CTA), 128-byte swizzle, rows beyond M read as zero.
        const cuuint64_t dims[2] = {static_cast<cuuint64_t>(K), static_cast<cuuint64_t>(M)};
        const cuuint64_t strides[1] = {static_cast<cuuint64_t>(K) * 2};
        const cuuint32_t box[2] = {kBK, static_cast<cuuint32_t>(pl.tn / pl.cg)};
        const cuuint32_t estr[2] = {1, 1};
        const CUresult r = encode(&tmap_a, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void*>(a), dims, strides, box, estr,
                                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) return set_error(FEATHER_ERR_CUDA, "cuTensorMapEncodeTiled(A) failed with CUresult %d", static_cast<int>(r));
    }

    MmParams p{};
    p.scale = scale;
    p.bias = bias;
    p.c = c;
    p.ws_counters = pl.splits > 1 ? reinterpret_cast<int*>(workspace) : nullptr;
    p.ws_partials = pl.splits > 1 ? reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(workspace) + pl.counter_bytes) : nullptr;
    p.status = status_dev;
    p.M = static_cast<int>(M);
    p.N = static_cast<int>(N);
    p.K = static_cast<int>(K);
    p.ldc = ldc;
    p.out_bf16 = output_dtype == FEATHER_OUT_BF16 ? 1 : 0;
    p.splits = pl.splits;
    p.tiles_n = pl.tiles_n;
    p.tiles_t = pl.tiles_t;
    p.num_units = pl.num_units;
    p.total_kb = pl.total_kb;

    int clusters = sms / pl.cg;
    if (pl.max_ctas > 0 && pl.max_ctas / pl.cg < clusters) clusters = pl.max_ctas / pl.cg;
    if (clusters < 1) clusters = 1;
    if (clusters > pl.num_units) clusters = pl.num_units;
    const int grid = clusters * pl.cg;

    cudaError_t e = cudaErrorInvalidValue;
    switch (pl.tn) {
        case 16: e = launch_tn<16>(pl.cg, tg, tmap_w, tmap_a, p, grid, stream); break;
        case 32: e = launch_tn<32>(pl.cg, tg, tmap_w, tmap_a, p, grid, stream); break;
        case 64: e = launch_tn<64>(pl.cg, tg, tmap_w, tmap_a, p, grid, stream); break;
        case 128: e = launch_tn<128>(pl.cg, tg, tmap_w, tmap_a, p, grid, stream); break;
        case 256: e = launch_tn<256>(pl.cg, tg, tmap_w, tmap_a, p, grid, stream); break;
        default: break;
    }
    if (e != cudaSuccess) return set_error(FEATHER_ERR_CUDA, "scaled_mm launch failed: %s", cudaGetErrorString(e));
    return FEATHER_OK;
}

}  // namespace feather

using namespace feather;

extern "C" int feather_scaled_mm_ex(const void* a, const uint8_t* b_prepacked, const float* scale, const void* bias, void* c,
                                    int64_t M, int64_t N, int64_t K, int64_t ldc, int output_dtype,
                                    const feather_mm_variant* variant, void* workspace, size_t workspace_bytes, int* status_dev,
                                    feather_stream_t stream) {
    return scaled_mm_impl(a, b_prepacked, scale, bias, c, M, N, K, ldc, output_dtype, variant, workspace, workspace_bytes, status_dev,
                          static_cast<cudaStream_t>(stream));
}

extern "C" int launch_scaled_mm(const void* a, const uint8_t* b_prepacked, const float* scale, const uint16_t* bias, uint16_t* c,
                                int64_t M, int64_t N, int64_t K, int has_scale, int has_bias, int, int, int, int, int, int b_dtype,
                                int output_dtype, feather_stream_t stream) {
    if (b_dtype != FEATHER_B_E5M2) {
        set_error(FEATHER_ERR_UNSUPPORTED, "only fp8e5m2 weights (b_dtype = 1) are supported");
        return 0;
    }
    feather_mm_variant v{};
    v.split_k = 1;   // no workspace through this signature
    const int st = scaled_mm_impl(a, b_prepacked, has_scale ? scale : nullptr, has_bias ? bias : nullptr, c, M, N, K, N, output_dtype, &v,
                                  nullptr, 0, nullptr, static_cast<cudaStream_t>(stream));
    return st == FEATHER_OK ? 1 : 0;
}

extern "C" size_t feather_scaled_mm_workspace_bytes(int64_t M, int64_t N, int64_t K, const feather_mm_variant* variant) {
    if (M <= 0 || N <= 0 || K <= 0) return 0;
    int sms = sm_count_of_current_device();
    Plan pl;
    if (!make_plan(M, N, K, variant, 0, false, sms, &pl)) return 0;
    return pl.ws_bytes;
}

extern "C" int feather_scaled_mm_choose(int64_t M, int64_t N, int64_t K, size_t workspace_bytes, feather_mm_variant* out) {
    if (out == nullptr || M <= 0 || N <= 0 || K <= 0) return set_error(FEATHER_ERR_BAD_ARGUMENT, "bad arguments");
    int sms = sm_count_of_current_device();
    Plan pl;
    if (!make_plan(M, N, K, nullptr, workspace_bytes, true, sms, &pl)) return set_error(FEATHER_ERR_UNSUPPORTED, "no variant");
    out->tokens_tile = pl.tn;
    out->cta_pair = pl.cg;
    out->split_k = pl.splits;
    out->transform_groups = pl.tg;
    out->max_ctas = 0;
    return FEATHER_OK;
}
