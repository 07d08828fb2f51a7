// fp16 activations @ prepacked fp8e5m2 weights -> fp16/bf16, fp32 accumulate, for sm_100a.
//
// Stands in for the reference's scaled_mm_kernel / launch_scaled_mm (kernel/hip/hip_kernel.cu:125-632).
// The design is not the reference's: the weight tile is the MMA "A" operand and lives in tensor memory.
//
//   out^T tile [128 weight columns n  x  TN tokens]  +=  up(W)[128 n x 16 k]  *  A^T[16 k x TN tokens]
//
//   producer warps  TMA: W bytes  [8 k16-blocks][128 n][16 B] (the prepacked layout, verbatim; 2 KB rows) -> smem ring
//                   TMA: A tokens 2 x [TN rows][64 k] fp16, 128-byte swizzle (one 3-D copy per k-block) -> operand ring
//   transform warps ld.shared 16 B (one n, 16 k) -> 8 x prmt (e5m2 -> fp16 is `byte << 8`, exact)
//                   -> tcgen05.st into the operand ring's TMEM half (64 columns per 128-k slot); fp16 W never touches smem
//   MMA warp(s)     tcgen05.mma kind::f16, A from TMEM, B (tokens) from smem descriptor, D fp32 in TMEM; tiles of at most
//                   128 tokens have two issuing threads (even / odd k-blocks, one accumulator each)
//   epilogue warps  tcgen05.ld (MMA fragment shape) -> *scale -> RTNE to out dtype -> +bias in out dtype -> stmatrix into a
//                   swizzled staging tile -> TMA store; split-K slices park fp32 partials in a workspace and the last
//                   slice to arrive reduces them in slice order.
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
#include <stdlib.h>
#include <string.h>

#include <mutex>
#include <type_traits>

#include "../../include/feather_b200.h"
#include "host_util.h"
#include "ptx.cuh"

namespace feather {

constexpr int kBW = 128;                      // weight columns per CTA = MMA M per CTA = TMEM lanes
constexpr int kBK = 128;                      // k per pipeline stage (one barrier round: 8 MMAs amortise the waits and commits)
constexpr int kSubK = 64;                     // k per 128-byte-swizzled token sub-tile (64 fp16 = one 128-byte row)
constexpr int kSubTiles = kBK / kSubK;        // token sub-tiles per stage
constexpr int kKSteps = kBK / 16;             // MMA k-steps per stage
constexpr int kWStageBytes = kBW * kBK;       // e5m2 bytes per stage
constexpr int kMaxTStages = 8;                // TMEM ring depth for upcast weights (upper bound)
constexpr int kTColsPerStage = kBK / 2;       // 32-bit TMEM columns per stage (two fp16 per column)
constexpr int kEpilogueWarps = 8;              // two groups of four (one warp per TMEM lane quarter in each)
constexpr int kMaxStages = 16;
// Split-K workspace: a fixed-size block of tile counters first (so the counters of any launch only ever overlap the counters of
// another, which every launch leaves at zero), then the fp32 partial tiles.
constexpr size_t kCounterBytes = 65536;
#ifndef FEATHER_STATIC_SCRATCH_BYTES
#define FEATHER_STATIC_SCRATCH_BYTES (8u << 20)
#endif

__host__ __device__ constexpr int pow2_at_least(int x) {
    int p = 32;
    while (p < x) p <<= 1;
    return p;
}

// OB: staging buffers per epilogue group.  1 for an ordinary launch; 2 when the blocks also go to peer GPUs, so that a block
// can be staged while NVLink is still taking the previous one.
template <int TN, int CG, int OB = 1>
struct Cfg {
    static_assert(TN == 16 || TN == 32 || TN == 64 || TN == 128 || TN == 192 || TN == 256, "tokens tile");
    static_assert(CG == 1 || CG == 2, "cta group");
    static constexpr int kTokLoad = TN / CG;              // token rows this CTA loads per stage
    static constexpr int kASubBytes = kTokLoad * 128;     // one sub-tile: 64 fp16 per row
    static constexpr int kAStageBytes = kASubBytes * kSubTiles;
    // One thread can issue a tcgen05.mma about every 55-70 cycles, whatever its size, so for tiles of at most 128 tokens
    // (64 cycles of tensor pipe per MMA) a single issuer is the bottleneck.  Those tiles use two issuing threads in two
    // warps: even k-blocks of a tile go to issuer 0, odd ones to issuer 1, each with an accumulator of its own (the
    // partial sums are added in the epilogue, always in the same order, so results stay reproducible).
    static constexpr int kIssuers = (TN <= 128) ? 2 : 1;
    // Tile buffers in TMEM: with two, the epilogue of one tile overlaps the MMAs of the next.  Narrow tiles are chosen when a CTA
    // has one tile anyway, and there the columns serve better as operand-ring slots (64 tokens: 6 slots instead of 4, 5 % faster).
    static constexpr int kAccs = (TN == 192) ? 2 : 1;
    static constexpr int kAccCols = kAccs * kIssuers * TN;
    static_assert(kAccCols <= 384, "accumulator columns");
    static constexpr int kTStagesRaw = (512 - kAccCols) / kTColsPerStage;
    static constexpr int kTStages = kTStagesRaw > kMaxTStages ? kMaxTStages : kTStagesRaw;   // TMEM ring depth
    static constexpr int kTmemCols = pow2_at_least(kAccCols + kTStages * kTColsPerStage);   // the ring may use fewer (kAStages) slots
    static constexpr int kBarrierBytes = 1024;
    static constexpr int kOutRows = TN < 32 ? TN : 32;                   // token rows per output staging buffer
    static constexpr int kOutBufBytes = kOutRows * kBW * 2;              // [2 tiles][rows][64 n] 16-bit
    // Staging buffers per epilogue group.  The memory comes out of the weight-byte ring, and that ring's depth matters more
    // than it looks: on one GPU the Wan ffn shapes ran at 1507 / 1540 TFLOP/s with five weight stages (one buffer), 1412 / 1370
    // with four (two buffers), and 912 / 762 with two (four buffers, a whole tile).  So an ordinary launch stages through one
    // buffer.  With peer destinations a tile's blocks leave at NVLink speed, and two buffers measured best (2 GPUs: 2754
    // TFLOP/s against 2699 with one and 1966 with four).
    static_assert(OB == 1 || (OB == 2 && TN == 256), "staging ring depth");
    static constexpr int kOutBufs = OB;
    static constexpr int kOutBytes = 2 * kOutBufs * kOutBufBytes;
    static constexpr int kSmemBudget = 227 * 1024 - 1024 /*alignment slack*/ - kBarrierBytes - kOutBytes;
    // One operand ring for the MMA warp: slot i holds a token tile in shared memory and the matching upcast weights in
    // tensor memory, so the single issuing thread waits on one barrier and commits to one barrier per k-block (its
    // instruction count per k-block bounds the speed of every tile narrower than 256 tokens).  The raw weight bytes have a
    // ring of their own (freed as soon as the transform warps have read them) that takes the rest of shared memory.
    static constexpr int kAStagesRaw = (kSmemBudget - 2 * kWStageBytes) / kAStageBytes;
    static constexpr int kAStages = kAStagesRaw > kTStages ? kTStages : kAStagesRaw;
    static constexpr int kWStagesRaw = (kSmemBudget - kAStages * kAStageBytes) / kWStageBytes;
    static constexpr int kWStages = kWStagesRaw > kMaxStages ? kMaxStages : kWStagesRaw;
    static constexpr int kSmemBytes = kAStages * kAStageBytes + kWStages * kWStageBytes + kOutBytes + kBarrierBytes + 1024;
    static_assert(kAStages >= 2 && kWStages >= 2, "ring depth");
    static_assert(kTmemCols <= 512, "TMEM columns");
    static_assert(kASubBytes % 1024 == 0, "swizzle atom alignment of token sub-tiles");
    static_assert((4 * kMaxStages + 2 * kMaxTStages + 2 * 2 + 1) * 8 + 16 <= kBarrierBytes, "barrier block");
};

struct MmParams {
    const float* scale;
    const void* bias;
    void* c;
    float* ws_partials;
    int* ws_counters;
    int* status;
    long long* stats;   // optional [32] cycle counters written by CTA 0 (profiling aid), or null
    int M, N, K;
    long long ldc;
    int out_bf16;  // dtype the scaled sum is rounded to and the bias is added in
    int flip_final;  // 1: the value is then cast once more, to the other 16-bit dtype, and stored as that (the caller's `y.to(dtype)`)
    int a_bf16;    // 1: the activations are bf16 (the weights are upcast to bf16 too, and the MMA runs bf16 x bf16)
    int w_e4m3;    // 1: the weight bytes are fp8e4m3fn; they are upcast to 1/256 of their value and scale_mul puts the factor back
    float scale_mul;
    // Un-merged LoRA folded into the accumulator: after the weight's k-blocks every tile runs lora_blocks more blocks of 64
    // "k" each, whose token operand is T' [M, R] (the down-projected activations) and whose weight operand is B' [R/8, N, 8],
    // both fp16 whatever the activations' dtype (the format is a field of each MMA instruction; no upcast), scaled so that
    // T' B'^T = (x A^T) B^T * strength / scale.
    int lora_blocks;
    int a3d;       // 1: the token tensor map is the 3-D form (64 k, M, K/64): one copy per k-block
    int c3d;       // 1: the output tensor maps are the 3-D form (64 n, M, N/64): one store per staged block and destination
    int tma_store; // 1: output rows are 16-byte aligned, the epilogue stores tiles with TMA; 0: plain 2-byte stores
    int n_dst;     // number of output buffers every tile is stored to (1, or one per GPU of a column-sharded linear)
    int scatter_rows;  // 0: every block goes to all n_dst buffers; > 0: buffer d owns the token rows [d * scatter_rows, (d + 1) * scatter_rows)
    int splits;
    int tiles_n, tiles_t, num_units, total_kb;
};

constexpr int kMaxDst = 8;
// One tensor map per destination of the output.  Destination 0 is the caller's own buffer; the others are the same
// [M, ldc] buffer in the memory of peer GPUs (NVLink), so a column shard lands in every rank's full output without a
// separate all-gather.  Stores only: no load ever reads peer memory here.
struct OutMaps {
    CUtensorMap m[kMaxDst];
};
// Tensor maps of the low-rank term: t = T' as (R, M) 16-bit with a (64, tokens per CTA) box in the 128-byte swizzle (one token
// sub-tile); b = B' as 8-byte elements (2N, R/8) with the weight map's (256, 8) box, which lands as [8][128 n][16 B] = one
// weight stage holding 64 ranks of 16-bit values.
struct LoraMaps {
    CUtensorMap t, b;
};

struct Unit {
    int tile, split, n0, tok0, kb_begin, kb_count;
    int kb_total;   // kb_count plus the low-rank blocks that follow the weight's k-blocks (0 without a LoRA term)
};

template <int TN, int CG>
__device__ __forceinline__ Unit decode_unit(const MmParams& p, int u) {
    Unit w;
    w.tile = u / p.splits;
    w.split = u - w.tile * p.splits;
    // Tiles are walked in bands of kBand token tiles, token tile fastest inside a band, so the CTAs that run at the same time
    // share a few token tiles and a few weight tiles (L2 locality) instead of one token tile and every weight tile.
    constexpr int kBand = 8;
    const int band_tiles = kBand * p.tiles_n;
    const int band = w.tile / band_tiles;
    const int in_band = w.tile - band * band_tiles;
    const int rows = p.tiles_t - band * kBand < kBand ? p.tiles_t - band * kBand : kBand;
    const int nt = in_band / rows;
    const int tt = band * kBand + in_band % rows;
    w.n0 = nt * kBW * CG;
    w.tok0 = tt * TN;
    const int base = p.total_kb / p.splits;
    const int rem = p.total_kb - base * p.splits;
    w.kb_begin = w.split * base + (w.split < rem ? w.split : rem);
    w.kb_count = base + (w.split < rem ? 1 : 0);
    w.kb_total = w.kb_count + p.lora_blocks;
    return w;
}

// Optional cycle accounting (MmParams::stats): each role of CTA 0 sums the SM cycles it spends in each of its waits.
// slots: 0 token producer total, 1 its wait for a free stage, 2/3 the same for the weight producer | 4 mma total, 5 mma wait acc-free, 6 mma wait tokens, 7 mma wait weights
//        8 transform(warp 0 of group 0) total, 9 wait weight bytes, 10 wait tmem-free | 12 epilogue(warp 0) total, 13 wait acc-full,
//        14 inside store chunks, 15 chunks
struct StatTimer {
    long long t0;
    bool on;
    __device__ __forceinline__ explicit StatTimer(bool enabled) : t0(0), on(enabled) {}
    __device__ __forceinline__ void start() {
        if (on) t0 = clock64();
    }
    __device__ __forceinline__ void stop(long long& acc) {
        if (on) acc += clock64() - t0;
    }
};

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

// flip: after rounding to the output dtype and adding the bias in it, cast once more to the other 16-bit dtype (what
// `y.to(dtype)` does after the reference's op, comfy_feather/ops.py:103) and return those bits.
__device__ __forceinline__ uint16_t finish_value(float acc, float scale, bool out_bf16, bool has_bias, uint16_t bias_bits, bool flip = false) {
    const float r = acc * scale;
    if (out_bf16) {
        __nv_bfloat16 v = __float2bfloat16_rn(r);
        if (has_bias) v = __float2bfloat16_rn(__bfloat162float(v) + __bfloat162float(__ushort_as_bfloat16(bias_bits)));
        if (flip) return __half_as_ushort(__float2half_rn(__bfloat162float(v)));
        return __bfloat16_as_ushort(v);
    }
    __half v = __float2half_rn(r);
    if (has_bias) v = __hadd(v, __ushort_as_half(bias_bits));
    if (flip) return __bfloat16_as_ushort(__float2bfloat16_rn(__half2float(v)));
    return __half_as_ushort(v);
}

// One word of weight bytes as two fp16-positioned halves h = [b_hi : 0 : b_lo : 0] (what `byte << 8` gives) -> the two MMA
// operand values.  mode bit 0: activations are bf16, so the operand must be bf16 too; bit 1: the bytes are e4m3fn.
//   e5m2 -> fp16   h itself (exact: e5m2 is the high byte of an fp16)
//   e4m3 -> fp16   sign | (b & 0x7F) << 7 is the value / 256 (exponent bias 7 read as 15; subnormals line up too), which the
//                  epilogue undoes through scale_mul; the two NaN codes 0x7F / 0xFF are mapped to an fp16 NaN
//   ... -> bf16    through fp32 (every fp16 value above is a bf16 value: at most 3 mantissa bits, exponent in range)
__device__ __forceinline__ uint32_t upcast_pair(uint32_t h, int mode) {
    if (mode & 2) {
        const uint32_t mag = h & 0x7F007F00u;
        uint32_t t = ((h >> 1) & 0x3F803F80u) | (h & 0x80008000u);
        t |= __vcmpeq2(mag, 0x7F007F00u) & 0x7E007E00u;
        h = t;
    }
    if (mode & 1) {
        const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&h));
        const __nv_bfloat162 b = __floats2bfloat162_rn(f.x, f.y);
        h = *reinterpret_cast<const uint32_t*>(&b);
    }
    return h;
}

// Two accumulator values of one output column (tokens j and j+1) -> packed out-dtype pair {lo = token j, hi = token j+1}:
// fp32 multiply by the scale, one packed round-to-nearest-even conversion, then the bias add in the output dtype.
__device__ __forceinline__ uint32_t finish_pair(float acc0, float acc1, float scale, bool out_bf16, bool has_bias, uint32_t bias2) {
    const float r0 = acc0 * scale, r1 = acc1 * scale;
    if (out_bf16) {
        __nv_bfloat162 v = __floats2bfloat162_rn(r0, r1);
        if (has_bias) v = __hadd2(v, *reinterpret_cast<const __nv_bfloat162*>(&bias2));
        return *reinterpret_cast<const uint32_t*>(&v);
    }
    __half2 v = __floats2half2_rn(r0, r1);
    if (has_bias) v = __hadd2(v, *reinterpret_cast<const __half2*>(&bias2));
    return *reinterpret_cast<const uint32_t*>(&v);
}

// EXT = false is the plain linear (fp16 activations, e5m2 weights, every block stored to all destinations); EXT = true adds, as
// run-time switches, bf16 activations, e4m3 weights, the low-rank (LoRA) blocks and row-sharded destinations.  The split keeps
// the single-thread loops of the plain kernel free of those branches: with them in, the Wan shapes ran 2-4 % slower.
template <int TN, int CG, int TG, int OB = 1, bool EXT = false>
__global__ void __launch_bounds__(32 * (kEpilogueWarps + 4 * TG + 2 + Cfg<TN, CG>::kIssuers), 1)
scaled_mm_kernel(const __grid_constant__ CUtensorMap tmap_w, const __grid_constant__ CUtensorMap tmap_a,
                 const __grid_constant__ OutMaps tmap_c, const __grid_constant__ LoraMaps tmap_l, const MmParams p) {
    using C = Cfg<TN, CG, OB>;
    constexpr int kStages = C::kAStages;                                  // operand ring depth (token tile + upcast weights per slot)
    constexpr int kWStages = C::kWStages;
    constexpr int kAccs = C::kAccs;
    constexpr int kFirstTransformWarp = kEpilogueWarps;
    constexpr int kProducerWarp = kEpilogueWarps + 4 * TG;
    constexpr int kMmaWarp = kProducerWarp + 1;
    constexpr int kWProducerWarp = kProducerWarp + 2;
    constexpr int kIssuers = C::kIssuers;
    constexpr int kMma2Warp = kProducerWarp + 3;                          // second issuer (exists only when kIssuers == 2)
    constexpr bool kPair = (CG == 2);

    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* const smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));

    const uint32_t smem_a = smem_base;                                   // [kStages][kAStageBytes]
    const uint32_t smem_w = smem_base + kStages * C::kAStageBytes;       // [kWStages][kWStageBytes]
    constexpr int kRingBytes = kStages * C::kAStageBytes + kWStages * kWStageBytes;
    const uint32_t smem_out = smem_base + kRingBytes;                    // [2][kOutRows][128] 16-bit output staging
    const uint32_t bar_base = smem_out + C::kOutBytes;                   // barrier block
    uint8_t* const bar_gen = smem_gen + kRingBytes + C::kOutBytes;

    const uint32_t bar_wfull = bar_base;                                 // [kWStages] weight bytes landed
    const uint32_t bar_wempty = bar_wfull + 8 * kMaxStages;              // [kWStages] weight bytes read by the 4 transform warps
    const uint32_t bar_full = bar_wempty + 8 * kMaxStages;               // [kStages] token tile landed (both CTAs of a pair) and weights upcast
    const uint32_t bar_empty = bar_full + 8 * kMaxStages;                // [kStages] slot no longer read by any MMA
    const uint32_t bar_accfull = bar_empty + 8 * kMaxStages;             // [2]
    const uint32_t bar_accempty = bar_accfull + 8 * 2;                   // [2]
    const uint32_t bar_drain = bar_accempty + 8 * 2;                     // [2] one per issuer
    constexpr int kWordsOff = (4 * kMaxStages + 2 * kMaxTStages + 2 * 2 + 1) * 8;
    volatile uint32_t* const tmem_slot = reinterpret_cast<volatile uint32_t*>(bar_gen + kWordsOff);
    volatile int* const abort_flag = reinterpret_cast<volatile int*>(bar_gen + kWordsOff + 4);
    volatile int* const last_flag = reinterpret_cast<volatile int*>(bar_gen + kWordsOff + 8);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const uint32_t rank = kPair ? cluster_ctarank() : 0u;
    const int cluster_id = blockIdx.x / CG;
    const int num_clusters = gridDim.x / CG;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kWStages; ++s) {
            mbar_init(bar_wfull + 8 * s, 1);
            mbar_init(bar_wempty + 8 * s, 4);
        }
        for (int s = 0; s < kStages; ++s) {
            mbar_init(bar_full + 8 * s, CG + 4 * CG);                    // token producer(s) + the four warps of one transform group per CTA
            mbar_init(bar_empty + 8 * s, 1);
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(bar_accfull + 8 * a, kIssuers);
            mbar_init(bar_accempty + 8 * a, kEpilogueWarps * CG);
        }
        mbar_init(bar_drain, 1);
        mbar_init(bar_drain + 8, 1);
        *abort_flag = 0;
        *last_flag = 0;
        fence_mbar_init();
        fence_proxy_async_smem();
    }
    if (warp == kProducerWarp && lane == 0) {
        prefetch_tmap(&tmap_a);
        if (p.tma_store)
            for (int d = 0; d < p.n_dst; ++d) prefetch_tmap(&tmap_c.m[d]);
    }
    if (warp == kWProducerWarp && lane == 0) prefetch_tmap(&tmap_w);
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
    // Everything above (barriers, tensor memory, tensor-map prefetch) touched no global memory and may have run while the
    // previous kernel on the stream was still draining (programmatic dependent launch); from here on its results are needed.
    pdl_launch_dependents();
    pdl_wait_for_previous_kernel();

    if (warp == kProducerWarp || warp == kWProducerWarp) {
        // ------------------------------------------------------------------ TMA producers (one lane each): token tiles / weight bytes
        // One copy instruction per ring slot, issued by lane 0.  The loop itself is run by the whole warp in lockstep, which
        // measured about a quarter less time per k-block than a loop run by lane 0 alone.  Ring slot and parity are running
        // values (no division) and the role is a compile-time parameter: at narrow tiles a producer's time per k-block is
        // close to the kernel's.
        {
            auto produce = [&](auto weights_tag) {
                constexpr bool kWeights = decltype(weights_tag)::value;
                constexpr uint32_t n_stages = kWeights ? kWStages : kStages;
                const uint32_t bar_free = kWeights ? bar_wempty : bar_empty;
                uint32_t s = 0, ph = 0, it = 0;
                bool ok = true;
                const bool stat = p.stats != nullptr && blockIdx.x == 0;
                StatTimer tt(stat), tw(stat);
                long long st_total = 0, st_wait = 0;
                const int n_coord = static_cast<int>(rank) * kBW * 2;                 // weight map counts 8-byte units: 2 per n
                [[maybe_unused]] const int tok_off = kPair ? static_cast<int>(rank) * C::kTokLoad : 0;   // token role of a pair only
                tt.start();
                for (int u = cluster_id; ok && u < p.num_units; u += num_clusters) {
                    const Unit w = decode_unit<TN, CG>(p, u);
                    int kb = w.kb_begin;
                    const int kb_total = EXT ? w.kb_total : w.kb_count;
                    for (int i = 0; i < kb_total; ++i, ++kb, ++it) {
                        const bool low_rank = EXT && i >= w.kb_count;                // block e = i - kb_count of the LoRA term
                        [[maybe_unused]] const int e = i - w.kb_count;
                        tw.start();
                        const bool free_ok = mbar_wait_warp(bar_free + 8 * s, ph ^ 1u, abort_flag, lane);
                        tw.stop(st_wait);
                        if (!free_ok) {
                            if (lane == 0) give_up<CG>(p, abort_flag, kRoleProducer, (kWeights ? 0x100 : 0) | s);
                            ok = false;
                            break;
                        }
                        if (lane != 0) {
                            // nothing to issue
                        } else if constexpr (kWeights) {
                            mbar_arrive_expect_tx(bar_wfull + 8 * s, kWStageBytes);
                            if (low_rank)
                                tma_load_2d(smem_w + s * kWStageBytes, &tmap_l.b, bar_wfull + 8 * s, w.n0 * 2 + n_coord, e * 8);
                            else
                                tma_load_2d(smem_w + s * kWStageBytes, &tmap_w, bar_wfull + 8 * s, w.n0 * 2 + n_coord, kb * kKSteps);
                        } else {
                            const uint32_t bar = kPair ? mapa_u32(bar_full + 8 * s, 0) : bar_full + 8 * s;
                            const uint32_t dst = smem_a + s * C::kAStageBytes;
                            const uint32_t tx_bytes = low_rank ? C::kASubBytes : C::kAStageBytes;     // a low-rank block is one sub-tile
                            if constexpr (!kPair)
                                mbar_arrive_expect_tx(bar, tx_bytes);
                            else
                                mbar_arrive_expect_tx_cluster(bar, tx_bytes);
                            if (low_rank) {
                                if constexpr (!kPair)
                                    tma_load_2d(dst, &tmap_l.t, bar, e * kSubK, w.tok0);
                                else
                                    tma_load_2d_pair(dst, &tmap_l.t, bar, e * kSubK, w.tok0 + tok_off);
                            } else if (p.a3d) {
                                if constexpr (!kPair)
                                    tma_load_3d(dst, &tmap_a, bar, 0, w.tok0, kb * kSubTiles);
                                else
                                    tma_load_3d_pair(dst, &tmap_a, bar, 0, w.tok0 + tok_off, kb * kSubTiles);
                            } else {
#pragma unroll
                                for (int sub = 0; sub < kSubTiles; ++sub) {
                                    if constexpr (!kPair)
                                        tma_load_2d(dst + sub * C::kASubBytes, &tmap_a, bar, kb * kBK + sub * kSubK, w.tok0);
                                    else
                                        tma_load_2d_pair(dst + sub * C::kASubBytes, &tmap_a, bar, kb * kBK + sub * kSubK, w.tok0 + tok_off);
                                }
                            }
                        }
                        if (++s == n_stages) {
                            s = 0;
                            ph ^= 1u;
                        }
                    }
                }
                tt.stop(st_total);
                if (stat && lane == 0) {
                    p.stats[kWeights ? 2 : 0] = st_total;
                    p.stats[kWeights ? 3 : 1] = st_wait;
                }
                if (!ok && lane == 0) {
                    // Let this CTA's own copies land before shared memory goes away: a bounded wait on the weight barriers armed
                    // most recently, and a short fixed pause for the token loads (their barrier may live in the pair's other CTA).
                    if constexpr (kWeights) {
                        const uint32_t back = it < n_stages ? it : n_stages;
                        for (uint32_t j = 1; j <= back; ++j) {
                            const uint32_t jt = it - j;
                            const uint64_t t0 = globaltimer_ns();
                            while (!mbar_try_wait(bar_wfull + 8 * (jt % n_stages), (jt / n_stages) & 1u) && globaltimer_ns() - t0 < 1000000ull) {
                            }
                        }
                    }
                    const uint64_t t1 = globaltimer_ns();
                    while (globaltimer_ns() - t1 < 20000ull) {
                    }
                }
            };
            if (warp == kWProducerWarp)
                produce(std::true_type{});
            else
                produce(std::false_type{});
        }
        __syncwarp();
    } else if (warp == kMmaWarp || (kIssuers == 2 && warp == kMma2Warp)) {
        // ------------------------------------------------------------------ MMA issuers (leader CTA, one lane per issuing warp)
        if (rank == 0 && lane == 0) {
            const uint32_t idesc_main = umma_idesc_f16(kBW * CG, TN, EXT && p.a_bf16 != 0);
            [[maybe_unused]] constexpr uint32_t idesc_low_rank = umma_idesc_f16(kBW * CG, TN, false);   // the LoRA term's operands are always fp16
            const uint32_t issuer = warp == kMmaWarp ? 0u : 1u;
            // One lane runs this loop (a loop that the whole warp runs in lockstep, with lane 0 issuing, measured slower: its
            // waits cost more).  It is written for instruction count: for tiles narrower than 256 tokens the tensor pipe
            // finishes a k-block sooner than one thread can issue its eight MMAs plus bookkeeping.  The ring cursor advances
            // incrementally; per k-block there is one barrier probe and one commit.  With two issuers, issuer j takes the
            // k-blocks i of a tile with i % 2 == j and accumulates them in accumulator j of the tile's buffer.
            uint32_t ui = 0, kblocks = 0;
            uint32_t s = 0, ph = 0;                                               // operand ring slot of the next k-block and its phase parity
            bool peeked = false;                                                  // this issuer's next slot was already seen full by its last probe
            bool ok = true;
            const bool stat = p.stats != nullptr && blockIdx.x == 0 && issuer == 0;
            StatTimer tt(stat), tw(stat);
            long long st_total = 0, st_acc = 0, st_ops = 0, st_events = 0;
            const uint64_t desc0 = umma_desc_kmajor_sw128(smem_a);
            auto advance = [&](uint32_t& slot, uint32_t& parity) {
                if (++slot == kStages) {
                    slot = 0;
                    parity ^= 1u;
                }
            };
            tt.start();
            for (int u = cluster_id; ok && u < p.num_units; u += num_clusters, ++ui) {
                const Unit w = decode_unit<TN, CG>(p, u);
                const uint32_t a = ui % kAccs;
                const uint32_t aph = (ui / kAccs) & 1u;
                tw.start();
                const bool acc_ok = mbar_wait(bar_accempty + 8 * a, aph ^ 1u, abort_flag);
                tw.stop(st_acc);
                if (!acc_ok) {
                    give_up<CG>(p, abort_flag, kRoleMma, 0x100);
                    break;
                }
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + (a * kIssuers + issuer) * TN;
                uint32_t accumulate = 0;                                          // this issuer's first MMA of a tile overwrites its accumulator
                const int kb_total = EXT ? w.kb_total : w.kb_count;
                for (int i = 0; i < kb_total; ++i) {
                    if (kIssuers == 2 && (static_cast<uint32_t>(i) & 1u) != issuer) {
                        advance(s, ph);
                        continue;
                    }
                    if (!peeked) {
                        tw.start();
                        const bool full_ok = mbar_wait(bar_full + 8 * s, ph, abort_flag);
                        tw.stop(st_ops);
                        ++st_events;
                        if (!full_ok) {
                            give_up<CG>(p, abort_flag, kRoleMma, 0x200 | s);
                            ok = false;
                            break;
                        }
                    }
                    // Probe this issuer's next slot now (non-blocking): the barrier's latency overlaps with the issue below, and
                    // only a phase that is still pending then is waited for at the top of that k-block.  Across a tile boundary
                    // the distance to the next own k-block varies, so nothing is probed there.
                    uint32_t sn = s, phn = ph;
#pragma unroll
                    for (int j = 0; j < kIssuers; ++j) advance(sn, phn);
                    peeked = (i + kIssuers < kb_total) && mbar_test_wait(bar_full + 8 * sn, phn);
                    tc_fence_after();
                    const uint32_t a_tmem = tmem_wring + s * kTColsPerStage;
                    const uint64_t b_stage = desc0 + static_cast<uint64_t>(s * (C::kAStageBytes >> 4));
                    const bool low_rank = EXT && i >= w.kb_count;
                    const int sub_tiles = low_rank ? 1 : kSubTiles;                    // a low-rank block holds 64 k: one sub-tile
                    const uint32_t idesc = low_rank ? idesc_low_rank : idesc_main;
#pragma unroll
                    for (int sub = 0; sub < kSubTiles; ++sub) {
                        if (!EXT || sub < sub_tiles) {
#pragma unroll
                            for (int ks = 0; ks < kSubK / 16; ++ks) {
                                // +32 bytes of K inside the 128-byte swizzle row = +2 in the descriptor's address field
                                umma_f16_ts<CG>(d_tmem, a_tmem + (sub * (kSubK / 16) + ks) * 8,
                                                b_stage + static_cast<uint64_t>(sub * (C::kASubBytes >> 4) + ks * 2), idesc, (sub | ks) != 0 ? 1u : accumulate);
                            }
                        }
                    }
                    if constexpr (!kPair)
                        umma_commit_1cta(bar_empty + 8 * s);
                    else
                        umma_commit_pair(bar_empty + 8 * s, 0x3);
                    accumulate = 1u;
                    advance(s, ph);
                    ++kblocks;
                }
                if (!ok) break;
                // every issuer commits (also one without a k-block in this tile): the barrier expects kIssuers arrivals
                if constexpr (!kPair)
                    umma_commit_1cta(bar_accfull + 8 * a);
                else
                    umma_commit_pair(bar_accfull + 8 * a, 0x3);
            }
            tt.stop(st_total);
            if (stat) {
                p.stats[4] = st_total;
                p.stats[5] = st_acc;
                p.stats[6] = st_ops;            // waits for a full operand slot (token tile + upcast weights) that the probe had not seen
                p.stats[7] = 0;
                p.stats[18] = st_events;        // how many such waits
                p.stats[22] = kblocks;          // k-blocks issued by issuer 0
            }
            // Nothing of this CTA pair may be torn down while an MMA is still reading it.
            if constexpr (!kPair)
                umma_commit_1cta(bar_drain + 8 * issuer);
            else
                umma_commit_2cta_local(bar_drain + 8 * issuer);
            {
                const uint64_t t0 = globaltimer_ns();
                while (!mbar_try_wait(bar_drain + 8 * issuer, 0) && globaltimer_ns() - t0 < kWaitLimitNs) {
                }
            }
        }
        __syncwarp();   // the idle lanes wait for the issuing lane here, not at the teardown barrier
    } else if (warp >= kFirstTransformWarp) {
        // ------------------------------------------------------------------ e5m2 -> fp16 into TMEM
        const int q = warp & 3;
        const int g = (warp - kFirstTransformWarp) >> 2;
        const uint32_t w_lane_off = static_cast<uint32_t>(q * 32 + lane) * 16u;
        const uint32_t t_lane = static_cast<uint32_t>(q * 32) << 16;
        const int up_mode = EXT ? ((p.a_bf16 ? 1 : 0) | (p.w_e4m3 ? 2 : 0)) : 0;
        // Running ring positions of the next k-block (weight-byte ring, operand ring) and whose turn it is; no division in the loop.
        uint32_t ws = 0, wph = 0, os = 0, oph = 0;
        int turn = 0;
        bool ok = true;
        const bool stat = p.stats != nullptr && blockIdx.x == 0 && warp == kFirstTransformWarp;
        StatTimer tt(stat), tw(stat);
        long long st_total = 0, st_bytes = 0, st_tmem = 0;
        tt.start();
        for (int u = cluster_id; ok && u < p.num_units; u += num_clusters) {
            const Unit w = decode_unit<TN, CG>(p, u);
            const int kb_total = EXT ? w.kb_total : w.kb_count;
            for (int i = 0; i < kb_total; ++i) {
                const uint32_t s = ws, ph = wph, t = os, tph = oph;
                const bool low_rank = EXT && i >= w.kb_count;
                const bool mine = turn == g;
                if (++ws == kWStages) {
                    ws = 0;
                    wph ^= 1u;
                }
                if (++os == kStages) {
                    os = 0;
                    oph ^= 1u;
                }
                if (++turn == TG) turn = 0;
                if (!mine) continue;
                tw.start();
                bool got = mbar_wait_warp(bar_wfull + 8 * s, ph, abort_flag, lane);
                tw.stop(st_bytes);
                tw.start();
                got = got && mbar_wait_warp(bar_empty + 8 * t, tph ^ 1u, abort_flag, lane);
                tw.stop(st_tmem);
                if (!got) {
                    if (lane == 0) give_up<CG>(p, abort_flag, kRoleTransform, (q << 8) | s);
                    ok = false;
                    break;
                }
                tc_fence_after();
                const uint32_t src = smem_w + s * kWStageBytes + w_lane_off;
                const uint32_t dst = tmem_wring + t_lane + t * kTColsPerStage;
                {
                    uint32_t x[kKSteps][4];
#pragma unroll
                    for (int j = 0; j < kKSteps; ++j)
                        asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];"
                                     : "=r"(x[j][0]), "=r"(x[j][1]), "=r"(x[j][2]), "=r"(x[j][3])
                                     : "r"(src + j * (kBW * 16)));
                    if (low_rank) {
                        // B' is fp16 already: 16 bytes are 8 ranks = 4 tensor-memory columns, no upcast
#pragma unroll
                        for (int j = 0; j < kKSteps; ++j) tmem_st_32x32b_x4(dst + j * 4, x[j]);
                    } else if (up_mode == 0) {
#pragma unroll
                        for (int j = 0; j < kKSteps; ++j) {
                            uint32_t v[8];
                            // bytes b0..b3 of a word are k, k+1, k+2, k+3; fp16(b) = b << 8
#pragma unroll
                            for (int i = 0; i < 4; ++i) {
                                v[2 * i] = __byte_perm(x[j][i], 0u, 0x1404);
                                v[2 * i + 1] = __byte_perm(x[j][i], 0u, 0x3424);
                            }
                            tmem_st_32x32b_x8(dst + j * 8, v);
                        }
                    } else {
                        // bf16 activations and / or e4m3 weights: a few more integer / convert instructions per pair
#pragma unroll
                        for (int j = 0; j < kKSteps; ++j) {
                            uint32_t v[8];
#pragma unroll
                            for (int i = 0; i < 4; ++i) {
                                v[2 * i] = upcast_pair(__byte_perm(x[j][i], 0u, 0x1404), up_mode);
                                v[2 * i + 1] = upcast_pair(__byte_perm(x[j][i], 0u, 0x3424), up_mode);
                            }
                            tmem_st_32x32b_x8(dst + j * 8, v);
                        }
                    }
                }
                tc_wait_st();
                tc_fence_before();
                __syncwarp();
                if (lane == 0) {
                    mbar_arrive(bar_wempty + 8 * s);
                    if constexpr (!kPair)
                        mbar_arrive(bar_full + 8 * t);
                    else
                        mbar_arrive_cluster(mapa_u32(bar_full + 8 * t, 0));
                }
            }
        }
        tt.stop(st_total);
        if (stat && lane == 0) {
            p.stats[8] = st_total;
            p.stats[9] = st_bytes;
            p.stats[10] = st_tmem;
        }
    } else {
        // ------------------------------------------------------------------ epilogue (warps 0..7)
        // Warp e reads the TMEM lanes of quarter e % 4 (its 32 output columns n); the two groups e / 4 take alternate blocks
        // of kOutRows accumulator columns (token rows), each group with its own staging buffer and named barrier.
        const int q = warp & 3;
        const int grp = warp >> 2;
        const bool group_leader = (threadIdx.x & 127) == 0;
        const uint32_t t_lane = static_cast<uint32_t>(q * 32) << 16;
        const float scale = (p.scale != nullptr ? __ldg(p.scale) : 1.0f) * (EXT ? p.scale_mul : 1.0f);
        const bool out_bf16 = p.out_bf16 != 0;
        const bool flip = p.flip_final != 0;
        const bool has_bias = p.bias != nullptr;
        uint16_t* const c16 = reinterpret_cast<uint16_t*>(p.c);
        constexpr int kTileCols = kBW * CG;
        constexpr int kOutRows = C::kOutRows;
        constexpr bool kHoldTile = TN == 256 && TG == 1 && kAccs == 1;
        const bool staged = p.tma_store != 0 && p.splits == 1;
        const uint32_t out_base = smem_out + grp * (C::kOutBufs * C::kOutBufBytes);
        uint32_t ui = 0;
        uint32_t out_flip = 0;                                             // blocks this group has staged so far (its staging ring position)
        // A warp whose wait ran out stays in the loop as a bystander (alive = false): it touches no tensor
        // memory but still joins every named barrier, so the other epilogue warps are never left waiting.
        bool alive = true;
        const bool stat = p.stats != nullptr && blockIdx.x == 0 && warp == 0;
        StatTimer tt(stat), tw(stat);
        long long st_total = 0, st_full = 0, st_emit = 0, st_chunks = 0;
        tt.start();
        for (int u = cluster_id; u < p.num_units; u += num_clusters, ++ui) {
            const Unit w = decode_unit<TN, CG>(p, u);
            const uint32_t a = ui % kAccs;
            const uint32_t aph = (ui / kAccs) & 1u;
            // The tile's bias values are fetched before the wait for its accumulator, so their latency is not part of the read-back.
            const int col_local = q * 32 + lane;                                  // column inside this CTA's 128
            const int col = static_cast<int>(rank) * kBW + col_local;             // column inside the tile
            const int n = w.n0 + col;
            const bool n_ok = n < p.N;
            const uint16_t bias_bits = (has_bias && n_ok) ? __ldg(reinterpret_cast<const uint16_t*>(p.bias) + n) : uint16_t(0);
            // the staged path's fragment layout: this thread's four output columns (one per matrix), bias duplicated into both halves of a word
            uint32_t bias2[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int nn = w.n0 + static_cast<int>(rank) * kBW + q * 32 + 8 * i + (lane >> 2);
                const uint32_t bb = (has_bias && nn < p.N) ? __ldg(reinterpret_cast<const uint16_t*>(p.bias) + nn) : 0u;
                bias2[i] = bb * 0x00010001u;
            }
            if (alive) {
                tw.start();
                const bool got = mbar_wait_warp(bar_accfull + 8 * a, aph, abort_flag, lane);
                tw.stop(st_full);
                if (!got) {
                    if (lane == 0) give_up<CG>(p, abort_flag, kRoleEpilogue, warp);
                    alive = false;
                }
            }
            tc_fence_after();
            const uint32_t src = tmem_base + t_lane + a * (kIssuers * TN);
            // With two issuers the tile's sum is split over two accumulators (even / odd k-blocks); a tile of one k-block has
            // nothing in the second.
            const bool two_sums = kIssuers == 2 && (EXT ? w.kb_total : w.kb_count) >= 2;
            // 16 accumulator columns starting at column c0 -> registers (fp32 bit patterns), both partial sums added.
            auto load_sum16 = [&](int c0, uint32_t (&v)[16]) {
                tmem_ld_32x32b_x16(src + c0, v);
                if (two_sums) {
                    uint32_t v2[16];
                    tmem_ld_32x32b_x16(src + TN + c0, v2);
                    tc_wait_ld();
#pragma unroll
                    for (int j = 0; j < 16; ++j) v[j] = __float_as_uint(__uint_as_float(v[j]) + __uint_as_float(v2[j]));
                } else {
                    tc_wait_ld();
                }
            };
            const int valid = p.M - w.tok0 < TN ? p.M - w.tok0 : TN;              // token columns of this tile that exist
            // The accumulator goes back to the MMA warp as soon as this warp's last TMEM load of the tile has landed.
            bool released = false;
            auto release_acc = [&]() {
                if (released) return;
                released = true;
                if (!alive) return;
                tc_fence_before();
                __syncwarp();
                if (lane == 0) {
                    if constexpr (!kPair)
                        mbar_arrive(bar_accempty + 8 * a);
                    else
                        mbar_arrive_cluster(mapa_u32(bar_accempty + 8 * a, 0));
                }
            };

            if (staged) {
                // Staged path: each group of four warps fills its shared-memory buffer with kOutRows token rows of the
                // CTA's 128 output columns and one thread hands the buffer to TMA.  The accumulator is read as MMA fragments
                // (thread t: TMEM lanes = output columns t/4 + 8i, token pairs 2(t%4), +1), each pair is scaled, converted
                // and packed into one word, and stmatrix transposes 8 token rows x 32 columns per instruction into the
                // buffer, which is two [rows][64 columns] tiles in the 128-byte swizzle the output tensor map declares
                // (row r keeps its 16-byte chunk c at chunk c ^ (r % 8), so the eight rows of a matrix hit distinct banks).
                // No shuffles and no sub-word stores; output type and bias are compile-time tags, chosen once per tile.
                const int first = grp * kOutRows;                                  // this group's blocks: first, first + 2*kOutRows, ...
                const int store_x = w.n0 + static_cast<int>(rank) * kBW;
                const uint32_t frag = src;                                         // lanes q*32 .. +15; +16 lanes for the upper half
                const uint32_t frag_hi = src + (16u << 16);
                // thread t supplies the address of row t % 8 of matrix t / 8
                const uint32_t st_lane = (q >> 1) * (kOutRows * 128) + (lane & 7) * 128 +
                                         (((static_cast<uint32_t>(q & 1) * 4 + (lane >> 3)) ^ (lane & 7)) << 4);
                // 256-token tiles with one transform group (the long-GEMM variant; 480 threads leave 128 registers each): three of
                // the group's four blocks are read, scaled, rounded and packed into 48 registers, then the fourth is read; the
                // accumulator goes back to the MMA warps as soon as the last load has landed, and only then are the blocks staged
                // and stored.  The tensor cores so wait for the
                // tensor-memory loads alone, not for the staging buffer's round trips through the store engine.  Output type,
                // bias and final cast are run-time (warp-uniform) branches here: one copy of this code keeps the values in
                // registers, eight copies made the compiler park them in local memory.
                auto drain_held = [&]() {
                    auto load16 = [&](int c, uint32_t (&lo)[8], uint32_t (&hi)[8]) {
                        tmem_ld_16x256b_x2(frag + c, lo);
                        tmem_ld_16x256b_x2(frag_hi + c, hi);
                    };
                    auto block_begin = [&]() {
                        if (group_leader) tma_store_wait_read<C::kOutBufs - 1>();  // the stores that read this buffer are done with it
                        asm volatile("bar.sync %0, 128;" ::"r"(2 + grp) : "memory");
                    };
                    auto block_end = [&](uint32_t buf, int c0) {
                        fence_proxy_async_smem();
                        asm volatile("bar.sync %0, 128;" ::"r"(2 + grp) : "memory");
                        if (group_leader) {
                            // a CTA whose 128 columns all lie beyond N (second CTA of the last pair) has nothing to store
                            int d_begin = 0, d_end = store_x < p.N ? p.n_dst : 0, row = w.tok0 + c0;
                            if (EXT && p.scatter_rows > 0 && d_end > 0) {
                                // row-sharded destinations: the block goes to the one buffer that owns its token rows
                                d_begin = row / p.scatter_rows;
                                row -= d_begin * p.scatter_rows;
                                d_end = d_begin + 1;
                            }
                            for (int d = d_begin; d < d_end; ++d) {
                                if (p.c3d) {
                                    tma_store_3d(&tmap_c.m[d], buf, 0, row, store_x >> 6);   // both 64-column tiles at once
                                } else {
                                    tma_store_2d(&tmap_c.m[d], buf, store_x, row);
                                    if (store_x + 64 < p.N) tma_store_2d(&tmap_c.m[d], buf + kOutRows * 128, store_x + 64, row);
                                }
                            }
                            tma_store_commit();
                        }
                    };
                    auto pack = [&](uint32_t x0, uint32_t x1, uint32_t b2) -> uint32_t {
                        const float r0 = __uint_as_float(x0) * scale, r1 = __uint_as_float(x1) * scale;
                        if (out_bf16) {
                            __nv_bfloat162 x = __floats2bfloat162_rn(r0, r1);
                            if (has_bias) x = __hadd2(x, *reinterpret_cast<const __nv_bfloat162*>(&b2));
                            if (flip) {
                                const float2 f = __bfloat1622float2(x);
                                const __half2 y = __floats2half2_rn(f.x, f.y);
                                return *reinterpret_cast<const uint32_t*>(&y);
                            }
                            return *reinterpret_cast<const uint32_t*>(&x);
                        } else {
                            __half2 x = __floats2half2_rn(r0, r1);
                            if (has_bias) x = __hadd2(x, *reinterpret_cast<const __half2*>(&b2));
                            if (flip) {
                                const float2 f = __half22float2(x);
                                const __nv_bfloat162 y = __floats2bfloat162_rn(f.x, f.y);
                                return *reinterpret_cast<const uint32_t*>(&y);
                            }
                            return *reinterpret_cast<const uint32_t*>(&x);
                        }
                    };
                    auto pack16 = [&](const uint32_t (&lo)[8], const uint32_t (&hi)[8], uint32_t (&dst)[16], auto half_tag) {
                        constexpr int kAt = decltype(half_tag)::value * 8;
#pragma unroll
                        for (int g = 0; g < 2; ++g) {
                            dst[kAt + 4 * g + 0] = pack(lo[4 * g], lo[4 * g + 1], bias2[0]);
                            dst[kAt + 4 * g + 1] = pack(lo[4 * g + 2], lo[4 * g + 3], bias2[1]);
                            dst[kAt + 4 * g + 2] = pack(hi[4 * g], hi[4 * g + 1], bias2[2]);
                            dst[kAt + 4 * g + 3] = pack(hi[4 * g + 2], hi[4 * g + 3], bias2[3]);
                        }
                    };
                    auto stage = [&](const uint32_t (&v)[16], uint32_t buf) {
#pragma unroll
                        for (int g = 0; g < 4; ++g) stmatrix_x4_trans(buf + st_lane + (8 * g) * 128, v[4 * g], v[4 * g + 1], v[4 * g + 2], v[4 * g + 3]);
                    };
                    constexpr int kBlocks = TN / (2 * kOutRows);
                    constexpr int kHeld = kBlocks > 1 ? kBlocks - 1 : 1;          // (only instantiated meaningfully for 256-token tiles)
                    uint32_t held[kHeld][16];
                    {
                        // Blocks 1.. of the group are parked first, then block 0 is read; the accumulator goes back as soon as block 0's
                        // last load has landed, before anything is staged.
                        uint32_t lo[8], hi[8], now[16];
#pragma unroll
                        for (int b = 0; b < kHeld; ++b) {
                            const int c0 = first + (b + 1) * 2 * kOutRows;
                            if (c0 < valid) {
                                load16(c0, lo, hi);
                                tc_wait_ld();
                                pack16(lo, hi, held[b], std::integral_constant<int, 0>{});
                                load16(c0 + 16, lo, hi);
                                tc_wait_ld();
                                pack16(lo, hi, held[b], std::integral_constant<int, 1>{});
                            }
                        }
                        if (first < valid) {
                            const uint32_t buf = out_base + (out_flip % C::kOutBufs) * C::kOutBufBytes;
                            load16(first, lo, hi);
                            tc_wait_ld();
                            pack16(lo, hi, now, std::integral_constant<int, 0>{});
                            load16(first + 16, lo, hi);
                            tc_wait_ld();
                            release_acc();
                            pack16(lo, hi, now, std::integral_constant<int, 1>{});
                            block_begin();
                            stage(now, buf);
                            block_end(buf, first);
                        }
                    }
                    release_acc();
#pragma unroll
                    for (int b = 0; b < kHeld; ++b) {
                        const int c0 = first + (b + 1) * 2 * kOutRows;
                        if (c0 < valid) {
                            const uint32_t buf = out_base + ((out_flip + static_cast<uint32_t>(b + 1)) % C::kOutBufs) * C::kOutBufBytes;
                            block_begin();
                            stage(held[b], buf);
                            block_end(buf, c0);
                        }
                    }
                };
                auto drain = [&](auto bf16_tag, auto bias_tag, auto flip_tag) {
                    constexpr bool kBf16 = decltype(bf16_tag)::value;
                    constexpr bool kBias = decltype(bias_tag)::value;
                    constexpr bool kFlip = decltype(flip_tag)::value;     // store the other 16-bit dtype (one more rounding)
                    auto pack = [&](uint32_t x0, uint32_t x1, uint32_t b2) -> uint32_t {
                        const float r0 = __uint_as_float(x0) * scale, r1 = __uint_as_float(x1) * scale;
                        if constexpr (kBf16) {
                            __nv_bfloat162 x = __floats2bfloat162_rn(r0, r1);
                            if constexpr (kBias) x = __hadd2(x, *reinterpret_cast<const __nv_bfloat162*>(&b2));
                            if constexpr (kFlip) {
                                const float2 f = __bfloat1622float2(x);
                                const __half2 y = __floats2half2_rn(f.x, f.y);
                                return *reinterpret_cast<const uint32_t*>(&y);
                            }
                            return *reinterpret_cast<const uint32_t*>(&x);
                        } else {
                            __half2 x = __floats2half2_rn(r0, r1);
                            if constexpr (kBias) x = __hadd2(x, *reinterpret_cast<const __half2*>(&b2));
                            if constexpr (kFlip) {
                                const float2 f = __half22float2(x);
                                const __nv_bfloat162 y = __floats2bfloat162_rn(f.x, f.y);
                                return *reinterpret_cast<const uint32_t*>(&y);
                            }
                            return *reinterpret_cast<const uint32_t*>(&x);
                        }
                    };
                    // 16 token rows (accumulator columns c .. c+15) -> rows row0 .. row0+15 of the staging buffer
                    auto store16 = [&](const uint32_t (&lo)[8], const uint32_t (&hi)[8], uint32_t buf, int row0) {
#pragma unroll
                        for (int g = 0; g < 2; ++g)
                            stmatrix_x4_trans(buf + st_lane + (row0 + 8 * g) * 128, pack(lo[4 * g], lo[4 * g + 1], bias2[0]), pack(lo[4 * g + 2], lo[4 * g + 3], bias2[1]),
                                              pack(hi[4 * g], hi[4 * g + 1], bias2[2]), pack(hi[4 * g + 2], hi[4 * g + 3], bias2[3]));
                    };
                    auto load16 = [&](int c, uint32_t (&lo)[8], uint32_t (&hi)[8]) {
                        tmem_ld_16x256b_x2(frag + c, lo);
                        tmem_ld_16x256b_x2(frag_hi + c, hi);
                    };
                    auto add_second = [&](int c, uint32_t (&lo)[8], uint32_t (&hi)[8]) {   // the odd k-blocks' partial sum
                        uint32_t lo2[8], hi2[8];
                        tmem_ld_16x256b_x2(frag + TN + c, lo2);
                        tmem_ld_16x256b_x2(frag_hi + TN + c, hi2);
                        tc_wait_ld();
    #pragma unroll
                        for (int j = 0; j < 8; ++j) {
                            lo[j] = __float_as_uint(__uint_as_float(lo[j]) + __uint_as_float(lo2[j]));
                            hi[j] = __float_as_uint(__uint_as_float(hi[j]) + __uint_as_float(hi2[j]));
                        }
                    };
                    // One bulk group per block: with two buffers the group before the last may still be reading.
                    auto block_begin = [&]() {
                        if (group_leader) tma_store_wait_read<C::kOutBufs - 1>();  // the stores that read this buffer are done with it
                        asm volatile("bar.sync %0, 128;" ::"r"(2 + grp) : "memory");
                    };
                    auto block_end = [&](uint32_t buf, int c0) {
                        fence_proxy_async_smem();
                        asm volatile("bar.sync %0, 128;" ::"r"(2 + grp) : "memory");
                        if (group_leader) {
                            // a CTA whose 128 columns all lie beyond N (second CTA of the last pair) has nothing to store
                            int d_begin = 0, d_end = store_x < p.N ? p.n_dst : 0, row = w.tok0 + c0;
                            if (EXT && p.scatter_rows > 0 && d_end > 0) {
                                // row-sharded destinations: the block goes to the one buffer that owns its token rows
                                d_begin = row / p.scatter_rows;
                                row -= d_begin * p.scatter_rows;
                                d_end = d_begin + 1;
                            }
                            for (int d = d_begin; d < d_end; ++d) {
                                if (p.c3d) {
                                    tma_store_3d(&tmap_c.m[d], buf, 0, row, store_x >> 6);   // both 64-column tiles at once
                                } else {
                                    tma_store_2d(&tmap_c.m[d], buf, store_x, row);
                                    if (store_x + 64 < p.N) tma_store_2d(&tmap_c.m[d], buf + kOutRows * 128, store_x + 64, row);
                                }
                            }
                            tma_store_commit();
                        }
                    };
                    constexpr int kPasses = kOutRows / 16;                         // 16 token rows per pass
                    if constexpr (kIssuers == 2) {
                        // Narrow tiles (two partial sums): loads are not overlapped with the conversion; the whole epilogue
                        // of such a tile is short against the weight stream it follows.
#pragma unroll 1
                        for (int c0 = first; c0 < valid; c0 += 2 * kOutRows) {
                            const bool last = c0 + 2 * kOutRows >= valid;
                            block_begin();
#pragma unroll
                            for (int ps = 0; ps < kPasses; ++ps) {
                                uint32_t lo[8], hi[8];
                                load16(c0 + 16 * ps, lo, hi);
                                if (two_sums)
                                    add_second(c0 + 16 * ps, lo, hi);
                                else
                                    tc_wait_ld();
                                if (last && ps == kPasses - 1) release_acc();
                                store16(lo, hi, out_base, 16 * ps);
                            }
                            block_end(out_base, c0);
                        }
                        release_acc();
                    } else {
                        // Wide tiles: the fragment loads of the next 16 token rows are in flight while the current 16 are
                        // converted and stored.
                        uint32_t lo[8], hi[8], lo_n[8], hi_n[8];
                        if (first < valid) load16(first, lo, hi);
#pragma unroll 1
                        for (int c0 = first; c0 < valid; c0 += 2 * kOutRows) {
                            const int next = c0 + 2 * kOutRows;
                            static_assert(kIssuers == 2 || kPasses == 2, "wide tiles stage 32 rows per block");
                            // The group's staging ring is used round-robin over all its blocks, across tiles.  The position is derived from
                            // the block's place in the tile plus a count carried between tiles: a counter bumped inside this loop
                            // made the compiler spill.
                            const uint32_t buf = out_base + ((out_flip + static_cast<uint32_t>(c0 - first) / (2 * kOutRows)) % C::kOutBufs) * C::kOutBufBytes;
                            tc_wait_ld();
                            load16(c0 + 16, lo_n, hi_n);
                            block_begin();
                            store16(lo, hi, buf, 0);
                            tc_wait_ld();
                            if (next < valid)
                                load16(next, lo, hi);
                            else
                                release_acc();
                            store16(lo_n, hi_n, buf, 16);
                            block_end(buf, c0);
                        }
                        release_acc();                                             // a group without any block in this tile
                    }
                };
                tw.start();
                if (alive && kHoldTile) {
                    if constexpr (kHoldTile) drain_held();
                } else if (alive) {
                    auto with_flip = [&](auto bf16_tag, auto bias_tag) {
                        if (flip) drain(bf16_tag, bias_tag, std::true_type{});
                        else drain(bf16_tag, bias_tag, std::false_type{});
                    };
                    if (out_bf16) {
                        if (has_bias) with_flip(std::true_type{}, std::true_type{});
                        else with_flip(std::true_type{}, std::false_type{});
                    } else {
                        if (has_bias) with_flip(std::false_type{}, std::true_type{});
                        else with_flip(std::false_type{}, std::false_type{});
                    }
                } else {
                    // bystander: joins the group's two barriers per block and nothing else
                    for (int c0 = first; c0 < valid; c0 += 2 * kOutRows) {
                        asm volatile("bar.sync %0, 128;" ::"r"(2 + grp) : "memory");
                        asm volatile("bar.sync %0, 128;" ::"r"(2 + grp) : "memory");
                    }
                }
                tw.stop(st_emit);
                if (first < valid) {
                    const uint32_t blocks = static_cast<uint32_t>(valid - first + 2 * kOutRows - 1) / (2 * kOutRows);
                    out_flip += blocks;
                    st_chunks += blocks;
                }
            } else if (p.splits == 1) {
                // Direct path (output rows that TMA cannot address: a row pitch that is not a multiple of 16 bytes)
                uint16_t* const c_col = c16 + static_cast<long long>(w.tok0) * p.ldc + n;
                if (alive) {
#pragma unroll 1
                    for (int c0 = grp * 16; c0 < valid; c0 += 32) {
                        uint32_t v[16];
                        load_sum16(c0, v);
                        if (c0 + 32 >= valid) release_acc();
                        if (n_ok) {
#pragma unroll
                            for (int j = 0; j < 16; ++j) {
                                if (c0 + j < valid)
                                    c_col[static_cast<long long>(c0 + j) * p.ldc] = finish_value(__uint_as_float(v[j]), scale, out_bf16, has_bias, bias_bits, flip);
                            }
                        }
                    }
                }
                release_acc();
            } else {
                // split-K: park this slice's fp32 partial, then the last slice to arrive reduces in slice order
                float* const part = p.ws_partials + (static_cast<long long>(w.tile) * p.splits + w.split) * (TN * kTileCols);
                if (alive) {
#pragma unroll 1
                    for (int c0 = grp * 16; c0 < valid; c0 += 32) {
                        uint32_t v[16];
                        load_sum16(c0, v);
#pragma unroll
                        for (int j = 0; j < 16; ++j) __stcg(part + (c0 + j) * kTileCols + col, __uint_as_float(v[j]));
                    }
                }
                release_acc();
                __threadfence();
                asm volatile("bar.sync 1, 256;" ::: "memory");
                int* const counter = p.ws_counters + w.tile * CG + static_cast<int>(rank);
                if (threadIdx.x == 0) {
                    const int old = atomicAdd(counter, 1);
                    *last_flag = (old == p.splits - 1) ? 1 : 0;
                }
                asm volatile("bar.sync 1, 256;" ::: "memory");
                const bool is_last = *last_flag != 0;
                if (is_last) {
                    __threadfence();
                    const float* const tile_part = p.ws_partials + static_cast<long long>(w.tile) * p.splits * (TN * kTileCols);
                    if (n_ok && alive) {
                        // Blocks of 8 token rows, alternating between the two warp groups.  The 8 loads of a slice are
                        // independent (and the next slices' loads can be hoisted), the additions stay in slice order.
                        const long long slice_stride = static_cast<long long>(TN) * kTileCols;
#pragma unroll 1
                        for (int c0 = grp * 8; c0 < valid; c0 += 16) {
                            float acc[8];
#pragma unroll
                            for (int i = 0; i < 8; ++i) acc[i] = 0.0f;
#pragma unroll 4
                            for (int sp = 0; sp < p.splits; ++sp) {
                                float v[8];
#pragma unroll
                                for (int i = 0; i < 8; ++i)
                                    v[i] = (c0 + i < valid) ? __ldcg(tile_part + sp * slice_stride + (c0 + i) * kTileCols + col) : 0.0f;
#pragma unroll
                                for (int i = 0; i < 8; ++i) acc[i] += v[i];
                            }
#pragma unroll
                            for (int i = 0; i < 8; ++i)
                                if (c0 + i < valid)
                                    c16[static_cast<long long>(w.tok0 + c0 + i) * p.ldc + n] = finish_value(acc[i], scale, out_bf16, has_bias, bias_bits, flip);
                        }
                    }
                }
                asm volatile("bar.sync 1, 256;" ::: "memory");   // everyone has read last_flag / the partials
                if (is_last && threadIdx.x == 0) *counter = 0;    // ready for the next launch
            }
        }
        tt.stop(st_total);
        if (stat && lane == 0) {
            p.stats[12] = st_total;
            p.stats[13] = st_full;
            p.stats[14] = st_emit;
            p.stats[15] = st_chunks;
        }
        if (group_leader) tma_store_wait_all<0>();               // shared memory must outlive the stores that read it
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

// Encoded tensor maps are cached (a small direct-mapped table): encoding three maps costs more host time than a
// small-M kernel runs.  The key holds everything the encoding depends on, so a changed pointer or shape is a miss.
struct TmapKey {
    const void* ptr;
    uint64_t d0, d1, d2, stride, stride2;
    uint32_t b0, b1, b2;
    int kind, device;
    bool operator==(const TmapKey& o) const {
        return ptr == o.ptr && d0 == o.d0 && d1 == o.d1 && d2 == o.d2 && stride == o.stride && stride2 == o.stride2 && b0 == o.b0 && b1 == o.b1 &&
               b2 == o.b2 && kind == o.kind && device == o.device;
    }
};
// d2 == 0: a 2-D map (d0 x d1, row pitch stride_bytes); otherwise 3-D with a third dimension of pitch stride2_bytes.
static CUresult cached_tmap(EncodeTiledFn encode, CUtensorMap* out, int kind, CUtensorMapDataType dtype, const void* ptr, uint64_t d0, uint64_t d1,
                            uint64_t stride_bytes, uint32_t b0, uint32_t b1, CUtensorMapSwizzle swz, CUtensorMapL2promotion promo, uint64_t d2 = 0,
                            uint64_t stride2_bytes = 0, uint32_t b2 = 0) {
    constexpr int kSlots = 64;
    static std::mutex mu;
    static TmapKey keys[kSlots];
    static CUtensorMap maps[kSlots];
    static bool used[kSlots];
    int dev = 0;
    cudaGetDevice(&dev);
    const TmapKey key{ptr, d0, d1, d2, stride_bytes, stride2_bytes, b0, b1, b2, kind, dev};
    const size_t h = (reinterpret_cast<uintptr_t>(ptr) >> 8) * 0x9E3779B97F4A7C15ull + d0 * 31 + d1 * 17 + b1 * 7 + kind;
    const int slot = static_cast<int>((h >> 20) % kSlots);
    {
        std::lock_guard<std::mutex> lock(mu);
        if (used[slot] && keys[slot] == key) {
            *out = maps[slot];
            return CUDA_SUCCESS;
        }
    }
    const cuuint64_t dims[3] = {d0, d1, d2};
    const cuuint64_t strides[2] = {stride_bytes, stride2_bytes};
    const cuuint32_t box[3] = {b0, b1, b2};
    const cuuint32_t estr[3] = {1, 1, 1};
    const CUresult r = encode(out, dtype, d2 == 0 ? 2 : 3, const_cast<void*>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, swz, promo,
                              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r == CUDA_SUCCESS) {
        std::lock_guard<std::mutex> lock(mu);
        keys[slot] = key;
        maps[slot] = *out;
        used[slot] = true;
    }
    return r;
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

static bool valid_tn(int tn) { return tn == 16 || tn == 32 || tn == 64 || tn == 128 || tn == 192 || tn == 256; }

// Shape heuristic.  Stands in for the reference's per-shape autotune over 28 tile configs
// (kernel/hip/utils.py:192-223): here the tile is fixed by the token count and the machine is filled by
// splitting K when the weight tiles alone cannot.
static bool make_plan(int64_t M, int64_t N, int64_t K, const feather_mm_variant* v, size_t ws_avail, bool ws_known, int sms, Plan* out) {
    Plan pl{};
    pl.total_kb = static_cast<int>((K + kBK - 1) / kBK);
    const int sm_total = sms > 0 ? sms : 148;
    int tn = v ? v->tokens_tile : 0;
    int cg = v ? v->cta_pair : 0;
    if (cg != 0 && cg != 1 && cg != 2) return false;
    // CTA pairs halve the token-tile traffic per SM; up to 64 tokens that traffic is small and single CTAs measured faster.
    const int cg_auto = (N >= 2 * kBW && M > 64) ? 2 : 1;
    if (tn == 0) {
        tn = M <= 16 ? 16 : M <= 32 ? 32 : M <= 64 ? 64 : M <= 128 ? 128 : 256;
        // One 256-token tile per column block leaves most SMs idle when N is small: two 128-token tiles instead.
        if (tn == 256 && M <= 256) {
            const int c = cg ? cg : cg_auto;
            if ((N + kBW * c - 1) / (kBW * c) < sm_total / c / 2) tn = 128;
        }
    }
    if (!valid_tn(tn)) return false;
    if (cg == 0) cg = cg_auto;
    pl.tn = tn;
    pl.cg = cg;
    pl.tiles_n = static_cast<int>((N + kBW * cg - 1) / (kBW * cg));
    pl.tiles_t = static_cast<int>((M + tn - 1) / tn);
    const long long tiles = static_cast<long long>(pl.tiles_n) * pl.tiles_t;
    if (tiles <= 0 || tiles > 0x3FFFFFFF) return false;
    const int clusters = sm_total / cg;
    pl.tg = v ? v->transform_groups : 0;
    // Two transform groups keep a narrow tile's weight stream fed; a long run of 256-token tiles is bound by the tensor
    // pipe and the power limit, where the four extra warps only cost (measured 2% under sustained load).
    if (pl.tg == 0) pl.tg = (tn == 256 && tiles >= 2 * clusters) ? 1 : 2;
    if (pl.tg != 1 && pl.tg != 2) return false;
    int splits = v ? v->split_k : 0;
    if (splits == 0) {
        splits = 1;
        if (tiles < 2 * clusters && pl.total_kb >= 4) {
            // Pick the K split that minimises (rounds of work units over the clusters) x (cycles per unit).  Measured on
            // B200: a k-block costs about 870 cycles for tiles up to 128 tokens (issue-bound) and 1150 for 256; a split
            // unit also parks an fp32 partial tile and one unit per tile reads them all back, about 1000 + 180 cycles per
            // token row of the tile (6 us at 64 tokens, 11 us at 128: 256-token tiles are never worth splitting).
            const long long stage_cycles = tn > 128 ? 1150 : 870;
            const long long split_cycles = 1000 + 180LL * tn;
            long long best = -1;
            for (int sp = 1; sp <= pl.total_kb / 2 && sp <= 32; ++sp) {
                const long long rounds = (tiles * sp + clusters - 1) / clusters;
                const long long per_unit = ((pl.total_kb + sp - 1) / sp) * stage_cycles + (sp > 1 ? split_cycles : 300);
                const long long cost = rounds * per_unit;
                if (best < 0 || cost < best) {
                    best = cost;
                    splits = sp;
                }
            }
        }
    const size_t per_split = static_cast<size_t>(tiles) * tn * kBW * cg * sizeof(float);
        const size_t counters = kCounterBytes;
        if (static_cast<size_t>(tiles) * cg * sizeof(int) > kCounterBytes) splits = 1;
        if (ws_known && splits > 1 && counters + per_split * splits > ws_avail) {
            // shrink to what the caller's scratch can hold
            size_t fit = ws_avail > counters ? (ws_avail - counters) / per_split : 0;
            splits = fit >= 2 ? static_cast<int>(fit) : 1;
        }
    }
    if (splits < 1 || splits > pl.total_kb) return false;
    if (splits > 1 && static_cast<size_t>(tiles) * cg * sizeof(int) > kCounterBytes) return false;
    pl.splits = splits;
    pl.num_units = static_cast<int>(tiles) * splits;
    pl.counter_bytes = splits > 1 ? kCounterBytes : 0;
    pl.ws_bytes = splits > 1 ? pl.counter_bytes + static_cast<size_t>(tiles) * splits * tn * kBW * cg * sizeof(float) : 0;
    pl.max_ctas = v ? v->max_ctas : 0;
    *out = pl;
    return true;
}

template <int TN, int CG, int TG, int OB = 1, bool EXT = false>
static cudaError_t launch_variant(const CUtensorMap& tw, const CUtensorMap& ta, const OutMaps& tc, const LoraMaps& tl, const MmParams& p, int grid,
                                  cudaStream_t stream) {
    using C = Cfg<TN, CG, OB>;
    auto kernel = scaled_mm_kernel<TN, CG, TG, OB, EXT>;
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
    cfg.blockDim = dim3(32 * (kEpilogueWarps + 4 * TG + 2 + Cfg<TN, CG>::kIssuers), 1, 1);
    cfg.dynamicSmemBytes = C::kSmemBytes;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = CG;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    // the CTAs may become resident and set up while the previous kernel on the stream drains; see pdl_wait_for_previous_kernel
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = getenv("FEATHER_NO_PDL") == nullptr ? 1 : 0;
    cfg.attrs = attr;
    cfg.numAttrs = 2;
    return cudaLaunchKernelEx(&cfg, kernel, tw, ta, tc, tl, p);
}

template <int TN, bool EXT>
cudaError_t launch_tn(int cg, int tg, bool deep_staging, const CUtensorMap& tw, const CUtensorMap& ta, const OutMaps& tc, const LoraMaps& tl,
                             const MmParams& p, int grid, cudaStream_t s) {
    if constexpr (TN == 256 && !EXT) {
        // pairs of 256-token tiles whose blocks also cross NVLink: two staging buffers per epilogue group
        if (deep_staging && cg == 2) return tg == 1 ? launch_variant<TN, 2, 1, 2>(tw, ta, tc, tl, p, grid, s) : launch_variant<TN, 2, 2, 2>(tw, ta, tc, tl, p, grid, s);
    }
    if (cg == 1) return tg == 1 ? launch_variant<TN, 1, 1, 1, EXT>(tw, ta, tc, tl, p, grid, s) : launch_variant<TN, 1, 2, 1, EXT>(tw, ta, tc, tl, p, grid, s);
    return tg == 1 ? launch_variant<TN, 2, 1, 1, EXT>(tw, ta, tc, tl, p, grid, s) : launch_variant<TN, 2, 2, 1, EXT>(tw, ta, tc, tl, p, grid, s);
}

// The extended instantiations (EXT = true) are compiled in a translation unit of their own (scaled_mm_ext.cu includes this
// file with FEATHER_TU_EXT defined and stops after the explicit instantiations below), so the two halves build in parallel.
#define FEATHER_FOR_EACH_TN(X) X(16) X(32) X(64) X(128) X(192) X(256)
#ifdef FEATHER_TU_EXT
#define FEATHER_INSTANTIATE(TN_) \
    template cudaError_t launch_tn<TN_, true>(int, int, bool, const CUtensorMap&, const CUtensorMap&, const OutMaps&, const LoraMaps&, const MmParams&, int, cudaStream_t);
FEATHER_FOR_EACH_TN(FEATHER_INSTANTIATE)
#else
#define FEATHER_DECLARE(TN_) \
    extern template cudaError_t launch_tn<TN_, true>(int, int, bool, const CUtensorMap&, const CUtensorMap&, const OutMaps&, const LoraMaps&, const MmParams&, int, cudaStream_t);
FEATHER_FOR_EACH_TN(FEATHER_DECLARE)
#endif

#ifndef FEATHER_TU_EXT
int small_m_launch(const void* a, const uint8_t* w, const float* scale, const void* bias, void* c, int64_t M, int64_t N, int64_t K, int64_t ldc,
                   int output_dtype, int flip_final, int sms, void* workspace, size_t workspace_bytes, cudaStream_t stream);   // small_m.cu
size_t small_m_workspace_bytes(int64_t M, int64_t N, int64_t K, int sms);                                                    // small_m.cu

// Operand and result types beyond the reference's fp16 x e5m2 -> out dtype.
struct Types {
    bool a_bf16 = false;     // activations are bf16
    bool w_e4m3 = false;     // weights are fp8e4m3fn
    int final_dtype = -1;    // dtype stored (FEATHER_OUT_*); -1: the output dtype itself
    // un-merged LoRA term folded into the accumulator (null: none): t = T' [M, R], lb = B' [R/8, N, 8], both fp16
    const void* lora_t = nullptr;
    const void* lora_b = nullptr;
    int64_t lora_rank = 0;
};

// Bandwidth-bound end: the register-streaming kernel, unless the caller pinned a tensor-memory variant or the output goes to
// several buffers.  Up to 16 tokens always; up to 24 tokens for weights of at most 32 MB, where the tensor-memory kernel's
// fixed cost (pipeline fill and drain, about 7 us) weighs more than the streaming kernel's extra MMAs (measured at 17-24 tokens:
// 11.7 against 15.3 us for 5120 x 5120, 10.9 against 14.5 us for 3072 x 9216, but 23.3 against 21.7 us for 5120 x 13824);
// up to 32 tokens on request.  split_k = 1 only says "no workspace" (the reference-ABI launcher passes it): the streaming
// kernel never needs a workspace to be correct, so that alone pins nothing.
static bool takes_streaming_kernel(const feather_mm_variant* variant, int64_t M, int64_t N, int64_t K, int n_extra) {
    const int which = variant ? variant->kernel : FEATHER_KERNEL_AUTO;
    const bool pinned = variant && (variant->tokens_tile || variant->cta_pair || variant->split_k > 1 || variant->transform_groups);
    const bool small_weight = N * K <= (int64_t(32) << 20);
    const bool by_choice = which == FEATHER_KERNEL_AUTO && !pinned && (M <= 16 || (M <= 24 && small_weight));
    return (which == FEATHER_KERNEL_STREAM || by_choice) && n_extra == 0 && M <= 32;
}

static int scaled_mm_impl(const void* a, const uint8_t* b, const float* scale, const void* bias, void* c, int64_t M, int64_t N,
                          int64_t K, int64_t ldc, int output_dtype, const feather_mm_variant* variant, void* workspace,
                          size_t workspace_bytes, int* status_dev, cudaStream_t stream, void* const* extra_dst = nullptr, int n_extra = 0,
                          int64_t scatter_rows = 0, Types types = Types()) {
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
    // Bandwidth-bound end (a few tokens): the register-streaming kernel, unless the caller pinned a tensor-memory variant.
    const int which = variant ? variant->kernel : 0;
    if (which != FEATHER_KERNEL_AUTO && which != FEATHER_KERNEL_TMEM && which != FEATHER_KERNEL_STREAM)
        return set_error(FEATHER_ERR_BAD_ARGUMENT, "variant.kernel must be 0 (auto), 1 (tensor memory) or 2 (streaming)");
    if (which == FEATHER_KERNEL_STREAM && M > 32) return set_error(FEATHER_ERR_UNSUPPORTED, "the streaming kernel handles at most 32 tokens");

    if (n_extra < 0 || n_extra > kMaxDst - 1) return set_error(FEATHER_ERR_BAD_ARGUMENT, "at most %d output buffers", kMaxDst);
    for (int d = 0; d < n_extra; ++d)
        if (extra_dst == nullptr || extra_dst[d] == nullptr || (reinterpret_cast<uintptr_t>(extra_dst[d]) & 15u) != 0)
            return set_error(FEATHER_ERR_BAD_ARGUMENT, "every output buffer must be non-null and 16-byte aligned");
    if (types.final_dtype != -1 && types.final_dtype != FEATHER_OUT_FP16 && types.final_dtype != FEATHER_OUT_BF16)
        return set_error(FEATHER_ERR_BAD_ARGUMENT, "final_dtype must be -1 (same as output_dtype), 0 (fp16) or 1 (bf16)");
    const int flip_final = (types.final_dtype != -1 && types.final_dtype != output_dtype) ? 1 : 0;
    // the streaming kernel multiplies fp16 activations by e5m2 weights only; the other operand types take the tensor-memory kernel
    const bool lora = types.lora_t != nullptr || types.lora_b != nullptr || types.lora_rank != 0;
    if (lora) {
        if (types.lora_t == nullptr || types.lora_b == nullptr || types.lora_rank <= 0 || types.lora_rank % kSubK != 0 || types.lora_rank > 4096)
            return set_error(FEATHER_ERR_BAD_ARGUMENT, "LoRA term: t and lb must not be null and the rank must be a positive multiple of %d (pad with zeros)", kSubK);
        if ((reinterpret_cast<uintptr_t>(types.lora_t) & 15u) != 0 || (reinterpret_cast<uintptr_t>(types.lora_b) & 15u) != 0)
            return set_error(FEATHER_ERR_BAD_ARGUMENT, "LoRA term: t and lb must be 16-byte aligned");
        if (n_extra != 0 || scatter_rows != 0) return set_error(FEATHER_ERR_UNSUPPORTED, "the LoRA term is not combined with sharded outputs");
    }
    const bool plain_operands = !types.a_bf16 && !types.w_e4m3 && !lora;
    if (plain_operands && takes_streaming_kernel(variant, M, N, K, n_extra))
        return small_m_launch(a, b, scale, bias, c, M, N, K, ldc, output_dtype, flip_final, sms, workspace, workspace_bytes, stream);
    if (which == FEATHER_KERNEL_STREAM)
        return set_error(FEATHER_ERR_UNSUPPORTED, "the streaming kernel writes one output buffer and takes fp16 activations and e5m2 weights");
    Plan pl;
    feather_mm_variant lora_variant{};
    if (lora) {
        // the low-rank blocks follow the weight's k-blocks of a tile, so the tile's K is not split across work units
        if (variant) lora_variant = *variant;
        if (lora_variant.split_k > 1) return set_error(FEATHER_ERR_UNSUPPORTED, "the LoRA term needs a variant without a K split");
        lora_variant.split_k = 1;
        variant = &lora_variant;
    }
    if (!make_plan(M, N, K, variant, workspace ? workspace_bytes : 0, true, sms, &pl))
        return set_error(FEATHER_ERR_UNSUPPORTED, "unsupported kernel variant");
    if (pl.splits > 1) {
        if (workspace == nullptr || workspace_bytes < pl.ws_bytes)
            return set_error(FEATHER_ERR_WORKSPACE, "split-K variant needs a larger workspace");
        if ((reinterpret_cast<uintptr_t>(workspace) & 15u) != 0) return set_error(FEATHER_ERR_BAD_ARGUMENT, "workspace must be 16-byte aligned");
    }
    // Upcasting to bf16 or from e4m3 takes several instructions per pair where e5m2 -> fp16 takes one `prmt`: with a single
    // transform group the upcast then sets the pace of 256-token tiles (measured 4.7-6.0 ms against 3.6 ms with two groups on the
    // Wan ffn-up shape), so those operand types get two groups unless the caller pinned the number.
    const bool slow_upcast = types.a_bf16 || types.w_e4m3;
    const int tg = (slow_upcast && !(variant && variant->transform_groups != 0)) ? 2 : pl.tg;

    EncodeTiledFn encode = encode_tiled_fn();
    if (encode == nullptr) return set_error(FEATHER_ERR_NO_DEVICE, "cuTensorMapEncodeTiled is not available from the driver");

    CUtensorMap tmap_w, tmap_a;
    OutMaps tmap_c;
    memset(&tmap_c, 0, sizeof(tmap_c));
    // TMA stores need 16-byte aligned output rows; otherwise (odd ldc, split-K) the epilogue stores 2 bytes at a time
    const bool tma_store = pl.splits == 1 && (ldc % 8) == 0 && (reinterpret_cast<uintptr_t>(c) & 15u) == 0;
    if (n_extra > 0 && !tma_store)
        return set_error(FEATHER_ERR_UNSUPPORTED, "several output buffers need 16-byte aligned rows (ldc %% 8 == 0) and a variant without split-K");
    {
        // W as 8-byte elements: one k16-block plane is a row of 2N elements (n-major, 16 B per n), so the 128 n of a tile
        // are 2048 contiguous bytes = 256 elements.  A box is 8 planes x 256 elements and lands as [8][128 n][16 B].
        // (A byte-typed box with a 16-byte inner extent would make the copy engine issue 512 16-byte rows per stage.)
        const CUresult r = cached_tmap(encode, &tmap_w, 0, CU_TENSOR_MAP_DATA_TYPE_UINT64, b, static_cast<uint64_t>(N) * 2,
                                       static_cast<uint64_t>(K / 16), static_cast<uint64_t>(N) * 16, kBW * 2, kKSteps, CU_TENSOR_MAP_SWIZZLE_NONE,
                                       CU_TENSOR_MAP_L2_PROMOTION_L2_256B);
        if (r != CUDA_SUCCESS) return set_error(FEATHER_ERR_CUDA, "cuTensorMapEncodeTiled(W) failed with CUresult %d", static_cast<int>(r));
    }
    // Row-sharded destinations (scatter_rows > 0): buffer d receives the blocks of token rows [d * scatter_rows, (d + 1) * scatter_rows)
    // and is described as a tensor of scatter_rows rows, so a block must not straddle two owners.
    if (scatter_rows < 0 || (scatter_rows > 0 && (scatter_rows % 32 != 0 || scatter_rows * (1 + n_extra) < M || scatter_rows * n_extra >= M || !tma_store)))
        return set_error(FEATHER_ERR_BAD_ARGUMENT,
                         "row-sharded output: rows per buffer must be a positive multiple of 32, the buffers must cover M, rows must be 16-byte aligned");
    const bool a3d = K % kSubK == 0;
    const bool c3d = N % 64 == 0;
    {
        // A as (K, M) fp16; a box is one sub-tile, 64 k x (tokens per CTA), 128-byte swizzle; rows beyond M and k beyond K read as zero.
        // When K is a multiple of 64 the same memory is described as (64 k, M, K/64) instead, so that one copy of a
        // (64, tokens, 2) box fetches both sub-tiles of a k-block: the producer thread pays per instruction, not per byte.
        // A k-block past the end of K reads as zero in either form (it lies outside the tensor, never in the next row).
        const CUresult r = a3d ? cached_tmap(encode, &tmap_a, 3, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, a, kSubK, static_cast<uint64_t>(M),
                                             static_cast<uint64_t>(K) * 2, kSubK, static_cast<uint32_t>(pl.tn / pl.cg), CU_TENSOR_MAP_SWIZZLE_128B,
                                             CU_TENSOR_MAP_L2_PROMOTION_L2_256B, static_cast<uint64_t>(K / kSubK), kSubK * 2, kSubTiles)
                               : cached_tmap(encode, &tmap_a, 1, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, a, static_cast<uint64_t>(K), static_cast<uint64_t>(M),
                                             static_cast<uint64_t>(K) * 2, kSubK, static_cast<uint32_t>(pl.tn / pl.cg), CU_TENSOR_MAP_SWIZZLE_128B,
                                             CU_TENSOR_MAP_L2_PROMOTION_L2_256B);
        if (r != CUDA_SUCCESS) return set_error(FEATHER_ERR_CUDA, "cuTensorMapEncodeTiled(A) failed with CUresult %d", static_cast<int>(r));
    }
    if (tma_store) {
        // C as (N, M) 16-bit with row pitch ldc; a box is 64 n x (up to 32) token rows in the 128-byte swizzle, clipped at N and M
        for (int d = 0; d <= n_extra; ++d) {
            void* const dst = d == 0 ? c : extra_dst[d - 1];
            // When N is a multiple of 64 the same memory is described as (64 n, M, N/64), so one store of a (64, rows, 2) box
            // writes both staged tiles: the storing thread pays per instruction (and per destination GPU).
            const uint32_t rows = static_cast<uint32_t>(pl.tn < 32 ? pl.tn : 32);
            // a row-sharded destination holds its owner's token rows only (the last one possibly fewer): rows beyond are clipped
            const int64_t c_rows = scatter_rows > 0 ? (M - d * scatter_rows < scatter_rows ? M - d * scatter_rows : scatter_rows) : M;
            const CUresult r = c3d ? cached_tmap(encode, &tmap_c.m[d], 4, CU_TENSOR_MAP_DATA_TYPE_UINT16, dst, 64, static_cast<uint64_t>(c_rows),
                                                 static_cast<uint64_t>(ldc) * 2, 64, rows, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE,
                                                 static_cast<uint64_t>(N / 64), 128, 2)
                                   : cached_tmap(encode, &tmap_c.m[d], 2, CU_TENSOR_MAP_DATA_TYPE_UINT16, dst, static_cast<uint64_t>(N),
                                                 static_cast<uint64_t>(c_rows), static_cast<uint64_t>(ldc) * 2, 64, rows, CU_TENSOR_MAP_SWIZZLE_128B,
                                                 CU_TENSOR_MAP_L2_PROMOTION_NONE);
            if (r != CUDA_SUCCESS) return set_error(FEATHER_ERR_CUDA, "cuTensorMapEncodeTiled(C) failed with CUresult %d", static_cast<int>(r));
        }
    }

    LoraMaps tmap_l;
    memset(&tmap_l, 0, sizeof(tmap_l));
    if (lora) {
        const uint64_t R = static_cast<uint64_t>(types.lora_rank);
        CUresult r = cached_tmap(encode, &tmap_l.t, 5, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, types.lora_t, R, static_cast<uint64_t>(M), R * 2, kSubK,
                                 static_cast<uint32_t>(pl.tn / pl.cg), CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B);
        if (r != CUDA_SUCCESS) return set_error(FEATHER_ERR_CUDA, "cuTensorMapEncodeTiled(LoRA T) failed with CUresult %d", static_cast<int>(r));
        r = cached_tmap(encode, &tmap_l.b, 6, CU_TENSOR_MAP_DATA_TYPE_UINT64, types.lora_b, static_cast<uint64_t>(N) * 2, R / 8, static_cast<uint64_t>(N) * 16,
                        kBW * 2, kKSteps, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B);
        if (r != CUDA_SUCCESS) return set_error(FEATHER_ERR_CUDA, "cuTensorMapEncodeTiled(LoRA B) failed with CUresult %d", static_cast<int>(r));
    }

    MmParams p{};
    p.lora_blocks = lora ? static_cast<int>(types.lora_rank / kSubK) : 0;
    p.a3d = a3d ? 1 : 0;
    p.c3d = c3d ? 1 : 0;
    p.tma_store = tma_store ? 1 : 0;
    p.n_dst = 1 + n_extra;
    p.scatter_rows = static_cast<int>(scatter_rows);
    // variant.staging: 0 = two staging buffers per group whenever blocks go to more than one buffer, 1 = never, 2 = always
    const int staging_mode = variant ? variant->staging : 0;
    if (staging_mode < 0 || staging_mode > 2) return set_error(FEATHER_ERR_BAD_ARGUMENT, "variant.staging must be 0 (auto), 1 (one buffer) or 2 (two buffers)");
    const bool deep_staging = tma_store && (staging_mode == 2 || (staging_mode == 0 && n_extra > 0));
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
    p.flip_final = flip_final;
    p.a_bf16 = types.a_bf16 ? 1 : 0;
    p.w_e4m3 = types.w_e4m3 ? 1 : 0;
    p.scale_mul = types.w_e4m3 ? 256.0f : 1.0f;
    // Read once per process.
    static const bool env_stats = getenv("FEATHER_STATS") != nullptr;
    // FEATHER_STATS=1: the caller's status buffer is at least 8 + 32*8 bytes and receives the cycle counters of CTA 0 after the status word
    if (status_dev != nullptr && env_stats) p.stats = reinterpret_cast<long long*>(status_dev + 2);
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

    // the plain kernel, or the one with the run-time switches for operand types, low-rank blocks and row-sharded destinations
    const bool ext = types.a_bf16 || types.w_e4m3 || lora || scatter_rows > 0;
    cudaError_t e = cudaErrorInvalidValue;
    switch (pl.tn) {
        case 16: e = ext ? launch_tn<16, true>(pl.cg, tg, deep_staging, tmap_w, tmap_a, tmap_c, tmap_l, p, grid, stream) : launch_tn<16, false>(pl.cg, tg, deep_staging, tmap_w, tmap_a, tmap_c, tmap_l, p, grid, stream); break;
        case 32: e = ext ? launch_tn<32, true>(pl.cg, tg, deep_staging, tmap_w, tmap_a, tmap_c, tmap_l, p, grid, stream) : launch_tn<32, false>(pl.cg, tg, deep_staging, tmap_w, tmap_a, tmap_c, tmap_l, p, grid, stream); break;
        case 64: e = ext ? launch_tn<64, true>(pl.cg, tg, deep_staging, tmap_w, tmap_a, tmap_c, tmap_l, p, grid, stream) : launch_tn<64, false>(pl.cg, tg, deep_staging, tmap_w, tmap_a, tmap_c, tmap_l, p, grid, stream); break;
        case 128: e = ext ? launch_tn<128, true>(pl.cg, tg, deep_staging, tmap_w, tmap_a, tmap_c, tmap_l, p, grid, stream) : launch_tn<128, false>(pl.cg, tg, deep_staging, tmap_w, tmap_a, tmap_c, tmap_l, p, grid, stream); break;
        case 192: e = ext ? launch_tn<192, true>(pl.cg, tg, deep_staging, tmap_w, tmap_a, tmap_c, tmap_l, p, grid, stream) : launch_tn<192, false>(pl.cg, tg, deep_staging, tmap_w, tmap_a, tmap_c, tmap_l, p, grid, stream); break;
        case 256: e = ext ? launch_tn<256, true>(pl.cg, tg, deep_staging, tmap_w, tmap_a, tmap_c, tmap_l, p, grid, stream) : launch_tn<256, false>(pl.cg, tg, deep_staging, tmap_w, tmap_a, tmap_c, tmap_l, p, grid, stream); break;
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

extern "C" int feather_scaled_mm_typed(const void* a, int a_dtype, const uint8_t* b_prepacked, int b_dtype, const float* scale, const void* bias, void* c,
                                       int64_t M, int64_t N, int64_t K, int64_t ldc, int output_dtype, int final_dtype,
                                       const feather_mm_variant* variant, void* workspace, size_t workspace_bytes, int* status_dev,
                                       feather_stream_t stream) {
    if (a_dtype != FEATHER_SRC_FP16 && a_dtype != FEATHER_SRC_BF16)
        return set_error(FEATHER_ERR_BAD_ARGUMENT, "a_dtype must be %d (bf16) or %d (fp16)", FEATHER_SRC_BF16, FEATHER_SRC_FP16);
    if (b_dtype != FEATHER_B_E5M2 && b_dtype != FEATHER_B_E4M3)
        return set_error(FEATHER_ERR_BAD_ARGUMENT, "b_dtype must be %d (fp8e4m3fn) or %d (fp8e5m2)", FEATHER_B_E4M3, FEATHER_B_E5M2);
    Types t;
    t.a_bf16 = a_dtype == FEATHER_SRC_BF16;
    t.w_e4m3 = b_dtype == FEATHER_B_E4M3;
    t.final_dtype = final_dtype;
    return scaled_mm_impl(a, b_prepacked, scale, bias, c, M, N, K, ldc, output_dtype, variant, workspace, workspace_bytes, status_dev,
                          static_cast<cudaStream_t>(stream), nullptr, 0, 0, t);
}

extern "C" int feather_scaled_mm_lora(const void* a, int a_dtype, const uint8_t* b_prepacked, const float* scale, const void* bias, void* c, int64_t M,
                                      int64_t N, int64_t K, int64_t ldc, int output_dtype, int final_dtype, const void* t, const void* lb_prepacked,
                                      int64_t rank, const feather_mm_variant* variant, int* status_dev, feather_stream_t stream) {
    if (a_dtype != FEATHER_SRC_FP16 && a_dtype != FEATHER_SRC_BF16)
        return set_error(FEATHER_ERR_BAD_ARGUMENT, "a_dtype must be %d (bf16) or %d (fp16)", FEATHER_SRC_BF16, FEATHER_SRC_FP16);
    Types ty;
    ty.a_bf16 = a_dtype == FEATHER_SRC_BF16;
    ty.final_dtype = final_dtype;
    ty.lora_t = t;
    ty.lora_b = lb_prepacked;
    ty.lora_rank = rank;
    return scaled_mm_impl(a, b_prepacked, scale, bias, c, M, N, K, ldc, output_dtype, variant, nullptr, 0, status_dev, static_cast<cudaStream_t>(stream),
                          nullptr, 0, 0, ty);
}

extern "C" int feather_scaled_mm_multi(const void* a, const uint8_t* b_prepacked, const float* scale, const void* bias, void* const* c_list_host,
                                       int n_dst, int64_t M, int64_t N, int64_t K, int64_t ldc, int output_dtype, const feather_mm_variant* variant,
                                       int* status_dev, feather_stream_t stream) {
    if (c_list_host == nullptr || n_dst < 1) return set_error(FEATHER_ERR_BAD_ARGUMENT, "c_list_host must hold at least one output buffer");
    feather_mm_variant v{};
    if (variant) v = *variant;
    v.split_k = 1;                      // every rank must add the k-blocks in the same order, and the stores go through TMA
    v.kernel = FEATHER_KERNEL_TMEM;
    return scaled_mm_impl(a, b_prepacked, scale, bias, c_list_host[0], M, N, K, ldc, output_dtype, &v, nullptr, 0, status_dev,
                          static_cast<cudaStream_t>(stream), c_list_host + 1, n_dst - 1);
}

extern "C" int feather_scaled_mm_scatter(const void* a, const uint8_t* b_prepacked, const float* scale, const void* bias, void* const* c_list_host,
                                         int n_dst, int64_t rows_per_dst, int64_t M, int64_t N, int64_t K, int64_t ldc, int output_dtype,
                                         const feather_mm_variant* variant, int* status_dev, feather_stream_t stream) {
    if (c_list_host == nullptr || n_dst < 1) return set_error(FEATHER_ERR_BAD_ARGUMENT, "c_list_host must hold at least one output buffer");
    if (rows_per_dst <= 0) return set_error(FEATHER_ERR_BAD_ARGUMENT, "rows_per_dst must be positive");
    feather_mm_variant v{};
    if (variant) v = *variant;
    v.split_k = 1;                      // blocks leave through TMA stores, which a K split through the workspace does not use
    v.kernel = FEATHER_KERNEL_TMEM;
    return scaled_mm_impl(a, b_prepacked, scale, bias, c_list_host[0], M, N, K, ldc, output_dtype, &v, nullptr, 0, status_dev,
                          static_cast<cudaStream_t>(stream), c_list_host + 1, n_dst - 1, rows_per_dst);
}

extern "C" int launch_scaled_mm(const void* a, const uint8_t* b_prepacked, const float* scale, const uint16_t* bias, uint16_t* c,
                                int64_t M, int64_t N, int64_t K, int has_scale, int has_bias, int, int, int, int, int, int b_dtype,
                                int output_dtype, feather_stream_t stream) {
    if (b_dtype != FEATHER_B_E5M2 && b_dtype != FEATHER_B_E4M3) {
        set_error(FEATHER_ERR_UNSUPPORTED, "b_dtype must be 0 (fp8e4m3fn) or 1 (fp8e5m2)");
        return 0;
    }
    feather_mm_variant v{};
    v.split_k = 1;   // no workspace through this signature
    Types t;
    t.w_e4m3 = b_dtype == FEATHER_B_E4M3;
    const int st = scaled_mm_impl(a, b_prepacked, has_scale ? scale : nullptr, has_bias ? bias : nullptr, c, M, N, K, N, output_dtype, &v,
                                  nullptr, 0, nullptr, static_cast<cudaStream_t>(stream), nullptr, 0, 0, t);
    return st == FEATHER_OK ? 1 : 0;
}

// ------------------------------------------------------------------------------------------------
// Entry point for callers that cannot allocate device memory: the split-K scratch is a fixed array that is part of
// this library's device image.
// ------------------------------------------------------------------------------------------------
constexpr size_t kStaticScratchBytes = FEATHER_STATIC_SCRATCH_BYTES;
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

// In host code `g_static_scratch` is only a handle for the runtime, not a device address: the address a kernel can use comes
// from cudaGetSymbolAddress, asked once per device with that device current.
static int static_scratch_of_current_device(void** out) {
    static std::mutex mu;
    static void* cached[64];
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess || dev < 0 || dev >= 64) return set_error(FEATHER_ERR_NO_DEVICE, "no current CUDA device");
    std::lock_guard<std::mutex> lock(mu);
    if (cached[dev] == nullptr) {
        void* ptr = nullptr;
        e = cudaGetSymbolAddress(&ptr, g_static_scratch);
        if (e != cudaSuccess || ptr == nullptr)
            return set_error(FEATHER_ERR_CUDA, "cudaGetSymbolAddress(static scratch) failed: %s", cudaGetErrorString(e));
        cached[dev] = ptr;
    }
    *out = cached[dev];
    return FEATHER_OK;
}

extern "C" size_t feather_scaled_mm_static_scratch_bytes(void) { return kStaticScratchBytes; }

extern "C" int feather_scaled_mm_static(const void* a, const uint8_t* b_prepacked, const float* scale, const void* bias, void* c, int64_t M,
                                        int64_t N, int64_t K, int64_t ldc, int output_dtype, const feather_mm_variant* variant,
                                        int* status_dev, feather_stream_t stream_) {
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    if (M < 0 || N <= 0 || K <= 0) return set_error(FEATHER_ERR_BAD_ARGUMENT, "M, N, K must be positive");
    if (M == 0) return FEATHER_OK;
    // The register-streaming kernel splits K across CTAs through the scratch when the weight's columns alone cannot fill the
    // SMs; it gets the built-in array like the tensor-memory kernel below, with the counter block cleared first.
    if (takes_streaming_kernel(variant, M, N, K, 0)) {
        void* scratch = nullptr;
        if (int st = static_scratch_of_current_device(&scratch)) return st;
        const cudaError_t e = cudaMemsetAsync(scratch, 0, kCounterBytes, stream);
        if (e != cudaSuccess) return set_error(FEATHER_ERR_CUDA, "clearing the tile counters failed: %s", cudaGetErrorString(e));
        return scaled_mm_impl(a, b_prepacked, scale, bias, c, M, N, K, ldc, output_dtype, variant, scratch, kStaticScratchBytes, status_dev, stream);
    }
    const int sms = sm_count_of_current_device();
    if (sms <= 0) return set_error(FEATHER_ERR_NO_DEVICE, "no CUDA device");
    // The same plan feather_scaled_mm_ex makes when it is handed a workspace of this size: a K split the library chose
    // itself is shrunk to what the array holds, and only a split the caller pinned can ask for more than there is.
    Plan pl;
    if (!make_plan(M, N, K, variant, kStaticScratchBytes, true, sms, &pl)) return set_error(FEATHER_ERR_UNSUPPORTED, "unsupported kernel variant");
    if (pl.ws_bytes > kStaticScratchBytes)
        return set_error(FEATHER_ERR_WORKSPACE,
                         "this variant needs %zu bytes of split-K scratch but the built-in scratch holds %zu; use feather_scaled_mm_ex with "
                         "a caller-provided workspace, or pass a variant with a smaller split_k",
                         pl.ws_bytes, kStaticScratchBytes);
    void* scratch = nullptr;
    if (pl.splits > 1) {
        if (int st = static_scratch_of_current_device(&scratch)) return st;
        // Every call shares the array and it keeps the previous call's contents.  Only the tile counters have to start at
        // zero; partial tiles are fully written before they are read.
        const size_t counter_bytes = static_cast<size_t>(pl.tiles_n) * pl.tiles_t * pl.cg * sizeof(int);
        const cudaError_t e = cudaMemsetAsync(scratch, 0, counter_bytes, stream);
        if (e != cudaSuccess) return set_error(FEATHER_ERR_CUDA, "clearing the tile counters failed: %s", cudaGetErrorString(e));
    }
    return scaled_mm_impl(a, b_prepacked, scale, bias, c, M, N, K, ldc, output_dtype, variant, scratch, scratch ? kStaticScratchBytes : 0, status_dev,
                          stream);
}

extern "C" size_t feather_scaled_mm_workspace_bytes(int64_t M, int64_t N, int64_t K, const feather_mm_variant* variant) {
    if (M <= 0 || N <= 0 || K <= 0) return 0;
    int sms = sm_count_of_current_device();
    if (takes_streaming_kernel(variant, M, N, K, 0)) return small_m_workspace_bytes(M, N, K, sms);
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
    out->kernel = takes_streaming_kernel(nullptr, M, N, K, 0) ? FEATHER_KERNEL_STREAM : FEATHER_KERNEL_TMEM;
    out->staging = 0;
    return FEATHER_OK;
}
#else
}  // namespace feather
#endif  // FEATHER_TU_EXT
