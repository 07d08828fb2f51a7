/*
 * bench_scaled_mm.c - a plain C program that times the mixed-precision GEMM through the C ABI of libfeather_b200,
 * with no Python and no PyTorch in the process.
 *
 * Counterpart of the reference's cpp_benchmarks/benchmark_scaled_mm_hip.cpp:27-45 (the extern "C" launcher declaration) and
 * :197-243 (10 warm-up launches, then 100 launches each bracketed by events; mean, standard deviation, TFLOPS with
 * FLOPs = 2 M N K as in :166,258).  It calls `launch_scaled_mm`, the entry point that keeps the reference's argument order,
 * and, with `--ex`, `feather_scaled_mm_ex` with a workspace (so a K split may be chosen).
 *
 * Build (see build.py: build_cbench):
 *   cc -std=c99 -O2 bench_scaled_mm.c -I<repo>/include -I$CUDA/include -L<pkg> -lfeather_b200 -L$CUDA/lib64 -lcudart -lm
 * Usage:  bench_scaled_mm [M N K] [--fp16] [--bias] [--ex] [--iters n] [--check]
 *   --check  compares 64 output elements with a host computation of the same sum (fp32 accumulation) and fails beyond 1e-2 * rms.
 */
#include <cuda_runtime_api.h>
#include <math.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include "feather_b200.h"

#define CHECK_CUDA(call)                                                                          \
    do {                                                                                          \
        cudaError_t e_ = (call);                                                                  \
        if (e_ != cudaSuccess) {                                                                  \
            fprintf(stderr, "%s failed: %s\n", #call, cudaGetErrorString(e_));                    \
            return 2;                                                                             \
        }                                                                                         \
    } while (0)

/* xorshift: the same numbers on every run */
static uint32_t rng_state = 0x12345678u;
static uint32_t rng_next(void) {
    uint32_t x = rng_state;
    x ^= x << 13;
    x ^= x >> 17;
    x ^= x << 5;
    return rng_state = x;
}
static float rng_uniform(void) { return (float)(rng_next() >> 8) * (1.0f / 16777216.0f) * 2.0f - 1.0f; }

/* float -> fp16 bits, round to nearest even (finite inputs well inside the fp16 range) */
static uint16_t f32_to_f16(float f) {
    uint32_t u;
    memcpy(&u, &f, 4);
    uint32_t sign = (u >> 16) & 0x8000u;
    int32_t exp = (int32_t)((u >> 23) & 0xFF) - 127 + 15;
    uint32_t man = u & 0x7FFFFFu;
    if (exp <= 0) return (uint16_t)sign; /* tiny: flush (inputs here never are) */
    uint32_t half = (uint32_t)exp << 10 | man >> 13;
    uint32_t rest = man & 0x1FFFu;
    if (rest > 0x1000u || (rest == 0x1000u && (half & 1u))) half++;
    return (uint16_t)(sign | half);
}
static float f16_to_f32(uint16_t h) {
    uint32_t sign = (uint32_t)(h & 0x8000u) << 16, exp = (h >> 10) & 0x1F, man = h & 0x3FFu, u;
    if (exp == 0) {
        float f = (float)man * (1.0f / 16777216.0f); /* man * 2^-24 */
        return sign ? -f : f;
    }
    u = sign | (exp - 15 + 127) << 23 | man << 13;
    float f;
    memcpy(&f, &u, 4);
    return f;
}
static float bf16_to_f32(uint16_t h) {
    uint32_t u = (uint32_t)h << 16;
    float f;
    memcpy(&f, &u, 4);
    return f;
}
/* e5m2 byte -> float: the byte is the high byte of an fp16 */
static float e5m2_to_f32(uint8_t b) { return f16_to_f32((uint16_t)((uint16_t)b << 8)); }

int main(int argc, char** argv) {
    int64_t M = 8192, N = 8192, K = 8192;
    int out_dtype = FEATHER_OUT_BF16, with_bias = 0, use_ex = 0, iters = 100, check = 0, npos = 0;
    for (int i = 1; i < argc; ++i) {
        if (!strcmp(argv[i], "--fp16")) out_dtype = FEATHER_OUT_FP16;
        else if (!strcmp(argv[i], "--bias")) with_bias = 1;
        else if (!strcmp(argv[i], "--ex")) use_ex = 1;
        else if (!strcmp(argv[i], "--check")) check = 1;
        else if (!strcmp(argv[i], "--iters") && i + 1 < argc) iters = atoi(argv[++i]);
        else if (npos == 0) { M = atoll(argv[i]); npos++; }
        else if (npos == 1) { N = atoll(argv[i]); npos++; }
        else if (npos == 2) { K = atoll(argv[i]); npos++; }
    }
    if (M <= 0 || N <= 0 || K <= 0 || K % 16 || iters < 1) {
        fprintf(stderr, "usage: %s [M N K] [--fp16] [--bias] [--ex] [--iters n] [--check]   (K %% 16 == 0)\n", argv[0]);
        return 1;
    }
    printf("libfeather_b200 version %d; M=%lld N=%lld K=%lld out=%s bias=%d entry=%s\n", feather_version(), (long long)M, (long long)N, (long long)K,
           out_dtype == FEATHER_OUT_BF16 ? "bf16" : "fp16", with_bias, use_ex ? "feather_scaled_mm_ex" : "launch_scaled_mm");

    size_t a_elems = (size_t)M * K, w_bytes = (size_t)K * N, c_elems = (size_t)M * N;
    uint16_t* ha = (uint16_t*)malloc(a_elems * 2);
    uint8_t* hw = (uint8_t*)malloc(w_bytes);
    uint16_t* hbias = (uint16_t*)calloc((size_t)N, 2);
    uint16_t* hc = (uint16_t*)malloc(c_elems * 2);
    if (!ha || !hw || !hbias || !hc) return 2;
    for (size_t i = 0; i < a_elems; ++i) ha[i] = f32_to_f16(rng_uniform());
    /* prepacked (K/16, N, 16) e5m2 codes: finite values only (exponent field below 31), both signs */
    for (size_t i = 0; i < w_bytes; ++i) {
        uint32_t r = rng_next();
        hw[i] = (uint8_t)(((r & 0x80u)) | ((r >> 8) % 0x7Bu));
    }
    const float scale = 1.0f / 4096.0f;

    void *da, *dw, *dc, *dbias, *dws;
    float* dscale;
    int* dstatus;
    const size_t ws_bytes = (size_t)64 << 20;
    CHECK_CUDA(cudaMalloc(&da, a_elems * 2));
    CHECK_CUDA(cudaMalloc(&dw, w_bytes));
    CHECK_CUDA(cudaMalloc(&dc, c_elems * 2));
    CHECK_CUDA(cudaMalloc(&dbias, (size_t)N * 2));
    CHECK_CUDA(cudaMalloc((void**)&dscale, 4));
    CHECK_CUDA(cudaMalloc((void**)&dstatus, 4));
    CHECK_CUDA(cudaMalloc(&dws, ws_bytes));
    CHECK_CUDA(cudaMemset(dws, 0, ws_bytes));
    CHECK_CUDA(cudaMemset(dstatus, 0, 4));
    CHECK_CUDA(cudaMemcpy(da, ha, a_elems * 2, cudaMemcpyHostToDevice));
    CHECK_CUDA(cudaMemcpy(dw, hw, w_bytes, cudaMemcpyHostToDevice));
    CHECK_CUDA(cudaMemcpy(dbias, hbias, (size_t)N * 2, cudaMemcpyHostToDevice));
    CHECK_CUDA(cudaMemcpy(dscale, &scale, 4, cudaMemcpyHostToDevice));
    cudaStream_t stream;
    CHECK_CUDA(cudaStreamCreate(&stream));

#define LAUNCH()                                                                                                                            \
    (use_ex ? feather_scaled_mm_ex(da, (const uint8_t*)dw, dscale, with_bias ? dbias : NULL, dc, M, N, K, N, out_dtype, NULL, dws, ws_bytes, \
                                   dstatus, (feather_stream_t)stream) == FEATHER_OK                                                         \
            : launch_scaled_mm(da, (const uint8_t*)dw, dscale, (const uint16_t*)dbias, (uint16_t*)dc, M, N, K, 1, with_bias, 1, 8, 4, 8, 2,  \
                               FEATHER_B_E5M2, out_dtype, (feather_stream_t)stream) == 1)

    for (int i = 0; i < 10; ++i) {
        if (!LAUNCH()) {
            fprintf(stderr, "launch failed: %s\n", feather_last_error_string());
            return 3;
        }
    }
    CHECK_CUDA(cudaStreamSynchronize(stream));
    cudaEvent_t e0, e1;
    CHECK_CUDA(cudaEventCreate(&e0));
    CHECK_CUDA(cudaEventCreate(&e1));
    double sum = 0.0, sumsq = 0.0, best = 1e30;
    for (int i = 0; i < iters; ++i) {
        CHECK_CUDA(cudaEventRecord(e0, stream));
        if (!LAUNCH()) return 3;
        CHECK_CUDA(cudaEventRecord(e1, stream));
        CHECK_CUDA(cudaEventSynchronize(e1));
        float ms = 0.0f;
        CHECK_CUDA(cudaEventElapsedTime(&ms, e0, e1));
        sum += ms;
        sumsq += (double)ms * ms;
        if (ms < best) best = ms;
    }
    int status = 0;
    CHECK_CUDA(cudaMemcpy(&status, dstatus, 4, cudaMemcpyDeviceToHost));
    if (status != 0) {
        fprintf(stderr, "device status word is %d: a kernel gave up on a bounded wait\n", status);
        return 4;
    }
    const double mean = sum / iters, var = sumsq / iters - mean * mean, flops = 2.0 * (double)M * (double)N * (double)K;
    printf("mean %.4f ms  std %.4f ms  min %.4f ms  ->  %.1f TFLOPS (mean), %.1f TFLOPS (best)\n", mean, sqrt(var > 0 ? var : 0), best,
           flops / (mean * 1e-3) / 1e12, flops / (best * 1e-3) / 1e12);

    int rc = 0;
    if (check) {
        CHECK_CUDA(cudaMemcpy(hc, dc, c_elems * 2, cudaMemcpyDeviceToHost));
        double max_err = 0.0, sq = 0.0;
        for (int s = 0; s < 64; ++s) {
            int64_t m = (int64_t)(rng_next() % (uint32_t)M), n = (int64_t)(rng_next() % (uint32_t)N);
            float acc = 0.0f;
            for (int64_t k = 0; k < K; ++k)
                acc += f16_to_f32(ha[m * K + k]) * e5m2_to_f32(hw[((k / 16) * N + n) * 16 + (k % 16)]);
            const float ref = acc * scale;
            const uint16_t bits = hc[m * N + n];
            const float got = out_dtype == FEATHER_OUT_BF16 ? bf16_to_f32(bits) : f16_to_f32(bits);
            const double err = fabs((double)got - (double)ref), ulp = fabs((double)ref) * (out_dtype == FEATHER_OUT_BF16 ? 1.0 / 128 : 1.0 / 1024);
            if (err - ulp > max_err) max_err = err - ulp;
            sq += (double)ref * ref;
        }
        const double rms = sqrt(sq / 64);
        printf("check: 64 sampled outputs, max error beyond one ulp %.3e, rms %.3e -> %s\n", max_err, rms, max_err <= 1e-2 * rms ? "ok" : "FAILED");
        if (max_err > 1e-2 * rms) rc = 5;
    }
    cudaFree(da); cudaFree(dw); cudaFree(dc); cudaFree(dbias); cudaFree(dscale); cudaFree(dstatus); cudaFree(dws);
    free(ha); free(hw); free(hbias); free(hc);
    return rc;
}
