// Low-bit conversion kernels (contract clauses L-1 .. L-6 of the reference's
// gemm/IDENTICAL_LOWBIT_CONTRACT.md) and the int8i32.v1 product.
//
// Reference kernels these replace: bf16_widen_kernel / bf16_narrow_kernel
// (gemm/checks/gemm_lowbit.mojo:166-187), quantize_rows_int8_kernel /
// dequantize_rows_int8_kernel (:435-477), identical_gemm_int8_flat_kernel
// (:480-511). All of them are HBM-bound byte work: 128-bit coalesced loads,
// one pass, grid sized from the element count.
#pragma once
#include "seams.cuh"

namespace b200i {

__global__ void to_bf16_kernel(unsigned short *__restrict__ dst, const float *__restrict__ src, long long count) {
    const long long stride = (long long)gridDim.x * blockDim.x;
    const long long i0 = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    const bool vec = ((reinterpret_cast<uintptr_t>(src) & 15) == 0) && ((reinterpret_cast<uintptr_t>(dst) & 7) == 0);
    const long long quads = vec ? count / 4 : 0;
    for (long long q = i0; q < quads; q += stride) {
        const float4 v = __ldg(reinterpret_cast<const float4 *>(src) + q);
        uint2 w;
        w.x = (unsigned)f32_to_bf16_bits_rne(v.x) | ((unsigned)f32_to_bf16_bits_rne(v.y) << 16);
        w.y = (unsigned)f32_to_bf16_bits_rne(v.z) | ((unsigned)f32_to_bf16_bits_rne(v.w) << 16);
        reinterpret_cast<uint2 *>(dst)[q] = w;
    }
    for (long long i = quads * 4 + i0; i < count; i += stride) dst[i] = f32_to_bf16_bits_rne(src[i]);
}

__global__ void from_bf16_kernel(float *__restrict__ dst, const unsigned short *__restrict__ src, long long count) {
    const long long stride = (long long)gridDim.x * blockDim.x;
    const long long i0 = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    const bool vec = ((reinterpret_cast<uintptr_t>(dst) & 15) == 0) && ((reinterpret_cast<uintptr_t>(src) & 7) == 0);
    const long long quads = vec ? count / 4 : 0;
    for (long long q = i0; q < quads; q += stride) {
        const uint2 w = __ldg(reinterpret_cast<const uint2 *>(src) + q);
        float4 v;
        v.x = __uint_as_float(w.x << 16);
        v.y = __uint_as_float(w.x & 0xFFFF0000u);
        v.z = __uint_as_float(w.y << 16);
        v.w = __uint_as_float(w.y & 0xFFFF0000u);
        reinterpret_cast<float4 *>(dst)[q] = v;
    }
    for (long long i = quads * 4 + i0; i < count; i += stride) dst[i] = bf16_bits_to_f32(src[i]);
}

// One warp per row: the row's absmax after the flush (a maximum is exact and
// order-free, so a shuffle butterfly is as good as any walk), the power-of-two
// exponent, then every value scaled, rounded half-even and clamped.
__global__ void quantize_int8_kernel(signed char *__restrict__ q, int *__restrict__ e, const float *__restrict__ x,
                                     long long rows, long long cols) {
    const int lane = threadIdx.x & 31;
    const long long warp = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const long long nwarps = ((long long)gridDim.x * blockDim.x) >> 5;
    for (long long r = warp; r < rows; r += nwarps) {
        const float *row = x + r * cols;
        float best = 0.f;
        for (long long c = lane; c < cols; c += 32) {
            float v = fabsf(ftz_bits(row[c]));
            if (v > best) best = v; // a NaN never compares greater and is skipped, as in the scalar walk
        }
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) best = fmaxf(best, __shfl_xor_sync(0xFFFFFFFFu, best, off));
        const int ex = int8_row_exponent(best);
        if (lane == 0) e[r] = ex;
        for (long long c = lane; c < cols; c += 32) q[r * cols + c] = quantize_int8_value(row[c], ex);
    }
}

__global__ void dequantize_int8_kernel(float *__restrict__ y, const signed char *__restrict__ q,
                                       const int *__restrict__ e, long long rows, long long cols) {
    const long long stride = (long long)gridDim.x * blockDim.x;
    const long long total = rows * cols;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
        const long long r = i / cols;
        y[i] = dequant_int8_pow2((int)q[i], pow2_f32(__ldg(e + r)));
    }
}

// int32 accumulator to float32 by the pinned spelling: a 20-bit high part and
// a 12-bit low part, both exact, one exact scaling, ONE rounding addition.
__device__ __forceinline__ float i32_to_f32_pinned(int v) {
    const bool neg = v < 0;
    const unsigned mag = neg ? (unsigned)(-(long long)v) : (unsigned)v;
    const float hi = (float)(int)(mag >> 12), lo = (float)(int)(mag & 0xFFFu);
    const float r = __fadd_rn(__fmul_rn(hi, 4096.0f), lo);
    return neg ? -r : r;
}

// int8i32.v1 at OP_NT, one thread per cell: order cannot move a bit of an
// exact integer sum, so the walk uses 4-wide dot products where aligned.
__global__ void gemm_int8_flat_kernel(float *__restrict__ c, const signed char *__restrict__ qa,
                                      const int *__restrict__ ea, const signed char *__restrict__ qb,
                                      const int *__restrict__ eb, int m, int n, int k) {
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (long long)m * n) return;
    const int i = (int)(idx / n), j = (int)(idx % n);
    const signed char *ra = qa + (size_t)i * k, *rb = qb + (size_t)j * k;
    int acc = 0;
    int p = 0;
    if ((k & 3) == 0 && ((reinterpret_cast<uintptr_t>(qa) | reinterpret_cast<uintptr_t>(qb)) & 3) == 0)
        for (; p + 3 < k; p += 4)
            acc = __dp4a(*reinterpret_cast<const int *>(ra + p), *reinterpret_cast<const int *>(rb + p), acc);
    for (; p < k; p++) acc += (int)ra[p] * (int)rb[p];
    const long long esum = (long long)ea[i] + (long long)eb[j];
    const int eclamped = esum > 1000 ? 1000 : (esum < -1000 ? -1000 : (int)esum);
    c[idx] = nan_canon(ftz_bits(__fmul_rn(i32_to_f32_pinned(acc), pow2_f32(eclamped))));
}

// Peak-rate probe for the roofline denominator: 16 independent accumulator
// chains per thread of bare fused multiply-adds, scalar (packed == 0) or as
// fma.rn.f32x2 pairs (packed == 1). 2 * 16 * iters flops per thread (scalar),
// twice that packed. The sum is stored so the chains cannot be removed.
__global__ void ffma_probe_kernel(float *out, int iters, int packed, float seed) {
    float x = seed + (float)threadIdx.x * 1e-9f, y = 0.999f;
    if (packed) {
        unsigned long long acc[16];
#pragma unroll
        for (int i = 0; i < 16; i++) acc[i] = pack2(x + i, x - i);
        const unsigned long long m2 = pack2(y, y), a2 = pack2(1e-3f, 2e-3f);
        for (int it = 0; it < iters; it++) {
#pragma unroll
            for (int i = 0; i < 16; i++) acc[i] = fma2_bare(acc[i], m2, a2);
        }
        float s = 0.f;
#pragma unroll
        for (int i = 0; i < 16; i++) { float lo, hi; unpack2(acc[i], lo, hi); s += lo + hi; }
        if (s == 123.456f) out[0] = s;
    } else {
        float acc[16];
#pragma unroll
        for (int i = 0; i < 16; i++) acc[i] = x + i;
        for (int it = 0; it < iters; it++) {
#pragma unroll
            for (int i = 0; i < 16; i++) acc[i] = __fmaf_rn(acc[i], y, 1e-3f);
        }
        float s = 0.f;
#pragma unroll
        for (int i = 0; i < 16; i++) s += acc[i];
        if (s == 123.456f) out[0] = s;
    }
}

} // namespace b200i
