// Device-side numeric seams of the identical-mode matrix product.
//
// Every arithmetic step a kernel in this library performs on an operand, an
// accumulator or a fold node is spelled through one of these helpers, so the
// rounding, the flush and the (absent) contraction are decided here and
// nowhere else. The translation unit is compiled with -fmad=false -ftz=false
// -prec-div=true -prec-sqrt=true and without fast-math; on top of that every
// multiply-add is an explicit fma.rn and every pinned product an explicit
// mul.rn, so the compiler has nothing left to choose.
//
// Reference spellings (paths relative to the reference project's root):
//   flush           checks/numerics.mojo:198-269
//   multiply-add    checks/numerics.mojo:272-282, checks/rtf_seam.mojo:6-12, :112-115
//   low-bit seams   checks/numerics.mojo:1548-1671
//   NaN canon       core/nan_canon.mojo:53-56
#pragma once
#include <cstdint>
#include <cuda_runtime.h>
#include <atomic>

namespace b200i {



constexpr int OP_NN = 0, OP_NT = 1, OP_TN = 2;
constexpr int K_LEAF_MIN = 128, MAX_LEAVES = 1024;

// Weight (right operand) storage kinds.
constexpr int W_F32 = 0;        // float32 words
constexpr int W_BF16 = 1;       // uint16 bf16 bit patterns, widened exactly
constexpr int W_INT8_EXP = 2;   // int8 codes + one int32 power-of-two exponent per row (the reference's format)
constexpr int W_INT8_SCALE = 3; // int8 codes + one float32 scale per row (extension, no reference counterpart)

__host__ __device__ inline long long leaf_size(long long k) {
    if (k <= 0) return 1;
    if (k <= K_LEAF_MIN) return k;
    long long p0 = (k + K_LEAF_MIN - 1) / K_LEAF_MIN;
    if (p0 <= MAX_LEAVES) return K_LEAF_MIN;
    return (k + MAX_LEAVES - 1) / MAX_LEAVES;
}
__host__ __device__ inline long long leaf_count(long long k) {
    if (k <= 0) return 0;
    long long l = leaf_size(k);
    return (k + l - 1) / l;
}

// ---- flush ---------------------------------------------------------------
// A nonzero word below the smallest normal becomes its signed zero; every
// other word, NaN payloads included, is returned unchanged.
__device__ __forceinline__ float ftz_bits(float x) {
    unsigned b = __float_as_uint(x);
    return ((b & 0x7F800000u) == 0u) ? __uint_as_float(b & 0x80000000u) : x;
}
// The one-instruction flush: x * 1 + (-0) with .ftz is exact, so its only
// effect is the flush of a subnormal to its signed zero. It may return the
// canonical NaN for a NaN with a payload; every product word is
// NaN-canonicalised at the store, so no caller can observe the difference.
__device__ __forceinline__ float ftz_hw(float x) {
    float y;
    asm("fma.rn.ftz.f32 %0, %1, 0f3F800000, 0f80000000;" : "=f"(y) : "f"(x));
    return y;
}

// ---- the multiply-add step -------------------------------------------------
// Contract step: ONE IEEE rounding with gradual underflow, THEN the flush.
// A single fma.rn.ftz is wrong in the window [2^-126 - 2^-150, 2^-126), where
// it flushes before rounding.
__device__ __forceinline__ float step_flush(float a, float b, float acc) { return ftz_hw(__fmaf_rn(a, b, acc)); }
// Admitted step: the bare fma. Exact contract arithmetic when no step result
// can be subnormal (see admit_key below).
__device__ __forceinline__ float step_bare(float a, float b, float acc) { return __fmaf_rn(a, b, acc); }

// Two independent IEEE fused multiply-adds in one instruction (sm_100 packed
// fp32): lane-wise identical to two fma.rn.f32.
__device__ __forceinline__ unsigned long long pack2(float lo, float hi) {
    unsigned long long r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
    return r;
}
__device__ __forceinline__ void unpack2(unsigned long long v, float &lo, float &hi) {
    asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ unsigned long long fma2_bare(unsigned long long a, unsigned long long b, unsigned long long c) {
    unsigned long long d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
    return d;
}
__device__ __forceinline__ unsigned long long ftz2_hw(unsigned long long x) {
    unsigned long long d;
    const unsigned long long ones = 0x3F8000003F800000ull, negz = 0x8000000080000000ull;
    asm("fma.rn.ftz.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(x), "l"(ones), "l"(negz));
    return d;
}

// ftz(a + b) for operands that are ALREADY flushed, in one instruction. Two floats
// that are zero or normal are multiples of 2^-149, so a sum below 2^-126 is exactly
// representable: nothing is rounded there, and flushing the result is the same as
// rounding first and flushing after (the window that breaks fma.rn.ftz cannot occur).
__device__ __forceinline__ float add_flushed(float a, float b) {
    float r;
    asm("add.rn.ftz.f32 %0, %1, %2;" : "=f"(r) : "f"(a), "f"(b));
    return r;
}

// fold-node addition: both children are already flushed; add, then flush.
__device__ __forceinline__ float fold_add(float x, float y) { return ftz_hw(__fadd_rn(x, y)); }

// ---- admission ---------------------------------------------------------------
// key(w) = (w << 1) - 2 as an unsigned word: both zeros map to 0xFFFFFFFE, a
// nonzero subnormal to a small value, a normal with biased exponent e to at
// least (e << 24) - 2. A staged window whose operands all satisfy
// key >= ADMIT_MIN has no subnormal operand and no nonzero operand with a
// biased exponent below 87; the sum of two such exponents is at least 174, so
// every product is a multiple of 2^-126, and so is every accumulator that
// started a leaf at +0.0 and has only taken admitted steps: no step result can
// be subnormal and the flush is the identity.
#ifdef B200I_SABOTAGE_ADMIT_ALWAYS
// Negative control (the reference's MOJOLEARN_GEMM_SABOTAGE_ADMIT_ALWAYS, gemm/checks/gemm_identical.mojo:1444): a
// second build in which every window is admitted, whatever it holds. The tests load it next to the real library and
// require the subnormal-forcing cases to FAIL under it, which shows that those cases would catch a broken admission
// test. Wrong bits are its only effect; it is never the library the package loads by default.
constexpr unsigned ADMIT_EXP = 0u;
constexpr unsigned ADMIT_MIN = 0u;
#else
constexpr unsigned ADMIT_EXP = 87u;
constexpr unsigned ADMIT_MIN = (ADMIT_EXP << 24) - 2u;
#endif
__device__ __forceinline__ unsigned admit_key(float x) { return (__float_as_uint(x) << 1) - 2u; }

// ---- NaN canonicalisation -----------------------------------------------------
__device__ __forceinline__ float nan_canon(float x) { return (x != x) ? __uint_as_float(0x7FC00000u) : x; }

// ---- low-bit seams ---------------------------------------------------------------
__device__ __forceinline__ float bf16_bits_to_f32(unsigned short bits) { return __uint_as_float((unsigned)bits << 16); }

__device__ __forceinline__ unsigned short f32_to_bf16_bits_rne(float x_in) {
    unsigned b = __float_as_uint(ftz_bits(x_in));
    if ((b & 0x7F800000u) == 0x7F800000u && (b & 0x007FFFFFu) != 0u) return (unsigned short)((b >> 16) | 0x0040u);
    unsigned lsb = (b >> 16) & 1u;
    return (unsigned short)((b + 0x7FFFu + lsb) >> 16);
}

__device__ __forceinline__ float pow2_f32(int e) {
    if (e > 127) return __uint_as_float(0x7F800000u);
    if (e < -126) return 0.0f;
    return __uint_as_float((unsigned)(e + 127) << 23);
}

__device__ __forceinline__ float round_half_even(float x) {
    const float magic = 12582912.0f; // 1.5 * 2^23
    if (x >= 0.0f) return __fsub_rn(__fadd_rn(x, magic), magic);
    return __fadd_rn(__fsub_rn(x, magic), magic);
}

__device__ __forceinline__ int int8_row_exponent(float absmax) {
    float a = ftz_bits(absmax);
    if (a == 0.0f || a != a) return 0;
    return (int)((__float_as_uint(a) >> 23) & 0xFFu) - 127 - 6;
}

__device__ __forceinline__ signed char quantize_int8_value(float x, int e) {
    if (x != x) return 0;
    float s = ftz_bits(__fmul_rn(ftz_bits(x), pow2_f32(-e)));
    float r = round_half_even(s);
    if (r != r) return 0;
    if (r > 127.0f) r = 127.0f;
    if (r < -127.0f) r = -127.0f;
    return (signed char)__float2int_rz(r);
}

// int8 code times a power of two (exact unless it leaves the normal range),
// then the flush; |code| <= 128 converts exactly.
__device__ __forceinline__ float dequant_int8_pow2(int code, float pow2) { return ftz_bits(__fmul_rn((float)code, pow2)); }

} // namespace b200i
