// Device-side portable math of the identical profile: the published Cephes
// single-precision algorithms in the reference's operation order, one IEEE
// rounding per written operation (every product, sum and quotient is an explicit
// round-to-nearest intrinsic, every fused step an explicit fma.rn, so the
// compiler has nothing to contract or reassociate).
//
// Reference spellings (checks/numerics.mojo of the reference): portable_expf
// :370-413, portable_logf :416-465, portable_sqrtf :503-571, sin/cos core
// :574-620 and :1177-1187, portable_powf :623-637, portable_divf :1035-1037,
// portable_rsqrtf :1040-1054, portable_siluf :1088-1094, portable_tanhf
// :1190-1219, erf/erfc :1222-1282, gelu :1285-1316, fmax :1319-1337.
#pragma once
#include "seams.cuh"

namespace b200i {

__device__ __forceinline__ float m_mul(float a, float b) { return __fmul_rn(a, b); }
__device__ __forceinline__ float m_add(float a, float b) { return __fadd_rn(a, b); }
__device__ __forceinline__ float m_sub(float a, float b) { return __fsub_rn(a, b); }
__device__ __forceinline__ float m_quo(float a, float b) { return __fdiv_rn(a, b); }
__device__ __forceinline__ float m_qnan() { return __uint_as_float(0x7FC00000u); }
__device__ __forceinline__ float m_pinf() { return __uint_as_float(0x7F800000u); }

__device__ __forceinline__ float p_expf(float x) {
    if (x != x) return x;
    if (x > 88.722835f) return m_pinf();
    if (x < -87.33655f) return 0.0f;
    const float t = __fmaf_rn(x, 1.4426950408889634f, 0.5f);
    const float zf = floorf(t);
    const int k = (int)zf;
    float r = __fmaf_rn(zf, -0.693359375f, x);
    r = __fmaf_rn(zf, 2.12194440e-4f, r);
    float q = 1.9875691500e-4f;
    q = __fmaf_rn(q, r, 1.3981999507e-3f);
    q = __fmaf_rn(q, r, 8.3334519073e-3f);
    q = __fmaf_rn(q, r, 4.1665795894e-2f);
    q = __fmaf_rn(q, r, 1.6666665459e-1f);
    q = __fmaf_rn(q, r, 5.0000001201e-1f);
    const float r2 = m_mul(r, r);
    float y = __fmaf_rn(q, r2, r);
    y = m_add(y, 1.0f);
    const int k1 = k >> 1, k2 = k - k1;
    y = m_mul(y, __uint_as_float((unsigned)(k1 + 127) << 23));
    y = m_mul(y, __uint_as_float((unsigned)(k2 + 127) << 23));
    if (y < 1.1754943508222875e-38f) return 0.0f;
    return y;
}

__device__ __forceinline__ float cephes_logf_core(float t, int e) {
    const float z = m_mul(t, t);
    float p = 7.0376836292e-2f;
    p = __fmaf_rn(p, t, -1.1514610310e-1f);
    p = __fmaf_rn(p, t, 1.1676998740e-1f);
    p = __fmaf_rn(p, t, -1.2420140846e-1f);
    p = __fmaf_rn(p, t, 1.4249322787e-1f);
    p = __fmaf_rn(p, t, -1.6668057665e-1f);
    p = __fmaf_rn(p, t, 2.0000714765e-1f);
    p = __fmaf_rn(p, t, -2.4999993993e-1f);
    p = __fmaf_rn(p, t, 3.3333331174e-1f);
    const float tz = m_mul(t, z);
    float y = m_mul(tz, p);
    const float ef = (float)e;
    y = __fmaf_rn(ef, -2.12194440e-4f, y);
    y = __fmaf_rn(-0.5f, z, y);
    const float r = m_add(t, y);
    return __fmaf_rn(ef, 0.693359375f, r);
}

__device__ __forceinline__ float p_logf(float x) {
    if (x != x) return x;
    if (fabsf(x) < 1.1754943508222875e-38f) x = 0.0f;
    if (x == 0.0f) return __uint_as_float(0xFF800000u);
    if (x < 0.0f) return m_qnan();
    if (x == m_pinf()) return x;
    const unsigned bits = __float_as_uint(x);
    int e = (int)((bits >> 23) & 0xFFu) - 126;
    float m = __uint_as_float((bits & 0x007FFFFFu) | 0x3F000000u);
    if (m < 0.7071067811865476f) { e -= 1; m = m_add(m, m); }
    return cephes_logf_core(m_sub(m, 1.0f), e);
}

__device__ __forceinline__ float p_powf(float x, float p) {
    if (p == 0.0f) return 1.0f;
    if (x != x || p != p) return m_qnan();
    if (x < 0.0f) return m_qnan();
    if (x == 0.0f) return p > 0.0f ? 0.0f : m_pinf();
    return p_expf(m_mul(p, p_logf(x)));
}

__device__ __forceinline__ float p_sqrtf(float x) {
    if (x != x) return x;
    if (fabsf(x) < 1.1754943508222875e-38f) return 0.0f;
    if (x < 0.0f) return m_qnan();
    if (x == m_pinf()) return x;
    bool scaled = false;
    if (x < __uint_as_float(0x0F800000u)) { x = m_mul(x, __uint_as_float(0x5F800000u)); scaled = true; }
    float y = __uint_as_float((__float_as_uint(x) >> 1) + 0x1FBD1DF5u);
#pragma unroll
    for (int it = 0; it < 3; it++) y = m_mul(0.5f, m_add(y, m_quo(x, y)));
    const unsigned yb = __float_as_uint(y);
    float best = y, r_best = fabsf(__fmaf_rn(-y, y, x));
#pragma unroll
    for (int kk = 0; kk < 4; kk++) {
        const unsigned delta = (unsigned)(kk / 2 + 1);
        const float c = __uint_as_float((kk % 2 == 0) ? yb - delta : yb + delta);
        const float r = fabsf(__fmaf_rn(-c, c, x));
        if (r < r_best) { best = c; r_best = r; }
    }
    if (scaled) best = m_mul(best, __uint_as_float(0x2F800000u));
    return best;
}

__device__ __forceinline__ float p_divf(float a, float b) { return ftz_bits(m_quo(ftz_bits(a), ftz_bits(b))); }

__device__ __forceinline__ float p_rsqrtf(float x_in) {
    const float x = ftz_bits(x_in);
    if (x != x) return x;
    if (x < 0.0f) return m_qnan();
    const float s = p_sqrtf(x);
    if (s == 0.0f) return m_pinf();
    if (s == m_pinf()) return 0.0f;
    return p_divf(1.0f, s);
}

__device__ __forceinline__ float cephes_sincosf_core(float x_abs, float sign_in, bool is_cos) {
    float x = x_abs;
    int j = (int)floorf(m_mul(x, 1.27323954473516f));
    float yj = (float)j;
    if (j & 1) { j += 1; yj = m_add(yj, 1.0f); }
    j &= 7;
    x = __fmaf_rn(yj, -0.78515625f, x);
    x = __fmaf_rn(yj, -2.4187564849853515625e-4f, x);
    x = __fmaf_rn(yj, -3.77489497744594108e-8f, x);
    float sign = sign_in;
    if (j > 3) { j -= 4; sign = -sign; }
    if (is_cos && j > 1) sign = -sign;
    const float z = m_mul(x, x);
    bool use_sin_poly = (j == 1 || j == 2);
    if (!is_cos) use_sin_poly = !use_sin_poly;
    float y;
    if (use_sin_poly) {
        float p = -1.9515295891e-4f;
        p = __fmaf_rn(p, z, 8.3321608736e-3f);
        p = __fmaf_rn(p, z, -1.6666654611e-1f);
        y = __fmaf_rn(m_mul(x, z), p, x);
    } else {
        float p = 2.443315711809948e-5f;
        p = __fmaf_rn(p, z, -1.388731625493765e-3f);
        p = __fmaf_rn(p, z, 4.166664568298827e-2f);
        y = __fmaf_rn(m_mul(z, z), p, __fmaf_rn(-0.5f, z, 1.0f));
    }
    return m_mul(sign, y);
}
__device__ __forceinline__ float p_cosf(float x) {
    if (x != x || fabsf(x) == m_pinf()) return m_qnan();
    return cephes_sincosf_core(fabsf(x), 1.0f, true);
}
__device__ __forceinline__ float p_sinf(float x_in) {
    if (x_in != x_in || fabsf(x_in) == m_pinf()) return m_qnan();
    const float x = ftz_bits(x_in);
    const float sign = (__float_as_uint(x) & 0x80000000u) ? -1.0f : 1.0f;
    return cephes_sincosf_core(fabsf(x), sign, false);
}

__device__ __forceinline__ float p_siluf(float x) {
    if (x != x) return x;
    const float e = p_expf(-x);
    return p_divf(x, m_add(e, 1.0f));
}

__device__ __forceinline__ float p_tanhf(float x_in) {
    const float xx = ftz_bits(x_in);
    if (xx != xx) return xx;
    if (xx == 0.0f) return xx;
    const float x = fabsf(xx);
    if (x > __uint_as_float(0x42317218u)) return xx < 0.0f ? -1.0f : 1.0f;
    if (x >= 0.625f) {
        const float e = p_expf(m_add(x, x));
        const float q = p_divf(2.0f, m_add(e, 1.0f));
        const float z = m_sub(1.0f, q);
        return xx < 0.0f ? -z : z;
    }
    const float zs = m_mul(x, x);
    float p = -5.70498872745e-3f;
    p = __fmaf_rn(p, zs, 2.06390887954e-2f);
    p = __fmaf_rn(p, zs, -5.37397155531e-2f);
    p = __fmaf_rn(p, zs, 1.33314422036e-1f);
    p = __fmaf_rn(p, zs, -3.33332819422e-1f);
    return __fmaf_rn(m_mul(p, zs), xx, xx);
}

__device__ __forceinline__ float cephes_erfcf_ge1(float a) {
    const float x = fabsf(a);
    float z = -m_mul(x, x);
    if (z < __uint_as_float(0xC2B17218u)) return a < 0.0f ? 2.0f : 0.0f;
    z = p_expf(z);
    const float q = p_divf(1.0f, x);
    const float y = m_mul(q, q);
    float p;
    if (x < 2.0f) {
        p = 2.326819970068386e-2f;
        p = __fmaf_rn(p, y, -1.387039388740657e-1f);
        p = __fmaf_rn(p, y, 3.687424674597105e-1f);
        p = __fmaf_rn(p, y, -5.824733027278666e-1f);
        p = __fmaf_rn(p, y, 6.210004621745983e-1f);
        p = __fmaf_rn(p, y, -4.944515323274145e-1f);
        p = __fmaf_rn(p, y, 3.404879937665872e-1f);
        p = __fmaf_rn(p, y, -2.741127028184656e-1f);
        p = __fmaf_rn(p, y, 5.638259427386472e-1f);
    } else {
        p = -10.47766399936249f;
        p = __fmaf_rn(p, y, 12.97719955372516f);
        p = __fmaf_rn(p, y, -7.495518717768503f);
        p = __fmaf_rn(p, y, 2.921019019210786f);
        p = __fmaf_rn(p, y, -1.015265279202700f);
        p = __fmaf_rn(p, y, 4.218463358204948e-1f);
        p = __fmaf_rn(p, y, -2.820767439740514e-1f);
        p = __fmaf_rn(p, y, 5.641895067754075e-1f);
    }
    const float t = ftz_bits(m_mul(z, q));
    float r = ftz_bits(m_mul(t, p));
    if (a < 0.0f) r = m_sub(2.0f, r);
    return r;
}
__device__ __forceinline__ float p_erff(float x_in) {
    const float x = ftz_bits(x_in);
    if (x != x) return x;
    if (fabsf(x) > 1.0f) return m_sub(1.0f, cephes_erfcf_ge1(x));
    const float z = m_mul(x, x);
    float p = 7.853861353153693e-5f;
    p = __fmaf_rn(p, z, -8.010193625184903e-4f);
    p = __fmaf_rn(p, z, 5.188327685732524e-3f);
    p = __fmaf_rn(p, z, -2.685381193529856e-2f);
    p = __fmaf_rn(p, z, 1.128358514861418e-1f);
    p = __fmaf_rn(p, z, -3.761262582423300e-1f);
    p = __fmaf_rn(p, z, 1.128379165726710f);
    return m_mul(x, p);
}
__device__ __forceinline__ float p_gelu_erf(float x_in) {
    const float x = ftz_bits(x_in);
    if (x != x) return x;
    const float e = p_erff(p_divf(x, __uint_as_float(0x3FB504F3u)));
    const float s = m_add(1.0f, e);
    const float h = ftz_bits(m_mul(x, 0.5f));
    return ftz_bits(m_mul(h, s));
}
__device__ __forceinline__ float p_gelu_tanh(float x_in) {
    const float x = ftz_bits(x_in);
    if (x != x) return x;
    const float c3 = __uint_as_float(0x3D372713u), kk = __uint_as_float(0x3F4C422Au);
    const float x2 = ftz_bits(m_mul(x, x));
    const float x3 = ftz_bits(m_mul(x2, x));
    const float cx = ftz_bits(m_mul(c3, x3));
    const float inner = ftz_bits(m_add(x, cx));
    const float arg = ftz_bits(m_mul(kk, inner));
    const float t = p_tanhf(arg);
    const float s = m_add(1.0f, t);
    const float h = ftz_bits(m_mul(x, 0.5f));
    return ftz_bits(m_mul(h, s));
}

// a float as an unsigned key whose integer order is the float's total order
__device__ __forceinline__ unsigned order_key(float v) {
    const unsigned b = __float_as_uint(v);
    return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}
__device__ __forceinline__ float order_unkey(unsigned k) {
    return __uint_as_float((k & 0x80000000u) ? (k & 0x7FFFFFFFu) : ~k);
}

// ---- store epilogues of the product -------------------------------------------------------------
// The reference's GEMM_EPI_PLUS_BIAS and GEMM_EPI_BIAS_ACT (gemm/checks/gemm_identical.mojo:8869-8912, :9483-9491):
// the finished product word, then one plain add of the column's bias (transformer_oracle.mojo:1344-1372), then the
// activation of an ungated MLP (S20 and the GELU variants), each with the flush the separate seams apply. The words
// are those of the product followed by b200i_bias_add and b200i_act_mul; only the launches are saved. `c` is the
// product's stored word (root flushed, NaN canonical).
struct Epilogue {
    const float *bias; // one word per output column, or NULL
    int act;           // EPI_ACT_*
};
// Codes 4 to 6 are the GATED activations over a product whose weight rows were interleaved (row 2j = gate_j, row
// 2j + 1 = up_j): output column j of the [m, n / 2] result is ftz(act(gate) * up), S20-S21 with SiLU, or GELU in its
// place (transformer_oracle.mojo:2580-2620). A thread that owns two adjacent product columns owns one such pair.
enum { EPI_ACT_NONE = 0, EPI_ACT_GELU_ERF = 1, EPI_ACT_GELU_TANH = 2, EPI_ACT_SILU = 3, EPI_PAIR_SWIGLU = 4, EPI_PAIR_GEGLU_ERF = 5,
       EPI_PAIR_GEGLU_TANH = 6 };
__host__ __device__ __forceinline__ bool epilogue_on(const Epilogue &e) { return e.bias != nullptr || e.act != EPI_ACT_NONE; }
__host__ __device__ __forceinline__ bool epilogue_pairs(const Epilogue &e) { return e.act >= EPI_PAIR_SWIGLU; }
// gate and up are the product's stored words of columns 2j and 2j + 1
__device__ __noinline__ float epilogue_pair_apply(float gate, float up, const float *bias, int act, long long j) {
    if (bias) {
        gate = ftz_bits(__fadd_rn(ftz_bits(gate), ftz_bits(__ldg(bias + 2 * j))));
        up = ftz_bits(__fadd_rn(ftz_bits(up), ftz_bits(__ldg(bias + 2 * j + 1))));
    }
    const float z = ftz_bits(gate);
    float a;
    if (act == EPI_PAIR_SWIGLU) a = ftz_bits(p_siluf(z));
    else if (act == EPI_PAIR_GEGLU_TANH) a = ftz_bits(p_gelu_tanh(z));
    else a = ftz_bits(p_gelu_erf(z));
    return ftz_bits(__fmul_rn(a, ftz_bits(up)));
}
__device__ __noinline__ float epilogue_apply(float c, const float *bias, int act, long long col) {
    if (bias) c = ftz_bits(__fadd_rn(ftz_bits(c), ftz_bits(__ldg(bias + col))));
    if (act == EPI_ACT_GELU_ERF) c = ftz_bits(p_gelu_erf(ftz_bits(c)));
    else if (act == EPI_ACT_GELU_TANH) c = ftz_bits(p_gelu_tanh(ftz_bits(c)));
    else if (act == EPI_ACT_SILU) c = ftz_bits(p_siluf(ftz_bits(c)));
    return c;
}
// A product kernel stores its words exactly as it does without an epilogue and then, only when one is asked for,
// walks its own cells once more through this function (a thread re-reads what it wrote itself). The call is kept out
// of line and out of the store loops on purpose: inlined there, or called from there, it costs every product
// registers and spills in its hottest code for the sake of the few that carry a bias.
__device__ __forceinline__ void epilogue_cell(float *cell, const Epilogue &e, long long col) {
    *cell = epilogue_apply(*cell, e.bias, e.act, col);
}

} // namespace b200i
