/*
 * CPU oracle for the `mojolearn.identical.gemm.fp32.v1` matrix product and the
 * low-bit weight-storage seams that feed it.
 *
 * THIS FILE IS TEST INFRASTRUCTURE. It is the checker the CUDA path is held
 * to, and the scalar CPU baseline the benchmark times beside the GPU. Nothing
 * in the shipped package may call it: only the test-suite, the smoke check and
 * the benchmark's CPU-baseline leg load the library built from it.
 *
 * It is a plain-C restatement of the reference's normative host algorithm.
 * Every function cites the reference file and lines it follows (paths are
 * relative to the reference project's root). The reference itself is Mojo and
 * cannot be compiled in this environment, so the restatement is pinned
 * instead by the reference's committed golden hashes (identity card and
 * verify table; see tests/test_oracle_golden.py).
 *
 * Build rules that matter for the bits: -ffp-contract=off (the compiler never
 * fuses on its own), fmaf() is the one fused multiply-add (hardware FMA via
 * -mfma), no fast-math, and the MXCSR flush/denormals-are-zero bits are
 * cleared around every entry so that gradual underflow is what the hardware
 * computes and the flush is what this file spells.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#if defined(__x86_64__)
#include <xmmintrin.h>
#endif

#define ORACLE_API __attribute__((visibility("default")))

enum { OP_NN = 0, OP_NT = 1, OP_TN = 2 }; /* gemm/contract.mojo OP_* ids */

enum { K_LEAF_MIN = 128, MAX_LEAVES = 1024 }; /* gemm/contract.mojo:140, :170 */

/* ---- floating-point environment ---------------------------------------- */

/* The reference pins the caller's IEEE environment with FTZ/DAZ clear on every
 * worker (core/host_parallel.mojo:15-33). */
static unsigned fpenv_enter(void) {
#if defined(__x86_64__)
    unsigned old = _mm_getcsr();
    _mm_setcsr(old & ~(0x8000u | 0x0040u));
    return old;
#else
    return 0;
#endif
}
static void fpenv_leave(unsigned old) {
#if defined(__x86_64__)
    _mm_setcsr(old);
#else
    (void)old;
#endif
}

/* ---- bit helpers --------------------------------------------------------- */

static inline uint32_t f2u(float x) { uint32_t u; memcpy(&u, &x, 4); return u; }
static inline float u2f(uint32_t u) { float x; memcpy(&x, &u, 4); return x; }

/* checks/numerics.mojo:263-269 (the integer spelling): a nonzero word whose
 * exponent field is zero becomes its sign bit; everything else is unchanged. */
static inline float ftz(float x) {
    uint32_t b = f2u(x);
    if ((b & 0x7F800000u) == 0u && (b & 0x007FFFFFu) != 0u) return u2f(b & 0x80000000u);
    return x;
}

/* checks/numerics.mojo:272-282: the contraction pin is one IEEE fused
 * multiply-add, rounded once. */
static inline float mul_add(float a, float b, float c) { return fmaf(a, b, c); }

ORACLE_API float oracle_ftz(float x) { return ftz(x); }

/* ---- leaf partition and fold-tree addressing ------------------------------ */

/* gemm/contract.mojo:173-211 */
ORACLE_API int64_t oracle_leaf_size(int64_t k) {
    if (k <= 0) return 1;
    if (k <= K_LEAF_MIN) return k;
    int64_t p0 = (k + K_LEAF_MIN - 1) / K_LEAF_MIN;
    if (p0 <= MAX_LEAVES) return K_LEAF_MIN;
    return (k + MAX_LEAVES - 1) / MAX_LEAVES;
}

/* gemm/contract.mojo:214-228 */
ORACLE_API int64_t oracle_leaf_count_at(int64_t k, int64_t leaf) {
    if (k <= 0) return 0;
    if (leaf < 1) leaf = 1;
    return (k + leaf - 1) / leaf;
}
ORACLE_API int64_t oracle_leaf_count(int64_t k) { return oracle_leaf_count_at(k, oracle_leaf_size(k)); }

/* gemm/contract.mojo:317-384 */
ORACLE_API int64_t oracle_fold_level_width(int64_t p, int64_t d) {
    if (p <= 0) return 0;
    if (d <= 0) return p;
    if (d >= 40) return 1;
    int64_t den = (int64_t)1 << d;
    return (p + den - 1) / den;
}
ORACLE_API int64_t oracle_fold_level_count(int64_t p) {
    if (p <= 0) return 0;
    int64_t levels = 1, w = p;
    while (w > 1) { w = (w + 1) / 2; levels++; }
    return levels;
}
ORACLE_API int64_t oracle_fold_level_base(int64_t p, int64_t d) {
    int64_t base = 0;
    for (int64_t dd = 0; dd < d; dd++) base += oracle_fold_level_width(p, dd);
    return base;
}
ORACLE_API int64_t oracle_fold_node_total(int64_t p) { return oracle_fold_level_base(p, oracle_fold_level_count(p)); }
ORACLE_API int64_t oracle_fold_node_addr(int64_t p, int64_t d, int64_t q) { return oracle_fold_level_base(p, d) + q; }
ORACLE_API int oracle_fold_node_is_carry(int64_t p, int64_t d, int64_t q) {
    if (d < 1) return 0;
    return 2 * q + 1 >= oracle_fold_level_width(p, d - 1);
}

/* ---- the product ----------------------------------------------------------- */

/* gemm/host/gemm_oracle.mojo:122-137: one arithmetic, three addressings. */
static inline float a_at(const float *a, int op, int64_t i, int64_t p, int64_t m, int64_t k) {
    return op == OP_TN ? a[p * m + i] : a[i * k + p];
}
static inline float b_at(const float *b, int op, int64_t p, int64_t j, int64_t n, int64_t k) {
    return op == OP_NT ? b[j * k + p] : b[p * n + j];
}

/* gemm/host/gemm_oracle.mojo:146-206: p ascending from a +0.0 seed, one fused
 * multiply-add per step, every seam flushed. */
static float leaf_partial(const float *a, const float *b, int op, int64_t i, int64_t j, int64_t m, int64_t n,
                          int64_t k, int64_t pb, int64_t pe) {
    float acc = 0.0f;
    for (int64_t p = pb; p < pe; p++)
        acc = ftz(mul_add(ftz(a_at(a, op, i, p, m, k)), ftz(b_at(b, op, p, j, n, k)), acc));
    return ftz(acc);
}

/* gemm/host/gemm_oracle.mojo:218-272: adjacent pairs (2q, 2q+1); an odd tail
 * is carried bit for bit; P == 0 is +0.0; P == 1 performs no addition.
 * Folds in place over `v` (length p). */
static float fold_tree(float *v, int64_t p) {
    if (p == 0) return 0.0f;
    int64_t width = p;
    while (width > 1) {
        int64_t pairs = width / 2;
        for (int64_t q = 0; q < pairs; q++) v[q] = ftz(ftz(v[2 * q]) + ftz(v[2 * q + 1]));
        if (width & 1) v[pairs] = v[width - 1];
        width = pairs + (width & 1);
    }
    return ftz(v[0]);
}

ORACLE_API float oracle_fold_balanced_tree(const float *partials, int64_t p) {
    unsigned env = fpenv_enter();
    float *v = (float *)malloc(sizeof(float) * (size_t)(p > 0 ? p : 1));
    if (p > 0) memcpy(v, partials, sizeof(float) * (size_t)p);
    float r = fold_tree(v, p);
    free(v);
    fpenv_leave(env);
    return r;
}

/* Alternatives the contract names as WRONG, kept so the separation fixtures
 * can show each one differs from the tree above (gemm_oracle_check.mojo
 * F5 serial fold, F7 zero padding to a power of two, F8 stride pairing). */
ORACLE_API float oracle_fold_serial(const float *partials, int64_t p) {
    unsigned env = fpenv_enter();
    float acc = p > 0 ? ftz(partials[0]) : 0.0f;
    for (int64_t t = 1; t < p; t++) acc = ftz(acc + ftz(partials[t]));
    fpenv_leave(env);
    return ftz(acc);
}
ORACLE_API float oracle_fold_padded_pow2(const float *partials, int64_t p) {
    unsigned env = fpenv_enter();
    int64_t w = 1;
    while (w < p) w <<= 1;
    float *v = (float *)calloc((size_t)w, sizeof(float));
    if (p > 0) memcpy(v, partials, sizeof(float) * (size_t)p);
    float r = fold_tree(v, w);
    free(v);
    fpenv_leave(env);
    return r;
}
ORACLE_API float oracle_fold_stride(const float *partials, int64_t p) {
    unsigned env = fpenv_enter();
    int64_t w = 1;
    while (w < p) w <<= 1;
    float *v = (float *)calloc((size_t)w, sizeof(float));
    if (p > 0) memcpy(v, partials, sizeof(float) * (size_t)p);
    /* red[t] += red[t + step], only where the partner is a real leaf */
    for (int64_t step = w / 2; step >= 1; step /= 2)
        for (int64_t t = 0; t < step; t++)
            if (t + step < p) v[t] = ftz(ftz(v[t]) + ftz(v[t + step]));
    float r = ftz(v[0]);
    free(v);
    fpenv_leave(env);
    return r;
}

/* gemm/host/gemm_oracle.mojo:275-371, at an explicit leaf size (`leaf` equal
 * to oracle_leaf_size(k) is the contract's answer; any other value is an
 * adversary for the separation fixtures). Returns 0, or 1 on a refusal. */
ORACLE_API int oracle_gemm_at_leaf(float *c, const float *a, const float *b, int op, int64_t m, int64_t n,
                                   int64_t k, int64_t leaf) {
    if (op != OP_NN && op != OP_NT && op != OP_TN) return 1;
    if (m < 0 || n < 0 || k < 0) return 1;
    unsigned env = fpenv_enter();
    int64_t pc = oracle_leaf_count_at(k, leaf);
    int64_t el = leaf < 1 ? 1 : leaf;
    float *parts = (float *)malloc(sizeof(float) * (size_t)(pc > 0 ? pc : 1));
    for (int64_t i = 0; i < m; i++)
        for (int64_t j = 0; j < n; j++) {
            if (pc == 1) {
                c[i * n + j] = ftz(leaf_partial(a, b, op, i, j, m, n, k, 0, k));
                continue;
            }
            for (int64_t t = 0; t < pc; t++) {
                int64_t pb = t * el, pe = (t + 1) * el;
                if (pe > k) pe = k;
                parts[t] = leaf_partial(a, b, op, i, j, m, n, k, pb, pe);
            }
            c[i * n + j] = fold_tree(parts, pc);
        }
    free(parts);
    fpenv_leave(env);
    return 0;
}

/* gemm/host/gemm_oracle.mojo:355-371: THE NORMATIVE ANSWER. */
ORACLE_API int oracle_gemm(float *c, const float *a, const float *b, int op, int64_t m, int64_t n, int64_t k) {
    return oracle_gemm_at_leaf(c, a, b, op, m, n, k, oracle_leaf_size(k));
}

/* gemm/host/gemm_oracle.mojo:473-524: the whole-k single chain. Diagnostic
 * only; equals oracle_gemm exactly when k <= 128. */
ORACLE_API int oracle_gemm_serial(float *c, const float *a, const float *b, int op, int64_t m, int64_t n, int64_t k) {
    return oracle_gemm_at_leaf(c, a, b, op, m, n, k, k > 0 ? k : 1);
}

/* One cell with the multiply and the add left unfused (separation fixture F3)
 * or flushed before rounding instead of after (F4). mode 0 = contract,
 * 1 = unfused, 2 = no flush at all (gradual underflow kept). */
ORACLE_API float oracle_chain_variant(const float *a, const float *b, int64_t len, int mode) {
    unsigned env = fpenv_enter();
    float acc = 0.0f;
    for (int64_t p = 0; p < len; p++) {
        if (mode == 0) acc = ftz(mul_add(ftz(a[p]), ftz(b[p]), acc));
        else if (mode == 1) { volatile float prod = ftz(a[p]) * ftz(b[p]); acc = ftz(ftz(prod) + acc); }
        else acc = mul_add(a[p], b[p], acc);
    }
    fpenv_leave(env);
    return mode == 2 ? acc : ftz(acc);
}

/* core/nan_canon.mojo:53-56: every NaN word of a product that crosses the
 * host boundary becomes the one quiet NaN 0x7FC00000. */
ORACLE_API void oracle_nan_canon(float *c, int64_t count) {
    for (int64_t t = 0; t < count; t++) {
        uint32_t b = f2u(c[t]);
        if ((b & 0x7F800000u) == 0x7F800000u && (b & 0x007FFFFFu) != 0u) c[t] = u2f(0x7FC00000u);
    }
}

/* ---- low-bit seams (gemm/IDENTICAL_LOWBIT_CONTRACT.md L-1 .. L-6) -------- */

/* checks/numerics.mojo:1548-1551 */
static inline float bf16_to_f32(uint16_t bits) { return u2f((uint32_t)bits << 16); }

/* checks/numerics.mojo:1554-1570: flush, then round to nearest even on the
 * discarded 16 bits; a NaN keeps sign and top payload and is forced quiet. */
static inline uint16_t f32_to_bf16_rne(float x_in) {
    uint32_t b = f2u(ftz(x_in));
    if ((b & 0x7F800000u) == 0x7F800000u && (b & 0x007FFFFFu) != 0u) return (uint16_t)((b >> 16) | 0x0040u);
    uint32_t lsb = (b >> 16) & 1u;
    return (uint16_t)((b + 0x7FFFu + lsb) >> 16);
}

/* checks/numerics.mojo:1580-1586: the 1.5*2^23 magic constant, |x| <= 2^22. */
static inline float round_half_even(float x) {
    const float magic = 12582912.0f;
    volatile float t;
    if (x >= 0.0f) { t = x + magic; return t - magic; }
    t = x - magic;
    return t + magic;
}

/* checks/numerics.mojo:1589-1597: no subnormal scales. */
static inline float pow2_f32(int64_t e) {
    if (e > 127) return u2f(0x7F800000u);
    if (e < -126) return 0.0f;
    return u2f((uint32_t)(e + 127) << 23);
}

/* checks/numerics.mojo:1600-1604 */
static inline int f32_exponent(float x) { return (int)((f2u(x) >> 23) & 0xFFu) - 127; }

/* checks/numerics.mojo:1607-1627: 20-bit high part and 12-bit low part, each
 * exact, one exact scaling and ONE rounding addition. */
static inline float i32_to_f32_pinned(int32_t v) {
    int neg = v < 0;
    int64_t wide = v;
    if (neg) wide = -wide;
    uint32_t mag = (uint32_t)wide;
    float hi = (float)(int32_t)(mag >> 12);
    float lo = (float)(int32_t)(mag & 0xFFFu);
    volatile float scaled = hi * 4096.0f;
    float r = scaled + lo;
    return neg ? -r : r;
}

/* checks/numerics.mojo:1636-1643 */
static inline int int8_row_exponent(float absmax) {
    float a = ftz(absmax);
    if (a == 0.0f || a != a) return 0;
    return f32_exponent(a) - 6;
}

/* checks/numerics.mojo:1646-1662 */
static inline int8_t quantize_int8_value(float x, int e) {
    if (x != x) return 0;
    volatile float prod = ftz(x) * pow2_f32(-(int64_t)e);
    float s = ftz(prod);
    float r = round_half_even(s);
    if (r != r) return 0; /* 0 * inf when the scale overflows: the code stays zero (tools/identity_break.py:4120-4122) */
    if (r > 127.0f) r = 127.0f;
    if (r < -127.0f) r = -127.0f;
    return (int8_t)(int)r;
}

/* checks/numerics.mojo:1665-1671 */
static inline float dequant_int8_pinned(int32_t acc, int64_t e_sum) {
    volatile float prod = i32_to_f32_pinned(acc) * pow2_f32(e_sum);
    return ftz(prod);
}

/* gemm/host/gemm_lowbit_oracle.mojo:98-118 */
ORACLE_API void oracle_from_bf16(float *dst, const uint16_t *src, int64_t count) {
    for (int64_t t = 0; t < count; t++) dst[t] = bf16_to_f32(src[t]);
}
ORACLE_API void oracle_to_bf16(uint16_t *dst, const float *src, int64_t count) {
    for (int64_t t = 0; t < count; t++) dst[t] = f32_to_bf16_rne(src[t]);
}

/* gemm/host/gemm_lowbit_oracle.mojo:168-198: absmax after the flush (exact
 * and order-free), the row exponent, then every value scaled, rounded, clamped. */
ORACLE_API void oracle_quantize_int8(int8_t *q, int32_t *e, const float *x, int64_t rows, int64_t cols) {
    unsigned env = fpenv_enter();
    for (int64_t r = 0; r < rows; r++) {
        float best = 0.0f;
        for (int64_t c = 0; c < cols; c++) {
            float v = ftz(x[r * cols + c]);
            if (v < 0.0f) v = -v;
            if (v > best) best = v;
        }
        int ex = int8_row_exponent(best);
        e[r] = ex;
        for (int64_t c = 0; c < cols; c++) q[r * cols + c] = quantize_int8_value(x[r * cols + c], ex);
    }
    fpenv_leave(env);
}

/* gemm/host/gemm_lowbit_oracle.mojo:201-214: q * 2^e, the float32 matrix an
 * int8 weight store stands for. */
ORACLE_API void oracle_dequantize_int8(float *y, const int8_t *q, const int32_t *e, int64_t rows, int64_t cols) {
    unsigned env = fpenv_enter();
    for (int64_t r = 0; r < rows; r++)
        for (int64_t c = 0; c < cols; c++) y[r * cols + c] = dequant_int8_pinned((int32_t)q[r * cols + c], e[r]);
    fpenv_leave(env);
}

/* EXTENSION with no reference counterpart (parity unpinned): int8 codes with a
 * general float32 scale per row. One pinned product per weight, spelled like
 * the reference's dequant seam: W = ftz(mul_rn(f32(code), scale)). */
ORACLE_API void oracle_dequantize_int8_scaled(float *y, const int8_t *q, const float *scale, int64_t rows, int64_t cols) {
    unsigned env = fpenv_enter();
    for (int64_t r = 0; r < rows; r++)
        for (int64_t c = 0; c < cols; c++) {
            volatile float prod = (float)q[r * cols + c] * scale[r];
            y[r * cols + c] = ftz(prod);
        }
    fpenv_leave(env);
}

/* gemm/host/gemm_lowbit_oracle.mojo:217-251: int8i32.v1 at OP_NT, the exact
 * integer sum then one dequantization per cell. */
ORACLE_API int oracle_gemm_int8(float *c, const int8_t *qa, const int32_t *ea, const int8_t *qb, const int32_t *eb,
                                int64_t m, int64_t n, int64_t k) {
    if (m < 0 || n < 0 || k < 0 || k > 131072) return 1;
    unsigned env = fpenv_enter();
    for (int64_t i = 0; i < m; i++)
        for (int64_t j = 0; j < n; j++) {
            int32_t acc = 0;
            for (int64_t p = 0; p < k; p++) acc += (int32_t)qa[i * k + p] * (int32_t)qb[j * k + p];
            c[i * n + j] = dequant_int8_pinned(acc, (int64_t)ea[i] + (int64_t)eb[j]);
        }
    fpenv_leave(env);
    return 0;
}

/* ---- the fifteen-bit profile, mojolearn.identical.gemm.int15i64.v1 (gemm/IDENTICAL_LOWBIT_CONTRACT.md section 6) ---- */

/* checks/numerics_int15.mojo:57-68 (clause W-1): e = floor(log2 absmax) - 13; an all-zero row takes 0. */
static inline int int15_row_exponent(float absmax) {
    float a = ftz(absmax);
    if (a == 0.0f || a != a) return 0;
    return f32_exponent(a) - 13;
}

/* checks/numerics_int15.mojo:71-104 (W-2): clamp(rne(ftz(ftz(x) * 2^-e)), -16383, 16383); a NaN, before or after the
 * scaling (0 * inf), codes to 0. */
static inline int16_t quantize_int15_value(float x, int e) {
    if (x != x) return 0;
    volatile float prod = ftz(x) * pow2_f32(-(int64_t)e);
    float s = ftz(prod);
    if (s != s) return 0;
    float r = round_half_even(s);
    if (r > 16383.0f) r = 16383.0f;
    if (r < -16383.0f) r = -16383.0f;
    return (int16_t)(int)r;
}

/* checks/numerics_int15.mojo:139-182 (W-6): the Int64 sum as a float32, round to nearest even: a 24-bit high part and a
 * 24-bit low part, one exact scaling and ONE rounding addition; at and above 2^48 the low sixteen bits become a sticky bit. */
static inline float i64_to_f32_pinned(int64_t v) {
    int neg = v < 0;
    uint64_t mag = (uint64_t)v;
    if (neg) mag = (uint64_t)0 - mag;
    int reduced = 0;
    if (mag >= ((uint64_t)1 << 48)) {
        uint64_t lost = mag & 0xFFFFu;
        mag >>= 16;
        if (lost != 0) mag |= 1u;
        reduced = 1;
    }
    float hi = (float)(int32_t)(mag >> 24);
    float lo = (float)(int32_t)(mag & 0xFFFFFFu);
    volatile float scaled = hi * 16777216.0f;
    volatile float r = scaled + lo;
    if (reduced) r = r * 65536.0f;
    return neg ? -r : r;
}

/* checks/numerics_int15.mojo:185-192 (W-7) */
static inline float dequant_int15_pinned(int64_t acc, int64_t e_sum) {
    volatile float prod = i64_to_f32_pinned(acc) * pow2_f32(e_sum);
    return ftz(prod);
}

/* gemm/host/gemm_int15_oracle.mojo:71-86 and :109-116: the row's absmax (int8i32.v1's), the codes, and their two int8
 * planes: lo = code mod 128 as a floor modulus in [0, 127], hi = floor(code / 128) in [-128, 127] (W-3). */
ORACLE_API void oracle_quantize_int15(int8_t *hi, int8_t *lo, int32_t *e, const float *x, int64_t rows, int64_t cols) {
    unsigned env = fpenv_enter();
    for (int64_t r = 0; r < rows; r++) {
        float best = 0.0f;
        for (int64_t c = 0; c < cols; c++) {
            float v = ftz(x[r * cols + c]);
            if (v < 0.0f) v = -v;
            if (v > best) best = v;
        }
        int ex = int15_row_exponent(best);
        e[r] = ex;
        for (int64_t c = 0; c < cols; c++) {
            int32_t code = quantize_int15_value(x[r * cols + c], ex);
            lo[r * cols + c] = (int8_t)(code & 127);
            hi[r * cols + c] = (int8_t)(code >> 7); /* arithmetic shift of a negative int32: gcc and clang, as the reference's */
        }
    }
    fpenv_leave(env);
}

/* gemm/host/gemm_int15_oracle.mojo:98-108: ftz(code * 2^e) through the pinned seam. */
ORACLE_API void oracle_dequantize_int15(float *y, const int8_t *hi, const int8_t *lo, const int32_t *e, int64_t rows, int64_t cols) {
    unsigned env = fpenv_enter();
    for (int64_t r = 0; r < rows; r++)
        for (int64_t c = 0; c < cols; c++) {
            int64_t code = (int64_t)hi[r * cols + c] * 128 + (int64_t)lo[r * cols + c];
            y[r * cols + c] = dequant_int15_pinned(code, e[r]);
        }
    fpenv_leave(env);
}

/* gemm/host/gemm_int15_oracle.mojo:124-134, :185-210: OP_NT, the exact Int64 sum of code products, one dequantisation per
 * cell; k above INT15_MAX_K = 65536 is refused. */
ORACLE_API int oracle_gemm_int15(float *c, const int8_t *ah, const int8_t *al, const int32_t *ea, const int8_t *bh, const int8_t *bl,
                                 const int32_t *eb, int64_t m, int64_t n, int64_t k) {
    if (m < 0 || n < 0 || k < 0 || k > 65536) return 1;
    unsigned env = fpenv_enter();
    for (int64_t i = 0; i < m; i++)
        for (int64_t j = 0; j < n; j++) {
            int64_t acc = 0;
            for (int64_t p = 0; p < k; p++) {
                int32_t a = (int32_t)ah[i * k + p] * 128 + (int32_t)al[i * k + p];
                int32_t b = (int32_t)bh[j * k + p] * 128 + (int32_t)bl[j * k + p];
                acc += (int64_t)(a * b);
            }
            c[i * n + j] = dequant_int15_pinned(acc, (int64_t)ea[i] + (int64_t)eb[j]);
        }
    fpenv_leave(env);
    return 0;
}

/* ---- identity-card helpers -------------------------------------------------- */

/* core/identity_trace.mojo:22-31, :89-114: FNV-1a 64 over little-endian bytes. */
ORACLE_API uint64_t oracle_fnv1a64(const void *data, int64_t nbytes) {
    const uint8_t *p = (const uint8_t *)data;
    uint64_t h = 0xCBF29CE484222325ull;
    for (int64_t t = 0; t < nbytes; t++) { h ^= p[t]; h *= 0x100000001B3ull; }
    return h;
}

/* bench/gemm_card_main.mojo:292-311: a value exact in float32,
 * (mix(i, salt) % 2097151 - 1048575) / 2^20. */
ORACLE_API void oracle_card_fill(float *dst, int64_t count, int64_t salt) {
    for (int64_t i = 0; i < count; i++) {
        uint64_t z = (uint64_t)(i + 1) * 0x9E3779B97F4A7C15ull + (uint64_t)(salt + 1) * 0xBF58476D1CE4E5B9ull;
        z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
        z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
        z ^= z >> 31;
        int64_t num = (int64_t)(z % 2097151ull) - 1048575;
        dst[i] = (float)num / 1048576.0f;
    }
}

ORACLE_API int oracle_abi(void) { return 1; }
