/*
 * CPU oracle for the decoder-block seams around the identical-mode matrix
 * product: normalisation, rotary table, eager attention with serial key-axis
 * chains, activations, residuals, embedding gather, greedy argmax.
 *
 * THIS FILE IS TEST INFRASTRUCTURE (see oracle.c). It restates, in plain C,
 * the reference's host oracle for one decoder block and the portable math it
 * is built from. Paths are relative to the reference project's root:
 *   seams S1..S23          transformer/IDENTICAL_TRANSFORMER_CONTRACT.md:207-240
 *   block forward          transformer/checks/transformer_oracle.mojo:1762-2658
 *   norm variants          transformer/checks/transformer_oracle.mojo:1223-1341
 *   bias, rotary apply     transformer/checks/transformer_oracle.mojo:1344-1372, :1375-1500
 *   rotary table           transformer/checks/transformer_oracle.mojo:415-640
 *   span helpers           core/host_lanes.mojo:225-362
 *   portable math          checks/numerics.mojo:370-639, :1025-1054, :1079-1094, :1177-1337
 *   embedding gather       embedding/checks/embedding_oracle.mojo:369-382
 * The portable functions are the published Cephes single-precision
 * algorithms (expf, logf, sinf/cosf, tanhf, erff/erfcf) in the reference's
 * operation order; every `fmaf` below is one of the reference's explicit
 * fused multiply-adds and every other operation is a separate IEEE rounding
 * (the file is compiled with -ffp-contract=off).
 *
 * Pinned by the verify table's `transformer`, `transformer-bf16w` and
 * `transformer-int8w` infer cells on nine fixtures (tests/test_oracle_decoder.py).
 */
#include <math.h>
#include <pthread.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#include <xmmintrin.h>

#define DEC_API __attribute__((visibility("default")))

int rows_gemm(float *c, const float *a, const float *b, int op, int64_t m, int64_t n, int64_t k, int threads);

static inline uint32_t f2u(float x) { uint32_t u; memcpy(&u, &x, 4); return u; }
static inline float u2f(uint32_t u) { float x; memcpy(&x, &u, 4); return x; }
static inline float ftz(float x) {
    uint32_t b = f2u(x);
    if ((b & 0x7F800000u) == 0u) return u2f(b & 0x80000000u);
    return x;
}
/* every product, sum and quotient goes through a volatile so that no compiler can fuse or reassociate it */
static inline float mul(float a, float b) { volatile float r = a * b; return r; }
static inline float add(float a, float b) { volatile float r = a + b; return r; }
static inline float sub(float a, float b) { volatile float r = a - b; return r; }
static inline float quo(float a, float b) { volatile float r = a / b; return r; }
#define QNAN u2f(0x7FC00000u)
#define PINF u2f(0x7F800000u)

/* ---- portable math ------------------------------------------------------------ */

/* checks/numerics.mojo:370-413 */
DEC_API float p_expf(float x) {
    if (x != x) return x;
    if (x > 88.722835f) return PINF;
    if (x < -87.33655f) return 0.0f;
    float t = fmaf(x, 1.4426950408889634f, 0.5f);
    float zf = floorf(t);
    int32_t k = (int32_t)zf;
    float r = fmaf(zf, -0.693359375f, x);
    r = fmaf(zf, 2.12194440e-4f, r);
    float q = 1.9875691500e-4f;
    q = fmaf(q, r, 1.3981999507e-3f);
    q = fmaf(q, r, 8.3334519073e-3f);
    q = fmaf(q, r, 4.1665795894e-2f);
    q = fmaf(q, r, 1.6666665459e-1f);
    q = fmaf(q, r, 5.0000001201e-1f);
    float r2 = mul(r, r);
    float y = fmaf(q, r2, r);
    y = add(y, 1.0f);
    int32_t k1 = k >> 1, k2 = k - k1;
    y = mul(y, u2f((uint32_t)(k1 + 127) << 23));
    y = mul(y, u2f((uint32_t)(k2 + 127) << 23));
    if (y < 1.1754943508222875e-38f) return 0.0f;
    return y;
}

/* checks/numerics.mojo:444-465 */
static float cephes_logf_core(float t, int e) {
    float z = mul(t, t);
    float p = 7.0376836292e-2f;
    p = fmaf(p, t, -1.1514610310e-1f);
    p = fmaf(p, t, 1.1676998740e-1f);
    p = fmaf(p, t, -1.2420140846e-1f);
    p = fmaf(p, t, 1.4249322787e-1f);
    p = fmaf(p, t, -1.6668057665e-1f);
    p = fmaf(p, t, 2.0000714765e-1f);
    p = fmaf(p, t, -2.4999993993e-1f);
    p = fmaf(p, t, 3.3333331174e-1f);
    float tz = mul(t, z);
    float y = mul(tz, p);
    float ef = (float)e;
    y = fmaf(ef, -2.12194440e-4f, y);
    y = fmaf(-0.5f, z, y);
    float r = add(t, y);
    return fmaf(ef, 0.693359375f, r);
}

/* checks/numerics.mojo:416-441 */
DEC_API float p_logf(float x) {
    if (x != x) return x;
    if (fabsf(x) < 1.1754943508222875e-38f) x = 0.0f;
    if (x == 0.0f) return u2f(0xFF800000u);
    if (x < 0.0f) return QNAN;
    if (x == PINF) return x;
    uint32_t bits = f2u(x);
    int e = (int)((bits >> 23) & 0xFFu) - 126;
    float m = u2f((bits & 0x007FFFFFu) | 0x3F000000u);
    if (m < 0.7071067811865476f) { e -= 1; m = add(m, m); }
    return cephes_logf_core(sub(m, 1.0f), e);
}

/* checks/numerics.mojo:623-637 */
DEC_API float p_powf(float x, float p) {
    if (p == 0.0f) return 1.0f;
    if (x != x || p != p) return QNAN;
    if (x < 0.0f) return QNAN;
    if (x == 0.0f) return p > 0.0f ? 0.0f : PINF;
    return p_expf(mul(p, p_logf(x)));
}

/* checks/numerics.mojo:503-571: Newton from the exponent-halving seed, then the best of five neighbours by residual */
DEC_API float p_sqrtf(float x) {
    if (x != x) return x;
    if (fabsf(x) < 1.1754943508222875e-38f) return 0.0f;
    if (x < 0.0f) return QNAN;
    if (x == PINF) return x;
    int scaled = 0;
    if (x < u2f(0x0F800000u)) { x = mul(x, u2f(0x5F800000u)); scaled = 1; }
    float y = u2f((f2u(x) >> 1) + 0x1FBD1DF5u);
    for (int it = 0; it < 3; it++) y = mul(0.5f, add(y, quo(x, y)));
    uint32_t yb = f2u(y);
    float best = y, r_best = fabsf(fmaf(-y, y, x));
    for (int kk = 0; kk < 4; kk++) {
        uint32_t delta = (uint32_t)(kk / 2 + 1);
        float c = u2f((kk % 2 == 0) ? yb - delta : yb + delta);
        float r = fabsf(fmaf(-c, c, x));
        if (r < r_best) { best = c; r_best = r; }
    }
    if (scaled) best = mul(best, u2f(0x2F800000u));
    return best;
}

/* checks/numerics.mojo:1035-1037 */
DEC_API float p_divf(float a, float b) { return ftz(quo(ftz(a), ftz(b))); }

/* checks/numerics.mojo:1040-1054 */
DEC_API float p_rsqrtf(float x_in) {
    float x = ftz(x_in);
    if (x != x) return x;
    if (x < 0.0f) return QNAN;
    float s = p_sqrtf(x);
    if (s == 0.0f) return PINF;
    if (s == PINF) return 0.0f;
    return p_divf(1.0f, s);
}

/* checks/numerics.mojo:583-620: octant, three-part Cody-Waite reduction, both polynomials */
static float cephes_sincosf_core(float x_abs, float sign_in, int is_cos) {
    float x = x_abs;
    int j = (int)floorf(mul(x, 1.27323954473516f));
    float yj = (float)j;
    if (j & 1) { j += 1; yj = add(yj, 1.0f); }
    j &= 7;
    x = fmaf(yj, -0.78515625f, x);
    x = fmaf(yj, -2.4187564849853515625e-4f, x);
    x = fmaf(yj, -3.77489497744594108e-8f, x);
    float sign = sign_in;
    if (j > 3) { j -= 4; sign = -sign; }
    if (is_cos && j > 1) sign = -sign;
    float z = mul(x, x);
    int use_sin_poly = (j == 1 || j == 2);
    if (!is_cos) use_sin_poly = !use_sin_poly;
    float y;
    if (use_sin_poly) {
        float p = -1.9515295891e-4f;
        p = fmaf(p, z, 8.3321608736e-3f);
        p = fmaf(p, z, -1.6666654611e-1f);
        y = fmaf(mul(x, z), p, x);
    } else {
        float p = 2.443315711809948e-5f;
        p = fmaf(p, z, -1.388731625493765e-3f);
        p = fmaf(p, z, 4.166664568298827e-2f);
        y = fmaf(mul(z, z), p, fmaf(-0.5f, z, 1.0f));
    }
    return mul(sign, y);
}
/* checks/numerics.mojo:574-580, :1177-1187 */
DEC_API float p_cosf(float x) {
    if (x != x || fabsf(x) == PINF) return QNAN;
    return cephes_sincosf_core(fabsf(x), 1.0f, 1);
}
DEC_API float p_sinf(float x_in) {
    if (x_in != x_in || fabsf(x_in) == PINF) return QNAN;
    float x = ftz(x_in);
    float sign = (f2u(x) & 0x80000000u) ? -1.0f : 1.0f;
    return cephes_sincosf_core(fabsf(x), sign, 0);
}

/* checks/numerics.mojo:1088-1094: x / (1 + exp(-x)), ONE division */
DEC_API float p_siluf(float x) {
    if (x != x) return x;
    float e = p_expf(-x);
    return p_divf(x, add(e, 1.0f));
}

/* checks/numerics.mojo:1190-1219 */
DEC_API float p_tanhf(float x_in) {
    float xx = ftz(x_in);
    if (xx != xx) return xx;
    if (xx == 0.0f) return xx;
    float x = fabsf(xx);
    if (x > u2f(0x42317218u)) return xx < 0.0f ? -1.0f : 1.0f;
    if (x >= 0.625f) {
        float e = p_expf(add(x, x));
        float q = p_divf(2.0f, add(e, 1.0f));
        float z = sub(1.0f, q);
        return xx < 0.0f ? -z : z;
    }
    float zs = mul(x, x);
    float p = -5.70498872745e-3f;
    p = fmaf(p, zs, 2.06390887954e-2f);
    p = fmaf(p, zs, -5.37397155531e-2f);
    p = fmaf(p, zs, 1.33314422036e-1f);
    p = fmaf(p, zs, -3.33332819422e-1f);
    return fmaf(mul(p, zs), xx, xx);
}

/* checks/numerics.mojo:1222-1260 */
static float cephes_erfcf_ge1(float a) {
    float x = fabsf(a);
    float z = -mul(x, x);
    if (z < u2f(0xC2B17218u)) return a < 0.0f ? 2.0f : 0.0f;
    z = p_expf(z);
    float q = p_divf(1.0f, x);
    float y = mul(q, q);
    float p;
    if (x < 2.0f) {
        p = 2.326819970068386e-2f;
        p = fmaf(p, y, -1.387039388740657e-1f);
        p = fmaf(p, y, 3.687424674597105e-1f);
        p = fmaf(p, y, -5.824733027278666e-1f);
        p = fmaf(p, y, 6.210004621745983e-1f);
        p = fmaf(p, y, -4.944515323274145e-1f);
        p = fmaf(p, y, 3.404879937665872e-1f);
        p = fmaf(p, y, -2.741127028184656e-1f);
        p = fmaf(p, y, 5.638259427386472e-1f);
    } else {
        p = -10.47766399936249f;
        p = fmaf(p, y, 12.97719955372516f);
        p = fmaf(p, y, -7.495518717768503f);
        p = fmaf(p, y, 2.921019019210786f);
        p = fmaf(p, y, -1.015265279202700f);
        p = fmaf(p, y, 4.218463358204948e-1f);
        p = fmaf(p, y, -2.820767439740514e-1f);
        p = fmaf(p, y, 5.641895067754075e-1f);
    }
    float t = ftz(mul(z, q));
    float r = ftz(mul(t, p));
    if (a < 0.0f) r = sub(2.0f, r);
    return r;
}
/* checks/numerics.mojo:1263-1282 */
DEC_API float p_erff(float x_in) {
    float x = ftz(x_in);
    if (x != x) return x;
    if (fabsf(x) > 1.0f) return sub(1.0f, cephes_erfcf_ge1(x));
    float z = mul(x, x);
    float p = 7.853861353153693e-5f;
    p = fmaf(p, z, -8.010193625184903e-4f);
    p = fmaf(p, z, 5.188327685732524e-3f);
    p = fmaf(p, z, -2.685381193529856e-2f);
    p = fmaf(p, z, 1.128358514861418e-1f);
    p = fmaf(p, z, -3.761262582423300e-1f);
    p = fmaf(p, z, 1.128379165726710f);
    return mul(x, p);
}
/* checks/numerics.mojo:1285-1296 */
DEC_API float p_gelu_erf(float x_in) {
    float x = ftz(x_in);
    if (x != x) return x;
    float e = p_erff(p_divf(x, u2f(0x3FB504F3u)));
    float s = add(1.0f, e);
    float h = ftz(mul(x, 0.5f));
    return ftz(mul(h, s));
}
/* checks/numerics.mojo:1299-1316 */
DEC_API float p_gelu_tanh(float x_in) {
    float x = ftz(x_in);
    if (x != x) return x;
    float c3 = u2f(0x3D372713u), kk = u2f(0x3F4C422Au);
    float x2 = ftz(mul(x, x));
    float x3 = ftz(mul(x2, x));
    float cx = ftz(mul(c3, x3));
    float inner = ftz(add(x, cx));
    float arg = ftz(mul(kk, inner));
    float t = p_tanhf(arg);
    float s = add(1.0f, t);
    float h = ftz(mul(x, 0.5f));
    return ftz(mul(h, s));
}

/* checks/numerics.mojo:1319-1337: a maximum that does not depend on argument order or fold shape */
static inline uint32_t order_key(float v) {
    uint32_t b = f2u(v);
    return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}
DEC_API float p_fmaxf(float a_in, float b_in) {
    if (a_in != a_in || b_in != b_in) return QNAN;
    float a = ftz(a_in), b = ftz(b_in);
    return order_key(b) > order_key(a) ? b : a;
}

/* ---- a parallel loop over independent items (rows, heads): which thread runs an item moves no bit ---- */
typedef void (*par_body_t)(int64_t item, void *ctx);
typedef struct { par_body_t body; void *ctx; int64_t lo, hi; } par_span_t;
static void *par_run(void *arg) {
    par_span_t *sp = (par_span_t *)arg;
    unsigned env = _mm_getcsr();
    _mm_setcsr(env & ~(0x8000u | 0x0040u)); /* IEEE gradual underflow in this thread too: the flush is spelled, not inherited */
    for (int64_t i = sp->lo; i < sp->hi; i++) sp->body(i, sp->ctx);
    _mm_setcsr(env);
    return NULL;
}
static void par_for(int64_t items, int threads, par_body_t body, void *ctx) {
    if (threads < 1) threads = 1;
    if (threads > 64) threads = 64;
    if ((int64_t)threads > items) threads = (int)(items > 0 ? items : 1);
    par_span_t sp[64];
    pthread_t th[64];
    for (int t = 0; t < threads; t++) {
        sp[t].body = body; sp[t].ctx = ctx;
        sp[t].lo = items * t / threads; sp[t].hi = items * (t + 1) / threads;
        if (t + 1 < threads) pthread_create(&th[t], NULL, par_run, &sp[t]);
    }
    par_run(&sp[threads - 1]);
    for (int t = 0; t + 1 < threads; t++) pthread_join(th[t], NULL);
}

/* ---- block configuration -------------------------------------------------------- */

enum { NORM_RMS = 0, NORM_LAYER = 1, NORM_RMS_OFFSET = 2 };
enum { MLP_SWIGLU = 0, MLP_GELU_ERF = 1, MLP_GELU_TANH = 2, MLP_SILU = 3, MLP_GEGLU_ERF = 4, MLP_GEGLU_TANH = 5 };
/* weight slots of one block (NULL when the option is off) */
enum { W_NORM1 = 0, W_NORM1_B, W_Q, W_Q_B, W_K, W_K_B, W_V, W_V_B, W_O, W_O_B, W_NORM2, W_NORM2_B, W_GATE, W_GATE_B, W_UP,
       W_UP_B, W_DOWN, W_DOWN_B, W_SLOTS };

typedef struct {
    int32_t d_model, n_heads, n_kv_heads, head_dim, inter;
    int32_t norm_kind, norm_bias, qkv_bias, o_bias, mlp_kind, mlp_bias;
    int32_t rope;   /* 1 = rotary on q and k (the reference's block); 0 = none (extension for learned positions) */
    int32_t window; /* 0 = full causal */
    float norm_eps, rope_theta;
    /* the option record of transformer/block_options.mojo:40-70 beyond the fields above */
    int32_t rope_scaling;              /* 0 none, 1 linear, 2 llama3 */
    float rope_factor, rope_low_freq_factor, rope_high_freq_factor;
    int32_t rope_original_max_positions;
    int32_t rope_dim;                  /* 0 = head_dim (partial rotary otherwise) */
    int32_t qk_norm;                   /* an RMSNorm over each head's vector of q and of k, before the rotation */
    float attn_softcap;                /* 0 = none */
} block_cfg_t;
/* two more weight slots when qk_norm is on */
enum { W_Q_NORM = W_SLOTS, W_K_NORM, W_SLOTS_OPT };

/* transformer/checks/transformer_oracle.mojo:1223-1341 */
typedef struct { float *out; const float *src, *w, *bias; int64_t dm; float eps; int kind; } norm_ctx_t;
static void norm_row(int64_t t, void *vctx) {
    const norm_ctx_t *c = (const norm_ctx_t *)vctx;
    const int64_t dm = c->dm;
    const float *x = c->src + t * dm, *w = c->w, *bias = c->bias;
    float *out = c->out;
    const float eps = c->eps;
    const int kind = c->kind;
    if (kind == NORM_LAYER) {
        float acc = 0.0f;
        for (int64_t j = 0; j < dm; j++) acc = ftz(add(ftz(acc), ftz(x[j])));
        float mean = ftz(p_divf(acc, (float)dm));
        float acc2 = 0.0f;
        for (int64_t j = 0; j < dm; j++) {
            float dev = ftz(sub(ftz(x[j]), mean));
            acc2 = ftz(fmaf(dev, dev, acc2));
        }
        float variance = ftz(p_divf(acc2, (float)dm));
        float rstd = ftz(p_rsqrtf(ftz(add(variance, eps))));
        for (int64_t j = 0; j < dm; j++) {
            float dev = ftz(sub(ftz(x[j]), mean));
            float inner = ftz(mul(dev, rstd));
            float y = ftz(mul(ftz(w[j]), inner));
            if (bias) y = ftz(add(ftz(y), ftz(bias[j])));
            out[t * dm + j] = y;
        }
        return;
    }
    float acc = 0.0f;
    for (int64_t j = 0; j < dm; j++) {
        float xj = ftz(x[j]);
        acc = ftz(fmaf(xj, xj, acc));
    }
    float mean = ftz(p_divf(acc, (float)dm));
    float rstd = ftz(p_rsqrtf(ftz(add(mean, eps))));
    for (int64_t j = 0; j < dm; j++) {
        float inner = ftz(mul(ftz(x[j]), rstd));
        float wj = ftz(w[j]);
        if (kind == NORM_RMS_OFFSET) wj = ftz(add(1.0f, wj));
        out[t * dm + j] = ftz(mul(wj, inner));
    }
}
static void norm_rows(float *out, const float *src, const float *w, const float *bias, int64_t m, int64_t dm, float eps, int kind,
                      int threads) {
    norm_ctx_t c = {out, src, w, bias, dm, eps, kind};
    par_for(m, m * dm >= 65536 ? threads : 1, norm_row, &c);
}
DEC_API void dec_norm(float *out, const float *src, const float *w, const float *bias, int64_t m, int64_t dm, float eps,
                      int kind) {
    norm_rows(out, src, w, bias, m, dm, eps, kind, 1);
}

/* transformer/checks/transformer_oracle.mojo:1344-1372 */
static void add_bias(float *buf, const float *bias, int64_t rows, int64_t width) {
    for (int64_t t = 0; t < rows; t++)
        for (int64_t j = 0; j < width; j++) buf[t * width + j] = ftz(add(ftz(buf[t * width + j]), ftz(bias[j])));
}

/* Seam S6 with the options: transformer/checks/transformer_oracle.mojo:423-497 (rope_inv_freq_scaled). Linear scaling
 * is one division by the factor; llama3 rescales by wavelength, every division through the portable division, both
 * products rounded on their own and the final add unfused. */
static float rope_inv_freq(int64_t i, int64_t rope_dim, float theta, int scaling, float factor_in, float lo_in, float hi_in,
                           int64_t original) {
    float e = ftz(p_divf((float)(2 * i), (float)rope_dim));
    float inv = ftz(p_divf(1.0f, p_powf(theta, e)));
    if (scaling == 1) {
        inv = ftz(p_divf(inv, ftz(factor_in)));
    } else if (scaling == 2) {
        float factor = ftz(factor_in), lo_f = ftz(lo_in), hi_f = ftz(hi_in), old = (float)original;
        float low_wl = ftz(p_divf(old, lo_f)), high_wl = ftz(p_divf(old, hi_f));
        float two_pi = u2f(0x40C90FDBu);
        float wl = ftz(p_divf(two_pi, inv));
        float inv_l = inv;
        if (wl > low_wl) inv_l = ftz(p_divf(inv, factor));
        int medium = !(wl < high_wl) && !(wl > low_wl);
        if (medium) {
            float ratio = ftz(p_divf(old, wl));
            float num = ftz(sub(ratio, lo_f)), den = ftz(sub(hi_f, lo_f));
            float smooth = ftz(p_divf(num, den));
            float one_minus = ftz(sub(1.0f, smooth));
            float t1 = ftz(mul(one_minus, inv_l));
            t1 = ftz(p_divf(t1, factor));
            float t2 = ftz(mul(smooth, inv_l));
            inv_l = ftz(add(ftz(t1), ftz(t2)));
        }
        inv = inv_l;
    }
    return inv;
}

/* S6-S8 with the option record: cos and sin [l, rope_dim / 2] for positions [pos0, pos0 + l) */
DEC_API void dec_rope_table_opts(float *cosv, float *sinv, int64_t pos0, int64_t l, int64_t rope_dim, float theta, int scaling,
                                 float factor, float lo, float hi, int64_t original) {
    unsigned env = _mm_getcsr();
    _mm_setcsr(env & ~(0x8000u | 0x0040u));
    int64_t half = rope_dim / 2;
    for (int64_t i = 0; i < half; i++) {
        float inv = rope_inv_freq(i, rope_dim, theta, scaling, factor, lo, hi, original);
        for (int64_t p = 0; p < l; p++) {
            float angle = ftz(mul((float)(pos0 + p), ftz(inv)));
            cosv[p * half + i] = ftz(p_cosf(angle));
            sinv[p * half + i] = ftz(p_sinf(angle));
        }
    }
    _mm_setcsr(env);
}

/* transformer/checks/transformer_oracle.mojo:539-640 (S6, S7, S8) for positions [pos0, pos0 + l) */
DEC_API void dec_rope_table(float *cosv, float *sinv, int64_t pos0, int64_t l, int64_t head_dim, float theta) {
    unsigned env = _mm_getcsr();
    _mm_setcsr(env & ~(0x8000u | 0x0040u));
    int64_t half = head_dim / 2;
    for (int64_t i = 0; i < half; i++) {
        float e = ftz(p_divf((float)(2 * i), (float)head_dim));
        float inv = ftz(p_divf(1.0f, p_powf(theta, e)));
        for (int64_t p = 0; p < l; p++) {
            float angle = ftz(mul((float)(pos0 + p), ftz(inv)));
            cosv[p * half + i] = ftz(p_cosf(angle));
            sinv[p * half + i] = ftz(p_sinf(angle));
        }
    }
    _mm_setcsr(env);
}

/* transformer/checks/transformer_oracle.mojo:1375-1500 (S9, S10): halves pairing, three roundings */
static void apply_rope(float *out, const float *src, int64_t n_head, int64_t hd, int64_t m, int64_t l, const float *cosv,
                       const float *sinv, int64_t rd) {
    /* rd = rotated columns of a head (:1433-1440 of the reference oracle): the rest pass through, flushed on load */
    int64_t half = rd / 2, width = n_head * hd;
    for (int64_t t = 0; t < m; t++) {
        int64_t li = t % l;
        for (int64_t h = 0; h < n_head; h++) {
            int64_t base = t * width + h * hd;
            for (int64_t j = 0; j < hd; j++) {
                if (j >= rd) { out[base + j] = ftz(src[base + j]); continue; }
                int64_t ci = j < half ? j : j - half;
                float rot = j < half ? -ftz(src[base + j + half]) : ftz(src[base + j - half]);
                float c = ftz(cosv[li * half + ci]), s = ftz(sinv[li * half + ci]);
                float pa = ftz(mul(ftz(src[base + j]), c));
                float pb = ftz(mul(rot, s));
                out[base + j] = ftz(add(ftz(pa), ftz(pb)));
            }
        }
    }
}

static float *falloc(int64_t n) { return (float *)malloc(sizeof(float) * (size_t)(n > 0 ? n : 1)); }

/*
 * Eager attention of one call (S11-S19): ctx[b*l, n_heads*head_dim] from rotated queries q[b*l, n_heads*head_dim] and
 * caches [b, n_kv_heads, cap, head_dim] holding `used` positions, this call's l included; window 0 = full causal.
 * transformer/checks/transformer_oracle.mojo:2373-2546. One (sequence, head) pair per item: heads never read each other.
 */
typedef struct {
    float *ctx; const float *qr, *kcache, *vcache;
    int64_t l, nh, nkv, hd, cap, key_lo, s, own0, window;
    float softcap;
} attn_ctx_t;
static void attn_pair(int64_t item, void *vctx) {
    const attn_ctx_t *c = (const attn_ctx_t *)vctx;
    const int64_t l = c->l, nh = c->nh, nkv = c->nkv, hd = c->hd, cap = c->cap, key_lo = c->key_lo, s = c->s, own0 = c->own0,
                  window = c->window, qw = nh * hd, n_rep = nh / nkv;
    const int64_t bb = item / nh, h = item % nh, kv = h / n_rep;
    /* attention scale, computed once: ftz(rsqrt(head_dim)) (transformer/checks/transformer_fixture.mojo:134-136) */
    const float scale = ftz(p_rsqrtf((float)hd));
    const float mfill = u2f(0xFF7FFFFFu), ufill = 0.0f;
    float *qmat = falloc(l * hd), *kmat = falloc(s * hd), *cell = falloc(l * s), *ex = falloc(s), *acc = falloc(hd);
    for (int64_t qi = 0; qi < l; qi++) memcpy(qmat + qi * hd, c->qr + (bb * l + qi) * qw + h * hd, sizeof(float) * hd);
    const float *kbase = c->kcache + ((bb * nkv + kv) * cap + key_lo) * hd;
    const float *vbase = c->vcache + ((bb * nkv + kv) * cap + key_lo) * hd;
    memcpy(kmat, kbase, sizeof(float) * s * hd);
    rows_gemm(cell, qmat, kmat, 1, l, s, hd, 1); /* S11: gemm fp32.v1, k = head_dim */
    _mm_setcsr(_mm_getcsr() & ~(0x8000u | 0x0040u));
    for (int64_t qi = 0; qi < l; qi++) {
        int64_t jlo = 0, jhi = own0 + qi;
        if (jhi > s - 1) jhi = s - 1;
        if (window > 0) { jlo = own0 + qi - window + 1; if (jlo < 0) jlo = 0; }
        float *row = cell + qi * s;
        /* S12 scale, S13 mask ADD (never a select), S14 row max over the WHOLE row */
        float mx = 0.0f;
        for (int64_t j = 0; j < s; j++) {
            float sc = ftz(mul(ftz(row[j]), scale));
            if (f2u(c->softcap) != 0u) { /* transformer_oracle.mojo:2269-2281: after the scale, before the mask */
                const float cap_f = ftz(c->softcap);
                const float th = ftz(p_tanhf(ftz(p_divf(sc, cap_f))));
                sc = ftz(mul(th, cap_f));
            }
            float mk = ftz(add(ftz(sc), (j < jlo || j > jhi) ? mfill : ufill));
            row[j] = mk;
            mx = j == 0 ? ftz(mk) : p_fmaxf(mx, ftz(mk));
        }
        float fm = ftz(mx);
        /* S15, S16 over the visible keys; S17 serial denominator; S18 one division per weight */
        float den = 0.0f;
        for (int64_t j = jlo; j <= jhi; j++) {
            ex[j] = ftz(p_expf(ftz(sub(ftz(row[j]), fm))));
            den = ftz(add(ftz(den), ftz(ex[j])));
        }
        den = ftz(den);
        for (int64_t j = jlo; j <= jhi; j++) ex[j] = ftz(p_divf(ftz(ex[j]), den));
        /* S19: serial ascending value sum, one fused multiply-add per key (not a GEMM). The keys are the outer loop and
         * the features the inner one: each feature's chain still sees its keys in ascending order, one accumulator. */
        float *o = c->ctx + (bb * l + qi) * qw + h * hd;
        for (int64_t d = 0; d < hd; d++) acc[d] = 0.0f;
        for (int64_t j = jlo; j <= jhi; j++) {
            const float wj = ftz(ex[j]);
            const float *vr = vbase + j * hd;
            for (int64_t d = 0; d < hd; d++) acc[d] = ftz(fmaf(wj, ftz(vr[d]), acc[d]));
        }
        for (int64_t d = 0; d < hd; d++) o[d] = acc[d];
    }
    free(qmat); free(kmat); free(cell); free(ex); free(acc);
}
DEC_API int dec_attention(float *ctx, const float *qr, const float *kcache, const float *vcache, int64_t b, int64_t l, int64_t nh,
                          int64_t nkv, int64_t hd, int64_t cap, int64_t used, int64_t window, float softcap, int threads) {
    if (b <= 0 || l <= 0 || nh <= 0 || nkv <= 0 || nh % nkv != 0 || hd <= 0 || used < l || used > cap) return 1;
    const int64_t pos0 = used - l;
    int64_t key_lo = 0;
    if (window > 0 && pos0 - (window - 1) > 0) key_lo = pos0 - (window - 1);
    attn_ctx_t c = {ctx, qr, kcache, vcache, l, nh, nkv, hd, cap, key_lo, used - key_lo, pos0 - key_lo, window, softcap};
    par_for(b * nh, threads, attn_pair, &c);
    return 0;
}

/* S20, S21: the activation of one row of the MLP (rows are independent) */
typedef struct { float *act; const float *gate, *up; int64_t inter; int mlp_kind, gated; } act_ctx_t;
static void act_row(int64_t t, void *vctx) {
    const act_ctx_t *c = (const act_ctx_t *)vctx;
    for (int64_t i = t * c->inter; i < (t + 1) * c->inter; i++) {
        float z = ftz(c->gated ? c->gate[i] : c->up[i]);
        float a;
        if (c->mlp_kind == MLP_SWIGLU || c->mlp_kind == MLP_SILU) a = ftz(p_siluf(z)); /* S20 */
        else if (c->mlp_kind == MLP_GELU_TANH || c->mlp_kind == MLP_GEGLU_TANH) a = ftz(p_gelu_tanh(z));
        else a = ftz(p_gelu_erf(z));
        c->act[i] = c->gated ? ftz(mul(ftz(a), ftz(c->up[i]))) : a; /* S21 */
    }
}

/*
 * One decoder block, forward, with its KV cache. x and y are [b, l, d_model];
 * kcache / vcache are [b, n_kv_heads, cap, head_dim] and hold `used` positions
 * on entry, `used + l` on exit. Returns 0, or 1 on a refusal.
 * transformer/checks/transformer_oracle.mojo:1762-2658 (eager attention arm).
 */
DEC_API int dec_block_forward(const block_cfg_t *cfg, const float *const *w, const float *x, float *y, int64_t b, int64_t l,
                              float *kcache, float *vcache, int64_t cap, int64_t used, int threads) {
    const int64_t dm = cfg->d_model, nh = cfg->n_heads, nkv = cfg->n_kv_heads, hd = cfg->head_dim, inter = cfg->inter;
    if (b <= 0 || l <= 0 || nh <= 0 || nkv <= 0 || nh % nkv != 0 || (hd & 1) || dm <= 0 || inter <= 0) return 1;
    const int64_t qw = nh * hd, kw = nkv * hd, m = b * l;
    const int64_t pos0 = used, s_abs = pos0 + l;
    if (s_abs > cap) return 1;
    const int64_t window = cfg->window;
    unsigned env = _mm_getcsr();
    _mm_setcsr(env & ~(0x8000u | 0x0040u));

    float *n1 = falloc(m * dm), *q = falloc(m * qw), *k = falloc(m * kw), *v = falloc(m * kw);
    norm_rows(n1, x, w[W_NORM1], cfg->norm_bias ? w[W_NORM1_B] : NULL, m, dm, cfg->norm_eps, cfg->norm_kind, threads);
    rows_gemm(q, n1, w[W_Q], 1, m, qw, dm, threads);
    rows_gemm(k, n1, w[W_K], 1, m, kw, dm, threads);
    rows_gemm(v, n1, w[W_V], 1, m, kw, dm, threads);
    if (cfg->qkv_bias) { add_bias(q, w[W_Q_B], m, qw); add_bias(k, w[W_K_B], m, kw); add_bias(v, w[W_V_B], m, kw); }
    if (cfg->qk_norm) {
        /* transformer_oracle.mojo:1950-1975: an RMSNorm over each head's vector of q and of k, before the rotation; the
         * offset form when the block's norm is the offset form, the plain form otherwise, never a bias */
        const int kind = cfg->norm_kind == NORM_RMS_OFFSET ? NORM_RMS_OFFSET : NORM_RMS;
        float *qn = falloc(m * qw), *kn = falloc(m * kw);
        norm_rows(qn, q, w[W_Q_NORM], NULL, m * nh, hd, cfg->norm_eps, kind, threads);
        norm_rows(kn, k, w[W_K_NORM], NULL, m * nkv, hd, cfg->norm_eps, kind, threads);
        memcpy(q, qn, sizeof(float) * (size_t)(m * qw));
        memcpy(k, kn, sizeof(float) * (size_t)(m * kw));
        free(qn); free(kn);
        _mm_setcsr(env & ~(0x8000u | 0x0040u));
    }
    float *qr = q, *kr = k;
    if (cfg->rope) {
        const int64_t rd = cfg->rope_dim > 0 ? cfg->rope_dim : hd;
        if (rd > hd || (rd & 1)) return 1;
        float *cosv = falloc(l * (rd / 2)), *sinv = falloc(l * (rd / 2));
        dec_rope_table_opts(cosv, sinv, pos0, l, rd, cfg->rope_theta, cfg->rope_scaling, cfg->rope_factor, cfg->rope_low_freq_factor,
                            cfg->rope_high_freq_factor, cfg->rope_original_max_positions);
        _mm_setcsr(env & ~(0x8000u | 0x0040u));
        qr = falloc(m * qw);
        kr = falloc(m * kw);
        apply_rope(qr, q, nh, hd, m, l, cosv, sinv, rd);
        apply_rope(kr, k, nkv, hd, m, l, cosv, sinv, rd);
        free(cosv); free(sinv);
    }
    /* cache append (a copy, not a seam) */
    for (int64_t t = 0; t < m; t++) {
        int64_t bb = t / l, li = t % l;
        for (int64_t kv = 0; kv < nkv; kv++)
            for (int64_t d = 0; d < hd; d++) {
                int64_t dst = ((bb * nkv + kv) * cap + pos0 + li) * hd + d;
                kcache[dst] = kr[t * kw + kv * hd + d];
                vcache[dst] = v[t * kw + kv * hd + d];
            }
    }
    float *ctx = falloc(m * qw);
    dec_attention(ctx, qr, kcache, vcache, b, l, nh, nkv, hd, cap, s_abs, window, cfg->attn_softcap, threads);
    _mm_setcsr(env & ~(0x8000u | 0x0040u));
    float *op = falloc(m * dm), *r1 = falloc(m * dm);
    rows_gemm(op, ctx, w[W_O], 1, m, dm, qw, threads);
    _mm_setcsr(env & ~(0x8000u | 0x0040u));
    if (cfg->o_bias) add_bias(op, w[W_O_B], m, dm);
    for (int64_t i = 0; i < m * dm; i++) r1[i] = ftz(add(ftz(x[i]), ftz(op[i]))); /* S22 */
    float *n2 = falloc(m * dm), *up = falloc(m * inter), *gate = NULL, *act = falloc(m * inter), *down = falloc(m * dm);
    norm_rows(n2, r1, w[W_NORM2], cfg->norm_bias ? w[W_NORM2_B] : NULL, m, dm, cfg->norm_eps, cfg->norm_kind, threads);
    const int gated = cfg->mlp_kind == MLP_SWIGLU || cfg->mlp_kind == MLP_GEGLU_ERF || cfg->mlp_kind == MLP_GEGLU_TANH;
    if (gated) {
        gate = falloc(m * inter);
        rows_gemm(gate, n2, w[W_GATE], 1, m, inter, dm, threads);
        if (cfg->mlp_bias) add_bias(gate, w[W_GATE_B], m, inter);
    }
    rows_gemm(up, n2, w[W_UP], 1, m, inter, dm, threads);
    _mm_setcsr(env & ~(0x8000u | 0x0040u));
    if (cfg->mlp_bias) add_bias(up, w[W_UP_B], m, inter);
    act_ctx_t actx = {act, gate, up, inter, cfg->mlp_kind, gated};
    par_for(m, m * inter >= 65536 ? threads : 1, act_row, &actx);
    rows_gemm(down, act, w[W_DOWN], 1, m, dm, inter, threads);
    _mm_setcsr(env & ~(0x8000u | 0x0040u));
    if (cfg->mlp_bias) add_bias(down, w[W_DOWN_B], m, dm);
    for (int64_t i = 0; i < m * dm; i++) y[i] = ftz(add(ftz(r1[i]), ftz(down[i]))); /* S23 */
    if (qr != q) free(qr);
    if (kr != k) free(kr);
    free(n1); free(q); free(k); free(v); free(ctx); free(op); free(r1); free(n2); free(up); free(gate); free(act); free(down);
    _mm_setcsr(env);
    return 0;
}

/* embedding/checks/embedding_oracle.mojo:369-382: Y = ftz(W[id]); an id outside the table is refused */
DEC_API int dec_embedding(float *y, const float *table, const int32_t *ids, int64_t n, int64_t vocab, int64_t width) {
    for (int64_t t = 0; t < n; t++) {
        if (ids[t] < 0 || ids[t] >= vocab) return 1;
        for (int64_t j = 0; j < width; j++) y[t * width + j] = ftz(table[(int64_t)ids[t] * width + j]);
    }
    return 0;
}

/* learned positions (extension, no reference model): one plain add, ftz(ftz(a) + ftz(b)) */
DEC_API void dec_add_positions(float *x, const float *pos_table, int64_t b, int64_t l, int64_t pos0, int64_t width) {
    unsigned env = _mm_getcsr();
    _mm_setcsr(env & ~(0x8000u | 0x0040u));
    for (int64_t t = 0; t < b * l; t++)
        for (int64_t j = 0; j < width; j++)
            x[t * width + j] = ftz(add(ftz(x[t * width + j]), ftz(pos_table[(pos0 + t % l) * width + j])));
    _mm_setcsr(env);
}

/* greedy: the largest logit, ties to the lowest id (python/mojolearn/models/causal_lm.py:190) */
DEC_API void dec_argmax(int32_t *out, const float *logits, int64_t rows, int64_t vocab) {
    for (int64_t r = 0; r < rows; r++) {
        const float *p = logits + r * vocab;
        int64_t best = 0;
        for (int64_t j = 1; j < vocab; j++)
            if (p[j] > p[best]) best = j;
        out[r] = (int32_t)best;
    }
}
