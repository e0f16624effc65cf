/*
 * The reference's CPU product at CPU speed, restated in C with AVX2 + FMA.
 *
 * THIS FILE IS TEST INFRASTRUCTURE: the timed CPU baseline of the benchmark
 * and a faster checker for shapes the scalar oracle (oracle.c) would take
 * minutes over. It must return the scalar oracle's bits for every input;
 * tests/test_oracle_rows.py holds it to that.
 *
 * It follows the strategy of gemm/host/gemm_host_rows.mojo (paths relative to
 * the reference project's root):
 *   - operands flushed once into packed copies: the left operand row-major
 *     [m x k], the right operand in panels of 32 columns, each [k x 32]
 *     contiguous, columns past n filled with +0.0 and never stored
 *     (:233-290);
 *   - the 32 cells of one output row and one panel advance together down p,
 *     four 8-lane accumulators, one lane per cell, each lane its own serial
 *     chain (:163-198);
 *   - the per-step flush is deferred: a tracker keeps the lane-wise minimum of
 *     ((bits - 1) & 0x7FFFFFFF) over every raw result, which is below
 *     0x007FFFFF exactly when one was subnormal, and only then is the group
 *     recomputed with a flush at every step (:29-38, :185-194);
 *   - the balanced fold runs in place over the leaf partials (:201-225);
 *   - m <= 4 rows skip the packing and flush at every step (:369-445);
 *   - the work is split over threads by rows or by panels, one task per 2^20
 *     multiply-adds at most (:448-464, :467-556).
 * None of this can move a bit: a cell's arithmetic is the scalar chain's.
 */
#define _GNU_SOURCE
#include <immintrin.h>
#include <math.h>
#include <pthread.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define ROWS_API __attribute__((visibility("default")))

enum { OP_NN = 0, OP_NT = 1, OP_TN = 2 };
enum { LANES = 8, CHAINS = 4, PANEL = LANES * CHAINS, SMALL_M = 4 };
#define SERIAL_FMAS ((int64_t)1 << 20)

int64_t oracle_leaf_size(int64_t k);
int64_t oracle_leaf_count_at(int64_t k, int64_t leaf);

static inline uint32_t f2u(float x) { uint32_t u; memcpy(&u, &x, 4); return u; }
static inline float u2f(uint32_t u) { float x; memcpy(&x, &u, 4); return x; }
static inline float ftz1(float x) {
    uint32_t b = f2u(x);
    if ((b & 0x7F800000u) == 0u) return u2f(b & 0x80000000u);
    return x;
}
static inline __m256 ftz8(__m256 x) {
    __m256i bits = _mm256_castps_si256(x);
    __m256i tiny = _mm256_cmpeq_epi32(_mm256_and_si256(bits, _mm256_set1_epi32(0x7F800000)), _mm256_setzero_si256());
    __m256i sign = _mm256_and_si256(bits, _mm256_set1_epi32((int)0x80000000u));
    return _mm256_castsi256_ps(_mm256_blendv_epi8(bits, sign, tiny));
}

/* ---- packing ----------------------------------------------------------------- */

static void pack_left(const float *a, int op, int64_t m, int64_t k, float *ap, int64_t lo, int64_t hi) {
    if (op == OP_TN) {
        for (int64_t p = 0; p < k; p++)
            for (int64_t i = lo; i < hi; i++) ap[i * k + p] = ftz1(a[p * m + i]);
        return;
    }
    for (int64_t t = lo * k; t < hi * k; t++) ap[t] = ftz1(a[t]);
}

static void pack_right(const float *b, int op, int64_t n, int64_t k, float *bp, int64_t glo, int64_t ghi) {
    for (int64_t g = glo; g < ghi; g++) {
        int64_t j0 = g * PANEL;
        int64_t width = n - j0 < PANEL ? n - j0 : PANEL;
        float *panel = bp + g * k * PANEL;
        for (int64_t p = 0; p < k; p++)
            for (int64_t jj = 0; jj < PANEL; jj++) {
                float v = 0.0f;
                if (jj < width) v = ftz1(op == OP_NT ? b[(j0 + jj) * k + p] : b[p * n + j0 + jj]);
                panel[p * PANEL + jj] = v;
            }
    }
}

/* ---- one leaf of one row against one panel ----------------------------------- */

static void leaf_flushed(const float *arow, const float *panel, int64_t pb, int64_t pe, float *dst) {
    for (int q = 0; q < CHAINS; q++) {
        __m256 acc = _mm256_setzero_ps();
        for (int64_t p = pb; p < pe; p++)
            acc = ftz8(_mm256_fmadd_ps(_mm256_set1_ps(arow[p]), _mm256_loadu_ps(panel + p * PANEL + q * LANES), acc));
        _mm256_storeu_ps(dst + q * LANES, acc);
    }
}

static void leaf_deferred(const float *arow, const float *panel, int64_t pb, int64_t pe, float *dst) {
    const __m256i one = _mm256_set1_epi32(1), absm = _mm256_set1_epi32(0x7FFFFFFF);
    __m256 c0 = _mm256_setzero_ps(), c1 = c0, c2 = c0, c3 = c0;
    __m256i e0 = _mm256_set1_epi32(-1), e1 = e0, e2 = e0, e3 = e0;
    for (int64_t p = pb; p < pe; p++) {
        __m256 s = _mm256_set1_ps(arow[p]);
        const float *row = panel + p * PANEL;
        c0 = _mm256_fmadd_ps(s, _mm256_loadu_ps(row), c0);
        c1 = _mm256_fmadd_ps(s, _mm256_loadu_ps(row + LANES), c1);
        c2 = _mm256_fmadd_ps(s, _mm256_loadu_ps(row + 2 * LANES), c2);
        c3 = _mm256_fmadd_ps(s, _mm256_loadu_ps(row + 3 * LANES), c3);
        e0 = _mm256_min_epu32(e0, _mm256_and_si256(_mm256_sub_epi32(_mm256_castps_si256(c0), one), absm));
        e1 = _mm256_min_epu32(e1, _mm256_and_si256(_mm256_sub_epi32(_mm256_castps_si256(c1), one), absm));
        e2 = _mm256_min_epu32(e2, _mm256_and_si256(_mm256_sub_epi32(_mm256_castps_si256(c2), one), absm));
        e3 = _mm256_min_epu32(e3, _mm256_and_si256(_mm256_sub_epi32(_mm256_castps_si256(c3), one), absm));
    }
    __m256i em = _mm256_min_epu32(_mm256_min_epu32(e0, e1), _mm256_min_epu32(e2, e3));
    uint32_t lanes[LANES];
    _mm256_storeu_si256((__m256i *)lanes, em);
    uint32_t lowest = 0xFFFFFFFFu;
    for (int t = 0; t < LANES; t++)
        if (lanes[t] < lowest) lowest = lanes[t];
    if (lowest < 0x007FFFFFu) { /* a raw result was subnormal: the flush was not the identity */
        leaf_flushed(arow, panel, pb, pe, dst);
        return;
    }
    _mm256_storeu_ps(dst, c0);
    _mm256_storeu_ps(dst + LANES, c1);
    _mm256_storeu_ps(dst + 2 * LANES, c2);
    _mm256_storeu_ps(dst + 3 * LANES, c3);
}

/* rows of `width` floats, `pcount` of them; the root lands in row 0 */
static void fold_rows(float *sp, int64_t pcount, int64_t width) {
    int64_t w = pcount;
    while (w > 1) {
        int64_t pairs = w / 2;
        for (int64_t q = 0; q < pairs; q++) {
            float *dst = sp + q * width;
            const float *l = sp + 2 * q * width, *r = l + width;
            for (int64_t j = 0; j < width; j += LANES)
                _mm256_storeu_ps(dst + j, ftz8(_mm256_add_ps(_mm256_loadu_ps(l + j), _mm256_loadu_ps(r + j))));
        }
        if (w & 1) memmove(sp + pairs * width, sp + (w - 1) * width, sizeof(float) * (size_t)width);
        w = pairs + (w & 1);
    }
}

static void tile(const float *ap, const float *bp, float *c, int64_t n, int64_t k, int64_t lo, int64_t hi,
                 int64_t glo, int64_t ghi) {
    if (hi <= lo || ghi <= glo) return;
    int64_t leaf = oracle_leaf_size(k), pcount = oracle_leaf_count_at(k, leaf);
    float *scratch = (float *)malloc(sizeof(float) * (size_t)(pcount > 0 ? pcount : 1) * PANEL);
    for (int64_t g = glo; g < ghi; g++) {
        const float *panel = bp + g * k * PANEL;
        int64_t j0 = g * PANEL;
        int64_t width = n - j0 < PANEL ? n - j0 : PANEL;
        for (int64_t i = lo; i < hi; i++) {
            if (pcount == 0) {
                for (int64_t jj = 0; jj < width; jj++) c[i * n + j0 + jj] = 0.0f;
                continue;
            }
            for (int64_t t = 0; t < pcount; t++) {
                int64_t pb = t * leaf, pe = pb + leaf < k ? pb + leaf : k;
                leaf_deferred(ap + i * k, panel, pb, pe, scratch + t * PANEL);
            }
            fold_rows(scratch, pcount, PANEL);
            memcpy(c + i * n + j0, scratch, sizeof(float) * (size_t)width);
        }
    }
    free(scratch);
}

/* ---- m <= 4: no packed copies, a flush at every step --------------------------- */

static void small_m(const float *a, const float *b, float *c, int op, int64_t m, int64_t n, int64_t k, int64_t jlo,
                    int64_t jhi) {
    if (jhi <= jlo) return;
    int64_t leaf = oracle_leaf_size(k), pcount = oracle_leaf_count_at(k, leaf);
    int64_t width = m * LANES;
    float *scratch = (float *)malloc(sizeof(float) * (size_t)(pcount > 0 ? pcount : 1) * (size_t)width);
    for (int64_t j0 = jlo; j0 < jhi; j0 += LANES) {
        int64_t cnt = jhi - j0 < LANES ? jhi - j0 : LANES;
        for (int64_t t = 0; t < pcount; t++) {
            int64_t pb = t * leaf, pe = pb + leaf < k ? pb + leaf : k;
            float *dst = scratch + t * width;
            __m256 acc[SMALL_M];
            for (int i = 0; i < SMALL_M; i++) acc[i] = _mm256_setzero_ps();
            for (int64_t p = pb; p < pe; p++) {
                float lanes[LANES];
                for (int64_t jj = 0; jj < LANES; jj++) {
                    int64_t j = j0 + jj;
                    lanes[jj] = j < jhi ? (op == OP_NT ? b[j * k + p] : b[p * n + j]) : 0.0f;
                }
                __m256 bv = ftz8(_mm256_loadu_ps(lanes));
                for (int64_t i = 0; i < m; i++) {
                    float av = ftz1(op == OP_TN ? a[p * m + i] : a[i * k + p]);
                    acc[i] = ftz8(_mm256_fmadd_ps(_mm256_set1_ps(av), bv, acc[i]));
                }
            }
            for (int64_t i = 0; i < m; i++) _mm256_storeu_ps(dst + i * LANES, acc[i]);
        }
        if (pcount == 0)
            for (int64_t t = 0; t < width; t++) scratch[t] = 0.0f;
        fold_rows(scratch, pcount, width);
        for (int64_t i = 0; i < m; i++) memcpy(c + i * n + j0, scratch + i * LANES, sizeof(float) * (size_t)cnt);
    }
    free(scratch);
}

/* ---- thread split --------------------------------------------------------------- */

typedef struct {
    const float *a, *b;
    float *c, *ap, *bp;
    int op, by_rows, phase;
    int64_t m, n, k, npan, rchunk, pchunk, bchunk, index;
} task_t;

static inline int64_t min64(int64_t x, int64_t y) { return x < y ? x : y; }

static void *run_task(void *arg) {
    task_t *t = (task_t *)arg;
    unsigned old = _mm_getcsr();
    _mm_setcsr(old & ~(0x8000u | 0x0040u)); /* every worker: FTZ and DAZ clear */
    int64_t i = t->index;
    if (t->phase == 0) {
        pack_left(t->a, t->op, t->m, t->k, t->ap, min64(i * t->rchunk, t->m), min64((i + 1) * t->rchunk, t->m));
        pack_right(t->b, t->op, t->n, t->k, t->bp, min64(i * t->pchunk, t->npan), min64((i + 1) * t->pchunk, t->npan));
    } else if (t->phase == 1) {
        if (t->by_rows)
            tile(t->ap, t->bp, t->c, t->n, t->k, min64(i * t->rchunk, t->m), min64((i + 1) * t->rchunk, t->m), 0, t->npan);
        else
            tile(t->ap, t->bp, t->c, t->n, t->k, 0, t->m, min64(i * t->pchunk, t->npan), min64((i + 1) * t->pchunk, t->npan));
    } else {
        small_m(t->a, t->b, t->c, t->op, t->m, t->n, t->k, min64(i * t->bchunk * LANES, t->n),
                min64((i + 1) * t->bchunk * LANES, t->n));
    }
    _mm_setcsr(old);
    return NULL;
}

static void fan_out(task_t *proto, int64_t tasks, int phase) {
    pthread_t *th = (pthread_t *)malloc(sizeof(pthread_t) * (size_t)tasks);
    task_t *ts = (task_t *)malloc(sizeof(task_t) * (size_t)tasks);
    for (int64_t i = 0; i < tasks; i++) {
        ts[i] = *proto;
        ts[i].phase = phase;
        ts[i].index = i;
        if (i + 1 < tasks) pthread_create(&th[i], NULL, run_task, &ts[i]);
    }
    run_task(&ts[tasks - 1]);
    for (int64_t i = 0; i + 1 < tasks; i++) pthread_join(th[i], NULL);
    free(th);
    free(ts);
}

/* Returns 0; 1 on a refusal; 2 when the host has no AVX2/FMA. `threads` is the
 * worker count the caller allows (the reference's policy is one per physical
 * core); the split never gives a task fewer than 2^20 multiply-adds. */
ROWS_API int rows_gemm(float *c, const float *a, const float *b, int op, int64_t m, int64_t n, int64_t k, int threads) {
    if (op != OP_NN && op != OP_NT && op != OP_TN) return 1;
    if (m < 0 || n < 0 || k < 0) return 1;
    if (!__builtin_cpu_supports("avx2") || !__builtin_cpu_supports("fma")) return 2;
    if (m == 0 || n == 0) return 0;
    if (threads < 1) threads = 1;
    int64_t work = m * n * (k > 1 ? k : 1);
    task_t proto;
    memset(&proto, 0, sizeof proto);
    proto.a = a; proto.b = b; proto.c = c; proto.op = op; proto.m = m; proto.n = n; proto.k = k;
    if (m <= SMALL_M) {
        int64_t cblocks = (n + LANES - 1) / LANES;
        int64_t tasks = 1;
        if (work >= SERIAL_FMAS) tasks = min64(min64(threads, cblocks), work / SERIAL_FMAS);
        if (tasks < 1) tasks = 1;
        proto.bchunk = (cblocks + tasks - 1) / tasks;
        fan_out(&proto, tasks, 2);
        return 0;
    }
    int64_t npan = (n + PANEL - 1) / PANEL;
    proto.npan = npan;
    proto.ap = (float *)malloc(sizeof(float) * (size_t)(m * k > 0 ? m * k : 1));
    proto.bp = (float *)malloc(sizeof(float) * (size_t)(npan * k * PANEL > 0 ? npan * k * PANEL : 1));
    int64_t units = m > npan ? m : npan;
    int64_t tasks = work < SERIAL_FMAS ? 1 : min64(min64(threads, units), work / SERIAL_FMAS);
    if (tasks < 1) tasks = 1;
    proto.rchunk = (m + tasks - 1) / tasks;
    proto.pchunk = (npan + tasks - 1) / tasks;
    proto.by_rows = m >= 2 * tasks;
    fan_out(&proto, tasks, 0);
    fan_out(&proto, tasks, 1);
    free(proto.ap);
    free(proto.bp);
    return 0;
}
