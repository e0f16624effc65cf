// The skinny product against a PREPACKED weight: a decoder's batched decode step
// (up to 32 activation rows) where the weight is static and may be laid out once.
//
// Numerical plan: the contract's (see gemm_tile.cuh). Execution plan for B200:
//
//   weight, once per layer:  skinny_pack_w_kernel rewrites W[n][k] (float32, bf16 bits
//       or int8 codes, as stored) into column-tile-major panels P[tile][k][256] of the
//       SAME storage type, so the 256 columns a CTA owns are side by side for every k
//       and any run of k-steps is one contiguous block. Beside the panels: one float32
//       factor per column (int8 kinds) and one admission flag per (tile, 16-step window).
//   activations, once per call: skinny_pack_a_kernel transposes A[m][k] into At[k][BM]
//       (flushed, rows past m zero) with one admission flag per window.
//   gemm_skinny_packed_kernel: a CTA owns BM rows x 256 columns and a group of leaves.
//       One elected thread streams stages of 64 / 32 / 16 k-steps (int8 / bf16 / float32:
//       16 KB of weight panel plus the matching slice of At) into a shared-memory ring
//       with two cp.async.bulk copies per stage, completion on an mbarrier. A thread owns
//       all BM rows of two columns, accumulators packed along m (the activation pairs come
//       out of shared memory ready for fma.rn.f32x2), and materialises its own two weights
//       per k-step exactly (int8: prmt + one exact fma on the biased code). Nothing is
//       staged through registers and no CTA-wide barrier sits in the k loop.
//
// Every wait on an mbarrier is bounded; one that runs out sets the status word read by
// b200i_decode_status (6 = refill, 7 = consumer) and the kernel runs on to its end.
#pragma once
#include "decode.cuh"
#include "gemm_skinny.cuh"

namespace b200i {

constexpr int SKP_THREADS = 128, SKP_BN = 256, SKP_STAGES = 3, SKP_B_STAGE_BYTES = 16384, SKP_PER_SM = 3;
__host__ __device__ constexpr int skp_esize(int wk) { return wk == W_F32 ? 4 : (wk == W_BF16 ? 2 : 1); }
__host__ __device__ constexpr int skp_stage_k(int wk) { return SKP_B_STAGE_BYTES / (SKP_BN * skp_esize(wk)); }
__host__ __device__ constexpr int skp_smem_bytes(int wk, int bm) {
    return SKP_STAGES * (SKP_B_STAGE_BYTES + skp_stage_k(wk) * bm * 4) + 2 * SKP_STAGES * 8 + 16;
}

// ---- packed weight layout: [panels][factors][flags] ---------------------------------------
struct SkpWeightLayout {
    size_t tiles, panel_bytes, factor_off, flag_off, total;
};
inline SkpWeightLayout skp_weight_layout(long long n, long long k, int wk) {
    SkpWeightLayout l;
    l.tiles = (size_t)((n + SKP_BN - 1) / SKP_BN);
    l.panel_bytes = l.tiles * SKP_BN * (size_t)k * skp_esize(wk);
    l.factor_off = (l.panel_bytes + 255) / 256 * 256;
    l.flag_off = l.factor_off + l.tiles * SKP_BN * 4;
    l.total = (l.flag_off + l.tiles * (size_t)((k + KS - 1) / KS) + 255) / 256 * 256;
    return l;
}
inline bool skinny_packed_fits(long long m, long long n, long long k) { return skinny_plan_fits(m, n, k, OP_NT); }

// grid (windows, tiles), 256 threads: thread c owns column c of the tile
template <int WK>
__global__ void __launch_bounds__(SKP_BN) skinny_pack_w_kernel(unsigned char *__restrict__ packed, const void *__restrict__ w,
                                                               const void *__restrict__ scale, int n, int k, size_t factor_off,
                                                               size_t flag_off) {
    constexpr int ES = skp_esize(WK);
    const int win = blockIdx.x, tile = blockIdx.y, c = threadIdx.x;
    const int row = tile * SKP_BN + c, k0 = win * KS;
    const bool live = row < n;
    unsigned key = 0xFFFFFFFFu;
    unsigned char *panel = packed + ((size_t)tile * k + k0) * SKP_BN * ES;
    float factor = 0.f;
    if (WK == W_INT8_EXP || WK == W_INT8_SCALE) {
        if (live) factor = (WK == W_INT8_EXP) ? pow2_f32(__ldg(static_cast<const int *>(scale) + row)) : __ldg(static_cast<const float *>(scale) + row);
        if (win == 0) reinterpret_cast<float *>(packed + factor_off)[(size_t)tile * SKP_BN + c] = factor;
    }
#pragma unroll
    for (int kk = 0; kk < KS; kk++) { // k is a multiple of 16: every window is whole
        const size_t off = (size_t)row * k + k0 + kk;
        if (WK == W_F32) {
            const float v = live ? __ldg(static_cast<const float *>(w) + off) : 0.f;
            key = min(key, admit_key(ftz_bits(v)));
            reinterpret_cast<float *>(panel)[(size_t)kk * SKP_BN + c] = v;
        } else if (WK == W_BF16) {
            const unsigned short v = live ? __ldg(static_cast<const unsigned short *>(w) + off) : (unsigned short)0;
            key = min(key, admit_key(ftz_bits(bf16_bits_to_f32(v))));
            reinterpret_cast<unsigned short *>(panel)[(size_t)kk * SKP_BN + c] = v;
        } else {
            const signed char v = live ? __ldg(static_cast<const signed char *>(w) + off) : (signed char)0;
            key = min(key, admit_key(dequant_int8_pow2((int)v, factor)));
            reinterpret_cast<signed char *>(panel)[(size_t)kk * SKP_BN + c] = v;
        }
    }
    const int ok = __syncthreads_and(key >= ADMIT_MIN);
    if (c == 0) packed[flag_off + (size_t)tile * (k / KS) + win] = (unsigned char)(ok ? 1 : 0);
}

// grid (windows), 128 threads: At[k][BM] and one flag per window
template <int BM>
__global__ void __launch_bounds__(128) skinny_pack_a_kernel(float *__restrict__ at, unsigned char *__restrict__ flags,
                                                            const float *__restrict__ a, int m, int k) {
    const int k0 = blockIdx.x * KS, tid = threadIdx.x;
    const int r = tid % BM, q = tid / BM; // row, quad of k inside the window
    unsigned key = 0xFFFFFFFFu;
    if (q < 4) {
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        if (r < m) v = __ldg(reinterpret_cast<const float4 *>(a + (size_t)r * k + k0 + 4 * q));
        v.x = ftz_bits(v.x); v.y = ftz_bits(v.y); v.z = ftz_bits(v.z); v.w = ftz_bits(v.w);
        key = key4(v, key);
        float *dst = at + (size_t)(k0 + 4 * q) * BM + r;
        dst[0] = v.x; dst[BM] = v.y; dst[2 * BM] = v.z; dst[3 * BM] = v.w;
    }
    const int ok = __syncthreads_and(key >= ADMIT_MIN);
    if (tid == 0) flags[blockIdx.x] = (unsigned char)(ok ? 1 : 0);
}

struct SkinnyPackedArgs {
    const float *at;              // [k][BM]
    const unsigned char *aflags;  // [k / 16]
    const unsigned char *packed;  // the packed weight
    size_t factor_off, flag_off;
    float *c, *ws;
    int m, n, k, leaf, leaves, group_leaves, groups;
};

// the two weights of this thread at k-step kk of a stage, as the float32 words the fp32 plan sees
template <int WK>
__device__ __forceinline__ void skp_weights(const unsigned char *bs, int kk, int tid, bool quick, float f0, float f1, float nb0,
                                            float nb1, float &b0, float &b1) {
    if (WK == W_F32) {
        const float2 v = *reinterpret_cast<const float2 *>(bs + ((size_t)kk * SKP_BN + 2 * tid) * 4);
        b0 = v.x; b1 = v.y;
    } else if (WK == W_BF16) {
        const unsigned v = *reinterpret_cast<const unsigned *>(bs + ((size_t)kk * SKP_BN + 2 * tid) * 2);
        b0 = __uint_as_float(v << 16);
        b1 = __uint_as_float(v & 0xFFFF0000u);
    } else {
        const unsigned v = *reinterpret_cast<const unsigned short *>(bs + (size_t)kk * SKP_BN + 2 * tid);
        if (quick) {
            const unsigned x = v ^ 0x8080u;
            const float c0 = __uint_as_float(__byte_perm(x, 0x4B000000u, 0x7540)), c1 = __uint_as_float(__byte_perm(x, 0x4B000000u, 0x7541));
            if (WK == W_INT8_EXP) {
                b0 = __fmaf_rn(c0, f0, nb0);
                b1 = __fmaf_rn(c1, f1, nb1);
            } else {
                b0 = __fmul_rn(__fsub_rn(c0, 8388736.0f), f0);
                b1 = __fmul_rn(__fsub_rn(c1, 8388736.0f), f1);
            }
        } else {
            b0 = dequant_int8_pow2((int)(signed char)(v & 0xFFu), f0);
            b1 = dequant_int8_pow2((int)(signed char)((v >> 8) & 0xFFu), f1);
        }
    }
}

template <int WK, int BM, int MINB>
__global__ void __launch_bounds__(SKP_THREADS, MINB) gemm_skinny_packed_kernel(const SkinnyPackedArgs g) {
    constexpr int ES = skp_esize(WK), KSTG = skp_stage_k(WK), A_STAGE = KSTG * BM * 4, STAGE = SKP_B_STAGE_BYTES + A_STAGE;
    constexpr int CELLS = BM * 2;
    extern __shared__ __align__(128) unsigned char skp_smem[];
    unsigned long long *full = reinterpret_cast<unsigned long long *>(skp_smem + SKP_STAGES * STAGE);
    unsigned long long *empty = full + SKP_STAGES;

    const int tid = threadIdx.x, lane = tid & 31;
    const int tile = blockIdx.x;
    const int t_first = blockIdx.y * g.group_leaves;
    const int t_end = min(t_first + g.group_leaves, g.leaves);
    if (tid == 0) {
#pragma unroll
        for (int i = 0; i < SKP_STAGES; i++) {
            mbar_init(&full[i], 1);
            mbar_init(&empty[i], SKP_THREADS / 32);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();

    // ---- the copy stream (thread 0): stages of up to KSTG k-steps, never across a leaf ----
    const unsigned char *bpanel = g.packed + (size_t)tile * g.k * SKP_BN * ES;
    int pt = t_first, pkoff = 0, pissued = 0;
    auto issue_next = [&]() {
        if (pt >= t_end) return;
        const int kb = pt * g.leaf, leaf_len = min(g.leaf, g.k - kb);
        const int len = min(KSTG, leaf_len - pkoff), slot = pissued % SKP_STAGES;
        unsigned char *dst = skp_smem + (size_t)slot * STAGE;
        const unsigned abytes = (unsigned)len * BM * 4u, bbytes = (unsigned)len * SKP_BN * ES;
        mbar_expect_tx(&full[slot], abytes + bbytes);
        bulk_copy_g2s(dst, g.at + (size_t)(kb + pkoff) * BM, abytes, &full[slot]);
        bulk_copy_g2s(dst + A_STAGE, bpanel + (size_t)(kb + pkoff) * SKP_BN * ES, bbytes, &full[slot]);
        pissued++;
        pkoff += KSTG;
        if (pkoff >= leaf_len) { pkoff = 0; pt++; }
    };
    if (tid == 0) {
        for (int i = 0; i < SKP_STAGES - 1; i++) issue_next();
    }

    // ---- this thread's two columns ----
    float f0 = 0.f, f1 = 0.f, nb0 = 0.f, nb1 = 0.f;
    bool quick = true, wfast = true;
    if (WK == W_INT8_EXP || WK == W_INT8_SCALE) {
        const float2 f = *reinterpret_cast<const float2 *>(g.packed + g.factor_off + ((size_t)tile * SKP_BN + 2 * tid) * 4);
        f0 = f.x; f1 = f.y;
        nb0 = -8388736.0f * f0;
        nb1 = -8388736.0f * f1;
        const unsigned e0 = (__float_as_uint(f0) >> 23) & 0xFFu, e1 = (__float_as_uint(f1) >> 23) & 0xFFu;
        const bool dead0 = f0 == 0.f, dead1 = f1 == 0.f; // a padded column: codes are zero, any spelling gives zero
        quick = (dead0 || (e0 >= 27u && e0 <= 227u)) && (dead1 || (e1 >= 27u && e1 <= 227u));
        wfast = quick && (dead0 || e0 >= ADMIT_EXP) && (dead1 || e1 >= ADMIT_EXP); // |code * factor| >= |factor| for a nonzero code
    }
    const unsigned char *bflags = g.packed + g.flag_off + (size_t)tile * (g.k / KS);

    unsigned long long acc[BM / 2][2];
#pragma unroll
    for (int i = 0; i < BM / 2; i++) { acc[i][0] = 0ull; acc[i][1] = 0ull; }
    float stack[FOLD_LEVELS][CELLS];

    // the weights of a k-step as duplicated pairs; fetched one k-step ahead so that the read, the byte
    // permutes and the exact fma of the dequantisation are off the critical path of the packed fmas
    auto weights = [&](const unsigned char *bs, int kk, bool flush, unsigned long long &p0, unsigned long long &p1) {
        float b0, b1;
        skp_weights<WK>(bs, kk, tid, quick, f0, f1, nb0, nb1, b0, b1);
        if (flush) { b0 = ftz_bits(b0); b1 = ftz_bits(b1); }
        p0 = pack2(b0, b0);
        p1 = pack2(b1, b1);
    };
    auto fmas = [&](const float *as, int kk, bool flush, unsigned long long p0, unsigned long long p1) {
#pragma unroll
        for (int q = 0; q < BM / 4; q++) {
            const ulonglong2 a4 = *reinterpret_cast<const ulonglong2 *>(as + (size_t)kk * BM + 4 * q); // already flushed
            acc[2 * q][0] = fma2_bare(a4.x, p0, acc[2 * q][0]);
            acc[2 * q][1] = fma2_bare(a4.x, p1, acc[2 * q][1]);
            acc[2 * q + 1][0] = fma2_bare(a4.y, p0, acc[2 * q + 1][0]);
            acc[2 * q + 1][1] = fma2_bare(a4.y, p1, acc[2 * q + 1][1]);
            if (flush) {
                acc[2 * q][0] = ftz2_hw(acc[2 * q][0]);
                acc[2 * q][1] = ftz2_hw(acc[2 * q][1]);
                acc[2 * q + 1][0] = ftz2_hw(acc[2 * q + 1][0]);
                acc[2 * q + 1][1] = ftz2_hw(acc[2 * q + 1][1]);
            }
        }
    };
    auto unpack_cells = [&](float (&v)[CELLS], bool clear_acc) {
#pragma unroll
        for (int i = 0; i < BM / 2; i++)
#pragma unroll
            for (int c = 0; c < 2; c++) {
                float v0, v1;
                unpack2(acc[i][c], v0, v1);
                v[(2 * i) * 2 + c] = ftz_hw(v0);
                v[(2 * i + 1) * 2 + c] = ftz_hw(v1);
                if (clear_acc) acc[i][c] = 0ull;
            }
    };
    auto push_leaf = [&](int local_leaf) {
        float v[CELLS];
        unpack_cells(v, true);
        int lvl = 0;
        for (int bits = local_leaf; bits & 1; bits >>= 1, lvl++) {
#pragma unroll
            for (int c = 0; c < CELLS; c++) v[c] = fold_add(stack[lvl][c], v[c]);
        }
#pragma unroll
        for (int c = 0; c < CELLS; c++) stack[lvl][c] = v[c];
    };

    int slot = 0, stage_no = 0;
    unsigned phase = 0;
    bool alive = true;
    for (int t = t_first; t < t_end; t++) {
        const int kb = t * g.leaf, leaf_len = min(g.leaf, g.k - kb);
        bool leaf_clean = true;
        for (int soff = 0; soff < leaf_len; soff += KSTG) {
            const int slen = min(KSTG, leaf_len - soff);
            if (alive && !mbar_wait(&full[slot], phase)) {
                if (lane == 0) atomicExch(&g_decode_status, 7);
                alive = false;
            }
            const unsigned char *base = skp_smem + (size_t)slot * STAGE;
            const float *as = reinterpret_cast<const float *>(base);
            const unsigned char *bs = base + A_STAGE;
            for (int woff = 0; woff < slen; woff += KS) {
                const int len = min(KS, slen - woff), win = (kb + soff + woff) / KS;
                const bool admitted = wfast && (__ldg(g.aflags + win) & __ldg(bflags + win)) != 0;
                if (admitted && leaf_clean && len == KS) {
                    unsigned long long p0, p1, n0 = 0ull, n1 = 0ull;
                    weights(bs, woff, false, p0, p1);
#pragma unroll
                    for (int kk = 0; kk < KS; kk++) {
                        if (kk + 1 < KS) weights(bs, woff + kk + 1, false, n0, n1);
                        fmas(as, woff + kk, false, p0, p1);
                        p0 = n0;
                        p1 = n1;
                    }
                } else {
                    leaf_clean = false;
#pragma unroll 1
                    for (int kk = 0; kk < len; kk++) {
                        unsigned long long p0, p1;
                        weights(bs, woff + kk, true, p0, p1);
                        fmas(as, woff + kk, true, p0, p1);
                    }
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&empty[slot]);
            if (tid == 0) {
                if (stage_no >= 1) {
                    const int prev = stage_no - 1;
                    if (alive && !mbar_wait(&empty[prev % SKP_STAGES], (unsigned)(prev / SKP_STAGES) & 1u)) {
                        atomicExch(&g_decode_status, 6);
                        alive = false;
                    }
                }
                issue_next();
            }
            stage_no++;
            if (++slot == SKP_STAGES) { slot = 0; phase ^= 1u; }
        }
        if (t + 1 < t_end) push_leaf(t - t_first);
    }

    const int count = t_end - t_first;
    float *out = g.groups > 1 ? g.ws + (size_t)blockIdx.y * (size_t)g.m * (size_t)g.n : g.c;
    float v[CELLS];
    unpack_cells(v, false);
    if (count > 1) {
        const int last = count - 1;
        for (int lvl = 0; lvl < FOLD_LEVELS; lvl++)
            if ((last >> lvl) & 1) {
#pragma unroll
                for (int c = 0; c < CELLS; c++) v[c] = fold_add(stack[lvl][c], v[c]);
            }
    }
    const int col = tile * SKP_BN + 2 * tid;
#pragma unroll
    for (int i = 0; i < BM; i++) {
        if (i >= g.m) break;
        if (col < g.n) out[(size_t)i * g.n + col] = nan_canon(ftz_hw(v[i * 2]));
        if (col + 1 < g.n) out[(size_t)i * g.n + col + 1] = nan_canon(ftz_hw(v[i * 2 + 1]));
    }
}

} // namespace b200i
