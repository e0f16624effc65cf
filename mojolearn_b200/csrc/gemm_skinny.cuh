// The skinny identical-mode product: C[m,n] = A[m,k] . W[n,k]^T for 5..32
// activation rows (a decoder's batched decode step), any weight storage kind.
//
// Numerical plan: the contract's (see gemm_tile.cuh). Execution plan for B200:
// with so few rows the work per weight is small, so the instruction mix is what
// matters. A thread owns ALL rows of CPT output columns; its accumulators are
// packed along m, so the activation pairs (a[m], a[m+1]) come out of shared memory
// as 64-bit halves of a 128-bit read with no packing instruction at all, and only
// the CPT weight words of a k-step need duplicating. One k-step is BM/4 broadcast
// reads of A, one read of B and BM/2 * CPT packed fused multiply-adds
// (fma.rn.f32x2), e.g. 8 + 1 reads and 32 fmas at BM = 32.
// The weight window is loaded 16 k-steps ahead as raw bytes (one 128-bit load per
// row for int8), materialised exactly at store time (int8: prmt + one exact fma on
// the biased code) and written k-major with 128-bit stores. Admission, the window
// rule, the leaf-group split and the fold stack are the tile kernel's.
#pragma once
#include "gemm_tile.cuh"

namespace b200i {

constexpr int SK_THREADS = 128;

template <int WK>
struct SkinnyRaw { // one weight row's window: 16 elements
    static constexpr int WORDS = WK == W_F32 ? 16 : (WK == W_BF16 ? 8 : 4);
    unsigned w[WORDS];
    unsigned f; // int8 kinds: the row's raw exponent / scale word
};

template <int WK>
__device__ __forceinline__ void skinny_load_row(SkinnyRaw<WK> &r, const void *base, const void *scale, long long row, int n,
                                                int k, int k0) {
    constexpr int ES = WK == W_F32 ? 4 : (WK == W_BF16 ? 2 : 1);
    r.f = 0u;
    if (row < n && k0 < k) { // k is a multiple of 16: a window is wholly inside the row or wholly outside
        const uint4 *p = reinterpret_cast<const uint4 *>(static_cast<const unsigned char *>(base) + ((size_t)row * k + k0) * ES);
#pragma unroll
        for (int q = 0; q < SkinnyRaw<WK>::WORDS / 4; q++) {
            const uint4 v = __ldg(p + q);
            r.w[4 * q] = v.x; r.w[4 * q + 1] = v.y; r.w[4 * q + 2] = v.z; r.w[4 * q + 3] = v.w;
        }
        if (WK == W_INT8_EXP || WK == W_INT8_SCALE) r.f = __ldg(static_cast<const unsigned *>(scale) + row);
    } else {
#pragma unroll
        for (int q = 0; q < SkinnyRaw<WK>::WORDS; q++) r.w[q] = 0u;
    }
}

// The 16 elements of a raw row window as the float32 words the fp32 plan sees;
// returns the window's admission key (the minimum of admit_key over the words).
// For a quickly dequantised int8 row a nonzero word is at least the row factor in
// magnitude, so the factor's exponent alone decides.
template <int WK>
__device__ __forceinline__ unsigned skinny_widen(const SkinnyRaw<WK> &r, float (&v)[16]) {
    unsigned key = 0xFFFFFFFFu;
    if (WK == W_F32) {
#pragma unroll
        for (int e = 0; e < 16; e++) { v[e] = __uint_as_float(r.w[e]); key = min(key, admit_key(v[e])); }
    } else if (WK == W_BF16) {
#pragma unroll
        for (int e = 0; e < 8; e++) {
            v[2 * e] = __uint_as_float(r.w[e] << 16);
            v[2 * e + 1] = __uint_as_float(r.w[e] & 0xFFFF0000u);
            key = min(key, min(admit_key(v[2 * e]), admit_key(v[2 * e + 1])));
        }
    } else {
        const float factor = (WK == W_INT8_EXP) ? pow2_f32((int)r.f) : __uint_as_float(r.f);
        const unsigned fexp = (__float_as_uint(factor) >> 23) & 0xFFu;
        if (fexp >= 27u && fexp <= 227u) { // products stay normal and finite: the exact short spellings
            const float nbias = -8388736.0f * factor;
#pragma unroll
            for (int q = 0; q < 4; q++) {
                const unsigned x = r.w[q] ^ 0x80808080u;
                const float b0 = __uint_as_float(__byte_perm(x, 0x4B000000u, 0x7540)), b1 = __uint_as_float(__byte_perm(x, 0x4B000000u, 0x7541));
                const float b2 = __uint_as_float(__byte_perm(x, 0x4B000000u, 0x7542)), b3 = __uint_as_float(__byte_perm(x, 0x4B000000u, 0x7543));
                if (WK == W_INT8_EXP) {
                    v[4 * q] = __fmaf_rn(b0, factor, nbias); v[4 * q + 1] = __fmaf_rn(b1, factor, nbias);
                    v[4 * q + 2] = __fmaf_rn(b2, factor, nbias); v[4 * q + 3] = __fmaf_rn(b3, factor, nbias);
                } else {
                    v[4 * q] = __fmul_rn(__fsub_rn(b0, 8388736.0f), factor); v[4 * q + 1] = __fmul_rn(__fsub_rn(b1, 8388736.0f), factor);
                    v[4 * q + 2] = __fmul_rn(__fsub_rn(b2, 8388736.0f), factor); v[4 * q + 3] = __fmul_rn(__fsub_rn(b3, 8388736.0f), factor);
                }
            }
            key = fexp >= ADMIT_EXP ? 0xFFFFFFFEu : 0u;
        } else {
#pragma unroll
            for (int q = 0; q < 4; q++)
#pragma unroll
                for (int e = 0; e < 4; e++) {
                    v[4 * q + e] = dequant_int8_pow2((int)(signed char)((r.w[q] >> (8 * e)) & 0xFFu), factor);
                    key = min(key, admit_key(v[4 * q + e]));
                }
        }
    }
    return key;
}

// BM rows per CTA, split over RSPLIT thread groups of SK_THREADS / RSPLIT threads; a
// thread owns TR = BM / RSPLIT rows of CPT columns.
template <int BM, int CPT, int RSPLIT>
struct SkinnyShape {
    static constexpr int CT = SK_THREADS / RSPLIT; // column threads
    static constexpr int TR = BM / RSPLIT;         // rows per thread
    static constexpr int BN = CT * CPT;
    static constexpr int LQ = CPT < 4 ? CPT : 4;   // columns per shared-memory store vector
    static constexpr int ROW_GROUPS = BN / LQ;     // groups of LQ weight rows to stage per window
    static constexpr int GROUPS = (ROW_GROUPS + SK_THREADS - 1) / SK_THREADS; // per thread
    static constexpr int SMEM_BYTES = 2 * KS * (BM + BN) * 4;
};

template <int WK, int BM, int CPT, int RSPLIT, int MINB>
__global__ void __launch_bounds__(SK_THREADS, MINB) gemm_skinny_kernel(const GemmArgs g) {
    using S = SkinnyShape<BM, CPT, RSPLIT>;
    constexpr int BN = S::BN, LQ = S::LQ, NG = S::GROUPS, TR = S::TR, CT = S::CT, CELLS = TR * CPT;
    extern __shared__ __align__(16) float sk_smem[];
    float (*As)[KS][BM] = reinterpret_cast<float (*)[KS][BM]>(sk_smem);
    float (*Bs)[KS][BN] = reinterpret_cast<float (*)[KS][BN]>(sk_smem + 2 * KS * BM);

    const int tid = threadIdx.x;
    const int ctid = tid % CT, row0 = (tid / CT) * TR; // this thread's column slot and first row
    const int bn0 = blockIdx.x * BN;
    const int t_first = blockIdx.y * g.group_leaves;
    const int t_end = min(t_first + g.group_leaves, g.leaves);

    unsigned long long acc[TR / 2][CPT];
#pragma unroll
    for (int i = 0; i < TR / 2; i++)
#pragma unroll
        for (int c = 0; c < CPT; c++) acc[i][c] = 0ull;
    float stack[FOLD_LEVELS][CELLS];

    // staging state: this thread's weight rows (NG groups of LQ rows) and its share of the activation window
    SkinnyRaw<WK> braw[NG][LQ];
    float4 araw;
    const bool a_owner = tid < BM * 4; // BM rows x 4 quads of k
    const int a_row = tid / 4, a_kq = tid % 4;
    unsigned stage_key;

    auto load_window = [&](int t, int koff) {
        const int k0 = t * g.leaf + koff;
#pragma unroll
        for (int gi = 0; gi < NG; gi++)
#pragma unroll
            for (int r = 0; r < LQ; r++)
                if (tid + SK_THREADS * gi < S::ROW_GROUPS)
                    skinny_load_row<WK>(braw[gi][r], g.b, g.bscale, (long long)bn0 + (long long)(tid + SK_THREADS * gi) * LQ + r, g.n, g.k, k0);
        araw = make_float4(0.f, 0.f, 0.f, 0.f);
        if (a_owner && a_row < g.m && k0 + 4 * a_kq < g.k)
            araw = __ldg(reinterpret_cast<const float4 *>(g.a + (size_t)a_row * g.k + k0 + 4 * a_kq));
    };
    auto store_window = [&](int buf) {
        stage_key = 0xFFFFFFFFu;
#pragma unroll
        for (int gi = 0; gi < NG; gi++) {
            if (tid + SK_THREADS * gi >= S::ROW_GROUPS) break;
            float v[LQ][16];
#pragma unroll
            for (int r = 0; r < LQ; r++) {
                stage_key = min(stage_key, skinny_widen<WK>(braw[gi][r], v[r]));
            }
            const int col = (tid + SK_THREADS * gi) * LQ;
#pragma unroll
            for (int e = 0; e < 16; e++) {
                if (LQ == 4) *reinterpret_cast<float4 *>(&Bs[buf][e][col]) = make_float4(v[0][e], v[1][e], v[2][e], v[3][e]);
                else if (LQ == 2) *reinterpret_cast<float2 *>(&Bs[buf][e][col]) = make_float2(v[0][e], v[LQ - 1][e]);
                else Bs[buf][e][col] = v[0][e];
            }
        }
        if (a_owner) {
            stage_key = key4(araw, stage_key);
            As[buf][4 * a_kq + 0][a_row] = araw.x;
            As[buf][4 * a_kq + 1][a_row] = araw.y;
            As[buf][4 * a_kq + 2][a_row] = araw.z;
            As[buf][4 * a_kq + 3][a_row] = araw.w;
        }
    };

    // this thread's columns inside the tile: CPT consecutive columns (two halves when CPT is 8)
    auto col_of = [&](int c) { return CPT == 8 ? (c / 4) * (BN / 2) + ctid * 4 + (c % 4) : ctid * CPT + c; };

    auto step = [&](int buf, int kk, bool flush) {
        float bv[CPT];
        if (CPT == 8) {
            const float4 lo = *reinterpret_cast<const float4 *>(&Bs[buf][kk][ctid * 4]);
            const float4 hi = *reinterpret_cast<const float4 *>(&Bs[buf][kk][BN / 2 + ctid * 4]);
            bv[0] = lo.x; bv[1] = lo.y; bv[2] = lo.z; bv[3] = lo.w;
            bv[CPT - 4] = hi.x; bv[CPT - 3] = hi.y; bv[CPT - 2] = hi.z; bv[CPT - 1] = hi.w;
        } else if (CPT == 4) {
            const float4 v = *reinterpret_cast<const float4 *>(&Bs[buf][kk][ctid * 4]);
            bv[0] = v.x; bv[1] = v.y; bv[CPT - 2] = v.z; bv[CPT - 1] = v.w;
        } else if (CPT == 2) {
            const float2 v = *reinterpret_cast<const float2 *>(&Bs[buf][kk][ctid * 2]);
            bv[0] = v.x; bv[CPT - 1] = v.y;
        } else {
            bv[0] = Bs[buf][kk][ctid];
        }
        unsigned long long b2[CPT];
#pragma unroll
        for (int c = 0; c < CPT; c++) {
            const float b = flush ? ftz_bits(bv[c]) : bv[c];
            b2[c] = pack2(b, b);
        }
#pragma unroll
        for (int q = 0; q < TR / 4; q++) {
            // four activation rows of this k-step: two packed pairs straight out of one 128-bit read
            ulonglong2 a4 = *reinterpret_cast<const ulonglong2 *>(&As[buf][kk][row0 + 4 * q]);
            if (flush) {
                float x0, x1, x2, x3;
                unpack2(a4.x, x0, x1);
                unpack2(a4.y, x2, x3);
                a4.x = pack2(ftz_bits(x0), ftz_bits(x1));
                a4.y = pack2(ftz_bits(x2), ftz_bits(x3));
            }
#pragma unroll
            for (int c = 0; c < CPT; c++) {
                acc[2 * q][c] = fma2_bare(a4.x, b2[c], acc[2 * q][c]);
                acc[2 * q + 1][c] = fma2_bare(a4.y, b2[c], acc[2 * q + 1][c]);
                if (flush) {
                    acc[2 * q][c] = ftz2_hw(acc[2 * q][c]);
                    acc[2 * q + 1][c] = ftz2_hw(acc[2 * q + 1][c]);
                }
            }
        }
    };

    // cell index of (row pair i, half h, column c): level-major fold walks all cells
    auto unpack_cells = [&](float (&v)[CELLS], bool clear_acc) {
#pragma unroll
        for (int i = 0; i < TR / 2; i++)
#pragma unroll
            for (int c = 0; c < CPT; c++) {
                float v0, v1;
                unpack2(acc[i][c], v0, v1);
                v[(2 * i) * CPT + c] = ftz_hw(v0);
                v[(2 * i + 1) * CPT + c] = ftz_hw(v1);
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

    if (t_first < t_end) {
        int t = t_first, koff = 0;
        load_window(t, koff);
        store_window(0);
        bool admitted = __syncthreads_and(stage_key >= ADMIT_MIN);
        bool leaf_clean = true;
        int buf = 0;
        while (true) {
            const int leaf_len = min(g.leaf, g.k - t * g.leaf);
            const int len = min(KS, leaf_len - koff);
            int nt = t, nkoff = koff + KS;
            if (nkoff >= leaf_len) { nt = t + 1; nkoff = 0; }
            const bool more = nt < t_end;
            if (more) load_window(nt, nkoff);
            if (admitted && leaf_clean && len == KS) {
#pragma unroll
                for (int kk = 0; kk < KS; kk++) step(buf, kk, false);
            } else {
                leaf_clean = false;
#pragma unroll 1
                for (int kk = 0; kk < len; kk++) step(buf, kk, true);
            }
            if (nt != t) {
                if (more) push_leaf(t - t_first);
                leaf_clean = true;
            }
            if (!more) break;
            store_window(buf ^ 1);
            admitted = __syncthreads_and(stage_key >= ADMIT_MIN);
            buf ^= 1;
            t = nt;
            koff = nkoff;
        }
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
    if (CPT == 2 && g.groups == 1 && epilogue_pairs(g.epi)) { // this thread's two columns are one (gate, up) pair
        const int col = bn0 + col_of(0);
        if (col + 1 < g.n)
            for (int i = 0; i < TR && row0 + i < g.m; i++)
                g.c[(size_t)(row0 + i) * (g.n / 2) + col / 2] =
                    epilogue_pair_apply(nan_canon(ftz_hw(v[i * CPT])), nan_canon(ftz_hw(v[i * CPT + 1])), g.epi.bias, g.epi.act, col / 2);
        return;
    }
#pragma unroll
    for (int i = 0; i < TR; i++) {
        if (row0 + i >= g.m) break;
#pragma unroll
        for (int c = 0; c < CPT; c++) {
            const int col = bn0 + col_of(c);
            if (col < g.n) out[(size_t)(row0 + i) * g.n + col] = nan_canon(ftz_hw(v[i * CPT + c]));
        }
    }
    if (g.groups == 1 && epilogue_on(g.epi)) { // this thread's own cells once more (see epilogue_cell)
        for (int i = 0; i < TR && row0 + i < g.m; i++)
            for (int c = 0; c < CPT; c++) {
                const int col = bn0 + col_of(c);
                if (col < g.n) epilogue_cell(out + (size_t)(row0 + i) * g.n + col, g.epi, col);
            }
    }
}

inline bool skinny_plan_fits(long long m, long long n, long long k, int op) {
    if (op != OP_NT || m < 1 || m > 32 || n < 1) return false;
    if (k % 16 != 0 || k > 131072) return false;
    if (k > K_LEAF_MIN && leaf_size(k) != K_LEAF_MIN) return false;
    return true;
}

template <int WK, int BM, int CPT, int RSPLIT, int MINB>
inline void launch_skinny_cfg(const GemmArgs &g, int groups, cudaStream_t st) {
    using S = SkinnyShape<BM, CPT, RSPLIT>;
    static std::atomic<bool> configured[64];
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 64 && !configured[dev]) {
        cudaFuncSetAttribute(gemm_skinny_kernel<WK, BM, CPT, RSPLIT, MINB>, cudaFuncAttributeMaxDynamicSharedMemorySize, S::SMEM_BYTES);
        configured[dev] = true;
    }
    dim3 grid((unsigned)((g.n + S::BN - 1) / S::BN), (unsigned)groups);
    gemm_skinny_kernel<WK, BM, CPT, RSPLIT, MINB><<<grid, SK_THREADS, S::SMEM_BYTES, st>>>(g);
}

// columns per thread for the row count (8, 16 or 32 rows of accumulators), and CTAs per SM
constexpr int SK_CPT = 2;                           // at 8, 16 and 32 rows alike (three and four measured within 5 %)
constexpr int SK_MINB8 = 5, SK_MINB16 = 5, SK_MINB32 = 3;
inline int skinny_bn(int) { return SK_THREADS * SK_CPT; }
inline int skinny_per_sm(int m) { return m <= 8 ? SK_MINB8 : (m <= 16 ? SK_MINB16 : SK_MINB32); }

template <int WK>
inline void launch_skinny_wk(const GemmArgs &g, int groups, cudaStream_t st) {
    if (g.m <= 8) launch_skinny_cfg<WK, 8, SK_CPT, 1, SK_MINB8>(g, groups, st);
    else if (g.m <= 16) launch_skinny_cfg<WK, 16, SK_CPT, 1, SK_MINB16>(g, groups, st);
    else launch_skinny_cfg<WK, 32, SK_CPT, 1, SK_MINB32>(g, groups, st);
}

inline void launch_skinny(const GemmArgs &g, int groups, cudaStream_t st) {
    switch (g.wkind) {
    case W_F32: launch_skinny_wk<W_F32>(g, groups, st); break;
    case W_BF16: launch_skinny_wk<W_BF16>(g, groups, st); break;
    case W_INT8_EXP: launch_skinny_wk<W_INT8_EXP>(g, groups, st); break;
    default: launch_skinny_wk<W_INT8_SCALE>(g, groups, st); break;
    }
}

} // namespace b200i
