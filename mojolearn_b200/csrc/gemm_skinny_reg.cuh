// The skinny product for low-bit weights with the weight window held in registers.
//
// Same numerical plan as gemm_skinny.cuh, and the same idea of a thread that owns
// whole output columns with its accumulators packed along m. Two things differ.
// (1) A thread only ever needs the weights of its OWN columns, so they never touch
// shared memory: each window is one 128-bit load per weight row (int8; two for
// bf16) straight into registers, fetched one window ahead and widened exactly, one
// element per k-step, right where it is used. Only the activations are staged: a
// chunk of up to skr_chunk_leaves(BM) leaves of the CTA's rows is transposed into shared
// memory once, with one admission key per 16-step window, so the k loop itself has
// no barrier at all.
// (2) CPT columns per thread and an optional split of the rows over blockIdx.z are
// template parameters. Measured on 32 x 16384 x 2048 int8, two, three and four
// columns per thread and a 16-row split all land within 5 % of each other (the k-step
// is 8 broadcast reads + 2 dequantisations + 32 packed fmas at two columns; the wider
// tiles trade shared-memory wavefronts for registers and resident warps), so the
// default stays two columns, which keeps three CTAs per SM at 32 rows.
// Admission is decided per thread (the chunk's activation key and the thread's own
// weight rows); the bare chain and the flushing chain give the same bits whenever a
// window is admitted, so threads of a warp may disagree without changing a result.
#pragma once
#include "gemm_skinny.cuh"

namespace b200i {

// leaves of activations staged at a time: 32 KiB at 32 rows, 16 KiB at 16 and 8
constexpr int skr_chunk_leaves(int bm) { return bm >= 16 ? 2 : 32 / bm; }

constexpr int skr_smem_bytes(int bm, int leaf) {
    return skr_chunk_leaves(bm) * leaf * bm * 4 + skr_chunk_leaves(bm) * (leaf / KS) * 4;
}

template <int WK>
__device__ __forceinline__ void skr_load_row(SkinnyRaw<WK> &r, const unsigned char *row_base, bool live, int k0) {
    constexpr int ES = WK == W_BF16 ? 2 : 1;
    if (live) {
        const uint4 *p = reinterpret_cast<const uint4 *>(row_base + (size_t)k0 * ES);
#pragma unroll
        for (int q = 0; q < SkinnyRaw<WK>::WORDS / 4; q++) {
            const uint4 v = __ldg(p + q);
            r.w[4 * q] = v.x; r.w[4 * q + 1] = v.y; r.w[4 * q + 2] = v.z; r.w[4 * q + 3] = v.w;
        }
    } else {
#pragma unroll
        for (int q = 0; q < SkinnyRaw<WK>::WORDS; q++) r.w[q] = 0u;
    }
}

// Element e (0..15) of a raw window as the float32 word the plan sees, for a row whose
// quick int8 spelling applies (factor exponent in [27, 227]) or for bf16.
template <int WK>
__device__ __forceinline__ float skr_elem(const SkinnyRaw<WK> &r, int e, float factor, float nbias) {
    if (WK == W_BF16) {
        const unsigned w = r.w[e >> 1];
        return __uint_as_float((e & 1) ? (w & 0xFFFF0000u) : (w << 16));
    } else {
        // r.w holds the codes with the sign bit flipped: code + 128 as an unsigned byte under 2^23's exponent
        const float b = __uint_as_float(__byte_perm(r.w[e >> 2], 0x4B000000u, 0x7540u + (unsigned)(e & 3)));
        if (WK == W_INT8_EXP) return __fmaf_rn(b, factor, nbias);
        return __fmul_rn(__fsub_rn(b, 8388736.0f), factor);
    }
}

// BM rows per CTA (blockIdx.z picks which), CPT columns per thread.
template <int WK, int BM, int CPT, int MINB>
__global__ void __launch_bounds__(SK_THREADS, MINB) gemm_skinny_reg_kernel(const GemmArgs g) {
    static_assert(WK != W_F32, "float32 weights use the shared-memory skinny kernel");
    constexpr int CELLS = BM * CPT, ES = WK == W_BF16 ? 2 : 1, BN = SK_THREADS * CPT;
    constexpr bool INT8 = WK != W_BF16;
    constexpr int SKR_CHUNK_LEAVES = BM >= 16 ? 2 : 32 / BM; // skr_chunk_leaves(BM)
    extern __shared__ __align__(16) float skr_smem[];
    const int chunk_k = SKR_CHUNK_LEAVES * g.leaf;
    float *As = skr_smem;                                                            // [chunk_k][BM]
    unsigned *wkeys = reinterpret_cast<unsigned *>(skr_smem + (size_t)chunk_k * BM); // [chunk_k / KS]

    const int tid = threadIdx.x;
    const int row0 = blockIdx.z * BM, rows = min(BM, g.m - row0);
    const int t_first = blockIdx.y * g.group_leaves;
    const int t_end = min(t_first + g.group_leaves, g.leaves);

    unsigned long long acc[BM / 2][CPT];
#pragma unroll
    for (int i = 0; i < BM / 2; i++)
#pragma unroll
        for (int c = 0; c < CPT; c++) acc[i][c] = 0ull;
    float stack[FOLD_LEVELS][CELLS];

    // this thread's weight rows
    const long long wrow = (long long)blockIdx.x * BN + (long long)CPT * tid;
    const unsigned char *base[CPT];
    bool live[CPT];
    float factor[CPT], nbias[CPT];
    SkinnyRaw<WK> cur[CPT], nxt[CPT]; // .f is the row's exponent / scale word, read once
    bool quick = true;                // every row takes the short exact int8 spelling and is admitted by its factor alone
#pragma unroll
    for (int c = 0; c < CPT; c++) {
        live[c] = wrow + c < g.n;
        base[c] = static_cast<const unsigned char *>(g.b) + (size_t)(live[c] ? wrow + c : 0) * g.k * ES;
        unsigned f = 0u;
        if (INT8 && live[c]) f = __ldg(static_cast<const unsigned *>(g.bscale) + wrow + c);
        cur[c].f = nxt[c].f = f;
        factor[c] = nbias[c] = 0.f;
        if (INT8) {
            factor[c] = !live[c] ? 1.0f : ((WK == W_INT8_EXP) ? pow2_f32((int)f) : __uint_as_float(f)); // a dead row is all-zero codes
            nbias[c] = -8388736.0f * factor[c];
            const unsigned fexp = (__float_as_uint(factor[c]) >> 23) & 0xFFu;
            quick = quick && fexp >= ADMIT_EXP && fexp <= 227u;
        }
    }

    auto load_next = [&](int k0) {
#pragma unroll
        for (int c = 0; c < CPT; c++) skr_load_row<WK>(nxt[c], base[c], live[c], k0);
    };
    // one k-step: b2[c] holds column c's weight in both halves (already flushed when flush is set)
    auto fma_rows = [&](const float *arow, const unsigned long long (&b2)[CPT], bool flush) {
#pragma unroll
        for (int q = 0; q < BM / 4; q++) {
            ulonglong2 a4 = *reinterpret_cast<const ulonglong2 *>(arow + 4 * q);
            if (flush) {
                float y0, y1, y2, y3;
                unpack2(a4.x, y0, y1);
                unpack2(a4.y, y2, y3);
                a4.x = pack2(ftz_bits(y0), ftz_bits(y1));
                a4.y = pack2(ftz_bits(y2), ftz_bits(y3));
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
    auto unpack_cells = [&](float (&v)[CELLS], bool clear_acc) {
#pragma unroll
        for (int i = 0; i < BM / 2; i++)
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

    if (t_first < t_end) load_next(t_first * g.leaf);
    for (int tc = t_first; tc < t_end; tc += SKR_CHUNK_LEAVES) {
        // ---- stage the chunk's activations: As[kloc][row], one admission key per window ----
        const int kb = tc * g.leaf, ke = min(min(tc + SKR_CHUNK_LEAVES, t_end) * g.leaf, g.k);
        const int quads = (ke - kb) / 4;
        if (tc != t_first) __syncthreads(); // the previous chunk is fully consumed
        for (int w = tid; w < (ke - kb) / KS; w += SK_THREADS) wkeys[w] = 0xFFFFFFFFu;
        __syncthreads();
        for (int idx0 = 0; idx0 < quads * BM; idx0 += 4 * SK_THREADS) {
            float4 v[4];
#pragma unroll
            for (int u = 0; u < 4; u++) {
                const int idx = idx0 + u * SK_THREADS + tid, r = idx % BM, q = idx / BM;
                v[u] = make_float4(0.f, 0.f, 0.f, 0.f);
                if (q < quads && r < rows) v[u] = __ldg(reinterpret_cast<const float4 *>(g.a + (size_t)(row0 + r) * g.k + kb + 4 * q));
            }
#pragma unroll
            for (int u = 0; u < 4; u++) {
                const int idx = idx0 + u * SK_THREADS + tid, r = idx % BM, q = idx / BM;
                if (q < quads) {
                    float *dst = As + (size_t)(4 * q) * BM + r;
                    dst[0] = v[u].x; dst[BM] = v[u].y; dst[2 * BM] = v[u].z; dst[3 * BM] = v[u].w;
                    const unsigned key = key4(v[u], 0xFFFFFFFFu);
                    if (key < ADMIT_MIN) atomicMin(&wkeys[q / 4], key);
                }
            }
        }
        __syncthreads();

        // ---- the chunk's leaves: weights from registers, activations from shared memory ----
        const int tc_end = min(tc + SKR_CHUNK_LEAVES, t_end);
        for (int t = tc; t < tc_end; t++) {
            const int leaf_len = min(g.leaf, g.k - t * g.leaf);
            bool leaf_clean = true;
            for (int koff = 0; koff < leaf_len; koff += KS) {
                unsigned key = 0xFFFFFFFFu;
#pragma unroll
                for (int c = 0; c < CPT; c++) {
#pragma unroll
                    for (int q = 0; q < SkinnyRaw<WK>::WORDS; q++) cur[c].w[q] = nxt[c].w[q];
                    if (!INT8) {
#pragma unroll
                        for (int q = 0; q < SkinnyRaw<WK>::WORDS; q++)
                            key = min(key, min(admit_key(__uint_as_float(cur[c].w[q] << 16)), admit_key(__uint_as_float(cur[c].w[q] & 0xFFFF0000u))));
                    }
                }
                int nt = t, nkoff = koff + KS;
                if (nkoff >= leaf_len) { nt = t + 1; nkoff = 0; }
                if (nt < t_end) load_next(nt * g.leaf + nkoff);
                const int kloc = (t - tc) * g.leaf + koff;
                key = min(key, wkeys[kloc / KS]);
                const float *arow = As + (size_t)kloc * BM;
                if (leaf_clean && quick && key >= ADMIT_MIN) {
                    if (INT8) {
#pragma unroll
                        for (int c = 0; c < CPT; c++)
#pragma unroll
                            for (int q = 0; q < 4; q++) cur[c].w[q] ^= 0x80808080u;
                    }
#pragma unroll
                    for (int kk = 0; kk < KS; kk++) {
                        unsigned long long b2[CPT];
#pragma unroll
                        for (int c = 0; c < CPT; c++) {
                            const float w = skr_elem<WK>(cur[c], kk, factor[c], nbias[c]);
                            b2[c] = pack2(w, w);
                        }
                        fma_rows(arow + kk * BM, b2, false);
                    }
                } else {
                    // the defining chain, one k-step at a time: the low element of each raw window, then shift it out
                    leaf_clean = false;
#pragma unroll 1
                    for (int kk = 0; kk < KS; kk++) {
                        float w[CPT];
#pragma unroll
                        for (int c = 0; c < CPT; c++) {
                            if (INT8) {
                                w[c] = dequant_int8_pow2((int)(signed char)(cur[c].w[0] & 0xFFu), factor[c]);
#pragma unroll
                                for (int q = 0; q < 3; q++) cur[c].w[q] = __funnelshift_r(cur[c].w[q], cur[c].w[q + 1], 8);
                                cur[c].w[3] >>= 8;
                            } else {
                                w[c] = __uint_as_float(cur[c].w[0] << 16);
#pragma unroll
                                for (int q = 0; q < 7; q++) cur[c].w[q] = __funnelshift_r(cur[c].w[q], cur[c].w[q + 1], 16);
                                cur[c].w[7] >>= 16;
                            }
                        }
                        unsigned long long b2[CPT];
#pragma unroll
                        for (int c = 0; c < CPT; c++) b2[c] = pack2(ftz_bits(w[c]), ftz_bits(w[c]));
                        fma_rows(arow + kk * BM, b2, true);
                    }
                }
            }
            if (t + 1 < t_end) push_leaf(t - t_first);
        }
    }

    const int count = t_end - t_first;
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
    float *out = g.groups > 1 ? g.ws + (size_t)blockIdx.y * (size_t)g.m * (size_t)g.n : g.c;
    if (CPT == 2 && g.groups == 1 && epilogue_pairs(g.epi)) { // this thread's two columns are one (gate, up) pair
        if (wrow + 1 < g.n)
            for (int i = 0; i < rows; i++)
                g.c[(size_t)(row0 + i) * (g.n / 2) + wrow / 2] =
                    epilogue_pair_apply(nan_canon(ftz_hw(v[i * CPT])), nan_canon(ftz_hw(v[i * CPT + 1])), g.epi.bias, g.epi.act, wrow / 2);
        return;
    }
#pragma unroll
    for (int i = 0; i < BM; i++) {
        if (i >= rows) break;
#pragma unroll
        for (int c = 0; c < CPT; c++)
            if (wrow + c < g.n) out[(size_t)(row0 + i) * g.n + wrow + c] = nan_canon(ftz_hw(v[i * CPT + c]));
    }
    if (g.groups == 1 && epilogue_on(g.epi)) { // this thread's own cells once more (see epilogue_cell)
        for (int i = 0; i < rows; i++)
            for (int c = 0; c < CPT; c++)
                if (wrow + c < g.n) epilogue_cell(out + (size_t)(row0 + i) * g.n + wrow + c, g.epi, wrow + c);
    }
}

// Thread tile for a row count: BM rows per CTA (the rows are split over blockIdx.z when m > BM),
// CPT columns per thread, CTAs per SM.
constexpr int SKR_CPT = 2;
constexpr int SKR_MINB8 = 5, SKR_MINB16 = 5, SKR_MINB32 = 3;
inline int skr_bm(int m) { return m <= 8 ? 8 : (m <= 16 ? 16 : 32); }
inline int skr_bn(int) { return SK_THREADS * SKR_CPT; }
inline int skr_per_sm(int m) { return m <= 8 ? SKR_MINB8 : (m <= 16 ? SKR_MINB16 : SKR_MINB32); }

template <int WK, int BM, int CPT, int MINB>
inline void launch_skinny_reg_cfg(const GemmArgs &g, int groups, cudaStream_t st) {
    static std::atomic<bool> configured[64];
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 64 && !configured[dev]) {
        cudaFuncSetAttribute(gemm_skinny_reg_kernel<WK, BM, CPT, MINB>, cudaFuncAttributeMaxDynamicSharedMemorySize, skr_smem_bytes(BM, K_LEAF_MIN));
        configured[dev] = true;
    }
    dim3 grid((unsigned)((g.n + SK_THREADS * CPT - 1) / (SK_THREADS * CPT)), (unsigned)groups, (unsigned)((g.m + BM - 1) / BM));
    gemm_skinny_reg_kernel<WK, BM, CPT, MINB><<<grid, SK_THREADS, skr_smem_bytes(BM, g.leaf), st>>>(g);
}

template <int WK>
inline void launch_skinny_reg_wk(const GemmArgs &g, int groups, int sms, cudaStream_t st) {
    // A narrow product (one rank's column shard of a layer) has too few column tiles x leaf groups to fill the device:
    // its rows are then split over more CTAs (8 or 16 rows each instead of 32) until at least half of the SMs have one.
    // A cell's chain does not change with the CTA that runs it. Measured on one GPU running rank 0's share of a 24-layer
    // decode step (batch 32, d_model 2048, int8): 3.24 against 3.52 ms at 8 ranks, 3.79 against 3.92 at 4, 5.11 against 5.18
    // at 2; splitting up to one CTA per SM, or up to 1.5, measured within 1 % of this rule.
    int bm = skr_bm(g.m);
    const long long tiles = (g.n + skr_bn(g.m) - 1) / skr_bn(g.m);
    while (bm > 8 && tiles * groups * ((g.m + bm - 1) / bm) * 2 <= sms) bm /= 2;
    if (bm <= 8) launch_skinny_reg_cfg<WK, 8, SKR_CPT, SKR_MINB8>(g, groups, st);
    else if (bm <= 16) launch_skinny_reg_cfg<WK, 16, SKR_CPT, SKR_MINB16>(g, groups, st);
    else launch_skinny_reg_cfg<WK, 32, SKR_CPT, SKR_MINB32>(g, groups, st);
}

// low-bit weight kinds only; the caller keeps float32 weights on launch_skinny
inline void launch_skinny_reg(const GemmArgs &g, int groups, int sms, cudaStream_t st) {
    switch (g.wkind) {
    case W_BF16: launch_skinny_reg_wk<W_BF16>(g, groups, sms, st); break;
    case W_INT8_EXP: launch_skinny_reg_wk<W_INT8_EXP>(g, groups, sms, st); break;
    default: launch_skinny_reg_wk<W_INT8_SCALE>(g, groups, sms, st); break;
    }
}

} // namespace b200i
