// The tiled identical-mode GEMM kernel for sm_100a.
//
// NUMERICAL PLAN (fixed by the contract, gemm/IDENTICAL_FP32_CONTRACT.md and
// gemm/host/gemm_oracle.mojo:146-371 of the reference): k is cut into leaves of
// leaf_size(k) elements; a cell's leaf partial is ONE accumulator seeded +0.0
// and advanced p-ascending by acc = ftz(fma_rn(ftz(a), ftz(b), acc)); the
// partials are folded by the fixed adjacent-pair tree with an odd tail carried.
//
// EXECUTION PLAN (free, and chosen here for B200): a CTA owns a BM x BN tile of
// C and a power-of-two aligned group of leaves. Operands are staged global ->
// registers -> shared memory in windows of 16 k-steps, double buffered, with
// 128-bit loads and stores; while a window is staged every thread folds the
// admission key of the words it touched, and the __syncthreads_and that
// publishes the window also publishes whether it is admitted. An admitted
// window runs the bare packed fma (fma.rn.f32x2: two cells per instruction,
// which leaves issue slots for the shared-memory loads); any other window, and
// the rest of its leaf, runs fma + flush. A window never crosses a leaf
// boundary and a ragged k tail is looped, never zero padded (a padded step
// would turn a -0.0 accumulator into +0.0). At a leaf boundary the partial is
// pushed on a per-thread binary-counter stack, which merges (2q, 2q+1) pairs
// as soon as both exist and carries an odd tail at the drain: the contract's
// tree evaluated in streaming order.
#pragma once
#include "seams.cuh"
#include "seams_math.cuh"

namespace b200i {

struct GemmArgs {
    const float *a;     // left operand, float32
    const void *b;      // right operand, storage per wkind
    const void *bscale; // int32 exponents or float32 scales, one per right-operand row (int8 kinds)
    float *c;           // m x n output
    float *ws;          // group nodes [groups][m][n] when groups > 1
    int m, n, k, op, wkind;
    int leaf, leaves;         // L and P
    int group_leaves, groups; // S (a power of two) and ceil(P / S)
    int vec_a, vec_b, vec_c;  // operand may be read / written with 128-bit accesses
    int tiles_n;
    int dec_smem_limit;       // decode plan: shared memory a CTA may use (decides one or two CTAs per SM)
    Epilogue epi;             // bias / activation applied where the product's output is stored
};

constexpr int KS = 16;       // k-steps per staged window
constexpr int FOLD_LEVELS = 11; // 2^10 = MAX_LEAVES

template <int BM, int BN, int RM, int RN>
struct TileShape {
    static constexpr int TX = BN / (4 * RN), TY = BM / (4 * RM), THREADS = TX * TY;
    static constexpr int TM = 4 * RM, TN = 4 * RN;
    static constexpr int UNITS = BM + BN; // staging units of 16 words each
    static constexpr int UPT = (UNITS + THREADS - 1) / THREADS;
    static constexpr int SMEM_BYTES = (2 * 16 * (BM + BN) + TM * TN * THREADS) * 4;
};

// ---- staging -------------------------------------------------------------------
// A unit is 16 words of one operand's window: either 4 rows x 4 consecutive k
// of a k-contiguous operand (transposed through registers on the way to shared
// memory) or 4 k-rows x 4 consecutive cells of a cell-contiguous operand.

// Raw words of one unit as they come out of global memory. Nothing here touches
// a loaded value, so the loads stay in flight while the previous window computes;
// widening, dequantisation and the admission key happen at store time.
struct UnitRaw {
    uint4 w[4];    // float32: 4 words; bf16: 4 patterns in .x/.y; int8: 4 codes in .x
    unsigned f[4]; // int8 kinds, k-contiguous: the row's raw exponent or scale word
};

__device__ __forceinline__ uint4 ld4_words(const float *p, bool vec, int valid) {
    uint4 r = make_uint4(0u, 0u, 0u, 0u);
    if (valid <= 0) return r;
    if (vec) return __ldg(reinterpret_cast<const uint4 *>(p));
    r.x = __float_as_uint(__ldg(p));
    if (valid > 1) r.y = __float_as_uint(__ldg(p + 1));
    if (valid > 2) r.z = __float_as_uint(__ldg(p + 2));
    if (valid > 3) r.w = __float_as_uint(__ldg(p + 3));
    return r;
}
__device__ __forceinline__ uint4 ld4_halves(const unsigned short *p, bool vec, int valid) {
    uint4 r = make_uint4(0u, 0u, 0u, 0u);
    if (valid <= 0) return r;
    if (vec) {
        const uint2 w = __ldg(reinterpret_cast<const uint2 *>(p));
        r.x = w.x;
        r.y = w.y;
        return r;
    }
    r.x = __ldg(p);
    if (valid > 1) r.x |= (unsigned)__ldg(p + 1) << 16;
    if (valid > 2) r.y = __ldg(p + 2);
    if (valid > 3) r.y |= (unsigned)__ldg(p + 3) << 16;
    return r;
}
__device__ __forceinline__ uint4 ld4_bytes(const signed char *p, bool vec, int valid) {
    uint4 r = make_uint4(0u, 0u, 0u, 0u);
    if (valid <= 0) return r;
    if (vec) {
        r.x = (unsigned)__ldg(reinterpret_cast<const int *>(p));
        return r;
    }
    r.x = (unsigned)(unsigned char)__ldg(p);
    if (valid > 1) r.x |= (unsigned)(unsigned char)__ldg(p + 1) << 8;
    if (valid > 2) r.x |= (unsigned)(unsigned char)__ldg(p + 2) << 16;
    if (valid > 3) r.x |= (unsigned)(unsigned char)__ldg(p + 3) << 24;
    return r;
}

__device__ __forceinline__ unsigned key4(float4 v, unsigned k) {
    k = min(k, admit_key(v.x));
    k = min(k, admit_key(v.y));
    k = min(k, admit_key(v.z));
    k = min(k, admit_key(v.w));
    return k;
}

// Loads one unit of the left operand (E = BM, origin e0 = first row of the
// tile) or of the right operand (E = BN). `kcontig` says the operand's storage
// is contiguous along k.
template <int E>
__device__ __forceinline__ void unit_load(UnitRaw &r, int u, const void *base, int wkind, const void *scale, bool kcontig,
                                          bool vec, int e0, int extent, int kdim, int k0) {
    const int lane_e = u % (E / 4), quad = u / (E / 4);
    if (kcontig) {
        const int kk = k0 + 4 * quad;
        const int kvalid = kdim - kk;
#pragma unroll
        for (int c = 0; c < 4; c++) {
            const int row = e0 + 4 * lane_e + c;
            const int valid = (row < extent) ? kvalid : 0;
            const size_t off = (size_t)row * (size_t)kdim + (size_t)kk;
            r.f[c] = 0u;
            if (wkind == W_F32) r.w[c] = ld4_words(static_cast<const float *>(base) + off, vec, valid);
            else if (wkind == W_BF16) r.w[c] = ld4_halves(static_cast<const unsigned short *>(base) + off, vec, valid);
            else {
                if (valid > 0) r.f[c] = __ldg(static_cast<const unsigned *>(scale) + row);
                r.w[c] = ld4_bytes(static_cast<const signed char *>(base) + off, vec, valid);
            }
        }
    } else {
        const int col = e0 + 4 * lane_e;
        const int cvalid = extent - col;
#pragma unroll
        for (int c = 0; c < 4; c++) {
            const int kk = k0 + 4 * quad + c;
            const int valid = (kk < kdim) ? cvalid : 0;
            const size_t off = (size_t)kk * (size_t)extent + (size_t)col;
            r.f[c] = 0u;
            if (wkind == W_BF16) r.w[c] = ld4_halves(static_cast<const unsigned short *>(base) + off, vec, valid);
            else r.w[c] = ld4_words(static_cast<const float *>(base) + off, vec, valid);
        }
    }
}

// The float32 words a unit stands for: exact widening / dequantisation.
__device__ __forceinline__ void unit_widen(const UnitRaw &r, int wkind, float4 (&v)[4]) {
#pragma unroll
    for (int c = 0; c < 4; c++) {
        const uint4 w = r.w[c];
        if (wkind == W_F32) {
            v[c] = make_float4(__uint_as_float(w.x), __uint_as_float(w.y), __uint_as_float(w.z), __uint_as_float(w.w));
        } else if (wkind == W_BF16) {
            v[c] = make_float4(__uint_as_float(w.x << 16), __uint_as_float(w.x & 0xFFFF0000u), __uint_as_float(w.y << 16),
                               __uint_as_float(w.y & 0xFFFF0000u));
        } else {
            const float factor = (wkind == W_INT8_EXP) ? pow2_f32((int)r.f[c]) : __uint_as_float(r.f[c]);
            const int word = (int)w.x;
            v[c] = make_float4(dequant_int8_pow2((int)(signed char)(word & 0xFF), factor),
                               dequant_int8_pow2((int)(signed char)((word >> 8) & 0xFF), factor),
                               dequant_int8_pow2((int)(signed char)((word >> 16) & 0xFF), factor),
                               dequant_int8_pow2(word >> 24, factor));
        }
    }
}

template <int E>
__device__ __forceinline__ void unit_store(const float4 (&r)[4], int u, float (*dst)[E], bool kcontig) {
    const int lane_e = u % (E / 4), quad = u / (E / 4);
    if (kcontig) {
        *reinterpret_cast<float4 *>(&dst[4 * quad + 0][4 * lane_e]) = make_float4(r[0].x, r[1].x, r[2].x, r[3].x);
        *reinterpret_cast<float4 *>(&dst[4 * quad + 1][4 * lane_e]) = make_float4(r[0].y, r[1].y, r[2].y, r[3].y);
        *reinterpret_cast<float4 *>(&dst[4 * quad + 2][4 * lane_e]) = make_float4(r[0].z, r[1].z, r[2].z, r[3].z);
        *reinterpret_cast<float4 *>(&dst[4 * quad + 3][4 * lane_e]) = make_float4(r[0].w, r[1].w, r[2].w, r[3].w);
    } else {
#pragma unroll
        for (int c = 0; c < 4; c++) *reinterpret_cast<float4 *>(&dst[4 * quad + c][4 * lane_e]) = r[c];
    }
}

// ---- the kernel -------------------------------------------------------------------

template <int BM, int BN, int RM, int RN, int MINB>
__global__ void __launch_bounds__((TileShape<BM, BN, RM, RN>::THREADS), MINB) gemm_tile_kernel(const GemmArgs g) {
    using S = TileShape<BM, BN, RM, RN>;
    constexpr int TM = S::TM, TN = S::TN, NT = S::THREADS, UPT = S::UPT;
    // dynamic shared memory: two pages of each operand window, then level 0 of the fold stack
    extern __shared__ __align__(16) float tile_smem[];
    float (*As)[KS][BM] = reinterpret_cast<float (*)[KS][BM]>(tile_smem);
    float (*Bs)[KS][BN] = reinterpret_cast<float (*)[KS][BN]>(tile_smem + 2 * KS * BM);
    float (*level0)[NT] = reinterpret_cast<float (*)[NT]>(tile_smem + 2 * KS * (BM + BN)); // [cell][thread]: conflict free

    const int tid = threadIdx.x;
    const int tx = tid % S::TX, ty = tid / S::TX;
    const int bm0 = (blockIdx.x / g.tiles_n) * BM;
    const int bn0 = (blockIdx.x % g.tiles_n) * BN;
    const bool a_kcontig = (g.op != OP_TN);
    const bool b_kcontig = (g.op == OP_NT);

    const int t_first = blockIdx.y * g.group_leaves;
    const int t_end = min(t_first + g.group_leaves, g.leaves);

    // accumulators: TM rows x TN/2 packed column pairs
    unsigned long long acc[TM][TN / 2];
#pragma unroll
    for (int i = 0; i < TM; i++)
#pragma unroll
        for (int j = 0; j < TN / 2; j++) acc[i][j] = 0ull;

    float stack[FOLD_LEVELS - 1][TM * TN]; // levels 1.. in local memory (level 0 is in shared memory)

    UnitRaw stage[UPT];
    unsigned stage_key;

    auto load_window = [&](int t, int koff) { // loads only: nothing waits on them until store_window
        const int k0 = t * g.leaf + koff;
#pragma unroll
        for (int i = 0; i < UPT; i++) {
            const int u = tid + i * NT;
            if (u < BM) unit_load<BM>(stage[i], u, g.a, W_F32, nullptr, a_kcontig, g.vec_a, bm0, g.m, g.k, k0);
            else if (u < BM + BN)
                unit_load<BN>(stage[i], u - BM, g.b, g.wkind, g.bscale, b_kcontig, g.vec_b, bn0, g.n, g.k, k0);
        }
    };
    auto store_window = [&](int buf) { // widen, fold the admission key, store
        stage_key = 0xFFFFFFFFu;
#pragma unroll
        for (int i = 0; i < UPT; i++) {
            const int u = tid + i * NT;
            if (u < BM + BN) {
                float4 v[4];
                unit_widen(stage[i], u < BM ? W_F32 : g.wkind, v);
#pragma unroll
                for (int c = 0; c < 4; c++) stage_key = key4(v[c], stage_key);
                if (u < BM) unit_store<BM>(v, u, As[buf], a_kcontig);
                else unit_store<BN>(v, u - BM, Bs[buf], b_kcontig);
            }
        }
    };

    auto read_operands = [&](int buf, int kk, float (&av)[TM], float (&bv)[TN]) {
#pragma unroll
        for (int r = 0; r < RM; r++) {
            const float4 v = *reinterpret_cast<const float4 *>(&As[buf][kk][r * (BM / RM) + ty * 4]);
            av[4 * r + 0] = v.x; av[4 * r + 1] = v.y; av[4 * r + 2] = v.z; av[4 * r + 3] = v.w;
        }
#pragma unroll
        for (int r = 0; r < RN; r++) {
            const float4 v = *reinterpret_cast<const float4 *>(&Bs[buf][kk][r * (BN / RN) + tx * 4]);
            bv[4 * r + 0] = v.x; bv[4 * r + 1] = v.y; bv[4 * r + 2] = v.z; bv[4 * r + 3] = v.w;
        }
    };
    auto step_fast = [&](int buf, int kk) {
        float av[TM], bv[TN];
        read_operands(buf, kk, av, bv);
        unsigned long long b2[TN / 2];
#pragma unroll
        for (int j = 0; j < TN / 2; j++) b2[j] = pack2(bv[2 * j], bv[2 * j + 1]);
#pragma unroll
        for (int i = 0; i < TM; i++) {
            const unsigned long long a2 = pack2(av[i], av[i]);
#pragma unroll
            for (int j = 0; j < TN / 2; j++) acc[i][j] = fma2_bare(a2, b2[j], acc[i][j]);
        }
    };
    auto step_slow = [&](int buf, int kk) {
        float av[TM], bv[TN];
        read_operands(buf, kk, av, bv);
        unsigned long long b2[TN / 2];
#pragma unroll
        for (int j = 0; j < TN / 2; j++) b2[j] = pack2(ftz_bits(bv[2 * j]), ftz_bits(bv[2 * j + 1]));
#pragma unroll
        for (int i = 0; i < TM; i++) {
            const float af = ftz_bits(av[i]);
            const unsigned long long a2 = pack2(af, af);
#pragma unroll
            for (int j = 0; j < TN / 2; j++) acc[i][j] = ftz2_hw(fma2_bare(a2, b2[j], acc[i][j]));
        }
    };

    // leaf boundary: push the partial on the binary-counter stack. The merge depth
    // depends on the leaf index alone, so the walk is level-major: all TM*TN loads
    // of a level are independent and in flight together.
    auto push_leaf = [&](int local_leaf) {
        float v[TM * TN];
#pragma unroll
        for (int i = 0; i < TM; i++)
#pragma unroll
            for (int j = 0; j < TN / 2; j++) {
                float v0, v1;
                unpack2(acc[i][j], v0, v1);
                v[i * TN + 2 * j] = ftz_hw(v0);
                v[i * TN + 2 * j + 1] = ftz_hw(v1);
                acc[i][j] = 0ull;
            }
        if ((local_leaf & 1) == 0) { // an even leaf waits at level 0 for its right sibling
#pragma unroll
            for (int c = 0; c < TM * TN; c++) level0[c][tid] = v[c];
            return;
        }
#pragma unroll
        for (int c = 0; c < TM * TN; c++) v[c] = fold_add(level0[c][tid], v[c]);
        int lvl = 1;
        for (int bits = local_leaf >> 1; bits & 1; bits >>= 1, lvl++) {
#pragma unroll
            for (int c = 0; c < TM * TN; c++) v[c] = fold_add(stack[lvl - 1][c], v[c]);
        }
#pragma unroll
        for (int c = 0; c < TM * TN; c++) stack[lvl - 1][c] = v[c];
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
            // the window after this one
            int nt = t, nkoff = koff + KS;
            if (nkoff >= leaf_len) { nt = t + 1; nkoff = 0; }
            const bool more = nt < t_end;
            if (more) load_window(nt, nkoff);

            const bool fast = admitted && leaf_clean && len == KS;
            if (fast) {
#pragma unroll
                for (int kk = 0; kk < KS; kk++) step_fast(buf, kk);
            } else {
                leaf_clean = false;
#pragma unroll 1
                for (int kk = 0; kk < len; kk++) step_slow(buf, kk);
            }
            if (nt != t) { // this window closed its leaf; the group's last leaf stays in registers for the drain
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

    // Drain and store. The group's last partial is still in registers: pushing it
    // would merge it with every level whose bit is set in its index below the first
    // clear bit, and the drain would then add the remaining occupied levels in
    // ascending order (the carry rule). Together: add stack[l] for every set bit l of
    // (count - 1), ascending, level-major so the loads of a level fly together.
    const int count = t_end - t_first;
    float *out = g.groups > 1 ? g.ws + (size_t)blockIdx.y * (size_t)g.m * (size_t)g.n : g.c;
    float v[TM * TN];
#pragma unroll
    for (int i = 0; i < TM; i++)
#pragma unroll
        for (int j = 0; j < TN / 2; j++) {
            float v0, v1;
            unpack2(acc[i][j], v0, v1);
            v[i * TN + 2 * j] = ftz_hw(v0);
            v[i * TN + 2 * j + 1] = ftz_hw(v1);
        }
    if (count > 1) {
        const int last = count - 1;
        if (last & 1) {
#pragma unroll
            for (int c = 0; c < TM * TN; c++) v[c] = fold_add(level0[c][tid], v[c]);
        }
        for (int lvl = 1; lvl < FOLD_LEVELS; lvl++)
            if ((last >> lvl) & 1) {
#pragma unroll
                for (int c = 0; c < TM * TN; c++) v[c] = fold_add(stack[lvl - 1][c], v[c]);
            }
    }
#pragma unroll
    for (int i = 0; i < TM; i++) {
        const int row = bm0 + (i / 4) * (BM / RM) + ty * 4 + (i % 4);
#pragma unroll
        for (int jr = 0; jr < RN; jr++) {
            float vals[4];
#pragma unroll
            for (int e = 0; e < 4; e++) vals[e] = nan_canon(ftz_hw(v[i * TN + jr * 4 + e]));
            const int col = bn0 + jr * (BN / RN) + tx * 4;
            if (row < g.m) {
                float *dst = out + (size_t)row * (size_t)g.n + col;
                if (g.vec_c && col + 3 < g.n) *reinterpret_cast<float4 *>(dst) = make_float4(vals[0], vals[1], vals[2], vals[3]);
                else
                    for (int e = 0; e < 4; e++)
                        if (col + e < g.n) dst[e] = vals[e];
            }
        }
    }
}

// The store epilogue of the tiled and packed plans, as a pass of its own over the finished output: those kernels'
// store loops hold 64 live cells per thread and are left exactly as they are (a product large enough for them does
// not notice one more elementwise launch; the plans for small products apply the epilogue where they store).
__global__ void epilogue_rows_kernel(float *__restrict__ c, long long cells, int n, Epilogue epi) {
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < cells; i += stride) epilogue_cell(c + i, epi, i % n);
}

// Folds the group nodes of a split product: node g of cell c is ws[g][c]; the
// nodes are the level-log2(S) row of the contract's tree, so the same
// adjacent-pair fold with an odd tail carried finishes it. The fold is streamed
// through the binary-counter stack the product kernels use (a node is pushed,
// merging while the counter's low bits are set; the last node drains the
// stack): the stack lives in registers, VEC consecutive cells per thread.
constexpr int MAX_GROUPS = 64;
constexpr int GROUP_LEVELS = 6; // 2^6 = MAX_GROUPS
// The finished cells of one thread: canonical NaN, the store, and the store epilogue where one is asked for.
template <int VEC>
__device__ __forceinline__ void fold_finish(const float (&v)[VEC], float *__restrict__ c, long long idx, Epilogue epi, int n) {
    if (VEC == 4 && epilogue_pairs(epi)) {
        // gated activation: the four cells are two (gate, up) pairs of one row; the output has n / 2 columns
        const long long row = idx / n, col = idx - row * n;
        float2 o;
        o.x = epilogue_pair_apply(nan_canon(ftz_hw(v[0])), nan_canon(ftz_hw(v[1 % VEC])), epi.bias, epi.act, col / 2);
        o.y = epilogue_pair_apply(nan_canon(ftz_hw(v[2 % VEC])), nan_canon(ftz_hw(v[3 % VEC])), epi.bias, epi.act, col / 2 + 1);
        *reinterpret_cast<float2 *>(c + row * (n / 2) + col / 2) = o;
        return;
    }
    if (VEC == 4) {
        *reinterpret_cast<float4 *>(c + idx) = make_float4(nan_canon(ftz_hw(v[0])), nan_canon(ftz_hw(v[1 % VEC])),
                                                           nan_canon(ftz_hw(v[2 % VEC])), nan_canon(ftz_hw(v[3 % VEC])));
    } else {
        c[idx] = nan_canon(ftz_hw(v[0]));
    }
    if (epilogue_on(epi))
        for (int e = 0; e < VEC; e++) epilogue_cell(c + idx + e, epi, (idx + e) % n);
}

// One step of the binary-counter fold: node number `gi` of `count` arrives in v; on return v is the root when gi was the
// last node, otherwise it has been merged into the stack.
template <int VEC, int LEVELS>
__device__ __forceinline__ void fold_push(float (&stack)[LEVELS][VEC], float (&v)[VEC], int gi, int last) {
    if (gi == last) { // the last node drains the stack
#pragma unroll
        for (int lvl = 0; lvl < LEVELS; lvl++)
            if ((last >> lvl) & 1) {
#pragma unroll
                for (int e = 0; e < VEC; e++) v[e] = fold_add(stack[lvl][e], v[e]);
            }
    } else {
        bool placed = false;
#pragma unroll
        for (int lvl = 0; lvl < LEVELS; lvl++) {
            if (placed) continue;
            if ((gi >> lvl) & 1) {
#pragma unroll
                for (int e = 0; e < VEC; e++) v[e] = fold_add(stack[lvl][e], v[e]);
            } else {
#pragma unroll
                for (int e = 0; e < VEC; e++) stack[lvl][e] = v[e];
                placed = true;
            }
        }
    }
}

// The same fold for a product split into MANY groups over FEW cells (a narrow weight cut into 32 or 64 single-leaf
// groups: the column shard of one rank): a thread walking all nodes of its cells alone is a chain of L2 round trips, so
// the groups are cut into blocks of eight (aligned subtrees of the fold tree, the last one possibly ragged), warp s of
// the CTA folds block s of 32 x 4 cells with all eight nodes in flight at once, and warp 0 folds the block roots, which
// form the same adjacent-pair tree three levels up.
constexpr int FOLD_SUB = 8;
__global__ void __launch_bounds__(32 * MAX_GROUPS / FOLD_SUB) fold_groups_split_kernel(const float *__restrict__ ws, float *__restrict__ c, long long cells,
                                                                                       int groups, Epilogue epi, int n) {
    __shared__ float4 roots[MAX_GROUPS / FOLD_SUB][32];
    const int lane = threadIdx.x & 31, sub = threadIdx.x >> 5;
    const int subs = (groups + FOLD_SUB - 1) / FOLD_SUB;
    const long long idx = ((long long)blockIdx.x * 32 + lane) * 4;
    const bool live = idx < cells;
    const int g0 = sub * FOLD_SUB, count = min(FOLD_SUB, groups - g0);
    float v[4] = {0.f, 0.f, 0.f, 0.f};
    if (live) {
        float4 x[FOLD_SUB];
#pragma unroll
        for (int j = 0; j < FOLD_SUB; j++)
            if (j < count) x[j] = __ldcg(reinterpret_cast<const float4 *>(ws + (size_t)(g0 + j) * (size_t)cells + idx));
        float stack[3][4];
#pragma unroll
        for (int j = 0; j < FOLD_SUB; j++) {
            if (j >= count) break;
            v[0] = x[j].x; v[1] = x[j].y; v[2] = x[j].z; v[3] = x[j].w;
            fold_push<4, 3>(stack, v, j, count - 1);
        }
        roots[sub][lane] = make_float4(v[0], v[1], v[2], v[3]);
    }
    __syncthreads();
    if (sub != 0 || !live) return;
    float stack[3][4];
    for (int s2 = 0; s2 < subs; s2++) {
        const float4 t = roots[s2][lane];
        v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
        fold_push<4, 3>(stack, v, s2, subs - 1);
    }
    fold_finish<4>(v, c, idx, epi, n);
}

template <int VEC>
__global__ void __launch_bounds__(256) fold_groups_kernel(const float *__restrict__ ws, float *__restrict__ c, long long cells,
                                                          int groups, Epilogue epi, int n) {
    const long long idx = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * VEC;
    if (idx >= cells) return;
    float stack[GROUP_LEVELS][VEC];
    float v[VEC];
    // Eight nodes are requested at a time: a lone thread's chain of additions waits on memory once per eight nodes
    // instead of once per node (a deep product split into 64 single-leaf groups was 64 L2 round trips long).
    constexpr int AHEAD = 8;
    const int last = groups - 1;
    for (int g0 = 0; g0 < groups; g0 += AHEAD) {
        float x[AHEAD][VEC];
#pragma unroll
        for (int j = 0; j < AHEAD; j++) {
            if (g0 + j >= groups) break;
            const float *src = ws + (size_t)(g0 + j) * (size_t)cells + idx;
            if (VEC == 4) {
                const float4 t = __ldcg(reinterpret_cast<const float4 *>(src));
                x[j][0] = t.x; x[j][1 % VEC] = t.y; x[j][2 % VEC] = t.z; x[j][3 % VEC] = t.w;
            } else {
                x[j][0] = __ldcg(src);
            }
        }
#pragma unroll
        for (int j = 0; j < AHEAD; j++) {
            const int gi = g0 + j;
            if (gi >= groups) break;
#pragma unroll
            for (int e = 0; e < VEC; e++) v[e] = x[j][e];
            if (gi == last) { // the last node drains the stack
#pragma unroll
                for (int lvl = 0; lvl < GROUP_LEVELS; lvl++)
                    if ((last >> lvl) & 1) {
#pragma unroll
                        for (int e = 0; e < VEC; e++) v[e] = fold_add(stack[lvl][e], v[e]);
                    }
            } else {
                bool placed = false;
#pragma unroll
                for (int lvl = 0; lvl < GROUP_LEVELS; lvl++) {
                    if (placed) continue;
                    if ((gi >> lvl) & 1) {
#pragma unroll
                        for (int e = 0; e < VEC; e++) v[e] = fold_add(stack[lvl][e], v[e]);
                    } else {
#pragma unroll
                        for (int e = 0; e < VEC; e++) stack[lvl][e] = v[e];
                        placed = true;
                    }
                }
            }
        }
    }
    fold_finish<VEC>(v, c, idx, epi, n);
}

inline void launch_fold_groups(const float *ws, float *c, long long cells, int groups, cudaStream_t st, Epilogue epi = Epilogue{nullptr, 0},
                               int n = 1) {
    const bool vec = cells % 4 == 0 && ((reinterpret_cast<uintptr_t>(ws) | reinterpret_cast<uintptr_t>(c)) & 15u) == 0;
    if (vec && groups > FOLD_SUB)
        fold_groups_split_kernel<<<(unsigned)((cells / 4 + 31) / 32), 32 * ((groups + FOLD_SUB - 1) / FOLD_SUB), 0, st>>>(ws, c, cells, groups, epi, n);
    else if (vec) fold_groups_kernel<4><<<(unsigned)((cells / 4 + 255) / 256), 256, 0, st>>>(ws, c, cells, groups, epi, n);
    else fold_groups_kernel<1><<<(unsigned)((cells + 255) / 256), 256, 0, st>>>(ws, c, cells, groups, epi, n);
}

// One thread per cell, whole product serial: the on-device restatement of the
// oracle, used by the self-check entry point and as the reference every tiled
// plan is compared with on the device.
__global__ void gemm_flat_kernel(const GemmArgs g) {
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (long long)g.m * g.n) return;
    const int i = (int)(idx / g.n), j = (int)(idx % g.n);
    float stack[FOLD_LEVELS];
    for (int t = 0; t < g.leaves; t++) {
        const int pb = t * g.leaf, pe = min(pb + g.leaf, g.k);
        float acc = 0.f;
        for (int p = pb; p < pe; p++) {
            const float av = (g.op == OP_TN) ? g.a[(size_t)p * g.m + i] : g.a[(size_t)i * g.k + p];
            const size_t boff = (g.op == OP_NT) ? (size_t)j * g.k + p : (size_t)p * g.n + j;
            float bv;
            if (g.wkind == W_F32) bv = static_cast<const float *>(g.b)[boff];
            else if (g.wkind == W_BF16) bv = bf16_bits_to_f32(static_cast<const unsigned short *>(g.b)[boff]);
            else {
                const float f = (g.wkind == W_INT8_EXP) ? pow2_f32(static_cast<const int *>(g.bscale)[j])
                                                        : static_cast<const float *>(g.bscale)[j];
                bv = dequant_int8_pow2(static_cast<const signed char *>(g.b)[boff], f);
            }
            acc = step_flush(ftz_bits(av), ftz_bits(bv), acc);
        }
        float v = ftz_hw(acc);
        int lvl = 0;
        for (int bits = t; bits & 1; bits >>= 1, lvl++) v = fold_add(stack[lvl], v);
        stack[lvl] = v;
    }
    float v = 0.f;
    bool have = false;
    for (int lvl = 0; lvl < FOLD_LEVELS; lvl++)
        if ((g.leaves >> lvl) & 1) {
            v = have ? fold_add(stack[lvl], v) : stack[lvl];
            have = true;
        }
    g.c[idx] = nan_canon(ftz_hw(v));
}

} // namespace b200i
