// The large identical-mode product on packed operands: a warp-specialised,
// bulk-copy fed version of the 128 x 128 tile plan.
//
// Numerical plan: the contract's (see gemm_tile.cuh). Execution plan for B200:
//
//   1. pack_operand_kernel rewrites each operand once per product into tile-major
//      panels P[tile][k][128]: 128 rows (or columns) of the operand side by side
//      for every k, already materialised to float32 (bf16 widened, int8
//      dequantised) and flushed, rows past the edge zero. It also writes one
//      admission flag per (tile, 16-step window): 1 when every word of the window
//      passes the admission test of seams.cuh. The pass moves (m + n) * k words,
//      against m * n * k fused multiply-adds in the product.
//   2. gemm_packed_kernel: a CTA owns a 128 x 128 output tile. In panel layout the
//      operands of a window are ONE contiguous 8 KB block each, so one elected
//      thread streams them into a ring of shared-memory stages with two
//      cp.async.bulk copies per window (completion on an mbarrier), refilling the
//      slot of the window before the one it has just finished, and the eight
//      warps walk the stages. Nothing is staged through registers, no
//      CTA-wide barrier sits in the k loop, and the admission test of a window is
//      one flag read. A consumer thread owns 8 x 8 cells as packed pairs
//      (fma.rn.f32x2), exactly the inner loop of the tile kernel.
//
// Every wait on an mbarrier is bounded; one that runs out sets the status word
// read by b200i_decode_status (4 = producer, 5 = consumer) and the kernel runs on
// to its end without the data.
#pragma once
#include "decode.cuh"
#include "gemm_tile.cuh"

namespace b200i {

constexpr int PK_TILE = 128;                        // rows of A / columns of B per panel and per CTA
constexpr int PK_STAGES = 6;                        // ring depth (three to six stages measure the same)
constexpr int PK_STAGE_FLOATS = 2 * KS * PK_TILE;   // A window then B window
constexpr int PK_CONSUMERS = 8;                     // warps (256 threads, 8 x 8 cells each)
constexpr int PK_THREADS = 32 * PK_CONSUMERS;
constexpr int PK_SMEM_BYTES = PK_STAGES * PK_STAGE_FLOATS * 4 + 2 * PK_STAGES * 8 + 16;

__host__ __device__ inline int pk_windows_per_leaf(int leaf) { return (leaf + KS - 1) / KS; }
inline size_t pk_panel_floats(long long extent, long long k) { return (size_t)((extent + PK_TILE - 1) / PK_TILE) * PK_TILE * (size_t)k; }
inline size_t pk_flag_bytes(long long extent, long long k) {
    const size_t n = (size_t)((extent + PK_TILE - 1) / PK_TILE) * (size_t)leaf_count(k) * (size_t)pk_windows_per_leaf((int)leaf_size(k));
    return (n + 255) / 256 * 256;
}
// scratch of the packed plan for one product, group nodes excluded
inline size_t pk_workspace_bytes(long long m, long long n, long long k) {
    return (pk_panel_floats(m, k) + pk_panel_floats(n, k)) * 4 + pk_flag_bytes(m, k) + pk_flag_bytes(n, k);
}

struct PackArgs {
    float *panel;
    unsigned char *flags;
    const void *x;
    const void *scale;
    int extent, k, leaf, leaves, wpl;
    int kcontig; // 1: x is [extent][k]; 0: x is [k][extent]
    int vec;     // k-contiguous, every 8-step run of a thread starts on a 16-byte (float32) / element-size * 8 boundary
};

__device__ __forceinline__ float pk_element(const void *x, const void *scale, int wkind, size_t off, int row) {
    if (wkind == W_F32) return ftz_bits(__ldg(static_cast<const float *>(x) + off));
    if (wkind == W_BF16) return ftz_bits(bf16_bits_to_f32(__ldg(static_cast<const unsigned short *>(x) + off)));
    const float f = (wkind == W_INT8_EXP) ? pow2_f32(__ldg(static_cast<const int *>(scale) + row)) : __ldg(static_cast<const float *>(scale) + row);
    return dequant_int8_pow2((int)__ldg(static_cast<const signed char *>(x) + off), f);
}

// grid (leaves, tiles); 256 threads: thread (r = tid % 128, half = tid / 128) owns row r of the tile and 8 of a
// window's 16 k-steps, so the panel is written in 512-byte runs
template <int WK>
__global__ void __launch_bounds__(256) pack_operand_kernel(const PackArgs a) {
    const int t = blockIdx.x, tile = blockIdx.y;
    const int r = threadIdx.x % PK_TILE, half = threadIdx.x / PK_TILE;
    const int row = tile * PK_TILE + r;
    const bool live = row < a.extent;
    const int kb = t * a.leaf, leaf_len = min(a.leaf, a.k - kb);
    float *panel = a.panel + (size_t)tile * (size_t)a.k * PK_TILE;
    for (int w = 0, koff = 0; koff < leaf_len; w++, koff += KS) {
        const int len = min(KS, leaf_len - koff);
        unsigned key = 0xFFFFFFFFu;
        float v[8];
        if (a.vec && live && len == KS) { // this thread's 8 k-steps are contiguous in the operand: 32, 16 or 8 bytes
            const size_t off = (size_t)row * a.k + kb + koff + half * 8;
            if (WK == W_F32) {
                const float4 lo = __ldg(reinterpret_cast<const float4 *>(static_cast<const float *>(a.x) + off));
                const float4 hi = __ldg(reinterpret_cast<const float4 *>(static_cast<const float *>(a.x) + off) + 1);
                v[0] = lo.x; v[1] = lo.y; v[2] = lo.z; v[3] = lo.w; v[4] = hi.x; v[5] = hi.y; v[6] = hi.z; v[7] = hi.w;
#pragma unroll
                for (int e = 0; e < 8; e++) v[e] = ftz_bits(v[e]);
            } else if (WK == W_BF16) {
                const uint4 w = __ldg(reinterpret_cast<const uint4 *>(static_cast<const unsigned short *>(a.x) + off));
                const unsigned ws[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
                for (int e = 0; e < 4; e++) {
                    v[2 * e] = ftz_bits(__uint_as_float(ws[e] << 16));
                    v[2 * e + 1] = ftz_bits(__uint_as_float(ws[e] & 0xFFFF0000u));
                }
            } else {
                const uint2 w = __ldg(reinterpret_cast<const uint2 *>(static_cast<const signed char *>(a.x) + off));
                const float f = (WK == W_INT8_EXP) ? pow2_f32(__ldg(static_cast<const int *>(a.scale) + row))
                                                   : __ldg(static_cast<const float *>(a.scale) + row);
#pragma unroll
                for (int e = 0; e < 8; e++) {
                    const unsigned word = e < 4 ? w.x : w.y;
                    v[e] = dequant_int8_pow2((int)(signed char)((word >> (8 * (e & 3))) & 0xFFu), f);
                }
            }
        } else {
#pragma unroll
            for (int e = 0; e < 8; e++) {
                const int kk = kb + koff + half * 8 + e;
                v[e] = 0.f;
                if (live && half * 8 + e < len)
                    v[e] = pk_element(a.x, a.scale, WK, a.kcontig ? (size_t)row * a.k + kk : (size_t)kk * a.extent + row, row);
            }
        }
#pragma unroll
        for (int e = 0; e < 8; e++) {
            if (half * 8 + e < len) {
                key = min(key, admit_key(v[e]));
                panel[(size_t)(kb + koff + half * 8 + e) * PK_TILE + r] = v[e];
            }
        }
        const int ok = __syncthreads_and(key >= ADMIT_MIN);
        if (threadIdx.x == 0) a.flags[((size_t)tile * a.leaves + t) * a.wpl + w] = (unsigned char)(ok ? 1 : 0);
    }
}

struct PackedGemmArgs {
    const float *pa, *pb;               // panels
    const unsigned char *fa, *fb;       // window flags
    float *c, *ws;
    int m, n, k, leaf, leaves, wpl;
    int group_leaves, groups, tiles_n, vec_c;
};

__global__ void __launch_bounds__(PK_THREADS, 2) gemm_packed_kernel(const PackedGemmArgs g) {
    constexpr int TM = 8, TN = 8, CELLS = TM * TN;
    extern __shared__ __align__(128) float pk_smem[];
    unsigned long long *full = reinterpret_cast<unsigned long long *>(pk_smem + PK_STAGES * PK_STAGE_FLOATS);
    unsigned long long *empty = full + PK_STAGES;

    const int tid = threadIdx.x, lane = tid & 31;
    const int tile_m = blockIdx.x / g.tiles_n, tile_n = blockIdx.x % g.tiles_n;
    const int t_first = blockIdx.y * g.group_leaves;
    const int t_end = min(t_first + g.group_leaves, g.leaves);

    if (tid == 0) {
#pragma unroll
        for (int i = 0; i < PK_STAGES; i++) {
            mbar_init(&full[i], 1);
            mbar_init(&empty[i], PK_CONSUMERS);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();

    // ---- the copy stream: thread 0 walks the same windows PK_STAGES - 1 ahead of the compute ----
    const float *pa = g.pa + (size_t)tile_m * (size_t)g.k * PK_TILE;
    const float *pb = g.pb + (size_t)tile_n * (size_t)g.k * PK_TILE;
    int pt = t_first, pkoff = 0, pissued = 0; // next window to copy
    auto issue_next = [&]() {                 // thread 0 only
        if (pt >= t_end) return;
        const int kb = pt * g.leaf, leaf_len = min(g.leaf, g.k - kb);
        const int len = min(KS, leaf_len - pkoff), slot = pissued % PK_STAGES;
        float *dst = pk_smem + slot * PK_STAGE_FLOATS;
        const unsigned bytes = (unsigned)len * PK_TILE * 4u;
        mbar_expect_tx(&full[slot], 2u * bytes);
        bulk_copy_g2s(dst, pa + (size_t)(kb + pkoff) * PK_TILE, bytes, &full[slot]);
        bulk_copy_g2s(dst + KS * PK_TILE, pb + (size_t)(kb + pkoff) * PK_TILE, bytes, &full[slot]);
        pissued++;
        pkoff += KS;
        if (pkoff >= leaf_len) { pkoff = 0; pt++; }
    };
    if (tid == 0) {
        for (int i = 0; i < PK_STAGES - 1; i++) issue_next();
    }

    const int tx = tid % 16, ty = tid / 16;
    const int wpl = g.wpl;
    const unsigned char *fa = g.fa + (size_t)tile_m * g.leaves * wpl;
    const unsigned char *fb = g.fb + (size_t)tile_n * g.leaves * wpl;

    unsigned long long acc[TM][TN / 2];
#pragma unroll
    for (int i = 0; i < TM; i++)
#pragma unroll
        for (int j = 0; j < TN / 2; j++) acc[i][j] = 0ull;
    float stack[FOLD_LEVELS][CELLS];

    auto read_operands = [&](const float *as, const float *bs, int kk, float (&av)[TM], float (&bv)[TN]) {
#pragma unroll
        for (int r = 0; r < 2; r++) {
            const float4 v = *reinterpret_cast<const float4 *>(as + kk * PK_TILE + r * 64 + ty * 4);
            av[4 * r + 0] = v.x; av[4 * r + 1] = v.y; av[4 * r + 2] = v.z; av[4 * r + 3] = v.w;
            const float4 u = *reinterpret_cast<const float4 *>(bs + kk * PK_TILE + r * 64 + tx * 4);
            bv[4 * r + 0] = u.x; bv[4 * r + 1] = u.y; bv[4 * r + 2] = u.z; bv[4 * r + 3] = u.w;
        }
    };
    auto step_fast = [&](const float *as, const float *bs, int kk) {
        float av[TM], bv[TN];
        read_operands(as, bs, kk, av, bv);
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
    auto step_slow = [&](const float *as, const float *bs, int kk) { // panel words are already flushed
        float av[TM], bv[TN];
        read_operands(as, bs, kk, av, bv);
        unsigned long long b2[TN / 2];
#pragma unroll
        for (int j = 0; j < TN / 2; j++) b2[j] = pack2(bv[2 * j], bv[2 * j + 1]);
#pragma unroll
        for (int i = 0; i < TM; i++) {
            const unsigned long long a2 = pack2(av[i], av[i]);
#pragma unroll
            for (int j = 0; j < TN / 2; j++) acc[i][j] = ftz2_hw(fma2_bare(a2, b2[j], acc[i][j]));
        }
    };
    auto unpack_cells = [&](float (&v)[CELLS], bool clear_acc) {
#pragma unroll
        for (int i = 0; i < TM; i++)
#pragma unroll
            for (int j = 0; j < TN / 2; j++) {
                float v0, v1;
                unpack2(acc[i][j], v0, v1);
                v[i * TN + 2 * j] = ftz_hw(v0);
                v[i * TN + 2 * j + 1] = ftz_hw(v1);
                if (clear_acc) acc[i][j] = 0ull;
            }
    };
    auto push_leaf = [&](int local_leaf) { // binary-counter stack, level-major (see gemm_tile.cuh)
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

    int stage = 0, window = 0;
    unsigned phase = 0;
    bool alive = true;
    for (int t = t_first; t < t_end; t++) {
        const int kb = t * g.leaf, leaf_len = min(g.leaf, g.k - kb);
        bool leaf_clean = true;
        for (int w = 0, koff = 0; koff < leaf_len; w++, koff += KS) {
            const int len = min(KS, leaf_len - koff);
            const bool admitted = (__ldg(fa + (size_t)t * wpl + w) & __ldg(fb + (size_t)t * wpl + w)) != 0;
            if (alive && !mbar_wait(&full[stage], phase)) {
                if (lane == 0) atomicExch(&g_decode_status, 5);
                alive = false;
            }
            const float *as = pk_smem + stage * PK_STAGE_FLOATS, *bs = as + KS * PK_TILE;
            if (admitted && leaf_clean && len == KS) {
#pragma unroll
                for (int kk = 0; kk < KS; kk++) step_fast(as, bs, kk);
            } else {
                leaf_clean = false;
#pragma unroll 1
                for (int kk = 0; kk < len; kk++) step_slow(as, bs, kk);
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&empty[stage]);
            if (tid == 0) {
                // the slot of the window before this one is free once all eight warps have left it; they have had a
                // whole window to do so
                if (window >= 1) {
                    const int prev = window - 1;
                    if (alive && !mbar_wait(&empty[prev % PK_STAGES], (unsigned)(prev / PK_STAGES) & 1u)) {
                        atomicExch(&g_decode_status, 4);
                        alive = false;
                    }
                }
                issue_next();
            }
            window++;
            if (++stage == PK_STAGES) { stage = 0; phase ^= 1u; }
        }
        if (t + 1 < t_end) push_leaf(t - t_first); // the group's last leaf stays in registers for the drain
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
    const int bm0 = tile_m * PK_TILE, bn0 = tile_n * PK_TILE;
#pragma unroll
    for (int i = 0; i < TM; i++) {
        const int row = bm0 + (i / 4) * 64 + ty * 4 + (i % 4);
#pragma unroll
        for (int jr = 0; jr < 2; jr++) {
            float vals[4];
#pragma unroll
            for (int e = 0; e < 4; e++) vals[e] = nan_canon(ftz_hw(v[i * TN + jr * 4 + e]));
            const int col = bn0 + jr * 64 + tx * 4;
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

} // namespace b200i
