// The row-streaming decode plan for low-bit weights at one to four activation rows.
//
// decode_kernel (decode.cuh) gives a lane one weight row and one leaf. For bf16 and int8 weights that
// plan is bound by its own instruction stream, not by HBM: with valid data already resident in the ring
// and nothing left to wait for it takes as long as the complete kernel (20 us of 21 on int8
// [11008, 4096]), at about nine warp instructions per weight. This kernel does the same arithmetic in
// fewer instructions:
//   - a lane owns one weight row and TWO adjacent leaves and walks them together: the two chains are the halves
//     of one packed fma.rn.f32x2 (lane-wise identical to two fma.rn.f32), and the two int8 codes of a step are
//     dequantised by one packed fma as well. One accumulator per cell, p ascending, as always;
//   - the activations are staged ONCE per CTA (they are the same for every weight row), interleaved by leaf pair
//     ({x[2j][p], x[2j+1][p]} side by side) so that a 128-bit read delivers two steps of ready operand pairs, and
//     their admission key is folded once per leaf instead of once per (8 rows x 4 leaves) task;
//   - the stage holds weights only, so the shared memory that frees becomes ring depth; the sixteen consumer
//     warps of the one CTA per SM are split into groups that each own two ring slots and work on different
//     stages at the same time, and no warp visits a stage it has no work in;
//   - the first three levels of the fold tree are taken in registers (one in the lane, two by shuffles), so one
//     node per eight leaves reaches shared memory.
// A task whose leaves are not all 128 long (the end of a k that is not a multiple of 128), a leaf whose operands
// fail admission and a row scale outside the range in which the one-fma dequantisation is exact fall back to
// decode.cuh's per-leaf chains (flushed, or with the pinned spelling), reading the activations from global memory.
//
// Every mbarrier wait is bounded and reports through the library's status word like decode_kernel's.
#pragma once
#include "decode.cuh"

namespace b200i {

constexpr int DP_MAX_M = 4;           // activation rows
constexpr int DP_CONSUMERS = 16;
constexpr int DP_THREADS = 32 * (DP_CONSUMERS + 1);
constexpr int DP_ROWS = 8;            // weight rows per stage
constexpr int DP_TASK_LEAVES = 8;     // leaves per warp task (4 row pairs x 8 leaves = 32 lanes)
constexpr int DP_CHUNK_BYTES = 4096;  // bytes of one weight row per stage, at most
constexpr int DP_X_SKEW = 4;          // floats between the leaf pairs of a staged activation row: the four pairs a warp reads
                                      // at once then sit in different banks and one wavefront serves all of them
constexpr int DP_X_BYTES_MAX = 98304; // staged activations, at most
constexpr int DP_SMEM_LIMIT = 220 * 1024;
constexpr int DP_FOLD_ROWS = 128;      // rows whose partials are folded together
constexpr int DP_ROWS_MAX = 4096;     // weight rows per CTA, at most (their factors live in shared memory)
__host__ __device__ inline int dp_rows_per_cta(long long n, int grid) { return (int)((n + grid - 1) / grid); }

struct PairLayout {
    int stages, lps, chunk_k, pitch, xstride; // xstride: floats between activation rows in shared memory
    size_t stage_bytes, part_off, x_off, key_off, fac_off, stage_off, bar_off, total;
};

// `rows`: the most weight rows one CTA owns (their scales are staged once, as float32 factors).
__host__ __device__ inline PairLayout pair_layout(int m, int k, int wkind, int rows) {
    PairLayout l;
    const int es = dec_esize(wkind);
    const int leaf = (int)leaf_size(k), leaves = (int)leaf_count(k);
    int lps = DP_CHUNK_BYTES / es / leaf;
    if (lps < 1) lps = 1;
    if (lps > leaves) lps = leaves;
    l.lps = lps;
    l.chunk_k = lps * leaf;
    l.pitch = l.chunk_k * es + 16;
    l.stage_bytes = ((size_t)DP_ROWS * l.pitch + 127) / 128 * 128;
    l.xstride = (2 * leaf + DP_X_SKEW) * ((leaves + 1) / 2); // leaf pairs, interleaved, a 16-byte skew between pairs
    size_t off = 0;
    l.part_off = off;
    off += (size_t)m * ((leaves + DP_TASK_LEAVES - 1) / DP_TASK_LEAVES) * DP_FOLD_ROWS * 4; // level-3 nodes of 128 rows
    l.x_off = off;
    off += ((size_t)m * l.xstride * 4 + 127) / 128 * 128;
    l.key_off = off;
    off += ((size_t)m * leaves * 4 + 127) / 128 * 128;
    l.fac_off = off;
    if (wkind != W_BF16) off += ((size_t)rows * 4 + 127) / 128 * 128;
    l.stage_off = off;
    const long long room = (long long)DP_SMEM_LIMIT - 384 - (long long)off;
    int stages = room > 0 ? (int)(room / (long long)l.stage_bytes) : 0;
    if (stages > 16) stages = 16;
    l.stages = stages;
    off += (size_t)(stages > 0 ? stages : 0) * l.stage_bytes;
    l.bar_off = off; // full[16], empty[16], the producer's stage counter
    off += 384;
    l.total = off;
    return l;
}

// Stages in work at once (one group of warps each) for a ring of `stages` slots: all the warps if the ring leaves two
// slots of look-ahead, never more than the ring.
__host__ __device__ inline int dp_groups(int stages, int tps) {
    int g = DP_CONSUMERS / tps, cap = stages - 2 > stages / 2 ? stages - 2 : stages / 2;
    return g < cap ? g : cap;
}

inline bool decode_pair_fits(long long m, long long n, long long k, int op, int wkind, int grid) {
    if (wkind == W_F32 || m > DP_MAX_M || !decode_plan_fits(m, n, k, op, wkind)) return false;
    if (n < 16ll * grid || dp_rows_per_cta(n, grid) > DP_ROWS_MAX) return false;
    const PairLayout l = pair_layout((int)m, (int)k, wkind, dp_rows_per_cta(n, grid));
    if ((size_t)m * l.xstride * 4 > (size_t)DP_X_BYTES_MAX || l.stages < 2) return false;
    // at least four warps at work: with long activation rows the ring is too short and decode_kernel does better
    const int tps = (l.lps + DP_TASK_LEAVES - 1) / DP_TASK_LEAVES;
    return dp_groups(l.stages, tps) * tps >= 4;
}

__device__ __forceinline__ void dp_consumer_sync() { asm volatile("bar.sync 1, %0;" ::"n"(32 * DP_CONSUMERS) : "memory"); }

// Walks the weights of two leaves of one row (w0, w1: shared memory, 16-byte aligned) against the interleaved
// activations xi[m][p][2] and advances the packed accumulators (low half: the first leaf, high half: the second).
// Bare steps only, 128 of them; the caller decides admission afterwards.
template <int WK, int M>
__device__ __forceinline__ void pair_chain(const unsigned char *w0, const unsigned char *w1, const float *xi, int xstride, float f,
                                           unsigned long long (&acc)[M], unsigned &wkey) {
    constexpr int EPV = WK == W_BF16 ? 8 : 16; // elements per 128-bit read
    const unsigned long long fac2 = pack2(f, f);
    const unsigned long long nb2 = pack2(-8388736.0f * f, -8388736.0f * f); // exact for power-of-two factors
    const unsigned long long unbias2 = pack2(-8388736.0f, -8388736.0f), ones2 = 0x3F8000003F800000ull, negz2 = 0x8000000080000000ull;
    uint4 na = *reinterpret_cast<const uint4 *>(w0), nb = *reinterpret_cast<const uint4 *>(w1);
#pragma unroll
    for (int p0 = 0; p0 < K_LEAF_MIN; p0 += EPV) {
        const uint4 va = na, vb = nb;
        if (p0 + EPV < K_LEAF_MIN) { // the next read is in flight while this one is walked
            na = *reinterpret_cast<const uint4 *>(w0 + (size_t)(p0 + EPV) * (16 / EPV));
            nb = *reinterpret_cast<const uint4 *>(w1 + (size_t)(p0 + EPV) * (16 / EPV));
        }
        const unsigned ra[4] = {va.x, va.y, va.z, va.w}, rb[4] = {vb.x, vb.y, vb.z, vb.w};
        unsigned long long w2[EPV];
        if (WK == W_BF16) {
#pragma unroll
            for (int q = 0; q < 4; q++) {
                const float a0 = __uint_as_float(ra[q] << 16), a1 = __uint_as_float(ra[q] & 0xFFFF0000u);
                const float b0 = __uint_as_float(rb[q] << 16), b1 = __uint_as_float(rb[q] & 0xFFFF0000u);
                wkey = min(wkey, min(min(admit_key(a0), admit_key(a1)), min(admit_key(b0), admit_key(b1))));
                w2[2 * q] = pack2(a0, b0);
                w2[2 * q + 1] = pack2(a1, b1);
            }
        } else {
#pragma unroll
            for (int q = 0; q < 4; q++) {
                const unsigned xa = ra[q] ^ 0x80808080u, xb = rb[q] ^ 0x80808080u;
                const unsigned long long b2[4] = {pack2(biased_code<0>(xa), biased_code<0>(xb)), pack2(biased_code<1>(xa), biased_code<1>(xb)),
                                                  pack2(biased_code<2>(xa), biased_code<2>(xb)), pack2(biased_code<3>(xa), biased_code<3>(xb))};
#pragma unroll
                for (int e = 0; e < 4; e++) {
                    // exponent scales: code * 2^e out of one fma on the biased code, exact. General scales: one exact
                    // subtraction, then ONE rounding product (x * f + (-0) is mul.rn's word, signed zeros included).
                    if (WK == W_INT8_EXP) w2[4 * q + e] = fma2_bare(b2[e], fac2, nb2);
                    else w2[4 * q + e] = fma2_bare(fma2_bare(b2[e], ones2, unbias2), fac2, negz2);
                }
            }
        }
#pragma unroll
        for (int e = 0; e < EPV; e += 2) {
            float4 xv[M]; // {x0[p], x1[p], x0[p+1], x1[p+1]}: two steps of operand pairs, already paired
#pragma unroll
            for (int mi = 0; mi < M; mi++) xv[mi] = *reinterpret_cast<const float4 *>(xi + (size_t)mi * xstride + 2 * (p0 + e));
#pragma unroll
            for (int mi = 0; mi < M; mi++) {
                acc[mi] = fma2_bare(pack2(xv[mi].x, xv[mi].y), w2[e], acc[mi]);
                acc[mi] = fma2_bare(pack2(xv[mi].z, xv[mi].w), w2[e + 1], acc[mi]);
            }
        }
    }
}

template <int WK, int M>
__global__ void __launch_bounds__(DP_THREADS, 1) decode_pair_kernel(const GemmArgs g) {
    extern __shared__ __align__(128) unsigned char smem[];
    const PairLayout lay = pair_layout(M, g.k, WK, dp_rows_per_cta(g.n, gridDim.x));
    float *part = reinterpret_cast<float *>(smem + lay.part_off);
    float *xs = reinterpret_cast<float *>(smem + lay.x_off);
    unsigned *xkeys = reinterpret_cast<unsigned *>(smem + lay.key_off);
    float *fac = reinterpret_cast<float *>(smem + lay.fac_off);
    unsigned char *stage_base = smem + lay.stage_off;
    unsigned long long *full = reinterpret_cast<unsigned long long *>(smem + lay.bar_off);
    unsigned long long *empty = full + 16;
    const int lps = lay.lps, pitch = lay.pitch, xstride = lay.xstride;
    const size_t stage_bytes = lay.stage_bytes;

    constexpr int ES = WK == W_BF16 ? 2 : 1;
    constexpr int NCONS = 32 * DP_CONSUMERS;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int leaves = g.leaves, leaf = g.leaf, k = g.k, n = g.n;
    const int nodes = (leaves + DP_TASK_LEAVES - 1) / DP_TASK_LEAVES; // fold-tree nodes of level 3 per cell: what reaches shared memory
    const int chunks = (leaves + lps - 1) / lps;
    const int tps = (lps + DP_TASK_LEAVES - 1) / DP_TASK_LEAVES; // warp tasks per stage = warps per group
    // Stages in work at once, one group of warps each: stage s goes to group s % groups and to ring slot s % nst. A group
    // does not see every use of a slot, and a phase-parity wait cannot tell "one phase behind" from "done"; so the
    // producer publishes how many stages it has issued, and a group looks for a stage's data only once that stage has
    // been issued: by then the slot's previous use has been consumed, so its phase is the one before the awaited one.
    const int groups = dp_groups(lay.stages, tps);
    const int nst = lay.stages;
    volatile int *issued = reinterpret_cast<volatile int *>(full + 32);
    const size_t row_bytes = (size_t)k * ES;
    const size_t chunk_bytes = (size_t)lay.chunk_k * ES;

    const int r_begin = (int)((long long)blockIdx.x * n / gridDim.x);
    const int r_end = (int)((long long)(blockIdx.x + 1) * n / gridDim.x);
    const int blocks = (r_end - r_begin + DP_ROWS - 1) / DP_ROWS;
    if (tid == 0) {
        for (int s = 0; s < nst; s++) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], tps);
        }
        *issued = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();

    if (warp == DP_CONSUMERS) {
        // ---------------- producer: keep the ring full of weight rows ----------------
        const unsigned char *wbase = static_cast<const unsigned char *>(g.b);
        int s_index = 0;
        for (int b = 0; b < blocks; b++) {
            const int row0 = r_begin + b * DP_ROWS;
            const int valid = min(DP_ROWS, r_end - row0);
            for (int c = 0; c < chunks; c++, s_index++) {
                const int slot = s_index % nst;
                const unsigned round = (unsigned)(s_index / nst);
                if (round > 0) {
                    bool ok = true;
                    if (lane == 0) ok = mbar_wait(&empty[slot], (round - 1) & 1u);
                    ok = __shfl_sync(0xFFFFFFFFu, ok ? 1 : 0, 0) != 0;
                    if (!ok) {
                        if (lane == 0) atomicExch(&g_decode_status, 1);
                        return;
                    }
                }
                const size_t koff = (size_t)c * chunk_bytes;
                const unsigned bytes = (unsigned)min(chunk_bytes, row_bytes - koff);
                unsigned char *slot_base = stage_base + (size_t)slot * stage_bytes;
                if (lane == 0) mbar_expect_tx(&full[slot], bytes * (unsigned)valid);
                __syncwarp();
                if (lane < valid)
                    bulk_copy_g2s(slot_base + (size_t)lane * pitch, wbase + (size_t)(row0 + lane) * row_bytes + koff, bytes, &full[slot]);
                __syncwarp();
                if (lane == 0) *issued = s_index + 1;
            }
        }
        return;
    }

    // ---------------- consumers ----------------
    // The activations, once: xs[m][leaf pair][p][2], and one admission key per (row, leaf). When every leaf is 128 long
    // a warp's 32 quads are exactly one leaf of one row, so the key is folded on the way in.
    const bool keys_inline = leaf == K_LEAF_MIN && k % K_LEAF_MIN == 0;
    for (int idx = tid; idx < M * (k / 4); idx += NCONS) {
        const int mi = idx / (k / 4), p = (idx - mi * (k / 4)) * 4, t = p / leaf;
        const float4 v = __ldg(reinterpret_cast<const float4 *>(g.a + (size_t)mi * k + p));
        float *dst = xs + (size_t)mi * xstride + (size_t)(t >> 1) * (2 * leaf + DP_X_SKEW) + 2 * (p - t * leaf) + (t & 1);
        dst[0] = v.x;
        dst[2] = v.y;
        dst[4] = v.z;
        dst[6] = v.w;
        if (keys_inline) {
            unsigned key = key4(v, 0xFFFFFFFFu);
#pragma unroll
            for (int off = 1; off < 32; off <<= 1) key = min(key, __shfl_xor_sync(0xFFFFFFFFu, key, off));
            if (lane == 0) xkeys[mi * leaves + t] = key;
        }
    }
    if (!keys_inline) { // keys from global memory, a warp per (row, leaf)
        for (int it = warp; it < M * leaves; it += DP_CONSUMERS) {
            const int mi = it / leaves, t = it - mi * leaves;
            const int len = min(leaf, k - t * leaf);
            unsigned key = 0xFFFFFFFFu;
            for (int q = lane; q < len / 4; q += 32) key = key4(__ldg(reinterpret_cast<const float4 *>(g.a + (size_t)mi * k + (size_t)t * leaf) + q), key);
#pragma unroll
            for (int off = 1; off < 32; off <<= 1) key = min(key, __shfl_xor_sync(0xFFFFFFFFu, key, off));
            if (lane == 0) xkeys[it] = key;
        }
    }
    // the factors of this CTA's rows, once: a global load per block of rows would sit in the path of every block
    if (WK == W_INT8_EXP || WK == W_INT8_SCALE)
        for (int idx = tid; idx < r_end - r_begin; idx += NCONS)
            fac[idx] = (WK == W_INT8_EXP) ? pow2_f32(__ldg(static_cast<const int *>(g.bscale) + r_begin + idx))
                                          : __ldg(static_cast<const float *>(g.bscale) + r_begin + idx);
    dp_consumer_sync();

    // Group q (warps q * tps ...) takes the stages s = q, q + groups, ...; warp `tw` of the group takes eight leaves of the
    // stage. A lane is (weight row, leaf pair): eight rows by four pairs.
    const int gw = warp / tps, tw = warp - gw * tps;
    const int r = lane & 7, jpl = lane >> 3;
    bool alive = true;
    for (int b0 = 0; b0 < blocks; b0 += DP_FOLD_ROWS / DP_ROWS) {
        const int fold_row0 = r_begin + b0 * DP_ROWS;
        const int fold_valid = min(DP_FOLD_ROWS, r_end - fold_row0);
        const int s_lo = b0 * chunks, s_hi = min(b0 + DP_FOLD_ROWS / DP_ROWS, blocks) * chunks;
        for (int s = s_lo + (gw - s_lo % groups + groups) % groups; gw < groups && s < s_hi && alive; s += groups) {
            const int b = s / chunks, c = s - b * chunks;
            const int slot = s % nst;
            const unsigned round = (unsigned)(s / nst);
            const int row0 = r_begin + b * DP_ROWS;
            const bool row_ok = row0 + r < r_end;
            float f = 1.0f;
            bool quick = true, fast = true; // int8 kinds: the row's factor decides admission and the dequantisation spelling
            if (WK == W_INT8_EXP || WK == W_INT8_SCALE) {
                if (row_ok) f = fac[b * DP_ROWS + r];
                const unsigned fexp = (__float_as_uint(f) >> 23) & 0xFFu;
                fast = fexp >= ADMIT_EXP;                                     // |code * factor| >= |factor| for a nonzero code
                quick = __all_sync(0xFFFFFFFFu, fexp >= 27u && fexp <= 227u); // products stay normal and finite
            }
            const int j0 = tw * DP_TASK_LEAVES + 2 * jpl; // this lane's first leaf within the stage
            const int t0 = c * lps + j0;
            const bool ok0 = j0 < lps && t0 < leaves, ok1 = ok0 && j0 + 1 < lps && t0 + 1 < leaves;
            const int len0 = ok0 ? min(leaf, k - t0 * leaf) : 0, len1 = ok1 ? min(leaf, k - (t0 + 1) * leaf) : 0;
            // every lane observes the completion itself: it reads what the copy engine wrote
            bool ok = true;
            for (unsigned spin = 0; *issued <= s; spin++)
                if (spin >= DEC_SPIN_LIMIT) {
                    ok = false;
                    break;
                }
            ok = __all_sync(0xFFFFFFFFu, ok && mbar_wait(&full[slot], round & 1u));
            if (!ok) {
                if (lane == 0) atomicExch(&g_decode_status, 2);
                alive = false;
                break;
            }
            // lanes without a leaf walk leaf 0 of their row (inside the stage) and are never stored
            const unsigned char *w0 = stage_base + (size_t)slot * stage_bytes + (size_t)r * pitch + (size_t)(ok0 ? j0 : 0) * leaf * ES;
            const unsigned char *w1 = ok1 ? w0 + (size_t)leaf * ES : w0;
            const float *xg = g.a + (size_t)(ok0 ? t0 : 0) * leaf; // the fallbacks read the activations where they came from
            float v0[M], v1[M];
            unsigned wkey = 0xFFFFFFFFu;
            // the packed walk needs every leaf of the task to be 128 long (a missing second leaf walks the first one twice)
            if (quick && __all_sync(0xFFFFFFFFu, !ok0 || (len0 == K_LEAF_MIN && (!ok1 || len1 == K_LEAF_MIN)))) {
                unsigned long long acc[M];
#pragma unroll
                for (int mi = 0; mi < M; mi++) acc[mi] = 0ull;
                pair_chain<WK, M>(w0, w1, xs + (size_t)((ok0 ? t0 : 0) >> 1) * (2 * leaf + DP_X_SKEW), xstride, f, acc, wkey);
#pragma unroll
                for (int mi = 0; mi < M; mi++) unpack2(acc[mi], v0[mi], v1[mi]);
            } else { // leaf by leaf: short leaves, or a scale outside the quick range (the pinned dequantisation)
#pragma unroll
                for (int mi = 0; mi < M; mi++) v0[mi] = v1[mi] = 0.f;
                if (quick) {
                    leaf_chain<WK, M, false, true, false>(w0, xg, k, len0, f, v0, wkey);
                    leaf_chain<WK, M, false, true, false>(w1, xg + leaf, k, len1, f, v1, wkey);
                } else {
                    leaf_chain<WK, M, false, false, false>(w0, xg, k, len0, f, v0, wkey);
                    leaf_chain<WK, M, false, false, false>(w1, xg + leaf, k, len1, f, v1, wkey);
                }
            }
            // rows past the matrix and leaves past the stage never decide and are never stored
            unsigned xkey = 0xFFFFFFFFu;
#pragma unroll
            for (int mi = 0; mi < M; mi++) {
                if (ok0) xkey = min(xkey, xkeys[mi * leaves + t0]);
                if (ok1) xkey = min(xkey, xkeys[mi * leaves + t0 + 1]);
            }
            const bool admitted = !(ok0 && row_ok) || (wkey >= ADMIT_MIN && fast && xkey >= ADMIT_MIN);
            if (!__all_sync(0xFFFFFFFFu, admitted)) {
                unsigned unused = 0;
#pragma unroll
                for (int mi = 0; mi < M; mi++) v0[mi] = v1[mi] = 0.f;
                leaf_chain<WK, M, true, false, false>(w0, xg, k, len0, f, v0, unused);
                leaf_chain<WK, M, true, false, false>(w1, xg + leaf, k, len1, f, v1, unused);
            }
            // The first three fold levels in registers: the lane's own two leaves, then the pairs 2 and 4 leaves to the
            // right by shuffle; a node whose right sibling lies past the last leaf is carried unchanged.
#pragma unroll
            for (int mi = 0; mi < M; mi++) {
                float v = ftz_hw(v0[mi]);
                if (ok1) v = fold_add(v, ftz_hw(v1[mi]));
#pragma unroll
                for (int d = 1; d < 3; d++) {
                    const float o = __shfl_xor_sync(0xFFFFFFFFu, v, 4 << d);
                    if ((jpl & ((1 << d) - 1)) == 0 && ok0 && t0 + (1 << d) < leaves) v = fold_add(v, o);
                }
                if (jpl == 0 && ok0) part[((size_t)mi * nodes + t0 / DP_TASK_LEAVES) * DP_FOLD_ROWS + (b - b0) * DP_ROWS + r] = v;
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&empty[slot]);
        }
        // every consumer warp reaches every barrier below, whatever happened above
        dp_consumer_sync();
        // The rest of the fold, in place and level by level: a node lives in the slot of its leftmost child, so a pair's sum
        // lands where its left child was and an odd tail is carried by not moving at all.
        for (int d = 0; (1 << d) < nodes; d++) {
            const int step = 1 << d, width = (nodes + step - 1) >> d, pairs = width >> 1;
            for (int idx = tid; idx < M * pairs * DP_FOLD_ROWS; idx += NCONS) {
                const int r = idx % DP_FOLD_ROWS, q = (idx / DP_FOLD_ROWS) % pairs, mi = idx / (DP_FOLD_ROWS * pairs);
                float *left = part + ((size_t)mi * nodes + (size_t)q * 2 * step) * DP_FOLD_ROWS + r;
                *left = fold_add(*left, left[(size_t)step * DP_FOLD_ROWS]);
            }
            dp_consumer_sync();
        }
        for (int idx = tid; idx < M * DP_FOLD_ROWS; idx += NCONS) {
            const int r = idx % DP_FOLD_ROWS, mi = idx / DP_FOLD_ROWS;
            if (r < fold_valid && alive) {
                g.c[(size_t)mi * n + fold_row0 + r] = nan_canon(ftz_hw(part[(size_t)mi * nodes * DP_FOLD_ROWS + r]));
                if (epilogue_on(g.epi)) epilogue_cell(g.c + (size_t)mi * n + fold_row0 + r, g.epi, fold_row0 + r);
            }
        }
        dp_consumer_sync();
    }
}

template <int WK>
inline int launch_decode_pair_m(const GemmArgs &g, int grid, size_t smem, cudaStream_t st) {
#define B200I_DP_CASE(MM)                                                                                             \
    case MM:                                                                                                          \
        cudaFuncSetAttribute(decode_pair_kernel<WK, MM>, cudaFuncAttributeMaxDynamicSharedMemorySize, DP_SMEM_LIMIT); \
        decode_pair_kernel<WK, MM><<<grid, DP_THREADS, smem, st>>>(g);                                                \
        break;
    switch (g.m) {
        B200I_DP_CASE(1)
        B200I_DP_CASE(2)
        B200I_DP_CASE(3)
        B200I_DP_CASE(4)
    default:
        return 0;
    }
#undef B200I_DP_CASE
    return 1;
}

// The decode plan's launch: the row-pair kernel where it applies, decode_kernel otherwise. Returns the number of kernels launched.
inline int launch_decode_plan(const GemmArgs &g, int sms, cudaStream_t st) {
    if (decode_pair_fits(g.m, g.n, g.k, OP_NT, g.wkind, sms)) {
        const PairLayout lay = pair_layout(g.m, g.k, g.wkind, dp_rows_per_cta(g.n, sms));
        switch (g.wkind) {
        case W_BF16: return launch_decode_pair_m<W_BF16>(g, sms, lay.total, st);
        case W_INT8_EXP: return launch_decode_pair_m<W_INT8_EXP>(g, sms, lay.total, st);
        default: return launch_decode_pair_m<W_INT8_SCALE>(g, sms, lay.total, st);
        }
    }
    return launch_decode(g, sms, st);
}

} // namespace b200i
