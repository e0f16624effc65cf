// The row-streaming decode plan: C[m,n] = A[m,k] . W[n,k]^T for a handful of
// activation rows (m <= 8) against a weight matrix that is read exactly once.
//
// This is the HBM-bound end of the product (a decoder's matrix-vector work and
// the lm_head at small batch), so the plan is built around the weight stream:
//   - a producer warp keeps a ring of shared-memory stages full with bulk
//     asynchronous copies (cp.async.bulk, the untiled TMA path; completion is
//     counted on an mbarrier). A stage is 8 weight rows by up to 4 KiB of k,
//     one copy per row: the copy engine's cost is per copy, so the copies are
//     as long as shared memory allows. The activations of the same k range
//     ride in the same stage. No register or issue slot of a computing warp
//     is spent on the stream;
//   - a consumer warp walks 8 rows x 4 leaves at a time: lane = (row, leaf),
//     each lane one serial p-ascending chain per activation row, which is the
//     contract's leaf partial, one lane per cell. A 128-bit read serves a
//     quarter warp, whose 8 lanes sit on 8 rows (16-byte skewed pitch: no bank
//     conflict) and one leaf (the activation word is a broadcast);
//   - the leaf partials of 64 rows meet in shared memory and every consumer
//     thread folds them in place, level by level, by the contract's
//     adjacent-pair tree;
//   - the weight is materialised on the way in (bf16: a shift; int8: the code
//     times its row's power of two, exact), exactly as the fp32 plan sees it.
// A leaf runs the bare fma first and is recomputed with the per-step flush only
// if its operands fail the admission test (see seams.cuh), the same
// deferred-flush idea the reference's CPU path uses
// (gemm/host/gemm_host_rows.mojo:29-38).
//
// Every mbarrier wait is bounded: a wait that runs out records a status word
// and the kernel winds down instead of spinning.
#pragma once
#include "gemm_tile.cuh"
#include "seams.cuh"

namespace b200i {

constexpr int DECODE_MAX_M = 8;
// Lane mapping: lane = (row, leaf). With one or two activation rows the stream is
// the cost, so a warp walks 8 rows x 4 leaves and the copies are 4 KiB long; with
// more activation rows the arithmetic is the cost, so all 32 lanes share one leaf
// (every activation read is then a single broadcast) and the copies are 1 KiB.
__host__ __device__ constexpr int dec_rw(int m) { return m <= 2 ? 8 : 32; }
constexpr int DEC_CONSUMERS = 8;             // consumer warps
constexpr int DEC_THREADS = 32 * (DEC_CONSUMERS + 1);
constexpr int DEC_FOLD_ROWS = 64;            // rows whose partials are folded together
__host__ __device__ constexpr int dec_max_chunk(int m) { return m <= 2 ? 4096 : 1024; } // bytes of one weight row per stage, at most
constexpr int DEC_X_STAGE_BYTES = 16384;     // activation bytes per stage, at most
constexpr int DEC_SMEM_LIMIT = 220 * 1024;      // one CTA per SM
constexpr int DEC_SMEM_LIMIT_PAIR = 110 * 1024; // two CTAs per SM: twice the serial chains in flight, half the ring each
constexpr unsigned DEC_SPIN_LIMIT = 1u << 22;

__device__ int g_decode_status = 0; // 0 = ok; nonzero = a bounded wait ran out (value says where)

struct DecodeLayout {
    int stages;
    int chunk_k;        // k elements of a row per stage (a multiple of the leaf size)
    int lps;            // leaves per stage
    int pitch;          // bytes between weight rows in a stage
    size_t x_bytes;     // activation bytes per stage
    size_t stage_bytes; // one ring slot: the weight rows, then the activations
    size_t part_off, stage_off, bar_off, total;
};

__host__ __device__ inline int dec_esize(int wkind) { return wkind == W_F32 ? 4 : (wkind == W_BF16 ? 2 : 1); }

__host__ __device__ inline DecodeLayout decode_layout(int m, int k, int wkind, int smem_limit = DEC_SMEM_LIMIT) {
    DecodeLayout l;
    const int es = dec_esize(wkind);
    const int leaf = (int)leaf_size(k), leaves = (int)leaf_count(k);
    const int rw = dec_rw(m);
    int chunk_k = dec_max_chunk(m) / es;
    if (chunk_k > DEC_X_STAGE_BYTES / (4 * m)) chunk_k = DEC_X_STAGE_BYTES / (4 * m);
    int lps = chunk_k / leaf;
    if (lps < 1) lps = 1;
    if (lps > leaves) lps = leaves;
    l.lps = lps;
    l.chunk_k = lps * leaf;
    l.pitch = l.chunk_k * es + 16;
    l.x_bytes = (size_t)m * l.chunk_k * 4;
    l.stage_bytes = ((size_t)rw * l.pitch + l.x_bytes + 127) / 128 * 128;
    size_t off = 0;
    l.part_off = off;
    off += (size_t)m * leaves * DEC_FOLD_ROWS * 4;
    off = (off + 127) / 128 * 128;
    l.stage_off = off;
    long long room = (long long)smem_limit - 256 - (long long)off;
    int stages = room > 0 ? (int)(room / (long long)l.stage_bytes) : 0;
    if (stages > 6) stages = 6;
    l.stages = stages;
    off += (size_t)(stages > 0 ? stages : 0) * l.stage_bytes;
    l.bar_off = off;
    off += 128;
    l.total = off;
    return l;
}

inline bool decode_plan_fits(long long m, long long n, long long k, int op, int wkind = W_F32) {
    if (op != OP_NT || m < 1 || m > DECODE_MAX_M || n < 1) return false;
    if (k % 16 != 0 || k > 131072) return false; // 16-byte rows for every storage kind; leaves of 128 (or one short leaf)
    if (k > K_LEAF_MIN && leaf_size(k) != K_LEAF_MIN) return false;
    DecodeLayout l = decode_layout((int)m, (int)k, wkind);
    return l.stages >= 2;
}

// ---- mbarrier / bulk-copy primitives ---------------------------------------------------
__device__ __forceinline__ unsigned smem_u32(const void *p) { return (unsigned)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(unsigned long long *bar, unsigned count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(unsigned long long *bar, unsigned bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(unsigned long long *bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// Bounded wait on a phase parity. Returns false when the limit ran out.
__device__ __forceinline__ bool mbar_wait(unsigned long long *bar, unsigned parity) {
    for (unsigned spin = 0; spin < DEC_SPIN_LIMIT; spin++) {
        unsigned done;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(done)
            : "r"(smem_u32(bar)), "r"(parity)
            : "memory");
        if (done) return true;
    }
    return false;
}
__device__ __forceinline__ void bulk_copy_g2s(void *dst, const void *src, unsigned bytes, unsigned long long *bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(smem_u32(dst)),
                 "l"(src), "r"(bytes), "r"(smem_u32(bar))
                 : "memory");
}
__device__ __forceinline__ void consumer_sync() { asm volatile("bar.sync 1, %0;" ::"n"(32 * DEC_CONSUMERS) : "memory"); }

// ---- one leaf of one row: the chain --------------------------------------------------------
// int8 code in byte `i` of `word ^ 0x80808080`, as the float 2^23 + (code + 128): exact by construction.
template <int I>
__device__ __forceinline__ float biased_code(unsigned word_x80) {
    return __uint_as_float(__byte_perm(word_x80, 0x4B000000u, 0x7540 + I));
}

// The weight words of one 128-bit read, materialised to float32 exactly as the
// fp32 plan would see them. QUICK (int8 kinds, factor well inside the normal
// range): code * 2^e comes out of one fma on the biased code, exact because the
// true product is representable; the general scale takes one exact subtraction
// and ONE rounding product. Otherwise the pinned spelling with the flush.
template <int WK, bool QUICK>
__device__ __forceinline__ void widen16(const uint4 raw, float factor, float nbias, float (&wv)[16]) {
    const unsigned r[4] = {raw.x, raw.y, raw.z, raw.w};
    if (WK == W_F32) {
#pragma unroll
        for (int q = 0; q < 4; q++) wv[q] = __uint_as_float(r[q]);
    } else if (WK == W_BF16) {
#pragma unroll
        for (int q = 0; q < 4; q++) {
            wv[2 * q] = __uint_as_float(r[q] << 16);
            wv[2 * q + 1] = __uint_as_float(r[q] & 0xFFFF0000u);
        }
    } else if (QUICK) {
#pragma unroll
        for (int q = 0; q < 4; q++) {
            const unsigned x = r[q] ^ 0x80808080u;
            const float b0 = biased_code<0>(x), b1 = biased_code<1>(x), b2 = biased_code<2>(x), b3 = biased_code<3>(x);
            if (WK == W_INT8_EXP) {
                wv[4 * q + 0] = __fmaf_rn(b0, factor, nbias);
                wv[4 * q + 1] = __fmaf_rn(b1, factor, nbias);
                wv[4 * q + 2] = __fmaf_rn(b2, factor, nbias);
                wv[4 * q + 3] = __fmaf_rn(b3, factor, nbias);
            } else {
                wv[4 * q + 0] = __fmul_rn(__fsub_rn(b0, 8388736.0f), factor);
                wv[4 * q + 1] = __fmul_rn(__fsub_rn(b1, 8388736.0f), factor);
                wv[4 * q + 2] = __fmul_rn(__fsub_rn(b2, 8388736.0f), factor);
                wv[4 * q + 3] = __fmul_rn(__fsub_rn(b3, 8388736.0f), factor);
            }
        }
    } else {
#pragma unroll
        for (int q = 0; q < 4; q++)
#pragma unroll
            for (int e = 0; e < 4; e++)
                wv[4 * q + e] = dequant_int8_pow2((int)(signed char)((r[q] >> (8 * e)) & 0xFFu), factor);
    }
}

// Walks `len` weights of one row (shared memory, 16-byte aligned) against
// xs[m][0..len) and advances acc[m]: one serial chain per cell, p ascending.
// FLUSH selects the per-step flush; the bare walk also folds the admission key
// of float32 / bf16 weights.
template <int WK, int M, bool FLUSH, bool QUICK, bool FULL>
__device__ __forceinline__ void leaf_chain(const unsigned char *w, const float *xs, int xstride, int len, float factor,
                                           float (&acc)[M], unsigned &wkey) {
    constexpr int EPV = WK == W_F32 ? 4 : (WK == W_BF16 ? 8 : 16); // elements per 128-bit read
    const float nbias = -8388736.0f * factor; // exact for a power-of-two factor
    const int steps = FULL ? K_LEAF_MIN : len;
#pragma unroll(FULL ? (EPV == 16 ? 2 : 4) : 1)
    for (int p0 = 0; p0 < steps; p0 += EPV) {
        float wv[16];
        widen16<WK, QUICK>(*reinterpret_cast<const uint4 *>(w + (size_t)p0 * (16 / EPV)), factor, nbias, wv);
#pragma unroll
        for (int e = 0; e < EPV; e += 4) {
            float xv[M][4];
#pragma unroll
            for (int mi = 0; mi < M; mi++) {
                const float4 t = *reinterpret_cast<const float4 *>(xs + (size_t)mi * xstride + p0 + e);
                xv[mi][0] = t.x; xv[mi][1] = t.y; xv[mi][2] = t.z; xv[mi][3] = t.w;
            }
#pragma unroll
            for (int st = 0; st < 4; st++) { // a leaf length is a multiple of 16 here, so no step is past the leaf
                float wf = wv[e + st];
                if (FLUSH) wf = ftz_bits(wf);
                else if (WK == W_F32 || WK == W_BF16) wkey = min(wkey, admit_key(wf));
#pragma unroll
                for (int mi = 0; mi < M; mi++)
                    acc[mi] = FLUSH ? step_flush(ftz_bits(xv[mi][st]), wf, acc[mi]) : step_bare(xv[mi][st], wf, acc[mi]);
            }
        }
    }
}

// Admission key of one leaf of the staged activations, folded by the lanes that
// share the leaf: they split the m x len words and combine with shuffles.
template <int M, int DEC_RW>
__device__ __forceinline__ unsigned leaf_x_key(const float *xs, int xstride, int len, int row) {
    unsigned key = 0xFFFFFFFFu;
    const int quads = len / 4;
    for (int idx = row; idx < M * quads; idx += DEC_RW) {
        const int mi = idx / quads, q = idx % quads;
        key = key4(*reinterpret_cast<const float4 *>(xs + (size_t)mi * xstride + 4 * q), key);
    }
#pragma unroll
    for (int off = 1; off < DEC_RW; off <<= 1) key = min(key, __shfl_xor_sync(0xFFFFFFFFu, key, off));
    return key;
}

template <int WK, int M>
__global__ void __launch_bounds__(DEC_THREADS, 2) decode_kernel(const GemmArgs g) {
    extern __shared__ __align__(128) unsigned char smem[];
    constexpr int DEC_RW = dec_rw(M), DEC_SUBS = 32 / DEC_RW;
    const DecodeLayout lay = decode_layout(M, g.k, WK, g.dec_smem_limit);
    float *part = reinterpret_cast<float *>(smem + lay.part_off);
    unsigned char *stage_base = smem + lay.stage_off;
    unsigned long long *full = reinterpret_cast<unsigned long long *>(smem + lay.bar_off);
    unsigned long long *empty = full + 8;
    const int nst = lay.stages, lps = lay.lps, pitch = lay.pitch, xstride = lay.chunk_k;
    const size_t stage_bytes = lay.stage_bytes;

    constexpr int ES = WK == W_F32 ? 4 : (WK == W_BF16 ? 2 : 1);
    constexpr int NCONS = 32 * DEC_CONSUMERS;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int leaves = g.leaves, leaf = g.leaf, k = g.k, n = g.n;
    const int chunks = (leaves + lps - 1) / lps;                 // stages per 8-row block
    const int tasks_per_stage = (lps + DEC_SUBS - 1) / DEC_SUBS; // a task is 8 rows x up to 4 leaves
    const size_t row_bytes = (size_t)k * ES;
    const size_t chunk_bytes = (size_t)lay.chunk_k * ES;

    // this CTA's contiguous share of the weight rows
    const int r_begin = (int)((long long)blockIdx.x * n / gridDim.x);
    const int r_end = (int)((long long)(blockIdx.x + 1) * n / gridDim.x);
    const int blocks = (r_end - r_begin + DEC_RW - 1) / DEC_RW;

    if (tid == 0) {
        for (int s = 0; s < nst; s++) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], DEC_CONSUMERS);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();

    if (warp == DEC_CONSUMERS) {
        // ---------------- producer: keep the ring full ----------------
        const unsigned char *wbase = static_cast<const unsigned char *>(g.b);
        int s_index = 0;
        bool alive = true;
        for (int b = 0; b < blocks && alive; b++) {
            const int row0 = r_begin + b * DEC_RW;
            const int valid = min(DEC_RW, r_end - row0);
            for (int c = 0; c < chunks && alive; c++, s_index++) {
                const int slot = s_index % nst;
                const unsigned round = (unsigned)(s_index / nst);
                if (round > 0) {
                    bool ok = true;
                    if (lane == 0) ok = mbar_wait(&empty[slot], (round - 1) & 1u);
                    ok = __shfl_sync(0xFFFFFFFFu, ok ? 1 : 0, 0) != 0;
                    if (!ok) {
                        if (lane == 0) atomicExch(&g_decode_status, 1);
                        alive = false;
                        break;
                    }
                }
                const size_t koff = (size_t)c * chunk_bytes;
                const unsigned bytes = (unsigned)min(chunk_bytes, row_bytes - koff);
                const unsigned xbytes = bytes / ES * 4; // the same k range of one activation row
                unsigned char *slot_base = stage_base + (size_t)slot * stage_bytes;
                if (lane == 0) mbar_expect_tx(&full[slot], bytes * (unsigned)valid + xbytes * (unsigned)M);
                __syncwarp();
                if (lane < valid)
                    bulk_copy_g2s(slot_base + (size_t)lane * pitch, wbase + (size_t)(row0 + lane) * row_bytes + koff, bytes,
                                  &full[slot]);
                if (lane < M)
                    bulk_copy_g2s(slot_base + (size_t)DEC_RW * pitch + (size_t)lane * xstride * 4,
                                  g.a + (size_t)lane * k + (size_t)c * xstride, xbytes, &full[slot]);
            }
        }
        return;
    }

    // ---------------- consumers ----------------
    // Every consumer warp waits on and releases EVERY stage in order (so no warp is
    // ever more than the ring ahead of another); the tasks of a stage (8 rows x 4
    // leaves each) go round the warps.
    const int row = lane % DEC_RW, sub = lane / DEC_RW;
    int s_index = 0, task_index = 0;
    bool alive = true;
    for (int b0 = 0; b0 < blocks; b0 += DEC_FOLD_ROWS / DEC_RW) {
        const int fold_row0 = r_begin + b0 * DEC_RW;
        const int fold_valid = min(DEC_FOLD_ROWS, r_end - fold_row0);
        for (int b = b0; b < min(b0 + DEC_FOLD_ROWS / DEC_RW, blocks); b++) {
            const int row0 = r_begin + b * DEC_RW;
            const int valid = min(DEC_RW, r_end - row0);
            const bool row_ok = row < valid;
            float factor = 1.0f;
            bool quick = true, wfast = true; // int8 kinds: the row's factor decides admission and the dequantisation spelling
            if (WK == W_INT8_EXP || WK == W_INT8_SCALE) {
                if (row_ok)
                    factor = (WK == W_INT8_EXP) ? pow2_f32(__ldg(static_cast<const int *>(g.bscale) + row0 + row))
                                                : __ldg(static_cast<const float *>(g.bscale) + row0 + row);
                const unsigned fexp = (__float_as_uint(factor) >> 23) & 0xFFu;
                wfast = fexp >= ADMIT_EXP;                               // |code * factor| >= |factor| for a nonzero code
                quick = __all_sync(0xFFFFFFFFu, fexp >= 27u && fexp <= 227u); // products stay normal and finite
            }
            for (int c = 0; c < chunks && alive; c++, s_index++) {
                const int slot = s_index % nst;
                const unsigned round = (unsigned)(s_index / nst);
                // every lane observes the completion itself: it reads what the copy engine wrote
                const bool ok = __all_sync(0xFFFFFFFFu, mbar_wait(&full[slot], round & 1u));
                if (!ok) {
                    if (lane == 0) atomicExch(&g_decode_status, 2);
                    alive = false;
                    break;
                }
                const unsigned char *slot_base = stage_base + (size_t)slot * stage_bytes;
                const float *xstage = reinterpret_cast<const float *>(slot_base + (size_t)DEC_RW * pitch);
                for (int tau = 0; tau < tasks_per_stage; tau++, task_index++) {
                    if (task_index % DEC_CONSUMERS != warp) continue;
                    const int j = tau * DEC_SUBS + sub; // this lane's leaf within the stage
                    const int t = c * lps + j;
                    const bool leaf_ok = j < lps && t < leaves;
                    const int len = leaf_ok ? min(leaf, k - t * leaf) : 0;
                    const unsigned char *w = slot_base + (size_t)row * pitch + (size_t)j * leaf * ES;
                    const float *x = xstage + (size_t)j * leaf;
                    const unsigned xkey = leaf_x_key<M, DEC_RW>(x, xstride, len, row); // len 0 reads nothing; every lane takes the shuffles
                    float acc[M];
#pragma unroll
                    for (int mi = 0; mi < M; mi++) acc[mi] = 0.f;
                    unsigned wkey = 0xFFFFFFFFu;
                    const bool all_full = __all_sync(0xFFFFFFFFu, len == K_LEAF_MIN);
                    if (quick && all_full) leaf_chain<WK, M, false, true, true>(w, x, xstride, len, factor, acc, wkey);
                    else if (quick) leaf_chain<WK, M, false, true, false>(w, x, xstride, len, factor, acc, wkey);
                    else leaf_chain<WK, M, false, false, false>(w, x, xstride, len, factor, acc, wkey);
                    // rows past the block and leaves past the stage never decide and are never stored
                    const bool admitted = !(row_ok && leaf_ok) || (wkey >= ADMIT_MIN && wfast && xkey >= ADMIT_MIN);
                    if (!__all_sync(0xFFFFFFFFu, admitted)) {
#pragma unroll
                        for (int mi = 0; mi < M; mi++) acc[mi] = 0.f;
                        leaf_chain<WK, M, true, false, false>(w, x, xstride, len, factor, acc, wkey);
                    }
                    if (leaf_ok) {
                        const int fr = (b - b0) * DEC_RW + row;
#pragma unroll
                        for (int mi = 0; mi < M; mi++) part[((size_t)mi * leaves + t) * DEC_FOLD_ROWS + fr] = ftz_hw(acc[mi]);
                    }
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(&empty[slot]);
            }
        }
        // every consumer warp reaches every barrier below, whatever happened above
        consumer_sync();
        // The fold, in place and level by level with every consumer thread: the node
        // (d, q) lives in the slot of its leftmost leaf, q * 2^d, so a pair's sum lands
        // where its left child was and an odd tail is carried by not moving at all.
        for (int d = 0; (1 << d) < leaves; d++) {
            const int step = 1 << d, width = (leaves + step - 1) >> d, pairs = width >> 1;
            for (int idx = tid; idx < M * pairs * DEC_FOLD_ROWS; idx += NCONS) {
                const int r = idx % DEC_FOLD_ROWS, q = (idx / DEC_FOLD_ROWS) % pairs, mi = idx / (DEC_FOLD_ROWS * pairs);
                float *left = part + ((size_t)mi * leaves + (size_t)q * 2 * step) * DEC_FOLD_ROWS + r;
                *left = fold_add(*left, left[(size_t)step * DEC_FOLD_ROWS]);
            }
            consumer_sync();
        }
        for (int idx = tid; idx < M * DEC_FOLD_ROWS; idx += NCONS) {
            const int r = idx % DEC_FOLD_ROWS, mi = idx / DEC_FOLD_ROWS;
            if (r < fold_valid && alive)
                g.c[(size_t)mi * n + fold_row0 + r] = nan_canon(ftz_hw(part[(size_t)mi * leaves * DEC_FOLD_ROWS + r]));
            if (r < fold_valid && alive && epilogue_on(g.epi)) epilogue_cell(g.c + (size_t)mi * n + fold_row0 + r, g.epi, fold_row0 + r);
        }
        consumer_sync();
    }
}

template <int WK>
inline int launch_decode_m(const GemmArgs &g, int grid, size_t smem, cudaStream_t st) {
#define B200I_DEC_CASE(MM)                                                                                        \
    case MM:                                                                                                      \
        cudaFuncSetAttribute(decode_kernel<WK, MM>, cudaFuncAttributeMaxDynamicSharedMemorySize, DEC_SMEM_LIMIT); \
        decode_kernel<WK, MM><<<grid, DEC_THREADS, smem, st>>>(g);                                                \
        break;
    switch (g.m) {
        B200I_DEC_CASE(1)
        B200I_DEC_CASE(2)
        B200I_DEC_CASE(3)
        B200I_DEC_CASE(4)
        B200I_DEC_CASE(5)
        B200I_DEC_CASE(6)
        B200I_DEC_CASE(7)
        B200I_DEC_CASE(8)
    default:
        return 0;
    }
#undef B200I_DEC_CASE
    return 1;
}

// Returns the number of kernels launched.
inline int launch_decode(const GemmArgs &g_in, int sms, cudaStream_t st) {
    GemmArgs g = g_in;
    // Low-bit weights at one or two activation rows are bound by the latency of the serial chains, not by the
    // stream: two CTAs per SM (a ring of at least two stages each) double the chains in flight. Float32
    // weights already run at the stream's rate with one CTA and the deeper ring.
    const DecodeLayout pair = decode_layout(g.m, g.k, g.wkind, DEC_SMEM_LIMIT_PAIR);
    const bool two = g.wkind != W_F32 && pair.stages >= 2 && (long long)g.n >= 16ll * sms;
    g.dec_smem_limit = two ? DEC_SMEM_LIMIT_PAIR : DEC_SMEM_LIMIT;
    const DecodeLayout lay = decode_layout(g.m, g.k, g.wkind, g.dec_smem_limit);
    int grid = sms * (two ? 2 : 1);
    const int max_grid = (g.n + 7) / 8; // no CTA with fewer than ~8 rows
    if (grid > max_grid) grid = max_grid;
    if (grid < 1) grid = 1;
    switch (g.wkind) {
    case W_F32: return launch_decode_m<W_F32>(g, grid, lay.total, st);
    case W_BF16: return launch_decode_m<W_BF16>(g, grid, lay.total, st);
    case W_INT8_EXP: return launch_decode_m<W_INT8_EXP>(g, grid, lay.total, st);
    default: return launch_decode_m<W_INT8_SCALE>(g, grid, lay.total, st);
    }
}

} // namespace b200i
