// The row-streaming decode plan: C[m,n] = A[m,k] . W[n,k]^T for a handful of
// activation rows (m <= 8) against a weight matrix that is read exactly once.
//
// This is the HBM-bound end of the product (a decoder's matrix-vector work and
// the lm_head at small batch), so the plan is built around the weight stream:
//   - a producer warp keeps a ring of shared-memory stages full with bulk
//     asynchronous copies (cp.async.bulk, the untiled TMA path: one 1 KiB copy
//     per weight row per stage, completion counted on an mbarrier), so tens of
//     KiB per SM are in flight at all times and no register or issue slot is
//     spent on the stream;
//   - eight consumer warps each own one LEAF of a stage: lane r walks row r's
//     128 weights of that leaf p-ascending with one accumulator per activation
//     row, which is the contract's serial chain, one lane per cell;
//   - the leaf partials of a 32-row block meet in shared memory and one thread
//     per cell folds them by the contract's adjacent-pair tree;
//   - the weight is materialised on the way in (bf16: a shift; int8: the code
//     times its row's power of two, exact), exactly as the fp32 plan would see it.
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
constexpr int DEC_ROWS = 32;                 // weight rows per block = lanes of a consumer warp
constexpr int DEC_CONSUMERS = 8;             // consumer warps
constexpr int DEC_THREADS = 32 * (DEC_CONSUMERS + 1);
constexpr int DEC_CHUNK_BYTES = 1024;        // bytes of one weight row per stage
constexpr int DEC_PITCH = DEC_CHUNK_BYTES + 16; // row pitch in a stage: 16-byte skew keeps 128-bit reads conflict free
constexpr int DEC_SMEM_LIMIT = 220 * 1024;
constexpr unsigned DEC_SPIN_LIMIT = 1u << 22;

__device__ int g_decode_status = 0; // 0 = ok; nonzero = a bounded wait ran out (value says where)

struct DecodeLayout {
    int stages;
    size_t x_bytes;     // activation bytes per stage: m rows x (leaves per stage x 128) floats
    size_t stage_bytes; // one ring slot: the weight tile, then the activation tile
    size_t part_off, stage_off, bar_off, total;
};

__host__ __device__ inline int dec_esize(int wkind) { return wkind == W_F32 ? 4 : (wkind == W_BF16 ? 2 : 1); }

__host__ __device__ inline DecodeLayout decode_layout(int m, int k, int leaves, int wkind) {
    DecodeLayout l;
    const int lps = DEC_CHUNK_BYTES / (K_LEAF_MIN * dec_esize(wkind));
    l.x_bytes = (size_t)m * lps * K_LEAF_MIN * 4;
    l.stage_bytes = (size_t)DEC_ROWS * DEC_PITCH + l.x_bytes;
    size_t off = 0;
    l.part_off = off;
    off += (size_t)m * leaves * DEC_ROWS * 4;
    off = (off + 127) / 128 * 128;
    l.stage_off = off;
    long long room = (long long)DEC_SMEM_LIMIT - 256 - (long long)off;
    int stages = room > 0 ? (int)(room / (long long)l.stage_bytes) : 0;
    if (stages > 4) stages = 4;
    l.stages = stages;
    off += (size_t)(stages > 0 ? stages : 0) * l.stage_bytes;
    l.bar_off = off;
    off += 128;
    l.total = off;
    return l;
}

inline bool decode_plan_fits(long long m, long long n, long long k, int op, int wkind = W_F32) {
    if (op != OP_NT || m < 1 || m > DECODE_MAX_M || n < 1) return false;
    if (k % 16 != 0 || k > 131072) return false; // 16-byte rows for every storage kind; leaves of 128
    if (k > K_LEAF_MIN && leaf_size(k) != K_LEAF_MIN) return false;
    DecodeLayout l = decode_layout((int)m, (int)k, (int)leaf_count(k), wkind);
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

// ---- one leaf of one row: the chain ----------------------------------------------------
// Walks `len` weights of storage kind WK starting at `w` (shared memory, 16-byte
// aligned) against xs[m][0..len) and advances acc[0..M). FLUSH selects the
// per-step flush; the bare walk also folds the admission key of the weights.
template <int WK, int M, bool FLUSH>
__device__ __forceinline__ void leaf_chain(const unsigned char *w, const float *xs, int xstride, int len, float factor,
                                           float (&acc)[M], unsigned &wkey) {
    constexpr int EPV = WK == W_F32 ? 4 : (WK == W_BF16 ? 8 : 16); // elements per 128-bit read
    for (int p0 = 0; p0 < len; p0 += EPV) {
        const uint4 raw = *reinterpret_cast<const uint4 *>(w + (size_t)p0 * (16 / EPV));
        float wv[EPV];
        if (WK == W_F32) {
            wv[0] = __uint_as_float(raw.x); wv[1] = __uint_as_float(raw.y);
            wv[2] = __uint_as_float(raw.z); wv[3] = __uint_as_float(raw.w);
        } else if (WK == W_BF16) {
            const unsigned r[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
            for (int q = 0; q < 4; q++) {
                wv[2 * q] = __uint_as_float(r[q] << 16);
                wv[2 * q + 1] = __uint_as_float(r[q] & 0xFFFF0000u);
            }
        } else {
            const unsigned r[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
            for (int q = 0; q < 4; q++)
#pragma unroll
                for (int e = 0; e < 4; e++) {
                    const int code = (int)(signed char)((r[q] >> (8 * e)) & 0xFFu);
                    wv[4 * q + e] = dequant_int8_pow2(code, factor);
                }
        }
#pragma unroll
        for (int e = 0; e < EPV; e += 4) {
            float xv[M][4];
#pragma unroll
            for (int mi = 0; mi < M; mi++) {
                const float4 t = *reinterpret_cast<const float4 *>(xs + (size_t)mi * xstride + p0 + e);
                xv[mi][0] = t.x; xv[mi][1] = t.y; xv[mi][2] = t.z; xv[mi][3] = t.w;
            }
#pragma unroll
            for (int s = 0; s < 4; s++) { // len is a multiple of 16, so no step here is past the leaf
                float wf = wv[e + s];
                if (FLUSH) wf = ftz_bits(wf);
                else if (WK == W_F32 || WK == W_BF16) wkey = min(wkey, admit_key(wf));
#pragma unroll
                for (int mi = 0; mi < M; mi++)
                    acc[mi] = FLUSH ? step_flush(ftz_bits(xv[mi][s]), wf, acc[mi]) : step_bare(xv[mi][s], wf, acc[mi]);
            }
        }
    }
}

// Admission key of one leaf of the staged activations: the lanes split the
// m x len words between them and vote.
template <int M>
__device__ __forceinline__ bool leaf_x_admitted(const float *xs, int xstride, int len, int lane) {
    unsigned key = 0xFFFFFFFFu;
    const int quads = len / 4;
    for (int idx = lane; idx < M * quads; idx += 32) {
        const int mi = idx / quads, q = idx % quads;
        key = key4(*reinterpret_cast<const float4 *>(xs + (size_t)mi * xstride + 4 * q), key);
    }
    return __all_sync(0xFFFFFFFFu, key >= ADMIT_MIN);
}

template <int WK, int M>
__global__ void __launch_bounds__(DEC_THREADS, 1) decode_kernel(const GemmArgs g) {
    extern __shared__ __align__(128) unsigned char smem[];
    const DecodeLayout lay = decode_layout(M, g.k, g.leaves, WK);
    float *part = reinterpret_cast<float *>(smem + lay.part_off);
    unsigned char *stage_base = smem + lay.stage_off;
    unsigned long long *full = reinterpret_cast<unsigned long long *>(smem + lay.bar_off);
    unsigned long long *empty = full + 4;
    const int nst = lay.stages;
    const size_t stage_bytes = lay.stage_bytes;

    constexpr int ES = WK == W_F32 ? 4 : (WK == W_BF16 ? 2 : 1);
    constexpr int LPS = DEC_CHUNK_BYTES / (K_LEAF_MIN * ES); // leaves per stage: 8, 4 or 2
    constexpr int XSTRIDE = LPS * K_LEAF_MIN;                 // floats per activation row in a stage
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int leaves = g.leaves, k = g.k, n = g.n;
    const int chunks = (leaves + LPS - 1) / LPS; // stages per row block
    const size_t row_bytes = (size_t)k * ES;

    // this CTA's contiguous share of the weight rows
    const int r_begin = (int)((long long)blockIdx.x * n / gridDim.x);
    const int r_end = (int)((long long)(blockIdx.x + 1) * n / gridDim.x);
    const int blocks = (r_end - r_begin + DEC_ROWS - 1) / DEC_ROWS;

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
            const int row0 = r_begin + b * DEC_ROWS;
            const int valid = min(DEC_ROWS, r_end - row0);
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
                const size_t koff = (size_t)c * DEC_CHUNK_BYTES;
                const unsigned bytes = (unsigned)min((size_t)DEC_CHUNK_BYTES, row_bytes - koff);
                const unsigned xbytes = bytes / ES * 4; // the same k range of one activation row
                unsigned char *slot_base = stage_base + (size_t)slot * stage_bytes;
                if (lane == 0) mbar_expect_tx(&full[slot], bytes * (unsigned)valid + xbytes * (unsigned)M);
                __syncwarp();
                if (lane < valid)
                    bulk_copy_g2s(slot_base + (size_t)lane * DEC_PITCH, wbase + (size_t)(row0 + lane) * row_bytes + koff, bytes,
                                  &full[slot]);
                if (lane < M)
                    bulk_copy_g2s(slot_base + (size_t)DEC_ROWS * DEC_PITCH + (size_t)lane * XSTRIDE * 4,
                                  g.a + (size_t)lane * k + (size_t)c * XSTRIDE, xbytes, &full[slot]);
            }
        }
        return;
    }

    // ---------------- consumers ----------------
    // Every consumer warp waits on and releases EVERY stage in order (so no warp is
    // ever more than the ring ahead of another), and computes the one leaf of the
    // stage whose index is congruent to the warp modulo the consumer count.
    int s_index = 0;
    bool alive = true;
    for (int b = 0; b < blocks; b++) {
        const int row0 = r_begin + b * DEC_ROWS;
        const int valid = min(DEC_ROWS, r_end - row0);
        const bool row_ok = lane < valid;
        float factor = 0.f;
        bool wfast = true; // int8 kinds: the row's factor decides admission
        if (WK == W_INT8_EXP || WK == W_INT8_SCALE) {
            if (row_ok)
                factor = (WK == W_INT8_EXP) ? pow2_f32(__ldg(static_cast<const int *>(g.bscale) + row0 + lane))
                                            : __ldg(static_cast<const float *>(g.bscale) + row0 + lane);
            const unsigned fexp = (__float_as_uint(factor) >> 23) & 0xFFu;
            wfast = fexp >= ADMIT_EXP; // |code * factor| >= |factor| for a nonzero code
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
            // the leaf of this stage that belongs to this warp, if any
            const int j = (warp - (c * LPS) % DEC_CONSUMERS + DEC_CONSUMERS) % DEC_CONSUMERS;
            const int t = c * LPS + j;
            if (j < LPS && t < leaves) {
                const int len = min(g.leaf, k - t * g.leaf);
                const unsigned char *slot_base = stage_base + (size_t)slot * stage_bytes;
                const unsigned char *w = slot_base + (size_t)lane * DEC_PITCH + (size_t)j * K_LEAF_MIN * ES;
                const float *x = reinterpret_cast<const float *>(slot_base + (size_t)DEC_ROWS * DEC_PITCH) + (size_t)j * K_LEAF_MIN;
                const bool xfast = leaf_x_admitted<M>(x, XSTRIDE, len, lane);
                float acc[M];
#pragma unroll
                for (int mi = 0; mi < M; mi++) acc[mi] = 0.f;
                unsigned wkey = 0xFFFFFFFFu;
                leaf_chain<WK, M, false>(w, x, XSTRIDE, len, factor, acc, wkey);
                bool admitted = (wkey >= ADMIT_MIN) && wfast && xfast;
                if (!row_ok) admitted = true;
                if (!__all_sync(0xFFFFFFFFu, admitted)) {
#pragma unroll
                    for (int mi = 0; mi < M; mi++) acc[mi] = 0.f;
                    leaf_chain<WK, M, true>(w, x, XSTRIDE, len, factor, acc, wkey);
                }
#pragma unroll
                for (int mi = 0; mi < M; mi++) part[((size_t)mi * leaves + t) * DEC_ROWS + lane] = ftz_hw(acc[mi]);
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&empty[slot]);
        }
        // every consumer warp reaches both barriers, whatever happened above
        consumer_sync();
        // fold: one thread per cell of the block
        for (int cell = tid; cell < M * DEC_ROWS; cell += 32 * DEC_CONSUMERS) {
            const int mi = cell / DEC_ROWS, r = cell % DEC_ROWS;
            if (r < valid && alive) {
                float stack[FOLD_LEVELS];
                float v = 0.f;
                for (int t = 0; t < leaves; t++) {
                    v = part[((size_t)mi * leaves + t) * DEC_ROWS + r];
                    if (t + 1 == leaves) break; // the last partial stays in a register for the drain
                    int lvl = 0;
                    for (int bits = t; bits & 1; bits >>= 1, lvl++) v = fold_add(stack[lvl], v);
                    stack[lvl] = v;
                }
                for (int lvl = 0, last = leaves - 1; lvl < FOLD_LEVELS; lvl++)
                    if ((last >> lvl) & 1) v = fold_add(stack[lvl], v);
                g.c[(size_t)mi * n + row0 + r] = nan_canon(ftz_hw(v));
            }
        }
        consumer_sync();
    }
}

template <int WK>
inline int launch_decode_m(const GemmArgs &g, int grid, size_t smem, cudaStream_t st) {
#define B200I_DEC_CASE(MM)                                                                                        \
    case MM:                                                                                                      \
        cudaFuncSetAttribute(decode_kernel<WK, MM>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);      \
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
inline int launch_decode(const GemmArgs &g, int sms, cudaStream_t st) {
    const DecodeLayout lay = decode_layout(g.m, g.k, g.leaves, g.wkind);
    int grid = sms;
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
