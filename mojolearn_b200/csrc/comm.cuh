// Store-side fan-out of finished output columns to the other GPUs of one node.
//
// The multi-device rule of the reference is "copies only, never an order"
// (training/byte_lm_parallel.mojo:2-8, core/multi_gpu.mojo:46-50 of the reference): a rank
// computes its output columns with the full contraction and the ranks exchange finished
// float32 words. Here that exchange is one small kernel per gather instead of a library
// collective. The rank that owns a column slice [m, w] writes every word of it, paired with
// the current epoch number, into a receive area inside every other rank's exchange buffer
// (one 64-bit scalar store, which arrives whole: the word and its tag can never be seen apart), and
// copies the slice into its own gathered matrix [m, world * w]. The same kernel then reads
// the receive areas the other ranks fill in ITS buffer, waits for each word's tag to show the
// current epoch, and places the word in the gathered matrix. No fence and no separate flag:
// the critical path is one NVLink write flight. Peer memory is touched by plain st.global
// only; all loads are local; nothing here is a bulk or tensor copy.
//
// A rank's exchange buffer is one allocation that every peer maps:
//   u64 area[site][src rank][m * w]       (word, epoch tag) pairs, at caller-chosen byte offsets
// A "site" is one gather of a model step; an "epoch" is one step (a device counter that the
// caller advances once per step with comm_advance_kernel, so that a replayed CUDA graph
// counts by itself). Tags only grow, and a buffer starts as zeros, so a stale pair can never
// pass for a fresh one. Reuse of a site's area in the next epoch is safe when a step has at
// least two sites: a rank can only write site i of epoch t+1 after it finished site i-1 of
// epoch t+1 (or the last site of epoch t, for i = 0), which needed every rank's words for that
// site, and a rank sends those only after its own kernel for site i of epoch t, the only
// reader of that area, has finished (stream order). The caller keeps site 0 in a region no
// other site uses, which covers i = 0 when the shapes change between steps.
//
// Every wait is bounded (wall-clock nanoseconds on the GPU's global timer); a wait that runs
// out records status 8 in the library's status word and the thread gives up its remaining words.
#pragma once
#include <cuda_runtime.h>

#include "decode.cuh"    // g_decode_status
#include "gemm_tile.cuh" // fold_push, FOLD_SUB, MAX_GROUPS and the store epilogue

namespace b200i {

constexpr int COMM_MAX_WORLD = 8;
constexpr int COMM_THREADS = 256;
enum { COMM_SEND_RECV = 0, COMM_SEND = 1, COMM_RECV = 2 };

struct CommPeers {
    unsigned char *base[COMM_MAX_WORLD]; // every rank's exchange buffer as mapped into this process (own at [rank])
};

__device__ __forceinline__ unsigned long long comm_now_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
// A (word, tag) pair travels as ONE 64-bit scalar: a vector access is a set of element accesses, and only an
// element (here 64 bits) is guaranteed to arrive whole. The two-pair forms move two such elements.
__device__ __forceinline__ unsigned long long comm_pair(unsigned word, unsigned tag) { return ((unsigned long long)tag << 32) | word; }
__device__ __forceinline__ void comm_poll2(const void *p, unsigned long long &a, unsigned long long &b) {
    asm volatile("ld.volatile.global.v2.u64 {%0, %1}, [%2];" : "=l"(a), "=l"(b) : "l"(p) : "memory");
}
__device__ __forceinline__ unsigned long long comm_poll1(const void *p) {
    unsigned long long v;
    asm volatile("ld.volatile.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void comm_put2(void *p, unsigned long long a, unsigned long long b) {
    asm volatile("st.volatile.global.v2.u64 [%0], {%1, %2};" ::"l"(p), "l"(a), "l"(b) : "memory");
}
__device__ __forceinline__ void comm_put1(void *p, unsigned long long v) {
    asm volatile("st.volatile.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}

__global__ void comm_advance_kernel(int *epoch_word) { *epoch_word += 1; }

// out[m, world * w] (row pitch out_ld) <- this rank's src[m, w] (row pitch src_ld) and every peer's slice.
// `area` = byte offset of the site's receive areas in every exchange buffer. PAIR: two words per thread and
// step (w even, pitches even, 8-byte aligned pointers).
template <bool PAIR>
__global__ void __launch_bounds__(COMM_THREADS)
comm_gather_kernel(CommPeers peers, const int *epoch_word, const float *__restrict__ src, long long src_ld, float *__restrict__ out,
                   long long out_ld, long long area, int m, int w, int world, int rank, int mode, unsigned long long wait_ns) {
    const unsigned e = (unsigned)*epoch_word;
    constexpr int V = PAIR ? 2 : 1;
    const int wv = w / V;
    const long long items = (long long)m * wv, count = (long long)m * w; // words of one rank's slice
    const long long stride = (long long)gridDim.x * COMM_THREADS, i0 = (long long)blockIdx.x * COMM_THREADS + threadIdx.x;
    if (mode != COMM_RECV) {
        for (long long i = i0; i < items; i += stride) {
            const long long r = i / wv;
            const int c = (int)(i - r * wv) * V;
            const long long at = r * w + c; // index inside the slice
            if (PAIR) {
                const float2 v = *reinterpret_cast<const float2 *>(src + r * src_ld + c);
                *reinterpret_cast<float2 *>(out + r * out_ld + (long long)rank * w + c) = v;
                const unsigned long long p0 = comm_pair(__float_as_uint(v.x), e), p1 = comm_pair(__float_as_uint(v.y), e);
                for (int j = 1; j < world; j++) { // the peers starting after this rank: the links load evenly
                    const int p = rank + j < world ? rank + j : rank + j - world;
                    comm_put2(peers.base[p] + area + ((long long)rank * count + at) * 8, p0, p1);
                }
            } else {
                const float v = src[r * src_ld + c];
                out[r * out_ld + (long long)rank * w + c] = v;
                for (int j = 1; j < world; j++) {
                    const int p = rank + j < world ? rank + j : rank + j - world;
                    comm_put1(peers.base[p] + area + ((long long)rank * count + at) * 8, comm_pair(__float_as_uint(v), e));
                }
            }
        }
    }
    if (mode == COMM_SEND) return;
    const unsigned long long t0 = comm_now_ns();
    bool alive = true;
    const unsigned char *mine = peers.base[rank] + area;
    for (int j = 1; j < world && alive; j++) {
        const int p = rank + j < world ? rank + j : rank + j - world;
        for (long long i = i0; i < items && alive; i += stride) {
            const long long r = i / wv;
            const int c = (int)(i - r * wv) * V;
            const long long at = r * w + c;
            unsigned spins = 0;
            if (PAIR) {
                const unsigned char *q = mine + ((long long)p * count + at) * 8;
                unsigned long long a, b;
                comm_poll2(q, a, b);
                while ((unsigned)(a >> 32) != e || (unsigned)(b >> 32) != e) {
                    if ((++spins & 63u) == 0u && comm_now_ns() - t0 > wait_ns) { alive = false; break; }
                    comm_poll2(q, a, b);
                }
                if (alive) *reinterpret_cast<float2 *>(out + r * out_ld + (long long)p * w + c) = make_float2(__uint_as_float((unsigned)a), __uint_as_float((unsigned)b));
            } else {
                const unsigned char *q = mine + ((long long)p * count + at) * 8;
                unsigned long long v = comm_poll1(q);
                while ((unsigned)(v >> 32) != e) {
                    if ((++spins & 63u) == 0u && comm_now_ns() - t0 > wait_ns) { alive = false; break; }
                    v = comm_poll1(q);
                }
                if (alive) out[r * out_ld + (long long)p * w + c] = __uint_as_float((unsigned)v);
            }
        }
    }
    if (!alive) atomicExch(&g_decode_status, 8);
}

// The same gather for a slice that is still a set of leaf-group nodes: ws[groups][m * n] as a split product leaves
// them. The kernel folds the nodes exactly as fold_groups_split_kernel does (blocks of eight groups per warp, the
// block roots three levels up by warp 0), finishes the cells (canonical NaN, bias and activation, or the gated pair
// store that halves the width), writes them to its own columns of `out` and to every peer, and then receives the
// peers' columns. One launch instead of a fold launch plus a gather launch after every sharded product of a decode
// step, and the finished slice is never written to memory on its own. n a multiple of 4; a thread owns four
// consecutive cells of one row.
__global__ void __launch_bounds__(32 * MAX_GROUPS / FOLD_SUB)
comm_fold_gather_kernel(CommPeers peers, const int *epoch_word, const float *__restrict__ ws, int groups, Epilogue epi, float *__restrict__ out,
                        long long out_ld, long long area, int m, int n, int world, int rank, int mode, unsigned long long wait_ns) {
    __shared__ float4 roots[MAX_GROUPS / FOLD_SUB][32];
    const unsigned e = (unsigned)*epoch_word;
    const bool gated = epilogue_pairs(epi);
    const int w = gated ? n / 2 : n; // width of the finished slice
    const long long cells = (long long)m * n, count = (long long)m * w;
    const int lane = threadIdx.x & 31, sub = threadIdx.x >> 5;
    const int subs = (groups + FOLD_SUB - 1) / FOLD_SUB;
    const long long idx = ((long long)blockIdx.x * 32 + lane) * 4;
    const bool live = idx < cells;
    const int g0 = sub * FOLD_SUB, gcount = min(FOLD_SUB, groups - g0);
    float v[4] = {0.f, 0.f, 0.f, 0.f};
    if (live) {
        float4 x[FOLD_SUB];
#pragma unroll
        for (int j = 0; j < FOLD_SUB; j++)
            if (j < gcount) x[j] = __ldcg(reinterpret_cast<const float4 *>(ws + (size_t)(g0 + j) * (size_t)cells + idx));
        float stack[3][4];
#pragma unroll
        for (int j = 0; j < FOLD_SUB; j++) {
            if (j >= gcount) break;
            v[0] = x[j].x; v[1] = x[j].y; v[2] = x[j].z; v[3] = x[j].w;
            fold_push<4, 3>(stack, v, j, gcount - 1);
        }
        roots[sub][lane] = make_float4(v[0], v[1], v[2], v[3]);
    }
    __syncthreads();
    if (sub == 0 && live) {
        float stack[3][4];
        for (int s2 = 0; s2 < subs; s2++) {
            const float4 t = roots[s2][lane];
            v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
            fold_push<4, 3>(stack, v, s2, subs - 1);
        }
        const long long r = idx / n, col = idx - r * n;
        float f[4];
        int nf;
        long long c0; // first column of this thread's finished words inside the slice
        if (gated) {
            f[0] = epilogue_pair_apply(nan_canon(ftz_hw(v[0])), nan_canon(ftz_hw(v[1])), epi.bias, epi.act, col / 2);
            f[1] = epilogue_pair_apply(nan_canon(ftz_hw(v[2])), nan_canon(ftz_hw(v[3])), epi.bias, epi.act, col / 2 + 1);
            nf = 2; c0 = col / 2;
        } else {
#pragma unroll
            for (int q = 0; q < 4; q++) {
                f[q] = nan_canon(ftz_hw(v[q]));
                if (epilogue_on(epi)) f[q] = epilogue_apply(f[q], epi.bias, epi.act, col + q);
            }
            nf = 4; c0 = col;
        }
        float *own = out + r * out_ld + (long long)rank * w + c0;
        *reinterpret_cast<float2 *>(own) = make_float2(f[0], f[1]);
        if (nf == 4) *reinterpret_cast<float2 *>(own + 2) = make_float2(f[2], f[3]);
        const long long at = r * w + c0;
        for (int j = 1; j < world; j++) {
            const int p = rank + j < world ? rank + j : rank + j - world;
            unsigned char *q = peers.base[p] + area + ((long long)rank * count + at) * 8;
            comm_put2(q, comm_pair(__float_as_uint(f[0]), e), comm_pair(__float_as_uint(f[1]), e));
            if (nf == 4) comm_put2(q + 16, comm_pair(__float_as_uint(f[2]), e), comm_pair(__float_as_uint(f[3]), e));
        }
    }
    if (mode == COMM_SEND) return;
    // receive: two words per thread and step over the whole grid, as comm_gather_kernel<true> does
    const int wv = w / 2;
    const long long items = (long long)m * wv;
    const long long stride = (long long)gridDim.x * blockDim.x, i0 = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    const unsigned long long t0 = comm_now_ns();
    bool alive = true;
    const unsigned char *mine = peers.base[rank] + area;
    for (int j = 1; j < world && alive; j++) {
        const int p = rank + j < world ? rank + j : rank + j - world;
        for (long long i = i0; i < items && alive; i += stride) {
            const long long r = i / wv;
            const int c = (int)(i - r * wv) * 2;
            const unsigned char *q = mine + ((long long)p * count + r * w + c) * 8;
            unsigned spins = 0;
            unsigned long long a, b;
            comm_poll2(q, a, b);
            while ((unsigned)(a >> 32) != e || (unsigned)(b >> 32) != e) {
                if ((++spins & 63u) == 0u && comm_now_ns() - t0 > wait_ns) { alive = false; break; }
                comm_poll2(q, a, b);
            }
            if (alive) *reinterpret_cast<float2 *>(out + r * out_ld + (long long)p * w + c) = make_float2(__uint_as_float((unsigned)a), __uint_as_float((unsigned)b));
        }
    }
    if (!alive) atomicExch(&g_decode_status, 8);
}

} // namespace b200i
