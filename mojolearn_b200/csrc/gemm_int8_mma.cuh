// int8i32.v1 product on the fifth-generation tensor cores: C[i][j] = ftz(f32(sum_p qa[i][p] * qb[j][p]) * 2^(ea[i] + eb[j])).
//
// This is the one profile of the path where a tensor-core MMA is contract-legal: the sum of products of int8 codes
// is an exact int32 (k <= 131072 keeps it inside 31 bits), so the order in which the hardware adds cannot move a bit
// (gemm/IDENTICAL_LOWBIT_CONTRACT.md:66-109 of the reference; its sm_80 form is gemm/checks/gemm_int8_mma.mojo:263-281,
// :545-620). The float32 products cannot use it: they round once per step.
//
// One CTA of 128 threads owns a 128 x 128 tile of C. Both operands are K-major (rows of codes), which is the layout
// tcgen05.mma.kind::i8 takes without a transpose:
//   - 128 bytes of k of the tile's 128 + 128 rows are brought into shared memory by 16-byte cp.async copies (zero
//     filled past the matrix edge and past k), straight into the canonical no-swizzle K-major form: 8 rows x 16 bytes
//     = one 128-byte core matrix; core matrices of one row group lie side by side along k (leading byte offset 128),
//     row groups follow each other (stride byte offset 1024). Two stages, so the copies of the next k-block run under
//     the MMAs of this one;
//   - one thread issues four tcgen05.mma (M 128, N 128, K 32) per stage; the accumulator is 128 lanes x 128 columns of
//     int32 in tensor memory; a tcgen05.commit per stage arrives on the mbarrier that guards the reuse of its buffer;
//   - after the last commit the four warps read their 32 lanes of the accumulator with tcgen05.ld, convert with the
//     pinned int32 -> float32 spelling, scale by the exact power of two and store.
// Every mbarrier wait is bounded; a wait that runs out records status 9, and the CTA still frees its tensor memory.
#pragma once
#include "decode.cuh" // mbarrier helpers, g_decode_status
#include "lowbit.cuh"

namespace b200i {

constexpr int I8_TILE = 128;   // rows of A and of B per CTA
constexpr int I8_KB = 128;     // bytes of k per stage
constexpr int I8_STAGES = 2;
constexpr int I8_THREADS = 128;
constexpr int I8_OPERAND_BYTES = I8_TILE * I8_KB;                  // one operand of one stage
constexpr int I8_SMEM_BYTES = I8_STAGES * 2 * I8_OPERAND_BYTES + 64; // + barriers and the tensor-memory address
constexpr unsigned I8_TMEM_COLS = 128;

// K-major, no swizzle: start address, leading (k) and stride (row group) byte offsets in 16-byte units, descriptor version 1.
__device__ __forceinline__ unsigned long long i8_smem_desc(unsigned smem_addr) {
    return (unsigned long long)((smem_addr & 0x3FFFFu) >> 4) | ((unsigned long long)(128u >> 4) << 16) |
           ((unsigned long long)(1024u >> 4) << 32) | (1ull << 46);
}
// D = S32, A = B = signed 8-bit, both K-major, N = 128, M = 128.
constexpr unsigned I8_IDESC = (2u << 4) | (1u << 7) | (1u << 10) | ((unsigned)(I8_TILE >> 3) << 17) | ((unsigned)(I8_TILE >> 4) << 24);

__device__ __forceinline__ void i8_mma(unsigned tmem_d, unsigned long long adesc, unsigned long long bdesc, unsigned accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(I8_IDESC), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void i8_commit(unsigned long long *bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void i8_cp16(void *dst, const void *src, unsigned src_bytes) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_u32(dst)), "l"(src), "r"(src_bytes) : "memory");
}

// Copies 128 bytes of k (from byte k0) of `rows` rows starting at row0 into one operand buffer. A warp instruction
// covers 8 rows x 64 bytes: whole 32-byte sectors of global memory, and four conflict-free 128-byte core matrices.
__device__ __forceinline__ void i8_load_operand(unsigned char *buf, const signed char *src, int row0, int rows_total, int k, int k0, int tid) {
#pragma unroll
    for (int it = 0; it < I8_TILE * (I8_KB / 16) / I8_THREADS; it++) { // 8 copies per thread
        const int idx = it * I8_THREADS + tid;
        const int lane = idx & 31, w = idx >> 5;          // w in 0..31
        const int r = (w >> 1) * 8 + (lane & 7);           // 16 row groups x 8 rows
        const int chunk = (w & 1) * 4 + (lane >> 3);       // 16-byte chunk of the 128 bytes: 0..7
        const int row = row0 + r, kb = k0 + chunk * 16;
        const bool in = row < rows_total && kb < k;        // k is a multiple of 16: a chunk is inside or outside as a whole
        const signed char *from = in ? src + (size_t)row * k + kb : src;
        i8_cp16(buf + ((r >> 3) * (I8_KB / 16) + chunk) * 128 + (r & 7) * 16, from, in ? 16u : 0u);
    }
}

__global__ void __launch_bounds__(I8_THREADS) gemm_int8_mma_kernel(float *__restrict__ c, const signed char *__restrict__ qa,
                                                                   const int *__restrict__ ea, const signed char *__restrict__ qb,
                                                                   const int *__restrict__ eb, int m, int n, int k) {
    extern __shared__ __align__(128) unsigned char smem[];
    unsigned char *abuf = smem, *bbuf = smem + I8_STAGES * I8_OPERAND_BYTES;
    unsigned long long *done = reinterpret_cast<unsigned long long *>(smem + I8_STAGES * 2 * I8_OPERAND_BYTES); // done[2]: stage free again; done[2]: all MMAs over
    unsigned *tmem_slot = reinterpret_cast<unsigned *>(done + 4);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int row0 = blockIdx.x * I8_TILE, col0 = blockIdx.y * I8_TILE;
    const int kt_count = (k + I8_KB - 1) / I8_KB;

    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(I8_TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    if (tid == 0) {
        mbar_init(&done[0], 1);
        mbar_init(&done[1], 1);
        mbar_init(&done[2], 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const unsigned tmem_d = *tmem_slot;

    bool alive = true;
    i8_load_operand(abuf, qa, row0, m, k, 0, tid);
    i8_load_operand(bbuf, qb, col0, n, k, 0, tid);
    asm volatile("cp.async.commit_group;" ::: "memory");
    for (int kt = 0; kt < kt_count; kt++) {
        const int buf = kt & 1;
        if (kt + 1 < kt_count) {
            const int nbuf = (kt + 1) & 1;
            // the MMAs that read this buffer were committed at step kt - 1: its ((kt - 1) / 2)-th use
            if (kt >= 1 && alive && !mbar_wait(&done[nbuf], (unsigned)(((kt - 1) >> 1) & 1))) alive = false;
            i8_load_operand(abuf + nbuf * I8_OPERAND_BYTES, qa, row0, m, k, (kt + 1) * I8_KB, tid);
            i8_load_operand(bbuf + nbuf * I8_OPERAND_BYTES, qb, col0, n, k, (kt + 1) * I8_KB, tid);
            asm volatile("cp.async.commit_group;" ::: "memory");
            asm volatile("cp.async.wait_group 1;" ::: "memory");
        } else {
            asm volatile("cp.async.wait_group 0;" ::: "memory");
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); // the copies were generic-proxy writes; the MMA reads through the async proxy
        __syncthreads();
        if (tid == 0) {
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const unsigned a0 = smem_u32(abuf + buf * I8_OPERAND_BYTES), b0 = smem_u32(bbuf + buf * I8_OPERAND_BYTES);
#pragma unroll
            for (int j = 0; j < I8_KB / 32; j++) // K = 32 per instruction: two core matrices along k
                i8_mma(tmem_d, i8_smem_desc(a0 + j * 256), i8_smem_desc(b0 + j * 256), (kt > 0 || j > 0) ? 1u : 0u);
            i8_commit(&done[buf]);
            if (kt + 1 == kt_count) i8_commit(&done[2]);
        }
    }
    if (alive && !mbar_wait(&done[2], 0u)) alive = false;
    if (!__syncthreads_and(alive ? 1 : 0)) {
        if (tid == 0) atomicExch(&g_decode_status, 9);
        alive = false;
    }
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");

    if (alive) {
        // warp w reads lanes 32 w .. 32 w + 31 of the accumulator: row = lane, 32 columns per read
        const int row = row0 + warp * 32 + lane;
        const long long ea_row = row < m ? (long long)ea[row] : 0;
#pragma unroll 1
        for (int cb = 0; cb < I8_TILE; cb += 32) {
            unsigned v[32];
            asm volatile(
                "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, %17, %18, %19, "
                "%20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
                : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]), "=r"(v[9]),
                  "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]), "=r"(v[17]), "=r"(v[18]),
                  "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]),
                  "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
                : "r"(tmem_d + ((unsigned)(warp * 32) << 16) + (unsigned)cb)
                : "memory");
            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
            if (row < m) {
#pragma unroll
                for (int j = 0; j < 32; j++) {
                    const int col = col0 + cb + j;
                    if (col < n) {
                        const long long esum = ea_row + (long long)__ldg(eb + col);
                        const int eclamped = esum > 1000 ? 1000 : (esum < -1000 ? -1000 : (int)esum);
                        c[(size_t)row * n + col] = nan_canon(ftz_bits(__fmul_rn(i32_to_f32_pinned((int)v[j]), pow2_f32(eclamped))));
                    }
                }
            }
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_d), "r"(I8_TMEM_COLS) : "memory");
}

// k a multiple of 16 and 16-byte aligned operands: every 16-byte copy is then aligned and inside one row.
inline bool gemm_int8_mma_fits(const void *qa, const void *qb, long long k) {
    return k % 16 == 0 && ((reinterpret_cast<uintptr_t>(qa) | reinterpret_cast<uintptr_t>(qb)) & 15) == 0;
}

inline void launch_gemm_int8_mma(float *c, const signed char *qa, const int *ea, const signed char *qb, const int *eb, int m, int n, int k,
                                 cudaStream_t st) {
    cudaFuncSetAttribute(gemm_int8_mma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, I8_SMEM_BYTES);
    const dim3 grid((unsigned)((m + I8_TILE - 1) / I8_TILE), (unsigned)((n + I8_TILE - 1) / I8_TILE));
    gemm_int8_mma_kernel<<<grid, I8_THREADS, I8_SMEM_BYTES, st>>>(c, qa, ea, qb, eb, m, n, k);
}

} // namespace b200i
