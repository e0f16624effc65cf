// int8i32.v1 product on the fifth-generation tensor cores: C[i][j] = ftz(f32(sum_p qa[i][p] * qb[j][p]) * 2^(ea[i] + eb[j])).
//
// This is the one profile of the path where a tensor-core MMA is contract-legal: the sum of products of int8 codes
// is an exact int32 (k <= 131072 keeps it inside 31 bits), so the order in which the hardware adds cannot move a bit
// (gemm/IDENTICAL_LOWBIT_CONTRACT.md:66-109 of the reference; its sm_80 form is gemm/checks/gemm_int8_mma.mojo:263-281,
// :545-620). The float32 products cannot use it: they round once per step.
//
// One CTA of 128 threads owns a 128 x TN tile of C (TN = 256, or 128 when 256-wide tiles would not fill the device).
// Both operands are K-major (rows of codes), which is the layout tcgen05.mma.kind::i8 takes without a transpose:
//   - 128 bytes of k of the tile's 128 + TN rows are brought into shared memory by 16-byte cp.async copies (zero
//     filled past the matrix edge and past k), straight into the canonical no-swizzle K-major form: 8 rows x 16 bytes
//     = one 128-byte core matrix; core matrices of one row group lie side by side along k (leading byte offset 128),
//     row groups follow each other (stride byte offset 1024). A ring of S stages keeps S - 1 k-blocks in flight under
//     the MMAs of the current one;
//   - one thread issues four tcgen05.mma (M 128, N TN, K 32) per stage; the accumulator is 128 lanes x TN columns of
//     int32 in tensor memory; a tcgen05.commit per stage arrives on the mbarrier that guards the reuse of its buffer;
//   - after the last commit the four warps read their 32 lanes of the accumulator with tcgen05.ld, convert with the
//     pinned int32 -> float32 spelling, scale by the exact power of two and store.
// Every mbarrier wait is bounded; a wait that runs out records status 9, and the CTA still frees its tensor memory.
#pragma once
#include "decode.cuh" // mbarrier helpers, g_decode_status
#include "lowbit.cuh"

namespace b200i {

constexpr int I8_TILE_M = 128; // rows of A per CTA = lanes of the accumulator
constexpr int I8_KB = 128;     // bytes of k per stage
constexpr int I8_THREADS = 128;
__host__ __device__ constexpr int i8_smem_bytes(int tn, int stages) { return stages * (I8_TILE_M + tn) * I8_KB + 256; } // + barriers, tensor-memory address

// K-major, no swizzle: start address, leading (k) and stride (row group) byte offsets in 16-byte units, descriptor version 1.
__device__ __forceinline__ unsigned long long i8_smem_desc(unsigned smem_addr) {
    return (unsigned long long)((smem_addr & 0x3FFFFu) >> 4) | ((unsigned long long)(128u >> 4) << 16) |
           ((unsigned long long)(1024u >> 4) << 32) | (1ull << 46);
}
// D = S32, A = B = signed 8-bit, both K-major, N = tn, M = 128.
__host__ __device__ constexpr unsigned i8_idesc(int tn) {
    return (2u << 4) | (1u << 7) | (1u << 10) | ((unsigned)(tn >> 3) << 17) | ((unsigned)(I8_TILE_M >> 4) << 24);
}

__device__ __forceinline__ void i8_mma(unsigned tmem_d, unsigned long long adesc, unsigned long long bdesc, unsigned idesc, unsigned accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void i8_commit(unsigned long long *bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void i8_cp16(void *dst, const void *src, unsigned src_bytes) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_u32(dst)), "l"(src), "r"(src_bytes) : "memory");
}

// Copies 128 bytes of k (from byte k0) of ROWS rows starting at row0 into one operand buffer. A warp instruction
// covers 8 rows x 64 bytes: whole 32-byte sectors of global memory, and four conflict-free 128-byte core matrices.
template <int ROWS>
__device__ __forceinline__ void i8_load_operand(unsigned char *buf, const signed char *src, int row0, int rows_total, int k, int k0, int tid) {
#pragma unroll
    for (int it = 0; it < ROWS * (I8_KB / 16) / I8_THREADS; it++) {
        const int idx = it * I8_THREADS + tid;
        const int lane = idx & 31, w = idx >> 5;
        const int r = (w >> 1) * 8 + (lane & 7);           // ROWS / 8 row groups x 8 rows
        const int chunk = (w & 1) * 4 + (lane >> 3);       // 16-byte chunk of the 128 bytes: 0..7
        const int row = row0 + r, kb = k0 + chunk * 16;
        const bool in = row < rows_total && kb < k;        // k is a multiple of 16: a chunk is inside or outside as a whole
        const signed char *from = in ? src + (size_t)row * k + kb : src;
        i8_cp16(buf + ((r >> 3) * (I8_KB / 16) + chunk) * 128 + (r & 7) * 16, from, in ? 16u : 0u);
    }
}

template <int TN, int S>
__global__ void __launch_bounds__(I8_THREADS) gemm_int8_mma_kernel(float *__restrict__ c, const signed char *__restrict__ qa,
                                                                   const int *__restrict__ ea, const signed char *__restrict__ qb,
                                                                   const int *__restrict__ eb, int m, int n, int k) {
    extern __shared__ __align__(128) unsigned char smem[];
    constexpr int A_BYTES = I8_TILE_M * I8_KB, B_BYTES = TN * I8_KB;
    unsigned char *abuf = smem, *bbuf = smem + S * A_BYTES;
    unsigned long long *done = reinterpret_cast<unsigned long long *>(smem + S * (A_BYTES + B_BYTES)); // done[s]: stage s free again; done[S]: all MMAs over
    unsigned *tmem_slot = reinterpret_cast<unsigned *>(done + S + 1);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int row0 = blockIdx.x * I8_TILE_M, col0 = blockIdx.y * TN;
    const int kt_count = (k + I8_KB - 1) / I8_KB;

    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"((unsigned)TN) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    if (tid == 0) {
        for (int s = 0; s <= S; s++) mbar_init(&done[s], 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const unsigned tmem_d = *tmem_slot;

    bool alive = true;
    // one commit group per k-block, empty ones included, so that "all but the newest S - 1 groups" is always "block kt landed"
    for (int s = 0; s < S - 1; s++) {
        if (s < kt_count) {
            i8_load_operand<I8_TILE_M>(abuf + s * A_BYTES, qa, row0, m, k, s * I8_KB, tid);
            i8_load_operand<TN>(bbuf + s * B_BYTES, qb, col0, n, k, s * I8_KB, tid);
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    }
    for (int kt = 0; kt < kt_count; kt++) {
        const int buf = kt % S, nxt = kt + S - 1;
        if (nxt < kt_count) {
            const int nbuf = nxt % S;
            // the buffer's previous block was kt - 1: wait for the MMAs committed then, its (nxt / S - 1)-th use
            if (nxt >= S && alive && !mbar_wait(&done[nbuf], (unsigned)((nxt / S - 1) & 1))) alive = false;
            i8_load_operand<I8_TILE_M>(abuf + nbuf * A_BYTES, qa, row0, m, k, nxt * I8_KB, tid);
            i8_load_operand<TN>(bbuf + nbuf * B_BYTES, qb, col0, n, k, nxt * I8_KB, tid);
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
        asm volatile("cp.async.wait_group %0;" ::"n"(S - 1) : "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); // the copies were generic-proxy writes; the MMA reads through the async proxy
        __syncthreads();
        if (tid == 0) {
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const unsigned a0 = smem_u32(abuf + buf * A_BYTES), b0 = smem_u32(bbuf + buf * B_BYTES);
#pragma unroll
            for (int j = 0; j < I8_KB / 32; j++) // K = 32 per instruction: two core matrices along k
                i8_mma(tmem_d, i8_smem_desc(a0 + j * 256), i8_smem_desc(b0 + j * 256), i8_idesc(TN), (kt > 0 || j > 0) ? 1u : 0u);
            i8_commit(&done[buf]);
            if (kt + 1 == kt_count) i8_commit(&done[S]);
        }
    }
    if (alive && !mbar_wait(&done[S], 0u)) alive = false;
    if (!__syncthreads_and(alive ? 1 : 0)) {
        if (tid == 0) atomicExch(&g_decode_status, 9);
        alive = false;
    }
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");

    if (alive) {
        // Warp w reads lanes 32 w .. 32 w + 31 of the accumulator, 32 columns per read: a thread then holds 32 cells of ONE
        // row, which would store as 32 scattered sectors per instruction. The block is turned through shared memory (the
        // operand buffers are free now; 33-word pitch, no bank conflicts either way) so that a thread owns one column of 32
        // rows and every store instruction writes 128 contiguous bytes of a row.
        unsigned *turn = reinterpret_cast<unsigned *>(smem) + warp * (32 * 33);
        const int rbase = row0 + warp * 32;
        const int ea_mine = rbase + lane < m ? ea[rbase + lane] : 0;
#pragma unroll 1
        for (int cb = 0; cb < TN; cb += 32) {
            if (col0 + cb >= n) break; // uniform over the CTA
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
#pragma unroll
            for (int j = 0; j < 32; j++) turn[lane * 33 + j] = v[j];
            __syncwarp();
            const int col = col0 + cb + lane;
            const long long eb_mine = col < n ? (long long)__ldg(eb + col) : 0;
#pragma unroll 4
            for (int rr = 0; rr < 32; rr++) {
                const long long esum = (long long)__shfl_sync(0xFFFFFFFFu, ea_mine, rr) + eb_mine;
                const int eclamped = esum > 1000 ? 1000 : (esum < -1000 ? -1000 : (int)esum);
                if (rbase + rr < m && col < n)
                    c[(size_t)(rbase + rr) * n + col] = nan_canon(ftz_bits(__fmul_rn(i32_to_f32_pinned((int)turn[rr * 33 + lane]), pow2_f32(eclamped))));
            }
            __syncwarp();
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_d), "r"((unsigned)TN) : "memory");
}

// k a multiple of 16 and 16-byte aligned operands: every 16-byte copy is then aligned and inside one row.
inline bool gemm_int8_mma_fits(const void *qa, const void *qb, long long m, long long n, long long k) {
    return k % 16 == 0 && ((reinterpret_cast<uintptr_t>(qa) | reinterpret_cast<uintptr_t>(qb)) & 15) == 0 &&
           (m + I8_TILE_M - 1) / I8_TILE_M <= 0x7FFFFFFFll && (n + 127) / 128 <= 65535;
}

template <int TN, int S>
inline void launch_gemm_int8_mma_as(float *c, const signed char *qa, const int *ea, const signed char *qb, const int *eb, int m, int n, int k,
                                    cudaStream_t st) {
    cudaFuncSetAttribute(gemm_int8_mma_kernel<TN, S>, cudaFuncAttributeMaxDynamicSharedMemorySize, i8_smem_bytes(TN, S));
    const dim3 grid((unsigned)((m + I8_TILE_M - 1) / I8_TILE_M), (unsigned)((n + TN - 1) / TN));
    gemm_int8_mma_kernel<TN, S><<<grid, I8_THREADS, i8_smem_bytes(TN, S), st>>>(c, qa, ea, qb, eb, m, n, k);
}

inline void launch_gemm_int8_mma(float *c, const signed char *qa, const int *ea, const signed char *qb, const int *eb, int m, int n, int k,
                                 int sms, cudaStream_t st) {
    // 256-wide tiles (two CTAs per SM) read a third fewer operand bytes per multiply-add and measure 15 to 25 % faster on
    // large products; they are taken when there are enough of them to fill the device twice, 128-wide ones (three CTAs
    // per SM) otherwise. More stages measured slower in every shape tried: what hides a CTA's copy, MMA and store phases
    // is the other CTAs of its SM, and a deeper ring leaves room for fewer of them.
    const long long wide = (long long)((m + I8_TILE_M - 1) / I8_TILE_M) * ((n + 255) / 256);
    if (wide >= 2ll * sms) launch_gemm_int8_mma_as<256, 2>(c, qa, ea, qb, eb, m, n, k, st);
    else launch_gemm_int8_mma_as<128, 2>(c, qa, ea, qb, eb, m, n, k, st);
}

} // namespace b200i
