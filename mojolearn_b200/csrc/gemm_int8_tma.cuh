// The int8i32.v1 product as a persistent, warp-specialised tensor-core kernel.
//
// gemm_int8_mma.cuh moves its operand tiles with per-thread cp.async copies and a CTA barrier per 128 bytes of k, and
// that is what bounds it (tensor pipe 12 % busy, long-scoreboard stalls). Here the tile traffic is taken off the threads:
//   - warp 0, one lane: the producer. Two tensor-map bulk copies (cp.async.bulk.tensor.2d; every CTA fetches its own tiles) per k-block bring
//     128 rows of A and 256 rows of B, 128 bytes of k each, into a ring of four 48 KB stages in the 128-byte swizzled
//     K-major layout; edges and the k tail are zero-filled by the copy engine; completion is counted on the stage's mbarrier;
//   - warp 1, one lane: the MMA issuer. Four tcgen05.mma.kind::i8 (M 128, N 256, K 32) per stage, the shared-memory
//     descriptor stepped 32 bytes along k inside the swizzle atom; a tcgen05.commit hands the stage back to the producer and,
//     after a tile's last k-block, hands the accumulator to the store warps;
//   - warps 2 to 9: the store (two warps per quarter of the accumulator's lanes, half the columns each). Two accumulators of 256 columns fill the 512 columns of tensor memory, so a tile's conversion
//     and store (the same turned, coalesced store as gemm_int8_mma_kernel's) run under the next tile's MMAs.
// One CTA per SM walks tiles blockIdx.x, blockIdx.x + gridDim.x, ... Every wait is bounded (status 9).
#pragma once
#include <cuda.h>

#include "gemm_int8_mma.cuh"

namespace b200i {

constexpr int T8_BM = 128, T8_BN = 256, T8_BK = 128, T8_STAGES = 4;
constexpr int T8_STORE_WARPS = 8, T8_THREADS = 32 * (2 + T8_STORE_WARPS);
constexpr int T8_A_BYTES = T8_BM * T8_BK, T8_B_BYTES = T8_BN * T8_BK, T8_STAGE_BYTES = T8_A_BYTES + T8_B_BYTES;
constexpr int T8_TURN_BYTES = T8_STORE_WARPS * 32 * 33 * 4;
constexpr int T8_SMEM_BYTES = 1024 + T8_STAGES * T8_STAGE_BYTES + T8_TURN_BYTES + 256; // 1024: room to align the ring
constexpr unsigned T8_TMEM_COLS = 512;

// K-major, 128-byte swizzle: rows of 128 bytes, groups of eight rows 1024 bytes apart; descriptor version 1.
__device__ __forceinline__ unsigned long long t8_smem_desc(unsigned smem_addr) {
    return (unsigned long long)((smem_addr & 0x3FFFFu) >> 4) | (1ull << 16) | ((unsigned long long)(1024u >> 4) << 32) | (1ull << 46) |
           (2ull << 61);
}
__device__ __forceinline__ void t8_tma_load(void *dst, const CUtensorMap *map, unsigned long long *bar, int c0, int c1) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::"r"(smem_u32(dst)),
                 "l"(reinterpret_cast<unsigned long long>(map)), "r"(smem_u32(bar)), "r"(c0), "r"(c1)
                 : "memory");
}

__global__ void __launch_bounds__(T8_THREADS, 1) gemm_int8_tma_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                                                                      float *__restrict__ c, const int *__restrict__ ea, const int *__restrict__ eb,
                                                                      int m, int n, int k, int tiles_n, int tiles) {
    extern __shared__ __align__(128) unsigned char smem[];
    unsigned char *ring = smem + ((1024u - (smem_u32(smem) & 1023u)) & 1023u); // the swizzle atom wants 1024-byte aligned tiles
    unsigned *turn_all = reinterpret_cast<unsigned *>(ring + T8_STAGES * T8_STAGE_BYTES);
    unsigned long long *full = reinterpret_cast<unsigned long long *>(ring + T8_STAGES * T8_STAGE_BYTES + T8_TURN_BYTES);
    unsigned long long *empty = full + T8_STAGES, *tfull = empty + T8_STAGES, *tempty = tfull + 2;
    unsigned *tmem_slot = reinterpret_cast<unsigned *>(tempty + 2);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int kt_count = (k + T8_BK - 1) / T8_BK;

    if (tid == 0) {
        for (int s = 0; s < T8_STAGES; s++) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], 1);
        }
        for (int a = 0; a < 2; a++) {
            mbar_init(&tfull[a], 1);
            mbar_init(&tempty[a], T8_STORE_WARPS);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(T8_TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const unsigned tmem = *tmem_slot;

    if (warp == 0) {
        if (lane == 0) { // ---------------- producer ----------------
            int it = 0;
            bool alive = true;
            for (int tile = blockIdx.x; tile < tiles && alive; tile += gridDim.x) {
                const int tm = tile / tiles_n, tn = tile - tm * tiles_n;
                for (int kt = 0; kt < kt_count; kt++, it++) {
                    const int s = it % T8_STAGES;
                    const unsigned ph = (unsigned)(it / T8_STAGES) & 1u;
                    if (!mbar_wait(&empty[s], ph ^ 1u)) { // a fresh barrier counts as released
                        atomicExch(&g_decode_status, 9);
                        alive = false;
                        break;
                    }
                    unsigned char *st = ring + s * T8_STAGE_BYTES;
                    mbar_expect_tx(&full[s], (unsigned)T8_STAGE_BYTES);
                    t8_tma_load(st, &map_a, &full[s], kt * T8_BK, tm * T8_BM);
                    t8_tma_load(st + T8_A_BYTES, &map_b, &full[s], kt * T8_BK, tn * T8_BN);
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) { // ---------------- MMA issuer ----------------
            int it = 0, ti = 0;
            bool alive = true;
            for (int tile = blockIdx.x; tile < tiles && alive; tile += gridDim.x, ti++) {
                const int acc = ti & 1;
                const unsigned aph = (unsigned)(ti >> 1) & 1u;
                if (!mbar_wait(&tempty[acc], aph ^ 1u)) {
                    atomicExch(&g_decode_status, 9);
                    break;
                }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const unsigned d = tmem + (unsigned)(acc * T8_BN);
                for (int kt = 0; kt < kt_count; kt++, it++) {
                    const int s = it % T8_STAGES;
                    const unsigned ph = (unsigned)(it / T8_STAGES) & 1u;
                    if (!mbar_wait(&full[s], ph)) {
                        atomicExch(&g_decode_status, 9);
                        alive = false;
                        break;
                    }
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const unsigned a0 = smem_u32(ring + s * T8_STAGE_BYTES), b0 = a0 + T8_A_BYTES;
#pragma unroll
                    for (int j = 0; j < T8_BK / 32; j++)
                        i8_mma(d, t8_smem_desc(a0 + j * 32), t8_smem_desc(b0 + j * 32), i8_idesc(T8_BN), (kt > 0 || j > 0) ? 1u : 0u);
                    i8_commit(&empty[s]); // the stage is free when these MMAs have read it
                }
                if (alive) i8_commit(&tfull[acc]); // the accumulator is whole when every MMA of the tile is done
            }
        }
    } else { // ---------------- store warps ----------------
        // a warp may read the quarter (warp % 4) of the accumulator's 128 lanes; the two warps of a quarter split the columns
        const int q = warp & 3, half = (warp - 2) >> 2;
        unsigned *turn = turn_all + (warp - 2) * (32 * 33);
        int ti = 0;
        for (int tile = blockIdx.x; tile < tiles; tile += gridDim.x, ti++) {
            const int tm = tile / tiles_n, tn = tile - tm * tiles_n;
            const int acc = ti & 1;
            const unsigned aph = (unsigned)(ti >> 1) & 1u;
            if (!__all_sync(0xFFFFFFFFu, mbar_wait(&tfull[acc], aph))) {
                if (lane == 0) atomicExch(&g_decode_status, 9);
                break;
            }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const int rbase = tm * T8_BM + q * 32, col0 = tn * T8_BN;
            const int ea_mine = rbase + lane < m ? ea[rbase + lane] : 0;
#pragma unroll 1
            for (int cb = half * (T8_BN / 2); cb < (half + 1) * (T8_BN / 2); cb += 32) {
                if (col0 + cb >= n) break; // uniform over the warp
                unsigned v[32];
                asm volatile(
                    "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, %17, %18, %19, "
                    "%20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
                    : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]), "=r"(v[9]),
                      "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]), "=r"(v[17]), "=r"(v[18]),
                      "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]),
                      "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
                    : "r"(tmem + ((unsigned)(q * 32) << 16) + (unsigned)(acc * T8_BN + cb))
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
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(&tempty[acc]); // the MMA issuer may overwrite this accumulator
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 1) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(T8_TMEM_COLS) : "memory");
}

// ---- host side: tensor maps through the driver entry point (no link against the driver library) ----
typedef CUresult (*T8EncodeFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *, const cuuint32_t *,
                               const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
inline T8EncodeFn t8_encode_fn() {
    static T8EncodeFn fn = [] {
        void *p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess) p = nullptr;
        return reinterpret_cast<T8EncodeFn>(p);
    }();
    return fn;
}
// rows x k bytes, row-major; a box of box_rows rows x 128 bytes, 128-byte swizzle, zero fill outside
inline bool t8_make_map(CUtensorMap *map, const void *base, long long rows, long long k, int box_rows) {
    T8EncodeFn fn = t8_encode_fn();
    if (!fn) return false;
    const cuuint64_t dims[2] = {(cuuint64_t)k, (cuuint64_t)rows}, strides[1] = {(cuuint64_t)k};
    const cuuint32_t box[2] = {(cuuint32_t)T8_BK, (cuuint32_t)box_rows}, estr[2] = {1u, 1u};
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void *>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
              CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// Returns false when the tensor maps cannot be made (the caller then takes gemm_int8_mma_kernel).
inline bool launch_gemm_int8_tma(float *c, const signed char *qa, const int *ea, const signed char *qb, const int *eb, int m, int n, int k,
                                 int sms, cudaStream_t st) {
    alignas(64) CUtensorMap map_a, map_b;
    if (!t8_make_map(&map_a, qa, m, k, T8_BM) || !t8_make_map(&map_b, qb, n, k, T8_BN)) return false;
    const int tiles_m = (m + T8_BM - 1) / T8_BM, tiles_n = (n + T8_BN - 1) / T8_BN, tiles = tiles_m * tiles_n;
    cudaFuncSetAttribute(gemm_int8_tma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, T8_SMEM_BYTES);
    gemm_int8_tma_kernel<<<tiles < sms ? tiles : sms, T8_THREADS, T8_SMEM_BYTES, st>>>(map_a, map_b, c, ea, eb, m, n, k, tiles_n, tiles);
    return true;
}

} // namespace b200i
