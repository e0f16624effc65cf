// The fifteen-bit profile, mojolearn.identical.gemm.int15i64.v1 (gemm/IDENTICAL_LOWBIT_CONTRACT.md section 6 of the
// reference, clauses W-1 to W-8; seams checks/numerics_int15.mojo, answers gemm/host/gemm_int15_oracle.mojo).
//
// An operand is three arrays: two int8 planes hi and lo (code = hi * 128 + lo, lo in [0, 127], hi in [-128, 127]) and one
// int32 exponent per row. The product is the exact integer sum of code products, converted to float32 with one rounding and
// scaled by 2^(ea + eb). With a = ah * 128 + al and b = bh * 128 + bl that sum is HH * 2^14 + (HL + LH) * 2^7 + LL, three
// int32 sums of int8 products, exact for k <= 65536: so the planes go through the same tcgen05.mma kind::i8 path as the
// int8i32 product (gemm_int8_mma.cuh), four MMAs per 32 steps of k into three accumulators in tensor memory, and the
// recombination happens in int64 in the store. This is the reference's MMA plan of clause W-8; FLAT (one thread per cell,
// the sum in int64) serves k that is not a multiple of 16. Both are the profile: an exact sum has one value.
#pragma once
#include "gemm_int8_mma.cuh"
#include "gemm_int8_tma.cuh"

namespace b200i {

constexpr long long INT15_MAX_K = 65536;

// ---- seams ---------------------------------------------------------------------------------------------------------------
// W-1: e = floor(log2 absmax) - 13, read from the exponent field; an all-zero row (after the flush) and a NaN take 0.
__device__ __forceinline__ int int15_row_exponent(float absmax) {
    const float a = ftz_bits(absmax);
    if (a == 0.0f || a != a) return 0;
    return (int)((__float_as_uint(a) >> 23) & 0xFFu) - 127 - 13;
}
// W-2: clamp(rne(ftz(ftz(x) * 2^-e)), -16383, 16383); a NaN codes to 0 before the scaling and after it (0 * inf).
__device__ __forceinline__ int quantize_int15_value(float x, int e) {
    if (x != x) return 0;
    const float s = ftz_bits(__fmul_rn(ftz_bits(x), pow2_f32(-e)));
    if (s != s) return 0;
    float r = round_half_even(s);
    if (r > 16383.0f) r = 16383.0f;
    if (r < -16383.0f) r = -16383.0f;
    return __float2int_rz(r);
}
// W-6: the int64 sum as a float32, round to nearest even: a 24-bit high and a 24-bit low part (each exact, each converted
// from an int32), one exact scaling and ONE rounding addition; at and above 2^48 the low sixteen bits become a sticky bit.
__device__ __forceinline__ float i64_to_f32_pinned(long long v) {
    const bool neg = v < 0;
    unsigned long long mag = (unsigned long long)v;
    if (neg) mag = 0ull - mag;
    bool reduced = false;
    if (mag >= (1ull << 48)) {
        const unsigned long long lost = mag & 0xFFFFull;
        mag >>= 16;
        if (lost != 0ull) mag |= 1ull;
        reduced = true;
    }
    const float hi = (float)(int)(mag >> 24), lo = (float)(int)(mag & 0xFFFFFFull);
    float r = __fadd_rn(__fmul_rn(hi, 16777216.0f), lo);
    if (reduced) r = __fmul_rn(r, 65536.0f);
    return neg ? -r : r;
}
// W-7: ftz(f32(sum) * 2^(ea + eb)); pow2_f32 is the infinity above 127 and +0.0 below -126.
__device__ __forceinline__ float dequant_int15_pinned(long long acc, long long e_sum) {
    const int e = e_sum > 1000 ? 1000 : (e_sum < -1000 ? -1000 : (int)e_sum);
    return ftz_bits(__fmul_rn(i64_to_f32_pinned(acc), pow2_f32(e)));
}

// ---- conversions: one warp per row, like the int8 quantizer -----------------------------------------------------------------
__global__ void quantize_int15_kernel(signed char *__restrict__ hi, signed char *__restrict__ lo, int *__restrict__ e,
                                      const float *__restrict__ x, long long rows, long long cols) {
    const int lane = threadIdx.x & 31;
    const long long warp = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const long long nwarps = ((long long)gridDim.x * blockDim.x) >> 5;
    for (long long r = warp; r < rows; r += nwarps) {
        const float *row = x + r * cols;
        float best = 0.f;
        for (long long c = lane; c < cols; c += 32) {
            const float v = fabsf(ftz_bits(row[c]));
            if (v > best) best = v; // a NaN never compares greater and is skipped
        }
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) best = fmaxf(best, __shfl_xor_sync(0xFFFFFFFFu, best, off));
        const int ex = int15_row_exponent(best);
        if (lane == 0) e[r] = ex;
        for (long long c = lane; c < cols; c += 32) {
            const int code = quantize_int15_value(row[c], ex);
            lo[r * cols + c] = (signed char)(code & 127); // W-3: a floor modulus, the low seven bits of the two's complement word
            hi[r * cols + c] = (signed char)(code >> 7);  // an arithmetic shift: floor(code / 128)
        }
    }
}

__global__ void dequantize_int15_kernel(float *__restrict__ y, const signed char *__restrict__ hi, const signed char *__restrict__ lo,
                                        const int *__restrict__ e, long long rows, long long cols) {
    const long long stride = (long long)gridDim.x * blockDim.x;
    const long long total = rows * cols;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride)
        y[i] = dequant_int15_pinned((long long)hi[i] * 128 + (long long)lo[i], (long long)__ldg(e + i / cols));
}

// ---- FLAT: one thread per cell, the sum of code products in int64 ----------------------------------------------------------
__global__ void gemm_int15_flat_kernel(float *__restrict__ c, const signed char *__restrict__ ah, const signed char *__restrict__ al,
                                       const int *__restrict__ ea, const signed char *__restrict__ bh, const signed char *__restrict__ bl,
                                       const int *__restrict__ eb, int m, int n, int k) {
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (long long)m * n) return;
    const int i = (int)(idx / n), j = (int)(idx % n);
    const size_t ra = (size_t)i * k, rb = (size_t)j * k;
    long long acc = 0;
    for (int p = 0; p < k; p++)
        acc += (long long)(((int)ah[ra + p] * 128 + (int)al[ra + p]) * ((int)bh[rb + p] * 128 + (int)bl[rb + p]));
    c[idx] = nan_canon(dequant_int15_pinned(acc, (long long)ea[i] + (long long)eb[j]));
}

// ---- MMA: the planes on the tensor cores ---------------------------------------------------------------------------------------
// A CTA of 128 threads owns a 128 x 64 tile; three int32 accumulators of 64 columns each (HH, HL + LH, LL) live in 192 of
// its 256 tensor-memory columns; two ring stages of 128 bytes of k of the four planes (48 KB per stage): two CTAs per SM.
constexpr int I15_TN = 64, I15_STAGES = 2;
constexpr int I15_STAGE_BYTES = 2 * (I8_TILE_M + I15_TN) * I8_KB;
constexpr int I15_SMEM_BYTES = I15_STAGES * I15_STAGE_BYTES + 256;
constexpr unsigned I15_TMEM_COLS = 256;

__global__ void __launch_bounds__(I8_THREADS) gemm_int15_mma_kernel(float *__restrict__ c, const signed char *__restrict__ ah,
                                                                    const signed char *__restrict__ al, const int *__restrict__ ea,
                                                                    const signed char *__restrict__ bh, const signed char *__restrict__ bl,
                                                                    const int *__restrict__ eb, int m, int n, int k) {
    extern __shared__ __align__(128) unsigned char smem[];
    constexpr int A_BYTES = I8_TILE_M * I8_KB, B_BYTES = I15_TN * I8_KB, S = I15_STAGES;
    // a stage: A hi, A lo, B hi, B lo
    unsigned long long *done = reinterpret_cast<unsigned long long *>(smem + S * I15_STAGE_BYTES);
    unsigned *tmem_slot = reinterpret_cast<unsigned *>(done + S + 1);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int row0 = blockIdx.x * I8_TILE_M, col0 = blockIdx.y * I15_TN;
    const int kt_count = (k + I8_KB - 1) / I8_KB;

    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(I15_TMEM_COLS) : "memory");
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

    auto load_stage = [&](int buf, int k0) {
        unsigned char *st = smem + buf * I15_STAGE_BYTES;
        i8_load_operand<I8_TILE_M>(st, ah, row0, m, k, k0, tid);
        i8_load_operand<I8_TILE_M>(st + A_BYTES, al, row0, m, k, k0, tid);
        i8_load_operand<I15_TN>(st + 2 * A_BYTES, bh, col0, n, k, k0, tid);
        i8_load_operand<I15_TN>(st + 2 * A_BYTES + B_BYTES, bl, col0, n, k, k0, tid);
    };

    bool alive = true;
    for (int s = 0; s < S - 1; s++) { // one commit group per k-block, empty ones included
        if (s < kt_count) load_stage(s, s * I8_KB);
        asm volatile("cp.async.commit_group;" ::: "memory");
    }
    for (int kt = 0; kt < kt_count; kt++) {
        const int buf = kt % S, nxt = kt + S - 1;
        if (nxt < kt_count) {
            const int nbuf = nxt % S;
            if (nxt >= S && alive && !mbar_wait(&done[nbuf], (unsigned)((nxt / S - 1) & 1))) alive = false;
            load_stage(nbuf, nxt * I8_KB);
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
        asm volatile("cp.async.wait_group %0;" ::"n"(S - 1) : "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        __syncthreads();
        if (tid == 0) {
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const unsigned st = smem_u32(smem + buf * I15_STAGE_BYTES);
            const unsigned a_hi = st, a_lo = st + A_BYTES, b_hi = st + 2 * A_BYTES, b_lo = st + 2 * A_BYTES + B_BYTES;
#pragma unroll
            for (int j = 0; j < I8_KB / 32; j++) {
                const unsigned more = (kt > 0 || j > 0) ? 1u : 0u;
                const unsigned long long dah = i8_smem_desc(a_hi + j * 256), dal = i8_smem_desc(a_lo + j * 256);
                const unsigned long long dbh = i8_smem_desc(b_hi + j * 256), dbl = i8_smem_desc(b_lo + j * 256);
                i8_mma(tmem_d, dah, dbh, i8_idesc(I15_TN), more);               // HH
                i8_mma(tmem_d + I15_TN, dah, dbl, i8_idesc(I15_TN), more);      // HL ...
                i8_mma(tmem_d + I15_TN, dal, dbh, i8_idesc(I15_TN), 1u);        // ... + LH: one int32 (W-4)
                i8_mma(tmem_d + 2 * I15_TN, dal, dbl, i8_idesc(I15_TN), more);  // LL
            }
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
        // A thread reads 32 columns of its row from each accumulator and recombines them in int64 (W-5); the block of
        // 32 x 32 sums is then turned through shared memory so that a store instruction writes a row segment.
        unsigned long long *turn = reinterpret_cast<unsigned long long *>(smem) + warp * (32 * 33);
        const int rbase = row0 + warp * 32;
        const int ea_mine = rbase + lane < m ? ea[rbase + lane] : 0;
#pragma unroll 1
        for (int cb = 0; cb < I15_TN; cb += 32) {
            if (col0 + cb >= n) break; // uniform over the CTA
            long long sum[32];
#pragma unroll
            for (int part = 0; part < 3; part++) {
                unsigned v[32];
                asm volatile(
                    "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, %17, %18, %19, "
                    "%20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
                    : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]), "=r"(v[9]),
                      "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]), "=r"(v[17]), "=r"(v[18]),
                      "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]),
                      "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
                    : "r"(tmem_d + ((unsigned)(warp * 32) << 16) + (unsigned)(part * I15_TN + cb))
                    : "memory");
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
                for (int j = 0; j < 32; j++) {
                    const long long piece = (long long)(int)v[j];
                    sum[j] = part == 0 ? piece * 16384 : (part == 1 ? sum[j] + piece * 128 : sum[j] + piece);
                }
            }
#pragma unroll
            for (int j = 0; j < 32; j++) turn[lane * 33 + j] = (unsigned long long)sum[j];
            __syncwarp();
            const int col = col0 + cb + lane;
            const long long eb_mine = col < n ? (long long)__ldg(eb + col) : 0;
#pragma unroll 4
            for (int rr = 0; rr < 32; rr++) {
                const long long esum = (long long)__shfl_sync(0xFFFFFFFFu, ea_mine, rr) + eb_mine;
                if (rbase + rr < m && col < n)
                    c[(size_t)(rbase + rr) * n + col] = nan_canon(dequant_int15_pinned((long long)turn[rr * 33 + lane], esum));
            }
            __syncwarp();
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 0) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_d), "r"(I15_TMEM_COLS) : "memory");
}

inline bool gemm_int15_mma_fits(const void *ah, const void *al, const void *bh, const void *bl, long long m, long long n, long long k) {
    const uintptr_t all = reinterpret_cast<uintptr_t>(ah) | reinterpret_cast<uintptr_t>(al) | reinterpret_cast<uintptr_t>(bh) | reinterpret_cast<uintptr_t>(bl);
    return k % 16 == 0 && (all & 15) == 0 && (m + I8_TILE_M - 1) / I8_TILE_M <= 0x7FFFFFFFll && (n + I15_TN - 1) / I15_TN <= 65535;
}

inline void launch_gemm_int15_mma(float *c, const signed char *ah, const signed char *al, const int *ea, const signed char *bh,
                                  const signed char *bl, const int *eb, int m, int n, int k, cudaStream_t st) {
    cudaFuncSetAttribute(gemm_int15_mma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, I15_SMEM_BYTES);
    const dim3 grid((unsigned)((m + I8_TILE_M - 1) / I8_TILE_M), (unsigned)((n + I15_TN - 1) / I15_TN));
    gemm_int15_mma_kernel<<<grid, I8_THREADS, I15_SMEM_BYTES, st>>>(c, ah, al, ea, bh, bl, eb, m, n, k);
}

// ---- the same plan as a persistent, warp-specialised kernel (the structure of gemm_int8_tma_kernel) --------------------------
// One CTA per SM walks 128 x 64 tiles. A stage is 128 bytes of k of the four planes (A hi, A lo: 128 rows; B hi, B lo: 64
// rows; 48 KB), brought by four tensor-map copies into the 128-byte swizzled K-major layout, three stages; the MMA lane
// issues HH, HL, LH, LL per 32 steps of k into three accumulators of 64 columns; two such accumulator sets (at columns 0 and
// 256 of tensor memory) let the eight store warps recombine, convert and store one tile under the next tile's MMAs.
constexpr int F15_STAGES = 3, F15_STAGE_BYTES = 2 * T8_A_BYTES + 2 * I15_TN * T8_BK, F15_ACC_STRIDE = 256;
constexpr int F15_TURN_BYTES = T8_STORE_WARPS * 32 * 33 * 8;
constexpr int F15_SMEM_BYTES = 1024 + F15_STAGES * F15_STAGE_BYTES + F15_TURN_BYTES + 256;

__global__ void __launch_bounds__(T8_THREADS, 1)
gemm_int15_tma_kernel(const __grid_constant__ CUtensorMap map_ah, const __grid_constant__ CUtensorMap map_al, const __grid_constant__ CUtensorMap map_bh,
                      const __grid_constant__ CUtensorMap map_bl, float *__restrict__ c, const int *__restrict__ ea, const int *__restrict__ eb, int m,
                      int n, int k, int tiles_n, int tiles) {
    extern __shared__ __align__(128) unsigned char smem[];
    constexpr int B_BYTES = I15_TN * T8_BK;
    unsigned char *ring = smem + ((1024u - (smem_u32(smem) & 1023u)) & 1023u);
    unsigned long long *turn_all = reinterpret_cast<unsigned long long *>(ring + F15_STAGES * F15_STAGE_BYTES);
    unsigned long long *full = reinterpret_cast<unsigned long long *>(ring + F15_STAGES * F15_STAGE_BYTES + F15_TURN_BYTES);
    unsigned long long *empty = full + F15_STAGES, *tfull = empty + F15_STAGES, *tempty = tfull + 2;
    unsigned *tmem_slot = reinterpret_cast<unsigned *>(tempty + 2);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int kt_count = (k + T8_BK - 1) / T8_BK;

    if (tid == 0) {
        for (int s = 0; s < F15_STAGES; s++) {
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
                    const int s = it % F15_STAGES;
                    const unsigned ph = (unsigned)(it / F15_STAGES) & 1u;
                    if (!mbar_wait(&empty[s], ph ^ 1u)) {
                        atomicExch(&g_decode_status, 9);
                        alive = false;
                        break;
                    }
                    unsigned char *st = ring + s * F15_STAGE_BYTES;
                    mbar_expect_tx(&full[s], (unsigned)F15_STAGE_BYTES);
                    t8_tma_load(st, &map_ah, &full[s], kt * T8_BK, tm * T8_BM);
                    t8_tma_load(st + T8_A_BYTES, &map_al, &full[s], kt * T8_BK, tm * T8_BM);
                    t8_tma_load(st + 2 * T8_A_BYTES, &map_bh, &full[s], kt * T8_BK, tn * I15_TN);
                    t8_tma_load(st + 2 * T8_A_BYTES + B_BYTES, &map_bl, &full[s], kt * T8_BK, tn * I15_TN);
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
                const unsigned d = tmem + (unsigned)(acc * F15_ACC_STRIDE);
                for (int kt = 0; kt < kt_count; kt++, it++) {
                    const int s = it % F15_STAGES;
                    const unsigned ph = (unsigned)(it / F15_STAGES) & 1u;
                    if (!mbar_wait(&full[s], ph)) {
                        atomicExch(&g_decode_status, 9);
                        alive = false;
                        break;
                    }
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const unsigned a_hi = smem_u32(ring + s * F15_STAGE_BYTES), a_lo = a_hi + T8_A_BYTES, b_hi = a_hi + 2 * T8_A_BYTES, b_lo = b_hi + B_BYTES;
#pragma unroll
                    for (int j = 0; j < T8_BK / 32; j++) {
                        const unsigned more = (kt > 0 || j > 0) ? 1u : 0u;
                        const unsigned long long dah = t8_smem_desc(a_hi + j * 32), dal = t8_smem_desc(a_lo + j * 32);
                        const unsigned long long dbh = t8_smem_desc(b_hi + j * 32), dbl = t8_smem_desc(b_lo + j * 32);
                        i8_mma(d, dah, dbh, i8_idesc(I15_TN), more);              // HH
                        i8_mma(d + I15_TN, dah, dbl, i8_idesc(I15_TN), more);     // HL ...
                        i8_mma(d + I15_TN, dal, dbh, i8_idesc(I15_TN), 1u);       // ... + LH
                        i8_mma(d + 2 * I15_TN, dal, dbl, i8_idesc(I15_TN), more); // LL
                    }
                    i8_commit(&empty[s]);
                }
                if (alive) i8_commit(&tfull[acc]);
            }
        }
    } else { // ---------------- store warps: quarter of the lanes (warp % 4), half of the 64 columns each ----------------
        const int q = warp & 3, half = (warp - 2) >> 2;
        unsigned long long *turn = turn_all + (warp - 2) * (32 * 33);
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
            const int rbase = tm * T8_BM + q * 32, cb = half * 32, col0 = tn * I15_TN;
            if (col0 + cb < n) { // uniform over the warp
                const int ea_mine = rbase + lane < m ? ea[rbase + lane] : 0;
                long long sum[32];
#pragma unroll
                for (int part = 0; part < 3; part++) {
                    unsigned v[32];
                    asm volatile(
                        "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, %17, %18, %19, "
                        "%20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
                        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]), "=r"(v[9]),
                          "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]), "=r"(v[17]), "=r"(v[18]),
                          "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]),
                          "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
                        : "r"(tmem + ((unsigned)(q * 32) << 16) + (unsigned)(acc * F15_ACC_STRIDE + part * I15_TN + cb))
                        : "memory");
                    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
                    for (int j = 0; j < 32; j++) {
                        const long long piece = (long long)(int)v[j];
                        sum[j] = part == 0 ? piece * 16384 : (part == 1 ? sum[j] + piece * 128 : sum[j] + piece);
                    }
                }
#pragma unroll
                for (int j = 0; j < 32; j++) turn[lane * 33 + j] = (unsigned long long)sum[j];
                __syncwarp();
                const int col = col0 + cb + lane;
                const long long eb_mine = col < n ? (long long)__ldg(eb + col) : 0;
#pragma unroll 4
                for (int rr = 0; rr < 32; rr++) {
                    const long long esum = (long long)__shfl_sync(0xFFFFFFFFu, ea_mine, rr) + eb_mine;
                    if (rbase + rr < m && col < n)
                        c[(size_t)(rbase + rr) * n + col] = nan_canon(dequant_int15_pinned((long long)turn[rr * 33 + lane], esum));
                }
            }
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(&tempty[acc]);
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 1) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(T8_TMEM_COLS) : "memory");
}

// Returns false when the tensor maps cannot be made (the caller then takes gemm_int15_mma_kernel).
inline bool launch_gemm_int15_tma(float *c, const signed char *ah, const signed char *al, const int *ea, const signed char *bh, const signed char *bl,
                                  const int *eb, int m, int n, int k, int sms, cudaStream_t st) {
    alignas(64) CUtensorMap map_ah, map_al, map_bh, map_bl;
    if (!t8_make_map(&map_ah, ah, m, k, T8_BM) || !t8_make_map(&map_al, al, m, k, T8_BM) || !t8_make_map(&map_bh, bh, n, k, I15_TN) ||
        !t8_make_map(&map_bl, bl, n, k, I15_TN))
        return false;
    const int tiles_m = (m + T8_BM - 1) / T8_BM, tiles_n = (n + I15_TN - 1) / I15_TN, tiles = tiles_m * tiles_n;
    cudaFuncSetAttribute(gemm_int15_tma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, F15_SMEM_BYTES);
    gemm_int15_tma_kernel<<<tiles < sms ? tiles : sms, T8_THREADS, F15_SMEM_BYTES, st>>>(map_ah, map_al, map_bh, map_bl, c, ea, eb, m, n, k, tiles_n, tiles);
    return true;
}

} // namespace b200i
