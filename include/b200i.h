/*
 * b200i: the identical-mode matrix product of mojolearn on NVIDIA B200 (sm_100a).
 *
 * A C ABI in the style of the reference's adapter ABI v1
 * (adapters/native/abi.h:7-33 of the reference): every scalar argument is an
 * int64_t, storage is caller-owned, contiguous and row-major, and valid until
 * the call returns; a call returns 0 on success and 1 on a refusal or an
 * error, with a NUL-terminated message in the caller's buffer (`err`, of
 * `err_cap` bytes; may be NULL). Nothing here takes a framework type.
 *
 * Two families of entry points:
 *   - `b200i_*` on DEVICE pointers: asynchronous on the caller's CUDA stream
 *     (`stream` is a cudaStream_t passed as void*, NULL = the default stream).
 *     The caller orders producers before the call on that stream.
 *   - `b200i_host_*` on HOST pointers: synchronous, like the reference's
 *     CPython doors (bindings/_mojolearn_linalg.mojo:160-208): upload, compute,
 *     download, complete before return.
 * Every product word is NaN-canonicalised to 0x7FC00000 at the store
 * (core/nan_canon.mojo:53-56 of the reference).
 *
 * Orientation codes are the contract's (gemm/contract.mojo): NN = 0, NT = 1,
 * TN = 2. All matrices are row-major without a leading dimension.
 */
#ifndef B200I_H
#define B200I_H
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define B200I_OP_NN 0
#define B200I_OP_NT 1
#define B200I_OP_TN 2

/* right-operand (weight) storage kinds */
#define B200I_W_F32 0        /* float32 words */
#define B200I_W_BF16 1       /* uint16 bf16 bit patterns */
#define B200I_W_INT8_EXP 2   /* int8 codes + int32 power-of-two exponent per row */
#define B200I_W_INT8_SCALE 3 /* int8 codes + float32 scale per row (extension) */

/* --- identity of the loaded binary ---------------------------------------------------
 * Replace linalg_numeric_mode / linalg_profile_version / linalg_numerical_profile /
 * lowbit_profile_version / linalg_vendor (bindings/_mojolearn_linalg.mojo:143-157)
 * and mojolearn_adapter_abi (adapters/native/abi.h). */
int64_t b200i_abi(void);                        /* 1 */
int64_t b200i_numeric_mode(void);               /* 1 = identical; there is no other build */
int64_t b200i_profile_version(void);            /* 1 */
int64_t b200i_lowbit_profile_version(void);     /* 1 */
const char *b200i_numerical_profile(void);      /* "mojolearn.identical.gemm.fp32.v1" */
const char *b200i_vendor(void);                 /* "cuda" */
int64_t b200i_device_count(void);               /* visible CUDA devices, 0 if none */

/* --- the product, device pointers -------------------------------------------------------
 * C[m,n] = op(A) . op(B) under mojolearn.identical.gemm.fp32.v1. Replaces
 * identical_gemm_into (gemm/checks/gemm_identical.mojo:6062) behind
 * gemm_binding(c, a, b, [m,n,k,op]) (bindings/_mojolearn_linalg.mojo:160-208).
 * `ws` is scratch of at least b200i_workspace_bytes(m,n,k) bytes (may be NULL
 * when that is 0). Refuses m, n, k <= 0 (gemm/host_entry.mojo:115-126), an
 * unknown op, NULL or misaligned storage. */
int64_t b200i_gemm_f32(int64_t device, void *stream, float *c, const float *a, const float *b, int64_t m, int64_t n,
                       int64_t k, int64_t op, void *ws, int64_t ws_bytes, char *err, int64_t err_cap);

/* The same product with the right operand held in weight storage `wkind`:
 * the weight is materialised exactly (bf16: bits << 16; int8: code * 2^e,
 * flushed) on its way into the tile and the fp32 plan runs on it. Replaces
 * identical_gemm_bf16w_into (gemm/checks/gemm_lowbit.mojo:369-395) and the
 * dequantize-then-fp32 path of the low-bit inference blocks
 * (gemm/host/gemm_lowbit_oracle.mojo:201-214). `bscale` is the int32 exponent
 * or float32 scale vector (one entry per row of B; int8 kinds need op = NT),
 * NULL otherwise. */
int64_t b200i_gemm_w(int64_t device, void *stream, float *c, const float *a, const void *b, const void *bscale,
                     int64_t wkind, int64_t m, int64_t n, int64_t k, int64_t op, void *ws, int64_t ws_bytes,
                     char *err, int64_t err_cap);

/* Same, with the execution plan forced: plan 0 = one thread per cell (the
 * on-device restatement of the oracle), 1 = 128x128 tiles, 2 = 64x64 tiles,
 * 3 = the row-streaming decode plan, 4 = 32x128 tiles; `group_leaves` = leaves per group (a
 * power of two, 0 = no split). Every plan returns the same bits; the tests
 * hold them to that (the reference's launch-invariance gate,
 * gemm/checks/gemm_device_check.mojo:1016). */
int64_t b200i_gemm_w_plan(int64_t device, void *stream, float *c, const float *a, const void *b, const void *bscale,
                          int64_t wkind, int64_t m, int64_t n, int64_t k, int64_t op, int64_t plan,
                          int64_t group_leaves, void *ws, int64_t ws_bytes, char *err, int64_t err_cap);

/* 1 when the row-streaming decode plan accepts the shape (op NT, m <= 8, k a
 * multiple of 16 with 128-element leaves, leaf partials and two ring stages
 * within shared memory), else 0. */
int64_t b200i_decode_plan_fits(int64_t m, int64_t n, int64_t k, int64_t op, int64_t wkind);

/* Scratch bytes the product needs for this shape on the current device. */
int64_t b200i_workspace_bytes(int64_t m, int64_t n, int64_t k);

/* --- conversions, device pointers ----------------------------------------------------------
 * Replace to_bf16 / from_bf16 / quantize_int8 / dequantize_int8
 * (bindings/_mojolearn_linalg.mojo:354-398, :490-526; kernels
 * gemm/checks/gemm_lowbit.mojo:166-187, :435-477). */
int64_t b200i_to_bf16(int64_t device, void *stream, uint16_t *dst, const float *src, int64_t count, char *err,
                      int64_t err_cap);
int64_t b200i_from_bf16(int64_t device, void *stream, float *dst, const uint16_t *src, int64_t count, char *err,
                        int64_t err_cap);
int64_t b200i_quantize_int8(int64_t device, void *stream, int8_t *codes, int32_t *exponents, const float *x,
                            int64_t rows, int64_t cols, char *err, int64_t err_cap);
int64_t b200i_dequantize_int8(int64_t device, void *stream, float *y, const int8_t *codes, const int32_t *exponents,
                              int64_t rows, int64_t cols, char *err, int64_t err_cap);

/* int8i32.v1 product at OP_NT: exact int32 sum of code products, one
 * dequantisation per cell. Replaces identical_gemm_int8_into
 * (gemm/checks/gemm_lowbit.mojo:557-589). Refuses k > 131072. */
int64_t b200i_gemm_int8(int64_t device, void *stream, float *c, const int8_t *qa, const int32_t *ea, const int8_t *qb,
                        const int32_t *eb, int64_t m, int64_t n, int64_t k, char *err, int64_t err_cap);

/* --- host-pointer twins (synchronous) -----------------------------------------------------------
 * The reference's public calls take host buffers and return when the answer
 * is in host memory (gemm/host_entry.mojo:79-197). */
int64_t b200i_host_gemm_w(int64_t device, float *c, const float *a, const void *b, const void *bscale, int64_t wkind,
                          int64_t m, int64_t n, int64_t k, int64_t op, char *err, int64_t err_cap);
int64_t b200i_host_to_bf16(int64_t device, uint16_t *dst, const float *src, int64_t count, char *err, int64_t err_cap);
int64_t b200i_host_from_bf16(int64_t device, float *dst, const uint16_t *src, int64_t count, char *err,
                             int64_t err_cap);
int64_t b200i_host_quantize_int8(int64_t device, int8_t *codes, int32_t *exponents, const float *x, int64_t rows,
                                 int64_t cols, char *err, int64_t err_cap);
int64_t b200i_host_dequantize_int8(int64_t device, float *y, const int8_t *codes, const int32_t *exponents,
                                   int64_t rows, int64_t cols, char *err, int64_t err_cap);
int64_t b200i_host_gemm_int8(int64_t device, float *c, const int8_t *qa, const int32_t *ea, const int8_t *qb,
                             const int32_t *eb, int64_t m, int64_t n, int64_t k, char *err, int64_t err_cap);

/* Status word of the decode plan's bounded waits on `device` (synchronises the
 * device): 0 = no wait ever ran out; 1 / 2 = the producer / a consumer gave up
 * waiting on a stage; -1 = the word could not be read. A nonzero word is cleared
 * by the read. No reference counterpart:
 * the reference has no device-side wait. */
int64_t b200i_decode_status(int64_t device);

/* Roofline probe: `blocks` CTAs of 256 threads, each thread 16 independent
 * chains of `iters` bare fused multiply-adds (scalar, or fma.rn.f32x2 pairs when
 * `packed` is 1): 2*16*iters flops per thread, doubled when packed. The caller
 * times it. `scratch` is one device float. No reference counterpart. */
int64_t b200i_ffma_probe(int64_t device, void *stream, float *scratch, int64_t blocks, int64_t iters, int64_t packed,
                         char *err, int64_t err_cap);

/* Kernels launched by this library since load (all devices); the benchmark
 * reports the difference over its timed region. */
int64_t b200i_launch_count(void);

#ifdef __cplusplus
}
#endif
#endif
