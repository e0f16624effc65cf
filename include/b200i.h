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
 * 3 = the row-streaming decode plan (up to 8 rows), 4 = 32x128 tiles, 5 = 128x64 tiles,
 * 6 = the skinny plan (op NT, up to 32 activation rows, k a multiple of 16, 16-byte aligned
 * operands), 7 = the packed plan (operands repacked into tile-major panels in the workspace,
 * then 128x128 tiles fed by bulk copies; needs a 256-byte aligned workspace of
 * b200i_plan_workspace_bytes); `group_leaves` = leaves per group (a power of two, 0 = no split). Every plan returns the same bits; the tests
 * hold them to that (the reference's launch-invariance gate,
 * gemm/checks/gemm_device_check.mojo:1016). */
int64_t b200i_gemm_w_plan(int64_t device, void *stream, float *c, const float *a, const void *b, const void *bscale,
                          int64_t wkind, int64_t m, int64_t n, int64_t k, int64_t op, int64_t plan,
                          int64_t group_leaves, void *ws, int64_t ws_bytes, char *err, int64_t err_cap);

/* The product with a store epilogue: bias (one float32 per output column, or NULL) is added to the
 * finished word, then `act` is applied: 0 = none, 1 = gelu (erf), 2 = gelu (tanh), 3 = silu. Replaces
 * the reference's GEMM_EPI_PLUS_BIAS and GEMM_EPI_BIAS_ACT stores (gemm/checks/gemm_identical.mojo
 * :8869-8912, :9483-9491): the words are those of b200i_gemm_w followed by b200i_bias_add and the
 * ungated b200i_act_mul, with one launch instead of three. `plan` and `group_leaves` as for
 * b200i_gemm_w_plan (-1, 0 = automatic).
 * act 4 / 5 / 6 = the GATED activations silu(gate)*up / gelu(gate)*up / gelu_tanh(gate)*up (S20-S21) over a weight
 * whose rows were interleaved by the caller (row 2j = gate_j, row 2j + 1 = up_j; a bias interleaved the same way):
 * c is then [m, n / 2]. Only the skinny plans spell it (a thread there owns both columns of a pair); it is refused
 * by name for a shape outside them (b200i_pair_epilogue_fits says which), and the caller then runs the product
 * and b200i_act_mul with `interleaved` = 1. */
int64_t b200i_gemm_w_epilogue(int64_t device, void *stream, float *c, const float *a, const void *b, const void *bscale, int64_t wkind,
                              int64_t m, int64_t n, int64_t k, int64_t op, const float *bias, int64_t act, int64_t plan,
                              int64_t group_leaves, void *ws, int64_t ws_bytes, char *err, int64_t err_cap);

/* b200i_gemm_w_epilogue with the automatic plan, except that a product split into leaf groups is
 * left unfolded for a caller that folds it elsewhere (b200i_comm_gather_nodes, the gather after a
 * column-sharded product): *nodes = the number of nodes per cell left in ws[nodes][m * n], and c is
 * untouched; *nodes = 1 means c holds the finished product with its epilogue, as usual (the plan did
 * not split, or n is not a multiple of 4). */
int64_t b200i_gemm_w_nodes(int64_t device, void *stream, float *c, const float *a, const void *b, const void *bscale, int64_t wkind,
                           int64_t m, int64_t n, int64_t k, int64_t op, const float *bias, int64_t act, void *ws, int64_t ws_bytes,
                           int64_t *nodes, char *err, int64_t err_cap);
int64_t b200i_pair_epilogue_fits(int64_t m, int64_t n, int64_t k, int64_t op);

/* Device timing of the product's main kernel, for benchmarks. While enabled (enable = 1 also
 * clears the record) every product call records a CUDA event pair on its stream around its main
 * kernel: the tile, packed, skinny or decode kernel, not the packing passes or the group fold.
 * b200i_kernel_timing_read waits for the recorded events and returns their summed milliseconds
 * and count (at most 4096 calls are recorded), then clears the record. Not for use while a
 * stream is being captured. No reference counterpart. */
int64_t b200i_kernel_timing(int64_t enable);
int64_t b200i_kernel_timing_read(double *total_ms, int64_t *launches);

/* Scratch a forced plan needs for the shape (group nodes, and the packed plan's panels and flags);
 * plan -1 is b200i_workspace_bytes. */
int64_t b200i_plan_workspace_bytes(int64_t m, int64_t n, int64_t k, int64_t plan, int64_t group_leaves);

/* 1 when the row-streaming decode plan accepts the shape (op NT, m <= 8, k a
 * multiple of 16 with 128-element leaves, leaf partials and two ring stages
 * within shared memory), else 0. */
int64_t b200i_decode_plan_fits(int64_t m, int64_t n, int64_t k, int64_t op, int64_t wkind);

/* The float32 product for callers that must not allocate: code running inside an
 * allocator hook or a memory-pool callback, a real-time serving loop with a fixed
 * device-memory budget, or a host that hands this library raw pointers and forbids
 * it cudaMalloc. It has no counterpart in the reference. Same arithmetic and same
 * bits as b200i_gemm_f32; the difference is where the split plan's scratch (the
 * leaf-group nodes) lives: in a fixed 16 MiB array inside the library image, which
 * every GPU that loads the library holds until the process exits. The call itself
 * makes no cudaMalloc, cudaFree or other allocating call, and records no timing
 * events. The 16 MiB are the limit of the scratch, not of the shapes: when the
 * leaf split the cost model prefers would need more, the call runs the same tiles
 * with the leaves in fewer, larger groups (down to no split, which needs no
 * scratch) -- the same bits from fewer CTAs, so a very deep product with few
 * output tiles runs slower here than through b200i_gemm_f32 with caller scratch.
 * b200i_noalloc_scratch_bytes says how much of the array a shape will use; a need
 * above 16 MiB would be refused with a message naming both sizes. The first call
 * on each device looks up the array's device address (a synchronous runtime
 * query), so make that first call before any stream capture begins. What the CUDA
 * driver does on the first launch of a kernel is outside this library: with lazy
 * module loading it may load code, and the first use of a tile shape sets a
 * function attribute. A caller entering a no-allocation region should first run
 * one product of each kind it will need (one split, one unsplit; small, medium and
 * large outputs pick different tile shapes), or set CUDA_MODULE_LOADING=EAGER.
 * All calls on a device share the one array: nothing in it has to start at zero
 * (every node a launch reads was written by that launch), but two calls that
 * overlap on the GPU, on different streams or threads, race on it. */
int64_t b200i_gemm_f32_noalloc(int64_t device, void *stream, float *c, const float *a, const float *b, int64_t m, int64_t n,
                               int64_t k, int64_t op, char *err, int64_t err_cap);
int64_t b200i_noalloc_scratch_bytes(int64_t m, int64_t n, int64_t k);

/* Scratch bytes the product needs for this shape. The answer depends on the SM count of the
 * device that is CURRENT when this is called: call it with the device current that the product
 * will later be given. */
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
 * (gemm/checks/gemm_lowbit.mojo:557-589) and the tensor-core form
 * gemm/checks/gemm_int8_mma.mojo:545-620. Refuses k > 131072. With k a multiple
 * of 16 and 16-byte aligned code storage the sum runs as tcgen05 int8 MMAs into
 * an int32 accumulator in tensor memory (any order of an exact integer sum gives
 * the same word); otherwise one thread walks each cell. */
int64_t b200i_gemm_int8(int64_t device, void *stream, float *c, const int8_t *qa, const int32_t *ea, const int8_t *qb,
                        const int32_t *eb, int64_t m, int64_t n, int64_t k, char *err, int64_t err_cap);

/* The fifteen-bit profile, mojolearn.identical.gemm.int15i64.v1 (gemm/IDENTICAL_LOWBIT_CONTRACT.md section 6; seams
 * checks/numerics_int15.mojo, answers gemm/host/gemm_int15_oracle.mojo). An operand is two int8 planes (code = hi * 128 +
 * lo, lo in [0, 127], hi in [-128, 127]) and one int32 exponent per row, e = floor(log2 absmax) - 13. Replace
 * quantize_rows_int15_kernel, dequantize and identical_gemm_int15 (gemm/checks/gemm_int15.mojo; door
 * family_lin_quantize_int15 / _dequantize_int15 / _matmul_int15, python/mojolearn/_linalg_impl.py:381-419). The product is
 * OP_NT: the exact int64 sum of code products, one rounding to float32, one power-of-two scaling per cell. With k a multiple
 * of 16 and 16-byte aligned planes it runs as tcgen05 int8 MMAs on the planes into three int32 accumulators (HH, HL + LH,
 * LL) recombined in int64 in the store; otherwise one thread walks each cell. Refuses k > 65536. */
int64_t b200i_quantize_int15(int64_t device, void *stream, int8_t *hi, int8_t *lo, int32_t *exponents, const float *x, int64_t rows,
                             int64_t cols, char *err, int64_t err_cap);
int64_t b200i_dequantize_int15(int64_t device, void *stream, float *y, const int8_t *hi, const int8_t *lo, const int32_t *exponents,
                               int64_t rows, int64_t cols, char *err, int64_t err_cap);
int64_t b200i_gemm_int15(int64_t device, void *stream, float *c, const int8_t *ah, const int8_t *al, const int32_t *ea, const int8_t *bh,
                         const int8_t *bl, const int32_t *eb, int64_t m, int64_t n, int64_t k, char *err, int64_t err_cap);

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
int64_t b200i_host_quantize_int15(int64_t device, int8_t *hi, int8_t *lo, int32_t *exponents, const float *x, int64_t rows, int64_t cols,
                                  char *err, int64_t err_cap);
int64_t b200i_host_dequantize_int15(int64_t device, float *y, const int8_t *hi, const int8_t *lo, const int32_t *exponents, int64_t rows,
                                    int64_t cols, char *err, int64_t err_cap);
int64_t b200i_host_gemm_int15(int64_t device, float *c, const int8_t *ah, const int8_t *al, const int32_t *ea, const int8_t *bh,
                              const int8_t *bl, const int32_t *eb, int64_t m, int64_t n, int64_t k, char *err, int64_t err_cap);

/* --- decoder-block seams, device pointers, asynchronous on the caller's stream -------------------
 * The non-GEMM steps of the reference's decoder block, each spelled as the
 * reference pins it (transformer/IDENTICAL_TRANSFORMER_CONTRACT.md:207-240; host
 * oracle transformer/checks/transformer_oracle.mojo). They replace the device
 * block's stages behind transformer_forward / transformer_decode_step
 * (bindings/_mojolearn_transformer.mojo:1209-1230) and the primitive doors
 * embedding_forward / rms_norm_forward (bindings/_mojolearn_training.mojo:575-587, :607-619). */

/* kind 0 = RMSNorm (S1-S4), 1 = LayerNorm (bias optional), 2 = RMSNorm with weight 1 + w.
 * out and x are [rows, width]; transformer_oracle.mojo:1223-1341. */
int64_t b200i_norm(int64_t device, void *stream, float *out, const float *x, const float *w, const float *bias, int64_t rows,
                   int64_t width, double eps, int64_t kind, char *err, int64_t err_cap);
/* The residual add and the norm that follows it in one pass: sum_out = ftz(ftz(x) + ftz(delta)) (S22 / S23),
 * out = norm(sum_out) as b200i_norm. Same bits as b200i_add then b200i_norm. */
int64_t b200i_add_norm(int64_t device, void *stream, float *out, float *sum_out, const float *x, const float *delta, const float *w,
                       const float *bias, int64_t rows, int64_t width, double eps, int64_t kind, char *err, int64_t err_cap);
/* The fresh q | k | v rows of a call in one pass: q rotated into qr [b*l, n_heads*head_dim], k rotated into its cache
 * slots, v copied into its cache slots: b200i_rope_apply on q and k plus b200i_kv_append on k and v, same bits.
 * Sources share the row pitch src_ld (they may be column blocks of one fused product); cosv / sinv NULL = no rotation;
 * `position` not NULL = the cached-token count is read from that device word (as the _at entries), else pos0.
 * `rope_dim` = rotated columns of a head (0 = head_dim; the tables are then [l, rope_dim / 2]): the rest of a head's
 * columns pass through, flushed (partial rotary, transformer/checks/transformer_oracle.mojo:1433-1440). */
int64_t b200i_qkv_rope_cache(int64_t device, void *stream, float *qr, float *kcache, float *vcache, const float *q, const float *k,
                             const float *v, int64_t src_ld, const float *cosv, const float *sinv, int64_t b, int64_t l,
                             int64_t n_heads, int64_t n_kv, int64_t head_dim, int64_t cap, int64_t pos0, const int32_t *position,
                             int64_t rope_dim, char *err, int64_t err_cap);
/* cos and sin [l, head_dim/2] for absolute positions pos0 .. pos0+l-1 (S6-S8); positions stay below 8192. */
int64_t b200i_rope_table(int64_t device, void *stream, float *cosv, float *sinv, int64_t pos0, int64_t l, int64_t head_dim,
                         double theta, char *err, int64_t err_cap);
/* The table under the block's option record (transformer/block_options.mojo:40-70, spelled as
 * transformer/checks/transformer_oracle.mojo:423-497): cos and sin [l, rope_dim / 2]; scaling 0 = none, 1 = linear
 * (inverse frequencies divided by `factor`), 2 = llama3 (rescaled by wavelength between the two frequency factors
 * against original_max_positions). `position` not NULL = the first position is read from that device word, else pos0. */
int64_t b200i_rope_table_opts(int64_t device, void *stream, float *cosv, float *sinv, int64_t pos0, const int32_t *position, int64_t l,
                              int64_t rope_dim, double theta, int64_t scaling, double factor, double low_freq_factor,
                              double high_freq_factor, int64_t original_max_positions, char *err, int64_t err_cap);
/* out[rows, n_heads*head_dim] = rotate(src) with the table of the call's l positions (S9-S10); not in place.
 * `src_ld` is the row pitch of src in floats (0 = contiguous rows): the projection may be a column block of
 * one fused q|k|v product. */
int64_t b200i_rope_apply(int64_t device, void *stream, float *out, const float *src, const float *cosv, const float *sinv,
                         int64_t rows, int64_t l, int64_t n_heads, int64_t head_dim, int64_t src_ld, int64_t rope_dim, char *err,
                         int64_t err_cap);
/* cache[b, n_kv, cap, head_dim] <- src[b*l, n_kv*head_dim] (row pitch src_ld, 0 = contiguous) at positions
 * pos0 .. pos0+l-1 (a copy). */
int64_t b200i_kv_append(int64_t device, void *stream, float *cache, const float *src, int64_t b, int64_t l, int64_t n_kv,
                        int64_t head_dim, int64_t cap, int64_t pos0, int64_t src_ld, char *err, int64_t err_cap);
/* ctx[b*l, n_heads*head_dim] from rotated queries q[b*l, n_heads*head_dim] and caches holding `used`
 * positions, this call's l included (S11-S19: eager attention, serial key-axis chains). `scores` is
 * scratch of b*n_heads*l*min(used, window or used) floats; a call of 2 to 8 query rows per sequence with
 * head_dim a multiple of 4 runs as one kernel that keeps its score rows in shared memory (the reference's fused
 * attention, transformer/impl/llama/fused_attention.mojo:5: same fold order, nothing materialised) and leaves
 * the scratch untouched. head_dim <= 128. `softcap` (0 = none) caps every scaled score as cap * tanh(score / cap)
 * before the mask is added (transformer_oracle.mojo:2269-2281). */
/* Floats of score scratch b200i_attention / b200i_attention_at need for (b, l, n_heads, s keys): the whole block for a
 * decode step; for a prompt the block of as many sequences as fit 4 GB (at least one): a larger batch is walked through
 * that scratch a few sequences at a time. */
int64_t b200i_attention_scratch_floats(int64_t b, int64_t l, int64_t n_heads, int64_t s);
int64_t b200i_attention(int64_t device, void *stream, float *ctx, const float *q, const float *kcache, const float *vcache,
                        float *scores, int64_t b, int64_t l, int64_t n_heads, int64_t n_kv, int64_t head_dim, int64_t cap,
                        int64_t used, int64_t window, double softcap, char *err, int64_t err_cap);
/* kind 0 = silu(gate)*up, 1 = gelu_erf(up), 2 = gelu_tanh(up), 3 = silu(up), 4 / 5 = gelu(gate)*up (S20-S21).
 * out is [rows, width] contiguous; gate and up are [rows, width] with row pitch in_ld (0 = contiguous).
 * `interleaved` = 1: gate and up are the even and odd columns of ONE [rows, 2 * width] matrix (pass its first
 * element as `gate`, `up` is ignored, in_ld its row pitch): the layout of a product over interleaved weight rows. */
int64_t b200i_act_mul(int64_t device, void *stream, float *out, const float *gate, const float *up, int64_t rows, int64_t width,
                      int64_t in_ld, int64_t kind, int64_t interleaved, char *err, int64_t err_cap);
/* out = ftz(ftz(a) + ftz(b)) (S22, S23); may be in place. */
int64_t b200i_add(int64_t device, void *stream, float *out, const float *a, const float *b, int64_t count, char *err, int64_t err_cap);
/* buf[rows, width] += bias[width], one plain add per cell (transformer_oracle.mojo:1344-1372). */
int64_t b200i_bias_add(int64_t device, void *stream, float *buf, const float *bias, int64_t rows, int64_t width, char *err,
                       int64_t err_cap);
/* y[n, width] = ftz(table[ids[n]]); status[0] becomes 1 if an id is outside [0, vocab)
 * (embedding/checks/embedding_oracle.mojo:369-382). */
int64_t b200i_embedding(int64_t device, void *stream, float *y, const float *table, const int32_t *ids, int64_t n, int64_t vocab,
                        int64_t width, int32_t *status, char *err, int64_t err_cap);
/* x[rows, width] += pos[pos0 + row % l] (learned positions; an extension, the reference's block always rotates). */
int64_t b200i_add_positions(int64_t device, void *stream, float *x, const float *pos, int64_t rows, int64_t l, int64_t pos0,
                            int64_t width, char *err, int64_t err_cap);
/* The position-on-device twins, for a decode step captured once as a CUDA graph and replayed:
 * a replayed launch cannot take the number of cached tokens as an argument, so these read it
 * from `position`, one device int32 holding the tokens cached BEFORE the call (the pos0 of the
 * calls above; `used` = *position + l). Same arithmetic, same bits. The launch is sized for the
 * whole cache, `scores` must hold b*n_heads*l*min(cap, window - 1 + l or cap) floats, and the
 * caller keeps *position + l within cap and below 8192 (a write past the cache is skipped).
 * b200i_advance_position adds `delta` to the word on the stream. No reference counterpart: the
 * reference's resident decode session (python/mojolearn/models/causal_lm.py:197-201) keeps its
 * position on the host. */
int64_t b200i_rope_table_at(int64_t device, void *stream, float *cosv, float *sinv, const int32_t *position, int64_t l,
                            int64_t head_dim, double theta, char *err, int64_t err_cap);
int64_t b200i_kv_append_at(int64_t device, void *stream, float *cache, const float *src, int64_t b, int64_t l, int64_t n_kv,
                           int64_t head_dim, int64_t cap, const int32_t *position, int64_t src_ld, char *err, int64_t err_cap);
int64_t b200i_attention_at(int64_t device, void *stream, float *ctx, const float *q, const float *kcache, const float *vcache,
                           float *scores, int64_t b, int64_t l, int64_t n_heads, int64_t n_kv, int64_t head_dim, int64_t cap,
                           const int32_t *position, int64_t window, double softcap, char *err, int64_t err_cap);
int64_t b200i_add_positions_at(int64_t device, void *stream, float *x, const float *pos, int64_t rows, int64_t l,
                               const int32_t *position, int64_t width, char *err, int64_t err_cap);
int64_t b200i_advance_position(int64_t device, void *stream, int32_t *position, int64_t delta, char *err, int64_t err_cap);
/* out[rows] = index of the largest logit, ties to the lowest id (python/mojolearn/models/causal_lm.py:190). */
int64_t b200i_argmax(int64_t device, void *stream, int32_t *out, const float *logits, int64_t rows, int64_t vocab, char *err,
                     int64_t err_cap);

/* --- exchange of finished output columns between the GPUs of one node ------------------------------
 * Output-column sharding (weight rows [r*N/g, (r+1)*N/g) on rank r, full k) needs the column slices
 * [m, N/g] of all ranks side by side as [m, N] on every rank. The reference's multi-device rule is
 * that such an exchange only copies finished words and never chooses an arithmetic order
 * (training/byte_lm_parallel.mojo:2-8, core/multi_gpu.mojo:46-50); this is that copy as one small
 * kernel per gather over peer-mapped memory instead of a collective library call. The owner of a
 * slice stores each word, paired with the step's epoch number in one 64-bit store, into a receive
 * area in every other rank's exchange buffer; the same kernel reads the areas the other ranks fill
 * in its own buffer, waiting (bounded: a word that has not arrived after 4 s sets status 8 of
 * b200i_decode_status) for each pair's tag, and writes the gathered matrix. One process per GPU,
 * all on one node.
 *   b200i_comm_create    allocates this rank's exchange buffer of `bytes` (zeroed) and returns an
 *                        opaque object in *comm.
 *   b200i_comm_export    writes the buffer's 64-byte CUDA IPC handle; the caller carries it to the
 *                        other processes (any host channel), which pass it to b200i_comm_attach.
 *                        After every rank attached every other rank, and before the first gather,
 *                        the caller runs a host barrier.
 *   b200i_comm_attach_local  the same for two exchanges inside one process on one device (tests).
 *   b200i_comm_advance   asynchronous on `stream`: starts a new epoch (one model step). Every rank
 *                        calls it once per step, before the step's first gather.
 *   b200i_comm_gather    asynchronous on `stream`: out[m, world * w] (row pitch out_ld floats, 0 =
 *                        world * w; caller-owned device memory) from this rank's src[m, w] (row pitch
 *                        src_ld, 0 = w) and the other ranks' slices. `area_bytes` places the gather's
 *                        receive areas (m * w * world * 8 bytes) in the exchange buffers; every rank
 *                        issues the same gathers in the same order with the same areas. Areas of
 *                        one step must not overlap, a step must have at least two gathers, and the
 *                        first gather's area must not overlap any other gather's of any step.
 *                        mode 0 = send and receive; 1 = send only; 2 = receive only (src ignored).
 *   b200i_comm_gather_nodes  the same gather for a slice that b200i_gemm_w_nodes left as `nodes`
 *                        (2 to 64) leaf-group nodes ws[nodes][m * n]: the kernel folds them in the
 *                        contract's order, applies the store epilogue (bias, act; a gated act halves
 *                        the slice's width w to n / 2) and sends the finished words. n a multiple of
 *                        4; mode 0 or 1. Bitwise the result of the finished product followed by
 *                        b200i_comm_gather, in one launch instead of two.
 *   b200i_comm_destroy   after a host barrier: unmaps the peers and frees the buffer. */
int64_t b200i_comm_create(int64_t device, int64_t rank, int64_t world, int64_t bytes, void **comm, char *err, int64_t err_cap);
int64_t b200i_comm_export(void *comm, void *handle, int64_t handle_bytes, char *err, int64_t err_cap);
int64_t b200i_comm_attach(void *comm, int64_t peer, const void *handle, char *err, int64_t err_cap);
int64_t b200i_comm_attach_local(void *comm, int64_t peer, void *other, char *err, int64_t err_cap);
int64_t b200i_comm_advance(void *comm, void *stream, char *err, int64_t err_cap);
int64_t b200i_comm_gather(void *comm, void *stream, int64_t mode, int64_t area_bytes, float *out, int64_t out_ld, const float *src,
                          int64_t m, int64_t w, int64_t src_ld, char *err, int64_t err_cap);
int64_t b200i_comm_gather_nodes(void *comm, void *stream, int64_t mode, int64_t area_bytes, float *out, int64_t out_ld, const float *ws,
                                int64_t nodes, int64_t m, int64_t n, const float *bias, int64_t act, char *err, int64_t err_cap);
int64_t b200i_comm_destroy(void *comm);

/* Status word of the bounded device-side waits on `device` (synchronises the
 * device): 0 = no wait ever ran out; 1 / 2 = the decode plan's producer / a consumer
 * gave up waiting on a stage, 3 = the decode attention's value ring, 4 / 5 = the
 * packed plan's ring, 8 = a wait for a peer GPU's tagged words, 9 = the int8
 * tensor-core product's stage or completion barrier; -1 = the word could not be read. A nonzero word is
 * cleared by the read. A kernel whose wait ran out skips its stores, so its output
 * is incomplete. The b200i_host_* calls read the word after their final
 * synchronise and return status 1 with a message, like any other error (the
 * reference's status + message buffer, adapters/native/c_api.mojo:64-72). The
 * device-pointer calls are asynchronous and cannot: their caller reads this word
 * when it next synchronises (mojolearn_b200.torch_ops.check_status, CausalLM.generate
 * and the decode sessions do). The reference has no device-side wait.
 * b200i_debug_set_status writes the word from the host, for tests of that reporting
 * path: no kernel is ever made to time out to produce a nonzero word. */
int64_t b200i_decode_status(int64_t device);
int64_t b200i_debug_set_status(int64_t device, int64_t value);

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
