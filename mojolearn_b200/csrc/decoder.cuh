// The decoder-block seams around the matrix product, as CUDA kernels.
//
// Each kernel spells exactly the reference's pinned seam (paths relative to the
// reference project's root; seam numbers from
// transformer/IDENTICAL_TRANSFORMER_CONTRACT.md:207-240):
//   norm_kernel          S1-S4 and the LayerNorm / offset variants, transformer/checks/transformer_oracle.mojo:1223-1341
//   rope_table_kernel    S6-S8, transformer/checks/transformer_oracle.mojo:539-640
//   rope_apply_kernel    S9-S10 (halves pairing, three roundings), :1375-1500
//   attn_scores_kernel   S11 (gemm fp32.v1 cells, k = head_dim, one leaf), S12 scale, S13 mask ADD, :2230-2372
//   attn_context_kernel  S14 row max (order free), S15-S16 exp, S17 serial denominator, S18 one division per
//                        weight, S19 serial value sum (NOT a GEMM), :2373-2472 and core/host_lanes.mojo:271-330
//   act_mul_kernel       S20-S21 and the GELU variants, :2580-2620
//   add_kernel           S22 / S23 residuals; bias_add_kernel :1344-1372
//   embedding_kernel     Y = ftz(W[id]), embedding/checks/embedding_oracle.mojo:369-382
//   argmax_kernel        greedy, ties to the lowest id, python/mojolearn/models/causal_lm.py:190
// Serial chains stay serial: the order of a chain is the contract, so the
// parallelism is across rows, heads and feature lanes, never inside a chain.
// These kernels are HBM- or latency-bound byte work around the GEMMs: coalesced
// 128-byte row segments, one warp per row or one thread per element, grids sized
// from the row count.
#pragma once
#include "decode.cuh" // mbarrier and bulk-copy primitives, the status word of the bounded waits
#include "seams_math.cuh"

namespace b200i {

constexpr int NORM_RMS = 0, NORM_LAYER = 1, NORM_RMS_OFFSET = 2;
constexpr int ACT_SWIGLU = 0, ACT_GELU_ERF = 1, ACT_GELU_TANH = 2, ACT_SILU = 3, ACT_GEGLU_ERF = 4, ACT_GEGLU_TANH = 5;

// ---- normalisation: one warp per row -------------------------------------------------------
// The sum of squares (or of deviations) is ONE serial chain over the row.
//
// norm_rows_kernel stages the row in shared memory first (every load of the row in
// flight at once, 128-bit where the row allows), then every lane runs the same
// chain on 128-bit broadcast reads: one dependent fma per element and nothing else
// on the critical path. norm_kernel is the same arithmetic for rows too wide for
// shared memory, the values broadcast by shuffle.
//
// Admission for the sum of squares: with every nonzero term at or above 2^-63 in
// magnitude each square is a normal number, the accumulator only grows, and no
// step result can be subnormal, so the bare fma is the contract's step.
#ifdef B200I_SABOTAGE_ADMIT_ALWAYS
constexpr unsigned NORM_ADMIT_MIN = 0u;
#else
constexpr unsigned NORM_ADMIT_MIN = (64u << 24) - 2u;
#endif
// With `delta` the row normalised is the residual sum ftz(ftz(src) + ftz(delta)) (seam S22 / S23), which is
// also written to `sum_out`: the residual add and the norm that always follows it, in one pass over the row.
constexpr int NORM_WREG = 16; // 128-bit words of the weight row a lane can hold: rows up to 2048 wide
__global__ void __launch_bounds__(128) norm_rows_kernel(float *__restrict__ out, const float *__restrict__ src, const float *__restrict__ w,
                                                        const float *__restrict__ bias, long long rows, int dm, float eps, int kind,
                                                        const float *__restrict__ delta, float *__restrict__ sum_out) {
    extern __shared__ __align__(16) float norm_smem[];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const long long row = (long long)blockIdx.x * (blockDim.x >> 5) + warp;
    if (row >= rows) return; // warps are independent: only warp-level barriers below
    // The weight row does not depend on the chain: a lane asks for its words of it before anything else, so that the
    // last phase finds them in registers instead of paying a round trip to L2 per 512 columns after the chain.
    const bool w_early = (dm % 4 == 0) && dm <= NORM_WREG * 128 && ((reinterpret_cast<uintptr_t>(w) & 15) == 0);
    float4 wreg[NORM_WREG];
    if (w_early) {
#pragma unroll
        for (int u = 0; u < NORM_WREG; u++)
            wreg[u] = (lane * 4 + u * 128 < dm) ? __ldg(reinterpret_cast<const float4 *>(w + lane * 4 + u * 128)) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
    const int pitch = (dm + 3) & ~3;
    float *xs = norm_smem + (size_t)warp * pitch;
    const float *x = src + row * dm;
    const float *dl = delta ? delta + row * dm : nullptr;
    float *so = sum_out ? sum_out + row * dm : nullptr;
    const bool vec = (dm % 4 == 0) && ((reinterpret_cast<uintptr_t>(x) & 15) == 0) &&
                     (!dl || ((reinterpret_cast<uintptr_t>(dl) & 15) == 0 && (reinterpret_cast<uintptr_t>(so) & 15) == 0));
    unsigned key = 0xFFFFFFFFu;
    if (vec) {
        // eight 128-bit loads per lane in flight: a lone warp has no other warp to hide a load behind
        for (int j0 = lane * 4; j0 < dm; j0 += 8 * 128) {
            float4 v[8];
#pragma unroll
            for (int u = 0; u < 8; u++)
                v[u] = (j0 + u * 128 < dm) ? *reinterpret_cast<const float4 *>(x + j0 + u * 128) : make_float4(0.f, 0.f, 0.f, 0.f);
            if (dl) {
                float4 d[8];
#pragma unroll
                for (int u = 0; u < 8; u++)
                    d[u] = (j0 + u * 128 < dm) ? *reinterpret_cast<const float4 *>(dl + j0 + u * 128) : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
                for (int u = 0; u < 8; u++) {
                    v[u].x = __fadd_rn(ftz_bits(v[u].x), ftz_bits(d[u].x)); v[u].y = __fadd_rn(ftz_bits(v[u].y), ftz_bits(d[u].y));
                    v[u].z = __fadd_rn(ftz_bits(v[u].z), ftz_bits(d[u].z)); v[u].w = __fadd_rn(ftz_bits(v[u].w), ftz_bits(d[u].w));
                }
            }
#pragma unroll
            for (int u = 0; u < 8; u++) {
                if (j0 + u * 128 >= dm) break;
                v[u].x = ftz_bits(v[u].x); v[u].y = ftz_bits(v[u].y); v[u].z = ftz_bits(v[u].z); v[u].w = ftz_bits(v[u].w);
                key = min(min(key, admit_key(v[u].x)), min(admit_key(v[u].y), min(admit_key(v[u].z), admit_key(v[u].w))));
                *reinterpret_cast<float4 *>(xs + j0 + u * 128) = v[u];
                if (so) *reinterpret_cast<float4 *>(so + j0 + u * 128) = v[u];
            }
        }
    } else {
        for (int j = lane; j < dm; j += 32) {
            float v = ftz_bits(x[j]);
            if (dl) v = ftz_bits(__fadd_rn(v, ftz_bits(dl[j])));
            key = min(key, admit_key(v));
            xs[j] = v;
            if (so) so[j] = v;
        }
    }
    for (int j = dm + lane; j < pitch; j += 32) xs[j] = 0.f;
    __syncwarp();
    const int dm4 = dm & ~3;
    if (kind == NORM_LAYER) {
        float acc = 0.f;
#pragma unroll 4
        for (int j = 0; j < dm4; j += 4) {
            const float4 v = *reinterpret_cast<const float4 *>(xs + j);
            acc = add_flushed(add_flushed(add_flushed(add_flushed(acc, v.x), v.y), v.z), v.w);
        }
        for (int j = dm4; j < dm; j++) acc = add_flushed(acc, xs[j]);
        const float mean = ftz_bits(p_divf(acc, (float)dm));
        __syncwarp();
        key = 0xFFFFFFFFu;
        for (int j = lane; j < dm; j += 32) {
            const float v = ftz_bits(__fsub_rn(xs[j], mean));
            key = min(key, admit_key(v));
            xs[j] = v;
        }
        __syncwarp();
    }
    const bool bare = __all_sync(0xFFFFFFFFu, key >= NORM_ADMIT_MIN);
    float acc = 0.f;
    if (bare) {
#pragma unroll 4
        for (int j = 0; j < dm4; j += 4) {
            const float4 v = *reinterpret_cast<const float4 *>(xs + j);
            acc = step_bare(v.x, v.x, acc);
            acc = step_bare(v.y, v.y, acc);
            acc = step_bare(v.z, v.z, acc);
            acc = step_bare(v.w, v.w, acc);
        }
        for (int j = dm4; j < dm; j++) acc = step_bare(xs[j], xs[j], acc);
    } else {
#pragma unroll 2
        for (int j = 0; j < dm4; j += 4) {
            const float4 v = *reinterpret_cast<const float4 *>(xs + j);
            acc = step_flush(v.x, v.x, acc);
            acc = step_flush(v.y, v.y, acc);
            acc = step_flush(v.z, v.z, acc);
            acc = step_flush(v.w, v.w, acc);
        }
        for (int j = dm4; j < dm; j++) acc = step_flush(xs[j], xs[j], acc);
    }
    const float var = ftz_bits(p_divf(acc, (float)dm));
    const float rstd = ftz_bits(p_rsqrtf(ftz_bits(__fadd_rn(var, eps))));
    auto finish = [&](float xv, float wv, float bv) {
        const float inner = ftz_bits(__fmul_rn(xv, rstd));
        float wj = ftz_bits(wv);
        if (kind == NORM_RMS_OFFSET) wj = ftz_bits(__fadd_rn(1.0f, wj));
        float y = ftz_bits(__fmul_rn(wj, inner));
        if (kind == NORM_LAYER && bias) y = ftz_bits(__fadd_rn(y, ftz_bits(bv)));
        return y;
    };
    const bool vec_out = vec && ((reinterpret_cast<uintptr_t>(w) & 15) == 0) && ((reinterpret_cast<uintptr_t>(out) & 15) == 0) &&
                         (!bias || (reinterpret_cast<uintptr_t>(bias) & 15) == 0);
    if (vec_out) {
        const bool has_bias = kind == NORM_LAYER && bias;
        auto finish4 = [&](int j, const float4 wq, const float4 bq) {
            const float4 xv = *reinterpret_cast<const float4 *>(xs + j);
            float4 y;
            y.x = finish(xv.x, wq.x, bq.x); y.y = finish(xv.y, wq.y, bq.y);
            y.z = finish(xv.z, wq.z, bq.z); y.w = finish(xv.w, wq.w, bq.w);
            *reinterpret_cast<float4 *>(out + row * dm + j) = y;
        };
        const float4 zero4 = make_float4(0.f, 0.f, 0.f, 0.f);
        if (w_early && !has_bias) { // the weights are already in registers
#pragma unroll
            for (int u = 0; u < NORM_WREG; u++) {
                const int j = lane * 4 + u * 128;
                if (j < dm) finish4(j, wreg[u], zero4);
            }
        } else {
            for (int j0 = lane * 4; j0 < dm; j0 += 4 * 128) {
                float4 wv[4], bv[4];
#pragma unroll
                for (int u = 0; u < 4; u++) {
                    const bool in = j0 + u * 128 < dm;
                    wv[u] = in ? *reinterpret_cast<const float4 *>(w + j0 + u * 128) : zero4;
                    bv[u] = (in && has_bias) ? *reinterpret_cast<const float4 *>(bias + j0 + u * 128) : zero4;
                }
#pragma unroll
                for (int u = 0; u < 4; u++) {
                    const int j = j0 + u * 128;
                    if (j >= dm) break;
                    finish4(j, wv[u], bv[u]);
                }
            }
        }
    } else {
        for (int j = lane; j < dm; j += 32) out[row * dm + j] = finish(xs[j], w[j], (kind == NORM_LAYER && bias) ? bias[j] : 0.f);
    }
}

__global__ void norm_kernel(float *__restrict__ out, const float *__restrict__ src, const float *__restrict__ w,
                            const float *__restrict__ bias, long long rows, int dm, float eps, int kind) {
    const int lane = threadIdx.x & 31;
    const long long row = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    if (row >= rows) return;
    const float *x = src + row * dm;
    float mean = 0.f;
    if (kind == NORM_LAYER) {
        float acc = 0.f;
        for (int j0 = 0; j0 < dm; j0 += 32) {
            const float mine = (j0 + lane < dm) ? ftz_bits(x[j0 + lane]) : 0.f;
            if (j0 + 32 <= dm) {
#pragma unroll
                for (int j = 0; j < 32; j++) acc = add_flushed(acc, __shfl_sync(0xFFFFFFFFu, mine, j));
            } else {
                for (int j = 0; j < dm - j0; j++) acc = add_flushed(acc, __shfl_sync(0xFFFFFFFFu, mine, j));
            }
        }
        mean = ftz_bits(p_divf(acc, (float)dm));
    }
    unsigned key = 0xFFFFFFFFu;
    for (int j = lane; j < dm; j += 32) {
        float v = ftz_bits(x[j]);
        if (kind == NORM_LAYER) v = ftz_bits(__fsub_rn(v, mean));
        key = min(key, admit_key(v));
    }
    const bool bare = __all_sync(0xFFFFFFFFu, key >= NORM_ADMIT_MIN);
    float acc = 0.f;
    for (int j0 = 0; j0 < dm; j0 += 32) {
        float mine = (j0 + lane < dm) ? ftz_bits(x[j0 + lane]) : 0.f;
        if (kind == NORM_LAYER) mine = ftz_bits(__fsub_rn(mine, mean));
        if (j0 + 32 <= dm && bare) {
#pragma unroll
            for (int j = 0; j < 32; j++) {
                const float v = __shfl_sync(0xFFFFFFFFu, mine, j);
                acc = step_bare(v, v, acc);
            }
        } else {
            const int cnt = min(32, dm - j0);
            for (int j = 0; j < cnt; j++) {
                const float v = __shfl_sync(0xFFFFFFFFu, mine, j);
                acc = step_flush(v, v, acc);
            }
        }
    }
    const float var = ftz_bits(p_divf(acc, (float)dm));
    const float rstd = ftz_bits(p_rsqrtf(ftz_bits(__fadd_rn(var, eps))));
    for (int j = lane; j < dm; j += 32) {
        float v = ftz_bits(x[j]);
        if (kind == NORM_LAYER) v = ftz_bits(__fsub_rn(v, mean));
        const float inner = ftz_bits(__fmul_rn(v, rstd));
        float wj = ftz_bits(w[j]);
        if (kind == NORM_RMS_OFFSET) wj = ftz_bits(__fadd_rn(1.0f, wj));
        float y = ftz_bits(__fmul_rn(wj, inner));
        if (kind == NORM_LAYER && bias) y = ftz_bits(__fadd_rn(y, ftz_bits(bias[j])));
        out[row * dm + j] = y;
    }
}

// ---- rotary table and application -----------------------------------------------------------
// The option record of the rotary table (transformer/block_options.mojo:40-70 of the reference): scaling 0 none,
// 1 linear (one division of the inverse frequency by the factor), 2 llama3 (rescaling by wavelength), spelled as
// transformer/checks/transformer_oracle.mojo:423-497: every division the portable one, both products of the
// interpolation rounded on their own, the final add unfused. `rope_dim` = rotated columns of a head.
struct RopeOptions {
    float theta;
    int scaling;
    float factor, low_freq_factor, high_freq_factor;
    int original_max_positions;
};
__device__ __forceinline__ float rope_inv_freq(int i, int rope_dim, const RopeOptions &o) {
    const float e = ftz_bits(p_divf((float)(2 * i), (float)rope_dim));
    float inv = ftz_bits(p_divf(1.0f, p_powf(o.theta, e)));
    if (o.scaling == 1) {
        inv = ftz_bits(p_divf(inv, ftz_bits(o.factor)));
    } else if (o.scaling == 2) {
        const float factor = ftz_bits(o.factor), lo_f = ftz_bits(o.low_freq_factor), hi_f = ftz_bits(o.high_freq_factor);
        const float old = (float)o.original_max_positions;
        const float low_wl = ftz_bits(p_divf(old, lo_f)), high_wl = ftz_bits(p_divf(old, hi_f));
        const float wl = ftz_bits(p_divf(__uint_as_float(0x40C90FDBu), inv)); // 2 pi
        float inv_l = inv;
        if (wl > low_wl) inv_l = ftz_bits(p_divf(inv, factor));
        if (!(wl < high_wl) && !(wl > low_wl)) {
            const float ratio = ftz_bits(p_divf(old, wl));
            const float num = ftz_bits(__fsub_rn(ratio, lo_f)), den = ftz_bits(__fsub_rn(hi_f, lo_f));
            const float smooth = ftz_bits(p_divf(num, den));
            const float one_minus = ftz_bits(__fsub_rn(1.0f, smooth));
            float t1 = ftz_bits(__fmul_rn(one_minus, inv_l));
            t1 = ftz_bits(p_divf(t1, factor));
            const float t2 = ftz_bits(__fmul_rn(smooth, inv_l));
            inv_l = ftz_bits(__fadd_rn(ftz_bits(t1), ftz_bits(t2)));
        }
        inv = inv_l;
    }
    return inv;
}
__global__ void rope_table_opts_kernel(float *__restrict__ cosv, float *__restrict__ sinv, int pos0, int l, int rope_dim, RopeOptions o,
                                       const int *__restrict__ pos_dev) {
    if (pos_dev) pos0 = *pos_dev;
    const int half = rope_dim / 2;
    const int idx = blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= l * half) return;
    const int p = idx / half, i = idx % half;
    const float inv = rope_inv_freq(i, rope_dim, o);
    const float angle = ftz_bits(__fmul_rn((float)(pos0 + p), ftz_bits(inv)));
    cosv[idx] = ftz_bits(p_cosf(angle));
    sinv[idx] = ftz_bits(p_sinf(angle));
}

__global__ void rope_table_kernel(float *__restrict__ cosv, float *__restrict__ sinv, int pos0, int l, int head_dim,
                                  float theta, const int *__restrict__ pos_dev) {
    if (pos_dev) pos0 = *pos_dev;
    const int half = head_dim / 2;
    const int idx = blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= l * half) return;
    const int p = idx / half, i = idx % half;
    const float e = ftz_bits(p_divf((float)(2 * i), (float)head_dim));
    const float inv = ftz_bits(p_divf(1.0f, p_powf(theta, e)));
    const float angle = ftz_bits(__fmul_rn((float)(pos0 + p), ftz_bits(inv)));
    cosv[idx] = ftz_bits(p_cosf(angle));
    sinv[idx] = ftz_bits(p_sinf(angle));
}

// `ld` is the row pitch of src in floats (the projections may be column blocks of one fused product).
__global__ void rope_apply_kernel(float *__restrict__ out, const float *__restrict__ src, const float *__restrict__ cosv,
                                  const float *__restrict__ sinv, long long m, int l, int n_head, int hd, long long ld, int rd) {
    // rd = rotated columns of a head (partial rotary, transformer_oracle.mojo:1433-1440): the rest pass through, flushed
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    const long long width = (long long)n_head * hd;
    if (idx >= m * width) return;
    const long long t = idx / width, si = t * ld + idx % width;
    const int j = (int)(idx % hd), half = rd / 2, li = (int)(t % l);
    if (j >= rd) { out[idx] = ftz_bits(src[si]); return; }
    const int ci = j < half ? j : j - half;
    const float partner = j < half ? -ftz_bits(src[si + half]) : ftz_bits(src[si - half]);
    const float c = ftz_bits(cosv[li * half + ci]), s = ftz_bits(sinv[li * half + ci]);
    const float pa = ftz_bits(__fmul_rn(ftz_bits(src[si]), c));
    const float pb = ftz_bits(__fmul_rn(partner, s));
    out[idx] = ftz_bits(__fadd_rn(pa, pb));
}

// KV cache append: a copy, not a seam. cache is [b, n_kv, cap, hd]; src is [b*l, n_kv*hd] with row pitch ld.
__global__ void kv_append_kernel(float *__restrict__ cache, const float *__restrict__ src, int b, int l, int n_kv, int hd,
                                 int cap, int pos0, const int *__restrict__ pos_dev, long long ld) {
    if (pos_dev) pos0 = *pos_dev;
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    const long long total = (long long)b * l * n_kv * hd;
    if (idx >= total) return;
    const int d = (int)(idx % hd);
    const int kv = (int)((idx / hd) % n_kv);
    const long long t = idx / ((long long)hd * n_kv);
    const int bb = (int)(t / l), li = (int)(t % l);
    if (pos0 + li >= cap) return; // the host refuses such a call; a replayed graph must not write past the cache either
    cache[(((long long)bb * n_kv + kv) * cap + pos0 + li) * hd + d] = src[t * ld + (long long)kv * hd + d];
}

// One pass over the fresh q | k | v rows of a call: q rotated into `qr` (contiguous), k rotated straight into its
// cache slot, v copied into its cache slot. The arithmetic per element is rope_apply_kernel's (S9-S10) and the
// placement kv_append_kernel's; `rope` = 0 copies q and k unrotated. q has row pitch ldq, k and v ldkv.
__global__ void qkv_rope_cache_kernel(float *__restrict__ qr, float *__restrict__ kcache, float *__restrict__ vcache,
                                      const float *__restrict__ q, const float *__restrict__ k, const float *__restrict__ v,
                                      long long ldq, long long ldkv, const float *__restrict__ cosv, const float *__restrict__ sinv, int b, int l,
                                      int nh, int nkv, int hd, int cap, int pos0, const int *__restrict__ pos_dev, int rope, int rd) {
    if (pos_dev) pos0 = *pos_dev;
    const long long wq = (long long)nh * hd, wk = (long long)nkv * hd, per_row = wq + 2 * wk;
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (long long)b * l * per_row) return;
    const long long t = idx / per_row;
    const long long c = idx % per_row;
    const int li = (int)(t % l), bb = (int)(t / l), half = rd / 2;
    const float *src = c < wq ? q : (c < wq + wk ? k : v);
    const long long col = c < wq ? c : (c < wq + wk ? c - wq : c - wq - wk);
    const long long si = t * (c < wq ? ldq : ldkv) + col;
    const int j = (int)(col % hd);
    float val;
    if (c < wq + wk && rope && j >= rd) {
        val = ftz_bits(src[si]); // partial rotary: a column past the rotated ones passes through, flushed on load
    } else if (c < wq + wk && rope) {
        const int ci = j < half ? j : j - half;
        const float partner = j < half ? -ftz_bits(src[si + half]) : ftz_bits(src[si - half]);
        const float cs = ftz_bits(cosv[li * half + ci]), sn = ftz_bits(sinv[li * half + ci]);
        const float pa = ftz_bits(__fmul_rn(ftz_bits(src[si]), cs));
        const float pb = ftz_bits(__fmul_rn(partner, sn));
        val = ftz_bits(__fadd_rn(pa, pb));
    } else {
        val = src[si];
    }
    if (c < wq) {
        qr[t * wq + col] = val;
    } else {
        if (pos0 + li >= cap) return; // the host refuses such a call; a replayed graph must not write past the cache either
        float *cache = c < wq + wk ? kcache : vcache;
        const int kv = (int)(col / hd);
        cache[(((long long)bb * nkv + kv) * cap + pos0 + li) * hd + j] = val;
    }
}

// ---- a position read on the device ------------------------------------------------------------
// A decode step replayed from a captured graph cannot take its position as a launch
// argument. Every kernel that depends on the number of cached tokens therefore also
// accepts `pos_dev`, a device word holding it; when it is not null it overrides the
// by-value arguments, and the key range of the attention kernels is derived from it
// exactly as the host derives it (pos0 = cached tokens before this call).
__device__ __forceinline__ void attn_geometry(const int *pos_dev, int l, int cap, int window, int &key_lo, int &s, int &own0) {
    if (!pos_dev) return;
    const int pos0 = *pos_dev;
    int used = pos0 + l;
    if (used > cap) used = cap;
    key_lo = (window > 0 && pos0 - (window - 1) > 0) ? pos0 - (window - 1) : 0;
    s = used - key_lo;
    own0 = pos0 - key_lo;
}
__global__ void advance_position_kernel(int *pos_dev, int delta) { *pos_dev += delta; }


// Score seams S12 (scale) and the optional soft cap between it and the mask (transformer_oracle.mojo:2269-2281,
// Gemma 2's attn_logit_softcapping): cap * tanh(score / cap), one portable division, one portable tanh and one
// product, each flushed. `softcap` 0 (all bits) = none.
__device__ __forceinline__ float score_scale_cap(float dot, float scale, float softcap) {
    float sc = ftz_bits(__fmul_rn(ftz_hw(dot), scale));
    if (__float_as_uint(softcap) != 0u) {
        const float cap = ftz_bits(softcap);
        const float th = ftz_bits(p_tanhf(ftz_bits(p_divf(sc, cap))));
        sc = ftz_bits(__fmul_rn(th, cap));
    }
    return sc;
}

// ---- attention scores -------------------------------------------------------------------------
// scores[b, h, qi, j] = ftz(ftz(ftz(q . k) * scale) + fill), the dot being one
// gemm fp32.v1 leaf (k = head_dim <= 128: a single serial chain from +0.0).
// A CTA owns a 64 x 64 tile of one (batch, head); a thread owns 4 x 4 cells.
constexpr int ATT_T = 64, ATT_KC = 32;
__global__ void __launch_bounds__(256) attn_scores_kernel(float *__restrict__ scores, const float *__restrict__ q,
                                                          const float *__restrict__ kcache, int b, int l, int nh, int nkv, int hd,
                                                          int cap, int key_lo, int s, int own0, int window,
                                                          const int *__restrict__ pos_dev, float softcap) {
    attn_geometry(pos_dev, l, cap, window, key_lo, s, own0);
    if ((int)blockIdx.x * ATT_T >= s) return;
    // the attention scale, ftz(rsqrt(head_dim)) in the portable spelling: a pure function of head_dim
    const float scale = ftz_bits(p_rsqrtf((float)hd));
    __shared__ __align__(16) float qs[ATT_KC][ATT_T + 4]; // pitch 68 words: rows stay 16-byte aligned
    __shared__ __align__(16) float ks[ATT_KC][ATT_T + 4];
    const int bh = blockIdx.z, bb = bh / nh, h = bh % nh, kv = h / (nh / nkv);
    const int q0 = blockIdx.y * ATT_T, j0 = blockIdx.x * ATT_T;
    const int tid = threadIdx.x, tx = tid % 16, ty = tid / 16;
    const long long qw = (long long)nh * hd;
    const float *qbase = q + ((long long)bb * l) * qw + (long long)h * hd;
    const float *kbase = kcache + (((long long)bb * nkv + kv) * cap + key_lo) * hd;
    const float mfill = __uint_as_float(0xFF7FFFFFu);
    // A tile no query of which can see any of its keys: every cell is ftz(score + (-FLT_MAX)). When every
    // operand word of the tile is finite and below 2^40 in magnitude, |score| < 2^88 is under half an ulp of
    // FLT_MAX (2^103), so the sum IS -FLT_MAX and the dot products need not be formed.
    const int q_hi = min(q0 + ATT_T, l) - 1;
    // (with a soft cap the scores are bounded by the cap instead; the shortcut is simply not taken then)
    const bool tile_masked = __float_as_uint(softcap) == 0u &&
                             (j0 > own0 + q_hi || (window > 0 && j0 + ATT_T - 1 < own0 + q0 - window + 1));
    if (tile_masked) {
        bool small = true;
        const int warp = tid >> 5, lane = tid & 31;
        const bool vec = (hd % 4 == 0) && (((reinterpret_cast<uintptr_t>(qbase) | reinterpret_cast<uintptr_t>(kbase)) & 15u) == 0);
        for (int r = warp; r < ATT_T; r += 8) { // a warp per row, lanes along the row: no division by head_dim
            const float *qr = qbase + (long long)(q0 + r) * qw, *kr = kbase + (long long)(j0 + r) * hd;
            const bool qlive = q0 + r < l, klive = j0 + r < s;
            if (vec) {
                for (int p = lane * 4; p < hd; p += 128) {
                    if (qlive) {
                        const float4 v = *reinterpret_cast<const float4 *>(qr + p);
                        small = small && ((__float_as_uint(v.x) >> 23) & 0xFFu) < 167u && ((__float_as_uint(v.y) >> 23) & 0xFFu) < 167u &&
                                ((__float_as_uint(v.z) >> 23) & 0xFFu) < 167u && ((__float_as_uint(v.w) >> 23) & 0xFFu) < 167u;
                    }
                    if (klive) {
                        const float4 v = *reinterpret_cast<const float4 *>(kr + p);
                        small = small && ((__float_as_uint(v.x) >> 23) & 0xFFu) < 167u && ((__float_as_uint(v.y) >> 23) & 0xFFu) < 167u &&
                                ((__float_as_uint(v.z) >> 23) & 0xFFu) < 167u && ((__float_as_uint(v.w) >> 23) & 0xFFu) < 167u;
                    }
                }
            } else {
                for (int p = lane; p < hd; p += 32) {
                    if (qlive) small = small && ((__float_as_uint(qr[p]) >> 23) & 0xFFu) < 167u;
                    if (klive) small = small && ((__float_as_uint(kr[p]) >> 23) & 0xFFu) < 167u;
                }
            }
        }
        if (__syncthreads_and(small)) {
#pragma unroll
            for (int i = 0; i < 4; i++) {
                const int qi = q0 + ty * 4 + i;
                if (qi >= l) continue;
#pragma unroll
                for (int jj = 0; jj < 4; jj++) {
                    const int j = j0 + tx * 4 + jj;
                    if (j < s) scores[((long long)bh * l + qi) * s + j] = mfill;
                }
            }
            return;
        }
    }
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; i++)
#pragma unroll
        for (int j = 0; j < 4; j++) acc[i][j] = 0.f;
    bool clean = true; // every chunk so far passed admission: the chains have only taken bare steps
    for (int p0 = 0; p0 < hd; p0 += ATT_KC) {
        unsigned key = 0xFFFFFFFFu;
        for (int idx = tid; idx < ATT_T * ATT_KC; idx += 256) {
            const int r = idx / ATT_KC, p = idx % ATT_KC;
            const bool pk = p0 + p < hd;
            const float qv = (pk && q0 + r < l) ? ftz_bits(qbase[(long long)(q0 + r) * qw + p0 + p]) : 0.f;
            const float kvv = (pk && j0 + r < s) ? ftz_bits(kbase[(long long)(j0 + r) * hd + p0 + p]) : 0.f;
            key = min(key, min(admit_key(qv), admit_key(kvv)));
            qs[p][r] = qv;
            ks[p][r] = kvv;
        }
        clean = __syncthreads_and(key >= ADMIT_MIN) && clean;
        const int pn = min(ATT_KC, hd - p0);
        if (clean) {
#pragma unroll 8
            for (int p = 0; p < pn; p++) {
                const float4 a4 = *reinterpret_cast<const float4 *>(&qs[p][ty * 4]);
                const float4 c4 = *reinterpret_cast<const float4 *>(&ks[p][tx * 4]);
                const float a[4] = {a4.x, a4.y, a4.z, a4.w}, c[4] = {c4.x, c4.y, c4.z, c4.w};
#pragma unroll
                for (int i = 0; i < 4; i++)
#pragma unroll
                    for (int j = 0; j < 4; j++) acc[i][j] = step_bare(a[i], c[j], acc[i][j]);
            }
        } else {
            for (int p = 0; p < pn; p++) {
                const float4 a4 = *reinterpret_cast<const float4 *>(&qs[p][ty * 4]);
                const float4 c4 = *reinterpret_cast<const float4 *>(&ks[p][tx * 4]);
                const float a[4] = {a4.x, a4.y, a4.z, a4.w}, c[4] = {c4.x, c4.y, c4.z, c4.w};
#pragma unroll
                for (int i = 0; i < 4; i++)
#pragma unroll
                    for (int j = 0; j < 4; j++) acc[i][j] = step_flush(a[i], c[j], acc[i][j]);
            }
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const int qi = q0 + ty * 4 + i;
        if (qi >= l) continue;
        int jlo = 0, jhi = own0 + qi;
        if (jhi > s - 1) jhi = s - 1;
        if (window > 0) { jlo = own0 + qi - window + 1; if (jlo < 0) jlo = 0; }
#pragma unroll
        for (int jj = 0; jj < 4; jj++) {
            const int j = j0 + tx * 4 + jj;
            if (j >= s) continue;
            const float sc = score_scale_cap(acc[i][jj], scale, softcap);
            const float fill = (j < jlo || j > jhi) ? mfill : 0.0f;
            scores[((long long)bh * l + qi) * s + j] = ftz_bits(__fadd_rn(sc, fill));
        }
    }
}

// ---- asynchronous copies into shared memory (cp.async): no register staging, so the bytes a
// warp keeps in flight are bounded by shared memory, not by registers.
__device__ __forceinline__ void cp_async16(void *smem, const void *gmem) {
    const unsigned dst = (unsigned)__cvta_generic_to_shared(smem);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(gmem) : "memory");
}
__device__ __forceinline__ void cp_async8(void *smem, const void *gmem) {
    const unsigned dst = (unsigned)__cvta_generic_to_shared(smem);
    asm volatile("cp.async.ca.shared.global [%0], [%1], 8;" ::"r"(dst), "l"(gmem) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }
// `count` floats, contiguous on both sides, by the threads t, t + nthreads, ...; head_dim is
// even, so every row starts on 8 bytes, and on 16 when head_dim is a multiple of 4
__device__ __forceinline__ void cp_async_floats(float *dst, const float *src, int count, bool vec16, int t, int nthreads) {
    if (vec16) {
        for (int c = t * 4; c < count; c += nthreads * 4) cp_async16(dst + c, src + c);
    } else {
        for (int c = t * 2; c < count; c += nthreads * 2) cp_async8(dst + c, src + c);
    }
}
__device__ __forceinline__ unsigned key_of4(float4 v) {
    return min(min(admit_key(v.x), admit_key(v.y)), min(admit_key(v.z), admit_key(v.w)));
}

// The same scores for a handful of query rows (a decode step): one lane per key, one
// serial chain per (query, key) over head_dim. A warp copies the cache rows of its 32
// keys (16 KB at head_dim 128) straight into padded shared memory with cp.async, all
// of them in flight at once, then lane j walks row j with 128-bit reads (the padding
// makes them conflict-free). LQ is the query-row count rounded up to a power of two,
// a template parameter so that absent rows cost no issue slots. The chain first runs
// the bare fma while folding the admission key of what it reads; a lane whose row (or
// the query) fails the product's admission test walks its chain again with the
// flushed step, which is the contract's spelling for any operands.
constexpr int ATT_SMALL_Q = 8, ATT_KT_PITCH = K_LEAF_MIN + 4;
template <int LQ>
constexpr int attn_scores_small_smem() { return (LQ * K_LEAF_MIN + 4 * 32 * ATT_KT_PITCH) * (int)sizeof(float); }
template <int LQ>
__global__ void __launch_bounds__(128) attn_scores_small_kernel(float *__restrict__ scores, const float *__restrict__ q,
                                                                const float *__restrict__ kcache, int b, int l, int nh, int nkv,
                                                                int hd, int cap, int key_lo, int s, int own0, int window,
                                                                const int *__restrict__ pos_dev, float softcap) {
    attn_geometry(pos_dev, l, cap, window, key_lo, s, own0);
    if ((int)blockIdx.x * 128 >= s) return;
    extern __shared__ __align__(16) float att_smem[];
    float (*qs)[K_LEAF_MIN] = reinterpret_cast<float (*)[K_LEAF_MIN]>(att_smem);
    const int bh = blockIdx.y, bb = bh / nh, h = bh % nh, kv = h / (nh / nkv);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    float (*kt)[ATT_KT_PITCH] = reinterpret_cast<float (*)[ATT_KT_PITCH]>(att_smem + LQ * K_LEAF_MIN) + warp * 32;
    const int j0 = blockIdx.x * 128 + warp * 32;
    const bool vec16 = (hd % 4) == 0;
    const float *kbase = kcache + (((long long)bb * nkv + kv) * cap + key_lo) * hd;
    const int rows = min(32, s - j0); // keys of this warp that exist (uniform across the warp; may be <= 0)
    if (vec16) {
        // one instruction per cache row: lane t moves the 16 bytes at float 4t of the row
        const float *src = kbase + (long long)j0 * hd + lane * 4;
        float *dst = &kt[0][lane * 4];
        if (lane * 4 < hd) {
            if (rows == 32) {
#pragma unroll
                for (int r = 0; r < 32; r++) cp_async16(dst + r * ATT_KT_PITCH, src + (long long)r * hd);
            } else {
                for (int r = 0; r < rows; r++) cp_async16(dst + r * ATT_KT_PITCH, src + (long long)r * hd);
            }
        }
    } else {
        for (int r = 0; r < rows; r++) cp_async_floats(&kt[r][0], kbase + (long long)(j0 + r) * hd, hd, false, lane, 32);
    }
    for (int r = max(rows, 0); r < 32; r++)
        for (int c = lane; c < hd; c += 32) kt[r][c] = 0.f;
    cp_async_commit();
    __shared__ float scale_s;
    if (threadIdx.x == 0) scale_s = ftz_bits(p_rsqrtf((float)hd)); // a pure function of head_dim: one thread spells it
    const long long qw = (long long)nh * hd;
    unsigned qkey = 0xFFFFFFFFu;
    for (int idx = threadIdx.x; idx < LQ * hd; idx += 128) {
        const int i = idx / hd, p = idx % hd;
        const float v = i < l ? ftz_bits(q[((long long)bb * l + i) * qw + (long long)h * hd + p]) : 0.f;
        qkey = min(qkey, admit_key(v));
        qs[i][p] = v;
    }
    const bool q_ok = __syncthreads_and(qkey >= ADMIT_MIN);
    const float scale = scale_s;
    cp_async_wait<0>();
    __syncwarp();
    const float *krow = &kt[lane][0];
    float acc[LQ];
    bool exact = false;
    if (q_ok && vec16) {
        unsigned kkey = 0xFFFFFFFFu;
#pragma unroll
        for (int i = 0; i < LQ; i++) acc[i] = 0.f;
#pragma unroll 8
        for (int p = 0; p < hd; p += 4) {
            const float4 kvv = *reinterpret_cast<const float4 *>(krow + p);
            kkey = min(kkey, key_of4(kvv));
#pragma unroll
            for (int i = 0; i < LQ; i++) {
                const float4 qv = *reinterpret_cast<const float4 *>(&qs[i][p]);
                acc[i] = step_bare(qv.x, kvv.x, acc[i]);
                acc[i] = step_bare(qv.y, kvv.y, acc[i]);
                acc[i] = step_bare(qv.z, kvv.z, acc[i]);
                acc[i] = step_bare(qv.w, kvv.w, acc[i]);
            }
        }
        exact = kkey >= ADMIT_MIN;
    }
    if (!exact) {
#pragma unroll
        for (int i = 0; i < LQ; i++) acc[i] = 0.f;
        for (int p = 0; p < hd; p++) {
            const float kvv = ftz_bits(krow[p]);
#pragma unroll
            for (int i = 0; i < LQ; i++) acc[i] = step_flush(qs[i][p], kvv, acc[i]);
        }
    }
    const int j = j0 + lane;
    if (j >= s) return;
    const float mfill = __uint_as_float(0xFF7FFFFFu);
#pragma unroll
    for (int i = 0; i < LQ; i++) {
        if (i >= l) break;
        int jlo = 0, jhi = own0 + i;
        if (jhi > s - 1) jhi = s - 1;
        if (window > 0) { jlo = own0 + i - window + 1; if (jlo < 0) jlo = 0; }
        const float sc = score_scale_cap(acc[i], scale, softcap);
        scores[((long long)bh * l + i) * s + j] = ftz_bits(__fadd_rn(sc, (j < jlo || j > jhi) ? mfill : 0.0f));
    }
}

// ---- softmax and value sum ----------------------------------------------------------------------
// A CTA owns 32 consecutive query rows of one (batch, head): eight warps of four rows.
// The masked scores are overwritten in place by exp(s - max) and then by the weights.
// Every chain of the seam stays serial per row; the four rows of a warp are four
// independent chains walked together, so a value word read from the staged tile serves
// four rows and a 128-bit broadcast read delivers the four rows' weights of one key.
// A lane owns DPL consecutive features. A tile of 32 keys runs the bare fma when the
// staged values and the four rows' weights pass admission and no earlier tile of the
// warp needed the flushed step (a flushed accumulator need not be a multiple of 2^-126).
constexpr int CTX_WARPS = 8, CTX_RPW = 4, CTX_ROWS = CTX_WARPS * CTX_RPW, CTX_KT = 32, CTX_MAX_HD = 256;
inline size_t attn_context_smem(int hd) { return ((size_t)CTX_KT * hd + (size_t)CTX_KT * CTX_ROWS) * sizeof(float); }
// DPL = feature slots per lane (head_dim / 32 rounded up to 1, 2 or 4): a template parameter so that absent
// slots cost no issue slots.
template <int DPL>
__global__ void __launch_bounds__(32 * CTX_WARPS) attn_context_kernel(float *__restrict__ ctx, float *__restrict__ scores,
                                                                       const float *__restrict__ vcache, int b, int l, int nh,
                                                                       int nkv, int hd, int cap, int key_lo, int s, int own0,
                                                                       int window, const int *__restrict__ pos_dev) {
    attn_geometry(pos_dev, l, cap, window, key_lo, s, own0);
    extern __shared__ __align__(16) float ctx_smem[];
    float *vtile = ctx_smem;                         // [CTX_KT][hd], flushed
    float *wt = ctx_smem + (size_t)CTX_KT * hd;      // [CTX_KT][CTX_ROWS]: a key's values for the CTA's rows
    const int bh = blockIdx.y, bb = bh / nh, h = bh % nh, kv = h / (nh / nkv);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int q_first = blockIdx.x * CTX_ROWS, q0 = q_first + warp * CTX_RPW;
    float *mine = wt + warp * CTX_RPW;               // this warp's four columns of wt
    bool active[CTX_RPW];
    float *row[CTX_RPW];
    int jlo[CTX_RPW], jhi[CTX_RPW];
    float den[CTX_RPW], fm[CTX_RPW];
    bool all_active = true;
#pragma unroll
    for (int r = 0; r < CTX_RPW; r++) {
        const int qi = q0 + r;
        active[r] = qi < l;
        all_active = all_active && active[r];
        row[r] = scores + ((long long)bh * l + (active[r] ? qi : 0)) * s;
        jlo[r] = 0;
        jhi[r] = min(own0 + qi, s - 1);
        if (window > 0) jlo[r] = max(own0 + qi - window + 1, 0);
        if (!active[r]) { jlo[r] = 0; jhi[r] = -1; }
        den[r] = 0.f;
        fm[r] = 0.f;
        if (active[r]) {
            // S14: the row maximum over the WHOLE row, as a total-order key (fold shape is free)
            unsigned best = 0u;
            for (int j = lane; j < s; j += 32) best = max(best, order_key(ftz_bits(row[r][j])));
#pragma unroll
            for (int off = 16; off > 0; off >>= 1) best = max(best, __shfl_xor_sync(0xFFFFFFFFu, best, off));
            fm[r] = ftz_bits(order_unkey(best));
        }
    }
    // S15, S16 in parallel; S17 serial ascending over the visible keys of each row
    if (window == 0 && all_active) {
        // the four rows start at key 0: walk the tiles together, the exponentials of a key side by side in wt
        for (int j0 = 0; j0 <= jhi[CTX_RPW - 1]; j0 += 32) {
            const int j = j0 + lane;
            float e[CTX_RPW];
#pragma unroll
            for (int r = 0; r < CTX_RPW; r++) {
                e[r] = 0.f;
                if (j <= jhi[r]) {
                    e[r] = ftz_bits(p_expf(ftz_bits(__fsub_rn(ftz_bits(row[r][j]), fm[r]))));
                    row[r][j] = e[r];
                }
            }
            *reinterpret_cast<float4 *>(mine + lane * CTX_ROWS) = make_float4(e[0], e[1], e[2], e[CTX_RPW - 1]);
            __syncwarp();
            if (j0 + 31 <= jhi[0]) { // whole tile visible to all four rows (jhi ascends with the row)
#pragma unroll
                for (int t = 0; t < 32; t++) {
                    const float4 e4 = *reinterpret_cast<const float4 *>(mine + t * CTX_ROWS);
                    den[0] = add_flushed(den[0], e4.x);
                    den[1] = add_flushed(den[1], e4.y);
                    den[2] = add_flushed(den[2], e4.z);
                    den[CTX_RPW - 1] = add_flushed(den[CTX_RPW - 1], e4.w);
                }
            } else { // the rows end inside the tile, each at its own key: one walk, a row steps while the key is its own
                const int tmax = min(31, jhi[CTX_RPW - 1] - j0);
#pragma unroll 4
                for (int t = 0; t <= tmax; t++) {
                    const float4 e4 = *reinterpret_cast<const float4 *>(mine + t * CTX_ROWS);
                    const float ev[CTX_RPW] = {e4.x, e4.y, e4.z, e4.w};
#pragma unroll
                    for (int r = 0; r < CTX_RPW; r++)
                        if (j0 + t <= jhi[r]) den[r] = add_flushed(den[r], ev[r]);
                }
            }
            __syncwarp();
        }
    } else {
#pragma unroll
        for (int r = 0; r < CTX_RPW; r++) {
            if (!active[r]) continue;
            for (int j0 = jlo[r]; j0 <= jhi[r]; j0 += 32) {
                const int j = j0 + lane;
                float e = 0.f;
                if (j <= jhi[r]) {
                    e = ftz_bits(p_expf(ftz_bits(__fsub_rn(ftz_bits(row[r][j]), fm[r]))));
                    row[r][j] = e;
                }
                const int cnt = min(32, jhi[r] - j0 + 1);
                // every term is already flushed: add.rn.ftz is the seam's add-then-flush in one instruction
                for (int t = 0; t < cnt; t++) den[r] = add_flushed(den[r], __shfl_sync(0xFFFFFFFFu, e, t));
            }
        }
    }
    // S18 + S19 over value tiles shared by the CTA's rows
    float acc[CTX_RPW][DPL];
#pragma unroll
    for (int r = 0; r < CTX_RPW; r++)
#pragma unroll
        for (int i = 0; i < DPL; i++) acc[r][i] = 0.f;
    const float *vbase = vcache + (((long long)bb * nkv + kv) * cap + key_lo) * hd;
    const bool vec = (hd % 4 == 0) && ((reinterpret_cast<uintptr_t>(vbase) & 15u) == 0);
    // keys any row of this CTA can see
    const int q_last = min(l - 1, q_first + CTX_ROWS - 1);
    int t_lo = 0, t_hi = min(s - 1, own0 + q_last);
    if (window > 0) { t_lo = own0 + q_first - window + 1; if (t_lo < 0) t_lo = 0; }
    bool clean = true; // every step of this warp's rows so far was an admitted bare fma
    int jmax = -1;
#pragma unroll
    for (int r = 0; r < CTX_RPW; r++) jmax = max(jmax, jhi[r]);
    for (int j0 = (t_lo / CTX_KT) * CTX_KT; j0 <= t_hi; j0 += CTX_KT) {
        __syncthreads();
        unsigned vkey = 0xFFFFFFFFu;
        if (vec && j0 + CTX_KT <= s) { // the tile is one contiguous block of the cache
            const float4 *src = reinterpret_cast<const float4 *>(vbase + (long long)j0 * hd);
            float4 *dst = reinterpret_cast<float4 *>(vtile);
            for (int idx = threadIdx.x; idx < CTX_KT * hd / 4; idx += 32 * CTX_WARPS) {
                float4 v = src[idx];
                v.x = ftz_bits(v.x); v.y = ftz_bits(v.y); v.z = ftz_bits(v.z); v.w = ftz_bits(v.w);
                vkey = min(vkey, key_of4(v));
                dst[idx] = v;
            }
        } else {
            for (int idx = threadIdx.x; idx < CTX_KT * hd; idx += 32 * CTX_WARPS) {
                const int jj = idx / hd;
                const float v = (j0 + jj < s) ? ftz_bits(vbase[(long long)(j0 + jj) * hd + idx % hd]) : 0.f;
                vkey = min(vkey, admit_key(v));
                vtile[idx] = v;
            }
        }
        const bool v_ok = __syncthreads_and(vkey >= ADMIT_MIN);
        if (jmax < j0) continue; // no row of this warp sees the tile (uniform per warp)
        const int j = j0 + lane;
        float wgt[CTX_RPW];
        unsigned wkey = 0xFFFFFFFFu;
        bool full = hd == DPL * 32, heads = hd == DPL * 32; // heads: every live row's range starts at or before the tile
#pragma unroll
        for (int r = 0; r < CTX_RPW; r++) {
            wgt[r] = 0.f;
            if (j >= jlo[r] && j <= jhi[r]) {
                wgt[r] = ftz_bits(p_divf(ftz_bits(row[r][j]), den[r]));
                row[r][j] = wgt[r];
            }
            wkey = min(wkey, admit_key(wgt[r]));
            full = full && jlo[r] <= j0 && jhi[r] >= j0 + CTX_KT - 1;
            heads = heads && (jlo[r] <= j0 || jhi[r] < j0);
        }
        *reinterpret_cast<float4 *>(mine + lane * CTX_ROWS) = make_float4(wgt[0], wgt[1], wgt[2], wgt[CTX_RPW - 1]);
        __syncwarp();
        const bool w_ok = __all_sync(0xFFFFFFFFu, wkey >= ADMIT_MIN);
        // one key of the tile for the warp's four rows; `bare_c` and `ragged` are constants at every call site
        auto key_step = [&](int t, const bool bare_c, const bool ragged) {
            const float4 w4 = *reinterpret_cast<const float4 *>(mine + t * CTX_ROWS);
            const float w[CTX_RPW] = {w4.x, w4.y, w4.z, w4.w};
            float v[DPL];
            if (DPL == 4) {
                const float4 x = *reinterpret_cast<const float4 *>(vtile + t * hd + lane * 4);
                v[0] = x.x; v[1 % DPL] = x.y; v[2 % DPL] = x.z; v[3 % DPL] = x.w;
            } else if (DPL == 2) {
                const float2 x = *reinterpret_cast<const float2 *>(vtile + t * hd + lane * 2);
                v[0] = x.x; v[1 % DPL] = x.y;
            } else {
                v[0] = vtile[t * hd + lane];
            }
#pragma unroll
            for (int r = 0; r < CTX_RPW; r++) {
                if (ragged && j0 + t > jhi[r]) continue;
#pragma unroll
                for (int i = 0; i < DPL; i++) acc[r][i] = bare_c ? step_bare(w[r], v[i], acc[r][i]) : step_flush(w[r], v[i], acc[r][i]);
            }
        };
        if (full) { // a whole tile for all four rows, every feature slot live: unrolled
            const bool bare = clean && v_ok && w_ok;
            clean = bare;
            if (bare) {
#pragma unroll
                for (int t = 0; t < CTX_KT; t++) key_step(t, true, false);
            } else {
#pragma unroll 8
                for (int t = 0; t < CTX_KT; t++) key_step(t, false, false);
            }
        } else if (heads) { // the rows end inside the tile, each at its own key (the diagonal tile of a causal prompt)
            const bool bare = clean && v_ok && w_ok;
            clean = bare;
            const int tmax = min(CTX_KT - 1, jmax - j0);
            if (bare) {
#pragma unroll 4
                for (int t = 0; t <= tmax; t++) key_step(t, true, true);
            } else {
#pragma unroll 4
                for (int t = 0; t <= tmax; t++) key_step(t, false, true);
            }
        } else {
            clean = false;
#pragma unroll
            for (int r = 0; r < CTX_RPW; r++) {
                const int a = max(jlo[r], j0), z = min(jhi[r], j0 + CTX_KT - 1);
                for (int jk = a; jk <= z; jk++) {
                    const float wv = mine[(jk - j0) * CTX_ROWS + r];
#pragma unroll
                    for (int i = 0; i < DPL; i++) {
                        const int d = lane * DPL + i;
                        if (d < hd) acc[r][i] = step_flush(wv, vtile[(jk - j0) * hd + d], acc[r][i]);
                    }
                }
            }
        }
    }
#pragma unroll
    for (int r = 0; r < CTX_RPW; r++) {
        if (!active[r]) continue;
        float *o = ctx + ((long long)bb * l + q0 + r) * ((long long)nh * hd) + (long long)h * hd;
#pragma unroll
        for (int i = 0; i < DPL; i++) {
            const int d = lane * DPL + i;
            if (d < hd) o[d] = acc[r][i];
        }
    }
}

// The same seams with ONE CTA per query row, for a decode step (few query rows, long
// key axis): the row's weights are built once in shared memory (the denominator by
// one warp, shuffle rounds), then thread d walks the value chain of feature d down
// the keys. The cache rows of 32 keys at a time are one contiguous block (16 KB at
// head_dim 128): thread 0 moves each block into a ring of CTX_ST stages with one bulk
// copy (cp.async.bulk, completion on an mbarrier), the first stages issued before the
// softmax phases, so a CTA keeps up to 32 KB outstanding to HBM while the chain runs.
// A head_dim that is not a multiple of 4 leaves rows off the 16-byte grid the bulk
// copy needs; those caches go through per-thread cp.async instead.
// Every wait on an mbarrier is bounded; one that runs out sets the status word read by
// b200i_decode_status (value 3) and the kernel carries on to its end.
// Three stages and a 4K-key weight row fit four CTAs on an SM. A call with few CTAs (a head-sharded rank, a small
// batch) gets up to CTX_ST_MAX stages instead: what bounds it is the bytes one CTA keeps in flight.
constexpr int CTX_NB = 32, CTX_ST = 3, CTX_ST_MAX = 12;
inline size_t attn_context_row_smem(int s_grid, int hd, int stages = CTX_ST) {
    return ((size_t)((s_grid + 3) & ~3) + (size_t)stages * CTX_NB * hd) * sizeof(float);
}
__global__ void __launch_bounds__(128) attn_context_row_kernel(float *__restrict__ ctx, float *__restrict__ scores,
                                                                const float *__restrict__ vcache, int b, int l, int nh, int nkv,
                                                                int hd, int cap, int key_lo, int s, int own0, int window,
                                                                const int *__restrict__ pos_dev, int s_grid, int stages) {
    attn_geometry(pos_dev, l, cap, window, key_lo, s, own0);
    extern __shared__ __align__(16) float ctx_smem[];
    float *wrow = ctx_smem;                        // [s] weights of this row
    float *ring = ctx_smem + ((s_grid + 3) & ~3);  // [stages][CTX_NB * hd]
    __shared__ unsigned red[4];
    __shared__ float den_s;
    __shared__ __align__(8) unsigned long long full[CTX_ST_MAX];
    const int r = blockIdx.x; // (bh, qi)
    const int bh = r / l, qi = r % l, bb = bh / nh, h = bh % nh, kv = h / (nh / nkv);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    float *row = scores + (long long)r * s;
    int jlo = 0, jhi = own0 + qi;
    if (jhi > s - 1) jhi = s - 1;
    if (window > 0) { jlo = own0 + qi - window + 1; if (jlo < 0) jlo = 0; }
    const float *vbase = vcache + (((long long)bb * nkv + kv) * cap + key_lo) * hd;
    const bool bulk = (hd % 4) == 0;
    if (!bulk) stages = CTX_ST; // the per-thread copies count their groups at compile time
    const int nstages = (jhi - jlo + CTX_NB) / CTX_NB;
    if (bulk && tid == 0) {
        for (int i = 0; i < stages; i++) mbar_init(&full[i], 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    auto issue = [&](int k) { // stage k: keys jlo + 32k ..., into slot k % stages
        if (bulk) {
            if (tid == 0 && k < nstages) {
                const int first = jlo + k * CTX_NB, keys = min(CTX_NB, jhi - first + 1);
                const unsigned bytes = (unsigned)(keys * hd) * 4u;
                mbar_expect_tx(&full[k % stages], bytes);
                bulk_copy_g2s(ring + (size_t)(k % stages) * CTX_NB * hd, vbase + (long long)first * hd, bytes, &full[k % stages]);
            }
        } else { // always one commit, so that the groups count stages
            if (k < nstages) {
                const int first = jlo + k * CTX_NB, keys = min(CTX_NB, jhi - first + 1);
                cp_async_floats(ring + (size_t)(k % stages) * CTX_NB * hd, vbase + (long long)first * hd, keys * hd, false, tid, 128);
            }
            cp_async_commit();
        }
    };
    for (int k = 0; k < stages - 1; k++) issue(k);
    unsigned best = 0u;
    for (int j = tid; j < s; j += 128) best = max(best, order_key(ftz_bits(row[j])));
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) best = max(best, __shfl_xor_sync(0xFFFFFFFFu, best, off));
    if (lane == 0) red[warp] = best;
    __syncthreads();
    best = max(max(red[0], red[1]), max(red[2], red[3]));
    const float fm = ftz_bits(order_unkey(best));
    for (int j = jlo + tid; j <= jhi; j += 128) wrow[j] = ftz_bits(p_expf(ftz_bits(__fsub_rn(ftz_bits(row[j]), fm))));
    __syncthreads();
    if (warp == 0) { // S17: serial ascending, every value already flushed
        float den = 0.f;
        for (int j0 = jlo; j0 <= jhi; j0 += 32) {
            const float e = (j0 + lane <= jhi) ? wrow[j0 + lane] : 0.f;
            if (j0 + 31 <= jhi) {
#pragma unroll
                for (int t = 0; t < 32; t++) den = add_flushed(den, __shfl_sync(0xFFFFFFFFu, e, t));
            } else {
                for (int t = 0; t < jhi - j0 + 1; t++) den = add_flushed(den, __shfl_sync(0xFFFFFFFFu, e, t));
            }
        }
        if (lane == 0) den_s = den;
    }
    __syncthreads();
    const float den = den_s;
    for (int j = jlo + tid; j <= jhi; j += 128) {
        const float wgt = ftz_bits(p_divf(wrow[j], den));
        wrow[j] = wgt;
        row[j] = wgt;
    }
    float acc = 0.f;
    bool clean = true; // every step of this thread's chain so far was an admitted bare fma
    for (int k = 0; k < nstages; k++) {
        issue(k + stages - 1); // refills the slot the previous turn finished with
        if (bulk) {
            if (!mbar_wait(&full[k % stages], (unsigned)(k / stages) & 1u) && lane == 0) atomicExch(&g_decode_status, 3);
        } else {
            cp_async_wait<CTX_ST - 1>(); // this thread's copies of stage k have landed
        }
        __syncthreads(); // everyone's copies are visible (the first turn also orders the weights above)
        if (tid < hd) {
            const float *vs = ring + (size_t)(k % stages) * CTX_NB * hd + tid;
            const int first = jlo + k * CTX_NB;
            if (first + CTX_NB - 1 <= jhi) {
                // A thread's chain reads its own feature of the 32 values and the 32 weights: when all of them pass
                // the product's admission test and every earlier step of the chain was admitted too, the bare fma is
                // the contract's step (no result can be subnormal). The walk runs bare while folding the key and is
                // redone with the flushed step only when the key fails.
                const float before = acc;
                unsigned key = 0xFFFFFFFFu;
                if (clean) {
#pragma unroll
                    for (int u = 0; u < CTX_NB; u++) {
                        const float wj = wrow[first + u], vj = vs[u * hd];
                        key = min(key, min(admit_key(wj), admit_key(vj)));
                        acc = step_bare(wj, vj, acc);
                    }
                }
                if (!clean || key < ADMIT_MIN) {
                    clean = false;
                    acc = before;
#pragma unroll
                    for (int u = 0; u < CTX_NB; u++) acc = step_flush(wrow[first + u], ftz_bits(vs[u * hd]), acc);
                }
            } else {
                clean = false;
                for (int u = 0; first + u <= jhi; u++) acc = step_flush(wrow[first + u], ftz_bits(vs[u * hd]), acc);
            }
        }
        __syncthreads(); // the slot is free for the copy the next turn issues
    }
    if (tid < hd) ctx[((long long)bb * l + qi) * ((long long)nh * hd) + (long long)h * hd + tid] = acc;
}

// ---- decode-step attention in one kernel ------------------------------------------------------------
// Scores, softmax and value sum of up to eight query rows of one (sequence, head) in ONE CTA: the masked score rows
// live in shared memory and never reach global memory (the reference's fused attention: "same fold order, nothing
// materialised in HBM", transformer/impl/llama/fused_attention.mojo:5 of the reference). The seams and their order
// are those of attn_scores_small_kernel and attn_context_row_kernel above, spelled once more around one shared
// score buffer:
//   scores   a warp stages the cache rows of `kkeys` keys (up to 32) with cp.async (`nkb` tiles in flight per warp) and
//            lane j walks row j: one serial chain per (query, key) over head_dim, bare while its operands pass
//            admission, flushed otherwise; S12 scale, S13 mask ADD;
//   softmax  S14 row max over the WHOLE row, S15-S16 exp, S17 the serial denominator (one warp per row, shuffle
//            rounds), S18 one division per weight;
//   values   thread d walks feature d down the keys, one chain per query row, the cache rows of `vkeys` keys moved by
//            one bulk copy into a ring of `stages` slots (the key tiles' shared memory, reused).
// The host picks kkeys, nkb, vkeys and stages from the number of CTAs in the call: enough CTAs per SM that the call
// is one wave, and whatever shared memory that leaves each CTA is spent on bytes in flight.
// head_dim must be a multiple of 4 and at most 128. Every mbarrier wait is bounded (status 3).
constexpr int ATD_THREADS = 128, ATD_WARPS = 4;
__host__ __device__ inline size_t atd_region_floats(int hd, int kkeys, int nkb, int vkeys, int stages) {
    const size_t ktiles = (size_t)ATD_WARPS * nkb * kkeys * ATT_KT_PITCH, ring = (size_t)stages * vkeys * hd;
    return ktiles > ring ? ktiles : ring;
}
inline size_t attn_decode_smem(int lq, int s_grid, int hd, int kkeys, int nkb, int vkeys, int stages) {
    return ((size_t)lq * K_LEAF_MIN + (size_t)lq * ((s_grid + 3) & ~3) + atd_region_floats(hd, kkeys, nkb, vkeys, stages)) * sizeof(float);
}
constexpr int ATD_MAX_STAGES = 12;
template <int LQ>
__global__ void __launch_bounds__(ATD_THREADS) attn_decode_kernel(float *__restrict__ ctx, const float *__restrict__ q,
                                                                  const float *__restrict__ kcache, const float *__restrict__ vcache,
                                                                  int b, int l, int nh, int nkv, int hd, int cap, int key_lo, int s,
                                                                  int own0, int window, const int *__restrict__ pos_dev, int s_grid,
                                                                  int kkeys, int nkb, int vkeys, int stages, float softcap) {
    attn_geometry(pos_dev, l, cap, window, key_lo, s, own0);
    extern __shared__ __align__(16) float atd_smem[];
    const int spitch = (s_grid + 3) & ~3;
    float (*qs)[K_LEAF_MIN] = reinterpret_cast<float (*)[K_LEAF_MIN]>(atd_smem);
    float *sc = atd_smem + LQ * K_LEAF_MIN;            // [LQ][spitch]: masked scores, then exponentials, then weights
    float *region = sc + (size_t)LQ * spitch;          // key tiles first, the value ring afterwards
    __shared__ unsigned red[LQ][ATD_WARPS];
    __shared__ float fm_s[LQ], den_s[LQ], scale_s;
    __shared__ __align__(8) unsigned long long full[ATD_MAX_STAGES];
    const int bh = blockIdx.x, bb = bh / nh, h = bh % nh, kv = h / (nh / nkv);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const float *kbase = kcache + (((long long)bb * nkv + kv) * cap + key_lo) * hd;
    const float *vbase = vcache + (((long long)bb * nkv + kv) * cap + key_lo) * hd;
    const long long qw = (long long)nh * hd;
    const float mfill = __uint_as_float(0xFF7FFFFFu);

    // ---- the query rows, flushed, and their admission key ----
    if (tid == 0) {
        scale_s = ftz_bits(p_rsqrtf((float)hd)); // a pure function of head_dim: one thread spells it
        for (int i = 0; i < stages; i++) mbar_init(&full[i], 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    unsigned qkey = 0xFFFFFFFFu;
    for (int idx = tid; idx < LQ * hd; idx += ATD_THREADS) {
        const int i = idx / hd, p = idx % hd;
        const float v = i < l ? ftz_bits(q[((long long)bb * l + i) * qw + (long long)h * hd + p]) : 0.f;
        qkey = min(qkey, admit_key(v));
        qs[i][p] = v;
    }
    const bool q_ok = __syncthreads_and(qkey >= ADMIT_MIN);
    const float scale = scale_s;

    // ---- scores: this warp's key tiles, NKB of them in flight ----
    const int tiles = (s + kkeys - 1) / kkeys;
    float *kt_w = region + (size_t)warp * nkb * kkeys * ATT_KT_PITCH;
    auto fetch = [&](int n) { // the n-th tile of this warp into buffer n % nkb; always one commit group
        const int tile = warp + n * ATD_WARPS;
        if (tile < tiles) {
            const int j0 = tile * kkeys, rows = min(kkeys, s - j0);
            float *dst = kt_w + (size_t)(n % nkb) * kkeys * ATT_KT_PITCH + lane * 4;
            const float *src = kbase + (long long)j0 * hd + lane * 4;
            if (lane * 4 < hd)
                for (int r = 0; r < rows; r++) cp_async16(dst + r * ATT_KT_PITCH, src + (long long)r * hd);
        }
        cp_async_commit();
    };
    for (int n = 0; n < nkb - 1; n++) fetch(n);
    for (int n = 0; warp + n * ATD_WARPS < tiles; n++) {
        fetch(n + nkb - 1);
        if (nkb == 1) cp_async_wait<0>();
        else if (nkb == 2) cp_async_wait<1>();
        else cp_async_wait<2>();
        __syncwarp();
        const int j0 = (warp + n * ATD_WARPS) * kkeys, j = j0 + lane;
        const float *krow = kt_w + (size_t)(n % nkb) * kkeys * ATT_KT_PITCH + (size_t)lane * ATT_KT_PITCH;
        float acc[LQ];
        bool exact = false;
        if (lane < kkeys && j < s) {
            if (q_ok) {
                unsigned kkey = 0xFFFFFFFFu;
#pragma unroll
                for (int i = 0; i < LQ; i++) acc[i] = 0.f;
#pragma unroll 8
                for (int p = 0; p < hd; p += 4) {
                    const float4 kvv = *reinterpret_cast<const float4 *>(krow + p);
                    kkey = min(kkey, key_of4(kvv));
#pragma unroll
                    for (int i = 0; i < LQ; i++) {
                        const float4 qv = *reinterpret_cast<const float4 *>(&qs[i][p]);
                        acc[i] = step_bare(qv.x, kvv.x, acc[i]);
                        acc[i] = step_bare(qv.y, kvv.y, acc[i]);
                        acc[i] = step_bare(qv.z, kvv.z, acc[i]);
                        acc[i] = step_bare(qv.w, kvv.w, acc[i]);
                    }
                }
                exact = kkey >= ADMIT_MIN;
            }
            if (!exact) {
#pragma unroll
                for (int i = 0; i < LQ; i++) acc[i] = 0.f;
                for (int p = 0; p < hd; p++) {
                    const float kvv = ftz_bits(krow[p]);
#pragma unroll
                    for (int i = 0; i < LQ; i++) acc[i] = step_flush(qs[i][p], kvv, acc[i]);
                }
            }
#pragma unroll
            for (int i = 0; i < LQ; i++) {
                if (i >= l) break;
                int jlo = 0, jhi = own0 + i;
                if (jhi > s - 1) jhi = s - 1;
                if (window > 0) { jlo = own0 + i - window + 1; if (jlo < 0) jlo = 0; }
                const float v = score_scale_cap(acc[i], scale, softcap);
                sc[(size_t)i * spitch + j] = ftz_bits(__fadd_rn(v, (j < jlo || j > jhi) ? mfill : 0.0f));
            }
        }
        __syncwarp(); // the buffer is free for the fetch of the next turn
    }
    cp_async_wait<0>();
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); // the bulk copies below rewrite memory these threads wrote and read
    __syncthreads(); // every score is in place; the key tiles are dead and their memory becomes the value ring

    // ---- the value ring starts while the softmax runs ----
    int jlo_all = 0, jhi_all = min(own0 + l - 1, s - 1); // the keys any row of this call can see
    if (window > 0) jlo_all = max(own0 - window + 1, 0);
    const int nstages = (jhi_all - jlo_all + vkeys) / vkeys;
    auto issue = [&](int k) { // stage k: keys jlo_all + vkeys * k ..., into slot k % stages
        if (tid == 0 && k < nstages) {
            const int first = jlo_all + k * vkeys, keys = min(vkeys, jhi_all - first + 1);
            const unsigned bytes = (unsigned)(keys * hd) * 4u;
            mbar_expect_tx(&full[k % stages], bytes);
            bulk_copy_g2s(region + (size_t)(k % stages) * vkeys * hd, vbase + (long long)first * hd, bytes, &full[k % stages]);
        }
    };
    for (int k = 0; k < stages - 1; k++) issue(k);

    // ---- softmax, row by row seams, rows side by side ----
#pragma unroll
    for (int i = 0; i < LQ; i++) {
        if (i >= l) break;
        unsigned best = 0u;
        for (int j = tid; j < s; j += ATD_THREADS) best = max(best, order_key(ftz_bits(sc[(size_t)i * spitch + j])));
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) best = max(best, __shfl_xor_sync(0xFFFFFFFFu, best, off));
        if (lane == 0) red[i][warp] = best;
    }
    __syncthreads();
    if (tid < LQ && tid < l) fm_s[tid] = ftz_bits(order_unkey(max(max(red[tid][0], red[tid][1]), max(red[tid][2], red[tid][3]))));
    __syncthreads();
#pragma unroll
    for (int i = 0; i < LQ; i++) {
        if (i >= l) break;
        int jlo = 0, jhi = min(own0 + i, s - 1);
        if (window > 0) jlo = max(own0 + i - window + 1, 0);
        const float fm = fm_s[i];
        float *row = sc + (size_t)i * spitch;
        for (int j = jlo + tid; j <= jhi; j += ATD_THREADS) row[j] = ftz_bits(p_expf(ftz_bits(__fsub_rn(ftz_bits(row[j]), fm))));
    }
    __syncthreads();
    for (int i = warp; i < l; i += ATD_WARPS) { // S17: serial ascending, every value already flushed; one warp per row
        int jlo = 0, jhi = min(own0 + i, s - 1);
        if (window > 0) jlo = max(own0 + i - window + 1, 0);
        const float *row = sc + (size_t)i * spitch;
        float den = 0.f;
        for (int j0 = jlo; j0 <= jhi; j0 += 32) {
            const float e = (j0 + lane <= jhi) ? row[j0 + lane] : 0.f;
            if (j0 + 31 <= jhi) {
#pragma unroll
                for (int t = 0; t < 32; t++) den = add_flushed(den, __shfl_sync(0xFFFFFFFFu, e, t));
            } else {
                for (int t = 0; t < jhi - j0 + 1; t++) den = add_flushed(den, __shfl_sync(0xFFFFFFFFu, e, t));
            }
        }
        if (lane == 0) den_s[i] = den;
    }
    __syncthreads();
#pragma unroll
    for (int i = 0; i < LQ; i++) {
        if (i >= l) break;
        int jlo = 0, jhi = min(own0 + i, s - 1);
        if (window > 0) jlo = max(own0 + i - window + 1, 0);
        const float den = den_s[i];
        float *row = sc + (size_t)i * spitch;
        for (int j = jlo + tid; j <= jhi; j += ATD_THREADS) row[j] = ftz_bits(p_divf(row[j], den));
    }
    // (the first turn's barrier below orders the weights before the chains read them)

    // ---- S19: thread d walks feature d down the keys, one chain per query row ----
    float acc[LQ];
    int rlo[LQ], rhi[LQ];
#pragma unroll
    for (int i = 0; i < LQ; i++) {
        acc[i] = 0.f;
        rhi[i] = i < l ? min(own0 + i, s - 1) : -1;
        rlo[i] = (window > 0) ? max(own0 + i - window + 1, 0) : 0;
    }
    bool alive = true;
    for (int k = 0; k < nstages; k++) {
        issue(k + stages - 1); // refills the slot the previous turn finished with
        if (alive && !mbar_wait(&full[k % stages], (unsigned)(k / stages) & 1u)) {
            if (lane == 0) atomicExch(&g_decode_status, 3);
            alive = false;
        }
        __syncthreads();
        if (tid < hd) {
            const float *vs = region + (size_t)(k % stages) * vkeys * hd + tid;
            const int first = jlo_all + k * vkeys;
            const int keys = min(vkeys, jhi_all - first + 1);
            if (LQ == 1) {
                int u = 0;
                for (; u + 16 <= keys; u += 16) {
#pragma unroll
                    for (int t = 0; t < 16; t++) acc[0] = step_flush(sc[first + u + t], ftz_bits(vs[(u + t) * hd]), acc[0]);
                }
                for (; u < keys; u++) acc[0] = step_flush(sc[first + u], ftz_bits(vs[u * hd]), acc[0]);
            } else {
                for (int u = 0; u < keys; u++) {
                    const float v = ftz_bits(vs[u * hd]);
                    const int j = first + u;
#pragma unroll
                    for (int i = 0; i < LQ; i++)
                        if (j >= rlo[i] && j <= rhi[i]) acc[i] = step_flush(sc[(size_t)i * spitch + j], v, acc[i]);
                }
            }
        }
        __syncthreads(); // the slot is free for the copy the next turn issues
    }
    if (tid < hd) {
#pragma unroll
        for (int i = 0; i < LQ; i++)
            if (i < l) ctx[((long long)bb * l + i) * qw + (long long)h * hd + tid] = acc[i];
    }
}

// ---- elementwise seams --------------------------------------------------------------------------
// out is [rows, width] contiguous; gate and up have row pitch ld and column step cs (2 when they are the even and
// odd columns of one matrix: a product over interleaved weight rows)
__global__ void act_mul_kernel(float *__restrict__ out, const float *gate, const float *up, long long rows, long long width, long long ld,
                               int kind, int cs) {
    const long long stride = (long long)gridDim.x * blockDim.x, count = rows * width;
    const bool gated = kind == ACT_SWIGLU || kind == ACT_GEGLU_ERF || kind == ACT_GEGLU_TANH;
    for (long long o = (long long)blockIdx.x * blockDim.x + threadIdx.x; o < count; o += stride) {
        const long long i = (o / width) * ld + (o % width) * cs;
        const float z = ftz_bits(gated ? gate[i] : up[i]);
        float a;
        if (kind == ACT_SWIGLU || kind == ACT_SILU) a = ftz_bits(p_siluf(z));
        else if (kind == ACT_GELU_TANH || kind == ACT_GEGLU_TANH) a = ftz_bits(p_gelu_tanh(z));
        else a = ftz_bits(p_gelu_erf(z));
        out[o] = gated ? ftz_bits(__fmul_rn(a, ftz_bits(up[i]))) : a;
    }
}

__global__ void add_kernel(float *__restrict__ out, const float *__restrict__ a, const float *__restrict__ b, long long count) {
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < count; i += stride)
        out[i] = ftz_bits(__fadd_rn(ftz_bits(a[i]), ftz_bits(b[i])));
}

__global__ void bias_add_kernel(float *__restrict__ buf, const float *__restrict__ bias, long long rows, int width) {
    const long long stride = (long long)gridDim.x * blockDim.x, total = rows * width;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride)
        buf[i] = ftz_bits(__fadd_rn(ftz_bits(buf[i]), ftz_bits(bias[i % width])));
}

// status[0] is set to 1 when a token id falls outside the table (the row is then zero filled)
__global__ void embedding_kernel(float *__restrict__ y, const float *__restrict__ table, const int *__restrict__ ids,
                                 long long n, int vocab, int width, int *__restrict__ status) {
    const long long stride = (long long)gridDim.x * blockDim.x, total = n * width;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
        const long long t = i / width;
        const int id = ids[t];
        if (id < 0 || id >= vocab) {
            y[i] = 0.f;
            if (i % width == 0) atomicExch(status, 1);
        } else {
            y[i] = ftz_bits(table[(long long)id * width + i % width]);
        }
    }
}

// learned positions (an extension: the reference's block always rotates): one plain add
__global__ void add_positions_kernel(float *__restrict__ x, const float *__restrict__ pos, long long rows, int l, int pos0,
                                     int width, const int *__restrict__ pos_dev) {
    if (pos_dev) pos0 = *pos_dev;
    const long long stride = (long long)gridDim.x * blockDim.x, total = rows * width;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += stride) {
        const long long t = i / width;
        x[i] = ftz_bits(__fadd_rn(ftz_bits(x[i]), ftz_bits(pos[(long long)(pos0 + t % l) * width + i % width])));
    }
}

// greedy argmax, one CTA per row. The scalar walk starts from element 0, visits the
// indices ascending and replaces on strictly greater, so its answer is the lowest
// index among the largest non-NaN values, or 0 when element 0 is a NaN (nothing
// compares greater than a NaN). "Larger value, then lower index" is associative, so
// the candidates combine in any order: four loads per thread in flight, shuffles
// inside a warp, one round through shared memory.
constexpr int ARGMAX_THREADS = 1024;
__device__ __forceinline__ void argmax_take(float &best, int &idx, float v, int j) {
    if (v == v && (idx < 0 || v > best || (v == best && j < idx))) { best = v; idx = j; }
}
__global__ void __launch_bounds__(ARGMAX_THREADS) argmax_kernel(int *__restrict__ out, const float *__restrict__ logits, int vocab) {
    __shared__ float bv[32];
    __shared__ int bi[32];
    const float *p = logits + (long long)blockIdx.x * vocab;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    float best = 0.f;
    int idx = -1;
    for (int j0 = tid; j0 < vocab; j0 += 4 * ARGMAX_THREADS) {
        float v[4];
#pragma unroll
        for (int u = 0; u < 4; u++) v[u] = (j0 + u * ARGMAX_THREADS < vocab) ? p[j0 + u * ARGMAX_THREADS] : __uint_as_float(0x7FC00000u);
#pragma unroll
        for (int u = 0; u < 4; u++) argmax_take(best, idx, v[u], j0 + u * ARGMAX_THREADS);
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
        const float ov = __shfl_xor_sync(0xFFFFFFFFu, best, off);
        const int oi = __shfl_xor_sync(0xFFFFFFFFu, idx, off);
        if (oi >= 0) argmax_take(best, idx, ov, oi);
    }
    if (lane == 0) { bv[warp] = best; bi[warp] = idx; }
    __syncthreads();
    if (warp == 0) {
        best = bv[lane];
        idx = bi[lane];
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) {
            const float ov = __shfl_xor_sync(0xFFFFFFFFu, best, off);
            const int oi = __shfl_xor_sync(0xFFFFFFFFu, idx, off);
            if (oi >= 0) argmax_take(best, idx, ov, oi);
        }
        if (lane == 0) {
            const float first = p[0];
            out[blockIdx.x] = (first != first || idx < 0) ? 0 : idx;
        }
    }
}

} // namespace b200i
