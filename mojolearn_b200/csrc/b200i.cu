// The C ABI of libb200i.so: argument checks, plan selection, launches.
// Declarations and the reference interfaces they replace are in include/b200i.h.
#include <atomic>
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <mutex>
#include <vector>

#include "../../include/b200i.h"
#include "comm.cuh"
#include "decode.cuh"
#include "decode_pair.cuh"
#include "gemm_int8_mma.cuh"
#include "gemm_int8_tma.cuh"
#include "gemm_int15.cuh"
#include "decoder.cuh"
#include "gemm_tile.cuh"
#include "gemm_skinny.cuh"
#include "gemm_packed.cuh"
#include "gemm_skinny_reg.cuh"
#include "lowbit.cuh"

using namespace b200i;

namespace {

std::atomic<long long> g_launches{0};

int64_t fail(char *err, int64_t cap, const char *fmt, ...) {
    if (err && cap > 0) {
        va_list ap;
        va_start(ap, fmt);
        vsnprintf(err, (size_t)cap, fmt, ap);
        va_end(ap);
    }
    return 1;
}
void clear(char *err, int64_t cap) {
    if (err && cap > 0) err[0] = 0;
}

#define CUDA_TRY(expr)                                                                                      \
    do {                                                                                                    \
        cudaError_t e_ = (expr);                                                                            \
        if (e_ != cudaSuccess) return fail(err, err_cap, "b200i: %s failed: %s", #expr, cudaGetErrorString(e_)); \
    } while (0)

constexpr int MAX_DEVICES = 64;
struct DeviceInfo {
    int sms = 148;
    bool known = false;
};
DeviceInfo g_info[MAX_DEVICES];
std::mutex g_mu;

int sm_count(int device) {
    if (device < 0 || device >= MAX_DEVICES) return 148;
    std::lock_guard<std::mutex> lock(g_mu);
    if (!g_info[device].known) {
        int v = 0;
        if (cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, device) == cudaSuccess && v > 0) g_info[device].sms = v;
        g_info[device].known = true;
    }
    return g_info[device].sms;
}

int select_device(int64_t device, char *err, int64_t err_cap, int *out) {
    int dev = 0;
    if (device >= 0) {
        dev = (int)device;
        CUDA_TRY(cudaSetDevice(dev));
    } else {
        CUDA_TRY(cudaGetDevice(&dev));
    }
    if (dev < 0 || dev >= MAX_DEVICES) return fail(err, err_cap, "b200i: device %d is outside the %d devices this library tracks", dev, MAX_DEVICES);
    *out = dev;
    return 0;
}

// The status word of the bounded device-side waits, read and cleared. Every host-pointer entry calls this after its
// final synchronise, so a wait that ran out can never return as a silent success; device-pointer callers read it
// through b200i_decode_status when they next synchronise.
int64_t check_wait_status(char *err, int64_t err_cap, const char *who) {
    int v = 0, zero = 0;
    CUDA_TRY(cudaMemcpyFromSymbol(&v, g_decode_status, sizeof(int)));
    if (v == 0) return 0;
    CUDA_TRY(cudaMemcpyToSymbol(g_decode_status, &zero, sizeof(int)));
    return fail(err, err_cap, "%s: a bounded device-side wait ran out (status %d); the output is incomplete", who, v);
}

// ---- plans -----------------------------------------------------------------------------
enum { PLAN_AUTO = -1, PLAN_FLAT = 0, PLAN_T128 = 1, PLAN_T64 = 2, PLAN_DECODE = 3, PLAN_T32 = 4, PLAN_T128X64 = 5, PLAN_SKINNY = 6, PLAN_PACKED = 7 };

// Up to this many rows the weight-streaming decode plan wins; above, the skinny plan. Low-bit weights
// switch earlier: at three and four rows the decode kernel's serial chains cost more than the register
// skinny kernel's eight-row tile (int8 [11008, 4096]: 44 us against 37 us at four rows, 40 against 36 at
// three), except on a very wide weight, where the decode kernel's row streams run at their best
// ([50304, 2048]: bf16 79 us against 98 at four rows, int8 60 against 69 at three).
constexpr int DECODE_PREFER_M = 4;
constexpr long long DECODE_WIDE_N = 32768;
constexpr int DECODE_PREFER_M_LOWBIT = 2;

struct Plan {
    int kind;
    int group_leaves; // S
    int groups;       // G
};

struct TileCfg {
    int kind, bm, bn, per_sm;
    double eff; // fraction of the fused-multiply-add peak the kernel sustains on a full tile (measured)
};
const TileCfg TILE_CFGS[] = {
    {PLAN_T128, 128, 128, 2, 0.55},
    {PLAN_T64, 64, 64, 3, 0.33},
    {PLAN_T32, 32, 128, 4, 0.40},
};

int pow2_floor(int v) {
    int p = 1;
    while (p * 2 <= v) p *= 2;
    return p;
}

// Modelled time of a tiled plan in SM cycles: waves of CTAs over the SM slots,
// each CTA running its share of the leaves, plus the traffic of the group nodes
// and the second launch when the leaves are split.
double tiled_cost(const TileCfg &cfg, long long m, long long n, int leaf, int leaves, int s, int sms) {
    const long long tiles = ((m + cfg.bm - 1) / cfg.bm) * ((n + cfg.bn - 1) / cfg.bn);
    const int groups = (leaves + s - 1) / s;
    const long long ctas = tiles * groups;
    const long long slots = (long long)sms * cfg.per_sm;
    const long long waves = (ctas + slots - 1) / slots;
    const double cta = (double)cfg.bm * cfg.bn * (double)leaf * s * cfg.per_sm / (128.0 * cfg.eff);
    double t = (double)waves * cta + 4000.0;
    if (groups > 1) t += (double)groups * m * n * 8.0 / 2500.0 + 6000.0; // node write + read at HBM rate, second launch
    return t;
}

Plan choose_plan(long long m, long long n, long long k, int sms) {
    const int leaf = (int)leaf_size(k), leaves = (int)leaf_count(k);
    Plan best{PLAN_T128, leaves > 0 ? leaves : 1, 1};
    double best_t = 1e300;
    const int max_s = pow2_floor(leaves > 0 ? leaves : 1) * ((leaves & (leaves - 1)) ? 2 : 1);
    for (const TileCfg &cfg : TILE_CFGS) {
        for (int s = max_s; s >= 1; s /= 2) {
            const int groups = (leaves + s - 1) / s;
            if (groups > MAX_GROUPS) break;
            const double t = tiled_cost(cfg, m, n, leaf, leaves, s, sms);
            if (t < best_t) { best_t = t; best = Plan{cfg.kind, s, groups}; }
        }
    }
    if (best.groups <= 1) best.group_leaves = leaves > 0 ? leaves : 1;
    return best;
}

// The skinny plan's leaf split. Float32 weights (shared-memory kernel): the largest
// power-of-two group that still gives every CTA slot of the device a CTA, else
// single leaves. Low-bit weights (register kernel): the split minimises a modelled
// time in microseconds fitted to measurements on B200 -- rounds of CTAs per SM times
// (leaves per CTA at the kernel's sustained rate, slower while an SM holds fewer than
// three CTAs, plus a fixed cost per CTA), plus the second launch and the L2-resident
// node traffic of the group fold.
Plan choose_skinny(long long m, long long n, long long k, int sms, bool lowbit) {
    const int leaves = (int)leaf_count(k) > 0 ? (int)leaf_count(k) : 1;
    const int max_s = pow2_floor(leaves) * ((leaves & (leaves - 1)) ? 2 : 1);
    int min_s = 1;
    while ((leaves + min_s - 1) / min_s > MAX_GROUPS) min_s *= 2;
    int best = min_s;
    if (lowbit) {
        const int bm = skr_bm((int)m), bn = skr_bn((int)m);
        const long long tiles = ((n + bn - 1) / bn) * ((m + bm - 1) / bm);
        const double rate = bm >= 32 ? 0.25e6 : (bm >= 16 ? 0.20e6 : 0.15e6); // flops per microsecond per SM
        // a CTA's leaf: its multiply-adds at that rate, or its weight bytes at an SM's share of the HBM stream
        const double leaf_us = std::max(2.0 * bm * bn * (double)leaf_size(k) / rate, (double)bn * (double)leaf_size(k) / 40.0e3);
        double best_t = 1e300;
        for (int s = max_s; s >= min_s; s /= 2) {
            const int groups = (leaves + s - 1) / s;
            const long long ctas = tiles * groups;
            const long long rounds = (ctas + sms - 1) / sms;
            double thin = ctas <= sms ? 1.25 : (ctas <= 2 * sms ? 1.08 : 1.0);
            double t = (double)rounds * (s * leaf_us * thin + 0.4);
            if (groups > 1) t += 2.5 + (double)groups * m * n * 8.0 / 7.5e6;
            if (t < best_t) { best_t = t; best = s; }
        }
    } else {
        const long long col_ctas = (n + skinny_bn((int)m) - 1) / skinny_bn((int)m);
        const long long want = (long long)sms * skinny_per_sm((int)m) * 9 / 10;
        for (int s = max_s; s >= min_s; s /= 2)
            if (col_ctas * ((leaves + s - 1) / s) >= want) { best = s; break; }
    }
    Plan p{PLAN_SKINNY, best, (leaves + best - 1) / best};
    if (p.groups <= 1) p.group_leaves = leaves;
    return p;
}

bool aligned(const void *p, size_t a) { return (reinterpret_cast<uintptr_t>(p) & (a - 1)) == 0; }

// ---- optional device timing of the product's main kernel ------------------------------------
// While enabled, every product call records a CUDA event pair on its stream around its main
// kernel (the tile / packed / skinny / decode kernel; not the packing passes, not the group fold).
struct KernelTiming {
    bool on = false;
    int used = 0;
    std::vector<cudaEvent_t> ev; // pairs
};
KernelTiming g_timing;
std::mutex g_timing_mu;
constexpr int TIMING_MAX_PAIRS = 4096;
thread_local bool t_no_timing = false; // set by the allocation-free entry: creating an event may allocate
int timing_begin(cudaStream_t st) {
    if (t_no_timing) return -1;
    std::lock_guard<std::mutex> lock(g_timing_mu);
    if (!g_timing.on || g_timing.used >= TIMING_MAX_PAIRS) return -1;
    const int slot = g_timing.used++;
    while ((int)g_timing.ev.size() < 2 * (slot + 1)) {
        cudaEvent_t e;
        if (cudaEventCreate(&e) != cudaSuccess) { cudaGetLastError(); g_timing.used = slot; return -1; }
        g_timing.ev.push_back(e);
    }
    cudaEventRecord(g_timing.ev[2 * slot], st);
    return slot;
}
void timing_end(int slot, cudaStream_t st) {
    if (slot < 0) return;
    std::lock_guard<std::mutex> lock(g_timing_mu);
    cudaEventRecord(g_timing.ev[2 * slot + 1], st);
}

size_t round256(size_t v) { return (v + 255) / 256 * 256; }

// rows below which packing the operands costs more than the bulk-copy pipeline returns
constexpr long long PACKED_MIN_EXTENT = 256;
// The packed plan replaces the 128 x 128 tile plan from 256 rows and columns up, and any tile plan when the rows
// are one or two (nearly) full rows of 128 x 128 tiles over a wide, deep product (128 x 11008 x 4096: 305 us
// against 370 us for the 32 x 128 tiles).
inline bool packed_candidate(int tile_kind, long long m, long long n, long long k) {
    if (tile_kind == PLAN_T128 && m >= PACKED_MIN_EXTENT && n >= PACKED_MIN_EXTENT) return true;
    const long long padded = (m + PK_TILE - 1) / PK_TILE * PK_TILE;
    return tile_kind != PLAN_FLAT && m >= 117 && m <= 256 && padded * 10 <= m * 11 && n >= 2048 && k >= 1024;
}
size_t packed_need(long long m, long long n, long long k, int groups) {
    return round256(groups > 1 ? (size_t)groups * m * n * 4 : 0) + pk_workspace_bytes(m, n, k);
}

// The packed plan's leaf split: with at least two CTAs per slot of the device the tiles alone keep every SM busy
// (a CTA left alone on an SM in the last wave runs at nearly twice the speed, so a partial wave costs little)
// and a split would only add group nodes; below that, the tile plan's split stands.
Plan packed_split(const Plan &tile_plan, long long m, long long n, long long k, int sms) {
    const long long tiles = ((m + PK_TILE - 1) / PK_TILE) * ((n + PK_TILE - 1) / PK_TILE);
    Plan p = tile_plan;
    p.kind = PLAN_PACKED;
    const int leaves = (int)leaf_count(k) > 0 ? (int)leaf_count(k) : 1;
    if (tiles >= 4ll * sms) { p.groups = 1; p.group_leaves = leaves; return p; }
    // Few tiles: split the leaves so that the CTA slots (two per SM) fill in whole waves. Modelled time in
    // microseconds: waves x (leaves per CTA at 21.8 us per 128-step leaf -- a 128 x 128 tile at the kernel's
    // measured rate -- plus 1 us per CTA), plus the second launch and the L2-resident node traffic of the fold.
    const long long slots = 2ll * sms;
    const double leaf_us = 21.8 * (double)leaf_size(k) / 128.0;
    const int max_s = pow2_floor(leaves) * ((leaves & (leaves - 1)) ? 2 : 1);
    int min_s = 1;
    while ((leaves + min_s - 1) / min_s > MAX_GROUPS) min_s *= 2;
    int best = max_s;
    double best_t = 1e300;
    for (int sl = max_s; sl >= min_s; sl /= 2) {
        const int groups = (leaves + sl - 1) / sl;
        // a last wave that fills at most half the slots leaves its CTAs alone on their SMs, at nearly twice the speed
        const long long ctas = tiles * groups, whole = ctas / slots, rest = ctas % slots;
        const double waves = (double)whole + (rest == 0 ? 0.0 : (2 * rest <= slots ? 0.55 : 1.0));
        double t = waves * (sl * leaf_us + 1.0);
        if (groups > 1) t += 3.0 + (double)groups * m * n * 8.0 / 7.5e6;
        if (t < best_t) { best_t = t; best = sl; }
    }
    p.group_leaves = best;
    p.groups = (leaves + best - 1) / best;
    if (p.groups <= 1) p.group_leaves = leaves;
    return p;
}

template <int WK>
void launch_pack(const PackArgs &a, cudaStream_t st) {
    dim3 grid((unsigned)a.leaves, (unsigned)((a.extent + PK_TILE - 1) / PK_TILE));
    pack_operand_kernel<WK><<<grid, 256, 0, st>>>(a);
}

// Packs both operands into `scratch` (panels, then flags) and runs the packed kernel.
void packed_configure() {
    static std::atomic<bool> configured[64];
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 64 && !configured[dev]) {
        cudaFuncSetAttribute(gemm_packed_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, PK_SMEM_BYTES);
        configured[dev] = true;
    }
}
void launch_pack_b(const PackArgs &b, int wkind, cudaStream_t st) {
    if (wkind == W_F32) launch_pack<W_F32>(b, st);
    else if (wkind == W_BF16) launch_pack<W_BF16>(b, st);
    else if (wkind == W_INT8_EXP) launch_pack<W_INT8_EXP>(b, st);
    else launch_pack<W_INT8_SCALE>(b, st);
}

int launch_packed(const GemmArgs &g, int groups, unsigned char *scratch, cudaStream_t st) {
    packed_configure();
    const int wpl = pk_windows_per_leaf(g.leaf);
    float *pa = reinterpret_cast<float *>(scratch);
    float *pb = pa + pk_panel_floats(g.m, g.k);
    unsigned char *fa = reinterpret_cast<unsigned char *>(pb + pk_panel_floats(g.n, g.k));
    unsigned char *fb = fa + pk_flag_bytes(g.m, g.k);
    const bool k8 = (g.k % 8 == 0) && (g.leaves == 1 || g.leaf % 8 == 0);
    PackArgs a{pa, fa, g.a, nullptr, g.m, g.k, g.leaf, g.leaves, wpl, g.op != OP_TN, g.op != OP_TN && k8 && aligned(g.a, 16)};
    launch_pack<W_F32>(a, st);
    PackArgs b{pb, fb, g.b, g.bscale, g.n, g.k, g.leaf, g.leaves, wpl, g.op == OP_NT, g.op == OP_NT && k8 && aligned(g.b, 16)};
    launch_pack_b(b, g.wkind, st);
    PackedGemmArgs p{pa, pb, fa, fb, g.c, g.ws, g.m, g.n, g.k, g.leaf, g.leaves, wpl, g.group_leaves, groups,
                     (g.n + PK_TILE - 1) / PK_TILE, g.vec_c};
    dim3 grid((unsigned)(((g.m + PK_TILE - 1) / PK_TILE) * p.tiles_n), (unsigned)groups);
    const int tslot = timing_begin(st);
    gemm_packed_kernel<<<grid, PK_THREADS, PK_SMEM_BYTES, st>>>(p);
    timing_end(tslot, st);
    return 3;
}

template <int BM, int BN, int RM, int RN, int MINB>
void launch_tile(GemmArgs &g, int groups, cudaStream_t st) {
    using S = TileShape<BM, BN, RM, RN>;
    static std::atomic<bool> configured[64];
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 64 && !configured[dev]) {
        cudaFuncSetAttribute(gemm_tile_kernel<BM, BN, RM, RN, MINB>, cudaFuncAttributeMaxDynamicSharedMemorySize, S::SMEM_BYTES);
        configured[dev] = true;
    }
    g.tiles_n = (g.n + BN - 1) / BN;
    dim3 grid((unsigned)(((g.m + BM - 1) / BM) * g.tiles_n), (unsigned)groups);
    gemm_tile_kernel<BM, BN, RM, RN, MINB><<<grid, S::THREADS, S::SMEM_BYTES, st>>>(g);
}

unsigned grid_for(long long work_items, int block, int sms) {
    long long blocks = (work_items + block - 1) / block;
    const long long cap = (long long)sms * 16;
    if (blocks > cap) blocks = cap;
    if (blocks < 1) blocks = 1;
    return (unsigned)blocks;
}

int64_t launch_product(int dev, cudaStream_t st, float *c, const float *a, const void *b, const void *bscale, int wkind,
                       int64_t m, int64_t n, int64_t k, int op, int plan_kind, int64_t group_leaves, void *ws,
                       int64_t ws_bytes, char *err, int64_t err_cap, Epilogue epi = Epilogue{nullptr, EPI_ACT_NONE},
                       int64_t *leave_nodes = nullptr) {
    // leave_nodes: the caller folds the leaf-group nodes itself (the gather that follows a sharded product does); on
    // return it holds the number of nodes per cell left in ws, 1 when c is finished as usual
    if (leave_nodes) *leave_nodes = 1;
    if (m <= 0 || n <= 0 || k <= 0)
        return fail(err, err_cap, "identical gemm: m, n and k must be positive (got m=%lld n=%lld k=%lld)", (long long)m,
                    (long long)n, (long long)k);
    if (op != OP_NN && op != OP_NT && op != OP_TN) return fail(err, err_cap, "identical gemm: unknown op %d", op);
    if (wkind < W_F32 || wkind > W_INT8_SCALE) return fail(err, err_cap, "identical gemm: unknown weight kind %d", wkind);
    if ((wkind == W_INT8_EXP || wkind == W_INT8_SCALE) && op != OP_NT)
        return fail(err, err_cap, "identical gemm: int8 weight storage is row-scaled and needs op NT");
    if ((wkind == W_INT8_EXP || wkind == W_INT8_SCALE) && !bscale)
        return fail(err, err_cap, "identical gemm: int8 weight storage needs its per-row exponents or scales");
    if (!c || !a || !b) return fail(err, err_cap, "identical gemm: null storage");
    if (m > 0x7FFFFFFF || n > 0x7FFFFFFF || k > 0x7FFFFFFF || m * n > 0x7FFFFFFFll * 64)
        return fail(err, err_cap, "identical gemm: extent out of range");
    if (!aligned(c, 4) || !aligned(a, 4) || (wkind == W_F32 && !aligned(b, 4)) || (wkind == W_BF16 && !aligned(b, 2)))
        return fail(err, err_cap, "identical gemm: misaligned storage");

    GemmArgs g;
    g.a = a; g.b = b; g.bscale = bscale; g.c = c; g.ws = static_cast<float *>(ws);
    g.m = (int)m; g.n = (int)n; g.k = (int)k; g.op = op; g.wkind = wkind;
    g.leaf = (int)leaf_size(k);
    g.leaves = (int)leaf_count(k);
    g.epi = epi;

    Plan plan;
    if (plan_kind == PLAN_AUTO) {
        plan = choose_plan(m, n, k, sm_count(dev));
        if (packed_candidate(plan.kind, m, n, k)) {
            const Plan packed = packed_split(plan, m, n, k, sm_count(dev));
            if (ws && aligned(ws, 256) && (size_t)ws_bytes >= packed_need(m, n, k, packed.groups)) plan = packed;
        }
        const bool al16 = aligned(b, 16) && aligned(a, 16);
        const bool dec = decode_plan_fits(m, n, k, op, wkind) && al16;
        const bool skinny = skinny_plan_fits(m, n, k, op) && al16;
        const bool wide = n >= DECODE_WIDE_N && (wkind == W_BF16 || m == 3);
        // low-bit weights: the leaf-pair decode kernel wherever it fits (up to four rows), else the rule above
        const bool pair = wkind != W_F32 && decode_pair_fits(m, n, k, op, wkind, sm_count(dev));
        const int prefer_m = pair ? DP_MAX_M : ((wkind != W_F32 && skinny && !wide) ? DECODE_PREFER_M_LOWBIT : DECODE_PREFER_M);
        if (dec && m <= prefer_m && !(skinny && epilogue_pairs(g.epi))) plan = Plan{PLAN_DECODE, g.leaves, 1}; // (a gated store needs the skinny plan)
        else if (skinny) plan = choose_skinny(m, n, k, sm_count(dev), wkind != W_F32);
        else if (dec) plan = Plan{PLAN_DECODE, g.leaves, 1};
    } else {
        plan.kind = plan_kind;
        int s = group_leaves > 0 ? (int)group_leaves : g.leaves;
        if (s & (s - 1)) {
            if (s < g.leaves) return fail(err, err_cap, "identical gemm: a leaf group must be a power of two");
        }
        if (s > g.leaves) s = g.leaves;
        plan.group_leaves = s;
        plan.groups = (g.leaves + s - 1) / s;
        if (plan.groups > 1 && (s & (s - 1))) return fail(err, err_cap, "identical gemm: a leaf group must be a power of two");
        if (plan.groups > MAX_GROUPS) return fail(err, err_cap, "identical gemm: more than %d leaf groups", MAX_GROUPS);
        if (plan.kind == PLAN_FLAT || plan.kind == PLAN_DECODE) { plan.groups = 1; plan.group_leaves = g.leaves; }
    }
    g.group_leaves = plan.group_leaves;
    g.groups = plan.groups;
    if (plan.groups > 1) {
        const int64_t need = (int64_t)plan.groups * m * n * 4;
        if (!ws || ws_bytes < need)
            return fail(err, err_cap, "identical gemm: workspace of %lld bytes needed, %lld given", (long long)need,
                        (long long)ws_bytes);
    }

    // 128-bit access is legal when the contiguous axis keeps every vector inside a row and aligned
    const bool a_kc = (op != OP_TN), b_kc = (op == OP_NT);
    const bool leaf_ok = (g.leaves == 1) || (g.leaf % 4 == 0);
    g.vec_a = a_kc ? (k % 4 == 0 && leaf_ok && aligned(a, 16)) : (m % 4 == 0 && aligned(a, 16));
    const size_t balign = wkind == W_F32 ? 16 : (wkind == W_BF16 ? 8 : 4);
    g.vec_b = b_kc ? (k % 4 == 0 && leaf_ok && aligned(b, balign)) : (n % 4 == 0 && aligned(b, balign));
    g.vec_c = (n % 4 == 0) && aligned(c, 16) && (plan.groups == 1 || aligned(ws, 16));

    if (epilogue_pairs(g.epi)) {
        // a gated activation needs both columns of a pair in one thread: the skinny plans, whose threads own adjacent
        // columns, apply it in their own store or in the group fold; no other plan spells it
        const bool fold_ok = plan.groups == 1 || (((long long)m * n) % 4 == 0 && aligned(ws, 16) && aligned(c, 8));
        if (plan.kind != PLAN_SKINNY || n % 4 != 0 || !fold_ok)
            return fail(err, err_cap, "identical gemm: the gated store activation needs the skinny plan (up to 32 rows, op NT, k a multiple of 16) and n a multiple of 4");
    }
    int tslot = -1;
    if (plan.kind != PLAN_PACKED) tslot = timing_begin(st);
    if (plan.kind == PLAN_FLAT) {
        const long long cells = (long long)m * n;
        gemm_flat_kernel<<<(unsigned)((cells + 127) / 128), 128, 0, st>>>(g);
        g_launches++;
    } else if (plan.kind == PLAN_DECODE) {
        if (!decode_plan_fits(m, n, k, op, wkind) || !aligned(b, 16) || !aligned(a, 16))
            return fail(err, err_cap, "identical gemm: the decode plan needs op NT, m <= %d, k a multiple of 16 and 16-byte aligned weights", DECODE_MAX_M);
        g_launches += launch_decode_plan(g, sm_count(dev), st);
    } else if (plan.kind == PLAN_T128) {
        launch_tile<128, 128, 2, 2, 2>(g, plan.groups, st);
        g_launches++;
    } else if (plan.kind == PLAN_T64) {
        launch_tile<64, 64, 1, 1, 3>(g, plan.groups, st);
        g_launches++;
    } else if (plan.kind == PLAN_T32) {
        launch_tile<32, 128, 1, 2, 4>(g, plan.groups, st);
        g_launches++;
    } else if (plan.kind == PLAN_T128X64) {
        launch_tile<128, 64, 2, 1, 3>(g, plan.groups, st);
        g_launches++;
    } else if (plan.kind == PLAN_PACKED) {
        const size_t nodes = round256(plan.groups > 1 ? (size_t)plan.groups * m * n * 4 : 0);
        if (!ws || !aligned(ws, 256) || (size_t)ws_bytes < packed_need(m, n, k, plan.groups))
            return fail(err, err_cap, "identical gemm: the packed plan needs a 256-byte aligned workspace of %lld bytes, %lld given",
                        (long long)packed_need(m, n, k, plan.groups), (long long)ws_bytes);
        g_launches += launch_packed(g, plan.groups, static_cast<unsigned char *>(ws) + nodes, st);
    } else if (plan.kind == PLAN_SKINNY) {
        if (!skinny_plan_fits(m, n, k, op) || !aligned(b, 16) || !aligned(a, 16))
            return fail(err, err_cap, "identical gemm: the skinny plan needs op NT, m <= 32, k a multiple of 16 and 16-byte aligned operands");
        // low-bit weights stay in registers; float32 windows are too wide for that and go through shared memory
        if (g.wkind != W_F32) launch_skinny_reg(g, plan.groups, sm_count(dev), st);
        else launch_skinny(g, plan.groups, st);
        g_launches++;
    } else {
        return fail(err, err_cap, "identical gemm: unknown plan %d", plan.kind);
    }
    timing_end(tslot, st);
    if (plan.groups > 1 && leave_nodes && n % 4 == 0 && aligned(ws, 16)) {
        *leave_nodes = plan.groups;
    } else if (plan.groups > 1) {
        const long long cells = (long long)m * n;
        launch_fold_groups(g.ws, c, cells, plan.groups, st, g.epi, g.n);
        g_launches++;
    } else if (epilogue_on(g.epi) && plan.kind != PLAN_SKINNY && plan.kind != PLAN_DECODE) {
        // the tiled, packed and flat plans store plain product words; their epilogue is a pass of its own
        const long long cells = (long long)m * n;
        epilogue_rows_kernel<<<grid_for(cells, 256, sm_count(dev)), 256, 0, st>>>(c, cells, (int)n, g.epi);
        g_launches++;
    }
    CUDA_TRY(cudaGetLastError());
    return 0;
}

// Grow-only per-device scratch for the host-pointer twins.
constexpr int HOST_CHUNKS = 8; // row chunks of a pipelined host-pointer product
struct HostPool {
    void *buf[5] = {nullptr, nullptr, nullptr, nullptr, nullptr};
    size_t cap[5] = {0, 0, 0, 0, 0};
    cudaStream_t stream = nullptr;                      // compute (and the only stream of the unpipelined twins)
    cudaStream_t s_in = nullptr, s_out = nullptr;       // host-to-device and device-to-host copies of the pipelined product
    cudaEvent_t ev[1 + 2 * HOST_CHUNKS] = {};           // weight landed; chunk landed / chunk computed
    bool pipe_ready = false;
};
HostPool g_pool[64];
std::mutex g_pool_mu;

cudaError_t pool_get(int dev, int slot, size_t bytes, void **out) {
    HostPool &p = g_pool[dev];
    if (p.cap[slot] < bytes) {
        if (p.buf[slot]) cudaFree(p.buf[slot]);
        p.buf[slot] = nullptr;
        p.cap[slot] = 0;
        size_t want = bytes + (bytes >> 3) + 256;
        cudaError_t e = cudaMalloc(&p.buf[slot], want);
        if (e != cudaSuccess) return e;
        p.cap[slot] = want;
    }
    *out = p.buf[slot];
    return cudaSuccess;
}

size_t wkind_elem_bytes(int wkind) { return wkind == W_F32 ? 4 : (wkind == W_BF16 ? 2 : 1); }

} // namespace


extern "C" {

int64_t b200i_abi(void) { return 1; }
int64_t b200i_numeric_mode(void) { return 1; }
int64_t b200i_profile_version(void) { return 1; }
int64_t b200i_lowbit_profile_version(void) { return 1; }
const char *b200i_numerical_profile(void) { return "mojolearn.identical.gemm.fp32.v1"; }
const char *b200i_vendor(void) { return "cuda"; }
int64_t b200i_device_count(void) {
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess) { cudaGetLastError(); return 0; }
    return n;
}
int64_t b200i_launch_count(void) { return g_launches.load(); }
int64_t b200i_decode_plan_fits(int64_t m, int64_t n, int64_t k, int64_t op, int64_t wkind) {
    return decode_plan_fits(m, n, k, (int)op, (int)wkind) ? 1 : 0;
}

int64_t b200i_decode_status(int64_t device) {
    if (device >= 0 && cudaSetDevice((int)device) != cudaSuccess) { cudaGetLastError(); return -1; }
    int v = 0, zero = 0;
    if (cudaMemcpyFromSymbol(&v, g_decode_status, sizeof(int)) != cudaSuccess) { cudaGetLastError(); return -1; }
    if (v != 0 && cudaMemcpyToSymbol(g_decode_status, &zero, sizeof(int)) != cudaSuccess) { cudaGetLastError(); return -1; }
    return v;
}

int64_t b200i_debug_set_status(int64_t device, int64_t value) {
    if (device >= 0 && cudaSetDevice((int)device) != cudaSuccess) { cudaGetLastError(); return -1; }
    const int v = (int)value;
    if (cudaMemcpyToSymbol(g_decode_status, &v, sizeof(int)) != cudaSuccess) { cudaGetLastError(); return -1; }
    return 0;
}

int64_t b200i_workspace_bytes(int64_t m, int64_t n, int64_t k) {
    if (m <= 0 || n <= 0 || k <= 0) return 0;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) { cudaGetLastError(); dev = -1; }
    Plan p = choose_plan(m, n, k, sm_count(dev));
    int groups = p.groups;
    if (packed_candidate(p.kind, m, n, k))
        return (int64_t)packed_need(m, n, k, packed_split(p, m, n, k, sm_count(dev)).groups);
    if (skinny_plan_fits(m, n, k, OP_NT)) { // the plan an NT product with aligned operands takes instead
        for (int lowbit = 0; lowbit < 2; lowbit++) {
            const Plan q = choose_skinny(m, n, k, sm_count(dev), lowbit != 0);
            if (q.groups > groups) groups = q.groups;
        }
    }
    return groups > 1 ? (int64_t)groups * m * n * 4 : 0;
}

int64_t b200i_kernel_timing(int64_t enable) {
    std::lock_guard<std::mutex> lock(g_timing_mu);
    g_timing.on = enable != 0;
    if (enable) g_timing.used = 0;
    return 0;
}

int64_t b200i_kernel_timing_read(double *total_ms, int64_t *launches) {
    std::lock_guard<std::mutex> lock(g_timing_mu);
    double sum = 0.0;
    for (int i = 0; i < g_timing.used; i++) {
        float ms = 0.f;
        if (cudaEventSynchronize(g_timing.ev[2 * i + 1]) != cudaSuccess ||
            cudaEventElapsedTime(&ms, g_timing.ev[2 * i], g_timing.ev[2 * i + 1]) != cudaSuccess) {
            cudaGetLastError();
            return 1;
        }
        sum += ms;
    }
    if (total_ms) *total_ms = sum;
    if (launches) *launches = g_timing.used;
    g_timing.used = 0;
    return 0;
}

int64_t b200i_plan_workspace_bytes(int64_t m, int64_t n, int64_t k, int64_t plan, int64_t group_leaves) {
    if (m <= 0 || n <= 0 || k <= 0) return 0;
    if (plan == PLAN_AUTO) return b200i_workspace_bytes(m, n, k);
    const int64_t leaves = leaf_count(k);
    int64_t s = group_leaves > 0 ? group_leaves : leaves;
    if (s > leaves) s = leaves;
    const int64_t groups = (plan == PLAN_FLAT || plan == PLAN_DECODE) ? 1 : (leaves + s - 1) / s;
    if (plan == PLAN_PACKED) return (int64_t)packed_need(m, n, k, (int)groups);
    return groups > 1 ? groups * m * n * 4 : 0;
}

int64_t b200i_pair_epilogue_fits(int64_t m, int64_t n, int64_t k, int64_t op) {
    return (skinny_plan_fits(m, n, k, (int)op) && n % 4 == 0) ? 1 : 0;
}

int64_t b200i_gemm_w_plan(int64_t device, void *stream, float *c, const float *a, const void *b, const void *bscale,
                          int64_t wkind, int64_t m, int64_t n, int64_t k, int64_t op, int64_t plan, int64_t group_leaves,
                          void *ws, int64_t ws_bytes, char *err, int64_t err_cap) {
    clear(err, err_cap);
    int dev;
    if (select_device(device, err, err_cap, &dev)) return 1;
    return launch_product(dev, static_cast<cudaStream_t>(stream), c, a, b, bscale, (int)wkind, m, n, k, (int)op, (int)plan,
                          group_leaves, ws, ws_bytes, err, err_cap);
}

int64_t b200i_gemm_w(int64_t device, void *stream, float *c, const float *a, const void *b, const void *bscale,
                     int64_t wkind, int64_t m, int64_t n, int64_t k, int64_t op, void *ws, int64_t ws_bytes, char *err,
                     int64_t err_cap) {
    return b200i_gemm_w_plan(device, stream, c, a, b, bscale, wkind, m, n, k, op, PLAN_AUTO, 0, ws, ws_bytes, err, err_cap);
}

int64_t b200i_gemm_f32(int64_t device, void *stream, float *c, const float *a, const float *b, int64_t m, int64_t n,
                       int64_t k, int64_t op, void *ws, int64_t ws_bytes, char *err, int64_t err_cap) {
    return b200i_gemm_w_plan(device, stream, c, a, b, nullptr, W_F32, m, n, k, op, PLAN_AUTO, 0, ws, ws_bytes, err, err_cap);
}

int64_t b200i_gemm_w_epilogue(int64_t device, void *stream, float *c, const float *a, const void *b, const void *bscale, int64_t wkind,
                              int64_t m, int64_t n, int64_t k, int64_t op, const float *bias, int64_t act, int64_t plan,
                              int64_t group_leaves, void *ws, int64_t ws_bytes, char *err, int64_t err_cap) {
    clear(err, err_cap);
    int dev;
    if (select_device(device, err, err_cap, &dev)) return 1;
    if (act < EPI_ACT_NONE || act > EPI_PAIR_GEGLU_TANH) return fail(err, err_cap, "identical gemm: unknown store activation %lld", (long long)act);
    if (bias && !aligned(bias, 4)) return fail(err, err_cap, "identical gemm: misaligned storage");
    return launch_product(dev, static_cast<cudaStream_t>(stream), c, a, b, bscale, (int)wkind, m, n, k, (int)op, (int)plan, group_leaves, ws,
                          ws_bytes, err, err_cap, Epilogue{bias, (int)act});
}

int64_t b200i_gemm_w_nodes(int64_t device, void *stream, float *c, const float *a, const void *b, const void *bscale, int64_t wkind,
                           int64_t m, int64_t n, int64_t k, int64_t op, const float *bias, int64_t act, void *ws, int64_t ws_bytes,
                           int64_t *nodes, char *err, int64_t err_cap) {
    clear(err, err_cap);
    int dev;
    if (select_device(device, err, err_cap, &dev)) return 1;
    if (!nodes) return fail(err, err_cap, "identical gemm: nowhere to report the node count");
    if (act < EPI_ACT_NONE || act > EPI_PAIR_GEGLU_TANH) return fail(err, err_cap, "identical gemm: unknown store activation %lld", (long long)act);
    if (bias && !aligned(bias, 4)) return fail(err, err_cap, "identical gemm: misaligned storage");
    return launch_product(dev, static_cast<cudaStream_t>(stream), c, a, b, bscale, (int)wkind, m, n, k, (int)op, PLAN_AUTO, 0, ws, ws_bytes, err,
                          err_cap, Epilogue{bias, (int)act}, nodes);
}

int64_t b200i_to_bf16(int64_t device, void *stream, uint16_t *dst, const float *src, int64_t count, char *err,
                      int64_t err_cap) {
    clear(err, err_cap);
    if (count < 0 || (count > 0 && (!dst || !src))) return fail(err, err_cap, "to_bf16: null storage or negative count");
    if (count == 0) return 0;
    int dev;
    if (select_device(device, err, err_cap, &dev)) return 1;
    to_bf16_kernel<<<grid_for((count + 3) / 4, 256, sm_count(dev)), 256, 0, static_cast<cudaStream_t>(stream)>>>(dst, src, count);
    g_launches++;
    CUDA_TRY(cudaGetLastError());
    return 0;
}

int64_t b200i_from_bf16(int64_t device, void *stream, float *dst, const uint16_t *src, int64_t count, char *err,
                        int64_t err_cap) {
    clear(err, err_cap);
    if (count < 0 || (count > 0 && (!dst || !src))) return fail(err, err_cap, "from_bf16: null storage or negative count");
    if (count == 0) return 0;
    int dev;
    if (select_device(device, err, err_cap, &dev)) return 1;
    from_bf16_kernel<<<grid_for((count + 3) / 4, 256, sm_count(dev)), 256, 0, static_cast<cudaStream_t>(stream)>>>(dst, src, count);
    g_launches++;
    CUDA_TRY(cudaGetLastError());
    return 0;
}

int64_t b200i_quantize_int8(int64_t device, void *stream, int8_t *codes, int32_t *exponents, const float *x, int64_t rows,
                            int64_t cols, char *err, int64_t err_cap) {
    clear(err, err_cap);
    if (rows <= 0 || cols <= 0) return fail(err, err_cap, "quantize_int8: rows and cols must be positive");
    if (!codes || !exponents || !x) return fail(err, err_cap, "quantize_int8: null storage");
    int dev;
    if (select_device(device, err, err_cap, &dev)) return 1;
    quantize_int8_kernel<<<grid_for(rows * 32, 256, sm_count(dev)), 256, 0, static_cast<cudaStream_t>(stream)>>>(reinterpret_cast<signed char *>(codes), exponents, x, rows, cols);
    g_launches++;
    CUDA_TRY(cudaGetLastError());
    return 0;
}

int64_t b200i_dequantize_int8(int64_t device, void *stream, float *y, const int8_t *codes, const int32_t *exponents,
                              int64_t rows, int64_t cols, char *err, int64_t err_cap) {
    clear(err, err_cap);
    if (rows <= 0 || cols <= 0) return fail(err, err_cap, "dequantize_int8: rows and cols must be positive");
    if (!codes || !exponents || !y) return fail(err, err_cap, "dequantize_int8: null storage");
    int dev;
    if (select_device(device, err, err_cap, &dev)) return 1;
    dequantize_int8_kernel<<<grid_for(rows * cols, 256, sm_count(dev)), 256, 0, static_cast<cudaStream_t>(stream)>>>(y, reinterpret_cast<const signed char *>(codes), exponents, rows, cols);
    g_launches++;
    CUDA_TRY(cudaGetLastError());
    return 0;
}

int64_t b200i_gemm_int8(int64_t device, void *stream, float *c, const int8_t *qa, const int32_t *ea, const int8_t *qb,
                        const int32_t *eb, int64_t m, int64_t n, int64_t k, char *err, int64_t err_cap) {
    clear(err, err_cap);
    if (m <= 0 || n <= 0 || k <= 0) return fail(err, err_cap, "identical int8 gemm: m, n and k must be positive");
    if (k > 131072) return fail(err, err_cap, "identical int8 gemm: k = %lld exceeds INT8_MAX_K = 131072", (long long)k);
    if (!c || !qa || !ea || !qb || !eb) return fail(err, err_cap, "identical int8 gemm: null storage");
    int dev;
    if (select_device(device, err, err_cap, &dev)) return 1;
    const long long cells = m * n;
    // the tensor-core kernel wherever its 16-byte copies are aligned (k a multiple of 16); one thread per cell otherwise
    if (gemm_int8_mma_fits(qa, qb, m, n, k)) {
        const signed char *sa = reinterpret_cast<const signed char *>(qa), *sb = reinterpret_cast<const signed char *>(qb);
        const int sms = sm_count(dev);
        // enough 128 x 256 tiles for every SM: the persistent kernel fed by tensor-map copies; else the per-tile kernel
        const long long wide = ((m + T8_BM - 1) / T8_BM) * ((n + T8_BN - 1) / T8_BN);
        if (wide < sms || !launch_gemm_int8_tma(c, sa, ea, sb, eb, (int)m, (int)n, (int)k, sms, static_cast<cudaStream_t>(stream)))
            launch_gemm_int8_mma(c, sa, ea, sb, eb, (int)m, (int)n, (int)k, sms, static_cast<cudaStream_t>(stream));
    }
    else
        gemm_int8_flat_kernel<<<(unsigned)((cells + 127) / 128), 128, 0, static_cast<cudaStream_t>(stream)>>>(c, reinterpret_cast<const signed char *>(qa), ea, reinterpret_cast<const signed char *>(qb), eb, (int)m, (int)n, (int)k);
    g_launches++;
    CUDA_TRY(cudaGetLastError());
    return 0;
}

int64_t b200i_quantize_int15(int64_t device, void *stream, int8_t *hi, int8_t *lo, int32_t *exponents, const float *x, int64_t rows,
                             int64_t cols, char *err, int64_t err_cap) {
    clear(err, err_cap);
    if (rows <= 0 || cols <= 0) return fail(err, err_cap, "quantize_int15: rows and cols must be positive");
    if (!hi || !lo || !exponents || !x) return fail(err, err_cap, "quantize_int15: null storage");
    int dev;
    if (select_device(device, err, err_cap, &dev)) return 1;
    quantize_int15_kernel<<<grid_for(rows * 32, 256, sm_count(dev)), 256, 0, static_cast<cudaStream_t>(stream)>>>(reinterpret_cast<signed char *>(hi), reinterpret_cast<signed char *>(lo), exponents, x, rows, cols);
    g_launches++;
    CUDA_TRY(cudaGetLastError());
    return 0;
}

int64_t b200i_dequantize_int15(int64_t device, void *stream, float *y, const int8_t *hi, const int8_t *lo, const int32_t *exponents,
                               int64_t rows, int64_t cols, char *err, int64_t err_cap) {
    clear(err, err_cap);
    if (rows <= 0 || cols <= 0) return fail(err, err_cap, "dequantize_int15: rows and cols must be positive");
    if (!hi || !lo || !exponents || !y) return fail(err, err_cap, "dequantize_int15: null storage");
    int dev;
    if (select_device(device, err, err_cap, &dev)) return 1;
    dequantize_int15_kernel<<<grid_for(rows * cols, 256, sm_count(dev)), 256, 0, static_cast<cudaStream_t>(stream)>>>(y, reinterpret_cast<const signed char *>(hi), reinterpret_cast<const signed char *>(lo), exponents, rows, cols);
    g_launches++;
    CUDA_TRY(cudaGetLastError());
    return 0;
}

int64_t b200i_gemm_int15(int64_t device, void *stream, float *c, const int8_t *ah, const int8_t *al, const int32_t *ea, const int8_t *bh,
                         const int8_t *bl, const int32_t *eb, int64_t m, int64_t n, int64_t k, char *err, int64_t err_cap) {
    clear(err, err_cap);
    if (m <= 0 || n <= 0 || k <= 0) return fail(err, err_cap, "identical int15 gemm: m, n and k must be positive");
    if (k > INT15_MAX_K) return fail(err, err_cap, "identical int15 gemm: k = %lld exceeds INT15_MAX_K = 65536", (long long)k);
    if (!c || !ah || !al || !ea || !bh || !bl || !eb) return fail(err, err_cap, "identical int15 gemm: null storage");
    int dev;
    if (select_device(device, err, err_cap, &dev)) return 1;
    const signed char *sah = reinterpret_cast<const signed char *>(ah), *sal = reinterpret_cast<const signed char *>(al);
    const signed char *sbh = reinterpret_cast<const signed char *>(bh), *sbl = reinterpret_cast<const signed char *>(bl);
    // the tensor-core plan wherever its 16-byte copies are aligned (k a multiple of 16); one thread per cell otherwise
    if (gemm_int15_mma_fits(ah, al, bh, bl, m, n, k)) {
        // enough 128 x 64 tiles for every SM: the persistent kernel fed by tensor-map copies; else the per-tile kernel
        const int sms = sm_count(dev);
        const long long tiles = ((m + T8_BM - 1) / T8_BM) * ((n + I15_TN - 1) / I15_TN);
        if (tiles < 2ll * sms || !launch_gemm_int15_tma(c, sah, sal, ea, sbh, sbl, eb, (int)m, (int)n, (int)k, sms, static_cast<cudaStream_t>(stream)))
            launch_gemm_int15_mma(c, sah, sal, ea, sbh, sbl, eb, (int)m, (int)n, (int)k, static_cast<cudaStream_t>(stream));
    }
    else
        gemm_int15_flat_kernel<<<(unsigned)((m * n + 127) / 128), 128, 0, static_cast<cudaStream_t>(stream)>>>(c, sah, sal, ea, sbh, sbl, eb, (int)m, (int)n, (int)k);
    g_launches++;
    CUDA_TRY(cudaGetLastError());
    return 0;
}

int64_t b200i_ffma_probe(int64_t device, void *stream, float *scratch, int64_t blocks, int64_t iters, int64_t packed,
                         char *err, int64_t err_cap) {
    clear(err, err_cap);
    if (!scratch || blocks <= 0 || iters <= 0) return fail(err, err_cap, "ffma_probe: bad arguments");
    int dev;
    if (select_device(device, err, err_cap, &dev)) return 1;
    ffma_probe_kernel<<<(unsigned)blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(scratch, (int)iters, (int)packed, 1.0f);
    g_launches++;
    CUDA_TRY(cudaGetLastError());
    return 0;
}

// ---- the product without any allocation ---------------------------------------------------------
// Scratch for the split plan lives in the library image itself: a fixed device array
// that every GPU loading the library carries until the process exits.
constexpr size_t STATIC_SCRATCH_BYTES = 16u << 20;
static __device__ __align__(256) unsigned char g_static_scratch[STATIC_SCRATCH_BYTES];
static void *g_static_scratch_ptr[MAX_DEVICES]; // per device: the array's DEVICE address (the symbol itself is only a host-side stand-in)
static std::mutex g_static_scratch_mu;

// The plan the allocation-free entry runs: the tile plan the cost model prefers when its leaf-group nodes fit the
// built-in scratch, else the same tiles with the leaves split into fewer, larger groups (powers of two, so every
// group is still a subtree of the contract's fold), down to no split at all, which needs no scratch. The bits do
// not depend on the split; only the number of CTAs does.
static Plan noalloc_plan(int64_t m, int64_t n, int64_t k, int sms) {
    Plan plan = choose_plan(m, n, k, sms);
    const int leaves = (int)leaf_count(k) > 0 ? (int)leaf_count(k) : 1;
    while (plan.groups > 1 && (int64_t)plan.groups * m * n * 4 > (int64_t)STATIC_SCRATCH_BYTES) {
        plan.group_leaves *= 2;
        plan.groups = (leaves + plan.group_leaves - 1) / plan.group_leaves;
    }
    if (plan.groups <= 1) { plan.groups = 1; plan.group_leaves = leaves; }
    return plan;
}

int64_t b200i_noalloc_scratch_bytes(int64_t m, int64_t n, int64_t k) {
    if (m <= 0 || n <= 0 || k <= 0) return 0;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) { cudaGetLastError(); dev = -1; }
    const Plan plan = noalloc_plan(m, n, k, sm_count(dev));
    return plan.groups > 1 ? (int64_t)plan.groups * m * n * 4 : 0;
}

int64_t b200i_gemm_f32_noalloc(int64_t device, void *stream, float *c, const float *a, const float *b, int64_t m, int64_t n,
                               int64_t k, int64_t op, char *err, int64_t err_cap) {
    clear(err, err_cap);
    int dev;
    if (select_device(device, err, err_cap, &dev)) return 1;
    void *scratch = nullptr;
    {
        std::lock_guard<std::mutex> lock(g_static_scratch_mu);
        if (!g_static_scratch_ptr[dev]) {
            // once per device, with that device current: ask the runtime where the array lives on it
            void *p = nullptr;
            CUDA_TRY(cudaGetSymbolAddress(&p, g_static_scratch));
            g_static_scratch_ptr[dev] = p;
        }
        scratch = g_static_scratch_ptr[dev];
    }
    if (m <= 0 || n <= 0 || k <= 0)
        return fail(err, err_cap, "identical gemm: m, n and k must be positive (got m=%lld n=%lld k=%lld)", (long long)m,
                    (long long)n, (long long)k);
    const Plan plan = noalloc_plan(m, n, k, sm_count(dev));
    const int64_t need = plan.groups > 1 ? (int64_t)plan.groups * m * n * 4 : 0;
    if (need > (int64_t)STATIC_SCRATCH_BYTES) // cannot happen while an unsplit plan needs no scratch; kept as the guard of that assumption
        return fail(err, err_cap,
                    "identical gemm: this shape needs %lld bytes of scratch and the built-in scratch holds %lld; "
                    "call b200i_gemm_f32 with scratch of b200i_workspace_bytes(m, n, k) bytes instead",
                    (long long)need, (long long)STATIC_SCRATCH_BYTES);
    t_no_timing = true; // the benchmark's event pairs are created on demand, which may allocate
    const int64_t rc = launch_product(dev, static_cast<cudaStream_t>(stream), c, a, b, nullptr, W_F32, m, n, k, (int)op, plan.kind,
                                      plan.groups > 1 ? plan.group_leaves : 0, scratch, (int64_t)STATIC_SCRATCH_BYTES, err, err_cap);
    t_no_timing = false;
    return rc;
}

// ---- decoder-block seams (device pointers, asynchronous on the caller's stream) ----------------

#define SEAM_PROLOGUE()                                          \
    clear(err, err_cap);                                         \
    int dev;                                                     \
    if (select_device(device, err, err_cap, &dev)) return 1;     \
    cudaStream_t st = static_cast<cudaStream_t>(stream)

int64_t b200i_norm(int64_t device, void *stream, float *out, const float *x, const float *w, const float *bias, int64_t rows,
                   int64_t width, double eps, int64_t kind, char *err, int64_t err_cap) {
    SEAM_PROLOGUE();
    if (rows <= 0 || width <= 0 || !out || !x || !w) return fail(err, err_cap, "norm: bad arguments");
    if (kind < NORM_RMS || kind > NORM_RMS_OFFSET) return fail(err, err_cap, "norm: norm kind %lld is not spelled", (long long)kind);
    if (bias && kind != NORM_LAYER) return fail(err, err_cap, "norm: an RMSNorm carries no bias (norm_bias needs layernorm)");
    const int wpc = rows >= 1024 ? 4 : 1; // warps (rows) per CTA: few rows spread over the SMs
    const size_t smem = (size_t)wpc * (size_t)((width + 3) & ~3ll) * sizeof(float);
    if (smem <= 200 * 1024) {
        static std::atomic<bool> configured[64];
        if (dev >= 0 && dev < 64 && !configured[dev]) {
            CUDA_TRY(cudaFuncSetAttribute(norm_rows_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
            configured[dev] = true;
        }
        norm_rows_kernel<<<(unsigned)((rows + wpc - 1) / wpc), 32 * wpc, smem, st>>>(out, x, w, bias, rows, (int)width, (float)eps, (int)kind,
                                                                                     nullptr, nullptr);
    } else {
        const long long threads = rows * 32;
        norm_kernel<<<(unsigned)((threads + 255) / 256), 256, 0, st>>>(out, x, w, bias, rows, (int)width, (float)eps, (int)kind);
    }
    g_launches++;
    CUDA_TRY(cudaGetLastError());
    return 0;
}

int64_t b200i_add_norm(int64_t device, void *stream, float *out, float *sum_out, const float *x, const float *delta, const float *w,
                       const float *bias, int64_t rows, int64_t width, double eps, int64_t kind, char *err, int64_t err_cap) {
    SEAM_PROLOGUE();
    if (rows <= 0 || width <= 0 || !out || !sum_out || !x || !delta || !w) return fail(err, err_cap, "add_norm: bad arguments");
    if (kind < NORM_RMS || kind > NORM_RMS_OFFSET) return fail(err, err_cap, "norm: norm kind %lld is not spelled", (long long)kind);
    if (bias && kind != NORM_LAYER) return fail(err, err_cap, "norm: an RMSNorm carries no bias (norm_bias needs layernorm)");
    const int wpc = rows >= 1024 ? 4 : 1;
    const size_t smem = (size_t)wpc * (size_t)((width + 3) & ~3ll) * sizeof(float);
    if (smem <= 200 * 1024) {
        static std::atomic<bool> configured[64];
        if (dev >= 0 && dev < 64 && !configured[dev]) {
            CUDA_TRY(cudaFuncSetAttribute(norm_rows_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
            configured[dev] = true;
        }
        norm_rows_kernel<<<(unsigned)((rows + wpc - 1) / wpc), 32 * wpc, smem, st>>>(out, x, w, bias, rows, (int)width, (float)eps, (int)kind,
                                                                                     delta, sum_out);
        g_launches++;
    } else { // a row too wide for shared memory: the two seams one after the other
        const long long count = rows * width;
        add_kernel<<<grid_for(count, 256, sm_count(dev)), 256, 0, st>>>(sum_out, x, delta, count);
        norm_kernel<<<(unsigned)((rows * 32 + 255) / 256), 256, 0, st>>>(out, sum_out, w, bias, rows, (int)width, (float)eps, (int)kind);
        g_launches += 2;
    }
    CUDA_TRY(cudaGetLastError());
    return 0;
}

int64_t b200i_qkv_rope_cache(int64_t device, void *stream, float *qr, float *kcache, float *vcache, const float *q, const float *k,
                             const float *v, int64_t src_ld, const float *cosv, const float *sinv, int64_t b, int64_t l,
                             int64_t n_heads, int64_t n_kv, int64_t head_dim, int64_t cap, int64_t pos0, const int32_t *position,
                             int64_t rope_dim, char *err, int64_t err_cap) {
    SEAM_PROLOGUE();
    if (rope_dim == 0) rope_dim = head_dim;
    if (rope_dim < 0 || rope_dim > head_dim || (rope_dim & 1))
        return fail(err, err_cap, "transformer: the rotary table's rope_dim %lld does not fit head_dim %lld REFUSED", (long long)rope_dim, (long long)head_dim);
    if (b <= 0 || l <= 0 || n_heads <= 0 || n_kv <= 0 || head_dim <= 0 || (head_dim & 1) || !qr || !kcache || !vcache || !q || !k || !v ||
        qr == q)
        return fail(err, err_cap, "qkv_rope_cache: bad arguments");
    if ((cosv == nullptr) != (sinv == nullptr)) return fail(err, err_cap, "qkv_rope_cache: give both tables or neither");
    if (!position) {
        if (pos0 < 0) return fail(err, err_cap, "qkv_rope_cache: bad arguments");
        if (pos0 + l > cap)
            return fail(err, err_cap, "transformer: this call would use %lld KV slots and the cache holds %lld REFUSED", (long long)(pos0 + l),
                        (long long)cap);
    } else if (l > cap) {
        return fail(err, err_cap, "qkv_rope_cache: bad arguments");
    }
    const long long total = b * l * (n_heads + 2 * n_kv) * head_dim;
    const long long ldq = src_ld ? src_ld : n_heads * head_dim, ldkv = src_ld ? src_ld : n_kv * head_dim;
    if (ldq < n_heads * head_dim || ldkv < n_kv * head_dim) return fail(err, err_cap, "qkv_rope_cache: the row pitch is below the row width");
    qkv_rope_cache_kernel<<<(unsigned)((total + 255) / 256), 256, 0, st>>>(qr, kcache, vcache, q, k, v, ldq, ldkv, cosv, sinv, (int)b, (int)l,
                                                                           (int)n_heads, (int)n_kv, (int)head_dim, (int)cap, (int)pos0,
                                                                           position, cosv ? 1 : 0, (int)rope_dim);
    g_launches++;
    CUDA_TRY(cudaGetLastError());
    return 0;
}

int64_t b200i_rope_table(int64_t device, void *stream, float *cosv, float *sinv, int64_t pos0, int64_t l, int64_t head_dim,
                         double theta, char *err, int64_t err_cap) {
    SEAM_PROLOGUE();
    if (l <= 0 || head_dim <= 0 || (head_dim & 1) || !cosv || !sinv) return fail(err, err_cap, "rope_table: bad arguments");
    if (pos0 < 0 || pos0 + l > 8192)
        return fail(err, err_cap, "rope_table: absolute position %lld is at or beyond 8192, the domain of the sine and cosine reduction",
                    (long long)(pos0 + l - 1));
    const long long n = l * (head_dim / 2);
    rope_table_kernel<<<(unsigned)((n + 127) / 128), 128, 0, st>>>(cosv, sinv, (int)pos0, (int)l, (int)head_dim, (float)theta, nullptr);
    g_launches++;
    CUDA_TRY(cudaGetLastError());
    return 0;
}

int64_t b200i_rope_table_at(int64_t device, void *stream, float *cosv, float *sinv, const int32_t *position, int64_t l,
                            int64_t head_dim, double theta, char *err, int64_t err_cap) {
    SEAM_PROLOGUE();
    if (l <= 0 || head_dim <= 0 || (head_dim & 1) || !cosv || !sinv || !position) return fail(err, err_cap, "rope_table: bad arguments");
    const long long n = l * (head_dim / 2);
    rope_table_kernel<<<(unsigned)((n + 127) / 128), 128, 0, st>>>(cosv, sinv, 0, (int)l, (int)head_dim, (float)theta, position);
    g_launches++;
    CUDA_TRY(cudaGetLastError());
    return 0;
}

int64_t b200i_rope_table_opts(int64_t device, void *stream, float *cosv, float *sinv, int64_t pos0, const int32_t *position, int64_t l,
                              int64_t rope_dim, double theta, int64_t scaling, double factor, double low_freq_factor,
                              double high_freq_factor, int64_t original_max_positions, char *err, int64_t err_cap) {
    SEAM_PROLOGUE();
    if (l <= 0 || rope_dim <= 0 || (rope_dim & 1) || !cosv || !sinv) return fail(err, err_cap, "rope_table: bad arguments");
    if (scaling < 0 || scaling > 2) return fail(err, err_cap, "transformer options: rope_scaling %lld is not spelled", (long long)scaling);
    if (!(theta > 0.0) || (scaling != 0 && !(factor > 0.0))) return fail(err, err_cap, "transformer options: rope_theta and the rope_scaling factor must be positive");
    if (scaling == 2 && (!(low_freq_factor > 0.0) || !(high_freq_factor > 0.0) || high_freq_factor == low_freq_factor || original_max_positions <= 0))
        return fail(err, err_cap, "transformer options: llama3 rope_scaling needs positive, distinct frequency factors and original positions");
    if (!position && (pos0 < 0 || pos0 + l > 8192 * (scaling == 1 ? (long long)factor : 1)))
        return fail(err, err_cap, "rope_table: absolute position %lld puts the angle at or beyond 8192, the domain of the sine and cosine reduction",
                    (long long)(pos0 + l - 1));
    const long long n = l * (rope_dim / 2);
    RopeOptions o{(float)theta, (int)scaling, (float)factor, (float)low_freq_factor, (float)high_freq_factor, (int)original_max_positions};
    rope_table_opts_kernel<<<(unsigned)((n + 127) / 128), 128, 0, st>>>(cosv, sinv, (int)pos0, (int)l, (int)rope_dim, o, position);
    g_launches++;
    CUDA_TRY(cudaGetLastError());
    return 0;
}

int64_t b200i_rope_apply(int64_t device, void *stream, float *out, const float *src, const float *cosv, const float *sinv,
                         int64_t rows, int64_t l, int64_t n_heads, int64_t head_dim, int64_t src_ld, int64_t rope_dim, char *err,
                         int64_t err_cap) {
    SEAM_PROLOGUE();
    if (rope_dim == 0) rope_dim = head_dim;
    if (rope_dim < 0 || rope_dim > head_dim || (rope_dim & 1))
        return fail(err, err_cap, "transformer: the rotary table's rope_dim %lld does not fit head_dim %lld REFUSED", (long long)rope_dim, (long long)head_dim);
    if (rows <= 0 || l <= 0 || n_heads <= 0 || head_dim <= 0 || (head_dim & 1) || !out || !src || out == src)
        return fail(err, err_cap, "rope_apply: bad arguments (the rotation is not in place)");
    if (src_ld == 0) src_ld = n_heads * head_dim;
    if (src_ld < n_heads * head_dim) return fail(err, err_cap, "rope_apply: the row pitch is below the row width");
    const long long n = rows * n_heads * head_dim;
    rope_apply_kernel<<<(unsigned)((n + 255) / 256), 256, 0, st>>>(out, src, cosv, sinv, rows, (int)l, (int)n_heads, (int)head_dim, src_ld, (int)rope_dim);
    g_launches++;
    CUDA_TRY(cudaGetLastError());
    return 0;
}

int64_t b200i_kv_append(int64_t device, void *stream, float *cache, const float *src, int64_t b, int64_t l, int64_t n_kv,
                        int64_t head_dim, int64_t cap, int64_t pos0, int64_t src_ld, char *err, int64_t err_cap) {
    SEAM_PROLOGUE();
    if (src_ld == 0) src_ld = n_kv * head_dim;
    if (b <= 0 || l <= 0 || n_kv <= 0 || head_dim <= 0 || pos0 < 0 || !cache || !src || src_ld < n_kv * head_dim)
        return fail(err, err_cap, "kv_append: bad arguments");
    if (pos0 + l > cap)
        return fail(err, err_cap, "transformer: this call would use %lld KV slots and the cache holds %lld REFUSED", (long long)(pos0 + l),
                    (long long)cap);
    const long long n = b * l * n_kv * head_dim;
    kv_append_kernel<<<(unsigned)((n + 255) / 256), 256, 0, st>>>(cache, src, (int)b, (int)l, (int)n_kv, (int)head_dim, (int)cap, (int)pos0,
                                                                  nullptr, src_ld);
    g_launches++;
    CUDA_TRY(cudaGetLastError());
    return 0;
}

int64_t b200i_kv_append_at(int64_t device, void *stream, float *cache, const float *src, int64_t b, int64_t l, int64_t n_kv,
                           int64_t head_dim, int64_t cap, const int32_t *position, int64_t src_ld, char *err, int64_t err_cap) {
    SEAM_PROLOGUE();
    if (src_ld == 0) src_ld = n_kv * head_dim;
    if (b <= 0 || l <= 0 || n_kv <= 0 || head_dim <= 0 || l > cap || !cache || !src || !position || src_ld < n_kv * head_dim)
        return fail(err, err_cap, "kv_append: bad arguments");
    const long long n = b * l * n_kv * head_dim;
    kv_append_kernel<<<(unsigned)((n + 255) / 256), 256, 0, st>>>(cache, src, (int)b, (int)l, (int)n_kv, (int)head_dim, (int)cap, 0, position,
                                                                  src_ld);
    g_launches++;
    CUDA_TRY(cudaGetLastError());
    return 0;
}

// `s_grid` sizes the launch (the key count, or its upper bound when the position is read on the device)
static int64_t attention_launch(int dev, cudaStream_t st, float *ctx, const float *q, const float *kcache, const float *vcache,
                                float *scores, int64_t b, int64_t l, int64_t n_heads, int64_t n_kv, int64_t head_dim, int64_t cap,
                                int key_lo, int s, int own0, int s_grid, int64_t window, const int32_t *position, float softcap,
                                char *err, int64_t err_cap) {
    if (l >= 2 && l <= ATT_SMALL_Q && head_dim % 4 == 0 && head_dim <= K_LEAF_MIN) {
        // A few query rows per sequence (a chunked prompt's tail, speculative steps): scores, softmax and value sum in
        // one kernel, the score rows in shared memory, every key and value row read once for all the query rows. The
        // fewer CTAs the call has, the more shared memory each one spends on bytes in flight. A single query row
        // stays on the two kernels below: measured on B200 (batch 32, 16 heads, 1030 keys) the fused form is 8 %
        // slower on the whole decode step there, because its CTAs run their score, softmax and value phases in step
        // and the memory system idles through everyone's serial softmax, and with few (sequence, head) pairs the
        // scores kernel's split over key tiles is what keeps all SMs loading.
        const int lq = l == 1 ? 1 : (l == 2 ? 2 : (l <= 4 ? 4 : 8));
        const long long ctas = b * n_heads;
        const int sms = sm_count(dev);
        long long per_sm = (ctas + sms - 1) / sms; // CTAs an SM must hold for the call to be one wave
        if (per_sm > 6) per_sm = 6;
        const long long fixed = (long long)lq * K_LEAF_MIN + (long long)lq * ((s_grid + 3) & ~3);
        const long long room = (226ll * 1024 / per_sm - 1280) / 4 - fixed; // floats for the key tiles / the value ring
        int kkeys = 32, nkb = (int)(room / (ATD_WARPS * 32 * ATT_KT_PITCH));
        if (nkb > 3) nkb = 3;
        if (nkb < 1) { // not even one full tile per warp: fewer keys per tile
            nkb = 1;
            kkeys = (int)(room / (ATD_WARPS * ATT_KT_PITCH));
        }
        const int vkeys = room >= 4ll * 32 * head_dim ? 32 : 16;
        int stages = (int)(room / (vkeys * head_dim));
        if (stages > ATD_MAX_STAGES) stages = ATD_MAX_STAGES;
        if (kkeys >= 8 && stages >= 2) {
            const size_t smem = attn_decode_smem(lq, s_grid, (int)head_dim, kkeys, nkb, vkeys, stages);
#define DECODE_FUSED(LQ)                                                                                                          \
    do {                                                                                                                          \
        static std::atomic<bool> configured[64];                                                                                  \
        if (dev >= 0 && dev < 64 && !configured[dev]) {                                                                           \
            CUDA_TRY(cudaFuncSetAttribute(attn_decode_kernel<LQ>, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024));      \
            configured[dev] = true;                                                                                               \
        }                                                                                                                         \
        attn_decode_kernel<LQ><<<(unsigned)ctas, ATD_THREADS, smem, st>>>(ctx, q, kcache, vcache, (int)b, (int)l, (int)n_heads,   \
                                                                          (int)n_kv, (int)head_dim, (int)cap, key_lo, s, own0,   \
                                                                          (int)window, position, s_grid, kkeys, nkb, vkeys,      \
                                                                          stages, softcap);                                      \
    } while (0)
            if (lq == 1) DECODE_FUSED(1);
            else if (lq == 2) DECODE_FUSED(2);
            else if (lq == 4) DECODE_FUSED(4);
            else DECODE_FUSED(8);
#undef DECODE_FUSED
            g_launches++;
            CUDA_TRY(cudaGetLastError());
            return 0;
        }
    }
    if (l <= ATT_SMALL_Q) {
        dim3 gs((unsigned)((s_grid + 127) / 128), (unsigned)(b * n_heads));
#define SCORES_SMALL(LQ)                                                                                                          \
    do {                                                                                                                          \
        static std::atomic<bool> configured[64];                                                                                          \
        if (dev >= 0 && dev < 64 && !configured[dev]) {                                                                           \
            CUDA_TRY(cudaFuncSetAttribute(attn_scores_small_kernel<LQ>, cudaFuncAttributeMaxDynamicSharedMemorySize,              \
                                          attn_scores_small_smem<LQ>()));                                                         \
            configured[dev] = true;                                                                                               \
        }                                                                                                                         \
        attn_scores_small_kernel<LQ><<<gs, 128, attn_scores_small_smem<LQ>(), st>>>(\
            scores, q, kcache, (int)b, (int)l, (int)n_heads, (int)n_kv, (int)head_dim, (int)cap, key_lo, s, own0, (int)window,    \
            position, softcap);                                                                                                   \
    } while (0)
        if (l == 1) SCORES_SMALL(1);
        else if (l == 2) SCORES_SMALL(2);
        else if (l <= 4) SCORES_SMALL(4);
        else SCORES_SMALL(8);
#undef SCORES_SMALL
    } else {
        dim3 g1((unsigned)((s_grid + ATT_T - 1) / ATT_T), (unsigned)((l + ATT_T - 1) / ATT_T), (unsigned)(b * n_heads));
        attn_scores_kernel<<<g1, 256, 0, st>>>(scores, q, kcache, (int)b, (int)l, (int)n_heads, (int)n_kv, (int)head_dim, (int)cap, key_lo, s,
                                                 own0, (int)window, position, softcap);
    }
    if (l <= ATT_SMALL_Q && (size_t)s_grid * sizeof(float) <= 40 * 1024) {
        static std::atomic<bool> configured[64];
        if (dev >= 0 && dev < 64 && !configured[dev]) {
            CUDA_TRY(cudaFuncSetAttribute(attn_context_row_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024));
            configured[dev] = true;
        }
        // enough CTAs per SM for one wave (four at most); the shared memory that leaves a CTA becomes ring stages
        const long long rows = b * n_heads * l;
        long long per_sm = (rows + sm_count(dev) - 1) / sm_count(dev);
        if (per_sm > 4) per_sm = 4;
        long long stages = ((226ll * 1024 / per_sm - 1280) / 4 - ((s_grid + 3) & ~3)) / (CTX_NB * head_dim);
        if (stages > CTX_ST_MAX) stages = CTX_ST_MAX;
        if (stages < CTX_ST) stages = CTX_ST;
        attn_context_row_kernel<<<(unsigned)rows, 128, attn_context_row_smem(s_grid, (int)head_dim, (int)stages), st>>>(
            ctx, scores, vcache, (int)b, (int)l, (int)n_heads, (int)n_kv, (int)head_dim, (int)cap, key_lo, s, own0, (int)window, position,
            s_grid, (int)stages);
    } else {
        dim3 g2((unsigned)((l + CTX_ROWS - 1) / CTX_ROWS), (unsigned)(b * n_heads));
#define CONTEXT_ROWS(DPL)                                                                                                     \
    attn_context_kernel<DPL><<<g2, 32 * CTX_WARPS, attn_context_smem((int)head_dim), st>>>(\
        ctx, scores, vcache, (int)b, (int)l, (int)n_heads, (int)n_kv, (int)head_dim, (int)cap, key_lo, s, own0, (int)window, position)
        if (head_dim <= 32) CONTEXT_ROWS(1);
        else if (head_dim <= 64) CONTEXT_ROWS(2);
        else CONTEXT_ROWS(4);
#undef CONTEXT_ROWS
    }
    g_launches += 2;
    CUDA_TRY(cudaGetLastError());
    return 0;
}

static int64_t attention_check(int64_t b, int64_t l, int64_t n_heads, int64_t n_kv, int64_t head_dim, const void *ctx, const void *q,
                               const void *kcache, const void *vcache, const void *scores, char *err, int64_t err_cap) {
    if (b <= 0 || l <= 0 || n_heads <= 0 || n_kv <= 0 || n_heads % n_kv != 0 || head_dim <= 0 || !ctx || !q || !kcache || !vcache || !scores)
        return fail(err, err_cap, "attention: bad arguments");
    if (head_dim > K_LEAF_MIN || head_dim > CTX_MAX_HD)
        return fail(err, err_cap, "attention: head_dim %lld above 128 needs the leaf partition of the product, which this kernel does not spell",
                    (long long)head_dim);
    if (b * n_heads > 65535) return fail(err, err_cap, "attention: batch x heads above 65535");
    return 0;
}

// A prompt's score block [b * heads, l, s] is consumed by the softmax / value kernel right after it is written, so it
// need not exist for the whole batch at once: above ATT_SCRATCH_FLOATS the batch is walked a few sequences at a time
// through one scratch. The bound only caps the scratch (4 GB): walking the serving benchmark's prompt one sequence at a time
// (a 67 MB block that stays in L2 between the two kernels instead of 2 GB through HBM) measured 5.5 % SLOWER on the whole
// prefill (2242 against 2124 ms), because eight launches of 512 value-chain CTAs have eight tails where one launch of 4096
// has one.
constexpr long long ATT_SCRATCH_FLOATS = 1ll << 30;
static int64_t attention_batch_chunk(int64_t b, int64_t l, int64_t n_heads, int64_t s_grid) {
    if (l <= ATT_SMALL_Q) return b;
    const long long per = (long long)n_heads * l * s_grid;
    long long c = per > 0 ? ATT_SCRATCH_FLOATS / per : b;
    if (c < 1) c = 1;
    return c < b ? c : b;
}
static int64_t attention_chunked(int dev, cudaStream_t st, float *ctx, const float *q, const float *kcache, const float *vcache, float *scores,
                                 int64_t b, int64_t l, int64_t n_heads, int64_t n_kv, int64_t head_dim, int64_t cap, int key_lo, int s, int own0,
                                 int s_grid, int64_t window, const int32_t *position, float softcap, char *err, int64_t err_cap) {
    const int64_t step = attention_batch_chunk(b, l, n_heads, s_grid);
    for (int64_t b0 = 0; b0 < b; b0 += step) {
        const int64_t nb = b - b0 < step ? b - b0 : step;
        const size_t qoff = (size_t)b0 * l * n_heads * head_dim, coff = (size_t)b0 * n_kv * cap * head_dim;
        if (attention_launch(dev, st, ctx + qoff, q + qoff, kcache + coff, vcache + coff, scores, nb, l, n_heads, n_kv, head_dim, cap, key_lo, s,
                             own0, s_grid, window, position, softcap, err, err_cap))
            return 1;
    }
    return 0;
}

int64_t b200i_attention_scratch_floats(int64_t b, int64_t l, int64_t n_heads, int64_t s) {
    if (b <= 0 || l <= 0 || n_heads <= 0 || s <= 0) return 0;
    return attention_batch_chunk(b, l, n_heads, s) * n_heads * l * s;
}

int64_t b200i_attention(int64_t device, void *stream, float *ctx, const float *q, const float *kcache, const float *vcache,
                        float *scores, int64_t b, int64_t l, int64_t n_heads, int64_t n_kv, int64_t head_dim, int64_t cap,
                        int64_t used, int64_t window, double softcap, char *err, int64_t err_cap) {
    SEAM_PROLOGUE();
    if (attention_check(b, l, n_heads, n_kv, head_dim, ctx, q, kcache, vcache, scores, err, err_cap)) return 1;
    if (used < l || used > cap) return fail(err, err_cap, "attention: the cache holds %lld positions, this call's %lld included", (long long)used, (long long)l);
    const int64_t pos0 = used - l;
    int64_t key_lo = 0;
    if (window > 0 && pos0 - (window - 1) > 0) key_lo = pos0 - (window - 1);
    const int s = (int)(used - key_lo), own0 = (int)(pos0 - key_lo);
    return attention_chunked(dev, st, ctx, q, kcache, vcache, scores, b, l, n_heads, n_kv, head_dim, cap, (int)key_lo, s, own0, s, window,
                             nullptr, (float)softcap, err, err_cap);
}

int64_t b200i_attention_at(int64_t device, void *stream, float *ctx, const float *q, const float *kcache, const float *vcache,
                           float *scores, int64_t b, int64_t l, int64_t n_heads, int64_t n_kv, int64_t head_dim, int64_t cap,
                           const int32_t *position, int64_t window, double softcap, char *err, int64_t err_cap) {
    SEAM_PROLOGUE();
    if (attention_check(b, l, n_heads, n_kv, head_dim, ctx, q, kcache, vcache, scores, err, err_cap)) return 1;
    if (!position || l > cap) return fail(err, err_cap, "attention: bad arguments");
    int64_t s_max = cap; // the most keys any position can see
    if (window > 0 && window - 1 + l < s_max) s_max = window - 1 + l;
    return attention_chunked(dev, st, ctx, q, kcache, vcache, scores, b, l, n_heads, n_kv, head_dim, cap, 0, (int)s_max, 0, (int)s_max, window,
                             position, (float)softcap, err, err_cap);
}

int64_t b200i_act_mul(int64_t device, void *stream, float *out, const float *gate, const float *up, int64_t rows, int64_t width,
                      int64_t in_ld, int64_t kind, int64_t interleaved, char *err, int64_t err_cap) {
    SEAM_PROLOGUE();
    const bool gated = kind == ACT_SWIGLU || kind == ACT_GEGLU_ERF || kind == ACT_GEGLU_TANH;
    if (interleaved) {
        if (!gated || !gate) return fail(err, err_cap, "act_mul: the interleaved layout is the gated MLP's");
        if (in_ld == 0) in_ld = 2 * width;
        if (in_ld < 2 * width) return fail(err, err_cap, "act_mul: bad arguments");
        up = gate + 1;
    } else if (in_ld == 0) {
        in_ld = width;
    }
    if (rows <= 0 || width <= 0 || (!interleaved && in_ld < width) || !out || !up || kind < ACT_SWIGLU || kind > ACT_GEGLU_TANH)
        return fail(err, err_cap, "act_mul: bad arguments");
    if (gated && !gate) return fail(err, err_cap, "act_mul: a gated MLP needs its gate projection");
    act_mul_kernel<<<grid_for(rows * width, 256, sm_count(dev)), 256, 0, st>>>(out, gate, up, rows, width, in_ld, (int)kind, interleaved ? 2 : 1);
    g_launches++;
    CUDA_TRY(cudaGetLastError());
    return 0;
}

int64_t b200i_add(int64_t device, void *stream, float *out, const float *a, const float *b, int64_t count, char *err, int64_t err_cap) {
    SEAM_PROLOGUE();
    if (count <= 0 || !out || !a || !b) return fail(err, err_cap, "add: bad arguments");
    add_kernel<<<grid_for(count, 256, sm_count(dev)), 256, 0, st>>>(out, a, b, count);
    g_launches++;
    CUDA_TRY(cudaGetLastError());
    return 0;
}

int64_t b200i_bias_add(int64_t device, void *stream, float *buf, const float *bias, int64_t rows, int64_t width, char *err,
                       int64_t err_cap) {
    SEAM_PROLOGUE();
    if (rows <= 0 || width <= 0 || !buf || !bias) return fail(err, err_cap, "bias_add: bad arguments");
    bias_add_kernel<<<grid_for(rows * width, 256, sm_count(dev)), 256, 0, st>>>(buf, bias, rows, (int)width);
    g_launches++;
    CUDA_TRY(cudaGetLastError());
    return 0;
}

int64_t b200i_embedding(int64_t device, void *stream, float *y, const float *table, const int32_t *ids, int64_t n, int64_t vocab,
                        int64_t width, int32_t *status, char *err, int64_t err_cap) {
    SEAM_PROLOGUE();
    if (n <= 0 || vocab <= 0 || width <= 0 || !y || !table || !ids || !status) return fail(err, err_cap, "embedding: bad arguments");
    embedding_kernel<<<grid_for(n * width, 256, sm_count(dev)), 256, 0, st>>>(y, table, ids, n, (int)vocab, (int)width, status);
    g_launches++;
    CUDA_TRY(cudaGetLastError());
    return 0;
}

int64_t b200i_add_positions(int64_t device, void *stream, float *x, const float *pos, int64_t rows, int64_t l, int64_t pos0,
                            int64_t width, char *err, int64_t err_cap) {
    SEAM_PROLOGUE();
    if (rows <= 0 || l <= 0 || width <= 0 || pos0 < 0 || !x || !pos) return fail(err, err_cap, "add_positions: bad arguments");
    add_positions_kernel<<<grid_for(rows * width, 256, sm_count(dev)), 256, 0, st>>>(x, pos, rows, (int)l, (int)pos0, (int)width, nullptr);
    g_launches++;
    CUDA_TRY(cudaGetLastError());
    return 0;
}

int64_t b200i_add_positions_at(int64_t device, void *stream, float *x, const float *pos, int64_t rows, int64_t l,
                               const int32_t *position, int64_t width, char *err, int64_t err_cap) {
    SEAM_PROLOGUE();
    if (rows <= 0 || l <= 0 || width <= 0 || !x || !pos || !position) return fail(err, err_cap, "add_positions: bad arguments");
    add_positions_kernel<<<grid_for(rows * width, 256, sm_count(dev)), 256, 0, st>>>(x, pos, rows, (int)l, 0, (int)width, position);
    g_launches++;
    CUDA_TRY(cudaGetLastError());
    return 0;
}

int64_t b200i_advance_position(int64_t device, void *stream, int32_t *position, int64_t delta, char *err, int64_t err_cap) {
    SEAM_PROLOGUE();
    if (!position) return fail(err, err_cap, "advance_position: bad arguments");
    advance_position_kernel<<<1, 1, 0, st>>>(position, (int)delta);
    g_launches++;
    CUDA_TRY(cudaGetLastError());
    return 0;
}

int64_t b200i_argmax(int64_t device, void *stream, int32_t *out, const float *logits, int64_t rows, int64_t vocab, char *err,
                     int64_t err_cap) {
    SEAM_PROLOGUE();
    if (rows <= 0 || vocab <= 0 || !out || !logits) return fail(err, err_cap, "argmax: bad arguments");
    argmax_kernel<<<(unsigned)rows, ARGMAX_THREADS, 0, st>>>(out, logits, (int)vocab);
    g_launches++;
    CUDA_TRY(cudaGetLastError());
    return 0;
}

// ---- exchange of finished output columns between the GPUs of one node (see comm.cuh) ---------------

namespace {
struct Comm {
    int dev = 0, rank = 0, world = 1;
    size_t bytes = 0;          // the exchange buffer: the receive areas of every site
    unsigned char *base = nullptr;
    int *epoch = nullptr;      // this rank's epoch word
    CommPeers peers{};
    bool mapped[COMM_MAX_WORLD] = {};
    bool local[COMM_MAX_WORLD] = {}; // attached by pointer inside this process (tests), not through an IPC handle
};
constexpr unsigned long long COMM_WAIT_NS = 4000000000ull; // a peer that has not delivered after 4 s is reported, not awaited
} // namespace

int64_t b200i_comm_create(int64_t device, int64_t rank, int64_t world, int64_t bytes, void **comm, char *err, int64_t err_cap) {
    clear(err, err_cap);
    if (!comm || world < 1 || world > COMM_MAX_WORLD || rank < 0 || rank >= world || bytes <= 0 || bytes % 16)
        return fail(err, err_cap, "comm_create: bad arguments (1 <= world <= %d, bytes a positive multiple of 16)", COMM_MAX_WORLD);
    int dev;
    if (select_device(device, err, err_cap, &dev)) return 1;
    Comm *c = new Comm();
    c->dev = dev; c->rank = (int)rank; c->world = (int)world;
    c->bytes = (size_t)bytes;
    cudaError_t e = cudaMalloc(reinterpret_cast<void **>(&c->base), c->bytes);
    if (e == cudaSuccess) e = cudaMalloc(reinterpret_cast<void **>(&c->epoch), 256);
    if (e == cudaSuccess) e = cudaMemset(c->base, 0, c->bytes); // tag 0 everywhere: no epoch ever has it
    if (e == cudaSuccess) e = cudaMemset(c->epoch, 0, 256);
    if (e == cudaSuccess) e = cudaDeviceSynchronize();
    if (e != cudaSuccess) {
        if (c->base) cudaFree(c->base);
        if (c->epoch) cudaFree(c->epoch);
        delete c;
        return fail(err, err_cap, "comm_create: %s", cudaGetErrorString(e));
    }
    c->peers.base[rank] = c->base;
    c->mapped[rank] = true;
    *comm = c;
    return 0;
}

int64_t b200i_comm_export(void *comm, void *handle, int64_t handle_bytes, char *err, int64_t err_cap) {
    clear(err, err_cap);
    Comm *c = static_cast<Comm *>(comm);
    if (!c || !handle || handle_bytes < (int64_t)sizeof(cudaIpcMemHandle_t)) return fail(err, err_cap, "comm_export: the handle buffer must hold %d bytes", (int)sizeof(cudaIpcMemHandle_t));
    CUDA_TRY(cudaSetDevice(c->dev));
    cudaIpcMemHandle_t h;
    CUDA_TRY(cudaIpcGetMemHandle(&h, c->base));
    memcpy(handle, &h, sizeof(h));
    return 0;
}

int64_t b200i_comm_attach(void *comm, int64_t peer, const void *handle, char *err, int64_t err_cap) {
    clear(err, err_cap);
    Comm *c = static_cast<Comm *>(comm);
    if (!c || !handle || peer < 0 || peer >= c->world || peer == c->rank || c->mapped[peer]) return fail(err, err_cap, "comm_attach: bad peer %lld", (long long)peer);
    CUDA_TRY(cudaSetDevice(c->dev));
    cudaIpcMemHandle_t h;
    memcpy(&h, handle, sizeof(h));
    void *p = nullptr;
    CUDA_TRY(cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess));
    c->peers.base[peer] = static_cast<unsigned char *>(p);
    c->mapped[peer] = true;
    return 0;
}

int64_t b200i_comm_attach_local(void *comm, int64_t peer, void *other, char *err, int64_t err_cap) {
    clear(err, err_cap);
    Comm *c = static_cast<Comm *>(comm), *o = static_cast<Comm *>(other);
    if (!c || !o || peer < 0 || peer >= c->world || peer == c->rank || c->mapped[peer] || o->rank != peer || o->world != c->world ||
        o->bytes != c->bytes || o->dev != c->dev)
        return fail(err, err_cap, "comm_attach_local: the other exchange must be rank %lld of the same world, size and device", (long long)peer);
    c->peers.base[peer] = o->base;
    c->mapped[peer] = c->local[peer] = true;
    return 0;
}

int64_t b200i_comm_advance(void *comm, void *stream, char *err, int64_t err_cap) {
    clear(err, err_cap);
    Comm *c = static_cast<Comm *>(comm);
    if (!c) return fail(err, err_cap, "comm_advance: no exchange");
    CUDA_TRY(cudaSetDevice(c->dev));
    comm_advance_kernel<<<1, 1, 0, static_cast<cudaStream_t>(stream)>>>(c->epoch);
    g_launches++;
    CUDA_TRY(cudaGetLastError());
    return 0;
}

int64_t b200i_comm_gather(void *comm, void *stream, int64_t mode, int64_t area_bytes, float *out, int64_t out_ld, const float *src,
                          int64_t m, int64_t w, int64_t src_ld, char *err, int64_t err_cap) {
    clear(err, err_cap);
    Comm *c = static_cast<Comm *>(comm);
    if (!c) return fail(err, err_cap, "comm_gather: no exchange");
    if (mode < COMM_SEND_RECV || mode > COMM_RECV) return fail(err, err_cap, "comm_gather: bad mode");
    for (int p = 0; p < c->world; p++)
        if (!c->mapped[p]) return fail(err, err_cap, "comm_gather: rank %d's buffer is not attached", p);
    if (!out || m <= 0 || w <= 0 || area_bytes < 0 || area_bytes % 16 || (mode != COMM_RECV && !src)) return fail(err, err_cap, "comm_gather: bad arguments");
    if (src_ld == 0) src_ld = w;
    if (out_ld == 0) out_ld = w * c->world;
    if (src_ld < w || out_ld < w * c->world) return fail(err, err_cap, "comm_gather: a row pitch is below its row width");
    if ((size_t)area_bytes + (size_t)m * (size_t)w * c->world * 8 > c->bytes)
        return fail(err, err_cap, "comm_gather: the site's receive areas do not fit the exchange buffer");
    CUDA_TRY(cudaSetDevice(c->dev));
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const bool pair = w % 2 == 0 && src_ld % 2 == 0 && out_ld % 2 == 0 && aligned(out, 8) && (mode == COMM_RECV || aligned(src, 8));
    const long long items = pair ? m * (w / 2) : m * w;
    long long blocks = (items + COMM_THREADS - 1) / COMM_THREADS;
    const long long cap = 2ll * sm_count(c->dev);
    const unsigned grid = (unsigned)(blocks < 1 ? 1 : (blocks > cap ? cap : blocks));
    if (pair)
        comm_gather_kernel<true><<<grid, COMM_THREADS, 0, st>>>(c->peers, c->epoch, src, src_ld, out, out_ld, area_bytes, (int)m, (int)w, c->world,
                                                                c->rank, (int)mode, COMM_WAIT_NS);
    else
        comm_gather_kernel<false><<<grid, COMM_THREADS, 0, st>>>(c->peers, c->epoch, src, src_ld, out, out_ld, area_bytes, (int)m, (int)w, c->world,
                                                                 c->rank, (int)mode, COMM_WAIT_NS);
    g_launches++;
    CUDA_TRY(cudaGetLastError());
    return 0;
}

int64_t b200i_comm_gather_nodes(void *comm, void *stream, int64_t mode, int64_t area_bytes, float *out, int64_t out_ld, const float *ws,
                                int64_t nodes, int64_t m, int64_t n, const float *bias, int64_t act, char *err, int64_t err_cap) {
    clear(err, err_cap);
    Comm *c = static_cast<Comm *>(comm);
    if (!c) return fail(err, err_cap, "comm_gather_nodes: no exchange");
    if (mode != COMM_SEND_RECV && mode != COMM_SEND) return fail(err, err_cap, "comm_gather_nodes: bad mode");
    for (int p = 0; p < c->world; p++)
        if (!c->mapped[p]) return fail(err, err_cap, "comm_gather_nodes: rank %d's buffer is not attached", p);
    if (act < EPI_ACT_NONE || act > EPI_PAIR_GEGLU_TANH) return fail(err, err_cap, "comm_gather_nodes: unknown store activation %lld", (long long)act);
    if (!out || !ws || m <= 0 || n <= 0 || n % 4 || nodes < 2 || nodes > MAX_GROUPS || area_bytes < 0 || area_bytes % 16 || m * n > 0x7FFFFFFFll)
        return fail(err, err_cap, "comm_gather_nodes: bad arguments (n a multiple of 4, 2 to %d nodes)", MAX_GROUPS);
    const int64_t w = act >= EPI_PAIR_SWIGLU ? n / 2 : n;
    if (out_ld == 0) out_ld = w * c->world;
    if (out_ld < w * c->world || out_ld % 2 || !aligned(out, 8) || !aligned(ws, 16) || (bias && !aligned(bias, 4)))
        return fail(err, err_cap, "comm_gather_nodes: misaligned storage or a row pitch below the row width");
    if ((size_t)area_bytes + (size_t)m * (size_t)w * c->world * 8 > c->bytes)
        return fail(err, err_cap, "comm_gather_nodes: the site's receive areas do not fit the exchange buffer");
    CUDA_TRY(cudaSetDevice(c->dev));
    const long long cells = m * n;
    const unsigned subs = (unsigned)((nodes + FOLD_SUB - 1) / FOLD_SUB);
    comm_fold_gather_kernel<<<(unsigned)((cells / 4 + 31) / 32), 32 * subs, 0, static_cast<cudaStream_t>(stream)>>>(
        c->peers, c->epoch, ws, (int)nodes, Epilogue{bias, (int)act}, out, out_ld, area_bytes, (int)m, (int)n, c->world, c->rank, (int)mode, COMM_WAIT_NS);
    g_launches++;
    CUDA_TRY(cudaGetLastError());
    return 0;
}

int64_t b200i_comm_destroy(void *comm) {
    Comm *c = static_cast<Comm *>(comm);
    if (!c) return 0;
    cudaSetDevice(c->dev);
    cudaDeviceSynchronize();
    for (int p = 0; p < c->world; p++)
        if (p != c->rank && c->mapped[p] && !c->local[p]) cudaIpcCloseMemHandle(c->peers.base[p]);
    cudaFree(c->base);
    cudaFree(c->epoch);
    cudaGetLastError();
    delete c;
    return 0;
}

// ---- host-pointer twins -------------------------------------------------------------------

// The host-pointer product, pipelined over three streams (PCIe is full duplex): host-to-device copies, packing and
// multiplying, device-to-host copies. A tall left operand (m >= 1024) is cut by ROWS: the weight crosses and is
// packed once, the rows of A cross in chunks while earlier chunks are multiplied and their rows of C return. A wide
// k-contiguous weight under a short left operand (op NT, n >= 2048) is cut by weight rows, that is by COLUMNS of C:
// A crosses and is packed once, the weight crosses in chunks, each chunk's columns are computed into a dense block
// and return through a strided copy. Every chunk is a product of its own, so the bits are those of the whole
// product (a cell reads one row of A and one row of the weight). Returns 0 done, 1 error, -1 not applicable (the
// caller runs the plain path).
static int64_t host_gemm_pipelined(int dev, HostPool &pool, float *c, const float *a, const void *b, const void *bscale, int wkind,
                                   int64_t m, int64_t n, int64_t k, int op, char *err, int64_t err_cap) {
    // cut the larger operand: its copy is the one worth hiding under the arithmetic and the return copy
    const bool rows_ok = op != OP_TN && m >= 4 * PACKED_MIN_EXTENT && n >= PACKED_MIN_EXTENT;
    const bool cols_ok = op == OP_NT && n >= 8 * PACKED_MIN_EXTENT && m >= 1;
    const bool weight_larger = (double)n * (double)wkind_elem_bytes(wkind) > 2.0 * (double)m * 4.0;
    const bool by_cols = cols_ok && (!rows_ok || weight_larger);
    const bool by_rows = rows_ok && !by_cols;
    if (!by_rows && !by_cols) return -1;
    const int64_t extent = by_rows ? m : n;
    const int64_t per = ((extent + 3) / 4 + PK_TILE - 1) / PK_TILE * PK_TILE; // about four chunks, whole tiles
    const int nch = (int)((extent + per - 1) / per);
    if (nch < 2 || nch > HOST_CHUNKS) return -1;
    if (!pool.pipe_ready) {
        CUDA_TRY(cudaStreamCreateWithFlags(&pool.s_in, cudaStreamNonBlocking));
        CUDA_TRY(cudaStreamCreateWithFlags(&pool.s_out, cudaStreamNonBlocking));
        for (auto &e : pool.ev) CUDA_TRY(cudaEventCreateWithFlags(&e, cudaEventDisableTiming));
        pool.pipe_ready = true;
    }
    const size_t es = wkind_elem_bytes(wkind);
    const size_t abytes = (size_t)m * k * 4, bbytes = (size_t)n * k * es, cbytes = (size_t)m * n * 4;
    const size_t sbytes = (wkind >= W_INT8_EXP) ? (size_t)n * 4 : 0;
    const size_t wsbytes = pk_workspace_bytes(m, n, k);
    void *da, *db, *dc, *ds = nullptr, *dw = nullptr;
    CUDA_TRY(pool_get(dev, 0, abytes, &da));
    CUDA_TRY(pool_get(dev, 1, bbytes, &db));
    CUDA_TRY(pool_get(dev, 2, cbytes, &dc));
    if (sbytes) CUDA_TRY(pool_get(dev, 3, sbytes, &ds));
    CUDA_TRY(pool_get(dev, 4, wsbytes, &dw));
    packed_configure();
    const int leaf = (int)leaf_size(k), leaves = (int)leaf_count(k), wpl = pk_windows_per_leaf(leaf);
    float *pa = static_cast<float *>(dw);
    float *pb = pa + pk_panel_floats(m, k);
    unsigned char *fa = reinterpret_cast<unsigned char *>(pb + pk_panel_floats(n, k));
    unsigned char *fb = fa + pk_flag_bytes(m, k);
    const bool k8 = (k % 8 == 0) && (leaves == 1 || leaf % 8 == 0);
    const int tiles_m = (int)((m + PK_TILE - 1) / PK_TILE), tiles_n = (int)((n + PK_TILE - 1) / PK_TILE);
    // everything queued below waits for whatever the compute stream still holds from an earlier call
    CUDA_TRY(cudaEventRecord(pool.ev[0], pool.stream));
    CUDA_TRY(cudaStreamWaitEvent(pool.s_in, pool.ev[0], 0));
    CUDA_TRY(cudaStreamWaitEvent(pool.s_out, pool.ev[0], 0));
    // the operand that is not cut crosses first and is packed once
    if (by_rows) {
        CUDA_TRY(cudaMemcpyAsync(db, b, bbytes, cudaMemcpyHostToDevice, pool.s_in));
        if (sbytes) CUDA_TRY(cudaMemcpyAsync(ds, bscale, sbytes, cudaMemcpyHostToDevice, pool.s_in));
    } else {
        CUDA_TRY(cudaMemcpyAsync(da, a, abytes, cudaMemcpyHostToDevice, pool.s_in));
    }
    CUDA_TRY(cudaEventRecord(pool.ev[0], pool.s_in));
    CUDA_TRY(cudaStreamWaitEvent(pool.stream, pool.ev[0], 0));
    if (by_rows) {
        PackArgs pbargs{pb, fb, db, ds, (int)n, (int)k, leaf, leaves, wpl, op == OP_NT, op == OP_NT && k8};
        launch_pack_b(pbargs, wkind, pool.stream);
    } else {
        PackArgs paargs{pa, fa, da, nullptr, (int)m, (int)k, leaf, leaves, wpl, 1, k8};
        launch_pack<W_F32>(paargs, pool.stream);
    }
    g_launches++;
    for (int i = 0; i < nch; i++) {
        const int64_t x0 = i * per, cnt = (extent - x0 < per) ? extent - x0 : per;
        const int64_t tile0 = x0 / PK_TILE;
        if (by_rows) {
            float *dai = static_cast<float *>(da) + (size_t)x0 * k, *dci = static_cast<float *>(dc) + (size_t)x0 * n;
            CUDA_TRY(cudaMemcpyAsync(dai, a + (size_t)x0 * k, (size_t)cnt * k * 4, cudaMemcpyHostToDevice, pool.s_in));
            CUDA_TRY(cudaEventRecord(pool.ev[1 + 2 * i], pool.s_in));
            CUDA_TRY(cudaStreamWaitEvent(pool.stream, pool.ev[1 + 2 * i], 0));
            float *pai = pa + (size_t)tile0 * k * PK_TILE;
            unsigned char *fai = fa + (size_t)tile0 * leaves * wpl;
            PackArgs paargs{pai, fai, dai, nullptr, (int)cnt, (int)k, leaf, leaves, wpl, 1, k8};
            launch_pack<W_F32>(paargs, pool.stream);
            PackedGemmArgs p{pai, pb, fai, fb, dci, nullptr, (int)cnt, (int)n, (int)k, leaf, leaves, wpl, leaves, 1, tiles_n, (n % 4 == 0) ? 1 : 0};
            dim3 grid((unsigned)(((cnt + PK_TILE - 1) / PK_TILE) * tiles_n), 1u);
            gemm_packed_kernel<<<grid, PK_THREADS, PK_SMEM_BYTES, pool.stream>>>(p);
            CUDA_TRY(cudaEventRecord(pool.ev[2 + 2 * i], pool.stream));
            CUDA_TRY(cudaStreamWaitEvent(pool.s_out, pool.ev[2 + 2 * i], 0));
            CUDA_TRY(cudaMemcpyAsync(c + (size_t)x0 * n, dci, (size_t)cnt * n * 4, cudaMemcpyDeviceToHost, pool.s_out));
        } else {
            unsigned char *dbi = static_cast<unsigned char *>(db) + (size_t)x0 * k * es;
            float *dci = static_cast<float *>(dc) + (size_t)m * x0; // a dense [m, cnt] block
            CUDA_TRY(cudaMemcpyAsync(dbi, static_cast<const unsigned char *>(b) + (size_t)x0 * k * es, (size_t)cnt * k * es,
                                     cudaMemcpyHostToDevice, pool.s_in));
            if (sbytes)
                CUDA_TRY(cudaMemcpyAsync(static_cast<unsigned char *>(ds) + (size_t)x0 * 4, static_cast<const unsigned char *>(bscale) + (size_t)x0 * 4,
                                         (size_t)cnt * 4, cudaMemcpyHostToDevice, pool.s_in));
            CUDA_TRY(cudaEventRecord(pool.ev[1 + 2 * i], pool.s_in));
            CUDA_TRY(cudaStreamWaitEvent(pool.stream, pool.ev[1 + 2 * i], 0));
            float *pbi = pb + (size_t)tile0 * k * PK_TILE;
            unsigned char *fbi = fb + (size_t)tile0 * leaves * wpl;
            PackArgs pbargs{pbi, fbi, dbi, sbytes ? static_cast<unsigned char *>(ds) + (size_t)x0 * 4 : nullptr, (int)cnt, (int)k, leaf, leaves,
                            wpl, 1, k8};
            launch_pack_b(pbargs, wkind, pool.stream);
            const int tiles_nc = (int)((cnt + PK_TILE - 1) / PK_TILE);
            PackedGemmArgs p{pa, pbi, fa, fbi, dci, nullptr, (int)m, (int)cnt, (int)k, leaf, leaves, wpl, leaves, 1, tiles_nc,
                             (cnt % 4 == 0 && (m * x0) % 4 == 0) ? 1 : 0};
            dim3 grid((unsigned)(tiles_m * tiles_nc), 1u);
            gemm_packed_kernel<<<grid, PK_THREADS, PK_SMEM_BYTES, pool.stream>>>(p);
            CUDA_TRY(cudaEventRecord(pool.ev[2 + 2 * i], pool.stream));
            CUDA_TRY(cudaStreamWaitEvent(pool.s_out, pool.ev[2 + 2 * i], 0));
            CUDA_TRY(cudaMemcpy2DAsync(c + x0, (size_t)n * 4, dci, (size_t)cnt * 4, (size_t)cnt * 4, (size_t)m, cudaMemcpyDeviceToHost, pool.s_out));
        }
        g_launches += 2;
    }
    CUDA_TRY(cudaGetLastError());
    CUDA_TRY(cudaStreamSynchronize(pool.s_out));
    CUDA_TRY(cudaStreamSynchronize(pool.stream));
    CUDA_TRY(cudaStreamSynchronize(pool.s_in));
    return check_wait_status(err, err_cap, "identical gemm");
}

int64_t b200i_host_gemm_w(int64_t device, float *c, const float *a, const void *b, const void *bscale, int64_t wkind,
                          int64_t m, int64_t n, int64_t k, int64_t op, char *err, int64_t err_cap) {
    clear(err, err_cap);
    if (m <= 0 || n <= 0 || k <= 0)
        return fail(err, err_cap, "identical gemm: m, n and k must be positive (got m=%lld n=%lld k=%lld)", (long long)m,
                    (long long)n, (long long)k);
    if (wkind < W_F32 || wkind > W_INT8_SCALE) return fail(err, err_cap, "identical gemm: unknown weight kind %lld", (long long)wkind);
    if (!c || !a || !b) return fail(err, err_cap, "identical gemm: null storage");
    int dev;
    if (select_device(device, err, err_cap, &dev)) return 1;
    std::lock_guard<std::mutex> lock(g_pool_mu);
    HostPool &pool = g_pool[dev];
    if (!pool.stream) CUDA_TRY(cudaStreamCreateWithFlags(&pool.stream, cudaStreamNonBlocking));
    if (op != OP_NN && op != OP_NT && op != OP_TN) return fail(err, err_cap, "identical gemm: unknown op %lld", (long long)op);
    if ((wkind == W_INT8_EXP || wkind == W_INT8_SCALE) && (op != OP_NT || !bscale))
        return fail(err, err_cap, "identical gemm: int8 weight storage is row-scaled: it needs op NT and its per-row exponents or scales");
    {
        const int64_t piped = host_gemm_pipelined(dev, pool, c, a, b, bscale, (int)wkind, m, n, k, (int)op, err, err_cap);
        if (piped >= 0) return piped;
    }
    const size_t abytes = (size_t)m * k * 4, bbytes = (size_t)n * k * wkind_elem_bytes((int)wkind), cbytes = (size_t)m * n * 4;
    const size_t sbytes = (wkind >= W_INT8_EXP) ? (size_t)n * 4 : 0;
    const int64_t wsbytes = b200i_workspace_bytes(m, n, k);
    void *da, *db, *dc, *ds = nullptr, *dw = nullptr;
    CUDA_TRY(pool_get(dev, 0, abytes, &da));
    CUDA_TRY(pool_get(dev, 1, bbytes, &db));
    CUDA_TRY(pool_get(dev, 2, cbytes, &dc));
    if (sbytes) CUDA_TRY(pool_get(dev, 3, sbytes, &ds));
    if (wsbytes) CUDA_TRY(pool_get(dev, 4, (size_t)wsbytes, &dw));
    CUDA_TRY(cudaMemcpyAsync(da, a, abytes, cudaMemcpyHostToDevice, pool.stream));
    CUDA_TRY(cudaMemcpyAsync(db, b, bbytes, cudaMemcpyHostToDevice, pool.stream));
    if (sbytes) {
        if (!bscale) return fail(err, err_cap, "identical gemm: int8 weight storage needs its per-row exponents or scales");
        CUDA_TRY(cudaMemcpyAsync(ds, bscale, sbytes, cudaMemcpyHostToDevice, pool.stream));
    }
    if (launch_product(dev, pool.stream, static_cast<float *>(dc), static_cast<const float *>(da), db, ds, (int)wkind, m, n, k,
                       (int)op, PLAN_AUTO, 0, dw, wsbytes, err, err_cap))
        return 1;
    CUDA_TRY(cudaMemcpyAsync(c, dc, cbytes, cudaMemcpyDeviceToHost, pool.stream));
    CUDA_TRY(cudaStreamSynchronize(pool.stream));
    return check_wait_status(err, err_cap, "identical gemm");
}

#define HOST_PREP()                                                                  \
    clear(err, err_cap);                                                             \
    int dev;                                                                         \
    if (select_device(device, err, err_cap, &dev)) return 1;                         \
    std::lock_guard<std::mutex> lock(g_pool_mu);                                     \
    HostPool &pool = g_pool[dev];                                                    \
    if (!pool.stream) CUDA_TRY(cudaStreamCreateWithFlags(&pool.stream, cudaStreamNonBlocking))

int64_t b200i_host_to_bf16(int64_t device, uint16_t *dst, const float *src, int64_t count, char *err, int64_t err_cap) {
    if (count < 0) return fail(err, err_cap, "to_bf16: negative count");
    if (count == 0) { clear(err, err_cap); return 0; }
    HOST_PREP();
    void *ds, *dd;
    CUDA_TRY(pool_get(dev, 0, (size_t)count * 4, &ds));
    CUDA_TRY(pool_get(dev, 1, (size_t)count * 2, &dd));
    CUDA_TRY(cudaMemcpyAsync(ds, src, (size_t)count * 4, cudaMemcpyHostToDevice, pool.stream));
    if (b200i_to_bf16(dev, pool.stream, static_cast<uint16_t *>(dd), static_cast<const float *>(ds), count, err, err_cap)) return 1;
    CUDA_TRY(cudaMemcpyAsync(dst, dd, (size_t)count * 2, cudaMemcpyDeviceToHost, pool.stream));
    CUDA_TRY(cudaStreamSynchronize(pool.stream));
    return check_wait_status(err, err_cap, "b200i host call");
}

int64_t b200i_host_from_bf16(int64_t device, float *dst, const uint16_t *src, int64_t count, char *err, int64_t err_cap) {
    if (count < 0) return fail(err, err_cap, "from_bf16: negative count");
    if (count == 0) { clear(err, err_cap); return 0; }
    HOST_PREP();
    void *ds, *dd;
    CUDA_TRY(pool_get(dev, 0, (size_t)count * 2, &ds));
    CUDA_TRY(pool_get(dev, 1, (size_t)count * 4, &dd));
    CUDA_TRY(cudaMemcpyAsync(ds, src, (size_t)count * 2, cudaMemcpyHostToDevice, pool.stream));
    if (b200i_from_bf16(dev, pool.stream, static_cast<float *>(dd), static_cast<const uint16_t *>(ds), count, err, err_cap)) return 1;
    CUDA_TRY(cudaMemcpyAsync(dst, dd, (size_t)count * 4, cudaMemcpyDeviceToHost, pool.stream));
    CUDA_TRY(cudaStreamSynchronize(pool.stream));
    return check_wait_status(err, err_cap, "b200i host call");
}

int64_t b200i_host_quantize_int8(int64_t device, int8_t *codes, int32_t *exponents, const float *x, int64_t rows,
                                 int64_t cols, char *err, int64_t err_cap) {
    if (rows <= 0 || cols <= 0) return fail(err, err_cap, "quantize_int8: rows and cols must be positive");
    HOST_PREP();
    void *dx, *dq, *de;
    CUDA_TRY(pool_get(dev, 0, (size_t)rows * cols * 4, &dx));
    CUDA_TRY(pool_get(dev, 1, (size_t)rows * cols, &dq));
    CUDA_TRY(pool_get(dev, 2, (size_t)rows * 4, &de));
    CUDA_TRY(cudaMemcpyAsync(dx, x, (size_t)rows * cols * 4, cudaMemcpyHostToDevice, pool.stream));
    if (b200i_quantize_int8(dev, pool.stream, static_cast<int8_t *>(dq), static_cast<int32_t *>(de), static_cast<const float *>(dx),
                            rows, cols, err, err_cap))
        return 1;
    CUDA_TRY(cudaMemcpyAsync(codes, dq, (size_t)rows * cols, cudaMemcpyDeviceToHost, pool.stream));
    CUDA_TRY(cudaMemcpyAsync(exponents, de, (size_t)rows * 4, cudaMemcpyDeviceToHost, pool.stream));
    CUDA_TRY(cudaStreamSynchronize(pool.stream));
    return check_wait_status(err, err_cap, "b200i host call");
}

int64_t b200i_host_dequantize_int8(int64_t device, float *y, const int8_t *codes, const int32_t *exponents, int64_t rows,
                                   int64_t cols, char *err, int64_t err_cap) {
    if (rows <= 0 || cols <= 0) return fail(err, err_cap, "dequantize_int8: rows and cols must be positive");
    HOST_PREP();
    void *dy, *dq, *de;
    CUDA_TRY(pool_get(dev, 0, (size_t)rows * cols * 4, &dy));
    CUDA_TRY(pool_get(dev, 1, (size_t)rows * cols, &dq));
    CUDA_TRY(pool_get(dev, 2, (size_t)rows * 4, &de));
    CUDA_TRY(cudaMemcpyAsync(dq, codes, (size_t)rows * cols, cudaMemcpyHostToDevice, pool.stream));
    CUDA_TRY(cudaMemcpyAsync(de, exponents, (size_t)rows * 4, cudaMemcpyHostToDevice, pool.stream));
    if (b200i_dequantize_int8(dev, pool.stream, static_cast<float *>(dy), static_cast<const int8_t *>(dq),
                              static_cast<const int32_t *>(de), rows, cols, err, err_cap))
        return 1;
    CUDA_TRY(cudaMemcpyAsync(y, dy, (size_t)rows * cols * 4, cudaMemcpyDeviceToHost, pool.stream));
    CUDA_TRY(cudaStreamSynchronize(pool.stream));
    return check_wait_status(err, err_cap, "b200i host call");
}

int64_t b200i_host_gemm_int8(int64_t device, float *c, const int8_t *qa, const int32_t *ea, const int8_t *qb,
                             const int32_t *eb, int64_t m, int64_t n, int64_t k, char *err, int64_t err_cap) {
    if (m <= 0 || n <= 0 || k <= 0) return fail(err, err_cap, "identical int8 gemm: m, n and k must be positive");
    if (k > 131072) return fail(err, err_cap, "identical int8 gemm: k = %lld exceeds INT8_MAX_K = 131072", (long long)k);
    HOST_PREP();
    void *dqa, *dqb, *dc, *dea, *deb;
    CUDA_TRY(pool_get(dev, 0, (size_t)m * k, &dqa));
    CUDA_TRY(pool_get(dev, 1, (size_t)n * k, &dqb));
    CUDA_TRY(pool_get(dev, 2, (size_t)m * n * 4, &dc));
    CUDA_TRY(pool_get(dev, 3, (size_t)m * 4, &dea));
    CUDA_TRY(pool_get(dev, 4, (size_t)n * 4, &deb));
    CUDA_TRY(cudaMemcpyAsync(dqa, qa, (size_t)m * k, cudaMemcpyHostToDevice, pool.stream));
    CUDA_TRY(cudaMemcpyAsync(dqb, qb, (size_t)n * k, cudaMemcpyHostToDevice, pool.stream));
    CUDA_TRY(cudaMemcpyAsync(dea, ea, (size_t)m * 4, cudaMemcpyHostToDevice, pool.stream));
    CUDA_TRY(cudaMemcpyAsync(deb, eb, (size_t)n * 4, cudaMemcpyHostToDevice, pool.stream));
    if (b200i_gemm_int8(dev, pool.stream, static_cast<float *>(dc), static_cast<const int8_t *>(dqa), static_cast<const int32_t *>(dea),
                        static_cast<const int8_t *>(dqb), static_cast<const int32_t *>(deb), m, n, k, err, err_cap))
        return 1;
    CUDA_TRY(cudaMemcpyAsync(c, dc, (size_t)m * n * 4, cudaMemcpyDeviceToHost, pool.stream));
    CUDA_TRY(cudaStreamSynchronize(pool.stream));
    return check_wait_status(err, err_cap, "b200i host call");
}

int64_t b200i_host_quantize_int15(int64_t device, int8_t *hi, int8_t *lo, int32_t *exponents, const float *x, int64_t rows, int64_t cols,
                                  char *err, int64_t err_cap) {
    if (rows <= 0 || cols <= 0) return fail(err, err_cap, "quantize_int15: rows and cols must be positive");
    HOST_PREP();
    void *dx, *dh, *dl, *de;
    CUDA_TRY(pool_get(dev, 0, (size_t)rows * cols * 4, &dx));
    CUDA_TRY(pool_get(dev, 1, (size_t)rows * cols, &dh));
    CUDA_TRY(pool_get(dev, 2, (size_t)rows * cols, &dl));
    CUDA_TRY(pool_get(dev, 3, (size_t)rows * 4, &de));
    CUDA_TRY(cudaMemcpyAsync(dx, x, (size_t)rows * cols * 4, cudaMemcpyHostToDevice, pool.stream));
    if (b200i_quantize_int15(dev, pool.stream, static_cast<int8_t *>(dh), static_cast<int8_t *>(dl), static_cast<int32_t *>(de),
                             static_cast<const float *>(dx), rows, cols, err, err_cap))
        return 1;
    CUDA_TRY(cudaMemcpyAsync(hi, dh, (size_t)rows * cols, cudaMemcpyDeviceToHost, pool.stream));
    CUDA_TRY(cudaMemcpyAsync(lo, dl, (size_t)rows * cols, cudaMemcpyDeviceToHost, pool.stream));
    CUDA_TRY(cudaMemcpyAsync(exponents, de, (size_t)rows * 4, cudaMemcpyDeviceToHost, pool.stream));
    CUDA_TRY(cudaStreamSynchronize(pool.stream));
    return check_wait_status(err, err_cap, "b200i host call");
}

int64_t b200i_host_dequantize_int15(int64_t device, float *y, const int8_t *hi, const int8_t *lo, const int32_t *exponents, int64_t rows,
                                    int64_t cols, char *err, int64_t err_cap) {
    if (rows <= 0 || cols <= 0) return fail(err, err_cap, "dequantize_int15: rows and cols must be positive");
    HOST_PREP();
    void *dy, *dh, *dl, *de;
    CUDA_TRY(pool_get(dev, 0, (size_t)rows * cols * 4, &dy));
    CUDA_TRY(pool_get(dev, 1, (size_t)rows * cols, &dh));
    CUDA_TRY(pool_get(dev, 2, (size_t)rows * cols, &dl));
    CUDA_TRY(pool_get(dev, 3, (size_t)rows * 4, &de));
    CUDA_TRY(cudaMemcpyAsync(dh, hi, (size_t)rows * cols, cudaMemcpyHostToDevice, pool.stream));
    CUDA_TRY(cudaMemcpyAsync(dl, lo, (size_t)rows * cols, cudaMemcpyHostToDevice, pool.stream));
    CUDA_TRY(cudaMemcpyAsync(de, exponents, (size_t)rows * 4, cudaMemcpyHostToDevice, pool.stream));
    if (b200i_dequantize_int15(dev, pool.stream, static_cast<float *>(dy), static_cast<const int8_t *>(dh), static_cast<const int8_t *>(dl),
                               static_cast<const int32_t *>(de), rows, cols, err, err_cap))
        return 1;
    CUDA_TRY(cudaMemcpyAsync(y, dy, (size_t)rows * cols * 4, cudaMemcpyDeviceToHost, pool.stream));
    CUDA_TRY(cudaStreamSynchronize(pool.stream));
    return check_wait_status(err, err_cap, "b200i host call");
}

int64_t b200i_host_gemm_int15(int64_t device, float *c, const int8_t *ah, const int8_t *al, const int32_t *ea, const int8_t *bh,
                              const int8_t *bl, const int32_t *eb, int64_t m, int64_t n, int64_t k, char *err, int64_t err_cap) {
    if (m <= 0 || n <= 0 || k <= 0) return fail(err, err_cap, "identical int15 gemm: m, n and k must be positive");
    if (k > INT15_MAX_K) return fail(err, err_cap, "identical int15 gemm: k = %lld exceeds INT15_MAX_K = 65536", (long long)k);
    HOST_PREP();
    // the two planes of an operand share one pool slot, the second one 256-byte aligned behind the first
    const size_t aplane = ((size_t)m * k + 255) / 256 * 256, bplane = ((size_t)n * k + 255) / 256 * 256;
    void *da, *db, *dc, *dea, *deb;
    CUDA_TRY(pool_get(dev, 0, 2 * aplane, &da));
    CUDA_TRY(pool_get(dev, 1, 2 * bplane, &db));
    CUDA_TRY(pool_get(dev, 2, (size_t)m * n * 4, &dc));
    CUDA_TRY(pool_get(dev, 3, (size_t)m * 4, &dea));
    CUDA_TRY(pool_get(dev, 4, (size_t)n * 4, &deb));
    int8_t *dah = static_cast<int8_t *>(da), *dal = dah + aplane, *dbh = static_cast<int8_t *>(db), *dbl = dbh + bplane;
    CUDA_TRY(cudaMemcpyAsync(dah, ah, (size_t)m * k, cudaMemcpyHostToDevice, pool.stream));
    CUDA_TRY(cudaMemcpyAsync(dal, al, (size_t)m * k, cudaMemcpyHostToDevice, pool.stream));
    CUDA_TRY(cudaMemcpyAsync(dbh, bh, (size_t)n * k, cudaMemcpyHostToDevice, pool.stream));
    CUDA_TRY(cudaMemcpyAsync(dbl, bl, (size_t)n * k, cudaMemcpyHostToDevice, pool.stream));
    CUDA_TRY(cudaMemcpyAsync(dea, ea, (size_t)m * 4, cudaMemcpyHostToDevice, pool.stream));
    CUDA_TRY(cudaMemcpyAsync(deb, eb, (size_t)n * 4, cudaMemcpyHostToDevice, pool.stream));
    if (b200i_gemm_int15(dev, pool.stream, static_cast<float *>(dc), dah, dal, static_cast<const int32_t *>(dea), dbh, dbl,
                         static_cast<const int32_t *>(deb), m, n, k, err, err_cap))
        return 1;
    CUDA_TRY(cudaMemcpyAsync(c, dc, (size_t)m * n * 4, cudaMemcpyDeviceToHost, pool.stream));
    CUDA_TRY(cudaStreamSynchronize(pool.stream));
    return check_wait_status(err, err_cap, "b200i host call");
}

} // extern "C"
