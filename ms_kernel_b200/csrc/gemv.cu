// Host side of the weight-only GEMV entry points: argument checks, the split-K
// plan, kernel selection.  Replaces the launchers at csrc/w_gemv.cu:1410-1570
// of the reference.
#include <cstdlib>
#include <mutex>

#include "gemv_mma.cuh"
#include "gemv_umma.cuh"

namespace msaq {

// generic path, defined in gemv_generic.cu
size_t gemv_generic_workspace(int64_t M, int64_t OUT, int64_t NB);
int gemv_run_generic(const __nv_bfloat16* X, const int8_t* se, const uint8_t* up, const uint8_t* sh, void* Y,
                     float* Yf, int64_t M, int64_t OUT, int64_t NB, const Fmt& f, bool cm, void* ws,
                     cudaStream_t st);
namespace {

// ---- tuned path (u4/gs2, column-major planes, OUT % 16 == 0) --------------------
struct MmaPlan {
    GemvSchedule sch;        // sch.nb counts units of `kb` K blocks
    int kb;
    size_t xprep_off, xprep_bytes, partial_off, total;      // status word at 0, counters at 256, then these
};

bool mma_eligible(int64_t OUT, int u, int gs, bool cm) { return cm && u == 4 && gs == 2 && OUT % 16 == 0; }
// the tensor-memory kernel also decodes the 5+3 and 6+2 bit formats
bool umma_eligible(int64_t OUT, int u, int gs, bool cm) { return cm && u >= 2 && u <= 4 && gs == 2 && OUT % 16 == 0; }

MmaPlan plan_mma(int64_t M, int64_t OUT, int64_t NB, int fmt = GF_MSAQ_U4) {
    MmaPlan p;
    GemvSchedule& s = p.sch;
    const int64_t rows = M < GM_MP * GM_MAX_PASSES ? M : GM_MP * GM_MAX_PASSES;
    const int passes = (int)((rows + GM_MP - 1) / GM_MP);
    s.nb = (int)NB;
    p.kb = 1;
    long long slots = (long long)GM_CTAS_PER_SM * sm_count();
    // The smallest problems (a tensor-parallel shard of a few MB) run one CTA per SM: fewer partial sums per tile
    // to hand off and add up, and the whole of a CTA's share fits its ring at once (8192x1024 and 1280x8192, one
    // row: 13.3 / 14.1 -> 11.2 us; from about 10 MB on three CTAs per SM are faster again).
    if (OUT * NB * gm_col_bytes(fmt) <= (9LL << 20)) slots = sm_count();
    // Widest tile (fewest, largest TMA copies) that keeps the number of CTAs sharing one tile --
    // and with it the partial sums the finishing warp has to add up -- at or below 32.
    // The 1024-column tile (16 accumulators per thread, half as many barrier hand-offs per byte) pays for a
    // single row: 57344x8192 77 -> 68 us; with four rows it measured slower than 512 columns (41.7 against 32.7 us
    // on 28672x4096).
    // (the MXINT8 twin is built for 512- and 256-column tiles, one K block per stage)
    const int min_tc = fmt == GF_MXINT8 ? GM_MAX_TC / 4 : GM_GROUP;
    for (int tc = (M == 1 && fmt == GF_MSAQ_U4) ? GM_MAX_TC : GM_MAX_TC / 2; tc >= min_tc; tc >>= 1) {
        s.tc = tc;
        s.col_tiles = (int)((OUT + tc - 1) / tc);
        const long long units = s.units();
        s.grid = (int)(units < slots ? units : slots);
        if (tc == min_tc || (s.grid + s.col_tiles - 1) / s.col_tiles <= 32) break;      // 8, 16 and 64 measured slower
    }
    // Launches of one or two passes (up to eight rows) on half- or quarter-width tiles: two or four K blocks per ring
    // stage, for the same cut in hand-offs per byte the wider tile gives (8192x28672: 44.5 -> 41.3 us at one row,
    // 54.9 -> 50.8 us at four).
    if (fmt == GF_MSAQ_U4 && passes <= 2 && (s.tc == GM_MAX_TC / 2 || s.tc == GM_MAX_TC / 4) && NB >= 4) {
        p.kb = s.tc == GM_MAX_TC / 2 ? 2 : 4;           // the widest tile's bytes per stage either way
        s.nb = (int)((NB + p.kb - 1) / p.kb);
        const long long u2 = s.units();
        s.grid = (int)(u2 < slots ? u2 : slots);
    }
    const long long units = s.units();
    s.max_slots = (int)(((long long)s.nb * s.grid + units - 1) / units) + 1;
    const int per_sm = (s.grid + sm_count() - 1) / sm_count();
    const int stage = p.kb * gm_stage_bytes(s.tc, passes, fmt);
    int stages = (200 * 1024 / per_sm) / stage;
    if (stages > GM_MAX_STAGES) stages = GM_MAX_STAGES;
    if (stages < 2) stages = 2;
    s.stages = stages;
    p.xprep_bytes = ((size_t)NB * passes * GM_XREC + 255) & ~(size_t)255;
    const size_t ctl = (256 + (size_t)s.col_tiles * GM_WARPS * sizeof(unsigned long long) + 255) & ~(size_t)255;
    p.xprep_off = ctl > WS_CTL_BYTES ? ctl : WS_CTL_BYTES;            // the control region: status word, then the tile counters
    p.partial_off = p.xprep_off + p.xprep_bytes;
    p.total = p.partial_off + (((size_t)s.max_slots * rows * OUT * sizeof(float) + 255) & ~(size_t)255);
    return p;
}

template <int PASSES, int TC, int KB, bool INK, int FMT = GF_MSAQ_U4, bool PUSH = false>
int launch_mma_ink(const GemvMmaArgs& a, cudaStream_t st) {
    static int configured[64] = {};                      // largest dynamic smem size set per device
    const int smem = a.sch.stages * KB * gm_stage_bytes(TC, PASSES, FMT) + a.table_bytes;
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 64 && configured[dev] < smem) {
        if (cudaFuncSetAttribute(gemv_u4gs2_mma_kernel<PASSES, TC, KB, INK, FMT, PUSH>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 smem) != cudaSuccess)
            return fail(MSAQ_ERR_CUDA, "cannot reserve %d bytes of shared memory", smem);
        configured[dev] = smem;
    }
    launch_chained(gemv_u4gs2_mma_kernel<PASSES, TC, KB, INK, FMT, PUSH>, dim3(a.sch.grid), dim3(GM_THREADS), smem, st, a);
    count_launch();
    return check_launch(FMT == GF_MXINT8 ? "gemv_mxint8_mma" : "gemv_u4gs2_mma");
}

// the MXINT8 twin: half- or quarter-width tiles, one K block per stage, records from the staging kernel
template <int PASSES>
int launch_mma_mx(const GemvMmaArgs& a, cudaStream_t st) {
    return a.sch.tc == GM_MAX_TC / 2 ? launch_mma_ink<PASSES, GM_MAX_TC / 2, 1, false, GF_MXINT8>(a, st)
                                     : launch_mma_ink<PASSES, GM_MAX_TC / 4, 1, false, GF_MXINT8>(a, st);
}

template <int PASSES, int TC, int KB = 1>
int launch_mma(const GemvMmaArgs& a, cudaStream_t st) {
    if constexpr (TC < GM_GROUP) {
        return fail(MSAQ_ERR_ARG, "tile narrower than a column group");
    } else {
        if constexpr (PASSES <= 2) {                       // the push variant serves up to eight rows
            if (a.push.world) {
                if constexpr (PASSES == 1) {
                    if (a.xmode >= 0) return launch_mma_ink<PASSES, TC, KB, true, GF_MSAQ_U4, true>(a, st);
                }
                return launch_mma_ink<PASSES, TC, KB, false, GF_MSAQ_U4, true>(a, st);
            }
        }
        if (a.push.world) return fail(MSAQ_ERR_UNSUPPORTED, "the push variant serves up to eight rows");
        if constexpr (PASSES == 1) {
            if (a.xmode >= 0) return launch_mma_ink<PASSES, TC, KB, true>(a, st);
        }
        return launch_mma_ink<PASSES, TC, KB, false>(a, st);
    }
}

template <int PASSES>
int launch_mma_tc(const GemvMmaArgs& a, int kb, cudaStream_t st) {
    if (kb > 1) {
        if constexpr (PASSES <= 2)
            return kb == 2 ? launch_mma<PASSES, GM_MAX_TC / 2, 2>(a, st) : launch_mma<PASSES, GM_MAX_TC / 4, 4>(a, st);
        return fail(MSAQ_ERR_ARG, "several K blocks per stage are planned for launches of up to two passes only");
    }
    if (a.sch.tc == GM_MAX_TC) {
        if constexpr (PASSES == 1) return launch_mma<1, GM_MAX_TC>(a, st);
        return fail(MSAQ_ERR_ARG, "the widest tiles are planned for single-pass launches only");
    }
    if (a.sch.tc == GM_MAX_TC / 2) return launch_mma<PASSES, GM_MAX_TC / 2>(a, st);
    if (a.sch.tc == GM_MAX_TC / 4) return launch_mma<PASSES, GM_MAX_TC / 4>(a, st);
    return launch_mma<PASSES, GM_MAX_TC / 8>(a, st);
}

// ---- tensor-memory path (u4/gs2, column-major planes, OUT % 16 == 0, M >= GU_MIN_M) ----------
constexpr int64_t GU_MIN_M = 9;

struct UmmaPlan {
    GemvSchedule sch;
    size_t xs_bytes, ctl_off, partial_off, total;
};

UmmaPlan plan_umma(int64_t M, int64_t OUT, int64_t NB, int u) {
    UmmaPlan p;
    GemvSchedule& s = p.sch;
    const int64_t rows = M < GU_MAX_N ? M : GU_MAX_N;
    s.tc = GU_TR;
    s.nb = (int)NB;
    s.col_tiles = (int)((OUT + GU_TR - 1) / GU_TR);
    const long long units = s.units(), slots = sm_count();
    s.grid = (int)(units < slots ? units : slots);
    s.max_slots = (int)(((long long)s.nb * s.grid + units - 1) / units) + 1;
    int stages = (226 * 1024 - GU_ABUFS * GU_ABUF_BYTES) / gu_stage(u);
    if (stages > GU_MAX_STAGES) stages = GU_MAX_STAGES;
    s.stages = stages;
    p.xs_bytes = ((size_t)NB * GU_XTILE + 255) & ~(size_t)255;
    p.ctl_off = p.xs_bytes;                                        // status word
    p.partial_off = p.ctl_off + 256;
    p.total = p.partial_off + (((size_t)s.max_slots * rows * OUT * sizeof(float) + 255) & ~(size_t)255);
    return p;
}

template <int U>
int launch_umma(const GemvUmmaArgs& a, int smem, cudaStream_t st) {
    static int configured[64] = {};                      // largest dynamic smem size set per device
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 64 && configured[dev] < smem) {
        if (cudaFuncSetAttribute(gemv_umma_kernel<U>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess)
            return fail(MSAQ_ERR_CUDA, "cannot reserve %d bytes of shared memory", smem);
        configured[dev] = smem;
    }
    launch_chained(gemv_umma_kernel<U>, dim3(a.sch.grid), dim3(GU_THREADS), (size_t)smem, st, a);
    count_launch();
    return check_launch("gemv_umma");
}

int run_umma(const __nv_bfloat16* X, const int8_t* se, const uint8_t* up, const uint8_t* sh, void* Y, float* Yf,
             int64_t M, int64_t OUT, int64_t NB, int u, void* ws, cudaStream_t st) {
    const UmmaPlan p = plan_umma(M, OUT, NB, u);
    uint8_t* base = static_cast<uint8_t*>(ws) + WS_CTL_BYTES;
    int* status = reinterpret_cast<int*>(base + p.ctl_off);
    float* partial = reinterpret_cast<float*>(base + p.partial_off);
    for (int64_t m0 = 0; m0 < M; m0 += GU_MAX_N) {        // more than 128 rows: one launch pair per 128-row tile
        const int rows = (int)(M - m0 < GU_MAX_N ? M - m0 : GU_MAX_N);
        const int64_t threads = NB * ((rows + 7) / 8 * 8) * 4;
        launch_chained(gemv_umma_xprep_kernel, dim3((unsigned)((threads + 255) / 256)), dim3(256), 0, st,
                       X + m0 * NB * BLOCK, base, status, m0 == 0 ? 1 : 0, rows, (int)NB);
        count_launch();
        if (int rc = check_launch("gemv_umma_xprep")) return rc;
        const GemvSchedule sch = p.sch;
        const int smem = sch.stages * gu_stage(u) + GU_ABUFS * GU_ABUF_BYTES;
        GemvUmmaArgs a{se, up, sh, base, partial, status, sticky_status(), static_cast<__nv_bfloat16*>(Y), Yf, (int)m0, rows, (int)OUT, sch};
        const int rc = u == 4 ? launch_umma<4>(a, smem, st) : u == 3 ? launch_umma<3>(a, smem, st) : launch_umma<2>(a, smem, st);
        if (rc) return rc;
        // every CTA boundary on a tile boundary: all tiles were written directly; otherwise some tile has partials
        if (!(sch.units() % sch.grid == 0 && (sch.units() / sch.grid) % sch.nb == 0)) {
            const int64_t quads = (int64_t)rows * (OUT / 4);
            launch_chained(gemv_umma_combine_kernel, dim3((unsigned)((quads + 255) / 256)), dim3(256), 0, st,
                           static_cast<const float*>(partial), static_cast<const int*>(status),
                           static_cast<__nv_bfloat16*>(Y), Yf, sch, (int)m0, rows, (int)OUT);
            count_launch();
            if (int rc = check_launch("gemv_umma_combine")) return rc;
        }
    }
    return MSAQ_OK;
}

// Glue fused in front of the GEMV (see XprepMode); mode XP_PLAIN when absent.
struct Prologue {
    int mode;
    const void* r;       // XP_ADD_NORM: addend [M][K]
    int r_is_f32;
    void* h_out;         // XP_ADD_NORM: the sum, bf16 [M][K]
    float eps;
};

int launch_xprep(const XprepArgs& xa, int mode, unsigned grid, cudaStream_t st) {
    switch (mode) {
        case XP_RMSNORM: launch_chained(gemv_xprep_kernel<XP_RMSNORM>, dim3(grid), dim3(128), 0, st, xa); break;
        case XP_SILU_MUL: launch_chained(gemv_xprep_kernel<XP_SILU_MUL>, dim3(grid), dim3(128), 0, st, xa); break;
        case XP_ADD_NORM: launch_chained(gemv_xprep_kernel<XP_ADD_NORM>, dim3(grid), dim3(128), 0, st, xa); break;
        default: launch_chained(gemv_xprep_kernel<XP_PLAIN>, dim3(grid), dim3(128), 0, st, xa); break;
    }
    count_launch();
    return check_launch("gemv_xprep");
}

int run_mma(const __nv_bfloat16* X, const Prologue& pro, const int8_t* se, const uint8_t* up, const uint8_t* sh,
            void* Y, float* Yf, int64_t M, int64_t OUT, int64_t NB, void* ws, cudaStream_t st, int fmt = GF_MSAQ_U4,
            const PeerPush* push = nullptr, const void* res = nullptr) {
    const MmaPlan p = plan_mma(M, OUT, NB, fmt);
    uint8_t* base = static_cast<uint8_t*>(ws);
    int* status = reinterpret_cast<int*>(base);
    unsigned long long* counters = reinterpret_cast<unsigned long long*>(base + 256);
    uint8_t* xprep = base + p.xprep_off;
    float* partial = reinterpret_cast<float*>(base + p.partial_off);
    const int64_t tile_rows = GM_MP * GM_MAX_PASSES, K = NB * BLOCK;
    const int64_t ldx = pro.mode == XP_SILU_MUL ? 2 * K : K;
    for (int64_t m0 = 0; m0 < M; m0 += tile_rows) {        // more than 16 rows: one launch per 16-row tile
        const int rows = (int)(M - m0 < tile_rows ? M - m0 : tile_rows);
        const int passes = (rows + GM_MP - 1) / GM_MP;
        const int warps = (int)NB * passes * GM_MP;
        XprepArgs xa{};
        xa.X = X + m0 * ldx;
        xa.R = pro.r ? static_cast<const uint8_t*>(pro.r) + m0 * K * (pro.r_is_f32 ? 4 : 2) : nullptr;
        xa.h_out = pro.h_out ? static_cast<__nv_bfloat16*>(pro.h_out) + m0 * K : nullptr;
        xa.xprep = xprep;
        xa.M = rows;
        xa.NB = (int)NB;
        xa.passes = passes;
        xa.ldx = (int)ldx;
        xa.r_is_f32 = pro.r_is_f32;
        xa.eps = pro.eps;
        xa.natural = fmt == GF_MXINT8 ? 1 : 0;
        // Up to four rows, no prologue, and no CTA streams more than eighteen K blocks (the small problems, where fixed
        // costs are most of the time): the main kernel stages the activations itself -- each of its nine warps writes
        // one or two records into a table in shared memory while the first copies are in flight -- and no launch runs in
        // front (4096x4096, one row: 11.8 -> 10.3 us).  With a prologue in front, or more blocks per CTA, the
        // separate staging kernel is the faster arrangement: it runs under the tail of the kernel before it, while
        // staging inside delays the consumers' start (measured on the 70B layer's GEMVs, one and eight GPUs).
        GemvSchedule sch = p.sch;
        const long long max_iter = (sch.units() + sch.grid - 1) / sch.grid;
        const long long table = max_iter * p.kb * GM_XREC;
        const bool in_kernel = fmt == GF_MSAQ_U4 && passes == 1 && pro.mode == XP_PLAIN && option_inkernel_staging() &&
                               table <= GM_MAX_TABLE;
        const uint32_t tag = next_call_tag();
        if (in_kernel) {
            const int per_sm = (sch.grid + sm_count() - 1) / sm_count();
            int stages = (200 * 1024 / per_sm - (int)table) / (p.kb * gm_stage_bytes(sch.tc, passes, fmt));
            sch.stages = stages > GM_MAX_STAGES ? GM_MAX_STAGES : stages < 2 ? 2 : stages;
        } else if (int rc = launch_xprep(xa, pro.mode, (unsigned)((warps * 32 + 127) / 128), st)) {
            return rc;
        }
        GemvMmaArgs a{se, up, sh, xprep, partial, counters, status, sticky_status(), static_cast<__nv_bfloat16*>(Y), Yf,
                      (int)m0, rows, (int)OUT, (int)NB, sch, option_wait_polls(), option_test_skip_stage(),
                      in_kernel ? pro.mode : -1, xa.X, xa.R, xa.h_out, (int)ldx, pro.r_is_f32, pro.eps, tag,
                      in_kernel ? (int)table : 0, 0, option_early_weights() ? 1 : 0, push ? *push : PeerPush{},
                      static_cast<const __nv_bfloat16*>(res)};
        // the ring depth was planned for the first tile's pass count; a last, smaller tile may go deeper but need not
        int rc;
        if (fmt == GF_MXINT8) {
            switch (passes) {
                case 1: rc = launch_mma_mx<1>(a, st); break;
                case 2: rc = launch_mma_mx<2>(a, st); break;
                case 3: rc = launch_mma_mx<3>(a, st); break;
                default: rc = launch_mma_mx<4>(a, st); break;
            }
            if (rc) return rc;
            continue;
        }
        switch (passes) {
            case 1: rc = launch_mma_tc<1>(a, p.kb, st); break;
            case 2: rc = launch_mma_tc<2>(a, p.kb, st); break;
            case 3: rc = launch_mma_tc<3>(a, p.kb, st); break;
            default: rc = launch_mma_tc<4>(a, p.kb, st); break;
        }
        if (rc) return rc;
    }
    return MSAQ_OK;
}

bool mma_usable(const int8_t* se, const uint8_t* up, const uint8_t* sh, const void* ws, int64_t OUT, int u, int gs,
                bool cm) {
    return mma_eligible(OUT, u, gs, cm) &&
           !((reinterpret_cast<uintptr_t>(up) | reinterpret_cast<uintptr_t>(sh) | reinterpret_cast<uintptr_t>(se) |
              reinterpret_cast<uintptr_t>(ws)) & 15);
}

int gemv_dispatch(const void* X, const int8_t* se, const uint8_t* up, const uint8_t* sh, void* Y, float* Yf,
                  int64_t M, int64_t OUT, int64_t NB, int u, int gs, bool cm, void* ws, size_t ws_bytes,
                  void* stream) {
    Fmt f;
    if (!make_fmt(u, gs, &f)) return fail(MSAQ_ERR_UNSUPPORTED, "unsupported format u=%d gs=%d", u, gs);
    if (!X || !se || !up || !sh || !Y) return fail(MSAQ_ERR_ARG, "null pointer");
    if (M <= 0 || OUT <= 0 || NB <= 0) return fail(MSAQ_ERR_ARG, "M, OUT and NB must be positive");
    if (M > INT32_MAX || OUT > INT32_MAX || NB * BLOCK > INT32_MAX) return fail(MSAQ_ERR_ARG, "size exceeds 2^31");
    if (cm && (reinterpret_cast<uintptr_t>(up) & 3)) return fail(MSAQ_ERR_ARG, "upper_cm must be 4-byte aligned");
    if (int rc = require_sm100()) return rc;
    const size_t need = msaq_wonly_gemv_workspace(M, OUT, NB, u, gs);
    if (!ws || ws_bytes < need)
        return fail(MSAQ_ERR_WORKSPACE, "workspace of %zu bytes needed, %zu given", need, ws ? ws_bytes : (size_t)0);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const __nv_bfloat16* x = static_cast<const __nv_bfloat16*>(X);

    const bool aligned = !((reinterpret_cast<uintptr_t>(up) | reinterpret_cast<uintptr_t>(sh) |
                            reinterpret_cast<uintptr_t>(se) | reinterpret_cast<uintptr_t>(ws)) & 15);
    // the tensor-memory epilogue stores 16 outputs at a time: Y (and Y_f32) must be 16-byte aligned for it
    const bool tm_ok = aligned && umma_eligible(OUT, u, gs, cm) && option_tensor_memory() &&
                       !((reinterpret_cast<uintptr_t>(Y) | reinterpret_cast<uintptr_t>(Yf)) & 15);
    // u = 4 keeps up to eight rows on the integer-MMA kernel; the 5+3 and 6+2 bit formats have no such kernel
    if (tm_ok && (u != 4 || M >= GU_MIN_M)) return run_umma(x, se, up, sh, Y, Yf, M, OUT, NB, u, ws, st);
    // the integer-MMA kernel's finishing warps store four outputs at a time: 8-byte aligned bf16, 16-byte aligned fp32
    const bool out_ok = !((reinterpret_cast<uintptr_t>(Y) & 7) | (reinterpret_cast<uintptr_t>(Yf) & 15));
    if (mma_usable(se, up, sh, ws, OUT, u, gs, cm) && out_ok)
        return run_mma(x, Prologue{XP_PLAIN, nullptr, 0, nullptr, 0.0f}, se, up, sh, Y, Yf, M, OUT, NB, ws, st);

    return gemv_run_generic(x, se, up, sh, Y, Yf, M, OUT, NB, f, cm, static_cast<uint8_t*>(ws) + WS_CTL_BYTES, st);
}

}  // namespace
}  // namespace msaq

using namespace msaq;

extern "C" size_t msaq_wonly_gemv_workspace(int64_t M, int64_t OUT, int64_t NB, int u, int gs) {
    if (M <= 0 || OUT <= 0 || NB <= 0) return 0;
    size_t bytes = gemv_generic_workspace(M, OUT, NB) + WS_CTL_BYTES;
    if (mma_eligible(OUT, u, gs, true)) {
        const size_t tuned = plan_mma(M, OUT, NB).total;
        if (tuned > bytes) bytes = tuned;
    }
    if (umma_eligible(OUT, u, gs, true) && (u != 4 || M >= GU_MIN_M)) {
        const size_t tm = plan_umma(M, OUT, NB, u).total + WS_CTL_BYTES;
        if (tm > bytes) bytes = tm;
    }
    return bytes;
}

extern "C" int msaq_wonly_gemv(const void* x, const int8_t* scale_exp, const uint8_t* upper, const uint8_t* shared,
                               void* y, float* y_f32, int64_t OUT, int64_t NB, int u, int gs, void* workspace,
                               size_t workspace_bytes, void* stream) {
    return gemv_dispatch(x, scale_exp, upper, shared, y, y_f32, 1, OUT, NB, u, gs, false, workspace, workspace_bytes,
                         stream);
}

extern "C" int msaq_wonly_gemv_wide(const void* x, const int8_t* scale_exp, const uint8_t* upper_cm,
                                    const uint8_t* shared_cm, void* y, float* y_f32, int64_t OUT, int64_t NB, int u,
                                    int gs, void* workspace, size_t workspace_bytes, void* stream) {
    return gemv_dispatch(x, scale_exp, upper_cm, shared_cm, y, y_f32, 1, OUT, NB, u, gs, true, workspace,
                         workspace_bytes, stream);
}

extern "C" int msaq_wonly_gemv_batched(const void* X, const int8_t* scale_exp, const uint8_t* upper_cm,
                                       const uint8_t* shared_cm, void* Y, float* Y_f32, int64_t M, int64_t OUT,
                                       int64_t NB, int u, int gs, void* workspace, size_t workspace_bytes,
                                       void* stream) {
    return gemv_dispatch(X, scale_exp, upper_cm, shared_cm, Y, Y_f32, M, OUT, NB, u, gs, true, workspace,
                         workspace_bytes, stream);
}

// ---- GEMV with the layer glue in front of it fused into the activation staging ---------------
extern "C" size_t msaq_wonly_gemv_fused_workspace(int64_t M, int64_t OUT, int64_t NB, int u, int gs) {
    const size_t g = msaq_wonly_gemv_workspace(M, OUT, NB, u, gs);
    if (g == 0) return 0;
    return ((g + 255) & ~(size_t)255) + (((size_t)M * NB * BLOCK * 2 + 255) & ~(size_t)255);
}

extern "C" int msaq_wonly_gemv_fused(const void* x, int prologue, const void* addend, int addend_is_f32, float eps,
                                     void* h_out, const int8_t* scale_exp, const uint8_t* upper_cm,
                                     const uint8_t* shared_cm, void* y, float* y_f32, int64_t M, int64_t OUT,
                                     int64_t NB, int u, int gs, void* workspace, size_t workspace_bytes,
                                     void* stream) {
    if (prologue < MSAQ_PRO_NONE || prologue > MSAQ_PRO_ADD_RMSNORM)
        return fail(MSAQ_ERR_ARG, "unknown prologue %d", prologue);
    if (prologue == MSAQ_PRO_NONE)
        return gemv_dispatch(x, scale_exp, upper_cm, shared_cm, y, y_f32, M, OUT, NB, u, gs, true, workspace,
                             workspace_bytes, stream);
    Fmt f;
    if (!make_fmt(u, gs, &f)) return fail(MSAQ_ERR_UNSUPPORTED, "unsupported format u=%d gs=%d", u, gs);
    if (!x || !scale_exp || !upper_cm || !shared_cm || !y) return fail(MSAQ_ERR_ARG, "null pointer");
    if (prologue == MSAQ_PRO_ADD_RMSNORM && (!addend || !h_out))
        return fail(MSAQ_ERR_ARG, "the add+rmsnorm prologue needs an addend and h_out");
    if (M <= 0 || OUT <= 0 || NB <= 0) return fail(MSAQ_ERR_ARG, "M, OUT and NB must be positive");
    if (prologue == MSAQ_PRO_ADD_RMSNORM) {
        // Every thread block re-reads whole rows of x and addend for the row norm while others write h_out:
        // an in-place update would let some of them see the sum already applied.
        const uintptr_t h0 = reinterpret_cast<uintptr_t>(h_out), h1 = h0 + (size_t)M * NB * BLOCK * 2;
        const uintptr_t x0 = reinterpret_cast<uintptr_t>(x), x1 = x0 + (size_t)M * NB * BLOCK * 2;
        const uintptr_t a0 = reinterpret_cast<uintptr_t>(addend), a1 = a0 + (size_t)M * NB * BLOCK * (addend_is_f32 ? 4 : 2);
        if ((h0 < x1 && x0 < h1) || (h0 < a1 && a0 < h1))
            return fail(MSAQ_ERR_ARG, "h_out must not overlap x or addend (no in-place residual update)");
    }
    if (M > INT32_MAX || OUT > INT32_MAX || NB * BLOCK > INT32_MAX / 2) return fail(MSAQ_ERR_ARG, "size exceeds 2^31");
    if (int rc = require_sm100()) return rc;
    const size_t need = msaq_wonly_gemv_fused_workspace(M, OUT, NB, u, gs);
    if (!workspace || workspace_bytes < need)
        return fail(MSAQ_ERR_WORKSPACE, "workspace of %zu bytes needed, %zu given", need,
                    workspace ? workspace_bytes : (size_t)0);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const int64_t K = NB * BLOCK;
    const bool vec_ok = !((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(addend)) & 15) &&
                        !((reinterpret_cast<uintptr_t>(y) & 7) | (reinterpret_cast<uintptr_t>(y_f32) & 15));
    // fused staging belongs to the integer-MMA kernel; batches the tensor-memory kernel takes run the glue separately
    const bool small = M < GU_MIN_M || !option_tensor_memory();
    if (mma_usable(scale_exp, upper_cm, shared_cm, workspace, OUT, u, gs, true) && vec_ok && small) {
        const Prologue pro{prologue, addend, addend_is_f32, h_out, eps};
        return run_mma(static_cast<const __nv_bfloat16*>(x), pro, scale_exp, upper_cm, shared_cm, y, y_f32, M, OUT, NB,
                       workspace, st);
    }
    // Other formats: the glue runs as kernels of its own into the tail of the workspace.
    const size_t g = (msaq_wonly_gemv_workspace(M, OUT, NB, u, gs) + 255) & ~(size_t)255;
    void* tmp = static_cast<uint8_t*>(workspace) + g;
    int rc = MSAQ_OK;
    if (prologue == MSAQ_PRO_RMSNORM) rc = msaq_rmsnorm(x, tmp, M, K, eps, stream);
    else if (prologue == MSAQ_PRO_SILU_MUL) rc = msaq_silu_mul(x, tmp, M, K, stream);
    else {
        rc = msaq_add_residual(x, addend, addend_is_f32, h_out, M * K, stream);
        if (!rc) rc = msaq_rmsnorm(h_out, tmp, M, K, eps, stream);
    }
    if (rc) return rc;
    return gemv_dispatch(tmp, scale_exp, upper_cm, shared_cm, y, y_f32, M, OUT, NB, u, gs, true, workspace, g, stream);
}

// ---- fused GEMV with the residual add behind it ------------------------------------------------
extern "C" int msaq_wonly_gemv_fused_add(const void* x, int prologue, float eps, const int8_t* scale_exp,
                                         const uint8_t* upper_cm, const uint8_t* shared_cm, const void* residual, void* y,
                                         int64_t M, int64_t OUT, int64_t NB, int u, int gs, void* workspace,
                                         size_t workspace_bytes, void* stream) {
    if (prologue != MSAQ_PRO_NONE && prologue != MSAQ_PRO_RMSNORM && prologue != MSAQ_PRO_SILU_MUL)
        return fail(MSAQ_ERR_ARG, "prologue %d: none, rmsnorm or SiLU*mul", prologue);
    if (!x || !scale_exp || !upper_cm || !shared_cm || !residual || !y) return fail(MSAQ_ERR_ARG, "null pointer");
    if (M <= 0 || OUT <= 0 || NB <= 0) return fail(MSAQ_ERR_ARG, "M, OUT and NB must be positive");
    if (M > INT32_MAX || OUT > INT32_MAX || NB * BLOCK > INT32_MAX / 2) return fail(MSAQ_ERR_ARG, "size exceeds 2^31");
    if (int rc = require_sm100()) return rc;
    const size_t need = msaq_wonly_gemv_fused_workspace(M, OUT, NB, u, gs);
    if (!workspace || workspace_bytes < need)
        return fail(MSAQ_ERR_WORKSPACE, "workspace of %zu bytes needed, %zu given", need, workspace ? workspace_bytes : (size_t)0);
    const bool ok = !((reinterpret_cast<uintptr_t>(x) & 15) | (reinterpret_cast<uintptr_t>(y) & 7) |
                      (reinterpret_cast<uintptr_t>(residual) & 7)) && M < GU_MIN_M &&
                    mma_usable(scale_exp, upper_cm, shared_cm, workspace, OUT, u, gs, true);
    if (ok) {
        const Prologue pro{prologue, nullptr, 0, nullptr, eps};
        return run_mma(static_cast<const __nv_bfloat16*>(x), pro, scale_exp, upper_cm, shared_cm, y, nullptr, M, OUT, NB,
                       workspace, static_cast<cudaStream_t>(stream), GF_MSAQ_U4, nullptr, residual);
    }
    // every other format and size: the same two steps as separate kernels (identical roundings)
    if (int rc = msaq_wonly_gemv_fused(x, prologue, nullptr, 0, eps, nullptr, scale_exp, upper_cm, shared_cm, y, nullptr, M, OUT,
                                       NB, u, gs, workspace, workspace_bytes, stream))
        return rc;
    return msaq_add_residual(residual, y, 0, y, M * OUT, stream);
}

// ---- GEMV of a row-parallel projection with the exchange's push inside --------------------
extern "C" int msaq_wonly_gemv_fused_push(const void* x, int prologue, const void* addend, int addend_is_f32, float eps,
                                          void* h_out, const int8_t* scale_exp, const uint8_t* upper_cm,
                                          const uint8_t* shared_cm, int64_t M, int64_t OUT, int64_t NB, int u, int gs,
                                          void* const* peer_bufs, int rank, int world, int parity, void* workspace,
                                          size_t workspace_bytes, void* stream) {
    if (prologue < MSAQ_PRO_NONE || prologue > MSAQ_PRO_ADD_RMSNORM) return fail(MSAQ_ERR_ARG, "unknown prologue %d", prologue);
    if (!x || !scale_exp || !upper_cm || !shared_cm || !peer_bufs) return fail(MSAQ_ERR_ARG, "null pointer");
    if (prologue == MSAQ_PRO_ADD_RMSNORM && (!addend || !h_out))
        return fail(MSAQ_ERR_ARG, "the add+rmsnorm prologue needs an addend and h_out");
    if (M <= 0 || OUT <= 0 || NB <= 0) return fail(MSAQ_ERR_ARG, "M, OUT and NB must be positive");
    if (world < 2 || world > 8 || rank < 0 || rank >= world) return fail(MSAQ_ERR_ARG, "world must be 2..8 and rank inside it");
    if (parity != 0 && parity != 1) return fail(MSAQ_ERR_ARG, "parity must be 0 or 1");
    if (M > INT32_MAX || OUT > INT32_MAX || NB * BLOCK > INT32_MAX / 2) return fail(MSAQ_ERR_ARG, "size exceeds 2^31");
    if (int rc = require_sm100()) return rc;
    const bool vec_ok = !((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(addend)) & 15);
    if (M >= GU_MIN_M || (M * OUT) % 4 || !vec_ok || !workspace ||
        !mma_usable(scale_exp, upper_cm, shared_cm, workspace, OUT, u, gs, true))
        return fail(MSAQ_ERR_UNSUPPORTED, "the push is built into the integer-MMA GEMV only (u=4, gs=2, up to 8 rows, aligned "
                                          "column-major planes): run the GEMV and msaq_peer_exchange separately");
    const size_t need = msaq_wonly_gemv_fused_workspace(M, OUT, NB, u, gs);
    if (workspace_bytes < need) return fail(MSAQ_ERR_WORKSPACE, "workspace of %zu bytes needed, %zu given", need, workspace_bytes);
    PeerPush push{};
    for (int r = 0; r < world; ++r) {
        if (!peer_bufs[r] || (reinterpret_cast<uintptr_t>(peer_bufs[r]) & 15)) return fail(MSAQ_ERR_ARG, "bad peer buffer %d", r);
        push.buf[r] = static_cast<float*>(peer_bufs[r]);
    }
    push.n = M * OUT;
    push.world = world;
    push.rank = rank;
    push.parity = parity;
    const Prologue pro{prologue, addend, addend_is_f32, h_out, eps};
    return run_mma(static_cast<const __nv_bfloat16*>(x), pro, scale_exp, upper_cm, shared_cm, nullptr, nullptr, M, OUT, NB,
                   workspace, static_cast<cudaStream_t>(stream), GF_MSAQ_U4, &push);
}

// ---- GEMV without any allocation ---------------------------------------------------------
// Scratch for msaq_wonly_gemv_wide_static lives in the library image: one array per GPU that
// loads the library, held until the process exits.
namespace {
static __device__ __align__(256) unsigned char g_static_scratch[MSAQ_STATIC_SCRATCH_BYTES];
std::mutex g_static_mutex;
void* g_static_ptr[64] = {};

// Device address of the array on the current device.  The array's name is only a host-side
// handle; the address a kernel can use comes from cudaGetSymbolAddress, asked once per device
// while that device is current.
int static_scratch(void** out) {
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64)
        return msaq::fail(MSAQ_ERR_CUDA, "no usable current device for the static scratch");
    std::lock_guard<std::mutex> lock(g_static_mutex);
    if (!g_static_ptr[dev]) {
        void* p = nullptr;
        const cudaError_t e = cudaGetSymbolAddress(&p, g_static_scratch);
        if (e != cudaSuccess || !p)
            return msaq::fail(MSAQ_ERR_CUDA, "cudaGetSymbolAddress(static scratch): %s", cudaGetErrorString(e));
        g_static_ptr[dev] = p;
    }
    *out = g_static_ptr[dev];
    return MSAQ_OK;
}
}  // namespace

extern "C" size_t msaq_static_scratch_bytes(void) { return MSAQ_STATIC_SCRATCH_BYTES; }

extern "C" int msaq_wonly_gemv_wide_static(const void* x, const int8_t* scale_exp, const uint8_t* upper_cm,
                                           const uint8_t* shared_cm, void* y, float* y_f32, int64_t OUT, int64_t NB,
                                           int u, int gs, void* stream) {
    const size_t need = msaq_wonly_gemv_workspace(1, OUT, NB, u, gs);
    if (need == 0) return msaq::fail(MSAQ_ERR_ARG, "OUT and NB must be positive");
    if (need > MSAQ_STATIC_SCRATCH_BYTES)
        return msaq::fail(MSAQ_ERR_WORKSPACE,
                          "this GEMV needs %zu bytes of scratch, the built-in scratch holds %zu: use "
                          "msaq_wonly_gemv_wide with a caller-owned workspace", need, (size_t)MSAQ_STATIC_SCRATCH_BYTES);
    void* scratch = nullptr;
    if (int rc = static_scratch(&scratch)) return rc;
    return msaq_wonly_gemv_wide(x, scale_exp, upper_cm, shared_cm, y, y_f32, OUT, NB, u, gs, scratch,
                                MSAQ_STATIC_SCRATCH_BYTES, stream);
}

// ---- plain MXINT8 GEMV (the reference's matched baseline, csrc/mxint8.cu:196-253) ----------------------
extern "C" size_t msaq_mxint8_gemv_workspace(int64_t M, int64_t OUT, int64_t NB) {
    if (M <= 0 || OUT <= 0 || NB <= 0) return 0;
    return plan_mma(M, OUT, NB, GF_MXINT8).total;
}

extern "C" int msaq_mxint8_gemv_batched_wide(const void* X, const int8_t* scale_exp, const int8_t* qweight_cm, void* Y,
                                             float* Y_f32, int64_t M, int64_t OUT, int64_t NB, void* workspace,
                                             size_t workspace_bytes, void* stream) {
    if (!X || !scale_exp || !qweight_cm || !Y) return fail(MSAQ_ERR_ARG, "null pointer");
    if (M <= 0 || OUT <= 0 || NB <= 0) return fail(MSAQ_ERR_ARG, "M, OUT and NB must be positive");
    if (M > INT32_MAX || OUT > INT32_MAX || NB * BLOCK > INT32_MAX) return fail(MSAQ_ERR_ARG, "size exceeds 2^31");
    if (OUT % 16) return fail(MSAQ_ERR_UNSUPPORTED, "the MXINT8 GEMV needs OUT to be a multiple of 16");
    if ((reinterpret_cast<uintptr_t>(scale_exp) | reinterpret_cast<uintptr_t>(qweight_cm) | reinterpret_cast<uintptr_t>(workspace) |
         reinterpret_cast<uintptr_t>(Y_f32)) & 15)
        return fail(MSAQ_ERR_ARG, "planes, workspace and Y_f32 must be 16-byte aligned");
    if (reinterpret_cast<uintptr_t>(Y) & 7) return fail(MSAQ_ERR_ARG, "Y must be 8-byte aligned");
    if (int rc = require_sm100()) return rc;
    const size_t need = msaq_mxint8_gemv_workspace(M, OUT, NB);
    if (!workspace || workspace_bytes < need)
        return fail(MSAQ_ERR_WORKSPACE, "workspace of %zu bytes needed, %zu given", need, workspace ? workspace_bytes : (size_t)0);
    return run_mma(static_cast<const __nv_bfloat16*>(X), Prologue{XP_PLAIN, nullptr, 0, nullptr, 0.0f}, scale_exp,
                   reinterpret_cast<const uint8_t*>(qweight_cm), nullptr, Y, Y_f32, M, OUT, NB, workspace,
                   static_cast<cudaStream_t>(stream), GF_MXINT8);
}

extern "C" int msaq_mxint8_gemv_wide(const void* x, const int8_t* scale_exp, const int8_t* qweight_cm, void* y, float* y_f32,
                                     int64_t OUT, int64_t NB, void* workspace, size_t workspace_bytes, void* stream) {
    return msaq_mxint8_gemv_batched_wide(x, scale_exp, qweight_cm, y, y_f32, 1, OUT, NB, workspace, workspace_bytes, stream);
}

#ifdef MSAQ_TRACE
// diagnostic build only: the per-thread-block time stamps of the last staging and main kernel launches
extern "C" int msaq_debug_trace(unsigned long long* host_out) {
    return cudaMemcpyFromSymbol(host_out, msaq::g_trace, sizeof(msaq::g_trace)) == cudaSuccess ? 0 : 1;
}
#endif
