// Host side of the weight-only GEMV entry points: argument checks, the split-K
// plan, kernel selection.  Replaces the launchers at csrc/w_gemv.cu:1410-1570
// of the reference.
#include "gemv_generic.cuh"

namespace msaq {
namespace {

struct GemvPlan {
    int mr;          // activation rows per CTA pass
    int mtiles;      // ceil(M / mr)
    int colblocks;   // ceil(OUT / GEMV_COLS)
    int splits;      // K ranges
    int blocks_per_split;
};

GemvPlan plan_generic(int64_t M, int64_t OUT, int64_t NB) {
    GemvPlan p;
    p.mr = M >= 8 ? 8 : (M >= 4 ? 4 : (M >= 2 ? 2 : 1));
    p.mtiles = (int)((M + p.mr - 1) / p.mr);
    p.colblocks = (int)((OUT + GEMV_COLS - 1) / GEMV_COLS);
    const int64_t ctas = (int64_t)p.colblocks * p.mtiles;
    int64_t want = (4LL * sm_count() + ctas - 1) / ctas;          // ~4 CTAs per SM in flight
    if (want > NB) want = NB;
    if (want > 32) want = 32;
    if (want < 1) want = 1;
    p.blocks_per_split = (int)((NB + want - 1) / want);
    p.splits = (int)((NB + p.blocks_per_split - 1) / p.blocks_per_split);
    return p;
}

template <int U, bool CM>
void launch_generic(const GemvPlan& p, const __nv_bfloat16* X, const int8_t* se, const uint8_t* up,
                    const uint8_t* sh, float* partial, int M, int OUT, int NB, const Fmt& f, cudaStream_t st) {
    dim3 grid(p.colblocks, p.splits, p.mtiles);
#define MSAQ_GO(MR) gemv_generic_kernel<U, CM, MR><<<grid, GEMV_COLS, 0, st>>>( \
        X, se, up, sh, partial, M, OUT, NB, f.lg_gs, f.UB, f.SB, p.blocks_per_split)
    switch (p.mr) {
        case 1: MSAQ_GO(1); break;
        case 2: MSAQ_GO(2); break;
        case 4: MSAQ_GO(4); break;
        default: MSAQ_GO(8); break;
    }
#undef MSAQ_GO
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
    float* partial = static_cast<float*>(ws);

    const GemvPlan p = plan_generic(M, OUT, NB);
    if (cm) {
        if (u == 4) launch_generic<4, true>(p, x, se, up, sh, partial, (int)M, (int)OUT, (int)NB, f, st);
        else if (u == 3) launch_generic<3, true>(p, x, se, up, sh, partial, (int)M, (int)OUT, (int)NB, f, st);
        else launch_generic<2, true>(p, x, se, up, sh, partial, (int)M, (int)OUT, (int)NB, f, st);
    } else {
        if (u == 4) launch_generic<4, false>(p, x, se, up, sh, partial, (int)M, (int)OUT, (int)NB, f, st);
        else if (u == 3) launch_generic<3, false>(p, x, se, up, sh, partial, (int)M, (int)OUT, (int)NB, f, st);
        else launch_generic<2, false>(p, x, se, up, sh, partial, (int)M, (int)OUT, (int)NB, f, st);
    }
    count_launch();
    if (int rc = check_launch("gemv_generic")) return rc;
    const int64_t n = M * OUT;
    splitk_combine_kernel<<<(unsigned)((n + 255) / 256), 256, 0, st>>>(partial, static_cast<__nv_bfloat16*>(Y), Yf, n,
                                                                       p.splits);
    count_launch();
    return check_launch("splitk_combine");
}

}  // namespace
}  // namespace msaq

using namespace msaq;

extern "C" size_t msaq_wonly_gemv_workspace(int64_t M, int64_t OUT, int64_t NB, int u, int gs) {
    (void)u; (void)gs;
    if (M <= 0 || OUT <= 0 || NB <= 0) return 0;
    const GemvPlan p = plan_generic(M, OUT, NB);
    size_t bytes = (size_t)p.splits * (size_t)M * (size_t)OUT * sizeof(float);
    return (bytes + 255) & ~(size_t)255;
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
