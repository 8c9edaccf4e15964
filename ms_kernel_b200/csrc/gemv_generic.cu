// Generic weight-only GEMV path: split-K plan and launches of the kernels in
// gemv_generic.cuh (its own translation unit so that it compiles in parallel
// with the tuned kernels).
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
#define MSAQ_GO(MR) launch_chained(gemv_generic_kernel<U, CM, MR>, dim3(grid), dim3(GEMV_COLS), 0, st, \
        X, se, up, sh, partial, M, OUT, NB, f.lg_gs, f.UB, f.SB, p.blocks_per_split)
    switch (p.mr) {
        case 1: MSAQ_GO(1); break;
        case 2: MSAQ_GO(2); break;
        case 4: MSAQ_GO(4); break;
        default: MSAQ_GO(8); break;
    }
#undef MSAQ_GO
}

}  // namespace

size_t gemv_generic_workspace(int64_t M, int64_t OUT, int64_t NB) {
    const GemvPlan p = plan_generic(M, OUT, NB);
    const size_t bytes = (size_t)p.splits * (size_t)M * (size_t)OUT * sizeof(float);
    return (bytes + 255) & ~(size_t)255;
}

int gemv_run_generic(const __nv_bfloat16* x, const int8_t* se, const uint8_t* up, const uint8_t* sh, void* Y,
                     float* Yf, int64_t M, int64_t OUT, int64_t NB, const Fmt& f, bool cm, void* ws,
                     cudaStream_t st) {
    float* partial = static_cast<float*>(ws);
    const GemvPlan p = plan_generic(M, OUT, NB);
    const int u = f.u;
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
    launch_chained(splitk_combine_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, st, partial, static_cast<__nv_bfloat16*>(Y), Yf, n,
                                                                       p.splits);
    count_launch();
    return check_launch("splitk_combine");
}

}  // namespace msaq
