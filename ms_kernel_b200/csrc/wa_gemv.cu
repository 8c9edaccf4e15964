// The steps on either side of the weight-only decode path in the reference's harness
// (tests/harness_batchsweep.py:77-111, 210-243): the W+A decode GEMV, whose activations are quantised at
// run time into the same MSAQ-signed format as the weights, and the one-off dequantisation of a packed
// weight to bf16 that the reference's prefill feeds to a dense GEMM.
//
// Behaviour replaced: quant_act_msaq_kernel (csrc/wa_gemm.cu:82-108), wa_gemv / wa_gemv_batched
// (csrc/w_gemv.cu:846-1098) and ms_dequant_bf16_kernel (csrc/w_gemv.cu:1242-1275) of the reference.
//
// W+A on this hardware is the weight-only kernel on other inputs: the quantised activation q * 2^e (|q| <=
// 127) is an exact bf16 value, and an exact bf16 value within 2^7 of its block maximum is exact in the
// 16-bit block fixed point the integer-MMA GEMV stages its activations in.  So Y = sum_blocks 2^(ea+ew) *
// intdot(qx, qw), the reference's W+A result, comes out of the same kernels fed the dequantised
// activations; only the activation quantiser is new.
#include "msaq_common.cuh"
#include "sm100_ptx.cuh"

namespace msaq {
namespace {

// One warp per (row, 32-block): the MSAQ-signed int8 word of each element, the block exponent, and (for the
// GEMV that follows) the word's value as bf16.
__global__ void __launch_bounds__(256)
quant_act_kernel(const __nv_bfloat16* __restrict__ X, int8_t* __restrict__ qX, int8_t* __restrict__ sa_exp,
                 __nv_bfloat16* __restrict__ Xdq, int64_t blocks, int64_t NB, Fmt f) {
    chain_release();
    chain_wait();
    const int64_t w = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    if (w >= blocks) return;
    const int64_t i = w * BLOCK + lane;                       // rows are contiguous: element (m, blk*32 + lane)
    int up, sh;
    const int e = quantize_lane(__bfloat162float(X[i]), lane, f, &up, &sh);
    const int word = up * (1 << f.u) + sh;
    if (qX) qX[i] = (int8_t)word;
    if (sa_exp && lane == 0) sa_exp[w] = (int8_t)e;
    if (Xdq) Xdq[i] = __float2bfloat16_rn((float)word * exp2_int(e));     // exact: at most 8 significant bits
}

// One thread per (output row o, block): the 32 dequantised weights as bf16 into Wbf[K][OUT] (consecutive
// threads write consecutive o).
__global__ void __launch_bounds__(256)
dequant_bf16_kernel(const int8_t* __restrict__ scale_exp, const uint8_t* __restrict__ upper_cm,
                    const uint8_t* __restrict__ shared_cm, __nv_bfloat16* __restrict__ Wbf, int64_t OUT, Fmt f) {
    chain_release();
    chain_wait();
    const int64_t o = (int64_t)blockIdx.x * 256 + threadIdx.x;
    const int64_t blk = blockIdx.y;
    if (o >= OUT) return;
    const int64_t base = blk * OUT + o;
    uint32_t uw[7], sw[3] = {0u, 0u, 0u};
    const uint32_t* src = reinterpret_cast<const uint32_t*>(upper_cm + base * f.UB);     // UB is a multiple of 4
#pragma unroll
    for (int i = 0; i < 6; ++i) uw[i] = (i * 4 < f.UB) ? src[i] : 0u;
    uw[6] = 0u;
    for (int i = 0; i < f.SB; ++i) sw[i >> 2] |= (uint32_t)shared_cm[base * f.SB + i] << ((i & 3) * 8);
    const float scale = exp2_int((int)scale_exp[base]);
#pragma unroll 4
    for (int k = 0; k < BLOCK; ++k) {
        const int q = code_from_words(uw, k, f.wbits) * (1 << f.u) + code_from_words(sw, k >> f.lg_gs, f.u);
        Wbf[(blk * BLOCK + k) * OUT + o] = __float2bfloat16_rn((float)q * scale);
    }
}

int launch_quant(const void* X, int8_t* qX, int8_t* sa, void* Xdq, int64_t M, int64_t K, int u, int gs, void* stream) {
    Fmt f;
    if (!make_fmt(u, gs, &f)) return fail(MSAQ_ERR_UNSUPPORTED, "unsupported format u=%d gs=%d", u, gs);
    if (!X) return fail(MSAQ_ERR_ARG, "X is null");
    if (M <= 0 || K <= 0 || K % BLOCK) return fail(MSAQ_ERR_ARG, "M must be positive and K a positive multiple of 32");
    const int64_t blocks = M * (K / BLOCK);
    launch_chained(quant_act_kernel, dim3((unsigned)((blocks + 7) / 8)), dim3(256), 0, static_cast<cudaStream_t>(stream),
                   static_cast<const __nv_bfloat16*>(X), qX, sa, static_cast<__nv_bfloat16*>(Xdq), blocks, K / BLOCK, f);
    count_launch();
    return check_launch("quant_act");
}

}  // namespace
}  // namespace msaq

using namespace msaq;

extern "C" int msaq_quant_act(const void* X, int8_t* qX, int8_t* sa_exp, int64_t M, int64_t K, int u, int gs, void* stream) {
    if (!qX || !sa_exp) return fail(MSAQ_ERR_ARG, "null pointer");
    return launch_quant(X, qX, sa_exp, nullptr, M, K, u, gs, stream);
}

extern "C" size_t msaq_wa_gemv_workspace(int64_t M, int64_t OUT, int64_t NB, int u, int gs) {
    const size_t g = msaq_wonly_gemv_workspace(M, OUT, NB, u, gs);
    if (g == 0) return 0;
    return ((g + 255) & ~(size_t)255) + (((size_t)M * NB * BLOCK * 2 + 255) & ~(size_t)255);
}

extern "C" int msaq_wa_gemv_batched(const void* X, const int8_t* scale_exp, const uint8_t* upper_cm,
                                    const uint8_t* shared_cm, void* Y, float* Y_f32, int64_t M, int64_t OUT, int64_t NB,
                                    int u, int gs, void* workspace, size_t workspace_bytes, void* stream) {
    if (M <= 0 || OUT <= 0 || NB <= 0) return fail(MSAQ_ERR_ARG, "M, OUT and NB must be positive");
    const size_t need = msaq_wa_gemv_workspace(M, OUT, NB, u, gs);
    if (!workspace || workspace_bytes < need)
        return fail(MSAQ_ERR_WORKSPACE, "workspace of %zu bytes needed, %zu given", need, workspace ? workspace_bytes : (size_t)0);
    const size_t g = (msaq_wonly_gemv_workspace(M, OUT, NB, u, gs) + 255) & ~(size_t)255;
    void* xdq = static_cast<uint8_t*>(workspace) + g;
    if (int rc = launch_quant(X, nullptr, nullptr, xdq, M, NB * BLOCK, u, gs, stream)) return rc;
    return msaq_wonly_gemv_batched(xdq, scale_exp, upper_cm, shared_cm, Y, Y_f32, M, OUT, NB, u, gs, workspace, g, stream);
}

extern "C" int msaq_wa_gemv(const void* x, const int8_t* scale_exp, const uint8_t* upper_cm, const uint8_t* shared_cm,
                            void* y, float* y_f32, int64_t OUT, int64_t NB, int u, int gs, void* workspace,
                            size_t workspace_bytes, void* stream) {
    return msaq_wa_gemv_batched(x, scale_exp, upper_cm, shared_cm, y, y_f32, 1, OUT, NB, u, gs, workspace, workspace_bytes,
                                stream);
}

extern "C" int msaq_dequant_bf16(const int8_t* scale_exp, const uint8_t* upper_cm, const uint8_t* shared_cm, void* Wbf,
                                 int64_t OUT, int64_t K, int u, int gs, void* stream) {
    Fmt f;
    if (!make_fmt(u, gs, &f)) return fail(MSAQ_ERR_UNSUPPORTED, "unsupported format u=%d gs=%d", u, gs);
    if (!scale_exp || !upper_cm || !shared_cm || !Wbf) return fail(MSAQ_ERR_ARG, "null pointer");
    if (OUT <= 0 || K <= 0 || K % BLOCK) return fail(MSAQ_ERR_ARG, "K must be a positive multiple of 32");
    if (K / BLOCK > 65535) return fail(MSAQ_ERR_ARG, "K exceeds the supported range");
    if (reinterpret_cast<uintptr_t>(upper_cm) & 3) return fail(MSAQ_ERR_ARG, "upper_cm must be 4-byte aligned");
    launch_chained(dequant_bf16_kernel, dim3((unsigned)((OUT + 255) / 256), (unsigned)(K / BLOCK)), dim3(256), 0,
                   static_cast<cudaStream_t>(stream), scale_exp, upper_cm, shared_cm, static_cast<__nv_bfloat16*>(Wbf), OUT, f);
    count_launch();
    return check_launch("dequant_bf16");
}
