// Thin inline-PTX wrappers used by the tuned kernels: mbarriers, TMA bulk
// copies (cp.async.bulk), warp-level integer MMA.  sm_100a only.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

namespace msaq {

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return (uint32_t)__cvta_generic_to_shared(p);
}

// Programmatic dependent launch.  A kernel launched with the programmatic-serialisation
// attribute may start while the kernel before it in the stream is still draining.
// chain_wait() blocks until that kernel has completed and its writes are visible: nothing a
// predecessor wrote may be read, and nothing it may still read may be written, before it.
// chain_release() lets the NEXT kernel's CTAs be scheduled from now on instead of at this
// grid's exit; the short glue kernels call it first thing, so that the launch of a streaming
// kernel behind them overlaps them.  The streaming kernels themselves do not: measured on
// B200, dependents made resident during a long kernel's tail slowed the decoder layer step
// from 233 to 282 us.  Both are no-ops in a kernel launched the ordinary way.
__device__ __forceinline__ void chain_release() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void chain_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}

// Make freshly initialised barriers visible to the async (TMA) proxy.
__device__ __forceinline__ void mbar_init_fence() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}

__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}

// Bounded wait: gives up after a fixed number of polls and reports failure, so
// that a lost copy can never hang the GPU.  Returns true when the phase completed.
constexpr uint32_t MBAR_FAST_POLLS = 2048;
constexpr uint32_t MBAR_MAX_POLLS = 1u << 20;          // default limit; the host passes option_wait_polls()
__device__ __forceinline__ bool mbar_wait_bounded(uint32_t bar, uint32_t parity, uint32_t max_polls = MBAR_MAX_POLLS) {
    for (uint32_t i = 0; i < max_polls; ++i) {
        if (mbar_try_wait(bar, parity)) return true;
        if (i >= MBAR_FAST_POLLS) __nanosleep(128);
    }
    return false;
}

// A wait gave up: mark this call's status word (the finishing code turns the outputs into NaN) and
// OR `bit` into the library's sticky per-device word that msaq_wait_status() reports to the host.
constexpr int WAIT_FAIL_GEMV_MMA = 1, WAIT_FAIL_GEMV_UMMA = 2, WAIT_FAIL_KV_DECODE = 4, BAD_APPEND_POS = 8,
              PEER_EXCHANGE_TIMEOUT = 16;
__device__ __forceinline__ void report_wait_failure(int* status, int value, int* sticky, int bit) {
    atomicExch(status, value);
    if (sticky) atomicOr(sticky, bit);
}

// TMA bulk copy global -> shared of `bytes` (multiple of 16, both addresses
// 16-byte aligned); completion is signalled on `bar` as transferred bytes.
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst), "l"(src), "r"(bytes), "r"(bar)
                 : "memory");
}

// D(16x8,s32) = A(16x32,s8,row) * B(32x8,s8,col) + C.
__device__ __forceinline__ void mma_s8_16832(int (&d)[4], const uint32_t (&a)[4], const uint32_t (&b)[2],
                                             const int (&c)[4]) {
    asm volatile(
        "mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%11,%12,%13};"
        : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]), "r"(c[0]), "r"(c[1]), "r"(c[2]),
          "r"(c[3]));
}

// Same with a zero accumulator input.
__device__ __forceinline__ void mma_s8_16832_z(int (&d)[4], const uint32_t (&a)[4], const uint32_t (&b)[2]) {
    asm volatile(
        "mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
        : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]), "r"(0));
}

// Same with the accumulator input {0, c, 0, c}: a per-thread constant added to the odd result columns for free.
__device__ __forceinline__ void mma_s8_16832_c(int (&d)[4], const uint32_t (&a)[4], const uint32_t (&b)[2], int c) {
    asm volatile(
        "mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%11,%10,%11};"
        : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]), "r"(0), "r"(c));
}

// Shared-memory loads with a register base and a compile-time byte offset, so
// that one address register per plane serves a whole stage.
template <int OFF>
__device__ __forceinline__ uint2 lds64(uint32_t base) {
    uint2 v;
    asm volatile("ld.shared.v2.u32 {%0,%1}, [%2+%3];" : "=r"(v.x), "=r"(v.y) : "r"(base), "n"(OFF));
    return v;
}
template <int OFF>
__device__ __forceinline__ uint32_t lds32(uint32_t base) {
    uint32_t v;
    asm volatile("ld.shared.u32 %0, [%1+%2];" : "=r"(v) : "r"(base), "n"(OFF));
    return v;
}
template <int OFF>
__device__ __forceinline__ int lds_s8(uint32_t base) {
    int v;
    asm volatile("ld.shared.s8 %0, [%1+%2];" : "=r"(v) : "r"(base), "n"(OFF));
    return v;
}

// Explicit single-instruction logic ops: the compiler otherwise splits these
// three-input expressions.
__device__ __forceinline__ uint32_t and_or(uint32_t a, uint32_t mask, uint32_t c) {      // (a & mask) | c
    uint32_t r;
    asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(r) : "r"(a), "r"(mask), "r"(c));
    return r;
}
__device__ __forceinline__ uint32_t and_xor(uint32_t a, uint32_t mask, uint32_t c) {     // (a & mask) ^ c
    uint32_t r;
    asm("lop3.b32 %0, %1, %2, %3, 0x6A;" : "=r"(r) : "r"(a), "r"(mask), "r"(c));
    return r;
}
__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
    uint32_t r;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(sel));
    return r;
}

// Unsigned A (u8) x signed B (s8), zero accumulator input.
__device__ __forceinline__ void mma_u8s8_16832_z(int (&d)[4], const uint32_t (&a)[4], const uint32_t (&b)[2]) {
    asm volatile(
        "mma.sync.aligned.m16n8k32.row.col.s32.u8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
        : "=r"(d[0]), "=r"(d[1]), "=r"(d[2]), "=r"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]), "r"(0));
}

// Transposing 8-bit matrix loads: lane (g = lane/4, t = lane%4) receives, for each 16x16-byte
// matrix whose row addresses the lanes supply (lanes 0-15 matrix 0, lanes 16-31 matrix 1),
// the bytes of rows 4t..4t+3 in column g and in column g+8.
__device__ __forceinline__ void ldmatrix_t8_x2(uint32_t (&r)[4], uint32_t row_addr) {
    asm volatile("ldmatrix.sync.aligned.m16n16.x2.trans.shared.b8 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(row_addr));
}
__device__ __forceinline__ void ldmatrix_t8_x1(uint32_t (&r)[2], uint32_t row_addr) {
    asm volatile("ldmatrix.sync.aligned.m16n16.x1.trans.shared.b8 {%0,%1}, [%2];"
                 : "=r"(r[0]), "=r"(r[1]) : "r"(row_addr));
}

}  // namespace msaq
