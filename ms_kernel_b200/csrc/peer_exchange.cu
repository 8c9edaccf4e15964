// The exchange step of the tensor-parallel decode layer: sum of one small fp32 vector per rank
// ([B, hidden], 32 KB at B = 1) over NVLink peer memory, optionally with the residual add behind it.
// The reference has no multi-GPU code; this replaces a library all-reduce (NCCL: 16.5 us at two ranks for this
// message; a copy + barrier + reduce + barrier one-shot kernel: 14 us at two ranks, about 30 us at eight) with a
// push: every rank stores its partial sums straight into its slot of every peer's buffer (plain peer stores, no
// multicast, no TMA), counts itself on the peer's flag with a release at system scope, waits once for the other
// ranks' counts on its own flag, and adds the slots up in rank order (so every rank gets the same bits).
//
// Buffers: each rank owns `2 x world x n` floats (two parities x one slot per source rank) and, behind them, two
// flag words and two done-counters, all zero before the first call.  Successive exchanges alternate parity; a rank
// can run at most one exchange ahead of a peer (it needs the peer's push to get past its own wait), so two parities
// are enough, and the last thread block to leave an exchange puts that parity's flag back to zero for its next use.
// Every wait is bounded: a rank whose peers never arrive gives up, reports through the status word and writes NaN.
#include "msaq_common.cuh"
#include "sm100_ptx.cuh"

namespace msaq {
namespace {

constexpr int PX_MAX_WORLD = 8;
constexpr int PX_THREADS = 256;

struct PeerArgs {
    float* buf[PX_MAX_WORLD];        // buf[r]: rank r's exchange memory as mapped into this process
    const float* partial;            // this rank's contribution, [n]
    const __nv_bfloat16* residual;   // optional: out = bf16(residual + sum)
    void* out;                       // fp32 [n], or bf16 [n] with a residual
    int* sticky;                     // the library's per-device status word
    int64_t n;
    int rank, world, parity;
    uint32_t max_polls;
};

__device__ __forceinline__ unsigned int* px_flag(float* base, int world, int64_t n, int parity) {
    return reinterpret_cast<unsigned int*>(base + 2 * (int64_t)world * n) + parity;
}

__global__ void __launch_bounds__(PX_THREADS)
peer_exchange_kernel(const PeerArgs a) {
    chain_wait();
    __shared__ int ok_sh;
    const int64_t i0 = ((int64_t)blockIdx.x * PX_THREADS + threadIdx.x) * 4;
    const bool live = i0 < a.n;                              // n is a multiple of 4
    float4 mine = make_float4(0.f, 0.f, 0.f, 0.f);
    if (live) {
        mine = *reinterpret_cast<const float4*>(a.partial + i0);
        // push: my slot in every peer's buffer of this parity
        for (int r = 0; r < a.world; ++r) {
            if (r == a.rank) continue;
            float* dst = a.buf[r] + ((int64_t)a.parity * a.world + a.rank) * a.n + i0;
            *reinterpret_cast<float4*>(dst) = mine;
        }
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence_system();
        for (int r = 0; r < a.world; ++r) {
            if (r == a.rank) continue;
            asm volatile("red.release.sys.global.add.u32 [%0], 1;" ::"l"(px_flag(a.buf[r], a.world, a.n, a.parity)) : "memory");
        }
        // wait for the other ranks' thread blocks (each counts itself once per peer)
        unsigned int* flag = px_flag(a.buf[a.rank], a.world, a.n, a.parity);
        const unsigned int want = (unsigned int)(a.world - 1) * gridDim.x;
        int ok = 0;
        // ranks start a step up to a host jitter apart, so this limit is generous: 4 x the poll option, with
        // 2 us naps once the first thousand polls have passed (seconds at the default, milliseconds in the tests)
        const uint64_t limit = 4ull * a.max_polls;
        for (uint64_t p = 0; p < limit; ++p) {
            unsigned int v;
            asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(flag) : "memory");
            if (v >= want) { ok = 1; break; }
            if (p > 64) __nanosleep(p < 1024 ? 100 : 2000);
        }
        if (!ok && a.sticky) atomicOr(a.sticky, PEER_EXCHANGE_TIMEOUT);
        ok_sh = ok;
    }
    __syncthreads();
    if (live) {
        float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
        if (ok_sh) {
            for (int r = 0; r < a.world; ++r) {              // rank order: the same sum on every rank
                float4 v = mine;
                if (r != a.rank) {
                    const float* src = a.buf[a.rank] + ((int64_t)a.parity * a.world + r) * a.n + i0;
                    v = __ldcv(reinterpret_cast<const float4*>(src));
                }
                s.x += v.x; s.y += v.y; s.z += v.z; s.w += v.w;
            }
        } else {
            s.x = s.y = s.z = s.w = __int_as_float(0x7FC00000);
        }
        if (a.residual) {
            const uint2 hb = *reinterpret_cast<const uint2*>(a.residual + i0);
            __nv_bfloat162 o0 = __floats2bfloat162_rn(bf16_lo(hb.x) + s.x, bf16_hi(hb.x) + s.y);
            __nv_bfloat162 o1 = __floats2bfloat162_rn(bf16_lo(hb.y) + s.z, bf16_hi(hb.y) + s.w);
            uint2 ob;
            ob.x = *reinterpret_cast<uint32_t*>(&o0);
            ob.y = *reinterpret_cast<uint32_t*>(&o1);
            *reinterpret_cast<uint2*>(static_cast<__nv_bfloat16*>(a.out) + i0) = ob;
        } else {
            *reinterpret_cast<float4*>(static_cast<float*>(a.out) + i0) = s;
        }
    }
    // the last thread block to get here re-arms this parity: flag and done-counter back to zero
    __syncthreads();
    if (threadIdx.x == 0) {
        unsigned int* done = px_flag(a.buf[a.rank], a.world, a.n, 2 + a.parity);
        if (atomicAdd(done, 1u) == gridDim.x - 1) {
            *px_flag(a.buf[a.rank], a.world, a.n, a.parity) = 0u;
            *done = 0u;
            __threadfence_system();
        }
    }
}

}  // namespace
}  // namespace msaq

using namespace msaq;

extern "C" size_t msaq_peer_exchange_bytes(int world, int64_t n) {
    if (world < 2 || world > PX_MAX_WORLD || n <= 0) return 0;
    return (size_t)2 * world * n * sizeof(float) + 256;
}

extern "C" int msaq_peer_exchange(const float* partial, const void* residual, void* out, void* const* peer_bufs, int rank,
                                  int world, int64_t n, int parity, void* stream) {
    if (!partial || !out || !peer_bufs) return fail(MSAQ_ERR_ARG, "null pointer");
    if (world < 2 || world > PX_MAX_WORLD || rank < 0 || rank >= world)
        return fail(MSAQ_ERR_ARG, "world must be 2..%d and rank inside it", PX_MAX_WORLD);
    if (n <= 0 || n % 4) return fail(MSAQ_ERR_ARG, "n must be a positive multiple of 4");
    if (parity != 0 && parity != 1) return fail(MSAQ_ERR_ARG, "parity must be 0 or 1");
    if ((reinterpret_cast<uintptr_t>(partial) | reinterpret_cast<uintptr_t>(out)) & 15)
        return fail(MSAQ_ERR_ARG, "partial and out must be 16-byte aligned");
    if (residual && (reinterpret_cast<uintptr_t>(residual) & 7)) return fail(MSAQ_ERR_ARG, "residual must be 8-byte aligned");
    PeerArgs a{};
    for (int r = 0; r < world; ++r) {
        if (!peer_bufs[r] || (reinterpret_cast<uintptr_t>(peer_bufs[r]) & 15)) return fail(MSAQ_ERR_ARG, "bad peer buffer %d", r);
        a.buf[r] = static_cast<float*>(peer_bufs[r]);
    }
    a.partial = partial;
    a.residual = static_cast<const __nv_bfloat16*>(residual);
    a.out = out;
    a.sticky = sticky_status();
    a.n = n;
    a.rank = rank;
    a.world = world;
    a.parity = parity;
    a.max_polls = option_wait_polls();
    if (int rc = require_sm100()) return rc;
    const unsigned grid = (unsigned)((n / 4 + PX_THREADS - 1) / PX_THREADS);
    launch_chained(peer_exchange_kernel, dim3(grid), dim3(PX_THREADS), 0, static_cast<cudaStream_t>(stream), a);
    count_launch();
    return check_launch("peer_exchange");
}
