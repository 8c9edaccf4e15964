// The exchange step of the tensor-parallel decode layer: sum of one small fp32 vector per rank
// ([B, hidden], 32 KB at B = 1) over NVLink peer memory, optionally with the residual add behind it.
// The reference has no multi-GPU code; this replaces a library all-reduce.  For this message the cost is latency
// (measured at two ranks, back to back in a CUDA graph: NCCL 24 us, a copy + barrier + reduce + barrier one-shot
// kernel 13.7 us, a push with a fence and a counted flag 9.3 us), so the data carries its own flag: every rank
// stores its partial sums into its slot of every peer's buffer as 16-byte words {x0, seq, x1, seq} (plain peer
// stores, no multicast, no TMA; each 8-byte half is written whole and validates itself), and every thread polls its
// own words in its own memory until they carry this exchange's sequence number -- no fence, no flag, no barrier
// between thread blocks.  The slots are added up in rank order, so every rank gets the same bits.
//
// Buffers: each rank owns `2 x world` slots of 2 n floats (two parities x one slot per source rank) and, behind
// them, a sequence number and a done-counter per parity, all zero before the first call.  Successive exchanges
// alternate parity; a rank can run at most one exchange ahead of a peer (it needs the peer's push to finish its
// own), so a slot is never overwritten while its reader still wants the previous message.  The sequence number of
// a parity lives in device memory and is advanced by the last thread block to leave, which is what lets one
// captured launch be replayed.  Every wait is bounded: a rank whose peers never arrive gives up, reports through
// the status word and writes NaN.
#include "msaq_common.cuh"
#include "sm100_ptx.cuh"

namespace msaq {
namespace {

constexpr int PX_MAX_WORLD = 8;
constexpr int PX_THREADS = 256;

struct PeerArgs {
    float* buf[PX_MAX_WORLD];        // buf[r]: rank r's exchange memory as mapped into this process
    const float* partial;            // this rank's contribution, [n]; null: it was pushed already (by the GEMV that
                                     // produced it, msaq_wonly_gemv_fused_push), into this rank's own slot too
    const __nv_bfloat16* residual;   // optional: out = bf16(residual + sum)
    void* out;                       // fp32 [n], or bf16 [n] with a residual
    int* sticky;                     // the library's per-device status word
    int64_t n;
    int rank, world, parity;
    uint32_t max_polls;
};

// control words behind the slots: [0..1] sequence number per parity, [2..3] done-counter per parity
__device__ __forceinline__ unsigned int* px_ctl(float* base, int world, int64_t n) {
    return reinterpret_cast<unsigned int*>(base + 4 * (int64_t)world * n);
}
__device__ __forceinline__ void px_store(float* dst, float x0, float x1, uint32_t seq) {
    asm volatile("st.volatile.global.v4.u32 [%0], {%1, %2, %3, %2};" ::"l"(dst), "r"(__float_as_uint(x0)), "r"(seq),
                 "r"(__float_as_uint(x1)) : "memory");
}

__global__ void __launch_bounds__(PX_THREADS)
peer_exchange_kernel(const PeerArgs a) {
    chain_release();                                         // the next kernel may be scheduled; it waits for this one
    chain_wait();
    unsigned int* ctl = px_ctl(a.buf[a.rank], a.world, a.n);
    const uint32_t seq = *reinterpret_cast<volatile unsigned int*>(ctl + a.parity) + 1u;
    const int64_t i0 = ((int64_t)blockIdx.x * PX_THREADS + threadIdx.x) * 4;
    if (i0 < a.n) {                                          // n is a multiple of 4
        const bool pushed = a.partial == nullptr;
        const float4 mine = pushed ? make_float4(0.f, 0.f, 0.f, 0.f) : *reinterpret_cast<const float4*>(a.partial + i0);
        for (int r = 0; r < a.world && !pushed; ++r) {       // push: my slot in every peer's buffer of this parity
            if (r == a.rank) continue;
            float* dst = a.buf[r] + (((int64_t)a.parity * a.world + a.rank) * a.n + i0) * 2;
            px_store(dst, mine.x, mine.y, seq);
            px_store(dst + 4, mine.z, mine.w, seq);
        }
        // ranks start a step up to a host jitter apart, so the limit is generous: 4 x the poll option, with
        // 2 us naps once the first thousand polls have passed (seconds at the default, milliseconds in the tests).
        // All slots are polled together: the loads of a round go out back to back and only then are their sequence
        // numbers looked at, so a round costs one load latency whatever the number of ranks (polling rank after rank
        // made the wait grow by two dependent loads per rank: 11 us per exchange at eight ranks).
        const uint64_t limit = 4ull * a.max_polls;
        uint64_t polls = 0;
        bool ok = true;
        float x[PX_MAX_WORLD][4];
        uint32_t pending = 0;                                // bit 2r + k: half k of rank r's slot not seen yet
#pragma unroll
        for (int r = 0; r < PX_MAX_WORLD; ++r)
            if (r < a.world && (r != a.rank || pushed)) pending |= 3u << (2 * r);
        const float* base = a.buf[a.rank] + ((int64_t)a.parity * a.world * a.n + i0) * 2;
        while (pending) {
            uint32_t w[PX_MAX_WORLD][2][4];
#pragma unroll
            for (int r = 0; r < PX_MAX_WORLD; ++r) {
#pragma unroll
                for (int k = 0; k < 2; ++k) {
                    if (pending >> (2 * r + k) & 1u) {
                        const float* src = base + (int64_t)r * a.n * 2 + 4 * k;
                        asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];"
                                     : "=r"(w[r][k][0]), "=r"(w[r][k][1]), "=r"(w[r][k][2]), "=r"(w[r][k][3]) : "l"(src) : "memory");
                    }
                }
            }
#pragma unroll
            for (int r = 0; r < PX_MAX_WORLD; ++r) {
#pragma unroll
                for (int k = 0; k < 2; ++k) {
                    if ((pending >> (2 * r + k) & 1u) && w[r][k][1] == seq && w[r][k][3] == seq) {
                        x[r][2 * k] = __uint_as_float(w[r][k][0]);
                        x[r][2 * k + 1] = __uint_as_float(w[r][k][2]);
                        pending &= ~(1u << (2 * r + k));
                    }
                }
            }
            if (!pending) break;
            if (++polls >= limit) { ok = false; break; }
            if (polls > 64) __nanosleep(polls < 1024 ? 100 : 2000);
        }
        float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int r = 0; r < PX_MAX_WORLD; ++r) {             // rank order: the same sum on every rank
            if (r < a.world) {
                if (r == a.rank && !pushed) { s.x += mine.x; s.y += mine.y; s.z += mine.z; s.w += mine.w; }
                else { s.x += x[r][0]; s.y += x[r][1]; s.z += x[r][2]; s.w += x[r][3]; }
            }
        }
        if (!ok) {
            if (a.sticky) atomicOr(a.sticky, PEER_EXCHANGE_TIMEOUT);
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
    // the last thread block to get here advances this parity's sequence number (every block has read it by then)
    __syncthreads();
    if (threadIdx.x == 0) {
        if (atomicAdd(ctl + 2 + a.parity, 1u) == gridDim.x - 1) {
            ctl[2 + a.parity] = 0u;
            ctl[a.parity] = seq;
        }
    }
}

}  // namespace
}  // namespace msaq

using namespace msaq;

extern "C" size_t msaq_peer_exchange_bytes(int world, int64_t n) {
    if (world < 2 || world > PX_MAX_WORLD || n <= 0) return 0;
    return (size_t)4 * world * n * sizeof(float) + 256;
}

extern "C" int msaq_peer_exchange(const float* partial, const void* residual, void* out, void* const* peer_bufs, int rank,
                                  int world, int64_t n, int parity, void* stream) {
    if (!out || !peer_bufs) return fail(MSAQ_ERR_ARG, "null pointer");
    if (world < 2 || world > PX_MAX_WORLD || rank < 0 || rank >= world)
        return fail(MSAQ_ERR_ARG, "world must be 2..%d and rank inside it", PX_MAX_WORLD);
    if (n <= 0 || n % 4) return fail(MSAQ_ERR_ARG, "n must be a positive multiple of 4");
    if (parity != 0 && parity != 1) return fail(MSAQ_ERR_ARG, "parity must be 0 or 1");
    if ((reinterpret_cast<uintptr_t>(partial) & 15) || (reinterpret_cast<uintptr_t>(out) & (residual ? 7 : 15)))
        return fail(MSAQ_ERR_ARG, "partial and an fp32 out must be 16-byte aligned, a bf16 out 8-byte aligned");
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
