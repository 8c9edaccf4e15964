// Error plumbing, launch accounting and device queries shared by the entry points.
#include <atomic>
#include <chrono>
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <mutex>
#include <set>
#include <utility>

#include "msaq_common.cuh"

namespace msaq {

namespace {
thread_local char g_err[512] = "";
std::atomic<unsigned long long> g_launches{0};
}  // namespace

int fail(int code, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
    return code;
}

int check_launch(const char* what) {
    const cudaError_t e = cudaPeekAtLastError();
    if (e != cudaSuccess) {
        cudaGetLastError();   // clear the non-sticky launch-configuration error
        return fail(MSAQ_ERR_CUDA, "%s: %s", what, cudaGetErrorString(e));
    }
    return MSAQ_OK;
}

namespace {
std::atomic<int> g_opt_chained{-1};
std::atomic<int> g_opt_tmem{1};
std::atomic<int> g_opt_polls{1 << 20};
std::atomic<int> g_opt_inkernel{1};
std::atomic<int> g_opt_early{0};
std::atomic<uint32_t> g_call_tag{0};
std::atomic<int> g_opt_skip{-1};

// One status word per GPU that loads the library: kernels OR a bit into it when a bounded wait
// gives up or an append position is out of range; msaq_wait_status() reads and clears it.
__device__ int g_sticky_status;
std::atomic<int*> g_sticky_ptr[64];
}  // namespace

bool option_early_weights() { return g_opt_early.load(std::memory_order_relaxed) != 0; }
bool option_inkernel_staging() { return g_opt_inkernel.load(std::memory_order_relaxed) != 0; }

uint32_t next_call_tag() {
    uint32_t t = g_call_tag.load(std::memory_order_relaxed);
    if (t == 0) {
        // first use: start somewhere unpredictable, so that whatever a fresh workspace holds is unlikely to look like a tag
        uint32_t seed = (uint32_t)std::chrono::steady_clock::now().time_since_epoch().count() * 2654435761u;
        seed ^= (uint32_t)(uintptr_t)&g_call_tag;
        uint32_t expected = 0;
        g_call_tag.compare_exchange_strong(expected, seed | 1u);
    }
    for (;;) {
        t = (g_call_tag.fetch_add(1, std::memory_order_relaxed) + 1) & 0x7FFFFFFFu;      // 31 bits: the top bit marks "being cleared"
        if (t != 0) return t;
    }
}

unsigned option_wait_polls() { return (unsigned)g_opt_polls.load(std::memory_order_relaxed); }
int option_test_skip_stage() { return g_opt_skip.load(std::memory_order_relaxed); }

void prefer_max_shared(const void* kernel) {
    static std::mutex mu;
    static std::set<std::pair<const void*, int>> done;
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess) return;
    std::lock_guard<std::mutex> lock(mu);
    if (!option_early_weights()) return;
    if (!done.insert({kernel, dev}).second) return;
    // a preference, not a requirement: a failure here changes nothing but the overlap
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared) != cudaSuccess)
        cudaGetLastError();
}

int* sticky_status() {
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
    int* p = g_sticky_ptr[dev].load(std::memory_order_acquire);
    if (!p) {
        void* q = nullptr;
        if (cudaGetSymbolAddress(&q, g_sticky_status) != cudaSuccess) {
            cudaGetLastError();
            return nullptr;
        }
        p = static_cast<int*>(q);
        g_sticky_ptr[dev].store(p, std::memory_order_release);
    }
    return p;
}

bool option_chained_launch() {
    int v = g_opt_chained.load(std::memory_order_relaxed);
    if (v < 0) {                                  // first use: MSAQ_CHAINED_LAUNCH=0 in the environment turns it off
        const char* e = getenv("MSAQ_CHAINED_LAUNCH");
        v = (e && e[0] == '0') ? 0 : 1;
        g_opt_chained.store(v, std::memory_order_relaxed);
    }
    return v != 0;
}

bool option_tensor_memory() { return g_opt_tmem.load(std::memory_order_relaxed) != 0; }

void count_launch(int n) { g_launches.fetch_add((unsigned long long)n, std::memory_order_relaxed); }

// Per-device cache; filled on first use by whichever thread gets there (the
// values are idempotent, so a benign double fill is harmless).
namespace {
constexpr int MAX_DEV = 64;
std::atomic<int> g_sm[MAX_DEV];
std::atomic<int> g_cc[MAX_DEV];

int current_device_attr(std::atomic<int>* cache, cudaDeviceAttr attr) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= MAX_DEV) return 0;
    int v = cache[dev].load(std::memory_order_relaxed);
    if (v == 0) {
        if (cudaDeviceGetAttribute(&v, attr, dev) != cudaSuccess) return 0;
        cache[dev].store(v, std::memory_order_relaxed);
    }
    return v;
}
}  // namespace

int sm_count() {
    const int n = current_device_attr(g_sm, cudaDevAttrMultiProcessorCount);
    return n > 0 ? n : 148;
}

int require_sm100() {
    const int major = current_device_attr(g_cc, cudaDevAttrComputeCapabilityMajor);
    if (major != 10) return fail(MSAQ_ERR_DEVICE, "current device has compute capability major %d; this library is built for sm_100a only", major);
    return MSAQ_OK;
}

}  // namespace msaq

extern "C" int msaq_version(void) { return 1000; }
extern "C" const char* msaq_last_error(void) { return msaq::g_err; }
extern "C" int msaq_set_option(int option, int value) {
    switch (option) {
        case MSAQ_OPT_CHAINED_LAUNCH: msaq::g_opt_chained.store(value ? 1 : 0, std::memory_order_relaxed); return MSAQ_OK;
        case MSAQ_OPT_TENSOR_MEMORY: msaq::g_opt_tmem.store(value ? 1 : 0, std::memory_order_relaxed); return MSAQ_OK;
        case MSAQ_OPT_WAIT_POLLS:
            if (value < 1) return msaq::fail(MSAQ_ERR_ARG, "the poll limit must be positive");
            msaq::g_opt_polls.store(value, std::memory_order_relaxed);
            return MSAQ_OK;
        case MSAQ_OPT_TEST_SKIP_STAGE: msaq::g_opt_skip.store(value < 0 ? -1 : value, std::memory_order_relaxed); return MSAQ_OK;
        case MSAQ_OPT_INKERNEL_STAGING: msaq::g_opt_inkernel.store(value ? 1 : 0, std::memory_order_relaxed); return MSAQ_OK;
        case MSAQ_OPT_EARLY_WEIGHTS: msaq::g_opt_early.store(value ? 1 : 0, std::memory_order_relaxed); return MSAQ_OK;
        default: return msaq::fail(MSAQ_ERR_ARG, "unknown option %d", option);
    }
}
extern "C" int msaq_get_option(int option) {
    switch (option) {
        case MSAQ_OPT_CHAINED_LAUNCH: return msaq::option_chained_launch() ? 1 : 0;
        case MSAQ_OPT_TENSOR_MEMORY: return msaq::option_tensor_memory() ? 1 : 0;
        case MSAQ_OPT_WAIT_POLLS: return (int)msaq::option_wait_polls();
        case MSAQ_OPT_TEST_SKIP_STAGE: return msaq::option_test_skip_stage();
        case MSAQ_OPT_INKERNEL_STAGING: return msaq::option_inkernel_staging() ? 1 : 0;
        case MSAQ_OPT_EARLY_WEIGHTS: return msaq::g_opt_early.load(std::memory_order_relaxed);
        default: return msaq::fail(MSAQ_ERR_ARG, "unknown option %d", option);
    }
}
extern "C" unsigned long long msaq_launch_count(void) { return msaq::g_launches.load(std::memory_order_relaxed); }

extern "C" int msaq_wait_status(int clear, void* stream, int* status_out) {
    if (!status_out) return msaq::fail(MSAQ_ERR_ARG, "null pointer");
    int* p = msaq::sticky_status();
    if (!p) return msaq::fail(MSAQ_ERR_CUDA, "the status word of the current device cannot be located");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    int v = 0;
    cudaError_t e = cudaMemcpyAsync(&v, p, sizeof(int), cudaMemcpyDeviceToHost, st);
    if (e == cudaSuccess && clear) e = cudaMemsetAsync(p, 0, sizeof(int), st);
    if (e == cudaSuccess) e = cudaStreamSynchronize(st);
    if (e != cudaSuccess) return msaq::fail(MSAQ_ERR_CUDA, "reading the status word: %s", cudaGetErrorString(e));
    *status_out = v;
    return MSAQ_OK;
}
