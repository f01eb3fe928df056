// Error plumbing, version and device queries of the C ABI.
#include "common.cuh"

namespace fl {

static thread_local char g_err[512] = "";

void set_error(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
}

static unsigned long long g_launches = 0;
void count_launch() { __atomic_add_fetch(&g_launches, 1ull, __ATOMIC_RELAXED); }

// Ring of event pairs around the dominant kernel of the profiled entry points.
constexpr int PROFILE_SLOTS = 256;
static int g_profile_on = 0;
static int g_profile_n = 0;
static cudaEvent_t g_ev_begin[PROFILE_SLOTS];
static cudaEvent_t g_ev_end[PROFILE_SLOTS];
static cudaEvent_t g_ev_end_own[PROFILE_SLOTS];
static bool g_ev_made = false;

// Mode 2 (fl_profile_enable(2)): instead of one bracket per call, every profile_mark() along an
// entry point's launch sequence records an event; sample i is the time from mark i to mark i + 1.
void profile_mark(cudaStream_t st) {
    if (g_profile_on != 2 || g_profile_n >= PROFILE_SLOTS) return;
    cudaEventRecord(g_ev_begin[g_profile_n], st);
    if (g_profile_n > 0) g_ev_end[g_profile_n - 1] = g_ev_begin[g_profile_n];
    ++g_profile_n;
}

void profile_begin(cudaStream_t st) {
    if (g_profile_on != 1 || g_profile_n >= PROFILE_SLOTS) return;
    cudaEventRecord(g_ev_begin[g_profile_n], st);
}
void profile_end(cudaStream_t st) {
    if (g_profile_on != 1 || g_profile_n >= PROFILE_SLOTS) return;
    cudaEventRecord(g_ev_end[g_profile_n], st);
    ++g_profile_n;
}

int sm_count() {
    static int cached[64];
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
    if (cached[dev] == 0) {
        int v = 0;
        if (cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || v <= 0)
            v = 148;
        cached[dev] = v;
    }
    return cached[dev];
}

int smem_optin_bytes() {
    static int cached[64];
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 227 * 1024;
    if (cached[dev] == 0) {
        int v = 0;
        if (cudaDeviceGetAttribute(&v, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev) != cudaSuccess ||
            v <= 0)
            v = 227 * 1024;
        cached[dev] = v;
    }
    return cached[dev];
}

}  // namespace fl

extern "C" int fl_version(void) { return 100; }

extern "C" const char* fl_last_error(void) { return fl::g_err; }

extern "C" int fl_device_ok(void) {
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess || n <= 0) {
        cudaGetLastError();
        return 0;
    }
    int dev = 0, major = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return 0;
    if (cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev) != cudaSuccess) return 0;
    return major == 10 ? 1 : 0;
}

extern "C" unsigned long long fl_launch_count(void) { return __atomic_load_n(&fl::g_launches, __ATOMIC_RELAXED); }

extern "C" int fl_profile_enable(int on) {
    using namespace fl;
    if (on && !g_ev_made) {
        for (int i = 0; i < PROFILE_SLOTS; ++i) {
            FL_CHECK_CUDA(cudaEventCreate(&g_ev_begin[i]));
            FL_CHECK_CUDA(cudaEventCreate(&g_ev_end[i]));
            g_ev_end_own[i] = g_ev_end[i];
        }
        g_ev_made = true;
    }
    if (g_ev_made && g_profile_on == 2) {
        // mode 2 aliased the end events to the following marks: give every slot its own event back
        for (int i = 0; i < PROFILE_SLOTS; ++i) g_ev_end[i] = g_ev_end_own[i];
    }
    g_profile_on = on == 2 ? 2 : (on ? 1 : 0);
    g_profile_n = 0;
    return FL_OK;
}

extern "C" int fl_profile_count(void) { return fl::g_profile_n; }

extern "C" int fl_profile_read_ms(int i, float* ms) {
    using namespace fl;
    FL_CHECK_ARG(ms && i >= 0 && i < (g_profile_on == 2 ? g_profile_n - 1 : g_profile_n), "fl_profile_read_ms: no such sample %d", i);
    FL_CHECK_CUDA(cudaEventSynchronize(g_ev_end[i]));
    FL_CHECK_CUDA(cudaEventElapsedTime(ms, g_ev_begin[i], g_ev_end[i]));
    return FL_OK;
}
