// Shared helpers for the flashlib_b200 kernels: error plumbing for the C ABI and the
// warp-level sorting network used by every top-k pool in this library.
#pragma once

#include <cuda_runtime.h>
#include <cuda_fp16.h>
#include <stdint.h>
#include <stdarg.h>
#include <stdio.h>
#include <math.h>

#include "../../include/flashlib_b200.h"

namespace fl {

// ---- host-side error plumbing ------------------------------------------------------
void set_error(const char* fmt, ...);
void count_launch();
// Profiling hooks (no-ops unless fl_profile_enable(1) was called): bracket the dominant
// kernel of an entry point with CUDA events recorded on the caller's stream.
void profile_begin(cudaStream_t st);
void profile_end(cudaStream_t st);
// fl_profile_enable(2): one event per mark along an entry point's launch sequence.
void profile_mark(cudaStream_t st);

#define FL_CHECK_ARG(cond, ...)                                                         \
    do {                                                                                \
        if (!(cond)) {                                                                  \
            ::fl::set_error(__VA_ARGS__);                                               \
            return FL_EINVAL;                                                           \
        }                                                                               \
    } while (0)

#define FL_CHECK_CUDA(expr)                                                             \
    do {                                                                                \
        cudaError_t e__ = (expr);                                                       \
        if (e__ != cudaSuccess) {                                                       \
            ::fl::set_error("%s failed: %s (%s:%d)", #expr, cudaGetErrorString(e__),    \
                            __FILE__, __LINE__);                                        \
            return FL_ECUDA;                                                            \
        }                                                                               \
    } while (0)

// Every kernel launch in the library goes through this macro: it counts the launch
// (fl_launch_count) and surfaces launch-configuration errors.
#define FL_CHECK_LAUNCH()                                                               \
    do {                                                                                \
        ::fl::count_launch();                                                           \
        FL_CHECK_CUDA(cudaGetLastError());                                              \
    } while (0)

static inline int64_t round_up(int64_t a, int64_t b) { return (a + b - 1) / b * b; }
static inline int64_t ceil_div(int64_t a, int64_t b) { return (a + b - 1) / b; }
static inline int pow2_ceil(int v) { int p = 1; while (p < v) p <<= 1; return p; }

// Number of SMs of the current device (cached per device).
int sm_count();
// Opt-in dynamic shared memory limit of the current device in bytes.
int smem_optin_bytes();

// ---- device-side helpers -----------------------------------------------------------
constexpr unsigned FULL_MASK = 0xffffffffu;
constexpr uint32_t INVALID_ID = 0xffffffffu;

// Element types of the caller's rows (FL_DTYPE_* of the C ABI): fp32, or 16-bit storage that is
// widened to fp32 on load (exactly: every bf16 / fp16 value is an fp32 value).
constexpr int DT_F32 = FL_DTYPE_F32, DT_BF16 = FL_DTYPE_BF16, DT_F16 = FL_DTYPE_F16;
static inline int dt_size(int dt) { return dt == DT_F32 ? 4 : 2; }
// Four consecutive elements can be fetched with one load: 16 bytes of fp32, 8 bytes of 16-bit values.
static inline bool dt_vec_ok(const void* p, int64_t ld, int dt) {
    return (ld % 4 == 0) && ((reinterpret_cast<uintptr_t>(p) & (dt == DT_F32 ? 15 : 7)) == 0);
}

#if defined(__CUDACC__)

__device__ __forceinline__ float neg_inf() { return __int_as_float(0xff800000); }
__device__ __forceinline__ float pos_inf() { return __int_as_float(0x7f800000); }

__device__ __forceinline__ float f16_bits_to_f32(unsigned short h) { return __half2float(__ushort_as_half(h)); }
// Element i of a row array of type dt, as fp32.
__device__ __forceinline__ float ld_elem(const void* base, int64_t i, int dt) {
    if (dt == DT_F32) return __ldg(static_cast<const float*>(base) + i);
    const unsigned short h = __ldg(static_cast<const unsigned short*>(base) + i);
    return dt == DT_BF16 ? __uint_as_float((uint32_t)h << 16) : f16_bits_to_f32(h);
}
// Elements i .. i+3 (the address must allow one load: see dt_vec_ok).
__device__ __forceinline__ float4 ld_elem4(const void* base, int64_t i, int dt) {
    if (dt == DT_F32) return __ldg(reinterpret_cast<const float4*>(static_cast<const float*>(base) + i));
    const uint2 w = __ldg(reinterpret_cast<const uint2*>(static_cast<const unsigned short*>(base) + i));
    if (dt == DT_BF16)
        return make_float4(__uint_as_float(w.x << 16), __uint_as_float(w.x & 0xffff0000u), __uint_as_float(w.y << 16),
                           __uint_as_float(w.y & 0xffff0000u));
    return make_float4(f16_bits_to_f32((unsigned short)(w.x & 0xffffu)), f16_bits_to_f32((unsigned short)(w.x >> 16)),
                       f16_bits_to_f32((unsigned short)(w.y & 0xffffu)), f16_bits_to_f32((unsigned short)(w.y >> 16)));
}
__device__ __forceinline__ int dt_size_dev(int dt) { return dt == DT_F32 ? 4 : 2; }
// Address of row r (ld in elements).
__host__ __device__ __forceinline__ const void* row_at(const void* base, int64_t r, int64_t ld, int dt) {
    return static_cast<const char*>(base) + r * ld * (dt == DT_F32 ? 4 : 2);
}

// Bitonic sorting network over NPL*32 (key, id) pairs held NPL per lane; the element at
// register r of lane l has position r*32 + l.  Sorts by DESCENDING key.  With TIEBREAK,
// equal keys are ordered by ascending id, which makes the order total and the result
// independent of where the elements started.
template <int NPL, bool TIEBREAK>
__device__ __forceinline__ void warp_sort_desc(float (&key)[NPL], uint32_t (&id)[NPL]) {
    const int lane = threadIdx.x & 31;
#pragma unroll
    for (int k = 2; k <= NPL * 32; k <<= 1) {
#pragma unroll
        for (int j = k >> 1; j > 0; j >>= 1) {
            if (j >= 32) {
                const int jr = j >> 5;
#pragma unroll
                for (int r = 0; r < NPL; ++r) {
                    const int pr = r ^ jr;
                    if (pr > r) {
                        const bool desc_block = (((r << 5) & k) == 0);
                        const float a = key[r], b = key[pr];
                        const uint32_t ia = id[r], ib = id[pr];
                        // "a should come after b" in a descending block
                        bool a_lt_b = a < b;
                        bool a_gt_b = a > b;
                        if (TIEBREAK) {
                            a_lt_b = a_lt_b || (a == b && ia > ib);
                            a_gt_b = a_gt_b || (a == b && ia < ib);
                        }
                        const bool sw = desc_block ? a_lt_b : a_gt_b;
                        if (sw) {
                            key[r] = b; key[pr] = a;
                            id[r] = ib; id[pr] = ia;
                        }
                    }
                }
            } else {
#pragma unroll
                for (int r = 0; r < NPL; ++r) {
                    const int p = (r << 5) | lane;
                    const float ok = __shfl_xor_sync(FULL_MASK, key[r], j);
                    const uint32_t oi = __shfl_xor_sync(FULL_MASK, id[r], j);
                    const bool lower = (lane & j) == 0;
                    const bool desc_block = ((p & k) == 0);
                    const bool take_max = (lower == desc_block);
                    bool o_gt = ok > key[r];
                    bool o_lt = ok < key[r];
                    if (TIEBREAK) {
                        o_gt = o_gt || (ok == key[r] && oi < id[r]);
                        o_lt = o_lt || (ok == key[r] && oi > id[r]);
                    }
                    const bool take = take_max ? o_gt : o_lt;
                    if (take) { key[r] = ok; id[r] = oi; }
                }
            }
        }
    }
}

// Merges two DESCENDING sequences of NPL*32 (key, id) pairs (same position layout as
// warp_sort_desc) and leaves the NPL*32 largest of their union in (ka, ia), descending.
// Position p of the result is first max(a[p], b[N-1-p]) -- that picks the N largest and
// forms a bitonic sequence -- which the final stages of the bitonic network then sort.
template <int NPL, bool TIEBREAK>
__device__ __forceinline__ void warp_merge_desc(float (&ka)[NPL], uint32_t (&ia)[NPL], const float (&kb)[NPL],
                                                const uint32_t (&ib)[NPL]) {
    const int lane = threadIdx.x & 31;
#pragma unroll
    for (int r = 0; r < NPL; ++r) {
        const float ok = __shfl_sync(FULL_MASK, kb[NPL - 1 - r], 31 - lane);
        const uint32_t oi = __shfl_sync(FULL_MASK, ib[NPL - 1 - r], 31 - lane);
        bool take = ok > ka[r];
        if (TIEBREAK) take = take || (ok == ka[r] && oi < ia[r]);
        if (take) { ka[r] = ok; ia[r] = oi; }
    }
    constexpr int k = NPL * 32;
#pragma unroll
    for (int j = k >> 1; j > 0; j >>= 1) {
        if (j >= 32) {
            const int jr = j >> 5;
#pragma unroll
            for (int r = 0; r < NPL; ++r) {
                const int pr = r ^ jr;
                if (pr > r) {
                    const float a = ka[r], b = ka[pr];
                    const uint32_t xa = ia[r], xb = ia[pr];
                    bool a_lt_b = a < b;
                    if (TIEBREAK) a_lt_b = a_lt_b || (a == b && xa > xb);
                    if (a_lt_b) { ka[r] = b; ka[pr] = a; ia[r] = xb; ia[pr] = xa; }
                }
            }
        } else {
#pragma unroll
            for (int r = 0; r < NPL; ++r) {
                const float ok = __shfl_xor_sync(FULL_MASK, ka[r], j);
                const uint32_t oi = __shfl_xor_sync(FULL_MASK, ia[r], j);
                const bool lower = (lane & j) == 0;       // the lower position keeps the larger key
                bool o_gt = ok > ka[r];
                bool o_lt = ok < ka[r];
                if (TIEBREAK) {
                    o_gt = o_gt || (ok == ka[r] && oi < ia[r]);
                    o_lt = o_lt || (ok == ka[r] && oi > ia[r]);
                }
                const bool take = lower ? o_gt : o_lt;
                if (take) { ka[r] = ok; ia[r] = oi; }
            }
        }
    }
}

// Compacts one row's candidate pool: reads `cnt` (score, id) entries from sc/idv (any
// address space), keeps the K1 best (largest score) at positions [0, K1) in descending
// order and returns the new threshold: the K1-th best score, or -inf while fewer than
// K1 entries exist.  NPL*32 must be >= the pool capacity.  All 32 lanes must call it.
template <int NPL>
__device__ __forceinline__ float warp_pool_compact(float* sc, uint32_t* idv, int cnt, int K1) {
    const int lane = threadIdx.x & 31;
    float key[NPL];
    uint32_t id[NPL];
#pragma unroll
    for (int r = 0; r < NPL; ++r) {
        const int e = (r << 5) | lane;
        const bool ok = e < cnt;
        key[r] = ok ? sc[e] : neg_inf();
        id[r] = ok ? idv[e] : INVALID_ID;
    }
    warp_sort_desc<NPL, false>(key, id);
    float thr = neg_inf();
#pragma unroll
    for (int r = 0; r < NPL; ++r) {
        const int e = (r << 5) | lane;
        if (e < K1) { sc[e] = key[r]; idv[e] = id[r]; }
        if (((K1 - 1) >> 5) == r) thr = __shfl_sync(FULL_MASK, key[r], (K1 - 1) & 31);
    }
    __syncwarp();
    return thr;
}

// Bitonic sort of n (power of two) entries in shared memory: larger key first, smaller id first
// among equal keys.  All THREADS threads of the block must call it.
template <int THREADS>
__device__ __forceinline__ void block_sort_desc(float* key, uint32_t* id, int n) {
    for (int size = 2; size <= n; size <<= 1) {
        for (int stride = size >> 1; stride > 0; stride >>= 1) {
            __syncthreads();
            for (int i = threadIdx.x; i < (n >> 1); i += THREADS) {
                const int a = 2 * i - (i & (stride - 1));
                const int b = a + stride;
                const float ka = key[a], kb = key[b];
                const uint32_t ia = id[a], ib = id[b];
                const bool a_first = ka > kb || (ka == kb && ia <= ib);
                const bool desc = (a & size) == 0;
                if (a_first != desc) { key[a] = kb; key[b] = ka; id[a] = ib; id[b] = ia; }
            }
        }
    }
    __syncthreads();
}

// Largest-value update of a float in global memory (compare-and-swap; a few writers at most).
__device__ __forceinline__ void atomic_max_f32(float* addr, float v) {
    int* ai = reinterpret_cast<int*>(addr);
    int old = *reinterpret_cast<volatile int*>(ai);
    while (__int_as_float(old) < v) {
        const int assumed = old;
        old = atomicCAS(ai, assumed, __float_as_int(v));
        if (old == assumed) break;
    }
}

#endif  // __CUDACC__

}  // namespace fl
