// k-means device work: nearest-centroid assignment, per-cluster sums/counts and the
// centroid finalisation with per-centroid shift.
#include "common.cuh"
#include "simt_tile.cuh"

namespace fl {

__global__ void kmeans_halfnorm_kernel(const float* __restrict__ x, int n, int d, int64_t ld,
                                       float* __restrict__ out) {
    const int lane = threadIdx.x & 31;
    const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (row >= n) return;
    const float* p = x + (int64_t)row * ld;
    float s = 0.f;
    for (int c = lane; c < d; c += 32) { const float v = __ldg(p + c); s += v * v; }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(FULL_MASK, s, o);
    if (lane == 0) out[row] = 0.5f * s;
}

// Exact fp32 assignment: 64 points per block against all centroids in tiles of 128.
// The candidates maximise <x,c> - ||c||^2/2, i.e. minimise ||x - c||^2.  The best TWO by that score are
// kept and re-scored with fp32 sum (x - c)^2: where two centroids lie closer together than the
// rounding of the expanded score resolves (near-duplicate centroids), the expansion alone -- which is
// all the reference's kernels and its CPU path use -- picks either; the direct distance picks the
// nearer.  On exact ties the lowest centroid index wins.
template <int TQ>
__global__ void __launch_bounds__(256) kmeans_assign_simt_kernel(
    const float* __restrict__ x, int64_t n, int64_t ldx, const float* __restrict__ c, int K, int64_t ldc,
    int d, const float* __restrict__ hnorm, int32_t* __restrict__ labels, int vecx, int vecc, int64_t xbs, int64_t cbs) {
    using T = SimtTile<TQ>;
    constexpr int BQ = T::BQ;
    extern __shared__ __align__(16) float smem[];
    const int tid = threadIdx.x;
    const int tx = tid & 15, ty = tid >> 4;
    const int64_t row0 = (int64_t)blockIdx.x * BQ;
    // batch item blockIdx.y: its own rows, centroids, half norms and labels
    x += (int64_t)blockIdx.y * xbs;
    c += (int64_t)blockIdx.y * cbs;
    hnorm += (int64_t)blockIdx.y * K;
    labels += (int64_t)blockIdx.y * n;

    const void* qrow[T::QL];
#pragma unroll
    for (int i = 0; i < T::QL; ++i) {
        const int r = (i * 256 + tid) >> 3;
        qrow[i] = (r < BQ && row0 + r < n) ? x + (row0 + r) * ldx : nullptr;
    }
    float best[TQ], sec[TQ];
    int bidx[TQ], sidx[TQ];
#pragma unroll
    for (int i = 0; i < TQ; ++i) { best[i] = sec[i] = neg_inf(); bidx[i] = sidx[i] = 0x7fffffff; }
    auto beats = [](float a, int ai, float b, int bi) { return a > b || (a == b && ai < bi); };

    for (int tile = 0; tile < K; tile += 128) {
        const void* drow[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int gr = tile + ((i * 256 + tid) >> 3);
            drow[i] = gr < K ? c + (int64_t)gr * ldc : nullptr;
        }
        float acc[TQ][8];
        simt_cross_tile<TQ>(qrow, drow, d, vecx != 0, vecc != 0, smem, acc);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const int col = tile + ((j < 4) ? (tx * 4 + j) : (64 + tx * 4 + (j - 4)));
            if (col < K) {
                const float hv = __ldg(hnorm + col);
#pragma unroll
                for (int i = 0; i < TQ; ++i) {
                    const float s = acc[i][j] - hv;
                    if (beats(s, col, best[i], bidx[i])) { sec[i] = best[i]; sidx[i] = bidx[i]; best[i] = s; bidx[i] = col; }
                    else if (beats(s, col, sec[i], sidx[i])) { sec[i] = s; sidx[i] = col; }
                }
            }
        }
    }
    // the 16 threads sharing a point row sit in one half warp
#pragma unroll
    for (int i = 0; i < TQ; ++i) {
#pragma unroll
        for (int o = 8; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(FULL_MASK, best[i], o), os = __shfl_xor_sync(FULL_MASK, sec[i], o);
            const int oi = __shfl_xor_sync(FULL_MASK, bidx[i], o), osi = __shfl_xor_sync(FULL_MASK, sidx[i], o);
            if (beats(ob, oi, best[i], bidx[i])) {
                // the other side's best leads: the runner-up is this side's best or the other side's second
                if (beats(os, osi, best[i], bidx[i])) { sec[i] = os; sidx[i] = osi; } else { sec[i] = best[i]; sidx[i] = bidx[i]; }
                best[i] = ob; bidx[i] = oi;
            } else if (beats(ob, oi, sec[i], sidx[i])) {
                sec[i] = ob; sidx[i] = oi;
            }
        }
        // every thread of the row now holds the same two candidates: direct distances, 16 lanes across the row
        const int64_t r = row0 + ty * TQ + i;
        int label = bidx[i];
        if (sidx[i] != 0x7fffffff) {               // (uniform over the half warp)
            float d1 = 0.f, d2 = 0.f;
            if (r < n) {
                const float* xp = x + r * ldx;
                const float* c1 = c + (int64_t)bidx[i] * ldc;
                const float* c2 = c + (int64_t)sidx[i] * ldc;
                for (int t = tx; t < d; t += 16) {
                    const float xv = __ldg(xp + t);
                    const float e1 = xv - __ldg(c1 + t), e2 = xv - __ldg(c2 + t);
                    d1 += e1 * e1;
                    d2 += e2 * e2;
                }
            }
#pragma unroll
            for (int o = 8; o > 0; o >>= 1) {
                d1 += __shfl_xor_sync(FULL_MASK, d1, o);
                d2 += __shfl_xor_sync(FULL_MASK, d2, o);
            }
            if (d2 < d1 || (d2 == d1 && sidx[i] < bidx[i])) label = sidx[i];
        }
        if (tx == 0 && r < n) labels[r] = label;
    }
}

// One warp per chunk of rows; consecutive rows with the same label are summed in
// registers and flushed with one atomic add per feature per run.
template <int DPL>
__global__ void kmeans_update_kernel(const float* __restrict__ x, int64_t n, int64_t ldx, int d,
                                     const int32_t* __restrict__ labels, int K, float* __restrict__ sums,
                                     int32_t* __restrict__ cnts, int rows_per_warp, int dbase, int64_t nb, int Kb) {
    const int lane = threadIdx.x & 31;
    const int64_t w = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const int64_t r0 = w * rows_per_warp;
    if (r0 >= n) return;
    const int64_t r1 = min(n, r0 + (int64_t)rows_per_warp);
    float acc[DPL];
#pragma unroll
    for (int i = 0; i < DPL; ++i) acc[i] = 0.f;
    int cur = -1, run = 0;
    for (int64_t r = r0; r < r1; ++r) {
        int lab = __ldg(labels + r);
        if (lab >= 0 && lab < Kb) lab += (int)(r / nb) * Kb; else lab = -1;
        if (lab != cur) {
            if (cur >= 0 && cur < K) {
#pragma unroll
                for (int i = 0; i < DPL; ++i) {
                    const int cidx = dbase + i * 32 + lane;
                    if (cidx < d) atomicAdd(sums + (int64_t)cur * d + cidx, acc[i]);
                }
                if (lane == 0 && dbase == 0) atomicAdd(cnts + cur, run);
            }
#pragma unroll
            for (int i = 0; i < DPL; ++i) acc[i] = 0.f;
            cur = lab;
            run = 0;
        }
        const float* p = x + r * ldx;
#pragma unroll
        for (int i = 0; i < DPL; ++i) {
            const int cidx = dbase + i * 32 + lane;
            if (cidx < d) acc[i] += __ldg(p + cidx);
        }
        ++run;
    }
    if (cur >= 0 && cur < K) {
#pragma unroll
        for (int i = 0; i < DPL; ++i) {
            const int cidx = dbase + i * 32 + lane;
            if (cidx < d) atomicAdd(sums + (int64_t)cur * d + cidx, acc[i]);
        }
        if (lane == 0 && dbase == 0) atomicAdd(cnts + cur, run);
    }
}

// Same, for rows and sums that allow 16-byte accesses (d, ldx multiples of 4, aligned bases): each
// lane owns 4 contiguous features per 128, the next row is fetched while the current one is
// accumulated, and a run is flushed with one 16-byte atomic add per lane.
template <int V>
__global__ void kmeans_update_vec_kernel(const float* __restrict__ x, int64_t n, int64_t ldx, int d,
                                         const int32_t* __restrict__ labels, int K, float* __restrict__ sums,
                                         int32_t* __restrict__ cnts, int rows_per_warp, int64_t nb, int Kb) {
    const int lane = threadIdx.x & 31;
    const int64_t w = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const int64_t r0 = w * rows_per_warp;
    if (r0 >= n) return;
    const int64_t r1 = min(n, r0 + (int64_t)rows_per_warp);
    float4 acc[V], nxt[V];
    auto load_row = [&](int64_t r, float4 (&v)[V]) {
        const float* p = x + r * ldx;
#pragma unroll
        for (int i = 0; i < V; ++i) {
            const int cidx = (i * 32 + lane) * 4;
            v[i] = cidx < d ? __ldg(reinterpret_cast<const float4*>(p + cidx)) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
    };
    auto flush = [&](int cur, int run) {
        if (cur < 0 || cur >= K) return;
#pragma unroll
        for (int i = 0; i < V; ++i) {
            const int cidx = (i * 32 + lane) * 4;
            if (cidx < d) atomicAdd(reinterpret_cast<float4*>(sums + (int64_t)cur * d + cidx), acc[i]);
        }
        if (lane == 0) atomicAdd(cnts + cur, run);
    };
#pragma unroll
    for (int i = 0; i < V; ++i) acc[i] = make_float4(0.f, 0.f, 0.f, 0.f);
    // label of row r in the stacked problem: batch item r / nb owns clusters [item * Kb, (item + 1) * Kb)
    auto label_of = [&](int64_t r) {
        const int l = __ldg(labels + r);
        return (l >= 0 && l < Kb) ? l + (int)(r / nb) * Kb : -1;
    };
    int cur = -1, run = 0;
    int lab_n = label_of(r0);
    load_row(r0, nxt);
    for (int64_t r = r0; r < r1; ++r) {
        const int lab = lab_n;
        float4 v[V];
#pragma unroll
        for (int i = 0; i < V; ++i) v[i] = nxt[i];
        if (r + 1 < r1) {
            lab_n = label_of(r + 1);
            load_row(r + 1, nxt);
        }
        if (lab != cur) {
            flush(cur, run);
#pragma unroll
            for (int i = 0; i < V; ++i) acc[i] = make_float4(0.f, 0.f, 0.f, 0.f);
            cur = lab;
            run = 0;
        }
#pragma unroll
        for (int i = 0; i < V; ++i) { acc[i].x += v[i].x; acc[i].y += v[i].y; acc[i].z += v[i].z; acc[i].w += v[i].w; }
        ++run;
    }
    flush(cur, run);
}

// Incremental form of the update: sums and counts already hold the result for the labels in `prev`;
// only the points whose label differs from it are touched -- their row is taken out of the old
// cluster's sum and added to the new one's -- and `prev` is brought up to date.  One warp per 32
// consecutive points: the lanes compare the labels, then the warp handles the changed points one
// by one with all lanes across the row.  After the first Lloyd iterations under 1 % of the points
// change sides, so this reads the two label arrays and a few rows instead of every row.
__global__ void kmeans_update_delta_kernel(const float* __restrict__ x, int64_t n, int64_t ldx, int d,
                                           const int32_t* __restrict__ labels, int32_t* __restrict__ prev, int K,
                                           float* __restrict__ sums, int32_t* __restrict__ cnts, int vec) {
    const int lane = threadIdx.x & 31;
    const int64_t nwarps = ((int64_t)gridDim.x * blockDim.x) >> 5;
    for (int64_t base = (((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5) * 32; base < n; base += nwarps * 32) {
        const int64_t r = base + lane;
        int lab = -1, old = -1;
        if (r < n) {
            lab = __ldg(labels + r);
            old = prev[r];
            if (lab < 0 || lab >= K) lab = -1;
            if (old < 0 || old >= K) old = -1;
            if (lab != old) prev[r] = lab;
        }
        unsigned changed = __ballot_sync(FULL_MASK, lab != old);
        while (changed) {
            const int src = __ffs(changed) - 1;
            changed &= changed - 1;
            const int to = __shfl_sync(FULL_MASK, lab, src), from = __shfl_sync(FULL_MASK, old, src);
            const float* p = x + (base + src) * ldx;
            if (vec) {
                for (int c = lane * 4; c < d; c += 128) {
                    const float4 v = __ldg(reinterpret_cast<const float4*>(p + c));
                    if (from >= 0) atomicAdd(reinterpret_cast<float4*>(sums + (int64_t)from * d + c), make_float4(-v.x, -v.y, -v.z, -v.w));
                    if (to >= 0) atomicAdd(reinterpret_cast<float4*>(sums + (int64_t)to * d + c), v);
                }
            } else {
                for (int c = lane; c < d; c += 32) {
                    const float v = __ldg(p + c);
                    if (from >= 0) atomicAdd(sums + (int64_t)from * d + c, -v);
                    if (to >= 0) atomicAdd(sums + (int64_t)to * d + c, v);
                }
            }
            if (lane == 0) {
                if (from >= 0) atomicAdd(cnts + from, -1);
                if (to >= 0) atomicAdd(cnts + to, 1);
            }
        }
    }
}

// One block per centroid.
__global__ void __launch_bounds__(128) kmeans_finalize_kernel(const float* __restrict__ sums,
                                                              const int32_t* __restrict__ cnts,
                                                              const float* __restrict__ old_c,
                                                              float* __restrict__ new_c,
                                                              float* __restrict__ shift, int K, int d) {
    const int j = blockIdx.x;
    const int cnt = cnts[j];
    const float fc = (float)cnt;
    float s = 0.f;
    for (int t = threadIdx.x; t < d; t += blockDim.x) {
        const float o = old_c[(int64_t)j * d + t];
        const float v = cnt > 0 ? sums[(int64_t)j * d + t] / fc : o;
        new_c[(int64_t)j * d + t] = v;
        const float df = v - o;
        s += df * df;
    }
    __shared__ float red[4];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(FULL_MASK, s, o);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = s;
    __syncthreads();
    if (threadIdx.x == 0) shift[j] = sqrtf(red[0] + red[1] + red[2] + red[3]);
}

}  // namespace fl

using namespace fl;

extern "C" int64_t fl_kmeans_assign_workspace_bytes(int64_t n, int K, int d) {
    (void)n; (void)d;
    if (K < 1) return 0;
    return round_up((int64_t)K * 4, 1024);
}

extern "C" int fl_kmeans_assign_f32(const float* x, int64_t n, int64_t ldx, const float* c, int K,
                                    int64_t ldc, int d, int32_t* labels, void* ws, int64_t ws_bytes,
                                    void* stream) {
    FL_CHECK_ARG(n >= 0 && K >= 1 && d >= 1 && ldx >= d && ldc >= d, "fl_kmeans_assign_f32: bad shape");
    if (n == 0) return FL_OK;
    FL_CHECK_ARG(x && c && labels && ws, "fl_kmeans_assign_f32: null pointer");
    if (ws_bytes < fl_kmeans_assign_workspace_bytes(n, K, d)) {
        set_error("fl_kmeans_assign_f32: workspace too small");
        return FL_EWORKSPACE;
    }
    cudaStream_t st = (cudaStream_t)stream;
    float* hnorm = static_cast<float*>(ws);
    kmeans_halfnorm_kernel<<<(unsigned)ceil_div(K, 8), 256, 0, st>>>(c, K, d, ldc, hnorm);
    FL_CHECK_LAUNCH();
    const int vecx = (ldx % 4 == 0) && ((reinterpret_cast<uintptr_t>(x) & 15) == 0);
    const int vecc = (ldc % 4 == 0) && ((reinterpret_cast<uintptr_t>(c) & 15) == 0);
    constexpr int TQ = 4;
    const size_t smem = sizeof(float) * SimtTile<TQ>::SLAB_FLOATS;
    FL_CHECK_CUDA(cudaFuncSetAttribute(kmeans_assign_simt_kernel<TQ>,
                                       cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    profile_begin(st);
    kmeans_assign_simt_kernel<TQ><<<(unsigned)ceil_div(n, SimtTile<TQ>::BQ), 256, smem, st>>>(
        x, n, ldx, c, K, ldc, d, hnorm, labels, vecx, vecc, 0, 0);
    profile_end(st);
    FL_CHECK_LAUNCH();
    return FL_OK;
}

// ---------------------------------------------------------------------------------------
// Assignment without a caller-provided workspace.
//
// Some hosts of this library may only launch work: a plugin that is handed a stream and its
// input/output buffers but no allocator, a service that gave all device memory to its own
// pool at start-up, a latency-critical loop that must not meet cudaMalloc's device-wide
// synchronisation.  For them the per-centroid half norms, the one piece of scratch the
// assignment needs, live in a fixed array that is part of the loaded library image.
//
// The array holds FL_KMEANS_NOALLOC_MAX_K floats (64 KiB) on every GPU that loads the library
// and stays there until the process exits.  Every call on a device uses the same array and
// leaves its half norms behind: each call overwrites the K entries it reads before reading
// them, so nothing has to be cleared, but two calls that overlap on one GPU (different
// streams, no ordering between them) race on it and must be serialised by the caller.
static __device__ __align__(256) float g_kmeans_noalloc_hnorm[FL_KMEANS_NOALLOC_MAX_K];

// Device address of the array for the current device.  Host code cannot use the symbol's
// name as a pointer, so the address is looked up once per device (with that device current)
// and cached.  The first call on a device does this look-up, which is why that call should
// happen before any stream capture begins.
static int kmeans_noalloc_scratch(float** out) {
    static float* cached[64];
    int dev = 0;
    FL_CHECK_CUDA(cudaGetDevice(&dev));
    FL_CHECK_ARG(dev >= 0 && dev < 64, "fl_kmeans_assign_noalloc_f32: device ordinal %d out of range", dev);
    if (cached[dev] == nullptr) {
        float* ptr = nullptr;
        FL_CHECK_CUDA(cudaGetSymbolAddress((void**)&ptr, g_kmeans_noalloc_hnorm));
        cached[dev] = ptr;
    }
    *out = cached[dev];
    return FL_OK;
}

extern "C" int fl_kmeans_assign_noalloc_f32(const float* x, int64_t n, int64_t ldx, const float* c, int K,
                                            int64_t ldc, int d, int32_t* labels, void* stream) {
    FL_CHECK_ARG(n >= 0 && K >= 1 && d >= 1 && ldx >= d && ldc >= d, "fl_kmeans_assign_noalloc_f32: bad shape");
    if (K > FL_KMEANS_NOALLOC_MAX_K) {
        set_error("fl_kmeans_assign_noalloc_f32: K=%d exceeds the built-in scratch of %d centroids; "
                  "use fl_kmeans_assign_f32 with a workspace", K, FL_KMEANS_NOALLOC_MAX_K);
        return FL_EUNSUPPORTED;
    }
    if (n == 0) return FL_OK;
    FL_CHECK_ARG(x && c && labels, "fl_kmeans_assign_noalloc_f32: null pointer");
    float* hnorm = nullptr;
    const int rc = kmeans_noalloc_scratch(&hnorm);
    if (rc != FL_OK) return rc;
    cudaStream_t st = (cudaStream_t)stream;
    kmeans_halfnorm_kernel<<<(unsigned)ceil_div(K, 8), 256, 0, st>>>(c, K, d, ldc, hnorm);
    FL_CHECK_LAUNCH();
    const int vecx = (ldx % 4 == 0) && ((reinterpret_cast<uintptr_t>(x) & 15) == 0);
    const int vecc = (ldc % 4 == 0) && ((reinterpret_cast<uintptr_t>(c) & 15) == 0);
    constexpr int TQ = 4;
    const size_t smem = sizeof(float) * SimtTile<TQ>::SLAB_FLOATS;
    FL_CHECK_CUDA(cudaFuncSetAttribute(kmeans_assign_simt_kernel<TQ>,
                                       cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    kmeans_assign_simt_kernel<TQ><<<(unsigned)ceil_div(n, SimtTile<TQ>::BQ), 256, smem, st>>>(
        x, n, ldx, c, K, ldc, d, hnorm, labels, vecx, vecc, 0, 0);
    FL_CHECK_LAUNCH();
    return FL_OK;
}

// Sums / counts of `n` stacked rows: batch item i owns rows [i nb, (i + 1) nb) and clusters
// [i Kb, (i + 1) Kb) of the K = items x Kb stacked clusters (one item: nb = n, Kb = K).
static int kmeans_update_impl(const float* x, int64_t n, int64_t ldx, int d, const int32_t* labels, int K, float* sums,
                              int32_t* cnts, int64_t nb, int Kb, cudaStream_t st) {
    FL_CHECK_CUDA(cudaMemsetAsync(sums, 0, sizeof(float) * (size_t)K * d, st));
    FL_CHECK_CUDA(cudaMemsetAsync(cnts, 0, sizeof(int32_t) * (size_t)K, st));
    if (n == 0) return FL_OK;
    FL_CHECK_ARG(x && labels, "fl_kmeans_update_f32: null pointer");
    const int rows_per_warp = 16;
    const int64_t warps = ceil_div(n, rows_per_warp);
    const unsigned grid = (unsigned)ceil_div(warps, 8);
    const bool vec = d % 4 == 0 && ldx % 4 == 0 && d <= 512 && ((reinterpret_cast<uintptr_t>(x) & 15) == 0) &&
                     ((reinterpret_cast<uintptr_t>(sums) & 15) == 0);
    if (vec) {
        if (d <= 128) kmeans_update_vec_kernel<1><<<grid, 256, 0, st>>>(x, n, ldx, d, labels, K, sums, cnts, rows_per_warp, nb, Kb);
        else if (d <= 256) kmeans_update_vec_kernel<2><<<grid, 256, 0, st>>>(x, n, ldx, d, labels, K, sums, cnts, rows_per_warp, nb, Kb);
        else kmeans_update_vec_kernel<4><<<grid, 256, 0, st>>>(x, n, ldx, d, labels, K, sums, cnts, rows_per_warp, nb, Kb);
        FL_CHECK_LAUNCH();
        return FL_OK;
    }
    for (int dbase = 0; dbase < d; dbase += 256) {
        const int rem = d - dbase;
        if (rem <= 32)
            kmeans_update_kernel<1><<<grid, 256, 0, st>>>(x, n, ldx, d, labels, K, sums, cnts, rows_per_warp, dbase, nb, Kb);
        else if (rem <= 64)
            kmeans_update_kernel<2><<<grid, 256, 0, st>>>(x, n, ldx, d, labels, K, sums, cnts, rows_per_warp, dbase, nb, Kb);
        else if (rem <= 128)
            kmeans_update_kernel<4><<<grid, 256, 0, st>>>(x, n, ldx, d, labels, K, sums, cnts, rows_per_warp, dbase, nb, Kb);
        else
            kmeans_update_kernel<8><<<grid, 256, 0, st>>>(x, n, ldx, d, labels, K, sums, cnts, rows_per_warp, dbase, nb, Kb);
        FL_CHECK_LAUNCH();
    }
    return FL_OK;
}

extern "C" int fl_kmeans_update_f32(const float* x, int64_t n, int64_t ldx, int d, const int32_t* labels,
                                    int K, float* sums, int32_t* cnts, void* stream) {
    FL_CHECK_ARG(n >= 0 && K >= 1 && d >= 1 && ldx >= d, "fl_kmeans_update_f32: bad shape");
    FL_CHECK_ARG(sums && cnts, "fl_kmeans_update_f32: null pointer");
    return kmeans_update_impl(x, n, ldx, d, labels, K, sums, cnts, n > 0 ? n : 1, K, (cudaStream_t)stream);
}

extern "C" int fl_kmeans_update_delta_f32(const float* x, int64_t n, int64_t ldx, int d, const int32_t* labels,
                                          int32_t* prev_labels, int K, float* sums, int32_t* cnts, void* stream) {
    FL_CHECK_ARG(n >= 0 && K >= 1 && d >= 1 && ldx >= d, "fl_kmeans_update_delta_f32: bad shape");
    FL_CHECK_ARG(sums && cnts, "fl_kmeans_update_delta_f32: null pointer");
    if (n == 0) return FL_OK;
    FL_CHECK_ARG(x && labels && prev_labels, "fl_kmeans_update_delta_f32: null pointer");
    const int vec = d % 4 == 0 && ldx % 4 == 0 && ((reinterpret_cast<uintptr_t>(x) & 15) == 0) &&
                    ((reinterpret_cast<uintptr_t>(sums) & 15) == 0);
    int64_t blocks = ceil_div(ceil_div(n, 32), 8);
    if (blocks > (int64_t)sm_count() * 16) blocks = (int64_t)sm_count() * 16;
    kmeans_update_delta_kernel<<<(unsigned)blocks, 256, 0, (cudaStream_t)stream>>>(x, n, ldx, d, labels, prev_labels, K, sums,
                                                                                  cnts, vec);
    FL_CHECK_LAUNCH();
    return FL_OK;
}

extern "C" int fl_kmeans_update_batch_f32(const float* x, int batch, int64_t n, int64_t ldx, int d, const int32_t* labels,
                                          int K, float* sums, int32_t* cnts, void* stream) {
    FL_CHECK_ARG(batch >= 1 && n >= 0 && K >= 1 && d >= 1 && ldx >= d, "fl_kmeans_update_batch_f32: bad shape");
    FL_CHECK_ARG((int64_t)batch * K < (1ll << 31) && (int64_t)batch * n < (1ll << 40), "fl_kmeans_update_batch_f32: too large");
    FL_CHECK_ARG(sums && cnts, "fl_kmeans_update_batch_f32: null pointer");
    return kmeans_update_impl(x, (int64_t)batch * n, ldx, d, labels, batch * K, sums, cnts, n > 0 ? n : 1, K, (cudaStream_t)stream);
}

extern "C" int64_t fl_kmeans_assign_batch_workspace_bytes(int batch, int64_t n, int K, int d) {
    (void)n; (void)d;
    if (batch < 1 || K < 1) return 0;
    return round_up((int64_t)batch * K * 4, 1024);
}

extern "C" int fl_kmeans_assign_batch_f32(const float* x, int batch, int64_t n, int64_t ldx, int64_t x_batch_stride,
                                          const float* c, int K, int64_t ldc, int64_t c_batch_stride, int d,
                                          int32_t* labels, void* ws, int64_t ws_bytes, void* stream) {
    FL_CHECK_ARG(batch >= 1 && batch <= 65535 && n >= 0 && K >= 1 && d >= 1 && ldx >= d && ldc >= d,
                 "fl_kmeans_assign_batch_f32: bad shape");
    if (n == 0) return FL_OK;
    FL_CHECK_ARG(x && c && labels && ws, "fl_kmeans_assign_batch_f32: null pointer");
    FL_CHECK_ARG(c_batch_stride == (int64_t)K * ldc, "fl_kmeans_assign_batch_f32: the centroid sets must lie back to back");
    if (ws_bytes < fl_kmeans_assign_batch_workspace_bytes(batch, n, K, d)) {
        set_error("fl_kmeans_assign_batch_f32: workspace too small");
        return FL_EWORKSPACE;
    }
    cudaStream_t st = (cudaStream_t)stream;
    float* hnorm = static_cast<float*>(ws);
    // the centroid sets are contiguous: one pass gives the half norms of all batch items
    kmeans_halfnorm_kernel<<<(unsigned)ceil_div((int64_t)batch * K, 8), 256, 0, st>>>(c, batch * K, d, ldc, hnorm);
    FL_CHECK_LAUNCH();
    const int vecx = (ldx % 4 == 0) && (x_batch_stride % 4 == 0) && ((reinterpret_cast<uintptr_t>(x) & 15) == 0);
    const int vecc = (ldc % 4 == 0) && ((reinterpret_cast<uintptr_t>(c) & 15) == 0);
    constexpr int TQ = 4;
    const size_t smem = sizeof(float) * SimtTile<TQ>::SLAB_FLOATS;
    FL_CHECK_CUDA(cudaFuncSetAttribute(kmeans_assign_simt_kernel<TQ>,
                                       cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    kmeans_assign_simt_kernel<TQ><<<dim3((unsigned)ceil_div(n, SimtTile<TQ>::BQ), (unsigned)batch), 256, smem, st>>>(
        x, n, ldx, c, K, ldc, d, hnorm, labels, vecx, vecc, x_batch_stride, c_batch_stride);
    FL_CHECK_LAUNCH();
    return FL_OK;
}

extern "C" int fl_kmeans_finalize_f32(const float* sums, const int32_t* cnts, const float* old_c,
                                      float* new_c, float* shift, int K, int d, void* stream) {
    FL_CHECK_ARG(K >= 1 && d >= 1, "fl_kmeans_finalize_f32: bad shape");
    FL_CHECK_ARG(sums && cnts && old_c && new_c && shift, "fl_kmeans_finalize_f32: null pointer");
    kmeans_finalize_kernel<<<(unsigned)K, 128, 0, (cudaStream_t)stream>>>(sums, cnts, old_c, new_c, shift, K, d);
    FL_CHECK_LAUNCH();
    return FL_OK;
}
