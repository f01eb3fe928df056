// Tensor-core k-means assignment: the sample rows play the queries and the centroids the
// database of the kNN candidate kernel (knn_tc.cu); a lean per-point kernel then re-scores
// the few best candidates exactly, proves the winner against the scoring error bound and
// queues the points it cannot prove for the exact CUDA-core path.
#include "knn_internal.h"
#include "pool.cuh"
#include <cuda_bf16.h>

namespace fl {

// Split operand planes.  An fp32 value v is carried as hi = bf16(v) and lo = bf16(v - hi); the
// plane rows hold [hi | lo | hi] (samples) and [hi | hi | lo] (centroids), so one bf16 product
// over 3 d_pad columns yields  hi.hi + lo.hi + hi.lo,  i.e. the fp32 inner product up to the
// dropped lo.lo term and the second-order residuals: a relative error of about 3 * 2^-18 of
// ||x|| ||c|| instead of 2^-8.  Used when 3 d_pad columns of a 128-row tile fit in shared
// memory (d <= 128).
__device__ __forceinline__ void bf16_split(float v, __nv_bfloat16& hi, __nv_bfloat16& lo) {
    hi = __float2bfloat16_rn(v);
    lo = __float2bfloat16_rn(v - __bfloat162float(hi));
}

// Sample side: [n_pad][3 d_pad + 16], ones in the three columns that meet the centroid plane's
// split -||c||^2/2 terms.
__global__ void split_x_plane_kernel(const float* __restrict__ x, int64_t n, int64_t ldx, int d,
                                     __nv_bfloat16* __restrict__ out, int64_t n_pad, int d_pad) {
    const int pitch = 3 * d_pad + PLANE_AUG_COLS;
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n_pad * pitch) return;
    const int64_t r = i / pitch;
    const int c = (int)(i - r * pitch);
    __nv_bfloat16 o = __float2bfloat16_rn(0.f);
    if (r < n) {
        if (c < 3 * d_pad) {
            const int part = c / d_pad, f = c - part * d_pad;
            if (f < d) {
                __nv_bfloat16 hi, lo;
                bf16_split(__ldg(x + r * ldx + f), hi, lo);
                o = part == 1 ? lo : hi;
            }
        } else if (c < 3 * d_pad + 3) {
            o = __float2bfloat16_rn(1.f);
        }
    }
    out[i] = o;
}

// Centroid side, one warp per row: [m_pad][3 d_pad + 16] rows, ||c||^2/2 per row and the
// largest row norm.  Padding rows score -3e38.
__global__ void split_c_plane_kernel(const float* __restrict__ c, int64_t m, int d, int64_t ld,
                                     __nv_bfloat16* __restrict__ rows, float* __restrict__ hnorm,
                                     unsigned int* __restrict__ maxnorm_bits, int64_t m_pad, int d_pad) {
    const int lane = threadIdx.x & 31;
    const int64_t row = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (row >= m_pad) return;
    const int pitch = 3 * d_pad + PLANE_AUG_COLS;
    __nv_bfloat16* o = rows + row * pitch;
    if (row >= m) {
        for (int t = lane; t < pitch; t += 32) o[t] = __float2bfloat16_rn(t == 3 * d_pad ? -3.0e38f : 0.f);
        if (lane == 0) hnorm[row] = pos_inf();
        return;
    }
    const float* p = c + row * ld;
    float s = 0.f;
    for (int t = lane; t < d_pad; t += 32) {
        const float v = (t < d) ? __ldg(p + t) : 0.f;
        s += v * v;
        __nv_bfloat16 hi, lo;
        bf16_split(v, hi, lo);
        o[t] = hi;
        o[d_pad + t] = hi;
        o[2 * d_pad + t] = lo;
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) s += __shfl_xor_sync(FULL_MASK, s, off);
    if (lane == 0) {
        hnorm[row] = 0.5f * s;
        atomicMax(maxnorm_bits, __float_as_uint(sqrtf(s)));
    }
    if (lane < PLANE_AUG_COLS) {
        const float nh = -0.5f * s;
        const __nv_bfloat16 h1 = __float2bfloat16_rn(nh);
        const float r1 = nh - __bfloat162float(h1);
        const __nv_bfloat16 h2 = __float2bfloat16_rn(r1);
        const float r2 = r1 - __bfloat162float(h2);
        const __nv_bfloat16 h3 = __float2bfloat16_rn(r2);
        o[3 * d_pad + lane] = lane == 0 ? h1 : lane == 1 ? h2 : lane == 2 ? h3 : __float2bfloat16_rn(0.f);
    }
}

// Eight lanes per point, four points per warp.  The scoring pass left, for each half of the
// centroid columns, the best and second-best score and the best centroid.  Both best centroids
// are re-scored with exact fp32 sum (x - c)^2; the closer one wins (lower index on exact ties).
// Every other centroid scored at most `bound` = the larger of the two second-best scores (plus
// the 2^-16 relative perturbation of carrying the column index in the score's low mantissa
// bits), so the label is proven when its exact distance is below ||x||^2 - 2 (bound + eps);
// otherwise the point is queued for the exact path.
__global__ void __launch_bounds__(128) assign_finalize_kernel(
    const float* __restrict__ x, int64_t n, int64_t ldx, const float* __restrict__ c, int K, int64_t ldc, int d,
    int vec, const float* __restrict__ asg_sc, const uint32_t* __restrict__ asg_id, float eps_rel,
    const float* __restrict__ maxnorm, int32_t* __restrict__ labels, int* __restrict__ fb_count,
    int* __restrict__ fb_list, int fb_cap) {
    const int sl = threadIdx.x & 7;
    const int64_t pt_raw = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 3;
    const bool live = pt_raw < n;
    const int64_t pt = live ? pt_raw : n - 1;          // idle groups shadow the last point
    const float4 sc = __ldg(reinterpret_cast<const float4*>(asg_sc + pt * 4));   // b1_0, b2_0, b1_1, b2_1
    const uint2 ids = __ldg(reinterpret_cast<const uint2*>(asg_id + pt * 2));
    const bool v0 = ids.x < (uint32_t)K && sc.x > -1e37f;   // false: no real centroid in that half
    const bool v1 = ids.y < (uint32_t)K && sc.z > -1e37f;
    const float* xp = x + pt * ldx;
    const float* c0 = c + (int64_t)(v0 ? ids.x : 0u) * ldc;
    const float* c1 = c + (int64_t)(v1 ? ids.y : 0u) * ldc;
    float qsq = 0.f, a0 = 0.f, a1 = 0.f;
    if (vec) {
#pragma unroll 4
        for (int t = sl * 4; t < d; t += 32) {
            const float4 xv = __ldg(reinterpret_cast<const float4*>(xp + t));
            const float4 p0 = __ldg(reinterpret_cast<const float4*>(c0 + t));
            const float4 p1 = __ldg(reinterpret_cast<const float4*>(c1 + t));
            qsq += xv.x * xv.x + xv.y * xv.y + xv.z * xv.z + xv.w * xv.w;
            float e0 = xv.x - p0.x, e1 = xv.y - p0.y, e2 = xv.z - p0.z, e3 = xv.w - p0.w;
            a0 += e0 * e0 + e1 * e1 + e2 * e2 + e3 * e3;
            e0 = xv.x - p1.x; e1 = xv.y - p1.y; e2 = xv.z - p1.z; e3 = xv.w - p1.w;
            a1 += e0 * e0 + e1 * e1 + e2 * e2 + e3 * e3;
        }
    } else {
        for (int t = sl; t < d; t += 8) {
            const float xv = __ldg(xp + t);
            const float e0 = xv - __ldg(c0 + t), e1 = xv - __ldg(c1 + t);
            qsq += xv * xv; a0 += e0 * e0; a1 += e1 * e1;
        }
    }
#pragma unroll
    for (int o = 4; o > 0; o >>= 1) {
        qsq += __shfl_xor_sync(FULL_MASK, qsq, o);
        a0 += __shfl_xor_sync(FULL_MASK, a0, o);
        a1 += __shfl_xor_sync(FULL_MASK, a1, o);
    }
    if (!live || sl != 0) return;
    float best_d = pos_inf();
    uint32_t best_i = INVALID_ID;
    if (v0) { best_d = a0; best_i = ids.x; }
    if (v1 && (a1 < best_d || (a1 == best_d && ids.y < best_i))) { best_d = a1; best_i = ids.y; }
    float bound = fmaxf(sc.y, sc.w);
    bool ok = best_i != INVALID_ID;
    if (ok && bound > -1e37f) {
        bound += fabsf(bound) * 3.1e-5f;                       // index bits in the mantissa: 2^-15 relative
        const float mn = __ldg(maxnorm);
        const float eps = eps_rel * sqrtf(qsq) * mn;
        const float lb = qsq - 2.f * (bound + eps);
        const float slack = 1e-5f * (qsq + mn * mn);
        ok = best_d < lb - slack;
    }
    labels[pt] = ok ? (int32_t)best_i : 0;
    if (!ok) {
        const int i = atomicAdd(fb_count, 1);
        if (i < fb_cap) fb_list[i] = (int)pt;
    }
}

struct AssignTcWs {
    int64_t n_pad; int d_pad, pitch; int fb_cap;
    int split;          // 1: split (hi/lo) operand planes of 3 d_pad columns
    int nsplit_fb; int64_t rows_per_split_fb;
    PlaneLayout cl;
    int64_t off_cplane, off_xplane, off_asg_sc, off_asg_id, off_tau, off_cnt, off_fblist, off_fbpart_sc,
        off_fbpart_id, off_fbdist, bytes;
};

// Split planes need the 128-row sample tile of 3 d_pad columns resident in shared memory
// beside a three-slot TMA ring: d <= 128.
static int assign_tc_split(int d) { return d <= 128; }

static int64_t take(int64_t& cur, int64_t bytes) {
    const int64_t o = cur;
    cur += round_up(bytes > 0 ? bytes : 1, 1024);
    return o;
}

static AssignTcWs assign_tc_plan(int64_t n, int K, int d, int have_xplane) {
    AssignTcWs w{};
    w.n_pad = round_up(n, 128);
    w.split = assign_tc_split(d);
    w.d_pad = (int)round_up(d, 64) * (w.split ? 3 : 1);
    w.pitch = w.d_pad + PLANE_AUG_COLS;
    w.cl = plane_layout(K, w.d_pad);     // same row count, hnorm and meta blocks; d_pad feature columns
    w.fb_cap = (int)n;   // every point may take the exact path: no overflow case to report
    simt_split_plan(w.fb_cap, K, 32, d, &w.nsplit_fb, &w.rows_per_split_fb);
    int64_t cur = 0;
    w.off_cplane = take(cur, w.cl.bytes);
    w.off_xplane = have_xplane ? -1 : take(cur, w.n_pad * w.pitch * 2);
    w.off_asg_sc = take(cur, w.n_pad * 4 * 4);
    w.off_asg_id = take(cur, w.n_pad * 2 * 4);
    w.off_tau = take(cur, w.n_pad * 4);
    w.off_cnt = take(cur, 1024);
    w.off_fblist = take(cur, (int64_t)w.fb_cap * 4);
    w.off_fbpart_sc = take(cur, (int64_t)w.fb_cap * w.nsplit_fb * 32 * 4);
    w.off_fbpart_id = take(cur, (int64_t)w.fb_cap * w.nsplit_fb * 32 * 4);
    w.off_fbdist = take(cur, n * 4);
    w.bytes = cur;
    return w;
}

int assign_tc_supported(int64_t n, int K, int d) {
    if (n < 1 || K < 1 || d > 256) return 0;
    return 1;
}

}  // namespace fl

using namespace fl;

extern "C" int64_t fl_kmeans_xplane_bytes(int64_t n, int d) {
    if (n < 1 || d < 1) return 0;
    return round_up(n, 128) * (round_up(d, 64) * (assign_tc_split(d) ? 3 : 1) + PLANE_AUG_COLS) * 2;
}

static int launch_x_plane(const float* x, int64_t n, int64_t ldx, int d, void* plane, cudaStream_t st) {
    const int64_t n_pad = round_up(n, 128);
    const int d_pad = (int)round_up(d, 64);
    if (!assign_tc_split(d)) return launch_query_plane(x, n, ldx, d, plane, n_pad, d_pad, st);
    const int64_t total = n_pad * (3 * d_pad + PLANE_AUG_COLS);
    split_x_plane_kernel<<<(unsigned)ceil_div(total, 256), 256, 0, st>>>(
        x, n, ldx, d, reinterpret_cast<__nv_bfloat16*>(plane), n_pad, d_pad);
    FL_CHECK_LAUNCH();
    return FL_OK;
}

static int launch_c_plane(const float* c, int K, int d, int64_t ldc, char* cpl, const PlaneLayout& L, cudaStream_t st) {
    if (!assign_tc_split(d)) return launch_plane_build(c, K, d, ldc, cpl, st);
    FL_CHECK_CUDA(cudaMemsetAsync(cpl + L.off_meta, 0, 1024, st));
    const int wpb = 8;
    split_c_plane_kernel<<<(unsigned)ceil_div(L.m_pad, wpb), wpb * 32, 0, st>>>(
        c, K, d, ldc, reinterpret_cast<__nv_bfloat16*>(cpl + L.off_rows), reinterpret_cast<float*>(cpl + L.off_hnorm),
        reinterpret_cast<unsigned int*>(cpl + L.off_meta), L.m_pad, (int)round_up(d, 64));
    FL_CHECK_LAUNCH();
    return FL_OK;
}

extern "C" int fl_kmeans_prepare_x_f32(const float* x, int64_t n, int d, int64_t ldx, void* xplane,
                                       int64_t xplane_bytes, void* stream) {
    FL_CHECK_ARG(x && xplane && n >= 1 && d >= 1 && ldx >= d, "fl_kmeans_prepare_x_f32: bad arguments");
    if (xplane_bytes < fl_kmeans_xplane_bytes(n, d)) { set_error("fl_kmeans_prepare_x_f32: plane buffer too small"); return FL_EWORKSPACE; }
    return launch_x_plane(x, n, ldx, d, xplane, (cudaStream_t)stream);
}

extern "C" int64_t fl_kmeans_assign_tc_workspace_bytes(int64_t n, int K, int d, int have_xplane) {
    if (!assign_tc_supported(n, K, d)) return 0;
    return assign_tc_plan(n, K, d, have_xplane).bytes;
}

extern "C" int fl_kmeans_assign_tc_f32(const float* x, int64_t n, int64_t ldx, const void* xplane, const float* c,
                                       int K, int64_t ldc, int d, int32_t* labels, void* ws, int64_t ws_bytes,
                                       int32_t* status, void* stream) {
    FL_CHECK_ARG(n >= 0 && K >= 1 && d >= 1 && ldx >= d && ldc >= d, "fl_kmeans_assign_tc_f32: bad shape");
    if (!assign_tc_supported(n > 0 ? n : 1, K, d)) { set_error("fl_kmeans_assign_tc_f32: d=%d > 256 is not supported", d); return FL_EUNSUPPORTED; }
    if (n == 0) return FL_OK;
    FL_CHECK_ARG(x && c && labels && ws, "fl_kmeans_assign_tc_f32: null pointer");
    FL_CHECK_ARG((reinterpret_cast<uintptr_t>(ws) & 255) == 0, "fl_kmeans_assign_tc_f32: workspace must be 256-byte aligned");
    FL_CHECK_ARG(n < (1ll << 31), "fl_kmeans_assign_tc_f32: more than 2^31 rows");
    const AssignTcWs w = assign_tc_plan(n, K, d, xplane != nullptr);
    if (ws_bytes < w.bytes) { set_error("fl_kmeans_assign_tc_f32: workspace %lld < %lld bytes", (long long)ws_bytes, (long long)w.bytes); return FL_EWORKSPACE; }
    cudaStream_t st = (cudaStream_t)stream;
    char* base = static_cast<char*>(ws);
    if (status) FL_CHECK_CUDA(cudaMemsetAsync(status, 0, sizeof(int32_t) * FL_STATUS_WORDS, st));

    // centroid plane (database side)
    char* cpl = base + w.off_cplane;
    {
        const int rc = launch_c_plane(c, K, d, ldc, cpl, w.cl, st);
        if (rc != FL_OK) return rc;
    }
    // sample plane (query side)
    const char* xpl = static_cast<const char*>(xplane);
    if (!xpl) {
        int rc = launch_x_plane(x, n, ldx, d, base + w.off_xplane, st);
        if (rc != FL_OK) return rc;
        xpl = base + w.off_xplane;
    }
    int* fb_count = reinterpret_cast<int*>(base + w.off_cnt);
    int* fb_list = reinterpret_cast<int*>(base + w.off_fblist);
    FL_CHECK_CUDA(cudaMemsetAsync(fb_count, 0, 1024, st));
    const int vecx = (ldx % 4 == 0) && ((reinterpret_cast<uintptr_t>(x) & 15) == 0);
    const int vecc = (ldc % 4 == 0) && ((reinterpret_cast<uintptr_t>(c) & 15) == 0);
    const int vec = vecx && vecc && (d % 4 == 0);
    {
        float* tau = reinterpret_cast<float*>(base + w.off_tau);
        int rc = launch_fill_f32(tau, w.n_pad, -INFINITY, st);
        if (rc != FL_OK) return rc;
        TcKnnParams tp{};
        tp.qplane = xpl; tp.nq = n; tp.nq_pad = w.n_pad;
        tp.dbrows = cpl + w.cl.off_rows; tp.hnorm = reinterpret_cast<const float*>(cpl + w.cl.off_hnorm);
        tp.m = K; tp.m_pad = w.cl.m_pad; tp.d_pad = w.cl.d_pad;
        tp.tau = tau; tp.status = status;
        float* asg_sc = reinterpret_cast<float*>(base + w.off_asg_sc);
        uint32_t* asg_id = reinterpret_cast<uint32_t*>(base + w.off_asg_id);
        profile_begin(st);
        rc = launch_assign_tc(tp, asg_sc, asg_id, st);
        profile_end(st);
        if (rc != FL_OK) return rc;
        // scoring error relative to ||x|| max||c||: 2^-8 for plain bf16 operands; for split
        // operands 3 * 2^-18 from the dropped terms plus the fp32 accumulation of 400 products
        const float eps_rel = w.split ? 4e-5f : 0.004f;
        assign_finalize_kernel<<<(unsigned)ceil_div(n, 16), 128, 0, st>>>(
            x, n, ldx, c, K, ldc, d, vec, asg_sc, asg_id, eps_rel, reinterpret_cast<const float*>(cpl + w.cl.off_meta),
            labels, fb_count, fb_list, w.fb_cap);
        FL_CHECK_LAUNCH();
    }
    {
        const int rc = launch_fallback_fixup(fb_count, w.fb_cap, status, tc_pool_size(1), st);
        if (rc != FL_OK) return rc;
    }

    // points whose label could not be proven: exact CUDA-core scoring + exact re-rank, k = 1
    SimtKnnParams sp{};
    sp.q = x; sp.ldq = ldx; sp.qlist = fb_list; sp.count_dev = fb_count; sp.count = 0;
    sp.db = c; sp.m = K; sp.ldb = ldc; sp.d = d;
    sp.hnorm = reinterpret_cast<const float*>(cpl + w.cl.off_hnorm);
    sp.K1 = 32; sp.cap = simt_pool_cap(32); sp.npl = sp.cap / 32; sp.keep = simt_pool_keep(32, 1); sp.nsplit = w.nsplit_fb; sp.rows_per_split = w.rows_per_split_fb;
    sp.part_sc = reinterpret_cast<float*>(base + w.off_fbpart_sc);
    sp.part_id = reinterpret_cast<uint32_t*>(base + w.off_fbpart_id);
    sp.vecq = vecx; sp.vecd = vecc;
    int rc = launch_knn_simt(sp, w.fb_cap, st);
    if (rc != FL_OK) return rc;
    FinalizeParams fp{};
    fp.q = x; fp.ldq = ldx; fp.qlist = fb_list; fp.count_dev = fb_count; fp.count = 0;
    fp.db = c; fp.m = K; fp.ldb = ldc; fp.d = d; fp.vec = vec;
    fp.part_sc = sp.part_sc; fp.part_id = sp.part_id; fp.nsplit = w.nsplit_fb; fp.K1 = 32;
    fp.k = 1; fp.rerank = 9; fp.row_offset = 0;
    fp.out_dist = reinterpret_cast<float*>(base + w.off_fbdist); fp.out_idx = labels; fp.verify = 0;
    return launch_knn_finalize(fp, w.fb_cap, st);
}
