// Tensor-core k-means assignment: the sample rows play the queries and the centroids the
// database of the kNN candidate kernel (knn_tc.cu); a lean per-point kernel then re-scores
// the few best candidates exactly, proves the winner against the scoring error bound and
// queues the points it cannot prove for the exact CUDA-core path.
#include "knn_internal.h"
#include "pool.cuh"
#include <cuda_bf16.h>

namespace fl {

// Split operand planes.  An fp32 value v is carried as hi = bf16(v) and lo = bf16(v - hi); the
// plane rows hold [hi | lo | hi | ones] (samples) and [hi | hi | lo | norm terms] (centroids), so one bf16 product
// over 3 d_pad columns yields  hi.hi + lo.hi + hi.lo,  i.e. the fp32 inner product up to the
// dropped lo.lo term and the second-order residuals: a relative error of about 3 * 2^-18 of
// ||x|| ||c|| instead of 2^-8.  Used when 3 d_pad columns of a 128-row tile fit in shared
// memory (d <= 128).
__device__ __forceinline__ void bf16_split(float v, __nv_bfloat16& hi, __nv_bfloat16& lo) {
    hi = __float2bfloat16_rn(v);
    lo = __float2bfloat16_rn(v - __bfloat162float(hi));
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

// Sample side of the second stage: the points listed in `rows` (live count on the device, at most
// `cap`), one warp per row in a grid-stride loop, written as split rows [hi | lo | hi | ones].
// With `tau_out` (kNN second stage) row r also gets its starting threshold: the exact k-th distance
// d_k found so far (prev_dist [point][k]) bounds the true one from above, so every true neighbour
// scores at least (||x||^2 - d_k) / 2 exactly and at most eps = eps_rel ||x|| *maxnorm less in
// this stage; the threshold sits 2 eps and the proof's slack below that, so that a pool that never
// overflowed proves its row.
__global__ void split_x_gather_kernel(const float* __restrict__ x, int64_t ldx, int d, const int* __restrict__ rows,
                                      const int* __restrict__ rows_count, int cap, __nv_bfloat16* __restrict__ out,
                                      int d_pad, const float* __restrict__ prev_dist, int k,
                                      const float* __restrict__ maxnorm, float eps_rel, float* __restrict__ tau_out) {
    const int lane = threadIdx.x & 31;
    const int pitch = 3 * d_pad + PLANE_AUG_COLS;
    int count = *rows_count;
    count = count < cap ? count : cap;
    const int nwarps = (gridDim.x * blockDim.x) >> 5;
    if (tau_out != nullptr) {
        // rows of the last live tile beyond the list's end hold stale memory: they must never append
        const int tile_end = (count + 127) & ~127;
        for (int r = count + blockIdx.x * blockDim.x + threadIdx.x; r < tile_end; r += gridDim.x * blockDim.x) tau_out[r] = pos_inf();
    }
    for (int r = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; r < count; r += nwarps) {
        const int64_t pt = rows[r];
        const float* src = x + pt * ldx;
        __nv_bfloat16* o = out + (int64_t)r * pitch;
        float qsq = 0.f;
        for (int t = lane; t < d_pad; t += 32) {
            __nv_bfloat16 hi, lo;
            const float v = t < d ? __ldg(src + t) : 0.f;
            qsq += v * v;
            bf16_split(v, hi, lo);
            o[t] = hi;
            o[d_pad + t] = lo;
            o[2 * d_pad + t] = hi;
        }
        if (lane < PLANE_AUG_COLS) o[3 * d_pad + lane] = __float2bfloat16_rn(lane < 3 ? 1.f : 0.f);
        if (tau_out != nullptr) {
#pragma unroll
            for (int off = 16; off > 0; off >>= 1) qsq += __shfl_xor_sync(FULL_MASK, qsq, off);
            if (lane == 0) {
                const float dk = prev_dist[pt * k + (k - 1)];
                const float mn = __ldg(maxnorm);
                float tau = neg_inf();
                if (dk < pos_inf())
                    tau = 0.5f * (qsq - dk) - 2.f * eps_rel * sqrtf(qsq) * mn - 1e-5f * (qsq + mn * mn);
                tau_out[r] = tau;
            }
        }
    }
}

// Eight lanes per point, four points per warp, grid-stride.  The scoring pass left, for each half
// of the centroid columns, the best and second-best score and the best centroid of scoring row r.
// Row r is point r (first stage) or point rows[r] (second stage, live count on the device).
// Both best centroids are re-scored with exact fp32 sum (x - c)^2; the closer one wins (lower
// index on exact ties).  Every other centroid scored at most `bound` = the larger of the two
// second-best scores (plus the 2^-16 relative perturbation of carrying the column index in the
// score's low mantissa bits), so the label is proven when its exact distance is below
// ||x||^2 - 2 (bound + eps); otherwise the point goes to the `next` list (the next, more precise
// stage) or, when that is absent or full, to the exact-path list.
__global__ void __launch_bounds__(128) assign_finalize_kernel(
    const float* __restrict__ x, int64_t n, int64_t ldx, const float* __restrict__ c, int K, int64_t ldc, int d,
    int vec, const float* __restrict__ asg_sc, const uint32_t* __restrict__ asg_id, float eps_rel,
    const float* __restrict__ maxnorm, int32_t* __restrict__ labels, const int* __restrict__ rows,
    const int* __restrict__ rows_count, int* __restrict__ next_count, int* __restrict__ next_list, int next_cap,
    int* __restrict__ fb_count, int* __restrict__ fb_list, int fb_cap, int scores_by_point) {
    const int sl = threadIdx.x & 7;
    int64_t live = n;
    if (rows_count != nullptr) { const int64_t cnt = *rows_count; live = cnt < n ? cnt : n; }
    const int64_t ngroups = ((int64_t)gridDim.x * blockDim.x) >> 3;
    const int64_t rounds = (live + ngroups - 1) / ngroups;
    for (int64_t it = 0; it < rounds; ++it) {
        const int64_t r_raw = it * ngroups + (((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 3);
        const bool alive = r_raw < live;
        const int64_t r = alive ? r_raw : live - 1;          // idle groups shadow the last row
        const int64_t pt = rows != nullptr ? (int64_t)rows[r] : r;
        // the scores sit at the scoring row: the list position (points gathered for their own scoring
        // pass) or the point itself (a list of points that were scored in place)
        const int64_t sr = scores_by_point ? pt : r;
        const float4 sc = __ldg(reinterpret_cast<const float4*>(asg_sc + sr * 4));   // b1_0, b2_0, b1_1, b2_1
        const uint2 ids = __ldg(reinterpret_cast<const uint2*>(asg_id + sr * 2));
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
        if (!alive || sl != 0) continue;
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
            bool queued = false;
            if (next_count != nullptr) {
                const int i = atomicAdd(next_count, 1);
                if (i < next_cap) { next_list[i] = (int)pt; queued = true; }
            }
            if (!queued) {
                const int i = atomicAdd(fb_count, 1);
                if (i < fb_cap) fb_list[i] = (int)pt;
            }
        }
    }
}

// ||x||^2 of every sample row (one warp per row); the scoring error bound of a point needs it.
__global__ void rowsq_kernel(const float* __restrict__ x, int64_t n, int d, int64_t ld, float* __restrict__ out) {
    const int lane = threadIdx.x & 31;
    const int64_t row = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (row >= n) return;
    const float* p = x + row * ld;
    float s = 0.f;
    for (int c = lane; c < d; c += 32) { const float v = __ldg(p + c); s += v * v; }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(FULL_MASK, s, o);
    if (lane == 0) out[row] = s;
}

// First-stage proof from the scores alone, one thread per point: the best-scoring centroid is the
// nearest one if its score leads the runner-up's by more than twice the scoring error bound (every
// score is within eps of the exact <x,c> - ||c||^2/2, so the exact scores keep that order).  No
// sample row and no centroid is read -- 28 bytes per point instead of its 4 d -- at the price of a
// lead of 2 eps where the exact re-scoring of assign_finalize_kernel needs eps; what the lead does
// not decide goes to the `next` list (the second stage, whose bound is a hundred times smaller).
__global__ void __launch_bounds__(256) assign_by_lead_kernel(
    int64_t n, int K, const float* __restrict__ asg_sc, const uint32_t* __restrict__ asg_id, const float* __restrict__ xsq,
    float eps_rel, const float* __restrict__ maxnorm, int32_t* __restrict__ labels, int* __restrict__ next_count,
    int* __restrict__ next_list, int next_cap, int* __restrict__ fb_count, int* __restrict__ fb_list, int fb_cap) {
    const int64_t pt = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (pt >= n) return;
    const float4 sc = __ldg(reinterpret_cast<const float4*>(asg_sc + pt * 4));   // b1_0, b2_0, b1_1, b2_1
    const uint2 ids = __ldg(reinterpret_cast<const uint2*>(asg_id + pt * 2));
    const bool v0 = ids.x < (uint32_t)K && sc.x > -1e37f;   // false: no real centroid in that half
    const bool v1 = ids.y < (uint32_t)K && sc.z > -1e37f;
    const bool first = v0 && (!v1 || sc.x >= sc.z);
    const float best = first ? sc.x : sc.z;
    const uint32_t best_i = first ? ids.x : ids.y;
    float second = first ? sc.y : sc.w;                      // runner-up of the winner's half ...
    if (v0 && v1) second = fmaxf(second, first ? sc.z : sc.x);   // ... or the other half's best
    bool ok = v0 || v1;
    if (ok && second > -1e37f) {
        const float q2 = __ldg(xsq + pt), mn = __ldg(maxnorm);
        const float eps = eps_rel * sqrtf(q2) * mn;
        // the column index rides in the low mantissa bits of both scores: 2^-15 relative each
        const float lead = (best - fabsf(best) * 3.1e-5f) - (second + fabsf(second) * 3.1e-5f);
        ok = lead > 2.f * eps + 1e-5f * (q2 + mn * mn);
    }
    labels[pt] = ok ? (int32_t)best_i : 0;
    if (!ok) {
        bool queued = false;
        if (next_count != nullptr) {
            const int i = atomicAdd(next_count, 1);
            if (i < next_cap) { next_list[i] = (int)pt; queued = true; }
        }
        if (!queued) {
            const int i = atomicAdd(fb_count, 1);
            if (i < fb_cap) fb_list[i] = (int)pt;
        }
    }
}

struct AssignTcWs {
    int64_t n_pad; int d_pad, pitch; int fb_cap;
    int split;          // 1: a second stage with split (hi/lo) operand planes of 3 d_pad columns
    int l1_cap; int64_t l1_pad; int pitch3;
    int nsplit_fb; int64_t rows_per_split_fb; int fb_bq, fb_blocks;
    PlaneLayout cl, cl3;
    int64_t off_cplane, off_cplane3, off_xplane, off_xsq, off_xsplit, off_asg_sc, off_asg_id, off_tau, off_cnt, off_l0list, off_l1list,
        off_fblist, off_fbpart_sc, off_fbpart_id, off_fbdist, bytes;
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
    w.d_pad = (int)round_up(d, 64);
    w.pitch = w.d_pad + PLANE_AUG_COLS;
    w.pitch3 = 3 * w.d_pad + PLANE_AUG_COLS;
    w.cl = plane_layout(K, w.d_pad);
    w.cl3 = plane_layout(K, 3 * w.d_pad);     // same row count, hnorm and meta blocks; 3 d_pad feature columns
    w.fb_cap = (int)n;   // every point may take the exact path: no overflow case to report
    // second stage: room for half of the points (more unproven points than that take the exact path)
    w.l1_cap = w.split ? (int)((n + 1) / 2) : 0;
    w.l1_pad = round_up(w.l1_cap > 0 ? w.l1_cap : 1, 128);
    simt_split_plan(w.fb_cap, K, 32, d, &w.nsplit_fb, &w.rows_per_split_fb);
    // the exact pass spreads a fixed grid over the live points (simt_dyn_split): one pool per
    // (block, query slot) at most
    w.fb_bq = simt_block_queries(32);
    w.fb_blocks = (int)(ceil_div(w.fb_cap, w.fb_bq > 0 ? w.fb_bq : 1) * w.nsplit_fb);
    if (w.fb_blocks < 4 * sm_count()) w.fb_blocks = 4 * sm_count();
    const int64_t fb_pools = (int64_t)w.fb_blocks * (w.fb_bq > 0 ? w.fb_bq : 1);
    int64_t cur = 0;
    w.off_cplane = take(cur, w.cl.bytes);
    w.off_cplane3 = w.split ? take(cur, w.cl3.bytes) : -1;
    w.off_xplane = have_xplane ? -1 : take(cur, w.n_pad * w.pitch * 2);
    w.off_xsq = have_xplane ? -1 : take(cur, w.n_pad * 4);
    w.off_xsplit = w.split ? take(cur, w.l1_pad * w.pitch3 * 2) : -1;
    w.off_asg_sc = take(cur, w.n_pad * 4 * 4);
    w.off_asg_id = take(cur, w.n_pad * 2 * 4);
    w.off_tau = take(cur, w.n_pad * 4);
    w.off_cnt = take(cur, 1024);
    w.off_l0list = take(cur, (w.split ? n : 1) * 4);
    w.off_l1list = take(cur, (int64_t)(w.l1_cap > 0 ? w.l1_cap : 1) * 4);
    w.off_fblist = take(cur, (int64_t)w.fb_cap * 4);
    w.off_fbpart_sc = take(cur, fb_pools * 32 * 4);
    w.off_fbpart_id = take(cur, fb_pools * 32 * 4);
    w.off_fbdist = take(cur, n * 4);
    w.bytes = cur;
    return w;
}

int split_plane_supported(int d) { return assign_tc_split(d); }

// Split database plane [hi | hi | lo | norm terms] in the layout plane_layout(m, 3 d_pad).
int launch_split_db_plane(const float* c, int64_t m, int d, int64_t ldc, void* plane, cudaStream_t st) {
    const int d_pad = (int)round_up(d, 64);
    const PlaneLayout L = plane_layout(m, 3 * d_pad);
    char* pl = static_cast<char*>(plane);
    FL_CHECK_CUDA(cudaMemsetAsync(pl + L.off_meta, 0, 1024, st));
    const int wpb = 8;
    split_c_plane_kernel<<<(unsigned)ceil_div(L.m_pad, wpb), wpb * 32, 0, st>>>(
        c, m, d, ldc, reinterpret_cast<__nv_bfloat16*>(pl + L.off_rows), reinterpret_cast<float*>(pl + L.off_hnorm),
        reinterpret_cast<unsigned int*>(pl + L.off_meta), L.m_pad, d_pad);
    FL_CHECK_LAUNCH();
    return FL_OK;
}

int launch_split_query_gather(const float* x, int64_t ldx, int d, const int* rows, const int* rows_count, int cap,
                              void* out, int d_pad, const float* prev_dist, int k, const float* maxnorm, float eps_rel,
                              float* tau_out, cudaStream_t st) {
    split_x_gather_kernel<<<(unsigned)(8 * sm_count()), 256, 0, st>>>(x, ldx, d, rows, rows_count, cap,
                                                                     static_cast<__nv_bfloat16*>(out), d_pad, prev_dist, k,
                                                                     maxnorm, eps_rel, tau_out);
    FL_CHECK_LAUNCH();
    return FL_OK;
}

int assign_tc_supported(int64_t n, int K, int d) {
    if (n < 1 || K < 1 || d > 256) return 0;
    return 1;
}

}  // namespace fl

using namespace fl;

extern "C" int64_t fl_kmeans_xplane_bytes(int64_t n, int d) {
    if (n < 1 || d < 1) return 0;
    // the bf16 rows, then ||x||^2 of every row (f32 [n_pad])
    return round_up(round_up(n, 128) * (round_up(d, 64) + PLANE_AUG_COLS) * 2, 1024) + round_up(n, 128) * 4;
}

extern "C" int fl_kmeans_prepare_x_f32(const float* x, int64_t n, int d, int64_t ldx, void* xplane,
                                       int64_t xplane_bytes, void* stream) {
    FL_CHECK_ARG(x && xplane && n >= 1 && d >= 1 && ldx >= d, "fl_kmeans_prepare_x_f32: bad arguments");
    if (xplane_bytes < fl_kmeans_xplane_bytes(n, d)) { set_error("fl_kmeans_prepare_x_f32: plane buffer too small"); return FL_EWORKSPACE; }
    const int64_t n_pad = round_up(n, 128);
    const int rc = launch_query_plane(x, n, ldx, d, xplane, n_pad, (int)round_up(d, 64), (cudaStream_t)stream);
    if (rc != FL_OK) return rc;
    float* xsq = reinterpret_cast<float*>(static_cast<char*>(xplane) + round_up(n_pad * (round_up(d, 64) + PLANE_AUG_COLS) * 2, 1024));
    rowsq_kernel<<<(unsigned)ceil_div(n, 8), 256, 0, (cudaStream_t)stream>>>(x, n, d, ldx, xsq);
    FL_CHECK_LAUNCH();
    return FL_OK;
}

extern "C" int64_t fl_kmeans_assign_tc_workspace_bytes(int64_t n, int K, int d, int have_xplane) {
    if (!assign_tc_supported(n, K, d)) return 0;
    return assign_tc_plan(n, K, d, have_xplane).bytes;
}

// Two stages.  (1) plain bf16 planes: every point is scored against every centroid; labels the
// proof accepts (scoring error 2^-8 ||x|| max||c||) are final.  (2) d <= 128: the unproven points
// (a device-side list) are gathered into split planes and scored again, error 4e-5: nearly all of
// the rest is proven.  What is left takes the exact CUDA-core path.
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

    // centroid planes (database side): plain, and split for the second stage
    char* cpl = base + w.off_cplane;
    int rc = launch_plane_build(c, K, d, ldc, cpl, st);
    if (rc != FL_OK) return rc;
    char* cpl3 = nullptr;
    if (w.split) {
        cpl3 = base + w.off_cplane3;
        rc = launch_split_db_plane(c, K, d, ldc, cpl3, st);
        if (rc != FL_OK) return rc;
    }
    // sample plane (query side)
    const char* xpl = static_cast<const char*>(xplane);
    const float* xsq;
    if (!xpl) {
        rc = launch_query_plane(x, n, ldx, d, base + w.off_xplane, w.n_pad, w.d_pad, st);
        if (rc != FL_OK) return rc;
        xpl = base + w.off_xplane;
        float* xs = reinterpret_cast<float*>(base + w.off_xsq);
        rowsq_kernel<<<(unsigned)ceil_div(n, 8), 256, 0, st>>>(x, n, d, ldx, xs);
        FL_CHECK_LAUNCH();
        xsq = xs;
    } else {
        xsq = reinterpret_cast<const float*>(xpl + round_up(w.n_pad * w.pitch * 2, 1024));
    }
    int* counters = reinterpret_cast<int*>(base + w.off_cnt);
    int* fb_count = counters;          // points for the exact path
    int* l1_count = counters + 64;     // points for the second stage
    int* fb_list = reinterpret_cast<int*>(base + w.off_fblist);
    int* l1_list = reinterpret_cast<int*>(base + w.off_l1list);
    int* l0_count = counters + 128;    // points the scores' lead did not decide
    int* l0_list = reinterpret_cast<int*>(base + w.off_l0list);
    FL_CHECK_CUDA(cudaMemsetAsync(counters, 0, 1024, st));
    const int vecx = (ldx % 4 == 0) && ((reinterpret_cast<uintptr_t>(x) & 15) == 0);
    const int vecc = (ldc % 4 == 0) && ((reinterpret_cast<uintptr_t>(c) & 15) == 0);
    const int vec = vecx && vecc && (d % 4 == 0);
    float* tau = reinterpret_cast<float*>(base + w.off_tau);
    float* asg_sc = reinterpret_cast<float*>(base + w.off_asg_sc);
    uint32_t* asg_id = reinterpret_cast<uint32_t*>(base + w.off_asg_id);
    const unsigned fin_grid = (unsigned)(4 * sm_count());      // grid-stride finalisation
    const float* maxnorm = reinterpret_cast<const float*>(cpl + w.cl.off_meta);

    // ---- stage 1: plain bf16 ---------------------------------------------------------------
    {
        rc = launch_fill_f32(tau, w.n_pad, -INFINITY, st);
        if (rc != FL_OK) return rc;
        TcKnnParams tp{};
        tp.qplane = xpl; tp.nq = n; tp.nq_pad = w.n_pad;
        tp.dbrows = cpl + w.cl.off_rows; tp.hnorm = reinterpret_cast<const float*>(cpl + w.cl.off_hnorm);
        tp.m = K; tp.m_pad = w.cl.m_pad; tp.d_pad = w.cl.d_pad;
        tp.tau = tau; tp.status = status;
        profile_begin(st);
        rc = launch_assign_tc(tp, asg_sc, asg_id, nullptr, st);
        profile_end(st);
        if (rc != FL_OK) return rc;
        // scoring error relative to ||x|| max||c||: 2^-8 for plain bf16 operands, rounded up
        if (w.split) {
            // a second, far more precise stage follows: decide what the scores' lead decides
            // without touching the rows
            assign_by_lead_kernel<<<(unsigned)ceil_div(n, 256), 256, 0, st>>>(
                n, K, asg_sc, asg_id, xsq, 0.004f, maxnorm, labels, l0_count, l0_list, (int)n, fb_count, fb_list, w.fb_cap);
            FL_CHECK_LAUNCH();
            // ... then, for the undecided ones only, the exact distances to the two half-winners, which
            // need half the lead; what is still open goes to the second stage
            assign_finalize_kernel<<<fin_grid, 128, 0, st>>>(
                x, n, ldx, c, K, ldc, d, vec, asg_sc, asg_id, 0.004f, maxnorm, labels, l0_list, l0_count,
                l1_count, l1_list, w.l1_cap, fb_count, fb_list, w.fb_cap, 1);
        } else {
            assign_finalize_kernel<<<fin_grid, 128, 0, st>>>(
                x, n, ldx, c, K, ldc, d, vec, asg_sc, asg_id, 0.004f, maxnorm, labels, nullptr, nullptr,
                nullptr, l1_list, w.l1_cap, fb_count, fb_list, w.fb_cap, 0);
        }
        FL_CHECK_LAUNCH();
    }
    // ---- stage 2: split planes for the unproven points --------------------------------------
    if (w.split) {
        __nv_bfloat16* xs = reinterpret_cast<__nv_bfloat16*>(base + w.off_xsplit);
        split_x_gather_kernel<<<(unsigned)(8 * sm_count()), 256, 0, st>>>(x, ldx, d, l1_list, l1_count, w.l1_cap, xs, w.d_pad,
                                                                         nullptr, 0, nullptr, 0.f, nullptr);
        FL_CHECK_LAUNCH();
        TcKnnParams tp{};
        tp.qplane = xs; tp.nq = w.l1_cap; tp.nq_pad = w.l1_pad;
        tp.dbrows = cpl3 + w.cl3.off_rows; tp.hnorm = reinterpret_cast<const float*>(cpl3 + w.cl3.off_hnorm);
        tp.m = K; tp.m_pad = w.cl3.m_pad; tp.d_pad = w.cl3.d_pad;
        tp.tau = tau; tp.status = status;
        rc = launch_assign_tc(tp, asg_sc, asg_id, l1_count, st);
        if (rc != FL_OK) return rc;
        // split operands: 3 * 2^-18 from the dropped terms plus the fp32 accumulation of 400 products
        assign_finalize_kernel<<<fin_grid, 128, 0, st>>>(
            x, w.l1_cap, ldx, c, K, ldc, d, vec, asg_sc, asg_id, 4e-5f, maxnorm, labels, l1_list, l1_count,
            nullptr, nullptr, 0, fb_count, fb_list, w.fb_cap, 0);
        FL_CHECK_LAUNCH();
    }
    rc = launch_fallback_fixup(fb_count, w.fb_cap, status, tc_pool_size(1), st);
    if (rc != FL_OK) return rc;

    // points whose label could not be proven: exact CUDA-core scoring + exact re-rank, k = 1
    SimtKnnParams sp{};
    sp.q = x; sp.ldq = ldx; sp.qlist = fb_list; sp.count_dev = fb_count; sp.count = 0;
    sp.db = c; sp.m = K; sp.ldb = ldc; sp.d = d;
    sp.hnorm = reinterpret_cast<const float*>(cpl + w.cl.off_hnorm);
    sp.K1 = 32; sp.cap = simt_pool_cap(32); sp.npl = sp.cap / 32; sp.keep = simt_pool_keep(32, 1);
    sp.nsplit = w.nsplit_fb; sp.rows_per_split = w.rows_per_split_fb;
    sp.dyn_blocks = w.fb_blocks; sp.dyn_bq = w.fb_bq;
    sp.part_sc = reinterpret_cast<float*>(base + w.off_fbpart_sc);
    sp.part_id = reinterpret_cast<uint32_t*>(base + w.off_fbpart_id);
    sp.vecq = vecx; sp.vecd = vecc;
    rc = launch_knn_simt(sp, w.fb_cap, st);
    if (rc != FL_OK) return rc;
    FinalizeParams fp{};
    fp.q = x; fp.ldq = ldx; fp.qlist = fb_list; fp.count_dev = fb_count; fp.count = 0;
    fp.db = c; fp.m = K; fp.ldb = ldc; fp.d = d; fp.vec = vec;
    fp.part_sc = sp.part_sc; fp.part_id = sp.part_id; fp.nsplit = w.nsplit_fb; fp.K1 = 32;
    fp.dyn_blocks = w.fb_blocks; fp.dyn_bq = w.fb_bq;
    fp.k = 1; fp.rerank = 9; fp.row_offset = 0;
    fp.out_dist = reinterpret_cast<float*>(base + w.off_fbdist); fp.out_idx = labels; fp.verify = 0;
    return launch_knn_finalize(fp, w.fb_cap, st);
}
