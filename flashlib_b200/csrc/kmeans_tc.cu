// Tensor-core k-means assignment: the sample rows play the queries and the centroids the
// database of the kNN candidate kernel (knn_tc.cu); a lean per-point kernel then re-scores
// the few best candidates exactly, proves the winner against the scoring error bound and
// queues the points it cannot prove for the exact CUDA-core path.
#include "knn_internal.h"
#include "pool.cuh"
#include <cuda_bf16.h>

namespace fl {

constexpr int ASSIGN_RERANK = 8;     // candidates re-scored exactly per point
constexpr int64_t ASSIGN_CHUNK = 262144;   // points per tensor-core launch (bounds the workspace)

// One warp per point.  `plen` published (score, centroid) entries per point (2 per lane for
// plen = 64); the ASSIGN_RERANK best scores are re-scored with exact fp32 sum (x - c)^2, the
// closest wins (lowest index on exact ties).  Every centroid that was not re-scored scored at
// most `bound` = max(published thresholds, best score not re-scored); the label is proven when
// its exact distance is below ||x||^2 - 2 (bound + eps).
__global__ void __launch_bounds__(128) assign_finalize_kernel(
    const float* __restrict__ x, int64_t n, int64_t ldx, const float* __restrict__ c, int K, int64_t ldc, int d,
    int vec, const float* __restrict__ part_sc, const uint32_t* __restrict__ part_id, int plen,
    const float* __restrict__ part_tau, int ntau, float eps_rel, const float* __restrict__ maxnorm,
    int32_t* __restrict__ labels, int* __restrict__ fb_count, int* __restrict__ fb_list, int fb_cap,
    int64_t point0) {
    const int lane = threadIdx.x & 31;
    const int64_t slot = (int64_t)blockIdx.x * 4 + (threadIdx.x >> 5);
    if (slot >= n) return;
    const int64_t pt = point0 + slot;
    float s0 = neg_inf(), s1 = neg_inf();
    uint32_t i0 = INVALID_ID, i1 = INVALID_ID;
    {
        const float* ps = part_sc + slot * plen;
        const uint32_t* pi = part_id + slot * plen;
        if (lane < plen) { i0 = pi[lane]; s0 = ps[lane]; }
        if (lane + 32 < plen) { i1 = pi[lane + 32]; s1 = ps[lane + 32]; }
        if (i0 >= (uint32_t)K) { i0 = INVALID_ID; s0 = neg_inf(); }
        if (i1 >= (uint32_t)K) { i1 = INVALID_ID; s1 = neg_inf(); }
    }
    float u = neg_inf();
    for (int i = lane; i < ntau; i += 32) u = fmaxf(u, part_tau[slot * ntau + i]);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) u = fmaxf(u, __shfl_xor_sync(FULL_MASK, u, o));

    const float* xp = x + pt * ldx;
    float qsq = 0.f;
    if (vec) {
        for (int t = lane * 4; t < d; t += 128) {
            const float4 v = __ldg(reinterpret_cast<const float4*>(xp + t));
            qsq += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
        }
    } else {
        for (int t = lane; t < d; t += 32) { const float v = __ldg(xp + t); qsq += v * v; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) qsq += __shfl_xor_sync(FULL_MASK, qsq, o);

    float best_d = pos_inf();
    uint32_t best_i = INVALID_ID;
#pragma unroll 1
    for (int r = 0; r < ASSIGN_RERANK; ++r) {
        float m = fmaxf(s0, s1);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(FULL_MASK, m, o));
        if (!(m > neg_inf())) break;                       // no candidate left (warp uniform)
        const unsigned who = __ballot_sync(FULL_MASK, s0 == m || s1 == m);
        const int src = __ffs(who) - 1;
        uint32_t cid = INVALID_ID;
        if (lane == src) {
            if (s0 == m) { cid = i0; s0 = neg_inf(); } else { cid = i1; s1 = neg_inf(); }
        }
        cid = __shfl_sync(FULL_MASK, cid, src);
        const float* cp = c + (int64_t)cid * ldc;
        float a = 0.f;
        if (vec) {
            for (int t = lane * 4; t < d; t += 128) {
                const float4 xv = __ldg(reinterpret_cast<const float4*>(xp + t));
                const float4 cv = __ldg(reinterpret_cast<const float4*>(cp + t));
                const float d0 = xv.x - cv.x, d1 = xv.y - cv.y, d2 = xv.z - cv.z, d3 = xv.w - cv.w;
                a += d0 * d0 + d1 * d1 + d2 * d2 + d3 * d3;
            }
        } else {
            for (int t = lane; t < d; t += 32) { const float df = __ldg(xp + t) - __ldg(cp + t); a += df * df; }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) a += __shfl_xor_sync(FULL_MASK, a, o);
        if (a < best_d || (a == best_d && cid < best_i)) { best_d = a; best_i = cid; }
    }
    float rest = fmaxf(s0, s1);   // best score that was not re-scored
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) rest = fmaxf(rest, __shfl_xor_sync(FULL_MASK, rest, o));
    const float bound = fmaxf(u, rest);
    bool ok = best_i != INVALID_ID;
    if (ok && bound > neg_inf()) {
        const float mn = __ldg(maxnorm);
        const float eps = eps_rel * sqrtf(qsq) * mn;
        const float lb = qsq - 2.f * (bound + eps);
        const float slack = 1e-5f * (qsq + mn * mn);
        ok = best_d < lb - slack;
    }
    if (lane == 0) {
        labels[pt] = ok ? (int32_t)best_i : 0;
        if (!ok) {
            const int i = atomicAdd(fb_count, 1);
            if (i < fb_cap) fb_list[i] = (int)pt;
        }
    }
}

struct AssignTcWs {
    int64_t chunk, n_pad_chunk; int d_pad, pitch, nsplit; int64_t tiles_per_split; int fb_cap;
    int nsplit_fb; int64_t rows_per_split_fb;
    PlaneLayout cl;
    int64_t off_cplane, off_xplane, off_part_sc, off_part_id, off_part_tau, off_tau, off_cnt, off_fblist,
        off_fbpart_sc, off_fbpart_id, off_fbdist, bytes;
};

static int64_t take(int64_t& cur, int64_t bytes) {
    const int64_t o = cur;
    cur += round_up(bytes > 0 ? bytes : 1, 1024);
    return o;
}

static AssignTcWs assign_tc_plan(int64_t n, int K, int d, int have_xplane) {
    AssignTcWs w{};
    w.chunk = n < ASSIGN_CHUNK ? n : ASSIGN_CHUNK;
    w.n_pad_chunk = round_up(w.chunk, 128);
    w.d_pad = (int)round_up(d, 64);
    w.pitch = w.d_pad + PLANE_AUG_COLS;
    w.cl = plane_layout(K, d);
    // one range per point tile: the per-point kernel reads a single published pool
    w.nsplit = 1;
    w.tiles_per_split = w.cl.m_pad / 256;
    w.fb_cap = (int)n;   // every point may take the exact path: no overflow case to report
    simt_split_plan(w.fb_cap, K, 32, d, &w.nsplit_fb, &w.rows_per_split_fb);
    int64_t cur = 0;
    w.off_cplane = take(cur, w.cl.bytes);
    w.off_xplane = have_xplane ? -1 : take(cur, round_up(n, 128) * w.pitch * 2);
    const int plen = tc_partial_len(1);
    w.off_part_sc = take(cur, w.n_pad_chunk * w.nsplit * plen * 4);
    w.off_part_id = take(cur, w.n_pad_chunk * w.nsplit * plen * 4);
    w.off_part_tau = take(cur, w.n_pad_chunk * w.nsplit * tc_taus_per_range() * 4);
    w.off_tau = take(cur, w.n_pad_chunk * 4);
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
    return round_up(n, 128) * (round_up(d, 64) + PLANE_AUG_COLS) * 2;
}

extern "C" int fl_kmeans_prepare_x_f32(const float* x, int64_t n, int d, int64_t ldx, void* xplane,
                                       int64_t xplane_bytes, void* stream) {
    FL_CHECK_ARG(x && xplane && n >= 1 && d >= 1 && ldx >= d, "fl_kmeans_prepare_x_f32: bad arguments");
    if (xplane_bytes < fl_kmeans_xplane_bytes(n, d)) { set_error("fl_kmeans_prepare_x_f32: plane buffer too small"); return FL_EWORKSPACE; }
    return launch_query_plane(x, n, ldx, d, xplane, round_up(n, 128), (int)round_up(d, 64), (cudaStream_t)stream);
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
        const int rc = launch_plane_build(c, K, d, ldc, cpl, st);
        if (rc != FL_OK) return rc;
    }
    // sample plane (query side)
    const char* xpl = static_cast<const char*>(xplane);
    if (!xpl) {
        int rc = launch_query_plane(x, n, ldx, d, base + w.off_xplane, round_up(n, 128), w.d_pad, st);
        if (rc != FL_OK) return rc;
        xpl = base + w.off_xplane;
    }
    int* fb_count = reinterpret_cast<int*>(base + w.off_cnt);
    int* fb_list = reinterpret_cast<int*>(base + w.off_fblist);
    FL_CHECK_CUDA(cudaMemsetAsync(fb_count, 0, 1024, st));
    const int vecx = (ldx % 4 == 0) && ((reinterpret_cast<uintptr_t>(x) & 15) == 0);
    const int vecc = (ldc % 4 == 0) && ((reinterpret_cast<uintptr_t>(c) & 15) == 0);
    const int vec = vecx && vecc && (d % 4 == 0);
    const int plen = tc_partial_len(1);

    for (int64_t p0 = 0; p0 < n; p0 += w.chunk) {
        const int64_t cn = (n - p0 < w.chunk) ? n - p0 : w.chunk;
        const int64_t cn_pad = round_up(cn, 128);
        float* tau = reinterpret_cast<float*>(base + w.off_tau);
        {
            const int rc = launch_fill_f32(tau, cn_pad, -INFINITY, st);
            if (rc != FL_OK) return rc;
        }
        TcKnnParams tp{};
        tp.qplane = xpl + p0 * w.pitch * 2; tp.nq = cn; tp.nq_pad = cn_pad;
        tp.dbrows = cpl + w.cl.off_rows; tp.hnorm = reinterpret_cast<const float*>(cpl + w.cl.off_hnorm);
        tp.m = K; tp.m_pad = w.cl.m_pad; tp.d_pad = w.cl.d_pad; tp.K1 = tc_pool_size(1);
        tp.nsplit = w.nsplit; tp.tiles_per_split = w.tiles_per_split;
        tp.part_sc = reinterpret_cast<float*>(base + w.off_part_sc);
        tp.part_id = reinterpret_cast<uint32_t*>(base + w.off_part_id);
        tp.part_tau = reinterpret_cast<float*>(base + w.off_part_tau);
        tp.tau = tau; tp.status = status;
        profile_begin(st);
        int rc = launch_knn_tc(tp, st);
        profile_end(st);
        if (rc != FL_OK) return rc;
        assign_finalize_kernel<<<(unsigned)ceil_div(cn, 4), 128, 0, st>>>(
            x, cn, ldx, c, K, ldc, d, vec, tp.part_sc, tp.part_id, plen * w.nsplit, tp.part_tau,
            w.nsplit * tc_taus_per_range(), 0.004f, reinterpret_cast<const float*>(cpl + w.cl.off_meta), labels,
            fb_count, fb_list, w.fb_cap, p0);
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
    sp.K1 = 32; sp.cap = 64; sp.npl = 2; sp.nsplit = w.nsplit_fb; sp.rows_per_split = w.rows_per_split_fb;
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
