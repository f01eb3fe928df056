// Host orchestration of fl_knn_f32 plus the small helper kernels around it (half norms,
// bf16 query plane, fallback bookkeeping), the shard merge and the exact gather.
#include "knn_internal.h"
#include "pool.cuh"
#include <cuda_bf16.h>

namespace fl {

// out[i] = ||x_i||^2 / 2
// ||x||^2 / 2 per row and (maxnorm_bits, zero-initialised) the largest row norm.
// (blockIdx.y: problem of a batch, rows bstride elements further, norms n further.)
__global__ void halfnorm_kernel(const void* __restrict__ x, int64_t n, int d, int64_t ld,
                                float* __restrict__ out, unsigned int* __restrict__ maxnorm_bits, int dt,
                                int64_t bstride = 0) {
    const int lane = threadIdx.x & 31;
    const int64_t row = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (row >= n) return;
    x = static_cast<const char*>(x) + (int64_t)blockIdx.y * bstride * dt_size_dev(dt);
    out += (int64_t)blockIdx.y * n;
    const void* p = row_at(x, row, ld, dt);
    float s = 0.f;
    for (int c = lane; c < d; c += 32) { const float v = ld_elem(p, c, dt); s += v * v; }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(FULL_MASK, s, o);
    if (lane == 0) {
        out[row] = 0.5f * s;
        atomicMax(maxnorm_bits, __float_as_uint(sqrtf(s)));    // norms are >= 0: their bit patterns order like the values
    }
}

// Relative bound (of ||q|| max||x||) on the error of an fp32 score <q,x> - ||x||^2/2 accumulated on
// the CUDA cores: the exact re-rank walks past the k + 8 best scores while rows that close could
// still change the answer.
constexpr float SIMT_EPS_REL = 4e-6f;

// bf16 query plane [nq_pad][d_pad + 16]: the features, zero padding, and ones in the three
// columns that meet the database plane's split -||x||^2/2 terms.
__global__ void query_plane_kernel(const void* __restrict__ q, int64_t nq, int64_t ldq, int d,
                                   __nv_bfloat16* __restrict__ out, int64_t nq_pad, int d_pad, int dt) {
    const int pitch = d_pad + PLANE_AUG_COLS;
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const int64_t total = nq_pad * pitch;
    if (i >= total) return;
    const int64_t r = i / pitch;
    const int c = (int)(i - r * pitch);
    float v = 0.f;
    if (r < nq) {
        if (c < d) v = ld_elem(row_at(q, r, ldq, dt), c, dt);
        else if (c >= d_pad && c < d_pad + 3) v = 1.f;
    }
    out[i] = __float2bfloat16_rn(v);
}

int launch_query_plane(const void* q, int64_t nq, int64_t ldq, int d, void* qplane, int64_t nq_pad,
                       int d_pad, cudaStream_t st, int dt) {
    const int64_t total = nq_pad * (d_pad + PLANE_AUG_COLS);
    query_plane_kernel<<<(unsigned)ceil_div(total, 256), 256, 0, st>>>(
        q, nq, ldq, d, reinterpret_cast<__nv_bfloat16*>(qplane), nq_pad, d_pad, dt);
    FL_CHECK_LAUNCH();
    return FL_OK;
}

__global__ void fill_f32_kernel(float* p, int64_t n, float v) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) p[i] = v;
}

// Clamps the fallback count to the list capacity and publishes it (and the number of rows the
// split-plane stage took) in the status words.
__global__ void fallback_fixup_kernel(int* fb_count, int fb_cap, int32_t* status, int K1, const int* s2_count = nullptr,
                                      int s2_cap = 0) {
    int c = *fb_count;
    if (status && s2_count) { const int c2 = *s2_count; status[FL_STATUS_STAGE2] = c2 < s2_cap ? c2 : s2_cap; }
    if (status) {
        status[FL_STATUS_FALLBACK] = c;
        status[FL_STATUS_POOL] = K1;
        if (c > fb_cap && status[FL_STATUS_ERROR] == 0) status[FL_STATUS_ERROR] = FL_EWORKSPACE;
    }
    if (c > fb_cap) *fb_count = fb_cap;
}

int launch_fill_f32(float* p, int64_t n, float v, cudaStream_t st) {
    fill_f32_kernel<<<(unsigned)ceil_div(n, 256), 256, 0, st>>>(p, n, v);
    FL_CHECK_LAUNCH();
    return FL_OK;
}
int launch_fallback_fixup(int* fb_count, int fb_cap, int32_t* status, int K1, cudaStream_t st) {
    fallback_fixup_kernel<<<1, 1, 0, st>>>(fb_count, fb_cap, status, K1);
    FL_CHECK_LAUNCH();
    return FL_OK;
}

// ---- workspace layout -----------------------------------------------------------------
struct KnnWs {
    int mode, K1, K1f;
    int kg;                                    // k that selects the tensor-core pool geometry (see knn_geometry_k)
    int deep, plen;                            // tensor-core path: deep pools, published entries per (query, range)
    int nsplit; int64_t rows_per_split;        // main pass (SIMT: rows; TC: tiles of 256)
    int nsplit_fb; int64_t rows_per_split_fb;  // fallback pass
    int64_t nq_pad; int d_pad; int fb_cap; int fb_bq, fb_blocks;
    int64_t off_hnorm, off_qplane, off_part_sc, off_part_id, off_part_tau, off_part_cnt, off_seed_cls, off_tau, off_cert, off_cnt, off_fblist,
        off_fbpart_sc, off_fbpart_id, bytes;
    // second stage (split hi/lo planes) for the rows the first proof rejects
    int s2;                                    // 1: planned
    int s2_cap; int64_t s2_pad;                // rows the stage takes (the rest go to the exact path), padded to tiles
    int s2_nsplit; int64_t s2_tiles_per_split; int s2_plen;
    int64_t off_s2_list, off_s2_qplane, off_s2_tau, off_s2_part_sc, off_s2_part_id, off_s2_part_tau, off_s2_part_cnt;
};

static int64_t take(int64_t& cur, int64_t bytes) {
    const int64_t o = cur;
    cur += round_up(bytes > 0 ? bytes : 1, 1024);
    return o;
}

// Rows the split-plane stage takes: every query up to 65 536 (near-duplicate data can fail the bf16
// proof for all of them), a quarter of the queries beyond that, at most 262 144 (1 GB of pools).
static int knn_stage2_rows(int64_t nq) {
    if (nq <= 65536) return (int)nq;
    int64_t c = nq / 4;
    if (c < 65536) c = 65536;
    if (c > 262144) c = 262144;
    return (int)c;
}

// More than 256 features: the resident query tile (up to 132 KB at d = 512) leaves no room for pools
// in shared memory, so small k takes the large-k geometry too (pools in global memory, block-per-
// query finalisation, the seeding rule of k = 17).
static int knn_geometry_k(int d, int k) { return (d > 256 && k < 17) ? 17 : k; }

static KnnWs knn_ws_plan(int64_t nq, int64_t m, int d, int k, int mode, int staged = 0) {
    KnnWs w{};
    w.mode = mode;
    w.kg = k;
    int64_t cur = 0;
    if (mode == FL_KNN_BF16_RERANK) {
        const int k_real = k;
        k = knn_geometry_k(d, k);
        w.kg = k;
        w.K1 = tc_pool_size(k);
        w.K1f = simt_pool_size(k_real);
        w.nq_pad = tc_query_rows_padded(nq);
        w.d_pad = (int)round_up(d, 64);
        const int64_t m_pad = round_up(m, 256);
        tc_split_plan(w.nq_pad, m_pad, k, &w.nsplit, &w.rows_per_split);
        // Every query may fail its proof (near-duplicate or offset data): the list holds them all, so
        // no row is ever returned unproven.  The exact pass sizes its partial storage by blocks, not
        // by rows x ranges (simt_dyn_split), so the cost of the full list is nq pools of K1f entries.
        w.fb_cap = (int)nq;
        // range split of a non-dynamic fallback pass (kept for the plan's completeness; the
        // dynamic split below is what runs): at least 4 tiles per split
        int64_t s = (int64_t)(128ll << 20) / ((int64_t)w.fb_cap * w.K1f * 8);
        const int64_t tiles = ceil_div(m, 128);
        if (s > tiles / 4) s = tiles / 4;
        if (s > 128) s = 128;
        if (s < 1) s = 1;
        w.rows_per_split_fb = round_up(ceil_div(m, s), 128);
        w.nsplit_fb = (int)ceil_div(m, w.rows_per_split_fb);
        w.off_hnorm = -1;
        w.off_qplane = take(cur, w.nq_pad * (w.d_pad + PLANE_AUG_COLS) * 2);
        w.deep = tc_use_deep_pools(k, w.d_pad, w.nsplit, w.nq_pad);
        w.plen = w.deep ? tc_deep_partial_len() : tc_partial_len(k);
        if (w.deep) w.K1 = tc_deep_pool_size();
        w.off_part_sc = take(cur, w.nq_pad * w.nsplit * (int64_t)w.plen * 4);
        w.off_part_id = take(cur, w.nq_pad * w.nsplit * (int64_t)w.plen * 4);
        w.off_part_tau = take(cur, w.nq_pad * w.nsplit * tc_taus_per_range() * 4);
        w.off_part_cnt = take(cur, w.nq_pad * w.nsplit * tc_taus_per_range() * 4);
        w.off_seed_cls = take(cur, w.nq_pad * 32 * 4);
        w.off_tau = take(cur, w.nq_pad * 4);
        w.off_cert = take(cur, w.nq_pad * 4);
        w.off_cnt = take(cur, 1024);
        w.off_fblist = take(cur, (int64_t)w.fb_cap * 4);
        // the fallback scan spreads its blocks over the live slots (simt_dyn_split): at most
        // one pool per block
        w.fb_bq = simt_block_queries(w.K1f);
        // four blocks per SM either way: enough ranges for a handful of rows, no long tail of
        // blocks that only find out they have nothing to do
        w.fb_blocks = 4 * sm_count();
        if (w.fb_blocks < ceil_div(w.fb_cap, w.fb_bq > 0 ? w.fb_bq : 1)) w.fb_blocks = (int)ceil_div(w.fb_cap, w.fb_bq > 0 ? w.fb_bq : 1);
        const int64_t fb_pools = (int64_t)w.fb_blocks * (w.fb_bq > 0 ? w.fb_bq : 1);
        w.off_fbpart_sc = take(cur, fb_pools * w.K1f * 4);
        w.off_fbpart_id = take(cur, fb_pools * w.K1f * 4);
        if (staged && split_plane_supported(d)) {
            w.s2 = 1;
            w.s2_cap = knn_stage2_rows(nq);
            w.s2_pad = round_up(w.s2_cap, 128);
            w.s2_plen = tc_partial_len(17);            // the large global-memory pools
            // Ranges: the live row count is only known on the device and is usually a small part of
            // the capacity, so plan for an eighth of it (more ranges keep the SMs busy when few query
            // tiles are live), within 256 MB of pools.
            int64_t plan_rows = round_up(ceil_div(w.s2_cap, 8), 128);
            tc_split_plan(plan_rows, m_pad, 17, &w.s2_nsplit, &w.s2_tiles_per_split);
            const int64_t n_tiles = m_pad / 256;
            while (w.s2_nsplit > 1 && w.s2_pad * w.s2_nsplit * (int64_t)w.s2_plen * 8 > (256ll << 20)) {
                w.s2_tiles_per_split = ceil_div(n_tiles, w.s2_nsplit - 1);
                w.s2_nsplit = (int)ceil_div(n_tiles, w.s2_tiles_per_split);
            }
            w.off_s2_list = take(cur, (int64_t)w.s2_cap * 4);
            w.off_s2_qplane = take(cur, w.s2_pad * (3 * w.d_pad + PLANE_AUG_COLS) * 2);
            w.off_s2_tau = take(cur, w.s2_pad * 4);
            w.off_s2_part_sc = take(cur, w.s2_pad * w.s2_nsplit * (int64_t)w.s2_plen * 4);
            w.off_s2_part_id = take(cur, w.s2_pad * w.s2_nsplit * (int64_t)w.s2_plen * 4);
            w.off_s2_part_tau = take(cur, w.s2_pad * w.s2_nsplit * tc_taus_per_range() * 4);
            w.off_s2_part_cnt = take(cur, w.s2_pad * w.s2_nsplit * tc_taus_per_range() * 4);
        }
    } else {
        w.K1 = simt_pool_size(k);
        w.K1f = w.K1;
        simt_split_plan(nq, m, w.K1, d, &w.nsplit, &w.rows_per_split);
        w.off_hnorm = take(cur, m * 4);
        w.off_part_sc = take(cur, nq * w.nsplit * (int64_t)w.K1 * 4);
        w.off_part_id = take(cur, nq * w.nsplit * (int64_t)w.K1 * 4);
        w.off_cnt = take(cur, 1024);
    }
    w.bytes = cur;
    return w;
}


static int resolve_mode(int64_t nq, int64_t m, int d, int k, int mode) {
    if (mode == FL_KNN_AUTO) return tc_knn_auto(nq, m, d, k) ? FL_KNN_BF16_RERANK : FL_KNN_EXACT_SIMT;
    return mode;
}

// ---- shard merge ------------------------------------------------------------------------
// One warp per row: streams the candidates in chunks of 32, keeps the k best (dist, idx).
template <int NPL1>
__global__ void __launch_bounds__(128) topk_merge_kernel(const float* __restrict__ cd,
                                                         const int32_t* __restrict__ ci, int64_t nq,
                                                         int ncand, int k, float* __restrict__ od,
                                                         int32_t* __restrict__ oi) {
    const int lane = threadIdx.x & 31;
    const int64_t row = (int64_t)blockIdx.x * 4 + (threadIdx.x >> 5);
    if (row >= nq) return;
    constexpr int N2 = 2 * NPL1;
    float key[N2];
    uint32_t id[N2];
#pragma unroll
    for (int r = 0; r < NPL1; ++r) { key[r] = neg_inf(); id[r] = INVALID_ID; }
    const float* d = cd + row * ncand;
    const int32_t* ix = ci + row * ncand;
    for (int base = 0; base < ncand; base += NPL1 * 32) {
#pragma unroll
        for (int r = 0; r < NPL1; ++r) {
            const int e = base + ((r << 5) | lane);
            const bool ok = e < ncand && ix[e] >= 0;
            key[NPL1 + r] = ok ? -d[e] : neg_inf();
            id[NPL1 + r] = ok ? (uint32_t)ix[e] : INVALID_ID;
        }
        warp_sort_desc<N2, true>(key, id);
    }
#pragma unroll
    for (int r = 0; r < NPL1; ++r) {
        const int e = (r << 5) | lane;
        if (e < k) {
            const bool ok = id[r] != INVALID_ID;
            od[row * k + e] = ok ? -key[r] : pos_inf();
            oi[row * k + e] = ok ? (int32_t)id[r] : -1;
        }
    }
}

// ---- exact gather ---------------------------------------------------------------------
template <typename IdxT>
__global__ void gather_l2sq_kernel(const float* __restrict__ x, int64_t n, int64_t ldx,
                                   const float* __restrict__ c, int64_t m, int64_t ldc, int d,
                                   const IdxT* __restrict__ idx, int k, float* __restrict__ out) {
    const int lane = threadIdx.x & 31;
    const int64_t pair = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (pair >= n * k) return;
    const int64_t i = pair / k;
    const int64_t j = (int64_t)idx[pair];
    if (j < 0 || j >= m) {
        if (lane == 0) out[pair] = pos_inf();
        return;
    }
    const float* xp = x + i * ldx;
    const float* cp = c + j * ldc;
    float s = 0.f;
    for (int t = lane; t < d; t += 32) { const float df = __ldg(xp + t) - __ldg(cp + t); s += df * df; }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(FULL_MASK, s, o);
    if (lane == 0) out[pair] = s;
}

}  // namespace fl

using namespace fl;

extern "C" int fl_knn_resolve_mode(int64_t nq, int64_t m, int d, int k) {
    return resolve_mode(nq, m, d, k, FL_KNN_AUTO);
}

extern "C" int64_t fl_knn_workspace_bytes(int64_t nq, int64_t m, int d, int k, int mode) {
    if (nq < 1 || m < 1 || d < 1 || k < 1) return 0;
    mode = resolve_mode(nq, m, d, k, mode);
    return knn_ws_plan(nq, m, d, k, mode).bytes;
}

// Argument checks shared by the kNN entry points; resolves FL_KNN_AUTO.
static int knn_check_args(const char* who, const void* q, int64_t nq, int64_t ldq, const void* db, int64_t m,
                          int64_t ldb, int d, int k, int* mode, const void* plane, int64_t row_offset,
                          const float* out_dist, const int32_t* out_idx, const void* ws) {
    FL_CHECK_ARG(nq >= 0 && m >= 1 && d >= 1, "%s: bad shape nq=%lld m=%lld d=%d", who, (long long)nq, (long long)m, d);
    FL_CHECK_ARG(k >= 1 && k <= m, "%s: k must be in [1, m=%lld] (got %d)", who, (long long)m, k);
    FL_CHECK_ARG(ldq >= d && ldb >= d, "%s: leading dimensions smaller than d", who);
    FL_CHECK_ARG(m < (1ll << 31) && nq < (1ll << 31), "%s: more than 2^31 rows", who);
    FL_CHECK_ARG(row_offset >= 0 && row_offset + m <= (1ll << 31), "%s: row_offset + m exceeds int32 index range", who);
    if (k > 512) {
        set_error("%s: k=%d > 512 is not supported", who, k);
        return FL_EUNSUPPORTED;
    }
    if (nq == 0) return FL_OK;
    FL_CHECK_ARG(q && db && out_dist && out_idx && ws, "%s: null pointer", who);
    FL_CHECK_ARG((reinterpret_cast<uintptr_t>(ws) & 255) == 0, "%s: workspace must be 256-byte aligned", who);
    if (*mode == FL_KNN_BF16_RERANK && tc_knn_supported(nq, m, d, k) != FL_OK) {
        set_error("%s: shape (nq=%lld m=%lld d=%d k=%d) outside the tensor-core kernel's range", who,
                  (long long)nq, (long long)m, d, k);
        return FL_EUNSUPPORTED;
    }
    *mode = resolve_mode(nq, m, d, k, *mode);
    if (*mode == FL_KNN_BF16_RERANK) {
        FL_CHECK_ARG(plane != nullptr, "%s: the tensor-core mode needs the plane built by fl_knn_prepare_db_f32", who);
        FL_CHECK_ARG((reinterpret_cast<uintptr_t>(plane) & 255) == 0, "%s: plane must be 256-byte aligned", who);
    }
    FL_CHECK_ARG(*mode == FL_KNN_EXACT_SIMT || *mode == FL_KNN_BF16_RERANK, "%s: unknown mode %d", who, *mode);
    return FL_OK;
}

// The tensor-core path in three phases, so that a row-sharded caller can exchange the seeding
// results between the first and the second:
//   TC_PREP    status / counters cleared, thresholds -inf, bf16 query plane built in the workspace
//   TC_SEED    class maxima of the seeding sample into `seed_cls`
//   TC_SCORE   thresholds from `seed_cls` (lowered by the cross-shard margin when `gmaxnorm` is
//              given), scoring pass, finalisation, exact pass for what could not be proven
enum { TC_PREP = 1, TC_SEED = 2, TC_SCORE = 4 };

static int knn_tc_phases(int phases, const void* q, int64_t nq, int64_t ldq, const void* db, int64_t m, int64_t ldb,
                         int d, int k, const void* plane, int64_t row_offset, float* seed_cls, const float* gmaxnorm,
                         float* out_dist, int32_t* out_idx, void* ws, int64_t ws_bytes, int32_t* status,
                         cudaStream_t st, const void* split_plane = nullptr, int dt = DT_F32) {
    const KnnWs w = knn_ws_plan(nq, m, d, k, FL_KNN_BF16_RERANK, split_plane != nullptr);
    if (ws_bytes < w.bytes) {
        set_error("fl_knn: workspace %lld < %lld bytes", (long long)ws_bytes, (long long)w.bytes);
        return FL_EWORKSPACE;
    }
    char* base = static_cast<char*>(ws);
    const int vecq = dt_vec_ok(q, ldq, dt);
    const int vecd = dt_vec_ok(db, ldb, dt);
    const int vec = vecq && vecd && (d % 4 == 0);
    const PlaneLayout L = plane_layout(m, d);
    const char* pl = static_cast<const char*>(plane);
    int* fb_count = reinterpret_cast<int*>(base + w.off_cnt);
    int* fb_list = reinterpret_cast<int*>(base + w.off_fblist);
    float* tau = reinterpret_cast<float*>(base + w.off_tau);
    float* cert = reinterpret_cast<float*>(base + w.off_cert);
    if (seed_cls == nullptr) seed_cls = reinterpret_cast<float*>(base + w.off_seed_cls);

    TcKnnParams tp{};
    tp.qplane = base + w.off_qplane; tp.nq = nq; tp.nq_pad = w.nq_pad;
    tp.dbrows = pl + L.off_rows; tp.hnorm = reinterpret_cast<const float*>(pl + L.off_hnorm);
    tp.m = m; tp.m_pad = L.m_pad; tp.d_pad = L.d_pad; tp.K1 = w.K1;
    tp.nsplit = w.nsplit; tp.tiles_per_split = w.rows_per_split;
    tp.part_sc = reinterpret_cast<float*>(base + w.off_part_sc);
    tp.part_id = reinterpret_cast<uint32_t*>(base + w.off_part_id);
    tp.tau = tau; tp.status = status;
    tp.part_tau = reinterpret_cast<float*>(base + w.off_part_tau);
    tp.part_cnt = reinterpret_cast<int*>(base + w.off_part_cnt);
    tp.deep_pools = w.deep;
    tp.seed_cls = seed_cls;
    tp.k = w.kg;
    int rc;

    if (phases & TC_SCORE) FL_CHECK_CUDA(cudaMemsetAsync(fb_count, 0, 1024, st));
    if (phases & TC_PREP) {
        if (status) FL_CHECK_CUDA(cudaMemsetAsync(status, 0, sizeof(int32_t) * FL_STATUS_WORDS, st));
        rc = launch_fill_f32(tau, w.nq_pad, -INFINITY, st);
        if (rc != FL_OK) return rc;
        rc = launch_query_plane(q, nq, ldq, d, base + w.off_qplane, w.nq_pad, w.d_pad, st, dt);
        if (rc != FL_OK) return rc;
    }
    if (phases & TC_SEED) {
        if (phases & TC_SCORE) profile_begin(st);
        rc = launch_knn_tc_seed(tp, st);
        if (rc != FL_OK) return rc;
    }
    if (!(phases & TC_SCORE)) return FL_OK;

    if (!(phases & TC_PREP)) {
        rc = launch_fill_f32(tau, w.nq_pad, -INFINITY, st);
        if (rc != FL_OK) return rc;
    }
    if (!(phases & TC_SEED)) profile_begin(st);
    TcSeedMargin mg{};
    mg.dt = dt;
    if (gmaxnorm != nullptr) {
        mg.q = q; mg.ldq = ldq; mg.d = d; mg.nq = nq; mg.maxnorm = gmaxnorm; mg.eps_rel = 0.004f; mg.cert_out = cert;
    } else if (tc_seed_dense(L.m_pad, w.kg)) {
        mg.q = q; mg.ldq = ldq; mg.d = d; mg.nq = nq; mg.eps_rel = 0.004f; mg.cert_out = nullptr;
        mg.maxnorm = reinterpret_cast<const float*>(pl + L.off_meta);
    }
    rc = launch_knn_tc_seed_select(tp, mg, st);
    if (rc != FL_OK) return rc;
    rc = launch_knn_tc_scoring(tp, st);
    profile_end(st);
    if (rc != FL_OK) return rc;

    FinalizeParams fp{};
    fp.dt = dt;
    fp.q = q; fp.ldq = ldq; fp.qlist = nullptr; fp.count_dev = nullptr; fp.count = nq;
    fp.db = db; fp.m = m; fp.ldb = ldb; fp.d = d; fp.vec = vec;
    // Re-rank the tc_partial_len best scores of the union of the published pools; what the
    // scoring pass left out is bounded by the thresholds it published.
    fp.part_sc = tp.part_sc; fp.part_id = tp.part_id; fp.nsplit = w.nsplit; fp.K1 = w.plen;
    fp.k = k; fp.rerank = fp.K1; fp.row_offset = row_offset;
    fp.part_tau = tp.part_tau; fp.ntau = w.nsplit * tc_taus_per_range();
    fp.out_dist = out_dist; fp.out_idx = out_idx;
    fp.verify = 1; fp.eps_rel = 0.004f;  // 2^-8 operand rounding of both bf16 factors, rounded up
    // a sharded caller's error bound must hold for rows of every shard: the largest norm of all
    fp.maxnorm = gmaxnorm != nullptr ? gmaxnorm : reinterpret_cast<const float*>(pl + L.off_meta);
    fp.cert_tau = gmaxnorm != nullptr ? cert : nullptr;
    fp.fb_count = fb_count; fp.fb_list = fb_list; fp.fb_cap = w.fb_cap;
    fp.part_cnt = tp.part_cnt;
    int* s2_count = fb_count + 64;
    int* s2_list = w.s2 ? reinterpret_cast<int*>(base + w.off_s2_list) : nullptr;
    if (w.s2) { fp.next_count = s2_count; fp.next_list = s2_list; fp.next_cap = w.s2_cap; }
    rc = tc_knn_big(w.kg) ? launch_knn_finalize_big(fp, nq, st) : launch_knn_finalize(fp, nq, st);
    if (rc != FL_OK) return rc;

    // Second stage: the rejected rows are scored again with split (hi/lo) operands -- an error
    // bound a hundred times smaller -- against the split database plane, each starting from the
    // threshold its k-th distance so far implies; the same proof then accepts nearly all of them.
    if (w.s2) {
        const PlaneLayout L3 = plane_layout(m, 3 * w.d_pad);
        const char* pl3 = static_cast<const char*>(split_plane);
        const float* maxnorm3 = reinterpret_cast<const float*>(pl3 + L3.off_meta);
        const float eps2 = 4e-5f;   // 3 * 2^-18 from the dropped lo.lo and rounded lo terms, plus fp32 accumulation
        float* tau2 = reinterpret_cast<float*>(base + w.off_s2_tau);
        rc = launch_split_query_gather(static_cast<const float*>(q), ldq, d, s2_list, s2_count, w.s2_cap, base + w.off_s2_qplane, w.d_pad, out_dist, k,
                                       maxnorm3, eps2, tau2, st);
        if (rc != FL_OK) return rc;
        TcKnnParams t2{};
        t2.qplane = base + w.off_s2_qplane; t2.nq = w.s2_cap; t2.nq_pad = w.s2_pad;
        t2.dbrows = pl3 + L3.off_rows; t2.hnorm = reinterpret_cast<const float*>(pl3 + L3.off_hnorm);
        t2.m = m; t2.m_pad = L3.m_pad; t2.d_pad = L3.d_pad; t2.K1 = tc_pool_size(17);
        t2.nsplit = w.s2_nsplit; t2.tiles_per_split = w.s2_tiles_per_split;
        t2.part_sc = reinterpret_cast<float*>(base + w.off_s2_part_sc);
        t2.part_id = reinterpret_cast<uint32_t*>(base + w.off_s2_part_id);
        t2.part_tau = reinterpret_cast<float*>(base + w.off_s2_part_tau);
        t2.part_cnt = reinterpret_cast<int*>(base + w.off_s2_part_cnt);
        t2.tau = tau2; t2.status = status; t2.k = k; t2.big_pools = 1; t2.nq_dev = s2_count;
        rc = launch_knn_tc_scoring(t2, st);
        if (rc != FL_OK) return rc;
        FinalizeParams f2 = fp;
        f2.qlist = s2_list; f2.count_dev = s2_count; f2.count = w.s2_cap;
        f2.part_sc = t2.part_sc; f2.part_id = t2.part_id; f2.nsplit = w.s2_nsplit; f2.K1 = w.s2_plen;
        f2.rerank = f2.K1; f2.part_tau = t2.part_tau; f2.ntau = w.s2_nsplit * tc_taus_per_range();
        f2.part_cnt = t2.part_cnt; f2.eps_rel = eps2; f2.maxnorm = maxnorm3; f2.cert_tau = nullptr;
        f2.next_count = nullptr; f2.next_list = nullptr; f2.next_cap = 0;
        rc = launch_knn_finalize_big(f2, w.s2_cap, st);
        if (rc != FL_OK) return rc;
    }
    fallback_fixup_kernel<<<1, 1, 0, st>>>(fb_count, w.fb_cap, status, w.K1, w.s2 ? s2_count : nullptr, w.s2_cap);
    FL_CHECK_LAUNCH();

    // Rows whose pool could not be proven complete: exact CUDA-core pass over the list.
    SimtKnnParams sp{};
    sp.dt = dt;
    sp.q = q; sp.ldq = ldq; sp.qlist = fb_list; sp.count_dev = fb_count; sp.count = 0;
    sp.db = db; sp.m = m; sp.ldb = ldb; sp.d = d;
    sp.hnorm = reinterpret_cast<const float*>(pl + L.off_hnorm);
    sp.K1 = w.K1f; sp.cap = simt_pool_cap(w.K1f); sp.npl = sp.cap / 32; sp.keep = simt_pool_keep(w.K1f, k);
    sp.nsplit = w.nsplit_fb; sp.rows_per_split = w.rows_per_split_fb;
    sp.dyn_blocks = w.fb_blocks; sp.dyn_bq = w.fb_bq;
    sp.part_sc = reinterpret_cast<float*>(base + w.off_fbpart_sc);
    sp.part_id = reinterpret_cast<uint32_t*>(base + w.off_fbpart_id);
    sp.vecq = vecq; sp.vecd = vecd;
    rc = launch_knn_simt(sp, w.fb_cap, st);
    if (rc != FL_OK) return rc;
    FinalizeParams ff = fp;
    ff.qlist = fb_list; ff.count_dev = fb_count; ff.count = 0;
    ff.part_sc = sp.part_sc; ff.part_id = sp.part_id; ff.nsplit = w.nsplit_fb; ff.K1 = w.K1f;
    // as in the exact mode: walk until k distances are safe against the fp32 scoring error; last pass
    ff.rerank = simt_pool_keep(w.K1f, k); ff.verify = 1; ff.eps_rel = SIMT_EPS_REL; ff.part_tau = nullptr; ff.ntau = 0;
    ff.fb_count = nullptr; ff.fb_list = nullptr; ff.fb_cap = 0;
    ff.cert_tau = nullptr;
    ff.next_count = nullptr; ff.next_list = nullptr; ff.next_cap = 0;
    ff.dyn_blocks = w.fb_blocks; ff.dyn_bq = w.fb_bq;
    return launch_knn_finalize(ff, w.fb_cap, st);
}

// Every dtype and both stages behind one body: fl_knn_f32 / fl_knn_staged_f32 / fl_knn_rows.
static int knn_rows_impl(const char* who, const void* q, int64_t nq, int64_t ldq, const void* db, int64_t m, int64_t ldb,
                         int d, int k, int dt, int mode, const void* plane, const void* split_plane, int64_t row_offset,
                         float* out_dist, int32_t* out_idx, void* ws, int64_t ws_bytes, int32_t* status, void* stream) {
    FL_CHECK_ARG(dt == DT_F32 || dt == DT_BF16 || dt == DT_F16, "%s: unknown dtype %d", who, dt);
    int rc = knn_check_args(who, q, nq, ldq, db, m, ldb, d, k, &mode, plane, row_offset, out_dist, out_idx, ws);
    if (rc != FL_OK || nq == 0) return rc;
    cudaStream_t st = (cudaStream_t)stream;
    if (split_plane != nullptr) {
        FL_CHECK_ARG(mode == FL_KNN_BF16_RERANK && dt == DT_F32, "%s: the split-plane stage goes with fp32 rows and the tensor-core mode", who);
        FL_CHECK_ARG(split_plane_supported(d), "%s: d=%d > 128 has no split plane", who, d);
        FL_CHECK_ARG((reinterpret_cast<uintptr_t>(split_plane) & 255) == 0, "%s: split plane must be 256-byte aligned", who);
    }
    if (mode == FL_KNN_BF16_RERANK)
        return knn_tc_phases(TC_PREP | TC_SEED | TC_SCORE, q, nq, ldq, db, m, ldb, d, k, plane, row_offset, nullptr,
                             nullptr, out_dist, out_idx, ws, ws_bytes, status, st, split_plane, dt);

    const KnnWs w = knn_ws_plan(nq, m, d, k, mode);
    if (ws_bytes < w.bytes) {
        set_error("%s: workspace %lld < %lld bytes", who, (long long)ws_bytes, (long long)w.bytes);
        return FL_EWORKSPACE;
    }
    char* base = static_cast<char*>(ws);
    const int vecq = dt_vec_ok(q, ldq, dt);
    const int vecd = dt_vec_ok(db, ldb, dt);
    const int vec = vecq && vecd && (d % 4 == 0);
    if (status) FL_CHECK_CUDA(cudaMemsetAsync(status, 0, sizeof(int32_t) * FL_STATUS_WORDS, st));
    FL_CHECK_CUDA(cudaMemsetAsync(base + w.off_cnt, 0, 1024, st));
    const float* hnorm;
    const float* maxnorm;
    if (plane) {
        const PlaneLayout L = plane_layout(m, d);
        hnorm = reinterpret_cast<const float*>(static_cast<const char*>(plane) + L.off_hnorm);
        maxnorm = reinterpret_cast<const float*>(static_cast<const char*>(plane) + L.off_meta);
    } else {
        float* h = reinterpret_cast<float*>(base + w.off_hnorm);
        unsigned int* mx = reinterpret_cast<unsigned int*>(base + w.off_cnt) + 128;    // cleared above
        halfnorm_kernel<<<(unsigned)ceil_div(m, 8), 256, 0, st>>>(db, m, d, ldb, h, mx, dt);
        FL_CHECK_LAUNCH();
        hnorm = h;
        maxnorm = reinterpret_cast<const float*>(mx);
    }
    SimtKnnParams sp{};
    sp.dt = dt;
    sp.q = q; sp.ldq = ldq; sp.qlist = nullptr; sp.count_dev = nullptr; sp.count = nq;
    sp.db = db; sp.m = m; sp.ldb = ldb; sp.d = d; sp.hnorm = hnorm;
    sp.K1 = w.K1; sp.cap = simt_pool_cap(w.K1); sp.npl = sp.cap / 32; sp.keep = simt_pool_keep(w.K1, k);
    sp.nsplit = w.nsplit; sp.rows_per_split = w.rows_per_split;
    sp.part_sc = reinterpret_cast<float*>(base + w.off_part_sc);
    sp.part_id = reinterpret_cast<uint32_t*>(base + w.off_part_id);
    sp.vecq = vecq; sp.vecd = vecd;
    profile_begin(st);
    rc = launch_knn_simt(sp, nq, st);
    profile_end(st);
    if (rc != FL_OK) return rc;

    FinalizeParams fp{};
    fp.dt = dt;
    fp.q = q; fp.ldq = ldq; fp.qlist = nullptr; fp.count_dev = nullptr; fp.count = nq;
    fp.db = db; fp.m = m; fp.ldb = ldb; fp.d = d; fp.vec = vec;
    fp.part_sc = sp.part_sc; fp.part_id = sp.part_id; fp.nsplit = w.nsplit; fp.K1 = w.K1;
    // The walk over the merged pool (best score first) ends once k exact distances lie below what the
    // next score allows, the fp32 scoring error included -- usually after k + 8 entries, further where
    // many rows sit within that error of the k-th neighbour.  Nothing is queued: this is the last pass.
    // (The scan's compactions keep simt_pool_keep entries per pool: down to that depth the merged list
    // misses no row that scored above its entries, so that is how far the walk may go.)
    fp.k = k; fp.rerank = simt_pool_keep(w.K1, k); fp.row_offset = row_offset;
    fp.out_dist = out_dist; fp.out_idx = out_idx; fp.verify = 1; fp.eps_rel = SIMT_EPS_REL; fp.maxnorm = maxnorm;
    rc = launch_knn_finalize(fp, nq, st);
    if (rc != FL_OK) return rc;
    if (status) {
        fallback_fixup_kernel<<<1, 1, 0, st>>>(reinterpret_cast<int*>(base + w.off_cnt), 1 << 30,
                                               status, w.K1);
        FL_CHECK_LAUNCH();
    }
    return FL_OK;
}

extern "C" int fl_knn_f32(const float* q, int64_t nq, int64_t ldq, const float* db, int64_t m,
                          int64_t ldb, int d, int k, int mode, const void* plane, int64_t row_offset,
                          float* out_dist, int32_t* out_idx, void* ws, int64_t ws_bytes,
                          int32_t* status, void* stream) {
    return knn_rows_impl("fl_knn_f32", q, nq, ldq, db, m, ldb, d, k, DT_F32, mode, plane, nullptr, row_offset, out_dist,
                         out_idx, ws, ws_bytes, status, stream);
}

extern "C" int fl_knn_rows(const void* q, int64_t nq, int64_t ldq, const void* db, int64_t m, int64_t ldb, int d, int k,
                           int dtype, int mode, const void* plane, int64_t row_offset, float* out_dist, int32_t* out_idx,
                           void* ws, int64_t ws_bytes, int32_t* status, void* stream) {
    return knn_rows_impl("fl_knn_rows", q, nq, ldq, db, m, ldb, d, k, dtype, mode, plane, nullptr, row_offset, out_dist,
                         out_idx, ws, ws_bytes, status, stream);
}

// ---- batch of small problems, exact mode ---------------------------------------------------
struct KnnBatchWs { int K1, nsplit; int64_t rows_per_split; int64_t off_hnorm, off_part_sc, off_part_id, off_cnt, bytes; };

static KnnBatchWs knn_batch_plan(int batch, int64_t nq, int64_t m, int d, int k) {
    KnnBatchWs w{};
    w.K1 = simt_pool_size(k);
    // the batch fills the GPU: ranges only as far as one problem alone would want them divided by the batch
    simt_split_plan(nq * batch, m, w.K1, d, &w.nsplit, &w.rows_per_split);
    int64_t cur = 0;
    w.off_hnorm = take(cur, (int64_t)batch * m * 4);
    w.off_part_sc = take(cur, (int64_t)batch * nq * w.nsplit * w.K1 * 4);
    w.off_part_id = take(cur, (int64_t)batch * nq * w.nsplit * w.K1 * 4);
    w.off_cnt = take(cur, 1024);
    w.bytes = cur;
    return w;
}

extern "C" int64_t fl_knn_batch_workspace_bytes(int batch, int64_t nq, int64_t m, int d, int k) {
    if (batch < 1 || nq < 1 || m < 1 || d < 1 || k < 1 || k > 512) return 0;
    return knn_batch_plan(batch, nq, m, d, k).bytes;
}

extern "C" int fl_knn_batch_f32(const float* q, int batch, int64_t nq, int64_t ldq, int64_t q_bstride, const float* db,
                                int64_t m, int64_t ldb, int64_t db_bstride, int d, int k, float* out_dist, int32_t* out_idx,
                                void* ws, int64_t ws_bytes, void* stream) {
    FL_CHECK_ARG(batch >= 1 && batch <= 65535, "fl_knn_batch_f32: batch must be in [1, 65535] (got %d)", batch);
    int mode = FL_KNN_EXACT_SIMT;
    int rc = knn_check_args("fl_knn_batch_f32", q, nq, ldq, db, m, ldb, d, k, &mode, nullptr, 0, out_dist, out_idx, ws);
    if (rc != FL_OK || nq == 0) return rc;
    FL_CHECK_ARG(q_bstride >= 0 && db_bstride >= 0, "fl_knn_batch_f32: negative batch stride");
    const KnnBatchWs w = knn_batch_plan(batch, nq, m, d, k);
    if (ws_bytes < w.bytes) { set_error("fl_knn_batch_f32: workspace %lld < %lld bytes", (long long)ws_bytes, (long long)w.bytes); return FL_EWORKSPACE; }
    cudaStream_t st = (cudaStream_t)stream;
    char* base = static_cast<char*>(ws);
    const int vecq = dt_vec_ok(q, ldq, DT_F32) && q_bstride % 4 == 0;
    const int vecd = dt_vec_ok(db, ldb, DT_F32) && db_bstride % 4 == 0;
    const int vec = vecq && vecd && (d % 4 == 0);
    FL_CHECK_CUDA(cudaMemsetAsync(base + w.off_cnt, 0, 1024, st));
    float* hnorm = reinterpret_cast<float*>(base + w.off_hnorm);
    unsigned int* mx = reinterpret_cast<unsigned int*>(base + w.off_cnt) + 128;     // largest row norm of the whole batch
    halfnorm_kernel<<<dim3((unsigned)ceil_div(m, 8), (unsigned)batch), 256, 0, st>>>(db, m, d, ldb, hnorm, mx, DT_F32, db_bstride);
    FL_CHECK_LAUNCH();
    SimtKnnParams sp{};
    sp.dt = DT_F32;
    sp.q = q; sp.ldq = ldq; sp.count = nq; sp.db = db; sp.m = m; sp.ldb = ldb; sp.d = d; sp.hnorm = hnorm;
    sp.K1 = w.K1; sp.cap = simt_pool_cap(w.K1); sp.npl = sp.cap / 32; sp.keep = simt_pool_keep(w.K1, k);
    sp.nsplit = w.nsplit; sp.rows_per_split = w.rows_per_split;
    sp.part_sc = reinterpret_cast<float*>(base + w.off_part_sc);
    sp.part_id = reinterpret_cast<uint32_t*>(base + w.off_part_id);
    sp.vecq = vecq; sp.vecd = vecd;
    sp.batch = batch; sp.q_bstride = q_bstride; sp.db_bstride = db_bstride;
    rc = launch_knn_simt(sp, nq, st);
    if (rc != FL_OK) return rc;
    FinalizeParams fp{};
    fp.dt = DT_F32;
    fp.q = q; fp.ldq = ldq; fp.count = nq; fp.db = db; fp.m = m; fp.ldb = ldb; fp.d = d; fp.vec = vec;
    fp.part_sc = sp.part_sc; fp.part_id = sp.part_id; fp.nsplit = w.nsplit; fp.K1 = w.K1;
    fp.k = k; fp.rerank = simt_pool_keep(w.K1, k); fp.row_offset = 0;
    fp.out_dist = out_dist; fp.out_idx = out_idx; fp.verify = 1; fp.eps_rel = SIMT_EPS_REL;
    fp.maxnorm = reinterpret_cast<const float*>(mx);
    fp.batch = batch; fp.q_bstride = q_bstride; fp.db_bstride = db_bstride;
    return launch_knn_finalize(fp, nq, st);
}

extern "C" int64_t fl_knn_seed_floats(int64_t nq) {
    if (nq < 1) return 0;
    return tc_query_rows_padded(nq) * 32;
}

extern "C" int fl_knn_seed_f32(const float* q, int64_t nq, int64_t ldq, int d, int k, const void* plane, int64_t m,
                               float* seed_cls, void* ws, int64_t ws_bytes, int32_t* status, void* stream) {
    FL_CHECK_ARG(nq >= 0 && m >= 1 && d >= 1 && k >= 1 && ldq >= d, "fl_knn_seed_f32: bad shape");
    if (nq == 0) return FL_OK;
    FL_CHECK_ARG(q && plane && seed_cls && ws, "fl_knn_seed_f32: null pointer");
    FL_CHECK_ARG((reinterpret_cast<uintptr_t>(ws) & 255) == 0 && (reinterpret_cast<uintptr_t>(plane) & 255) == 0 &&
                 (reinterpret_cast<uintptr_t>(seed_cls) & 15) == 0, "fl_knn_seed_f32: misaligned buffer");
    // a shard with fewer than k rows still takes part (its maxima count for the other shards)
    if (tc_knn_supported(nq, m, d, k < 112 ? k : 112) != FL_OK) {
        set_error("fl_knn_seed_f32: shape (nq=%lld m=%lld d=%d) outside the tensor-core kernel's range", (long long)nq, (long long)m, d);
        return FL_EUNSUPPORTED;
    }
    return knn_tc_phases(TC_PREP | TC_SEED, q, nq, ldq, nullptr, m, d, d, k, plane, 0, seed_cls, nullptr, nullptr,
                         nullptr, ws, ws_bytes, status, (cudaStream_t)stream);
}

extern "C" int fl_knn_seeded_f32(const float* q, int64_t nq, int64_t ldq, const float* db, int64_t m, int64_t ldb,
                                 int d, int k, const void* plane, int64_t row_offset, const float* seed_cls,
                                 const float* global_maxnorm, float* out_dist, int32_t* out_idx, void* ws,
                                 int64_t ws_bytes, int32_t* status, void* stream) {
    int mode = FL_KNN_BF16_RERANK;
    int rc = knn_check_args("fl_knn_seeded_f32", q, nq, ldq, db, m, ldb, d, k, &mode, plane, row_offset, out_dist, out_idx, ws);
    if (rc != FL_OK || nq == 0) return rc;
    FL_CHECK_ARG(seed_cls != nullptr && global_maxnorm != nullptr, "fl_knn_seeded_f32: null pointer");
    return knn_tc_phases(TC_SCORE, q, nq, ldq, db, m, ldb, d, k, plane, row_offset, const_cast<float*>(seed_cls),
                         global_maxnorm, out_dist, out_idx, ws, ws_bytes, status, (cudaStream_t)stream);
}

extern "C" int64_t fl_knn_plane_maxnorm_offset(int64_t m, int d) {
    if (m < 1 || d < 1) return -1;
    return plane_layout(m, d).off_meta;
}

extern "C" int fl_debug_tc_experiment(int flags, unsigned wait_us) {
    tc_debug_set(flags, wait_us);
    return FL_OK;
}

extern "C" int fl_topk_merge_f32(const float* cand_dist, const int32_t* cand_idx, int64_t nq, int ncand,
                                 int k, float* out_dist, int32_t* out_idx, void* stream) {
    FL_CHECK_ARG(nq >= 0 && ncand >= 1 && k >= 1, "fl_topk_merge_f32: bad shape");
    if (k > 512) { set_error("fl_topk_merge_f32: k=%d > 512 is not supported", k); return FL_EUNSUPPORTED; }
    if (nq == 0) return FL_OK;
    FL_CHECK_ARG(cand_dist && cand_idx && out_dist && out_idx, "fl_topk_merge_f32: null pointer");
    cudaStream_t st = (cudaStream_t)stream;
    const unsigned grid = (unsigned)ceil_div(nq, 4);
    const int K1 = simt_pool_size(k);
    switch (K1 / 32) {
        case 1: topk_merge_kernel<1><<<grid, 128, 0, st>>>(cand_dist, cand_idx, nq, ncand, k, out_dist, out_idx); break;
        case 2: topk_merge_kernel<2><<<grid, 128, 0, st>>>(cand_dist, cand_idx, nq, ncand, k, out_dist, out_idx); break;
        case 4: topk_merge_kernel<4><<<grid, 128, 0, st>>>(cand_dist, cand_idx, nq, ncand, k, out_dist, out_idx); break;
        case 8: topk_merge_kernel<8><<<grid, 128, 0, st>>>(cand_dist, cand_idx, nq, ncand, k, out_dist, out_idx); break;
        default: topk_merge_kernel<16><<<grid, 128, 0, st>>>(cand_dist, cand_idx, nq, ncand, k, out_dist, out_idx); break;
    }
    FL_CHECK_LAUNCH();
    return FL_OK;
}

extern "C" int fl_gather_l2sq_f32(const float* x, int64_t n, int64_t ldx, const float* c, int64_t m,
                                  int64_t ldc, int d, const void* idx, int idx_is_i64, int k, float* out,
                                  void* stream) {
    FL_CHECK_ARG(n >= 0 && m >= 1 && d >= 1 && k >= 1 && ldx >= d && ldc >= d, "fl_gather_l2sq_f32: bad shape");
    if (n == 0) return FL_OK;
    FL_CHECK_ARG(x && c && idx && out, "fl_gather_l2sq_f32: null pointer");
    cudaStream_t st = (cudaStream_t)stream;
    const unsigned grid = (unsigned)ceil_div(n * k, 8);
    if (idx_is_i64)
        gather_l2sq_kernel<int64_t><<<grid, 256, 0, st>>>(x, n, ldx, c, m, ldc, d,
                                                          static_cast<const int64_t*>(idx), k, out);
    else
        gather_l2sq_kernel<int32_t><<<grid, 256, 0, st>>>(x, n, ldx, c, m, ldc, d,
                                                          static_cast<const int32_t*>(idx), k, out);
    FL_CHECK_LAUNCH();
    return FL_OK;
}

extern "C" int64_t fl_knn_split_plane_bytes(int64_t m, int d) {
    if (m < 1 || d < 1 || !split_plane_supported(d)) return 0;
    return plane_layout(m, 3 * (int)round_up(d, 64)).bytes;
}

extern "C" int fl_knn_prepare_split_f32(const float* db, int64_t m, int d, int64_t ld, void* split_plane,
                                        int64_t split_plane_bytes, void* stream) {
    FL_CHECK_ARG(m >= 1 && d >= 1 && ld >= d, "fl_knn_prepare_split_f32: bad shape m=%lld d=%d ld=%lld", (long long)m, d,
                 (long long)ld);
    FL_CHECK_ARG(db && split_plane, "fl_knn_prepare_split_f32: null pointer");
    FL_CHECK_ARG((reinterpret_cast<uintptr_t>(split_plane) & 255) == 0, "fl_knn_prepare_split_f32: plane must be 256-byte aligned");
    const int64_t need = fl_knn_split_plane_bytes(m, d);
    if (need == 0) { set_error("fl_knn_prepare_split_f32: d=%d > 128 has no split plane", d); return FL_EUNSUPPORTED; }
    if (split_plane_bytes < need) {
        set_error("fl_knn_prepare_split_f32: plane buffer %lld < %lld bytes", (long long)split_plane_bytes, (long long)need);
        return FL_EWORKSPACE;
    }
    return launch_split_db_plane(db, m, d, ld, split_plane, (cudaStream_t)stream);
}

extern "C" int64_t fl_knn_staged_workspace_bytes(int64_t nq, int64_t m, int d, int k) {
    if (nq < 1 || m < 1 || d < 1 || k < 1 || tc_knn_supported(nq, m, d, k) != FL_OK) return 0;
    return knn_ws_plan(nq, m, d, k, FL_KNN_BF16_RERANK, 1).bytes;
}

extern "C" int fl_knn_staged_f32(const float* q, int64_t nq, int64_t ldq, const float* db, int64_t m, int64_t ldb, int d,
                                 int k, const void* plane, const void* split_plane, int64_t row_offset, float* out_dist,
                                 int32_t* out_idx, void* ws, int64_t ws_bytes, int32_t* status, void* stream) {
    return knn_rows_impl("fl_knn_staged_f32", q, nq, ldq, db, m, ldb, d, k, DT_F32, FL_KNN_BF16_RERANK, plane, split_plane,
                         row_offset, out_dist, out_idx, ws, ws_bytes, status, stream);
}

// Test hook: runs only the tensor-core scoring pass for up to 128 queries and writes the
// scores s = <q,x> - ||x||^2/2 of every (query, database row) pair, so a test can compare
// the MMA pipeline with a plain matrix product.
extern "C" int fl_debug_knn_tc_scores(const float* q, int64_t nq, int64_t ldq, int d, const void* plane,
                                      int64_t m, float* scores, int64_t ld_scores, void* ws, int64_t ws_bytes,
                                      int32_t* status, void* stream) {
    FL_CHECK_ARG(q && plane && scores && ws && nq >= 1 && nq <= 128 && m >= 1 && d >= 1, "fl_debug_knn_tc_scores: bad arguments");
    if (d > 256 || tc_knn_supported(nq, m, d, 10) != FL_OK) { set_error("fl_debug_knn_tc_scores: unsupported shape"); return FL_EUNSUPPORTED; }
    const KnnWs w = knn_ws_plan(nq, m, d, 10, FL_KNN_BF16_RERANK);
    if (ws_bytes < w.bytes) { set_error("fl_debug_knn_tc_scores: workspace too small"); return FL_EWORKSPACE; }
    const PlaneLayout L = plane_layout(m, d);
    FL_CHECK_ARG(ld_scores >= L.m_pad, "fl_debug_knn_tc_scores: ld_scores must cover the padded row count %lld", (long long)L.m_pad);
    cudaStream_t st = (cudaStream_t)stream;
    char* base = static_cast<char*>(ws);
    const char* pl = static_cast<const char*>(plane);
    float* tau = reinterpret_cast<float*>(base + w.off_tau);
    if (status) FL_CHECK_CUDA(cudaMemsetAsync(status, 0, sizeof(int32_t) * FL_STATUS_WORDS, st));
    fill_f32_kernel<<<(unsigned)ceil_div(w.nq_pad, 256), 256, 0, st>>>(tau, w.nq_pad, -INFINITY);
    FL_CHECK_LAUNCH();
    int rc = launch_query_plane(q, nq, ldq, d, base + w.off_qplane, w.nq_pad, w.d_pad, st);
    if (rc != FL_OK) return rc;
    TcKnnParams tp{};
    tp.qplane = base + w.off_qplane; tp.nq = nq; tp.nq_pad = w.nq_pad;
    tp.dbrows = pl + L.off_rows; tp.hnorm = reinterpret_cast<const float*>(pl + L.off_hnorm);
    tp.m = m; tp.m_pad = L.m_pad; tp.d_pad = L.d_pad; tp.K1 = w.K1;
    tp.nsplit = w.nsplit; tp.tiles_per_split = w.rows_per_split;
    tp.part_sc = reinterpret_cast<float*>(base + w.off_part_sc);
    tp.part_id = reinterpret_cast<uint32_t*>(base + w.off_part_id);
    tp.tau = tau; tp.status = status;
    tp.part_tau = reinterpret_cast<float*>(base + w.off_part_tau);
    return launch_knn_tc_debug(tp, scores, ld_scores, st);
}

// Debug aid: copies the per-CTA cycle counters of the last tensor-core kNN launch on the
// current device to host memory (16 counters for each of up to 160 CTAs; synchronises).
extern "C" int fl_debug_tc_prof_read(unsigned long long* host_out, int words) {
    FL_CHECK_ARG(host_out && words > 0, "fl_debug_tc_prof_read: bad arguments");
    return tc_prof_read(host_out, words);
}
