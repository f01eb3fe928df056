// IVF-Flat fine scan: groups the (query, probe) pairs by inverted list on the device,
// scans every probed list once per group of queries with the exact CUDA-core scoring
// kernel and merges each query's per-probe pools with an exact fp32 re-rank.
#include "knn_internal.h"
#include "pool.cuh"

namespace fl {

__global__ void ivf_count_kernel(const int32_t* __restrict__ probed, int64_t npairs, int nlist,
                                 int* __restrict__ cnt) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= npairs) return;
    const int c = probed[i];
    if (c >= 0 && c < nlist) atomicAdd(cnt + c, 1);
}

// Single block: exclusive scans of the per-list pair counts and group counts.
__global__ void __launch_bounds__(1024) ivf_scan_kernel(const int* __restrict__ cnt, int nlist, int bq,
                                                        const int64_t* __restrict__ list_offsets,
                                                        int* __restrict__ pair_off,
                                                        int* __restrict__ item_off, int* __restrict__ cursor) {
    __shared__ int s_pair[1024];
    __shared__ int s_item[1024];
    __shared__ int carry_pair, carry_item;
    const int t = threadIdx.x;
    if (t == 0) { carry_pair = 0; carry_item = 0; }
    __syncthreads();
    for (int base = 0; base < nlist; base += 1024) {
        const int c = base + t;
        int np = 0, ni = 0;
        if (c < nlist) {
            np = cnt[c];
            // a list without rows contributes no work item; its pairs keep empty pools
            const bool has_rows = list_offsets[c + 1] > list_offsets[c];
            ni = has_rows ? (np + bq - 1) / bq : 0;
        }
        s_pair[t] = np;
        s_item[t] = ni;
        __syncthreads();
        for (int o = 1; o < 1024; o <<= 1) {
            const int a = t >= o ? s_pair[t - o] : 0;
            const int b = t >= o ? s_item[t - o] : 0;
            __syncthreads();
            s_pair[t] += a;
            s_item[t] += b;
            __syncthreads();
        }
        if (c < nlist) {
            pair_off[c] = carry_pair + s_pair[t] - np;
            item_off[c] = carry_item + s_item[t] - ni;
            cursor[c] = 0;
        }
        __syncthreads();
        if (t == 1023) { carry_pair += s_pair[t]; carry_item += s_item[t]; }
        __syncthreads();
    }
    if (t == 0) { pair_off[nlist] = carry_pair; item_off[nlist] = carry_item; }
}

__global__ void ivf_scatter_kernel(const int32_t* __restrict__ probed, int64_t npairs, int nlist,
                                   const int* __restrict__ pair_off, int* __restrict__ cursor,
                                   int* __restrict__ sorted_pair) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= npairs) return;
    const int c = probed[i];
    if (c < 0 || c >= nlist) return;
    const int pos = pair_off[c] + atomicAdd(cursor + c, 1);
    sorted_pair[pos] = (int)i;
}

__global__ void ivf_fill_kernel(float* sc, uint32_t* id, int64_t n) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) { sc[i] = neg_inf(); id[i] = INVALID_ID; }
}

__global__ void ivf_halfnorm_kernel(const float* __restrict__ x, int64_t n, int d, int64_t ld,
                                    float* __restrict__ out) {
    const int lane = threadIdx.x & 31;
    const int64_t row = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (row >= n) return;
    const float* p = x + row * ld;
    float s = 0.f;
    for (int c = lane; c < d; c += 32) { const float v = __ldg(p + c); s += v * v; }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(FULL_MASK, s, o);
    if (lane == 0) out[row] = 0.5f * s;
}

struct IvfWs {
    int K1, bq;
    int64_t max_items;
    int64_t off_cnt, off_pair_off, off_item_off, off_cursor, off_sorted, off_part_sc, off_part_id,
        off_hnorm, off_tau, bytes;
};

static int64_t take(int64_t& cur, int64_t bytes) {
    const int64_t o = cur;
    cur += round_up(bytes > 0 ? bytes : 1, 1024);
    return o;
}

static IvfWs ivf_ws_plan(int64_t nq, int nprobe, int nlist, int64_t m, int k) {
    IvfWs w{};
    w.K1 = simt_pool_size(k);
    w.bq = simt_block_queries(w.K1);
    const int64_t npairs = nq * nprobe;
    w.max_items = ceil_div(npairs, w.bq > 0 ? w.bq : 16) + nlist;
    int64_t cur = 0;
    w.off_cnt = take(cur, (int64_t)(nlist + 1) * 4);
    w.off_pair_off = take(cur, (int64_t)(nlist + 1) * 4);
    w.off_item_off = take(cur, (int64_t)(nlist + 1) * 4);
    w.off_cursor = take(cur, (int64_t)(nlist + 1) * 4);
    w.off_sorted = take(cur, npairs * 4);
    w.off_part_sc = take(cur, npairs * w.K1 * 4);
    w.off_part_id = take(cur, npairs * w.K1 * 4);
    w.off_hnorm = take(cur, m * 4);
    w.off_tau = take(cur, nq * 4);
    w.bytes = cur;
    return w;
}

// Groups the (query, probe) pairs by list: per-list pair counts, exclusive scans of the pairs and
// of the work items (groups of bq pairs; lists without rows get none), pair ids sorted by list.
int launch_ivf_group(const int32_t* probed, int64_t npairs, int nlist, int bq, const int64_t* list_offsets, int* cnt,
                     int* pair_off, int* item_off, int* cursor, int* sorted_pair, cudaStream_t st) {
    FL_CHECK_CUDA(cudaMemsetAsync(cnt, 0, sizeof(int) * (size_t)(nlist + 1), st));
    ivf_count_kernel<<<(unsigned)ceil_div(npairs, 256), 256, 0, st>>>(probed, npairs, nlist, cnt);
    FL_CHECK_LAUNCH();
    ivf_scan_kernel<<<1, 1024, 0, st>>>(cnt, nlist, bq, list_offsets, pair_off, item_off, cursor);
    FL_CHECK_LAUNCH();
    ivf_scatter_kernel<<<(unsigned)ceil_div(npairs, 256), 256, 0, st>>>(probed, npairs, nlist, pair_off, cursor, sorted_pair);
    FL_CHECK_LAUNCH();
    return FL_OK;
}

// ---- index build: cell-contiguous (CSR) layout from per-row list labels ------------------
// The rows are cut into units of `unit_rows` consecutive rows.  cnt[u][l] counts the rows of unit
// u with label l; a scan down the units turns it into the rank, within list l, of the unit's first
// such row.  One warp then walks its unit in row order and gives every row its position
// list_offsets[l] + rank -- rows of one list keep their original order (a stable partition, the
// order of a stable argsort by label) -- and a last kernel moves the rows.
__global__ void ivf_build_count_kernel(const int32_t* __restrict__ labels, int64_t m, int nlist, int64_t unit_rows,
                                       int* __restrict__ cnt) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= m) return;
    const int l = labels[i];
    if (l >= 0 && l < nlist) atomicAdd(cnt + (i / unit_rows) * nlist + l, 1);
}

// Thread per list: exclusive scan of cnt[.][l] down the units (in place), total[l] = list length.
__global__ void ivf_build_colscan_kernel(int* __restrict__ cnt, int64_t units, int nlist, int* __restrict__ total) {
    const int l = blockIdx.x * blockDim.x + threadIdx.x;
    if (l >= nlist) return;
    int run = 0;
    for (int64_t u = 0; u < units; ++u) {
        const int c = cnt[u * nlist + l];
        cnt[u * nlist + l] = run;
        run += c;
    }
    total[l] = run;
}

// Single block: list_offsets = exclusive scan of the list lengths (int64), and the longest list.
__global__ void __launch_bounds__(1024) ivf_build_offsets_kernel(const int* __restrict__ total, int nlist,
                                                                 int64_t* __restrict__ list_offsets,
                                                                 int32_t* __restrict__ max_len) {
    __shared__ long long s_v[1024];
    __shared__ long long carry;
    __shared__ int s_max;
    const int t = threadIdx.x;
    if (t == 0) { carry = 0; s_max = 0; }
    __syncthreads();
    for (int base = 0; base < nlist; base += 1024) {
        const int c = base + t;
        const int n = c < nlist ? total[c] : 0;
        atomicMax(&s_max, n);
        s_v[t] = n;
        __syncthreads();
        for (int o = 1; o < 1024; o <<= 1) {
            const long long a = t >= o ? s_v[t - o] : 0;
            __syncthreads();
            s_v[t] += a;
            __syncthreads();
        }
        if (c < nlist) list_offsets[c] = carry + s_v[t] - n;
        __syncthreads();
        if (t == 1023) carry += s_v[t];
        __syncthreads();
    }
    if (t == 0) { list_offsets[nlist] = carry; if (max_len) *max_len = s_max; }
}

// One warp per unit, 32 rows per step in row order: position of every row in the list-sorted layout.
// Lanes with the same label are ranked by lane (match_any), the unit's running count of each label
// lives in its row of `cnt` (only this warp touches it).  Rows with a label outside [0, nlist) get -1.
__global__ void ivf_build_rank_kernel(const int32_t* __restrict__ labels, int64_t m, int nlist, int64_t unit_rows,
                                      int* __restrict__ cnt, const int64_t* __restrict__ list_offsets,
                                      int64_t* __restrict__ pos) {
    const int lane = threadIdx.x & 31;
    const int64_t u = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const int64_t r0 = u * unit_rows;
    if (r0 >= m) return;
    const int64_t r1 = min(m, r0 + unit_rows);
    int* mine = cnt + u * nlist;
    for (int64_t base = r0; base < r1; base += 32) {
        const int64_t r = base + lane;
        int l = r < r1 ? labels[r] : -1;
        if (l >= nlist) l = -1;
        const unsigned same = __match_any_sync(FULL_MASK, l);
        const int before = __popc(same & ((1u << lane) - 1u));
        int start = 0;
        if (l >= 0) start = mine[l];
        __syncwarp();
        if (l >= 0 && before == 0) mine[l] = start + __popc(same);     // the first lane of each label advances it
        __syncwarp();
        if (r < r1) pos[r] = l >= 0 ? list_offsets[l] + start + before : -1;
    }
}

// One warp per row: the row goes to its position, ids[position] = the row's original index.
__global__ void ivf_build_move_kernel(const float* __restrict__ x, int64_t m, int64_t ldx, int d,
                                      const int64_t* __restrict__ pos, float* __restrict__ data, int64_t* __restrict__ ids) {
    const int lane = threadIdx.x & 31;
    const int64_t r = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (r >= m) return;
    const int64_t p = pos[r];
    if (p < 0) return;
    const float* src = x + r * ldx;
    float* dst = data + p * d;
    for (int c = lane; c < d; c += 32) dst[c] = __ldg(src + c);
    if (lane == 0) ids[p] = r;
}

struct IvfBuildWs { int64_t unit_rows, units, off_cnt, off_total, off_pos, bytes; };
static IvfBuildWs ivf_build_plan(int64_t m, int nlist) {
    IvfBuildWs w{};
    // units of at least 2048 rows, few enough that the count matrix stays below 2^24 entries
    int64_t ur = 2048;
    const int64_t need = ceil_div(m * (int64_t)nlist, (int64_t)1 << 24);
    if (need > ur) ur = round_up(need, 32);
    w.unit_rows = ur;
    w.units = ceil_div(m, ur);
    int64_t cur = 0;
    w.off_cnt = take(cur, w.units * nlist * 4);
    w.off_total = take(cur, (int64_t)nlist * 4);
    w.off_pos = take(cur, m * 8);
    w.bytes = cur;
    return w;
}

}  // namespace fl

using namespace fl;

// out[i] = pos[i] >= 0 ? ids[pos[i]] : -1
__global__ void ivf_map_ids_kernel(const int32_t* __restrict__ pos, const int64_t* __restrict__ ids, int64_t n, int64_t m,
                                   int64_t* __restrict__ out) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const int32_t p = pos[i];
    out[i] = (p >= 0 && p < m) ? __ldg(ids + p) : -1;
}

extern "C" int fl_ivf_map_ids(const int32_t* pos, const int64_t* ids, int64_t n, int64_t m, int64_t* out, void* stream) {
    FL_CHECK_ARG(n >= 0 && m >= 0, "fl_ivf_map_ids: bad shape");
    if (n == 0) return FL_OK;
    FL_CHECK_ARG(pos && ids && out, "fl_ivf_map_ids: null pointer");
    ivf_map_ids_kernel<<<(unsigned)ceil_div(n, 256), 256, 0, (cudaStream_t)stream>>>(pos, ids, n, m, out);
    FL_CHECK_LAUNCH();
    return FL_OK;
}

extern "C" int64_t fl_ivf_build_workspace_bytes(int64_t m, int nlist) {
    if (m < 1 || nlist < 1) return 0;
    return ivf_build_plan(m, nlist).bytes;
}

extern "C" int fl_ivf_build_csr_f32(const float* x, int64_t m, int64_t ldx, int d, const int32_t* labels, int nlist,
                                    float* data, int64_t* ids, int64_t* list_offsets, int32_t* max_list_len,
                                    void* ws, int64_t ws_bytes, void* stream) {
    FL_CHECK_ARG(m >= 1 && d >= 1 && nlist >= 1 && ldx >= d, "fl_ivf_build_csr_f32: bad shape");
    FL_CHECK_ARG(x && labels && data && ids && list_offsets && ws, "fl_ivf_build_csr_f32: null pointer");
    FL_CHECK_ARG(m < (1ll << 31), "fl_ivf_build_csr_f32: more than 2^31 rows");
    const IvfBuildWs w = ivf_build_plan(m, nlist);
    if (ws_bytes < w.bytes) { set_error("fl_ivf_build_csr_f32: workspace %lld < %lld bytes", (long long)ws_bytes, (long long)w.bytes); return FL_EWORKSPACE; }
    cudaStream_t st = (cudaStream_t)stream;
    char* base = static_cast<char*>(ws);
    int* cnt = reinterpret_cast<int*>(base + w.off_cnt);
    int* total = reinterpret_cast<int*>(base + w.off_total);
    int64_t* pos = reinterpret_cast<int64_t*>(base + w.off_pos);
    FL_CHECK_CUDA(cudaMemsetAsync(cnt, 0, (size_t)(w.units * nlist) * 4, st));
    ivf_build_count_kernel<<<(unsigned)ceil_div(m, 256), 256, 0, st>>>(labels, m, nlist, w.unit_rows, cnt);
    FL_CHECK_LAUNCH();
    ivf_build_colscan_kernel<<<(unsigned)ceil_div(nlist, 128), 128, 0, st>>>(cnt, w.units, nlist, total);
    FL_CHECK_LAUNCH();
    ivf_build_offsets_kernel<<<1, 1024, 0, st>>>(total, nlist, list_offsets, max_list_len);
    FL_CHECK_LAUNCH();
    ivf_build_rank_kernel<<<(unsigned)ceil_div(w.units, 4), 128, 0, st>>>(labels, m, nlist, w.unit_rows, cnt, list_offsets, pos);
    FL_CHECK_LAUNCH();
    ivf_build_move_kernel<<<(unsigned)ceil_div(m, 8), 256, 0, st>>>(x, m, ldx, d, pos, data, ids);
    FL_CHECK_LAUNCH();
    return FL_OK;
}

extern "C" int64_t fl_ivf_fine_scan_workspace_bytes(int64_t nq, int nprobe, int nlist, int64_t m, int d,
                                                    int k) {
    (void)d;
    if (nq < 1 || nprobe < 1 || nlist < 1 || k < 1 || m < 1) return 0;
    return ivf_ws_plan(nq, nprobe, nlist, m, k).bytes;
}

extern "C" int fl_ivf_fine_scan_f32(const float* q, int64_t nq, int64_t ldq, const float* data, int64_t m,
                                    int64_t ldd, int d, const int64_t* list_offsets, int nlist,
                                    const int32_t* probed, int nprobe, int k, const float* data_hnorm,
                                    float* out_dist, int32_t* out_pos, void* ws, int64_t ws_bytes,
                                    void* stream) {
    FL_CHECK_ARG(nq >= 0 && m >= 1 && d >= 1 && nlist >= 1 && nprobe >= 1 && k >= 1,
                 "fl_ivf_fine_scan_f32: bad shape");
    FL_CHECK_ARG(ldq >= d && ldd >= d, "fl_ivf_fine_scan_f32: leading dimensions smaller than d");
    FL_CHECK_ARG(m < (1ll << 31) && nq * (int64_t)nprobe < (1ll << 31), "fl_ivf_fine_scan_f32: too many rows or pairs");
    if (k > 512) { set_error("fl_ivf_fine_scan_f32: k=%d > 512 is not supported", k); return FL_EUNSUPPORTED; }
    if (nq == 0) return FL_OK;
    FL_CHECK_ARG(q && data && list_offsets && probed && out_dist && out_pos && ws, "fl_ivf_fine_scan_f32: null pointer");
    FL_CHECK_ARG((reinterpret_cast<uintptr_t>(ws) & 255) == 0, "fl_ivf_fine_scan_f32: workspace must be 256-byte aligned");
    const IvfWs w = ivf_ws_plan(nq, nprobe, nlist, m, k);
    if (w.bq == 0) { set_error("fl_ivf_fine_scan_f32: pool does not fit shared memory"); return FL_EUNSUPPORTED; }
    if (ws_bytes < w.bytes) {
        set_error("fl_ivf_fine_scan_f32: workspace %lld < %lld bytes", (long long)ws_bytes, (long long)w.bytes);
        return FL_EWORKSPACE;
    }
    cudaStream_t st = (cudaStream_t)stream;
    char* base = static_cast<char*>(ws);
    int* cnt = reinterpret_cast<int*>(base + w.off_cnt);
    int* pair_off = reinterpret_cast<int*>(base + w.off_pair_off);
    int* item_off = reinterpret_cast<int*>(base + w.off_item_off);
    int* cursor = reinterpret_cast<int*>(base + w.off_cursor);
    int* sorted_pair = reinterpret_cast<int*>(base + w.off_sorted);
    float* part_sc = reinterpret_cast<float*>(base + w.off_part_sc);
    uint32_t* part_id = reinterpret_cast<uint32_t*>(base + w.off_part_id);
    const int64_t npairs = nq * nprobe;

    const float* hnorm = data_hnorm;
    if (!hnorm) {
        float* h = reinterpret_cast<float*>(base + w.off_hnorm);
        ivf_halfnorm_kernel<<<(unsigned)ceil_div(m, 8), 256, 0, st>>>(data, m, d, ldd, h);
        FL_CHECK_LAUNCH();
        hnorm = h;
    }
    FL_CHECK_CUDA(cudaMemsetAsync(cnt, 0, (size_t)(nlist + 1) * 4, st));
    ivf_count_kernel<<<(unsigned)ceil_div(npairs, 256), 256, 0, st>>>(probed, npairs, nlist, cnt);
    FL_CHECK_LAUNCH();
    ivf_scan_kernel<<<1, 1024, 0, st>>>(cnt, nlist, w.bq, list_offsets, pair_off, item_off, cursor);
    FL_CHECK_LAUNCH();
    ivf_scatter_kernel<<<(unsigned)ceil_div(npairs, 256), 256, 0, st>>>(probed, npairs, nlist, pair_off, cursor,
                                                                        sorted_pair);
    FL_CHECK_LAUNCH();
    ivf_fill_kernel<<<(unsigned)ceil_div(npairs * w.K1, 256), 256, 0, st>>>(part_sc, part_id, npairs * w.K1);
    FL_CHECK_LAUNCH();

    SimtKnnParams sp{};
    sp.q = q; sp.ldq = ldq; sp.db = data; sp.m = m; sp.ldb = ldd; sp.d = d; sp.hnorm = hnorm;
    sp.K1 = w.K1; sp.cap = simt_pool_cap(w.K1); sp.npl = sp.cap / 32; sp.keep = simt_pool_keep(w.K1, k); sp.nsplit = 1; sp.rows_per_split = m;
    sp.part_sc = part_sc; sp.part_id = part_id;
    sp.vecq = (ldq % 4 == 0) && ((reinterpret_cast<uintptr_t>(q) & 15) == 0);
    sp.vecd = (ldd % 4 == 0) && ((reinterpret_cast<uintptr_t>(data) & 15) == 0);
    sp.ivf = 1; sp.nlist = nlist; sp.nprobe = nprobe; sp.bq_items = w.bq;
    sp.item_off = item_off; sp.pair_off = pair_off; sp.sorted_pair = sorted_pair;
    sp.list_offsets = list_offsets;
    sp.tau_q = reinterpret_cast<float*>(base + w.off_tau);
    {
        const int rc = launch_fill_f32(sp.tau_q, nq, -INFINITY, st);
        if (rc != FL_OK) return rc;
    }
    profile_begin(st);
    int rc = launch_knn_simt(sp, w.max_items, st);
    profile_end(st);
    if (rc != FL_OK) return rc;

    FinalizeParams fp{};
    fp.q = q; fp.ldq = ldq; fp.count = nq; fp.db = data; fp.m = m; fp.ldb = ldd; fp.d = d;
    fp.vec = sp.vecq && sp.vecd && (d % 4 == 0);
    fp.part_sc = part_sc; fp.part_id = part_id; fp.nsplit = nprobe; fp.K1 = w.K1;
    fp.k = k; fp.rerank = (k + 8 < w.K1) ? k + 8 : w.K1; fp.row_offset = 0;
    fp.out_dist = out_dist; fp.out_idx = out_pos; fp.verify = 0;
    return launch_knn_finalize(fp, nq, st);
}
