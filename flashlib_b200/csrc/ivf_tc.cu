// IVF-Flat fine scan on the tensor-core candidate kernel (knn_tc.cu).
//
// Index side (once per index): a bf16 operand plane of the list-sorted rows in which every
// non-empty list is padded to whole tiles of 256 rows, so a database tile never straddles two
// lists and padding rows can never be candidates (they score -3e38), plus the map from plane
// rows back to data rows.
//
// Search side (per call): the (query, probe) pairs are grouped by list on the device; every
// group of up to 128 pairs of one list becomes one query tile of a gathered bf16 query plane
// and one work item of the scoring kernel: that query tile against the tiles of its list.  The
// kernel publishes a candidate pool and a threshold per gathered row; the finalisation kernel
// (one warp per query) follows the pair -> gathered-row map to the query's nprobe pools, re-scores
// the candidates exactly and proves the result against the scoring error bound.  Queries it
// cannot prove are recomputed by an exact per-query scan of their probed lists.
#include "knn_internal.h"
#include "plane.h"
#include "pool.cuh"
#include <cuda_bf16.h>

namespace fl {

constexpr int IVF_TC_BQ = 128;       // pairs per query tile
constexpr int IVF_TC_TILE = 256;     // database rows per tile

struct IvfPlaneLayout {
    int64_t rows_max;      // plane rows: every list padded to whole tiles
    PlaneLayout pl;        // rows / half norms / max norm, as for a kNN database of rows_max rows
    int64_t off_tile_off;  // i32 [nlist + 1]: first tile of every list (exclusive scan)
    int64_t off_row_map;   // i32 [rows_max]: data row of every plane row, -1 for padding
    int64_t bytes;
};

static IvfPlaneLayout ivf_plane_layout(int64_t m, int nlist, int d) {
    IvfPlaneLayout L{};
    L.rows_max = round_up(m + (int64_t)(IVF_TC_TILE - 1) * nlist, IVF_TC_TILE);
    L.pl = plane_layout(L.rows_max, d);
    L.off_tile_off = L.pl.bytes;
    L.off_row_map = L.off_tile_off + round_up((int64_t)(nlist + 1) * 4, 1024);
    L.bytes = L.off_row_map + round_up(L.rows_max * 4, 1024);
    return L;
}

// Single block: exclusive scan of the tiles per list.
__global__ void __launch_bounds__(1024) ivf_tile_scan_kernel(const int64_t* __restrict__ list_offsets, int nlist,
                                                             int* __restrict__ tile_off) {
    __shared__ int s_t[1024];
    __shared__ int carry;
    const int t = threadIdx.x;
    if (t == 0) carry = 0;
    __syncthreads();
    for (int base = 0; base < nlist; base += 1024) {
        const int c = base + t;
        int nt = 0;
        if (c < nlist) nt = (int)((list_offsets[c + 1] - list_offsets[c] + IVF_TC_TILE - 1) / IVF_TC_TILE);
        s_t[t] = nt;
        __syncthreads();
        for (int o = 1; o < 1024; o <<= 1) {
            const int a = t >= o ? s_t[t - o] : 0;
            __syncthreads();
            s_t[t] += a;
            __syncthreads();
        }
        if (c < nlist) tile_off[c] = carry + s_t[t] - nt;
        __syncthreads();
        if (t == 1023) carry += s_t[t];
        __syncthreads();
    }
    if (t == 0) tile_off[nlist] = carry;
}

// One block per list: data row of every plane row of the list (row_map is pre-filled with -1).
__global__ void ivf_row_map_kernel(const int64_t* __restrict__ list_offsets, const int* __restrict__ tile_off,
                                   int* __restrict__ row_map) {
    const int c = blockIdx.x;
    const int64_t r0 = list_offsets[c];
    const int len = (int)(list_offsets[c + 1] - r0);
    const int64_t p0 = (int64_t)tile_off[c] * IVF_TC_TILE;
    for (int r = threadIdx.x; r < len; r += blockDim.x) row_map[p0 + r] = (int)(r0 + r);
}

// One warp per plane row: bf16 features, the split -||x||^2/2 columns, half norm, max norm.
__global__ void ivf_plane_rows_kernel(const float* __restrict__ data, int64_t ld, int d, const int* __restrict__ row_map,
                                      int64_t rows_max, __nv_bfloat16* __restrict__ rows, float* __restrict__ hnorm,
                                      unsigned int* __restrict__ maxnorm_bits, int d_pad) {
    const int lane = threadIdx.x & 31;
    const int64_t row = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (row >= rows_max) return;
    const int pitch = d_pad + PLANE_AUG_COLS;
    __nv_bfloat16* o = rows + row * pitch;
    const int src = __ldg(row_map + row);
    if (src < 0) {
        for (int c = lane; c < pitch; c += 32) o[c] = __float2bfloat16_rn(c == d_pad ? -3.0e38f : 0.f);
        if (lane == 0) hnorm[row] = pos_inf();
        return;
    }
    const float* p = data + (int64_t)src * ld;
    float s = 0.f;
    for (int c = lane; c < d_pad; c += 32) {
        const float v = (c < d) ? __ldg(p + c) : 0.f;
        s += v * v;
        o[c] = __float2bfloat16_rn(v);
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
        o[d_pad + lane] = lane == 0 ? h1 : lane == 1 ? h2 : lane == 2 ? h3 : __float2bfloat16_rn(0.f);
    }
}

// One block per list: the work items of the list (groups of IVF_TC_BQ of its pairs), the pair
// of every gathered query row and the gathered row of every pair (pair_row is pre-filled with -1).
__global__ void ivf_tc_items_kernel(const int* __restrict__ cnt, const int* __restrict__ pair_off,
                                    const int* __restrict__ item_off, const int* __restrict__ sorted_pair,
                                    const int* __restrict__ tile_off, int nlist, int* __restrict__ item_t0,
                                    int* __restrict__ item_t1, int* __restrict__ grow, int* __restrict__ pair_row,
                                    int* __restrict__ live_rows) {
    const int c = blockIdx.x;
    if (c == 0 && threadIdx.x == 0) *live_rows = item_off[nlist] * IVF_TC_BQ;
    const int n = cnt[c];
    const int t0 = tile_off[c], t1 = tile_off[c + 1];
    if (n == 0 || t1 == t0) return;     // nobody probes the list, or it has no rows (no item: ivf_scan_kernel)
    const int items = (n + IVF_TC_BQ - 1) / IVF_TC_BQ;
    for (int g = 0; g < items; ++g) {
        const int item = item_off[c] + g;
        if (threadIdx.x == 0) { item_t0[item] = t0; item_t1[item] = t1; }
        for (int j = threadIdx.x; j < IVF_TC_BQ; j += blockDim.x) {
            const int idx = g * IVF_TC_BQ + j;
            const int pair = idx < n ? sorted_pair[pair_off[c] + idx] : -1;
            grow[item * IVF_TC_BQ + j] = pair;
            if (pair >= 0) pair_row[pair] = item * IVF_TC_BQ + j;
        }
    }
}

// Order in which the scoring kernel deals the items to its CTAs: longest list ranges first, so that the
// round-robin deal gives every CTA a similar number of tiles (list lengths spread over a factor of
// five around their mean).  An item's place is the number of items that come before it (more tiles, or
// as many and a smaller index): eight threads per item count over an eighth of the table each, 32 items
// per block.  Entries past the live items count -1 tiles, come last and are never visited.
constexpr int IVF_ORDER_MAX = 4096;
__global__ void __launch_bounds__(256) ivf_tc_item_order_kernel(const int* __restrict__ item_t0, const int* __restrict__ item_t1,
                                                                const int* __restrict__ live_rows, int max_items,
                                                                int* __restrict__ order) {
    __shared__ int s_key[IVF_ORDER_MAX];
    const int n_items = *live_rows / IVF_TC_BQ;
    for (int i = threadIdx.x; i < max_items; i += 256) s_key[i] = i < n_items ? item_t1[i] - item_t0[i] : -1;
    __syncthreads();
    const int i = blockIdx.x * 32 + (threadIdx.x >> 3), sub = threadIdx.x & 7;
    const bool mine = i < max_items;
    const int ki = mine ? s_key[i] : 0;
    int place = 0;
    if (mine) {
        for (int j = sub; j < max_items; j += 8) {
            const int kj = s_key[j];
            place += (kj > ki || (kj == ki && j < i)) ? 1 : 0;
        }
    }
    place += __shfl_xor_sync(FULL_MASK, place, 1);
    place += __shfl_xor_sync(FULL_MASK, place, 2);
    place += __shfl_xor_sync(FULL_MASK, place, 4);
    if (mine && sub == 0) order[place] = i;
}

// One warp per gathered query row (grid-stride over the live rows): the bf16 row of the pair's
// query with ones in the norm columns and a -inf starting threshold; rows without a pair are
// zero and get a +inf threshold, so nothing is ever a candidate for them.
__global__ void ivf_tc_gather_kernel(const float* __restrict__ q, int64_t ldq, int d, int nprobe,
                                     const int* __restrict__ grow, const int* __restrict__ live_rows,
                                     __nv_bfloat16* __restrict__ qplane, float* __restrict__ tau,
                                     int* __restrict__ row_query, int d_pad) {
    const int lane = threadIdx.x & 31;
    const int pitch = d_pad + PLANE_AUG_COLS;
    const int live = *live_rows;
    const int nwarps = (gridDim.x * blockDim.x) >> 5;
    for (int r = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; r < live; r += nwarps) {
        const int pair = grow[r];
        __nv_bfloat16* o = qplane + (int64_t)r * pitch;
        if (pair < 0) {
            for (int c = lane; c < pitch; c += 32) o[c] = __float2bfloat16_rn(0.f);
            if (lane == 0) { tau[r] = pos_inf(); row_query[r] = -1; }
            continue;
        }
        const float* src = q + (int64_t)(pair / nprobe) * ldq;
        for (int c = lane; c < d_pad; c += 32) o[c] = __float2bfloat16_rn(c < d ? __ldg(src + c) : 0.f);
        if (lane < PLANE_AUG_COLS) o[d_pad + lane] = __float2bfloat16_rn(lane < 3 ? 1.f : 0.f);
        if (lane == 0) { tau[r] = neg_inf(); row_query[r] = pair / nprobe; }
    }
}

// Starting threshold of every query from the seeding pass.  The pass left, for every gathered row
// (= one (query, probed list) pair), the 32 class maxima of the first tiles of that list: disjoint
// sets of rows, and the lists of one query are disjoint too.  One warp per query folds its pairs'
// maxima into the 32 largest and takes the `rank`-th: at least `rank` >= k rows of the probed
// lists score that much.  The threshold is that score lowered by twice the scoring error bound
// (plus the fp32 slack): the k best exact distances then lie below the bound the finalisation
// derives from the threshold, so its proof holds for every query whose pools never overflow --
// a threshold without the margin would cut closer to the k-th neighbour than the proof can see.
__global__ void __launch_bounds__(128) ivf_tc_seed_select_kernel(const float* __restrict__ seed_cls,
                                                                 const int* __restrict__ pair_row, int64_t nq, int nprobe,
                                                                 int rank, const float* __restrict__ q, int64_t ldq, int d,
                                                                 const float* __restrict__ maxnorm, float eps_rel,
                                                                 float* __restrict__ tau_q) {
    const int lane = threadIdx.x & 31;
    const int64_t qi = (int64_t)blockIdx.x * 4 + (threadIdx.x >> 5);
    if (qi >= nq) return;
    float pick;
    if (nprobe <= 16) {
        // lane = class: every lane holds its class maximum of up to 16 pairs; `rank` rounds each
        // take the largest value left in the warp away from the lane that holds it
        float v[16];
#pragma unroll
        for (int j = 0; j < 16; ++j) {
            const int r = j < nprobe ? __ldg(pair_row + qi * nprobe + j) : -1;
            v[j] = r >= 0 ? __ldg(seed_cls + (int64_t)r * 32 + lane) : neg_inf();
        }
        pick = neg_inf();
        for (int round = 0; round < rank; ++round) {
            float m = v[0];
#pragma unroll
            for (int j = 1; j < 16; ++j) m = fmaxf(m, v[j]);
            float wmax = m;
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) wmax = fmaxf(wmax, __shfl_xor_sync(FULL_MASK, wmax, o));
            pick = wmax;
            if (!(wmax > neg_inf())) break;            // fewer than `rank` rows were sampled
            const unsigned owners = __ballot_sync(FULL_MASK, m == wmax);
            if (lane == __ffs(owners) - 1) {
                bool gone = false;                     // one copy only: equal scores are different rows
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                    const bool hit = !gone && v[j] == wmax;
                    v[j] = hit ? neg_inf() : v[j];
                    gone = gone || hit;
                }
            }
        }
    } else {
        float key[1] = {neg_inf()};
        uint32_t id[1] = {0};
        for (int j = 0; j < nprobe; ++j) {
            const int r = __ldg(pair_row + qi * nprobe + j);
            if (r < 0) continue;                       // the list has no rows (no work item, no maxima)
            float kin[1] = {__ldg(seed_cls + (int64_t)r * 32 + lane)};
            uint32_t iin[1] = {0};
            warp_sort_desc<1, false>(kin, iin);
            warp_merge_desc<1, false>(key, id, kin, iin);
        }
        pick = __shfl_sync(FULL_MASK, key[0], rank - 1);     // -inf while fewer than `rank` rows were sampled
    }
    float qsq = 0.f;
    for (int c = lane; c < d; c += 32) { const float v = __ldg(q + qi * ldq + c); qsq += v * v; }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) qsq += __shfl_xor_sync(FULL_MASK, qsq, o);
    const float mn = __ldg(maxnorm);
    if (pick > neg_inf()) pick -= 2.f * eps_rel * sqrtf(qsq) * mn + 1e-5f * (qsq + mn * mn);
    if (lane == 0) tau_q[qi] = pick;
}

// Finalisation of the inverted-file scan: one warp per query.
//
// The scoring pass left, per gathered row (= (query, probed list) pair) and warpgroup, a pool of up
// to IVF_POOL (score, plane row) pairs in global memory with its entry count and final threshold;
// every row of the query's probed lists that is in no pool scored at most u = the largest of those
// thresholds.  The warp collects the entries above u, sorts them by score, re-scores them in that
// order with exact fp32 sum (q - x)^2 and stops once k exact distances lie below the lower bound that
// the next score puts on everything not yet re-scored; the result is the k rows of least exact
// distance, ordered by (distance, row).  When more than IVF_LIST entries lie above u a floor keeps
// the best few dozen (what it drops counts as not re-scored).  A query whose proof fails, or whose
// pools hold more than IVF_GATHER entries, is queued for the exact scan.
constexpr int IVF_POOL = 64, IVF_LIST = 256, IVF_GATHER = 1024;

template <int NPL>
__device__ __forceinline__ void ivf_rerank(const float* __restrict__ s_sc, const uint32_t* __restrict__ s_id, int total,
                                           const float* __restrict__ qp, const float* __restrict__ data, int64_t ldd, int d,
                                           int vec, int k, float u, float qsq, float eps, float slack, float* out_dist,
                                           int32_t* out_pos, bool& proven) {
    const int lane = threadIdx.x & 31;
    float key[NPL];
    uint32_t id[NPL];
#pragma unroll
    for (int r = 0; r < NPL; ++r) {
        const int e = (r << 5) | lane;
        key[r] = e < total ? s_sc[e] : neg_inf();
        id[r] = e < total ? s_id[e] : INVALID_ID;
    }
    warp_sort_desc<NPL, false>(key, id);
    float bound = u;
    bool stop = false;
    float dist[NPL];
#pragma unroll
    for (int r = 0; r < NPL; ++r) dist[r] = pos_inf();
#pragma unroll
    for (int r = 0; r < NPL; ++r) {
        for (int l0 = 0; l0 < 32; l0 += 4) {
            if (stop || (r << 5) + l0 >= total) break;
            if ((l0 & 7) == 0 && (r << 5) + l0 >= ((k + 7) & ~7)) {
                const float nxt = __shfl_sync(FULL_MASK, key[r], l0);
                const float T = qsq - 2.f * (fmaxf(nxt, u) + eps) - slack;
                int below = 0;
#pragma unroll
                for (int rr = 0; rr < NPL; ++rr) below += __popc(__ballot_sync(FULL_MASK, dist[rr] < T));
                if (below >= k) { stop = true; bound = fmaxf(u, nxt); break; }
            }
            uint32_t cid[4];
            float a[4];
#pragma unroll
            for (int t = 0; t < 4; ++t) {
                cid[t] = __shfl_sync(FULL_MASK, id[r], l0 + t);
                a[t] = 0.f;
            }
            if (vec) {
                for (int c = lane * 4; c < d; c += 128) {
                    const float4 qv = __ldg(reinterpret_cast<const float4*>(qp + c));
#pragma unroll
                    for (int t = 0; t < 4; ++t) {
                        if (cid[t] != INVALID_ID) {
                            const float4 xv = __ldg(reinterpret_cast<const float4*>(data + (int64_t)cid[t] * ldd + c));
                            const float d0 = qv.x - xv.x, d1 = qv.y - xv.y, d2 = qv.z - xv.z, d3 = qv.w - xv.w;
                            a[t] += d0 * d0 + d1 * d1 + d2 * d2 + d3 * d3;
                        }
                    }
                }
            } else {
                for (int c = lane; c < d; c += 32) {
                    const float qv = __ldg(qp + c);
#pragma unroll
                    for (int t = 0; t < 4; ++t) {
                        if (cid[t] != INVALID_ID) {
                            const float df = qv - __ldg(data + (int64_t)cid[t] * ldd + c);
                            a[t] += df * df;
                        }
                    }
                }
            }
#pragma unroll
            for (int t = 0; t < 4; ++t) {
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) a[t] += __shfl_xor_sync(FULL_MASK, a[t], o);
                if (lane == l0 + t && cid[t] != INVALID_ID) dist[r] = a[t];
            }
        }
    }
    float k2[NPL];
    uint32_t id2[NPL];
#pragma unroll
    for (int r = 0; r < NPL; ++r) {
        const bool ok = dist[r] < pos_inf();
        k2[r] = ok ? -dist[r] : neg_inf();
        id2[r] = ok ? id[r] : INVALID_ID;
    }
    warp_sort_desc<NPL, true>(k2, id2);
    float dk = pos_inf();
#pragma unroll
    for (int r = 0; r < NPL; ++r) {
        if (((k - 1) >> 5) == r) {
            const float v = __shfl_sync(FULL_MASK, k2[r], (k - 1) & 31);
            dk = (v > neg_inf()) ? -v : pos_inf();
        }
    }
    // every row that was not re-scored has a score <= bound: its distance is at least qsq - 2 (bound + eps)
    proven = bound == neg_inf() || dk < qsq - 2.f * (bound + eps) - slack;
#pragma unroll
    for (int r = 0; r < NPL; ++r) {
        const int e = (r << 5) | lane;
        if (e < k) {
            const bool ok = id2[r] != INVALID_ID;
            out_dist[e] = ok ? -k2[r] : pos_inf();
            out_pos[e] = ok ? (int32_t)id2[r] : -1;
        }
    }
}

__global__ void __launch_bounds__(128) ivf_tc_finalize_kernel(
    const float* __restrict__ q, int64_t nq, int64_t ldq, int d, int vec, const float* __restrict__ data, int64_t ldd,
    const int* __restrict__ pair_row, int nprobe, const float2* __restrict__ pools, const int* __restrict__ pool_cnt,
    const float* __restrict__ pool_tau, const int* __restrict__ row_map, int64_t rows_max, int k, float eps_rel,
    const float* __restrict__ maxnorm, float* __restrict__ out_dist, int32_t* __restrict__ out_pos, int* fb_count,
    int* fb_list) {
    __shared__ float s_sc[4][IVF_GATHER];
    __shared__ uint32_t s_id[4][IVF_GATHER];
    __shared__ int s_poff[4][32];
    __shared__ int s_pool[4][32];
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    const int64_t qi = (int64_t)blockIdx.x * 4 + w;
    if (qi >= nq) return;
    const float* qp = q + qi * ldq;
    float qsq = 0.f;
    for (int c = lane; c < d; c += 32) { const float v = __ldg(qp + c); qsq += v * v; }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) qsq += __shfl_xor_sync(FULL_MASK, qsq, o);
    const float mn = __ldg(maxnorm);
    const float eps = eps_rel * sqrtf(qsq) * mn;
    const float slack = 1e-5f * (qsq + mn * mn);

    // Gather: 32 pools at a time, one pool per lane for the bookkeeping (gathered row, entry count,
    // threshold: independent loads), then the pools' entries are copied to the warp's list at
    // the offsets a prefix sum of the counts gives, 32 entries per round trip whatever pool they sit in.
    float u = neg_inf();
    int total = 0;
    bool overflow = false;
    for (int base = 0; base < 2 * nprobe; base += 32) {
        const int pi = base + lane;
        int r = -1, n = 0;
        if (pi < 2 * nprobe) r = __ldg(pair_row + qi * nprobe + (pi >> 1));
        if (r >= 0) {
            n = __ldg(pool_cnt + (int64_t)r * 2 + (pi & 1));
            n = n < IVF_POOL ? n : IVF_POOL;
            u = fmaxf(u, __ldg(pool_tau + (int64_t)r * 2 + (pi & 1)));
        }
        int off = n;                                  // inclusive prefix sum of the counts
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const int t = __shfl_up_sync(FULL_MASK, off, o);
            if (lane >= o) off += t;
        }
        const int chunk_total = __shfl_sync(FULL_MASK, off, 31);
        off += total - n;                             // exclusive, from the list's start
        if (total + chunk_total > IVF_GATHER) { overflow = true; break; }
        // The lanes share the chunk's entries evenly (a pool holds a handful of entries, so a loop over the
        // pools would spend one memory round trip per pool): entry idx of the list belongs to the last
        // pool whose offset is <= idx (empty pools share the offset of the next one and sort before it).
        s_poff[w][lane] = off;
        s_pool[w][lane] = (int)(r >= 0 ? r * 2 + (pi & 1) : 0);
        __syncwarp();
        for (int idx = total + lane; idx < total + chunk_total; idx += 32) {
            int lo = 0, hi = 31;
            while (lo < hi) {
                const int mid = (lo + hi + 1) >> 1;
                if (s_poff[w][mid] <= idx) lo = mid; else hi = mid - 1;
            }
            const float2 v = pools[(int64_t)s_pool[w][lo] * IVF_POOL + (idx - s_poff[w][lo])];
            s_sc[w][idx] = v.x;
            s_id[w][idx] = __float_as_uint(v.y);
        }
        __syncwarp();
        total += chunk_total;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) u = fmaxf(u, __shfl_xor_sync(FULL_MASK, u, o));
    __syncwarp();
    bool proven = false;
    float* od = out_dist + qi * k;
    int32_t* op = out_pos + qi * k;
    if (!overflow) {
        // plane rows -> data rows (padding rows and entries at or below u drop out), and, when more
        // than IVF_LIST entries are left, a floor f0 that keeps about the best (k + 14) x a few:
        // the (k+14)-th largest of the 32 lane maxima, as in the kNN finalisation
        float lmax = neg_inf();
        for (int e = lane; e < total; e += 32) {
            const uint32_t raw = s_id[w][e];
            int mapped = -1;
            if (s_sc[w][e] > u && raw < (uint32_t)rows_max) mapped = __ldg(row_map + raw);
            s_id[w][e] = mapped >= 0 ? (uint32_t)mapped : INVALID_ID;
            if (mapped < 0) s_sc[w][e] = neg_inf(); else lmax = fmaxf(lmax, s_sc[w][e]);
        }
        __syncwarp();
        float cut = u;
        if (total > IVF_LIST) {
            int rank = 0;
#pragma unroll
            for (int j = 0; j < 32; ++j) {
                const float o = __shfl_sync(FULL_MASK, lmax, j);
                rank += (o > lmax || (o == lmax && j < lane)) ? 1 : 0;
            }
            const int want = k + 14 < 32 ? k + 14 : 32;
            const unsigned sel = __ballot_sync(FULL_MASK, rank == want - 1);
            cut = fmaxf(u, __shfl_sync(FULL_MASK, lmax, __ffs(sel) - 1));
        }
        // compact the list in place to the entries above the cut (cut == u: drops only the invalid ones)
        const unsigned lt = (1u << lane) - 1u;
        int kept = 0;
        for (int e0 = 0; e0 < total; e0 += 32) {
            const int e = e0 + lane;
            float sc = neg_inf();
            uint32_t id = INVALID_ID;
            if (e < total) { sc = s_sc[w][e]; id = s_id[w][e]; }
            const bool keep = id != INVALID_ID && (cut == u ? true : sc >= cut);
            const unsigned mask = __ballot_sync(FULL_MASK, keep);
            __syncwarp();
            if (keep) { const int pos = kept + __popc(mask & lt); s_sc[w][pos] = sc; s_id[w][pos] = id; }   // pos <= e
            kept += __popc(mask);
            __syncwarp();
        }
        if (kept <= IVF_LIST) {
            // rows dropped by the floor scored below it: they count as "not re-scored"
            const float bound0 = cut;
            if (kept <= 64) ivf_rerank<2>(s_sc[w], s_id[w], kept, qp, data, ldd, d, vec, k, bound0, qsq, eps, slack, od, op, proven);
            else if (kept <= 128) ivf_rerank<4>(s_sc[w], s_id[w], kept, qp, data, ldd, d, vec, k, bound0, qsq, eps, slack, od, op, proven);
            else ivf_rerank<8>(s_sc[w], s_id[w], kept, qp, data, ldd, d, vec, k, bound0, qsq, eps, slack, od, op, proven);
        }
    }
    if (!proven && lane == 0) fb_list[atomicAdd(fb_count, 1)] = (int)qi;      // the list holds every query
}

// Exact scan for the queries the proof rejected: a block walks the rows of a listed query's probed
// lists (four rows per warp and step, fp32 sum (q - x)^2 with the summation order of the finalisation
// kernel), collects rows closer than the running k-th distance and compacts the collection with a
// block sort whenever it is half full.  With fewer listed queries than blocks a query's lists are
// dealt to several blocks (`parts`); each leaves its k best in `scratch` and the last one to finish
// (a ticket per query in `done`, zeroed by the caller) merges them.
constexpr int IVFX_THREADS = 256, IVFX_CAP = 4096, IVFX_CHUNK = 2048;
__global__ void __launch_bounds__(IVFX_THREADS) ivf_exact_query_kernel(
    const float* __restrict__ q, int64_t ldq, const float* __restrict__ data, int64_t ldd, int d, int vec,
    const int64_t* __restrict__ list_offsets, int nlist, const int32_t* __restrict__ probed, int nprobe, int k,
    const int* __restrict__ fb_list, const int* __restrict__ fb_count, float* __restrict__ out_dist,
    int32_t* __restrict__ out_pos, float2* __restrict__ scratch, int* __restrict__ done) {
    __shared__ float s_key[IVFX_CAP];       // -distance: the block sort puts larger keys first
    __shared__ uint32_t s_id[IVFX_CAP];
    __shared__ __align__(16) float s_q[512];
    __shared__ int s_n;
    __shared__ float s_T;
    __shared__ int s_last;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int count = *fb_count;
    const int G = (int)gridDim.x;
    int parts = 1;
    if (count > 0 && count < G) { parts = G / count; if (parts > nprobe) parts = nprobe; if (parts > 16) parts = 16; }
    const int items = count * parts;        // parts > 1: items <= G, one item per block
    for (int item = blockIdx.x; item < items; item += G) {
        const int slot = item / parts, part = item - slot * parts;
        const int qi = fb_list[slot];
        __syncthreads();
        for (int c = tid; c < d; c += IVFX_THREADS) s_q[c] = __ldg(q + (int64_t)qi * ldq + c);
        if (tid == 0) { s_n = 0; s_T = pos_inf(); }
        __syncthreads();
        auto compact = [&]() {
            // all threads; keeps the k best, tightens the threshold
            const int n = s_n;
            int P = 32;
            while (P < n) P <<= 1;
            for (int i = n + tid; i < P; i += IVFX_THREADS) { s_key[i] = neg_inf(); s_id[i] = INVALID_ID; }
            block_sort_desc<IVFX_THREADS>(s_key, s_id, P);
            if (tid == 0) {
                s_n = n < k ? n : k;
                if (n >= k) s_T = -s_key[k - 1];
            }
            __syncthreads();
        };
        for (int j = part; j < nprobe; j += parts) {
            const int c = probed[(int64_t)qi * nprobe + j];
            if (c < 0 || c >= nlist) continue;
            const int64_t r0 = list_offsets[c], r1 = list_offsets[c + 1];
            for (int64_t base = r0; base < r1; base += IVFX_CHUNK) {
                const int64_t end = base + IVFX_CHUNK < r1 ? base + IVFX_CHUNK : r1;
                const float T = s_T;
                // four rows per warp and step: a lone block is bound by load latency, so the loads of
                // four rows are in flight together
                constexpr int RW = 4;
                for (int64_t r = base + warp * RW; r < end; r += (IVFX_THREADS / 32) * RW) {
                    float a[RW];
#pragma unroll
                    for (int u = 0; u < RW; ++u) a[u] = 0.f;
                    if (vec) {
                        for (int t = lane * 4; t < d; t += 128) {
                            const float4 qv = *reinterpret_cast<const float4*>(s_q + t);
                            float4 xv[RW];
#pragma unroll
                            for (int u = 0; u < RW; ++u)
                                xv[u] = r + u < end ? __ldg(reinterpret_cast<const float4*>(data + (r + u) * ldd + t)) : qv;
#pragma unroll
                            for (int u = 0; u < RW; ++u) {
                                const float d0 = qv.x - xv[u].x, d1 = qv.y - xv[u].y, d2 = qv.z - xv[u].z, d3 = qv.w - xv[u].w;
                                a[u] += d0 * d0 + d1 * d1 + d2 * d2 + d3 * d3;
                            }
                        }
                    } else {
                        for (int t = lane; t < d; t += 32) {
                            const float qv = s_q[t];
                            float xv[RW];
#pragma unroll
                            for (int u = 0; u < RW; ++u) xv[u] = r + u < end ? __ldg(data + (r + u) * ldd + t) : qv;
#pragma unroll
                            for (int u = 0; u < RW; ++u) { const float df = qv - xv[u]; a[u] += df * df; }
                        }
                    }
#pragma unroll
                    for (int u = 0; u < RW; ++u) {
#pragma unroll
                        for (int o = 16; o > 0; o >>= 1) a[u] += __shfl_xor_sync(FULL_MASK, a[u], o);
                        if (lane == 0 && r + u < end && a[u] <= T) {
                            const int pos = atomicAdd(&s_n, 1);
                            s_key[pos] = -a[u];          // <= IVFX_CHUNK appends per chunk, <= IVFX_CHUNK kept before it
                            s_id[pos] = (uint32_t)(r + u);
                        }
                    }
                }
                __syncthreads();
                const int n_now = s_n;      // read by every thread before anyone appends again
                __syncthreads();
                if (n_now > IVFX_CAP - IVFX_CHUNK) compact();
            }
        }
        __syncthreads();
        compact();
        if (parts > 1) {
            // leave this part's k best for the merge; the last block of the query does it
            const int n = s_n;
            for (int e = tid; e < k; e += IVFX_THREADS)
                scratch[(int64_t)item * k + e] = e < n ? make_float2(s_key[e], __uint_as_float(s_id[e]))
                                                       : make_float2(neg_inf(), __uint_as_float(INVALID_ID));
            __threadfence();
            __syncthreads();
            if (tid == 0) s_last = atomicAdd(done + slot, 1) == parts - 1;
            __syncthreads();
            if (!s_last) continue;
            __threadfence();
            const int total = parts * k;            // <= 16 * 16
            for (int e = tid; e < total; e += IVFX_THREADS) {
                const float2 v = __ldcg(scratch + (int64_t)slot * parts * k + e);
                s_key[e] = v.x;
                s_id[e] = __float_as_uint(v.y);
            }
            if (tid == 0) s_n = total;
            __syncthreads();
            compact();
            // (padding entries carry -inf keys: they sort last and count as absent below)
        }
        const int n = s_n;
        for (int e = tid; e < k; e += IVFX_THREADS) {
            const bool have = e < n && s_id[e] != INVALID_ID;
            out_dist[(int64_t)qi * k + e] = have ? -s_key[e] : pos_inf();
            out_pos[(int64_t)qi * k + e] = have ? (int32_t)s_id[e] : -1;
        }
    }
}

struct IvfTcWs {
    int64_t npairs, max_items, cap_rows; int d_pad, pitch;
    int64_t off_cnt, off_pair_off, off_item_off, off_cursor, off_sorted, off_pair_row, off_item_t0, off_item_t1,
        off_grow, off_row_query, off_tau_q, off_counters, off_qplane, off_tau, off_seed_cls, off_pools, off_part_cnt, off_part_tau, off_fblist,
        off_x_scratch, off_x_done, off_item_order, bytes;
};

static int64_t take(int64_t& cur, int64_t bytes) {
    const int64_t o = cur;
    cur += round_up(bytes > 0 ? bytes : 1, 1024);
    return o;
}

static IvfTcWs ivf_tc_plan(int64_t nq, int nprobe, int nlist, int d, int k) {
    IvfTcWs w{};
    w.npairs = nq * nprobe;
    w.max_items = ceil_div(w.npairs, IVF_TC_BQ) + nlist;
    w.cap_rows = w.max_items * IVF_TC_BQ;
    w.d_pad = (int)round_up(d, 64);
    w.pitch = w.d_pad + PLANE_AUG_COLS;
    (void)k;
    int64_t cur = 0;
    w.off_cnt = take(cur, (int64_t)(nlist + 1) * 4);
    w.off_pair_off = take(cur, (int64_t)(nlist + 1) * 4);
    w.off_item_off = take(cur, (int64_t)(nlist + 1) * 4);
    w.off_cursor = take(cur, (int64_t)(nlist + 1) * 4);
    w.off_sorted = take(cur, w.npairs * 4);
    w.off_pair_row = take(cur, w.npairs * 4);
    w.off_item_t0 = take(cur, w.max_items * 4);
    w.off_item_t1 = take(cur, w.max_items * 4);
    w.off_grow = take(cur, w.cap_rows * 4);
    w.off_row_query = take(cur, w.cap_rows * 4);
    w.off_tau_q = take(cur, nq * 4);
    w.off_counters = take(cur, 1024);
    w.off_qplane = take(cur, w.cap_rows * w.pitch * 2);
    w.off_tau = take(cur, w.cap_rows * 4);
    w.off_seed_cls = take(cur, w.cap_rows * 32 * 4);
    w.off_pools = take(cur, w.cap_rows * tc_taus_per_range() * tc_pair_pool_cap() * 8);
    w.off_part_cnt = take(cur, w.cap_rows * tc_taus_per_range() * 4);
    w.off_part_tau = take(cur, w.cap_rows * tc_taus_per_range() * 4);
    w.off_fblist = take(cur, nq * 4);
    // exact pass over a handful of queries: per-block partial results and a ticket per query
    w.off_x_scratch = take(cur, (int64_t)2 * sm_count() * 16 * 8);
    w.off_x_done = take(cur, (int64_t)2 * sm_count() * 4);
    w.off_item_order = take(cur, w.max_items * 4);
    w.bytes = cur;
    return w;
}

static int ivf_tc_supported(int64_t nq, int nprobe, int nlist, int64_t m, int d, int k) {
    if (nq < 1 || nprobe < 1 || nlist < 1 || m < 1) return 0;
    if (k > 16 || d > 256) return 0;      // resident query tile + ring: four slots up to 128 features, three up to 256
    if (nq * (int64_t)nprobe >= (1ll << 31) / IVF_TC_BQ || m + (int64_t)IVF_TC_TILE * nlist >= (1ll << 31)) return 0;
    return 1;
}

}  // namespace fl

using namespace fl;

extern "C" int64_t fl_ivf_plane_bytes(int64_t m, int nlist, int d) {
    if (m < 1 || nlist < 1 || d < 1 || d > 256) return 0;
    return ivf_plane_layout(m, nlist, d).bytes;
}

extern "C" int fl_ivf_prepare_f32(const float* data, int64_t m, int64_t ldd, int d, const int64_t* list_offsets,
                                  int nlist, void* plane, int64_t plane_bytes, void* stream) {
    FL_CHECK_ARG(m >= 1 && d >= 1 && nlist >= 1 && ldd >= d, "fl_ivf_prepare_f32: bad shape");
    FL_CHECK_ARG(data && list_offsets && plane, "fl_ivf_prepare_f32: null pointer");
    FL_CHECK_ARG((reinterpret_cast<uintptr_t>(plane) & 255) == 0, "fl_ivf_prepare_f32: plane must be 256-byte aligned");
    if (d > 256) { set_error("fl_ivf_prepare_f32: d=%d > 256 is not supported", d); return FL_EUNSUPPORTED; }
    const IvfPlaneLayout L = ivf_plane_layout(m, nlist, d);
    if (plane_bytes < L.bytes) { set_error("fl_ivf_prepare_f32: plane buffer %lld < %lld bytes", (long long)plane_bytes, (long long)L.bytes); return FL_EWORKSPACE; }
    cudaStream_t st = (cudaStream_t)stream;
    char* base = static_cast<char*>(plane);
    int* tile_off = reinterpret_cast<int*>(base + L.off_tile_off);
    int* row_map = reinterpret_cast<int*>(base + L.off_row_map);
    FL_CHECK_CUDA(cudaMemsetAsync(row_map, 0xFF, (size_t)L.rows_max * 4, st));
    FL_CHECK_CUDA(cudaMemsetAsync(base + L.pl.off_meta, 0, 1024, st));
    ivf_tile_scan_kernel<<<1, 1024, 0, st>>>(list_offsets, nlist, tile_off);
    FL_CHECK_LAUNCH();
    ivf_row_map_kernel<<<(unsigned)nlist, 256, 0, st>>>(list_offsets, tile_off, row_map);
    FL_CHECK_LAUNCH();
    const int wpb = 8;
    ivf_plane_rows_kernel<<<(unsigned)ceil_div(L.rows_max, wpb), wpb * 32, 0, st>>>(
        data, ldd, d, row_map, L.rows_max, reinterpret_cast<__nv_bfloat16*>(base + L.pl.off_rows),
        reinterpret_cast<float*>(base + L.pl.off_hnorm), reinterpret_cast<unsigned int*>(base + L.pl.off_meta),
        L.pl.d_pad);
    FL_CHECK_LAUNCH();
    return FL_OK;
}

extern "C" int64_t fl_ivf_fine_scan_tc_workspace_bytes(int64_t nq, int nprobe, int nlist, int64_t m, int d, int k) {
    if (!ivf_tc_supported(nq, nprobe, nlist, m, d, k)) return 0;
    return ivf_tc_plan(nq, nprobe, nlist, d, k).bytes;
}

extern "C" int fl_ivf_fine_scan_tc_f32(const float* q, int64_t nq, int64_t ldq, const float* data, int64_t m,
                                       int64_t ldd, int d, const int64_t* list_offsets, int nlist,
                                       const int32_t* probed, int nprobe, int k, const void* ivf_plane,
                                       float* out_dist, int32_t* out_pos, void* ws, int64_t ws_bytes,
                                       int32_t* status, void* stream) {
    FL_CHECK_ARG(nq >= 0 && m >= 1 && d >= 1 && nlist >= 1 && nprobe >= 1 && k >= 1, "fl_ivf_fine_scan_tc_f32: bad shape");
    FL_CHECK_ARG(ldq >= d && ldd >= d, "fl_ivf_fine_scan_tc_f32: leading dimensions smaller than d");
    if (nq == 0) return FL_OK;
    if (!ivf_tc_supported(nq, nprobe, nlist, m, d, k)) {
        set_error("fl_ivf_fine_scan_tc_f32: k=%d / d=%d / sizes outside the tensor-core scan (k <= 16, d <= 256)", k, d);
        return FL_EUNSUPPORTED;
    }
    FL_CHECK_ARG(q && data && list_offsets && probed && ivf_plane && out_dist && out_pos && ws, "fl_ivf_fine_scan_tc_f32: null pointer");
    FL_CHECK_ARG((reinterpret_cast<uintptr_t>(ws) & 255) == 0 && (reinterpret_cast<uintptr_t>(ivf_plane) & 255) == 0,
                 "fl_ivf_fine_scan_tc_f32: workspace and plane must be 256-byte aligned");
    const IvfTcWs w = ivf_tc_plan(nq, nprobe, nlist, d, k);
    if (ws_bytes < w.bytes) { set_error("fl_ivf_fine_scan_tc_f32: workspace %lld < %lld bytes", (long long)ws_bytes, (long long)w.bytes); return FL_EWORKSPACE; }
    const IvfPlaneLayout L = ivf_plane_layout(m, nlist, d);
    cudaStream_t st = (cudaStream_t)stream;
    char* base = static_cast<char*>(ws);
    const char* pl = static_cast<const char*>(ivf_plane);
    const int* tile_off = reinterpret_cast<const int*>(pl + L.off_tile_off);
    const int* row_map = reinterpret_cast<const int*>(pl + L.off_row_map);
    int* cnt = reinterpret_cast<int*>(base + w.off_cnt);
    int* pair_off = reinterpret_cast<int*>(base + w.off_pair_off);
    int* item_off = reinterpret_cast<int*>(base + w.off_item_off);
    int* cursor = reinterpret_cast<int*>(base + w.off_cursor);
    int* sorted_pair = reinterpret_cast<int*>(base + w.off_sorted);
    int* pair_row = reinterpret_cast<int*>(base + w.off_pair_row);
    int* item_t0 = reinterpret_cast<int*>(base + w.off_item_t0);
    int* item_t1 = reinterpret_cast<int*>(base + w.off_item_t1);
    int* grow = reinterpret_cast<int*>(base + w.off_grow);
    int* counters = reinterpret_cast<int*>(base + w.off_counters);
    int* live_rows = counters;
    int* fb_count = counters + 64;
    int* fb_list = reinterpret_cast<int*>(base + w.off_fblist);
    float* tau = reinterpret_cast<float*>(base + w.off_tau);
    if (status) FL_CHECK_CUDA(cudaMemsetAsync(status, 0, sizeof(int32_t) * FL_STATUS_WORDS, st));
    FL_CHECK_CUDA(cudaMemsetAsync(counters, 0, 1024, st));
    FL_CHECK_CUDA(cudaMemsetAsync(pair_row, 0xFF, (size_t)w.npairs * 4, st));

    profile_mark(st);      // 0: grouping
    // group the pairs by list, cut every list's pairs into query tiles
    int rc = launch_ivf_group(probed, w.npairs, nlist, IVF_TC_BQ, list_offsets, cnt, pair_off, item_off, cursor,
                              sorted_pair, st);
    if (rc != FL_OK) return rc;
    profile_mark(st);      // 1: item table
    ivf_tc_items_kernel<<<(unsigned)nlist, 128, 0, st>>>(cnt, pair_off, item_off, sorted_pair, tile_off, nlist, item_t0,
                                                        item_t1, grow, pair_row, live_rows);
    FL_CHECK_LAUNCH();
    // item order for the scoring launch (tables of up to 4 096 items; larger ones are dealt in list order)
    int* item_order = nullptr;
    if (w.max_items <= IVF_ORDER_MAX) {
        item_order = reinterpret_cast<int*>(base + w.off_item_order);
        ivf_tc_item_order_kernel<<<(unsigned)((w.max_items + 31) / 32), 256, 0, st>>>(item_t0, item_t1, live_rows,
                                                                                     (int)w.max_items, item_order);
        FL_CHECK_LAUNCH();
    }
    profile_mark(st);      // 2: gathered query plane
    ivf_tc_gather_kernel<<<(unsigned)(8 * sm_count()), 256, 0, st>>>(
        q, ldq, d, nprobe, grow, live_rows, reinterpret_cast<__nv_bfloat16*>(base + w.off_qplane), tau,
        reinterpret_cast<int*>(base + w.off_row_query), w.d_pad);
    FL_CHECK_LAUNCH();
    float* tau_q = reinterpret_cast<float*>(base + w.off_tau_q);

    TcKnnParams tp{};
    tp.qplane = base + w.off_qplane; tp.nq = w.cap_rows; tp.nq_pad = w.cap_rows;
    tp.dbrows = pl + L.pl.off_rows; tp.hnorm = reinterpret_cast<const float*>(pl + L.pl.off_hnorm);
    tp.m = L.rows_max; tp.m_pad = L.pl.m_pad; tp.d_pad = L.pl.d_pad; tp.K1 = tc_deep_pool_size();
    tp.deep_pools = 0;
    tp.nsplit = 1; tp.tiles_per_split = L.pl.m_pad / IVF_TC_TILE;
    tp.pair_pools = base + w.off_pools;                    // pools in global memory, four ring slots
    tp.part_cnt = reinterpret_cast<int*>(base + w.off_part_cnt);
    tp.tau = tau; tp.status = status;
    tp.part_tau = reinterpret_cast<float*>(base + w.off_part_tau);
    tp.k = k;
    tp.nq_dev = live_rows; tp.item_t0 = item_t0; tp.item_t1 = item_t1;
    tp.row_query = reinterpret_cast<const int*>(base + w.off_row_query); tp.tau_q = tau_q;
    profile_begin(st);
    profile_mark(st);      // 3: seeding pass
    // Seeding: the first tile of every (list, query group) item with the branch-free class-maxima
    // epilogue, then one threshold per query that k + 6 rows of its probed lists reach.  Without it
    // every pool starts cold and most of the scan is spent inserting and compacting.
    {
        TcKnnParams sd = tp;
        sd.seed_cls = reinterpret_cast<float*>(base + w.off_seed_cls);
        sd.item_tile_cap = 1;
        rc = launch_knn_tc_seed(sd, st);
        if (rc != FL_OK) return rc;
        const int rank = k + 6 < 32 ? k + 6 : 32;
        profile_mark(st);  // 4: threshold selection
        ivf_tc_seed_select_kernel<<<(unsigned)ceil_div(nq, 4), 128, 0, st>>>(
            sd.seed_cls, pair_row, nq, nprobe, rank, q, ldq, d, reinterpret_cast<const float*>(pl + L.pl.off_meta), 0.004f, tau_q);
        FL_CHECK_LAUNCH();
    }
    profile_mark(st);      // 5: scoring pass
    tp.item_order = item_order;
    rc = launch_knn_tc(tp, st);
    profile_end(st);
    profile_mark(st);      // 6: finalisation
    if (rc != FL_OK) return rc;

    const int vecq = (ldq % 4 == 0) && ((reinterpret_cast<uintptr_t>(q) & 15) == 0);
    const int vecd = (ldd % 4 == 0) && ((reinterpret_cast<uintptr_t>(data) & 15) == 0);
    static_assert(IVF_POOL == 64, "pool geometry of the scoring kernel's global-pool mode");
    const int vec = vecq && vecd && (d % 4 == 0);
    ivf_tc_finalize_kernel<<<(unsigned)ceil_div(nq, 4), 128, 0, st>>>(
        q, nq, ldq, d, vec, data, ldd, pair_row, nprobe, reinterpret_cast<const float2*>(base + w.off_pools), tp.part_cnt,
        tp.part_tau, row_map, L.rows_max, k, 0.004f, reinterpret_cast<const float*>(pl + L.pl.off_meta), out_dist, out_pos,
        fb_count, fb_list);
    FL_CHECK_LAUNCH();
    profile_mark(st);      // 7: exact pass for unproven queries
    rc = launch_fallback_fixup(fb_count, (int)nq, status, tc_deep_pool_size(), st);
    if (rc != FL_OK) return rc;
    FL_CHECK_CUDA(cudaMemsetAsync(base + w.off_x_done, 0, (size_t)2 * sm_count() * 4, st));
    ivf_exact_query_kernel<<<(unsigned)(2 * sm_count()), IVFX_THREADS, 0, st>>>(
        q, ldq, data, ldd, d, vec, list_offsets, nlist, probed, nprobe, k, fb_list, fb_count, out_dist, out_pos,
        reinterpret_cast<float2*>(base + w.off_x_scratch), reinterpret_cast<int*>(base + w.off_x_done));
    FL_CHECK_LAUNCH();
    profile_mark(st);      // 8: end
    return FL_OK;
}
