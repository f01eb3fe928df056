// Pool finalisation kernels (one warp per query slot): templates shared by the two translation units
// that instantiate them (fp32 rows in knn_finalize.cu, 16-bit rows in knn_finalize_rows16.cu).
#pragma once
#include "knn_internal.h"
#include "pool.cuh"

namespace fl {

// ------------------------------------------------------------------------------------
// Finalisation: one warp per query slot.
//
// Input: `nsplit` published pools of K1 (score, row) entries per slot, and (tensor-core path)
// the thresholds of the scoring pass: every row it did not publish scored at most u = the
// largest threshold.  Output: the k rows of least exact fp32 distance among the candidates,
// ordered by (distance, row).  With verification on, the result is accepted only when the k-th
// exact distance lies below qsq - 2 (bound + eps), where `bound` is an upper bound on the
// score of every row that was not re-scored exactly; otherwise the slot is queued for the
// exact path.
//
// Candidates are taken in two attempts.  The first keeps only scores above u (entries at or
// below u can never satisfy the proof) and at or above a floor f0 chosen so that a few dozen
// entries survive, which are sorted once; dropped entries scored at most max(u, f0).  If that
// set cannot be proven (or overflows), the second attempt sorts every pool and merges the K1
// best, with bound = max(u, K1-th best).
// ------------------------------------------------------------------------------------
// F32: the rows are fp32 (the element type is then a compile-time fact of the re-rank loops).
template <int NPL1, bool INDIRECT, bool DYN, bool F32>
__device__ __forceinline__ void finalize_slot(const FinalizeParams& p, const int64_t slot, const int64_t count) {
    const int lane = threadIdx.x & 31;
    const int dt = F32 ? DT_F32 : p.dt;
    const int64_t qi = p.qlist ? (int64_t)p.qlist[slot] : slot;
    const int K1 = p.K1;
    const int nsplit = DYN ? simt_dyn_split(count, p.dyn_bq, p.dyn_blocks, p.m).nsplit : p.nsplit;
    // pool s of this slot: offset of its first entry (negative: the pool does not exist)
    auto pool_base = [&](int s) -> int64_t {
        if (!INDIRECT) return (slot * nsplit + s) * (int64_t)K1;
        const int row = __ldg(p.pool_row + slot * nsplit + s);
        return row >= 0 ? (int64_t)row * K1 : -1;
    };
    // published id -> database row, INVALID_ID for padding rows of the operand plane
    auto real_id = [&](uint32_t raw) -> uint32_t {
        if (!INDIRECT) return raw < (uint32_t)p.m ? raw : INVALID_ID;
        if (raw >= (uint32_t)p.id_bound) return INVALID_ID;
        const int mapped = __ldg(p.id_map + raw);
        return mapped >= 0 ? (uint32_t)mapped : INVALID_ID;
    };
    const float* psc = p.part_sc;
    const uint32_t* pid = p.part_id;

    float u = neg_inf();
    if (p.part_tau != nullptr) {
        const int per_pool = p.ntau / nsplit;
        for (int i = lane; i < p.ntau; i += 32) {
            int64_t t = slot * p.ntau + i;
            if (INDIRECT) {
                const int row = __ldg(p.pool_row + slot * nsplit + i / per_pool);
                t = row >= 0 ? (int64_t)row * per_pool + i % per_pool : -1;
            }
            if (t >= 0) u = fmaxf(u, p.part_tau[t]);
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) u = fmaxf(u, __shfl_xor_sync(FULL_MASK, u, o));
    }

    const void* qp = row_at(p.q, qi, p.ldq, dt);
    float qsq = 0.f;
    if (p.vec) {
        for (int c = lane * 4; c < p.d; c += 128) {
            const float4 v = ld_elem4(qp, c, dt);
            qsq += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
        }
    } else {
        for (int c = lane; c < p.d; c += 32) { const float v = ld_elem(qp, c, dt); qsq += v * v; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) qsq += __shfl_xor_sync(FULL_MASK, qsq, o);
    float eps = 0.f, slack = 0.f;
    if (p.verify) {
        const float mn = __ldg(p.maxnorm);
        eps = p.eps_rel * sqrtf(qsq) * mn;
        slack = 1e-5f * (qsq + mn * mn);
    }

    constexpr bool HAS_FILTER = NPL1 <= 4;
    __shared__ float s_sc[HAS_FILTER ? 4 : 1][HAS_FILTER ? 32 * NPL1 : 1];
    __shared__ uint32_t s_id[HAS_FILTER ? 4 : 1][HAS_FILTER ? 32 * NPL1 : 1];
    const bool try_filter = HAS_FILTER && p.verify && p.part_tau != nullptr && u > neg_inf();

    for (int attempt = try_filter ? 0 : 1; attempt < 2; ++attempt) {
        float key[NPL1];
        uint32_t id[NPL1];
        float bound;
        if (attempt == 0) {
            // Each lane notes the best score it meets; the (k+14)-th largest of the 32 lane maxima
            // is a floor with at least k+14 entries at or above it and, scores being spread evenly
            // over the lanes, rarely more than fit the list.  Pool slots are ordered (best kept
            // entries first), so the slot a lane reads rotates from pool to pool.
            float* wsc = s_sc[HAS_FILTER ? (threadIdx.x >> 5) : 0];
            uint32_t* wid = s_id[HAS_FILTER ? (threadIdx.x >> 5) : 0];
            float lmax = neg_inf();
            // (the pools were written by earlier launches: read-only loads, which the compiler may
            // issue for several pools before the first one is consumed)
#pragma unroll 4
            for (int s = 0; s < nsplit; ++s) {
                const int64_t pb = pool_base(s);
                if (pb < 0) continue;
#pragma unroll
                for (int r = 0; r < NPL1; ++r) {
                    const int e = (r << 5) | ((lane + 5 * s + 16 * r) & 31);
                    const float sc = __ldg(psc + pb + e);
                    // (padding rows of an operand plane score -3e38: no need to look their ids up)
                    if (__ldg(pid + pb + e) != INVALID_ID) lmax = fmaxf(lmax, sc);
                }
            }
            int rank = 0;
#pragma unroll
            for (int j = 0; j < 32; ++j) {
                const float o = __shfl_sync(FULL_MASK, lmax, j);
                rank += (o > lmax || (o == lmax && j < lane)) ? 1 : 0;
            }
            const int want = p.k + 14 < 32 ? p.k + 14 : 32;
            const unsigned sel = __ballot_sync(FULL_MASK, rank == want - 1);
            const float f0 = __shfl_sync(FULL_MASK, lmax, __ffs(sel) - 1);
            const unsigned lt = (1u << lane) - 1u;
            int total = 0;
#pragma unroll 4
            for (int s = 0; s < nsplit; ++s) {
                const int64_t pb = pool_base(s);
                if (pb < 0) continue;
#pragma unroll
                for (int r = 0; r < NPL1; ++r) {
                    const int e = (r << 5) | lane;
                    const float sc = __ldg(psc + pb + e);
                    const bool pass = sc > u && sc >= f0;
                    const uint32_t cid = pass ? real_id(__ldg(pid + pb + e)) : INVALID_ID;
                    const bool keep = pass && cid != INVALID_ID;
                    const unsigned mask = __ballot_sync(FULL_MASK, keep);
                    const int pos = total + __popc(mask & lt);
                    if (keep && pos < 32 * NPL1) { wsc[pos] = sc; wid[pos] = cid; }
                    total += __popc(mask);
                }
            }
            __syncwarp();
            if (total > 32 * NPL1) continue;
#pragma unroll
            for (int r = 0; r < NPL1; ++r) {
                const int e = (r << 5) | lane;
                key[r] = e < total ? wsc[e] : neg_inf();
                id[r] = e < total ? wid[e] : INVALID_ID;
            }
            __syncwarp();
            warp_sort_desc<NPL1, false>(key, id);
            bound = fmaxf(u, f0);
        } else {
            // Every pool is sorted on its own and merged into the running list with one bitonic
            // merge step.  The K1-th kept score covers what this merge dropped.
            float kin[NPL1];
            uint32_t iin[NPL1];
#pragma unroll
            for (int r = 0; r < NPL1; ++r) { key[r] = neg_inf(); id[r] = INVALID_ID; }
            for (int s = 0; s < nsplit; ++s) {
                const int64_t pb = pool_base(s);
                if (pb < 0) continue;
#pragma unroll
                for (int r = 0; r < NPL1; ++r) {
                    const int e = (r << 5) | lane;
                    const uint32_t cid = real_id(pid[pb + e]);
                    const bool real = cid != INVALID_ID;   // padding rows of the operand plane never count
                    kin[r] = real ? psc[pb + e] : neg_inf();
                    iin[r] = real ? cid : INVALID_ID;
                }
                warp_sort_desc<NPL1, false>(kin, iin);
                warp_merge_desc<NPL1, false>(key, id, kin, iin);
            }
            bound = __shfl_sync(FULL_MASK, id[NPL1 - 1], 31) != INVALID_ID
                        ? __shfl_sync(FULL_MASK, key[NPL1 - 1], 31) : neg_inf();
            bound = fmaxf(bound, u);
        }

        // Exact fp32 distances of the first `rerank` entries, best score first.  With
        // verification on, the walk stops as soon as k of the exact distances seen so far lie
        // below the lower bound that the next entry's score (and `bound`) puts on every row not
        // yet re-scored.
        bool stop = false;
        float dist[NPL1];
#pragma unroll
        for (int r = 0; r < NPL1; ++r) dist[r] = pos_inf();
#pragma unroll
        for (int r = 0; r < NPL1; ++r) {
            for (int l0 = 0; l0 < 32; l0 += 4) {
                if (stop || (r << 5) + l0 >= p.rerank) break;
                if (p.verify && (l0 & 7) == 0 && (r << 5) + l0 >= ((p.k + 7) & ~7)) {
                    const float nxt = __shfl_sync(FULL_MASK, key[r], l0);
                    const float T = qsq - 2.f * (fmaxf(nxt, bound) + eps) - slack;
                    int cnt = 0;
#pragma unroll
                    for (int rr = 0; rr < NPL1; ++rr) cnt += __popc(__ballot_sync(FULL_MASK, dist[rr] < T));
                    if (cnt >= p.k) { stop = true; bound = fmaxf(bound, nxt); break; }
                }
                uint32_t cid[4];
                float a[4];
#pragma unroll
                for (int t = 0; t < 4; ++t) {
                    cid[t] = __shfl_sync(FULL_MASK, id[r], l0 + t);
                    if ((r << 5) + l0 + t >= p.rerank) cid[t] = INVALID_ID;
                    a[t] = 0.f;
                }
                if (p.vec) {
                    for (int c = lane * 4; c < p.d; c += 128) {
                        const float4 qv = ld_elem4(qp, c, dt);
#pragma unroll
                        for (int t = 0; t < 4; ++t) {
                            if (cid[t] != INVALID_ID) {
                                const float4 xv = ld_elem4(row_at(p.db, cid[t], p.ldb, dt), c, dt);
                                const float d0 = qv.x - xv.x, d1 = qv.y - xv.y, d2 = qv.z - xv.z,
                                            d3 = qv.w - xv.w;
                                a[t] += d0 * d0 + d1 * d1 + d2 * d2 + d3 * d3;
                            }
                        }
                    }
                } else {
                    for (int c = lane; c < p.d; c += 32) {
                        const float qv = ld_elem(qp, c, dt);
#pragma unroll
                        for (int t = 0; t < 4; ++t) {
                            if (cid[t] != INVALID_ID) {
                                const float df = qv - ld_elem(row_at(p.db, cid[t], p.ldb, dt), c, dt);
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

        // Order by (exact distance, row) ascending.
        float k2[NPL1];
        uint32_t id2[NPL1];
#pragma unroll
        for (int r = 0; r < NPL1; ++r) {
            const bool ok = dist[r] < pos_inf();
            k2[r] = ok ? -dist[r] : neg_inf();
            id2[r] = ok ? id[r] : INVALID_ID;
        }
        warp_sort_desc<NPL1, true>(k2, id2);
        float dk = pos_inf();
#pragma unroll
        for (int r = 0; r < NPL1; ++r) {
            if (((p.k - 1) >> 5) == r) {
                const float v = __shfl_sync(FULL_MASK, k2[r], (p.k - 1) & 31);
                dk = (v > neg_inf()) ? -v : pos_inf();
            }
        }

        // Verification: every row that was not re-scored has a score <= bound, so its exact
        // distance is at least qsq - 2 (bound + eps).
        bool proven = true;
        if (p.verify && bound > neg_inf()) proven = dk < qsq - 2.f * (bound + eps) - slack;
        if (!proven && p.cert_tau != nullptr) proven = bound <= __ldg(p.cert_tau + qi);
        if (!proven && attempt == 0) continue;
#pragma unroll
        for (int r = 0; r < NPL1; ++r) {
            const int e = (r << 5) | lane;
            if (e < p.k) {
                const bool ok = id2[r] != INVALID_ID;
                p.out_dist[qi * p.k + e] = ok ? -k2[r] : pos_inf();
                p.out_idx[qi * p.k + e] = ok ? (int32_t)((int64_t)id2[r] + p.row_offset) : -1;
            }
        }
        if (!proven && lane == 0 && p.fb_count != nullptr) {
            bool queued = false;
            if (p.next_count != nullptr) {
                const int i = atomicAdd(p.next_count, 1);
                if (i < p.next_cap) { p.next_list[i] = (int)qi; queued = true; }
            }
            if (!queued) {
                const int i = atomicAdd(p.fb_count, 1);
                if (i < p.fb_cap) p.fb_list[i] = (int)qi;
            }
        }
        break;
    }
}

// One warp per slot, grid-stride: the slot count may only be known on the device, and a grid
// sized for the largest possible count would mostly launch blocks that have nothing to do.
template <int NPL1, bool INDIRECT, bool DYN, bool F32>
__global__ void __launch_bounds__(128) knn_finalize_kernel(FinalizeParams p) {
    if (p.count_dev == nullptr) {
        // slot count known at launch: one slot per warp
        const int64_t slot = (int64_t)blockIdx.x * 4 + (threadIdx.x >> 5);
        if (slot < p.count) finalize_slot<NPL1, INDIRECT, DYN, F32>(p, slot, p.count);
        return;
    }
    const int64_t count = (int64_t)(*p.count_dev);
    for (int64_t slot = (int64_t)blockIdx.x * 4 + (threadIdx.x >> 5); slot < count; slot += (int64_t)gridDim.x * 4) {
        finalize_slot<NPL1, INDIRECT, DYN, F32>(p, slot, count);
        __syncwarp();
    }
}

// Batch of independent problems (plain pools of a static scan, fp32 or 16-bit rows): problem
// blockIdx.y runs the same code on shifted operands, pools and outputs.
template <int NPL1>
__global__ void __launch_bounds__(128) knn_finalize_batch_kernel(FinalizeParams p) {
    const int64_t b = blockIdx.y;
    p.q = static_cast<const char*>(p.q) + b * p.q_bstride * dt_size_dev(p.dt);
    p.db = static_cast<const char*>(p.db) + b * p.db_bstride * dt_size_dev(p.dt);
    const int64_t pools = p.count * p.nsplit * (int64_t)p.K1;
    p.part_sc += b * pools;
    p.part_id += b * pools;
    p.out_dist += b * p.count * p.k;
    p.out_idx += b * p.count * p.k;
    const int64_t slot = (int64_t)blockIdx.x * 4 + (threadIdx.x >> 5);
    if (slot < p.count) finalize_slot<NPL1, false, false, false>(p, slot, p.count);
}

// The launch of the warp-per-slot kernel for one element type (F32: fp32 rows; otherwise 16-bit rows).
template <bool F32>
static int launch_finalize_rows(const FinalizeParams& p, unsigned grid, bool indirect, bool dyn, cudaStream_t st) {
#define FL_FINALIZE_CASE(N)                                                                     \
    case N:                                                                                     \
        if (dyn) knn_finalize_kernel<N, false, true, F32><<<grid, 128, 0, st>>>(p);            \
        else knn_finalize_kernel<N, false, false, F32><<<grid, 128, 0, st>>>(p);               \
        break;
    switch (p.K1 / 32) {
        FL_FINALIZE_CASE(1)
        FL_FINALIZE_CASE(2)
        case 4:
            if (indirect) knn_finalize_kernel<4, true, false, F32><<<grid, 128, 0, st>>>(p);
            else if (dyn) knn_finalize_kernel<4, false, true, F32><<<grid, 128, 0, st>>>(p);
            else knn_finalize_kernel<4, false, false, F32><<<grid, 128, 0, st>>>(p);
            break;
        FL_FINALIZE_CASE(8)
        FL_FINALIZE_CASE(16)
        default:
            set_error("unsupported pool size %d", p.K1);
            return FL_EUNSUPPORTED;
    }
#undef FL_FINALIZE_CASE
    FL_CHECK_LAUNCH();
    return FL_OK;
}

// Defined in knn_finalize_rows16.cu: the same launches for 16-bit rows, and the batched form.
int launch_finalize_rows16(const FinalizeParams& p, unsigned grid, bool indirect, bool dyn, cudaStream_t st);
int launch_finalize_batch(const FinalizeParams& p, dim3 grid, cudaStream_t st);

}  // namespace fl
