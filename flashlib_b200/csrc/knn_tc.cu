// Tensor-core candidate pass of the exact kNN: a persistent, warp-specialised sm_100a
// kernel.  Per work item (one tile of 128 queries x one contiguous range of database
// tiles) it keeps the bf16 query tile resident in shared memory, streams bf16 database
// tiles of 256 rows through a TMA ring, multiplies them with tcgen05.mma into two
// 128 x 256 fp32 accumulators in tensor memory (so the next tile's MMAs overlap the
// current tile's epilogue) and, in the epilogue, turns every accumulator row into scores
//     s = <q, x> - ||x||^2 / 2          (larger = closer)
// that feed a per-query candidate pool in shared memory.  Nothing of the 128 x 256 score
// tile ever reaches global memory; a pool of K1 = 32 (score, row) pairs per query and
// range is all that is written.
//
// Warp roles (192 threads): warps 0-3 epilogue (warp w reads TMEM lanes 32w..32w+31, one
// query row per thread), warp 4 TMA producer, warp 5 MMA issuer and TMEM owner.
// Every wait is bounded; a wait that gives up raises a CTA-wide abort flag, records where
// it happened in the status words and every role falls through to the common exit.
#include "knn_internal.h"
#include "pool.cuh"
#include "tc_ptx.cuh"

namespace fl {

using namespace tc;

constexpr int TC_BM = 128;            // queries per tile (MMA M)
constexpr int TC_BN = 256;            // database rows per tile (MMA N)
constexpr int TC_BK = 64;             // bf16 features per shared-memory chunk (128 bytes)
constexpr int TC_K1 = 32;             // pool size per query
constexpr int TC_CAP = 64;            // pool capacity before compaction
constexpr int TC_PSTR = TC_CAP + 1;   // padded pool row stride (bank spread)
constexpr int TC_A_CHUNK = TC_BM * 128;   // bytes of one K-chunk of the query tile
constexpr int TC_B_STAGE = TC_BN * 128;   // bytes of one K-chunk of a database tile
constexpr int TC_MAX_STAGES = 6;
constexpr uint64_t TC_WAIT_NS = 2000000000ull;   // 2 s per wait

struct TcSmemPlan {
    int nkc, nstage;
    int off_a, off_b, off_pool_sc, off_pool_id, off_hbuf, off_bar, bytes;
};

static TcSmemPlan tc_smem_plan(int d_pad, int smem_limit) {
    TcSmemPlan s{};
    s.nkc = d_pad / TC_BK;
    int cur = 0;
    s.off_a = cur; cur += s.nkc * TC_A_CHUNK;
    const int pool = TC_BM * TC_PSTR * 4;
    const int fixed = cur + 2 * pool + 4 * TC_BN * 4 + 256 + 1024 /* alignment slack */;
    int ns = (smem_limit - fixed) / TC_B_STAGE;
    if (ns > TC_MAX_STAGES) ns = TC_MAX_STAGES;
    s.nstage = ns;
    s.off_b = cur; cur += (ns > 0 ? ns : 0) * TC_B_STAGE;
    s.off_pool_sc = cur; cur += pool;
    s.off_pool_id = cur; cur += pool;
    s.off_hbuf = cur; cur += 4 * TC_BN * 4;
    s.off_bar = cur; cur += 256;
    s.bytes = cur + 1024;
    return s;
}

struct TcKernelParams {
    int n_qtiles, n_tiles, nsplit, tiles_per_split, nkc, nstage;
    int off_b, off_pool_sc, off_pool_id, off_hbuf, off_bar;
    int64_t nq_pad;
    const float* hnorm;
    float* part_sc; uint32_t* part_id;
    float* tau;
    int32_t* status;
    float* dbg_scores;       // optional: [128][n_tiles*256] scores of query tile 0
    int64_t dbg_ld;
};

__device__ __forceinline__ void tc_report_timeout(int32_t* status, int role, int which) {
    if (status) {
        if (atomicCAS(status + FL_STATUS_ERROR, 0, FL_ETIMEOUT) == 0) status[FL_STATUS_WHERE] = (role << 16) | which;
    }
}

struct TcPoolState { int cnt; float tau; };

// Slow path of the epilogue, entered by the whole warp when at least one lane holds a score
// above its row's threshold: the hitting lanes append their passing scores to their rows'
// pools, then the warp compacts every pool that is nearly full.  Kept out of line so the
// streaming loop stays small.
static __device__ __noinline__ TcPoolState tc_pool_update(bool hit, float s0, float s1, float s2, float s3,
                                                          float s4, float s5, float s6, float s7, uint32_t cb,
                                                          float* my_sc, uint32_t* my_id, float* warp_sc,
                                                          uint32_t* warp_id, int cnt, float tau) {
    const int lane = threadIdx.x & 31;
    if (hit) {
        const float s[8] = {s0, s1, s2, s3, s4, s5, s6, s7};
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            if (s[j] > tau) { my_sc[cnt] = s[j]; my_id[cnt] = cb + j; ++cnt; }
        }
    }
    unsigned need = __ballot_sync(FULL_MASK, cnt > TC_CAP - 8);
    if (need) __syncwarp();
    while (need) {
        const int src = __ffs(need) - 1;
        need &= need - 1;
        const int n = __shfl_sync(FULL_MASK, cnt, src);
        const float thr = warp_pool_compact<TC_CAP / 32>(warp_sc + src * TC_PSTR, warp_id + src * TC_PSTR, n, TC_K1);
        if (lane == src) { cnt = min(n, TC_K1); tau = fmaxf(tau, thr); }
    }
    TcPoolState r;
    r.cnt = cnt;
    r.tau = tau;
    return r;
}

__global__ void __launch_bounds__(192, 1)
knn_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_db,
              const TcKernelParams p) {
    extern __shared__ uint8_t smem_raw[];
    // the swizzled operand tiles need 1024-byte aligned shared memory
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    const uint32_t sbase = smem_u32(smem);
    const uint32_t a_addr = sbase;                      // nkc chunks of 16 KB
    const uint32_t b_addr = sbase + p.off_b;            // nstage stages of 32 KB
    float* pool_sc = reinterpret_cast<float*>(smem + p.off_pool_sc);
    uint32_t* pool_id = reinterpret_cast<uint32_t*>(smem + p.off_pool_id);
    float* hbuf = reinterpret_cast<float*>(smem + p.off_hbuf);
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + p.off_bar);
    // barrier slots: [0, 6) full, [6, 12) empty, 12 a_full, 13 a_empty, 14-15 tmem_full, 16-17 tmem_empty
    const uint32_t bar0 = smem_u32(bars);
    auto BAR = [&](int i) { return bar0 + 8u * i; };
    constexpr int B_FULL = 0, B_EMPTY = 6, B_AFULL = 12, B_AEMPTY = 13, B_TFULL = 14, B_TEMPTY = 16;
    volatile int* abort_flag = reinterpret_cast<volatile int*>(bars + 20);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 21);

    const int tid = threadIdx.x;
    const int warp = tid >> 5, lane = tid & 31;

    if (tid == 0) {
        for (int i = 0; i < TC_MAX_STAGES; ++i) { mbar_init(BAR(B_FULL + i), 1); mbar_init(BAR(B_EMPTY + i), 1); }
        mbar_init(BAR(B_AFULL), 1);
        mbar_init(BAR(B_AEMPTY), 1);
        for (int i = 0; i < 2; ++i) { mbar_init(BAR(B_TFULL + i), 1); mbar_init(BAR(B_TEMPTY + i), 4); }
        *abort_flag = 0;
        fence_barrier_init();
    }
    if (warp == 4 && lane == 0) { prefetch_tensormap(&map_q); prefetch_tensormap(&map_db); }
    if (warp == 5) {
        tmem_alloc(smem_u32(tmem_slot), 512);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;

    const int n_items = p.n_qtiles * p.nsplit;

    if (warp == 4) {
        // ------------------------------ TMA producer --------------------------------------
        if (lane == 0) {
            uint32_t fill = 0;     // database chunks issued so far
            uint32_t item_no = 0;
            bool ok = true;
            for (int it = blockIdx.x; it < n_items && ok; it += gridDim.x, ++item_no) {
                const int split = it / p.n_qtiles, qt = it - split * p.n_qtiles;
                const int t0 = split * p.tiles_per_split;
                const int t1 = min(p.n_tiles, t0 + p.tiles_per_split);
                if (!mbar_wait(BAR(B_AEMPTY), (item_no & 1) ^ 1, abort_flag, TC_WAIT_NS)) {
                    tc_report_timeout(p.status, 4, B_AEMPTY); ok = false; break;
                }
                mbar_expect_tx(BAR(B_AFULL), p.nkc * TC_A_CHUNK);
                for (int kc = 0; kc < p.nkc; ++kc)
                    tma_load_2d(a_addr + kc * TC_A_CHUNK, &map_q, kc * TC_BK, qt * TC_BM, BAR(B_AFULL));
                for (int t = t0; t < t1 && ok; ++t) {
                    for (int kc = 0; kc < p.nkc; ++kc, ++fill) {
                        const int s = fill % p.nstage;
                        const uint32_t ph = (fill / p.nstage) & 1;
                        if (!mbar_wait(BAR(B_EMPTY + s), ph ^ 1, abort_flag, TC_WAIT_NS)) {
                            tc_report_timeout(p.status, 4, B_EMPTY + s); ok = false; break;
                        }
                        mbar_expect_tx(BAR(B_FULL + s), TC_B_STAGE);
                        tma_load_2d(b_addr + s * TC_B_STAGE, &map_db, kc * TC_BK, t * TC_BN, BAR(B_FULL + s));
                    }
                }
            }
            if (!ok) {
                // give copies already in flight a bounded time to land before the CTA exits
                const uint64_t t_start = globaltimer_ns();
                while (globaltimer_ns() - t_start < 2000000ull) { }
            }
        }
    } else if (warp == 5) {
        // ------------------------------ MMA issuer -----------------------------------------
        if (lane == 0) {
            constexpr uint32_t idesc = umma_idesc_bf16(TC_BM, TC_BN);
            uint32_t use = 0;      // database chunks consumed so far
            uint32_t tile_no = 0;  // tiles issued so far (accumulator ring position)
            uint32_t item_no = 0;
            bool ok = true;
            for (int it = blockIdx.x; it < n_items && ok; it += gridDim.x, ++item_no) {
                const int split = it / p.n_qtiles;
                const int t0 = split * p.tiles_per_split;
                const int t1 = min(p.n_tiles, t0 + p.tiles_per_split);
                if (!mbar_wait(BAR(B_AFULL), item_no & 1, abort_flag, TC_WAIT_NS)) {
                    tc_report_timeout(p.status, 5, B_AFULL); ok = false; break;
                }
                for (int t = t0; t < t1 && ok; ++t, ++tile_no) {
                    const int b = tile_no & 1;
                    if (!mbar_wait(BAR(B_TEMPTY + b), ((tile_no >> 1) & 1) ^ 1, abort_flag, TC_WAIT_NS)) {
                        tc_report_timeout(p.status, 5, B_TEMPTY + b); ok = false; break;
                    }
                    tc_fence_after_sync();
                    const uint32_t d_tmem = tmem_base + b * TC_BN;
                    for (int kc = 0; kc < p.nkc; ++kc, ++use) {
                        const int s = use % p.nstage;
                        const uint32_t ph = (use / p.nstage) & 1;
                        if (!mbar_wait(BAR(B_FULL + s), ph, abort_flag, TC_WAIT_NS)) {
                            tc_report_timeout(p.status, 5, B_FULL + s); ok = false; break;
                        }
                        tc_fence_after_sync();
                        const uint64_t da = umma_desc(a_addr + kc * TC_A_CHUNK);
                        const uint64_t db = umma_desc(b_addr + s * TC_B_STAGE);
#pragma unroll
                        for (int k4 = 0; k4 < TC_BK / 16; ++k4) {
                            // +32 bytes per 16-feature step inside the 128-byte swizzled row
                            umma_bf16(d_tmem, da + 2 * k4, db + 2 * k4, idesc, (kc | k4) != 0 ? 1u : 0u);
                        }
                        umma_commit(BAR(B_EMPTY + s));   // stage reusable once these MMAs retire
                    }
                    if (ok) umma_commit(BAR(B_TFULL + b));
                }
                if (ok) umma_commit(BAR(B_AEMPTY));       // query tile reusable
            }
        }
    } else {
        // ------------------------------ epilogue warps --------------------------------------
        float* my_sc = pool_sc + (warp * 32 + lane) * TC_PSTR;
        uint32_t* my_id = pool_id + (warp * 32 + lane) * TC_PSTR;
        float* hb = hbuf + warp * TC_BN;
        const uint32_t lane_taddr = tmem_base + (uint32_t(warp * 32) << 16);
        uint32_t tile_no = 0;
        bool ok = true;
        for (int it = blockIdx.x; it < n_items && ok; it += gridDim.x) {
            const int split = it / p.n_qtiles, qt = it - split * p.n_qtiles;
            const int t0 = split * p.tiles_per_split;
            const int t1 = min(p.n_tiles, t0 + p.tiles_per_split);
            const int64_t qrow = (int64_t)qt * TC_BM + warp * 32 + lane;
            const float tau_in = __ldcg(p.tau + qrow);
            float tau = tau_in;
            int cnt = 0;
            // half norms of the first tile of the range
            float4 h0 = __ldg(reinterpret_cast<const float4*>(p.hnorm + (int64_t)t0 * TC_BN + lane * 8));
            float4 h1 = __ldg(reinterpret_cast<const float4*>(p.hnorm + (int64_t)t0 * TC_BN + lane * 8 + 4));
            for (int t = t0; t < t1; ++t, ++tile_no) {
                __syncwarp();
                *reinterpret_cast<float4*>(hb + lane * 8) = h0;
                *reinterpret_cast<float4*>(hb + lane * 8 + 4) = h1;
                __syncwarp();
                if (t + 1 < t1) {
                    h0 = __ldg(reinterpret_cast<const float4*>(p.hnorm + (int64_t)(t + 1) * TC_BN + lane * 8));
                    h1 = __ldg(reinterpret_cast<const float4*>(p.hnorm + (int64_t)(t + 1) * TC_BN + lane * 8 + 4));
                }
                const int b = tile_no & 1;
                if (!__all_sync(FULL_MASK, mbar_wait(BAR(B_TFULL + b), (tile_no >> 1) & 1, abort_flag, TC_WAIT_NS))) {
                    if (lane == 0) tc_report_timeout(p.status, warp, B_TFULL + b);
                    ok = false;
                    break;
                }
                tc_fence_after_sync();
                const uint32_t tile_taddr = lane_taddr + b * TC_BN;
                const uint32_t row_base = (uint32_t)t * TC_BN;

                uint32_t va[32], vb[32];
                auto process = [&](uint32_t (&v)[32], int slice) {
                    const float* hs = hb + slice * 32;
#pragma unroll
                    for (int g = 0; g < 4; ++g) {
                        const float4 ha = *reinterpret_cast<const float4*>(hs + g * 8);
                        const float4 hc = *reinterpret_cast<const float4*>(hs + g * 8 + 4);
                        float s[8];
                        s[0] = __uint_as_float(v[g * 8 + 0]) - ha.x;
                        s[1] = __uint_as_float(v[g * 8 + 1]) - ha.y;
                        s[2] = __uint_as_float(v[g * 8 + 2]) - ha.z;
                        s[3] = __uint_as_float(v[g * 8 + 3]) - ha.w;
                        s[4] = __uint_as_float(v[g * 8 + 4]) - hc.x;
                        s[5] = __uint_as_float(v[g * 8 + 5]) - hc.y;
                        s[6] = __uint_as_float(v[g * 8 + 6]) - hc.z;
                        s[7] = __uint_as_float(v[g * 8 + 7]) - hc.w;
                        if (p.dbg_scores != nullptr && qt == 0) {
#pragma unroll
                            for (int j = 0; j < 8; ++j)
                                p.dbg_scores[(int64_t)(warp * 32 + lane) * p.dbg_ld + row_base + slice * 32 + g * 8 + j] = s[j];
                        }
                        const float m = fmaxf(fmax3(s[0], s[1], s[2]), fmaxf(fmax3(s[3], s[4], s[5]), fmaxf(s[6], s[7])));
                        const bool hit = m > tau;
                        if (__any_sync(FULL_MASK, hit)) {
                            const TcPoolState r = tc_pool_update(hit, s[0], s[1], s[2], s[3], s[4], s[5], s[6], s[7],
                                                                 row_base + slice * 32 + g * 8, my_sc, my_id,
                                                                 pool_sc + warp * 32 * TC_PSTR,
                                                                 pool_id + warp * 32 * TC_PSTR, cnt, tau);
                            cnt = r.cnt;
                            tau = r.tau;
                        }
                    }
                };

                tmem_ld_32x32b_x32(tile_taddr, va);
                tmem_ld_wait();
                reg_fence32(va);
#pragma unroll 1
                for (int sp = 0; sp < TC_BN / 64; ++sp) {
                    tmem_ld_32x32b_x32(tile_taddr + (2 * sp + 1) * 32, vb);
                    process(va, 2 * sp);
                    tmem_ld_wait();
                    reg_fence32(vb);
                    if (sp + 1 < TC_BN / 64) {
                        tmem_ld_32x32b_x32(tile_taddr + (2 * sp + 2) * 32, va);
                    } else {
                        // every column of this accumulator is in registers: hand it back
                        tc_fence_before_sync();
                        __syncwarp();
                        if (lane == 0) mbar_arrive(BAR(B_TEMPTY + b));
                    }
                    process(vb, 2 * sp + 1);
                    if (sp + 1 < TC_BN / 64) {
                        tmem_ld_wait();
                        reg_fence32(va);
                    }
                }
            }
            if (!ok) break;
            // end of the item: sort every row's pool, publish it and the row's threshold
            __syncwarp();
#pragma unroll 1
            for (int src = 0; src < 32; ++src) {
                const int n = __shfl_sync(FULL_MASK, cnt, src);
                float* rsc = pool_sc + (warp * 32 + src) * TC_PSTR;
                uint32_t* rid = pool_id + (warp * 32 + src) * TC_PSTR;
                const float thr = warp_pool_compact<TC_CAP / 32>(rsc, rid, n, TC_K1);
                if (lane == src) tau = fmaxf(tau, thr);
                const int64_t q = (int64_t)qt * TC_BM + warp * 32 + src;
                const int64_t o = (q * p.nsplit + split) * TC_K1;
                p.part_sc[o + lane] = rsc[lane];
                p.part_id[o + lane] = rid[lane];
                __syncwarp();
            }
            if (tau > tau_in) __stcg(p.tau + qrow, tau);
        }
    }

    // ------------------------------ common exit ----------------------------------------------
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 5) {
        tc_fence_after_sync();
        tmem_dealloc(tmem_base, 512);
    }
}

// ---- host side ---------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode_fn() {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void* ptr = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) != cudaSuccess ||
            qres != cudaDriverEntryPointSuccess)
            return nullptr;
        fn = reinterpret_cast<EncodeTiledFn>(ptr);
    }
    return fn;
}

// 2-D bf16 row-major tensor [rows][cols], box = 64 columns x box_rows rows, 128-byte swizzle.
static int make_map_bf16(CUtensorMap* map, const void* base, int64_t rows, int cols, int box_rows) {
    EncodeTiledFn fn = get_encode_fn();
    if (!fn) { set_error("cuTensorMapEncodeTiled is not available from the driver"); return FL_ECUDA; }
    cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)cols * 2};
    cuuint32_t box[2] = {(cuuint32_t)TC_BK, (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) { set_error("cuTensorMapEncodeTiled failed with code %d", (int)r); return FL_ECUDA; }
    return FL_OK;
}

int tc_pool_size(int k) { (void)k; return TC_K1; }

int tc_knn_supported(int64_t nq, int64_t m, int d, int k) {
    if (nq < 1 || m < 1) return FL_EUNSUPPORTED;
    if (k > 16) return FL_EUNSUPPORTED;             // pool of 32 leaves the verification margin
    if (d > 256) return FL_EUNSUPPORTED;            // resident query tile: up to 4 chunks of 64 features
    if (round_up(m, 256) / 256 > (1 << 23)) return FL_EUNSUPPORTED;
    return FL_OK;
}

// Auto mode takes the tensor-core path once the problem is large enough to amortise it.
int tc_knn_auto(int64_t nq, int64_t m, int d, int k) {
    if (tc_knn_supported(nq, m, d, k) != FL_OK) return 0;
    return (m >= 2048 && nq * m >= (int64_t(1) << 24)) ? 1 : 0;
}

void tc_split_plan(int64_t nq_pad, int64_t m_pad, int* nsplit, int64_t* tiles_per_split) {
    const int64_t n_qtiles = nq_pad / TC_BM;
    const int64_t n_tiles = m_pad / TC_BN;
    const int sms = sm_count();
    int64_t max_s = n_tiles / 8;
    if (max_s > 64) max_s = 64;
    if (max_s < 1) max_s = 1;
    double best_eff = -1.0;
    int64_t best_s = 1;
    for (int64_t s = 1; s <= max_s; ++s) {
        const int64_t tps = ceil_div(n_tiles, s);
        const int64_t s_eff = ceil_div(n_tiles, tps);
        const int64_t items = n_qtiles * s_eff;
        const int64_t grid = items < sms ? items : sms;
        const int64_t waves = ceil_div(items, grid);
        // SMs busy over the run, counting idle SMs when there are fewer items than SMs
        const double eff = (double)items / (double)(waves * sms);
        if (eff > best_eff * 1.02) { best_eff = eff; best_s = s_eff; }
    }
    *tiles_per_split = ceil_div(n_tiles, best_s);
    *nsplit = (int)ceil_div(n_tiles, *tiles_per_split);
}

static int launch_tc_impl(const TcKnnParams& p, float* dbg, int64_t dbg_ld, cudaStream_t st) {
    CUtensorMap map_q, map_db;
    int rc = make_map_bf16(&map_q, p.qplane, p.nq_pad, p.d_pad, TC_BM);
    if (rc != FL_OK) return rc;
    rc = make_map_bf16(&map_db, p.dbrows, p.m_pad, p.d_pad, TC_BN);
    if (rc != FL_OK) return rc;
    const TcSmemPlan sp = tc_smem_plan(p.d_pad, smem_optin_bytes());
    if (sp.nstage < 2) { set_error("tensor-core kNN: feature dimension %d leaves no room for the TMA ring", p.d_pad); return FL_EUNSUPPORTED; }
    TcKernelParams kp{};
    kp.n_qtiles = (int)(p.nq_pad / TC_BM);
    kp.n_tiles = (int)(p.m_pad / TC_BN);
    kp.nsplit = p.nsplit;
    kp.tiles_per_split = (int)p.tiles_per_split;
    kp.nkc = sp.nkc; kp.nstage = sp.nstage;
    kp.off_b = sp.off_b; kp.off_pool_sc = sp.off_pool_sc; kp.off_pool_id = sp.off_pool_id;
    kp.off_hbuf = sp.off_hbuf; kp.off_bar = sp.off_bar;
    kp.nq_pad = p.nq_pad; kp.hnorm = p.hnorm; kp.part_sc = p.part_sc; kp.part_id = p.part_id;
    kp.tau = p.tau; kp.status = p.status; kp.dbg_scores = dbg; kp.dbg_ld = dbg_ld;
    const int items = kp.n_qtiles * kp.nsplit;
    const int grid = items < sm_count() ? items : sm_count();
    FL_CHECK_CUDA(cudaFuncSetAttribute(knn_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, sp.bytes));
    knn_tc_kernel<<<grid, 192, sp.bytes, st>>>(map_q, map_db, kp);
    FL_CHECK_LAUNCH();
    return FL_OK;
}

int launch_knn_tc(const TcKnnParams& p, cudaStream_t st) { return launch_tc_impl(p, nullptr, 0, st); }
int launch_knn_tc_debug(const TcKnnParams& p, float* dbg, int64_t dbg_ld, cudaStream_t st) {
    return launch_tc_impl(p, dbg, dbg_ld, st);
}

}  // namespace fl
