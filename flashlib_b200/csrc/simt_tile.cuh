// CUDA-core (fp32 FFMA) tile contraction shared by the exact kNN kernel and the exact
// k-means assign kernel: a block of 256 threads computes the BQ x 128 block of inner
// products <q_i, x_j> over the full feature dimension, streaming both operands through
// shared memory in slabs of 32 features with register-staged double buffering.
#pragma once
#include "common.cuh"

namespace fl {

template <int TQ>
struct SimtTile {
    static constexpr int BQ = 16 * TQ;           // queries per block
    static constexpr int BN = 128;               // database rows per tile
    static constexpr int KS = 32;                // features per slab
    static constexpr int QSTR = BQ + 4;          // padded strides keep float4 alignment
    static constexpr int DSTR = BN + 4;
    static constexpr int QL = (BQ * 8 + 255) / 256;  // float4 loads per thread per Q slab
    static constexpr int SLAB_FLOATS = 2 * KS * (QSTR + DSTR);
};

__device__ __forceinline__ float4 load4_guard(const void* row, int kb, int d, bool vec, int dt) {
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    if (row == nullptr) return v;
    if (vec && kb + 3 < d) return ld_elem4(row, kb, dt);
    if (kb < d) v.x = ld_elem(row, kb, dt);
    if (kb + 1 < d) v.y = ld_elem(row, kb + 1, dt);
    if (kb + 2 < d) v.z = ld_elem(row, kb + 2, dt);
    if (kb + 3 < d) v.w = ld_elem(row, kb + 3, dt);
    return v;
}

// qrow[i] / drow[i]: row pointers (or nullptr for rows outside the problem) of the
// float4 groups this thread stages: group g = i*256 + tid covers row g/8, features
// (g%8)*4 .. +3 of each slab.  acc[i][j] receives <q[ty*TQ+i], x[col(j)]> with
// col(j) = tx*4 + j for j < 4 and 64 + tx*4 + (j-4) otherwise (tx = tid%16, ty = tid/16).
// dtq / dtd: element types of the query and database rows (DT_*), widened to fp32 on load.
template <int TQ>
__device__ __forceinline__ void simt_cross_tile(const void* const (&qrow)[SimtTile<TQ>::QL],
                                                const void* const (&drow)[4], int d, bool vecq,
                                                bool vecd, float* smem, float (&acc)[TQ][8], int dtq = DT_F32,
                                                int dtd = DT_F32) {
    using T = SimtTile<TQ>;
    const int tid = threadIdx.x;
    const int tx = tid & 15, ty = tid >> 4;
    float* Qs = smem;                          // [2][KS][QSTR]
    float* Ds = smem + 2 * T::KS * T::QSTR;    // [2][KS][DSTR]
#pragma unroll
    for (int i = 0; i < TQ; ++i)
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[i][j] = 0.f;

    float4 rq[T::QL], rd[4];
    const int kq = (tid & 7) * 4;  // feature offset of this thread's groups inside a slab
    const int nslab = (d + T::KS - 1) / T::KS;

    auto fetch = [&](int slab) {
        const int kb = slab * T::KS + kq;
#pragma unroll
        for (int i = 0; i < T::QL; ++i) rq[i] = load4_guard(qrow[i], kb, d, vecq, dtq);
#pragma unroll
        for (int i = 0; i < 4; ++i) rd[i] = load4_guard(drow[i], kb, d, vecd, dtd);
    };
    auto stash = [&](int buf) {
        float* qs = Qs + buf * T::KS * T::QSTR;
        float* ds = Ds + buf * T::KS * T::DSTR;
#pragma unroll
        for (int i = 0; i < T::QL; ++i) {
            const int g = i * 256 + tid;
            const int r = g >> 3;
            if (r < T::BQ) {
                qs[(kq + 0) * T::QSTR + r] = rq[i].x;
                qs[(kq + 1) * T::QSTR + r] = rq[i].y;
                qs[(kq + 2) * T::QSTR + r] = rq[i].z;
                qs[(kq + 3) * T::QSTR + r] = rq[i].w;
            }
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int r = (i * 256 + tid) >> 3;
            ds[(kq + 0) * T::DSTR + r] = rd[i].x;
            ds[(kq + 1) * T::DSTR + r] = rd[i].y;
            ds[(kq + 2) * T::DSTR + r] = rd[i].z;
            ds[(kq + 3) * T::DSTR + r] = rd[i].w;
        }
    };

    fetch(0);
    stash(0);
    __syncthreads();
    for (int s = 0; s < nslab; ++s) {
        const int buf = s & 1;
        if (s + 1 < nslab) fetch(s + 1);
        const float* qs = Qs + buf * T::KS * T::QSTR + ty * TQ;
        const float* ds = Ds + buf * T::KS * T::DSTR + tx * 4;
#pragma unroll 8
        for (int kk = 0; kk < T::KS; ++kk) {
            float a[TQ];
            if (TQ == 4) {
                const float4 v = *reinterpret_cast<const float4*>(qs + kk * T::QSTR);
                a[0] = v.x; a[1 % TQ] = v.y; a[2 % TQ] = v.z; a[3 % TQ] = v.w;
            } else if (TQ == 2) {
                const float2 v = *reinterpret_cast<const float2*>(qs + kk * T::QSTR);
                a[0] = v.x; a[1 % TQ] = v.y;
            } else {
                a[0] = qs[kk * T::QSTR];
            }
            const float4 b0 = *reinterpret_cast<const float4*>(ds + kk * T::DSTR);
            const float4 b1 = *reinterpret_cast<const float4*>(ds + kk * T::DSTR + 64);
#pragma unroll
            for (int i = 0; i < TQ; ++i) {
                acc[i][0] = fmaf(a[i], b0.x, acc[i][0]);
                acc[i][1] = fmaf(a[i], b0.y, acc[i][1]);
                acc[i][2] = fmaf(a[i], b0.z, acc[i][2]);
                acc[i][3] = fmaf(a[i], b0.w, acc[i][3]);
                acc[i][4] = fmaf(a[i], b1.x, acc[i][4]);
                acc[i][5] = fmaf(a[i], b1.y, acc[i][5]);
                acc[i][6] = fmaf(a[i], b1.z, acc[i][6]);
                acc[i][7] = fmaf(a[i], b1.w, acc[i][7]);
            }
        }
        if (s + 1 < nslab) stash(buf ^ 1);
        __syncthreads();
    }
}

}  // namespace fl
