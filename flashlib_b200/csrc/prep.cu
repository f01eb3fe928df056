// Row norms and the database operand plane (bf16 rows + half squared norms) that the
// tensor-core kNN / assign kernels stream with TMA.
#include "common.cuh"
#include "knn_internal.h"
#include <cuda_bf16.h>

namespace fl {

// One warp per row; out[row] = sum of squares in fp32.
__global__ void rownorm_kernel(const float* __restrict__ x, int64_t n, int d, int64_t ld,
                               float* __restrict__ out) {
    const int lane = threadIdx.x & 31;
    const int64_t row = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (row >= n) return;
    const float* p = x + row * ld;
    float s = 0.f;
    const bool vec = ((ld & 3) == 0) && ((reinterpret_cast<uintptr_t>(x) & 15) == 0);
    if (vec) {
        const int d4 = d >> 2;
        const float4* p4 = reinterpret_cast<const float4*>(p);
        for (int c = lane; c < d4; c += 32) {
            const float4 v = __ldg(p4 + c);
            s += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
        }
        for (int c = (d4 << 2) + lane; c < d; c += 32) { const float v = p[c]; s += v * v; }
    } else {
        for (int c = lane; c < d; c += 32) { const float v = p[c]; s += v * v; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(FULL_MASK, s, o);
    if (lane == 0) out[row] = s;
}

// One warp per plane row: converts the fp32 row to bf16 (round to nearest even), zero
// pads columns [d, d_pad), writes ||x||^2/2 (+inf for padding rows) and folds the row's
// norm into the plane-wide maximum (non-negative floats order like their bit patterns).
// Columns [d_pad, d_pad+3) carry -||x||^2/2 split into three bf16 terms (their sum is exact
// to 2^-24 relative); multiplied by the ones the query plane holds in the same columns they
// make the tensor-core product come out as <q,x> - ||x||^2/2.  Padding rows carry a huge
// negative value there so they can never rank.
// Rows of 16-bit storage (dt): bf16 values enter the plane as they are, fp16 values are rounded to
// bf16 like fp32 ones; the norms are those of the stored values.
__global__ void plane_build_kernel(const void* __restrict__ db, int64_t m, int d, int64_t ld,
                                   __nv_bfloat16* __restrict__ rows, float* __restrict__ hnorm,
                                   unsigned int* __restrict__ maxnorm_bits, int64_t m_pad, int d_pad, int dt) {
    const int lane = threadIdx.x & 31;
    const int64_t row = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (row >= m_pad) return;
    const int pitch = d_pad + PLANE_AUG_COLS;
    __nv_bfloat16* o = rows + row * pitch;
    if (row >= m) {
        for (int c = lane; c < pitch; c += 32) o[c] = __float2bfloat16_rn(c == d_pad ? -3.0e38f : 0.f);
        if (lane == 0) hnorm[row] = pos_inf();
        return;
    }
    const void* p = row_at(db, row, ld, dt);
    float s = 0.f;
    for (int c = lane; c < d_pad; c += 32) {
        const float v = (c < d) ? ld_elem(p, c, dt) : 0.f;
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

PlaneLayout plane_layout(int64_t m, int d) {
    PlaneLayout L;
    L.m_pad = round_up(m, 256);
    L.d_pad = (int)round_up(d, 64);
    L.pitch = L.d_pad + PLANE_AUG_COLS;
    L.off_rows = 0;
    L.off_hnorm = round_up(L.m_pad * (int64_t)L.pitch * 2, 1024);
    L.off_meta = L.off_hnorm + round_up(L.m_pad * 4, 1024);
    L.bytes = L.off_meta + 1024;
    return L;
}

// Fills `plane` (layout plane_layout(m, d)) for the fp32 rows of db.
int launch_plane_build(const void* db, int64_t m, int d, int64_t ld, void* plane, cudaStream_t st, int dt) {
    const PlaneLayout L = plane_layout(m, d);
    char* base = static_cast<char*>(plane);
    FL_CHECK_CUDA(cudaMemsetAsync(base + L.off_meta, 0, 1024, st));
    const int wpb = 8;
    plane_build_kernel<<<(unsigned)ceil_div(L.m_pad, wpb), wpb * 32, 0, st>>>(
        db, m, d, ld, reinterpret_cast<__nv_bfloat16*>(base + L.off_rows),
        reinterpret_cast<float*>(base + L.off_hnorm), reinterpret_cast<unsigned int*>(base + L.off_meta),
        L.m_pad, L.d_pad, dt);
    FL_CHECK_LAUNCH();
    return FL_OK;
}

}  // namespace fl

using namespace fl;

extern "C" int fl_rownorm_f32(const float* x, int64_t n, int d, int64_t ld, float* out, void* stream) {
    FL_CHECK_ARG(n >= 0 && d >= 1 && ld >= d, "fl_rownorm_f32: bad shape n=%lld d=%d ld=%lld",
                 (long long)n, d, (long long)ld);
    if (n == 0) return FL_OK;
    FL_CHECK_ARG(x && out, "fl_rownorm_f32: null pointer");
    const int wpb = 8;
    rownorm_kernel<<<(unsigned)ceil_div(n, wpb), wpb * 32, 0, (cudaStream_t)stream>>>(x, n, d, ld, out);
    FL_CHECK_LAUNCH();
    return FL_OK;
}

extern "C" int64_t fl_knn_plane_bytes(int64_t m, int d) {
    if (m < 1 || d < 1) return 0;
    return plane_layout(m, d).bytes;
}

extern "C" int fl_knn_prepare_db_rows(const void* db, int dtype, int64_t m, int d, int64_t ld, void* plane,
                                      int64_t plane_bytes, void* stream) {
    FL_CHECK_ARG(m >= 1 && d >= 1 && ld >= d, "fl_knn_prepare_db: bad shape m=%lld d=%d ld=%lld",
                 (long long)m, d, (long long)ld);
    FL_CHECK_ARG(dtype == DT_F32 || dtype == DT_BF16 || dtype == DT_F16, "fl_knn_prepare_db: unknown dtype %d", dtype);
    FL_CHECK_ARG(db && plane, "fl_knn_prepare_db: null pointer");
    FL_CHECK_ARG((reinterpret_cast<uintptr_t>(plane) & 255) == 0,
                 "fl_knn_prepare_db: plane must be 256-byte aligned");
    const PlaneLayout L = plane_layout(m, d);
    if (plane_bytes < L.bytes) {
        set_error("fl_knn_prepare_db: plane buffer %lld < %lld bytes", (long long)plane_bytes,
                  (long long)L.bytes);
        return FL_EWORKSPACE;
    }
    return launch_plane_build(db, m, d, ld, plane, (cudaStream_t)stream, dtype);
}

extern "C" int fl_knn_prepare_db_f32(const float* db, int64_t m, int d, int64_t ld, void* plane,
                                     int64_t plane_bytes, void* stream) {
    return fl_knn_prepare_db_rows(db, DT_F32, m, d, ld, plane, plane_bytes, stream);
}
