// Layout of the database operand plane produced by fl_knn_prepare_db_f32.
#pragma once
#include <stdint.h>

namespace fl {

struct PlaneLayout {
    int64_t m_pad;      // rows, multiple of 256
    int d_pad;          // feature columns, multiple of 64
    int pitch;          // bf16 elements per plane row: d_pad features + 16 norm columns
    int64_t off_rows;   // bf16 [m_pad][pitch]
    int64_t off_hnorm;  // f32 [m_pad], ||x||^2 / 2, +inf for padding rows
    int64_t off_meta;   // f32 [4]: [0] = max row norm
    int64_t bytes;
};

PlaneLayout plane_layout(int64_t m, int d);

// Columns appended to every plane row: the tensor-core kernels fold the -||x||^2/2 term of
// the score into the matrix product through them (see prep.cu).
constexpr int PLANE_AUG_COLS = 16;

}  // namespace fl
