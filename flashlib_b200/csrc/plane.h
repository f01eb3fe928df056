// Layout of the database operand plane produced by fl_knn_prepare_db_f32.
#pragma once
#include <stdint.h>

namespace fl {

struct PlaneLayout {
    int64_t m_pad;      // rows, multiple of 256
    int d_pad;          // columns, multiple of 64
    int64_t off_rows;   // bf16 [m_pad][d_pad]
    int64_t off_hnorm;  // f32 [m_pad], ||x||^2 / 2, +inf for padding rows
    int64_t off_meta;   // f32 [4]: [0] = max row norm
    int64_t bytes;
};

PlaneLayout plane_layout(int64_t m, int d);

}  // namespace fl
