// Tensor maps of one forward call on the tensor-core paths (built on the host per call).
#pragma once

#include <cuda.h>

#include "ma_common.cuh"

namespace ma {

struct alignas(64) TcMaps {
  CUtensorMap q_blk, q_col, k_blk, v_blk, out_col;
  CUtensorMap ar_blk, ar_col, al_blk, al_col, y_blk, y_col;
};

struct TcPlan {
  TcMaps maps;
  int qk_dtype;
};

}  // namespace ma
