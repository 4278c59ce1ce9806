#include "ht_forest_tiled.cuh"

namespace ht {

int forward_tiled(const ht_forest_problem *, const float *, const float *, const int32_t *, const float *, float *,
                  cudaStream_t) {
  return HT_ERR_UNSUPPORTED;
}

}  // namespace ht
