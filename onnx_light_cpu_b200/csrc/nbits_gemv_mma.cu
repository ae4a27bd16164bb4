// Decode on warp-level tensor-core MMA with an exact 3-way bf16 split of the activations.
// Not built yet: the launcher reports "unsupported" so callers get MNB_ERR_UNSUPPORTED.
#include "nbits_common.cuh"

namespace mnb {

const char *LaunchGemvMma(const WeightView &, const float *, std::int64_t, OutputView, int *,
                          cudaStream_t, int) {
  return nullptr;
}

} // namespace mnb
