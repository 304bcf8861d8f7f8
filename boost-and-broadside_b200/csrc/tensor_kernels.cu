// Tensor-core (tcgen05) trunk kernels: placeholder until the engine lands.
#include "tensor_kernels.h"

namespace bnb {
namespace tensor {

bool supported(int, int, int) { return false; }
size_t scratch_bytes(int, const BnbBatch&, int) { return 0; }
size_t packed_spatial_bytes(int) { return 0; }
size_t packed_temporal_bytes(int) { return 0; }
int pack_spatial(const BnbSpatialWeights&, int, int, void*, cudaStream_t) { return BNB_ERR_UNSUPPORTED_DIMS; }
int pack_temporal(const BnbTemporalWeights&, int, void*, cudaStream_t) { return BNB_ERR_UNSUPPORTED_DIMS; }
int spatial_block(const BnbSpatialWeights&, int, int, const float*, const uint8_t*, float*, const BnbBatch&, int,
                  void*, size_t, cudaStream_t) { return BNB_ERR_UNSUPPORTED_DIMS; }
int temporal_block(const BnbTemporalWeights&, int, const float*, float*, const float*, float*, const uint8_t*,
                   const uint8_t*, const BnbBatch&, int, void*, size_t, cudaStream_t) { return BNB_ERR_UNSUPPORTED_DIMS; }
int trunk(const BnbSpatialWeights*, const BnbTemporalWeights*, int, int, int, int, int, const float*, const uint8_t*,
          float*, const float*, float*, const uint8_t*, const uint8_t*, const BnbBatch&, int, void*, size_t,
          cudaStream_t) { return BNB_ERR_UNSUPPORTED_DIMS; }

}  // namespace tensor
}  // namespace bnb
