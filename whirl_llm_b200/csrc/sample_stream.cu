#include "kernels.h"
namespace wb {
bool sample_stream_supported(const SelectArgs&, int) { return false; }
cudaError_t sample_stream_launch(const SelectArgs&, int, int, cudaStream_t) { return cudaErrorNotSupported; }
}  // namespace wb
