// placeholder: tensor-core decode kernel not built yet
#include "gh_kernels.cuh"
namespace gh {
bool decode_mma_supported( const Shape&, uint32_t ) { return false; }
cudaError_t decode_mma_prepare() { return cudaSuccess; }
uint32_t decode_mma_tile_tokens() { return 64; }
cudaError_t launch_decode_mma( const DecodeArgs&, const CUtensorMap*, cudaStream_t, uint64_t* ) { return cudaErrorNotSupported; }
}
