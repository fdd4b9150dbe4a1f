// Instantiations of the tcgen05 convolution kernel for 32-channel tiles staged in 32-channel
// slabs (a translation unit of its own so that the tile shapes compile in parallel).
#include "conv_tc_dev.cuh"

namespace occ {

bool tc_launch_32_32(const TcParams &p, int mode, int grid, size_t smem, cudaStream_t s) {
  return tc_launch_mode<32, 32, true>(p, mode, grid, smem, s);
}

bool tc_launch_32_32_duo(const TcParams &p, int mode, int grid, size_t smem, cudaStream_t s) {
  return tc_launch_mode_duo<32, 32>(p, mode, grid, smem, s);
}

}  // namespace occ
