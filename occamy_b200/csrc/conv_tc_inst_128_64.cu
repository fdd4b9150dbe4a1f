// Instantiations of the tcgen05 convolution kernel for 128-channel tiles staged in 64-channel
// slabs (a translation unit of its own so that the tile shapes compile in parallel).
#include "conv_tc_dev.cuh"

namespace occ {

bool tc_launch_128_64(const TcParams &p, int mode, int grid, size_t smem, cudaStream_t s) {
  return tc_launch_mode<128, 64, true>(p, mode, grid, smem, s);
}

bool tc_launch_128_64_duo(const TcParams &p, int mode, int grid, size_t smem, cudaStream_t s) {
  return tc_launch_mode_duo<128, 64>(p, mode, grid, smem, s);
}

}  // namespace occ
