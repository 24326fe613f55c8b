// Launch of the partial-attention forward: picks the kernel for the head dimension.
//   D = 128  flash_fwd_row.cu   one thread per query row, exp turns between the two Q tiles' warps: the tensor
//                               pipe and the ex2 unit need the same 1024 clocks per 64-key step, and this
//                               schedule keeps both closest to busy (measured against the other kernel).
//   D = 64   flash_fwd_pair.cu  two threads per query row, three S buffers per Q tile: the ex2 unit needs twice
//                               the clocks of the tensor pipe, so what counts is how densely the softmax warps
//                               keep it fed.
// -DDTB_FLASH128_PAIR=1 builds the two-threads-per-row kernel for D = 128 as well (A/B measurements).
#include "flash_fwd_sm100.cuh"

namespace dtb {

template <int D>
cudaError_t launch_flash_row(const CUtensorMap&, const CUtensorMap&, const CUtensorMap&, const FlashParams&, cudaStream_t);
template <int D>
cudaError_t launch_flash_pair(const CUtensorMap&, const CUtensorMap&, const CUtensorMap&, const FlashParams&, cudaStream_t);

#ifndef DTB_FLASH128_PAIR
#define DTB_FLASH128_PAIR 0
#endif

template <>
cudaError_t launch_flash<128>(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv, const FlashParams& p,
                              cudaStream_t stream) {
#if DTB_FLASH128_PAIR
  return launch_flash_pair<128>(tq, tk, tv, p, stream);
#else
  return launch_flash_row<128>(tq, tk, tv, p, stream);
#endif
}

template <>
cudaError_t launch_flash<64>(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv, const FlashParams& p,
                             cudaStream_t stream) {
  return launch_flash_pair<64>(tq, tk, tv, p, stream);
}

// both kernels walk the keys in tiles of 64
int flash_kv_box_rows(int head_dim) {
  (void)head_dim;
  return 64;
}

#ifdef DTB_FLASH_TIMING
cudaError_t read_flash_timing_row(long long* host, int n);
cudaError_t read_flash_timing_pair(long long* host, int n);
cudaError_t read_flash_timing(long long* host, int n, int head_dim) {
  return (head_dim == 128 && !DTB_FLASH128_PAIR) ? read_flash_timing_row(host, n) : read_flash_timing_pair(host, n);
}
#endif

}  // namespace dtb
