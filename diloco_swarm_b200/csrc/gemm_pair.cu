// Instantiations and launcher of the CTA-pair tcgen05 GEMM kernel (gemm_kernels.cuh): 256 x 256 tiles on
// two CTAs of a cluster (cta_group::2), one instantiation per epilogue class.
#include "gemm_kernels.cuh"
#include "dswarm.h"

namespace dsw {

namespace {
constexpr int kMaxDevices = 64;

template <int MODE>
int launch_pair_mode(const CUtensorMap& ta, const CUtensorMap& tb, const GemmArgs& g, int num_sms, int max_ctas,
                     cudaStream_t st) {
  static bool attr_set[kMaxDevices] = {false};          // the attribute is per device
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return -2;
  if (!attr_set[dev]) {
    if (cudaFuncSetAttribute(gemm_pair_kernel<MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize, PairSmem::TOTAL) !=
        cudaSuccess)
      return -2;
    attr_set[dev] = true;
  }
  const int tiles = ((g.M + 255) / 256) * ((g.N + PAIR_BN - 1) / PAIR_BN) * (g.split_k > 1 ? g.split_k : 1);
  int pairs = num_sms / 2;
  if (max_ctas > 0 && pairs > max_ctas / 2) pairs = max_ctas / 2 > 0 ? max_ctas / 2 : 1;
  if (pairs > tiles) pairs = tiles;
  gemm_pair_kernel<MODE><<<2 * pairs, GEMM_THREADS, PairSmem::TOTAL, st>>>(ta, tb, g);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}
}  // namespace

int launch_pair(const CUtensorMap& ta, const CUtensorMap& tb, const GemmArgs& g, int num_sms, int max_ctas,
                cudaStream_t st) {
  switch (epi_class(g.mode)) {
    case EPI_GELU: return launch_pair_mode<EPI_GELU>(ta, tb, g, num_sms, max_ctas, st);
    case EPI_RESID: return launch_pair_mode<EPI_RESID>(ta, tb, g, num_sms, max_ctas, st);
    case EPI_MUL: return launch_pair_mode<EPI_MUL>(ta, tb, g, num_sms, max_ctas, st);
    case EPI_ATOMIC_F32: return launch_pair_mode<EPI_ATOMIC_F32>(ta, tb, g, num_sms, max_ctas, st);
    case EPI_STORE: return launch_pair_mode<EPI_STORE>(ta, tb, g, num_sms, max_ctas, st);
    default: return -13;
  }
}

}  // namespace dsw
DSW_BOUNDS_TU(dsw_bounds_gemm_pair)
namespace dsw {

int load_pair_kernels() {
  cudaFuncAttributes a;
  int bad = 0;
  bad |= cudaFuncGetAttributes(&a, gemm_pair_kernel<EPI_STORE>) != cudaSuccess;
  bad |= cudaFuncGetAttributes(&a, gemm_pair_kernel<EPI_GELU>) != cudaSuccess;
  bad |= cudaFuncGetAttributes(&a, gemm_pair_kernel<EPI_RESID>) != cudaSuccess;
  bad |= cudaFuncGetAttributes(&a, gemm_pair_kernel<EPI_MUL>) != cudaSuccess;
  bad |= cudaFuncGetAttributes(&a, gemm_pair_kernel<EPI_ATOMIC_F32>) != cudaSuccess;
  return bad ? -1 : 0;
}

}  // namespace dsw
