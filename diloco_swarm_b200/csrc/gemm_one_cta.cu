// Instantiations and launcher of the one-CTA tcgen05 GEMM kernel (gemm_kernels.cuh): 128 x 128 and
// 128 x 256 tiles, one instantiation per epilogue class.
#include "gemm_kernels.cuh"
#include "dswarm.h"

namespace dsw {

namespace {
constexpr int kMaxDevices = 64;

template <int BN, int NSTAGE, int MODE>
int launch_one(const CUtensorMap& ta, const CUtensorMap& tb, const GemmArgs& g, int num_sms, int max_ctas,
               cudaStream_t st) {
  using L = SmemLayout<BN, NSTAGE>;
  static bool attr_set[kMaxDevices] = {false};          // the attribute is per device
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return -2;
  if (!attr_set[dev]) {
    if (cudaFuncSetAttribute(gemm_kernel<BN, NSTAGE, MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize, L::TOTAL) !=
        cudaSuccess)
      return -2;
    attr_set[dev] = true;
  }
  const int tiles = ((g.M + BM - 1) / BM) * ((g.N + BN - 1) / BN) * (g.split_k > 1 ? g.split_k : 1);
  int grid = tiles < num_sms ? tiles : num_sms;
  if (max_ctas > 0 && grid > max_ctas) grid = max_ctas;
  gemm_kernel<BN, NSTAGE, MODE><<<grid, GEMM_THREADS, L::TOTAL, st>>>(ta, tb, g);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

template <int BN, int NSTAGE>
int launch_bn(const CUtensorMap& ta, const CUtensorMap& tb, const GemmArgs& g, int num_sms, int max_ctas,
              cudaStream_t st) {
  switch (epi_class(g.mode)) {
    case EPI_GELU: return launch_one<BN, NSTAGE, EPI_GELU>(ta, tb, g, num_sms, max_ctas, st);
    case EPI_RESID: return launch_one<BN, NSTAGE, EPI_RESID>(ta, tb, g, num_sms, max_ctas, st);
    case EPI_MUL: return launch_one<BN, NSTAGE, EPI_MUL>(ta, tb, g, num_sms, max_ctas, st);
    case EPI_ATOMIC_F32: return launch_one<BN, NSTAGE, EPI_ATOMIC_F32>(ta, tb, g, num_sms, max_ctas, st);
    case EPI_STORE: return launch_one<BN, NSTAGE, EPI_STORE>(ta, tb, g, num_sms, max_ctas, st);
    default: return -13;
  }
}

template <int BN, int NSTAGE>
int load_bn() {
  cudaFuncAttributes a;
  int bad = 0;
  bad |= cudaFuncGetAttributes(&a, gemm_kernel<BN, NSTAGE, EPI_STORE>) != cudaSuccess;
  bad |= cudaFuncGetAttributes(&a, gemm_kernel<BN, NSTAGE, EPI_GELU>) != cudaSuccess;
  bad |= cudaFuncGetAttributes(&a, gemm_kernel<BN, NSTAGE, EPI_RESID>) != cudaSuccess;
  bad |= cudaFuncGetAttributes(&a, gemm_kernel<BN, NSTAGE, EPI_MUL>) != cudaSuccess;
  bad |= cudaFuncGetAttributes(&a, gemm_kernel<BN, NSTAGE, EPI_ATOMIC_F32>) != cudaSuccess;
  return bad;
}
}  // namespace

int launch_one_cta(int bn, const CUtensorMap& ta, const CUtensorMap& tb, const GemmArgs& g, int num_sms, int max_ctas,
                   cudaStream_t st) {
  if (bn == 256) return launch_bn<256, 4>(ta, tb, g, num_sms, max_ctas, st);
  return launch_bn<128, 6>(ta, tb, g, num_sms, max_ctas, st);
}

}  // namespace dsw
DSW_BOUNDS_TU(dsw_bounds_gemm_one_cta)
namespace dsw {

int load_one_cta_kernels() { return (load_bn<256, 4>() | load_bn<128, 6>()) ? -1 : 0; }

}  // namespace dsw
