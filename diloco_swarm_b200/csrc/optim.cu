// Fused optimiser kernels over flat fp32 buffers.
//
// Reference: clip_grad_norm_ over the rank's stage shard then torch AdamW with
// one parameter group (src/train.py:255-257, src/utils.py:61), i.e. foreach
// kernels over ~75 tensors with several passes each.  Here the stage's
// parameters, gradients and moments are single flat buffers: one pass computes
// the squared norm, one pass applies clip scale + AdamW, refreshes the bf16
// compute copy of the weights and clears the gradient.
#include "ptx.cuh"
#include "dswarm.h"

namespace dsw {

__global__ void __launch_bounds__(512)
sumsq_kernel(const float* __restrict__ g, long long n, float* __restrict__ out) {
  __shared__ float sh[16];
  float acc = 0.f;
  const long long n4 = n / 4;
  const float4* g4 = reinterpret_cast<const float4*>(g);
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n4; i += (long long)gridDim.x * blockDim.x) {
    if (!DSW_OK(4 * i + 4 <= n)) continue;
    const float4 v = g4[i];
    acc += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
  }
  if (blockIdx.x == 0 && threadIdx.x < n - n4 * 4) { const float v = g[n4 * 4 + threadIdx.x]; acc += v * v; }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  if ((threadIdx.x & 31) == 0) sh[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x < 32) {
    acc = threadIdx.x < (blockDim.x >> 5) ? sh[threadIdx.x] : 0.f;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
    if (threadIdx.x == 0) atomicAdd(out, acc);
  }
}

// stats[0] = sum of squares (input), stats[1] = norm, stats[2] = clip coefficient
// (torch.nn.utils.clip_grad_norm_: max_norm / (norm + 1e-6), clamped to 1).
__global__ void clip_coef_kernel(float* stats, float max_norm) {
  const float norm = sqrtf(stats[0]);
  stats[1] = norm;
  stats[2] = max_norm > 0.f ? fminf(1.f, max_norm / (norm + 1e-6f)) : 1.f;
}

__global__ void __launch_bounds__(512)
adamw_kernel(float* __restrict__ p, float* __restrict__ g, float* __restrict__ m, float* __restrict__ v,
             __nv_bfloat16* __restrict__ p16, long long n, float lr, float b1, float b2, float eps, float wd,
             float bias1, float bias2_sqrt, const float* __restrict__ coef_ptr, int zero_grad) {
  const float coef = coef_ptr ? coef_ptr[0] : 1.f;
  const float step_size = lr / bias1;
  const float decay = 1.f - lr * wd;
  const long long n4 = n / 4;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n4; i += (long long)gridDim.x * blockDim.x) {
    if (!DSW_OK(4 * i + 4 <= n)) continue;
    float4 pp = reinterpret_cast<float4*>(p)[i];
    float4 gg = reinterpret_cast<float4*>(g)[i];
    float4 mm = reinterpret_cast<float4*>(m)[i];
    float4 vv = reinterpret_cast<float4*>(v)[i];
    float* P = &pp.x; float* G = &gg.x; float* Mo = &mm.x; float* Vo = &vv.x;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float gr = G[j] * coef;
      Mo[j] = b1 * Mo[j] + (1.f - b1) * gr;
      Vo[j] = b2 * Vo[j] + (1.f - b2) * gr * gr;
      const float denom = sqrtf(Vo[j]) / bias2_sqrt + eps;
      P[j] = P[j] * decay - step_size * (Mo[j] / denom);
    }
    reinterpret_cast<float4*>(p)[i] = pp;
    reinterpret_cast<float4*>(m)[i] = mm;
    reinterpret_cast<float4*>(v)[i] = vv;
    if (zero_grad) reinterpret_cast<float4*>(g)[i] = make_float4(0.f, 0.f, 0.f, 0.f);
    if (p16) reinterpret_cast<uint2*>(p16)[i] = make_uint2(pack_bf16(pp.x, pp.y), pack_bf16(pp.z, pp.w));
  }
  // tail (n not a multiple of 4)
  if (blockIdx.x == 0 && threadIdx.x < n - n4 * 4) {
    const long long i = n4 * 4 + threadIdx.x;
    const float gr = g[i] * coef;
    const float mo = b1 * m[i] + (1.f - b1) * gr;
    const float vo = b2 * v[i] + (1.f - b2) * gr * gr;
    const float pv = p[i] * decay - step_size * (mo / (sqrtf(vo) / bias2_sqrt + eps));
    p[i] = pv; m[i] = mo; v[i] = vo;
    if (zero_grad) g[i] = 0.f;
    if (p16) p16[i] = __float2bfloat16(pv);
  }
}

// Plain SGD with optional (Nesterov) momentum, torch semantics, for --train.inner_optimizer @sgd.
__global__ void __launch_bounds__(512)
sgd_kernel(float* __restrict__ p, float* __restrict__ g, float* __restrict__ buf, __nv_bfloat16* __restrict__ p16,
           long long n, float lr, float mu, int nesterov, const float* __restrict__ coef_ptr, int zero_grad) {
  const float coef = coef_ptr ? coef_ptr[0] : 1.f;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    if (!DSW_OK(i >= 0 && i < n)) continue;
    const float gr = g[i] * coef;
    float upd = gr;
    if (mu != 0.f) {
      const float b = mu * buf[i] + gr;
      buf[i] = b;
      upd = nesterov ? gr + mu * b : b;
    }
    const float pv = p[i] - lr * upd;
    p[i] = pv;
    if (zero_grad) g[i] = 0.f;
    if (p16) p16[i] = __float2bfloat16(pv);
  }
}

}  // namespace dsw

using namespace dsw;

// stats is a device float[3]; stats[0] must be zero before the first dsw_sumsq of a step.
extern "C" int dsw_sumsq(const float* g, long long n, float* stats, cudaStream_t st) {
  if (reinterpret_cast<uintptr_t>(g) & 15) return -11;
  sumsq_kernel<<<148 * 2, 512, 0, st>>>(g, n, stats);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}
extern "C" int dsw_clip_coef(float* stats, float max_norm, cudaStream_t st) {
  clip_coef_kernel<<<1, 1, 0, st>>>(stats, max_norm);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}
// step is the 1-based optimiser step (bias correction); coef may be null.
extern "C" int dsw_adamw(float* p, float* g, float* m, float* v, void* p16, long long n, float lr, float b1, float b2,
                         float eps, float wd, int step, const float* coef, int zero_grad, cudaStream_t st) {
  if ((reinterpret_cast<uintptr_t>(p) | reinterpret_cast<uintptr_t>(g) | reinterpret_cast<uintptr_t>(m) |
       reinterpret_cast<uintptr_t>(v)) & 15)
    return -11;
  const float bias1 = 1.f - powf(b1, (float)step);
  const float bias2_sqrt = sqrtf(1.f - powf(b2, (float)step));
  adamw_kernel<<<148 * 4, 512, 0, st>>>(p, g, m, v, (__nv_bfloat16*)p16, n, lr, b1, b2, eps, wd, bias1, bias2_sqrt,
                                        coef, zero_grad);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}
extern "C" int dsw_sgd(float* p, float* g, float* buf, void* p16, long long n, float lr, float mu, int nesterov,
                       const float* coef, int zero_grad, cudaStream_t st) {
  sgd_kernel<<<148 * 4, 512, 0, st>>>(p, g, buf, (__nv_bfloat16*)p16, n, lr, mu, nesterov, coef, zero_grad);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

DSW_BOUNDS_TU(dsw_bounds_optim)

extern "C" int dsw_load_optim() {
  cudaFuncAttributes a;
  int bad = 0;
  bad |= cudaFuncGetAttributes(&a, sumsq_kernel) != cudaSuccess;
  bad |= cudaFuncGetAttributes(&a, clip_coef_kernel) != cudaSuccess;
  bad |= cudaFuncGetAttributes(&a, adamw_kernel) != cudaSuccess;
  bad |= cudaFuncGetAttributes(&a, sgd_kernel) != cudaSuccess;
  return bad ? -1 : 0;
}
