// C ABI of libdswarm_cuda.so.  Every entry point takes raw device pointers and
// the stream to launch on, returns 0 on success or a negative code, and never
// synchronises.  Kernels that can wait (mbarriers, peer flags) report give-ups
// through an int status word in device memory (see ptx.cuh for the codes).
#pragma once
#include <cuda_runtime.h>

// Largest grid of the cross-GPU kernels: one wave on a 148-SM part, so every
// block is resident while it waits for its counterpart on the peers.
#define DSW_MAX_COLL_BLOCKS 148

#ifdef __cplusplus
extern "C" {
#endif

int dsw_gemm_bf16(const void* A, long long lda, int a_mn_major, const void* B, long long ldb, int b_mn_major,
                  int M, int N, int K, int mode, int split_k, void* out, long long ldo, const float* bias,
                  const void* resid, long long ldr, void* aux_out, const void* aux_in, long long ldaux, int bn,
                  int max_ctas, int* status, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
