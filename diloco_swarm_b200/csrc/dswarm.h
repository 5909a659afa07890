// C ABI of libdswarm_cuda.so: every exported entry point, in one place.
//
// Conventions.  Every entry point takes raw device pointers and the stream to
// launch on, returns 0 on success or a negative code, and never synchronises.
// bf16 arrays are passed as void*, fp32 arrays as float*, token ids / targets /
// masks as 64-bit integers.  Return codes: -3 a launch failed, -10 a shape the
// kernel does not cover (sizes must be multiples of 8 elements unless noted),
// -11 a pointer that is not 16-byte aligned, -12 an unknown tile width.
// Kernels that can wait (mbarriers, peer flags) never spin without a limit: a
// wait that runs out writes a code into the optional `status` word in device
// memory (1 = an mbarrier wait ran out, 2 = a peer GPU did not arrive,
// 3 = an index was out of range) and the kernel returns.
//
// Every source file of the library includes this header, so a definition that
// drifts from its declaration here does not compile.
#pragma once
#include <stddef.h>
#include <cuda_runtime.h>

// Largest grid of the cross-GPU kernels: one wave on a 148-SM part, so every
// block is resident while it waits for its counterpart on the peers.
#define DSW_MAX_COLL_BLOCKS 148

// Epilogue modes of dsw_gemm_bf16.
#define DSW_EPI_STORE 0       // out(bf16) = acc (+ bias)
#define DSW_EPI_GELU 1        // out(bf16) = gelu(acc + bias), exact erf form; aux_out (bf16, optional) = gelu'(acc + bias)
#define DSW_EPI_RESID 2       // out(bf16) = acc + bias + resid
#define DSW_EPI_MUL 3         // out(bf16) = acc * aux_in (with the aux_out of DSW_EPI_GELU: the GELU backward)
#define DSW_EPI_ATOMIC_F32 4  // out(fp32) += acc, safe under split-K
#define DSW_EPI_STORE_F32 5   // out(fp32) = acc

#ifdef __cplusplus
extern "C" {
#endif

// ---------------------------------------------------------------- GEMM (gemm_tcgen05.cu)
// out[M,N] = A * B^T-or-B with fp32 accumulation on the tcgen05 tensor cores.
// A: [M,K] row-major (a_mn_major = 0) or [K,M] row-major (1); B: [N,K] (b_mn_major = 0) or [K,N] (1);
// lda/ldb/ldo/ldr/ldaux are row pitches in elements.  bn = 128 or 256 picks the one-CTA tile width,
// 512 the CTA-pair kernel (256 x 256 per pair).  split_k > 1 only with DSW_EPI_ATOMIC_F32.
// max_ctas > 0 caps the grid.
int dsw_gemm_bf16(const void* A, long long lda, int a_mn_major, const void* B, long long ldb, int b_mn_major,
                  int M, int N, int K, int mode, int split_k, void* out, long long ldo, const float* bias,
                  const void* resid, long long ldr, void* aux_out, const void* aux_in, long long ldaux, int bn,
                  int max_ctas, int* status, cudaStream_t stream);
// Tracing build of the library only (-DDSWARM_TRACE): device buffer of 512 int64 that receives the timeline
// stamps of CTA 0's MMA thread and first epilogue warp (null switches it off).  A no-op in the shipped build.
int dsw_gemm_set_trace(long long* buf);

// ---------------------------------------------------------------- attention (attention.cu)
// Causal flash attention over a packed activation qkv: bf16 [B*T, 3*nh*hs] (Q | K | V, head h at columns
// h*hs of each).  out: bf16 [B*T, nh*hs]; lse: fp32 [B*nh*T].  hs is 64 or 32, T a multiple of 128.
int dsw_attention_fwd(const void* qkv, void* out, float* lse, int B, int T, int nh, int hs, float scale,
                      int* status, cudaStream_t st);
// dqkv: bf16 like qkv.  dq_acc: fp32 [B*T, nh*hs] and Dvec: fp32 [B*nh*T] are work arrays, contents irrelevant.
int dsw_attention_bwd(const void* qkv, const void* out, const void* dout, const float* lse, void* dqkv,
                      float* dq_acc, float* Dvec, int B, int T, int nh, int hs, float scale, int* status,
                      cudaStream_t st);
int dsw_attention_set_trace(long long* buf);

// ---------------------------------------------------------------- LayerNorm, embedding, loss, casts (elementwise.cu)
// x, y: bf16 [M, d]; gamma, beta: fp32 [d]; mean, rstd: fp32 [M] (written).  d <= 2048.
int dsw_layernorm_fwd(const void* x, const float* gamma, const float* beta, void* y, float* mean, float* rstd,
                      int M, int d, float eps, cudaStream_t st);
// Number of blocks dsw_layernorm_bwd launches for M rows = rows of scratch it needs.
int dsw_layernorm_bwd_blocks(int M);
// dx = LayerNorm backward of dy (+ dres when given: the residual branch's gradient).  dgamma, dbeta and the
// optional dres_sum (column sum of dres) are fp32 [d] and are accumulated (+=).
// scratch: fp32 [dsw_layernorm_bwd_blocks(M)][3][d], contents irrelevant on entry.
int dsw_layernorm_bwd(const void* dy, const void* x, const float* gamma, const float* mean, const float* rstd,
                      const void* dres, void* dx, float* dgamma, float* dbeta, float* dres_sum, float* scratch,
                      int M, int d, cudaStream_t st);
// out[N] (fp32) += column sums of x: bf16 [M, N] with row pitch ld.
int dsw_colsum_accum(const void* x, long long ld, float* out, int M, int N, cudaStream_t st);
// y[b,t,:] = bf16(wte[ids[b,t]] + wpe[t]); an id outside [0, V) sets status 3 and reads row 0.
int dsw_embedding_fwd(const long long* ids, const float* wte, const float* wpe, void* y, int B, int T, int d, int V,
                      int* status, cudaStream_t st);
// dwte[ids[b,t]] += dx[b,t], dwpe[t] += sum_b dx[b,t]; fp32 atomics for the token rows.
int dsw_embedding_bwd(const long long* ids, const void* dx, float* dwte, float* dwpe, int B, int T, int d, int V,
                      cudaStream_t st);
// The same sums in a fixed order: sorted / perm = stable ascending sort of the B*T ids and their positions.
int dsw_embedding_bwd_sorted(const long long* sorted, const long long* perm, const void* dx, float* dwte,
                             float* dwpe, int B, int T, int d, int V, cudaStream_t st);
// count[0] += number of non-zero mask entries; the caller clears count first.
int dsw_mask_count(const long long* mask, int M, float* count, cudaStream_t st);
// Masked mean cross-entropy over bf16 logits [M, V] (row pitch ld): loss_acc += scale * mean loss; with
// write_grad the logits are overwritten by d(loss)/d(logits).  mask may be null (count must then hold M).
int dsw_cross_entropy(void* logits, long long ld, const long long* targets, const long long* mask,
                      const float* count, float scale, float* loss_acc, int M, int V, int write_grad, int* status,
                      cudaStream_t st);
int dsw_cast_f32_bf16(const float* src, void* dst, long long n, cudaStream_t st);
int dsw_cast_bf16_f32(const void* src, float* dst, long long n, cudaStream_t st);

// ---------------------------------------------------------------- optimisers (optim.cu)
// stats: device float[3] = {sum of squares, norm, clip coefficient}; stats[0] must be zero before the
// first dsw_sumsq of a step.  dsw_clip_coef turns the sum into the norm and min(1, max_norm / norm).
int dsw_sumsq(const float* g, long long n, float* stats, cudaStream_t st);
int dsw_clip_coef(float* stats, float max_norm, cudaStream_t st);
// One pass over flat fp32 buffers: g *= coef[0] (when coef is given), decoupled-weight-decay Adam,
// p16 = bf16(p), optionally g = 0.  step is the 1-based optimiser step.
int dsw_adamw(float* p, float* g, float* m, float* v, void* p16, long long n, float lr, float b1, float b2,
              float eps, float wd, int step, const float* coef, int zero_grad, cudaStream_t st);
// SGD with optional (Nesterov) momentum; buf may be null when mu == 0.
int dsw_sgd(float* p, float* g, float* buf, void* p16, long long n, float lr, float mu, int nesterov,
            const float* coef, int zero_grad, cudaStream_t st);

// ---------------------------------------------------------------- symmetric memory and fused collectives (collectives.cu)
// A buffer that the other replicas of a stage can map: allocate (zero-filled), export a 64-byte CUDA IPC
// handle, import a peer's handle, and the matching release calls.
int dsw_symm_alloc(size_t bytes, void** ptr);
int dsw_symm_free(void* ptr);
int dsw_symm_export(void* ptr, void* handle64);
int dsw_symm_import(const void* handle64, void** ptr);
int dsw_symm_unimport(void* ptr);
int dsw_max_peers();
// Stream-ordered flags and copies without kernels (the copy-engine pipeline transport): the stream waits
// until the 32-bit word at addr (this device's memory) is >= value; the stream writes value to addr (own or
// mapped peer memory) after all earlier work on it; the stream copies bytes between device pointers (either
// may be a mapped peer buffer).  -1: the driver lacks stream memory operations.
int dsw_stream_wait_geq32(void* addr, unsigned value, cudaStream_t st);
int dsw_stream_write32(void* addr, unsigned value, cudaStream_t st);
int dsw_copy_async(void* dst, const void* src, size_t bytes, cudaStream_t st);
// bufs / flags: host arrays of R device pointers in replica order (this replica's own buffer at index
// `rank`).  seq: a number that grows by 2 per call, the same on every replica.  wait_limit <= 0 picks the
// default bound of the peer waits; use_barrier = 0 (single-GPU arithmetic checks) skips them; blocks <= 0
// picks the default grid.  Replica `rank` owns elements [rank*shard, (rank+1)*shard).
// DiLoCo outer step: mean of the replicas' weights, pseudo-gradient against theta_g, (Nesterov) momentum
// update of the owned shard, new weights stored into every replica.
int dsw_outer_sync(void* const* bufs, void* const* flags, float* theta_g, float* mom, long long n, long long shard,
                   int rank, int R, float lr, float mu, int nesterov, unsigned seq, long long wait_limit,
                   int use_barrier, int blocks, int* status, cudaStream_t st);
// Average of grad[offset, offset+count) over the replicas, fp32 or bf16 on the wire (bufs then holds the
// bf16 staging buffers).  phase_mask = 7 in real runs; its bits (1 cast-in, 2 reduce, 4 widen-out) let a
// single-GPU arithmetic check run the phases of the emulated replicas one after the other.
int dsw_grad_allreduce(void* const* bufs, void* const* flags, float* grad, long long offset, long long count,
                       long long shard, int rank, int R, int wire_bf16, unsigned seq, long long wait_limit,
                       int use_barrier, int phase_mask, int blocks, int* status, cudaStream_t st);

// The same two with the reduction inside the NVSwitch (multimem.ld_reduce / multimem.st): mc is the multicast
// address of the buffer whose unicast views are bufs[0..R-1] (for wire_bf16 the bf16 staging buffers).  R >= 2.
int dsw_outer_sync_nvls(void* const* bufs, void* mc, void* const* flags, float* theta_g, float* mom, long long n,
                        long long shard, int rank, int R, float lr, float mu, int nesterov, unsigned seq,
                        long long wait_limit, int blocks, int* status, cudaStream_t st);
int dsw_grad_allreduce_nvls(void* const* bufs, void* mc, void* const* flags, float* grad, long long offset,
                            long long count, long long shard, int rank, int R, int wire_bf16, unsigned seq,
                            long long wait_limit, int blocks, int* status, cudaStream_t st);

// ---------------------------------------------------------------- bounds-checking build (-DDSWARM_BOUNDS)
// First failed bounds check since the last call: 0 = none, else 100000 * unit + source line (units: 1
// elementwise.cu, 2 optim.cu, 3 collectives.cu, 4 gemm_one_cta.cu, 5 gemm_pair.cu).  The shipped build has no
// checks and returns 0.  The per-unit readers return that unit's line.
int dsw_bounds_status();
int dsw_bounds_elementwise();
int dsw_bounds_optim();
int dsw_bounds_collectives();
int dsw_bounds_gemm_one_cta();
int dsw_bounds_gemm_pair();
// Bounds build: one check fails on purpose, without touching memory, so that the report path can be tested
// (returns 1); shipped build: nothing happens (returns 0).
int dsw_bounds_selftest(cudaStream_t st);

// ---------------------------------------------------------------- module loading
// Load every kernel of a source file on the current device now, so that no first launch has to wait for
// the device to go idle while a pipeline receive is spinning on it.
int dsw_load_gemm();
int dsw_load_attention();
int dsw_load_elementwise();
int dsw_load_optim();
int dsw_load_collectives();

#ifdef __cplusplus
}
#endif
