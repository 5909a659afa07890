// The two stage-wide synchronisations as single kernels over peer memory, and
// the small runtime that gives every replica pointers into its peers' buffers.
//
// (1) DiLoCo outer sync.  Reference (src/train.py:261-269, src/utils.py:213-226,
//     src/comm.py:117-123): copy every parameter to the host, subtract, one gloo
//     all-reduce per parameter, torch SGD-Nesterov on the host copy, copy back.
//     Here replica r of a stage owns slice r of the flat parameter buffer.  One
//     kernel reads that slice of theta_local from all R replicas over NVLink
//     (plain peer loads), forms the mean, the pseudo-gradient against its shard
//     of theta_global, updates its shard of the momentum, and stores the new
//     weights into every replica's theta_local.  All replicas hold the same
//     theta_global, so mean_j(theta_g - theta_j) = theta_g - mean_j(theta_j)
//     and only the owner of a slice needs theta_global and momentum for it.
// (2) Per-step gradient all-reduce of plain SWARM (src/comm.py:117-123 on
//     gradients): same slice ownership; sum over peers, times 1/R, stored to
//     every peer.  Optional bf16 wire format: gradients are cast to bf16 into a
//     peer-visible staging buffer, summed in fp32, scaled, sent back as bf16
//     and widened into the fp32 main gradient, all inside the one kernel.
//
// Cross-GPU ordering: a block-level barrier over flag words in each replica's
// own memory.  Arrival = st.release.sys of a sequence number into the peer's
// flag; wait = bounded ld.acquire.sys polling of the local flag.  Sequence
// numbers only grow, so flags are never reset.  A wait that runs out writes
// ST_PEER_TIMEOUT to the status word and the kernel returns; nothing traps.
// Grids are at most one wave, so every block of every replica is resident
// while it waits for its counterpart.
#include <cuda.h>
#include <mutex>
#include "ptx.cuh"
#include "dswarm.h"
#include "coll_index.h"

namespace dsw {

constexpr int MAX_PEERS = 8;

struct PeerTable {
  void* buf[MAX_PEERS];          // the symmetric buffer on each replica
  uint32_t* flags[MAX_PEERS];    // flag words on each replica: [num_blocks][MAX_PEERS]
};

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// Barrier of block `blockIdx.x` with the same block on every replica.
// Returns false (for the whole block) if a peer did not arrive in time.
__device__ __forceinline__ bool peer_barrier(const PeerTable& pt, int rank, int R, uint32_t seq, long long limit,
                                             int* status, int* sh_ok) {
  __syncthreads();
  if (threadIdx.x == 0) *sh_ok = 1;
  __syncthreads();
  if (threadIdx.x < R) {
    const int peer = threadIdx.x;
    __threadfence_system();
    st_release_sys(pt.flags[peer] + blockIdx.x * MAX_PEERS + rank, seq);
    const uint32_t* mine = pt.flags[rank] + blockIdx.x * MAX_PEERS + peer;
    const long long t0 = clock64();
    while (int32_t(ld_acquire_sys(mine) - seq) < 0) {
      if (clock64() - t0 > limit) {
        *sh_ok = 0;
        if (status) atomicCAS(status, 0, ST_PEER_TIMEOUT);
        break;
      }
    }
  }
  __syncthreads();
  return *sh_ok != 0;
}

__device__ __forceinline__ float4 ld_f4(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ void st_f4(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }

struct OuterArgs {
  PeerTable pt;
  float* theta_g;     // this replica's shard of the global weights  [shard]
  float* mom;         // this replica's shard of the Nesterov buffer [shard]
  long long n;        // elements in the flat parameter buffer (multiple of 4)
  long long shard;    // elements per shard (multiple of 4); shard r = [r*shard, min(n,(r+1)*shard))
  int rank, R;
  float lr, mu;
  int nesterov;
  uint32_t seq;       // barrier uses seq and seq+1
  long long wait_limit;
  int use_barrier;    // 0 only when all "replicas" are emulated by sequential launches on one GPU
  int* status;
};

__global__ void __launch_bounds__(512)
outer_sync_kernel(OuterArgs a) {
  __shared__ int sh_ok;
  if (a.use_barrier && !peer_barrier(a.pt, a.rank, a.R, a.seq, a.wait_limit, a.status, &sh_ok)) return;
  const long long lo = (long long)a.rank * a.shard;
  const long long hi = min(a.n, lo + a.shard);
  const float invR = 1.f / a.R;
  const long long stride = 4LL * gridDim.x * blockDim.x;
  // two independent float4 columns per thread and iteration: all 2R peer loads are issued before
  // the first one is consumed, which doubles the bytes each thread keeps in flight on the links
  for (long long i0 = lo + 4 * (blockIdx.x * (long long)blockDim.x + threadIdx.x); i0 < hi; i0 += 2 * stride) {
    const long long idx[2] = {i0, i0 + stride};
    float4 s[2] = {make_float4(0.f, 0.f, 0.f, 0.f), make_float4(0.f, 0.f, 0.f, 0.f)};
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      if (idx[u] < hi && DSW_OK(idx[u] >= 0 && idx[u] + 4 <= a.n)) {
#pragma unroll
        for (int j = 0; j < MAX_PEERS; ++j) {
          if (j < a.R) {
            const float4 v = ld_f4(reinterpret_cast<const float*>(a.pt.buf[j]) + idx[u]);
            s[u].x += v.x; s[u].y += v.y; s[u].z += v.z; s[u].w += v.w;
          }
        }
      }
    }
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      if (idx[u] >= hi) continue;
      const long long i = idx[u];
      const long long k = i - lo;
      float4 tg = ld_f4(a.theta_g + k);
      float4 mb = ld_f4(a.mom + k);
      float* S = &s[u].x; float* T = &tg.x; float* B = &mb.x;
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const float delta = T[c] - S[c] * invR;              // averaged pseudo-gradient
        float upd = delta;
        if (a.mu != 0.f) {
          B[c] = a.mu * B[c] + delta;                        // first step: buffer starts at 0, so it becomes delta
          upd = a.nesterov ? delta + a.mu * B[c] : B[c];
        }
        T[c] = T[c] - a.lr * upd;
      }
      st_f4(a.theta_g + k, tg);
      st_f4(a.mom + k, mb);
#pragma unroll
      for (int j = 0; j < MAX_PEERS; ++j)
        if (j < a.R) st_f4(reinterpret_cast<float*>(a.pt.buf[j]) + i, tg);
    }
  }
  if (a.use_barrier) peer_barrier(a.pt, a.rank, a.R, a.seq + 1, a.wait_limit, a.status, &sh_ok);
}

struct GradArgs {
  PeerTable pt;        // fp32 wire: the main-gradient buffers; bf16 wire: the staging buffers
  float* grad;         // this replica's fp32 main gradient (same as pt.buf[rank] for the fp32 wire)
  long long offset;    // bucket start (elements, multiple of 8)
  long long count;     // bucket length (multiple of 8)
  long long shard;     // per-replica slice of the bucket (multiple of 8)
  int rank, R;
  float scale;         // 1/R
  uint32_t seq;        // uses seq .. seq+1
  long long wait_limit;
  int use_barrier;
  int phase_mask;      // emulation only: bit0 cast-in, bit1 reduce, bit2 widen-out (all set in real runs)
  int* status;
};

__global__ void __launch_bounds__(512)
grad_allreduce_f32_kernel(GradArgs a) {
  __shared__ int sh_ok;
  if (a.use_barrier && !peer_barrier(a.pt, a.rank, a.R, a.seq, a.wait_limit, a.status, &sh_ok)) return;
  const long long lo = a.offset + (long long)a.rank * a.shard;
  const long long hi = min(a.offset + a.count, lo + a.shard);
  const long long stride = 4LL * gridDim.x * blockDim.x;
  for (long long i0 = lo + 4 * (blockIdx.x * (long long)blockDim.x + threadIdx.x); i0 < hi; i0 += 2 * stride) {
    const long long idx[2] = {i0, i0 + stride};          // two columns per thread: 2R peer loads in flight
    float4 s[2] = {make_float4(0.f, 0.f, 0.f, 0.f), make_float4(0.f, 0.f, 0.f, 0.f)};
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      if (idx[u] < hi && DSW_OK(idx[u] >= 0 && idx[u] + 4 <= a.offset + a.count)) {
#pragma unroll
        for (int j = 0; j < MAX_PEERS; ++j) {
          if (j < a.R) {
            const float4 v = ld_f4(reinterpret_cast<const float*>(a.pt.buf[j]) + idx[u]);
            s[u].x += v.x; s[u].y += v.y; s[u].z += v.z; s[u].w += v.w;
          }
        }
      }
    }
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      if (idx[u] >= hi) continue;
      s[u].x *= a.scale; s[u].y *= a.scale; s[u].z *= a.scale; s[u].w *= a.scale;
#pragma unroll
      for (int j = 0; j < MAX_PEERS; ++j)
        if (j < a.R) st_f4(reinterpret_cast<float*>(a.pt.buf[j]) + idx[u], s[u]);
    }
  }
  if (a.use_barrier) peer_barrier(a.pt, a.rank, a.R, a.seq + 1, a.wait_limit, a.status, &sh_ok);
}

// bf16 wire.  Three phases separated by the per-block barrier; all three walk the bucket with the
// slice-wise map of coll_index.h, so the vectors block b reads after a barrier are exactly those block b
// of the owning replica wrote before it (a plain grid-stride over the whole bucket would not give that:
// with slices that are not a multiple of the grid's stride, block b would read what another block of
// the peer wrote, and nobody waits for that block).
__global__ void __launch_bounds__(512)
grad_allreduce_bf16_kernel(GradArgs a) {
  __shared__ int sh_ok;
  const long long tid = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  const long long nth = (long long)gridDim.x * blockDim.x;
  __nv_bfloat16* stage = reinterpret_cast<__nv_bfloat16*>(a.pt.buf[a.rank]);
  // phase 0: own fp32 gradient -> bf16 staging (peer-visible), every slice
  if (a.phase_mask & 1) {
    dsw_for_each_owned(a.offset, a.count, a.shard, 0, a.R, tid, nth, 8, [&](long long i) {
      if (!DSW_OK(i >= a.offset && i + 8 <= a.offset + a.count)) return;
      const float4 x = ld_f4(a.grad + i), y = ld_f4(a.grad + i + 4);
      *reinterpret_cast<uint4*>(stage + i) =
          make_uint4(pack_bf16(x.x, x.y), pack_bf16(x.z, x.w), pack_bf16(y.x, y.y), pack_bf16(y.z, y.w));
    });
  }
  if (a.use_barrier && !peer_barrier(a.pt, a.rank, a.R, a.seq, a.wait_limit, a.status, &sh_ok)) return;
  // phase 1: reduce my slice over all peers in fp32, scale, send back as bf16
  if (a.phase_mask & 2) {
    dsw_for_each_owned(a.offset, a.count, a.shard, a.rank, a.rank + 1, tid, nth, 8, [&](long long i) {
      if (!DSW_OK(i >= a.offset && i + 8 <= a.offset + a.count)) return;
      float s[8] = {0, 0, 0, 0, 0, 0, 0, 0};
#pragma unroll
      for (int j = 0; j < MAX_PEERS; ++j) {
        if (j < a.R) {
          const uint4 u = *reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(a.pt.buf[j]) + i);
          const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
          for (int c = 0; c < 4; ++c) { const float2 f = unpack_bf16(w[c]); s[2 * c] += f.x; s[2 * c + 1] += f.y; }
        }
      }
      const uint4 o = make_uint4(pack_bf16(s[0] * a.scale, s[1] * a.scale), pack_bf16(s[2] * a.scale, s[3] * a.scale),
                                 pack_bf16(s[4] * a.scale, s[5] * a.scale), pack_bf16(s[6] * a.scale, s[7] * a.scale));
#pragma unroll
      for (int j = 0; j < MAX_PEERS; ++j)
        if (j < a.R) *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(a.pt.buf[j]) + i) = o;
    });
  }
  if (a.use_barrier && !peer_barrier(a.pt, a.rank, a.R, a.seq + 1, a.wait_limit, a.status, &sh_ok)) return;
  // phase 2: widen the averaged bucket into the fp32 main gradient, every slice
  if (a.phase_mask & 4) {
    dsw_for_each_owned(a.offset, a.count, a.shard, 0, a.R, tid, nth, 8, [&](long long i) {
      if (!DSW_OK(i >= a.offset && i + 8 <= a.offset + a.count)) return;
      const uint4 u = *reinterpret_cast<const uint4*>(stage + i);
      const float2 f0 = unpack_bf16(u.x), f1 = unpack_bf16(u.y), f2 = unpack_bf16(u.z), f3 = unpack_bf16(u.w);
      st_f4(a.grad + i, make_float4(f0.x, f0.y, f1.x, f1.y));
      st_f4(a.grad + i + 4, make_float4(f2.x, f2.y, f3.x, f3.y));
    });
  }
}

// ------------------------------------------------------------------ NVLS variants
// The same two synchronisations with the reduction done inside the NVSwitch: the buffers are bound to a
// multicast object, `multimem.ld_reduce` on the multicast address returns the sum over all replicas of one
// 16-byte vector (one load crosses this GPU's links instead of R - 1), and `multimem.st` stores a vector into
// every replica at once (one store instead of R).  Per GPU and direction the links then carry 1/R of the
// buffer in and 1/R out, against (R - 1)/R each way for the peer-load kernels.  Slice ownership, the flag
// barrier (plain peer stores / loads on the flag words) and the bounded waits are unchanged.
__device__ __forceinline__ float4 mm_ld_reduce_f4(const float* mc) {
  float4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0, %1, %2, %3}, [%4];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(mc) : "memory");
  return v;
}
__device__ __forceinline__ void mm_st_f4(float* mc, float4 v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};"
               ::"l"(mc), "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w) : "memory");
}
// eight bf16 values: summed over the replicas with fp32 accumulation inside the switch
__device__ __forceinline__ uint4 mm_ld_reduce_bf16x8(const __nv_bfloat16* mc) {
  uint4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(mc) : "memory");
  return v;
}
__device__ __forceinline__ void mm_st_bf16x8(__nv_bfloat16* mc, uint4 v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.bf16x2 [%0], {%1, %2, %3, %4};"
               ::"l"(mc), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}

__global__ void __launch_bounds__(512)
outer_sync_nvls_kernel(OuterArgs a, float* mc) {
  __shared__ int sh_ok;
  if (a.use_barrier && !peer_barrier(a.pt, a.rank, a.R, a.seq, a.wait_limit, a.status, &sh_ok)) return;
  const long long lo = (long long)a.rank * a.shard;
  const long long hi = min(a.n, lo + a.shard);
  const float invR = 1.f / a.R;
  const long long stride = 4LL * gridDim.x * blockDim.x;
  for (long long i0 = lo + 4 * (blockIdx.x * (long long)blockDim.x + threadIdx.x); i0 < hi; i0 += 2 * stride) {
    const long long idx[2] = {i0, i0 + stride};
    float4 s[2];
#pragma unroll
    for (int u = 0; u < 2; ++u)
      if (idx[u] < hi && DSW_OK(idx[u] >= 0 && idx[u] + 4 <= a.n)) s[u] = mm_ld_reduce_f4(mc + idx[u]);
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      if (idx[u] >= hi) continue;
      const long long k = idx[u] - lo;
      float4 tg = ld_f4(a.theta_g + k);
      float4 mb = ld_f4(a.mom + k);
      float* S = &s[u].x; float* T = &tg.x; float* B = &mb.x;
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const float delta = T[c] - S[c] * invR;
        float upd = delta;
        if (a.mu != 0.f) {
          B[c] = a.mu * B[c] + delta;
          upd = a.nesterov ? delta + a.mu * B[c] : B[c];
        }
        T[c] = T[c] - a.lr * upd;
      }
      st_f4(a.theta_g + k, tg);
      st_f4(a.mom + k, mb);
      mm_st_f4(mc + idx[u], tg);
    }
  }
  if (a.use_barrier) peer_barrier(a.pt, a.rank, a.R, a.seq + 1, a.wait_limit, a.status, &sh_ok);
}

__global__ void __launch_bounds__(512)
grad_allreduce_nvls_f32_kernel(GradArgs a, float* mc) {
  __shared__ int sh_ok;
  if (a.use_barrier && !peer_barrier(a.pt, a.rank, a.R, a.seq, a.wait_limit, a.status, &sh_ok)) return;
  const long long tid = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  const long long nth = (long long)gridDim.x * blockDim.x;
  dsw_for_each_owned(a.offset, a.count, a.shard, a.rank, a.rank + 1, tid, nth, 4, [&](long long i) {
    if (!DSW_OK(i >= a.offset && i + 4 <= a.offset + a.count)) return;
    float4 s = mm_ld_reduce_f4(mc + i);
    s.x *= a.scale; s.y *= a.scale; s.z *= a.scale; s.w *= a.scale;
    mm_st_f4(mc + i, s);
  });
  if (a.use_barrier) peer_barrier(a.pt, a.rank, a.R, a.seq + 1, a.wait_limit, a.status, &sh_ok);
}

// bf16 wire through the switch: cast into the (multicast-bound) staging buffer, reduce the own slice with
// fp32 accumulation in the switch, scale, store to every replica's staging at once, widen.
__global__ void __launch_bounds__(512)
grad_allreduce_nvls_bf16_kernel(GradArgs a, __nv_bfloat16* mc) {
  __shared__ int sh_ok;
  const long long tid = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  const long long nth = (long long)gridDim.x * blockDim.x;
  __nv_bfloat16* stage = reinterpret_cast<__nv_bfloat16*>(a.pt.buf[a.rank]);
  dsw_for_each_owned(a.offset, a.count, a.shard, 0, a.R, tid, nth, 8, [&](long long i) {
    if (!DSW_OK(i >= a.offset && i + 8 <= a.offset + a.count)) return;
    const float4 x = ld_f4(a.grad + i), y = ld_f4(a.grad + i + 4);
    *reinterpret_cast<uint4*>(stage + i) =
        make_uint4(pack_bf16(x.x, x.y), pack_bf16(x.z, x.w), pack_bf16(y.x, y.y), pack_bf16(y.z, y.w));
  });
  if (a.use_barrier && !peer_barrier(a.pt, a.rank, a.R, a.seq, a.wait_limit, a.status, &sh_ok)) return;
  dsw_for_each_owned(a.offset, a.count, a.shard, a.rank, a.rank + 1, tid, nth, 8, [&](long long i) {
    if (!DSW_OK(i >= a.offset && i + 8 <= a.offset + a.count)) return;
    const uint4 u = mm_ld_reduce_bf16x8(mc + i);
    const uint32_t w[4] = {u.x, u.y, u.z, u.w};
    uint32_t o[4];
#pragma unroll
    for (int c = 0; c < 4; ++c) { const float2 f = unpack_bf16(w[c]); o[c] = pack_bf16(f.x * a.scale, f.y * a.scale); }
    mm_st_bf16x8(mc + i, make_uint4(o[0], o[1], o[2], o[3]));
  });
  if (a.use_barrier && !peer_barrier(a.pt, a.rank, a.R, a.seq + 1, a.wait_limit, a.status, &sh_ok)) return;
  dsw_for_each_owned(a.offset, a.count, a.shard, 0, a.R, tid, nth, 8, [&](long long i) {
    if (!DSW_OK(i >= a.offset && i + 8 <= a.offset + a.count)) return;
    const uint4 u = *reinterpret_cast<const uint4*>(stage + i);
    const float2 f0 = unpack_bf16(u.x), f1 = unpack_bf16(u.y), f2 = unpack_bf16(u.z), f3 = unpack_bf16(u.w);
    st_f4(a.grad + i, make_float4(f0.x, f0.y, f1.x, f1.y));
    st_f4(a.grad + i + 4, make_float4(f2.x, f2.y, f3.x, f3.y));
  });
}

static void fill_table(PeerTable& pt, void* const* bufs, void* const* flags, int R) {
  for (int j = 0; j < MAX_PEERS; ++j) {
    pt.buf[j] = j < R ? bufs[j] : nullptr;
    pt.flags[j] = j < R && flags ? reinterpret_cast<uint32_t*>(flags[j]) : nullptr;
  }
}

}  // namespace dsw

using namespace dsw;

// ------------------------------------------------------------------ runtime (IPC)
extern "C" int dsw_symm_alloc(size_t bytes, void** ptr) {
  if (cudaMalloc(ptr, bytes) != cudaSuccess) return -1;
  return cudaMemset(*ptr, 0, bytes) == cudaSuccess ? 0 : -2;
}
extern "C" int dsw_symm_free(void* ptr) { return cudaFree(ptr) == cudaSuccess ? 0 : -1; }
extern "C" int dsw_symm_export(void* ptr, void* handle64) {
  cudaIpcMemHandle_t h;
  if (cudaIpcGetMemHandle(&h, ptr) != cudaSuccess) return -1;
  static_assert(sizeof(h) == 64, "ipc handle size");
  memcpy(handle64, &h, 64);
  return 0;
}
extern "C" int dsw_symm_import(const void* handle64, void** ptr) {
  cudaIpcMemHandle_t h;
  memcpy(&h, handle64, 64);
  cudaError_t e = cudaIpcOpenMemHandle(ptr, h, cudaIpcMemLazyEnablePeerAccess);
  return e == cudaSuccess ? 0 : -(int)e;
}
extern "C" int dsw_symm_unimport(void* ptr) { return cudaIpcCloseMemHandle(ptr) == cudaSuccess ? 0 : -1; }
extern "C" int dsw_max_peers() { return MAX_PEERS; }

// ------------------------------------------------------------------ stream-ordered flags and copies
// What the copy-engine pipeline transport (parallel/ce_comm.py) is made of: a stream waits until a 32-bit
// word in device memory reaches a value, a stream writes such a word (also into a peer's memory), and a
// stream copies between two device pointers of which one may be a peer's.  None of the three runs a kernel,
// so a transfer that waits for its peer holds no SM (a posted NCCL receive is a resident kernel, and one
// blocked SM is enough to stretch a persistent GEMM with static tile assignment to two waves).
namespace {
typedef CUresult (*WaitValue32Fn)(CUstream, CUdeviceptr, cuuint32_t, unsigned int);
typedef CUresult (*WriteValue32Fn)(CUstream, CUdeviceptr, cuuint32_t, unsigned int);
WaitValue32Fn g_wait32 = nullptr;
WriteValue32Fn g_write32 = nullptr;
std::once_flag g_memops_once;
void load_memops() {
  std::call_once(g_memops_once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuStreamWaitValue32", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      g_wait32 = reinterpret_cast<WaitValue32Fn>(p);
    p = nullptr;
    if (cudaGetDriverEntryPoint("cuStreamWriteValue32", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      g_write32 = reinterpret_cast<WriteValue32Fn>(p);
  });
}
}  // namespace

// The stream waits until *addr >= value (unsigned, wrap-aware as the driver defines it).  addr: device memory
// of the current device, 4-byte aligned.
extern "C" int dsw_stream_wait_geq32(void* addr, unsigned value, cudaStream_t st) {
  load_memops();
  if (!g_wait32) return -1;
  if (reinterpret_cast<uintptr_t>(addr) & 3) return -11;
  const CUresult r = g_wait32(reinterpret_cast<CUstream>(st), reinterpret_cast<CUdeviceptr>(addr), value,
                              CU_STREAM_WAIT_VALUE_GEQ);
  return r == CUDA_SUCCESS ? 0 : -(int)r - 100;
}
// The stream stores value into *addr once everything queued before it is done.  addr may point into a peer's
// memory that this process has mapped.
extern "C" int dsw_stream_write32(void* addr, unsigned value, cudaStream_t st) {
  load_memops();
  if (!g_write32) return -1;
  if (reinterpret_cast<uintptr_t>(addr) & 3) return -11;
  const CUresult r = g_write32(reinterpret_cast<CUstream>(st), reinterpret_cast<CUdeviceptr>(addr), value,
                               CU_STREAM_WRITE_VALUE_DEFAULT);
  return r == CUDA_SUCCESS ? 0 : -(int)r - 100;
}
// Device-to-device copy on the stream (copy engines); either pointer may be a mapped peer buffer.
extern "C" int dsw_copy_async(void* dst, const void* src, size_t bytes, cudaStream_t st) {
  const cudaError_t e = cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToDevice, st);
  return e == cudaSuccess ? 0 : -(int)e - 100;
}

// ------------------------------------------------------------------ launchers
// bufs / flags: host arrays of R device pointers (replica order).  flags may be
// null when use_barrier == 0.  blocks <= 0 picks the default grid.
extern "C" int dsw_outer_sync(void* const* bufs, void* const* flags, float* theta_g, float* mom, long long n,
                              long long shard, int rank, int R, float lr, float mu, int nesterov, unsigned seq,
                              long long wait_limit, int use_barrier, int blocks, int* status, cudaStream_t st) {
  if (R < 1 || R > MAX_PEERS || n % 4 || shard % 4) return -10;
  OuterArgs a;
  fill_table(a.pt, bufs, flags, R);
  a.theta_g = theta_g; a.mom = mom; a.n = n; a.shard = shard; a.rank = rank; a.R = R;
  a.lr = lr; a.mu = mu; a.nesterov = nesterov; a.seq = seq;
  a.wait_limit = wait_limit > 0 ? wait_limit : WAIT_CYCLES_LIMIT;
  a.use_barrier = use_barrier; a.status = status;
  if (blocks <= 0) blocks = DSW_MAX_COLL_BLOCKS;
  if (blocks > DSW_MAX_COLL_BLOCKS) blocks = DSW_MAX_COLL_BLOCKS;
  outer_sync_kernel<<<blocks, 512, 0, st>>>(a);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

extern "C" int dsw_grad_allreduce(void* const* bufs, void* const* flags, float* grad, long long offset,
                                  long long count, long long shard, int rank, int R, int wire_bf16, unsigned seq,
                                  long long wait_limit, int use_barrier, int phase_mask, int blocks, int* status,
                                  cudaStream_t st) {
  if (R < 1 || R > MAX_PEERS || offset % 8 || count % 8 || shard % 8) return -10;
  GradArgs a;
  fill_table(a.pt, bufs, flags, R);
  a.grad = grad; a.offset = offset; a.count = count; a.shard = shard; a.rank = rank; a.R = R;
  a.scale = 1.f / R; a.seq = seq;
  a.wait_limit = wait_limit > 0 ? wait_limit : WAIT_CYCLES_LIMIT;
  a.use_barrier = use_barrier; a.phase_mask = phase_mask; a.status = status;
  if (blocks <= 0) blocks = DSW_MAX_COLL_BLOCKS;
  if (blocks > DSW_MAX_COLL_BLOCKS) blocks = DSW_MAX_COLL_BLOCKS;
  if (wire_bf16) grad_allreduce_bf16_kernel<<<blocks, 512, 0, st>>>(a);
  else           grad_allreduce_f32_kernel<<<blocks, 512, 0, st>>>(a);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

// NVLS variants: mc = the multicast address of the same buffer that bufs[rank] is this replica's unicast view
// of (the fp32 weights / gradient, or the bf16 staging buffer when wire_bf16 is set).  R >= 2.
extern "C" int dsw_outer_sync_nvls(void* const* bufs, void* mc, void* const* flags, float* theta_g, float* mom,
                                   long long n, long long shard, int rank, int R, float lr, float mu, int nesterov,
                                   unsigned seq, long long wait_limit, int blocks, int* status, cudaStream_t st) {
  if (R < 2 || R > MAX_PEERS || n % 4 || shard % 4 || mc == nullptr) return -10;
  OuterArgs a;
  fill_table(a.pt, bufs, flags, R);
  a.theta_g = theta_g; a.mom = mom; a.n = n; a.shard = shard; a.rank = rank; a.R = R;
  a.lr = lr; a.mu = mu; a.nesterov = nesterov; a.seq = seq;
  a.wait_limit = wait_limit > 0 ? wait_limit : WAIT_CYCLES_LIMIT;
  a.use_barrier = 1; a.status = status;
  if (blocks <= 0 || blocks > DSW_MAX_COLL_BLOCKS) blocks = DSW_MAX_COLL_BLOCKS;
  outer_sync_nvls_kernel<<<blocks, 512, 0, st>>>(a, reinterpret_cast<float*>(mc));
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

extern "C" int dsw_grad_allreduce_nvls(void* const* bufs, void* mc, void* const* flags, float* grad, long long offset,
                                       long long count, long long shard, int rank, int R, int wire_bf16, unsigned seq,
                                       long long wait_limit, int blocks, int* status, cudaStream_t st) {
  if (R < 2 || R > MAX_PEERS || offset % 8 || count % 8 || shard % 8 || mc == nullptr) return -10;
  GradArgs a;
  fill_table(a.pt, bufs, flags, R);
  a.grad = grad; a.offset = offset; a.count = count; a.shard = shard; a.rank = rank; a.R = R;
  a.scale = 1.f / R; a.seq = seq;
  a.wait_limit = wait_limit > 0 ? wait_limit : WAIT_CYCLES_LIMIT;
  a.use_barrier = 1; a.phase_mask = 7; a.status = status;
  if (blocks <= 0 || blocks > DSW_MAX_COLL_BLOCKS) blocks = DSW_MAX_COLL_BLOCKS;
  if (wire_bf16) grad_allreduce_nvls_bf16_kernel<<<blocks, 512, 0, st>>>(a, reinterpret_cast<__nv_bfloat16*>(mc));
  else           grad_allreduce_nvls_f32_kernel<<<blocks, 512, 0, st>>>(a, reinterpret_cast<float*>(mc));
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

DSW_BOUNDS_TU(dsw_bounds_collectives)

extern "C" int dsw_load_collectives() {
  cudaFuncAttributes a;
  int bad = 0;
  bad |= cudaFuncGetAttributes(&a, outer_sync_kernel) != cudaSuccess;
  bad |= cudaFuncGetAttributes(&a, grad_allreduce_f32_kernel) != cudaSuccess;
  bad |= cudaFuncGetAttributes(&a, grad_allreduce_bf16_kernel) != cudaSuccess;
  bad |= cudaFuncGetAttributes(&a, outer_sync_nvls_kernel) != cudaSuccess;
  bad |= cudaFuncGetAttributes(&a, grad_allreduce_nvls_f32_kernel) != cudaSuccess;
  bad |= cudaFuncGetAttributes(&a, grad_allreduce_nvls_bf16_kernel) != cudaSuccess;
  return bad ? -1 : 0;
}
