// bf16 GEMM on the 5th-generation tensor cores: D[M,N] = op(A) * op(B), fp32
// accumulation in tensor memory, operands staged in shared memory by TMA.
//
// Replaces the library GEMMs behind the reference's nn.Linear calls and their
// autograd backward (src/model.py:44-45,83-84,118 and src/model.py:205-209):
//   forward   y  = x  W^T      A = x  [M,K] K-major,  B = W [N,K] K-major
//   dgrad     dx = dy W        A = dy [M,K] K-major,  B = W [K,N] N-major
//   wgrad     dW = dy^T x      A = dy [K,M] M-major,  B = x [K,N] N-major
// with the elementwise work fused into the epilogue (bias, exact GELU and its
// derivative, residual add, fp32 accumulation into the main gradient).
//
// Structure: persistent CTAs (one per SM), 320 threads.
//   warp 0      TMA producer: fills a ring of NSTAGE {A,B} k-blocks
//   warp 1      allocates TMEM, issues tcgen05.mma (one elected lane)
//   warps 2..9  epilogue: tcgen05.ld of the finished accumulator, math, stores
//               (two warps per TMEM lane quarter, each takes half of the columns)
// Two accumulators (2 x BN columns of TMEM) let the epilogue of tile i overlap
// the main loop of tile i+1.  No thread-block clusters and no multicast loads.
#include <cuda.h>
#include <cstdio>
#include <mutex>
#include "ptx.cuh"
#include "dswarm.h"

namespace dsw {

__device__ __forceinline__ long long gemm_gtimer() {
  long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
// In-kernel timeline stamps exist only in the tracing build of the library (-DDSWARM_TRACE, used by
// benchmarks/timelines.py); the shipped kernels carry none of it.
#ifdef DSWARM_TRACE
#define GEMM_TRACE(buf, slot) do { if ((buf) != nullptr && (slot) < 512) (buf)[(slot)++] = gemm_gtimer(); } while (0)
#else
#define GEMM_TRACE(buf, slot) do { } while (0)
#endif

constexpr int BM = 128;
constexpr int BK = 64;          // one 128-byte swizzle row of bf16
constexpr int UMMA_K = 16;
constexpr int EPI_WARPS = 8;          // two per TMEM lane quarter, each takes half of the tile's columns
constexpr int GEMM_THREADS = 32 * (2 + EPI_WARPS);

enum EpiMode : int {
  EPI_STORE = 0,        // out = acc (+ bias)
  EPI_GELU = 1,         // aux_out = acc + bias ; out = gelu(aux_out)
  EPI_RESID = 2,        // out = acc + bias + resid
  EPI_DGELU = 3,        // out = acc * gelu'(aux_in)
  EPI_ATOMIC_F32 = 4,   // out_f32 += acc   (split-K safe)
  EPI_STORE_F32 = 5,    // out_f32 = acc
};

struct GemmArgs {
  int M, N, K;
  int a_mn_major, b_mn_major;
  int mode;
  int split_k;
  void* out; long long ldo;
  const float* bias;
  const __nv_bfloat16* resid; long long ldr;
  __nv_bfloat16* aux_out; const __nv_bfloat16* aux_in; long long ldaux;
  int* status;
  long long* trace;     // optional: CTA 0's MMA thread stores %globaltimer stamps per k-block (tuning aid)
};

// ------------------------------------------------------------------ epilogue
// A thread owns one accumulator row (that is how tcgen05.ld hands the data out), but a store in
// which every lane writes 16 bytes of a different row touches 32 cache lines per instruction.  So
// each warp passes its 32-row slab through a private 4 KB tile of shared memory (32 rows x 128
// bytes, 16-byte chunks XOR-swizzled by row, conflict-free both ways) and writes it out with
// lane = (row within a group of 4, 16-byte chunk): every store, residual / aux load or fp32
// reduction instruction then covers 4 rows x 128 contiguous bytes.
//
// The accumulator is drained in chunks of 32 columns with the tcgen05.ld of chunk c+1 in flight
// while chunk c is converted, so a thread holds 64 accumulator registers at most.  Two chunks fill
// one bf16 slab (64 columns = 128 bytes per row); an fp32 chunk is a slab by itself.  Everything
// the slab needs from global memory besides the accumulator (bias, residual, GELU pre-activation)
// is requested at the top of the slab, before the wait for the accumulator, in one batch: issued
// one by one between the stores of the write-out, each load would cost a full memory round trip.
constexpr int EPI_STAGE_BYTES = 32 * 128;

// columns [16*q, 16*q + 16) of a 64-column bf16 slab (q = 0..3 -> 16-byte chunks 2q, 2q+1) ...
// generic form: `w` holds NW 32-bit words of this thread's row, starting at 16-byte chunk `c0`.
template <int NW>
__device__ __forceinline__ void stage_words(uint8_t* stage, int lane, int c0, const uint32_t (&w)[NW]) {
#pragma unroll
  for (int c = 0; c < NW / 4; ++c)
    *reinterpret_cast<uint4*>(stage + lane * 128 + (((c0 + c) ^ (lane & 7)) << 4)) =
        make_uint4(w[4 * c], w[4 * c + 1], w[4 * c + 2], w[4 * c + 3]);
}

// Visit the staged slab in write-out order: iteration i, this lane handles row i*4 + (lane >> 3),
// 16-byte chunk lane & 7.
template <class F>
__device__ __forceinline__ void unstage_rows(const uint8_t* stage, int lane, F&& emit) {
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int rl = i * 4 + (lane >> 3), ch = lane & 7;
    const uint4 d = *reinterpret_cast<const uint4*>(stage + rl * 128 + ((ch ^ (rl & 7)) << 4));
    emit(i, rl, ch, d);
  }
}

// NCOLS accumulator columns (a multiple of 64) starting at TMEM address t_addr, rows row_base..+31
// (one per lane), output columns col_base..+NCOLS-1.  `release` is called once, right after the last
// TMEM load has landed, so the MMA thread can refill the accumulator while the last slab is written.
template <int MODE, int NCOLS, class Release>
__device__ __forceinline__ void epilogue_warp(const GemmArgs& g, uint32_t t_addr, int row_base, int lane, int col_base,
                                              uint8_t* stage, Release&& release) {
  constexpr bool F32 = MODE == EPI_ATOMIC_F32 || MODE == EPI_STORE_F32;
  constexpr int NCH = NCOLS / 32;
  uint32_t r[2][32];
  tmem_ld_32x32(t_addr, r[0]);
  if constexpr (F32) {
#pragma unroll
    for (int c = 0; c < NCH; ++c) {
      tmem_ld_wait();
      if (c + 1 < NCH) tmem_ld_32x32(t_addr + (c + 1) * 32, r[(c + 1) & 1]);
      else release();
      const int cb = col_base + c * 32;
      if (cb >= g.N) continue;
      __syncwarp();                                   // the previous slab has been read out
      stage_words<32>(stage, lane, 0, r[c & 1]);
      __syncwarp();
      unstage_rows(stage, lane, [&](int, int rl, int ch, const uint4& d) {
        const int row = row_base + rl, col = cb + ch * 4;
        if (row < g.M && col < g.N) {
          float* o = reinterpret_cast<float*>(g.out) + (long long)row * g.ldo + col;
          if (MODE == EPI_ATOMIC_F32)
            asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(o), "f"(__uint_as_float(d.x)),
                         "f"(__uint_as_float(d.y)), "f"(__uint_as_float(d.z)), "f"(__uint_as_float(d.w))
                         : "memory");
          else
            *reinterpret_cast<uint4*>(o) = d;
        }
      });
    }
  } else {
    constexpr int NSLAB = NCOLS / 64;
    constexpr bool EXTRA = MODE == EPI_RESID || MODE == EPI_DGELU;
    const int my_ch = lane & 7, my_r = lane >> 3;
#pragma unroll
    for (int s = 0; s < NSLAB; ++s) {
      const int col0 = col_base + s * 64;
      const bool slab_ok = col0 < g.N;
      // ---- requests to global memory for this slab, all at once
      uint4 x[EXTRA ? 8 : 1];
      if constexpr (EXTRA) {
        const __nv_bfloat16* src = MODE == EPI_RESID ? g.resid : g.aux_in;
        const long long ld = MODE == EPI_RESID ? g.ldr : g.ldaux;
        const int col = col0 + my_ch * 8;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const int row = row_base + i * 4 + my_r;
          x[i] = (row < g.M && col < g.N) ? __ldg(reinterpret_cast<const uint4*>(src + (long long)row * ld + col))
                                          : make_uint4(0, 0, 0, 0);
        }
      }
      uint32_t post[MODE == EPI_GELU ? 32 : 1];      // gelu(acc + bias) of the slab, packed, until the pre-activation is out
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const int c = 2 * s + h;
        const int cb = col0 + h * 32;
        tmem_ld_wait();
        if (c + 1 < NCH) tmem_ld_32x32(t_addr + (c + 1) * 32, r[(c + 1) & 1]);
        else release();
        if (!slab_ok) continue;
        // bias (an L1 hit after the first tile row), add, round; the GELU value is formed from the same
        // fp32 sum and parked in registers until the pre-activation slab has been written out
        uint32_t w[16];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const float4 bb = (g.bias != nullptr && cb + 4 * i < g.N) ? __ldg(reinterpret_cast<const float4*>(g.bias + cb) + i)
                                                                   : make_float4(0.f, 0.f, 0.f, 0.f);
          const float v0 = __uint_as_float(r[c & 1][4 * i]) + bb.x, v1 = __uint_as_float(r[c & 1][4 * i + 1]) + bb.y;
          const float v2 = __uint_as_float(r[c & 1][4 * i + 2]) + bb.z, v3 = __uint_as_float(r[c & 1][4 * i + 3]) + bb.w;
          w[2 * i] = pack_bf16(v0, v1);
          w[2 * i + 1] = pack_bf16(v2, v3);
          if constexpr (MODE == EPI_GELU) {
            post[16 * h + 2 * i] = pack_bf16(gelu_fast(v0), gelu_fast(v1));
            post[16 * h + 2 * i + 1] = pack_bf16(gelu_fast(v2), gelu_fast(v3));
          }
        }
        if (h == 0) __syncwarp();                     // the previous slab has been read out
        stage_words<16>(stage, lane, 4 * h, w);
      }
      if (!slab_ok) continue;
      __syncwarp();
      if constexpr (MODE == EPI_GELU) {
        unstage_rows(stage, lane, [&](int, int rl, int ch, const uint4& d) {
          const int row = row_base + rl, col = col0 + ch * 8;
          if (row < g.M && col < g.N) *reinterpret_cast<uint4*>(g.aux_out + (long long)row * g.ldaux + col) = d;
        });
        __syncwarp();
        uint32_t w0[16], w1[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) { w0[i] = post[i]; w1[i] = post[16 + i]; }
        stage_words<16>(stage, lane, 0, w0);
        stage_words<16>(stage, lane, 4, w1);
        __syncwarp();
      }
      unstage_rows(stage, lane, [&](int i, int rl, int ch, uint4 d) {
        const int row = row_base + rl, col = col0 + ch * 8;
        if (row >= g.M || col >= g.N) return;
        if constexpr (EXTRA) {
          uint32_t du[4] = {d.x, d.y, d.z, d.w};
          const uint32_t xu[4] = {x[i].x, x[i].y, x[i].z, x[i].w};
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            const float2 a = unpack_bf16(du[q]), e = unpack_bf16(xu[q]);
            du[q] = MODE == EPI_RESID ? pack_bf16(a.x + e.x, a.y + e.y)
                                      : pack_bf16(a.x * gelu_grad_fast(e.x), a.y * gelu_grad_fast(e.y));
          }
          d = make_uint4(du[0], du[1], du[2], du[3]);
        }
        *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(g.out) + (long long)row * g.ldo + col) = d;
      });
    }
  }
}

// One tile's worth of epilogue for this warp, dispatched on the mode once per tile.
template <int NCOLS, class Release>
__device__ __forceinline__ void drain_tile(const GemmArgs& g, uint32_t t_addr, int row_base, int lane, int col_base,
                                           bool has_k, uint8_t* stage, Release&& release) {
  if (!has_k) { release(); return; }
  switch (g.mode) {
    case EPI_GELU: epilogue_warp<EPI_GELU, NCOLS>(g, t_addr, row_base, lane, col_base, stage, release); break;
    case EPI_RESID: epilogue_warp<EPI_RESID, NCOLS>(g, t_addr, row_base, lane, col_base, stage, release); break;
    case EPI_DGELU: epilogue_warp<EPI_DGELU, NCOLS>(g, t_addr, row_base, lane, col_base, stage, release); break;
    case EPI_ATOMIC_F32: epilogue_warp<EPI_ATOMIC_F32, NCOLS>(g, t_addr, row_base, lane, col_base, stage, release); break;
    case EPI_STORE_F32: epilogue_warp<EPI_STORE_F32, NCOLS>(g, t_addr, row_base, lane, col_base, stage, release); break;
    default: epilogue_warp<EPI_STORE, NCOLS>(g, t_addr, row_base, lane, col_base, stage, release); break;
  }
}

template <int BN, int NSTAGE>
struct SmemLayout {
  static constexpr int A_BYTES = BM * BK * 2;
  static constexpr int B_BYTES = BN * BK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int EPI_OFFSET = NSTAGE * STAGE_BYTES;              // per-warp epilogue staging tiles
  static constexpr int BAR_OFFSET = EPI_OFFSET + EPI_WARPS * EPI_STAGE_BYTES;
  static constexpr int TOTAL = BAR_OFFSET + 256 + 1024;   // barriers + alignment slack
};

template <int BN, int NSTAGE>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b, GemmArgs g) {
  using L = SmemLayout<BN, NSTAGE>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + L::BAR_OFFSET);
  uint64_t* empty_bar = full_bar + NSTAGE;
  uint64_t* acc_full = empty_bar + NSTAGE;      // [2]
  uint64_t* acc_empty = acc_full + 2;           // [2]
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(acc_empty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_holder + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  const int tiles_m = (g.M + BM - 1) / BM;
  const int tiles_n = (g.N + BN - 1) / BN;
  const int kb_total = (g.K + BK - 1) / BK;
  const int splits = g.split_k > 1 ? g.split_k : 1;
  const int kb_per_split = (kb_total + splits - 1) / splits;
  const int num_tiles = tiles_m * tiles_n * splits;

  if (threadIdx.x == 0) {
    for (int s = 0; s < NSTAGE; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
    for (int b = 0; b < 2; ++b) { mbar_init(&acc_full[b], 1); mbar_init(&acc_empty[b], EPI_WARPS); }
    *abort_flag = 0;
    mbar_fence_init();
    fence_proxy_async();
  }
  if (warp == 1) {
    tmem_alloc(tmem_holder, 2 * BN);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_holder;

  if (warp == 0) {
    // ------------------------------------------------------------ producer
    if (lane == 0) {
      tma_prefetch_desc(&tmap_a);
      tma_prefetch_desc(&tmap_b);
      uint32_t it = 0;
      bool ok = true;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
        const int ks = tile / (tiles_m * tiles_n);
        const int rem = tile - ks * tiles_m * tiles_n;
        const int m0 = (rem % tiles_m) * BM;
        const int n0 = (rem / tiles_m) * BN;
        const int kb0 = ks * kb_per_split;
        const int kb1 = min(kb_total, kb0 + kb_per_split);
        for (int kb = kb0; kb < kb1; ++kb, ++it) {
          const int s = it % NSTAGE;
          const uint32_t ph = (it / NSTAGE) & 1;
          if (!mbar_wait(&empty_bar[s], ph ^ 1, abort_flag, g.status)) { ok = false; break; }
          uint8_t* sa = smem + s * L::STAGE_BYTES;
          uint8_t* sb = sa + L::A_BYTES;
          mbar_expect_tx(&full_bar[s], L::STAGE_BYTES);
          const int k0 = kb * BK;
          if (!g.a_mn_major) {
            tma_load_2d(sa, &tmap_a, &full_bar[s], k0, m0);
          } else {
#pragma unroll
            for (int c = 0; c < BM / 64; ++c) tma_load_2d(sa + c * 8192, &tmap_a, &full_bar[s], m0 + 64 * c, k0);
          }
          if (!g.b_mn_major) {
            tma_load_2d(sb, &tmap_b, &full_bar[s], k0, n0);
          } else {
#pragma unroll
            for (int c = 0; c < BN / 64; ++c) tma_load_2d(sb + c * 8192, &tmap_b, &full_bar[s], n0 + 64 * c, k0);
          }
        }
      }
      if (!ok) {
        // give loads that are still in flight a bounded chance to land before the CTA exits
        for (int s = 0; s < NSTAGE; ++s) {
          for (int spin = 0; spin < 100000; ++spin)
            if (mbar_try_wait(&full_bar[s], 0) || mbar_try_wait(&full_bar[s], 1)) break;
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      const uint32_t idesc = make_idesc_bf16(BM, BN, g.a_mn_major, g.b_mn_major);
      const uint32_t desc_hi = smem_desc_hi(1024);
      const uint32_t a_lbo = g.a_mn_major ? 8192 : 16, b_lbo = g.b_mn_major ? 8192 : 16;
      const uint32_t a_step = g.a_mn_major ? (2048 >> 4) : (32 >> 4), b_step = g.b_mn_major ? (2048 >> 4) : (32 >> 4);
      uint32_t it = 0;
      uint32_t tcount = 0;
      bool ok = true;
      long long* tr = blockIdx.x == 0 ? g.trace : nullptr;
      int tslot = 0;
      for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++tcount) {
        const int ks = tile / (tiles_m * tiles_n);
        const int kb0 = ks * kb_per_split;
        const int kb1 = min(kb_total, kb0 + kb_per_split);
        const int ab = tcount & 1;
        const uint32_t aph = (tcount >> 1) & 1;
        if (!mbar_wait(&acc_empty[ab], aph ^ 1, abort_flag, g.status)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + ab * BN;
        uint32_t accumulate = 0;
        for (int kb = kb0; kb < kb1; ++kb, ++it) {
          const int s = it % NSTAGE;
          const uint32_t ph = (it / NSTAGE) & 1;
          GEMM_TRACE(tr, tslot);
          if (!mbar_wait(&full_bar[s], ph, abort_flag, g.status)) { ok = false; break; }
          GEMM_TRACE(tr, tslot);
          // no tcgen05 fence here: the operands were written by TMA (async proxy) and the mbarrier
          // wait orders them; a fence per k-block only delays the next MMAs behind the previous ones
          const uint32_t sa = smem_u32(smem + s * L::STAGE_BYTES);
          const uint32_t sb = sa + L::A_BYTES;
          // K-major: 16 elements = 32 bytes further along the swizzled row per MMA.
          // MN-major: 16 k-rows of 128 bytes further down.  Only the low descriptor word moves.
          uint32_t a_lo = smem_desc_lo(sa, a_lbo), b_lo = smem_desc_lo(sb, b_lbo);
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            umma_bf16_lohi(d_tmem, a_lo, b_lo, desc_hi, idesc, accumulate);
            a_lo += a_step; b_lo += b_step;
            accumulate = 1;
          }
          GEMM_TRACE(tr, tslot);
          umma_commit(&empty_bar[s]);      // frees the smem stage when these MMAs retire
          GEMM_TRACE(tr, tslot);
        }
        if (ok) umma_commit(&acc_full[ab]);  // accumulator complete
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue
    const int q = warp & 3;                 // TMEM lane quarter this warp may read
    const int half = (warp - 2) >> 2;       // which half of the tile's columns
    uint32_t tcount = 0;
    bool ok = true;
    for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++tcount) {
      const int ks = tile / (tiles_m * tiles_n);
      const int rem = tile - ks * tiles_m * tiles_n;
      const int m0 = (rem % tiles_m) * BM;
      const int n0 = (rem / tiles_m) * BN;
      const int ab = tcount & 1;
      const uint32_t aph = (tcount >> 1) & 1;
      const bool has_k = ks * kb_per_split < kb_total;
      if (!mbar_wait(&acc_full[ab], aph, abort_flag, g.status)) { ok = false; break; }
      tc_fence_after();
      const uint32_t t_addr = tmem_base + ab * BN + half * (BN / 2) + (uint32_t(q * 32) << 16);
      drain_tile<BN / 2>(g, t_addr, m0 + q * 32, lane, n0 + half * (BN / 2), has_k,
                                       smem + L::EPI_OFFSET + (warp - 2) * EPI_STAGE_BYTES, [&] {
        tmem_ld_wait();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(&acc_empty[ab]);
      });
    }
  }

  // ---------------------------------------------------------------- teardown
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 2 * BN);
  }
}

// ------------------------------------------------------------------ CTA-pair variant
// 256 x 256 output tile per cluster of two CTAs (tcgen05 cta_group::2).  Each CTA
// loads only its half of A (128 rows) and its half of B (128 columns) per k-block,
// 32 KB instead of the 48 KB a lone 128 x 256 CTA needs for the same FLOPs, which is
// what matters once the main loop is bound by L2-to-shared-memory traffic.  The
// leader CTA (cluster rank 0) issues the MMAs for both; each CTA drains its own
// 128 rows of the accumulator from its own TMEM.
//   full[s]      in the leader, 2 arrivals (one producer per CTA) + both CTAs' bytes
//   empty[s]     in each CTA, released by one multicast tcgen05.commit of the leader
//   acc_full[b]  in each CTA, same mechanism
//   acc_empty[b] in the leader, one arrival per epilogue warp of both CTAs
// KSUB k-blocks share one full/empty barrier pair (KSUB = 2: a stage is two 64-wide k-blocks, so the issuing
// thread pays one barrier wait and one commit per eight MMAs instead of per four).
constexpr int PAIR_BN = 256;
constexpr int PAIR_STAGES = 6;          // k-blocks resident in shared memory
struct PairSmem {
  static constexpr int A_BYTES = 128 * BK * 2;
  static constexpr int B_BYTES = 128 * BK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int EPI_OFFSET = PAIR_STAGES * STAGE_BYTES;
  static constexpr int BAR_OFFSET = EPI_OFFSET + EPI_WARPS * EPI_STAGE_BYTES;
  static constexpr int TOTAL = BAR_OFFSET + 256 + 1024;
};

template <int KSUB>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(GEMM_THREADS, 1)
gemm_pair_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b, GemmArgs g) {
  using L = PairSmem;
  constexpr int NSTAGE = PAIR_STAGES / KSUB;          // barrier pairs; each covers KSUB k-blocks
  static_assert(PAIR_STAGES % KSUB == 0, "stages must divide into groups");
  constexpr int BN = PAIR_BN;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + L::BAR_OFFSET);
  uint64_t* empty_bar = full_bar + NSTAGE;
  uint64_t* acc_full = empty_bar + NSTAGE;
  uint64_t* acc_empty = acc_full + 2;
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(acc_empty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_holder + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();          // 0 = leader
  const int pair = blockIdx.x >> 1;
  const int num_pairs = gridDim.x >> 1;

  const int tiles_m = (g.M + 255) / 256;
  const int tiles_n = (g.N + BN - 1) / BN;
  const int kb_total = (g.K + BK - 1) / BK;
  const int splits = g.split_k > 1 ? g.split_k : 1;
  const int kb_per_split = (kb_total + splits - 1) / splits;
  const int num_tiles = tiles_m * tiles_n * splits;

  if (threadIdx.x == 0) {
    for (int s = 0; s < NSTAGE; ++s) { mbar_init(&full_bar[s], 2); mbar_init(&empty_bar[s], 1); }
    for (int b = 0; b < 2; ++b) { mbar_init(&acc_full[b], 1); mbar_init(&acc_empty[b], 2 * EPI_WARPS); }
    *abort_flag = 0;
    mbar_fence_init();
    fence_proxy_async();
  }
  if (warp == 1) {
    tmem_alloc_pair(tmem_holder, 2 * BN);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();                 // both CTAs' barriers exist before anyone arrives remotely
  tc_fence_after();
  const uint32_t tmem_base = *tmem_holder;

  if (warp == 0) {
    // ------------------------------------------------------------ producer (one per CTA)
    if (lane == 0) {
      tma_prefetch_desc(&tmap_a);
      tma_prefetch_desc(&tmap_b);
      uint32_t it = 0;
      bool ok = true;
      for (int tile = pair; tile < num_tiles && ok; tile += num_pairs) {
        const int ks = tile / (tiles_m * tiles_n);
        const int rem = tile - ks * tiles_m * tiles_n;
        const int m0 = (rem % tiles_m) * 256 + int(rank) * 128;     // this CTA's rows of A
        const int n0 = (rem / tiles_m) * BN + int(rank) * 128;      // this CTA's columns of B
        const int kb0 = ks * kb_per_split;
        const int kb1 = min(kb_total, kb0 + kb_per_split);
        for (int kb = kb0; kb < kb1; kb += KSUB, ++it) {
          const int s = it % NSTAGE;
          const uint32_t ph = (it / NSTAGE) & 1;
          const int nsub = min(KSUB, kb1 - kb);
          if (!mbar_wait(&empty_bar[s], ph ^ 1, abort_flag, g.status)) { ok = false; break; }
          const uint32_t full_leader = map_to_cta(smem_u32(&full_bar[s]), 0);
          mbar_expect_tx_cluster(full_leader, nsub * L::STAGE_BYTES);
          for (int sub = 0; sub < nsub; ++sub) {
            uint8_t* sa = smem + (s * KSUB + sub) * L::STAGE_BYTES;
            uint8_t* sb = sa + L::A_BYTES;
            const int k0 = (kb + sub) * BK;
            if (!g.a_mn_major) {
              tma_load_2d_pair(sa, &tmap_a, full_leader, k0, m0);
            } else {
              tma_load_2d_pair(sa, &tmap_a, full_leader, m0, k0);
              tma_load_2d_pair(sa + 8192, &tmap_a, full_leader, m0 + 64, k0);
            }
            if (!g.b_mn_major) {
              tma_load_2d_pair(sb, &tmap_b, full_leader, k0, n0);
            } else {
              tma_load_2d_pair(sb, &tmap_b, full_leader, n0, k0);
              tma_load_2d_pair(sb + 8192, &tmap_b, full_leader, n0 + 64, k0);
            }
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer (leader CTA only)
    if (lane == 0 && rank == 0) {
      const uint32_t idesc = make_idesc_bf16(256, BN, g.a_mn_major, g.b_mn_major);
      const uint32_t desc_hi = smem_desc_hi(1024);
      const uint32_t a_lbo = g.a_mn_major ? 8192 : 16, b_lbo = g.b_mn_major ? 8192 : 16;
      const uint32_t a_step = g.a_mn_major ? (2048 >> 4) : (32 >> 4), b_step = g.b_mn_major ? (2048 >> 4) : (32 >> 4);
      uint32_t it = 0;
      uint32_t tcount = 0;
      bool ok = true;
      long long* tr = blockIdx.x == 0 ? g.trace : nullptr;
      int tslot = 0;
      for (int tile = pair; tile < num_tiles && ok; tile += num_pairs, ++tcount) {
        const int ks = tile / (tiles_m * tiles_n);
        const int kb0 = ks * kb_per_split;
        const int kb1 = min(kb_total, kb0 + kb_per_split);
        const int ab = tcount & 1;
        const uint32_t aph = (tcount >> 1) & 1;
        if (!mbar_wait(&acc_empty[ab], aph ^ 1, abort_flag, g.status)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + ab * BN;
        uint32_t accumulate = 0;
        for (int kb = kb0; kb < kb1; kb += KSUB, ++it) {
          const int s = it % NSTAGE;
          const uint32_t ph = (it / NSTAGE) & 1;
          const int nsub = min(KSUB, kb1 - kb);
          GEMM_TRACE(tr, tslot);
          if (!mbar_wait(&full_bar[s], ph, abort_flag, g.status)) { ok = false; break; }
          GEMM_TRACE(tr, tslot);
          // no tcgen05 fence here: the operands were written by TMA (async proxy) and the mbarrier
          // wait orders them; a fence per k-block only delays the next MMAs behind the previous ones
#pragma unroll
          for (int sub = 0; sub < KSUB; ++sub) {
            if (sub < nsub) {
              const uint32_t sa = smem_u32(smem + (s * KSUB + sub) * L::STAGE_BYTES);
              const uint32_t sb = sa + L::A_BYTES;
              uint32_t a_lo = smem_desc_lo(sa, a_lbo), b_lo = smem_desc_lo(sb, b_lbo);
#pragma unroll
              for (int k = 0; k < BK / UMMA_K; ++k) {
                umma_bf16_pair_lohi(d_tmem, a_lo, b_lo, desc_hi, idesc, accumulate);
                a_lo += a_step; b_lo += b_step;
                accumulate = 1;
              }
            }
          }
          GEMM_TRACE(tr, tslot);
          umma_commit_pair_all(smem_u32(&empty_bar[s]), 0x3);     // frees the stage in both CTAs
          GEMM_TRACE(tr, tslot);
        }
        if (ok) {
          umma_commit_pair_all(smem_u32(&acc_full[ab]), 0x3);
        }
      }
    }
  } else {
    // ------------------------------------------------------------ epilogue (both CTAs, own 128 rows)
    const int q = warp & 3;
    const int half = (warp - 2) >> 2;
    uint32_t tcount = 0;
    bool ok = true;
    for (int tile = pair; tile < num_tiles && ok; tile += num_pairs, ++tcount) {
      const int ks = tile / (tiles_m * tiles_n);
      const int rem = tile - ks * tiles_m * tiles_n;
      const int m0 = (rem % tiles_m) * 256 + int(rank) * 128;
      const int n0 = (rem / tiles_m) * BN;
      const int ab = tcount & 1;
      const uint32_t aph = (tcount >> 1) & 1;
      const bool has_k = ks * kb_per_split < kb_total;
      if (!mbar_wait(&acc_full[ab], aph, abort_flag, g.status)) { ok = false; break; }
      tc_fence_after();
      const uint32_t t_addr = tmem_base + ab * BN + half * (BN / 2) + (uint32_t(q * 32) << 16);
      drain_tile<BN / 2>(g, t_addr, m0 + q * 32, lane, n0 + half * (BN / 2), has_k,
                                       smem + L::EPI_OFFSET + (warp - 2) * EPI_STAGE_BYTES, [&] {
        tmem_ld_wait();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster(map_to_cta(smem_u32(&acc_empty[ab]), 0));
      });
    }
  }

  // ---------------------------------------------------------------- teardown
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();                 // the peer may still be arriving on this CTA's barriers until here
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, 2 * BN);
  }
}

// ------------------------------------------------------------------ host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  });
  return fn;
}

// 2-D bf16 tensor map: `inner` contiguous elements, `outer` rows of `ld` elements.
int make_tmap_bf16_2d(CUtensorMap* tm, const void* ptr, long long inner, long long outer, long long ld,
                      int box_inner, int box_outer) {
  EncodeTiledFn enc = get_encode();
  if (!enc) return -1;
  cuuint64_t dims[2] = {(cuuint64_t)inner, (cuuint64_t)outer};
  cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
  cuuint32_t box[2] = {(cuuint32_t)box_inner, (cuuint32_t)box_outer};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(tm, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : -(int)r - 100;
}

// 2-D fp32 tensor map, 128-byte swizzle (box_inner * 4 bytes must be 128).
int make_tmap_f32_2d(CUtensorMap* tm, const void* ptr, long long inner, long long outer, long long ld, int box_inner,
                     int box_outer) {
  EncodeTiledFn enc = get_encode();
  if (!enc) return -1;
  cuuint64_t dims[2] = {(cuuint64_t)inner, (cuuint64_t)outer};
  cuuint64_t strides[1] = {(cuuint64_t)ld * 4};
  cuuint32_t box[2] = {(cuuint32_t)box_inner, (cuuint32_t)box_outer};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(tm, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : -(int)r - 100;
}

// 3-D map over a [rows, ncol * inner] matrix seen as (inner, ncol, rows), 128-byte swizzle.  The box may be wider
// than `inner`: the columns past it are out of bounds, so loads fill them with zeros and stores skip them.
int make_tmap_3d(CUtensorMap* tm, int is_f32, const void* ptr, long long inner, long long ncol, long long rows,
                 long long ld, int box_inner, int box_rows) {
  EncodeTiledFn enc = get_encode();
  if (!enc) return -1;
  const cuuint64_t es = is_f32 ? 4 : 2;
  cuuint64_t dims[3] = {(cuuint64_t)inner, (cuuint64_t)ncol, (cuuint64_t)rows};
  cuuint64_t strides[2] = {(cuuint64_t)inner * es, (cuuint64_t)ld * es};
  cuuint32_t box[3] = {(cuuint32_t)box_inner, 1, (cuuint32_t)box_rows};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = enc(tm, is_f32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3,
                   const_cast<void*>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : -(int)r - 100;
}

static int g_num_sms = 0;

template <int BN, int NSTAGE>
static int launch(const CUtensorMap& ta, const CUtensorMap& tb, const GemmArgs& g, int max_ctas, cudaStream_t st) {
  using L = SmemLayout<BN, NSTAGE>;
  static bool attr_set = false;
  if (!attr_set) {
    if (cudaFuncSetAttribute(gemm_kernel<BN, NSTAGE>, cudaFuncAttributeMaxDynamicSharedMemorySize, L::TOTAL) !=
        cudaSuccess)
      return -2;
    attr_set = true;
  }
  const int tiles = ((g.M + BM - 1) / BM) * ((g.N + BN - 1) / BN) * (g.split_k > 1 ? g.split_k : 1);
  int grid = tiles < g_num_sms ? tiles : g_num_sms;
  if (max_ctas > 0 && grid > max_ctas) grid = max_ctas;
  gemm_kernel<BN, NSTAGE><<<grid, GEMM_THREADS, L::TOTAL, st>>>(ta, tb, g);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}


static int g_pair_ksub = 2;

static int launch_pair(const CUtensorMap& ta, const CUtensorMap& tb, const GemmArgs& g, int max_ctas, cudaStream_t st) {
  static bool attr_set = false;
  if (!attr_set) {
    if (cudaFuncSetAttribute(gemm_pair_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, PairSmem::TOTAL) !=
            cudaSuccess ||
        cudaFuncSetAttribute(gemm_pair_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, PairSmem::TOTAL) !=
            cudaSuccess)
      return -2;
    attr_set = true;
  }
  const int tiles = ((g.M + 255) / 256) * ((g.N + PAIR_BN - 1) / PAIR_BN) * (g.split_k > 1 ? g.split_k : 1);
  int pairs = g_num_sms / 2;
  if (max_ctas > 0 && pairs > max_ctas / 2) pairs = max_ctas / 2 > 0 ? max_ctas / 2 : 1;
  if (pairs > tiles) pairs = tiles;
  if (g_pair_ksub == 2) gemm_pair_kernel<2><<<2 * pairs, GEMM_THREADS, PairSmem::TOTAL, st>>>(ta, tb, g);
  else                  gemm_pair_kernel<1><<<2 * pairs, GEMM_THREADS, PairSmem::TOTAL, st>>>(ta, tb, g);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

}  // namespace dsw

using namespace dsw;

// Tuning knob of the CTA-pair kernel: k-blocks per barrier pair (1 or 2).
extern "C" int dsw_gemm_set_pair_ksub(int ksub) {
  if (ksub != 1 && ksub != 2) return -10;
  dsw::g_pair_ksub = ksub;
  return 0;
}

static long long* g_gemm_trace = nullptr;
// Register (or clear) a device buffer of 512 int64 for the one-CTA kernel's MMA-thread timeline.
extern "C" int dsw_gemm_set_trace(long long* buf) { g_gemm_trace = buf; return 0; }

// A: [M,K] row-major (a_mn_major = 0) or [K,M] row-major (1); lda = row pitch in
// elements.  B: [N,K] (b_mn_major = 0) or [K,N] (1).  All pitches and the
// contiguous extents must be multiples of 8 elements; pointers 16-byte aligned.
// bn = 128 or 256 selects the tile width; max_ctas > 0 caps the grid (to leave
// SMs to a concurrent kernel).  Returns 0 or a negative error code.
extern "C" int dsw_gemm_bf16(const void* A, long long lda, int a_mn_major, const void* B, long long ldb,
                             int b_mn_major, int M, int N, int K, int mode, int split_k, void* out, long long ldo,
                             const float* bias, const void* resid, long long ldr, void* aux_out, const void* aux_in,
                             long long ldaux, int bn, int max_ctas, int* status, cudaStream_t stream) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  if ((lda | ldb | ldo) % 8 || N % 8 || (a_mn_major ? M % 8 : K % 8) || (b_mn_major ? N % 8 : K % 8)) return -10;
  if ((reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(B) | reinterpret_cast<uintptr_t>(out)) & 15)
    return -11;
  if (bn != 128 && bn != 256 && bn != 512) return -12;   // 512 = CTA-pair kernel (256 x 256 per cluster)
  if (g_num_sms == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&g_num_sms, cudaDevAttrMultiProcessorCount, dev);
  }
  CUtensorMap ta, tb;
  int rc;
  if (!a_mn_major) rc = make_tmap_bf16_2d(&ta, A, K, M, lda, BK, BM);
  else             rc = make_tmap_bf16_2d(&ta, A, M, K, lda, 64, BK);
  if (rc) return rc;
  if (!b_mn_major) rc = make_tmap_bf16_2d(&tb, B, K, N, ldb, BK, bn == 512 ? 128 : bn);
  else             rc = make_tmap_bf16_2d(&tb, B, N, K, ldb, 64, BK);
  if (rc) return rc;
  GemmArgs g;
  g.M = M; g.N = N; g.K = K;
  g.a_mn_major = a_mn_major; g.b_mn_major = b_mn_major;
  g.mode = mode; g.split_k = split_k;
  g.out = out; g.ldo = ldo; g.bias = bias;
  g.resid = reinterpret_cast<const __nv_bfloat16*>(resid); g.ldr = ldr;
  g.aux_out = reinterpret_cast<__nv_bfloat16*>(aux_out);
  g.aux_in = reinterpret_cast<const __nv_bfloat16*>(aux_in); g.ldaux = ldaux;
  g.status = status;
  g.trace = g_gemm_trace;
  if (bn == 512) return launch_pair(ta, tb, g, max_ctas, stream);
  if (bn == 256) return launch<256, 4>(ta, tb, g, max_ctas, stream);
  return launch<128, 6>(ta, tb, g, max_ctas, stream);
}

// Force the module that holds these kernels to load now (see dsw_load_all).
extern "C" int dsw_load_gemm() {
  cudaFuncAttributes a;
  if (cudaFuncGetAttributes(&a, gemm_kernel<256, 4>) != cudaSuccess) return -1;
  if (cudaFuncGetAttributes(&a, gemm_kernel<128, 6>) != cudaSuccess) return -1;
  if (cudaFuncGetAttributes(&a, gemm_pair_kernel<1>) != cudaSuccess) return -1;
  if (cudaFuncGetAttributes(&a, gemm_pair_kernel<2>) != cudaSuccess) return -1;
  return 0;
}
