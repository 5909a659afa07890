// Device side of the tcgen05 GEMMs: epilogue, the one-CTA kernel and the CTA-pair kernel, as templates.
// Each kernel is a template on its epilogue class; gemm_one_cta.cu and gemm_pair.cu instantiate them
// (two translation units, so the fifteen kernels compile side by side) and gemm_tcgen05.cu holds the
// host entry point.
#pragma once
#include <cuda.h>
#include "ptx.cuh"

namespace dsw {

__device__ __forceinline__ long long gemm_gtimer() {
  long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
// In-kernel timeline stamps exist only in the tracing build of the library (-DDSWARM_TRACE, used by
// benchmarks/timelines.py); the shipped kernels carry none of it.
#ifdef DSWARM_TRACE
#define GEMM_TRACE(buf, slot) do { if ((buf) != nullptr && (slot) < 256) (buf)[(slot)++] = gemm_gtimer(); } while (0)
#define GEMM_TRACE2(buf, slot) do { if ((buf) != nullptr && (slot) < 255) (buf)[(slot)++] = gemm_gtimer(); } while (0)
#else
#define GEMM_TRACE(buf, slot) do { } while (0)
#define GEMM_TRACE2(buf, slot) do { } while (0)
#endif

constexpr int BM = 128;
constexpr int BK = 64;          // one 128-byte swizzle row of bf16
constexpr int UMMA_K = 16;
constexpr int EPI_WARPS = 16;         // four per TMEM lane quarter, each takes a quarter of the tile's columns
constexpr int EPI_WARP0 = 4;          // warps 2 and 3 only keep the epilogue warps aligned with the TMEM lane quarters
constexpr int GEMM_THREADS = 32 * (EPI_WARP0 + EPI_WARPS);

enum EpiMode : int {
  EPI_STORE = 0,        // out = acc (+ bias)
  EPI_GELU = 1,         // out = gelu(acc + bias) ; aux_out (optional) = gelu'(acc + bias), what the backward multiplies by
  EPI_RESID = 2,        // out = acc + bias + resid
  EPI_MUL = 3,          // out = acc * aux_in  (aux_in = the gelu' saved by EPI_GELU: the GELU backward)
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
// Sixteen warps drain a finished accumulator: four per TMEM lane quarter (a warp may only read the
// 32 lanes of its quarter), each taking a quarter of the tile's columns.  With four epilogue warps
// per scheduler the latencies of one warp's TMEM load, shared-memory round trip and global loads
// are covered by the others; with two they were not, and the epilogue of a K = 768 tile took longer
// than the tile's main loop.
//
// A thread owns one accumulator row (that is how tcgen05.ld hands the data out), but a store in
// which every lane writes 16 bytes of a different row touches 32 cache lines per instruction.  So
// each warp passes its rows through a private 2 KB tile of shared memory, 32 rows x 64 bytes with
// the 16-byte chunks rotated by (row / 2) so that writes by row and reads by row group are both
// conflict-free, and writes it out with lane = (row within a group of 8, 16-byte chunk): every
// store, residual / aux load or fp32 reduction instruction then covers 8 rows x 64 contiguous bytes.
//
// The accumulator is drained in chunks of 32 columns (16 for fp32 outputs: 64 bytes per row either
// way).  Everything a chunk needs from global memory besides the accumulator (residual, saved GELU
// derivative) is requested before the wait for the accumulator, in one batch; the TMEM load of the
// next chunk is issued as soon as this chunk's registers have been converted, so it runs under the
// staging and the stores.
constexpr int EPI_STAGE_BYTES = 32 * 64;

// This thread's row: NW 32-bit words = NW / 4 consecutive 16-byte chunks starting at chunk 0.
__device__ __forceinline__ void stage_row64(uint8_t* stage, int lane, const uint32_t (&w)[16]) {
#pragma unroll
  for (int c = 0; c < 4; ++c)
    *reinterpret_cast<uint4*>(stage + lane * 64 + (((c + (lane >> 1)) & 3) << 4)) =
        make_uint4(w[4 * c], w[4 * c + 1], w[4 * c + 2], w[4 * c + 3]);
}
// Write-out order: iteration i, this lane handles row i*8 + (lane >> 2), 16-byte chunk lane & 3.
template <class F>
__device__ __forceinline__ void unstage_rows64(const uint8_t* stage, int lane, F&& emit) {
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int rl = i * 8 + (lane >> 2), ch = lane & 3;
    const uint4 d = *reinterpret_cast<const uint4*>(stage + rl * 64 + (((ch + (rl >> 1)) & 3) << 4));
    emit(i, rl, ch, d);
  }
}

// NCOLS accumulator columns (a multiple of 32) starting at TMEM address t_addr, rows row_base..+31
// (one per lane), output columns col_base..+NCOLS-1.  `release` is called once, right after the last
// TMEM load has landed, so the MMA thread can refill the accumulator while the last chunk is written.
template <int MODE, int NCOLS, class Release>
__device__ __forceinline__ void epilogue_warp(const GemmArgs& g, uint32_t t_addr, int row_base, int lane, int col_base,
                                              uint8_t* stage, Release&& release) {
  if constexpr (MODE == EPI_ATOMIC_F32) {     // both fp32 outputs: accumulate (split-K safe) or plain store
    constexpr int NCH = NCOLS / 16;
    uint32_t r[16];
    tmem_ld_32x16(t_addr, r);
#pragma unroll
    for (int c = 0; c < NCH; ++c) {
      const int cb = col_base + c * 16;
      tmem_ld_wait();
      uint32_t w[16];
#pragma unroll
      for (int i = 0; i < 16; ++i) w[i] = r[i];
      if (c + 1 < NCH) tmem_ld_32x16(t_addr + (c + 1) * 16, r);
      else release();
      if (cb >= g.N) continue;
      __syncwarp();                                   // the previous chunk has been read out
      stage_row64(stage, lane, w);
      __syncwarp();
      unstage_rows64(stage, lane, [&](int, int rl, int ch, const uint4& d) {
        const int row = row_base + rl, col = cb + ch * 4;
        if (row < g.M && col < g.N) {
          float* o = reinterpret_cast<float*>(g.out) + (long long)row * g.ldo + col;
          if (g.mode == EPI_ATOMIC_F32)
            asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(o), "f"(__uint_as_float(d.x)),
                         "f"(__uint_as_float(d.y)), "f"(__uint_as_float(d.z)), "f"(__uint_as_float(d.w))
                         : "memory");
          else
            *reinterpret_cast<uint4*>(o) = d;
        }
      });
    }
  } else {
    constexpr int NCH = NCOLS / 32;
    constexpr bool EXTRA = MODE == EPI_RESID || MODE == EPI_MUL;
    const int my_ch = lane & 3, my_r = lane >> 2;
    uint32_t r[32];
    tmem_ld_32x32(t_addr, r);
#pragma unroll
    for (int c = 0; c < NCH; ++c) {
      const int cb = col_base + c * 32;
      const bool chunk_ok = cb < g.N;
      // ---- requests to global memory for this chunk, all at once, ahead of the accumulator
      uint4 x[EXTRA ? 4 : 1];
      if constexpr (EXTRA) {
        const __nv_bfloat16* src = MODE == EPI_RESID ? g.resid : g.aux_in;
        const long long ld = MODE == EPI_RESID ? g.ldr : g.ldaux;
        const int col = cb + my_ch * 8;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int row = row_base + i * 8 + my_r;
          x[i] = (row < g.M && col < g.N) ? __ldg(reinterpret_cast<const uint4*>(src + (long long)row * ld + col))
                                          : make_uint4(0, 0, 0, 0);
        }
      }
      tmem_ld_wait();
      // bias (an L1 hit after the first tile row), add, round.  GELU: activation and derivative come out of
      // one evaluation of the fp32 sum; the derivative waits in registers until the activation chunk is out
      uint32_t w[16];
      uint32_t post[MODE == EPI_GELU ? 16 : 1];
      if (chunk_ok) {
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const float4 bb = (g.bias != nullptr && cb + 4 * i < g.N) ? __ldg(reinterpret_cast<const float4*>(g.bias + cb) + i)
                                                                   : make_float4(0.f, 0.f, 0.f, 0.f);
          const float v0 = __uint_as_float(r[4 * i]) + bb.x, v1 = __uint_as_float(r[4 * i + 1]) + bb.y;
          const float v2 = __uint_as_float(r[4 * i + 2]) + bb.z, v3 = __uint_as_float(r[4 * i + 3]) + bb.w;
          if constexpr (MODE == EPI_GELU) {
            f2 ga, da, gb, db;
            gelu_pair(v0, v1, ga, da);
            gelu_pair(v2, v3, gb, db);
            w[2 * i] = pack_bf16_f2(ga);
            w[2 * i + 1] = pack_bf16_f2(gb);
            post[2 * i] = pack_bf16_f2(da);
            post[2 * i + 1] = pack_bf16_f2(db);
          } else {
            w[2 * i] = pack_bf16(v0, v1);
            w[2 * i + 1] = pack_bf16(v2, v3);
          }
        }
      }
      if (c + 1 < NCH) tmem_ld_32x32(t_addr + (c + 1) * 32, r);
      else release();
      if (!chunk_ok) continue;
      __syncwarp();                                   // the previous chunk has been read out
      stage_row64(stage, lane, w);
      __syncwarp();
      unstage_rows64(stage, lane, [&](int i, int rl, int ch, uint4 d) {
        const int row = row_base + rl, col = cb + ch * 8;
        if (row >= g.M || col >= g.N) return;
        if (!DSW_OK(col + 8 <= g.N && col + 8 <= g.ldo && rl >= 0 && rl < 32)) return;
        if constexpr (EXTRA) {
          uint32_t du[4] = {d.x, d.y, d.z, d.w};
          const uint32_t xu[4] = {x[i].x, x[i].y, x[i].z, x[i].w};
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            const float2 a = unpack_bf16(du[q]), e = unpack_bf16(xu[q]);
            du[q] = MODE == EPI_RESID ? pack_bf16(a.x + e.x, a.y + e.y) : pack_bf16(a.x * e.x, a.y * e.y);
          }
          d = make_uint4(du[0], du[1], du[2], du[3]);
        }
        *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(g.out) + (long long)row * g.ldo + col) = d;
      });
      if constexpr (MODE == EPI_GELU) {
        if (g.aux_out != nullptr) {
          __syncwarp();
          stage_row64(stage, lane, post);
          __syncwarp();
          unstage_rows64(stage, lane, [&](int, int rl, int ch, const uint4& d) {
            const int row = row_base + rl, col = cb + ch * 8;
            if (row < g.M && col < g.N) *reinterpret_cast<uint4*>(g.aux_out + (long long)row * g.ldaux + col) = d;
          });
        }
      }
    }
  }
}

// The residual / saved-derivative operand of a tile, asked into L2 one tile ahead: the epilogue's loads of it
// then cost an L2 round trip instead of a DRAM one, which otherwise sits exposed once per chunk.
// Same lane-to-address map as the loads in epilogue_warp; one request per 32-byte sector.
template <int MODE, int NCOLS>
__device__ __forceinline__ void prefetch_extra(const GemmArgs& g, int row_base, int lane, int col_base) {
  if constexpr (MODE == EPI_RESID || MODE == EPI_MUL) {
    const __nv_bfloat16* src = MODE == EPI_RESID ? g.resid : g.aux_in;
    const long long ld = MODE == EPI_RESID ? g.ldr : g.ldaux;
    if (lane & 1) return;
#pragma unroll
    for (int c = 0; c < NCOLS / 32; ++c) {
      const int col = col_base + c * 32 + (lane & 3) * 8;
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int row = row_base + i * 8 + (lane >> 2);
        if (row < g.M && col < g.N)
          asm volatile("prefetch.global.L2 [%0];" ::"l"(src + (long long)row * ld + col));
      }
    }
  }
}

// One tile's worth of epilogue for this warp.  MODE is the kernel's compile-time epilogue class: a kernel
// that switched on the mode at run time carried the registers of every epilogue at once and spilled.
template <int MODE, int NCOLS, class Release>
__device__ __forceinline__ void drain_tile(const GemmArgs& g, uint32_t t_addr, int row_base, int lane, int col_base,
                                           bool has_k, uint8_t* stage, Release&& release) {
  if (!has_k) { release(); return; }
  epilogue_warp<MODE, NCOLS>(g, t_addr, row_base, lane, col_base, stage, release);
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

template <int BN, int NSTAGE, int MODE>
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
  } else if (warp >= EPI_WARP0) {
    // ------------------------------------------------------------ epilogue
    const int q = warp & 3;                 // TMEM lane quarter this warp may read
    const int part = (warp - EPI_WARP0) >> 2;   // which quarter of the tile's columns
    uint32_t tcount = 0;
    bool ok = true;
    auto prefetch_tile = [&](int tile) {
      if (tile >= num_tiles) return;
      const int rem = tile % (tiles_m * tiles_n);
      prefetch_extra<MODE, BN / 4>(g, (rem % tiles_m) * BM + q * 32, lane, (rem / tiles_m) * BN + part * (BN / 4));
    };
    prefetch_tile(blockIdx.x);
    for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++tcount) {
      const int ks = tile / (tiles_m * tiles_n);
      const int rem = tile - ks * tiles_m * tiles_n;
      const int m0 = (rem % tiles_m) * BM;
      const int n0 = (rem / tiles_m) * BN;
      const int ab = tcount & 1;
      const uint32_t aph = (tcount >> 1) & 1;
      const bool has_k = ks * kb_per_split < kb_total;
      prefetch_tile(tile + gridDim.x);
      if (!mbar_wait(&acc_full[ab], aph, abort_flag, g.status)) { ok = false; break; }
      tc_fence_after();
      const uint32_t t_addr = tmem_base + ab * BN + part * (BN / 4) + (uint32_t(q * 32) << 16);
      drain_tile<MODE, BN / 4>(g, t_addr, m0 + q * 32, lane, n0 + part * (BN / 4), has_k,
                         smem + L::EPI_OFFSET + (warp - EPI_WARP0) * EPI_STAGE_BYTES, [&] {
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

constexpr int PAIR_KSUB = 2;           // k-blocks per barrier pair

template <int MODE>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(GEMM_THREADS, 1)
gemm_pair_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b, GemmArgs g) {
  using L = PairSmem;
  constexpr int KSUB = PAIR_KSUB;
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
  } else if (warp >= EPI_WARP0) {
    // ------------------------------------------------------------ epilogue (both CTAs, own 128 rows)
    const int q = warp & 3;
    const int part = (warp - EPI_WARP0) >> 2;
    uint32_t tcount = 0;
    bool ok = true;
    // tracing build: the first epilogue warp of CTA 0 stamps (waiting for the accumulator, got it, tile
    // written out) into the second half of the buffer
    long long* etr = (blockIdx.x == 0 && warp == EPI_WARP0 && lane == 0 && g.trace != nullptr) ? g.trace + 256 : nullptr;
    int eslot = 0;
    (void)etr; (void)eslot;
    auto prefetch_tile = [&](int tile) {
      if (tile >= num_tiles) return;
      const int rem = tile % (tiles_m * tiles_n);
      prefetch_extra<MODE, BN / 4>(g, (rem % tiles_m) * 256 + int(rank) * 128 + q * 32, lane,
                                   (rem / tiles_m) * BN + part * (BN / 4));
    };
    prefetch_tile(pair);
    for (int tile = pair; tile < num_tiles && ok; tile += num_pairs, ++tcount) {
      const int ks = tile / (tiles_m * tiles_n);
      const int rem = tile - ks * tiles_m * tiles_n;
      const int m0 = (rem % tiles_m) * 256 + int(rank) * 128;
      const int n0 = (rem / tiles_m) * BN;
      const int ab = tcount & 1;
      const uint32_t aph = (tcount >> 1) & 1;
      const bool has_k = ks * kb_per_split < kb_total;
      prefetch_tile(tile + num_pairs);
      GEMM_TRACE2(etr, eslot);
      if (!mbar_wait(&acc_full[ab], aph, abort_flag, g.status)) { ok = false; break; }
      GEMM_TRACE2(etr, eslot);
      tc_fence_after();
      const uint32_t t_addr = tmem_base + ab * BN + part * (BN / 4) + (uint32_t(q * 32) << 16);
      drain_tile<MODE, BN / 4>(g, t_addr, m0 + q * 32, lane, n0 + part * (BN / 4), has_k,
                         smem + L::EPI_OFFSET + (warp - EPI_WARP0) * EPI_STAGE_BYTES, [&] {
        tmem_ld_wait();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive_cluster(map_to_cta(smem_u32(&acc_empty[ab]), 0));
      });
      GEMM_TRACE2(etr, eslot);
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


// Epilogue classes the kernels are instantiated for; both fp32 outputs share one.
__host__ __device__ constexpr int epi_class(int mode) { return mode == EPI_STORE_F32 ? EPI_ATOMIC_F32 : mode; }

// Defined in gemm_one_cta.cu / gemm_pair.cu.  bn = 128 or 256 for the one-CTA kernel.
int launch_one_cta(int bn, const CUtensorMap& ta, const CUtensorMap& tb, const GemmArgs& g, int num_sms, int max_ctas,
                   cudaStream_t st);
int launch_pair(const CUtensorMap& ta, const CUtensorMap& tb, const GemmArgs& g, int num_sms, int max_ctas,
                cudaStream_t st);
int load_one_cta_kernels();
int load_pair_kernels();

}  // namespace dsw
