// Causal flash attention forward on tcgen05 tensor cores, head size 64 or 32.
//
// Replaces the reference's F.scaled_dot_product_attention(q, k, v, is_causal=True)
// (src/model.py:66-67).  Input is the packed [B*T, 3*d] output of the QKV
// projection (Q | K | V, head h at columns h*hs of each part); output is the
// [B*T, d] tensor that feeds the output projection, plus the per-row log-sum-exp
// that the backward pass needs.
//
// A work item is (128 query rows, batch, head); persistent CTAs walk the items.
// Warps 0-3 own one query row per thread: they read the score row from tensor
// memory once, do the online softmax on it in registers and write P to shared
// memory.  The output row stays in tensor memory: every P V product accumulates
// onto it, and the row threads rescale it in place only when the running maximum
// has grown by more than 2^8 since the last rescale (until then P is computed
// against the older maximum, which is exact algebra and safe in bf16/fp32 range).
// Warp 4 issues the MMAs, warp 5 the TMA loads.
//   S = Q K_j^T          A = Q  [128 x 64]  K-major,  B = K_j [128 x 64] K-major   -> TMEM, 128 columns
//   O_j = P V_j          A = P  [128 x 128] K-major (written by the softmax warps
//                        in the 128-byte-swizzled layout),  B = V_j [128 x 64] N-major -> TMEM, 64 columns
// K/V tiles are double buffered; two CTAs fit on an SM (112 KB shared memory,
// 256 TMEM columns each), so one CTA's MMAs run under the other's softmax.
// Only kv tiles up to the diagonal are visited; the diagonal tile is masked.
//
// Head size 32 (the 4-head, 128-wide test model) runs the same tiles: its tensor maps describe the matrix as
// (32 columns, head, row) and the 64-column box reaches past the head, so TMA fills the right half of each
// operand tile with zeros.  Q K^T and dO V^T are unchanged by the zero columns, the output tiles get zero
// right halves, and the epilogues write the first 32 columns only.
#include <cuda.h>
#include "ptx.cuh"
#include "dswarm.h"

namespace dsw {

int make_tmap_bf16_2d(CUtensorMap* tm, const void* ptr, long long inner, long long outer, long long ld,
                      int box_inner, int box_outer);
int make_tmap_f32_2d(CUtensorMap* tm, const void* ptr, long long inner, long long outer, long long ld, int box_inner,
                     int box_outer);
int make_tmap_3d(CUtensorMap* tm, int is_f32, const void* ptr, long long inner, long long ncol, long long rows,
                 long long ld, int box_inner, int box_rows);

// [128 x 64] operand tile of column block `cb` (= part * heads + head) at `row`.
__device__ __forceinline__ void att_load_tile(void* dst, const CUtensorMap* tm, uint64_t* bar, int hs, int cb, int row) {
  if (hs == 64) tma_load_2d(dst, tm, bar, cb * 64, row);
  else          tma_load_3d(dst, tm, bar, 0, cb, row);
}

// Optional in-kernel timeline for tuning: when a trace buffer is registered (dsw_attention_set_trace),
// CTA 0 stores %globaltimer values at its phase boundaries: [0,256) row-warp 0, [256,512) MMA thread.
__device__ __forceinline__ long long gtimer() {
  long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
// In-kernel timeline stamps exist only in the tracing build (-DDSWARM_TRACE, benchmarks/timelines.py).
#ifdef DSWARM_TRACE
#define ATT_TRACE(buf, base, slot) do { if ((buf) != nullptr && (slot) < 256) (buf)[(base) + (slot)++] = gtimer(); } while (0)
#else
#define ATT_TRACE(buf, base, slot) do { } while (0)
#endif

constexpr int ATT_BQ = 128;        // query rows per work item
constexpr int ATT_BK = 128;        // kv rows per step
constexpr int ATT_HS = 64;
constexpr int ATT_THREADS = 256;          // warps 0-3 softmax, 4 MMA, 5 TMA, 6-7 only lend their registers
constexpr int ATT_TILE_BYTES = 128 * 64 * 2;     // one [128 x 64] bf16 tile

struct AttSmem {
  static constexpr int Q_OFF = 0;
  static constexpr int K_OFF = Q_OFF + ATT_TILE_BYTES;            // 2 stages
  static constexpr int V_OFF = K_OFF + 2 * ATT_TILE_BYTES;        // 2 stages
  static constexpr int P_OFF = V_OFF + 2 * ATT_TILE_BYTES;        // [2 k-blocks][128 rows][64]
  static constexpr int BAR_OFF = P_OFF + 2 * ATT_TILE_BYTES;
  // Two CTAs share an SM only if each stays under (227 KB - 2 KB) / 2 = 115200 bytes, so
  // there is no room for alignment slack: the dynamic segment is declared 1024-aligned
  // and the kernel checks that it really is.
  static constexpr int TOTAL = BAR_OFF + 128;
};

// max(a, b, c) in one instruction (sm_100 has the three-input form)
__device__ __forceinline__ float fmax3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}

__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// byte offset of element (row, col) of a [128 x 128] bf16 operand stored as two
// 64-column k-blocks in the 128-byte-swizzled K-major layout
__device__ __forceinline__ uint32_t p_offset(int row, int col) {
  const int kb = col >> 6, c = col & 63;
  return kb * ATT_TILE_BYTES + row * 128 + ((((c >> 3) ^ (row & 7)) << 4) | ((c & 7) << 1));
}

// Work items of a persistent launch: item = (query or kv tile, batch*head), listed heaviest first; CTA c of G
// takes items c, 2G-1-c, 2G+c, ... (a snake over the rounds), which evens out the tile counts per CTA.
// Returns false when round r holds no item for this CTA.
__device__ __forceinline__ bool att_item(int r, int c, int G, int total, int& idx) {
  idx = r * G + ((r & 1) ? G - 1 - c : c);
  return idx < total;
}

__global__ void __launch_bounds__(ATT_THREADS, 2)
attention_fwd_kernel(const __grid_constant__ CUtensorMap tmap_qkv, __nv_bfloat16* __restrict__ out,
                     float* __restrict__ lse_out, int T, int nh, int n_bh, int hs, float scale_log2, int* status,
                     long long* trace) {
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* smem = smem_raw;
  if (smem_u32(smem) & 1023) {            // swizzled operand tiles need 1024-byte alignment
    if (threadIdx.x == 0 && status) atomicCAS(status, 0, ST_BAD_ARG);
    return;
  }
  // Every barrier below completes one phase per kv tile (q_full / q_empty: per work item), counted over the
  // whole life of the CTA: g is the number of tiles, w the number of items this CTA has finished.
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + AttSmem::BAR_OFF);
  uint64_t* q_full = bars;            // Q of the item loaded
  uint64_t* kv_full = bars + 1;       // 2 stages
  uint64_t* kv_empty = bars + 3;      // 2 stages
  uint64_t* s_full = bars + 5;        // S ready in TMEM
  uint64_t* p_full = bars + 6;        // P written to smem (4 warps arrive)
  uint64_t* o_full = bars + 7;        // P V accumulated in TMEM
  uint64_t* o_free = bars + 8;        // per item: the output rows have been read out of TMEM (4 warps arrive)
  uint64_t* s_free = bars + 9;        // S read out of TMEM (4 warps arrive)
  uint64_t* q_empty = bars + 10;      // all S products of the item done: Q may be overwritten
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(bars + 11);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_holder + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nq = T / ATT_BQ;
  const int total = nq * n_bh;
  const int G = gridDim.x, cta = blockIdx.x;
  const int rounds = (total + G - 1) / G;
  const int d = nh * hs;
  long long* tr = blockIdx.x == 0 ? trace : nullptr;
  int tslot = 0;

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1); mbar_init(q_empty, 1);
    for (int i = 0; i < 2; ++i) { mbar_init(&kv_full[i], 1); mbar_init(&kv_empty[i], 1); }
    mbar_init(s_full, 1); mbar_init(p_full, 4); mbar_init(o_full, 1); mbar_init(o_free, 4);
    mbar_init(s_free, 4);
    *abort_flag = 0;
    mbar_fence_init();
    fence_proxy_async();
  }
  if (warp == 4) {
    tmem_alloc(tmem_holder, 256);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  // Two CTAs share the SM's registers: 128 per thread at launch.  The softmax warps keep a whole score row
  // (128 values) in registers, so their warpgroup takes 216 and the other warpgroup (one MMA-issuing and one
  // TMA-issuing thread) drops to 40.
  // (each role changes its own allotment at the top of its branch)
  const uint32_t tmem_base = *tmem_holder;
  const uint32_t tmem_s = tmem_base;            // 128 columns
  const uint32_t tmem_o = tmem_base + 128;      // 64 columns

  if (warp >= 4) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 40;");          // the whole warpgroup, one instruction
  }
  if (warp >= 6) {
    // nothing to do: these warps exist so that the register hand-over works on whole warpgroups
  } else if (warp == 5) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      tma_prefetch_desc(&tmap_qkv);
      uint32_t g = 0, w = 0;
      bool ok = true;
      for (int r = 0; r < rounds && ok; ++r) {
        int idx;
        if (!att_item(r, cta, G, total, idx)) continue;
        const int qi = nq - 1 - idx / n_bh, bh = idx % n_bh;
        const int b = bh / nh, h = bh - b * nh;
        if (w > 0 && !mbar_wait(q_empty, (w - 1) & 1, abort_flag, status)) break;
        mbar_expect_tx(q_full, ATT_TILE_BYTES);
        att_load_tile(smem + AttSmem::Q_OFF, &tmap_qkv, q_full, hs, h, b * T + qi * ATT_BQ);
        for (int j = 0; j <= qi; ++j, ++g) {
          const int s = g & 1;
          if (!mbar_wait(&kv_empty[s], ((g >> 1) & 1) ^ 1, abort_flag, status)) { ok = false; break; }
          mbar_expect_tx(&kv_full[s], 2 * ATT_TILE_BYTES);
          const int kvrow = b * T + j * ATT_BK;
          att_load_tile(smem + AttSmem::K_OFF + s * ATT_TILE_BYTES, &tmap_qkv, &kv_full[s], hs, nh + h, kvrow);
          att_load_tile(smem + AttSmem::V_OFF + s * ATT_TILE_BYTES, &tmap_qkv, &kv_full[s], hs, 2 * nh + h, kvrow);
        }
        ++w;
      }
    }
  } else if (warp == 4) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      const uint32_t idesc_s = make_idesc_bf16(128, 128, 0, 0);
      const uint32_t idesc_o = make_idesc_bf16(128, 64, 0, 1);
      const uint32_t desc_hi = smem_desc_hi(1024);
      const uint32_t q_lo = smem_desc_lo(smem_u32(smem + AttSmem::Q_OFF), 16);
      const uint32_t p_lo = smem_desc_lo(smem_u32(smem + AttSmem::P_OFF), 16);
      // S of global tile gt = Q K^T into the (single) score buffer; `first` / `last`: position in its item wi
      auto issue_s = [&](uint32_t gt, uint32_t wi, bool first, bool last) -> bool {
        if (first && !mbar_wait(q_full, wi & 1, abort_flag, status)) return false;
        const int st = gt & 1;
        if (!mbar_wait(&kv_full[st], (gt >> 1) & 1, abort_flag, status)) return false;
        const uint32_t k_lo = smem_desc_lo(smem_u32(smem + AttSmem::K_OFF + st * ATT_TILE_BYTES), 16);
#pragma unroll
        for (int k = 0; k < ATT_HS / 16; ++k)
          umma_bf16_lohi(tmem_s, q_lo + k * 2, k_lo + k * 2, desc_hi, idesc_s, k > 0);
        umma_commit(s_full);
        if (last) umma_commit(q_empty);
        ATT_TRACE(tr, 256, tslot);          // S issued
        return true;
      };
      uint32_t g = 0, w = 0;
      bool ok = true;
      for (int r = 0; r < rounds && ok; ++r) {
        int idx;
        if (!att_item(r, cta, G, total, idx)) continue;
        const int n_kv = nq - idx / n_bh;
        // the item after this one (its first score tile is issued during this item's last tile)
        int next_n_kv = 0;
        for (int r2 = r + 1, idx2; r2 < rounds; ++r2)
          if (att_item(r2, cta, G, total, idx2)) { next_n_kv = nq - idx2 / n_bh; break; }
        if (g == 0) ok = issue_s(0, 0, true, n_kv == 1);
        for (int j = 0; j < n_kv && ok; ++j, ++g) {
          const int s = g & 1;
          const uint32_t v_lo = smem_desc_lo(smem_u32(smem + AttSmem::V_OFF + s * ATT_TILE_BYTES), ATT_TILE_BYTES);
          // The next score tile goes first, as soon as the softmax warps have read this one for the last
          // time (they are still turning its last columns into P): they need the next S next, while the
          // P V product is only folded in after their first pass over it.
          const bool more = j + 1 < n_kv;
          if (more || next_n_kv > 0) {
            if (!mbar_wait(s_free, g & 1, abort_flag, status)) { ok = false; break; }
            tc_fence_after();
            const bool okk = more ? issue_s(g + 1, w, false, j + 2 == n_kv) : issue_s(g + 1, w + 1, true, next_n_kv == 1);
            if (!okk) { ok = false; break; }
          }
          // P of this tile is in shared memory (and the output rows are rescaled if they had to be)
          if (!mbar_wait(p_full, g & 1, abort_flag, status)) { ok = false; break; }
          ATT_TRACE(tr, 256, tslot);          // P ready
          // a new item starts its output from zero: the previous item's must have been read out
          if (j == 0 && w > 0 && !mbar_wait(o_free, (w - 1) & 1, abort_flag, status)) { ok = false; break; }
          tc_fence_after();
#pragma unroll
          for (int k = 0; k < ATT_BK / 16; ++k)          // P: 32 bytes along the row per step, second k-block after 4
            umma_bf16_lohi(tmem_o, p_lo + (k >> 2) * (ATT_TILE_BYTES >> 4) + (k & 3) * 2, v_lo + k * (2048 >> 4), desc_hi,
                           idesc_o, (j > 0 || k > 0));
          umma_commit(o_full);
          umma_commit(&kv_empty[s]);
          ATT_TRACE(tr, 256, tslot);          // PV issued
        }
        ++w;
      }
    }
  } else {
    // ------------------------------------------------------------ softmax + output (thread = query row)
    asm volatile("setmaxnreg.inc.sync.aligned.u32 216;");
    const int r = warp * 32 + lane;                      // row within the tile = TMEM lane
    const uint32_t lane_addr = uint32_t(warp * 32) << 16;
    uint8_t* sp = smem + AttSmem::P_OFF;
    if (threadIdx.x != 0) tr = nullptr;
    uint32_t g = 0;
    bool ok = true;
    for (int rr = 0; rr < rounds && ok; ++rr) {
      int idx;
      if (!att_item(rr, cta, G, total, idx)) continue;
      const int qi = nq - 1 - idx / n_bh, bh = idx % n_bh;
      const int b = bh / nh, h = bh - b * nh;
      const int n_kv = qi + 1;
      float m = -INFINITY, l = 0.f;           // m: the maximum P is computed against (log2 units)
      for (int j = 0; j < n_kv && ok; ++j, ++g) {
        ATT_TRACE(tr, 0, tslot);              // waiting for S
        if (!mbar_wait(s_full, g & 1, abort_flag, status)) { ok = false; break; }
        tc_fence_after();
        ATT_TRACE(tr, 0, tslot);              // S arrived
        // the whole score row into registers; the score buffer is free for the next tile at once
        uint32_t v[4][32];
#pragma unroll
        for (int c = 0; c < 4; ++c) tmem_ld_32x32(tmem_s + lane_addr + c * 32, v[c]);
        tmem_ld_wait();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(s_free);
        const bool diag = j == qi;
        // row maximum (four independent chains); on the diagonal tile only columns <= r count
        float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
        if (!diag) {
#pragma unroll
          for (int c = 0; c < 4; ++c)
#pragma unroll
            for (int i = 0; i < 32; i += 8) {
              mx4[0] = fmax3(mx4[0], __uint_as_float(v[c][i]), __uint_as_float(v[c][i + 1]));
              mx4[1] = fmax3(mx4[1], __uint_as_float(v[c][i + 2]), __uint_as_float(v[c][i + 3]));
              mx4[2] = fmax3(mx4[2], __uint_as_float(v[c][i + 4]), __uint_as_float(v[c][i + 5]));
              mx4[3] = fmax3(mx4[3], __uint_as_float(v[c][i + 6]), __uint_as_float(v[c][i + 7]));
            }
        } else {
#pragma unroll
          for (int c = 0; c < 4; ++c)
#pragma unroll
            for (int i = 0; i < 32; ++i)
              if (c * 32 + i <= r) mx4[i & 3] = fmaxf(mx4[i & 3], __uint_as_float(v[c][i]));
        }
        const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3])) * scale_log2;
        ATT_TRACE(tr, 0, tslot);              // maximum done
        if (j == 0) {
          m = mx;
        } else {
          // the previous product must be done: it reads the P tile that is about to be overwritten, and it
          // accumulates onto the output rows that may be rescaled here
          if (!mbar_wait(o_full, (g - 1) & 1, abort_flag, status)) { ok = false; break; }
          const bool grow = mx > m + 8.f;
          if (__any_sync(0xffffffffu, grow)) {          // rare after the first tiles
            tc_fence_after();
            const float alpha = grow ? fast_exp2(m - mx) : 1.f;
            if (grow) { m = mx; l *= alpha; }
#pragma unroll
            for (int c0 = 0; c0 < ATT_HS; c0 += 32) {
              uint32_t ov[32];
              tmem_ld_32x32(tmem_o + lane_addr + c0, ov);
              tmem_ld_wait();
#pragma unroll
              for (int i = 0; i < 32; ++i) ov[i] = __float_as_uint(__uint_as_float(ov[i]) * alpha);
              tmem_st_32x32(tmem_o + lane_addr + c0, ov);
            }
            tmem_st_wait();
          }
        }
        ATT_TRACE(tr, 0, tslot);              // output rows ready for the next product
        // probabilities -> shared memory (bf16, swizzled K-major), row sum
        float sum4[4] = {0.f, 0.f, 0.f, 0.f};
        f2 sum2[2] = {f2_bcast(0.f), f2_bcast(0.f)};      // off the diagonal: packed pairs (two columns per instruction)
        const f2 sc2 = f2_bcast(scale_log2), nm2 = f2_bcast(-m);
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          uint32_t pk[16];
          if (!diag) {
#pragma unroll
            for (int i = 0; i < 32; i += 2) {
              float x0, x1;
              f2_split(f2_fma(f2_make(__uint_as_float(v[c][i]), __uint_as_float(v[c][i + 1])), sc2, nm2), x0, x1);
              const float p0 = fast_exp2(x0), p1 = fast_exp2(x1);
              sum2[(i >> 1) & 1] = f2_add(sum2[(i >> 1) & 1], f2_make(p0, p1));
              pk[i >> 1] = pack_bf16(p0, p1);
            }
          } else {
#pragma unroll
            for (int i = 0; i < 32; i += 2) {
              const float p0 = c * 32 + i <= r ? fast_exp2(__uint_as_float(v[c][i]) * scale_log2 - m) : 0.f;
              const float p1 = c * 32 + i + 1 <= r ? fast_exp2(__uint_as_float(v[c][i + 1]) * scale_log2 - m) : 0.f;
              sum4[i & 3] += p0; sum4[(i + 1) & 3] += p1;
              pk[i >> 1] = pack_bf16(p0, p1);
            }
          }
#pragma unroll
          for (int i = 0; i < 16; i += 4)
            *reinterpret_cast<uint4*>(sp + p_offset(r, c * 32 + 2 * i)) = make_uint4(pk[i], pk[i + 1], pk[i + 2], pk[i + 3]);
        }
        {
          float a0, a1;
          f2_split(f2_add(sum2[0], sum2[1]), a0, a1);
          l += (sum4[0] + sum4[1]) + (sum4[2] + sum4[3]) + (a0 + a1);
        }
        ATT_TRACE(tr, 0, tslot);              // P written
        fence_proxy_async();          // make the generic-proxy writes of P visible to the tensor core
        tc_fence_before();            // orders the rescaled output rows before the product that follows the arrive
        __syncwarp();
        if (lane == 0) mbar_arrive(p_full);
      }
      if (!ok || !mbar_wait(o_full, (g - 1) & 1, abort_flag, status)) { ok = false; break; }
      tc_fence_after();
      const float inv = 1.f / l;
      const int row0 = b * T + qi * ATT_BQ;                // first global row of this query tile
      __nv_bfloat16* dst = out + (long long)(row0 + r) * d + h * hs;
      uint32_t ov[2][32];
      tmem_ld_32x32(tmem_o + lane_addr, ov[0]);
      tmem_ld_32x32(tmem_o + lane_addr + 32, ov[1]);
      tmem_ld_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(o_free);          // the next item's first product may overwrite the rows
#pragma unroll
      for (int i = 0; i < ATT_HS; i += 8)
        if (i < hs) {
          const uint32_t* o = ov[i >> 5] + (i & 31);
          *reinterpret_cast<uint4*>(dst + i) =
              make_uint4(pack_bf16(__uint_as_float(o[0]) * inv, __uint_as_float(o[1]) * inv),
                         pack_bf16(__uint_as_float(o[2]) * inv, __uint_as_float(o[3]) * inv),
                         pack_bf16(__uint_as_float(o[4]) * inv, __uint_as_float(o[5]) * inv),
                         pack_bf16(__uint_as_float(o[6]) * inv, __uint_as_float(o[7]) * inv));
        }
      // natural-log LSE of the scaled scores
      lse_out[(long long)bh * T + qi * ATT_BQ + r] = (m + log2f(l)) * 0.6931471805599453f;
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 4) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 256);
  }
}


// ------------------------------------------------------------------ backward
// One CTA per (128 kv rows, batch, head); it walks the query tiles i >= j (causal).
// Per query tile, with thread = query row for the softmax algebra:
//   S  = Q_i K_j^T,  dP = dO_i V_j^T                         -> TMEM (2 x 128 columns)
//   P  = exp(S*scale - lse),  dS = P * (dP - D) * scale      -> shared memory, bf16, swizzled
//   dV += P^T dO_i,  dK += dS^T Q_i   (accumulate in TMEM over i),  dQ_i = dS K_j (fresh)
// The P / dS tiles are written once and read through two descriptors: K-major
// (rows = queries) for dQ, and M-major (rows of the transposed operand = kv) for dV / dK;
// the [128 x 64] Q_i, dO_i, K_j tiles likewise serve as K-major A and as N-major B.
// dQ is accumulated across kv tiles with fp32 bulk reductions into a scratch tensor
// and converted to bf16 afterwards; dK and dV leave as two bulk stores per item.
//
// Eleven warps.  Row warps 0-7 (thread = query row, two threads per row, 64 columns each):
// wait sdp_full, take S and dP out of TMEM in one load group, arrive sdp_read, compute P / dS
// in registers, wait dq_full of the step before (its products read P / dS), write P / dS,
// arrive pds_full, then stage the dQ of the step before for the reducer.  MMA warp (one
// thread): issues the S / dP pair of step i+1 as soon as sdp_read of step i is complete (also
// for the first step of the next work item: K and V are double-buffered by item parity),
// then, on pds_full, dV, dK (releasing the Q / dO stage), dQ.  TMA warp (one thread): K / V
// of the item into the buffer of its parity, Q / dO pairs into two stages.  Reducer warp (one
// thread): one bulk reduce-add per staged dQ tile, two bulk stores per item for dK / dV
// (staged by the row warps in the P buffer, head size 64; with 32 the row warps store them).
// Every wait is bounded; a wait that runs out sets the CTA's abort flag and the status word.
struct AttBwdSmem {
  static constexpr int KV_BYTES = 2 * ATT_TILE_BYTES;               // K_j then V_j
  static constexpr int K_OFF = 0;                                   // 2 buffers (item parity) of (K, V)
  static constexpr int V_OFF = K_OFF + ATT_TILE_BYTES;
  static constexpr int QSTAGES = 2;                                 // (Q_i, dO_i) pairs in flight
  static constexpr int Q_OFF = K_OFF + 2 * KV_BYTES;
  static constexpr int DO_OFF = Q_OFF + QSTAGES * ATT_TILE_BYTES;
  static constexpr int P_OFF = DO_OFF + QSTAGES * ATT_TILE_BYTES;   // 2 k-blocks
  static constexpr int DS_OFF = P_OFF + 2 * ATT_TILE_BYTES;         // 2 k-blocks
  static constexpr int DQ_OFF = DS_OFF + 2 * ATT_TILE_BYTES;        // fp32 [2 halves][128 rows][32], 128-byte swizzled
  static constexpr int BAR_OFF = DQ_OFF + 2 * ATT_TILE_BYTES;
  static constexpr int TOTAL = BAR_OFF + 256 + 1024;
};


// D[bh, t] = sum_c dO[t, h*hs + c] * O[t, h*hs + c], and dq_acc[t, :] = 0.  One warp per token row: 16-byte
// loads, one head's hs columns lie in hs/8 neighbouring lanes (hs = 64 or 32), which a few shuffles add up.
__global__ void __launch_bounds__(256)
attention_bwd_prep_kernel(const __nv_bfloat16* __restrict__ out, const __nv_bfloat16* __restrict__ dout,
                          float* __restrict__ D, float* __restrict__ dq_acc, int B, int T, int nh, int hs) {
  const int lane = threadIdx.x & 31;
  const int d = nh * hs, chunks = d >> 3, lanes_per_head = hs >> 3;
  const long long rows = (long long)B * T;
  const long long warps = ((long long)gridDim.x * blockDim.x) >> 5;
  for (long long row = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5; row < rows; row += warps) {
    const int b = int(row / T), t = int(row - (long long)b * T);
    const uint4* po = reinterpret_cast<const uint4*>(out + row * d);
    const uint4* pg = reinterpret_cast<const uint4*>(dout + row * d);
    float4* pz = reinterpret_cast<float4*>(dq_acc + row * d);
    for (int u0 = 0; u0 < chunks; u0 += 32) {
      const int u = u0 + lane;
      float v = 0.f;
      if (u < chunks) {
        const uint4 a = po[u], g = pg[u];
        const uint32_t aw[4] = {a.x, a.y, a.z, a.w}, gw[4] = {g.x, g.y, g.z, g.w};
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const float2 x = unpack_bf16(aw[k]), y = unpack_bf16(gw[k]);
          v += x.x * y.x + x.y * y.y;
        }
        pz[2 * u] = make_float4(0.f, 0.f, 0.f, 0.f);
        pz[2 * u + 1] = make_float4(0.f, 0.f, 0.f, 0.f);
      }
      for (int o = lanes_per_head >> 1; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
      if (u < chunks && (lane & (lanes_per_head - 1)) == 0) D[((long long)b * nh + u / lanes_per_head) * T + t] = v;
    }
  }
}

// dqkv[:, 0:d] = bf16(dq_acc)
__global__ void __launch_bounds__(256)
attention_dq_convert_kernel(const float* __restrict__ dq_acc, __nv_bfloat16* __restrict__ dqkv, long long rows, int d) {
  const int per_row = d / 8;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < rows * per_row;
       i += (long long)gridDim.x * blockDim.x) {
    const long long row = i / per_row;
    const int col = int(i - row * per_row) * 8;
    const float4 a = *reinterpret_cast<const float4*>(dq_acc + row * d + col);
    const float4 b = *reinterpret_cast<const float4*>(dq_acc + row * d + col + 4);
    *reinterpret_cast<uint4*>(dqkv + row * 3 * d + col) =
        make_uint4(pack_bf16(a.x, a.y), pack_bf16(a.z, a.w), pack_bf16(b.x, b.y), pack_bf16(b.z, b.w));
  }
}

// 32 columns of one query row: P = exp2(S * scale_log2 - lse2), dS = P * (dP - D) * scale, both packed to bf16
// pairs.  MASKED: columns past `r` (above the diagonal) give zero.
template <bool MASKED, int N>
__device__ __forceinline__ void bwd_row_chunk(const uint32_t (&sv)[N], const uint32_t (&dpv)[N], uint32_t* pk_p,
                                              uint32_t* pk_ds, int c0, int r, float scale_log2, float lse2,
                                              float Dr, float scale) {
  // packed fp32 pairs: one instruction per two columns for everything but the exponentials and the packing
  const f2 sc = f2_bcast(scale_log2), nl = f2_bcast(-lse2), s2 = f2_bcast(scale), nd = f2_bcast(-Dr * scale);
#pragma unroll
  for (int c = 0; c < N; c += 2) {
    const f2 x = f2_fma(f2_make(__uint_as_float(sv[c]), __uint_as_float(sv[c + 1])), sc, nl);
    float x0, x1;
    f2_split(x, x0, x1);
    float p0 = fast_exp2(x0), p1 = fast_exp2(x1);
    if (MASKED) {
      p0 = c0 + c <= r ? p0 : 0.f;
      p1 = c0 + c + 1 <= r ? p1 : 0.f;
    }
    const f2 u = f2_fma(f2_make(__uint_as_float(dpv[c]), __uint_as_float(dpv[c + 1])), s2, nd);    // (dP - D) * scale
    pk_p[c >> 1] = pack_bf16(p0, p1);
    pk_ds[c >> 1] = pack_bf16_f2(f2_mul(f2_make(p0, p1), u));
  }
}

constexpr int ATT_BWD_ROW_WARPS = 8;     // two per TMEM lane quarter: each thread takes half of its row's columns
constexpr int ATT_BWD_THREADS = 32 * (ATT_BWD_ROW_WARPS + 3);    // + MMA issuer, TMA producer, dQ reducer

__global__ void __launch_bounds__(ATT_BWD_THREADS, 1)
attention_bwd_kernel(const __grid_constant__ CUtensorMap tmap_qkv, const __grid_constant__ CUtensorMap tmap_do,
                     const __grid_constant__ CUtensorMap tmap_dq, const __grid_constant__ CUtensorMap tmap_dkv,
                     const float* __restrict__ lse, const float* __restrict__ Dvec, __nv_bfloat16* __restrict__ dqkv,
                     int T, int nh, int n_bh, int hs,
                     float scale, int* status, long long* trace) {
  using L = AttBwdSmem;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  // Persistent: one CTA per SM walks work items (kv tile, batch*head).  The per-step barriers complete one
  // phase per step, kv_full / kv_empty / dkv_free one per item, counted over the life of the CTA
  // (g = steps done, w = items done).
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::BAR_OFF);
  uint64_t* kv_full = bars;            // 2: K, V of the item loaded (buffer = item parity)
  uint64_t* kv_empty = bars + 2;       // 2: every MMA of the item done: its K, V may be overwritten
  uint64_t* q_full = bars + 4;         // QSTAGES stages of (Q_i, dO_i)
  uint64_t* q_empty = bars + 6;        // QSTAGES
  uint64_t* sdp_full = bars + 8;       // S and dP ready
  uint64_t* pds_full = bars + 9;       // P and dS in shared memory (8 warps arrive)
  uint64_t* dq_full = bars + 10;       // dV/dK/dQ MMAs of this step done
  uint64_t* dq_free = bars + 11;       // dQ read out of TMEM (8 warps arrive)
  uint64_t* dkv_free = bars + 12;      // dK, dV of the item read out of TMEM (8 warps arrive)
  uint64_t* sdp_read = bars + 13;      // S and dP of this step read out of TMEM (8 warps arrive)
  uint64_t* dq_staged = bars + 14;     // dQ of this step staged in shared memory (8 warps arrive)
  uint64_t* dq_stage_free = bars + 15; // the reduction of this step's dQ has read the staging tile
  uint64_t* dkv_staged = bars + 16;    // dK, dV of the item staged in the P buffer (8 warps arrive; hs = 64)
  uint64_t* dkv_stored = bars + 17;    // their bulk stores have read the P buffer
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(bars + 18);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_holder + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nq = T / ATT_BQ;
  const int total = nq * n_bh;                   // items, heaviest first: kv tile 0 meets every query tile
  const int G = gridDim.x, cta = blockIdx.x;
  const int rounds = (total + G - 1) / G;
  const int d = nh * hs;
  const float scale_log2 = scale * 1.4426950408889634f;
  long long* tr = blockIdx.x == 0 ? trace : nullptr;
  int tslot = 0;

  if (threadIdx.x == 0) {
    for (int i = 0; i < 2; ++i) { mbar_init(&kv_full[i], 1); mbar_init(&kv_empty[i], 1); }
    for (int i = 0; i < L::QSTAGES; ++i) { mbar_init(&q_full[i], 1); mbar_init(&q_empty[i], 1); }
    mbar_init(sdp_full, 1); mbar_init(pds_full, ATT_BWD_ROW_WARPS); mbar_init(dq_full, 1);
    mbar_init(dq_free, ATT_BWD_ROW_WARPS); mbar_init(dkv_free, ATT_BWD_ROW_WARPS);
    mbar_init(sdp_read, ATT_BWD_ROW_WARPS);
    mbar_init(dq_staged, ATT_BWD_ROW_WARPS); mbar_init(dq_stage_free, 1);
    mbar_init(dkv_staged, ATT_BWD_ROW_WARPS); mbar_init(dkv_stored, 1);
    *abort_flag = 0;
    mbar_fence_init();
    fence_proxy_async();
  }
  constexpr int MMA_WARP = ATT_BWD_ROW_WARPS, TMA_WARP = ATT_BWD_ROW_WARPS + 1, RED_WARP = ATT_BWD_ROW_WARPS + 2;
  if (warp == MMA_WARP) {
    tmem_alloc(tmem_holder, 512);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_holder;
  const uint32_t tm_s = tmem_base, tm_dp = tmem_base + 128, tm_dv = tmem_base + 256, tm_dk = tmem_base + 320,
                 tm_dq = tmem_base + 384;

  if (warp == TMA_WARP) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      tma_prefetch_desc(&tmap_qkv);
      tma_prefetch_desc(&tmap_do);
      uint32_t g = 0, w = 0;
      bool ok = true;
      for (int r = 0; r < rounds && ok; ++r) {
        int idx;
        if (!att_item(r, cta, G, total, idx)) continue;
        const int j = idx / n_bh, bh = idx % n_bh;
        const int b = bh / nh, h = bh - b * nh;
        const int steps = nq - j;
        // K and V of the item go into the buffer of its parity, free since the item two back finished: they
        // are on their way while the item before still runs
        const int kb = w & 1;
        if (!mbar_wait(&kv_empty[kb], ((w >> 1) & 1) ^ 1, abort_flag, status)) break;
        const int kvrow = b * T + j * ATT_BK;
        mbar_expect_tx(&kv_full[kb], 2 * ATT_TILE_BYTES);
        att_load_tile(smem + L::K_OFF + kb * L::KV_BYTES, &tmap_qkv, &kv_full[kb], hs, nh + h, kvrow);
        att_load_tile(smem + L::V_OFF + kb * L::KV_BYTES, &tmap_qkv, &kv_full[kb], hs, 2 * nh + h, kvrow);
        for (int it = 0; it < steps; ++it, ++g) {
          const int s = g % L::QSTAGES;
          if (!mbar_wait(&q_empty[s], ((g / L::QSTAGES) & 1) ^ 1, abort_flag, status)) { ok = false; break; }
          mbar_expect_tx(&q_full[s], 2 * ATT_TILE_BYTES);
          const int qrow = b * T + (j + it) * ATT_BQ;
          att_load_tile(smem + L::Q_OFF + s * ATT_TILE_BYTES, &tmap_qkv, &q_full[s], hs, h, qrow);
          att_load_tile(smem + L::DO_OFF + s * ATT_TILE_BYTES, &tmap_do, &q_full[s], hs, h, qrow);
          // The pair two steps on is asked into L2 now: its load can only start when its stage is released, and
          // the time from there to the data is on the issuing thread's path.
          if (hs == 64 && it + 2 < steps) {
            tma_prefetch_l2_2d(&tmap_qkv, h * 64, qrow + 2 * ATT_BQ);
            tma_prefetch_l2_2d(&tmap_do, h * 64, qrow + 2 * ATT_BQ);
          }
        }
        ++w;
      }
    }
  } else if (warp == MMA_WARP) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      const uint32_t id_s = make_idesc_bf16(128, 128, 0, 0);      // Q K^T and dO V^T
      const uint32_t id_t = make_idesc_bf16(128, 64, 1, 1);       // P^T dO and dS^T Q : A M-major, B N-major
      const uint32_t id_q = make_idesc_bf16(128, 64, 0, 1);       // dS K : A K-major, B N-major
      // Descriptor low words: K-major operands (leading offset 16) step 32 bytes per MMA, M/N-major ones
      // (leading offset = one tile) step 16 rows of 128 bytes; the high word is the same for all.
      constexpr uint32_t KSTEP = 32 >> 4, MNSTEP = 2048 >> 4, TILE16 = ATT_TILE_BYTES >> 4;
      const uint32_t desc_hi = smem_desc_hi(1024);
      // K and V descriptors of buffer 0; buffer 1 lies KVBUF16 further
      const uint32_t k_km0 = smem_desc_lo(smem_u32(smem + L::K_OFF), 16), v_km0 = smem_desc_lo(smem_u32(smem + L::V_OFF), 16);
      const uint32_t k_mn0 = smem_desc_lo(smem_u32(smem + L::K_OFF), ATT_TILE_BYTES);
      constexpr uint32_t KVBUF16 = L::KV_BYTES >> 4;
      const uint32_t p_mn = smem_desc_lo(smem_u32(smem + L::P_OFF), ATT_TILE_BYTES);
      const uint32_t ds_mn = smem_desc_lo(smem_u32(smem + L::DS_OFF), ATT_TILE_BYTES);
      const uint32_t ds_km = smem_desc_lo(smem_u32(smem + L::DS_OFF), 16);
      uint32_t g = 0, w = 0;
      bool ok = true;
      // S = Q K^T and dP = dO V^T of global step gs, which belongs to item wi (operands: Q/dO stage
      // gs % QSTAGES, K/V buffer wi & 1).  The row threads must have read the pair of the step before out of
      // TMEM; the first step of an item also waits for its K and V.
      auto issue_sdp = [&](uint32_t gs, uint32_t wi, bool first_of_item) -> bool {
        const int st = gs % L::QSTAGES, kb = wi & 1;
        if (gs > 0 && !mbar_wait(sdp_read, (gs - 1) & 1, abort_flag, status)) return false;
        if (first_of_item && !mbar_wait(&kv_full[kb], (wi >> 1) & 1, abort_flag, status)) return false;
        if (!mbar_wait(&q_full[st], (gs / L::QSTAGES) & 1, abort_flag, status)) return false;
        tc_fence_after();
        const uint32_t q_km = smem_desc_lo(smem_u32(smem + L::Q_OFF + st * ATT_TILE_BYTES), 16);
        const uint32_t do_km = smem_desc_lo(smem_u32(smem + L::DO_OFF + st * ATT_TILE_BYTES), 16);
        const uint32_t k_km = k_km0 + kb * KVBUF16, v_km = v_km0 + kb * KVBUF16;
#pragma unroll
        for (int k = 0; k < 4; ++k) umma_bf16_lohi(tm_s, q_km + k * KSTEP, k_km + k * KSTEP, desc_hi, id_s, k > 0);
#pragma unroll
        for (int k = 0; k < 4; ++k) umma_bf16_lohi(tm_dp, do_km + k * KSTEP, v_km + k * KSTEP, desc_hi, id_s, k > 0);
        umma_commit(sdp_full);
        ATT_TRACE(tr, 256, tslot);          // S, dP issued
        return true;
      };
      for (int r = 0; r < rounds && ok; ++r) {
        int idx;
        if (!att_item(r, cta, G, total, idx)) continue;
        const int steps = nq - idx / n_bh;
        bool more = false;                  // does this CTA have another item after this one?
        for (int r2 = r + 1; r2 < rounds && !more; ++r2) {
          int idx2;
          more = att_item(r2, cta, G, total, idx2);
        }
        const int kb = w & 1;
        const uint32_t k_mn = k_mn0 + kb * KVBUF16;
        if (w == 0) ok = issue_sdp(0, 0, true);
        for (int it = 0; it < steps && ok; ++it, ++g) {
          const int s = g % L::QSTAGES;
          const uint32_t sq = smem_u32(smem + L::Q_OFF + s * ATT_TILE_BYTES);
          const uint32_t sdo = smem_u32(smem + L::DO_OFF + s * ATT_TILE_BYTES);
          const uint32_t q_mn = smem_desc_lo(sq, ATT_TILE_BYTES), do_mn = smem_desc_lo(sdo, ATT_TILE_BYTES);
          // The next step's pair goes as soon as the row threads have S and dP of this one in registers, while
          // they are still writing P / dS: they find it finished when they come back for it.  Across items
          // too: the next item's K and V sit in the other buffer.
          if (it + 1 < steps) {
            if (!issue_sdp(g + 1, w, false)) { ok = false; break; }
          } else if (more) {
            if (!issue_sdp(g + 1, w + 1, true)) { ok = false; break; }
          }
          if (!mbar_wait(pds_full, g & 1, abort_flag, status)) { ok = false; break; }
          ATT_TRACE(tr, 256, tslot);          // P, dS ready
          // a new item starts its dV / dK sums from zero: the previous item's must have been read out
          if (it == 0 && w > 0 && !mbar_wait(dkv_free, (w - 1) & 1, abort_flag, status)) { ok = false; break; }
          tc_fence_after();
#pragma unroll
          for (int k = 0; k < 8; ++k)       // dV += P^T dO_i   (K = query rows, 16 per step)
            umma_bf16_lohi(tm_dv, p_mn + k * MNSTEP, do_mn + k * MNSTEP, desc_hi, id_t, (it > 0 || k > 0));
#pragma unroll
          for (int k = 0; k < 8; ++k)       // dK += dS^T Q_i
            umma_bf16_lohi(tm_dk, ds_mn + k * MNSTEP, q_mn + k * MNSTEP, desc_hi, id_t, (it > 0 || k > 0));
          umma_commit(&q_empty[s]);         // Q_i and dO_i have their last readers queued: the stage reloads early
          // the previous step's dQ has been read out of TMEM (the row threads do that right after their hand-over)
          if (g > 0 && !mbar_wait(dq_free, (g - 1) & 1, abort_flag, status)) { ok = false; break; }
          tc_fence_after();
#pragma unroll
          for (int k = 0; k < 8; ++k)       // dQ_i = dS K_j     (K = kv rows)
            umma_bf16_lohi(tm_dq, ds_km + (k >> 2) * TILE16 + (k & 3) * KSTEP, k_mn + k * MNSTEP, desc_hi, id_q, k > 0);
          umma_commit(dq_full);
          if (it + 1 == steps) umma_commit(&kv_empty[kb]);
          ATT_TRACE(tr, 256, tslot);          // dV, dK, dQ issued
        }
        ++w;
      }
    }
  } else if (warp == RED_WARP) {
    // ------------------------------------------------------------ dQ reducer
    // One TMA reduce-add per staged dQ tile into the fp32 dQ scratch.  Issuing a bulk reduction can hold the
    // issuing thread for most of a microsecond while earlier reductions drain into L2, so a thread of its own
    // does it: nothing on a row thread's path waits for global atomics.
    if (lane == 0) {
      uint32_t g = 0, w = 0;
      bool ok = true;
      for (int rr = 0; rr < rounds && ok; ++rr) {
        int idx;
        if (!att_item(rr, cta, G, total, idx)) continue;
        const int j = idx / n_bh, bh = idx % n_bh;
        const int b = bh / nh, h = bh - b * nh;
        for (int i = j; i < nq; ++i, ++g) {
          if (!mbar_wait(dq_staged, g & 1, abort_flag, status)) { ok = false; break; }
          const int row_g = b * T + i * ATT_BQ;
          if (hs == 64) {
#pragma unroll
            for (int hh = 0; hh < 2; ++hh)
              asm volatile("cp.reduce.async.bulk.tensor.2d.global.shared::cta.add.tile.bulk_group [%0, {%1, %2}], [%3];"
                           ::"l"(&tmap_dq), "r"(h * ATT_HS + hh * 32), "r"(row_g),
                             "r"(smem_u32(smem + L::DQ_OFF + hh * ATT_TILE_BYTES))
                           : "memory");
          } else {          // 32 columns per head: the first staging half is the whole dQ tile
            asm volatile("cp.reduce.async.bulk.tensor.3d.global.shared::cta.add.tile.bulk_group [%0, {%1, %2, %3}], [%4];"
                         ::"l"(&tmap_dq), "r"(0), "r"(h), "r"(row_g), "r"(smem_u32(smem + L::DQ_OFF))
                         : "memory");
          }
          asm volatile("cp.async.bulk.commit_group;" ::: "memory");
          asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
          mbar_arrive(dq_stage_free);
        }
        if (ok && hs == 64) {
          // dK and dV of the item: two [128 x 64] bf16 tiles staged in the P buffer, one bulk store each
          if (!mbar_wait(dkv_staged, w & 1, abort_flag, status)) break;
          const int kvrow = b * T + j * ATT_BK;
#pragma unroll
          for (int which = 0; which < 2; ++which)
            asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.tile.bulk_group [%0, {%1, %2}], [%3];"
                         ::"l"(&tmap_dkv), "r"(((which + 1) * nh + h) * ATT_HS), "r"(kvrow),
                           "r"(smem_u32(smem + L::P_OFF + which * ATT_TILE_BYTES))
                         : "memory");
          asm volatile("cp.async.bulk.commit_group;" ::: "memory");
          asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
          mbar_arrive(dkv_stored);
        }
        ++w;
      }
      asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");     // reductions and stores complete before exit
    }
  } else {
    // ------------------------------------------------------------ row threads
    const int q4 = warp & 3, half = warp >> 2;     // TMEM lane quarter, column half
    const int r = q4 * 32 + lane;
    const uint32_t lane_addr = uint32_t(q4 * 32) << 16;
    uint8_t* sp = smem + L::P_OFF;
    uint8_t* sds = smem + L::DS_OFF;
    bool ok = true;
    if (threadIdx.x != 0) tr = nullptr;
    uint8_t* sdq = smem + L::DQ_OFF + half * ATT_TILE_BYTES;     // this thread's half: [128 rows][32 fp32]
    uint32_t g = 0, w = 0;
    float lse_next = 0.f, D_next = 0.f;
    // dQ of global step gs: TMEM -> registers -> swizzled shared tile, which the reducer warp adds into the
    // fp32 dQ scratch.
    auto drain_dq = [&](uint32_t gs) -> bool {
      if (!mbar_wait(dq_full, gs & 1, abort_flag, status)) return false;
      tc_fence_after();
      ATT_TRACE(tr, 0, tslot);                // dQ product done
      uint32_t v[32];
      tmem_ld_32x32(tm_dq + lane_addr + half * 32, v);
      tmem_ld_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(dq_free);
      // the previous reduction must have finished reading the staging tile
      if (gs > 0 && !mbar_wait(dq_stage_free, (gs - 1) & 1, abort_flag, status)) return false;
      ATT_TRACE(tr, 0, tslot);                // the previous reduction has let go of the staging tile
#pragma unroll
      for (int c = 0; c < 8; ++c)
        *reinterpret_cast<uint4*>(sdq + r * 128 + ((c ^ (r & 7)) << 4)) = make_uint4(v[4 * c], v[4 * c + 1], v[4 * c + 2], v[4 * c + 3]);
      fence_proxy_async();
      __syncwarp();
      if (lane == 0) mbar_arrive(dq_staged);
      ATT_TRACE(tr, 0, tslot);                // staged
      return true;
    };
    for (int rr = 0; rr < rounds && ok; ++rr) {
      int idx;
      if (!att_item(rr, cta, G, total, idx)) continue;
      const int j = idx / n_bh, bh = idx % n_bh;
      const int b = bh / nh, h = bh - b * nh;
      const int steps = nq - j;
      // where the next item's first step finds its row statistics (-1: this is the CTA's last item)
      int stat_after = -1;
      for (int r2 = rr + 1; r2 < rounds; ++r2) {
        int idx2;
        if (att_item(r2, cta, G, total, idx2)) {
          stat_after = (idx2 % n_bh) * T + (idx2 / n_bh) * ATT_BQ + r;
          break;
        }
      }
      for (int it = 0; it < steps && ok; ++it, ++g) {
        const int i = j + it;
        const int stat = bh * T + i * ATT_BQ + r;       // < 2^31: the launcher checks B * nh * T
        // row statistics: loaded for the CTA's first step, fetched one step ahead (across items too) after that
        const float lse2 = (g == 0 ? lse[stat] : lse_next) * 1.4426950408889634f;
        const float Dr = g == 0 ? Dvec[stat] : D_next;
        ATT_TRACE(tr, 0, tslot);              // step start
        if (!mbar_wait(sdp_full, g & 1, abort_flag, status)) { ok = false; break; }
        tc_fence_after();
        {
          const int sn = it + 1 < steps ? stat + ATT_BQ : stat_after;
          if (sn >= 0) { lse_next = lse[sn]; D_next = Dvec[sn]; }
        }
        ATT_TRACE(tr, 0, tslot);              // S, dP arrived
        // P and dS of this thread's 64 columns, in registers: the previous step's products may still be
        // reading the shared P / dS tiles
        uint32_t pk_p[2][16], pk_ds[2][16];
        {
          // all 64 columns of S and of dP leave TMEM in one go (a TMEM load takes a few hundred nanoseconds from
          // issue to data, whatever its width: four loads in a row would cost four such waits)
          uint32_t raw[4][2][16];
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            tmem_ld_32x16(tm_s + lane_addr + half * 64 + q * 16, raw[q][0]);
            tmem_ld_32x16(tm_dp + lane_addr + half * 64 + q * 16, raw[q][1]);
          }
          tmem_ld_wait();
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            const int c0 = half * 64 + q * 16;
            uint32_t* op = &pk_p[q >> 1][(q & 1) * 8];
            uint32_t* ods = &pk_ds[q >> 1][(q & 1) * 8];
            if (it == 0) bwd_row_chunk<true, 16>(raw[q][0], raw[q][1], op, ods, c0, r, scale_log2, lse2, Dr, scale);
            else         bwd_row_chunk<false, 16>(raw[q][0], raw[q][1], op, ods, c0, r, scale_log2, lse2, Dr, scale);
          }
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(sdp_read);   // S and dP are in registers: the next pair may replace them
        ATT_TRACE(tr, 0, tslot);              // P, dS computed
        // the previous step's products must be done with P / dS before they are overwritten (the last step of
        // the item before was waited for when its dQ was taken out)
        if (it > 0 && !mbar_wait(dq_full, (g - 1) & 1, abort_flag, status)) { ok = false; break; }
        // ... and the bulk stores of the item before with the dK / dV tiles staged in the P buffer
        if (it == 0 && w > 0 && hs == 64 && !mbar_wait(dkv_stored, (w - 1) & 1, abort_flag, status)) { ok = false; break; }
#pragma unroll
        for (int cc = 0; cc < 2; ++cc) {
#pragma unroll
          for (int c = 0; c < 32; c += 8) {
            const int q = c >> 1;
            *reinterpret_cast<uint4*>(sds + p_offset(r, half * 64 + cc * 32 + c)) =
                make_uint4(pk_ds[cc][q], pk_ds[cc][q + 1], pk_ds[cc][q + 2], pk_ds[cc][q + 3]);
          }
        }
#pragma unroll
        for (int cc = 0; cc < 2; ++cc) {
#pragma unroll
          for (int c = 0; c < 32; c += 8) {
            const int q = c >> 1;
            *reinterpret_cast<uint4*>(sp + p_offset(r, half * 64 + cc * 32 + c)) =
                make_uint4(pk_p[cc][q], pk_p[cc][q + 1], pk_p[cc][q + 2], pk_p[cc][q + 3]);
          }
        }
        ATT_TRACE(tr, 0, tslot);              // P, dS written
        fence_proxy_async();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(pds_full);
        // the previous step's dQ leaves after the hand-over, off the critical path (the next dQ product
        // waits for its read-out)
        if (it > 0 && !drain_dq(g - 1)) { ok = false; break; }
      }
      // the last step's dQ; its barrier also says that every dV / dK product of the item is done
      if (!ok || !drain_dq(g - 1)) { ok = false; break; }
      // dV and dK rows of this kv tile (TMEM lane = kv row)
      __nv_bfloat16* row = dqkv + (long long)(b * T + j * ATT_BK + r) * 3 * d + h * hs;
      uint32_t vk[32], vv[32];
      tmem_ld_32x32(tm_dk + lane_addr + half * 32, vk);
      tmem_ld_32x32(tm_dv + lane_addr + half * 32, vv);
      tmem_ld_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(dkv_free);          // the next item's first products may overwrite the sums
      if (hs == 64) {
        // staged as two 128-byte-swizzled [128 x 64] bf16 tiles (dK, dV) in the P buffer, which nothing reads
        // any more; the reducer warp stores them with one bulk copy each
#pragma unroll
        for (int which = 0; which < 2; ++which) {
          const uint32_t* v = which == 0 ? vk : vv;
#pragma unroll
          for (int c = 0; c < 4; ++c)
            *reinterpret_cast<uint4*>(sp + which * ATT_TILE_BYTES + r * 128 + (((half * 4 + c) ^ (r & 7)) << 4)) = make_uint4(
                pack_bf16(__uint_as_float(v[8 * c]), __uint_as_float(v[8 * c + 1])),
                pack_bf16(__uint_as_float(v[8 * c + 2]), __uint_as_float(v[8 * c + 3])),
                pack_bf16(__uint_as_float(v[8 * c + 4]), __uint_as_float(v[8 * c + 5])),
                pack_bf16(__uint_as_float(v[8 * c + 6]), __uint_as_float(v[8 * c + 7])));
        }
        fence_proxy_async();
        __syncwarp();
        if (lane == 0) mbar_arrive(dkv_staged);
      } else if (half * 32 < hs) {
#pragma unroll
        for (int which = 0; which < 2; ++which) {
          __nv_bfloat16* dst = row + (which == 0 ? d : 2 * d) + half * 32;
#pragma unroll
          for (int c = 0; c < 32; c += 8) {
            const uint32_t* v = which == 0 ? vk : vv;
            *reinterpret_cast<uint4*>(dst + c) = make_uint4(
                pack_bf16(__uint_as_float(v[c]), __uint_as_float(v[c + 1])),
                pack_bf16(__uint_as_float(v[c + 2]), __uint_as_float(v[c + 3])),
                pack_bf16(__uint_as_float(v[c + 4]), __uint_as_float(v[c + 5])),
                pack_bf16(__uint_as_float(v[c + 6]), __uint_as_float(v[c + 7])));
          }
        }
      }
      ++w;
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == MMA_WARP) {
    tc_fence_after();
    tmem_dealloc(tmem_base, 512);
  }
}

}  // namespace dsw

using namespace dsw;

static long long* g_att_trace = nullptr;

static int att_num_sms() {
  static int n = 0;
  if (n == 0) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess ||
        n <= 0)
      n = 148;
  }
  return n;
}
// Register (or clear, with nullptr) a device buffer of 512 int64 for the in-kernel timeline.
extern "C" int dsw_attention_set_trace(long long* buf) { g_att_trace = buf; return 0; }

// qkv: bf16 [B*T, 3*nh*hs]; out: bf16 [B*T, nh*hs]; lse: fp32 [B*nh*T].
// Requires hs == 64 or 32 and T a multiple of 128.
extern "C" int dsw_attention_fwd(const void* qkv, void* out, float* lse, int B, int T, int nh, int hs, float scale,
                                 int* status, cudaStream_t st) {
  if ((hs != 64 && hs != 32) || T % ATT_BQ != 0) return -10;
  const int d = nh * hs;
  CUtensorMap tm;
  int rc = hs == 64 ? make_tmap_bf16_2d(&tm, qkv, 3LL * d, (long long)B * T, 3LL * d, 64, 128)
                    : make_tmap_3d(&tm, 0, qkv, hs, 3LL * nh, (long long)B * T, 3LL * d, 64, 128);
  if (rc) return rc;
  static bool attr_set = false;
  if (!attr_set) {
    if (cudaFuncSetAttribute(attention_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, AttSmem::TOTAL) !=
        cudaSuccess)
      return -2;
    attr_set = true;
  }
  // persistent: two CTAs per SM walk the work items
  const int total = (T / ATT_BQ) * B * nh;
  const int G = total < 2 * att_num_sms() ? total : 2 * att_num_sms();
  attention_fwd_kernel<<<G, ATT_THREADS, AttSmem::TOTAL, st>>>(tm, (__nv_bfloat16*)out, lse, T, nh, B * nh, hs,
                                                               scale * 1.4426950408889634f, status, g_att_trace);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

// qkv, out, dout as in the forward; lse from the forward.  dqkv: bf16 [B*T, 3*d] (all of it is written).
// dq_acc: fp32 scratch [B*T, d]; Dvec: fp32 scratch [B*nh*T].  Both are overwritten.
extern "C" int dsw_attention_bwd(const void* qkv, const void* out, const void* dout, const float* lse, void* dqkv,
                                 float* dq_acc, float* Dvec, int B, int T, int nh, int hs, float scale, int* status,
                                 cudaStream_t st) {
  if ((hs != 64 && hs != 32) || T % ATT_BQ != 0 || (long long)B * nh * T >= (1LL << 31)) return -10;
  const int d = nh * hs;
  const long long rows = (long long)B * T;
  CUtensorMap tq, tdo, tdq, tdkv;
  int rc;
  if (hs == 64) {
    rc = make_tmap_bf16_2d(&tq, qkv, 3LL * d, rows, 3LL * d, 64, 128);
    if (!rc) rc = make_tmap_bf16_2d(&tdkv, dqkv, 3LL * d, rows, 3LL * d, 64, 128);
    if (!rc) rc = make_tmap_bf16_2d(&tdo, dout, d, rows, d, 64, 128);
    if (!rc) rc = make_tmap_f32_2d(&tdq, dq_acc, d, rows, d, 32, 128);
  } else {
    rc = make_tmap_3d(&tq, 0, qkv, hs, 3LL * nh, rows, 3LL * d, 64, 128);
    tdkv = tq;            // not used with 32 columns per head: dK and dV are stored by the row threads
    if (!rc) rc = make_tmap_3d(&tdo, 0, dout, hs, nh, rows, d, 64, 128);
    if (!rc) rc = make_tmap_3d(&tdq, 1, dq_acc, hs, nh, rows, d, 32, 128);
  }
  if (rc) return rc;
  static bool attr_set = false;
  if (!attr_set) {
    if (cudaFuncSetAttribute(attention_bwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, AttBwdSmem::TOTAL) !=
        cudaSuccess)
      return -2;
    attr_set = true;
  }
  // D = rowsum(dO * O) per head, and the dQ accumulator zeroed in the same pass
  {
    const long long want = (rows * 32 + 255) / 256;
    const int cap = att_num_sms() * 16;
    attention_bwd_prep_kernel<<<(unsigned)(want < cap ? want : cap), 256, 0, st>>>(
        (const __nv_bfloat16*)out, (const __nv_bfloat16*)dout, Dvec, dq_acc, B, T, nh, hs);
  }
  // persistent: one CTA per SM walks the work items
  const int total = (T / ATT_BK) * B * nh;
  const int G = total < att_num_sms() ? total : att_num_sms();
  attention_bwd_kernel<<<G, ATT_BWD_THREADS, AttBwdSmem::TOTAL, st>>>(tq, tdo, tdq, tdkv, lse, Dvec, (__nv_bfloat16*)dqkv, T, nh,
                                                                       B * nh, hs, scale, status, g_att_trace);
  attention_dq_convert_kernel<<<148 * 4, 256, 0, st>>>(dq_acc, (__nv_bfloat16*)dqkv, (long long)B * T, d);
  return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

extern "C" int dsw_load_attention() {
  cudaFuncAttributes a;
  int bad = 0;
  bad |= cudaFuncGetAttributes(&a, attention_fwd_kernel) != cudaSuccess;
  bad |= cudaFuncGetAttributes(&a, attention_bwd_kernel) != cudaSuccess;
  bad |= cudaFuncGetAttributes(&a, attention_bwd_prep_kernel) != cudaSuccess;
  bad |= cudaFuncGetAttributes(&a, attention_dq_convert_kernel) != cudaSuccess;
  return bad ? -1 : 0;
}
