// C ABI of libdswarm_host.so: seeded SWARM routing and the static per-rank plan.
// Plain C++17, no CUDA: every rank (and the CPU-only tools) evaluates these
// functions and gets the same tables.
//
// Ranks of stage s are {s, s+S, s+2S, ...}.  path[mb*S + s] is the global rank
// that serves microbatch mb at stage s.  alive (optional) is one byte per rank.
#pragma once
#include <stdint.h>

#define DSW_OP_FWD 0       // forward of one microbatch
#define DSW_OP_BWD 1       // backward of one microbatch
#define DSW_OP_FWD_BWD 2   // last stage: forward immediately followed by backward

#define DSW_ROUTE_UNIFORM 0    // every hop an independent uniform draw over the live replicas
#define DSW_ROUTE_BALANCED 1   // per stage a seeded permutation of an evenly filled assignment

#ifdef __cplusplus
extern "C" {
#endif

// Returns 0, or -1 if some stage has no live replica.
int dsw_route(uint64_t seed, uint64_t step, int S, int world, int M, const uint8_t* alive, int mode,
              int32_t* path);
// Hops land on live replica r of the next stage with probability weights[r] / (live weights of that stage).
int dsw_route_weighted(uint64_t seed, uint64_t step, int S, int world, int M, const uint8_t* alive,
                       const double* weights, int32_t* path);
// Writes the ops of `rank` as records {kind, mb, prev_rank, next_rank} into ops (capacity max_ops records)
// and returns their count; -2 if the simulation stalls, -3 if max_ops is too small.  cost_f / cost_b
// (optional) are per-stage forward and backward times for the simulation; forward_only = 1 gives the
// evaluation plan.
int dsw_plan(int S, int world, int M, int cap, const int32_t* path, const float* cost_f, const float* cost_b,
             int forward_only, int rank, int32_t* ops, int max_ops);

// Thread-to-element map of the fused collectives (coll_index.h), for tests: out[v] = block that touches
// vector v of the bucket in `phase` (0 cast-in, 1 reduce, 2 widen-out) on replica `rank`, -1 if none.
// Returns 0, or -1 on bad arguments.
int dsw_coll_touch_map(long long offset, long long count, long long shard, int R, int rank, int phase, int grid,
                       int block, int vec, int32_t* out);

#ifdef __cplusplus
}
#endif
