// Seeded SWARM routing and the static per-rank execution plan.
//
// The reference picks the next-stage replica of every microbatch with an
// unseeded random.choice on the sender (src/comm.py:91), the receiver takes
// messages from any source (src/comm.py:67), and step completion is a counter
// in a TCP store polled by every rank (src/world.py:73-94).  Here every rank
// evaluates the same counter-based generator, so the whole routing table of a
// step is known everywhere in advance: receivers know their sources, nobody
// polls a store, and each rank knows which backward is its last one (which is
// what lets the gradient all-reduce start bucket by bucket).
//
// The plan of a rank is the order in which it runs forwards and backwards.  It
// is obtained by replaying the reference's greedy policy (prefer a forward
// while fewer than `cap` microbatches are stashed, else a backward,
// src/train.py:188,230; the last stage runs forward and backward back to
// back, src/train.py:211-226) in a deterministic discrete-event simulation
// that all ranks compute identically.  Any order that is a valid causal
// execution is deadlock-free for in-order point-to-point channels; the
// simulation yields one.
#include <cstdint>
#include <cstring>
#include <deque>
#include <vector>
#include <algorithm>
#include <limits>
#include "dswarm_host.h"

namespace {

// Philox4x32-10 (Salmon et al., SC'11).
struct Philox {
  static inline void round(uint32_t c[4], const uint32_t k[2]) {
    const uint64_t p0 = 0xD2511F53ull * c[0];
    const uint64_t p1 = 0xCD9E8D57ull * c[2];
    const uint32_t hi0 = uint32_t(p0 >> 32), lo0 = uint32_t(p0);
    const uint32_t hi1 = uint32_t(p1 >> 32), lo1 = uint32_t(p1);
    const uint32_t n0 = hi1 ^ c[1] ^ k[0];
    const uint32_t n1 = lo1;
    const uint32_t n2 = hi0 ^ c[3] ^ k[1];
    const uint32_t n3 = lo0;
    c[0] = n0; c[1] = n1; c[2] = n2; c[3] = n3;
  }
  static inline uint32_t draw(uint64_t seed, uint64_t step, uint32_t mb, uint32_t boundary) {
    uint32_t c[4] = {uint32_t(step), uint32_t(step >> 32), mb, boundary};
    uint32_t k[2] = {uint32_t(seed), uint32_t(seed >> 32)};
    for (int i = 0; i < 10; ++i) {
      round(c, k);
      k[0] += 0x9E3779B9u;
      k[1] += 0xBB67AE85u;
    }
    return c[0];
  }
};

struct Msg {
  double t;      // arrival time
  int from;      // sender rank (tie-break)
  int seq;       // sender-side sequence number (keeps per-pair FIFO order)
  int mb;
  bool operator<(const Msg& o) const {
    if (t != o.t) return t < o.t;
    if (from != o.from) return from < o.from;
    return seq < o.seq;
  }
};

struct RankState {
  double t_free = 0.0;
  std::vector<Msg> fq, bq;   // kept sorted; small
  int inflight = 0;
  int sent = 0;
};

inline void push_sorted(std::vector<Msg>& q, const Msg& m) {
  q.insert(std::upper_bound(q.begin(), q.end(), m), m);
}

}  // namespace

extern "C" {

// Ranks of stage s are {s, s+S, s+2S, ...} (src/world.py:96-97).
// path[mb*S + s] = global rank that serves microbatch mb at stage s.
// Microbatch mb starts at the (mb mod R0)-th live replica of stage 0
// (round-robin chunks, src/sampler.py:35-38); every later hop is a uniform
// draw over the live replicas of the next stage.
// Returns 0, or -1 if some stage has no live replica.
// mode 0: every hop is an independent uniform draw (the reference's behaviour).
// mode 1: balanced: per stage, a seeded random permutation of an evenly filled
//         assignment, so every live replica serves floor or ceil of M/R microbatches
//         while each microbatch's replica is still uniformly distributed.
int dsw_route(uint64_t seed, uint64_t step, int S, int world, int M,
              const uint8_t* alive, int mode, int32_t* path) {
  std::vector<std::vector<int>> live(S);
  for (int r = 0; r < world; ++r)
    if (!alive || alive[r]) live[r % S].push_back(r);
  for (int s = 0; s < S; ++s)
    if (live[s].empty()) return -1;
  for (int mb = 0; mb < M; ++mb) {
    path[mb * S + 0] = live[0][mb % int(live[0].size())];
    if (mode == 0) {
      for (int s = 1; s < S; ++s) {
        const uint32_t u = Philox::draw(seed, step, uint32_t(mb), uint32_t(s - 1));
        path[mb * S + s] = live[s][u % uint32_t(live[s].size())];
      }
    }
  }
  if (mode == 1) {
    std::vector<int> slot(M);
    for (int s = 1; s < S; ++s) {
      const int L = int(live[s].size());
      for (int mb = 0; mb < M; ++mb) slot[mb] = mb % L;
      for (int i = M - 1; i > 0; --i) {        // Fisher-Yates with counter-based draws
        const uint32_t u = Philox::draw(seed ^ 0x5bd1e995u, step, uint32_t(i), uint32_t(s - 1));
        std::swap(slot[i], slot[u % uint32_t(i + 1)]);
      }
      // a random rotation removes the bias of "mb % L" when L does not divide M
      const uint32_t rot = Philox::draw(seed ^ 0x5bd1e995u, step, 0xffffffffu, uint32_t(s - 1));
      for (int mb = 0; mb < M; ++mb) path[mb * S + s] = live[s][(slot[mb] + rot) % uint32_t(L)];
    }
  }
  return 0;
}

// Throughput-weighted wiring (the SWARM paper's rule; the reference draws uniformly): the first stage keeps
// its round-robin chunks, every later hop lands on live replica r of the next stage with probability
// weights[r] / sum of the live weights of that stage.  Non-positive weights count as zero; a stage whose
// live weights are all zero falls back to a uniform draw.  Returns 0, or -1 if a stage has no live replica.
int dsw_route_weighted(uint64_t seed, uint64_t step, int S, int world, int M, const uint8_t* alive,
                       const double* weights, int32_t* path) {
  std::vector<std::vector<int>> live(S);
  for (int r = 0; r < world; ++r)
    if (!alive || alive[r]) live[r % S].push_back(r);
  for (int s = 0; s < S; ++s)
    if (live[s].empty()) return -1;
  std::vector<std::vector<double>> cum(S);
  for (int s = 1; s < S; ++s) {
    double acc = 0.0;
    for (int r : live[s]) {
      acc += weights && weights[r] > 0.0 ? weights[r] : 0.0;
      cum[s].push_back(acc);
    }
  }
  for (int mb = 0; mb < M; ++mb) {
    path[mb * S + 0] = live[0][mb % int(live[0].size())];
    for (int s = 1; s < S; ++s) {
      const uint32_t u = Philox::draw(seed ^ 0x27d4eb2fu, step, uint32_t(mb), uint32_t(s - 1));
      const double total = cum[s].back();
      if (total <= 0.0) {
        path[mb * S + s] = live[s][u % uint32_t(live[s].size())];
        continue;
      }
      const double x = (double(u) + 0.5) / 4294967296.0 * total;
      const size_t k = size_t(std::upper_bound(cum[s].begin(), cum[s].end(), x) - cum[s].begin());
      path[mb * S + s] = live[s][std::min(k, live[s].size() - 1)];
    }
  }
  return 0;
}

// Op record: {kind, mb, prev_rank, next_rank}; kind 0 = forward, 1 = backward,
// 2 = forward immediately followed by backward (last stage).
// forward_only = 1 gives the evaluation plan (src/train.py:76-141).
// Writes the ops of `rank` into ops (capacity max_ops records) and returns
// their count; -2 if the simulation stalls (cannot happen for cap >= 1),
// -3 if max_ops is too small.
int dsw_plan(int S, int world, int M, int cap, const int32_t* path,
             const float* cost_f, const float* cost_b, int forward_only,
             int rank, int32_t* ops, int max_ops) {
  if (cap < 1) cap = 1;
  std::vector<RankState> st(world);
  // microbatches enter stage 0 at time 0 in index order
  for (int mb = 0; mb < M; ++mb) {
    const int r0 = path[mb * S];
    st[r0].fq.push_back(Msg{0.0, -1, mb, mb});
  }
  long remaining = 0;
  for (int mb = 0; mb < M; ++mb) remaining += forward_only ? S : 2 * S;
  int n_out = 0;
  const double INF = std::numeric_limits<double>::infinity();
  while (remaining > 0) {
    int best = -1, best_kind = -1;
    double best_t = INF;
    for (int r = 0; r < world; ++r) {
      RankState& s = st[r];
      const int stage = r % S;
      const bool last = stage == S - 1;
      const bool can_f = !s.fq.empty() && (forward_only || last || s.inflight < cap);
      const bool can_b = !s.bq.empty();
      if (!can_f && !can_b) continue;
      const double af = can_f ? s.fq.front().t : INF;
      const double ab = can_b ? s.bq.front().t : INF;
      const double t = std::max(s.t_free, std::min(af, ab));
      // at time t, prefer a forward if one has arrived
      const int kind = (can_f && af <= t) ? 0 : 1;
      if (t < best_t) { best_t = t; best = r; best_kind = kind; }
    }
    if (best < 0) return -2;
    RankState& s = st[best];
    const int stage = best % S;
    const bool last = stage == S - 1;
    Msg m;
    int kind = best_kind;
    if (kind == 0) { m = s.fq.front(); s.fq.erase(s.fq.begin()); }
    else           { m = s.bq.front(); s.bq.erase(s.bq.begin()); }
    const int mb = m.mb;
    const int prev = stage > 0 ? path[mb * S + stage - 1] : -1;
    const int next = !last ? path[mb * S + stage + 1] : -1;
    double dur;
    if (kind == 0) {
      dur = cost_f ? cost_f[stage] : 1.0;
      if (last && !forward_only) { kind = 2; dur += cost_b ? cost_b[stage] : 2.0; }
    } else {
      dur = cost_b ? cost_b[stage] : 2.0;
    }
    const double t_end = best_t + dur;
    s.t_free = t_end;
    if (kind == 0) {
      remaining -= 1;
      if (!forward_only) s.inflight += 1;
      if (next >= 0) push_sorted(st[next].fq, Msg{t_end, best, s.sent++, mb});
    } else if (kind == 2) {
      remaining -= 2;
      if (prev >= 0) push_sorted(st[prev].bq, Msg{t_end, best, s.sent++, mb});
    } else {
      remaining -= 1;
      s.inflight -= 1;
      if (prev >= 0) push_sorted(st[prev].bq, Msg{t_end, best, s.sent++, mb});
    }
    if (best == rank) {
      if (n_out >= max_ops) return -3;
      int32_t* o = ops + 4 * n_out++;
      o[0] = kind; o[1] = mb; o[2] = prev; o[3] = next;
    }
  }
  return n_out;
}

}  // extern "C"
