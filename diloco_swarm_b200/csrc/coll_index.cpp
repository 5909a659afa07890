// Host-side view of the fused collectives' thread-to-element map (coll_index.h),
// so that a CPU test can check the property the per-block barrier relies on.
#include <cstdint>
#include "coll_index.h"
#include "dswarm_host.h"

// out[v] (count / vec entries, one per vector of the bucket) = index of the block whose threads touch
// that vector in `phase` on replica `rank`, or -1 when the phase does not touch it there.
// phase 0 = cast-in (every slice), 1 = reduce (the replica's own slice), 2 = widen-out (every slice).
// Returns 0, or -1 on bad arguments.
extern "C" int dsw_coll_touch_map(long long offset, long long count, long long shard, int R, int rank,
                                  int phase, int grid, int block, int vec, int32_t* out) {
  if (R < 1 || rank < 0 || rank >= R || grid < 1 || block < 1 || vec < 1 || phase < 0 || phase > 2) return -1;
  if (offset % vec || count % vec || shard % vec) return -1;
  const long long nvec = count / vec;
  for (long long v = 0; v < nvec; ++v) out[v] = -1;
  const long long nth = (long long)grid * block;
  const int lo = phase == 1 ? rank : 0, hi = phase == 1 ? rank + 1 : R;
  for (long long tid = 0; tid < nth; ++tid) {
    const int32_t b = int32_t(tid / block);
    dsw_for_each_owned(offset, count, shard, lo, hi, tid, nth, vec, [&](long long i) {
      out[(i - offset) / vec] = b;
    });
  }
  return 0;
}
