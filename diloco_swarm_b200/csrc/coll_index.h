// Which thread of which block touches which elements in the fused collectives.
//
// The cross-GPU barrier of these kernels is per block index: block b of a
// replica waits only for block b of every peer.  So whatever block b reads
// after a barrier must have been written, before that barrier, by block b of
// the replica that owns the memory.  That holds when every phase of a kernel
// walks a bucket slice by slice with the same thread-to-element map inside a
// slice: element p (in vectors of `vec` elements) of slice s belongs to global
// thread p mod nth on every replica and in every phase, whether the phase
// covers all slices (cast-in, widen-out) or only the replica's own (reduce).
//
// Shared by collectives.cu (device) and coll_index.cpp (host, where a CPU test
// checks the property for many bucket sizes, replica counts and grids).
#pragma once

#if defined(__CUDACC__)
#define DSW_HD __host__ __device__ __forceinline__
#else
#define DSW_HD inline
#endif

// Calls f(i) for the first element i of every vector that global thread `tid`
// of `nth` owns in slices [slice_lo, slice_hi) of the bucket
// [offset, offset + count); slice s is [offset + s*shard, offset + (s+1)*shard)
// clipped to the bucket.  offset, count and shard are multiples of vec.
template <class F>
DSW_HD void dsw_for_each_owned(long long offset, long long count, long long shard, int slice_lo, int slice_hi,
                               long long tid, long long nth, int vec, F&& f) {
  const long long end = offset + count;
  for (int s = slice_lo; s < slice_hi; ++s) {
    const long long lo = offset + (long long)s * shard;
    const long long hi = lo + shard < end ? lo + shard : end;
    for (long long i = lo + vec * tid; i < hi; i += vec * nth) f(i);
  }
}
