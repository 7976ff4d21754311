/*
 * b200wkv_debug - schedule queries of libb200wkv.so that exist for its tests.  Not part of the
 * boundary a host framework binds (that is b200wkv.h); no jaxrwkv interface corresponds to them.
 * Neither call touches a GPU.
 */
#ifndef B200WKV_DEBUG_H_
#define B200WKV_DEBUG_H_

#ifdef __cplusplus
extern "C" {
#endif

/* Work split used by the tensor-core kernels that cut sequences into runs of 64-token blocks.
 * split_plan: grid size and segments per sequence chosen for `chains` = B*H sequences of `n_blk`
 * blocks with `per_sm` resident thread blocks per SM (the SM count is that of the current device,
 * 148 when there is none).  runs: the pieces thread block `cta` of `grid` walks, in walking order, as
 * (sequence, first segment, one-past-last segment) triples written to `runs` (at most `capacity` of
 * them); returns their number. */
int b200wkv_debug_split_plan(int chains, int n_blk, int per_sm, int* grid, int* seg);
int b200wkv_debug_runs(int chains, int seg, int grid, int cta, int* runs, int capacity);

#ifdef __cplusplus
}
#endif
#endif  /* B200WKV_DEBUG_H_ */
