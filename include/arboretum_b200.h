/* C ABI of libarboretum.so (B200 build).
 *
 * The first fourteen functions are the reference's python-wrapper ABI
 * (python-wrapper/arboretum_wrapper.h:4-39), re-exported one to one so that the
 * reference's python-package/arboretum/core.py loads this library unchanged.
 * Every function returns NULL on success, else a NUL-terminated message owned by
 * the library (valid until the next failing call on the same thread).  Handles
 * are opaque; a NULL handle passed to a free function is ignored.  Unlike the
 * reference no call ever exits the process or lets a C++ exception escape.
 *
 * The functions below the "additive" line do not exist in the reference.
 */
#ifndef ARBORETUM_B200_H
#define ARBORETUM_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef void *VoidPointer;

/* arboretum_wrapper.h:6-9 / arboretum_wrapper.cu:16-39.  `data` is row-major
 * [nrow][ncol] fp32, `categories` row-major [nrow][ccol] or NULL; both are
 * copied.  `missing` is accepted and ignored, like in the reference. */
const char *ACreateFromDenseMatrix(const float *data, const unsigned int *categories, int nrow,
                                   int ncol, int ccol, float missing, VoidPointer *out);
/* arboretum_wrapper.h:11 / .cu:41-55 */
const char *ASetY(VoidPointer data, const float *y);
/* arboretum_wrapper.h:13 / .cu:57-71 */
const char *ASetLabel(VoidPointer data, const unsigned char *labels);
/* arboretum_wrapper.h:15 / .cu:73-86 */
const char *ASetWeights(VoidPointer data, const float *weights);
/* arboretum_wrapper.h:17-18 / .cu:88-99: nested JSON configuration */
const char *AInitGarden(const char *configuration, VoidPointer *garden);
/* arboretum_wrapper.h:20-21 / .cu:101-111: one boosting round (labels_count trees).
 * The first call quantises `data` and binds the garden to it. */
const char *AGrowTree(VoidPointer garden, VoidPointer data, const float *grad);
/* arboretum_wrapper.h:23 / .cu:180-191 */
const char *AAppendLastTree(VoidPointer garden, VoidPointer data);
/* arboretum_wrapper.h:25-26 / .cu:153-178: *out = new float[rows * labels] */
const char *AGetY(VoidPointer garden, VoidPointer data, const float **out);
/* arboretum_wrapper.h:28-29 / .cu:113-139: n_rounds == -1 means all trees */
const char *APredict(VoidPointer garden, VoidPointer data, const float **out, const int n_rounds);
/* arboretum_wrapper.h:31 / .cu:141-145: *model = heap C string (argument order as there) */
const char *ADumpModel(const char **model, VoidPointer garden);
/* arboretum_wrapper.h:33 / .cu:147-151 */
const char *ALoadModel(const char *model, VoidPointer garden);
/* arboretum_wrapper.h:35-39 / .cu:193-205 */
const char *AFreeDMatrix(VoidPointer ptr);
const char *AFreeGarden(VoidPointer ptr);
const char *ADeleteArray(float *in);

/* ------------------------------- additive ---------------------------------- */

/* Rows that are already binned (uint8 ids < hist_size, row-major [nrow][ncol]);
 * the reference ingests fp32 only (arboretum_wrapper.h:6-9).  `bins` may point to host or
 * to device memory (rows generated or decoded on the GPU); so may ASetY's `y` for a matrix
 * that lives in device memory. */
const char *ACreateFromBinnedMatrix(const uint8_t *bins, int64_t nrow, int ncol, int hist_size,
                                    VoidPointer *out);
/* Thresholds computed elsewhere (e.g. on the whole data set before sharding rows
 * over GPUs): thr is [ncol][hist_size], size[f] = bins in use.  Must precede the
 * first AGrowTree. */
const char *ASetThresholds(VoidPointer data, const float *thr, const int *size, int hist_size);
/* Quantise now (what the first AGrowTree would do) and read the result back:
 * thr [ncol][hist_size], size [ncol], bins [nrow][ncol] uint16; any may be NULL. */
const char *AQuantize(VoidPointer data, int hist_size, int missing_bin, float *thr, int *size,
                      uint16_t *bins);
/* Training-time predictions of the bound DMatrix, internal scale, [labels][rows]. */
const char *AGetTrainY(VoidPointer garden, float *out);
/* Split records of level `level` of the last grown tree: arrays of 1 << level
 * entries (node_begin: one more).  Sums are in gradient units. */
const char *AGetLevelStats(VoidPointer garden, int level, unsigned *node_begin, float *gain,
                           int *fid, int *bin, double *left_g, double *left_h, double *tot_g,
                           double *tot_h, unsigned *left_count);
/* The same for tree `tree_in_round` (0 .. labels_count - 1, -1 = the last) of the last round:
 * multi:softmax grows one tree per class in every round. */
const char *AGetLevelStatsOf(VoidPointer garden, int tree_in_round, int level, unsigned *node_begin,
                             float *gain, int *fid, int *bin, double *left_g, double *left_h,
                             double *tot_g, double *tot_h, unsigned *left_count);
/* The fixed-point steps of the last round: every gradient (hessian) entered the histograms
 * as an integer multiple of *g_step (*h_step), off from its float value by less than one
 * step. */
const char *AGetGradientStep(VoidPointer garden, double *g_step, double *h_step);
/* CUDA-event timing of the kernel classes: switch on, then read a JSON summary. */
const char *ASetProfile(VoidPointer garden, int on);
const char *AGetTimings(VoidPointer garden, const char **json);
/* One histogram launch over host buffers (kernel-level parity and measurement):
 * bins row-major [nrow][ncol] of `bin_bytes`-byte ids, grad [nrow] (pair == 0) or
 * [nrow][2]; rowid (NULL = identity) grouped by node with node_begin[n_nodes + 1];
 * out_g / out_h [n_nodes][ncol][hist_size + 1] doubles.  When `reps` > 0 the
 * launch is repeated and its mean device time is stored in *ms. */
const char *ABuildHistogram(const void *bins, int bin_bytes, int64_t nrow, int ncol, int hist_size,
                            const float *grad, int pair, const unsigned *rowid,
                            const unsigned *node_begin, int n_nodes, int quant_bits, double *out_g,
                            double *out_h, int reps, float *ms);
/* The same launch with the subtraction trick (hist_grad_sum.cu:6-33,288-290 of the reference):
 * nodes 2p and 2p + 1 are the children of parent p, whose sums parent_g / parent_h
 * [n_nodes / 2][ncol][hist_size + 1] are given (multiples of the fixed-point step, e.g.
 * integers); only the smaller child of every pair is scanned (ties: the left one), the other
 * is parent - scanned. */
const char *ABuildHistogramFromParents(const void *bins, int bin_bytes, int64_t nrow, int ncol, int hist_size,
                                       const float *grad, int pair, const unsigned *rowid,
                                       const unsigned *node_begin, int n_nodes, int quant_bits,
                                       const double *parent_g, const double *parent_h, double *out_g,
                                       double *out_h);
/* Multi-GPU: rows are sharded over one process per GPU; every level's histogram
 * is summed over the ranks with ncclAllReduce, and the first AGrowTree finds the
 * thresholds of the whole data set with the other ranks (unless ASetThresholds gave
 * them), so bins and trees equal those of the unsharded matrix.  `id` is the 128-byte
 * ncclUniqueId made by rank 0 (ANcclUniqueId) and sent to the others by the host.
 * The first communicator of a process is kept until the process exits; a later Garden
 * of the same rank and world size attaches it when AInitNccl is given id128 == NULL
 * (no bootstrap, no host traffic).  Gardens that share a communicator must not train at
 * the same time. */
const char *ANcclUniqueId(char *id128);
const char *AInitNccl(VoidPointer garden, int rank, int world, const char *id128);

/* No counterpart in the reference.  The waits of the exchange between row shards over peer
 * memory are bounded: a peer that never answers makes a kernel give up after a time limit,
 * record where, and return (the host then reports an error after the tree; the context stays
 * usable).  This call exercises exactly that wait on a word that nothing sets, on the
 * current device: *timed_out becomes 1, *waited_ms about limit_ms (at most 2000). */
const char *APeerWaitProbe(double limit_ms, int *timed_out, double *waited_ms);

/* No counterpart in the reference.  Threshold search of ONE feature for callers that
 * must not allocate device memory (a process whose GPU memory is owned by one
 * arena, a fixed-budget service, a latency-critical section): `sorted_device` holds
 * the column's n values in ascending fp32 radix order in device memory,
 * `thr_device` receives hist_size thresholds (device memory), `stream` is a
 * cudaStream_t (NULL = default stream).  The call only launches kernels; its
 * scratch is a 128 KB array inside the library image, which every GPU that loads
 * the library holds until the process exits.  n may not exceed 67,108,864 (2^26):
 * larger columns return an error and should go through AQuantize.  The first call on
 * a device looks the array's address up (cudaGetSymbolAddress) and may make the
 * runtime load the library's kernels, which takes device memory once: make one
 * warm-up call before a section that must not allocate.  All calls on a device share the array, so two
 * calls that overlap on the GPU (different streams, different threads) race; calls
 * on one stream are safe.  Nothing of an earlier call's scratch contents is read. */
const char *AThresholdsNoAlloc(const float *sorted_device, long long n, int hist_size,
                               float *thr_device, void *stream);

/* Additive (no counterpart in the reference): the library takes its device memory from the
 * current device's stream-ordered pool and keeps what it frees, so that the next matrix or
 * model does not pay for cudaMalloc again; this call hands the unused part back to the
 * driver (for a process that shares the GPU with other allocators), together with the few
 * small pinned host blocks it keeps for the same reason. */
const char *AReleaseCachedMemory(void);

/* Additive (no counterpart in the reference): measures, on the current device, how many
 * (gradient, hessian) pair updates per second the histogram kernels' two shared-memory
 * reductions sustain when nothing else is done (no loads, staging or stores) -- the
 * ceiling of their inner loop.  `steps` x 8 updates per thread of a full grid; a few
 * thousand steps run for a millisecond. */
const char *ASharedAtomicPeak(int steps, double *pair_updates_per_s);

#ifdef __cplusplus
}
#endif
#endif /* ARBORETUM_B200_H */
