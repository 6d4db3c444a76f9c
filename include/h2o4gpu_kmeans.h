/* C ABI of the B200 k-means engine (libh2o4gpu_kmeans.so).
 *
 * Plain pointers and sizes only.  Every function returns 0 on success and a
 * negative KM_E* code on failure; kmeans_last_error() gives the message of the
 * calling thread's last failure.  Nothing here exits the process, installs a
 * signal handler or throws across the boundary.
 *
 * Section 1 are the reference's exported functions for this path, with the
 * reference's names, parameter order and types.  In the reference they have C++
 * linkage (src/include/solver/kmeans.h:56-76; defined in
 * src/gpu/kmeans/kmeans_h2o4gpu.cu:1060-1097) and are reached through SWIG
 * (src/swig/solver/kmeans.i:1-13).  This library exports them twice: with C++
 * linkage, so code compiled against the reference's header links unchanged, and
 * as the extern "C" names below for ctypes / cgo / JNI style bindings.
 */
#ifndef H2O4GPU_KMEANS_H_
#define H2O4GPU_KMEANS_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- error codes -------------------------------------------------------- */
#define KM_OK 0
#define KM_EINVAL (-1)   /* bad argument (null pointer, k < 1, rows == 0, ...)        */
#define KM_ENOMEM (-2)   /* device or host allocation failed (the reference's -1,    */
                         /* src/gpu/kmeans/kmeans_impl.h:105)                        */
#define KM_ECUDA (-3)    /* a CUDA runtime call or kernel launch failed              */
#define KM_ENODEV (-4)   /* no usable CUDA device / bad device id                    */
#define KM_ENCCL (-5)    /* NCCL missing or a collective failed                      */
#define KM_ENONFINITE (-6) /* NaN or Inf in the data or the centroids                */
#define KM_ETIMEOUT (-7) /* a bounded device-side wait gave up                       */
#define KM_ESTATE (-8)   /* call out of order on a handle (no data, no centroids)    */

const char* kmeans_last_error(void);
/* Of the calling thread's last kmeans_fit_* / make_ptr_*_kmeans fit: Lloyd iterations run
 * (sklearn's n_iter_: up to and including the first one that changed no label) and the sum of
 * squared distances of the rows to their centres (sklearn's inertia_, which the reference's
 * wrapper leaves None, src/interface_py/h2o4gpu/solvers/kmeans.py:187). */
int kmeans_last_fit_info(int* iterations, double* inertia);
/* Device buffers come from one memory pool per device that keeps freed memory for the next
 * call (the reference allocates and frees per call through thrust::device_vector,
 * src/gpu/kmeans/kmeans_h2o4gpu.cu:672-683, 795-812).  This returns everything the pools hold
 * and no live handle uses to the driver.  H2O4GPU_KM_POOL=0 in the environment turns the
 * pools off. */
int kmeans_trim_memory(void);

/* Every wait inside a kernel (for a peer GPU's flag in the multi-GPU exchanges, for an mbarrier in the
 * tensor-core kernels) is bounded: when it runs out the kernel records a code, finishes normally and
 * the call returns KM_ETIMEOUT; the reference exit()s on any device error
 * (src/gpu/kmeans/kmeans_general.h:20-29).  This sets the two limits for the process, in milliseconds
 * (defaults: about 2000 and 3000; a value <= 0 restores the default). */
int kmeans_set_wait_limits(double peer_wait_ms, double mbarrier_wait_ms);
/* Runs one such wait into its limit on device gpu_id, with nothing faulting: which = 0 launches the
 * push all-reduce kernel for a world of two ranks of which the second never delivers, which = 1 a
 * one-warp kernel that waits on an mbarrier nothing arrives at.  Returns KM_ETIMEOUT (the expected
 * outcome; *device_code receives the code the kernel recorded: 11 peer flag, 9 mbarrier) and leaves
 * the device usable.  Set short limits first. */
int kmeans_selftest_wait_timeout(int gpu_id, int which, int* device_code);

/* ---- 1. the reference's entry points ------------------------------------ */

/* Fit (dopredict == 0) or predict (dopredict == 1).
 * Replaces make_ptr_float_kmeans / make_ptr_double_kmeans
 * (src/include/solver/kmeans.h:56-68; src/gpu/kmeans/kmeans_h2o4gpu.cu:977-991,
 * 1060-1082).  Argument meaning as in the reference: verbose = log level,
 * seed < 0 = nondeterministic, devices = (gpu_id + i) % visible for i < n_gpu,
 * mTrain = rows, n = cols, srcdata row-major rows x cols on the host,
 * threshold compared with the summed squared centroid shift
 * (src/gpu/kmeans/kmeans_impl.h:191-208), centroids = k x cols row-major.
 *   init_from_data 0: first k rows of a seeded shuffle (kmeans_h2o4gpu.cu:662-693)
 *   init_from_data 1: k-means|| on the device (kmeans_h2o4gpu.cu:729-742)
 *   init_from_data 2: EXTENSION - start from `centroids` (the reference ignores
 *                     that argument in fit, kmeans_h2o4gpu.cu:983-986).
 * Outputs: if *pred_centroids / *pred_labels is non-NULL on entry it is a caller
 * buffer of k*cols values / rows int32 and is written in place; if it is NULL the
 * library allocates it (release with kmeans_free).  The reference always
 * allocates and never frees (kmeans_h2o4gpu.cu:767-781).  All rows are labelled
 * (the reference drops rows % n_gpu trailing rows, kmeans_h2o4gpu.cu:649). */
int kmeans_fit_f32(int verbose, int seed, int gpu_id, int n_gpu, size_t rows, size_t cols,
                   int k, int max_iterations, int init_from_data, float threshold,
                   const float* srcdata, const float* centroids, float** pred_centroids,
                   int** pred_labels);
int kmeans_fit_f64(int verbose, int seed, int gpu_id, int n_gpu, size_t rows, size_t cols,
                   int k, int max_iterations, int init_from_data, double threshold,
                   const double* srcdata, const double* centroids, double** pred_centroids,
                   int** pred_labels);
/* predict = the dopredict == 1 branch (src/gpu/kmeans/kmeans_h2o4gpu.cu:817-889) */
int kmeans_predict_f32(int verbose, int gpu_id, int n_gpu, size_t rows, size_t cols, int k,
                       const float* srcdata, const float* centroids, int** pred_labels);
int kmeans_predict_f64(int verbose, int gpu_id, int n_gpu, size_t rows, size_t cols, int k,
                       const double* srcdata, const double* centroids, int** pred_labels);
/* Replaces kmeans_transform_float / kmeans_transform_double
 * (src/include/solver/kmeans.h:70-76; kmeans_h2o4gpu.cu:891-975, 1085-1097):
 * squared distances |xn + cn - 2 x.c| (src/gpu/kmeans/kmeans_labels.cu:173-176),
 * ONE column-major rows x k block over the whole matrix, which is the layout
 * src/interface_py/h2o4gpu/solvers/kmeans.py:420-421 reshapes with order='F'. */
int kmeans_transform_f32(int verbose, int gpu_id, int n_gpu, size_t rows, size_t cols, int k,
                         const float* srcdata, const float* centroids, float** preds);
int kmeans_transform_f64(int verbose, int gpu_id, int n_gpu, size_t rows, size_t cols, int k,
                         const double* srcdata, const double* centroids, double** preds);
/* Frees a buffer the library allocated for a NULL output pointer. */
void kmeans_free(void* p);

/* Device count as the wrapper needs it (replaces the count half of
 * get_gpu_info_c, src/gpu/utils.cu:57-90, used by
 * src/interface_py/h2o4gpu/util/gpu.py:14-38). */
int kmeans_device_count(void);

/* ---- 2. resident engine (extension) -------------------------------------
 * The reference re-uploads X on every call (kmeans_h2o4gpu.cu:672-683) and so
 * cannot hold a 100 GB shard or time the Lloyd loop alone.  A handle keeps one
 * row shard per local device resident.  dtype: 0 = float32, 1 = float64.
 * A handle drives `n_local` devices of this process; with world_size > n_local
 * several processes (one per GPU) cooperate through NCCL, rank = world_rank0 +
 * local index.  nccl_id is the 128-byte ncclUniqueId shared by all processes
 * (NULL when world_size == n_local: the library creates the communicators). */
typedef struct km_engine* kmeans_handle_t;

int kmeans_create(kmeans_handle_t* out, int dtype, int n_local, const int* device_ids,
                  int world_rank0, int world_size, const void* nccl_id);
int kmeans_destroy(kmeans_handle_t h);
/* 128-byte NCCL unique id for kmeans_create (rank 0 makes it, the caller ships it). */
int kmeans_nccl_unique_id(void* out128);

/* Attach a shard that already lives on local device `local` (borrowed pointer,
 * row-major rows x cols, 16-byte aligned).  n_total = rows over all ranks. */
int kmeans_attach_device(kmeans_handle_t h, int local, const void* dX, size_t rows, size_t cols,
                         size_t n_total);
/* Upload a host matrix: rows are split contiguously over the local devices
 * (balanced split: rows / n rows each, the first rows % n devices one more; every row
 * covered, no device empty while rows >= n).  order 'r' = row-major, 'c' = column-major
 * (the two layouts of copy_data, src/gpu/kmeans/kmeans_h2o4gpu.h:24-42). */
int kmeans_upload_host(kmeans_handle_t h, const void* X, size_t rows, size_t cols, char order);
/* The same for a host matrix of another element type.  The reference's wrapper converts every
 * input to float32 / float64 on the host before the call (`_to_np`,
 * src/interface_py/h2o4gpu/solvers/utils.py:46-96; kmeans.py:508-521); here the bytes cross the
 * bus as they are (a quarter of them for 8-bit data) and a kernel converts them into the
 * handle's dtype with the rounding of numpy's astype. */
#define KM_DTYPE_F32 0
#define KM_DTYPE_F64 1
#define KM_DTYPE_F16 2
#define KM_DTYPE_I8 3
#define KM_DTYPE_U8 4   /* also numpy bool */
#define KM_DTYPE_I16 5
#define KM_DTYPE_U16 6
#define KM_DTYPE_I32 7
#define KM_DTYPE_U32 8
#define KM_DTYPE_I64 9
#define KM_DTYPE_U64 10
int kmeans_upload_host_typed(kmeans_handle_t h, const void* X, int src_dtype, size_t rows, size_t cols,
                             char order);

/* Sample weights for the next fits / inertia on this handle: `count` values of the handle's dtype,
 * one per local row, shard after shard (NULL: back to unit weights).  A row then adds w * x to its
 * centroid's sum and w to its count, and inertia is the weighted sum - the meaning of
 * fit(X, sample_weight=w) in the wrapper (src/interface_py/h2o4gpu/solvers/kmeans.py:800-804), which
 * the reference can only serve on the CPU.  Weights must be finite and >= 0, not all zero; they enter
 * as 30-bit fixed-point numbers relative to the largest one.  Attaching or uploading other data drops
 * them. */
int kmeans_set_sample_weight(kmeans_handle_t h, const void* weights, size_t count);

/* flags for kmeans_fit_resident */
#define KM_FIT_NO_FINAL_ASSIGN 1 /* skip the closing E-step (benchmark loops)        */
#define KM_FIT_FORCE_SIMT 2      /* never take the tcgen05 distance kernel           */
#define KM_FIT_FORCE_SPLIT 4     /* never take the fused small-k kernel              */
#define KM_FIT_CHECK_EVERY_ITER 8 /* host reads shift/label changes each iteration   */
#define KM_FIT_FULL_SUMS 16       /* recompute the centroid sums from every row in every
                                  * iteration (default: exact incremental update once few
                                  * labels change; same bits either way)              */
#define KM_FIT_PRESPLIT 32        /* d = 64 tensor-core path: build the fp16-split copy of the rows now, whatever
                                    the iteration count (by default only fits of 16 iterations or more pay for it) */

/* Lloyd iterations on the resident shards from k x cols host centroids.
 * Stops after max_iter, or earlier when threshold > 0 and the summed squared
 * shift drops below it, or (with KM_FIT_CHECK_EVERY_ITER) when no label changed. */
int kmeans_fit_resident(kmeans_handle_t h, int k, int max_iter, double threshold,
                        const void* init_centroids, int flags);
/* One E-step on the resident shards with the handle's current centroids (its CUDA-event time on
 * device 0 is left in kmeans_stats.ms_assign). */
int kmeans_assign_resident(kmeans_handle_t h);
int kmeans_set_centroids(kmeans_handle_t h, int k, const void* centroids);
/* Initial centroids from the attached data, computed on the device(s) of a one-process
 * handle: method 0 = the first k rows of a seeded shuffle (copy_centroids_shuffled,
 * src/gpu/kmeans/kmeans_h2o4gpu.cu:662-669, 687-693), method 1 = k-means|| followed by a
 * weighted k-means++ over the candidates (kmeans_parallel / kmeans_plus_plus,
 * kmeans_h2o4gpu.cu:154-279, 331-563), what init_from_data = 1 runs.  out: k x cols
 * row-major host buffer of the handle's dtype; rows_out (may be NULL): the k global row
 * indices the centroids were taken from.  seed < 0 draws a seed.  Leaves the handle's
 * centroid table in an unspecified state; follow with kmeans_fit_resident. */
int kmeans_init_resident(kmeans_handle_t h, int k, int seed, int method, void* out_host, long long* rows_out);
int kmeans_get_centroids(kmeans_handle_t h, void* out_host);
/* labels of local shard `local`, rows int32, to host / as a device pointer */
int kmeans_get_labels(kmeans_handle_t h, int local, int32_t* out_host);
int kmeans_labels_device(kmeans_handle_t h, int local, const int32_t** out_dev);
/* squared distances of shard `local` into a column-major block with leading
 * dimension ld (>= shard rows), written to host memory */
int kmeans_transform_resident(kmeans_handle_t h, int local, void* out_host, size_t ld);

typedef struct kmeans_stats {
  int iterations;          /* Lloyd iterations executed                              */
  int n_iter_converged;    /* first iteration after which no label changed, +1; else 0 */
  int relocations;         /* empty-cluster relocations over the whole fit           */
  int path;                /* 1 fused small-k, 2 SIMT tiles, 3 tcgen05 (of the last fit or transform) */
  int gpu_launches;        /* kernels launched by the last fit (all local devices)   */
  int incremental_iterations; /* iterations (device 0) whose centroid sums were updated from
                               * the rows that changed label instead of recomputed       */
  double last_shift_sq;    /* summed squared centroid shift of the last iteration    */
  double inertia;          /* sum of squared distances after the closing E-step, or -1 */
  double seconds_upload;   /* host-side wall time of the last upload                 */
  double seconds_fit;      /* wall time of the last kmeans_fit_resident              */
  float ms_assign;         /* CUDA-event time of the distance+argmin kernel, summed  */
  float ms_update;         /* ... of the sum / count / finalize kernels              */
  float ms_loop;           /* ... of the whole iteration loop on device 0            */
  float ms_final_assign;   /* ... of the closing E-step of the last fit (0 if skipped) */
  long long refined_rows;  /* rows (device 0, summed over iterations) whose two best */
                           /* scores were within the fast kernel's error bound and   */
                           /* were re-evaluated exactly                              */
  float ms_transform;      /* CUDA-event time of the kernels of the last kmeans_transform_resident */
  int allreduce_path;      /* per-iteration exchange of the last fit: 0 none (one rank), 1 one-shot push
                            * over peer memory, 2 ncclAllReduce                                   */
} kmeans_stats;
int kmeans_get_stats(kmeans_handle_t h, kmeans_stats* out);
/* Sum of squared distances of every row to its assigned centre (direct
 * differences in double, all ranks): sklearn's inertia_, which the reference's
 * GPU path never sets (src/interface_py/h2o4gpu/solvers/kmeans.py:187). */
int kmeans_inertia(kmeans_handle_t h, double* out);

/* ---- 3. kernel-level entry points (host pointers; used by the parity tests
 * that restate the reference's kernel tests, tests/cpp/gpu/kmeans/*.cu) ------ */
/* un-normalised sums (k x cols, as double) and counts of one labelled shard:
 * the quantity calculate_centroids produces (src/gpu/kmeans/kmeans_centroids.h:40-75) */
int kmeans_centroid_sums_f32(int gpu_id, const float* X, const int32_t* labels, size_t rows,
                             size_t cols, int k, double* sums, int64_t* counts);
int kmeans_centroid_sums_f64(int gpu_id, const double* X, const int32_t* labels, size_t rows,
                             size_t cols, int k, double* sums, int64_t* counts);

/* No counterpart in the reference.  Same result as kmeans_centroid_sums_f32 for a
 * shard that already lives on the current device, for callers that cannot call
 * cudaMalloc where they call it: a serving loop whose device-memory budget is
 * fixed after start-up, or a host that does not accept the implicit device-wide
 * synchronisation of cudaMalloc / cudaFree in the middle of its pipeline.  All
 * working memory is one static device array inside the library (229,440 bytes,
 * held by every GPU that loads the library until the process exits), hence the
 * limit k * cols <= 24576 and k <= 4096; larger sizes return KM_EINVAL.
 * dX (rows x cols row-major), dLabels, dSums (k x cols doubles) and dCounts
 * (k int64) are device pointers; `stream` is a cudaStream_t (NULL = default
 * stream).  The work is enqueued on that stream and the call returns without
 * waiting; it calls no cudaMalloc / cudaFree.  Rows whose label is outside [0, k)
 * are skipped; the data must be finite.  The first call on a device looks up
 * the array's address and raises a shared-memory limit: it should come before
 * any stream capture.  Every call on a device uses the same array, which keeps the
 * previous call's contents until the next call clears them: calls whose GPU
 * work overlaps (other streams) race and must be serialised by the caller. */
int kmeans_centroid_sums_noalloc_f32(const float* dX, const int32_t* dLabels, size_t rows, size_t cols,
                                     int k, double* dSums, long long* dCounts, void* stream);

/* ---- 4. synthetic data on the device (benchmark inputs too large for the host)
 * Fills dX (rows x cols row-major on the current device `gpu_id`) with
 * centers[comp(row)] + sigma * N(0,1); comp drawn from `weights` (NULL = equal).
 * kind 1 instead draws the image-like distribution (0 w.p. 0.8 else 1..255).
 * row0 = global index of the first row, so shards of one matrix are disjoint
 * streams of one counter-based generator. */
int kmeans_synth_f32(int gpu_id, float* dX, size_t rows, size_t cols, size_t row0, int kind,
                     const float* centers_host, int n_comp, const float* weights_host,
                     float sigma, uint64_t seed);
int kmeans_synth_f64(int gpu_id, double* dX, size_t rows, size_t cols, size_t row0, int kind,
                     const double* centers_host, int n_comp, const double* weights_host,
                     double sigma, uint64_t seed);

#ifdef __cplusplus
} /* extern "C" */

/* C++-linkage spellings of the reference's header, forwarded to the above. */
int make_ptr_float_kmeans(int dopredict, int verbose, int seed, int gpu_id, int n_gpu,
                          size_t mTrain, size_t n, int k, int max_iterations, int init_from_data,
                          float threshold, const float* srcdata, const float* centroids,
                          float** pred_centroids, int** pred_labels);
int make_ptr_double_kmeans(int dopredict, int verbose, int seed, int gpu_id, int n_gpu,
                           size_t mTrain, size_t n, int k, int max_iterations,
                           int init_from_data, double threshold, const double* srcdata,
                           const double* centroids, double** pred_centroids, int** pred_labels);
int kmeans_transform_float(int verbose, int gpu_id, int n_gpu, size_t m, size_t n, int k,
                           const float* srcdata, const float* centroids, float** preds);
int kmeans_transform_double(int verbose, int gpu_id, int n_gpu, size_t m, size_t n, int k,
                            const double* srcdata, const double* centroids, double** preds);
#endif

#endif /* H2O4GPU_KMEANS_H_ */
