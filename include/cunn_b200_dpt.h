/*
 * nn.DataParallelTable as a C API (libTHCUNN.so): the reference's batch-sharded data parallelism
 * (DataParallelTable.lua) over the GPUs of one box, with NCCL for the two exchanges it has.
 *
 * The reference keeps one replica of a module per GPU inside one Lua process, scatters the batch,
 * runs the replicas (serially, or on one worker thread per GPU after :threads()), gathers the outputs,
 * reduces the gradients onto GPU 1 and broadcasts GPU 1's parameters (DataParallelTable.lua:182-321).
 * Here a table owns, per replica, the flat parameter vector, a LOCAL gradient vector the module's
 * accGradParameters calls write into, and a VISIBLE gradient vector; backward ends with
 *       visible += allreduce_sum(local);  local = 0
 * on every replica, so all replicas hold the summed gradient and apply the same update (no root fan-in,
 * no broadcast after the first one), and gradients still accumulate correctly over several backward calls
 * between zeroGradParameters (the reference gets that by zeroing the non-root replicas after each reduce,
 * DataParallelTable.lua:258-263).  BN running statistics are per replica and never exchanged, as in the
 * reference.  The all-reduce runs on a communication stream of its own, bucket by bucket: a bucket is
 * enqueued as soon as the caller marks it ready (an event on the compute stream), so the exchange of the
 * last layers' gradients overlaps the backward pass of the first layers.
 *
 * Replicas live either all in this process (cunn_b200_dpt_add: one communicator per GPU from
 * ncclCommInitAll, optional worker thread per GPU) or one per process (cunn_b200_dpt_add_rank:
 * ncclCommInitRank with an id made by cunn_b200_dpt_unique_id on rank 0 and carried to the other ranks by
 * the caller).  NCCL is loaded at run time (libnccl.so.2, or the path in cunn_b200_dpt_nccl_load).
 *
 * Every function returns 0 on success; otherwise cunn_b200_last_error() describes the failure.
 */
#ifndef CUNN_B200_DPT_H
#define CUNN_B200_DPT_H

#include "cunn_b200.h"

#ifdef __cplusplus
extern "C" {
#endif

typedef struct cunn_b200_dpt cunn_b200_dpt;

/* The shard rule, DataParallelTable.lua:469-479 (sliceRange): with n rows and g replicas the first n mod g
 * replicas get floor(n/g)+1 rows, the rest floor(n/g); 0-based start.  Replicas with 0 rows are skipped. */
CUNN_API void cunn_b200_dpt_slice_range(long long n, int g, int i, long long *start, long long *count);

/* Loads NCCL (path == NULL: the CUNN_B200_NCCL_LIB variable, else "libnccl.so.2"). Idempotent. */
CUNN_API int cunn_b200_dpt_nccl_load(const char *path);
/* 128 bytes identifying a new communicator clique (ncclGetUniqueId); rank 0 makes it, every rank passes it on. */
CUNN_API int cunn_b200_dpt_unique_id(void *out128);

/* nn.DataParallelTable(dimension, flattenParams, usenccl), DataParallelTable.lua:44-73.  `dimension` is the
 * 0-based dimension inputs are split along (only 0, the batch, is supported); parameters are always flat
 * and NCCL is always used, so the other two arguments are accepted for interface parity only. */
CUNN_API cunn_b200_dpt *cunn_b200_dpt_create(int dimension, int flatten_params, int use_nccl);
CUNN_API void cunn_b200_dpt_destroy(cunn_b200_dpt *t);

/* :add(module, gpuTable), DataParallelTable.lua:136-159: replicas of a module with `nparams` parameters on the
 * given GPUs of this process.  Allocates params / local grads / visible grads (zeroed) on every GPU. */
CUNN_API int cunn_b200_dpt_add(cunn_b200_dpt *t, const int *gpus, int ngpus, long long nparams);
/* One replica in this process on `device`, rank `rank` of `world` processes that share `unique_id`. */
CUNN_API int cunn_b200_dpt_add_rank(cunn_b200_dpt *t, int device, int rank, int world, const void *unique_id128,
                                    long long nparams);
/* Uses communicators the caller already owns (ncclComm_t handles, one per local replica) instead of creating them. */
CUNN_API int cunn_b200_dpt_adopt_comms(cunn_b200_dpt *t, void *const *comms, int ncomms);

CUNN_API int cunn_b200_dpt_local_replicas(const cunn_b200_dpt *t);     /* replicas in this process */
CUNN_API int cunn_b200_dpt_world(const cunn_b200_dpt *t);              /* replicas in the whole table */
CUNN_API int cunn_b200_dpt_replica_rank(const cunn_b200_dpt *t, int replica);
CUNN_API int cunn_b200_dpt_replica_device(const cunn_b200_dpt *t, int replica);
CUNN_API long long cunn_b200_dpt_param_count(const cunn_b200_dpt *t);
CUNN_API float *cunn_b200_dpt_params(cunn_b200_dpt *t, int replica);          /* flat parameters (getParameters) */
CUNN_API float *cunn_b200_dpt_grads(cunn_b200_dpt *t, int replica);           /* LOCAL gradients: modules accumulate here */
CUNN_API float *cunn_b200_dpt_visible_grads(cunn_b200_dpt *t, int replica);   /* summed over replicas after backward */
/* Makes the replica use the caller's flat buffers (each param_count floats on the replica's GPU, never freed by the
 * table) instead of the ones the table allocated, e.g. buffers a module already owns. */
CUNN_API int cunn_b200_dpt_set_buffers(cunn_b200_dpt *t, int replica, float *params, float *local_grads, float *visible_grads);
CUNN_API cunn_stream_t cunn_b200_dpt_stream(cunn_b200_dpt *t, int replica);   /* the replica's compute stream */
/* Makes the replica compute on the caller's stream instead of the table's own (the table never destroys it). */
CUNN_API int cunn_b200_dpt_set_stream(cunn_b200_dpt *t, int replica, cunn_stream_t stream);

/* :threads(), DataParallelTable.lua:88-93,681-754: one persistent worker thread per local replica. */
CUNN_API int cunn_b200_dpt_threads(cunn_b200_dpt *t);
/* impl:exec(closure), DataParallelTable.lua:653-664 / :724-739: runs fn(ctx, replica, device, stream) for every
 * local replica — on its worker thread if :threads() was called, else one after another with the device set —
 * and returns when all have RETURNED (work they enqueued may still be running).  Non-zero if any fn returned
 * non-zero (the first such value). */
typedef int (*cunn_b200_dpt_fn)(void *ctx, int replica, int device, cunn_stream_t stream);
CUNN_API int cunn_b200_dpt_exec(cunn_b200_dpt *t, cunn_b200_dpt_fn fn, void *ctx);

/* _distribute, DataParallelTable.lua:527-578: copies the rows of `src` (host or device memory, `rows` rows of
 * row_bytes each) that the shard rule gives each LOCAL replica into dst[replica] on that replica's stream;
 * rows_out[replica] receives the count.  In rank mode the table's world and the replica's rank select the shard. */
CUNN_API int cunn_b200_dpt_scatter(cunn_b200_dpt *t, const void *src, long long rows, size_t row_bytes, void *const *dst,
                                   long long *rows_out);
/* _concat, DataParallelTable.lua:583-623: the inverse, local replicas' rows into `dst` (host or device) at their
 * shard offsets.  The caller synchronises the replicas' streams before reading dst. */
CUNN_API int cunn_b200_dpt_gather(cunn_b200_dpt *t, void *const *src, long long rows, size_t row_bytes, void *dst);

/* syncParameters, DataParallelTable.lua:283-294: every replica's parameters := those of rank 0. */
CUNN_API int cunn_b200_dpt_sync_parameters(cunn_b200_dpt *t);
/* zeroGradParameters, DataParallelTable.lua:300-313: zeroes local and visible gradients on all replicas. */
CUNN_API int cunn_b200_dpt_zero_grad_parameters(cunn_b200_dpt *t);
/* updateParameters(lr), DataParallelTable.lua:315-321: params -= lr * visible grads, on every replica. */
CUNN_API int cunn_b200_dpt_update_parameters(cunn_b200_dpt *t, float lr);

/* Gradient buckets.  ends[b] is the END offset (in floats) of bucket b in the flat gradient; buckets are listed in
 * the order they become ready during backward, i.e. from the LAST layers to the first: bucket b covers
 * [ends[b+1], ends[b]) with ends[nbuckets] taken as 0 and ends[0] == nparams.  Default: one bucket. */
CUNN_API int cunn_b200_dpt_set_buckets(cunn_b200_dpt *t, const long long *ends, int nbuckets);
/* The kernels that produce bucket `bucket` of `replica`'s local gradient are enqueued on its compute stream:
 * records an event there and enqueues the bucket's all-reduce on the replica's communication stream behind it.
 * In one-process mode the collective is enqueued once all local replicas have marked the bucket. */
CUNN_API int cunn_b200_dpt_bucket_ready(cunn_b200_dpt *t, int replica, int bucket);
/* End of backward, DataParallelTable.lua:247-265: all-reduces the buckets not yet marked, then on every replica
 * visible += local, local = 0, and the compute stream waits for the communication stream. */
CUNN_API int cunn_b200_dpt_reduce(cunn_b200_dpt *t);

/* Watchdog: polls ncclCommGetAsyncError on every communicator until the communication streams have drained or
 * timeout_seconds pass.  On an asynchronous error or on timeout it aborts the communicators (ncclCommAbort),
 * marks the table failed (later collectives return an error) and returns non-zero. */
CUNN_API int cunn_b200_dpt_watchdog(cunn_b200_dpt *t, double timeout_seconds);

/* Serialisation, DataParallelTable.lua:355-448 (__write / __read): the GPU assignment first, then replica 0's flat
 * parameters and an opaque `extra` blob (e.g. replica 0's BN running statistics); gradients and scratch are not
 * stored.  cunn_b200_dpt_file_* work on host arrays; cunn_b200_dpt_write stores a live table and
 * cunn_b200_dpt_read_params loads a file's parameters into every replica of a table of the same parameter count.
 * `ngpus_wanted` is the reference's deserializeNGPUs (:357-393): 0 keeps the stored assignment, which must then
 * fit this machine; n > 0 re-assigns the replicas to GPUs 0..n-1. */
CUNN_API int cunn_b200_dpt_file_write(const char *path, const int *gpus, int ngpus, const float *params, long long nparams,
                                      const void *extra, long long extra_bytes);
CUNN_API int cunn_b200_dpt_file_info(const char *path, int *ngpus, long long *nparams, long long *extra_bytes);
CUNN_API int cunn_b200_dpt_file_read(const char *path, int ngpus_wanted, int gpus_available, int *gpus, float *params,
                                     void *extra);
CUNN_API int cunn_b200_dpt_write(cunn_b200_dpt *t, const char *path, const void *extra, long long extra_bytes);
CUNN_API int cunn_b200_dpt_read_params(cunn_b200_dpt *t, const char *path, void *extra);

#ifdef __cplusplus
}
#endif
#endif /* CUNN_B200_DPT_H */
