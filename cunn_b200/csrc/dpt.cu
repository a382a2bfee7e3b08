// nn.DataParallelTable as a C API: replicas over the GPUs of one box, NCCL for the gradient sum and the parameter
// broadcast, buckets released by events so that the exchange overlaps the backward pass.  See
// include/cunn_b200_dpt.h for the interface and the reference lines each call mirrors.
#include "common.cuh"
#include "../../include/cunn_b200_dpt.h"

#include <dlfcn.h>
#include <nccl.h>      // types and prototypes only: the library is loaded at run time
#include <stdlib.h>
#include <string.h>

#include <algorithm>
#include <atomic>
#include <chrono>
#include <condition_variable>
#include <functional>
#include <mutex>
#include <string>
#include <thread>
#include <vector>

namespace cunn {
namespace dpt {

// ---- NCCL, loaded at run time ---------------------------------------------------------------------------------
// The process may already hold a libnccl of its own (a Python host with torch does); dlopen by soname then returns
// that copy, so two NCCLs never meet in one process.
struct Nccl {
    void *handle = nullptr;
    decltype(&ncclGetUniqueId) GetUniqueId = nullptr;
    decltype(&ncclCommInitRank) CommInitRank = nullptr;
    decltype(&ncclCommInitAll) CommInitAll = nullptr;
    decltype(&ncclCommDestroy) CommDestroy = nullptr;
    decltype(&ncclCommAbort) CommAbort = nullptr;
    decltype(&ncclCommGetAsyncError) CommGetAsyncError = nullptr;
    decltype(&ncclAllReduce) AllReduce = nullptr;
    decltype(&ncclBroadcast) Broadcast = nullptr;
    decltype(&ncclGroupStart) GroupStart = nullptr;
    decltype(&ncclGroupEnd) GroupEnd = nullptr;
    decltype(&ncclGetErrorString) GetErrorString = nullptr;
};
static Nccl g_nccl;
static std::mutex g_nccl_mutex;

static int nccl_load(const char *path)
{
    std::lock_guard<std::mutex> lock(g_nccl_mutex);
    if (g_nccl.handle && !path) return 0;
    const char *env = getenv("CUNN_B200_NCCL_LIB");
    const char *name = path ? path : (env && *env ? env : "libnccl.so.2");
    void *h = dlopen(name, RTLD_NOW | RTLD_LOCAL);
    if (!h) return fail("cannot load NCCL (%s): %s", name, dlerror());
    Nccl n;
    n.handle = h;
#define CUNN_NCCL_SYM(field, symbol)                                                 \
    n.field = (decltype(n.field))dlsym(h, symbol);                                   \
    if (!n.field) return fail("%s has no symbol %s", name, symbol);
    CUNN_NCCL_SYM(GetUniqueId, "ncclGetUniqueId")
    CUNN_NCCL_SYM(CommInitRank, "ncclCommInitRank")
    CUNN_NCCL_SYM(CommInitAll, "ncclCommInitAll")
    CUNN_NCCL_SYM(CommDestroy, "ncclCommDestroy")
    CUNN_NCCL_SYM(CommAbort, "ncclCommAbort")
    CUNN_NCCL_SYM(CommGetAsyncError, "ncclCommGetAsyncError")
    CUNN_NCCL_SYM(AllReduce, "ncclAllReduce")
    CUNN_NCCL_SYM(Broadcast, "ncclBroadcast")
    CUNN_NCCL_SYM(GroupStart, "ncclGroupStart")
    CUNN_NCCL_SYM(GroupEnd, "ncclGroupEnd")
    CUNN_NCCL_SYM(GetErrorString, "ncclGetErrorString")
#undef CUNN_NCCL_SYM
    g_nccl = n;
    return 0;
}

#define CUNN_NCCL(call)                                                                                        \
    do {                                                                                                       \
        ncclResult_t r_ = (call);                                                                              \
        if (r_ != ncclSuccess) return cunn::fail("%s failed: %s", #call, g_nccl.GetErrorString(r_));           \
    } while (0)

// ---- kernels ---------------------------------------------------------------------------------------------------
// visible += local; local = 0   (the tail of backward)
__global__ void __launch_bounds__(256)
fold_grads_kernel(float *__restrict__ visible, float *__restrict__ local, long long n)
{
    const long long n4 = n / 4;
    float4 *v4 = reinterpret_cast<float4 *>(visible), *l4 = reinterpret_cast<float4 *>(local);
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n4; i += (long long)gridDim.x * blockDim.x) {
        float4 a = v4[i];
        const float4 b = l4[i];
        a.x += b.x; a.y += b.y; a.z += b.z; a.w += b.w;
        v4[i] = a;
        l4[i] = make_float4(0.f, 0.f, 0.f, 0.f);
    }
    for (long long i = n4 * 4 + blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
        visible[i] += local[i];
        local[i] = 0.f;
    }
}

// params -= lr * grads
__global__ void __launch_bounds__(256)
sgd_kernel(float *__restrict__ p, const float *__restrict__ g, long long n, float lr)
{
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
        p[i] = fmaf(-lr, g[i], p[i]);
}

static int grid_for(long long n)
{
    return (int)std::max(1LL, std::min(ceil_div_ll(std::max(n / 4, 1LL), 256), (long long)sm_count() * 8));
}

// ---- file format ---------------------------------------------------------------------------------------------------
// [magic "CUNNDPT1"][int32 ngpus][int32 gpus[ngpus]][int64 nparams][int64 extra_bytes][float params[nparams]][extra]
static const char kMagic[8] = {'C', 'U', 'N', 'N', 'D', 'P', 'T', '1'};

struct FileHeader {
    int ngpus = 0;
    std::vector<int> gpus;
    long long nparams = 0, extra_bytes = 0;
};

static int read_header(FILE *f, const char *path, FileHeader &h)
{
    char magic[8];
    if (fread(magic, 1, 8, f) != 8 || memcmp(magic, kMagic, 8) != 0) return fail("%s is not a DataParallelTable file", path);
    int32_t n = 0;
    if (fread(&n, 4, 1, f) != 1 || n < 1 || n > 1024) return fail("%s: bad GPU count", path);
    h.ngpus = n;
    h.gpus.resize(n);
    for (int i = 0; i < n; ++i) {
        int32_t g = 0;
        if (fread(&g, 4, 1, f) != 1) return fail("%s: truncated GPU assignment", path);
        h.gpus[i] = g;
    }
    int64_t np = 0, eb = 0;
    if (fread(&np, 8, 1, f) != 1 || fread(&eb, 8, 1, f) != 1 || np < 0 || eb < 0) return fail("%s: truncated header", path);
    h.nparams = np;
    h.extra_bytes = eb;
    return 0;
}

}  // namespace dpt
}  // namespace cunn

using namespace cunn;
using namespace cunn::dpt;

extern "C" CUNN_API void cunn_b200_dpt_slice_range(long long n, int g, int i, long long *start, long long *count)
{
    const long long per = g > 0 ? n / g : 0, extra = g > 0 ? n % g : 0;
    *start = (long long)i * per + std::min<long long>(i, extra);
    *count = per + (i < extra ? 1 : 0);
}

extern "C" CUNN_API int cunn_b200_dpt_nccl_load(const char *path)
{
    clear_error();
    return nccl_load(path);
}

extern "C" CUNN_API int cunn_b200_dpt_unique_id(void *out128)
{
    clear_error();
    if (nccl_load(nullptr)) return 1;
    static_assert(sizeof(ncclUniqueId) == 128, "ncclUniqueId is 128 bytes");
    ncclUniqueId id;
    CUNN_NCCL(g_nccl.GetUniqueId(&id));
    memcpy(out128, &id, sizeof(id));
    return 0;
}

extern "C" CUNN_API int cunn_b200_dpt_file_write(const char *path, const int *gpus, int ngpus, const float *params, long long nparams,
                                                 const void *extra, long long extra_bytes)
{
    clear_error();
    CUNN_CHECK_ARG(path && gpus && ngpus >= 1 && nparams >= 0 && extra_bytes >= 0 && (params || nparams == 0) && (extra || extra_bytes == 0),
                   "bad arguments to the DataParallelTable writer");
    FILE *f = fopen(path, "wb");
    CUNN_CHECK_ARG(f, "cannot open %s for writing", path);
    bool ok = fwrite(kMagic, 1, 8, f) == 8;
    const int32_t n = ngpus;
    ok = ok && fwrite(&n, 4, 1, f) == 1;
    for (int i = 0; ok && i < ngpus; ++i) {
        const int32_t g = gpus[i];
        ok = fwrite(&g, 4, 1, f) == 1;
    }
    const int64_t np = nparams, eb = extra_bytes;
    ok = ok && fwrite(&np, 8, 1, f) == 1 && fwrite(&eb, 8, 1, f) == 1;
    ok = ok && (nparams == 0 || fwrite(params, sizeof(float), (size_t)nparams, f) == (size_t)nparams);
    ok = ok && (extra_bytes == 0 || fwrite(extra, 1, (size_t)extra_bytes, f) == (size_t)extra_bytes);
    ok = (fclose(f) == 0) && ok;
    CUNN_CHECK_ARG(ok, "short write to %s", path);
    return 0;
}

extern "C" CUNN_API int cunn_b200_dpt_file_info(const char *path, int *ngpus, long long *nparams, long long *extra_bytes)
{
    clear_error();
    FILE *f = fopen(path, "rb");
    CUNN_CHECK_ARG(f, "cannot open %s", path);
    FileHeader h;
    const int rc = read_header(f, path, h);
    fclose(f);
    if (rc) return rc;
    if (ngpus) *ngpus = h.ngpus;
    if (nparams) *nparams = h.nparams;
    if (extra_bytes) *extra_bytes = h.extra_bytes;
    return 0;
}

// The GPU assignment follows the reference's __read (DataParallelTable.lua:373-393): with deserializeNGPUs set the
// replicas are re-assigned to GPUs 0 .. n-1; otherwise the stored assignment is kept and must fit this machine.
extern "C" CUNN_API int cunn_b200_dpt_file_read(const char *path, int ngpus_wanted, int gpus_available, int *gpus, float *params,
                                                void *extra)
{
    clear_error();
    FILE *f = fopen(path, "rb");
    CUNN_CHECK_ARG(f, "cannot open %s", path);
    FileHeader h;
    if (read_header(f, path, h)) { fclose(f); return 1; }
    bool ok = true;
    if (params) ok = h.nparams == 0 || fread(params, sizeof(float), (size_t)h.nparams, f) == (size_t)h.nparams;
    else ok = fseek(f, (long)(h.nparams * (long long)sizeof(float)), SEEK_CUR) == 0;
    if (ok && extra && h.extra_bytes) ok = fread(extra, 1, (size_t)h.extra_bytes, f) == (size_t)h.extra_bytes;
    fclose(f);
    CUNN_CHECK_ARG(ok, "%s is truncated", path);
    if (ngpus_wanted > 0) {
        CUNN_CHECK_ARG(gpus_available <= 0 || ngpus_wanted <= gpus_available, "Asked for %d GPUs but only %d are available", ngpus_wanted,
                       gpus_available);
        if (gpus)
            for (int i = 0; i < ngpus_wanted; ++i) gpus[i] = i;
        return 0;
    }
    for (int i = 0; i < h.ngpus; ++i) {
        CUNN_CHECK_ARG(gpus_available <= 0 || h.gpus[i] < gpus_available,
                       "Model was saved with GPU %d but only %d GPUs are available; pass the number of GPUs to use instead", h.gpus[i],
                       gpus_available);
        if (gpus) gpus[i] = h.gpus[i];
    }
    return 0;
}

// ---- the table -------------------------------------------------------------------------------------------------------
namespace cunn {
namespace dpt {

struct Worker {
    std::thread th;
    std::mutex m;
    std::condition_variable cv;
    std::function<int()> job;
    bool has_job = false, done = false, quit = false;
    int result = 0;
};

struct Replica {
    int device = -1, rank = 0;
    float *params = nullptr, *local = nullptr, *visible = nullptr;
    bool own_buffers = true;
    cudaStream_t compute = nullptr, comm_stream = nullptr;
    bool own_compute = false;
    ncclComm_t comm = nullptr;
    bool own_comm = false;
    cudaEvent_t comm_done = nullptr;
    std::vector<cudaEvent_t> bucket_ev;      // one per bucket: "the bucket's gradients are enqueued"
    std::vector<char> marked;                // bucket marked ready during this backward
    Worker *worker = nullptr;
};

}  // namespace dpt
}  // namespace cunn

struct cunn_b200_dpt {
    int dimension = 0;
    long long nparams = 0;
    int world = 0;
    bool rank_mode = false, failed = false;
    std::vector<cunn::dpt::Replica> reps;
    std::vector<long long> ends{};           // bucket end offsets, last layers first; empty = one bucket
    std::vector<int> marks;                  // local replicas that marked bucket b
    std::vector<char> issued;                // bucket b's all-reduce is enqueued
    std::mutex m;
};

namespace cunn {
namespace dpt {

struct DeviceGuard {
    int prev = -1;
    explicit DeviceGuard(int dev) { cudaGetDevice(&prev); if (dev >= 0 && dev != prev) cudaSetDevice(dev); }
    ~DeviceGuard() { if (prev >= 0) cudaSetDevice(prev); }
};

static int nbuckets(const cunn_b200_dpt *t) { return t->ends.empty() ? 1 : (int)t->ends.size(); }
static void bucket_range(const cunn_b200_dpt *t, int b, long long *lo, long long *hi)
{
    if (t->ends.empty()) { *lo = 0; *hi = t->nparams; return; }
    *hi = t->ends[b];
    *lo = b + 1 < (int)t->ends.size() ? t->ends[b + 1] : 0;
}

static int alloc_replica(cunn_b200_dpt *t, Replica &r)
{
    DeviceGuard g(r.device);
    const size_t bytes = (size_t)std::max<long long>(t->nparams, 1) * sizeof(float);
    CUNN_CUDA(cudaMalloc(&r.params, bytes));
    CUNN_CUDA(cudaMalloc(&r.local, bytes));
    CUNN_CUDA(cudaMalloc(&r.visible, bytes));
    CUNN_CUDA(cudaMemset(r.params, 0, bytes));
    CUNN_CUDA(cudaMemset(r.local, 0, bytes));
    CUNN_CUDA(cudaMemset(r.visible, 0, bytes));
    CUNN_CUDA(cudaStreamCreateWithFlags(&r.compute, cudaStreamNonBlocking));
    r.own_compute = true;
    CUNN_CUDA(cudaStreamCreateWithFlags(&r.comm_stream, cudaStreamNonBlocking));
    CUNN_CUDA(cudaEventCreateWithFlags(&r.comm_done, cudaEventDisableTiming));
    return 0;
}

static int make_bucket_events(cunn_b200_dpt *t)
{
    const int nb = nbuckets(t);
    for (Replica &r : t->reps) {
        if (r.device < 0) continue;
        DeviceGuard g(r.device);
        for (cudaEvent_t e : r.bucket_ev) cudaEventDestroy(e);
        r.bucket_ev.assign(nb, nullptr);
        for (int b = 0; b < nb; ++b) CUNN_CUDA(cudaEventCreateWithFlags(&r.bucket_ev[b], cudaEventDisableTiming));
        r.marked.assign(nb, 0);
    }
    t->marks.assign(nb, 0);
    t->issued.assign(nb, 0);
    return 0;
}

// Enqueues bucket b's all-reduce on every local replica's communication stream, behind the bucket's events.
static int issue_bucket(cunn_b200_dpt *t, int b)
{
    t->issued[b] = 1;
    if (t->world <= 1) return 0;
    CUNN_CHECK_ARG(!t->failed, "the table's communicators were aborted");
    long long lo, hi;
    bucket_range(t, b, &lo, &hi);
    if (hi <= lo) return 0;
    for (Replica &r : t->reps) {
        DeviceGuard g(r.device);
        CUNN_CUDA(cudaStreamWaitEvent(r.comm_stream, r.bucket_ev[b], 0));
    }
    CUNN_NCCL(g_nccl.GroupStart());
    for (Replica &r : t->reps) {
        DeviceGuard g(r.device);
        const ncclResult_t res = g_nccl.AllReduce(r.local + lo, r.local + lo, (size_t)(hi - lo), ncclFloat, ncclSum, r.comm, r.comm_stream);
        if (res != ncclSuccess) {
            g_nccl.GroupEnd();
            return fail("ncclAllReduce failed: %s", g_nccl.GetErrorString(res));
        }
    }
    CUNN_NCCL(g_nccl.GroupEnd());
    return 0;
}

static void worker_loop(Worker *w, int device)
{
    if (device >= 0) cudaSetDevice(device);
    std::unique_lock<std::mutex> lock(w->m);
    for (;;) {
        w->cv.wait(lock, [w] { return w->has_job || w->quit; });
        if (w->quit) return;
        std::function<int()> job = std::move(w->job);
        w->has_job = false;
        lock.unlock();
        const int rc = job();
        lock.lock();
        w->result = rc;
        w->done = true;
        w->cv.notify_all();
    }
}

static void abort_comms(cunn_b200_dpt *t)
{
    for (Replica &r : t->reps)
        if (r.comm && g_nccl.CommAbort) {
            g_nccl.CommAbort(r.comm);
            r.comm = nullptr;
        }
    t->failed = true;
}

}  // namespace dpt
}  // namespace cunn

extern "C" CUNN_API cunn_b200_dpt *cunn_b200_dpt_create(int dimension, int, int)
{
    clear_error();
    if (dimension != 0) {
        fail("only the batch dimension (0) can be split, got %d", dimension);
        return nullptr;
    }
    return new cunn_b200_dpt();
}

extern "C" CUNN_API void cunn_b200_dpt_destroy(cunn_b200_dpt *t)
{
    if (!t) return;
    for (Replica &r : t->reps) {
        if (r.worker) {
            {
                std::lock_guard<std::mutex> lock(r.worker->m);
                r.worker->quit = true;
            }
            r.worker->cv.notify_all();
            r.worker->th.join();
            delete r.worker;
        }
        if (r.device < 0) continue;
        DeviceGuard g(r.device);
        if (r.comm_stream) cudaStreamSynchronize(r.comm_stream);
        if (r.compute) cudaStreamSynchronize(r.compute);
        if (r.comm && r.own_comm && g_nccl.CommDestroy) g_nccl.CommDestroy(r.comm);
        for (cudaEvent_t e : r.bucket_ev) cudaEventDestroy(e);
        if (r.comm_done) cudaEventDestroy(r.comm_done);
        if (r.comm_stream) cudaStreamDestroy(r.comm_stream);
        if (r.compute && r.own_compute) cudaStreamDestroy(r.compute);
        if (r.own_buffers) {
            cudaFree(r.params);
            cudaFree(r.local);
            cudaFree(r.visible);
        }
    }
    delete t;
}

extern "C" CUNN_API int cunn_b200_dpt_add(cunn_b200_dpt *t, const int *gpus, int ngpus, long long nparams)
{
    clear_error();
    CUNN_CHECK_ARG(t && gpus && ngpus >= 1 && nparams >= 0, "bad arguments");
    CUNN_CHECK_ARG(t->reps.empty(), "the table already holds a module");
    int ndev = 0;
    CUNN_CUDA(cudaGetDeviceCount(&ndev));
    for (int i = 0; i < ngpus; ++i) CUNN_CHECK_ARG(gpus[i] >= 0 && gpus[i] < ndev, "GPU %d is not available (%d devices)", gpus[i], ndev);
    t->nparams = nparams;
    t->world = ngpus;
    t->rank_mode = false;
    t->reps.resize(ngpus);
    for (int i = 0; i < ngpus; ++i) {
        t->reps[i].device = gpus[i];
        t->reps[i].rank = i;
        if (alloc_replica(t, t->reps[i])) return 1;
    }
    if (ngpus > 1) {
        if (nccl_load(nullptr)) return 1;
        std::vector<ncclComm_t> comms(ngpus);
        CUNN_NCCL(g_nccl.CommInitAll(comms.data(), ngpus, gpus));
        for (int i = 0; i < ngpus; ++i) { t->reps[i].comm = comms[i]; t->reps[i].own_comm = true; }
    }
    return make_bucket_events(t);
}

extern "C" CUNN_API int cunn_b200_dpt_add_rank(cunn_b200_dpt *t, int device, int rank, int world, const void *unique_id128, long long nparams)
{
    clear_error();
    CUNN_CHECK_ARG(t && world >= 1 && rank >= 0 && rank < world && nparams >= 0, "bad arguments");
    CUNN_CHECK_ARG(t->reps.empty(), "the table already holds a module");
    t->nparams = nparams;
    t->world = world;
    t->rank_mode = true;
    t->reps.resize(1);
    t->reps[0].device = device;
    t->reps[0].rank = rank;
    if (alloc_replica(t, t->reps[0])) return 1;
    if (world > 1) {
        CUNN_CHECK_ARG(unique_id128, "a unique id is needed for more than one rank");
        if (nccl_load(nullptr)) return 1;
        ncclUniqueId id;
        memcpy(&id, unique_id128, sizeof(id));
        DeviceGuard g(device);
        CUNN_NCCL(g_nccl.CommInitRank(&t->reps[0].comm, world, id, rank));
        t->reps[0].own_comm = true;
    }
    return make_bucket_events(t);
}

extern "C" CUNN_API int cunn_b200_dpt_adopt_comms(cunn_b200_dpt *t, void *const *comms, int ncomms)
{
    clear_error();
    CUNN_CHECK_ARG(t && comms && ncomms >= 1, "bad arguments");
    if (nccl_load(nullptr)) return 1;
    if (t->reps.empty()) {               // communicators only: a table whose watchdog can be driven without replicas
        t->reps.resize(ncomms);
        t->world = std::max(t->world, ncomms);
    }
    CUNN_CHECK_ARG((int)t->reps.size() == ncomms, "%d communicators for %d local replicas", ncomms, (int)t->reps.size());
    for (int i = 0; i < ncomms; ++i) {
        Replica &r = t->reps[i];
        if (r.comm && r.own_comm) g_nccl.CommDestroy(r.comm);
        r.comm = (ncclComm_t)comms[i];
        r.own_comm = false;
    }
    t->failed = false;
    return 0;
}

extern "C" CUNN_API int cunn_b200_dpt_local_replicas(const cunn_b200_dpt *t) { return t ? (int)t->reps.size() : 0; }
extern "C" CUNN_API int cunn_b200_dpt_world(const cunn_b200_dpt *t) { return t ? t->world : 0; }
extern "C" CUNN_API int cunn_b200_dpt_replica_rank(const cunn_b200_dpt *t, int i) { return t->reps[i].rank; }
extern "C" CUNN_API int cunn_b200_dpt_replica_device(const cunn_b200_dpt *t, int i) { return t->reps[i].device; }
extern "C" CUNN_API long long cunn_b200_dpt_param_count(const cunn_b200_dpt *t) { return t->nparams; }
extern "C" CUNN_API float *cunn_b200_dpt_params(cunn_b200_dpt *t, int i) { return t->reps[i].params; }
extern "C" CUNN_API float *cunn_b200_dpt_grads(cunn_b200_dpt *t, int i) { return t->reps[i].local; }
extern "C" CUNN_API float *cunn_b200_dpt_visible_grads(cunn_b200_dpt *t, int i) { return t->reps[i].visible; }
extern "C" CUNN_API cunn_stream_t cunn_b200_dpt_stream(cunn_b200_dpt *t, int i) { return (cunn_stream_t)t->reps[i].compute; }

extern "C" CUNN_API int cunn_b200_dpt_set_stream(cunn_b200_dpt *t, int i, cunn_stream_t stream)
{
    clear_error();
    CUNN_CHECK_ARG(t && i >= 0 && i < (int)t->reps.size(), "bad replica index");
    Replica &r = t->reps[i];
    if (r.compute && r.own_compute) {
        DeviceGuard g(r.device);
        cudaStreamSynchronize(r.compute);
        cudaStreamDestroy(r.compute);
    }
    r.compute = (cudaStream_t)stream;
    r.own_compute = false;
    return 0;
}

extern "C" CUNN_API int cunn_b200_dpt_set_buffers(cunn_b200_dpt *t, int i, float *params, float *local_grads, float *visible_grads)
{
    clear_error();
    CUNN_CHECK_ARG(t && i >= 0 && i < (int)t->reps.size() && params && local_grads && visible_grads, "bad arguments");
    Replica &r = t->reps[i];
    if (r.own_buffers) {
        DeviceGuard g(r.device);
        cudaStreamSynchronize(r.compute);
        cudaFree(r.params);
        cudaFree(r.local);
        cudaFree(r.visible);
    }
    r.params = params; r.local = local_grads; r.visible = visible_grads;
    r.own_buffers = false;
    return 0;
}

extern "C" CUNN_API int cunn_b200_dpt_threads(cunn_b200_dpt *t)
{
    clear_error();
    CUNN_CHECK_ARG(t && !t->reps.empty(), "add a module before :threads()");
    for (Replica &r : t->reps) {
        if (r.worker) continue;
        r.worker = new Worker();
        r.worker->th = std::thread(worker_loop, r.worker, r.device);
    }
    return 0;
}

extern "C" CUNN_API int cunn_b200_dpt_exec(cunn_b200_dpt *t, cunn_b200_dpt_fn fn, void *ctx)
{
    clear_error();
    CUNN_CHECK_ARG(t && fn, "bad arguments");
    int first = 0;
    const int n = (int)t->reps.size();
    if (n > 0 && t->reps[0].worker) {
        for (int i = 0; i < n; ++i) {
            Replica &r = t->reps[i];
            std::lock_guard<std::mutex> lock(r.worker->m);
            r.worker->job = [fn, ctx, i, &r]() { return fn(ctx, i, r.device, (cunn_stream_t)r.compute); };
            r.worker->has_job = true;
            r.worker->done = false;
            r.worker->cv.notify_all();
        }
        for (int i = 0; i < n; ++i) {
            Worker *w = t->reps[i].worker;
            std::unique_lock<std::mutex> lock(w->m);
            w->cv.wait(lock, [w] { return w->done; });
            if (w->result && !first) first = w->result;
        }
    } else {
        for (int i = 0; i < n; ++i) {
            Replica &r = t->reps[i];
            DeviceGuard g(r.device);
            const int rc = fn(ctx, i, r.device, (cunn_stream_t)r.compute);
            if (rc && !first) first = rc;
        }
    }
    if (first) return fail("a replica's function returned %d", first);
    return 0;
}

extern "C" CUNN_API int cunn_b200_dpt_scatter(cunn_b200_dpt *t, const void *src, long long rows, size_t row_bytes, void *const *dst,
                                              long long *rows_out)
{
    clear_error();
    CUNN_CHECK_ARG(t && dst && rows >= 0 && (src || rows == 0), "bad arguments");
    for (size_t i = 0; i < t->reps.size(); ++i) {
        Replica &r = t->reps[i];
        long long start, count;
        cunn_b200_dpt_slice_range(rows, t->world, r.rank, &start, &count);
        if (rows_out) rows_out[i] = count;
        if (count == 0) continue;                               // batches smaller than the GPU count use fewer replicas
        CUNN_CHECK_ARG(dst[i], "no destination for replica %zu", i);
        DeviceGuard g(r.device);
        CUNN_CUDA(cudaMemcpyAsync(dst[i], (const char *)src + (size_t)start * row_bytes, (size_t)count * row_bytes, cudaMemcpyDefault, r.compute));
    }
    return 0;
}

extern "C" CUNN_API int cunn_b200_dpt_gather(cunn_b200_dpt *t, void *const *src, long long rows, size_t row_bytes, void *dst)
{
    clear_error();
    CUNN_CHECK_ARG(t && src && rows >= 0 && (dst || rows == 0), "bad arguments");
    for (size_t i = 0; i < t->reps.size(); ++i) {
        Replica &r = t->reps[i];
        long long start, count;
        cunn_b200_dpt_slice_range(rows, t->world, r.rank, &start, &count);
        if (count == 0) continue;
        CUNN_CHECK_ARG(src[i], "no source for replica %zu", i);
        DeviceGuard g(r.device);
        CUNN_CUDA(cudaMemcpyAsync((char *)dst + (size_t)start * row_bytes, src[i], (size_t)count * row_bytes, cudaMemcpyDefault, r.compute));
    }
    return 0;
}

extern "C" CUNN_API int cunn_b200_dpt_sync_parameters(cunn_b200_dpt *t)
{
    clear_error();
    CUNN_CHECK_ARG(t && !t->reps.empty(), "empty table");
    if (t->world <= 1 || t->nparams == 0) return 0;
    CUNN_CHECK_ARG(!t->failed, "the table's communicators were aborted");
    CUNN_NCCL(g_nccl.GroupStart());
    for (Replica &r : t->reps) {
        DeviceGuard g(r.device);
        const ncclResult_t res = g_nccl.Broadcast(r.params, r.params, (size_t)t->nparams, ncclFloat, 0, r.comm, r.compute);
        if (res != ncclSuccess) {
            g_nccl.GroupEnd();
            return fail("ncclBroadcast failed: %s", g_nccl.GetErrorString(res));
        }
    }
    CUNN_NCCL(g_nccl.GroupEnd());
    return 0;
}

extern "C" CUNN_API int cunn_b200_dpt_zero_grad_parameters(cunn_b200_dpt *t)
{
    clear_error();
    CUNN_CHECK_ARG(t, "null table");
    for (Replica &r : t->reps) {
        DeviceGuard g(r.device);
        CUNN_CUDA(cudaMemsetAsync(r.local, 0, (size_t)t->nparams * sizeof(float), r.compute));
        CUNN_CUDA(cudaMemsetAsync(r.visible, 0, (size_t)t->nparams * sizeof(float), r.compute));
    }
    return 0;
}

extern "C" CUNN_API int cunn_b200_dpt_update_parameters(cunn_b200_dpt *t, float lr)
{
    clear_error();
    CUNN_CHECK_ARG(t, "null table");
    if (t->nparams == 0) return 0;
    for (Replica &r : t->reps) {
        DeviceGuard g(r.device);
        sgd_kernel<<<grid_for(t->nparams * 4), 256, 0, r.compute>>>(r.params, r.visible, t->nparams, lr);
        CUNN_LAUNCH_CHECK("parameter update");
    }
    return 0;
}

extern "C" CUNN_API int cunn_b200_dpt_set_buckets(cunn_b200_dpt *t, const long long *ends, int n)
{
    clear_error();
    CUNN_CHECK_ARG(t && ends && n >= 1, "bad arguments");
    CUNN_CHECK_ARG(ends[0] == t->nparams, "the first bucket must end at the parameter count (%lld), got %lld", t->nparams, ends[0]);
    for (int b = 1; b < n; ++b) CUNN_CHECK_ARG(ends[b] <= ends[b - 1] && ends[b] >= 0, "bucket ends must not increase");
    std::lock_guard<std::mutex> lock(t->m);
    t->ends.assign(ends, ends + n);
    return make_bucket_events(t);
}

extern "C" CUNN_API int cunn_b200_dpt_bucket_ready(cunn_b200_dpt *t, int replica, int bucket)
{
    clear_error();
    CUNN_CHECK_ARG(t && replica >= 0 && replica < (int)t->reps.size() && bucket >= 0 && bucket < nbuckets(t), "bad replica or bucket index");
    std::lock_guard<std::mutex> lock(t->m);
    Replica &r = t->reps[replica];
    CUNN_CHECK_ARG(!r.marked[bucket], "bucket %d of replica %d was already marked ready in this backward pass", bucket, replica);
    {
        DeviceGuard g(r.device);
        CUNN_CUDA(cudaEventRecord(r.bucket_ev[bucket], r.compute));
    }
    r.marked[bucket] = 1;
    if (++t->marks[bucket] == (int)t->reps.size()) return issue_bucket(t, bucket);
    return 0;
}

extern "C" CUNN_API int cunn_b200_dpt_reduce(cunn_b200_dpt *t)
{
    clear_error();
    CUNN_CHECK_ARG(t && !t->reps.empty(), "empty table");
    std::lock_guard<std::mutex> lock(t->m);
    const int nb = nbuckets(t);
    for (int b = 0; b < nb; ++b) {
        if (t->issued[b]) continue;
        for (Replica &r : t->reps)
            if (!r.marked[b]) {
                DeviceGuard g(r.device);
                CUNN_CUDA(cudaEventRecord(r.bucket_ev[b], r.compute));
                r.marked[b] = 1;
            }
        if (issue_bucket(t, b)) return 1;
    }
    for (Replica &r : t->reps) {
        DeviceGuard g(r.device);
        if (t->world > 1) {
            CUNN_CUDA(cudaEventRecord(r.comm_done, r.comm_stream));
            CUNN_CUDA(cudaStreamWaitEvent(r.compute, r.comm_done, 0));
        }
        if (t->nparams > 0) {
            fold_grads_kernel<<<grid_for(t->nparams), 256, 0, r.compute>>>(r.visible, r.local, t->nparams);
            CUNN_LAUNCH_CHECK("gradient fold");
        }
        std::fill(r.marked.begin(), r.marked.end(), 0);
    }
    std::fill(t->marks.begin(), t->marks.end(), 0);
    std::fill(t->issued.begin(), t->issued.end(), 0);
    return 0;
}

extern "C" CUNN_API int cunn_b200_dpt_watchdog(cunn_b200_dpt *t, double timeout_seconds)
{
    clear_error();
    CUNN_CHECK_ARG(t, "null table");
    if (t->failed) return fail("the table's communicators were aborted");
    const auto t0 = std::chrono::steady_clock::now();
    for (;;) {
        bool idle = true;
        for (Replica &r : t->reps) {
            if (r.comm) {
                ncclResult_t async = ncclSuccess;
                const ncclResult_t res = g_nccl.CommGetAsyncError(r.comm, &async);
                if (res != ncclSuccess || (async != ncclSuccess && async != ncclInProgress)) {
                    const ncclResult_t bad = res != ncclSuccess ? res : async;
                    std::string msg = g_nccl.GetErrorString(bad);
                    abort_comms(t);
                    return fail("NCCL reported an asynchronous error on rank %d (%s); communicators aborted", r.rank, msg.c_str());
                }
                if (async == ncclInProgress) idle = false;
            }
            if (r.comm_stream) {
                DeviceGuard g(r.device);
                const cudaError_t q = cudaStreamQuery(r.comm_stream);
                if (q == cudaErrorNotReady) idle = false;
                else if (q != cudaSuccess) {
                    abort_comms(t);
                    return fail("communication stream of rank %d failed: %s; communicators aborted", r.rank, cudaGetErrorString(q));
                }
            }
        }
        if (idle) return 0;
        const double el = std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count();
        if (el > timeout_seconds) {
            abort_comms(t);
            return fail("collectives did not finish within %.3f s; communicators aborted", timeout_seconds);
        }
        std::this_thread::sleep_for(std::chrono::microseconds(200));
    }
}

extern "C" CUNN_API int cunn_b200_dpt_write(cunn_b200_dpt *t, const char *path, const void *extra, long long extra_bytes)
{
    clear_error();
    CUNN_CHECK_ARG(t && !t->reps.empty() && path, "bad arguments");
    Replica &r = t->reps[0];
    std::vector<float> host((size_t)t->nparams);
    {
        DeviceGuard g(r.device);
        CUNN_CUDA(cudaStreamSynchronize(r.compute));
        if (t->nparams) CUNN_CUDA(cudaMemcpy(host.data(), r.params, (size_t)t->nparams * sizeof(float), cudaMemcpyDeviceToHost));
    }
    std::vector<int> gpus;
    if (t->rank_mode) for (int i = 0; i < t->world; ++i) gpus.push_back(i);          // one replica per process: GPU = rank on this box
    else for (Replica &q : t->reps) gpus.push_back(q.device);
    return cunn_b200_dpt_file_write(path, gpus.data(), (int)gpus.size(), host.data(), t->nparams, extra, extra_bytes);
}

extern "C" CUNN_API int cunn_b200_dpt_read_params(cunn_b200_dpt *t, const char *path, void *extra)
{
    clear_error();
    CUNN_CHECK_ARG(t && !t->reps.empty() && path, "bad arguments");
    long long np = 0, eb = 0;
    int ng = 0;
    if (cunn_b200_dpt_file_info(path, &ng, &np, &eb)) return 1;
    CUNN_CHECK_ARG(np == t->nparams, "%s holds %lld parameters, the table has %lld", path, np, t->nparams);
    std::vector<float> host((size_t)np);
    if (cunn_b200_dpt_file_read(path, t->world, 0, nullptr, host.data(), extra)) return 1;
    for (Replica &r : t->reps) {
        DeviceGuard g(r.device);
        if (np) CUNN_CUDA(cudaMemcpyAsync(r.params, host.data(), (size_t)np * sizeof(float), cudaMemcpyHostToDevice, r.compute));
        CUNN_CUDA(cudaStreamSynchronize(r.compute));
    }
    return 0;
}
