/* A stand-in for libnccl used only by the CPU tests of the DataParallelTable watchdog: it exports the symbols the
 * library resolves at run time, moves no data, and lets the test choose what ncclCommGetAsyncError reports. */
#include <stddef.h>

typedef int ncclResult_t;
typedef struct fake_comm *ncclComm_t;
typedef struct { char internal[128]; } ncclUniqueId;

static int g_async = 0;       /* value ncclCommGetAsyncError hands out (0 success, 2 system error, 7 in progress) */
static int g_aborts = 0;

void fake_nccl_set_async(int v) { g_async = v; }
int fake_nccl_aborts(void) { return g_aborts; }
void fake_nccl_reset(void) { g_async = 0; g_aborts = 0; }

ncclResult_t ncclGetUniqueId(ncclUniqueId *id) { for (int i = 0; i < 128; ++i) id->internal[i] = (char)i; return 0; }
ncclResult_t ncclCommInitRank(ncclComm_t *c, int n, ncclUniqueId id, int r) { (void)n; (void)id; (void)r; *c = (ncclComm_t)0x10; return 0; }
ncclResult_t ncclCommInitAll(ncclComm_t *c, int n, const int *d) { (void)d; for (int i = 0; i < n; ++i) c[i] = (ncclComm_t)(size_t)(0x10 + i); return 0; }
ncclResult_t ncclCommDestroy(ncclComm_t c) { (void)c; return 0; }
ncclResult_t ncclCommAbort(ncclComm_t c) { (void)c; ++g_aborts; return 0; }
ncclResult_t ncclCommGetAsyncError(ncclComm_t c, ncclResult_t *e) { (void)c; *e = g_async; return 0; }
ncclResult_t ncclAllReduce(const void *s, void *r, size_t n, int t, int o, ncclComm_t c, void *st) { (void)s; (void)r; (void)n; (void)t; (void)o; (void)c; (void)st; return 0; }
ncclResult_t ncclBroadcast(const void *s, void *r, size_t n, int t, int root, ncclComm_t c, void *st) { (void)s; (void)r; (void)n; (void)t; (void)root; (void)c; (void)st; return 0; }
ncclResult_t ncclGroupStart(void) { return 0; }
ncclResult_t ncclGroupEnd(void) { return 0; }
const char *ncclGetErrorString(ncclResult_t r) { return r == 2 ? "unhandled system error" : r == 7 ? "in progress" : "fake nccl"; }
