// Data-parallel gradient buckets over NCCL behind the C ABI (xlstm_dp_*).
//
// The reference trains on one GPU (one CudaContext::new(0), src/gpu/mod.rs:134), so these entry
// points have no twin there. They are what a host that trains one replica per GPU calls around its
// backward pass: flat fp32 gradient buckets are registered once; the moment the backward pass has
// finished writing a bucket the host calls xlstm_dp_bucket_start, which orders a SUM all-reduce of
// that bucket behind the producing stream on a library-owned side stream, so the reduction runs
// while the layers below are still computing; xlstm_dp_wait makes the optimizer's stream wait for
// every reduction started since the last wait (the place of AdamwQueue::flush in the reference's
// step, src/gpu/hierarchical.rs:1696-1746).
//
// NCCL is bound at run time (dlopen of libnccl.so.2, preferring a copy the process has already
// loaded), so the library itself does not link it and hosts that never call xlstm_dp_* do not need it.
// The communicator is either created here from a unique id the host distributes (xlstm_dp_unique_id
// / xlstm_dp_init) or adopted from the host (xlstm_dp_init_comm). Plain NCCL only: no peer-memory
// operands, no multicast loads. State is kept per device; calls for one device come from one thread.
#include <dlfcn.h>
#include <string.h>

#include <vector>

#include "common.cuh"

namespace xl {
namespace dp {

// The handful of NCCL declarations used here (ABI-stable since NCCL 2.x).
typedef struct ncclComm* ncclComm_t;
struct ncclUniqueId { char internal[128]; };
typedef int ncclResult_t;
static constexpr int kNcclFloat32 = 7, kNcclSum = 0;

struct Api {
    void* handle = nullptr;
    ncclResult_t (*GetUniqueId)(ncclUniqueId*) = nullptr;
    ncclResult_t (*CommInitRank)(ncclComm_t*, int, ncclUniqueId, int) = nullptr;
    ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
    ncclResult_t (*AllReduce)(const void*, void*, size_t, int, int, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*CommCount)(const ncclComm_t, int*) = nullptr;
    const char* (*GetErrorString)(ncclResult_t) = nullptr;
};

static Api* api() {
    static Api a;
    static bool tried = false;
    if (tried) return a.handle ? &a : nullptr;
    tried = true;
    const char* names[] = {"libnccl.so.2", "libnccl.so"};
    void* h = nullptr;
    for (const char* n : names) {  // a copy the process already holds (e.g. the one a host framework bundles) wins
        h = dlopen(n, RTLD_NOW | RTLD_NOLOAD | RTLD_GLOBAL);
        if (h) break;
    }
    for (int i = 0; !h && i < 2; ++i) h = dlopen(names[i], RTLD_NOW | RTLD_GLOBAL);
    if (!h) return nullptr;
    a.GetUniqueId = (decltype(a.GetUniqueId))dlsym(h, "ncclGetUniqueId");
    a.CommInitRank = (decltype(a.CommInitRank))dlsym(h, "ncclCommInitRank");
    a.CommDestroy = (decltype(a.CommDestroy))dlsym(h, "ncclCommDestroy");
    a.AllReduce = (decltype(a.AllReduce))dlsym(h, "ncclAllReduce");
    a.CommCount = (decltype(a.CommCount))dlsym(h, "ncclCommCount");
    a.GetErrorString = (decltype(a.GetErrorString))dlsym(h, "ncclGetErrorString");
    if (!a.GetUniqueId || !a.CommInitRank || !a.CommDestroy || !a.AllReduce || !a.CommCount || !a.GetErrorString) return nullptr;
    a.handle = h;
    return &a;
}

struct Bucket {
    float* ptr;
    size_t n;
    cudaEvent_t produced, reduced;
    bool started;
};

struct State {
    ncclComm_t comm = nullptr;
    bool owns_comm = false;
    int nranks = 0;
    cudaStream_t side = nullptr;
    std::vector<Bucket> buckets;
};

static State g_state[64];

static State* state() {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
    return &g_state[dev];
}

#define XL_NCCL(a, expr)                                                       \
    do {                                                                       \
        ncclResult_t r__ = (expr);                                             \
        if (r__ != 0) {                                                        \
            xl::set_error("%s failed: %s", #expr, (a)->GetErrorString(r__));   \
            return XLSTM_ERR_CUDA;                                             \
        }                                                                      \
    } while (0)

static int adopt(State* s, Api* a, ncclComm_t comm, bool owns) {
    if (s->comm) { set_error("xlstm_dp: this device already has a communicator (call xlstm_dp_shutdown first)"); return XLSTM_ERR_ARG; }
    XL_NCCL(a, a->CommCount(comm, &s->nranks));
    int lo = 0, hi = 0;
    XL_CUDA(cudaDeviceGetStreamPriorityRange(&lo, &hi));
    // the reductions must not queue behind the backward pass they overlap with: highest priority
    XL_CUDA(cudaStreamCreateWithPriority(&s->side, cudaStreamNonBlocking, hi));
    s->comm = comm;
    s->owns_comm = owns;
    return XLSTM_OK;
}

}  // namespace dp
}  // namespace xl

using namespace xl;
using namespace xl::dp;

extern "C" int xlstm_dp_unique_id(void* out128) {
    XL_CHECK_ARG(out128, "xlstm_dp_unique_id: null pointer");
    Api* a = api();
    if (!a) { set_error("xlstm_dp: libnccl.so.2 could not be loaded"); return XLSTM_ERR_CUDA; }
    XL_NCCL(a, a->GetUniqueId((ncclUniqueId*)out128));
    return XLSTM_OK;
}

extern "C" int xlstm_dp_init(int nranks, int rank, const void* unique_id128) {
    XL_CHECK_ARG(unique_id128 && nranks >= 1 && rank >= 0 && rank < nranks, "xlstm_dp_init: bad arguments (nranks=%d rank=%d)", nranks, rank);
    Api* a = api();
    if (!a) { set_error("xlstm_dp: libnccl.so.2 could not be loaded"); return XLSTM_ERR_CUDA; }
    State* s = state();
    if (!s) { set_error("xlstm_dp_init: no current CUDA device"); return XLSTM_ERR_CUDA; }
    if (s->comm) { set_error("xlstm_dp: this device already has a communicator (call xlstm_dp_shutdown first)"); return XLSTM_ERR_ARG; }
    ncclUniqueId id;
    memcpy(&id, unique_id128, sizeof(id));
    ncclComm_t comm = nullptr;
    XL_NCCL(a, a->CommInitRank(&comm, nranks, id, rank));
    int rc = adopt(s, a, comm, true);
    if (rc) a->CommDestroy(comm);
    return rc;
}

extern "C" int xlstm_dp_init_comm(void* nccl_comm) {
    XL_CHECK_ARG(nccl_comm, "xlstm_dp_init_comm: null communicator");
    Api* a = api();
    if (!a) { set_error("xlstm_dp: libnccl.so.2 could not be loaded"); return XLSTM_ERR_CUDA; }
    State* s = state();
    if (!s) { set_error("xlstm_dp_init_comm: no current CUDA device"); return XLSTM_ERR_CUDA; }
    return adopt(s, a, (ncclComm_t)nccl_comm, false);
}

extern "C" int xlstm_dp_world(void) {
    State* s = state();
    return (s && s->comm) ? s->nranks : 0;
}

extern "C" int xlstm_dp_bucket_register(float* grads, size_t n) {
    State* s = state();
    if (!s || !s->comm) { set_error("xlstm_dp_bucket_register: no communicator on this device"); return XLSTM_ERR_ARG; }
    XL_CHECK_ARG(grads && n > 0, "xlstm_dp_bucket_register: empty bucket");
    Bucket b = {grads, n, nullptr, nullptr, false};
    XL_CUDA(cudaEventCreateWithFlags(&b.produced, cudaEventDisableTiming));
    XL_CUDA(cudaEventCreateWithFlags(&b.reduced, cudaEventDisableTiming));
    s->buckets.push_back(b);
    return (int)s->buckets.size() - 1;
}

extern "C" int xlstm_dp_bucket_start(int index, void* producer_stream) {
    State* s = state();
    if (!s || !s->comm) { set_error("xlstm_dp_bucket_start: no communicator on this device"); return XLSTM_ERR_ARG; }
    XL_CHECK_ARG(index >= 0 && index < (int)s->buckets.size(), "xlstm_dp_bucket_start: no bucket %d", index);
    Bucket& b = s->buckets[index];
    XL_CHECK_ARG(!b.started, "xlstm_dp_bucket_start: bucket %d was started and not waited for", index);
    Api* a = api();
    XL_CUDA(cudaEventRecord(b.produced, (cudaStream_t)producer_stream));
    XL_CUDA(cudaStreamWaitEvent(s->side, b.produced, 0));
    XL_NCCL(a, a->AllReduce(b.ptr, b.ptr, b.n, kNcclFloat32, kNcclSum, s->comm, s->side));
    XL_CUDA(cudaEventRecord(b.reduced, s->side));
    b.started = true;
    return XLSTM_OK;
}

extern "C" int xlstm_dp_wait(void* stream) {
    State* s = state();
    if (!s || !s->comm) { set_error("xlstm_dp_wait: no communicator on this device"); return XLSTM_ERR_ARG; }
    for (Bucket& b : s->buckets) {
        if (!b.started) continue;
        XL_CUDA(cudaStreamWaitEvent((cudaStream_t)stream, b.reduced, 0));
        b.started = false;
    }
    return XLSTM_OK;
}

extern "C" int xlstm_dp_shutdown(void) {
    State* s = state();
    if (!s || !s->comm) return XLSTM_OK;
    if (s->side) cudaStreamSynchronize(s->side);
    for (Bucket& b : s->buckets) {
        cudaEventDestroy(b.produced);
        cudaEventDestroy(b.reduced);
    }
    s->buckets.clear();
    Api* a = api();
    if (s->owns_comm && a) a->CommDestroy(s->comm);
    if (s->side) cudaStreamDestroy(s->side);
    *s = State();
    return XLSTM_OK;
}
