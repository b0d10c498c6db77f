// N-column sharding of a large GEMM over the GPUs of one node.
//
// The reference is single-GPU; its only multi-device code moves data through host memory
// (src/universal/runtime/multi_gpu.rs:64-159).  Here the GEMM shards naturally: GPU r computes
// C[:, r*N/g : (r+1)*N/g] = A * B[:, slice] with A replicated and its slice of B local (in the NT layout the
// slice is rows [r*N/g, (r+1)*N/g) of WT[N,K], contiguous).  No exchange is needed in the computation.
// When the caller wants every GPU to hold all of C, each rank's kernel stores straight into slot `rank` of a
// rank-major buffer C_g[g][M][N/g] and one in-place ncclAllGather over NVLink completes it.
// NCCL is loaded at run time (dlopen) so the core library has no link-time dependency on it.
#include "runtime_internal.h"

#include <dlfcn.h>

using namespace t0;

namespace {

typedef struct ncclComm* ncclComm_t;
typedef int ncclResult_t;
typedef int ncclDataType_t;
constexpr ncclDataType_t kNcclFloat32 = 7;

struct NcclApi {
    void* handle = nullptr;
    ncclResult_t (*CommInitAll)(ncclComm_t*, int, const int*) = nullptr;
    ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
    ncclResult_t (*AllGather)(const void*, void*, size_t, ncclDataType_t, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*GroupStart)() = nullptr;
    ncclResult_t (*GroupEnd)() = nullptr;
    const char* (*GetErrorString)(ncclResult_t) = nullptr;
};

NcclApi* nccl() {
    static NcclApi api;
    static std::once_flag once;
    std::call_once(once, [] {
        for (const char* name : {"libnccl.so.2", "libnccl.so"}) {
            api.handle = dlopen(name, RTLD_NOW | RTLD_GLOBAL);
            if (api.handle) break;
        }
        if (!api.handle) return;
        api.CommInitAll = (decltype(api.CommInitAll))dlsym(api.handle, "ncclCommInitAll");
        api.CommDestroy = (decltype(api.CommDestroy))dlsym(api.handle, "ncclCommDestroy");
        api.AllGather = (decltype(api.AllGather))dlsym(api.handle, "ncclAllGather");
        api.GroupStart = (decltype(api.GroupStart))dlsym(api.handle, "ncclGroupStart");
        api.GroupEnd = (decltype(api.GroupEnd))dlsym(api.handle, "ncclGroupEnd");
        api.GetErrorString = (decltype(api.GetErrorString))dlsym(api.handle, "ncclGetErrorString");
    });
    return (api.handle && api.CommInitAll && api.AllGather && api.GroupStart && api.GroupEnd) ? &api : nullptr;
}

}  // namespace

struct t0_mg {
    std::vector<t0_runtime*> rts;
    std::vector<ncclComm_t> comms;   // created on first gather
    // host-operand call: per-GPU operand buffers (grow-only) and the event that marks a GPU's slice of A as uploaded
    std::vector<Scratch> dev_a, dev_b, dev_c;
    std::vector<cudaEvent_t> a_ready;
};

extern "C" {

int t0_shard_columns(uint32_t n, uint32_t n_gpus, uint32_t rank, uint32_t* first_col, uint32_t* n_cols) {
    if (!first_col || !n_cols) return fail(T0_ERR_INVALID, "null output");
    if (n_gpus == 0 || rank >= n_gpus) return fail(T0_ERR_INVALID, "rank %u of %u", rank, n_gpus);
    // equal blocks keep every rank's slice a whole number of 256-column tiles at the benchmark sizes and make the
    // gathered layout C_g[g][M][N/g] regular; a ragged N is refused rather than silently unbalanced
    if (n % n_gpus) return fail(T0_ERR_INVALID, "N=%u is not divisible by the number of GPUs %u", n, n_gpus);
    *n_cols = n / n_gpus;
    *first_col = rank * (n / n_gpus);
    return T0_OK;
}

int t0_mg_new(int n_gpus, t0_mg** out) {
    if (!out) return fail(T0_ERR_INVALID, "null output");
    *out = nullptr;
    int n_dev = 0;
    if (cudaGetDeviceCount(&n_dev) != cudaSuccess || n_dev == 0) return fail(T0_ERR_CUDA, "no CUDA device available; this library has no CPU fallback");
    if (n_gpus <= 0 || n_gpus > n_dev) return fail(T0_ERR_INVALID, "%d GPUs requested, %d present", n_gpus, n_dev);
    std::unique_ptr<t0_mg> mg(new t0_mg());
    for (int d = 0; d < n_gpus; ++d) {
        t0_runtime* rt = nullptr;
        int rc = t0_rt_new(d, &rt);
        if (rc != T0_OK) { for (t0_runtime* r : mg->rts) t0_rt_free(r); return rc; }
        mg->rts.push_back(rt);
    }
    *out = mg.release();
    return T0_OK;
}

void t0_mg_free(t0_mg* mg) {
    if (!mg) return;
    NcclApi* api = nccl();
    for (ncclComm_t c : mg->comms) if (api && api->CommDestroy) api->CommDestroy(c);
    for (size_t r = 0; r < mg->rts.size(); ++r) {
        DeviceGuard guard(mg->rts[r]->device);
        cudaStreamSynchronize(mg->rts[r]->stream);
        for (std::vector<Scratch>* v : {&mg->dev_a, &mg->dev_b, &mg->dev_c})
            if (r < v->size() && (*v)[r].ptr) cudaFree((*v)[r].ptr);
        if (r < mg->a_ready.size() && mg->a_ready[r]) cudaEventDestroy(mg->a_ready[r]);
    }
    for (t0_runtime* r : mg->rts) t0_rt_free(r);
    delete mg;
}

int t0_mg_size(const t0_mg* mg) { return mg ? (int)mg->rts.size() : 0; }
t0_runtime* t0_mg_runtime(t0_mg* mg, int rank) { return (mg && rank >= 0 && rank < (int)mg->rts.size()) ? mg->rts[rank] : nullptr; }

int t0_mg_synchronize(t0_mg* mg) {
    if (!mg) return fail(T0_ERR_INVALID, "null handle");
    int first = T0_OK;
    for (t0_runtime* r : mg->rts) { int rc = t0_rt_synchronize(r); if (rc != T0_OK && first == T0_OK) first = rc; }
    return first;
}

int t0_mg_gemm_sharded(t0_mg* mg, const uint64_t* x, const uint64_t* b_slice, const uint64_t* y_slice, uint32_t m, uint32_t n, uint32_t k,
                       uint32_t tile_n, int pair_cta) {
    if (!mg || !x || !b_slice || !y_slice) return fail(T0_ERR_INVALID, "null argument");
    const uint32_t g = (uint32_t)mg->rts.size();
    uint32_t first = 0, n_local = 0;
    int rc = t0_shard_columns(n, g, 0, &first, &n_local);
    if (rc != T0_OK) return rc;
    // launch on every GPU before waiting on any
    for (uint32_t r = 0; r < g; ++r) {
        t0_gemm_args a;
        memset(&a, 0, sizeof a);
        a.x = x[r]; a.b = b_slice[r]; a.y = y_slice[r];
        a.m = m; a.n = n_local; a.k = k; a.tile_n = tile_n; a.transpose = T0_NT; a.swap_grid = 1; a.pair_cta = (uint8_t)pair_cta;
        rc = t0_gemm_launch(mg->rts[r], &a);
        if (rc != T0_OK) return rc;
    }
    return T0_OK;
}

int t0_mg_gemm_sharded_gathered(t0_mg* mg, const uint64_t* x, const uint64_t* b_slice, const uint64_t* c_gathered, uint32_t m, uint32_t n,
                                uint32_t k) {
    if (!mg || !x || !b_slice || !c_gathered) return fail(T0_ERR_INVALID, "null argument");
    const uint32_t g = (uint32_t)mg->rts.size();
    if (g > kMaxPeerY + 1) return fail(T0_ERR_UNSUPPORTED, "at most %u GPUs", kMaxPeerY + 1);
    uint32_t first = 0, n_local = 0;
    int rc = t0_shard_columns(n, g, 0, &first, &n_local);
    if (rc != T0_OK) return rc;
    // every GPU must be able to store into every other GPU's buffer
    for (uint32_t r = 0; r < g; ++r) {
        DeviceGuard guard(mg->rts[r]->device);
        for (uint32_t d = 0; d < g; ++d) {
            if (d == r) continue;
            int can = 0;
            cudaDeviceCanAccessPeer(&can, mg->rts[r]->device, mg->rts[d]->device);
            if (!can) return fail(T0_ERR_UNSUPPORTED, "GPU %d cannot address GPU %d's memory: use t0_mg_gemm_sharded and t0_mg_all_gather_c", mg->rts[r]->device, mg->rts[d]->device);
            cudaError_t e = cudaDeviceEnablePeerAccess(mg->rts[d]->device, 0);
            if (e != cudaSuccess && e != cudaErrorPeerAccessAlreadyEnabled) return fail(T0_ERR_CUDA, "cudaDeviceEnablePeerAccess: %s", cudaGetErrorString(e));
            cudaGetLastError();
        }
    }
    const size_t slot = (size_t)m * n_local * sizeof(float);
    for (uint32_t r = 0; r < g; ++r) {
        t0_gemm_args a;
        memset(&a, 0, sizeof a);
        a.x = x[r]; a.b = b_slice[r]; a.y = c_gathered[r] + r * slot;
        a.m = m; a.n = n_local; a.k = k; a.transpose = T0_NT; a.swap_grid = 1;
        uint64_t peers[kMaxPeerY];
        uint32_t np = 0;
        for (uint32_t d = 0; d < g; ++d)
            if (d != r) peers[np++] = c_gathered[d] + r * slot;      // slot r of GPU d's buffer
        rc = t0_gemm_launch_gather(mg->rts[r], &a, peers, np);
        if (rc != T0_OK) return rc;
    }
    return T0_OK;
}

int t0_mg_gemm_sharded_host(t0_mg* mg, const void* x_host, const void* wt_host, void* y_host, uint32_t m, uint32_t n, uint32_t k) {
    if (!mg || !x_host || !wt_host || !y_host) return fail(T0_ERR_INVALID, "null argument");
    const uint32_t g = (uint32_t)mg->rts.size();
    if (m == 0 || n == 0) return T0_OK;
    if (k == 0 || k % 8) return fail(T0_ERR_UNSUPPORTED, "K=%u must be a positive multiple of 8", k);
    uint32_t first = 0, n_local = 0;
    int rc = t0_shard_columns(n, g, 0, &first, &n_local);
    if (rc != T0_OK) return rc;
    if (mg->dev_a.size() != g) {
        mg->dev_a.resize(g); mg->dev_b.resize(g); mg->dev_c.resize(g); mg->a_ready.resize(g, nullptr);
        for (uint32_t r = 0; r < g; ++r) {
            DeviceGuard guard(mg->rts[r]->device);
            T0_CUDA(cudaEventCreateWithFlags(&mg->a_ready[r], cudaEventDisableTiming));
            // direct peer copies over NVLink where the devices allow it (an error here only means the copies are staged)
            for (uint32_t s2 = 0; s2 < g; ++s2)
                if (s2 != r && cudaDeviceEnablePeerAccess(mg->rts[s2]->device, 0) != cudaSuccess) cudaGetLastError();
        }
    }
    const size_t row_bytes = (size_t)k * 2;
    const uint32_t rows_per = ceil_div(m, g);
    // 1. every GPU uploads ITS rows of A (A crosses the host link once in total), then its block of WT
    for (uint32_t r = 0; r < g; ++r) {
        t0_runtime* rt = mg->rts[r];
        rc = check_rt(rt);
        if (rc != T0_OK) return rc;
        DeviceGuard guard(rt->device);
        rc = ensure_scratch(rt, mg->dev_a[r], (size_t)m * row_bytes);
        if (rc == T0_OK) rc = ensure_scratch(rt, mg->dev_b[r], (size_t)n_local * row_bytes);
        if (rc == T0_OK) rc = ensure_scratch(rt, mg->dev_c[r], (size_t)m * n_local * 4);
        if (rc != T0_OK) return rc;
        const uint32_t r0 = std::min(m, r * rows_per), r1 = std::min(m, (r + 1) * rows_per);
        if (r1 > r0)
            T0_CUDA(cudaMemcpyAsync((uint8_t*)mg->dev_a[r].ptr + (size_t)r0 * row_bytes, (const uint8_t*)x_host + (size_t)r0 * row_bytes,
                                    (size_t)(r1 - r0) * row_bytes, cudaMemcpyHostToDevice, rt->stream));
        T0_CUDA(cudaEventRecord(mg->a_ready[r], rt->stream));
        T0_CUDA(cudaMemcpyAsync(mg->dev_b[r].ptr, (const uint8_t*)wt_host + (size_t)r * n_local * row_bytes, (size_t)n_local * row_bytes,
                                cudaMemcpyHostToDevice, rt->stream));
    }
    // 2. every GPU pulls the other GPUs' rows of A from their memories (plain peer copies), multiplies, and returns its
    //    column block of C into the caller's row-major y (a strided copy)
    for (uint32_t r = 0; r < g; ++r) {
        t0_runtime* rt = mg->rts[r];
        DeviceGuard guard(rt->device);
        for (uint32_t d = 1; d < g; ++d) {
            const uint32_t s2 = (r + d) % g;                       // staggered, so the sources are not all asked at once
            const uint32_t r0 = std::min(m, s2 * rows_per), r1 = std::min(m, (s2 + 1) * rows_per);
            if (r1 == r0) continue;
            T0_CUDA(cudaStreamWaitEvent(rt->stream, mg->a_ready[s2], 0));
            T0_CUDA(cudaMemcpyPeerAsync((uint8_t*)mg->dev_a[r].ptr + (size_t)r0 * row_bytes, rt->device,
                                        (const uint8_t*)mg->dev_a[s2].ptr + (size_t)r0 * row_bytes, mg->rts[s2]->device,
                                        (size_t)(r1 - r0) * row_bytes, rt->stream));
        }
        t0_gemm_args a;
        memset(&a, 0, sizeof a);
        a.x = (uint64_t)(uintptr_t)mg->dev_a[r].ptr; a.b = (uint64_t)(uintptr_t)mg->dev_b[r].ptr; a.y = (uint64_t)(uintptr_t)mg->dev_c[r].ptr;
        a.m = m; a.n = n_local; a.k = k; a.transpose = T0_NT; a.swap_grid = 1;
        rc = t0_gemm_launch(rt, &a);
        if (rc != T0_OK) return rc;
        T0_CUDA(cudaMemcpy2DAsync((uint8_t*)y_host + (size_t)r * n_local * 4, (size_t)n * 4, mg->dev_c[r].ptr, (size_t)n_local * 4,
                                  (size_t)n_local * 4, m, cudaMemcpyDeviceToHost, rt->stream));
    }
    // a GPU's copy of A may still be read by its peers when its own work is done: wait for all of them
    return t0_mg_synchronize(mg);
}

int t0_mg_all_gather_c(t0_mg* mg, const uint64_t* c_gathered, uint32_t m, uint32_t n) {
    if (!mg || !c_gathered) return fail(T0_ERR_INVALID, "null argument");
    const int g = (int)mg->rts.size();
    if (n % (uint32_t)g) return fail(T0_ERR_INVALID, "N=%u is not divisible by the number of GPUs %d", n, g);
    if (g == 1) return T0_OK;
    NcclApi* api = nccl();
    if (!api) return fail(T0_ERR_UNSUPPORTED, "libnccl.so.2 could not be loaded: the gathered C needs NCCL");
    if (mg->comms.empty()) {
        std::vector<int> devs(g);
        for (int r = 0; r < g; ++r) devs[r] = mg->rts[r]->device;
        mg->comms.resize(g);
        ncclResult_t e = api->CommInitAll(mg->comms.data(), g, devs.data());
        if (e != 0) { mg->comms.clear(); return fail(T0_ERR_CUDA, "ncclCommInitAll: %s", api->GetErrorString ? api->GetErrorString(e) : "error"); }
    }
    const size_t count = (size_t)m * (n / g);   // floats per rank
    api->GroupStart();
    ncclResult_t first_err = 0;
    for (int r = 0; r < g; ++r) {
        DeviceGuard guard(mg->rts[r]->device);
        float* recv = (float*)c_gathered[r];
        // in place: this rank's block already sits in slot r (the GEMM stored it there)
        ncclResult_t e = api->AllGather(recv + (size_t)r * count, recv, count, kNcclFloat32, mg->comms[r], mg->rts[r]->stream);
        if (e != 0 && first_err == 0) first_err = e;
    }
    ncclResult_t e = api->GroupEnd();
    if (first_err == 0) first_err = e;
    if (first_err != 0) return fail(T0_ERR_CUDA, "ncclAllGather: %s", api->GetErrorString ? api->GetErrorString(first_err) : "error");
    return T0_OK;
}

}  // extern "C"
