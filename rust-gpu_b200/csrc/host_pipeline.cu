// GEMMs whose operands and results live in HOST memory, pipelined over PCIe.
//
// The reference's host-facing GEMM calls upload, dispatch and read back one after the other (T0BlasLib::gemm,
// src/universal/math/blas.rs:18-100; ignis::ops::bf16_matmul::dispatch_gemm_forward, src/ignis/ops/bf16_matmul.rs:61-190).
// At 4096^3 the GEMM itself takes 0.11 ms on a B200 while the operands (64 MiB in, 64 MiB out) need 2.4 ms on the
// link, so a caller with several problems is bound by how well the two directions of the link are kept busy.  This entry
// takes an array of problems and runs three queues: uploads, kernels, downloads.  Problem i+1 is uploaded while problem
// i is computed and downloaded; two staging sets on the device are enough because a kernel is short against a copy.
//
//   upload queue : [wait kernel i-2] A_i, B_i (, bias_i) -> set i%2                     record up[i%2]
//   kernel queue : wait up[i%2], [wait download i-2]     t0_gemm_launch on the set       record gemm[i%2]
//   download q.  : wait gemm[i%2]                         C_i -> host                    record down[i%2]
//
// The kernel queue is the runtime's own stream, so everything the caller queued before is ordered before the first
// kernel.  The call returns when every result is in host memory.  Host memory should be page-locked (cudaHostAlloc or
// cudaHostRegister); with pageable memory the copies are staged by the driver and do not overlap.
#include "runtime_internal.h"

namespace t0 {

struct HostPipe {
    static constexpr int kSets = 2;
    cudaStream_t up = nullptr, down = nullptr;
    Scratch a[kSets], b[kSets], c[kSets], bias[kSets];
    cudaEvent_t up_done[kSets] = {}, gemm_done[kSets] = {}, down_done[kSets] = {};
};

void host_pipe_free(t0_runtime* rt) {
    HostPipe* hp = (HostPipe*)rt->host_pipe;
    if (!hp) return;
    if (hp->up) { cudaStreamSynchronize(hp->up); cudaStreamDestroy(hp->up); }
    if (hp->down) { cudaStreamSynchronize(hp->down); cudaStreamDestroy(hp->down); }
    for (int s = 0; s < HostPipe::kSets; ++s) {
        for (Scratch* x : {&hp->a[s], &hp->b[s], &hp->c[s], &hp->bias[s]})
            if (x->ptr) cudaFree(x->ptr);
        for (cudaEvent_t e : {hp->up_done[s], hp->gemm_done[s], hp->down_done[s]})
            if (e) cudaEventDestroy(e);
    }
    delete hp;
    rt->host_pipe = nullptr;
}

namespace {

int host_pipe_get(t0_runtime* rt, HostPipe** out) {
    if (!rt->host_pipe) {
        std::unique_ptr<HostPipe> hp(new HostPipe());
        T0_CUDA(cudaStreamCreateWithFlags(&hp->up, cudaStreamNonBlocking));
        T0_CUDA(cudaStreamCreateWithFlags(&hp->down, cudaStreamNonBlocking));
        for (int s = 0; s < HostPipe::kSets; ++s) {
            T0_CUDA(cudaEventCreateWithFlags(&hp->up_done[s], cudaEventDisableTiming));
            T0_CUDA(cudaEventCreateWithFlags(&hp->gemm_done[s], cudaEventDisableTiming));
            T0_CUDA(cudaEventCreateWithFlags(&hp->down_done[s], cudaEventDisableTiming));
        }
        rt->host_pipe = hp.release();
    }
    *out = (HostPipe*)rt->host_pipe;
    return T0_OK;
}

// staging buffers are private to this file and only grown while all three queues are idle
int grow(Scratch& s, size_t bytes) {
    if (bytes <= s.size) return T0_OK;
    if (s.ptr) cudaFree(s.ptr);
    s.ptr = nullptr; s.size = 0;
    const size_t want = (bytes + (1u << 20) - 1) & ~(size_t)((1u << 20) - 1);
    T0_CUDA(cudaMalloc(&s.ptr, want));
    s.size = want;
    return T0_OK;
}

struct Sizes { size_t a, b, c, bias; };

bool wants_bias(const t0_gemm_args& g) {
    if (g.n_tile_epilogue) {
        for (uint32_t i = 0; i < g.n_tile_epilogue && i < T0_TILE_MAX_EPILOGUE; ++i)
            if (g.tile_epilogue[i] == T0_TEPI_BIAS_ADD) return true;
        return false;
    }
    return g.epilogue != T0_EPI_STORE_F32;
}

}  // namespace
}  // namespace t0

using namespace t0;

extern "C" {

int t0_gemm_launch_host_batch(t0_runtime* rt, const t0_gemm_args* args, size_t count) {
    int rc = check_rt(rt);
    if (rc != T0_OK) return rc;
    if (!args && count) return fail(T0_ERR_INVALID, "null arguments");
    if (count == 0) return T0_OK;
    std::vector<Sizes> sz(count);
    Sizes most = {0, 0, 0, 0};
    for (size_t i = 0; i < count; ++i) {
        const t0_gemm_args& g = args[i];
        if (g.planes) return fail(T0_ERR_INVALID, "problem %zu: split-K planes cannot be returned to the host; leave planes 0", i);
        if (g.m == 0 || g.n == 0 || g.k == 0) return fail(T0_ERR_INVALID, "problem %zu: empty shape %ux%ux%u", i, g.m, g.n, g.k);
        if (!g.x || !g.b || !g.y) return fail(T0_ERR_INVALID, "problem %zu: null host pointer", i);
        const bool bias = wants_bias(g);
        if (bias && !g.bias) return fail(T0_ERR_INVALID, "problem %zu: the epilogue adds a bias but bias is null", i);
        sz[i].a = (size_t)g.m * g.k * 2;
        sz[i].b = (size_t)g.n * g.k * 2;
        sz[i].c = (size_t)g.m * g.n * (g.out_bf16 ? 2 : 4);
        sz[i].bias = bias ? (size_t)g.n * 4 : 0;
        most.a = std::max(most.a, sz[i].a); most.b = std::max(most.b, sz[i].b);
        most.c = std::max(most.c, sz[i].c); most.bias = std::max(most.bias, sz[i].bias);
    }
    DeviceGuard guard(rt->device);
    HostPipe* hp = nullptr;
    rc = host_pipe_get(rt, &hp);
    if (rc != T0_OK) return rc;
    // the previous call left all three queues idle, so the staging sets may be replaced here
    const int sets = count > 1 ? HostPipe::kSets : 1;
    for (int s = 0; s < sets; ++s) {
        if ((rc = grow(hp->a[s], most.a)) != T0_OK || (rc = grow(hp->b[s], most.b)) != T0_OK || (rc = grow(hp->c[s], most.c)) != T0_OK ||
            (rc = grow(hp->bias[s], most.bias)) != T0_OK)
            return rc;
    }

    int result = T0_OK;
    for (size_t i = 0; i < count && result == T0_OK; ++i) {
        const int s = (int)(i % (size_t)sets);
        const t0_gemm_args& g = args[i];
        cudaError_t e = cudaSuccess;
        auto step = [&](cudaError_t r) { if (e == cudaSuccess) e = r; };
        // uploads: the set's operands were last read by the kernel of problem i - sets
        if (i >= (size_t)sets) step(cudaStreamWaitEvent(hp->up, hp->gemm_done[s], 0));
        step(cudaMemcpyAsync(hp->a[s].ptr, (const void*)(uintptr_t)g.x, sz[i].a, cudaMemcpyHostToDevice, hp->up));
        step(cudaMemcpyAsync(hp->b[s].ptr, (const void*)(uintptr_t)g.b, sz[i].b, cudaMemcpyHostToDevice, hp->up));
        if (sz[i].bias) step(cudaMemcpyAsync(hp->bias[s].ptr, (const void*)(uintptr_t)g.bias, sz[i].bias, cudaMemcpyHostToDevice, hp->up));
        step(cudaEventRecord(hp->up_done[s], hp->up));
        // kernel: needs the operands, and the set's result buffer copied out (problem i - sets)
        step(cudaStreamWaitEvent(rt->stream, hp->up_done[s], 0));
        if (i >= (size_t)sets) step(cudaStreamWaitEvent(rt->stream, hp->down_done[s], 0));
        if (e != cudaSuccess) { result = fail(T0_ERR_CUDA, "host GEMM pipeline, problem %zu: %s", i, cudaGetErrorString(e)); break; }
        t0_gemm_args d = g;
        d.x = (uint64_t)(uintptr_t)hp->a[s].ptr;
        d.b = (uint64_t)(uintptr_t)hp->b[s].ptr;
        d.y = (uint64_t)(uintptr_t)hp->c[s].ptr;
        d.bias = sz[i].bias ? (uint64_t)(uintptr_t)hp->bias[s].ptr : 0;
        result = t0_gemm_launch(rt, &d);
        if (result != T0_OK) break;
        step(cudaEventRecord(hp->gemm_done[s], rt->stream));
        // download
        step(cudaStreamWaitEvent(hp->down, hp->gemm_done[s], 0));
        step(cudaMemcpyAsync((void*)(uintptr_t)g.y, hp->c[s].ptr, sz[i].c, cudaMemcpyDeviceToHost, hp->down));
        step(cudaEventRecord(hp->down_done[s], hp->down));
        if (e != cudaSuccess) result = fail(T0_ERR_CUDA, "host GEMM pipeline, problem %zu: %s", i, cudaGetErrorString(e));
    }
    // drain all three queues whatever happened, then look at the device status word
    cudaError_t e1 = cudaStreamSynchronize(hp->up);
    cudaError_t e2 = cudaStreamSynchronize(hp->down);
    int rs = check_status_after_sync(rt);
    if (result != T0_OK) return result;
    if (e1 != cudaSuccess || e2 != cudaSuccess) {
        rt->poisoned.store(true);
        return fail(T0_ERR_CUDA, "host GEMM pipeline: %s", cudaGetErrorString(e1 != cudaSuccess ? e1 : e2));
    }
    return rs;
}

int t0_gemm_launch_host(t0_runtime* rt, const t0_gemm_args* args) { return t0_gemm_launch_host_batch(rt, args, 1); }

}  // extern "C"
