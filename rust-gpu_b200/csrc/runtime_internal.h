// Internal definitions shared by the translation units that implement the runtime-facing C ABI.
#pragma once

#include <algorithm>
#include <atomic>
#include <cstdlib>
#include <map>
#include <memory>
#include <mutex>
#include <string>
#include <vector>

#include "kernels.h"

struct t0_buffer {
    t0_runtime* rt;
    void* dptr;
    size_t size;       // pool size class (4 KiB multiple)
};

struct t0_kernel {
    std::string name;
    uint32_t kernarg_size;
    int kind;          // 0 = gemm_gen config, 1 = TileIR spec, 2 = INT4 dequant (reference wire format)
    uint32_t group_log2 = 0;
    bool out_bf16 = false;
    t0_gemm_config cfg;
    t0_tile_gemm spec;
};

struct Scratch {
    void* ptr = nullptr;
    size_t size = 0;
};

struct t0_runtime {
    int device = 0;
    int sm_count = 148;
    cudaStream_t stream = nullptr;
    cudaEvent_t ev_start = nullptr, ev_stop = nullptr;
    std::mutex mu;
    std::map<size_t, std::vector<t0_buffer*>> pool;       // BufferPool.cache
    size_t cached_bytes = 0;
    std::map<uintptr_t, size_t> live;                      // device allocations handed out (for kernarg validation)
    std::map<std::string, std::unique_ptr<t0_kernel>> kernels;
    std::atomic<bool> poisoned{false};
    std::atomic<uint64_t> launches{0};
    std::atomic<size_t> slot{0};
    std::atomic<uint64_t> wait_limit_ns{0};   // limit of a single device-side barrier wait; 0 = the kernels' default
    std::atomic<int> drop_next_load{0};       // self-test hook: the next GEMM launch leaves out one operand load
    bool static_scratch_cleared = false;      // t0_w4a16_gemm_static: this runtime has zeroed the shared counters once
    int* d_status = nullptr;     // device error word written by kernels whose bounded wait expired
    int* h_status = nullptr;     // pinned mirror
    unsigned long long* d_probe = nullptr;   // {cycles, ns} of the last GEMM kernel's CTA 0
    void* d_peer_maps = nullptr;             // gathered output: device slot for the destinations' tensor maps (made on first use)
    std::vector<uint64_t> peer_maps_key;     // destinations and shape the slot currently describes
    Scratch scratch_a, scratch_b, scratch_planes;
    Scratch scratch_w4;          // W4A16: slab arrival counters + straddling pieces
    Scratch scratch_w;           // W4A16 general path: dequantised weights
    Scratch scratch_cvt_a, scratch_cvt_b, scratch_cvt_c;   // f32 entries: bf16 copies of the operands, f32 product before alpha/beta
    void* host_pipe = nullptr;   // host-operand GEMM pipeline (streams, events, staging sets), made on first use
};

namespace t0 {

void host_pipe_free(t0_runtime* rt);   // host_pipeline.cu

#define T0_CUDA(expr)                                                                                  \
    do {                                                                                               \
        cudaError_t _e = (expr);                                                                       \
        if (_e != cudaSuccess) return fail(T0_ERR_CUDA, "%s: %s", #expr, cudaGetErrorString(_e));      \
    } while (0)

struct DeviceGuard {
    int prev = -1;
    explicit DeviceGuard(int dev) {
        cudaGetDevice(&prev);
        if (prev != dev) cudaSetDevice(dev);
        else prev = -1;
    }
    ~DeviceGuard() { if (prev >= 0) cudaSetDevice(prev); }
};

inline int check_rt(const t0_runtime* rt) {
    if (!rt) return fail(T0_ERR_INVALID, "null runtime");
    if (rt->poisoned.load(std::memory_order_relaxed))
        return fail(T0_ERR_POISONED, "runtime poisoned after a device failure - refusing dispatch");   // gpu_context.rs:311-313
    return T0_OK;
}

// Grow-only scratch areas (staging copies, split-K planes). Growing waits for the stream first.
inline int ensure_scratch(t0_runtime* rt, Scratch& s, size_t bytes) {
    if (bytes <= s.size) return T0_OK;
    T0_CUDA(cudaStreamSynchronize(rt->stream));
    if (s.ptr) cudaFree(s.ptr);
    s.ptr = nullptr; s.size = 0;
    size_t want = (bytes + (1u << 20) - 1) & ~(size_t)((1u << 20) - 1);
    T0_CUDA(cudaMalloc(&s.ptr, want));
    s.size = want;
    return T0_OK;
}

// After a synchronising call: read the device error word; a non-zero value poisons the runtime.
inline int check_status_after_sync(t0_runtime* rt) {
    cudaError_t e = cudaMemcpyAsync(rt->h_status, rt->d_status, sizeof(int), cudaMemcpyDeviceToHost, rt->stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(rt->stream);
    if (e != cudaSuccess) {
        rt->poisoned.store(true);
        return fail(T0_ERR_CUDA, "device failure while waiting: %s", cudaGetErrorString(e));
    }
    if (*rt->h_status != 0) {
        int code = *rt->h_status;
        rt->poisoned.store(true);
        cudaMemsetAsync(rt->d_status, 0, sizeof(int), rt->stream);
        return fail(T0_ERR_TIMEOUT, "a bounded device-side wait expired (status 0x%08x: role %d, work item %d)", code,
                    (code >> 24) & 0xFF, code & 0xFFFFFF);
    }
    return T0_OK;
}

}  // namespace t0
