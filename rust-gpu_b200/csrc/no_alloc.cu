// A W4A16 entry point that never allocates.
//
// Who needs it: callers that run the fused INT4 GEMM at a point where device memory may not be allocated or freed — a
// serving loop that has handed all free HBM to its KV cache, a latency-critical section where an allocator call
// (which can synchronise the device) is not acceptable, or any code that must not fail for lack of memory once it has
// started.  `t0_w4a16_gemm` grows a scratch area inside the runtime on first use and for larger grids; this entry keeps
// the scratch (arrival counters and the partial pieces of bands shared between CTAs) in a fixed array that is part of
// the loaded module, so nothing is ever requested from the allocator.
//
// Limits that follow from the fixed size: M <= 16 (the fused kernel; larger M would need a K x N scratch matrix),
// N <= 4096 bands of 256 columns, and a grid of at most kMaxCtas CTAs (one per SM).  Anything larger is refused with
// T0_ERR_UNSUPPORTED and a message.
//
// The array is shared by every call on a device.  The counters must be zero when a call starts: the module loader
// zero-fills the array, and a kernel that runs to completion returns every counter it used to zero.  A kernel that gave up
// on a bounded wait does not: its runtime is poisoned, and a caller recovers by making a new runtime, so the FIRST static
// call of every runtime clears the counter region with a stream-ordered memset (no allocation) before its kernel.  Do not
// keep using the static entry from other, still healthy runtimes of the same device after such a failure without making
// them anew: they would read the stale counters.  Two calls that overlap in time on the same device (different streams or
// runtimes) race on the counters and pieces; calls on one runtime's stream are ordered and safe.  The first call on a
// device looks up the array's address (`cudaGetSymbolAddress`), so make that first call before starting any stream capture.
#include "runtime_internal.h"

namespace t0 {
size_t w4a16_fixed_scratch_bytes(uint32_t ctas);
size_t w4a16_counter_region_bytes();
int w4a16_fused_launch_fixed(t0_runtime* rt, uint64_t a, uint64_t packed, uint64_t scales, uint64_t zeros, uint64_t y, uint32_t M, uint32_t N,
                             uint32_t K, uint32_t group, void* scratch, size_t scratch_bytes);
}  // namespace t0

using namespace t0;

namespace {

constexpr uint32_t kMaxCtas = 160;                                   // B200 has 148 SMs; one CTA per SM
constexpr size_t kScratchBytes = 16 * 1024 + (size_t)kMaxCtas * 2 * 16 * 256 * sizeof(float);   // 16 KiB counters + 5 MiB pieces

static __device__ __align__(256) unsigned char g_w4_fixed_scratch[kScratchBytes];

constexpr int kMaxDevices = 64;
std::mutex g_setup_mu;
void* g_scratch_ptr[kMaxDevices] = {};

}  // namespace

extern "C" {

size_t t0_w4a16_gemm_static_scratch_bytes(void) { return kScratchBytes; }

int t0_w4a16_gemm_static(t0_runtime* rt, uint64_t a, uint64_t packed, uint64_t scales, uint64_t zeros, uint64_t y, uint32_t M, uint32_t N,
                         uint32_t K, uint32_t group) {
    int rc = check_rt(rt);
    if (rc != T0_OK) return rc;
    if (rt->device < 0 || rt->device >= kMaxDevices) return fail(T0_ERR_UNSUPPORTED, "device index %d out of range", rt->device);
    if (w4a16_fixed_scratch_bytes(kMaxCtas) > kScratchBytes) return fail(T0_ERR_UNSUPPORTED, "fixed scratch is smaller than the kernel's layout");
    DeviceGuard guard(rt->device);
    void* scratch = nullptr;
    {
        std::lock_guard<std::mutex> g(g_setup_mu);
        if (!g_scratch_ptr[rt->device]) {
            // set-up, once per device, with that device current: the address of this device's copy of the array
            void* ptr = nullptr;
            cudaError_t e = cudaGetSymbolAddress((void**)&ptr, g_w4_fixed_scratch);
            if (e != cudaSuccess || !ptr) return fail(T0_ERR_CUDA, "cudaGetSymbolAddress(fixed W4A16 scratch): %s", cudaGetErrorString(e));
            g_scratch_ptr[rt->device] = ptr;
        }
        scratch = g_scratch_ptr[rt->device];
    }
    if (!rt->static_scratch_cleared) {
        // counters left behind by a kernel that unwound on an expired wait (in a runtime since poisoned) would make this
        // runtime's bands never see their last contributor: start from zero, ordered before the kernel on the same stream
        T0_CUDA(cudaMemsetAsync(scratch, 0, w4a16_counter_region_bytes(), rt->stream));
        rt->static_scratch_cleared = true;
    }
    return w4a16_fused_launch_fixed(rt, a, packed, scales, zeros, y, M, N, K, group, scratch, kScratchBytes);
}

}  // extern "C"
