// mnq_dequant_matmul_static: the fused operator for callers that must not allocate.
//
// Who needs it.  The decode kernels split K across CTAs when a layer has few output rows and
// then need scratch memory for partial sums and arrival counters.  Normally the caller
// brings that scratch as the `workspace` argument, which means somebody called cudaMalloc
// (or torch's allocator) for it.  Some callers cannot: code running inside a region where
// device allocation is forbidden or would deadlock (a memory-pool callback, a real-time
// serving loop with a frozen memory budget, a plugin handed only its input and output
// buffers by a host runtime that owns all device memory).  For them this entry point uses
// a fixed scratch area that is part of the library image itself.
//
// The scratch is the file-scope array below: kStaticScratchBytes of device memory on every
// GPU that loads the library, held until the process exits.  On the host the array's name
// is only a handle, not a device address; the address is obtained once per device with
// cudaGetSymbolAddress (in this file, with that device current) and handed to the kernels.
#include <atomic>

#include "mnq_common.cuh"

namespace mnq {
namespace {

constexpr size_t kStaticScratchBytes = MNQ_STATIC_SCRATCH_BYTES;   // 4 MiB: 64 KiB of arrival counters, then partial sums

static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

constexpr int kMaxDevices = 64;
// device address of g_static_scratch per device ordinal; several host threads may make a device's
// first call together (each resolves the same address; the atomic makes that well defined)
std::atomic<void*> g_scratch_addr[kMaxDevices];

// Device address of the scratch array on the current device.  The first call on a device
// resolves it (a synchronous runtime call, not capturable); later calls read the cache.
int static_scratch(void** out)
{
    int dev = 0;
    int rc = check_cuda(cudaGetDevice(&dev), "cudaGetDevice");
    if (rc) return rc;
    if (dev < 0 || dev >= kMaxDevices) return fail(MNQ_INVALID_ARGUMENT, "dequant_matmul_static: device ordinal %d", dev);
    void* ptr = g_scratch_addr[dev].load(std::memory_order_acquire);
    if (!ptr) {
        rc = check_cuda(cudaGetSymbolAddress(&ptr, g_static_scratch), "cudaGetSymbolAddress(static scratch)");
        if (rc) return rc;
        if (!ptr) return fail(MNQ_INTERNAL_ERROR, "dequant_matmul_static: null scratch address");
        g_scratch_addr[dev].store(ptr, std::memory_order_release);
    }
    *out = ptr;
    return MNQ_SUCCESS;
}

}  // namespace
}  // namespace mnq

using namespace mnq;

extern "C" {

int mnq_dequant_matmul_static(const void* activations, const void* weights_packed, const void* scales,
                              const void* zeros, void* out, int64_t M, int64_t N, int64_t K, int64_t lda,
                              int64_t ldc, int32_t group_size, int32_t quant_type, int32_t act_dtype,
                              int32_t scale_dtype, void* stream)
{
    // Problems whose split-K scratch would not fit are refused, not silently run slower.
    const size_t need = mnq_workspace_bytes(M, N, K, group_size, quant_type);
    if (need > kStaticScratchBytes)
        return fail(MNQ_INVALID_ARGUMENT,
                    "dequant_matmul_static: this problem wants %zu bytes of scratch, the built-in area holds %zu "
                    "(use mnq_dequant_matmul with a caller-provided workspace)",
                    need, kStaticScratchBytes);
    void* scratch = nullptr;
    if (need > 0 && M > 0 && N > 0 && K > 0) {
        const int rc = static_scratch(&scratch);
        if (rc) return rc;
        // The array keeps whatever the previous call left.  Partial sums are always written
        // before they are read; the arrival counters must start at zero, so clear them.
        const int rc2 = check_cuda(cudaMemsetAsync(scratch, 0, kCounterBytes, static_cast<cudaStream_t>(stream)),
                                   "cudaMemsetAsync(static scratch counters)");
        if (rc2) return rc2;
    }
    return mnq_dequant_matmul(activations, weights_packed, scales, zeros, out, M, N, K, lda, ldc, group_size,
                              quant_type, act_dtype, scale_dtype, scratch, scratch ? kStaticScratchBytes : 0, stream);
}

}  // extern "C"
