// Forward-with-stash for callers that must not allocate device memory.
//
// Some callers of this library cannot call cudaMalloc (or anything that does it for them, such as a framework
// allocator): a plug-in whose host hands every component a fixed device-memory budget at start-up, or a latency-critical
// loop that cannot afford the device-wide synchronisation an allocation implies. qmlp_network_forward needs a caller
// allocated stash buffer; the entry point below runs the same kernel with the stash in a fixed array that is part of this
// library's device image instead.
//
// Consequences of that choice, all visible to the caller:
//   * the array (QMLP_STATIC_SCRATCH_BYTES) is reserved on every GPU whose context loads this library, until exit;
//   * batches whose stash does not fit are rejected with an error, never truncated;
//   * there is ONE array per device: every call writes it, so two calls that overlap on the GPU (different streams,
//     different networks, different threads) race on it. It keeps the contents of the last call. Nothing in it has
//     to start at zero: the forward kernel overwrites every stash row of the batch before anything reads it;
//   * the first call on a device looks the array's device address up (and may load or build the kernels of the network,
//     like any first call); make that first call before starting a stream capture.
#include "host.hpp"

#include <atomic>

#include <cuda_runtime.h>

namespace {

// Stash of the forward pass: (encoded input + all pre-activations) * 2 bytes per point, points rounded up to 32.
// 32 MiB holds 65 536 points of a 32 -> 64 -> 64 -> 16 network (352 bytes per point).
static __device__ __align__(256) unsigned char g_forwardScratch[QMLP_STATIC_SCRATCH_BYTES];

// In host code `g_forwardScratch` is only a handle for the runtime, not a device address. The address differs per
// device, so it is looked up once per device with that device current.
void* scratchAddressOnCurrentDevice()
{
    static std::atomic<void*> address[64];
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) throw qmlp::cuda_error(std::string("cudaGetDevice: ") + cudaGetErrorString(e));
    if (dev < 0 || dev >= 64) throw qmlp::cuda_error("device index out of range");
    void* ptr = address[dev].load(std::memory_order_acquire);
    if (ptr == nullptr) {
        e = cudaGetSymbolAddress(&ptr, g_forwardScratch);
        if (e != cudaSuccess || ptr == nullptr)
            throw qmlp::cuda_error(std::string("cudaGetSymbolAddress(static scratch): ") + cudaGetErrorString(e));
        address[dev].store(ptr, std::memory_order_release);
    }
    return ptr;
}

} // namespace

extern "C" int qmlp_network_forward_static_scratch(qmlp_network_t* net, const qmlp_tensor_t* input, qmlp_tensor_t* output,
                                                   qmlp_stream_t stream)
{
    try {
        if (net == nullptr || input == nullptr || output == nullptr) throw std::runtime_error("null argument");
        if (input->ndim != 2) throw std::runtime_error("input has the wrong dimension, expected 2");
        const long long points = input->sizes[0];
        // the point count is compared before anything is multiplied, so that no product can wrap
        const long long maxPoints = static_cast<long long>(QMLP_STATIC_SCRATCH_BYTES) / (net->impl->stashHalfsPerPoint() * 2) / 32 * 32;
        if (points < 0) throw std::runtime_error("negative point count");
        if (points > maxPoints) {
            throw std::runtime_error(qmlp::format(
                "batch of %lld points needs more forward stash than the %zu bytes of static scratch "
                "(at most %lld points for this network); use qmlp_network_forward with a caller-allocated buffer",
                points, static_cast<size_t>(QMLP_STATIC_SCRATCH_BYTES), maxPoints));
        }
        void* scratch = scratchAddressOnCurrentDevice();
        qmlp::forwardWithStashAt(*net->impl, input, output, scratch, stream);
        return QMLP_OK;
    } catch (const qmlp::configuration_error& e) {
        return qmlp::reportError(QMLP_ERROR_CONFIGURATION, e.what());
    } catch (const qmlp::cuda_error& e) {
        return qmlp::reportError(QMLP_ERROR_CUDA, e.what());
    } catch (const qmlp::compile_error& e) {
        return qmlp::reportError(QMLP_ERROR_COMPILE, e.what());
    } catch (const std::exception& e) {
        return qmlp::reportError(QMLP_ERROR_RUNTIME, e.what());
    }
}

extern "C" int qmlp_static_scratch(void** device_address, size_t* bytes)
{
    try {
        if (device_address) *device_address = scratchAddressOnCurrentDevice();
        if (bytes) *bytes = static_cast<size_t>(QMLP_STATIC_SCRATCH_BYTES);
        return QMLP_OK;
    } catch (const qmlp::cuda_error& e) {
        return qmlp::reportError(QMLP_ERROR_CUDA, e.what());
    } catch (const std::exception& e) {
        return qmlp::reportError(QMLP_ERROR_RUNTIME, e.what());
    }
}
