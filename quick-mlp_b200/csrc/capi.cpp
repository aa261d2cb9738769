// extern "C" entry points of libqmlp_b200.so: argument checks in the style of the reference's CHECK_* macros
// (src_cpp/include/qmlp/errors.h:78-90), launch-argument marshalling, and exception -> status-code translation.
#include "host.hpp"
#include "generic_kernels.h"

#include <algorithm>
#include <cmath>
#include <cstring>

#include <cuda_runtime.h>

using namespace qmlp;

namespace {

thread_local std::string g_lastError;

int fail(int code, const std::string& msg)
{
    g_lastError = msg;
    return code;
}

#define QMLP_TRY try {
#define QMLP_CATCH                                                                         \
    }                                                                                      \
    catch (const qmlp::configuration_error& e) { return fail(QMLP_ERROR_CONFIGURATION, e.what()); } \
    catch (const qmlp::cuda_error& e) { return fail(QMLP_ERROR_CUDA, e.what()); }          \
    catch (const qmlp::compile_error& e) { return fail(QMLP_ERROR_COMPILE, e.what()); }    \
    catch (const std::exception& e) { return fail(QMLP_ERROR_RUNTIME, e.what()); }         \
    catch (...) { return fail(QMLP_ERROR_RUNTIME, "unknown error"); }                      \
    return QMLP_OK;

void checkCuda(cudaError_t e, const char* what)
{
    if (e != cudaSuccess) throw cuda_error(std::string(what) + ": " + cudaGetErrorString(e));
}
void checkLaunch(int e, const char* what)
{
    if (e != 0) throw cuda_error(std::string(what) + ": " + cudaGetErrorString(static_cast<cudaError_t>(e)));
}

void checkDefined(const qmlp_tensor_t* t, const char* name)
{
    if (t == nullptr || t->ndim <= 0) throw std::runtime_error(std::string(name) + " is undefined");
    bool empty = false;
    for (int i = 0; i < t->ndim && i < 2; ++i) empty = empty || t->sizes[i] == 0;
    if (t->data == nullptr && !empty) throw std::runtime_error(std::string(name) + " is undefined");
}
void checkDim(const qmlp_tensor_t* t, int dim, const char* name)
{
    checkDefined(t, name);
    if (t->ndim != dim) throw std::runtime_error(format("%s has the wrong dimension, expected %d but got %d", name, dim, t->ndim));
}
void checkSize(const qmlp_tensor_t* t, int d, int64_t size, const char* name)
{
    if (t->sizes[d] != size)
        throw std::runtime_error(format("%s has the wrong size at dimension %d, expected %lld but got %lld", name, d,
                                        static_cast<long long>(size), static_cast<long long>(t->sizes[d])));
}
void checkDtype(const qmlp_tensor_t* t, int precision, const char* name)
{
    static const char* names[] = {"float", "half", "double"};
    if (t->precision != precision)
        throw std::runtime_error(format("%s has the wrong data type, expected %s", name, names[precision]));
}

void fillCommon(Network& n, kernel::LaunchArgs& a, const qmlp_tensor_t* input)
{
    std::memset(&a, 0, sizeof a);
    a.numel = input->sizes[0];
    a.input = static_cast<const float*>(input->data);
    a.inS0 = input->strides[0];
    a.inS1 = input->strides[1];
    if (!n.paramInference.defined()) throw std::runtime_error("Inference parameters not defined, call setNetworkParameter(...) first");
    if ((reinterpret_cast<uintptr_t>(n.paramInference.data) & 15) != 0)
        throw std::runtime_error("the network parameter vector must be 16-byte aligned");
    a.weights = static_cast<const __half*>(n.paramInference.data);
    a.gradWeights = static_cast<float*>(n.paramGradients.data);
    a.numSMs = Library::instance().smCount();
    a.forcePath = Library::instance().kernelPath;
    a.status = Library::instance().statusWord();
    n.fillGrids(a);
    for (int i = 0; i < a.numGrids; ++i) a.grids[i].status = a.status;
    for (int i = 0; i < n.numEncodings(); ++i) {
        auto e = n.encoding(i);
        if (e->hasParameters() && !e->paramInference.defined())
            throw std::runtime_error(format("encoding %d has parameters but none are bound (setParameter)", i));
    }
}

void checkIO(Network& n, const qmlp_tensor_t* input, const qmlp_tensor_t* output, const char* outName)
{
    // src_cpp/src/fused_network.cpp:509-516
    checkDim(input, 2, "input");
    checkDim(output, 2, outName);
    checkSize(input, 1, n.channelsIn(), "input");
    checkSize(output, 1, n.channelsOut(), outName);
    checkSize(output, 0, input->sizes[0], outName);
    checkDtype(input, QMLP_FLOAT, "input");
    checkDtype(output, QMLP_FLOAT, outName);
}

// Optional per-kernel device timing (qmlp_set_kernel_timing): an event pair around every launch the library makes,
// read back and summed per kernel by qmlp_read_kernel_timing. Off by default: the events cost a little.
struct KernelTimer {
    struct Record { int id; cudaEvent_t begin, end; };
    std::mutex mutex;
    bool enabled = false;
    std::vector<Record> records;
} g_timer;

constexpr int KERNEL_ID_ADAM = 100, KERNEL_ID_REFRESH_HALF = 101;

struct TimedLaunch {
    int id;
    cudaStream_t stream;
    cudaEvent_t begin = nullptr, end = nullptr;
    TimedLaunch(int kernelId, cudaStream_t s) : id(kernelId), stream(s)
    {
        if (!g_timer.enabled) return;
        if (cudaEventCreate(&begin) != cudaSuccess || cudaEventCreate(&end) != cudaSuccess) { begin = end = nullptr; return; }
        cudaEventRecord(begin, stream);
    }
    ~TimedLaunch()
    {
        if (!begin) return;
        cudaEventRecord(end, stream);
        std::lock_guard<std::mutex> lock(g_timer.mutex);
        g_timer.records.push_back({id, begin, end});
    }
};

// The launch arguments with the sizes of the scratch buffers they point to, for bounds-checking instantiations: the stash
// and the delta stash hold n32 rows of the network's widths, the planes planeStride points of the encoded channels.
kernel::LaunchArgs withScratchSizes(const Network& n, const kernel::LaunchArgs& a)
{
    kernel::LaunchArgs b = a;
    const long long n32 = (a.numel + 31) / 32 * 32;
    const long long shrink = Library::instance().boundsShrink;
    b.fwdTmpHalfs = a.fwdTmp ? std::max<long long>(1, n32 * n.stashHalfsPerPoint() - shrink) : 0;
    b.adjTmpHalfs = a.adjTmp ? std::max<long long>(1, n32 * n.deltaHalfsPerPoint() - shrink) : 0;
    b.planeHalfs = a.planes ? std::max<long long>(1, a.planeStride * n.encodedChannels() - shrink) : 0;
    return b;
}

void launchModule(Network& n, KernelModule& m, int kernelId, const kernel::LaunchArgs& a, qmlp_stream_t stream)
{
    TimedLaunch timed(kernelId, static_cast<cudaStream_t>(stream));
    int launches = 0;
    const kernel::LaunchArgs b = withScratchSizes(n, a);
    checkLaunch(m.launch(kernelId, &b, static_cast<cudaStream_t>(stream), &launches), "kernel launch failed");
    n.launchCount += launches;
}

void launchNet(Network& n, int kernelId, const kernel::LaunchArgs& a, qmlp_stream_t stream)
{
    if (a.numel <= 0) return;
    auto m = n.module(n.currentHalfMask());
    launchModule(n, *m, kernelId, a, stream);
}

// Backward launch. With `planes` (n32 x encoded channels halfs) and table gradients but no input gradients requested,
// the scatter of the table gradients can run as its own kernel (kernels/grid_planes.cuh) after the backward kernel.
// Both ways are bound by the L2 reduction rate (one 32-byte sector per clock and slice). The separate kernel merges
// neighbouring rows of two fp32 features into one 16-byte reduction (a quarter fewer L2 operations; config 3: 951 ->
// 848 us); with wider rows nothing can be merged and the fused scatter, which hides under the backward kernel's MMA
// phases, is faster (config 4: 1627 us fused, 2058 us split). Hence: split only if every grid has two features, or if
// the points are sorted into bins (`sorted`: a.input is the sorted copy and a.binStart its bin table), where the
// separate kernel sums the coarse levels in shared memory whatever the row width.
bool splitScatterChosen(Network& n, const kernel::LaunchArgs& a, bool havePlanes, bool sorted)
{
    bool gridGrad = false, twoFeatures = true;
    for (int i = 0; i < a.numGrids; ++i) gridGrad = gridGrad || a.grids[i].grad != nullptr;
    for (int i = 0; i < n.numEncodings(); ++i)
        if (auto* g = dynamic_cast<EncodingHashGrid*>(n.encoding(i).get())) {
            twoFeatures = twoFeatures && g->features() == 2;
            gridGrad = gridGrad && !g->isLine();
        }
    const int want = Library::instance().splitScatter;
    return havePlanes && gridGrad && (a.flags & kernel::FLAG_GRAD_ENCODINGS) != 0 && (a.flags & kernel::FLAG_GRAD_INPUT) == 0 &&
           Library::instance().kernelPath != 1 && (want == 1 || (want != 0 && (twoFeatures || sorted)));
}

void launchBackward(Network& n, kernel::LaunchArgs& a, __half* planes, int64_t n32, qmlp_stream_t stream, bool sorted = false,
                    bool scatterNow = true)
{
    const bool split = splitScatterChosen(n, a, planes != nullptr, sorted);
    if (split) {
        a.flags |= kernel::FLAG_SPLIT_SCATTER;
        a.planes = planes;
        a.planeStride = n32;
    }
    launchNet(n, kernel::KERNEL_BACKWARD, a, stream);
    if (split && scatterNow) launchNet(n, sorted ? kernel::KERNEL_SCATTER_SORTED : kernel::KERNEL_SCATTER_PLANES, a, stream);
}

// layout of the adjoint scratch: [delta of every layer, if weight gradients | adjoint feature planes, if table
// gradients], the second part 256-byte aligned
size_t adjointDeltaBytes(const Network& n, int64_t n32, int flags)
{
    return (flags & QMLP_GRADIENTS_NETWORK_WEIGHTS) ? static_cast<size_t>(n32) * n.deltaHalfsPerPoint() * 2 : 0;
}
size_t adjointPlaneBytes(const Network& n, int64_t n32, int flags)
{
    bool anyGrid = false;
    for (int i = 0; i < n.numEncodings(); ++i) anyGrid = anyGrid || n.encoding(i)->hasParameters();
    // also reserved when input gradients are requested on top (the planes are not used then), so that scratch sized
    // for a set of flags is large enough for every subset of it
    const bool wanted = anyGrid && (flags & QMLP_GRADIENTS_INPUT_ENCODINGS) != 0;
    return wanted ? static_cast<size_t>(n32) * n.encodedChannels() * 2 : 0;
}

} // namespace

namespace qmlp {

int reportError(int code, const char* message) { return fail(code, message ? message : ""); }

void forwardWithStashAt(Network& n, const qmlp_tensor_t* input, qmlp_tensor_t* output, void* tmp, qmlp_stream_t stream)
{
    std::lock_guard<std::mutex> lock(n.mutex);
    checkIO(n, input, output, "output");
    if ((reinterpret_cast<uintptr_t>(tmp) & 15) != 0) throw std::runtime_error("stash memory must be 16-byte aligned");
    kernel::LaunchArgs a;
    fillCommon(n, a, input);
    a.output = static_cast<float*>(output->data);
    a.outS0 = output->strides[0];
    a.outS1 = output->strides[1];
    a.fwdTmp = static_cast<__half*>(tmp);
    launchNet(n, kernel::KERNEL_FORWARD, a, stream);
}

} // namespace qmlp

extern "C" {

const char* qmlp_last_error(void) { return g_lastError.c_str(); }

int qmlp_is_cuda_available(void)
{
    int n = 0;
    return cudaGetDeviceCount(&n) == cudaSuccess && n > 0 ? 1 : 0;
}

int qmlp_set_log_level(const char* level)
{
    QMLP_TRY
    const std::string s = level ? level : "";
    int l;
    if (s == "off") l = 4;
    else if (s == "debug") l = 0;
    else if (s == "info") l = 1;
    else if (s == "warn") l = 2;
    else if (s == "error") l = 3;
    else throw std::runtime_error("Unknown log level '" + s + "', expected one of off, debug, info, warn, error");
    Library::instance().logLevel = l;
    QMLP_CATCH
}

int qmlp_set_compile_debug_mode(int enabled) { Library::instance().debugMode = enabled != 0; return QMLP_OK; }
int qmlp_is_compile_debug_mode(void) { return Library::instance().debugMode ? 1 : 0; }
int qmlp_set_kernel_cache_dir(const char* dir) { Library::instance().cacheDir = dir ? dir : ""; return QMLP_OK; }
const char* qmlp_get_kernel_cache_dir(void)
{
    static thread_local std::string s;
    s = Library::instance().resolveCacheDir();
    return s.c_str();
}
int qmlp_set_kernel_include_dir(const char* dir) { Library::instance().includeDir = dir ? dir : ""; return QMLP_OK; }

int qmlp_set_kernel_path(int path)
{
    QMLP_TRY
    if (path < 0 || path > 3)
        throw std::runtime_error("kernel path must be 0 (best for spec and batch), 1 (mma.sync only), 2 (level-major grid pass) or 3 (tcgen05 at any batch size)");
    Library::instance().kernelPath = path;
    QMLP_CATCH
}

int qmlp_set_tuning(const char* key, int value)
{
    QMLP_TRY
    const std::string k = key ? key : "";
    Library& lib = Library::instance();
    if (k == "sort_points") lib.sortPoints = value;
    else if (k == "split_scatter") lib.splitScatter = value;
    else if (k == "scatter_runs") lib.runAggregation = value;
    else if (k == "bounds_check") lib.boundsCheck = value > 0;
    else if (k == "bounds_shrink") lib.boundsShrink = value > 0 ? value : 0;
    else throw std::runtime_error("unknown tuning key '" + k + "' (sort_points, split_scatter, scatter_runs, bounds_check, bounds_shrink)");
    QMLP_CATCH
}

int qmlp_set_kernel_timing(int enabled)
{
    std::lock_guard<std::mutex> lock(g_timer.mutex);
    g_timer.enabled = enabled != 0;
    return QMLP_OK;
}

int qmlp_read_kernel_timing(int max_entries, int* kernel_ids, float* milliseconds, int* launches)
{
    std::vector<KernelTimer::Record> records;
    {
        std::lock_guard<std::mutex> lock(g_timer.mutex);
        records.swap(g_timer.records);
    }
    int n = 0;
    for (auto& r : records) {
        float ms = 0.f;
        const bool ok = cudaEventSynchronize(r.end) == cudaSuccess && cudaEventElapsedTime(&ms, r.begin, r.end) == cudaSuccess;
        cudaEventDestroy(r.begin);
        cudaEventDestroy(r.end);
        if (!ok || !kernel_ids || !milliseconds || !launches) continue;
        int at = 0;
        while (at < n && kernel_ids[at] != r.id) ++at;
        if (at == n) {
            if (n >= max_entries) continue;
            kernel_ids[n] = r.id; milliseconds[n] = 0.f; launches[n] = 0;
            ++n;
        }
        milliseconds[at] += ms;
        launches[at] += 1;
    }
    return n;
}

int qmlp_device_status(int* status)
{
    QMLP_TRY
    if (!status) throw std::runtime_error("null argument");
    int* w = Library::instance().statusWord();
    checkCuda(cudaDeviceSynchronize(), "cudaDeviceSynchronize");
    checkCuda(cudaMemcpy(status, w, sizeof(int), cudaMemcpyDeviceToHost), "cudaMemcpy");
    if (*status != 0) checkCuda(cudaMemset(w, 0, sizeof(int)), "cudaMemset");
    QMLP_CATCH
}

// ---- network -------------------------------------------------------------------------------------------------------
int qmlp_network_create(const char* cfg_json, const char* parent_dir, qmlp_network_t** out)
{
    QMLP_TRY
    if (!cfg_json || !out) throw std::runtime_error("null argument");
    Json cfg = Json::parse(cfg_json);
    auto net = std::make_shared<Network>(cfg, parent_dir ? parent_dir : ".");
    auto* h = new qmlp_network{net};
    for (int i = 0; i < net->numEncodings(); ++i) net->encodingHandles.push_back(new qmlp_encoding{net->encoding(i)});
    *out = h;
    QMLP_CATCH
}

void qmlp_network_destroy(qmlp_network_t* net)
{
    if (!net) return;
    for (auto* e : net->impl->encodingHandles) delete e;
    delete net;
}

int qmlp_network_channels_in(const qmlp_network_t* net) { return net->impl->channelsIn(); }
int qmlp_network_channels_out(const qmlp_network_t* net) { return net->impl->channelsOut(); }
int qmlp_network_num_layers(const qmlp_network_t* net) { return net->impl->numLayers(); }
int qmlp_network_num_encodings(const qmlp_network_t* net) { return net->impl->numEncodings(); }
int64_t qmlp_network_parameter_count(const qmlp_network_t* net) { return net->impl->parameterCount(); }
int qmlp_network_parameter_precision(const qmlp_network_t*, int usage) { return usage == QMLP_INFERENCE ? QMLP_HALF : QMLP_FLOAT; }
int64_t qmlp_network_launch_count(const qmlp_network_t* net) { return net->impl->launchCount; }

int qmlp_network_layer_info(const qmlp_network_t* net, int layer, int* channels_in, int* channels_out, int* use_bias,
                            int64_t* weights_start, int64_t* bias_start)
{
    QMLP_TRY
    if (layer < 0 || layer >= net->impl->numLayers()) throw std::runtime_error("Layer index out of bounds");
    const LayerSpec& l = net->impl->layer(layer);
    if (channels_in) *channels_in = l.channelsIn;
    if (channels_out) *channels_out = l.channelsOut;
    if (use_bias) *use_bias = l.useBias ? 1 : 0;
    if (weights_start) *weights_start = l.weightsStart;
    if (bias_start) *bias_start = l.biasStart;
    QMLP_CATCH
}

int qmlp_network_encoding(qmlp_network_t* net, int idx, qmlp_encoding_t** out)
{
    QMLP_TRY
    if (idx < 0 || idx >= net->impl->numEncodings()) throw std::runtime_error("Array index out of bounds");
    *out = net->impl->encodingHandles[idx];
    QMLP_CATCH
}

int qmlp_network_set_parameter(qmlp_network_t* net, const qmlp_tensor_t* tensor, int usage)
{
    QMLP_TRY
    net->impl->setParameter(tensor, usage);
    QMLP_CATCH
}

int qmlp_network_initialize_parameters_host(qmlp_network_t* net, uint64_t seed, uint16_t* dst_half)
{
    QMLP_TRY
    if (!dst_half) throw std::runtime_error("null destination");
    net->impl->initializeHost(seed, dst_half);
    QMLP_CATCH
}

int qmlp_network_initialize_parameters(qmlp_network_t* net, uint64_t seed)
{
    QMLP_TRY
    Network& n = *net->impl;
    if (!n.paramInference.defined()) throw std::runtime_error("Inference parameters not defined, call setNetworkParameter(...) first");
    std::vector<uint16_t> host(static_cast<size_t>(n.parameterCount()));
    n.initializeHost(seed, host.data());
    checkCuda(cudaMemcpy(n.paramInference.data, host.data(), host.size() * 2, cudaMemcpyHostToDevice), "cudaMemcpy");
    QMLP_CATCH
}

int qmlp_network_compile(qmlp_network_t* net, int grid_half_mask)
{
    QMLP_TRY
    net->impl->module(static_cast<unsigned>(grid_half_mask));
    QMLP_CATCH
}

int qmlp_network_clear_cached_kernels(qmlp_network_t* net)
{
    QMLP_TRY
    net->impl->clearModules();
    QMLP_CATCH
}

// inference on device tensors; the caller holds the network's mutex
static void inferenceLocked(Network& n, const qmlp_tensor_t* input, qmlp_tensor_t* output, qmlp_stream_t stream)
{
    checkIO(n, input, output, "output");
    kernel::LaunchArgs a;
    fillCommon(n, a, input);
    a.output = static_cast<float*>(output->data);
    a.outS0 = output->strides[0];
    a.outS1 = output->strides[1];
    // Encode level by level into planes, chunk by chunk, then run the layer chain on the planes
    // (kernels/grid_planes.cuh): when the tables are much larger than L2 (the level in work stays L2-resident), and when
    // the gather dominates a large batch (96 or more table rows per point: the dedicated pass keeps four light CTAs per
    // SM on nothing but gathers and runs at the SM's L2-request rate; config 3 at 2^20 points 0.40 -> 0.34 ms, while
    // config 4 with 72 rows per point and a heavier layer chain is level). kernelPath 2 forces this path.
    const int path = Library::instance().kernelPath;
    const bool gatherBound = n.gathersPerPoint() >= 96 && a.numel >= (1 << 18);
    const bool wantPlanes = !n.planesUnsupported && a.numGrids > 0 && a.numel > 0 &&
                            (path == 2 || (path == 0 && (n.gridTableBytes() > (96ll << 20) || gatherBound)));
    if (wantPlanes) {
        // Chunk: as many points as fit in 512 MB of planes, at most 2^22. A level's table is fetched from HBM once per
        // chunk, so large chunks amortise it; the planes themselves are streamed (written once, read once).
        const int64_t rowBytes = static_cast<int64_t>(n.encodedChannels()) * 2;
        int64_t cap = 1 << 16;
        while (cap < (1 << 22) && cap * 2 * rowBytes <= (512ll << 20)) cap *= 2;
        const int64_t need = std::min<int64_t>(cap, (a.numel + 65535) / 65536 * 65536);
        n.claimDevice();
        if (n.planeCapacity < need) {
            if (n.planes) {
                checkCuda(cudaStreamSynchronize(static_cast<cudaStream_t>(stream)), "cudaStreamSynchronize");
                checkCuda(cudaFree(n.planes), "cudaFree(feature planes)");
                n.planes = nullptr;
                n.planeCapacity = 0;
            }
            checkCuda(cudaMalloc(&n.planes, static_cast<size_t>(need * rowBytes)), "cudaMalloc(feature planes)");
            n.planeCapacity = need;
        }
        auto m = n.module(n.currentHalfMask());
        const long long total = a.numel;
        const float* in0 = a.input;
        float* out0 = a.output;
        bool ok = true;
        for (long long c0 = 0; c0 < total && ok; c0 += n.planeCapacity) {
            a.numel = std::min<long long>(n.planeCapacity, total - c0);
            a.input = in0 + c0 * a.inS0;
            a.output = out0 + c0 * a.outS0;
            a.planes = static_cast<__half*>(n.planes);
            a.planeStride = n.planeCapacity;
            int launches = 0;
            int e;
            {
                TimedLaunch timed(kernel::KERNEL_ENCODE_PLANES, static_cast<cudaStream_t>(stream));
                const kernel::LaunchArgs sized = withScratchSizes(n, a);
                e = m->launch(kernel::KERNEL_ENCODE_PLANES, &sized, static_cast<cudaStream_t>(stream), &launches);
            }
            if (e == static_cast<int>(cudaErrorNotSupported) && c0 == 0) { n.planesUnsupported = true; ok = false; break; }
            checkLaunch(e, "kernel launch failed");
            n.launchCount += launches;
            launchModule(n, *m, kernel::KERNEL_INFERENCE_PLANES, a, stream);
        }
        if (ok) return;
        a.numel = total;
        a.input = in0;
        a.output = out0;
    }
    launchNet(n, kernel::KERNEL_INFERENCE, a, stream);
}

int qmlp_network_inference(qmlp_network_t* net, const qmlp_tensor_t* input, qmlp_tensor_t* output, qmlp_stream_t stream)
{
    QMLP_TRY
    Network& n = *net->impl;
    std::lock_guard<std::mutex> lock(n.mutex);
    inferenceLocked(n, input, output, stream);
    QMLP_CATCH
}

int qmlp_network_inference_host(qmlp_network_t* net, const float* host_input, float* host_output, int64_t num_points,
                                int64_t chunk_points, qmlp_stream_t stream)
{
    QMLP_TRY
    Network& n = *net->impl;
    std::lock_guard<std::mutex> lock(n.mutex);
    if (num_points < 0 || chunk_points < 0) throw std::runtime_error("negative point count");
    if (num_points == 0) return QMLP_OK;
    if (!host_input || !host_output) throw std::runtime_error("null host buffer");
    const int cin = n.channelsIn(), cout = n.channelsOut();
    // default chunk: an eighth of the batch, between 2^16 and 2^20 points (measured best on a PCIe 5 x16 host link:
    // 8 chunks of 2^19 points). Smaller chunks pay more per-copy overhead, larger ones a longer pipeline fill (first
    // upload) and drain (last kernel + download).
    int64_t chunk = chunk_points;
    if (chunk == 0) {
        chunk = 1 << 16;
        while (chunk < (1 << 20) && chunk * 8 < num_points) chunk *= 2;
    }
    chunk = std::min(chunk, num_points);
    n.claimDevice();
    HostPipeline& hp = n.hostPipeline;
    hp.reserve(chunk, cin, cout);
    const cudaStream_t user = static_cast<cudaStream_t>(stream);
    // uploads start after the work already queued on the caller's stream (e.g. a parameter update)
    checkCuda(cudaEventRecord(hp.start, user), "cudaEventRecord");
    checkCuda(cudaStreamWaitEvent(hp.copyIn, hp.start, 0), "cudaStreamWaitEvent");
    checkCuda(cudaStreamWaitEvent(hp.copyOut, hp.start, 0), "cudaStreamWaitEvent");
    int64_t k = 0;
    for (int64_t p0 = 0; p0 < num_points; p0 += chunk, ++k) {
        const int s = static_cast<int>(k % HostPipeline::SLOTS);
        const int64_t m = std::min(chunk, num_points - p0);
        if (k >= HostPipeline::SLOTS) {
            // the slot's previous kernel has consumed its input; its previous download has left its output
            checkCuda(cudaStreamWaitEvent(hp.copyIn, hp.computed[s], 0), "cudaStreamWaitEvent");
            checkCuda(cudaStreamWaitEvent(user, hp.downloaded[s], 0), "cudaStreamWaitEvent");
        }
        checkCuda(cudaMemcpyAsync(hp.in[s], host_input + p0 * cin, static_cast<size_t>(m) * cin * 4, cudaMemcpyHostToDevice, hp.copyIn),
                  "cudaMemcpyAsync(host to device)");
        checkCuda(cudaEventRecord(hp.uploaded[s], hp.copyIn), "cudaEventRecord");
        checkCuda(cudaStreamWaitEvent(user, hp.uploaded[s], 0), "cudaStreamWaitEvent");
        qmlp_tensor_t ti{hp.in[s], QMLP_FLOAT, 2, {m, cin}, {cin, 1}};
        qmlp_tensor_t to{hp.out[s], QMLP_FLOAT, 2, {m, cout}, {cout, 1}};
        inferenceLocked(n, &ti, &to, stream);
        checkCuda(cudaEventRecord(hp.computed[s], user), "cudaEventRecord");
        checkCuda(cudaStreamWaitEvent(hp.copyOut, hp.computed[s], 0), "cudaStreamWaitEvent");
        checkCuda(cudaMemcpyAsync(host_output + p0 * cout, hp.out[s], static_cast<size_t>(m) * cout * 4, cudaMemcpyDeviceToHost, hp.copyOut),
                  "cudaMemcpyAsync(device to host)");
        checkCuda(cudaEventRecord(hp.downloaded[s], hp.copyOut), "cudaEventRecord");
    }
    // the caller's stream completes when the last downloads have landed
    for (int s = 0; s < HostPipeline::SLOTS && s < k; ++s)
        checkCuda(cudaStreamWaitEvent(user, hp.downloaded[s], 0), "cudaStreamWaitEvent");
    QMLP_CATCH
}

int qmlp_network_forward_memory(qmlp_network_t* net, int64_t num_elements, int, size_t* bytes)
{
    QMLP_TRY
    // encoded input + pre-activations, fp16, rows rounded up to the warp size (src_cpp/src/fused_network.cpp:674-681)
    const int64_t n32 = (num_elements + 31) / 32 * 32;
    *bytes = static_cast<size_t>(n32) * net->impl->stashHalfsPerPoint() * 2;
    QMLP_CATCH
}

int qmlp_network_forward(qmlp_network_t* net, const qmlp_tensor_t* input, qmlp_tensor_t* output, void* tmp_memory,
                         qmlp_stream_t stream)
{
    QMLP_TRY
    Network& n = *net->impl;
    std::lock_guard<std::mutex> lock(n.mutex);
    checkIO(n, input, output, "output");
    if (!tmp_memory && input->sizes[0] > 0) throw std::runtime_error("tmpMemory is null");
    if ((reinterpret_cast<uintptr_t>(tmp_memory) & 15) != 0) throw std::runtime_error("tmpMemory must be 16-byte aligned");
    kernel::LaunchArgs a;
    fillCommon(n, a, input);
    a.output = static_cast<float*>(output->data);
    a.outS0 = output->strides[0];
    a.outS1 = output->strides[1];
    a.fwdTmp = static_cast<__half*>(tmp_memory);
    launchNet(n, kernel::KERNEL_FORWARD, a, stream);
    QMLP_CATCH
}

int qmlp_network_zero_gradients(qmlp_network_t* net, qmlp_stream_t stream)
{
    QMLP_TRY
    Network& n = *net->impl;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (n.paramGradients.defined())
        checkCuda(cudaMemsetAsync(n.paramGradients.data, 0, static_cast<size_t>(n.parameterCount()) * 4, s), "cudaMemsetAsync");
    for (int i = 0; i < n.numEncodings(); ++i) {
        auto e = n.encoding(i);
        if (e->paramGradients.defined())
            checkCuda(cudaMemsetAsync(e->paramGradients.data, 0, static_cast<size_t>(e->parameterCount()) * 4, s), "cudaMemsetAsync");
    }
    QMLP_CATCH
}

int qmlp_network_adjoint_memory(qmlp_network_t* net, int64_t num_elements, int adjoint_flags, size_t* bytes)
{
    QMLP_TRY
    // delta of every layer, fp16, only needed for the weight gradients (src_cpp/src/fused_network.cpp:997-1002), and the
    // adjoint feature planes of the level-major table-gradient scatter
    const int64_t n32 = (num_elements + 31) / 32 * 32;
    const size_t planes = adjointPlaneBytes(*net->impl, n32, adjoint_flags);
    const size_t delta = adjointDeltaBytes(*net->impl, n32, adjoint_flags);
    *bytes = planes ? (delta + 255) / 256 * 256 + planes : delta;
    QMLP_CATCH
}

int qmlp_network_adjoint(qmlp_network_t* net, const qmlp_tensor_t* input, const qmlp_tensor_t* adj_output, int adjoint_flags,
                         qmlp_tensor_t* adj_input, const void* tmp_forward, void* tmp_adjoint, qmlp_stream_t stream)
{
    QMLP_TRY
    Network& n = *net->impl;
    std::lock_guard<std::mutex> lock(n.mutex);
    // src_cpp/src/fused_network.cpp:1015-1036
    checkIO(n, input, adj_output, "adjOutput");
    const int64_t numel = input->sizes[0];
    const bool gIn = adjoint_flags & QMLP_GRADIENTS_INPUT;
    const bool gW = adjoint_flags & QMLP_GRADIENTS_NETWORK_WEIGHTS;
    const bool gE = adjoint_flags & QMLP_GRADIENTS_INPUT_ENCODINGS;
    if (gIn) {
        if (adj_input == nullptr || adj_input->ndim <= 0 || adj_input->data == nullptr)
            throw std::runtime_error("Input gradients requested, but adjInput is undefined");
        checkDim(adj_input, 2, "adjInput");
        checkSize(adj_input, 1, n.channelsIn(), "adjInput");
        checkSize(adj_input, 0, numel, "adjInput");
        checkDtype(adj_input, QMLP_FLOAT, "adjInput");
    }
    if (!tmp_forward && numel > 0) throw std::runtime_error("tmpMemoryForward is null: run forward() first");
    if (gW) {
        if (!n.paramGradients.defined()) throw std::runtime_error("Weight gradients requested, but no gradient tensor is bound (setNetworkParameter(..., GRADIENTS))");
        if (!tmp_adjoint && numel > 0) throw std::runtime_error("tmpMemoryAdjoint is null");
    }
    if (tmp_adjoint && (reinterpret_cast<uintptr_t>(tmp_adjoint) & 15) != 0) throw std::runtime_error("adjoint scratch memory must be 16-byte aligned");
    kernel::LaunchArgs a;
    fillCommon(n, a, input);
    a.adjOutput = static_cast<const float*>(adj_output->data);
    a.aoS0 = adj_output->strides[0];
    a.aoS1 = adj_output->strides[1];
    if (gIn) {
        a.adjInput = static_cast<float*>(adj_input->data);
        a.aiS0 = adj_input->strides[0];
        a.aiS1 = adj_input->strides[1];
    }
    a.fwdTmp = const_cast<__half*>(static_cast<const __half*>(tmp_forward));
    a.adjTmp = static_cast<__half*>(tmp_adjoint);
    a.flags = (gIn ? kernel::FLAG_GRAD_INPUT : 0) | (gW ? kernel::FLAG_GRAD_WEIGHTS : 0) | (gE ? kernel::FLAG_GRAD_ENCODINGS : 0);
    if (a.flags == 0) return QMLP_OK;
    const int64_t n32 = (numel + 31) / 32 * 32;
    __half* planes = nullptr;   // a caller that passes no adjoint scratch gets the fused scatter
    if (tmp_adjoint && adjointPlaneBytes(n, n32, adjoint_flags) > 0)
        planes = reinterpret_cast<__half*>(static_cast<unsigned char*>(tmp_adjoint) + (adjointDeltaBytes(n, n32, adjoint_flags) + 255) / 256 * 256);
    launchBackward(n, a, planes, n32, stream);
    if (gW) launchNet(n, kernel::KERNEL_WGRAD, a, stream);
    QMLP_CATCH
}

// ---- encodings -----------------------------------------------------------------------------------------------------
int qmlp_encoding_create(const char* cfg_json, qmlp_encoding_t** out)
{
    QMLP_TRY
    if (!cfg_json || !out) throw std::runtime_error("null argument");
    *out = new qmlp_encoding{createEncoding(Json::parse(cfg_json))};
    QMLP_CATCH
}
void qmlp_encoding_destroy(qmlp_encoding_t* enc) { delete enc; }
const char* qmlp_encoding_to_json(qmlp_encoding_t* enc) { enc->impl->jsonCache = enc->impl->toJson().dump(); return enc->impl->jsonCache.c_str(); }
const char* qmlp_encoding_id(qmlp_encoding_t* enc) { enc->impl->idCache = enc->impl->id(); return enc->impl->idCache.c_str(); }
int qmlp_encoding_max_input_channel(const qmlp_encoding_t* enc) { return enc->impl->maxInputChannel(); }
int qmlp_encoding_num_output_channels(const qmlp_encoding_t* enc) { return enc->impl->numOutputChannels(); }
int qmlp_encoding_has_parameters(const qmlp_encoding_t* enc) { return enc->impl->hasParameters() ? 1 : 0; }
int64_t qmlp_encoding_parameter_count(const qmlp_encoding_t* enc) { return enc->impl->parameterCount(); }
int qmlp_encoding_parameter_precision(const qmlp_encoding_t*, int) { return QMLP_FLOAT; }

int qmlp_encoding_grid_levels(const qmlp_encoding_t* enc, int max_levels, int64_t* memory_offset, int32_t* resolution,
                              int32_t* hash_grid_size, int32_t* hashed)
{
    auto* g = dynamic_cast<EncodingHashGrid*>(enc->impl.get());
    if (!g) return 0;
    const auto& t = g->levelTable();
    for (int i = 0; i < static_cast<int>(t.size()) && i < max_levels; ++i) {
        if (memory_offset) memory_offset[i] = t[i].memoryOffset;
        if (resolution) resolution[i] = t[i].resolution;
        if (hash_grid_size) hash_grid_size[i] = t[i].hashGridSize;
        if (hashed) hashed[i] = t[i].hashed ? 1 : 0;
    }
    return static_cast<int>(t.size());
}

int qmlp_encoding_set_parameter(qmlp_encoding_t* enc, const qmlp_tensor_t* tensor, int usage)
{
    QMLP_TRY
    enc->impl->setParameter(tensor, usage);
    QMLP_CATCH
}

int qmlp_encoding_zero_gradients(qmlp_encoding_t* enc, qmlp_stream_t stream)
{
    QMLP_TRY
    if (enc->impl->paramGradients.defined())
        checkCuda(cudaMemsetAsync(enc->impl->paramGradients.data, 0, static_cast<size_t>(enc->impl->parameterCount()) * 4,
                                  static_cast<cudaStream_t>(stream)), "cudaMemsetAsync");
    QMLP_CATCH
}

int qmlp_encoding_compile(qmlp_encoding_t* enc, int half_table)
{
    QMLP_TRY
    enc->impl->standaloneModule(half_table != 0 && enc->impl->isGrid());
    QMLP_CATCH
}

static void encodingArgs(Encoding& e, kernel::LaunchArgs& a, const qmlp_tensor_t* input)
{
    std::memset(&a, 0, sizeof a);
    a.numel = input->sizes[0];
    a.input = static_cast<const float*>(input->data);
    a.inS0 = input->strides[0];
    a.inS1 = input->strides[1];
    a.numSMs = Library::instance().smCount();
    if (e.isGrid()) {
        if (!e.paramInference.defined()) throw std::runtime_error("the encoding has parameters but none are bound");
        e.fillGrid(a.grids[0]);
        a.numGrids = 1;
    }
}

int qmlp_encoding_forward(qmlp_encoding_t* enc, const qmlp_tensor_t* input, qmlp_tensor_t* output, qmlp_stream_t stream,
                          const qmlp_tensor_t* parameters)
{
    QMLP_TRY
    Encoding& e = *enc->impl;
    // src_cpp/src/iencoding.cpp:15-24
    checkDim(input, 2, "input");
    checkDim(output, 2, "output");
    checkDtype(input, QMLP_FLOAT, "input");
    checkDtype(output, QMLP_FLOAT, "output");
    checkSize(output, 0, input->sizes[0], "output");
    if (!(input->sizes[1] > e.maxInputChannel())) throw std::runtime_error("input has too few channels for this encoding");
    if (!(output->sizes[1] >= e.numOutputChannels())) throw std::runtime_error("output has too few channels for this encoding");
    if (output->strides[1] != 1) throw std::runtime_error("The output stride along the channels must be 1");
    BoundTensor saved = e.paramInference;
    const bool overwrite = e.hasParameters() && parameters != nullptr && parameters->ndim > 0;
    if (overwrite) e.setParameter(parameters, QMLP_INFERENCE);
    try {
        kernel::LaunchArgs a;
        encodingArgs(e, a, input);
        a.output = static_cast<float*>(output->data);
        a.outS0 = output->strides[0];
        a.outS1 = output->strides[1];
        if (a.numel > 0) {
            auto m = e.standaloneModule(e.paramInference.precision == QMLP_HALF && e.isGrid());
            checkLaunch(m->launch(kernel::KERNEL_ENCODING_FORWARD, &a, static_cast<cudaStream_t>(stream), nullptr), "kernel launch failed");
        }
    } catch (...) {
        if (overwrite) e.paramInference = saved;
        throw;
    }
    if (overwrite) e.paramInference = saved;
    QMLP_CATCH
}

int qmlp_encoding_adjoint(qmlp_encoding_t* enc, const qmlp_tensor_t* input, const qmlp_tensor_t* adj_output,
                          qmlp_tensor_t* adj_input, qmlp_stream_t stream, const qmlp_tensor_t* parameters,
                          qmlp_tensor_t* parameter_gradients, int adjoint_mode)
{
    QMLP_TRY
    Encoding& e = *enc->impl;
    // src_cpp/src/iencoding.cpp:101-118
    checkDim(input, 2, "input");
    checkDim(adj_output, 2, "adjOutput");
    checkDtype(input, QMLP_FLOAT, "input");
    checkDtype(adj_output, QMLP_FLOAT, "adjOutput");
    checkSize(adj_output, 0, input->sizes[0], "adjOutput");
    if (!(input->sizes[1] > e.maxInputChannel())) throw std::runtime_error("input has too few channels for this encoding");
    if (!(adj_output->sizes[1] >= e.numOutputChannels())) throw std::runtime_error("adjOutput has too few channels for this encoding");
    const bool gIn = adjoint_mode & QMLP_ENCODING_INPUT_GRADIENTS;
    bool gP = (adjoint_mode & QMLP_ENCODING_PARAM_GRADIENTS) && e.hasParameters();
    if (gIn) {
        checkDim(adj_input, 2, "adjInput");
        checkDtype(adj_input, QMLP_FLOAT, "adjInput");
        checkSize(adj_input, 0, input->sizes[0], "adjInput");
        checkSize(adj_input, 1, input->sizes[1], "adjInput");
    }
    BoundTensor savedP = e.paramInference, savedG = e.paramGradients;
    const bool owP = e.hasParameters() && parameters != nullptr && parameters->ndim > 0;
    const bool owG = e.hasParameters() && parameter_gradients != nullptr && parameter_gradients->ndim > 0;
    try {
        if (owP) e.setParameter(parameters, QMLP_INFERENCE);
        if (owG) e.setParameter(parameter_gradients, QMLP_GRADIENTS);
        if (gP && !e.paramGradients.defined()) throw std::runtime_error("parameter gradients requested, but no gradient tensor is bound");
        kernel::LaunchArgs a;
        encodingArgs(e, a, input);
        a.adjOutput = static_cast<const float*>(adj_output->data);
        a.aoS0 = adj_output->strides[0];
        a.aoS1 = adj_output->strides[1];
        if (gIn) {
            a.adjInput = static_cast<float*>(adj_input->data);
            a.aiS0 = adj_input->strides[0];
            a.aiS1 = adj_input->strides[1];
        }
        a.flags = (gIn ? 1 : 0) | (gP ? 2 : 0);
        if (a.numel > 0 && a.flags != 0) {
            auto m = e.standaloneModule(e.paramInference.precision == QMLP_HALF && e.isGrid());
            checkLaunch(m->launch(kernel::KERNEL_ENCODING_ADJOINT, &a, static_cast<cudaStream_t>(stream), nullptr), "kernel launch failed");
        }
    } catch (...) {
        e.paramInference = savedP;
        e.paramGradients = savedG;
        throw;
    }
    e.paramInference = savedP;
    e.paramGradients = savedG;
    QMLP_CATCH
}

// ---- activations ---------------------------------------------------------------------------------------------------
int qmlp_activation_create(const char* key_or_json, qmlp_activation_t** out)
{
    QMLP_TRY
    if (!key_or_json || !out) throw std::runtime_error("null argument");
    ActivationFactory factory;
    *out = new qmlp_activation{factory.getOrInline(key_or_json)};
    QMLP_CATCH
}
void qmlp_activation_destroy(qmlp_activation_t* act) { delete act; }
const char* qmlp_activation_id(qmlp_activation_t* act) { return act->impl->id().c_str(); }
const char* qmlp_activation_to_json(qmlp_activation_t* act) { act->impl->jsonCache = act->impl->toJson().dump(); return act->impl->jsonCache.c_str(); }

int qmlp_activation_compile(qmlp_activation_t* act)
{
    QMLP_TRY
    act->impl->module();
    QMLP_CATCH
}

static void activationLaunch(qmlp_activation_t* act, int kernelId, const qmlp_tensor_t* input, const qmlp_tensor_t* adjOut,
                             qmlp_tensor_t* output, qmlp_stream_t stream)
{
    // src_cpp/src/activation.cpp:66-74, 108-120
    checkDim(input, 2, "input");
    checkDim(output, 2, "output");
    checkDtype(input, QMLP_HALF, "input");
    checkDtype(output, QMLP_HALF, "output");
    checkSize(output, 0, input->sizes[0], "output");
    checkSize(output, 1, input->sizes[1], "output");
    kernel::ActivationArgs a;
    std::memset(&a, 0, sizeof a);
    a.rows = input->sizes[0];
    a.cols = input->sizes[1];
    a.input = static_cast<const __half*>(input->data);
    a.inS0 = input->strides[0];
    a.inS1 = input->strides[1];
    a.output = static_cast<__half*>(output->data);
    a.outS0 = output->strides[0];
    a.outS1 = output->strides[1];
    if (adjOut) {
        checkDim(adjOut, 2, "adjOutput");
        checkDtype(adjOut, QMLP_HALF, "adjOutput");
        checkSize(adjOut, 0, input->sizes[0], "adjOutput");
        checkSize(adjOut, 1, input->sizes[1], "adjOutput");
        a.adjOutput = static_cast<const __half*>(adjOut->data);
        a.aoS0 = adjOut->strides[0];
        a.aoS1 = adjOut->strides[1];
    }
    if (a.rows * a.cols == 0) return;
    auto m = act->impl->module();
    checkLaunch(m->launch(kernelId, &a, static_cast<cudaStream_t>(stream), nullptr), "kernel launch failed");
}

int qmlp_activation_forward(qmlp_activation_t* act, const qmlp_tensor_t* input, qmlp_tensor_t* output, qmlp_stream_t stream)
{
    QMLP_TRY
    activationLaunch(act, kernel::KERNEL_ACTIVATION_FORWARD, input, nullptr, output, stream);
    QMLP_CATCH
}

int qmlp_activation_adjoint(qmlp_activation_t* act, const qmlp_tensor_t* input, const qmlp_tensor_t* adj_output,
                            qmlp_tensor_t* adj_input, qmlp_stream_t stream)
{
    QMLP_TRY
    activationLaunch(act, kernel::KERNEL_ACTIVATION_ADJOINT, input, adj_output, adj_input, stream);
    QMLP_CATCH
}

} // extern "C"

// ---- fused training step -------------------------------------------------------------------------------------------
// Workspace of one step, every part 256-byte aligned: forward stash and delta stash; dLoss/dOut; feature planes (forward
// features first, then their adjoints); the copies of points and targets in bin order and the bin tables of the
// spatially binned step (only for networks with a grid encoding).
struct TrainerLayout {
    size_t adjOut = 0, planes = 0, sortedInput = 0, sortedTarget = 0, bins = 0, total = 0;
    int binCount = 0;
};
static TrainerLayout trainerLayout(const Network& n, int64_t n32)
{
    auto align = [](size_t b) { return (b + 255) / 256 * 256; };
    TrainerLayout l;
    size_t b = align(static_cast<size_t>(n32) * (n.stashHalfsPerPoint() + n.deltaHalfsPerPoint()) * 2);
    l.adjOut = b;
    b = align(b + static_cast<size_t>(n32) * n.channelsOut() * 4);
    l.planes = b;
    b = align(b + adjointPlaneBytes(n, n32, QMLP_GRADIENTS_NETWORK_WEIGHTS | QMLP_GRADIENTS_INPUT_ENCODINGS));
    const int dims = n.sortDimensions();
    if (dims > 0) {
        l.binCount = kernel::sort_bin_count(dims);
        l.sortedInput = b;
        b = align(b + static_cast<size_t>(n32) * n.channelsIn() * 4);
        l.sortedTarget = b;
        b = align(b + static_cast<size_t>(n32) * n.channelsOut() * 4);
        l.bins = b;
        b = align(b + (static_cast<size_t>(l.binCount) * 3 + 1) * 4);
    }
    l.total = b;
    return l;
}

struct qmlp_trainer {
    std::shared_ptr<Network> net;
    qmlp_trainer_config_t cfg;
    std::vector<int64_t> segStart; // 0: network, 1+i: encoding i (-1 without parameters)
    int64_t fusedCount = 0;
    float *master = nullptr, *grad = nullptr, *m = nullptr, *v = nullptr;
    uint16_t* half = nullptr;
};

extern "C" {

int qmlp_trainer_create(qmlp_network_t* net, const qmlp_trainer_config_t* cfg, qmlp_trainer_t** out)
{
    QMLP_TRY
    if (!net || !cfg || !out) throw std::runtime_error("null argument");
    auto* t = new qmlp_trainer;
    t->net = net->impl;
    t->cfg = *cfg;
    // segments start on 64-element boundaries so that every table keeps vector alignment in all four buffers
    auto align = [](int64_t x) { return (x + 63) / 64 * 64; };
    int64_t pos = 0;
    t->segStart.push_back(0);
    pos = align(t->net->parameterCount());
    for (int i = 0; i < t->net->numEncodings(); ++i) {
        auto e = t->net->encoding(i);
        if (e->hasParameters()) { t->segStart.push_back(pos); pos = align(pos + e->parameterCount()); }
        else t->segStart.push_back(-1);
    }
    t->fusedCount = pos;
    *out = t;
    QMLP_CATCH
}

void qmlp_trainer_destroy(qmlp_trainer_t* tr) { delete tr; }
int64_t qmlp_trainer_fused_count(const qmlp_trainer_t* tr) { return tr->fusedCount; }
int64_t qmlp_trainer_segment_start(const qmlp_trainer_t* tr, int segment)
{
    if (segment < 0 || segment >= static_cast<int>(tr->segStart.size())) return -1;
    return tr->segStart[segment];
}

int qmlp_trainer_workspace_bytes(qmlp_trainer_t* tr, int64_t num_elements, size_t* bytes)
{
    QMLP_TRY
    const int64_t n32 = (num_elements + 31) / 32 * 32;
    *bytes = trainerLayout(*tr->net, n32).total;
    QMLP_CATCH
}

int qmlp_trainer_bind(qmlp_trainer_t* tr, float* master, float* gradient, float* adam_m, float* adam_v, uint16_t* half_copy)
{
    QMLP_TRY
    if (!master || !gradient || !adam_m || !adam_v || !half_copy) throw std::runtime_error("null buffer");
    for (const void* p : {static_cast<const void*>(master), static_cast<const void*>(gradient), static_cast<const void*>(adam_m),
                          static_cast<const void*>(adam_v), static_cast<const void*>(half_copy)})
        if ((reinterpret_cast<uintptr_t>(p) & 15) != 0) throw std::runtime_error("trainer buffers must be 16-byte aligned");
    tr->master = master; tr->grad = gradient; tr->m = adam_m; tr->v = adam_v; tr->half = half_copy;
    Network& n = *tr->net;
    qmlp_tensor_t t;
    std::memset(&t, 0, sizeof t);
    t.ndim = 1; t.strides[0] = 1;
    t.sizes[0] = n.parameterCount();
    t.data = half_copy; t.precision = QMLP_HALF;
    n.setParameter(&t, QMLP_INFERENCE);
    t.data = gradient; t.precision = QMLP_FLOAT;
    n.setParameter(&t, QMLP_GRADIENTS);
    for (int i = 0; i < n.numEncodings(); ++i) {
        auto e = n.encoding(i);
        if (!e->hasParameters()) continue;
        const int64_t s = tr->segStart[1 + i];
        t.sizes[0] = e->parameterCount();
        if (tr->cfg.grid_half_copy) { t.data = half_copy + s; t.precision = QMLP_HALF; }
        else { t.data = master + s; t.precision = QMLP_FLOAT; }
        e->setParameter(&t, QMLP_INFERENCE);
        t.data = gradient + s; t.precision = QMLP_FLOAT;
        e->setParameter(&t, QMLP_GRADIENTS);
    }
    QMLP_CATCH
}

int qmlp_trainer_refresh_half(qmlp_trainer_t* tr, qmlp_stream_t stream)
{
    QMLP_TRY
    if (!tr->master) throw std::runtime_error("trainer buffers are not bound");
    {
        TimedLaunch timed(KERNEL_ID_REFRESH_HALF, static_cast<cudaStream_t>(stream));
        checkCuda(kernel::launchRefreshHalf(tr->master, tr->half, tr->fusedCount, Library::instance().smCount(),
                                            static_cast<cudaStream_t>(stream)), "refresh_half");
    }
    tr->net->launchCount += 1;
    QMLP_CATCH
}

int qmlp_trainer_gradients(qmlp_trainer_t* tr, const qmlp_tensor_t* input, const qmlp_tensor_t* target, int64_t global_points,
                           void* workspace, size_t workspace_bytes, float* loss_sum, qmlp_stream_t stream)
{
    return qmlp_trainer_gradients_part(tr, input, target, global_points, workspace, workspace_bytes, loss_sum, 3, stream);
}

int qmlp_trainer_gradients_part(qmlp_trainer_t* tr, const qmlp_tensor_t* input, const qmlp_tensor_t* target, int64_t global_points,
                                void* workspace, size_t workspace_bytes, float* loss_sum, int parts, qmlp_stream_t stream)
{
    QMLP_TRY
    const int what = parts & 0xff;
    const int levelBegin = (parts >> 8) & 0xff, levelEnd = (parts >> 16) & 0xff;
    if (!(what == 1 || what == 2 || what == 3 || what == 4 || what == 8))
        throw std::runtime_error("parts must be 1 (up to the table gradients), 2 (weight gradients), 3 (both), 4 (up to the adjoint "
                                 "feature planes, scatter deferred) or 8 | first << 8 | end << 16 (scatter of a range of grid levels)");
    if (!tr->master) throw std::runtime_error("trainer buffers are not bound");
    Network& n = *tr->net;
    std::lock_guard<std::mutex> lock(n.mutex);
    checkIO(n, input, target, "target");
    const int64_t numel = input->sizes[0];
    size_t need = 0;
    qmlp_trainer_workspace_bytes(tr, numel, &need);
    if (workspace_bytes < need) throw std::runtime_error(format("workspace too small: %zu bytes given, %zu needed", workspace_bytes, need));
    if (!workspace || (reinterpret_cast<uintptr_t>(workspace) & 255) != 0) throw std::runtime_error("workspace must be 256-byte aligned");
    if (global_points <= 0) global_points = numel;
    const int64_t n32 = (numel + 31) / 32 * 32;
    const TrainerLayout lay = trainerLayout(n, n32);
    kernel::LaunchArgs a;
    fillCommon(n, a, input);
    unsigned char* ws = static_cast<unsigned char*>(workspace);
    a.fwdTmp = reinterpret_cast<__half*>(ws);
    a.adjTmp = a.fwdTmp + static_cast<size_t>(n32) * n.stashHalfsPerPoint();
    float* adjOut = reinterpret_cast<float*>(ws + lay.adjOut);
    // forward with stash; the output slot receives dLoss/dOut = 2 (out - target) / (global_points * C)
    a.output = adjOut;
    a.outS0 = n.channelsOut();
    a.outS1 = 1;
    a.target = static_cast<const float*>(target->data);
    a.tS0 = target->strides[0];
    a.tS1 = target->strides[1];
    a.lossScale = static_cast<float>(2.0 / (static_cast<double>(global_points) * n.channelsOut()));
    a.lossSum = loss_sum;
    bool anyGrid = false;
    for (int i = 0; i < n.numEncodings(); ++i) anyGrid = anyGrid || n.encoding(i)->hasParameters();
    __half* planes = anyGrid ? reinterpret_cast<__half*>(ws + lay.planes) : nullptr;
    // Gather-dominated batches (same rule as inference): the encodings are computed one grid level at a time into
    // the plane region of the workspace, which is free until the backward kernel writes the adjoint planes there,
    // and the forward kernel reads its layer-0 operand from the planes.
    const Library& lib = Library::instance();
    const int path = lib.kernelPath;
    const bool wantPlanes = planes != nullptr && !n.planesUnsupported && a.numGrids > 0 && numel > 0 &&
                            (path == 2 || (path == 0 && n.gathersPerPoint() >= 96 && numel >= (1 << 18)));
    // Spatially sorted step (kernels/sorted_scatter.cuh), on request only (qmlp_set_tuning("sort_points", 1)): the points
    // and targets are copied into bin order first and every kernel of the step works on the copies. Measured on the
    // 3-D hash-grid benchmark network (2^20 uniformly random points): the gather gets quicker (289 -> 227 us) and the
    // scatter sends a quarter fewer reductions, but reductions of neighbouring points arrive at the L2 together and
    // queue up behind each other on the same sectors (scatter 538 -> 639 us), and the sort itself takes 70 to 140 us: a
    // net loss for random batches, so it is not chosen automatically.
    const bool wantSort = lay.binCount > 0 && !n.sortUnsupported && path != 1 && numel > 0 && lib.sortPoints == 1;
    bool sorted = false;
    if (wantSort) {
        a.binCounts = reinterpret_cast<unsigned int*>(ws + lay.bins);
        a.binStart = a.binCounts + lay.binCount;
        a.binCursor = a.binStart + lay.binCount + 1;
        a.sortedInput = reinterpret_cast<float*>(ws + lay.sortedInput);
        a.sortedTarget = reinterpret_cast<float*>(ws + lay.sortedTarget);
        a.runAggregation = lib.runAggregation;
        if (what & 5) {
            auto m = n.module(n.currentHalfMask());
            int launches = 0;
            int e;
            {
                TimedLaunch timed(kernel::KERNEL_SORT_POINTS, static_cast<cudaStream_t>(stream));
                e = m->launch(kernel::KERNEL_SORT_POINTS, &a, static_cast<cudaStream_t>(stream), &launches);
            }
            if (e == static_cast<int>(cudaErrorNotSupported)) {
                n.sortUnsupported = true;
            } else {
                checkLaunch(e, "kernel launch failed");
                n.launchCount += launches;
                sorted = true;
            }
        } else {
            sorted = true;   // the first part of this step sorted; the kernels of the second part read no points
        }
        if (sorted) {
            a.input = a.sortedInput;
            a.inS0 = n.channelsIn();
            a.inS1 = 1;
            a.target = a.sortedTarget;
            a.tS0 = n.channelsOut();
            a.tS1 = 1;
        }
    }
    if (what & 5) {
        bool done = false;
        if (wantPlanes) {
            a.planes = planes;
            a.planeStride = n32;
            auto m = n.module(n.currentHalfMask());
            int launches = 0;
            int e;
            {
                TimedLaunch timed(kernel::KERNEL_ENCODE_PLANES, static_cast<cudaStream_t>(stream));
                const kernel::LaunchArgs sized = withScratchSizes(n, a);
                e = m->launch(kernel::KERNEL_ENCODE_PLANES, &sized, static_cast<cudaStream_t>(stream), &launches);
            }
            if (e == static_cast<int>(cudaErrorNotSupported)) {
                n.planesUnsupported = true;
            } else {
                checkLaunch(e, "kernel launch failed");
                n.launchCount += launches;
                launchNet(n, kernel::KERNEL_FORWARD_LOSS_PLANES, a, stream);
                done = true;
            }
        }
        if (!done) launchNet(n, kernel::KERNEL_FORWARD_LOSS, a, stream);
    }
    a.adjOutput = adjOut;
    a.aoS0 = n.channelsOut();
    a.aoS1 = 1;
    a.flags = kernel::FLAG_GRAD_WEIGHTS | (anyGrid ? kernel::FLAG_GRAD_ENCODINGS : 0);
    if (what == 1 || what == 3) launchBackward(n, a, planes, n32, stream, sorted);
    if (what == 4) {
        if (sorted || !splitScatterChosen(n, a, planes != nullptr, sorted))
            throw std::runtime_error("the scatter of this network is not a kernel of its own (qmlp_trainer_scatter_levels returns 0): use parts = 1");
        launchBackward(n, a, planes, n32, stream, sorted, /*scatterNow=*/false);
    }
    if (what == 8) {
        if (sorted || !splitScatterChosen(n, a, planes != nullptr, sorted))
            throw std::runtime_error("the scatter of this network is not a kernel of its own (qmlp_trainer_scatter_levels returns 0)");
        if (levelEnd <= levelBegin) throw std::runtime_error("empty range of grid levels");
        a.flags |= kernel::FLAG_SPLIT_SCATTER;
        a.planes = planes;
        a.planeStride = n32;
        a.scatterLevelBegin = levelBegin;
        a.scatterLevelEnd = levelEnd;
        launchNet(n, kernel::KERNEL_SCATTER_PLANES, a, stream);
    }
    if (what & 2) launchNet(n, kernel::KERNEL_WGRAD, a, stream);
    QMLP_CATCH
}

int qmlp_trainer_scatter_levels(qmlp_trainer_t* tr, int max_levels, int64_t* fused_begin, int64_t* fused_end)
{
    // levels of all plain grids in scatter order with their element ranges in the fused vectors; 0 when the table
    // gradients are not scattered by a kernel of their own (rows wider than two features, a line integration, the
    // mma.sync-only kernel path, the sorted step)
    Network& n = *tr->net;
    const Library& lib = Library::instance();
    if (lib.kernelPath == 1 || lib.sortPoints == 1 || lib.splitScatter == 0) return 0;
    bool two = true, any = false;
    for (int i = 0; i < n.numEncodings(); ++i)
        if (auto* g = dynamic_cast<EncodingHashGrid*>(n.encoding(i).get())) {
            if (g->isLine()) return 0;
            two = two && g->features() == 2;
            any = true;
        }
    if (!any || (!two && lib.splitScatter != 1)) return 0;
    int count = 0;
    for (int i = 0; i < n.numEncodings(); ++i) {
        auto* g = dynamic_cast<EncodingHashGrid*>(n.encoding(i).get());
        if (!g) continue;
        const auto& t = g->levelTable();
        const int64_t seg = tr->segStart[1 + i];
        for (size_t l = 0; l < t.size(); ++l, ++count) {
            if (count >= max_levels) continue;
            if (fused_begin) fused_begin[count] = seg + t[l].memoryOffset;
            if (fused_end) fused_end[count] = seg + (l + 1 < t.size() ? t[l + 1].memoryOffset : g->parameterCount());
        }
    }
    return count;
}

int qmlp_trainer_update(qmlp_trainer_t* tr, int64_t step, float grad_scale, qmlp_stream_t stream)
{
    QMLP_TRY
    if (!tr->master) throw std::runtime_error("trainer buffers are not bound");
    if (step < 1) throw std::runtime_error("step is 1-based");
    const double bc1 = 1.0 - std::pow(static_cast<double>(tr->cfg.beta1), static_cast<double>(step));
    const double bc2 = 1.0 - std::pow(static_cast<double>(tr->cfg.beta2), static_cast<double>(step));
    {
        TimedLaunch timed(KERNEL_ID_ADAM, static_cast<cudaStream_t>(stream));
        checkCuda(kernel::launchAdam(tr->master, tr->grad, tr->m, tr->v, tr->half, tr->fusedCount, grad_scale, tr->cfg.beta1,
                                     tr->cfg.beta2, static_cast<float>(tr->cfg.learning_rate / bc1),
                                     static_cast<float>(1.0 / std::sqrt(bc2)), tr->cfg.epsilon, Library::instance().smCount(),
                                     static_cast<cudaStream_t>(stream)), "adam");
    }
    tr->net->launchCount += 1;
    QMLP_CATCH
}

} // extern "C"
