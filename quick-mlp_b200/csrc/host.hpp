// Host-side model of a fused network: activations, encodings, layer chain, parameter layout, and the per-spec
// kernel instantiation handle. Mirrors the reference classes behind the C ABI:
//   qmlp::Activation / ActivationFactory   src_cpp/include/qmlp/activation.h:29-147
//   qmlp::IEncoding / EncodingIdentity / EncodingHashGrid / EncodingFactory
//                                          src_cpp/include/qmlp/iencoding.h:36-201, encoding_hashgrid.h:45-127
//   qmlp::FusedNetwork                     src_cpp/include/qmlp/fused_network.h:16-340
#pragma once
#include <cstdint>
#include <map>
#include <memory>
#include <mutex>
#include <string>
#include <vector>

#include "json.hpp"
#include "kernels/launch_args.h"
#include "../../include/qmlp_b200.h"

namespace qmlp {

class cuda_error : public std::runtime_error {
public:
    explicit cuda_error(const std::string& m) : std::runtime_error(m) {}
};
class compile_error : public std::runtime_error {
public:
    explicit compile_error(const std::string& m) : std::runtime_error(m) {}
};

std::string format(const char* fmt, ...);
void logMessage(int level, const std::string& msg); // 0 debug, 1 info, 2 warn, 3 error
inline int roundUp(int x, int m) { return ((x + m - 1) / m) * m; }

// ---- library-wide state (QuickMLP singleton, src_cpp/include/qmlp/qmlp.h:14-94) -------------------------------------
struct Library {
    static Library& instance();
    std::mutex mutex;
    int logLevel = 1;
    bool debugMode = false;
    std::string cacheDir;   // per-spec instantiations (.cu + .so)
    std::string includeDir; // kernel template headers
    std::string nvcc;
    std::string resolveCacheDir();
    std::string resolveIncludeDir();
    int smCount(); // of the current device
    int kernelPath = 0;    // 0: best kernels for the spec, 1: mma.sync kernels only
    // tuning switches of the training step (qmlp_set_tuning): -1 = decided per network and batch
    int sortPoints = -1;      // spatially sorted step (kernels/sorted_scatter.cuh): 1 on whenever instantiated, else off
    int splitScatter = -1;    // table-gradient scatter as its own kernel: 0 inside the backward kernel, 1 separate
    int runAggregation = 1;   // coarse levels of the sorted scatter: corner sums of a run of points in one cell kept in registers
    // kernels instantiated with QMLP_BOUNDS_CHECK: every table row, stash offset and plane offset is tested against the
    // size the host declares; an access outside is skipped and reported through the status word
    bool boundsCheck = false;
    int64_t boundsShrink = 0; // test hook: declare tables and scratch buffers this many elements smaller than they are
    int* statusWord();     // device word of the current device that kernels set when a bounded wait gives up
};

// ---- per-spec kernel instantiation ------------------------------------------------------------------------------
struct KernelModule {
    std::string name;
    void* handle = nullptr;
    qmlp_spec_launch_fn launch = nullptr;
};
// Finds (cache) or builds (nvcc) and loads the shared object instantiating `source`.
std::shared_ptr<KernelModule> getKernelModule(const std::string& kind, const std::string& source);

// ---- activations ---------------------------------------------------------------------------------------------------
class Activation {
public:
    Activation(const std::string& id, const std::string& forward, const std::string& adjoint);
    explicit Activation(const Json& cfg);
    const std::string& id() const { return id_; }
    const std::string& forward() const { return forward_; }
    const std::string& adjoint() const { return adjoint_; }
    // name of the device functor type and, for non built-in snippets, its definition
    std::string functorName() const;
    std::string functorDefinition() const;
    bool isBuiltin() const { return builtin_; }
    Json toJson() const;
    std::shared_ptr<KernelModule> module(); // stand-alone kernels, built lazily
    std::string jsonCache;

private:
    std::string id_, forward_, adjoint_;
    bool builtin_ = false;
    std::shared_ptr<KernelModule> module_;
};
typedef std::shared_ptr<Activation> Activation_ptr;

class ActivationFactory {
public:
    // src_cpp/src/activation.cpp:152-210
    ActivationFactory(const Json& cfg, const std::string& parent);
    ActivationFactory(); // built-ins only
    Activation_ptr get(const std::string& key) const;
    Activation_ptr getOrInline(const std::string& key);

private:
    void parseArray(const Json& j);
    void parseFile(const std::string& path);
    std::map<std::string, Activation_ptr> activations_;
};
const char* builtinActivationsJson();

// ---- encodings -----------------------------------------------------------------------------------------------------
struct BoundTensor {
    void* data = nullptr;
    int precision = QMLP_FLOAT;
    bool defined() const { return data != nullptr; }
};

class Encoding {
public:
    virtual ~Encoding() = default;
    virtual Json toJson() const = 0;
    virtual std::string id() const = 0;
    virtual int maxInputChannel() const = 0;
    virtual int numOutputChannels() const = 0;
    virtual bool hasParameters() const { return false; }
    virtual int64_t parameterCount() const { return 0; }
    virtual bool isGrid() const { return false; }   // owns a grid table (a slot of LaunchArgs::grids)
    virtual bool isLine() const { return false; }   // line integration over its grid
    // C++ type of the device-side descriptor, e.g. "EncGrid<0,3,16,2,true,0,0,false>"
    virtual std::string deviceType(int outOffset, int slot, bool halfTable) const = 0;
    virtual void setParameter(const qmlp_tensor_t* t, int usage);
    virtual void fillGrid(kernel::GridP& g) const {}
    std::shared_ptr<KernelModule> standaloneModule(bool halfTable);

    BoundTensor paramInference, paramGradients;
    std::string jsonCache, idCache;

private:
    std::shared_ptr<KernelModule> standalone_[4];   // [fp32 | fp16 table] x [regular | bounds-checking]
};
typedef std::shared_ptr<Encoding> Encoding_ptr;

class EncodingIdentity : public Encoding {
public:
    explicit EncodingIdentity(const Json& cfg);
    Json toJson() const override;
    std::string id() const override { return "Identity"; }
    int maxInputChannel() const override { return start_ + n_ - 1; }
    int numOutputChannels() const override { return n_; }
    std::string deviceType(int outOffset, int slot, bool halfTable) const override;

private:
    int start_, n_;
};

struct GridLevel {
    int64_t memoryOffset;
    int resolution;
    int hashGridSize;
    bool hashed;
};

class EncodingHashGrid : public Encoding {
public:
    explicit EncodingHashGrid(const Json& cfg);
    Json toJson() const override;
    std::string id() const override { return "HashGrid"; }
    int maxInputChannel() const override { return start_ + dim_ - 1; }
    int numOutputChannels() const override { return concat_ ? levels_ * features_ : features_; }
    bool hasParameters() const override { return true; }
    int64_t parameterCount() const override { return numParameters_; }
    bool isGrid() const override { return true; }
    std::string deviceType(int outOffset, int slot, bool halfTable) const override;
    void setParameter(const qmlp_tensor_t* t, int usage) override;
    void fillGrid(kernel::GridP& g) const override;
    const std::vector<GridLevel>& levelTable() const { return table_; }
    int features() const { return features_; }
    int dimension() const { return dim_; }
    Json gridJson() const;   // the hash grid's own configuration (id "HashGrid")

protected:
    int start_, dim_, levels_, features_, log2Hashmap_, hashmapSize_, minRes_, maxRes_;
    bool concat_;
    bool hasScale_ = false;
    double perLevelScale_ = 0;
    std::vector<float> boxMin_, boxSize_, boxInvSize_;
    std::vector<GridLevel> table_;
    int64_t numParameters_ = 0;
};

// EncodingLineIntegration, src_cpp/include/qmlp/encoding_line_integration.h / src_cpp/src/encoding_line_integration.cpp:
// ray start + direction in, the child volume (a hash grid on the sample position) integrated along the ray out.
// The child's table is this encoding's parameter.
class EncodingLineIntegration : public EncodingHashGrid {
public:
    explicit EncodingLineIntegration(const Json& cfg);
    Json toJson() const override;
    std::string id() const override { return "LineIntegration"; }
    int maxInputChannel() const override { return rayStart_ + dim_ * 2 - 1; }
    bool isLine() const override { return true; }
    std::string deviceType(int outOffset, int slot, bool halfTable) const override;
    void fillGrid(kernel::GridP& g) const override;

private:
    int rayStart_;
    float stepsize_;
    bool average_;
};

Encoding_ptr createEncoding(const Json& cfg); // EncodingFactory::create, src_cpp/src/iencoding.cpp:221-228

// ---- network -------------------------------------------------------------------------------------------------------
struct LayerSpec {
    int channelsIn = 0, channelsOut = 0;
    bool useBias = false;
    Activation_ptr activation;                   // the layer's activation, or the first entry of a per-channel array
    std::vector<Activation_ptr> perChannel;      // one per (unpadded) output channel when the array is not uniform
    int64_t weightsStart = 0, biasStart = -1;
};

// Device staging of the host-memory inference entry point: three chunk slots (input + output), an upload and a
// download stream, and the events that chain upload -> kernel -> download per slot. Created at the first such call on a
// network, grown when a larger chunk is asked for, released with the network.
struct HostPipeline {
    static constexpr int SLOTS = 3;
    cudaStream_t copyIn = nullptr, copyOut = nullptr;
    cudaEvent_t start = nullptr;
    cudaEvent_t uploaded[SLOTS] = {}, computed[SLOTS] = {}, downloaded[SLOTS] = {};
    float* in[SLOTS] = {};
    float* out[SLOTS] = {};
    int64_t capacity = 0;   // points per slot
    void reserve(int64_t points, int channelsIn, int channelsOut);
    void release();
};

class Network {
public:
    Network(const Json& cfg, const std::string& parent);
    int channelsIn() const { return channelsIn_; }
    int channelsOut() const { return channelsOut_; }
    int numLayers() const { return static_cast<int>(layers_.size()); }
    int numEncodings() const { return static_cast<int>(encodings_.size()); }
    int64_t parameterCount() const { return numParameters_; }
    const LayerSpec& layer(int i) const { return layers_.at(i); }
    Encoding_ptr encoding(int i) const;
    int encodedChannels() const { return encodedChannels_; }
    int stashHalfsPerPoint() const;   // encoded input + all pre-activations
    int deltaHalfsPerPoint() const;   // all deltas

    void setParameter(const qmlp_tensor_t* t, int usage);
    void initializeHost(uint64_t seed, uint16_t* dst) const;
    std::string generateSource(unsigned halfMask) const;
    std::shared_ptr<KernelModule> module(unsigned halfMask);
    unsigned currentHalfMask() const;
    void fillGrids(kernel::LaunchArgs& a) const;
    void clearModules();

    ~Network();
    int64_t gridTableBytes() const;   // bytes of all bound grid tables (what the gather walks through)
    int gathersPerPoint() const;      // table rows fetched per point by all plain grid encodings: sum of levels * 2^D
    int sortDimensions() const;       // dimension of the grid whose bounding box bins the points of a training step (0: none)
    // level-major encoding pass (inference of networks with tables larger than L2): chunk buffer, allocated at the
    // first such call and kept until the network is destroyed
    void* planes = nullptr;
    int64_t planeCapacity = 0;        // points per chunk
    bool planesUnsupported = false;   // the spec has no instantiation of the plane kernels
    bool sortUnsupported = false;     // the spec has no instantiation of the point sort
    HostPipeline hostPipeline;
    int ownedDevice = -1;             // device the library-owned buffers above live on (-1: none allocated yet)
    void claimDevice();               // first call: remember the current device; later calls: it must be the same

    BoundTensor paramInference, paramGradients;
    std::vector<qmlp_encoding*> encodingHandles; // owned wrappers handed out through the C ABI
    int64_t launchCount = 0;
    std::mutex mutex;

private:
    int channelsIn_, channelsOut_;
    int encodedChannels_ = 0;
    int64_t numParameters_ = 0;
    std::vector<Encoding_ptr> encodings_;
    std::vector<LayerSpec> layers_;
    std::map<unsigned, std::shared_ptr<KernelModule>> modules_;
};

// Used by entry points that live outside capi.cpp: record an error for qmlp_last_error() and return its code;
// run forward-with-stash with the stash at `tmp` (argument checks and launch exactly as qmlp_network_forward).
int reportError(int code, const char* message);
void forwardWithStashAt(Network& net, const qmlp_tensor_t* input, qmlp_tensor_t* output, void* tmp, qmlp_stream_t stream);

} // namespace qmlp

// opaque C handles
struct qmlp_network { std::shared_ptr<qmlp::Network> impl; };
struct qmlp_encoding { qmlp::Encoding_ptr impl; };
struct qmlp_activation { qmlp::Activation_ptr impl; };
