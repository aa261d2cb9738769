// qmlp::FusedNetwork (src_cpp/include/qmlp/fused_network.h:16-340) over the C ABI: the reference's public methods with
// their argument order and meaning, each a forwarding call into libqmlp_b200.so. The kernels, the per-spec
// instantiation and the parameter layout live behind qmlp_b200.h.
#pragma once
#include <filesystem>
#include <memory>
#include <random>
#include <string>
#include <vector>

#include <cuda.h>

#include "iencoding.h"
#include "qmlp.h"
#include "tmp_memory.h"

namespace qmlp {

class FusedNetwork {
public:
    // additive flags: what adjoint() differentiates with respect to (fused_network.h:22-34)
    enum AdjointMode {
        GRADIENTS_INPUT = 0x1,
        GRADIENTS_NETWORK_WEIGHTS = 0x2,
        GRADIENTS_INPUT_ENCODINGS = 0x4,
        ADJOINT_MODE_MAX_COMBINATIONS = 8
    };
    typedef int AdjointModeFlags;

    static constexpr int MATRIX_SIZE = 16;
    static constexpr int WARP_SIZE = 32;
    static constexpr int MAX_SHARED_MEMORY_BYTES = 227 * 1024;

    // cfg: the JSON text of the network specification; parent: the folder activation files are resolved against
    // (fused_network.h:149-156)
    FusedNetwork(const std::string& cfgJson, const std::filesystem::path& parent)
    {
        qmlp_network_t* h = nullptr;
        detail::check(qmlp_network_create(cfgJson.c_str(), parent.string().c_str(), &h));
        handle_.reset(h, qmlp_network_destroy);
        const int n = qmlp_network_num_encodings(h);
        for (int i = 0; i < n; ++i) {
            qmlp_encoding_t* e = nullptr;
            detail::check(qmlp_network_encoding(h, i, &e));
            encodings_.push_back(IEncoding_ptr(new IEncoding(e, handle_)));
        }
    }
#ifdef QMLP_HAS_NLOHMANN_JSON
    FusedNetwork(const nlohmann::json& cfg, const std::filesystem::path& parent) : FusedNetwork(cfg.dump(), parent) {}
#endif
    FusedNetwork(const FusedNetwork&) = delete;
    FusedNetwork& operator=(const FusedNetwork&) = delete;

    const std::vector<IEncoding_ptr>& encodings() const { return encodings_; }
    int numEncodings() const { return static_cast<int>(encodings_.size()); }
    IEncoding_ptr encoding(int idx)
    {
        if (idx < 0 || idx >= numEncodings()) throw std::runtime_error("Array index out of bounds");
        return encodings_[idx];
    }
    int channelsIn() const { return qmlp_network_channels_in(handle_.get()); }
    int channelsOut() const { return qmlp_network_channels_out(handle_.get()); }
    Tensor::Precision precisionIn() const { return Tensor::FLOAT; }
    Tensor::Precision precisionOut() const { return Tensor::FLOAT; }
    int numLayers() const { return qmlp_network_num_layers(handle_.get()); }

    int networkParameterCount() const { return static_cast<int>(qmlp_network_parameter_count(handle_.get())); }
    // INFERENCE: half, GRADIENTS: float (src_cpp/src/fused_network.cpp:247-255)
    Tensor::Precision networkParameterPrecision(Tensor::Usage usage) const
    {
        return qmlp_network_parameter_precision(handle_.get(), usage) == QMLP_HALF ? Tensor::HALF : Tensor::FLOAT;
    }
    // binds the flat parameter vector (INFERENCE) or the gradient vector (GRADIENTS); the memory stays the caller's
    void setNetworkParameter(const Tensor& tensor, Tensor::Usage usage)
    {
        const qmlp_tensor_t t = tensor.view();
        detail::check(qmlp_network_set_parameter(handle_.get(), &t, usage));
        (usage == Tensor::INFERENCE ? parametersInference_ : parametersGradients_) = tensor;
    }
    // U(+-1/sqrt(fan_in)) over the bound inference parameters (src_cpp/src/fused_network.cpp:280-312); the library draws
    // from its own portable generator seeded with one value of `rng`
    void initializeInferenceParameters(std::default_random_engine& rng)
    {
        detail::check(qmlp_network_initialize_parameters(handle_.get(), static_cast<uint64_t>(rng())));
    }
    // view of one layer's weight matrix (Cout x Cin, row-major) or bias (Cout) inside a flat vector at rawPtr
    // (fused_network.h:189-219)
    Tensor networkParameter(int layer, bool bias, void* rawPtr, Tensor::Precision precision)
    {
        int cin = 0, cout = 0, useBias = 0;
        int64_t ws = 0, bs = 0;
        detail::check(qmlp_network_layer_info(handle_.get(), layer, &cin, &cout, &useBias, &ws, &bs));
        char* base = static_cast<char*>(rawPtr);
        const int b = Tensor::bytesPerEntryOf(precision);
        if (bias) {
            if (!useBias) return Tensor();
            return Tensor(base + bs * b, precision, {cout}, {1});
        }
        return Tensor(base + ws * b, precision, {cout, cin}, {cin, 1});
    }
    Tensor networkParameter(int layer, bool bias, Tensor::Usage usage)
    {
        Tensor& p = usage == Tensor::INFERENCE ? parametersInference_ : parametersGradients_;
        if (!p.defined()) throw std::runtime_error("no parameter tensor is bound for this usage (setNetworkParameter)");
        return networkParameter(layer, bias, p.rawPtr(), p.precision());
    }

    // fused inference: fp32 (N, channelsIn) -> fp32 (N, channelsOut) (fused_network.h:221-227)
    void inference(const Tensor& input, Tensor& output, CUstream stream)
    {
        const qmlp_tensor_t in = input.view();
        qmlp_tensor_t out = output.view();
        detail::check(qmlp_network_inference(handle_.get(), &in, &out, stream));
    }
    // bytes of scratch forward() fills for adjoint() (fused_network.h:229-247)
    size_t forwardMemory(int numElements, AdjointModeFlags adjointFlags)
    {
        size_t bytes = 0;
        detail::check(qmlp_network_forward_memory(handle_.get(), numElements, adjointFlags, &bytes));
        return bytes;
    }
    size_t forwardMemory(const Tensor& input, AdjointModeFlags adjointFlags) { return forwardMemory(input.size(0), adjointFlags); }
    void forward(const Tensor& input, Tensor& output, void* tmpMemory, CUstream stream)
    {
        const qmlp_tensor_t in = input.view();
        qmlp_tensor_t out = output.view();
        detail::check(qmlp_network_forward(handle_.get(), &in, &out, tmpMemory, stream));
    }
    // clears the bound gradient tensors of the network and of its encodings (fused_network.h:261-265)
    void zeroGradients()
    {
        detail::check(qmlp_network_zero_gradients(handle_.get(), nullptr));
        cudaStreamSynchronize(nullptr);   // the reference's cudaMemset is synchronous
    }
    size_t adjointMemory(int numElements, AdjointModeFlags adjointFlags)
    {
        size_t bytes = 0;
        detail::check(qmlp_network_adjoint_memory(handle_.get(), numElements, adjointFlags, &bytes));
        return bytes;
    }
    size_t adjointMemory(const Tensor& input, AdjointModeFlags adjointFlags) { return adjointMemory(input.size(0), adjointFlags); }
    // gradients are added to the bound gradient tensors and to adjInput (fused_network.h:289-311)
    void adjoint(const Tensor& input, const Tensor& adjOutput, AdjointModeFlags adjointFlags, Tensor& adjInput,
                 const void* tmpMemoryForward, void* tmpMemoryAdjoint, CUstream stream)
    {
        const qmlp_tensor_t in = input.view(), ao = adjOutput.view();
        qmlp_tensor_t ai = adjInput.view();
        detail::check(qmlp_network_adjoint(handle_.get(), &in, &ao, adjointFlags, &ai, tmpMemoryForward, tmpMemoryAdjoint, stream));
    }
    void clearCachedKernels() { detail::check(qmlp_network_clear_cached_kernels(handle_.get())); }

    qmlp_network_t* handle() { return handle_.get(); }   // for the entry points that have no reference counterpart

private:
    std::shared_ptr<qmlp_network_t> handle_;
    std::vector<IEncoding_ptr> encodings_;
    Tensor parametersInference_, parametersGradients_;
};
typedef std::shared_ptr<FusedNetwork> FusedNetwork_ptr;

} // namespace qmlp
