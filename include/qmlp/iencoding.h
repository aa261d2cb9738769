// qmlp::IEncoding, EncodingFactory and the concrete encodings (src_cpp/include/qmlp/iencoding.h:36-201,
// encoding_identity.h:9-30, encoding_hashgrid.h:22-127, encoding_line_integration.h) over the C ABI. One class serves
// all encodings: which one it is follows from the "id" of its configuration, as in EncodingFactory::create
// (src_cpp/src/iencoding.cpp:221-228); the code-generation hooks of the reference interface (qualifiedName, fillCode,
// fillParameterConstant) have no meaning behind this interface and are not declared.
#pragma once
#include <memory>
#include <optional>
#include <string>
#include <vector>

#include <cuda.h>

#include "activation.h"

namespace qmlp {

class FusedNetwork;

class IEncoding {
public:
    enum AdjointMode { INPUT_GRADIENTS = 0x1, PARAM_GRADIENTS = 0x2, ALL_GRADIENTS = INPUT_GRADIENTS | PARAM_GRADIENTS };

    // from the JSON text of an encoding ({"id": "Identity" | "HashGrid" | "LineIntegration", ...})
    explicit IEncoding(const std::string& cfgJson)
    {
        qmlp_encoding_t* h = nullptr;
        detail::check(qmlp_encoding_create(cfgJson.c_str(), &h));
        handle_.reset(h, qmlp_encoding_destroy);
    }
#ifdef QMLP_HAS_NLOHMANN_JSON
    explicit IEncoding(const nlohmann::json& cfg) : IEncoding(cfg.dump()) {}
    nlohmann::json toJson() const { return nlohmann::json::parse(toJsonString()); }
#endif
    virtual ~IEncoding() = default;

    std::string toJsonString() const { return qmlp_encoding_to_json(handle_.get()); }
    std::string id() const { return qmlp_encoding_id(handle_.get()); }
    int maxInputChannel() const { return qmlp_encoding_max_input_channel(handle_.get()); }
    int numOutputChannels() const { return qmlp_encoding_num_output_channels(handle_.get()); }
    bool hasParameters() const { return qmlp_encoding_has_parameters(handle_.get()) != 0; }
    Tensor::Precision parameterPrecision(Tensor::Usage usage) const
    {
        return qmlp_encoding_parameter_precision(handle_.get(), usage) == QMLP_HALF ? Tensor::HALF : Tensor::FLOAT;
    }
    int parameterCount() const { return static_cast<int>(qmlp_encoding_parameter_count(handle_.get())); }
    // binds the inference table or the gradient table; the memory stays the caller's (iencoding.h:84-90)
    void setParameter(const Tensor& tensor, Tensor::Usage usage)
    {
        const qmlp_tensor_t t = tensor.view();
        detail::check(qmlp_encoding_set_parameter(handle_.get(), &t, usage));
    }
    void zeroGradients() { detail::check(qmlp_encoding_zero_gradients(handle_.get(), nullptr)); }

    // stand-alone encoding of fp32 (B, C) points into fp32 (B, >= numOutputChannels) (iencoding.h:107-115)
    void forward(const Tensor& input, Tensor& output, CUstream stream, const std::optional<const Tensor>& parametersForward = std::nullopt)
    {
        const qmlp_tensor_t in = input.view();
        qmlp_tensor_t out = output.view();
        qmlp_tensor_t p{};
        if (parametersForward) p = parametersForward->view();
        detail::check(qmlp_encoding_forward(handle_.get(), &in, &out, stream, parametersForward ? &p : nullptr));
    }
    void adjoint(const Tensor& input, const Tensor& adjOutput, Tensor& adjInput, CUstream stream,
                 const std::optional<const Tensor>& parametersForward = std::nullopt,
                 const std::optional<const Tensor>& parametersGradients = std::nullopt, int adjointMode = ALL_GRADIENTS)
    {
        const qmlp_tensor_t in = input.view(), ao = adjOutput.view();
        qmlp_tensor_t ai = adjInput.view(), p{}, g{};
        if (parametersForward) p = parametersForward->view();
        if (parametersGradients) g = parametersGradients->view();
        detail::check(qmlp_encoding_adjoint(handle_.get(), &in, &ao, &ai, stream, parametersForward ? &p : nullptr,
                                            parametersGradients ? &g : nullptr, adjointMode));
    }

    // level table of a grid encoding (src_cpp/src/encoding_hashgrid.cpp:41-97); empty for other encodings
    struct Level { int64_t memoryOffset; int resolution; int hashGridSize; bool hashed; };
    std::vector<Level> levels() const
    {
        const int n = qmlp_encoding_grid_levels(handle_.get(), 0, nullptr, nullptr, nullptr, nullptr);
        std::vector<int64_t> off(n);
        std::vector<int32_t> res(n), size(n), hashed(n);
        if (n > 0) qmlp_encoding_grid_levels(handle_.get(), n, off.data(), res.data(), size.data(), hashed.data());
        std::vector<Level> out(n);
        for (int i = 0; i < n; ++i) out[i] = Level{off[i], res[i], size[i], hashed[i] != 0};
        return out;
    }

protected:
    friend class FusedNetwork;
    // an encoding that belongs to a network: the network owns the handle
    IEncoding(qmlp_encoding_t* borrowed, std::shared_ptr<void> owner) : handle_(borrowed, [owner](qmlp_encoding_t*) {}) {}
    std::shared_ptr<qmlp_encoding_t> handle_;
};
typedef std::shared_ptr<IEncoding> IEncoding_ptr;

namespace detail {
inline void requireId(const IEncoding& e, const char* id)
{
    if (e.id() != id) throw configuration_error(std::string("the configuration describes a '") + e.id() + "' encoding, expected '" + id + "'");
}
} // namespace detail

class EncodingIdentity : public IEncoding {
public:
    static std::string ID() { return "Identity"; }
    explicit EncodingIdentity(const std::string& cfgJson) : IEncoding(cfgJson) { detail::requireId(*this, "Identity"); }
    EncodingIdentity(int startChannel, int numChannels)
        : IEncoding("{\"id\": \"Identity\", \"start_in\": " + std::to_string(startChannel) + ", \"n_in\": " + std::to_string(numChannels) + "}")
    {
    }
};

class EncodingHashGrid : public IEncoding {
public:
    static std::string ID() { return "HashGrid"; }
    explicit EncodingHashGrid(const std::string& cfgJson) : IEncoding(cfgJson) { detail::requireId(*this, "HashGrid"); }
    int numLevels() const { return static_cast<int>(levels().size()); }
};

class EncodingLineIntegration : public IEncoding {
public:
    static std::string ID() { return "LineIntegration"; }
    explicit EncodingLineIntegration(const std::string& cfgJson) : IEncoding(cfgJson) { detail::requireId(*this, "LineIntegration"); }
};

class EncodingFactory {
    EncodingFactory() = default;

public:
    static EncodingFactory& Instance()
    {
        static EncodingFactory f;
        return f;
    }
    IEncoding_ptr create(const std::string& cfgJson) { return std::make_shared<IEncoding>(cfgJson); }
#ifdef QMLP_HAS_NLOHMANN_JSON
    IEncoding_ptr create(const nlohmann::json& cfg) { return create(cfg.dump()); }
#endif
};

} // namespace qmlp
