// TorchScript custom classes torch.classes.qmlp_cu.{QuickMLP, Network, Encoding, Activation}: the class, method and
// argument names of the reference's PyTorch bindings (src_cpp/pytorch-bindings/src/bindings.cpp:102-122,
// bind_network.cpp:348-411, bind_encoding.cpp:167-197, bind_activation.cpp:82-98), implemented over the header-only C++
// class layer (include/qmlp/*.h) and so over the C ABI of libqmlp_b200.so. PyTorch supplies device memory, the current
// stream and the autograd graph; all arithmetic is in the library's kernels.
#include <mutex>

#include <c10/cuda/CUDAGuard.h>
#include <c10/cuda/CUDAStream.h>
#include <torch/custom_class.h>
#include <torch/script.h>

#include <qmlp/fused_network.h>

namespace {

using torch::Tensor;
using torch::autograd::AutogradContext;
using torch::autograd::variable_list;

CUstream currentStream() { return c10::cuda::getCurrentCUDAStream().stream(); }

// non-owning view of a torch tensor (role of qmlp::wrap, src_cpp/pytorch-bindings/src/bindings.cpp:25-60)
qmlp::Tensor wrap(const Tensor& t)
{
    if (!t.defined()) return qmlp::Tensor();
    TORCH_CHECK(t.is_cuda(), "tensor must live on a CUDA device");
    TORCH_CHECK(t.dim() >= 1 && t.dim() <= 2, "only 1-D and 2-D tensors are supported");
    qmlp::Tensor::Precision p;
    if (t.scalar_type() == torch::kFloat32) p = qmlp::Tensor::FLOAT;
    else if (t.scalar_type() == torch::kFloat16) p = qmlp::Tensor::HALF;
    else if (t.scalar_type() == torch::kFloat64) p = qmlp::Tensor::DOUBLE;
    else TORCH_CHECK(false, "unsupported dtype");
    std::vector<int32_t> sizes, strides;
    for (int64_t i = 0; i < t.dim(); ++i) {
        sizes.push_back(static_cast<int32_t>(t.size(i)));
        strides.push_back(static_cast<int32_t>(t.stride(i)));
    }
    return qmlp::Tensor(t.data_ptr(), p, sizes, strides);
}

template <class F>
auto guarded(F f) -> decltype(f())
{
    try {
        return f();
    } catch (const qmlp::configuration_error& e) {
        TORCH_CHECK(false, "configuration error: ", e.what());
    }
}

// ---- QuickMLP ------------------------------------------------------------------------------------------------------------
struct QuickMLPBindings : torch::CustomClassHolder {
    static void setCompileDebugMode(bool enable) { qmlp::QuickMLP::Instance().setCompileDebugMode(enable); }
    static bool isCompileDebugMode() { return qmlp::QuickMLP::Instance().isCompileDebugMode(); }
    static void setLogLevel(const std::string& level) { qmlp::QuickMLP::Instance().setLogLevel(level); }
    static bool isCudaAvailable() { return qmlp::QuickMLP::Instance().isCudaAvailable(); }
};

// ---- Activation -----------------------------------------------------------------------------------------------------------
struct ActivationBindings;
using ActivationBindings_ptr = c10::intrusive_ptr<ActivationBindings>;

struct ActivationBindings : torch::CustomClassHolder {
    std::string cfg_;
    std::unique_ptr<qmlp::Activation> a_;
    explicit ActivationBindings(const std::string& cfg) : cfg_(cfg)
    {
        guarded([&] { a_ = std::make_unique<qmlp::Activation>(cfg); return 0; });
    }
    std::string cfg() const { return cfg_; }
    Tensor inference(const Tensor& input)
    {
        Tensor output = torch::empty(input.sizes(), input.options().memory_format(c10::MemoryFormat::Contiguous));
        c10::cuda::CUDAGuard guard(input.device());
        qmlp::Tensor out = wrap(output);
        a_->forward(wrap(input), out, currentStream());
        return output;
    }
    Tensor adjoint(const Tensor& input, const Tensor& adjOutput)
    {
        Tensor adjInput = torch::empty(input.sizes(), input.options().memory_format(c10::MemoryFormat::Contiguous));
        c10::cuda::CUDAGuard guard(input.device());
        qmlp::Tensor ai = wrap(adjInput);
        a_->adjoint(wrap(input), wrap(adjOutput.contiguous()), ai, currentStream());
        return adjInput;
    }
    static Tensor forward(const ActivationBindings_ptr& self, const Tensor& input);
};

struct ActivationFunction : torch::autograd::Function<ActivationFunction> {
    static Tensor forward(AutogradContext* ctx, const Tensor& input, const ActivationBindings_ptr& self)
    {
        ctx->saved_data["self"] = self;
        ctx->save_for_backward({input});
        return self->inference(input);
    }
    static variable_list backward(AutogradContext* ctx, variable_list grad)
    {
        auto self = ctx->saved_data["self"].toCustomClass<ActivationBindings>();
        return {self->adjoint(ctx->get_saved_variables()[0], grad[0]), Tensor()};
    }
};
Tensor ActivationBindings::forward(const ActivationBindings_ptr& self, const Tensor& input) { return ActivationFunction::apply(input, self); }

// ---- Encoding -------------------------------------------------------------------------------------------------------------
struct EncodingBindings;
using EncodingBindings_ptr = c10::intrusive_ptr<EncodingBindings>;

struct EncodingBindings : torch::CustomClassHolder {
    std::string cfg_;
    qmlp::IEncoding_ptr e_;
    explicit EncodingBindings(const std::string& cfg) : cfg_(cfg)
    {
        guarded([&] { e_ = qmlp::EncodingFactory::Instance().create(cfg); return 0; });
    }
    explicit EncodingBindings(qmlp::IEncoding_ptr e) : cfg_(e->toJsonString()), e_(std::move(e)) {}
    std::string cfg() const { return cfg_; }
    int64_t maxInputChannel() const { return e_->maxInputChannel(); }
    int64_t numOutputChannels() const { return e_->numOutputChannels(); }
    bool hasParameters() const { return e_->hasParameters(); }
    std::string toJson() const { return e_->toJsonString(); }
    Tensor createInferenceParameters() const
    {
        TORCH_CHECK(e_->hasParameters(), "this encoding has no parameters");
        return torch::empty({e_->parameterCount()}, torch::dtype(torch::kFloat32).device(torch::kCUDA));
    }
    Tensor createGradientParameters() const
    {
        TORCH_CHECK(e_->hasParameters(), "this encoding has no parameters");
        return torch::zeros({e_->parameterCount()}, torch::dtype(torch::kFloat32).device(torch::kCUDA));
    }
    Tensor inferenceWithParameter(const Tensor& input, const Tensor& parameter)
    {
        Tensor output = torch::empty({input.size(0), numOutputChannels()}, input.options().dtype(torch::kFloat32));
        c10::cuda::CUDAGuard guard(input.device());
        qmlp::Tensor out = wrap(output);
        if (parameter.defined() && parameter.numel() > 0) e_->forward(wrap(input), out, currentStream(), wrap(parameter));
        else e_->forward(wrap(input), out, currentStream());
        return output;
    }
    Tensor inference(const Tensor& input) { return inferenceWithParameter(input, Tensor()); }
    // (adjoint of the input, adjoint of the parameter); what is not asked for stays undefined
    std::tuple<Tensor, Tensor> adjointWithFlags(const Tensor& input, const Tensor& parameter, const Tensor& adjOutput, bool wantInput, bool wantParam)
    {
        const bool hasParam = parameter.defined() && parameter.numel() > 0;
        Tensor adjInput = wantInput ? torch::zeros_like(input) : Tensor();
        Tensor adjParam = (wantParam && hasParam) ? torch::zeros(parameter.sizes(), parameter.options().dtype(torch::kFloat32)) : Tensor();
        c10::cuda::CUDAGuard guard(input.device());
        qmlp::Tensor ai = wrap(adjInput);
        const int mode = (wantInput ? qmlp::IEncoding::INPUT_GRADIENTS : 0) | (adjParam.defined() ? qmlp::IEncoding::PARAM_GRADIENTS : 0);
        std::optional<const qmlp::Tensor> p, g;
        if (hasParam) p.emplace(wrap(parameter));
        if (adjParam.defined()) g.emplace(wrap(adjParam));
        e_->adjoint(wrap(input), wrap(adjOutput.contiguous()), ai, currentStream(), p, g, mode);
        return {adjInput, adjParam};
    }
    Tensor adjoint(const Tensor& input, const Tensor& adjOutput) { return std::get<0>(adjointWithFlags(input, Tensor(), adjOutput, true, false)); }
    std::tuple<Tensor, Tensor> adjointWithParameter(const Tensor& input, const Tensor& parameter, const Tensor& adjOutput)
    {
        return adjointWithFlags(input, parameter, adjOutput, true, true);
    }
    static Tensor forward(const EncodingBindings_ptr& self, const Tensor& input);
    static Tensor forwardWithParameter(const EncodingBindings_ptr& self, const Tensor& input, const Tensor& parameter);
};

struct EncodingFunction : torch::autograd::Function<EncodingFunction> {
    static Tensor forward(AutogradContext* ctx, const Tensor& input, const Tensor& parameter, const EncodingBindings_ptr& self)
    {
        ctx->saved_data["self"] = self;
        ctx->save_for_backward({input, parameter});
        return self->inferenceWithParameter(input, parameter);
    }
    static variable_list backward(AutogradContext* ctx, variable_list grad)
    {
        auto self = ctx->saved_data["self"].toCustomClass<EncodingBindings>();
        const auto saved = ctx->get_saved_variables();
        auto g = self->adjointWithFlags(saved[0], saved[1], grad[0], ctx->needs_input_grad(0), ctx->needs_input_grad(1));
        return {std::get<0>(g), std::get<1>(g), Tensor()};
    }
};
Tensor EncodingBindings::forward(const EncodingBindings_ptr& self, const Tensor& input) { return EncodingFunction::apply(input, Tensor(), self); }
Tensor EncodingBindings::forwardWithParameter(const EncodingBindings_ptr& self, const Tensor& input, const Tensor& parameter)
{
    return EncodingFunction::apply(input, parameter, self);
}

// ---- Network --------------------------------------------------------------------------------------------------------------
struct NetworkBindings;
using NetworkBindings_ptr = c10::intrusive_ptr<NetworkBindings>;

struct NetworkBindings : torch::CustomClassHolder {
    std::string cfg_, parent_;
    std::unique_ptr<qmlp::FusedNetwork> n_;
    std::mutex mutex_;   // the bound parameter pointers are state of the network (bind_network.h:20)

    NetworkBindings(const std::string& cfg, const std::string& parent) : cfg_(cfg), parent_(parent)
    {
        guarded([&] { n_ = std::make_unique<qmlp::FusedNetwork>(cfg, parent); return 0; });
    }
    std::string cfg() const { return cfg_; }
    std::string parent() const { return parent_; }
    static int64_t MatrixSize() { return qmlp::FusedNetwork::MATRIX_SIZE; }
    static int64_t WarpSize() { return qmlp::FusedNetwork::WARP_SIZE; }
    static int64_t MaxSharedMemoryBytes() { return qmlp::FusedNetwork::MAX_SHARED_MEMORY_BYTES; }
    int64_t numEncodings() const { return n_->numEncodings(); }
    EncodingBindings_ptr encoding(int64_t idx) { return c10::make_intrusive<EncodingBindings>(n_->encoding(static_cast<int>(idx))); }
    int64_t channelsIn() const { return n_->channelsIn(); }
    int64_t channelsOut() const { return n_->channelsOut(); }
    int64_t numLayers() const { return n_->numLayers(); }
    int64_t networkParameterCount() const { return n_->networkParameterCount(); }
    Tensor createInferenceParameters() const
    {
        return torch::zeros({networkParameterCount()}, torch::dtype(torch::kFloat16).device(torch::kCUDA));
    }
    void initializeInferenceParameters(Tensor dst)
    {
        TORCH_CHECK(dst.scalar_type() == torch::kFloat16 && dst.dim() == 1 && dst.size(0) == networkParameterCount() && dst.is_cuda(),
                    "expected a CUDA float16 vector with num_network_parameters() entries");
        std::lock_guard<std::mutex> lock(mutex_);
        n_->setNetworkParameter(wrap(dst), qmlp::Tensor::INFERENCE);
        std::default_random_engine rng(static_cast<unsigned>(torch::randint(1 << 30, {1}).item<int64_t>()));
        n_->initializeInferenceParameters(rng);
    }
    // view into a flat parameter (or gradient) vector: weight matrix or bias of one layer, sharing its memory
    Tensor view(int64_t layer, bool bias, Tensor parameters)
    {
        TORCH_CHECK(parameters.dim() == 1 && parameters.size(0) == networkParameterCount(), "expected a vector with num_network_parameters() entries");
        const auto p = parameters.scalar_type() == torch::kFloat16 ? qmlp::Tensor::HALF : qmlp::Tensor::FLOAT;
        qmlp::Tensor v = n_->networkParameter(static_cast<int>(layer), bias, parameters.data_ptr(), p);
        if (!v.defined()) return torch::empty({0}, parameters.options());
        const int64_t offset = (static_cast<char*>(v.rawPtr()) - static_cast<char*>(parameters.data_ptr())) / parameters.element_size();
        if (bias) return parameters.slice(0, offset, offset + v.size(0));
        return parameters.slice(0, offset, offset + static_cast<int64_t>(v.size(0)) * v.size(1)).view({v.size(0), v.size(1)});
    }

    void bind(const Tensor& halfParameters, const std::vector<Tensor>& encodingParameters)
    {
        n_->setNetworkParameter(wrap(halfParameters), qmlp::Tensor::INFERENCE);
        for (size_t i = 0; i < encodingParameters.size() && i < static_cast<size_t>(n_->numEncodings()); ++i)
            if (encodingParameters[i].defined() && encodingParameters[i].numel() > 0)
                n_->encoding(static_cast<int>(i))->setParameter(wrap(encodingParameters[i]), qmlp::Tensor::INFERENCE);
    }
    static Tensor toHalf(const Tensor& p) { return p.scalar_type() == torch::kFloat16 ? p : p.to(torch::kFloat16); }

    Tensor inference(const Tensor& input, const Tensor& networkParameters, const std::vector<Tensor>& encodingParameters)
    {
        c10::cuda::CUDAGuard guard(input.device());
        Tensor output = torch::empty({input.size(0), channelsOut()}, input.options().dtype(torch::kFloat32));
        const Tensor half = toHalf(networkParameters.detach());
        std::lock_guard<std::mutex> lock(mutex_);
        bind(half, encodingParameters);
        qmlp::Tensor out = wrap(output);
        n_->inference(wrap(input), out, currentStream());
        return output;
    }
    static Tensor forward(const NetworkBindings_ptr& self, const Tensor& input, const Tensor& networkParameters,
                          const std::vector<Tensor>& encodingParameters);
};

// inputs: input, network parameters, then one tensor per encoding (empty: no parameters)
struct NetworkFunction : torch::autograd::Function<NetworkFunction> {
    static Tensor forward(AutogradContext* ctx, const NetworkBindings_ptr& self, int64_t flags, const Tensor& input,
                          const Tensor& networkParameters, at::TensorList encodingList)
    {
        // (an at::TensorList argument is what autograd walks for inputs; a std::vector would count as one opaque value)
        const std::vector<Tensor> encodingParameters(encodingList.begin(), encodingList.end());
        c10::cuda::CUDAGuard guard(input.device());
        const Tensor half = NetworkBindings::toHalf(networkParameters.detach());
        Tensor tmp = torch::empty({static_cast<int64_t>(std::max<size_t>(self->n_->forwardMemory(static_cast<int>(input.size(0)), static_cast<int>(flags)), 16))},
                                  input.options().dtype(torch::kUInt8));
        Tensor output = torch::empty({input.size(0), self->channelsOut()}, input.options().dtype(torch::kFloat32));
        {
            std::lock_guard<std::mutex> lock(self->mutex_);
            self->bind(half, encodingParameters);
            qmlp::Tensor out = wrap(output);
            self->n_->forward(wrap(input.detach()), out, tmp.data_ptr(), currentStream());
        }
        ctx->saved_data["self"] = self;
        ctx->saved_data["flags"] = flags;
        ctx->saved_data["param_dtype"] = static_cast<int64_t>(networkParameters.scalar_type());
        variable_list saved = {input, half, tmp};
        for (const auto& p : encodingParameters) saved.push_back(p);
        ctx->save_for_backward(saved);
        return output;
    }
    static variable_list backward(AutogradContext* ctx, variable_list grad)
    {
        auto self = ctx->saved_data["self"].toCustomClass<NetworkBindings>();
        const int flags = static_cast<int>(ctx->saved_data["flags"].toInt());
        const auto saved = ctx->get_saved_variables();
        const Tensor& input = saved[0];
        const Tensor& half = saved[1];
        const Tensor& tmp = saved[2];
        std::vector<Tensor> enc(saved.begin() + 3, saved.end());
        c10::cuda::CUDAGuard guard(input.device());
        const Tensor gradOutput = grad[0].contiguous();
        Tensor adjInput = (flags & qmlp::FusedNetwork::GRADIENTS_INPUT) ? torch::zeros_like(input) : Tensor();
        Tensor adjParams;
        std::vector<Tensor> adjEnc(enc.size());
        {
            std::lock_guard<std::mutex> lock(self->mutex_);
            self->bind(half, enc);
            if (flags & qmlp::FusedNetwork::GRADIENTS_NETWORK_WEIGHTS) {
                adjParams = torch::zeros(half.sizes(), half.options().dtype(torch::kFloat32));
                self->n_->setNetworkParameter(wrap(adjParams), qmlp::Tensor::GRADIENTS);
            }
            for (size_t i = 0; i < enc.size() && i < static_cast<size_t>(self->n_->numEncodings()); ++i) {
                const bool want = (flags & qmlp::FusedNetwork::GRADIENTS_INPUT_ENCODINGS) && enc[i].defined() && enc[i].numel() > 0 &&
                                  ctx->needs_input_grad(2 + i);   // edges are counted over the tensor arguments only
                if (want) {
                    adjEnc[i] = torch::zeros(enc[i].sizes(), enc[i].options().dtype(torch::kFloat32));
                    self->n_->encoding(static_cast<int>(i))->setParameter(wrap(adjEnc[i]), qmlp::Tensor::GRADIENTS);
                } else if (self->n_->encoding(static_cast<int>(i))->hasParameters()) {
                    self->n_->encoding(static_cast<int>(i))->setParameter(qmlp::Tensor(), qmlp::Tensor::GRADIENTS);
                }
            }
            Tensor adjTmp = torch::empty({static_cast<int64_t>(std::max<size_t>(self->n_->adjointMemory(static_cast<int>(input.size(0)), flags), 16))},
                                         input.options().dtype(torch::kUInt8));
            qmlp::Tensor ai = wrap(adjInput);
            self->n_->adjoint(wrap(input), wrap(gradOutput), flags, ai, tmp.data_ptr(), adjTmp.data_ptr(), currentStream());
        }
        if (adjParams.defined())
            adjParams = adjParams.to(static_cast<c10::ScalarType>(ctx->saved_data["param_dtype"].toInt()));
        variable_list out = {Tensor(), Tensor(), adjInput, adjParams};
        for (auto& g : adjEnc) out.push_back(g);
        return out;
    }
};

Tensor NetworkBindings::forward(const NetworkBindings_ptr& self, const Tensor& input, const Tensor& networkParameters,
                                const std::vector<Tensor>& encodingParameters)
{
    int64_t flags = 0;
    if (input.requires_grad()) flags |= qmlp::FusedNetwork::GRADIENTS_INPUT;
    if (networkParameters.requires_grad()) flags |= qmlp::FusedNetwork::GRADIENTS_NETWORK_WEIGHTS;
    for (const auto& p : encodingParameters)
        if (p.defined() && p.requires_grad()) flags |= qmlp::FusedNetwork::GRADIENTS_INPUT_ENCODINGS;
    if (flags == 0 || !torch::GradMode::is_enabled()) return self->inference(input, networkParameters, encodingParameters);
    return NetworkFunction::apply(self, flags, input, networkParameters, at::TensorList(encodingParameters));
}

} // namespace

TORCH_LIBRARY(qmlp_cu, m)
{
    m.class_<QuickMLPBindings>("QuickMLP")
        .def_static("set_compile_debug_mode", &QuickMLPBindings::setCompileDebugMode)
        .def_static("is_compile_debug_mode", &QuickMLPBindings::isCompileDebugMode)
        .def_static("set_log_level", &QuickMLPBindings::setLogLevel)
        .def_static("is_cuda_available", &QuickMLPBindings::isCudaAvailable);

    m.class_<ActivationBindings>("Activation")
        .def(torch::init<std::string>())
        .def("cfg", &ActivationBindings::cfg)
        .def("inference", &ActivationBindings::inference)
        .def("adjoint", &ActivationBindings::adjoint)
        .def("forward", [](const ActivationBindings_ptr& self, const Tensor& input) { return ActivationBindings::forward(self, input); })
        .def_pickle([](const ActivationBindings_ptr& self) -> std::string { return self->cfg(); },
                    [](std::string state) -> ActivationBindings_ptr { return c10::make_intrusive<ActivationBindings>(std::move(state)); });

    m.class_<EncodingBindings>("Encoding")
        .def(torch::init<std::string>())
        .def("cfg", &EncodingBindings::cfg)
        .def("max_input_channel", &EncodingBindings::maxInputChannel)
        .def("num_output_channels", &EncodingBindings::numOutputChannels)
        .def("has_parameters", &EncodingBindings::hasParameters)
        .def("to_json", &EncodingBindings::toJson)
        .def("create_inference_parameters", &EncodingBindings::createInferenceParameters)
        .def("create_gradient_parameters", &EncodingBindings::createGradientParameters)
        .def("inference", &EncodingBindings::inference)
        .def("adjoint", &EncodingBindings::adjoint)
        .def("inference_with_parameter", &EncodingBindings::inferenceWithParameter)
        .def("adjoint_with_parameter", &EncodingBindings::adjointWithParameter)
        .def("forward", [](const EncodingBindings_ptr& self, const Tensor& input) { return EncodingBindings::forward(self, input); })
        .def("forward_with_parameter", [](const EncodingBindings_ptr& self, const Tensor& input, const Tensor& parameter) {
            return EncodingBindings::forwardWithParameter(self, input, parameter);
        })
        .def_pickle([](const EncodingBindings_ptr& self) -> std::string { return self->cfg(); },
                    [](std::string state) -> EncodingBindings_ptr { return c10::make_intrusive<EncodingBindings>(std::move(state)); });

    m.class_<NetworkBindings>("Network")
        .def(torch::init<std::string, std::string>(), "", {torch::arg("cfg"), torch::arg("parent") = "."})
        .def("cfg", &NetworkBindings::cfg)
        .def("parent", &NetworkBindings::parent)
        .def_static("MatrixSize", &NetworkBindings::MatrixSize)
        .def_static("WarpSize", &NetworkBindings::WarpSize)
        .def_static("MaxSharedMemoryBytes", &NetworkBindings::MaxSharedMemoryBytes)
        .def("num_encodings", &NetworkBindings::numEncodings)
        .def("encoding", &NetworkBindings::encoding)
        .def("channels_in", &NetworkBindings::channelsIn)
        .def("channels_out", &NetworkBindings::channelsOut)
        .def("num_layers", &NetworkBindings::numLayers)
        .def("num_network_parameters", &NetworkBindings::networkParameterCount)
        .def("create_inference_parameters", &NetworkBindings::createInferenceParameters)
        .def("initialize_inference_parameters", &NetworkBindings::initializeInferenceParameters)
        .def("parameter_view", &NetworkBindings::view)
        .def("inference", &NetworkBindings::inference, "",
             {torch::arg("input"), torch::arg("network_parameters"), torch::arg("encoding_parameters") = std::vector<Tensor>()})
        .def("forward",
             [](const NetworkBindings_ptr& self, const Tensor& input, const Tensor& networkParameters, const std::vector<Tensor>& encodingParameters) {
                 return NetworkBindings::forward(self, input, networkParameters, encodingParameters);
             },
             "", {torch::arg("input"), torch::arg("network_parameters"), torch::arg("encoding_parameters") = std::vector<Tensor>()})
        .def_pickle([](const NetworkBindings_ptr& self) -> std::vector<std::string> { return {self->cfg(), self->parent()}; },
                    [](std::vector<std::string> state) -> NetworkBindings_ptr {
                        TORCH_CHECK(state.size() == 2, "Corrupt state");
                        return c10::make_intrusive<NetworkBindings>(std::move(state[0]), std::move(state[1]));
                    });
}
