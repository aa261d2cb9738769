// Activations, encodings, network spec, parameter layout and source generation for the per-spec instantiation.
#include "host.hpp"

#include <cmath>
#include <cstdarg>
#include <cstring>
#include <fstream>
#include <random>
#include <cctype>
#include <set>
#include <sstream>
#include <sys/stat.h>

#include <cuda_fp16.h>
#include <cuda_runtime.h>

namespace qmlp {

std::string format(const char* fmt, ...)
{
    char buf[2048];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof buf, fmt, ap);
    va_end(ap);
    return buf;
}

static bool fileExists(const std::string& p)
{
    struct stat st;
    return ::stat(p.c_str(), &st) == 0 && S_ISREG(st.st_mode);
}

// =====================================================================================================================
// activations
// =====================================================================================================================
const char* builtinActivationsJson()
{
    // same four entries as the reference's src_cpp/include/qmlp/builtin-activations.json:1-21
    return R"json([
 {"id": "relu", "forward": "z = __hgt(x, hZERO()) ? x : hZERO()", "adjoint": "adjx = __hgt(x, hZERO()) ? adjz : hZERO()"},
 {"id": "celu", "forward": "z = __hgt(x, hZERO()) ? x : __hsub(hexp(x), __float2half(1.0f))", "adjoint": "adjx = __hgt(x, hZERO()) ? adjz : __hmul(adjz, hexp(x))"},
 {"id": "sine", "forward": "z = hsin(x)", "adjoint": "adjx = __hmul(hcos(x), adjz)"},
 {"id": "identity", "forward": "z = x", "adjoint": "adjx = adjz"}
])json";
}

static std::string stripSpaces(const std::string& s)
{
    std::string o;
    for (char c : s) if (c != ' ' && c != '\t' && c != '\n' && c != '\r' && c != ';') o += c;
    return o;
}

// A snippet pair that matches a built-in word for word gets the hand-written half2 functor.
static const char* builtinFunctorFor(const std::string& fwd, const std::string& adj)
{
    static const struct { const char* f; const char* a; const char* name; } table[] = {
        {"z=__hgt(x,hZERO())?x:hZERO()", "adjx=__hgt(x,hZERO())?adjz:hZERO()", "BuiltinRelu"},
        {"z=__hgt(x,hZERO())?x:__hsub(hexp(x),__float2half(1.0f))", "adjx=__hgt(x,hZERO())?adjz:__hmul(adjz,hexp(x))", "BuiltinCelu"},
        {"z=hsin(x)", "adjx=__hmul(hcos(x),adjz)", "BuiltinSine"},
        {"z=x", "adjx=adjz", "BuiltinIdentity"},
    };
    const std::string f = stripSpaces(fwd), a = stripSpaces(adj);
    for (const auto& t : table) if (f == t.f && a == t.a) return t.name;
    return nullptr;
}

Activation::Activation(const std::string& id, const std::string& forward, const std::string& adjoint)
    : id_(id), forward_(forward), adjoint_(adjoint)
{
    // src_cpp/src/activation.cpp:31-37
    // (checked by hand rather than with std::regex: its template instances carry process-wide "unique" symbols, and in a
    // process that holds a second copy of the C++ runtime - an extension module linked against a static libstdc++ is
    // enough - the tables of the two get mixed and regex_match crashes)
    bool identifier = !id.empty() && (std::isalpha(static_cast<unsigned char>(id[0])) || id[0] == '_');
    for (char c : id) identifier = identifier && (std::isalnum(static_cast<unsigned char>(c)) || c == '_');
    if (!identifier)
        throw configuration_error(format("id of the activation function is not a valid C++ identifier: %s", id.c_str()));
    builtin_ = builtinFunctorFor(forward, adjoint) != nullptr;
}

Activation::Activation(const Json& cfg)
    : Activation(cfg.at("id").asString(), cfg.at("forward").asString(), cfg.at("adjoint").asString())
{
}

std::string Activation::functorName() const
{
    if (const char* b = builtinFunctorFor(forward_, adjoint_)) return b;
    return "ScalarActivation<activations::" + id_ + ">";
}

std::string Activation::functorDefinition() const
{
    if (builtin_) return "";
    // same shape as the struct the reference generates (src_cpp/src/activation.cpp:15-28)
    std::ostringstream o;
    o << "struct " << id_ << " {\n"
      << "    static __device__ __forceinline__ half forward(half x) { half z; " << forward_ << " ; return z; }\n"
      << "    static __device__ __forceinline__ half adjoint(half x, half adjz) { half adjx; " << adjoint_ << " ; return adjx; }\n"
      << "};\n";
    return o.str();
}

Json Activation::toJson() const
{
    Json j = Json::object();
    j.set("id", Json::string(id_));
    j.set("forward", Json::string(forward_));
    j.set("adjoint", Json::string(adjoint_));
    return j;
}

std::shared_ptr<KernelModule> Activation::module()
{
    if (module_) return module_;
    std::ostringstream s;
    s << "// stand-alone activation kernels for '" << id_ << "'\n#include \"standalone.cuh\"\nusing namespace qmlp::kernel;\n"
      << "namespace {\nnamespace activations {\n" << functorDefinition() << "}\n}\n"
      << "extern \"C\" int qmlp_spec_abi() { return QMLP_SPEC_ABI_VERSION; }\n"
      << "extern \"C\" int qmlp_spec_launch(int kernel, const void* args, cudaStream_t s, int* launches)\n"
      << "{ return ActivationLaunchers<" << functorName() << ">::launch(kernel, args, s, launches); }\n";
    module_ = getKernelModule("act", s.str());
    return module_;
}

void ActivationFactory::parseArray(const Json& j)
{
    if (!j.isArray()) throw configuration_error("Activation file is expected to contain an array object as the root element");
    for (const auto& e : j.items()) {
        try {
            auto a = std::make_shared<Activation>(e);
            activations_.emplace(a->id(), a);
        } catch (const std::exception& ex) {
            throw configuration_error(std::string("Parsing the activation configuration failed. ") + ex.what());
        }
    }
}

void ActivationFactory::parseFile(const std::string& path)
{
    std::ifstream in(path);
    std::stringstream ss;
    ss << in.rdbuf();
    parseArray(Json::parse(ss.str()));
}

ActivationFactory::ActivationFactory() { parseArray(Json::parse(builtinActivationsJson())); }

ActivationFactory::ActivationFactory(const Json& cfg, const std::string& parent)
{
    if (!cfg.isArray()) throw configuration_error("The activation specification tag must contain an array");
    for (const auto& element : cfg.items()) {
        if (element.isString()) {
            const std::string filename = element.asString();
            // 1. direct, 2. relative to parent, 3. shipped with the library (src_cpp/src/activation.cpp:166-197)
            if (fileExists(filename)) { parseFile(filename); continue; }
            if (!filename.empty() && filename[0] == '/')
                throw configuration_error(format("Absolute path '%s' does not exist. Can't continue resolving the activation file, relative path required", filename.c_str()));
            const std::string rel = (parent.empty() ? std::string(".") : parent) + "/" + filename;
            if (fileExists(rel)) { parseFile(rel); continue; }
            if (filename == "qmlp/builtin-activations.json") { parseArray(Json::parse(builtinActivationsJson())); continue; }
            throw configuration_error(format("Path to activation file '%s' could not be resolved. Is the filename correct?", filename.c_str()));
        } else if (element.isObject()) {
            try {
                auto a = std::make_shared<Activation>(element);
                activations_.emplace(a->id(), a);
            } catch (const std::exception& ex) {
                throw configuration_error(std::string("Parsing the activation configuration failed. ") + ex.what());
            }
        } else {
            throw configuration_error(format("Unknown type of element '%s', only filenames (strings) or in-place specifications (objects) supported.", element.dump().c_str()));
        }
    }
}

Activation_ptr ActivationFactory::get(const std::string& key) const
{
    auto it = activations_.find(key);
    if (it == activations_.end()) throw configuration_error(format("No activation with id '%s' found!", key.c_str()));
    return it->second;
}

Activation_ptr ActivationFactory::getOrInline(const std::string& key)
{
    if (key.empty()) throw std::runtime_error("empty key");
    size_t p = key.find_first_not_of(" \t\r\n");
    if (p != std::string::npos && key[p] == '{') return std::make_shared<Activation>(Json::parse(key));
    return get(key);
}

// =====================================================================================================================
// encodings
// =====================================================================================================================
void Encoding::setParameter(const qmlp_tensor_t*, int) {}

std::shared_ptr<KernelModule> Encoding::standaloneModule(bool halfTable)
{
    auto& m = standalone_[(halfTable ? 1 : 0) + (Library::instance().boundsCheck ? 2 : 0)];
    if (m) return m;
    std::ostringstream s;
    s << "// stand-alone encoding kernels: " << toJson().dump() << "\n#include \"standalone.cuh\"\nusing namespace qmlp::kernel;\n"
      << "namespace {\nstruct EncSpec {\n    static constexpr int NUM_ENCODINGS = 1;\n    template <int E> struct Enc;\n};\n"
      << "template <> struct EncSpec::Enc<0> : " << deviceType(0, 0, halfTable) << " {};\n}\n"
      << "extern \"C\" int qmlp_spec_abi() { return QMLP_SPEC_ABI_VERSION; }\n"
      << "extern \"C\" int qmlp_spec_launch(int kernel, const void* args, cudaStream_t s, int* launches)\n"
      << "{ return EncodingLaunchers<EncSpec>::launch(kernel, args, s, launches); }\n";
    m = getKernelModule("enc", s.str());
    return m;
}

EncodingIdentity::EncodingIdentity(const Json& cfg) : start_(cfg.at("start_in").asInt()), n_(cfg.at("n_in").asInt())
{
    if (start_ < 0) throw configuration_error(format("Start channel must be non-negative, but is %d", start_));
    if (n_ <= 0) throw configuration_error(format("Num channels must be positive, but is %d", n_));
}

Json EncodingIdentity::toJson() const
{
    Json j = Json::object();
    j.set("id", Json::string(id()));
    j.set("start_in", Json::number(start_));
    j.set("n_in", Json::number(n_));
    return j;
}

std::string EncodingIdentity::deviceType(int outOffset, int, bool) const
{
    return format("EncIdentity<%d, %d, %d>", start_, n_, outOffset);
}

static std::vector<float> vectorOrUnit(const std::vector<float>& v, int d, float unit)
{
    if (v.empty()) return std::vector<float>(d, unit);
    if (static_cast<int>(v.size()) != d)
        throw std::runtime_error(format("If a bounding box vector is specified, its dimension must match the configured dimension. Expected %d, actual %d", d, static_cast<int>(v.size())));
    return v;
}

EncodingHashGrid::EncodingHashGrid(const Json& cfg)
    : start_(cfg.at("start_in").asInt()), dim_(cfg.at("n_in").asInt()), levels_(cfg.at("n_levels").asInt()),
      features_(cfg.at("n_features_per_level").asInt()), log2Hashmap_(cfg.at("log2_hashmap_size").asInt()),
      hashmapSize_(log2Hashmap_ > 0 ? 1 << log2Hashmap_ : -1), minRes_(cfg.at("min_resolution").asInt()),
      maxRes_(cfg.at("max_resolution").asInt())
{
    // unknown strings map to the first enum entry, concat (NLOHMANN_JSON_SERIALIZE_ENUM, encoding_hashgrid.cpp:12-15)
    concat_ = cfg.at("combination_mode").asString() != "add";
    boxMin_ = vectorOrUnit(cfg.valueFloats("bounding_box_min"), dim_, -0.5f);
    boxSize_ = vectorOrUnit(cfg.valueFloats("bounding_box_size"), dim_, 1.0f);
    boxInvSize_.resize(boxSize_.size());
    for (size_t i = 0; i < boxSize_.size(); ++i) boxInvSize_[i] = 1.f / boxSize_[i];
    if (cfg.contains("per_level_scale")) { hasScale_ = true; perLevelScale_ = cfg.at("per_level_scale").asDouble(); }

    // src_cpp/src/encoding_hashgrid.cpp:57-62
    if (dim_ < 1 || dim_ > 6) throw std::runtime_error(format("Expected 'dimension' to be in [1,6], but got %d", dim_));
    if (levels_ <= 0) throw std::runtime_error(format("num_levels must be positive but is %d", levels_));
    if (levels_ > kernel::MAX_GRID_LEVELS) throw std::runtime_error(format("num_levels must be at most %d", kernel::MAX_GRID_LEVELS));
    if (features_ <= 0) throw std::runtime_error(format("num_features_per_level must be positive but is %d", features_));
    if (minRes_ <= 0) throw std::runtime_error(format("min_resolution must be positive but is %d", minRes_));
    if (maxRes_ < minRes_ && !hasScale_ && levels_ > 1) throw std::runtime_error("max_resolution must be larger than min_resolution");

    // level table, src_cpp/src/encoding_hashgrid.cpp:64-96 (double precision exp/log/pow, floor)
    double levelScale = 1;
    if (hasScale_) levelScale = perLevelScale_; // extension key: res_l = floor(min_resolution * per_level_scale^l)
    else if (levels_ > 1) levelScale = std::exp((std::log(maxRes_) - std::log(minRes_)) / (levels_ - 1));
    numParameters_ = 0;
    for (int l = 0; l < levels_; ++l) {
        const int resolution = static_cast<int>(std::floor(minRes_ * std::pow(levelScale, l)));
        size_t required = 1;
        for (int d = 0; d < dim_; ++d) required *= static_cast<size_t>(resolution);
        if (hashmapSize_ < 0 || required <= static_cast<size_t>(hashmapSize_)) {
            table_.push_back({numParameters_, resolution, 0, false});
            numParameters_ += static_cast<int64_t>(required) * features_;
        } else {
            table_.push_back({numParameters_, resolution, hashmapSize_, true});
            numParameters_ += static_cast<int64_t>(hashmapSize_) * features_;
        }
    }
    if (numParameters_ > 0xffffffffLL)
        throw std::runtime_error("grid too large: element offsets are 32-bit as in the reference kernels");
}

Json EncodingHashGrid::toJson() const { return gridJson(); }

Json EncodingHashGrid::gridJson() const
{
    Json j = Json::object();
    j.set("id", Json::string("HashGrid"));
    j.set("start_in", Json::number(start_));
    j.set("n_in", Json::number(dim_));
    j.set("n_levels", Json::number(levels_));
    j.set("n_features_per_level", Json::number(features_));
    j.set("log2_hashmap_size", Json::number(log2Hashmap_));
    j.set("min_resolution", Json::number(minRes_));
    j.set("max_resolution", Json::number(maxRes_));
    j.set("combination_mode", Json::string(concat_ ? "concat" : "add"));
    Json bm = Json::array(), bs = Json::array();
    for (float v : boxMin_) bm.push(Json::number(v));
    for (float v : boxSize_) bs.push(Json::number(v));
    j.set("bounding_box_min", bm);
    j.set("bounding_box_size", bs);
    if (hasScale_) j.set("per_level_scale", Json::number(perLevelScale_));
    return j;
}

std::string EncodingHashGrid::deviceType(int outOffset, int slot, bool halfTable) const
{
    return format("EncGrid<%d, %d, %d, %d, %s, %d, %d, %s>", start_, dim_, levels_, features_, concat_ ? "true" : "false",
                  outOffset, slot, halfTable ? "true" : "false");
}

void EncodingHashGrid::setParameter(const qmlp_tensor_t* t, int usage)
{
    BoundTensor b;
    if (t != nullptr && t->ndim > 0 && t->data != nullptr) {
        // src_cpp/src/encoding_hashgrid.cpp:190-197 (+ HALF accepted for the gather table)
        const bool okType = t->precision == QMLP_FLOAT || (usage == QMLP_INFERENCE && t->precision == QMLP_HALF);
        if (!okType) throw std::runtime_error("Wrong data type for the encoding parameter");
        if (t->ndim != 1) throw std::runtime_error(format("Tensor has the wrong dimension, expected 1 but got %d", t->ndim));
        if (t->sizes[0] != numParameters_)
            throw std::runtime_error(format("Tensor has the wrong size at dimension 0, expected %lld but got %lld",
                                            static_cast<long long>(numParameters_), static_cast<long long>(t->sizes[0])));
        if (t->strides[0] != 1) throw std::runtime_error("encoding parameters must be contiguous");
        b.data = t->data;
        b.precision = t->precision;
    }
    if (usage == QMLP_INFERENCE) paramInference = b;
    else paramGradients = b;
}

void EncodingHashGrid::fillGrid(kernel::GridP& g) const
{
    g.table = paramInference.data;
    g.grad = static_cast<float*>(paramGradients.data);
    g.tableIsHalf = paramInference.precision == QMLP_HALF ? 1 : 0;
    for (int i = 0; i < kernel::MAX_GRID_DIMS; ++i) {
        g.boxMin[i] = i < dim_ ? boxMin_[i] : 0.f;
        g.boxInvSize[i] = i < dim_ ? boxInvSize_[i] : 1.f;
        g.boxSize[i] = i < dim_ ? boxSize_[i] : 1.f;
    }
    g.stepsize = 0.f;
    // what bounds-checking instantiations compare every row against (boundsShrink: a test hook that declares the table
    // smaller than it is, so that the check can be seen to fire without any access leaving the real table)
    const int64_t shrink = Library::instance().boundsShrink;
    g.tableCount = static_cast<unsigned long long>(std::max<int64_t>(0, numParameters_ - shrink));
    g.status = nullptr;
    for (int l = 0; l < levels_; ++l) {
        g.levels[l].offset = static_cast<unsigned int>(table_[l].memoryOffset);
        g.levels[l].resolution = table_[l].resolution;
        g.levels[l].hashGridSize = static_cast<unsigned int>(table_[l].hashGridSize);
        g.levels[l].hashed = table_[l].hashed ? 1 : 0;
    }
    // whole-row vector access needs row-size alignment of both tables
    const size_t rowBytesT = static_cast<size_t>(features_) * (g.tableIsHalf ? 2 : 4);
    const size_t alignT = rowBytesT >= 16 ? 16 : rowBytesT;
    const size_t rowBytesG = static_cast<size_t>(features_) * 4;
    const size_t alignG = rowBytesG >= 16 ? 16 : rowBytesG;
    const bool pow2 = (features_ & (features_ - 1)) == 0;
    bool ok = pow2 && features_ >= 2;
    if (g.table && (reinterpret_cast<uintptr_t>(g.table) % alignT) != 0) ok = false;
    if (g.grad && (reinterpret_cast<uintptr_t>(g.grad) % alignG) != 0) ok = false;
    g.vecOk = ok ? 1 : 0;
}

// child volume of a line integration: a hash grid that reads the sample position, channels 0 .. n_in-1
// (parseChild, src_cpp/src/encoding_line_integration.cpp:31-39)
static Json lineChildConfig(const Json& cfg)
{
    Json child = cfg.at("volume");
    if (!child.isObject() || child.at("id").asString() != "HashGrid")
        throw configuration_error("Child encoding for LineIntegration could not be created");
    child.set("start_in", Json::number(0));
    child.set("n_in", Json::number(cfg.at("n_in").asInt()));
    return child;
}

EncodingLineIntegration::EncodingLineIntegration(const Json& cfg)
    : EncodingHashGrid(lineChildConfig(cfg)), rayStart_(cfg.at("start_in").asInt()),
      stepsize_(static_cast<float>(cfg.at("stepsize").asDouble())), average_(cfg.at("blending").asString() == "average")
{
    // unknown blending strings map to the first enum entry, additive (NLOHMANN_JSON_SERIALIZE_ENUM,
    // src_cpp/src/encoding_line_integration.cpp:9-12)
    if (!(stepsize_ > 0.f)) throw std::runtime_error(format("Stepsize must be positive, but is %g", stepsize_));
    if (rayStart_ < 0) throw configuration_error(format("Start channel must be non-negative, but is %d", rayStart_));
    // the reference's ray / box intersection is written for three dimensions only (encoding_line_integration.cuh:13-49)
    if (dim_ != 3) throw configuration_error(format("LineIntegration needs a three-dimensional volume, but n_in is %d", dim_));
}

Json EncodingLineIntegration::toJson() const
{
    Json j = Json::object();
    j.set("id", Json::string(id()));
    j.set("start_in", Json::number(rayStart_));
    j.set("n_in", Json::number(dim_));
    j.set("volume", gridJson());
    j.set("stepsize", Json::number(stepsize_));
    j.set("blending", Json::string(average_ ? "average" : "additive"));
    return j;
}

std::string EncodingLineIntegration::deviceType(int outOffset, int slot, bool halfTable) const
{
    return format("EncLine<%d, %d, %d, %d, %s, %d, %d, %s, %s>", rayStart_, dim_, levels_, features_, concat_ ? "true" : "false",
                  outOffset, slot, halfTable ? "true" : "false", average_ ? "true" : "false");
}

void EncodingLineIntegration::fillGrid(kernel::GridP& g) const
{
    EncodingHashGrid::fillGrid(g);
    g.stepsize = stepsize_;
}

Encoding_ptr createEncoding(const Json& cfg)
{
    const std::string id = cfg.at("id").asString();
    if (id == "Identity") return std::make_shared<EncodingIdentity>(cfg);
    if (id == "HashGrid") return std::make_shared<EncodingHashGrid>(cfg);
    if (id == "LineIntegration") return std::make_shared<EncodingLineIntegration>(cfg);
    throw configuration_error(format("No encoding with id '%s' found", id.c_str()));
}

// =====================================================================================================================
// network
// =====================================================================================================================
Network::Network(const Json& cfg, const std::string& parent)
    : channelsIn_(cfg.at("num_inputs").asInt()), channelsOut_(cfg.at("num_outputs").asInt())
{
    // compile options of the reference (src_cpp/src/fused_network.cpp:45-69) are accepted and ignored: block sizes,
    // shared-memory skew and per-layer weight-update streams are fixed by the kernel design here.
    if (cfg.contains("options")) {
        static const std::set<std::string> known = {"overwrite_blocksize_inference", "overwrite_blocksize_forward",
            "overwrite_blocksize_backward", "overwrite_blocksize_weight_update", "skew_shared_memory", "parallel_weight_update"};
        for (const auto& kv : cfg.at("options").members())
            logMessage(0, (known.count(kv.first) ? "option ignored by this implementation: " : "unknown option: ") + kv.first);
    }

    ActivationFactory activationFactory(cfg.at("activation_specification"), parent);

    const Json& encodingSpecs = cfg.at("encodings");
    if (!encodingSpecs.isArray()) throw configuration_error("Illegal type for 'encodings', array expected");
    int grids = 0;
    for (const auto& e : encodingSpecs.items()) {
        Encoding_ptr enc = createEncoding(e);
        if (enc->maxInputChannel() >= channelsIn_)
            throw configuration_error(format("Input channels for encoding '%s' out of bounds (num channels=%d)", enc->id().c_str(), channelsIn_));
        encodedChannels_ += enc->numOutputChannels();
        if (enc->isGrid()) ++grids;
        encodings_.push_back(enc);
    }
    if (encodings_.empty()) throw configuration_error("At least one encoding is required");
    if (grids > kernel::MAX_GRIDS) throw configuration_error(format("At most %d grid encodings are supported", kernel::MAX_GRIDS));

    const Json& networkSpecs = cfg.at("network");
    if (!networkSpecs.isArray()) throw configuration_error("Expected a json-array for the network configuration");
    if (networkSpecs.empty()) throw configuration_error("Empty network!");

    // The first layer consumes the summed encoding outputs. The reference initialises it with num_inputs
    // (src_cpp/src/fused_network.cpp:95,102), which is only right for identity encodings covering every input.
    int prevInput = encodedChannels_;
    for (const auto& e : networkSpecs.items()) {
        try {
            LayerSpec s;
            s.channelsIn = prevInput;
            s.channelsOut = e.at("n_out").asInt();
            s.useBias = e.at("bias").asBool();
            const Json& ae = e.at("activation");
            if (ae.isString()) {
                s.activation = activationFactory.get(ae.asString());
            } else if (ae.isArray()) {
                if (static_cast<int>(ae.size()) != s.channelsOut)
                    throw configuration_error(format("If you specify individual activations per channel, then the number of activations (%d) must match the number of output channels (%d)",
                                                     static_cast<int>(ae.size()), s.channelsOut));
                // the reference parses such arrays and then refuses them at code generation (fused_network.cpp:447);
                // here a non-uniform array becomes a per-channel functor (generateSource)
                bool uniform = true;
                for (const auto& e2 : ae.items()) {
                    if (!e2.isString()) throw configuration_error("Per-channel activations must be specified as a string");
                    Activation_ptr a = activationFactory.get(e2.asString());
                    if (!s.perChannel.empty() && s.perChannel.front()->id() != a->id()) uniform = false;
                    s.perChannel.push_back(a);
                }
                s.activation = s.perChannel.front();
                if (uniform) s.perChannel.clear();
            } else {
                throw configuration_error("Unknown type for the activations, expected string or array");
            }
            if (s.channelsOut <= 0) throw configuration_error("n_out must be positive");
            prevInput = s.channelsOut;
            layers_.push_back(s);
        } catch (const configuration_error& ex) {
            throw configuration_error(format("Parser error when processing network layer %d: %s", static_cast<int>(layers_.size()), ex.what()));
        }
    }
    if (channelsOut_ != prevInput)
        throw configuration_error(format("The channel count of the last layer (%d) does not match the number of outputs specified at the top of the config file (%d)", prevInput, channelsOut_));

    // padding to multiples of 16, src_cpp/src/fused_network.cpp:146-187
    for (size_t i = 0; i < layers_.size(); ++i) {
        const int cur = layers_[i].channelsIn, padded = roundUp(cur, 16);
        if (cur == padded) continue;
        layers_[i].channelsIn = padded;
        if (i == 0) {
            logMessage(2, format("need to pad the network input channels from the encodings (%d channels) to the next multiple of the matrix size (16). These extra channels are padded with zeros and are thus wasted.", cur));
        } else {
            layers_[i - 1].channelsOut = padded;
            logMessage(2, format("The hidden channels between layer %d and %d are specified to be %d wide; the network has been increased to %d channels.", static_cast<int>(i) - 1, static_cast<int>(i), cur, padded));
        }
    }
    {
        const int cur = layers_.back().channelsOut, padded = roundUp(cur, 16);
        if (cur != padded) {
            layers_.back().channelsOut = padded;
            logMessage(0, format("the last layer's output is not a multiple of 16 but %d, hence padding required", cur));
        }
    }
    for (const auto& l : layers_)
        if (l.channelsIn > 256 || l.channelsOut > 256)
            throw configuration_error("layer widths above 256 channels are not supported by the fused kernels");

    // offsets: all weights first, then the biases of biased layers, src_cpp/src/fused_network.cpp:189-206
    numParameters_ = 0;
    for (auto& l : layers_) { l.weightsStart = numParameters_; numParameters_ += static_cast<int64_t>(l.channelsIn) * l.channelsOut; }
    for (auto& l : layers_) {
        if (l.useBias) { l.biasStart = numParameters_; numParameters_ += l.channelsOut; }
        else l.biasStart = -1;
    }
}

Network::~Network()
{
    if (planes != nullptr) cudaFree(planes);
    hostPipeline.release();
}

static void pipelineCheck(cudaError_t e, const char* what)
{
    if (e != cudaSuccess) throw cuda_error(std::string(what) + ": " + cudaGetErrorString(e));
}

void HostPipeline::reserve(int64_t points, int channelsIn, int channelsOut)
{
    if (copyIn == nullptr) {
        pipelineCheck(cudaStreamCreateWithFlags(&copyIn, cudaStreamNonBlocking), "cudaStreamCreate");
        pipelineCheck(cudaStreamCreateWithFlags(&copyOut, cudaStreamNonBlocking), "cudaStreamCreate");
        pipelineCheck(cudaEventCreateWithFlags(&start, cudaEventDisableTiming), "cudaEventCreate");
        for (int s = 0; s < SLOTS; ++s) {
            pipelineCheck(cudaEventCreateWithFlags(&uploaded[s], cudaEventDisableTiming), "cudaEventCreate");
            pipelineCheck(cudaEventCreateWithFlags(&computed[s], cudaEventDisableTiming), "cudaEventCreate");
            pipelineCheck(cudaEventCreateWithFlags(&downloaded[s], cudaEventDisableTiming), "cudaEventCreate");
        }
    }
    if (points <= capacity) return;
    // cudaFree waits for the device, so no earlier call still uses the old slots
    for (int s = 0; s < SLOTS; ++s) {
        if (in[s]) cudaFree(in[s]);
        if (out[s]) cudaFree(out[s]);
        in[s] = out[s] = nullptr;
    }
    capacity = 0;
    for (int s = 0; s < SLOTS; ++s) {
        pipelineCheck(cudaMalloc(&in[s], static_cast<size_t>(points) * channelsIn * sizeof(float)), "cudaMalloc(upload slot)");
        pipelineCheck(cudaMalloc(&out[s], static_cast<size_t>(points) * channelsOut * sizeof(float)), "cudaMalloc(download slot)");
    }
    capacity = points;
}

void HostPipeline::release()
{
    for (int s = 0; s < SLOTS; ++s) {
        if (in[s]) cudaFree(in[s]);
        if (out[s]) cudaFree(out[s]);
        if (uploaded[s]) cudaEventDestroy(uploaded[s]);
        if (computed[s]) cudaEventDestroy(computed[s]);
        if (downloaded[s]) cudaEventDestroy(downloaded[s]);
        in[s] = out[s] = nullptr;
        uploaded[s] = computed[s] = downloaded[s] = nullptr;
    }
    if (start) cudaEventDestroy(start);
    if (copyIn) cudaStreamDestroy(copyIn);
    if (copyOut) cudaStreamDestroy(copyOut);
    start = nullptr;
    copyIn = copyOut = nullptr;
    capacity = 0;
}

void Network::claimDevice()
{
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) throw cuda_error("cudaGetDevice failed");
    if (ownedDevice < 0) ownedDevice = dev;
    else if (ownedDevice != dev)
        throw std::runtime_error(format("this network keeps staging buffers on device %d and cannot run this call on device %d; "
                                        "create one network object per device", ownedDevice, dev));
}

int Network::gathersPerPoint() const
{
    int g = 0;
    for (const auto& e : encodings_)
        if (auto* h = dynamic_cast<const EncodingHashGrid*>(e.get()))
            if (!h->isLine()) g += static_cast<int>(h->levelTable().size()) << h->dimension();
    return g;
}

int Network::sortDimensions() const
{
    for (const auto& e : encodings_)
        if (auto* h = dynamic_cast<const EncodingHashGrid*>(e.get()))
            return h->isLine() ? 0 : h->dimension();   // a line integration samples many positions per point: no bins
    return 0;
}

int64_t Network::gridTableBytes() const
{
    int64_t b = 0;
    for (const auto& e : encodings_)
        if (e->isGrid() && e->paramInference.defined()) b += e->parameterCount() * (e->paramInference.precision == QMLP_HALF ? 2 : 4);
    return b;
}

Encoding_ptr Network::encoding(int i) const
{
    if (i < 0 || i >= static_cast<int>(encodings_.size())) throw std::runtime_error("Array index out of bounds");
    return encodings_[i];
}

int Network::stashHalfsPerPoint() const
{
    int n = layers_.front().channelsIn;
    for (const auto& l : layers_) n += l.channelsOut;
    return n;
}

int Network::deltaHalfsPerPoint() const
{
    int n = 0;
    for (const auto& l : layers_) n += l.channelsOut;
    return n;
}

void Network::setParameter(const qmlp_tensor_t* t, int usage)
{
    // src_cpp/src/fused_network.cpp:257-278
    if (t == nullptr || t->ndim != 1 || t->sizes[0] != numParameters_)
        throw std::runtime_error(format("Illegal tensor shape, 1D tensor with %lld entries required", static_cast<long long>(numParameters_)));
    const int expected = usage == QMLP_INFERENCE ? QMLP_HALF : QMLP_FLOAT;
    if (t->precision != expected)
        throw std::runtime_error("Wrong data type for the parameter. See parameterPrecision() for the expected format");
    if (t->strides[0] != 1) throw std::runtime_error("network parameters must be contiguous");
    BoundTensor b;
    b.data = t->data;
    b.precision = t->precision;
    if (usage == QMLP_INFERENCE) paramInference = b;
    else if (usage == QMLP_GRADIENTS) paramGradients = b;
    else throw std::runtime_error("Unknown usage");
}

void Network::initializeHost(uint64_t seed, uint16_t* dst) const
{
    // src_cpp/src/fused_network.cpp:280-307: per layer U(-1/sqrt(Cin), 1/sqrt(Cin)) over the padded weight matrix
    // (row by row), then over the bias, one engine for the whole network.
    std::default_random_engine rng(static_cast<std::default_random_engine::result_type>(seed));
    for (const auto& l : layers_) {
        const float bound = 1.0f / std::sqrt(static_cast<float>(l.channelsIn));
        std::uniform_real_distribution<float> distr(-bound, +bound);
        for (int i = 0; i < l.channelsOut; ++i)
            for (int j = 0; j < l.channelsIn; ++j) {
                __half h = __float2half(distr(rng));
                std::memcpy(dst + l.weightsStart + static_cast<int64_t>(i) * l.channelsIn + j, &h, 2);
            }
        if (l.useBias)
            for (int i = 0; i < l.channelsOut; ++i) {
                __half h = __float2half(distr(rng));
                std::memcpy(dst + l.biasStart + i, &h, 2);
            }
    }
}

unsigned Network::currentHalfMask() const
{
    unsigned mask = 0;
    int slot = 0;
    for (const auto& e : encodings_) {
        if (!e->isGrid()) continue;
        if (e->paramInference.defined() && e->paramInference.precision == QMLP_HALF) mask |= 1u << slot;
        ++slot;
    }
    return mask;
}

void Network::fillGrids(kernel::LaunchArgs& a) const
{
    int slot = 0;
    for (const auto& e : encodings_) {
        if (!e->isGrid()) continue;
        e->fillGrid(a.grids[slot]);
        ++slot;
    }
    a.numGrids = slot;
}

std::string Network::generateSource(unsigned halfMask) const
{
    std::ostringstream s;
    s << "// fused-network instantiation; layers:";
    for (const auto& l : layers_)
        s << " " << l.channelsIn << "->" << l.channelsOut << (l.useBias ? "+b" : "") << ":"
          << (l.perChannel.empty() ? l.activation->id() : std::string("per-channel"));
    s << "\n#include \"standalone.cuh\"\nusing namespace qmlp::kernel;\nnamespace {\nnamespace activations {\n";
    std::set<std::string> seen;
    for (const auto& l : layers_) {
        if (!l.activation->isBuiltin() && seen.insert(l.activation->id()).second) s << l.activation->functorDefinition();
        for (const auto& a : l.perChannel)
            if (!a->isBuiltin() && seen.insert(a->id()).second) s << a->functorDefinition();
    }
    s << "}\n";
    // per-channel arrays: one functor per such layer, an if-chain over runs of equal activations; the padding
    // channels behind the last one pass values through (they carry zeros)
    for (int i = 0; i < numLayers(); ++i) {
        const auto& pc = layers_[i].perChannel;
        if (pc.empty()) continue;
        std::ostringstream fwd, adj;
        size_t b = 0;
        while (b < pc.size()) {
            size_t e = b;
            while (e < pc.size() && pc[e]->id() == pc[b]->id()) ++e;
            fwd << "        if (c < " << e << ") return " << pc[b]->functorName() << "::forward(x);\n";
            adj << "        if (c < " << e << ") return " << pc[b]->functorName() << "::adjoint(x, adjz);\n";
            b = e;
        }
        s << "struct PerChannelAct" << i << " : PerChannelActivation<PerChannelAct" << i << "> {\n"
          << "    static __device__ __forceinline__ half forward1(half x, int c)\n    {\n" << fwd.str() << "        return x;\n    }\n"
          << "    static __device__ __forceinline__ half adjoint1(half x, half adjz, int c)\n    {\n" << adj.str() << "        return adjz;\n    }\n};\n";
    }
    int maxWidth = 0;
    for (const auto& l : layers_) maxWidth = std::max(maxWidth, std::max(l.channelsIn, l.channelsOut));
    const int nl = numLayers();
    bool anyLine = false;
    for (const auto& e : encodings_) anyLine = anyLine || e->isLine();
    auto arr = [&](const char* name, auto get) {
        s << "    static constexpr int " << name << "[" << nl << "] = {";
        for (int i = 0; i < nl; ++i) s << (i ? ", " : "") << get(layers_[i]);
        s << "};\n";
    };
    s << "struct Spec {\n"
      << "    static constexpr int NUM_INPUTS = " << channelsIn_ << ", NUM_OUTPUTS = " << channelsOut_ << ", NUM_LAYERS = " << nl
      << ", ENC_CHANNELS = " << encodedChannels_ << ", NUM_ENCODINGS = " << numEncodings() << ";\n"
      << "    static constexpr int WARPS = 8, MIN_BLOCKS = " << (maxWidth <= 64 ? 2 : 1) << ";\n"
      << "    static constexpr bool HAS_LINE = " << (anyLine ? "true" : "false") << ";\n";
    arr("CIN", [](const LayerSpec& l) { return static_cast<long long>(l.channelsIn); });
    arr("COUT", [](const LayerSpec& l) { return static_cast<long long>(l.channelsOut); });
    arr("WOFF", [](const LayerSpec& l) { return static_cast<long long>(l.weightsStart); });
    arr("BOFF", [](const LayerSpec& l) { return static_cast<long long>(l.biasStart); });
    s << "    template <int L> struct Act;\n    template <int E> struct Enc;\n};\n";
    for (int i = 0; i < nl; ++i)
        s << "template <> struct Spec::Act<" << i << "> : "
          << (layers_[i].perChannel.empty() ? layers_[i].activation->functorName() : "PerChannelAct" + std::to_string(i)) << " {};\n";
    int off = 0, slot = 0;
    for (int i = 0; i < numEncodings(); ++i) {
        const auto& e = encodings_[i];
        const bool half = e->isGrid() && ((halfMask >> slot) & 1u);
        s << "template <> struct Spec::Enc<" << i << "> : " << e->deviceType(off, slot, half) << " {};\n";
        off += e->numOutputChannels();
        if (e->isGrid()) ++slot;
    }
    s << "}\nextern \"C\" int qmlp_spec_abi() { return QMLP_SPEC_ABI_VERSION; }\n"
      << "extern \"C\" int qmlp_spec_launch(int kernel, const void* args, cudaStream_t s, int* launches)\n"
      << "{ return NetworkLaunchers<Spec>::launch(kernel, args, s, launches); }\n";
    return s.str();
}

std::shared_ptr<KernelModule> Network::module(unsigned halfMask)
{
    // bounds-checking instantiations are separate shared objects: bit 31 of the cache key
    const unsigned key = halfMask | (Library::instance().boundsCheck ? 0x80000000u : 0u);
    auto it = modules_.find(key);
    if (it != modules_.end()) return it->second;
    auto m = getKernelModule("net", generateSource(halfMask));
    modules_[key] = m;
    return m;
}

void Network::clearModules() { modules_.clear(); }

} // namespace qmlp
