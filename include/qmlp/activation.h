// qmlp::Activation / ActivationFactory (src_cpp/include/qmlp/activation.h:29-147) over the C ABI.
#pragma once
#include <map>
#include <memory>
#include <string>

#include <cuda.h>

#include "tensor.h"
#if __has_include(<nlohmann/json.hpp>)
#include <nlohmann/json.hpp>
#define QMLP_HAS_NLOHMANN_JSON 1
#endif

namespace qmlp {

namespace detail {
// "abc\n" -> \"abc\\n\" for the few places where a JSON text is put together by hand
inline std::string jsonQuote(const std::string& s)
{
    std::string o = "\"";
    for (char c : s) {
        switch (c) {
        case '"': o += "\\\""; break;
        case '\\': o += "\\\\"; break;
        case '\n': o += "\\n"; break;
        case '\t': o += "\\t"; break;
        case '\r': o += "\\r"; break;
        default: o += c;
        }
    }
    return o + "\"";
}
// value of a top-level string member of a flat JSON object ("" if absent)
inline std::string jsonStringMember(const std::string& json, const std::string& key)
{
    const std::string needle = "\"" + key + "\"";
    size_t at = json.find(needle);
    if (at == std::string::npos) return "";
    at = json.find(':', at + needle.size());
    if (at == std::string::npos) return "";
    at = json.find('"', at);
    if (at == std::string::npos) return "";
    std::string out;
    for (size_t i = at + 1; i < json.size() && json[i] != '"'; ++i) {
        if (json[i] == '\\' && i + 1 < json.size()) {
            const char c = json[++i];
            out += c == 'n' ? '\n' : c == 't' ? '\t' : c == 'r' ? '\r' : c;
        } else {
            out += json[i];
        }
    }
    return out;
}
} // namespace detail

class Activation {
public:
    // id + forward / adjoint code snippets over `half x` -> `z`, and `x`, `adjz` -> `adjx` (activation.h:29-37)
    Activation(const std::string& id, const std::string& forward, const std::string& adjoint)
        : Activation("{\"id\": " + detail::jsonQuote(id) + ", \"forward\": " + detail::jsonQuote(forward) + ", \"adjoint\": " +
                     detail::jsonQuote(adjoint) + "}")
    {
    }
    // a built-in id ("relu", "celu", "sine", "identity") or the JSON text of {id, forward, adjoint}
    explicit Activation(const std::string& keyOrJson)
    {
        qmlp_activation_t* h = nullptr;
        detail::check(qmlp_activation_create(keyOrJson.c_str(), &h));
        handle_.reset(h, qmlp_activation_destroy);
        json_ = qmlp_activation_to_json(h);
        id_ = qmlp_activation_id(h);
        forward_ = detail::jsonStringMember(json_, "forward");
        adjoint_ = detail::jsonStringMember(json_, "adjoint");
    }
#ifdef QMLP_HAS_NLOHMANN_JSON
    explicit Activation(const nlohmann::json& cfg) : Activation(cfg.dump()) {}
    nlohmann::json toJson() const { return nlohmann::json::parse(json_); }
#endif
    const std::string& toJsonString() const { return json_; }
    const std::string& id() const { return id_; }
    const std::string& forward() const { return forward_; }
    const std::string& adjoint() const { return adjoint_; }
    // the device functor the reference generates from the snippets (src_cpp/src/activation.cpp:13-40)
    std::string code() const
    {
        return "struct " + id_ + "\n{\n    static __device__ half forward(half x) {\n        half z;\n        " + forward_ +
               ";\n        return z;\n    }\n    static __device__ half adjoint(half x, half adjz) {\n        half adjx;\n        " +
               adjoint_ + ";\n        return adjx;\n    }\n};\n";
    }
    // element-wise on half tensors of shape (B, C) (activation.h:73-92)
    void forward(const Tensor& input, Tensor& output, CUstream stream)
    {
        const qmlp_tensor_t in = input.view();
        qmlp_tensor_t out = output.view();
        detail::check(qmlp_activation_forward(handle_.get(), &in, &out, stream));
    }
    void adjoint(const Tensor& input, const Tensor& adjOutput, Tensor& adjInput, CUstream stream)
    {
        const qmlp_tensor_t in = input.view(), ao = adjOutput.view();
        qmlp_tensor_t ai = adjInput.view();
        detail::check(qmlp_activation_adjoint(handle_.get(), &in, &ao, &ai, stream));
    }

private:
    std::shared_ptr<qmlp_activation_t> handle_;
    std::string json_, id_, forward_, adjoint_;
};
typedef std::shared_ptr<Activation> Activation_ptr;

// Resolves ids to activations (activation.h:103-147). Behind this interface the built-ins and the files named in a
// network's "activation_specification" are resolved by the library itself when a network is created; this class serves
// callers that ask for a stand-alone activation.
class ActivationFactory {
    std::map<std::string, Activation_ptr> cache_;

public:
    // a built-in id or an inline JSON object; throws if the key is neither
    Activation_ptr getOrInline(const std::string& key)
    {
        auto it = cache_.find(key);
        if (it != cache_.end()) return it->second;
        auto a = std::make_shared<Activation>(key);
        cache_[key] = a;
        return a;
    }
    Activation_ptr get(const std::string& key) { return getOrInline(key); }
};

} // namespace qmlp
