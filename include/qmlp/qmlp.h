// qmlp::QuickMLP (src_cpp/include/qmlp/qmlp.h:14-94): process-wide entry object. Logger and kernel loader of the
// reference have no counterpart behind this interface (the library logs to stdout and instantiates its own kernel
// templates); what remains are the switches a caller sets.
#pragma once
#include <string>

#include "errors.h"

namespace qmlp {

class QuickMLP {
    QuickMLP() = default;

public:
    QuickMLP(const QuickMLP&) = delete;
    QuickMLP& operator=(const QuickMLP&) = delete;
    static QuickMLP& Instance()
    {
        static QuickMLP instance;
        return instance;
    }
    bool isCudaAvailable() const { return qmlp_is_cuda_available() != 0; }
    void checkCudaAvailable() const
    {
        if (!isCudaAvailable()) throw std::runtime_error("CUDA is not available, QuickMLP can't be used");
    }
    // "off", "debug", "info", "warn", "error" (src_cpp/src/qmlp.cpp:56-78)
    void setLogLevel(const std::string& levelName) { detail::check(qmlp_set_log_level(levelName.c_str())); }
    void setCompileDebugMode(bool enable) { detail::check(qmlp_set_compile_debug_mode(enable ? 1 : 0)); }
    bool isCompileDebugMode() const { return qmlp_is_compile_debug_mode() != 0; }
};

} // namespace qmlp
