// qmlp::configuration_error and the translation of C-ABI status codes back into the exceptions the reference
// throws (src_cpp/include/qmlp/errors.h:9-30: configuration_error; :78-90: CHECK_* -> std::runtime_error).
// Part of the header-only C++ class layer over libqmlp_b200.so: same class and method names as the reference's
// qmlp:: classes, every method a forwarding call into the C ABI of qmlp_b200.h.
#pragma once
#include <exception>
#include <stdexcept>
#include <string>

#include "../qmlp_b200.h"

namespace qmlp {

class configuration_error : public std::exception {
    std::string message_;

public:
    explicit configuration_error(std::string message) : message_(std::move(message)) {}
    const char* what() const noexcept override { return message_.c_str(); }
};

namespace detail {
// QMLP_ERROR_CONFIGURATION -> configuration_error, everything else -> std::runtime_error, each with the library's message
inline void check(int status)
{
    if (status == QMLP_OK) return;
    const char* m = qmlp_last_error();
    const std::string message = m ? m : "unknown error";
    if (status == QMLP_ERROR_CONFIGURATION) throw configuration_error(message);
    throw std::runtime_error(message);
}
} // namespace detail

} // namespace qmlp
