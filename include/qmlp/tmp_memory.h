// qmlp::TmpMemory (src_cpp/include/qmlp/tmp_memory.h:14-36): scoped device scratch for forward() / adjoint().
#pragma once
#include <cuda_runtime.h>

#include "errors.h"

namespace qmlp {

class TmpMemory {
    void* memory_ = nullptr;

public:
    explicit TmpMemory(size_t numBytes)
    {
        if (numBytes == 0) return;
        const cudaError_t e = cudaMalloc(&memory_, numBytes);
        if (e != cudaSuccess) throw std::runtime_error(std::string("cudaMalloc: ") + cudaGetErrorString(e));
    }
    ~TmpMemory() { if (memory_) cudaFree(memory_); }
    TmpMemory(const TmpMemory&) = delete;
    TmpMemory& operator=(const TmpMemory&) = delete;
    void* get() { return memory_; }
    const void* get() const { return memory_; }
};

} // namespace qmlp
