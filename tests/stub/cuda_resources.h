// Test stand-in for the reference header of the same name: the members of
// cudatrader::CudaMemory<T> that ltc_attn_shim.hpp uses, declared from the reference's public
// interface (include/cuda_resources.h:531-770).  Only for the syntax check of the shim on
// machines that do not have the reference checkout.
#pragma once
#include <cuda_runtime.h>
#include <cstddef>
namespace cudatrader {
template <typename T>
class CudaMemory {
public:
    CudaMemory() = default;
    explicit CudaMemory(size_t size, cudaStream_t stream = nullptr, size_t alignment = 256);
    CudaMemory(CudaMemory&& other) noexcept;
    CudaMemory& operator=(CudaMemory&& other) noexcept;
    CudaMemory(const CudaMemory&) = delete;
    CudaMemory& operator=(const CudaMemory&) = delete;
    ~CudaMemory();
    T* get() const;
    size_t size() const;
    size_t bytes() const;
    void copyFromHost(const T* hostData, cudaStream_t stream = nullptr) const;
    void copyToHost(T* hostData, cudaStream_t stream = nullptr) const;
    void memset(int value, cudaStream_t stream = nullptr) const;
};
}  // namespace cudatrader
