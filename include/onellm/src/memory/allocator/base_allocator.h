// Drop-in for src/memory/allocator/base_allocator.h of oneLLM (:5-17): the interface the layer
// classes allocate their scratch through.  Malloc returns the buffer; its first argument is ignored.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>

#include <cstddef>

class BaseAllocator {
public:
    virtual ~BaseAllocator() {}
    template <typename T>
    void* Malloc(T* ptr, size_t size, bool is_host)
    {
        return deviceMalloc(static_cast<void*>(ptr), size, is_host);
    }
    virtual void* deviceMalloc(void* ptr, size_t size, bool is_host = false) = 0;
    virtual void deviceFree(void* ptr, bool is_host = false) = 0;
};
