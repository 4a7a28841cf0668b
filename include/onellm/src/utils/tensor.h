// Drop-in for src/utils/tensor.h of oneLLM: Device / DataType (:12-28), getTensorType<T> (:30-54),
// the non-owning Tensor view (:56-144) and the name -> Tensor map the layer classes exchange
// (TensorMap, :161-298).  Same public names and behaviour; additions are marked.
#pragma once
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdint>
#include <initializer_list>
#include <iostream>
#include <sstream>
#include <string>
#include <type_traits>
#include <unordered_map>
#include <utility>
#include <vector>

#include "src/utils/macro.h"
#include "src/utils/string_utils.h"

enum Device { CPU_PINNED, CPU, GPU };

enum DataType { FP32, FP16, INT8, INT32, BOOL, BYTES, UNSUPPORTED };

template <typename T>
DataType getTensorType()
{
    using U = typename std::remove_cv<T>::type;
    return std::is_same<U, float>::value    ? FP32
           : std::is_same<U, half>::value   ? FP16
           : std::is_same<U, int>::value    ? INT32
           : std::is_same<U, int8_t>::value ? INT8
           : std::is_same<U, bool>::value   ? BOOL
           : std::is_same<U, char>::value   ? BYTES
                                            : UNSUPPORTED;
}

// addition: bytes per element, 0 for UNSUPPORTED
inline size_t getTypeSize(DataType t)
{
    switch (t) {
        case FP32: case INT32: return 4;
        case FP16: return 2;
        case INT8: case BOOL: case BYTES: return 1;
        default: return 0;
    }
}

// addition: the dtype tag of the onellm_b200 C ABI for a floating-point tensor type
inline int onellmDtype(DataType t)
{
    ONELLM_CHECK_WITH_INFO(t == FP32 || t == FP16, "the kernels take FP32 or FP16 tensors");
    return t == FP16 ? ONELLM_F16 : ONELLM_F32;
}

// A view: where the bytes live, what they are, their extents.  Never owns `data`
// (buffers belong to an allocator, weights to their weight struct).
struct Tensor {
    Device location = GPU;
    DataType dtype = UNSUPPORTED;
    std::vector<int> shape;
    void* data = nullptr;

    Tensor() = default;
    Tensor(const Device location_, const DataType dtype_, const std::vector<int> shape_, void* data_ = nullptr)
        : location(location_), dtype(dtype_), shape(shape_), data(data_)
    {
    }

    // number of elements; 0 for a view without data or shape
    int size() const
    {
        if (data == nullptr || shape.empty()) return 0;
        long n = 1;
        for (int d : shape) n *= d;
        return static_cast<int>(n);
    }

    template <typename T>
    inline T getVal(int id) const
    {
        return static_cast<T*>(data)[id];
    }

    // element 0 of a HOST tensor
    template <typename T>
    inline T getVal() const
    {
        ONELLM_CHECK(location == CPU);
        return getVal<T>(0);
    }

    template <typename T>
    inline T* getPtr() const
    {
        return static_cast<T*>(data);
    }

    template <typename T>
    inline T* getPtrByOffset(int offset) const
    {
        return static_cast<T*>(data) + offset;
    }

    std::string DeviceString() const { return location == CPU ? "CPU" : (location == CPU_PINNED ? "CPU_PINNED" : "GPU"); }

    std::string toString() const
    {
        static const char* const names[] = {"FP32", "FP16", "INT8", "INT32", "BOOL", "BYTES", "UNSUPPORTED"};
        return fmtstr("Tensor[where=%s, type=%s, shape=%s, data=%p]", DeviceString().c_str(), names[(int)dtype],
                      vec2str(shape).c_str(), data);
    }
};

// addition: the int a one-element tensor holds, wherever its bytes live.  The layer classes pass
// host integers (step, layer_id) in tensors whose `location` tag is not reliable, so the pointer
// itself is asked.
inline int readScalarInt(const Tensor* t)
{
    ONELLM_CHECK_WITH_INFO(t && t->data, "readScalarInt: empty tensor");
    cudaPointerAttributes attr;
    const cudaError_t rc = cudaPointerGetAttributes(&attr, t->data);
    if (rc != cudaSuccess) (void)cudaGetLastError();
    if (rc == cudaSuccess && attr.type == cudaMemoryTypeDevice) {
        int v = 0;
        CHECK(cudaMemcpy(&v, t->data, sizeof(int), cudaMemcpyDeviceToHost));
        return v;
    }
    return *static_cast<const int*>(t->data);
}

inline bool isHostPointer(const void* p)
{
    cudaPointerAttributes attr;
    const cudaError_t rc = cudaPointerGetAttributes(&attr, p);
    if (rc != cudaSuccess) {
        (void)cudaGetLastError();
        return true;
    }
    return attr.type == cudaMemoryTypeUnregistered || attr.type == cudaMemoryTypeHost;
}

// element-wise equality of two HOST float tensors
inline bool operator==(Tensor& t1, Tensor& t2)
{
    if (t1.size() != t2.size()) return false;
    const float* a = static_cast<const float*>(t1.data);
    const float* b = static_cast<const float*>(t2.data);
    for (int i = 0; i < t1.size(); i++)
        if (a[i] != b[i]) {
            std::cout << "two tensor is not equal!\n";
            return false;
        }
    return true;
}

struct TensorMap {
    std::unordered_map<std::string, Tensor> tensor_map_;

    TensorMap() = default;
    // tensors without data or extent are dropped, as the reference does (:165-175)
    TensorMap(std::initializer_list<std::pair<std::string, Tensor>> tensor_map)
    {
        for (const auto& kv : tensor_map) {
            if (isValid(kv.second)) insert(kv.first, kv.second);
            else std::cout << "this is not a valid tensor, skip to insert into tensormap" << std::endl;
        }
    }
    // the reference's version of this constructor iterates its own (empty) member and inserts
    // nothing (:177-192); this one copies the valid entries of its argument
    TensorMap(const std::unordered_map<std::string, Tensor>& tensor_map)
    {
        for (const auto& kv : tensor_map)
            if (isValid(kv.second)) insert(kv.first, kv.second);
    }

    inline size_t size() const { return tensor_map_.size(); }
    inline bool isExist(const std::string& key) const { return tensor_map_.count(key) != 0; }
    inline bool isValid(const Tensor& tensor) { return tensor.size() > 0 && tensor.data != nullptr; }

    inline void insert(const std::string& key, const Tensor& value) { tensor_map_[key] = value; }
    inline void insert(std::pair<std::string, Tensor> p) { tensor_map_.insert(p); }

    inline Tensor& at(const std::string& key)
    {
        ONELLM_CHECK_WITH_INFO(isExist(key), fmtstr("Cannot find a tensor of name %s in the tensor map (keys: %s)", key.c_str(),
                                                    vec2str(keys()).c_str()));
        return tensor_map_.at(key);
    }
    inline Tensor& operator[](const std::string& key) { return at(key); }

    template <typename T>
    inline T getVal(const std::string& key) const
    {
        return tensor_map_.at(key).getVal<T>();
    }
    template <typename T>
    inline T getValByOffset(const std::string& key, int index) const
    {
        return tensor_map_.at(key).getVal<T>(index);
    }
    template <typename T>
    inline T* getPtr(const std::string& key) const
    {
        return tensor_map_.at(key).getPtr<T>();
    }
    template <typename T>
    inline T* getPtrWithOffset(const std::string& key, int index) const
    {
        return tensor_map_.at(key).getPtrByOffset<T>(index);
    }

    std::vector<std::string> keys() const
    {
        std::vector<std::string> names;
        names.reserve(tensor_map_.size());
        for (const auto& kv : tensor_map_) names.push_back(kv.first);
        return names;
    }

    std::string toString()
    {
        std::ostringstream os;
        os << "{";
        bool first = true;
        for (const auto& kv : tensor_map_) {
            os << (first ? "" : ", ") << kv.first << ": " << kv.second.toString();
            first = false;
        }
        os << "}";
        return os.str();
    }
};
