// Drop-in for src/memory/allocator/cuda_allocator.h of oneLLM (:32-185): a caching device allocator
// behind BaseAllocator.  deviceFree keeps a block for reuse instead of returning it to the driver, so
// the per-forward alloc/free pairs of the layer classes stop costing a cudaMalloc after the first
// pass.  Same policy knobs as the reference: sizes rounded up to 32 bytes; blocks above 1 MiB are
// reused only by requests within 1 MiB of their size (best fit); small blocks by first fit; idle small
// blocks are returned to the driver once 1 GiB of them has piled up.  Differences: the bookkeeping is
// one size-ordered index per device instead of linear scans, unknown pointers are freed with
// cudaFree as before, nothing is printed, and the class is safe to call from several host threads.
#pragma once
#include <cuda_runtime.h>

#include <map>
#include <mutex>
#include <unordered_map>

#include "src/memory/allocator/base_allocator.h"

class CudaAllocator : public BaseAllocator {
    struct Block {
        size_t size;
        bool big;
        bool in_use;
    };
    static constexpr size_t kAlign = 32, kBigThreshold = 1u << 20, kBigSlack = 1u << 20, kTrimAt = 1u << 30;

    std::unordered_map<void*, Block> blocks_;      // every block this allocator got from the driver
    std::multimap<size_t, void*> idle_small_;      // size -> pointer, blocks not handed out
    std::multimap<size_t, void*> idle_big_;
    size_t idle_small_bytes_ = 0;
    int dev_id = 0;
    std::mutex mu_;

    void* take(std::multimap<size_t, void*>& idle, size_t size, size_t max_size)
    {
        auto it = idle.lower_bound(size);  // smallest idle block that fits
        if (it == idle.end() || it->first > max_size) return nullptr;
        void* p = it->second;
        idle.erase(it);
        blocks_[p].in_use = true;
        return p;
    }
    void trimSmall()
    {
        for (auto& kv : idle_small_) {
            cudaFree(kv.second);
            blocks_.erase(kv.second);
        }
        idle_small_.clear();
        idle_small_bytes_ = 0;
    }

public:
    CudaAllocator() { cudaGetDevice(&dev_id); }
    CudaAllocator(const CudaAllocator&) = delete;
    CudaAllocator& operator=(const CudaAllocator&) = delete;
    ~CudaAllocator() override
    {
        for (auto& kv : blocks_) cudaFree(kv.first);
    }

    void* deviceMalloc(void* /*ptr*/, size_t size, bool is_host = false) override
    {
        size = (size + kAlign - 1) / kAlign * kAlign;
        void* p = nullptr;
        if (is_host) return cudaMallocHost(&p, size) == cudaSuccess ? p : nullptr;
        std::lock_guard<std::mutex> lock(mu_);
        const bool big = size > kBigThreshold;
        if (big) {
            p = take(idle_big_, size, size + kBigSlack - 1);
        } else {
            p = take(idle_small_, size, static_cast<size_t>(-1));
            if (p) idle_small_bytes_ -= blocks_[p].size;
        }
        if (p) return p;
        if (cudaMalloc(&p, size) != cudaSuccess) {
            trimSmall();  // give cached memory back and try once more
            if (cudaMalloc(&p, size) != cudaSuccess) return nullptr;
        }
        blocks_[p] = Block{size, big, true};
        return p;
    }

    void deviceFree(void* ptr, bool is_host = false) override
    {
        if (ptr == nullptr) return;
        if (is_host) {
            cudaFreeHost(ptr);
            return;
        }
        std::lock_guard<std::mutex> lock(mu_);
        auto it = blocks_.find(ptr);
        if (it == blocks_.end()) {  // not ours: hand it to the driver, as the reference does
            cudaFree(ptr);
            return;
        }
        if (!it->second.in_use) return;  // double free of a cached block
        it->second.in_use = false;
        if (it->second.big) {
            idle_big_.emplace(it->second.size, ptr);
        } else {
            idle_small_.emplace(it->second.size, ptr);
            idle_small_bytes_ += it->second.size;
            if (idle_small_bytes_ > kTrimAt) trimSmall();
        }
    }

    // additions: bytes held from the driver / bytes currently handed out
    size_t reservedBytes()
    {
        std::lock_guard<std::mutex> lock(mu_);
        size_t n = 0;
        for (auto& kv : blocks_) n += kv.second.size;
        return n;
    }
    size_t activeBytes()
    {
        std::lock_guard<std::mutex> lock(mu_);
        size_t n = 0;
        for (auto& kv : blocks_) n += kv.second.in_use ? kv.second.size : 0;
        return n;
    }
};
