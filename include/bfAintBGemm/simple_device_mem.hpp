// RAII buffers of the host driver (interface of the reference's bfAintBGemm/simple_device_mem.hpp:5-40), with the
// device side backed by the C ABI (afb_malloc / afb_free) instead of hipMalloc / hipFree.  Unlike the reference, a
// failed device allocation is not ignored: GetBuffer() then returns nullptr and ok() is false.
#pragma once
#include <cstddef>
#include <cstdlib>
#include "afb_capi.h"

struct SimpleMem {
    SimpleMem() = default;
    explicit SimpleMem(std::size_t) {}
    virtual void* GetBuffer() = 0;
    virtual ~SimpleMem() = default;
    bool ok() const { return p_mem_ != nullptr; }
    void* p_mem_ = nullptr;
};

struct SimpleDeviceMem : SimpleMem {
    SimpleDeviceMem() = delete;
    explicit SimpleDeviceMem(std::size_t bytes) : SimpleMem(bytes) {
        if (afb_malloc(&p_mem_, bytes) != AFB_OK) p_mem_ = nullptr;
    }
    void* GetBuffer() override { return p_mem_; }
    ~SimpleDeviceMem() override { if (p_mem_) (void)afb_free(p_mem_); }
};

struct SimpleHostMem : SimpleMem {
    SimpleHostMem() = delete;
    explicit SimpleHostMem(std::size_t bytes) : SimpleMem(bytes) { p_mem_ = std::malloc(bytes ? bytes : 1); }
    void* GetBuffer() override { return p_mem_; }
    ~SimpleHostMem() override { std::free(p_mem_); }
};
