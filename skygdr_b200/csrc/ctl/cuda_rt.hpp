// The few CUDA runtime calls a host program of the control plane needs, bound at run time with dlopen, so that
// these programs build with g++ alone and start on machines without a GPU (they then refuse the GPU modes with a
// message). SKYGDR_CUDART names the library to load; tests point it at a stand-in that works on host memory, the
// same way the signal collectors are tested against a stand-in NVML.
//
// The reference's server links the runtime directly and exits at start-up without a GPU (src/gpu_server.cu:37-46).
#pragma once
#include <dlfcn.h>

#include <cstddef>
#include <cstdlib>
#include <string>

namespace skygdr {

class CudaRt {
public:
    enum { kHostToDevice = 1, kDeviceToHost = 2 };       // cudaMemcpyKind

    int (*SetDevice)(int) = nullptr;
    int (*Malloc)(void**, size_t) = nullptr;
    int (*Free)(void*) = nullptr;
    int (*HostAlloc)(void**, size_t, unsigned) = nullptr;
    int (*FreeHost)(void*) = nullptr;
    int (*MemcpyAsync)(void*, const void*, size_t, int, void*) = nullptr;
    int (*StreamCreateWithFlags)(void**, unsigned) = nullptr;
    int (*StreamSynchronize)(void*) = nullptr;
    int (*StreamDestroy)(void*) = nullptr;
    const char* (*GetErrorString)(int) = nullptr;

    // Empty string on success, else why the runtime cannot be used.
    std::string load() {
        const char* env = std::getenv("SKYGDR_CUDART");
        const char* names[] = {env, "libcudart.so.12", "libcudart.so.13", "libcudart.so", "/usr/local/cuda/lib64/libcudart.so"};
        for (const char* n : names) {
            if (!n || !*n) continue;
            handle_ = dlopen(n, RTLD_NOW | RTLD_LOCAL);
            if (handle_) break;
            if (n == env) return std::string("cannot load SKYGDR_CUDART=") + env + ": " + dlerror();
        }
        if (!handle_) return "no CUDA runtime library found (libcudart.so.12)";
        bool ok = sym(SetDevice, "cudaSetDevice") && sym(Malloc, "cudaMalloc") && sym(Free, "cudaFree") && sym(HostAlloc, "cudaHostAlloc") &&
                  sym(FreeHost, "cudaFreeHost") && sym(MemcpyAsync, "cudaMemcpyAsync") && sym(StreamCreateWithFlags, "cudaStreamCreateWithFlags") &&
                  sym(StreamSynchronize, "cudaStreamSynchronize") && sym(StreamDestroy, "cudaStreamDestroy") && sym(GetErrorString, "cudaGetErrorString");
        return ok ? "" : "the CUDA runtime library lacks a needed symbol";
    }
    std::string err(int code) const { return GetErrorString ? GetErrorString(code) : "cuda error " + std::to_string(code); }

private:
    template <class F>
    bool sym(F& f, const char* name) {
        f = reinterpret_cast<F>(dlsym(handle_, name));
        return f != nullptr;
    }
    void* handle_ = nullptr;
};

}  // namespace skygdr
