// CUDARuntime.h — the CUDA backend class of the runtime's device-abstraction seam.
//
// Same class name, namespace and public member signatures as the reference's
// src/runtime/CUDARuntime.h:11-56, so the reference engine's forward_layer_cuda
// (src/runtime/TenzoEngine.cpp:1369-1418) compiles and links against this implementation
// unchanged. The reference class only probes for libcuda and then returns false from every
// execute* call (src/runtime/CUDARuntime.cpp:48-66); this one runs the sm_100a kernels.
//
// Calling convention (what forward_layer_cuda passes): HOST pointers, weights in the TL1 layout
// [N/64][K/2][32], M == 1. Each call stages its operands on the device, launches, copies the
// result back and returns true; false means the call did nothing (bad arguments or no device).
// This per-operator path exists for drop-in compatibility; the resident engine behind tenzo.h
// is the fast path.
#ifndef TENZO_CUDA_RUNTIME_H
#define TENZO_CUDA_RUNTIME_H

#include <cstddef>
#include <cstdint>
#include <string>

namespace tenzo {

class __attribute__((visibility("default"))) CUDARuntime {
public:
    static CUDARuntime& getInstance();

    bool initialize();
    bool isAvailable() const { return initialized_; }
    std::string getDeviceName() const { return device_name_; }

    // out[n] = float(sum_k w[n][k] * a_k) * ((max|act|/31) * scale), a = round(act * 31/max|act|):
    // the reference CPU kernel's arithmetic (TenzoEngine.cpp:22-146) with `scale` the per-tensor
    // weight scale, for M rows of activations.
    bool executeBitLinearTL1(const float* d_act, const uint8_t* d_weight, float* d_out,
                             size_t M, size_t K, size_t N, float scale);

    // out = in * (1/sqrt(mean(in^2)+eps)) * weight   (TenzoEngine.cpp:148-166)
    bool executeRMSNorm(const float* d_in, const float* d_weight, float* d_out, size_t dim, float eps = 1e-5f);

    // C[M,N] = A[M,K] * B[K,N], row-major fp32.
    bool executeGemmF32(const float* d_A, const float* d_B, float* d_C, size_t M, size_t K, size_t N);

private:
    CUDARuntime();
    ~CUDARuntime();
    bool ensure(size_t act_bytes, size_t w_bytes, size_t out_bytes);

    bool initialized_ = false;
    bool using_vulkan_translation_ = false;   // always false: there is no translation layer here
    std::string device_name_ = "CUDA Not Initialized";
    void* stream_ = nullptr;
    void* d_act_ = nullptr; size_t act_cap_ = 0;
    void* d_w_ = nullptr;   size_t w_cap_ = 0;
    void* d_out_ = nullptr; size_t out_cap_ = 0;
    void* d_ws_ = nullptr;  size_t ws_cap_ = 0;
};

}  // namespace tenzo

// Flat C handles on the class, for callers without a C++ toolchain (ctypes, cgo, ...): 1 = done, 0 = nothing was done.
extern "C" {
__attribute__((visibility("default"))) int tenzo_hal_initialize(void);
__attribute__((visibility("default"))) int tenzo_hal_bitlinear_tl1_host(const float* act, const uint8_t* w, float* out, size_t M, size_t K, size_t N, float scale);
__attribute__((visibility("default"))) int tenzo_hal_rmsnorm_host(const float* in, const float* w, float* out, size_t dim, float eps);
__attribute__((visibility("default"))) int tenzo_hal_gemm_f32_host(const float* A, const float* B, float* C, size_t M, size_t K, size_t N);
// execute* calls of the class that have reached the device so far in this process
__attribute__((visibility("default"))) unsigned long long tenzo_hal_call_count(void);
}

#endif  // TENZO_CUDA_RUNTIME_H
