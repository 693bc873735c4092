// tenzo::CUDARuntime — per-operator CUDA backend with host-pointer operands (see
// include/CUDARuntime.h). Replaces the reference's stub, src/runtime/CUDARuntime.cpp:17-113.
#include <cuda_runtime.h>

#include <cstring>

#include "../../include/CUDARuntime.h"
#include "../../include/tenzo_kernels.h"

namespace tenzo {

namespace {
// Plain tiled fp32 GEMM; only reachable through executeGemmF32, which no decode path calls.
__global__ void gemm_f32_kernel(const float* A, const float* B, float* C, int M, int K, int N) {
    __shared__ float sa[16][17], sb[16][17];
    const int row = blockIdx.y * 16 + threadIdx.y, col = blockIdx.x * 16 + threadIdx.x;
    float acc = 0.0f;
    for (int k0 = 0; k0 < K; k0 += 16) {
        sa[threadIdx.y][threadIdx.x] = (row < M && k0 + threadIdx.x < K) ? A[(size_t)row * K + k0 + threadIdx.x] : 0.0f;
        sb[threadIdx.y][threadIdx.x] = (col < N && k0 + threadIdx.y < K) ? B[(size_t)(k0 + threadIdx.y) * N + col] : 0.0f;
        __syncthreads();
#pragma unroll
        for (int k = 0; k < 16; ++k) acc = __fmaf_rn(sa[threadIdx.y][k], sb[k][threadIdx.x], acc);
        __syncthreads();
    }
    if (row < M && col < N) C[(size_t)row * N + col] = acc;
}

bool grow(void*& p, size_t& cap, size_t need) {
    if (need <= cap) return true;
    if (p) cudaFree(p);
    p = nullptr;
    cap = 0;
    if (cudaMalloc(&p, need) != cudaSuccess) return false;
    cap = need;
    return true;
}
}  // namespace

CUDARuntime& CUDARuntime::getInstance() {
    static CUDARuntime instance;
    return instance;
}

CUDARuntime::CUDARuntime() {}

CUDARuntime::~CUDARuntime() {
    // Device memory is released with the context at process exit; freeing here could run after
    // the CUDA runtime has already shut down.
}

bool CUDARuntime::initialize() {
    if (initialized_) return true;
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess || n == 0) {
        device_name_ = "CUDA Backend Unavailable";
        return false;
    }
    int dev = 0;
    cudaDeviceProp prop;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaGetDeviceProperties(&prop, dev) != cudaSuccess) return false;
    if (prop.major != 10) {   // kernels are built for sm_100a only
        device_name_ = std::string("CUDA Backend Unavailable (needs sm_100, found ") + prop.name + ")";
        return false;
    }
    cudaStream_t st;
    if (cudaStreamCreateWithFlags(&st, cudaStreamNonBlocking) != cudaSuccess) return false;
    stream_ = st;
    device_name_ = prop.name;
    initialized_ = true;
    return true;
}

bool CUDARuntime::ensure(size_t act_bytes, size_t w_bytes, size_t out_bytes) {
    return grow(d_act_, act_cap_, act_bytes) && grow(d_w_, w_cap_, w_bytes) && grow(d_out_, out_cap_, out_bytes);
}

static unsigned long long g_hal_calls = 0;   // execute* calls that reached the device (see tenzo_hal_call_count)

bool CUDARuntime::executeBitLinearTL1(const float* act, const uint8_t* weight, float* out,
                                      size_t M, size_t K, size_t N, float scale) {
    if (!initialized_ && !initialize()) return false;
    ++g_hal_calls;
    if (!act || !weight || !out || M == 0 || K == 0 || N == 0 || (K & 1) || (N % 64) || K > 16384) return false;
    cudaStream_t st = static_cast<cudaStream_t>(stream_);
    const size_t wb = N * K / 4, nb = N / 64;
    if (!ensure(M * K * 4, wb, M * N * 4)) return false;
    const size_t ws_bytes = tenzo_cuda_tl1_gemv_workspace_bytes((int)M, (int)K);
    if (!grow(d_ws_, ws_cap_, ws_bytes)) return false;
    if (cudaMemcpyAsync(d_act_, act, M * K * 4, cudaMemcpyHostToDevice, st) != cudaSuccess) return false;
    if (cudaMemcpyAsync(d_w_, weight, wb, cudaMemcpyHostToDevice, st) != cudaSuccess) return false;
    tenzo_tl1_gemv_args g;
    std::memset(&g, 0, sizeof g);
    g.x = static_cast<const float*>(d_act_); g.x_stride = (int)K; g.do_norm = 0; g.eps = 1e-5f;
    g.w = static_cast<const uint8_t*>(d_w_); g.n_blocks = (int)nb; g.K = (int)K;
    g.seg_end[0] = g.seg_end[1] = g.seg_end[2] = (int)nb; g.seg_scale[0] = scale;
    g.epilogue = TENZO_EPI_STORE; g.out = static_cast<float*>(d_out_); g.out_stride = (int)N; g.batch = (int)M;
    g.workspace = d_ws_;
    if (tenzo_cuda_tl1_gemv(&g, st) != 0) return false;
    if (cudaMemcpyAsync(out, d_out_, M * N * 4, cudaMemcpyDeviceToHost, st) != cudaSuccess) return false;
    return cudaStreamSynchronize(st) == cudaSuccess;
}

bool CUDARuntime::executeRMSNorm(const float* in, const float* weight, float* out, size_t dim, float eps) {
    if (!initialized_ && !initialize()) return false;
    ++g_hal_calls;
    if (!in || !out || dim == 0 || dim > 16384) return false;
    cudaStream_t st = static_cast<cudaStream_t>(stream_);
    if (!ensure(dim * 4, dim * 4, dim * 4)) return false;
    if (cudaMemcpyAsync(d_act_, in, dim * 4, cudaMemcpyHostToDevice, st) != cudaSuccess) return false;
    if (weight && cudaMemcpyAsync(d_w_, weight, dim * 4, cudaMemcpyHostToDevice, st) != cudaSuccess) return false;
    if (tenzo_cuda_rmsnorm_quant(static_cast<const float*>(d_act_), weight ? static_cast<const float*>(d_w_) : nullptr, 1, eps,
                                 (int)dim, 31, 1, (int)dim, static_cast<float*>(d_out_), nullptr, nullptr, st) != 0)
        return false;
    if (cudaMemcpyAsync(out, d_out_, dim * 4, cudaMemcpyDeviceToHost, st) != cudaSuccess) return false;
    return cudaStreamSynchronize(st) == cudaSuccess;
}

bool CUDARuntime::executeGemmF32(const float* A, const float* B, float* C, size_t M, size_t K, size_t N) {
    if (!initialized_ && !initialize()) return false;
    if (!A || !B || !C || M == 0 || K == 0 || N == 0) return false;
    cudaStream_t st = static_cast<cudaStream_t>(stream_);
    if (!ensure(M * K * 4, K * N * 4, M * N * 4)) return false;
    if (cudaMemcpyAsync(d_act_, A, M * K * 4, cudaMemcpyHostToDevice, st) != cudaSuccess) return false;
    if (cudaMemcpyAsync(d_w_, B, K * N * 4, cudaMemcpyHostToDevice, st) != cudaSuccess) return false;
    dim3 grid((unsigned)((N + 15) / 16), (unsigned)((M + 15) / 16)), block(16, 16);
    gemm_f32_kernel<<<grid, block, 0, st>>>(static_cast<const float*>(d_act_), static_cast<const float*>(d_w_),
                                            static_cast<float*>(d_out_), (int)M, (int)K, (int)N);
    if (cudaGetLastError() != cudaSuccess) return false;
    if (cudaMemcpyAsync(C, d_out_, M * N * 4, cudaMemcpyDeviceToHost, st) != cudaSuccess) return false;
    return cudaStreamSynchronize(st) == cudaSuccess;
}

}  // namespace tenzo

// Flat C handles on the class for callers without a C++ toolchain (ctypes, cgo, ...).
extern "C" {
__attribute__((visibility("default"))) int tenzo_hal_initialize(void) { return tenzo::CUDARuntime::getInstance().initialize() ? 1 : 0; }
__attribute__((visibility("default"))) int tenzo_hal_bitlinear_tl1_host(const float* act, const uint8_t* w, float* out,
                                                                        size_t M, size_t K, size_t N, float scale) {
    return tenzo::CUDARuntime::getInstance().executeBitLinearTL1(act, w, out, M, K, N, scale) ? 1 : 0;
}
__attribute__((visibility("default"))) int tenzo_hal_rmsnorm_host(const float* in, const float* w, float* out, size_t dim, float eps) {
    return tenzo::CUDARuntime::getInstance().executeRMSNorm(in, w, out, dim, eps) ? 1 : 0;
}
// How many execute* calls of the backend class have run so far in this process: lets a host that links an engine against the
// class check that its device path really went through it.
__attribute__((visibility("default"))) unsigned long long tenzo_hal_call_count(void) { return tenzo::g_hal_calls; }
__attribute__((visibility("default"))) int tenzo_hal_gemm_f32_host(const float* A, const float* B, float* C, size_t M, size_t K, size_t N) {
    return tenzo::CUDARuntime::getInstance().executeGemmF32(A, B, C, M, K, N) ? 1 : 0;
}
}
