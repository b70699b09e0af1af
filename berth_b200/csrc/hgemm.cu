// Plain fp16 GEMM c[m][ldc] = a[m][k] . b[k][n] behind berth_prefill_hgemm
// (crates/berth-kernels/src/prefill_lin.rs:54-64,163-205, csrc/prefill_lin/linear.cu:387-420,
// csrc/prefill_lin/hgemm.cu:192-268 of berth).  berth runs it through cublasGemmEx with fp32
// accumulation (its own f16acc kernel only on the parts it was tuned for); so does this: a plain dense
// GEMM is library work, the kernels of this repository are the ones that decode.  cuBLAS is taken at the
// first call with dlopen, so that the library itself has no link-time dependency on it and every other
// entry point works where cuBLAS is absent.
#include "common.cuh"
#include "../../include/berth_b200.h"

#include <cublas_v2.h>
#include <dlfcn.h>

#include <mutex>

namespace berth {
namespace {

struct Cublas {
    cublasStatus_t (*create)(cublasHandle_t*) = nullptr;
    cublasStatus_t (*set_stream)(cublasHandle_t, cudaStream_t) = nullptr;
    cublasStatus_t (*gemm_ex)(cublasHandle_t, cublasOperation_t, cublasOperation_t, int, int, int, const void*, const void*,
                              cudaDataType, int, const void*, cudaDataType, int, const void*, void*, cudaDataType, int,
                              cublasComputeType_t, cublasGemmAlgo_t) = nullptr;
    cublasHandle_t handle[kMaxDevices] = {};
};

Cublas& cublas()
{
    static Cublas c;
    static std::once_flag once;
    std::call_once(once, [] {
        void* lib = nullptr;
        for (const char* name : {"libcublas.so.12", "libcublas.so", "/usr/local/cuda/lib64/libcublas.so.12"}) {
            lib = dlopen(name, RTLD_NOW | RTLD_GLOBAL);
            if (lib) break;
        }
        if (!lib) return;
        c.create = reinterpret_cast<decltype(c.create)>(dlsym(lib, "cublasCreate_v2"));
        c.set_stream = reinterpret_cast<decltype(c.set_stream)>(dlsym(lib, "cublasSetStream_v2"));
        c.gemm_ex = reinterpret_cast<decltype(c.gemm_ex)>(dlsym(lib, "cublasGemmEx"));
    });
    if (!c.create || !c.set_stream || !c.gemm_ex) throw std::runtime_error("prefill hgemm: cuBLAS (libcublas.so.12) could not be loaded");
    return c;
}

std::mutex g_hgemm_mu;

}  // namespace
}  // namespace berth

extern "C" int berth_prefill_hgemm(const void* a, const void* b, void* c, int size_m, int size_k, int size_n, int ldc, int c_fp32,
                                   void* stream)
{
    using namespace berth;
    CallState& st = prefill_state();
    return guarded(st, [&] {
        if (!a || !b || !c) throw std::runtime_error("prefill hgemm: null device pointer");
        if (size_m < 1 || size_k < 1 || size_n < 1 || ldc < size_n) throw std::runtime_error("prefill hgemm: bad shape");
        Cublas& cb = cublas();
        const int device = current_device();
        std::lock_guard<std::mutex> lock(g_hgemm_mu);
        if (!cb.handle[device] && cb.create(&cb.handle[device]) != CUBLAS_STATUS_SUCCESS)
            throw std::runtime_error("prefill hgemm: cublasCreate failed");
        if (cb.set_stream(cb.handle[device], (cudaStream_t) stream) != CUBLAS_STATUS_SUCCESS)
            throw std::runtime_error("prefill hgemm: cublasSetStream failed");
        // row-major c = a . b is column-major c^T (n x m, ld ldc) = b^T (n x k, ld n) . a^T (k x m, ld k)
        const float alpha = 1.f, beta = 0.f;
        const cublasStatus_t rc = cb.gemm_ex(cb.handle[device], CUBLAS_OP_N, CUBLAS_OP_N, size_n, size_m, size_k, &alpha, b, CUDA_R_16F,
                                             size_n, a, CUDA_R_16F, size_k, &beta, c, c_fp32 ? CUDA_R_32F : CUDA_R_16F, ldc,
                                             CUBLAS_COMPUTE_32F, CUBLAS_GEMM_DEFAULT_TENSOR_OP);
        if (rc != CUBLAS_STATUS_SUCCESS) throw std::runtime_error("prefill hgemm: cublasGemmEx failed (" + std::to_string(int(rc)) + ")");
        cuda_ok(cudaPeekAtLastError(), "cublasGemmEx");
        st.launch = "cublasGemmEx";
    });
}
