// The library matrix product (cuBLAS), called directly: the same kernels as through torch.mm at a
// third of the host time per call, which counts when a step launches hundreds of kernels.
//
// cuBLAS is found at run time in the process (the host program has loaded it already), so this
// library has no link-time dependency on it.  Row-major y (M x N) = x (M x K) . W (K x N) is the
// column-major product y^T = W^T . x^T: W and x are passed as they lie.
#include "common.cuh"
#include <cublas_v2.h>
#include <dlfcn.h>
#include <mutex>

namespace {

typedef cublasStatus_t (*CreateFn)(cublasHandle_t*);
typedef cublasStatus_t (*SetStreamFn)(cublasHandle_t, cudaStream_t);
typedef cublasStatus_t (*SetWorkspaceFn)(cublasHandle_t, void*, size_t);
typedef cublasStatus_t (*GemmExFn)(cublasHandle_t, cublasOperation_t, cublasOperation_t, int, int, int, const void*,
                                   const void*, cudaDataType, int, const void*, cudaDataType, int, const void*, void*,
                                   cudaDataType, int, cublasComputeType_t, cublasGemmAlgo_t);

struct Blas {
    cublasHandle_t handle = nullptr;
    SetStreamFn set_stream = nullptr;
    SetWorkspaceFn set_workspace = nullptr;
    GemmExFn gemm_ex = nullptr;
    bool ok = false;
    int device = -1;                 // the device that was current when the handle was made
    void* workspace = nullptr;       // given once by the caller; set again after every change of stream
    size_t workspace_bytes = 0;
    cudaStream_t stream = nullptr;
    bool stream_set = false;
};

Blas& blas() {
    static Blas b;
    static std::once_flag once;
    std::call_once(once, []() {
        void* lib = dlopen("libcublas.so.12", RTLD_NOW | RTLD_NOLOAD);
        if (!lib) lib = dlopen("libcublas.so.12", RTLD_NOW);
        if (!lib) lib = dlopen("libcublas.so", RTLD_NOW);
        if (!lib) return;
        CreateFn create = reinterpret_cast<CreateFn>(dlsym(lib, "cublasCreate_v2"));
        b.set_stream = reinterpret_cast<SetStreamFn>(dlsym(lib, "cublasSetStream_v2"));
        b.set_workspace = reinterpret_cast<SetWorkspaceFn>(dlsym(lib, "cublasSetWorkspace_v2"));
        b.gemm_ex = reinterpret_cast<GemmExFn>(dlsym(lib, "cublasGemmEx"));
        if (!create || !b.set_stream || !b.set_workspace || !b.gemm_ex) return;
        if (create(&b.handle) != CUBLAS_STATUS_SUCCESS) return;
        cudaGetDevice(&b.device);
        b.ok = true;
    });
    return b;
}

}  // namespace

// 1 if the library was found and a handle made.  `workspace` (device memory that the caller keeps
// alive) is what the library uses for split-K partial sums: with a fixed workspace its calls can be
// captured into CUDA graphs.  cublasSetStream puts the handle's workspace back to the library's own
// pool, so the workspace is remembered here and set again whenever the stream changes.
TIS_API int tis_gemm_library_init(void* workspace, size_t bytes) {
    Blas& b = blas();
    if (!b.ok) return 0;
    b.workspace = workspace;
    b.workspace_bytes = bytes;
    if (workspace && bytes && b.set_workspace(b.handle, workspace, bytes) != CUBLAS_STATUS_SUCCESS) return 0;
    return 1;
}

// y = x . W, bfloat16 operands, float32 accumulation; y bfloat16 or (out_f32) float32.  Strides in elements.
TIS_API int tis_gemm_library(const void* x, int ldx, const void* w, int ldw, void* out, int ldo, int M, int N, int K,
                             int out_f32, cudaStream_t stream) {
    if (M <= 0 || N <= 0) return TIS_OK;
    Blas& b = blas();
    if (!b.ok) {
        tis_set_error("gemm_library: cuBLAS was not found in the process");
        return TIS_CUDA_ERROR;
    }
    int dev = -1;
    cudaGetDevice(&dev);
    if (dev != b.device) {
        tis_set_error("gemm_library: the handle was made on device %d, device %d is current", b.device, dev);
        return TIS_CUDA_ERROR;
    }
    if (!b.stream_set || b.stream != stream) {
        if (b.set_stream(b.handle, stream) != CUBLAS_STATUS_SUCCESS) {
            tis_set_error("gemm_library: cublasSetStream failed");
            return TIS_CUDA_ERROR;
        }
        if (b.workspace && b.workspace_bytes &&
            b.set_workspace(b.handle, b.workspace, b.workspace_bytes) != CUBLAS_STATUS_SUCCESS) {
            tis_set_error("gemm_library: cublasSetWorkspace failed");
            return TIS_CUDA_ERROR;
        }
        b.stream = stream;
        b.stream_set = true;
    }
    const float alpha = 1.f, beta = 0.f;
    const cublasStatus_t st = b.gemm_ex(b.handle, CUBLAS_OP_N, CUBLAS_OP_N, N, M, K, &alpha, w, CUDA_R_16BF, ldw, x,
                                        CUDA_R_16BF, ldx, &beta, out, out_f32 ? CUDA_R_32F : CUDA_R_16BF, ldo,
                                        CUBLAS_COMPUTE_32F, CUBLAS_GEMM_DEFAULT);
    if (st != CUBLAS_STATUS_SUCCESS) {
        tis_set_error("gemm_library: cublasGemmEx failed with status %d (M %d N %d K %d)", (int)st, M, N, K);
        return TIS_CUDA_ERROR;
    }
    return TIS_OK;
}
