// Shared device helpers: storage types, 32-bit conversions, block reductions.
//
// Every kernel of this library computes in 32-bit floating point; T is only the type
// in which activations, weights and cache pages are stored (float or bfloat16).
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>

#define TIS_API extern "C" __attribute__((visibility("default")))

// Error codes returned by the extern "C" launchers (0 = launched).
enum TisStatus : int {
    TIS_OK = 0,
    TIS_BAD_SIZE = 1,      // a size the kernel refuses (message in tis_last_error())
    TIS_BAD_DTYPE = 2,
    TIS_CUDA_ERROR = 3,
};

void tis_set_error(const char* fmt, ...);
int tis_check_launch(const char* what);

enum TisDtype : int { TIS_F32 = 0, TIS_BF16 = 1 };

typedef __nv_bfloat16 bf16;

__device__ __forceinline__ float to_f32(float x) { return x; }
__device__ __forceinline__ float to_f32(bf16 x) { return __bfloat162float(x); }

template <typename T> __device__ __forceinline__ T from_f32(float x);
template <> __device__ __forceinline__ float from_f32<float>(float x) { return x; }
template <> __device__ __forceinline__ bf16 from_f32<bf16>(float x) { return __float2bfloat16_rn(x); }

// ---- 16-byte vectors: 8 bfloat16 or 4 float -------------------------------------------
template <typename T> struct Vec16;
template <> struct Vec16<float> {
    static constexpr int N = 4;
    static __device__ __forceinline__ void load(const float* p, float (&v)[4]) {
        const float4 x = *reinterpret_cast<const float4*>(p);
        v[0] = x.x; v[1] = x.y; v[2] = x.z; v[3] = x.w;
    }
    static __device__ __forceinline__ void store(float* p, const float (&v)[4]) {
        *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
    }
};
template <> struct Vec16<bf16> {
    static constexpr int N = 8;
    static __device__ __forceinline__ void load(const bf16* p, float (&v)[8]) {
        const uint4 raw = *reinterpret_cast<const uint4*>(p);
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float2 f = __bfloat1622float2(h[i]);
            v[2 * i] = f.x; v[2 * i + 1] = f.y;
        }
    }
    static __device__ __forceinline__ void store(bf16* p, const float (&v)[8]) {
        uint4 raw;
        __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&raw);
#pragma unroll
        for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
        *reinterpret_cast<uint4*>(p) = raw;
    }
};

// ---- cache row format ---------------------------------------------------------------------
// A cache row (keys or values of one position and kv head: hd elements) is stored as 16-byte
// chunks permuted by the position.  Rows of a multiple of eight chunks (head sizes that are
// multiples of 64 in bfloat16): logical chunk c lies at chunk c XOR (position mod 8), the
// 128-byte swizzle of the tensor-core operand layouts applied in memory.  Other rows: at chunk
// (c + position) mod (chunks per row).  Either way a run of rows copied unchanged into shared
// memory (one bulk copy per page) is read by ldmatrix without bank conflicts, with no padding
// between rows; and a box of 64 elements x 8k rows of the first kind, copied by the TMA engine
// without swizzling, is at once the canonical 128-byte-swizzled operand tile of tcgen05.mma.
__device__ __forceinline__ int cache_chunk(int logical_chunk, int position, int chunks_per_row) {
    return (chunks_per_row & 7) == 0 ? (logical_chunk ^ (position & 7)) : (logical_chunk + position) % chunks_per_row;
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
// The factor a norm of the RMS family multiplies a row with, from the row's sum of squares s over a width d:
// kind 0: sqrt(d) / (sqrt(s) + eps) (eps added to the L2 norm); kind 1: rsqrt(s / d + eps).  Both are
// num / (sqrt(s * mul + add) + plus) with constants the host works out, so that a kernel has no case to tell apart.
enum { TIS_NORM_L2_EPS = 0, TIS_NORM_MEAN_EPS = 1 };
struct NormFactor {
    float num, mul, add, plus;
    __device__ __forceinline__ float of(float sum_sq) const { return num / (sqrtf(fmaf(sum_sq, mul, add)) + plus); }
};
inline NormFactor norm_factor(int kind, int width, float eps) {
    NormFactor f;
    const float d = (float)(width > 0 ? width : 1);
    if (kind == TIS_NORM_MEAN_EPS) { f.num = 1.f; f.mul = 1.f / d; f.add = eps; f.plus = 0.f; }
    else { f.num = sqrtf(d); f.mul = 1.f; f.add = 0.f; f.plus = eps; }
    return f;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Block-wide sum / max for blockDim.x a multiple of 32 (<= 1024); `red` holds 33 floats.
// All threads get the result.  Two calls need no barrier in between from the caller.
__device__ __forceinline__ float block_sum(float v, float* red) {
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = blockDim.x >> 5;
    v = warp_sum(v);
    __syncthreads();                 // `red` may still be read from an earlier call
    if (lane == 0) red[w] = v;
    __syncthreads();
    float t = (lane < nw) ? red[lane] : 0.f;
    t = warp_sum(t);
    return t;
}
__device__ __forceinline__ float block_max(float v, float* red) {
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = blockDim.x >> 5;
    v = warp_max(v);
    __syncthreads();
    if (lane == 0) red[w] = v;
    __syncthreads();
    float t = (lane < nw) ? red[lane] : -INFINITY;
    t = warp_max(t);
    return t;
}

// ---- programmatic dependent launch -------------------------------------------------------
// Kernels of a step form a chain, each reading what the one before wrote.  Launched with the
// attribute below a kernel may start while the kernel before it still runs: it tells the
// hardware at once that the kernel after it may start too (pdl_launch_dependents), does what
// does not depend on the kernel before (metadata, weights), and then waits for it (pdl_wait)
// before it reads or writes anything else.  Inside a CUDA graph the launches become
// programmatic edges.  TIS_NO_PDL=1 in the environment turns the attribute off.
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;\n" ::); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;\n" ::: "memory"); }

bool tis_pdl_enabled();

template <typename... KArgs, typename... Args>
inline cudaError_t tis_launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                              Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = tis_pdl_enabled() ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}

// Dispatch on the storage dtype inside a launcher.
#define TIS_DISPATCH_DTYPE(dtype, T, ...)                                   \
    do {                                                                    \
        if ((dtype) == TIS_F32) { typedef float T; __VA_ARGS__; }           \
        else if ((dtype) == TIS_BF16) { typedef bf16 T; __VA_ARGS__; }      \
        else { tis_set_error("unknown dtype code %d", (int)(dtype)); return TIS_BAD_DTYPE; } \
    } while (0)
