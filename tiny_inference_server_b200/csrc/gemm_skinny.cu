// Matrix products with few rows: y (M x N) = x (M x K) . W (K x N), bfloat16, M <= 64 —
// the projections of a decode step, which are bound by streaming W from HBM once.
//
// A CTA owns a strip of 64 columns of W and one share of K; the `ksplit` CTAs that share
// a strip form a thread-block cluster and add their partial sums through distributed
// shared memory, so no partial result touches global memory and the output is written once,
// through the epilogue (plain store, or SwiGLU gating of a [32 gate | 32 up] strip).
//
// W tiles (64 rows of K x 64 columns) and x tiles come by cp.async into up to eight stages
// (all of a CTA's share of W when it is at most 512 rows of K, else a ring);
// products are mma.sync m16n8k16 with float32 accumulation (x as the row operand from
// ldmatrix, W as the column operand from ldmatrix.trans).
//
// Programmatic dependent launch: the kernel is launched so that it may start while the kernel
// before it still runs.  It orders its first W tiles at once — weights do not depend on
// anything — and only then waits (griddepcontrol.wait) for the kernel before it, whose output
// is x.  So the weight stream of one projection overlaps the tail of the kernel before.
#include "common.cuh"
#include <cooperative_groups.h>

namespace {

constexpr int BN = 64;            // columns of a strip
constexpr int BK = 64;            // rows of K per tile
constexpr int NTH = 128;
constexpr int WROW = BN + 8;      // padded shared-memory rows: conflict-free ldmatrix
constexpr int XROW = BK + 8;
constexpr int MAX_STAGES = 4;     // W tiles a CTA keeps in shared memory (9 KB each), at most 8

enum { EPI_STORE = 0, EPI_SWIGLU = 1 };

struct GemmParams {
    const bf16* x; int ldx;
    const bf16* w; int ldw;
    bf16* out; int ldo;
    int M, N, K;
    int kc;                       // rows of K per CTA of a cluster (a multiple of BK)
    int epi;
    int stages;                   // ring length: min(tiles per CTA, MAX_STAGES)
};

__device__ __forceinline__ void cp16(void* smem, const void* gmem, int bytes) {
    const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(s), "l"(gmem), "r"(bytes));
}
__device__ __forceinline__ void cp_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void cp_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }

__device__ __forceinline__ void ldsm_x4(unsigned (&r)[4], const void* smem) {
    const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s));
}
__device__ __forceinline__ void ldsm_x4_t(unsigned (&r)[4], const void* smem) {
    const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s));
}
__device__ __forceinline__ void mma16816(float (&c)[4], const unsigned (&a)[4], unsigned b0, unsigned b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// W tile: rows k0..k0+63 (zero beyond k_end), columns n0..n0+63 (zero beyond N)
__device__ __forceinline__ void load_w(bf16* ws, const GemmParams& p, int k0, int k_end, int n0, int tid) {
#pragma unroll
    for (int i = tid; i < BK * (BN / 8); i += NTH) {
        const int r = i >> 3, c = i & 7;
        const int k = k0 + r, n = n0 + c * 8;
        const bool ok = k < k_end && n < p.N;
        cp16(ws + r * WROW + c * 8, ok ? p.w + (size_t)k * p.ldw + n : p.w, ok ? 16 : 0);
    }
}
// x tile: rows 0..MT*16-1 (zero beyond M), K columns k0..k0+63 (zero beyond k_end)
template <int MT>
__device__ __forceinline__ void load_x(bf16* xs, const GemmParams& p, int k0, int k_end, int tid) {
#pragma unroll
    for (int i = tid; i < MT * 16 * (BK / 8); i += NTH) {
        const int r = i >> 3, c = i & 7;
        const int k = k0 + c * 8;
        const bool ok = r < p.M && k < k_end;
        cp16(xs + r * XROW + c * 8, ok ? p.x + (size_t)r * p.ldx + k : p.x, ok ? 16 : 0);
    }
}

template <int MT>
__global__ void __launch_bounds__(NTH) gemm_skinny_kernel(const GemmParams p) {
    namespace cg = cooperative_groups;
    extern __shared__ __align__(16) unsigned char smem[];
    constexpr int W_ELEMS = BK * WROW, X_ELEMS = MT * 16 * XROW;
    const int STAGES = p.stages;
    bf16* w_st = reinterpret_cast<bf16*>(smem);                       // STAGES x W tile
    bf16* x_st = w_st + STAGES * W_ELEMS;                             // STAGES x x tile
    float* red = reinterpret_cast<float*>(smem);                      // after the loop: [MT*16][BN] partial sums

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    cg::cluster_group cluster = cg::this_cluster();
    const unsigned rank = cluster.block_rank(), ksplit = cluster.num_blocks();
    const int n0 = blockIdx.x * BN;
    const int k_begin = (int)rank * p.kc;
    const int k_end = min(p.K, k_begin + p.kc);
    const int nkt = k_end > k_begin ? (k_end - k_begin + BK - 1) / BK : 0;

    // let the kernel after this one start its own prologue as soon as it can
    asm volatile("griddepcontrol.launch_dependents;\n" ::);

    // weights first: they depend on nothing.  With at most `stages` tiles per CTA the whole share
    // of W is ordered here, before the wait, and streams in while the kernel before still runs.
    const int pre = nkt < STAGES ? nkt : (nkt == STAGES ? STAGES : STAGES - 1);
    for (int s = 0; s < pre; ++s) load_w(w_st + s * W_ELEMS, p, k_begin + s * BK, k_end, n0, tid);
    cp_commit();
    // x is the output of the kernel before this one
    asm volatile("griddepcontrol.wait;\n" ::: "memory");
    for (int s = 0; s < pre; ++s) {
        load_x<MT>(x_st + s * X_ELEMS, p, k_begin + s * BK, k_end, tid);
        cp_commit();                     // one group per tile: tile s is ready when all but pre-1-s groups are done
    }

    float acc[MT][2][4];
#pragma unroll
    for (int m = 0; m < MT; ++m)
#pragma unroll
        for (int j = 0; j < 2; ++j) { acc[m][j][0] = acc[m][j][1] = acc[m][j][2] = acc[m][j][3] = 0.f; }

    for (int it = 0; it < nkt; ++it) {
        // groups in flight after tile `it`: the x tiles it+1..pre-1 of the prologue, or (ring) the
        // refills ordered in the iterations before
        const int later = it < pre ? (pre - 1 - it) + (it > 0 && nkt > STAGES ? it : 0) : STAGES - 2;
        if (later <= 0) cp_wait<0>();
        else if (later == 1) cp_wait<1>();
        else if (later == 2) cp_wait<2>();
        else if (later == 3) cp_wait<3>();
        else if (later == 4) cp_wait<4>();
        else if (later == 5) cp_wait<5>();
        else if (later == 6) cp_wait<6>();
        else cp_wait<7>();
        __syncthreads();
        if (nkt > STAGES) {
            const int nx = it + STAGES - 1;        // the stage of tile it-1 is free now
            if (nx < nkt) {
                load_w(w_st + (nx % STAGES) * W_ELEMS, p, k_begin + nx * BK, k_end, n0, tid);
                load_x<MT>(x_st + (nx % STAGES) * X_ELEMS, p, k_begin + nx * BK, k_end, tid);
            }
            cp_commit();
        }
        const bf16* ws = w_st + (it % STAGES) * W_ELEMS;
        const bf16* xs = x_st + (it % STAGES) * X_ELEMS;
#pragma unroll
        for (int kk = 0; kk < BK / 16; ++kk) {
            unsigned b[4];
            // rows k 16kk..16kk+15, the warp's 16 columns: (k 0-7, n 0-7), (k 8-15, n 0-7), (k 0-7, n 8-15), (k 8-15, n 8-15)
            ldsm_x4_t(b, ws + (kk * 16 + (((lane >> 3) & 1) << 3) + (lane & 7)) * WROW + warp * 16 + ((lane >> 4) << 3));
#pragma unroll
            for (int m = 0; m < MT; ++m) {
                unsigned a[4];
                // rows m*16.., k 16kk..: (r 0-7, k 0-7), (r 8-15, k 0-7), (r 0-7, k 8-15), (r 8-15, k 8-15)
                ldsm_x4(a, xs + (m * 16 + (((lane >> 3) & 1) << 3) + (lane & 7)) * XROW + kk * 16 + ((lane >> 4) << 3));
                mma16816(acc[m][0], a, b[0], b[1]);
                mma16816(acc[m][1], a, b[2], b[3]);
            }
        }
    }
    cp_wait<0>();
    __syncthreads();                    // all warps are done with the staging memory

    // partial sums of this CTA into shared memory
    const int g = lane >> 2, t = lane & 3;
#pragma unroll
    for (int m = 0; m < MT; ++m)
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            const int col = warp * 16 + j * 8 + 2 * t;
            red[(m * 16 + g) * BN + col] = acc[m][j][0];
            red[(m * 16 + g) * BN + col + 1] = acc[m][j][1];
            red[(m * 16 + g + 8) * BN + col] = acc[m][j][2];
            red[(m * 16 + g + 8) * BN + col + 1] = acc[m][j][3];
        }
    cluster.sync();

    // rank r adds up rows r, r + ksplit, ... over all CTAs of the cluster and writes them;
    // two rows at a time (threads 0-63 and 64-127), one column per thread
    __shared__ float pair[2][BN];
    const int half = tid >> 6, col = tid & 63;
    for (int base = (int)rank; base < p.M; base += 2 * (int)ksplit) {      // the same trips for every thread
        const int row = base + half * (int)ksplit;
        const bool valid = row < p.M;
        float sum = 0.f;
        if (valid)
            for (unsigned r = 0; r < ksplit; ++r) sum += cluster.map_shared_rank(red, r)[row * BN + col];
        if (p.epi == EPI_STORE) {
            if (valid && n0 + col < p.N) p.out[(size_t)row * p.ldo + n0 + col] = __float2bfloat16_rn(sum);
        } else {
            // the strip is [32 gate | 32 up]: out column strip*32 + j = silu(gate_j) * up_j
            pair[half][col] = sum;
            __syncthreads();
            if (valid && col < 32) {
                const float gt = pair[half][col], up = pair[half][col + 32];
                p.out[(size_t)row * p.ldo + blockIdx.x * 32 + col] = __float2bfloat16_rn(gt / (1.f + expf(-gt)) * up);
            }
            __syncthreads();
        }
    }
    cluster.sync();                     // nobody leaves while its shared memory may still be read
}

}  // namespace

// x (M x K, row stride ldx), w (K x N, row stride ldw), out (M x N or M x N/2 for the SwiGLU
// epilogue, row stride ldo): bfloat16.  ksplit: CTAs per strip (1, 2, 4 or 8).
TIS_API int tis_gemm_skinny(const void* x, int ldx, const void* w, int ldw, void* out, int ldo, int M, int N, int K,
                            int ksplit, int epi, cudaStream_t stream) {
    if (M <= 0 || N <= 0 || K <= 0) return TIS_OK;
    if (M > 64) {
        tis_set_error("gemm_skinny: %d rows; this kernel takes at most 64", M);
        return TIS_BAD_SIZE;
    }
    if (N % 8 || K % 8 || ldx % 8 || ldw % 8) {
        tis_set_error("gemm_skinny: N %d, K %d and the row strides %d, %d must be multiples of 8 (16-byte copies)",
                      N, K, ldx, ldw);
        return TIS_BAD_SIZE;
    }
    if (!(ksplit == 1 || ksplit == 2 || ksplit == 4 || ksplit == 8)) {
        tis_set_error("gemm_skinny: ksplit %d must be 1, 2, 4 or 8", ksplit);
        return TIS_BAD_SIZE;
    }
    if (epi == EPI_SWIGLU && N % 64) {
        tis_set_error("gemm_skinny: the SwiGLU epilogue needs N %d to be a multiple of 64", N);
        return TIS_BAD_SIZE;
    }
    GemmParams p;
    p.x = (const bf16*)x; p.ldx = ldx; p.w = (const bf16*)w; p.ldw = ldw; p.out = (bf16*)out; p.ldo = ldo;
    p.M = M; p.N = N; p.K = K; p.epi = epi;
    p.kc = ((K + ksplit - 1) / ksplit + BK - 1) / BK * BK;
    const int mt = M <= 16 ? 1 : (M <= 32 ? 2 : 4);
    const int tiles = p.kc / BK;
    p.stages = tiles < MAX_STAGES ? tiles : MAX_STAGES;
    const size_t stage = (size_t)p.stages * (BK * WROW + mt * 16 * XROW) * sizeof(bf16);
    const size_t redb = (size_t)mt * 16 * BN * sizeof(float);
    const size_t smem = stage > redb ? stage : redb;

    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((N + BN - 1) / BN, ksplit, 1);
    cfg.blockDim = dim3(NTH, 1, 1);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attrs[2];
    attrs[0].id = cudaLaunchAttributeClusterDimension;
    attrs[0].val.clusterDim.x = 1;
    attrs[0].val.clusterDim.y = ksplit;
    attrs[0].val.clusterDim.z = 1;
    attrs[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attrs[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attrs;
    cfg.numAttrs = tis_pdl_enabled() ? 2 : 1;
    cudaError_t e;
    static bool configured = false;
    if (!configured) {
        cudaFuncSetAttribute(gemm_skinny_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024);
        cudaFuncSetAttribute(gemm_skinny_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024);
        cudaFuncSetAttribute(gemm_skinny_kernel<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024);
        configured = true;
    }
    if (mt == 1) e = cudaLaunchKernelEx(&cfg, gemm_skinny_kernel<1>, p);
    else if (mt == 2) e = cudaLaunchKernelEx(&cfg, gemm_skinny_kernel<2>, p);
    else e = cudaLaunchKernelEx(&cfg, gemm_skinny_kernel<4>, p);
    if (e != cudaSuccess) {
        tis_set_error("gemm_skinny: %s", cudaGetErrorString(e));
        return TIS_CUDA_ERROR;
    }
    return tis_check_launch("gemm_skinny");
}
