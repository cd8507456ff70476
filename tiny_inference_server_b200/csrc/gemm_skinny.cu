// Matrix products with few rows: y (M x N) = x (M x K) . W (K x N), bfloat16, M <= 64 —
// the projections of a decode step, which are bound by streaming W from HBM once.
//
// A CTA owns a strip of 64 columns of W and one share of K; the `ksplit` CTAs that share
// a strip form a thread-block cluster and add their partial sums through distributed
// shared memory (pushed to the CTA that owns a row: cluster_reduce.cuh), so no partial result
// touches global memory and the output is written once, through the epilogue (plain store, or
// SwiGLU gating of a [32 gate | 32 up] strip).
//
// Two more things let a pre-norm block run without a kernel for its norms.  The product that ends a
// mixer or a feed-forward can add its result to the float32 residual stream itself (EPI_RESIDUAL): it
// writes the new stream, the stream times the weight of the norm that follows (bfloat16: the rows of the
// next product) and, per row and strip, the sum of squares of the new stream.  And the product that reads
// such rows multiplies row r of its result by sqrt(width) / (sqrt(sum of the row's partial sums) + eps):
// the norm's factor of a row is a scalar, so it can be applied after the product instead of before.
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
#include "cluster_reduce.cuh"
#include "timeline.cuh"
#include <cooperative_groups.h>

namespace {

using cluster_reduce::EPI_STORE;
using cluster_reduce::EPI_SWIGLU;
using cluster_reduce::EPI_RESIDUAL;

constexpr int BN = 64;            // columns of a strip
constexpr int BK = 64;            // rows of K per tile
constexpr int NTH = 128;
constexpr int WROW = BN + 8;      // padded shared-memory rows: conflict-free ldmatrix
constexpr int XROW = BK + 8;
constexpr int MAX_STAGES = 4;     // W tiles a CTA keeps in shared memory (9 KB each), at most 8

struct GemmParams {
    const bf16* x; int ldx;
    const bf16* w; int ldw;
    int K;
    int kc;                       // rows of K per CTA of a cluster (a multiple of BK)
    int stages;                   // ring length: min(tiles per CTA, MAX_STAGES)
    cluster_reduce::Epilogue e;   // rows, columns, where the result goes
    TIS_TIMELINE_MEMBER           // (instrumented builds only; stamps: 0 entry, 1 weights ordered, 2 dependency wait over,
                                  //  3 first tile ready, 4 loop done, 5 cluster barrier passed, 6 stored)
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
        const bool ok = k < k_end && n < p.e.N;
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
        const bool ok = r < p.e.M && k < k_end;
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
    float* recv = reinterpret_cast<float*>(x_st + STAGES * X_ELEMS);  // partial sums pushed by the cluster
    __shared__ __align__(8) unsigned long long recv_bar;
    __shared__ float pair[2][BN];
    __shared__ float row_factor[MT * 16];

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    cg::cluster_group cluster = cg::this_cluster();
    const unsigned rank = cluster.block_rank(), ksplit = cluster.num_blocks();
    const int n0 = blockIdx.x * BN;
    const int k_begin = (int)rank * p.kc;
    const int k_end = min(p.K, k_begin + p.kc);
    const int nkt = k_end > k_begin ? (k_end - k_begin + BK - 1) / BK : 0;

    // let the kernel after this one start its own prologue as soon as it can
    TIS_STAMP(p, 0);
    asm volatile("griddepcontrol.launch_dependents;\n" ::);
    if (tid == 0) cluster_reduce::init_barrier(&recv_bar, rank, ksplit, p.e.M);
    cluster_reduce::cluster_arrive();        // waited for after the loop: by then every CTA's barrier is ready

    // weights first: they depend on nothing.  With at most `stages` tiles per CTA the whole share
    // of W is ordered here, before the wait, and streams in while the kernel before still runs.
    const int pre = nkt < STAGES ? nkt : (nkt == STAGES ? STAGES : STAGES - 1);
    for (int s = 0; s < pre; ++s) load_w(w_st + s * W_ELEMS, p, k_begin + s * BK, k_end, n0, tid);
    cp_commit();
    // x is the output of the kernel before this one
    TIS_STAMP(p, 1);
    asm volatile("griddepcontrol.wait;\n" ::: "memory");
    TIS_STAMP(p, 2);
    for (int s = 0; s < pre; ++s) {
        load_x<MT>(x_st + s * X_ELEMS, p, k_begin + s * BK, k_end, tid);
        cp_commit();                     // one group per tile: tile s is ready when all but pre-1-s groups are done
    }
    // the norm's factor of each row, from the partial sums the kernel before left: the loads now, the rest after the loop
    cluster_reduce::RowFactorLoads<MT> factors;
    factors.order(p.e, row_factor, tid);

    float acc[MT][2][4];
#pragma unroll
    for (int m = 0; m < MT; ++m)
#pragma unroll
        for (int j = 0; j < 2; ++j) { acc[m][j][0] = acc[m][j][1] = acc[m][j][2] = acc[m][j][3] = 0.f; }

    // a tile's products: all fragments of the tile first, then independent chains of accumulators (one per
    // k16 step for up to 32 rows, two otherwise), so that the latency of a step is not paid once per step
    constexpr int CHAINS = MT <= 2 ? BK / 16 : 2;
    float accs[CHAINS - 1][MT][2][4];
#pragma unroll
    for (int ch = 0; ch < CHAINS - 1; ++ch)
#pragma unroll
        for (int m = 0; m < MT; ++m)
#pragma unroll
            for (int j = 0; j < 2; ++j) { accs[ch][m][j][0] = accs[ch][m][j][1] = accs[ch][m][j][2] = accs[ch][m][j][3] = 0.f; }
    auto tile_products = [&](const bf16* ws, const bf16* xs) {
        unsigned b[BK / 16][4];
#pragma unroll
        for (int kk = 0; kk < BK / 16; ++kk)
            // rows k 16kk..16kk+15, the warp's 16 columns: (k 0-7, n 0-7), (k 8-15, n 0-7), (k 0-7, n 8-15), (k 8-15, n 8-15)
            ldsm_x4_t(b[kk], ws + (kk * 16 + (((lane >> 3) & 1) << 3) + (lane & 7)) * WROW + warp * 16 + ((lane >> 4) << 3));
#pragma unroll
        for (int m = 0; m < MT; ++m) {
            unsigned a[BK / 16][4];
#pragma unroll
            for (int kk = 0; kk < BK / 16; ++kk)
                // rows m*16.., k 16kk..: (r 0-7, k 0-7), (r 8-15, k 0-7), (r 0-7, k 8-15), (r 8-15, k 8-15)
                ldsm_x4(a[kk], xs + (m * 16 + (((lane >> 3) & 1) << 3) + (lane & 7)) * XROW + kk * 16 + ((lane >> 4) << 3));
#pragma unroll
            for (int kk = 0; kk < BK / 16; ++kk) {
                const int ch = kk % CHAINS;
                if (ch == 0) {
                    mma16816(acc[m][0], a[kk], b[kk][0], b[kk][1]);
                    mma16816(acc[m][1], a[kk], b[kk][2], b[kk][3]);
                } else {
                    mma16816(accs[ch - 1][m][0], a[kk], b[kk][0], b[kk][1]);
                    mma16816(accs[ch - 1][m][1], a[kk], b[kk][2], b[kk][3]);
                }
            }
        }
    };

    if (nkt <= STAGES) {
        // the whole share is in flight already: one wait, one barrier, no barrier between tiles
        cp_wait<0>();
        __syncthreads();
        TIS_STAMP(p, 3);
        for (int it = 0; it < nkt; ++it) tile_products(w_st + it * W_ELEMS, x_st + it * X_ELEMS);
    } else {
        for (int it = 0; it < nkt; ++it) {
            // groups in flight after tile `it`: the x tiles it+1..pre-1 of the prologue, or the
            // refills ordered in the iterations before
            const int later = it < pre ? (pre - 1 - it) + (it > 0 ? it : 0) : STAGES - 2;
            if (later <= 0) cp_wait<0>();
            else if (later == 1) cp_wait<1>();
            else if (later == 2) cp_wait<2>();
            else if (later == 3) cp_wait<3>();
            else if (later == 4) cp_wait<4>();
            else if (later == 5) cp_wait<5>();
            else if (later == 6) cp_wait<6>();
            else cp_wait<7>();
            __syncthreads();
            if (it == 0) TIS_STAMP(p, 3);
            const int nx = it + STAGES - 1;        // the stage of tile it-1 is free now
            if (nx < nkt) {
                load_w(w_st + (nx % STAGES) * W_ELEMS, p, k_begin + nx * BK, k_end, n0, tid);
                load_x<MT>(x_st + (nx % STAGES) * X_ELEMS, p, k_begin + nx * BK, k_end, tid);
            }
            cp_commit();
            tile_products(w_st + (it % STAGES) * W_ELEMS, x_st + (it % STAGES) * X_ELEMS);
        }
    }
#pragma unroll
    for (int m = 0; m < MT; ++m)
#pragma unroll
        for (int j = 0; j < 2; ++j)
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int ch = 0; ch < CHAINS - 1; ++ch) acc[m][j][i] += accs[ch][m][j][i];
    TIS_STAMP(p, 4);
    cp_wait<0>();
    factors.finish(p.e, row_factor, tid);
    __syncthreads();                    // row_factor is written (also when this CTA had no tile)
    cluster_reduce::cluster_wait();     // every CTA of the cluster has initialised its barrier
    TIS_STAMP(p, 5);
    cluster_reduce::push_reduce_store<MT>(acc, p.e, recv, &recv_bar, pair, row_factor, rank, ksplit, blockIdx.x,
                                          gridDim.x, tid);
    TIS_STAMP(p, 6);
}

}  // namespace

// x (M x K, row stride ldx), w (K x N, row stride ldw), out (M x N or M x N/2 for the SwiGLU
// epilogue, row stride ldo): bfloat16.  ksplit: CTAs per strip (1, 2, 4 or 8).
//
// in_ss (may be null): [M][in_parts] float32 partial sums of squares; row r of the product is multiplied by
// the norm's factor norm_factor(in_kind, in_width, in_eps).of(sum of in_ss[r]) (common.cuh) before the epilogue.
// epi 2 (EPI_RESIDUAL): res [M][ldr] float32 += product; out = bfloat16(res * norm_w[column]);
// out_ss [M][ceil(N / 64)] = sums of squares of the new res by strip of 64 columns.
// fault (may be null): set to 8 when the wait for the cluster's partial sums runs out.
TIS_API int tis_gemm_skinny_fused(const void* x, int ldx, const void* w, int ldw, void* out, int ldo, int M, int N, int K,
                                  int ksplit, int epi, const float* in_ss, int in_parts, float in_eps, int in_width, int in_kind,
                                  float* res, int ldr, const float* norm_w, float* out_ss, int* fault,
                                  cudaStream_t stream) {
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
    if (epi < EPI_STORE || epi > EPI_RESIDUAL) {
        tis_set_error("gemm_skinny: unknown epilogue %d", epi);
        return TIS_BAD_SIZE;
    }
    if (epi == EPI_SWIGLU && N % 64) {
        tis_set_error("gemm_skinny: the SwiGLU epilogue needs N %d to be a multiple of 64", N);
        return TIS_BAD_SIZE;
    }
    if (epi == EPI_RESIDUAL && (res == nullptr || norm_w == nullptr || out_ss == nullptr || ldr % 2 || ldo % 2 ||
                                (reinterpret_cast<uintptr_t>(res) | reinterpret_cast<uintptr_t>(norm_w)) % 8 ||
                                reinterpret_cast<uintptr_t>(out) % 4)) {
        tis_set_error("gemm_skinny: the residual epilogue needs the stream, the norm's weight and room for the partial "
                      "sums, even row strides (%d, %d) and aligned pointers", ldr, ldo);
        return TIS_BAD_SIZE;
    }
    if (in_ss != nullptr && (in_parts <= 0 || in_width <= 0 || in_kind < TIS_NORM_L2_EPS || in_kind > TIS_NORM_MEAN_EPS)) {
        tis_set_error("gemm_skinny: %d partial sums a row over a width of %d, norm kind %d", in_parts, in_width, in_kind);
        return TIS_BAD_SIZE;
    }
    GemmParams p;
    p.x = (const bf16*)x; p.ldx = ldx; p.w = (const bf16*)w; p.ldw = ldw; p.K = K;
    p.e.out = (bf16*)out; p.e.ldo = ldo; p.e.M = M; p.e.N = N; p.e.epi = epi;
    p.e.in_ss = in_ss; p.e.in_parts = in_parts; p.e.in_factor = norm_factor(in_kind, in_width, in_eps);
    p.e.res = res; p.e.ldr = ldr; p.e.norm_w = norm_w; p.e.out_ss = out_ss; p.e.fault = fault;
    TIS_TIMELINE_TAKE(p);
    p.kc = ((K + ksplit - 1) / ksplit + BK - 1) / BK * BK;
    const int mt = M <= 16 ? 1 : (M <= 32 ? 2 : 4);
    const int tiles = p.kc / BK;
    p.stages = tiles < MAX_STAGES ? tiles : MAX_STAGES;
    const size_t stage = (size_t)p.stages * (BK * WROW + mt * 16 * XROW) * sizeof(bf16);
    const size_t smem = stage + cluster_reduce::recv_floats(mt * 16, ksplit) * sizeof(float);

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
        cudaFuncSetAttribute(gemm_skinny_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, 224 * 1024);
        cudaFuncSetAttribute(gemm_skinny_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, 224 * 1024);
        cudaFuncSetAttribute(gemm_skinny_kernel<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, 224 * 1024);
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

TIS_API int tis_gemm_skinny(const void* x, int ldx, const void* w, int ldw, void* out, int ldo, int M, int N, int K,
                            int ksplit, int epi, cudaStream_t stream) {
    if (epi == EPI_RESIDUAL) {
        tis_set_error("gemm_skinny: the residual epilogue goes through tis_gemm_skinny_fused");
        return TIS_BAD_SIZE;
    }
    return tis_gemm_skinny_fused(x, ldx, w, ldw, out, ldo, M, N, K, ksplit, epi, nullptr, 0, 0.f, 0, 0, nullptr, 0, nullptr,
                                 nullptr, nullptr, stream);
}
