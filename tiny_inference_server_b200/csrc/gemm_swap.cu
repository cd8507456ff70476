// Matrix products with up to 64 rows on the fifth-generation tensor cores, operands swapped:
// y (M x N) = x (M x K) . W (K x N), bfloat16 — computed as y^T = W^T . x^T, so that the 128 rows of a
// tcgen05.mma tile are 128 *columns of W* and its narrow side (16, 32 or 64) holds the rows of x.  The
// tensor cores then do no work on padding, the accumulator is 128 lanes x M columns of tensor memory,
// and W — the only operand of any size, streamed from HBM once — goes from the TMA engine to the tensor
// cores without passing through a thread: no ldmatrix, no mma.sync, no issue slots spent on it.
//
// A CTA owns a strip of 128 columns of W and one share of K; the CTAs that share a strip are a
// thread-block cluster and add their partial sums through distributed shared memory (as gemm_skinny.cu).
// Roles, specialised by warp:
//   warp 0   one lane orders W (two 64 x 64 boxes a step of 64 of K, 128-byte swizzle: W^T as the MN-major
//            first operand, used as it lies) into a ring of stages — before the dependency wait, weights
//            depend on nothing — and then the matching boxes of x (64 of K x M rows: the K-major second
//            operand) after it;
//   warp 1   owns the tensor memory; one lane issues four tcgen05.mma (k16) per stage and hands the
//            stage back with tcgen05.commit;
//   warps 2-5 read the accumulator (tcgen05.ld: a thread holds the M values of its column), leave them
//            in shared memory, and after the cluster barrier each CTA adds up and stores its share of the
//            rows (plain store, or SwiGLU gating of [32 gate | 32 up] column blocks).
// Every wait on an mbarrier is bounded; one that runs out sets the fault word, every role leaves its
// loop, and the tensor memory is freed.
#include "tc_common.cuh"
#include <cooperative_groups.h>

namespace {

using namespace tc;

constexpr int BN = 128;                     // columns of W a CTA owns (the M of the tcgen05 tile)
constexpr int BK = 64;                      // 64 bfloat16 = one 128-byte swizzle row
constexpr int NTH = 192;
constexpr int W_BYTES = 2 * 64 * BK * 2;    // two boxes of 64 rows of K x 64 columns: 16 KB
constexpr int MAX_STAGES = 8;

enum { EPI_STORE = 0, EPI_SWIGLU = 1 };

struct SwapParams {
    bf16* out; int ldo;
    int M, N, K;
    int kc;                                 // rows of K per CTA of a cluster (a multiple of BK)
    int stages;
    int epi;
    int* fault;
};

// first operand MN-major (bit 15), second K-major, an m x n tile (see instr_desc in tc_common.cuh)
__host__ __device__ constexpr unsigned instr_desc_swapped(int m, int n) {
    return (1u << 4) | (1u << 7) | (1u << 10) | (1u << 15) | (0u << 16) | ((unsigned)(n >> 3) << 17) |
           ((unsigned)(m >> 4) << 24);
}

template <int NB>                           // rows of x, padded: 16, 32 or 64
__global__ void __launch_bounds__(NTH, 1)
gemm_swap_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x, const SwapParams p) {
    namespace cg = cooperative_groups;
    constexpr int X_BYTES = NB * BK * 2;                     // NB rows of 128 bytes
    constexpr int STAGE_BYTES = W_BYTES + (X_BYTES < 1024 ? 1024 : X_BYTES);
    constexpr unsigned TMEM_COLS = NB < 32 ? 32 : NB;
    constexpr unsigned IDESC = instr_desc_swapped(BN, NB);

    extern __shared__ unsigned char smem_raw[];
    unsigned char* tiles = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    float* red = reinterpret_cast<float*>(tiles);            // after the loop: [NB][BN] partial sums, row-major by x row
    __shared__ unsigned long long full_w[MAX_STAGES], full_x[MAX_STAGES], empty[MAX_STAGES], acc_full;
    __shared__ unsigned tmem_base_slot;
    __shared__ int abort_flag;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    cg::cluster_group cluster = cg::this_cluster();
    const unsigned rank = cluster.block_rank(), ksplit = cluster.num_blocks();
    const int n0 = blockIdx.x * BN;
    const int k_begin = (int)rank * p.kc;
    const int k_end = min(p.K, k_begin + p.kc);
    const int nkt = k_end > k_begin ? (k_end - k_begin + BK - 1) / BK : 0;
    const int STAGES = p.stages;

    pdl_launch_dependents();
    if (threadIdx.x == 0) {
        for (int s = 0; s < MAX_STAGES; ++s) { mbar_init(&full_w[s], 1); mbar_init(&full_x[s], 1); mbar_init(&empty[s], 1); }
        mbar_init(&acc_full, 1);
        abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
        prefetch_map(&map_w);
        prefetch_map(&map_x);
    }
    if (warp == 1) tmem_alloc(&tmem_base_slot, TMEM_COLS);
    fence_before();
    __syncthreads();
    fence_after();
    const unsigned tmem_base = tmem_base_slot;
    volatile int* abort = &abort_flag;

    if (warp == 0) {
        if (lane == 0) {
            // weights of the first stages at once; x only after the kernel before this one is done
            const int first = nkt < STAGES ? nkt : STAGES;
            for (int it = 0; it < first; ++it) {
                unsigned char* st = tiles + it * STAGE_BYTES;
                mbar_arrive_expect_tx(&full_w[it], W_BYTES);
                tma_load_2d(st, &map_w, n0, k_begin + it * BK, &full_w[it]);
                tma_load_2d(st + W_BYTES / 2, &map_w, n0 + 64, k_begin + it * BK, &full_w[it]);
            }
            pdl_wait();
            for (int it = 0; it < nkt && !*abort; ++it) {
                const int s = it % STAGES;
                unsigned char* st = tiles + s * STAGE_BYTES;
                if (it >= STAGES) {
                    if (!mbar_wait(&empty[s], ((it / STAGES) - 1) & 1, abort, p.fault, 8)) break;
                    mbar_arrive_expect_tx(&full_w[s], W_BYTES);
                    tma_load_2d(st, &map_w, n0, k_begin + it * BK, &full_w[s]);
                    tma_load_2d(st + W_BYTES / 2, &map_w, n0 + 64, k_begin + it * BK, &full_w[s]);
                }
                mbar_arrive_expect_tx(&full_x[s], X_BYTES);
                tma_load_2d(st + W_BYTES, &map_x, k_begin + it * BK, 0, &full_x[s]);
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            bool ok = true;
            for (int it = 0; it < nkt; ++it) {
                const int s = it % STAGES;
                if (!mbar_wait(&full_w[s], (it / STAGES) & 1, abort, p.fault, 8) ||
                    !mbar_wait(&full_x[s], (it / STAGES) & 1, abort, p.fault, 8)) { ok = false; break; }
                fence_after();
                const unsigned w = smem_u32(tiles + s * STAGE_BYTES), x = w + W_BYTES;
#pragma unroll
                for (int kk = 0; kk < BK / 16; ++kk) {
                    // W^T: 16 rows of K further = two groups of eight 128-byte rows; the second 64 columns lie one
                    // box (8 KB) further.  x: 16 elements of K further = 32 bytes inside the swizzled 128-byte row.
                    const unsigned long long da = smem_desc(w + kk * 2048, W_BYTES / 2, 1024);
                    const unsigned long long db = smem_desc(x + kk * 32, 16, 1024);
                    umma(tmem_base, da, db, IDESC, (it | kk) != 0);
                }
                umma_commit(&empty[s]);                   // the stage is free when these products have read it
            }
            if (ok) umma_commit(&acc_full);
            else *abort = 1;
        }
    } else {
        const int quarter = warp & 3;                     // the 32 lanes of tensor memory this warp may read
        const int col = quarter * 32 + lane;              // column of the strip = lane of tensor memory
        if (nkt > 0) {
            if (mbar_wait(&acc_full, 0, abort, p.fault, 8)) {
                fence_after();
                const unsigned taddr = tmem_base + ((unsigned)(quarter * 32) << 16);
#pragma unroll
                for (int c = 0; c < (NB + 31) / 32; ++c) {
                    float v[32];
                    tmem_ld32(taddr + c * 32, v);
#pragma unroll
                    for (int r = 0; r < 32; ++r)
                        if (c * 32 + r < NB) red[(c * 32 + r) * BN + col] = v[r];
                }
            }
        } else {
            for (int r = 0; r < NB; ++r) red[r * BN + col] = 0.f;
        }
        fence_before();
    }
    // (the staging memory is free: every product has read it before acc_full, and `red` overlays only it)
    cluster.sync();

    if (warp >= 2 && !*abort) {
        // rank r adds up rows r, r + ksplit, ... of x over all CTAs of the cluster: four columns a thread
        // (16-byte loads from the other CTAs' shared memory), four rows at a time
        const int t = (warp - 2) * 32 + lane;
        const int c4 = t & 31, j0 = t >> 5;
        const int mine = p.M > (int)rank ? (p.M - (int)rank + (int)ksplit - 1) / (int)ksplit : 0;
        if (p.epi == EPI_STORE) {
            for (int j = j0; j < mine; j += 4) {
                const int row = (int)rank + j * (int)ksplit;
                float4 sum = make_float4(0.f, 0.f, 0.f, 0.f);
                for (unsigned r = 0; r < ksplit; ++r) {
                    const float4 v = *reinterpret_cast<const float4*>(cluster.map_shared_rank(red, r) + row * BN + c4 * 4);
                    sum.x += v.x; sum.y += v.y; sum.z += v.z; sum.w += v.w;
                }
                const int n = n0 + c4 * 4;
                bf16* o = p.out + (size_t)row * p.ldo + n;
                if (n + 3 < p.N && (reinterpret_cast<uintptr_t>(o) & 7) == 0) {
                    const __nv_bfloat162 lo = __floats2bfloat162_rn(sum.x, sum.y), hi = __floats2bfloat162_rn(sum.z, sum.w);
                    uint2 raw;
                    raw.x = *reinterpret_cast<const unsigned*>(&lo);
                    raw.y = *reinterpret_cast<const unsigned*>(&hi);
                    *reinterpret_cast<uint2*>(o) = raw;
                } else {
                    const float s4[4] = {sum.x, sum.y, sum.z, sum.w};
                    for (int e = 0; e < 4; ++e)
                        if (n + e < p.N) o[e] = __float2bfloat16_rn(s4[e]);
                }
            }
        } else if ((c4 & 8) == 0) {
            // the strip is [32 gate | 32 up | 32 gate | 32 up]: a thread of a gate block adds up its four gates and
            // the four ups 32 columns further, and writes four gated values
            for (int j = j0; j < mine; j += 4) {
                const int row = (int)rank + j * (int)ksplit;
                float4 g = make_float4(0.f, 0.f, 0.f, 0.f), u = g;
                for (unsigned r = 0; r < ksplit; ++r) {
                    const float* src = cluster.map_shared_rank(red, r) + row * BN + c4 * 4;
                    const float4 a = *reinterpret_cast<const float4*>(src), b2 = *reinterpret_cast<const float4*>(src + 32);
                    g.x += a.x; g.y += a.y; g.z += a.z; g.w += a.w;
                    u.x += b2.x; u.y += b2.y; u.z += b2.z; u.w += b2.w;
                }
                if (n0 + c4 * 4 < p.N) {
                    const int oc = (n0 >> 1) + (c4 >> 4) * 32 + (c4 & 7) * 4;
                    bf16* o = p.out + (size_t)row * p.ldo + oc;
                    o[0] = __float2bfloat16_rn(g.x / (1.f + expf(-g.x)) * u.x);
                    o[1] = __float2bfloat16_rn(g.y / (1.f + expf(-g.y)) * u.y);
                    o[2] = __float2bfloat16_rn(g.z / (1.f + expf(-g.z)) * u.z);
                    o[3] = __float2bfloat16_rn(g.w / (1.f + expf(-g.w)) * u.w);
                }
            }
        }
    }
    cluster.sync();                     // nobody leaves while its shared memory may still be read
    if (warp == 1) {
        fence_after();
        tmem_free(tmem_base, TMEM_COLS);
    }
}

template <int NB>
int launch_swap(const CUtensorMap& mw, const CUtensorMap& mx, SwapParams p, int ksplit, cudaStream_t stream) {
    constexpr int X_BYTES = NB * BK * 2;
    constexpr int STAGE_BYTES = W_BYTES + (X_BYTES < 1024 ? 1024 : X_BYTES);
    const int tiles = p.kc / BK;
    int stages = tiles < MAX_STAGES ? tiles : MAX_STAGES;
    while (stages > 2 && (size_t)stages * STAGE_BYTES > 96 * 1024) --stages;     // two CTAs to an SM
    p.stages = stages;
    size_t smem = (size_t)stages * STAGE_BYTES;
    const size_t redb = (size_t)NB * BN * sizeof(float);
    if (smem < redb) smem = redb;
    smem += 1024;
    static bool configured = false;
    auto kernel = gemm_swap_kernel<NB>;
    if (!configured) {
        if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 128 * 1024) != cudaSuccess)
            return tis_check_launch("gemm_swap (shared memory)");
        configured = true;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((p.N + BN - 1) / BN, ksplit, 1);
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
    const cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, mw, mx, p);
    if (e != cudaSuccess) {
        tis_set_error("gemm_swap: %s", cudaGetErrorString(e));
        return TIS_CUDA_ERROR;
    }
    return tis_check_launch("gemm_swap");
}

}  // namespace

// x (M <= 64 rows x K, row stride ldx), w (K x N, row stride ldw), out (M x N, or M x N/2 for the SwiGLU epilogue of
// [32 gate | 32 up] column blocks; row stride ldo): bfloat16.  ksplit: CTAs per strip of 128 columns (1, 2, 4 or 8).
// Refuses what the TMA engine cannot address: K, N and the strides must be multiples of 8 elements and the pointers
// 16-byte aligned.
TIS_API int tis_gemm_swap(const void* x, int ldx, const void* w, int ldw, void* out, int ldo, int M, int N, int K,
                          int ksplit, int epi, int* fault, cudaStream_t stream) {
    if (M <= 0 || N <= 0 || K <= 0) return TIS_OK;
    if (M > 64) {
        tis_set_error("gemm_swap: %d rows; this kernel takes at most 64", M);
        return TIS_BAD_SIZE;
    }
    if ((K % 8) || (N % 8) || (ldx % 8) || (ldw % 8) ||
        (reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(w)) % 16) {
        tis_set_error("gemm_swap: N %d, K %d and the row strides %d, %d must be multiples of 8 and the pointers "
                      "16-byte aligned", N, K, ldx, ldw);
        return TIS_BAD_SIZE;
    }
    if (!(ksplit == 1 || ksplit == 2 || ksplit == 4 || ksplit == 8)) {
        tis_set_error("gemm_swap: ksplit %d must be 1, 2, 4 or 8", ksplit);
        return TIS_BAD_SIZE;
    }
    if (epi != EPI_STORE && epi != EPI_SWIGLU) {
        tis_set_error("gemm_swap: unknown epilogue %d", epi);
        return TIS_BAD_SIZE;
    }
    if (epi == EPI_SWIGLU && N % 64) {
        tis_set_error("gemm_swap: the SwiGLU epilogue needs N %d to be a multiple of 64", N);
        return TIS_BAD_SIZE;
    }
    const int nb = M <= 16 ? 16 : (M <= 32 ? 32 : 64);
    CUtensorMap mw, mx;
    if (!tensor_map(w, N, K, ldw, BK, true, &mw) || !tensor_map(x, K, M, ldx, nb, true, &mx)) return TIS_CUDA_ERROR;
    SwapParams p;
    p.out = (bf16*)out; p.ldo = ldo; p.M = M; p.N = N; p.K = K; p.epi = epi; p.fault = fault; p.stages = 0;
    p.kc = ((K + ksplit - 1) / ksplit + BK - 1) / BK * BK;
    if (nb == 16) return launch_swap<16>(mw, mx, p, ksplit, stream);
    if (nb == 32) return launch_swap<32>(mw, mx, p, ksplit, stream);
    return launch_swap<64>(mw, mx, p, ksplit, stream);
}
