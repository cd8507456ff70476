// Matrix products with up to 64 rows on the fifth-generation tensor cores, operands swapped:
// y (M x N) = x (M x K) . W (K x N), bfloat16 — computed as y^T = W^T . x^T, so that the 128 rows of a
// tcgen05.mma tile are 128 *columns of W* and its narrow side (16, 32 or 64) holds the rows of x.  The
// tensor cores then do no work on padding, the accumulator is 128 lanes x M columns of tensor memory,
// and W — the only operand of any size, streamed from HBM once — goes from the TMA engine to the tensor
// cores without passing through a thread: no ldmatrix, no mma.sync, no issue slots spent on it.
//
// A CTA owns a strip of 128 columns of W and one share of K; the CTAs that share a strip are a
// thread-block cluster and add their partial sums through distributed shared memory, pushed to the CTA
// that owns a row of x (as gemm_skinny.cu; see cluster_reduce.cuh for why pushed).
// Roles, specialised by warp:
//   warp 0   one lane orders W (two 64 x 64 boxes a step of 64 of K, 128-byte swizzle: W^T as the MN-major
//            first operand, used as it lies) into a ring of stages — before the dependency wait, weights
//            depend on nothing — and then the matching boxes of x (64 of K x M rows: the K-major second
//            operand) after it;
//   warp 1   owns the tensor memory; one lane issues four tcgen05.mma (k16) per stage and hands the
//            stage back with tcgen05.commit;
//   warps 2-5 read the accumulator (tcgen05.ld: a thread holds the M values of its column), send each row's
//            partial sums to the rank that owns the row (st.async counted on its mbarrier), and add up
//            and store the rows this CTA owns (plain store, SwiGLU gating of [32 gate | 32 up] column
//            blocks, or the residual epilogue; the norm's factor per row as in gemm_skinny.cu).
// Every wait on an mbarrier is bounded; one that runs out sets the fault word, every role leaves its
// loop, and the tensor memory is freed.
#include "tc_common.cuh"
#include "cluster_reduce.cuh"
#include <cooperative_groups.h>

namespace {

using namespace tc;
using cluster_reduce::EPI_STORE;
using cluster_reduce::EPI_SWIGLU;
using cluster_reduce::EPI_RESIDUAL;

constexpr int BN = 128;                     // columns of W a CTA owns (the M of the tcgen05 tile)
constexpr int BK = 64;                      // 64 bfloat16 = one 128-byte swizzle row
constexpr int NTH = 192;
constexpr int W_BYTES = 2 * 64 * BK * 2;    // two boxes of 64 rows of K x 64 columns: 16 KB
constexpr int MAX_STAGES = 8;

struct SwapParams {
    int K;
    int kc;                                 // rows of K per CTA of a cluster (a multiple of BK)
    int stages;
    cluster_reduce::Epilogue e;             // rows, columns, where the result goes, the fault word
};

// rows of x a rank owns at most, and the floats it receives: [source rank][owned row][128 columns]
__host__ __device__ inline int swap_rows_per_rank(int nb, int ksplit) { return (nb + ksplit - 1) / ksplit; }

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
    __shared__ unsigned long long full_w[MAX_STAGES], full_x[MAX_STAGES], empty[MAX_STAGES], acc_full, recv_bar;
    __shared__ unsigned tmem_base_slot;
    __shared__ int abort_flag;
    __shared__ float row_factor[NB];

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    cg::cluster_group cluster = cg::this_cluster();
    const unsigned rank = cluster.block_rank(), ksplit = cluster.num_blocks();
    const int n0 = blockIdx.x * BN;
    const int k_begin = (int)rank * p.kc;
    const int k_end = min(p.K, k_begin + p.kc);
    const int nkt = k_end > k_begin ? (k_end - k_begin + BK - 1) / BK : 0;
    const int STAGES = p.stages;
    const int rpr = swap_rows_per_rank(NB, (int)ksplit);
    // the staging area also holds the accumulator on its way out ([NB][BN] floats); behind it what the cluster pushes
    const size_t stage_area = (size_t)STAGES * STAGE_BYTES > (size_t)NB * BN * 4 ? (size_t)STAGES * STAGE_BYTES : (size_t)NB * BN * 4;
    float* recv = reinterpret_cast<float*>(tiles + stage_area);                      // [ksplit][rpr][BN] pushed partial sums
    const int mine = p.e.M > (int)rank ? (p.e.M - (int)rank + (int)ksplit - 1) / (int)ksplit : 0;   // rows this rank owns

    pdl_launch_dependents();
    if (threadIdx.x == 0) {
        for (int s = 0; s < MAX_STAGES; ++s) { mbar_init(&full_w[s], 1); mbar_init(&full_x[s], 1); mbar_init(&empty[s], 1); }
        mbar_init(&acc_full, 1);
        mbar_init(&recv_bar, 1);
        abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
        mbar_arrive_expect_tx(&recv_bar, (unsigned)(mine * BN * 4) * ksplit);     // every rank sends each owned row
        prefetch_map(&map_w);
        prefetch_map(&map_x);
    }
    if (warp == 1) tmem_alloc(&tmem_base_slot, TMEM_COLS);
    fence_before();
    __syncthreads();
    fence_after();
    cluster_reduce::cluster_arrive();        // waited for before the first push: by then every CTA's barrier is ready
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
                    if (!mbar_wait(&empty[s], ((it / STAGES) - 1) & 1, abort, p.e.fault, 8)) break;
                    mbar_arrive_expect_tx(&full_w[s], W_BYTES);
                    tma_load_2d(st, &map_w, n0, k_begin + it * BK, &full_w[s]);
                    tma_load_2d(st + W_BYTES / 2, &map_w, n0 + 64, k_begin + it * BK, &full_w[s]);
                }
                mbar_arrive_expect_tx(&full_x[s], X_BYTES);
                tma_load_2d(st + W_BYTES, &map_x, k_begin + it * BK, 0, &full_x[s]);
            }
        }
        __syncwarp();
        cluster_reduce::cluster_wait();
    } else if (warp == 1) {
        if (lane == 0) {
            bool ok = true;
            for (int it = 0; it < nkt; ++it) {
                const int s = it % STAGES;
                if (!mbar_wait(&full_w[s], (it / STAGES) & 1, abort, p.e.fault, 8) ||
                    !mbar_wait(&full_x[s], (it / STAGES) & 1, abort, p.e.fault, 8)) { ok = false; break; }
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
        __syncwarp();
        cluster_reduce::cluster_wait();
    } else {
        const int quarter = warp & 3;                     // the 32 lanes of tensor memory this warp may read
        const int col = quarter * 32 + lane;              // column of the strip = lane of tensor memory
        const int t = (warp - 2) * 32 + lane;
        // the norm's factor of each row, from the partial sums the kernel before left
        pdl_wait();
        if (p.e.in_ss != nullptr) {
            for (int r = warp - 2; r < p.e.M; r += 4) {
                float sq = 0.f;
                for (int i = lane; i < p.e.in_parts; i += 32) sq += p.e.in_ss[(size_t)r * p.e.in_parts + i];
                sq = warp_sum(sq);
                if (lane == 0) row_factor[r] = p.e.in_factor.of(sq);
            }
        }
        cluster_reduce::cluster_wait();
        // push: every row's partial sums of this CTA to the rank that owns the row
        const unsigned recv_base = cluster_reduce::shared_addr(recv), bar_base = cluster_reduce::shared_addr(&recv_bar);
        const bool have = nkt > 0 && mbar_wait(&acc_full, 0, abort, p.e.fault, 8);
        if (have) fence_after();
        const unsigned taddr = tmem_base + ((unsigned)(quarter * 32) << 16);
        // the accumulator goes through the staging memory (free now: every product has read it), so that a thread
        // can send four columns of a row at once
        float* red = reinterpret_cast<float*>(tiles);            // [NB][BN], row-major by x row
#pragma unroll
        for (int c = 0; c < (NB + 31) / 32; ++c) {
            float v[32];
            if (have) tmem_ld32(taddr + c * 32, v);
#pragma unroll
            for (int r = 0; r < 32; ++r)
                if (c * 32 + r < NB) red[(c * 32 + r) * BN + col] = have ? v[r] : 0.f;
        }
        fence_before();
        asm volatile("bar.sync 2, 128;\n" ::: "memory");          // red and row_factor are written (the four epilogue warps)
        for (int i = t; i < p.e.M * (BN / 4); i += 128) {
            const int row = i / (BN / 4), q = i - row * (BN / 4);
            const unsigned owner = (unsigned)row % ksplit;
            const unsigned at = recv_base + (unsigned)((((int)rank * rpr + row / (int)ksplit) * BN + q * 4) * 4);
            const float4 v = *reinterpret_cast<const float4*>(red + row * BN + q * 4);
            asm volatile("st.async.shared::cluster.mbarrier::complete_tx::bytes.v4.f32 [%0], {%1, %2, %3, %4}, [%5];\n"
                         ::"r"(cluster_reduce::map_to_rank(at, owner)), "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w),
                           "r"(cluster_reduce::map_to_rank(bar_base, owner)) : "memory");
        }
        // wait for the partials of all ranks (bounded; a wait that runs out is flagged and the result not to be used)
        {
            unsigned done = 0;
            for (int spin = 0; spin < (1 << 22) && !done; ++spin)
                asm volatile("{\n.reg .pred p;\nmbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n"
                             "selp.u32 %0, 1, 0, p;\n}\n" : "=r"(done) : "r"(bar_base), "r"(0u) : "memory");
            if (!done && p.e.fault != nullptr) atomicExch(p.e.fault, 8);
        }
        // this rank adds up the rows it owns from its own shared memory: four columns a thread, four rows at a time
        const int c4 = t & 31, j0 = t >> 5;
        const bool scaled = p.e.in_ss != nullptr;
        const int n = n0 + c4 * 4;
        if (p.e.epi == EPI_STORE || p.e.epi == EPI_RESIDUAL) {
            float4 nw = make_float4(0.f, 0.f, 0.f, 0.f);
            if (p.e.epi == EPI_RESIDUAL && n < p.e.N) nw = *reinterpret_cast<const float4*>(p.e.norm_w + n);
            for (int j = j0; j < mine; j += 4) {
                const int row = (int)rank + j * (int)ksplit;
                float4 sum = make_float4(0.f, 0.f, 0.f, 0.f);
                for (unsigned r = 0; r < ksplit; ++r) {
                    const float4 v = *reinterpret_cast<const float4*>(recv + ((int)r * rpr + j) * BN + c4 * 4);
                    sum.x += v.x; sum.y += v.y; sum.z += v.z; sum.w += v.w;
                }
                if (scaled) { const float f = row_factor[row]; sum.x *= f; sum.y *= f; sum.z *= f; sum.w *= f; }
                bf16* o = p.e.out + (size_t)row * p.e.ldo + n;
                if (p.e.epi == EPI_RESIDUAL) {
                    // the stream += the product; out = the stream times the next norm's weight; sums of squares
                    // of the new stream by strip of 64 columns (16 threads a strip)
                    float sq = 0.f;
                    if (n < p.e.N) {                                  // N is a multiple of 8: n + 3 is inside too
                        float4* at = reinterpret_cast<float4*>(p.e.res + (size_t)row * p.e.ldr + n);
                        float4 v = *at;
                        v.x += sum.x; v.y += sum.y; v.z += sum.z; v.w += sum.w;
                        *at = v;
                        sq = v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
                        sum = make_float4(v.x * nw.x, v.y * nw.y, v.z * nw.z, v.w * nw.w);
                    }
#pragma unroll
                    for (int off = 8; off > 0; off >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, off);
                    const int strip = (n0 >> 6) + (c4 >> 4);
                    if ((c4 & 15) == 0 && strip * 64 < p.e.N) p.e.out_ss[(size_t)row * ((p.e.N + 63) / 64) + strip] = sq;
                }
                if (n + 3 < p.e.N && (reinterpret_cast<uintptr_t>(o) & 7) == 0) {
                    const __nv_bfloat162 lo = __floats2bfloat162_rn(sum.x, sum.y), hi = __floats2bfloat162_rn(sum.z, sum.w);
                    uint2 raw;
                    raw.x = *reinterpret_cast<const unsigned*>(&lo);
                    raw.y = *reinterpret_cast<const unsigned*>(&hi);
                    *reinterpret_cast<uint2*>(o) = raw;
                } else {
                    const float s4[4] = {sum.x, sum.y, sum.z, sum.w};
                    for (int e = 0; e < 4; ++e)
                        if (n + e < p.e.N) o[e] = __float2bfloat16_rn(s4[e]);
                }
            }
        } else if ((c4 & 8) == 0) {
            // the strip is [32 gate | 32 up | 32 gate | 32 up]: a thread of a gate block adds up its four gates and
            // the four ups 32 columns further, and writes four gated values
            for (int j = j0; j < mine; j += 4) {
                const int row = (int)rank + j * (int)ksplit;
                float4 g = make_float4(0.f, 0.f, 0.f, 0.f), u = g;
                for (unsigned r = 0; r < ksplit; ++r) {
                    const float* src = recv + ((int)r * rpr + j) * BN + c4 * 4;
                    const float4 a = *reinterpret_cast<const float4*>(src), b2 = *reinterpret_cast<const float4*>(src + 32);
                    g.x += a.x; g.y += a.y; g.z += a.z; g.w += a.w;
                    u.x += b2.x; u.y += b2.y; u.z += b2.z; u.w += b2.w;
                }
                if (scaled) {
                    const float f = row_factor[row];
                    g.x *= f; g.y *= f; g.z *= f; g.w *= f; u.x *= f; u.y *= f; u.z *= f; u.w *= f;
                }
                if (n < p.e.N) {
                    const int oc = (n0 >> 1) + (c4 >> 4) * 32 + (c4 & 7) * 4;
                    bf16* o = p.e.out + (size_t)row * p.e.ldo + oc;
                    o[0] = __float2bfloat16_rn(g.x / (1.f + expf(-g.x)) * u.x);
                    o[1] = __float2bfloat16_rn(g.y / (1.f + expf(-g.y)) * u.y);
                    o[2] = __float2bfloat16_rn(g.z / (1.f + expf(-g.z)) * u.z);
                    o[3] = __float2bfloat16_rn(g.w / (1.f + expf(-g.w)) * u.w);
                }
            }
        }
    }
    __syncthreads();                    // every read of the tensor memory is done
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
    const size_t recvb = (size_t)ksplit * swap_rows_per_rank(NB, ksplit) * BN * sizeof(float);
    while (stages > 2 && (size_t)stages * STAGE_BYTES + recvb > 108 * 1024) --stages;     // two CTAs to an SM
    p.stages = stages;
    const size_t redb = (size_t)NB * BN * sizeof(float);
    const size_t stage_area = (size_t)stages * STAGE_BYTES > redb ? (size_t)stages * STAGE_BYTES : redb;
    const size_t smem = stage_area + recvb + 1024;
    static bool configured = false;
    auto kernel = gemm_swap_kernel<NB>;
    if (!configured) {
        if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024) != cudaSuccess)
            return tis_check_launch("gemm_swap (shared memory)");
        configured = true;
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((p.e.N + BN - 1) / BN, ksplit, 1);
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
// 16-byte aligned.  in_ss .. out_ss: as in tis_gemm_skinny_fused (epi 2 = the residual epilogue).
TIS_API int tis_gemm_swap_fused(const void* x, int ldx, const void* w, int ldw, void* out, int ldo, int M, int N, int K,
                                int ksplit, int epi, const float* in_ss, int in_parts, float in_eps, int in_width, int in_kind,
                                float* res, int ldr, const float* norm_w, float* out_ss, int* fault, cudaStream_t stream) {
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
    if (epi < EPI_STORE || epi > EPI_RESIDUAL) {
        tis_set_error("gemm_swap: unknown epilogue %d", epi);
        return TIS_BAD_SIZE;
    }
    if (epi == EPI_SWIGLU && N % 64) {
        tis_set_error("gemm_swap: the SwiGLU epilogue needs N %d to be a multiple of 64", N);
        return TIS_BAD_SIZE;
    }
    if (epi == EPI_RESIDUAL && (res == nullptr || norm_w == nullptr || out_ss == nullptr || ldr % 4 ||
                                (reinterpret_cast<uintptr_t>(res) | reinterpret_cast<uintptr_t>(norm_w)) % 16)) {
        tis_set_error("gemm_swap: the residual epilogue needs the stream, the norm's weight and room for the partial "
                      "sums, a row stride (%d) that is a multiple of 4 and 16-byte aligned pointers", ldr);
        return TIS_BAD_SIZE;
    }
    if (in_ss != nullptr && (in_parts <= 0 || in_width <= 0 || in_kind < TIS_NORM_L2_EPS || in_kind > TIS_NORM_MEAN_EPS)) {
        tis_set_error("gemm_swap: %d partial sums a row over a width of %d, norm kind %d", in_parts, in_width, in_kind);
        return TIS_BAD_SIZE;
    }
    const int nb = M <= 16 ? 16 : (M <= 32 ? 32 : 64);
    CUtensorMap mw, mx;
    if (!tensor_map(w, N, K, ldw, BK, true, &mw) || !tensor_map(x, K, M, ldx, nb, true, &mx)) return TIS_CUDA_ERROR;
    SwapParams p;
    p.K = K; p.stages = 0;
    p.e.out = (bf16*)out; p.e.ldo = ldo; p.e.M = M; p.e.N = N; p.e.epi = epi; p.e.fault = fault;
    p.e.in_ss = in_ss; p.e.in_parts = in_parts; p.e.in_factor = norm_factor(in_kind, in_width, in_eps);
    p.e.res = res; p.e.ldr = ldr; p.e.norm_w = norm_w; p.e.out_ss = out_ss;
    p.kc = ((K + ksplit - 1) / ksplit + BK - 1) / BK * BK;
    if (nb == 16) return launch_swap<16>(mw, mx, p, ksplit, stream);
    if (nb == 32) return launch_swap<32>(mw, mx, p, ksplit, stream);
    return launch_swap<64>(mw, mx, p, ksplit, stream);
}

TIS_API int tis_gemm_swap(const void* x, int ldx, const void* w, int ldw, void* out, int ldo, int M, int N, int K,
                          int ksplit, int epi, int* fault, cudaStream_t stream) {
    if (epi == EPI_RESIDUAL) {
        tis_set_error("gemm_swap: the residual epilogue goes through tis_gemm_swap_fused");
        return TIS_BAD_SIZE;
    }
    return tis_gemm_swap_fused(x, ldx, w, ldw, out, ldo, M, N, K, ksplit, epi, nullptr, 0, 0.f, 0, 0, nullptr, 0, nullptr,
                               nullptr, fault, stream);
}
