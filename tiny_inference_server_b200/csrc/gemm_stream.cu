// Matrix products with few rows, fed by the TMA engine: y (M x N) = x (M x K) . W (K x N), bfloat16,
// M <= 64 — the projections of a decode step, bound by streaming W from HBM once.
//
// Work is cut as in gemm_skinny.cu: a CTA owns a strip of 64 columns of W and one share of K; the
// CTAs that share a strip are a thread-block cluster and add their partial sums through distributed
// shared memory.  What differs is how W comes: the whole share of a CTA (up to 512 rows of K, 64 KB)
// is ordered at once by one thread as 64 x 64 boxes of a tensor map (cp.async.bulk.tensor.2d, 128-byte
// swizzle, zeros beyond N and K), each box counted on an mbarrier of its own — and it is ordered
// by a warp that never waits for the kernel before this one (griddepcontrol.wait), because weights
// depend on nothing.  So all bytes of the product are in flight from the start, the four consumer warps
// spend no issue slots on copies, and the loop has no CTA-wide barrier: a warp waits for a box and
// multiplies (mma.sync m16n8k16, x from shared memory by ldmatrix, W by ldmatrix.trans through the swizzle).
// Shares of more than 512 rows of K are walked in rounds of eight boxes.
// Every wait on an mbarrier is bounded; one that runs out sets the fault word.
// The epilogues are those of gemm_skinny.cu, the residual epilogue and the norm's factor per row among them.
#include "tc_common.cuh"
#include "cluster_reduce.cuh"
#include "timeline.cuh"
#include <cooperative_groups.h>

namespace {

using namespace tc;
using cluster_reduce::EPI_STORE;
using cluster_reduce::EPI_SWIGLU;
using cluster_reduce::EPI_RESIDUAL;

constexpr int BN = 64;            // columns of a strip
constexpr int BK = 64;            // rows of K per box
constexpr int NTH = 128;
constexpr int BOX_ELEMS = BK * BN;
constexpr int BOX_BYTES = BOX_ELEMS * 2;
constexpr int MAX_BOXES = 8;      // boxes a CTA keeps in shared memory (a round)

struct StreamParams {
    const bf16* x; int ldx;
    int K;
    int kc;                       // rows of K per CTA of a cluster (a multiple of BK)
    int boxes;                    // boxes in shared memory: min(kc / BK, MAX_BOXES)
    cluster_reduce::Epilogue e;   // rows, columns, where the result goes, the fault word
    TIS_TIMELINE_MEMBER           // (instrumented builds only; stamps as in gemm_skinny.cu: 3 = first box landed)
};

__device__ __forceinline__ void cp16(void* smem, const void* gmem, int bytes) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(smem_u32(smem)), "l"(gmem), "r"(bytes));
}
__device__ __forceinline__ void ldsm_x4(unsigned (&r)[4], const void* smem) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_u32(smem)));
}
__device__ __forceinline__ void ldsm_x4_t(unsigned (&r)[4], unsigned addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void mma16816(float (&c)[4], const unsigned (&a)[4], unsigned b0, unsigned b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// A fifth warp does nothing but order weights (one lane orders the boxes); the four consumer warps never
// meet inside the loop.  (The same with the producer warp copying 16-byte chunks by cp.async instead was
// measured too: 9.1 us against 6.3 us for the down projection, one warp cannot issue them fast enough.)
template <int MT>
__global__ void __launch_bounds__(NTH + 32) gemm_stream_kernel(const __grid_constant__ CUtensorMap wmap, const StreamParams p) {
    namespace cg = cooperative_groups;
    extern __shared__ unsigned char smem_raw[];
    // boxes at 1024-byte boundaries: the swizzle is a function of the address
    unsigned char* base = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    __shared__ __align__(8) unsigned long long bars[MAX_BOXES], empty[MAX_BOXES];
    __shared__ int abort_flag;
    __shared__ float pair[2][BN];
    __shared__ float row_factor[MT * 16];
    __shared__ __align__(8) unsigned long long recv_bar;
    constexpr int BOX_SM = BOX_ELEMS;                                 // elements of a box in shared memory
    const int xrow = p.kc + 8;                                        // padded rows: 16 bytes apart modulo 128
    bf16* w_sm = reinterpret_cast<bf16*>(base);                       // boxes x [64 k][WROW]
    bf16* xs = w_sm + (size_t)p.boxes * BOX_SM;                       // [MT*16][xrow]: this CTA's share of K
    float* recv = reinterpret_cast<float*>(xs + (size_t)MT * 16 * xrow);   // partial sums pushed by the cluster

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const bool producer = warp == NTH / 32;
    cg::cluster_group cluster = cg::this_cluster();
    const unsigned rank = cluster.block_rank(), ksplit = cluster.num_blocks();
    const int n0 = blockIdx.x * BN;
    const int k_begin = (int)rank * p.kc;
    const int k_end = min(p.K, k_begin + p.kc);
    const int nkt = k_end > k_begin ? (k_end - k_begin + BK - 1) / BK : 0;

    TIS_STAMP(p, 0);
    asm volatile("griddepcontrol.launch_dependents;\n" ::);
    if (tid == 0) {
        abort_flag = 0;
        for (int b = 0; b < MAX_BOXES; ++b) { mbar_init(&bars[b], 1); mbar_init(&empty[b], NTH / 32); }
        cluster_reduce::init_barrier(&recv_bar, rank, ksplit, p.e.M);
    }
    __syncthreads();
    cluster_reduce::cluster_arrive();        // waited for after the loop: by then every CTA's barrier is ready

    constexpr int CHAINS = MT <= 2 ? BK / 16 : 2;          // independent chains of accumulators
    float acc[MT][2][4], accs[CHAINS - 1][MT][2][4];
#pragma unroll
    for (int m = 0; m < MT; ++m)
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            acc[m][j][0] = acc[m][j][1] = acc[m][j][2] = acc[m][j][3] = 0.f;
#pragma unroll
            for (int ch = 0; ch < CHAINS - 1; ++ch) accs[ch][m][j][0] = accs[ch][m][j][1] = accs[ch][m][j][2] = accs[ch][m][j][3] = 0.f;
        }

    cluster_reduce::RowFactorLoads<MT> factors;
    if (producer) {
        // weights depend on nothing: no wait for the kernel before.  Box `it` goes to slot it % boxes, once
        // every consumer warp is done with the box that was there a round earlier.
        bool alive = true;
        for (int it = 0; it < nkt; ++it) {
            const int b = it % p.boxes;
            if (it >= p.boxes) {
                if (alive) alive = mbar_wait(&empty[b], (unsigned)(((it / p.boxes) - 1) & 1), &abort_flag, p.e.fault, 7);
                asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
            }
            if (lane == 0) {
                mbar_arrive_expect_tx(&bars[b], BOX_BYTES);
                tma_load_2d(w_sm + (size_t)b * BOX_SM, &wmap, n0, k_begin + it * BK, &bars[b]);
            }
        }
    } else {
    // x is the output of the kernel before this one
    TIS_STAMP(p, 1);
    asm volatile("griddepcontrol.wait;\n" ::: "memory");
    TIS_STAMP(p, 2);
    {
        const int kw = nkt * BK;                   // columns of xs that the loop reads
        const int per_row = kw / 8;
        for (int i = tid; i < MT * 16 * per_row; i += NTH) {
            const int r = i / per_row, c = (i - r * per_row) * 8;
            const int k = k_begin + c;
            const bool ok = r < p.e.M && k < k_end;
            cp16(xs + (size_t)r * xrow + c, ok ? p.x + (size_t)r * p.ldx + k : p.x, ok ? 16 : 0);
        }
        asm volatile("cp.async.commit_group;\n" ::);
        // the norm's factor of each row, from the partial sums the kernel before left: the loads now, the rest after the loop
        factors.order(p.e, row_factor, tid);
        asm volatile("cp.async.wait_group 0;\n" ::: "memory");
    }
    asm volatile("bar.sync 1, 128;\n" ::: "memory");          // xs is visible to every consumer warp

    const unsigned w_base = smem_u32(w_sm);
    // ldmatrix.trans of the warp's 16 columns: lane -> (row inside the k16 block, 16-byte chunk of the box row)
    const int b_row = (((lane >> 3) & 1) << 3) + (lane & 7);
    const int b_chunk = warp * 2 + (lane >> 4);
    bool alive = true;
    for (int it = 0; it < nkt; ++it) {
        const int b = it % p.boxes;
        if (alive) alive = mbar_wait(&bars[b], (unsigned)((it / p.boxes) & 1), &abort_flag, p.e.fault, 6);
        if (!alive) continue;                      // a wait ran out: no more waits, the result is not to be used
        if (it == 0) TIS_STAMP(p, 3);
        const unsigned box = w_base + (unsigned)b * (BOX_SM * 2);
        // all fragments of the box first, then independent chains of accumulators (one per k16 step for up to
        // 32 rows, two otherwise): the latency of a step is not paid once per step
        unsigned bf[BK / 16][4];
#pragma unroll
        for (int kk = 0; kk < BK / 16; ++kk) {
            const int row = kk * 16 + b_row;
            ldsm_x4_t(bf[kk], box + row * 128 + ((b_chunk ^ (row & 7)) << 4));
        }
#pragma unroll
        for (int m = 0; m < MT; ++m) {
            unsigned a[BK / 16][4];
#pragma unroll
            for (int kk = 0; kk < BK / 16; ++kk)
                ldsm_x4(a[kk], xs + (size_t)(m * 16 + (((lane >> 3) & 1) << 3) + (lane & 7)) * xrow + it * BK + kk * 16 +
                                   ((lane >> 4) << 3));
#pragma unroll
            for (int kk = 0; kk < BK / 16; ++kk) {
                const int ch = kk % CHAINS;
                if (ch == 0) {
                    mma16816(acc[m][0], a[kk], bf[kk][0], bf[kk][1]);
                    mma16816(acc[m][1], a[kk], bf[kk][2], bf[kk][3]);
                } else {
                    mma16816(accs[ch - 1][m][0], a[kk], bf[kk][0], bf[kk][1]);
                    mma16816(accs[ch - 1][m][1], a[kk], bf[kk][2], bf[kk][3]);
                }
            }
        }
        if (nkt > p.boxes) {                       // the slot is taken again a round later
            __syncwarp();
            if (lane == 0) mbar_arrive(&empty[b]);
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
    factors.finish(p.e, row_factor, tid);
    asm volatile("bar.sync 1, 128;\n" ::: "memory");          // row_factor is written
    }   // consumers
    cluster_reduce::cluster_wait();         // every CTA of the cluster has initialised its barrier
    TIS_STAMP(p, 5);
    if (!producer)
        cluster_reduce::push_reduce_store<MT>(acc, p.e, recv, &recv_bar, pair, row_factor, rank, ksplit, blockIdx.x,
                                              gridDim.x, tid);
    TIS_STAMP(p, 6);
}

}  // namespace

// x (M x K, row stride ldx), w (K x N, row stride ldw), out (M x N, or M x N/2 for the SwiGLU epilogue of
// [32 gate | 32 up] column blocks; row stride ldo): bfloat16.  ksplit: CTAs per strip (1, 2, 4 or 8).
// Refuses what the TMA engine cannot address: K, N and the strides must be multiples of 8 elements and
// the pointers 16-byte aligned.  in_ss .. out_ss: as in tis_gemm_skinny_fused.
TIS_API int tis_gemm_stream_fused(const void* x, int ldx, const void* w, int ldw, void* out, int ldo, int M, int N, int K,
                                  int ksplit, int epi, const float* in_ss, int in_parts, float in_eps, int in_width, int in_kind,
                                  float* res, int ldr, const float* norm_w, float* out_ss, int* fault,
                                  cudaStream_t stream) {
    if (M <= 0 || N <= 0 || K <= 0) return TIS_OK;
    if (M > 64) {
        tis_set_error("gemm_stream: %d rows; this kernel takes at most 64", M);
        return TIS_BAD_SIZE;
    }
    if ((K % 8) || (N % 8) || (ldx % 8) || (ldw % 8) ||
        (reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(w)) % 16) {
        tis_set_error("gemm_stream: N %d, K %d and the row strides %d, %d must be multiples of 8 and the pointers "
                      "16-byte aligned", N, K, ldx, ldw);
        return TIS_BAD_SIZE;
    }
    if (!(ksplit == 1 || ksplit == 2 || ksplit == 4 || ksplit == 8)) {
        tis_set_error("gemm_stream: ksplit %d must be 1, 2, 4 or 8", ksplit);
        return TIS_BAD_SIZE;
    }
    if (epi < EPI_STORE || epi > EPI_RESIDUAL) {
        tis_set_error("gemm_stream: unknown epilogue %d", epi);
        return TIS_BAD_SIZE;
    }
    if (epi == EPI_RESIDUAL && (res == nullptr || norm_w == nullptr || out_ss == nullptr || ldr % 2 || ldo % 2 ||
                                (reinterpret_cast<uintptr_t>(res) | reinterpret_cast<uintptr_t>(norm_w)) % 8 ||
                                reinterpret_cast<uintptr_t>(out) % 4)) {
        tis_set_error("gemm_stream: the residual epilogue needs the stream, the norm's weight and room for the partial "
                      "sums, even row strides (%d, %d) and aligned pointers", ldr, ldo);
        return TIS_BAD_SIZE;
    }
    if (in_ss != nullptr && (in_parts <= 0 || in_width <= 0 || in_kind < TIS_NORM_L2_EPS || in_kind > TIS_NORM_MEAN_EPS)) {
        tis_set_error("gemm_stream: %d partial sums a row over a width of %d, norm kind %d", in_parts, in_width, in_kind);
        return TIS_BAD_SIZE;
    }
    if (epi == EPI_SWIGLU && N % 64) {
        tis_set_error("gemm_stream: the SwiGLU epilogue needs N %d to be a multiple of 64", N);
        return TIS_BAD_SIZE;
    }
    CUtensorMap wm;
    if (!tensor_map(w, N, K, ldw, BK, true, &wm)) return TIS_CUDA_ERROR;
    StreamParams p;
    p.x = (const bf16*)x; p.ldx = ldx; p.K = K;
    p.e.out = (bf16*)out; p.e.ldo = ldo; p.e.M = M; p.e.N = N; p.e.epi = epi; p.e.fault = fault;
    p.e.in_ss = in_ss; p.e.in_parts = in_parts; p.e.in_factor = norm_factor(in_kind, in_width, in_eps);
    p.e.res = res; p.e.ldr = ldr; p.e.norm_w = norm_w; p.e.out_ss = out_ss;
    TIS_TIMELINE_TAKE(p);
    p.kc = ((K + ksplit - 1) / ksplit + BK - 1) / BK * BK;
    const int mt = M <= 16 ? 1 : (M <= 32 ? 2 : 4);
    const int tiles = p.kc / BK;
    p.boxes = tiles < MAX_BOXES ? tiles : MAX_BOXES;
    const size_t stage = (size_t)p.boxes * BOX_BYTES + (size_t)mt * 16 * (p.kc + 8) * sizeof(bf16);
    const size_t smem = stage + cluster_reduce::recv_floats(mt * 16, ksplit) * sizeof(float) + 1024;   // + room to align the boxes
    if (smem > 224 * 1024) {
        tis_set_error("gemm_stream: %d rows x %d of K per CTA need %zu bytes of shared memory (limit 224 KB)", M, p.kc, smem);
        return TIS_BAD_SIZE;
    }

    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((N + BN - 1) / BN, ksplit, 1);
    cfg.blockDim = dim3(NTH + 32, 1, 1);
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
        cudaFuncSetAttribute(gemm_stream_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, 224 * 1024);
        cudaFuncSetAttribute(gemm_stream_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, 224 * 1024);
        cudaFuncSetAttribute(gemm_stream_kernel<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, 224 * 1024);
        configured = true;
    }
    if (mt == 1) e = cudaLaunchKernelEx(&cfg, gemm_stream_kernel<1>, wm, p);
    else if (mt == 2) e = cudaLaunchKernelEx(&cfg, gemm_stream_kernel<2>, wm, p);
    else e = cudaLaunchKernelEx(&cfg, gemm_stream_kernel<4>, wm, p);
    if (e != cudaSuccess) {
        tis_set_error("gemm_stream: %s", cudaGetErrorString(e));
        return TIS_CUDA_ERROR;
    }
    return tis_check_launch("gemm_stream");
}

TIS_API int tis_gemm_stream(const void* x, int ldx, const void* w, int ldw, void* out, int ldo, int M, int N, int K,
                            int ksplit, int epi, int* fault, cudaStream_t stream) {
    if (epi == EPI_RESIDUAL) {
        tis_set_error("gemm_stream: the residual epilogue goes through tis_gemm_stream_fused");
        return TIS_BAD_SIZE;
    }
    return tis_gemm_stream_fused(x, ldx, w, ldw, out, ldo, M, N, K, ksplit, epi, nullptr, 0, 0.f, 0, 0, nullptr, 0, nullptr,
                                 nullptr, fault, stream);
}
