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
#include "tc_common.cuh"
#include <cooperative_groups.h>

namespace {

using namespace tc;

constexpr int BN = 64;            // columns of a strip
constexpr int BK = 64;            // rows of K per box
constexpr int NTH = 128;
constexpr int BOX_ELEMS = BK * BN;
constexpr int BOX_BYTES = BOX_ELEMS * 2;
constexpr int MAX_BOXES = 8;      // boxes a CTA keeps in shared memory (a round)

enum { EPI_STORE = 0, EPI_SWIGLU = 1 };

struct StreamParams {
    const bf16* x; int ldx;
    bf16* out; int ldo;
    int M, N, K;
    int kc;                       // rows of K per CTA of a cluster (a multiple of BK)
    int boxes;                    // boxes in shared memory: min(kc / BK, MAX_BOXES)
    int epi;
    int* fault;
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
    constexpr int BOX_SM = BOX_ELEMS;                                 // elements of a box in shared memory
    const int xrow = p.kc + 8;                                        // padded rows: 16 bytes apart modulo 128
    bf16* w_sm = reinterpret_cast<bf16*>(base);                       // boxes x [64 k][WROW]
    bf16* xs = w_sm + (size_t)p.boxes * BOX_SM;                       // [MT*16][xrow]: this CTA's share of K
    float* red = reinterpret_cast<float*>(base);                      // after the loop: [MT*16][BN] partial sums

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const bool producer = warp == NTH / 32;
    cg::cluster_group cluster = cg::this_cluster();
    const unsigned rank = cluster.block_rank(), ksplit = cluster.num_blocks();
    const int n0 = blockIdx.x * BN;
    const int k_begin = (int)rank * p.kc;
    const int k_end = min(p.K, k_begin + p.kc);
    const int nkt = k_end > k_begin ? (k_end - k_begin + BK - 1) / BK : 0;

    asm volatile("griddepcontrol.launch_dependents;\n" ::);
    if (tid == 0) {
        abort_flag = 0;
        for (int b = 0; b < MAX_BOXES; ++b) { mbar_init(&bars[b], 1); mbar_init(&empty[b], NTH / 32); }
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    __syncthreads();

    float acc[MT][2][4];
#pragma unroll
    for (int m = 0; m < MT; ++m)
#pragma unroll
        for (int j = 0; j < 2; ++j) { acc[m][j][0] = acc[m][j][1] = acc[m][j][2] = acc[m][j][3] = 0.f; }

    if (producer) {
        // weights depend on nothing: no wait for the kernel before.  Box `it` goes to slot it % boxes, once
        // every consumer warp is done with the box that was there a round earlier.
        bool alive = true;
        for (int it = 0; it < nkt; ++it) {
            const int b = it % p.boxes;
            if (it >= p.boxes) {
                if (alive) alive = mbar_wait(&empty[b], (unsigned)(((it / p.boxes) - 1) & 1), &abort_flag, p.fault, 7);
                asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
            }
            if (lane == 0) {
                mbar_arrive_expect_tx(&bars[b], BOX_BYTES);
                tma_load_2d(w_sm + (size_t)b * BOX_SM, &wmap, n0, k_begin + it * BK, &bars[b]);
            }
        }
    } else {
    // x is the output of the kernel before this one
    asm volatile("griddepcontrol.wait;\n" ::: "memory");
    {
        const int kw = nkt * BK;                   // columns of xs that the loop reads
        const int per_row = kw / 8;
        for (int i = tid; i < MT * 16 * per_row; i += NTH) {
            const int r = i / per_row, c = (i - r * per_row) * 8;
            const int k = k_begin + c;
            const bool ok = r < p.M && k < k_end;
            cp16(xs + (size_t)r * xrow + c, ok ? p.x + (size_t)r * p.ldx + k : p.x, ok ? 16 : 0);
        }
        asm volatile("cp.async.commit_group;\n" ::);
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
        if (alive) alive = mbar_wait(&bars[b], (unsigned)((it / p.boxes) & 1), &abort_flag, p.fault, 6);
        if (!alive) continue;                      // a wait ran out: no more waits, the result is not to be used
        const unsigned box = w_base + (unsigned)b * (BOX_SM * 2);
#pragma unroll
        for (int kk = 0; kk < BK / 16; ++kk) {
            unsigned bf[4];
            const int row = kk * 16 + b_row;
            ldsm_x4_t(bf, box + row * 128 + ((b_chunk ^ (row & 7)) << 4));
#pragma unroll
            for (int m = 0; m < MT; ++m) {
                unsigned a[4];
                ldsm_x4(a, xs + (size_t)(m * 16 + (((lane >> 3) & 1) << 3) + (lane & 7)) * xrow + it * BK + kk * 16 +
                               ((lane >> 4) << 3));
                mma16816(acc[m][0], a, bf[0], bf[1]);
                mma16816(acc[m][1], a, bf[2], bf[3]);
            }
        }
        if (nkt > p.boxes) {                       // the slot is taken again a round later
            __syncwarp();
            if (lane == 0) mbar_arrive(&empty[b]);
        }
    }
    }   // consumers
    __syncthreads();                    // all warps are done with the staging memory

    // partial sums of this CTA into shared memory
    const int g = lane >> 2, t = lane & 3;
    if (!producer)
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
    const int half = (tid >> 6) & 1, col = tid & 63;
    if (!producer)
    for (int row0 = (int)rank; row0 < p.M; row0 += 2 * (int)ksplit) {      // the same trips for every consumer thread
        const int row = row0 + half * (int)ksplit;
        const bool valid = row < p.M;
        float sum = 0.f;
        if (valid)
            for (unsigned r = 0; r < ksplit; ++r) sum += cluster.map_shared_rank(red, r)[row * BN + col];
        if (p.epi == EPI_STORE) {
            if (valid && n0 + col < p.N) p.out[(size_t)row * p.ldo + n0 + col] = __float2bfloat16_rn(sum);
        } else {
            // the strip is [32 gate | 32 up]: out column strip*32 + j = silu(gate_j) * up_j
            pair[half][col] = sum;
            asm volatile("bar.sync 1, 128;\n" ::: "memory");
            if (valid && col < 32) {
                const float gt = pair[half][col], up = pair[half][col + 32];
                p.out[(size_t)row * p.ldo + blockIdx.x * 32 + col] = __float2bfloat16_rn(gt / (1.f + expf(-gt)) * up);
            }
            asm volatile("bar.sync 1, 128;\n" ::: "memory");
        }
    }
    cluster.sync();                     // nobody leaves while its shared memory may still be read
}

}  // namespace

// x (M x K, row stride ldx), w (K x N, row stride ldw), out (M x N, or M x N/2 for the SwiGLU epilogue of
// [32 gate | 32 up] column blocks; row stride ldo): bfloat16.  ksplit: CTAs per strip (1, 2, 4 or 8).
// Refuses what the TMA engine cannot address: K, N and the strides must be multiples of 8 elements and
// the pointers 16-byte aligned.
TIS_API int tis_gemm_stream(const void* x, int ldx, const void* w, int ldw, void* out, int ldo, int M, int N, int K,
                            int ksplit, int epi, int* fault, cudaStream_t stream) {
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
    if (epi != EPI_STORE && epi != EPI_SWIGLU) {
        tis_set_error("gemm_stream: unknown epilogue %d", epi);
        return TIS_BAD_SIZE;
    }
    if (epi == EPI_SWIGLU && N % 64) {
        tis_set_error("gemm_stream: the SwiGLU epilogue needs N %d to be a multiple of 64", N);
        return TIS_BAD_SIZE;
    }
    CUtensorMap wm;
    if (!tensor_map(w, N, K, ldw, BK, true, &wm)) return TIS_CUDA_ERROR;
    StreamParams p;
    p.x = (const bf16*)x; p.ldx = ldx; p.out = (bf16*)out; p.ldo = ldo;
    p.M = M; p.N = N; p.K = K; p.epi = epi; p.fault = fault;
    p.kc = ((K + ksplit - 1) / ksplit + BK - 1) / BK * BK;
    const int mt = M <= 16 ? 1 : (M <= 32 ? 2 : 4);
    const int tiles = p.kc / BK;
    p.boxes = tiles < MAX_BOXES ? tiles : MAX_BOXES;
    const size_t stage = (size_t)p.boxes * BOX_BYTES + (size_t)mt * 16 * (p.kc + 8) * sizeof(bf16);
    const size_t redb = (size_t)mt * 16 * BN * sizeof(float);
    const size_t smem = (stage > redb ? stage : redb) + 1024;        // room to align the boxes
    if (smem > 200 * 1024) {
        tis_set_error("gemm_stream: %d rows x %d of K per CTA need %zu bytes of shared memory (limit 200 KB)", M, p.kc, smem);
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
        cudaFuncSetAttribute(gemm_stream_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
        cudaFuncSetAttribute(gemm_stream_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
        cudaFuncSetAttribute(gemm_stream_kernel<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
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
