// Matrix products with many rows on the fifth-generation tensor cores:
// y (M x N) = x (M x K) . W (K x N), bfloat16 in, float32 accumulation — the projections of
// prompt portions.  Epilogues: plain bfloat16 store, or SwiGLU gating of [32 gate | 32 up]
// column blocks (the result then has N/2 columns), so the gate/up product never goes to memory.
//
// One persistent CTA per SM walks output tiles of 128 rows x BN columns (BN = 256, 192 or 128).
// Three roles, specialised by warp:
//   warp 0   one lane orders the operand tiles from the TMA engine (cp.async.bulk.tensor.2d
//            with the 128-byte swizzle; rows beyond M, columns beyond N and K beyond its end
//            are filled with zeros by the engine) into a ring of shared-memory stages;
//   warp 1   owns the tensor memory (tcgen05.alloc) and one lane issues tcgen05.mma:
//            x tile as the K-major operand, W tile as the MN-major operand (W lies (K, N) in
//            memory, N contiguous, and is used as it is), accumulator in tensor memory;
//            tcgen05.commit hands a stage back to warp 0 and a finished accumulator to the
//            epilogue;
//   warps 2-5 read the accumulator (tcgen05.ld, one row per thread), apply the epilogue and
//            store.  The accumulator is double-buffered: the epilogue of one tile runs under
//            the products of the next.
// All hand-offs are mbarriers; every wait is bounded and a wait that runs out sets the fault
// word, lets every role leave its loop, and the tensor memory is freed before the CTA ends.
#include "tc_common.cuh"

namespace {

using namespace tc;

constexpr int BM = 128;
constexpr int BK = 64;                      // 64 bfloat16 = one 128-byte swizzle row
constexpr int NTH = 192;
constexpr int A_BYTES = BM * BK * 2;        // 16 KB
constexpr int BOX_B_BYTES = 64 * BK * 2;    // a W box: 64 rows of K x 64 columns = 8 KB

enum { EPI_STORE = 0, EPI_SWIGLU = 1 };

struct TcParams {
    bf16* out; int ldo;
    int M, N, K;
    int tiles_m, tiles_n;
    int* fault;
};

template <int BN, int STAGES, int EPI>
__global__ void __launch_bounds__(NTH, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, const TcParams p) {
    constexpr int B_BYTES = (BN / 64) * BOX_B_BYTES;
    constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
    constexpr unsigned TMEM_COLS = BN > 128 ? 512 : 256;  // two accumulators of BN float32 columns (a power of two)
    constexpr unsigned IDESC = instr_desc(BM, BN, true);

    extern __shared__ unsigned char smem_raw[];
    // operand tiles at 1024-byte boundaries: the swizzle is a function of the address
    unsigned char* tiles = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    __shared__ unsigned long long full[STAGES], empty[STAGES], acc_full[2], acc_empty[2];
    __shared__ unsigned tmem_base_slot;
    __shared__ int abort_flag;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int num_tiles = p.tiles_m * p.tiles_n;
    const int kt_count = (p.K + BK - 1) / BK;

    pdl_launch_dependents();
    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
        for (int b = 0; b < 2; ++b) { mbar_init(&acc_full[b], 1); mbar_init(&acc_empty[b], 4); }
        abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
        prefetch_map(&map_a);
        prefetch_map(&map_b);
    }
    if (warp == 1) {
        tmem_alloc(&tmem_base_slot, TMEM_COLS);
    }
    fence_before();
    __syncthreads();
    fence_after();
    const unsigned tmem_base = tmem_base_slot;
    volatile int* abort = &abort_flag;
    pdl_wait();                                           // x is the output of the kernel before

    if (warp == 0) {
        if (lane == 0) {
            int it = 0;
            for (int tile = blockIdx.x; tile < num_tiles && !*abort; tile += gridDim.x) {
                const int m0 = (tile % p.tiles_m) * BM, n0 = (tile / p.tiles_m) * BN;
                for (int kt = 0; kt < kt_count; ++kt, ++it) {
                    const int s = it % STAGES;
                    if (!mbar_wait(&empty[s], ((it / STAGES) & 1) ^ 1, abort, p.fault, 5)) break;
                    unsigned char* a = tiles + s * STAGE_BYTES;
                    mbar_arrive_expect_tx(&full[s], STAGE_BYTES);
                    tma_load_2d(a, &map_a, kt * BK, m0, &full[s]);
#pragma unroll
                    for (int j = 0; j < BN / 64; ++j)
                        tma_load_2d(a + A_BYTES + j * BOX_B_BYTES, &map_b, n0 + j * 64, kt * BK, &full[s]);
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            int it = 0, acc_it = 0;
            for (int tile = blockIdx.x; tile < num_tiles && !*abort; tile += gridDim.x, ++acc_it) {
                const int b = acc_it & 1;
                if (!mbar_wait(&acc_empty[b], ((acc_it >> 1) & 1) ^ 1, abort, p.fault, 5)) break;
                fence_after();
                const unsigned d = tmem_base + b * BN;
                bool ok = true;
                for (int kt = 0; kt < kt_count; ++kt, ++it) {
                    const int s = it % STAGES;
                    if (!mbar_wait(&full[s], (it / STAGES) & 1, abort, p.fault, 5)) { ok = false; break; }
                    fence_after();
                    const unsigned a = smem_u32(tiles + s * STAGE_BYTES), w = a + A_BYTES;
#pragma unroll
                    for (int kk = 0; kk < BK / 16; ++kk) {
                        // x: 16 elements of K further = 32 bytes inside the swizzled 128-byte row;
                        // W: 16 rows of K further = two groups of eight 128-byte rows
                        const unsigned long long da = smem_desc(a + kk * 32, 16, 1024);
                        const unsigned long long db = smem_desc(w + kk * 2048, BOX_B_BYTES, 1024);
                        umma(d, da, db, IDESC, (kt | kk) != 0);
                    }
                    umma_commit(&empty[s]);               // the stage is free when these products have read it
                }
                if (!ok) break;
                umma_commit(&acc_full[b]);
            }
        }
    } else {
        const int quarter = warp & 3;                     // the 32 lanes of tensor memory this warp may read
        int acc_it = 0;
        for (int tile = blockIdx.x; tile < num_tiles && !*abort; tile += gridDim.x, ++acc_it) {
            const int b = acc_it & 1;
            const int m0 = (tile % p.tiles_m) * BM, n0 = (tile / p.tiles_m) * BN;
            if (!mbar_wait(&acc_full[b], (acc_it >> 1) & 1, abort, p.fault, 5)) break;
            fence_after();
            const int row = m0 + quarter * 32 + lane;
            const unsigned taddr = tmem_base + ((unsigned)(quarter * 32) << 16) + b * BN;
            if (EPI == EPI_STORE) {
#pragma unroll 1
                for (int c = 0; c < BN / 32; ++c) {
                    float v[32];
                    tmem_ld32(taddr + c * 32, v);
                    if (row < p.M) {
                        bf16* o = p.out + (size_t)row * p.ldo + n0 + c * 32;
#pragma unroll
                        for (int q = 0; q < 4; ++q)
                            if (n0 + c * 32 + q * 8 < p.N) store8(o + q * 8, v + q * 8);
                    }
                }
            } else {
#pragma unroll 1
                for (int c = 0; c < BN / 64; ++c) {
                    float g[32], u[32];
                    tmem_ld32(taddr + c * 64, g);
                    tmem_ld32(taddr + c * 64 + 32, u);
                    if (row < p.M && n0 + c * 64 < p.N) {
#pragma unroll
                        for (int i = 0; i < 32; ++i) g[i] = g[i] / (1.f + __expf(-g[i])) * u[i];
                        bf16* o = p.out + (size_t)row * p.ldo + (n0 >> 1) + c * 32;
#pragma unroll
                        for (int q = 0; q < 4; ++q) store8(o + q * 8, g + q * 8);
                    }
                }
            }
            fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&acc_empty[b]);
        }
    }

    if (*abort) {
        // a wait ran out: give copies that may still be in flight time to land before the
        // shared memory is given up
        for (int i = 0; i < 1000; ++i) __nanosleep(1000);
    }
    fence_before();
    __syncthreads();
    if (warp == 1) {
        fence_after();
        tmem_free(tmem_base, TMEM_COLS);
    }
}

// ---- host side ----------------------------------------------------------------------------

template <int BN, int STAGES, int EPI>
int launch(const CUtensorMap& ma, const CUtensorMap& mb, TcParams p, cudaStream_t stream) {
    constexpr int smem = STAGES * (A_BYTES + (BN / 64) * BOX_B_BYTES) + 1024;
    static bool configured = false;
    auto kernel = gemm_tc_kernel<BN, STAGES, EPI>;
    if (!configured) {
        if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess)
            return tis_check_launch("gemm_tc (shared memory)");
        configured = true;
    }
    p.tiles_m = (p.M + BM - 1) / BM;
    p.tiles_n = (p.N + BN - 1) / BN;
    const int tiles = p.tiles_m * p.tiles_n;
    const int grid = tiles < sm_count() ? tiles : sm_count();
    tis_launch(kernel, dim3(grid), dim3(NTH), (size_t)smem, stream, ma, mb, p);
    return tis_check_launch("gemm_tc");
}

}  // namespace

// y = x . W on the tcgen05 tensor cores.  x (M x K, row stride ldx), W (K x N, row stride ldw),
// out (M x N, or M x N/2 with epi = 1), all bfloat16, strides in elements.  Refuses what the
// TMA engine cannot address: K, N and the strides must be multiples of 8 elements and the
// pointers 16-byte aligned; with epi = 1, N must be a multiple of 64.
TIS_API int tis_gemm_tc(const void* x, int ldx, const void* w, int ldw, void* out, int ldo, int M, int N, int K,
                        int epi, int* fault, cudaStream_t stream) {
    if (M <= 0 || N <= 0) return TIS_OK;
    if (K <= 0 || (K % 8) || (N % 8) || (ldx % 8) || (ldw % 8) || (ldo % 8) ||
        (reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(w) | reinterpret_cast<uintptr_t>(out)) % 16) {
        tis_set_error("gemm_tc: M %d N %d K %d strides %d %d %d: K, N and the strides must be multiples of 8 and the "
                      "pointers 16-byte aligned", M, N, K, ldx, ldw, ldo);
        return TIS_BAD_SIZE;
    }
    if (epi != EPI_STORE && epi != EPI_SWIGLU) {
        tis_set_error("gemm_tc: unknown epilogue %d", epi);
        return TIS_BAD_SIZE;
    }
    if (epi == EPI_SWIGLU && (N % 64)) {
        tis_set_error("gemm_tc: the SwiGLU epilogue takes N a multiple of 64, got %d", N);
        return TIS_BAD_SIZE;
    }
    CUtensorMap ma, mb;
    if (!tensor_map(x, K, M, ldx, BM, true, &ma) || !tensor_map(w, N, K, ldw, BK, true, &mb)) return TIS_CUDA_ERROR;
    TcParams p;
    p.out = static_cast<bf16*>(out);
    p.ldo = ldo;
    p.M = M; p.N = N; p.K = K;
    p.tiles_m = p.tiles_n = 0;
    p.fault = fault;
    // The tile width that needs the least time by a simple count: rounds of tiles over the SMs
    // times the width of a tile plus its fixed cost.
    const int tm = (M + BM - 1) / BM, sms = sm_count();
    int best = 256;
    long long best_cost = -1;
    for (int bn : {256, 192, 128}) {
        const long long tiles = (long long)tm * ((N + bn - 1) / bn);
        const long long cost = ((tiles + sms - 1) / sms) * (bn + 32);
        if (best_cost < 0 || cost < best_cost) { best = bn; best_cost = cost; }
    }
    if (epi == EPI_STORE) {
        if (best == 256) return launch<256, 4, EPI_STORE>(ma, mb, p, stream);
        if (best == 192) return launch<192, 5, EPI_STORE>(ma, mb, p, stream);
        return launch<128, 6, EPI_STORE>(ma, mb, p, stream);
    }
    if (best == 256) return launch<256, 4, EPI_SWIGLU>(ma, mb, p, stream);
    if (best == 192) return launch<192, 5, EPI_SWIGLU>(ma, mb, p, stream);
    return launch<128, 6, EPI_SWIGLU>(ma, mb, p, stream);
}
