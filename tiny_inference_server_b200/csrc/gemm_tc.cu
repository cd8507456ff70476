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
#include "common.cuh"
#include <cuda.h>
#include <mutex>
#include <unordered_map>
#include <string.h>

namespace {

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

__device__ __forceinline__ unsigned smem_u32(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(unsigned long long* bar, int count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_arrive(unsigned long long* bar) {
    asm volatile("{\n.reg .b64 st;\nmbarrier.arrive.shared::cta.b64 st, [%0];\n}\n" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(unsigned long long* bar, int bytes) {
    asm volatile("{\n.reg .b64 st;\nmbarrier.arrive.expect_tx.shared::cta.b64 st, [%0], %1;\n}\n"
                 ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
// Bounded wait for the phase with this parity.  Returns false when it ran out or when another
// role gave up before (`abort`); the caller then leaves its loop.
constexpr int MBAR_SPINS = 1 << 20;
__device__ __forceinline__ bool mbar_wait(unsigned long long* bar, unsigned parity, volatile int* abort, int* fault) {
    unsigned done = 0;
    for (int spin = 0; spin < MBAR_SPINS; ++spin) {
        asm volatile("{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}\n"
                     : "=r"(done) : "r"(smem_u32(bar)), "r"(parity) : "memory");
        if (done) return true;
        if ((spin & 1023) == 1023 && *abort) return false;
    }
    *abort = 1;
    atomicExch(fault, 5);
    return false;
}

__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* map, int x, int y, unsigned long long* bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];\n"
                 ::"r"(smem_u32(dst)), "l"(reinterpret_cast<unsigned long long>(map)), "r"(smem_u32(bar)), "r"(x), "r"(y)
                 : "memory");
}

// Shared-memory matrix descriptor of tcgen05.mma: start address, leading and stride byte
// offsets in units of 16 bytes, descriptor version 1, 128-byte swizzle.
__device__ __forceinline__ unsigned long long smem_desc(unsigned addr, unsigned lbo_bytes, unsigned sbo_bytes) {
    return (unsigned long long)((addr >> 4) & 0x3FFFu) | ((unsigned long long)((lbo_bytes >> 4) & 0x3FFFu) << 16) |
           ((unsigned long long)((sbo_bytes >> 4) & 0x3FFFu) << 32) | (1ull << 46) | (2ull << 61);
}
// Instruction descriptor of kind::f16: float32 accumulator, bfloat16 operands, the first
// operand K-major, the second MN-major, M = 128.
__host__ __device__ constexpr unsigned instr_desc(int n) {
    return (1u << 4) | (1u << 7) | (1u << 10) | (0u << 15) | (1u << 16) | ((unsigned)(n >> 3) << 17) |
           ((unsigned)(BM >> 4) << 24);
}
__device__ __forceinline__ void umma(unsigned tmem_d, unsigned long long a, unsigned long long b, unsigned idesc,
                                     unsigned accumulate) {
    asm volatile("{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\n"
                 "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}\n"
                 ::"r"(tmem_d), "l"(a), "l"(b), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit(unsigned long long* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n"
                 ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory"); }

// 32 consecutive accumulator columns of this thread's row (lane of tensor memory).
__device__ __forceinline__ void tmem_ld32(unsigned taddr, float (&v)[32]) {
    unsigned r[32];
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 "
                 "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
                 "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                   "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
                   "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
                   "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
                 : "r"(taddr));
    asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
#pragma unroll
    for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
}

__device__ __forceinline__ void store8(bf16* p, const float* v) {
    uint4 raw;
    __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
    *reinterpret_cast<uint4*>(p) = raw;
}

template <int BN, int STAGES, int EPI>
__global__ void __launch_bounds__(NTH, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, const TcParams p) {
    constexpr int B_BYTES = (BN / 64) * BOX_B_BYTES;
    constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
    constexpr unsigned TMEM_COLS = BN > 128 ? 512 : 256;  // two accumulators of BN float32 columns (a power of two)
    constexpr unsigned IDESC = instr_desc(BN);

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
        asm volatile("prefetch.tensormap [%0];\n" ::"l"(reinterpret_cast<unsigned long long>(&map_a)) : "memory");
        asm volatile("prefetch.tensormap [%0];\n" ::"l"(reinterpret_cast<unsigned long long>(&map_b)) : "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n"
                     ::"r"(smem_u32(&tmem_base_slot)), "r"(TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
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
                    if (!mbar_wait(&empty[s], ((it / STAGES) & 1) ^ 1, abort, p.fault)) break;
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
                if (!mbar_wait(&acc_empty[b], ((acc_it >> 1) & 1) ^ 1, abort, p.fault)) break;
                tc_fence_after();
                const unsigned d = tmem_base + b * BN;
                bool ok = true;
                for (int kt = 0; kt < kt_count; ++kt, ++it) {
                    const int s = it % STAGES;
                    if (!mbar_wait(&full[s], (it / STAGES) & 1, abort, p.fault)) { ok = false; break; }
                    tc_fence_after();
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
            if (!mbar_wait(&acc_full[b], (acc_it >> 1) & 1, abort, p.fault)) break;
            tc_fence_after();
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
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&acc_empty[b]);
        }
    }

    if (*abort) {
        // a wait ran out: give copies that may still be in flight time to land before the
        // shared memory is given up
        for (int i = 0; i < 1000; ++i) __nanosleep(1000);
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
    }
}

// ---- host side ----------------------------------------------------------------------------

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = []() -> EncodeTiledFn {
        void* f = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &f, cudaEnableDefault, &q) != cudaSuccess ||
            q != cudaDriverEntryPointSuccess)
            return nullptr;
        return reinterpret_cast<EncodeTiledFn>(f);
    }();
    return fn;
}

struct MapKey {
    const void* ptr; long long inner, outer, ld; int box_outer;
    bool operator==(const MapKey& o) const {
        return ptr == o.ptr && inner == o.inner && outer == o.outer && ld == o.ld && box_outer == o.box_outer;
    }
};
struct MapKeyHash {
    size_t operator()(const MapKey& k) const {
        size_t h = reinterpret_cast<size_t>(k.ptr);
        h = h * 1000003u ^ (size_t)k.inner;
        h = h * 1000003u ^ (size_t)k.outer;
        h = h * 1000003u ^ (size_t)k.ld;
        return h * 1000003u ^ (size_t)k.box_outer;
    }
};

// A tensor map of a row-major bfloat16 matrix (outer rows of `inner` elements, row stride ld
// elements) read in boxes of 64 elements x box_outer rows with the 128-byte swizzle.  Maps
// are descriptions only (no device memory) and are kept by address and shape.
bool tensor_map(const void* ptr, long long inner, long long outer, long long ld, int box_outer, CUtensorMap* out) {
    static std::mutex mu;
    static std::unordered_map<MapKey, CUtensorMap, MapKeyHash> cache;
    const MapKey key{ptr, inner, outer, ld, box_outer};
    std::lock_guard<std::mutex> lock(mu);
    auto it = cache.find(key);
    if (it != cache.end()) { *out = it->second; return true; }
    EncodeTiledFn enc = encode_fn();
    if (!enc) { tis_set_error("gemm_tc: the driver has no cuTensorMapEncodeTiled"); return false; }
    const cuuint64_t dims[2] = {(cuuint64_t)inner, (cuuint64_t)outer};
    const cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
    const cuuint32_t box[2] = {64, (cuuint32_t)box_outer};
    const cuuint32_t estr[2] = {1, 1};
    CUtensorMap m;
    const CUresult r = enc(&m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                           CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                           CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) { tis_set_error("gemm_tc: cuTensorMapEncodeTiled failed with %d", (int)r); return false; }
    if (cache.size() > 4096) cache.clear();
    cache.emplace(key, m);
    *out = m;
    return true;
}

int sm_count() {
    static int n = []() {
        int dev = 0, v = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev);
        return v > 0 ? v : 148;
    }();
    return n;
}

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
    if (!tensor_map(x, K, M, ldx, BM, &ma) || !tensor_map(w, N, K, ldw, BK, &mb)) return TIS_CUDA_ERROR;
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
