// Split-K reduction inside a thread-block cluster by pushing, and the epilogues of the weight-streaming products.
//
// The CTAs of a cluster hold partial sums of the same 64-column strip, each over its share of K.  Row r of the
// strip is owned by rank r % ksplit.  Every CTA writes its partial sums of a row straight from its accumulator
// registers into the owner's shared memory with st.async, each store counting its bytes on the owner's mbarrier
// (complete_tx); the owner expects ksplit x (rows it owns) x 256 bytes, waits for that barrier (acquire, cluster
// scope), adds up the ksplit partials from its OWN shared memory and runs the epilogue.  Against reading the
// partials of the others after a cluster barrier, this costs one one-way trip across the cluster instead of
// three round trips: no barrier before the reduction, no fence, no remote loads, and no barrier before the CTAs
// leave (nothing reads a CTA's memory but the CTA itself; a CTA leaves only after every partial meant for it
// has arrived).  The only cluster barrier is split: arrive when the kernel starts (after the mbarrier is
// initialised), wait just before the first push, when everybody has long arrived.  The wait on the mbarrier is
// bounded; one that runs out sets the fault word.
#pragma once
#include "common.cuh"

namespace cluster_reduce {

constexpr int STRIP = 64;             // columns of a strip
constexpr int CONSUMERS = 128;        // threads that hold accumulators: four warps, 16 columns each
enum { EPI_STORE = 0, EPI_SWIGLU = 1, EPI_RESIDUAL = 2 };

struct Epilogue {
    bf16* out; int ldo;
    int M, N;
    int epi;
    // rows that still lack their norm's factor: partial sums of squares [M][in_parts] (null: none)
    const float* in_ss; int in_parts; NormFactor in_factor;
    // EPI_RESIDUAL: the stream [M][ldr] (read and written), the next norm's weight [N], partial sums out [M][strips]
    float* res; int ldr; const float* norm_w; float* out_ss;
    int* fault;
};

// rows a rank owns at most, and the floats of its receive buffer: [source rank][owned row][64 columns]
__host__ __device__ inline int rows_per_rank(int rows_padded, int ksplit) { return (rows_padded + ksplit - 1) / ksplit; }
__host__ __device__ inline size_t recv_floats(int rows_padded, int ksplit) {
    return (size_t)ksplit * rows_per_rank(rows_padded, ksplit) * STRIP;
}

__device__ __forceinline__ unsigned shared_addr(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }
__device__ __forceinline__ unsigned map_to_rank(unsigned addr, unsigned rank) {
    unsigned r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;\n" : "=r"(r) : "r"(addr), "r"(rank));
    return r;
}
__device__ __forceinline__ void cluster_arrive() { asm volatile("barrier.cluster.arrive.release.aligned;\n" ::: "memory"); }
__device__ __forceinline__ void cluster_wait() { asm volatile("barrier.cluster.wait.acquire.aligned;\n" ::: "memory"); }

// thread 0 of the CTA, before cluster_arrive(): the barrier expects the bytes of the rows this rank owns (rows
// rank, rank + ksplit, ... below M) from every CTA of the cluster, its own among them
__device__ __forceinline__ void init_barrier(unsigned long long* bar, unsigned rank, unsigned ksplit, int M) {
    const int owned = (int)rank < M ? (M - 1 - (int)rank) / (int)ksplit + 1 : 0;
    asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;\n" ::"r"(shared_addr(bar)));
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(shared_addr(bar)),
                 "r"((unsigned)(owned * STRIP * 4) * ksplit) : "memory");
}

// The norm's factor of each row, from the partial sums of squares the kernel before left, in two halves so that the
// loads are not waited for before the loop: `RowFactorLoads::order` (consumer threads, after the dependency wait)
// only issues the loads — all rows at once, eight, four or two lanes a row, up to eight partial sums a lane — and
// `finish` (after the loop, before the barrier that precedes the epilogue) adds them up and writes the factors
// to shared memory.  More partial sums a row than that are added up at once in `order`, a warp per row.
template <int MT>              // 16 * MT rows at most: the kernel for up to 16 rows has only its own case
struct RowFactorLoads {
    float part[8];
    int shift;                  // a row is shared by 1 << shift lanes (3: up to 16 rows, 2: up to 32, 1: up to 64); 0: nothing deferred
    __device__ __forceinline__ void order(const Epilogue& e, float* row_factor, int tid) {
        shift = 0;
        if (e.in_ss == nullptr) return;
        const int warp = tid >> 5, lane = tid & 31;
        if (e.M <= 16 && e.in_parts <= 64) {          // the decode step's case, with constants
            shift = 3;
            const int row = tid >> 3, l = tid & 7;
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const int i = l + 8 * j;
                part[j] = (row < e.M && i < e.in_parts) ? e.in_ss[(size_t)row * e.in_parts + i] : 0.f;
            }
            return;
        }
        const int sh = e.M <= 32 ? 2 : 1;
        if (MT > 1 && e.in_parts <= (8 << sh)) {
            shift = sh;
            const int row = tid >> sh, l = tid & ((1 << sh) - 1);
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const int i = l + (j << sh);
                part[j] = (row < e.M && i < e.in_parts) ? e.in_ss[(size_t)row * e.in_parts + i] : 0.f;
            }
            return;
        }
        for (int r = warp; r < e.M; r += CONSUMERS / 32) {
            float s = 0.f;
            for (int i = lane; i < e.in_parts; i += 32) s += e.in_ss[(size_t)r * e.in_parts + i];
            s = warp_sum(s);
            if (lane == 0) row_factor[r] = e.in_factor.of(s);
        }
    }
    __device__ __forceinline__ void finish(const Epilogue& e, float* row_factor, int tid) const {
        if (shift == 0) return;                       // (the same for every consumer thread)
        float s = 0.f;
#pragma unroll
        for (int j = 0; j < 8; ++j) s += part[j];
        s += __shfl_xor_sync(0xffffffffu, s, 1);
        if (MT == 1 || shift > 1) s += __shfl_xor_sync(0xffffffffu, s, 2);
        if (MT == 1 || shift > 2) s += __shfl_xor_sync(0xffffffffu, s, 4);
        const int sh = MT == 1 ? 3 : shift;
        const int row = tid >> sh;
        if ((tid & ((1 << sh) - 1)) == 0 && row < e.M) row_factor[row] = e.in_factor.of(s);
    }
};

// Called by the 128 consumer threads (tid 0..127; warp w holds columns 16w..16w+15 of the strip as two n8
// fragments of mma.m16n8k16 per 16 rows), after every thread of the cluster has passed cluster_wait().
//   recv: this CTA's receive buffer (recv_floats(MT * 16, ksplit) floats); recv_bar: its barrier;
//   pair: [2][64] floats of shared memory; row_factor: [MT * 16] floats (read when e.in_ss is set);
//   strip: index of the strip (its first column is strip * 64), strips: strips of the product.
template <int MT>
__device__ __forceinline__ void push_reduce_store(const float (&acc)[MT][2][4], const Epilogue& e, float* recv,
                                                  unsigned long long* recv_bar, float (*pair)[STRIP],
                                                  const float* row_factor, unsigned rank, unsigned ksplit, int strip,
                                                  int strips, int tid) {
    const int warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
    const int rpr = rows_per_rank(MT * 16, (int)ksplit);
    const unsigned recv_base = shared_addr(recv), bar_addr = shared_addr(recv_bar);

    // push: each row's partial sums to the rank that owns the row
#pragma unroll
    for (int m = 0; m < MT; ++m)
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int row = m * 16 + g + 8 * h;
            if (row < e.M) {
                const unsigned owner = (unsigned)row % ksplit;
                const int li = row / (int)ksplit;
                const unsigned at = map_to_rank(recv_base + (unsigned)(((rank * rpr + li) * STRIP + warp * 16 + 2 * t) * 4), owner);
                const unsigned bar = map_to_rank(bar_addr, owner);
#pragma unroll
                for (int j = 0; j < 2; ++j)
                    asm volatile("st.async.shared::cluster.mbarrier::complete_tx::bytes.v2.f32 [%0], {%1, %2}, [%3];\n"
                                 ::"r"(at + j * 32), "f"(acc[m][j][2 * h]), "f"(acc[m][j][2 * h + 1]), "r"(bar) : "memory");
            }
        }

    // what the residual epilogue reads besides the partial sums does not depend on them: the norm's weight and
    // the stream of the first row this warp owns are on their way while the partials arrive
    const int c2 = 2 * lane, n2 = strip * STRIP + c2;
    const bool inside2 = n2 < e.N;                                        // N is a multiple of 8: n2 + 1 is inside too
    float2 nw = make_float2(0.f, 0.f), first_old = make_float2(0.f, 0.f);
    if (e.epi == EPI_RESIDUAL && inside2) {
        nw = *reinterpret_cast<const float2*>(e.norm_w + n2);
        const int row = warp * (int)ksplit + (int)rank;
        if (row < e.M) first_old = *reinterpret_cast<const float2*>(e.res + (size_t)row * e.ldr + n2);
    }

    // wait for the partials of all ranks (bounded)
    {
        unsigned done = 0;
        for (int spin = 0; spin < (1 << 22) && !done; ++spin)
            asm volatile("{\n.reg .pred p;\nmbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n"
                         "selp.u32 %0, 1, 0, p;\n}\n" : "=r"(done) : "r"(bar_addr), "r"(0u) : "memory");
        // a wait that ran out: flag it and go on (all threads take the same path: no barrier below is left waiting);
        // the result is then not to be used
        if (!done && e.fault != nullptr) atomicExch(e.fault, 8);
    }

    const bool scaled = e.in_ss != nullptr;
    if (e.epi == EPI_RESIDUAL) {
        // a warp per owned row, two columns per lane
        const int c = c2, n = n2;
        const bool inside = inside2;
        for (int li = warp; li * (int)ksplit + (int)rank < e.M; li += CONSUMERS / 32) {
            const int row = li * (int)ksplit + (int)rank;
            float2 sum = make_float2(0.f, 0.f);
            for (unsigned r = 0; r < ksplit; ++r) {
                const float2 v = *reinterpret_cast<const float2*>(recv + (r * rpr + li) * STRIP + c);
                sum.x += v.x; sum.y += v.y;
            }
            if (scaled) { sum.x *= row_factor[row]; sum.y *= row_factor[row]; }
            float sq = 0.f;
            if (inside) {
                float2* at = reinterpret_cast<float2*>(e.res + (size_t)row * e.ldr + n);
                float2 v = li == warp ? first_old : *at;
                v.x += sum.x; v.y += sum.y;
                *at = v;
                *reinterpret_cast<__nv_bfloat162*>(e.out + (size_t)row * e.ldo + n) = __floats2bfloat162_rn(v.x * nw.x, v.y * nw.y);
                sq = v.x * v.x + v.y * v.y;
            }
            sq = warp_sum(sq);
            if (lane == 0) e.out_ss[(size_t)row * strips + strip] = sq;
        }
        return;
    }

    // two owned rows at a time (threads 0-63 and 64-127), one column per thread
    const int half = tid >> 6, col = tid & 63;
    for (int li0 = 0; li0 * (int)ksplit + (int)rank < e.M; li0 += 2) {     // the same trips for every thread
        const int li = li0 + half;
        const int row = li * (int)ksplit + (int)rank;
        const bool valid = row < e.M;
        float sum = 0.f;
        if (valid) {
            for (unsigned r = 0; r < ksplit; ++r) sum += recv[(r * rpr + li) * STRIP + col];
            if (scaled) sum *= row_factor[row];
        }
        if (e.epi == EPI_STORE) {
            if (valid && strip * STRIP + col < e.N) e.out[(size_t)row * e.ldo + strip * STRIP + col] = __float2bfloat16_rn(sum);
        } else {
            // the strip is [32 gate | 32 up]: out column strip*32 + j = silu(gate_j) * up_j
            pair[half][col] = sum;
            asm volatile("bar.sync 1, 128;\n" ::: "memory");
            if (valid && col < 32) {
                const float gt = pair[half][col], up = pair[half][col + 32];
                e.out[(size_t)row * e.ldo + strip * 32 + col] = __float2bfloat16_rn(gt / (1.f + expf(-gt)) * up);
            }
            asm volatile("bar.sync 1, 128;\n" ::: "memory");
        }
    }
}

}  // namespace cluster_reduce
