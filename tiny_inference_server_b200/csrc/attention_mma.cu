// Causal attention of step rows over the paged bfloat16 cache on the tensor cores
// (mma.sync m16n8k16, float32 accumulation), for decode rows and for portions of
// prompts, with the keys split over several CTAs when that gives more parallelism.
//
// This file is compiled once per head size: -DTIS_HD=<multiple of 16, 16..256>.
//
// Work is cut into *tiles*: up to R consecutive rows of one request.  A CTA takes one
// (tile, kv head, key split).  All G query heads that share the kv head are packed with
// the rows into the M dimension of the products (packed row m = row * G + head), so a
// key or value is read from HBM once per kv head, not once per query head.
//
//   MODE_ROWS  64 packed rows a CTA; warp w owns packed rows 16w..16w+15 and walks all keys.
//   MODE_KEYS  16 packed rows a CTA (a decode row with up to 16 query heads per kv head);
//              warp w owns keys 16w..16w+15 of every 64-key tile; the four warps' partial
//              results are merged through shared memory at the end.
//
// Keys and values of 64 positions are staged in shared memory by the TMA engine: one bulk
// copy (cp.async.bulk) per page's share of the tile (any page size), counted on an mbarrier
// per stage.  The cache stores each row with its 16-byte chunks permuted by the position
// (common.cuh), so the rows can lie dense in shared memory, exactly as copied, and ldmatrix
// still meets no bank conflict (head sizes 64, 128, 256; a few two-way conflicts at others).
// Every wait on an mbarrier is bounded; one that runs out sets the fault word.
// Scores, running maximum, sum and the output accumulate in float32; probabilities are
// rounded to bfloat16 for the P.V product (as paged_attention_kernels.py:108 upstream).
// With two to eight key splits the splits of a (tile, kv head) are one thread-block cluster
// and merge through distributed shared memory.  With more (only callers that ask for them:
// the engine plans at most eight) a CTA writes a normalised partial output and its log2-sum
// to scratch memory and `attn_merge_kernel` merges them.
#include "common.cuh"
#include "cluster_reduce.cuh"
#include "timeline.cuh"
#include <cooperative_groups.h>
#include <cstdlib>

#ifndef TIS_HD
#error "compile with -DTIS_HD=<head size>"
#endif

constexpr int HD = TIS_HD;
constexpr int KT = 64;               // keys per staged tile
constexpr int RS = HD;               // shared-memory row stride (elements): rows lie dense, as in the cache
constexpr int NTHREADS = 128;
// Stages of the copy pipeline: a launch parameter.  With many CTAs (prompt portions, large decode
// batches) two stages leave room for three CTAs per SM at head size 128, which counts for more than a
// deeper pipeline.  A decode step of few requests has fewer CTAs than the GPU has room for; what then
// bounds the kernel is the bytes it has in flight, so each CTA takes as many stages as still let all
// CTAs be resident at once (attn_launch).
constexpr int STAGE_BYTES = 2 * KT * RS * 2;
constexpr int MAX_STAGES = 8;
constexpr int MAX_CLUSTER = 16;      // key splits that merge inside one thread-block cluster (above 8: keys mode only)
constexpr int NCH = HD / 8;          // 16-byte chunks of a cache row (permuted by the position: common.cuh)
constexpr int KSTEPS = HD / 16;      // k16 steps of Q.K^T
constexpr int DTILES = HD / 8;       // n8 tiles of the output
static_assert(HD % 16 == 0 && HD >= 16 && HD <= 256, "head size must be a multiple of 16 in 16..256");

enum { MODE_ROWS = 0, MODE_KEYS = 1 };

struct AttnParams {
    const bf16* q; int q_stride;
    bf16* out; int out_stride;
    const bf16* plane; const int* block_table; int bt_stride; int num_pages;
    const int* positions; const int* row_slot;
    const int* tile_row0; const int* tile_rows;
    int H, KVH, G, page_size, window;
    float scale_log2;
    int keys_per_split, num_splits;
    float* part_o; float* part_lse;
    int cluster_merge;      // the splits of a (tile, kv head) are one thread-block cluster and merge through
                            // distributed shared memory: no scratch (2..8 splits); else scratch + merge kernel
    int* fault;
    int stages;             // stages of the copy pipeline (2..MAX_STAGES)
    int recv_offset;        // bytes from the start of shared memory to where the cluster's partial results land
    // rotary encoding and cache write done by this kernel (decode rows; see FUSED below)
    const float* rope_cos; const float* rope_sin;   // [positions][HD/2]
    bf16* plane_w;          // the plane, writable: where the row's key and value go (null: another entry fills it)
    TIS_TIMELINE_MEMBER     // (instrumented builds only; the decode kernel's stamps: 0 entry, 1 before and 2 after the
                            //  dependency wait, 3 first tile landed, 4 last tile landed, 5 loop done, 6 partial results
                            //  pushed, 7 partials of the cluster arrived, 8 stored)
};

// ---- mbarrier and bulk-copy (TMA) helpers --------------------------------------------
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
// One row of `bytes` (a multiple of 16) from global to shared memory by the TMA engine; the
// bytes are counted on `bar` when they have landed.
__device__ __forceinline__ void bulk_copy_g2s(void* dst, const void* src, int bytes, unsigned long long* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];\n"
                 ::"r"(smem_u32(dst)), "l"(src), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}
// Wait for the phase with this parity, at most MBAR_SPINS polls: a wait that runs out sets
// the fault word and goes on (the kernel never hangs; its result is then not to be used).
constexpr int MBAR_SPINS = 1 << 20;
__device__ __forceinline__ void mbar_wait(unsigned long long* bar, unsigned parity, int* fault) {
    unsigned done = 0;
    for (int spin = 0; spin < MBAR_SPINS; ++spin) {
        asm volatile("{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}\n"
                     : "=r"(done) : "r"(smem_u32(bar)), "r"(parity) : "memory");
        if (done) return;
    }
    atomicExch(fault, 4);
}
// the same for a barrier that CTAs of the cluster complete (acquire at cluster scope)
__device__ __forceinline__ void mbar_wait_cluster(unsigned long long* bar, unsigned parity, int* fault) {
    unsigned done = 0;
    for (int spin = 0; spin < MBAR_SPINS; ++spin) {
        asm volatile("{\n.reg .pred p;\nmbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n"
                     "selp.u32 %0, 1, 0, p;\n}\n" : "=r"(done) : "r"(smem_u32(bar)), "r"(parity) : "memory");
        if (done) return;
    }
    atomicExch(fault, 4);
}
__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
    return y;
}

__device__ __forceinline__ void ldmatrix_x4(unsigned (&r)[4], const void* smem) {
    const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s));
}
__device__ __forceinline__ void ldmatrix_x4_trans(unsigned (&r)[4], const void* smem) {
    const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const unsigned (&a)[4], unsigned b0, unsigned b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ unsigned pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<unsigned*>(&v);
}

// Page id of the segment that thread `tid` leads in the tile that starts at position kt
// (-1: no such segment).  Segment s of a tile is its share of logical page kt / page_size + s;
// threads 2s and 2s+1 lead its keys and its values.
__device__ __forceinline__ int fetch_page(const AttnParams& p, const int* bt, int kt, int hi, int tid) {
    const int lp = kt / p.page_size + (tid >> 1);
    const long long first = (long long)lp * p.page_size;
    if (first >= kt + KT || first >= hi) return -1;
    return bt[lp];
}

// Stage keys and values of positions kt..kt+63 of the slot.  The rows of one page lie
// together in the cache, so one bulk copy brings a page's share of the tile (keys or values)
// into the dense shared-memory tile: threads 2s / 2s+1 order segment s.  Rows of positions
// outside [lo, hi) are zero-filled by thread pairs.  Every thread arrives on the stage's
// mbarrier, leaders with the bytes they ordered.  `page` is the leader's page id (fetch_page).
__device__ __forceinline__ void load_tile(bf16* stage, unsigned long long* bar, const AttnParams& p, int page,
                                          int kvh, int kt, int lo, int hi, int tid) {
    const int which = tid & 1;
    // zero-fill: thread pair (row = tid/2, which) if its position is outside the range
    {
        const int j = kt + (tid >> 1);
        if (j < lo || j >= hi) {
            bf16* dst = stage + (which * KT + (tid >> 1)) * RS;
            const uint4 z = make_uint4(0u, 0u, 0u, 0u);
#pragma unroll
            for (int c = 0; c < NCH; ++c) *reinterpret_cast<uint4*>(dst + c * 8) = z;
        }
    }
    // segment leader
    const int lp = kt / p.page_size + (tid >> 1);
    const long long pfirst = (long long)lp * p.page_size;
    int j0 = (int)(pfirst > kt ? pfirst : kt);
    if (j0 < lo) j0 = lo;
    long long j1 = pfirst + p.page_size;
    if (j1 > kt + KT) j1 = kt + KT;
    if (j1 > hi) j1 = hi;
    const int nrows = (int)(j1 - j0);
    if (pfirst < kt + KT && nrows > 0) {
        if (page >= 0 && page < p.num_pages) {
            const bf16* src = p.plane + (((size_t)page * 2 + which) * p.KVH + kvh) * (size_t)p.page_size * HD +
                              (size_t)(j0 - pfirst) * HD;
            const int bytes = nrows * HD * 2;
            mbar_arrive_expect_tx(bar, bytes);
            bulk_copy_g2s(stage + (which * KT + (j0 - kt)) * RS, src, bytes, bar);
            return;
        }
        atomicExch(p.fault, 3);
    }
    mbar_arrive(bar);
}

// NR: packed rows a thread keeps softmax state for.  2: rows g and g+8 of the 16 a warp owns.
// 1: only row g -- the tile has at most 8 packed rows (a decode row with up to 8 query heads per
// kv head), rows 8..15 are padding and all their bookkeeping is left out.
// NG: key groups (rows mode only).  NG groups of four warps work on the same 64 packed rows;
// group g walks the staged key tiles g, g + NG, ... with stages and barriers of its own, and the
// groups' results are merged through shared memory at the end.  A long prompt's last tiles see
// thousands of keys while its first see a few: three groups cut the longest CTA's path to a third,
// and with one CTA of twelve warps per SM the heavy tiles, launched first, are followed by the
// light ones as SMs fall free.
// FUSED (keys mode, tiles of exactly one row — a decode step): q of the row is still unrotated and its
// key and value are not in the cache yet; they stand behind the queries in the row of `q`
// ([H*HD queries | KVH*HD keys | KVH*HD values], the output of the q/kv projection).  The kernel rotates
// the queries in registers as it loads them (half-split pairs, the whole head rotated: the launcher checks),
// and the CTA whose key split holds the row's own position rotates the key, writes key and value into the
// row's page for later steps, and puts them into its staged tile in place of what the copy brought.
// This kernel is then the only one of the step that writes the plane, so with `plane_w` set it may
// order its first key tiles before it waits for the kernel before it.
// The merge of the key splits of a (tile, kv head), for the 128 threads of a CTA that hold partial results
// (warp w: a quarter of the keys of every tile).  First the four warps, through the staging area (every tile has
// landed and been read): one partial result per query row.  Then over the splits by pushing (as the split-K sums of
// the weight-streaming products, cluster_reduce.cuh): output dims are owned in blocks of eight, block d by rank
// d % splits; every CTA sends its partial of a block to the owner (st.async, counted on the owner's mbarrier), the
// owner combines the partials of the splits from its own shared memory and writes the output.  No cluster barrier
// after the loop, no remote load, and a CTA leaves when it has what it owns.  Before the kernel's loop:
// merge_barrier_init by one thread, then cluster_arrive by all.
struct MergeShape {
    unsigned ns, rank;          // splits (CTAs of the cluster), this CTA's
    int pairs;                  // query rows of the tile: rows * G
    int own_blocks;             // blocks of eight dims this rank owns
    int OW;                     // floats a query row of a split takes at an owner
};
__device__ __forceinline__ MergeShape merge_shape(int num_splits, int split, int rows, int G) {
    MergeShape ms;
    ms.ns = (unsigned)num_splits; ms.rank = (unsigned)split;
    ms.pairs = rows * G;
    ms.own_blocks = split < DTILES ? (DTILES - 1 - split) / num_splits + 1 : 0;
    ms.OW = ((DTILES + num_splits - 1) / num_splits) * 8 + 4;
    return ms;
}
__device__ __forceinline__ void merge_barrier_init(unsigned long long* merge_bar, const MergeShape& ms) {
    mbar_init(merge_bar, 1);
    asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    // from each split and for each query row: its blocks, the row's maximum and sum
    mbar_arrive_expect_tx(merge_bar, ms.own_blocks ? (int)ms.ns * ms.pairs * (ms.own_blocks * 8 + 2) * 4 : 0);
}

template <int NR>
__device__ __forceinline__ void merge_splits_by_pushing(const AttnParams& p, unsigned char* smem_raw, float* recv,
                                                        unsigned long long* merge_bar, const MergeShape& ms,
                                                        const float (&o)[DTILES][4], const float (&m_run)[2],
                                                        const float (&l_run)[2], int G, int row0, int kvh) {
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int g_lane = lane >> 2, t_lane = lane & 3;
    const unsigned ns = ms.ns, rank = ms.rank;
    const int pairs = ms.pairs, own_blocks = ms.own_blocks, OW = ms.OW;
    TIS_STAMP(p, 5);
    asm volatile("bar.sync 1, 128;\n" ::: "memory");
    constexpr int HDP = HD + 4;
    float* mo = reinterpret_cast<float*>(smem_raw);          // [4][16][HDP]
    float* mm = mo + 4 * 16 * HDP;                           // [4][16]
    float* ml = mm + 4 * 16;                                 // [4][16]
#pragma unroll
    for (int i = 0; i < NR; ++i) {
        const int m = g_lane + 8 * i;
        if (t_lane == 0) { mm[warp * 16 + m] = m_run[i]; ml[warp * 16 + m] = l_run[i]; }
#pragma unroll
        for (int d = 0; d < DTILES; ++d)
            *reinterpret_cast<float2*>(mo + (warp * 16 + m) * HDP + d * 8 + 2 * t_lane) = make_float2(o[d][2 * i], o[d][2 * i + 1]);
    }
    asm volatile("bar.sync 1, 128;\n" ::: "memory");
    cluster_reduce::cluster_wait();
    const unsigned recv_base = cluster_reduce::shared_addr(recv), bar_base = cluster_reduce::shared_addr(merge_bar);
    constexpr int QUADS = HD / 4;                            // groups of four dims of a query row
    for (int u = tid; u < pairs * QUADS; u += NTHREADS) {
        const int m = u / QUADS, q = u - m * QUADS;
        float mw[4], mt = -INFINITY;
#pragma unroll
        for (int w = 0; w < 4; ++w) { mw[w] = mm[w * 16 + m]; mt = fmaxf(mt, mw[w]); }
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
        float lsum = 0.f;
#pragma unroll
        for (int w = 0; w < 4; ++w) {
            const float f = mw[w] == -INFINITY ? 0.f : fast_exp2(mw[w] - mt);
            const float4 v = *reinterpret_cast<const float4*>(mo + (w * 16 + m) * HDP + 4 * q);
            lsum += ml[w * 16 + m] * f;
            acc.x += v.x * f; acc.y += v.y * f; acc.z += v.z * f; acc.w += v.w * f;
        }
        const int block = q >> 1;
        const unsigned owner = (unsigned)block % ns;
        const unsigned at = recv_base + (unsigned)((((int)rank * pairs + m) * OW + (block / (int)ns) * 8 + (q & 1) * 4) * 4);
        asm volatile("st.async.shared::cluster.mbarrier::complete_tx::bytes.v4.f32 [%0], {%1, %2, %3, %4}, [%5];\n"
                     ::"r"(cluster_reduce::map_to_rank(at, owner)), "f"(acc.x), "f"(acc.y), "f"(acc.z), "f"(acc.w),
                       "r"(cluster_reduce::map_to_rank(bar_base, owner)) : "memory");
        // the row's maximum and sum go to every rank that owns a block: quad q sends them to rank q
        if (q < (int)ns && q < DTILES) {
            const unsigned ml_at = recv_base + (unsigned)((((int)rank * pairs + m) * OW + OW - 4) * 4);
            asm volatile("st.async.shared::cluster.mbarrier::complete_tx::bytes.v2.f32 [%0], {%1, %2}, [%3];\n"
                         ::"r"(cluster_reduce::map_to_rank(ml_at, (unsigned)q)), "f"(mt), "f"(lsum),
                           "r"(cluster_reduce::map_to_rank(bar_base, (unsigned)q)) : "memory");
        }
    }
    TIS_STAMP(p, 6);
    mbar_wait_cluster(merge_bar, 0u, p.fault);              // bounded
    TIS_STAMP(p, 7);
    const int own_dims = own_blocks * 8;
    for (int idx = tid; idx < pairs * own_dims; idx += NTHREADS) {
        const int m = idx / own_dims, c = idx - m * own_dims;
        const int d = ((c >> 3) * (int)ns + (int)rank) * 8 + (c & 7);
        const int r = m / G, g = m - r * G;
        const float* from = recv + m * OW;
        const int step_sp = pairs * OW;
        float mt = -INFINITY;
#pragma unroll 8
        for (unsigned sp = 0; sp < ns; ++sp) mt = fmaxf(mt, from[sp * step_sp + OW - 4]);
        float acc = 0.f, lsum = 0.f;
        if (mt != -INFINITY) {
#pragma unroll 8
            for (unsigned sp = 0; sp < ns; ++sp) {
                const float msp = from[sp * step_sp + OW - 4];
                const float f = msp == -INFINITY ? 0.f : fast_exp2(msp - mt);
                lsum += from[sp * step_sp + OW - 3] * f;
                acc += from[sp * step_sp + c] * f;
            }
        }
        p.out[(size_t)(row0 + r) * p.out_stride + (size_t)(kvh * G + g) * HD + d] =
            __float2bfloat16_rn(lsum > 0.f ? acc / lsum : 0.f);
    }
    TIS_STAMP(p, 8);
}

template <int MODE, int NR, int NG, bool FUSED = false>
__global__ void __launch_bounds__(NTHREADS * NG)
attn_mma_kernel(const AttnParams p) {
    static_assert(NG == 1 || MODE == MODE_ROWS, "key groups are for row tiles");
    static_assert(!FUSED || (MODE == MODE_KEYS && HD % 32 == 0), "the fused rotary path is for decode rows");
    constexpr int NT = MODE == MODE_ROWS ? 8 : 2;        // n8 key tiles a warp scores per staged tile
    constexpr int KB = MODE == MODE_ROWS ? 4 : 1;        // k16 key blocks a warp multiplies with V
    constexpr int STAGE_ELEMS = 2 * KT * RS;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    __shared__ int sh_first;
    __shared__ __align__(8) unsigned long long bars_all[NG * MAX_STAGES];
    __shared__ __align__(8) unsigned long long merge_bar;
    const int STAGES = p.stages;

    pdl_launch_dependents();         // tiles, slots, positions and block tables below are step metadata,
                                     // not written by the kernel before; pdl_wait() comes before q and the cache
    const int grp = NG == 1 ? 0 : (int)threadIdx.x / NTHREADS;          // key group of this thread
    const int tid = NG == 1 ? (int)threadIdx.x : (int)threadIdx.x % NTHREADS;   // thread inside its group
    bf16* stages = reinterpret_cast<bf16*>(smem_raw) + (size_t)grp * STAGES * STAGE_ELEMS;   // STAGES x (K[64][RS], V[64][RS])
    unsigned long long* bars = bars_all + grp * STAGES;
    // with key groups: heaviest tiles (the last rows of a prompt) first
    const int tile = NG == 1 ? (int)blockIdx.x : (int)(gridDim.x - 1 - blockIdx.x);
    const int kvh = blockIdx.y, split = blockIdx.z;
    const int warp = tid >> 5, lane = tid & 31;
    const int g_lane = lane >> 2, t_lane = lane & 3;
    // (no tile arrays: tile i is row i alone — a decode step — and two dependent loads fewer before the first copy)
    const int row0 = p.tile_row0 != nullptr ? p.tile_row0[tile] : tile, rows = p.tile_rows != nullptr ? p.tile_rows[tile] : 1;
    const int G = p.G;

    // first valid row of the tile (rows of a stage that lags the trunk start with padding)
    if (threadIdx.x == 0) {
        for (int st = 0; st < NG * STAGES; ++st) mbar_init(&bars_all[st], NTHREADS);
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    // key splits that are one cluster merge by pushing (merge_splits_by_pushing): what the cluster sends this CTA
    // lands behind the stages
    const bool pushed_merge = MODE == MODE_KEYS && p.num_splits > 1 && p.cluster_merge;
    const MergeShape ms = merge_shape(p.num_splits, split, rows, G);
    float* recv = reinterpret_cast<float*>(smem_raw + p.recv_offset);
    if (pushed_merge) {
        if (threadIdx.x == 0) merge_barrier_init(&merge_bar, ms);
        cluster_reduce::cluster_arrive();        // waited for before the first push
    }
    if (warp == 0 && grp == 0) {
        const bool v0 = lane < rows && p.row_slot[row0 + lane] >= 0;
        const bool v1 = lane + 32 < rows && p.row_slot[row0 + lane + 32] >= 0;
        const unsigned b0 = __ballot_sync(0xffffffffu, v0), b1 = __ballot_sync(0xffffffffu, v1);
        if (lane == 0) sh_first = b0 ? __ffs(b0) - 1 : (b1 ? 32 + __ffs(b1) - 1 : -1);
    }
    __syncthreads();
    const int first = sh_first;

    // the two packed rows of this thread
    const int mbase = (MODE == MODE_ROWS ? warp * 16 : 0) + g_lane;
    int r_idx[2], head[2], hi_row[2], lo_row[2];
    bool valid[2];
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const int m = mbase + 8 * i;
        const int r = m / G, g = m - r * G;
        valid[i] = i < NR && r < rows && first >= 0 && r >= first;
        r_idx[i] = row0 + (valid[i] ? r : 0);
        head[i] = kvh * G + g;
        const int pos = valid[i] ? p.positions[r_idx[i]] : 0;
        hi_row[i] = valid[i] ? pos + 1 : 0;
        lo_row[i] = (valid[i] && p.window > 0 && hi_row[i] > p.window) ? hi_row[i] - p.window : 0;
    }

    // key range of the tile and of this split
    int range_lo = 0, range_hi = 0, slot = -1;
    if (first >= 0) {
        slot = p.row_slot[row0 + rows - 1];
        const int pos_first = p.positions[row0 + first], pos_last = p.positions[row0 + rows - 1];
        range_hi = pos_last + 1;
        range_lo = (p.window > 0 && pos_first + 1 > p.window) ? pos_first + 1 - p.window : 0;
        range_lo = max(range_lo, split * p.keys_per_split);
        range_hi = min(range_hi, (split + 1) * p.keys_per_split);
    }
    const bool empty = first < 0 || range_lo >= range_hi;

    float o[DTILES][4];
#pragma unroll
    for (int d = 0; d < DTILES; ++d) { o[d][0] = o[d][1] = o[d][2] = o[d][3] = 0.f; }
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
    // block table and the first page ids are step metadata too: fetch them before the wait
    const int* bt = p.block_table + (size_t)(slot >= 0 ? slot : 0) * p.bt_stride;
    const int kt0 = (range_lo / KT) * KT;
    const int ntiles_all = empty ? 0 : (range_hi - kt0 + KT - 1) / KT;
    const int ntiles = ntiles_all > grp ? (ntiles_all - grp + NG - 1) / NG : 0;     // tiles of this group
    // the group's j-th tile starts at position kt0 + (grp + j * NG) * KT
    int page = ntiles == 0 ? -1 : fetch_page(p, bt, kt0 + grp * KT, range_hi, tid);
    // FUSED: does this CTA's split hold the row's own position?  Then it writes the row's key and value.
    int own_pos = -1, own_page = -1;
    if (FUSED && !empty && p.plane_w != nullptr) {
        const int pos = p.positions[row0 + rows - 1];
        if (pos >= range_lo && pos < range_hi) {
            own_pos = pos;
            own_page = bt[pos / p.page_size];
            if (own_page < 0 || own_page >= p.num_pages) {
                if (tid == 0) atomicExch(p.fault, 3);
                own_page = -1;
            }
        }
    }
    const int ktg_early = kt0 + grp * KT;
    const bool early = FUSED && p.plane_w != nullptr;      // nothing but this kernel writes the plane in this step
    if (early && ntiles > 0) {
        for (int st = 0; st < STAGES - 1; ++st) {
            if (st < ntiles) {
                const int page_next = fetch_page(p, bt, ktg_early + (st + 1) * NG * KT, range_hi, tid);
                load_tile(stages + st * STAGE_ELEMS, &bars[st], p, page, kvh, ktg_early + st * NG * KT, range_lo, range_hi, tid);
                page = page_next;
            }
        }
    }
    pdl_wait();

    if (ntiles > 0) {
        // query fragments straight from global memory: a0 (row g, k 2t..), a1 (row g+8), a2 (row g, k 2t+8..), a3
        unsigned qa[KSTEPS][4];
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const bf16* qrow = p.q + (size_t)r_idx[i] * p.q_stride + (size_t)head[i] * HD;
#pragma unroll
            for (int kk = 0; kk < KSTEPS; ++kk) {
                unsigned w0 = 0u, w1 = 0u;
                if (valid[i]) {
                    w0 = *reinterpret_cast<const unsigned*>(qrow + kk * 16 + 2 * t_lane);
                    w1 = *reinterpret_cast<const unsigned*>(qrow + kk * 16 + 8 + 2 * t_lane);
                }
                qa[kk][i] = w0;
                qa[kk][2 + i] = w1;
            }
        }
        if (FUSED) {
            // rotate the queries: column c of a head pairs with c + HD/2, which the same thread holds KSTEPS/2
            // fragments further on; one position for the whole tile (it has one row)
            const int pos = p.positions[row0 + rows - 1];
            const float* cs = p.rope_cos + (size_t)pos * (HD / 2);
            const float* sn = p.rope_sin + (size_t)pos * (HD / 2);
#pragma unroll
            for (int kk = 0; kk < KSTEPS / 2; ++kk) {
#pragma unroll
                for (int hf = 0; hf < 2; ++hf) {               // columns kk*16 + 2t (+1), and those + 8
                    const float2 c2 = *reinterpret_cast<const float2*>(cs + kk * 16 + hf * 8 + 2 * t_lane);
                    const float2 s2 = *reinterpret_cast<const float2*>(sn + kk * 16 + hf * 8 + 2 * t_lane);
#pragma unroll
                    for (int i = 0; i < NR; ++i) {
                        const float2 x1 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&qa[kk][2 * hf + i]));
                        const float2 x2 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&qa[kk + KSTEPS / 2][2 * hf + i]));
                        qa[kk][2 * hf + i] = pack_bf16(x1.x * c2.x - x2.x * s2.x, x1.y * c2.y - x2.y * s2.y);
                        qa[kk + KSTEPS / 2][2 * hf + i] = pack_bf16(x2.x * c2.x + x1.x * s2.x, x2.y * c2.y + x1.y * s2.y);
                    }
                }
            }
        }
        const int ktg = kt0 + grp * KT;        // the group's first tile; its tiles are NG * KT apart
        constexpr int KSTRIDE = NG * KT;

        // prologue: order STAGES-1 tiles; the page id a thread needs for the tile after is
        // fetched one tile ahead, so its latency is off the path
        for (int st = 0; st < STAGES - 1; ++st) {
            if (st < ntiles && !early) {
                const int page_next = fetch_page(p, bt, ktg + (st + 1) * KSTRIDE, range_hi, tid);
                load_tile(stages + st * STAGE_ELEMS, &bars[st], p, page, kvh, ktg + st * KSTRIDE, range_lo, range_hi, tid);
                page = page_next;
            }
        }
        for (int it = 0; it < ntiles; ++it) {
            const int kt = ktg + it * KSTRIDE;
            const int stg = it % STAGES;
            bf16* cur = stages + stg * STAGE_ELEMS;
            // everyone (of this group) is done reading the stage of tile it-1 ...
            if (NG == 1) __syncthreads();
            else asm volatile("bar.sync %0, 128;\n" ::"r"(grp + 1) : "memory");
            {
                const int nx = it + STAGES - 1;    // ... which tile it+STAGES-1 takes
                if (nx < ntiles) {
                    const int page_next = fetch_page(p, bt, ktg + (nx + 1) * KSTRIDE, range_hi, tid);
                    asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
                    load_tile(stages + (nx % STAGES) * STAGE_ELEMS, &bars[nx % STAGES], p, page, kvh, ktg + nx * KSTRIDE,
                              range_lo, range_hi, tid);
                    page = page_next;
                }
            }
            mbar_wait(&bars[stg], (unsigned)((it / STAGES) & 1), p.fault);     // tile `it` has landed

            if (FUSED && own_pos >= 0 && it == ntiles - 1) {
                // the row's own key (rotated) and value: into the page, and into the staged tile in place of
                // whatever the copy found at that position.  Warp 0: key chunk pairs; warp 1: value chunks.
                const bf16* krow = p.q + (size_t)(row0 + rows - 1) * p.q_stride + (size_t)(p.H + kvh) * HD;
                const bf16* vrow = krow + (size_t)p.KVH * HD;
                const int in_tile = own_pos - kt;
                bf16* k_sm = cur + in_tile * RS;
                bf16* v_sm = cur + (KT + in_tile) * RS;
                bf16* k_gl = own_page < 0 ? nullptr
                    : p.plane_w + (((size_t)own_page * 2) * p.KVH + kvh) * (size_t)p.page_size * HD +
                      (size_t)(own_pos % p.page_size) * HD;
                bf16* v_gl = own_page < 0 ? nullptr : k_gl + (size_t)p.KVH * p.page_size * HD;
                if (warp == 0 && lane < NCH / 2) {
                    const int c = lane;
                    float x1[8], x2[8], o1[8], o2[8];
                    Vec16<bf16>::load(krow + c * 8, x1);
                    Vec16<bf16>::load(krow + HD / 2 + c * 8, x2);
                    const float* cs = p.rope_cos + (size_t)own_pos * (HD / 2) + c * 8;
                    const float* sn = p.rope_sin + (size_t)own_pos * (HD / 2) + c * 8;
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        o1[j] = x1[j] * cs[j] - x2[j] * sn[j];
                        o2[j] = x2[j] * cs[j] + x1[j] * sn[j];
                    }
                    const int ch1 = cache_chunk(c, own_pos, NCH) * 8, ch2 = cache_chunk(c + NCH / 2, own_pos, NCH) * 8;
                    Vec16<bf16>::store(k_sm + ch1, o1);
                    Vec16<bf16>::store(k_sm + ch2, o2);
                    if (k_gl != nullptr) {
                        Vec16<bf16>::store(k_gl + ch1, o1);
                        Vec16<bf16>::store(k_gl + ch2, o2);
                    }
                } else if (warp == 1 && lane < NCH) {
                    const int c = lane;
                    const uint4 raw = *reinterpret_cast<const uint4*>(vrow + c * 8);
                    const int ch = cache_chunk(c, own_pos, NCH) * 8;
                    *reinterpret_cast<uint4*>(v_sm + ch) = raw;
                    if (v_gl != nullptr) *reinterpret_cast<uint4*>(v_gl + ch) = raw;
                }
                __syncthreads();
            }

            const bf16* ks = cur;
            const bf16* vs = cur + KT * RS;
            const int kofs = MODE == MODE_ROWS ? 0 : warp * 16;      // first key of this warp inside the tile

            // ---- S = Q K^T
            float s[NT][4];
#pragma unroll
            for (int j = 0; j < NT; ++j) { s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f; }
#pragma unroll
            for (int j = 0; j < NT; j += 2) {
#pragma unroll
                for (int kk = 0; kk < KSTEPS; ++kk) {
                    unsigned b[4];
                    const int key = kofs + j * 8 + ((lane >> 4) << 3) + (lane & 7);
                    const int chunk = cache_chunk(2 * kk + ((lane >> 3) & 1), kt + key, NCH);   // permuted by the position
                    ldmatrix_x4(b, ks + key * RS + chunk * 8);
                    mma_bf16(s[j], qa[kk], b[0], b[1]);
                    mma_bf16(s[j + 1], qa[kk], b[2], b[3]);
                }
            }
            // ---- scale, mask (only where a row's range ends inside this tile), online softmax
            float mx[2] = {-INFINITY, -INFINITY};
            const int t_lo = kt + kofs, t_hi = kt + kofs + NT * 8;
            const bool interior = t_lo >= range_lo && t_hi <= range_hi && t_lo >= lo_row[0] && t_hi <= hi_row[0] &&
                                  (NR == 1 || (t_lo >= lo_row[1] && t_hi <= hi_row[1]));
            if (interior) {
#pragma unroll
                for (int j = 0; j < NT; ++j) {
#pragma unroll
                    for (int e = 0; e < 2 * NR; ++e) {
                        const float v = s[j][e] * p.scale_log2;
                        s[j][e] = v;
                        mx[e >> 1] = fmaxf(mx[e >> 1], v);
                    }
                }
            } else {
#pragma unroll
                for (int j = 0; j < NT; ++j) {
#pragma unroll
                    for (int e = 0; e < 2 * NR; ++e) {
                        const int i = e >> 1;
                        const int kidx = kt + kofs + j * 8 + 2 * t_lane + (e & 1);
                        const bool ok = kidx >= lo_row[i] && kidx < hi_row[i] && kidx >= range_lo && kidx < range_hi;
                        const float v = ok ? s[j][e] * p.scale_log2 : -INFINITY;
                        s[j][e] = v;
                        mx[i] = fmaxf(mx[i], v);
                    }
                }
            }
            float alpha[2] = {1.f, 1.f}, m_safe[2] = {0.f, 0.f};
#pragma unroll
            for (int i = 0; i < NR; ++i) {
                mx[i] = fmaxf(mx[i], __shfl_xor_sync(0xffffffffu, mx[i], 1));
                mx[i] = fmaxf(mx[i], __shfl_xor_sync(0xffffffffu, mx[i], 2));
                const float m_new = fmaxf(m_run[i], mx[i]);
                m_safe[i] = (m_new == -INFINITY) ? 0.f : m_new;
                alpha[i] = (m_run[i] == -INFINITY) ? 0.f : fast_exp2(m_run[i] - m_safe[i]);
                m_run[i] = m_new;
            }
            float psum[2] = {0.f, 0.f};
#pragma unroll
            for (int j = 0; j < NT; ++j) {
#pragma unroll
                for (int e = 0; e < 2 * NR; ++e) {
                    const int i = e >> 1;
                    const float pv = fast_exp2(s[j][e] - m_safe[i]);  // 2^-inf = 0 for masked keys
                    s[j][e] = pv;
                    psum[i] += pv;
                }
                if (NR == 1) { s[j][2] = 0.f; s[j][3] = 0.f; }
            }
#pragma unroll
            for (int i = 0; i < NR; ++i) l_run[i] = l_run[i] * alpha[i] + psum[i];
            // the running maxima settle after a few tiles; skip the rescaling when none moved
            if (__any_sync(0xffffffffu, alpha[0] != 1.f || alpha[1] != 1.f)) {
#pragma unroll
                for (int d = 0; d < DTILES; ++d) {
                    o[d][0] *= alpha[0]; o[d][1] *= alpha[0];
                    if (NR == 2) { o[d][2] *= alpha[1]; o[d][3] *= alpha[1]; }
                }
            }
            // ---- O += P V
#pragma unroll
            for (int kb = 0; kb < KB; ++kb) {
                unsigned pa[4];
                pa[0] = pack_bf16(s[2 * kb][0], s[2 * kb][1]);
                pa[1] = pack_bf16(s[2 * kb][2], s[2 * kb][3]);
                pa[2] = pack_bf16(s[2 * kb + 1][0], s[2 * kb + 1][1]);
                pa[3] = pack_bf16(s[2 * kb + 1][2], s[2 * kb + 1][3]);
                const int key = kofs + kb * 16 + (((lane >> 3) & 1) << 3) + (lane & 7);
#pragma unroll
                for (int d = 0; d < DTILES; d += 2) {
                    unsigned b[4];
                    ldmatrix_x4_trans(b, vs + key * RS + cache_chunk(d + (lane >> 4), kt + key, NCH) * 8);
                    mma_bf16(o[d], pa, b[0], b[1]);
                    mma_bf16(o[d + 1], pa, b[2], b[3]);
                }
            }
        }
    }

    // ---- key groups: groups 1.. hand their maxima, sums and outputs to group 0
    if (NG > 1) {
        constexpr int PER = 4 + DTILES * 4;            // floats a thread hands over
        float* xg = reinterpret_cast<float*>(smem_raw);    // [NG-1][PER][128], element-major: no bank conflicts
        __syncthreads();                               // every group is done with its stages
        if (grp > 0) {
            float* dst = xg + (size_t)(grp - 1) * PER * NTHREADS + tid;
            dst[0] = m_run[0]; dst[NTHREADS] = m_run[1]; dst[2 * NTHREADS] = l_run[0]; dst[3 * NTHREADS] = l_run[1];
#pragma unroll
            for (int d = 0; d < DTILES; ++d)
#pragma unroll
                for (int e = 0; e < 4; ++e) dst[(4 + d * 4 + e) * NTHREADS] = o[d][e];
        }
        __syncthreads();
        if (grp > 0) return;                           // only group 0 writes the output (no barrier follows)
        for (int g2 = 1; g2 < NG; ++g2) {
            const float* src = xg + (size_t)(g2 - 1) * PER * NTHREADS + tid;
            float fa[2], fb[2];
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                const float mg = src[i * NTHREADS], lg = src[(2 + i) * NTHREADS];
                const float mn = fmaxf(m_run[i], mg);
                fa[i] = (m_run[i] == -INFINITY) ? 0.f : fast_exp2(m_run[i] - mn);
                fb[i] = (mg == -INFINITY) ? 0.f : fast_exp2(mg - mn);
                l_run[i] = l_run[i] * fa[i] + lg * fb[i];
                m_run[i] = mn;
            }
#pragma unroll
            for (int d = 0; d < DTILES; ++d)
#pragma unroll
                for (int e = 0; e < 4; ++e) o[d][e] = o[d][e] * fa[e >> 1] + src[(4 + d * 4 + e) * NTHREADS] * fb[e >> 1];
        }
    }

    // ---- row sums over the four lanes that share a row
#pragma unroll
    for (int i = 0; i < NR; ++i) {
        l_run[i] += __shfl_xor_sync(0xffffffffu, l_run[i], 1);
        l_run[i] += __shfl_xor_sync(0xffffffffu, l_run[i], 2);
    }

    if (pushed_merge) {
        merge_splits_by_pushing<NR>(p, smem_raw, recv, &merge_bar, ms, o, m_run, l_run, G, row0, kvh);
    } else if (MODE == MODE_KEYS) {
        // merge the four warps (each saw a quarter of the keys) through shared memory
        __syncthreads();
        float* mo = reinterpret_cast<float*>(smem_raw);          // [4][16][HD]
        float* mm = mo + 4 * 16 * HD;                            // [4][16]
        float* ml = mm + 4 * 16;                                 // [4][16]
#pragma unroll
        for (int i = 0; i < NR; ++i) {
            const int m = g_lane + 8 * i;
            if (t_lane == 0) { mm[warp * 16 + m] = m_run[i]; ml[warp * 16 + m] = l_run[i]; }
#pragma unroll
            for (int d = 0; d < DTILES; ++d) {
                mo[(warp * 16 + m) * HD + d * 8 + 2 * t_lane] = o[d][2 * i];
                mo[(warp * 16 + m) * HD + d * 8 + 2 * t_lane + 1] = o[d][2 * i + 1];
            }
        }
        __syncthreads();
        for (int idx = tid; idx < 16 * HD; idx += NTHREADS) {
            const int m = idx / HD, d = idx - m * HD;
            const int r = m / G, g = m - r * G;
            if (r >= rows) continue;
            const int row = row0 + r, hq = kvh * G + g;
            float mt = -INFINITY;
#pragma unroll
            for (int w = 0; w < 4; ++w) mt = fmaxf(mt, mm[w * 16 + m]);
            float lt = 0.f, acc = 0.f;
            if (mt != -INFINITY) {
#pragma unroll
                for (int w = 0; w < 4; ++w) {
                    const float mw = mm[w * 16 + m];
                    const float f = (mw == -INFINITY) ? 0.f : exp2f(mw - mt);
                    lt += ml[w * 16 + m] * f;
                    acc += mo[(w * 16 + m) * HD + d] * f;
                }
            }
            const float val = lt > 0.f ? acc / lt : 0.f;
            if (p.num_splits == 1) {
                p.out[(size_t)row * p.out_stride + (size_t)hq * HD + d] = __float2bfloat16_rn(val);
            } else {
                const size_t pr = ((size_t)row * p.H + hq) * p.num_splits + split;
                p.part_o[pr * HD + d] = val;
                if (d == 0) p.part_lse[pr] = lt > 0.f ? mt + log2f(lt) : -INFINITY;
            }
        }
    } else {
        if (p.num_splits > 1 && p.cluster_merge) __syncthreads();     // all warps are done with the last tile
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const int m = mbase + 8 * i;
            const int r = m / G, g = m - r * G;
            if (r >= rows) continue;
            const int row = row0 + r, hq = kvh * G + g;
            const float inv = l_run[i] > 0.f ? 1.f / l_run[i] : 0.f;
            if (p.num_splits == 1) {
                bf16* dst = p.out + (size_t)row * p.out_stride + (size_t)hq * HD;
#pragma unroll
                for (int d = 0; d < DTILES; ++d)
                    *reinterpret_cast<unsigned*>(dst + d * 8 + 2 * t_lane) = pack_bf16(o[d][2 * i] * inv, o[d][2 * i + 1] * inv);
            } else if (p.cluster_merge) {
                // this split's normalised rows into shared memory (the staging area is free now)
                float* cm_o = reinterpret_cast<float*>(smem_raw);        // [64][HD]
                float* cm_lse = cm_o + 64 * HD;                          // [64]
#pragma unroll
                for (int d = 0; d < DTILES; ++d) {
                    cm_o[m * HD + d * 8 + 2 * t_lane] = o[d][2 * i] * inv;
                    cm_o[m * HD + d * 8 + 2 * t_lane + 1] = o[d][2 * i + 1] * inv;
                }
                if (t_lane == 0) cm_lse[m] = l_run[i] > 0.f ? m_run[i] + log2f(l_run[i]) : -INFINITY;
            } else {
                const size_t pr = ((size_t)row * p.H + hq) * p.num_splits + split;
#pragma unroll
                for (int d = 0; d < DTILES; ++d) {
                    p.part_o[pr * HD + d * 8 + 2 * t_lane] = o[d][2 * i] * inv;
                    p.part_o[pr * HD + d * 8 + 2 * t_lane + 1] = o[d][2 * i + 1] * inv;
                }
                if (t_lane == 0) p.part_lse[pr] = l_run[i] > 0.f ? m_run[i] + log2f(l_run[i]) : -INFINITY;
            }
        }
        if (p.num_splits > 1 && p.cluster_merge) {
            // the splits of this (tile, kv head) are one cluster: merge through distributed shared memory
            namespace cg = cooperative_groups;
            cg::cluster_group cluster = cg::this_cluster();
            float* cm_o = reinterpret_cast<float*>(smem_raw);
            float* cm_lse = cm_o + 64 * HD;
            cluster.sync();
            const int ns = p.num_splits;
            const int pairs = rows * G;
            for (int idx = (int)cluster.block_rank() * NTHREADS + tid; idx < pairs * HD; idx += ns * NTHREADS) {
                const int m = idx / HD, d = idx - m * HD;
                const int r = m / G, g = m - r * G;
                float mt = -INFINITY;
                for (int sp = 0; sp < ns; ++sp) mt = fmaxf(mt, cluster.map_shared_rank(cm_lse, sp)[m]);
                float acc = 0.f, wsum = 0.f;
                if (mt != -INFINITY) {
                    for (int sp = 0; sp < ns; ++sp) {
                        const float l = cluster.map_shared_rank(cm_lse, sp)[m];
                        if (l == -INFINITY) continue;
                        const float w = fast_exp2(l - mt);
                        wsum += w;
                        acc += w * cluster.map_shared_rank(cm_o, sp)[m * HD + d];
                    }
                }
                p.out[(size_t)(row0 + r) * p.out_stride + (size_t)(kvh * G + g) * HD + d] =
                    __float2bfloat16_rn(wsum > 0.f ? acc / wsum : 0.f);
            }
            cluster.sync();
        }
    }
}

// ----------------------------------------------------------------------------------------------
// Decode tiles with a warp of their own for the copies.
//
// The kernel above runs its four warps in lock step: every thread helps to order the next tile and
// a CTA-wide barrier separates the tiles, so each tile costs the slowest warp plus the barrier, and a
// tile's copy is only ordered when the tile before it is done.  At decode (a handful of packed rows,
// a CTA per key split) that chain of instructions and barriers is what bounds the kernel, not the
// bytes.  Here a fifth warp does nothing but order tiles, as far ahead as there are stages; the four
// consumer warps (warp w: keys 16w..16w+15 of every staged tile, as above) never meet each other
// inside the loop.  Hand-offs are mbarriers: full[stage] (the producer's 32 lanes arrive, the
// segment leaders with the bytes they ordered) and empty[stage] (one arrival per consumer warp).
// Same tiles, same split of the keys, same merge of the splits inside the cluster as MODE_KEYS
// above; with FUSED the same rotary encoding and cache write.  Pages of at least 4 positions
// (a tile then has at most 16 page segments: two lanes each).
// ----------------------------------------------------------------------------------------------
constexpr int DEC_THREADS = NTHREADS + 32;

__device__ __forceinline__ int fetch_page_lane(const AttnParams& p, const int* bt, int kt, int hi, int lane) {
    return fetch_page(p, bt, kt, hi, lane);
}

// load_tile for one warp: lanes 2s / 2s+1 lead the keys / values of page segment s; rows of positions
// outside [lo, hi) are zero-filled by the lanes in turn; every lane arrives on the stage's barrier.
__device__ __forceinline__ void load_tile_warp(bf16* stage, unsigned long long* bar, const AttnParams& p, int page,
                                               int kvh, int kt, int lo, int hi, int lane) {
    if (kt < lo || kt + KT > hi) {
        const uint4 z = make_uint4(0u, 0u, 0u, 0u);
        for (int i = lane; i < 2 * KT; i += 32) {
            const int which = i & 1, row = i >> 1;
            const int j = kt + row;
            if (j < lo || j >= hi) {
                bf16* dst = stage + (which * KT + row) * RS;
#pragma unroll
                for (int c = 0; c < NCH; ++c) *reinterpret_cast<uint4*>(dst + c * 8) = z;
            }
        }
    }
    const int which = lane & 1;
    const int lp = kt / p.page_size + (lane >> 1);
    const long long pfirst = (long long)lp * p.page_size;
    int j0 = (int)(pfirst > kt ? pfirst : kt);
    if (j0 < lo) j0 = lo;
    long long j1 = pfirst + p.page_size;
    if (j1 > kt + KT) j1 = kt + KT;
    if (j1 > hi) j1 = hi;
    const int nrows = (int)(j1 - j0);
    if (pfirst < kt + KT && nrows > 0) {
        if (page >= 0 && page < p.num_pages) {
            const bf16* src = p.plane + (((size_t)page * 2 + which) * p.KVH + kvh) * (size_t)p.page_size * HD +
                              (size_t)(j0 - pfirst) * HD;
            const int bytes = nrows * HD * 2;
            mbar_arrive_expect_tx(bar, bytes);
            bulk_copy_g2s(stage + (which * KT + (j0 - kt)) * RS, src, bytes, bar);
            return;
        }
        atomicExch(p.fault, 3);
    }
    mbar_arrive(bar);
}

template <int NR, bool FUSED>
__global__ void __launch_bounds__(DEC_THREADS, HD <= 128 ? 2 : 1)
attn_decode_kernel(const AttnParams p) {
    static_assert(!FUSED || HD % 32 == 0, "the fused rotary path rotates pairs of k16 fragments");
    constexpr int NT = 2;                                // n8 key tiles a warp scores per staged tile
    constexpr int STAGE_ELEMS = 2 * KT * RS;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    __shared__ int sh_first;
    __shared__ __align__(16) float rope_sh[HD];                       // FUSED: the row's cosines, then its sines
    __shared__ __align__(8) unsigned long long full[MAX_STAGES], empty[MAX_STAGES], merge_bar;
    const int STAGES = p.stages;

    TIS_STAMP(p, 0);
    pdl_launch_dependents();
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const bool producer = warp == NTHREADS / 32;
    bf16* stages = reinterpret_cast<bf16*>(smem_raw);
    const int tile = blockIdx.x, kvh = blockIdx.y, split = blockIdx.z;
    const int g_lane = lane >> 2, t_lane = lane & 3;
    // (no tile arrays: tile i is row i alone — a decode step — and two dependent loads fewer before the first copy)
    const int row0 = p.tile_row0 != nullptr ? p.tile_row0[tile] : tile, rows = p.tile_rows != nullptr ? p.tile_rows[tile] : 1;
    const int G = p.G;

    // the merge of the splits (merge_splits_by_pushing): the barrier that counts what the cluster sends this CTA
    const MergeShape ms = merge_shape(p.num_splits, split, rows, G);
    float* recv = reinterpret_cast<float*>(smem_raw + p.recv_offset);
    if (tid == 0) {
        for (int st = 0; st < STAGES; ++st) { mbar_init(&full[st], 32); mbar_init(&empty[st], NTHREADS / 32); }
        merge_barrier_init(&merge_bar, ms);
    }
    cluster_reduce::cluster_arrive();        // waited for before the first push: by then every CTA's barrier is ready
    // what a thread needs of the last row of the tile does not depend on which rows are valid: its loads go out
    // together with the one that finds the first valid row, not after it (a CTA that starts late has its first copy
    // a trip to the L2 cache earlier)
    const int slot_last = p.row_slot[row0 + rows - 1], pos_last_early = p.positions[row0 + rows - 1];
    if (warp == 0) {
        const bool v0 = lane < rows && p.row_slot[row0 + lane] >= 0;
        const unsigned b0 = __ballot_sync(0xffffffffu, v0);
        if (lane == 0) sh_first = b0 ? __ffs(b0) - 1 : -1;       // a tile of this kind has at most 16 rows
    }
    __syncthreads();
    const int first = sh_first;

    const int mbase = g_lane;
    int r_idx[2], head[2], hi_row[2], lo_row[2];
    bool valid[2];
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const int m = mbase + 8 * i;
        const int r = m / G, g = m - r * G;
        valid[i] = i < NR && r < rows && first >= 0 && r >= first;
        r_idx[i] = row0 + (valid[i] ? r : 0);
        head[i] = kvh * G + g;
        const int pos = valid[i] ? p.positions[r_idx[i]] : 0;
        hi_row[i] = valid[i] ? pos + 1 : 0;
        lo_row[i] = (valid[i] && p.window > 0 && hi_row[i] > p.window) ? hi_row[i] - p.window : 0;
    }
    int range_lo = 0, range_hi = 0, slot = -1;
    if (first >= 0) {
        slot = slot_last;
        const int pos_last = pos_last_early;
        const int pos_first = first == rows - 1 ? pos_last : p.positions[row0 + first];
        range_hi = pos_last + 1;
        range_lo = (p.window > 0 && pos_first + 1 > p.window) ? pos_first + 1 - p.window : 0;
        range_lo = max(range_lo, split * p.keys_per_split);
        range_hi = min(range_hi, (split + 1) * p.keys_per_split);
    }
    const bool none = first < 0 || range_lo >= range_hi;
    const int* bt = p.block_table + (size_t)(slot >= 0 ? slot : 0) * p.bt_stride;
    const int kt0 = (range_lo / KT) * KT;
    const int ntiles = none ? 0 : (range_hi - kt0 + KT - 1) / KT;

    float o[DTILES][4];
#pragma unroll
    for (int d = 0; d < DTILES; ++d) { o[d][0] = o[d][1] = o[d][2] = o[d][3] = 0.f; }
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};

    if (producer) {
        // with FUSED and a plane of its own this kernel is the only one of the step that writes the plane:
        // no tile depends on the kernel before, and the copies start at once
        if (!(FUSED && p.plane_w != nullptr)) pdl_wait();
        int page = ntiles == 0 ? -1 : fetch_page_lane(p, bt, kt0, range_hi, lane);
        for (int it = 0; it < ntiles; ++it) {
            const int stg = it % STAGES;
            const int kt = kt0 + it * KT;
            const int page_next = fetch_page_lane(p, bt, kt + KT, range_hi, lane);
            if (it >= STAGES) {
                mbar_wait(&empty[stg], (unsigned)(((it / STAGES) - 1) & 1), p.fault);   // every consumer warp is done with it
                asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
            }
            load_tile_warp(stages + stg * STAGE_ELEMS, &full[stg], p, page, kvh, kt, range_lo, range_hi, lane);
            page = page_next;
        }
        cluster_reduce::cluster_wait();
    } else {
        // FUSED: does this CTA's split hold the row's own position?  Then it writes the row's key and value.
        int own_pos = -1, own_page = -1;
        if (FUSED && !none && p.plane_w != nullptr) {
            const int pos = p.positions[row0 + rows - 1];
            if (pos >= range_lo && pos < range_hi) {
                own_pos = pos;
                own_page = bt[pos / p.page_size];
                if (own_page < 0 || own_page >= p.num_pages) {
                    if (tid == 0) atomicExch(p.fault, 3);
                    own_page = -1;
                }
            }
        }
        // the angles of the row's position do not depend on the kernel before: the consumer warps bring them into
        // shared memory while they would only wait (in registers they would not fit beside the queries)
        if (FUSED && ntiles > 0) {
            const int pos = p.positions[row0 + rows - 1];
            for (int i = tid; i < HD / 4; i += NTHREADS) {              // HD / 2 cosines and as many sines, four a thread
                const float* src = i < HD / 8 ? p.rope_cos + (size_t)pos * (HD / 2) + 4 * i
                                              : p.rope_sin + (size_t)pos * (HD / 2) + 4 * (i - HD / 8);
                *reinterpret_cast<float4*>(rope_sh + 4 * i) = *reinterpret_cast<const float4*>(src);
            }
        }
        asm volatile("bar.sync 1, 128;\n" ::: "memory");
        TIS_STAMP(p, 1);
        pdl_wait();
        TIS_STAMP(p, 2);
        if (ntiles > 0) {
            unsigned qa[KSTEPS][4];
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                const bf16* qrow = p.q + (size_t)r_idx[i] * p.q_stride + (size_t)head[i] * HD;
#pragma unroll
                for (int kk = 0; kk < KSTEPS; ++kk) {
                    unsigned w0 = 0u, w1 = 0u;
                    if (valid[i]) {
                        w0 = *reinterpret_cast<const unsigned*>(qrow + kk * 16 + 2 * t_lane);
                        w1 = *reinterpret_cast<const unsigned*>(qrow + kk * 16 + 8 + 2 * t_lane);
                    }
                    qa[kk][i] = w0;
                    qa[kk][2 + i] = w1;
                }
            }
            if (FUSED) {
                const float* cs = rope_sh;
                const float* sn = rope_sh + HD / 2;
#pragma unroll
                for (int kk = 0; kk < KSTEPS / 2; ++kk) {
#pragma unroll
                    for (int hf = 0; hf < 2; ++hf) {
                        const float2 c2 = *reinterpret_cast<const float2*>(cs + kk * 16 + hf * 8 + 2 * t_lane);
                        const float2 s2 = *reinterpret_cast<const float2*>(sn + kk * 16 + hf * 8 + 2 * t_lane);
#pragma unroll
                        for (int i = 0; i < NR; ++i) {
                            const float2 x1 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&qa[kk][2 * hf + i]));
                            const float2 x2 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&qa[kk + KSTEPS / 2][2 * hf + i]));
                            qa[kk][2 * hf + i] = pack_bf16(x1.x * c2.x - x2.x * s2.x, x1.y * c2.y - x2.y * s2.y);
                            qa[kk + KSTEPS / 2][2 * hf + i] = pack_bf16(x2.x * c2.x + x1.x * s2.x, x2.y * c2.y + x1.y * s2.y);
                        }
                    }
                }
            }
            for (int it = 0; it < ntiles; ++it) {
                const int kt = kt0 + it * KT;
                const int stg = it % STAGES;
                bf16* cur = stages + stg * STAGE_ELEMS;
                mbar_wait(&full[stg], (unsigned)((it / STAGES) & 1), p.fault);         // tile `it` has landed
                if (it == 0) TIS_STAMP(p, 3);
                if (it == ntiles - 1) TIS_STAMP(p, 4);

                if (FUSED && own_pos >= 0 && it == ntiles - 1) {
                    const bf16* krow = p.q + (size_t)(row0 + rows - 1) * p.q_stride + (size_t)(p.H + kvh) * HD;
                    const bf16* vrow = krow + (size_t)p.KVH * HD;
                    const int in_tile = own_pos - kt;
                    bf16* k_sm = cur + in_tile * RS;
                    bf16* v_sm = cur + (KT + in_tile) * RS;
                    bf16* k_gl = own_page < 0 ? nullptr
                        : p.plane_w + (((size_t)own_page * 2) * p.KVH + kvh) * (size_t)p.page_size * HD +
                          (size_t)(own_pos % p.page_size) * HD;
                    bf16* v_gl = own_page < 0 ? nullptr : k_gl + (size_t)p.KVH * p.page_size * HD;
                    if (warp == 0 && lane < NCH / 2) {
                        const int c = lane;
                        float x1[8], x2[8], o1[8], o2[8];
                        Vec16<bf16>::load(krow + c * 8, x1);
                        Vec16<bf16>::load(krow + HD / 2 + c * 8, x2);
                        const float* cs = rope_sh + c * 8;                  // (the row's own position: the angles above)
                        const float* sn = rope_sh + HD / 2 + c * 8;
#pragma unroll
                        for (int j = 0; j < 8; ++j) {
                            o1[j] = x1[j] * cs[j] - x2[j] * sn[j];
                            o2[j] = x2[j] * cs[j] + x1[j] * sn[j];
                        }
                        const int ch1 = cache_chunk(c, own_pos, NCH) * 8, ch2 = cache_chunk(c + NCH / 2, own_pos, NCH) * 8;
                        Vec16<bf16>::store(k_sm + ch1, o1);
                        Vec16<bf16>::store(k_sm + ch2, o2);
                        if (k_gl != nullptr) {
                            Vec16<bf16>::store(k_gl + ch1, o1);
                            Vec16<bf16>::store(k_gl + ch2, o2);
                        }
                    } else if (warp == 1 && lane < NCH) {
                        const int c = lane;
                        const uint4 raw = *reinterpret_cast<const uint4*>(vrow + c * 8);
                        const int ch = cache_chunk(c, own_pos, NCH) * 8;
                        *reinterpret_cast<uint4*>(v_sm + ch) = raw;
                        if (v_gl != nullptr) *reinterpret_cast<uint4*>(v_gl + ch) = raw;
                    }
                    asm volatile("bar.sync 1, 128;\n" ::: "memory");       // the consumer warps only
                }

                const bf16* ks = cur;
                const bf16* vs = cur + KT * RS;
                const int kofs = warp * 16;
                float s[NT][4];
#pragma unroll
                for (int j = 0; j < NT; ++j) { s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f; }
#pragma unroll
                for (int kk = 0; kk < KSTEPS; ++kk) {
                    unsigned b[4];
                    const int key = kofs + ((lane >> 4) << 3) + (lane & 7);
                    const int chunk = cache_chunk(2 * kk + ((lane >> 3) & 1), kt + key, NCH);
                    ldmatrix_x4(b, ks + key * RS + chunk * 8);
                    mma_bf16(s[0], qa[kk], b[0], b[1]);
                    mma_bf16(s[1], qa[kk], b[2], b[3]);
                }
                float mx[2] = {-INFINITY, -INFINITY};
                const int t_lo = kt + kofs, t_hi = kt + kofs + NT * 8;
                const bool interior = t_lo >= range_lo && t_hi <= range_hi && t_lo >= lo_row[0] && t_hi <= hi_row[0] &&
                                      (NR == 1 || (t_lo >= lo_row[1] && t_hi <= hi_row[1]));
                if (interior) {
#pragma unroll
                    for (int j = 0; j < NT; ++j)
#pragma unroll
                        for (int e = 0; e < 2 * NR; ++e) {
                            const float v = s[j][e] * p.scale_log2;
                            s[j][e] = v;
                            mx[e >> 1] = fmaxf(mx[e >> 1], v);
                        }
                } else {
#pragma unroll
                    for (int j = 0; j < NT; ++j)
#pragma unroll
                        for (int e = 0; e < 2 * NR; ++e) {
                            const int i = e >> 1;
                            const int kidx = kt + kofs + j * 8 + 2 * t_lane + (e & 1);
                            const bool ok = kidx >= lo_row[i] && kidx < hi_row[i] && kidx >= range_lo && kidx < range_hi;
                            const float v = ok ? s[j][e] * p.scale_log2 : -INFINITY;
                            s[j][e] = v;
                            mx[i] = fmaxf(mx[i], v);
                        }
                }
                float alpha[2] = {1.f, 1.f}, m_safe[2] = {0.f, 0.f};
#pragma unroll
                for (int i = 0; i < NR; ++i) {
                    mx[i] = fmaxf(mx[i], __shfl_xor_sync(0xffffffffu, mx[i], 1));
                    mx[i] = fmaxf(mx[i], __shfl_xor_sync(0xffffffffu, mx[i], 2));
                    const float m_new = fmaxf(m_run[i], mx[i]);
                    m_safe[i] = (m_new == -INFINITY) ? 0.f : m_new;
                    alpha[i] = (m_run[i] == -INFINITY) ? 0.f : fast_exp2(m_run[i] - m_safe[i]);
                    m_run[i] = m_new;
                }
                float psum[2] = {0.f, 0.f};
#pragma unroll
                for (int j = 0; j < NT; ++j) {
#pragma unroll
                    for (int e = 0; e < 2 * NR; ++e) {
                        const int i = e >> 1;
                        const float pv = fast_exp2(s[j][e] - m_safe[i]);
                        s[j][e] = pv;
                        psum[i] += pv;
                    }
                    if (NR == 1) { s[j][2] = 0.f; s[j][3] = 0.f; }
                }
#pragma unroll
                for (int i = 0; i < NR; ++i) l_run[i] = l_run[i] * alpha[i] + psum[i];
                if (__any_sync(0xffffffffu, alpha[0] != 1.f || alpha[1] != 1.f)) {
#pragma unroll
                    for (int d = 0; d < DTILES; ++d) {
                        o[d][0] *= alpha[0]; o[d][1] *= alpha[0];
                        if (NR == 2) { o[d][2] *= alpha[1]; o[d][3] *= alpha[1]; }
                    }
                }
                unsigned pa[4];
                pa[0] = pack_bf16(s[0][0], s[0][1]);
                pa[1] = pack_bf16(s[0][2], s[0][3]);
                pa[2] = pack_bf16(s[1][0], s[1][1]);
                pa[3] = pack_bf16(s[1][2], s[1][3]);
                const int key = kofs + (((lane >> 3) & 1) << 3) + (lane & 7);
#pragma unroll
                for (int d = 0; d < DTILES; d += 2) {
                    unsigned b[4];
                    ldmatrix_x4_trans(b, vs + key * RS + cache_chunk(d + (lane >> 4), kt + key, NCH) * 8);
                    mma_bf16(o[d], pa, b[0], b[1]);
                    mma_bf16(o[d + 1], pa, b[2], b[3]);
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(&empty[stg]);                   // this warp is done with the stage
            }
        }
#pragma unroll
        for (int i = 0; i < NR; ++i) {
            l_run[i] += __shfl_xor_sync(0xffffffffu, l_run[i], 1);
            l_run[i] += __shfl_xor_sync(0xffffffffu, l_run[i], 2);
        }
        merge_splits_by_pushing<NR>(p, smem_raw, recv, &merge_bar, ms, o, m_run, l_run, G, row0, kvh);
    }
}

// out[row, head] = sum_s w_s * part_o[row, head, s],  w_s = 2^(lse_s - max) / sum, for the rows of one tile
__global__ void attn_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_lse,
                                  bf16* __restrict__ out, int out_stride, const int* __restrict__ tile_row0,
                                  const int* __restrict__ tile_rows, int H, int num_splits) {
    const int tile = blockIdx.y, hq = blockIdx.x;
    const int row0 = tile_row0 != nullptr ? tile_row0[tile] : tile, rows = tile_rows != nullptr ? tile_rows[tile] : 1;
    for (int r = 0; r < rows; ++r) {
        const int row = row0 + r;
        const size_t pr = ((size_t)row * H + hq) * num_splits;
        float mt = -INFINITY;
        for (int s = 0; s < num_splits; ++s) mt = fmaxf(mt, part_lse[pr + s]);
        for (int d = threadIdx.x; d < HD; d += blockDim.x) {
            float acc = 0.f, wsum = 0.f;
            if (mt != -INFINITY) {
                for (int s = 0; s < num_splits; ++s) {
                    const float l = part_lse[pr + s];
                    if (l == -INFINITY) continue;
                    const float w = exp2f(l - mt);
                    wsum += w;
                    acc += w * part_o[(pr + s) * HD + d];
                }
            }
            out[(size_t)row * out_stride + (size_t)hq * HD + d] = __float2bfloat16_rn(wsum > 0.f ? acc / wsum : 0.f);
        }
    }
}

static size_t smem_bytes(int mode, int stages = 2) {
    size_t stage = (size_t)stages * STAGE_BYTES;
    size_t merge = mode == MODE_KEYS ? (size_t)(4 * 16 * (HD + 4) + 2 * 4 * 16) * sizeof(float)
                                     : (size_t)(64 * HD + 64) * sizeof(float);
    return stage > merge ? stage : merge;
}

TIS_API int tis_attn_head_dim() { return HD; }

// CTAs of one SM that run at a time (registers and shared memory), times the SMs of the device.
TIS_API int tis_attn_resident_ctas(int mode, int half) {
    int per_sm = 0, dev = 0, sms = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    const size_t smem = smem_bytes(mode);
    if (mode == MODE_ROWS) {
        cudaFuncSetAttribute(attn_mma_kernel<MODE_ROWS, 2, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, attn_mma_kernel<MODE_ROWS, 2, 1>, NTHREADS, smem);
    } else if (half) {
        // (the keys-mode kernels may be launched with more stages than two: their limit stays at the most)
        cudaFuncSetAttribute(attn_mma_kernel<MODE_KEYS, 1, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024);
        cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, attn_mma_kernel<MODE_KEYS, 1, 1>, NTHREADS, smem);
    } else {
        cudaFuncSetAttribute(attn_mma_kernel<MODE_KEYS, 2, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024);
        cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, attn_mma_kernel<MODE_KEYS, 2, 1>, NTHREADS, smem);
    }
    cudaGetLastError();
    return per_sm > 0 && sms > 0 ? per_sm * sms : 148 * 2;
}

// Scratch the caller must provide when num_splits > 1: floats for part_o and part_lse.
TIS_API size_t tis_attn_scratch_floats(int n_rows, int H, int num_splits) {
    return num_splits > 1 ? (size_t)n_rows * H * num_splits * (HD + 1) : 0;
}

// mode: 0 rows (tiles of up to 64/G rows), 1 keys (tiles of up to 16/G rows).
// max_tile_rows: the most rows any tile has (0: unknown); keys-mode tiles of at most 8 packed
// rows take a kernel that keeps no state for the padding rows.
// CTAs of a mode that one SM holds at a time: tis_attn_resident_ctas.
// decode tiles: the kernel with a producer warp (1) or the lock-step kernel (0); TIS_ATTN_DECODE_WS in the
// environment of the process, read once
static const bool g_decode_ws = []() { const char* e = getenv("TIS_ATTN_DECODE_WS"); return !(e && e[0] == '0'); }();

static int attn_launch(int mode, const void* q, int q_stride, void* out, int out_stride, const void* plane,
                       const int* block_table, int bt_stride, int num_pages, const int* positions,
                       const int* row_slot, const int* tile_row0, const int* tile_rows, int num_tiles,
                       int max_tile_rows, int n_rows, int H, int KVH, int page_size, int window, float scale,
                       int keys_per_split, int num_splits, float* scratch, int* fault, cudaStream_t stream,
                       const float* rope_cos, const float* rope_sin, int write_kv) {
    if (num_tiles <= 0) return TIS_OK;
    const bool fused = rope_cos != nullptr;
    if (fused && (mode != MODE_KEYS || max_tile_rows != 1 || HD % 32 != 0 || rope_sin == nullptr)) {
        tis_set_error("attention: the rotary encoding is done inside the kernel only for tiles of one row (got %d) in "
                      "keys mode and head sizes that are multiples of 32 (this library: %d)", max_tile_rows, HD);
        return TIS_BAD_SIZE;
    }
    const int G = KVH > 0 ? H / KVH : 0;
    const int mpack = mode == MODE_ROWS ? 64 : 16;
    if (KVH <= 0 || H % KVH) {
        tis_set_error("attention: %d query heads are not a multiple of %d kv heads", H, KVH);
        return TIS_BAD_SIZE;
    }
    if (G > mpack) {
        tis_set_error("attention: %d query heads per kv head exceed the %d packed rows of this mode", G, mpack);
        return TIS_BAD_SIZE;
    }
    if (keys_per_split <= 0 || keys_per_split % KT || num_splits <= 0) {
        tis_set_error("attention: keys per split %d must be a positive multiple of %d", keys_per_split, KT);
        return TIS_BAD_SIZE;
    }
    if (KVH > 65535 || num_splits > 65535) {
        tis_set_error("attention: %d kv heads or %d splits exceed the grid", KVH, num_splits);
        return TIS_BAD_SIZE;
    }
    if (num_splits > (mode == MODE_KEYS ? MAX_CLUSTER : 8) && scratch == nullptr) {
        tis_set_error("attention: %d key splits need scratch memory", num_splits);
        return TIS_BAD_SIZE;
    }
    AttnParams p;
    p.q = (const bf16*)q; p.q_stride = q_stride; p.out = (bf16*)out; p.out_stride = out_stride;
    p.plane = (const bf16*)plane; p.block_table = block_table; p.bt_stride = bt_stride; p.num_pages = num_pages;
    p.positions = positions; p.row_slot = row_slot; p.tile_row0 = tile_row0; p.tile_rows = tile_rows;
    p.H = H; p.KVH = KVH; p.G = G; p.page_size = page_size; p.window = window;
    p.scale_log2 = scale * 1.4426950408889634f;
    p.keys_per_split = keys_per_split; p.num_splits = num_splits;
    p.part_o = scratch;
    p.part_lse = scratch ? scratch + (size_t)n_rows * H * num_splits * HD : nullptr;
    p.cluster_merge = (num_splits > 1 && num_splits <= (mode == MODE_KEYS && scratch == nullptr ? MAX_CLUSTER : 8)) ? 1 : 0;
    p.fault = fault;
    p.rope_cos = rope_cos; p.rope_sin = rope_sin;
    p.plane_w = (fused && write_kv) ? (bf16*)plane : nullptr;
    TIS_TIMELINE_TAKE(p);
    // decode tiles go to the kernel with a producer warp where its layout allows (page segments: two lanes each)
    // and while all its CTAs are resident at once, two to an SM (its 160 threads hold as many registers as allow
    // two; the lock-step kernel fits three).  Measured on a B200 at head size 128, context 4096, us a launch,
    // lock-step -> producer warp: batch 1 12.7 -> 11.2, batch 4 16.1 -> 13.6, batch 8 18.8 -> 15.2 (192 CTAs);
    // batch 16 23.2 -> 30.8 (384 CTAs, a second wave), batch 64 64.8 -> 87.5.
    static int sm_count = 0;
    if (sm_count == 0) {
        int dev = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev);
        if (sm_count <= 0) sm_count = 148;
    }
    const bool warp_specialised = mode == MODE_KEYS && page_size >= 4 && g_decode_ws &&
                                  (num_splits == 1 || p.cluster_merge) &&
                                  (long long)num_tiles * KVH * num_splits <= 2LL * sm_count;
    // stages: two; for decode tiles of a grid that leaves SMs empty anyway (fewer CTAs than SMs) as many as
    // fit one CTA per SM and a split has tiles to fill (measured inside the decode step of the 0.9B model:
    // batch 1, 24 CTAs, six stages: 1.289 -> 1.235 ms a step); the kernel with a producer warp, whose copies
    // run ahead of the consumers, takes three wherever two CTAs of three stages fit an SM.
    // the kernel with a producer warp also keeps, beside the stages, what the cluster pushes to it for the merge:
    // from each split, for each query row of a tile, its output blocks, the row's maximum and sum
    size_t recv_bytes = 0;
    if (warp_specialised || (mode == MODE_KEYS && p.cluster_merge)) {
        const int pairs = max_tile_rows > 0 ? max_tile_rows * G : 16;
        recv_bytes = (size_t)num_splits * pairs * (((HD / 8 + num_splits - 1) / num_splits) * 8 + 4) * sizeof(float);
    }
    int stages = 2;
    if (mode == MODE_KEYS) {
        const int sms = sm_count;
        const long long ctas = (long long)num_tiles * KVH * num_splits;
        const int tiles_per_split = keys_per_split / KT;
        for (int cand = 3; cand <= MAX_STAGES; ++cand) {
            const size_t need = (warp_specialised ? (size_t)cand * STAGE_BYTES : smem_bytes(MODE_KEYS, cand)) + recv_bytes;
            if (need > 220 * 1024 || cand - 1 > tiles_per_split) break;
            // the kernel with a producer warp: no more stages than a split has tiles (shared memory that it leaves
            // free lets its CTAs start beside those of the product before it, and order their tiles, earlier)
            if (warp_specialised && cand > tiles_per_split) break;
            // the kernel with a producer warp keeps three stages wherever two CTAs of them fit an SM
            const bool fits_twice = warp_specialised && cand == 3 && 2 * (need + 1024) <= 220 * 1024;
            if (ctas > (long long)sms && !fits_twice) break;
            stages = cand;
        }
    }
    p.stages = stages;
    // the partial results of the cluster land behind the stages (and behind what the four warps of a CTA merge in)
    const size_t front = warp_specialised ? (size_t)stages * STAGE_BYTES : smem_bytes(mode, stages);
    p.recv_offset = (int)front;
    const size_t smem = front + recv_bytes;
    if (smem > 220 * 1024) {
        tis_set_error("attention: %d stages and the merge of %d splits need %zu bytes of shared memory", stages, num_splits, smem);
        return TIS_BAD_SIZE;
    }
    dim3 grid(num_tiles, KVH, num_splits);
    static bool configured = false;          // once per process (and before any stream capture)
    if (!configured) {
        cudaFuncSetAttribute(attn_mma_kernel<MODE_ROWS, 2, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             (int)smem_bytes(MODE_ROWS));
        cudaFuncSetAttribute(attn_mma_kernel<MODE_KEYS, 2, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024);
        cudaFuncSetAttribute(attn_mma_kernel<MODE_KEYS, 1, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024);
        cudaFuncSetAttribute(attn_mma_kernel<MODE_KEYS, 2, 1>, cudaFuncAttributeNonPortableClusterSizeAllowed, 1);
        cudaFuncSetAttribute(attn_mma_kernel<MODE_KEYS, 1, 1>, cudaFuncAttributeNonPortableClusterSizeAllowed, 1);
#if TIS_HD % 32 == 0
        cudaFuncSetAttribute(attn_mma_kernel<MODE_KEYS, 2, 1, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024);
        cudaFuncSetAttribute(attn_mma_kernel<MODE_KEYS, 1, 1, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024);
        cudaFuncSetAttribute(attn_mma_kernel<MODE_KEYS, 2, 1, true>, cudaFuncAttributeNonPortableClusterSizeAllowed, 1);
        cudaFuncSetAttribute(attn_mma_kernel<MODE_KEYS, 1, 1, true>, cudaFuncAttributeNonPortableClusterSizeAllowed, 1);
#endif
        cudaFuncSetAttribute(attn_decode_kernel<1, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024);
        cudaFuncSetAttribute(attn_decode_kernel<2, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024);
        cudaFuncSetAttribute(attn_decode_kernel<1, false>, cudaFuncAttributeNonPortableClusterSizeAllowed, 1);
        cudaFuncSetAttribute(attn_decode_kernel<2, false>, cudaFuncAttributeNonPortableClusterSizeAllowed, 1);
#if TIS_HD % 32 == 0
        cudaFuncSetAttribute(attn_decode_kernel<1, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024);
        cudaFuncSetAttribute(attn_decode_kernel<2, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 220 * 1024);
        cudaFuncSetAttribute(attn_decode_kernel<1, true>, cudaFuncAttributeNonPortableClusterSizeAllowed, 1);
        cudaFuncSetAttribute(attn_decode_kernel<2, true>, cudaFuncAttributeNonPortableClusterSizeAllowed, 1);
#endif
        cudaGetLastError();
        if (3 * smem_bytes(MODE_ROWS) <= 227 * 1024)
            cudaFuncSetAttribute(attn_mma_kernel<MODE_ROWS, 2, 3>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 (int)(3 * smem_bytes(MODE_ROWS)));
        configured = true;
    }
    {
        // with 2..8 splits the splits of a (tile, kv head) form a thread-block cluster
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = grid;
        cfg.blockDim = dim3(NTHREADS);
        cfg.dynamicSmemBytes = smem;
        cfg.stream = stream;
        cudaLaunchAttribute attrs[3];
        int na = 0;
        if (p.cluster_merge) {
            attrs[na].id = cudaLaunchAttributeClusterDimension;
            attrs[na].val.clusterDim.x = 1;
            attrs[na].val.clusterDim.y = 1;
            attrs[na].val.clusterDim.z = num_splits;
            ++na;
        }
        if (tis_pdl_enabled()) {
            attrs[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
            attrs[na].val.programmaticStreamSerializationAllowed = 1;
            ++na;
        }
        cfg.attrs = attrs;
        cfg.numAttrs = na;
        // a long prompt from (near) its start: three key groups per CTA, heaviest tiles first
        const bool groups3 = mode == MODE_ROWS && num_splits == 1 && keys_per_split >= 512 &&
                             3 * smem_bytes(MODE_ROWS) <= 227 * 1024;
        if (groups3) {
            cfg.blockDim = dim3(3 * NTHREADS);
            cfg.dynamicSmemBytes = 3 * smem_bytes(MODE_ROWS);
            cudaLaunchKernelEx(&cfg, attn_mma_kernel<MODE_ROWS, 2, 3>, p);
        } else if (mode == MODE_ROWS) cudaLaunchKernelEx(&cfg, attn_mma_kernel<MODE_ROWS, 2, 1>, p);
        else if (warp_specialised) {
            cfg.blockDim = dim3(DEC_THREADS);
            if (!p.cluster_merge) {            // one split: a cluster of one, the same merge
                attrs[na].id = cudaLaunchAttributeClusterDimension;
                attrs[na].val.clusterDim.x = 1;
                attrs[na].val.clusterDim.y = 1;
                attrs[na].val.clusterDim.z = 1;
                cfg.numAttrs = ++na;
            }
            const bool nr1 = max_tile_rows > 0 && max_tile_rows * G <= 8;
#if TIS_HD % 32 == 0
            if (fused && nr1) cudaLaunchKernelEx(&cfg, attn_decode_kernel<1, true>, p);
            else if (fused) cudaLaunchKernelEx(&cfg, attn_decode_kernel<2, true>, p);
            else
#endif
            if (nr1) cudaLaunchKernelEx(&cfg, attn_decode_kernel<1, false>, p);
            else cudaLaunchKernelEx(&cfg, attn_decode_kernel<2, false>, p);
        }
#if TIS_HD % 32 == 0
        else if (fused && G <= 8) cudaLaunchKernelEx(&cfg, attn_mma_kernel<MODE_KEYS, 1, 1, true>, p);
        else if (fused) cudaLaunchKernelEx(&cfg, attn_mma_kernel<MODE_KEYS, 2, 1, true>, p);
#endif
        else if (max_tile_rows > 0 && max_tile_rows * G <= 8) cudaLaunchKernelEx(&cfg, attn_mma_kernel<MODE_KEYS, 1, 1>, p);
        else cudaLaunchKernelEx(&cfg, attn_mma_kernel<MODE_KEYS, 2, 1>, p);
    }
    int st = tis_check_launch("attn_mma");
    if (st != TIS_OK) return st;
    if (num_splits > 1 && !p.cluster_merge) {
        dim3 mg(H, num_tiles);
        attn_merge_kernel<<<mg, HD < 128 ? (HD < 32 ? 32 : HD) : 128, 0, stream>>>(p.part_o, p.part_lse, (bf16*)out, out_stride,
                                                                                  tile_row0, tile_rows, H, num_splits);
        st = tis_check_launch("attn_merge");
    }
    return st;
}

TIS_API int tis_attn_mma(int mode, const void* q, int q_stride, void* out, int out_stride, const void* plane,
                         const int* block_table, int bt_stride, int num_pages, const int* positions,
                         const int* row_slot, const int* tile_row0, const int* tile_rows, int num_tiles,
                         int max_tile_rows, int n_rows, int H, int KVH, int page_size, int window, float scale,
                         int keys_per_split, int num_splits, float* scratch, int* fault, cudaStream_t stream) {
    return attn_launch(mode, q, q_stride, out, out_stride, plane, block_table, bt_stride, num_pages, positions, row_slot,
                       tile_row0, tile_rows, num_tiles, max_tile_rows, n_rows, H, KVH, page_size, window, scale,
                       keys_per_split, num_splits, scratch, fault, stream, nullptr, nullptr, 0);
}

// Decode rows (tiles of one row, keys mode) whose rotary encoding and cache write this kernel does itself:
// `qkv` rows are [H*HD queries | KVH*HD keys | KVH*HD values] as the projection left them (only the queries
// when write_kv is 0: another entry of the schedule fills the plane); cos/sin [positions][HD/2] float32,
// half-split pairs, the whole head rotated.  At most eight key splits (they merge inside a cluster).
TIS_API int tis_attn_decode_rope(const void* qkv, int q_stride, void* out, int out_stride, void* plane,
                                 const int* block_table, int bt_stride, int num_pages, const int* positions,
                                 const int* row_slot, const int* tile_row0, const int* tile_rows, int num_tiles,
                                 int n_rows, int H, int KVH, int page_size, int window, float scale,
                                 int keys_per_split, int num_splits, const float* rope_cos, const float* rope_sin,
                                 int write_kv, int* fault, cudaStream_t stream) {
    if (rope_cos == nullptr || rope_sin == nullptr) {
        tis_set_error("attn_decode_rope: no rotary tables");
        return TIS_BAD_SIZE;
    }
    if (num_splits > MAX_CLUSTER) {
        tis_set_error("attn_decode_rope: %d key splits; at most 16", num_splits);
        return TIS_BAD_SIZE;
    }
    return attn_launch(MODE_KEYS, qkv, q_stride, out, out_stride, plane, block_table, bt_stride, num_pages, positions,
                       row_slot, tile_row0, tile_rows, num_tiles, 1, n_rows, H, KVH, page_size, window, scale,
                       keys_per_split, num_splits, nullptr, fault, stream, rope_cos, rope_sin, write_kv);
}


// ----------------------------------------------------------------------------------
// The same decode attention for callers that must not allocate (attention_noalloc.h):
// the partial results of the key splits go to a fixed array inside this library.
// ----------------------------------------------------------------------------------
#include "attention_noalloc.h"

static __device__ __align__(256) float g_noalloc_scratch[TIS_NOALLOC_SCRATCH_FLOATS];

// In host code `g_noalloc_scratch` is only a handle for the runtime, not an address a
// kernel may use; the device address is looked up once per device and kept here.
static float* g_noalloc_ptr[64] = {nullptr};

TIS_API int tis_attn_decode_noalloc(const void* q, int q_stride, void* out, int out_stride, const void* plane,
                                    const int* block_table, int bt_stride, int num_pages, const int* positions,
                                    const int* row_slot, const int* tile_row0, const int* tile_rows, int num_tiles,
                                    int n_rows, int H, int KVH, int page_size, int window, float scale,
                                    int keys_per_split, int num_splits, int* fault, cudaStream_t stream) {
    if (n_rows <= 0 || H <= 0 || num_splits <= 0) {
        tis_set_error("attn_decode_noalloc: %d rows, %d heads, %d splits", n_rows, H, num_splits);
        return TIS_BAD_SIZE;
    }
    const size_t need = (size_t)n_rows * H * num_splits * (HD + 1);
    if (need > (size_t)TIS_NOALLOC_SCRATCH_FLOATS) {
        tis_set_error("attn_decode_noalloc: %d rows x %d heads x %d splits need %zu floats of scratch; the built-in "
                      "array holds %u (use fewer splits or rows, or tis_attn_mma with scratch of your own)",
                      n_rows, H, num_splits, need, (unsigned)TIS_NOALLOC_SCRATCH_FLOATS);
        return TIS_BAD_SIZE;
    }
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess || dev < 0 || dev >= 64) {
        tis_set_error("attn_decode_noalloc: cudaGetDevice: %s (device %d)", cudaGetErrorString(e), dev);
        return TIS_CUDA_ERROR;
    }
    if (g_noalloc_ptr[dev] == nullptr) {
        // set-up, once per device, with that device current
        float* ptr = nullptr;
        e = cudaGetSymbolAddress((void**)&ptr, g_noalloc_scratch);
        if (e != cudaSuccess || ptr == nullptr) {
            tis_set_error("attn_decode_noalloc: cudaGetSymbolAddress: %s", cudaGetErrorString(e));
            return TIS_CUDA_ERROR;
        }
        g_noalloc_ptr[dev] = ptr;
    }
    // one split needs no scratch at all; tis_attn_mma ignores the pointer then
    return tis_attn_mma(MODE_KEYS, q, q_stride, out, out_stride, plane, block_table, bt_stride, num_pages, positions,
                        row_slot, tile_row0, tile_rows, num_tiles, 0, n_rows, H, KVH, page_size, window, scale,
                        keys_per_split, num_splits, g_noalloc_ptr[dev], fault, stream);
}
