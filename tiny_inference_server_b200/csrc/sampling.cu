// Sampling from rows of 32-bit logits, in the order of the upstream sampler
// (server.py:22-50): repetition penalty over the tokens seen so far, division
// by the temperature, top-k, top-p, softmax, one draw.  Greedy rows (temperature 0 or
// top_k 1) take the arg-max of the penalised logits, lowest index on ties.
//
// A row belongs to a cluster of up to eight CTAs (fewer when there are many rows); rank c
// holds entries [c S, (c+1) S) of the row.  The first pass reads the logits once, applies
// penalty and temperature, keeps the result in shared memory (every later pass reads it
// there) and finds the maximum and its lowest index.  What the ranks have to agree on goes
// the same way every time: each rank writes its part (a maximum, a sum, a histogram) into
// its own place in EVERY rank's shared memory, one cluster barrier, and each rank adds up
// the parts in rank order, so that all ranks hold the same bits and take the same branches.
// The places are double-buffered: a rank may run one exchange ahead of the slowest.
//
// No sort is made.  The k-th largest value, and the value at which the descending
// cumulative probability first passes p, are found by radix selection over the ordered
// bit pattern of the floats: four passes of 8 bits with a histogram of counts (top-k)
// or of probability mass (top-p).  The high bits of most floats of a row are the same, so
// most entries of the first pass meet in a few bins: every lane has a copy of the histogram
// of its own (bin b of lane l in bank l: the atomic additions of a warp never collide), and
// a thread adds up runs of entries of the same bin before it touches it.  The copies are
// then added up, and a warp finds the bin with a suffix sum.  All entries equal to a threshold
// are kept; upstream's sort leaves the order of equal values open as well.
//
// The draw is by inverse CDF in index order with one Philox4x32-10 number per row,
// keyed by (seed, counter): the same seed, counter and logits give the same token.
// Threads add up the kept mass of contiguous runs of entries, one scan over the CTA and
// one exchange give every run its place in the CDF, and the rank whose range holds the
// drawn number finds the entry.
//
// A row whose share per rank is larger than the shared memory (a vocabulary of more than
// about 360,000 entries) is read from the logits in every pass instead.
#include "cluster_reduce.cuh"

#define SAMPLE_THREADS 1024
#define SAMPLE_MAX_CLUSTER 8
#define SAMPLE_NONE 0x7fffffff
#define SAMPLE_LANE_HIST (256 * 32)

struct Philox {
    static __device__ __forceinline__ void round(uint32_t (&c)[4], uint32_t k0, uint32_t k1) {
        const uint32_t M0 = 0xD2511F53u, M1 = 0xCD9E8D57u;
        const uint32_t hi0 = __umulhi(M0, c[0]), lo0 = M0 * c[0];
        const uint32_t hi1 = __umulhi(M1, c[2]), lo1 = M1 * c[2];
        const uint32_t n0 = hi1 ^ c[1] ^ k0, n1 = lo1, n2 = hi0 ^ c[3] ^ k1, n3 = lo0;
        c[0] = n0; c[1] = n1; c[2] = n2; c[3] = n3;
    }
    static __device__ __forceinline__ uint32_t draw(uint64_t seed, uint64_t counter) {
        uint32_t c[4] = {(uint32_t)counter, (uint32_t)(counter >> 32), 0u, 0u};
        uint32_t k0 = (uint32_t)seed, k1 = (uint32_t)(seed >> 32);
#pragma unroll
        for (int i = 0; i < 10; ++i) {
            round(c, k0, k1);
            k0 += 0x9E3779B9u;
            k1 += 0xBB67AE85u;
        }
        return c[0];
    }
};

// order-preserving map float -> uint32 (larger float, larger key)
__device__ __forceinline__ uint32_t float_key(float x) {
    const uint32_t b = __float_as_uint(x);
    return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}
__device__ __forceinline__ float key_float(uint32_t k) {
    const uint32_t b = (k & 0x80000000u) ? (k & 0x7fffffffu) : ~k;
    return __uint_as_float(b);
}

struct RowView {
    const float* logits;
    const uint32_t* seen;    // bitmap of the tokens of the request so far, or null
    float penalty;
    float inv_temp;
    __device__ __forceinline__ float at(int i) const {
        float x = logits[i];
        if (seen != nullptr && ((seen[i >> 5] >> (i & 31)) & 1u)) x = x > 0.f ? x / penalty : x * penalty;
        return x * inv_temp;
    }
};


namespace {

struct Shared {
    float red[33];
    unsigned int slots[2][SAMPLE_MAX_CLUSTER][256];          // every rank's histogram: counts, or masses as float bits
    unsigned int merged[256];                                // the histogram of the row
    unsigned int parts[2][SAMPLE_MAX_CLUSTER][2];            // every rank's part of a small exchange
    float warp_part[32];
    unsigned int picked[2];                                  // bin, and the rank left to descend
    float picked_above;
    int tok;
    int last;
};

__device__ __forceinline__ void cluster_sync() {
    cluster_reduce::cluster_arrive();
    cluster_reduce::cluster_wait();
}
__device__ __forceinline__ void store_at_rank(const void* local, unsigned rank, unsigned v) {
    asm volatile("st.shared::cluster.u32 [%0], %1;\n"
                 ::"r"(cluster_reduce::map_to_rank(cluster_reduce::shared_addr(local), rank)), "r"(v) : "memory");
}

// The row's token: written, and marked in the row of seen tokens.  A row of logits that are no numbers has no
// maximum and keeps nothing: it gets token 0 rather than a write outside the bitmap.
__device__ __forceinline__ void write_token(int tok, int V, int* out, uint32_t* seen_row) {
    if (tok < 0 || tok >= V) tok = 0;
    *out = tok;
    if (seen_row != nullptr) atomicOr(&seen_row[tok >> 5], 1u << (tok & 31));
}

// The entries of a row that this CTA holds.
struct Slice {
    RowView row;
    const float* staged;     // shared memory copy of at(base + j), or null
    int base, n;
    __device__ __forceinline__ float at(int j) const { return staged != nullptr ? staged[j] : row.at(base + j); }
};

// Two words of every rank, the same in every rank afterwards: parts[buf][c] = what rank c gave.
__device__ __forceinline__ void exchange(Shared& sh, int& buf, unsigned ranks, unsigned rank, unsigned a, unsigned b) {
    buf ^= 1;
    if (threadIdx.x < ranks) {
        store_at_rank(&sh.parts[buf][rank][0], threadIdx.x, a);
        store_at_rank(&sh.parts[buf][rank][1], threadIdx.x, b);
    }
    cluster_sync();
}

// Radix selection over the keys of the entries kept so far (key >= keep_key).  COUNT: the key of the
// want-th largest.  MASS: the key at which the descending sum of exp(x - M) first passes `target`.
template <bool MASS>
__device__ __forceinline__ uint32_t radix_threshold(Shared& sh, unsigned* lane_hist, const Slice& sl, int& hbuf,
                                                    unsigned ranks, unsigned rank, uint32_t keep_key, float M,
                                                    unsigned want, float target) {
    const int tid = threadIdx.x, lane = tid & 31;
    uint32_t prefix = 0u, mask = 0u;
    float above_total = 0.f;                  // MASS: mass of the entries above the prefix's range
    for (int shift = 24; shift >= 0; shift -= 8) {
        for (int i = tid; i < 256 * 32; i += SAMPLE_THREADS) lane_hist[i] = 0u;
        __syncthreads();
        int cur = -1;
        unsigned cnt = 0u;
        float acc = 0.f;
        for (int j = tid; j < sl.n; j += SAMPLE_THREADS) {
            const float x = sl.at(j);
            const uint32_t k = float_key(x);
            if ((k & mask) != prefix || k < keep_key) continue;
            const int b = (int)((k >> shift) & 255u);
            if (b != cur) {
                if (cur >= 0) {
                    if (MASS) atomicAdd(reinterpret_cast<float*>(&lane_hist[cur * 32 + lane]), acc);
                    else atomicAdd(&lane_hist[cur * 32 + lane], cnt);
                }
                cur = b; cnt = 0u; acc = 0.f;
            }
            if (MASS) acc += expf(x - M); else ++cnt;
        }
        if (cur >= 0) {
            if (MASS) atomicAdd(reinterpret_cast<float*>(&lane_hist[cur * 32 + lane]), acc);
            else atomicAdd(&lane_hist[cur * 32 + lane], cnt);
        }
        __syncthreads();
        {   // the 32 copies of a bin into one: four threads a bin, eight copies each, turned so that banks differ
            const int bin = tid >> 2, part = tid & 3;
            unsigned su = 0u;
            float sf = 0.f;
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const unsigned v = lane_hist[bin * 32 + part * 8 + ((i + (lane >> 2)) & 7)];
                if (MASS) sf += __uint_as_float(v); else su += v;
            }
            if (MASS) {
                sf += __shfl_xor_sync(0xffffffffu, sf, 1);
                sf += __shfl_xor_sync(0xffffffffu, sf, 2);
                su = __float_as_uint(sf);
            } else {
                su += __shfl_xor_sync(0xffffffffu, su, 1);
                su += __shfl_xor_sync(0xffffffffu, su, 2);
            }
            if (part == 0)
                for (unsigned c = 0; c < ranks; ++c) store_at_rank(&sh.slots[hbuf ^ 1][rank][bin], c, su);
        }
        hbuf ^= 1;
        cluster_sync();
        if (tid < 256) {                      // the ranks' parts of a bin, added up in rank order
            unsigned mu = 0u;
            float mf = 0.f;
            for (unsigned c = 0; c < ranks; ++c) {
                const unsigned v = sh.slots[hbuf][c][tid];
                if (MASS) mf += __uint_as_float(v); else mu += v;
            }
            sh.merged[tid] = MASS ? __float_as_uint(mf) : mu;
        }
        __syncthreads();
        if (tid < 32) {
            // lane l: bins 8l .. 8l+7; from the top bin down, the first bin at which the sum reaches the goal
            unsigned hu[8], tu = 0u;
            float hf[8], tf = 0.f;
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const unsigned v = sh.merged[8 * lane + j];
                hu[j] = MASS ? 0u : v;
                hf[j] = MASS ? __uint_as_float(v) : 0.f;
                tu += hu[j]; tf += hf[j];
            }
            unsigned su = tu;                 // sums over this lane and the lanes above it
            float sf = tf;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const unsigned u = __shfl_down_sync(0xffffffffu, su, o);
                const float f = __shfl_down_sync(0xffffffffu, sf, o);
                if (lane + o < 32) { su += u; sf += f; }
            }
            unsigned above_u = su - tu;
            float above_f = __shfl_down_sync(0xffffffffu, sf, 1);
            above_f = above_total + (lane == 31 ? 0.f : above_f);
            int found = -1;
#pragma unroll
            for (int j = 7; j >= 0; --j) {
                const int b = 8 * lane + j;
                if (found < 0 && b > 0) {
                    if (MASS ? (above_f + hf[j] > target) : (above_u + hu[j] >= want)) found = b;
                    else { above_u += hu[j]; above_f += hf[j]; }
                }
            }
            // no bin above bin 0 reaches the goal: bin 0, with everything above it (lane 0 has added that up)
            const unsigned has = __ballot_sync(0xffffffffu, found >= 0);
            const int src = has ? 31 - __clz((int)has) : 0;
            const int b_sel = has ? __shfl_sync(0xffffffffu, found, src) : 0;
            const unsigned au = __shfl_sync(0xffffffffu, above_u, src);
            const float af = __shfl_sync(0xffffffffu, above_f, src);
            if (lane == 0) {
                sh.picked[0] = (unsigned)b_sel;
                sh.picked[1] = want - au;
                sh.picked_above = af;
            }
        }
        __syncthreads();
        prefix |= (sh.picked[0] << shift);
        mask |= (255u << shift);
        if (MASS) above_total = sh.picked_above; else want = sh.picked[1];
        // every entry of the bin is wanted: the bin's lowest key is the threshold, whatever the bits below say
        if (!MASS && sh.merged[sh.picked[0]] == want) break;
    }
    return prefix;
}

__global__ void __launch_bounds__(SAMPLE_THREADS)
sample_rows_kernel(const float* __restrict__ logits, int V, int share, int stage,
                   const float* __restrict__ temps, const int* __restrict__ top_ks, const float* __restrict__ top_ps,
                   const float* __restrict__ penalties, const int* __restrict__ slots,
                   uint32_t* __restrict__ seen_bitmap, int bitmap_words,
                   const unsigned long long* __restrict__ seeds, const unsigned long long* __restrict__ counters,
                   int* __restrict__ out_tokens, float* __restrict__ probs_out) {
    extern __shared__ float dynamic_shared[];
    unsigned* lane_hist = reinterpret_cast<unsigned*>(dynamic_shared);    // [256 bins][32 lanes]
    float* staged_row = dynamic_shared + SAMPLE_LANE_HIST;
    __shared__ Shared sh;

    unsigned ranks, rank;
    asm volatile("mov.u32 %0, %%cluster_nctarank;\n" : "=r"(ranks));
    asm volatile("mov.u32 %0, %%cluster_ctarank;\n" : "=r"(rank));
    cluster_reduce::cluster_arrive();             // waited for before the first write to another CTA
    const int r = blockIdx.x / ranks, tid = threadIdx.x, lane = tid & 31, wid = tid >> 5;
    const float temp = temps[r];
    const int top_k = top_ks[r];
    const float top_p = top_ps[r];
    const int slot = slots != nullptr ? slots[r] : -1;
    const float pen = penalties[r];
    uint32_t* seen_row = (slot >= 0 && seen_bitmap != nullptr) ? seen_bitmap + (size_t)slot * bitmap_words : nullptr;
    const bool greedy = !(temp > 0.f) || top_k == 1;

    Slice sl;
    sl.row.logits = logits + (size_t)r * V;
    sl.row.seen = (pen != 1.0f) ? seen_row : nullptr;
    sl.row.penalty = pen;
    sl.row.inv_temp = greedy ? 1.f : 1.f / temp;
    sl.base = (int)rank * share;
    sl.n = max(0, min(share, V - sl.base));
    sl.staged = nullptr;
    int xbuf = 0, hbuf = 0;

    // ---- the row into shared memory; its maximum and the lowest index of that
    float best = -INFINITY;
    int best_i = SAMPLE_NONE;
    for (int j = tid; j < sl.n; j += SAMPLE_THREADS) {
        const float x = sl.row.at(sl.base + j);
        if (stage && !greedy) staged_row[j] = x;
        if (x > best || (x == best && best_i == SAMPLE_NONE)) { best = x; best_i = sl.base + j; }   // j grows: the first of equal values stays
    }
    if (stage) sl.staged = staged_row;
    const float m_own = block_max(best, sh.red);
    {
        int cand = (best == m_own) ? best_i : SAMPLE_NONE;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) cand = min(cand, __shfl_xor_sync(0xffffffffu, cand, o));
        if (tid == 0) sh.tok = SAMPLE_NONE;
        __syncthreads();
        if (lane == 0) atomicMin(&sh.tok, cand);
        __syncthreads();
    }
    cluster_reduce::cluster_wait();               // every CTA of the cluster has started
    exchange(sh, xbuf, ranks, rank, __float_as_uint(m_own), (unsigned)sh.tok);
    float M = -INFINITY;
    int tok_max = SAMPLE_NONE;
    for (unsigned c = 0; c < ranks; ++c) M = fmaxf(M, __uint_as_float(sh.parts[xbuf][c][0]));
    for (unsigned c = 0; c < ranks; ++c)
        if (__uint_as_float(sh.parts[xbuf][c][0]) == M) tok_max = min(tok_max, (int)sh.parts[xbuf][c][1]);

    if (greedy) {
        if (tok_max == SAMPLE_NONE) tok_max = 0;
        if (probs_out != nullptr)
            for (int j = tid; j < sl.n; j += SAMPLE_THREADS)
                probs_out[(size_t)r * V + sl.base + j] = (sl.base + j == tok_max) ? 1.f : 0.f;
        if (rank == 0 && tid == 0) write_token(tok_max, V, out_tokens + r, seen_row);
        return;
    }

    // ---- top-k: key of the k-th largest value
    uint32_t thr_key = 0u;                    // keep entries with key >= thr_key
    if (top_k > 0 && top_k < V)
        thr_key = radix_threshold<false>(sh, lane_hist, sl, hbuf, ranks, rank, 0u, M, (unsigned)top_k, 0.f);

    // ---- top-p: among the entries kept so far, the value at which the descending
    // cumulative probability first passes p (that entry is kept, server.py:44-48)
    if (top_p > 0.f && top_p < 1.f) {
        float z = 0.f;
        for (int j = tid; j < sl.n; j += SAMPLE_THREADS) {
            const float x = sl.at(j);
            if (float_key(x) >= thr_key) z += expf(x - M);
        }
        z = block_sum(z, sh.red);
        exchange(sh, xbuf, ranks, rank, __float_as_uint(z), 0u);
        float z_all = 0.f;
        for (unsigned c = 0; c < ranks; ++c) z_all += __uint_as_float(sh.parts[xbuf][c][0]);
        const uint32_t p_key = radix_threshold<true>(sh, lane_hist, sl, hbuf, ranks, rank, thr_key, M, 0u, top_p * z_all);
        if (p_key > thr_key) thr_key = p_key;
    }

    // ---- the kept mass of this CTA's entries, in runs of `per` entries a thread (odd: no bank conflicts)
    const int per = ((sl.n + SAMPLE_THREADS - 1) / SAMPLE_THREADS) | 1;
    const int lo = min(sl.n, tid * per), hi = min(sl.n, lo + per);
    float mine = 0.f;
    int last = -1;                            // the last kept entry
    for (int j = lo; j < hi; ++j) {
        const float x = sl.at(j);
        if (float_key(x) >= thr_key) { mine += expf(x - M); last = sl.base + j; }
    }
    float inc = mine;                         // inclusive scan over the CTA
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const float t = __shfl_up_sync(0xffffffffu, inc, o);
        if (lane >= o) inc += t;
    }
    if (tid == 0) { sh.tok = SAMPLE_NONE; sh.last = -1; }
    __syncthreads();
    if (lane == 31) sh.warp_part[wid] = inc;
    if (last >= 0) atomicMax(&sh.last, last);
    __syncthreads();
    const float wsum = sh.warp_part[lane];
    float winc = wsum;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const float t = __shfl_up_sync(0xffffffffu, winc, o);
        if (lane >= o) winc += t;
    }
    const float before_warp = __shfl_sync(0xffffffffu, winc - wsum, wid);
    const float own_total = __shfl_sync(0xffffffffu, winc, 31);
    exchange(sh, xbuf, ranks, rank, __float_as_uint(own_total), (unsigned)sh.last);

    // ---- normaliser, and one draw by inverse CDF in index order
    float zf = 0.f;
    for (unsigned c = 0; c < ranks; ++c) zf += __uint_as_float(sh.parts[xbuf][c][0]);
    if (probs_out != nullptr) {
        for (int j = tid; j < sl.n; j += SAMPLE_THREADS) {
            const float x = sl.at(j);
            probs_out[(size_t)r * V + sl.base + j] = (float_key(x) >= thr_key) ? expf(x - M) / zf : 0.f;
        }
        cluster_sync();                       // the row's bit of the drawn token is set below: after every read of the bitmap
    }
    const uint32_t bits = Philox::draw(seeds[r], counters[r]);
    const float u = (float)(bits >> 8) * (1.0f / 16777216.0f);
    const float target = u * zf;
    // the first rank at which the cumulative mass passes the target holds the token; none (rounding left the
    // target at or beyond the total): the last kept entry of the row
    float before = 0.f;
    int owner = -1, last_all = -1;
    for (unsigned c = 0; c < ranks; ++c) {
        const float t = __uint_as_float(sh.parts[xbuf][c][0]);
        last_all = max(last_all, (int)sh.parts[xbuf][c][1]);
        if (owner < 0) {
            if (before + t > target) owner = (int)c; else before += t;
        }
    }
    if (owner < 0) {
        if (rank == 0 && tid == 0) write_token(last_all, V, out_tokens + r, seen_row);
        return;
    }
    if ((int)rank != owner) return;
    float running = before + before_warp + (inc - mine);
    for (int j = lo; j < hi; ++j) {
        const float x = sl.at(j);
        if (float_key(x) >= thr_key) {
            running += expf(x - M);
            if (running > target) { atomicMin(&sh.tok, sl.base + j); break; }
        }
    }
    __syncthreads();
    // rounding inside the CTA left the target beyond its sum: its last kept entry
    if (tid == 0) write_token(sh.tok != SAMPLE_NONE ? sh.tok : sh.last, V, out_tokens + r, seen_row);
}

int stage_limit = -1;        // floats of a row that a CTA may keep in shared memory; -1: what the device allows

}  // namespace

// For tests: the most entries of a row that a CTA keeps in shared memory (0: none, every pass reads the
// logits; -1: what the device allows).
TIS_API int tis_sample_stage_limit(int floats) {
    stage_limit = floats;
    return TIS_OK;
}

TIS_API int tis_sample_rows(const float* logits, int k, int V, const float* temps, const int* top_ks,
                            const float* top_ps, const float* penalties, const int* slots,
                            uint32_t* seen_bitmap, int bitmap_words, const unsigned long long* seeds,
                            const unsigned long long* counters, int* out_tokens, float* probs_out,
                            cudaStream_t stream) {
    if (k <= 0) return TIS_OK;
    if (V <= 0) {
        tis_set_error("sample_rows: vocabulary size %d", V);
        return TIS_BAD_SIZE;
    }
    static int device_floats = -1;
    if (device_floats < 0) {
        cudaFuncAttributes fa;
        cudaError_t e = cudaFuncGetAttributes(&fa, sample_rows_kernel);
        const int most = 227 * 1024 - (e == cudaSuccess ? (int)fa.sharedSizeBytes : 0) - 1024;
        const int room = most - SAMPLE_LANE_HIST * 4;
        if (e == cudaSuccess) e = cudaFuncSetAttribute(sample_rows_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, most);
        if (e != cudaSuccess) {
            tis_set_error("sample_rows: %s", cudaGetErrorString(e));
            return TIS_CUDA_ERROR;
        }
        device_floats = room / 4;
    }
    const int room = stage_limit < 0 ? device_floats : (stage_limit < device_floats ? stage_limit : device_floats);
    // CTAs a row: as many as leave every CTA a run of 1024 entries and all clusters resident at once; more
    // when the row's share would not fit into a CTA's shared memory
    int ranks = SAMPLE_MAX_CLUSTER;
    while (ranks > 1 && ((long long)k * ranks > 148 || V < ranks * SAMPLE_THREADS)) ranks >>= 1;
    while (ranks < SAMPLE_MAX_CLUSTER && (V + ranks - 1) / ranks > room && V >= 2 * ranks) ranks <<= 1;
    const int share = (V + ranks - 1) / ranks;
    const int stage = share <= room ? 1 : 0;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)(k * ranks), 1, 1);
    cfg.blockDim = dim3(SAMPLE_THREADS, 1, 1);
    cfg.dynamicSmemBytes = (SAMPLE_LANE_HIST + (stage ? (size_t)share : 0)) * sizeof(float);
    cfg.stream = stream;
    cudaLaunchAttribute attrs[1];
    attrs[0].id = cudaLaunchAttributeClusterDimension;
    attrs[0].val.clusterDim.x = (unsigned)ranks;
    attrs[0].val.clusterDim.y = 1;
    attrs[0].val.clusterDim.z = 1;
    cfg.attrs = attrs;
    cfg.numAttrs = 1;
    const cudaError_t e = cudaLaunchKernelEx(&cfg, sample_rows_kernel, logits, V, share, stage, temps, top_ks, top_ps,
                                             penalties, slots, seen_bitmap, bitmap_words, seeds, counters, out_tokens,
                                             probs_out);
    if (e != cudaSuccess) {
        tis_set_error("sample_rows: %s", cudaGetErrorString(e));
        return TIS_CUDA_ERROR;
    }
    return tis_check_launch("sample_rows");
}

// Mark tokens (a prompt) in the bitmap row of a request slot.
__global__ void bitmap_set_kernel(uint32_t* __restrict__ row, const int* __restrict__ tokens, int n) {
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) {
        const int t = tokens[i];
        atomicOr(&row[t >> 5], 1u << (t & 31));
    }
}

TIS_API int tis_bitmap_set(uint32_t* bitmap_row, const int* tokens, int n, cudaStream_t stream) {
    if (n <= 0) return TIS_OK;
    int blocks = (n + 255) / 256;
    if (blocks > 64) blocks = 64;
    bitmap_set_kernel<<<blocks, 256, 0, stream>>>(bitmap_row, tokens, n);
    return tis_check_launch("bitmap_set");
}
