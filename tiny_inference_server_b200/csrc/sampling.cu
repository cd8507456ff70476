// Sampling from rows of 32-bit logits, in the order of the upstream sampler
// (server.py:22-50): repetition penalty over the tokens seen so far, division
// by the temperature, top-k, top-p, softmax, one draw.  Greedy rows (temperature 0 or
// top_k 1) take the arg-max of the penalised logits, lowest index on ties.
//
// A row belongs to a cluster of up to eight CTAs (fewer when there are many rows).  The
// first pass, the maximum and its lowest index, is shared out over the cluster in
// interleaved runs of 1024 entries; every CTA writes its (maximum, index) into the first
// CTA's shared memory, and after one cluster barrier the first CTA holds the row's.  A
// greedy row is done then; for the others the first CTA goes on alone.
//
// No sort is made.  The k-th largest value, and the value at which the descending
// cumulative probability first passes p, are found by radix selection over the ordered
// bit pattern of the floats: four passes of 8 bits with a histogram of counts (top-k)
// or of probability mass (top-p) in shared memory.  All entries equal to a threshold
// are kept; upstream's sort leaves the order of equal values open as well.
//
// The draw is by inverse CDF in index order with one Philox4x32-10 number per row,
// keyed by (seed, counter): the same seed, counter and logits give the same token.
#include "cluster_reduce.cuh"

#define SAMPLE_THREADS 1024
#define SAMPLE_MAX_CLUSTER 8

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

__global__ void __launch_bounds__(SAMPLE_THREADS)
sample_rows_kernel(const float* __restrict__ logits, int V, const float* __restrict__ temps,
                   const int* __restrict__ top_ks, const float* __restrict__ top_ps,
                   const float* __restrict__ penalties, const int* __restrict__ slots,
                   uint32_t* __restrict__ seen_bitmap, int bitmap_words,
                   const unsigned long long* __restrict__ seeds, const unsigned long long* __restrict__ counters,
                   int* __restrict__ out_tokens, float* __restrict__ probs_out) {
    __shared__ float red[33];
    __shared__ float hist_f[256];
    __shared__ unsigned int hist_u[256];
    __shared__ float warp_part[32];
    __shared__ unsigned int sh_u[2];
    __shared__ float sh_f[2];
    __shared__ int sh_tok;
    __shared__ float part_max[SAMPLE_MAX_CLUSTER];
    __shared__ int part_tok[SAMPLE_MAX_CLUSTER];

    unsigned ranks, rank;
    asm volatile("mov.u32 %0, %%cluster_nctarank;\n" : "=r"(ranks));
    asm volatile("mov.u32 %0, %%cluster_ctarank;\n" : "=r"(rank));
    const int r = blockIdx.x / ranks, tid = threadIdx.x;
    if (ranks > 1) cluster_reduce::cluster_arrive();      // waited for before the first write to another CTA
    const float temp = temps[r];
    const int top_k = top_ks[r];
    const float top_p = top_ps[r];
    const int slot = slots != nullptr ? slots[r] : -1;
    const float pen = penalties[r];
    uint32_t* seen_row = (slot >= 0 && seen_bitmap != nullptr) ? seen_bitmap + (size_t)slot * bitmap_words : nullptr;
    const bool greedy = !(temp > 0.f) || top_k == 1;

    RowView row;
    row.logits = logits + (size_t)r * V;
    row.seen = (pen != 1.0f) ? seen_row : nullptr;
    row.penalty = pen;
    row.inv_temp = greedy ? 1.f : 1.f / temp;

    // ---- maximum and its lowest index: this CTA's runs of the row, then over the cluster
    float best = -INFINITY;
    int best_i = 0x7fffffff;
    for (int i = (int)rank * SAMPLE_THREADS + tid; i < V; i += SAMPLE_THREADS * (int)ranks) {
        const float x = row.at(i);
        if (x > best || (x == best && i < best_i)) { best = x; best_i = i; }
    }
    float M = block_max(best, red);
    {
        int cand = (best == M) ? best_i : 0x7fffffff;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) cand = min(cand, __shfl_xor_sync(0xffffffffu, cand, o));
        if (tid == 0) sh_tok = 0x7fffffff;
        __syncthreads();
        if ((tid & 31) == 0) atomicMin(&sh_tok, cand);
        __syncthreads();
    }
    if (ranks > 1) {
        cluster_reduce::cluster_wait();           // every CTA of the cluster has started
        if (tid == 0) {
            const unsigned at_max = cluster_reduce::map_to_rank(cluster_reduce::shared_addr(&part_max[rank]), 0u);
            const unsigned at_tok = cluster_reduce::map_to_rank(cluster_reduce::shared_addr(&part_tok[rank]), 0u);
            asm volatile("st.shared::cluster.f32 [%0], %1;\n" ::"r"(at_max), "f"(M) : "memory");
            asm volatile("st.shared::cluster.s32 [%0], %1;\n" ::"r"(at_tok), "r"(sh_tok) : "memory");
        }
        cluster_reduce::cluster_arrive();         // release: the two stores above
        cluster_reduce::cluster_wait();
        if (rank != 0) return;                    // nothing reads the memory of these CTAs
        float m_all = part_max[0];
        for (unsigned c = 1; c < ranks; ++c) m_all = fmaxf(m_all, part_max[c]);
        int tok_all = 0x7fffffff;
        for (unsigned c = 0; c < ranks; ++c)
            if (part_max[c] == m_all) tok_all = min(tok_all, part_tok[c]);
        M = m_all;
        if (tid == 0) sh_tok = tok_all;
        __syncthreads();
    }
    if (greedy) {
        const int tok = sh_tok;
        if (probs_out != nullptr)
            for (int i = tid; i < V; i += SAMPLE_THREADS) probs_out[(size_t)r * V + i] = (i == tok) ? 1.f : 0.f;
        if (tid == 0) {
            out_tokens[r] = tok;
            if (seen_row != nullptr) atomicOr(&seen_row[tok >> 5], 1u << (tok & 31));
        }
        return;
    }

    // ---- top-k: key of the k-th largest value
    uint32_t thr_key = 0u;                    // keep entries with key >= thr_key
    if (top_k > 0 && top_k < V) {
        uint32_t prefix = 0u, mask = 0u;
        unsigned int want = (unsigned int)top_k;      // rank still to descend, among entries matching the prefix
        for (int shift = 24; shift >= 0; shift -= 8) {
            if (tid < 256) hist_u[tid] = 0u;
            __syncthreads();
            for (int i = tid; i < V; i += SAMPLE_THREADS) {
                const uint32_t k = float_key(row.at(i));
                if ((k & mask) == prefix) atomicAdd(&hist_u[(k >> shift) & 255u], 1u);
            }
            __syncthreads();
            if (tid == 0) {
                unsigned int above = 0u;
                int b = 255;
                for (; b > 0; --b) {
                    if (above + hist_u[b] >= want) break;
                    above += hist_u[b];
                }
                sh_u[0] = (unsigned int)b;
                sh_u[1] = want - above;
            }
            __syncthreads();
            prefix |= (sh_u[0] << shift);
            mask |= (255u << shift);
            want = sh_u[1];
            __syncthreads();
        }
        thr_key = prefix;
    }

    // ---- top-p: among the entries kept so far, the value at which the descending
    // cumulative probability first passes p (that entry is kept, server.py:44-48)
    if (top_p > 0.f && top_p < 1.f) {
        float z = 0.f;
        for (int i = tid; i < V; i += SAMPLE_THREADS) {
            const float x = row.at(i);
            if (float_key(x) >= thr_key) z += expf(x - M);
        }
        z = block_sum(z, red);
        const float target = top_p * z;
        uint32_t prefix = 0u, mask = 0u;
        float above_total = 0.f;               // mass of entries strictly above the prefix's range
        for (int shift = 24; shift >= 0; shift -= 8) {
            if (tid < 256) hist_f[tid] = 0.f;
            __syncthreads();
            for (int i = tid; i < V; i += SAMPLE_THREADS) {
                const float x = row.at(i);
                const uint32_t k = float_key(x);
                if (k >= thr_key && (k & mask) == prefix) atomicAdd(&hist_f[(k >> shift) & 255u], expf(x - M));
            }
            __syncthreads();
            if (tid == 0) {
                float above = above_total;
                int b = 255;
                for (; b > 0; --b) {
                    if (above + hist_f[b] > target) break;
                    above += hist_f[b];
                }
                sh_u[0] = (unsigned int)b;
                sh_f[0] = above;
            }
            __syncthreads();
            prefix |= (sh_u[0] << shift);
            mask |= (255u << shift);
            above_total = sh_f[0];
            __syncthreads();
        }
        if (prefix > thr_key) thr_key = prefix;
    }

    // ---- normaliser of the kept entries
    float zf = 0.f;
    for (int i = tid; i < V; i += SAMPLE_THREADS) {
        const float x = row.at(i);
        if (float_key(x) >= thr_key) zf += expf(x - M);
    }
    zf = block_sum(zf, red);
    if (probs_out != nullptr) {
        for (int i = tid; i < V; i += SAMPLE_THREADS) {
            const float x = row.at(i);
            probs_out[(size_t)r * V + i] = (float_key(x) >= thr_key) ? expf(x - M) / zf : 0.f;
        }
    }

    // ---- one draw by inverse CDF in index order
    const uint32_t bits = Philox::draw(seeds[r], counters[r]);
    const float u = (float)(bits >> 8) * (1.0f / 16777216.0f);
    const float target = u * zf;
    if (tid == 0) sh_tok = 0x7fffffff;
    __syncthreads();
    float running = 0.f;                       // mass of all entries before this round (same in every thread)
    const int lane = tid & 31, wid = tid >> 5;
    for (int base = 0; base < V; base += SAMPLE_THREADS) {
        const int i = base + tid;
        float mine = 0.f;
        if (i < V) {
            const float x = row.at(i);
            if (float_key(x) >= thr_key) mine = expf(x - M);
        }
        // inclusive scan over the CTA
        float inc = mine;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const float t = __shfl_up_sync(0xffffffffu, inc, o);
            if (lane >= o) inc += t;
        }
        if (lane == 31) warp_part[wid] = inc;
        __syncthreads();
        const float wsum = warp_part[lane];
        float winc = wsum;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const float t = __shfl_up_sync(0xffffffffu, winc, o);
            if (lane >= o) winc += t;
        }
        const float before_warp = __shfl_sync(0xffffffffu, winc - wsum, wid);
        const float total = __shfl_sync(0xffffffffu, winc, 31);
        // the first kept entry whose inclusive cumulative mass passes the target
        if (mine > 0.f && running + before_warp + inc > target) atomicMin(&sh_tok, i);
        running += total;
        __syncthreads();
        if (sh_tok != 0x7fffffff) break;
    }
    if (sh_tok == 0x7fffffff) {
        // rounding left the target at or beyond the total: take the last kept entry
        __syncthreads();
        if (tid == 0) sh_tok = -1;
        __syncthreads();
        int last = -1;
        for (int i = tid; i < V; i += SAMPLE_THREADS)
            if (float_key(row.at(i)) >= thr_key) last = max(last, i);
        atomicMax(&sh_tok, last);
        __syncthreads();
    }
    if (tid == 0) {
        const int tok = sh_tok;
        out_tokens[r] = tok;
        if (seen_row != nullptr) atomicOr(&seen_row[tok >> 5], 1u << (tok & 31));
    }
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
    // CTAs a row: as many as leave every CTA a run of its own and all clusters resident at once
    int ranks = SAMPLE_MAX_CLUSTER;
    while (ranks > 1 && ((long long)k * ranks > 148 || (long long)(ranks - 1) * SAMPLE_THREADS >= V)) ranks >>= 1;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)(k * ranks), 1, 1);
    cfg.blockDim = dim3(SAMPLE_THREADS, 1, 1);
    cfg.stream = stream;
    cudaLaunchAttribute attrs[1];
    attrs[0].id = cudaLaunchAttributeClusterDimension;
    attrs[0].val.clusterDim.x = (unsigned)ranks;
    attrs[0].val.clusterDim.y = 1;
    attrs[0].val.clusterDim.z = 1;
    cfg.attrs = attrs;
    cfg.numAttrs = 1;
    const cudaError_t e = cudaLaunchKernelEx(&cfg, sample_rows_kernel, logits, V, temps, top_ks, top_ps, penalties, slots,
                                             seen_bitmap, bitmap_words, seeds, counters, out_tokens, probs_out);
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
