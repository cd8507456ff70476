// Attention of step rows over the paged cache, on CUDA cores, everything in 32-bit
// arithmetic.  This is the kernel of the float32 path (keys, values and probabilities
// stay float) and works for bfloat16 pages too.
//
// One CTA per (query head, row).  The row at position p of the request in slot s reads
// keys lo..p of the plane through the request's block table, lo = 0 or p-window+1.
// Keys are taken 128 at a time: every thread scores one key, the CTA agrees on the new
// running maximum, then the threads split the head dimension and add the 128 weighted
// value rows (online softmax, as paged_attention_kernels.py:88-111 upstream, in base e).
// Cache rows are stored with their 16-byte chunks permuted by the position (common.cuh).
#include "common.cuh"

#define SIMT_KEYS 128

// q . k for one cache row of position `pos`: the row's 16-byte chunks are permuted by the
// position (cache_chunk in common.cuh).
template <typename T>
__device__ __forceinline__ float dot_row(const float* __restrict__ q, const T* __restrict__ k, int hd, int pos) {
    constexpr int N = Vec16<T>::N;
    const int nch = hd / N;
    float acc = 0.f;
    for (int c = 0; c < nch; ++c) {
        float v[N];
        Vec16<T>::load(k + cache_chunk(c, pos, nch) * N, v);
        const float* qq = q + c * N;
#pragma unroll
        for (int j = 0; j < N; ++j) acc += qq[j] * v[j];
    }
    return acc;
}

template <typename T>
__global__ void __launch_bounds__(SIMT_KEYS)
paged_attention_simt_kernel(const T* __restrict__ q, int q_stride, T* __restrict__ out, int out_stride,
                            const T* __restrict__ plane, const int* __restrict__ block_table, int bt_stride,
                            int num_pages, const int* __restrict__ positions, const int* __restrict__ row_slot,
                            int H, int KVH, int hd, int page_size, int window, float scale,
                            int* __restrict__ fault) {
    extern __shared__ float smem[];
    float* qs = smem;                      // hd
    float* ps = smem + hd;                 // SIMT_KEYS
    long long* voff = reinterpret_cast<long long*>(ps + SIMT_KEYS);   // SIMT_KEYS (hd is a multiple of 16: aligned)
    __shared__ float red[33];

    const int h = blockIdx.x, r = blockIdx.y, tid = threadIdx.x;
    T* o = out + (size_t)r * out_stride + (size_t)h * hd;
    const int slot = row_slot[r];
    if (slot < 0) {
        for (int i = tid; i < hd; i += SIMT_KEYS) o[i] = from_f32<T>(0.f);
        return;
    }
    const int pos = positions[r];
    const int hi = pos + 1;
    const int lo = (window > 0 && hi > window) ? hi - window : 0;
    const int kvh = h / (H / KVH);
    const T* qrow = q + (size_t)r * q_stride + (size_t)h * hd;
    for (int i = tid; i < hd; i += SIMT_KEYS) qs[i] = to_f32(qrow[i]);
    __syncthreads();

    const int* bt = block_table + (size_t)slot * bt_stride;
    const size_t page_elems = (size_t)2 * KVH * page_size * hd;
    const size_t v_shift = (size_t)KVH * page_size * hd;

    float acc0 = 0.f, acc1 = 0.f;          // dims tid and tid + 128 of the output (hd <= 256)
    float m = -INFINITY, l = 0.f;
    for (int t0 = lo; t0 < hi; t0 += SIMT_KEYS) {
        const int j = t0 + tid;
        float s = -INFINITY;
        long long ko = -1;
        if (j < hi) {
            const int page = bt[j / page_size];
            if (page < 0 || page >= num_pages) {
                atomicExch(fault, 2);
            } else {
                ko = (long long)((size_t)page * page_elems + ((size_t)kvh * page_size + (j % page_size)) * hd);
                s = dot_row<T>(qs, plane + ko, hd, j) * scale;
            }
        }
        voff[tid] = ko < 0 ? -1 : ko + (long long)v_shift;
        const float m_new = fmaxf(m, block_max(s, red));
        const float p = (s == -INFINITY) ? 0.f : expf(s - m_new);
        ps[tid] = p;
        const float alpha = (m == -INFINITY) ? 0.f : expf(m - m_new);
        l = l * alpha + block_sum(p, red);     // barriers inside also publish ps and voff
        m = m_new;
        acc0 *= alpha;
        acc1 *= alpha;
        const int cnt = min(SIMT_KEYS, hi - t0);
        constexpr int N = Vec16<T>::N;
        const int nch = hd / N;
        if (tid < hd) {
            const int c = tid / N, e = tid % N;
            for (int jj = 0; jj < cnt; ++jj) {
                const long long vo = voff[jj];
                if (vo >= 0) acc0 += ps[jj] * to_f32(plane[vo + cache_chunk(c, t0 + jj, nch) * N + e]);
            }
        }
        if (tid + SIMT_KEYS < hd) {
            const int c = (tid + SIMT_KEYS) / N, e = (tid + SIMT_KEYS) % N;
            for (int jj = 0; jj < cnt; ++jj) {
                const long long vo = voff[jj];
                if (vo >= 0) acc1 += ps[jj] * to_f32(plane[vo + cache_chunk(c, t0 + jj, nch) * N + e]);
            }
        }
        __syncthreads();                       // ps, voff are rewritten by the next tile
    }
    const float inv = l > 0.f ? 1.f / l : 0.f;
    if (tid < hd) o[tid] = from_f32<T>(acc0 * inv);
    if (tid + SIMT_KEYS < hd) o[tid + SIMT_KEYS] = from_f32<T>(acc1 * inv);
}

TIS_API int tis_paged_attention_simt(int dtype, const void* q, int q_stride, void* out, int out_stride,
                                     const void* plane, const int* block_table, int bt_stride, int num_pages,
                                     const int* positions, const int* row_slot, int n, int H, int KVH, int hd,
                                     int page_size, int window, float scale, int* fault, cudaStream_t stream) {
    if (n <= 0) return TIS_OK;
    if (hd % 16 || hd <= 0 || hd > 256) {
        tis_set_error("paged_attention: head size %d is not a multiple of 16 in 16..256", hd);
        return TIS_BAD_SIZE;
    }
    if (KVH <= 0 || H % KVH) {
        tis_set_error("paged_attention: %d query heads are not a multiple of %d kv heads", H, KVH);
        return TIS_BAD_SIZE;
    }
    if (n > 65535) {
        tis_set_error("paged_attention: %d rows in one step exceed 65535", n);
        return TIS_BAD_SIZE;
    }
    const size_t smem = (size_t)(hd + SIMT_KEYS) * sizeof(float) + SIMT_KEYS * sizeof(long long);
    dim3 grid(H, n);
    TIS_DISPATCH_DTYPE(dtype, T,
        paged_attention_simt_kernel<T><<<grid, SIMT_KEYS, smem, stream>>>(
            (const T*)q, q_stride, (T*)out, out_stride, (const T*)plane, block_table, bt_stride, num_pages,
            positions, row_slot, H, KVH, hd, page_size, window, scale, fault));
    return tis_check_launch("paged_attention_simt");
}
