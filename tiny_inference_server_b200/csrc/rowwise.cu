// Row-wise kernels: embedding gather, fused residual-add + RMSNorm, rotary position
// encoding fused with the write of keys and values into cache pages, SwiGLU gating,
// and the input of a multi-token-prediction head.
//
// One CTA per row of the step.  A row whose request slot is negative is padding: it
// writes nothing into the cache and its outputs are never read.
#include "common.cuh"
#include <cstdlib>

// ----------------------------------------------------------------------------------
// embedding: residual[r, :] = table[token[r], :]   (the 32-bit residual stream starts here)
// ----------------------------------------------------------------------------------
template <typename T>
__global__ void embed_rows_kernel(const T* __restrict__ table, const int* __restrict__ tokens,
                                  float* __restrict__ out, int d) {
    pdl_launch_dependents();
    pdl_wait();
    const int r = blockIdx.x;
    const T* src = table + (size_t)tokens[r] * d;
    float* dst = out + (size_t)r * d;
    constexpr int N = Vec16<T>::N;
    if (d % N == 0) {
        for (int i = threadIdx.x * N; i < d; i += blockDim.x * N) {
            float v[N];
            Vec16<T>::load(src + i, v);
#pragma unroll
            for (int j = 0; j < N; ++j) dst[i + j] = v[j];
        }
    } else {
        for (int i = threadIdx.x; i < d; i += blockDim.x) dst[i] = to_f32(src[i]);
    }
}

TIS_API int tis_embed_rows(int dtype, const void* table, const int* tokens, float* out, int n, int d,
                           cudaStream_t stream) {
    if (n <= 0) return TIS_OK;
    TIS_DISPATCH_DTYPE(dtype, T,
        tis_launch(embed_rows_kernel<T>, dim3(n), dim3(256), 0, stream, (const T*)table, tokens, out, d));
    return tis_check_launch("embed_rows");
}

// ----------------------------------------------------------------------------------
// residual += delta ; out = residual * sqrt(d) / (||residual||_2 + eps) * scale
// (eps is added to the L2 norm itself: main_models_new.py:38-42 of the upstream project)
// ----------------------------------------------------------------------------------
template <typename T>
__global__ void add_rmsnorm_kernel(float* __restrict__ res, const T* __restrict__ delta,
                                   const float* __restrict__ scale, float eps, T* __restrict__ out, int d) {
    extern __shared__ float row[];
    __shared__ float red[33];
    pdl_launch_dependents();
    pdl_wait();
    const size_t base = (size_t)blockIdx.x * d;
    constexpr int N = Vec16<T>::N;
    const bool vec = (d % N == 0);
    float ss = 0.f;
    if (vec) {
        for (int i = threadIdx.x * N; i < d; i += blockDim.x * N) {
            float v[N];
#pragma unroll
            for (int j = 0; j < N; j += 4) {
                const float4 x = *reinterpret_cast<const float4*>(res + base + i + j);
                v[j] = x.x; v[j + 1] = x.y; v[j + 2] = x.z; v[j + 3] = x.w;
            }
            if (delta != nullptr) {
                float dv[N];
                Vec16<T>::load(delta + base + i, dv);
#pragma unroll
                for (int j = 0; j < N; ++j) v[j] += dv[j];
#pragma unroll
                for (int j = 0; j < N; j += 4)
                    *reinterpret_cast<float4*>(res + base + i + j) = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
            }
#pragma unroll
            for (int j = 0; j < N; ++j) { row[i + j] = v[j]; ss += v[j] * v[j]; }
        }
    } else {
        for (int i = threadIdx.x; i < d; i += blockDim.x) {
            float v = res[base + i];
            if (delta != nullptr) {
                v += to_f32(delta[base + i]);
                res[base + i] = v;
            }
            row[i] = v;
            ss += v * v;
        }
    }
    ss = block_sum(ss, red);
    const float inv = sqrtf((float)d) / (sqrtf(ss) + eps);
    if (out == nullptr) return;
    if (vec) {
        for (int i = threadIdx.x * N; i < d; i += blockDim.x * N) {
            float v[N];
#pragma unroll
            for (int j = 0; j < N; ++j) v[j] = row[i + j] * inv * scale[i + j];
            Vec16<T>::store(out + base + i, v);
        }
    } else {
        for (int i = threadIdx.x; i < d; i += blockDim.x) out[base + i] = from_f32<T>(row[i] * inv * scale[i]);
    }
}

// The same for many rows: a warp per row, the row in registers (CH 16-byte chunks of the output
// type per lane), one pass over memory, no shared memory and no block-wide barrier.
template <typename T, int CH>
__global__ void __launch_bounds__(256)
add_rmsnorm_rows_kernel(float* __restrict__ res, const T* __restrict__ delta, const float* __restrict__ scale,
                        float eps, T* __restrict__ out, int n, int d) {
    pdl_launch_dependents();
    pdl_wait();
    constexpr int N = Vec16<T>::N;
    const int r = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    if (r >= n) return;
    const size_t base = (size_t)r * d;
    float v[CH][N];
    float ss = 0.f;
#pragma unroll
    for (int k = 0; k < CH; ++k) {
        const int i = (lane + 32 * k) * N;
        if (i < d) {
#pragma unroll
            for (int j = 0; j < N; j += 4) {
                const float4 x = *reinterpret_cast<const float4*>(res + base + i + j);
                v[k][j] = x.x; v[k][j + 1] = x.y; v[k][j + 2] = x.z; v[k][j + 3] = x.w;
            }
            if (delta != nullptr) {
                float dv[N];
                Vec16<T>::load(delta + base + i, dv);
#pragma unroll
                for (int j = 0; j < N; ++j) v[k][j] += dv[j];
#pragma unroll
                for (int j = 0; j < N; j += 4)
                    *reinterpret_cast<float4*>(res + base + i + j) = make_float4(v[k][j], v[k][j + 1], v[k][j + 2], v[k][j + 3]);
            }
#pragma unroll
            for (int j = 0; j < N; ++j) ss += v[k][j] * v[k][j];
        }
    }
    if (out == nullptr) return;
    ss = warp_sum(ss);
    const float inv = sqrtf((float)d) / (sqrtf(ss) + eps);
#pragma unroll
    for (int k = 0; k < CH; ++k) {
        const int i = (lane + 32 * k) * N;
        if (i < d) {
            float o[N];
#pragma unroll
            for (int j = 0; j < N; j += 4) {
                const float4 sc = *reinterpret_cast<const float4*>(scale + i + j);
                o[j] = v[k][j] * inv * sc.x; o[j + 1] = v[k][j + 1] * inv * sc.y;
                o[j + 2] = v[k][j + 2] * inv * sc.z; o[j + 3] = v[k][j + 3] * inv * sc.w;
            }
            Vec16<T>::store(out + base + i, o);
        }
    }
}

template <typename T, int CH>
static void launch_add_rmsnorm_rows(float* residual, const T* delta, const float* scale, float eps, T* out, int n,
                                    int d, cudaStream_t stream) {
    const int threads = 128;          // four rows a CTA (measured at 2048 x 1536: 9.0 us; eight rows 10.0 us)
    const int rows = threads / 32;
    tis_launch(add_rmsnorm_rows_kernel<T, CH>, dim3((n + rows - 1) / rows), dim3(threads), 0, stream, residual, delta, scale,
               eps, out, n, d);
}

TIS_API int tis_add_rmsnorm(int dtype, float* residual, const void* delta, const float* scale, float eps,
                            void* out, int n, int d, cudaStream_t stream) {
    if (n <= 0) return TIS_OK;
    if ((size_t)d * sizeof(float) > 96 * 1024) {
        tis_set_error("add_rmsnorm: width %d too large (one row must fit 96 KB of shared memory)", d);
        return TIS_BAD_SIZE;
    }
    // many rows (enough for eight a CTA to fill the GPU) of a width that a warp can keep in registers:
    // the warp-per-row kernel
    if (n >= 1024) {
        const int per_lane = dtype == TIS_BF16 ? 8 : 4;
        const int chunks = (d + 32 * per_lane - 1) / (32 * per_lane);
        if (d % per_lane == 0 && chunks <= 8) {
            TIS_DISPATCH_DTYPE(dtype, T, {
                if (chunks <= 2) launch_add_rmsnorm_rows<T, 2>(residual, (const T*)delta, scale, eps, (T*)out, n, d, stream);
                else if (chunks <= 4) launch_add_rmsnorm_rows<T, 4>(residual, (const T*)delta, scale, eps, (T*)out, n, d, stream);
                else if (chunks <= 6) launch_add_rmsnorm_rows<T, 6>(residual, (const T*)delta, scale, eps, (T*)out, n, d, stream);
                else launch_add_rmsnorm_rows<T, 8>(residual, (const T*)delta, scale, eps, (T*)out, n, d, stream);
            });
            return tis_check_launch("add_rmsnorm");
        }
    }
    const int threads = d >= 2048 ? 512 : 256;
    const size_t smem = (size_t)d * sizeof(float);
    TIS_DISPATCH_DTYPE(dtype, T, {
        if (smem > 48 * 1024)
            cudaFuncSetAttribute(add_rmsnorm_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        tis_launch(add_rmsnorm_kernel<T>, dim3(n), dim3(threads), smem, stream, residual, (const T*)delta, scale, eps,
                   (T*)out, d);
    });
    return tis_check_launch("add_rmsnorm");
}

// ----------------------------------------------------------------------------------
// Rows that still lack their norm's factor (the stream times the norm's weight, and partial sums of squares
// of the stream, as the residual epilogue of the weight-streaming products leaves them), made whole:
// out[r] = rows[r] * norm_factor(kind, width, eps).of(sum of parts[r]).  For readers that cannot apply the
// factor themselves.
__global__ void __launch_bounds__(256)
scale_rows_kernel(const bf16* __restrict__ rows, int ld, const float* __restrict__ parts, int n_parts, NormFactor factor,
                  bf16* __restrict__ out, int ldo, int d) {
    __shared__ float red[33];
    pdl_launch_dependents();
    pdl_wait();
    const int r = blockIdx.x;
    float s = 0.f;
    for (int i = threadIdx.x; i < n_parts; i += blockDim.x) s += parts[(size_t)r * n_parts + i];
    s = block_sum(s, red);
    const float f = factor.of(s);
    for (int i = threadIdx.x; i < d; i += blockDim.x)
        out[(size_t)r * ldo + i] = __float2bfloat16_rn(__bfloat162float(rows[(size_t)r * ld + i]) * f);
}

TIS_API int tis_scale_rows(const void* rows, int ld, const float* parts, int n_parts, float eps, int kind, void* out,
                           int ldo, int n, int d, cudaStream_t stream) {
    if (n <= 0 || d <= 0) return TIS_OK;
    if (n_parts <= 0 || kind < TIS_NORM_L2_EPS || kind > TIS_NORM_MEAN_EPS) {
        tis_set_error("scale_rows: %d partial sums a row, norm kind %d", n_parts, kind);
        return TIS_BAD_SIZE;
    }
    tis_launch(scale_rows_kernel, dim3(n), dim3(256), 0, stream, (const bf16*)rows, ld, parts, n_parts,
               norm_factor(kind, d, eps), (bf16*)out, ldo, d);
    return tis_check_launch("scale_rows");
}

// ----------------------------------------------------------------------------------
// rotary position encoding of q and k, and the write of k, v into the row's page.
//
// qkv row layout: [H*hd queries | KVH*hd keys | KVH*hd values] (keys before values, as
// the upstream kv_proj: main_models_new.py:104-106).  q is rotated in place.
// plane layout: [page][2 (k, v)][KVH][page_size][hd]; inside a row the 16-byte chunks are
// permuted by the position (cache_chunk in common.cuh).
// pairing: half-split (i, i + rot/2) as upstream rotate_half (main_models_new.py:71-73),
// or interleaved (2i, 2i+1); only the first `rot` entries of a head are rotated.
// cos/sin tables: [positions][rot/2] float.
// ----------------------------------------------------------------------------------
template <typename T>
__global__ void rope_kv_write_kernel(T* __restrict__ qkv, int row_stride, const int* __restrict__ positions,
                                     const int* __restrict__ row_slot, const float* __restrict__ cos_t,
                                     const float* __restrict__ sin_t, T* __restrict__ plane,
                                     const int* __restrict__ block_table, int bt_stride, int num_pages,
                                     int H, int KVH, int hd, int rot, int interleaved, int page_size,
                                     int write_kv, int* __restrict__ fault, int n, int tpr) {
    pdl_launch_dependents();
    // `tpr` threads of a CTA share a row (a power of two that divides the block): few rows (decode) get a CTA
    // each, the rows of a prompt portion 64 threads each, so that all of them are resident at once
    const int r = blockIdx.x * (blockDim.x / tpr) + threadIdx.x / tpr;
    const int tid = threadIdx.x % tpr;
    const int nthr = tpr;
    if (r >= n) return;
    const int slot = row_slot[r];              // step metadata: not written by the kernel before
    if (slot < 0) return;
    const int pos = positions[r];
    int page = -1;
    if (write_kv) {                            // the block table is step metadata too
        page = block_table[(size_t)slot * bt_stride + pos / page_size];
        if (page < 0 || page >= num_pages) {
            if (tid == 0) atomicExch(fault, 1);
            page = -1;
        }
    }
    pdl_wait();
    T* row = qkv + (size_t)r * row_stride;
    const int half = rot >> 1;
    const float* cs = cos_t + (size_t)pos * half;
    const float* sn = sin_t + (size_t)pos * half;
    constexpr int N = Vec16<T>::N;                 // elements of a 16-byte chunk
    const int nch = hd / N;                        // chunks of a cache row
    const bool fast = !interleaved && rot == hd && (half % N) == 0;

    const int in_page = pos % page_size;
    T* kdst = page >= 0 ? plane + ((size_t)page * 2 * KVH * page_size + in_page) * hd : nullptr;   // + h*page_size*hd
    T* vdst = page >= 0 ? kdst + (size_t)KVH * page_size * hd : nullptr;
    const T* ksrc = row + (size_t)H * hd;
    const T* vsrc = ksrc + (size_t)KVH * hd;

    if (fast && nthr % (half / N) == 0) {
        // the threads of a row divide evenly over the chunk pairs of a head: a thread keeps one chunk pair
        // (c, c + half/N) for every head it visits, so its cosines and sines are loaded once
        const int cpairs = half / N;
        const int c = tid % cpairs;
        float cv[N], sv[N];
#pragma unroll
        for (int j = 0; j < N; j += 4) {
            const float4 cc = *reinterpret_cast<const float4*>(cs + c * N + j);
            const float4 sc = *reinterpret_cast<const float4*>(sn + c * N + j);
            cv[j] = cc.x; cv[j + 1] = cc.y; cv[j + 2] = cc.z; cv[j + 3] = cc.w;
            sv[j] = sc.x; sv[j + 1] = sc.y; sv[j + 2] = sc.z; sv[j + 3] = sc.w;
        }
        const int heads = H + (page >= 0 ? KVH : 0);           // query heads, then (when written) key heads
        for (int hh = tid / cpairs; hh < heads; hh += nthr / cpairs) {
            const bool is_k = hh >= H;
            const int h = is_k ? hh - H : hh;
            const T* src = (is_k ? ksrc : row) + (size_t)h * hd;
            float x1[N], x2[N], o1[N], o2[N];
            Vec16<T>::load(src + c * N, x1);
            Vec16<T>::load(src + half + c * N, x2);
#pragma unroll
            for (int j = 0; j < N; ++j) {
                o1[j] = x1[j] * cv[j] - x2[j] * sv[j];
                o2[j] = x2[j] * cv[j] + x1[j] * sv[j];
            }
            if (!is_k) {
                T* dst = row + (size_t)h * hd;
                Vec16<T>::store(dst + c * N, o1);
                Vec16<T>::store(dst + half + c * N, o2);
            } else {
                T* dst = kdst + (size_t)h * page_size * hd;
                Vec16<T>::store(dst + cache_chunk(c, pos, nch) * N, o1);
                Vec16<T>::store(dst + cache_chunk(c + cpairs, pos, nch) * N, o2);
            }
        }
        if (page >= 0) {
            for (int w = tid; w < KVH * nch; w += nthr) {
                const int h = w / nch, cc = w - h * nch;
                float v[N];
                Vec16<T>::load(vsrc + (size_t)h * hd + cc * N, v);
                Vec16<T>::store(vdst + (size_t)h * page_size * hd + cache_chunk(cc, pos, nch) * N, v);
            }
        }
        return;
    }
    if (fast) {
        // one work item = the chunk pair (c, c + half/N) of one head: both halves of N rotation pairs
        const int cpairs = half / N;
        const int q_items = H * cpairs, k_items = page >= 0 ? KVH * cpairs : 0, v_items = page >= 0 ? KVH * nch : 0;
        for (int w = tid; w < q_items + k_items + v_items; w += nthr) {
            if (w < q_items + k_items) {
                const bool is_k = w >= q_items;
                const int ww = is_k ? w - q_items : w;
                const int h = ww / cpairs, c = ww - h * cpairs;
                const T* src = (is_k ? ksrc : row) + (size_t)h * hd;
                float x1[N], x2[N], cv[N], sv[N], o1[N], o2[N];
                Vec16<T>::load(src + c * N, x1);
                Vec16<T>::load(src + half + c * N, x2);
#pragma unroll
                for (int j = 0; j < N; j += 4) {
                    const float4 cc = *reinterpret_cast<const float4*>(cs + c * N + j);
                    const float4 sc = *reinterpret_cast<const float4*>(sn + c * N + j);
                    cv[j] = cc.x; cv[j + 1] = cc.y; cv[j + 2] = cc.z; cv[j + 3] = cc.w;
                    sv[j] = sc.x; sv[j + 1] = sc.y; sv[j + 2] = sc.z; sv[j + 3] = sc.w;
                }
#pragma unroll
                for (int j = 0; j < N; ++j) {
                    o1[j] = x1[j] * cv[j] - x2[j] * sv[j];
                    o2[j] = x2[j] * cv[j] + x1[j] * sv[j];
                }
                if (!is_k) {
                    T* dst = row + (size_t)h * hd;
                    Vec16<T>::store(dst + c * N, o1);
                    Vec16<T>::store(dst + half + c * N, o2);
                } else {
                    T* dst = kdst + (size_t)h * page_size * hd;
                    Vec16<T>::store(dst + cache_chunk(c, pos, nch) * N, o1);
                    Vec16<T>::store(dst + cache_chunk(c + cpairs, pos, nch) * N, o2);
                }
            } else {
                const int ww = w - q_items - k_items;
                const int h = ww / nch, c = ww - h * nch;
                float v[N];
                Vec16<T>::load(vsrc + (size_t)h * hd + c * N, v);
                Vec16<T>::store(vdst + (size_t)h * page_size * hd + cache_chunk(c, pos, nch) * N, v);
            }
        }
        return;
    }

    // general pairing (interleaved, or only part of the head rotated): element by element
    for (int w = tid; w < H * half; w += nthr) {
        const int h = w / half, i = w - h * half;
        const int a = interleaved ? 2 * i : i, b = interleaved ? 2 * i + 1 : i + half;
        T* x = row + (size_t)h * hd;
        const float x1 = to_f32(x[a]), x2 = to_f32(x[b]);
        const float c = cs[i], s = sn[i];
        x[a] = from_f32<T>(x1 * c - x2 * s);
        x[b] = from_f32<T>(x2 * c + x1 * s);
    }
    if (page < 0) return;
    for (int w = tid; w < KVH * half; w += nthr) {
        const int h = w / half, i = w - h * half;
        const int a = interleaved ? 2 * i : i, b = interleaved ? 2 * i + 1 : i + half;
        const float x1 = to_f32(ksrc[h * hd + a]), x2 = to_f32(ksrc[h * hd + b]);
        const float c = cs[i], s = sn[i];
        T* o = kdst + (size_t)h * page_size * hd;
        o[cache_chunk(a / N, pos, nch) * N + a % N] = from_f32<T>(x1 * c - x2 * s);
        o[cache_chunk(b / N, pos, nch) * N + b % N] = from_f32<T>(x2 * c + x1 * s);
    }
    if (rot < hd) {
        const int rest = hd - rot;
        for (int w = tid; w < KVH * rest; w += nthr) {
            const int h = w / rest, i = rot + (w - h * rest);
            kdst[(size_t)h * page_size * hd + cache_chunk(i / N, pos, nch) * N + i % N] = ksrc[h * hd + i];
        }
    }
    for (int w = tid; w < KVH * hd; w += nthr) {
        const int h = w / hd, i = w - h * hd;
        vdst[(size_t)h * page_size * hd + cache_chunk(i / N, pos, nch) * N + i % N] = vsrc[w];
    }
}

TIS_API int tis_rope_kv_write(int dtype, void* qkv, int row_stride, const int* positions, const int* row_slot,
                              const float* cos_t, const float* sin_t, void* plane, const int* block_table,
                              int bt_stride, int num_pages, int n, int H, int KVH, int hd, int rot,
                              int interleaved, int page_size, int write_kv, int* fault, cudaStream_t stream) {
    if (n <= 0) return TIS_OK;
    if (rot % 2 || rot > hd || rot < 0) {
        tis_set_error("rope_kv_write: rotary size %d must be even and at most the head size %d", rot, hd);
        return TIS_BAD_SIZE;
    }
    if (hd % 8) {
        tis_set_error("rope_kv_write: head size %d must be a multiple of 8 (cache rows are stored in 16-byte chunks)", hd);
        return TIS_BAD_SIZE;
    }
    // measured at 2048 rows of the 0.9B model (us inside a graph): 32 threads a row 7.0, 64: 7.1, 128: 8.4,
    // a CTA a row 12.7
    const int tpr = n >= 128 ? 64 : 256;
    const int rows_per_block = 256 / tpr;
    const int blocks = (n + rows_per_block - 1) / rows_per_block;
    TIS_DISPATCH_DTYPE(dtype, T,
        tis_launch(rope_kv_write_kernel<T>, dim3(blocks), dim3(256), 0, stream, (T*)qkv, row_stride, positions, row_slot,
                   cos_t, sin_t, (T*)plane, block_table, bt_stride, num_pages, H, KVH, hd, rot, interleaved, page_size,
                   write_kv, fault, n, tpr));
    return tis_check_launch("rope_kv_write");
}

// ----------------------------------------------------------------------------------
// SwiGLU gating: out[r, j] = silu(gate_j) * up_j   (main_models_new.py:51).  The input row
// holds gate and up in alternating blocks of `block` columns: [gate 0..b-1 | up 0..b-1 |
// gate b..2b-1 | ...]; block = F is the plain layout [all gates | all ups].
// ----------------------------------------------------------------------------------
template <typename T>
__global__ void swiglu_kernel(const T* __restrict__ gu, T* __restrict__ out, int F, int block, size_t total) {
    pdl_launch_dependents();
    pdl_wait();
    constexpr int N = Vec16<T>::N;
    if (block % N == 0) {
        // two 16-byte items per thread and trip, all four loads ordered before the first use
        const unsigned nvec = (unsigned)(total / N);
        const unsigned fv = (unsigned)(F / N);
        const unsigned stride = gridDim.x * blockDim.x;
        for (unsigned idx = blockIdx.x * blockDim.x + threadIdx.x; idx < nvec; idx += 2 * stride) {
            const unsigned idx2 = idx + stride;
            const bool two = idx2 < nvec;
            const unsigned r1 = idx / fv, r2 = two ? idx2 / fv : r1;
            const int j1 = (int)(idx - r1 * fv) * N, j2 = two ? (int)(idx2 - r2 * fv) * N : j1;
            const int b1 = j1 / block, b2 = j2 / block;
            const T* s1 = gu + (size_t)r1 * 2 * F + (size_t)b1 * 2 * block + (j1 - b1 * block);
            const T* s2 = gu + (size_t)r2 * 2 * F + (size_t)b2 * 2 * block + (j2 - b2 * block);
            float g1[N], u1[N], g2[N], u2[N], o[N];
            Vec16<T>::load(s1, g1);
            Vec16<T>::load(s1 + block, u1);
            Vec16<T>::load(s2, g2);
            Vec16<T>::load(s2 + block, u2);
#pragma unroll
            for (int k = 0; k < N; ++k) o[k] = g1[k] / (1.f + __expf(-g1[k])) * u1[k];
            Vec16<T>::store(out + (size_t)r1 * F + j1, o);
            if (two) {
#pragma unroll
                for (int k = 0; k < N; ++k) o[k] = g2[k] / (1.f + __expf(-g2[k])) * u2[k];
                Vec16<T>::store(out + (size_t)r2 * F + j2, o);
            }
        }
        return;
    }
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
         idx += (size_t)gridDim.x * blockDim.x) {
        const size_t r = idx / F;
        const int j = (int)(idx - r * F);
        const int b = j / block;
        const T* src = gu + r * 2 * F + (size_t)b * 2 * block + (j - b * block);
        const float g = to_f32(src[0]);
        const float u = to_f32(src[block]);
        out[idx] = from_f32<T>(g / (1.f + expf(-g)) * u);
    }
}

TIS_API int tis_swiglu(int dtype, const void* gu, void* out, int n, int F, int block, cudaStream_t stream) {
    if (n <= 0) return TIS_OK;
    if (block <= 0 || F % block) {
        tis_set_error("swiglu: block %d does not divide the hidden size %d", block, F);
        return TIS_BAD_SIZE;
    }
    const size_t total = (size_t)n * F;
    if (total / 4 >= 0xffffffffu) {
        tis_set_error("swiglu: %d x %d elements are more than this kernel indexes", n, F);
        return TIS_BAD_SIZE;
    }
    size_t blocks = (total / 16 + 255) / 256;
    if (blocks < 1) blocks = 1;
    if (blocks > 148 * 16) blocks = 148 * 16;
    TIS_DISPATCH_DTYPE(dtype, T,
        tis_launch(swiglu_kernel<T>, dim3((unsigned)blocks), dim3(256), 0, stream, (const T*)gu, (T*)out, F, block,
                   total));
    return tis_check_launch("swiglu");
}

// ----------------------------------------------------------------------------------
// residual += delta  (when no norm follows)
// ----------------------------------------------------------------------------------
template <typename T>
__global__ void residual_add_kernel(float* __restrict__ res, const T* __restrict__ delta, size_t total) {
    pdl_launch_dependents();
    pdl_wait();
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
         idx += (size_t)gridDim.x * blockDim.x)
        res[idx] += to_f32(delta[idx]);
}

TIS_API int tis_residual_add(int dtype, float* residual, const void* delta, int n, int d, cudaStream_t stream) {
    if (n <= 0) return TIS_OK;
    const size_t total = (size_t)n * d;
    size_t blocks = (total + 255) / 256;
    if (blocks > 148 * 16) blocks = 148 * 16;
    TIS_DISPATCH_DTYPE(dtype, T,
        tis_launch(residual_add_kernel<T>, dim3((unsigned)blocks), dim3(256), 0, stream, residual, (const T*)delta,
                   total));
    return tis_check_launch("residual_add");
}

// ----------------------------------------------------------------------------------
// Input of an MTP head (main_models_new.py:164): out[r] = [ h_prev of the row before r |
// rmsnorm(table[token[r]]) ].  The row before the first row of a request in this step
// is the row saved in the request's state slot by the step before; the first row's
// CTA then saves h_prev[last row of the request in this step] there for the next step.
// ----------------------------------------------------------------------------------
template <typename T>
__global__ void mtp_input_kernel(const T* __restrict__ h_prev, T* __restrict__ state,
                                 const int* __restrict__ row_slot, const int* __restrict__ row_last,
                                 const int* __restrict__ tokens, const T* __restrict__ table,
                                 const float* __restrict__ scale, float eps, T* __restrict__ out, int d) {
    extern __shared__ float row[];
    __shared__ float red[33];
    pdl_launch_dependents();
    pdl_wait();
    const int r = blockIdx.x;
    const int slot = row_slot[r];
    if (slot < 0) return;
    T* o = out + (size_t)r * 2 * d;
    const bool first = (r == 0) || (row_slot[r - 1] != slot);
    if (first) {
        T* st = state + (size_t)slot * d;
        const T* keep = h_prev + (size_t)row_last[r] * d;
        for (int i = threadIdx.x; i < d; i += blockDim.x) {
            o[i] = st[i];
            st[i] = keep[i];
        }
    } else {
        const T* src = h_prev + (size_t)(r - 1) * d;
        for (int i = threadIdx.x; i < d; i += blockDim.x) o[i] = src[i];
    }
    const T* e = table + (size_t)tokens[r] * d;
    float ss = 0.f;
    for (int i = threadIdx.x; i < d; i += blockDim.x) {
        const float v = to_f32(e[i]);
        row[i] = v;
        ss += v * v;
    }
    ss = block_sum(ss, red);
    const float inv = sqrtf((float)d) / (sqrtf(ss) + eps);
    for (int i = threadIdx.x; i < d; i += blockDim.x) o[d + i] = from_f32<T>(row[i] * inv * scale[i]);
}

TIS_API int tis_mtp_input(int dtype, const void* h_prev, void* state, const int* row_slot, const int* row_last,
                          const int* tokens, const void* table, const float* scale, float eps, void* out,
                          int n, int d, cudaStream_t stream) {
    if (n <= 0) return TIS_OK;
    if ((size_t)d * sizeof(float) > 96 * 1024) {
        tis_set_error("mtp_input: width %d too large (one row must fit 96 KB of shared memory)", d);
        return TIS_BAD_SIZE;
    }
    const size_t smem = (size_t)d * sizeof(float);
    TIS_DISPATCH_DTYPE(dtype, T, {
        if (smem > 48 * 1024)
            cudaFuncSetAttribute(mtp_input_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        tis_launch(mtp_input_kernel<T>, dim3(n), dim3(256), smem, stream, (const T*)h_prev, (T*)state, row_slot,
                   row_last, tokens, (const T*)table, scale, eps, (T*)out, d);
    });
    return tis_check_launch("mtp_input");
}
