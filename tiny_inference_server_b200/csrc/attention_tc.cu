// Causal attention of long prompt portions over the paged cache on the fifth-generation
// tensor cores (head sizes 64 and 128, bfloat16).
//
// A CTA owns up to 128 consecutive rows (positions pos0..pos0+rows-1) of one request and one
// query head, and walks the keys 128 at a time.  Three roles, specialised by warp:
//   warps 0 and 10   the TMA engine's clients: warp 0 brings the Q tile once (128-byte swizzle)
//            and then the keys of every key tile, warp 10 the values, each into a ring of
//            shared-memory slots of its own (keys are needed early, values late: with rings of
//            their own the key loads run ahead), one box of 64 elements x page_size rows per page
//            and half of the head (lanes order the pages of a tile side by side).  The cache
//            keeps rows XOR-swizzled by the position, so the boxes, copied as the bytes lie, are
//            at once the swizzled operand tiles;
//   warps 1 and 11   issue the products (one lane each; warp 1 also owns the tensor memory):
//            warp 1 S = Q K^T into one of two score buffers in tensor memory (keys as the K-major
//            operand), warp 11 O += P V (values as the MN-major operand, P from shared memory);
//            two issuing threads, so that one's wait for a barrier does not idle the tensor cores;
//   warps 2-5 and 6-9: two softmax groups, one thread per query row each.  Even key tiles go
//            to the first group, odd ones to the second, each with a score buffer, a P buffer,
//            an output accumulator in tensor memory and running maximum and sum of its own, so
//            the softmax of one tile runs under the products and the softmax of the next; the
//            two halves are merged at the end.  A thread reads its row of S (tcgen05.ld),
//            scales, masks, does the online softmax in float32 and writes P in bfloat16 into
//            shared memory in the operand layout.  The running maximum is only raised when the
//            row's new maximum exceeds it by more than 2^8 (the exponentials stay small enough);
//            O in tensor memory is then rescaled (tcgen05.ld, tcgen05.st).
// All hand-offs are mbarriers with bounded waits; a wait that runs out sets the fault word and
// every role leaves; tensor memory is freed on every path.
#include "tc_common.cuh"

#ifndef TIS_HD
#define TIS_HD 128
#endif

#if (TIS_HD % 64 == 0) && (TIS_HD <= 128)

namespace {

using namespace tc;

constexpr int HD = TIS_HD;
constexpr int HALVES = HD / 64;             // 128-byte column blocks of a row
constexpr int BM = 128;                     // query rows of a CTA
constexpr int BN = 128;                     // keys of a tile
constexpr int NTH = 384;
constexpr int HALF_BYTES = 128 * 128;       // 128 rows x 128 bytes: one swizzled column block
constexpr int Q_BYTES = HALVES * HALF_BYTES;
constexpr int P_BYTES = 2 * HALF_BYTES;     // 128 rows x 128 keys, bfloat16 (one per softmax group)
constexpr int SLOT_BYTES = HALVES * HALF_BYTES;   // keys or values of one tile
constexpr int SLOTS = HD == 128 ? 2 : 4;     // per ring (keys, values)
constexpr unsigned TMEM_COLS = 512;
constexpr unsigned COL_S = 0;               // two score buffers of 128 columns
constexpr unsigned COL_O = 256;             // two output accumulators of up to 128 columns
constexpr float RESCALE_STEP = 8.f;         // in units of log2

struct TcAttnParams {
    bf16* out; int out_stride;
    const int* block_table; int bt_stride; int num_pages;
    const int* positions; const int* row_slot;
    const int* tile_row0; const int* tile_rows; int num_tiles;
    int H, KVH, page_size, window;
    float scale_log2;
    int* fault;
};

__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
    return y;
}

__global__ void __launch_bounds__(NTH, 1)
attn_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_kv, const TcAttnParams p) {
    extern __shared__ unsigned char smem_raw[];
    unsigned char* base = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    unsigned char* q_smem = base;
    unsigned char* p_smem = base + Q_BYTES;
    unsigned char* k_slots = p_smem + 2 * P_BYTES;
    unsigned char* v_slots = k_slots + SLOTS * SLOT_BYTES;
    __shared__ unsigned long long q_full, full_k[SLOTS], empty_k[SLOTS], full_v[SLOTS], empty_v[SLOTS], s_full[2], p_full[2], o_done[2];
    __shared__ unsigned tmem_base_slot;
    __shared__ int abort_flag;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    pdl_launch_dependents();

    // heaviest tiles (the last rows of a prompt see the most keys) first
    const int tile = p.num_tiles - 1 - (int)blockIdx.x / p.H;
    const int head = (int)blockIdx.x % p.H;
    const int kvh = head / (p.H / p.KVH);
    const int row0 = p.tile_row0[tile];
    const int nrows = min(p.tile_rows[tile], BM);
    if (nrows <= 0) return;
    // A stage that runs behind the trunk sees the first rows of a prompt as padding (slot -1,
    // position 0): the tile's request and last position are those of its last row.
    const int slot = p.row_slot[row0 + nrows - 1];
    if (slot < 0) return;                                 // padding only: the whole CTA leaves together
    const int pos0 = p.positions[row0];                   // the smallest position of the tile
    const int hi = p.positions[row0 + nrows - 1] + 1;     // keys [.., hi) are visible to the last row
    const int lo_first = p.window > 0 ? max(0, pos0 - p.window + 1) : 0;
    const int tile_begin = lo_first & ~(BN - 1);
    const int T = (hi - tile_begin + BN - 1) / BN;

    if (threadIdx.x == 0) {
        mbar_init(&q_full, 1);
        for (int s = 0; s < SLOTS; ++s) {
            mbar_init(&full_k[s], 1); mbar_init(&empty_k[s], 1);
            mbar_init(&full_v[s], 1); mbar_init(&empty_v[s], 1);
        }
        mbar_init(&s_full[0], 1); mbar_init(&s_full[1], 1);
        mbar_init(&p_full[0], 4); mbar_init(&p_full[1], 4);
        mbar_init(&o_done[0], 1); mbar_init(&o_done[1], 1);
        abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
        prefetch_map(&map_q);
        prefetch_map(&map_kv);
    }
    if (warp == 1) tmem_alloc(&tmem_base_slot, TMEM_COLS);
    fence_before();
    __syncthreads();
    fence_after();
    const unsigned tmem_base = tmem_base_slot;
    volatile int* abort = &abort_flag;
    pdl_wait();                                           // q and the cache rows of this step come from the kernel before

    if (warp == 0 || warp == 10) {
        // ---- loads: warp 0 keys (and Q), warp 10 values -----------------------------------------
        const int kv = warp == 0 ? 0 : 1;
        unsigned long long* full = kv ? full_v : full_k;
        unsigned long long* empty = kv ? empty_v : empty_k;
        unsigned char* ring = kv ? v_slots : k_slots;
        const int ppt = BN / p.page_size;                 // pages of a key tile (1..8)
        const int* bt = p.block_table + (size_t)slot * p.bt_stride;
        auto page_of = [&](int j) -> int {
            if (lane >= ppt) return 0;
            const int key0 = tile_begin + j * BN + lane * p.page_size;
            if (key0 >= hi || key0 + p.page_size <= lo_first) return 0;   // no row sees it: any page will do
            const int pg = bt[key0 / p.page_size];
            if (pg < 0 || pg >= p.num_pages) { atomicExch(p.fault, 3); return 0; }
            return pg;
        };
        if (kv == 0 && lane == 0) {
            mbar_arrive_expect_tx(&q_full, Q_BYTES);
#pragma unroll
            for (int hh = 0; hh < HALVES; ++hh)
                tma_load_2d(q_smem + hh * HALF_BYTES, &map_q, head * HD + hh * 64, row0, &q_full);
        }
        int page_next = page_of(0);
        for (int j = 0; j < T; ++j) {
            const int page = page_next;
            page_next = j + 1 < T ? page_of(j + 1) : 0;
            const int s = j % SLOTS;
            int got = 1;
            if (lane == 0) got = mbar_wait(&empty[s], ((j / SLOTS) & 1) ^ 1, abort, p.fault, 6) ? 1 : 0;
            got = __shfl_sync(0xffffffffu, got, 0);
            if (!got) break;
            if (lane == 0) mbar_arrive_expect_tx(&full[s], SLOT_BYTES);
            __syncwarp();
            if (lane < ppt) {
                unsigned char* dst = ring + (size_t)s * SLOT_BYTES + lane * p.page_size * 128;
                const int y = ((page * 2 + kv) * p.KVH + kvh) * p.page_size;
#pragma unroll
                for (int hh = 0; hh < HALVES; ++hh) tma_load_2d(dst + hh * HALF_BYTES, &map_kv, hh * 64, y, &full[s]);
            }
        }
    } else if (warp == 1) {
        // ---- products, first kind: S_j = Q K_j^T into score buffer j & 1 ----------------------------
        if (lane == 0) {
            constexpr unsigned IDESC_S = instr_desc(BM, BN, false);
            const unsigned long long q_desc0 = smem_desc(smem_u32(q_smem), 16, 1024);
            const unsigned long long k_desc0 = smem_desc(smem_u32(k_slots), 16, 1024);
            bool ok = mbar_wait(&q_full, 0, abort, p.fault, 6);
            for (int j = 0; j < T && ok; ++j) {
                const int g = j & 1, i = j >> 1, s = j % SLOTS;
                // the group has read the scores of its tile before (it hands P over after that)
                if (i > 0 && !mbar_wait(&p_full[g], (i - 1) & 1, abort, p.fault, 6)) break;
                if (!mbar_wait(&full_k[s], (j / SLOTS) & 1, abort, p.fault, 6)) break;
                fence_after();
                // descriptors differ from the ring's first one only in the start address (units of 16 bytes)
                const unsigned long long kd = k_desc0 + (unsigned long long)((s * SLOT_BYTES) >> 4);
                const unsigned d = tmem_base + COL_S + g * BN;
#pragma unroll
                for (int kk = 0; kk < HD / 16; ++kk) {
                    const unsigned long long off = (unsigned long long)(((kk >> 2) * HALF_BYTES + (kk & 3) * 32) >> 4);
                    umma(d, q_desc0 + off, kd + off, IDESC_S, kk != 0);
                }
                umma_commit(&empty_k[s]);
                umma_commit(&s_full[g]);
            }
        }
    } else if (warp == 11) {
        // ---- products, second kind: O_g += P_j V_j.  An issuing thread of its own: while one thread
        // waits for a barrier the other keeps the tensor cores fed. ------------------------------------
        if (lane == 0) {
            constexpr unsigned IDESC_O = instr_desc(BM, HD, true);
            const unsigned long long p_desc0 = smem_desc(smem_u32(p_smem), 16, 1024);
            const unsigned long long v_desc0 = smem_desc(smem_u32(v_slots), HALF_BYTES, 1024);
            for (int j = 0; j < T; ++j) {
                const int g = j & 1, i = j >> 1, s = j % SLOTS;
                if (!mbar_wait(&p_full[g], i & 1, abort, p.fault, 6)) break;
                if (!mbar_wait(&full_v[s], (j / SLOTS) & 1, abort, p.fault, 6)) break;
                fence_after();
                const unsigned long long vd = v_desc0 + (unsigned long long)((s * SLOT_BYTES) >> 4);
                const unsigned long long pd = p_desc0 + (unsigned long long)((g * P_BYTES) >> 4);
                const unsigned d = tmem_base + COL_O + g * 128;
#pragma unroll
                for (int kk = 0; kk < BN / 16; ++kk) {    // 16 keys: 32 bytes along a row of P, 16 rows of V
                    umma(d, pd + (unsigned long long)(((kk >> 2) * HALF_BYTES + (kk & 3) * 32) >> 4),
                         vd + (unsigned long long)((kk * 2048) >> 4), IDESC_O, (i | kk) != 0);
                }
                umma_commit(&empty_v[s]);
                umma_commit(&o_done[g]);
            }
        }
    } else {
        // ---- softmax: one thread per query row in each of the two groups ----------------------
        const int g = warp >= 6 ? 1 : 0;                  // warps 2-5 and 6-9
        const int quarter = warp & 3;                     // the lanes of tensor memory this warp may touch
        const int r = quarter * 32 + lane;
        const bool row_ok = r < nrows && p.row_slot[row0 + r] >= 0;
        const int qpos = row_ok ? p.positions[row0 + r] : 0;
        const int lo_r = p.window > 0 ? max(0, qpos - p.window + 1) : 0;
        const int lo_last = p.window > 0 ? max(0, hi - p.window) : 0;      // the last row's first key
        const unsigned lane_bits = (unsigned)(quarter * 32) << 16;
        const unsigned col_s = COL_S + g * BN, col_o = COL_O + g * 128;
        unsigned char* pg_smem = p_smem + g * P_BYTES;
        const bool warp_has_rows = __any_sync(0xffffffffu, row_ok);
        float m_used = -INFINITY, l_sum = 0.f;
        bool ok = true;
        int i = 0;                                        // tiles of this group so far
        for (int j = g; j < T; j += 2, ++i) {
            if (!__all_sync(0xffffffffu, mbar_wait(&s_full[g], i & 1, abort, p.fault, 6))) { ok = false; break; }
            fence_after();
            if (!warp_has_rows) {
                // a warp whose 32 rows are all beyond the tile: its rows of P are zero, once and for all
                if (i == 0) {
#pragma unroll
                    for (int c = 0; c < 16; ++c)
                        *reinterpret_cast<uint4*>(pg_smem + r * 128 + (c >> 3) * HALF_BYTES + ((c & 7) << 4)) = make_uint4(0u, 0u, 0u, 0u);
                    asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
                }
                fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(&p_full[g]);
                continue;
            }
            const int kt = tile_begin + j * BN;
            // Two passes over the row of S, 64 columns at a time (the row stays in tensor memory until
            // this group hands P over): first the maximum, then the exponentials.
            const bool whole = kt + BN - 1 <= pos0 && kt >= lo_last;      // every row of the tile sees every key
            const bool plain = whole && row_ok;
            auto load64 = [&](int half, float (&s)[64]) {
                tmem_ld32_issue(tmem_base + lane_bits + col_s + half * 64, s);
                tmem_ld32_issue(tmem_base + lane_bits + col_s + half * 64 + 32, s + 32);
                tmem_ld_wait();
                tmem_ld_arrived(s);
                if (!plain) {
#pragma unroll
                    for (int e = 0; e < 64; ++e) {
                        const int key = kt + half * 64 + e;
                        s[e] = (row_ok && key <= qpos && key >= lo_r) ? s[e] : -INFINITY;
                    }
                }
            };
            // the row's maximum of the raw scores (the scale is positive), four chains side by side
            float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll 1
            for (int half = 0; half < 2; ++half) {
                float s[64];
                load64(half, s);
#pragma unroll
                for (int e = 0; e < 64; ++e) mx4[e & 3] = fmaxf(mx4[e & 3], s[e]);
            }
            const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3])) * p.scale_log2;
            // raise the reference maximum only when the row's maximum left it far behind
            const bool raise = mx > m_used + RESCALE_STEP || (m_used == -INFINITY && mx > -INFINITY);
            float alpha = 1.f;
            if (raise) {
                alpha = m_used == -INFINITY ? 0.f : fast_exp2(m_used - mx);
                m_used = mx;
                l_sum *= alpha;
            }
            // the products of the group's tile before are done: O may be rescaled, P overwritten
            if (i > 0 && !__all_sync(0xffffffffu, mbar_wait(&o_done[g], (i - 1) & 1, abort, p.fault, 6))) { ok = false; break; }
            if (i > 0 && __any_sync(0xffffffffu, raise)) {
                fence_after();
#pragma unroll 1
                for (int c = 0; c < HD / 32; ++c) {
                    float o[32];
                    tmem_ld32(tmem_base + lane_bits + col_o + c * 32, o);
#pragma unroll
                    for (int e = 0; e < 32; ++e) o[e] *= alpha;
                    tmem_st32(tmem_base + lane_bits + col_o + c * 32, o);
                }
                fence_before();
            }
            const float neg_m = m_used == -INFINITY ? 0.f : -m_used;
            float ps4[4] = {0.f, 0.f, 0.f, 0.f};
            unsigned char* prow = pg_smem + r * 128;
#pragma unroll 1
            for (int half = 0; half < 2; ++half) {
                float s[64];
                load64(half, s);
#pragma unroll
                for (int c = 0; c < 8; ++c) {             // eight keys: one 16-byte chunk of the row of P
                    unsigned pk[4];
#pragma unroll
                    for (int e = 0; e < 8; e += 2) {
                        const float a = fast_exp2(fmaf(s[c * 8 + e], p.scale_log2, neg_m));   // 2^-inf = 0 for masked keys
                        const float b = fast_exp2(fmaf(s[c * 8 + e + 1], p.scale_log2, neg_m));
                        ps4[e >> 1] += a + b;
                        __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
                        pk[e >> 1] = *reinterpret_cast<unsigned*>(&h);
                    }
                    *reinterpret_cast<uint4*>(prow + half * HALF_BYTES + ((c ^ (r & 7)) << 4)) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
                }
            }
            l_sum += (ps4[0] + ps4[1]) + (ps4[2] + ps4[3]);
            asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
            fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&p_full[g]);
        }
        // ---- merge the two groups' halves; each group stores half of the columns -------------
        if (i > 0 && ok) ok = __all_sync(0xffffffffu, mbar_wait(&o_done[g], (i - 1) & 1, abort, p.fault, 6));
        // the group's P buffer is free now: it carries the row's maximum and sum to the other group
        reinterpret_cast<float*>(pg_smem)[r] = m_used;
        reinterpret_cast<float*>(pg_smem)[BM + r] = l_sum;
        fence_before();
        asm volatile("bar.sync 1, 256;\n" ::: "memory");        // both groups' products are done, sums are in place
        fence_after();
        if (ok && !*abort) {
            const float* mg0 = reinterpret_cast<const float*>(p_smem);
            const float* mg1 = reinterpret_cast<const float*>(p_smem + P_BYTES);
            const float m0 = mg0[r], m1 = mg1[r], l0 = mg0[BM + r], l1 = mg1[BM + r];
            const float m = fmaxf(m0, m1);
            const float w0 = m0 == -INFINITY ? 0.f : fast_exp2(m0 - m);
            const float w1 = (T < 2 || m1 == -INFINITY) ? 0.f : fast_exp2(m1 - m);
            const float l = l0 * w0 + l1 * w1;
            const float inv = l > 0.f ? 1.f / l : 0.f;
            constexpr int COLS = HD / 2;                  // this group's share of the columns
#pragma unroll 1
            for (int c = 0; c < COLS / 32; ++c) {
                const int col = g * COLS + c * 32;
                float o0[32], o1[32];
                tmem_ld32_issue(tmem_base + lane_bits + COL_O + col, o0);
                if (T >= 2) tmem_ld32_issue(tmem_base + lane_bits + COL_O + 128 + col, o1);
                tmem_ld_wait();
                tmem_ld_arrived(o0);
                if (T >= 2) tmem_ld_arrived(o1);
                if (r < nrows) {                          // padding rows inside the tile get zeros
#pragma unroll
                    for (int e = 0; e < 32; ++e) o0[e] = row_ok ? (o0[e] * w0 + (T >= 2 ? o1[e] * w1 : 0.f)) * inv : 0.f;
                    bf16* dst = p.out + (size_t)(row0 + r) * p.out_stride + head * HD + col;
#pragma unroll
                    for (int q = 0; q < 4; ++q) store8(dst + q * 8, o0 + q * 8);
                }
            }
            fence_before();
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

}  // namespace

TIS_API int tis_attn_tc_supported() { return 1; }

// Attention of `num_tiles` tiles of up to 128 consecutive rows of one request each.  q is
// (n, >= H*hd) with row stride q_stride, out (n, H*hd); plane is [pages, 2, KVH, page_size, hd];
// page_size 16, 32, 64 or 128.
TIS_API int tis_attn_tc(const void* q, int q_stride, int n_rows, void* out, int out_stride, const void* plane,
                        const int* block_table, int bt_stride, int num_pages, const int* positions,
                        const int* row_slot, const int* tile_row0, const int* tile_rows, int num_tiles, int H,
                        int KVH, int page_size, int window, float scale, int* fault, cudaStream_t stream) {
    if (num_tiles <= 0) return TIS_OK;
    if (page_size != 16 && page_size != 32 && page_size != 64 && page_size != 128) {
        tis_set_error("attn_tc: page size %d; this kernel takes 16, 32, 64 or 128", page_size);
        return TIS_BAD_SIZE;
    }
    if (KVH <= 0 || H % KVH || (q_stride % 8) || (out_stride % 8) ||
        (reinterpret_cast<uintptr_t>(q) | reinterpret_cast<uintptr_t>(out) | reinterpret_cast<uintptr_t>(plane)) % 16) {
        tis_set_error("attn_tc: heads %d/%d, strides %d %d: strides must be multiples of 8 and pointers 16-byte aligned",
                      H, KVH, q_stride, out_stride);
        return TIS_BAD_SIZE;
    }
    CUtensorMap mq, mkv;
    if (!tensor_map(q, (long long)H * HD, n_rows, q_stride, BM, true, &mq)) return TIS_CUDA_ERROR;
    if (!tensor_map(plane, HD, (long long)num_pages * 2 * KVH * page_size, HD, page_size, false, &mkv)) return TIS_CUDA_ERROR;
    constexpr int smem = Q_BYTES + 2 * P_BYTES + 2 * SLOTS * SLOT_BYTES + 1024;
    static bool configured = false;
    if (!configured) {
        if (cudaFuncSetAttribute(attn_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess)
            return tis_check_launch("attn_tc (shared memory)");
        configured = true;
    }
    TcAttnParams p;
    p.out = static_cast<bf16*>(out); p.out_stride = out_stride;
    p.block_table = block_table; p.bt_stride = bt_stride; p.num_pages = num_pages;
    p.positions = positions; p.row_slot = row_slot;
    p.tile_row0 = tile_row0; p.tile_rows = tile_rows; p.num_tiles = num_tiles;
    p.H = H; p.KVH = KVH; p.page_size = page_size; p.window = window;
    p.scale_log2 = scale * 1.4426950408889634f;
    p.fault = fault;
    tis_launch(attn_tc_kernel, dim3(num_tiles * H), dim3(NTH), (size_t)smem, stream, mq, mkv, p);
    return tis_check_launch("attn_tc");
}

#else

TIS_API int tis_attn_tc_supported() { return 0; }

TIS_API int tis_attn_tc(const void*, int, int, void*, int, const void*, const int*, int, int, const int*, const int*,
                        const int*, const int*, int, int, int, int, int, float, int*, cudaStream_t) {
    tis_set_error("attn_tc: built for a head size it does not take (64 and 128 only)");
    return TIS_BAD_SIZE;
}

#endif
