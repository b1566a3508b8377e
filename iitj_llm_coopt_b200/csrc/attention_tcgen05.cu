// Paged causal attention for prompt portions on the fifth-generation tensor cores
// (bfloat16, head size 128, page sizes 8 .. 128 that divide 128).
//
// One CTA = 128 queries of one request x one query head.  Keys and values walk through shared
// memory in tiles of 128 keys; each page of a tile is one TMA box per 64-dim half, placed at
// its row offset of the 128-byte-swizzled tile, so the paged cache needs no gather pass.
//
//   S = Q K^T      tcgen05.mma, M = 128 queries, N = 128 keys, K = 128 dims, both operands K-major
//                  in shared memory; S lands in tensor memory (two buffers of 128 columns).
//   softmax        eight warps, two threads per query row (64 of the tile's 128 keys each): a thread reads
//                  its part of the row of S with tcgen05.ld (a TMEM lane is a row: no shuffles), masks by
//                  position, takes the maximum (the two halves meet through shared memory), exponentiates
//                  in float32 and writes P as bfloat16 into a swizzled shared tile.
//   O_tile = P V   tcgen05.mma, M = 128 queries, N = 128 dims, K = 128 keys; P is K-major, V is
//                  MN-major (a key's 128 dims are contiguous), so the V tile is used as it was loaded.
//   accumulate     the same threads read O_tile from tensor memory and fold it into a float32 row
//                  accumulator in registers with the online-softmax correction.
//
// The MMA warp issues S of tile j+1 before P V of tile j, so the tensor core works on the next
// scores while the softmax warps work on the current ones.  Replaces flash_attn_varlen_func
// (engine/model.py:204-207) for portions; same masking and float32 statistics as the mma.sync
// kernel of attention_bf16.cu, which remains for other head and page sizes.
//
// Every mbarrier wait is bounded; a wait that runs out records a code (llm_attention_tcgen05_status)
// and the CTA falls through to its teardown, where the tensor memory is freed.
#include "tcgen05_common.cuh"

namespace {

typedef __nv_bfloat16 bf16;

constexpr int kRows = 128;        // queries per CTA (UMMA M)
constexpr int kKeys = 128;        // keys per tile
constexpr int kDim = 128;         // head size
constexpr int kHalfBytes = 128 * 128;          // one 64-column half of a [128 x 128] bf16 tile: 128 rows x 128 bytes
constexpr int kTileBytes = 2 * kHalfBytes;     // 32 KiB
constexpr int kThreads = 320;     // warp 0: loads, warp 1: MMA + TMEM, warps 2-9: softmax and output
constexpr int kSoftmaxThreads = 256;
constexpr int kCols = 64;         // columns of S (keys) and of O (dims) per softmax thread
constexpr uint32_t kTmemCols = 512;            // S0 | S1 | O0 | O1, 128 float32 columns each

__device__ int g_attn_status = 0;
__device__ __forceinline__ void attn_give_up(int code) { atomicCAS(&g_attn_status, 0, (code << 16) | (int)(blockIdx.x & 0xffff)); }

__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

__device__ __forceinline__ float ex2(float x) {          // 2^x, x <= 0 here; one MUFU instruction
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// This thread's 64 columns of one S or O buffer (its TMEM lane) in one round trip.
__device__ __forceinline__ void load_cols(uint32_t addr, uint32_t (&r)[kCols]) {
    tmem_ld32(addr, *reinterpret_cast<uint32_t(*)[32]>(&r[0]));
    tmem_ld32(addr + 32, *reinterpret_cast<uint32_t(*)[32]>(&r[32]));
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// Maximum over the 64 scores; k0 = key of the first one.
template <bool MASK>
__device__ __forceinline__ float row_max(const uint32_t (&r)[kCols], int k0, int row_pos, int row_lo) {
    float mx = -INFINITY;
#pragma unroll
    for (int c = 0; c < kCols; ++c) {
        if (MASK) {
            const int key = k0 + c;
            if (key <= row_pos && key >= row_lo) mx = fmaxf(mx, __uint_as_float(r[c]));
        } else {
            mx = fmaxf(mx, __uint_as_float(r[c]));
        }
    }
    return mx;
}

// P = 2^(S * sl - mu) of the 64 scores as bfloat16 into this thread's row of one half of the swizzled P tile
// (`p_half` = that half's base: 128 rows of 128 bytes); returns the sum.
template <bool MASK>
__device__ __forceinline__ float row_exp(const uint32_t (&r)[kCols], unsigned char* p_half, int row, float sl, float mu,
                                         int k0, int row_pos, int row_lo) {
    float sum = 0.f;
    unsigned char* prow = p_half + row * 128;
#pragma unroll
    for (int c0 = 0; c0 < kCols; c0 += 8) {          // 8 keys = one 16-byte chunk
        uint32_t packed[4];
#pragma unroll
        for (int c = 0; c < 8; c += 2) {
            float p0 = ex2(fmaf(__uint_as_float(r[c0 + c]), sl, -mu));
            float p1 = ex2(fmaf(__uint_as_float(r[c0 + c + 1]), sl, -mu));
            if (MASK) {
                const int key = k0 + c0 + c;
                if (key > row_pos || key < row_lo) p0 = 0.f;
                if (key + 1 > row_pos || key + 1 < row_lo) p1 = 0.f;
            }
            sum += p0 + p1;
            packed[c >> 1] = pack2(p0, p1);
        }
        *reinterpret_cast<uint4*>(prow + (((c0 >> 3) ^ (row & 7)) << 4)) = make_uint4(packed[0], packed[1], packed[2], packed[3]);
    }
    return sum;
}

struct AttnArgs {
    const int* block_table;
    int table_width;
    const int4* tiles;            // {first token row, rows (<= 128), position of the first row, request}
    bf16* out;
    int out_stride;
    int heads, kv_heads, page_size, window;
    float sl;                     // softmax scale * log2(e)
};

__global__ void __launch_bounds__(kThreads, 1)
attn_prefill_tcgen05_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_kv,
                            const AttnArgs a) {
    extern __shared__ unsigned char smem_raw[];
    unsigned char* base = reinterpret_cast<unsigned char*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    unsigned char* q_tile = base;                                  // 32 KiB
    unsigned char* k_tile[2] = {base + kTileBytes, base + 2 * kTileBytes};
    unsigned char* v_tile[2] = {base + 3 * kTileBytes, base + 4 * kTileBytes};
    unsigned char* p_tile = base + 5 * kTileBytes;                 // 32 KiB
    __shared__ __align__(8) uint64_t q_full, k_full[2], k_empty[2], v_full[2], v_empty[2], s_full[2], s_empty[2],
        p_full, p_empty, o_full[2], o_empty[2];
    __shared__ uint32_t tmem_slot;
    __shared__ volatile int failed;
    __shared__ volatile float xchg[2][2][kRows];   // [tile parity][column half][row]: partial row maxima; sums at the end
    __shared__ volatile int xflag[2][2][kRows];    // tile number + 1 for which xchg holds a value

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int4 td = a.tiles[gridDim.x - 1 - blockIdx.x];           // longest tiles (latest queries) first
    const int tok0 = td.x, rows = td.y, pos0 = td.z, req = td.w;
    const int h = blockIdx.y, hk = h / (a.heads / a.kv_heads);
    const int pos_last = pos0 + rows - 1;
    const int lo0 = a.window > 0 ? max(0, pos0 - a.window + 1) : 0;
    const int k_begin = lo0 & ~(kKeys - 1);
    const int n_tiles = (pos_last - k_begin) / kKeys + 1;

    if (threadIdx.x == 0) {
        mbar_init(&q_full, 1);
        for (int s = 0; s < 2; ++s) {
            mbar_init(&k_full[s], 1); mbar_init(&k_empty[s], 1); mbar_init(&v_full[s], 1); mbar_init(&v_empty[s], 1);
            mbar_init(&s_full[s], 1); mbar_init(&s_empty[s], kSoftmaxThreads); mbar_init(&o_full[s], 1); mbar_init(&o_empty[s], kSoftmaxThreads);
        }
        mbar_init(&p_full, kSoftmaxThreads);
        mbar_init(&p_empty, 1);
        failed = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    for (int i = threadIdx.x; i < 2 * 2 * kRows; i += kThreads) (&xflag[0][0][0])[i] = 0;
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_slot)), "r"(kTmemCols));
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::);
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = tmem_slot;
    pdl_trigger();
    pdl_wait();            // queries, keys and values all come from the kernels before this one

    if (warp == 0) {
        // ---- loads: lane 0 keeps the barriers, lane p fetches page p of every tile (its block-table entry
        //      and the four boxes of that page: K and V, two 64-dim halves each) ----------------------------
        if (lane == 0) {
            mbar_expect_tx(&q_full, kTileBytes);
            tma_load_2d(q_tile, &map_q, &q_full, h * kDim, tok0);
            tma_load_2d(q_tile + kHalfBytes, &map_q, &q_full, h * kDim + 64, tok0);
        }
        const int* table = a.block_table + (size_t)req * a.table_width;
        const int ps = a.page_size, pages_per_tile = kKeys / ps;
        int page = 0;
        if (lane < pages_per_tile) page = table[min(k_begin / ps + lane, a.table_width - 1)];
        for (int j = 0; j < n_tiles; ++j) {
            const int s = j & 1;
            int ok = 1;
            if (lane == 0) {
                if (j >= 2 && (!mbar_wait(&k_empty[s], ((j >> 1) - 1) & 1) || !mbar_wait(&v_empty[s], ((j >> 1) - 1) & 1))) {
                    attn_give_up(1); failed = 1; ok = 0;
                } else {
                    mbar_expect_tx(&k_full[s], kTileBytes);
                    mbar_expect_tx(&v_full[s], kTileBytes);
                }
            }
            ok = __shfl_sync(0xffffffffu, ok, 0);
            if (!ok) break;
            if (lane < pages_per_tile) {
                const int row = (page * 2 * a.kv_heads + hk) * ps;               // K rows of this page; V rows kv_heads * ps further
                unsigned char* kd = k_tile[s] + lane * ps * 128;
                unsigned char* vd = v_tile[s] + lane * ps * 128;
                tma_load_2d(kd, &map_kv, &k_full[s], 0, row);
                tma_load_2d(kd + kHalfBytes, &map_kv, &k_full[s], 64, row);
                tma_load_2d(vd, &map_kv, &v_full[s], 0, row + a.kv_heads * ps);
                tma_load_2d(vd + kHalfBytes, &map_kv, &v_full[s], 64, row + a.kv_heads * ps);
                // the next tile's page id (keys past the request's end are masked: any valid page will do)
                if (j + 1 < n_tiles) page = table[min((k_begin + (j + 1) * kKeys) / ps + lane, a.table_width - 1)];
            }
        }
    } else if (warp == 1 && lane == 0) {
        // ---- MMA issuer --------------------------------------------------------------------------
        constexpr uint32_t idesc_s = umma_idesc(kRows, kKeys);                         // Q, K both K-major
        constexpr uint32_t idesc_o = umma_idesc(kRows, kDim) | (1u << 16);             // P K-major, V MN-major
        bool ok = mbar_wait(&q_full, 0);
        if (!ok) { attn_give_up(2); failed = 1; }
        auto issue_pv = [&](int i) {
            const int s = i & 1;
            if (!mbar_wait(&v_full[s], (i >> 1) & 1) || !mbar_wait(&p_full, i & 1) ||
                (i >= 2 && !mbar_wait(&o_empty[s], ((i >> 1) - 1) & 1))) { attn_give_up(3); failed = 1; return false; }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
            for (int kk = 0; kk < kKeys / 16; ++kk) {
                const uint64_t da = umma_desc(p_tile + (kk >> 2) * kHalfBytes) + 2 * (kk & 3);
                const uint64_t db = umma_desc_mn(v_tile[s] + kk * 16 * 128, kHalfBytes);
                umma_f16(tmem + 256 + s * 128, da, db, idesc_o, kk > 0 ? 1u : 0u);
            }
            umma_commit(&v_empty[s]);
            umma_commit(&p_empty);
            umma_commit(&o_full[s]);
            return true;
        };
        for (int j = 0; j < n_tiles && ok; ++j) {
            const int s = j & 1;
            if (!mbar_wait(&k_full[s], (j >> 1) & 1) || (j >= 2 && !mbar_wait(&s_empty[s], ((j >> 1) - 1) & 1))) {
                attn_give_up(4); failed = 1; ok = false; break;
            }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
            for (int kk = 0; kk < kDim / 16; ++kk) {
                const uint64_t da = umma_desc(q_tile + (kk >> 2) * kHalfBytes) + 2 * (kk & 3);
                const uint64_t db = umma_desc(k_tile[s] + (kk >> 2) * kHalfBytes) + 2 * (kk & 3);
                umma_f16(tmem + s * 128, da, db, idesc_s, kk > 0 ? 1u : 0u);
            }
            umma_commit(&k_empty[s]);
            umma_commit(&s_full[s]);
            if (j >= 1) ok = issue_pv(j - 1);
        }
        if (ok) issue_pv(n_tiles - 1);
    } else if (warp >= 2) {
        // ---- softmax, accumulation, output: two threads per query row, 64 columns each --------------
        const int quarter = warp & 3;                  // TMEM lanes [32 * quarter, +32) are readable by this warp
        const int half = (warp - 2) >> 2;              // which 64 keys of a tile / which 64 output dims
        const int row = quarter * 32 + lane;
        const uint32_t lane_addr = tmem + ((uint32_t)(quarter * 32) << 16) + half * kCols;
        const int row_pos = pos0 + row;
        const int row_lo = a.window > 0 ? row_pos - a.window + 1 : 0;
        unsigned char* p_half = p_tile + half * kHalfBytes;
        float acc[kCols];
#pragma unroll
        for (int d = 0; d < kCols; ++d) acc[d] = 0.f;
        float m = -INFINITY, l = 0.f, corr_prev = 1.f;
        bool ok = true;
        // The two threads of a row hand each other a value through shared memory: write it, publish the tile
        // number, wait (bounded) for the partner's.  No block-wide barrier, so a thread that gave up cannot
        // leave its partner stuck.
        auto exchange = [&](int buf, int stamp, float mine, float& theirs) {
            xchg[buf][half][row] = mine;
            __threadfence_block();
            xflag[buf][half][row] = stamp;
            for (uint32_t i = 0; i < kSpinLimit; ++i) {
                if (xflag[buf][half ^ 1][row] == stamp) {
                    __threadfence_block();
                    theirs = xchg[buf][half ^ 1][row];
                    return true;
                }
            }
            return false;
        };
        auto fold = [&](int i, float corr) {          // acc = acc * corr + O_tile(i), this thread's 64 dims
            const int s = i & 1;
            if (!mbar_wait(&o_full[s], (i >> 1) & 1)) { attn_give_up(5); failed = 1; return false; }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            uint32_t r[kCols];
            load_cols(lane_addr + 256 + s * 128, r);
#pragma unroll
            for (int c = 0; c < kCols; ++c) acc[c] = fmaf(acc[c], corr, __uint_as_float(r[c]));
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            mbar_arrive(&o_empty[s]);
            return true;
        };
        for (int j = 0; j < n_tiles; ++j) {
            const int s = j & 1, k0 = k_begin + j * kKeys + half * kCols;
            if (!mbar_wait(&s_full[s], (j >> 1) & 1)) { attn_give_up(6); failed = 1; ok = false; break; }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const int t0 = k_begin + j * kKeys;
            const bool need_mask = (t0 + kKeys - 1 > pos0) || (a.window > 0 && t0 < pos_last - a.window + 1);
            const uint32_t s_addr = lane_addr + s * 128;
            uint32_t sc[kCols];
            load_cols(s_addr, sc);
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            mbar_arrive(&s_empty[s]);                                    // S of this buffer is in registers now
            float mx = need_mask ? row_max<true>(sc, k0, row_pos, row_lo) : row_max<false>(sc, k0, row_pos, row_lo);
            float other;
            if (!exchange(s, j + 1, mx, other)) { attn_give_up(8); failed = 1; ok = false; break; }
            mx = fmaxf(mx, other);
            const float m_new = fmaxf(m, mx * a.sl);
            const float mu = m_new == -INFINITY ? 0.f : m_new;      // a row with no visible key yet
            const float corr = ex2(m - mu);
            m = m_new;
            // the P tile is free once P V of the previous tile has read it
            if (j >= 1 && !mbar_wait(&p_empty, (j - 1) & 1)) { attn_give_up(7); failed = 1; ok = false; break; }
            const float sum = need_mask ? row_exp<true>(sc, p_half, row, a.sl, mu, k0, row_pos, row_lo)
                                        : row_exp<false>(sc, p_half, row, a.sl, mu, k0, row_pos, row_lo);
            l = l * corr + sum;
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // P must be visible to the tensor core
            mbar_arrive(&p_full);
            if (j >= 1 && !fold(j - 1, corr_prev)) { ok = false; break; }
            corr_prev = corr;
        }
        if (ok) ok = fold(n_tiles - 1, corr_prev);
        // the row sum is the two halves' sums (both are relative to the same running maximum)
        float l_other = 0.f;
        if (ok && !exchange(0, n_tiles + 1, l, l_other)) { attn_give_up(9); failed = 1; ok = false; }
        if (ok && !failed && row < rows) {
            const float inv = 1.0f / (l + l_other);
            bf16* dst = a.out + (size_t)(tok0 + row) * a.out_stride + (size_t)h * kDim + half * kCols;
#pragma unroll
            for (int d = 0; d < kCols; d += 8) {
                *reinterpret_cast<uint4*>(dst + d) =
                    make_uint4(pack2(acc[d] * inv, acc[d + 1] * inv), pack2(acc[d + 2] * inv, acc[d + 3] * inv),
                               pack2(acc[d + 4] * inv, acc[d + 5] * inv), pack2(acc[d + 6] * inv, acc[d + 7] * inv));
            }
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(kTmemCols));
    }
}

}  // namespace

// 1 if the tcgen05 prefill kernel takes this geometry.
LLM_API int llm_attention_tcgen05_supported(int heads, int kv_heads, int head_dim, int page_size) {
    return head_dim == 128 && kv_heads > 0 && heads % kv_heads == 0 && page_size >= 8 && page_size <= 128 &&
           (128 % page_size) == 0;
}

// q: [tokens, q_stride] bf16 with head h at columns [h * 128, h * 128 + 128); cache layer [pages, 2, kv_heads, page, 128];
// tiles: [n_tiles] int4 {first token row, rows (<= 128), position of the first row, request}.
LLM_API int llm_attention_prefill_tcgen05(const void* q, int q_stride, int tokens, const void* cache, long long cache_pages,
                                          const int* block_table, int table_width, const int* tiles, int n_tiles,
                                          void* out, int out_stride, int heads, int kv_heads, int head_dim,
                                          int page_size, int window, float scale, cudaStream_t stream) {
    if (n_tiles == 0) return 0;
    if (!llm_attention_tcgen05_supported(heads, kv_heads, head_dim, page_size))
        LLM_FAIL(-1, "attention_prefill_tcgen05: heads %d / kv_heads %d / head_dim %d / page %d not supported", heads,
                 kv_heads, head_dim, page_size);
    if (heads > 65535) LLM_FAIL(-1, "attention_prefill_tcgen05: too many heads");
    if (out_stride % 8) LLM_FAIL(-1, "attention_prefill_tcgen05: out_stride must be a multiple of 8");
    CUtensorMap mq, mkv;
    if (int rc = llm_tensor_map_2d(q, (uint64_t)tokens, (uint64_t)q_stride, kRows, 64, &mq)) return rc;
    const uint64_t kv_rows = (uint64_t)cache_pages * 2 * kv_heads * page_size;
    if (kv_rows > 0x7fffffffull) LLM_FAIL(-1, "attention_prefill_tcgen05: the cache layer has too many rows for 32-bit TMA coordinates");
    if (int rc = llm_tensor_map_2d(cache, kv_rows, kDim, (uint32_t)page_size, 64, &mkv)) return rc;
    AttnArgs a;
    a.block_table = block_table;
    a.table_width = table_width;
    a.tiles = (const int4*)tiles;
    a.out = (bf16*)out;
    a.out_stride = out_stride;
    a.heads = heads;
    a.kv_heads = kv_heads;
    a.page_size = page_size;
    a.window = window;
    a.sl = scale * 1.4426950408889634f;
    const size_t smem = 6 * kTileBytes + 1024;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(attn_prefill_tcgen05_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) LLM_FAIL(-2, "attention_prefill_tcgen05: %s", cudaGetErrorString(e));
        configured = true;
    }
    llm_launch(attn_prefill_tcgen05_kernel, dim3(n_tiles, heads), kThreads, smem, stream, mq, mkv, a);
    LLM_CHECK_LAUNCH("attention_prefill_tcgen05");
    return 0;
}

LLM_API int llm_attention_tcgen05_status() {
    int v = 0, zero = 0;
    if (cudaMemcpyFromSymbol(&v, g_attn_status, sizeof(int)) != cudaSuccess) return -1;
    if (v) cudaMemcpyToSymbol(g_attn_status, &zero, sizeof(int));
    return v;
}
