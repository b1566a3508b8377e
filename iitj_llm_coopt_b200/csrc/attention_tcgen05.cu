// Paged causal attention for prompt portions on the fifth-generation tensor cores
// (bfloat16, head sizes 64 and 128, page sizes 8 .. 128 that divide 128).
//
// One CTA = 128 query positions of one request x two query heads of one key/value group (the last head of
// a group with an odd number of heads runs alone).  Both heads see the same keys, so every key/value tile
// is loaded once for two tiles of scores, and the two heads' chains (scores -> softmax -> P V) run in
// ping-pong: while the softmax warps of one head work, the tensor core serves the other.  Keys and values
// walk through shared memory in tiles of 128 keys; each page of a tile is one TMA box per 64-dim half,
// placed at its row offset of the 128-byte-swizzled tile, so the paged cache needs no gather pass.
//
//   S = Q K^T      tcgen05.mma, M = 128 queries, N = 128 keys, K = the head's dims, both operands K-major in
//                  shared memory; S lands in tensor memory (128 float32 columns per head).
//   softmax        four warps per head, one thread per query row: it reads its row of S with tcgen05.ld (a
//                  TMEM lane is a row: no shuffles), masks by position, takes the maximum, exponentiates in
//                  float32 and writes P as bfloat16 back over the first 64 columns of S (tcgen05.st).
//   O += P V       tcgen05.mma with P read from tensor memory and V MN-major from shared memory (a key's
//                  dims are contiguous, so the V tile is used as it was loaded); O stays in tensor memory for
//                  the whole sequence of key tiles.
//   rescaling      P is taken relative to a running maximum that is only moved when a row's maximum has
//                  grown by more than 2^8; then, and only then, the row of O is read, scaled and written
//                  back before the next P V.  The sum l follows the same reference, so O / l is exact.
//
// Replaces flash_attn_varlen_func (engine/model.py:204-207) for portions; same masking and float32
// statistics as the mma.sync kernel of attention_bf16.cu, which remains for page sizes that do not divide 128.
//
// Every mbarrier wait is bounded; a wait that runs out records a code (llm_attention_tcgen05_status)
// and the CTA falls through to its teardown, where the tensor memory is freed.
#include "tcgen05_common.cuh"

#include <cstdlib>
#include <type_traits>

namespace {

typedef __nv_bfloat16 bf16;

constexpr int kRows = 128;        // queries per CTA and head (UMMA M)
constexpr int kKeys = 128;        // keys per tile
constexpr int kHalfBytes = 128 * 128;          // 64 dims of 128 rows (queries or keys) as bf16: 128 rows x 128 bytes
template <int D> __host__ __device__ constexpr int tile_bytes() { return (D / 64) * kHalfBytes; }   // a [128 x D] tile: 16 or 32 KiB
constexpr int kThreads = 320;     // warp 0: loads, warp 1: MMA + TMEM, warps 2-5: softmax of head A, warps 6-9: of head B
constexpr int kGroupThreads = 128;
constexpr uint32_t kTmemCols = 512;            // S_A | S_B | O_A | O_B, 128 float32 columns each (O uses the head's dims)
#ifndef LLM_ATTN_V_STAGES
#define LLM_ATTN_V_STAGES 3
#endif
constexpr int kVStages = LLM_ATTN_V_STAGES;       // shared-memory stages of value tiles (the keys have two)
constexpr int kMinSplitTiles = 16;              // key tiles per split, about (the count of splits is rounded)
constexpr float kRescaleStep = 8.0f;           // in log2 units: P stays below 2^8
constexpr float kOnePassLimit = 100.0f;        // a one-pass tile whose maximum is this far above the reference is void (status 9)

__device__ int g_attn_status = 0;
__device__ __forceinline__ void attn_give_up(int code) { atomicCAS(&g_attn_status, 0, (code << 16) | (int)(blockIdx.x & 0xffff)); }

__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

__device__ __forceinline__ float ex2(float x) {          // 2^x; one MUFU instruction
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
          "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]) : "memory");
}
// D[tmem] (+)= A[tmem] . B[smem]: the A operand (P) is read from tensor memory.
__device__ __forceinline__ void umma_f16_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
        ::"r"(tmem_d), "r"(tmem_a), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}

// Packed float32 pairs (sm_100: one instruction multiplies-and-adds, or adds, two values) and the three-input maximum:
// they halve the instruction count of the softmax's arithmetic, which shares its issue slots with the exponentials.
__device__ __forceinline__ unsigned long long pair_of(float lo, float hi) {
    unsigned long long r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
    return r;
}
__device__ __forceinline__ unsigned long long pair_of_bits(uint32_t lo, uint32_t hi) {
    unsigned long long r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "r"(lo), "r"(hi));
    return r;
}
__device__ __forceinline__ void split_pair(unsigned long long v, float& lo, float& hi) {
    asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ unsigned long long fma_pair(unsigned long long a, unsigned long long b, unsigned long long c) {
    unsigned long long r;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
    return r;
}
__device__ __forceinline__ unsigned long long add_pair(unsigned long long a, unsigned long long b) {
    unsigned long long r;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
    return r;
}
__device__ __forceinline__ float max3(float a, float b, float c) {
    float r;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(b), "f"(c));
    return r;
}

// Maximum of 32 scores (keys k0 .. k0+31) with four independent chains.
template <bool MASK>
__device__ __forceinline__ float chunk_max(const uint32_t (&r)[32], int k0, int row_pos, int row_lo, float mx) {
    float m0 = mx, m1 = -INFINITY, m2 = -INFINITY, m3 = -INFINITY;
    if constexpr (!MASK) {
#pragma unroll
        for (int c = 0; c < 32; c += 8) {
            m0 = max3(m0, __uint_as_float(r[c]), __uint_as_float(r[c + 1]));
            m1 = max3(m1, __uint_as_float(r[c + 2]), __uint_as_float(r[c + 3]));
            m2 = max3(m2, __uint_as_float(r[c + 4]), __uint_as_float(r[c + 5]));
            m3 = max3(m3, __uint_as_float(r[c + 6]), __uint_as_float(r[c + 7]));
        }
    } else {
#pragma unroll
        for (int c = 0; c < 32; c += 4) {
            float a0 = __uint_as_float(r[c]), a1 = __uint_as_float(r[c + 1]), a2 = __uint_as_float(r[c + 2]), a3 = __uint_as_float(r[c + 3]);
            const int key = k0 + c;
            if (key > row_pos || key < row_lo) a0 = -INFINITY;
            if (key + 1 > row_pos || key + 1 < row_lo) a1 = -INFINITY;
            if (key + 2 > row_pos || key + 2 < row_lo) a2 = -INFINITY;
            if (key + 3 > row_pos || key + 3 < row_lo) a3 = -INFINITY;
            m0 = fmaxf(m0, a0); m1 = fmaxf(m1, a1); m2 = fmaxf(m2, a2); m3 = fmaxf(m3, a3);
        }
    }
    return fmaxf(fmaxf(m0, m1), fmaxf(m2, m3));
}

// P = 2^(S * sl - mu) of 32 scores, packed as 16 columns of two bfloat16; adds to four partial sums (sum[i] takes the
// keys i, i + 4, ... of the chunk in both forms, so a row's sum does not depend on whether its tile was masked).
template <bool MASK>
__device__ __forceinline__ void chunk_exp(const uint32_t (&r)[32], uint32_t (&packed)[16], float sl, float mu, int k0, int row_pos,
                                          int row_lo, float (&sum)[4]) {
    if constexpr (!MASK) {
        const unsigned long long sl2 = pair_of(sl, sl), nmu2 = pair_of(-mu, -mu);
        unsigned long long s01 = pair_of(sum[0], sum[1]), s23 = pair_of(sum[2], sum[3]);
#pragma unroll
        for (int c = 0; c < 32; c += 4) {
            float x0, x1, x2, x3;
            split_pair(fma_pair(pair_of_bits(r[c], r[c + 1]), sl2, nmu2), x0, x1);
            split_pair(fma_pair(pair_of_bits(r[c + 2], r[c + 3]), sl2, nmu2), x2, x3);
            const float p0 = ex2(x0), p1 = ex2(x1), p2 = ex2(x2), p3 = ex2(x3);
            s01 = add_pair(s01, pair_of(p0, p1));
            s23 = add_pair(s23, pair_of(p2, p3));
            packed[c >> 1] = pack2(p0, p1);
            packed[(c >> 1) + 1] = pack2(p2, p3);
        }
        split_pair(s01, sum[0], sum[1]);
        split_pair(s23, sum[2], sum[3]);
    } else {
#pragma unroll
        for (int c = 0; c < 32; c += 4) {
            float p0 = ex2(fmaf(__uint_as_float(r[c]), sl, -mu)), p1 = ex2(fmaf(__uint_as_float(r[c + 1]), sl, -mu));
            float p2 = ex2(fmaf(__uint_as_float(r[c + 2]), sl, -mu)), p3 = ex2(fmaf(__uint_as_float(r[c + 3]), sl, -mu));
            const int key = k0 + c;
            if (key > row_pos || key < row_lo) p0 = 0.f;
            if (key + 1 > row_pos || key + 1 < row_lo) p1 = 0.f;
            if (key + 2 > row_pos || key + 2 < row_lo) p2 = 0.f;
            if (key + 3 > row_pos || key + 3 < row_lo) p3 = 0.f;
            sum[0] += p0; sum[1] += p1; sum[2] += p2; sum[3] += p3;
            packed[c >> 1] = pack2(p0, p1);
            packed[(c >> 1) + 1] = pack2(p2, p3);
        }
    }
}

struct AttnArgs {
    const int* block_table;
    int table_width;
    const int4* tiles;            // {first token row, rows (<= 128), position of the first row, request}
    bf16* out;
    int out_stride;
    int heads, kv_heads, page_size, window;
    int splits;                   // CTAs along the keys of a query tile (> 1: partial results go to scratch, see attn_tc_merge_kernel)
    float* part_o;                // [tile][head][split][128 rows][128] float32, relative to the split's reference maximum
    float* part_ml;               // [tile][head][split][128 rows][2]: reference maximum (log2 units), sum
    int per_cta;                  // query heads per CTA: 2 (ping-pong), or 1 when that fills more of the GPU
    int pairs;                    // CTAs per key/value group: ceil(heads per group / per_cta)
    float sl;                     // softmax scale * log2(e)
    int one_pass;                 // tiles after a request's first: one softmax pass (see the kernel); 0: always two (IITJ_ATTN_ONE_PASS=0)
};

template <int D>
__global__ void __launch_bounds__(kThreads, 1)
attn_prefill_tcgen05_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_kv,
                            const AttnArgs a) {
    extern __shared__ unsigned char smem_raw[];
    constexpr int kDim = D, kTileBytes = tile_bytes<D>(), kHalves = D / 64;
    static_assert(D == 64 || D == 128, "head sizes 64 and 128");
    unsigned char* base = reinterpret_cast<unsigned char*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    unsigned char* q_tile[2] = {base, base + kTileBytes};                          // head A, head B
    unsigned char* k_tile[2] = {base + 2 * kTileBytes, base + 3 * kTileBytes};
    // Three stages for the values: a value tile is handed back only when both heads' P V of its keys are done, one
    // tile's time after the keys' stage, and with two stages its successor's boxes came in about 300 clocks late every tile.
    unsigned char* v_tile[3] = {base + 4 * kTileBytes, base + 5 * kTileBytes, base + 6 * kTileBytes};   // (the last only with three stages)
    __shared__ __align__(8) uint64_t q_full, k_full[2], k_empty[2], v_full[kVStages], v_empty[kVStages], s_full[2], p_full[2], o_done[2];
    __shared__ uint32_t tmem_slot;
    __shared__ volatile int failed;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // Blocks are handed out with x running fastest: the block's number in that order is cut so that all heads of
    // one query tile follow each other, and the tiles are taken from the end of the list (sorted by context on the
    // host): the tiles with the most keys start first, the short ones fill the gaps at the end of the launch.
    const unsigned lin = blockIdx.x + gridDim.x * blockIdx.y;
    const int tile_id = (int)gridDim.x - 1 - (int)(lin / gridDim.y), by = (int)(lin % gridDim.y);
    const int4 td = a.tiles[tile_id];
    const int tok0 = td.x, rows = td.y, pos0 = td.z, req = td.w;
    const int group = a.heads / a.kv_heads;
    const int hk = by / a.pairs, pr = by - hk * a.pairs;
    const int head_a = hk * group + a.per_cta * pr;
    const int n_heads = (a.per_cta == 2 && 2 * pr + 1 < group) ? 2 : 1;      // heads this CTA serves
    const int pos_last = pos0 + rows - 1;
    const int lo0 = a.window > 0 ? max(0, pos0 - a.window + 1) : 0;
    // this CTA's share of the query tile's key tiles (all of them without splits)
    const int split = blockIdx.z;
    const int k_first = lo0 & ~(kKeys - 1);
    const int all_tiles = (pos_last - k_first) / kKeys + 1;
    // the launch allows a.splits CTAs per tile and head; a tile uses as many as leave each about 16 key tiles or more
    // (decided here, from the tile's own context, so that a captured graph follows a prompt as it grows)
    const int eff_splits = max(1, min(a.splits, (all_tiles + kMinSplitTiles / 2) / kMinSplitTiles));
    const int per_split = (all_tiles + eff_splits - 1) / eff_splits;
    const int k_begin = k_first + split * per_split * kKeys;
    const int n_tiles = split < eff_splits ? max(0, min(all_tiles - split * per_split, per_split)) : 0;

    if (n_tiles == 0) return;      // a split past the end of this tile's keys: nothing to do (the merge leaves it out by index)

    if (threadIdx.x == 0) {
        mbar_init(&q_full, 1);
        for (int s = 0; s < 2; ++s) {
            mbar_init(&k_full[s], 1); mbar_init(&k_empty[s], 1);
            mbar_init(&s_full[s], 1); mbar_init(&p_full[s], kGroupThreads / 32); mbar_init(&o_done[s], 1);
        }
        for (int s = 0; s < kVStages; ++s) { mbar_init(&v_full[s], 1); mbar_init(&v_empty[s], 1); }
        failed = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
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
        //      and the boxes of that page: K and V, one per 64 dims) --------------------------------------
        if (lane == 0) {
            mbar_expect_tx(&q_full, n_heads * kTileBytes);
            for (int x = 0; x < n_heads; ++x) {
#pragma unroll
                for (int h = 0; h < kHalves; ++h)
                    tma_load_2d(q_tile[x] + h * kHalfBytes, &map_q, &q_full, (head_a + x) * kDim + 64 * h, tok0);
            }
        }
        const int* table = a.block_table + (size_t)req * a.table_width;
        const int ps = a.page_size, pages_per_tile = kKeys / ps;
        int page = 0;
        if (lane < pages_per_tile) page = table[min(k_begin / ps + lane, a.table_width - 1)];
        for (int j = 0; j < n_tiles; ++j) {
            const int s = j & 1, sv = j % kVStages;
            int ok = 1;
            if (lane == 0) {
                if ((j >= 2 && !mbar_wait(&k_empty[s], ((j >> 1) - 1) & 1)) ||
                    (j >= kVStages && !mbar_wait(&v_empty[sv], ((j / kVStages) - 1) & 1))) {
                    attn_give_up(1); failed = 1; ok = 0;
                } else {
                    mbar_expect_tx(&k_full[s], kTileBytes);
                    mbar_expect_tx(&v_full[sv], kTileBytes);
                }
            }
            ok = __shfl_sync(0xffffffffu, ok, 0);
            if (!ok) break;
            if (lane < pages_per_tile) {
                const int row = (page * 2 * a.kv_heads + hk) * ps;               // K rows of this page; V rows kv_heads * ps further
                unsigned char* kd = k_tile[s] + lane * ps * 128;
                unsigned char* vd = v_tile[sv] + lane * ps * 128;
#pragma unroll
                for (int h = 0; h < kHalves; ++h) {
                    tma_load_2d(kd + h * kHalfBytes, &map_kv, &k_full[s], 64 * h, row);
                    tma_load_2d(vd + h * kHalfBytes, &map_kv, &v_full[sv], 64 * h, row + a.kv_heads * ps);
                }
                // the next tile's page id (keys past the request's end are masked: any valid page will do)
                if (j + 1 < n_tiles) page = table[min((k_begin + (j + 1) * kKeys) / ps + lane, a.table_width - 1)];
            }
        }
    } else if (warp == 1 && lane == 0) {
        // ---- MMA issuer --------------------------------------------------------------------------
        // Order: S_A(0) S_B(0), then per key tile j: PV_A(j) S_A(j+1) PV_B(j) S_B(j+1).  The tensor core runs
        // its instructions in the order of issue, so S_x(j+1) overwrites P_x(j) only after PV_x(j) has read it.
        constexpr uint32_t idesc_s = umma_idesc(kRows, kKeys);                         // Q, K both K-major
        constexpr uint32_t idesc_o = umma_idesc(kRows, kDim) | (1u << 16);             // P from TMEM, V MN-major
        bool ok = mbar_wait(&q_full, 0);
        if (!ok) { attn_give_up(2); failed = 1; }
        // Descriptors are built once; inside the loops only constants are added.
        const uint64_t dq[2] = {umma_desc(q_tile[0]), umma_desc(q_tile[1])};
        const uint64_t dk[2] = {umma_desc(k_tile[0]), umma_desc(k_tile[1])};
        const uint64_t dv[3] = {umma_desc_mn(v_tile[0], kHalfBytes), umma_desc_mn(v_tile[1], kHalfBytes), umma_desc_mn(v_tile[2], kHalfBytes)};
        auto issue_s = [&](int x, int j) {
            const uint64_t da = x ? dq[1] : dq[0], db = (j & 1) ? dk[1] : dk[0];
#pragma unroll
            for (int kk = 0; kk < kDim / 16; ++kk) {
                const uint64_t off = (uint64_t)((kk >> 2) * (kHalfBytes >> 4) + 2 * (kk & 3));
                umma_f16(tmem + x * 128, da + off, db + off, idesc_s, kk > 0 ? 1u : 0u);
            }
            umma_commit(&s_full[x]);
        };
        auto issue_pv = [&](int x, int j) {
            if (!mbar_wait(&p_full[x], j & 1)) { attn_give_up(3); failed = 1; return false; }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const int sv = j % kVStages;
            const uint64_t db = sv == 0 ? dv[0] : sv == 1 ? dv[1] : dv[2];
#pragma unroll
            for (int kk = 0; kk < kKeys / 16; ++kk)
                umma_f16_ts(tmem + 256 + x * 128, tmem + x * 128 + kk * 8, db + (uint64_t)(kk * ((16 * 128) >> 4)), idesc_o,
                            (j > 0 || kk > 0) ? 1u : 0u);
            // The tensor core completes its instructions in the order of issue, so the scores of tile j + 1 being there
            // (s_full) tell the softmax warps that O holds tile j too; only after the last tile nothing follows.
            if (j == n_tiles - 1) umma_commit(&o_done[x]);
            return true;
        };
        if (ok) {
            if (!mbar_wait(&k_full[0], 0)) { attn_give_up(4); failed = 1; ok = false; }
        }
        if (ok) {
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            for (int x = 0; x < n_heads; ++x) issue_s(x, 0);
            umma_commit(&k_empty[0]);
        }
        for (int j = 0; j < n_tiles && ok; ++j) {
            const int s = j & 1, s1 = (j + 1) & 1;
            const bool more = j + 1 < n_tiles;
            if (!mbar_wait(&v_full[j % kVStages], (j / kVStages) & 1)) { attn_give_up(5); failed = 1; ok = false; break; }
            if (!(ok = issue_pv(0, j))) break;
            if (more) {
                if (!mbar_wait(&k_full[s1], ((j + 1) >> 1) & 1)) { attn_give_up(4); failed = 1; ok = false; break; }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                issue_s(0, j + 1);
            }
            if (n_heads == 2) {
                if (!(ok = issue_pv(1, j))) break;
                if (more) issue_s(1, j + 1);
            }
            umma_commit(&v_empty[j % kVStages]);
            if (more) umma_commit(&k_empty[s1]);
        }
    } else if (warp >= 2 && ((warp - 2) >> 2) < n_heads) {
        // ---- softmax and output: one thread per query row of one head ---------------------------------
        const int x = (warp - 2) >> 2;                 // head A or B
        const int quarter = warp & 3;                  // TMEM lanes [32 * quarter, +32) are readable by this warp
        const int row = quarter * 32 + lane;
        const uint32_t s_addr = tmem + ((uint32_t)(quarter * 32) << 16) + x * 128;
        const uint32_t o_addr = s_addr + 256;
        const int row_pos = pos0 + row;
        const int row_lo = a.window > 0 ? row_pos - a.window + 1 : 0;
        float m = -INFINITY, l = 0.f;                  // reference maximum (log2 units) and sum relative to it
        bool ok = true;
        for (int j = 0; j < n_tiles; ++j) {
            if (!mbar_wait(&s_full[x], j & 1)) { attn_give_up(6); failed = 1; ok = false; break; }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const int t0 = k_begin + j * kKeys;
            const bool need_mask = (t0 + kKeys - 1 > pos0) || (a.window > 0 && t0 < pos_last - a.window + 1);
            uint32_t ca[32], cb[32];
            float sums[4] = {0.f, 0.f, 0.f, 0.f};
            // A tile without masked keys, after the first one, when every row of the warp has a reference already: ONE
            // pass.  P is taken relative to the reference as it stands while the tile's maximum is taken on the way; only
            // if that maximum turns out more than the step above some row's reference (rare after the first tiles) are
            // the tile's P, the row's O and its sum scaled down afterwards, by a whole power of two (exact in bfloat16).
            if (a.one_pass && j > 0 && !need_mask && __all_sync(0xffffffffu, m != -INFINITY)) {
                float mx = -INFINITY;
                uint32_t packed[16];
                tmem_ld32(s_addr, ca);
#pragma unroll 1
                for (int c0 = 0; c0 < kKeys; c0 += 64) {
                    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                    tmem_ld32(s_addr + c0 + 32, cb);
                    mx = chunk_max<false>(ca, t0 + c0, row_pos, row_lo, mx);
                    chunk_exp<false>(ca, packed, a.sl, m, t0 + c0, row_pos, row_lo, sums);
                    tmem_st16(s_addr + (c0 >> 1), packed);
                    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                    if (c0 + 64 < kKeys) tmem_ld32(s_addr + c0 + 64, ca);
                    mx = chunk_max<false>(cb, t0 + c0 + 32, row_pos, row_lo, mx);
                    chunk_exp<false>(cb, packed, a.sl, m, t0 + c0 + 32, row_pos, row_lo, sums);
                    tmem_st16(s_addr + (c0 >> 1) + 16, packed);
                }
                float sum = (sums[0] + sums[1]) + (sums[2] + sums[3]);
                const float grown = mx * a.sl - m;
                if (__any_sync(0xffffffffu, grown > kRescaleStep)) {
                    // beyond this the exponentials above may have left float32's range: the result is void, and said to be
                    if (grown > kOnePassLimit) attn_give_up(9);
                    const int k = grown > kRescaleStep ? (int)fminf(ceilf(grown), 126.f) : 0;
                    const float f = __int_as_float((127 - k) << 23);            // 2^-k
                    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");   // P is read back below
                    // (O of the tiles so far is complete: the scores of this tile were issued after their P V)
#pragma unroll 1
                    for (int c = 0; c < kDim; c += 16) {
                        uint32_t o[16];
                        tmem_ld16(o_addr + c, o);
                        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
                        for (int i = 0; i < 16; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * f);
                        tmem_st16(o_addr + c, o);
                    }
#pragma unroll 1
                    for (int c = 0; c < kKeys / 2; c += 16) {
                        uint32_t pp[16];
                        tmem_ld16(s_addr + c, pp);
                        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
                        for (int i = 0; i < 16; ++i)
                            pp[i] = pack2(__uint_as_float(pp[i] << 16) * f, __uint_as_float(pp[i] & 0xffff0000u) * f);
                        tmem_st16(s_addr + c, pp);
                    }
                    l *= f;
                    sum *= f;
                    m += (float)k;
                }
                l += sum;
            } else {
            // Two passes over the row of S in chunks of 32 columns, each chunk's load issued while the chunk
            // before it is worked on: pass 1 takes the maximum, pass 2 exponentiates and writes P.
            auto pass_max = [&](auto tag) {
                constexpr bool MASK = decltype(tag)::value;
                float mx = -INFINITY;
                tmem_ld32(s_addr, ca);
#pragma unroll 1
                for (int c0 = 0; c0 < kKeys; c0 += 64) {
                    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                    tmem_ld32(s_addr + c0 + 32, cb);
                    mx = chunk_max<MASK>(ca, t0 + c0, row_pos, row_lo, mx);
                    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                    if (c0 + 64 < kKeys) tmem_ld32(s_addr + c0 + 64, ca);
                    mx = chunk_max<MASK>(cb, t0 + c0 + 32, row_pos, row_lo, mx);
                }
                return mx;
            };
            const float mx = need_mask ? pass_max(std::true_type{}) : pass_max(std::false_type{});
            tmem_ld32(s_addr, ca);                                   // pass 2's first chunk, in flight during the decision
            // move the reference only when the maximum has grown by more than the step (always from -inf)
            const float m_tile = mx * a.sl;
            const bool move = m_tile > m + kRescaleStep || (m == -INFINITY && m_tile > -INFINITY);
            if (j > 0 && __any_sync(0xffffffffu, move)) {
                // O of the tiles so far is complete (the scores of this tile were issued after their P V): its rows are scaled
                const float f = move ? ex2(m - m_tile) : 1.0f;      // 0 when the row had no visible key so far
#pragma unroll 1
                for (int c = 0; c < kDim; c += 16) {
                    uint32_t o[16];
                    tmem_ld16(o_addr + c, o);
                    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
                    for (int i = 0; i < 16; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * f);
                    tmem_st16(o_addr + c, o);
                }
                l *= f;
            }
            if (move) m = m_tile;
            const float mu = m == -INFINITY ? 0.f : m;      // a row with no visible key yet
            auto pass_exp = [&](auto tag) {
                constexpr bool MASK = decltype(tag)::value;
                uint32_t packed[16];
#pragma unroll 1
                for (int c0 = 0; c0 < kKeys; c0 += 64) {
                    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                    tmem_ld32(s_addr + c0 + 32, cb);
                    chunk_exp<MASK>(ca, packed, a.sl, mu, t0 + c0, row_pos, row_lo, sums);
                    tmem_st16(s_addr + (c0 >> 1), packed);           // keys c0 .. c0+31 as 16 columns of two bfloat16
                    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                    if (c0 + 64 < kKeys) tmem_ld32(s_addr + c0 + 64, ca);
                    chunk_exp<MASK>(cb, packed, a.sl, mu, t0 + c0 + 32, row_pos, row_lo, sums);
                    tmem_st16(s_addr + (c0 >> 1) + 16, packed);
                }
            };
            if (need_mask) pass_exp(std::true_type{}); else pass_exp(std::false_type{});
            const float sum = (sums[0] + sums[1]) + (sums[2] + sums[3]);
            l += sum;
            }
            asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(&p_full[x]);              // one arrival per warp
        }
        if (ok && !mbar_wait(&o_done[x], 0)) { attn_give_up(8); failed = 1; ok = false; }
        if (ok && !failed && eff_splits > 1) {
            // partial result of this split: O as it stands (relative to m), and (m, l) of the row
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const size_t slot = ((size_t)tile_id * a.heads + head_a + x) * a.splits + split;
            float* dst = a.part_o + (slot * kRows + row) * kDim;
#pragma unroll 1
            for (int c = 0; c < kDim; c += 32) {
                uint32_t o[32];
                tmem_ld32(o_addr + c, o);
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                if (row < rows) {
#pragma unroll
                    for (int d = 0; d < 32; d += 4)
                        *reinterpret_cast<uint4*>(dst + c + d) = make_uint4(o[d], o[d + 1], o[d + 2], o[d + 3]);
                }
            }
            if (row < rows) {
                a.part_ml[(slot * kRows + row) * 2] = m;
                a.part_ml[(slot * kRows + row) * 2 + 1] = l;
            }
        } else if (ok && !failed) {
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const float inv = 1.0f / l;
            bf16* dst = a.out + (size_t)(tok0 + row) * a.out_stride + (size_t)(head_a + x) * kDim;
#pragma unroll 1
            for (int c = 0; c < kDim; c += 32) {
                uint32_t o[32];
                tmem_ld32(o_addr + c, o);
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                if (row < rows) {
#pragma unroll
                    for (int d = 0; d < 32; d += 8)
                        *reinterpret_cast<uint4*>(dst + c + d) =
                            make_uint4(pack2(__uint_as_float(o[d]) * inv, __uint_as_float(o[d + 1]) * inv),
                                       pack2(__uint_as_float(o[d + 2]) * inv, __uint_as_float(o[d + 3]) * inv),
                                       pack2(__uint_as_float(o[d + 4]) * inv, __uint_as_float(o[d + 5]) * inv),
                                       pack2(__uint_as_float(o[d + 6]) * inv, __uint_as_float(o[d + 7]) * inv));
                }
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

// Adds the partial results of a query tile's key splits: out = sum_s O_s 2^(m_s - M) / sum_s l_s 2^(m_s - M).
// One block per (query row, head), one thread per output dim, all loads asked for at
// once; splits that got no key tile are left out by index; a tile that was not split needs nothing.
constexpr int kMaxKeySplits = 16;
constexpr int kMergeRows = 1;

template <int D>
__global__ void __launch_bounds__(D)
attn_tc_merge_kernel(const AttnArgs a) {
    constexpr int kDim = D;
    pdl_trigger();
    pdl_wait();
    const int tile_id = blockIdx.x / (kRows / kMergeRows), row0 = (blockIdx.x % (kRows / kMergeRows)) * kMergeRows;
    const int head = blockIdx.y, d = threadIdx.x, sub = 0;
    const int4 td = a.tiles[tile_id];
    const int tok0 = td.x, rows = td.y, pos0 = td.z;
    const int pos_last = pos0 + rows - 1;
    const int lo0 = a.window > 0 ? max(0, pos0 - a.window + 1) : 0;
    const int all_tiles = (pos_last - (lo0 & ~(kKeys - 1))) / kKeys + 1;
    const int eff_splits = max(1, min(a.splits, (all_tiles + kMinSplitTiles / 2) / kMinSplitTiles));
    if (eff_splits == 1) return;                                   // the one CTA wrote the result itself
    const int per_split = (all_tiles + eff_splits - 1) / eff_splits;
    const int n_valid = (all_tiles + per_split - 1) / per_split;
    const size_t slot0 = ((size_t)tile_id * a.heads + head) * a.splits;
    for (int row = row0 + sub; row < min(rows, row0 + kMergeRows); ++row) {
        float pm[kMaxKeySplits], pl[kMaxKeySplits], po[kMaxKeySplits];
#pragma unroll
        for (int s = 0; s < kMaxKeySplits; ++s) {
            if (s < n_valid) {
                pm[s] = a.part_ml[((slot0 + s) * kRows + row) * 2];
                pl[s] = a.part_ml[((slot0 + s) * kRows + row) * 2 + 1];
                po[s] = a.part_o[((slot0 + s) * kRows + row) * kDim + d];
            }
        }
        float M = -INFINITY;
#pragma unroll
        for (int s = 0; s < kMaxKeySplits; ++s)
            if (s < n_valid) M = fmaxf(M, pm[s]);
        float L = 0.f, O = 0.f;
#pragma unroll
        for (int s = 0; s < kMaxKeySplits; ++s) {
            if (s < n_valid) {
                const float f = pm[s] == -INFINITY ? 0.f : exp2f(pm[s] - M);
                L += pl[s] * f;
                O += po[s] * f;
            }
        }
        a.out[(size_t)(tok0 + row) * a.out_stride + (size_t)head * kDim + d] = __float2bfloat16_rn(O / L);
    }
}

}  // namespace

// 1 if the tcgen05 prefill kernel takes this geometry.
LLM_API int llm_attention_tcgen05_supported(int heads, int kv_heads, int head_dim, int page_size) {
    return (head_dim == 64 || head_dim == 128) && kv_heads > 0 && heads % kv_heads == 0 && page_size >= 8 && page_size <= 128 &&
           (128 % page_size) == 0;
}

// q: [tokens, q_stride] bf16 with head h at columns [h * head_dim, (h + 1) * head_dim); cache layer [pages, 2, kv_heads, page, head_dim];
// tiles: [n_tiles] int4 {first token row, rows (<= 128), position of the first row, request}.
LLM_API int llm_attention_prefill_tcgen05(const void* q, int q_stride, int tokens, const void* cache, long long cache_pages,
                                          const int* block_table, int table_width, const int* tiles, int n_tiles,
                                          void* out, int out_stride, int heads, int kv_heads, int head_dim,
                                          int page_size, int window, float scale, int splits, float* part_o,
                                          float* part_ml, cudaStream_t stream) {
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
    if (int rc = llm_tensor_map_2d(cache, kv_rows, (uint64_t)head_dim, (uint32_t)page_size, 64, &mkv)) return rc;
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
    static const int one_pass = [] { const char* e = getenv("IITJ_ATTN_ONE_PASS"); return (e && e[0] == '0') ? 0 : 1; }();
    a.one_pass = one_pass;
    // Two heads per CTA share each key/value tile and keep the tensor core busier; with few CTAs one head per
    // CTA spreads the work over more SMs (512 queries over 8192 keys at 32 heads: 168 -> 125 us).
    int dev = 0, sms = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    const int group = heads / kv_heads;
    a.per_cta = (group >= 2 && (long long)n_tiles * kv_heads * ((group + 1) / 2) * splits >= sms) ? 2 : 1;
    static const int forced = [] { const char* e = getenv("IITJ_ATTN_HEADS_PER_CTA"); return e ? atoi(e) : 0; }();   // measurements
    if (forced == 1 || (forced == 2 && group >= 2)) a.per_cta = forced;
    a.pairs = (group + a.per_cta - 1) / a.per_cta;
    const size_t smem = (4 + kVStages) * (size_t)(head_dim == 64 ? tile_bytes<64>() : tile_bytes<128>()) + 1024;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(attn_prefill_tcgen05_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             (4 + kVStages) * tile_bytes<128>() + 1024);
        if (e == cudaSuccess)
            e = cudaFuncSetAttribute(attn_prefill_tcgen05_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     (4 + kVStages) * tile_bytes<64>() + 1024);
        if (e != cudaSuccess) LLM_FAIL(-2, "attention_prefill_tcgen05: %s", cudaGetErrorString(e));
        configured = true;
    }
    if (splits < 1 || splits > kMaxKeySplits) LLM_FAIL(-1, "attention_prefill_tcgen05: splits %d out of range (1..%d)", splits, kMaxKeySplits);
    if (splits > 1 && (!part_o || !part_ml)) LLM_FAIL(-1, "attention_prefill_tcgen05: key splits need scratch");
    a.splits = splits;
    a.part_o = part_o;
    a.part_ml = part_ml;
    const dim3 grid(n_tiles, kv_heads * a.pairs, splits), merge_grid(n_tiles * (kRows / kMergeRows), heads);
    if (head_dim == 64) llm_launch(attn_prefill_tcgen05_kernel<64>, grid, kThreads, smem, stream, mq, mkv, a);
    else llm_launch(attn_prefill_tcgen05_kernel<128>, grid, kThreads, smem, stream, mq, mkv, a);
    LLM_CHECK_LAUNCH("attention_prefill_tcgen05");
    if (splits > 1) {
        if (head_dim == 64) llm_launch(attn_tc_merge_kernel<64>, merge_grid, 64, 0, stream, a);
        else llm_launch(attn_tc_merge_kernel<128>, merge_grid, 128, 0, stream, a);
        LLM_CHECK_LAUNCH("attention_prefill_tcgen05 merge");
    }
    return 0;
}

const int* llm_attention_tcgen05_status_word() {
    void* p = nullptr;
    return cudaGetSymbolAddress(&p, g_attn_status) == cudaSuccess ? static_cast<const int*>(p) : nullptr;
}

LLM_API int llm_attention_tcgen05_status() {
    int v = 0, zero = 0;
    if (cudaMemcpyFromSymbol(&v, g_attn_status, sizeof(int)) != cudaSuccess) return -1;
    if (v) cudaMemcpyToSymbol(g_attn_status, &zero, sizeof(int));
    return v;
}

LLM_TRACE_EXPORT(attention_tcgen05)
