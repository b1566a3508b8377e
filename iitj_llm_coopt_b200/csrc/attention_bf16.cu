// bfloat16 paged attention on the tensor cores (mma.sync m16n8k16, float32 accumulation),
// head sizes 64 and 128, groups of up to 16 query heads per key/value head.
//
//   attn_prefill_kernel  prompt portions: one CTA = 64 queries of one request x one query head;
//                        keys/values walk through shared memory in tiles of 64 keys fetched
//                        page by page with cp.async (any page size); online softmax in float32;
//                        causal mask by position, optional sliding window.
//   attn_decode_kernel   single decoded tokens: one CTA = one request x one key/value head x one
//                        range of keys ("split"); the group's query heads are the rows of the
//                        16-row MMA tile, so a key/value tile is read once for the whole group.
//                        With more than one split the partial (max, sum, output) go to scratch
//                        memory and attn_merge_kernel combines them.  Its FUSED form takes the
//                        float32 k-split partial sums of the qkv product instead of finished
//                        queries: every CTA adds and rotates its group's queries itself, and
//                        the CTA whose keys end with the token adds, rotates and stores the
//                        token's key and value (engine/model.py:199-203) and uses them from
//                        shared memory, so no kernel runs between the product and the attention.
//
// Replaces flash_attn_varlen_func with block_table (engine/model.py:204-207, 244-247).
// Softmax statistics, the running output and all sums are float32; P is rounded to bfloat16
// only as the operand of P.V.  Tiles start at multiples of 64 of the key position, so a
// query's result does not depend on the batch it is computed in.
#include "tcgen05_common.cuh"      // mbarriers with bounded waits, TMA tile loads, the cache of tensor maps

#include <mutex>

namespace {

typedef __nv_bfloat16 bf16;

constexpr int kTile = 64;       // keys per shared-memory tile
constexpr int kThreads = 128;   // 4 warps
constexpr int kStages = 3;

__device__ __forceinline__ void cp_async16(uint32_t dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(dst), "l"(src));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;\n" ::"n"(N));
}
__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

// Element offset of 16-byte chunk `c` of row `r` in a [rows][D] bf16 tile whose chunks are
// XOR-swizzled by the row, so that the 8 rows an ldmatrix reads fall into different banks.
template <int D> __device__ __forceinline__ int tile_off(int r, int c) { return r * D + ((c ^ (r & 7)) << 3); }
// The same for a tile that TMA boxes with the 128-byte swizzle filled (attn_decode_tma_kernel): per 64 dims a block of
// [64 rows][128 bytes], the eight chunks of a row XOR-swizzled by the row.
__device__ __forceinline__ int tma_tile_off(int r, int c) { return (c >> 3) * (64 * 64) + r * 64 + (((c & 7) ^ (r & 7)) << 3); }
template <int D, bool TMA> __device__ __forceinline__ int kv_tile_off(int r, int c) { return TMA ? tma_tile_off(r, c) : tile_off<D>(r, c); }

// Page ids of the rows of tile [key0, key0 + 64) that this thread copies (rows past `key_last`
// repeat that key: their scores are masked by the caller, and no page beyond the request's
// is touched).  Thread t copies chunk t % CH of rows t / CH, t / CH + RPI, ...
template <int D> struct TileMap {
    static constexpr int CH = D / 8;              // 16-byte chunks per row
    static constexpr int RPI = kThreads / CH;     // rows covered per pass of the CTA
    static constexpr int ITERS = kTile / RPI;
};

template <int D>
__device__ __forceinline__ void tile_pages(int (&pg)[TileMap<D>::ITERS], const int* __restrict__ table, int key0,
                                           int key_last, int page_size, int page_shift) {
    const int r0 = threadIdx.x / TileMap<D>::CH;
#pragma unroll
    for (int j = 0; j < TileMap<D>::ITERS; ++j) {
        const int key = min(key0 + r0 + j * TileMap<D>::RPI, key_last);
        pg[j] = table[page_shift >= 0 ? key >> page_shift : key / page_size];
    }
}

// Issue the copies of one K tile and one V tile (same pages, V plane `v_off` elements after K).
template <int D>
__device__ __forceinline__ void load_kv_tiles(bf16* ktile, bf16* vtile, const bf16* __restrict__ kplane, size_t v_off,
                                              const int (&pg)[TileMap<D>::ITERS], int key0, int key_last, int page_size,
                                              int page_shift, size_t page_stride) {
    const int c = threadIdx.x % TileMap<D>::CH, r0 = threadIdx.x / TileMap<D>::CH;
#pragma unroll
    for (int j = 0; j < TileMap<D>::ITERS; ++j) {
        const int r = r0 + j * TileMap<D>::RPI;
        const int key = min(key0 + r, key_last);
        const int off = page_shift >= 0 ? key & (page_size - 1) : key % page_size;
        const bf16* src = kplane + (size_t)pg[j] * page_stride + (size_t)off * D + c * 8;
        cp_async16(smem_u32(ktile + tile_off<D>(r, c)), src);
        cp_async16(smem_u32(vtile + tile_off<D>(r, c)), src + v_off);
    }
}

// S[16 x 16 keys] for one warp: rows = the A fragments `qa`, keys = tile rows [r0, r0 + 16).
template <int D, bool TMA = false>
__device__ __forceinline__ void qk_16keys(float (&s0)[4], float (&s1)[4], const uint32_t (&qa)[D / 16][4],
                                          const bf16* ktile, int r0, int lane) {
#pragma unroll
    for (int kt = 0; kt < D / 16; ++kt) {
        uint32_t b[4];
        const int row = r0 + ((lane >> 4) << 3) + (lane & 7);
        const int chunk = 2 * kt + ((lane >> 3) & 1);
        ldmatrix_x4(b, smem_u32(ktile + kv_tile_off<D, TMA>(row, chunk)));
        mma_bf16(s0, qa[kt], b[0], b[1]);
        mma_bf16(s1, qa[kt], b[2], b[3]);
    }
}

// O[16 x D] += P[16 x 16 keys] . V[16 keys x D], V rows = tile rows [r0, r0 + 16).
template <int D, bool TMA = false>
__device__ __forceinline__ void pv_16keys(float (&o)[D / 8][4], const uint32_t (&pa)[4], const bf16* vtile, int r0, int lane) {
#pragma unroll
    for (int n2 = 0; n2 < D / 16; ++n2) {
        uint32_t b[4];
        const int row = r0 + (((lane >> 3) & 1) << 3) + (lane & 7);
        const int chunk = 2 * n2 + (lane >> 4);
        ldmatrix_x4_trans(b, smem_u32(vtile + kv_tile_off<D, TMA>(row, chunk)));
        mma_bf16(o[2 * n2], pa, b[0], b[1]);
        mma_bf16(o[2 * n2 + 1], pa, b[2], b[3]);
    }
}

// One online-softmax update for the two rows (g, g + 8) a thread holds, over 16 keys
// (s0: keys 0-7, s1: keys 8-15 of the slice).  Scores arrive raw; `sl` = scale * log2(e).
// Returns the bf16 A fragment of P and rescales `o`.
template <int D>
__device__ __forceinline__ void softmax_16keys(float (&s0)[4], float (&s1)[4], float (&m)[2], float (&l)[2],
                                               float (&o)[D / 8][4], uint32_t (&pa)[4], float sl) {
    float mx0 = fmaxf(fmaxf(s0[0], s0[1]), fmaxf(s1[0], s1[1]));
    float mx1 = fmaxf(fmaxf(s0[2], s0[3]), fmaxf(s1[2], s1[3]));
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
    const float mn0 = fmaxf(m[0], mx0 * sl), mn1 = fmaxf(m[1], mx1 * sl);
    const float mu0 = mn0 == -INFINITY ? 0.f : mn0, mu1 = mn1 == -INFINITY ? 0.f : mn1;  // nothing visible yet
    const float c0 = exp2f(m[0] - mu0), c1 = exp2f(m[1] - mu1);
    m[0] = mn0;
    m[1] = mn1;
    float p00 = exp2f(s0[0] * sl - mu0), p01 = exp2f(s0[1] * sl - mu0), p02 = exp2f(s0[2] * sl - mu1), p03 = exp2f(s0[3] * sl - mu1);
    float p10 = exp2f(s1[0] * sl - mu0), p11 = exp2f(s1[1] * sl - mu0), p12 = exp2f(s1[2] * sl - mu1), p13 = exp2f(s1[3] * sl - mu1);
    l[0] = l[0] * c0 + (p00 + p01 + p10 + p11);
    l[1] = l[1] * c1 + (p02 + p03 + p12 + p13);
    // (a factor of exactly 1 changes nothing: once the rows' maxima stand, which is most tiles, the warp skips the scaling)
    if (__any_sync(0xffffffffu, c0 != 1.0f || c1 != 1.0f)) {
#pragma unroll
        for (int n = 0; n < D / 8; ++n) {
            o[n][0] *= c0; o[n][1] *= c0; o[n][2] *= c1; o[n][3] *= c1;
        }
    }
    pa[0] = pack_bf16(p00, p01);
    pa[1] = pack_bf16(p02, p03);
    pa[2] = pack_bf16(p10, p11);
    pa[3] = pack_bf16(p12, p13);
}

// ---------------------------------------------------------------------------------------
// prompt portions
// ---------------------------------------------------------------------------------------
// tiles[i] = {first token row, rows (<= 64), position of the first row, request}
template <int D>
__global__ void __launch_bounds__(kThreads)
attn_prefill_kernel(const bf16* __restrict__ q, int q_stride, const bf16* __restrict__ cache,
                    const int* __restrict__ block_table, int table_width, const int4* __restrict__ tiles,
                    bf16* __restrict__ out, int out_stride, int heads, int kv_heads, int page_size, int page_shift,
                    int window, float sl) {
    pdl_trigger();
    pdl_wait();
    extern __shared__ __align__(128) unsigned char smem_raw[];
    bf16* qtile = reinterpret_cast<bf16*>(smem_raw);              // [64][D]
    bf16* kv = qtile + kTile * D;                                 // [2 stages][K,V][64][D]
    // Blocks are handed out with x running fastest: the block's number in that order is cut so that all heads of
    // one query tile follow each other, tiles taken from the end of the list (the host sorts it by context), so
    // the tiles with the most keys start first and the short ones fill the gaps at the end of the launch.
    const unsigned lin = blockIdx.x + gridDim.x * blockIdx.y;
    const int4 td = tiles[gridDim.x - 1 - lin / gridDim.y];
    const int tok0 = td.x, rows = td.y, pos0 = td.z, req = td.w;
    const int h = (int)(lin % gridDim.y), hk = h / (heads / kv_heads);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t4 = lane & 3;
    const int* table = block_table + (size_t)req * table_width;
    const size_t plane = (size_t)kv_heads * page_size * D;
    const bf16* kplane = cache + (size_t)hk * page_size * D;
    const int pos_last = pos0 + rows - 1;
    const int lo0 = window > 0 ? max(0, pos0 - window + 1) : 0;
    const int k_begin = lo0 & ~(kTile - 1);
    const int n_tiles = (pos_last - k_begin) / kTile + 1;

    // Q tile (rows past `rows` are zero)
    constexpr int CH = D / 8;
    for (int i = threadIdx.x; i < kTile * CH; i += kThreads) {
        const int r = i / CH, c = i % CH;
        bf16* dst = qtile + tile_off<D>(r, c);
        if (r < rows)
            cp_async16(smem_u32(dst), q + (size_t)(tok0 + r) * q_stride + (size_t)h * D + c * 8);
        else
            *reinterpret_cast<uint4*>(dst) = make_uint4(0, 0, 0, 0);
    }
    auto stage_k = [&](int s) { return kv + (size_t)s * 2 * kTile * D; };
    auto stage_v = [&](int s) { return kv + (size_t)s * 2 * kTile * D + kTile * D; };
    int pg[TileMap<D>::ITERS];
    tile_pages<D>(pg, table, k_begin, pos_last, page_size, page_shift);
    load_kv_tiles<D>(stage_k(0), stage_v(0), kplane, plane, pg, k_begin, pos_last, page_size, page_shift, 2 * plane);
    cp_async_commit();
    if (n_tiles > 1) tile_pages<D>(pg, table, k_begin + kTile, pos_last, page_size, page_shift);

    uint32_t qa[D / 16][4];
    float o[D / 8][4];
#pragma unroll
    for (int n = 0; n < D / 8; ++n) o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f;
    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
    const int row_pos0 = pos0 + warp * 16 + g, row_pos1 = row_pos0 + 8;  // positions of this thread's two rows

    for (int it = 0; it < n_tiles; ++it) {
        const int k0 = k_begin + it * kTile;
        if (it + 1 < n_tiles) {
            load_kv_tiles<D>(stage_k((it + 1) & 1), stage_v((it + 1) & 1), kplane, plane, pg, k0 + kTile, pos_last,
                             page_size, page_shift, 2 * plane);
            cp_async_commit();
            if (it + 2 < n_tiles) tile_pages<D>(pg, table, k0 + 2 * kTile, pos_last, page_size, page_shift);
            cp_async_wait<1>();
        } else {
            cp_async_wait<0>();
        }
        __syncthreads();
        if (it == 0) {
#pragma unroll
            for (int kt = 0; kt < D / 16; ++kt) {
                const int row = warp * 16 + (((lane >> 3) & 1) << 3) + (lane & 7);
                ldmatrix_x4(qa[kt], smem_u32(qtile + tile_off<D>(row, 2 * kt + (lane >> 4))));
            }
        }
        const bf16* kt_s = stage_k(it & 1);
        const bf16* vt_s = stage_v(it & 1);
        // S = Q K^T for the 64 keys of the tile: 8 column blocks of 8 keys
        float sc[kTile / 8][4];
#pragma unroll
        for (int n = 0; n < kTile / 8; ++n) sc[n][0] = sc[n][1] = sc[n][2] = sc[n][3] = 0.f;
#pragma unroll
        for (int ks = 0; ks < kTile / 16; ++ks) qk_16keys<D>(sc[2 * ks], sc[2 * ks + 1], qa, kt_s, ks * 16, lane);
        const bool need_mask = (k0 + kTile - 1 > pos0) || (window > 0 && k0 < pos_last - window + 1);
        if (need_mask) {
            const int lo_a = window > 0 ? row_pos0 - window + 1 : 0, lo_b = window > 0 ? row_pos1 - window + 1 : 0;
#pragma unroll
            for (int n = 0; n < kTile / 8; ++n) {
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                    const int key = k0 + n * 8 + 2 * t4 + e;
                    if (key > row_pos0 || key < lo_a) sc[n][e] = -INFINITY;
                    if (key > row_pos1 || key < lo_b) sc[n][2 + e] = -INFINITY;
                }
            }
        }
        // one online-softmax update per tile
        float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
        for (int n = 0; n < kTile / 8; ++n) {
            mx0 = fmaxf(mx0, fmaxf(sc[n][0], sc[n][1]));
            mx1 = fmaxf(mx1, fmaxf(sc[n][2], sc[n][3]));
        }
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
        const float mn0 = fmaxf(m[0], mx0 * sl), mn1 = fmaxf(m[1], mx1 * sl);
        const float mu0 = mn0 == -INFINITY ? 0.f : mn0, mu1 = mn1 == -INFINITY ? 0.f : mn1;
        const float c0 = exp2f(m[0] - mu0), c1 = exp2f(m[1] - mu1);
        m[0] = mn0;
        m[1] = mn1;
        float sum0 = 0.f, sum1 = 0.f;
        uint32_t pa[kTile / 16][4];
#pragma unroll
        for (int n = 0; n < kTile / 8; ++n) {
            const float p0 = exp2f(sc[n][0] * sl - mu0), p1 = exp2f(sc[n][1] * sl - mu0);
            const float p2 = exp2f(sc[n][2] * sl - mu1), p3 = exp2f(sc[n][3] * sl - mu1);
            sum0 += p0 + p1;
            sum1 += p2 + p3;
            pa[n >> 1][(n & 1) * 2] = pack_bf16(p0, p1);
            pa[n >> 1][(n & 1) * 2 + 1] = pack_bf16(p2, p3);
        }
        l[0] = l[0] * c0 + sum0;
        l[1] = l[1] * c1 + sum1;
#pragma unroll
        for (int n = 0; n < D / 8; ++n) {
            o[n][0] *= c0; o[n][1] *= c0; o[n][2] *= c1; o[n][3] *= c1;
        }
#pragma unroll
        for (int ks = 0; ks < kTile / 16; ++ks) pv_16keys<D>(o, pa[ks], vt_s, ks * 16, lane);
        __syncthreads();   // the stage is refilled two iterations later
    }
    // row sums live in 4 lanes each
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        l[r] += __shfl_xor_sync(0xffffffffu, l[r], 1);
        l[r] += __shfl_xor_sync(0xffffffffu, l[r], 2);
    }
    const int r0 = warp * 16 + g, r1 = r0 + 8;
    const float i0 = 1.f / l[0], i1 = 1.f / l[1];
#pragma unroll
    for (int n = 0; n < D / 8; ++n) {
        const int col = h * D + n * 8 + 2 * t4;
        if (r0 < rows)
            *reinterpret_cast<uint32_t*>(out + (size_t)(tok0 + r0) * out_stride + col) = pack_bf16(o[n][0] * i0, o[n][1] * i0);
        if (r1 < rows)
            *reinterpret_cast<uint32_t*>(out + (size_t)(tok0 + r1) * out_stride + col) = pack_bf16(o[n][2] * i1, o[n][3] * i1);
    }
}

// ---------------------------------------------------------------------------------------
// decoded tokens (one query per request), keys split over CTAs
// ---------------------------------------------------------------------------------------
// part_o [items, heads, max_splits, D] float32 (unnormalised, relative to the split's max),
// part_ml [items, heads, max_splits, 2] float32 (max in the log2 domain, sum).
//
// Contract of the callers: keys_per_split * max_splits covers every item's keys (from the 64-aligned start of its
// window to its position).  The kernels cannot trust a foreign caller with that, so an item that would need more
// splits is cut down to max_splits (its last keys are then left out: the result is wrong, but nothing is read or
// written outside the partials of its own (item, head)), and a code is left in g_decode_status.
__device__ int g_decode_status = 0;            // 0 ok; else (6 << 16) | item of the first item that did not fit

// What the FUSED form reads instead of finished queries.
struct QkvParts {
    const float* parts;        // [splits][tokens][(heads + 2 kv_heads) * D] float32 partial sums of the qkv product
    int splits;
    size_t split_stride;       // elements between two splits
    const float* cos_table;    // [tokens][D / 2]
    const float* sin_table;
    const int* slots;          // [tokens] page * page_size + offset of each token's key and value
    bf16* cache;               // the same cache layer, for the store
};

// FUSED prologue of a decode CTA, run by its `nthreads` computing threads (`tid` among them): adds the qkv product's
// partial sums of the group's queries, rotates them and leaves them in q_new [16][D]; the CTA whose keys end with the
// token (`owner`) also adds and rotates the key, adds the value, leaves both in kv_new [2][D] and stores them in
// the cache.  Items of four neighbouring dims: per rotated head D/8 of them (dims i.. and i + D/2..), per value head
// D/4.  The arithmetic is that of rope_store_sum_kernel, and the results are rounded to bfloat16 as it rounds them, so
// both routes hand the same queries, keys and values to the products that follow.
template <int D>
__device__ __forceinline__ void decode_fused_prologue(const QkvParts& f, int tok, int hk, int G, int heads, int kv_heads,
                                                      int page_size, int page_shift, size_t plane, bool owner, bf16* q_new,
                                                      bf16* kv_new, int tid, int nthreads) {
    constexpr int half = D / 2, hp = D / 8, per_head = D / 4;
    const float* row = f.parts + (size_t)tok * ((size_t)(heads + 2 * kv_heads) * D);
    const int n_q = G * hp;
    const int n_work = n_q + (owner ? hp + per_head : 0);
    size_t kdst = 0;
    if (owner) {
        const int slot = f.slots[tok];
        const int page = page_shift >= 0 ? slot >> page_shift : slot / page_size;
        const int off = page_shift >= 0 ? slot & (page_size - 1) : slot % page_size;
        kdst = (size_t)page * 2 * plane + (size_t)hk * page_size * D + (size_t)off * D;
    }
    for (int w = tid; w < n_work; w += nthreads) {
        if (w < n_q + hp) {
            const bool is_q = w < n_q;
            const int h = is_q ? hk * G + w / hp : heads + hk;
            const int i = (w % hp) * 4;
            const float4 a = sum_parts4(row + (size_t)h * D + i, f.splits, f.split_stride);
            const float4 b = sum_parts4(row + (size_t)h * D + i + half, f.splits, f.split_stride);
            const float4 c = *reinterpret_cast<const float4*>(f.cos_table + (size_t)tok * half + i);
            const float4 sg = *reinterpret_cast<const float4*>(f.sin_table + (size_t)tok * half + i);
            uint2 lo2, hi2;
            lo2.x = pack_bf16(a.x * c.x - b.x * sg.x, a.y * c.y - b.y * sg.y);
            lo2.y = pack_bf16(a.z * c.z - b.z * sg.z, a.w * c.w - b.w * sg.w);
            hi2.x = pack_bf16(b.x * c.x + a.x * sg.x, b.y * c.y + a.y * sg.y);
            hi2.y = pack_bf16(b.z * c.z + a.z * sg.z, b.w * c.w + a.w * sg.w);
            bf16* dst = is_q ? q_new + (w / hp) * D : kv_new;
            *reinterpret_cast<uint2*>(dst + i) = lo2;
            *reinterpret_cast<uint2*>(dst + i + half) = hi2;
            if (!is_q) {
                *reinterpret_cast<uint2*>(f.cache + kdst + i) = lo2;
                *reinterpret_cast<uint2*>(f.cache + kdst + i + half) = hi2;
            }
        } else {
            const int i = (w - n_q - hp) * 4;
            const float4 v = sum_parts4(row + (size_t)(heads + kv_heads + hk) * D + i, f.splits, f.split_stride);
            uint2 v2;
            v2.x = pack_bf16(v.x, v.y);
            v2.y = pack_bf16(v.z, v.w);
            *reinterpret_cast<uint2*>(kv_new + D + i) = v2;
            *reinterpret_cast<uint2*>(f.cache + kdst + plane + i) = v2;
        }
    }
}

// The A fragments of the group's query heads: rows 0 .. G-1 of the MMA tile (row g at qrow0 + g * D for g < 8 given by
// the caller as its own row pointer); the other rows are zero.
template <int D>
__device__ __forceinline__ void decode_query_fragments(uint32_t (&qa)[D / 16][4], const bf16* qrow0, int g, int t4, int G) {
    const bf16* qrow1 = qrow0 + 8 * D;
#pragma unroll
    for (int kt = 0; kt < D / 16; ++kt) {
        qa[kt][0] = g < G ? *reinterpret_cast<const uint32_t*>(qrow0 + kt * 16 + 2 * t4) : 0u;
        qa[kt][1] = g + 8 < G ? *reinterpret_cast<const uint32_t*>(qrow1 + kt * 16 + 2 * t4) : 0u;
        qa[kt][2] = g < G ? *reinterpret_cast<const uint32_t*>(qrow0 + kt * 16 + 8 + 2 * t4) : 0u;
        qa[kt][3] = g + 8 < G ? *reinterpret_cast<const uint32_t*>(qrow1 + kt * 16 + 8 + 2 * t4) : 0u;
    }
}

// One warp's scores, softmax update and P V of its 16 keys [k0, k0 + 16) of a tile (tile rows r0 ..); keys outside
// [lo, c1) are masked.
template <int D, bool TMA>
__device__ __forceinline__ void decode_warp_tile(const uint32_t (&qa)[D / 16][4], const bf16* ktile, const bf16* vtile, int r0,
                                                 int k0, int lo, int c1, float sl, float (&m)[2], float (&l)[2],
                                                 float (&o)[D / 8][4], int lane) {
    const int t4 = lane & 3;
    float s0[4] = {0.f, 0.f, 0.f, 0.f}, s1[4] = {0.f, 0.f, 0.f, 0.f};
    qk_16keys<D, TMA>(s0, s1, qa, ktile, r0, lane);
    if (k0 + 16 > c1 || k0 < lo) {
        const int kb = k0 + 2 * t4;
#pragma unroll
        for (int e = 0; e < 2; ++e) {
            if (kb + e >= c1 || kb + e < lo) s0[e] = s0[2 + e] = -INFINITY;
            if (kb + 8 + e >= c1 || kb + 8 + e < lo) s1[e] = s1[2 + e] = -INFINITY;
        }
    }
    uint32_t pa[4];
    softmax_16keys<D>(s0, s1, m, l, o, pa, sl);
    pv_16keys<D, TMA>(o, pa, vtile, r0, lane);
}

// The end of a decode CTA: its four computing warps (each saw other keys) are merged through `scratch`
// ([4][16][D] + 2 x [4][16] floats of shared memory that nobody reads any more), rows < G only, and the result goes to
// `out` (one split) or to the partials.  `sync` is the barrier of the computing threads.
template <int D, typename Sync>
__device__ __forceinline__ void decode_finish(float (&o)[D / 8][4], float (&m)[2], float (&l)[2], float* scratch, int warp,
                                              int lane, int tid, int nthreads, int G, int hk, int heads, int tok, int item,
                                              int split, int n_splits, int max_splits, float* part_o, float* part_ml,
                                              bf16* out, int out_stride, Sync sync) {
    const int g = lane >> 2, t4 = lane & 3;
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        l[r] += __shfl_xor_sync(0xffffffffu, l[r], 1);
        l[r] += __shfl_xor_sync(0xffffffffu, l[r], 2);
    }
    float* sm_o = scratch;                                        // [4][16][D]
    float* sm_m = sm_o + 4 * 16 * D;                              // [4][16]
    float* sm_l = sm_m + 4 * 16;                                  // [4][16]
#pragma unroll
    for (int n = 0; n < D / 8; ++n) {
        const int col = n * 8 + 2 * t4;
        if (g < G) { sm_o[(warp * 16 + g) * D + col] = o[n][0]; sm_o[(warp * 16 + g) * D + col + 1] = o[n][1]; }
        if (g + 8 < G) { sm_o[(warp * 16 + g + 8) * D + col] = o[n][2]; sm_o[(warp * 16 + g + 8) * D + col + 1] = o[n][3]; }
    }
    if (t4 == 0) {
        sm_m[warp * 16 + g] = m[0]; sm_l[warp * 16 + g] = l[0];
        sm_m[warp * 16 + g + 8] = m[1]; sm_l[warp * 16 + g + 8] = l[1];
    }
    sync();
    for (int i = tid; i < G * D; i += nthreads) {
        const int r = i / D, d = i % D;
        float M = -INFINITY;
#pragma unroll
        for (int w = 0; w < 4; ++w) M = fmaxf(M, sm_m[w * 16 + r]);
        float L = 0.f, O = 0.f;
#pragma unroll
        for (int w = 0; w < 4; ++w) {
            const float mw = sm_m[w * 16 + r];
            const float f = mw == -INFINITY ? 0.f : exp2f(mw - M);
            L += sm_l[w * 16 + r] * f;
            O += sm_o[(w * 16 + r) * D + d] * f;
        }
        const int head = hk * G + r;
        if (n_splits == 1) {
            out[(size_t)tok * out_stride + (size_t)head * D + d] = __float2bfloat16_rn(O / L);
        } else {
            const size_t base = ((size_t)item * heads + head) * max_splits + split;
            part_o[base * D + d] = O;
            if (d == 0) { part_ml[base * 2] = M; part_ml[base * 2 + 1] = L; }
        }
    }
}

template <int D, bool FUSED>
__global__ void __launch_bounds__(kThreads)
attn_decode_kernel(const bf16* __restrict__ q, int q_stride, const bf16* __restrict__ cache,
                   const int* __restrict__ block_table, int table_width, const int* __restrict__ items,
                   const int* __restrict__ token_request, const int* __restrict__ positions,
                   float* __restrict__ part_o, float* __restrict__ part_ml, bf16* __restrict__ out, int out_stride,
                   int heads, int kv_heads, int page_size, int page_shift, int window, float sl, int keys_per_split,
                   int max_splits, const QkvParts f) {
    pdl_trigger();
    extern __shared__ __align__(128) unsigned char smem_raw[];
    __shared__ __align__(16) bf16 q_new[FUSED ? 16 * D : 8];      // FUSED: the group's rotated queries
    __shared__ __align__(16) bf16 kv_new[FUSED ? 2 * D : 8];      // FUSED: the token's rotated key, its value
    bf16* kv = reinterpret_cast<bf16*>(smem_raw);                 // [kStages][K,V][64][D]
    const int split = blockIdx.x, hk = blockIdx.y, item = blockIdx.z;
    const int tok = items[item];
    const int pos = positions[tok];
    const int lo = window > 0 ? max(0, pos - window + 1) : 0;
    const int k_begin = lo & ~(kTile - 1);
    int n_splits = (pos - k_begin) / keys_per_split + 1;
    if (n_splits > max_splits) {                                  // the caller's contract is broken: see g_decode_status
        if (split == 0 && hk == 0 && threadIdx.x == 0) atomicCAS(&g_decode_status, 0, (6 << 16) | (item & 0xffff));
        n_splits = max_splits;
    }
    if (split >= n_splits) return;
    const int c0 = k_begin + split * keys_per_split;
    const int c1 = min(c0 + keys_per_split, pos + 1);             // keys [c0, c1)
    const int n_tiles = (c1 - c0 + kTile - 1) / kTile;
    const int G = heads / kv_heads;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t4 = lane & 3;
    const int* table = block_table + (size_t)token_request[tok] * table_width;
    const size_t plane = (size_t)kv_heads * page_size * D;
    const bf16* kplane = cache + (size_t)hk * page_size * D;
    auto stage_k = [&](int s) { return kv + (size_t)s * 2 * kTile * D; };
    auto stage_v = [&](int s) { return kv + (size_t)s * 2 * kTile * D + kTile * D; };

    // The step's index arrays were copied in before its first kernel, and keys and values of positions before
    // `pos` were stored by earlier steps: tiles that end before `pos` are requested ahead of the wait for the
    // kernel before this one (which stores the token's own key and value, and writes the queries).
    int pg[TileMap<D>::ITERS];
    bool waited = false;
#pragma unroll
    for (int s = 0; s < kStages - 1; ++s) {
        if (!waited && c0 + (s + 1) * kTile > pos) { pdl_wait(); waited = true; }
        if (s < n_tiles) {
            tile_pages<D>(pg, table, c0 + s * kTile, pos, page_size, page_shift);
            load_kv_tiles<D>(stage_k(s), stage_v(s), kplane, plane, pg, c0 + s * kTile, pos, page_size, page_shift, 2 * plane);
        }
        cp_async_commit();
    }
    if (!waited) pdl_wait();
    // page ids of the tile that the first iteration will request, fetched one iteration ahead from here on
    if (kStages - 1 < n_tiles) tile_pages<D>(pg, table, c0 + (kStages - 1) * kTile, pos, page_size, page_shift);
    const bool owner = FUSED && c1 == pos + 1;                    // this CTA's keys end with the token itself
    if constexpr (FUSED) {
        decode_fused_prologue<D>(f, tok, hk, G, heads, kv_heads, page_size, page_shift, plane, owner, q_new, kv_new,
                                 (int)threadIdx.x, kThreads);
        __syncthreads();
    }
    uint32_t qa[D / 16][4];
    decode_query_fragments<D>(qa, FUSED ? q_new + g * D : q + (size_t)tok * q_stride + (size_t)(hk * G + g) * D, g, t4, G);
    float o[D / 8][4];
#pragma unroll
    for (int n = 0; n < D / 8; ++n) o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f;
    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};

    for (int it = 0; it < n_tiles; ++it) {
        const int nxt = it + kStages - 1;
        cp_async_wait<kStages - 2>();
        __syncthreads();                      // tile `it` has landed; stage (it-1)%S is free again
        if (nxt < n_tiles)
            load_kv_tiles<D>(stage_k(nxt % kStages), stage_v(nxt % kStages), kplane, plane, pg, c0 + nxt * kTile, pos,
                             page_size, page_shift, 2 * plane);
        cp_async_commit();
        if (nxt + 1 < n_tiles) tile_pages<D>(pg, table, c0 + (nxt + 1) * kTile, pos, page_size, page_shift);
        if constexpr (FUSED) if (owner && it == n_tiles - 1) {
            // the copy fetched the token's slot as it was before this step: its row, and the rows after it (which
            // repeat it and are masked), get the key and value computed above
            constexpr int CH = D / 8;
            const int r_new = pos - (c0 + it * kTile);
            bf16* kt = stage_k(it % kStages);
            bf16* vt = stage_v(it % kStages);
            for (int i = threadIdx.x; i < (kTile - r_new) * CH; i += kThreads) {
                const int r = r_new + i / CH, c = i % CH;
                *reinterpret_cast<uint4*>(kt + tile_off<D>(r, c)) = *reinterpret_cast<const uint4*>(kv_new + c * 8);
                *reinterpret_cast<uint4*>(vt + tile_off<D>(r, c)) = *reinterpret_cast<const uint4*>(kv_new + D + c * 8);
            }
            __syncthreads();
        }
        const int k0 = c0 + it * kTile + warp * 16;               // this warp's 16 keys of the tile
        if (k0 < c1)
            decode_warp_tile<D, false>(qa, stage_k(it % kStages), stage_v(it % kStages), warp * 16, k0, lo, c1, sl, m, l, o, lane);
    }
    cp_async_wait<0>();
    __syncthreads();
    decode_finish<D>(o, m, l, reinterpret_cast<float*>(smem_raw), warp, lane, (int)threadIdx.x, kThreads, G, hk, heads, tok,
                     item, split, n_splits, max_splits, part_o, part_ml, out, out_stride, [] { __syncthreads(); });
}

// The same decode CTA with its keys and values brought in by TMA: the cache layer is one [rows, D] matrix to the
// tensor map, a page's 64 dims of one key/value head are one box (page sizes 8 .. 64 that divide 64), and the boxes of
// a tile of 64 keys land at their row offsets of 128-byte-swizzled [64 keys][64 dims] blocks.  Warp 4 fetches (lane p
// page p of every tile: its block-table entry, then the boxes of K and V), warps 0-3 compute as above; stages change
// hands over mbarriers (full: the bytes have landed; empty: the four computing warps are done), so no barrier of the
// whole CTA sits in the loop, a thread issues no copy of its own, and the loading warp runs ahead of the others by
// as many stages as there are.  Keys past the token's own are not read from the cache as they are there (the rows
// are masked; a page past the token's is replaced by the token's page).  Bounded waits: a wait that runs out leaves
// (7 << 16 | item) in g_decode_status and the CTA writes nothing.
constexpr int kTmaThreads = 160;
// Stages of 64 keys: three at head size 128 (96 KiB, two CTAs per SM).  At head size 64 six (the same 96 KiB) measured
// 1 to 2 % ahead of three and four in whole decode steps of a 16-layer model of width 2048.
#ifndef LLM_TMA_STAGES_64
#define LLM_TMA_STAGES_64 6
#endif
#ifndef LLM_TMA_STAGES_128
#define LLM_TMA_STAGES_128 3
#endif
template <int D> __host__ __device__ constexpr int tma_stages() { return D == 64 ? LLM_TMA_STAGES_64 : LLM_TMA_STAGES_128; }

template <int D, bool FUSED>
__global__ void __launch_bounds__(kTmaThreads)
attn_decode_tma_kernel(const __grid_constant__ CUtensorMap map_kv, const bf16* __restrict__ q, int q_stride,
                       const int* __restrict__ block_table, int table_width, const int* __restrict__ items,
                       const int* __restrict__ token_request, const int* __restrict__ positions,
                       float* __restrict__ part_o, float* __restrict__ part_ml, bf16* __restrict__ out, int out_stride,
                       int heads, int kv_heads, int page_size, int page_shift, int window, float sl, int keys_per_split,
                       int max_splits, const QkvParts f) {
    pdl_trigger();
    extern __shared__ unsigned char smem_raw[];
    unsigned char* base = reinterpret_cast<unsigned char*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    __shared__ __align__(16) bf16 q_new[FUSED ? 16 * D : 8];
    __shared__ __align__(16) bf16 kv_new[FUSED ? 2 * D : 8];
    constexpr int kStages = tma_stages<D>();                      // (shadows the copying kernels' count)
    __shared__ __align__(8) uint64_t full_bar[kStages], empty_bar[kStages];
    __shared__ volatile int failed;
    constexpr int kPlaneBytes = kTile * D * 2;                    // one K or V tile
    constexpr int kHalves = D / 64;
    const int split = blockIdx.x, hk = blockIdx.y, item = blockIdx.z;
    const int tok = items[item];
    const int pos = positions[tok];
    const int lo = window > 0 ? max(0, pos - window + 1) : 0;
    const int k_begin = lo & ~(kTile - 1);
    int n_splits = (pos - k_begin) / keys_per_split + 1;
    if (n_splits > max_splits) {
        if (split == 0 && hk == 0 && threadIdx.x == 0) atomicCAS(&g_decode_status, 0, (6 << 16) | (item & 0xffff));
        n_splits = max_splits;
    }
    if (split >= n_splits) return;
    const int c0 = k_begin + split * keys_per_split;
    const int c1 = min(c0 + keys_per_split, pos + 1);
    const int n_tiles = (c1 - c0 + kTile - 1) / kTile;
    const int G = heads / kv_heads;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t4 = lane & 3;
    auto stage_k = [&](int s) { return reinterpret_cast<bf16*>(base + (size_t)s * 2 * kPlaneBytes); };
    auto stage_v = [&](int s) { return reinterpret_cast<bf16*>(base + (size_t)s * 2 * kPlaneBytes + kPlaneBytes); };
    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 4); }
        failed = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();

    if (warp == 4) {
        // ---- loads ------------------------------------------------------------------------------------------
        const int* table = block_table + (size_t)token_request[tok] * table_width;
        const int pages_per_tile = kTile >> page_shift;
        // page of this lane's rows of tile `t` (a page past the token's own: the token's, see above)
        auto page_of = [&](int t) { return table[min(c0 + t * kTile + (lane << page_shift), pos) >> page_shift]; };
        int page = lane < pages_per_tile ? page_of(0) : 0;
        bool waited = false;
        for (int it = 0; it < n_tiles; ++it) {
            const int s = it % kStages;
            // tiles that end before `pos` hold what earlier steps stored: they are requested ahead of the wait for the
            // kernel before this one (which stores the token's own key and value in the form that is not FUSED)
            if (!waited && c0 + (it + 1) * kTile > pos) { pdl_wait(); waited = true; }
            int ok = 1;
            if (lane == 0) {
                if (it >= kStages && !mbar_wait(&empty_bar[s], ((it / kStages) - 1) & 1)) {
                    atomicCAS(&g_decode_status, 0, (7 << 16) | (item & 0xffff));
                    failed = 1;
                    ok = 0;
                } else {
                    mbar_expect_tx(&full_bar[s], 2 * kPlaneBytes);
                }
            }
            ok = __shfl_sync(0xffffffffu, ok, 0);
            if (!ok) break;
            if (lane < pages_per_tile) {
                const int row = (page * 2 * kv_heads + hk) * page_size;         // K rows of this page; V rows kv_heads * page_size on
                unsigned char* kd = reinterpret_cast<unsigned char*>(stage_k(s)) + (size_t)(lane << page_shift) * 128;
                unsigned char* vd = reinterpret_cast<unsigned char*>(stage_v(s)) + (size_t)(lane << page_shift) * 128;
#pragma unroll
                for (int h = 0; h < kHalves; ++h) {
                    tma_load_2d(kd + h * (kTile * 128), &map_kv, &full_bar[s], 64 * h, row);
                    tma_load_2d(vd + h * (kTile * 128), &map_kv, &full_bar[s], 64 * h, row + kv_heads * page_size);
                }
                if (it + 1 < n_tiles) page = page_of(it + 1);
            }
        }
        return;
    }

    // ---- the four computing warps ---------------------------------------------------------------------------
    auto sync_compute = [] { asm volatile("bar.sync 1, 128;" ::: "memory"); };
    pdl_wait();
    const bool owner = FUSED && c1 == pos + 1;
    if constexpr (FUSED) {
        const size_t plane = (size_t)kv_heads * page_size * D;
        decode_fused_prologue<D>(f, tok, hk, G, heads, kv_heads, page_size, page_shift, plane, owner, q_new, kv_new,
                                 (int)threadIdx.x, 128);
        sync_compute();
    }
    uint32_t qa[D / 16][4];
    decode_query_fragments<D>(qa, FUSED ? q_new + g * D : q + (size_t)tok * q_stride + (size_t)(hk * G + g) * D, g, t4, G);
    float o[D / 8][4];
#pragma unroll
    for (int n = 0; n < D / 8; ++n) o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f;
    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
    for (int it = 0; it < n_tiles; ++it) {
        const int s = it % kStages;
        if (!mbar_wait(&full_bar[s], (it / kStages) & 1)) {
            atomicCAS(&g_decode_status, 0, (7 << 16) | (item & 0xffff));
            failed = 1;
            break;
        }
        const int k0 = c0 + it * kTile + warp * 16;               // this warp's 16 keys of the tile
        if (k0 < c1) {
            if constexpr (FUSED) {
                // the box fetched the token's slot as it was before this step or as the prologue stored it, whichever
                // came first: the warp that holds the token's row writes the key and value computed above over it
                const int r_new = pos - (c0 + it * kTile);
                if (owner && it == n_tiles - 1 && (r_new >> 4) == warp) {
                    if (lane < D / 8) {
                        *reinterpret_cast<uint4*>(stage_k(s) + tma_tile_off(r_new, lane)) = *reinterpret_cast<const uint4*>(kv_new + lane * 8);
                        *reinterpret_cast<uint4*>(stage_v(s) + tma_tile_off(r_new, lane)) = *reinterpret_cast<const uint4*>(kv_new + D + lane * 8);
                    }
                    __syncwarp();
                }
            }
            if (k0 + 16 > c1) {
                // rows past the last key were read as they lie in the cache: P is 0 there, but 0 x a slot that was never
                // written need not be, so their values are zeroed
                const int first = c1 - k0;
                for (int i = lane; i < (16 - first) * (D / 8); i += 32)
                    *reinterpret_cast<uint4*>(stage_v(s) + tma_tile_off(warp * 16 + first + i / (D / 8), i % (D / 8))) = make_uint4(0u, 0u, 0u, 0u);
                __syncwarp();
            }
            decode_warp_tile<D, true>(qa, stage_k(s), stage_v(s), warp * 16, k0, lo, c1, sl, m, l, o, lane);
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&empty_bar[s]);
    }
    sync_compute();                           // every warp is done with the stages: they become the merge's scratch
    if (failed) return;
    decode_finish<D>(o, m, l, reinterpret_cast<float*>(base), warp, lane, (int)threadIdx.x, 128, G, hk, heads, tok, item, split,
                     n_splits, max_splits, part_o, part_ml, out, out_stride, sync_compute);
}

// All loads of a thread are asked for at once (the partial results of every possible split, and the position
// that tells how many of them count): the kernel is one round trip to memory long instead of four.
constexpr int kMergeSplits = 16;
constexpr int kMaxMergeSplits = 1024;          // most key splits of one item (the merge keeps their maxima and sums in shared memory)

constexpr int kMergeGroups = 4;                // many splits: thread groups that share a (item, head)'s splits among them

template <int D>
__global__ void __launch_bounds__(D * kMergeGroups)
attn_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml, const int* __restrict__ items,
                  const int* __restrict__ positions, bf16* __restrict__ out, int out_stride, int heads, int window,
                  int keys_per_split, int max_splits) {
    pdl_trigger();
    pdl_wait();
    const int item = blockIdx.x, head = blockIdx.y, d = threadIdx.x;      // (blockDim.y > 1 only with many splits, see below)
    const size_t base = ((size_t)item * heads + head) * max_splits;
    float pm[kMergeSplits], pl[kMergeSplits], po[kMergeSplits];
    if (max_splits <= kMergeSplits) {
#pragma unroll
        for (int s = 0; s < kMergeSplits; ++s) {
            if (s < max_splits) {
                pm[s] = part_ml[(base + s) * 2];
                pl[s] = part_ml[(base + s) * 2 + 1];
                po[s] = part_o[(base + s) * D + d];
            }
        }
    }
    const int tok = items[item];
    const int pos = positions[tok];
    const int lo = window > 0 ? max(0, pos - window + 1) : 0;
    const int n_splits = min((pos - (lo & ~(kTile - 1))) / keys_per_split + 1, max_splits);   // (cut down as in the decode kernel)
    if (n_splits == 1) return;                                    // the decode kernel wrote the result itself
    float M = -INFINITY, L = 0.f, O = 0.f;
    if (max_splits <= kMergeSplits) {
        // splits past n_splits were not written by this launch: they are left out by index, never by value
#pragma unroll
        for (int s = 0; s < kMergeSplits; ++s)
            if (s < n_splits) M = fmaxf(M, pm[s]);
#pragma unroll
        for (int s = 0; s < kMergeSplits; ++s) {
            if (s < n_splits) {
                const float f = exp2f(pm[s] - M);
                L += pl[s] * f;
                O += po[s] * f;
            }
        }
    } else {
        // Many splits (a single request with a long context): the splits' maxima and sums go through shared memory
        // once, then blockDim.y groups of D threads share the splits among them (group g takes the splits g, g + groups,
        // ...: eight loads at a time) and their sums meet in shared memory in group order.
        __shared__ float sm_w[kMaxMergeSplits], sm_l[kMaxMergeSplits];
        __shared__ float grp_o[kMergeGroups][D], grp_l[kMergeGroups];
        const int grp = threadIdx.y, groups = blockDim.y;
        for (int sidx = grp * D + d; sidx < n_splits; sidx += groups * D) {    // (n_splits <= kMaxMergeSplits, checked by the launcher)
            sm_w[sidx] = part_ml[(base + sidx) * 2];
            sm_l[sidx] = part_ml[(base + sidx) * 2 + 1];
        }
        __syncthreads();
        for (int s = 0; s < n_splits; ++s) M = fmaxf(M, sm_w[s]);
        int s = grp;
        for (; s + 7 * groups < n_splits; s += 8 * groups) {
            float v[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) v[i] = part_o[(base + s + i * groups) * D + d];
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const float f = exp2f(sm_w[s + i * groups] - M);
                L += sm_l[s + i * groups] * f;
                O += v[i] * f;
            }
        }
        for (; s < n_splits; s += groups) {
            const float f = exp2f(sm_w[s] - M);
            L += sm_l[s] * f;
            O += part_o[(base + s) * D + d] * f;
        }
        if (groups > 1) {
            grp_o[grp][d] = O;
            if (d == 0) grp_l[grp] = L;
            __syncthreads();
            if (grp > 0) return;
            O = 0.f; L = 0.f;
            for (int g = 0; g < groups; ++g) { O += grp_o[g][d]; L += grp_l[g]; }
        }
    }
    out[(size_t)tok * out_stride + (size_t)head * D + d] = __float2bfloat16_rn(O / L);
}

// log2(page_size) if it is a power of two, else -1 (the kernels then divide)
int page_shift_of(int page_size) {
    int s = 0;
    while ((1 << s) < page_size) ++s;
    return (1 << s) == page_size ? s : -1;
}

// Opts a kernel in to `bytes` of dynamic shared memory.  The largest size set so far is remembered per device and
// kernel in a small fixed table (no heap), so that a launch costs no driver call once it is set.
struct SmemRecord { int dev; const void* fn; size_t bytes; };
SmemRecord g_smem_records[128];
int g_smem_count = 0;
std::mutex g_smem_mutex;

template <typename K> int set_smem(K kernel, size_t bytes, const char* name) {
    if (bytes + 8 * 1024 <= 48 * 1024) return 0;   // (a kernel's static shared memory counts toward the 48 KiB that need no opt-in)
    int dev = 0;
    cudaGetDevice(&dev);
    const void* fn = reinterpret_cast<const void*>(kernel);
    std::lock_guard<std::mutex> lock(g_smem_mutex);
    SmemRecord* rec = nullptr;
    for (int i = 0; i < g_smem_count && !rec; ++i)
        if (g_smem_records[i].dev == dev && g_smem_records[i].fn == fn) rec = &g_smem_records[i];
    if (rec && bytes <= rec->bytes) return 0;
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
    if (e != cudaSuccess) LLM_FAIL(-2, "%s: %s", name, cudaGetErrorString(e));
    if (!rec && g_smem_count < 128) { rec = &g_smem_records[g_smem_count++]; rec->dev = dev; rec->fn = fn; rec->bytes = 0; }
    if (rec) rec->bytes = bytes;       // (a full table only means that the attribute is set again next time)
    return 0;
}

}  // namespace

// 1 if the tensor-core kernels take this shape, else 0 (the caller then uses the general kernel).
LLM_API int llm_attention_bf16_supported(int heads, int kv_heads, int head_dim) {
    return (head_dim == 64 || head_dim == 128) && kv_heads > 0 && heads % kv_heads == 0 && heads / kv_heads <= 16;
}

// tiles: [n_tiles] int4 {first token row, rows, position of the first row, request}
LLM_API int llm_attention_prefill_bf16(const void* q, int q_stride, const void* cache, const int* block_table,
                                       int table_width, const int* tiles, int n_tiles, void* out, int out_stride,
                                       int heads, int kv_heads, int head_dim, int page_size, int window, float scale,
                                       cudaStream_t stream) {
    if (n_tiles == 0) return 0;
    if (!llm_attention_bf16_supported(heads, kv_heads, head_dim))
        LLM_FAIL(-1, "attention_prefill_bf16: heads %d / kv_heads %d / head_dim %d not supported", heads, kv_heads, head_dim);
    if (heads > 65535) LLM_FAIL(-1, "attention_prefill_bf16: too many heads");
    const float sl = scale * 1.4426950408889634f;
    const int page_shift = page_shift_of(page_size);
    dim3 grid(n_tiles, heads);
    auto launch = [&](auto kern, int D) {
        const size_t smem = (size_t)(kTile * D + 2 * 2 * kTile * D) * sizeof(bf16);
        if (set_smem(kern, smem, "attention_prefill_bf16")) return -2;
        llm_launch(kern, grid, kThreads, smem, stream, (const bf16*)q, q_stride, (const bf16*)cache, block_table, table_width,
                                               (const int4*)tiles, (bf16*)out, out_stride, heads, kv_heads, page_size,
                                               page_shift, window, sl);
        LLM_CHECK_LAUNCH("attention_prefill_bf16");
        return 0;
    };
    return head_dim == 64 ? launch(attn_prefill_kernel<64>, 64) : launch(attn_prefill_kernel<128>, 128);
}

// items: [n_items] token rows of the decoded tokens.  part_o needs n_items*heads*max_splits*head_dim floats,
// part_ml n_items*heads*max_splits*2 floats (both unused when max_splits == 1).
namespace {
int launch_decode(const void* q, int q_stride, const void* cache, long long cache_pages, const int* block_table,
                  int table_width, const int* items, int n_items, const int* token_request, const int* positions,
                  float* part_o, float* part_ml, void* out, int out_stride, int heads, int kv_heads, int head_dim,
                  int page_size, int window, float scale, int keys_per_split, int max_splits, const QkvParts* fused,
                  cudaStream_t stream);
}

// 1 if the decode kernel that fetches keys and values by TMA takes this shape (head sizes 64 and 128, pages of 8, 16,
// 32 or 64 tokens), else 0: llm_attention_decode_bf16 and its fused form take the rest.
LLM_API int llm_attention_decode_tma_supported(int heads, int kv_heads, int head_dim, int page_size) {
    return llm_attention_bf16_supported(heads, kv_heads, head_dim) &&
           (page_size == 8 || page_size == 16 || page_size == 32 || page_size == 64);
}

LLM_API int llm_attention_decode_bf16(const void* q, int q_stride, const void* cache, const int* block_table,
                                      int table_width, const int* items, int n_items, const int* token_request,
                                      const int* positions, float* part_o, float* part_ml, void* out, int out_stride,
                                      int heads, int kv_heads, int head_dim, int page_size, int window, float scale,
                                      int keys_per_split, int max_splits, cudaStream_t stream) {
    return launch_decode(q, q_stride, cache, 0, block_table, table_width, items, n_items, token_request, positions, part_o,
                         part_ml, out, out_stride, heads, kv_heads, head_dim, page_size, window, scale, keys_per_split,
                         max_splits, nullptr, stream);
}

// The same with keys and values fetched by TMA: `cache_pages` is the count of pages of the cache layer (its first
// dimension), which the tensor map needs; shapes as llm_attention_decode_tma_supported says.
LLM_API int llm_attention_decode_bf16_tma(const void* q, int q_stride, const void* cache, long long cache_pages,
                                          const int* block_table, int table_width, const int* items, int n_items,
                                          const int* token_request, const int* positions, float* part_o, float* part_ml,
                                          void* out, int out_stride, int heads, int kv_heads, int head_dim, int page_size,
                                          int window, float scale, int keys_per_split, int max_splits, cudaStream_t stream) {
    if (cache_pages <= 0 || !llm_attention_decode_tma_supported(heads, kv_heads, head_dim, page_size))
        LLM_FAIL(-1, "attention_decode_bf16_tma: heads %d / kv_heads %d / head_dim %d / page %d / %lld pages not supported",
                 heads, kv_heads, head_dim, page_size, cache_pages);
    return launch_decode(q, q_stride, cache, cache_pages, block_table, table_width, items, n_items, token_request, positions,
                         part_o, part_ml, out, out_stride, heads, kv_heads, head_dim, page_size, window, scale,
                         keys_per_split, max_splits, nullptr, stream);
}

// The same for single decoded tokens whose qkv product was left as k-split partial sums: `parts`
// [splits][tokens][(heads + 2 kv_heads) * head_dim] float32 (`split_stride` elements apart, at most 8 splits),
// cos / sin [tokens][head_dim / 2] of the tokens' positions (all dims rotated), `slots` [tokens] where each token's
// key and value go in `cache`.  Adds the parts, rotates queries and keys, stores key and value, and attends, in
// one kernel.  Every token of the step must be one of `items` (a token left out would never be stored).
LLM_API int llm_attention_decode_bf16_fused(const float* parts, int splits, long long split_stride, const float* cos_table,
                                            const float* sin_table, const int* slots, void* cache, const int* block_table,
                                            int table_width, const int* items, int n_items, const int* token_request,
                                            const int* positions, float* part_o, float* part_ml, void* out, int out_stride,
                                            int heads, int kv_heads, int head_dim, int page_size, int window, float scale,
                                            int keys_per_split, int max_splits, cudaStream_t stream) {
    if (!parts || !cos_table || !sin_table || !slots) LLM_FAIL(-1, "attention_decode_bf16_fused: parts, tables and slots are needed");
    if (splits < 1 || splits > kMaxParts || split_stride % 4 || ((heads + 2 * kv_heads) * head_dim) % 4)
        LLM_FAIL(-1, "attention_decode_bf16_fused: 1 to %d splits with a stride that is a multiple of 4 (got %d, %lld)",
                 kMaxParts, splits, split_stride);
    QkvParts f{parts, splits, (size_t)split_stride, cos_table, sin_table, slots, (bf16*)cache};
    return launch_decode(nullptr, 0, cache, 0, block_table, table_width, items, n_items, token_request, positions, part_o,
                         part_ml, out, out_stride, heads, kv_heads, head_dim, page_size, window, scale, keys_per_split,
                         max_splits, &f, stream);
}

// The fused form with keys and values fetched by TMA (`cache_pages` as in llm_attention_decode_bf16_tma).
LLM_API int llm_attention_decode_bf16_fused_tma(const float* parts, int splits, long long split_stride, const float* cos_table,
                                                const float* sin_table, const int* slots, void* cache, long long cache_pages,
                                                const int* block_table, int table_width, const int* items, int n_items,
                                                const int* token_request, const int* positions, float* part_o, float* part_ml,
                                                void* out, int out_stride, int heads, int kv_heads, int head_dim,
                                                int page_size, int window, float scale, int keys_per_split, int max_splits,
                                                cudaStream_t stream) {
    if (!parts || !cos_table || !sin_table || !slots) LLM_FAIL(-1, "attention_decode_bf16_fused_tma: parts, tables and slots are needed");
    if (splits < 1 || splits > kMaxParts || split_stride % 4 || ((heads + 2 * kv_heads) * head_dim) % 4)
        LLM_FAIL(-1, "attention_decode_bf16_fused_tma: 1 to %d splits with a stride that is a multiple of 4 (got %d, %lld)",
                 kMaxParts, splits, split_stride);
    if (cache_pages <= 0 || !llm_attention_decode_tma_supported(heads, kv_heads, head_dim, page_size))
        LLM_FAIL(-1, "attention_decode_bf16_fused_tma: heads %d / kv_heads %d / head_dim %d / page %d / %lld pages not supported",
                 heads, kv_heads, head_dim, page_size, cache_pages);
    QkvParts f{parts, splits, (size_t)split_stride, cos_table, sin_table, slots, (bf16*)cache};
    return launch_decode(nullptr, 0, cache, cache_pages, block_table, table_width, items, n_items, token_request, positions,
                         part_o, part_ml, out, out_stride, heads, kv_heads, head_dim, page_size, window, scale,
                         keys_per_split, max_splits, &f, stream);
}

namespace {
int launch_decode(const void* q, int q_stride, const void* cache, long long cache_pages, const int* block_table,
                  int table_width, const int* items, int n_items, const int* token_request, const int* positions,
                  float* part_o, float* part_ml, void* out, int out_stride, int heads, int kv_heads, int head_dim,
                  int page_size, int window, float scale, int keys_per_split, int max_splits, const QkvParts* fused,
                  cudaStream_t stream) {
    if (n_items == 0) return 0;
    if (!llm_attention_bf16_supported(heads, kv_heads, head_dim))
        LLM_FAIL(-1, "attention_decode_bf16: heads %d / kv_heads %d / head_dim %d not supported", heads, kv_heads, head_dim);
    if (keys_per_split <= 0 || keys_per_split % kTile) LLM_FAIL(-1, "attention_decode_bf16: keys_per_split must be a multiple of 64");
    if (max_splits < 1 || max_splits > kMaxMergeSplits || kv_heads > 65535 || n_items > 65535)
        LLM_FAIL(-1, "attention_decode_bf16: grid out of range (1 to %d splits, at most 65535 items and key/value heads)", kMaxMergeSplits);
    if (max_splits > 1 && (!part_o || !part_ml)) LLM_FAIL(-1, "attention_decode_bf16: scratch is missing");
    const float sl = scale * 1.4426950408889634f;
    const int page_shift = page_shift_of(page_size);
    dim3 grid(max_splits, kv_heads, n_items);
    auto launch = [&](auto kern, auto merge, int D) {
        size_t smem = (size_t)kStages * 2 * kTile * D * sizeof(bf16);
        const size_t merge_smem = (size_t)(4 * 16 * D + 2 * 4 * 16) * sizeof(float);
        if (merge_smem > smem) smem = merge_smem;
        if (set_smem(kern, smem, "attention_decode_bf16")) return -2;
        llm_launch(kern, grid, kThreads, smem, stream, (const bf16*)q, q_stride, (const bf16*)cache, block_table, table_width, items,
                                               token_request, positions, part_o, part_ml, (bf16*)out, out_stride, heads,
                                               kv_heads, page_size, page_shift, window, sl, keys_per_split, max_splits,
                                               fused ? *fused : QkvParts{});
        LLM_CHECK_LAUNCH("attention_decode_bf16");
        if (max_splits > 1) {
            llm_launch(merge, dim3(n_items, heads), dim3(D, max_splits > kMergeSplits ? kMergeGroups : 1), 0, stream, part_o, part_ml, items, positions, (bf16*)out, out_stride, heads,
                                                          window, keys_per_split, max_splits);
            LLM_CHECK_LAUNCH("attention_merge");
        }
        return 0;
    };
    if (cache_pages > 0) {
        // keys and values by TMA: the cache layer as a [pages * 2 * kv_heads * page_size, head_dim] matrix, one box per page and 64 dims
        const uint64_t kv_rows = (uint64_t)cache_pages * 2 * kv_heads * page_size;
        if (kv_rows > 0x7fffffffull) LLM_FAIL(-1, "attention_decode_bf16_tma: the cache layer has too many rows for 32-bit TMA coordinates");
        CUtensorMap mkv;
        if (int rc = llm_tensor_map_2d(cache, kv_rows, (uint64_t)head_dim, (uint32_t)page_size, 64, &mkv)) return rc;
        auto launch_tma = [&](auto kern, auto merge, int D) {
            size_t smem = (size_t)(D == 64 ? tma_stages<64>() : tma_stages<128>()) * 2 * kTile * D * sizeof(bf16);
            const size_t merge_smem = (size_t)(4 * 16 * D + 2 * 4 * 16) * sizeof(float);
            if (merge_smem > smem) smem = merge_smem;
            smem += 1024;                          // the stages start at a multiple of 1024 bytes (128-byte swizzle)
            if (set_smem(kern, smem, "attention_decode_bf16_tma")) return -2;
            llm_launch(kern, grid, kTmaThreads, smem, stream, mkv, (const bf16*)q, q_stride, block_table, table_width, items,
                       token_request, positions, part_o, part_ml, (bf16*)out, out_stride, heads, kv_heads, page_size,
                       page_shift, window, sl, keys_per_split, max_splits, fused ? *fused : QkvParts{});
            LLM_CHECK_LAUNCH("attention_decode_bf16_tma");
            if (max_splits > 1) {
                llm_launch(merge, dim3(n_items, heads), dim3(D, max_splits > kMergeSplits ? kMergeGroups : 1), 0, stream, part_o, part_ml, items, positions, (bf16*)out, out_stride,
                           heads, window, keys_per_split, max_splits);
                LLM_CHECK_LAUNCH("attention_merge");
            }
            return 0;
        };
        if (fused)
            return head_dim == 64 ? launch_tma(attn_decode_tma_kernel<64, true>, attn_merge_kernel<64>, 64)
                                  : launch_tma(attn_decode_tma_kernel<128, true>, attn_merge_kernel<128>, 128);
        return head_dim == 64 ? launch_tma(attn_decode_tma_kernel<64, false>, attn_merge_kernel<64>, 64)
                              : launch_tma(attn_decode_tma_kernel<128, false>, attn_merge_kernel<128>, 128);
    }
    if (fused)
        return head_dim == 64 ? launch(attn_decode_kernel<64, true>, attn_merge_kernel<64>, 64)
                              : launch(attn_decode_kernel<128, true>, attn_merge_kernel<128>, 128);
    return head_dim == 64 ? launch(attn_decode_kernel<64, false>, attn_merge_kernel<64>, 64)
                          : launch(attn_decode_kernel<128, false>, attn_merge_kernel<128>, 128);
}
}  // namespace

const int* llm_attention_decode_status_word() {
    void* p = nullptr;
    return cudaGetSymbolAddress(&p, g_decode_status) == cudaSuccess ? static_cast<const int*>(p) : nullptr;
}

// Reads and clears the status word of the decode attention: 0, or (6 << 16 | item) of the first item whose keys
// keys_per_split * max_splits did not cover (its result is wrong: the caller broke the contract stated above).
LLM_API int llm_attention_decode_status() {
    int v = 0, zero = 0;
    if (cudaMemcpyFromSymbol(&v, g_decode_status, sizeof(int)) != cudaSuccess) return -1;
    if (v) cudaMemcpyToSymbol(g_decode_status, &zero, sizeof(int));
    return v;
}

// ---------------------------------------------------------------------------------------
// The same decode attention with its scratch inside the library (see llm_no_alloc.h).
// ---------------------------------------------------------------------------------------
#include "llm_no_alloc.h"

#include <mutex>

namespace {

// Partials of the split-key decode kernel for callers without an allocator.  In host code
// this name is only a handle for cudaGetSymbolAddress; the kernels get the device address.
static __device__ __align__(256) float g_static_scratch[LLM_STATIC_SCRATCH_FLOATS];

constexpr int kMaxDevices = 64;
float* g_static_scratch_ptr[kMaxDevices] = {};
std::mutex g_static_scratch_mutex;

// Device address of the array on the current device; looked up once per device.
int static_scratch_address(float** ptr) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) LLM_FAIL(-2, "attention_decode_bf16_static: cudaGetDevice: %s", cudaGetErrorString(e));
    if (dev < 0 || dev >= kMaxDevices) LLM_FAIL(-1, "attention_decode_bf16_static: device index %d out of range", dev);
    std::lock_guard<std::mutex> lock(g_static_scratch_mutex);
    if (!g_static_scratch_ptr[dev]) {
        void* p = nullptr;
        e = cudaGetSymbolAddress(&p, g_static_scratch);
        if (e != cudaSuccess || !p)
            LLM_FAIL(-2, "attention_decode_bf16_static: cudaGetSymbolAddress: %s", cudaGetErrorString(e));
        g_static_scratch_ptr[dev] = static_cast<float*>(p);
    }
    *ptr = g_static_scratch_ptr[dev];
    return 0;
}

}  // namespace

LLM_API int llm_attention_decode_bf16_static(const void* q, int q_stride, const void* cache, const int* block_table,
                                             int table_width, const int* items, int n_items, const int* token_request,
                                             const int* positions, void* out, int out_stride, int heads, int kv_heads,
                                             int head_dim, int page_size, int window, float scale, int keys_per_split,
                                             int max_splits, cudaStream_t stream) {
    if (n_items <= 0) return 0;
    if (heads <= 0 || head_dim <= 0 || max_splits < 1)
        LLM_FAIL(-1, "attention_decode_bf16_static: heads, head_dim and max_splits must be positive");
    const unsigned long long rows = (unsigned long long)n_items * heads * max_splits;
    const unsigned long long need = rows * (unsigned long long)(head_dim + 2);
    if (need > LLM_STATIC_SCRATCH_FLOATS)
        LLM_FAIL(-1, "attention_decode_bf16_static: %d items x %d heads x %d splits x head_dim %d need %llu floats of "
                     "scratch, the built-in array holds %u; use fewer items or splits per call, or "
                     "llm_attention_decode_bf16 with your own scratch",
                 n_items, heads, max_splits, head_dim, need, LLM_STATIC_SCRATCH_FLOATS);
    float* scratch = nullptr;
    if (int rc = static_scratch_address(&scratch)) return rc;
    float* part_o = scratch;                        // rows * head_dim floats
    float* part_ml = scratch + rows * head_dim;     // rows * 2 floats
    return llm_attention_decode_bf16(q, q_stride, cache, block_table, table_width, items, n_items, token_request,
                                     positions, part_o, part_ml, out, out_stride, heads, kv_heads, head_dim, page_size,
                                     window, scale, keys_per_split, max_splits, stream);
}

LLM_TRACE_EXPORT(attention_bf16)
