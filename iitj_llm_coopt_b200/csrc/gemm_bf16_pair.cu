// bfloat16 matrix products for many tokens (prompt portions): y = x . W^T with x [T, K] and W [N, K]
// row-major (F.linear of engine/model.py:194, 208, 210-211, 218), float32 accumulation in tensor memory.
//
// A persistent kernel of CTA pairs (clusters of two).  A pair owns a tile of 256 tokens x 256 accumulator
// columns and issues tcgen05.mma.cta_group::2 (M = 256, N = 256, K = 16): each CTA stages its own 128 token
// rows of x and 128 of the 256 weight rows per 64-wide k-block (TMA, 128-byte swizzle, no multicast), the
// tensor cores of both SMs read both halves of the weights, and each CTA's tensor memory holds the
// accumulator of its own 128 tokens.  Two accumulators (2 x 256 columns) alternate, so the epilogue warps
// drain tile i while the MMAs of tile i+1 run.
//
// Roles per CTA: warp 0 TMA producer, warp 1 tensor-memory allocation and (leader CTA only) MMA issue,
// warps 2-9 epilogue.  Barriers: full[s] in the leader collects the bytes of both CTAs' loads; empty[s]
// and acc_full[a] exist in both CTAs and are signalled by tcgen05.commit with a two-CTA mask; acc_empty[a]
// in the leader counts the sixteen epilogue warps of the pair.
//
// SwiGLU variant: the 256 accumulator columns are 128 gate columns (weight rows f0.., staged by the
// leader) and the 128 up columns of the same features (rows I + f0.., staged by its peer); the epilogue
// writes silu(gate) * up (engine/model.py:251-252), so the [T, 2I] intermediate never exists.
//
// Filling the last round ("stream-K" on the tail): with T tiles on C clusters the last T mod C tiles would
// leave clusters idle.  Those tail tiles are instead cut along k into C equal runs of k-blocks, one per
// cluster.  A cluster whose run starts inside a tile adds up its k-blocks, writes the float32 partial sums to
// scratch and counts itself on that tile's counter; the cluster that started the tile waits (bounded) for
// the counter, adds the partial sums in cluster order and stores the tile.  A cluster finishes its partial
// run before it starts to wait for anybody, so no wait can depend on itself.  Counters and scratch are
// touched only after griddepcontrol.wait, so back-to-back launches on one stream may share them.
//
// Leaving: a bfloat16 tile goes from tensor memory through registers into a 128-byte-swizzled staging tile
// per epilogue warp (32 rows x 64 columns) and from there to global memory by a TMA store, which also clips
// rows and columns past the matrix; float32 results and unaligned outputs are stored from registers.
//
// Every wait on an mbarrier is bounded; a wait that runs out records a code (llm_gemm_bf16_pair_status)
// and all roles fall through to the teardown, where the pair frees its tensor memory.
#include "tcgen05_common.cuh"

namespace {

typedef __nv_bfloat16 bf16;

constexpr int kTokCta = 128;                   // token rows per CTA (UMMA M = 256 over the pair)
constexpr int kAccCols = 256;                  // accumulator columns (UMMA N)
constexpr int kBlockK = 64;                    // 128 bytes per row: one swizzle row
constexpr int kStages = 6;
constexpr int kHalfBytes = 128 * kBlockK * 2;  // 16 KiB: one operand tile of one CTA
constexpr int kStageBytes = 2 * kHalfBytes;    // x tile then W tile
constexpr int kThreads = 320;                  // warp 0 TMA, warp 1 MMA, warps 2-9 epilogue
constexpr int kEpiWarps = 8;                   // per CTA; two per quarter of the TMEM lanes, half of the columns each
constexpr int kTmemCols = 512;
constexpr int kStoreBytes = 32 * 128;          // one epilogue warp's staging tile for a TMA store: 32 rows of 128 bytes

__device__ int g_pair_status = 0;
__device__ __forceinline__ void give_up(int code) { atomicCAS(&g_pair_status, 0, (code << 16) | (int)(blockIdx.x & 0xffff)); }

__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
// Address of the same shared-memory location in the CTA `rank` of this cluster.
__device__ __forceinline__ uint32_t map_to_cta(uint32_t addr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
    return r;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_remote(uint32_t cluster_addr) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// TMA tile load of a CTA pair: the bytes are counted on the barrier at `bar_cluster_addr`, which may
// lie in the other CTA of the pair.
__device__ __forceinline__ void tma_load_2d_pair(void* smem_dst, const CUtensorMap* map, uint32_t bar_cluster_addr, int x, int y) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(smem_u32(smem_dst)), "l"(map), "r"(bar_cluster_addr), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void umma_f16_pair(uint32_t tmem_d, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
// Arrives on the barrier at this offset in both CTAs of the pair once all MMAs issued so far are done.
__device__ __forceinline__ void umma_commit_pair(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                 ::"r"(smem_u32(bar)), "h"((uint16_t)3) : "memory");
}

struct PairArgs {
    void* out;            // [tokens, ldc] bf16 or f32
    int out_f32;
    int n_feat;           // output features (I for SwiGLU, else N)
    int tokens;
    int ldc;
    int k_blocks;
    int tok_tiles;        // ceil(tokens / 256)
    int feat_tiles;       // ceil(n_feat / features per tile)
    int n_tiles;          // tok_tiles * feature tiles
    int vec_ok;           // rows of `out` allow 16-byte stores
    int tma_out;          // `out` is bfloat16 with a tensor map: tiles leave through shared memory and TMA stores
    int full_rounds;      // rounds in which cluster c runs tile c + round * clusters whole
    int tail;             // tiles after the full rounds that are cut along k over all clusters (0: none)
    float* partials;      // [clusters][2][128][256] float32 partial sums of tail tiles
    int* counters;        // [2 * tail]: parts arrived, owner warps done; zero between launches
};

enum ItemMode { ITEM_WHOLE = 0, ITEM_OWNER = 1, ITEM_PART = 2 };
struct Item {
    int tile, k0, k1;     // k-blocks [k0, k1) of the tile
    int mode;             // whole tile; first run of a tile (adds the parts and stores); a later run (writes a part)
    int n_parts;          // ITEM_OWNER: the next n_parts clusters hold the other runs of this tile
};

// The i-th piece of work of cluster c out of C, the same for every role of the pair; false past the end.
__device__ __forceinline__ bool get_item(const PairArgs& a, int c, int C, int i, Item& it) {
    const int n_kb = a.k_blocks;
    it.mode = ITEM_WHOLE; it.n_parts = 0; it.k0 = 0; it.k1 = n_kb;
    if (i < a.full_rounds) {
        it.tile = c + i * C;
        return it.tile < a.n_tiles;
    }
    const int j = i - a.full_rounds;
    if (a.tail == 0 || j > 1) return false;
    const long long U = (long long)a.tail * n_kb;
    const long long u0 = (long long)c * U / C, u1 = (long long)(c + 1) * U / C;
    int ta = (int)(u0 / n_kb);
    long long ta_end = (long long)(ta + 1) * n_kb;
    if (j == 0) {
        it.k0 = (int)(u0 - (long long)ta * n_kb);
        it.k1 = (int)((u1 < ta_end ? u1 : ta_end) - (long long)ta * n_kb);
    } else {
        if (u1 <= ta_end) return false;
        ++ta;
        it.k0 = 0;
        it.k1 = (int)(u1 - ta_end);
        ta_end += n_kb;
    }
    if (it.k1 <= it.k0) return false;
    it.tile = a.full_rounds * C + ta;
    if (it.k0 > 0) {
        it.mode = ITEM_PART;
    } else if (it.k1 < n_kb) {
        it.mode = ITEM_OWNER;
        for (int q = c + 1; q < C && (long long)q * U / C < ta_end; ++q) ++it.n_parts;
    }
    return true;
}

// Tile `t` of the grid -> (feature tile, token tile).  Token tiles are walked in groups of eight with the
// feature tiles outside the group, so the clusters that run at the same time share a few x tiles and a few
// W tiles in L2 whatever the number of tokens.
__device__ __forceinline__ void tile_coords(const PairArgs& a, int t, int& ft, int& tt) {
    const int group_tiles = 8 * a.feat_tiles;
    const int g = t / group_tiles, r = t - g * group_tiles;
    const int rest = a.tok_tiles - g * 8;
    const int gsize = rest < 8 ? rest : 8;
    ft = r / gsize;
    tt = g * 8 + (r - ft * gsize);
}

__device__ __forceinline__ uint32_t pack_bf16(float a, float b) {
    __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&v);
}
__device__ __forceinline__ int ld_acquire(const int* p) {
    int v;
    asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

template <bool SWIGLU>
__global__ void __launch_bounds__(kThreads, 1)
gemm_pair_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w,
                 const __grid_constant__ CUtensorMap map_out, const PairArgs a) {
    extern __shared__ unsigned char smem_raw[];
    unsigned char* tiles = reinterpret_cast<unsigned char*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    __shared__ __align__(8) uint64_t full_bar[kStages], empty_bar[kStages], acc_full[2], acc_empty[2];
    __shared__ uint32_t tmem_base_slot;
    __shared__ volatile int failed;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();
    const bool leader = rank == 0;
    const int cluster_id = blockIdx.x >> 1, n_clusters = gridDim.x >> 1;
    constexpr int kFeatTile = SWIGLU ? 128 : 256;   // output features per tile

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
        for (int s = 0; s < 2; ++s) { mbar_init(&acc_full[s], 1); mbar_init(&acc_empty[s], 2 * kEpiWarps); }
        failed = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_slot)), "r"(kTmemCols));
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::);
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    cluster_sync_all();                       // the peer's barriers exist before anything signals them
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = tmem_base_slot;

    pdl_trigger();

    if (warp == 0 && lane == 0) {
        // ---- producer: this CTA's half of both operands ----------------------------------------
        // A cursor walks the k-blocks of this cluster's items; `rows` gives the first row of each operand.
        struct Cursor { int i, kb, k1, tok_row, w_row; bool valid; };
        auto open_item = [&](Cursor& cu) {
            Item it;
            cu.valid = get_item(a, cluster_id, n_clusters, cu.i, it);
            if (!cu.valid) return;
            int ft, tt;
            tile_coords(a, it.tile, ft, tt);
            cu.kb = it.k0; cu.k1 = it.k1;
            cu.tok_row = tt * 256 + (int)rank * kTokCta;
            // each CTA stages half of the MMA's 256 weight rows: gate rows (leader) and up rows (peer), or the
            // two halves of the tile's features
            cu.w_row = SWIGLU ? (int)rank * a.n_feat + ft * 128 : ft * 256 + (int)rank * 128;
        };
        auto advance = [&](Cursor& cu) {
            if (++cu.kb == cu.k1) { ++cu.i; open_item(cu); }
        };
        auto full_addr = [&](int s) { return map_to_cta(smem_u32(&full_bar[s]), 0); };   // the leader's barrier
        // The weights depend on no earlier kernel: the first ring of weight tiles is requested before the
        // wait for the previous kernel, the activation tiles (its output) after it.
        Cursor cw, cx;
        cw.i = 0; open_item(cw);
        int pre = 0;
        for (; pre < kStages && cw.valid; ++pre) {
            if (leader) mbar_expect_tx(&full_bar[pre], 2 * kStageBytes);
            tma_load_2d_pair(tiles + (size_t)pre * kStageBytes + kHalfBytes, &map_w, full_addr(pre), cw.kb * kBlockK, cw.w_row);
            advance(cw);
        }
        pdl_wait();
        cx.i = 0; open_item(cx);
        for (int i = 0; i < pre; ++i) {
            tma_load_2d_pair(tiles + (size_t)i * kStageBytes, &map_x, full_addr(i), cx.kb * kBlockK, cx.tok_row);
            advance(cx);
        }
        int s = 0;
        uint32_t parity = 0;                          // of the first reuse of a stage
        while (cx.valid) {
            if (!mbar_wait(&empty_bar[s], parity)) { give_up(1); failed = 1; break; }
            unsigned char* st = tiles + (size_t)s * kStageBytes;
            const uint32_t bar = full_addr(s);
            if (leader) mbar_expect_tx(&full_bar[s], 2 * kStageBytes);
            tma_load_2d_pair(st + kHalfBytes, &map_w, bar, cx.kb * kBlockK, cx.w_row);
            tma_load_2d_pair(st, &map_x, bar, cx.kb * kBlockK, cx.tok_row);
            advance(cx);
            if (++s == kStages) { s = 0; parity ^= 1; }
        }
    } else if (warp == 1 && lane == 0 && leader) {
        // ---- MMA issuer of the pair ---------------------------------------------------------------
        constexpr uint32_t idesc = umma_idesc(256, kAccCols);
        int s = 0;
        uint32_t parity = 0;
        bool ok = true;
        Item it;
        for (int i = 0; ok && get_item(a, cluster_id, n_clusters, i, it); ++i) {
            const int as = i & 1, use = i >> 1;
            if (use > 0 && !mbar_wait(&acc_empty[as], (use - 1) & 1)) { give_up(4); failed = 1; break; }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint32_t acc = tmem_base + (uint32_t)(as * kAccCols);
            for (int kb = it.k0; kb < it.k1; ++kb) {
                if (!mbar_wait(&full_bar[s], parity)) { give_up(2); failed = 1; ok = false; break; }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                unsigned char* st = tiles + (size_t)s * kStageBytes;
                const uint64_t da = umma_desc(st), db = umma_desc(st + kHalfBytes);
#pragma unroll
                for (int k = 0; k < kBlockK / 16; ++k)
                    umma_f16_pair(acc, da + 2 * k, db + 2 * k, idesc, (kb > it.k0 || k > 0) ? 1u : 0u);
                umma_commit_pair(&empty_bar[s]);
                if (++s == kStages) { s = 0; parity ^= 1; }
            }
            umma_commit_pair(&acc_full[as]);
        }
    } else if (warp >= 2) {
        // ---- epilogue: tensor memory -> registers -> global -----------------------------------------
        const int quarter = warp & 3;             // a warp may only read TMEM lanes [32 * (warp % 4), +32)
        const int half = (warp - 2) >> 2;         // which half of the columns this warp drains
        const int row = quarter * 32 + lane;      // accumulator row of this thread
        const uint32_t lane_addr = tmem_base + ((uint32_t)(quarter * 32) << 16);
        const uint32_t acc_empty_leader[2] = {map_to_cta(smem_u32(&acc_empty[0]), 0), map_to_cta(smem_u32(&acc_empty[1]), 0)};
        constexpr int kCols = SWIGLU ? 64 : 128;  // output columns per warp
        unsigned char* stage_out = tiles + (size_t)kStages * kStageBytes + (size_t)(warp - 2) * kStoreBytes;
        pdl_wait();                               // nothing is stored before the previous kernel has finished
        Item it;
        for (int i = 0; get_item(a, cluster_id, n_clusters, i, it); ++i) {
            const int as = i & 1, use = i >> 1;
            if (!mbar_wait(&acc_full[as], use & 1) || failed) { if (!failed) give_up(3); failed = 1; break; }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint32_t acc = lane_addr + (uint32_t)(as * kAccCols);
            const int ti = it.tile - a.full_rounds * n_clusters;     // index among the tail tiles
            if (it.mode == ITEM_PART) {
                // raw float32 sums of this run: [cluster][rank][256 columns][128 rows], so that the 32 rows of a
                // warp are 128 contiguous bytes
                float* dst = a.partials + ((size_t)cluster_id * 2 + rank) * 128 * kAccCols + (size_t)(half * 128) * 128 + row;
#pragma unroll 1
                for (int c0 = 0; c0 < 128; c0 += 32) {
                    uint32_t g[32];
                    tmem_ld32(acc + half * 128 + c0, g);
                    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
                    for (int c = 0; c < 32; ++c) dst[(size_t)(c0 + c) * 128] = __uint_as_float(g[c]);
                }
                asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                __threadfence();
                __syncwarp();
                if (lane == 0) {
                    mbar_arrive_remote(acc_empty_leader[as]);
                    atomicAdd(&a.counters[2 * ti], 1);
                }
                continue;
            }
            if (it.mode == ITEM_OWNER) {
                int ok = 1;
                if (lane == 0) {
                    const int want = 2 * kEpiWarps * it.n_parts;
                    ok = 0;
                    for (uint32_t spin = 0; spin < (1u << 20); ++spin) {
                        if (ld_acquire(&a.counters[2 * ti]) >= want) { ok = 1; break; }
                        __nanosleep(64);
                    }
                }
                ok = __shfl_sync(0xffffffffu, ok, 0);
                if (!ok) { give_up(5); failed = 1; }      // the tile is stored without the missing parts
            }
            int ft, tt;
            tile_coords(a, it.tile, ft, tt);
            const int tok = tt * 256 + (int)rank * kTokCta + row;
            const int feat0 = ft * kFeatTile + half * kCols;
            const bool row_ok = tok < a.tokens;
            const float* part0 = a.partials + ((size_t)(cluster_id + 1) * 2 + rank) * 128 * kAccCols + row;
#pragma unroll 1
            for (int c0 = 0; c0 < kCols; c0 += 32) {
                uint32_t g[32];
                float v[32];
                if (feat0 + c0 >= a.n_feat) break;          // uniform over the warp
                const int gcol = half * kCols + c0;          // accumulator column of g[0]
                tmem_ld32(acc + gcol, g);
                if (SWIGLU) {
                    uint32_t u[32];
                    tmem_ld32(acc + 128 + gcol, u);
                    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                    if (it.mode == ITEM_OWNER) {
                        for (int p = 0; p < it.n_parts; ++p) {
                            const float* src = part0 + (size_t)p * 2 * 128 * kAccCols + (size_t)gcol * 128;
#pragma unroll
                            for (int c = 0; c < 32; ++c) {
                                g[c] = __float_as_uint(__uint_as_float(g[c]) + __ldcg(src + (size_t)c * 128));
                                u[c] = __float_as_uint(__uint_as_float(u[c]) + __ldcg(src + (size_t)(128 + c) * 128));
                            }
                        }
                    }
#pragma unroll
                    for (int c = 0; c < 32; ++c) {
                        const float gv = __uint_as_float(g[c]);
                        v[c] = gv / (1.0f + __expf(-gv)) * __uint_as_float(u[c]);
                    }
                } else {
                    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
                    for (int c = 0; c < 32; ++c) v[c] = __uint_as_float(g[c]);
                    if (it.mode == ITEM_OWNER) {
                        for (int p = 0; p < it.n_parts; ++p) {
                            const float* src = part0 + (size_t)p * 2 * 128 * kAccCols + (size_t)gcol * 128;
#pragma unroll
                            for (int c = 0; c < 32; ++c) v[c] += __ldcg(src + (size_t)c * 128);
                        }
                    }
                }
                const int f = feat0 + c0;
                if (a.tma_out) {
                    // 32 columns = 64 bytes of this thread's row, as four 16-byte pieces of the swizzled staging tile
                    const int sub = (c0 >> 5) & 1;
                    if (sub == 0) {             // the tile's previous store must have read it
                        if (lane == 0) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
                        __syncwarp();
                    }
                    const uint32_t row_addr = smem_u32(stage_out) + lane * 128;
#pragma unroll
                    for (int q = 0; q < 4; ++q) {
                        const uint32_t dst = row_addr + (uint32_t)(((sub * 4 + q) ^ (lane & 7)) << 4);
                        asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(dst), "r"(pack_bf16(v[8 * q], v[8 * q + 1])),
                                     "r"(pack_bf16(v[8 * q + 2], v[8 * q + 3])), "r"(pack_bf16(v[8 * q + 4], v[8 * q + 5])),
                                     "r"(pack_bf16(v[8 * q + 6], v[8 * q + 7])) : "memory");
                    }
                    if (sub == 1 || c0 + 32 >= kCols || f + 32 >= a.n_feat) {
                        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                        __syncwarp();
                        if (lane == 0 && tok - lane < a.tokens) {
                            asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];"
                                         ::"l"(&map_out), "r"(smem_u32(stage_out)), "r"(f & ~63), "r"(tok) : "memory");
                            asm volatile("cp.async.bulk.commit_group;" ::: "memory");
                        }
                    }
                    continue;
                }
                if (!row_ok) continue;
                const bool whole = a.vec_ok && f + 32 <= a.n_feat;
                if (a.out_f32) {
                    float* dst = (float*)a.out + (size_t)tok * a.ldc + f;
                    if (whole) {
#pragma unroll
                        for (int c = 0; c < 32; c += 4) *reinterpret_cast<float4*>(dst + c) = make_float4(v[c], v[c + 1], v[c + 2], v[c + 3]);
                    } else {
#pragma unroll
                        for (int c = 0; c < 32; ++c)
                            if (f + c < a.n_feat) dst[c] = v[c];
                    }
                } else {
                    bf16* dst = (bf16*)a.out + (size_t)tok * a.ldc + f;
                    if (whole) {
#pragma unroll
                        for (int c = 0; c < 32; c += 8)
                            *reinterpret_cast<uint4*>(dst + c) = make_uint4(pack_bf16(v[c], v[c + 1]), pack_bf16(v[c + 2], v[c + 3]),
                                                                            pack_bf16(v[c + 4], v[c + 5]), pack_bf16(v[c + 6], v[c + 7]));
                    } else {
#pragma unroll
                        for (int c = 0; c < 32; ++c)
                            if (f + c < a.n_feat) dst[c] = __float2bfloat16_rn(v[c]);
                    }
                }
            }
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) {
                mbar_arrive_remote(acc_empty_leader[as]);
                if (it.mode == ITEM_OWNER && atomicAdd(&a.counters[2 * ti + 1], 1) == 2 * kEpiWarps - 1) {
                    a.counters[2 * ti] = 0;           // every owner warp has seen the count: ready for the next launch
                    a.counters[2 * ti + 1] = 0;
                }
            }
        }
        if (lane == 0) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");     // this warp's stores are complete
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    cluster_sync_all();                       // both CTAs are done with the pair's tensor memory and barriers
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols));
    }
}

constexpr size_t kSmemBytes = (size_t)kStages * kStageBytes + (size_t)kEpiWarps * kStoreBytes + 1024;

// Clusters of two that the device runs at once (0 after an error); sets the kernel's shared-memory limit.
template <bool SWIGLU>
int pair_clusters_of() {
    static int max_clusters = 0;               // per instantiation; the same on every device of one kind
    if (max_clusters) return max_clusters;
    auto kern = gemm_pair_kernel<SWIGLU>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemBytes);
    if (e != cudaSuccess) {
        snprintf(llm_error_buffer(), 512, "gemm_bf16_pair: cudaFuncSetAttribute: %s", cudaGetErrorString(e));
        return 0;
    }
    cudaLaunchConfig_t probe = {};
    cudaLaunchAttribute pa[1];
    pa[0].id = cudaLaunchAttributeClusterDimension;
    pa[0].val.clusterDim.x = 2; pa[0].val.clusterDim.y = 1; pa[0].val.clusterDim.z = 1;
    int dev = 0, sms = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    probe.gridDim = dim3(sms & ~1); probe.blockDim = dim3(kThreads); probe.dynamicSmemBytes = kSmemBytes;
    probe.attrs = pa; probe.numAttrs = 1;
    int n = 0;
    e = cudaOccupancyMaxActiveClusters(&n, kern, &probe);
    if (e != cudaSuccess || n < 1) { cudaGetLastError(); n = sms / 2; }
    if (n > sms / 2) n = sms / 2;
    max_clusters = n;
    return n;
}
int pair_clusters(bool swiglu) { return swiglu ? pair_clusters_of<true>() : pair_clusters_of<false>(); }

template <bool SWIGLU>
int launch_pair(const CUtensorMap& mx, const CUtensorMap& mw, const CUtensorMap& mo, const PairArgs& a, int clusters, cudaStream_t stream) {
    auto kern = gemm_pair_kernel<SWIGLU>;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(2 * clusters);
    cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = kSmemBytes;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
    cfg.numAttrs = 1;
    if (llm_pdl_enabled()) {
        attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[1].val.programmaticStreamSerializationAllowed = 1;
        cfg.numAttrs = 2;
    }
    cfg.attrs = attr;
    cudaError_t e = cudaLaunchKernelEx(&cfg, kern, mx, mw, mo, a);
    if (e != cudaSuccess) LLM_FAIL(-2, "gemm_bf16_pair: %s", cudaGetErrorString(e));
    return 0;
}

}  // namespace

// Scratch the tail split needs: floats of partial sums (`what` 0) and ints of counters (`what` 1, zeroed once
// by the caller); 0 if the kernel cannot be set up.
LLM_API int llm_gemm_bf16_pair_scratch(int what) {
    const int c0 = pair_clusters(false), c1 = pair_clusters(true);
    const int c = c0 > c1 ? c0 : c1;
    return what == 0 ? c * 2 * 128 * kAccCols : 2 * c;
}

// out = x . w^T for many tokens.  x [tokens, K] bf16, w [n (or 2n with swiglu), K] bf16;
// out bf16 (out_f32 == 0) or float32 [tokens, ldc].  With `partials` and `counters` (sizes from
// llm_gemm_bf16_pair_scratch) the tiles of the last, partly filled round are cut along k over all clusters.
LLM_API int llm_gemm_bf16_pair(const void* x, const void* w, void* out, int out_f32, int tokens, int n, int K, int ldc,
                               int swiglu, float* partials, int* counters, cudaStream_t stream) {
    if (tokens == 0 || n == 0) return 0;
    if (K % 8) LLM_FAIL(-1, "gemm_bf16_pair: K %d must be a multiple of 8", K);
    if (swiglu && out_f32) LLM_FAIL(-1, "gemm_bf16_pair: the SwiGLU variant writes bfloat16");
    const int w_rows = swiglu ? 2 * n : n;
    CUtensorMap mx, mw;
    if (int rc = llm_tensor_map_2d(x, tokens, K, 128, kBlockK, &mx)) return rc;
    if (int rc = llm_tensor_map_2d(w, w_rows, K, 128, kBlockK, &mw)) return rc;
    PairArgs a;
    a.out = out;
    a.out_f32 = out_f32;
    a.n_feat = n;
    a.tokens = tokens;
    a.ldc = ldc;
    a.k_blocks = (K + kBlockK - 1) / kBlockK;
    a.tok_tiles = (tokens + 255) / 256;
    a.feat_tiles = (n + (swiglu ? 127 : 255)) / (swiglu ? 128 : 256);
    const long long tiles = (long long)a.tok_tiles * a.feat_tiles;
    if (tiles > (1 << 30)) LLM_FAIL(-1, "gemm_bf16_pair: too many tiles");
    a.n_tiles = (int)tiles;
    const int max_clusters = pair_clusters(swiglu != 0);
    if (max_clusters < 1) return -2;
    // Whole tiles round by round; the last round is cut along k when it would leave a fifth of the clusters
    // or more idle and k is long: writing, awaiting and adding the partial sums costs about as much as a
    // third of a 4096-deep tile, so the cut pays from about 8192 on (measured at 2048 tokens of the 8B shapes:
    // K = 4096: 54 -> 59 us, K = 14336: 186 -> 178 us; at 4096 tokens 428 -> 383 us).
    int clusters = a.n_tiles < max_clusters ? a.n_tiles : max_clusters;
    a.full_rounds = (a.n_tiles + clusters - 1) / clusters;
    a.tail = 0;
    a.partials = partials;
    a.counters = counters;
    const int rem = a.n_tiles % max_clusters;
    if (partials && counters && rem > 0 && rem * 5 <= max_clusters * 4 && a.k_blocks >= 128) {
        clusters = max_clusters;
        a.full_rounds = a.n_tiles / max_clusters;
        a.tail = rem;
    }
    const int elem = out_f32 ? 4 : 2;
    a.vec_ok = (((uintptr_t)out & 15) == 0 && ((size_t)ldc * elem) % 16 == 0) ? 1 : 0;
    // bfloat16 results whose rows are packed and 16-byte aligned leave by TMA stores
    CUtensorMap mo = mx;
    a.tma_out = (!out_f32 && ldc == n && n % 8 == 0 && ((uintptr_t)out & 15) == 0) ? 1 : 0;
    if (a.tma_out)
        if (int rc = llm_tensor_map_2d(out, tokens, n, 32, 64, &mo)) return rc;
    return swiglu ? launch_pair<true>(mx, mw, mo, a, clusters, stream) : launch_pair<false>(mx, mw, mo, a, clusters, stream);
}

const int* llm_gemm_bf16_pair_status_word() {
    void* p = nullptr;
    return cudaGetSymbolAddress(&p, g_pair_status) == cudaSuccess ? static_cast<const int*>(p) : nullptr;
}

// Reads and clears the status word: 0, or (code << 16 | block) of the first CTA whose wait ran out (code 1: producer
// waiting for a free stage, 2: MMA issuer waiting for data, 3: epilogue waiting for an accumulator, 4: MMA issuer
// waiting for a drained accumulator, 5: a tile's owner waiting for the other clusters' partial sums).
LLM_API int llm_gemm_bf16_pair_status() {
    int v = 0, zero = 0;
    if (cudaMemcpyFromSymbol(&v, g_pair_status, sizeof(int)) != cudaSuccess) return -1;
    if (v) cudaMemcpyToSymbol(g_pair_status, &zero, sizeof(int));
    return v;
}

LLM_TRACE_EXPORT(gemm_bf16_pair)
