// bfloat16 matrix products on the fifth-generation tensor cores: y = x . W^T with x [T, K]
// and W [N, K] row-major (F.linear of engine/model.py:194, 208, 210-211, 218), float32
// accumulation in tensor memory.
//
// The weight rows are the 128-row side of the MMA tile ("swap-AB"): one CTA owns 128 output
// features and a tile of 16..256 tokens, so a decode step with a handful of tokens still
// streams full weight tiles.  Operands arrive by TMA (cp.async.bulk.tensor, 128-byte
// swizzle, no multicast) into a ring of shared-memory stages; one thread issues
// tcgen05.mma (kind::f16, M = 128, N = token tile, K = 16 per instruction) with shared-
// memory descriptors; completion of a stage's MMAs frees the stage through tcgen05.commit;
// four epilogue warps read the accumulator with tcgen05.ld and store the transposed tile.
//
// Variants:
//   SWIGLU    W holds gate rows then up rows; the CTA keeps two accumulators (gate, up) for
//             the same 128 features and writes silu(gate) * up (engine/model.py:210-211,
//             251-252), so the [T, 2I] intermediate is never written.
//   HALF      the SwiGLU product of at most 128 tokens (one token tile): the 128 MMA rows are 64 gate rows and
//             the 64 up rows of the same features (two TMA boxes per stage), one accumulator; the epilogue
//             warps that hold the up rows hand them to the warps with the gate rows through shared memory,
//             16 tokens at a time.  Twice as many CTAs as the form above, two of them per SM, so the k range
//             needs no split and no kernel adds partial sums.
//   split-K   when a product has too few tiles to fill the GPU, the k range is split over
//             CTAs; partial sums go to float32 scratch and splitk_reduce_kernel adds them in
//             split order (and applies SwiGLU, or rounds to bfloat16), unless the caller leaves the
//             sums to the kernel that reads the result (`defer`: llm_add_rmsnorm, llm_rope_store).
//
// Every wait on an mbarrier is bounded; a wait that runs out records a code in a status
// word (llm_gemm_bf16_status), and the CTA falls through to its teardown (TMEM is freed).
#include "tcgen05_common.cuh"

#include <mutex>
#include <unordered_map>

namespace {

typedef __nv_bfloat16 bf16;

constexpr int kFeatTile = 128;                 // UMMA M
constexpr int kBlockK = 64;                    // elements per k-block: 128 bytes = one swizzle row
constexpr int kThreads = 192;                  // warp 0: TMA, warp 1: MMA + TMEM alloc, warps 2-5: epilogue
constexpr int kMaxStages = 12;

__device__ int g_status = 0;                   // 0 ok; else (code << 16) | block id of the first CTA that gave up
__device__ __forceinline__ void give_up(int code) { atomicCAS(&g_status, 0, (code << 16) | (int)(blockIdx.x & 0xffff)); }

enum OutMode { OUT_BF16 = 0, OUT_F32 = 1, OUT_PARTIAL = 2 };

struct GemmArgs {
    void* out;            // [tokens, ldc] bf16 or f32, or partials [splits, tokens, ldc] f32
    int out_mode;
    int n_feat;           // output features handled by the grid's feature tiles (I for SwiGLU, else N)
    int up_row_offset;    // SwiGLU: row of W where the up rows start (= I); partial column offset likewise
    int tokens;
    int ldc;
    int k_blocks;         // ceil(K / 64)
    int splits;
    int stages;
};

template <int N_TOK, bool SWIGLU, bool HALF = false>
__global__ void __launch_bounds__(kThreads, 2)
gemm_tn_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x, const GemmArgs a) {
    static_assert(!HALF || (SWIGLU && N_TOK <= 128), "the half-tile form is the SwiGLU product of one token tile of at most 128");
    constexpr int kABytes = kFeatTile * kBlockK * 2;               // 16 KiB per weight tile
    constexpr int kBBytes = N_TOK * kBlockK * 2;
    constexpr int kWTiles = (SWIGLU && !HALF) ? 2 : 1;             // weight tiles (and accumulators) per stage
    constexpr int kStageBytes = kWTiles * kABytes + kBBytes;
    constexpr int kTmemCols = kWTiles * N_TOK < 32 ? 32 : kWTiles * N_TOK;
    static_assert(kTmemCols <= 512 && (kTmemCols & (kTmemCols - 1)) == 0, "TMEM columns must be a power of two up to 512");

    extern __shared__ unsigned char smem_raw[];
    unsigned char* tiles = reinterpret_cast<unsigned char*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    __shared__ __align__(8) uint64_t full_bar[kMaxStages], empty_bar[kMaxStages], accum_bar;
    __shared__ uint32_t tmem_base_slot;
    __shared__ volatile int failed;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int feat0 = blockIdx.x * (HALF ? kFeatTile / 2 : kFeatTile), split = blockIdx.y, tok0 = blockIdx.z * N_TOK;
    const int kb0 = (int)((long long)split * a.k_blocks / a.splits), kb1 = (int)((long long)(split + 1) * a.k_blocks / a.splits);
    const int n_kb = kb1 - kb0;
    const int stages = a.stages;

    if (threadIdx.x == 0) {
        for (int s = 0; s < stages; ++s) { mbar_init(&full_bar[s], 1); mbar_init(&empty_bar[s], 1); }
        mbar_init(&accum_bar, 1);
        failed = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_slot)), "r"(kTmemCols));
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::);
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = tmem_base_slot;

    pdl_trigger();
    if (warp == 0 && lane == 0) {
        // ---- producer: TMA loads into the ring --------------------------------------------
        // The weights depend on no earlier kernel: the first ring of weight tiles is requested before
        // the wait for the previous kernel, the activation tiles (its output) after it.
        const int pre = n_kb < stages ? n_kb : stages;
        for (int i = 0; i < pre; ++i) {
            unsigned char* st = tiles + (size_t)i * kStageBytes;
            mbar_expect_tx(&full_bar[i], kStageBytes);
            const int k = (kb0 + i) * kBlockK;
            tma_load_2d(st, &map_w, &full_bar[i], k, feat0);
            if (SWIGLU) tma_load_2d(st + (HALF ? kABytes / 2 : kABytes), &map_w, &full_bar[i], k, a.up_row_offset + feat0);
        }
        pdl_wait();
        for (int i = 0; i < pre; ++i)
            tma_load_2d(tiles + (size_t)i * kStageBytes + kWTiles * kABytes, &map_x, &full_bar[i],
                        (kb0 + i) * kBlockK, tok0);
        for (int i = pre; i < n_kb; ++i) {
            const int s = i % stages;
            if (!mbar_wait(&empty_bar[s], ((i / stages) - 1) & 1)) { give_up(1); failed = 1; break; }
            unsigned char* st = tiles + (size_t)s * kStageBytes;
            mbar_expect_tx(&full_bar[s], kStageBytes);
            const int k = (kb0 + i) * kBlockK;
            tma_load_2d(st, &map_w, &full_bar[s], k, feat0);
            if (SWIGLU) tma_load_2d(st + (HALF ? kABytes / 2 : kABytes), &map_w, &full_bar[s], k, a.up_row_offset + feat0);
            tma_load_2d(st + kWTiles * kABytes, &map_x, &full_bar[s], k, tok0);
        }
    } else if (warp == 1 && lane == 0) {
        // ---- MMA issuer ---------------------------------------------------------------------
        constexpr uint32_t idesc = umma_idesc(kFeatTile, N_TOK);
        bool ok = true;
        for (int i = 0; i < n_kb && ok; ++i) {
            const int s = i % stages;
            if (!mbar_wait(&full_bar[s], (i / stages) & 1)) { give_up(2); failed = 1; ok = false; break; }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            unsigned char* st = tiles + (size_t)s * kStageBytes;
            const uint64_t da = umma_desc(st), db = umma_desc(st + kWTiles * kABytes);
            const uint64_t da2 = kWTiles == 2 ? umma_desc(st + kABytes) : 0;
#pragma unroll
            for (int k = 0; k < kBlockK / 16; ++k) {
                const uint32_t acc = (i > 0 || k > 0) ? 1u : 0u;
                umma_f16(tmem_base, da + 2 * k, db + 2 * k, idesc, acc);          // +32 bytes per K step of 16
                if (kWTiles == 2) umma_f16(tmem_base + N_TOK, da2 + 2 * k, db + 2 * k, idesc, acc);
            }
            umma_commit(&empty_bar[s]);           // the stage is free once these MMAs have read it
        }
        umma_commit(&accum_bar);                  // the accumulator is complete (also on the give-up path)
    } else if (warp >= 2) {
        // ---- epilogue: TMEM -> registers -> global, transposed ------------------------------
        const int quarter = warp & 3;             // a warp may only read TMEM lanes [32 * (warp % 4), +32)
        const int feat = feat0 + quarter * 32 + lane;
        pdl_wait();                               // nothing is stored before the previous kernel has finished
        if constexpr (HALF) {
            // lanes 0-63 of the accumulator are gate rows, lanes 64-127 the up rows of the same 64 features: per 16
            // tokens the upper two warps hand their values over through one of two buffers, the lower two finish
            __shared__ float up_rows[2][16 * (kFeatTile / 2)];
            const bool ok = n_kb > 0 && mbar_wait(&accum_bar, 0) && !failed;
            if (!ok && n_kb > 0 && !failed) give_up(3);
            const int f = (quarter & 1) * 32 + lane;              // feature of this lane inside the tile
            if (ok) asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll 1
            for (int c0 = 0; c0 < N_TOK; c0 += 16) {
                uint32_t g[16];
                float* hand = up_rows[(c0 >> 4) & 1];
                const bool live = ok && tok0 + c0 < a.tokens;
                if (live) {
                    tmem_ld16(tmem_base + ((uint32_t)(quarter * 32) << 16) + c0, g);
                    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                    if (quarter >= 2) {
#pragma unroll
                        for (int c = 0; c < 16; ++c) hand[c * (kFeatTile / 2) + f] = __uint_as_float(g[c]);
                    }
                }
                asm volatile("bar.sync 1, 128;" ::: "memory");       // the four epilogue warps, whatever happened above
                if (live && quarter < 2 && feat0 + f < a.n_feat) {
#pragma unroll
                    for (int c = 0; c < 16; ++c) {
                        const int tok = tok0 + c0 + c;
                        if (tok >= a.tokens) break;
                        const float gv = __uint_as_float(g[c]);
                        const float v = gv / (1.0f + expf(-gv)) * hand[c * (kFeatTile / 2) + f];
                        ((bf16*)a.out)[(size_t)tok * a.ldc + feat0 + f] = __float2bfloat16_rn(v);
                    }
                }
            }
        } else
        if (n_kb > 0 && mbar_wait(&accum_bar, 0) && !failed) {
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint32_t lane_addr = tmem_base + ((uint32_t)(quarter * 32) << 16);
#pragma unroll 1
            for (int c0 = 0; c0 < N_TOK; c0 += 16) {
                uint32_t g[16], u[16];
                tmem_ld16(lane_addr + c0, g);
                if (SWIGLU) tmem_ld16(lane_addr + N_TOK + c0, u);
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                if (feat < a.n_feat) {
#pragma unroll
                    for (int c = 0; c < 16; ++c) {
                        const int tok = tok0 + c0 + c;
                        if (tok >= a.tokens) break;
                        const float gv = __uint_as_float(g[c]);
                        if (a.out_mode == OUT_PARTIAL) {
                            float* dst = (float*)a.out + ((size_t)split * a.tokens + tok) * a.ldc;
                            dst[feat] = gv;
                            if (SWIGLU) dst[a.up_row_offset + feat] = __uint_as_float(u[c]);
                        } else {
                            float v = gv;
                            if (SWIGLU) v = gv / (1.0f + expf(-gv)) * __uint_as_float(u[c]);
                            if (a.out_mode == OUT_F32) ((float*)a.out)[(size_t)tok * a.ldc + feat] = v;
                            else ((bf16*)a.out)[(size_t)tok * a.ldc + feat] = __float2bfloat16_rn(v);
                        }
                    }
                }
            }
        } else if (n_kb > 0 && !failed) {
            give_up(3);
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols));
    }
}

// out[t, f] = sum over splits of part[s, t, f]  (SwiGLU: silu(sum gate) * sum up), four features per thread.
template <bool SWIGLU, typename TO>
__global__ void splitk_reduce_kernel(const float* __restrict__ part, TO* __restrict__ out, int splits, int tokens,
                                     int n_feat, int ld_part, int up_offset, int ldc) {
    pdl_trigger();
    pdl_wait();
    const int f4 = n_feat / 4;
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < (size_t)tokens * f4;
         idx += (size_t)gridDim.x * blockDim.x) {
        const int t = (int)(idx / f4), f = (int)(idx % f4) * 4;
        float4 g = make_float4(0.f, 0.f, 0.f, 0.f), u = g;
        for (int s = 0; s < splits; ++s) {
            const float* row = part + ((size_t)s * tokens + t) * ld_part;
            const float4 a = *reinterpret_cast<const float4*>(row + f);
            g.x += a.x; g.y += a.y; g.z += a.z; g.w += a.w;
            if (SWIGLU) {
                const float4 b = *reinterpret_cast<const float4*>(row + up_offset + f);
                u.x += b.x; u.y += b.y; u.z += b.z; u.w += b.w;
            }
        }
        if (SWIGLU) {
            g.x = g.x / (1.0f + expf(-g.x)) * u.x; g.y = g.y / (1.0f + expf(-g.y)) * u.y;
            g.z = g.z / (1.0f + expf(-g.z)) * u.z; g.w = g.w / (1.0f + expf(-g.w)) * u.w;
        }
        TO* dst = out + (size_t)t * ldc + f;
        dst[0] = from_f32<TO>(g.x); dst[1] = from_f32<TO>(g.y); dst[2] = from_f32<TO>(g.z); dst[3] = from_f32<TO>(g.w);
    }
}

// ---- host: tensor maps ------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
    });
    return fn;
}

struct MapKey {
    const void* ptr; uint64_t rows, cols; uint32_t box_rows, box_cols;
    bool operator==(const MapKey& o) const {
        return ptr == o.ptr && rows == o.rows && cols == o.cols && box_rows == o.box_rows && box_cols == o.box_cols;
    }
};
struct MapKeyHash {
    size_t operator()(const MapKey& k) const {
        return std::hash<const void*>()(k.ptr) ^ ((size_t)k.rows * 1000003u) ^ ((size_t)k.cols * 7919u) ^
               ((size_t)k.box_rows << 20) ^ ((size_t)k.box_cols << 40);
    }
};
std::unordered_map<MapKey, CUtensorMap, MapKeyHash> g_maps;
std::mutex g_maps_mutex;

}  // namespace

int llm_tensor_map_2d(const void* ptr, uint64_t rows, uint64_t cols, uint32_t box_rows, uint32_t box_cols, CUtensorMap* out) {
    std::lock_guard<std::mutex> lock(g_maps_mutex);
    const MapKey key{ptr, rows, cols, box_rows, box_cols};
    auto it = g_maps.find(key);
    if (it != g_maps.end()) { *out = it->second; return 0; }
    EncodeTiledFn fn = encode_fn();
    if (!fn) LLM_FAIL(-2, "tensor map: cuTensorMapEncodeTiled is not available from this driver");
    if (((uintptr_t)ptr & 15) || (cols % 8)) LLM_FAIL(-1, "tensor map: matrices must be 16-byte aligned with a row length that is a multiple of 8 (got %llu)", (unsigned long long)cols);
    if (box_cols * 2 > 128 || box_rows > 256) LLM_FAIL(-1, "tensor map: box %u x %u does not fit the 128-byte swizzle", box_cols, box_rows);
    cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)cols * 2};
    cuuint32_t box[2] = {(cuuint32_t)box_cols, (cuuint32_t)box_rows};
    cuuint32_t elem[2] = {1, 1};
    CUtensorMap m;
    CUresult r = fn(&m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, elem,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) LLM_FAIL(-2, "tensor map: cuTensorMapEncodeTiled failed with code %d", (int)r);
    if (g_maps.size() > 4096) g_maps.clear();
    g_maps.emplace(key, m);
    *out = m;
    return 0;
}

namespace {

template <int N_TOK, bool SWIGLU, bool HALF = false>
int launch_tile(const CUtensorMap& mw, const CUtensorMap& mx, GemmArgs a, dim3 grid, cudaStream_t stream) {
    constexpr int stage_bytes = ((SWIGLU && !HALF) ? 2 : 1) * kFeatTile * kBlockK * 2 + N_TOK * kBlockK * 2;
    // shared memory for the ring: 200 KiB (one CTA per SM), or about half of it when the caller wants two
    // CTAs per SM (more CTAs in flight for products with few tiles)
    int stages = ((a.stages > 0 ? a.stages : 200) * 1024) / stage_bytes;
    if (stages > kMaxStages) stages = kMaxStages;
    if (stages < 2) stages = 2;
    a.stages = stages;
    const size_t smem = (size_t)stages * stage_bytes + 1024;
    auto kern = gemm_tn_kernel<N_TOK, SWIGLU, HALF>;
    static size_t configured = 0;              // largest size set so far, one per instantiation
    if (smem > configured) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) LLM_FAIL(-2, "gemm_bf16: cudaFuncSetAttribute: %s", cudaGetErrorString(e));
        configured = smem;
    }
    llm_launch(kern, grid, kThreads, smem, stream, mw, mx, a);
    LLM_CHECK_LAUNCH("gemm_bf16");
    return 0;
}

}  // namespace

// Token tile the kernel uses for `tokens` rows of x.
LLM_API int llm_gemm_bf16_token_tile(int tokens) {
    return tokens <= 16 ? 16 : tokens <= 32 ? 32 : tokens <= 64 ? 64 : tokens <= 128 ? 128 : 256;
}

// out = x . w^T.   x [tokens, K] bf16, w [n (or 2n with swiglu), K] bf16.
// out_f32 == 0: out is bf16 [tokens, ldc]; out_f32 != 0: float32 [tokens, ldc].
// splits > 1 needs `scratch` with splits * tokens * (swiglu ? 2n : n) floats; the reduction runs right after,
// unless `defer` is set: then the partial sums [splits][tokens][n] stay in scratch for the kernel that reads
// the result (llm_add_rmsnorm, llm_rope_store) and `out` is not written.
// smem_kb: shared memory of one CTA's ring in KiB (0 = 200: one CTA per SM; about 100 lets two CTAs share an SM).
// half: the SwiGLU product of at most 128 tokens with 64 gate and 64 up rows per CTA (n % 64 == 0, no split).
LLM_API int llm_gemm_bf16(const void* x, const void* w, void* out, int out_f32, int tokens, int n, int K, int ldc,
                          int swiglu, int splits, float* scratch, int smem_kb, int defer, int half, cudaStream_t stream) {
    if (tokens == 0 || n == 0) return 0;
    if (K % 8) LLM_FAIL(-1, "gemm_bf16: K %d must be a multiple of 8", K);
    if (swiglu && out_f32) LLM_FAIL(-1, "gemm_bf16: the SwiGLU variant writes bfloat16");
    const int k_blocks = (K + kBlockK - 1) / kBlockK;
    if (splits < 1) splits = 1;
    if (splits > k_blocks) splits = k_blocks;
    if (splits > 1 && !scratch) LLM_FAIL(-1, "gemm_bf16: split-K needs scratch");
    if (splits > 1 && (n % 4)) LLM_FAIL(-1, "gemm_bf16: split-K needs n %% 4 == 0");
    const int w_rows = swiglu ? 2 * n : n;
    const int tile = llm_gemm_bf16_token_tile(tokens);
    if (half && (!swiglu || tile > 128 || n % (kFeatTile / 2) || splits != 1))
        LLM_FAIL(-1, "gemm_bf16: the half-tile form is the unsplit SwiGLU product of at most 128 tokens with n %% 64 == 0");
    CUtensorMap mw, mx;
    if (int rc = llm_tensor_map_2d(w, w_rows, K, half ? kFeatTile / 2 : kFeatTile, kBlockK, &mw)) return rc;
    if (int rc = llm_tensor_map_2d(x, tokens, K, tile, kBlockK, &mx)) return rc;
    GemmArgs a;
    a.out = splits > 1 ? (void*)scratch : out;
    a.out_mode = splits > 1 ? OUT_PARTIAL : (out_f32 ? OUT_F32 : OUT_BF16);
    a.n_feat = n;
    a.up_row_offset = swiglu ? n : 0;
    a.tokens = tokens;
    a.ldc = splits > 1 ? w_rows : ldc;
    a.k_blocks = k_blocks;
    a.splits = splits;
    a.stages = smem_kb;          // launch_tile turns the budget into a stage count
    dim3 grid(half ? n / (kFeatTile / 2) : (n + kFeatTile - 1) / kFeatTile, splits, (tokens + tile - 1) / tile);
    if (grid.y > 65535 || grid.z > 65535) LLM_FAIL(-1, "gemm_bf16: grid out of range");
    int rc;
    if (half) {
        switch (tile) {
            case 16: return launch_tile<16, true, true>(mw, mx, a, grid, stream);
            case 32: return launch_tile<32, true, true>(mw, mx, a, grid, stream);
            case 64: return launch_tile<64, true, true>(mw, mx, a, grid, stream);
            default: return launch_tile<128, true, true>(mw, mx, a, grid, stream);
        }
    }
#define LLM_GEMM_CASE(T)                                                                       \
    case T: rc = swiglu ? launch_tile<T, true>(mw, mx, a, grid, stream) : launch_tile<T, false>(mw, mx, a, grid, stream); break;
    switch (tile) {
        LLM_GEMM_CASE(16)
        LLM_GEMM_CASE(32)
        LLM_GEMM_CASE(64)
        LLM_GEMM_CASE(128)
        LLM_GEMM_CASE(256)
        default: LLM_FAIL(-1, "gemm_bf16: no kernel for a token tile of %d", tile);
    }
#undef LLM_GEMM_CASE
    if (rc) return rc;
    if (defer && swiglu) LLM_FAIL(-1, "gemm_bf16: the SwiGLU sums cannot be deferred");
    if (splits > 1 && !defer) {
        const size_t work = (size_t)tokens * (n / 4);
        const int blocks = (int)((work + 255) / 256 < 148 * 8 ? (work + 255) / 256 : 148 * 8);
        if (swiglu)
            llm_launch(splitk_reduce_kernel<true, bf16>, blocks, 256, 0, stream, scratch, (bf16*)out, splits, tokens, n, w_rows, n, ldc);
        else if (out_f32)
            llm_launch(splitk_reduce_kernel<false, float>, blocks, 256, 0, stream, scratch, (float*)out, splits, tokens, n, w_rows, 0, ldc);
        else
            llm_launch(splitk_reduce_kernel<false, bf16>, blocks, 256, 0, stream, scratch, (bf16*)out, splits, tokens, n, w_rows, 0, ldc);
        LLM_CHECK_LAUNCH("gemm_bf16_reduce");
    }
    return 0;
}

// ---- a wait that runs out, on purpose (tests) ---------------------------------------------------------------
// One thread sets up an mbarrier that nobody will ever arrive on and waits for it with the kernels' own bounded
// wait, cut to `polls` polls; when the wait gives up it records code 7 in the status word, exactly as a product's
// CTA records its code, and the kernel returns.  No copy and no MMA is in flight and no tensor memory is held, so
// there is nothing to clean up: the kernel shows what the host sees of a wait that ran out.
namespace {
__global__ void wait_probe_kernel(uint32_t polls) {
    __shared__ __align__(8) uint64_t bar;
    if (threadIdx.x == 0) {
        mbar_init(&bar, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        if (!mbar_wait(&bar, 0, polls)) give_up(7);
    }
}
}  // namespace

LLM_API int llm_gemm_bf16_wait_probe(int polls, cudaStream_t stream) {
    if (polls < 1 || polls > (1 << 16)) LLM_FAIL(-1, "gemm_bf16_wait_probe: 1 to 65536 polls");
    wait_probe_kernel<<<1, 32, 0, stream>>>((uint32_t)polls);
    LLM_CHECK_LAUNCH("gemm_bf16_wait_probe");
    return 0;
}

const int* llm_gemm_bf16_status_word() {
    void* p = nullptr;
    return cudaGetSymbolAddress(&p, g_status) == cudaSuccess ? static_cast<const int*>(p) : nullptr;
}

// Reads and clears the status word: 0, or (code << 16 | block) of the first CTA whose wait ran out
// (code 1: producer waiting for a free stage, 2: MMA issuer waiting for data, 3: epilogue waiting for the accumulator).
LLM_API int llm_gemm_bf16_status() {
    int v = 0, zero = 0;
    if (cudaMemcpyFromSymbol(&v, g_status, sizeof(int)) != cudaSuccess) return -1;
    if (v) cudaMemcpyToSymbol(g_status, &zero, sizeof(int));
    return v;
}

LLM_TRACE_EXPORT(gemm_bf16)
