// Paged causal attention, general form: any head size that is a multiple of 16 up to 256,
// any number of heads and groups, any page size, optional sliding window, float32 or
// bfloat16 storage, float32 arithmetic throughout.  It is the whole of the float32 path
// (prompt portions and decoded tokens alike) and the bfloat16 path's fallback for head
// sizes that the tensor-core kernels do not take.
//
// Replaces flash_attn_varlen_func with block_table (engine/model.py:204-207): a query at
// position p of request b sees the keys at positions [lo, p] of that request, lo = 0 or
// p - window + 1; softmax(scale * q.k) in float32; out = P.V; query head g reads key/value
// head g / (heads / kv_heads).
//
// One warp per (token, head).  Keys are walked in tiles of 32 that start at multiples of
// 32 of the key position, so the order of every sum depends only on the query's own
// position: the result does not change with how the tokens were cut into steps or what
// else is in the batch.
#include "common.cuh"

namespace {

constexpr int kWarps = 4;
constexpr int kMaxHeadDim = 256;

template <typename T>
__device__ __forceinline__ float dot_row(const T* __restrict__ k, const float* __restrict__ q, int d);

template <>
__device__ __forceinline__ float dot_row<float>(const float* __restrict__ k, const float* __restrict__ q, int d) {
    float acc = 0.f;
    for (int i = 0; i < d; i += 4) {
        const float4 kv = *reinterpret_cast<const float4*>(k + i);
        acc = fmaf(kv.x, q[i], acc);
        acc = fmaf(kv.y, q[i + 1], acc);
        acc = fmaf(kv.z, q[i + 2], acc);
        acc = fmaf(kv.w, q[i + 3], acc);
    }
    return acc;
}

template <>
__device__ __forceinline__ float dot_row<__nv_bfloat16>(const __nv_bfloat16* __restrict__ k,
                                                         const float* __restrict__ q, int d) {
    float acc = 0.f;
    for (int i = 0; i < d; i += 8) {
        const uint4 raw = *reinterpret_cast<const uint4*>(k + i);
        const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float2 f = __bfloat1622float2(p[j]);
            acc = fmaf(f.x, q[i + 2 * j], acc);
            acc = fmaf(f.y, q[i + 2 * j + 1], acc);
        }
    }
    return acc;
}

template <typename T>
__global__ void __launch_bounds__(kWarps * 32)
attn_generic_kernel(const T* __restrict__ q, int q_stride, const T* __restrict__ cache,
                    const int* __restrict__ block_table, int table_width,
                    const int* __restrict__ token_request, const int* __restrict__ positions,
                    T* __restrict__ out, int out_stride, int tokens, int heads, int kv_heads,
                    int head_dim, int page_size, int window, float scale) {
    pdl_trigger();
    pdl_wait();
    __shared__ __align__(16) float q_smem[kWarps][kMaxHeadDim];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const long long item = (long long)blockIdx.x * kWarps + warp;
    if (item >= (long long)tokens * heads) return;  // whole warp leaves together
    const int t = (int)(item / heads), h = (int)(item % heads);
    const int hk = h / (heads / kv_heads);
    const int pos = positions[t];
    const int lo = window > 0 ? max(0, pos - window + 1) : 0;
    const int* table = block_table + (size_t)token_request[t] * table_width;

    float* qs = q_smem[warp];
    const T* qrow = q + (size_t)t * q_stride + (size_t)h * head_dim;
    for (int i = lane; i < head_dim; i += 32) qs[i] = to_f32(qrow[i]);
    __syncwarp();

    const size_t plane = (size_t)kv_heads * page_size * head_dim;
    const size_t head_off = (size_t)hk * page_size * head_dim;
    constexpr int kOwn = kMaxHeadDim / 32;  // output dims per lane: lane, lane + 32, ...
    float acc[kOwn];
#pragma unroll
    for (int i = 0; i < kOwn; ++i) acc[i] = 0.f;
    float m = -INFINITY, l = 0.f;

    for (int k0 = lo & ~31; k0 <= pos; k0 += 32) {
        const int j = k0 + lane;
        const bool valid = j >= lo && j <= pos;
        long long koff = 0;
        float s = -INFINITY;
        if (valid) {
            const int page = table[j / page_size];
            koff = (long long)((size_t)page * 2 * plane + head_off + (size_t)(j % page_size) * head_dim);
            s = scale * dot_row<T>(cache + koff, qs, head_dim);
        }
        const float m_new = fmaxf(m, warp_max(s));   // finite: every tile holds a visible key
        const float corr = expf(m - m_new);          // 0 on the first tile (m = -inf)
        const float p = valid ? expf(s - m_new) : 0.f;
        l = l * corr + warp_sum(p);
#pragma unroll
        for (int i = 0; i < kOwn; ++i) acc[i] *= corr;
        for (int jj = 0; jj < 32; ++jj) {
            const float pj = __shfl_sync(0xffffffffu, p, jj);
            const long long vo = __shfl_sync(0xffffffffu, koff, jj);
            if (pj == 0.f) continue;  // same for the whole warp
            const T* vrow = cache + vo + plane;
#pragma unroll
            for (int i = 0; i < kOwn; ++i) {
                const int d = lane + 32 * i;
                if (d < head_dim) acc[i] = fmaf(pj, to_f32(vrow[d]), acc[i]);
            }
        }
        m = m_new;
    }
    T* orow = out + (size_t)t * out_stride + (size_t)h * head_dim;
    const float inv = 1.0f / l;
#pragma unroll
    for (int i = 0; i < kOwn; ++i) {
        const int d = lane + 32 * i;
        if (d < head_dim) orow[d] = from_f32<T>(acc[i] * inv);
    }
}

}  // namespace

LLM_API int llm_attention_generic(const void* q, int q_stride, const void* cache, const int* block_table,
                                  int table_width, const int* token_request, const int* positions,
                                  void* out, int out_stride, int dtype, int tokens, int heads,
                                  int kv_heads, int head_dim, int page_size, int window, float scale,
                                  cudaStream_t stream) {
    if (tokens == 0) return 0;
    if (head_dim % 16 || head_dim <= 0 || head_dim > kMaxHeadDim)
        LLM_FAIL(-1, "attention: head_dim %d is not a multiple of 16 in [16, %d]", head_dim, kMaxHeadDim);
    if (kv_heads <= 0 || heads % kv_heads)
        LLM_FAIL(-1, "attention: heads %d is not a multiple of kv_heads %d", heads, kv_heads);
    const long long items = (long long)tokens * heads;
    const long long blocks = (items + kWarps - 1) / kWarps;
    if (blocks > 0x7fffffffLL) LLM_FAIL(-1, "attention: too many (token, head) pairs: %lld", items);
    return llm_dispatch_dtype(dtype, [&](auto tag) {
        using T = decltype(tag);
        llm_launch(attn_generic_kernel<T>, (unsigned)blocks, kWarps * 32, 0, stream, 
            (const T*)q, q_stride, (const T*)cache, block_table, table_width, token_request, positions,
            (T*)out, out_stride, tokens, heads, kv_heads, head_dim, page_size, window, scale);
        LLM_CHECK_LAUNCH("attention_generic");
        return 0;
    });
}

LLM_TRACE_EXPORT(attention_generic)
