// Row-wise kernels: embedding gather, (residual add +) RMSNorm, rotary position encoding
// fused with the key/value cache write, SiLU-and-multiply.
//
// The residual stream is float32 in both precisions: `residual += delta` and the norm's
// statistics are computed in float32, only the norm's output is rounded to the model type.
#include "common.cuh"

// ---------------------------------------------------------------------------------------
// embedding: out[t, :] = scale * table[ids[t], :]   (float32 residual stream)
// replaces F.embedding of the reference (engine/model.py:191)
// ---------------------------------------------------------------------------------------
template <typename TW>
__global__ void embed_kernel(const int* __restrict__ ids, const TW* __restrict__ table,
                             float* __restrict__ out, int width, int vocab, float scale) {
    const int t = blockIdx.x;
    const int id = ids[t];
    const bool ok = id >= 0 && id < vocab;  // the host refuses such ids; never read out of range
    const TW* src = table + (size_t)(ok ? id : 0) * width;
    float* dst = out + (size_t)t * width;
    for (int i = threadIdx.x; i < width; i += blockDim.x) dst[i] = ok ? scale * to_f32(src[i]) : 0.f;
}

LLM_API int llm_embed(const int* ids, const void* table, int table_dtype, float* out, int tokens,
                      int width, int vocab, float scale, cudaStream_t stream) {
    if (tokens == 0) return 0;
    return llm_dispatch_dtype(table_dtype, [&](auto tag) {
        using TW = decltype(tag);
        embed_kernel<TW><<<tokens, 256, 0, stream>>>(ids, (const TW*)table, out, width, vocab, scale);
        LLM_CHECK_LAUNCH("embed");
        return 0;
    });
}

// ---------------------------------------------------------------------------------------
// add + RMSNorm.  For output row r (source row s = rows ? rows[r] : r):
//     v = residual[s] + delta[s]          (delta optional)
//     residual[s] = v                     (only when rows == nullptr and delta != nullptr)
//     out[r] = v * rsqrt(mean(v^2) + eps) * weight
// Formula: engine/model.py:85-89; the add-then-norm form: engine/model.py:236.
// ---------------------------------------------------------------------------------------
template <typename TD, typename TW>
__global__ void add_rmsnorm_kernel(float* __restrict__ residual, const TD* __restrict__ delta,
                                   const int* __restrict__ rows, const TW* __restrict__ weight,
                                   TD* __restrict__ out, int width, float eps) {
    extern __shared__ float row_buf[];  // width floats
    __shared__ float red[32];
    const int r = blockIdx.x;
    const size_t s = rows ? (size_t)rows[r] : (size_t)r;
    float* res = residual + s * width;
    const TD* dl = delta ? delta + s * width : nullptr;
    float ss = 0.f;
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        float v = res[i];
        if (dl) {
            v += to_f32(dl[i]);
            if (!rows) res[i] = v;
        }
        row_buf[i] = v;
        ss += v * v;
    }
    const float total = block_sum(ss, red);
    const float inv = 1.0f / sqrtf(total / (float)width + eps);
    TD* o = out + (size_t)r * width;
    for (int i = threadIdx.x; i < width; i += blockDim.x)
        o[i] = from_f32<TD>(row_buf[i] * inv * to_f32(weight[i]));
}

LLM_API int llm_add_rmsnorm(float* residual, const void* delta, const int* rows, const void* weight,
                            int weight_dtype, void* out, int dtype, int out_rows, int width, float eps,
                            cudaStream_t stream) {
    if (out_rows == 0) return 0;
    const size_t smem = (size_t)width * sizeof(float);
    if (smem > 200 * 1024) LLM_FAIL(-1, "add_rmsnorm: width %d is larger than 51200", width);
    return llm_dispatch_dtype(dtype, [&](auto tag) {
        using TD = decltype(tag);
        return llm_dispatch_dtype(weight_dtype, [&](auto wtag) {
            using TW = decltype(wtag);
            auto kern = add_rmsnorm_kernel<TD, TW>;
            if (smem > 48 * 1024) {
                cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
                if (e != cudaSuccess) LLM_FAIL(-2, "add_rmsnorm: %s", cudaGetErrorString(e));
            }
            kern<<<out_rows, 256, smem, stream>>>(residual, (const TD*)delta, rows, (const TW*)weight,
                                                  (TD*)out, width, eps);
            LLM_CHECK_LAUNCH("add_rmsnorm");
            return 0;
        });
    });
}

// ---------------------------------------------------------------------------------------
// Rotary position encoding (half-split "neox" pairing: engine/model.py:92-94, 199-200) applied
// in place to the query heads, and to the key heads on their way into the paged cache,
// together with the value copy (engine/model.py:201-203).  Angles are position * inv_freq in
// float32 and sin/cos are evaluated in float32 for both precisions.
//
// qkv:  [tokens, (heads + 2*kv_heads) * head_dim], query heads first, then keys, then values.
// cache layer: [pages, 2, kv_heads, page_size, head_dim]; slot = page * page_size + offset;
//              slot < 0 means "do not store" for that token.
// rotary_dim <= head_dim: dims [0, rotary_dim) are rotated in pairs (i, i + rotary_dim/2),
//              the rest pass through.  rotary_dim == 0 stores without rotating.
// ---------------------------------------------------------------------------------------
template <typename T>
__global__ void rope_store_kernel(T* __restrict__ qkv, const int* __restrict__ positions,
                                  const float* __restrict__ inv_freq, const int* __restrict__ slots,
                                  T* __restrict__ cache, int heads, int kv_heads, int head_dim,
                                  int rotary_dim, int page_size) {
    const int t = blockIdx.x;
    const int half = rotary_dim / 2;
    const int row_width = (heads + 2 * kv_heads) * head_dim;
    T* row = qkv + (size_t)t * row_width;
    const float pos = (float)positions[t];
    const int slot = slots ? slots[t] : -1;
    const size_t plane = (size_t)kv_heads * page_size * head_dim;  // one of K or V of one page
    size_t kbase = 0;
    if (slot >= 0) {
        const int page = slot / page_size, off = slot % page_size;
        kbase = (size_t)page * 2 * plane + (size_t)off * head_dim;
    }
    const size_t head_stride = (size_t)page_size * head_dim;

    // rotated pairs of query and key heads
    const int rot_heads = heads + kv_heads;
    for (int w = threadIdx.x; w < rot_heads * half; w += blockDim.x) {
        const int h = w / half, i = w % half;
        const float angle = pos * inv_freq[i];
        float s, c;
        sincosf(angle, &s, &c);
        T* x = row + (size_t)h * head_dim;
        const float x1 = to_f32(x[i]), x2 = to_f32(x[i + half]);
        const T o1 = from_f32<T>(x1 * c - x2 * s);
        const T o2 = from_f32<T>(x2 * c + x1 * s);
        if (h < heads) {
            x[i] = o1;
            x[i + half] = o2;
        } else if (slot >= 0) {
            T* dst = cache + kbase + (size_t)(h - heads) * head_stride;
            dst[i] = o1;
            dst[i + half] = o2;
        }
    }
    if (slot < 0) return;
    // key dims that are not rotated
    const int pass = head_dim - rotary_dim;
    for (int w = threadIdx.x; w < kv_heads * pass; w += blockDim.x) {
        const int h = w / pass, i = rotary_dim + w % pass;
        cache[kbase + (size_t)h * head_stride + i] = row[(size_t)(heads + h) * head_dim + i];
    }
    // values
    const T* v = row + (size_t)(heads + kv_heads) * head_dim;
    for (int w = threadIdx.x; w < kv_heads * head_dim; w += blockDim.x) {
        const int h = w / head_dim, i = w % head_dim;
        cache[kbase + plane + (size_t)h * head_stride + i] = v[(size_t)h * head_dim + i];
    }
}

LLM_API int llm_rope_store(void* qkv, const int* positions, const float* inv_freq, const int* slots,
                           void* cache, int dtype, int tokens, int heads, int kv_heads, int head_dim,
                           int rotary_dim, int page_size, cudaStream_t stream) {
    if (tokens == 0) return 0;
    if (rotary_dim < 0 || rotary_dim > head_dim || (rotary_dim & 1))
        LLM_FAIL(-1, "rope_store: rotary_dim %d must be even and at most head_dim %d", rotary_dim, head_dim);
    return llm_dispatch_dtype(dtype, [&](auto tag) {
        using T = decltype(tag);
        rope_store_kernel<T><<<tokens, 256, 0, stream>>>((T*)qkv, positions, inv_freq, slots, (T*)cache,
                                                         heads, kv_heads, head_dim, rotary_dim, page_size);
        LLM_CHECK_LAUNCH("rope_store");
        return 0;
    });
}

// ---------------------------------------------------------------------------------------
// act[t, i] = silu(gu[t, i]) * gu[t, inner + i]   (engine/model.py:210-211, 251-252), float32 math
// ---------------------------------------------------------------------------------------
template <typename T>
__global__ void silu_mul_kernel(const T* __restrict__ gu, T* __restrict__ act, int inner, size_t total) {
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
         idx += (size_t)gridDim.x * blockDim.x) {
        const size_t t = idx / inner, i = idx % inner;
        const float g = to_f32(gu[t * 2 * inner + i]);
        const float u = to_f32(gu[t * 2 * inner + inner + i]);
        act[idx] = from_f32<T>(g / (1.0f + expf(-g)) * u);
    }
}

LLM_API int llm_silu_mul(const void* gu, void* act, int dtype, int tokens, int inner, cudaStream_t stream) {
    const size_t total = (size_t)tokens * inner;
    if (total == 0) return 0;
    const int blocks = (int)((total + 255) / 256 < 148 * 16 ? (total + 255) / 256 : 148 * 16);
    return llm_dispatch_dtype(dtype, [&](auto tag) {
        using T = decltype(tag);
        silu_mul_kernel<T><<<blocks, 256, 0, stream>>>((const T*)gu, (T*)act, inner, total);
        LLM_CHECK_LAUNCH("silu_mul");
        return 0;
    });
}
