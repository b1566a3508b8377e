// Row-wise kernels: embedding gather, (residual add +) RMSNorm, rotary position encoding
// fused with the key/value cache write, SiLU-and-multiply.
//
// The residual stream is float32 in both precisions: `residual += delta` and the norm's
// statistics are computed in float32, only the norm's output is rounded to the model type.
#include "common.cuh"

#include <stdlib.h>

// ---------------------------------------------------------------------------------------
// embedding: out[t, :] = scale * table[ids[t], :]   (float32 residual stream)
// replaces F.embedding of the reference (engine/model.py:191)
// ---------------------------------------------------------------------------------------
template <typename TW>
__global__ void embed_kernel(const int* __restrict__ ids, const TW* __restrict__ table,
                             float* __restrict__ out, int width, int vocab, float scale) {
    pdl_trigger();
    pdl_wait();
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
        llm_launch(embed_kernel<TW>, tokens, 256, 0, stream, ids, (const TW*)table, out, width, vocab, scale);
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
// With `splits` > 0 delta is the float32 partial sums [splits][rows][width] of a matrix product split along
// k (`split_stride` elements apart); they are added here in split order, which saves the product its own
// reduction kernel.
// ---------------------------------------------------------------------------------------
template <typename TD, typename TW>
__global__ void add_rmsnorm_kernel(float* __restrict__ residual, const TD* __restrict__ delta,
                                   const int* __restrict__ rows, const TW* __restrict__ weight,
                                   TD* __restrict__ out, int width, float eps, int splits, size_t split_stride) {
    pdl_trigger();
    pdl_wait();
    extern __shared__ float row_buf[];  // width floats
    __shared__ float red[32];
    const int r = blockIdx.x;
    const size_t s = rows ? (size_t)rows[r] : (size_t)r;
    float* res = residual + s * width;
    const TD* dl = delta ? delta + s * width : nullptr;
    const float* parts = splits > 0 ? reinterpret_cast<const float*>(delta) + s * width : nullptr;
    float ss = 0.f;
    for (int i = threadIdx.x; i < width; i += blockDim.x) {
        float v = res[i];
        if (dl) {
            if (parts) {
                float d = 0.f;
                for (int k = 0; k < splits; ++k) d += parts[(size_t)k * split_stride + i];
                v += d;
            } else {
                v += to_f32(dl[i]);
            }
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

// Four elements per thread and step (width % 4 == 0): all of a thread's loads are in flight at once.
template <typename T> struct Vec4;
template <> struct Vec4<float> {
    static __device__ __forceinline__ float4 load(const float* p) { return *reinterpret_cast<const float4*>(p); }
    static __device__ __forceinline__ void store(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
};
template <> struct Vec4<__nv_bfloat16> {
    static __device__ __forceinline__ float4 load(const __nv_bfloat16* p) {
        const uint2 raw = *reinterpret_cast<const uint2*>(p);
        const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
        const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
        return make_float4(a.x, a.y, b.x, b.y);
    }
    static __device__ __forceinline__ void store(__nv_bfloat16* p, float4 v) {
        __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
        uint2 raw;
        raw.x = *reinterpret_cast<uint32_t*>(&a);
        raw.y = *reinterpret_cast<uint32_t*>(&b);
        *reinterpret_cast<uint2*>(p) = raw;
    }
};

template <typename TD, typename TW, int PER_THREAD>
__global__ void __launch_bounds__(256) add_rmsnorm_vec_kernel(float* __restrict__ residual, const TD* __restrict__ delta,
                                       const int* __restrict__ rows, const TW* __restrict__ weight,
                                       TD* __restrict__ out, int width, float eps, int splits, size_t split_stride) {
    pdl_trigger();
    pdl_wait();
    __shared__ float red[32];
    const int r = blockIdx.x;
    const size_t s = rows ? (size_t)rows[r] : (size_t)r;
    float* res = residual + s * width;
    const TD* dl = delta ? delta + s * width : nullptr;
    const float* parts = splits > 0 ? reinterpret_cast<const float*>(delta) + s * width : nullptr;
    float4 v[PER_THREAD];
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < PER_THREAD; ++j) {
        const int i = (threadIdx.x + j * blockDim.x) * 4;
        v[j] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (i < width) {
            v[j] = Vec4<float>::load(res + i);
            if (parts) {
                const float4 d = sum_parts4(parts + i, splits, split_stride);
                v[j].x += d.x; v[j].y += d.y; v[j].z += d.z; v[j].w += d.w;
            } else if (dl) {
                const float4 d = Vec4<TD>::load(dl + i);
                v[j].x += d.x; v[j].y += d.y; v[j].z += d.z; v[j].w += d.w;
            }
        }
    }
#pragma unroll
    for (int j = 0; j < PER_THREAD; ++j) {
        const int i = (threadIdx.x + j * blockDim.x) * 4;
        if (i < width) {
            if (dl && !rows) Vec4<float>::store(res + i, v[j]);
            ss += v[j].x * v[j].x + v[j].y * v[j].y + v[j].z * v[j].z + v[j].w * v[j].w;
        }
    }
    const float total = block_sum(ss, red);
    const float inv = 1.0f / sqrtf(total / (float)width + eps);
    TD* o = out + (size_t)r * width;
#pragma unroll
    for (int j = 0; j < PER_THREAD; ++j) {
        const int i = (threadIdx.x + j * blockDim.x) * 4;
        if (i < width) {
            const float4 w = Vec4<TW>::load(weight + i);
            Vec4<TD>::store(o + i, make_float4(v[j].x * inv * w.x, v[j].y * inv * w.y, v[j].z * inv * w.z, v[j].w * inv * w.w));
        }
    }
}

// Few rows (decode): a row is shared by a cluster of blocks, each with width / cluster columns, so that the
// reads (above all of partial sums) are spread over more SMs; each block pushes its sum of squares into the
// shared memory of all blocks of the cluster, and after one cluster barrier every block adds them in block order.
template <typename TD, typename TW, int PER_THREAD>
__global__ void __launch_bounds__(256)
add_rmsnorm_cluster_kernel(float* __restrict__ residual, const TD* __restrict__ delta, const int* __restrict__ rows,
                           const TW* __restrict__ weight, TD* __restrict__ out, int width, float eps, int splits,
                           size_t split_stride, int cluster) {
    pdl_trigger();
    pdl_wait();
    __shared__ float red[32];
    __shared__ float all_ss[8];               // the sums of squares of the cluster's blocks, pushed here by each of them
    const int c = (int)llm_cluster_rank();
    const int r = blockIdx.x / cluster;
    const size_t s = rows ? (size_t)rows[r] : (size_t)r;
    float* res = residual + s * width;
    const TD* dl = delta ? delta + s * width : nullptr;
    const float* parts = splits > 0 ? reinterpret_cast<const float*>(delta) + s * width : nullptr;
    const int cols = width / cluster, col0 = c * cols;       // this block's columns (a multiple of 4)
    float4 v[PER_THREAD], w[PER_THREAD];
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < PER_THREAD; ++j) {
        const int i = (threadIdx.x + j * blockDim.x) * 4;
        v[j] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (i < cols) {
            v[j] = Vec4<float>::load(res + col0 + i);
            w[j] = Vec4<TW>::load(weight + col0 + i);       // asked for now, used after the sums have met
            if (parts) {
                const float4 d = sum_parts4(parts + col0 + i, splits, split_stride);
                v[j].x += d.x; v[j].y += d.y; v[j].z += d.z; v[j].w += d.w;
            } else if (dl) {
                const float4 d = Vec4<TD>::load(dl + col0 + i);
                v[j].x += d.x; v[j].y += d.y; v[j].z += d.z; v[j].w += d.w;
            }
            if (dl && !rows) Vec4<float>::store(res + col0 + i, v[j]);
            ss += v[j].x * v[j].x + v[j].y * v[j].y + v[j].z * v[j].z + v[j].w * v[j].w;
        }
    }
    const float mine = block_sum(ss, red);
    if ((int)threadIdx.x < cluster) llm_cluster_write(&all_ss[c], (uint32_t)threadIdx.x, mine);
    llm_cluster_sync();                       // every block's sum has arrived in every block; no remote access after this
    float total = 0.f;
#pragma unroll
    for (int k = 0; k < 8; ++k)
        if (k < cluster) total += all_ss[k];  // in block order in every block: the same total everywhere
    const float inv = 1.0f / sqrtf(total / (float)width + eps);
    TD* o = out + (size_t)r * width + col0;
#pragma unroll
    for (int j = 0; j < PER_THREAD; ++j) {
        const int i = (threadIdx.x + j * blockDim.x) * 4;
        if (i < cols)
            Vec4<TD>::store(o + i, make_float4(v[j].x * inv * w[j].x, v[j].y * inv * w[j].y, v[j].z * inv * w[j].z, v[j].w * inv * w[j].w));
    }
}

LLM_API int llm_add_rmsnorm(float* residual, const void* delta, const int* rows, const void* weight,
                            int weight_dtype, void* out, int dtype, int out_rows, int width, float eps,
                            int splits, long long split_stride, cudaStream_t stream) {
    if (out_rows == 0) return 0;
    if (splits > 0 && (!delta || split_stride % 4 || splits > kMaxParts))
        LLM_FAIL(-1, "add_rmsnorm: partial sums need a pointer, a stride that is a multiple of 4 and at most %d splits (%d)", kMaxParts, splits);
    const size_t smem = (size_t)width * sizeof(float);
    if (smem > 200 * 1024) LLM_FAIL(-1, "add_rmsnorm: width %d is larger than 51200", width);
    return llm_dispatch_dtype(dtype, [&](auto tag) {
        using TD = decltype(tag);
        return llm_dispatch_dtype(weight_dtype, [&](auto wtag) {
            using TW = decltype(wtag);
            if (width % 4 == 0 && out_rows < 512) {
                // few rows: clusters of up to eight blocks per row, up to 256 threads with up to 4 float4 each
                // (IITJ_NORM_CLUSTER = 1, 2 or 4 for measurements: batch 8 of the 8B shape 5.02 / 4.85 / 4.79 ms per step
                // against 4.80 with 8)
                static const int max_cluster = getenv("IITJ_NORM_CLUSTER") ? atoi(getenv("IITJ_NORM_CLUSTER")) : 8;
                int cluster = max_cluster >= 1 && max_cluster <= 8 ? max_cluster : 8;
                while (cluster > 1 && (width % (4 * cluster) || width / (4 * cluster) < 32)) cluster >>= 1;
                const int vecs = width / (4 * cluster);
                int threads = (vecs + 31) / 32 * 32;
                if (threads > 256) threads = 256;
                const int per = (vecs + threads - 1) / threads;
                if (per <= 4) {
                    auto go = [&](auto kern) {
                        llm_launch_cluster(kern, out_rows * cluster, threads, 0, stream, cluster, residual, (const TD*)delta, rows,
                                           (const TW*)weight, (TD*)out, width, eps, splits, (size_t)split_stride, cluster);
                    };
                    if (per <= 1) go(add_rmsnorm_cluster_kernel<TD, TW, 1>);
                    else if (per <= 2) go(add_rmsnorm_cluster_kernel<TD, TW, 2>);
                    else go(add_rmsnorm_cluster_kernel<TD, TW, 4>);
                    LLM_CHECK_LAUNCH("add_rmsnorm");
                    return 0;
                }
            }
            if (width % 4 == 0 && width <= 4 * 256 * 16) {
                // many rows: one block of 256 threads per row with up to 16 float4 each (bytes in flight per SM)
                const int vecs = width / 4;
                int threads = (vecs + 31) / 32 * 32;
                if (threads > 256) threads = 256;
                const int per = (vecs + threads - 1) / threads;
                auto go = [&](auto kern) {
                    llm_launch(kern, out_rows, threads, 0, stream, residual, (const TD*)delta, rows, (const TW*)weight, (TD*)out, width, eps,
                               splits, (size_t)split_stride);
                };
                if (per <= 1) go(add_rmsnorm_vec_kernel<TD, TW, 1>);
                else if (per <= 2) go(add_rmsnorm_vec_kernel<TD, TW, 2>);
                else if (per <= 4) go(add_rmsnorm_vec_kernel<TD, TW, 4>);
                else if (per <= 8) go(add_rmsnorm_vec_kernel<TD, TW, 8>);
                else go(add_rmsnorm_vec_kernel<TD, TW, 16>);
                LLM_CHECK_LAUNCH("add_rmsnorm");
                return 0;
            }
            auto kern = add_rmsnorm_kernel<TD, TW>;
            if (smem > 48 * 1024) {
                cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
                if (e != cudaSuccess) LLM_FAIL(-2, "add_rmsnorm: %s", cudaGetErrorString(e));
            }
            llm_launch(kern, out_rows, 256, smem, stream, residual, (const TD*)delta, rows, (const TW*)weight,
                                                  (TD*)out, width, eps, splits, (size_t)split_stride);
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
                                  const float* __restrict__ inv_freq, const float* __restrict__ cos_table,
                                  const float* __restrict__ sin_table, const int* __restrict__ slots,
                                  T* __restrict__ cache, int heads, int kv_heads, int head_dim,
                                  int rotary_dim, int page_size) {
    pdl_trigger();
    pdl_wait();
    __shared__ __align__(16) float cs[128], sn[128];  // rotary_dim / 2 <= 128 (head_dim <= 256)
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
    if (cos_table) {   // the step's table: one row of rotary_dim / 2 cosines and sines per token
        for (int i = threadIdx.x; i < half; i += blockDim.x) {
            cs[i] = cos_table[(size_t)t * half + i];
            sn[i] = sin_table[(size_t)t * half + i];
        }
    } else {
        for (int i = threadIdx.x; i < half; i += blockDim.x) sincosf(pos * inv_freq[i], &sn[i], &cs[i]);
    }
    __syncthreads();

    // rotated pairs of query and key heads, four neighbouring pairs per step where the size allows
    const int rot_heads = heads + kv_heads;
    if (half % 4 == 0) {
        const int hp = half / 4;
        for (int w = threadIdx.x; w < rot_heads * hp; w += blockDim.x) {
            const int h = w / hp, i = (w % hp) * 4;
            T* x = row + (size_t)h * head_dim;
            const float4 a = Vec4<T>::load(x + i), b = Vec4<T>::load(x + i + half);
            const float4 c = *reinterpret_cast<const float4*>(cs + i), sg = *reinterpret_cast<const float4*>(sn + i);
            const float4 lo4 = make_float4(a.x * c.x - b.x * sg.x, a.y * c.y - b.y * sg.y, a.z * c.z - b.z * sg.z, a.w * c.w - b.w * sg.w);
            const float4 hi4 = make_float4(b.x * c.x + a.x * sg.x, b.y * c.y + a.y * sg.y, b.z * c.z + a.z * sg.z, b.w * c.w + a.w * sg.w);
            T* dst = nullptr;
            if (h < heads) dst = x;
            else if (slot >= 0) dst = cache + kbase + (size_t)(h - heads) * head_stride;
            if (dst) {
                Vec4<T>::store(dst + i, lo4);
                Vec4<T>::store(dst + i + half, hi4);
            }
        }
    } else {
        const int hp = half / 2;
        for (int w = threadIdx.x; w < rot_heads * hp; w += blockDim.x) {
            const int h = w / hp, i = (w % hp) * 2;
            T* x = row + (size_t)h * head_dim;
            const float a0 = to_f32(x[i]), a1 = to_f32(x[i + 1]), b0 = to_f32(x[i + half]), b1 = to_f32(x[i + half + 1]);
            const T o0 = from_f32<T>(a0 * cs[i] - b0 * sn[i]), o1 = from_f32<T>(a1 * cs[i + 1] - b1 * sn[i + 1]);
            const T p0 = from_f32<T>(b0 * cs[i] + a0 * sn[i]), p1 = from_f32<T>(b1 * cs[i + 1] + a1 * sn[i + 1]);
            T* dst = nullptr;
            if (h < heads) dst = x;
            else if (slot >= 0) dst = cache + kbase + (size_t)(h - heads) * head_stride;
            if (dst) {
                dst[i] = o0; dst[i + 1] = o1; dst[i + half] = p0; dst[i + half + 1] = p1;
            }
        }
    }
    if (slot < 0) return;
    // key dims that are not rotated
    const int pass = head_dim - rotary_dim;
    for (int w = threadIdx.x; w < kv_heads * pass; w += blockDim.x) {
        const int h = w / pass, i = rotary_dim + w % pass;
        cache[kbase + (size_t)h * head_stride + i] = row[(size_t)(heads + h) * head_dim + i];
    }
    // values, 16 bytes at a time (head_dim is a multiple of 16 elements)
    constexpr int V16 = 16 / sizeof(T);
    const T* v = row + (size_t)(heads + kv_heads) * head_dim;
    const int per_head = head_dim / V16;
    for (int w = threadIdx.x; w < kv_heads * per_head; w += blockDim.x) {
        const int h = w / per_head, i = (w % per_head) * V16;
        *reinterpret_cast<uint4*>(cache + kbase + plane + (size_t)h * head_stride + i) =
            *reinterpret_cast<const uint4*>(v + (size_t)h * head_dim + i);
    }
}

// The same for a qkv that still lies in the float32 partial sums [splits][tokens][row_width] of a k-split
// product (rotary_dim == head_dim, head_dim % 8 == 0, at most kMaxParts splits): the sums are taken here in
// split order, the rotated queries go to `q_out` (row width as qkv), keys and values to the cache.  One block
// per token and group of eight heads; every thread has all loads of its item in flight at once.
constexpr int kSumHeads = 8;

template <typename T>
__global__ void rope_store_sum_kernel(const float* __restrict__ parts, int splits, size_t split_stride,
                                      T* __restrict__ q_out, const int* __restrict__ positions,
                                      const float* __restrict__ inv_freq, const float* __restrict__ cos_table,
                                      const float* __restrict__ sin_table, const int* __restrict__ slots,
                                      T* __restrict__ cache, int heads, int kv_heads, int head_dim, int page_size) {
    pdl_trigger();
    pdl_wait();
    const int t = blockIdx.x;
    const int half = head_dim / 2, hp = half / 4, per_head = head_dim / 4;
    const int all_heads = heads + 2 * kv_heads, rot_heads = heads + kv_heads;
    const int row_width = all_heads * head_dim;
    const float* row = parts + (size_t)t * row_width;
    T* qrow = q_out + (size_t)t * row_width;
    const int slot = slots ? slots[t] : -1;
    const size_t plane = (size_t)kv_heads * page_size * head_dim;
    size_t kbase = 0;
    if (slot >= 0) {
        const int page = slot / page_size, off = slot % page_size;
        kbase = (size_t)page * 2 * plane + (size_t)off * head_dim;
    }
    const size_t head_stride = (size_t)page_size * head_dim;
    const int h0 = blockIdx.y * kSumHeads;
    // items of this block: per rotated head `hp` pairs of four dims, per value head `per_head` groups of four
    for (int w = threadIdx.x; w < kSumHeads * per_head; w += blockDim.x) {
        const int h = h0 + w / per_head, j = w % per_head;
        if (h >= all_heads) break;
        if (h < rot_heads) {
            if (j >= hp) continue;
            const int i = j * 4;
            const float4 a = sum_parts4(row + h * head_dim + i, splits, split_stride);
            const float4 b = sum_parts4(row + h * head_dim + i + half, splits, split_stride);
            float4 c, sg;
            if (cos_table) {
                c = *reinterpret_cast<const float4*>(cos_table + (size_t)t * half + i);
                sg = *reinterpret_cast<const float4*>(sin_table + (size_t)t * half + i);
            } else {
                const float pos = (float)positions[t];
                sincosf(pos * inv_freq[i], &sg.x, &c.x); sincosf(pos * inv_freq[i + 1], &sg.y, &c.y);
                sincosf(pos * inv_freq[i + 2], &sg.z, &c.z); sincosf(pos * inv_freq[i + 3], &sg.w, &c.w);
            }
            const float4 lo4 = make_float4(a.x * c.x - b.x * sg.x, a.y * c.y - b.y * sg.y, a.z * c.z - b.z * sg.z, a.w * c.w - b.w * sg.w);
            const float4 hi4 = make_float4(b.x * c.x + a.x * sg.x, b.y * c.y + a.y * sg.y, b.z * c.z + a.z * sg.z, b.w * c.w + a.w * sg.w);
            T* dst = nullptr;
            if (h < heads) dst = qrow + (size_t)h * head_dim;
            else if (slot >= 0) dst = cache + kbase + (size_t)(h - heads) * head_stride;
            if (dst) {
                Vec4<T>::store(dst + i, lo4);
                Vec4<T>::store(dst + i + half, hi4);
            }
        } else if (slot >= 0) {
            const int i = j * 4;
            Vec4<T>::store(cache + kbase + plane + (size_t)(h - rot_heads) * head_stride + i,
                           sum_parts4(row + h * head_dim + i, splits, split_stride));
        }
    }
}

// cos[t, i] = cos(positions[t] * inv_freq[i]), sin likewise: computed once per step and shared by all
// layers with the same position encoding (float32 angles, float32 sincosf).
__global__ void rope_table_kernel(const int* __restrict__ positions, const float* __restrict__ inv_freq,
                                  float* __restrict__ cos_table, float* __restrict__ sin_table, int tokens, int half) {
    pdl_trigger();
    pdl_wait();
    const int idx = blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= tokens * half) return;
    const int t = idx / half, i = idx % half;
    sincosf((float)positions[t] * inv_freq[i], &sin_table[idx], &cos_table[idx]);
}

LLM_API int llm_rope_table(const int* positions, const float* inv_freq, float* cos_table, float* sin_table,
                           int tokens, int half, cudaStream_t stream) {
    if (tokens == 0 || half == 0) return 0;
    const int total = tokens * half;
    llm_launch(rope_table_kernel, (total + 255) / 256, 256, 0, stream, positions, inv_freq, cos_table, sin_table, tokens, half);
    LLM_CHECK_LAUNCH("rope_table");
    return 0;
}

LLM_API int llm_rope_store(void* qkv, const int* positions, const float* inv_freq, const float* cos_table,
                           const float* sin_table, const int* slots, void* cache, int dtype, int tokens, int heads, int kv_heads, int head_dim,
                           int rotary_dim, int page_size, const float* parts, int splits, long long split_stride, cudaStream_t stream) {
    if (tokens == 0) return 0;
    if (parts) {
        if (rotary_dim != head_dim || head_dim % 8 || splits < 1 || splits > kMaxParts || split_stride % 4)
            LLM_FAIL(-1, "rope_store: partial sums need rotary_dim == head_dim (%d, %d), a multiple of 8, and 1..%d splits (%d)",
                     rotary_dim, head_dim, kMaxParts, splits);
        return llm_dispatch_dtype(dtype, [&](auto tag) {
            using T = decltype(tag);
            const dim3 grid(tokens, (heads + 2 * kv_heads + kSumHeads - 1) / kSumHeads);
            llm_launch(rope_store_sum_kernel<T>, grid, 256, 0, stream, parts, splits, (size_t)split_stride, (T*)qkv, positions, inv_freq,
                       cos_table, sin_table, slots, (T*)cache, heads, kv_heads, head_dim, page_size);
            LLM_CHECK_LAUNCH("rope_store");
            return 0;
        });
    }
    if (rotary_dim < 0 || rotary_dim > head_dim || (rotary_dim & 3) || head_dim % 16 || head_dim > 256)
        LLM_FAIL(-1, "rope_store: rotary_dim %d must be a multiple of 4 and at most head_dim %d (a multiple of 16 up to 256)",
                 rotary_dim, head_dim);
    return llm_dispatch_dtype(dtype, [&](auto tag) {
        using T = decltype(tag);
        llm_launch(rope_store_kernel<T>, tokens, 256, 0, stream, (T*)qkv, positions, inv_freq, cos_table, sin_table, slots, (T*)cache,
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
    pdl_trigger();
    pdl_wait();
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
         idx += (size_t)gridDim.x * blockDim.x) {
        const size_t t = idx / inner, i = idx % inner;
        const float g = to_f32(gu[t * 2 * inner + i]);
        const float u = to_f32(gu[t * 2 * inner + inner + i]);
        act[idx] = from_f32<T>(g / (1.0f + expf(-g)) * u);
    }
}

// inner % 8 == 0: eight elements per thread and step (16-byte loads in bfloat16)
template <typename T>
__global__ void silu_mul_vec_kernel(const T* __restrict__ gu, T* __restrict__ act, int inner, size_t total8) {
    pdl_trigger();
    pdl_wait();
    const int inner8 = inner / 8;
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total8;
         idx += (size_t)gridDim.x * blockDim.x) {
        const size_t t = idx / inner8, i = (idx % inner8) * 8;
        const T* gp = gu + t * 2 * inner + i;
        const float4 g0 = Vec4<T>::load(gp), g1 = Vec4<T>::load(gp + 4);
        const float4 u0 = Vec4<T>::load(gp + inner), u1 = Vec4<T>::load(gp + inner + 4);
        T* dst = act + t * inner + i;
        Vec4<T>::store(dst, make_float4(g0.x / (1.0f + expf(-g0.x)) * u0.x, g0.y / (1.0f + expf(-g0.y)) * u0.y,
                                        g0.z / (1.0f + expf(-g0.z)) * u0.z, g0.w / (1.0f + expf(-g0.w)) * u0.w));
        Vec4<T>::store(dst + 4, make_float4(g1.x / (1.0f + expf(-g1.x)) * u1.x, g1.y / (1.0f + expf(-g1.y)) * u1.y,
                                            g1.z / (1.0f + expf(-g1.z)) * u1.z, g1.w / (1.0f + expf(-g1.w)) * u1.w));
    }
}

LLM_API int llm_silu_mul(const void* gu, void* act, int dtype, int tokens, int inner, cudaStream_t stream) {
    const size_t total = (size_t)tokens * inner;
    if (total == 0) return 0;
    return llm_dispatch_dtype(dtype, [&](auto tag) {
        using T = decltype(tag);
        if (inner % 8 == 0) {
            const size_t total8 = total / 8;
            const int blocks = (int)((total8 + 255) / 256 < 148 * 32 ? (total8 + 255) / 256 : 148 * 32);
            llm_launch(silu_mul_vec_kernel<T>, blocks, 256, 0, stream, (const T*)gu, (T*)act, inner, total8);
        } else {
            const int blocks = (int)((total + 255) / 256 < 148 * 16 ? (total + 255) / 256 : 148 * 16);
            llm_launch(silu_mul_kernel<T>, blocks, 256, 0, stream, (const T*)gu, (T*)act, inner, total);
        }
        LLM_CHECK_LAUNCH("silu_mul");
        return 0;
    });
}

// ---------------------------------------------------------------------------------------
// small float32 helpers: x *= scale (a head with a logit scale), and out = sum over the first
// dimension of parts [splits, n] (k-split partial sums whose reader is no kernel of this library)
// ---------------------------------------------------------------------------------------
namespace {

__global__ void scale_kernel(float* __restrict__ x, float scale, size_t n) {
    pdl_trigger();
    pdl_wait();
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) x[i] *= scale;
}

// parts are added in split order, as every other reader of deferred sums adds them
template <typename TO>
__global__ void sum_parts_kernel(const float* __restrict__ parts, TO* __restrict__ out, int splits, size_t n) {
    pdl_trigger();
    pdl_wait();
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        float a = parts[i];
        for (int s = 1; s < splits; ++s) a += parts[(size_t)s * n + i];
        out[i] = from_f32<TO>(a);
    }
}

}  // namespace

LLM_API int llm_scale_f32(float* x, float scale, long long n, cudaStream_t stream) {
    if (n <= 0) return 0;
    const int blocks = (int)((n + 255) / 256 < 148 * 16 ? (n + 255) / 256 : 148 * 16);
    llm_launch(scale_kernel, blocks, 256, 0, stream, x, scale, (size_t)n);
    LLM_CHECK_LAUNCH("scale_f32");
    return 0;
}

// out [n] (dtype `out_dtype`) = parts[0] + parts[1] + ... + parts[splits - 1], each [n] float32
LLM_API int llm_sum_parts(const float* parts, void* out, int out_dtype, int splits, long long n, cudaStream_t stream) {
    if (n <= 0 || splits <= 0) return 0;
    const int blocks = (int)((n + 255) / 256 < 148 * 16 ? (n + 255) / 256 : 148 * 16);
    return llm_dispatch_dtype(out_dtype, [&](auto tag) {
        using T = decltype(tag);
        llm_launch(sum_parts_kernel<T>, blocks, 256, 0, stream, parts, (T*)out, splits, (size_t)n);
        LLM_CHECK_LAUNCH("sum_parts");
        return 0;
    });
}

LLM_TRACE_EXPORT(elementwise)
