// Token sampling from float32 logits: greedy (argmax, the lowest index wins a tie) and
// temperature sampling, mixed row by row in one launch.
//
// The reference samples with softmax(logits / T) followed by torch.multinomial
// (engine/spec_decode.py:12-17).  Here a row with temperature T > 0 takes
//     argmax_i ( logits[i] / T + g_i ),   g_i = -log(-log(u_i)),
// which draws from exactly that softmax (the Gumbel-max identity) in one pass over the
// row.  u_i comes from a counter-based generator keyed by a 64-bit value per row that the
// host derives from (engine seed, request seed, index of the token in its request), so a
// request's tokens do not depend on what else is in the batch.
#include "common.cuh"

#include <mutex>

namespace {

// The library's health words (see common.cuh), copied out beside the sampled ids by the last kernel of a call.
struct HealthWords { const int* word[kHealthWords]; };

__device__ __forceinline__ void copy_health(const HealthWords& hw, int* health_out) {
    if (health_out && blockIdx.x == 0 && threadIdx.x < kHealthWords)
        health_out[threadIdx.x] = hw.word[threadIdx.x] ? *hw.word[threadIdx.x] : 0;
}

__device__ __forceinline__ uint64_t mix64(uint64_t z) {  // splitmix64 finaliser
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}

__device__ __forceinline__ float gumbel(uint64_t key, uint32_t i) {
    const uint64_t r = mix64(key + 0x9E3779B97F4A7C15ull * (uint64_t)(i + 1));
    const float u = ((float)(uint32_t)(r >> 40) + 0.5f) * (1.0f / 16777216.0f);  // (0, 1)
    return -logf(-logf(u));
}

__global__ void __launch_bounds__(1024)
sample_kernel(const float* __restrict__ logits, int ld, const float* __restrict__ temperature,
              const unsigned long long* __restrict__ keys, int* __restrict__ out, int vocab, const HealthWords hw,
              int* __restrict__ health_out) {
    pdl_trigger();
    pdl_wait();
    copy_health(hw, health_out);
    __shared__ float best_v[32];
    __shared__ int best_i[32];
    const int r = blockIdx.x;
    const float* row = logits + (size_t)r * ld;
    const float T = temperature ? temperature[r] : 0.f;
    const uint64_t key = keys ? keys[r] : 0ull;
    float bv = -INFINITY;
    int bi = 0x7fffffff;
    for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
        float v = row[i];
        if (T > 0.f) v = v / T + gumbel(key, (uint32_t)i);
        if (v > bv || (v == bv && i < bi)) { bv = v; bi = i; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (lane == 0) { best_v[warp] = bv; best_i[warp] = bi; }
    __syncthreads();
    if (warp == 0) {
        const int nwarp = blockDim.x >> 5;
        bv = lane < nwarp ? best_v[lane] : -INFINITY;
        bi = lane < nwarp ? best_i[lane] : 0x7fffffff;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
        }
        if (lane == 0) out[r] = bi == 0x7fffffff ? 0 : bi;  // a row of NaNs yields token 0
    }
}

constexpr int kChunk = 2048;   // vocabulary entries per block of the two-stage form

// Stage 1: the best (value, index) of one chunk of one row.
__global__ void __launch_bounds__(256)
sample_chunk_kernel(const float* __restrict__ logits, int ld, const float* __restrict__ temperature,
                    const unsigned long long* __restrict__ keys, float* __restrict__ part_v, int* __restrict__ part_i,
                    int vocab, int chunks) {
    pdl_trigger();
    pdl_wait();
    __shared__ float best_v[8];
    __shared__ int best_i[8];
    const int c = blockIdx.x, r = blockIdx.y;
    const float* row = logits + (size_t)r * ld;
    const float T = temperature ? temperature[r] : 0.f;
    const uint64_t key = keys ? keys[r] : 0ull;
    const int end = min(vocab, (c + 1) * kChunk);
    float bv = -INFINITY;
    int bi = 0x7fffffff;
    for (int i = c * kChunk + threadIdx.x; i < end; i += 256) {
        float v = row[i];
        if (T > 0.f) v = v / T + gumbel(key, (uint32_t)i);
        if (v > bv || (v == bv && i < bi)) { bv = v; bi = i; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (lane == 0) { best_v[warp] = bv; best_i[warp] = bi; }
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int w = 1; w < 8; ++w)
            if (best_v[w] > bv || (best_v[w] == bv && best_i[w] < bi)) { bv = best_v[w]; bi = best_i[w]; }
        part_v[(size_t)r * chunks + c] = bv;
        part_i[(size_t)r * chunks + c] = bi;
    }
}

// Stage 2: the best over a row's chunks (one warp per row).
__global__ void __launch_bounds__(32)
sample_pick_kernel(const float* __restrict__ part_v, const int* __restrict__ part_i, int* __restrict__ out, int chunks,
                   const HealthWords hw, int* __restrict__ health_out) {
    pdl_trigger();
    pdl_wait();
    copy_health(hw, health_out);
    const int r = blockIdx.x;
    float bv = -INFINITY;
    int bi = 0x7fffffff;
    for (int c = threadIdx.x; c < chunks; c += 32) {
        const float v = part_v[(size_t)r * chunks + c];
        const int i = part_i[(size_t)r * chunks + c];
        if (v > bv || (v == bv && i < bi)) { bv = v; bi = i; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
    }
    if (threadIdx.x == 0) out[r] = bi == 0x7fffffff ? 0 : bi;
}

// Device addresses of the health words on the current device, looked up once per device.
constexpr int kMaxDevices = 64;
HealthWords g_health[kMaxDevices];
bool g_health_known[kMaxDevices] = {};
std::mutex g_health_mutex;

int health_words(HealthWords* out) {
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) LLM_FAIL(-2, "sample: cudaGetDevice: %s", cudaGetErrorString(e));
    if (dev < 0 || dev >= kMaxDevices) LLM_FAIL(-1, "sample: device index %d out of range", dev);
    std::lock_guard<std::mutex> lock(g_health_mutex);
    if (!g_health_known[dev]) {
        g_health[dev].word[0] = llm_gemm_bf16_status_word();
        g_health[dev].word[1] = llm_gemm_bf16_pair_status_word();
        g_health[dev].word[2] = llm_attention_tcgen05_status_word();
        g_health[dev].word[3] = llm_attention_decode_status_word();
        for (int i = 0; i < kHealthWords; ++i)
            if (!g_health[dev].word[i]) LLM_FAIL(-2, "sample: the address of health word %d could not be looked up", i);
        g_health_known[dev] = true;
    }
    *out = g_health[dev];
    return 0;
}

}  // namespace

// dst[i] = src[rows[i]] where rows[i] >= 0: feeds the ids sampled by the previous step into this step's token
// slots on the device, so the host can launch a step before it has read the previous step's tokens.
__global__ void gather_tokens_kernel(int* __restrict__ dst, const int* __restrict__ src, const int* __restrict__ rows, int n) {
    pdl_trigger();
    pdl_wait();
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n && rows[i] >= 0) dst[i] = src[rows[i]];
}

LLM_API int llm_gather_tokens(int* dst, const int* src, const int* rows, int n, cudaStream_t stream) {
    if (n == 0) return 0;
    llm_launch(gather_tokens_kernel, (n + 255) / 256, 256, 0, stream, dst, src, rows, n);
    LLM_CHECK_LAUNCH("gather_tokens");
    return 0;
}

// Number of floats of scratch llm_sample wants for `rows` rows of `vocab` logits (0: none needed).
LLM_API int llm_sample_scratch_floats(int rows, int vocab) {
    const int chunks = (vocab + kChunk - 1) / kChunk;
    return chunks > 1 ? 2 * rows * chunks : 0;
}

// scratch: llm_sample_scratch_floats(rows, vocab) floats, or null to scan each row with a single block.
// health_out: null, or kHealthWords (4) ints that receive the library's status words as they stand when this call's
// last kernel runs (tcgen05 product, CTA-pair product, tcgen05 attention, decode attention; 0 = fine).  The words
// are not cleared: the llm_*_status functions do that.
LLM_API int llm_sample(const float* logits, int ld, const float* temperature, const unsigned long long* keys,
                       int* out, int rows, int vocab, float* scratch, int* health_out, cudaStream_t stream) {
    if (rows == 0) return 0;
    HealthWords hw = {};
    if (health_out)
        if (int rc = health_words(&hw)) return rc;
    const int chunks = (vocab + kChunk - 1) / kChunk;
    if (scratch && chunks > 1) {
        if (rows > 65535) LLM_FAIL(-1, "sample: too many rows");
        float* part_v = scratch;
        int* part_i = reinterpret_cast<int*>(scratch + (size_t)rows * chunks);
        llm_launch(sample_chunk_kernel, dim3(chunks, rows), 256, 0, stream, logits, ld, temperature, keys, part_v, part_i, vocab, chunks);
        LLM_CHECK_LAUNCH("sample");
        llm_launch(sample_pick_kernel, rows, 32, 0, stream, (const float*)part_v, (const int*)part_i, out, chunks, hw, health_out);
        LLM_CHECK_LAUNCH("sample_pick");
        return 0;
    }
    llm_launch(sample_kernel, rows, 1024, 0, stream, logits, ld, temperature, keys, out, vocab, hw, health_out);
    LLM_CHECK_LAUNCH("sample");
    return 0;
}

LLM_TRACE_EXPORT(sample)
