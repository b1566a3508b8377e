// Shared helpers of the sm_100a kernels: element types, conversions, reductions, error text.
//
// Every launcher is an `extern "C"` function that takes raw device pointers, explicit sizes
// and a stream, launches on that stream, allocates nothing and returns 0 or a negative
// code after leaving a message that `llm_last_error()` returns.  The Python side
// (kernels/__init__.py) checks shapes, dtypes and contiguity before it calls in.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#define LLM_API extern "C" __attribute__((visibility("default")))

enum LlmDtype { LLM_F32 = 0, LLM_BF16 = 1 };

// ---- error reporting (host) ------------------------------------------------------------
char* llm_error_buffer();  // defined in runtime.cu; one buffer per process

#define LLM_FAIL(code, ...)                                        \
    do {                                                           \
        snprintf(llm_error_buffer(), 512, __VA_ARGS__);            \
        return (code);                                             \
    } while (0)

#define LLM_CHECK_LAUNCH(name)                                                       \
    do {                                                                             \
        cudaError_t e_ = cudaGetLastError();                                         \
        if (e_ != cudaSuccess) LLM_FAIL(-2, "%s: %s", name, cudaGetErrorString(e_)); \
    } while (0)

// ---- health words (host) -----------------------------------------------------------------
// Kernels with bounded waits, and kernels that check a caller's contract on the device, leave a code in a status
// word of their file when something went wrong (0 = fine).  These return the words' device addresses on the current
// device (null if the lookup fails); llm_sample copies the words out beside the sampled ids, so a serving loop
// sees them at the place where it reads its tokens anyway, without a synchronisation of its own.
constexpr int kHealthWords = 4;
const int* llm_gemm_bf16_status_word();          // gemm_bf16.cu
const int* llm_gemm_bf16_pair_status_word();     // gemm_bf16_pair.cu
const int* llm_attention_tcgen05_status_word();  // attention_tcgen05.cu
const int* llm_attention_decode_status_word();   // attention_bf16.cu

// ---- element conversions (device) ------------------------------------------------------
__device__ __forceinline__ float to_f32(float v) { return v; }
__device__ __forceinline__ float to_f32(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) {
    return __float2bfloat16_rn(v);
}

// ---- reductions ------------------------------------------------------------------------
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Sum over a block whose size is a multiple of 32 (at most 1024).  The order of additions
// depends only on blockDim, never on the data or on other blocks, so a row's result is
// the same in whatever batch it is computed.
__device__ __forceinline__ float block_sum(float v, float* scratch /* >= 32 floats */) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
    v = warp_sum(v);
    __syncthreads();  // scratch may still be read from an earlier call
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    float t = (lane < nwarp) ? scratch[lane] : 0.f;
    return warp_sum(t);
}

// ---- partial sums of a k-split matrix product ---------------------------------------------
// Sum of up to kMaxParts partial sums of four neighbouring elements, all loads in flight at once; the parts are
// added in split order, so every kernel that reads a deferred sum gets the same value.
constexpr int kMaxParts = 8;

__device__ __forceinline__ float4 sum_parts4(const float* p, int splits, size_t split_stride) {
    float4 e[kMaxParts];
#pragma unroll
    for (int k = 0; k < kMaxParts; ++k)
        if (k < splits) e[k] = *reinterpret_cast<const float4*>(p + (size_t)k * split_stride);
    float4 a = e[0];
#pragma unroll
    for (int k = 1; k < kMaxParts; ++k)
        if (k < splits) { a.x += e[k].x; a.y += e[k].y; a.z += e[k].z; a.w += e[k].w; }
    return a;
}

// ---- programmatic dependent launch ---------------------------------------------------------
// Every kernel of this library is launched with the "programmatic stream serialization"
// attribute (unless llm_set_pdl(0)): its CTAs may be scheduled while the kernel before it in
// the stream is still running, do work that depends on nothing that kernel writes (barrier
// set-up, tensor-memory allocation, weight prefetch), and then block in pdl_wait() until the
// earlier kernel has completed and its writes are visible.  pdl_trigger() at a kernel's top
// tells the scheduler that the next kernel may start as soon as resources allow.  Both are
// no-ops in a launch without the attribute.
#ifdef LLM_TRACE
// Measurement build (-DLLM_TRACE): the first thread of every kernel's first block notes the global timer when
// the kernel starts and when its wait for the kernel before it returns; one buffer per source file, read
// with llm_trace_dump_<file>().
namespace {
__device__ unsigned long long llm_trace_buf[1 << 14];
__device__ unsigned int llm_trace_n;
__device__ __forceinline__ void llm_trace_mark(unsigned what) {
    if (threadIdx.x == 0 && threadIdx.y == 0 && blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0) {
        unsigned long long t;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
        const unsigned i = atomicAdd(&llm_trace_n, 1u);
        if (i < (1u << 14)) llm_trace_buf[i] = (t << 4) | what;
    }
}
}  // namespace
#define LLM_TRACE_EXPORT(name)                                                                          \
    LLM_API int llm_trace_dump_##name(unsigned long long* host, int cap) {                              \
        unsigned int n = 0, zero = 0;                                                                   \
        cudaMemcpyFromSymbol(&n, llm_trace_n, sizeof(n));                                               \
        if ((int)n > cap) n = cap;                                                                      \
        if (n > (1u << 14)) n = 1u << 14;                                                               \
        cudaMemcpyFromSymbol(host, llm_trace_buf, sizeof(unsigned long long) * n);                      \
        cudaMemcpyToSymbol(llm_trace_n, &zero, sizeof(zero));                                           \
        return (int)n;                                                                                  \
    }
#else
#define LLM_TRACE_EXPORT(name)
__device__ __forceinline__ void llm_trace_mark(unsigned) {}
#endif
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); llm_trace_mark(1); }
__device__ __forceinline__ void pdl_trigger() { llm_trace_mark(0); asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

bool llm_pdl_enabled();  // runtime.cu

template <typename... KArgs, typename... Args>
static inline cudaError_t llm_launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                     Args&&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    if (llm_pdl_enabled()) {
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
    }
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

// The same for a kernel whose blocks form clusters of `cluster_x` along x (distributed shared memory).
template <typename... KArgs, typename... Args>
static inline cudaError_t llm_launch_cluster(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                             unsigned cluster_x, Args&&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = cluster_x; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
    cfg.numAttrs = 1;
    if (llm_pdl_enabled()) {
        attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[1].val.programmaticStreamSerializationAllowed = 1;
        cfg.numAttrs = 2;
    }
    cfg.attrs = attr;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

// ---- thread-block clusters (device) -------------------------------------------------------
__device__ __forceinline__ uint32_t llm_cluster_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void llm_cluster_sync() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// Stores `v` at the same shared-memory location in block `rank` of this cluster.
__device__ __forceinline__ void llm_cluster_write(float* local, uint32_t rank, float v) {
    uint32_t addr;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(addr) : "r"((uint32_t)__cvta_generic_to_shared(local)), "r"(rank));
    asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(addr), "f"(v) : "memory");
}

template <typename F> static inline int llm_dispatch_dtype(int dtype, F&& f) {
    if (dtype == LLM_F32) return f(float{});
    if (dtype == LLM_BF16) return f(__nv_bfloat16{});
    LLM_FAIL(-1, "unknown dtype code %d", dtype);
}
