// Row-wise kernels of a layer whose parts are normed on both sides ("sandwich" norms), and the two
// element-wise steps its parts need.
//
// norm_add: the norm BEHIND a part, the residual sum and the norm in front of the next part in one
// launch, one block per token. y holds `terms` result rows per token (a part that leaves several
// partial results, e.g. one per chosen expert, has them added here in index order):
//     s = sum_k y[t * terms + k]         (32-bit, fixed order)
//     x[t] += s / sqrt(mean(s^2) + eps_post) * gain_post
//     h[t]  = x[t] / sqrt(mean(x[t]^2) + eps_next) * gain_next        (if gain_next; run dtype)
// Both sums of squares are reduced in one fixed order (thread order, lanes, warps), so a row's
// result does not depend on the batch.
//
// gelu: the tanh form, in place.  sigmoid_gate: out *= sigmoid(gate), rows with strides.
// fill: a constant into a 32-bit buffer.  add_terms: x[t] += the sum of a token's result rows.
#include "common.cuh"

using namespace llmb;

LLMB_DEFINE_LAST_ERROR(llmb_post_norm)

constexpr int THREADS = 256;

__device__ __forceinline__ float block_sum(float v, float* scratch) {
    v = warp_sum(v);
    int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    float total = 0.f;
#pragma unroll
    for (int w = 0; w < THREADS / 32; ++w) total += scratch[w];
    return total;
}

template <typename TOut>
__global__ void __launch_bounds__(THREADS)
norm_add_kernel(const float* __restrict__ y, int terms, const float* __restrict__ gain_post, float eps_post,
                float* __restrict__ x, const float* __restrict__ gain_next, float eps_next, TOut* __restrict__ h,
                int hidden) {
    extern __shared__ float row[];         // [hidden]
    __shared__ float scratch[THREADS / 32];
    griddep_launch();
    griddep_wait();
    size_t t = blockIdx.x;
    float sq = 0.f;
    for (int c = threadIdx.x; c < hidden; c += THREADS) {
        float s = 0.f;
        for (int k = 0; k < terms; ++k) s += y[(t * terms + k) * hidden + c];
        row[c] = s;
        sq = fmaf(s, s, sq);
    }
    float rstd = 1.0f / sqrtf(block_sum(sq, scratch) / (float)hidden + eps_post);
    sq = 0.f;
    for (int c = threadIdx.x; c < hidden; c += THREADS) {
        float v = x[t * hidden + c] + row[c] * rstd * gain_post[c];
        x[t * hidden + c] = v;
        row[c] = v;
        sq = fmaf(v, v, sq);
    }
    if (!gain_next) return;
    rstd = 1.0f / sqrtf(block_sum(sq, scratch) / (float)hidden + eps_next);
    for (int c = threadIdx.x; c < hidden; c += THREADS)
        h[t * hidden + c] = from_float<TOut>(row[c] * rstd * gain_next[c]);
}

LLMB_EXPORT int llmb_norm_add(const float* y, int terms, const float* gain_post, float eps_post, float* x,
                              const float* gain_next, float eps_next, void* h, int h_dtype, int n_rows, int hidden,
                              cudaStream_t stream) {
    if (n_rows == 0) return LLMB_OK;
    LLMB_REQUIRE(hidden > 0 && terms > 0 && y && x && gain_post, "norm_add: bad sizes or a missing array");
    LLMB_REQUIRE(!gain_next || h, "norm_add: the next norm has no output");
    size_t smem = sizeof(float) * (size_t)hidden;
    LLMB_REQUIRE(smem <= 200 * 1024, "norm_add: a row of %d values does not fit in shared memory", hidden);
#define LLMB_NORM_ADD(T)                                                                                           \
    do {                                                                                                           \
        if (smem > 48 * 1024)                                                                                      \
            LLMB_CUDA(cudaFuncSetAttribute(norm_add_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)); \
        LLMB_CUDA(llmb::launch(norm_add_kernel<T>, dim3(n_rows), dim3(THREADS), smem, stream, true, y, terms,      \
                               gain_post, eps_post, x, gain_next, eps_next, (T*)h, hidden));                       \
    } while (0)
    if (h_dtype == LLMB_DTYPE_F32) LLMB_NORM_ADD(float);
    else if (h_dtype == LLMB_DTYPE_BF16) LLMB_NORM_ADD(__nv_bfloat16);
    else return fail(LLMB_ERR_ARGUMENT, "norm_add: unknown dtype %d", h_dtype);
#undef LLMB_NORM_ADD
    return check_launch("norm_add");
}
LLMB_PACKED(llmb_norm_add)

__device__ __forceinline__ float gelu_tanh(float z) {
    return 0.5f * z * (1.0f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
}

// 16 bytes a thread where the address allows it (`vectors`), the last elements one by one
template <typename T>
__global__ void gelu_kernel(T* __restrict__ a, long long n, int vectors) {
    griddep_launch();
    griddep_wait();
    constexpr int VEC = 16 / sizeof(T);
    long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (vectors) {
        long long first = i * VEC;
        if (first + VEC <= n) {
            uint4 raw = reinterpret_cast<const uint4*>(a)[i];
            T* e = reinterpret_cast<T*>(&raw);
#pragma unroll
            for (int j = 0; j < VEC; ++j) e[j] = from_float<T>(gelu_tanh(to_float(e[j])));
            reinterpret_cast<uint4*>(a)[i] = raw;
        } else {
            for (long long k = first; k < n; ++k) a[k] = from_float<T>(gelu_tanh(to_float(a[k])));
        }
        return;
    }
    if (i < n) a[i] = from_float<T>(gelu_tanh(to_float(a[i])));
}

LLMB_EXPORT int llmb_gelu(void* a, int dtype, long long n, cudaStream_t stream) {
    if (n == 0) return LLMB_OK;
    LLMB_REQUIRE(n > 0 && a, "gelu: bad size");
    int vectors = ((size_t)a % 16) == 0;
    long long per_thread = vectors ? (dtype == LLMB_DTYPE_F32 ? 4 : 8) : 1;
    long long threads = (n + per_thread - 1) / per_thread;
    unsigned blocks = (unsigned)((threads + 255) / 256);
    if (dtype == LLMB_DTYPE_F32)
        LLMB_CUDA(llmb::launch(gelu_kernel<float>, dim3(blocks), dim3(256), 0, stream, true, (float*)a, n, vectors));
    else if (dtype == LLMB_DTYPE_BF16)
        LLMB_CUDA(llmb::launch(gelu_kernel<__nv_bfloat16>, dim3(blocks), dim3(256), 0, stream, true, (__nv_bfloat16*)a, n, vectors));
    else return fail(LLMB_ERR_ARGUMENT, "gelu: unknown dtype %d", dtype);
    return check_launch("gelu");
}
LLMB_PACKED(llmb_gelu)

// `vectors`: 16 bytes a thread (width, both strides and both addresses allow it)
template <typename T>
__global__ void sigmoid_gate_kernel(T* __restrict__ out, int out_stride, const T* __restrict__ gate, int gate_stride,
                                    int width, long long total, int vectors) {
    griddep_launch();
    griddep_wait();
    constexpr int VEC = 16 / sizeof(T);
    long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (vectors) {
        int per_row = width / VEC;
        if (i >= total / VEC) return;
        long long t = i / per_row;
        int c = (int)(i % per_row) * VEC;
        uint4 g_raw = *reinterpret_cast<const uint4*>(gate + t * gate_stride + c);
        uint4* dst = reinterpret_cast<uint4*>(out + t * out_stride + c);
        uint4 v_raw = *dst;
        const T* g = reinterpret_cast<const T*>(&g_raw);
        T* v = reinterpret_cast<T*>(&v_raw);
#pragma unroll
        for (int j = 0; j < VEC; ++j) v[j] = from_float<T>(to_float(v[j]) / (1.0f + expf(-to_float(g[j]))));
        *dst = v_raw;
        return;
    }
    if (i >= total) return;
    long long t = i / width;
    int c = (int)(i % width);
    float g = to_float(gate[t * gate_stride + c]);
    float v = to_float(out[t * out_stride + c]);
    out[t * out_stride + c] = from_float<T>(v / (1.0f + expf(-g)));
}

LLMB_EXPORT int llmb_sigmoid_gate(void* out, int out_stride, const void* gate, int gate_stride, int dtype, int n_rows,
                                  int width, cudaStream_t stream) {
    if (n_rows == 0) return LLMB_OK;
    LLMB_REQUIRE(width > 0 && out_stride >= width && gate_stride >= width, "sigmoid_gate: bad widths");
    long long total = (long long)n_rows * width;
    int vec = dtype == LLMB_DTYPE_F32 ? 4 : 8;
    int vectors = width % vec == 0 && out_stride % vec == 0 && gate_stride % vec == 0 && ((size_t)out % 16) == 0 &&
                  ((size_t)gate % 16) == 0;
    long long threads = vectors ? total / vec : total;
    unsigned blocks = (unsigned)((threads + 255) / 256);
    if (dtype == LLMB_DTYPE_F32)
        LLMB_CUDA(llmb::launch(sigmoid_gate_kernel<float>, dim3(blocks), dim3(256), 0, stream, true, (float*)out, out_stride,
                               (const float*)gate, gate_stride, width, total, vectors));
    else if (dtype == LLMB_DTYPE_BF16)
        LLMB_CUDA(llmb::launch(sigmoid_gate_kernel<__nv_bfloat16>, dim3(blocks), dim3(256), 0, stream, true,
                               (__nv_bfloat16*)out, out_stride, (const __nv_bfloat16*)gate, gate_stride, width, total, vectors));
    else return fail(LLMB_ERR_ARGUMENT, "sigmoid_gate: unknown dtype %d", dtype);
    return check_launch("sigmoid_gate");
}
LLMB_PACKED(llmb_sigmoid_gate)

__global__ void add_terms_kernel(float* __restrict__ x, const float* __restrict__ y, int terms, int hidden, long long total) {
    griddep_launch();
    griddep_wait();
    long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    long long t = i / hidden;
    int c = (int)(i % hidden);
    float s = 0.f;
    for (int k = 0; k < terms; ++k) s += y[(t * terms + k) * hidden + c];
    x[i] += s;
}

// x[t] += sum_k y[t * terms + k] (the terms in index order)
LLMB_EXPORT int llmb_add_terms(float* x, const float* y, int terms, int n_rows, int hidden, cudaStream_t stream) {
    if (n_rows == 0) return LLMB_OK;
    LLMB_REQUIRE(terms > 0 && hidden > 0 && x && y, "add_terms: bad sizes");
    long long total = (long long)n_rows * hidden;
    LLMB_CUDA(llmb::launch(add_terms_kernel, dim3((unsigned)((total + 255) / 256)), dim3(256), 0, stream, true, x, y, terms,
                           hidden, total));
    return check_launch("add_terms");
}
LLMB_PACKED(llmb_add_terms)

__global__ void fill_kernel(float* __restrict__ x, long long n, float value) {
    griddep_launch();
    griddep_wait();
    long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) x[i] = value;
}

LLMB_EXPORT int llmb_fill(float* x, long long n, float value, cudaStream_t stream) {
    if (n == 0) return LLMB_OK;
    LLMB_REQUIRE(n > 0 && x, "fill: bad size");
    LLMB_CUDA(llmb::launch(fill_kernel, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, stream, true, x, n, value));
    return check_launch("fill");
}
LLMB_PACKED(llmb_fill)
