// A state-space recurrence with one scalar decay per head (the "state-space duality" form of
// Dao and Gu's Mamba-2 layer): per head a state S [N, V], token by token
//     S_t = exp(rate * dt_t) S_{t-1} + dt_t B_t x_t^T,      y_t = S_t^T C_t + D x_t
// with x (H heads of V), B and C (G groups of N, a group serving H / G heads) behind one causal
// convolution per channel (with bias) and silu, dt_t = softplus(. + dt_bias) per head and rate = -exp(A_log);
// y is multiplied by silu(z) and then divided by its root mean square in `norm_groups` equal parts of the
// H V channels, times a weight per channel.
//
// The projection row of a token is [z (H V) | x (H V) | B (G N) | C (G N) | dt (H) | ...] in the run's
// dtype; everything behind it is 32-bit. Per sequence the state is one 32-bit row: the convolution's last
// taps - 1 inputs [taps - 1, C] (C = H V + 2 G N channels, oldest first), then S [H, N, V].
//
// prepare     one block per token: convolution (state rows stand before the step's first token), bias, silu,
//             the step size and the decay, into a 32-bit work row [x | B | C | dt (H) | decay (H)].
// conv_state  the convolution's new last inputs; runs behind prepare, which reads the old ones.
// scan        every column of S is a recurrence of its own. A warp holds COLS columns of one head: lane l the
//             state elements n = l, l + 32, .. of each; per token it fades the state, adds dt B x, and sums
//             S C over n (a lane's elements in rising order, then the lanes as a butterfly), so a token's
//             result depends on nothing but the sequence before it. The next token's row is requested while
//             the current one is folded in. A block is four warps (4 * COLS neighbouring columns), the grid
//             (column tiles, heads, sequences).
// finish      y silu(z), the grouped norm, the weight and a scale, rounded to the run's dtype.
#include "common.cuh"

using namespace llmb;

LLMB_DEFINE_LAST_ERROR(llmb_state_space)

constexpr int THREADS = 256;
constexpr int MAX_TAPS = 16;
constexpr int SCAN_WARPS = 4;
constexpr int COLS = 4;          // columns of S a warp holds

__device__ __forceinline__ float silu(float z) { return z / (1.0f + expf(-z)); }

template <typename T>
__global__ void __launch_bounds__(THREADS)
ssm_prepare_kernel(const T* __restrict__ proj, int ld, const float* __restrict__ taps, const float* __restrict__ conv_bias,
                   int n_taps, const float* __restrict__ state, long long state_stride, const int* __restrict__ tok_seq,
                   const int* __restrict__ cu_seqlens, const int* __restrict__ slot_ids, const float* __restrict__ rate,
                   const float* __restrict__ dt_bias, float* __restrict__ work, int work_ld, int inner, int C, int H) {
    griddep_launch();
    griddep_wait();
    int t = blockIdx.x;
    int seq = tok_seq[t];
    int i = t - cu_seqlens[seq];
    const float* st = state + (long long)slot_ids[seq] * state_stride;
    const T* in = proj + inner;            // the convolved channels stand behind z
    float* out = work + (size_t)t * work_ld;
    for (int c = threadIdx.x; c < C; c += THREADS) {
        float acc = conv_bias ? conv_bias[c] : 0.f;
        for (int j = 0; j < n_taps; ++j) {
            int d = n_taps - 1 - j;
            float v = i - d >= 0 ? to_float(in[(size_t)(t - d) * ld + c]) : st[(size_t)(n_taps - 1 - (d - i)) * C + c];
            acc = fmaf(taps[(size_t)c * n_taps + j], v, acc);
        }
        out[c] = silu(acc);
    }
    const T* steps = proj + (size_t)t * ld + inner + C;
    for (int a = threadIdx.x; a < H; a += THREADS) {
        float z = to_float(steps[a]) + dt_bias[a];
        float dt = z > 20.0f ? z : log1pf(expf(z));
        out[C + a] = dt;
        out[C + H + a] = expf(rate[a] * dt);
    }
}

template <typename T>
__global__ void ssm_conv_state_kernel(const T* __restrict__ proj, int ld, int n_taps, float* __restrict__ state,
                                      long long state_stride, const int* __restrict__ cu_seqlens,
                                      const int* __restrict__ slot_ids, int inner, int C) {
    griddep_launch();
    griddep_wait();
    int c = blockIdx.x * blockDim.x + threadIdx.x, b = blockIdx.y;
    if (c >= C) return;
    int first = cu_seqlens[b], n = cu_seqlens[b + 1] - first;
    if (n <= 0) return;
    float* st = state + (long long)slot_ids[b] * state_stride;
    const T* in = proj + inner;
    float held[MAX_TAPS];
    for (int r = 0; r < n_taps - 1; ++r) {
        int src = n - (n_taps - 1) + r;
        held[r] = src >= 0 ? to_float(in[(size_t)(first + src) * ld + c]) : st[(size_t)(r + n) * C + c];
    }
    for (int r = 0; r < n_taps - 1; ++r) st[(size_t)r * C + c] = held[r];
}

// PER: state elements a lane holds of each column (N <= 32 * PER)
template <int PER>
__global__ void __launch_bounds__(SCAN_WARPS * 32)
ssm_scan_kernel(const float* __restrict__ work, int work_ld, float* __restrict__ state, long long state_stride,
                int conv_floats, const int* __restrict__ cu_seqlens, const int* __restrict__ slot_ids,
                const float* __restrict__ skip, float* __restrict__ y, int inner, int C, int H, int G, int N, int V) {
    griddep_launch();
    griddep_wait();
    int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    int head = blockIdx.y, seq = blockIdx.z;
    int v0 = (blockIdx.x * SCAN_WARPS + warp) * COLS;
    if (v0 >= V) return;
    int first = cu_seqlens[seq], n_new = cu_seqlens[seq + 1] - first;
    if (n_new <= 0) return;
    int group = head / (H / G);
    float* S = state + (long long)slot_ids[seq] * state_stride + conv_floats + (size_t)head * N * V;
    float s[PER][COLS];
#pragma unroll
    for (int i = 0; i < PER; ++i) {
        int n = lane + 32 * i;
#pragma unroll
        for (int c = 0; c < COLS; ++c) s[i][c] = (n < N && v0 + c < V) ? S[(size_t)n * V + v0 + c] : 0.f;
    }
    const int b_at = inner + group * N, c_at = inner + G * N + group * N, x_at = head * V + v0;
    float d_skip = skip ? skip[head] : 0.f;
    float nb[PER], nc[PER], nx[COLS], ndt, ndecay;
    auto fetch = [&](int t) {
        const float* row = work + (size_t)(first + t) * work_ld;
#pragma unroll
        for (int i = 0; i < PER; ++i) {
            int n = lane + 32 * i;
            nb[i] = n < N ? row[b_at + n] : 0.f;
            nc[i] = n < N ? row[c_at + n] : 0.f;
        }
#pragma unroll
        for (int c = 0; c < COLS; ++c) nx[c] = v0 + c < V ? row[x_at + c] : 0.f;
        ndt = row[C + head];
        ndecay = row[C + H + head];
    };
    fetch(0);
    for (int t = 0; t < n_new; ++t) {
        float b[PER], cc[PER], x[COLS], dt = ndt, decay = ndecay;
#pragma unroll
        for (int i = 0; i < PER; ++i) { b[i] = nb[i]; cc[i] = nc[i]; }
#pragma unroll
        for (int c = 0; c < COLS; ++c) x[c] = nx[c];
        if (t + 1 < n_new) fetch(t + 1);
        float sum[COLS];
#pragma unroll
        for (int c = 0; c < COLS; ++c) sum[c] = 0.f;
#pragma unroll
        for (int i = 0; i < PER; ++i) {
            float write = dt * b[i];
#pragma unroll
            for (int c = 0; c < COLS; ++c) {
                s[i][c] = fmaf(decay, s[i][c], write * x[c]);
                sum[c] = fmaf(s[i][c], cc[i], sum[c]);
            }
        }
#pragma unroll
        for (int c = 0; c < COLS; ++c) sum[c] = warp_sum(sum[c]);
        if (lane < COLS && v0 + lane < V) {
            float mine = sum[0], xv = x[0];
#pragma unroll
            for (int c = 1; c < COLS; ++c)
                if (lane == c) { mine = sum[c]; xv = x[c]; }
            y[(size_t)(first + t) * inner + x_at + lane] = fmaf(d_skip, xv, mine);
        }
    }
#pragma unroll
    for (int i = 0; i < PER; ++i) {
        int n = lane + 32 * i;
#pragma unroll
        for (int c = 0; c < COLS; ++c)
            if (n < N && v0 + c < V) S[(size_t)n * V + v0 + c] = s[i][c];
    }
}

// one block per token; a warp takes a part of the channels at a time
template <typename T>
__global__ void __launch_bounds__(THREADS)
ssm_finish_kernel(const float* __restrict__ y, const T* __restrict__ proj, int ld, const float* __restrict__ weight,
                  float eps, int parts, float out_scale, T* __restrict__ mixed, int mixed_ld, int inner) {
    griddep_launch();
    griddep_wait();
    int t = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    int width = inner / parts;
    const float* row = y + (size_t)t * inner;
    const T* z = proj + (size_t)t * ld;
    T* out = mixed + (size_t)t * mixed_ld;
    for (int p = warp; p < parts; p += THREADS / 32) {
        float sq = 0.f;
        for (int d = lane; d < width; d += 32) {
            int c = p * width + d;
            float v = row[c] * silu(to_float(z[c]));
            sq = fmaf(v, v, sq);
        }
        float factor = 1.0f / sqrtf(warp_sum(sq) / (float)width + eps);
        for (int d = lane; d < width; d += 32) {
            int c = p * width + d;
            float v = row[c] * silu(to_float(z[c])) * factor * weight[c];
            out[c] = from_float<T>(out_scale == 1.0f ? v : v * out_scale);
        }
    }
}

// Floats of a token's work row: [x | B | C | dt | decay], rounded up to a multiple of four.
LLMB_EXPORT int llmb_state_space_work_width(int H, int G, int N, int V) { return (H * V + 2 * G * N + 2 * H + 3) / 4 * 4; }

// proj [T, ld >= 2 H V + 2 G N + H] in `dtype`; taps float32 [C, n_taps] (the last column the current token's),
// conv_bias float32 [C] or null; state float32 [slots, state_stride >= (n_taps - 1) C + H N V]; rate, dt_bias,
// skip float32 [H] (skip may be null); weight float32 [H V]; work float32 [T, work_ld]; y float32 [T, H V];
// mixed [T, mixed_ld] in `dtype` receives the H V result columns.
LLMB_EXPORT int llmb_state_space(const void* proj, int ld, int dtype, const float* taps, const float* conv_bias,
                                 int n_taps, float* state, long long state_stride, const int* tok_seq,
                                 const int* cu_seqlens, const int* slot_ids, const float* rate, const float* dt_bias,
                                 const float* skip, const float* weight, float eps, int parts, float out_scale,
                                 float* work, int work_ld, float* y, void* mixed, int mixed_ld, int n_tokens, int n_seqs,
                                 int H, int G, int N, int V, cudaStream_t stream) {
    if (n_tokens == 0) return LLMB_OK;
    LLMB_REQUIRE(H > 0 && G > 0 && H % G == 0 && N > 0 && V > 0, "state_space: %d heads in %d groups, state %d x %d", H, G, N, V);
    LLMB_REQUIRE(N <= 256, "state_space: a state of %d rows (up to 256 are built)", N);
    LLMB_REQUIRE(n_taps >= 1 && n_taps <= MAX_TAPS, "state_space: %d taps (1 to %d are built)", n_taps, MAX_TAPS);
    int inner = H * V, C = inner + 2 * G * N;
    LLMB_REQUIRE(parts > 0 && inner % parts == 0, "state_space: %d channels in %d parts", inner, parts);
    LLMB_REQUIRE(work_ld >= C + 2 * H && ld >= inner + C + H, "state_space: rows too short");
    LLMB_REQUIRE(n_seqs > 0 && n_seqs <= 65535 && H <= 65535, "state_space: bad sizes");
    int conv_floats = (n_taps - 1) * C;
    dim3 scan_grid((V + SCAN_WARPS * COLS - 1) / (SCAN_WARPS * COLS), H, n_seqs);
#define LLMB_SSM(T)                                                                                                    \
    do {                                                                                                               \
        LLMB_CUDA(llmb::launch(ssm_prepare_kernel<T>, dim3(n_tokens), dim3(THREADS), 0, stream, true, (const T*)proj,  \
                               ld, taps, conv_bias, n_taps, (const float*)state, state_stride, tok_seq, cu_seqlens,    \
                               slot_ids, rate, dt_bias, work, work_ld, inner, C, H));                                  \
        if (n_taps > 1)                                                                                                \
            LLMB_CUDA(llmb::launch(ssm_conv_state_kernel<T>, dim3((C + 127) / 128, n_seqs), dim3(128), 0, stream, true, \
                                   (const T*)proj, ld, n_taps, state, state_stride, cu_seqlens, slot_ids, inner, C));  \
    } while (0)
    if (dtype == LLMB_DTYPE_F32) LLMB_SSM(float);
    else if (dtype == LLMB_DTYPE_BF16) LLMB_SSM(__nv_bfloat16);
    else return fail(LLMB_ERR_ARGUMENT, "state_space: unknown dtype %d", dtype);
#undef LLMB_SSM
#define LLMB_SCAN(PER)                                                                                                  \
    LLMB_CUDA(llmb::launch(ssm_scan_kernel<PER>, scan_grid, dim3(SCAN_WARPS * 32), 0, stream, true, (const float*)work, \
                           work_ld, state, state_stride, conv_floats, cu_seqlens, slot_ids, skip, y, inner, C, H, G, N, V))
    if (N <= 32) LLMB_SCAN(1);
    else if (N <= 64) LLMB_SCAN(2);
    else if (N <= 128) LLMB_SCAN(4);
    else LLMB_SCAN(8);
#undef LLMB_SCAN
    if (dtype == LLMB_DTYPE_F32)
        LLMB_CUDA(llmb::launch(ssm_finish_kernel<float>, dim3(n_tokens), dim3(THREADS), 0, stream, true, (const float*)y,
                               (const float*)proj, ld, weight, eps, parts, out_scale, (float*)mixed, mixed_ld, inner));
    else
        LLMB_CUDA(llmb::launch(ssm_finish_kernel<__nv_bfloat16>, dim3(n_tokens), dim3(THREADS), 0, stream, true,
                               (const float*)y, (const __nv_bfloat16*)proj, ld, weight, eps, parts, out_scale,
                               (__nv_bfloat16*)mixed, mixed_ld, inner));
    return check_launch("state_space");
}
LLMB_PACKED(llmb_state_space)
