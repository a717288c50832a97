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
// taps - 1 inputs [taps - 1, C] (C = H V + 2 G N channels, oldest first), then S [H, V, N] (a column of a head's
// state, the N rows that one value element reads, is contiguous).
//
// prepare     one block per token: convolution (state rows stand before the step's first token), bias, silu,
//             the step size and the decay, into a 32-bit work row [x | B | C | dt (H) | decay (H)].
// conv_state  the convolution's new last inputs; runs behind prepare, which reads the old ones.
// scan        every column of S is a recurrence of its own. A warp holds COLS columns of one head: lane l the
//             state rows n = l, l + 32, .. of each; per token it fades the state, adds dt B x, and sums
//             S C over n (a lane's rows in rising order, then the lanes as a butterfly), so a token's
//             result depends on nothing but the sequence before it. Tokens are staged in shared memory a
//             chunk at a time, the next chunk requested under the current, and the partial sums of several
//             tokens meet in one butterfly. A block holds 32 neighbouring columns, the grid is
//             (column tiles, heads, sequences).
// finish      y silu(z), the grouped norm, the weight and a scale, rounded to the run's dtype.
#include "common.cuh"

using namespace llmb;

LLMB_DEFINE_LAST_ERROR(llmb_state_space)

constexpr int THREADS = 256;
constexpr int MAX_TAPS = 16;

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

__device__ __forceinline__ void copy4(float* smem, const float* global) {
    unsigned s = (unsigned)__cvta_generic_to_shared(smem);
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;\n" ::"r"(s), "l"(global));
}
__device__ __forceinline__ void copy16(float* smem, const float* global) {
    unsigned s = (unsigned)__cvta_generic_to_shared(smem);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(s), "l"(global));
}
__device__ __forceinline__ void copies_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int LEFT> __device__ __forceinline__ void copies_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(LEFT)); }

// One level of a butterfly over COUNT values a lane: lanes whose bit OFFSET is set keep the upper half of the
// values and hand over the lower half, the others the reverse; what stays is own + partner's. After the
// levels 16, 8, 4, 2, 1 on 32 values lane l holds the sum over all lanes of value l. Every value's sum runs through
// the same tree of lane pairs (l, l ^ 16), then (l, l ^ 8), ..., whatever its index: a sum does not depend on the
// place of its token in a group.
template <int COUNT, int OFFSET>
__device__ __forceinline__ void fold(float (&v)[32], int lane) {
    bool up = (lane & OFFSET) != 0;
#pragma unroll
    for (int k = 0; k < COUNT; ++k) {
        float send = up ? v[k] : v[COUNT + k];
        float keep = up ? v[COUNT + k] : v[k];
        v[k] = keep + __shfl_xor_sync(0xffffffffu, send, OFFSET);
    }
}

// PER: state rows a lane holds of each column (N <= 32 * PER). A block: WARPS warps of COLS columns each, the
// columns [blockIdx.x * TILE, + TILE) of head blockIdx.y for sequence blockIdx.z. Tokens are staged in shared memory
// a chunk at a time (the group's B and C rows, the tile's x, the head's step size and decay), the next chunk requested
// under the current; a warp folds GROUP = 32 / COLS tokens into its columns, keeps the 32 partial sums of S C a lane,
// and adds them over the lanes with one butterfly for all of them. Steps of many tokens run few columns a warp and
// many warps (the chain from token to token is short, so what counts is how many warps an SM has to choose from);
// steps of one token a sequence run many columns a warp (the butterfly is paid once a warp). A token's sums are
// the same bits either way: a lane holds the same rows, and the lanes meet in the same order.
template <int PER, int COLS, int WARPS>
__global__ void __launch_bounds__(WARPS * 32)
ssm_scan_kernel(const float* __restrict__ work, int work_ld, float* __restrict__ state, long long state_stride,
                int conv_floats, const int* __restrict__ cu_seqlens, const int* __restrict__ slot_ids,
                const float* __restrict__ skip, float* __restrict__ y, int inner, int C, int H, int G, int N, int V,
                int vectors) {
    constexpr int TILE = WARPS * COLS;         // columns a block holds
    constexpr int GROUP = 32 / COLS;           // tokens whose partial sums meet in one butterfly
    constexpr int CHUNK = GROUP > 8 ? GROUP : 8;   // tokens staged at a time
    extern __shared__ float staged[];      // [2][CHUNK][row]: B (N) | C (N) | x (TILE) | dt | decay
    griddep_launch();
    griddep_wait();
    int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    int head = blockIdx.y, seq = blockIdx.z;
    int tile0 = blockIdx.x * TILE, v0 = tile0 + warp * COLS;
    int first = cu_seqlens[seq], n_new = cu_seqlens[seq + 1] - first;
    if (n_new <= 0) return;
    int group = head / (H / G);
    const int row = 2 * N + TILE + 4;      // (dt, decay and two floats that keep every row on a 16-byte boundary)
    const int b_at = inner + group * N, c_at = inner + G * N + group * N, x_at = head * V + tile0;
    float* S = state + (long long)slot_ids[seq] * state_stride + conv_floats + (size_t)head * N * V;   // [V, N]
    float s[PER][COLS];
#pragma unroll
    for (int i = 0; i < PER; ++i) {
        int n = lane + 32 * i;
#pragma unroll
        for (int c = 0; c < COLS; ++c) s[i][c] = (n < N && v0 + c < V) ? S[(size_t)(v0 + c) * N + n] : 0.f;
    }
    float d_skip = skip ? skip[head] : 0.f;
    auto request = [&](int chunk) {
        float* to = staged + (chunk & 1) * CHUNK * row;
        int t0 = chunk * CHUNK, count = min(CHUNK, n_new - t0);
        if (vectors) {
            // 16 bytes a copy (sizes, strides and addresses allow it): a copy of 4 bytes a lane costs the load unit as
            // much as one of 16; one token a warp at a time
            const int quads = (2 * N + TILE) / 4;
            for (int t = warp; t < count; t += WARPS) {
                const float* from = work + (size_t)(first + t0 + t) * work_ld;
                float* row_to = to + t * row;
                for (int q = lane; q < quads; q += 32) {
                    int r = 4 * q;
                    if (r < 2 * N) copy16(row_to + r, from + (r < N ? b_at + r : c_at + r - N));
                    else if (tile0 + r - 2 * N < V) copy16(row_to + r, from + x_at + r - 2 * N);
                }
                if (lane < 2) copy4(row_to + 2 * N + TILE + lane, from + C + lane * H + head);          // dt, then decay
            }
        } else {
            for (int t = 0; t < count; ++t) {
                const float* from = work + (size_t)(first + t0 + t) * work_ld;
                float* row_to = to + t * row;
                for (int r = threadIdx.x; r < 2 * N; r += WARPS * 32)
                    copy4(row_to + r, from + (r < N ? b_at + r : c_at + r - N));
                if (threadIdx.x < TILE) { if (tile0 + threadIdx.x < V) copy4(row_to + 2 * N + threadIdx.x, from + x_at + threadIdx.x); }
                else if (threadIdx.x < TILE + 2) copy4(row_to + 2 * N + threadIdx.x, from + C + (threadIdx.x - TILE) * H + head);
            }
        }
        copies_commit();
    };
    // one token of a group: fade, write, and the lane's share of S C for each column
    auto token = [&](const float* tok, float (&sums)[32], int j, bool live) {
        float dt = live ? tok[2 * N + TILE] : 0.f, decay = live ? tok[2 * N + TILE + 1] : 1.f;
        float x[COLS];                     // times the step size
#pragma unroll
        for (int c = 0; c < COLS; ++c) x[c] = (live && v0 + c < V) ? dt * tok[2 * N + warp * COLS + c] : 0.f;
#pragma unroll
        for (int c = 0; c < COLS; ++c) sums[j * COLS + c] = 0.f;
#pragma unroll
        for (int i = 0; i < PER; ++i) {
            int n = lane + 32 * i;
            float b = (live && n < N) ? tok[n] : 0.f, cc = (live && n < N) ? tok[N + n] : 0.f;
#pragma unroll
            for (int c = 0; c < COLS; ++c) {
                s[i][c] = fmaf(decay, s[i][c], b * x[c]);           // (a token beyond the step: decay 1, nothing written)
                sums[j * COLS + c] = fmaf(s[i][c], cc, sums[j * COLS + c]);
            }
        }
    };
    int n_chunks = (n_new + CHUNK - 1) / CHUNK;
    request(0);
    for (int chunk = 0; chunk < n_chunks; ++chunk) {
        if (chunk + 1 < n_chunks) { request(chunk + 1); copies_wait<1>(); }
        else copies_wait<0>();
        __syncthreads();
        const float* from = staged + (chunk & 1) * CHUNK * row;
        int t0 = chunk * CHUNK, count = min(CHUNK, n_new - t0);
        for (int g0 = 0; g0 < count; g0 += GROUP) {
            float sums[32];
            if (g0 + GROUP <= count) {
#pragma unroll
                for (int j = 0; j < GROUP; ++j) token(from + (g0 + j) * row, sums, j, true);
            } else {
#pragma unroll
                for (int j = 0; j < GROUP; ++j) token(from + (g0 + j) * row, sums, j, g0 + j < count);
            }
            fold<16, 16>(sums, lane);
            fold<8, 8>(sums, lane);
            fold<4, 4>(sums, lane);
            fold<2, 2>(sums, lane);
            fold<1, 1>(sums, lane);
            int j = lane / COLS, c = lane % COLS;           // lane l holds token l / COLS, column l % COLS of the group
            if (g0 + j < count && v0 + c < V) {
                float xv = from[(g0 + j) * row + 2 * N + warp * COLS + c];
                y[(size_t)(first + t0 + g0 + j) * inner + head * V + v0 + c] = fmaf(d_skip, xv, sums[0]);
            }
        }
        __syncthreads();                   // the stage is requested again two chunks on
    }
#pragma unroll
    for (int i = 0; i < PER; ++i) {
        int n = lane + 32 * i;
#pragma unroll
        for (int c = 0; c < COLS; ++c)
            if (n < N && v0 + c < V) S[(size_t)(v0 + c) * N + n] = s[i][c];
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
// conv_bias float32 [C] or null; state float32 [slots, state_stride >= (n_taps - 1) C + H V N]; rate, dt_bias,
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
    // steps of one token a sequence: 8 columns a warp, 4 warps; steps with more tokens: 2 columns a warp, 16 warps
    bool single = n_tokens <= n_seqs;
    int cols = single ? 8 : 2, warps = single ? 4 : 16;
    int tile = warps * cols, chunk = 32 / cols > 8 ? 32 / cols : 8;
    dim3 scan_grid((V + tile - 1) / tile, H, n_seqs);
    size_t scan_smem = sizeof(float) * 2 * chunk * (2 * N + tile + 4);
    int vectors = N % 4 == 0 && V % 4 == 0 && work_ld % 4 == 0 && ((size_t)work % 16) == 0;
#define LLMB_SCAN_AS(PER, COLS, WARPS)                                                                                   \
    do {                                                                                                                 \
        if (scan_smem > 48 * 1024)                                                                                       \
            LLMB_CUDA(cudaFuncSetAttribute(ssm_scan_kernel<PER, COLS, WARPS>, cudaFuncAttributeMaxDynamicSharedMemorySize, \
                                           (int)scan_smem));                                                             \
        LLMB_CUDA(llmb::launch(ssm_scan_kernel<PER, COLS, WARPS>, scan_grid, dim3(WARPS * 32), scan_smem, stream, true,  \
                               (const float*)work, work_ld, state, state_stride, conv_floats, cu_seqlens, slot_ids, skip, \
                               y, inner, C, H, G, N, V, vectors));                                                       \
    } while (0)
#define LLMB_SCAN(PER)                                     \
    do {                                                   \
        if (single) LLMB_SCAN_AS(PER, 8, 4);               \
        else LLMB_SCAN_AS(PER, 2, 16);                     \
    } while (0)
    if (N <= 32) LLMB_SCAN(1);
    else if (N <= 64) LLMB_SCAN(2);
    else if (N <= 128) LLMB_SCAN(4);
    else LLMB_SCAN(8);
#undef LLMB_SCAN
#undef LLMB_SCAN_AS
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
