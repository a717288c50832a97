// The gated delta rule: a linear recurrence whose state is one matrix M [dim, vdim] per head (S in the code),
//     M_t = a_t M_{t-1} + k_t w_t^T,   w_t = b_t (v_t - a_t M_{t-1}^T k_t),   o_t = M_t^T q_t
// (the state fades by a_t, then the row w_t is written under the key k_t: what the state already holds under that key is
// taken off first; the read-out sees the token's own write),
// behind short causal convolutions (with silu) on the q, k and v projections, unit-length q and k,
// a sigmoid step size b_t and a decay a_t = exp(rate * softplus(. + dt_bias)) per head, and in front of
// a head-wise RMS norm with a silu gate.
//
// The projection row of a token is [q (G*D) | k (G*D) | v (H*V) | gate (H*V) | b (H) | a (H) | ...]
// in the run's dtype; everything behind it is 32-bit. Per sequence the state is one 32-bit row:
// the convolution's last taps - 1 inputs [taps - 1, C] (C = 2 G D + H V, oldest first), then S [H, D, V].
//
// prepare  one block per token: convolution (state rows stand before the step's first token), silu,
//          unit norms, beta, decay and k.q, into a 32-bit work row [qn | kn | v | beta | decay | kq (G)].
// conv_state  the convolution's new last inputs; runs behind prepare, which reads the old ones.
// scan     one block per (columns of S, head, sequence) walks the sequence's tokens in order. Every
//          column of S is a recurrence of its own: a thread holds 16 elements of two columns, DS threads
//          a pair of columns; the two sums over dim use the state before the decay
//          (o_t = a_t M_{t-1}^T q_t + w_t (k_t . q_t), and M_{t-1}^T k_t is summed before the decay), so both
//          run as independent chains and are added over the DS threads by shuffles. Tokens are
//          staged in shared memory eight at a time, the next eight requested under the current.
// finish   o / sqrt(mean(o^2) + eps) * weight * silu(gate) per head, rounded to the run's dtype.
#include "common.cuh"

using namespace llmb;

LLMB_DEFINE_LAST_ERROR(llmb_delta_rule)

constexpr int THREADS = 256;
constexpr int MAX_TAPS = 16;
constexpr int CHUNK = 16;        // tokens staged at a time

__device__ __forceinline__ float silu(float z) { return z / (1.0f + expf(-z)); }

template <typename T>
__global__ void __launch_bounds__(THREADS)
delta_prepare_kernel(const T* __restrict__ proj, int ld, const float* __restrict__ taps, int n_taps,
                     const float* __restrict__ state, long long state_stride, const int* __restrict__ tok_seq,
                     const int* __restrict__ cu_seqlens, const int* __restrict__ slot_ids,
                     const float* __restrict__ rate, const float* __restrict__ dt_bias, float unit_eps,
                     float* __restrict__ work, int work_ld, int H, int G, int D, int V) {
    extern __shared__ float row[];         // [C]
    griddep_launch();
    griddep_wait();
    int t = blockIdx.x;
    int seq = tok_seq[t];
    int i = t - cu_seqlens[seq];
    const float* st = state + (long long)slot_ids[seq] * state_stride;
    int GD = G * D, C = 2 * GD + H * V;
    for (int c = threadIdx.x; c < C; c += THREADS) {
        float acc = 0.f;
        for (int j = 0; j < n_taps; ++j) {
            int d = n_taps - 1 - j;
            float in = i - d >= 0 ? to_float(proj[(size_t)(t - d) * ld + c]) : st[(size_t)(n_taps - 1 - (d - i)) * C + c];
            acc = fmaf(taps[(size_t)c * n_taps + j], in, acc);
        }
        row[c] = silu(acc);
    }
    __syncthreads();
    float* out = work + (size_t)t * work_ld;
    int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (int g = warp; g < G; g += THREADS / 32) {
        float sq = 0.f, sk = 0.f;
        for (int d = lane; d < D; d += 32) {
            float a = row[g * D + d], b = row[GD + g * D + d];
            sq = fmaf(a, a, sq);
            sk = fmaf(b, b, sk);
        }
        float rq = 1.0f / sqrtf(warp_sum(sq) + unit_eps) * (1.0f / sqrtf((float)D));
        float rk = 1.0f / sqrtf(warp_sum(sk) + unit_eps);
        float dot = 0.f;
        for (int d = lane; d < D; d += 32) {
            float a = row[g * D + d] * rq, b = row[GD + g * D + d] * rk;
            out[g * D + d] = a;
            out[GD + g * D + d] = b;
            dot = fmaf(a, b, dot);
        }
        dot = warp_sum(dot);
        if (lane == 0) out[C + 2 * H + g] = dot;
    }
    for (int e = threadIdx.x; e < H * V; e += THREADS) out[2 * GD + e] = row[2 * GD + e];
    const T* in = proj + (size_t)t * ld + 2 * GD + 2 * H * V;
    for (int a = threadIdx.x; a < H; a += THREADS) {
        float b = to_float(in[a]);
        out[C + a] = 1.0f / (1.0f + expf(-b));
        float z = to_float(in[H + a]) + dt_bias[a];
        float sp = z > 20.0f ? z : log1pf(expf(z));
        out[C + H + a] = expf(rate[a] * sp);
    }
}

template <typename T>
__global__ void delta_conv_state_kernel(const T* __restrict__ proj, int ld, int n_taps, float* __restrict__ state,
                                        long long state_stride, const int* __restrict__ cu_seqlens,
                                        const int* __restrict__ slot_ids, int C) {
    griddep_launch();
    griddep_wait();
    int c = blockIdx.x * blockDim.x + threadIdx.x, b = blockIdx.y;
    if (c >= C) return;
    int first = cu_seqlens[b], n = cu_seqlens[b + 1] - first;
    if (n <= 0) return;
    float* st = state + (long long)slot_ids[b] * state_stride;
    float held[MAX_TAPS];
    for (int r = 0; r < n_taps - 1; ++r) {
        int src = n - (n_taps - 1) + r;
        held[r] = src >= 0 ? to_float(proj[(size_t)(first + src) * ld + c]) : st[(size_t)(r + n) * C + c];
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

// two 32-bit floats in one 64-bit register and the packed arithmetic on them (each half rounded as the scalar form)
typedef unsigned long long pair_t;
__device__ __forceinline__ pair_t pack2(float lo, float hi) {
    pair_t r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
    return r;
}
__device__ __forceinline__ void unpack2(pair_t v, float& lo, float& hi) { asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v)); }
__device__ __forceinline__ pair_t fma2(pair_t a, pair_t b, pair_t c) {
    pair_t d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
    return d;
}
__device__ __forceinline__ pair_t mul2(pair_t a, pair_t b) {
    pair_t d;
    asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}

constexpr int SCAN_THREADS = 128;
constexpr int NC = 2;            // columns of S a thread holds
constexpr int PAD = 4;           // floats between the slices of a staged q or k: a quarter warp's 16-byte loads fall into
                                 // different banks

// DS threads share a pair of columns (DS a power of two up to 32), each DPT elements of both: lanes that follow each
// other hold neighbouring column pairs of the same slice (their loads of q and k are one address), lanes 32 / DS
// apart the slices. A step is a chain of dependent instructions (sums, shuffles, the update), so what counts is how
// many warps a scheduler can turn to: DPT = 8 gives twice the warps of 16 for the same state.
template <int DPT, int DS>
__global__ void __launch_bounds__(SCAN_THREADS)
delta_scan_kernel(const float* __restrict__ work, int work_ld, float* __restrict__ state, long long state_stride,
                  long long s_offset, const int* __restrict__ cu_seqlens, const int* __restrict__ slot_ids,
                  float* __restrict__ out, int out_ld, int H, int G, int D, int V, int vectors) {
    extern __shared__ __align__(16) float stage[];   // two buffers of [CHUNK] x (q [DS][DPT + PAD] | k likewise | v [VC] | beta, decay, kq, -)
    griddep_launch();
    int a = blockIdx.y, b = blockIdx.z;
    int g = a / (H / G);
    constexpr int pairs_per_warp = 32 / DS;
    constexpr int VC = (SCAN_THREADS / DS) * NC;
    int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    int slice = lane / pairs_per_warp;
    int local_col = (warp * pairs_per_warp + lane % pairs_per_warp) * NC;
    int col = blockIdx.x * VC + local_col;
    constexpr int Dq = DS * (DPT + PAD);
    constexpr int per_token = 2 * Dq + VC + 4, buffer = CHUNK * per_token;
    int GD = G * D, C = 2 * GD + H * V;
    griddep_wait();
    int first = cu_seqlens[b], n = cu_seqlens[b + 1] - first;
    if (n <= 0) return;
    float* S_global = state + (long long)slot_ids[b] * state_stride + s_offset + (size_t)a * D * V;
    bool two = (V % 2 == 0) && ((reinterpret_cast<uintptr_t>(S_global) & 7) == 0) && col + 1 < V;
    float S[NC][DPT];
#pragma unroll
    for (int e = 0; e < DPT; ++e) {
        int d = slice * DPT + e;
        if (two && d < D) {
            float2 pair = *reinterpret_cast<const float2*>(S_global + (size_t)d * V + col);
            S[0][e] = pair.x;
            S[1][e] = pair.y;
        } else {
#pragma unroll
            for (int c = 0; c < NC; ++c) S[c][e] = (d < D && col + c < V) ? S_global[(size_t)d * V + col + c] : 0.f;
        }
    }
    // neighbouring elements of a column share a register pair: the sums and the update run as packed multiply-adds
    pair_t S2[NC][DPT / 2];
#pragma unroll
    for (int c = 0; c < NC; ++c)
#pragma unroll
        for (int p2 = 0; p2 < DPT / 2; ++p2) S2[c][p2] = pack2(S[c][2 * p2], S[c][2 * p2 + 1]);
    // the padding of q and k (between slices and beyond D) stays zero in both buffers
    for (int i = threadIdx.x; i < 2 * buffer; i += SCAN_THREADS) stage[i] = 0.f;
    __syncthreads();
    auto request = [&](int chunk, float* buf) {
        int base = chunk * CHUNK;
        int count = min(CHUNK, n - base);
        for (int tt = warp; tt < count; tt += SCAN_THREADS / 32) {          // a warp a token
            const float* src = work + (size_t)(first + base + tt) * work_ld;
            float* dst = buf + tt * per_token;
            if (vectors) {
                // 16 bytes a copy: D, V and the row's length are multiples of 4, so no copy straddles a slice's or D's end
                int qk = D / 4, vs = min(VC, V - (int)blockIdx.x * VC) / 4;
                for (int i = lane; i < 2 * qk + vs; i += 32) {
                    if (i < 2 * qk) {
                        int which = i >= qk, e = (i - which * qk) * 4;
                        copy16(dst + which * Dq + (e / DPT) * (DPT + PAD) + e % DPT, src + which * GD + g * D + e);
                    } else {
                        int j = (i - 2 * qk) * 4;
                        copy16(dst + 2 * Dq + j, src + 2 * GD + a * V + blockIdx.x * VC + j);
                    }
                }
            } else {
                for (int e = lane; e < 2 * D + VC; e += 32) {
                    if (e < 2 * D) {
                        int which = e >= D, d = e - which * D;
                        copy4(dst + which * Dq + (d / DPT) * (DPT + PAD) + d % DPT, src + which * GD + g * D + d);
                    } else {
                        int j = blockIdx.x * VC + (e - 2 * D);
                        if (j < V) copy4(dst + 2 * Dq + (e - 2 * D), src + 2 * GD + a * V + j);
                    }
                }
            }
            if (lane < 3) {
                int at = lane == 0 ? C + a : (lane == 1 ? C + H + a : C + 2 * H + g);
                copy4(dst + 2 * Dq + VC + lane, src + at);
            }
        }
        asm volatile("cp.async.commit_group;\n" ::);
    };
    int n_chunks = (n + CHUNK - 1) / CHUNK;
    request(0, stage);
    for (int chunk = 0; chunk < n_chunks; ++chunk) {
        float* buf = stage + (chunk & 1) * buffer;
        if (chunk + 1 < n_chunks) {
            request(chunk + 1, stage + ((chunk + 1) & 1) * buffer);
            asm volatile("cp.async.wait_group 1;\n" ::);
        } else {
            asm volatile("cp.async.wait_group 0;\n" ::);
        }
        __syncthreads();
        int count = min(CHUNK, n - chunk * CHUNK);
        for (int tt = 0; tt < count; ++tt) {
            const float* tok = buf + tt * per_token;
            const float4* q4 = reinterpret_cast<const float4*>(tok + slice * (DPT + PAD));
            const float4* k4 = reinterpret_cast<const float4*>(tok + Dq + slice * (DPT + PAD));
            pair_t kp[DPT / 2];
            pair_t sk[NC][2], sq[NC][2];               // two chains of pairs a sum: a quarter of the latency of one chain
#pragma unroll
            for (int c = 0; c < NC; ++c) { sk[c][0] = sk[c][1] = sq[c][0] = sq[c][1] = 0ull; }
#pragma unroll
            for (int e = 0; e < DPT / 4; ++e) {
                float4 kv = k4[e], qv = q4[e];
                pair_t k01 = pack2(kv.x, kv.y), k23 = pack2(kv.z, kv.w), q01 = pack2(qv.x, qv.y), q23 = pack2(qv.z, qv.w);
                kp[2 * e] = k01;
                kp[2 * e + 1] = k23;
#pragma unroll
                for (int c = 0; c < NC; ++c) {
                    sk[c][0] = fma2(S2[c][2 * e], k01, sk[c][0]); sq[c][0] = fma2(S2[c][2 * e], q01, sq[c][0]);
                    sk[c][1] = fma2(S2[c][2 * e + 1], k23, sk[c][1]); sq[c][1] = fma2(S2[c][2 * e + 1], q23, sq[c][1]);
                }
            }
            float tk[NC], tq[NC];
#pragma unroll
            for (int c = 0; c < NC; ++c) {
                float a0, a1, a2, a3;
                unpack2(sk[c][0], a0, a1);
                unpack2(sk[c][1], a2, a3);
                tk[c] = (a0 + a1) + (a2 + a3);
                unpack2(sq[c][0], a0, a1);
                unpack2(sq[c][1], a2, a3);
                tq[c] = (a0 + a1) + (a2 + a3);
            }
#pragma unroll
            for (int offset = 16; offset >= pairs_per_warp; offset >>= 1) {
#pragma unroll
                for (int c = 0; c < NC; ++c) {
                    tk[c] += __shfl_xor_sync(0xffffffffu, tk[c], offset);
                    tq[c] += __shfl_xor_sync(0xffffffffu, tq[c], offset);
                }
            }
            float2 v = *reinterpret_cast<const float2*>(tok + 2 * Dq + local_col);
            float beta = tok[2 * Dq + VC], decay = tok[2 * Dq + VC + 1], kq = tok[2 * Dq + VC + 2];
            float u[NC], o[NC];
            u[0] = beta * (v.x - decay * tk[0]);
            u[1] = beta * (v.y - decay * tk[1]);
#pragma unroll
            for (int c = 0; c < NC; ++c) {
                o[c] = fmaf(u[c], kq, decay * tq[c]);
                pair_t u2 = pack2(u[c], u[c]), d2 = pack2(decay, decay);
#pragma unroll
                for (int p2 = 0; p2 < DPT / 2; ++p2) S2[c][p2] = fma2(kp[p2], u2, mul2(d2, S2[c][p2]));
            }
            if (slice == 0) {
                float* dst = out + (size_t)(first + chunk * CHUNK + tt) * out_ld + a * V + col;
                if (two && (out_ld % 2 == 0) && ((reinterpret_cast<uintptr_t>(out) & 7) == 0)) *reinterpret_cast<float2*>(dst) = make_float2(o[0], o[1]);
                else {
#pragma unroll
                    for (int c = 0; c < NC; ++c)
                        if (col + c < V) dst[c] = o[c];
                }
            }
        }
        __syncthreads();
    }
#pragma unroll
    for (int c = 0; c < NC; ++c)
#pragma unroll
        for (int p2 = 0; p2 < DPT / 2; ++p2) unpack2(S2[c][p2], S[c][2 * p2], S[c][2 * p2 + 1]);
#pragma unroll
    for (int e = 0; e < DPT; ++e) {
        int d = slice * DPT + e;
        if (two && d < D) {
            *reinterpret_cast<float2*>(S_global + (size_t)d * V + col) = make_float2(S[0][e], S[1][e]);
        } else {
#pragma unroll
            for (int c = 0; c < NC; ++c)
                if (d < D && col + c < V) S_global[(size_t)d * V + col + c] = S[c][e];
        }
    }
}

template <typename T>
__global__ void __launch_bounds__(THREADS)
delta_finish_kernel(const float* __restrict__ o, int o_ld, const T* __restrict__ gate, int gate_ld,
                    const float* __restrict__ weight, float eps, T* __restrict__ mixed, int mixed_ld, int H, int V) {
    griddep_launch();
    griddep_wait();
    size_t t = blockIdx.x;
    int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (int a = warp; a < H; a += THREADS / 32) {
        const float* row = o + t * o_ld + a * V;
        float sq = 0.f;
        for (int j = lane; j < V; j += 32) sq = fmaf(row[j], row[j], sq);
        float rstd = 1.0f / sqrtf(warp_sum(sq) / (float)V + eps);
        for (int j = lane; j < V; j += 32) {
            float z = to_float(gate[t * gate_ld + a * V + j]);
            mixed[t * mixed_ld + a * V + j] = from_float<T>(row[j] * rstd * weight[j] * silu(z));
        }
    }
}

// proj [T, ld] in `dtype`; taps float32 [C, n_taps]; state float32 [slots, state_stride] (conv rows, then S);
// work float32 [T, work_ld >= C + 2 H + G]; o float32 [T, H V]; mixed [T, mixed_ld] in `dtype`.
LLMB_EXPORT int llmb_delta_rule(const void* proj, int ld, int dtype, const float* taps, int n_taps, float* state,
                                long long state_stride, const int* tok_seq, const int* cu_seqlens, const int* slot_ids,
                                const float* rate, const float* dt_bias, float unit_eps, const float* norm_weight,
                                float eps, float* work, int work_ld, float* o, void* mixed, int mixed_ld, int n_tokens,
                                int n_seqs, int H, int G, int D, int V, cudaStream_t stream) {
    if (n_tokens == 0) return LLMB_OK;
    LLMB_REQUIRE(H > 0 && G > 0 && H % G == 0 && D > 0 && V > 0, "delta_rule: bad head sizes %d / %d / %d / %d", H, G, D, V);
    LLMB_REQUIRE(n_taps >= 1 && n_taps <= MAX_TAPS, "delta_rule: %d taps (1 to %d are built)", n_taps, MAX_TAPS);
    LLMB_REQUIRE(D <= 32 * 16, "delta_rule: a key size of %d (up to %d is built)", D, 32 * 16);
    // a long slice per thread (few shuffle levels, long runs of independent products) from a key size of 64 on
    int DPT = D >= 64 ? 32 : 8;
    int C = 2 * G * D + H * V;
    LLMB_REQUIRE(ld >= C + H * V + 2 * H && work_ld >= C + 2 * H + G, "delta_rule: rows too narrow");
    LLMB_REQUIRE(state_stride >= (long long)(n_taps - 1) * C + (long long)H * D * V, "delta_rule: state too small");
    LLMB_REQUIRE(((size_t)work % 4) == 0, "delta_rule: misaligned work rows");
    int DS = DPT == 32 ? 2 : 1;
    while (DS * DPT < D) DS *= 2;
    int VC = (SCAN_THREADS / DS) * NC;
    size_t smem_row = sizeof(float) * (size_t)C;
    size_t smem_scan = sizeof(float) * 2 * CHUNK * (size_t)(2 * DS * (DPT + PAD) + VC + 4);
    // 16-byte copies of a token's q, k and v into the scan's stage: every piece starts on a multiple of 4 floats
    int vectors = D % 4 == 0 && V % 4 == 0 && work_ld % 4 == 0 && ((size_t)work % 16) == 0 && (V % VC == 0 || V < VC);
    LLMB_REQUIRE(smem_row <= 200 * 1024, "delta_rule: a row of %d channels does not fit in shared memory", C);
    dim3 scan_grid((V + VC - 1) / VC, H, n_seqs);
    typedef void (*Scan)(const float*, int, float*, long long, long long, const int*, const int*, float*, int, int, int, int, int, int);
    Scan scan = nullptr;
    if (DPT == 8) scan = DS == 1 ? delta_scan_kernel<8, 1> : DS == 2 ? delta_scan_kernel<8, 2> : DS == 4 ? delta_scan_kernel<8, 4> : delta_scan_kernel<8, 8>;
    else scan = DS == 2 ? delta_scan_kernel<32, 2> : DS == 4 ? delta_scan_kernel<32, 4> : DS == 8 ? delta_scan_kernel<32, 8> : delta_scan_kernel<32, 16>;
    static size_t scan_configured[2][6] = {};
    int level = DS == 1 ? 0 : DS == 2 ? 1 : DS == 4 ? 2 : DS == 8 ? 3 : DS == 16 ? 4 : 5;
    if (smem_scan > 48 * 1024 && smem_scan > scan_configured[DPT == 32][level]) {
        LLMB_CUDA(cudaFuncSetAttribute(scan, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_scan));
        scan_configured[DPT == 32][level] = smem_scan;
    }
    long long s_offset = (long long)(n_taps - 1) * C;
#define LLMB_DELTA(T)                                                                                              \
    do {                                                                                                           \
        if (smem_row > 48 * 1024)                                                                                  \
            LLMB_CUDA(cudaFuncSetAttribute(delta_prepare_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize,   \
                                           (int)smem_row));                                                        \
        LLMB_CUDA(llmb::launch(delta_prepare_kernel<T>, dim3(n_tokens), dim3(THREADS), smem_row, stream, true,     \
                               (const T*)proj, ld, taps, n_taps, (const float*)state, state_stride, tok_seq,       \
                               cu_seqlens, slot_ids, rate, dt_bias, unit_eps, work, work_ld, H, G, D, V));         \
        if (n_taps > 1)                                                                                            \
            LLMB_CUDA(llmb::launch(delta_conv_state_kernel<T>, dim3((C + 127) / 128, n_seqs), dim3(128), 0, stream, \
                                   true, (const T*)proj, ld, n_taps, state, state_stride, cu_seqlens, slot_ids, C)); \
        LLMB_CUDA(llmb::launch(scan, scan_grid, dim3(SCAN_THREADS), smem_scan, stream, true,                       \
                               (const float*)work, work_ld, state, state_stride, s_offset, cu_seqlens, slot_ids,  \
                               o, H * V, H, G, D, V, vectors));                                                    \
        LLMB_CUDA(llmb::launch(delta_finish_kernel<T>, dim3(n_tokens), dim3(THREADS), 0, stream, true,             \
                               (const float*)o, H * V, (const T*)proj + C, ld, norm_weight, eps, (T*)mixed,        \
                               mixed_ld, H, V));                                                                   \
    } while (0)
    if (dtype == LLMB_DTYPE_F32) LLMB_DELTA(float);
    else if (dtype == LLMB_DTYPE_BF16) LLMB_DELTA(__nv_bfloat16);
    else return fail(LLMB_ERR_ARGUMENT, "delta_rule: unknown dtype %d", dtype);
#undef LLMB_DELTA
    return check_launch("delta_rule");
}
LLMB_PACKED(llmb_delta_rule)

// launches of one call (for the caller's count)
LLMB_EXPORT int llmb_delta_rule_launches(int n_taps) { return n_taps > 1 ? 4 : 3; }
