// A feed-forward of routed experts: every token is sent to the `top` experts with the largest router
// logits, its result is the sum of their results weighted by the softmax over the chosen logits.
//
// router   logits = W_r h + b in 32-bit (W_r and b are held in 32-bit; h is the normed input in the run's
//          dtype), the `top` largest (the lower index wins a tie), softmax over them. One block of 16 warps per token (a warp an
//          expert at a time), or, for steps of 512 tokens and more, four warps per four tokens (a weight row is
//          fetched once for the four). An
//          assignment is a pair (token, k): index t * top + k.
//          `scoring` 1 instead: scores s = softmax over ALL router outputs; the `top` largest of s + correction are
//          chosen (the correction takes part in the choice only), weights s / (sum of the chosen s + 1e-20). The
//          router may have more outputs than there are experts: the last ones are pass-through experts without
//          matrices whose result is the token's own row h (times the weight); a small kernel writes those rows,
//          the plan and the products see only the assignments of experts that have matrices.
//          `weight_scale` multiplies every weight (a constant in front of the whole feed-forward).
// plan     counts the assignments of every expert, lists them grouped by expert (inside an expert in rising
//          order, so the plan is a function of the routing alone) and cuts every expert's list into tiles of 32
//          (or, for the tcgen05 products, 128) rows: (expert, first row, rows) per tile. Nothing of this reaches
//          the host: the product kernels are launched with the largest possible tile count and blocks beyond the
//          plan's count leave at once, so a step can be captured and replayed.
// up       for every tile: act[s, :] = silu(W_gate,e h_t) * (W_up,e h_t) for the rows s of the sorted list
//          (h_t gathered through the list), one weight matrix [2 F, K] per expert (gate rows, then up).
// down     for every tile: y[t * top + k, :] = weight[t, k] * (W_down,e act[s, :]), 32-bit, written at the
//          assignment's own index; the sum over k is taken by the kernel behind (fixed order).
// Every output element is one sum over K in rising order, whatever else is in its tile: results do
// not depend on the batch.
//
// Three forms of the products: CUDA cores (any dtype, 32 x 64 tiles); for bfloat16 with K % 32 == 0, mma.sync
// tiles of 32 rows with 32-bit accumulation (few rows an expert: a decode step streams the weights once); and,
// for bfloat16 steps with many rows an expert, tcgen05 tiles of 128 rows: the rows of h are gathered in the
// sorted order once, TMA stages 128 gathered rows and 128 weight rows per k-block of 64 (for the gated product
// 64 gate rows and the 64 up rows of the same features), one thread issues tcgen05.mma into 128 columns of
// tensor memory, and four warps read the accumulator back for the activation or the routing weight.
#include <cuda.h>

#include "common.cuh"
#include "mma.cuh"
#include "tc.cuh"

using namespace llmb;

LLMB_DEFINE_LAST_ERROR(llmb_routed_experts)

constexpr int MAX_TOP = 16;
constexpr int TILE_M = 32;

__device__ __forceinline__ void load4(const float* p, float (&x)[4]) {
    float4 v = *reinterpret_cast<const float4*>(p);
    x[0] = v.x; x[1] = v.y; x[2] = v.z; x[3] = v.w;
}
__device__ __forceinline__ void load4(const __nv_bfloat16* p, float (&x)[4]) {
    uint2 v = *reinterpret_cast<const uint2*>(p);
    float2 lo = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&v.x));
    float2 hi = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&v.y));
    x[0] = lo.x; x[1] = lo.y; x[2] = hi.x; x[3] = hi.y;
}

// A block takes TOK tokens: a weight row fetched once serves all of them. A token's sum runs in the same order
// whatever TOK is (a lane's elements in rising order, then the lanes as a butterfly).
template <typename T, int TOK>
__global__ void __launch_bounds__(512)
router_kernel(const T* __restrict__ h, int ld, const float* __restrict__ w, const float* __restrict__ bias,
              int hidden, int E, int top, int* __restrict__ ids, float* __restrict__ weights, int n_tokens, int vectors,
              int scoring, const float* __restrict__ correction, float weight_scale) {
    extern __shared__ float logits[];      // [TOK][E]
    griddep_launch();
    griddep_wait();
    size_t t0 = (size_t)blockIdx.x * TOK;
    int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const T* rows[TOK];
#pragma unroll
    for (int i = 0; i < TOK; ++i) rows[i] = h + min(t0 + i, (size_t)n_tokens - 1) * ld;
    for (int e = warp; e < E; e += blockDim.x >> 5) {
        float acc[TOK];
#pragma unroll
        for (int i = 0; i < TOK; ++i) acc[i] = 0.f;
        const float* we = w + (size_t)e * hidden;
        if (vectors) {
            // four elements a lane a step (width, row length and addresses allow it: a property of the model, so a
            // token's sum has one order in every step)
#pragma unroll 2
            for (int c = 4 * lane; c < hidden; c += 128) {
                float wv[4];
                load4(we + c, wv);
#pragma unroll
                for (int i = 0; i < TOK; ++i) {
                    float x[4];
                    load4(rows[i] + c, x);
                    acc[i] = fmaf(wv[0], x[0], acc[i]);
                    acc[i] = fmaf(wv[1], x[1], acc[i]);
                    acc[i] = fmaf(wv[2], x[2], acc[i]);
                    acc[i] = fmaf(wv[3], x[3], acc[i]);
                }
            }
        } else {
#pragma unroll 4
            for (int c = lane; c < hidden; c += 32) {
                float wv = we[c];
#pragma unroll
                for (int i = 0; i < TOK; ++i) acc[i] = fmaf(wv, to_float(rows[i][c]), acc[i]);
            }
        }
#pragma unroll
        for (int i = 0; i < TOK; ++i) {
            float total = warp_sum(acc[i]);
            if (lane == 0) logits[i * E + e] = total + (bias ? bias[e] : 0.f);
        }
    }
    __syncthreads();
    if (threadIdx.x >= TOK || t0 + threadIdx.x >= (size_t)n_tokens) return;
    size_t t = t0 + threadIdx.x;
    float* mine = logits + threadIdx.x * E;
    float chosen[MAX_TOP];
    if (scoring == 1) {
        // softmax over every output (terms in index order), the choice by score + correction, the weights by score
        float largest = -INFINITY, total = 0.f;
        for (int e = 0; e < E; ++e) largest = fmaxf(largest, mine[e]);
        for (int e = 0; e < E; ++e) total += expf(mine[e] - largest);
        for (int e = 0; e < E; ++e) mine[e] = expf(mine[e] - largest) / total;      // scores: never negative
        float sum = 0.f;
        for (int k = 0; k < top; ++k) {
            int best = 0;
            float value = -INFINITY;
            for (int e = 0; e < E; ++e) {
                if (mine[e] < 0.f) continue;                  // taken already
                float c = mine[e] + (correction ? correction[e] : 0.f);
                if (c > value) { value = c; best = e; }
            }
            chosen[k] = mine[best];
            sum += chosen[k];
            ids[t * top + k] = best;
            mine[best] = -1.f;
        }
        for (int k = 0; k < top; ++k) weights[t * top + k] = chosen[k] / (sum + 1e-20f) * weight_scale;
        return;
    }
    for (int k = 0; k < top; ++k) {
        int best = 0;
        float value = -INFINITY;
        for (int e = 0; e < E; ++e)
            if (mine[e] > value) { value = mine[e]; best = e; }
        chosen[k] = value;
        ids[t * top + k] = best;
        mine[best] = -INFINITY;
    }
    float total = 0.f, largest = chosen[0];
    for (int k = 0; k < top; ++k) { chosen[k] = expf(chosen[k] - largest); total += chosen[k]; }
    for (int k = 0; k < top; ++k) weights[t * top + k] = chosen[k] / total * weight_scale;
}

// y[a, :] = weights[a] * h[a / top, :] for the assignments a of pass-through experts (ids[a] >= E): 32-bit rows at
// the assignment's own index, like the rows the down product leaves.
template <typename T>
__global__ void __launch_bounds__(256)
pass_through_kernel(const T* __restrict__ h, int ld, int top, const int* __restrict__ ids,
                    const float* __restrict__ weights, int E, int hidden, float* __restrict__ y) {
    griddep_launch();
    griddep_wait();
    int a = blockIdx.x;
    if (ids[a] < E) return;
    float wgt = weights[a];
    const T* row = h + (size_t)(a / top) * ld;
    for (int c = threadIdx.x; c < hidden; c += 256) y[(size_t)a * hidden + c] = wgt * to_float(row[c]);
}

// plan: [0, E] offsets | [E + 1] tile count | then three arrays of max_tiles: expert, first row, rows.
// Several blocks: every block counts all assignments (it needs every expert's offset), block 0 writes the offsets
// and the tiles, and block b lists the assignments of the experts b, b + blocks, ..: its warps take consecutive
// segments of the assignments, count their matches, and place them behind the segments before.
constexpr int PLAN_THREADS = 1024;
__global__ void __launch_bounds__(PLAN_THREADS)
plan_kernel(const int* __restrict__ ids, int n_assign, int E, int* __restrict__ sorted, int* __restrict__ plan,
            int max_tiles, int tile_m) {
    extern __shared__ int shared[];        // counts [E] | offsets [E + 1] | tile bases [E + 1] | a count per warp [32]
    int* counts = shared;
    int* offsets = shared + E;
    int* bases = shared + 2 * E + 1;
    int* warp_counts = shared + 3 * E + 2;
    griddep_launch();
    griddep_wait();
    int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    constexpr int n_warps = PLAN_THREADS / 32;
    for (int e = threadIdx.x; e < E; e += PLAN_THREADS) counts[e] = 0;
    __syncthreads();
    for (int i = threadIdx.x; i < n_assign; i += PLAN_THREADS)
        if (ids[i] < E) atomicAdd(&counts[ids[i]], 1);          // (an id beyond E is a pass-through expert: no rows)
    __syncthreads();
    if (threadIdx.x == 0) {
        int at = 0, tiles = 0;
        for (int e = 0; e < E; ++e) {
            offsets[e] = at;
            bases[e] = tiles;
            at += counts[e];
            tiles += (counts[e] + tile_m - 1) / tile_m;
        }
        offsets[E] = at;
        bases[E] = tiles;
        if (blockIdx.x == 0) plan[E + 1] = tiles < max_tiles ? tiles : max_tiles;
    }
    __syncthreads();
    if (blockIdx.x == 0) {
        for (int e = threadIdx.x; e <= E; e += PLAN_THREADS) plan[e] = offsets[e];
        int* tile_expert = plan + E + 2;
        int* tile_first = tile_expert + max_tiles;
        int* tile_rows = tile_first + max_tiles;
        for (int e = threadIdx.x; e < E; e += PLAN_THREADS) {
            int n = counts[e];
            for (int i = 0, tile = bases[e]; i < n && tile < max_tiles; i += tile_m, ++tile) {
                tile_expert[tile] = e;
                tile_first[tile] = offsets[e] + i;
                tile_rows[tile] = min(tile_m, n - i);
            }
        }
    }
    int segment = ((n_assign + n_warps - 1) / n_warps + 31) / 32 * 32;
    int begin = min(warp * segment, n_assign), end = min(begin + segment, n_assign);
    const unsigned below = (1u << lane) - 1u;
    for (int e = blockIdx.x; e < E; e += gridDim.x) {
        if (counts[e] == 0) continue;                 // (the same answer in every thread)
        int matches = 0;
        for (int i0 = begin; i0 < end; i0 += 32) {
            int i = i0 + lane;
            matches += __popc(__ballot_sync(0xffffffffu, i < end && ids[i] == e));
        }
        if (lane == 0) warp_counts[warp] = matches;
        __syncthreads();
        int at = offsets[e];
        for (int w = 0; w < warp; ++w) at += warp_counts[w];
        for (int i0 = begin; i0 < end; i0 += 32) {
            int i = i0 + lane;
            bool mine = i < end && ids[i] == e;
            unsigned mask = __ballot_sync(0xffffffffu, mine);
            if (mine) sorted[at + __popc(mask & below)] = i;
            at += __popc(mask);
        }
        __syncthreads();
    }
}

// ---------------------------------------------------------------------------------------------- CUDA cores

constexpr int BN = 64, BK = 16;

// GLU: W is [2 N, K] per expert (gate rows, then up rows), the result silu(gate) * up in T.
// else: the result weight[row] * sum in 32-bit at row `sorted[s]` of y.
template <typename T, bool GLU>
__global__ void __launch_bounds__(256)
expert_product_kernel(const T* __restrict__ A, int lda, int a_div, const T* __restrict__ W, long long w_stride, int N,
                      int K, const int* __restrict__ sorted, const int* __restrict__ plan, int E, int max_tiles,
                      T* __restrict__ act, float* __restrict__ y, const float* __restrict__ weights) {
    __shared__ float As[BK][TILE_M + 1];
    __shared__ float Bs[GLU ? 2 : 1][BK][BN + 1];
    griddep_launch();
    griddep_wait();
    int tile = blockIdx.y;
    if (tile >= plan[E + 1]) return;
    const int* tile_expert = plan + E + 2;
    int e = tile_expert[tile], first = tile_expert[max_tiles + tile], rows = tile_expert[2 * max_tiles + tile];
    const T* We = W + (long long)e * w_stride;
    int n0 = blockIdx.x * BN;
    int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
    float acc[GLU ? 2 : 1][2][4] = {};
    // which row of A a thread loads: two elements of the 32 x 16 tile
    int a_row = threadIdx.x >> 3, a_k = (threadIdx.x & 7) * 2;
    long long a_src = -1;
    if (a_row < rows) a_src = GLU ? (long long)(sorted[first + a_row] / a_div) * lda : (long long)(first + a_row) * lda;
    for (int k0 = 0; k0 < K; k0 += BK) {
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            int k = k0 + a_k + i;
            As[a_k + i][a_row] = (a_src >= 0 && k < K) ? to_float(A[a_src + k]) : 0.f;
        }
#pragma unroll
        for (int half = 0; half < (GLU ? 2 : 1); ++half)
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                int idx = threadIdx.x + i * 256;          // 64 x 16 elements
                int n = idx >> 4, kk = idx & 15;
                int col = n0 + n, k = k0 + kk;
                Bs[half][kk][n] = (col < N && k < K) ? to_float(We[(long long)(half * N + col) * K + k]) : 0.f;
            }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < BK; ++kk) {
            float a[2] = {As[kk][ty * 2], As[kk][ty * 2 + 1]};
#pragma unroll
            for (int half = 0; half < (GLU ? 2 : 1); ++half)
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    float b = Bs[half][kk][tx * 4 + j];
                    acc[half][0][j] = fmaf(a[0], b, acc[half][0][j]);
                    acc[half][1][j] = fmaf(a[1], b, acc[half][1][j]);
                }
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        int r = ty * 2 + i;
        if (r >= rows) continue;
        int s = first + r;
        if (GLU) {
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                int col = n0 + tx * 4 + j;
                if (col < N) {
                    float g = acc[0][i][j];
                    act[(long long)s * N + col] = from_float<T>(g / (1.0f + expf(-g)) * acc[GLU ? 1 : 0][i][j]);
                }
            }
        } else {
            int assignment = sorted[s];
            float wgt = weights[assignment];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                int col = n0 + tx * 4 + j;
                if (col < N) y[(long long)assignment * N + col] = wgt * acc[0][i][j];
            }
        }
    }
}

// ---------------------------------------------------------------------------------------------- tensor cores

// 32 rows x 128 columns a block of four warps (a warp: 32 x 32), k in steps of 32 through shared memory
// (cp.async, two stages); for GLU the 128 columns are 64 gate and the 64 up columns of the same features.
constexpr int TC_BN = 128, TC_BK = 32, TC_LD = TC_BK + 8;

template <bool GLU>
__global__ void __launch_bounds__(128)
expert_product_tc_kernel(const __nv_bfloat16* __restrict__ A, int lda, int a_div, const __nv_bfloat16* __restrict__ W,
                         long long w_stride, int N, int K, const int* __restrict__ sorted, const int* __restrict__ plan,
                         int E, int max_tiles, __nv_bfloat16* __restrict__ act, float* __restrict__ y,
                         const float* __restrict__ weights) {
    __shared__ __align__(16) __nv_bfloat16 As[2][TILE_M][TC_LD];
    __shared__ __align__(16) __nv_bfloat16 Bs[2][TC_BN][TC_LD];
    griddep_launch();
    griddep_wait();
    int tile = blockIdx.y;
    if (tile >= plan[E + 1]) return;
    const int* tile_expert = plan + E + 2;
    int e = tile_expert[tile], first = tile_expert[max_tiles + tile], rows = tile_expert[2 * max_tiles + tile];
    const __nv_bfloat16* We = W + (long long)e * w_stride;
    constexpr int FEATURES = GLU ? TC_BN / 2 : TC_BN;      // output features a block covers
    int n0 = blockIdx.x * FEATURES;
    int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // loads: A 32 rows x 4 pieces of 8 = 128 pieces, one a thread; B 128 rows x 4 pieces = 512, four a thread
    int a_row = threadIdx.x >> 2, a_piece = (threadIdx.x & 3) * 8;
    const __nv_bfloat16* a_src = nullptr;
    if (a_row < rows)
        a_src = A + (GLU ? (long long)(sorted[first + a_row] / a_div) * lda : (long long)(first + a_row) * lda);
    auto request = [&](int stage, int k0) {
        if (a_src) cp_async16(&As[stage][a_row][a_piece], a_src + k0 + a_piece);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            int idx = threadIdx.x + i * 128;
            int n = idx >> 2, piece = (idx & 3) * 8;
            int feature = GLU ? n0 + (n & 63) : n0 + n;
            long long w_row = GLU ? (long long)((n >> 6) * N + feature) : (long long)feature;
            if (feature < N) cp_async16(&Bs[stage][n][piece], We + w_row * K + k0 + piece);
        }
        cp_async_commit();
    };
    // rows and columns that are never loaded must read as zeros
    for (int i = threadIdx.x; i < 2 * TILE_M * TC_LD; i += 128) (&As[0][0][0])[i] = __float2bfloat16(0.f);
    for (int i = threadIdx.x; i < 2 * TC_BN * TC_LD; i += 128) (&Bs[0][0][0])[i] = __float2bfloat16(0.f);
    __syncthreads();
    float acc[2][4][4] = {};               // [row block of 16][column block of 8][fragment]
    int n_k = K / TC_BK;
    request(0, 0);
    for (int kb = 0; kb < n_k; ++kb) {
        int stage = kb & 1;
        if (kb + 1 < n_k) { request(stage ^ 1, (kb + 1) * TC_BK); cp_async_wait<1>(); }
        else cp_async_wait<0>();
        __syncthreads();
#pragma unroll
        for (int ks = 0; ks < TC_BK; ks += 16) {
            uint32_t a[2][4], b[2][4];
#pragma unroll
            for (int mi = 0; mi < 2; ++mi)
                ldmatrix_x4(a[mi], &As[stage][mi * 16 + (lane & 15)][ks + (lane >> 4) * 8]);
#pragma unroll
            for (int ni = 0; ni < 2; ++ni)       // 16 columns each: two 8-column blocks x two k halves
                ldmatrix_x4(b[ni], &Bs[stage][warp * 32 + ni * 16 + (lane & 7) + ((lane >> 4) << 3)][ks + ((lane >> 3) & 1) * 8]);
#pragma unroll
            for (int mi = 0; mi < 2; ++mi)
#pragma unroll
                for (int ni = 0; ni < 2; ++ni) {
                    mma_bf16(acc[mi][ni * 2], a[mi][0], a[mi][1], a[mi][2], a[mi][3], b[ni][0], b[ni][1]);
                    mma_bf16(acc[mi][ni * 2 + 1], a[mi][0], a[mi][1], a[mi][2], a[mi][3], b[ni][2], b[ni][3]);
                }
        }
        __syncthreads();
    }
    // accumulator element (mi, nj, f): row mi * 16 + lane / 4 + (f / 2) * 8, column warp * 32 + nj * 8 + (lane % 4) * 2 + f % 2
    if (GLU) {
        // gate columns live in warps 0-1, up columns in warps 2-3: exchanged through shared memory
        __shared__ float up[TILE_M][64 + 1];
        if (warp >= 2)
#pragma unroll
            for (int mi = 0; mi < 2; ++mi)
#pragma unroll
                for (int nj = 0; nj < 4; ++nj)
#pragma unroll
                    for (int f = 0; f < 4; ++f)
                        up[mi * 16 + (lane >> 2) + (f >> 1) * 8][(warp - 2) * 32 + nj * 8 + (lane & 3) * 2 + (f & 1)] = acc[mi][nj][f];
        __syncthreads();
        if (warp < 2)
#pragma unroll
            for (int mi = 0; mi < 2; ++mi)
#pragma unroll
                for (int nj = 0; nj < 4; ++nj)
#pragma unroll
                    for (int f = 0; f < 4; ++f) {
                        int r = mi * 16 + (lane >> 2) + (f >> 1) * 8;
                        int c = warp * 32 + nj * 8 + (lane & 3) * 2 + (f & 1);
                        int feature = n0 + c;
                        if (r < rows && feature < N) {
                            float g = acc[mi][nj][f];
                            act[(long long)(first + r) * N + feature] = __float2bfloat16_rn(g / (1.0f + expf(-g)) * up[r][c]);
                        }
                    }
    } else {
#pragma unroll
        for (int mi = 0; mi < 2; ++mi)
#pragma unroll
            for (int f2 = 0; f2 < 2; ++f2) {
                int r = mi * 16 + (lane >> 2) + f2 * 8;
                if (r >= rows) continue;
                int assignment = sorted[first + r];
                float wgt = weights[assignment];
#pragma unroll
                for (int nj = 0; nj < 4; ++nj)
#pragma unroll
                    for (int f = 0; f < 2; ++f) {
                        int col = n0 + warp * 32 + nj * 8 + (lane & 3) * 2 + f;
                        if (col < N) y[(long long)assignment * N + col] = wgt * acc[mi][nj][f2 * 2 + f];
                    }
            }
    }
}

// ---------------------------------------------------------------------------------------------- tcgen05

namespace wide {

using namespace llmb::tc;

constexpr int GM = 128, GK = 64, G_THREADS = 192;
constexpr int A_BYTES = GM * GK * 2;
// tiles of 128 columns: a ring of three stages, two blocks an SM; tiles of 256 columns (two thirds of the operand bytes
// per product): a ring of four, one block an SM
__host__ __device__ constexpr int stages_of(int gn) { return gn == 128 ? 3 : 4; }
__host__ __device__ constexpr size_t smem_of(int gn) { return 1024 + (size_t)stages_of(gn) * (A_BYTES + gn * GK * 2) + (2 * stages_of(gn) + 1) * 8 + 16; }

// Xs[s, :] = h[sorted[s] / top, :]: the rows of h in the order of the plan (16 bytes a thread a time).
__global__ void __launch_bounds__(256)
gather_rows_kernel(const __nv_bfloat16* __restrict__ h, int ld, int top, const int* __restrict__ sorted,
                   const int* __restrict__ plan, int E, int hidden, __nv_bfloat16* __restrict__ out) {
    griddep_launch();
    griddep_wait();
    int per_row = hidden / 8;
    long long total = (long long)plan[E] * per_row;            // the listed assignments (those of experts with matrices)
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        int s = (int)(i / per_row), c = (int)(i % per_row);
        const uint4* src = reinterpret_cast<const uint4*>(h + (long long)(sorted[s] / top) * ld) + c;
        reinterpret_cast<uint4*>(out + (long long)s * hidden)[c] = *src;
    }
}

// One block: the tile `blockIdx.y` of the plan (an expert's rows [first, first + rows) of the sorted list, at most
// 128) times GN accumulator columns: the output columns [blockIdx.x * (GLU ? GN / 2 : GN), ..) of that expert. A: [rows of the list, K] behind
// map_a. B: every expert's matrix stacked, [E * b_rows, K] behind map_b; GLU: an expert's b_rows = 2 N rows are N
// gate rows, then N up rows, and a stage holds GN / 2 gate rows and the GN / 2 up rows of the same features, so that the
// accumulator's first half are gates and its second half the ups. Warp 0: TMA producer. Warp 1: tensor memory and the
// products. Warps 2..5: epilogue, a thread a row. Every wait is bounded and reports through `status`.
template <bool GLU, int GN>
__global__ void __launch_bounds__(G_THREADS, GN == 128 ? 2 : 1)
expert_product_wide_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                           const int* __restrict__ plan, int E, int max_tiles, int b_rows, int N, int n_kblocks,
                           __nv_bfloat16* __restrict__ act, float* __restrict__ y, const int* __restrict__ sorted,
                           const float* __restrict__ weights, int* status) {
    constexpr int G_STAGES = stages_of(GN), B_BYTES = GN * GK * 2;
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    unsigned char* base = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    unsigned char* a_tiles = base;
    unsigned char* b_tiles = base + (size_t)G_STAGES * A_BYTES;
    uint64_t* full_bar = reinterpret_cast<uint64_t*>(b_tiles + (size_t)G_STAGES * B_BYTES);
    uint64_t* empty_bar = full_bar + G_STAGES;
    uint64_t* acc_bar = full_bar + 2 * G_STAGES;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_bar + 1);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    griddep_launch();
    griddep_wait();                                   // the plan is the work of the kernel before
    int tile = blockIdx.y;
    if (tile >= plan[E + 1]) return;                  // (before anything is allocated)
    const int* tile_expert = plan + E + 2;
    int e = tile_expert[tile], first = tile_expert[max_tiles + tile], rows = tile_expert[2 * max_tiles + tile];
    int n0 = blockIdx.x * (GLU ? GN / 2 : GN);
    int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_a) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_b) : "memory");
        for (int s = 0; s < G_STAGES; ++s) {
            mbar_init(smem_u32(&full_bar[s]), 1);
            mbar_init(smem_u32(&empty_bar[s]), 1);
        }
        mbar_init(smem_u32(acc_bar), 1);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(smem_u32(tmem_slot)), "r"(GN) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tcgen05_fence_before();
    __syncthreads();
    tcgen05_fence_after();
    uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        if (lane == 0) {
            int s = 0;
            uint32_t round = 0;
            int b_row = e * b_rows + n0;
            for (int kb = 0; kb < n_kblocks; ++kb) {
                if (!mbar_wait(smem_u32(&empty_bar[s]), (round & 1) ^ 1, abort_flag, status, 1)) break;
                uint32_t bar = smem_u32(&full_bar[s]);
                mbar_expect_tx(bar, A_BYTES + B_BYTES);
                tma_load_2d(smem_u32(a_tiles + (size_t)s * A_BYTES), &map_a, bar, kb * GK, first);
                if (GLU) {
                    tma_load_2d(smem_u32(b_tiles + (size_t)s * B_BYTES), &map_b, bar, kb * GK, b_row);
                    tma_load_2d(smem_u32(b_tiles + (size_t)s * B_BYTES + B_BYTES / 2), &map_b, bar, kb * GK, b_row + N);
                } else {
                    tma_load_2d(smem_u32(b_tiles + (size_t)s * B_BYTES), &map_b, bar, kb * GK, b_row);
                }
                if (++s == G_STAGES) { s = 0; ++round; }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            // instruction descriptor: D 32-bit, A and B bfloat16, both K-major, N = GN, M = 128
            constexpr uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(GN >> 3) << 17) | ((uint32_t)(GM >> 4) << 24);
            const uint64_t a_desc0 = smem_desc(smem_u32(a_tiles)), b_desc0 = smem_desc(smem_u32(b_tiles));
            int s = 0;
            uint32_t phase = 0;
            bool ok = true;
            for (int kb = 0; kb < n_kblocks; ++kb) {
                ok = mbar_wait(smem_u32(&full_bar[s]), phase, abort_flag, status, 2);
                if (!ok) break;
                tcgen05_fence_after();
                uint64_t a_desc = a_desc0 + (uint64_t)(s * (A_BYTES >> 4));
                uint64_t b_desc = b_desc0 + (uint64_t)(s * (B_BYTES >> 4));
#pragma unroll
                for (int k = 0; k < GK / 16; ++k)               // 16 k-values = 32 bytes inside the swizzled row
                    tcgen05_mma(tmem_base, a_desc + 2 * k, b_desc + 2 * k, idesc, (kb > 0 || k > 0) ? 1u : 0u);
                tcgen05_commit(smem_u32(&empty_bar[s]));
                if (++s == G_STAGES) { s = 0; phase ^= 1; }
            }
            if (ok) tcgen05_commit(smem_u32(acc_bar));
        }
    } else {
        int quarter = warp & 3;                                  // the 32 lanes of tensor memory this warp may read
        int row = quarter * 32 + lane;
        bool ok = mbar_wait(smem_u32(acc_bar), 0, abort_flag, status, 3);
        ok = __all_sync(0xffffffffu, ok);
        if (ok) {
            tcgen05_fence_after();
            uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16);
            bool live = row < rows;
            if (GLU) {
                __nv_bfloat16* out = act + (long long)(first + row) * N + n0;
                bool vector = N % 8 == 0;
#pragma unroll 1
                for (int c = 0; c < GN / 2; c += 16) {
                    uint32_t g[16], u[16];
                    tmem_ld16(taddr + c, g);
                    tmem_ld16(taddr + GN / 2 + c, u);
                    if (!live || n0 + c >= N) continue;
                    float v[16];
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        float gate = __uint_as_float(g[j]);
                        v[j] = gate / (1.0f + expf(-gate)) * __uint_as_float(u[j]);
                    }
                    if (vector && n0 + c + 16 <= N) {
                        uint32_t packed[8];
#pragma unroll
                        for (int j = 0; j < 8; ++j) {
                            __nv_bfloat162 two = __floats2bfloat162_rn(v[2 * j], v[2 * j + 1]);
                            packed[j] = *reinterpret_cast<uint32_t*>(&two);
                        }
                        uint4* dst = reinterpret_cast<uint4*>(out + c);
                        dst[0] = make_uint4(packed[0], packed[1], packed[2], packed[3]);
                        dst[1] = make_uint4(packed[4], packed[5], packed[6], packed[7]);
                    } else {
#pragma unroll
                        for (int j = 0; j < 16; ++j)
                            if (n0 + c + j < N) out[c + j] = __float2bfloat16_rn(v[j]);
                    }
                }
            } else {
                int assignment = live ? sorted[first + row] : 0;
                float wgt = live ? weights[assignment] : 0.f;
                float* out = y + (long long)assignment * N + n0;
                bool vector = N % 4 == 0;
#pragma unroll 1
                for (int c = 0; c < GN; c += 16) {
                    uint32_t r[16];
                    tmem_ld16(taddr + c, r);
                    if (!live || n0 + c >= N) continue;
                    if (vector && n0 + c + 16 <= N) {
#pragma unroll
                        for (int j = 0; j < 4; ++j)
                            reinterpret_cast<float4*>(out + c)[j] =
                                make_float4(wgt * __uint_as_float(r[4 * j]), wgt * __uint_as_float(r[4 * j + 1]),
                                            wgt * __uint_as_float(r[4 * j + 2]), wgt * __uint_as_float(r[4 * j + 3]));
                    } else {
#pragma unroll
                        for (int j = 0; j < 16; ++j)
                            if (n0 + c + j < N) out[c + j] = wgt * __uint_as_float(r[j]);
                    }
                }
            }
        }
    }

    // teardown: everyone meets, then the allocating warp frees the tensor memory
    tcgen05_fence_before();
    __syncthreads();
    if (*abort_flag) {
        for (int i = 0; i < 100; ++i) __nanosleep(10000);          // copies in flight land before shared memory is given up
        __syncthreads();
    }
    if (warp == 1) {
        tcgen05_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(GN) : "memory");
    }
}

}  // namespace wide

LLMB_EXPORT int llmb_routed_experts_status() {
    int* s = llmb::tc::status_word();
    if (!s) return -1;
    int v = *s;
    *s = 0;
    return v;
}

LLMB_EXPORT long long llmb_routed_experts_plan_ints(int n_tokens, int top, int E) {
    long long max_tiles = ((long long)n_tokens * top + TILE_M - 1) / TILE_M + E;
    return (long long)E + 2 + 3 * max_tiles;
}

// h [T, ld] in `dtype`; router float32 [E, hidden] and bias float32 [E] (or null); w_up [E, 2 F, hidden] (gate rows,
// then up rows) and w_down [E, hidden, F] in `dtype`; ids int32 [T * top], weights float32 [T * top], sorted
// int32 [T * top], plan int32 [plan_ints]; act [T * top, F] in `dtype`; y float32 [T * top, hidden]. `tensor_cores`:
// 0 CUDA cores only, 1 also the mma.sync tiles, 2 also the tcgen05 tiles of 128 rows, which need `gathered`
// (bfloat16 [T * top, hidden] scratch) and are taken when the step has that scratch, 3: those with 256 accumulator columns.
LLMB_EXPORT int llmb_routed_experts(const void* h, int ld, int dtype, const float* router, const float* router_bias,
                                    const void* w_up, const void* w_down, int* ids, float* weights, int* sorted,
                                    int* plan, void* act, float* y, void* gathered, int n_tokens, int hidden, int F,
                                    int E, int top, int tensor_cores, int scoring, const float* correction,
                                    int pass_through, float weight_scale, cudaStream_t stream) {
    if (n_tokens == 0) return LLMB_OK;
    LLMB_REQUIRE(hidden > 0 && F > 0 && E > 0 && top > 0 && pass_through >= 0 && top <= E + pass_through && top <= MAX_TOP,
                 "routed_experts: %d of %d experts (at most %d are chosen)", top, E + pass_through, MAX_TOP);
    LLMB_REQUIRE(scoring == 0 || scoring == 1, "routed_experts: scoring %d (0: softmax over the chosen, 1: over all)", scoring);
    int R = E + pass_through;                                  // outputs of the router
    LLMB_REQUIRE(E <= 2048, "routed_experts: %d experts (up to 2048 are built)", E);
    int n_assign = n_tokens * top;
    int max_tiles = (n_assign + TILE_M - 1) / TILE_M + E;
    dim3 grid_up((F + BN - 1) / BN, max_tiles), grid_down((hidden + BN - 1) / BN, max_tiles);
    long long up_stride = 2LL * F * hidden, down_stride = (long long)hidden * F;
    int router_vectors = hidden % 4 == 0 && ld % 4 == 0 && ((size_t)h % 16) == 0 && ((size_t)router % 16) == 0;
    bool aligned = ld % 8 == 0 && ((size_t)h % 16) == 0 && ((size_t)w_up % 16) == 0 && ((size_t)w_down % 16) == 0 &&
                   ((size_t)act % 16) == 0;
    bool wide_tiles = tensor_cores >= 2 && dtype == LLMB_DTYPE_BF16 && gathered && hidden % 8 == 0 && F % 8 == 0 && aligned &&
                      ((size_t)gathered % 16) == 0 && ((size_t)y % 16) == 0 && (long long)E * 2 * F < (1LL << 31) &&
                      (long long)E * hidden < (1LL << 31);
    int tile_m = wide_tiles ? wide::GM : TILE_M;
#define LLMB_EXPERTS(T)                                                                                            \
    do {                                                                                                           \
        if (n_tokens >= 512)                                                                                       \
            LLMB_CUDA(llmb::launch(router_kernel<T, 4>, dim3((n_tokens + 3) / 4), dim3(128), sizeof(float) * 4 * R, \
                                   stream, true, (const T*)h, ld, router, router_bias, hidden, R, top, ids,       \
                                   weights, n_tokens, router_vectors, scoring, correction, weight_scale));        \
        else                                                                                                       \
            LLMB_CUDA(llmb::launch(router_kernel<T, 1>, dim3(n_tokens), dim3(512), sizeof(float) * R, stream,     \
                                   true, (const T*)h, ld, router, router_bias, hidden, R, top, ids, weights,       \
                                   n_tokens, router_vectors, scoring, correction, weight_scale));                  \
        if (pass_through > 0)                                                                                      \
            LLMB_CUDA(llmb::launch(pass_through_kernel<T>, dim3(n_assign), dim3(256), 0, stream, true, (const T*)h, \
                                   ld, top, (const int*)ids, (const float*)weights, E, hidden, y));                \
        LLMB_CUDA(llmb::launch(plan_kernel, dim3(E < 64 ? E : 64), dim3(PLAN_THREADS),                             \
                               sizeof(int) * (3 * E + 2 + 32), stream, true, (const int*)ids, n_assign, E, sorted, \
                               plan, max_tiles, tile_m));                                                          \
    } while (0)
    if (dtype == LLMB_DTYPE_F32) LLMB_EXPERTS(float);
    else if (dtype == LLMB_DTYPE_BF16) LLMB_EXPERTS(__nv_bfloat16);
    else return fail(LLMB_ERR_ARGUMENT, "routed_experts: unknown dtype %d", dtype);
#undef LLMB_EXPERTS
    bool tc = tensor_cores && dtype == LLMB_DTYPE_BF16 && hidden % TC_BK == 0 && F % TC_BK == 0 && aligned;
    if (wide_tiles) {
        typedef __nv_bfloat16 B;
        using namespace wide;
        // tiles of 256 columns for long lists (measured at width 4096, 8 of 32 experts of 1792: 3.65 against 3.86 ms at 8,192
        // tokens, equal at 2,048, behind at width 2048) where the products are wide enough for them
        bool wide256 = tensor_cores >= 3 && F >= 128 && hidden >= 256 && (long long)n_assign >= 1024LL * E;
        int GN = wide256 ? 256 : 128;
        size_t smem = smem_of(GN);
        static bool configured = false;
        if (!configured) {
            LLMB_CUDA(cudaFuncSetAttribute(expert_product_wide_kernel<true, 128>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_of(128)));
            LLMB_CUDA(cudaFuncSetAttribute(expert_product_wide_kernel<false, 128>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_of(128)));
            LLMB_CUDA(cudaFuncSetAttribute(expert_product_wide_kernel<true, 256>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_of(256)));
            LLMB_CUDA(cudaFuncSetAttribute(expert_product_wide_kernel<false, 256>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_of(256)));
            configured = true;
        }
        int* status_dev = nullptr;
        int* status_host = llmb::tc::status_word();
        if (status_host) LLMB_CUDA(cudaHostGetDevicePointer((void**)&status_dev, status_host, 0));
        CUtensorMap map_x, map_up, map_act, map_down;
        int code = llmb::tc::make_map_2d(&map_x, gathered, n_assign, hidden, hidden, GK, GM);
        if (!code) code = llmb::tc::make_map_2d(&map_up, w_up, (long long)E * 2 * F, hidden, hidden, GK, GN / 2);
        if (!code) code = llmb::tc::make_map_2d(&map_act, act, n_assign, F, F, GK, GM);
        if (!code) code = llmb::tc::make_map_2d(&map_down, w_down, (long long)E * hidden, F, F, GK, GN);
        if (code) return code;
        int tiles = (n_assign + GM - 1) / GM + E;
        if (tiles > max_tiles) tiles = max_tiles;
        long long vectors = (long long)n_assign * (hidden / 8);
        int gather_blocks = (int)((vectors + 255) / 256 < 148 * 8 ? (vectors + 255) / 256 : 148 * 8);
        LLMB_CUDA(llmb::launch(gather_rows_kernel, dim3(gather_blocks), dim3(256), 0, stream, true, (const B*)h, ld, top,
                               (const int*)sorted, (const int*)plan, E, hidden, (B*)gathered));
        auto up = wide256 ? expert_product_wide_kernel<true, 256> : expert_product_wide_kernel<true, 128>;
        auto down = wide256 ? expert_product_wide_kernel<false, 256> : expert_product_wide_kernel<false, 128>;
        LLMB_CUDA(llmb::launch(up, dim3((F + GN / 2 - 1) / (GN / 2), tiles), dim3(G_THREADS), smem, stream, true, map_x, map_up,
                               (const int*)plan, E, max_tiles, 2 * F, F, (hidden + GK - 1) / GK, (B*)act, (float*)nullptr,
                               (const int*)sorted, (const float*)nullptr, status_dev));
        LLMB_CUDA(llmb::launch(down, dim3((hidden + GN - 1) / GN, tiles), dim3(G_THREADS), smem, stream, true, map_act, map_down,
                               (const int*)plan, E, max_tiles, hidden, hidden, (F + GK - 1) / GK, (B*)nullptr, y,
                               (const int*)sorted, (const float*)weights, status_dev));
    } else if (tc) {
        typedef __nv_bfloat16 B;
        LLMB_CUDA(llmb::launch(expert_product_tc_kernel<true>, dim3((F + 63) / 64, max_tiles), dim3(128), 0, stream, true,
                               (const B*)h, ld, top, (const B*)w_up, up_stride, F, hidden, (const int*)sorted,
                               (const int*)plan, E, max_tiles, (B*)act, (float*)nullptr, (const float*)nullptr));
        LLMB_CUDA(llmb::launch(expert_product_tc_kernel<false>, dim3((hidden + 127) / 128, max_tiles), dim3(128), 0, stream,
                               true, (const B*)act, F, 1, (const B*)w_down, down_stride, hidden, F, (const int*)sorted,
                               (const int*)plan, E, max_tiles, (B*)nullptr, y, (const float*)weights));
    } else if (dtype == LLMB_DTYPE_F32) {
        LLMB_CUDA(llmb::launch(expert_product_kernel<float, true>, grid_up, dim3(256), 0, stream, true, (const float*)h, ld,
                               top, (const float*)w_up, up_stride, F, hidden, (const int*)sorted, (const int*)plan, E,
                               max_tiles, (float*)act, (float*)nullptr, (const float*)nullptr));
        LLMB_CUDA(llmb::launch(expert_product_kernel<float, false>, grid_down, dim3(256), 0, stream, true,
                               (const float*)act, F, 1, (const float*)w_down, down_stride, hidden, F, (const int*)sorted,
                               (const int*)plan, E, max_tiles, (float*)nullptr, y, (const float*)weights));
    } else {
        typedef __nv_bfloat16 B;
        LLMB_CUDA(llmb::launch(expert_product_kernel<B, true>, grid_up, dim3(256), 0, stream, true, (const B*)h, ld, top,
                               (const B*)w_up, up_stride, F, hidden, (const int*)sorted, (const int*)plan, E, max_tiles,
                               (B*)act, (float*)nullptr, (const float*)nullptr));
        LLMB_CUDA(llmb::launch(expert_product_kernel<B, false>, grid_down, dim3(256), 0, stream, true, (const B*)act, F, 1,
                               (const B*)w_down, down_stride, hidden, F, (const int*)sorted, (const int*)plan, E,
                               max_tiles, (B*)nullptr, y, (const float*)weights));
    }
    return check_launch("routed_experts");
}
LLMB_PACKED(llmb_routed_experts)
