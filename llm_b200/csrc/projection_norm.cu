// What lies between a projection and the attention of a mixer that norms whole projections: an RMS
// norm over ALL query columns of a token (and one over all key columns), then the rotation of every
// head, then queries out and keys and values into the paged cache. One launch, one block per token.
//
// The row u[t] = [queries (q_width) | keys (k_width) | values (v_width) | anything else] is read once
// into shared memory as 32-bit values; the two sums of squares are reduced in a fixed order (thread
// order, then lanes, then warps), the factor 1 / sqrt(mean + eps) and the gain are applied in 32-bit,
// pairs are rotated in 32-bit by the angles of a table [positions, n_rot] (cosines, then sines; made in
// float64 by the position encoding), and only the stores round to the run's dtype. Without a gain a
// segment is not normed; without a table nothing rotates; with v_width == 0 there are no values (a mixer
// whose cached row serves as key and value).
//
// With norm_unit > 0 the norms run over units of that many columns instead (a head each: every unit of
// the queries and of the keys is divided by its own root mean square, and the gain has norm_unit elements
// that all units share); a warp takes a unit, its lanes the unit's elements in strides of 32.
// With mix_cache the values are blended before they are cached: v <- (1 - mix) v + mix * first, where
// `first` is the row that another layer's value cache (mix_cache, with its own page table and ring) holds
// for the same token, key/value head and element; that layer must have written the step's tokens before.
#include "common.cuh"

using namespace llmb;

LLMB_DEFINE_LAST_ERROR(llmb_projection_norm)

constexpr int THREADS = 256;

__device__ __forceinline__ float block_sum(float v, float* scratch) {
    v = warp_sum(v);
    int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    __syncthreads();                       // scratch may still be read from the call before
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    float total = 0.f;
#pragma unroll
    for (int w = 0; w < THREADS / 32; ++w) total += scratch[w];
    return total;
}

template <typename T>
__global__ void __launch_bounds__(THREADS)
norm_rope_cache_write_kernel(const T* __restrict__ u, int u_stride, int q_width, int k_width, int v_width,
                             const float* __restrict__ q_gain, const float* __restrict__ k_gain, float eps,
                             const float* __restrict__ rope_table, int n_rot, int rot_unit, int interleaved,
                             const int* __restrict__ tok_pos, const int* __restrict__ tok_seq, T* __restrict__ q_out,
                             int q_out_stride, const int* __restrict__ block_table, int table_stride, int ring_pages,
                             T* __restrict__ k_cache, int k_heads, T* __restrict__ v_cache, int v_heads,
                             int write_cache, int v_source, int norm_unit, const T* __restrict__ mix_cache,
                             const int* __restrict__ mix_table, int mix_table_stride, int mix_ring, float mix) {
    extern __shared__ float row[];         // [q_width + k_width]
    __shared__ float scratch[THREADS / 32];
    griddep_launch();
    griddep_wait();
    int t = blockIdx.x;
    const T* in = u + (size_t)t * u_stride;
    int qk = q_width + (write_cache ? k_width : 0);
    float sq_q = 0.f, sq_k = 0.f;
    for (int e = threadIdx.x; e < qk; e += THREADS) {
        float v = to_float(in[e]);
        row[e] = v;
        if (e < q_width) sq_q = fmaf(v, v, sq_q);
        else sq_k = fmaf(v, v, sq_k);
    }
    if (norm_unit > 0) {
        __syncthreads();
        int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
        for (int unit = warp; unit < qk / norm_unit; unit += THREADS / 32) {
            float* x = row + unit * norm_unit;
            const float* gain = unit * norm_unit < q_width ? q_gain : k_gain;
            if (!gain) continue;
            float sq = 0.f;
            for (int d = lane; d < norm_unit; d += 32) sq = fmaf(x[d], x[d], sq);
            float factor = 1.0f / sqrtf(warp_sum(sq) / (float)norm_unit + eps);
            for (int d = lane; d < norm_unit; d += 32) x[d] = x[d] * factor * gain[d];
        }
    } else {
        float q_scale = 1.f, k_scale = 1.f;
        if (q_gain) q_scale = 1.0f / sqrtf(block_sum(sq_q, scratch) / (float)q_width + eps);
        if (k_gain && write_cache) k_scale = 1.0f / sqrtf(block_sum(sq_k, scratch) / (float)k_width + eps);
        __syncthreads();
        for (int e = threadIdx.x; e < qk; e += THREADS) {
            bool is_q = e < q_width;
            const float* gain = is_q ? q_gain : k_gain;
            if (gain) row[e] = row[e] * (is_q ? q_scale : k_scale) * gain[is_q ? e : e - q_width];
        }
    }
    __syncthreads();
    int pos = tok_pos[t];
    const float* angles = rope_table ? rope_table + (size_t)pos * n_rot : nullptr;
    int half = n_rot / 2;
    size_t page = 0;
    int slot_row = pos % LLMB_PAGE;
    if (write_cache) page = (size_t)block_table[(size_t)tok_seq[t] * table_stride + (pos / LLMB_PAGE) % ring_pages];
    int k_dim = k_heads > 0 ? k_width / k_heads : 0;
    for (int e = threadIdx.x; e < qk; e += THREADS) {
        bool is_q = e < q_width;
        int local = is_q ? e : e - q_width;            // column inside the segment
        float v = row[e];
        if (angles) {
            int d = local % rot_unit;                  // element inside its unit
            if (d < n_rot) {
                int pair, partner;
                bool first;
                if (interleaved) { pair = d >> 1; first = (d & 1) == 0; partner = first ? e + 1 : e - 1; }
                else { first = d < half; pair = first ? d : d - half; partner = first ? e + half : e - half; }
                float c = angles[pair], s = angles[half + pair], other = row[partner];
                v = first ? v * c - other * s : v * c + other * s;
            }
        }
        if (is_q) {
            q_out[(size_t)t * q_out_stride + local] = from_float<T>(v);
        } else {
            int head = local / k_dim, d = local % k_dim;
            k_cache[((page * k_heads + head) * LLMB_PAGE + slot_row) * k_dim + d] = from_float<T>(v);
        }
    }
    if (write_cache && v_width > 0) {
        int v_dim = v_width / v_heads;
        const T* values = in + v_source;       // as projected: a source inside the key columns gives the keys before rotation
        size_t mix_page = 0;
        if (mix_cache) mix_page = (size_t)mix_table[(size_t)tok_seq[t] * mix_table_stride + (pos / LLMB_PAGE) % mix_ring];
        for (int e = threadIdx.x; e < v_width; e += THREADS) {
            int head = e / v_dim, d = e % v_dim;
            T value = values[e];
            if (mix_cache) {
                float first = to_float(mix_cache[((mix_page * v_heads + head) * LLMB_PAGE + slot_row) * v_dim + d]);
                value = from_float<T>((1.0f - mix) * to_float(value) + mix * first);
            }
            v_cache[((page * v_heads + head) * LLMB_PAGE + slot_row) * v_dim + d] = value;
        }
    }
}

// k_cache [pages, k_heads, 64, k_width / k_heads], v_cache [pages, v_heads, 64, v_width / v_heads] (v_width == 0: none).
// The values of a token are the v_width columns of u from column v_source on (q_width + k_width: the columns behind
// the keys; q_width: the keys themselves as projected, for a mixer without a value projection).
LLMB_EXPORT int llmb_norm_rope_cache_write(const void* u, int u_stride, int dtype, int q_width, int k_width, int v_width,
                                           const float* q_gain, const float* k_gain, float eps, const float* rope_table,
                                           int n_rot, int rot_unit, int interleaved, const int* tok_pos,
                                           const int* tok_seq, void* q_out, int q_out_stride, const int* block_table,
                                           int table_stride, int ring_pages, void* k_cache, int k_heads, void* v_cache,
                                           int v_heads, int write_cache, int v_source, int norm_unit,
                                           const void* mix_cache, const int* mix_table, int mix_table_stride,
                                           int mix_ring, float mix, int n_tokens, cudaStream_t stream) {
    if (n_tokens == 0) return LLMB_OK;
    LLMB_REQUIRE(q_width > 0 && k_width > 0 && v_width >= 0 && k_heads > 0 && k_width % k_heads == 0,
                 "norm_rope_cache_write: bad widths %d / %d / %d with %d key heads", q_width, k_width, v_width, k_heads);
    LLMB_REQUIRE(v_width == 0 || (v_heads > 0 && v_width % v_heads == 0 && v_cache),
                 "norm_rope_cache_write: %d value columns do not fit %d heads", v_width, v_heads);
    LLMB_REQUIRE(!rope_table || (n_rot > 0 && n_rot % 2 == 0 && n_rot <= rot_unit && q_width % rot_unit == 0 &&
                                 k_width % rot_unit == 0),
                 "norm_rope_cache_write: %d rotated elements do not fit units of %d", n_rot, rot_unit);
    LLMB_REQUIRE(ring_pages > 0, "norm_rope_cache_write: no pages");
    LLMB_REQUIRE(v_source >= 0, "norm_rope_cache_write: the values start at column %d", v_source);
    LLMB_REQUIRE(norm_unit >= 0 && (norm_unit == 0 || (q_width % norm_unit == 0 && k_width % norm_unit == 0)),
                 "norm_rope_cache_write: units of %d columns do not divide %d and %d", norm_unit, q_width, k_width);
    LLMB_REQUIRE(!mix_cache || (mix_table && mix_ring > 0 && v_width > 0 && mix_cache != v_cache),
                 "norm_rope_cache_write: values are blended with another layer's cache, which needs its page table");
    size_t smem = sizeof(float) * (size_t)(q_width + k_width);
    LLMB_REQUIRE(smem <= 200 * 1024, "norm_rope_cache_write: a row of %d + %d values does not fit in shared memory",
                 q_width, k_width);
#define LLMB_NORM_ROPE(T)                                                                                            \
    do {                                                                                                             \
        if (smem > 48 * 1024)                                                                                        \
            LLMB_CUDA(cudaFuncSetAttribute(norm_rope_cache_write_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, \
                                           (int)smem));                                                              \
        LLMB_CUDA(llmb::launch(norm_rope_cache_write_kernel<T>, dim3(n_tokens), dim3(THREADS), smem, stream, true,    \
                               (const T*)u, u_stride, q_width, k_width, v_width, q_gain, k_gain, eps, rope_table,   \
                               rope_table ? n_rot : 0, rot_unit > 0 ? rot_unit : 1, interleaved, tok_pos, tok_seq,   \
                               (T*)q_out, q_out_stride, block_table, table_stride, ring_pages, (T*)k_cache, k_heads, \
                               (T*)v_cache, v_heads, write_cache, v_source, norm_unit, (const T*)mix_cache,          \
                               mix_table, mix_table_stride, mix_ring, mix));                                        \
    } while (0)
    if (dtype == LLMB_DTYPE_F32) LLMB_NORM_ROPE(float);
    else if (dtype == LLMB_DTYPE_BF16) LLMB_NORM_ROPE(__nv_bfloat16);
    else return fail(LLMB_ERR_ARGUMENT, "norm_rope_cache_write: unknown dtype %d", dtype);
#undef LLMB_NORM_ROPE
    return check_launch("norm_rope_cache_write");
}

LLMB_PACKED(llmb_norm_rope_cache_write)
