// Causal attention without softmax over a paged cache whose keys and values may differ in size:
//   weight(query i, key j <= i) = sigmoid(scale * q_i . k_j + bias[head]),   out_i = sum_j weight * v_j
// (weights are not normalised over keys).  Scores, weights and the sums are fp32.
//
// rotate_store: rotate-half rotation of the first `rotary` elements of every query and key head (pair (i, i +
// rotary / 2), angle = float(position) * inv_freq[i] in fp32), queries to q_out, keys and values into the request's
// pages: k_pool [pages, kv_heads, page, D], v_pool [pages, kv_heads, page, V].
// attend: one block per (tile of up to 16 consecutive queries of a run, query head); keys are walked in tiles of 32
// in ascending order, so an output's sum has the same order however the tokens were cut into steps.
#include "common.cuh"

EMBER_DEFINE_LAST_ERROR

namespace ember {

template <typename T>
__global__ void rotate_store_kernel(const float* __restrict__ qkv, int ld, int H, int G, int D, int V,
                                    const float* __restrict__ inv_freq, int rotary,
                                    const int* __restrict__ positions, const int* __restrict__ seq_of,
                                    const int* __restrict__ block_table, int max_blocks, int page, int num_pages,
                                    T* __restrict__ q_out, T* __restrict__ k_pool, T* __restrict__ v_pool, int write_kv,
                                    int* __restrict__ err) {
    extern __shared__ float cs[];           // cos [rotary / 2], sin [rotary / 2]
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x, pos = positions[t], half = rotary >> 1;
    for (int i = threadIdx.x; i < half; i += blockDim.x) {
        float sn, c;
        sincosf((float)pos * inv_freq[i], &sn, &c);
        cs[i] = c; cs[half + i] = sn;
    }
    __syncthreads();
    const float* row = qkv + (size_t)t * ld;
    const int blk = block_table[(size_t)seq_of[t] * max_blocks + pos / page], slot = pos % page;
    const bool page_ok = blk >= 0 && blk < num_pages;
    if (write_kv && !page_ok && threadIdx.x == 0 && err) atomicOr(err, EMBER_ERR_PAGE_RANGE);
    // query and key heads: H + G heads of D
    for (int e = threadIdx.x; e < (H + G) * D; e += blockDim.x) {
        const int head = e / D, i = e - head * D;
        float v = row[e];
        if (i < rotary) {
            const int f = i < half ? i : i - half;
            const float other = row[head * D + (i < half ? i + half : i - half)];
            v = i < half ? v * cs[f] - other * cs[half + f] : v * cs[f] + other * cs[half + f];
        }
        if (head < H) q_out[(size_t)t * H * D + e] = from_float<T>(v);
        else if (write_kv && page_ok)
            k_pool[(((size_t)blk * G + (head - H)) * page + slot) * D + i] = from_float<T>(v);
    }
    if (write_kv && page_ok) {
        const float* vr = row + (size_t)(H + G) * D;
        for (int e = threadIdx.x; e < G * V; e += blockDim.x) {
            const int head = e / V, i = e - head * V;
            v_pool[(((size_t)blk * G + head) * page + slot) * V + i] = from_float<T>(vr[e]);
        }
    }
}

constexpr int SA_ROWS = 16, SA_KEYS = 32, SA_THREADS = 128;

// CM: value columns per thread (V <= 128 CM)
template <typename T, int CM>
__global__ void __launch_bounds__(SA_THREADS)
sigmoid_attention_kernel(const T* __restrict__ q, const T* __restrict__ k_pool, const T* __restrict__ v_pool,
                         T* __restrict__ out, int H, int G, int D, int V, const int* __restrict__ tiles,
                         const int* __restrict__ block_table, int max_blocks, int page, int num_pages, float scale,
                         const float* __restrict__ head_bias, int* __restrict__ err) {
    extern __shared__ float smem[];
    pdl_launch_dependents();
    pdl_wait();
    const int* tile = tiles + 4 * blockIdx.x;
    const int run = tile[0], row0 = tile[1], nq = tile[2], pos0 = tile[3];
    const int h = blockIdx.y, kv = h / (H / G);
    const int DP = D + 1;
    float* qs = smem;                                   // [SA_ROWS][D]
    float* ks = qs + SA_ROWS * D;                       // [SA_KEYS][D + 1]
    float* vs = ks + SA_KEYS * DP;                      // [SA_KEYS][V]
    float* ws = vs + SA_KEYS * V;                       // [SA_ROWS][SA_KEYS]
    for (int e = threadIdx.x; e < SA_ROWS * D; e += SA_THREADS) {
        const int r = e / D, i = e - r * D;
        qs[e] = r < nq ? to_float(q[((size_t)(row0 + r) * H + h) * D + i]) : 0.0f;
    }
    const float bias = head_bias ? head_bias[h] : 0.0f;
    float acc[SA_ROWS][CM];
#pragma unroll
    for (int r = 0; r < SA_ROWS; r++)
#pragma unroll
        for (int m = 0; m < CM; m++) acc[r][m] = 0.0f;
    const int n_keys = pos0 + nq;                       // keys 0 .. position of the last query
    const int* bt = block_table + (size_t)run * max_blocks;
    const int kk = threadIdx.x & 31, rg = threadIdx.x >> 5;
    for (int k0 = 0; k0 < n_keys; k0 += SA_KEYS) {
        __syncthreads();
        // keys and values of this tile (rows beyond the last key are zero)
        for (int e = threadIdx.x; e < SA_KEYS * D; e += SA_THREADS) {
            const int r = e / D, i = e - r * D, kp = k0 + r;
            float v = 0.0f;
            if (kp < n_keys) {
                const int blk = bt[kp / page];
                if (blk >= 0 && blk < num_pages) v = to_float(k_pool[(((size_t)blk * G + kv) * page + kp % page) * D + i]);
                else if (err) atomicOr(err, EMBER_ERR_PAGE_RANGE);
            }
            ks[r * DP + i] = v;
        }
        for (int e = threadIdx.x; e < SA_KEYS * V; e += SA_THREADS) {
            const int r = e / V, i = e - r * V, kp = k0 + r;
            float v = 0.0f;
            if (kp < n_keys) {
                const int blk = bt[kp / page];
                if (blk >= 0 && blk < num_pages) v = to_float(v_pool[(((size_t)blk * G + kv) * page + kp % page) * V + i]);
            }
            vs[e] = v;
        }
        __syncthreads();
        // weights: thread (key kk, rows rg, rg + 4, ...)
#pragma unroll
        for (int m = 0; m < SA_ROWS / 4; m++) {
            const int r = rg + 4 * m;
            float sc = 0.0f;
            for (int i = 0; i < D; i++) sc = fmaf(qs[r * D + i], ks[kk * DP + i], sc);
            const bool seen = r < nq && k0 + kk <= pos0 + r;
            ws[r * SA_KEYS + kk] = seen ? 1.0f / (1.0f + expf(-(sc * scale + bias))) : 0.0f;
        }
        __syncthreads();
        const int last = min(SA_KEYS, n_keys - k0);
        for (int x = 0; x < last; x++) {
            float vv[CM];
#pragma unroll
            for (int m = 0; m < CM; m++) {
                const int c = threadIdx.x + m * SA_THREADS;
                vv[m] = c < V ? vs[x * V + c] : 0.0f;
            }
#pragma unroll
            for (int r = 0; r < SA_ROWS; r++) {
                const float w = ws[r * SA_KEYS + x];
#pragma unroll
                for (int m = 0; m < CM; m++) acc[r][m] = fmaf(w, vv[m], acc[r][m]);
            }
        }
    }
#pragma unroll
    for (int r = 0; r < SA_ROWS; r++) {
        if (r >= nq) break;
#pragma unroll
        for (int m = 0; m < CM; m++) {
            const int c = threadIdx.x + m * SA_THREADS;
            if (c < V) out[((size_t)(row0 + r) * H + h) * V + c] = from_float<T>(acc[r][m]);
        }
    }
}

template <typename T>
int launch_attend(const void* q, const void* k_pool, const void* v_pool, void* out, int H, int G, int D, int V,
                  const int* tiles, int n_tiles, const int* bt, int max_blocks, int page, int num_pages, float scale,
                  const float* head_bias, int* err, cudaStream_t st) {
    const size_t smem = ((size_t)SA_ROWS * D + (size_t)SA_KEYS * (D + 1) + (size_t)SA_KEYS * V + SA_ROWS * SA_KEYS) * sizeof(float);
    if (smem > 200 * 1024) return fail("sigmoid_attention: heads of %d / %d do not fit in shared memory", D, V);
    const int cm = (V + SA_THREADS - 1) / SA_THREADS;
#define EMBER_SA_LAUNCH(CM)                                                                                              \
    do {                                                                                                                 \
        if (smem > 48 * 1024)                                                                                            \
            cudaFuncSetAttribute(sigmoid_attention_kernel<T, CM>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
        launch_kernel(sigmoid_attention_kernel<T, CM>, dim3(n_tiles, H), SA_THREADS, smem, st, (const T*)q, (const T*)k_pool,  \
                      (const T*)v_pool, (T*)out, H, G, D, V, tiles, bt, max_blocks, page, num_pages, scale, head_bias, err); \
    } while (0)
    if (cm <= 1) EMBER_SA_LAUNCH(1);
    else if (cm == 2) EMBER_SA_LAUNCH(2);
    else if (cm <= 4) EMBER_SA_LAUNCH(4);
    else return fail("sigmoid_attention: value heads of %d are wider than 512", V);
#undef EMBER_SA_LAUNCH
    return check_launch("sigmoid_attention");
}

}  // namespace ember

using namespace ember;

EMBER_API int ember_sigmoid_attention_tile_queries() { return SA_ROWS; }

EMBER_API int ember_rotate_store(const float* qkv, int ld, int T, int H, int G, int D, int V, const float* inv_freq, int rotary,
                                 const int* positions, const int* seq_of, const int* block_table, int max_blocks, int page,
                                 int num_pages, void* q_out, void* k_pool, void* v_pool, int dtype, int write_kv, int* err,
                                 void* stream) {
    if (T <= 0) return 0;
    if (H <= 0 || G <= 0 || D <= 0 || V <= 0 || ld < (H + G) * D + G * V) return fail("rotate_store: %d/%d heads of %d / %d in rows of %d", H, G, D, V, ld);
    if (rotary < 0 || rotary > D || (rotary & 1) || (rotary && !inv_freq)) return fail("rotate_store: rotation of %d in heads of %d", rotary, D);
    if (page <= 0 || max_blocks <= 0 || num_pages <= 0) return fail("rotate_store: bad cache geometry");
    cudaStream_t st = (cudaStream_t)stream;
    const size_t smem = (size_t)(rotary > 0 ? rotary : 2) * sizeof(float);
    if (dtype == EMBER_F32)
        launch_kernel(rotate_store_kernel<float>, T, 256, smem, st, qkv, ld, H, G, D, V, inv_freq, rotary, positions, seq_of, block_table,
                      max_blocks, page, num_pages, (float*)q_out, (float*)k_pool, (float*)v_pool, write_kv, err);
    else if (dtype == EMBER_BF16)
        launch_kernel(rotate_store_kernel<__nv_bfloat16>, T, 256, smem, st, qkv, ld, H, G, D, V, inv_freq, rotary, positions, seq_of,
                      block_table, max_blocks, page, num_pages, (__nv_bfloat16*)q_out, (__nv_bfloat16*)k_pool, (__nv_bfloat16*)v_pool,
                      write_kv, err);
    else
        return fail("rotate_store: unsupported dtype %d", dtype);
    return check_launch("rotate_store");
}

EMBER_API int ember_sigmoid_attention(const void* q, const void* k_pool, const void* v_pool, void* out, int dtype, int H, int G,
                                      int D, int V, const int* tiles, int n_tiles, const int* block_table, int max_blocks, int page,
                                      int num_pages, float scale, const float* head_bias, int* err, void* stream) {
    if (n_tiles <= 0) return 0;
    if (H <= 0 || G <= 0 || H % G || D <= 0 || V <= 0) return fail("sigmoid_attention: %d/%d heads of %d / %d", H, G, D, V);
    if (H > 65535) return fail("sigmoid_attention: too many heads for one launch");
    cudaStream_t st = (cudaStream_t)stream;
    if (dtype == EMBER_F32)
        return launch_attend<float>(q, k_pool, v_pool, out, H, G, D, V, tiles, n_tiles, block_table, max_blocks, page, num_pages, scale, head_bias, err, st);
    if (dtype == EMBER_BF16)
        return launch_attend<__nv_bfloat16>(q, k_pool, v_pool, out, H, G, D, V, tiles, n_tiles, block_table, max_blocks, page, num_pages, scale, head_bias, err, st);
    return fail("sigmoid_attention: unsupported dtype %d", dtype);
}
