// Causal attention without softmax over a paged cache whose keys and values may differ in size:
//   weight(query i, key j <= i) = sigmoid(scale * q_i . k_j + bias[head]),   out_i = sum_j weight * v_j
// (weights are not normalised over keys).  Scores, weights and the sums are fp32.
//
// rotate_store: rotate-half rotation of the first `rotary` elements of every query and key head (pair (i, i +
// rotary / 2), angle = float(position) * inv_freq[i] in fp32), queries to q_out, keys and values into the request's
// pages: k_pool [pages, kv_heads, page, D], v_pool [pages, kv_heads, page, V].
// attend: one block per (tile of consecutive queries of a run, heads of one key/value head): 16 (token, head) rows;
// keys are walked in tiles of 32 in ascending order, so an output's sum has the same order however the tokens were
// cut into steps.
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

// 8 consecutive elements of a cache row as floats (16-byte loads where the row allows them)
__device__ __forceinline__ void load_row_chunk(const __nv_bfloat16* src, float* dst, int n, bool whole) {
    if (whole) {
        const uint4 u = *reinterpret_cast<const uint4*>(src);
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
        for (int i = 0; i < 4; i++) { const float2 f = __bfloat1622float2(h[i]); dst[2 * i] = f.x; dst[2 * i + 1] = f.y; }
    } else {
        for (int i = 0; i < n; i++) dst[i] = __bfloat162float(src[i]);
    }
}
__device__ __forceinline__ void load_row_chunk(const float* src, float* dst, int n, bool whole) {
    if (whole) {
        const float4 a = reinterpret_cast<const float4*>(src)[0], b = reinterpret_cast<const float4*>(src)[1];
        dst[0] = a.x; dst[1] = a.y; dst[2] = a.z; dst[3] = a.w; dst[4] = b.x; dst[5] = b.y; dst[6] = b.z; dst[7] = b.w;
    } else {
        for (int i = 0; i < n; i++) dst[i] = src[i];
    }
}

// A block's rows are (query token, query head) pairs of one key/value head: `hpb` heads (a divisor of the group, at
// most 16) of 16 / hpb consecutive tokens, so a decode step reads a request's keys once for all heads of the group
// and a prompt portion fills the 16 rows.  Scores: a thread takes one key and four rows, four elements at a time;
// read-out: a thread takes value columns tid, tid + 128, ... of all rows, four keys at a time.
// CM: value columns per thread (V <= 128 CM).  Head sizes that are multiples of 8 are fetched with 16-byte loads.
template <typename T, int CM>
__global__ void __launch_bounds__(SA_THREADS)
sigmoid_attention_kernel(const T* __restrict__ q, const T* __restrict__ k_pool, const T* __restrict__ v_pool,
                         T* __restrict__ out, int H, int G, int D, int V, int hpb, const int* __restrict__ tiles,
                         const int* __restrict__ block_table, int max_blocks, int page, int num_pages, float scale,
                         const float* __restrict__ head_bias, int* __restrict__ err) {
    extern __shared__ __align__(16) float smem[];
    pdl_launch_dependents();
    pdl_wait();
    const int* tile = tiles + 4 * blockIdx.x;
    const int run = tile[0], row0 = tile[1], nq = tile[2], pos0 = tile[3];
    const int h0 = blockIdx.y * hpb, kv = h0 / (H / G);
    const int n_rows = nq * hpb;                        // row rr: token rr / hpb, head h0 + rr % hpb
    const int DP = (D + 3) / 4 * 4 + 4, VP = (V + 3) / 4 * 4;
    float* qs = smem;                                   // [SA_ROWS][DP]
    float* ks = qs + SA_ROWS * DP;                      // [SA_KEYS][DP]
    float* vs = ks + SA_KEYS * DP;                      // [SA_KEYS][VP]
    float* ws = vs + SA_KEYS * VP;                      // [SA_ROWS][SA_KEYS]
    for (int e = threadIdx.x; e < SA_ROWS * DP; e += SA_THREADS) {
        const int r = e / DP, i = e - r * DP;
        qs[e] = (r < n_rows && i < D) ? to_float(q[((size_t)(row0 + r / hpb) * H + h0 + r % hpb) * D + i]) : 0.0f;
    }
    for (int e = threadIdx.x; e < SA_KEYS * (DP - D); e += SA_THREADS)       // the padding of key rows stays zero
        ks[(e / (DP - D)) * DP + D + e % (DP - D)] = 0.0f;
    float acc[SA_ROWS][CM];
#pragma unroll
    for (int r = 0; r < SA_ROWS; r++)
#pragma unroll
        for (int m = 0; m < CM; m++) acc[r][m] = 0.0f;
    const int n_keys = pos0 + nq;                       // keys 0 .. position of the last query
    const int* bt = block_table + (size_t)run * max_blocks;
    const int kk = threadIdx.x & 31, rg = threadIdx.x >> 5;
    const int dchunks = (D + 7) / 8, vchunks = (V + 7) / 8;
    const bool d8 = (D & 7) == 0, v8 = (V & 7) == 0;
    for (int k0 = 0; k0 < n_keys; k0 += SA_KEYS) {
        __syncthreads();
        // keys and values of this tile as floats (rows beyond the last key are zero)
        for (int e = threadIdx.x; e < SA_KEYS * dchunks; e += SA_THREADS) {
            const int r = e / dchunks, c = e - r * dchunks, kp = k0 + r, n = min(8, D - 8 * c);
            float* dst = ks + r * DP + 8 * c;
            const int blk = kp < n_keys ? bt[kp / page] : -1;
            if (blk >= 0 && blk < num_pages) {
                load_row_chunk(k_pool + (((size_t)blk * G + kv) * page + kp % page) * D + 8 * c, dst, n, d8);
            } else {
                if (kp < n_keys && err) atomicOr(err, EMBER_ERR_PAGE_RANGE);
                for (int i = 0; i < n; i++) dst[i] = 0.0f;
            }
        }
        for (int e = threadIdx.x; e < SA_KEYS * vchunks; e += SA_THREADS) {
            const int r = e / vchunks, c = e - r * vchunks, kp = k0 + r, n = min(8, V - 8 * c);
            float* dst = vs + r * VP + 8 * c;
            const int blk = kp < n_keys ? bt[kp / page] : -1;
            if (blk >= 0 && blk < num_pages) {
                load_row_chunk(v_pool + (((size_t)blk * G + kv) * page + kp % page) * V + 8 * c, dst, n, v8);
            } else {
                for (int i = 0; i < n; i++) dst[i] = 0.0f;
            }
        }
        __syncthreads();
        // weights: thread (key kk, rows rg, rg + 4, rg + 8, rg + 12)
        if (rg < n_rows) {
            float sc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
            const float4* kp4 = reinterpret_cast<const float4*>(ks + kk * DP);
            for (int i = 0; i < DP / 4 - 1; i++) {
                const float4 kx = kp4[i];
#pragma unroll
                for (int m = 0; m < 4; m++) {
                    const float4 qx = reinterpret_cast<const float4*>(qs + (rg + 4 * m) * DP)[i];
                    sc[m] = fmaf(qx.x, kx.x, fmaf(qx.y, kx.y, fmaf(qx.z, kx.z, fmaf(qx.w, kx.w, sc[m]))));
                }
            }
#pragma unroll
            for (int m = 0; m < 4; m++) {
                const int r = rg + 4 * m;
                const bool seen = r < n_rows && k0 + kk <= pos0 + r / hpb;
                const float b = head_bias ? head_bias[h0 + r % hpb] : 0.0f;
                ws[r * SA_KEYS + kk] = seen ? 1.0f / (1.0f + expf(-(sc[m] * scale + b))) : 0.0f;
            }
        }
        __syncthreads();
        for (int x = 0; x < SA_KEYS; x += 4) {
            if (k0 + x >= n_keys) break;
            float vv[4][CM];
#pragma unroll
            for (int y = 0; y < 4; y++)
#pragma unroll
                for (int m = 0; m < CM; m++) {
                    const int c = threadIdx.x + m * SA_THREADS;
                    vv[y][m] = c < V ? vs[(x + y) * VP + c] : 0.0f;
                }
#pragma unroll
            for (int r = 0; r < SA_ROWS; r++) {
                if (r >= n_rows) break;
                const float4 w = *reinterpret_cast<const float4*>(ws + r * SA_KEYS + x);
#pragma unroll
                for (int m = 0; m < CM; m++)
                    acc[r][m] = fmaf(w.w, vv[3][m], fmaf(w.z, vv[2][m], fmaf(w.y, vv[1][m], fmaf(w.x, vv[0][m], acc[r][m]))));
            }
        }
    }
#pragma unroll
    for (int r = 0; r < SA_ROWS; r++) {
        if (r >= n_rows) break;
#pragma unroll
        for (int m = 0; m < CM; m++) {
            const int c = threadIdx.x + m * SA_THREADS;
            if (c < V) out[((size_t)(row0 + r / hpb) * H + h0 + r % hpb) * V + c] = from_float<T>(acc[r][m]);
        }
    }
}

// Query heads per block: the largest divisor of the group that is at most 16.
inline int heads_per_block(int group) {
    int h = group < SA_ROWS ? group : SA_ROWS;
    while (group % h) h--;
    return h;
}

// ------------------------------------------------------------------------ bfloat16 cache: tensor-core tiles
// The same attention for bfloat16 queries and cache with head sizes the tiles take (D a multiple of 16, V of 32).
// q . k runs on the tensor cores (mma.sync m16n8k16, bf16 operands, fp32 accumulation: what the fp32 multiply-adds
// of the kernel above compute from the same bf16 values).  Scores, sigmoid and weights are fp32; for the weight x
// value product a weight is cut into three bf16 pieces p = p1 + p2 + p3 (24 bits of mantissa: the fp32 weight, not a
// rounded one) and the three products are added in the fp32 accumulator.  A block: 16 (token, head) rows, 64-key
// tiles fetched with cp.async into two buffers; warp w takes keys 16 w .. 16 w + 15 of a tile for the scores and a
// quarter of the value columns for the read-out; the weights pass through shared memory.
constexpr int TC_KEYS = 64;

__device__ __forceinline__ void mma_bf16_16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}
// the three bf16 pieces of two fp32 weights, packed pairwise
__device__ __forceinline__ void split3(float x, float y, uint32_t& p1, uint32_t& p2, uint32_t& p3) {
    const float x1 = __bfloat162float(__float2bfloat16_rn(x)), y1 = __bfloat162float(__float2bfloat16_rn(y));
    const float xr = x - x1, yr = y - y1;
    const float x2 = __bfloat162float(__float2bfloat16_rn(xr)), y2 = __bfloat162float(__float2bfloat16_rn(yr));
    p1 = pack_bf16(x1, y1); p2 = pack_bf16(x2, y2); p3 = pack_bf16(xr - x2, yr - y2);
}

template <int DK, int NBV>          // DK: most 16-element steps of a head (D <= 16 DK); NBV: most 8-column blocks a warp reads out
__global__ void __launch_bounds__(128)
sigmoid_attention_tc_kernel(const __nv_bfloat16* __restrict__ q, const __nv_bfloat16* __restrict__ k_pool,
                            const __nv_bfloat16* __restrict__ v_pool, __nv_bfloat16* __restrict__ out, int H, int G, int D,
                            int V, int hpb, const int* __restrict__ tiles, const int* __restrict__ block_table, int max_blocks,
                            int page, int num_pages, float scale, const float* __restrict__ head_bias, int* __restrict__ err) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    pdl_launch_dependents();
    pdl_wait();
    const int* tile = tiles + 4 * blockIdx.x;
    const int run = tile[0], row0 = tile[1], nq = tile[2], pos0 = tile[3];
    const int h0 = blockIdx.y * hpb, kv = h0 / (H / G);
    const int n_rows = nq * hpb;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, g = lane >> 2, c = lane & 3;
    const int DP = D + 8, VP = V + 8, PP = TC_KEYS + 8;            // row pitches in elements
    __nv_bfloat16* Ks = reinterpret_cast<__nv_bfloat16*>(smem_raw);                 // [2][64][DP]
    __nv_bfloat16* Vs = Ks + 2 * TC_KEYS * DP;                                      // [2][64][VP]
    __nv_bfloat16* Ps = Vs + 2 * TC_KEYS * VP;                                      // [3][16][PP]
    const int dk = D >> 4, vw = V >> 2, nbv = vw >> 3;              // steps of 16, columns and 8-column blocks per warp
    const int n_keys = pos0 + nq;
    const int* bt = block_table + (size_t)run * max_blocks;

    // a thread fetches pieces of one key row (two threads a row, 32 bytes side by side): one look at the block table
    auto fetch = [&](int k0, int buf) {
        const int dch = D >> 3, vch = V >> 3;                      // 16-byte chunks a row (both even)
        const int r = threadIdx.x >> 1, kp = k0 + r;
        const int blk = kp < n_keys ? bt[kp / page] : -1;
        const bool ok = blk >= 0 && blk < num_pages;
        if (!ok && kp < n_keys && err && (threadIdx.x & 1) == 0) atomicOr(err, EMBER_ERR_PAGE_RANGE);
        const size_t at = ok ? ((size_t)blk * G + kv) * page + kp % page : 0;
        const __nv_bfloat16* ksrc = k_pool + at * D;
        const __nv_bfloat16* vsrc = v_pool + at * V;
        __nv_bfloat16* kdst = Ks + ((size_t)buf * TC_KEYS + r) * DP;
        __nv_bfloat16* vdst = Vs + ((size_t)buf * TC_KEYS + r) * VP;
        for (int ch = threadIdx.x & 1; ch < dch + vch; ch += 2) {
            const bool is_k = ch < dch;
            __nv_bfloat16* dst = is_k ? kdst + 8 * ch : vdst + 8 * (ch - dch);
            if (ok) {
                const __nv_bfloat16* src = is_k ? ksrc + 8 * ch : vsrc + 8 * (ch - dch);
                asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src));
            } else {
                *reinterpret_cast<uint4*>(dst) = make_uint4(0u, 0u, 0u, 0u);
            }
        }
        asm volatile("cp.async.commit_group;\n" ::: "memory");
    };

    // the queries of rows g and g + 8 as A operands, kept for the whole key range
    uint32_t qa[DK][4];
    {
        const int r0 = g, r1 = g + 8;
        const __nv_bfloat16* q0 = q + ((size_t)(row0 + r0 / hpb) * H + h0 + r0 % hpb) * D;
        const __nv_bfloat16* q1 = q + ((size_t)(row0 + r1 / hpb) * H + h0 + r1 % hpb) * D;
#pragma unroll
        for (int ks = 0; ks < DK; ks++) {
            if (ks < dk) {
                qa[ks][0] = r0 < n_rows ? *reinterpret_cast<const uint32_t*>(q0 + ks * 16 + 2 * c) : 0u;
                qa[ks][1] = r1 < n_rows ? *reinterpret_cast<const uint32_t*>(q1 + ks * 16 + 2 * c) : 0u;
                qa[ks][2] = r0 < n_rows ? *reinterpret_cast<const uint32_t*>(q0 + ks * 16 + 8 + 2 * c) : 0u;
                qa[ks][3] = r1 < n_rows ? *reinterpret_cast<const uint32_t*>(q1 + ks * 16 + 8 + 2 * c) : 0u;
            }
        }
    }
    const float bias0 = (head_bias && g < n_rows) ? head_bias[h0 + g % hpb] : 0.0f;
    const float bias1 = (head_bias && g + 8 < n_rows) ? head_bias[h0 + (g + 8) % hpb] : 0.0f;
    const int qpos0 = pos0 + g / hpb, qpos1 = pos0 + (g + 8) / hpb;
    float acc[NBV][4];
#pragma unroll
    for (int nb = 0; nb < NBV; nb++) acc[nb][0] = acc[nb][1] = acc[nb][2] = acc[nb][3] = 0.0f;

    fetch(0, 0);
    int buf = 0;
    for (int k0 = 0; k0 < n_keys; k0 += TC_KEYS, buf ^= 1) {
        asm volatile("cp.async.wait_group 0;\n" ::: "memory");
        __syncthreads();                                            // the tile is in; the other buffer and P are free
        if (k0 + TC_KEYS < n_keys) fetch(k0 + TC_KEYS, buf ^ 1);
        const __nv_bfloat16* Kt = Ks + (size_t)buf * TC_KEYS * DP;
        const __nv_bfloat16* Vt = Vs + (size_t)buf * TC_KEYS * VP;
        // scores of this warp's 16 keys, their weights in three pieces to shared memory
#pragma unroll
        for (int nb = 0; nb < 2; nb++) {
            float sc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
            const __nv_bfloat16* krow = Kt + (size_t)(16 * warp + 8 * nb + g) * DP + 2 * c;
#pragma unroll
            for (int ks = 0; ks < DK; ks++) {
                if (ks < dk) {
                    const uint32_t b0 = *reinterpret_cast<const uint32_t*>(krow + ks * 16);
                    const uint32_t b1 = *reinterpret_cast<const uint32_t*>(krow + ks * 16 + 8);
                    mma_bf16_16816(sc, qa[ks], b0, b1);
                }
            }
            const int key = k0 + 16 * warp + 8 * nb + 2 * c;        // this thread's columns: key, key + 1
            float w[4];
#pragma unroll
            for (int i = 0; i < 4; i++) {
                const int kp = key + (i & 1), qp = i < 2 ? qpos0 : qpos1;
                const bool seen = (i < 2 ? g : g + 8) < n_rows && kp <= qp;
                w[i] = seen ? 1.0f / (1.0f + expf(-(sc[i] * scale + (i < 2 ? bias0 : bias1)))) : 0.0f;
            }
            uint32_t p1, p2, p3;
            const int col = 16 * warp + 8 * nb + 2 * c;
            split3(w[0], w[1], p1, p2, p3);
            *reinterpret_cast<uint32_t*>(Ps + (0 * 16 + g) * PP + col) = p1;
            *reinterpret_cast<uint32_t*>(Ps + (1 * 16 + g) * PP + col) = p2;
            *reinterpret_cast<uint32_t*>(Ps + (2 * 16 + g) * PP + col) = p3;
            split3(w[2], w[3], p1, p2, p3);
            *reinterpret_cast<uint32_t*>(Ps + (0 * 16 + g + 8) * PP + col) = p1;
            *reinterpret_cast<uint32_t*>(Ps + (1 * 16 + g + 8) * PP + col) = p2;
            *reinterpret_cast<uint32_t*>(Ps + (2 * 16 + g + 8) * PP + col) = p3;
        }
        __syncthreads();
        // read-out of this warp's value columns
        const int kbs = min(TC_KEYS, n_keys - k0 + 15) >> 4;        // 16-key steps that hold a visible key
#pragma unroll
        for (int kb = 0; kb < TC_KEYS / 16; kb++) {
            if (kb < kbs) {
                uint32_t pa[3][4];
#pragma unroll
                for (int part = 0; part < 3; part++) {
                    const __nv_bfloat16* pr = Ps + (size_t)(part * 16 + g) * PP + kb * 16 + 2 * c;
                    pa[part][0] = *reinterpret_cast<const uint32_t*>(pr);
                    pa[part][1] = *reinterpret_cast<const uint32_t*>(pr + 8 * PP);
                    pa[part][2] = *reinterpret_cast<const uint32_t*>(pr + 8);
                    pa[part][3] = *reinterpret_cast<const uint32_t*>(pr + 8 * PP + 8);
                }
#pragma unroll
                for (int nb = 0; nb < NBV; nb++) {
                    if (nb < nbv) {
                        uint32_t b0, b1;
                        const __nv_bfloat16* vrow = Vt + (size_t)(kb * 16 + (lane & 15)) * VP + warp * vw + nb * 8;
                        asm volatile("ldmatrix.sync.aligned.m8n8.x2.trans.shared.b16 {%0,%1}, [%2];\n"
                                     : "=r"(b0), "=r"(b1) : "r"((uint32_t)__cvta_generic_to_shared(vrow)));
                        mma_bf16_16816(acc[nb], pa[2], b0, b1);     // smallest pieces first
                        mma_bf16_16816(acc[nb], pa[1], b0, b1);
                        mma_bf16_16816(acc[nb], pa[0], b0, b1);
                    }
                }
            }
        }
    }
#pragma unroll
    for (int nb = 0; nb < NBV; nb++) {
        if (nb < nbv) {
            const int col = warp * vw + nb * 8 + 2 * c;
            if (g < n_rows)
                *reinterpret_cast<uint32_t*>(out + ((size_t)(row0 + g / hpb) * H + h0 + g % hpb) * V + col) = pack_bf16(acc[nb][0], acc[nb][1]);
            if (g + 8 < n_rows)
                *reinterpret_cast<uint32_t*>(out + ((size_t)(row0 + (g + 8) / hpb) * H + h0 + (g + 8) % hpb) * V + col) =
                    pack_bf16(acc[nb][2], acc[nb][3]);
        }
    }
}

inline bool tc_attend_on() {
    static int on = -1;
    if (on < 0) { const char* e = getenv("EMBER_SIGMOID_ATTENTION_TC"); on = (e && e[0] == '0') ? 0 : 1; }
    return on != 0;
}

template <int DK, int NBV>
int launch_attend_tc(const void* q, const void* k_pool, const void* v_pool, void* out, int H, int G, int D, int V, int hpb,
                     const int* tiles, int n_tiles, const int* bt, int max_blocks, int page, int num_pages, float scale,
                     const float* head_bias, int* err, cudaStream_t st) {
    const size_t smem = ((size_t)2 * TC_KEYS * (D + 8) + (size_t)2 * TC_KEYS * (V + 8) + 3 * 16 * (TC_KEYS + 8)) * sizeof(__nv_bfloat16);
    if (smem > 48 * 1024) cudaFuncSetAttribute(sigmoid_attention_tc_kernel<DK, NBV>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    launch_kernel(sigmoid_attention_tc_kernel<DK, NBV>, dim3(n_tiles, H / hpb), 128, smem, st, (const __nv_bfloat16*)q,
                  (const __nv_bfloat16*)k_pool, (const __nv_bfloat16*)v_pool, (__nv_bfloat16*)out, H, G, D, V, hpb, tiles, bt, max_blocks,
                  page, num_pages, scale, head_bias, err);
    return check_launch("sigmoid_attention");
}

template <typename T>
int launch_attend(const void* q, const void* k_pool, const void* v_pool, void* out, int H, int G, int D, int V,
                  const int* tiles, int n_tiles, const int* bt, int max_blocks, int page, int num_pages, float scale,
                  const float* head_bias, int* err, cudaStream_t st) {
    const int DP = (D + 3) / 4 * 4 + 4, VP = (V + 3) / 4 * 4, hpb = heads_per_block(H / G);
    const size_t smem = ((size_t)(SA_ROWS + SA_KEYS) * DP + (size_t)SA_KEYS * VP + SA_ROWS * SA_KEYS) * sizeof(float);
    if (smem > 200 * 1024) return fail("sigmoid_attention: heads of %d / %d do not fit in shared memory", D, V);
    const int cm = (V + SA_THREADS - 1) / SA_THREADS;
#define EMBER_SA_LAUNCH(CM)                                                                                              \
    do {                                                                                                                 \
        if (smem > 48 * 1024)                                                                                            \
            cudaFuncSetAttribute(sigmoid_attention_kernel<T, CM>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
        launch_kernel(sigmoid_attention_kernel<T, CM>, dim3(n_tiles, H / hpb), SA_THREADS, smem, st, (const T*)q, (const T*)k_pool, \
                      (const T*)v_pool, (T*)out, H, G, D, V, hpb, tiles, bt, max_blocks, page, num_pages, scale, head_bias, err); \
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

EMBER_API int ember_sigmoid_attention_tile_queries(int group) { return group > 0 ? SA_ROWS / heads_per_block(group) : 0; }

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
    if (dtype == EMBER_BF16 && tc_attend_on() && D % 16 == 0 && V % 32 == 0 && D <= 256 && V <= 512) {
        const int hpb = heads_per_block(H / G);
#define EMBER_SA_TC(DK, NBV) launch_attend_tc<DK, NBV>(q, k_pool, v_pool, out, H, G, D, V, hpb, tiles, n_tiles, block_table, \
                                                       max_blocks, page, num_pages, scale, head_bias, err, st)
        if (D <= 128) return V <= 128 ? EMBER_SA_TC(8, 4) : EMBER_SA_TC(8, 16);
        return V <= 128 ? EMBER_SA_TC(16, 4) : EMBER_SA_TC(16, 16);
#undef EMBER_SA_TC
    }
    if (dtype == EMBER_BF16)
        return launch_attend<__nv_bfloat16>(q, k_pool, v_pool, out, H, G, D, V, tiles, n_tiles, block_table, max_blocks, page, num_pages, scale, head_bias, err, st);
    return fail("sigmoid_attention: unsupported dtype %d", dtype);
}
