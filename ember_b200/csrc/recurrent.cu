// Recurrent mixers over a ragged batch: a short causal convolution whose last inputs are carried per request, and
// three matrix-state recurrences (delta rule with a decay per key channel, matrix memory with exponential gating,
// selective state space with a scalar decay per head).  Everything that enters a recurrence is fp32: decays and
// their logarithms, softplus and exponentials, gates, unit norms, the state itself.
//
// A step's tokens are S runs (query_start [S + 1]); run s belongs to state slot slots[s].  A recurrence kernel runs
// one block per (run, head, tile of value columns): the block holds its [keys x columns] tile of the state in shared
// memory, walks the run's tokens in order and writes the tile back, so a prompt portion and a single decoded token
// are the same code and the state after a step does not depend on how the tokens were cut into steps.
#include "common.cuh"

EMBER_DEFINE_LAST_ERROR

namespace ember {

__device__ __forceinline__ float sigmoidf_(float x) { return 1.0f / (1.0f + expf(-x)); }
__device__ __forceinline__ float softplusf_(float x) { return x > 20.0f ? x : log1pf(expf(x)); }
__device__ __forceinline__ float logsigmoidf_(float x) { return fminf(x, 0.0f) - log1pf(expf(-fabsf(x))); }

// ------------------------------------------------------------------------------- short causal convolution + silu
// out[t, c] = silu(bias[c] + sum_j taps[c, j] * in(t - (n - 1 - j), c)); inputs before the run come from the
// request's carried inputs carry[slot][j][c] (j = 0 the oldest of n - 1), zeros for a new request.
__global__ void conv_silu_kernel(const float* __restrict__ x, int ldx, int c0, const float* __restrict__ taps,
                                 const float* __restrict__ bias, int n, const float* __restrict__ carry, long long carry_stride,
                                 const int* __restrict__ seq_of, const int* __restrict__ query_start,
                                 const int* __restrict__ slots, float* __restrict__ out, int C) {
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.y, c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= C) return;
    const int s = seq_of[t], first = query_start[s];
    const float* cs = carry + (size_t)slots[s] * carry_stride;
    float acc = bias ? bias[c] : 0.0f;
    for (int j = 0; j < n; j++) {
        const int src = t - (n - 1 - j);
        const float v = src >= first ? x[(size_t)src * ldx + c0 + c] : cs[(size_t)(n - 1 + src - first) * C + c];
        acc = fmaf(taps[(size_t)c * n + j], v, acc);
    }
    out[(size_t)t * C + c] = acc / (1.0f + expf(-acc));
}

// After the convolution: the request's last n - 1 inputs (from the run, or shifted down from what was carried).
__global__ void conv_carry_kernel(const float* __restrict__ x, int ldx, int c0, int n, float* __restrict__ carry,
                                  long long carry_stride, const int* __restrict__ query_start, const int* __restrict__ slots, int C) {
    pdl_launch_dependents();
    pdl_wait();
    const int s = blockIdx.y, c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= C) return;
    const int first = query_start[s], end = query_start[s + 1];
    float* cs = carry + (size_t)slots[s] * carry_stride;
    for (int j = 0; j < n - 1; j++) {                       // ascending: entry j reads entries above j only
        const int src = end - (n - 1) + j;
        cs[(size_t)j * C + c] = src >= first ? x[(size_t)src * ldx + c0 + c] : cs[(size_t)(n - 1 + src - first) * C + c];
    }
}

// ------------------------------------------------------------------------------------------- state tiles
// Shared memory of a recurrence block: the state tile [D][VT] (VT = blockDim.x columns), then vectors.
__device__ __forceinline__ void load_tile(float* tile, const float* __restrict__ S, int D, int V, int j, bool live) {
    const int VT = blockDim.x;
    for (int i = 0; i < D; i++) tile[i * VT + threadIdx.x] = live ? S[(size_t)i * V + j] : 0.0f;
}
__device__ __forceinline__ void store_tile(const float* tile, float* __restrict__ S, int D, int V, int j, bool live) {
    const int VT = blockDim.x;
    if (live)
        for (int i = 0; i < D; i++) S[(size_t)i * V + j] = tile[i * VT + threadIdx.x];
}

// ---------------------------------------------------------------------- delta rule, one decay per key channel
// Per head (value head h reads query/key head h / (H / G)):
//   S <- diag(g) S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q
// with q, k unit vectors (q also times D^-1/2), beta = sigmoid(.), g = exp(-exp(A_log) softplus(a + dt_bias)).
struct DeltaArgs {
    const float* conv; int ld_conv;        // [T, G D | G D | H V] after convolution and silu
    const float* beta; int ld_beta;        // [T, H] logits
    const float* a; int ld_a;              // [T, H D] decay logits (before the bias)
    const float* dt_bias;                  // [H D]
    const float* A_log;                    // [H]
    float* state; long long state_stride;  // [slot][H][D][V]
    float* out;                            // [T, H V]
    const int* query_start; const int* slots;
    int H, G, D, V;
    float key_eps;
};

__global__ void delta_scan_kernel(DeltaArgs p) {
    extern __shared__ float smem[];
    pdl_launch_dependents();
    pdl_wait();
    const int s = blockIdx.x, h = blockIdx.y, VT = blockDim.x, j = blockIdx.z * VT + threadIdx.x;
    const int D = p.D, V = p.V, kv = h / (p.H / p.G);
    const bool live = j < V;
    float* tile = smem;                       // [D][VT]
    float* vec = smem + (size_t)D * VT;       // 2 x (k[D], q[D], g[D])
    float* red = vec + 6 * D;                 // 2 x 2 x 32 partial sums
    float* S = p.state + (size_t)p.slots[s] * p.state_stride + (size_t)h * D * V;
    load_tile(tile, S, D, V, j, live);
    const float rate = expf(p.A_log[h]), qscale = 1.0f / sqrtf((float)D);
    const int first = p.query_start[s], end = p.query_start[s + 1];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = VT >> 5;
    const int off_k = p.G * D, off_v = 2 * p.G * D;
    for (int t = first; t < end; t++) {
        const int b = (t - first) & 1;
        float* kb = vec + b * 3 * D, *qb = kb + D, *gb = qb + D;
        const float* row = p.conv + (size_t)t * p.ld_conv;
        float sk = 0.0f, sq = 0.0f;
        for (int i = threadIdx.x; i < D; i += VT) {
            const float kr = row[off_k + kv * D + i], qr = row[kv * D + i];
            kb[i] = kr; qb[i] = qr;
            sk = fmaf(kr, kr, sk); sq = fmaf(qr, qr, sq);
            gb[i] = expf(-rate * softplusf_(p.a[(size_t)t * p.ld_a + h * D + i] + p.dt_bias[h * D + i]));
        }
        sk = warp_sum(sk); sq = warp_sum(sq);
        if (lane == 0) { red[b * 64 + warp] = sk; red[b * 64 + 32 + warp] = sq; }
        __syncthreads();
        sk = 0.0f; sq = 0.0f;
        for (int w = 0; w < nwarps; w++) { sk += red[b * 64 + w]; sq += red[b * 64 + 32 + w]; }
        const float kn = 1.0f / sqrtf(sk + p.key_eps), qn = qscale / sqrtf(sq + p.key_eps);
        if (live) {
            const float beta = sigmoidf_(p.beta[(size_t)t * p.ld_beta + h]);
            const float v = row[off_v + h * V + j];
            float acc = 0.0f;
            for (int i = 0; i < D; i++) {
                const float x = tile[i * VT + threadIdx.x] * gb[i];
                tile[i * VT + threadIdx.x] = x;
                acc = fmaf(x, kb[i] * kn, acc);
            }
            const float u = beta * (v - acc);
            float o = 0.0f;
            for (int i = 0; i < D; i++) {
                const float x = fmaf(kb[i] * kn, u, tile[i * VT + threadIdx.x]);
                tile[i * VT + threadIdx.x] = x;
                o = fmaf(x, qb[i], o);
            }
            p.out[(size_t)t * p.H * V + h * V + j] = o * qn;
        }
    }
    store_tile(tile, S, D, V, j, live);
}

// ------------------------------------------------------------- matrix memory with exponential input gate
// Per head, with log gates i~ = cap tanh((i + b_i) / cap), f~ = logsigmoid(cap tanh((f + b_f) / cap)) and a running
// maximum m (0 for a new request):
//   m' = max(f~ + m, i~);  S <- e^(f~ + m - m') S + e^(i~ - m') k v^T;  n likewise with k;
//   o = S^T q / (max(|n . q|, e^(-m')) + 1e-6),  q scaled by D^-1/2.
// Two kernels: the first walks a run once per head and leaves (keep, put, denominator) per token, carrying n and m;
// the second applies them to the tiles of S.
struct MemoryArgs {
    const float* proj; int ld;             // [T, ...]: q, k (H D each), v (H V), input and forget logits (H each)
    int off_q, off_k, off_v, off_i, off_f;
    const float* bias_i; const float* bias_f;   // [H]
    float cap;
    float* state; long long state_stride;  // [slot]: S [H][D][V], then n [H][D], then m [H]
    float* gates;                          // [T, H, 3]: keep, put, denominator
    float* out;                            // [T, H V]
    const int* query_start; const int* slots;
    int H, D, V;
};

__global__ void memory_gates_kernel(MemoryArgs p) {
    extern __shared__ float smem[];           // n [D]
    __shared__ float scratch[32];
    pdl_launch_dependents();
    pdl_wait();
    const int s = blockIdx.x, h = blockIdx.y, D = p.D, H = p.H;
    float* base = p.state + (size_t)p.slots[s] * p.state_stride + (size_t)H * D * p.V;
    float* nst = base + (size_t)h * D;
    float* mst = base + (size_t)H * D + h;
    const int first = p.query_start[s], end = p.query_start[s + 1];
    for (int i = threadIdx.x; i < D; i += blockDim.x) smem[i] = nst[i];
    float m = *mst;
    const float qscale = 1.0f / sqrtf((float)D);
    for (int t = first; t < end; t++) {
        const float* row = p.proj + (size_t)t * p.ld;
        const float ig = p.cap * tanhf((row[p.off_i + h] + p.bias_i[h]) / p.cap);
        const float fg = logsigmoidf_(p.cap * tanhf((row[p.off_f + h] + p.bias_f[h]) / p.cap));
        const float m_new = fmaxf(fg + m, ig);
        const float keep = expf(fg + m - m_new), put = expf(ig - m_new);
        m = m_new;
        float nq = 0.0f;
        for (int i = threadIdx.x; i < D; i += blockDim.x) {          // a thread owns its entries of n
            const float n = fmaf(put, row[p.off_k + h * D + i], keep * smem[i]);
            smem[i] = n;
            nq = fmaf(n, row[p.off_q + h * D + i] * qscale, nq);
        }
        nq = block_sum(nq, scratch);
        if (threadIdx.x == 0) {
            float* g = p.gates + ((size_t)t * H + h) * 3;
            g[0] = keep; g[1] = put; g[2] = fmaxf(fabsf(nq), expf(-m)) + 1e-6f;
        }
    }
    if (first < end) {
        for (int i = threadIdx.x; i < D; i += blockDim.x) nst[i] = smem[i];
        if (threadIdx.x == 0) *mst = m;
    }
}

__global__ void memory_scan_kernel(MemoryArgs p) {
    extern __shared__ float smem[];
    pdl_launch_dependents();
    pdl_wait();
    const int s = blockIdx.x, h = blockIdx.y, VT = blockDim.x, j = blockIdx.z * VT + threadIdx.x;
    const int D = p.D, V = p.V, H = p.H;
    const bool live = j < V;
    float* tile = smem;                       // [D][VT]
    float* vec = smem + (size_t)D * VT;       // 2 x (k[D], q[D])
    float* S = p.state + (size_t)p.slots[s] * p.state_stride + (size_t)h * D * V;
    load_tile(tile, S, D, V, j, live);
    const int first = p.query_start[s], end = p.query_start[s + 1];
    const float qscale = 1.0f / sqrtf((float)D);
    for (int t = first; t < end; t++) {
        const int b = (t - first) & 1;
        float* kb = vec + b * 2 * D, *qb = kb + D;
        const float* row = p.proj + (size_t)t * p.ld;
        for (int i = threadIdx.x; i < D; i += VT) {
            kb[i] = row[p.off_k + h * D + i];
            qb[i] = row[p.off_q + h * D + i] * qscale;
        }
        const float* g = p.gates + ((size_t)t * H + h) * 3;
        const float keep = g[0], put = g[1], den = g[2];
        __syncthreads();
        if (live) {
            const float pv = put * row[p.off_v + h * V + j];
            float o = 0.0f;
            for (int i = 0; i < D; i++) {
                const float x = fmaf(kb[i], pv, keep * tile[i * VT + threadIdx.x]);
                tile[i * VT + threadIdx.x] = x;
                o = fmaf(x, qb[i], o);
            }
            p.out[(size_t)t * H * V + h * V + j] = o / den;
        }
    }
    store_tile(tile, S, D, V, j, live);
}

// ------------------------------------------------------------------- selective state space, scalar decay per head
// Per head (head h reads B, C of group h / (H / G)), dt = softplus(dt_raw + dt_bias):
//   S <- e^(-e^(A_log) dt) S + dt B x^T  (S is N x V);  y = S^T C + D_skip x.
struct SsmArgs {
    const float* conv; int ld_conv;        // [T, H V | G N | G N] after convolution and silu: x, B, C
    const float* dt; int ld_dt;            // [T, H] raw step sizes
    const float* dt_bias; const float* A_log; const float* skip;   // [H]
    float* state; long long state_stride;  // [slot][H][N][V]
    float* out;                            // [T, H V]
    const int* query_start; const int* slots;
    int H, G, N, V;
};

__global__ void ssm_scan_kernel(SsmArgs p) {
    extern __shared__ float smem[];
    pdl_launch_dependents();
    pdl_wait();
    const int s = blockIdx.x, h = blockIdx.y, VT = blockDim.x, j = blockIdx.z * VT + threadIdx.x;
    const int N = p.N, V = p.V, H = p.H, g = h / (H / p.G);
    const bool live = j < V;
    float* tile = smem;                       // [N][VT]
    float* vec = smem + (size_t)N * VT;       // 2 x (B[N], C[N])
    float* S = p.state + (size_t)p.slots[s] * p.state_stride + (size_t)h * N * V;
    load_tile(tile, S, N, V, j, live);
    const float rate = expf(p.A_log[h]), bias = p.dt_bias[h], skip = p.skip[h];
    const int first = p.query_start[s], end = p.query_start[s + 1];
    const int off_b = H * V + g * N, off_c = H * V + p.G * N + g * N;
    for (int t = first; t < end; t++) {
        const int b = (t - first) & 1;
        float* Bb = vec + b * 2 * N, *Cb = Bb + N;
        const float* row = p.conv + (size_t)t * p.ld_conv;
        for (int i = threadIdx.x; i < N; i += VT) { Bb[i] = row[off_b + i]; Cb[i] = row[off_c + i]; }
        const float dt = softplusf_(p.dt[(size_t)t * p.ld_dt + h] + bias);
        const float keep = expf(-rate * dt);
        __syncthreads();
        if (live) {
            const float x = row[h * V + j], dx = dt * x;
            float y = 0.0f;
            for (int i = 0; i < N; i++) {
                const float v = fmaf(Bb[i], dx, keep * tile[i * VT + threadIdx.x]);
                tile[i * VT + threadIdx.x] = v;
                y = fmaf(v, Cb[i], y);
            }
            p.out[(size_t)t * H * V + h * V + j] = fmaf(skip, x, y);
        }
    }
    store_tile(tile, S, N, V, j, live);
}

// Columns per block: whole warps, at most 128, fewer while the state tile would not fit in shared memory.
inline int pick_columns(int D, int V, int extra_floats, size_t* smem) {
    int warps = (V + 31) / 32;
    if (warps > 4) warps = 4;
    while (warps > 1 && ((size_t)D * warps * 32 + extra_floats) * sizeof(float) > 96 * 1024) warps--;
    *smem = ((size_t)D * warps * 32 + extra_floats) * sizeof(float);
    return warps * 32;
}

template <typename K>
inline int allow_smem(K kernel, size_t smem, const char* what) {
    if (smem > 200 * 1024) return fail("%s: a state tile of %zu bytes does not fit in shared memory", what, smem);
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return fail("%s: %s", what, cudaGetErrorString(e));
    }
    return 0;
}

}  // namespace ember

using namespace ember;

EMBER_API int ember_conv_silu(const float* x, int ldx, int c0, const float* taps, const float* bias, int n, float* carry,
                              long long carry_stride, const int* seq_of, const int* query_start, const int* slots, float* out,
                              int T, int S, int C, void* stream) {
    if (T <= 0 || S <= 0) return 0;
    if (C <= 0 || n < 1 || n > 64 || ldx < c0 + C) return fail("conv_silu: %d channels from column %d in rows of %d, %d taps", C, c0, ldx, n);
    if (T > 65535 || S > 65535) return fail("conv_silu: %d tokens in %d runs are too many for one launch", T, S);
    cudaStream_t st = (cudaStream_t)stream;
    const unsigned bx = (unsigned)((C + 127) / 128);
    launch_kernel(conv_silu_kernel, dim3(bx, T), 128, 0, st, x, ldx, c0, taps, bias, n, (const float*)carry, carry_stride, seq_of,
                  query_start, slots, out, C);
    if (n > 1)
        launch_kernel(conv_carry_kernel, dim3(bx, S), 128, 0, st, x, ldx, c0, n, carry, carry_stride, query_start, slots, C);
    return check_launch("conv_silu");
}

EMBER_API int ember_delta_scan(const float* conv, int ld_conv, const float* beta, int ld_beta, const float* a, int ld_a,
                               const float* dt_bias, const float* A_log, float* state, long long state_stride, float* out,
                               const int* query_start, const int* slots, int S, int H, int G, int D, int V, float key_eps,
                               void* stream) {
    if (S <= 0) return 0;
    if (H <= 0 || G <= 0 || H % G || D <= 0 || V <= 0) return fail("delta_scan: %d/%d heads of %d x %d", H, G, D, V);
    if (S > 65535 || H > 65535) return fail("delta_scan: too many runs or heads for one launch");
    size_t smem;
    const int VT = pick_columns(D, V, 6 * D + 128, &smem);
    if (allow_smem(delta_scan_kernel, smem, "delta_scan")) return 1;
    DeltaArgs p{conv, ld_conv, beta, ld_beta, a, ld_a, dt_bias, A_log, state, state_stride, out, query_start, slots, H, G, D, V, key_eps};
    launch_kernel(delta_scan_kernel, dim3(S, H, (V + VT - 1) / VT), VT, smem, (cudaStream_t)stream, p);
    return check_launch("delta_scan");
}

EMBER_API int ember_memory_scan(const float* proj, int ld, int off_q, int off_k, int off_v, int off_i, int off_f,
                                const float* bias_i, const float* bias_f, float cap, float* state, long long state_stride,
                                float* gates, float* out, const int* query_start, const int* slots, int S, int H, int D, int V,
                                void* stream) {
    if (S <= 0) return 0;
    if (H <= 0 || D <= 0 || V <= 0 || !(cap > 0.0f)) return fail("memory_scan: %d heads of %d x %d, cap %g", H, D, V, cap);
    if (S > 65535 || H > 65535) return fail("memory_scan: too many runs or heads for one launch");
    size_t smem;
    const int VT = pick_columns(D, V, 4 * D, &smem);
    if (allow_smem(memory_scan_kernel, smem, "memory_scan")) return 1;
    if (allow_smem(memory_gates_kernel, (size_t)D * sizeof(float), "memory_scan")) return 1;
    MemoryArgs p{proj, ld, off_q, off_k, off_v, off_i, off_f, bias_i, bias_f, cap, state, state_stride, gates, out, query_start, slots, H, D, V};
    const int gate_threads = D >= 256 ? 256 : (D + 31) / 32 * 32;
    launch_kernel(memory_gates_kernel, dim3(S, H), gate_threads, (size_t)D * sizeof(float), (cudaStream_t)stream, p);
    launch_kernel(memory_scan_kernel, dim3(S, H, (V + VT - 1) / VT), VT, smem, (cudaStream_t)stream, p);
    return check_launch("memory_scan");
}

EMBER_API int ember_ssm_scan(const float* conv, int ld_conv, const float* dt, int ld_dt, const float* dt_bias, const float* A_log,
                             const float* skip, float* state, long long state_stride, float* out, const int* query_start,
                             const int* slots, int S, int H, int G, int N, int V, void* stream) {
    if (S <= 0) return 0;
    if (H <= 0 || G <= 0 || H % G || N <= 0 || V <= 0) return fail("ssm_scan: %d heads in %d groups, state %d x %d", H, G, N, V);
    if (S > 65535 || H > 65535) return fail("ssm_scan: too many runs or heads for one launch");
    size_t smem;
    const int VT = pick_columns(N, V, 4 * N, &smem);
    if (allow_smem(ssm_scan_kernel, smem, "ssm_scan")) return 1;
    SsmArgs p{conv, ld_conv, dt, ld_dt, dt_bias, A_log, skip, state, state_stride, out, query_start, slots, H, G, N, V};
    launch_kernel(ssm_scan_kernel, dim3(S, H, (V + VT - 1) / VT), VT, smem, (cudaStream_t)stream, p);
    return check_launch("ssm_scan");
}
