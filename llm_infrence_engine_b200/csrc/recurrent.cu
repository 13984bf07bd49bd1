// Mixers that carry a state of fixed size from token to token: the short causal convolution, the gated delta rule with a
// decay per key channel, and the state-space recurrence with a decay per head. T is the storage type of the projections
// (float or bfloat16); decays, step sizes, gates, unit norms and the states themselves are 32-bit.
//
// A step's batch is ragged: request r owns the rows seq_starts[r] .. seq_starts[r + 1] - 1, and its state lives in row
// seq_slots[r] of the state tensor (zeroed by the step when the request's first token is among the rows). The same kernels
// run a prompt portion of any length and a single decoded token: the recurrences walk their rows in order, so a position's
// result does not depend on how the request was cut into steps.
#include <math.h>

#include "common.cuh"

namespace {

__device__ __forceinline__ float softplus_f(float x) { return x > 20.f ? x : log1pf(expf(x)); }
__device__ __forceinline__ float sigmoid_f(float x) { return 1.0f / (1.0f + expf(-x)); }
__device__ __forceinline__ float silu_f(float x) { return x / (1.0f + expf(-x)); }

constexpr int CONV_MAX_TAPS = 8;
constexpr int CONV_CHUNK = 32;   // tokens of one request that a block walks; at least CONV_MAX_TAPS - 1

// y[t, c] = act(bias[c] + sum_j w[c, j] * u[t - taps + 1 + j, c]) over the rows of each request, where u before the step's
// first row comes from state[slot][taps - 1 + t][c] (t < 0: the request's last taps - 1 inputs of earlier steps) and the
// state is then moved on by the step's rows. A thread owns a channel; only the block of a request's first chunk reads the
// old state and writes the new one, each thread its own channel, so nothing races.
template <typename T>
__global__ void __launch_bounds__(128) causal_conv_kernel(const T* __restrict__ z, int z_stride, int C, const float* __restrict__ w,
                                                          const float* __restrict__ bias, float* __restrict__ state,
                                                          const int* __restrict__ seq_starts, const int* __restrict__ seq_slots,
                                                          T* __restrict__ out, int out_stride, int taps, int act) {
    pdl_trigger();
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    float wt[CONV_MAX_TAPS];
    float b = 0.f;
    if (c < C) {
#pragma unroll
        for (int j = 0; j < CONV_MAX_TAPS; ++j) wt[j] = j < taps ? w[(size_t)c * taps + j] : 0.f;
        if (bias) b = bias[c];
    }
    pdl_wait();
    if (c >= C) return;
    const int r = blockIdx.z;
    const int s0 = seq_starts[r], L = seq_starts[r + 1] - s0;
    const int t0 = blockIdx.y * CONV_CHUNK;
    if (t0 >= L) return;
    float* st = state + (size_t)seq_slots[r] * (taps - 1) * C + c;
    float old[CONV_MAX_TAPS - 1];
    if (t0 == 0) {
#pragma unroll
        for (int j = 0; j < CONV_MAX_TAPS - 1; ++j) old[j] = j < taps - 1 ? st[(size_t)j * C] : 0.f;
    }
    // win[j] = input at t - (taps - 1) + j for the token t being computed; shifted by one per token
    float win[CONV_MAX_TAPS];
#pragma unroll
    for (int j = 0; j < CONV_MAX_TAPS; ++j) win[j] = 0.f;
#pragma unroll
    for (int j = 0; j < CONV_MAX_TAPS - 1; ++j) {
        if (j < taps - 1) {
            const int t = t0 - (taps - 1) + j;   // the inputs before the chunk's first token
            win[j + 1] = t >= 0 ? to_f32(z[(size_t)(s0 + t) * z_stride + c]) : old[taps - 1 + t];
        }
    }
    const int t1 = min(L, t0 + CONV_CHUNK);
    for (int t = t0; t < t1; ++t) {
#pragma unroll
        for (int j = 0; j < CONV_MAX_TAPS - 1; ++j) win[j] = win[j + 1];
        const float u = to_f32(z[(size_t)(s0 + t) * z_stride + c]);
#pragma unroll
        for (int j = 0; j < CONV_MAX_TAPS; ++j)
            if (j == taps - 1) win[j] = u;
        float y = b;
#pragma unroll
        for (int j = 0; j < CONV_MAX_TAPS; ++j)
            if (j < taps) y = fmaf(wt[j], win[j], y);
        if (act == 1) y = silu_f(y);
        out[(size_t)(s0 + t) * out_stride + c] = from_f32<T>(y);
    }
    if (t0 == 0) {
        for (int i = 0; i < taps - 1; ++i) {
            const int t = L - (taps - 1) + i;
            st[(size_t)i * C] = t >= 0 ? to_f32(z[(size_t)(s0 + t) * z_stride + c]) : old[taps - 1 + t];
        }
    }
}

// ------------------------------------------------------------------------------------------------
// What the delta rule's recurrence reads, made from the projections in one parallel pass. One warp per (token, head):
//   decay[n, h, d] = exp(-exp(A_log[h]) * softplus(a[n, h, d] + dt_bias[h, d]))
//   (per_head: one decay per head, decay[n, h] = exp(-exp(A_log[h]) * softplus(a[n, h] + dt_bias[h])))
//   beta[n, h]     = sigmoid(b[n, h])
// and, by the first head of every key group g, the unit vectors
//   qn[n, g, :] = q / sqrt(sum q^2 + unit_eps) * q_scale,   kn[n, g, :] = k / sqrt(sum k^2 + unit_eps),   kq[n, g] = kn . qn
template <typename T>
__global__ void __launch_bounds__(128) delta_prepare_kernel(const T* __restrict__ qkv, int qkv_stride, int q_col, int k_col,
                                                            const T* __restrict__ a, int a_stride, const T* __restrict__ bsrc,
                                                            int b_stride, const float* __restrict__ A_log,
                                                            const float* __restrict__ dt_bias, float* __restrict__ qn,
                                                            float* __restrict__ kn, float* __restrict__ kq, float* __restrict__ decay,
                                                            float* __restrict__ beta, int N, int H, int G, int D, float q_scale,
                                                            float unit_eps, int per_head) {
    pdl_trigger();
    pdl_wait();
    const int item = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    if (item >= N * H) return;
    const int n = item / H, h = item % H;
    const float rate = expf(A_log[h]);
    if (per_head) {
        if (lane == 0) decay[(size_t)n * H + h] = expf(-rate * softplus_f(to_f32(a[(size_t)n * a_stride + h]) + dt_bias[h]));
    } else {
        for (int d = lane; d < D; d += 32) {
            const float x = to_f32(a[(size_t)n * a_stride + h * D + d]) + dt_bias[h * D + d];
            decay[((size_t)n * H + h) * D + d] = expf(-rate * softplus_f(x));
        }
    }
    if (lane == 0) beta[(size_t)n * H + h] = sigmoid_f(to_f32(bsrc[(size_t)n * b_stride + h]));
    const int per = H / G;
    if (h % per == 0) {
        const int g = h / per;
        const T* qr = qkv + (size_t)n * qkv_stride + q_col + g * D;
        const T* kr = qkv + (size_t)n * qkv_stride + k_col + g * D;
        float sq = 0.f, sk = 0.f, dot = 0.f;
        for (int d = lane; d < D; d += 32) {
            const float qv = to_f32(qr[d]), kv = to_f32(kr[d]);
            sq = fmaf(qv, qv, sq); sk = fmaf(kv, kv, sk); dot = fmaf(qv, kv, dot);
        }
        sq = warp_sum(sq); sk = warp_sum(sk); dot = warp_sum(dot);
        const float fq = q_scale / sqrtf(sq + unit_eps), fk = 1.0f / sqrtf(sk + unit_eps);
        for (int d = lane; d < D; d += 32) {
            qn[((size_t)n * G + g) * D + d] = to_f32(qr[d]) * fq;
            kn[((size_t)n * G + g) * D + d] = to_f32(kr[d]) * fk;
        }
        if (lane == 0) kq[(size_t)n * G + g] = dot * fq * fk;
    }
}

// ------------------------------------------------------------------------------------------------
// How both recurrences are laid out. Per head the state S is [D, DV] (D: key channels or state size). Its columns are
// independent of one another, and within a column a token's work is a sum over D, which sets the length of the chain from one
// token to the next: so PARTS lanes share a column (up to a whole warp for D of 128 and more), lane part j holding the entries
// d = 4 PARTS i + 4 j + c (c < 4) in registers; a warp owns 32 / PARTS columns, a block of eight warps 8 times that; a token
// costs D / PARTS steps per lane plus log2(PARTS) shuffles per sum. In memory a state is kept column by column ([DV][D]), so
// that a lane's entries are 16-byte pieces and a column's lanes read one contiguous run. Tokens arrive in tiles of SCAN_TILE
// through a two-stage ring in shared memory (the next tile lands while this one is worked on; rows padded with zeros to DMAX;
// the parts of a step read contiguous 16-byte pieces: no bank conflict), and with them the block's columns of the token's
// own input. The order of every sum is fixed by D alone, so a result does not depend on how many rows a step brings.
constexpr int SCAN_TILE = 8;    // (16 measured 6 % faster on a prompt of 2,048 rows and 15 to 60 % slower on decoded tokens)
constexpr int SCAN_THREADS = 256;
constexpr int SCAN_ALONE_ROWS = 64;   // steps whose longest request brings this many rows launch the scans alone

// The most lanes that may share a column for a padded size DMAX (a lane holds at least one 16-byte piece), and the lanes that do:
// as many as it takes to fill the device with one request's columns (heads x values), fewer where there are many columns, since every
// halving of the lanes halves the shuffles and the warps. The choice depends on the model's sizes alone, never on the batch or on the
// rows of a step: the order of a sum, and with it every bit of a result, is the same however a request is cut.
static inline int scan_parts(int dmax, int columns) {
    const int most = dmax >= 128 ? 32 : dmax / 4;
    int parts = most;
    while (parts > 8 && (long long)columns * parts > 65536) parts >>= 1;
    return parts;
}

__device__ __forceinline__ void cp_async16(void* dst, const void* src) {
    const uint32_t d = (uint32_t)__cvta_generic_to_shared(dst);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(d), "l"(src));
}
__device__ __forceinline__ void cp_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void cp_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }
template <int PARTS> __device__ __forceinline__ float parts_sum(float v) {
#pragma unroll
    for (int o = 1; o < PARTS; o <<= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// rows of `count` tokens, each D floats at src + (first + t) * stride, into dst[t][DMAX] (zeros beyond D)
template <int DMAX>
__device__ __forceinline__ void fetch_rows(float* dst, const float* __restrict__ src, size_t stride, int count, int D, bool vec) {
    constexpr int Q = DMAX / 4;
    for (int i = threadIdx.x; i < count * Q; i += SCAN_THREADS) {
        const int t = i / Q, d = (i % Q) * 4;
        float* o = dst + t * DMAX + d;
        const float* p = src + (size_t)t * stride + d;
        if (vec && d < D) {
            cp_async16(o, p);
        } else {
#pragma unroll
            for (int c = 0; c < 4; ++c) o[c] = d + c < D ? p[c] : 0.f;
        }
    }
}

// a lane's entries of its column of the state, from / to st[D] (the column's run in memory)
template <int DPL, int PARTS>
__device__ __forceinline__ void load_column(float* S, const float* st, int part, int D, bool live, bool vec) {
#pragma unroll
    for (int i = 0; i < DPL / 4; ++i) {
        const int d = 4 * PARTS * i + 4 * part;
        if (live && vec && d < D) {
            const float4 v = *reinterpret_cast<const float4*>(st + d);
            S[4 * i] = v.x; S[4 * i + 1] = v.y; S[4 * i + 2] = v.z; S[4 * i + 3] = v.w;
        } else {
#pragma unroll
            for (int c = 0; c < 4; ++c) S[4 * i + c] = (live && d + c < D) ? st[d + c] : 0.f;
        }
    }
}
template <int DPL, int PARTS>
__device__ __forceinline__ void store_column(const float* S, float* st, int part, int D, bool vec) {
#pragma unroll
    for (int i = 0; i < DPL / 4; ++i) {
        const int d = 4 * PARTS * i + 4 * part;
        if (vec && d < D) {
            *reinterpret_cast<float4*>(st + d) = make_float4(S[4 * i], S[4 * i + 1], S[4 * i + 2], S[4 * i + 3]);
        } else {
#pragma unroll
            for (int c = 0; c < 4; ++c)
                if (d + c < D) st[d + c] = S[4 * i + c];
        }
    }
}

// The gated delta rule. For every token, in order:
//   S <- decay (.) S (row d by decay[d]);  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q
// With S' = decay (.) S both products of a token are taken from S' in one pass over the registers: r = S'^T k and S'^T q, and
// then o = S'^T q + u (k . q), the last factor coming with the token. SCALAR: the decay is one number per token and head
// (decay [N, H]) and comes with the token's other numbers instead of as a row of D.
template <typename T, int DMAX, int PARTS, bool SCALAR>
__global__ void __launch_bounds__(SCAN_THREADS) delta_scan_kernel(const T* __restrict__ v, int v_stride, int v_col, const float* __restrict__ qn,
                                                                  const float* __restrict__ kn, const float* __restrict__ kq,
                                                                  const float* __restrict__ decay, const float* __restrict__ beta,
                                                                  float* __restrict__ state, const int* __restrict__ seq_starts,
                                                                  const int* __restrict__ seq_slots, float* __restrict__ out, int H, int G,
                                                                  int D, int DV) {
    constexpr int DPL = DMAX / PARTS, COLS = SCAN_THREADS / PARTS;
    extern __shared__ __align__(16) float scan_smem[];
    float* k_s = scan_smem;                              // [2][SCAN_TILE][DMAX]
    float* q_s = k_s + 2 * SCAN_TILE * DMAX;
    float* g_s = q_s + 2 * SCAN_TILE * DMAX;
    float* beta_s = g_s + 2 * SCAN_TILE * DMAX;          // [2][SCAN_TILE]
    float* kq_s = beta_s + 2 * SCAN_TILE;
    float* g1_s = kq_s + 2 * SCAN_TILE;                  // [2][SCAN_TILE]: the decay where it is one number per token
    float* v_s = g1_s + 2 * SCAN_TILE;                   // [2][SCAN_TILE][COLS]
    pdl_wait();
    const int part = threadIdx.x % PARTS;
    const int col = blockIdx.x * COLS + threadIdx.x / PARTS;
    const int h = blockIdx.y, r = blockIdx.z;
    const int g = h / (H / G);
    const bool live = col < DV;
    const bool vec = (D & 3) == 0;
    const int s0 = seq_starts[r], s1 = seq_starts[r + 1];
    float* st = state + (((size_t)seq_slots[r] * H + h) * DV + (live ? col : 0)) * D;
    float S[DPL];
    load_column<DPL, PARTS>(S, st, part, D, live, vec);
    auto fetch = [&](int base, int buf) {   // the rows of a tile: asynchronous copies
        const int count = min(SCAN_TILE, s1 - base);
        fetch_rows<DMAX>(k_s + buf * SCAN_TILE * DMAX, kn + ((size_t)base * G + g) * D, (size_t)G * D, count, D, vec);
        fetch_rows<DMAX>(q_s + buf * SCAN_TILE * DMAX, qn + ((size_t)base * G + g) * D, (size_t)G * D, count, D, vec);
        if constexpr (!SCALAR) fetch_rows<DMAX>(g_s + buf * SCAN_TILE * DMAX, decay + ((size_t)base * H + h) * D, (size_t)H * D, count, D, vec);
    };
    // A tile's numbers per token (beta, k . q) and the block's columns of v: loaded into registers a tile ahead, put into shared
    // memory after the tile's work, so that nobody waits for them. Thread i < SCAN_TILE holds token i's two numbers; the
    // threads from the end backwards hold v, VPT values each.
    constexpr int VPT = (SCAN_TILE * COLS + SCAN_THREADS - 1) / SCAN_THREADS;
    float pre_beta = 0.f, pre_kq = 0.f, pre_g = 1.f, pre_v[VPT];
    auto load_small = [&](int base) {
        const int count = min(SCAN_TILE, s1 - base);
        if (threadIdx.x < count) {
            pre_beta = beta[(size_t)(base + threadIdx.x) * H + h];
            pre_kq = kq[(size_t)(base + threadIdx.x) * G + g];
            if constexpr (SCALAR) pre_g = decay[(size_t)(base + threadIdx.x) * H + h];
        }
#pragma unroll
        for (int n = 0; n < VPT; ++n) {
            const int j = SCAN_THREADS - 1 - threadIdx.x + n * SCAN_THREADS;
            const int t = j / COLS, c = blockIdx.x * COLS + j % COLS;
            pre_v[n] = (j < count * COLS && c < DV) ? to_f32(v[(size_t)(base + t) * v_stride + v_col + h * DV + c]) : 0.f;
        }
    };
    auto store_small = [&](int buf) {
        if (threadIdx.x < SCAN_TILE) {
            beta_s[buf * SCAN_TILE + threadIdx.x] = pre_beta;
            kq_s[buf * SCAN_TILE + threadIdx.x] = pre_kq;
            if constexpr (SCALAR) g1_s[buf * SCAN_TILE + threadIdx.x] = pre_g;
        }
#pragma unroll
        for (int n = 0; n < VPT; ++n) {
            const int j = SCAN_THREADS - 1 - threadIdx.x + n * SCAN_THREADS;
            if (j < SCAN_TILE * COLS) v_s[buf * SCAN_TILE * COLS + j] = pre_v[n];
        }
    };
    const int my_col = threadIdx.x / PARTS;
    if (s0 < s1) {
        fetch(s0, 0);
        load_small(s0);
        store_small(0);
    }
    cp_commit();
    int buf = 0;
    for (int base = s0; base < s1; base += SCAN_TILE, buf ^= 1) {
        const int count = min(SCAN_TILE, s1 - base);
        const bool more = base + SCAN_TILE < s1;
        if (more) {
            fetch(base + SCAN_TILE, buf ^ 1);
            load_small(base + SCAN_TILE);
        }
        cp_commit();
        cp_wait<1>();
        __syncthreads();                       // this tile is in shared memory
        const float* kb = k_s + buf * SCAN_TILE * DMAX + 4 * part;
        const float* qb = q_s + buf * SCAN_TILE * DMAX + 4 * part;
        const float* gb = g_s + buf * SCAN_TILE * DMAX + 4 * part;
#pragma unroll
        for (int t = 0; t < SCAN_TILE; ++t) {
            if (t < count) {
                float rk0 = 0.f, rk1 = 0.f, rq0 = 0.f, rq1 = 0.f;
                float g1 = 1.f;
                if constexpr (SCALAR) g1 = g1_s[buf * SCAN_TILE + t];
#pragma unroll
                for (int i = 0; i < DPL / 4; ++i) {
                    const float4 k4 = *reinterpret_cast<const float4*>(kb + t * DMAX + 4 * PARTS * i);
                    const float4 q4 = *reinterpret_cast<const float4*>(qb + t * DMAX + 4 * PARTS * i);
                    const float4 g4 = SCALAR ? make_float4(g1, g1, g1, g1) : *reinterpret_cast<const float4*>(gb + t * DMAX + 4 * PARTS * i);
                    float* s = S + 4 * i;
                    s[0] *= g4.x; s[1] *= g4.y; s[2] *= g4.z; s[3] *= g4.w;
                    rk0 = fmaf(s[0], k4.x, rk0); rk1 = fmaf(s[1], k4.y, rk1); rk0 = fmaf(s[2], k4.z, rk0); rk1 = fmaf(s[3], k4.w, rk1);
                    rq0 = fmaf(s[0], q4.x, rq0); rq1 = fmaf(s[1], q4.y, rq1); rq0 = fmaf(s[2], q4.z, rq0); rq1 = fmaf(s[3], q4.w, rq1);
                }
                const float rk = parts_sum<PARTS>(rk0 + rk1), rq = parts_sum<PARTS>(rq0 + rq1);
                const float u = beta_s[buf * SCAN_TILE + t] * (v_s[(buf * SCAN_TILE + t) * COLS + my_col] - rk);
#pragma unroll
                for (int i = 0; i < DPL / 4; ++i) {
                    const float4 k4 = *reinterpret_cast<const float4*>(kb + t * DMAX + 4 * PARTS * i);
                    float* s = S + 4 * i;
                    s[0] = fmaf(k4.x, u, s[0]); s[1] = fmaf(k4.y, u, s[1]); s[2] = fmaf(k4.z, u, s[2]); s[3] = fmaf(k4.w, u, s[3]);
                }
                if (live && part == 0) out[(size_t)(base + t) * H * DV + h * DV + col] = fmaf(u, kq_s[buf * SCAN_TILE + t], rq);
            }
        }
        if (more) store_small(buf ^ 1);
        __syncthreads();                       // everyone is done with this stage before it is filled again
    }
    cp_wait<0>();
    // Only now may the next kernel's blocks move in: they would wait for this kernel's end, and a multiprocessor full of
    // waiting warps slowed this kernel's own long walk by a third (measured).
    pdl_trigger();
    if (live) store_column<DPL, PARTS>(S, st, part, D, vec);
}

// ------------------------------------------------------------------------------------------------
// The state-space recurrence with one decay per head. Per head, S is [NS, DV]; for every token, in order:
//   dt = softplus(dt_raw + dt_bias[h]);  S <- exp(-exp(A_log[h]) dt) S + dt B x^T;  y = S^T C + D[h] x
// B and C belong to the head's group and come straight from the convolution's result (type T), so their tiles are filled with
// plain loads a tile ahead; step size and decay are computed while a tile is loaded.
template <typename T, int NMAX, int PARTS>
__global__ void __launch_bounds__(SCAN_THREADS) ssm_scan_kernel(const T* __restrict__ xbc, int x_stride, int x_col, int b_col, int c_col,
                                                                const T* __restrict__ dt_raw, int dt_stride, const float* __restrict__ A_log,
                                                                const float* __restrict__ dt_bias, const float* __restrict__ Dskip,
                                                                float* __restrict__ state, const int* __restrict__ seq_starts,
                                                                const int* __restrict__ seq_slots, float* __restrict__ out, int H, int G,
                                                                int NS, int DV) {
    constexpr int DPL = NMAX / PARTS, COLS = SCAN_THREADS / PARTS;
    extern __shared__ __align__(16) float scan_smem[];
    float* b_s = scan_smem;                              // [2][SCAN_TILE][NMAX]
    float* c_s = b_s + 2 * SCAN_TILE * NMAX;
    float* a_s = c_s + 2 * SCAN_TILE * NMAX;             // [2][SCAN_TILE]
    float* dt_s = a_s + 2 * SCAN_TILE;
    float* x_s = dt_s + 2 * SCAN_TILE;                   // [2][SCAN_TILE][COLS]
    const int part = threadIdx.x % PARTS;
    const int col = blockIdx.x * COLS + threadIdx.x / PARTS;
    const int h = blockIdx.y, r = blockIdx.z;
    const int g = h / (H / G);
    const bool live = col < DV;
    const bool vec = (NS & 3) == 0;
    const float rate = expf(A_log[h]), bias = dt_bias[h], skip = Dskip[h];
    pdl_wait();
    const int s0 = seq_starts[r], s1 = seq_starts[r + 1];
    float* st = state + (((size_t)seq_slots[r] * H + h) * DV + (live ? col : 0)) * NS;
    float S[DPL];
    load_column<DPL, PARTS>(S, st, part, NS, live, vec);
    // A tile (B and C of its tokens, step size and decay, the block's columns of x) is loaded into registers a tile ahead and
    // put into shared memory after the tile's work, so that nobody waits for it.
    constexpr int BPT = (SCAN_TILE * NMAX + SCAN_THREADS - 1) / SCAN_THREADS;
    constexpr int XPT = (SCAN_TILE * COLS + SCAN_THREADS - 1) / SCAN_THREADS;
    float pre_b[BPT], pre_c[BPT], pre_x[XPT], pre_dt = 0.f;
    auto load_tile = [&](int base) {
        const int count = min(SCAN_TILE, s1 - base);
#pragma unroll
        for (int n = 0; n < BPT; ++n) {
            const int i = threadIdx.x + n * SCAN_THREADS;
            const int t = i / NMAX, d = i % NMAX;
            const bool in = t < count && d < NS;
            const size_t row = (size_t)(base + t) * x_stride;
            pre_b[n] = in ? to_f32(xbc[row + b_col + g * NS + d]) : 0.f;
            pre_c[n] = in ? to_f32(xbc[row + c_col + g * NS + d]) : 0.f;
        }
        if (threadIdx.x < count) pre_dt = to_f32(dt_raw[(size_t)(base + threadIdx.x) * dt_stride + h]);
#pragma unroll
        for (int n = 0; n < XPT; ++n) {
            const int j = SCAN_THREADS - 1 - threadIdx.x + n * SCAN_THREADS;
            const int t = j / COLS, c = blockIdx.x * COLS + j % COLS;
            pre_x[n] = (j < count * COLS && c < DV) ? to_f32(xbc[(size_t)(base + t) * x_stride + x_col + h * DV + c]) : 0.f;
        }
    };
    auto store_tile = [&](int buf) {
#pragma unroll
        for (int n = 0; n < BPT; ++n) {
            const int i = threadIdx.x + n * SCAN_THREADS;
            if (i < SCAN_TILE * NMAX) {
                b_s[buf * SCAN_TILE * NMAX + i] = pre_b[n];
                c_s[buf * SCAN_TILE * NMAX + i] = pre_c[n];
            }
        }
        if (threadIdx.x < SCAN_TILE) {
            const float dt = softplus_f(pre_dt + bias);
            dt_s[buf * SCAN_TILE + threadIdx.x] = dt;
            a_s[buf * SCAN_TILE + threadIdx.x] = expf(-rate * dt);
        }
#pragma unroll
        for (int n = 0; n < XPT; ++n) {
            const int j = SCAN_THREADS - 1 - threadIdx.x + n * SCAN_THREADS;
            if (j < SCAN_TILE * COLS) x_s[buf * SCAN_TILE * COLS + j] = pre_x[n];
        }
    };
    const int my_col = threadIdx.x / PARTS;
    if (s0 < s1) {
        load_tile(s0);
        store_tile(0);
    }
    int buf = 0;
    for (int base = s0; base < s1; base += SCAN_TILE, buf ^= 1) {
        const int count = min(SCAN_TILE, s1 - base);
        const bool more = base + SCAN_TILE < s1;
        __syncthreads();                       // this tile is in shared memory; everyone is done with the other stage
        if (more) load_tile(base + SCAN_TILE);
        const float* bb = b_s + buf * SCAN_TILE * NMAX + 4 * part;
        const float* cb = c_s + buf * SCAN_TILE * NMAX + 4 * part;
#pragma unroll
        for (int t = 0; t < SCAN_TILE; ++t) {
            if (t < count) {
                const float xv = x_s[(buf * SCAN_TILE + t) * COLS + my_col];
                const float a = a_s[buf * SCAN_TILE + t], u = dt_s[buf * SCAN_TILE + t] * xv;
                float y0 = 0.f, y1 = 0.f;
#pragma unroll
                for (int i = 0; i < DPL / 4; ++i) {
                    const float4 b4 = *reinterpret_cast<const float4*>(bb + t * NMAX + 4 * PARTS * i);
                    const float4 c4 = *reinterpret_cast<const float4*>(cb + t * NMAX + 4 * PARTS * i);
                    float* s = S + 4 * i;
                    s[0] = fmaf(a, s[0], b4.x * u); s[1] = fmaf(a, s[1], b4.y * u); s[2] = fmaf(a, s[2], b4.z * u); s[3] = fmaf(a, s[3], b4.w * u);
                    y0 = fmaf(s[0], c4.x, y0); y1 = fmaf(s[1], c4.y, y1); y0 = fmaf(s[2], c4.z, y0); y1 = fmaf(s[3], c4.w, y1);
                }
                const float y = parts_sum<PARTS>(y0 + y1);
                if (live && part == 0) out[(size_t)(base + t) * H * DV + h * DV + col] = fmaf(skip, xv, y);
            }
        }
        if (more) store_tile(buf ^ 1);         // (the other stage: nobody reads it before the next barrier)
    }
    pdl_trigger();                             // (not before: see the delta rule's kernel)
    if (live) store_column<DPL, PARTS>(S, st, part, NS, vec);
}

// ------------------------------------------------------------------------------------------------
// The selective scan with a state per channel and state index (the recurrence of Mamba). Per channel c, S[c] is NS numbers; for
// every token, in order:
//   dt = softplus(dt_raw[c] + dt_bias[c]);  S[c, n] <- exp(dt A[c, n]) S[c, n] + dt x[c] B[n];  y[c] = sum_n S[c, n] C[n] + D[c] x[c]
// with A = -exp(A_log) [C, NS], B and C shared by all channels of a token. The result leaves as y * silu(z) in the storage type.
// The layout is the one above with a channel in the place of a column: PARTS lanes share a channel, each with its entries of S and
// of A in registers; a block owns SCAN_THREADS / PARTS channels; tiles of SCAN_TILE tokens are loaded into registers a tile ahead.
template <typename T, int NMAX, int PARTS>
__global__ void __launch_bounds__(SCAN_THREADS) selective_scan_kernel(const T* __restrict__ x, int x_stride, const T* __restrict__ dt_raw, int dt_stride,
                                                                      const T* __restrict__ bc, int bc_stride, int b_col, int c_col,
                                                                      const T* __restrict__ z, int z_stride, const float* __restrict__ A_log,
                                                                      const float* __restrict__ dt_bias, const float* __restrict__ Dskip,
                                                                      float* __restrict__ state, const int* __restrict__ seq_starts,
                                                                      const int* __restrict__ seq_slots, T* __restrict__ out, int C, int NS) {
    constexpr int DPL = NMAX / PARTS, COLS = SCAN_THREADS / PARTS;
    extern __shared__ __align__(16) float scan_smem[];
    float* b_s = scan_smem;                              // [2][SCAN_TILE][NMAX]
    float* c_s = b_s + 2 * SCAN_TILE * NMAX;
    float* x_s = c_s + 2 * SCAN_TILE * NMAX;             // [2][SCAN_TILE][COLS]
    float* dt_s = x_s + 2 * SCAN_TILE * COLS;
    float* z_s = dt_s + 2 * SCAN_TILE * COLS;
    const int part = threadIdx.x % PARTS;
    const int my_col = threadIdx.x / PARTS;
    const int col = blockIdx.x * COLS + my_col;
    const int r = blockIdx.z;
    const bool live = col < C;
    const bool vec = (NS & 3) == 0;
    // the channel's rates and numbers do not depend on the kernel before: fetched before the wait
    float A[DPL];
    load_column<DPL, PARTS>(A, A_log + (size_t)(live ? col : 0) * NS, part, NS, live, vec);
#pragma unroll
    for (int i = 0; i < DPL; ++i) A[i] = -expf(A[i]);
    const float skip = live ? Dskip[col] : 0.f;
    pdl_wait();
    const int s0 = seq_starts[r], s1 = seq_starts[r + 1];
    float* st = state + ((size_t)seq_slots[r] * C + (live ? col : 0)) * NS;
    float S[DPL];
    load_column<DPL, PARTS>(S, st, part, NS, live, vec);
    constexpr int BPT = (SCAN_TILE * NMAX + SCAN_THREADS - 1) / SCAN_THREADS;
    constexpr int XPT = (SCAN_TILE * COLS + SCAN_THREADS - 1) / SCAN_THREADS;
    float pre_b[BPT], pre_c[BPT], pre_x[XPT], pre_dt[XPT], pre_z[XPT];
    auto load_tile = [&](int base) {
        const int count = min(SCAN_TILE, s1 - base);
#pragma unroll
        for (int n = 0; n < BPT; ++n) {
            const int i = threadIdx.x + n * SCAN_THREADS;
            const int t = i / NMAX, d = i % NMAX;
            const bool in = t < count && d < NS;
            const size_t row = (size_t)(base + t) * bc_stride;
            pre_b[n] = in ? to_f32(bc[row + b_col + d]) : 0.f;
            pre_c[n] = in ? to_f32(bc[row + c_col + d]) : 0.f;
        }
#pragma unroll
        for (int n = 0; n < XPT; ++n) {
            const int j = threadIdx.x + n * SCAN_THREADS;
            const int t = j / COLS, c = blockIdx.x * COLS + j % COLS;
            const bool in = j < count * COLS && c < C;
            pre_x[n] = in ? to_f32(x[(size_t)(base + t) * x_stride + c]) : 0.f;
            pre_z[n] = in ? to_f32(z[(size_t)(base + t) * z_stride + c]) : 0.f;
            pre_dt[n] = in ? softplus_f(to_f32(dt_raw[(size_t)(base + t) * dt_stride + c]) + dt_bias[c]) : 0.f;
        }
    };
    auto store_tile = [&](int buf) {
#pragma unroll
        for (int n = 0; n < BPT; ++n) {
            const int i = threadIdx.x + n * SCAN_THREADS;
            if (i < SCAN_TILE * NMAX) {
                b_s[buf * SCAN_TILE * NMAX + i] = pre_b[n];
                c_s[buf * SCAN_TILE * NMAX + i] = pre_c[n];
            }
        }
#pragma unroll
        for (int n = 0; n < XPT; ++n) {
            const int j = threadIdx.x + n * SCAN_THREADS;
            if (j < SCAN_TILE * COLS) {
                x_s[buf * SCAN_TILE * COLS + j] = pre_x[n];
                dt_s[buf * SCAN_TILE * COLS + j] = pre_dt[n];
                z_s[buf * SCAN_TILE * COLS + j] = pre_z[n];
            }
        }
    };
    if (s0 < s1) {
        load_tile(s0);
        store_tile(0);
    }
    int buf = 0;
    for (int base = s0; base < s1; base += SCAN_TILE, buf ^= 1) {
        const int count = min(SCAN_TILE, s1 - base);
        const bool more = base + SCAN_TILE < s1;
        __syncthreads();                       // this tile is in shared memory; everyone is done with the other stage
        if (more) load_tile(base + SCAN_TILE);
        const float* bb = b_s + buf * SCAN_TILE * NMAX + 4 * part;
        const float* cb = c_s + buf * SCAN_TILE * NMAX + 4 * part;
#pragma unroll
        for (int t = 0; t < SCAN_TILE; ++t) {
            if (t < count) {
                const float xv = x_s[(buf * SCAN_TILE + t) * COLS + my_col];
                const float dt = dt_s[(buf * SCAN_TILE + t) * COLS + my_col];
                const float u = dt * xv;
                float y0 = 0.f, y1 = 0.f;
#pragma unroll
                for (int i = 0; i < DPL / 4; ++i) {
                    const float4 b4 = *reinterpret_cast<const float4*>(bb + t * NMAX + 4 * PARTS * i);
                    const float4 c4 = *reinterpret_cast<const float4*>(cb + t * NMAX + 4 * PARTS * i);
                    float* sp = S + 4 * i;
                    const float* ap = A + 4 * i;
                    sp[0] = fmaf(expf(dt * ap[0]), sp[0], b4.x * u); sp[1] = fmaf(expf(dt * ap[1]), sp[1], b4.y * u);
                    sp[2] = fmaf(expf(dt * ap[2]), sp[2], b4.z * u); sp[3] = fmaf(expf(dt * ap[3]), sp[3], b4.w * u);
                    y0 = fmaf(sp[0], c4.x, y0); y1 = fmaf(sp[1], c4.y, y1); y0 = fmaf(sp[2], c4.z, y0); y1 = fmaf(sp[3], c4.w, y1);
                }
                const float y = parts_sum<PARTS>(y0 + y1);
                if (live && part == 0) {
                    const float zv = z_s[(buf * SCAN_TILE + t) * COLS + my_col];
                    out[(size_t)(base + t) * C + col] = from_f32<T>(fmaf(skip, xv, y) * silu_f(zv));
                }
            }
        }
        if (more) store_tile(buf ^ 1);         // (the other stage: nobody reads it before the next barrier)
    }
    pdl_trigger();                             // (not before: see the delta rule's kernel)
    if (live) store_column<DPL, PARTS>(S, st, part, NS, vec);
}

template <typename T>
int launch_conv(const T* z, int z_stride, int C, const float* w, const float* bias, float* state, const int* seq_starts,
                const int* seq_slots, T* out, int out_stride, int taps, int act, int R, int max_rows, cudaStream_t s) {
    const dim3 grid((C + 127) / 128, (max_rows + CONV_CHUNK - 1) / CONV_CHUNK, R);
    return launch_kernel(causal_conv_kernel<T>, grid, dim3(128), 0, s, z, z_stride, C, w, bias, state, seq_starts, seq_slots, out,
                         out_stride, taps, act);
}

template <typename T, int DM, int PARTS, bool SCALAR>
int launch_delta_scan_one(const T* v, int v_stride, int v_col, const float* qn, const float* kn, const float* kq, const float* decay,
                          const float* beta, float* state, const int* seq_starts, const int* seq_slots, float* out, int H, int G, int D, int DV,
                          int R, bool alone, cudaStream_t s) {
    constexpr int cols = SCAN_THREADS / PARTS;
    const dim3 grid((DV + cols - 1) / cols, H, R);
    const size_t smem = sizeof(float) * (2 * SCAN_TILE * (3 * DM + 3 + cols));
    if (smem > 48 * 1024) cudaFuncSetAttribute(delta_scan_kernel<T, DM, PARTS, SCALAR>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    return launch_kernel_on(alone, delta_scan_kernel<T, DM, PARTS, SCALAR>, grid, dim3(SCAN_THREADS), smem, s, v, v_stride, v_col, qn, kn, kq, decay,
                            beta, state, seq_starts, seq_slots, out, H, G, D, DV);
}

template <typename T, int DM, int PARTS>
int launch_delta_scan_as(const T* v, int v_stride, int v_col, const float* qn, const float* kn, const float* kq, const float* decay,
                         const float* beta, float* state, const int* seq_starts, const int* seq_slots, float* out, int H, int G, int D, int DV,
                         int R, bool alone, bool scalar, cudaStream_t s) {
    if (scalar)
        return launch_delta_scan_one<T, DM, PARTS, true>(v, v_stride, v_col, qn, kn, kq, decay, beta, state, seq_starts, seq_slots, out, H, G, D, DV, R, alone, s);
    return launch_delta_scan_one<T, DM, PARTS, false>(v, v_stride, v_col, qn, kn, kq, decay, beta, state, seq_starts, seq_slots, out, H, G, D, DV, R, alone, s);
}

template <typename T, int NM, int PARTS>
int launch_ssm_scan_as(const T* xbc, int x_stride, int x_col, int b_col, int c_col, const T* dt_raw, int dt_stride, const float* A_log,
                       const float* dt_bias, const float* Dskip, float* state, const int* seq_starts, const int* seq_slots, float* out, int H,
                       int G, int NS, int DV, int R, bool alone, cudaStream_t s) {
    constexpr int cols = SCAN_THREADS / PARTS;
    const dim3 grid((DV + cols - 1) / cols, H, R);
    const size_t smem = sizeof(float) * (2 * SCAN_TILE * (2 * NM + 2 + cols));
    if (smem > 48 * 1024) cudaFuncSetAttribute(ssm_scan_kernel<T, NM, PARTS>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    return launch_kernel_on(alone, ssm_scan_kernel<T, NM, PARTS>, grid, dim3(SCAN_THREADS), smem, s, xbc, x_stride, x_col, b_col, c_col, dt_raw,
                            dt_stride, A_log, dt_bias, Dskip, state, seq_starts, seq_slots, out, H, G, NS, DV);
}

// the padded size (16, 32, 64, 128 or 256) and the lanes per column (scan_parts) pick the instantiation
#define LLMIE_SCAN_DISPATCH(FN, SIZE, ...)                                                    \
    {                                                                                         \
        const int dm = SIZE <= 16 ? 16 : SIZE <= 32 ? 32 : SIZE <= 64 ? 64 : SIZE <= 128 ? 128 : 256; \
        const int parts = scan_parts(dm, H * DV);                                             \
        if (dm == 16) return FN<T, 16, 4>(__VA_ARGS__);                                       \
        if (dm == 32) return FN<T, 32, 8>(__VA_ARGS__);                                       \
        if (dm == 64) return parts == 16 ? FN<T, 64, 16>(__VA_ARGS__) : FN<T, 64, 8>(__VA_ARGS__); \
        if (dm == 128)                                                                        \
            return parts == 32 ? FN<T, 128, 32>(__VA_ARGS__) : parts == 16 ? FN<T, 128, 16>(__VA_ARGS__) : FN<T, 128, 8>(__VA_ARGS__); \
        return parts == 32 ? FN<T, 256, 32>(__VA_ARGS__) : parts == 16 ? FN<T, 256, 16>(__VA_ARGS__) : FN<T, 256, 8>(__VA_ARGS__); \
    }

template <typename T>
int launch_delta_scan(const T* v, int v_stride, int v_col, const float* qn, const float* kn, const float* kq, const float* decay,
                      const float* beta, float* state, const int* seq_starts, const int* seq_slots, float* out, int H, int G, int D,
                      int DV, int R, bool alone, bool scalar, cudaStream_t s) {
    LLMIE_SCAN_DISPATCH(launch_delta_scan_as, D, v, v_stride, v_col, qn, kn, kq, decay, beta, state, seq_starts, seq_slots, out, H, G, D, DV, R, alone, scalar, s)
}

template <typename T>
int launch_ssm_scan(const T* xbc, int x_stride, int x_col, int b_col, int c_col, const T* dt_raw, int dt_stride, const float* A_log,
                    const float* dt_bias, const float* Dskip, float* state, const int* seq_starts, const int* seq_slots, float* out,
                    int H, int G, int NS, int DV, int R, bool alone, cudaStream_t s) {
    LLMIE_SCAN_DISPATCH(launch_ssm_scan_as, NS, xbc, x_stride, x_col, b_col, c_col, dt_raw, dt_stride, A_log, dt_bias, Dskip, state, seq_starts,
                        seq_slots, out, H, G, NS, DV, R, alone, s)
}

template <typename T, int NM, int PARTS>
int launch_selective_scan_as(const T* x, int x_stride, const T* dt_raw, int dt_stride, const T* bc, int bc_stride, int b_col, int c_col, const T* z,
                             int z_stride, const float* A_log, const float* dt_bias, const float* Dskip, float* state, const int* seq_starts,
                             const int* seq_slots, T* out, int C, int NS, int R, bool alone, cudaStream_t s) {
    constexpr int cols = SCAN_THREADS / PARTS;
    const dim3 grid((C + cols - 1) / cols, 1, R);
    const size_t smem = sizeof(float) * (2 * SCAN_TILE * (2 * NM + 3 * cols));
    if (smem > 48 * 1024) cudaFuncSetAttribute(selective_scan_kernel<T, NM, PARTS>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    return launch_kernel_on(alone, selective_scan_kernel<T, NM, PARTS>, grid, dim3(SCAN_THREADS), smem, s, x, x_stride, dt_raw, dt_stride, bc, bc_stride,
                            b_col, c_col, z, z_stride, A_log, dt_bias, Dskip, state, seq_starts, seq_slots, out, C, NS);
}

template <typename T>
int launch_selective_scan(const T* x, int x_stride, const T* dt_raw, int dt_stride, const T* bc, int bc_stride, int b_col, int c_col, const T* z,
                          int z_stride, const float* A_log, const float* dt_bias, const float* Dskip, float* state, const int* seq_starts,
                          const int* seq_slots, T* out, int C, int NS, int R, bool alone, cudaStream_t s) {
    const int H = C, DV = 1;   // (the channels are the columns that fill the device)
    LLMIE_SCAN_DISPATCH(launch_selective_scan_as, NS, x, x_stride, dt_raw, dt_stride, bc, bc_stride, b_col, c_col, z, z_stride, A_log, dt_bias, Dskip,
                        state, seq_starts, seq_slots, out, C, NS, R, alone, s)
}

}  // namespace

// z: columns 0 .. C - 1 of rows of z_stride elements (the caller offsets the pointer); state [slots][taps - 1][C] float.
LLMIE_API int llmie_causal_conv(const void* z, int z_stride, int C, const float* w, const float* bias, float* state,
                                const int* seq_starts, const int* seq_slots, void* out, int out_stride, int taps, int act, int R,
                                int max_rows, int dtype, cudaStream_t s) {
    if (R <= 0 || max_rows <= 0 || C <= 0) return 0;
    if (taps < 1 || taps > CONV_MAX_TAPS || R > 65535 || (max_rows + CONV_CHUNK - 1) / CONV_CHUNK > 65535 || act < 0 || act > 1)
        return LLMIE_ERR_BAD_ARGUMENT;
    if (dtype == DT_F32)
        return launch_conv<float>((const float*)z, z_stride, C, w, bias, state, seq_starts, seq_slots, (float*)out, out_stride, taps, act, R, max_rows, s);
    return launch_conv<bf16>((const bf16*)z, z_stride, C, w, bias, state, seq_starts, seq_slots, (bf16*)out, out_stride, taps, act, R, max_rows, s);
}

LLMIE_API int llmie_delta_prepare(const void* qkv, int qkv_stride, int q_col, int k_col, const void* a, int a_stride, const void* b,
                                  int b_stride, const float* A_log, const float* dt_bias, float* qn, float* kn, float* kq, float* decay,
                                  float* beta, int N, int H, int G, int D, float q_scale, float unit_eps, int per_head, int dtype, cudaStream_t s) {
    if (N <= 0) return 0;
    if (H <= 0 || G <= 0 || H % G || D <= 0) return LLMIE_ERR_BAD_ARGUMENT;
    const dim3 grid(((size_t)N * H + 3) / 4);
    if (dtype == DT_F32)
        return launch_kernel(delta_prepare_kernel<float>, grid, dim3(128), 0, s, (const float*)qkv, qkv_stride, q_col, k_col, (const float*)a,
                             a_stride, (const float*)b, b_stride, A_log, dt_bias, qn, kn, kq, decay, beta, N, H, G, D, q_scale, unit_eps, per_head);
    return launch_kernel(delta_prepare_kernel<bf16>, grid, dim3(128), 0, s, (const bf16*)qkv, qkv_stride, q_col, k_col, (const bf16*)a, a_stride,
                         (const bf16*)b, b_stride, A_log, dt_bias, qn, kn, kq, decay, beta, N, H, G, D, q_scale, unit_eps, per_head);
}

// state [slots][H][DV][D] float (column by column); out [N][H * DV] float; decay [N][H][D], or [N][H] with per_head
LLMIE_API int llmie_delta_scan(const void* v, int v_stride, int v_col, const float* qn, const float* kn, const float* kq,
                               const float* decay, const float* beta, float* state, const int* seq_starts, const int* seq_slots,
                               float* out, int H, int G, int D, int DV, int R, int max_rows, int per_head, int dtype, cudaStream_t s) {
    if (R <= 0) return 0;
    if (H <= 0 || G <= 0 || H % G || D <= 0 || D > 256 || DV <= 0 || H > 65535 || R > 65535) return LLMIE_ERR_BAD_ARGUMENT;
    const bool alone = max_rows >= SCAN_ALONE_ROWS;   // a long walk: see launch_kernel_on
    if (dtype == DT_F32)
        return launch_delta_scan<float>((const float*)v, v_stride, v_col, qn, kn, kq, decay, beta, state, seq_starts, seq_slots, out, H, G, D, DV, R, alone, per_head != 0, s);
    return launch_delta_scan<bf16>((const bf16*)v, v_stride, v_col, qn, kn, kq, decay, beta, state, seq_starts, seq_slots, out, H, G, D, DV, R, alone, per_head != 0, s);
}

// state [slots][H][DV][NS] float (column by column); out [N][H * DV] float
LLMIE_API int llmie_ssm_scan(const void* xbc, int x_stride, int x_col, int b_col, int c_col, const void* dt_raw, int dt_stride,
                             const float* A_log, const float* dt_bias, const float* Dskip, float* state, const int* seq_starts,
                             const int* seq_slots, float* out, int H, int G, int NS, int DV, int R, int max_rows, int dtype, cudaStream_t s) {
    if (R <= 0) return 0;
    if (H <= 0 || G <= 0 || H % G || NS <= 0 || NS > 256 || DV <= 0 || H > 65535 || R > 65535) return LLMIE_ERR_BAD_ARGUMENT;
    const bool alone = max_rows >= SCAN_ALONE_ROWS;
    if (dtype == DT_F32)
        return launch_ssm_scan<float>((const float*)xbc, x_stride, x_col, b_col, c_col, (const float*)dt_raw, dt_stride, A_log, dt_bias, Dskip,
                                      state, seq_starts, seq_slots, out, H, G, NS, DV, R, alone, s);
    return launch_ssm_scan<bf16>((const bf16*)xbc, x_stride, x_col, b_col, c_col, (const bf16*)dt_raw, dt_stride, A_log, dt_bias, Dskip, state,
                                 seq_starts, seq_slots, out, H, G, NS, DV, R, alone, s);
}

// x, dt_raw, z: [N] rows of C channels (the caller offsets the pointers to their first column); bc: rows that hold B from column
// b_col and C from column c_col (NS entries each); A_log [C][NS], dt_bias [C], Dskip [C]; state [slots][C][NS] float; out [N][C].
LLMIE_API int llmie_selective_scan(const void* x, int x_stride, const void* dt_raw, int dt_stride, const void* bc, int bc_stride, int b_col,
                                   int c_col, const void* z, int z_stride, const float* A_log, const float* dt_bias, const float* Dskip,
                                   float* state, const int* seq_starts, const int* seq_slots, void* out, int C, int NS, int R, int max_rows,
                                   int dtype, cudaStream_t s) {
    if (R <= 0) return 0;
    if (C <= 0 || NS <= 0 || NS > 256 || R > 65535) return LLMIE_ERR_BAD_ARGUMENT;
    const bool alone = max_rows >= SCAN_ALONE_ROWS;
    if (dtype == DT_F32)
        return launch_selective_scan<float>((const float*)x, x_stride, (const float*)dt_raw, dt_stride, (const float*)bc, bc_stride, b_col, c_col,
                                            (const float*)z, z_stride, A_log, dt_bias, Dskip, state, seq_starts, seq_slots, (float*)out, C, NS, R, alone, s);
    return launch_selective_scan<bf16>((const bf16*)x, x_stride, (const bf16*)dt_raw, dt_stride, (const bf16*)bc, bc_stride, b_col, c_col,
                                       (const bf16*)z, z_stride, A_log, dt_bias, Dskip, state, seq_starts, seq_slots, (bf16*)out, C, NS, R, alone, s);
}
