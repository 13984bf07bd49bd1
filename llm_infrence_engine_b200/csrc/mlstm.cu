// The matrix memory with exponential gates (the mLSTM cell of xLSTM), as a recurrence over the rows of each request. T is the
// storage type of the projections (float or bfloat16); gates, their logarithms and exponentials, the running maximum, the memory
// and the normaliser are 32-bit.
//
// Per head, with q (already times dim^-1/2), k of D entries and v of DV, a log input gate i and a log forget gate f:
//   m_t = max(f_t + m_(t-1), i_t);  a_t = exp(f_t + m_(t-1) - m_t);  b_t = exp(i_t - m_t)
//   S_t = a_t S_(t-1) + b_t k_t v_t^T;   n_t = a_t n_(t-1) + b_t k_t;   o_t = S_t^T q_t / (max(|n_t . q_t|, exp(-m_t)) + 1e-6)
// S, n and m start at zero. The normaliser n is kept as one more column of the memory (a column whose v is 1), so a request's
// state is [H, DV + 1, D], column by column, plus m [H]. The scan leaves the numerators (S_t^T q_t and n_t . q_t) and m_t per
// token; the division, the norm of each head's result and the output gate are one kernel behind it.
//
// A step's batch is ragged (request r owns the rows seq_starts[r] .. seq_starts[r + 1] - 1, its state lives in row
// seq_slots[r]): a prompt portion of any length and a single decoded token are the same launch, a request's rows are walked in
// order, and the lanes that share a column depend on D alone, so a position's result does not depend on how the request was cut.
#include <math.h>

#include "common.cuh"

namespace {

constexpr int ML_THREADS = 128;
constexpr int ML_TILE = 8;   // tokens per stage; the gates of a tile are scanned by the first ML_TILE lanes of the first warp

__device__ __forceinline__ float sigmoid_f(float x) { return 1.0f / (1.0f + expf(-x)); }
// ln sigmoid(x) = min(x, 0) - ln(1 + exp(-|x|))
__device__ __forceinline__ float log_sigmoid_f(float x) { return fminf(x, 0.f) - log1pf(expf(-fabsf(x))); }

__device__ __forceinline__ void cp_async16(void* dst, const void* src) {
    const uint32_t d = (uint32_t)__cvta_generic_to_shared(dst);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(d), "l"(src));
}
__device__ __forceinline__ void cp_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void cp_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }

// One block per token: q (times q_scale) and k of every head as floats, and the two gates from their 32-bit pre-activations
// gates[n] = [W_i h (H) | W_f h (H)]:  i = cap tanh((x + b_i) / cap),  f = ln sigmoid(cap tanh((x + b_f) / cap)); cap <= 0: no cap.
template <typename T>
__global__ void __launch_bounds__(128) mlstm_prepare_kernel(const T* __restrict__ z, int z_stride, int q_col, int k_col, const float* __restrict__ gates,
                                                            int g_stride, const float* __restrict__ bias_i, const float* __restrict__ bias_f, float cap,
                                                            float q_scale, float* __restrict__ qf, float* __restrict__ kf, float* __restrict__ ig,
                                                            float* __restrict__ fg, int H, int D) {
    pdl_trigger();
    pdl_wait();
    const int n = blockIdx.x;
    const T* row = z + (size_t)n * z_stride;
    const int HD = H * D;
    for (int i = threadIdx.x; i < HD; i += blockDim.x) {
        qf[(size_t)n * HD + i] = to_f32(row[q_col + i]) * q_scale;
        kf[(size_t)n * HD + i] = to_f32(row[k_col + i]);
    }
    for (int h = threadIdx.x; h < H; h += blockDim.x) {
        float xi = gates[(size_t)n * g_stride + h] + bias_i[h];
        float xf = gates[(size_t)n * g_stride + H + h] + bias_f[h];
        if (cap > 0.f) { xi = cap * tanhf(xi / cap); xf = cap * tanhf(xf / cap); }
        ig[(size_t)n * H + h] = xi;
        fg[(size_t)n * H + h] = log_sigmoid_f(xf);
    }
}

template <int PARTS> __device__ __forceinline__ float parts_sum(float v) {
#pragma unroll
    for (int o = 1; o < PARTS; o <<= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// Block (x, h, r): COLS columns of head h of request r, PARTS lanes to a group of CPL columns, each lane holding DPL entries of each
// of them in registers (16-byte pieces, PARTS pieces apart). Rows of q and k come in tiles of ML_TILE tokens through a two-stage ring
// (cp.async); a tile's gates are loaded into registers a tile ahead by the first warp, which walks the chain of maxima over the tile
// and turns the gates into (a, b, m) per token, a token per lane, so the exponentials are taken once per token and block, not once
// per thread.
template <typename T, int DMAX, int PARTS, int CPL>
__global__ void __launch_bounds__(ML_THREADS) mlstm_scan_kernel(const T* __restrict__ v, int v_stride, int v_col, const float* __restrict__ qf,
                                                                const float* __restrict__ kf, const float* __restrict__ ig, const float* __restrict__ fg,
                                                                float* __restrict__ state, float* __restrict__ mstate, const int* __restrict__ seq_starts,
                                                                const int* __restrict__ seq_slots, float* __restrict__ num, float* __restrict__ m_out,
                                                                int H, int D, int DV) {
    constexpr int DPL = DMAX / PARTS, COLS = (ML_THREADS / PARTS) * CPL, Q = DMAX / 4;   // COLS: the block's columns, CPL to a group of lanes
    __shared__ __align__(16) float k_s[2][ML_TILE][DMAX];
    __shared__ __align__(16) float q_s[2][ML_TILE][DMAX];
    __shared__ float a_s[2][ML_TILE], b_s[2][ML_TILE], m_s[2][ML_TILE];
    __shared__ float v_s[2][ML_TILE][COLS];
    pdl_wait();
    const int part = threadIdx.x % PARTS, my_col = (threadIdx.x / PARTS) * CPL;   // the first of the lane group's CPL columns, within the block
    const int col = blockIdx.x * COLS + my_col;
    const int h = blockIdx.y, r = blockIdx.z;
    const int C = DV + 1;                 // the last column is the normaliser
    const bool vec = (D & 3) == 0;
    const int s0 = seq_starts[r], s1 = seq_starts[r + 1];
    const int slot = seq_slots[r];
    float* st = state + ((size_t)slot * H + h) * C * D;
    float S[CPL][DPL];
#pragma unroll
    for (int u = 0; u < CPL; ++u)
#pragma unroll
        for (int i = 0; i < DPL / 4; ++i) {
            const int d = 4 * PARTS * i + 4 * part;
#pragma unroll
            for (int c = 0; c < 4; ++c) S[u][4 * i + c] = (col + u < C && d + c < D) ? st[(size_t)(col + u) * D + d + c] : 0.f;
        }
    float m_carry = mstate[(size_t)slot * H + h];   // (every lane of the first warp keeps it)

    auto fetch = [&](int base, int buf) {
        const int count = min(ML_TILE, s1 - base);
        for (int i = threadIdx.x; i < count * Q; i += ML_THREADS) {
            const int t = i / Q, d = (i % Q) * 4;
            const size_t off = ((size_t)(base + t) * H + h) * D + d;
            if (vec && d < D) {
                cp_async16(&k_s[buf][t][d], kf + off);
                cp_async16(&q_s[buf][t][d], qf + off);
            } else {
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    k_s[buf][t][d + c] = d + c < D ? kf[off + c] : 0.f;
                    q_s[buf][t][d + c] = d + c < D ? qf[off + c] : 0.f;
                }
            }
        }
    };
    // a tile's gates (lane t < ML_TILE of the first warp: token t) and the block's columns of v, into registers a tile ahead
    constexpr int VPT = (ML_TILE * COLS + ML_THREADS - 1) / ML_THREADS;
    float pre_i = -INFINITY, pre_f = 0.f, pre_v[VPT];
    auto load_small = [&](int base) {
        const int count = min(ML_TILE, s1 - base);
        pre_i = -INFINITY;   // a token past the end changes nothing: m -> max(0 + m, -inf)
        pre_f = 0.f;
        if (threadIdx.x < count) {
            pre_i = ig[(size_t)(base + threadIdx.x) * H + h];
            pre_f = fg[(size_t)(base + threadIdx.x) * H + h];
        }
#pragma unroll
        for (int n = 0; n < VPT; ++n) {
            const int j = ML_THREADS - 1 - threadIdx.x + n * ML_THREADS;
            const int t = j / COLS, c = blockIdx.x * COLS + j % COLS;
            float x = 0.f;
            if (j < count * COLS) x = c < DV ? to_f32(v[(size_t)(base + t) * v_stride + v_col + h * DV + c]) : (c == DV ? 1.f : 0.f);
            pre_v[n] = x;
        }
    };
    auto store_small = [&](int buf) {
        if (threadIdx.x < 32) {
            // the chain m -> max(f + m, i) over the tile's tokens, walked by every lane of the warp in the tokens' order (each step
            // exactly as a token-by-token walk would take it, so the bits do not depend on where a tile begins); lane t keeps token t's
            float m_run = m_carry, m_prev = m_carry, m_t = m_carry;
#pragma unroll
            for (int t = 0; t < ML_TILE; ++t) {
                const float ft = __shfl_sync(0xffffffffu, pre_f, t), it = __shfl_sync(0xffffffffu, pre_i, t);
                const float m_new = fmaxf(ft + m_run, it);
                if ((int)threadIdx.x == t) { m_prev = m_run; m_t = m_new; }
                m_run = m_new;
            }
            if (threadIdx.x >= ML_TILE) m_t = m_run;
            if (threadIdx.x < ML_TILE) {
                a_s[buf][threadIdx.x] = expf(pre_f + m_prev - m_t);
                b_s[buf][threadIdx.x] = expf(pre_i - m_t);
                m_s[buf][threadIdx.x] = m_t;
            }
            m_carry = m_run;
        }
#pragma unroll
        for (int n = 0; n < VPT; ++n) {
            const int j = ML_THREADS - 1 - threadIdx.x + n * ML_THREADS;
            if (j < ML_TILE * COLS) v_s[buf][j / COLS][j % COLS] = pre_v[n];
        }
    };
    if (s0 < s1) {
        fetch(s0, 0);
        load_small(s0);
        store_small(0);
    }
    cp_commit();
    int buf = 0;
    for (int base = s0; base < s1; base += ML_TILE, buf ^= 1) {
        const int count = min(ML_TILE, s1 - base);
        const bool more = base + ML_TILE < s1;
        if (more) {
            fetch(base + ML_TILE, buf ^ 1);
            load_small(base + ML_TILE);
        }
        cp_commit();
        cp_wait<1>();
        __syncthreads();                       // this tile is in shared memory
        // the tile's tokens in order; every token's partial sums stay in registers and the lanes of a column add them up for all
        // tokens of the tile together (the shuffles of eight sums overlap instead of waiting for one another)
        float rq[ML_TILE][CPL];
#pragma unroll
        for (int t = 0; t < ML_TILE; ++t) {
#pragma unroll
            for (int u = 0; u < CPL; ++u) rq[t][u] = 0.f;
            if (t < count) {
                const float a = a_s[buf][t], b = b_s[buf][t];
                float bv[CPL], r0[CPL], r1[CPL];
#pragma unroll
                for (int u = 0; u < CPL; ++u) { bv[u] = b * v_s[buf][t][my_col + u]; r0[u] = 0.f; r1[u] = 0.f; }
#pragma unroll
                for (int i = 0; i < DPL / 4; ++i) {   // a piece of k and of q serves all of the lane's columns
                    const float4 k4 = *reinterpret_cast<const float4*>(&k_s[buf][t][4 * PARTS * i + 4 * part]);
                    const float4 q4 = *reinterpret_cast<const float4*>(&q_s[buf][t][4 * PARTS * i + 4 * part]);
#pragma unroll
                    for (int u = 0; u < CPL; ++u) {
                        float* s = S[u] + 4 * i;
                        s[0] = fmaf(bv[u], k4.x, a * s[0]); s[1] = fmaf(bv[u], k4.y, a * s[1]);
                        s[2] = fmaf(bv[u], k4.z, a * s[2]); s[3] = fmaf(bv[u], k4.w, a * s[3]);
                        r0[u] = fmaf(s[0], q4.x, r0[u]); r1[u] = fmaf(s[1], q4.y, r1[u]); r0[u] = fmaf(s[2], q4.z, r0[u]); r1[u] = fmaf(s[3], q4.w, r1[u]);
                    }
                }
#pragma unroll
                for (int u = 0; u < CPL; ++u) rq[t][u] = r0[u] + r1[u];
            }
        }
#pragma unroll
        for (int o = 1; o < PARTS; o <<= 1) {
#pragma unroll
            for (int t = 0; t < ML_TILE; ++t)
#pragma unroll
                for (int u = 0; u < CPL; ++u) rq[t][u] += __shfl_xor_sync(0xffffffffu, rq[t][u], o);
        }
        // every lane of the group holds all sums: lane t of the group stores token t's
#pragma unroll
        for (int t = 0; t < ML_TILE; ++t)
            if (t < count && part == (t % PARTS)) {
#pragma unroll
                for (int u = 0; u < CPL; ++u)
                    if (col + u < C) num[((size_t)(base + t) * H + h) * C + col + u] = rq[t][u];
            }
        if (blockIdx.x == 0 && threadIdx.x < count) m_out[(size_t)(base + threadIdx.x) * H + h] = m_s[buf][threadIdx.x];
        if (more) store_small(buf ^ 1);
        __syncthreads();                       // everyone is done with this stage before it is filled again
    }
    cp_wait<0>();
    pdl_trigger();
#pragma unroll
    for (int u = 0; u < CPL; ++u)
#pragma unroll
        for (int i = 0; i < DPL / 4; ++i) {
            const int d = 4 * PARTS * i + 4 * part;
#pragma unroll
            for (int c = 0; c < 4; ++c)
                if (col + u < C && d + c < D) st[(size_t)(col + u) * D + d + c] = S[u][4 * i + c];
        }
    if (blockIdx.x == 0 && threadIdx.x == 0 && s0 < s1) mstate[(size_t)slot * H + h] = m_carry;
}

// One block per (token, head): o = num / (max(|n . q|, exp(-m)) + 1e-6); o / sqrt(mean(o^2) + eps) * w[h * DV + j] * sigmoid(gate).
template <typename T>
__global__ void __launch_bounds__(128) mlstm_finish_kernel(const float* __restrict__ num, const float* __restrict__ m_t, const T* __restrict__ gate,
                                                           int gate_stride, const float* __restrict__ w, T* __restrict__ out, int H, int DV, float eps) {
    __shared__ float scratch[36];
    pdl_trigger();
    pdl_wait();
    const int n = blockIdx.x, h = blockIdx.y;
    const float* row = num + ((size_t)n * H + h) * (DV + 1);
    const float den = fmaxf(fabsf(row[DV]), expf(-m_t[(size_t)n * H + h])) + 1e-6f;
    float sq = 0.f;
    for (int j = threadIdx.x; j < DV; j += blockDim.x) { const float o = row[j] / den; sq = fmaf(o, o, sq); }
    const float rstd = 1.0f / sqrtf(block_sum(sq, scratch) / (float)DV + eps);
    for (int j = threadIdx.x; j < DV; j += blockDim.x) {
        const float o = row[j] / den;
        const float g = sigmoid_f(to_f32(gate[(size_t)n * gate_stride + (size_t)h * DV + j]));
        out[((size_t)n * H + h) * DV + j] = from_f32<T>(o * rstd * w[(size_t)h * DV + j] * g);
    }
}

template <typename T, int DM, int PARTS, int CPL>
int launch_scan_as(const T* v, int v_stride, int v_col, const float* qf, const float* kf, const float* ig, const float* fg, float* state, float* mstate,
                   const int* seq_starts, const int* seq_slots, float* num, float* m_out, int H, int D, int DV, int R, cudaStream_t s) {
    constexpr int COLS = (ML_THREADS / PARTS) * CPL;
    const dim3 grid((DV + 1 + COLS - 1) / COLS, H, R);
    return launch_kernel(mlstm_scan_kernel<T, DM, PARTS, CPL>, grid, dim3(ML_THREADS), 0, s, v, v_stride, v_col, qf, kf, ig, fg, state, mstate, seq_starts,
                         seq_slots, num, m_out, H, D, DV);
}

// The lanes that share a column depend on the padded key size alone (a lane holds one 16-byte piece of a short column, two from 64
// entries on: fewer lanes to add up over), and a group of lanes owns up to four columns side by side, so that a piece of k and of q,
// once fetched from shared memory, serves four columns: with one column to a group the kernel was bound by the instructions around the
// multiply-adds (31 % of the issue slots busy, a quarter of the instructions multiply-adds; 1.54 ms at 128 entries and 2,048 tokens).
template <typename T>
int launch_scan(const T* v, int v_stride, int v_col, const float* qf, const float* kf, const float* ig, const float* fg, float* state, float* mstate,
                const int* seq_starts, const int* seq_slots, float* num, float* m_out, int H, int D, int DV, int R, cudaStream_t s) {
#define ML_ARGS v, v_stride, v_col, qf, kf, ig, fg, state, mstate, seq_starts, seq_slots, num, m_out, H, D, DV, R, s
    if (D <= 16) return launch_scan_as<T, 16, 4, 1>(ML_ARGS);
    if (D <= 32) return launch_scan_as<T, 32, 8, 2>(ML_ARGS);
    if (D <= 64) return launch_scan_as<T, 64, 8, 4>(ML_ARGS);
    if (D <= 128) return launch_scan_as<T, 128, 16, 4>(ML_ARGS);
    return launch_scan_as<T, 256, 32, 4>(ML_ARGS);
#undef ML_ARGS
}

}  // namespace

// z [N, z_stride] holds q (H * D from q_col) and k (from k_col); gates [N, g_stride] float = [W_i h | W_f h]; outputs qf, kf [N, H, D],
// ig, fg [N, H], all float.
LLMIE_API int llmie_mlstm_prepare(const void* z, int z_stride, int q_col, int k_col, const float* gates, int g_stride, const float* bias_i,
                                  const float* bias_f, float cap, float q_scale, float* qf, float* kf, float* ig, float* fg, int N, int H, int D,
                                  int dtype, cudaStream_t s) {
    if (N <= 0) return 0;
    if (H <= 0 || D <= 0 || g_stride < 2 * H || q_col < 0 || k_col < 0 || !bias_i || !bias_f) return LLMIE_ERR_BAD_ARGUMENT;
    if (dtype == DT_F32)
        return launch_kernel(mlstm_prepare_kernel<float>, dim3(N), dim3(128), 0, s, (const float*)z, z_stride, q_col, k_col, gates, g_stride, bias_i, bias_f,
                             cap, q_scale, qf, kf, ig, fg, H, D);
    return launch_kernel(mlstm_prepare_kernel<bf16>, dim3(N), dim3(128), 0, s, (const bf16*)z, z_stride, q_col, k_col, gates, g_stride, bias_i, bias_f, cap,
                         q_scale, qf, kf, ig, fg, H, D);
}

// v: DV columns per head from v_col of rows of v_stride; state [slots, H, DV + 1, D], mstate [slots, H]; num [N, H, DV + 1], m_out [N, H].
LLMIE_API int llmie_mlstm_scan(const void* v, int v_stride, int v_col, const float* qf, const float* kf, const float* ig, const float* fg, float* state,
                               float* mstate, const int* seq_starts, const int* seq_slots, float* num, float* m_out, int H, int D, int DV, int R,
                               int dtype, cudaStream_t s) {
    if (R <= 0) return 0;
    if (H <= 0 || H > 65535 || R > 65535 || D <= 0 || D > 256 || DV <= 0) return LLMIE_ERR_BAD_ARGUMENT;
    if (dtype == DT_F32) return launch_scan<float>((const float*)v, v_stride, v_col, qf, kf, ig, fg, state, mstate, seq_starts, seq_slots, num, m_out, H, D, DV, R, s);
    return launch_scan<bf16>((const bf16*)v, v_stride, v_col, qf, kf, ig, fg, state, mstate, seq_starts, seq_slots, num, m_out, H, D, DV, R, s);
}

// gate: H * DV columns of rows of gate_stride (storage type); w [H * DV]; out [N, H * DV] of the storage type.
LLMIE_API int llmie_mlstm_finish(const float* num, const float* m_t, const void* gate, int gate_stride, const float* w, void* out, int N, int H, int DV,
                                 float eps, int dtype, cudaStream_t s) {
    if (N <= 0) return 0;
    if (H <= 0 || H > 65535 || DV <= 0) return LLMIE_ERR_BAD_ARGUMENT;
    int threads = 32;
    while (threads < 128 && threads < DV) threads *= 2;
    if (dtype == DT_F32)
        return launch_kernel(mlstm_finish_kernel<float>, dim3(N, H), dim3(threads), 0, s, num, m_t, (const float*)gate, gate_stride, w, (float*)out, H, DV, eps);
    return launch_kernel(mlstm_finish_kernel<bf16>, dim3(N, H), dim3(threads), 0, s, num, m_t, (const bf16*)gate, gate_stride, w, (bf16*)out, H, DV, eps);
}
