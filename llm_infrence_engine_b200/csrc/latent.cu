// Kernels around latent attention: the cache holds one row [c | r] per token (a normed latent and a rotated key part
// that all heads share); queries are carried into the latent space and the result is carried out of it by one small
// matrix per head.
//
//   latent_prepare:  z[n] = [dq (q_rank) | dkv (kv_rank) | r (rot_dim) | ...] -> cq[n] = rmsnorm(dq) * wq;
//                    cache row = [rmsnorm(dkv) * wkv | turn(r)]    (norms and angles in 32-bit)
//   head_matmul:     out[n][h][0:J] = x[n][h][0:K] @ M[h]   with M[h] = [K][J] row-major, 32-bit sums in the order of k;
//                    ABSORB also copies x[n][h][K:K+R] behind the J results, its first `rot_dims` entries turned by the
//                    token's angle; EXPAND multiplies result j by sigmoid(gate[n][h * J + j]).
//
// turn(): neighbouring pairs (2i, 2i+1): (u, v) -> (u cos - v sin, v cos + u sin) with cos/sin[n][i].
#include "common.cuh"

namespace {

template <typename T>
__global__ void latent_prepare_kernel(const T* __restrict__ z, int z_stride, int q_rank, int kv_rank, int rot_dim, int rot_dims,
                                      const float* __restrict__ wq, const float* __restrict__ wkv, float eps,
                                      const float* __restrict__ cos_t, const float* __restrict__ sin_t, const int* __restrict__ slots,
                                      T* __restrict__ pool, int page_size, int write, T* __restrict__ cq) {
    __shared__ float scratch[36];
    pdl_trigger();
    pdl_wait();
    const int n = blockIdx.x;
    const T* row = z + (size_t)n * z_stride;
    float ss = 0.f, rstd;
    if (q_rank > 0) {   // (q_rank 0: the queries are not made from a latent; only the cache row is written)
        for (int i = threadIdx.x; i < q_rank; i += blockDim.x) { const float v = to_f32(row[i]); ss = fmaf(v, v, ss); }
        ss = block_sum(ss, scratch);
        rstd = 1.0f / sqrtf(ss / (float)q_rank + eps);
        for (int i = threadIdx.x; i < q_rank; i += blockDim.x) cq[(size_t)n * q_rank + i] = from_f32<T>(to_f32(row[i]) * rstd * wq[i]);
    }
    if (!write) return;
    const T* c = row + q_rank;
    ss = 0.f;
    for (int i = threadIdx.x; i < kv_rank; i += blockDim.x) { const float v = to_f32(c[i]); ss = fmaf(v, v, ss); }
    ss = block_sum(ss, scratch);
    rstd = 1.0f / sqrtf(ss / (float)kv_rank + eps);
    const int slot = slots[n];   // page * page_size + offset; one key/value head
    T* dst = pool + (size_t)slot * (kv_rank + rot_dim);
    for (int i = threadIdx.x; i < kv_rank; i += blockDim.x) dst[i] = from_f32<T>(to_f32(c[i]) * rstd * wkv[i]);
    const T* r = c + kv_rank;
    const int half = rot_dims >> 1;
    for (int i = threadIdx.x; i < half; i += blockDim.x) {
        const float u = to_f32(r[2 * i]), v = to_f32(r[2 * i + 1]);
        const float cs = cos_t[(size_t)n * half + i], sn = sin_t[(size_t)n * half + i];
        dst[kv_rank + 2 * i] = from_f32<T>(u * cs - v * sn);
        dst[kv_rank + 2 * i + 1] = from_f32<T>(v * cs + u * sn);
    }
    for (int i = rot_dims + threadIdx.x; i < rot_dim; i += blockDim.x) dst[kv_rank + i] = r[i];
}

constexpr int TOK = 8;
// ABSORB_TAIL and GATE_ONLY: the products were made elsewhere (a batched library product wrote them into `out`); only the
// copy of the rotated parts, or the multiplication by the gate, is left.
enum { MODE_PLAIN = 0, MODE_ABSORB = 1, MODE_EXPAND = 2, MODE_ABSORB_TAIL = 3, MODE_GATE_ONLY = 4 };

// A block: up to TOK tokens, one head, 32 result columns (lane = column). Its four warps take a quarter of the inner dimension
// each, in order, and their partial sums are added in the order of the warps: every result is one fixed sequence of 32-bit
// multiply-adds, whatever the batch holds.
template <typename T>
__global__ void __launch_bounds__(128) head_matmul_kernel(const T* __restrict__ x, int x_stride, int x_head, const T* __restrict__ M,
                                                         T* __restrict__ out, int out_stride, int out_head, int N, int K, int J, int mode,
                                                         int R, int rot_dims, const float* __restrict__ cos_t,
                                                         const float* __restrict__ sin_t, const T* __restrict__ gate, int gate_stride) {
    extern __shared__ __align__(16) float xs[];   // [TOK][K], then [4][TOK][32] partial sums
    float* part = xs + TOK * K;
    pdl_trigger();
    pdl_wait();
    const int n0 = blockIdx.x * TOK, h = blockIdx.y, j0 = blockIdx.z * 32;
    const int nt = min(TOK, N - n0);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (mode == MODE_GATE_ONLY) {
        for (int i = threadIdx.x; i < nt * 32; i += blockDim.x) {
            const int t = i / 32, j = j0 + i % 32;
            if (j >= J) continue;
            T* o = out + (size_t)(n0 + t) * out_stride + (size_t)h * out_head + j;
            *o = from_f32<T>(to_f32(*o) * (1.0f / (1.0f + expf(-to_f32(gate[(size_t)(n0 + t) * gate_stride + (size_t)h * J + j])))));
        }
        return;
    }
    if (mode != MODE_ABSORB_TAIL) {
        for (int i = threadIdx.x; i < TOK * K; i += blockDim.x) {
            const int t = i / K, k = i % K;
            xs[i] = t < nt ? to_f32(x[(size_t)(n0 + t) * x_stride + (size_t)h * x_head + k]) : 0.f;
        }
        __syncthreads();
        const int j = j0 + lane;
        const int kq = (K + 3) / 4;
        const int k_lo = warp * kq, k_hi = min(K, k_lo + kq);
        float acc[TOK];
#pragma unroll
        for (int t = 0; t < TOK; ++t) acc[t] = 0.f;
        if (j < J) {
            const T* col = M + (size_t)h * K * J + j;
            int k = k_lo;
            for (; k + 8 <= k_hi; k += 8) {   // eight loads in flight
                float w[8];
#pragma unroll
                for (int u = 0; u < 8; ++u) w[u] = to_f32(col[(size_t)(k + u) * J]);
#pragma unroll
                for (int u = 0; u < 8; ++u)
#pragma unroll
                    for (int t = 0; t < TOK; ++t) acc[t] = fmaf(xs[t * K + k + u], w[u], acc[t]);
            }
            for (; k < k_hi; ++k) {
                const float w = to_f32(col[(size_t)k * J]);
#pragma unroll
                for (int t = 0; t < TOK; ++t) acc[t] = fmaf(xs[t * K + k], w, acc[t]);
            }
        }
#pragma unroll
        for (int t = 0; t < TOK; ++t) part[(warp * TOK + t) * 32 + lane] = acc[t];
        __syncthreads();
        for (int i = threadIdx.x; i < nt * 32; i += blockDim.x) {
            const int t = i / 32, jj = j0 + i % 32;
            if (jj >= J) continue;
            float v = part[(0 * TOK + t) * 32 + i % 32];
#pragma unroll
            for (int w = 1; w < 4; ++w) v += part[(w * TOK + t) * 32 + i % 32];
            if (mode == MODE_EXPAND) v *= 1.0f / (1.0f + expf(-to_f32(gate[(size_t)(n0 + t) * gate_stride + (size_t)h * J + jj])));
            out[(size_t)(n0 + t) * out_stride + (size_t)h * out_head + jj] = from_f32<T>(v);
        }
    }
    if ((mode != MODE_ABSORB && mode != MODE_ABSORB_TAIL) || blockIdx.z != 0) return;
    const int half = rot_dims >> 1;
    for (int i = threadIdx.x; i < nt * R; i += blockDim.x) {
        const int t = i / R, e = i % R, n = n0 + t;
        const T* src = x + (size_t)n * x_stride + (size_t)h * x_head + K;
        float v;
        if (e < rot_dims) {
            const int pr = e >> 1;
            const float cs = cos_t[(size_t)n * half + pr], sn = sin_t[(size_t)n * half + pr];
            const float a = to_f32(src[2 * pr]), b = to_f32(src[2 * pr + 1]);
            v = (e & 1) ? b * cs + a * sn : a * cs - b * sn;
        } else {
            v = to_f32(src[e]);
        }
        out[(size_t)n * out_stride + (size_t)h * out_head + J + e] = from_f32<T>(v);
    }
}

template <typename T>
int prepare(const T* z, int z_stride, int q_rank, int kv_rank, int rot_dim, int rot_dims, const float* wq, const float* wkv, float eps,
            const float* cos_t, const float* sin_t, const int* slots, T* pool, int page_size, int write, T* cq, int N, cudaStream_t s) {
    return launch_kernel(latent_prepare_kernel<T>, dim3(N), dim3(128), 0, s, z, z_stride, q_rank, kv_rank, rot_dim, rot_dims, wq, wkv, eps,
                         cos_t, sin_t, slots, pool, page_size, write, cq);
}

template <typename T>
int head_matmul(const T* x, int x_stride, int x_head, const T* M, T* out, int out_stride, int out_head, int N, int H, int K, int J, int mode,
                int R, int rot_dims, const float* cos_t, const float* sin_t, const T* gate, int gate_stride, cudaStream_t s) {
    const size_t smem = sizeof(float) * (TOK * (size_t)K + 4 * TOK * 32);
    const int jchunks = mode == MODE_ABSORB_TAIL ? 1 : (J + 31) / 32;   // the tail alone is one block's work per tokens and head
    if (smem > 200 * 1024 || H > 65535 || jchunks > 65535) return LLMIE_ERR_BAD_ARGUMENT;
    if (smem > 48 * 1024) cudaFuncSetAttribute(head_matmul_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    return launch_kernel(head_matmul_kernel<T>, dim3((N + TOK - 1) / TOK, H, jchunks), dim3(128), smem, s, x, x_stride, x_head, M, out, out_stride,
                         out_head, N, K, J, mode, R, rot_dims, cos_t, sin_t, gate, gate_stride);
}

}  // namespace

LLMIE_API int llmie_latent_prepare(const void* z, int z_stride, int q_rank, int kv_rank, int rot_dim, int rot_dims, const float* wq,
                                   const float* wkv, float eps, const float* cos_t, const float* sin_t, const int* slots, void* pool,
                                   int page_size, int write, void* cq, int N, int dtype, cudaStream_t s) {
    if (N <= 0) return 0;
    if (q_rank < 0 || (q_rank && (!wq || !cq)) || kv_rank < 1 || rot_dim < 0 || rot_dims < 0 || rot_dims > rot_dim || (rot_dims & 1) || (rot_dims && (!cos_t || !sin_t)) ||
        (write && (!slots || !pool)))
        return LLMIE_ERR_BAD_ARGUMENT;
    if (dtype == DT_F32)
        return prepare<float>((const float*)z, z_stride, q_rank, kv_rank, rot_dim, rot_dims, wq, wkv, eps, cos_t, sin_t, slots, (float*)pool, page_size, write, (float*)cq, N, s);
    return prepare<bf16>((const bf16*)z, z_stride, q_rank, kv_rank, rot_dim, rot_dims, wq, wkv, eps, cos_t, sin_t, slots, (bf16*)pool, page_size, write, (bf16*)cq, N, s);
}

// mode 0: plain; 1: absorb (R further entries of every head of x are copied behind the J results, the first rot_dims of them
// turned); 2: expand (results times sigmoid(gate)).
LLMIE_API int llmie_head_matmul(const void* x, int x_stride, int x_head, const void* M, void* out, int out_stride, int out_head, int N, int H,
                                int K, int J, int mode, int R, int rot_dims, const float* cos_t, const float* sin_t, const void* gate,
                                int gate_stride, int dtype, cudaStream_t s) {
    if (N <= 0) return 0;
    if (K < 1 || J < 1 || H < 1 || mode < 0 || mode > 4 || ((mode == 1 || mode == 3) && (rot_dims > R || (rot_dims & 1) || (rot_dims && (!cos_t || !sin_t)))) ||
        ((mode == 2 || mode == 4) && !gate))
        return LLMIE_ERR_BAD_ARGUMENT;
    if (dtype == DT_F32)
        return head_matmul<float>((const float*)x, x_stride, x_head, (const float*)M, (float*)out, out_stride, out_head, N, H, K, J, mode, R, rot_dims, cos_t, sin_t, (const float*)gate, gate_stride, s);
    return head_matmul<bf16>((const bf16*)x, x_stride, x_head, (const bf16*)M, (bf16*)out, out_stride, out_head, N, H, K, J, mode, R, rot_dims, cos_t, sin_t, (const bf16*)gate, gate_stride, s);
}
