// Layer norm with a weight (and, for the norm of a sublayer's input, an optional bias), for blocks that norm a sublayer's input AND its result:
//   x <- x + LN_post(y);  h = LN_pre(x)
// One kernel does either half or both, one block per row, the row in shared memory between the passes. Mean, variance
// (the mean of the squared deviations, taken in a second pass about the finished mean) and the scaling are 32-bit. Also here: the root-mean-square
// norm over groups of a row with a gate, and the mean of several rows each divided by its root mean square.
#include <math.h>

#include "common.cuh"

namespace {

__device__ __forceinline__ float sigmoid_f(float x) { return 1.0f / (1.0f + expf(-x)); }

// rows == nullptr: r = blockIdx.x and the updated x is stored; rows != nullptr: r = rows[blockIdx.x], nothing of x is stored.
// y (of type TY, or null): the sublayer's result whose layer norm (weight w_post) is added to x first; with clear_y the row of
// y is set to zero behind the read (it is then a float buffer that the next sublayer adds into).
// w_pre (or null): out[blockIdx.x] = LN(x) * w_pre (+ b_pre, if given) in type TO.
// Mean and reciprocal standard deviation of the H floats of buf, in two passes (the squared deviations are taken about the
// finished mean); every thread gets both. A thread reads the entries it wrote itself, so no barrier is needed before.
template <int VEC>
__device__ __forceinline__ void row_stats(const float* buf, int H, int step, float eps, float* scratch, float& mean, float& rstd) {
    float sum = 0.f;
    for (int i = threadIdx.x * VEC; i < H; i += step) {
        float v[VEC];
        if constexpr (VEC == 4) load4(buf + i, v); else v[0] = buf[i];   // (16-byte accesses: four floats apart, the threads would collide on the banks)
#pragma unroll
        for (int j = 0; j < VEC; ++j) sum += v[j];
    }
    mean = block_sum(sum, scratch) / (float)H;
    float sq = 0.f;
    for (int i = threadIdx.x * VEC; i < H; i += step) {
        float v[VEC];
        if constexpr (VEC == 4) load4(buf + i, v); else v[0] = buf[i];
#pragma unroll
        for (int j = 0; j < VEC; ++j) { const float d = v[j] - mean; sq = fmaf(d, d, sq); }
    }
    rstd = 1.0f / sqrtf(block_sum(sq, scratch) / (float)H + eps);
}

// post_plain: the sublayer's result is not normed before it is added, only scaled element by element: x <- x + y * w_post (a layer scale).
template <typename TY, typename TO, int VEC>
__global__ void layernorm_kernel(float* __restrict__ x, TY* __restrict__ y, const float* __restrict__ w_post, int clear_y,
                                 const float* __restrict__ w_pre, const float* __restrict__ b_pre, TO* __restrict__ out,
                                 const int* __restrict__ rows, int H, float eps, int post_plain) {
    extern __shared__ __align__(16) float ln_buf[];   // the row of x, the row of y, both weights (H floats each), 100 for the reductions
    float* x_buf = ln_buf;
    float* y_buf = x_buf + H;
    float* wp_buf = y_buf + H;
    float* wq_buf = wp_buf + H;
    float* scratch = wq_buf + H;
    const int step = blockDim.x * VEC;
    pdl_trigger();
    // the weights do not depend on the kernel before: they are fetched before the wait
    for (int i = threadIdx.x * VEC; i < H; i += step) {
        if constexpr (VEC == 4) {
            if (w_post) *reinterpret_cast<float4*>(wp_buf + i) = *reinterpret_cast<const float4*>(w_post + i);
            if (w_pre) *reinterpret_cast<float4*>(wq_buf + i) = *reinterpret_cast<const float4*>(w_pre + i);
        } else {
            if (w_post) wp_buf[i] = w_post[i];
            if (w_pre) wq_buf[i] = w_pre[i];
        }
    }
    pdl_wait();
    const int r = rows ? rows[blockIdx.x] : blockIdx.x;
    float* xr = x + (size_t)r * H;
    TY* yr = y ? y + (size_t)r * H : nullptr;
    // both rows are asked for at once: one trip to memory
    for (int i = threadIdx.x * VEC; i < H; i += step) {
        float v[VEC], u[VEC];
        if constexpr (VEC == 4) load4(xr + i, v); else v[0] = xr[i];
        if (yr) { if constexpr (VEC == 4) load4(yr + i, u); else u[0] = to_f32(yr[i]); }
        if constexpr (VEC == 4) { store4(x_buf + i, v); if (yr) store4(y_buf + i, u); } else { x_buf[i] = v[0]; if (yr) y_buf[i] = u[0]; }
        if (yr && clear_y) {
            const float zero[4] = {0.f, 0.f, 0.f, 0.f};
            if constexpr (VEC == 4) store4(yr + i, zero); else yr[i] = from_f32<TY>(0.f);
        }
    }
    if (yr) {
        float mean = 0.f, rstd = 1.f;
        if (!post_plain) row_stats<VEC>(y_buf, H, step, eps, scratch, mean, rstd);
        for (int i = threadIdx.x * VEC; i < H; i += step) {
            float v[VEC], u[VEC], w[VEC];
            if constexpr (VEC == 4) { load4(x_buf + i, v); load4(y_buf + i, u); load4(wp_buf + i, w); } else { v[0] = x_buf[i]; u[0] = y_buf[i]; w[0] = wp_buf[i]; }
#pragma unroll
            for (int j = 0; j < VEC; ++j) v[j] += (u[j] - mean) * rstd * w[j];
            if constexpr (VEC == 4) store4(x_buf + i, v); else x_buf[i] = v[0];
            if (!rows) { if constexpr (VEC == 4) store4(xr + i, v); else xr[i] = v[0]; }
        }
    }
    if (!w_pre) return;
    float mean, rstd;
    row_stats<VEC>(x_buf, H, step, eps, scratch, mean, rstd);
    TO* o = out + (size_t)blockIdx.x * H;
    for (int i = threadIdx.x * VEC; i < H; i += step) {
        float v[VEC], w[VEC];
        if constexpr (VEC == 4) { load4(x_buf + i, v); load4(wq_buf + i, w); } else { v[0] = x_buf[i]; w[0] = wq_buf[i]; }
#pragma unroll
        for (int j = 0; j < VEC; ++j) v[j] = (v[j] - mean) * rstd * w[j];
        if (b_pre) {
#pragma unroll
            for (int j = 0; j < VEC; ++j) v[j] += b_pre[i + j];
        }
        if constexpr (VEC == 4) store4(o + i, v); else o[i] = from_f32<TO>(v[0]);
    }
}

template <typename TY, typename TO>
int launch_layernorm(float* x, void* y, const float* w_post, int clear_y, const float* w_pre, const float* b_pre, void* out, const int* rows,
                     int n_out, int H, float eps, int post_plain, cudaStream_t s) {
    const size_t smem = (size_t)(4 * H + 100) * sizeof(float);
    const bool vec = H % 4 == 0 && ((uintptr_t)x % 16 == 0) && ((uintptr_t)y % 16 == 0) && ((uintptr_t)out % 16 == 0) &&
                     ((uintptr_t)w_post % 16 == 0) && ((uintptr_t)w_pre % 16 == 0);
    const int per = vec ? 4 : 1;
    int threads = 32;
    while (threads < 512 && threads * per * 2 <= H) threads *= 2;
    if (vec) {
        if (smem > 48 * 1024) cudaFuncSetAttribute(layernorm_kernel<TY, TO, 4>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        return launch_kernel(layernorm_kernel<TY, TO, 4>, dim3(n_out), dim3(threads), smem, s, x, (TY*)y, w_post, clear_y, w_pre, b_pre, (TO*)out, rows, H, eps, post_plain);
    }
    if (smem > 48 * 1024) cudaFuncSetAttribute(layernorm_kernel<TY, TO, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    return launch_kernel(layernorm_kernel<TY, TO, 1>, dim3(n_out), dim3(threads), smem, s, x, (TY*)y, w_post, clear_y, w_pre, b_pre, (TO*)out, rows, H, eps, post_plain);
}

// Root-mean-square norm over groups of `gs` consecutive channels, with a gate, one block per (row, group):
//   mode 0: v = x * silu(gate);            out = v / rms(v) * w                     (the gate comes before the norm)
//   mode 1: out = x / rms(x) * w * sigmoid(gate)                                    (the gate comes after it)
//   mode 2: out = x / rms(x) * w * silu(gate)
// w has w_len entries and channel c uses w[c % w_len] (one weight per channel, or one vector shared by all groups).
template <typename TG, typename TO>
__global__ void group_rmsnorm_gate_kernel(const float* __restrict__ x, const TG* __restrict__ gate, int gate_stride,
                                          const float* __restrict__ w, int w_len, TO* __restrict__ out, int C, int gs, float eps, int mode) {
    __shared__ float scratch[36];
    pdl_trigger();
    pdl_wait();
    const int n = blockIdx.x, c0 = blockIdx.y * gs;
    const float* xr = x + (size_t)n * C + c0;
    const TG* gr = gate + (size_t)n * gate_stride + c0;
    float sq = 0.f;
    for (int i = threadIdx.x; i < gs; i += blockDim.x) {
        float v = xr[i];
        if (mode == 0) { const float z = to_f32(gr[i]); v *= z / (1.0f + expf(-z)); }
        sq = fmaf(v, v, sq);
    }
    const float rstd = 1.0f / sqrtf(block_sum(sq, scratch) / (float)gs + eps);
    TO* o = out + (size_t)n * C + c0;
    for (int i = threadIdx.x; i < gs; i += blockDim.x) {
        float v = xr[i];
        const float z = to_f32(gr[i]);
        if (mode == 0) v *= z / (1.0f + expf(-z));
        v = v * rstd * w[(c0 + i) % w_len];
        if (mode == 1) v *= sigmoid_f(z);
        if (mode == 2) v *= z * sigmoid_f(z);
        o[i] = from_f32<TO>(v);
    }
}

// The same for groups of up to 256 channels: a warp per (row, group), the group's values in registers, no barrier.
template <typename TG, typename TO>
__global__ void __launch_bounds__(128) group_rmsnorm_gate_warp_kernel(const float* __restrict__ x, const TG* __restrict__ gate, int gate_stride,
                                                                      const float* __restrict__ w, int w_len, TO* __restrict__ out, int N, int C,
                                                                      int gs, float eps, int mode) {
    pdl_trigger();
    pdl_wait();
    const int groups = C / gs;
    const long long item = (long long)blockIdx.x * 4 + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    if (item >= (long long)N * groups) return;
    const int n = (int)(item / groups), c0 = (int)(item % groups) * gs;
    const float* xr = x + (size_t)n * C + c0;
    const TG* gr = gate + (size_t)n * gate_stride + c0;
    float v[8], z[8];   // gs <= 256
    float sq = 0.f;
#pragma unroll
    for (int k = 0; k < 8; ++k) {
        const int i = lane + 32 * k;
        v[k] = 0.f; z[k] = 0.f;
        if (i < gs) {
            v[k] = xr[i];
            z[k] = to_f32(gr[i]);
            if (mode == 0) v[k] *= z[k] / (1.0f + expf(-z[k]));
            sq = fmaf(v[k], v[k], sq);
        }
    }
    const float rstd = 1.0f / sqrtf(warp_sum(sq) / (float)gs + eps);
    TO* o = out + (size_t)n * C + c0;
#pragma unroll
    for (int k = 0; k < 8; ++k) {
        const int i = lane + 32 * k;
        if (i < gs) {
            float r = v[k] * rstd * w[(c0 + i) % w_len];
            if (mode == 1) r *= sigmoid_f(z[k]);
            if (mode == 2) r *= z[k] * sigmoid_f(z[k]);
            o[i] = from_f32<TO>(r);
        }
    }
}

// y[n] (+)= coef * (a[n] / rms(a[n]) * wa + b[n] / rms(b[n]) * wb): two sublayer results of one input, each normed by itself,
// then their mean. One block per row. The inputs may be float sums or rounded rows of a library product; with clear_a / clear_b
// an input is set to zero behind the read (a float buffer that the next sublayer adds into).
template <typename TA, typename TB>
__global__ void dual_rmsnorm_mix_kernel(TA* __restrict__ a, TB* __restrict__ b, const float* __restrict__ wa,
                                        const float* __restrict__ wb, float* __restrict__ y, int H, float eps, float coef, int accumulate,
                                        int clear_a, int clear_b) {
    __shared__ float scratch[36];
    pdl_trigger();
    pdl_wait();
    const size_t off = (size_t)blockIdx.x * H;
    float sa = 0.f, sb = 0.f;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        const float va = to_f32(a[off + i]), vb = to_f32(b[off + i]);
        sa = fmaf(va, va, sa);
        sb = fmaf(vb, vb, sb);
    }
    const float ra = 1.0f / sqrtf(block_sum(sa, scratch) / (float)H + eps);
    const float rb = 1.0f / sqrtf(block_sum(sb, scratch) / (float)H + eps);
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        const float v = coef * (to_f32(a[off + i]) * ra * wa[i] + to_f32(b[off + i]) * rb * wb[i]);
        if (clear_a) a[off + i] = from_f32<TA>(0.f);
        if (clear_b) b[off + i] = from_f32<TB>(0.f);
        y[off + i] = accumulate ? y[off + i] + v : v;
    }
}

// y[i] += ca * a[i] + cb * b[i]: two sublayer results of one input, each with a factor of its own. The inputs may be float sums or
// rounded rows of a library product; with clear_a / clear_b an input is set to zero behind the read.
template <typename TA, typename TB>
__global__ void weighted_pair_kernel(TA* __restrict__ a, TB* __restrict__ b, float ca, float cb, float* __restrict__ y, long long total,
                                     int clear_a, int clear_b) {
    pdl_trigger();
    pdl_wait();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const float v = fmaf(ca, to_f32(a[i]), cb * to_f32(b[i]));
    if (clear_a) a[i] = from_f32<TA>(0.f);
    if (clear_b) b[i] = from_f32<TB>(0.f);
    y[i] += v;
}

}  // namespace

LLMIE_API int llmie_weighted_pair(void* a, int a_dtype, void* b, int b_dtype, float ca, float cb, float* y, long long total, int clear_a,
                                  int clear_b, cudaStream_t s) {
    if (total <= 0) return 0;
    const dim3 grid((unsigned)((total + 255) / 256));
#define LLMIE_PAIR(TA, TB) return launch_kernel(weighted_pair_kernel<TA, TB>, grid, dim3(256), 0, s, (TA*)a, (TB*)b, ca, cb, y, total, clear_a, clear_b)
    if (a_dtype == DT_F32 && b_dtype == DT_F32) LLMIE_PAIR(float, float);
    if (a_dtype == DT_F32 && b_dtype == DT_BF16) LLMIE_PAIR(float, bf16);
    if (a_dtype == DT_BF16 && b_dtype == DT_F32) LLMIE_PAIR(bf16, float);
    if (a_dtype == DT_BF16 && b_dtype == DT_BF16) LLMIE_PAIR(bf16, bf16);
#undef LLMIE_PAIR
    return LLMIE_ERR_BAD_ARGUMENT;
}

LLMIE_API int llmie_layernorm(float* x, void* y, int y_dtype, const float* w_post, int clear_y, const float* w_pre, const float* b_pre, void* out,
                              int out_dtype, const int* rows, int n_out, int H, float eps, int post_plain, cudaStream_t s) {
    if (n_out <= 0) return 0;
    if (H <= 0 || (size_t)(4 * H + 100) * sizeof(float) > 200 * 1024 || (y && !w_post) || (w_pre && !out)) return LLMIE_ERR_BAD_ARGUMENT;
    if (y_dtype == DT_F32 && out_dtype == DT_F32) return launch_layernorm<float, float>(x, y, w_post, clear_y, w_pre, b_pre, out, rows, n_out, H, eps, post_plain, s);
    if (y_dtype == DT_F32 && out_dtype == DT_BF16) return launch_layernorm<float, bf16>(x, y, w_post, clear_y, w_pre, b_pre, out, rows, n_out, H, eps, post_plain, s);
    if (y_dtype == DT_BF16 && out_dtype == DT_BF16) return launch_layernorm<bf16, bf16>(x, y, w_post, clear_y, w_pre, b_pre, out, rows, n_out, H, eps, post_plain, s);
    return LLMIE_ERR_BAD_ARGUMENT;
}

LLMIE_API int llmie_group_rmsnorm_gate(const float* x, const void* gate, int gate_stride, int gate_dtype, const float* w, int w_len,
                                       void* out, int out_dtype, int N, int C, int gs, float eps, int mode, cudaStream_t s) {
    if (N <= 0) return 0;
    if (C <= 0 || gs <= 0 || C % gs || w_len <= 0 || C / gs > 65535 || mode < 0 || mode > 2) return LLMIE_ERR_BAD_ARGUMENT;
    int threads = 32;
    while (threads < 256 && threads * 2 <= gs) threads *= 2;
    const dim3 grid(N, C / gs);
    const long long items = (long long)N * (C / gs);
#define LLMIE_GRG(TG, TO)                                                                                                                        \
    {                                                                                                                                            \
        if (gs <= 256)   /* (the registers of a lane hold gs / 32 values: beyond 256 the block form is the better one) */                      \
            return launch_kernel(group_rmsnorm_gate_warp_kernel<TG, TO>, dim3((unsigned)((items + 3) / 4)), dim3(128), 0, s, x, (const TG*)gate, \
                                 gate_stride, w, w_len, (TO*)out, N, C, gs, eps, mode);                                                          \
        return launch_kernel(group_rmsnorm_gate_kernel<TG, TO>, grid, dim3(threads), 0, s, x, (const TG*)gate, gate_stride, w, w_len, (TO*)out,  \
                             C, gs, eps, mode);                                                                                                  \
    }
    if (gate_dtype == DT_F32 && out_dtype == DT_F32) LLMIE_GRG(float, float);
    if (gate_dtype == DT_BF16 && out_dtype == DT_BF16) LLMIE_GRG(bf16, bf16);
#undef LLMIE_GRG
    return LLMIE_ERR_BAD_ARGUMENT;
}

LLMIE_API int llmie_dual_rmsnorm_mix(void* a, int a_dtype, void* b, int b_dtype, const float* wa, const float* wb, float* y, int N, int H,
                                     float eps, float coef, int accumulate, int clear_a, int clear_b, cudaStream_t s) {
    if (N <= 0) return 0;
    if (H <= 0) return LLMIE_ERR_BAD_ARGUMENT;
    int threads = 32;
    while (threads < 512 && threads * 4 <= H) threads *= 2;
#define LLMIE_DUAL(TA, TB) return launch_kernel(dual_rmsnorm_mix_kernel<TA, TB>, dim3(N), dim3(threads), 0, s, (TA*)a, (TB*)b, wa, wb, y, H, eps, coef, \
                                                accumulate, clear_a, clear_b)
    if (a_dtype == DT_F32 && b_dtype == DT_F32) LLMIE_DUAL(float, float);
    if (a_dtype == DT_F32 && b_dtype == DT_BF16) LLMIE_DUAL(float, bf16);
    if (a_dtype == DT_BF16 && b_dtype == DT_F32) LLMIE_DUAL(bf16, float);
    if (a_dtype == DT_BF16 && b_dtype == DT_BF16) LLMIE_DUAL(bf16, bf16);
#undef LLMIE_DUAL
    return LLMIE_ERR_BAD_ARGUMENT;
}
