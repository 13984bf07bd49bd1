// A feed-forward of routed experts: the router's choice, the tokens sorted by expert, the experts' two products over the sorted
// rows (a grouped product: every tile of rows belongs to one expert and multiplies by that expert's matrix), and the weighted sum
// back into the residual stream. Everything is decided on the device (no host read of a count), so a step with routed experts is
// captured in a CUDA graph like any other. T is the storage type of activations and matrices (float or bfloat16); router scores,
// weights and the sum into the stream are 32-bit.
//
// The result of a token does not depend on what else is in the batch: a row of a grouped product is a sum over K in one fixed
// order whatever tile it falls into, and the weighted sum adds a token's experts in the order of its choice.
#include <math.h>

#include "common.cuh"

namespace {

constexpr int ROUTE_MAX_PER_LANE = 16;   // up to 512 router outputs
constexpr int MOE_TM = 32;               // rows of a tile of the grouped product
constexpr int MOE_TN = 64;
constexpr int MOE_TK = 16;
constexpr int SORT_THREADS = 1024;
constexpr int SORT_MAX_EXPERTS = 4096;

// One warp per token: s = softmax(logits) over all `total` router outputs; the `top` outputs with the largest s + correction are
// chosen (of equal scores the lower index first); their weights are s / (sum of the chosen s + 1e-20).
__global__ void __launch_bounds__(128) moe_route_kernel(const float* __restrict__ logits, const float* __restrict__ correction,
                                                        int* __restrict__ ids, float* __restrict__ weights, int N, int total, int top) {
    pdl_trigger();
    pdl_wait();
    const int n = blockIdx.x * 4 + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    if (n >= N) return;
    float s[ROUTE_MAX_PER_LANE], c[ROUTE_MAX_PER_LANE];
    float mx = -INFINITY;
#pragma unroll
    for (int j = 0; j < ROUTE_MAX_PER_LANE; ++j) {
        const int e = lane + 32 * j;
        s[j] = e < total ? logits[(size_t)n * total + e] : -INFINITY;
        mx = fmaxf(mx, s[j]);
    }
    mx = warp_max(mx);
    float sum = 0.f;
#pragma unroll
    for (int j = 0; j < ROUTE_MAX_PER_LANE; ++j) {
        const int e = lane + 32 * j;
        s[j] = e < total ? expf(s[j] - mx) : 0.f;
        sum += s[j];
    }
    sum = warp_sum(sum);
#pragma unroll
    for (int j = 0; j < ROUTE_MAX_PER_LANE; ++j) {
        const int e = lane + 32 * j;
        s[j] = s[j] / sum;
        c[j] = e < total ? s[j] + (correction ? correction[e] : 0.f) : -INFINITY;
    }
    float chosen_sum = 0.f;
    float my_w = 0.f;      // lane k keeps the k-th choice
    int my_id = 0;
    for (int k = 0; k < top; ++k) {
        float best = -INFINITY;
        int best_e = 0x7fffffff;
#pragma unroll
        for (int j = 0; j < ROUTE_MAX_PER_LANE; ++j) {
            const int e = lane + 32 * j;
            if (c[j] > best) { best = c[j]; best_e = e; }   // (ascending e within a lane: the lower index wins a tie)
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, o);
            const int oe = __shfl_xor_sync(0xffffffffu, best_e, o);
            if (ob > best || (ob == best && oe < best_e)) { best = ob; best_e = oe; }
        }
        float w = 0.f;
#pragma unroll
        for (int j = 0; j < ROUTE_MAX_PER_LANE; ++j)
            if (lane + 32 * j == best_e) { w = s[j]; c[j] = -INFINITY; }
        w = warp_sum(w);   // only the owner's lane holds it
        chosen_sum += w;
        if (lane == (k & 31)) { my_w = w; my_id = best_e; }
        if ((k & 31) == 31 || k == top - 1) {   // (more than 32 choices: written in rounds)
            // weights are divided below, once the sum is known: keep raw values in global memory for now
            const int k0 = k & ~31;
            if (k0 + lane <= k) { ids[(size_t)n * top + k0 + lane] = my_id; weights[(size_t)n * top + k0 + lane] = my_w; }
        }
    }
    __syncwarp();
    const float inv = 1.0f / (chosen_sum + 1e-20f);
    for (int k = lane; k < top; k += 32) weights[(size_t)n * top + k] *= inv;
}

// One block: the step's (token, choice) pairs counted per expert, the experts' runs laid out one behind the other, every pair
// given a place in its expert's run, and the runs cut into tiles of `tile_rows` rows. Choices of identity experts (ids >= E)
// take no place (place_of = -1).
//   offsets [E + 1]; perm [pairs]: place -> pair; place_of [pairs]: pair -> place or -1;
//   tiles [1 + 2 * max_tiles]: the number of tiles, then (expert, first place) of each
__global__ void __launch_bounds__(SORT_THREADS) moe_sort_kernel(const int* __restrict__ ids, int pairs, int E, int tile_rows, int* __restrict__ offsets,
                                                                 int* __restrict__ perm, int* __restrict__ place_of, int* __restrict__ tiles, int max_tiles) {
    __shared__ int count[SORT_MAX_EXPERTS];
    __shared__ int cursor[SORT_MAX_EXPERTS];
    pdl_trigger();
    for (int e = threadIdx.x; e < E; e += SORT_THREADS) count[e] = 0;
    pdl_wait();
    __syncthreads();
    for (int i = threadIdx.x; i < pairs; i += SORT_THREADS) {
        const int e = ids[i];
        if (e >= 0 && e < E) atomicAdd(&count[e], 1);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        int at = 0, nt = 0;
        for (int e = 0; e < E; ++e) {
            offsets[e] = at;
            cursor[e] = at;
            for (int r = 0; r < count[e]; r += tile_rows) {
                if (nt < max_tiles) { tiles[1 + 2 * nt] = e; tiles[2 + 2 * nt] = at + r; }
                ++nt;
            }
            at += count[e];
        }
        offsets[E] = at;
        tiles[0] = min(nt, max_tiles);
    }
    __syncthreads();
    for (int i = threadIdx.x; i < pairs; i += SORT_THREADS) {
        const int e = ids[i];
        if (e >= 0 && e < E) {
            const int p = atomicAdd(&cursor[e], 1);
            perm[p] = i;
            place_of[i] = p;
        } else {
            place_of[i] = -1;
        }
    }
}

__device__ __forceinline__ float silu_f(float x) { return x / (1.0f + expf(-x)); }

// The grouped product on the CUDA cores, one tile of MOE_TM places x MOE_TN outputs per block, the tile's expert from the list.
//   GATED: out[place, j] = silu(a . Wg[e][j]) * (a . Wu[e][j]) with W [E][2 F][K] (an expert's gate rows, then its up rows), out of type TO
//   else:  out[place, j] = a . W[e][j] with W [E][F][K]
// The row a of a place is x[row_map[place] / row_div] (the token of the pair that sits there), or x[place] without a map.
template <typename T, typename TO, bool GATED>
__global__ void __launch_bounds__(256) moe_gemm_kernel(const T* __restrict__ x, const int* __restrict__ row_map, int row_div, const T* __restrict__ w,
                                                       const int* __restrict__ offsets, const int* __restrict__ tiles, TO* __restrict__ out, int F,
                                                       int K) {
    __shared__ float a_s[MOE_TK][MOE_TM + 1];
    __shared__ float b_s[GATED ? 2 : 1][MOE_TK][MOE_TN + 1];
    __shared__ int rows_s[MOE_TM];
    pdl_trigger();
    pdl_wait();
    if ((int)blockIdx.y >= tiles[0]) return;
    const int e = tiles[1 + 2 * blockIdx.y], p0 = tiles[2 + 2 * blockIdx.y];
    const int p_end = min(offsets[e + 1], p0 + MOE_TM);
    const int n0 = blockIdx.x * MOE_TN;
    if (threadIdx.x < MOE_TM) {
        const int p = p0 + threadIdx.x;
        rows_s[threadIdx.x] = p < p_end ? (row_map ? row_map[p] / row_div : p) : -1;
    }
    __syncthreads();
    const T* we = w + (size_t)e * (GATED ? 2 : 1) * F * K;
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;   // outputs 4 tx .. 4 tx + 3 of places 2 ty, 2 ty + 1
    float acc[GATED ? 2 : 1][2][4] = {};
    for (int k0 = 0; k0 < K; k0 += MOE_TK) {
        for (int i = threadIdx.x; i < MOE_TM * MOE_TK; i += 256) {
            const int m = i / MOE_TK, k = i % MOE_TK;
            const int r = rows_s[m];
            a_s[k][m] = (r >= 0 && k0 + k < K) ? to_f32(x[(size_t)r * K + k0 + k]) : 0.f;
        }
        for (int i = threadIdx.x; i < MOE_TN * MOE_TK; i += 256) {
            const int n = i / MOE_TK, k = i % MOE_TK;
            const bool in = n0 + n < F && k0 + k < K;
            b_s[0][k][n] = in ? to_f32(we[(size_t)(n0 + n) * K + k0 + k]) : 0.f;
            if (GATED) b_s[GATED ? 1 : 0][k][n] = in ? to_f32(we[(size_t)(F + n0 + n) * K + k0 + k]) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < MOE_TK; ++k) {
            const float a0 = a_s[k][2 * ty], a1 = a_s[k][2 * ty + 1];
#pragma unroll
            for (int h = 0; h < (GATED ? 2 : 1); ++h) {
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const float b = b_s[h][k][4 * tx + j];
                    acc[h][0][j] = fmaf(a0, b, acc[h][0][j]);
                    acc[h][1][j] = fmaf(a1, b, acc[h][1][j]);
                }
            }
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        const int p = p0 + 2 * ty + i;
        if (p >= p_end) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int n = n0 + 4 * tx + j;
            if (n >= F) continue;
            const float v = GATED ? silu_f(acc[0][i][j]) * acc[GATED ? 1 : 0][i][j] : acc[0][i][j];
            out[(size_t)p * F + n] = from_f32<TO>(v);
        }
    }
}

// residual[t] += sum_k weight[t, k] * (y[place_of[t, k]] for an expert with matrices, h[t] itself for an identity expert), the
// experts of a token in the order of its choice. One block per token.
template <typename T>
__global__ void moe_combine_kernel(float* __restrict__ residual, const float* __restrict__ y, const T* __restrict__ h, const int* __restrict__ place_of,
                                   const float* __restrict__ weights, int top, int W) {
    pdl_trigger();
    pdl_wait();
    const int t = blockIdx.x;
    for (int i = threadIdx.x; i < W; i += blockDim.x) {
        float sum = 0.f;
        for (int k = 0; k < top; ++k) {
            const int p = place_of[(size_t)t * top + k];
            const float v = p >= 0 ? y[(size_t)p * W + i] : to_f32(h[(size_t)t * W + i]);
            sum = fmaf(weights[(size_t)t * top + k], v, sum);
        }
        residual[(size_t)t * W + i] += sum;
    }
}

}  // namespace

LLMIE_API int llmie_moe_route(const float* logits, const float* correction, int* ids, float* weights, int N, int total, int top, cudaStream_t s) {
    if (N <= 0) return 0;
    if (total <= 0 || total > 32 * ROUTE_MAX_PER_LANE || top <= 0 || top > total) return LLMIE_ERR_BAD_ARGUMENT;
    return launch_kernel(moe_route_kernel, dim3((N + 3) / 4), dim3(128), 0, s, logits, correction, ids, weights, N, total, top);
}

LLMIE_API int llmie_moe_tile_rows() { return MOE_TM; }

LLMIE_API int llmie_moe_sort(const int* ids, int pairs, int E, int* offsets, int* perm, int* place_of, int* tiles, int max_tiles, cudaStream_t s) {
    if (pairs <= 0) return 0;
    if (E <= 0 || E > SORT_MAX_EXPERTS || max_tiles <= 0) return LLMIE_ERR_BAD_ARGUMENT;
    return launch_kernel(moe_sort_kernel, dim3(1), dim3(SORT_THREADS), 0, s, ids, pairs, E, MOE_TM, offsets, perm, place_of, tiles, max_tiles);
}

// gated != 0: w [E][2 F][K], out [places][F] of the storage type; else w [E][F][K], out [places][F] float.
LLMIE_API int llmie_moe_gemm(const void* x, const int* row_map, int row_div, const void* w, const int* offsets, const int* tiles, int max_tiles,
                             void* out, int F, int K, int gated, int dtype, cudaStream_t s) {
    if (max_tiles <= 0) return 0;
    if (F <= 0 || K <= 0 || max_tiles > 65535 || (row_map && row_div <= 0)) return LLMIE_ERR_BAD_ARGUMENT;
    const dim3 grid((F + MOE_TN - 1) / MOE_TN, max_tiles);
    if (dtype == DT_F32) {
        if (gated) return launch_kernel(moe_gemm_kernel<float, float, true>, grid, dim3(256), 0, s, (const float*)x, row_map, row_div, (const float*)w, offsets, tiles, (float*)out, F, K);
        return launch_kernel(moe_gemm_kernel<float, float, false>, grid, dim3(256), 0, s, (const float*)x, row_map, row_div, (const float*)w, offsets, tiles, (float*)out, F, K);
    }
    if (gated) return launch_kernel(moe_gemm_kernel<bf16, bf16, true>, grid, dim3(256), 0, s, (const bf16*)x, row_map, row_div, (const bf16*)w, offsets, tiles, (bf16*)out, F, K);
    return launch_kernel(moe_gemm_kernel<bf16, float, false>, grid, dim3(256), 0, s, (const bf16*)x, row_map, row_div, (const bf16*)w, offsets, tiles, (float*)out, F, K);
}

LLMIE_API int llmie_moe_combine(float* residual, const float* y, const void* h, const int* place_of, const float* weights, int N, int top, int W,
                                int dtype, cudaStream_t s) {
    if (N <= 0) return 0;
    if (top <= 0 || W <= 0) return LLMIE_ERR_BAD_ARGUMENT;
    int threads = 32;
    while (threads < 256 && threads * 2 <= W) threads *= 2;
    if (dtype == DT_F32) return launch_kernel(moe_combine_kernel<float>, dim3(N), dim3(threads), 0, s, residual, y, (const float*)h, place_of, weights, top, W);
    return launch_kernel(moe_combine_kernel<bf16>, dim3(N), dim3(threads), 0, s, residual, y, (const bf16*)h, place_of, weights, top, W);
}
