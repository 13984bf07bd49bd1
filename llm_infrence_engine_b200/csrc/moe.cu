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
constexpr int MOE_TM = 4;                // most rows of a tile of the grouped product on the CUDA cores
constexpr int MOE_COLS = 32;             // outputs per block there
constexpr int MOE_ROWS_SMEM = 96 * 1024; // what a tile's rows may take of shared memory
constexpr int SORT_THREADS = 1024;
constexpr int SORT_MAX_EXPERTS = 4096;

// One warp per token: s = softmax(logits) over all `total` router outputs; the `top` outputs with the largest s + correction are
// chosen (of equal scores the lower index first); their weights are s / (sum of the chosen s + 1e-20).
// (one warp: token n's row of logits, in global or shared memory)
// `scoring` 1 instead: s = sigmoid(logits), every output by itself, and the weights are the chosen s as they are (not renormalised).
__device__ __forceinline__ void route_token(const float* __restrict__ row, const float* __restrict__ correction, int* __restrict__ ids,
                                            float* __restrict__ weights, int n, int total, int top, int lane, int scoring) {
    float s[ROUTE_MAX_PER_LANE], c[ROUTE_MAX_PER_LANE];
    float mx = -INFINITY;
#pragma unroll
    for (int j = 0; j < ROUTE_MAX_PER_LANE; ++j) {
        const int e = lane + 32 * j;
        s[j] = e < total ? row[e] : -INFINITY;
        mx = fmaxf(mx, s[j]);
    }
    mx = warp_max(mx);
    float sum = 0.f;
#pragma unroll
    for (int j = 0; j < ROUTE_MAX_PER_LANE; ++j) {
        const int e = lane + 32 * j;
        if (scoring == 1) s[j] = e < total ? 1.0f / (1.0f + expf(-s[j])) : 0.f;
        else s[j] = e < total ? expf(s[j] - mx) : 0.f;
        sum += s[j];
    }
    sum = scoring == 1 ? 1.f : warp_sum(sum);
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
    const float inv = scoring == 1 ? 1.0f : 1.0f / (chosen_sum + 1e-20f);
    for (int k = lane; k < top; k += 32) weights[(size_t)n * top + k] *= inv;
}

__global__ void __launch_bounds__(128) moe_route_kernel(const float* __restrict__ logits, const float* __restrict__ correction,
                                                        int* __restrict__ ids, float* __restrict__ weights, int N, int total, int top, int scoring) {
    pdl_trigger();
    pdl_wait();
    const int n = blockIdx.x * 4 + (threadIdx.x >> 5);
    if (n >= N) return;
    route_token(logits + (size_t)n * total, correction, ids, weights, n, total, top, threadIdx.x & 31, scoring);
}

// The router's product and its choice in one kernel, a block per token: the token's row lies in shared memory as floats, the warps
// share the router's outputs (a warp's lanes walk an output's weight row in 16-byte pieces; the sum runs over K in one order whatever
// the step holds), and the first warp chooses from the logits in shared memory. For the few rows of a decode step, where the product
// alone would be a kernel that walks K in one block.
constexpr int ROUTER_THREADS = 256;
template <typename T>
__global__ void __launch_bounds__(ROUTER_THREADS) moe_router_kernel(const T* __restrict__ h, const T* __restrict__ w, const float* __restrict__ correction,
                                                                    int* __restrict__ ids, float* __restrict__ weights, int K, int total, int top, int scoring) {
    extern __shared__ __align__(16) float router_smem[];   // [K] the row, then [total] the logits
    constexpr int VN = Vec16<T>::N;
    float* row = router_smem;
    float* logits = router_smem + ((K + 3) & ~3);
    pdl_trigger();
    const int n = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const bool vec = (K % VN) == 0 && ((uintptr_t)h & 15) == 0 && ((uintptr_t)w & 15) == 0;
    pdl_wait();
    const T* src = h + (size_t)n * K;
    if (vec) {
        for (int k = threadIdx.x * VN; k < K; k += ROUTER_THREADS * VN) {
            float v[VN];
            Vec16<T>::load(src + k, v);
#pragma unroll
            for (int i = 0; i < VN; ++i) row[k + i] = v[i];
        }
    } else {
        for (int k = threadIdx.x; k < K; k += ROUTER_THREADS) row[k] = to_f32(src[k]);
    }
    __syncthreads();
    for (int e = warp; e < total; e += ROUTER_THREADS / 32) {
        const T* we = w + (size_t)e * K;
        float acc = 0.f;
        if (vec) {
            for (int k = lane * VN; k < K; k += 32 * VN) {
                float v[VN];
                Vec16<T>::load(we + k, v);
#pragma unroll
                for (int i = 0; i < VN; ++i) acc = fmaf(row[k + i], v[i], acc);
            }
        } else {
            for (int k = lane; k < K; k += 32) acc = fmaf(row[k], to_f32(we[k]), acc);
        }
        acc = warp_sum(acc);
        if (lane == 0) logits[e] = acc;
    }
    __syncthreads();
    if (warp == 0) route_token(logits, correction, ids, weights, n, total, top, lane, scoring);
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

// The grouped product on the CUDA cores for FEW rows per expert (decode steps) and for float32: a tile is up to `tile_rows` (at
// most MOE_TM) places of one expert, whose rows of K numbers lie in shared memory as floats; a block owns MOE_COLS outputs, a warp
// MOE_COLS / 8 of them, taken together: the lanes walk the outputs' weight rows (and, GATED, the up rows of the same outputs)
// 16 bytes at a time, so the matrices are read once per tile in full lines, which is what bounds a decode step.
//   GATED: out[place, j] = silu(a . Wg[e][j]) * (a . Wu[e][j]) with W [E][2 F][K] (an expert's gate rows, then its up rows), out of type TO;
//          with limit > 0 the unit is min(g, limit) * sigmoid(alpha g) * (clamp(u, -limit, limit) + shift);
//          with row_scale the row a is first multiplied by row_scale[pair] (a weight on the expert's input, rounded as it would be stored)
//   else:  out[place, j] = a . W[e][j] with W [E][F][K]
// The row a of a place is x[row_map[place] / row_div] (the token of the pair that sits there), or x[place] without a map.
// A sum runs over K in one order whatever the tile holds: a place's result does not depend on its neighbours.
template <typename T, typename TO, bool GATED>
__global__ void __launch_bounds__(256, 2) moe_rows_kernel(const T* __restrict__ x, const int* __restrict__ row_map, int row_div, const T* __restrict__ w,
                                                       const int* __restrict__ offsets, const int* __restrict__ tiles, TO* __restrict__ out, int F,
                                                       int K, int tile_rows, const float* __restrict__ row_scale, float limit, float alpha, float shift) {
    extern __shared__ __align__(16) float moe_rows_smem[];   // [tile_rows][K]
    constexpr int VN = Vec16<T>::N;
    pdl_trigger();
    pdl_wait();
    if ((int)blockIdx.y >= tiles[0]) return;
    const int e = tiles[1 + 2 * blockIdx.y], p0 = tiles[2 + 2 * blockIdx.y];
    const int count = min(offsets[e + 1] - p0, tile_rows);
    const bool vec = (K % VN) == 0 && ((uintptr_t)x & 15) == 0 && ((uintptr_t)w & 15) == 0;
    for (int r = 0; r < count; ++r) {
        const int p = p0 + r;
        const T* src = x + (size_t)(row_map ? row_map[p] / row_div : p) * K;
        const float rs = (row_scale && row_map) ? row_scale[row_map[p]] : 1.f;   // the pair's weight on the expert's INPUT
        float* dst = moe_rows_smem + (size_t)r * K;
        if (vec) {
            for (int k = threadIdx.x * VN; k < K; k += 256 * VN) {
                float v[VN];
                Vec16<T>::load(src + k, v);
#pragma unroll
                for (int i = 0; i < VN; ++i) dst[k + i] = row_scale ? round_through<T>(v[i] * rs) : v[i];
            }
        } else {
            for (int k = threadIdx.x; k < K; k += 256) dst[k] = row_scale ? round_through<T>(to_f32(src[k]) * rs) : to_f32(src[k]);
        }
    }
    __syncthreads();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const T* we = w + (size_t)e * (GATED ? 2 : 1) * F * K;
    constexpr int CPW = MOE_COLS / 8;   // a warp's outputs, taken together: their weight rows are in flight at once
    const int j0 = blockIdx.x * MOE_COLS + warp * CPW;
    if (j0 >= F) return;
    const T* wrow[CPW];
#pragma unroll
    for (int c = 0; c < CPW; ++c) wrow[c] = we + (size_t)min(j0 + c, F - 1) * K;   // (an output past the end repeats the last: not stored)
    const size_t up = (size_t)F * K;   // from an output's gate row to its up row (read only when GATED)
    float ag[CPW][MOE_TM] = {}, au[GATED ? CPW : 1][MOE_TM] = {};
    if (vec) {
        for (int k = lane * VN; k < K; k += 32 * VN) {
            float g[CPW][VN], u[GATED ? CPW : 1][VN];
#pragma unroll
            for (int c = 0; c < CPW; ++c) {
                Vec16<T>::load(wrow[c] + k, g[c]);
                if (GATED) Vec16<T>::load(wrow[c] + up + k, u[GATED ? c : 0]);
            }
#pragma unroll
            for (int r = 0; r < MOE_TM; ++r) {
                if (r < count) {
                    const float* a = moe_rows_smem + (size_t)r * K + k;
#pragma unroll
                    for (int i = 0; i < VN; i += 4) {
                        const float4 av = *reinterpret_cast<const float4*>(a + i);
#pragma unroll
                        for (int c = 0; c < CPW; ++c) {
                            ag[c][r] = fmaf(av.x, g[c][i], ag[c][r]); ag[c][r] = fmaf(av.y, g[c][i + 1], ag[c][r]);
                            ag[c][r] = fmaf(av.z, g[c][i + 2], ag[c][r]); ag[c][r] = fmaf(av.w, g[c][i + 3], ag[c][r]);
                            if (GATED) {
                                float& s = au[GATED ? c : 0][r];
                                s = fmaf(av.x, u[GATED ? c : 0][i], s); s = fmaf(av.y, u[GATED ? c : 0][i + 1], s);
                                s = fmaf(av.z, u[GATED ? c : 0][i + 2], s); s = fmaf(av.w, u[GATED ? c : 0][i + 3], s);
                            }
                        }
                    }
                }
            }
        }
    } else {
        for (int k = lane; k < K; k += 32) {
            float g[CPW], u[GATED ? CPW : 1];
#pragma unroll
            for (int c = 0; c < CPW; ++c) {
                g[c] = to_f32(wrow[c][k]);
                if (GATED) u[GATED ? c : 0] = to_f32(wrow[c][up + k]);
            }
#pragma unroll
            for (int r = 0; r < MOE_TM; ++r) {
                if (r < count) {
                    const float a = moe_rows_smem[(size_t)r * K + k];
#pragma unroll
                    for (int c = 0; c < CPW; ++c) {
                        ag[c][r] = fmaf(a, g[c], ag[c][r]);
                        if (GATED) au[GATED ? c : 0][r] = fmaf(a, u[GATED ? c : 0], au[GATED ? c : 0][r]);
                    }
                }
            }
        }
    }
#pragma unroll
    for (int r = 0; r < MOE_TM; ++r) {
        if (r < count) {
#pragma unroll
            for (int c = 0; c < CPW; ++c) {
                const float sg = warp_sum(ag[c][r]);
                const float su = GATED ? warp_sum(au[GATED ? c : 0][r]) : 0.f;
                float res = sg;
                if (GATED) {
                    if (limit > 0.f) {   // the clamped unit
                        const float g = fminf(sg, limit), u = fminf(fmaxf(su, -limit), limit) + shift;
                        res = g / (1.0f + expf(-alpha * g)) * u;
                    } else {
                        res = silu_f(sg) * su;
                    }
                }
                if (lane == 0 && j0 + c < F) out[(size_t)(p0 + r) * F + j0 + c] = from_f32<TO>(res);
            }
        }
    }
}

// xs[place] = x[perm[place] / top] (times row_scale[perm[place]], where given) for the places that the sort filled (offsets[E] of them): the rows of the tokens, in the order
// of their experts, as the tensor-core grouped product reads them. One block per place.
__global__ void moe_gather_kernel(const bf16* __restrict__ x, const int* __restrict__ perm, const int* __restrict__ offsets, int E, int top,
                                  bf16* __restrict__ xs, int K, const float* __restrict__ row_scale) {
    pdl_trigger();
    pdl_wait();
    const int p = blockIdx.x;
    if (p >= offsets[E]) return;
    const uint4* src = reinterpret_cast<const uint4*>(x + (size_t)(perm[p] / top) * K);
    uint4* dst = reinterpret_cast<uint4*>(xs + (size_t)p * K);
    if (!row_scale) {
        for (int i = threadIdx.x; i < K / 8; i += blockDim.x) dst[i] = src[i];
        return;
    }
    const float rs = row_scale[perm[p]];   // the pair's weight on the expert's input
    for (int i = threadIdx.x; i < K / 8; i += blockDim.x) {
        float v[8];
        Vec16<bf16>::load(reinterpret_cast<const bf16*>(src + i), v);
        uint32_t w[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const __nv_bfloat162 b = __floats2bfloat162_rn(v[2 * j] * rs, v[2 * j + 1] * rs);
            w[j] = *reinterpret_cast<const uint32_t*>(&b);
        }
        dst[i] = make_uint4(w[0], w[1], w[2], w[3]);
    }
}

// residual[t] += sum_k weight[t, k] * (y[place_of[t, k]] for an expert with matrices, h[t] itself for an identity expert), the
// experts of a token in the order of its choice. Block (t, c): COMBINE_VEC columns per thread of token t from column
// c * blockDim.x * COMBINE_VEC on; the rows of a token's experts are fetched side by side (COMBINE_VEC 4: rows of 16-byte pieces).
template <typename T, int COMBINE_VEC>
__global__ void __launch_bounds__(256) moe_combine_kernel(float* __restrict__ residual, const float* __restrict__ y, const T* __restrict__ h,
                                                          const int* __restrict__ place_of, const float* __restrict__ weights, int top, int W) {
    pdl_trigger();
    pdl_wait();
    const int t = blockIdx.x;
    const int i = (blockIdx.y * blockDim.x + threadIdx.x) * COMBINE_VEC;
    if (i >= W) return;
    float sum[COMBINE_VEC] = {};
    for (int k = 0; k < top; ++k) {
        const int p = place_of[(size_t)t * top + k];
        const float wk = weights ? weights[(size_t)t * top + k] : 1.f;   // (no weights: they were put on the experts' inputs)
        float v[COMBINE_VEC];
        if (p >= 0) {
            if (COMBINE_VEC == 4) {
                const float4 q = *reinterpret_cast<const float4*>(y + (size_t)p * W + i);
                v[0] = q.x; v[1 % COMBINE_VEC] = q.y; v[2 % COMBINE_VEC] = q.z; v[3 % COMBINE_VEC] = q.w;
            } else {
                v[0] = y[(size_t)p * W + i];
            }
        } else {
#pragma unroll
            for (int j = 0; j < COMBINE_VEC; ++j) v[j] = to_f32(h[(size_t)t * W + i + j]);
        }
#pragma unroll
        for (int j = 0; j < COMBINE_VEC; ++j) sum[j] = fmaf(wk, v[j], sum[j]);
    }
    float* r = residual + (size_t)t * W + i;
    if (COMBINE_VEC == 4) {
        float4 q = *reinterpret_cast<float4*>(r);
        q.x += sum[0]; q.y += sum[1 % COMBINE_VEC]; q.z += sum[2 % COMBINE_VEC]; q.w += sum[3 % COMBINE_VEC];
        *reinterpret_cast<float4*>(r) = q;
    } else {
        r[0] += sum[0];
    }
}

}  // namespace

LLMIE_API int llmie_moe_route(const float* logits, const float* correction, int* ids, float* weights, int N, int total, int top, int scoring,
                              cudaStream_t s) {
    if (N <= 0) return 0;
    if (total <= 0 || total > 32 * ROUTE_MAX_PER_LANE || top <= 0 || top > total) return LLMIE_ERR_BAD_ARGUMENT;
    return launch_kernel(moe_route_kernel, dim3((N + 3) / 4), dim3(128), 0, s, logits, correction, ids, weights, N, total, top, scoring);
}

// ids, weights [N, top] from the rows h [N, K] and the router's matrix w [total, K] of the same type (float or bfloat16): the product in
// 32-bit and the choice, one launch. The row and the logits must fit the shared memory (K + total floats: up to about 50,000).
LLMIE_API int llmie_moe_router(const void* h, const void* w, const float* correction, int* ids, float* weights, int N, int K, int total, int top,
                               int scoring, int dtype, cudaStream_t s) {
    if (N <= 0) return 0;
    if (K <= 0 || total <= 0 || total > 32 * ROUTE_MAX_PER_LANE || top <= 0 || top > total) return LLMIE_ERR_BAD_ARGUMENT;
    const size_t smem = ((size_t)((K + 3) & ~3) + total) * sizeof(float);
    if (smem > 200 * 1024) return LLMIE_ERR_BAD_ARGUMENT;
    static size_t allowed_f = 48 * 1024, allowed_b = 48 * 1024;
    if (dtype == DT_F32) {
        if (smem > allowed_f) {
            cudaError_t e = cudaFuncSetAttribute(moe_router_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
            if (e != cudaSuccess) return (int)e;
            allowed_f = 200 * 1024;
        }
        return launch_kernel(moe_router_kernel<float>, dim3(N), dim3(ROUTER_THREADS), smem, s, (const float*)h, (const float*)w, correction, ids, weights, K,
                             total, top, scoring);
    }
    if (smem > allowed_b) {
        cudaError_t e = cudaFuncSetAttribute(moe_router_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
        if (e != cudaSuccess) return (int)e;
        allowed_b = 200 * 1024;
    }
    return launch_kernel(moe_router_kernel<bf16>, dim3(N), dim3(ROUTER_THREADS), smem, s, (const bf16*)h, (const bf16*)w, correction, ids, weights, K, total,
                         top, scoring);
}

// Rows per tile of the grouped product on the CUDA cores for rows of K numbers: as many as fit the shared memory, at most MOE_TM;
// 0: the rows are too long for it.
LLMIE_API int llmie_moe_tile_rows(int K) {
    if (K <= 0) return 0;
    const long long fit = MOE_ROWS_SMEM / ((long long)K * 4);
    return (int)(fit > MOE_TM ? MOE_TM : fit);
}

// tile_rows: the most places of a tile (what the product that follows wants: llmie_moe_tile_rows(K), or 128 for the tensor cores).
LLMIE_API int llmie_moe_sort(const int* ids, int pairs, int E, int tile_rows, int* offsets, int* perm, int* place_of, int* tiles, int max_tiles,
                             cudaStream_t s) {
    if (pairs <= 0) return 0;
    if (E <= 0 || E > SORT_MAX_EXPERTS || max_tiles <= 0 || tile_rows <= 0) return LLMIE_ERR_BAD_ARGUMENT;
    return launch_kernel(moe_sort_kernel, dim3(1), dim3(SORT_THREADS), 0, s, ids, pairs, E, tile_rows, offsets, perm, place_of, tiles, max_tiles);
}

template <typename T, typename TO, bool GATED>
static int launch_moe_rows(const void* x, const int* row_map, int row_div, const void* w, const int* offsets, const int* tiles, int max_tiles, void* out,
                           int F, int K, int tile_rows, const float* row_scale, float limit, float alpha, float shift, cudaStream_t s) {
    const size_t smem = (size_t)tile_rows * K * sizeof(float);
    static size_t allowed = 48 * 1024;
    if (smem > allowed) {
        cudaError_t e = cudaFuncSetAttribute(moe_rows_kernel<T, TO, GATED>, cudaFuncAttributeMaxDynamicSharedMemorySize, MOE_ROWS_SMEM);
        if (e != cudaSuccess) return (int)e;
        allowed = MOE_ROWS_SMEM;
    }
    const dim3 grid((F + MOE_COLS - 1) / MOE_COLS, max_tiles);
    return launch_kernel(moe_rows_kernel<T, TO, GATED>, grid, dim3(256), smem, s, (const T*)x, row_map, row_div, (const T*)w, offsets, tiles, (TO*)out, F, K,
                         tile_rows, row_scale, limit, alpha, shift);
}

// gated != 0: w [E][2 F][K], out [places][F] of the storage type; else w [E][F][K], out [places][F] float. tile_rows as given to the sort.
// row_scale [pairs] or null: a weight on every pair's input row (needs row_map); limit > 0: the clamped unit (see the kernel).
LLMIE_API int llmie_moe_gemm(const void* x, const int* row_map, int row_div, const void* w, const int* offsets, const int* tiles, int max_tiles,
                             void* out, int F, int K, int gated, int tile_rows, const float* row_scale, float limit, float alpha, float shift, int dtype,
                             cudaStream_t s) {
    if (max_tiles <= 0) return 0;
    if (F <= 0 || K <= 0 || max_tiles > 65535 || (row_map && row_div <= 0) || tile_rows <= 0 || tile_rows > MOE_TM || tile_rows > llmie_moe_tile_rows(K))
        return LLMIE_ERR_BAD_ARGUMENT;
    if (dtype == DT_F32) {
        if (gated) return launch_moe_rows<float, float, true>(x, row_map, row_div, w, offsets, tiles, max_tiles, out, F, K, tile_rows, row_scale, limit, alpha, shift, s);
        return launch_moe_rows<float, float, false>(x, row_map, row_div, w, offsets, tiles, max_tiles, out, F, K, tile_rows, row_scale, limit, alpha, shift, s);
    }
    if (gated) return launch_moe_rows<bf16, bf16, true>(x, row_map, row_div, w, offsets, tiles, max_tiles, out, F, K, tile_rows, row_scale, limit, alpha, shift, s);
    return launch_moe_rows<bf16, float, false>(x, row_map, row_div, w, offsets, tiles, max_tiles, out, F, K, tile_rows, row_scale, limit, alpha, shift, s);
}

// xs [pairs][K] bfloat16 (K a multiple of 8, 16-byte aligned rows): the tokens' rows in the order of the sort.
LLMIE_API int llmie_moe_gather(const void* x, const int* perm, const int* offsets, int E, int top, void* xs, int pairs, int K, const float* row_scale,
                               cudaStream_t s) {
    if (pairs <= 0) return 0;
    if (K <= 0 || K % 8 || top <= 0 || ((uintptr_t)x & 15) || ((uintptr_t)xs & 15)) return LLMIE_ERR_BAD_ARGUMENT;
    return launch_kernel(moe_gather_kernel, dim3(pairs), dim3(K / 8 < 256 ? (K / 8 < 32 ? 32 : K / 8) : 256), 0, s, (const bf16*)x, perm, offsets, E, top,
                         (bf16*)xs, K, row_scale);
}

LLMIE_API int llmie_moe_combine(float* residual, const float* y, const void* h, const int* place_of, const float* weights, int N, int top, int W,
                                int dtype, cudaStream_t s) {
    if (N <= 0) return 0;
    if (top <= 0 || W <= 0) return LLMIE_ERR_BAD_ARGUMENT;
    const bool vec = W % 4 == 0 && (((uintptr_t)residual | (uintptr_t)y) & 15) == 0;
    const int per = vec ? 4 : 1;
    int threads = 32;
    while (threads < 256 && threads * per < W) threads *= 2;
    const dim3 grid(N, (W + threads * per - 1) / (threads * per));
    if (grid.y > 65535) return LLMIE_ERR_BAD_ARGUMENT;
    if (dtype == DT_F32) {
        if (vec) return launch_kernel(moe_combine_kernel<float, 4>, grid, dim3(threads), 0, s, residual, y, (const float*)h, place_of, weights, top, W);
        return launch_kernel(moe_combine_kernel<float, 1>, grid, dim3(threads), 0, s, residual, y, (const float*)h, place_of, weights, top, W);
    }
    if (vec) return launch_kernel(moe_combine_kernel<bf16, 4>, grid, dim3(threads), 0, s, residual, y, (const bf16*)h, place_of, weights, top, W);
    return launch_kernel(moe_combine_kernel<bf16, 1>, grid, dim3(threads), 0, s, residual, y, (const bf16*)h, place_of, weights, top, W);
}
