// Paged attention whose heads talk to each other before the softmax: the scaled (and capped) scores of all query heads at one
// (query, key) pair are mixed by a matrix, score'_h = sum_g talk[h][g] score_g, and only then masked and normalised. A head's weights
// therefore need every head's scores, so one block serves ALL heads of a token, for one slice of its keys:
//
//   1. scores: a lane owns a key, walks its row once per group of query heads, and leaves cap(scale q_g . k) for every head g;
//   2. mix:    a thread owns a key and forms the H mixed scores from the H plain ones (the matrix lies in shared memory);
//   3. weights: a warp owns a head: maximum, exponentials and their sum over the slice's keys;
//   4. values: a thread owns output entries (head, dim) and sums weight * value over the slice's keys, in key order.
//
// Slices lie at fixed places of a request (`slice_keys`, at most TALK_MAX_SLICE), so every bit of a token's result depends on its own
// position alone; several slices are merged, and sink and output gate applied, by the merge kernel of the attention with extras
// (one slice: in this kernel, by the same formula). Storage is float or bfloat16, all arithmetic 32-bit. Window, kept first tokens
// and chunks are honoured as in the other kernels of the family; `talk == nullptr` leaves the scores unmixed.
#include "attention_ext.cuh"

namespace {

constexpr int TALK_THREADS = 256;
constexpr int TALK_WARPS = TALK_THREADS / 32;
constexpr int TALK_MAX_SLICE = 128;   // (with 256 a decode step of 8 requests at 4,096 keys has fewer blocks than there are multiprocessors)
constexpr int TALK_GC = 4;   // query heads of a group whose scores a lane forms from one pass over its key row
constexpr int TALK_MAX_E = 16;   // output entries (head, dim) per thread that the staged form of the value product keeps in registers
constexpr int TALK_V_CHUNK = 32;   // keys whose values are staged at a time, at most

// floats (and integers) of the block's arrays before the staged values, rounded up to 16 bytes
__host__ __device__ inline size_t talk_floats(int nq, int dk, int slice_keys) {
    const int dkp = (dk + 3) & ~3;
    const size_t n = (size_t)nq * dkp + (size_t)nq * nq + 2 * (size_t)nq * slice_keys + 2 * nq + slice_keys;
    return (n + 3) & ~(size_t)3;
}

template <typename T>
__global__ void __launch_bounds__(TALK_THREADS) paged_attn_talk_kernel(
    const T* __restrict__ q, int q_stride, const T* __restrict__ k_pool, const T* __restrict__ v_pool, const int* __restrict__ block_table,
    int max_blocks, const int* __restrict__ token_seq, const int* __restrict__ positions, const float* __restrict__ talk, T* __restrict__ out,
    float* __restrict__ part_acc, float* __restrict__ part_ml, int nq, int nkv, int dk, int dv, int page_size, float scale, int window,
    int num_splits, int slice_keys, int vec_ok, int v_chunk, attn_ext::Extras ex) {
    extern __shared__ __align__(16) float talk_smem[];
    const int dkp = (dk + 3) & ~3;
    float* qs = talk_smem;                       // [nq][dkp]
    float* tm = qs + (size_t)nq * dkp;           // [nq][nq]
    float* sc = tm + (size_t)nq * nq;            // [nq][slice_keys]: capped scores
    float* sm = sc + (size_t)nq * slice_keys;    // [nq][slice_keys]: mixed scores, then weights
    float* ml = sm + (size_t)nq * slice_keys;    // [2 nq]: maximum and sum per head
    int* rows = reinterpret_cast<int*>(ml + 2 * nq);   // [slice_keys]: the key's row of kv head 0 in the pools

    const int n = blockIdx.x, split = blockIdx.y;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int G = nq / nkv;
    const int p = positions[n];
    const int lo = attn_ext::first_visible(p, window, ex);
    const int kept = min(ex.keep_first, lo);
    const int hi = p + 1;
    const int start = split * slice_keys;
    const int end = min(hi, start + slice_keys);
    const int cnt = max(0, end - start);
    const T* gate_row = ex.gate_mode ? reinterpret_cast<const T*>(ex.gate) + (size_t)n * ex.gate_stride : nullptr;

    if (cnt == 0 || (start + cnt <= lo && start >= kept)) {   // nothing of this slice is visible
        for (int i = threadIdx.x; i < nq * dv; i += TALK_THREADS) {
            const int h = i / dv, dim = i % dv;
            if (num_splits == 1) {
                out[((size_t)n * nq + h) * dv + dim] = from_f32<T>(attn_ext::finish<T>(0.f, -INFINITY, 0.f, ex, h, dim, dv, gate_row));
            } else {
                const size_t slot = ((size_t)n * nq + h) * num_splits + split;
                part_acc[slot * dv + dim] = 0.f;
                if (dim == 0) { part_ml[slot * 2] = -INFINITY; part_ml[slot * 2 + 1] = 0.f; }
            }
        }
        return;
    }
    const int* table = block_table + (size_t)token_seq[n] * max_blocks;
    for (int i = threadIdx.x; i < nq * dkp; i += TALK_THREADS) {
        const int h = i / dkp, c = i % dkp;
        qs[i] = c < dk ? to_f32(q[(size_t)n * q_stride + (size_t)h * dk + c]) * scale : 0.f;
    }
    if (talk)
        for (int i = threadIdx.x; i < nq * nq; i += TALK_THREADS) tm[i] = talk[i];
    for (int kl = threadIdx.x; kl < cnt; kl += TALK_THREADS) {
        const int key = start + kl;
        rows[kl] = table[key / page_size] * nkv * page_size + key % page_size;
    }
    __syncthreads();

    // 1. capped scores of every head
    constexpr int VN = Vec16<T>::N;
    if (v_chunk > 0 && vec_ok) {
        // The keys of v_chunk positions at a time (all key/value heads) are brought into shared memory by 16-byte loads that run along
        // the rows (a lane that walks its own row in the pages fetches 16 bytes of a 32-byte sector at a time, and the rows of a
        // block's warps together do not stay in the first-level cache). There a lane owns a key and a warp the heads w, w + 8, ...:
        // rows lie 16 bytes further apart than they are long, so that the lanes' pieces fall into different banks.
        T* k_s = reinterpret_cast<T*>(talk_smem + talk_floats(nq, dk, slice_keys));
        const int row_elems = nkv * dk + VN, per16 = dk / VN;
        for (int c0 = 0; c0 < cnt; c0 += v_chunk) {
            const int nk = min(v_chunk, cnt - c0);
            __syncthreads();
            for (int i = threadIdx.x; i < nk * nkv * per16; i += TALK_THREADS) {
                const int j = i / (nkv * per16), r = i % (nkv * per16);
                const int kvh = r / per16, c = (r % per16) * VN;
                *reinterpret_cast<uint4*>(k_s + (size_t)j * row_elems + kvh * dk + c) =
                    *reinterpret_cast<const uint4*>(k_pool + (size_t)(rows[c0 + j] + kvh * page_size) * dk + c);
            }
            __syncthreads();
            if (lane < nk) {
                for (int h = warp; h < nq; h += TALK_WARPS) {
                    const T* kr = k_s + (size_t)lane * row_elems + (h / G) * dk;
                    const float* qh = qs + (size_t)h * dkp;
                    float s0 = 0.f, s1 = 0.f;
#pragma unroll 4
                    for (int c = 0; c < dk; c += VN) {
                        float kf[VN];
                        Vec16<T>::load(kr + c, kf);
#pragma unroll
                        for (int i = 0; i < VN; i += 2) { s0 = fmaf(qh[c + i], kf[i], s0); s1 = fmaf(qh[c + i + 1], kf[i + 1], s1); }
                    }
                    const float sv = s0 + s1;
                    sc[(size_t)h * slice_keys + c0 + lane] = ex.softcap > 0.f ? ex.softcap * tanhf(sv / ex.softcap) : sv;
                }
            }
        }
        __syncthreads();
    } else {
    for (int base = warp * 32; base < cnt; base += TALK_WARPS * 32) {
        const int kl = base + lane;
        if (kl >= cnt) continue;
        const int row0 = rows[kl];
        for (int kvh = 0; kvh < nkv; ++kvh) {
            const T* kr = k_pool + (size_t)(row0 + kvh * page_size) * dk;
            for (int g0 = 0; g0 < G; g0 += TALK_GC) {
                const float* qh = qs + (size_t)(kvh * G + g0) * dkp;
                float s[TALK_GC];
#pragma unroll
                for (int g = 0; g < TALK_GC; ++g) s[g] = 0.f;
                if (vec_ok) {
#pragma unroll 4
                    for (int c = 0; c < dk; c += VN) {   // (unrolled: four pieces of the row are in flight)
                        float kf[VN];
                        Vec16<T>::load(kr + c, kf);
#pragma unroll
                        for (int g = 0; g < TALK_GC; ++g)
                            if (g0 + g < G) {
#pragma unroll
                                for (int i = 0; i < VN; ++i) s[g] = fmaf(qh[g * dkp + c + i], kf[i], s[g]);
                            }
                    }
                } else {
                    for (int c = 0; c < dk; ++c) {
                        const float kf = to_f32(kr[c]);
#pragma unroll
                        for (int g = 0; g < TALK_GC; ++g)
                            if (g0 + g < G) s[g] = fmaf(qh[g * dkp + c], kf, s[g]);
                    }
                }
#pragma unroll
                for (int g = 0; g < TALK_GC; ++g)
                    if (g0 + g < G) {
                        const float v = ex.softcap > 0.f ? ex.softcap * tanhf(s[g] / ex.softcap) : s[g];
                        sc[(size_t)(kvh * G + g0 + g) * slice_keys + kl] = v;
                    }
            }
        }
    }
    __syncthreads();
    }

    // 2. the heads' scores mixed; keys that the mask hides get -inf
    for (int kl = threadIdx.x; kl < cnt; kl += TALK_THREADS) {
        const int key = start + kl;
        const bool seen = key >= lo || key < kept;
        for (int h = 0; h < nq; ++h) {
            float v;
            if (talk) {
                v = 0.f;
                for (int g = 0; g < nq; ++g) v = fmaf(tm[h * nq + g], sc[(size_t)g * slice_keys + kl], v);
            } else {
                v = sc[(size_t)h * slice_keys + kl];
            }
            sm[(size_t)h * slice_keys + kl] = seen ? v : -INFINITY;
        }
    }
    __syncthreads();

    // 3. per head: maximum, weights, their sum
    for (int h = warp; h < nq; h += TALK_WARPS) {
        float* row = sm + (size_t)h * slice_keys;
        float M = -INFINITY;
        for (int kl = lane; kl < cnt; kl += 32) M = fmaxf(M, row[kl]);
        M = warp_max(M);
        float L = 0.f;
        for (int kl = lane; kl < cnt; kl += 32) {
            const float w = M > -INFINITY ? expf(row[kl] - M) : 0.f;
            row[kl] = w;
            L += w;
        }
        L = warp_sum(L);
        if (lane == 0) { ml[2 * h] = M; ml[2 * h + 1] = L; }
    }
    __syncthreads();

    // 4. weights times values, the keys in order
    const T* v_base = v_pool ? v_pool : k_pool;
    const int v_row = v_pool ? dv : dk;
    if (v_chunk > 0) {
        // The values of v_chunk keys at a time (all key/value heads) are brought into shared memory by 16-byte loads that run along the
        // rows, then every thread adds up its entries (head, dim) from there: read straight from the pages, an entry's loads came one
        // group of four after the other and a block waited on latency.
        T* v_s = reinterpret_cast<T*>(talk_smem + talk_floats(nq, dk, slice_keys));
        const int row_elems = nkv * dv, per16 = dv / VN;
        const int E = (nq * dv + TALK_THREADS - 1) / TALK_THREADS;
        float acc[TALK_MAX_E];
#pragma unroll
        for (int e = 0; e < TALK_MAX_E; ++e) acc[e] = 0.f;
        for (int c0 = 0; c0 < cnt; c0 += v_chunk) {
            const int nk = min(v_chunk, cnt - c0);
            __syncthreads();
            for (int i = threadIdx.x; i < nk * nkv * per16; i += TALK_THREADS) {
                const int j = i / (nkv * per16), r = i % (nkv * per16);
                const int kvh = r / per16, c = (r % per16) * VN;
                *reinterpret_cast<uint4*>(v_s + (size_t)(j * nkv + kvh) * dv + c) =
                    *reinterpret_cast<const uint4*>(v_base + (size_t)(rows[c0 + j] + kvh * page_size) * v_row + c);
            }
            __syncthreads();
#pragma unroll
            for (int e = 0; e < TALK_MAX_E; ++e) {
                const int i = threadIdx.x + e * TALK_THREADS;
                if (e < E && i < nq * dv) {
                    const int h = i / dv, dim = i % dv;
                    const float* w = sm + (size_t)h * slice_keys + c0;
                    const T* vs = v_s + (size_t)(h / G) * dv + dim;
                    float a = acc[e];
                    for (int j = 0; j < nk; ++j) {
                        const float wj = w[j];
                        a = fmaf(wj, wj != 0.f ? to_f32(vs[(size_t)j * row_elems]) : 0.f, a);
                    }
                    acc[e] = a;
                }
            }
        }
#pragma unroll
        for (int e = 0; e < TALK_MAX_E; ++e) {
            const int i = threadIdx.x + e * TALK_THREADS;
            if (e < E && i < nq * dv) {
                const int h = i / dv, dim = i % dv;
                const float M = ml[2 * h], L = ml[2 * h + 1];
                if (num_splits == 1) {
                    out[((size_t)n * nq + h) * dv + dim] = from_f32<T>(attn_ext::finish<T>(acc[e], M, L, ex, h, dim, dv, gate_row));
                } else {
                    const size_t slot = ((size_t)n * nq + h) * num_splits + split;
                    part_acc[slot * dv + dim] = acc[e];
                    if (dim == 0) { part_ml[slot * 2] = M; part_ml[slot * 2 + 1] = L; }
                }
            }
        }
        return;
    }
    for (int i = threadIdx.x; i < nq * dv; i += TALK_THREADS) {   // (sizes the staged form does not take: straight from the pages)
        const int h = i / dv, dim = i % dv;
        const int kvh = h / G;
        const float* w = sm + (size_t)h * slice_keys;
        const T* vb = v_base + (size_t)kvh * page_size * v_row + dim;
        float A = 0.f;
        int kl = 0;
        for (; kl + 4 <= cnt; kl += 4) {   // four loads in flight; the order of the additions stays
            float x[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) x[u] = w[kl + u] != 0.f ? to_f32(vb[(size_t)rows[kl + u] * v_row]) : 0.f;
#pragma unroll
            for (int u = 0; u < 4; ++u) A = fmaf(w[kl + u], x[u], A);
        }
        for (; kl < cnt; ++kl)
            if (w[kl] != 0.f) A = fmaf(w[kl], to_f32(vb[(size_t)rows[kl] * v_row]), A);
        const float M = ml[2 * h], L = ml[2 * h + 1];
        if (num_splits == 1) {
            out[((size_t)n * nq + h) * dv + dim] = from_f32<T>(attn_ext::finish<T>(A, M, L, ex, h, dim, dv, gate_row));
        } else {
            const size_t slot = ((size_t)n * nq + h) * num_splits + split;
            part_acc[slot * dv + dim] = A;
            if (dim == 0) { part_ml[slot * 2] = M; part_ml[slot * 2 + 1] = L; }
        }
    }
}

size_t talk_smem_bytes(int nq, int dk, int slice_keys) { return sizeof(float) * talk_floats(nq, dk, slice_keys); }

template <typename T>
int paged_attention_talk(const T* q, int q_stride, const T* k_pool, const T* v_pool, const int* block_table, int max_blocks, const int* token_seq,
                         const int* positions, const float* talk, T* out, float* scratch, int N, int nq, int nkv, int dk, int dv, int page_size,
                         float scale, int window, int num_splits, int slice_keys, const attn_ext::Extras& ex, cudaStream_t s) {
    if (N <= 0) return 0;
    if (nkv <= 0 || nq % nkv || dk <= 0 || dv <= 0 || page_size <= 0 || num_splits < 1 || num_splits > 65535 || slice_keys < 32 ||
        slice_keys > TALK_MAX_SLICE || slice_keys % 32 || (num_splits > 1 && !scratch) || (!v_pool && dv > dk) || (ex.gate_mode && !ex.gate) ||
        ex.rel || ex.temp_every)
        return LLMIE_ERR_BAD_ARGUMENT;
    size_t smem = talk_smem_bytes(nq, dk, slice_keys);
    if (smem > 200 * 1024) return LLMIE_ERR_BAD_ARGUMENT;
    constexpr int VN = Vec16<T>::N;
    const int vec_ok = dk % VN == 0 && ((uintptr_t)k_pool % 16 == 0);
    // the values go through shared memory where a chunk of at least 8 keys fits beside the scores, the rows are made of 16-byte pieces
    // and a thread's entries fit its registers (sizes alone decide: a token's arithmetic is the same in every step)
    int v_chunk = 0;
    size_t per_key = 0;
    const int v_row = v_pool ? dv : dk;
    if (dv % VN == 0 && v_row % VN == 0 && ((uintptr_t)(v_pool ? v_pool : k_pool) % 16 == 0) && (long long)nq * dv <= (long long)TALK_MAX_E * TALK_THREADS) {
        per_key = (size_t)nkv * dv * sizeof(T);
        if (vec_ok && (size_t)(nkv * dk + VN) * sizeof(T) > per_key) per_key = (size_t)(nkv * dk + VN) * sizeof(T);   // (the keys' padded rows use the same room)
        size_t fit = (160 * 1024 > smem ? 160 * 1024 - smem : 0) / per_key;
        if (fit > (size_t)TALK_V_CHUNK) fit = TALK_V_CHUNK;
        v_chunk = (int)(fit & ~(size_t)7);
    }
    smem += (size_t)v_chunk * per_key;
    if (smem > 48 * 1024) cudaFuncSetAttribute(paged_attn_talk_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    float* part_acc = scratch;
    float* part_ml = scratch ? scratch + (size_t)N * nq * num_splits * dv : nullptr;
    paged_attn_talk_kernel<T><<<dim3(N, num_splits), TALK_THREADS, smem, s>>>(q, q_stride, k_pool, v_pool, block_table, max_blocks, token_seq, positions,
                                                                               talk, out, part_acc, part_ml, nq, nkv, dk, dv, page_size, scale, window,
                                                                               num_splits, slice_keys, vec_ok, v_chunk, ex);
    int rc = launch_status();
    if (rc) return rc;
    if (num_splits > 1) {
        attn_ext::attn_ext_combine_kernel<T><<<N * nq, 128, 0, s>>>(part_acc, part_ml, out, nq, dv, num_splits, ex);
        rc = launch_status();
    }
    return rc;
}

}  // namespace

// The largest slice (a multiple of 32, at most TALK_MAX_SLICE) whose scores of all heads fit the shared memory; 0: not even 32 keys do.
LLMIE_API int llmie_attention_talk_slice(int nq, int dk) {
    for (int sl = TALK_MAX_SLICE; sl >= 32; sl -= 32)
        if (talk_smem_bytes(nq, dk, sl) <= 200 * 1024) return sl;
    return 0;
}

// q: nq heads of dk from the rows' start (row stride q_stride); talk [nq, nq] float or null; sink [nq] or null; gate: one number per head
// (gate_mode 1) or per output entry (2) in rows of gate_stride. Scratch for num_splits > 1, in floats: N * nq * num_splits * (dv + 2).
// num_splits slices of slice_keys keys each must cover the longest context of the step.
LLMIE_API int llmie_paged_attention_talk(const void* q, int q_stride, const void* k_pool, const void* v_pool, const int* block_table, int max_blocks,
                                         const int* token_seq, const int* positions, const float* talk, void* out, float* scratch, int N, int nq,
                                         int nkv, int dk, int dv, int page_size, float scale, int window, int num_splits, int slice_keys,
                                         const float* sink, const void* gate, int gate_stride, int gate_mode, int keep_first, int chunk, float softcap,
                                         int dtype, cudaStream_t s) {
    attn_ext::Extras ex;
    ex.temp_coef = 0.f; ex.temp_every = 0;
    ex.rel = nullptr; ex.rows_of = nullptr; ex.n_rows_of = 0; ex.rel_rows = 0;
    ex.sink = sink; ex.gate = gate; ex.gate_stride = gate_stride; ex.gate_mode = gate_mode;
    ex.keep_first = keep_first; ex.chunk = chunk; ex.softcap = softcap;
    if (dtype == DT_F32)
        return paged_attention_talk<float>((const float*)q, q_stride, (const float*)k_pool, (const float*)v_pool, block_table, max_blocks, token_seq, positions,
                                           talk, (float*)out, scratch, N, nq, nkv, dk, dv, page_size, scale, window, num_splits, slice_keys, ex, s);
    return paged_attention_talk<bf16>((const bf16*)q, q_stride, (const bf16*)k_pool, (const bf16*)v_pool, block_table, max_blocks, token_seq, positions, talk,
                                      (bf16*)out, scratch, N, nq, nkv, dk, dv, page_size, scale, window, num_splits, slice_keys, ex, s);
}
