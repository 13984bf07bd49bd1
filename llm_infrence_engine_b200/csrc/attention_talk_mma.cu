// Attention whose heads talk, for steps with prompt portions in bfloat16: the tensor-core form. A tile is up to TT = 16 / Gs tokens
// of one request (Gs = query heads per key/value head) and ALL heads: warp w owns key/value head w, and its 16 rows are (token, head
// of its group), so no row of an m16 tile is wasted and a chunk of keys is fetched once for the tile's tokens. Per chunk of 32 keys:
//
//   1. keys and values of all key/value heads come into shared memory (cp.async along the rows, through the block table);
//   2. every warp makes the plain scores of its rows (mma.sync m16n8k16, queries and keys by ldmatrix), scales and caps them in
//      32-bit and leaves them in shared memory, laid out [token][key][head] (padded against bank conflicts);
//   3. every thread mixes the scores at its positions of the accumulator tile: score'_h = sum_g talk[h][g] score_g, 32-bit, on the
//      CUDA cores (the mix is H multiply-adds per score whatever the form), masks them and takes them into its rows' running maximum
//      and sum;
//   4. the weights, rounded to bfloat16, are the A operand of the products with the warp's values (ldmatrix.trans), accumulated in
//      registers over all chunks.
//
// Cap and exponentials take the fast forms here (this kernel serves bfloat16 only, where the weights are rounded to 8 bits anyway; the
// 32-bit path never comes this way). A tile walks all keys up to its last token's position itself (no slices, no merge); sink and gate per head close a row. Only the
// causal mask; sizes the form does not take (see llmie_attention_talk_mma_fits) go to the CUDA-core kernel.
#include "attention_ext.cuh"

namespace {

constexpr int TM_KEYS = 32;

__device__ __forceinline__ void ldsm_x4(uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3, const void* p) {
    const uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(a));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3, const void* p) {
    const uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n" : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(a));
}
__device__ __forceinline__ void mma_bf16(float* c, uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void cp_async16_z(void* dst, const void* src, int src_bytes) {   // src_bytes 0: zeros
    const uint32_t d = (uint32_t)__cvta_generic_to_shared(dst);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(d), "l"(src), "r"(src_bytes));
}
__device__ __forceinline__ void cp_commit_() { asm volatile("cp.async.commit_group;\n" ::); }
__device__ __forceinline__ void cp_wait_all() { asm volatile("cp.async.wait_group 0;\n" ::); }
__device__ __forceinline__ void cp_wait_one() { asm volatile("cp.async.wait_group 1;\n" ::); }   // all but the newest group have landed
__device__ __forceinline__ uint32_t pack2(float a, float b) {
    const __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<const uint32_t*>(&v);
}

struct TalkParams {
    const bf16* q; int q_stride;
    const bf16* k_pool; const bf16* v_pool;
    const int* block_table; int max_blocks;
    const int* token_seq; const int* positions; const int* tile_info;
    const float* talk;
    bf16* out;
    int nq, nkv, dk, page_size;
    float scale;
    attn_ext::Extras ex;
};

// NV: pairs of n8 tiles over the value entries (dv = 16 NV)
template <int NV>
__global__ void __launch_bounds__(256) attn_talk_mma_kernel(const TalkParams P) {
    extern __shared__ __align__(16) unsigned char tm_smem[];
    constexpr int dv = 16 * NV, vs = dv + 8;
    const int nq = P.nq, nkv = P.nkv, dk = P.dk, ks = dk + 8;
    const int Gs = nq / nkv, TT = 16 / Gs;
    const int nqp = (nq + 3) & ~3;
    bf16* Qs = reinterpret_cast<bf16*>(tm_smem);                       // [nkv][16][ks]: row (token, head of the group) of key/value head kvh
    bf16* Ks = Qs + (size_t)nkv * 16 * ks;                             // [nkv][TM_KEYS][ks]
    bf16* Vs = Ks + (size_t)nkv * TM_KEYS * ks;                        // [nkv][TM_KEYS][vs]
    // [TT][TM_KEYS][nqp + 4] (+ 4 more per token): scaled and capped scores. A (token, key)'s heads lie 16 bytes further apart than they
    // are long and a token's block 16 bytes further still, so that the 16-byte reads of a warp's positions (a quad's keys lie two apart,
    // its rows one or more tokens apart) fall into different banks
    float* sS = reinterpret_cast<float*>(Vs + (size_t)nkv * TM_KEYS * vs);
    const int srow = nqp + 4, stok = TM_KEYS * srow + 4;
    float* tmx = sS + (size_t)TT * stok;                               // [nq][nqp]: the mixing matrix
    int* rows_s = reinterpret_cast<int*>(tmx + (size_t)nq * nqp);      // [TM_KEYS]: where the chunk's keys lie in the pools

    const int tid = threadIdx.x, lane = tid & 31, w = tid >> 5;       // w: the warp's key/value head
    const int threads = nkv * 32;
    const int n0 = P.tile_info[2 * blockIdx.x], nt = P.tile_info[2 * blockIdx.x + 1];   // nt <= TT tokens from row n0
    const int* table = P.block_table + (size_t)P.token_seq[n0] * P.max_blocks;
    const int p_last = P.positions[n0 + nt - 1];

    for (int i = tid; i < nkv * 16 * (dk / 8); i += threads) {
        const int row = i / (dk / 8), c = (i % (dk / 8)) * 8;
        const int kvh = row / 16, r = row % 16, t = r / Gs, g = r % Gs;
        uint4 v = make_uint4(0, 0, 0, 0);
        if (t < nt) v = *reinterpret_cast<const uint4*>(P.q + (size_t)(n0 + t) * P.q_stride + (size_t)(kvh * Gs + g) * dk + c);
        *reinterpret_cast<uint4*>(Qs + (size_t)row * ks + c) = v;
    }
    for (int i = tid; i < nq * nqp; i += threads) {
        const int h = i / nqp, g = i % nqp;
        tmx[i] = g < nq ? (P.talk ? P.talk[h * nq + g] : (h == g ? 1.f : 0.f)) : 0.f;
    }
    for (int i = tid; i < TT * stok; i += threads) sS[i] = 0.f;   // (the columns that pad a row of heads to 16 bytes stay zero)

    // this thread's two rows of the warp's tile: (token, head)
    const int r0 = lane >> 2, r1 = r0 + 8, qd = lane & 3;
    const int t0 = r0 / Gs, t1 = r1 / Gs;
    const int h0 = w * Gs + r0 % Gs, h1 = w * Gs + r1 % Gs;
    const int pos0 = t0 < nt ? P.positions[n0 + t0] : -1, pos1 = t1 < nt ? P.positions[n0 + t1] : -1;
    float O[2 * NV][4];
#pragma unroll
    for (int j = 0; j < 2 * NV; ++j) { O[j][0] = O[j][1] = O[j][2] = O[j][3] = 0.f; }
    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;
    const int mi = lane >> 3, lr = lane & 7;
    const float inv_cap = P.ex.softcap > 0.f ? 1.0f / P.ex.softcap : 0.f;

    // A chunk's keys and its values are two groups of asynchronous copies: the keys of the NEXT chunk are asked for as soon as this
    // chunk's scores are made (they arrive under the mix and the value products), its values as soon as this chunk's are used up (they
    // arrive under the next chunk's scores).
    // (Nothing in these loops divides: a group of lanes, a power of two wide, walks the 16-byte pieces of one row; the rows are numbered
    // key/value head first; and a key's place in the pools is looked up once per chunk, by the first warp, into rows_s.)
    int pk_k = 1, pk_v = 1, sh_k = 0, sh_v = 0;
    while (pk_k < dk / 8) { pk_k <<= 1; ++sh_k; }
    while (pk_v < dv / 8) { pk_v <<= 1; ++sh_v; }
    auto place_rows = [&](int c0) {   // rows_s[key]: the row of key/value head 0 in the pools, or -1 past the tile's last key
        if (tid < TM_KEYS) {
            const int ka = c0 + tid;
            rows_s[tid] = ka <= p_last ? table[ka / P.page_size] * nkv * P.page_size + ka % P.page_size : -1;
        }
    };
    auto fetch_keys = [&](int c0) {
        if (c0 <= p_last)
            for (int rk = tid >> sh_k; rk < TM_KEYS * nkv; rk += threads >> sh_k) {
                const int c = (tid & (pk_k - 1)) * 8, kvh = rk >> 5, key = rk & (TM_KEYS - 1);
                if (c < dk) {
                    const int row = rows_s[key];
                    cp_async16_z(Ks + ((size_t)kvh * TM_KEYS + key) * ks + c, P.k_pool + (size_t)(row < 0 ? 0 : row + kvh * P.page_size) * dk + c,
                                 row < 0 ? 0 : 16);
                }
            }
        cp_commit_();
    };
    auto fetch_values = [&](int c0) {
        if (c0 <= p_last)
            for (int rk = tid >> sh_v; rk < TM_KEYS * nkv; rk += threads >> sh_v) {
                const int c = (tid & (pk_v - 1)) * 8, kvh = rk >> 5, key = rk & (TM_KEYS - 1);
                if (c < dv) {
                    const int row = rows_s[key];
                    cp_async16_z(Vs + ((size_t)kvh * TM_KEYS + key) * vs + c, P.v_pool + (size_t)(row < 0 ? 0 : row + kvh * P.page_size) * dv + c,
                                 row < 0 ? 0 : 16);
                }
            }
        cp_commit_();
    };
    place_rows(0);
    __syncthreads();
    fetch_keys(0);
    fetch_values(0);
    for (int c0 = 0; c0 <= p_last; c0 += TM_KEYS) {
        cp_wait_one();     // this chunk's keys have landed (its values may still be on their way)
        __syncthreads();   // ... for everyone (and, the first time, the queries and the matrix are in place)

        // 2. plain scores of the warp's rows against its key/value head's keys
        float S[4][4];
#pragma unroll
        for (int j = 0; j < 4; ++j) { S[j][0] = S[j][1] = S[j][2] = S[j][3] = 0.f; }
        const bf16* qrow = Qs + ((size_t)w * 16 + (lane & 15)) * ks + (lane >> 4) * 8;
        const bf16* krow = Ks + ((size_t)w * TM_KEYS + (mi >> 1) * 8 + lr) * ks + (mi & 1) * 8;
        for (int kk = 0; kk < dk; kk += 16) {
            uint32_t a0, a1, a2, a3, b0, b1, b2, b3;
            ldsm_x4(a0, a1, a2, a3, qrow + kk);
            ldsm_x4(b0, b1, b2, b3, krow + kk);
            mma_bf16(S[0], a0, a1, a2, a3, b0, b1);
            mma_bf16(S[1], a0, a1, a2, a3, b2, b3);
            ldsm_x4(b0, b1, b2, b3, krow + (size_t)16 * ks + kk);
            mma_bf16(S[2], a0, a1, a2, a3, b0, b1);
            mma_bf16(S[3], a0, a1, a2, a3, b2, b3);
        }
#pragma unroll
        for (int j = 0; j < 4; ++j)
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int t = i < 2 ? t0 : t1, h = i < 2 ? h0 : h1, key = j * 8 + 2 * qd + (i & 1);
                float v = S[j][i] * P.scale;
                if (P.ex.softcap > 0.f) v = P.ex.softcap * (1.0f - __fdividef(2.0f, __expf(2.0f * v * inv_cap) + 1.0f));   // cap * tanh(v / cap), fast forms
                if (t < TT) sS[(size_t)t * stok + key * srow + h] = v;
            }
        cp_wait_all();     // this chunk's values have landed
        place_rows(c0 + TM_KEYS);   // (this chunk's copies were all asked for before the loop came round)
        __syncthreads();   // the scores lie in shared memory, the values too, and the keys are used up
        fetch_keys(c0 + TM_KEYS);

        // 3. the mix at this thread's positions, the mask, the rows' running maximum and sum
        float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
        for (int j = 0; j < 4; ++j)
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int t = i < 2 ? t0 : t1, h = i < 2 ? h0 : h1, key = j * 8 + 2 * qd + (i & 1);
                const int pos = i < 2 ? pos0 : pos1;
                float v = -INFINITY;
                if (c0 + key <= pos) {
                    const float* src = sS + (size_t)t * stok + key * srow;
                    const float* mr = tmx + (size_t)h * nqp;
                    float a = 0.f;
                    for (int g = 0; g < nqp; g += 4) {
                        const float4 sv = *reinterpret_cast<const float4*>(src + g), mv = *reinterpret_cast<const float4*>(mr + g);
                        a = fmaf(mv.x, sv.x, a); a = fmaf(mv.y, sv.y, a); a = fmaf(mv.z, sv.z, a); a = fmaf(mv.w, sv.w, a);
                    }
                    v = a;
                }
                S[j][i] = v;
                if (i < 2) mx0 = fmaxf(mx0, v); else mx1 = fmaxf(mx1, v);
            }
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1)); mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1)); mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
        const float n0m = fmaxf(m0, mx0), n1m = fmaxf(m1, mx1);
        const float cr0 = m0 > -INFINITY ? __expf(m0 - n0m) : 1.f, cr1 = m1 > -INFINITY ? __expf(m1 - n1m) : 1.f;
        m0 = n0m; m1 = n1m;
        float s0 = 0.f, s1 = 0.f;
        uint32_t pa[4][2];   // per n8 tile: the weights of row r0 and of row r1, two keys each, as bfloat16
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            float p[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float mm = i < 2 ? m0 : m1;
                p[i] = S[j][i] > -INFINITY ? __expf(S[j][i] - mm) : 0.f;   // (the fast form: the weight is rounded to 8 bits next)
                p[i] = __bfloat162float(__float2bfloat16_rn(p[i]));   // (the sum runs over the weights as the values meet them)
            }
            s0 += p[0] + p[1]; s1 += p[2] + p[3];
            pa[j][0] = pack2(p[0], p[1]); pa[j][1] = pack2(p[2], p[3]);
        }
        s0 += __shfl_xor_sync(0xffffffffu, s0, 1); s0 += __shfl_xor_sync(0xffffffffu, s0, 2);
        s1 += __shfl_xor_sync(0xffffffffu, s1, 1); s1 += __shfl_xor_sync(0xffffffffu, s1, 2);
        l0 = l0 * cr0 + s0; l1 = l1 * cr1 + s1;
#pragma unroll
        for (int j = 0; j < 2 * NV; ++j) { O[j][0] *= cr0; O[j][1] *= cr0; O[j][2] *= cr1; O[j][3] *= cr1; }

        // 4. weights times the warp's values
        const bf16* vrow = Vs + ((size_t)w * TM_KEYS + (mi & 1) * 8 + lr) * vs + (mi >> 1) * 8;
#pragma unroll
        for (int j = 0; j < 2; ++j) {   // 16 keys at a time
            const uint32_t a0 = pa[2 * j][0], a1 = pa[2 * j][1], a2 = pa[2 * j + 1][0], a3 = pa[2 * j + 1][1];
#pragma unroll
            for (int nv = 0; nv < NV; ++nv) {
                uint32_t b0, b1, b2, b3;
                ldsm_x4_t(b0, b1, b2, b3, vrow + (size_t)j * 16 * vs + nv * 16);
                mma_bf16(O[2 * nv], a0, a1, a2, a3, b0, b1);
                mma_bf16(O[2 * nv + 1], a0, a1, a2, a3, b2, b3);
            }
        }
        __syncthreads();   // the values are used up (and so are the scores in shared memory)
        fetch_values(c0 + TM_KEYS);
    }
    cp_wait_all();

    // sink, division and gate per row, then the rows out
#pragma unroll
    for (int half = 0; half < 2; ++half) {
        const int t = half ? t1 : t0, h = half ? h1 : h0;
        if (t >= nt) continue;
        const int n = n0 + t;
        const bf16* gate_row = P.ex.gate_mode ? reinterpret_cast<const bf16*>(P.ex.gate) + (size_t)n * P.ex.gate_stride : nullptr;
        const float f = attn_ext::finish_scale<bf16>(half ? m1 : m0, half ? l1 : l0, P.ex, h, gate_row);
        bf16* o = P.out + ((size_t)n * nq + h) * dv + 2 * qd;
#pragma unroll
        for (int j = 0; j < 2 * NV; ++j)
            *reinterpret_cast<uint32_t*>(o + j * 8) = pack2(O[j][2 * half] * f, O[j][2 * half + 1] * f);
    }
}

size_t talk_mma_smem(int nq, int nkv, int dk, int dv) {
    const int Gs = nq / nkv, TT = 16 / Gs, nqp = (nq + 3) & ~3;
    return sizeof(bf16) * ((size_t)nkv * 16 * (dk + 8) + (size_t)nkv * TM_KEYS * (dk + 8) + (size_t)nkv * TM_KEYS * (dv + 8)) +
           sizeof(float) * ((size_t)TT * (TM_KEYS * (nqp + 4) + 4) + (size_t)nq * nqp) + sizeof(int) * TM_KEYS;
}

template <int NV>
int launch_talk_mma(const TalkParams& P, int tiles, size_t smem, cudaStream_t s) {
    if (smem > 48 * 1024) cudaFuncSetAttribute(attn_talk_mma_kernel<NV>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    attn_talk_mma_kernel<NV><<<tiles, P.nkv * 32, smem, s>>>(P);
    return launch_status();
}

}  // namespace

// Tokens per tile (16 / heads per key/value head) if the tensor-core form takes these sizes, else 0: heads per key/value head a power
// of two up to 16, at most 8 key/value heads (one warp each), keys a multiple of 16 up to 256 entries, values of 32, 64 or 128.
LLMIE_API int llmie_attention_talk_mma_fits(int nq, int nkv, int dk, int dv) {
    if (nkv < 1 || nkv > 8 || nq % nkv) return 0;
    const int Gs = nq / nkv;
    if (Gs > 16 || (Gs & (Gs - 1))) return 0;
    if (dk % 16 || dk > 256 || (dv != 32 && dv != 64 && dv != 128)) return 0;
    if (talk_mma_smem(nq, nkv, dk, dv) > 200 * 1024) return 0;
    return 16 / Gs;
}

// tile_info [tiles, 2]: (first row, rows) of tiles of up to llmie_attention_talk_mma_fits(...) consecutive rows of one request. q: nq heads
// of dk from the rows' start (16-byte aligned, row stride a multiple of 8); gate: one number per head in rows of gate_stride, or null.
LLMIE_API int llmie_paged_attention_talk_mma(const bf16* q, int q_stride, const bf16* k_pool, const bf16* v_pool, const int* block_table, int max_blocks,
                                             const int* token_seq, const int* positions, const int* tile_info, int tiles, const float* talk, bf16* out,
                                             int nq, int nkv, int dk, int dv, int page_size, float scale, const float* sink, const bf16* gate,
                                             int gate_stride, float softcap, cudaStream_t s) {
    if (tiles <= 0) return 0;
    if (!llmie_attention_talk_mma_fits(nq, nkv, dk, dv) || !v_pool || ((uintptr_t)q & 15) || q_stride % 8 || ((uintptr_t)k_pool & 15) ||
        ((uintptr_t)v_pool & 15) || page_size <= 0)
        return LLMIE_ERR_BAD_ARGUMENT;
    TalkParams P;
    P.q = q; P.q_stride = q_stride; P.k_pool = k_pool; P.v_pool = v_pool; P.block_table = block_table; P.max_blocks = max_blocks;
    P.token_seq = token_seq; P.positions = positions; P.tile_info = tile_info; P.talk = talk; P.out = out;
    P.nq = nq; P.nkv = nkv; P.dk = dk; P.page_size = page_size; P.scale = scale;
    P.ex.temp_coef = 0.f; P.ex.temp_every = 0; P.ex.rel = nullptr; P.ex.rows_of = nullptr; P.ex.n_rows_of = 0; P.ex.rel_rows = 0;
    P.ex.sink = sink; P.ex.gate = gate; P.ex.gate_stride = gate_stride; P.ex.gate_mode = gate ? 1 : 0;
    P.ex.keep_first = 0; P.ex.chunk = 0; P.ex.softcap = softcap;
    const size_t smem = talk_mma_smem(nq, nkv, dk, dv);
    if (dv == 32) return launch_talk_mma<2>(P, tiles, smem, s);
    if (dv == 64) return launch_talk_mma<4>(P, tiles, smem, s);
    return launch_talk_mma<8>(P, tiles, smem, s);
}
