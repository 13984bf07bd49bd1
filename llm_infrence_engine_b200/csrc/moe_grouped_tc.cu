// The grouped product of routed experts for MANY rows per expert (prompt portions), on the tcgen05 tensor cores of sm_100a.
//
// The (token, choice) pairs of a step lie sorted by expert ("places"); a device-side list cuts every expert's run of places into
// row tiles of up to 128 places: tiles[0] row tiles, then (expert, first place) of each; offsets[e + 1] ends expert e's run. A row
// tile multiplies by ITS expert's matrix, so the B operand's rows are taken at e * (rows of one expert's matrix) + the column
// tile. Rows of a tile past the end of its expert's run belong to the next expert (or to nobody): they are multiplied like the
// others, since a row of an MMA does not touch its neighbours, and not stored.
//
//   GATED   a [places, K] (the tokens' rows, gathered into the order of the places), w [E][2 F][K] (an expert's gate rows, then
//           its up rows): out[place, j] = silu(a . Wg[e][j]) * (a . Wu[e][j]) as bfloat16 [places, F]. The accumulator of a tile
//           is 128 lanes x 256 columns of tensor memory (gate sums, then up sums of the same outputs), one MMA of N = 256.
//   else    a [places, K], w [E][F][K]: out[place, j] = a . W[e][j] as float32 [places, F]. The tile is 256 outputs wide (two boxes
//           of 128 weight rows, one MMA of N = 256 as well): with 128 the kernel waited on the operands' way from L2.
//
// The kernel is persistent (one block per multiprocessor walks tiles blockIdx.x, + gridDim.x, ...; nobody on the host knows how
// many there are) and built like the gate/up kernel of the dense feed-forward: warp 0 one lane issues the TMA boxes of a K step
// of 64 into a ring of 4 stages, warp 1 one lane issues the MMAs and commits, warps 2-5 read the sums from tensor memory (thread
// = row) and store; two accumulators, so a tile's epilogue runs under the next tile's MMAs. Every wait is bounded.
#include "common.cuh"
#include "tcgen05.cuh"

namespace {

constexpr int BM = 128, BN = 128, BK = 64, STAGES = 4, UMMA_K = 16;
constexpr int A_BYTES = BM * BK * 2;
constexpr int EPI_THREADS = 128, THREADS = 64 + EPI_THREADS;

template <bool GATED>
__global__ void __launch_bounds__(THREADS) moe_grouped_tc_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_w,
                                                                  const int* __restrict__ offsets, const int* __restrict__ tile_list, void* __restrict__ out_,
                                                                  int F, int K, int* error_flag, float limit, float alpha, float shift) {
    constexpr int ACC_COLS = 2 * BN;                              // columns of tensor memory per accumulator
    constexpr int TILE_N = GATED ? BN : 2 * BN;                   // outputs per tile
    constexpr int B_BYTES = ACC_COLS * BK * 2, STAGE_BYTES = A_BYTES + B_BYTES;
    extern __shared__ unsigned char raw[];
    unsigned char* tiles = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(raw) + 1023) & ~(uintptr_t)1023);
    uint64_t* full = reinterpret_cast<uint64_t*>(tiles + STAGES * STAGE_BYTES);
    uint64_t* empty = full + STAGES;
    uint64_t* acc_full = empty + STAGES;   // [2] the MMAs of a tile have finished
    uint64_t* acc_free = acc_full + 2;     // [2] the epilogue has read the accumulator
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_free + 2);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    volatile int* issued = abort_flag + 1;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int n_tiles = (F + TILE_N - 1) / TILE_N, nkb = (K + BK - 1) / BK;
    const int w_rows = GATED ? 2 * F : F;   // rows of one expert's matrix

    if (tid == 0) {
        for (int s = 0; s < STAGES; ++s) { mbar_init(full + s, 1); mbar_init(empty + s, 1); }
        for (int s = 0; s < 2; ++s) { mbar_init(acc_full + s, 1); mbar_init(acc_free + s, EPI_THREADS / 32); }
        *abort_flag = 0;
        *issued = 0;
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_u32(tmem_slot)), "n"(512) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
    const uint32_t tmem = *tmem_slot;
    pdl_trigger();
    pdl_wait();   // the list of tiles, the rows and the places are what the kernels before this one wrote
    const int m_tiles = tile_list[0];
    const int num_tiles = m_tiles * n_tiles;

    if (warp == 0) {
        if (lane == 0) {
            asm volatile("prefetch.tensormap [%0];\n" ::"l"(&tmap_a) : "memory");
            asm volatile("prefetch.tensormap [%0];\n" ::"l"(&tmap_w) : "memory");
            int g = 0;
            bool ok = true;
            for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x) {
                const int mi = t % m_tiles, n0 = (t / m_tiles) * TILE_N;
                const int e = tile_list[1 + 2 * mi], p0 = tile_list[2 + 2 * mi];
                const int w0 = e * w_rows + n0;
                for (int kb = 0; kb < nkb; ++kb, ++g) {
                    const int s = g % STAGES;
                    if (g >= STAGES && !mbar_wait(empty + s, ((g / STAGES) & 1) ^ 1, abort_flag, error_flag, 51)) { ok = false; break; }
                    unsigned char* st = tiles + s * STAGE_BYTES;
                    mbar_expect_tx(full + s, STAGE_BYTES);
                    tma_load_2d(st, &tmap_a, kb * BK, p0, full + s);
                    tma_load_2d(st + A_BYTES, &tmap_w, kb * BK, w0, full + s);
                    // the second box: the up rows of the same outputs, or the next 128 outputs (rows past an expert's last are not stored)
                    tma_load_2d(st + A_BYTES + B_BYTES / 2, &tmap_w, kb * BK, w0 + (GATED ? F : BN), full + s);
                    *issued = g + 1;
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            // instruction descriptor: D float32, A and B bfloat16, both K-major, N = ACC_COLS, M = 128
            constexpr uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(ACC_COLS >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
            int g = 0, i = 0;
            bool ok = true;
            for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x, ++i) {
                const int buf = i & 1;
                if (i >= 2) ok = mbar_wait(acc_free + buf, ((i >> 1) & 1) ^ 1, abort_flag, error_flag, 52);
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
                const uint32_t d = tmem + (uint32_t)(buf * ACC_COLS);
                for (int kb = 0; kb < nkb; ++kb, ++g) {
                    const int s = g % STAGES;
                    ok = mbar_wait(full + s, (g / STAGES) & 1, abort_flag, error_flag, 53);
                    if (!ok) break;
                    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
                    const uint32_t a_addr = smem_u32(tiles + s * STAGE_BYTES);
                    const uint64_t a_desc = umma_desc(a_addr), b_desc = umma_desc(a_addr + A_BYTES);
#pragma unroll
                    for (int k = 0; k < BK / UMMA_K; ++k) umma_bf16(d, a_desc + 2 * k, b_desc + 2 * k, idesc, (kb > 0 || k > 0) ? 1u : 0u);
                    umma_commit(empty + s);
                }
                if (ok) umma_commit(acc_full + buf);
            }
        }
    } else {
        // ---------------------------------------------------------------- epilogue
        const int quarter = warp & 3;               // the 32 lanes of tensor memory this warp may read
        const int row = quarter * 32 + lane;
        int i = 0;
        bool ok = true;
        for (int t = blockIdx.x; t < num_tiles && ok; t += gridDim.x, ++i) {
            const int buf = i & 1;
            const int mi = t % m_tiles, n0 = (t / m_tiles) * TILE_N;
            const int e = tile_list[1 + 2 * mi], p0 = tile_list[2 + 2 * mi];
            const bool mine = p0 + row < offsets[e + 1];   // the place is one of this expert's
            ok = __all_sync(0xffffffffu, mbar_wait(acc_full + buf, (i >> 1) & 1, abort_flag, error_flag, 54));
            if (!ok) break;
            asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
            const uint32_t base = tmem + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(buf * ACC_COLS);
            if (GATED) {
                bf16* dst = reinterpret_cast<bf16*>(out_) + (size_t)(p0 + row) * F + n0;
#pragma unroll 2
                for (int c = 0; c < BN; c += 16) {
                    uint32_t gv[16], uv[16];
                    tmem_ld16(base + c, gv);
                    tmem_ld16(base + BN + c, uv);
                    asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
                    uint32_t packed[8];
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        float g0 = __uint_as_float(gv[2 * j]), g1 = __uint_as_float(gv[2 * j + 1]);
                        float u0 = __uint_as_float(uv[2 * j]), u1 = __uint_as_float(uv[2 * j + 1]);
                        float a0 = 1.0f;
                        if (limit > 0.f) {   // the clamped unit: min(g, limit) * sigmoid(alpha g) * (clamp(u) + shift)
                            g0 = fminf(g0, limit); g1 = fminf(g1, limit);
                            u0 = fminf(fmaxf(u0, -limit), limit) + shift;
                            u1 = fminf(fmaxf(u1, -limit), limit) + shift;
                            a0 = alpha;
                        }
                        const __nv_bfloat162 v = __floats2bfloat162_rn(__fdividef(g0, 1.0f + __expf(-a0 * g0)) * u0, __fdividef(g1, 1.0f + __expf(-a0 * g1)) * u1);
                        packed[j] = *reinterpret_cast<const uint32_t*>(&v);
                    }
                    if (mine) {
                        if (n0 + c + 8 <= F) *reinterpret_cast<uint4*>(dst + c) = make_uint4(packed[0], packed[1], packed[2], packed[3]);
                        if (n0 + c + 16 <= F) *reinterpret_cast<uint4*>(dst + c + 8) = make_uint4(packed[4], packed[5], packed[6], packed[7]);
                    }
                }
            } else {
                float* dst = reinterpret_cast<float*>(out_) + (size_t)(p0 + row) * F + n0;
#pragma unroll 2
                for (int c = 0; c < TILE_N; c += 16) {
                    uint32_t v[16];
                    tmem_ld16(base + c, v);
                    asm volatile("tcgen05.wait::ld.sync.aligned;\n" ::: "memory");
                    if (mine) {
#pragma unroll
                        for (int j = 0; j < 16; j += 4)
                            if (n0 + c + j + 4 <= F) *reinterpret_cast<uint4*>(dst + c + j) = make_uint4(v[j], v[j + 1], v[j + 2], v[j + 3]);
                    }
                }
            }
            asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
            __syncwarp();
            if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];\n" ::"r"(smem_u32(acc_free + buf)) : "memory");
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    __syncthreads();
    if (*abort_flag && tid == 0) {
        // gave up somewhere: let the copies that were started land before the block's shared memory goes away
        const int n_issued = *issued;
        for (int g = max(0, n_issued - STAGES); g < n_issued; ++g) {
            for (uint32_t i = 0; i < SPIN_LIMIT; ++i) {
                if (mbar_try_wait(full + g % STAGES, (g / STAGES) & 1)) break;
                __nanosleep(40);
            }
        }
    }
    __syncthreads();
    if (warp == 1) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem), "n"(512) : "memory");
}

template <bool GATED>
int launch_grouped(const bf16* a, int places, const bf16* w, int E, const int* offsets, const int* tile_list, int max_tiles, void* out, int F, int K,
                   int num_blocks, int* error_flag, float limit, float alpha, float shift, cudaStream_t s) {
    CUtensorMap ma, mw;
    int rc = tensor_map(a, places, K, BM, &ma);
    if (rc) return rc;
    rc = tensor_map(w, E * (GATED ? 2 : 1) * F, K, BN, &mw);
    if (rc) return rc;
    constexpr size_t smem = (size_t)STAGES * (A_BYTES + 2 * BN * BK * 2) + 1024 + 256;
    static bool set = false;
    if (!set) {
        cudaError_t e = cudaFuncSetAttribute(moe_grouped_tc_kernel<GATED>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        set = true;
    }
    const long long most = (long long)max_tiles * ((F + (GATED ? BN : 2 * BN) - 1) / (GATED ? BN : 2 * BN));
    const int grid = (int)(most < num_blocks ? most : num_blocks);
    return launch_kernel(moe_grouped_tc_kernel<GATED>, dim3(grid), dim3(THREADS), smem, s, ma, mw, offsets, tile_list, out, F, K, error_flag, limit, alpha, shift);
}

}  // namespace

// The most places of a row tile here: what the sort that makes the list is given.
LLMIE_API int llmie_moe_grouped_tc_rows() { return BM; }

// a [places, K] bfloat16 (rows in the order of the places), w [E][gated ? 2 F : F][K] bfloat16, offsets [E + 1] and tile_list
// [1 + 2 max_tiles] on the device as the sort leaves them (tiles of up to 128 places); out [places, F]: bfloat16 with `gated`,
// float32 without. K and F multiples of 8, bases 16-byte aligned. num_blocks: the persistent grid (the number of multiprocessors).
// limit > 0 (with `gated`): the unit is min(g, limit) * sigmoid(alpha g) * (clamp(u, -limit, limit) + shift) instead of silu(g) * u.
LLMIE_API int llmie_moe_grouped_tc(const bf16* a, int places, const bf16* w, int E, const int* offsets, const int* tile_list, int max_tiles, void* out,
                                    int F, int K, int gated, int num_blocks, int* error_flag, float limit, float alpha, float shift, cudaStream_t s) {
    if (places <= 0 || max_tiles <= 0) return 0;
    if (E <= 0 || F <= 0 || K <= 0 || K % 8 || F % 8 || ((uintptr_t)a & 15) || ((uintptr_t)w & 15) || ((uintptr_t)out & 15) || !error_flag ||
        num_blocks < 1 || (long long)E * 2 * F > 0x7fffffffLL)
        return LLMIE_ERR_BAD_ARGUMENT;
    if (gated) return launch_grouped<true>(a, places, w, E, offsets, tile_list, max_tiles, out, F, K, num_blocks, error_flag, limit, alpha, shift, s);
    return launch_grouped<false>(a, places, w, E, offsets, tile_list, max_tiles, out, F, K, num_blocks, error_flag, 0.f, 1.f, 0.f, s);
}
