// The routed feed-forward's products for steps of many rows, on the fifth-generation tensor cores: for every row tile
// of the plan, out[rows of the tile] = act(A[rows] . W[expert of the tile]^T), with tcgen05.mma, the accumulator in
// tensor memory and operands brought into 128-byte-swizzled shared memory by TMA - the warp roles, the stage ring, the
// two accumulators and the bounded waits of the engine's plain product (gemm_tcgen05.cu), with the tiles taken from a
// list that a kernel wrote instead of from M and N.
//
// Rows are (token, choice) pairs sorted by expert; every expert's run is padded to whole tiles of 128 rows, so a tile
// never holds rows of two experts and the padding rows (whatever they contain) are computed and never stored.
// A is [row capacity, K]; W is the experts' matrices stacked, [experts * N, K]; tile i of the plan is
// (expert, first row, rows in use); plan[0] is the number of tiles.  Columns beyond N run into the next expert's rows
// in shared memory and are masked at the store.  K % 8 == 0 (the 16-byte stride rule of TMA).
#include "tc_common.cuh"

namespace tc {

constexpr int BM = 128, BK = 64, BN = 256;
constexpr int A_BYTES = BM * BK * 2, B_BYTES = BN * BK * 2, STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int STAGES = 4, THREADS = 192;

struct Shared {
    uint64_t full[STAGES];
    uint64_t empty[STAGES];
    uint64_t accum_full[2];
    uint64_t accum_empty[2];
    uint32_t tmem_base;
    int failed;
};

// 32 consecutive accumulator columns of one row on their way to memory; ACT 1: relu(v)^2.  ACT 2: the columns are
// (gate, up) pairs and `out` points at the 16 results: g' sigmoid(1.702 g') (u' + 1), g' = min(g, limit), u' = clamp(u, +-limit);
// limit <= 0: silu(g) u.
template <int ACT>
__device__ __forceinline__ void store_chunk(const uint32_t* r, bf16* __restrict__ out, int n, int N, float limit) {
    if (ACT == 2) {
        float v[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            if (limit <= 0.f) {
                const float g = __uint_as_float(r[2 * i]);
                v[i] = g / (1.f + __expf(-g)) * __uint_as_float(r[2 * i + 1]);
                continue;
            }
            const float g = fminf(__uint_as_float(r[2 * i]), limit);
            const float u = fminf(fmaxf(__uint_as_float(r[2 * i + 1]), -limit), limit);
            v[i] = g / (1.f + __expf(-1.702f * g)) * (u + 1.f);
        }
        if (n + 32 <= N && (N & 15) == 0) {
            uint32_t packed[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                __nv_bfloat162 v2 = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
                packed[i] = *reinterpret_cast<uint32_t*>(&v2);
            }
            reinterpret_cast<uint4*>(out)[0] = make_uint4(packed[0], packed[1], packed[2], packed[3]);
            reinterpret_cast<uint4*>(out)[1] = make_uint4(packed[4], packed[5], packed[6], packed[7]);
        } else {
#pragma unroll
            for (int i = 0; i < 16; ++i)
                if (n + 2 * i + 1 < N) out[i] = __float2bfloat16_rn(v[i]);
        }
        return;
    }
    float v[32];
#pragma unroll
    for (int i = 0; i < 32; ++i) {
        v[i] = __uint_as_float(r[i]);
        if (ACT == 1) {
            v[i] = fmaxf(v[i], 0.f);
            v[i] *= v[i];
        }
    }
    if (n + 32 <= N && (N & 7) == 0) {
        uint32_t packed[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            __nv_bfloat162 v2 = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
            packed[i] = *reinterpret_cast<uint32_t*>(&v2);
        }
#pragma unroll
        for (int i = 0; i < 4; ++i)
            reinterpret_cast<uint4*>(out)[i] = make_uint4(packed[4 * i], packed[4 * i + 1], packed[4 * i + 2], packed[4 * i + 3]);
    } else {
#pragma unroll
        for (int i = 0; i < 32; ++i)
            if (n + i < N) out[i] = __float2bfloat16_rn(v[i]);
    }
}

template <int ACT>
__global__ void __launch_bounds__(THREADS, 1)
grouped_tcgen05_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_w, bf16* __restrict__ out,
                       const int* __restrict__ plan, const int* __restrict__ tile_list, int N, int K, float limit,
                       int* __restrict__ err) {
    extern __shared__ unsigned char smem_raw[];
    unsigned char* tiles = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    __shared__ Shared sh;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n_blocks = (N + BN - 1) / BN;
    const int num_tiles = plan[0] * n_blocks;            // written by the plan kernel, which ended before this one began
    const int kblocks = (K + BK - 1) / BK;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) { mbar_init(&sh.full[s], 1); mbar_init(&sh.empty[s], 1); }
        for (int b = 0; b < 2; ++b) { mbar_init(&sh.accum_full[b], 1); mbar_init(&sh.accum_empty[b], 4); }
        sh.failed = 0;
        asm volatile("fence.mbarrier_init.release.cluster;\n" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;\n" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;\n" ::"r"(smem_u32(&sh.tmem_base)), "r"(2 * BN) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;\n" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
    const uint32_t tmem = sh.tmem_base;

    // Tile t: row tile t / n_blocks of the plan, column block t % n_blocks (the column blocks of a row tile run side by side).
    if (warp == 0) {
        if (lane == 0) {
            asm volatile("prefetch.tensormap [%0];\n" ::"l"(&map_a) : "memory");
            asm volatile("prefetch.tensormap [%0];\n" ::"l"(&map_w) : "memory");
            uint32_t it = 0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
                const int* t = tile_list + 3 * (tile / n_blocks);
                const int row0 = t[1], w_row = t[0] * N + (tile % n_blocks) * BN;
                for (int kb = 0; kb < kblocks; ++kb, ++it) {
                    const int s = it % STAGES;
                    const uint32_t round = it / STAGES;
                    if (round > 0 && !mbar_wait(&sh.empty[s], (round - 1) & 1)) { atomicOr(err, KVB_DEV_TIMEOUT); sh.failed = 1; ok = false; break; }
                    mbar_expect_tx(&sh.full[s], STAGE_BYTES);
                    tma_load_2d(tiles + s * STAGE_BYTES, &map_a, kb * BK, row0, &sh.full[s]);
                    tma_load_2d(tiles + s * STAGE_BYTES + A_BYTES, &map_w, kb * BK, w_row, &sh.full[s]);
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            constexpr uint32_t idesc = instr_desc(BM, BN);
            uint32_t it = 0, local = 0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++local) {
                const int b = local & 1;
                const uint32_t use = local >> 1;
                if (use > 0 && !mbar_wait(&sh.accum_empty[b], (use - 1) & 1)) { atomicOr(err, KVB_DEV_TIMEOUT); sh.failed = 1; ok = false; break; }
                asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
                const uint32_t acc = tmem + b * BN;
                for (int kb = 0; kb < kblocks; ++kb, ++it) {
                    const int s = it % STAGES;
                    if (!mbar_wait(&sh.full[s], (it / STAGES) & 1)) { atomicOr(err, KVB_DEV_TIMEOUT); sh.failed = 1; ok = false; break; }
                    asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
                    const uint32_t a_addr = smem_u32(tiles + s * STAGE_BYTES), b_addr = a_addr + A_BYTES;
                    const uint64_t adesc = smem_desc(a_addr), bdesc = smem_desc(b_addr);
#pragma unroll
                    for (int k = 0; k < BK / 16; ++k)
                        umma(acc, adesc + 2 * k, bdesc + 2 * k, idesc, (kb | k) != 0 ? 1u : 0u);
                    umma_commit(&sh.empty[s]);
                }
                umma_commit(&sh.accum_full[b]);
            }
        }
    } else {
        const int quarter = warp & 3;
        uint32_t local = 0;
        bool ok = true;
        for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x, ++local) {
            const int* t = tile_list + 3 * (tile / n_blocks);
            const int row0 = t[1], rows = t[2], n0 = (tile % n_blocks) * BN;
            const int b = local & 1;
            const int m = quarter * 32 + lane;
            ok = mbar_wait(&sh.accum_full[b], (local >> 1) & 1);
            if (!ok) { if (lane == 0) { atomicOr(err, KVB_DEV_TIMEOUT); sh.failed = 1; } break; }
            asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
#pragma unroll 1
            for (int c = 0; c < BN / 32; ++c) {
                uint32_t r[32];
                tmem_ld32(tmem + ((uint32_t)(quarter * 32) << 16) + b * BN + c * 32, r);
                const int n = n0 + c * 32;
                if (m >= rows || n >= N) continue;
                if (ACT == 2) store_chunk<ACT>(r, out + (size_t)(row0 + m) * (N >> 1) + (n >> 1), n, N, limit);
                else store_chunk<ACT>(r, out + (size_t)(row0 + m) * N + n, n, N, limit);
            }
            asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(&sh.accum_empty[b]);
        }
    }

    asm volatile("tcgen05.fence::before_thread_sync;\n" ::: "memory");
    __syncthreads();
    if (sh.failed && threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) mbar_wait(&sh.full[s], 0);
    }
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;\n" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;\n" ::"r"(tmem), "r"(2 * BN) : "memory");
    }
}

// xs[place[p], :] = x[p / top, :] for every (row, choice) pair p: the step's rows in the order of the plan.
__global__ void gather_rows_kernel(const bf16* __restrict__ x, const int* __restrict__ place, bf16* __restrict__ xs, int top, int K) {
    const int p = blockIdx.x;
    const uint4* src = reinterpret_cast<const uint4*>(x + (size_t)(p / top) * K);
    uint4* dst = reinterpret_cast<uint4*>(xs + (size_t)place[p] * K);
    for (int i = threadIdx.x; i < K / 8; i += blockDim.x) dst[i] = src[i];
}

static int sm_count() {
    static int count = 0;
    if (!count) {
        int dev = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&count, cudaDevAttrMultiProcessorCount, dev);
    }
    return count;
}

}  // namespace tc

KVB_API int kvb_gather_rows(const void* x, const int* place, void* xs, int pairs, int top, int K, cudaStream_t stream) {
    if (pairs <= 0) return KVB_OK;
    if (K % 8 != 0 || top < 1) return KVB_ERR_SHAPE;
    tc::gather_rows_kernel<<<pairs, 128, 0, stream>>>((const bf16*)x, place, (bf16*)xs, top, K);
    return kvb_launch_status();
}

// a [row_capacity, K] in the plan's order (runs padded to 128 rows), w [experts * N, K], out [row_capacity, N] (act 2:
// [row_capacity, N / 2]); `max_tiles` bounds the plan's row tiles.
static int grouped_tcgen05(const void* a, const void* w, void* out, const int* plan, const int* tile_list, int max_tiles,
                           int row_capacity, int experts, int N, int K, int act, float limit, int* err, cudaStream_t stream) {
    using namespace tc;
    if (max_tiles <= 0) return KVB_OK;
    if (K % 8 != 0 || N < 1 || act < 0 || act > 2 || (act == 2 && N % 2 != 0)) return KVB_ERR_SHAPE;
    if (((uintptr_t)a | (uintptr_t)w | (uintptr_t)out) % 16 != 0) return KVB_ERR_ALIGN;
    CUtensorMap ma, mw;
    int rc = make_bf16_map(&ma, a, row_capacity, K, K, BM);
    if (rc != KVB_OK) return rc;
    rc = make_bf16_map(&mw, w, (long long)experts * N, K, K, BN);
    if (rc != KVB_OK) return rc;
    const size_t smem = (size_t)STAGES * STAGE_BYTES + 1024;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(grouped_tcgen05_kernel<0>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e == cudaSuccess) e = cudaFuncSetAttribute(grouped_tcgen05_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e == cudaSuccess) e = cudaFuncSetAttribute(grouped_tcgen05_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    const long long tiles = (long long)max_tiles * ((N + BN - 1) / BN);
    const int blocks = tiles < sm_count() ? (int)tiles : sm_count();
    if (act == 2)
        grouped_tcgen05_kernel<2><<<blocks, THREADS, smem, stream>>>(ma, mw, (bf16*)out, plan, tile_list, N, K, limit, err);
    else if (act == 1)
        grouped_tcgen05_kernel<1><<<blocks, THREADS, smem, stream>>>(ma, mw, (bf16*)out, plan, tile_list, N, K, limit, err);
    else
        grouped_tcgen05_kernel<0><<<blocks, THREADS, smem, stream>>>(ma, mw, (bf16*)out, plan, tile_list, N, K, limit, err);
    return kvb_launch_status();
}

KVB_API int kvb_grouped_gemm_tcgen05(const void* a, const void* w, void* out, const int* plan, const int* tile_list, int max_tiles,
                                     int row_capacity, int experts, int N, int K, int act, int* err, cudaStream_t stream) {
    if (act > 1) return KVB_ERR_SHAPE;
    return grouped_tcgen05(a, w, out, plan, tile_list, max_tiles, row_capacity, experts, N, K, act, 0.f, err, stream);
}

// The same with the activation's constant: act 2 is the clamped gated activation of (gate, up) column pairs with `limit`.
KVB_API int kvb_grouped_gemm_tcgen05_act(const void* a, const void* w, void* out, const int* plan, const int* tile_list,
                                         int max_tiles, int row_capacity, int experts, int N, int K, int act, float limit, int* err,
                                         cudaStream_t stream) {
    return grouped_tcgen05(a, w, out, plan, tile_list, max_tiles, row_capacity, experts, N, K, act, limit, err, stream);
}
