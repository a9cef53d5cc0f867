// A routed feed-forward (mixture of experts) on the device, with launches that do not depend on the routing.
//
//   route_top      per row: the `top` experts with the largest float32 logits, weights = softmax over those logits only,
//                  or the softmax over all experts' logits at the chosen ones, as they are
//   routed_plan    (row, choice) pairs sorted by expert: where each pair sits, and the list of row tiles per expert
//   grouped_gemm   for every tile: out[pair] = act(A[pair] . W[expert]^T); A gathered from the step's rows (the way up) or
//                  read in sorted order (the way down); float32 accumulation on the CUDA cores
//   routed_combine out[t] = base[t] + sum_s weight[t, s] * y[place of pair (t, s)], float32, in the order of s
//
// The grid of a grouped product is sized for the worst case, ceil(pairs / BM) + experts tiles; blocks beyond the
// tiles that the plan made return at once.  A pair's result does not depend on where it sits in its tile, so the
// (unordered) placement by atomic counters leaves every row's result what it would be alone.
#include "common.cuh"
#include "mma_tile.cuh"

#define MOE_MAX_EXPERTS 1024

// One warp per row.  Ties go to the lower expert index.
// `over_all`: weights are exp(z - max) / sum over ALL experts (not renormalised over the chosen).
__global__ void route_top_kernel(const float* __restrict__ logits, int* __restrict__ chosen, float* __restrict__ share, int T,
                                 int E, int top, int over_all) {
    pdl_wait();
    pdl_launch_dependents();
    const int lane = threadIdx.x & 31;
    const int r = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (r >= T) return;
    constexpr int PER = MOE_MAX_EXPERTS / 32;
    float z[PER];
#pragma unroll
    for (int c = 0; c < PER; ++c) {
        const int e = lane + 32 * c;
        z[c] = e < E ? logits[(size_t)r * E + e] : -FLT_MAX;
    }
    float first = 0.f, total = 0.f;
    if (over_all) {
        float biggest = -FLT_MAX;
#pragma unroll
        for (int c = 0; c < PER; ++c) biggest = fmaxf(biggest, z[c]);
        biggest = warp_max(biggest);
        float part = 0.f;
#pragma unroll
        for (int c = 0; c < PER; ++c)
            if (lane + 32 * c < E) part += expf(z[c] - biggest);
        total = warp_sum(part);
    }
    for (int s = 0; s < top; ++s) {
        float best = -FLT_MAX;
        int arg = 0x7fffffff;
#pragma unroll
        for (int c = 0; c < PER; ++c) {
            const int e = lane + 32 * c;
            if (e < E && (z[c] > best)) { best = z[c]; arg = e; }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, o);
            const int oa = __shfl_xor_sync(0xffffffffu, arg, o);
            if (ob > best || (ob == best && oa < arg)) { best = ob; arg = oa; }
        }
#pragma unroll
        for (int c = 0; c < PER; ++c)
            if (lane + 32 * c == arg) z[c] = -FLT_MAX;
        if (s == 0) first = best;                 // the largest of all: the softmax's reference point
        const float p = expf(best - first);
        if (!over_all) total += p;
        if (lane == 0) {
            chosen[(size_t)r * top + s] = arg;
            share[(size_t)r * top + s] = p;
        }
    }
    __syncwarp();
    if (lane == 0)
        for (int s = 0; s < top; ++s) share[(size_t)r * top + s] /= total;
}

static int launch_route_top(const float* logits, int* chosen, float* share, int T, int E, int top, int over_all, cudaStream_t stream) {
    if (T <= 0) return KVB_OK;
    if (E < 1 || E > MOE_MAX_EXPERTS || top < 1 || top > E) return KVB_ERR_SHAPE;
    const int warps = 4;
    kvb_launch(route_top_kernel, dim3((T + warps - 1) / warps), dim3(32 * warps), 0, stream, logits, chosen, share, T, E, top, over_all);
    return kvb_launch_status();
}

KVB_API int kvb_route_top(const float* logits, int* chosen, float* share, int T, int E, int top, cudaStream_t stream) {
    return launch_route_top(logits, chosen, share, T, E, top, 0, stream);
}

// `over_all` 1: the weights are the softmax over all experts at the chosen ones.
KVB_API int kvb_route_top_scores(const float* logits, int* chosen, float* share, int T, int E, int top, int over_all,
                                 cudaStream_t stream) {
    return launch_route_top(logits, chosen, share, T, E, top, over_all ? 1 : 0, stream);
}

// One block.  plan = [tile count | expert offsets (E + 1) | cursors (E)]; tiles[i] = (expert, first sorted row, rows).
// `pad_runs`: every expert's run of rows starts at a multiple of BM (the rows between the runs belong to no pair).
__global__ void routed_plan_kernel(const int* __restrict__ chosen, int pairs, int E, int BM, int pad_runs, int* __restrict__ place,
                                   int* __restrict__ sorted_pair, int* __restrict__ plan, int* __restrict__ tiles) {
    pdl_wait();
    pdl_launch_dependents();
    __shared__ int count[MOE_MAX_EXPERTS];
    __shared__ int offset[MOE_MAX_EXPERTS + 1];
    __shared__ int tile_base[MOE_MAX_EXPERTS + 1];
    for (int e = threadIdx.x; e < E; e += blockDim.x) count[e] = 0;
    __syncthreads();
    for (int p = threadIdx.x; p < pairs; p += blockDim.x) atomicAdd(&count[chosen[p]], 1);
    __syncthreads();
    if (threadIdx.x == 0) {
        int at = 0, tiles_at = 0;
        for (int e = 0; e < E; ++e) {
            offset[e] = at;
            tile_base[e] = tiles_at;
            at += pad_runs ? (count[e] + BM - 1) / BM * BM : count[e];
            tiles_at += (count[e] + BM - 1) / BM;
        }
        offset[E] = at;
        tile_base[E] = tiles_at;
        plan[0] = tiles_at;
    }
    __syncthreads();
    for (int e = threadIdx.x; e < E; e += blockDim.x) {
        const int n = count[e];
        for (int i = 0; i * BM < n; ++i) {
            int* t = tiles + 3 * (tile_base[e] + i);
            t[0] = e;
            t[1] = offset[e] + i * BM;
            t[2] = min(BM, n - i * BM);
        }
        count[e] = 0;                                  // now the expert's cursor
    }
    __syncthreads();
    for (int p = threadIdx.x; p < pairs; p += blockDim.x) {
        const int e = chosen[p];
        const int at = offset[e] + atomicAdd(&count[e], 1);
        place[p] = at;
        if (!pad_runs) sorted_pair[at] = p;
    }
}

KVB_API int kvb_routed_plan(const int* chosen, int pairs, int E, int BM, int pad_runs, int* place, int* sorted_pair, int* plan,
                            int* tiles, cudaStream_t stream) {
    if (pairs <= 0) return KVB_OK;
    if (E < 1 || E > MOE_MAX_EXPERTS || BM < 1) return KVB_ERR_SHAPE;
    kvb_launch(routed_plan_kernel, dim3(1), dim3(1024), 0, stream, chosen, pairs, E, BM, pad_runs, place, sorted_pair, plan, tiles);
    return kvb_launch_status();
}

// The clamped gated activation of a (gate, up) pair: g' sigmoid(1.702 g') (u' + 1), g' = min(g, limit), u' = clamp(u, -limit, limit);
// limit <= 0: the plain gated form silu(g) u.
__device__ __forceinline__ float clamped_swiglu(float g, float u, float limit) {
    if (limit <= 0.f) return g / (1.f + expf(-g)) * u;
    g = fminf(g, limit);
    u = fminf(fmaxf(u, -limit), limit);
    return g / (1.f + expf(-1.702f * g)) * (u + 1.f);
}

// ACT: 0 none, 1 relu(v)^2, 2 the clamped gated activation of column pairs (2 i, 2 i + 1) = (gate i, up i): out has N / 2
// columns.  `gather_div` > 0: row i of A is x[sorted_pair[i] / gather_div]; 0: row i of A is a[i].
template <typename T, int BM, int ACT>
__global__ void __launch_bounds__(256) grouped_gemm_simt_kernel(const T* __restrict__ a, const int* __restrict__ sorted_pair,
                                                                int gather_div, const T* __restrict__ w, T* __restrict__ out,
                                                                const int* __restrict__ plan, const int* __restrict__ tiles,
                                                                int N, int K, float limit) {
    pdl_wait();
    pdl_launch_dependents();
    if ((int)blockIdx.y >= plan[0]) return;
    constexpr int BN = 64, BK = 16, TM = BM / 16;
    __shared__ float as_s[BK][BM + 4];
    __shared__ float ws_s[BK][BN + 4];
    __shared__ int src_row[BM];
    const int tid = threadIdx.x;
    const int ty = tid / 16, tx = tid % 16;
    const int expert = tiles[3 * blockIdx.y], row0 = tiles[3 * blockIdx.y + 1], rows = tiles[3 * blockIdx.y + 2];
    const int n0 = blockIdx.x * BN;
    const T* we = w + (size_t)expert * N * K;
    for (int i = tid; i < BM; i += 256)
        src_row[i] = i < rows ? (gather_div > 0 ? sorted_pair[row0 + i] / gather_div : row0 + i) : -1;
    __syncthreads();

    float acc[TM][4];
#pragma unroll
    for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
    for (int k0 = 0; k0 < K; k0 += BK) {
        for (int e = tid; e < BM * BK; e += 256) {
            const int row = e / BK, kk = e % BK;
            const int src = src_row[row];
            as_s[kk][row] = (src >= 0 && k0 + kk < K) ? to_f32<T>(a[(size_t)src * K + k0 + kk]) : 0.f;
        }
        for (int e = tid; e < BN * BK; e += 256) {
            const int row = e / BK, kk = e % BK;
            const int gn = n0 + row;
            ws_s[kk][row] = (gn < N && k0 + kk < K) ? to_f32<T>(we[(size_t)gn * K + k0 + kk]) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < BK; ++kk) {
            float av[TM], b[4];
#pragma unroll
            for (int i = 0; i < TM; ++i) av[i] = as_s[kk][ty * TM + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) b[j] = ws_s[kk][tx * 4 + j];
#pragma unroll
            for (int i = 0; i < TM; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(av[i], b[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < TM; ++i) {
        const int row = ty * TM + i;
        if (row >= rows) continue;
        if (ACT == 2) {
#pragma unroll
            for (int j = 0; j < 4; j += 2) {
                const int gn = n0 + tx * 4 + j;
                if (gn + 1 < N) out[(size_t)(row0 + row) * (N / 2) + gn / 2] = from_f32<T>(clamped_swiglu(acc[i][j], acc[i][j + 1], limit));
            }
            continue;
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int gn = n0 + tx * 4 + j;
            if (gn >= N) continue;
            float v = acc[i][j];
            if (ACT == 1) {
                v = fmaxf(v, 0.f);
                v = v * v;
            }
            out[(size_t)(row0 + row) * N + gn] = from_f32<T>(v);
        }
    }
}

// The same on the tensor cores (bfloat16, K a multiple of 8, N even).
template <int MT, int ACT>
__global__ void __launch_bounds__(mt::THREADS) grouped_gemm_mma_kernel(const bf16* __restrict__ a, const int* __restrict__ sorted_pair,
                                                                       int gather_div, const bf16* __restrict__ w,
                                                                       bf16* __restrict__ out, const int* __restrict__ plan,
                                                                       const int* __restrict__ tiles, int N, int K, float limit) {
    pdl_wait();
    pdl_launch_dependents();
    if ((int)blockIdx.y >= plan[0]) return;
    constexpr int BM = 16 * MT;
    __shared__ __align__(16) mt::Smem<MT> sm;
    __shared__ int src_row[BM];
    const int expert = tiles[3 * blockIdx.y], row0 = tiles[3 * blockIdx.y + 1], rows = tiles[3 * blockIdx.y + 2];
    const int n0 = blockIdx.x * mt::BN;
    for (int i = threadIdx.x; i < BM; i += mt::THREADS)
        src_row[i] = i < rows ? (gather_div > 0 ? sorted_pair[row0 + i] / gather_div : row0 + i) : -1;
    __syncthreads();
    auto a_row = [&](int r) -> const bf16* { return src_row[r] >= 0 ? a + (size_t)src_row[r] * K : nullptr; };
    auto store = [&](int r, int c, float v0, float v1) {
        const int gn = n0 + c;
        if (r >= rows || gn >= N) return;
        if (ACT == 2) {                 // columns gn (even) and gn + 1 are gate and up of index gn / 2
            if (gn + 1 < N) out[(size_t)(row0 + r) * (N / 2) + gn / 2] = __float2bfloat16_rn(clamped_swiglu(v0, v1, limit));
            return;
        }
        if (ACT == 1) {
            v0 = fmaxf(v0, 0.f); v0 *= v0;
            v1 = fmaxf(v1, 0.f); v1 *= v1;
        }
        bf16* dst = out + (size_t)(row0 + r) * N + gn;
        if (gn + 1 < N) *reinterpret_cast<__nv_bfloat162*>(dst) = __floats2bfloat162_rn(v0, v1);
        else dst[0] = __float2bfloat16_rn(v0);
    };
    mt::tile_product<MT>(sm, a_row, w + ((size_t)expert * N + n0) * K, min(mt::BN, N - n0), K, store);
}

template <typename T, int BM>
static void launch_grouped(const T* a, const int* sorted_pair, int gather_div, const T* w, T* out, const int* plan,
                           const int* tiles, int max_tiles, int N, int K, int act, float limit, cudaStream_t stream) {
    dim3 grid((N + 63) / 64, max_tiles);
    if (act == 2)
        kvb_launch(grouped_gemm_simt_kernel<T, BM, 2>, grid, dim3(256), 0, stream, a, sorted_pair, gather_div, w, out, plan, tiles, N, K, limit);
    else if (act == 1)
        kvb_launch(grouped_gemm_simt_kernel<T, BM, 1>, grid, dim3(256), 0, stream, a, sorted_pair, gather_div, w, out, plan, tiles, N, K, limit);
    else
        kvb_launch(grouped_gemm_simt_kernel<T, BM, 0>, grid, dim3(256), 0, stream, a, sorted_pair, gather_div, w, out, plan, tiles, N, K, limit);
}

static int grouped_gemm(int dtype, const void* a, const int* sorted_pair, int gather_div, const void* w, void* out,
                        const int* plan, const int* tiles, int max_tiles, int BM, int N, int K, int act, float limit,
                        cudaStream_t stream) {
    if (max_tiles <= 0) return KVB_OK;
    if (N < 1 || K < 1 || (BM != 16 && BM != 64) || act < 0 || act > 2 || (act == 2 && N % 2 != 0)) return KVB_ERR_SHAPE;
    if (max_tiles > 65535) return KVB_ERR_LIMIT;
#define KVB_GROUPED(T, BM_)                                                                                                  \
    launch_grouped<T, BM_>((const T*)a, sorted_pair, gather_div, (const T*)w, (T*)out, plan, tiles, max_tiles, N, K, act, limit, stream)
    if (dtype == KVB_F32) {
        if (BM == 16) KVB_GROUPED(float, 16); else KVB_GROUPED(float, 64);
    } else if (dtype == KVB_BF16) {
        const bool aligned = K % 8 == 0 && N % 2 == 0 && ((uintptr_t)a | (uintptr_t)w) % 16 == 0 && (uintptr_t)out % 4 == 0;
        if (aligned && getenv("KVB_GROUPED_SIMT") == nullptr) {
            dim3 grid((N + 63) / 64, max_tiles);
            const bf16 *ab = (const bf16*)a, *wb = (const bf16*)w;
#define KVB_GROUPED_MMA(MT, ACT_) \
    kvb_launch(grouped_gemm_mma_kernel<MT, ACT_>, grid, dim3(mt::THREADS), 0, stream, ab, sorted_pair, gather_div, wb, (bf16*)out, plan, tiles, N, K, limit)
            if (BM == 16) { if (act == 2) KVB_GROUPED_MMA(1, 2); else if (act == 1) KVB_GROUPED_MMA(1, 1); else KVB_GROUPED_MMA(1, 0); }
            else { if (act == 2) KVB_GROUPED_MMA(4, 2); else if (act == 1) KVB_GROUPED_MMA(4, 1); else KVB_GROUPED_MMA(4, 0); }
#undef KVB_GROUPED_MMA
        } else if (BM == 16) {
            KVB_GROUPED(bf16, 16);
        } else {
            KVB_GROUPED(bf16, 64);
        }
    } else {
        return KVB_ERR_DTYPE;
    }
#undef KVB_GROUPED
    return kvb_launch_status();
}

// `BM` must be the one the plan was made with (16 or 64).
KVB_API int kvb_grouped_gemm(int dtype, const void* a, const int* sorted_pair, int gather_div, const void* w, void* out,
                             const int* plan, const int* tiles, int max_tiles, int BM, int N, int K, int act,
                             cudaStream_t stream) {
    if (act > 1) return KVB_ERR_SHAPE;
    return grouped_gemm(dtype, a, sorted_pair, gather_div, w, out, plan, tiles, max_tiles, BM, N, K, act, 0.f, stream);
}

// The same with the activation's constant: act 2 is the clamped gated activation with `limit`, out [rows, N / 2].
KVB_API int kvb_grouped_gemm_act(int dtype, const void* a, const int* sorted_pair, int gather_div, const void* w, void* out,
                                 const int* plan, const int* tiles, int max_tiles, int BM, int N, int K, int act, float limit,
                                 cudaStream_t stream) {
    return grouped_gemm(dtype, a, sorted_pair, gather_div, w, out, plan, tiles, max_tiles, BM, N, K, act, limit, stream);
}

// out[t, :] = base[t, :] (if given) + sum_s share[t, s] * y[place[t * top + s], :]
template <typename T>
__global__ void routed_combine_kernel(const T* __restrict__ y, const int* __restrict__ place, const float* __restrict__ share,
                                      const T* __restrict__ base, T* __restrict__ out, int top, int H) {
    pdl_wait();
    pdl_launch_dependents();
    const int t = blockIdx.x;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        float v = base ? to_f32<T>(base[(size_t)t * H + i]) : 0.f;
        for (int s = 0; s < top; ++s) v += share[(size_t)t * top + s] * to_f32<T>(y[(size_t)place[(size_t)t * top + s] * H + i]);
        out[(size_t)t * H + i] = from_f32<T>(v);
    }
}

static int routed_combine(int dtype, const void* y, const int* place, const float* share, const void* base, void* out, int T, int top,
                          int H, cudaStream_t stream) {
    if (T <= 0) return KVB_OK;
    if (dtype == KVB_F32)
        kvb_launch(routed_combine_kernel<float>, dim3(T), dim3(128), 0, stream, (const float*)y, place, share, (const float*)base,
                   (float*)out, top, H);
    else if (dtype == KVB_BF16)
        kvb_launch(routed_combine_kernel<bf16>, dim3(T), dim3(128), 0, stream, (const bf16*)y, place, share, (const bf16*)base,
                   (bf16*)out, top, H);
    else
        return KVB_ERR_DTYPE;
    return kvb_launch_status();
}

KVB_API int kvb_routed_combine(int dtype, const void* y, const int* place, const float* share, void* out, int T, int top, int H,
                               cudaStream_t stream) {
    return routed_combine(dtype, y, place, share, nullptr, out, T, top, H, stream);
}

// The same on top of `base` [T, H] (what every row takes besides its experts).
KVB_API int kvb_routed_combine_base(int dtype, const void* y, const int* place, const float* share, const void* base, void* out,
                                    int T, int top, int H, cudaStream_t stream) {
    return routed_combine(dtype, y, place, share, base, out, T, top, H, stream);
}
