// Attention over a cache of shared key rows (bfloat16, tensor cores): every head of a token scores the same row of
// Dk numbers per cached token, and the row's first Dv numbers are its value.  q [T, H * Dk], out [T, H * Dv].
//
// Because all heads read the same keys, the rows of a tile are (token, head) pairs: row m of a request's portion is
// token m / H, head m % H, and q and out are contiguous in m.  A decoded token with H heads fills a tile of 16 rows
// as well as 16 tokens of one head would; a key tile is read once for all heads.
//
// A block of 8 warps owns BM = 16 * MT rows and a run of keys [kb, ke) (a work item made on the host, see
// kernels/latent_plan.py).  Per tile of 64 keys, brought by cp.async into rows padded by 16 bytes:
//   scores   warp w takes keys 8 w .. 8 w + 7 for all MT row tiles (mma.sync m16n8k16 over Dk), scaled to base 2,
//            masked (causal by the row's own position, window) and written to shared memory as float32;
//   softmax  float32: running maximum and sum per row, p = 2^(s - m) rounded to bfloat16 for the second product,
//            the sum taken from the unrounded p;
//   values   warp w owns output columns [8 NV w, 8 NV (w + 1)) for all row tiles: O = O * 2^(m_old - m_new) + P . V,
//            V read from the same shared rows as the keys (ldmatrix.trans).
// With `nsplit` > 1 the items of a tile leave (O, m, l) in scratch and `latent_flash_merge_kernel` adds them in the
// order of the splits; the split depends on the step's tiles, not on which block runs first.
// Two key stages where shared memory allows (the next tile is requested before this one is used), else one.
// `window` > 0: a row at position p sees keys p - window + 1 .. p; the work list starts a tile's keys at the 64-key tile
// that holds the first key its first row sees, and keys before that key are not fetched (a windowed cache entry may have
// given their pages back) but zero-filled and masked.  `sink` (one logit per head, or null): the softmax's denominator
// also holds exp(sink[h]); the rows of a tile's first split start from (m, l) = (sink, 1) instead of (-inf, 0).
#include "common.cuh"

namespace lf {

constexpr int BN = 64;            // keys in a tile
constexpr int THREADS = 256;
constexpr float MASKED = -1e30f;

__device__ __forceinline__ uint32_t smem_addr(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void cp_async16(void* smem, const void* gmem, bool valid) {
    const int bytes = valid ? 16 : 0;   // 0 source bytes: the 16 destination bytes are zero-filled
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(smem_addr(smem)), "l"(gmem), "r"(bytes));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_group 0;\n" ::); }
__device__ __forceinline__ void cp_async_wait_one() { asm volatile("cp.async.wait_group 1;\n" ::); }
__device__ __forceinline__ void ldmatrix_x4(uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3, const void* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(smem_addr(p)));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3, const void* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(smem_addr(p)));
}
__device__ __forceinline__ void ldmatrix_x2_trans(uint32_t& r0, uint32_t& r1, const void* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x2.trans.shared.b16 {%0,%1}, [%2];\n" : "=r"(r0), "=r"(r1) : "r"(smem_addr(p)));
}
__device__ __forceinline__ void mma_bf16(float* c, const uint32_t* a, uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

struct Layout {
    int dk_pad, qs, rs, ss, ps;          // padded Dk; strides (elements) of the Q, key, score and P rows
    size_t q_off, k_off, s_off, p_off, st_off, total;
};

__host__ __device__ inline Layout make_layout(int MT, int NV, int Dk, int nstage) {
    Layout L;
    const int BM = 16 * MT;
    L.dk_pad = (Dk + 31) / 32 * 32;
    const int dv_pad = 64 * NV;
    L.qs = L.dk_pad + 8;
    L.rs = (L.dk_pad > dv_pad ? L.dk_pad : dv_pad) + 8;
    L.ss = BN + 8;
    L.ps = BN + 8;
    size_t at = 0;
    L.q_off = at;  at += (size_t)BM * L.qs * 2;
    L.k_off = at;  at += (size_t)nstage * BN * L.rs * 2;
    L.s_off = at;  at += (size_t)BM * L.ss * 4;
    L.p_off = at;  at += (size_t)BM * L.ps * 2;
    L.st_off = at; at += (size_t)BM * 4 * 4;          // m, l, corr, position of every row
    L.total = at;
    return L;
}

// Tiles of 64 rows with values of up to 256 numbers are held to 128 registers, so that two blocks share an SM and one's copies
// and softmax overlap the other's products.
template <int MT, int NV>
__global__ void __launch_bounds__(THREADS, (MT == 4 && NV <= 4) ? 2 : 1) latent_flash_kernel(
    const bf16* __restrict__ q, bf16* __restrict__ out, const bf16* __restrict__ k_pages, const int* __restrict__ block_table,
    int table_stride, const int* __restrict__ items, const int* __restrict__ seg_q_start, const int* __restrict__ seg_q_len,
    const int* __restrict__ seg_kv_len, float* __restrict__ part_o, float* __restrict__ part_ml, int H, int Dk, int Dv,
    int page_size, int window, float scale_log2, int nsplit, int nstage, const float* __restrict__ sink, int* __restrict__ err) {
    constexpr int BM = 16 * MT;
    extern __shared__ __align__(16) unsigned char smem[];
    const Layout L = make_layout(MT, NV, Dk, nstage);
    bf16* Qs = reinterpret_cast<bf16*>(smem + L.q_off);
    bf16* Ks = reinterpret_cast<bf16*>(smem + L.k_off);
    float* Ss = reinterpret_cast<float*>(smem + L.s_off);
    bf16* Ps = reinterpret_cast<bf16*>(smem + L.p_off);
    float* m_run = reinterpret_cast<float*>(smem + L.st_off);
    float* l_run = m_run + BM;
    float* corr = l_run + BM;
    int* rowpos = reinterpret_cast<int*>(corr + BM);

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, t4 = lane & 3;
    const int* item = items + 4 * blockIdx.x;
    const int seg = item[0], m0 = item[1], kb = item[2], ke = item[3];
    const int q_len = seg_q_len[seg], kv_len = seg_kv_len[seg];
    const int start = kv_len - q_len;                       // tokens cached before this step
    const int M_total = q_len * H;
    const size_t row_base = (size_t)seg_q_start[seg] * H + m0;   // q and out are contiguous in (token, head)
    const int* table = block_table + (size_t)seg * table_stride;
    const int key_lo = window > 0 ? max(0, start + m0 / H - window + 1) : 0;     // the first key any row of the tile sees
    const bool first_split = blockIdx.x % nsplit == 0;
    pdl_wait();
    pdl_launch_dependents();

    // ---- the rows: positions, running state, Q into shared memory -----------------------------------------------
    for (int r = tid; r < BM; r += THREADS) {
        const int m = m0 + r;
        rowpos[r] = m < M_total ? start + m / H : -1;
        const bool from_sink = sink != nullptr && first_split && m < M_total;
        m_run[r] = from_sink ? sink[m % H] * 1.4426950408889634f : MASKED;
        l_run[r] = from_sink ? 1.f : 0.f;
    }
    const int q_chunks = L.dk_pad / 8;
    for (int e = tid; e < BM * q_chunks; e += THREADS) {
        const int r = e / q_chunks, c = e - r * q_chunks;
        const bool valid = m0 + r < M_total && c * 8 < Dk;
        cp_async16(Qs + (size_t)r * L.qs + c * 8, q + (row_base + (valid ? r : 0)) * Dk + (valid ? c * 8 : 0), valid);
    }
    cp_async_commit();

    const int row_chunks = (L.rs - 8) / 8;                  // chunks of a key row in shared memory, padding columns included
    auto load_keys = [&](int tile, int stage) {
        bf16* dst = Ks + (size_t)stage * BN * L.rs;
        const int r = tid >> 2;                             // four threads share a key row
        const int j = kb + tile * BN + r;
        const bool there = j < ke && j >= key_lo;
        size_t off = 0;
        if (there) {
            const int page = __ldg(table + j / page_size);
            if (page < 0) atomicOr(err, KVB_DEV_BAD_PAGE);
            off = ((size_t)(page < 0 ? 0 : page) * page_size + (j % page_size)) * Dk;
        }
        for (int c = tid & 3; c < row_chunks; c += 4) {
            const bool valid = there && c * 8 < Dk;
            cp_async16(dst + (size_t)r * L.rs + c * 8, k_pages + off + (valid ? c * 8 : 0), valid);
        }
        cp_async_commit();
    };

    float o[MT][NV][4];
#pragma unroll
    for (int mt = 0; mt < MT; ++mt)
#pragma unroll
        for (int nv = 0; nv < NV; ++nv) o[mt][nv][0] = o[mt][nv][1] = o[mt][nv][2] = o[mt][nv][3] = 0.f;

    const int ntiles = (ke - kb + BN - 1) / BN;
    if (ntiles > 0) load_keys(0, 0);
    const int KS2 = L.dk_pad / 32;
    for (int tile = 0; tile < ntiles; ++tile) {
        const int stage = nstage == 2 ? (tile & 1) : 0;
        const bool ahead = nstage == 2 && tile + 1 < ntiles;
        if (ahead) load_keys(tile + 1, stage ^ 1);
        if (ahead) cp_async_wait_one(); else cp_async_wait_all();
        __syncthreads();
        const bf16* Kt = Ks + (size_t)stage * BN * L.rs;
        const int key0 = kb + tile * BN;

        // ---- scores of keys 8 warp .. 8 warp + 7 for every row tile ------------------------------------------------
        float s[MT][4];
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) s[mt][0] = s[mt][1] = s[mt][2] = s[mt][3] = 0.f;
#pragma unroll 3
        for (int k2 = 0; k2 < KS2; ++k2) {
            uint32_t b[4];
            ldmatrix_x4(b[0], b[1], b[2], b[3], Kt + (size_t)(8 * warp + (lane & 7)) * L.rs + k2 * 32 + (lane >> 3) * 8);
#pragma unroll
            for (int half = 0; half < 2; ++half) {
#pragma unroll
                for (int mt = 0; mt < MT; ++mt) {
                    uint32_t a[4];
                    ldmatrix_x4(a[0], a[1], a[2], a[3], Qs + (size_t)(mt * 16 + (lane & 15)) * L.qs + k2 * 32 + half * 16 + (lane >> 4) * 8);
                    mma_bf16(s[mt], a, b[2 * half], b[2 * half + 1]);
                }
            }
        }
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) {
#pragma unroll
            for (int hi = 0; hi < 2; ++hi) {             // rows g and g + 8: two columns each, stored as one 8-byte word
                const int r = mt * 16 + g + hi * 8;
                const int c = 8 * warp + 2 * t4;
                const int pos = rowpos[r];
                float2 v;
                {
                    const int j = key0 + c;
                    const bool seen = j < ke && j <= pos && (window <= 0 || j > pos - window);
                    v.x = seen ? s[mt][2 * hi] * scale_log2 : MASKED;
                }
                {
                    const int j = key0 + c + 1;
                    const bool seen = j < ke && j <= pos && (window <= 0 || j > pos - window);
                    v.y = seen ? s[mt][2 * hi + 1] * scale_log2 : MASKED;
                }
                *reinterpret_cast<float2*>(Ss + r * L.ss + c) = v;
            }
        }
        __syncthreads();

        // ---- softmax of the tile: TPR threads share a row -------------------------------------------------------------
        {
            constexpr int TPR = THREADS / BM, CPT = BN / TPR;
            const int r = tid / TPR, c0 = (tid % TPR) * CPT;
            float v[CPT];
            float mx = MASKED;
#pragma unroll
            for (int i = 0; i < CPT; i += 4) {
                const float4 f = *reinterpret_cast<const float4*>(Ss + r * L.ss + c0 + i);
                v[i] = f.x; v[i + 1] = f.y; v[i + 2] = f.z; v[i + 3] = f.w;
            }
#pragma unroll
            for (int i = 0; i < CPT; ++i) mx = fmaxf(mx, v[i]);
#pragma unroll
            for (int d = TPR / 2; d > 0; d >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, d));
            const float m_old = m_run[r];
            const float m_new = fmaxf(m_old, mx);
            float sum = 0.f;
            uint32_t packed[CPT / 2];
#pragma unroll
            for (int i = 0; i < CPT; i += 2) {
                const float p0 = v[i] > 0.5f * MASKED ? exp2f(v[i] - m_new) : 0.f;
                const float p1 = v[i + 1] > 0.5f * MASKED ? exp2f(v[i + 1] - m_new) : 0.f;
                sum += p0;
                sum += p1;
                __nv_bfloat162 pp = __floats2bfloat162_rn(p0, p1);
                packed[i / 2] = *reinterpret_cast<uint32_t*>(&pp);
            }
            if constexpr (CPT == 4) {
                *reinterpret_cast<uint2*>(Ps + r * L.ps + c0) = make_uint2(packed[0], packed[1]);
            } else {
#pragma unroll
                for (int i = 0; i < CPT / 8; ++i)
                    *reinterpret_cast<uint4*>(Ps + r * L.ps + c0 + 8 * i) = make_uint4(packed[4 * i], packed[4 * i + 1], packed[4 * i + 2], packed[4 * i + 3]);
            }
#pragma unroll
            for (int d = TPR / 2; d > 0; d >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, d);
            if (tid % TPR == 0) {
                const float cf = exp2f(m_old - m_new);
                corr[r] = cf;
                l_run[r] = l_run[r] * cf + sum;
                m_run[r] = m_new;
            }
        }
        __syncthreads();

        // ---- O = O * corr + P . V for this warp's columns --------------------------------------------------------------
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) {
            const float c0 = corr[mt * 16 + g], c1 = corr[mt * 16 + g + 8];
#pragma unroll
            for (int nv = 0; nv < NV; ++nv) {
                o[mt][nv][0] *= c0; o[mt][nv][1] *= c0; o[mt][nv][2] *= c1; o[mt][nv][3] *= c1;
            }
        }
#pragma unroll
        for (int kk = 0; kk < BN / 16; ++kk) {
            uint32_t b[NV][2];
            const int krow = kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
            if constexpr (NV == 1) {
                ldmatrix_x2_trans(b[0][0], b[0][1], Kt + (size_t)krow * L.rs + warp * 8);
            } else {
#pragma unroll
                for (int n2 = 0; n2 < NV / 2; ++n2)
                    ldmatrix_x4_trans(b[2 * n2][0], b[2 * n2][1], b[2 * n2 + 1][0], b[2 * n2 + 1][1],
                                      Kt + (size_t)krow * L.rs + warp * 8 * NV + n2 * 16 + (lane >> 4) * 8);
            }
#pragma unroll
            for (int mt = 0; mt < MT; ++mt) {
                uint32_t a[4];
                ldmatrix_x4(a[0], a[1], a[2], a[3], Ps + (size_t)(mt * 16 + (lane & 15)) * L.ps + kk * 16 + (lane >> 4) * 8);
#pragma unroll
                for (int nv = 0; nv < NV; ++nv) mma_bf16(o[mt][nv], a, b[nv][0], b[nv][1]);
            }
        }
        __syncthreads();                    // the stage and P may be overwritten now
        if (nstage == 1 && tile + 1 < ntiles) load_keys(tile + 1, 0);
    }
    cp_async_wait_all();                    // Q's group, if there was no tile at all

    // ---- the rows' results ---------------------------------------------------------------------------------------------
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) {
#pragma unroll
        for (int hi = 0; hi < 2; ++hi) {
            const int r = mt * 16 + g + hi * 8;
            if (m0 + r >= M_total) continue;
            if (nsplit == 1) {
                const float l = l_run[r];
                const float inv = l > 0.f ? 1.f / l : 0.f;
                bf16* orow = out + (row_base + r) * Dv;
#pragma unroll
                for (int nv = 0; nv < NV; ++nv) {
                    const int d = warp * 8 * NV + nv * 8 + 2 * t4;
                    if (d + 1 < Dv) {
                        *reinterpret_cast<__nv_bfloat162*>(orow + d) = __floats2bfloat162_rn(o[mt][nv][2 * hi] * inv, o[mt][nv][2 * hi + 1] * inv);
                    } else if (d < Dv) {
                        orow[d] = __float2bfloat16_rn(o[mt][nv][2 * hi] * inv);
                    }
                }
            } else {
                float* prow = part_o + ((size_t)blockIdx.x * BM + r) * Dv;
#pragma unroll
                for (int nv = 0; nv < NV; ++nv) {
                    const int d = warp * 8 * NV + nv * 8 + 2 * t4;
                    if (d < Dv) prow[d] = o[mt][nv][2 * hi];
                    if (d + 1 < Dv) prow[d + 1] = o[mt][nv][2 * hi + 1];
                }
            }
        }
    }
    if (nsplit > 1)
        for (int r = tid; r < BM; r += THREADS) {
            part_ml[((size_t)blockIdx.x * BM + r) * 2] = m_run[r];
            part_ml[((size_t)blockIdx.x * BM + r) * 2 + 1] = l_run[r];
        }
}

// out[row] = sum_s 2^(m_s - M) O_s[row] / sum_s 2^(m_s - M) l_s over the `nsplit` items of the row's tile.
// Grid (tiles, BM); the items of tile i are i * nsplit .. (i + 1) * nsplit - 1.  A block is MERGE_GROUPS x Dv / 4 threads:
// thread (g, c) adds four columns of the splits g, g + MERGE_GROUPS, ... (independent loads, all in flight at once), and the
// groups' sums are added in the order of the groups - a fixed order, whichever block runs first.
constexpr int MAX_SPLITS = 32, MERGE_GROUPS = 8;
__global__ void latent_flash_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                          const int* __restrict__ items, const int* __restrict__ seg_q_start,
                                          const int* __restrict__ seg_q_len, bf16* __restrict__ out, int H, int Dv, int BM,
                                          int nsplit) {
    __shared__ float weight[MAX_SPLITS];
    __shared__ float inv_s;
    extern __shared__ float4 sums[];                     // [MERGE_GROUPS][Dv / 4]
    const int first = blockIdx.x * nsplit, r = blockIdx.y;
    const int seg = items[4 * first], m0 = items[4 * first + 1];
    const int cols = Dv >> 2;
    const int g = threadIdx.x / cols, c = threadIdx.x - g * cols;
    pdl_wait();
    pdl_launch_dependents();
    if (m0 + r >= seg_q_len[seg] * H) return;
    const float4* base = reinterpret_cast<const float4*>(part_o + ((size_t)first * BM + r) * Dv) + c;
    const size_t step = (size_t)BM * cols;
    float4 v[MAX_SPLITS / MERGE_GROUPS];
#pragma unroll
    for (int i = 0; i < MAX_SPLITS / MERGE_GROUPS; ++i) {
        const int s = g + i * MERGE_GROUPS;
        v[i] = s < nsplit ? base[(size_t)s * step] : make_float4(0.f, 0.f, 0.f, 0.f);
    }
    if (threadIdx.x < 32) {
        const int s = threadIdx.x;
        const float* ml = part_ml + ((size_t)(first + (s < nsplit ? s : 0)) * BM + r) * 2;
        const float m = s < nsplit ? ml[0] : MASKED, l = s < nsplit ? ml[1] : 0.f;
        const float M = warp_max(m);
        const float w = exp2f(m - M);
        weight[s] = w;
        float total = 0.f;                               // summed in the order of the splits
        for (int i = 0; i < nsplit; ++i) total += __shfl_sync(0xffffffffu, w * l, i);
        if (s == 0) inv_s = total > 0.f ? 1.f / total : 0.f;
    }
    __syncthreads();
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int i = 0; i < MAX_SPLITS / MERGE_GROUPS; ++i) {
        const int s = g + i * MERGE_GROUPS;
        const float w = s < nsplit ? weight[s] : 0.f;
        acc.x += w * v[i].x; acc.y += w * v[i].y; acc.z += w * v[i].z; acc.w += w * v[i].w;
    }
    sums[g * cols + c] = acc;
    __syncthreads();
    if (g == 0) {
        float4 t = sums[c];
        for (int k = 1; k < MERGE_GROUPS; ++k) {
            const float4 u = sums[k * cols + c];
            t.x += u.x; t.y += u.y; t.z += u.z; t.w += u.w;
        }
        const float inv = inv_s;
        bf16* orow = out + ((size_t)seg_q_start[seg] * H + m0 + r) * Dv + 4 * c;
        *reinterpret_cast<__nv_bfloat162*>(orow) = __floats2bfloat162_rn(t.x * inv, t.y * inv);
        *reinterpret_cast<__nv_bfloat162*>(orow + 2) = __floats2bfloat162_rn(t.z * inv, t.w * inv);
    }
}

template <int MT, int NV>
static int launch(const bf16* q, bf16* out, const bf16* k_pages, const int* block_table, int table_stride, const int* items,
                  int n_items, const int* seg_q_start, const int* seg_q_len, const int* seg_kv_len, float* part_o, float* part_ml,
                  int H, int Dk, int Dv, int page_size, int window, float scale, int nsplit, const float* sink, int* err,
                  cudaStream_t stream) {
    int nstage = 2;
    Layout L = make_layout(MT, NV, Dk, nstage);
    // One stage where two stages would keep a second block off the SM (two blocks hide more than a second stage), or do not fit.
    const Layout one = make_layout(MT, NV, Dk, 1);
    const bool two_blocks = MT == 4 && NV <= 4;
    if (L.total > 220 * 1024 || (two_blocks && 2 * L.total > 220 * 1024 && 2 * one.total <= 220 * 1024)) {
        nstage = 1;
        L = one;
        if (L.total > 220 * 1024) return KVB_ERR_LIMIT;
    }
    static size_t configured = 0;                       // per instantiation
    if (L.total > configured) {
        if (cudaFuncSetAttribute(latent_flash_kernel<MT, NV>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)L.total) != cudaSuccess)
            return (int)cudaGetLastError();
        configured = L.total;
    }
    kvb_launch(latent_flash_kernel<MT, NV>, dim3(n_items), dim3(THREADS), L.total, stream, q, out, k_pages, block_table, table_stride,
               items, seg_q_start, seg_q_len, seg_kv_len, part_o, part_ml, H, Dk, Dv, page_size, window,
               scale * 1.4426950408889634f, nsplit, nstage, sink, err);
    return kvb_launch_status();
}

}  // namespace lf

// Whether the kernel takes these sizes (else the caller uses the generic kernel): 0 yes, negative no.
KVB_API int kvb_latent_flash_supports(int Dk, int Dv, int BM) {
    if (Dk % 8 != 0 || Dk < 8 || Dv < 4 || Dv % 4 != 0 || Dv > Dk || Dv > 512 || (BM != 16 && BM != 32 && BM != 64)) return KVB_ERR_SHAPE;
    const int NV = Dv <= 64 ? 1 : (Dv <= 128 ? 2 : (Dv <= 256 ? 4 : 8));
    return lf::make_layout(BM / 16, NV, Dk, 1).total <= 220 * 1024 ? KVB_OK : KVB_ERR_LIMIT;
}

// items: n_items x (segment, first row of the tile, first key, end of keys); the items of a tile are consecutive and
// every tile has `nsplit` of them.  part_o [n_items, BM, Dv] and part_ml [n_items, BM, 2] float32 are needed if nsplit > 1.
KVB_API int kvb_latent_flash(const void* q, void* out, const void* k_pages, const int* block_table, int table_stride,
                             const int* items, int n_items, int n_tiles, const int* seg_q_start, const int* seg_q_len,
                             const int* seg_kv_len, float* part_o, float* part_ml, int H, int Dk, int Dv, int BM, int page_size,
                             int window, float scale, int nsplit, const float* sink, int* err, cudaStream_t stream) {
    if (n_items <= 0) return KVB_OK;
    const int ok = kvb_latent_flash_supports(Dk, Dv, BM);
    if (ok != KVB_OK) return ok;
    if (nsplit < 1 || nsplit > lf::MAX_SPLITS || n_tiles * nsplit != n_items || (nsplit > 1 && (!part_o || !part_ml))) return KVB_ERR_SHAPE;
    const int NV = Dv <= 64 ? 1 : (Dv <= 128 ? 2 : (Dv <= 256 ? 4 : 8));
    int code = KVB_ERR_SHAPE;
#define KVB_LF(MT, NV_)                                                                                                      \
    code = lf::launch<MT, NV_>((const bf16*)q, (bf16*)out, (const bf16*)k_pages, block_table, table_stride, items, n_items,  \
                               seg_q_start, seg_q_len, seg_kv_len, part_o, part_ml, H, Dk, Dv, page_size, window, scale,    \
                               nsplit, sink, err, stream)
    if (BM == 16) {
        if (NV == 1) KVB_LF(1, 1); else if (NV == 2) KVB_LF(1, 2); else if (NV == 4) KVB_LF(1, 4); else KVB_LF(1, 8);
    } else if (BM == 32) {
        if (NV == 1) KVB_LF(2, 1); else if (NV == 2) KVB_LF(2, 2); else if (NV == 4) KVB_LF(2, 4); else KVB_LF(2, 8);
    } else {
        if (NV == 1) KVB_LF(4, 1); else if (NV == 2) KVB_LF(4, 2); else if (NV == 4) KVB_LF(4, 4); else KVB_LF(4, 8);
    }
#undef KVB_LF
    if (code != KVB_OK || nsplit == 1) return code;
    kvb_launch(lf::latent_flash_merge_kernel, dim3(n_tiles, BM), dim3(lf::MERGE_GROUPS * (Dv / 4)), (size_t)lf::MERGE_GROUPS * Dv * 4, stream, (const float*)part_o, (const float*)part_ml,
               items, seg_q_start, seg_q_len, (bf16*)out, H, Dv, BM, nsplit);
    return kvb_launch_status();
}
