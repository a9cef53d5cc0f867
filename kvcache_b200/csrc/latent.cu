// Operators of the latent-attention mixer and of blocks that normalise a sublayer's result before adding it.
//
//   norm_add_rmsnorm          h += norm(delta [* sigmoid(gate)]; dw) (or delta as it is), out = norm(h; w) (or h as it is) [| tail]
//   latent_norm_rope_append   the two latents of a row normalised, the shared key part rotated, the cache row written
//   head_linear               one small matrix product per head: out[t, h, :N] = x[t, h, :K] . W[h]^T, with the rotation
//                             of the head's trailing columns or a sigmoid gate in its epilogue
//
// Everything between loads and stores is float32: sums of squares, norms, angles, the gate.  Reductions run in a
// fixed order per row (`block_sum`), so a row's result does not depend on the rows beside it.
#include "common.cuh"
#include "mma_tile.cuh"

// ---------------------------------------------------------------------------------------------------------------
// One block per output row.  d = delta[r] (times sigmoid(gate[r]), element by element, if gate);
// v = h[r] + (dw ? d * rsqrt(mean(d^2) + deps) * dw : d); rows == null: h[r] = v.
// out[o, :H] = w ? v * rsqrt(mean(v^2) + eps) * w : v;  out[o, H:2H] = tail[r] if tail.  The row lives in shared memory.
template <typename T>
__global__ void norm_add_rmsnorm_kernel(float* __restrict__ h, const T* __restrict__ delta, const T* __restrict__ gate,
                                        const float* __restrict__ dw, float deps, const float* __restrict__ w, float eps,
                                        T* __restrict__ out, const int* __restrict__ rows, const float* __restrict__ tail, int H) {
    pdl_wait();
    pdl_launch_dependents();
    extern __shared__ float row_s[];          // [H] then 33 of scratch, then [H] for the gated delta if there is a gate
    float* scratch = row_s + H;
    float* gated_s = scratch + 33;
    const int o = blockIdx.x;
    const int r = rows ? rows[o] : o;
    float* hr = h + (size_t)r * H;
    const T* dr = delta ? delta + (size_t)r * H : nullptr;
    const T* gr = (delta && gate) ? gate + (size_t)r * H : nullptr;
    float dinv = 1.f;
    if (gr) {
        for (int i = threadIdx.x; i < H; i += blockDim.x)     // each thread reads back what it wrote itself
            gated_s[i] = to_f32<T>(dr[i]) / (1.f + expf(-to_f32<T>(gr[i])));
    }
    auto d_at = [&](int i) { return gr ? gated_s[i] : to_f32<T>(dr[i]); };
    if (dr && dw) {
        float ss = 0.f;
        for (int i = threadIdx.x; i < H; i += blockDim.x) {
            const float d = d_at(i);
            ss += d * d;
        }
        dinv = 1.f / sqrtf(block_sum(ss, scratch) / (float)H + deps);
    }
    float ss = 0.f;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        float v = hr[i];
        if (dr) v += dw ? d_at(i) * dinv * dw[i] : d_at(i);
        if (dr && !rows) hr[i] = v;
        row_s[i] = v;
        ss += v * v;
    }
    if (!out) return;
    float inv = 1.f;
    if (w) inv = 1.f / sqrtf(block_sum(ss, scratch) / (float)H + eps);
    const int stride = tail ? 2 * H : H;
    T* orow = out + (size_t)o * stride;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {     // each thread reads back what it wrote itself
        orow[i] = from_f32<T>(w ? row_s[i] * inv * w[i] : row_s[i]);
        if (tail) orow[H + i] = from_f32<T>(tail[(size_t)r * H + i]);
    }
}

KVB_API int kvb_norm_add_rmsnorm(int dtype, float* h, const void* delta, const void* gate, const float* dw, float deps,
                                 const float* w, float eps, void* out, const int* rows, const float* tail, int n_rows, int H,
                                 cudaStream_t stream) {
    if (n_rows <= 0) return KVB_OK;
    if (H < 1) return KVB_ERR_SHAPE;
    const size_t smem = (size_t)((gate ? 2 : 1) * H + 33) * sizeof(float);
    if (smem > 200 * 1024) return KVB_ERR_LIMIT;
    const int threads = H >= 2048 ? 512 : (H >= 512 ? 256 : 128);
    if (dtype == KVB_F32) {
        if (smem > 48 * 1024) cudaFuncSetAttribute(norm_add_rmsnorm_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        kvb_launch(norm_add_rmsnorm_kernel<float>, dim3(n_rows), dim3(threads), smem, stream, h, (const float*)delta, (const float*)gate,
                   dw, deps, w, eps, (float*)out, rows, tail, H);
    } else if (dtype == KVB_BF16) {
        if (smem > 48 * 1024) cudaFuncSetAttribute(norm_add_rmsnorm_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        kvb_launch(norm_add_rmsnorm_kernel<bf16>, dim3(n_rows), dim3(threads), smem, stream, h, (const bf16*)delta, (const bf16*)gate,
                   dw, deps, w, eps, (bf16*)out, rows, tail, H);
    } else {
        return KVB_ERR_DTYPE;
    }
    return kvb_launch_status();
}

// ---------------------------------------------------------------------------------------------------------------
// One block per row of the fused projection `proj` [T, P]: columns [0, q_rank) are the query latent (q_rank 0: there is
// none, and cq is not written), [kv_col, kv_col + kv_rank) the key/value latent, the next rot_dim the key part that all
// heads share.
//   cq[r]                 = norm(query latent; qw)
//   cache row of (r's request, r's position) = [norm(key/value latent; kw) | R_pos(shared key part)]
// R rotates the first 2 * rot_half numbers (t pairs with t + rot_half); the rest pass unchanged.
template <typename T>
__global__ void latent_norm_rope_append_kernel(const T* __restrict__ proj, int P, int q_rank, int kv_col, int kv_rank, int rot_dim,
                                               const float* __restrict__ qw, const float* __restrict__ kw, float eps,
                                               const float* __restrict__ cos_t, const float* __restrict__ sin_t, int rot_half,
                                               int table_len, const int* __restrict__ positions,
                                               const int* __restrict__ row_segment, const int* __restrict__ block_table,
                                               int table_stride, T* __restrict__ k_pages, int page_size, int write_kv,
                                               T* __restrict__ cq, int* __restrict__ err) {
    __shared__ float scratch[33];
    const int r = blockIdx.x;
    const int pos = positions[r];
    const int key_dim = kv_rank + rot_dim;
    T* dst = nullptr;
    if (write_kv) {
        const int page = block_table[(size_t)row_segment[r] * table_stride + pos / page_size];
        if (page < 0) {
            if (threadIdx.x == 0) atomicOr(err, KVB_DEV_BAD_PAGE);
        } else {
            dst = k_pages + ((size_t)page * page_size + (pos % page_size)) * key_dim;
        }
    }
    const bool pos_ok = pos >= 0 && pos < table_len;
    if (!pos_ok && threadIdx.x == 0) atomicOr(err, KVB_DEV_BAD_POS);
    const float* cr = cos_t + (size_t)(pos_ok ? pos : 0) * rot_half;
    const float* sr = sin_t + (size_t)(pos_ok ? pos : 0) * rot_half;
    pdl_wait();
    pdl_launch_dependents();
    const T* src = proj + (size_t)r * P;
    float sq = 0.f, sk = 0.f;
    for (int i = threadIdx.x; i < q_rank; i += blockDim.x) {
        const float v = to_f32<T>(src[i]);
        sq += v * v;
    }
    for (int i = threadIdx.x; i < kv_rank; i += blockDim.x) {
        const float v = to_f32<T>(src[kv_col + i]);
        sk += v * v;
    }
    const float qinv = q_rank > 0 ? 1.f / sqrtf(block_sum(sq, scratch) / (float)q_rank + eps) : 0.f;
    const float kinv = 1.f / sqrtf(block_sum(sk, scratch) / (float)kv_rank + eps);
    for (int i = threadIdx.x; i < q_rank; i += blockDim.x)
        cq[(size_t)r * q_rank + i] = from_f32<T>(to_f32<T>(src[i]) * qinv * qw[i]);
    if (!dst) return;
    for (int i = threadIdx.x; i < kv_rank; i += blockDim.x) dst[i] = from_f32<T>(to_f32<T>(src[kv_col + i]) * kinv * kw[i]);
    const T* kr = src + kv_col + kv_rank;
    for (int i = threadIdx.x; i < rot_dim; i += blockDim.x) {
        float x = to_f32<T>(kr[i]);
        if (i < 2 * rot_half) {
            const bool low = i < rot_half;
            const int t = low ? i : i - rot_half;
            const float xp = to_f32<T>(kr[low ? i + rot_half : i - rot_half]);
            x = low ? (x * cr[t] - xp * sr[t]) : (x * cr[t] + xp * sr[t]);
        }
        dst[kv_rank + i] = from_f32<T>(x);
    }
}

KVB_API int kvb_latent_norm_rope_append(int dtype, const void* proj, int P, int q_rank, int kv_col, int kv_rank, int rot_dim, const float* qw,
                                        const float* kw, float eps, const float* cos_t, const float* sin_t, int rot_half,
                                        int table_len, const int* positions, const int* row_segment, const int* block_table,
                                        int table_stride, void* k_pages, int page_size, int write_kv, void* cq, int T,
                                        int* err, cudaStream_t stream) {
    if (T <= 0) return KVB_OK;
    if (q_rank < 0 || kv_col < q_rank || kv_rank < 1 || rot_dim < 0 || 2 * rot_half > rot_dim || kv_col + kv_rank + rot_dim > P ||
        (q_rank > 0 && (qw == nullptr || cq == nullptr)))
        return KVB_ERR_SHAPE;
    const int threads = 128;
    if (dtype == KVB_F32)
        kvb_launch(latent_norm_rope_append_kernel<float>, dim3(T), dim3(threads), 0, stream, (const float*)proj, P, q_rank, kv_col, kv_rank,
                   rot_dim, qw, kw, eps, cos_t, sin_t, rot_half, table_len, positions, row_segment, block_table, table_stride,
                   (float*)k_pages, page_size, write_kv, (float*)cq, err);
    else if (dtype == KVB_BF16)
        kvb_launch(latent_norm_rope_append_kernel<bf16>, dim3(T), dim3(threads), 0, stream, (const bf16*)proj, P, q_rank, kv_col, kv_rank,
                   rot_dim, qw, kw, eps, cos_t, sin_t, rot_half, table_len, positions, row_segment, block_table, table_stride,
                   (bf16*)k_pages, page_size, write_kv, (bf16*)cq, err);
    else
        return KVB_ERR_DTYPE;
    return kvb_launch_status();
}

// ---------------------------------------------------------------------------------------------------------------
// out[t, h * os + n] = sum_k x[t, h * xs + k] * w[h, n, k]   (n < N, k < K), float32 accumulation on the CUDA cores:
// the form of the true 32-bit path and of shapes the tensor-core form refuses.  Tiles of BM x 64 outputs of one head,
// 16 of K at a time, K walked in the same order whatever T is.
//   gate:    out *= sigmoid(gate[t * gs + gc + h * os + n]), or, with `gate_heads`, sigmoid(gate[t * gs + gc + h]) (one number a head)
//   x_ld:    elements between rows of x (the heads' inputs may be columns of wider rows)
//   rot > 0: the head's trailing columns x[t, h * xs + K + i], i < rot, are rotated by the row's position (first
//            2 * rot_half of them; pair (i, i + rot_half)) and stored at out[t, h * os + N + i].
template <typename T, int BM>
__global__ void __launch_bounds__(256) head_linear_simt_kernel(const T* __restrict__ x, int xs, int x_ld, const T* __restrict__ w,
                                                               T* __restrict__ out, int os, int M, int N, int K, int H,
                                                               const T* __restrict__ gate, int gs, int gc, int gate_heads, int rot, int rot_half,
                                                               const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                                                               int table_len, const int* __restrict__ positions,
                                                               int* __restrict__ err) {
    pdl_wait();
    pdl_launch_dependents();
    constexpr int BN = 64, BK = 16, TM = BM / 16;
    __shared__ float xs_s[BK][BM + 4];
    __shared__ float ws_s[BK][BN + 4];
    const int tid = threadIdx.x;
    const int ty = tid / 16, tx = tid % 16;
    const int h = blockIdx.z;
    const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
    const size_t xrow = (size_t)x_ld, orow = (size_t)H * os;
    const T* xh = x + (size_t)h * xs;
    const T* wh = w + (size_t)h * N * K;

    float acc[TM][4];
#pragma unroll
    for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

    for (int k0 = 0; k0 < K; k0 += BK) {
        for (int e = tid; e < BM * BK; e += 256) {
            const int row = e / BK, kk = e % BK;
            const int gm = m0 + row;
            xs_s[kk][row] = (gm < M && k0 + kk < K) ? to_f32<T>(xh[(size_t)gm * xrow + k0 + kk]) : 0.f;
        }
        for (int e = tid; e < BN * BK; e += 256) {
            const int row = e / BK, kk = e % BK;
            const int gn = n0 + row;
            ws_s[kk][row] = (gn < N && k0 + kk < K) ? to_f32<T>(wh[(size_t)gn * K + k0 + kk]) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < BK; ++kk) {
            float a[TM], b[4];
#pragma unroll
            for (int i = 0; i < TM; ++i) a[i] = xs_s[kk][ty * TM + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) b[j] = ws_s[kk][tx * 4 + j];
#pragma unroll
            for (int i = 0; i < TM; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < TM; ++i) {
        const int gm = m0 + ty * TM + i;
        if (gm >= M) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int gn = n0 + tx * 4 + j;
            if (gn >= N) continue;
            float v = acc[i][j];
            if (gate) {
                const float g = to_f32<T>(gate[(size_t)gm * gs + gc + (gate_heads ? (size_t)h : (size_t)h * os + gn)]);
                v *= 1.f / (1.f + expf(-g));
            }
            out[(size_t)gm * orow + (size_t)h * os + gn] = from_f32<T>(v);
        }
    }
    if (rot > 0 && blockIdx.x == 0) {
        for (int e = tid; e < BM * rot; e += 256) {
            const int row = e / rot, i = e % rot;
            const int gm = m0 + row;
            if (gm >= M) continue;
            const int pos = positions[gm];
            const bool pos_ok = pos >= 0 && pos < table_len;
            if (!pos_ok) atomicOr(err, KVB_DEV_BAD_POS);
            const T* src = xh + (size_t)gm * xrow + K;
            float v = to_f32<T>(src[i]);
            if (i < 2 * rot_half && pos_ok) {
                const bool low = i < rot_half;
                const int t = low ? i : i - rot_half;
                const float vp = to_f32<T>(src[low ? i + rot_half : i - rot_half]);
                const float c = cos_t[(size_t)pos * rot_half + t], s = sin_t[(size_t)pos * rot_half + t];
                v = low ? (v * c - vp * s) : (v * c + vp * s);
            }
            out[(size_t)gm * orow + (size_t)h * os + N + i] = from_f32<T>(v);
        }
    }
}

// The same on the tensor cores (bfloat16; K, xs and the heads' offsets in steps of 8 elements, os even).
template <int MT>
__global__ void __launch_bounds__(mt::THREADS) head_linear_mma_kernel(const bf16* __restrict__ x, int xs, int x_ld, const bf16* __restrict__ w,
                                                                      bf16* __restrict__ out, int os, int M, int N, int K, int H,
                                                                      const bf16* __restrict__ gate, int gs, int gc, int gate_heads, int rot,
                                                                      int rot_half, const float* __restrict__ cos_t,
                                                                      const float* __restrict__ sin_t, int table_len,
                                                                      const int* __restrict__ positions, int* __restrict__ err) {
    pdl_wait();
    pdl_launch_dependents();
    constexpr int BM = 16 * MT;
    __shared__ __align__(16) mt::Smem<MT> sm;
    const int h = blockIdx.z, m0 = blockIdx.y * BM, n0 = blockIdx.x * mt::BN;
    const size_t xrow = (size_t)x_ld, orow = (size_t)H * os;
    const bf16* xh = x + (size_t)h * xs;
    auto a_row = [&](int r) -> const bf16* { return m0 + r < M ? xh + (size_t)(m0 + r) * xrow : nullptr; };
    auto store = [&](int r, int c, float v0, float v1) {
        const int gm = m0 + r, gn = n0 + c;
        if (gm >= M || gn >= N) return;
        bf16* dst = out + (size_t)gm * orow + (size_t)h * os + gn;
        if (gate && gate_heads) {
            const float s = 1.f / (1.f + expf(-__bfloat162float(gate[(size_t)gm * gs + gc + h])));
            v0 *= s;
            v1 *= s;
        } else if (gate) {
            const bf16* gp = gate + (size_t)gm * gs + gc + (size_t)h * os + gn;
            v0 *= 1.f / (1.f + expf(-__bfloat162float(gp[0])));
            if (gn + 1 < N) v1 *= 1.f / (1.f + expf(-__bfloat162float(gp[1])));
        }
        if (gn + 1 < N) *reinterpret_cast<__nv_bfloat162*>(dst) = __floats2bfloat162_rn(v0, v1);
        else dst[0] = __float2bfloat16_rn(v0);
    };
    mt::tile_product<MT>(sm, a_row, w + ((size_t)h * N + n0) * K, min(mt::BN, N - n0), K, store);
    if (rot > 0 && blockIdx.x == 0) {
        for (int e = threadIdx.x; e < BM * rot; e += mt::THREADS) {
            const int row = e / rot, i = e % rot;
            const int gm = m0 + row;
            if (gm >= M) continue;
            const int pos = positions[gm];
            const bool pos_ok = pos >= 0 && pos < table_len;
            if (!pos_ok) atomicOr(err, KVB_DEV_BAD_POS);
            const bf16* src = xh + (size_t)gm * xrow + K;
            float v = __bfloat162float(src[i]);
            if (i < 2 * rot_half && pos_ok) {
                const bool low = i < rot_half;
                const int t = low ? i : i - rot_half;
                const float vp = __bfloat162float(src[low ? i + rot_half : i - rot_half]);
                const float c = cos_t[(size_t)pos * rot_half + t], s = sin_t[(size_t)pos * rot_half + t];
                v = low ? (v * c - vp * s) : (v * c + vp * s);
            }
            out[(size_t)gm * orow + (size_t)h * os + N + i] = __float2bfloat16_rn(v);
        }
    }
}

template <typename T, int BM>
static void launch_head_linear(const T* x, int xs, int x_ld, const T* w, T* out, int os, int M, int N, int K, int H, const T* gate, int gs,
                               int gc, int gate_heads, int rot, int rot_half, const float* cos_t, const float* sin_t, int table_len,
                               const int* positions, int* err, cudaStream_t stream) {
    dim3 grid((N + 63) / 64, (M + BM - 1) / BM, H);
    kvb_launch(head_linear_simt_kernel<T, BM>, grid, dim3(256), 0, stream, x, xs, x_ld, w, out, os, M, N, K, H, gate, gs, gc, gate_heads, rot, rot_half,
               cos_t, sin_t, table_len, positions, err);
}

KVB_API int kvb_head_linear(int dtype, const void* x, int xs, int x_ld, const void* w, void* out, int os, int M, int N, int K, int H,
                            const void* gate, int gs, int gc, int gate_heads, int rot, int rot_half, const float* cos_t, const float* sin_t,
                            int table_len, const int* positions, int* err, cudaStream_t stream) {
    if (M <= 0 || H <= 0) return KVB_OK;
    if (N < 1 || K < 1 || xs < K + rot || os < N + rot || 2 * rot_half > rot || x_ld < H * xs) return KVB_ERR_SHAPE;
    if ((M + 15) / 16 > 65535 || H > 65535) return KVB_ERR_LIMIT;
#define KVB_HEAD_LINEAR(T, BM)                                                                                             \
    launch_head_linear<T, BM>((const T*)x, xs, x_ld, (const T*)w, (T*)out, os, M, N, K, H, (const T*)gate, gs, gc, gate_heads, rot, rot_half, cos_t, \
                              sin_t, table_len, positions, err, stream)
    if (dtype == KVB_F32) {
        if (M <= 16) KVB_HEAD_LINEAR(float, 16); else KVB_HEAD_LINEAR(float, 64);
    } else if (dtype == KVB_BF16) {
        const bool aligned = K % 8 == 0 && xs % 8 == 0 && x_ld % 8 == 0 && os % 2 == 0 && ((uintptr_t)x | (uintptr_t)w) % 16 == 0 &&
                             (uintptr_t)out % 4 == 0;
        if (aligned && getenv("KVB_HEAD_LINEAR_SIMT") == nullptr) {
            const bf16 *xb = (const bf16*)x, *wb = (const bf16*)w, *gb = (const bf16*)gate;
            if (M <= 16)
                kvb_launch(head_linear_mma_kernel<1>, dim3((N + 63) / 64, (M + 15) / 16, H), dim3(mt::THREADS), 0, stream, xb, xs, x_ld, wb,
                           (bf16*)out, os, M, N, K, H, gb, gs, gc, gate_heads, rot, rot_half, cos_t, sin_t, table_len, positions, err);
            else
                kvb_launch(head_linear_mma_kernel<4>, dim3((N + 63) / 64, (M + 63) / 64, H), dim3(mt::THREADS), 0, stream, xb, xs, x_ld, wb,
                           (bf16*)out, os, M, N, K, H, gb, gs, gc, gate_heads, rot, rot_half, cos_t, sin_t, table_len, positions, err);
        } else if (M <= 16) {
            KVB_HEAD_LINEAR(bf16, 16);
        } else {
            KVB_HEAD_LINEAR(bf16, 64);
        }
    } else {
        return KVB_ERR_DTYPE;
    }
#undef KVB_HEAD_LINEAR
    return kvb_launch_status();
}
