// Causal attention over cache pages for any mix of rows, any head size and either storage
// type: the kernel of the float32 path and the fallback of the bfloat16 one.
//
// One block per (row, query head).  The row's keys lo..pos (lo = 0, or pos - window + 1
// for a windowed layer) are visited in chunks of the block's width: each thread scores
// one key, the block takes the chunk's maximum and sum, and threads then own output
// dimensions for the weighted sum of values.  The running (max, sum, acc) update is the
// reference's online softmax (src/qwen_kernels.cu:159-176: m' = max(m, s), c = e^{m-m'},
// p = e^{s-m'}, l = l c + p, acc = acc c + p v; out = acc / l), the chunked form of it
// is the reference's two-pass block softmax (src/batched.cu:97-130).  kv_head = h / (Hq / Hkv)
// and scale applied after the dot product (src/qwen_kernels.cu:148-167).
// Chunk boundaries are counted from `lo`, so a row's summation order is the same however
// the step was cut.  `keep_first` (with a window): the request's first keys stay visible - the row then visits keys
// 0 .. min(keep_first, lo) - 1 and lo .. pos as one list.  `sink` (one logit per query head, or null): the softmax's
// denominator also holds exp(sink[h]), a key without a value; the running maximum and sum start from it.
// `cap` > 0: a score s (after the scale) becomes cap * tanh(s / cap).  `slopes` (one number per query head, or null): a
// key (pos - j) tokens back then loses slopes[h] * (pos - j).
#include "common.cuh"

#define ATTN_THREADS 128
#define ATTN_MAX_D 2048

template <typename T>
__global__ void paged_attention_generic_kernel(const T* __restrict__ q, const T* __restrict__ k_pages,
                                               const T* __restrict__ v_pages, const int* __restrict__ block_table,
                                               int table_stride, const int* __restrict__ positions,
                                               const int* __restrict__ row_segment, T* __restrict__ out, int Hq,
                                               int Hkv, int D, int Dv, int page_size, int window, int keep_first,
                                               const float* __restrict__ sink, float scale, float cap,
                                               const float* __restrict__ slopes, int* __restrict__ err) {
    pdl_wait();
    pdl_launch_dependents();
    extern __shared__ float smem[];
    float* q_s = smem;                    // [D]
    float* p_s = smem + D;                // [ATTN_THREADS]
    int* page_s = (int*)(p_s + ATTN_THREADS);  // [ATTN_THREADS] page offset of each key of the chunk
    float* scratch = (float*)(page_s + ATTN_THREADS);  // [33]

    const int r = blockIdx.x, h = blockIdx.y;
    const int hk = h / (Hq / Hkv);
    const int pos = positions[r];
    const int seg = row_segment[r];
    const int* table = block_table + (size_t)seg * table_stride;
    const int lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
    const int kept = min(keep_first, lo);          // keys before the window that stay visible
    const int visible = kept + pos - lo + 1;
    // Values as wide as the keys lie in a pool of their own; narrower ones (Dv < D) are the first Dv numbers of the key
    // rows themselves (a latent that serves as key and as value), and `v_pages` is then the key pool.
    const int v_stride = v_pages == k_pages ? D : Dv;

    const T* qr = q + ((size_t)r * Hq + h) * D;
    for (int d = threadIdx.x; d < D; d += blockDim.x) q_s[d] = to_f32<T>(qr[d]);
    __syncthreads();

    constexpr int DPT = ATTN_MAX_D / ATTN_THREADS;  // output dims per thread
    float acc[DPT];
#pragma unroll
    for (int i = 0; i < DPT; ++i) acc[i] = 0.f;
    float m = -FLT_MAX, l = 0.f;
    const float slope = slopes ? slopes[h] : 0.f;
    if (sink) {
        m = sink[h];
        l = 1.f;
    }

    for (int base = 0; base < visible; base += ATTN_THREADS) {
        const int i = base + threadIdx.x;
        const int j = i < kept ? i : lo + (i - kept);
        float s = -FLT_MAX;
        int off = -1;
        if (i < visible) {
            const int page = table[j / page_size];
            if (page < 0) {
                atomicOr(err, KVB_DEV_BAD_PAGE);
            } else {
                off = ((page * Hkv + hk) * page_size + (j % page_size));
                const T* kr = k_pages + (size_t)off * D;
                float dot = 0.f;
                for (int d = 0; d < D; ++d) dot += q_s[d] * to_f32<T>(kr[d]);
                s = dot * scale;
                if (cap > 0.f) s = cap * tanhf(s / cap);
                if (slopes) s -= slope * (float)(pos - j);
            }
        }
        const float cmax = block_max(s, scratch);
        const float m_new = fmaxf(m, cmax);
        const float corr = expf(m - m_new);
        const float p = (off >= 0) ? expf(s - m_new) : 0.f;
        p_s[threadIdx.x] = p;
        page_s[threadIdx.x] = off;
        const float csum = block_sum(p, scratch);   // also orders the writes to p_s / page_s
        l = l * corr + csum;
        m = m_new;
        const int n = min(ATTN_THREADS, visible - base);
#pragma unroll
        for (int i = 0; i < DPT; ++i) {
            const int d = threadIdx.x + i * ATTN_THREADS;
            if (d < Dv) {
                float a = acc[i] * corr;
                for (int t = 0; t < n; ++t) {
                    const int o = page_s[t];
                    if (o >= 0) a += p_s[t] * to_f32<T>(v_pages[(size_t)o * v_stride + d]);
                }
                acc[i] = a;
            }
        }
        __syncthreads();
    }
    T* orow = out + ((size_t)r * Hq + h) * Dv;
#pragma unroll
    for (int i = 0; i < DPT; ++i) {
        const int d = threadIdx.x + i * ATTN_THREADS;
        if (d < Dv) orow[d] = from_f32<T>(l > 0.f ? acc[i] / l : 0.f);
    }
}

KVB_API int kvb_paged_attention_generic(int dtype, const void* q, const void* k_pages, const void* v_pages,
                                        const int* block_table, int table_stride, const int* positions,
                                        const int* row_segment, void* out, int T, int Hq, int Hkv, int D,
                                        int page_size, int window, float scale, int* err, cudaStream_t stream);

// The same where a row's value is the first `Dv` numbers of its key row (one pool): out is [T, Hq * Dv].
KVB_API int kvb_paged_attention_shared(int dtype, const void* q, const void* k_pages, const int* block_table, int table_stride,
                                       const int* positions, const int* row_segment, void* out, int T, int Hq, int Hkv, int D,
                                       int Dv, int page_size, int window, float scale, int* err, cudaStream_t stream);

static int launch_generic(int dtype, const void* q, const void* k_pages, const void* v_pages, const int* block_table,
                          int table_stride, const int* positions, const int* row_segment, void* out, int T, int Hq, int Hkv,
                          int D, int Dv, int page_size, int window, float scale, int* err, cudaStream_t stream,
                          int keep_first = 0, const float* sink = nullptr, float cap = 0.f, const float* slopes = nullptr) {
    if (T <= 0) return KVB_OK;
    if (keep_first < 0) return KVB_ERR_SHAPE;
    if (window <= 0) keep_first = 0;
    if (D > ATTN_MAX_D || D < 1 || Dv < 1 || Dv > ATTN_MAX_D || (Dv > D && v_pages == k_pages) || Hkv < 1 || Hq % Hkv != 0)
        return KVB_ERR_SHAPE;
    const size_t smem = (size_t)(D + 2 * ATTN_THREADS + 33) * sizeof(float);
    dim3 grid(T, Hq);
    if (dtype == KVB_F32)
        kvb_launch(paged_attention_generic_kernel<float>, dim3(grid), dim3(ATTN_THREADS), smem, stream, 
            (const float*)q, (const float*)k_pages, (const float*)v_pages, block_table, table_stride, positions,
            row_segment, (float*)out, Hq, Hkv, D, Dv, page_size, window, keep_first, sink, scale, cap, slopes, err);
    else if (dtype == KVB_BF16)
        kvb_launch(paged_attention_generic_kernel<bf16>, dim3(grid), dim3(ATTN_THREADS), smem, stream, 
            (const bf16*)q, (const bf16*)k_pages, (const bf16*)v_pages, block_table, table_stride, positions,
            row_segment, (bf16*)out, Hq, Hkv, D, Dv, page_size, window, keep_first, sink, scale, cap, slopes, err);
    else
        return KVB_ERR_DTYPE;
    return kvb_launch_status();
}

KVB_API int kvb_paged_attention_generic(int dtype, const void* q, const void* k_pages, const void* v_pages,
                                        const int* block_table, int table_stride, const int* positions,
                                        const int* row_segment, void* out, int T, int Hq, int Hkv, int D,
                                        int page_size, int window, float scale, int* err, cudaStream_t stream) {
    if (v_pages == k_pages) return KVB_ERR_SHAPE;      // one pool for both is the other entry point's case
    return launch_generic(dtype, q, k_pages, v_pages, block_table, table_stride, positions, row_segment, out, T, Hq, Hkv, D, D,
                          page_size, window, scale, err, stream);
}

KVB_API int kvb_paged_attention_shared(int dtype, const void* q, const void* k_pages, const int* block_table, int table_stride,
                                       const int* positions, const int* row_segment, void* out, int T, int Hq, int Hkv, int D,
                                       int Dv, int page_size, int window, float scale, int* err, cudaStream_t stream) {
    return launch_generic(dtype, q, k_pages, k_pages, block_table, table_stride, positions, row_segment, out, T, Hq, Hkv, D, Dv,
                          page_size, window, scale, err, stream);
}

// Keys of D numbers and values of Dv numbers in pools of their own: out is [T, Hq * Dv].
KVB_API int kvb_paged_attention_kv(int dtype, const void* q, const void* k_pages, const void* v_pages, const int* block_table,
                                   int table_stride, const int* positions, const int* row_segment, void* out, int T, int Hq,
                                   int Hkv, int D, int Dv, int page_size, int window, float scale, int* err, cudaStream_t stream) {
    if (v_pages == k_pages) return KVB_ERR_SHAPE;
    return launch_generic(dtype, q, k_pages, v_pages, block_table, table_stride, positions, row_segment, out, T, Hq, Hkv, D, Dv,
                          page_size, window, scale, err, stream);
}

// Keys of D numbers and values of Dv numbers (pools of their own), a window that keeps the request's first `keep_first`
// keys visible, and a sink logit per query head in the softmax's denominator (`sink` null: none).
KVB_API int kvb_paged_attention_sink(int dtype, const void* q, const void* k_pages, const void* v_pages, const int* block_table,
                                     int table_stride, const int* positions, const int* row_segment, void* out, int T, int Hq,
                                     int Hkv, int D, int Dv, int page_size, int window, int keep_first, const float* sink,
                                     float scale, int* err, cudaStream_t stream) {
    if (v_pages == k_pages) return KVB_ERR_SHAPE;
    return launch_generic(dtype, q, k_pages, v_pages, block_table, table_stride, positions, row_segment, out, T, Hq, Hkv, D, Dv,
                          page_size, window, scale, err, stream, keep_first, sink);
}

// Every option at once.  `v_pages` null: a row's value is the first Dv numbers of its key row (one pool).  `window` is the
// caller's own (a layer may read a cache entry that keeps more than it sees).
KVB_API int kvb_paged_attention_ext(int dtype, const void* q, const void* k_pages, const void* v_pages, const int* block_table,
                                    int table_stride, const int* positions, const int* row_segment, void* out, int T, int Hq,
                                    int Hkv, int D, int Dv, int page_size, int window, int keep_first, const float* sink,
                                    float scale, float cap, const float* slopes, int* err, cudaStream_t stream) {
    if (cap < 0.f) return KVB_ERR_SHAPE;
    return launch_generic(dtype, q, k_pages, v_pages ? v_pages : k_pages, block_table, table_stride, positions, row_segment, out, T,
                          Hq, Hkv, D, Dv, page_size, window, scale, err, stream, keep_first, sink, cap, slopes);
}
