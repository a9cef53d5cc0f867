// Operators of mixers that carry a matrix per request and head from token to token, of gated heads, and of the
// hashed pair embedding.
//
//   matrix_state_scan   S_t = decay_t S_{t-1} + gain_t k_t v_t^T, o_t = S_t^T q_t over the tokens of every segment, from
//                       and into the request's state slot; two forms of decay (below)
//   head_norm_gate      out[t, h, :] = o[t, h, :] / rms(o[t, h, :]) * w * act(gate[t, h, :]) * scale
//   head_gate           out[t, h, :] = x[t, h, :] * sigmoid(gate[t, h]) * scale
//   bigram_embed        h[r] += table[(previous token * a + token * b) mod buckets], the table's last row at position 0;
//                       then the request's previous token becomes the last one of its segment
//
// The scan keeps everything in float32.  A lane owns one value channel (a column of S) of one head and keeps the
// column's key channels in registers for the whole segment (R of them; heads with more than 128 key channels split a
// column over KS = 2 neighbouring lanes), so a token costs a lane three multiply-adds per key channel - decay and add,
// read-out - and no exchange between lanes but the one that joins the parts of a split column.  The rows of 32 tokens at a
// time (q, k, the decays, the block's value channels) are staged in shared memory by the whole block and read from
// there as broadcasts; the exponential gates of those tokens are computed once for the block.  A column's sum over the
// key channels runs in one order whatever the step holds: a token's result is bit for bit the same in a prompt, a
// portion or alone.  State layout: [slot, head, key channel, value channel] (a warp's loads of a key channel's row coalesce).
//
// Long segments are cut into chunks of L tokens that run side by side, in three launches: (1) every chunk but a
// segment's last is scanned from an empty state and leaves its end state and its total decay in scratch; (2) per
// segment, the chunks' start states follow one from the other (start[c + 1] = decay[c] start[c] + local[c], for the
// exponential gates with their maxima: m' = max(F + m, m_local), weights e^{F + m - m'} and e^{m_local - m'}; for the
// delta rule, whose tokens mix the key channels, decay[c] is a matrix: launch (1) scans D more columns that start as the
// identity and take no k v^T, which leaves the product of the chunk's transitions); (3) every
// chunk is scanned again from its start state, now with read-outs, and a segment's last chunk leaves the state in the
// slot.  The arithmetic per token is the same as in one piece; the start states differ from it by float32 rounding.
#include "common.cuh"

enum { SCAN_CHANNEL_DECAY = 0, SCAN_EXP_GATES = 1, SCAN_DELTA_RULE = 2 };

__device__ __forceinline__ float log_sigmoid(float z) { return fminf(z, 0.f) - log1pf(expf(-fabsf(z))); }

// One float from global into shared memory without a register in between; many can be in flight per thread.
__device__ __forceinline__ void copy_async4(float* smem, const float* gmem) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;\n" ::"r"((uint32_t)__cvta_generic_to_shared(smem)), "l"(gmem));
}
__device__ __forceinline__ void copy_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
__device__ __forceinline__ void copy_async_wait_all() { asm volatile("cp.async.wait_group 0;\n" ::: "memory"); }

// Scratch of the chunked form; chunk ids count the chunks of all segments in the order of the segments.
struct ScanChunks {
    int L, S;              // tokens in a chunk; segments in the step
    float* local_S;        // [chunk, H, D, Dv]   end state of the chunk scanned from an empty state
    float* local_vec;      // [chunk, H, D]       channel decay: the product of the chunk's decays; exponential gates: its normaliser
    float* local_F;        // [chunk, H]          exponential gates: the sum of the chunk's log forget gates
    float* local_m;        // [chunk, H]          exponential gates: the chunk's maximum from an empty state
    float* start_S;        // [chunk, H, D, Dv]   state before the chunk's first token
    float* start_vec;      // [chunk, H, D]       exponential gates: the normaliser there
    float* start_m;        // [chunk, H]          exponential gates: the maximum there
    float* local_P;        // [chunk, H, D, D]    delta rule: the chunk's transition, the product of its tokens' diag(w) - (a u) u^T
};

// Which (segment, chunk of it) the chunk id is; false beyond the step's last chunk.
__device__ __forceinline__ bool find_chunk(int id, const ScanChunks& ch, const int* seg_q_len, int& seg, int& index, int& count) {
    int at = 0;
    for (int s = 0; s < ch.S; ++s) {
        const int nc = (seg_q_len[s] + ch.L - 1) / ch.L;
        if (id < at + nc) {
            seg = s; index = id - at; count = nc;
            return true;
        }
        at += nc;
    }
    return false;
}

enum { SCAN_LOCAL = 1, SCAN_FROM_START = 3 };
constexpr int SCAN_TILE = 32;          // tokens staged at a time
// Rows of key channels staged per token (q, k, then the mode's own), and the tokens staged at a time: the delta rule
// stages five rows a token and takes half the tokens, so that heads of 256 key channels still fit.
__host__ __device__ constexpr int scan_parts(int mode) { return mode == SCAN_CHANNEL_DECAY ? 3 : mode == SCAN_DELTA_RULE ? 5 : 2; }
__host__ __device__ constexpr int scan_tile(int mode) { return mode == SCAN_DELTA_RULE ? 16 : SCAN_TILE; }

// SCAN_CHANNEL_DECAY: decay per key channel d = sigmoid(z[r, h, d])^(1 / p0), gain 1; the launcher turns the logits z
//                     (`gate`, row stride gate_stride) into the decays in place before the scan, once for all warps.
// SCAN_EXP_GATES:     per head i = p0 tanh(gate[r, g0 + h] / p0), f = logsigmoid(p0 tanh(gate[r, g1 + h] / p0));
//                     m' = max(f + m, i); decay e^{f + m - m'}, gain e^{i - m'}; n' = decay n + gain k;
//                     o = S'^T q / (max(|n' . q|, e^{-m'}) + floor).  n: [slot, head, key channel], m: [slot, head].
// SCAN_DELTA_RULE:    S' = diag(w) S - (a u)(u^T S) + k v^T, both terms reading the old state: per key channel a decay w, the
//                     unit key u and the removal a u, staged from `gate` rows at g0 (w), g1 (u) and g1 + H * D (a u) - the
//                     launcher makes them from the projections before the scan.  A column first sums u . s over its key
//                     channels (joined over the KS parts of a split column), then updates them.  In SCAN_LOCAL columns
//                     Dv .. Dv + D - 1 carry the chunk's transition (see above) into ch.local_P.
// PASS: SCAN_LOCAL / SCAN_FROM_START - launches (1) and (3) of the chunked form; grid z counts chunks.  Segments in one
// piece are SCAN_FROM_START with chunks longer than any segment and no start states (`ch.start_S` null): from the slots.
// grid (column blocks, heads, segments or chunks); a warp holds 32 / KS columns.  The exponential-gate form takes one
// block per head: its n and m are kept by every warp (lane l: key channels l, l + 32, ...; the same arithmetic, the same
// bits), read at the start and written by the first warp at the end, with the loop's barriers in between.
template <int MODE, int R, int KS, int PASS>
__global__ void __launch_bounds__(512) matrix_state_scan_kernel(
    const float* __restrict__ proj, int P, int q_col, int k_col, int v_col, const float* __restrict__ gate, int gate_stride,
    int g0, int g1, float p0, float q_scale, float floor_, const int* __restrict__ seg_q_start,
    const int* __restrict__ seg_q_len, const int* __restrict__ seg_slot, float* __restrict__ memory,
    float* __restrict__ normalizer, float* __restrict__ maximum, float* __restrict__ out, int H, int D, int Dv, ScanChunks ch) {
    constexpr int RP = R + (KS > 1 ? 4 : 0);                   // a part's run in a staged row: 16 bytes of padding keep the parts' banks apart
    constexpr int RKP = RP * KS;                               // a staged row of key channels, zero beyond D
    constexpr int NPL = (R * KS + 31) / 32;                    // normaliser entries a lane keeps
    constexpr int COLS = 32 / KS;                              // columns of a warp
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
    const int h = blockIdx.y;
    const int part = lane % KS;                                // which run of R key channels of its column the lane holds
    const int VC = warps * COLS;                               // columns of the block
    const int col = blockIdx.x * VC + warp * COLS + lane / KS;
    constexpr bool WITH_TRANSITION = MODE == SCAN_DELTA_RULE && PASS == SCAN_LOCAL;
    const bool col_ok = col < (WITH_TRANSITION ? Dv + D : Dv);
    int seg = blockIdx.z, chunk = 0, chunks = 1;
    if (!find_chunk(blockIdx.z, ch, seg_q_len, seg, chunk, chunks)) return;
    const bool last_chunk = chunk == chunks - 1;
    if (PASS == SCAN_LOCAL && last_chunk) return;              // nobody starts from its end
    int r0 = seg_q_start[seg], n_rows = seg_q_len[seg];
    const int slot = seg_slot[seg];
    r0 += chunk * ch.L;
    n_rows = min(ch.L, n_rows - chunk * ch.L);
    pdl_wait();
    pdl_launch_dependents();
    __shared__ float gate_s[3][SCAN_TILE], max_s[SCAN_TILE + 1], carry_s[2];     // exponential gates: see the loop
    // Two staging buffers: while a tile of 32 tokens is computed, the next one's rows are already on their way
    // (asynchronous copies of 4 bytes: the rows' columns start anywhere).  q is staged as it is and the read-out is
    // multiplied by q_scale afterwards.  Key channels beyond D and value channels beyond Dv are zeroed once.
    extern __shared__ __align__(16) float tile_s[];
    constexpr int PARTS = scan_parts(MODE);
    constexpr int TILE = scan_tile(MODE);
    const int tile_floats = TILE * (PARTS * RKP + VC);
    auto at = [](int d) { return (d / R) * RP + d % R; };      // where key channel d lies in a staged row
    auto stage = [&](int which, int first_row, int rows) {
        float* q_b = tile_s + (size_t)which * tile_floats;
        float* k_b = q_b + TILE * RKP;
        float* a_b = k_b + TILE * RKP;
        float* u_b = a_b + TILE * RKP;                          // the delta rule's unit keys, then its removals
        float* v_b = q_b + TILE * PARTS * RKP;
        for (int idx = threadIdx.x; idx < rows * D; idx += blockDim.x) {
            const int row = idx / D, d = idx - row * D;
            const float* src = proj + (size_t)(first_row + row) * P;
            copy_async4(q_b + row * RKP + at(d), src + q_col + h * D + d);
            copy_async4(k_b + row * RKP + at(d), src + k_col + h * D + d);
            if (MODE != SCAN_EXP_GATES)
                copy_async4(a_b + row * RKP + at(d), gate + (size_t)(first_row + row) * gate_stride + g0 + h * D + d);
            if (MODE == SCAN_DELTA_RULE) {
                const float* grow = gate + (size_t)(first_row + row) * gate_stride + g1 + h * D + d;
                copy_async4(u_b + row * RKP + at(d), grow);
                copy_async4(u_b + (TILE + row) * RKP + at(d), grow + (size_t)H * D);
            }
        }
        const int v_cols = min(VC, Dv - (int)blockIdx.x * VC);
        for (int idx = threadIdx.x; idx < rows * v_cols; idx += blockDim.x) {
            const int row = idx / v_cols, c = idx - row * v_cols;
            copy_async4(v_b + row * VC + c, proj + (size_t)(first_row + row) * P + v_col + h * Dv + blockIdx.x * VC + c);
        }
        copy_async_commit();
    };
    for (int idx = threadIdx.x; idx < 2 * tile_floats; idx += blockDim.x) tile_s[idx] = 0.f;
    __syncthreads();
    if (n_rows > 0) stage(0, r0, min(TILE, n_rows));
    float S[R], nz[NPL], total[NPL];
    float* mem = memory + ((size_t)slot * H + h) * D * Dv;
    const size_t cid = (size_t)blockIdx.z * H + h;             // (chunk id, head) in the scratch arrays
    const bool from_slot = ch.start_S == nullptr;
    const float* from = from_slot ? mem : ch.start_S + cid * D * Dv;
#pragma unroll
    for (int i = 0; i < R; ++i) {
        const int d = part * R + i;
        S[i] = (PASS != SCAN_LOCAL && col_ok && d < D) ? from[(size_t)d * Dv + col] : 0.f;
        if (WITH_TRANSITION && d == col - Dv && d < D) S[i] = 1.f;     // no values are staged for these columns: their v is 0
    }
#pragma unroll
    for (int i = 0; i < NPL; ++i) total[i] = 1.f;
    if (MODE == SCAN_EXP_GATES) {
        const float* n_from = from_slot ? normalizer + ((size_t)slot * H + h) * D : ch.start_vec + cid * D;
#pragma unroll
        for (int i = 0; i < NPL; ++i) {
            const int d = lane + 32 * i;
            nz[i] = (PASS != SCAN_LOCAL && d < D) ? n_from[d] : 0.f;
        }
        if (threadIdx.x == 0) {
            // The running maximum, and the sum of the log forget gates.
            carry_s[0] = PASS == SCAN_LOCAL ? -FLT_MAX : from_slot ? maximum[(size_t)slot * H + h] : ch.start_m[cid];
            carry_s[1] = 0.f;
        }
        // Every warp has read n and m before the first may write them: the loop's first barrier comes before any write.
    }
#pragma unroll 1
    for (int t = 0; t < n_rows; ++t) {
        const int r = r0 + t, tt = t % TILE;
        if (tt == 0) {
            copy_async_wait_all();
            __syncthreads();                                   // this tile has landed, and the one before has been used up
            if (t + TILE < n_rows) stage(((t / TILE) + 1) & 1, r + TILE, min(TILE, n_rows - t - TILE));
            if (MODE == SCAN_EXP_GATES) {
                // The gates of the tile's tokens, once for the block: thread j takes token t + j's two logarithms, the
                // first thread walks the maximum through them, then thread j takes the token's three exponentials.
                const int j = threadIdx.x;
                float li = 0.f, lf = 0.f;
                if (j < SCAN_TILE && t + j < n_rows) {
                    const float* grow = gate + (size_t)(r + j) * gate_stride;
                    li = p0 * tanhf(grow[g0 + h] / p0);
                    lf = log_sigmoid(p0 * tanhf(grow[g1 + h] / p0));
                    gate_s[0][j] = lf;
                    gate_s[1][j] = li;
                }
                __syncthreads();
                if (j == 0) {
                    float mm = carry_s[0], ff = carry_s[1];
                    for (int u = 0; u < SCAN_TILE && t + u < n_rows; ++u) {
                        max_s[u] = mm;                               // the maximum before token t + u
                        mm = fmaxf(gate_s[0][u] + mm, gate_s[1][u]);
                        ff += gate_s[0][u];
                    }
                    max_s[SCAN_TILE] = mm;
                    carry_s[1] = ff;
                }
                __syncthreads();
                if (j < SCAN_TILE && t + j < n_rows) {
                    const float before = max_s[j], after = fmaxf(lf + before, li);
                    gate_s[0][j] = expf(lf + before - after);
                    gate_s[1][j] = expf(li - after);
                    gate_s[2][j] = expf(-after);
                }
                if (j == 0) carry_s[0] = max_s[SCAN_TILE];
            }
            __syncthreads();
        }
        const float* q_s = tile_s + (size_t)((t / TILE) & 1) * tile_floats;
        const float* k_s = q_s + TILE * RKP;
        const float* a_s = k_s + TILE * RKP;
        const float* v_s = q_s + TILE * PARTS * RKP;
        const float4* q4 = reinterpret_cast<const float4*>(q_s + tt * RKP + part * RP);
        const float4* k4 = reinterpret_cast<const float4*>(k_s + tt * RKP + part * RP);
        const float4* a4 = reinterpret_cast<const float4*>(a_s + tt * RKP + part * RP);
        const float v = v_s[tt * VC + warp * COLS + lane / KS];
        float keep = 1.f, gain = v, denom = 1.f;
        if (MODE == SCAN_EXP_GATES) {
            keep = gate_s[0][tt];
            const float take = gate_s[1][tt];
            gain = take * v;
            float dot = 0.f;
#pragma unroll
            for (int i = 0; i < NPL; ++i) {
                const int d = lane + 32 * i;
                if (d < D) {
                    nz[i] = keep * nz[i] + take * k_s[tt * RKP + at(d)];
                    dot += nz[i] * q_s[tt * RKP + at(d)];
                }
            }
            if (PASS != SCAN_LOCAL) denom = 1.f / (fmaxf(fabsf(warp_sum(dot) * q_scale), gate_s[2][tt]) + floor_);
        } else if (PASS == SCAN_LOCAL && blockIdx.x == 0 && warp == 0) {
#pragma unroll
            for (int i = 0; i < NPL; ++i) total[i] *= (lane + 32 * i < D) ? a_s[tt * RKP + at(lane + 32 * i)] : 1.f;
        }
        float o0 = 0.f, o1 = 0.f, o2 = 0.f, o3 = 0.f;          // four chains of multiply-adds instead of one of R
        const float4* b4 = a4;                                 // the delta rule's removals a u
        float read = 0.f;                                      // and u . s over the column's old state
        if (MODE == SCAN_DELTA_RULE) {
            const float4* u4 = reinterpret_cast<const float4*>(a_s + (TILE + tt) * RKP + part * RP);
            b4 = reinterpret_cast<const float4*>(a_s + (2 * TILE + tt) * RKP + part * RP);
#pragma unroll
            for (int i = 0; i < R; i += 4) {
                const float4 uu = u4[i >> 2];
                o0 = fmaf(uu.x, S[i], o0);
                o1 = fmaf(uu.y, S[i + 1], o1);
                o2 = fmaf(uu.z, S[i + 2], o2);
                o3 = fmaf(uu.w, S[i + 3], o3);
            }
            read = (o0 + o1) + (o2 + o3);
            if (KS >= 2) read += __shfl_xor_sync(0xffffffffu, read, 1);
            if (KS == 4) read += __shfl_xor_sync(0xffffffffu, read, 2);
            read = -read;
            o0 = o1 = o2 = o3 = 0.f;
        }
#pragma unroll
        for (int i = 0; i < R; i += 4) {
            const float4 kk = k4[i >> 2];
            float4 qq = make_float4(0.f, 0.f, 0.f, 0.f), aa = make_float4(keep, keep, keep, keep);
            if (PASS != SCAN_LOCAL) qq = q4[i >> 2];
            if (MODE != SCAN_EXP_GATES) aa = a4[i >> 2];
            if (MODE == SCAN_DELTA_RULE) {
                const float4 bb = b4[i >> 2];
                S[i] = fmaf(aa.x, S[i], fmaf(bb.x, read, kk.x * gain));
                S[i + 1] = fmaf(aa.y, S[i + 1], fmaf(bb.y, read, kk.y * gain));
                S[i + 2] = fmaf(aa.z, S[i + 2], fmaf(bb.z, read, kk.z * gain));
                S[i + 3] = fmaf(aa.w, S[i + 3], fmaf(bb.w, read, kk.w * gain));
            } else {
                S[i] = fmaf(aa.x, S[i], kk.x * gain);
                S[i + 1] = fmaf(aa.y, S[i + 1], kk.y * gain);
                S[i + 2] = fmaf(aa.z, S[i + 2], kk.z * gain);
                S[i + 3] = fmaf(aa.w, S[i + 3], kk.w * gain);
            }
            if (PASS != SCAN_LOCAL) {
                o0 = fmaf(S[i], qq.x, o0);
                o1 = fmaf(S[i + 1], qq.y, o1);
                o2 = fmaf(S[i + 2], qq.z, o2);
                o3 = fmaf(S[i + 3], qq.w, o3);
            }
        }
        if (PASS == SCAN_LOCAL) continue;                      // the state only
        float o = (o0 + o1) + (o2 + o3);
        if (KS >= 2) o += __shfl_xor_sync(0xffffffffu, o, 1);
        if (KS == 4) o += __shfl_xor_sync(0xffffffffu, o, 2);
        o *= q_scale;
        if (MODE == SCAN_EXP_GATES) o *= denom;
        if (part == 0 && col_ok) out[(size_t)r * H * Dv + h * Dv + col] = o;
    }
    if (n_rows <= 0) return;
    if (PASS == SCAN_FROM_START && !last_chunk) return;        // only a segment's last chunk leaves the state in the slot
    float* to = PASS == SCAN_LOCAL ? ch.local_S + cid * D * Dv : mem;
#pragma unroll
    for (int i = 0; i < R; ++i) {
        const int d = part * R + i;
        if (WITH_TRANSITION && col >= Dv) {
            if (col_ok && d < D) ch.local_P[(cid * D + d) * D + col - Dv] = S[i];
        } else if (col_ok && d < D) {
            to[(size_t)d * Dv + col] = S[i];
        }
    }
    if (blockIdx.x != 0 || warp != 0) return;
    if (MODE != SCAN_EXP_GATES) {
        if (PASS == SCAN_LOCAL && MODE == SCAN_CHANNEL_DECAY)
#pragma unroll
            for (int i = 0; i < NPL; ++i) {
                const int d = lane + 32 * i;
                if (d < D) ch.local_vec[cid * D + d] = total[i];
            }
        return;
    }
    float* n_to = PASS == SCAN_LOCAL ? ch.local_vec + cid * D : normalizer + ((size_t)slot * H + h) * D;
#pragma unroll
    for (int i = 0; i < NPL; ++i) {
        const int d = lane + 32 * i;
        if (d < D) n_to[d] = nz[i];
    }
    if (lane == 0) {                                           // thread 0: it wrote the carries itself
        if (PASS == SCAN_LOCAL) {
            ch.local_m[cid] = carry_s[0];
            ch.local_F[cid] = carry_s[1];
        } else {
            maximum[(size_t)slot * H + h] = carry_s[0];
        }
    }
}

// z -> sigmoid(z)^(1 / tau) = exp(logsigmoid(z) / tau), in place.
__global__ void channel_decay_kernel(float* __restrict__ z, size_t total, float tau) {
    pdl_wait();
    pdl_launch_dependents();
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x)
        z[i] = expf(log_sigmoid(z[i]) / tau);
}

// Launch (2) of the chunked form: a thread per element of a (segment, head)'s state walks the segment's chunks in order.
template <int MODE>
__global__ void scan_chunk_starts_kernel(const int* __restrict__ seg_q_len, const int* __restrict__ seg_slot,
                                         const float* __restrict__ memory, const float* __restrict__ normalizer,
                                         const float* __restrict__ maximum, int H, int D, int Dv, ScanChunks ch) {
    pdl_wait();
    pdl_launch_dependents();
    const int h = blockIdx.y, seg = blockIdx.z;
    int first = 0;
    for (int s = 0; s < seg; ++s) first += (seg_q_len[s] + ch.L - 1) / ch.L;
    const int chunks = (seg_q_len[seg] + ch.L - 1) / ch.L;
    if (chunks <= 0) return;
    const int slot = seg_slot[seg];
    const size_t per = (size_t)D * Dv;
    const float* mem = memory + ((size_t)slot * H + h) * per;
    for (size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x; e < per; e += (size_t)gridDim.x * blockDim.x) {
        const int d = (int)(e / Dv);
        float s = mem[e];
        float m = MODE == SCAN_EXP_GATES ? maximum[(size_t)slot * H + h] : 0.f;
        for (int c = 0; c < chunks; ++c) {
            const size_t cid = (size_t)(first + c) * H + h;
            ch.start_S[cid * per + e] = s;
            if (c + 1 == chunks) break;
            if (MODE == SCAN_CHANNEL_DECAY) {
                s = ch.local_vec[cid * D + d] * s + ch.local_S[cid * per + e];
            } else {
                const float F = ch.local_F[cid], ml = ch.local_m[cid];
                const float m1 = fmaxf(F + m, ml);
                s = expf(F + m - m1) * s + expf(ml - m1) * ch.local_S[cid * per + e];
                m = m1;
            }
        }
    }
    if (MODE == SCAN_EXP_GATES && blockIdx.x == 0)
        for (int d = threadIdx.x; d < D; d += blockDim.x) {
            float n = normalizer[((size_t)slot * H + h) * D + d];
            float m = maximum[(size_t)slot * H + h];
            for (int c = 0; c < chunks; ++c) {
                const size_t cid = (size_t)(first + c) * H + h;
                ch.start_vec[cid * D + d] = n;
                if (d == 0) ch.start_m[cid] = m;
                if (c + 1 == chunks) break;
                const float F = ch.local_F[cid], ml = ch.local_m[cid];
                const float m1 = fmaxf(F + m, ml);
                n = expf(F + m - m1) * n + expf(ml - m1) * ch.local_vec[cid * D + d];
                m = m1;
            }
        }
}

// Launch (2) for the delta rule: start[c + 1] = P[c] start[c] + local[c] - per chunk a product of the D x D transition with
// the D x Dv state, the chunks in order.  A block holds 32 columns of the state of one (segment, head) and all key
// channels; thread (ty, tx) of ceil(D / 4) x 8 holds rows 4 ty .. 4 ty + 3 and columns 4 tx .. 4 tx + 3 in registers.
// The P[c] pass through a ring of shared-memory stages, 32 of their columns at a time and transposed (so that a thread's
// four rows lie side by side); which tiles come does not depend on the states, so they are asked for three tiles ahead,
// and the next chunk's local state one chunk ahead.
constexpr int STARTS_STAGES = 4;
template <int N> __device__ __forceinline__ void copy_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N) : "memory"); }
__host__ __device__ constexpr int starts_row_stride(int D) { return (D + 3) / 4 * 4 + 4; }

__global__ void __launch_bounds__(512) delta_chunk_starts_kernel(const int* __restrict__ seg_q_len, const int* __restrict__ seg_slot,
                                                                 const float* __restrict__ memory, int H, int D, int Dv, ScanChunks ch) {
    pdl_wait();
    pdl_launch_dependents();
    extern __shared__ __align__(16) float starts_s[];
    const int DP = starts_row_stride(D);                       // a tile's row: P[.][j] for one j
    float* p_s = starts_s;                                     // [STARTS_STAGES][32][DP]
    float* col_s = starts_s + (size_t)STARTS_STAGES * 32 * DP; // [D][32]: the block's columns of start[c]
    const int h = blockIdx.y, seg = blockIdx.z;
    int first = 0;
    for (int s = 0; s < seg; ++s) first += (seg_q_len[s] + ch.L - 1) / ch.L;
    const int chunks = (seg_q_len[seg] + ch.L - 1) / ch.L;
    if (chunks <= 0) return;
    const int slot = seg_slot[seg];
    const size_t per = (size_t)D * Dv;
    const int tx = threadIdx.x & 7, ty = threadIdx.x >> 3;
    const int row0 = 4 * ty, col0 = blockIdx.x * 32 + 4 * tx;
    const bool rows_mine = row0 < D;
    const int tiles_per = (D + 31) / 32, total_tiles = (chunks - 1) * tiles_per;
    auto issue = [&](int q) {                                  // tile q of the walk into stage q % STARTS_STAGES
        if (q < total_tiles) {
            const int k = q / tiles_per, j0 = (q - k * tiles_per) * 32;
            const float* P = ch.local_P + ((size_t)(first + k) * H + h) * D * D + j0;
            float* dst = p_s + (size_t)(q % STARTS_STAGES) * 32 * DP;
            const int width = min(32, D - j0);
            const int j = threadIdx.x & 31;
            if (j < width)
                for (int row = threadIdx.x >> 5; row < D; row += blockDim.x >> 5) copy_async4(dst + j * DP + row, P + (size_t)row * D + j);
        }
        copy_async_commit();                                   // also when empty: the count of groups is what the waits go by
    };
    for (int q = 0; q < STARTS_STAGES - 1; ++q) issue(q);
    float s[4][4], local_next[4][4];
    auto fetch = [&](const float* from, float (&to)[4][4]) {
#pragma unroll
        for (int r = 0; r < 4; ++r)
#pragma unroll
            for (int cc = 0; cc < 4; ++cc)
                to[r][cc] = (from && row0 + r < D && col0 + cc < Dv) ? from[(size_t)(row0 + r) * Dv + col0 + cc] : 0.f;
    };
    fetch(memory + ((size_t)slot * H + h) * per, s);
    fetch(chunks > 1 ? ch.local_S + ((size_t)first * H + h) * per : nullptr, local_next);
    for (int k = 0; k < chunks; ++k) {
        const size_t cid = (size_t)(first + k) * H + h;
#pragma unroll
        for (int r = 0; r < 4; ++r)
#pragma unroll
            for (int cc = 0; cc < 4; ++cc)
                if (row0 + r < D && col0 + cc < Dv) ch.start_S[cid * per + (size_t)(row0 + r) * Dv + col0 + cc] = s[r][cc];
        if (k + 1 == chunks) break;
#pragma unroll
        for (int r = 0; r < 4; ++r)
            if (row0 + r < D) *reinterpret_cast<float4*>(col_s + (row0 + r) * 32 + 4 * tx) = make_float4(s[r][0], s[r][1], s[r][2], s[r][3]);
        float acc[4][4];
#pragma unroll
        for (int r = 0; r < 4; ++r)
#pragma unroll
            for (int cc = 0; cc < 4; ++cc) acc[r][cc] = local_next[r][cc];
        fetch(k + 2 < chunks ? ch.local_S + (cid + H) * per : nullptr, local_next);
        for (int jt = 0; jt < tiles_per; ++jt) {
            const int q = k * tiles_per + jt, j0 = jt * 32;
            copy_async_wait<STARTS_STAGES - 2>();              // this thread's share of tile q has landed
            __syncthreads();                                   // ... and everybody's; tile q - 1 has been used up; col_s is written
            issue(q + STARTS_STAGES - 1);                      // into the stage tile q - 1 had
            const float* tile = p_s + (size_t)(q % STARTS_STAGES) * 32 * DP + row0;
            const float* cols = col_s + j0 * 32 + 4 * tx;
            const int width = min(32, D - j0);
            auto step = [&](int j) {
                const float4 pv = *reinterpret_cast<const float4*>(tile + j * DP);
                const float4 sv = *reinterpret_cast<const float4*>(cols + j * 32);
                const float pr[4] = {pv.x, pv.y, pv.z, pv.w};
#pragma unroll
                for (int r = 0; r < 4; ++r) {
                    acc[r][0] = fmaf(pr[r], sv.x, acc[r][0]);
                    acc[r][1] = fmaf(pr[r], sv.y, acc[r][1]);
                    acc[r][2] = fmaf(pr[r], sv.z, acc[r][2]);
                    acc[r][3] = fmaf(pr[r], sv.w, acc[r][3]);
                }
            };
            if (rows_mine) {
                if (width == 32) {
#pragma unroll
                    for (int j = 0; j < 32; ++j) step(j);
                } else {
                    for (int j = 0; j < width; ++j) step(j);
                }
            }
        }
        __syncthreads();                                       // everybody has read col_s before it is written again
#pragma unroll
        for (int r = 0; r < 4; ++r)
#pragma unroll
            for (int cc = 0; cc < 4; ++cc) s[r][cc] = acc[r][cc];
    }
    copy_async_wait<0>();
}

template <int MODE, int R, int KS>
static int launch_scan(const float* proj, int P, int q_col, int k_col, int v_col, const float* gate, int gate_stride, int g0, int g1,
                        float p0, float q_scale, float floor_, const int* seg_q_start, const int* seg_q_len, const int* seg_slot,
                        float* memory, float* normalizer, float* maximum, float* out, int S, int H, int D, int Dv, ScanChunks ch,
                        int max_chunks, cudaStream_t stream) {
    constexpr int COLS = 32 / KS;
    constexpr int RKP = (R + (KS > 1 ? 4 : 0)) * KS;
    const int total_warps = (Dv + COLS - 1) / COLS;
    // The exponential-gate form: all of a head's columns in one block (the caller chose KS so that they are at most 16
    // warps).  The other: blocks of up to 16 warps, fewer where the staging buffers would not fit.
    int warps = MODE == SCAN_EXP_GATES ? total_warps : (total_warps < 16 ? total_warps : 16);
    auto bytes = [&](int w) { return 2 * (size_t)scan_tile(MODE) * (scan_parts(MODE) * RKP + w * COLS) * sizeof(float); };
    if (MODE != SCAN_EXP_GATES)
        while (warps > 1 && bytes(warps) > 200 * 1024) warps >>= 1;
    int col_blocks = (total_warps + warps - 1) / warps;
    const size_t smem = bytes(warps);
#define KVB_SCAN_PASS(PASS, Z)                                                                                                  \
    do {                                                                                                                        \
        if (smem + 2048 > 48 * 1024)                                                                                            \
            cudaFuncSetAttribute(matrix_state_scan_kernel<MODE, R, KS, PASS>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
        kvb_launch(matrix_state_scan_kernel<MODE, R, KS, PASS>, dim3(col_blocks, H, Z), dim3(32 * warps), smem, stream, proj, P,    \
                   q_col, k_col, v_col, gate, gate_stride, g0, g1, p0, q_scale, floor_, seg_q_start, seg_q_len, seg_slot, memory,    \
                   normalizer, maximum, out, H, D, Dv, ch);                                                                     \
    } while (0)
    if (smem > 220 * 1024 || warps > 16) return KVB_ERR_LIMIT;
    if (max_chunks <= 0) {
        ScanChunks whole = {};
        whole.L = 1 << 30;
        whole.S = S;
        ch = whole;
        KVB_SCAN_PASS(SCAN_FROM_START, S);
        return KVB_OK;
    }
    if constexpr (MODE == SCAN_DELTA_RULE) {
        const int state_blocks = col_blocks;
        col_blocks = ((Dv + D + COLS - 1) / COLS + warps - 1) / warps;     // the transition's columns beside the state's
        KVB_SCAN_PASS(SCAN_LOCAL, max_chunks);
        col_blocks = state_blocks;
        const int starts_threads = ((D + 3) / 4 * 8 + 31) / 32 * 32;
        if (starts_threads > 512) return KVB_ERR_LIMIT;
        const size_t starts_smem = (size_t)(STARTS_STAGES * 32 * starts_row_stride(D) + D * 32) * sizeof(float);
        if (starts_smem > 48 * 1024)
            cudaFuncSetAttribute(delta_chunk_starts_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)starts_smem);
        kvb_launch(delta_chunk_starts_kernel, dim3((Dv + 31) / 32, H, S), dim3(starts_threads), starts_smem, stream, seg_q_len, seg_slot,
                   (const float*)memory, H, D, Dv, ch);
        KVB_SCAN_PASS(SCAN_FROM_START, max_chunks);
        return KVB_OK;
    } else {
        KVB_SCAN_PASS(SCAN_LOCAL, max_chunks);
        kvb_launch(scan_chunk_starts_kernel<MODE>, dim3((D * Dv + 255) / 256, H, S), dim3(256), 0, stream, seg_q_len, seg_slot,
                   (const float*)memory, (const float*)normalizer, (const float*)maximum, H, D, Dv, ch);
        KVB_SCAN_PASS(SCAN_FROM_START, max_chunks);
        return KVB_OK;
    }
#undef KVB_SCAN_PASS
}

// proj: float32 [T, P] with q at q_col (H * D numbers), k at k_col, v at v_col (H * Dv).  `gate`: float32 rows of
// stride gate_stride - per-channel decay logits [T, H * D] (mode 0; overwritten by the decays), or the two gates'
// pre-activations at g0 and g1 (mode 1).  States: memory [slots, H, D, Dv], normalizer [slots, H, D], maximum [slots, H].
// `max_chunks` > 0: the chunked form with chunks of `chunk_len` tokens; `max_chunks` bounds the step's chunk count
// (sum over segments of ceil(len / chunk_len)) and `scratch` holds that many times H * (2 Dv D + 2 D + 3) floats, for the
// delta rule H * D * D more.
static int delta_rule_lanes = 0;       // lanes a column of the delta rule is spread over (0: as the other forms)
KVB_API int kvb_delta_rule_set_lanes(int lanes) {
    delta_rule_lanes = (lanes == 1 || lanes == 2 || lanes == 4) ? lanes : 0;
    return KVB_OK;
}

static int scan_any(int mode, const float* proj, int P, int q_col, int k_col, int v_col, const float* gate,
                    int gate_stride, int g0, int g1, float p0, float q_scale, float floor_, const int* seg_q_start,
                    const int* seg_q_len, const int* seg_slot, float* memory, float* normalizer, float* maximum,
                    float* out, int T, int S, int H, int D, int Dv, int chunk_len, int max_chunks, float* scratch,
                    cudaStream_t stream, bool decays_ready = false) {
    if (S <= 0) return KVB_OK;
    if (H < 1 || D < 1 || Dv < 1 || mode < SCAN_CHANNEL_DECAY || mode > SCAN_DELTA_RULE) return KVB_ERR_SHAPE;
    if (D > 256 || Dv > 512 || H > 65535 || S > 65535 || max_chunks > 65535) return KVB_ERR_LIMIT;
    if (max_chunks > 0 && (chunk_len < 1 || scratch == nullptr)) return KVB_ERR_SHAPE;
    ScanChunks ch = {};
    if (max_chunks > 0) {
        const size_t states = (size_t)max_chunks * H * Dv * D, vecs = (size_t)max_chunks * H * D, ones = (size_t)max_chunks * H;
        ch.L = chunk_len;
        ch.S = S;
        ch.local_S = scratch;
        ch.start_S = ch.local_S + states;
        ch.local_vec = ch.start_S + states;
        ch.start_vec = ch.local_vec + vecs;
        ch.local_F = ch.start_vec + vecs;
        ch.local_m = ch.local_F + ones;
        ch.start_m = ch.local_m + ones;
        ch.local_P = ch.start_m + ones;
    }
    if (mode == SCAN_CHANNEL_DECAY) {
        if (g0 != 0 || gate_stride != H * D) return KVB_ERR_SHAPE;       // the logits are rows of their own
        const size_t total = (size_t)T * H * D;
        size_t blocks = (total + 255) / 256;
        const size_t most = (size_t)kvb_sm_count() * 16;
        if (blocks > most) blocks = most;
        if (!decays_ready) kvb_launch(channel_decay_kernel, dim3((int)blocks), dim3(256), 0, stream, const_cast<float*>(gate), total, p0);
    }
    // A column's key channels over KS lanes, so that a lane holds at most 64 of them (measured at 128 key channels: 64 a
    // lane took 312 us where 128 took 489 and 32 took 475; at 64 key channels one lane a column 129 us, four 160);
    // fewer lanes where the exponential-gate form's block (all of a head's columns) would pass 16 warps.
    int ks = D <= 64 ? 1 : D <= 128 ? 2 : 4;
    if (mode == SCAN_DELTA_RULE && delta_rule_lanes > 0) ks = delta_rule_lanes;
    if (mode == SCAN_EXP_GATES)
        while (ks > 1 && (Dv + 32 / ks - 1) / (32 / ks) > 16) ks >>= 1;
    const int per_lane = (D + ks - 1) / ks;
    const int r = per_lane <= 16 ? 16 : per_lane <= 32 ? 32 : per_lane <= 64 ? 64 : 128;
    if (per_lane > 128) return KVB_ERR_LIMIT;
    int rc = KVB_ERR_LIMIT;
#define KVB_SCAN(MODE, R, KS)                                                                                                  \
    rc = launch_scan<MODE, R, KS>(proj, P, q_col, k_col, v_col, gate, gate_stride, g0, g1, p0, q_scale, floor_, seg_q_start,   \
                                  seg_q_len, seg_slot, memory, normalizer, maximum, out, S, H, D, Dv, ch, max_chunks, stream)
#define KVB_SCAN_KS(MODE, R)                                                                                                   \
    do {                                                                                                                      \
        if (ks == 4) KVB_SCAN(MODE, R, 4); else if (ks == 2) KVB_SCAN(MODE, R, 2); else KVB_SCAN(MODE, R, 1);                 \
    } while (0)
#define KVB_SCAN_SIZE(MODE)                                                                                                    \
    do {                                                                                                                      \
        if (r == 16) KVB_SCAN_KS(MODE, 16); else if (r == 32) KVB_SCAN_KS(MODE, 32);                                          \
        else if (r == 64) KVB_SCAN_KS(MODE, 64); else KVB_SCAN_KS(MODE, 128);                                                 \
    } while (0)
    if (mode == SCAN_CHANNEL_DECAY) KVB_SCAN_SIZE(SCAN_CHANNEL_DECAY);
    else if (mode == SCAN_EXP_GATES) KVB_SCAN_SIZE(SCAN_EXP_GATES);
    else KVB_SCAN_SIZE(SCAN_DELTA_RULE);
#undef KVB_SCAN_SIZE
#undef KVB_SCAN_KS
#undef KVB_SCAN
    if (rc != KVB_OK) return rc;
    return kvb_launch_status();
}

KVB_API int kvb_matrix_state_scan(int mode, const float* proj, int P, int q_col, int k_col, int v_col, const float* gate,
                                  int gate_stride, int g0, int g1, float p0, float q_scale, float floor_, const int* seg_q_start,
                                  const int* seg_q_len, const int* seg_slot, float* memory, float* normalizer, float* maximum,
                                  float* out, int T, int S, int H, int D, int Dv, int chunk_len, int max_chunks, float* scratch,
                                  cudaStream_t stream) {
    if (mode != SCAN_CHANNEL_DECAY && mode != SCAN_EXP_GATES) return KVB_ERR_SHAPE;
    return scan_any(mode, proj, P, q_col, k_col, v_col, gate, gate_stride, g0, g1, p0, q_scale, floor_, seg_q_start, seg_q_len,
                    seg_slot, memory, normalizer, maximum, out, T, S, H, D, Dv, chunk_len, max_chunks, scratch, stream);
}

// ---------------------------------------------------------------------------------------------------------------
// Lightning attention: one constant decay per head, and silu on the three projections.  One launch turns the float32 rows
// of the projection into what the channel-decay scan reads: q, k and v become silu(.) in place (columns q_col, k_col of
// H * D numbers and v_col of H * Dv), and decays[t, h * D + d] = decay[h] for the step's T rows.
__global__ void lightning_inputs_kernel(float* __restrict__ proj, int P, int q_col, int k_col, int v_col,
                                        const float* __restrict__ decay, float* __restrict__ decays, int H, int D, int Dv) {
    pdl_wait();
    pdl_launch_dependents();
    const int t = blockIdx.x;
    float* row = proj + (size_t)t * P;
    const int qk = H * D, hv = H * Dv;
    for (int i = threadIdx.x; i < 2 * qk + hv; i += blockDim.x) {
        float* at = i < qk ? row + q_col + i : i < 2 * qk ? row + k_col + (i - qk) : row + v_col + (i - 2 * qk);
        const float z = *at;
        *at = z / (1.f + expf(-z));
    }
    for (int i = threadIdx.x; i < qk; i += blockDim.x) decays[(size_t)t * qk + i] = decay[i / D];
}

// S = decay[h] S + k v^T, o = S^T q with q, k, v = silu of the projection's columns (overwritten by them); `decays`
// [T, H * D] float32 is scratch.  Prompts, portions and single tokens alike; long segments in chunks (see the top).
KVB_API int kvb_lightning_scan(float* proj, int P, int q_col, int k_col, int v_col, const float* decay, float* decays,
                               const int* seg_q_start, const int* seg_q_len, const int* seg_slot, float* memory, float* out, int T,
                               int S, int H, int D, int Dv, int chunk_len, int max_chunks, float* scratch, cudaStream_t stream) {
    if (S <= 0 || T <= 0) return KVB_OK;
    if (H < 1 || D < 1 || Dv < 1 || q_col < 0 || k_col < 0 || v_col < 0 || !decay || !decays) return KVB_ERR_SHAPE;
    kvb_launch(lightning_inputs_kernel, dim3(T), dim3(256), 0, stream, proj, P, q_col, k_col, v_col, decay, decays, H, D, Dv);
    return scan_any(SCAN_CHANNEL_DECAY, proj, P, q_col, k_col, v_col, decays, H * D, 0, 0, 1.f, 1.f, 0.f, seg_q_start, seg_q_len,
                    seg_slot, memory, nullptr, nullptr, out, T, S, H, D, Dv, chunk_len, max_chunks, scratch, stream, true);
}

// ---------------------------------------------------------------------------------------------------------------
// What the delta rule's recurrence reads besides r, k and v, per (token, head), all in float32: one warp each.
//   aux[t, 0 * HD + h D + d] = w  = exp(-rate * sigmoid(z[t, h D + d]))            decay of key channel d
//   aux[t, 1 * HD + h D + d] = u  = k / sqrt(sum_d k^2 + unit_eps)                 the head's unit key
//   aux[t, 2 * HD + h D + d] = a u, a = sigmoid(proj[t, a_col + h D + d])          what the state loses along u
__global__ void delta_rule_inputs_kernel(const float* __restrict__ proj, int P, int k_col, int a_col, const float* __restrict__ z,
                                         float rate, float unit_eps, float* __restrict__ aux, int pairs, int H, int D) {
    pdl_wait();
    pdl_launch_dependents();
    const int lane = threadIdx.x & 31;
    const int pair = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (pair >= pairs) return;
    const int t = pair / H, h = pair - t * H;
    const float* k = proj + (size_t)t * P + k_col + (size_t)h * D;
    const float* a = proj + (size_t)t * P + a_col + (size_t)h * D;
    const float* zr = z + (size_t)t * H * D + (size_t)h * D;
    float* dst = aux + (size_t)t * 3 * H * D + (size_t)h * D;
    float ss = 0.f;
    for (int d = lane; d < D; d += 32) ss += k[d] * k[d];
    const float inv = 1.f / sqrtf(warp_sum(ss) + unit_eps);
    for (int d = lane; d < D; d += 32) {
        const float u = k[d] * inv;
        dst[d] = expf(-rate / (1.f + expf(-zr[d])));
        dst[(size_t)H * D + d] = u;
        dst[(size_t)2 * H * D + d] = u / (1.f + expf(-a[d]));
    }
}

// The generalized delta rule over the tokens of every segment, from and into memory[slot] ([H, D, D], float32):
// S' = diag(w) S - (a u)(u^T S) + k v^T, out = S'^T r.  proj: float32 [T, P] with r, k, v and the removal logits at their
// columns (H * D numbers each); z: float32 [T, H * D], the decay logits; aux: float32 [T, 3 * H * D] of scratch.
// `max_chunks` > 0: the chunked form, as for the other scans, with `scratch` of max_chunks * H * (3 D D + 2 D + 3) floats.
KVB_API int kvb_delta_rule_scan(const float* proj, int P, int r_col, int k_col, int v_col, int a_col, const float* z, float rate,
                                float unit_eps, float* aux, const int* seg_q_start, const int* seg_q_len, const int* seg_slot,
                                float* memory, float* out, int T, int S, int H, int D, int chunk_len, int max_chunks, float* scratch,
                                cudaStream_t stream) {
    if (S <= 0 || T <= 0) return KVB_OK;
    if (H < 1 || D < 1 || aux == nullptr) return KVB_ERR_SHAPE;
    const int pairs = T * H, warps = 4;
    kvb_launch(delta_rule_inputs_kernel, dim3((pairs + warps - 1) / warps), dim3(32 * warps), 0, stream, proj, P, k_col, a_col, z, rate,
               unit_eps, aux, pairs, H, D);
    return scan_any(SCAN_DELTA_RULE, proj, P, r_col, k_col, v_col, aux, 3 * H * D, 0, H * D, 0.f, 1.f, 0.f, seg_q_start, seg_q_len,
                    seg_slot, memory, nullptr, nullptr, out, T, S, H, D, D, chunk_len, max_chunks, scratch, stream);
}

// ---------------------------------------------------------------------------------------------------------------
// One warp per (row, head).  o: float32 [T, H * Dv]; w: [Dv] (shared by the heads) or [H * Dv] (w_per_head);
// gate: float32 rows of stride gate_stride, the head's Dv numbers at gate_col + h * Dv; act 0: silu, 1: sigmoid.
// out (type T) rows of stride out_stride, written at out_col + h * Dv.
template <typename T>
__global__ void head_norm_gate_kernel(const float* __restrict__ o, const float* __restrict__ w, int w_per_head, float eps,
                                      const float* __restrict__ gate, int gate_stride, int gate_col, int act, float scale,
                                      T* __restrict__ out, int out_stride, int out_col, int pairs, int H, int Dv) {
    pdl_wait();
    pdl_launch_dependents();
    const int lane = threadIdx.x & 31;
    const int pair = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (pair >= pairs) return;
    const int t = pair / H, h = pair - t * H;
    const float* src = o + (size_t)t * H * Dv + (size_t)h * Dv;
    float ss = 0.f;
    for (int d = lane; d < Dv; d += 32) ss += src[d] * src[d];
    const float inv = 1.f / sqrtf(warp_sum(ss) / (float)Dv + eps);
    const float* g = gate + (size_t)t * gate_stride + gate_col + h * Dv;
    const float* wh = w + (w_per_head ? h * Dv : 0);
    T* dst = out + (size_t)t * out_stride + out_col + h * Dv;
    for (int d = lane; d < Dv; d += 32) {
        const float z = g[d];
        const float s = 1.f / (1.f + expf(-z));
        dst[d] = from_f32<T>(src[d] * inv * wh[d] * (act == 0 ? z * s : s) * scale);
    }
}

// The same with one root mean square over all of a row's heads (H * Dv numbers, a weight for each): a block per row.
template <typename T>
__global__ void row_norm_gate_kernel(const float* __restrict__ o, const float* __restrict__ w, float eps,
                                     const float* __restrict__ gate, int gate_stride, int gate_col, int act, float scale,
                                     T* __restrict__ out, int out_stride, int out_col, int W) {
    pdl_wait();
    pdl_launch_dependents();
    __shared__ float scratch[33];
    const int t = blockIdx.x;
    const float* src = o + (size_t)t * W;
    float ss = 0.f;
    for (int i = threadIdx.x; i < W; i += blockDim.x) ss += src[i] * src[i];
    const float inv = 1.f / sqrtf(block_sum(ss, scratch) / (float)W + eps);
    const float* g = gate + (size_t)t * gate_stride + gate_col;
    T* dst = out + (size_t)t * out_stride + out_col;
    for (int i = threadIdx.x; i < W; i += blockDim.x) {
        const float z = g[i];
        const float s = 1.f / (1.f + expf(-z));
        dst[i] = from_f32<T>(src[i] * inv * w[i] * (act == 0 ? z * s : s) * scale);
    }
}

// `w_per_head` 2: the root mean square runs over all H * Dv numbers of a row at once, and `w` has that many.
KVB_API int kvb_head_norm_gate(int out_dtype, const float* o, const float* w, int w_per_head, float eps, const float* gate,
                               int gate_stride, int gate_col, int act, float scale, void* out, int out_stride, int out_col,
                               int T, int H, int Dv, cudaStream_t stream) {
    if (T <= 0) return KVB_OK;
    if (H < 1 || Dv < 1 || act < 0 || act > 1 || w_per_head < 0 || w_per_head > 2) return KVB_ERR_SHAPE;
    if (w_per_head == 2) {
        const int W = H * Dv, threads = W >= 2048 ? 512 : W >= 512 ? 256 : 128;
        if (out_dtype == KVB_F32)
            kvb_launch(row_norm_gate_kernel<float>, dim3(T), dim3(threads), 0, stream, o, w, eps, gate, gate_stride, gate_col, act, scale,
                       (float*)out, out_stride, out_col, W);
        else if (out_dtype == KVB_BF16)
            kvb_launch(row_norm_gate_kernel<bf16>, dim3(T), dim3(threads), 0, stream, o, w, eps, gate, gate_stride, gate_col, act, scale,
                       (bf16*)out, out_stride, out_col, W);
        else
            return KVB_ERR_DTYPE;
        return kvb_launch_status();
    }
    const int pairs = T * H, warps = 4;
    dim3 grid((pairs + warps - 1) / warps), block(32 * warps);
    if (out_dtype == KVB_F32)
        kvb_launch(head_norm_gate_kernel<float>, grid, block, 0, stream, o, w, w_per_head, eps, gate, gate_stride, gate_col, act, scale,
                   (float*)out, out_stride, out_col, pairs, H, Dv);
    else if (out_dtype == KVB_BF16)
        kvb_launch(head_norm_gate_kernel<bf16>, grid, block, 0, stream, o, w, w_per_head, eps, gate, gate_stride, gate_col, act, scale,
                   (bf16*)out, out_stride, out_col, pairs, H, Dv);
    else
        return KVB_ERR_DTYPE;
    return kvb_launch_status();
}

// out[t, out_col + h * Dv + d] = x[t, h * xs + d] * sigmoid(gate[t, gate_col + h]) * scale (gate null: no sigmoid); xs >= Dv:
// a head of x may carry columns after its Dv numbers, which are left out.
template <typename T>
__global__ void head_gate_kernel(const T* __restrict__ x, int xs, const T* __restrict__ gate, int gate_stride, int gate_col, float scale,
                                 T* __restrict__ out, int out_stride, int out_col, int H, int Dv, size_t total) {
    pdl_wait();
    pdl_launch_dependents();
    const int width = H * Dv;
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x) {
        const size_t t = idx / width;
        const int c = (int)(idx - t * width);
        float v = to_f32<T>(x[(t * H + c / Dv) * xs + c % Dv]) * scale;
        if (gate) v *= 1.f / (1.f + expf(-to_f32<T>(gate[t * gate_stride + gate_col + c / Dv])));
        out[t * out_stride + out_col + c] = from_f32<T>(v);
    }
}

KVB_API int kvb_head_gate(int dtype, const void* x, int xs, const void* gate, int gate_stride, int gate_col, float scale, void* out,
                          int out_stride, int out_col, int T, int H, int Dv, cudaStream_t stream) {
    const size_t total = (size_t)T * H * Dv;
    if (total == 0) return KVB_OK;
    if (xs < Dv) return KVB_ERR_SHAPE;
    size_t blocks = (total + 255) / 256;
    const size_t most = (size_t)kvb_sm_count() * 16;
    if (blocks > most) blocks = most;
    if (dtype == KVB_F32)
        kvb_launch(head_gate_kernel<float>, dim3((int)blocks), dim3(256), 0, stream, (const float*)x, xs, (const float*)gate, gate_stride,
                   gate_col, scale, (float*)out, out_stride, out_col, H, Dv, total);
    else if (dtype == KVB_BF16)
        kvb_launch(head_gate_kernel<bf16>, dim3((int)blocks), dim3(256), 0, stream, (const bf16*)x, xs, (const bf16*)gate, gate_stride,
                   gate_col, scale, (bf16*)out, out_stride, out_col, H, Dv, total);
    else
        return KVB_ERR_DTYPE;
    return kvb_launch_status();
}

// ---------------------------------------------------------------------------------------------------------------
__device__ __forceinline__ int token_of(const int* ids, const int* src, const int* last, int r) {
    const int from = src ? src[r] : -1;
    return from >= 0 ? last[from] : ids[r];
}

// One block per row.  A token outside the vocabulary adds nothing (the embedding kernel has flagged it).
template <typename T>
__global__ void bigram_embed_kernel(const T* __restrict__ table, const int* __restrict__ ids, const int* __restrict__ src,
                                    const int* __restrict__ last, const int* __restrict__ positions,
                                    const int* __restrict__ row_segment, const int* __restrict__ seg_q_start,
                                    const int* __restrict__ seg_slot, const int* __restrict__ previous, float* __restrict__ h,
                                    int W, int buckets, int mul_prev, int mul_cur, int V) {
    pdl_wait();
    pdl_launch_dependents();
    const int r = blockIdx.x;
    const int tok = token_of(ids, src, last, r);
    if (tok < 0 || tok >= V) return;
    int row = buckets;
    if (positions[r] > 0) {
        const int seg = row_segment[r];
        const int before = r > seg_q_start[seg] ? token_of(ids, src, last, r - 1) : previous[seg_slot[seg]];
        row = (int)(((long long)before * mul_prev + (long long)tok * mul_cur) % buckets);
        if (row < 0) row += buckets;
    }
    const T* add = table + (size_t)row * W;
    float* dst = h + (size_t)r * W;
    for (int i = threadIdx.x; i < W; i += blockDim.x) dst[i] += to_f32<T>(add[i]);
}

__global__ void previous_token_kernel(const int* __restrict__ ids, const int* __restrict__ src, const int* __restrict__ last,
                                      const int* __restrict__ seg_q_start, const int* __restrict__ seg_q_len,
                                      const int* __restrict__ seg_slot, int* __restrict__ previous, int S) {
    pdl_wait();
    pdl_launch_dependents();
    const int s = blockIdx.x * blockDim.x + threadIdx.x;
    if (s < S && seg_q_len[s] > 0) previous[seg_slot[s]] = token_of(ids, src, last, seg_q_start[s] + seg_q_len[s] - 1);
}

KVB_API int kvb_bigram_embed(int dtype, const void* table, const int* ids, const int* src, const int* last, const int* positions,
                             const int* row_segment, const int* seg_q_start, const int* seg_q_len, const int* seg_slot,
                             int* previous, float* h, int T, int S, int W, int buckets, int mul_prev, int mul_cur, int V,
                             cudaStream_t stream) {
    if (T <= 0) return KVB_OK;
    if (buckets < 1 || W < 1) return KVB_ERR_SHAPE;
    const int threads = W >= 512 ? 256 : 128;
    if (dtype == KVB_F32)
        kvb_launch(bigram_embed_kernel<float>, dim3(T), dim3(threads), 0, stream, (const float*)table, ids, src, last, positions,
                   row_segment, seg_q_start, seg_slot, previous, h, W, buckets, mul_prev, mul_cur, V);
    else if (dtype == KVB_BF16)
        kvb_launch(bigram_embed_kernel<bf16>, dim3(T), dim3(threads), 0, stream, (const bf16*)table, ids, src, last, positions,
                   row_segment, seg_q_start, seg_slot, previous, h, W, buckets, mul_prev, mul_cur, V);
    else
        return KVB_ERR_DTYPE;
    int status = kvb_launch_status();
    if (status != KVB_OK) return status;
    kvb_launch(previous_token_kernel, dim3((S + 127) / 128), dim3(128), 0, stream, ids, src, last, seg_q_start, seg_q_len, seg_slot,
               previous, S);
    return kvb_launch_status();
}
