// Attention whose weights are not normalised over the keys: a visible key j gets
//     g_j = sigmoid((q . k_j) * scale + bias[head]),      o = sum_j g_j v_j,
// and which keys are visible is bounded by a chunk (query i sees j <= i with floor(j / chunk) =
// floor(i / chunk), chunks counted from the sequence's position 0) and, optionally, a window.
// Keys and values live in the paged cache; a value row may be narrower or wider than a key row.
//
// Before it: the preparation of the projected rows [q | k | v]: per head an RMS norm of q and of k with
// a weight vector shared by the heads, the rotation of the first rot_dims coordinates (i with
// i + rot_dims / 2, float32 tables), q written back in place, k and v into the cache.
#include "common.cuh"
#include <math.h>

typedef __nv_bfloat16 bf16;

// ---------------------------------------------------------------------------------------
// one block per (token, head of [q heads | k heads | v heads])
// ---------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(128)
qk_norm_rope_append_kernel(T* __restrict__ qkv, int ld, const float* __restrict__ q_w, const float* __restrict__ k_w,
                           float eps, const float* __restrict__ cos_t, const float* __restrict__ sin_t,
                           int table_positions, const int* __restrict__ pos, const int* __restrict__ slot,
                           const int* __restrict__ page_table, int max_pages, T* __restrict__ k_cache,
                           T* __restrict__ v_cache, int n_q, int n_kv, int dim, int vdim, int rot_dims,
                           int page_shift, int write_cache) {
    __shared__ float row[1024];
    __shared__ float red[128];
    ssb_pdl_launch_dependents();
    ssb_pdl_wait();
    const int t = blockIdx.x, hh = blockIdx.y, tid = threadIdx.x;
    const int s = slot[t];
    if (s < 0) return;
    const int p = pos[t];
    T* base = qkv + (size_t)t * ld;
    if (hh >= n_q + n_kv) {                               // a value head: a copy into the cache
        if (!write_cache) return;
        const int kvh = hh - n_q - n_kv;
        const T* src = base + (size_t)(n_q + n_kv) * dim + (size_t)kvh * vdim;
        T* dst = v_cache + ssb_cache_row(page_table, max_pages, s, p, page_shift, n_kv, kvh, vdim);
        for (int c = tid; c < vdim; c += 128) dst[c] = src[c];
        return;
    }
    const bool is_q = hh < n_q;
    if (!is_q && !write_cache) return;
    T* src = base + (size_t)hh * dim;
    const float* w = is_q ? q_w : k_w;
    float part = 0.f;
    for (int c = tid; c < dim; c += 128) {
        const float v = ssb_to_float(src[c]);
        row[c] = v;
        part = fmaf(v, v, part);
    }
    red[tid] = part;
    __syncthreads();
    for (int st = 64; st > 0; st >>= 1) {
        if (tid < st) red[tid] += red[tid + st];
        __syncthreads();
    }
    const float inv = w != nullptr ? 1.0f / sqrtf(red[0] / (float)dim + eps) : 1.0f;
    T* dst = is_q ? src : k_cache + ssb_cache_row(page_table, max_pages, s, p, page_shift, n_kv, hh - n_q, dim);
    const int half = rot_dims / 2;
    const bool turn = cos_t != nullptr && p < table_positions;
    for (int c = tid; c < dim; c += 128) {
        float v = row[c] * inv * (w ? w[c] : 1.0f);
        if (turn && c < rot_dims) {
            const int i = c < half ? c : c - half;
            const int other = c < half ? c + half : c - half;
            const float o = row[other] * inv * (w ? w[other] : 1.0f);
            const float cs = cos_t[(size_t)p * half + i], sn = sin_t[(size_t)p * half + i];
            v = c < half ? v * cs - o * sn : v * cs + o * sn;
        }
        dst[c] = ssb_from_float<T>(v);
    }
}

SSB_API int ssb_qk_norm_rope_append(void* qkv, int ld, int dtype, const float* q_w, const float* k_w, float eps,
                                    const float* cos_t, const float* sin_t, int table_positions, const int* pos,
                                    const int* slot, const int* page_table, int max_pages, void* k_cache,
                                    void* v_cache, int n_tokens, int n_q, int n_kv, int dim, int vdim, int rot_dims,
                                    int page_shift, int write_cache, int pdl, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (dim <= 0 || dim > 1024 || vdim <= 0 || rot_dims < 0 || rot_dims > dim || rot_dims % 2 || n_q + 2 * n_kv > 65535)
        return SSB_ERR_BAD_SIZE;
    const dim3 grid(n_tokens, n_q + 2 * n_kv);
    int rc;
    if (dtype == SSB_F32)
        rc = ssb_launch(qk_norm_rope_append_kernel<float>, grid, dim3(128), 0, stream, pdl != 0, (float*)qkv, ld, q_w, k_w, eps,
                        cos_t, sin_t, table_positions, pos, slot, page_table, max_pages, (float*)k_cache, (float*)v_cache,
                        n_q, n_kv, dim, vdim, rot_dims, page_shift, write_cache);
    else if (dtype == SSB_BF16)
        rc = ssb_launch(qk_norm_rope_append_kernel<bf16>, grid, dim3(128), 0, stream, pdl != 0, (bf16*)qkv, ld, q_w, k_w, eps,
                        cos_t, sin_t, table_positions, pos, slot, page_table, max_pages, (bf16*)k_cache, (bf16*)v_cache,
                        n_q, n_kv, dim, vdim, rot_dims, page_shift, write_cache);
    else
        return SSB_ERR_BAD_DTYPE;
    return rc ? rc : ssb_launch_status();
}

// ---------------------------------------------------------------------------------------
// The plain kernel: one block per (token, query head); a thread per key for the scores, a thread per
// value column for the sum; float32 throughout, keys in rising order.
// ---------------------------------------------------------------------------------------
constexpr int GA_THREADS = 128;
constexpr int GA_MAX_DIM = 1024;

template <typename T>
__global__ void __launch_bounds__(GA_THREADS)
sigmoid_attention_plain_kernel(const T* __restrict__ q, int ldq, const T* __restrict__ k_cache,
                               const T* __restrict__ v_cache, const int* __restrict__ pos, const int* __restrict__ slot,
                               const int* __restrict__ page_table, int max_pages, const float* __restrict__ bias,
                               T* __restrict__ out, int ldo, int n_q, int n_kv, int dim, int vdim, int page_shift,
                               int chunk, int window, float scale) {
    __shared__ float q_s[GA_MAX_DIM];
    __shared__ float g_s[GA_THREADS];
    ssb_pdl_launch_dependents();
    ssb_pdl_wait();
    const int t = blockIdx.x, h = blockIdx.y, tid = threadIdx.x;
    T* o = out + (size_t)t * ldo + (size_t)h * vdim;
    const int s = slot[t];
    if (s < 0) return;
    const int p = pos[t];
    int lo = chunk > 0 ? (p / chunk) * chunk : 0;
    if (window > 0) lo = max(lo, p - window + 1);
    const int kvh = h / (n_q / n_kv);
    const T* qp = q + (size_t)t * ldq + (size_t)h * dim;
    for (int d = tid; d < dim; d += GA_THREADS) q_s[d] = ssb_to_float(qp[d]);
    const float hb = bias ? bias[h] : 0.f;
    float acc[GA_MAX_DIM / GA_THREADS];
#pragma unroll
    for (int i = 0; i < GA_MAX_DIM / GA_THREADS; ++i) acc[i] = 0.f;
    __syncthreads();
    for (int base = lo; base <= p; base += GA_THREADS) {
        const int j = base + tid;
        float g = 0.f;
        if (j <= p) {
            const T* kr = k_cache + ssb_cache_row(page_table, max_pages, s, j, page_shift, n_kv, kvh, dim);
            float dot = 0.f;
            for (int d = 0; d < dim; ++d) dot = fmaf(q_s[d], ssb_to_float(kr[d]), dot);
            g = 1.0f / (1.0f + expf(-(dot * scale + hb)));
        }
        g_s[tid] = g;
        __syncthreads();
        const int n_in = min(GA_THREADS, p - base + 1);
#pragma unroll
        for (int i = 0; i < GA_MAX_DIM / GA_THREADS; ++i) {
            const int d = tid + i * GA_THREADS;
            if (d < vdim) {
                float a = acc[i];
                for (int jj = 0; jj < n_in; ++jj) {
                    const T* vr = v_cache + ssb_cache_row(page_table, max_pages, s, base + jj, page_shift, n_kv, kvh, vdim);
                    a = fmaf(g_s[jj], ssb_to_float(vr[d]), a);
                }
                acc[i] = a;
            }
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < GA_MAX_DIM / GA_THREADS; ++i) {
        const int d = tid + i * GA_THREADS;
        if (d < vdim) o[d] = ssb_from_float<T>(acc[i]);
    }
}

SSB_API int ssb_sigmoid_attention_plain(const void* q, int ldq, int dtype, const void* k_cache, const void* v_cache,
                                        const int* pos, const int* slot, const int* page_table, int max_pages,
                                        const float* bias, void* out, int ldo, int n_tokens, int n_q, int n_kv, int dim,
                                        int vdim, int page_shift, int chunk, int window, float scale, int pdl,
                                        cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (dim <= 0 || dim > GA_MAX_DIM || vdim <= 0 || vdim > GA_MAX_DIM || n_kv <= 0 || n_q % n_kv || n_q > 65535 ||
        chunk < 0 || window < 0)
        return SSB_ERR_BAD_SIZE;
    const dim3 grid(n_tokens, n_q);
    int rc;
    if (dtype == SSB_F32)
        rc = ssb_launch(sigmoid_attention_plain_kernel<float>, grid, dim3(GA_THREADS), 0, stream, pdl != 0, (const float*)q,
                        ldq, (const float*)k_cache, (const float*)v_cache, pos, slot, page_table, max_pages, bias,
                        (float*)out, ldo, n_q, n_kv, dim, vdim, page_shift, chunk, window, scale);
    else if (dtype == SSB_BF16)
        rc = ssb_launch(sigmoid_attention_plain_kernel<bf16>, grid, dim3(GA_THREADS), 0, stream, pdl != 0, (const bf16*)q,
                        ldq, (const bf16*)k_cache, (const bf16*)v_cache, pos, slot, page_table, max_pages, bias,
                        (bf16*)out, ldo, n_q, n_kv, dim, vdim, page_shift, chunk, window, scale);
    else
        return SSB_ERR_BAD_DTYPE;
    return rc ? rc : ssb_launch_status();
}

// ---------------------------------------------------------------------------------------
// The tensor-core kernel (mma.sync m16n8k16, bfloat16 operands, float32 sums).
//
// A block takes one sequence, one kv head and a tile of query rows; a row is a (new token, query head of
// the kv head's group) pair, heads fastest, so that the heads that share a kv head share its pages.  The
// sequence's pages from the first row's chunk start to the last row's position are streamed once through a
// two-stage cp.async ring (a page holds 64 keys of the kv head, contiguous).  Per page a warp takes
// S = Q K^T for its rows, turns it into weights in float32 (scale, head offset, sigmoid, zero outside the
// row's chunk, window and causal bound), and adds P V with P as hi + lo bfloat16 (two MMAs), which keeps
// 16 bits of a weight's mantissa.  No weight depends on another, so nothing is rescaled and partial sums
// simply add.
//   SPLIT = false: 64 rows a block, 16 a warp, every warp over all 64 keys of a page (prompts);
//   SPLIT = true:  16 rows a block, the four warps take 16 keys each of a page and their sums are added
//                  through shared memory at the end (decode steps: few rows, many keys).
// ---------------------------------------------------------------------------------------
#include "mma_helpers.cuh"

constexpr int GM_THREADS = 128;
constexpr int GM_PAGE = 64;

__device__ __forceinline__ void ldmatrix_x4_plain(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
    ldmatrix_x4(addr, r0, r1, r2, r3);
}

template <int DIM, int VDIM, bool SPLIT>
__global__ void __launch_bounds__(GM_THREADS)
sigmoid_attention_mma_kernel(const bf16* __restrict__ q, int ldq, const bf16* __restrict__ k_cache,
                             const bf16* __restrict__ v_cache, const int* __restrict__ cu_new,
                             const int* __restrict__ seq_start, const int* __restrict__ seq_slot,
                             const int* __restrict__ page_table, int max_pages, const float* __restrict__ bias,
                             bf16* __restrict__ out, int ldo, int n_q, int n_kv, int chunk, int window, float scale) {
    constexpr int ROWS = SPLIT ? 16 : 64;
    constexpr int KP = DIM + 8, VP = VDIM + 8;            // padded rows: ldmatrix without bank conflicts
    constexpr int NT = SPLIT ? 2 : 8;                     // key tiles of 8 a warp takes of a page
    extern __shared__ __align__(16) unsigned char gm_smem[];
    bf16* Ks = reinterpret_cast<bf16*>(gm_smem);          // [2][64][KP]
    bf16* Vs = Ks + 2 * GM_PAGE * KP;                     // [2][64][VP]
    const int b = blockIdx.z, kvh = blockIdx.y, tile = blockIdx.x;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t4 = lane & 3;
    ssb_pdl_launch_dependents();
    ssb_pdl_wait();
    const int slot = seq_slot[b];
    if (slot < 0) return;
    const int t0 = cu_new[b], n_new = cu_new[b + 1] - t0, start = seq_start[b];
    const int G = n_q / n_kv, n_rows = n_new * G;
    const int row0 = tile * ROWS;
    if (row0 >= n_rows) return;
    // keys the block needs: from the first row's lower bound to the last row's position
    const int tok_lo = row0 / G, tok_hi = min(n_new - 1, (row0 + ROWS - 1) / G);
    const int p_first = start + tok_lo, p_last = start + tok_hi;
    int key_lo = chunk > 0 ? (p_first / chunk) * chunk : 0;
    if (window > 0) key_lo = max(key_lo, p_first - window + 1);
    const int page_lo = key_lo / GM_PAGE, page_hi = p_last / GM_PAGE;
    const int* pages = page_table + (size_t)slot * max_pages;

    auto load_page = [&](int pg, int stage) {
        const int id = pages[pg];
        const bf16* ksrc = k_cache + ((size_t)id * n_kv + kvh) * GM_PAGE * DIM;
        const bf16* vsrc = v_cache + ((size_t)id * n_kv + kvh) * GM_PAGE * VDIM;
        bf16* kd = Ks + stage * GM_PAGE * KP;
        bf16* vd = Vs + stage * GM_PAGE * VP;
        for (int c = tid; c < GM_PAGE * (DIM / 8); c += GM_THREADS) {
            const int r = c / (DIM / 8), cc = c % (DIM / 8);
            cp_async16((uint32_t)__cvta_generic_to_shared(kd + r * KP + cc * 8), ksrc + r * DIM + cc * 8);
        }
        for (int c = tid; c < GM_PAGE * (VDIM / 8); c += GM_THREADS) {
            const int r = c / (VDIM / 8), cc = c % (VDIM / 8);
            cp_async16((uint32_t)__cvta_generic_to_shared(vd + r * VP + cc * 8), vsrc + r * VDIM + cc * 8);
        }
        cp_async_commit();
    };
    load_page(page_lo, 0);

    // this warp's rows: g and g + 8 of its 16
    const int wrow0 = row0 + (SPLIT ? 0 : warp * 16);
    int r_tok[2], r_head[2], r_pos[2], r_lo[2];
    bool r_ok[2];
    float r_bias[2];
#pragma unroll
    for (int e = 0; e < 2; ++e) {
        const int R = wrow0 + g + e * 8;
        r_ok[e] = R < n_rows;
        r_tok[e] = r_ok[e] ? R / G : 0;
        r_head[e] = kvh * G + (r_ok[e] ? R % G : 0);
        r_pos[e] = start + r_tok[e];
        int lo = chunk > 0 ? (r_pos[e] / chunk) * chunk : 0;
        if (window > 0) lo = max(lo, r_pos[e] - window + 1);
        r_lo[e] = lo;
        r_bias[e] = bias ? bias[r_head[e]] : 0.f;
    }
    const bool warp_live = wrow0 < n_rows;
    // the queries as A fragments: [k step][a0 a1 a2 a3]
    uint32_t qa[DIM / 16][4];
#pragma unroll
    for (int ks = 0; ks < DIM / 16; ++ks)
#pragma unroll
        for (int e = 0; e < 2; ++e) {
            const bf16* qr = q + (size_t)(t0 + r_tok[e]) * ldq + (size_t)r_head[e] * DIM + ks * 16 + 2 * t4;
            qa[ks][e] = r_ok[e] ? *reinterpret_cast<const uint32_t*>(qr) : 0u;
            qa[ks][e + 2] = r_ok[e] ? *reinterpret_cast<const uint32_t*>(qr + 8) : 0u;
        }
    float acc[VDIM / 8][4];
#pragma unroll
    for (int n = 0; n < VDIM / 8; ++n)
#pragma unroll
        for (int e = 0; e < 4; ++e) acc[n][e] = 0.f;

    for (int pg = page_lo; pg <= page_hi; ++pg) {
        const int stage = (pg - page_lo) & 1;
        if (pg + 1 <= page_hi) {
            load_page(pg + 1, stage ^ 1);
            cp_async_wait<1>();
        } else {
            cp_async_wait<0>();
        }
        __syncthreads();
        if (warp_live) {
            const bf16* kd = Ks + stage * GM_PAGE * KP;
            const bf16* vd = Vs + stage * GM_PAGE * VP;
            const int nt0 = SPLIT ? warp * 2 : 0;         // first key tile of 8 this warp takes
            float s[NT][4];
#pragma unroll
            for (int j = 0; j < NT; ++j)
#pragma unroll
                for (int e = 0; e < 4; ++e) s[j][e] = 0.f;
#pragma unroll
            for (int ks = 0; ks < DIM / 16; ++ks)
#pragma unroll
                for (int j = 0; j < NT; j += 2) {
                    // keys (nt0 + j) * 8 .. + 15, dims ks * 16 .. + 15: four 8 x 8 matrices
                    const int key = (nt0 + j) * 8 + (lane & 7) + (lane >> 4) * 8, dim = ks * 16 + ((lane >> 3) & 1) * 8;
                    uint32_t b0, b1, b2, b3;
                    ldmatrix_x4((uint32_t)__cvta_generic_to_shared(kd + key * KP + dim), b0, b1, b2, b3);
                    mma16816(s[j], qa[ks][0], qa[ks][1], qa[ks][2], qa[ks][3], b0, b1);
                    mma16816(s[j + 1], qa[ks][0], qa[ks][1], qa[ks][2], qa[ks][3], b2, b3);
                }
            // weights, float32: zero where the key is not visible to the row
            uint32_t p_hi[NT][2], p_lo[NT][2];
#pragma unroll
            for (int j = 0; j < NT; ++j) {
                const int key = pg * GM_PAGE + (nt0 + j) * 8 + 2 * t4;
                float w[4];
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int rr = e >> 1, kk = key + (e & 1);
                    const bool vis = r_ok[rr] && kk >= r_lo[rr] && kk <= r_pos[rr];
                    w[e] = vis ? 1.0f / (1.0f + __expf(-(s[j][e] * scale + r_bias[rr]))) : 0.f;
                }
                p_hi[j][0] = pack2(w[0], w[1]);
                p_hi[j][1] = pack2(w[2], w[3]);
                const __nv_bfloat162 h0 = *reinterpret_cast<__nv_bfloat162*>(&p_hi[j][0]);
                const __nv_bfloat162 h1 = *reinterpret_cast<__nv_bfloat162*>(&p_hi[j][1]);
                p_lo[j][0] = pack2(w[0] - __low2float(h0), w[1] - __high2float(h0));
                p_lo[j][1] = pack2(w[2] - __low2float(h1), w[3] - __high2float(h1));
            }
#pragma unroll
            for (int kk = 0; kk < NT / 2; ++kk) {         // 16 keys a step
                const int key0 = (nt0 + 2 * kk) * 8;
#pragma unroll
                for (int n = 0; n < VDIM / 8; n += 2) {
                    // keys key0 .. + 15, value columns n * 8 .. + 15, transposed: B fragments of two column tiles
                    const int key = key0 + (lane & 7) + ((lane >> 3) & 1) * 8, col = n * 8 + (lane >> 4) * 8;
                    uint32_t b0, b1, b2, b3;
                    ldmatrix_x4_trans((uint32_t)__cvta_generic_to_shared(vd + key * VP + col), b0, b1, b2, b3);
                    mma16816(acc[n], p_hi[2 * kk][0], p_hi[2 * kk][1], p_hi[2 * kk + 1][0], p_hi[2 * kk + 1][1], b0, b1);
                    mma16816(acc[n], p_lo[2 * kk][0], p_lo[2 * kk][1], p_lo[2 * kk + 1][0], p_lo[2 * kk + 1][1], b0, b1);
                    mma16816(acc[n + 1], p_hi[2 * kk][0], p_hi[2 * kk][1], p_hi[2 * kk + 1][0], p_hi[2 * kk + 1][1], b2, b3);
                    mma16816(acc[n + 1], p_lo[2 * kk][0], p_lo[2 * kk][1], p_lo[2 * kk + 1][0], p_lo[2 * kk + 1][1], b2, b3);
                }
            }
        }
        __syncthreads();                                  // the stage is free for the page after next
    }
    if (SPLIT) {
        // the four warps hold sums over different keys of the same 16 rows: add them in shared memory
        float* red = reinterpret_cast<float*>(gm_smem);   // [4][16][VDIM]
#pragma unroll
        for (int n = 0; n < VDIM / 8; ++n) {
            float* r = red + (size_t)warp * 16 * VDIM + n * 8 + 2 * t4;
            r[g * VDIM] = acc[n][0];
            r[g * VDIM + 1] = acc[n][1];
            r[(g + 8) * VDIM] = acc[n][2];
            r[(g + 8) * VDIM + 1] = acc[n][3];
        }
        __syncthreads();
        for (int e = tid; e < 16 * VDIM; e += GM_THREADS) {
            const int r = e / VDIM, c = e % VDIM, R = row0 + r;
            if (R >= n_rows) continue;
            const float sum = red[e] + red[16 * VDIM + e] + red[2 * 16 * VDIM + e] + red[3 * 16 * VDIM + e];
            out[(size_t)(t0 + R / G) * ldo + (size_t)(kvh * G + R % G) * VDIM + c] = __float2bfloat16_rn(sum);
        }
        return;
    }
    if (!warp_live) return;
#pragma unroll
    for (int e = 0; e < 2; ++e) {
        if (!r_ok[e]) continue;
        bf16* o = out + (size_t)(t0 + r_tok[e]) * ldo + (size_t)r_head[e] * VDIM + 2 * t4;
#pragma unroll
        for (int n = 0; n < VDIM / 8; ++n)
            *reinterpret_cast<uint32_t*>(o + n * 8) = pack2(acc[n][2 * e], acc[n][2 * e + 1]);
    }
}

template <int DIM, int VDIM, bool SPLIT>
static int launch_sigmoid_mma(const bf16* q, int ldq, const bf16* k_cache, const bf16* v_cache, const int* cu_new,
                              const int* seq_start, const int* seq_slot, const int* page_table, int max_pages,
                              const float* bias, bf16* out, int ldo, int n_seqs, int max_new, int n_q, int n_kv, int chunk,
                              int window, float scale, int pdl, cudaStream_t stream) {
    constexpr int ROWS = SPLIT ? 16 : 64;
    size_t smem = (size_t)2 * GM_PAGE * (DIM + 8 + VDIM + 8) * sizeof(bf16);
    if (SPLIT && smem < (size_t)4 * 16 * VDIM * sizeof(float)) smem = (size_t)4 * 16 * VDIM * sizeof(float);
    auto kern = sigmoid_attention_mma_kernel<DIM, VDIM, SPLIT>;
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
    }
    const int rows = max_new * (n_q / n_kv);
    const dim3 grid((rows + ROWS - 1) / ROWS, n_kv, n_seqs);
    if (grid.y > 65535 || grid.z > 65535) return SSB_ERR_BAD_SIZE;
    const int rc = ssb_launch(kern, grid, dim3(GM_THREADS), smem, stream, pdl != 0, q, ldq, k_cache, v_cache, cu_new,
                              seq_start, seq_slot, page_table, max_pages, bias, out, ldo, n_q, n_kv, chunk, window, scale);
    return rc ? rc : ssb_launch_status();
}

// q [T, ldq] bfloat16 (n_q x dim, normed and rotated); the caches' pages hold 64 tokens (page_shift 6); dim and
// vdim each one of 64, 96, 128; ldq and ldo multiples of 2 elements.  split: the decode form (16 rows a block).
SSB_API int ssb_sigmoid_attention_mma(const void* q, int ldq, const void* k_cache, const void* v_cache,
                                      const int* cu_new, const int* seq_start, const int* seq_slot,
                                      const int* page_table, int max_pages, const float* bias, void* out, int ldo,
                                      int n_seqs, int max_new, int n_q, int n_kv, int dim, int vdim, int page_shift,
                                      int chunk, int window, float scale, int split, int pdl, cudaStream_t stream) {
    if (n_seqs <= 0 || max_new <= 0) return 0;
    if (page_shift != 6 || n_kv <= 0 || n_q % n_kv || (ldq & 1) || (ldo & 1) || chunk < 0 || window < 0) return SSB_ERR_BAD_SIZE;
#define SSB_GM(D, V) \
    if (dim == D && vdim == V) \
        return split ? launch_sigmoid_mma<D, V, true>((const bf16*)q, ldq, (const bf16*)k_cache, (const bf16*)v_cache, cu_new, \
                                                      seq_start, seq_slot, page_table, max_pages, bias, (bf16*)out, ldo, n_seqs, \
                                                      max_new, n_q, n_kv, chunk, window, scale, pdl, stream) \
                     : launch_sigmoid_mma<D, V, false>((const bf16*)q, ldq, (const bf16*)k_cache, (const bf16*)v_cache, cu_new, \
                                                       seq_start, seq_slot, page_table, max_pages, bias, (bf16*)out, ldo, n_seqs, \
                                                       max_new, n_q, n_kv, chunk, window, scale, pdl, stream)
    SSB_GM(64, 64); SSB_GM(64, 128); SSB_GM(96, 64); SSB_GM(96, 96); SSB_GM(128, 64); SSB_GM(128, 128);
#undef SSB_GM
    return SSB_ERR_UNSUPPORTED;
}
