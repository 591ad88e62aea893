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
