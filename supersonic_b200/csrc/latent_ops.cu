// Latent attention: what lies between the fused projection and the attention itself.
//
// Input: a token's projected row, [H queries of (dim + rot_dim) | kv_rank + rot_dim], the second
// part being the low-rank row from which keys and values of all H heads derive.  Output: the
// token's cache row [rms(first kv_rank) * w | rotate(last rot_dim)] at its position, and the
// rotated rot_dim tails of the H queries behind the latent-space queries in q_abs.  The attention
// that follows works on these rows directly (see parts/latent_attention.py for the algebra).
// All arithmetic is float32.
#include "common.cuh"
#include <math.h>

typedef __nv_bfloat16 bf16;

template <typename T, typename TW>
__global__ void __launch_bounds__(256)
latent_prepare_kernel(T* __restrict__ proj, int ld, int c_off, T* __restrict__ q_abs, int ldq,
                      const TW* __restrict__ norm_w, float eps, const float* __restrict__ cos_t,
                      const float* __restrict__ sin_t, int table_positions, const int* __restrict__ pos,
                      const int* __restrict__ slot, const int* __restrict__ page_table, int max_pages,
                      T* __restrict__ cache, int n_heads, int dim, int rot_dim, int rot_dims, int kv_rank,
                      int page_shift, int write_cache, int interleaved) {
    __shared__ float red[256];
    const int t = blockIdx.x, tid = threadIdx.x;
    ssb_pdl_launch_dependents();
    ssb_pdl_wait();
    const int s = slot[t];
    if (s < 0) return;                                   // padding row
    const int p = pos[t];
    const int half = rot_dims / 2;
    const bool have = p < table_positions;
    const float* c_row = cos_t + (size_t)p * half;
    const float* s_row = sin_t + (size_t)p * half;
    T* row = proj + (size_t)t * ld;
    // queries: the rotated part of every head turned by the token's position, written behind the
    // head's latent-space query in q_abs ([head][kv_rank | rot_dim])
    const int qw = dim + rot_dim, aw = kv_rank + rot_dim;
    T* qa = q_abs + (size_t)t * ldq;
    for (int e = tid; e < n_heads * rot_dim; e += 256) {
        const int h = e / rot_dim, i = e % rot_dim;
        const T* x = row + (size_t)h * qw + dim;
        float v = ssb_to_float(x[i]);
        if (i < rot_dims) {
            int pair, first;
            if (interleaved) { pair = i >> 1; first = !(i & 1); }
            else { pair = i < half ? i : i - half; first = i < half; }
            const int j = interleaved ? (first ? i + 1 : i - 1) : (first ? i + half : i - half);
            const float c = have ? c_row[pair] : 1.f, sn = have ? s_row[pair] : 0.f;
            const float o = ssb_to_float(x[j]);
            v = first ? v * c - o * sn : v * c + o * sn;
        }
        qa[(size_t)h * aw + kv_rank + i] = ssb_from_float<T>(v);
    }
    if (!write_cache) return;
    // the latent: x / sqrt(mean(x^2) + eps) * w
    const T* lat = row + c_off;
    float part = 0.f;
    for (int c = tid; c < kv_rank; c += 256) {
        const float v = ssb_to_float(lat[c]);
        part = fmaf(v, v, part);
    }
    red[tid] = part;
    __syncthreads();
    for (int st = 128; st > 0; st >>= 1) {
        if (tid < st) red[tid] += red[tid + st];
        __syncthreads();
    }
    const float inv = 1.0f / sqrtf(red[0] / (float)kv_rank + eps);
    T* dst = cache + ssb_cache_row(page_table, max_pages, s, p, page_shift, 1, 0, aw);
    for (int c = tid; c < kv_rank; c += 256)
        dst[c] = ssb_from_float<T>(ssb_to_float(lat[c]) * inv * ssb_to_float(norm_w[c]));
    const T* kr = lat + kv_rank;
    for (int i = tid; i < rot_dim; i += 256) {
        float v = ssb_to_float(kr[i]);
        if (i < rot_dims) {
            int pair, first;
            if (interleaved) { pair = i >> 1; first = !(i & 1); }
            else { pair = i < half ? i : i - half; first = i < half; }
            const int j = interleaved ? (first ? i + 1 : i - 1) : (first ? i + half : i - half);
            const float c = have ? c_row[pair] : 1.f, sn = have ? s_row[pair] : 0.f;
            const float o = ssb_to_float(kr[j]);
            v = first ? v * c - o * sn : v * c + o * sn;
        }
        dst[kv_rank + i] = ssb_from_float<T>(v);
    }
}

// proj [T, ld]: queries from column 0, the low-rank row from column c_off; q_abs [T, ldq] gets the
// rotated query parts; the cache entry [pages][1][tokens][kv_rank + rot_dim] gets the token's row
SSB_API int ssb_latent_prepare(void* proj, int ld, int c_off, void* q_abs, int ldq, int dtype, const void* norm_w,
                               int w_dtype, float eps, const float* cos_t, const float* sin_t, int table_positions,
                               const int* pos, const int* slot, const int* page_table, int max_pages, void* cache,
                               int n_tokens, int n_heads, int dim, int rot_dim, int rot_dims, int kv_rank,
                               int page_shift, int write_cache, int interleaved, int pdl, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (rot_dims % 2 || rot_dims > rot_dim || rot_dims < 0 || kv_rank <= 0) return SSB_ERR_BAD_SIZE;
    int rc = 0;
#define SSB_PREP(T, TW) \
    rc = ssb_launch(latent_prepare_kernel<T, TW>, dim3(n_tokens), dim3(256), 0, stream, pdl != 0, (T*)proj, ld, c_off, \
                    (T*)q_abs, ldq, (const TW*)norm_w, eps, cos_t, sin_t, table_positions, pos, slot, page_table,  \
                    max_pages, (T*)cache, n_heads, dim, rot_dim, rot_dims, kv_rank, page_shift, write_cache, interleaved)
    if (dtype == SSB_F32 && w_dtype == SSB_F32) SSB_PREP(float, float);
    else if (dtype == SSB_BF16 && w_dtype == SSB_BF16) SSB_PREP(bf16, bf16);
    else if (dtype == SSB_BF16 && w_dtype == SSB_F32) SSB_PREP(bf16, float);
    else return SSB_ERR_BAD_DTYPE;
#undef SSB_PREP
    return rc ? rc : ssb_launch_status();
}
