// Linear recurrences with a matrix state per head, kept in float32 per sequence.
//
// Gated linear attention: with a decay a_t in (0, 1) per key channel,
//     S_t = diag(a_t) S_(t-1) + k_t v_t^T        (S: [dim, vdim] per head)
//     o_t = S_t^T q_t
// a_t = sigmoid(z_t)^(1/tau), evaluated as exp(log_sigmoid(z_t) / tau).  Everything that enters the
// recurrence is float32; q, k and v are read in their storage type and widened.
// The scan walks a sequence's new tokens in order, from the state the sequence's slot holds, and
// leaves the state there; a block owns a tile of value columns of one head of one sequence, so no
// sum depends on what else is in the batch.
#include "common.cuh"
#include <math.h>

typedef __nv_bfloat16 bf16;

constexpr int SCAN_COLS = 32;        // value columns a block owns
constexpr int SCAN_GROUPS = 8;       // row groups: thread (g, j) owns rows g, g + 8, ... of column j
constexpr int SCAN_MAX_ROWS = 32;    // rows per thread: dim up to 256

__device__ __forceinline__ float log_sigmoid(float z) {
    // log(1 / (1 + exp(-z))) without overflow on either side
    return fminf(z, 0.f) - log1pf(expf(-fabsf(z)));
}

template <typename T>
__global__ void __launch_bounds__(SCAN_COLS * SCAN_GROUPS)
gated_linear_scan_kernel(const T* __restrict__ proj, int ld, int q_off, int k_off, int v_off,
                         const float* __restrict__ z, int ldz, const float* __restrict__ z_bias,
                         float inv_tau, float q_scale, float* __restrict__ state,
                         const int* __restrict__ cu_new, const int* __restrict__ seq_slot,
                         float* __restrict__ out, int ldo, int n_heads, int dim, int vdim) {
    extern __shared__ float sm[];
    float* a_s = sm;                    // [dim] decay
    float* k_s = a_s + dim;             // [dim]
    float* q_s = k_s + dim;             // [dim]
    float* v_s = q_s + dim;             // [SCAN_COLS]
    float* o_s = v_s + SCAN_COLS;       // [SCAN_GROUPS][SCAN_COLS]
    const int b = blockIdx.x, h = blockIdx.y, j0 = blockIdx.z * SCAN_COLS;
    const int tid = threadIdx.x, j = tid % SCAN_COLS, g = tid / SCAN_COLS;
    ssb_pdl_launch_dependents();
    ssb_pdl_wait();
    const int slot = seq_slot[b];
    if (slot < 0) return;                                // padding row
    const int t0 = cu_new[b], t1 = cu_new[b + 1];
    const bool col = j0 + j < vdim;
    float* S = state + ((size_t)slot * n_heads + h) * dim * vdim;
    float s_reg[SCAN_MAX_ROWS];
#pragma unroll
    for (int r = 0; r < SCAN_MAX_ROWS; ++r) {
        const int i = g + r * SCAN_GROUPS;
        s_reg[r] = (col && i < dim) ? S[(size_t)i * vdim + j0 + j] : 0.f;
    }
    for (int t = t0; t < t1; ++t) {
        const T* row = proj + (size_t)t * ld;
        for (int i = tid; i < dim; i += SCAN_COLS * SCAN_GROUPS) {
            const float zz = z[(size_t)t * ldz + h * dim + i] + z_bias[h * dim + i];
            a_s[i] = expf(log_sigmoid(zz) * inv_tau);
            k_s[i] = ssb_to_float(row[k_off + h * dim + i]);
            q_s[i] = ssb_to_float(row[q_off + h * dim + i]) * q_scale;
        }
        if (tid < SCAN_COLS) v_s[tid] = (j0 + tid < vdim) ? ssb_to_float(row[v_off + h * vdim + j0 + tid]) : 0.f;
        __syncthreads();
        const float v = v_s[j];
        float o = 0.f;
#pragma unroll
        for (int r = 0; r < SCAN_MAX_ROWS; ++r) {
            const int i = g + r * SCAN_GROUPS;
            if (i < dim) {
                s_reg[r] = fmaf(a_s[i], s_reg[r], k_s[i] * v);
                o = fmaf(s_reg[r], q_s[i], o);
            }
        }
        o_s[g * SCAN_COLS + j] = o;
        __syncthreads();
        if (g == 0 && col) {
            float sum = 0.f;
#pragma unroll
            for (int gg = 0; gg < SCAN_GROUPS; ++gg) sum += o_s[gg * SCAN_COLS + j];
            out[(size_t)t * ldo + h * vdim + j0 + j] = sum;
        }
    }
#pragma unroll
    for (int r = 0; r < SCAN_MAX_ROWS; ++r) {
        const int i = g + r * SCAN_GROUPS;
        if (col && i < dim) S[(size_t)i * vdim + j0 + j] = s_reg[r];
    }
}

// proj [T, ld] holds q, k (n_heads x dim each) and v (n_heads x vdim) from the given columns;
// z [T, ldz] float32 is the decay's pre-activation without its bias z_bias [n_heads x dim];
// state [slots, n_heads, dim, vdim] float32; out [T, ldo] float32 gets o (n_heads x vdim)
SSB_API int ssb_gated_linear_scan(const void* proj, int ld, int dtype, int q_off, int k_off, int v_off,
                                  const float* z, int ldz, const float* z_bias, float tau, float q_scale,
                                  float* state, const int* cu_new, const int* seq_slot, float* out, int ldo,
                                  int n_seqs, int n_heads, int dim, int vdim, int pdl, cudaStream_t stream) {
    if (n_seqs <= 0) return 0;
    if (dim <= 0 || dim > SCAN_MAX_ROWS * SCAN_GROUPS || vdim <= 0 || !(tau > 0.f)) return SSB_ERR_BAD_SIZE;
    const dim3 grid(n_seqs, n_heads, (vdim + SCAN_COLS - 1) / SCAN_COLS);
    if (grid.y > 65535 || grid.z > 65535) return SSB_ERR_BAD_SIZE;
    const size_t smem = (3 * (size_t)dim + SCAN_COLS + SCAN_COLS * SCAN_GROUPS) * sizeof(float);
    int rc;
    if (dtype == SSB_F32)
        rc = ssb_launch(gated_linear_scan_kernel<float>, grid, dim3(SCAN_COLS * SCAN_GROUPS), smem, stream, pdl != 0,
                        (const float*)proj, ld, q_off, k_off, v_off, z, ldz, z_bias, 1.0f / tau, q_scale, state, cu_new,
                        seq_slot, out, ldo, n_heads, dim, vdim);
    else if (dtype == SSB_BF16)
        rc = ssb_launch(gated_linear_scan_kernel<bf16>, grid, dim3(SCAN_COLS * SCAN_GROUPS), smem, stream, pdl != 0,
                        (const bf16*)proj, ld, q_off, k_off, v_off, z, ldz, z_bias, 1.0f / tau, q_scale, state, cu_new,
                        seq_slot, out, ldo, n_heads, dim, vdim);
    else
        return SSB_ERR_BAD_DTYPE;
    return rc ? rc : ssb_launch_status();
}

// ---------------------------------------------------------------------------------------
// y[t, h, :] = o[t, h, :] / sqrt(mean(o[t, h, :]^2) + eps) * w * silu(gate[t, h, :]): a head's
// output normalised over its own width with one weight vector for all heads, then gated
// ---------------------------------------------------------------------------------------
template <typename T, typename TW>
__global__ void __launch_bounds__(128)
head_norm_gate_kernel(const float* __restrict__ o, int ldo, const TW* __restrict__ w, float eps,
                      const T* __restrict__ gate, int ldg, T* __restrict__ y, int ldy, int vdim) {
    __shared__ float red[128];
    const int t = blockIdx.x, h = blockIdx.y, tid = threadIdx.x;
    ssb_pdl_launch_dependents();
    ssb_pdl_wait();
    const float* src = o + (size_t)t * ldo + (size_t)h * vdim;
    float part = 0.f;
    for (int c = tid; c < vdim; c += 128) part = fmaf(src[c], src[c], part);
    red[tid] = part;
    __syncthreads();
    for (int s = 64; s > 0; s >>= 1) {
        if (tid < s) red[tid] += red[tid + s];
        __syncthreads();
    }
    const float inv = 1.0f / sqrtf(red[0] / (float)vdim + eps);
    const T* gr = gate + (size_t)t * ldg + (size_t)h * vdim;
    T* dst = y + (size_t)t * ldy + (size_t)h * vdim;
    for (int c = tid; c < vdim; c += 128) {
        const float gv = ssb_to_float(gr[c]);
        dst[c] = ssb_from_float<T>(src[c] * inv * ssb_to_float(w[c]) * (gv / (1.0f + expf(-gv))));
    }
}

SSB_API int ssb_head_norm_gate(const float* o, int ldo, const void* w, int w_dtype, float eps, const void* gate,
                               int ldg, void* y, int ldy, int dtype, int n_tokens, int n_heads, int vdim, int pdl,
                               cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (vdim <= 0 || n_heads <= 0 || n_heads > 65535) return SSB_ERR_BAD_SIZE;
    const dim3 grid(n_tokens, n_heads);
    int rc = 0;
#define SSB_HNG(T, TW) \
    rc = ssb_launch(head_norm_gate_kernel<T, TW>, grid, dim3(128), 0, stream, pdl != 0, o, ldo, (const TW*)w, eps, \
                    (const T*)gate, ldg, (T*)y, ldy, vdim)
    if (dtype == SSB_F32 && w_dtype == SSB_F32) SSB_HNG(float, float);
    else if (dtype == SSB_BF16 && w_dtype == SSB_BF16) SSB_HNG(bf16, bf16);
    else if (dtype == SSB_BF16 && w_dtype == SSB_F32) SSB_HNG(bf16, float);
    else return SSB_ERR_BAD_DTYPE;
#undef SSB_HNG
    return rc ? rc : ssb_launch_status();
}
